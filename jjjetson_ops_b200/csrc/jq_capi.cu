// C ABI of the library: argument checking, kernel selection, the reference-style host wrappers,
// resident weights, and the device description.  Declarations and the reference lines each entry
// point replaces are in include/jq_b200.h.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "jq_common.cuh"

namespace jq {

namespace {

thread_local std::string t_last_error;

__device__ int g_device_fault_word = 0;

constexpr int MAX_DEVICES = 64;
struct PerDevice {
    bool caps_ok = false;
    DeviceCaps caps;
    int *fault_ptr = nullptr;
    bool fault_ok = false;
};
PerDevice g_dev[MAX_DEVICES];
std::mutex g_dev_mutex;
std::atomic<int> g_options[JQ_OPT_COUNT_];

}  // namespace

namespace {
std::atomic<unsigned long long *> g_trace_buf{nullptr};
std::atomic<long long> g_trace_slots{0}, g_trace_next{0};
constexpr int TRACE_CTAS = 512;  // CTAs recorded per launch, 8 stamps of 8 bytes each
}
void *next_trace_slot() {
    unsigned long long *buf = g_trace_buf.load();
    if (buf == nullptr) return nullptr;
    const long long i = g_trace_next.fetch_add(1);
    if (i >= g_trace_slots.load()) return nullptr;
    return buf + (size_t)i * TRACE_CTAS * 8;
}

uint32_t wait_poll_limit() {
    const int v = option_value(JQ_OPT_WAIT_POLL_LIMIT);
    return v > 0 ? (uint32_t)v : (1u << 22);
}

int option_value(int option) {
    return option >= 0 && option < JQ_OPT_COUNT_ ? g_options[option].load(std::memory_order_relaxed) : 0;
}

int set_error(int status, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    t_last_error = buf;
    return status;
}

int cuda_error(cudaError_t e, const char *what) {
    // The runtime keeps a failed call's code as its "last error" until somebody reads it; take it, so that
    // the post-launch check of a later, unrelated call does not report this failure a second time.
    (void)cudaGetLastError();
    return set_error(JQ_ERR_CUDA, "%s failed: %s", what, cudaGetErrorString(e));
}

int device_caps(DeviceCaps *out) {
    int dev = 0;
    JQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return set_error(JQ_ERR_UNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    PerDevice &d = g_dev[dev];
    if (!d.caps_ok) {
        int major = 0, minor = 0;
        JQ_CUDA_TRY(cudaDeviceGetAttribute(&d.caps.sm_count, cudaDevAttrMultiProcessorCount, dev));
        JQ_CUDA_TRY(cudaDeviceGetAttribute(&d.caps.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        JQ_CUDA_TRY(cudaDeviceGetAttribute(&d.caps.smem_per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev));
        JQ_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        JQ_CUDA_TRY(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
        d.caps.cc = major * 10 + minor;
        d.caps_ok = true;
    }
    *out = d.caps;
    return JQ_OK;
}

int ensure_dynamic_smem(const void *kernel, int bytes, bool max_carveout) {
    struct Entry {
        const void *fn;
        int dev, bytes;
    };
    static std::vector<Entry> table;
    static std::mutex table_mutex;
    int dev = 0;
    JQ_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(table_mutex);
    Entry *e = nullptr;
    for (Entry &t : table) {
        if (t.fn == kernel && t.dev == dev) {
            e = &t;
            break;
        }
    }
    if (e != nullptr && e->bytes >= bytes) return JQ_OK;
    JQ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    if (e == nullptr) {
        if (max_carveout)
            JQ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        table.push_back(Entry{kernel, dev, bytes});
    } else {
        e->bytes = bytes;
    }
    return JQ_OK;
}

namespace {
std::atomic<unsigned long long> g_extent_shrink{0};
}
Extent make_extent(const void *base, unsigned long long bytes) {
    Extent e;
    e.base = base;
    const unsigned long long shrink = g_extent_shrink.load(std::memory_order_relaxed);
    e.bytes = bytes > shrink ? bytes - shrink : 0;
    return e;
}

MulMatBounds mul_mat_bounds(const void *d_w, const void *d_xq, const void *d_y, int64_t K, int64_t N, int64_t M, size_t y_elem_bytes) {
    MulMatBounds b;
    b.w = make_extent(d_w, (unsigned long long)N * (unsigned long long)(K / QK) * Q4_BYTES);
    b.xq = make_extent(d_xq, (unsigned long long)M * (unsigned long long)(K / SUPER) * Q8_BYTES);
    b.y = make_extent(d_y, (unsigned long long)M * (unsigned long long)N * y_elem_bytes);
    b.fault = BOUNDS_CHECK ? device_fault_ptr() : nullptr;
    return b;
}

int *device_fault_ptr() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    PerDevice &d = g_dev[dev];
    if (!d.fault_ok) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_fault_word) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        d.fault_ptr = static_cast<int *>(p);
        d.fault_ok = true;
    }
    return d.fault_ptr;
}

namespace {

int check_order(int order) {
    if (order != JQ_ORDER_KSUPER_COL && order != JQ_ORDER_COL_KSUPER)
        return set_error(JQ_ERR_INVALID_ARG, "unknown Q8_1 block order %d", order);
    return JQ_OK;
}
int check_s_mode(int s_mode) {
    if (s_mode != JQ_S_SUM_X && s_mode != JQ_S_D_SUM_Q)
        return set_error(JQ_ERR_INVALID_ARG, "unknown s_mode %d", s_mode);
    return JQ_OK;
}

int check_mul_mat_shape(int64_t K, int64_t N, int64_t M) {
    if (K < 0 || N < 0 || M < 0) return set_error(JQ_ERR_INVALID_ARG, "negative size (K=%lld N=%lld M=%lld)", (long long)K, (long long)N, (long long)M);
    // the two checks of mat_mul_q4_0_q8_1 (mm_q4_0_q8_1.cu:331-340)
    if (K % QK != 0) return set_error(JQ_ERR_SHAPE, "ncols_k must be multiple of %d", QK);
    if (K % SUPER != 0) return set_error(JQ_ERR_SHAPE, "ncols_k must be multiple of %d for block_q8_1_mmq", SUPER);
    if (K > (int64_t)1 << 30 || N > (int64_t)1 << 31 || M > (int64_t)1 << 31)
        return set_error(JQ_ERR_TOO_LARGE, "shape exceeds 32-bit kernel indexing");
    return JQ_OK;
}

// Smallest batch the automatic choice gives to the fp16-operand GEMM (unless JQ_OPT_PREFILL_EXACT): half a 128-column tile.
constexpr int64_t FP16_OPERANDS_MIN_COLUMNS = 64;

int dispatch_mul_mat(cudaStream_t st, const void *d_w, const void *d_xq, float *d_y, int64_t K, int64_t N,
                     int64_t M, int order, int kernel) {
    if (N == 0 || M == 0) return JQ_OK;
    if (K == 0) {
        JQ_CUDA_TRY(cudaMemsetAsync(d_y, 0, (size_t)M * N * sizeof(float), st));
        return JQ_OK;
    }
    switch (kernel) {
        case JQ_KERNEL_GENERIC: return launch_mmq_generic(st, d_w, d_xq, d_y, K, N, M, order);
        case JQ_KERNEL_GEMV_DP4A: return launch_gemv_dp4a(st, d_w, d_xq, nullptr, nullptr, d_y, K, N, M, order, 0);
        case JQ_KERNEL_GEMV_MMA: return launch_gemv_mma(st, d_w, d_xq, nullptr, nullptr, d_y, K, N, M, order, 0);
        case JQ_KERNEL_GEMM_MMA: return launch_gemm_mma(st, d_w, d_xq, d_y, K, N, M, order);
        case JQ_KERNEL_GEMM_TC: return launch_gemm_tc(st, d_w, d_xq, d_y, K, N, M, order);
        case JQ_KERNEL_GEMM_F16: return launch_gemm_f16(st, d_w, d_xq, d_y, K, N, M, order);
        case JQ_KERNEL_AUTO: break;
        default: return set_error(JQ_ERR_INVALID_ARG, "unknown kernel family %d", kernel);
    }
    int rc = JQ_ERR_UNSUPPORTED;
    if (M <= 2) rc = launch_gemv_dp4a(st, d_w, d_xq, nullptr, nullptr, d_y, K, N, M, order, 0);
    if (rc == JQ_ERR_UNSUPPORTED && M <= 8) rc = launch_gemv_mma(st, d_w, d_xq, nullptr, nullptr, d_y, K, N, M, order, 0);
    if (M > 8 && M <= 32 && order == JQ_ORDER_COL_KSUPER && K <= 6144) {
        // A handful of columns more than one GEMV pass takes: passes of eight columns (the weights of the
        // later passes come from L2) beat a GEMM tile that would be mostly padding (cfg2 shape: M = 16 in
        // 18.8 us against 41.7 us, M = 32 in 37 us against 44 us; from M = 40 on the GEMM wins).
        const size_t col_bytes = (size_t)(K / SUPER) * Q8_BYTES;  // one column's blocks are contiguous in this order
        for (int64_t m0 = 0; m0 < M; m0 += 8) {
            const int64_t mc = M - m0 < 8 ? M - m0 : 8;
            rc = launch_gemv_mma(st, d_w, static_cast<const uint8_t *>(d_xq) + (size_t)m0 * col_bytes, nullptr, nullptr,
                                 d_y + (size_t)m0 * N, K, N, mc, order, 0);
            if (rc != JQ_OK) break;
        }
        if (rc != JQ_OK && rc != JQ_ERR_UNSUPPORTED) return rc;
    }
    if (rc == JQ_ERR_UNSUPPORTED && M >= FP16_OPERANDS_MIN_COLUMNS && option_value(JQ_OPT_PREFILL_EXACT) == 0)
        rc = launch_gemm_f16(st, d_w, d_xq, d_y, K, N, M, order);  // refuses shapes outside its rules: the integer GEMM takes those
    if (rc == JQ_ERR_UNSUPPORTED && M > 8) rc = launch_gemm_mma(st, d_w, d_xq, d_y, K, N, M, order);
    if (rc == JQ_ERR_UNSUPPORTED) rc = launch_mmq_generic(st, d_w, d_xq, d_y, K, N, M, order);
    if (rc == JQ_OK) t_last_error.clear();
    return rc;
}


// Device-side alias of a pinned, mapped host buffer (nullptr for pageable memory).
void *mapped_alias(const void *host_ptr) {
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, host_ptr) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    if (attr.type != cudaMemoryTypeHost || attr.devicePointer == nullptr) return nullptr;
    return attr.devicePointer;
}

// Coalesced copy, used to write a small result straight into mapped host memory: for tens of KB
// one kernel is much quicker than a separate copy-engine transfer.
// With a single block it can also publish a completion ticket in mapped host memory, which the
// host polls instead of paying a stream synchronisation's wake-up latency.
__global__ void copy_f32_kernel(float *__restrict__ dst, const float *__restrict__ src, int64_t n,
                                volatile unsigned *done_flag, unsigned *count) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t i0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
    for (int64_t i = i0; i < n; i += stride) {
        if (i + 4 <= n) {
            *reinterpret_cast<float4 *>(dst + i) = *reinterpret_cast<const float4 *>(src + i);
        } else {
            for (int64_t j = i; j < n; ++j) dst[j] = src[j];
        }
    }
    if (done_flag != nullptr) {  // single-block launches only
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) {
            // completions are counted on the device (a captured graph can be replayed, and the count in host memory
            // is only ever written over the bus, never read)
            const unsigned c = *count + 1u;
            *count = c;
            *done_flag = c;
            __threadfence_system();
        }
    }
}


}  // namespace
}  // namespace jq

using namespace jq;

extern "C" {

const char *jq_status_string(int status) {
    switch (status) {
        case JQ_OK: return "ok";
        case JQ_ERR_INVALID_ARG: return "invalid argument";
        case JQ_ERR_SHAPE: return "unsupported shape";
        case JQ_ERR_ALIGN: return "misaligned pointer";
        case JQ_ERR_CUDA: return "CUDA runtime error";
        case JQ_ERR_UNSUPPORTED: return "unsupported on this path";
        case JQ_ERR_TIMEOUT: return "device-side wait timed out";
        case JQ_ERR_TOO_LARGE: return "request exceeds capacity";
        default: return "unknown status";
    }
}

const char *jq_last_error(void) { return t_last_error.c_str(); }

int jq_version(void) { return 100; }

int jq_set_option(int option, int value) {
    if (option < 0 || option >= JQ_OPT_COUNT_) return set_error(JQ_ERR_INVALID_ARG, "unknown option %d", option);
    g_options[option].store(value, std::memory_order_relaxed);
    return JQ_OK;
}

int jq_trace_enable(void *d_buf, int64_t n_launches) {
    g_trace_next.store(0);
    g_trace_slots.store(d_buf ? n_launches : 0);
    g_trace_buf.store(static_cast<unsigned long long *>(d_buf));
    return JQ_OK;
}

int jq_get_option(int option, int *value_out) {
    if (option < 0 || option >= JQ_OPT_COUNT_ || !value_out) return set_error(JQ_ERR_INVALID_ARG, "unknown option %d", option);
    *value_out = option_value(option);
    return JQ_OK;
}

size_t jq_q8_1_bytes(int64_t K, int64_t M) {
    if (K <= 0 || M <= 0) return 0;
    return (size_t)M * (size_t)((K + SUPER - 1) / SUPER) * Q8_BYTES;
}

size_t jq_q4_0_bytes(int64_t N, int64_t K) {
    if (K <= 0 || N <= 0) return 0;
    return (size_t)N * (size_t)(K / QK) * Q4_BYTES;
}

int jq_quantize_q8_1_device(void *stream, const float *d_x, void *d_xq, int64_t K, int64_t M, int order,
                            int s_mode) {
    if (K < 0 || M < 0) return set_error(JQ_ERR_INVALID_ARG, "negative size (K=%lld M=%lld)", (long long)K, (long long)M);
    if (int rc = check_order(order)) return rc;
    if (int rc = check_s_mode(s_mode)) return rc;
    if (K % QK != 0) return set_error(JQ_ERR_SHAPE, "K = %lld is not a multiple of %d", (long long)K, QK);
    if (K == 0 || M == 0) return JQ_OK;
    if (d_x == nullptr || d_xq == nullptr) return set_error(JQ_ERR_INVALID_ARG, "null pointer");
    if (((uintptr_t)d_x & 15u) != 0 || ((uintptr_t)d_xq & 15u) != 0)
        return set_error(JQ_ERR_ALIGN, "activations and Q8_1 blocks must be 16-byte aligned");
    return launch_quantize_q8_1(static_cast<cudaStream_t>(stream), d_x, d_xq, K, M, order, s_mode);
}

int jq_rms_norm_q8_1_device(void *stream, float *d_input, float *d_residual, const float *d_weight, float *d_normed,
                            void *d_xq, int64_t hidden_size, int64_t num_tokens, float epsilon, int order, int s_mode) {
    if (hidden_size <= 0 || num_tokens <= 0)
        return set_error(JQ_ERR_INVALID_ARG, "invalid hidden_size=%lld num_tokens=%lld", (long long)hidden_size, (long long)num_tokens);
    if (d_xq != nullptr) {
        if (int rc = check_order(order)) return rc;
        if (int rc = check_s_mode(s_mode)) return rc;
        if (((uintptr_t)d_xq & 15u) != 0) return set_error(JQ_ERR_ALIGN, "Q8_1 blocks must be 16-byte aligned");
    }
    if (d_input == nullptr || d_weight == nullptr) return set_error(JQ_ERR_INVALID_ARG, "null pointer");
    if (d_normed == nullptr && d_xq == nullptr && d_residual == nullptr)
        return set_error(JQ_ERR_INVALID_ARG, "no output requested");
    return launch_rms_norm_q8_1(static_cast<cudaStream_t>(stream), d_input, d_residual, d_weight, d_normed, d_xq, hidden_size,
                                num_tokens, epsilon, order, s_mode);
}

int jq_swiglu_q8_1_device(void *stream, const float *d_gate, const float *d_up, float *d_mid, void *d_xq,
                          int64_t intermediate_size, int64_t num_tokens, int order, int s_mode) {
    if (intermediate_size < 0 || num_tokens < 0) return set_error(JQ_ERR_INVALID_ARG, "negative size");
    if (intermediate_size == 0 || num_tokens == 0) return JQ_OK;
    if (d_xq != nullptr) {
        if (int rc = check_order(order)) return rc;
        if (int rc = check_s_mode(s_mode)) return rc;
        if (((uintptr_t)d_xq & 15u) != 0) return set_error(JQ_ERR_ALIGN, "Q8_1 blocks must be 16-byte aligned");
    }
    if (d_gate == nullptr || d_up == nullptr) return set_error(JQ_ERR_INVALID_ARG, "null pointer");
    if (d_mid == nullptr && d_xq == nullptr) return set_error(JQ_ERR_INVALID_ARG, "no output requested");
    return launch_swiglu_q8_1(static_cast<cudaStream_t>(stream), d_gate, d_up, d_mid, d_xq, intermediate_size, num_tokens, order,
                              s_mode);
}

int jq_mul_mat_q4_0_q8_1_device_ex(void *stream, const void *d_w, const void *d_xq, float *d_y, int64_t K,
                                   int64_t N, int64_t M, int order, int kernel) {
    if (int rc = check_mul_mat_shape(K, N, M)) return rc;
    if (int rc = check_order(order)) return rc;
    if (N == 0 || M == 0) return JQ_OK;
    if (d_y == nullptr || (K > 0 && (d_w == nullptr || d_xq == nullptr)))
        return set_error(JQ_ERR_INVALID_ARG, "null pointer");
    if (((uintptr_t)d_w & 1u) != 0) return set_error(JQ_ERR_ALIGN, "Q4_0 blocks must be 2-byte aligned");
    if (((uintptr_t)d_xq & 15u) != 0) return set_error(JQ_ERR_ALIGN, "Q8_1 blocks must be 16-byte aligned");
    if (((uintptr_t)d_y & 3u) != 0) return set_error(JQ_ERR_ALIGN, "output must be 4-byte aligned");
    return dispatch_mul_mat(static_cast<cudaStream_t>(stream), d_w, d_xq, d_y, K, N, M, order, kernel);
}

int jq_mul_mat_q4_0_q8_1_device(void *stream, const void *d_w, const void *d_xq, float *d_y, int64_t K,
                                int64_t N, int64_t M, int order) {
    return jq_mul_mat_q4_0_q8_1_device_ex(stream, d_w, d_xq, d_y, K, N, M, order, JQ_KERNEL_AUTO);
}

// The quantizer runs in the multiply kernel's own prologue (every CTA quantizes all the activations, its warps
// taking a pair of 128-value blocks each, about 0.5 us per 32 blocks) instead of a launch of its own (about 2.8 us
// in a dependent chain whatever the size) for up to four activation rows of K <= 4096 and one row of K <= 8192.
// Measured on cfg2 (cold weights), fused against two launches: M = 2 9.4 against 10.3 us, M = 4 10.8 against
// 11.8 us, M = 8 13.2 against 12.3 us; one row of K = 8192 22.4 against 27 us; one row of K = 11008 (seven
// consumer warps) 9.1 against 7.4 us.
inline bool fuse_quantizer_pays(int64_t M, int64_t K) {
    const int64_t n_super = K / SUPER, blocks = M * n_super;
    return (n_super <= 32 && blocks <= 128) || (n_super <= 64 && blocks <= 64);
}

int jq_linear_q4_0_device(void *stream, const void *d_w, const float *d_x, void *d_ws, float *d_y, int64_t K,
                          int64_t N, int64_t M, int s_mode) {
    if (int rc = check_mul_mat_shape(K, N, M)) return rc;
    if (int rc = check_s_mode(s_mode)) return rc;
    if (M == 0) return JQ_OK;
    if (K > 0 && (d_x == nullptr || d_ws == nullptr)) return set_error(JQ_ERR_INVALID_ARG, "null pointer");
    if (N > 0 && (d_y == nullptr || (K > 0 && d_w == nullptr))) return set_error(JQ_ERR_INVALID_ARG, "null pointer");
    if (((uintptr_t)d_x & 15u) != 0 || ((uintptr_t)d_ws & 15u) != 0)
        return set_error(JQ_ERR_ALIGN, "activations and workspace must be 16-byte aligned");
    if (((uintptr_t)d_w & 1u) != 0) return set_error(JQ_ERR_ALIGN, "Q4_0 blocks must be 2-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // Decode regime: with few activation blocks the quantizer runs in the multiply kernel's own
    // prologue (every CTA redoes it, which only pays while it is a handful of blocks per warp).
    if (K > 0 && N > 0 && M <= 8 && fuse_quantizer_pays(M, K)) {
        int rc = JQ_ERR_UNSUPPORTED;
        if (M <= 2) rc = launch_gemv_dp4a(st, d_w, nullptr, d_x, d_ws, d_y, K, N, M, JQ_ORDER_COL_KSUPER, s_mode);
        if (rc == JQ_ERR_UNSUPPORTED)
            rc = launch_gemv_mma(st, d_w, nullptr, d_x, d_ws, d_y, K, N, M, JQ_ORDER_COL_KSUPER, s_mode);
        if (rc != JQ_ERR_UNSUPPORTED) return rc;
    }
    if (K > 0) {
        if (int rc = launch_quantize_q8_1(st, d_x, d_ws, K, M, JQ_ORDER_COL_KSUPER, s_mode)) return rc;
    }
    return dispatch_mul_mat(st, d_w, d_ws, d_y, K, N, M, JQ_ORDER_COL_KSUPER, JQ_KERNEL_AUTO);
}

int jq_linear_q4_0_multi_device(void *stream, int n_mats, const void *const *d_w, const int64_t *N, float *const *d_y,
                                const float *d_x, const void *d_xq, void *d_ws, int64_t K, int64_t M, int s_mode) {
    if (n_mats < 1 || n_mats > 4) return set_error(JQ_ERR_INVALID_ARG, "1 to 4 weight matrices per call (got %d)", n_mats);
    if (d_w == nullptr || N == nullptr || d_y == nullptr) return set_error(JQ_ERR_INVALID_ARG, "null pointer");
    if ((d_x == nullptr) == (d_xq == nullptr)) return set_error(JQ_ERR_INVALID_ARG, "give either fp32 activations or Q8_1 blocks");
    if (int rc = check_s_mode(s_mode)) return rc;
    int64_t n_total = 0;
    for (int i = 0; i < n_mats; ++i) {
        if (int rc = check_mul_mat_shape(K, N[i], M)) return rc;
        if (N[i] > 0 && (d_y[i] == nullptr || (K > 0 && d_w[i] == nullptr))) return set_error(JQ_ERR_INVALID_ARG, "null pointer");
        if (((uintptr_t)d_w[i] & 1u) != 0) return set_error(JQ_ERR_ALIGN, "Q4_0 blocks must be 2-byte aligned");
        n_total += N[i];
    }
    if (M == 0 || n_total == 0) return JQ_OK;
    if (d_x != nullptr && K > 0 && d_ws == nullptr) return set_error(JQ_ERR_INVALID_ARG, "fp32 activations need a Q8_1 workspace");
    if (((uintptr_t)d_x & 15u) != 0 || ((uintptr_t)d_xq & 15u) != 0 || ((uintptr_t)d_ws & 15u) != 0)
        return set_error(JQ_ERR_ALIGN, "activations, Q8_1 blocks and workspace must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // one launch over the concatenated rows while the decode kernels take the shape
    bool all_rows = true;
    for (int i = 0; i < n_mats; ++i) all_rows = all_rows && N[i] > 0;
    if (K > 0 && M <= 8 && all_rows) {
        MultiMat mm{};
        mm.n = n_mats;
        for (int i = 0; i < n_mats; ++i) {
            mm.w[i] = d_w[i];
            mm.y[i] = d_y[i];
            mm.rows[i] = N[i];
        }
        const bool fuse_quantizer = d_x != nullptr && fuse_quantizer_pays(M, K);
        if (d_x != nullptr && !fuse_quantizer) {
            if (int rc = launch_quantize_q8_1(st, d_x, d_ws, K, M, JQ_ORDER_COL_KSUPER, s_mode)) return rc;
        }
        const float *xf = fuse_quantizer ? d_x : nullptr;
        const void *xq = fuse_quantizer ? nullptr : (d_x != nullptr ? d_ws : d_xq);
        int rc = JQ_ERR_UNSUPPORTED;
        if (M <= 2) rc = launch_gemv_dp4a(st, nullptr, xq, xf, fuse_quantizer ? d_ws : nullptr, nullptr, K, n_total, M,
                                          JQ_ORDER_COL_KSUPER, s_mode, nullptr, &mm);
        if (rc == JQ_ERR_UNSUPPORTED)
            rc = launch_gemv_mma(st, nullptr, xq, xf, fuse_quantizer ? d_ws : nullptr, nullptr, K, n_total, M, JQ_ORDER_COL_KSUPER,
                                 s_mode, &mm);
        if (rc != JQ_ERR_UNSUPPORTED) return rc;
        // not a shape for the decode kernels: the activations may already be quantized in d_ws, go on below
        if (d_x != nullptr && !fuse_quantizer) {
            d_xq = d_ws;
            d_x = nullptr;
        }
    }
    if (d_x != nullptr && K > 0) {
        if (int rc = launch_quantize_q8_1(st, d_x, d_ws, K, M, JQ_ORDER_COL_KSUPER, s_mode)) return rc;
        d_xq = d_ws;
    }
    for (int i = 0; i < n_mats; ++i) {
        if (N[i] == 0) continue;
        if (int rc = dispatch_mul_mat(st, d_w[i], d_xq, d_y[i], K, N[i], M, JQ_ORDER_COL_KSUPER, JQ_KERNEL_AUTO)) return rc;
    }
    return JQ_OK;
}

// ---- N-sharded decode: multiply + all-gather in one kernel -----------------------------------------

int jq_peer_alloc(size_t bytes, void **d_ptr, unsigned char *handle_out) {
    if (!d_ptr || !handle_out || bytes == 0) return set_error(JQ_ERR_INVALID_ARG, "jq_peer_alloc: bad argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == JQ_PEER_HANDLE_BYTES, "handle size");
    void *p = nullptr;
    JQ_CUDA_TRY(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return cuda_error(e, "jq_peer_alloc");
    }
    std::memcpy(handle_out, &h, sizeof(h));
    *d_ptr = p;
    return JQ_OK;
}

int jq_peer_open(const unsigned char *handle, void **d_ptr) {
    if (!d_ptr || !handle) return set_error(JQ_ERR_INVALID_ARG, "jq_peer_open: bad argument");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    JQ_CUDA_TRY(cudaIpcOpenMemHandle(d_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return JQ_OK;
}

int jq_peer_close(void *d_ptr) {
    if (d_ptr) JQ_CUDA_TRY(cudaIpcCloseMemHandle(d_ptr));
    return JQ_OK;
}

int jq_peer_free(void *d_ptr) {
    if (d_ptr) JQ_CUDA_TRY(cudaFree(d_ptr));
    return JQ_OK;
}

int jq_linear_q4_0_allgather_device(void *stream, const void *d_w, const float *d_x, void *d_ws, int64_t K,
                                    int64_t N_local, int64_t M, int s_mode, void *const *y_peers,
                                    void *const *flag_peers, int world, int rank, int64_t n_offset, int64_t N_total,
                                    size_t y_stride_bytes, int wait_previous, unsigned *d_epoch, int *d_counter) {
    if (int rc = check_mul_mat_shape(K, N_local, M)) return rc;
    if (int rc = check_s_mode(s_mode)) return rc;
    if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world)
        return set_error(JQ_ERR_INVALID_ARG, "world must be 1..%d and rank inside it (world=%d rank=%d)", MAX_PEERS, world, rank);
    if (!y_peers || !flag_peers || !d_counter || !d_epoch || !d_w || !d_x) return set_error(JQ_ERR_INVALID_ARG, "null pointer");
    if (n_offset < 0 || n_offset + N_local > N_total) return set_error(JQ_ERR_INVALID_ARG, "band [%lld, %lld) outside N_total = %lld",
                                                                       (long long)n_offset, (long long)(n_offset + N_local), (long long)N_total);
    if (M < 1 || N_local < 1 || K < 1) return set_error(JQ_ERR_INVALID_ARG, "empty shape");
    if (M > 2 && d_ws == nullptr) return set_error(JQ_ERR_INVALID_ARG, "M > 2 needs the Q8_1 workspace");
    // Everything a kernel of this call may refuse is checked before anything is queued: a rank that queued its
    // flag wait and then returned an error would leave every peer spinning for a band that never comes.
    if (K % 256 != 0) return set_error(JQ_ERR_UNSUPPORTED, "the fused all-gather needs K %% 256 == 0 (K = %lld)", (long long)K);
    if (((uintptr_t)d_w & 15u) != 0) return set_error(JQ_ERR_UNSUPPORTED, "the fused all-gather needs 16-byte aligned weights");
    if (((uintptr_t)d_x & 15u) != 0 || (d_ws && ((uintptr_t)d_ws & 15u) != 0))
        return set_error(JQ_ERR_ALIGN, "activations and workspace must be 16-byte aligned");
    GatherArgs ga;
    for (int q = 0; q < MAX_PEERS; ++q) {
        ga.y_peer[q] = q < world ? static_cast<float *>(y_peers[q]) : nullptr;
        ga.flag_peer[q] = q < world ? static_cast<uint32_t *>(flag_peers[q]) : nullptr;
        if (q < world && (!ga.y_peer[q] || !ga.flag_peer[q])) return set_error(JQ_ERR_INVALID_ARG, "null peer pointer %d", q);
    }
    ga.world = world;
    ga.rank = rank;
    ga.n_offset = n_offset;
    ga.N_total = N_total;
    ga.epoch_ptr = d_epoch;
    ga.y_stride_bytes = y_stride_bytes;
    ga.wait_previous = wait_previous;
    ga.counter = d_counter;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (M <= 2) {
        const int rc = launch_gemv_dp4a(st, d_w, nullptr, d_x, d_ws, nullptr, K, N_local, M, JQ_ORDER_COL_KSUPER, s_mode, &ga);
        if (rc != JQ_ERR_UNSUPPORTED || d_ws == nullptr) return rc;
    }
    // Larger batches (and decode shapes the streaming kernel refuses): quantize, then the tensor-core GEMM
    // whose epilogue stores its tiles into every rank's buffer.  The activations are this call's input, not
    // a gathered output the kernel could wait for itself: queue jq_allgather_wait_device first if they are.
    if (wait_previous) {
        if (int rc = launch_allgather_wait(st, ga.flag_peer[rank], world, d_epoch)) return rc;
    }
    if (int rc = launch_quantize_q8_1(st, d_x, d_ws, K, M, JQ_ORDER_COL_KSUPER, s_mode)) return rc;
    return launch_gemm_mma(st, d_w, d_ws, nullptr, K, N_local, M, JQ_ORDER_COL_KSUPER, &ga);
}

int jq_allgather_wait_device(void *stream, const void *d_flags, int world, const unsigned *d_epoch) {
    if (!d_flags || !d_epoch || world < 1 || world > MAX_PEERS) return set_error(JQ_ERR_INVALID_ARG, "bad pointer or world size");
    return launch_allgather_wait(static_cast<cudaStream_t>(stream), static_cast<const uint32_t *>(d_flags), world, d_epoch);
}

int jq_linear_q4_0_allgather_tagged_device(void *stream, const void *d_w, const float *d_x, const void *d_x_words,
                                           size_t x_stride_bytes, int64_t x_row_words, int64_t x_seg_len, int64_t x_seg_stride,
                                           int x_back, int64_t K, int64_t N_local, int64_t M, int s_mode, void *const *word_peers, int world,
                                           int rank, int64_t n_offset, int64_t N_total, size_t y_stride_bytes,
                                           unsigned long long *d_ticket) {
    if (int rc = check_mul_mat_shape(K, N_local, M)) return rc;
    if (int rc = check_s_mode(s_mode)) return rc;
    if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world)
        return set_error(JQ_ERR_INVALID_ARG, "world must be 1..%d and rank inside it (world=%d rank=%d)", MAX_PEERS, world, rank);
    if (!word_peers || !d_ticket || !d_w || (d_x == nullptr) == (d_x_words == nullptr))
        return set_error(JQ_ERR_INVALID_ARG, "null pointer, or not exactly one of d_x and d_x_words");
    if (n_offset < 0 || n_offset + N_local > N_total) return set_error(JQ_ERR_INVALID_ARG, "band [%lld, %lld) outside N_total = %lld",
                                                                       (long long)n_offset, (long long)(n_offset + N_local), (long long)N_total);
    if (M < 1 || N_local < 1 || K < 1) return set_error(JQ_ERR_INVALID_ARG, "empty shape");
    if (M > 2) return set_error(JQ_ERR_UNSUPPORTED, "the tagged all-gather is the decode form: M <= 2 (M = %lld)", (long long)M);
    if (K % 256 != 0) return set_error(JQ_ERR_UNSUPPORTED, "the fused all-gather needs K %% 256 == 0 (K = %lld)", (long long)K);
    if (((uintptr_t)d_w & 15u) != 0) return set_error(JQ_ERR_UNSUPPORTED, "the fused all-gather needs 16-byte aligned weights");
    if (d_x && ((uintptr_t)d_x & 15u) != 0) return set_error(JQ_ERR_ALIGN, "activations must be 16-byte aligned");
    if ((n_offset & 1) != 0 || (N_total & 1) != 0 || (y_stride_bytes & 15u) != 0)
        return set_error(JQ_ERR_ALIGN, "band offset and N_total must be even, the buffers 16-byte aligned");
    GatherArgs ga;
    for (int q = 0; q < MAX_PEERS; ++q) {
        ga.y_peer[q] = q < world ? static_cast<float *>(word_peers[q]) : nullptr;
        if (q < world && (!ga.y_peer[q] || ((uintptr_t)ga.y_peer[q] & 15u) != 0))
            return set_error(JQ_ERR_INVALID_ARG, "null or misaligned peer pointer %d", q);
    }
    if (d_x_words) {
        if (x_back < 0 || x_back > 64) return set_error(JQ_ERR_INVALID_ARG, "x_back = %d", x_back);
        if (x_seg_len < 8 || x_seg_len % 8 != 0 || K % x_seg_len != 0 || x_seg_stride < 0 || (x_seg_stride & 1) != 0 ||
            (x_row_words & 1) != 0 || ((uintptr_t)d_x_words & 15u) != 0 || (x_stride_bytes & 15u) != 0 ||
            (K / x_seg_len - 1) * x_seg_stride + x_seg_len > x_row_words)
            return set_error(JQ_ERR_INVALID_ARG, "activation words: segments of %lld every %lld words do not tile K = %lld inside a row of %lld",
                             (long long)x_seg_len, (long long)x_seg_stride, (long long)K, (long long)x_row_words);
        ga.x_words = static_cast<const unsigned long long *>(d_x_words);
        ga.x_stride_bytes = x_stride_bytes;
        ga.x_row_words = x_row_words;
        ga.x_seg_len = (int)x_seg_len;
        ga.x_seg_stride = x_seg_stride;
        ga.x_back = x_back;
        ga.x_wide = (x_seg_stride & 3) == 0 && (x_row_words & 3) == 0 && ((uintptr_t)d_x_words & 31u) == 0 && (x_stride_bytes & 31u) == 0;
    }
    ga.world = world;
    ga.rank = rank;
    ga.n_offset = n_offset;
    ga.N_total = N_total;
    ga.y_stride_bytes = y_stride_bytes;
    ga.ticket = d_ticket;
    return launch_gemv_dp4a(static_cast<cudaStream_t>(stream), d_w, nullptr, d_x, nullptr, nullptr, K, N_local, M, JQ_ORDER_COL_KSUPER,
                            s_mode, &ga);
}

int jq_allgather_tagged_read_device(void *stream, const void *d_words, size_t stride_bytes, int64_t M, int64_t N_total,
                                    const unsigned long long *d_ticket, float *d_out) {
    if (!d_words || !d_ticket || !d_out || M < 1 || N_total < 2 || (N_total & 1) != 0 || ((uintptr_t)d_words & 15u) != 0 ||
        ((uintptr_t)d_out & 7u) != 0 || (stride_bytes & 15u) != 0)
        return set_error(JQ_ERR_INVALID_ARG, "jq_allgather_tagged_read_device: bad pointer, size or alignment");
    return launch_allgather_tagged_read(static_cast<cudaStream_t>(stream), static_cast<const unsigned long long *>(d_words), stride_bytes,
                                        M, N_total, d_ticket, d_out);
}

// ---- the entry point that allocates nothing ---------------------------------------------------------
// Scratch for the quantized activations, part of the library image (see include/jq_b200.h).  In host
// code this name is only a handle for the runtime: the kernels must be given the device address that
// cudaGetSymbolAddress() returns for the device that is current at the time.
static __device__ __align__(256) uint8_t g_noalloc_ws[JQ_NOALLOC_WS_BYTES];

namespace {
struct NoAllocSlot {
    bool ready = false;
    void *ws = nullptr;
};
NoAllocSlot g_noalloc[jq::MAX_DEVICES];
std::mutex g_noalloc_mutex;

// Once per device, with that device current: resolve the array's address on that device.
int noalloc_workspace(void **out) {
    int dev = 0;
    JQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= jq::MAX_DEVICES) return set_error(JQ_ERR_UNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    NoAllocSlot &slot = g_noalloc[dev];
    if (!slot.ready) {
        void *ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_ws);
        if (e != cudaSuccess) return cuda_error(e, "cudaGetSymbolAddress(g_noalloc_ws)");
        if (ptr == nullptr) return set_error(JQ_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        slot.ws = ptr;
        slot.ready = true;
    }
    *out = slot.ws;
    return JQ_OK;
}
}  // namespace

int jq_linear_q4_0_device_noalloc(void *stream, const void *d_w, const float *d_x, float *d_y, int64_t K, int64_t N,
                                  int64_t M, int s_mode) {
    if (int rc = check_mul_mat_shape(K, N, M)) return rc;
    const size_t need = jq_q8_1_bytes(K, M);
    if (need > (size_t)JQ_NOALLOC_WS_BYTES)
        return set_error(JQ_ERR_TOO_LARGE,
                         "jq_linear_q4_0_device_noalloc: M = %lld, K = %lld need %zu bytes of Q8_1 scratch, the built-in "
                         "array holds %u; use jq_linear_q4_0_device with a caller-owned workspace",
                         (long long)M, (long long)K, need, (unsigned)JQ_NOALLOC_WS_BYTES);
    void *ws = nullptr;
    if (int rc = noalloc_workspace(&ws)) return rc;
    return jq_linear_q4_0_device(stream, d_w, d_x, ws, d_y, K, N, M, s_mode);
}

int jq_block_sums_q4_0_q8_1_device(void *stream, const void *d_w, const void *d_xq, int32_t *d_sums, int64_t K,
                                   int64_t N, int64_t M, int order) {
    if (int rc = check_mul_mat_shape(K, N, M)) return rc;
    if (int rc = check_order(order)) return rc;
    if (N == 0 || M == 0 || K == 0) return JQ_OK;
    if (d_w == nullptr || d_xq == nullptr || d_sums == nullptr) return set_error(JQ_ERR_INVALID_ARG, "null pointer");
    if (((uintptr_t)d_xq & 15u) != 0) return set_error(JQ_ERR_ALIGN, "Q8_1 blocks must be 16-byte aligned");
    return launch_block_sums(static_cast<cudaStream_t>(stream), d_w, d_xq, d_sums, K, N, M, order);
}

int jq_quantize_q4_0_device(void *stream, const float *d_w, void *d_wq, int64_t N, int64_t K) {
    if (N < 0 || K < 0) return set_error(JQ_ERR_INVALID_ARG, "negative size");
    if (K % QK != 0) return set_error(JQ_ERR_SHAPE, "K = %lld is not a multiple of %d", (long long)K, QK);
    if (N == 0 || K == 0) return JQ_OK;
    if (d_w == nullptr || d_wq == nullptr) return set_error(JQ_ERR_INVALID_ARG, "null pointer");
    if (((uintptr_t)d_w & 15u) != 0 || ((uintptr_t)d_wq & 1u) != 0)
        return set_error(JQ_ERR_ALIGN, "weights must be 16-byte aligned, Q4_0 output 2-byte aligned");
    return launch_quantize_q4_0(static_cast<cudaStream_t>(stream), d_w, d_wq, N, K);
}

int jq_device_fault(int clear, int *fault_out) {
    int *p = device_fault_ptr();
    if (p == nullptr) return set_error(JQ_ERR_CUDA, "cannot locate the device fault word");
    int v = 0;
    JQ_CUDA_TRY(cudaDeviceSynchronize());
    JQ_CUDA_TRY(cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost));
    if (clear && v != 0) {
        const int zero = 0;
        JQ_CUDA_TRY(cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice));
        if (int rc = reset_gemm_f16_split_state()) return rc;
    }
    if (fault_out) *fault_out = v;
    if (v == 3)
        return set_error(JQ_ERR_TIMEOUT, "a range check of the debug build failed: an access outside its buffer was skipped");
    if (v != 0)
        return set_error(JQ_ERR_TIMEOUT, "a kernel gave up on a bounded wait (%s): its results are not valid",
                         v == 2 ? "bands of an all-gather did not arrive" : "a bulk copy or pipeline stage did not complete");
    return JQ_OK;
}

int jq_bounds_checked(void) { return BOUNDS_CHECK ? 1 : 0; }

int jq_debug_set_extent_shrink(unsigned long long bytes) {
    g_extent_shrink.store(bytes, std::memory_order_relaxed);
    return JQ_OK;
}

// ---- host entry points -----------------------------------------------------------------------

namespace {

struct DeviceScratch {
    cudaStream_t stream = nullptr;
    void *ptrs[4] = {nullptr, nullptr, nullptr, nullptr};
    int n = 0;
    int alloc(void **out, size_t bytes) {
        *out = nullptr;
        if (bytes == 0) return JQ_OK;
        JQ_CUDA_TRY(cudaMallocAsync(out, bytes, stream));
        ptrs[n++] = *out;
        return JQ_OK;
    }
    int open() {
        JQ_CUDA_TRY(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
        return JQ_OK;
    }
    ~DeviceScratch() {
        if (stream) {
            for (int i = 0; i < n; ++i) cudaFreeAsync(ptrs[i], stream);
            cudaStreamSynchronize(stream);
            cudaStreamDestroy(stream);
        }
    }
};

}  // namespace

int jq_q8_1_host(const float *input, uint8_t *output, const int *dims, int ndims) {
    if (dims == nullptr || ndims < 1) return set_error(JQ_ERR_INVALID_ARG, "dims missing");
    const int64_t ne0 = dims[0];
    const int64_t ne1 = ndims > 1 ? dims[1] : 1;
    const int64_t ne2 = ndims > 2 ? dims[2] : 1;
    const int64_t ne3 = ndims > 3 ? dims[3] : 1;
    if (ne0 < 0 || ne1 < 0 || ne2 < 0 || ne3 < 0) return set_error(JQ_ERR_INVALID_ARG, "negative dimension");
    const int64_t M = ne1 * ne2 * ne3;  // every row of length ne0 is one column of the multiply
    if (ne0 == 0 || M == 0) return JQ_OK;
    if (input == nullptr || output == nullptr) return set_error(JQ_ERR_INVALID_ARG, "null pointer");
    if (ne0 % QK != 0) return set_error(JQ_ERR_SHAPE, "dims[0] = %lld is not a multiple of %d", (long long)ne0, QK);
    DeviceScratch s;
    if (int rc = s.open()) return rc;
    void *d_x, *d_y;
    const size_t in_bytes = (size_t)ne0 * M * sizeof(float), out_bytes = jq_q8_1_bytes(ne0, M);
    if (int rc = s.alloc(&d_x, in_bytes)) return rc;
    if (int rc = s.alloc(&d_y, out_bytes)) return rc;
    JQ_CUDA_TRY(cudaMemcpyAsync(d_x, input, in_bytes, cudaMemcpyHostToDevice, s.stream));
    if (int rc = launch_quantize_q8_1(s.stream, static_cast<const float *>(d_x), d_y, ne0, M, JQ_ORDER_KSUPER_COL, JQ_S_SUM_X))
        return rc;
    JQ_CUDA_TRY(cudaMemcpyAsync(output, d_y, out_bytes, cudaMemcpyDeviceToHost, s.stream));
    JQ_CUDA_TRY(cudaStreamSynchronize(s.stream));
    return JQ_OK;
}

int jq_parse_q8_1_output(const uint8_t *input, int8_t *qs_out, float *scale_out, float *sum_out, int64_t n_blocks) {
    if (n_blocks < 0) return set_error(JQ_ERR_INVALID_ARG, "negative block count");
    if (n_blocks == 0) return JQ_OK;
    if (!input || !qs_out || !scale_out || !sum_out) return set_error(JQ_ERR_INVALID_ARG, "null pointer");
    for (int64_t b = 0; b < n_blocks; ++b) {
        const uint8_t *blk = input + b * Q8_BYTES;
        std::memcpy(qs_out + b * SUPER, blk + Q8_QS_OFFSET, SUPER);
        for (int g = 0; g < 4; ++g) {
            __half h[2];
            std::memcpy(h, blk + 4 * g, 4);
            scale_out[b * 4 + g] = __half2float(h[0]);
            sum_out[b * 4 + g] = __half2float(h[1]);
        }
    }
    return JQ_OK;
}

int jq_mat_mul_q4_0_q8_1_host_ex(const void *weight_q4_0, const float *input, uint8_t *quant_workspace,
                                 float *output, const int *input_dims, int ndims, int nrows_out, int ncols_k,
                                 int s_mode) {
    if (input_dims == nullptr || ndims < 2) return set_error(JQ_ERR_INVALID_ARG, "input_dims needs at least 2 entries");
    const int64_t ne0 = input_dims[0], ne1 = input_dims[1];
    const int64_t ne2 = ndims > 2 ? input_dims[2] : 1, ne3 = ndims > 3 ? input_dims[3] : 1;
    if (ne0 != ncols_k) return set_error(JQ_ERR_SHAPE, "input_dims[0]=%lld must equal ncols_k=%d", (long long)ne0, ncols_k);
    if (nrows_out < 0 || ne1 < 0 || ne2 < 0 || ne3 < 0) return set_error(JQ_ERR_INVALID_ARG, "negative dimension");
    const int64_t K = ncols_k, N = nrows_out, M = ne1 * ne2 * ne3;
    if (int rc = check_mul_mat_shape(K, N, M)) return rc;
    if (int rc = check_s_mode(s_mode)) return rc;
    if (M == 0) return JQ_OK;
    if ((K > 0 && (input == nullptr || (N > 0 && weight_q4_0 == nullptr))) || (N > 0 && output == nullptr))
        return set_error(JQ_ERR_INVALID_ARG, "null pointer");
    DeviceScratch s;
    if (int rc = s.open()) return rc;
    void *d_w, *d_x, *d_ws, *d_y;
    const size_t w_bytes = jq_q4_0_bytes(N, K), x_bytes = (size_t)M * K * sizeof(float);
    const size_t ws_bytes = jq_q8_1_bytes(K, M), y_bytes = (size_t)M * N * sizeof(float);
    if (int rc = s.alloc(&d_w, w_bytes)) return rc;
    if (int rc = s.alloc(&d_x, x_bytes)) return rc;
    if (int rc = s.alloc(&d_ws, ws_bytes)) return rc;
    if (int rc = s.alloc(&d_y, y_bytes)) return rc;
    if (w_bytes) JQ_CUDA_TRY(cudaMemcpyAsync(d_w, weight_q4_0, w_bytes, cudaMemcpyHostToDevice, s.stream));
    if (x_bytes) JQ_CUDA_TRY(cudaMemcpyAsync(d_x, input, x_bytes, cudaMemcpyHostToDevice, s.stream));
    if (K > 0) {
        // the workspace keeps the order q8_1() writes (q8_1.cu:84-86) ...
        if (int rc = launch_quantize_q8_1(s.stream, static_cast<const float *>(d_x), d_ws, K, M, JQ_ORDER_KSUPER_COL, s_mode))
            return rc;
        if (quant_workspace) JQ_CUDA_TRY(cudaMemcpyAsync(quant_workspace, d_ws, ws_bytes, cudaMemcpyDeviceToHost, s.stream));
    }
    if (N > 0) {
        // ... and the multiply is told so, which the reference's own kernel is not (it reads
        // m * (K/128) + k/128, mm_q4_0_q8_1.cu:230) and therefore mixes columns for M > 1.
        if (int rc = dispatch_mul_mat(s.stream, d_w, d_ws, static_cast<float *>(d_y), K, N, M, JQ_ORDER_KSUPER_COL, JQ_KERNEL_AUTO))
            return rc;
        JQ_CUDA_TRY(cudaMemcpyAsync(output, d_y, y_bytes, cudaMemcpyDeviceToHost, s.stream));
    }
    JQ_CUDA_TRY(cudaStreamSynchronize(s.stream));
    return JQ_OK;
}

int jq_mat_mul_q4_0_q8_1_host(const void *weight_q4_0, const float *input, uint8_t *quant_workspace, float *output,
                              const int *input_dims, int ndims, int nrows_out, int ncols_k) {
    return jq_mat_mul_q4_0_q8_1_host_ex(weight_q4_0, input, quant_workspace, output, input_dims, ndims, nrows_out,
                                        ncols_k, JQ_S_SUM_X);
}

// ---- resident weights ----------------------------------------------------------------------------

struct jq_weights {
    void *d_w = nullptr;
    int64_t N = 0, K = 0;
    int device = 0;
    cudaStream_t stream = nullptr;
    void *d_x = nullptr, *d_ws = nullptr, *d_y = nullptr;
    int64_t m_cap = 0;
    // device aliases of the current call's host buffers (non-null when the buffer is pinned and mapped)
    const float *x_alias = nullptr;
    float *y_alias = nullptr;
    // completion ticket in pinned, mapped host memory (written by the copy kernel, polled by the host)
    unsigned *h_done = nullptr;
    unsigned *d_done = nullptr;
    unsigned *d_count = nullptr;  // the completion count kept on the device (the copy kernel never reads the one in host memory)
    unsigned ticket = 0;
    // the three launches of a zero-copy call (quantize, multiply, copy back) as one graph, built the
    // second time the same buffers and batch size are seen
    cudaGraphExec_t graph = nullptr;
    const void *graph_x = nullptr;
    const void *graph_y = nullptr;
    int64_t graph_m = 0;
    int graph_s_mode = 0;
    int graph_hits = 0;
};



int jq_weights_create(const void *host_w_q4_0, int64_t N, int64_t K, jq_weights **out) {
    if (out == nullptr) return set_error(JQ_ERR_INVALID_ARG, "null out pointer");
    *out = nullptr;
    if (int rc = check_mul_mat_shape(K, N, 0)) return rc;
    if (host_w_q4_0 == nullptr && N * K > 0) return set_error(JQ_ERR_INVALID_ARG, "null weights");
    jq_weights *w = new (std::nothrow) jq_weights();
    if (!w) return set_error(JQ_ERR_CUDA, "out of host memory");
    w->N = N;
    w->K = K;
    cudaError_t e = cudaGetDevice(&w->device);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&w->stream, cudaStreamNonBlocking);
    const size_t bytes = jq_q4_0_bytes(N, K);
    if (e == cudaSuccess && bytes) e = cudaMalloc(&w->d_w, bytes);
    if (e == cudaSuccess && bytes) e = cudaMemcpy(w->d_w, host_w_q4_0, bytes, cudaMemcpyHostToDevice);
    if (e == cudaSuccess && cudaHostAlloc(reinterpret_cast<void **>(&w->h_done), 64, cudaHostAllocMapped) == cudaSuccess) {
        *w->h_done = 0;
        if (cudaHostGetDevicePointer(reinterpret_cast<void **>(&w->d_done), w->h_done, 0) != cudaSuccess) w->d_done = nullptr;
        if (w->d_done != nullptr && (cudaMalloc(reinterpret_cast<void **>(&w->d_count), sizeof(unsigned)) != cudaSuccess ||
                                     cudaMemset(w->d_count, 0, sizeof(unsigned)) != cudaSuccess)) {
            (void)cudaGetLastError();
            w->d_done = nullptr;
        }
    } else {
        (void)cudaGetLastError();  // no ticket: completion falls back to stream synchronisation
    }
    if (e != cudaSuccess) {
        const int rc = cuda_error(e, "jq_weights_create");
        jq_weights_destroy(w);
        return rc;
    }
    *out = w;
    return JQ_OK;
}

int jq_weights_destroy(jq_weights *w) {
    if (!w) return JQ_OK;
    if (w->stream) cudaStreamSynchronize(w->stream);
    cudaFree(w->d_w);
    cudaFree(w->d_x);
    cudaFree(w->d_ws);
    cudaFree(w->d_y);
    if (w->graph) cudaGraphExecDestroy(w->graph);
    if (w->h_done) cudaFreeHost(w->h_done);
    cudaFree(w->d_count);
    if (w->stream) cudaStreamDestroy(w->stream);
    delete w;
    return JQ_OK;
}

const void *jq_weights_device_ptr(const jq_weights *w) { return w ? w->d_w : nullptr; }

int jq_linear_q4_0_host(jq_weights *w, const float *x, uint8_t *quant_workspace, float *y, int64_t M, int s_mode) {
    if (!w) return set_error(JQ_ERR_INVALID_ARG, "null weights handle");
    if (M < 0) return set_error(JQ_ERR_INVALID_ARG, "negative M");
    if (int rc = check_s_mode(s_mode)) return rc;
    if (M == 0) return JQ_OK;
    if (!x || !y) return set_error(JQ_ERR_INVALID_ARG, "null pointer");
    if (M > w->m_cap) {  // staging buffers grow, never shrink
        JQ_CUDA_TRY(cudaStreamSynchronize(w->stream));
        cudaFree(w->d_x);
        cudaFree(w->d_ws);
        cudaFree(w->d_y);
        w->d_x = w->d_ws = w->d_y = nullptr;
        w->m_cap = 0;
        JQ_CUDA_TRY(cudaMalloc(&w->d_x, (size_t)M * w->K * sizeof(float) + 16));
        JQ_CUDA_TRY(cudaMalloc(&w->d_ws, jq_q8_1_bytes(w->K, M) + 16));
        JQ_CUDA_TRY(cudaMalloc(&w->d_y, (size_t)M * w->N * sizeof(float) + 16));
        w->m_cap = M;
    }
    // Asked on every call: a buffer freed and allocated again may come back at the same address
    // with a different mapping, and a stale alias would be a wild device pointer.
    w->x_alias = static_cast<const float *>(mapped_alias(x));
    w->y_alias = static_cast<float *>(mapped_alias(y));
    const size_t y_count = (size_t)M * w->N;
    // Small decode batches from pinned, mapped host memory skip the copy engines: the quantizer
    // reads the activations over the bus itself and a copy kernel writes the result back.
    const bool zero_copy_in = w->x_alias != nullptr && M <= 8 && ((uintptr_t)w->x_alias & 15u) == 0 && w->K % SUPER == 0;
    const bool zero_copy_out = w->y_alias != nullptr && y_count * sizeof(float) <= (1u << 20) && ((uintptr_t)w->y_alias & 15u) == 0;
    const bool ticketed = zero_copy_in && zero_copy_out && y_count <= 65536 && w->d_done != nullptr && quant_workspace == nullptr;

    auto enqueue = [&]() -> int {
        if (zero_copy_in) {
            if (int rc = launch_quantize_q8_1(w->stream, w->x_alias, w->d_ws, w->K, M, JQ_ORDER_COL_KSUPER, s_mode)) return rc;
            if (int rc = dispatch_mul_mat(w->stream, w->d_w, w->d_ws, static_cast<float *>(w->d_y), w->K, w->N, M,
                                          JQ_ORDER_COL_KSUPER, JQ_KERNEL_AUTO))
                return rc;
        } else {
            JQ_CUDA_TRY(cudaMemcpyAsync(w->d_x, x, (size_t)M * w->K * sizeof(float), cudaMemcpyHostToDevice, w->stream));
            if (int rc = jq_linear_q4_0_device(w->stream, w->d_w, static_cast<const float *>(w->d_x), w->d_ws,
                                               static_cast<float *>(w->d_y), w->K, w->N, M, s_mode))
                return rc;
        }
        if (quant_workspace)
            JQ_CUDA_TRY(cudaMemcpyAsync(quant_workspace, w->d_ws, jq_q8_1_bytes(w->K, M), cudaMemcpyDeviceToHost, w->stream));
        if (zero_copy_out) {
            const int threads = ticketed ? 1024 : 256;
            const int blocks = ticketed ? 1 : (int)std::min<size_t>(8, (y_count / 4 + threads - 1) / threads + 1);
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)blocks);
            cfg.blockDim = dim3(threads);
            cfg.stream = w->stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            volatile unsigned *flag = ticketed ? w->d_done : nullptr;
            JQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, copy_f32_kernel, w->y_alias, static_cast<const float *>(w->d_y),
                                           (int64_t)y_count, flag, w->d_count));
        } else {
            JQ_CUDA_TRY(cudaMemcpyAsync(y, w->d_y, y_count * sizeof(float), cudaMemcpyDeviceToHost, w->stream));
        }
        return JQ_OK;
    };

    bool launched = false;
    if (ticketed) {
        const bool same = w->graph_x == w->x_alias && w->graph_y == w->y_alias && w->graph_m == M && w->graph_s_mode == s_mode;
        if (!same) {
            if (w->graph) {
                JQ_CUDA_TRY(cudaStreamSynchronize(w->stream));
                cudaGraphExecDestroy(w->graph);
                w->graph = nullptr;
            }
            w->graph_x = w->x_alias;  // the recorded launches hold the device aliases, so they are the key
            w->graph_y = w->y_alias;
            w->graph_m = M;
            w->graph_s_mode = s_mode;
            w->graph_hits = 0;
        } else if (w->graph == nullptr && ++w->graph_hits >= 2) {
            // third call with the same buffers: record the three launches once, replay them from now on
            cudaGraph_t g = nullptr;
            if (cudaStreamBeginCapture(w->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
                const int rc = enqueue();
                const cudaError_t e = cudaStreamEndCapture(w->stream, &g);
                if (rc == JQ_OK && e == cudaSuccess && g != nullptr) {
                    if (cudaGraphInstantiate(&w->graph, g, 0) != cudaSuccess) w->graph = nullptr;
                }
                if (g) cudaGraphDestroy(g);
            }
            (void)cudaGetLastError();
        }
        if (w->graph != nullptr) {
            JQ_CUDA_TRY(cudaGraphLaunch(w->graph, w->stream));
            launched = true;
        }
    }
    unsigned expect = 0;
    if (ticketed) expect = w->ticket + 1;  // the flag counts completed ticketed calls
    if (!launched) {
        if (int rc = enqueue()) {
            // part of the call may be queued: drain it and take the count as it stands, so that the next
            // call's expectation matches the device again
            cudaStreamSynchronize(w->stream);
            (void)cudaGetLastError();
            if (w->h_done) w->ticket = *static_cast<volatile unsigned *>(w->h_done);
            return rc;
        }
    }
    if (ticketed) w->ticket = expect;
    bool polled = false;
    if (ticketed) {
        volatile unsigned *h = w->h_done;
        for (long spin = 0; spin < 20000000L; ++spin) {
            if ((int)(*h - expect) >= 0) {
                polled = true;
                break;
            }
        }
    }
    if (!polled) {
        JQ_CUDA_TRY(cudaStreamSynchronize(w->stream));
        if (ticketed) w->ticket = *static_cast<volatile unsigned *>(w->h_done);  // resynchronise after a slow call
    }
    return JQ_OK;
}

// ---- device description -----------------------------------------------------------------------------

int jq_query_device_hw_info(int device, jq_device_hw_info *out) {
    if (!out) return set_error(JQ_ERR_INVALID_ARG, "null out pointer");
    std::memset(out, 0, sizeof(*out));
    cudaDeviceProp prop{};
    JQ_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    std::strncpy(out->name, prop.name, sizeof(out->name) - 1);
    out->device_id = device;
    out->cc_major = prop.major;
    out->cc_minor = prop.minor;
    out->sm_count = prop.multiProcessorCount;
    JQ_CUDA_TRY(cudaDeviceGetAttribute(&out->sm_clock_khz, cudaDevAttrClockRate, device));
    JQ_CUDA_TRY(cudaDeviceGetAttribute(&out->mem_clock_khz, cudaDevAttrMemoryClockRate, device));
    JQ_CUDA_TRY(cudaDeviceGetAttribute(&out->mem_bus_width_bits, cudaDevAttrGlobalMemoryBusWidth, device));
    out->smem_per_sm = prop.sharedMemPerMultiprocessor;
    out->smem_per_block_optin = prop.sharedMemPerBlockOptin;
    out->l2_bytes = (size_t)prop.l2CacheSize;
    out->global_mem_bytes = prop.totalGlobalMem;
    out->max_warps_per_sm = prop.maxThreadsPerMultiProcessor / (prop.warpSize > 0 ? prop.warpSize : 32);
    const int cc = prop.major * 10 + prop.minor;
    // per-SM tables: CUDA cores, schedulers, dense tensor MACs per clock.  The sm_100 tensor rates
    // are NVIDIA's published dense B200 peaks (2.25 PFLOP/s bf16, 4.5 POP/s int8) divided by
    // 148 SMs x 1.86 GHz.
    int tc_bf16_mac = 0, tc_int8_mac = 0;
    switch (cc) {
        case 80: out->fp32_cores_per_sm = 64; tc_bf16_mac = 1024; tc_int8_mac = 2048; break;
        case 86: case 87: case 89: out->fp32_cores_per_sm = 128; tc_bf16_mac = 512; tc_int8_mac = 1024; break;
        case 90: out->fp32_cores_per_sm = 128; tc_bf16_mac = 2048; tc_int8_mac = 4096; break;
        case 100: case 103: out->fp32_cores_per_sm = 128; tc_bf16_mac = 4096; tc_int8_mac = 8192; break;
        default: out->fp32_cores_per_sm = cc >= 100 ? 128 : 0; break;
    }
    out->warp_schedulers_per_sm = cc >= 70 ? 4 : 0;
    const double sm_hz = (double)out->sm_clock_khz * 1e3;
    out->peak_fp32_tflops = (double)out->sm_count * out->fp32_cores_per_sm * 2.0 * sm_hz / 1e12;
    out->peak_bf16_dense_tflops = (double)out->sm_count * tc_bf16_mac * 2.0 * sm_hz / 1e12;
    out->peak_int8_dense_tops = (double)out->sm_count * tc_int8_mac * 2.0 * sm_hz / 1e12;
    // DDR formula of the reference (device_hw_info.cuh:236-241); right for HBM too when the
    // runtime reports the data clock and the full bus width.
    out->peak_dram_gbs = (double)out->mem_clock_khz * 1e3 * (out->mem_bus_width_bits / 8.0) * 2.0 / 1e9;
    if (out->peak_dram_gbs > 0) out->ridge_int8_ops_per_byte = out->peak_int8_dense_tops * 1e12 / (out->peak_dram_gbs * 1e9);
    return JQ_OK;
}

}  // extern "C"
