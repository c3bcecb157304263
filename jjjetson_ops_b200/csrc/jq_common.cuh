// Shared definitions of the sm_100a Q4_0 x Q8_1 kernels: block layouts, error plumbing and the
// small PTX wrappers (mbarrier, bulk async copy, int8 mma) the kernels are built from.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/jq_b200.h"

namespace jq {

constexpr int QK = 32;          // values per Q4_0 block and per Q8_1 group
constexpr int Q4_BYTES = 18;    // block_q4_0: fp16 d + 16 nibble bytes
constexpr int SUPER = 128;      // values per block_q8_1_mmq
constexpr int Q8_BYTES = 144;   // 4 x half2 (d, s) + 128 int8
constexpr int Q8_QS_OFFSET = 16;

// Mirror of the reference's activation block (src/cuda/q8_1.cu:14-18).
struct __align__(16) BlockQ8_1Mmq {
    half2 ds4[4];
    int8_t qs[SUPER];
};
static_assert(sizeof(BlockQ8_1Mmq) == Q8_BYTES, "block_q8_1_mmq must be 144 bytes");

// ---- host-side error plumbing ------------------------------------------------------------
int set_error(int status, const char *fmt, ...);  // records the message, returns `status`
int cuda_error(cudaError_t e, const char *what);  // JQ_ERR_CUDA with the runtime's message

#define JQ_CUDA_TRY(expr)                                         \
    do {                                                          \
        cudaError_t jq_e_ = (expr);                               \
        if (jq_e_ != cudaSuccess) return ::jq::cuda_error(jq_e_, #expr); \
    } while (0)

// Per-device facts the launchers need; queried once per device.
struct DeviceCaps {
    int sm_count = 0;
    int smem_optin = 0;  // max dynamic shared memory per block (opt-in)
    int smem_per_sm = 0; // shared memory per multiprocessor
    int cc = 0;          // major*10 + minor
};
int device_caps(DeviceCaps *out);  // for the current device

// Raises a kernel's dynamic shared-memory limit to at least `bytes` on the current device.  The attribute
// belongs to the function and the device, not to a host thread, so the record of what has been set is
// process-wide (mutex-protected) and a limit is only ever raised.  `max_carveout` also asks for the largest
// shared-memory carve-out (kernels that want two CTAs of ~110 KB per SM).
int ensure_dynamic_smem(const void *kernel, int bytes, bool max_carveout = false);

int option_value(int option);       // process-wide settings of jq_set_option()
// Polls after which a bounded device-side wait gives up (JQ_OPT_WAIT_POLL_LIMIT; 2^22 by default).
uint32_t wait_poll_limit();
// Tracing aid (jq_trace_enable): device address where the next traced launch may write its
// per-CTA timestamps, or nullptr when tracing is off or the buffer is full.
void *next_trace_slot();

// Device address (on the current device) of the word a kernel sets when one of its bounded waits
// gives up; nullptr if it cannot be obtained.  Kernels receive it as a parameter.  The word keeps the highest
// code reported: 1 a wait for a copy, 2 a wait for another rank's data, 3 a range check of the debug build.
int *device_fault_ptr();

// ---- range-checked debug build (-DJQ_BOUNDS_CHECK) ----------------------------------------------
// Stands in for a memory checker: every global access of the kernels is checked against the extent of the
// buffer it belongs to (what the entry point was told through its shape arguments, not what was allocated),
// every shared-memory offset against the kernel's dynamic shared memory; an access that falls outside is
// skipped and the fault word is set to 3.  Without the flag the checks are not there (JQ_IN_EXTENT / JQ_IN_SHARED
// expand to `true`) and the larger kernel-parameter structures do not carry the extents.
struct Extent {
    const void *base = nullptr;
    unsigned long long bytes = 0;
};
// Extent of `bytes` at `base`, less the debug shrink (jq_debug_set_extent_shrink: lets a test see the checks
// fire on accesses that are in fact in range).
Extent make_extent(const void *base, unsigned long long bytes);
// The buffers of one multiply, for the kernels that take plain pointers.
struct MulMatBounds {
    Extent w, xq, y;
    int *fault = nullptr;
};
MulMatBounds mul_mat_bounds(const void *d_w, const void *d_xq, const void *d_y, int64_t K, int64_t N, int64_t M, size_t y_elem_bytes);
#ifdef JQ_BOUNDS_CHECK
constexpr bool BOUNDS_CHECK = true;
#else
constexpr bool BOUNDS_CHECK = false;
#endif

// ---- launchers implemented in the .cu files ----------------------------------------------
int launch_quantize_q8_1(cudaStream_t st, const float *d_x, void *d_xq, int64_t K, int64_t M,
                         int order, int s_mode);
int launch_quantize_q4_0(cudaStream_t st, const float *d_w, void *d_wq, int64_t N, int64_t K);
// producers.cu: RMSNorm (optionally with the residual add) and SwiGLU with the Q8_1 quantizer folded in
int launch_rms_norm_q8_1(cudaStream_t st, float *d_input, float *d_residual, const float *d_weight, float *d_normed,
                         void *d_xq, int64_t H, int64_t T, float epsilon, int order, int s_mode);
int launch_swiglu_q8_1(cudaStream_t st, const float *d_gate, const float *d_up, float *d_mid, void *d_xq, int64_t I,
                       int64_t T, int order, int s_mode);
int launch_mmq_generic(cudaStream_t st, const void *d_w, const void *d_xq, float *d_y, int64_t K,
                       int64_t N, int64_t M, int order);
int launch_block_sums(cudaStream_t st, const void *d_w, const void *d_xq, int32_t *d_sums, int64_t K,
                      int64_t N, int64_t M, int order);
// Optional epilogue of the dp4a GEMV for N-sharded layers: every rank stores its band of the output
// straight into all ranks' [M][N_total] buffers (peer-mapped memory, plain stores over NVLink) and
// the kernel ends only when every rank's band has arrived everywhere.
constexpr int MAX_PEERS = 8;
struct GatherArgs {
    float *y_peer[MAX_PEERS];        // base of each rank's output buffer, as mapped on this device
    uint32_t *flag_peer[MAX_PEERS];  // base of each rank's arrival flags (uint32[world])
    int world = 0, rank = 0;
    int64_t n_offset = 0, N_total = 0;
    uint32_t *epoch_ptr = nullptr;   // local device counter of finished all-gathers (zero before the first call).
                                     // This call is number *epoch_ptr + 1: it stores into buffer (number & 1),
                                     // raises the peers' flags to its number and then increments the counter.
    uint64_t y_stride_bytes = 0;     // distance between the two output buffers of a rank
    int wait_previous = 0;           // wait until all flags here have reached *epoch_ptr before reading x
    int *counter = nullptr;          // local int, zero before the first call (the kernel re-zeroes it)
    // Tagged-word form (M <= 2): an output value travels as one 8-byte word {fp32 bits, number of its all-gather},
    // the consumer polls the words it needs and no flag, release or acknowledgement is on the path.  y_peer then
    // holds each rank's pair of [M][N_total] word buffers; flag_peer, epoch_ptr, counter, wait_previous are unused.
    unsigned long long *ticket = nullptr;         // local 64-bit count, zero before the first call; non-null selects this
                                                  // form.  Every launch adds 65536 (in shares, one per CTA): the launch
                                                  // that finds t is all-gather number (t >> 16) + 1.
    const unsigned long long *x_words = nullptr;  // this rank's pair of word buffers whose all-gather number
                                                  // (t >> 16) - x_back is this launch's input, or nullptr: plain fp32
    int x_back = 0;                               // 0: the all-gather launched just before this one, 1: the one before that
    uint64_t x_stride_bytes = 0;                  // distance between the two buffers of that pair
    int64_t x_row_words = 0;                      // words per row there (that all-gather's N_total)
    int x_seg_len = 0;                            // activation k of a row is word (k / x_seg_len) * x_seg_stride +
    int64_t x_seg_stride = 0;                     // k % x_seg_len of that row (x_seg_len a multiple of 8)
    int x_wide = 0;                               // every lane's eight words start on a 32-byte boundary: 256-bit loads
};

// Waits (bounded) on the stream until all `world` flags have reached *d_epoch.
int launch_allgather_wait(cudaStream_t st, const uint32_t *d_flags, int world, const uint32_t *d_epoch);
// Tagged-word form: waits (bounded) for every word of the all-gather numbered *d_ticket >> 16 in this rank's pair
// of word buffers and writes the values as plain fp32 [M][N_total].
int launch_allgather_tagged_read(cudaStream_t st, const unsigned long long *d_words, uint64_t stride_bytes, int64_t M,
                                 int64_t N_total, const unsigned long long *d_ticket, float *d_out);

// Streaming GEMV family.  d_x_f32 != nullptr fuses the activation quantizer into the prologue
// (d_xq then receives the quantized blocks in JQ_ORDER_COL_KSUPER order, may be nullptr).
// Returns JQ_ERR_UNSUPPORTED when the shape or alignment rules of the fast path do not hold.
// With `multi`, several weight matrices that share K and the activations are multiplied in one launch
// (d_w, d_y are ignored and N is the sum of their rows).
struct MultiMat {
    int n;                 // 2..4
    const void *w[4];
    float *y[4];           // [M][rows[i]] each
    int64_t rows[4];
};
int launch_gemv_dp4a(cudaStream_t st, const void *d_w, const void *d_xq, const float *d_x_f32,
                     void *d_xq_out, float *d_y, int64_t K, int64_t N, int64_t M, int order,
                     int s_mode, const GatherArgs *gather = nullptr, const MultiMat *multi = nullptr);
int launch_gemv_mma(cudaStream_t st, const void *d_w, const void *d_xq, const float *d_x_f32,
                    void *d_xq_out, float *d_y, int64_t K, int64_t N, int64_t M, int order,
                    int s_mode, const MultiMat *multi = nullptr);
int launch_gemm_mma(cudaStream_t st, const void *d_w, const void *d_xq, float *d_y, int64_t K,
                    int64_t N, int64_t M, int order, const GatherArgs *gather = nullptr);
int launch_gemm_tc(cudaStream_t st, const void *d_w, const void *d_xq, float *d_y, int64_t K,
                   int64_t N, int64_t M, int order);
int launch_gemm_f16(cudaStream_t st, const void *d_w, const void *d_xq, float *d_y, int64_t K,
                    int64_t N, int64_t M, int order);
// Zeroes the per-tile counts of the fp16-operand GEMM's split-K epilogue (a kernel that gave up may have left them
// half-way); called when the fault word is cleared.
int reset_gemm_f16_split_state();

// ---- device helpers --------------------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ int64_t q8_block_index(int64_t ksuper, int64_t m, int64_t n_super, int64_t M,
                                                  int order) {
    return order == JQ_ORDER_KSUPER_COL ? ksuper * M + m : m * n_super + ksuper;
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h16) {
    return __half2float(__ushort_as_half((unsigned short)h16));
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// Shared-memory loads by 32-bit shared address: keeps address arithmetic in 32 bits and the load in
// the shared state space whatever the compiler can prove about the pointer.
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return (uint32_t)v;
}
__device__ __forceinline__ uint2 lds_v2(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// ---- mbarrier -------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// The fault word keeps the highest code reported (see device_fault_ptr()).
__device__ __forceinline__ void report_fault(int *fault, int code) {
#ifdef JQ_BOUNDS_CHECK
    if (fault != nullptr) atomicMax(fault, code);
#else
    if (fault != nullptr) atomicExch(fault, code);
#endif
}

// Range checks of the debug build: true when [p, p + n) lies inside the extent (always, in a normal build).
__device__ __forceinline__ bool in_extent(const Extent &e, const void *p, unsigned long long n, int *fault) {
    if (!BOUNDS_CHECK) return true;
    const unsigned long long a = (unsigned long long)p, b = (unsigned long long)e.base;
    const bool ok = a >= b && n <= e.bytes && a - b <= e.bytes - n;
    if (!ok) report_fault(fault, 3);
    return ok;
}
// ... and when [offset, offset + n) lies inside `total` bytes of shared memory.
__device__ __forceinline__ bool in_shared(unsigned long long offset, unsigned long long n, unsigned long long total, int *fault) {
    if (!BOUNDS_CHECK) return true;
    const bool ok = n <= total && offset <= total - n;
    if (!ok) report_fault(fault, 3);
    return ok;
}

// What the kernels write: in a normal build the conditions are the literal `true` and their arguments are not even
// evaluated, so the code is what it would be without the checks.
#ifdef JQ_BOUNDS_CHECK
#define JQ_IN_EXTENT(e, p, n, fault) ::jq::in_extent(e, p, n, fault)
#define JQ_IN_SHARED(offset, n, total, fault) ::jq::in_shared(offset, n, total, fault)
#else
#define JQ_IN_EXTENT(e, p, n, fault) true
#define JQ_IN_SHARED(offset, n, total, fault) true
#endif

// Bounded wait: gives up after `limit` polls, records the fault and reports false so that the
// caller can leave the kernel instead of hanging the GPU.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, int *fault,
                                                  uint32_t limit = (1u << 22)) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    report_fault(fault, 1);
    return false;
}

// 1-D bulk async copy global -> shared, completion counted in bytes on an mbarrier.
// Source, destination and size must all be multiples of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void *smem_dst, const void *gmem_src, uint32_t bytes,
                                         uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(smem_dst)),
        "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Named barrier over a subset of the CTA's warps.
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// D(16x8, s32) = A(16x32, u8 row) * B(32x8, s8 col) + C
__device__ __forceinline__ void mma_u8s8_16832(int (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2],
                                               const int (&c)[4]) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "r"(c[0]), "r"(c[1]),
          "r"(c[2]), "r"(c[3]));
}

// One 32-value group of the activation quantizer, as 8 lanes x 4 floats, following
// quantize_q8_1_kernel (src/cuda/q8_1.cu:55-79,101-103) operation by operation so that the int8
// values, fp16 d and fp16 sum come out bit-identical: max and sum by xor butterflies with
// offsets 4, 2, 1, d_inv = 127/amax by IEEE division, q = roundf(x * d_inv), d = 1/d_inv.
// Every lane of the warp must call it.  Returns the packed char4; ds holds (d, s) as fp16 bits.
__device__ __forceinline__ uint32_t quantize_group_q8_1(float4 xi, int s_mode, uint32_t *ds_bits) {
    float amax = fmaxf(fabsf(xi.x), fmaxf(fabsf(xi.y), fmaxf(fabsf(xi.z), fabsf(xi.w))));
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off, 32));
    }
    float sum = xi.x + xi.y + xi.z + xi.w;
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) {
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off, 32);
    }
    const float d_inv = amax > 0.0f ? 127.0f / amax : 0.0f;
    const int q0 = (int)roundf(xi.x * d_inv);
    const int q1 = (int)roundf(xi.y * d_inv);
    const int q2 = (int)roundf(xi.z * d_inv);
    const int q3 = (int)roundf(xi.w * d_inv);
    const __half dh = amax > 0.0f ? __float2half(1.0f / d_inv) : __ushort_as_half((unsigned short)0);
    __half sh;
    if (s_mode == JQ_S_SUM_X) {
        sh = __float2half(sum);
    } else {
        int isum = q0 + q1 + q2 + q3;
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) {
            isum += __shfl_xor_sync(0xFFFFFFFFu, isum, off, 32);
        }
        sh = __float2half(__half2float(dh) * (float)isum);
    }
    *ds_bits = (uint32_t)__half_as_ushort(dh) | ((uint32_t)__half_as_ushort(sh) << 16);
    return (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) |
           ((uint32_t)(q3 & 0xFF) << 24);
}

// The same quantizer with eight values per lane: lane l of a warp owns the values 8l .. 8l+7 of 256 consecutive
// ones (two neighbouring 128-value blocks), a 32-value group is four lanes.  Same results, bit for bit, as
// quantize_group_q8_1: the maximum and the integer sum do not depend on the order, and the sum of the floats is
// formed in the reference's order - per four consecutive values left to right, then the partners that the
// reference's xor-4, xor-2 and xor-1 steps pair up (q8_1.cu:62-68).  Half the instructions per value of the
// four-per-lane form (two shuffle rounds instead of three, scalar work shared by eight values).
// Every lane of the warp must call it.  q_out: the lane's eight int8 values; ds: (d, s) of its group.
__device__ __forceinline__ void quantize_8_per_lane_q8_1(const float (&v)[8], int s_mode, uint2 *q_out, uint32_t *ds_bits) {
    float amax = fmaxf(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))),
                       fmaxf(fmaxf(fabsf(v[4]), fabsf(v[5])), fmaxf(fabsf(v[6]), fabsf(v[7]))));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1, 32));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2, 32));
    const float d_inv = amax > 0.0f ? 127.0f / amax : 0.0f;
    int q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = (int)roundf(v[i] * d_inv);
    const __half dh = amax > 0.0f ? __float2half(1.0f / d_inv) : __ushort_as_half((unsigned short)0);
    __half sh;
    if (s_mode == JQ_S_SUM_X) {
        float sa = v[0] + v[1] + v[2] + v[3], sb = v[4] + v[5] + v[6] + v[7];
        sa += __shfl_xor_sync(0xFFFFFFFFu, sa, 2, 32);  // the reference's lanes i and i ^ 4
        sb += __shfl_xor_sync(0xFFFFFFFFu, sb, 2, 32);
        sa += __shfl_xor_sync(0xFFFFFFFFu, sa, 1, 32);  // i and i ^ 2
        sb += __shfl_xor_sync(0xFFFFFFFFu, sb, 1, 32);
        sh = __float2half(sa + sb);                      // i and i ^ 1
    } else {
        int isum = ((q[0] + q[1]) + (q[2] + q[3])) + ((q[4] + q[5]) + (q[6] + q[7]));
        isum += __shfl_xor_sync(0xFFFFFFFFu, isum, 1, 32);
        isum += __shfl_xor_sync(0xFFFFFFFFu, isum, 2, 32);
        sh = __float2half(__half2float(dh) * (float)isum);
    }
    *ds_bits = (uint32_t)__half_as_ushort(dh) | ((uint32_t)__half_as_ushort(sh) << 16);
    q_out->x = (uint32_t)(q[0] & 0xFF) | ((uint32_t)(q[1] & 0xFF) << 8) | ((uint32_t)(q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
    q_out->y = (uint32_t)(q[4] & 0xFF) | ((uint32_t)(q[5] & 0xFF) << 8) | ((uint32_t)(q[6] & 0xFF) << 16) | ((uint32_t)(q[7] & 0xFF) << 24);
}

#endif  // __CUDACC__

}  // namespace jq
