// Quantizers: fp32 activations -> block_q8_1_mmq, fp32 weights -> Q4_0.
//
// The activation quantizer replaces quantize_q8_1_kernel (reference src/cuda/q8_1.cu:20-104).
// It is a pure streaming kernel (reads 4 B, writes 1.125 B per value); one warp owns one
// 128-value block, one lane four consecutive floats, so a warp reads 512 contiguous bytes and
// writes 128 + 16 contiguous bytes.
#include "jq_common.cuh"

namespace jq {

namespace {

constexpr int QUANT_THREADS = 256;
constexpr int QUANT_UNROLL = 4;
struct QuantBounds {  // the buffers of one quantizer launch (range-checked debug build)
    Extent x, xq;
    int *fault = nullptr;
};

constexpr int QUANT_PAIR_UNROLL = 2;  // pairs in flight per warp (4 cost occupancy: 78 registers, 34 % warps active, 3 % slower)

// IDX is the type of the block counter: 32-bit whenever M * K / 128 fits (64-bit division costs more
// instructions than the quantization of a block itself).
template <typename IDX>
__global__ void __launch_bounds__(QUANT_THREADS)
quantize_q8_1_kernel_sm100(const float *__restrict__ x, uint8_t *__restrict__ xq, int64_t K, int64_t M,
                           int64_t n_super_, int order, int s_mode, const QuantBounds bounds) {
    // let the multiply that follows on the stream start its weight stream right away; wait for
    // whatever produced x before reading it
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const IDX n_super = (IDX)n_super_;
    const IDX warp0 = (IDX)(((int64_t)blockIdx.x * QUANT_THREADS + threadIdx.x) >> 5);
    const IDX n_warps = (IDX)(((int64_t)gridDim.x * QUANT_THREADS) >> 5);
    const IDX total = (IDX)(M * n_super_);

    for (IDX base = warp0; base < total; base += n_warps * QUANT_UNROLL) {
        float4 xi[QUANT_UNROLL];
        IDX row[QUANT_UNROLL], ks[QUANT_UNROLL];
#pragma unroll
        for (int u = 0; u < QUANT_UNROLL; ++u) {
            const IDX b = base + (IDX)u * n_warps;
            xi[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            row[u] = ks[u] = 0;
            if (b < total) {
                row[u] = b / n_super;
                ks[u] = b - row[u] * n_super;
                const int64_t k = (int64_t)ks[u] * SUPER + lane * 4;
                const float *src = x + (int64_t)row[u] * K + k;
                if (k < K && JQ_IN_EXTENT(bounds.x, src, sizeof(float4), bounds.fault)) xi[u] = __ldg(reinterpret_cast<const float4 *>(src));
            }
        }
#pragma unroll
        for (int u = 0; u < QUANT_UNROLL; ++u) {
            const IDX b = base + (IDX)u * n_warps;  // uniform across the warp
            if (b >= total) break;
            uint32_t ds;
            const uint32_t q = quantize_group_q8_1(xi[u], s_mode, &ds);
            uint8_t *blk = xq + q8_block_index(ks[u], row[u], n_super_, M, order) * Q8_BYTES;
            if (!JQ_IN_EXTENT(bounds.xq, blk, Q8_BYTES, bounds.fault)) continue;
            reinterpret_cast<uint32_t *>(blk + Q8_QS_OFFSET)[lane] = q;
            if ((lane & 7) == 0) reinterpret_cast<uint32_t *>(blk)[lane >> 3] = ds;
        }
    }
}

// The same kernel for rows that are whole pairs of 128-value blocks (K % 256 == 0): one warp owns two neighbouring
// blocks, one lane eight consecutive floats, so a warp reads 1 KB and writes 2 x 144 bytes, with half the
// instructions per value.  The four-values-per-lane kernel above is bound by instruction issue (about 110 warp
// instructions per 656 bytes moved: 3.5 TB/s is already two instructions per clock and SM), not by bytes in flight.
template <typename IDX>
__global__ void __launch_bounds__(QUANT_THREADS, 5)
quantize_q8_1_pairs_kernel_sm100(const float *__restrict__ x, uint8_t *__restrict__ xq, int64_t K, int64_t M, int64_t n_super_,
                                 int order, int s_mode, const QuantBounds bounds) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const IDX n_pairs_row = (IDX)(n_super_ >> 1);
    const IDX warp0 = (IDX)(((int64_t)blockIdx.x * QUANT_THREADS + threadIdx.x) >> 5);
    const IDX n_warps = (IDX)(((int64_t)gridDim.x * QUANT_THREADS) >> 5);
    const IDX total = (IDX)(M * (n_super_ >> 1));
    constexpr int U = QUANT_PAIR_UNROLL;  // pairs in flight per warp
    for (IDX base = warp0; base < total; base += n_warps * U) {
        float4 xa[U], xb[U];
        IDX row[U], pr[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const IDX p = base + (IDX)u * n_warps;
            xa[u] = xb[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            row[u] = pr[u] = 0;
            if (p < total) {
                row[u] = p / n_pairs_row;
                pr[u] = p - row[u] * n_pairs_row;
                const float4 *src = reinterpret_cast<const float4 *>(x + (int64_t)row[u] * K + (int64_t)pr[u] * (2 * SUPER)) + 2 * lane;
                if (JQ_IN_EXTENT(bounds.x, src, 2 * sizeof(float4), bounds.fault)) {
                    xa[u] = __ldg(src);
                    xb[u] = __ldg(src + 1);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const IDX p = base + (IDX)u * n_warps;  // uniform across the warp
            if (p >= total) break;
            const float v[8] = {xa[u].x, xa[u].y, xa[u].z, xa[u].w, xb[u].x, xb[u].y, xb[u].z, xb[u].w};
            uint2 q;
            uint32_t ds;
            quantize_8_per_lane_q8_1(v, s_mode, &q, &ds);
            const int64_t ks = 2 * (int64_t)pr[u] + (lane >> 4);  // this lane's block of the pair
            uint8_t *blk = xq + q8_block_index(ks, row[u], n_super_, M, order) * Q8_BYTES;
            if (!JQ_IN_EXTENT(bounds.xq, blk, Q8_BYTES, bounds.fault)) continue;
            reinterpret_cast<uint2 *>(blk + Q8_QS_OFFSET)[lane & 15] = q;
            if ((lane & 3) == 0) reinterpret_cast<uint32_t *>(blk)[(lane & 15) >> 2] = ds;
        }
    }
}

// fp32 [N][K] -> Q4_0.  Eight lanes own one 32-weight block.  The block's scale comes from the
// element of largest magnitude, the first one on ties, taken with its sign.
__global__ void __launch_bounds__(256)
quantize_q4_0_kernel_sm100(const float *__restrict__ w, uint8_t *__restrict__ wq, int64_t n_blocks) {
    const int lane = threadIdx.x & 31;
    const int sub = lane & 7;
    const int64_t group0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    const int64_t n_groups = ((int64_t)gridDim.x * blockDim.x) >> 3;
    const int64_t iters = (n_blocks + n_groups - 1) / n_groups;
    for (int64_t it = 0; it < iters; ++it) {
        const int64_t b = group0 + it * n_groups;
        const bool live = b < n_blocks;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) v = __ldg(reinterpret_cast<const float4 *>(w + b * QK) + sub);
        const float e[4] = {v.x, v.y, v.z, v.w};
        float amax = 0.0f, mx = 0.0f;
        int idx = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (amax < fabsf(e[j])) {
                amax = fabsf(e[j]);
                mx = e[j];
                idx = sub * 4 + j;
            }
        }
        if (amax == 0.0f) idx = 32;  // "nothing found yet": loses every tie
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) {
            const float oa = __shfl_xor_sync(0xFFFFFFFFu, amax, off, 32);
            const float om = __shfl_xor_sync(0xFFFFFFFFu, mx, off, 32);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, idx, off, 32);
            if (oa > amax || (oa == amax && oi < idx)) {
                amax = oa;
                mx = om;
                idx = oi;
            }
        }
        const float d = mx / -8.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        uint32_t packed = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // multiply and add round separately (no fused multiply-add), then truncate
            int q = (int)__fadd_rn(__fmul_rn(e[j], id), 8.5f);
            q = q > 15 ? 15 : q;
            packed |= (uint32_t)q << (8 * j);
        }
        const uint32_t hi = __shfl_xor_sync(0xFFFFFFFFu, packed, 4, 32);  // weights j+16 for lanes 0..3
        if (live && sub < 4) {
            const uint32_t bytes = packed | (hi << 4);
            uint8_t *o = wq + b * Q4_BYTES;
            uint16_t *o16 = reinterpret_cast<uint16_t *>(o + 2 + 4 * sub);  // 2-byte aligned only
            o16[0] = (uint16_t)(bytes & 0xFFFFu);
            o16[1] = (uint16_t)(bytes >> 16);
            if (sub == 0) *reinterpret_cast<uint16_t *>(o) = __half_as_ushort(__float2half(d));
        }
    }
}

}  // namespace

int launch_quantize_q8_1(cudaStream_t st, const float *d_x, void *d_xq, int64_t K, int64_t M, int order,
                         int s_mode) {
    const int64_t n_super = (K + SUPER - 1) / SUPER;
    const int64_t total = M * n_super;
    if (total == 0) return JQ_OK;
    DeviceCaps caps;
    if (int rc = device_caps(&caps)) return rc;
    const int warps_per_cta = QUANT_THREADS / 32;
    const bool pairs = K % (2 * SUPER) == 0;
    const int64_t units = pairs ? total / 2 : total;           // warp tasks: block pairs or single blocks
    const int unroll = pairs ? QUANT_PAIR_UNROLL : QUANT_UNROLL;
    int64_t ctas = (units + (int64_t)warps_per_cta * unroll - 1) / ((int64_t)warps_per_cta * unroll);
    const int64_t cap = (int64_t)caps.sm_count * 8 * 4;  // a few waves of resident CTAs
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(QUANT_THREADS);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const bool idx32 = total + (int64_t)ctas * QUANT_THREADS < (int64_t)0x7FFFFFFF;
    QuantBounds bounds;
    bounds.x = make_extent(d_x, (unsigned long long)M * (unsigned long long)K * sizeof(float));
    bounds.xq = make_extent(d_xq, (unsigned long long)total * Q8_BYTES);
    bounds.fault = BOUNDS_CHECK ? device_fault_ptr() : nullptr;
    if (pairs) {
        if (idx32) {
            JQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, quantize_q8_1_pairs_kernel_sm100<uint32_t>, d_x, static_cast<uint8_t *>(d_xq), K, M,
                                           n_super, order, s_mode, bounds));
        } else {
            JQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, quantize_q8_1_pairs_kernel_sm100<int64_t>, d_x, static_cast<uint8_t *>(d_xq), K, M,
                                           n_super, order, s_mode, bounds));
        }
    } else if (idx32) {
        JQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, quantize_q8_1_kernel_sm100<uint32_t>, d_x, static_cast<uint8_t *>(d_xq), K, M,
                                       n_super, order, s_mode, bounds));
    } else {
        JQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, quantize_q8_1_kernel_sm100<int64_t>, d_x, static_cast<uint8_t *>(d_xq), K, M,
                                       n_super, order, s_mode, bounds));
    }
    return JQ_OK;
}

int launch_quantize_q4_0(cudaStream_t st, const float *d_w, void *d_wq, int64_t N, int64_t K) {
    const int64_t n_blocks = N * (K / QK);
    if (n_blocks == 0) return JQ_OK;
    DeviceCaps caps;
    if (int rc = device_caps(&caps)) return rc;
    int64_t ctas = (n_blocks + 31) / 32;  // 32 blocks per 256-thread CTA per pass
    const int64_t cap = (int64_t)caps.sm_count * 32;
    if (ctas > cap) ctas = cap;
    (void)cudaGetLastError();  // a stale error of an earlier, unrelated call must not be taken for this launch's
    quantize_q4_0_kernel_sm100<<<(unsigned)ctas, 256, 0, st>>>(d_w, static_cast<uint8_t *>(d_wq), n_blocks);
    JQ_CUDA_TRY(cudaGetLastError());
    return JQ_OK;
}

}  // namespace jq
