// Producers of the quantized linear's input: the two kernels that run just ahead of it in the
// reference's transformer layer, with the Q8_1 quantizer folded in, so that the fp32 activation
// never makes the round trip through HBM and the separate quantize launch disappears.
//
//   rms_norm_q8_1_kernel   replaces rms_norm_fused_add_kernel (reference
//                          src/cuda/rms_norm_fused_add.cu:10-44, feeds the Q/K/V and gate/up
//                          linears, src/engine/transformer_runner.cpp:208-216, 311-321) and
//                          rms_norm_kernel (src/cuda/rms_norm.cu:12-41, feeds lm_head).
//   swiglu_q8_1_kernel     replaces swiglu_silu_mul_kernel (src/cuda/swiglu.cu:5-15, feeds the
//                          down linear, transformer_runner.cpp:324-328).
//
// Both compute the fp32 values with the reference's own operation order, so the fp32 outputs and
// therefore the quantized blocks are bit-identical to "reference kernel, then quantize_q8_1".
#include "jq_common.cuh"

namespace jq {

namespace {

constexpr int RMS_THREADS = 256;  // the reference's block size; the summation order depends on it

// Block sum with the reference's tree (include/cuda_utils.cuh:19-27, 49-65): shuffle-down inside
// each warp, one partial per warp through shared memory, shuffle-down over the partials in warp 0.
// Only thread 0 holds the result.
__device__ __forceinline__ float shuffle_down_sum(float v) {
    v += __shfl_down_sync(0xFFFFFFFFu, v, 16);
    v += __shfl_down_sync(0xFFFFFFFFu, v, 8);
    v += __shfl_down_sync(0xFFFFFFFFu, v, 4);
    v += __shfl_down_sync(0xFFFFFFFFu, v, 2);
    v += __shfl_down_sync(0xFFFFFFFFu, v, 1);
    return v;
}

__device__ __forceinline__ float block_sum_reference_order(float v, float *warp_partial) {
    v = shuffle_down_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) warp_partial[warp] = v;
    __syncthreads();
    v = (threadIdx.x < ((blockDim.x + 31) >> 5)) ? warp_partial[lane] : 0.f;
    if (warp == 0) v = shuffle_down_sum(v);
    return v;
}

// One CTA per token.  Thread t owns elements t, t + blockDim, ... exactly as in the reference, so
// the per-thread partial sums of squares, the block tree and rsqrtf give the same inverse RMS bit
// for bit.  The normalised row is staged in shared memory and quantized from there warp by warp
// (one warp per 128-value block, one lane four consecutive values: the quantizer's own mapping).
__global__ void __launch_bounds__(RMS_THREADS, 5)
rms_norm_q8_1_kernel(float *input, float *residual, const float *__restrict__ weight, float *normed_out,
                     uint8_t *__restrict__ xq, int H, int T, float epsilon, int n_super, int order, int s_mode) {
    // input, residual and normed_out carry no __restrict__: normed_out may be input itself (the reference's
    // in-place form); every read of a row happens before the barrier that precedes the first write to it
    extern __shared__ __align__(16) float row[];  // H floats
    __shared__ float warp_partial[32];
    __shared__ float inverse_rms;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int token = blockIdx.x;
    const int64_t base = (int64_t)token * H;

    // z = input (+ residual) into shared memory; the additions are elementwise, so 16-byte accesses
    // are free to use any thread-to-element mapping
    const bool vec = (H & 3) == 0 && ((uintptr_t)(input + base) & 15u) == 0 &&
                     (residual == nullptr || ((uintptr_t)(residual + base) & 15u) == 0);
    if (vec) {
        const float4 *in4 = reinterpret_cast<const float4 *>(input + base);
        float4 *res4 = reinterpret_cast<float4 *>(residual != nullptr ? residual + base : nullptr);
        float4 *row4 = reinterpret_cast<float4 *>(row);
        // four 16-byte loads of each operand in flight per thread before anything is stored (the buffers may alias
        // one another, so the compiler cannot hoist loads over stores by itself): a CTA spends half its life in the
        // reduction and quantization phases, and what is in flight during its load phase has to cover for that
        const int n4 = H >> 2, stride = blockDim.x;
        for (int i0 = threadIdx.x; i0 < n4; i0 += 4 * stride) {
            float4 z[4], r[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * stride;
                z[u] = i < n4 ? in4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            if (res4 != nullptr) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = i0 + u * stride;
                    r[u] = i < n4 ? res4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * stride;
                if (i < n4) {
                    if (res4 != nullptr) {
                        z[u] = make_float4(z[u].x + r[u].x, z[u].y + r[u].y, z[u].z + r[u].z, z[u].w + r[u].w);
                        res4[i] = z[u];
                    }
                    row4[i] = z[u];
                }
            }
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float z = input[base + i];
            if (residual != nullptr) {
                z = z + residual[base + i];
                residual[base + i] = z;
            }
            row[i] = z;
        }
    }
    __syncthreads();
    // sum of squares in the reference's order: thread t takes elements t, t + blockDim, ...
    float sum_square = 0.f;
    {
        int i = threadIdx.x;
        const int stride = blockDim.x;
        for (; i + 3 * stride < H; i += 4 * stride) {  // same elements in the same order, four loads in flight
            const float z0 = row[i], z1 = row[i + stride], z2 = row[i + 2 * stride], z3 = row[i + 3 * stride];
            sum_square = __fmaf_rn(z0, z0, sum_square);
            sum_square = __fmaf_rn(z1, z1, sum_square);
            sum_square = __fmaf_rn(z2, z2, sum_square);
            sum_square = __fmaf_rn(z3, z3, sum_square);
        }
        for (; i < H; i += stride) {
            const float z = row[i];
            sum_square = __fmaf_rn(z, z, sum_square);
        }
    }
    sum_square = block_sum_reference_order(sum_square, warp_partial);
    if (threadIdx.x == 0) inverse_rms = rsqrtf(sum_square / (float)H + epsilon);
    __syncthreads();
    const float inv = inverse_rms;
    const bool vec_out = vec && ((uintptr_t)weight & 15u) == 0 && (normed_out == nullptr || ((uintptr_t)(normed_out + base) & 15u) == 0);
    if (vec_out && xq != nullptr && (n_super & 1) == 0) {
        // Normalisation and quantization in one pass over the row: a warp takes a pair of neighbouring blocks, a lane
        // its eight consecutive values, (z * inv) * w goes to the fp32 output (if wanted) and into the quantizer
        // straight from registers.  Same products, same bits as normalising the row first; it saves the row's second
        // trip through shared memory, one block-wide barrier and a quarter of the kernel's instructions.
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
        for (int pr = warp; pr < (n_super >> 1); pr += n_warps) {
            const int e0 = pr * (2 * SUPER) + lane * 8;
            const float4 z0 = *reinterpret_cast<const float4 *>(row + e0), z1 = *reinterpret_cast<const float4 *>(row + e0 + 4);
            const float4 w0 = __ldg(reinterpret_cast<const float4 *>(weight + e0)), w1 = __ldg(reinterpret_cast<const float4 *>(weight + e0 + 4));
            const float v[8] = {__fmul_rn(__fmul_rn(z0.x, inv), w0.x), __fmul_rn(__fmul_rn(z0.y, inv), w0.y),
                                __fmul_rn(__fmul_rn(z0.z, inv), w0.z), __fmul_rn(__fmul_rn(z0.w, inv), w0.w),
                                __fmul_rn(__fmul_rn(z1.x, inv), w1.x), __fmul_rn(__fmul_rn(z1.y, inv), w1.y),
                                __fmul_rn(__fmul_rn(z1.z, inv), w1.z), __fmul_rn(__fmul_rn(z1.w, inv), w1.w)};
            if (normed_out != nullptr) {
                *reinterpret_cast<float4 *>(normed_out + base + e0) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4 *>(normed_out + base + e0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
            }
            uint2 q;
            uint32_t ds;
            quantize_8_per_lane_q8_1(v, s_mode, &q, &ds);
            uint8_t *blk = xq + q8_block_index(2 * pr + (lane >> 4), token, n_super, T, order) * Q8_BYTES;
            reinterpret_cast<uint2 *>(blk + Q8_QS_OFFSET)[lane & 15] = q;
            if ((lane & 3) == 0) reinterpret_cast<uint32_t *>(blk)[(lane & 15) >> 2] = ds;
        }
        return;
    }
    if (vec_out) {
        float4 *row4 = reinterpret_cast<float4 *>(row);
        const float4 *w4 = reinterpret_cast<const float4 *>(weight);
        float4 *out4 = reinterpret_cast<float4 *>(normed_out != nullptr ? normed_out + base : nullptr);
        for (int i = threadIdx.x; i < (H >> 2); i += blockDim.x) {
            const float4 z = row4[i], w = __ldg(w4 + i);
            const float4 y = make_float4(__fmul_rn(__fmul_rn(z.x, inv), w.x), __fmul_rn(__fmul_rn(z.y, inv), w.y),
                                         __fmul_rn(__fmul_rn(z.z, inv), w.z), __fmul_rn(__fmul_rn(z.w, inv), w.w));
            row4[i] = y;
            if (out4 != nullptr) out4[i] = y;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float y = __fmul_rn(__fmul_rn(row[i], inv), weight[i]);
            row[i] = y;
            if (normed_out != nullptr) normed_out[base + i] = y;
        }
    }
    if (xq == nullptr) return;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    if ((n_super & 1) == 0) {
        // whole pairs of blocks: a warp takes two neighbouring blocks, a lane eight consecutive values (half the
        // instructions per value of the four-per-lane form, same bits)
        for (int pr = warp; pr < (n_super >> 1); pr += n_warps) {
            const float4 a = *reinterpret_cast<const float4 *>(row + pr * (2 * SUPER) + lane * 8);
            const float4 b = *reinterpret_cast<const float4 *>(row + pr * (2 * SUPER) + lane * 8 + 4);
            const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            uint2 q;
            uint32_t ds;
            quantize_8_per_lane_q8_1(v, s_mode, &q, &ds);
            uint8_t *blk = xq + q8_block_index(2 * pr + (lane >> 4), token, n_super, T, order) * Q8_BYTES;
            reinterpret_cast<uint2 *>(blk + Q8_QS_OFFSET)[lane & 15] = q;
            if ((lane & 3) == 0) reinterpret_cast<uint32_t *>(blk)[(lane & 15) >> 2] = ds;
        }
        return;
    }
    for (int ks = warp; ks < n_super; ks += n_warps) {
        const float4 v = *reinterpret_cast<const float4 *>(row + ks * SUPER + lane * 4);
        uint32_t ds;
        const uint32_t q = quantize_group_q8_1(v, s_mode, &ds);
        uint8_t *blk = xq + q8_block_index(ks, token, n_super, T, order) * Q8_BYTES;
        reinterpret_cast<uint32_t *>(blk + Q8_QS_OFFSET)[lane] = q;
        if ((lane & 7) == 0) reinterpret_cast<uint32_t *>(blk)[lane >> 3] = ds;
    }
}

// silu(gate) * up with the reference's expression (swiglu.cu:5-7,13), one warp per 128-value block.
__device__ __forceinline__ float silu_mul(float g, float u) {
    return __fmul_rn(__fmul_rn(g, 1.0f / (1.0f + expf(-g))), u);
}

// IDX: 32-bit block counter whenever T * I / 128 fits (a 64-bit division per block would cost more than
// the block's arithmetic).
template <typename IDX>
__global__ void __launch_bounds__(256)
swiglu_q8_1_kernel(const float *gate, const float *up, float *mid, uint8_t *__restrict__ xq, int64_t I, int64_t T,
                   int64_t n_super_, int order, int s_mode) {
    // gate, up and mid may be the same buffer (in-place use): plain loads, each thread reads its own four
    // values before it writes them
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const IDX n_super = (IDX)n_super_;
    const IDX warp0 = (IDX)(((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    const IDX n_warps = (IDX)(((int64_t)gridDim.x * blockDim.x) >> 5);
    const IDX total = (IDX)(T * n_super_);
    if ((n_super_ & 1) == 0) {
        // whole pairs of blocks per row: a warp takes two neighbouring blocks, a lane eight consecutive values
        const IDX pairs_row = n_super >> 1, pairs = total >> 1;
        for (IDX p = warp0; p < pairs; p += n_warps) {
            const IDX t = p / pairs_row, pr = p - t * pairs_row;
            const int64_t off = (int64_t)t * I + (int64_t)pr * (2 * SUPER) + lane * 8;
            const float4 g0 = *reinterpret_cast<const float4 *>(gate + off), g1 = *reinterpret_cast<const float4 *>(gate + off + 4);
            const float4 u0 = *reinterpret_cast<const float4 *>(up + off), u1 = *reinterpret_cast<const float4 *>(up + off + 4);
            const float v[8] = {silu_mul(g0.x, u0.x), silu_mul(g0.y, u0.y), silu_mul(g0.z, u0.z), silu_mul(g0.w, u0.w),
                                silu_mul(g1.x, u1.x), silu_mul(g1.y, u1.y), silu_mul(g1.z, u1.z), silu_mul(g1.w, u1.w)};
            if (mid != nullptr) {
                *reinterpret_cast<float4 *>(mid + off) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4 *>(mid + off + 4) = make_float4(v[4], v[5], v[6], v[7]);
            }
            if (xq != nullptr) {
                uint2 q;
                uint32_t ds;
                quantize_8_per_lane_q8_1(v, s_mode, &q, &ds);
                uint8_t *blk = xq + q8_block_index(2 * (int64_t)pr + (lane >> 4), t, n_super_, T, order) * Q8_BYTES;
                reinterpret_cast<uint2 *>(blk + Q8_QS_OFFSET)[lane & 15] = q;
                if ((lane & 3) == 0) reinterpret_cast<uint32_t *>(blk)[(lane & 15) >> 2] = ds;
            }
        }
        return;
    }
    for (IDX b = warp0; b < total; b += n_warps) {
        const IDX t = b / n_super, ks = b - t * n_super;
        const int64_t off = (int64_t)t * I + (int64_t)ks * SUPER + lane * 4;
        const float4 g = *reinterpret_cast<const float4 *>(gate + off);
        const float4 u = *reinterpret_cast<const float4 *>(up + off);
        const float4 v = make_float4(silu_mul(g.x, u.x), silu_mul(g.y, u.y), silu_mul(g.z, u.z), silu_mul(g.w, u.w));
        if (mid != nullptr) *reinterpret_cast<float4 *>(mid + off) = v;
        if (xq != nullptr) {
            uint32_t ds;
            const uint32_t q = quantize_group_q8_1(v, s_mode, &ds);
            uint8_t *blk = xq + q8_block_index(ks, t, n_super_, T, order) * Q8_BYTES;
            reinterpret_cast<uint32_t *>(blk + Q8_QS_OFFSET)[lane] = q;
            if ((lane & 7) == 0) reinterpret_cast<uint32_t *>(blk)[lane >> 3] = ds;
        }
    }
}

// plain elementwise form for sizes that are not a multiple of 128 (no quantized output possible)
__global__ void swiglu_plain_kernel(const float *gate, const float *up, float *mid, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) mid[i] = silu_mul(gate[i], up[i]);
}

int launch_with_pdl(cudaLaunchConfig_t &cfg, cudaLaunchAttribute *attr) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return 0;
}

}  // namespace

int launch_rms_norm_q8_1(cudaStream_t st, float *d_input, float *d_residual, const float *d_weight, float *d_normed,
                         void *d_xq, int64_t H, int64_t T, float epsilon, int order, int s_mode) {
    if (H <= 0 || T <= 0) return set_error(JQ_ERR_INVALID_ARG, "rms_norm: invalid hidden_size=%lld num_tokens=%lld", (long long)H, (long long)T);
    if (d_xq != nullptr && H % SUPER != 0)
        return set_error(JQ_ERR_UNSUPPORTED, "rms_norm with Q8_1 output needs hidden_size %% 128 == 0 (got %lld)", (long long)H);
    if (H > (1 << 24) || T > 0x7FFFFFFF) return set_error(JQ_ERR_TOO_LARGE, "rms_norm: shape too large");
    DeviceCaps caps;
    if (int rc = device_caps(&caps)) return rc;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem + 1024 > (size_t)caps.smem_optin)
        return set_error(JQ_ERR_TOO_LARGE, "rms_norm: a row of %lld floats does not fit in shared memory", (long long)H);
    if (smem > 48 * 1024) {
        if (int rc = ensure_dynamic_smem(reinterpret_cast<const void *>(rms_norm_q8_1_kernel), (int)smem)) return rc;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)T);
    cfg.blockDim = dim3((unsigned)(H < RMS_THREADS ? H : RMS_THREADS));  // the reference's rule
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    launch_with_pdl(cfg, attr);
    const int n_super = (int)(H / SUPER);
    JQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, rms_norm_q8_1_kernel, d_input, d_residual, d_weight, d_normed,
                                   static_cast<uint8_t *>(d_xq), (int)H, (int)T, epsilon, n_super, order, s_mode));
    return JQ_OK;
}

int launch_swiglu_q8_1(cudaStream_t st, const float *d_gate, const float *d_up, float *d_mid, void *d_xq, int64_t I,
                       int64_t T, int order, int s_mode) {
    if (I <= 0 || T <= 0) return JQ_OK;
    const bool aligned = I % SUPER == 0 && ((uintptr_t)d_gate & 15u) == 0 && ((uintptr_t)d_up & 15u) == 0 &&
                         (d_mid == nullptr || ((uintptr_t)d_mid & 15u) == 0);
    if (!aligned) {
        if (d_xq != nullptr)
            return set_error(JQ_ERR_UNSUPPORTED, "swiglu with Q8_1 output needs intermediate_size %% 128 == 0 and 16-byte aligned buffers");
        if (d_mid == nullptr) return JQ_OK;
        const int64_t n = I * T;
        (void)cudaGetLastError();  // a stale error of an earlier, unrelated call must not be taken for this launch's
        swiglu_plain_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(d_gate, d_up, d_mid, n);
        JQ_CUDA_TRY(cudaGetLastError());
        return JQ_OK;
    }
    DeviceCaps caps;
    if (int rc = device_caps(&caps)) return rc;
    const int64_t n_super = I / SUPER, total = T * n_super;
    int64_t ctas = (total + 7) / 8;  // 8 warps, one block per warp and pass
    if (ctas < 1) ctas = 1;
    const int64_t cap = (int64_t)caps.sm_count * 8 * 4;
    if (ctas > cap) ctas = cap;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    launch_with_pdl(cfg, attr);
    if (total + ctas * 256 < (int64_t)0x7FFFFFFF) {
        JQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, swiglu_q8_1_kernel<uint32_t>, d_gate, d_up, d_mid, static_cast<uint8_t *>(d_xq), I, T,
                                       n_super, order, s_mode));
    } else {
        JQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, swiglu_q8_1_kernel<int64_t>, d_gate, d_up, d_mid, static_cast<uint8_t *>(d_xq), I, T,
                                       n_super, order, s_mode));
    }
    return JQ_OK;
}

}  // namespace jq
