// The any-shape Q4_0 x Q8_1 multiply and the int32 block-sum dump.
//
// This kernel is the safety net behind the streaming GEMV and the tensor-core GEMM: it takes
// any N, any M and any K % 128 == 0 with no alignment demand beyond the 2 bytes the Q4_0 block
// itself guarantees.  Per block it computes exactly what q4_0_q8_1_vec_dot_impl does
// (reference src/cuda/mm_q4_0_q8_1.cu:71-93): sumi by dp4a over unsigned nibbles, then
// d4 * (sumi * d8 - 8 * s8), accumulated in fp32.
#include "jq_common.cuh"

namespace jq {

namespace {

constexpr int GEN_COLS = 8;     // activation columns per warp
constexpr int GEN_WARPS = 8;    // rows per CTA

__device__ __forceinline__ uint32_t load_u32_2byte_aligned(const uint8_t *p) {
    const uint16_t *p16 = reinterpret_cast<const uint16_t *>(p);
    return (uint32_t)p16[0] | ((uint32_t)p16[1] << 16);
}

__device__ __forceinline__ int block_sumi(const uint8_t *wblk, const int *xq_ints) {
    int sumi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t w = load_u32_2byte_aligned(wblk + 2 + 4 * i);
        sumi = __dp4a((int)(w & 0x0F0F0F0Fu), xq_ints[i], sumi);             // weights 4i..4i+3
        sumi = __dp4a((int)((w >> 4) & 0x0F0F0F0Fu), xq_ints[i + 4], sumi);  // weights 16+4i..
    }
    return sumi;
}

__global__ void __launch_bounds__(GEN_WARPS * 32)
mmq_generic_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ xq, float *__restrict__ y,
                   int64_t K, int64_t N, int64_t M, int order, const MulMatBounds bounds) {
    const int lane = threadIdx.x & 31;
    const int64_t n = (int64_t)blockIdx.x * GEN_WARPS + (threadIdx.x >> 5);
    const int64_t m0 = (int64_t)blockIdx.y * GEN_COLS;
    if (n >= N) return;
    const int64_t nb = K / QK, n_super = K / SUPER;
    float acc[GEN_COLS];
#pragma unroll
    for (int c = 0; c < GEN_COLS; ++c) acc[c] = 0.0f;

    for (int64_t kb = lane; kb < nb; kb += 32) {
        const uint8_t *wblk = w + (n * nb + kb) * Q4_BYTES;
        if (!JQ_IN_EXTENT(bounds.w, wblk, Q4_BYTES, bounds.fault)) continue;
        const float d4 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(wblk));
        uint32_t wq[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) wq[i] = load_u32_2byte_aligned(wblk + 2 + 4 * i);
#pragma unroll
        for (int c = 0; c < GEN_COLS; ++c) {
            const int64_t m = m0 + c;
            if (m < M) {
                const uint8_t *xb = xq + q8_block_index(kb >> 2, m, n_super, M, order) * Q8_BYTES;
                if (!JQ_IN_EXTENT(bounds.xq, xb, Q8_BYTES, bounds.fault)) continue;
                const int sub = (int)(kb & 3);
                const int4 *xi = reinterpret_cast<const int4 *>(xb + Q8_QS_OFFSET + sub * QK);
                const int4 lo = __ldg(xi), hi = __ldg(xi + 1);
                const uint32_t ds = __ldg(reinterpret_cast<const uint32_t *>(xb) + sub);
                int sumi = 0;
                sumi = __dp4a((int)(wq[0] & 0x0F0F0F0Fu), lo.x, sumi);
                sumi = __dp4a((int)((wq[0] >> 4) & 0x0F0F0F0Fu), hi.x, sumi);
                sumi = __dp4a((int)(wq[1] & 0x0F0F0F0Fu), lo.y, sumi);
                sumi = __dp4a((int)((wq[1] >> 4) & 0x0F0F0F0Fu), hi.y, sumi);
                sumi = __dp4a((int)(wq[2] & 0x0F0F0F0Fu), lo.z, sumi);
                sumi = __dp4a((int)((wq[2] >> 4) & 0x0F0F0F0Fu), hi.z, sumi);
                sumi = __dp4a((int)(wq[3] & 0x0F0F0F0Fu), lo.w, sumi);
                sumi = __dp4a((int)((wq[3] >> 4) & 0x0F0F0F0Fu), hi.w, sumi);
                const float d8 = half_bits_to_float(ds & 0xFFFFu);
                const float s8 = half_bits_to_float(ds >> 16);
                acc[c] = fmaf(d4, fmaf((float)sumi, d8, -8.0f * s8), acc[c]);
            }
        }
    }
#pragma unroll
    for (int c = 0; c < GEN_COLS; ++c) {
        float v = acc[c];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off, 32);
        if (lane == 0 && m0 + c < M && JQ_IN_EXTENT(bounds.y, y + (m0 + c) * N + n, sizeof(float), bounds.fault)) y[(m0 + c) * N + n] = v;
    }
}

__global__ void __launch_bounds__(256)
block_sums_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ xq, int32_t *__restrict__ sums,
                  int64_t K, int64_t N, int64_t M, int order, const MulMatBounds bounds) {
    const int64_t nb = K / QK, n_super = K / SUPER;
    const int64_t total = N * nb;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / nb, kb = i - n * nb;
        const uint8_t *wblk = w + i * Q4_BYTES;
        if (!JQ_IN_EXTENT(bounds.w, wblk, Q4_BYTES, bounds.fault)) continue;
        for (int64_t m = 0; m < M; ++m) {
            const uint8_t *xb = xq + q8_block_index(kb >> 2, m, n_super, M, order) * Q8_BYTES;
            if (!JQ_IN_EXTENT(bounds.xq, xb, Q8_BYTES, bounds.fault) ||
                !JQ_IN_EXTENT(bounds.y, sums + (m * N + n) * nb + kb, sizeof(int32_t), bounds.fault))
                continue;
            const int *xi = reinterpret_cast<const int *>(xb + Q8_QS_OFFSET + (kb & 3) * QK);
            int x8[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) x8[j] = __ldg(xi + j);
            sums[(m * N + n) * nb + kb] = block_sumi(wblk, x8);
        }
    }
}

}  // namespace

int launch_mmq_generic(cudaStream_t st, const void *d_w, const void *d_xq, float *d_y, int64_t K, int64_t N,
                       int64_t M, int order) {
    if (N == 0 || M == 0) return JQ_OK;
    const int64_t gx = (N + GEN_WARPS - 1) / GEN_WARPS, gy = (M + GEN_COLS - 1) / GEN_COLS;
    if (gy > 65535) return set_error(JQ_ERR_TOO_LARGE, "generic multiply: M = %lld exceeds %d", (long long)M,
                                     65535 * GEN_COLS);
    (void)cudaGetLastError();  // a stale error of an earlier, unrelated call must not be taken for this launch's
    mmq_generic_kernel<<<dim3((unsigned)gx, (unsigned)gy), GEN_WARPS * 32, 0, st>>>(
        static_cast<const uint8_t *>(d_w), static_cast<const uint8_t *>(d_xq), d_y, K, N, M, order,
        mul_mat_bounds(d_w, d_xq, d_y, K, N, M, sizeof(float)));
    JQ_CUDA_TRY(cudaGetLastError());
    return JQ_OK;
}

int launch_block_sums(cudaStream_t st, const void *d_w, const void *d_xq, int32_t *d_sums, int64_t K,
                      int64_t N, int64_t M, int order) {
    const int64_t total = N * (K / QK);
    if (total == 0 || M == 0) return JQ_OK;
    int64_t ctas = (total + 255) / 256;
    if (ctas > 148 * 16) ctas = 148 * 16;
    (void)cudaGetLastError();  // a stale error of an earlier, unrelated call must not be taken for this launch's
    block_sums_kernel<<<(unsigned)ctas, 256, 0, st>>>(static_cast<const uint8_t *>(d_w),
                                                      static_cast<const uint8_t *>(d_xq), d_sums, K, N, M, order,
                                                      mul_mat_bounds(d_w, d_xq, d_sums, K, N, M, sizeof(int32_t) * (size_t)(K / QK)));
    JQ_CUDA_TRY(cudaGetLastError());
    return JQ_OK;
}

}  // namespace jq
