// Prefill-regime multiply on the 5th-generation tensor cores: tcgen05.mma.kind::i8 with TMEM
// accumulators, one 32-wide block per MMA, drained and rescaled block by block.
//
// Work to replace: q4_0_q8_1_mat_mul_kernel (reference src/cuda/mm_q4_0_q8_1.cu:164-289) for large
// batches.  A CTA owns a 128 (activation columns) x 128 (weight rows) tile of Y and is specialised
// by warp:
//
//   warps 0-7   drain warps.  TMEM lane = activation column m, TMEM column = weight row n.  Warp w
//               owns lanes 32*(w%4).. and columns 64*(w/4)..; per block it reads its 32 x 64 s32
//               sums with tcgen05.ld, rescales them and adds them to 64 fp32 registers per thread.
//   warp 8      allocates TMEM and issues the MMAs: per 32-wide block one 128 x 128 x 32
//               tcgen05.mma.kind::i8 (A = activations, s8; B = weight nibbles, u8) into one of two
//               accumulator buffers, then tcgen05.commit onto an mbarrier.
//   warps 9-12  producers.  Per 256-value chunk of K thread p loads weight row p (144 bytes) and
//               activation column p (2 x 144 bytes) with 16-byte loads, splits the nibbles in
//               registers and writes both as int8 tiles in the tensor core's canonical K-major
//               layout (8-row x 16-byte core matrices, 128 bytes apart along K, 256 bytes apart
//               along rows), plus fp32 tables of d4 and of (d8, -1.5*2^23*d8, -8*s8).
//
// Exact per-block scaling without integer work in the drain: before a buffer is used, the drain
// warps store the integer 0x4B400000 into it (tcgen05.st) and the MMA accumulates on top, so the
// value read back, taken as a float, is 1.5*2^23 + sumi exactly.  fma(that, d8, -1.5*2^23*d8) is
// round(sumi*d8) - the reference's own product (mm_q4_0_q8_1.cu:92) - then -8*s8 is added and the
// result is multiplied by d4 into the accumulator, all as packed fma.rn.f32x2 / add.rn.f32x2 over
// pairs of neighbouring weight rows.
//
// Every wait is a bounded poll; a wait that runs out sets the device fault word, and every warp
// still reaches the common exit where TMEM is released.
#include "jq_common.cuh"

namespace jq {

namespace {

constexpr int TC_BM = 128;   // activation columns per CTA (MMA M, TMEM lanes)
constexpr int TC_BN = 128;   // weight rows per CTA (MMA N, TMEM columns)
constexpr int TC_KB = 8;     // 32-wide blocks per pipeline stage (256 values of K)
constexpr int TC_STAGES = 2;
constexpr int TC_TILE = 4096;                      // one 128 x 32-byte int8 operand tile
constexpr int TC_A_OFF = 0;                        // activations: TC_KB tiles
constexpr int TC_B_OFF = TC_KB * TC_TILE;          // weights:     TC_KB tiles
constexpr int TC_D4_OFF = 2 * TC_KB * TC_TILE;     // float d4[TC_KB][128]
constexpr int TC_XS_OFF = TC_D4_OFF + TC_KB * 128 * 4;   // float4 (d8, c8, ms, 0)[TC_KB][128]
constexpr int TC_STAGE_BYTES = TC_XS_OFF + TC_KB * 128 * 16;
constexpr int TC_BAR_OFF = TC_STAGES * TC_STAGE_BYTES;
constexpr int TC_SMEM_BYTES = TC_BAR_OFF + 128;
constexpr int TC_DRAIN_WARPS = 8;
constexpr int TC_MMA_WARP = 8;
constexpr int TC_PROD_WARP0 = 9;
constexpr int TC_THREADS = 13 * 32;
constexpr uint32_t TC_TMEM_COLS = 256;             // two 128-column accumulator buffers
constexpr uint32_t TC_LBO = 128, TC_SBO = 256;     // canonical layout strides (bytes)
constexpr uint32_t MAGIC_I = 0x4B400000u;
constexpr float MAGIC_F = 12582912.0f;
constexpr uint32_t MASK4 = 0x0F0F0F0Fu;

struct TcParams {
    const uint8_t *w;
    const uint8_t *xq;
    float *y;
    int *fault;
    int64_t N, M;
    int K, order, n_super;
    uint32_t row_bytes;
};

__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(reinterpret_cast<uint64_t &>(d))
        : "l"(reinterpret_cast<const uint64_t &>(a)), "l"(reinterpret_cast<const uint64_t &>(b)),
          "l"(reinterpret_cast<const uint64_t &>(c)));
    return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
    float2 d;
    asm("add.rn.f32x2 %0, %1, %2;"
        : "=l"(reinterpret_cast<uint64_t &>(d))
        : "l"(reinterpret_cast<const uint64_t &>(a)), "l"(reinterpret_cast<const uint64_t &>(b)));
    return d;
}

__device__ __forceinline__ void sts_v4(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 lanes x 32 consecutive columns of 32-bit accumulator -> registers
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// the same constant into 32 lanes x 16 consecutive columns
__device__ __forceinline__ void tmem_st16_const(uint32_t taddr, uint32_t v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(taddr),
                 "r"(v)
                 : "memory");
}

// shared-memory matrix descriptor: K-major, no swizzle, version 1
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(TC_LBO >> 4) << 16) | ((uint64_t)(TC_SBO >> 4) << 32) |
           ((uint64_t)1 << 46);
}

// canonical position of the 16-byte K-chunk kc (0/1) of row r inside a 128 x 32-byte tile
__device__ __forceinline__ uint32_t tile_off(int r, int kc) {
    return (uint32_t)((r >> 3) * TC_SBO + kc * TC_LBO + (r & 7) * 16);
}

__global__ void __launch_bounds__(TC_THREADS, 1) gemm_q4_0_q8_1_tc_kernel(const TcParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + TC_BAR_OFF);
    uint64_t *stage_full = bars;        // [2] producers -> MMA warp and drain warps
    uint64_t *stage_empty = bars + 2;   // [2] drain warps -> producers
    uint64_t *acc_full = bars + 4;      // [2] MMA completion -> drain warps
    uint64_t *acc_empty = bars + 6;     // [2] drain warps (buffer read out and re-armed) -> MMA warp
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t n0 = (int64_t)blockIdx.x * TC_BN, m0 = (int64_t)blockIdx.y * TC_BM;
    const int n_chunks = p.K / (TC_KB * QK);

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&stage_full[s], 4);
            mbar_init(&stage_empty[s], TC_DRAIN_WARPS);
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], TC_DRAIN_WARPS);
        }
        fence_mbar_init();
    }
    if (warp == TC_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(TC_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(tmem_slot);

    if (warp < TC_DRAIN_WARPS) {
        // =============================== drain warps =======================================
        const int half = warp >> 2;                      // which 64 of the 128 weight rows
        const int row = (warp & 3) * 32 + lane;          // activation column inside the tile (TMEM lane)
        const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(half * 64);
        float2 acc[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = make_float2(0.f, 0.f);

        // arm both accumulator buffers
#pragma unroll
        for (int b = 0; b < 2; ++b) {
#pragma unroll
            for (int q = 0; q < 4; ++q) tmem_st16_const(t_lane + b * TC_BN + q * 16, MAGIC_I);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(&acc_empty[0]);
            mbar_arrive(&acc_empty[1]);
        }

        bool alive = true;
        for (int c = 0; c < n_chunks && alive; ++c) {
            const int s = c & 1;
            if (!mbar_wait_bounded(&stage_full[s], (uint32_t)(c >> 1) & 1u, p.fault)) {  // scale tables of the stage
                alive = false;
                break;
            }
            const uint32_t st = sbase + s * TC_STAGE_BYTES;
#pragma unroll 1
            for (int kb = 0; kb < TC_KB; ++kb) {
                const int g = c * TC_KB + kb;  // global block index
                const int buf = g & 1;
                if (!mbar_wait_bounded(&acc_full[buf], (uint32_t)(g >> 1) & 1u, p.fault)) {
                    alive = false;
                    break;
                }
                tc_fence_after();
                const uint4 xs = lds_v4(st + TC_XS_OFF + (kb * 128 + row) * 16);
                const float d8 = __uint_as_float(xs.x), c8 = __uint_as_float(xs.y), ms = __uint_as_float(xs.z);
                const float2 d8p = make_float2(d8, d8), c8p = make_float2(c8, c8), msp = make_float2(ms, ms);
                const uint32_t d4_addr = st + TC_D4_OFF + (kb * 128 + half * 64) * 4;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t v[32];
                    tmem_ld32(t_lane + buf * TC_BN + h * 32, v);
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const uint4 d4 = lds_v4(d4_addr + (h * 32 + q * 4) * 4);  // same address in every lane
                        float2 u0 = ffma2(make_float2(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1])), d8p, c8p);
                        float2 u1 = ffma2(make_float2(__uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3])), d8p, c8p);
                        u0 = fadd2(u0, msp);
                        u1 = fadd2(u1, msp);
                        acc[h * 16 + 2 * q] = ffma2(make_float2(__uint_as_float(d4.x), __uint_as_float(d4.y)), u0, acc[h * 16 + 2 * q]);
                        acc[h * 16 + 2 * q + 1] =
                            ffma2(make_float2(__uint_as_float(d4.z), __uint_as_float(d4.w)), u1, acc[h * 16 + 2 * q + 1]);
                    }
                }
                // re-arm the buffer for the MMA two blocks ahead and hand it back
#pragma unroll
                for (int q = 0; q < 4; ++q) tmem_st16_const(t_lane + buf * TC_BN + q * 16, MAGIC_I);
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&stage_empty[s]);  // tiles were consumed by the MMAs, tables by us
        }

        if (alive) {
            const int64_t m = m0 + row;
            if (m < p.M) {
                float *dst = p.y + m * p.N + n0 + half * 64;
                const int64_t n_left = p.N - (n0 + half * 64);
                if (n_left >= 64 && ((uintptr_t)dst & 15u) == 0) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        reinterpret_cast<float4 *>(dst)[j] = make_float4(acc[2 * j].x, acc[2 * j].y, acc[2 * j + 1].x, acc[2 * j + 1].y);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (2 * j < n_left) dst[2 * j] = acc[j].x;
                        if (2 * j + 1 < n_left) dst[2 * j + 1] = acc[j].y;
                    }
                }
            }
        }
    } else if (warp == TC_MMA_WARP) {
        // =============================== MMA issuer =========================================
        if (lane == 0) {
            // instruction descriptor: D = s32, A = s8, B = u8, both K-major, N = 128, M = 128
            const uint32_t idesc = (2u << 4) | (1u << 7) | (0u << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            bool alive = true;
            for (int c = 0; c < n_chunks && alive; ++c) {
                const int s = c & 1;
                if (!mbar_wait_bounded(&stage_full[s], (uint32_t)(c >> 1) & 1u, p.fault)) break;
                const uint32_t st = sbase + s * TC_STAGE_BYTES;
                for (int kb = 0; kb < TC_KB; ++kb) {
                    const int g = c * TC_KB + kb;
                    const int buf = g & 1;
                    if (!mbar_wait_bounded(&acc_empty[buf], (uint32_t)(g >> 1) & 1u, p.fault)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t da = tc_desc(st + TC_A_OFF + kb * TC_TILE);
                    const uint64_t db = tc_desc(st + TC_B_OFF + kb * TC_TILE);
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem + buf * TC_BN),
                        "l"(da), "l"(db), "r"(idesc), "r"(1u)
                        : "memory");
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                     smem_u32(&acc_full[buf]))
                                 : "memory");
                }
            }
        }
    } else {
        // =============================== producers ==========================================
        const int pt = tid - TC_PROD_WARP0 * 32;  // 0..127: weight row and activation column of the tile
        const int64_t n = min(n0 + pt, p.N - 1);  // rows / columns past the end are clamped, never stored
        const int64_t m = min(m0 + pt, p.M - 1);
        const uint8_t *wrow = p.w + n * p.row_bytes;
        for (int c = 0; c < n_chunks; ++c) {
            const int s = c & 1;
            // issue the global loads before waiting for the stage: they only need registers
            uint4 wv[9];
#pragma unroll
            for (int i = 0; i < 9; ++i) wv[i] = __ldg(reinterpret_cast<const uint4 *>(wrow + (size_t)c * 144) + i);
            uint4 xv[2][9];
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
                const uint8_t *xb = p.xq + q8_block_index(2 * c + ks, m, p.n_super, p.M, p.order) * Q8_BYTES;
#pragma unroll
                for (int i = 0; i < 9; ++i) xv[ks][i] = __ldg(reinterpret_cast<const uint4 *>(xb) + i);
            }
            if (c >= 2 && !mbar_wait_bounded(&stage_empty[s], (uint32_t)((c >> 1) - 1) & 1u, p.fault)) break;
            const uint32_t st = sbase + s * TC_STAGE_BYTES;

            // ---- weights: 8 blocks of 18 bytes out of 36 words, nibbles split into two 16-byte chunks
            const uint32_t *ww = reinterpret_cast<const uint32_t *>(wv);
#pragma unroll
            for (int j = 0; j < TC_KB; ++j) {
                uint32_t q[4], dbits;
                if ((j & 1) == 0) {  // block starts on a word boundary: [d | q0 q1] [q2..q5] ...
                    const int w0 = (j / 2) * 9;
                    dbits = ww[w0] & 0xFFFFu;
#pragma unroll
                    for (int t = 0; t < 4; ++t) q[t] = __funnelshift_r(ww[w0 + t], ww[w0 + t + 1], 16);
                } else {  // block starts in the middle of a word
                    const int w0 = (j / 2) * 9 + 4;
                    dbits = ww[w0] >> 16;
#pragma unroll
                    for (int t = 0; t < 4; ++t) q[t] = ww[w0 + 1 + t];
                }
                const uint32_t tile = st + TC_B_OFF + j * TC_TILE;
                sts_v4(tile + tile_off(pt, 0), make_uint4(q[0] & MASK4, q[1] & MASK4, q[2] & MASK4, q[3] & MASK4));
                sts_v4(tile + tile_off(pt, 1),
                       make_uint4((q[0] >> 4) & MASK4, (q[1] >> 4) & MASK4, (q[2] >> 4) & MASK4, (q[3] >> 4) & MASK4));
                sts_f32(st + TC_D4_OFF + (j * 128 + pt) * 4, half_bits_to_float(dbits));
            }
            // ---- activations: int8 values as they are, scales expanded to fp32
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
                const uint32_t dsw[4] = {xv[ks][0].x, xv[ks][0].y, xv[ks][0].z, xv[ks][0].w};
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int j = ks * 4 + g;
                    const uint32_t tile = st + TC_A_OFF + j * TC_TILE;
                    sts_v4(tile + tile_off(pt, 0), xv[ks][1 + 2 * g]);
                    sts_v4(tile + tile_off(pt, 1), xv[ks][2 + 2 * g]);
                    const float d8 = half_bits_to_float(dsw[g] & 0xFFFFu);
                    const float s8 = half_bits_to_float(dsw[g] >> 16);
                    sts_v4(st + TC_XS_OFF + (j * 128 + pt) * 16,
                           make_uint4(__float_as_uint(d8), __float_as_uint(-MAGIC_F * d8), __float_as_uint(-8.0f * s8), 0u));
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // tiles are read by the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(&stage_full[s]);
        }
    }

    // common exit: nobody touches TMEM any more, release it
    tc_fence_before();
    __syncthreads();
    if (warp == TC_MMA_WARP) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TC_TMEM_COLS) : "memory");
    }
}

}  // namespace

int launch_gemm_tc(cudaStream_t st, const void *d_w, const void *d_xq, float *d_y, int64_t K, int64_t N, int64_t M,
                   int order) {
    if (K % (TC_KB * QK) != 0) return set_error(JQ_ERR_UNSUPPORTED, "tcgen05 GEMM needs K %% 256 == 0 (K = %lld)", (long long)K);
    if (((uintptr_t)d_w & 15u) != 0 || ((uintptr_t)d_xq & 15u) != 0)
        return set_error(JQ_ERR_UNSUPPORTED, "tcgen05 GEMM needs 16-byte aligned operands");
    if (N == 0 || M == 0) return JQ_OK;
    DeviceCaps caps;
    if (int rc = device_caps(&caps)) return rc;
    if (caps.cc / 10 != 10) return set_error(JQ_ERR_UNSUPPORTED, "tcgen05 needs an sm_100-class device");
    const int64_t gx = (N + TC_BN - 1) / TC_BN, gy = (M + TC_BM - 1) / TC_BM;
    if (gy > 65535 || K > (1 << 24)) return set_error(JQ_ERR_UNSUPPORTED, "shape too large for the tcgen05 GEMM");
    TcParams p{};
    p.w = static_cast<const uint8_t *>(d_w);
    p.xq = static_cast<const uint8_t *>(d_xq);
    p.y = d_y;
    p.fault = device_fault_ptr();
    p.N = N;
    p.M = M;
    p.K = (int)K;
    p.order = order;
    p.n_super = (int)(K / SUPER);
    p.row_bytes = (uint32_t)(K / QK * Q4_BYTES);
    static thread_local int attr_done_dev = -1;
    int dev = 0;
    JQ_CUDA_TRY(cudaGetDevice(&dev));
    if (attr_done_dev != dev) {
        JQ_CUDA_TRY(cudaFuncSetAttribute(gemm_q4_0_q8_1_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES));
        attr_done_dev = dev;
    }
    gemm_q4_0_q8_1_tc_kernel<<<dim3((unsigned)gx, (unsigned)gy), TC_THREADS, TC_SMEM_BYTES, st>>>(p);
    JQ_CUDA_TRY(cudaGetLastError());
    return JQ_OK;
}

}  // namespace jq
