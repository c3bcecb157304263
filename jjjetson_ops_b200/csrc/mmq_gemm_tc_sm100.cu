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
//   warps 9-11  producers.  Per 256-value chunk of K a thread loads weight row p (144 bytes) and
//               activation column p (2 x 144 bytes) with 16-byte loads (p = its index, and p + 96), splits the nibbles in
//               registers and writes both as int8 tiles in the tensor core's canonical K-major
//               layout (8-row x 16-byte core matrices, 128 bytes apart along K, 256 bytes apart
//               along rows), plus fp32 tables of d4 and of (d8, -1.5*2^23*d8, -8*s8).
//
// Exact per-block scaling without integer work in the drain: before a buffer is used, the drain
// warps store the integer 0x4B400000 into it (tcgen05.st) and the MMA accumulates on top, so the
// value read back, taken as a float, is 1.5*2^23 + sumi exactly.  fma(that, d8, -1.5*2^23*d8) is
// round(sumi*d8) - the reference's own product (mm_q4_0_q8_1.cu:92) - which a second fma multiplies
// by d4 into the accumulator; both are packed fma.rn.f32x2 over pairs of neighbouring weight rows.
// The zero-point term -8*d4*s8 of the same formula is rank-1 per block, so it never touches the
// CUDA cores: per stage one tcgen05.mma.kind::f16 (A = s8, B = -8*d4, both exact in fp16, K = the
// stage's 8 blocks padded to 16) accumulates it in fp32 in a TMEM region of its own, added once at
// the end.  Three integer accumulator buffers keep the MMA latency off the drain's critical path.
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
constexpr int TC_ZA_OFF = 2 * TC_KB * TC_TILE;     // fp16 s8[128 columns][16] (8 blocks + 8 zeros), canonical layout
constexpr int TC_ZB_OFF = TC_ZA_OFF + TC_TILE;     // fp16 -8*d4[128 rows][16], canonical layout
constexpr int TC_D4_OFF = TC_ZB_OFF + TC_TILE;     // float d4[TC_KB][128]
constexpr int TC_XS_OFF = TC_D4_OFF + TC_KB * 128 * 4;   // float2 (d8, -1.5*2^23*d8)[TC_KB][128]
constexpr int TC_STAGE_BYTES = TC_XS_OFF + TC_KB * 128 * 8;
constexpr int TC_BAR_OFF = TC_STAGES * TC_STAGE_BYTES;
constexpr int TC_SMEM_BYTES = TC_BAR_OFF + 128;
constexpr int TC_DRAIN_WARPS = 8;
constexpr int TC_MMA_WARP = 8;
constexpr int TC_PROD_WARP0 = 9;
constexpr int TC_PROD_THREADS = 96;               // three producer warps: 12 warps x 168 registers fill the file
constexpr int TC_THREADS = 12 * 32;
constexpr int TC_ACC_BUFS = 3;                     // integer accumulator buffers of 128 columns
constexpr uint32_t TC_ZP_COL = TC_ACC_BUFS * TC_BN;  // fp32 zero-point accumulator, 128 columns
constexpr uint32_t TC_TMEM_COLS = 512;
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
    unsigned long long *trace;  // tracing aid: per 32-wide block, the SM clock at which each of CTA 0's 8 drain
                                // warps handed its accumulator buffer back (or nullptr)
};

__device__ __forceinline__ void tc_stamp(const TcParams &p, int g, int slot) {
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && g < 512) p.trace[g * 8 + slot] = (unsigned long long)clock64();
}

__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(reinterpret_cast<uint64_t &>(d))
        : "l"(reinterpret_cast<const uint64_t &>(a)), "l"(reinterpret_cast<const uint64_t &>(b)),
          "l"(reinterpret_cast<const uint64_t &>(c)));
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

// 32 lanes x 32 consecutive columns of 32-bit accumulator -> registers (completion: tcgen05.wait::ld)
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
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
    uint64_t *acc_full = bars + 4;      // [3] MMA completion -> drain warps
    uint64_t *acc_empty = bars + 7;     // [3] drain warps (buffer read out and re-armed) -> MMA warp
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 10);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t n0 = (int64_t)blockIdx.x * TC_BN, m0 = (int64_t)blockIdx.y * TC_BM;
    const int n_chunks = p.K / (TC_KB * QK);

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&stage_full[s], TC_PROD_THREADS / 32);
            mbar_init(&stage_empty[s], TC_DRAIN_WARPS);
        }
        for (int b = 0; b < TC_ACC_BUFS; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], TC_DRAIN_WARPS);
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

        // arm the accumulator buffers
#pragma unroll
        for (int b = 0; b < TC_ACC_BUFS; ++b) {
#pragma unroll
            for (int q = 0; q < 4; ++q) tmem_st16_const(t_lane + b * TC_BN + q * 16, MAGIC_I);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
#pragma unroll
            for (int b = 0; b < TC_ACC_BUFS; ++b) mbar_arrive(&acc_empty[b]);
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
                const int buf = g % TC_ACC_BUFS;
                if (!mbar_wait_bounded(&acc_full[buf], (uint32_t)(g / TC_ACC_BUFS) & 1u, p.fault)) {
                    alive = false;
                    break;
                }
                tc_fence_after();
                const uint2 xs = lds_v2(st + TC_XS_OFF + (kb * 128 + row) * 8);
                const float d8 = __uint_as_float(xs.x), c8 = __uint_as_float(xs.y);
                const float2 d8p = make_float2(d8, d8), c8p = make_float2(c8, c8);
                const uint32_t d4_addr = st + TC_D4_OFF + (kb * 128 + half * 64) * 4;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t v[32];
                    tmem_ld32_nowait(t_lane + buf * TC_BN + h * 32, v);
                    // the 32 weight scales of this half, fetched back to back while the TMEM load is in flight
                    uint4 d4[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) d4[q] = lds_v4(d4_addr + (h * 32 + q * 4) * 4);  // same address in every lane
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    // the sums are in registers: re-arm these columns right away, the stores overlap the arithmetic
                    tmem_st16_const(t_lane + buf * TC_BN + h * 32, MAGIC_I);
                    tmem_st16_const(t_lane + buf * TC_BN + h * 32 + 16, MAGIC_I);
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const float2 u0 = ffma2(make_float2(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1])), d8p, c8p);
                        const float2 u1 = ffma2(make_float2(__uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3])), d8p, c8p);
                        acc[h * 16 + 2 * q] =
                            ffma2(make_float2(__uint_as_float(d4[q].x), __uint_as_float(d4[q].y)), u0, acc[h * 16 + 2 * q]);
                        acc[h * 16 + 2 * q + 1] =
                            ffma2(make_float2(__uint_as_float(d4[q].z), __uint_as_float(d4[q].w)), u1, acc[h * 16 + 2 * q + 1]);
                    }
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);
                if (lane == 0) tc_stamp(p, g, warp);  // tracing aid: when each drain warp handed the buffer back
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&stage_empty[s]);  // tiles were consumed by the MMAs, tables by us
        }

        if (alive) {
            // zero-point term: complete once the last integer MMA (issued after it) has been seen
            tc_fence_after();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t v[32];
                tmem_ld32_nowait(t_lane + TC_ZP_COL + h * 32, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    acc[h * 16 + j].x += __uint_as_float(v[2 * j]);
                    acc[h * 16 + j].y += __uint_as_float(v[2 * j + 1]);
                }
            }
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
                tc_fence_after();
                {
                    // zero-point of the stage's 8 blocks: fp32 += s8[128 x 16] * (-8 d4)[128 x 16]^T, fp16 operands
                    const uint32_t idesc_zp = (1u << 4) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem + TC_ZP_COL),
                        "l"(tc_desc(st + TC_ZA_OFF)), "l"(tc_desc(st + TC_ZB_OFF)), "r"(idesc_zp), "r"(c > 0 ? 1u : 0u)
                        : "memory");
                }
                for (int kb = 0; kb < TC_KB; ++kb) {
                    const int g = c * TC_KB + kb;
                    const int buf = g % TC_ACC_BUFS;
                    if (!mbar_wait_bounded(&acc_empty[buf], (uint32_t)(g / TC_ACC_BUFS) & 1u, p.fault)) {
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
        const int pt0 = tid - TC_PROD_WARP0 * 32;  // 0..95; rows / columns pt0 and pt0 + 96 of the tile
        for (int c = 0; c < n_chunks; ++c) {
            const int s = c & 1;
            bool waited = false, dead = false;
            for (int pt = pt0; pt < 128 && !dead; pt += TC_PROD_THREADS) {
                const int64_t n = min(n0 + pt, p.N - 1);  // rows / columns past the end are clamped, never stored
                const int64_t m = min(m0 + pt, p.M - 1);
                // issue the global loads before waiting for the stage: they only need registers
                uint4 wv[9];
#pragma unroll
                for (int i = 0; i < 9; ++i) wv[i] = __ldg(reinterpret_cast<const uint4 *>(p.w + n * p.row_bytes + (size_t)c * 144) + i);
                // of the activation blocks only the scales pass through registers; the int8 values go
                // from global memory straight into their canonical tile positions (16-byte cp.async)
                const uint8_t *xb[2];
                uint4 xds[2];
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    xb[ks] = p.xq + q8_block_index(2 * c + ks, m, p.n_super, p.M, p.order) * Q8_BYTES;
                    xds[ks] = __ldg(reinterpret_cast<const uint4 *>(xb[ks]));
                }
                if (!waited) {
                    waited = true;
                    if (c >= 2 && !mbar_wait_bounded(&stage_empty[s], (uint32_t)((c >> 1) - 1) & 1u, p.fault)) {
                        dead = true;
                        break;
                    }
                }
                const uint32_t st = sbase + s * TC_STAGE_BYTES;
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const uint32_t tile = st + TC_A_OFF + (ks * 4 + g) * TC_TILE;
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(tile + tile_off(pt, 0)),
                                     "l"(xb[ks] + Q8_QS_OFFSET + 32 * g)
                                     : "memory");
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(tile + tile_off(pt, 1)),
                                     "l"(xb[ks] + Q8_QS_OFFSET + 32 * g + 16)
                                     : "memory");
                    }
                }

                // ---- weights: 8 blocks of 18 bytes out of 36 words, nibbles split into two 16-byte chunks
                const uint32_t *ww = reinterpret_cast<const uint32_t *>(wv);
                uint32_t zb[TC_KB];
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
                    zb[j] = dbits;
                }
                {
                    // -8 * d4 as fp16 (exact: a power of two; finite unless |d4| > 8188), 8 blocks + 8 zeros
                    uint32_t zw[4];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const __half2 d2 = __halves2half2(__ushort_as_half((unsigned short)zb[2 * t]),
                                                          __ushort_as_half((unsigned short)zb[2 * t + 1]));
                        const __half2 sc = __hmul2(d2, __float2half2_rn(-8.0f));
                        zw[t] = *reinterpret_cast<const uint32_t *>(&sc);
                    }
                    sts_v4(st + TC_ZB_OFF + tile_off(pt, 0), make_uint4(zw[0], zw[1], zw[2], zw[3]));
                    sts_v4(st + TC_ZB_OFF + tile_off(pt, 1), make_uint4(0u, 0u, 0u, 0u));
                }
                // ---- activation scales expanded to fp32, and s8 as fp16 for the zero-point MMA
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    const uint32_t dsw[4] = {xds[ks].x, xds[ks].y, xds[ks].z, xds[ks].w};
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const int j = ks * 4 + g;
                        const float d8 = half_bits_to_float(dsw[g] & 0xFFFFu);
                        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(st + TC_XS_OFF + (j * 128 + pt) * 8), "f"(d8),
                                     "f"(-MAGIC_F * d8)
                                     : "memory");
                    }
                }
                {
                    const uint32_t s01 = (xds[0].x >> 16) | (xds[0].y & 0xFFFF0000u), s23 = (xds[0].z >> 16) | (xds[0].w & 0xFFFF0000u);
                    const uint32_t s45 = (xds[1].x >> 16) | (xds[1].y & 0xFFFF0000u), s67 = (xds[1].z >> 16) | (xds[1].w & 0xFFFF0000u);
                    sts_v4(st + TC_ZA_OFF + tile_off(pt, 0), make_uint4(s01, s23, s45, s67));
                    sts_v4(st + TC_ZA_OFF + tile_off(pt, 1), make_uint4(0u, 0u, 0u, 0u));
                }
            }
            if (dead) break;
            asm volatile("cp.async.wait_all;" ::: "memory");
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
    p.trace = static_cast<unsigned long long *>(next_trace_slot());
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
