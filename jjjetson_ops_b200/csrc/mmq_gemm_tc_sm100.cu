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
//   warp 8      allocates TMEM and issues the MMAs: per 32-wide block a bias MMA and one
//               128 x 128 x 32 tcgen05.mma.kind::i8 (A = activations, s8; B = weight nibbles, u8)
//               into one of three accumulator buffers, then tcgen05.commit onto an mbarrier.
//   warps 9-11  producers.  K advances in stages of 128 values (one Q8_1 super-block, four Q4_0
//               blocks).  The 128 weight rows and 128 activation columns of a stage are 256 tasks
//               dealt to the 96 producer threads.  A weight task loads 72 bytes one stage ahead
//               into registers, splits the nibbles and writes four int8 tiles in the tensor core's
//               canonical K-major layout (8-row x 16-byte core matrices, 128 bytes apart along K,
//               256 bytes apart along rows) plus the fp32 table of d4.  An activation task sends
//               the int8 values from global memory straight to their tile positions (cp.async) and
//               writes the (d8, bias correction) table.  A stage is published one iteration after
//               it was issued, so the copies have a whole iteration to land.
//
// Exact per-block scaling without integer or conversion work in the drain.  Every accumulator is
// first set to 2^17 by an MMA of a constant tile with itself (32 * 64 * 64), more than the largest
// |sumi| = 32 * 127 * 15, and the block's MMA accumulates on top.  The result is a positive integer
// below 2^23, so its bit pattern read as a float is the subnormal (2^17 + sumi) * 2^-149, and
//     fma(that, d8 * 2^100, -2^17 * d8 * 2^-49) = round(sumi * d8) * 2^-49
// with a single rounding: the reference's own product (mm_q4_0_q8_1.cu:92) up to an exact power of
// two, which the second fma removes by multiplying with d4 * 2^49.  Both are packed fma.rn.f32x2
// over pairs of neighbouring weight rows; no value is ever flushed (fma.rn keeps subnormals).
// The zero-point term -8*d4*s8 of the same formula is rank-1 per block, so it never touches the
// CUDA cores: per stage one tcgen05.mma.kind::f16 (A = s8, B = -8*d4, both exact in fp16, K = the
// stage's 4 blocks padded to 16) accumulates it in fp32 in a TMEM region of its own, added once at
// the end.
//
// The drain is software-pipelined: iteration g starts the TMEM load of block g, adds block g-1 to
// the accumulators while the load is in flight, then converts block g and hands its buffer back.
// That needs 64 (load) + 64 (previous block) + 64 (accumulators) live registers, so the drain
// warp-groups grow their register allowance with setmaxnreg and the other warp-group shrinks.
//
// Every mbarrier wait is a bounded poll; a wait that runs out sets the device fault word, and every
// warp still reaches the common exit where TMEM is released.
#include "tc_common.cuh"

namespace jq {

namespace {

constexpr int TC_BM = 128;   // activation columns per CTA (MMA M, TMEM lanes)
constexpr int TC_BN = 128;   // weight rows per CTA (MMA N, TMEM columns)
constexpr int TC_KB = 4;     // 32-wide blocks per pipeline stage (one Q8_1 super-block of K)
constexpr int TC_KB_LOG2 = 2;
constexpr int TC_STAGES = 4;
constexpr int TC_A_OFF = 0;                        // activations: TC_KB tiles
constexpr int TC_B_OFF = TC_KB * TC_TILE;          // weights:     TC_KB tiles
constexpr int TC_ZA_OFF = 2 * TC_KB * TC_TILE;     // fp16 s8[128 columns][16] (4 blocks + 12 zeros), canonical layout
constexpr int TC_ZB_OFF = TC_ZA_OFF + TC_TILE;     // fp16 -8*d4[128 rows][16], canonical layout
constexpr int TC_D4_OFF = TC_ZB_OFF + TC_TILE;     // float (d4 * 2^49)[TC_KB][128]
constexpr int TC_XS_OFF = TC_D4_OFF + TC_KB * 128 * 4;   // float2 (d8 * 2^100, -2^17 * d8 * 2^-49)[TC_KB][128]
constexpr int TC_STAGE_BYTES = TC_XS_OFF + TC_KB * 128 * 8;
constexpr int TC_BIAS_OFF = TC_STAGES * TC_STAGE_BYTES;   // one operand tile with every byte = TC_BIAS_BYTE
constexpr int TC_BAR_OFF = TC_BIAS_OFF + TC_TILE;
constexpr int TC_SMEM_BYTES = TC_BAR_OFF + 128;
constexpr int TC_DRAIN_WARPS = 8;
constexpr int TC_MMA_WARP = 8;
constexpr int TC_PROD_WARP0 = 9;
constexpr int TC_PROD_THREADS = 96;
constexpr int TC_THREADS = 12 * 32;
// Registers per thread after setmaxnreg.  The CTA starts with 168 x 384 = 64512 registers and the two settings
// must not ask for more than that in total, or the second setmaxnreg.inc never returns.
constexpr int TC_DRAIN_REGS = 208;
constexpr int TC_PROD_REGS = 88;
static_assert(8 * TC_DRAIN_REGS + 4 * TC_PROD_REGS <= 12 * 168, "setmaxnreg budget exceeds the CTA's allocation");
constexpr int TC_ACC_BUFS = 3;                     // integer accumulator buffers of 128 columns
constexpr uint32_t TC_ZP_COL = TC_ACC_BUFS * TC_BN;  // fp32 zero-point accumulator, 128 columns
constexpr uint32_t TC_TMEM_COLS = 512;
constexpr uint32_t TC_BIAS_BYTE = 0x40u;           // 32 * 64 * 64 = 2^17
constexpr int TC_BIAS_LOG2 = 17;
constexpr int TC_D8_SHIFT = 100;                   // d8 is carried as d8 * 2^100 ...
constexpr int TC_D4_SHIFT = 149 - TC_D8_SHIFT;     // ... and d4 as d4 * 2^49: the powers of two cancel
constexpr uint32_t MASK4 = 0x0F0F0F0Fu;
// exact power-of-two factors as bit patterns: 2^100, 2^49 and -2^(17-49)
constexpr uint32_t D8_SCALE_BITS = (uint32_t)(127 + TC_D8_SHIFT) << 23;
constexpr uint32_t D4_SCALE_BITS = (uint32_t)(127 + TC_D4_SHIFT) << 23;
constexpr uint32_t C8_SCALE_BITS = 0x80000000u | ((uint32_t)(127 + TC_BIAS_LOG2 - TC_D4_SHIFT) << 23);

struct TcParams {
    const uint8_t *w;
    const uint8_t *xq;
    float *y;
    int *fault;
    int64_t N, M;
    int K, order, n_super;
    uint32_t row_bytes;
    unsigned long long *trace;  // tracing aid (or nullptr): SM clock stamps of CTA (0,0), 512 rows of 8
};

// Tracing aid.  Rows 0-127: per block, when each drain warp saw the accumulator complete; rows
// 128-255: when it had added the previous block; rows 256-383: when it handed the buffer back;
// rows 384-511: column 0 = when the MMA of the block was issued, columns 1-3 = when each producer
// warp published the stage that starts with the block.
__device__ __forceinline__ void tc_stamp(const TcParams &p, int g, int kind, int slot) {
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && g < 128) {
        p.trace[(kind * 128 + g) * 8 + slot] = (unsigned long long)clock64();
    }
}

__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(reinterpret_cast<uint64_t &>(d))
        : "l"(reinterpret_cast<const uint64_t &>(a)), "l"(reinterpret_cast<const uint64_t &>(b)),
          "l"(reinterpret_cast<const uint64_t &>(c)));
    return d;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}

// One weight task of a stage: the row's 72 bytes (already in registers) -> four int8 tiles,
// the d4 table and the row's fp16 zero-point operand.
__device__ __forceinline__ void tc_unpack_weight_row(uint32_t st, int r, const uint2 (&wv)[9]) {
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
        sts_v4(tile + tile_off(r, 0), make_uint4(q[0] & MASK4, q[1] & MASK4, q[2] & MASK4, q[3] & MASK4));
        sts_v4(tile + tile_off(r, 1), make_uint4((q[0] >> 4) & MASK4, (q[1] >> 4) & MASK4, (q[2] >> 4) & MASK4, (q[3] >> 4) & MASK4));
        sts_f32(st + TC_D4_OFF + (j * 128 + r) * 4, half_bits_to_float(dbits) * __uint_as_float(D4_SCALE_BITS));
        zb[j] = dbits;
    }
    // -8 * d4 as fp16 (exact: a power of two; finite unless |d4| > 8188); the 12 padding values stay zero
    uint32_t zw[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const __half2 d2 = __halves2half2(__ushort_as_half((unsigned short)zb[2 * t]), __ushort_as_half((unsigned short)zb[2 * t + 1]));
        const __half2 sc = __hmul2(d2, __float2half2_rn(-8.0f));
        zw[t] = *reinterpret_cast<const uint32_t *>(&sc);
    }
    sts_v4(st + TC_ZB_OFF + tile_off(r, 0), make_uint4(zw[0], zw[1], 0u, 0u));
}

// One activation task of a stage: the column's 128 int8 values go from global memory straight
// into the four tiles; the scales (already in registers) become the drain's table and the fp16
// zero-point operand.
__device__ __forceinline__ void tc_stage_activation_col(uint32_t st, int r, const uint8_t *xb, uint4 ds) {
#pragma unroll
    for (int j = 0; j < TC_KB; ++j) {
        const uint32_t tile = st + TC_A_OFF + j * TC_TILE;
        cp_async16(tile + tile_off(r, 0), xb + Q8_QS_OFFSET + 32 * j);
        cp_async16(tile + tile_off(r, 1), xb + Q8_QS_OFFSET + 32 * j + 16);
    }
    const uint32_t dsw[4] = {ds.x, ds.y, ds.z, ds.w};
#pragma unroll
    for (int j = 0; j < TC_KB; ++j) {
        const float d8 = half_bits_to_float(dsw[j] & 0xFFFFu);
        asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(st + TC_XS_OFF + (j * 128 + r) * 8),
                     "f"(d8 * __uint_as_float(D8_SCALE_BITS)), "f"(d8 * __uint_as_float(C8_SCALE_BITS))
                     : "memory");
    }
    const uint32_t s01 = (ds.x >> 16) | (ds.y & 0xFFFF0000u), s23 = (ds.z >> 16) | (ds.w & 0xFFFF0000u);
    sts_v4(st + TC_ZA_OFF + tile_off(r, 0), make_uint4(s01, s23, 0u, 0u));
}

__global__ void __launch_bounds__(TC_THREADS, 1) gemm_q4_0_q8_1_tc_kernel(const TcParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + TC_BAR_OFF);
    uint64_t *stage_full = bars;                          // [TC_STAGES] producers -> MMA warp and drain warps
    uint64_t *stage_empty = bars + TC_STAGES;             // [TC_STAGES] drain warps -> producers
    uint64_t *acc_full = bars + 2 * TC_STAGES;            // [TC_ACC_BUFS] MMA completion -> drain warps
    uint64_t *acc_empty = acc_full + TC_ACC_BUFS;         // [TC_ACC_BUFS] drain warps (buffer read out) -> MMA warp
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + TC_ACC_BUFS);
    static_assert((2 * TC_STAGES + 2 * TC_ACC_BUFS) * 8 + 4 <= 128, "barrier block too small");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t n0 = (int64_t)blockIdx.x * TC_BN, m0 = (int64_t)blockIdx.y * TC_BM;
    const int n_chunks = p.K / (TC_KB * QK);

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(&stage_full[s], TC_PROD_THREADS / 32);
            mbar_init(&stage_empty[s], TC_DRAIN_WARPS);
        }
        for (int b = 0; b < TC_ACC_BUFS; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], TC_DRAIN_WARPS);
        }
        fence_mbar_init();
    }
    if (tid < TC_TILE / 16) {
        // the bias tile, and the zero half (K = 8..15) of every stage's fp16 zero-point operands
        const uint32_t b4 = TC_BIAS_BYTE * 0x01010101u;
        sts_v4(sbase + TC_BIAS_OFF + tid * 16, make_uint4(b4, b4, b4, b4));
        if (tid < 128) {
            for (int s = 0; s < TC_STAGES; ++s) {
                sts_v4(sbase + s * TC_STAGE_BYTES + TC_ZA_OFF + tile_off(tid, 1), make_uint4(0u, 0u, 0u, 0u));
                sts_v4(sbase + s * TC_STAGE_BYTES + TC_ZB_OFF + tile_off(tid, 1), make_uint4(0u, 0u, 0u, 0u));
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // read by the tensor core
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
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(TC_DRAIN_REGS));
        const int half = warp >> 2;                      // which 64 of the 128 weight rows
        const int row = (warp & 3) * 32 + lane;          // activation column inside the tile (TMEM lane)
        const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(half * 64);
        float2 acc[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = make_float2(0.f, 0.f);

        // all accumulator buffers start out free
        if (lane == 0) {
#pragma unroll
            for (int b = 0; b < TC_ACC_BUFS; ++b) mbar_arrive(&acc_empty[b]);
        }

        const int n_blocks = n_chunks * TC_KB;
        float2 u[32];  // sumi * d8 (times 2^-49) of the previous block, for this thread's 64 weight rows
#pragma unroll
        for (int j = 0; j < 32; ++j) u[j] = make_float2(0.f, 0.f);
        uint32_t d4_prev = sbase + TC_D4_OFF + half * 64 * 4;  // the first iteration multiplies zeros by block 0's table
        bool alive = true;
#pragma unroll 1
        for (int g = 0; g < n_blocks; ++g) {
            const int c = g >> TC_KB_LOG2, kb = g & (TC_KB - 1), s = c % TC_STAGES;
            const int buf = g % TC_ACC_BUFS;
            const uint32_t st = sbase + s * TC_STAGE_BYTES;
            if (kb == 0 && !mbar_wait_bounded(&stage_full[s], (uint32_t)(c / TC_STAGES) & 1u, p.fault)) {  // the stage's tables
                alive = false;
                break;
            }
            if (!mbar_wait_bounded(&acc_full[buf], (uint32_t)(g / TC_ACC_BUFS) & 1u, p.fault)) {
                alive = false;
                break;
            }
            tc_fence_after();
            if (lane == 0) tc_stamp(p, g, 0, warp);
            uint32_t v0[32], v1[32];
            tmem_ld32_nowait(t_lane + buf * TC_BN, v0);
            tmem_ld32_nowait(t_lane + buf * TC_BN + 32, v1);
            const uint2 xs = lds_v2(st + TC_XS_OFF + (kb * 128 + row) * 8);

            // ---- block g-1 into the accumulators, while the load is in flight
#pragma unroll
            for (int hq = 0; hq < 4; ++hq) {
                uint4 d4[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) d4[q] = lds_v4(d4_prev + (hq * 4 + q) * 16);  // same address in every lane
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int e = hq * 4 + q;
                    acc[2 * e] = ffma2(make_float2(__uint_as_float(d4[q].x), __uint_as_float(d4[q].y)), u[2 * e], acc[2 * e]);
                    acc[2 * e + 1] = ffma2(make_float2(__uint_as_float(d4[q].z), __uint_as_float(d4[q].w)), u[2 * e + 1], acc[2 * e + 1]);
                }
            }
            if (kb == 0 && c > 0) {  // the previous stage's tables are no longer needed, nor its tiles
                __syncwarp();
                if (lane == 0) mbar_arrive(&stage_empty[(c - 1) % TC_STAGES]);
            }
            if (lane == 0) tc_stamp(p, g, 1, warp);

            // ---- block g: sums -> sumi * d8, buffer back to the MMA warp
            const float d8 = __uint_as_float(xs.x), c8 = __uint_as_float(xs.y);
            const float2 d8p = make_float2(d8, d8), c8p = make_float2(c8, c8);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                u[q] = ffma2(make_float2(__uint_as_float(v0[2 * q]), __uint_as_float(v0[2 * q + 1])), d8p, c8p);
                u[16 + q] = ffma2(make_float2(__uint_as_float(v1[2 * q]), __uint_as_float(v1[2 * q + 1])), d8p, c8p);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            if (lane == 0) tc_stamp(p, g, 2, warp);
            d4_prev = st + TC_D4_OFF + (kb * 128 + half * 64) * 4;
        }

        if (alive) {
            // the last block
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const uint4 d4 = lds_v4(d4_prev + e * 16);
                acc[2 * e] = ffma2(make_float2(__uint_as_float(d4.x), __uint_as_float(d4.y)), u[2 * e], acc[2 * e]);
                acc[2 * e + 1] = ffma2(make_float2(__uint_as_float(d4.z), __uint_as_float(d4.w)), u[2 * e + 1], acc[2 * e + 1]);
            }
            // zero-point term: complete, because its MMAs were issued before the last block's, which has been seen
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
        } else {
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        }
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(TC_PROD_REGS));
        if (warp == TC_MMA_WARP) {
            // =============================== MMA issuer =====================================
            if (lane == 0) {
                // instruction descriptor: D = s32, A = s8, B = u8, both K-major, N = 128, M = 128
                const uint32_t idesc = (2u << 4) | (1u << 7) | (0u << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
                // zero-point MMA: D = f32, A = B = f16, K = 16
                const uint32_t idesc_zp = (1u << 4) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
                const uint64_t dbias = tc_desc(sbase + TC_BIAS_OFF);
                bool alive = true;
                for (int c = 0; c < n_chunks && alive; ++c) {
                    const int s = c % TC_STAGES;
                    if (!mbar_wait_bounded(&stage_full[s], (uint32_t)(c / TC_STAGES) & 1u, p.fault)) break;
                    const uint32_t st = sbase + s * TC_STAGE_BYTES;
                    tc_fence_after();
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem + TC_ZP_COL),
                        "l"(tc_desc(st + TC_ZA_OFF)), "l"(tc_desc(st + TC_ZB_OFF)), "r"(idesc_zp), "r"(c > 0 ? 1u : 0u)
                        : "memory");
                    for (int kb = 0; kb < TC_KB; ++kb) {
                        const int g = c * TC_KB + kb;
                        const int buf = g % TC_ACC_BUFS;
                        if (!mbar_wait_bounded(&acc_empty[buf], (uint32_t)(g / TC_ACC_BUFS) & 1u, p.fault)) {
                            alive = false;
                            break;
                        }
                        tc_fence_after();
                        tc_stamp(p, g, 3, 0);
                        // accumulator = bias (overwriting), then += activations x nibbles
                        tc_mma_i8(tmem + buf * TC_BN, dbias, dbias, idesc, 0u);
                        tc_mma_i8(tmem + buf * TC_BN, tc_desc(st + TC_A_OFF + kb * TC_TILE), tc_desc(st + TC_B_OFF + kb * TC_TILE), idesc, 1u);
                        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                         smem_u32(&acc_full[buf]))
                                     : "memory");
                    }
                }
            }
        } else {
            // =============================== producers ======================================
            // Tasks of a stage: t < 128 is weight row t, t >= 128 is activation column t - 128;
            // this thread takes t = pt0, pt0 + 96 and pt0 + 192 (< 256).  Every branch is warp-uniform.
            const int pt0 = tid - TC_PROD_WARP0 * 32;  // 0..95
            const bool has_w1 = pt0 < 32;               // second weight row pt0 + 96
            const bool has_xa = pt0 >= 32;              // activation column pt0 - 32
            const bool has_xb = pt0 < 64;               // activation column pt0 + 64
            const int col_a = pt0 - 32, col_b = pt0 + 64;
            // rows / columns past the end are clamped: their results are never stored
            const uint8_t *w0p = p.w + min(n0 + pt0, p.N - 1) * (int64_t)p.row_bytes;
            const uint8_t *w1p = p.w + min(n0 + pt0 + 96, p.N - 1) * (int64_t)p.row_bytes;
            const int64_t m_a = min(m0 + col_a, p.M - 1), m_b = min(m0 + col_b, p.M - 1);
            uint2 wv0[9], wv1[9];
            uint4 ds_a = make_uint4(0u, 0u, 0u, 0u), ds_b = make_uint4(0u, 0u, 0u, 0u);
            const uint8_t *xb_a = nullptr, *xb_b = nullptr;
            auto load_chunk = [&](int c) {  // global -> registers, one stage ahead of its use
#pragma unroll
                for (int i = 0; i < 9; ++i) wv0[i] = __ldg(reinterpret_cast<const uint2 *>(w0p + (size_t)c * (TC_KB * Q4_BYTES)) + i);
                if (has_w1) {
#pragma unroll
                    for (int i = 0; i < 9; ++i) wv1[i] = __ldg(reinterpret_cast<const uint2 *>(w1p + (size_t)c * (TC_KB * Q4_BYTES)) + i);
                }
                if (has_xa) {
                    xb_a = p.xq + q8_block_index(c, m_a, p.n_super, p.M, p.order) * Q8_BYTES;
                    ds_a = __ldg(reinterpret_cast<const uint4 *>(xb_a));
                }
                if (has_xb) {
                    xb_b = p.xq + q8_block_index(c, m_b, p.n_super, p.M, p.order) * Q8_BYTES;
                    ds_b = __ldg(reinterpret_cast<const uint4 *>(xb_b));
                }
            };
            load_chunk(0);
            bool dead = false;
            for (int c = 0; c <= n_chunks; ++c) {  // one extra iteration publishes the last stage
                if (c < n_chunks) {
                    const int s = c % TC_STAGES;
                    if (c >= TC_STAGES && !mbar_wait_bounded(&stage_empty[s], (uint32_t)(c / TC_STAGES - 1) & 1u, p.fault)) {
                        dead = true;
                        break;
                    }
                    const uint32_t st = sbase + s * TC_STAGE_BYTES;
                    if (has_xa) tc_stage_activation_col(st, col_a, xb_a, ds_a);
                    if (has_xb) tc_stage_activation_col(st, col_b, xb_b, ds_b);
                    tc_unpack_weight_row(st, pt0, wv0);
                    if (has_w1) tc_unpack_weight_row(st, pt0 + 96, wv1);
                    if (c + 1 < n_chunks) load_chunk(c + 1);
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
                if (c >= 1) {
                    // stage c-1: its copies (all but the newest group) have landed, its stores are older still
                    asm volatile("cp.async.wait_group 1;" ::: "memory");
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // tiles are read by the tensor core
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&stage_full[(c - 1) % TC_STAGES]);
                    if (lane == 0 && ((c - 1) * TC_KB) < 128) tc_stamp(p, (c - 1) * TC_KB, 3, 1 + warp - TC_PROD_WARP0);
                }
            }
            if (dead) asm volatile("cp.async.wait_all;" ::: "memory");
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
    if (K % (TC_KB * QK) != 0) return set_error(JQ_ERR_UNSUPPORTED, "tcgen05 GEMM needs K %% 128 == 0 (K = %lld)", (long long)K);
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
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void *>(gemm_q4_0_q8_1_tc_kernel), TC_SMEM_BYTES)) return rc;
    (void)cudaGetLastError();  // a stale error of an earlier, unrelated call must not be taken for this launch's
    gemm_q4_0_q8_1_tc_kernel<<<dim3((unsigned)gx, (unsigned)gy), TC_THREADS, TC_SMEM_BYTES, st>>>(p);
    JQ_CUDA_TRY(cudaGetLastError());
    return JQ_OK;
}

}  // namespace jq
