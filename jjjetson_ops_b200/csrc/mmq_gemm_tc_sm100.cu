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
//   warp 8      allocates TMEM; one thread issues the MMAs: per 32-wide block a bias MMA and one
//               128 x 128 x 32 tcgen05.mma.kind::i8 (A = activations, s8; B = weight nibbles, u8)
//               into one of three accumulator buffers, then tcgen05.commit onto an mbarrier.
//   warp 9      one thread issues the tiled tensor copies (cp.async.bulk.tensor, no multicast).  K advances in
//               stages of 128 values (one Q8_1 super-block, four Q4_0 blocks).  The activations' int8 values
//               go straight into the tensor core's operand layout: eight copies of 16 bytes x 128 columns per
//               stage, each landing as one 2 KB slab of core matrices (8 columns x 16 bytes), so no thread ever
//               touches them; one more copy brings the 128 block headers (scales).  The weights come as raw
//               bytes, 144 bytes of each of the 128 rows per two stages.
//   warps 10-13 conversion.  Thread r splits the nibbles of weight row r (72 raw bytes per stage) into four
//               int8 tiles in the canonical K-major layout (8-row x 16-byte core matrices) and writes the fp32
//               table of d4 and the row's fp16 zero-point operand.
//   warps 14-15 from the headers of two activation columns per thread: the (d8, bias correction) table and
//               the columns' zero-point operands.
//               (Earlier the producers loaded "their" row per thread from global memory: a warp-wide load of
//               32 rows touches 32 cache lines, and those loads cost more than conversion and MMAs together.)
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
constexpr int TC_STAGES = 3;
constexpr int TC_A_OFF = 0;                        // activations: 8 slabs [128 columns][16 bytes], slab c = values 16c..16c+15
constexpr int TC_A_SLAB = 128 * 16;                //   (block j = slabs 2j, 2j+1: K-chunks 2048 bytes apart, 8-column groups 128)
constexpr int TC_B_OFF = TC_KB * TC_TILE;          // weights:     TC_KB tiles
constexpr int TC_ZA_OFF = 2 * TC_KB * TC_TILE;     // fp16 s8[128 columns][16] (4 blocks + 12 zeros), canonical layout
constexpr int TC_ZB_OFF = TC_ZA_OFF + TC_TILE;     // fp16 -8*d4[128 rows][16], canonical layout
constexpr int TC_D4_OFF = TC_ZB_OFF + TC_TILE;     // float (d4 * 2^49)[TC_KB][128]
constexpr int TC_XS_OFF = TC_D4_OFF + TC_KB * 128 * 4;   // float2 (d8 * 2^100, -2^17 * d8 * 2^-49)[TC_KB][128]
constexpr int TC_XH_OFF = TC_XS_OFF + TC_KB * 128 * 8;   // raw block headers [128 columns][16 bytes] as copied
constexpr int TC_STAGE_BYTES = TC_XH_OFF + 128 * 16;
constexpr int TC_X_TX_BYTES = 8 * TC_A_SLAB + 128 * 16;  // bytes the copies of one stage's activations deliver
constexpr int TC_RAWW_SLOTS = 2;                          // raw weights: 128 rows x 144 bytes = two stages per slot
constexpr int TC_RAWW_SLOT_BYTES = 128 * Q8_BYTES;
constexpr int TC_W_CHUNK = TC_KB * Q4_BYTES;              // 72 bytes of a weight row per stage
static_assert(2 * TC_W_CHUNK == Q8_BYTES, "a weight slot is two stages of 72 bytes per row");
constexpr int TC_RAWW_OFF = TC_STAGES * TC_STAGE_BYTES;
constexpr int TC_BIAS_OFF = TC_RAWW_OFF + TC_RAWW_SLOTS * TC_RAWW_SLOT_BYTES;   // one operand tile with every byte = TC_BIAS_BYTE
constexpr int TC_BAR_OFF = TC_BIAS_OFF + TC_TILE;
constexpr int TC_SMEM_BYTES = TC_BAR_OFF + 256;
static_assert(TC_STAGE_BYTES % 128 == 0 && TC_RAWW_OFF % 128 == 0, "tensor copies land on 128-byte boundaries");
static_assert(TC_SMEM_BYTES <= 227 * 1024, "stages do not fit in shared memory");
constexpr int TC_DRAIN_WARPS = 8;
constexpr int TC_MMA_WARP = 8;
constexpr int TC_COPY_WARP = 9;
constexpr int TC_CONV_WARP0 = 10;
constexpr int TC_CONV_WARPS = 4;                   // weight rows: one per thread
constexpr int TC_HDR_WARP0 = TC_CONV_WARP0 + TC_CONV_WARPS;
constexpr int TC_HDR_WARPS = 2;                    // activation headers: two columns per thread
constexpr int TC_THREADS = (TC_HDR_WARP0 + TC_HDR_WARPS) * 32;   // 512: four warps on each of the SM's four schedulers
// Registers per thread after setmaxnreg.  A CTA of 512 threads starts with 128 registers per thread, and the
// register file is one quarter per scheduler: warp w lives on scheduler w % 4, so each scheduler holds two drain
// warps and two of the others and has 4 x 128 registers per lane to hand out.  The two settings must stay within
// that, or the drain warps' setmaxnreg.inc never returns.
constexpr int TC_DRAIN_REGS = 208;
constexpr int TC_OTHER_REGS = 48;
static_assert(TC_DRAIN_WARPS == 8 && TC_THREADS == 512 && 2 * TC_DRAIN_REGS + 2 * TC_OTHER_REGS <= 4 * 128,
              "setmaxnreg budget exceeds a scheduler's share of the CTA's allocation");
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
#ifdef JQ_BOUNDS_CHECK
    Extent ext_y;  // range-checked debug build (the operand loads are tensor copies: their maps bound them)
#endif
    int64_t N, M;
    int K, order, n_super;
    uint32_t row_bytes;
    unsigned long long *trace;  // tracing aid (or nullptr): SM clock stamps of CTA (0,0), 512 rows of 8
};

// Tracing aid.  Rows 0-127: per block, when each drain warp saw the accumulator complete; rows
// 128-255: when it had added the previous block; rows 256-383: when it handed the buffer back;
// rows 384-511: column 0 = when the MMA of the block was issued, columns 1-4 = when each conversion
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

// One activation column of a stage: its block header (four (d, s) pairs, already in registers) becomes the
// drain's table and the fp16 zero-point operand.  The int8 values themselves were placed by the copy engine.
__device__ __forceinline__ void tc_stage_activation_header(uint32_t st, int r, uint4 ds) {
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

__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_q4_0_q8_1_tc_kernel(const TcParams p, const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + TC_BAR_OFF);
    uint64_t *stage_full = bars;                          // [TC_STAGES] conversion warps -> MMA warp and drain warps
    uint64_t *stage_empty = bars + TC_STAGES;             // [TC_STAGES] drain warps -> copy warp (and, through it, conversion)
    uint64_t *acc_full = bars + 2 * TC_STAGES;            // [TC_ACC_BUFS] MMA completion -> drain warps
    uint64_t *acc_empty = acc_full + TC_ACC_BUFS;         // [TC_ACC_BUFS] drain warps (buffer read out) -> MMA warp
    uint64_t *x_full = acc_empty + TC_ACC_BUFS;           // [TC_STAGES] copy engine (activation slabs + headers) -> conversion, MMA
    uint64_t *raww_full = x_full + TC_STAGES;             // [TC_RAWW_SLOTS] copy engine -> conversion warps
    uint64_t *raww_empty = raww_full + TC_RAWW_SLOTS;     // [TC_RAWW_SLOTS] conversion warps -> copy warp
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(raww_empty + TC_RAWW_SLOTS);
    static_assert((3 * TC_STAGES + 2 * TC_ACC_BUFS + 2 * TC_RAWW_SLOTS) * 8 + 4 <= 256, "barrier block too small");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t n0 = (int64_t)blockIdx.x * TC_BN, m0 = (int64_t)blockIdx.y * TC_BM;
    const int n_chunks = p.K / (TC_KB * QK);

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(&stage_full[s], TC_CONV_WARPS + TC_HDR_WARPS);
            mbar_init(&stage_empty[s], TC_DRAIN_WARPS);
            mbar_init(&x_full[s], 1);
        }
        for (int i = 0; i < TC_RAWW_SLOTS; ++i) {
            mbar_init(&raww_full[i], 1);
            mbar_init(&raww_empty[i], TC_CONV_WARPS);
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
#ifdef JQ_BOUNDS_CHECK
            const int64_t n_row = p.N - (n0 + half * 64) < 64 ? p.N - (n0 + half * 64) : 64;  // outputs of this lane's row
            const bool y_ok = m >= p.M || n_row <= 0 || in_extent(p.ext_y, p.y + m * p.N + n0 + half * 64, (unsigned long long)n_row * sizeof(float), p.fault);
#else
            const bool y_ok = true;
#endif
            if (m < p.M && y_ok) {
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
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(TC_OTHER_REGS));
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
                    const uint32_t par = (uint32_t)(c / TC_STAGES) & 1u;
                    // the conversion warps' tiles and tables, and the activation slabs the copy engine placed
                    if (!mbar_wait_bounded(&stage_full[s], par, p.fault) || !mbar_wait_bounded(&x_full[s], par, p.fault)) break;
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
                        tc_mma_i8(tmem + buf * TC_BN, tc_desc_strided(st + TC_A_OFF + kb * 2 * TC_A_SLAB, TC_A_SLAB, 128u),
                                  tc_desc(st + TC_B_OFF + kb * TC_TILE), idesc, 1u);
                        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                         smem_u32(&acc_full[buf]))
                                     : "memory");
                    }
                }
            }
        } else if (warp == TC_COPY_WARP) {
            // =============================== copy warp ======================================
            // One thread keeps the rings filled.  Activations of stage c: slab i (the 16 values 16 i .. 16 i + 15 of the
            // stage for all 128 columns) is one box of 16 bytes x 128 rows at byte 16 + 16 i of the columns' block;
            // the headers are the box at byte 0.  Weights: 144 bytes of each of the 128 rows per two stages.
            if (lane == 0) {
                for (int c = 0; c < n_chunks; ++c) {
                    const int s = c % TC_STAGES;
                    if ((c & 1) == 0) {
                        const int pair = c >> 1, ws = pair % TC_RAWW_SLOTS;
                        if (pair >= TC_RAWW_SLOTS && !mbar_wait_bounded(&raww_empty[ws], (uint32_t)(pair / TC_RAWW_SLOTS - 1) & 1u, p.fault)) break;
                        mbar_arrive_expect_tx(&raww_full[ws], TC_RAWW_SLOT_BYTES);
                        tma_load_2d(sbase + TC_RAWW_OFF + ws * TC_RAWW_SLOT_BYTES, &w_map, pair * Q8_BYTES, (int)n0, &raww_full[ws]);
                    }
                    // the slot's previous tiles have been multiplied and its tables read
                    if (c >= TC_STAGES && !mbar_wait_bounded(&stage_empty[s], (uint32_t)(c / TC_STAGES - 1) & 1u, p.fault)) break;
                    const uint32_t st = sbase + s * TC_STAGE_BYTES;
                    mbar_arrive_expect_tx(&x_full[s], TC_X_TX_BYTES);
                    // JQ_ORDER_KSUPER_COL: the tensor is [n_super * M blocks][144 bytes]; else [M columns][n_super * 144 bytes]
                    const int bx = p.order == JQ_ORDER_KSUPER_COL ? 0 : c * Q8_BYTES;
                    const int by = p.order == JQ_ORDER_KSUPER_COL ? (int)((int64_t)c * p.M + m0) : (int)m0;
                    tma_load_2d(st + TC_XH_OFF, &x_map, bx, by, &x_full[s]);
#pragma unroll
                    for (int i = 0; i < 8; ++i) tma_load_2d(st + TC_A_OFF + i * TC_A_SLAB, &x_map, bx + Q8_QS_OFFSET + 16 * i, by, &x_full[s]);
                }
            }
        } else {
            // =============================== conversion warps ===============================
            // Seeing a stage's activation copies complete also means its slot is free: the copy warp issued them only
            // after the drain warps had handed the slot back.
            const bool weights = warp < TC_HDR_WARP0;
            const int r = weights ? tid - TC_CONV_WARP0 * 32 : tid - TC_HDR_WARP0 * 32;  // weight row 0..127 / column pair 0..63
            for (int c = 0; c < n_chunks; ++c) {
                const int s = c % TC_STAGES, ws = (c >> 1) % TC_RAWW_SLOTS;
                bool ok = mbar_wait_bounded(&x_full[s], (uint32_t)(c / TC_STAGES) & 1u, p.fault);
                if (weights) ok = ok && mbar_wait_bounded(&raww_full[ws], (uint32_t)((c >> 1) / TC_RAWW_SLOTS) & 1u, p.fault);
                if (!__all_sync(0xFFFFFFFFu, ok)) break;
                const uint32_t st = sbase + s * TC_STAGE_BYTES;
                if (weights) {
                    const uint32_t raw = sbase + TC_RAWW_OFF + ws * TC_RAWW_SLOT_BYTES + r * Q8_BYTES + (c & 1) * TC_W_CHUNK;
                    uint2 wv[9];
#pragma unroll
                    for (int i = 0; i < 9; ++i) wv[i] = lds_v2(raw + i * 8);
                    tc_unpack_weight_row(st, r, wv);
                } else {
                    tc_stage_activation_header(st, r, lds_v4(st + TC_XH_OFF + r * 16));
                    tc_stage_activation_header(st, r + 64, lds_v4(st + TC_XH_OFF + (r + 64) * 16));
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // tiles are read by the tensor core
                __syncwarp();
                if (lane == 0) {
                    if (weights && (c & 1)) mbar_arrive(&raww_empty[ws]);  // both halves of the slot have been read
                    mbar_arrive(&stage_full[s]);
                    if (weights && (c * TC_KB) < 128) tc_stamp(p, c * TC_KB, 3, 1 + warp - TC_CONV_WARP0);
                }
            }
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
    // a weight row's pitch, K / 32 * 18 bytes, must be a multiple of 16 for the tensor copies
    if (K % (2 * SUPER) != 0) return set_error(JQ_ERR_UNSUPPORTED, "tcgen05 GEMM needs K %% 256 == 0 (K = %lld)", (long long)K);
    if (((uintptr_t)d_w & 15u) != 0 || ((uintptr_t)d_xq & 15u) != 0)
        return set_error(JQ_ERR_UNSUPPORTED, "tcgen05 GEMM needs 16-byte aligned operands");
    if (N == 0 || M == 0) return JQ_OK;
    DeviceCaps caps;
    if (int rc = device_caps(&caps)) return rc;
    if (caps.cc / 10 != 10) return set_error(JQ_ERR_UNSUPPORTED, "tcgen05 needs an sm_100-class device");
    const int64_t gx = (N + TC_BN - 1) / TC_BN, gy = (M + TC_BM - 1) / TC_BM;
    if (gy > 65535 || K > (1 << 24) || (K / SUPER) * M >= ((int64_t)1 << 31) || N >= ((int64_t)1 << 31))
        return set_error(JQ_ERR_UNSUPPORTED, "shape too large for the tcgen05 GEMM");
    TcParams p{};
    p.w = static_cast<const uint8_t *>(d_w);
    p.xq = static_cast<const uint8_t *>(d_xq);
    p.y = d_y;
    p.fault = device_fault_ptr();
#ifdef JQ_BOUNDS_CHECK
    p.ext_y = make_extent(d_y, (unsigned long long)M * (unsigned long long)N * sizeof(float));
#endif
    p.N = N;
    p.M = M;
    p.K = (int)K;
    p.order = order;
    p.n_super = (int)(K / SUPER);
    p.row_bytes = (uint32_t)(K / QK * Q4_BYTES);
    p.trace = static_cast<unsigned long long *>(next_trace_slot());
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void *>(gemm_q4_0_q8_1_tc_kernel), TC_SMEM_BYTES)) return rc;
    (void)cudaGetLastError();  // a stale error of an earlier, unrelated call must not be taken for this launch's
    CUtensorMap w_map, x_map;
    if (int rc = encode_byte_map(&w_map, d_w, p.row_bytes, (uint64_t)N, p.row_bytes, Q8_BYTES, 128)) return rc;
    const uint64_t x_row = (uint64_t)p.n_super * Q8_BYTES;
    if (int rc = order == JQ_ORDER_KSUPER_COL ? encode_byte_map(&x_map, d_xq, Q8_BYTES, (uint64_t)p.n_super * (uint64_t)M, Q8_BYTES, 16, 128)
                                              : encode_byte_map(&x_map, d_xq, x_row, (uint64_t)M, x_row, 16, 128))
        return rc;
    gemm_q4_0_q8_1_tc_kernel<<<dim3((unsigned)gx, (unsigned)gy), TC_THREADS, TC_SMEM_BYTES, st>>>(p, w_map, x_map);
    JQ_CUDA_TRY(cudaGetLastError());
    return JQ_OK;
}

}  // namespace jq
