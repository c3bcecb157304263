// Prefill-regime multiply with the block scales folded into the operands: both matrices are
// dequantised to fp16 on their way to the tensor core and multiplied by tcgen05.mma.kind::f16 with
// fp32 accumulation in tensor memory, so nothing is drained or rescaled between blocks.
//
// Work to replace: q4_0_q8_1_mat_mul_kernel (reference src/cuda/mm_q4_0_q8_1.cu:164-289) for large
// batches.  The reference adds, per 32-wide block, d4 * (sumi * d8 - 8 * s8) (mm_q4_0_q8_1.cu:92).
// With sumi = sum(q4 * q8) that is
//     sum_i ((q4_i - 8) * d4) * (q8_i * d8)   +   (-8 * d4) * (s8 - d8 * sum_i q8_i)
// The first term is a plain product of two fp16 matrices B[n][k] = (q4 - 8) * d4 and
// A[m][k] = q8 * d8; the second is rank one per block and joins the same accumulator as one more
// MMA per 128 values of K (operands s8 - d8 * sum(q8), computed in fp32, and -8 * d4, exact).  It
// vanishes up to the rounding of s8 when the quantizer stored s = d * sum(q), and carries the
// quantisation residue when it stored the sum of the unquantised values.
//
// Precision.  q4 - 8 and q8 are exact in fp16; their products with the fp16 scales are rounded once
// to fp16 (relative error <= 2^-11 per element), the accumulation is fp32.  The result differs from
// the reference formula by about 3e-4 of the largest output on the configurations this kernel is
// measured on, where the integer kernels differ by 1e-6: it meets the 1e-3 bound against the
// dequantised product but not bit-level parity of the per-block sums, which is why it is selected
// by name only.  Operands must stay inside fp16's range: |x| <= 65504 for the activations, and
// scales whose products are not subnormal (|d| * |q| >= 6.1e-5) keep full precision.
//
// A CTA owns a 128 (activation columns) x 128 (weight rows) tile of Y.  K advances in stages of 128
// values (one Q8_1 block per column, four Q4_0 blocks per row) through three rings:
//   raw rings       the quantized bytes as they lie in global memory, brought in by the copy engine:
//                   one tiled tensor copy per stage for the 128 activation blocks (128 rows x 144
//                   bytes), one per two stages for 144 bytes of each of the 128 weight rows.  A
//                   per-thread load of "its" row touches 32 cache lines per warp instruction and
//                   was measured to cost more than the conversion and the MMAs together.
//   operand ring    three stages.  Weights: eight 128 x 16 fp16 tiles in shared memory in the tensor
//                   core's canonical K-major layout.  Activations: tensor memory, lane = activation
//                   column, 64 columns holding the 128 values of K in order; the MMA reads its A
//                   operand from there, which halves the shared-memory traffic of a stage.
// Warps:
//   0-15   two groups of eight that take the stages in turn, so that one group's waits are covered
//          by the other's work.  In a group, four warps convert one weight row per thread (nibbles
//          become fp16 by the magic-number trick: 0x6400 | q is 1024 + q; then one exact subtraction
//          and one rounded multiplication by the scale) and four warps one activation column per
//          thread (int8 the same way; the 64 packed words go to tensor memory with tcgen05.st).
//   16     allocates tensor memory; one thread issues, per stage, the rank-one MMA and eight
//          128 x 128 x 16 MMAs, and tcgen05.commit hands the stage back to the producers.
//   17     one thread issues the tensor copies.
// After the last stage the sixteen producer warps read the 128 x 128 fp32 accumulator, turn it
// around in shared memory and store 128 contiguous bytes of an output row per instruction.
// Every mbarrier wait is a bounded poll; a wait that runs out sets the device fault word, and every
// warp still reaches the common exit where tensor memory is released.
#include "tc_common.cuh"

namespace jq {

namespace {

constexpr int HF_BM = 128;    // activation columns per CTA (MMA M, TMEM lanes)
constexpr int HF_BN = 128;    // weight rows per CTA (MMA N, TMEM columns)
constexpr int HF_KT = 8;      // operand tiles of 16 values of K per stage
constexpr int HF_STAGES = 3;  // fp16 operand stages: weights in shared memory, activations in tensor memory
constexpr int HF_B_OFF = 0;                           // weights: HF_KT tiles
constexpr int HF_ZA_OFF = HF_KT * TC_TILE;            // fp16 (s8 - d8 * sum q8)[128 columns][16] (4 blocks + 12 zeros)
constexpr int HF_ZB_OFF = HF_ZA_OFF + TC_TILE;        // fp16 (-8 * d4)[128 rows][16]
constexpr int HF_STAGE_BYTES = HF_ZB_OFF + TC_TILE;
// Rings of quantized bytes as they lie in global memory, filled by the copy engine (one tensor copy each):
// activations, one stage per slot: 128 blocks of 144 bytes; weights, two stages per slot: 128 rows x 144 bytes
constexpr int HF_RAWX_SLOTS = 3, HF_RAWW_SLOTS = 2;
constexpr int HF_W_CHUNK = 4 * Q4_BYTES;              // 72 bytes of a weight row per stage
constexpr int HF_RAW_SLOT_BYTES = 128 * Q8_BYTES;     // 18432, both rings
static_assert(2 * HF_W_CHUNK == Q8_BYTES, "a weight slot is two stages of 72 bytes per row");
constexpr int HF_RAWX_OFF = HF_STAGES * HF_STAGE_BYTES;
constexpr int HF_RAWW_OFF = HF_RAWX_OFF + HF_RAWX_SLOTS * HF_RAW_SLOT_BYTES;
constexpr int HF_BAR_OFF = HF_RAWW_OFF + HF_RAWW_SLOTS * HF_RAW_SLOT_BYTES;
constexpr int HF_SMEM_BYTES = HF_BAR_OFF + 256;
static_assert(HF_RAWX_OFF % 128 == 0 && HF_RAW_SLOT_BYTES % 128 == 0, "tensor copies land on 128-byte boundaries");
constexpr int HF_OUT_PITCH = 33;                      // words per row of a warp's 32 x 32 output staging block
constexpr int HF_GROUPS = 2;        // producer groups of 8 warps; group g converts the stages c with c % 2 == g
constexpr int HF_GROUP_WARPS = 8;
constexpr int HF_PROD_WARPS = HF_GROUPS * HF_GROUP_WARPS;
constexpr int HF_MMA_WARP = HF_PROD_WARPS;
constexpr int HF_COPY_WARP = HF_PROD_WARPS + 1;
constexpr int HF_THREADS = (HF_PROD_WARPS + 2) * 32;
static_assert(HF_RAWX_SLOTS == HF_STAGES, "stage c uses slot c % 3 of both the operand ring and the activation ring");
// Tensor memory: the fp32 accumulator in columns 0..127, then per stage the activation operand: lane = activation
// column, 64 columns of two fp16 values = the 128 values of K in order
constexpr uint32_t HF_TMEM_A_COL = 128, HF_TMEM_A_STAGE_COLS = 64;
constexpr uint32_t HF_TMEM_COLS = 512;
static_assert(HF_TMEM_A_COL + HF_STAGES * HF_TMEM_A_STAGE_COLS <= HF_TMEM_COLS, "tensor memory too small");
static_assert(HF_SMEM_BYTES <= 227 * 1024, "stages do not fit in shared memory");
static_assert(HF_PROD_WARPS * 32 * HF_OUT_PITCH * 4 <= HF_STAGES * HF_STAGE_BYTES, "output staging does not fit in the operand stages");

// fp16 constants, two per word
constexpr uint32_t H2_MAGIC_BYTES = 0x64646464u;  // high byte of 1024 + v for an 8-bit v
constexpr uint32_t H2_LOW_NIBBLE = 0x640F640Fu;   // keeps 1024 + (v & 15)
constexpr uint32_t H2_HIGH_NIBBLE = 0x64F064F0u;  // keeps 1024 + 16 * (v >> 4)
constexpr uint32_t H2_1032 = 0x64086408u;
constexpr uint32_t H2_1152 = 0x64806480u;
constexpr uint32_t H2_SIXTEENTH = 0x2C002C00u;
constexpr uint32_t H2_MINUS_72 = 0xD480D480u;

struct HfParams {
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
    unsigned long long *trace;  // tracing aid (or nullptr): SM clock stamps of CTA (0,0), rows of 8
    // Split K (few output tiles, long K): blockIdx.z takes the 128-value chunks [z * chunks_per_split, ...) and the
    // splits of a tile add their partial results to y in the order of z (so the sum is formed the same way every
    // time): tile_sem[tile] counts the epilogue warps that have finished, split z goes ahead at 16 * z, the last
    // warp of the last split puts the count back to zero.
    int k_splits, chunks_per_split;
    int *tile_sem;
    uint32_t poll_limit;
    int static_weights;  // the weight copies may start before the previous kernel in the stream has finished
};

// Counts of finished epilogue warps per output tile (split K); zero between launches.  Part of the library image, like
// the fault word: launches that split K must not overlap on one device (they do not on one stream).
constexpr int HF_MAX_SPLIT_TILES = 128;
__device__ int g_tile_sem[HF_MAX_SPLIT_TILES];

// Tracing aid.  Row c (stage, < 64) of block `who`: 0 = weight warp 0, 1 = activation warp 4, 2 = the MMA thread.
// Producer columns: 0 loop top, 1 past the barrier, 2 copies of stage c + 2 issued, 3 operand stage free,
// 4 converted, 5 published.  MMA columns: 0 stage seen full, 1 MMAs and commit issued.
__device__ __forceinline__ void hf_stamp(const HfParams &p, int who, int c, int slot) {
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && c < 64) {
        p.trace[((who * 64 + c) * 8) + slot] = (unsigned long long)clock64();
    }
}

// registers -> 32 lanes x 32 consecutive 32-bit columns of tensor memory (completion: tcgen05.wait::st)
__device__ __forceinline__ void tmem_st32_nowait(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}

// D(fp32, TMEM) (+)= A(fp16, TMEM: lane = row, two values of K per column) x B(fp16 tile in shared memory)^T, K = 16
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ __half2 as_h2(uint32_t v) { return *reinterpret_cast<const __half2 *>(&v); }
__device__ __forceinline__ uint32_t as_u32(__half2 v) { return *reinterpret_cast<const uint32_t *>(&v); }

// (v - offset) * scale: the subtraction is exact, the product is rounded once
__device__ __forceinline__ uint32_t h2_sub_scale(uint32_t v, uint32_t offset, __half2 scale) {
    return as_u32(__hmul2(__hsub2(as_h2(v), as_h2(offset)), scale));
}
// (v / 16 - 72) * scale for v = 1024 + 16 * q: the fma is exact (q - 8), the product is rounded once
__device__ __forceinline__ uint32_t h2_high_scale(uint32_t v, __half2 scale) {
    return as_u32(__hmul2(__hfma2(as_h2(v), as_h2(H2_SIXTEENTH), as_h2(H2_MINUS_72)), scale));
}

// One weight row of a stage (72 bytes = 18 words in registers) -> its 128 values (q4 - 8) * d4 in
// the eight weight tiles, and the row of the rank-one operand.
__device__ __forceinline__ void hf_convert_weight_row(uint32_t st, int r, const uint2 (&wv)[9]) {
    const uint32_t *ww = reinterpret_cast<const uint32_t *>(wv);
    uint32_t zb[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
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
        zb[j] = dbits;
        const __half2 d2 = as_h2(dbits | (dbits << 16));
        // byte i of the block holds value i (low nibble) and value i + 16 (high nibble): the low nibbles
        // fill tile 2j, the high nibbles tile 2j + 1; bytes 0-7 are K-chunk 0 of a tile, bytes 8-15 chunk 1
        const uint32_t tile_lo = st + HF_B_OFF + (2 * j) * TC_TILE, tile_hi = tile_lo + TC_TILE;
#pragma unroll
        for (int kc = 0; kc < 2; ++kc) {
            uint32_t lo[4], hi[4];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const uint32_t p01 = __byte_perm(q[2 * kc + t], H2_MAGIC_BYTES, 0x4140);  // 1024 + byte 0 | 1024 + byte 1
                const uint32_t p23 = __byte_perm(q[2 * kc + t], H2_MAGIC_BYTES, 0x4342);
                lo[2 * t] = h2_sub_scale(p01 & H2_LOW_NIBBLE, H2_1032, d2);
                lo[2 * t + 1] = h2_sub_scale(p23 & H2_LOW_NIBBLE, H2_1032, d2);
                hi[2 * t] = h2_high_scale(p01 & H2_HIGH_NIBBLE, d2);
                hi[2 * t + 1] = h2_high_scale(p23 & H2_HIGH_NIBBLE, d2);
            }
            sts_v4(tile_lo + tile_off(r, kc), make_uint4(lo[0], lo[1], lo[2], lo[3]));
            sts_v4(tile_hi + tile_off(r, kc), make_uint4(hi[0], hi[1], hi[2], hi[3]));
        }
    }
    // -8 * d4 as fp16 (exact: a power of two; finite unless |d4| > 8188); the 12 padding values stay zero
    const __half2 m8 = __float2half2_rn(-8.0f);
    sts_v4(st + HF_ZB_OFF + tile_off(r, 0),
           make_uint4(as_u32(__hmul2(as_h2(zb[0] | (zb[1] << 16)), m8)), as_u32(__hmul2(as_h2(zb[2] | (zb[3] << 16)), m8)), 0u, 0u));
}

// One activation column of a stage (a 144-byte block in registers) -> its 128 values q8 * d8, in K order, in the
// tensor-memory lane of the column (warp-collective: the 32 lanes are 32 neighbouring columns), and the column of
// the rank-one operand in shared memory.
__device__ __forceinline__ void hf_convert_activation_col(uint32_t st, int r, const uint4 (&xv)[9], uint32_t taddr) {
    const uint32_t dsw[4] = {xv[0].x, xv[0].y, xv[0].z, xv[0].w};
    float zc[4];
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {  // 64 values of K = 32 columns of tensor memory at a time
        uint32_t o[32];
#pragma unroll
        for (int j2 = 0; j2 < 2; ++j2) {
            const int j = 2 * jj + j2;
            const uint32_t dbits = dsw[j] & 0xFFFFu;
            const __half2 d2 = as_h2(dbits | (dbits << 16));
            int isum = 0;
#pragma unroll
            for (int h = 0; h < 2; ++h) {  // values 16h .. 16h + 15 of the block
                const uint4 v = xv[1 + 2 * j + h];
                const uint32_t wq[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    isum = __dp4a((int)wq[t], 0x01010101, isum);
                    const uint32_t wu = wq[t] ^ 0x80808080u;  // q + 128 in 1..255
                    o[j2 * 16 + h * 8 + 2 * t] = h2_sub_scale(__byte_perm(wu, H2_MAGIC_BYTES, 0x4140), H2_1152, d2);
                    o[j2 * 16 + h * 8 + 2 * t + 1] = h2_sub_scale(__byte_perm(wu, H2_MAGIC_BYTES, 0x4342), H2_1152, d2);
                }
            }
            // what the stored s differs by from d8 * sum(q8); d8 * isum is exact in fp32
            zc[j] = fmaf(-half_bits_to_float(dbits), (float)isum, half_bits_to_float(dsw[j] >> 16));
        }
        tmem_st32_nowait(taddr + jj * 32, o);
    }
    sts_v4(st + HF_ZA_OFF + tile_off(r, 0),
           make_uint4(as_u32(__floats2half2_rn(zc[0], zc[1])), as_u32(__floats2half2_rn(zc[2], zc[3])), 0u, 0u));
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__global__ void __launch_bounds__(HF_THREADS, 1)
gemm_q4_0_q8_1_f16_kernel(const HfParams p, const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + HF_BAR_OFF);
    uint64_t *stage_full = bars;                  // [HF_STAGES] producer warps -> MMA warp
    uint64_t *stage_empty = bars + HF_STAGES;     // [HF_STAGES] MMA completion -> producers
    uint64_t *acc_full = bars + 2 * HF_STAGES;    // all MMAs complete -> epilogue
    uint64_t *rawx_full = acc_full + 1;               // [HF_RAWX_SLOTS] copy engine -> activation warps
    uint64_t *rawx_empty = rawx_full + HF_RAWX_SLOTS; // [HF_RAWX_SLOTS] activation warps -> copy warp
    uint64_t *raww_full = rawx_empty + HF_RAWX_SLOTS; // [HF_RAWW_SLOTS] copy engine -> weight warps
    uint64_t *raww_empty = raww_full + HF_RAWW_SLOTS; // [HF_RAWW_SLOTS] weight warps -> copy warp
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(raww_empty + HF_RAWW_SLOTS);
    static_assert((2 * HF_STAGES + 1 + 2 * HF_RAWX_SLOTS + 2 * HF_RAWW_SLOTS) * 8 + 4 <= 256, "barrier block too small");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t n0 = (int64_t)blockIdx.x * HF_BN, m0 = (int64_t)blockIdx.y * HF_BM;
    // this CTA's chunks of K: c counts them from 0 (ring slots, parities), c0 + c is the chunk of the matrix (copies)
    const int c0 = (int)blockIdx.z * p.chunks_per_split;
    const int n_chunks = min(p.chunks_per_split, p.K / SUPER - c0);

    if (tid == 0) {
        for (int s = 0; s < HF_STAGES; ++s) {
            mbar_init(&stage_full[s], HF_GROUP_WARPS);
            mbar_init(&stage_empty[s], 1);
        }
        mbar_init(acc_full, 1);
        for (int i = 0; i < HF_RAWX_SLOTS; ++i) {
            mbar_init(&rawx_full[i], 1);
            mbar_init(&rawx_empty[i], 4);
        }
        for (int i = 0; i < HF_RAWW_SLOTS; ++i) {
            mbar_init(&raww_full[i], 1);
            mbar_init(&raww_empty[i], 4 * HF_GROUPS);  // the four weight warps of each group
        }
        fence_mbar_init();
    }
    if (tid < 128) {
        // the zero half (K = 8..15) of every stage's rank-one operands
        for (int s = 0; s < HF_STAGES; ++s) {
            sts_v4(sbase + s * HF_STAGE_BYTES + HF_ZA_OFF + tile_off(tid, 1), make_uint4(0u, 0u, 0u, 0u));
            sts_v4(sbase + s * HF_STAGE_BYTES + HF_ZB_OFF + tile_off(tid, 1), make_uint4(0u, 0u, 0u, 0u));
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // read by the tensor core
    }
    if (warp == HF_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(HF_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    // Programmatic dependent launch: everything above ran while the previous kernel (the activation quantizer, as a
    // rule) was still finishing; the activations are read, and the outputs written, only after it has.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp < HF_PROD_WARPS) {
        // =============================== producers, then epilogue ==============================
        // Two groups of eight warps take the stages in turn, so that one group's waits and conversion latencies are
        // covered by the other's work.  In a group, warps 0-3 convert one weight row per thread and warps 4-7 one
        // activation column per thread, from the raw rings the copy warp keeps filled.  All decisions are taken per
        // warp, so that aligned instructions stay convergent.
        const int group = warp / HF_GROUP_WARPS, gw = warp % HF_GROUP_WARPS;
        const bool is_w = gw < 4;
        const int row = (gw & 3) * 32 + lane;  // weight row or activation column inside the tile
        const bool stamps = lane == 0 && (gw & 3) == 0 && group == 0;
        bool alive = true;
#pragma unroll 1
        for (int c = group; c < n_chunks && alive; c += HF_GROUPS) {
            const int s = c % HF_STAGES;                   // slot of the operand ring and of the activation ring
            const uint32_t round = (uint32_t)(c / HF_STAGES);  // how often those rings have wrapped
            const int ws = (c >> 1) & 1;                   // weight slot of the stage pair
            if (stamps) hf_stamp(p, gw >> 2, c, 0);
            {
                const bool ok = is_w ? mbar_wait_bounded(&raww_full[ws], (uint32_t)(c >> 2) & 1u, p.fault)
                                     : mbar_wait_bounded(&rawx_full[s], round & 1u, p.fault);
                alive = __all_sync(0xFFFFFFFFu, ok) != 0;
            }
            if (stamps) hf_stamp(p, gw >> 2, c, 1);
            if (alive && round > 0) {
                const bool ok = mbar_wait_bounded(&stage_empty[s], (round - 1) & 1u, p.fault);
                alive = __all_sync(0xFFFFFFFFu, ok) != 0;
            }
            if (stamps) hf_stamp(p, gw >> 2, c, 3);
            if (alive) {
                const uint32_t st = sbase + s * HF_STAGE_BYTES;
                if (is_w) {
                    const uint32_t raw = sbase + HF_RAWW_OFF + ws * HF_RAW_SLOT_BYTES + row * Q8_BYTES + (c & 1) * HF_W_CHUNK;
                    uint2 v[9];
#pragma unroll
                    for (int i = 0; i < 9; ++i) v[i] = lds_v2(raw + i * 8);
                    hf_convert_weight_row(st, row, v);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&raww_empty[ws]);  // this warp's half of the slot has been read and used
                } else {
                    const uint32_t raw = sbase + HF_RAWX_OFF + s * HF_RAW_SLOT_BYTES + row * Q8_BYTES;
                    uint4 v[9];
#pragma unroll
                    for (int i = 0; i < 9; ++i) v[i] = lds_v4(raw + i * 16);
                    hf_convert_activation_col(st, row, v, tmem + ((uint32_t)((gw & 3) * 32) << 16) + HF_TMEM_A_COL + s * HF_TMEM_A_STAGE_COLS);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&rawx_empty[s]);
                    tc_fence_before();
                }
                if (stamps) hf_stamp(p, gw >> 2, c, 4);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // tiles are read by the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(&stage_full[s]);
                if (stamps) hf_stamp(p, gw >> 2, c, 5);
            }
        }

        // epilogue: warp w reads TMEM lanes 32 * (w % 4) .. (activation columns) and 32 of the 128 weight rows, and
        // turns the 32 x 32 block around in shared memory (the operand stages are free by now) so that a store
        // instruction writes 128 contiguous bytes of one output row
        if (alive && __all_sync(0xFFFFFFFFu, mbar_wait_bounded(acc_full, 0u, p.fault))) {
            tc_fence_after();
            asm volatile("griddepcontrol.wait;" ::: "memory");  // (long past: orders the stores to y after the previous kernel)
            const int cb = warp >> 2;  // which 32 of the 128 weight rows
            const uint32_t stage_blk = sbase + warp * (32 * HF_OUT_PITCH * 4);
            const int64_t m_first = m0 + (warp & 3) * 32;
            uint32_t v[32];
            tmem_ld32_nowait(tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(cb * 32), v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) sts_f32(stage_blk + (lane * HF_OUT_PITCH + j) * 4, __uint_as_float(v[j]));
            __syncwarp();
            const int64_t n = n0 + cb * 32 + lane;
            const int z = (int)blockIdx.z;
            int *sem = p.k_splits > 1 ? p.tile_sem + (blockIdx.y * gridDim.x + blockIdx.x) : nullptr;
            bool go = true;
            if (z > 0) {
                // the splits below this one have added their parts: all sixteen warps of each
                if (lane == 0) {
                    go = false;
                    for (uint32_t spin = 0; spin < p.poll_limit && !go; ++spin) {
                        int seen;
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(sem) : "memory");
                        go = seen >= HF_PROD_WARPS * z;
                    }
                    if (!go) report_fault(p.fault, 1);
                }
                go = __shfl_sync(0xFFFFFFFFu, go ? 1 : 0, 0) != 0;
                __threadfence();  // every lane's reads of y come after the count was seen
            }
            if (z > 0) {
                // all of this lane's partial sums of the earlier splits are requested before the first is used
                float prev[32];
#pragma unroll
                for (int rr = 0; rr < 32; ++rr) {
                    prev[rr] = 0.0f;
                    if (go && m_first + rr < p.M && n < p.N && JQ_IN_EXTENT(p.ext_y, p.y + (m_first + rr) * p.N + n, sizeof(float), p.fault))
                        prev[rr] = __ldcg(p.y + (m_first + rr) * p.N + n);
                }
#pragma unroll
                for (int rr = 0; rr < 32; ++rr) {
                    const float val = __uint_as_float(lds_u32(stage_blk + (rr * HF_OUT_PITCH + lane) * 4)) + prev[rr];
                    if (go && m_first + rr < p.M && n < p.N && JQ_IN_EXTENT(p.ext_y, p.y + (m_first + rr) * p.N + n, sizeof(float), p.fault))
                        p.y[(m_first + rr) * p.N + n] = val;
                }
            } else {
#pragma unroll 8
                for (int rr = 0; rr < 32; ++rr) {
                    const uint32_t val = lds_u32(stage_blk + (rr * HF_OUT_PITCH + lane) * 4);
                    if (m_first + rr < p.M && n < p.N && JQ_IN_EXTENT(p.ext_y, p.y + (m_first + rr) * p.N + n, sizeof(float), p.fault))
                        p.y[(m_first + rr) * p.N + n] = __uint_as_float(val);
                }
            }
            if (sem != nullptr) {
                __syncwarp();
                if (lane == 0) {
                    __threadfence();
                    const int before = atomicAdd(sem, 1);
                    if (before == HF_PROD_WARPS * p.k_splits - 1) atomicExch(sem, 0);  // the last warp of the last split re-arms the tile
                }
            }
        }
    } else if (warp == HF_COPY_WARP) {
        // =============================== copy warp =============================================
        // One thread keeps both raw rings filled: per stage one tensor copy of the 128 activation blocks, per pair
        // of stages one of 144 bytes of each of the 128 weight rows.
        if (lane == 0) {
            int xs = 0;
            uint32_t xround = 0;
            if (!p.static_weights) asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int c = 0; c < n_chunks; ++c) {
                if (c == 0 && p.static_weights) {
                    // the first pair of weight chunks is requested ahead of the wait for the previous kernel
                    mbar_arrive_expect_tx(&raww_full[0], HF_RAW_SLOT_BYTES);
                    tma_load_2d(sbase + HF_RAWW_OFF, &w_map, (c0 >> 1) * Q8_BYTES, (int)n0, &raww_full[0]);
                    asm volatile("griddepcontrol.wait;" ::: "memory");
                } else if ((c & 1) == 0) {
                    const int pair = c >> 1, ws = pair & 1;
                    if (pair >= HF_RAWW_SLOTS && !mbar_wait_bounded(&raww_empty[ws], (uint32_t)((pair >> 1) - 1) & 1u, p.fault)) break;
                    mbar_arrive_expect_tx(&raww_full[ws], HF_RAW_SLOT_BYTES);
                    tma_load_2d(sbase + HF_RAWW_OFF + ws * HF_RAW_SLOT_BYTES, &w_map, ((c0 + c) >> 1) * Q8_BYTES, (int)n0, &raww_full[ws]);
                }
                if (xround > 0 && !mbar_wait_bounded(&rawx_empty[xs], (xround - 1) & 1u, p.fault)) break;
                mbar_arrive_expect_tx(&rawx_full[xs], HF_RAW_SLOT_BYTES);
                if (p.order == JQ_ORDER_KSUPER_COL) {  // the tensor is [n_super * M blocks][144 bytes]
                    tma_load_2d(sbase + HF_RAWX_OFF + xs * HF_RAW_SLOT_BYTES, &x_map, 0, (int)((int64_t)(c0 + c) * p.M + m0), &rawx_full[xs]);
                } else {                               // the tensor is [M columns][n_super * 144 bytes]
                    tma_load_2d(sbase + HF_RAWX_OFF + xs * HF_RAW_SLOT_BYTES, &x_map, (c0 + c) * Q8_BYTES, (int)m0, &rawx_full[xs]);
                }
                if (++xs == HF_RAWX_SLOTS) {
                    xs = 0;
                    ++xround;
                }
            }
        }
    } else if (lane == 0) {
        // =============================== MMA issuer ============================================

        const uint32_t idesc = tc_idesc_f16(HF_BM, HF_BN);
        int s = 0;
        uint32_t parity = 0;
        bool alive = true;
        for (int c = 0; c < n_chunks; ++c) {
            if (!mbar_wait_bounded(&stage_full[s], parity, p.fault)) {
                alive = false;
                break;
            }
            const uint32_t st = sbase + s * HF_STAGE_BYTES;
            tc_fence_after();
            hf_stamp(p, 2, c, 0);
            tc_mma_f16(tmem, tc_desc(st + HF_ZA_OFF), tc_desc(st + HF_ZB_OFF), idesc, c > 0 ? 1u : 0u);
#pragma unroll
            for (int t = 0; t < HF_KT; ++t) {
                tc_mma_f16_ts(tmem, tmem + HF_TMEM_A_COL + s * HF_TMEM_A_STAGE_COLS + t * 8, tc_desc(st + HF_B_OFF + t * TC_TILE), idesc, 1u);
            }
            tc_commit(&stage_empty[s]);  // the stage may be overwritten once these MMAs have read it
            hf_stamp(p, 2, c, 1);
            if (++s == HF_STAGES) {
                s = 0;
                parity ^= 1u;
            }
        }
        if (alive) tc_commit(acc_full);
    }

    // common exit: nobody touches tensor memory any more, release it
    tc_fence_before();
    __syncthreads();
    if (warp == HF_MMA_WARP) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(HF_TMEM_COLS) : "memory");
    }
}

}  // namespace

int reset_gemm_f16_split_state() {
    void *sem = nullptr;
    JQ_CUDA_TRY(cudaGetSymbolAddress(&sem, g_tile_sem));
    JQ_CUDA_TRY(cudaMemset(sem, 0, sizeof(int) * HF_MAX_SPLIT_TILES));
    return JQ_OK;
}

int launch_gemm_f16(cudaStream_t st, const void *d_w, const void *d_xq, float *d_y, int64_t K, int64_t N, int64_t M,
                    int order) {
    // a weight row's pitch, K / 32 * 18 bytes, must be a multiple of 16 for the tensor copies
    if (K % (2 * SUPER) != 0) return set_error(JQ_ERR_UNSUPPORTED, "fp16-operand tcgen05 GEMM needs K %% 256 == 0 (K = %lld)", (long long)K);
    if (((uintptr_t)d_w & 15u) != 0 || ((uintptr_t)d_xq & 15u) != 0)
        return set_error(JQ_ERR_UNSUPPORTED, "fp16-operand tcgen05 GEMM needs 16-byte aligned operands");
    if (N == 0 || M == 0) return JQ_OK;
    DeviceCaps caps;
    if (int rc = device_caps(&caps)) return rc;
    if (caps.cc / 10 != 10) return set_error(JQ_ERR_UNSUPPORTED, "tcgen05 needs an sm_100-class device");
    const int64_t gx = (N + HF_BN - 1) / HF_BN, gy = (M + HF_BM - 1) / HF_BM;
    if (gy > 65535 || K > (1 << 24) || (K / SUPER) * M >= ((int64_t)1 << 31) || N >= ((int64_t)1 << 31))
        return set_error(JQ_ERR_UNSUPPORTED, "shape too large for the tcgen05 GEMM");
    HfParams p{};
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
    p.poll_limit = wait_poll_limit();
    p.static_weights = option_value(JQ_OPT_STATIC_WEIGHTS) != 0 ? 1 : 0;
    // Few tiles and a long K: two CTAs per tile, each half of K (whole pairs of chunks), so that twice as many SMs
    // convert operands; both are resident at once (the second adds to what the first stored, and waits for it).
    // Measured at M = 128, N = 4096 (32 tiles): K = 4096 28.9 -> 26.1 us, K = 8192 52.1 -> 37.9, K = 11008 68.2 ->
    // 46.5; three and four splits are no faster (44.3, 46.4 us at K = 11008): every further split adds an ordered
    // pass over the tile in y.
    const int n_chunks = (int)(K / SUPER);
    const int splits = gx * gy * 2 <= caps.sm_count && gx * gy <= HF_MAX_SPLIT_TILES && n_chunks >= 32 ? 2 : 1;
    p.chunks_per_split = ((n_chunks + splits - 1) / splits + 1) / 2 * 2;
    p.k_splits = (n_chunks + p.chunks_per_split - 1) / p.chunks_per_split;
    p.tile_sem = nullptr;
    if (p.k_splits > 1) {
        void *sem = nullptr;
        JQ_CUDA_TRY(cudaGetSymbolAddress(&sem, g_tile_sem));
        p.tile_sem = static_cast<int *>(sem);
    }
    CUtensorMap w_map, x_map;
    if (int rc = encode_byte_map(&w_map, d_w, p.row_bytes, (uint64_t)N, p.row_bytes, Q8_BYTES, 128)) return rc;
    const uint64_t x_row = (uint64_t)p.n_super * Q8_BYTES;
    if (int rc = order == JQ_ORDER_KSUPER_COL
                     ? encode_byte_map(&x_map, d_xq, Q8_BYTES, (uint64_t)p.n_super * (uint64_t)M, Q8_BYTES, Q8_BYTES, 128)
                     : encode_byte_map(&x_map, d_xq, x_row, (uint64_t)M, x_row, Q8_BYTES, 128))
        return rc;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void *>(gemm_q4_0_q8_1_f16_kernel), HF_SMEM_BYTES)) return rc;
    (void)cudaGetLastError();  // a stale error of an earlier, unrelated call must not be taken for this launch's
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)gx, (unsigned)gy, (unsigned)p.k_splits);
    cfg.blockDim = dim3(HF_THREADS);
    cfg.dynamicSmemBytes = HF_SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    JQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_q4_0_q8_1_f16_kernel, p, w_map, x_map));
    return JQ_OK;
}

}  // namespace jq
