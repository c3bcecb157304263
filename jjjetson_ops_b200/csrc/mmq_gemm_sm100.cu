// Prefill-regime multiply (M > 8): an int8 tensor-core GEMM with the per-block rescale folded into
// fp32 accumulators.
//
// Work to replace: q4_0_q8_1_mat_mul_kernel (reference src/cuda/mm_q4_0_q8_1.cu:164-289) for large
// batches, where the reference re-reads every 32-row weight tile once per 4 tokens and does all its
// arithmetic with dp4a.  Here a CTA owns a 128 (weight rows) x 128 (activation columns) tile of Y:
//
//   * K is walked in chunks of 256 values.  A chunk of the weight tile is 128 rows x 144 bytes
//     (8 Q4_0 blocks, a whole number of 16-byte units because K % 256 == 0); a chunk of the
//     activation tile is 128 columns x 2 block_q8_1_mmq.  Both arrive with 16-byte cp.async copies
//     in a 3-stage pipeline; row pitches of 144 and 304 bytes (16 x odd) keep the fragment loads of
//     eight rows x four consecutive words free of bank conflicts.
//   * Per 32-wide block, each warp (64 rows x 32 columns) issues 16 mma.m16n8k32 (u8 nibbles x s8
//     activations -> s32).  The nibbles are unpacked in registers: thread (g, t) of a warp loads
//     word t of the block, whose low nibbles are weights 4t..4t+3 and high nibbles 16+4t.., exactly
//     the two k ranges the A fragment asks of that thread.
//   * The accumulator fragment enters the mma holding the integer 0x4B400000: read back as a float
//     it is 1.5 * 2^23 + sumi exactly, so one fma with (d8, -1.5 * 2^23 * d8) yields round(sumi * d8)
//     with no int->float conversion, and a second fma adds d4 * that to the fp32 accumulator.  Both
//     are issued as packed fma.rn.f32x2 over the two adjacent columns a thread owns.
//   * The zero-point term -8 * d4 * s8 (mm_q4_0_q8_1.cu:92) is rank-1 per block.  It is added by one
//     fp16 mma.m16n8k8 per 8 blocks (A = -8 * d4, B = s8, both exact in fp16; fp32 accumulate into
//     the same fragment), instead of one more fma per element per block.
//
// The integer block sums are exact; the fp32 result differs from the reference kernel's only by
// summation order (the zero-point terms are added per 8 blocks rather than inside each block).
#include <cuda_fp16.h>

#include "jq_common.cuh"

namespace jq {

namespace {

// The CTA tile is (32 * RT weight rows) x (32 * CT activation columns): 8 warps, 2 along rows x 4
// along columns, each owning RT m16 row tiles and CT n8 column tiles.  RT = CT = 4 is the 128 x 128
// tile described above; RT = CT = 2 (64 x 64, two CTAs per SM) serves shapes whose 128 x 128 tiles
// would not fill the SMs (a 4096 -> 4096 projection at M = 128 is 32 of those, but 128 of these).
constexpr int GM_THREADS = 256;
constexpr int GM_STAGES = 3;
constexpr int GM_KCHUNK = 256;             // values of K per pipeline stage
constexpr int GM_W_PITCH = 144;            // bytes per weight row per chunk (8 blocks)
constexpr int GM_X_PITCH = 304;            // 2 x 144 bytes per column per chunk + 16 (bank spread)
template <int RT, int CT>
struct GemmTile {
    static constexpr int BN = 32 * RT, BM = 32 * CT;
    static constexpr int W_BYTES = BN * GM_W_PITCH, X_BYTES = BM * GM_X_PITCH;
    static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    static constexpr int SMEM = GM_STAGES * STAGE_BYTES;
    static constexpr int MIN_CTAS = SMEM <= 100 * 1024 ? 2 : 1;
};
constexpr uint32_t MASK4 = 0x0F0F0F0Fu;
constexpr int MAGIC_I = 0x4B400000;        // bit pattern of 1.5 * 2^23
constexpr float MAGIC_F = 12582912.0f;

__device__ __forceinline__ void cp_async_16(uint32_t smem_dst, const void *gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// d = a * b + c on two packed floats
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(reinterpret_cast<uint64_t &>(d))
        : "l"(reinterpret_cast<const uint64_t &>(a)), "l"(reinterpret_cast<const uint64_t &>(b)),
          "l"(reinterpret_cast<const uint64_t &>(c)));
    return d;
}

// D(16x8, f32) += A(16x8, f16 row) * B(8x8, f16 col)
__device__ __forceinline__ void mma_f16_1688(float (&d)[4], const uint32_t (&a)[2], uint32_t b) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(b));
}

struct GemmParams {
    const uint8_t *w;
    const uint8_t *xq;
    float *y;
    int64_t N, M;
    int K, order;
    int n_super;         // K / 128
    uint32_t row_bytes;  // K / 32 * 18
    int *fault;
    GatherArgs gather;   // world > 0: the tile goes to every rank's [M][N_total] buffer instead of y (all-gather epilogue)
#ifdef JQ_BOUNDS_CHECK
    MulMatBounds bounds; // range-checked debug build: extents of w, xq, y
    uint32_t smem_total; // ... and the launch's dynamic shared memory
#endif
};

constexpr uint32_t GM_GATHER_UNITS = 1u << 16;  // what one all-gather adds to each arrival count (shares of the CTAs sum to it)

template <int RT, int CT>
__device__ __forceinline__ void load_stage(const GemmParams &p, uint32_t smem_base, uint32_t stage_addr, int chunk, int64_t n0,
                                           int64_t m0, int tid) {
    constexpr int GM_BN = GemmTile<RT, CT>::BN, GM_BM = GemmTile<RT, CT>::BM, GM_W_BYTES = GemmTile<RT, CT>::W_BYTES;
    // weights: BN rows x 9 sixteen-byte units
#pragma unroll
    for (int i = 0; i < (GM_BN * 9 + GM_THREADS - 1) / GM_THREADS; ++i) {
        const int idx = tid + i * GM_THREADS;
        if (idx < GM_BN * 9) {
            const int row = idx / 9, part = idx - row * 9;
            // rows past the end are not loaded: whatever the stage holds there only reaches outputs that are never stored
            if (n0 + row < p.N) {
                const uint32_t dst = stage_addr + row * GM_W_PITCH + part * 16;
                const uint8_t *src = p.w + (n0 + row) * p.row_bytes + (size_t)chunk * GM_W_PITCH + part * 16;
                if (JQ_IN_EXTENT(p.bounds.w, src, 16, p.fault) && JQ_IN_SHARED(dst - smem_base, 16, p.smem_total, p.fault)) cp_async_16(dst, src);
            }
        }
    }
    // activations: BM columns x 2 blocks x 9 units
    const uint32_t xs = stage_addr + GM_W_BYTES;
#pragma unroll
    for (int i = 0; i < (GM_BM * 18 + GM_THREADS - 1) / GM_THREADS; ++i) {
        const int idx = tid + i * GM_THREADS;
        if (idx >= GM_BM * 18) break;
        const int col = idx / 18, part = idx - col * 18;
        const int ks = part / 9, unit = part - ks * 9;
        if (m0 + col < p.M) {  // columns past the end: as for the rows
            const int64_t blk = q8_block_index(2 * chunk + ks, m0 + col, p.n_super, p.M, p.order);
            const uint32_t dst = xs + col * GM_X_PITCH + ks * Q8_BYTES + unit * 16;
            const uint8_t *src = p.xq + blk * Q8_BYTES + unit * 16;
            if (JQ_IN_EXTENT(p.bounds.xq, src, 16, p.fault) && JQ_IN_SHARED(dst - smem_base, 16, p.smem_total, p.fault)) cp_async_16(dst, src);
        }
    }
}

template <int RT, int CT>
__global__ void __launch_bounds__(GM_THREADS, GemmTile<RT, CT>::MIN_CTAS) gemm_q4_0_q8_1_mma_kernel(const GemmParams p) {
    constexpr int GM_BN = GemmTile<RT, CT>::BN, GM_BM = GemmTile<RT, CT>::BM, GM_W_BYTES = GemmTile<RT, CT>::W_BYTES;
    constexpr int GM_STAGE_BYTES = GemmTile<RT, CT>::STAGE_BYTES;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int wn = warp & 1, wm = warp >> 1;  // warp tile: rows wn * 16 * RT .., columns wm * 8 * CT ..
    const int64_t n0 = (int64_t)blockIdx.x * GM_BN, m0 = (int64_t)blockIdx.y * GM_BM;
    const int n_chunks = p.K / GM_KCHUNK;

    float acc[RT][CT][4];  // [row tile][column tile][c0..c3]
#pragma unroll
    for (int i = 0; i < RT; ++i)
#pragma unroll
        for (int j = 0; j < CT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.0f;

#pragma unroll
    for (int s = 0; s < GM_STAGES - 1; ++s) {
        if (s < n_chunks) load_stage<RT, CT>(p, smem_base, smem_base + s * GM_STAGE_BYTES, s, n0, m0, tid);
        cp_async_commit();
    }

    const int magic4[4] = {MAGIC_I, MAGIC_I, MAGIC_I, MAGIC_I};

    for (int c = 0; c < n_chunks; ++c) {
        cp_async_wait<GM_STAGES - 2>();
        __syncthreads();  // chunk c has landed for everyone; stage (c-1)%S is free again
        {
            const int nc = c + GM_STAGES - 1;
            if (nc < n_chunks) load_stage<RT, CT>(p, smem_base, smem_base + (nc % GM_STAGES) * GM_STAGE_BYTES, nc, n0, m0, tid);
            cp_async_commit();
        }
        const uint32_t ws = smem_base + (c % GM_STAGES) * GM_STAGE_BYTES;
        const uint32_t xs = ws + GM_W_BYTES;
        const uint32_t w_lane = ws + (wn * 16 * RT + g) * GM_W_PITCH + 4 * t;
        const uint32_t x_frag = xs + (wm * 8 * CT + g) * GM_X_PITCH + Q8_QS_OFFSET + 4 * t;
        const uint32_t x_scale = xs + (wm * 8 * CT + 2 * t) * GM_X_PITCH;

#pragma unroll
        for (int jp = 0; jp < 4; ++jp) {  // pairs of blocks (even, odd): the pair starts 4-byte aligned
            const int ks = jp >> 1;       // which of the chunk's two activation blocks
            const int sub_e = (2 * jp) & 3, sub_o = sub_e + 1;
            // activation fragments and scales of the two blocks, CT column tiles
            uint32_t be[CT][2], bo[CT][2];
            float2 de[CT], ce[CT], d_o[CT], co[CT];
#pragma unroll
            for (int j = 0; j < CT; ++j) {
                const uint32_t xb = x_frag + j * 8 * GM_X_PITCH + ks * Q8_BYTES;
                be[j][0] = lds_u32(xb + sub_e * QK);
                be[j][1] = lds_u32(xb + sub_e * QK + 16);
                bo[j][0] = lds_u32(xb + sub_o * QK);
                bo[j][1] = lds_u32(xb + sub_o * QK + 16);
                const uint32_t sb = x_scale + j * 8 * GM_X_PITCH + ks * Q8_BYTES;
                const uint2 s0 = lds_v2(sb + 4 * sub_e);                 // column 2t: (d,s) of even, odd block
                const uint2 s1 = lds_v2(sb + GM_X_PITCH + 4 * sub_e);    // column 2t+1
                de[j] = make_float2(half_bits_to_float(s0.x & 0xFFFFu), half_bits_to_float(s1.x & 0xFFFFu));
                d_o[j] = make_float2(half_bits_to_float(s0.y & 0xFFFFu), half_bits_to_float(s1.y & 0xFFFFu));
                ce[j] = make_float2(-MAGIC_F * de[j].x, -MAGIC_F * de[j].y);
                co[j] = make_float2(-MAGIC_F * d_o[j].x, -MAGIC_F * d_o[j].y);
            }
#pragma unroll
            for (int i = 0; i < RT; ++i) {
                uint32_t a_e[4], a_o[4];
                float d4e[2], d4o[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t pr = w_lane + (i * 16 + h * 8) * GM_W_PITCH + jp * 2 * Q4_BYTES;
                    const uint32_t u0 = lds_u32(pr), u1 = lds_u32(pr + 4), u2 = lds_u32(pr + 20);
                    const uint32_t we = __funnelshift_r(u0, u1, 16);
                    a_e[h] = we & MASK4;
                    a_e[2 + h] = (we >> 4) & MASK4;
                    a_o[h] = u2 & MASK4;
                    a_o[2 + h] = (u2 >> 4) & MASK4;
                    const uint32_t prd = pr - 4 * t;
                    d4e[h] = half_bits_to_float(lds_u16(prd));
                    d4o[h] = half_bits_to_float(lds_u16(prd + Q4_BYTES));
                }
#pragma unroll
                for (int j = 0; j < CT; ++j) {
                    int c4[4];
                    mma_u8s8_16832(c4, a_e, be[j], magic4);
                    float2 lo = ffma2(make_float2(__int_as_float(c4[0]), __int_as_float(c4[1])), de[j], ce[j]);
                    float2 hi = ffma2(make_float2(__int_as_float(c4[2]), __int_as_float(c4[3])), de[j], ce[j]);
                    float2 a01 = ffma2(make_float2(d4e[0], d4e[0]), lo, make_float2(acc[i][j][0], acc[i][j][1]));
                    float2 a23 = ffma2(make_float2(d4e[1], d4e[1]), hi, make_float2(acc[i][j][2], acc[i][j][3]));
                    mma_u8s8_16832(c4, a_o, bo[j], magic4);
                    lo = ffma2(make_float2(__int_as_float(c4[0]), __int_as_float(c4[1])), d_o[j], co[j]);
                    hi = ffma2(make_float2(__int_as_float(c4[2]), __int_as_float(c4[3])), d_o[j], co[j]);
                    a01 = ffma2(make_float2(d4o[0], d4o[0]), lo, a01);
                    a23 = ffma2(make_float2(d4o[1], d4o[1]), hi, a23);
                    acc[i][j][0] = a01.x;
                    acc[i][j][1] = a01.y;
                    acc[i][j][2] = a23.x;
                    acc[i][j][3] = a23.y;
                }
            }
        }

        // zero-point term of the chunk's 8 blocks: acc += (-8 * d4)[16 x 8] * s8[8 x 8] per tile pair
        {
            uint32_t sfrag[CT];
#pragma unroll
            for (int j = 0; j < CT; ++j) {
                // B fragment: k = 2t, 2t+1 (blocks of the chunk), column g
                const uint32_t sb = xs + (wm * 8 * CT + j * 8 + g) * GM_X_PITCH + ((2 * t) >> 2) * Q8_BYTES + 4 * ((2 * t) & 3);
                const uint2 ds = lds_v2(sb);
                sfrag[j] = (ds.x >> 16) | (ds.y & 0xFFFF0000u);  // (s of block 2t, s of block 2t+1)
            }
#pragma unroll
            for (int i = 0; i < RT; ++i) {
                uint32_t dfrag[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t pr = ws + (wn * 16 * RT + i * 16 + h * 8 + g) * GM_W_PITCH + (2 * t) * Q4_BYTES;
                    const uint32_t lo = lds_u16(pr), hi = lds_u16(pr + Q4_BYTES);
                    const __half2 d2 = __halves2half2(__ushort_as_half((unsigned short)lo), __ushort_as_half((unsigned short)hi));
                    const __half2 scaled = __hmul2(d2, __float2half2_rn(-8.0f));  // exact: a power of two
                    dfrag[h] = *reinterpret_cast<const uint32_t *>(&scaled);
                }
#pragma unroll
                for (int j = 0; j < CT; ++j) mma_f16_1688(acc[i][j], dfrag, sfrag[j]);
            }
        }
    }
    cp_async_wait<0>();

    if (p.gather.world > 0) {
        // ---- all-gather epilogue: the tile is staged in shared memory ([column m][row n], n contiguous as
        // in y) and stored into every rank's [M][N_total] buffer through peer-mapped pointers, 16 bytes per
        // lane and 512 contiguous bytes per tile row; then this CTA adds its share to the arrival count each
        // rank keeps for this one (system-scope release, cumulative over the stores the barrier ordered
        // before it).  Nobody waits here: the consumer of the gathered output waits for the counts.
        const GatherArgs &ga = p.gather;
        constexpr int TP = GM_BN + 4;  // floats per staged tile row (padded against bank conflicts)
        float *tile = reinterpret_cast<float *>(smem);
        const uint32_t gather_epoch = *reinterpret_cast<const volatile uint32_t *>(ga.epoch_ptr) + 1u;
        __syncthreads();  // every warp is done with the pipeline stages
#pragma unroll
        for (int i = 0; i < RT; ++i) {
#pragma unroll
            for (int j = 0; j < CT; ++j) {
                const int nl = wn * 16 * RT + i * 16 + g, ml = wm * 8 * CT + j * 8 + 2 * t;
#pragma unroll
                for (int e = 0; e < 4; ++e) tile[(ml + (e & 1)) * TP + nl + (e >> 1) * 8] = acc[i][j][e];
            }
        }
        __syncthreads();
        const int64_t rows_here = min((int64_t)GM_BM, p.M - m0), cols_here = min((int64_t)GM_BN, p.N - n0);
        for (int q = 0; q < ga.world; ++q) {
            float *base = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(ga.y_peer[q]) +
                                                    (size_t)(gather_epoch & 1u) * ga.y_stride_bytes) +
                          m0 * ga.N_total + ga.n_offset + n0;
            const bool vec_ok = ((reinterpret_cast<uintptr_t>(base) | ((uintptr_t)ga.N_total * 4u)) & 15u) == 0;
            for (int idx = tid; idx < GM_BM * (GM_BN / 4); idx += GM_THREADS) {
                const int ml = idx / (GM_BN / 4), c4 = (idx - ml * (GM_BN / 4)) * 4;
                if (ml >= rows_here || c4 >= cols_here) continue;
                const float *src = tile + ml * TP + c4;
                float *dst = base + (int64_t)ml * ga.N_total + c4;
                if (vec_ok && c4 + 3 < cols_here) {
                    *reinterpret_cast<float4 *>(dst) = make_float4(src[0], src[1], src[2], src[3]);
                } else {
                    for (int e = 0; e < 4 && c4 + e < cols_here; ++e) dst[e] = src[e];
                }
            }
        }
        __syncthreads();  // all of this CTA's peer stores have been issued
        const uint32_t cta = blockIdx.y * gridDim.x + blockIdx.x, n_ctas = gridDim.x * gridDim.y;
        if (tid < ga.world) {
            const uint32_t share = (uint32_t)(((uint64_t)(cta + 1) * GM_GATHER_UNITS) / n_ctas - ((uint64_t)cta * GM_GATHER_UNITS) / n_ctas);
            asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(ga.flag_peer[tid] + ga.rank), "r"(share) : "memory");
        }
        if (tid == 0) {  // bookkeeping off the critical path: the last CTA advances this rank's own step number
            const int prev = atomicAdd(ga.counter, 1);
            if (prev == (int)n_ctas - 1) {
                *ga.counter = 0;
                *ga.epoch_ptr = gather_epoch;
            }
        }
        return;
    }

    // y[m * N + n]: thread owns rows g, g+8 and columns 2t, 2t+1 of each 16 x 8 tile
#pragma unroll
    for (int i = 0; i < RT; ++i) {
#pragma unroll
        for (int j = 0; j < CT; ++j) {
            const int64_t n = n0 + wn * 16 * RT + i * 16 + g;
            const int64_t m = m0 + wm * 8 * CT + j * 8 + 2 * t;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int64_t nn = n + (e >> 1) * 8, mm = m + (e & 1);
                if (nn < p.N && mm < p.M && JQ_IN_EXTENT(p.bounds.y, p.y + mm * p.N + nn, sizeof(float), p.fault)) p.y[mm * p.N + nn] = acc[i][j][e];
            }
        }
    }
}

}  // namespace

namespace {

template <int RT, int CT>
int run_gemm_mma(cudaStream_t st, GemmParams &p) {
    using Tile = GemmTile<RT, CT>;
#ifdef JQ_BOUNDS_CHECK
    p.smem_total = (uint32_t)Tile::SMEM;
#endif
    const int64_t gx = (p.N + Tile::BN - 1) / Tile::BN, gy = (p.M + Tile::BM - 1) / Tile::BM;
    if (gy > 65535) return set_error(JQ_ERR_UNSUPPORTED, "shape too large for the tensor-core GEMM");
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void *>(gemm_q4_0_q8_1_mma_kernel<RT, CT>), Tile::SMEM, true)) return rc;
    (void)cudaGetLastError();  // a stale error of an earlier, unrelated call must not be taken for this launch's
    gemm_q4_0_q8_1_mma_kernel<RT, CT><<<dim3((unsigned)gx, (unsigned)gy), GM_THREADS, Tile::SMEM, st>>>(p);
    JQ_CUDA_TRY(cudaGetLastError());
    return JQ_OK;
}

}  // namespace

int launch_gemm_mma(cudaStream_t st, const void *d_w, const void *d_xq, float *d_y, int64_t K, int64_t N, int64_t M,
                    int order, const GatherArgs *gather) {
    if (K % GM_KCHUNK != 0) return set_error(JQ_ERR_UNSUPPORTED, "tensor-core GEMM needs K %% 256 == 0 (K = %lld)", (long long)K);
    if (((uintptr_t)d_w & 15u) != 0 || ((uintptr_t)d_xq & 15u) != 0)
        return set_error(JQ_ERR_UNSUPPORTED, "tensor-core GEMM needs 16-byte aligned operands");
    if (N == 0 || M == 0) return JQ_OK;
    if (K > (1 << 24)) return set_error(JQ_ERR_UNSUPPORTED, "shape too large for the tensor-core GEMM");
    GemmParams p{};
    p.w = static_cast<const uint8_t *>(d_w);
    p.xq = static_cast<const uint8_t *>(d_xq);
    p.y = d_y;
    p.N = N;
    p.M = M;
    p.K = (int)K;
    p.order = order;
    p.n_super = (int)(K / SUPER);
    p.row_bytes = (uint32_t)(K / QK * Q4_BYTES);
    p.fault = device_fault_ptr();
#ifdef JQ_BOUNDS_CHECK
    p.bounds = mul_mat_bounds(d_w, d_xq, d_y, K, N, M, sizeof(float));
#endif
    if (gather != nullptr) p.gather = *gather;
    DeviceCaps caps;
    if (int rc = device_caps(&caps)) return rc;
    // 128 x 128 tiles unless they would leave a good part of the SMs without work
    const int64_t big_tiles = ((N + 127) / 128) * ((M + 127) / 128);
    if (big_tiles * 5 < (int64_t)caps.sm_count * 4) return run_gemm_mma<2, 2>(st, p);
    return run_gemm_mma<4, 4>(st, p);
}

}  // namespace jq
