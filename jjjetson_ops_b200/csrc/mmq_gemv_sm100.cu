// Decode-regime multiply (M <= 8): an HBM-streaming kernel for sm_100a.
//
// Work to replace: q4_0_q8_1_mat_mul_kernel (reference src/cuda/mm_q4_0_q8_1.cu:164-289) when the
// batch is a handful of columns.  There the whole cost is reading the Q4_0 weights once, so the
// kernel is organised around keeping HBM busy:
//
//   * one persistent CTA per SM owns a contiguous slab of weight rows;
//   * a producer thread streams the slab through a ring of shared-memory stages with 1-D bulk
//     async copies (cp.async.bulk, completion counted on an mbarrier), so many tens of KB per SM
//     are in flight without costing the compute warps a single load instruction;
//   * the activations (at most 8 columns) are quantized in the prologue if they arrive as fp32,
//     and then live in registers for the whole kernel;
//   * consumer warps read the 18-byte blocks out of shared memory, unpack nibbles in registers
//     and form the exact int32 block sums, with dp4a (M <= 2, one warp per row) or with one
//     int8 mma.m16n8k32 per 16 rows x 1 block (M <= 8, K split over the warps);
//   * per block the epilogue is the reference's: acc += d4 * (sumi * d8 - 8 * s8)
//     (mm_q4_0_q8_1.cu:92), with fp32 partial sums reduced by shuffles / through shared memory.
//
// The 18-byte block is only 2-byte aligned, but 8 blocks are 144 = 9 * 16 bytes, so with
// K % 256 == 0 and a 16-byte aligned base every row is a legal bulk-copy source.  Other shapes
// are refused here and fall to the generic kernel.
#include "jq_common.cuh"

namespace jq {

namespace {

constexpr int GV_MAX_STAGES = 8;
constexpr int GV_BAR_BYTES = 256;  // full[8] + empty[8] ring mbarriers, red_full[4] + red_empty[4] (+ spare)
constexpr int GV_RED_SLOTS = 4;
constexpr uint32_t MASK4 = 0x0F0F0F0Fu;

constexpr int GV_MAX_MATS = 4;

struct GemvParams {
    // Up to GV_MAX_MATS weight matrices that share K and the activations, treated as one matrix whose rows are
    // theirs in order (separate q / k / v or gate / up projections in one launch): matrix i owns the rows
    // [mat_begin[i], mat_begin[i + 1]) and writes to y_mat[i], an [M][its row count] array.  n_mats == 1:
    // plain single matrix (w, y).
    const uint8_t *w_mat[GV_MAX_MATS];
    float *y_mat[GV_MAX_MATS];
    int64_t mat_begin[GV_MAX_MATS + 1];
    int n_mats;
    const uint8_t *w;
    const uint8_t *xq;     // quantized activations (nullptr when x_f32 is given)
    const float *x_f32;    // raw activations to quantize in the prologue, or nullptr
    uint8_t *xq_out;       // where CTA 0 publishes the blocks it quantized, or nullptr
    float *y;
    int *fault;
    int64_t N;
    int K, M, order, s_mode;
    int n_super;           // K / 128
    uint32_t row_bytes;    // K / 32 * 18
    uint32_t row_stride;   // distance between rows inside a stage (>= row_bytes)
    uint32_t stage_bytes;
    uint32_t x_bytes;      // shared bytes reserved for the quantized activations
    uint32_t x_pitch;      // bytes between two activation rows there (padded against bank conflicts)
    int stages;
    int rows_per_stage;
    int prefetch_early;    // the weight stream may start before the preceding kernel in the stream has finished
    int early_stages;      // stages the producer may request before the activations are staged
    uint32_t x_copy_bytes; // > 0: the producer brings ready Q8_1 blocks in by bulk copy, straight to their place,
                           // queued ahead of the rest of the weight stream
    GatherArgs gather;     // all-gather epilogue (world == 0: plain store to y)
    uint32_t y_bytes;      // shared bytes of the band staging buffer [M][y_rows] (gather only)
    uint32_t y_rows;
    unsigned long long *trace;  // 8 timestamps per CTA of this launch (tracing aid), or nullptr
    uint32_t poll_limit;        // polls after which a bounded wait gives up
    uint32_t rows_q, rows_r;    // N = rows_q * grid + rows_r (see cta_row_range)
#ifdef JQ_BOUNDS_CHECK
    // range-checked debug build: extents of the buffers (per weight matrix / output), of the activations in whichever
    // form they come, of the workspace, of every rank's all-gather buffers, and the launch's dynamic shared memory
    Extent ext_w[GV_MAX_MATS], ext_y[GV_MAX_MATS], ext_x, ext_xq_out, ext_peer[MAX_PEERS], ext_x_words;
    uint32_t smem_total;
#endif
};

// offset of a shared-memory address inside the launch's dynamic shared memory
extern __shared__ __align__(128) uint8_t gv_dynamic_smem[];
__device__ __forceinline__ uint32_t dyn_offset(const void *p) { return smem_u32(p) - smem_u32(gv_dynamic_smem); }
// a bulk copy whose source lies inside extent `e` of the parameters and whose destination lies inside the dynamic
// shared memory (debug build); the plain copy otherwise
#ifdef JQ_BOUNDS_CHECK
#define JQ_BULK_G2S(p, e, dst, src, bytes, bar)                                                                          \
    do {                                                                                                                 \
        if (in_extent((p).e, src, bytes, (p).fault) && in_shared(dyn_offset(dst), bytes, (p).smem_total, (p).fault))     \
            bulk_g2s(dst, src, bytes, bar);                                                                              \
    } while (0)
#else
#define JQ_BULK_G2S(p, e, dst, src, bytes, bar) bulk_g2s(dst, src, bytes, bar)
#endif

// matrix that owns row r of the concatenation (n_mats is tiny: a linear scan)
__device__ __forceinline__ int mat_of_row(const GemvParams &p, int64_t r) {
    int i = 0;
    while (i + 1 < p.n_mats && r >= p.mat_begin[i + 1]) ++i;
    return i;
}
// where output (column m, row r of the concatenation) lives
__device__ __forceinline__ float *y_slot(const GemvParams &p, int m, int64_t r, int *mat = nullptr) {
    if (p.n_mats <= 1) return p.y + (size_t)m * p.N + r;
    const int i = mat_of_row(p, r);
    if (mat != nullptr) *mat = i;
    return p.y_mat[i] + (size_t)m * (p.mat_begin[i + 1] - p.mat_begin[i]) + (r - p.mat_begin[i]);
}
// store of output (column m, row r), range-checked in the debug build
__device__ __forceinline__ void store_y(const GemvParams &p, int m, int64_t r, float v) {
#ifdef JQ_BOUNDS_CHECK
    int mat = 0;
    float *dst = y_slot(p, m, r, &mat);
    if (in_extent(p.ext_y[mat], dst, sizeof(float), p.fault)) *dst = v;
#else
    *y_slot(p, m, r) = v;
#endif
}

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void trace_stamp(const GemvParams &p, int slot) {
    if (p.trace != nullptr) p.trace[(size_t)blockIdx.x * 8 + slot] = global_ns();
}

#ifdef JQ_TRACE_FINE
__device__ __forceinline__ void trace_fine(const GemvParams &p, int slot) {
    if (p.trace != nullptr) p.trace[(size_t)(blockIdx.x + 256) * 8 + slot] = global_ns();
}
#else
__device__ __forceinline__ void trace_fine(const GemvParams &, int) {}
#endif

// Programmatic dependent launch: let the next kernel in the stream be scheduled early, and wait
// for the previous one (and its memory operations) before touching anything it may have written.
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Rows of this CTA: N = q * grid + r, the first r CTAs own q + 1 rows.  q and r come from the host: a 64-bit
// division costs a thread several hundred cycles, and this sits between the predecessor's end and the first
// multiply.
__device__ __forceinline__ void cta_row_range(const GemvParams &p, int64_t *begin, int64_t *end) {
    const uint32_t b = blockIdx.x;
    *begin = (int64_t)b * p.rows_q + min(b, p.rows_r);
    *end = *begin + p.rows_q + (b < p.rows_r ? 1 : 0);
}

// The rows of this CTA, stage by stage: one contiguous slab per CTA, full stages of R rows and one
// shorter stage at the end.  (Dealing the stages out round-robin over the CTAs, so that the chip reads
// one contiguous window of the matrix at a time, was measured within +-3 % of this and dropped.)
struct RowWalk {
    int64_t base, step;       // stage c < n_main starts at base + c * step and has R rows
    int64_t tail_begin;       // the one shorter stage after them
    int tail_rows, n_main, n_chunks;
};
__device__ __forceinline__ RowWalk cta_row_walk(const GemvParams &p, int R) {
    RowWalk w;
    int64_t b, e;
    cta_row_range(p, &b, &e);
    w.n_main = (int)((uint32_t)(e - b) / (uint32_t)R);
    w.base = b;
    w.step = R;
    w.tail_begin = b + (int64_t)w.n_main * R;
    w.tail_rows = (int)(e - w.tail_begin);
    w.n_chunks = w.n_main + (w.tail_rows > 0 ? 1 : 0);
    return w;
}
__device__ __forceinline__ int64_t walk_stage(const RowWalk &w, int c, int R, int *rows) {
    if (c < w.n_main) {
        *rows = R;
        return w.base + (int64_t)c * w.step;
    }
    *rows = w.tail_rows;
    return w.tail_begin;
}

// Arrival counts: every all-gather adds GATHER_UNITS to the count a rank keeps for each sender, split over
// the sender's CTAs in shares that sum to exactly that (so the receiver need not know the sender's grid).
constexpr uint32_t GATHER_UNITS = 1u << 16;
__device__ __forceinline__ uint32_t gather_share() {
    return (uint32_t)(((uint64_t)(blockIdx.x + 1) * GATHER_UNITS) / gridDim.x - ((uint64_t)blockIdx.x * GATHER_UNITS) / gridDim.x);
}

// Lanes 0..world-1 of one warp poll this rank's arrival counts until all of all-gather number `epoch`
// has arrived from each sender (counts and the product wrap together modulo 2^32).
__device__ __forceinline__ void wait_flags(const uint32_t *flags, int world, uint32_t epoch, int lane, int *fault,
                                           uint32_t limit) {
    if (lane < world) {
        const uint32_t expected = epoch * GATHER_UNITS;
        bool seen = false;
        for (uint32_t spin = 0; spin < limit && !seen; ++spin) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + lane) : "memory");
            seen = (int32_t)(v - expected) >= 0;
        }
        if (!seen) report_fault(fault, 2);
    }
    __syncwarp();
}

// ---- tagged words: {fp32 bits, number of the all-gather} in one 8-byte store, which arrives whole ----------
__device__ __forceinline__ void st_word(unsigned long long *dst, float v, uint32_t tag) {
    const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(dst), "l"(w) : "memory");
}
// two neighbouring words (16-byte aligned): x, z their values, y, w their tags
__device__ __forceinline__ uint4 ld_words2(const unsigned long long *src) {
    uint4 r;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(src) : "memory");
    return r;
}

// four neighbouring words (32-byte aligned) in one load
__device__ __forceinline__ void ld_words4(const unsigned long long *src, uint4 *lo, uint4 *hi) {
    unsigned long long a0, a1, a2, a3;
    asm volatile("ld.volatile.global.v4.u64 {%0, %1, %2, %3}, [%4];" : "=l"(a0), "=l"(a1), "=l"(a2), "=l"(a3) : "l"(src) : "memory");
    *lo = make_uint4((uint32_t)a0, (uint32_t)(a0 >> 32), (uint32_t)a1, (uint32_t)(a1 >> 32));
    *hi = make_uint4((uint32_t)a2, (uint32_t)(a2 >> 32), (uint32_t)a3, (uint32_t)(a3 >> 32));
}

// Every word of all-gather number *ticket >> 16 -> plain fp32, each thread waiting (bounded) for its own words.
__global__ void __launch_bounds__(256) allgather_tagged_read_kernel(const unsigned long long *words, uint64_t stride_bytes,
                                                                    int64_t n_words, const unsigned long long *ticket,
                                                                    float *out, int *fault, uint32_t limit) {
    const uint32_t tag = (uint32_t)(*reinterpret_cast<const volatile unsigned long long *>(ticket) >> 16);
    const unsigned long long *src =
        reinterpret_cast<const unsigned long long *>(reinterpret_cast<const uint8_t *>(words) + (size_t)(tag & 1u) * stride_bytes);
    for (int64_t i = 2 * ((int64_t)blockIdx.x * blockDim.x + threadIdx.x); i < n_words; i += 2 * (int64_t)gridDim.x * blockDim.x) {
        uint4 w = make_uint4(0u, 0u, 0u, 0u);
        bool ok = false;
        for (uint32_t spin = 0; spin < limit && !ok; ++spin) {
            w = ld_words2(src + i);
            ok = w.y == tag && w.w == tag;
        }
        if (!ok) report_fault(fault, 2);
        *reinterpret_cast<float2 *>(out + i) = make_float2(__uint_as_float(w.x), __uint_as_float(w.z));
    }
}

__global__ void allgather_wait_kernel(const uint32_t *flags, int world, const uint32_t *epoch_ptr, int *fault,
                                      uint32_t limit) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t epoch = *reinterpret_cast<const volatile uint32_t *>(epoch_ptr);
    if (epoch != 0) wait_flags(flags, world, epoch, (int)threadIdx.x, fault, limit);
}

// Producer: walks the CTA's rows stage by stage.  With one copy per stage a single thread calls it;
// with one copy per row (PER_ROW: rows land a padded distance apart) the whole warp calls it, lane 0
// does the waiting and arms the barrier, and lane r issues the copy of row r, so that the sixteen
// copies of a stage are handed to the copy engine at once instead of one after the other.
// When the stream starts ahead of the previous kernel's end (static weights), only `early_stages`
// stages are requested up front: the activation loads that follow the wait would otherwise queue
// behind the whole ring's worth of weight traffic on this SM's path to L2.
// One thread waits until all of all-gather number `epoch` has arrived from every sender.
__device__ __forceinline__ bool wait_flags_serial(const uint32_t *flags, int world, uint32_t epoch, int *fault, uint32_t limit) {
    const uint32_t expected = epoch * GATHER_UNITS;
    for (int q = 0; q < world; ++q) {
        bool seen = false;
        for (uint32_t spin = 0; spin < limit && !seen; ++spin) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + q) : "memory");
            seen = (int32_t)(v - expected) >= 0;
        }
        if (!seen) {
            report_fault(fault, 2);
            return false;
        }
    }
    return true;
}

// The point in the producer's walk where the activations come in (one thread).  Old protocol: the consumer
// warps load them and the producer only waits until those loads have landed.  With x_copy_bytes the producer
// itself queues the ready blocks as bulk copies, ahead of the rest of the weight stream, after it has waited for
// the previous kernel (and, for an N-sharded layer that consumes a gathered output, for that output's bands).
__device__ __forceinline__ bool producer_activations(const GemvParams &p, uint64_t *x_ready, uint64_t *x_full, uint8_t *xs) {
    if (p.x_copy_bytes == 0) return !p.prefetch_early || mbar_wait_bounded(x_ready, 0u, p.fault, p.poll_limit);
    if (p.prefetch_early) griddep_wait();
    if (p.gather.world > 0 && p.gather.wait_previous) {
        const uint32_t done = *reinterpret_cast<const volatile uint32_t *>(p.gather.epoch_ptr);
        if (done != 0 && !wait_flags_serial(p.gather.flag_peer[p.gather.rank], p.gather.world, done, p.fault, p.poll_limit)) return false;
    }
    mbar_arrive_expect_tx(x_full, p.x_copy_bytes);
    const uint32_t per_row = (uint32_t)p.n_super * Q8_BYTES;
    for (int m = 0; m < p.M; ++m) JQ_BULK_G2S(p, ext_x, xs + (size_t)m * p.x_pitch, p.xq + (size_t)m * per_row, per_row, x_full);
    return true;
}

template <bool PER_ROW>
__device__ __forceinline__ void gemv_producer(const GemvParams &p, uint64_t *full, uint64_t *empty,
                                              uint64_t *x_ready, uint8_t *ring, int lane, uint64_t *x_full = nullptr,
                                              uint8_t *xs = nullptr) {
    const int R = p.rows_per_stage;
    const RowWalk walk = cta_row_walk(p, R);
    const int n_chunks = walk.n_chunks;
    int s = 0;
    uint32_t round = 0;
    bool x_done = false;
    // A sharded layer that consumes a gathered output waits several microseconds for the bands before its
    // activations can come in: with static weights the whole ring is requested first, it lands during that wait.
    const int early_stages =
        p.x_copy_bytes != 0 && p.prefetch_early && p.gather.world > 1 && p.gather.wait_previous ? p.stages : p.early_stages;
    for (int c = 0; c < n_chunks; ++c) {
        int rows;
        const int64_t r0 = walk_stage(walk, c, R, &rows);
        int ok = 1;
        if (lane == 0) {
            if (c == early_stages) {
                ok = producer_activations(p, x_ready, x_full, xs) ? 1 : 0;
                x_done = true;
            }
            if (ok && round > 0 && !mbar_wait_bounded(&empty[s], (round - 1) & 1u, p.fault, p.poll_limit)) ok = 0;
            if (ok) mbar_arrive_expect_tx(&full[s], (uint32_t)rows * p.row_bytes);
        }
        if (PER_ROW) {
            ok = __shfl_sync(0xFFFFFFFFu, ok, 0);  // also orders the copies after the barrier was armed
        }
        if (!ok) return;
        uint8_t *dst = ring + (size_t)s * p.stage_bytes;
        if (p.n_mats <= 1) {
            const uint8_t *src = p.w + r0 * p.row_bytes;
            if (PER_ROW) {
                for (int r = lane; r < rows; r += 32) {
                    JQ_BULK_G2S(p, ext_w[0], dst + (size_t)r * p.row_stride, src + (size_t)r * p.row_bytes, p.row_bytes, &full[s]);
                }
            } else {
                JQ_BULK_G2S(p, ext_w[0], dst, src, (uint32_t)rows * p.row_bytes, &full[s]);
            }
        } else if (PER_ROW) {
            for (int r = lane; r < rows; r += 32) {
                const int i = mat_of_row(p, r0 + r);
                JQ_BULK_G2S(p, ext_w[i], dst + (size_t)r * p.row_stride, p.w_mat[i] + (r0 + r - p.mat_begin[i]) * p.row_bytes,
                                 p.row_bytes, &full[s]);
            }
        } else {
            // a stage may straddle matrices: one copy per matrix it touches, landing back to back
            int64_t r = r0;
            int left = rows;
            while (left > 0) {
                const int i = mat_of_row(p, r);
                const int take = (int)min((int64_t)left, p.mat_begin[i + 1] - r);
                JQ_BULK_G2S(p, ext_w[i], dst, p.w_mat[i] + (r - p.mat_begin[i]) * p.row_bytes, (uint32_t)take * p.row_bytes, &full[s]);
                dst += (size_t)take * p.row_bytes;
                r += take;
                left -= take;
            }
        }
        if (++s == p.stages) {
            s = 0;
            ++round;
        }
    }
    // fewer stages than may be requested early: the activations still have to be brought in
    if (lane == 0 && !x_done && p.x_copy_bytes != 0) producer_activations(p, x_ready, x_full, xs);
}

// Prologue of the consumer warps: put the quantized activations into shared memory, laid out
// [m][k/128] as 144-byte blocks.  Either quantize fp32 input (bit-identical to the stand-alone
// quantizer) or copy already quantized blocks, honouring their order.
// One batch of the fused quantizer: U 128-value blocks per warp, indices base, base + NW, ...; all U are
// quantized together (no early exit inside the batch), so that their shuffle chains overlap.
template <int NW, int U>
__device__ __forceinline__ void quantize_batch(const GemvParams &p, uint8_t *xs, uint64_t *x_ready, int warp, int lane,
                                               int base, int total, bool first) {
    float4 xi[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int idx = base + u * NW;
        xi[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (idx < total) {
            const int m = idx / p.n_super, ks = idx - m * p.n_super;
            const float4 *src = reinterpret_cast<const float4 *>(p.x_f32 + (size_t)m * p.K + ks * SUPER) + lane;
            if (JQ_IN_EXTENT(p.ext_x, src, sizeof(float4), p.fault)) xi[u] = __ldg(src);
        }
    }
    if (first) {
        // this warp's first (usually only) batch of loads has landed: let the weight stream go on
        float touch = 0.0f;
#pragma unroll
        for (int u = 0; u < U; ++u) touch += xi[u].x;
        touch = __shfl_xor_sync(0xFFFFFFFFu, touch, 1, 32);
        if (lane == 0) {
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0]; // after %1" ::"r"(smem_u32(x_ready)), "f"(touch)
                         : "memory");
        }
        if (threadIdx.x == 0) trace_fine(p, 0);  // warp 0: x loads landed
    }
    uint32_t qv[U], dsv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) qv[u] = quantize_group_q8_1(xi[u], p.s_mode, &dsv[u]);
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int idx = base + u * NW;  // uniform across the warp
        if (idx < total) {
            const int m = idx / p.n_super, ks = idx - m * p.n_super;
            uint8_t *blk = xs + (size_t)m * p.x_pitch + (size_t)ks * Q8_BYTES;
            if (!JQ_IN_SHARED(dyn_offset(blk), Q8_BYTES, p.smem_total, p.fault)) continue;
            reinterpret_cast<uint32_t *>(blk + Q8_QS_OFFSET)[lane] = qv[u];
            if ((lane & 7) == 0) reinterpret_cast<uint32_t *>(blk)[lane >> 3] = dsv[u];
            if (p.xq_out != nullptr && blockIdx.x == 0) {
                uint8_t *g = p.xq_out + (size_t)idx * Q8_BYTES;  // JQ_ORDER_COL_KSUPER
                if (!JQ_IN_EXTENT(p.ext_xq_out, g, Q8_BYTES, p.fault)) continue;
                reinterpret_cast<uint32_t *>(g + Q8_QS_OFFSET)[lane] = qv[u];
                if ((lane & 7) == 0) reinterpret_cast<uint32_t *>(g)[lane >> 3] = dsv[u];
            }
        }
    }
}

// A pair of quantized blocks (eight values per lane) to its place in shared memory, and to the workspace by CTA 0.
__device__ __forceinline__ void store_pair_blocks(const GemvParams &p, uint8_t *xs, int pr, int lane, uint2 qv, uint32_t ds) {
    const int idx = 2 * pr + (lane >> 4);  // this lane's block, (m, ks) in row-major order
    const int m = idx / p.n_super, ks = idx - m * p.n_super;
    uint8_t *blk = xs + (size_t)m * p.x_pitch + (size_t)ks * Q8_BYTES;
    if (!JQ_IN_SHARED(dyn_offset(blk), Q8_BYTES, p.smem_total, p.fault)) return;
    reinterpret_cast<uint2 *>(blk + Q8_QS_OFFSET)[lane & 15] = qv;
    if ((lane & 3) == 0) reinterpret_cast<uint32_t *>(blk)[(lane & 15) >> 2] = ds;
    if (p.xq_out != nullptr && blockIdx.x == 0) {
        uint8_t *g = p.xq_out + (size_t)idx * Q8_BYTES;  // JQ_ORDER_COL_KSUPER
        if (!JQ_IN_EXTENT(p.ext_xq_out, g, Q8_BYTES, p.fault)) return;
        reinterpret_cast<uint2 *>(g + Q8_QS_OFFSET)[lane & 15] = qv;
        if ((lane & 3) == 0) reinterpret_cast<uint32_t *>(g)[(lane & 15) >> 2] = ds;
    }
}

template <int NW>
__device__ __forceinline__ void stage_activations(const GemvParams &p, uint8_t *xs, uint64_t *x_ready, int warp,
                                                  int lane, uint32_t x_tag = 0u) {
    const int total = p.M * p.n_super;
    bool arrived = false;  // this warp has told the producer that its first loads have landed
    if (p.gather.x_words != nullptr) {
        // The activations are the output of all-gather number x_tag, arriving as tagged words from every rank:
        // a lane polls its own eight words until all carry that number (they are the synchronisation: nothing
        // else is waited for), then the pair of blocks is quantized as below.
        const GatherArgs &ga = p.gather;
        const unsigned long long *xw = reinterpret_cast<const unsigned long long *>(
            reinterpret_cast<const uint8_t *>(ga.x_words) + (size_t)(x_tag & 1u) * ga.x_stride_bytes);
        const int pairs = total >> 1;
        for (int pr = warp; pr < pairs; pr += NW) {
            const int e = pr * (2 * SUPER) + 8 * lane;  // element of the [M][K] activations
            const int m = e / p.K, k = e - m * p.K;
            const int seg = k / ga.x_seg_len, j = k - seg * ga.x_seg_len;
            const unsigned long long *src = xw + (size_t)m * ga.x_row_words + (size_t)seg * ga.x_seg_stride + j;
            // (Measured and dropped: one lane per warp watching a single pair of words before all lanes look, 9.55
            // against 9.15 us per step on two GPUs: the words of different senders arrive microseconds apart, and the
            // lanes are better off each watching their own.)
            uint4 w[4];
#ifdef JQ_BOUNDS_CHECK
            for (int u = 0; u < 4; ++u) w[u] = make_uint4(0u, 0u, 0u, 0u);
#endif
            bool ok = false;
            const bool readable = JQ_IN_EXTENT(p.ext_x_words, src, 8 * sizeof(unsigned long long), p.fault);
            for (uint32_t spin = 0; readable && spin < p.poll_limit && !ok; ++spin) {
                if (ga.x_wide) {
                    // A thread's strong loads are carried out one after the other (four 16-byte loads of words that
                    // were all there took 3 us on a loaded GPU, two 32-byte loads 1.9 us), so as few as possible.
                    ld_words4(src, &w[0], &w[1]);
                    ld_words4(src + 4, &w[2], &w[3]);
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u) w[u] = ld_words2(src + 2 * u);
                }
                ok = true;
#pragma unroll
                for (int u = 0; u < 4; ++u) ok = ok && w[u].y == x_tag && w[u].w == x_tag;
            }
            if (!ok && readable) report_fault(p.fault, 2);
            __syncwarp();
            if (!arrived) {
                if (lane == 0) mbar_arrive(x_ready);
                arrived = true;
                if (threadIdx.x == 0) trace_fine(p, 0);  // warp 0: its words have arrived
            }
            const float v[8] = {__uint_as_float(w[0].x), __uint_as_float(w[0].z), __uint_as_float(w[1].x), __uint_as_float(w[1].z),
                                __uint_as_float(w[2].x), __uint_as_float(w[2].z), __uint_as_float(w[3].x), __uint_as_float(w[3].z)};
            uint2 qv;
            uint32_t ds;
            quantize_8_per_lane_q8_1(v, p.s_mode, &qv, &ds);
            store_pair_blocks(p, xs, pr, lane, qv, ds);
        }
    } else if (p.x_f32 != nullptr && (p.n_super & 1) == 0) {
        // Whole pairs of blocks (K % 256 == 0): warp w takes the pairs w, w + NW, ..., eight values per lane
        // (half the instructions per value of the four-per-lane form below, same bits).  All of a warp's loads
        // are issued before the first pair is quantized.
        const int pairs = total >> 1;
        constexpr int MAXP = 4;  // pairs per warp held in registers at once
        for (int p0 = warp; p0 < pairs; p0 += NW * MAXP) {
            float4 xa[MAXP], xb[MAXP];
#pragma unroll
            for (int u = 0; u < MAXP; ++u) {
                const int pr = p0 + u * NW;
                xa[u] = xb[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (pr < pairs) {
                    const float4 *src = reinterpret_cast<const float4 *>(p.x_f32 + (size_t)pr * (2 * SUPER)) + 2 * lane;
                    if (JQ_IN_EXTENT(p.ext_x, src, 2 * sizeof(float4), p.fault)) {
                        xa[u] = __ldg(src);
                        xb[u] = __ldg(src + 1);
                    }
                }
            }
            if (!arrived) {
                float touch = 0.0f;
#pragma unroll
                for (int u = 0; u < MAXP; ++u) touch += xa[u].x + xb[u].x;
                touch = __shfl_xor_sync(0xFFFFFFFFu, touch, 1, 32);
                if (lane == 0) {
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0]; // after %1" ::"r"(smem_u32(x_ready)), "f"(touch)
                                 : "memory");
                }
                arrived = true;
                if (threadIdx.x == 0) trace_fine(p, 0);  // warp 0: x loads landed
            }
#pragma unroll
            for (int u = 0; u < MAXP; ++u) {
                const int pr = p0 + u * NW;  // uniform across the warp
                if (pr >= pairs) break;
                const float v[8] = {xa[u].x, xa[u].y, xa[u].z, xa[u].w, xb[u].x, xb[u].y, xb[u].z, xb[u].w};
                uint2 qv;
                uint32_t ds;
                quantize_8_per_lane_q8_1(v, p.s_mode, &qv, &ds);
                store_pair_blocks(p, xs, pr, lane, qv, ds);
            }
        }
    } else if (p.x_f32 != nullptr) {
        arrived = warp < total;  // quantize_batch arrives for the warps that have a block
        // The prologue is bound by instruction issue (every CTA repeats it, ~100 instructions per block and
        // lane): a warp takes exactly the blocks it has to, two at a time when that covers them all
        // (one activation row of K = 4096 over 16 warps), else four at a time.
        if (total <= 2 * NW) {
            if (warp < total) quantize_batch<NW, 2>(p, xs, x_ready, warp, lane, warp, total, true);
        } else {
            for (int base = warp; base < total; base += NW * 4) {
                quantize_batch<NW, 4>(p, xs, x_ready, warp, lane, base, total, base == warp);
            }
        }
    } else {
        // 9 x 16 bytes per block
        for (int i = warp * 32 + lane; i < total * 9; i += NW * 32) {
            const int idx = i / 9, part = i - idx * 9;
            const int m = idx / p.n_super, ks = idx - m * p.n_super;
            const uint8_t *g = p.xq + (size_t)q8_block_index(ks, m, p.n_super, p.M, p.order) * Q8_BYTES;
#ifdef JQ_BOUNDS_CHECK
            uint4 *dst = reinterpret_cast<uint4 *>(xs + (size_t)m * p.x_pitch + (size_t)ks * Q8_BYTES) + part;
            if (in_extent(p.ext_x, g + 16 * part, 16, p.fault) && in_shared(dyn_offset(dst), 16, p.smem_total, p.fault))
                *dst = __ldg(reinterpret_cast<const uint4 *>(g) + part);
#else
            reinterpret_cast<uint4 *>(xs + (size_t)m * p.x_pitch + (size_t)ks * Q8_BYTES)[part] =
                __ldg(reinterpret_cast<const uint4 *>(g) + part);
#endif
        }
    }
    if (!arrived) {
        // copies issued above were consumed by their stores; warps without a group arrive at once
        __syncwarp();
        if (lane == 0) mbar_arrive(x_ready);
    }
    if (threadIdx.x == 0) trace_fine(p, 1);  // warp 0: its blocks are in shared memory
    named_bar_sync(1, NW * 32);
}

// unsigned bytes of a times signed bytes of b, accumulated in c
__device__ __forceinline__ int dp4a_u8s8(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// ------------------------------------------------------------------------------------------------
// dp4a variant: one warp per weight row, one lane per 128-value slice (four Q4_0 blocks = 72
// bytes, read as nine conflict-free 8-byte shared loads), activations of that slice in registers.
// A warp works on two rows at a time, one from each of two consecutive stages, so that the loads,
// the dp4a chains and the reduction of one row fill the latencies of the other.
// ------------------------------------------------------------------------------------------------

// The four blocks of one lane's slice of one row: acc[m] += d4 * (sumi * d8 - 8 * s8) per block.
template <int M_T>
__device__ __forceinline__ void dp4a_slice(const uint32_t (&wv)[18], const int (&xq)[M_T][32], const float (&xd)[M_T][4],
                                           const float (&xms)[M_T][4], float (&acc)[M_T]) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        // block b starts at byte 18 b of the 72: word 4.5 b
        uint32_t q[4], dbits;
        if ((b & 1) == 0) {
            const int w0 = (b / 2) * 9;
            dbits = wv[w0] & 0xFFFFu;
#pragma unroll
            for (int t = 0; t < 4; ++t) q[t] = __funnelshift_r(wv[w0 + t], wv[w0 + t + 1], 16);
        } else {
            const int w0 = (b / 2) * 9 + 4;
            dbits = wv[w0] >> 16;
#pragma unroll
            for (int t = 0; t < 4; ++t) q[t] = wv[w0 + 1 + t];
        }
        const float d4 = half_bits_to_float(dbits);
        // low nibbles as they are, high nibbles left in place (16 x their value, unsigned
        // bytes): 16 * sumi = 16 * lo + hi16 exactly, and xd carries d8 / 16
        int lo_acc[M_T], hi_acc[M_T];
#pragma unroll
        for (int m = 0; m < M_T; ++m) lo_acc[m] = hi_acc[m] = 0;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const uint32_t lo = q[t] & MASK4, hi16 = q[t] & (MASK4 << 4);
#pragma unroll
            for (int m = 0; m < M_T; ++m) {
                lo_acc[m] = dp4a_u8s8(lo, xq[m][8 * b + t], lo_acc[m]);
                hi_acc[m] = dp4a_u8s8(hi16, xq[m][8 * b + t + 4], hi_acc[m]);
            }
        }
#pragma unroll
        for (int m = 0; m < M_T; ++m) {
            const int s16 = lo_acc[m] * 16 + hi_acc[m];
            acc[m] = fmaf(d4, fmaf((float)s16, xd[m][b], xms[m][b]), acc[m]);
        }
    }
}

// The consumer warps of a CTA meet on an mbarrier (one arrival per warp) with a bounded wait: a warp whose wait for a
// stage ran out has left the kernel, and the others must not wait for it for ever, as they would at a hardware barrier.
__device__ __forceinline__ bool consumers_meet(uint64_t *bar, int lane, int *fault, uint32_t limit) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
    return mbar_wait_bounded(bar, 0u, fault, limit);
}

template <int M_T, int NSB, int NW, int MINB, bool TAGGED>
__global__ void __launch_bounds__((NW + 1) * 32, MINB) gemv_dp4a_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + GV_MAX_STAGES;
    uint64_t *x_ready = full + 24;
    uint64_t *x_full = full + 25;
    unsigned long long *ticket_slot = reinterpret_cast<unsigned long long *>(full + 26);
    uint64_t *meet = full + 27;  // two meetings of the consumer warps in the all-gather epilogues
    float *ybuf = reinterpret_cast<float *>(smem + GV_BAR_BYTES);
    uint8_t *xs = smem + GV_BAR_BYTES + p.y_bytes;
    uint8_t *ring = xs + p.x_bytes;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], NW);
        }
        mbar_init(x_ready, NW);
        mbar_init(x_full, 1);
        mbar_init(meet, NW);
        mbar_init(meet + 1, NW);
        fence_mbar_init();
        // Tagged all-gather: this launch's number comes from a count that every launch raises by 65536, a share per
        // CTA.  The next launch in the stream starts only after every CTA of this one has passed the trigger below,
        // i.e. has its share in: all CTAs of a launch read values in the same 65536-wide window.
        if (p.gather.ticket != nullptr) *ticket_slot = atomicAdd(p.gather.ticket, (unsigned long long)gather_share());
    }
    __syncthreads();

    if (threadIdx.x == 0) trace_stamp(p, 0);  // CTA started
    griddep_launch_dependents();
    if (warp == NW) {
        if (lane == 0) {
            if (!p.prefetch_early) griddep_wait();
            trace_stamp(p, 1);  // weight stream begins
            gemv_producer<false>(p, full, empty, x_ready, ring, 0, x_full, xs);
            trace_stamp(p, 2);  // last copy issued
        }
        return;
    }
    // everything that does not depend on the previous kernel comes before the wait for it
    int64_t r_begin, r_end;
    cta_row_range(p, &r_begin, &r_end);
    const int R = p.rows_per_stage;
    const RowWalk walk = cta_row_walk(p, R);
    const int n_chunks = walk.n_chunks;
    const uint32_t ring_addr = smem_u32(ring);
    const bool tracing = p.trace != nullptr && threadIdx.x == 0;

    // Activations may come from, and outputs may be read by, the previous kernel.  Activations that arrive as
    // tagged words order themselves: that kernel does not wait for its predecessor before its last instruction.
    // (The tagged form is an instance of its own: in one kernel its stores in the row loop cost the plain form two
    // registers and half a percent.)
    constexpr bool tagged = TAGGED;  // p.gather.ticket != nullptr
    const bool x_tagged = tagged && p.gather.x_words != nullptr;
    if (!x_tagged) griddep_wait();
    uint32_t gather_epoch = 0;  // number of this all-gather (previous ones finished: *epoch_ptr)
    uint32_t x_tag = 0;
    if (tagged) {
        const uint32_t launched = (uint32_t)(*ticket_slot >> 16);  // all-gathers launched before this one
        x_tag = launched - (uint32_t)p.gather.x_back;
        gather_epoch = launched + 1u;
    } else if (p.gather.world > 0) {
        const uint32_t done = *reinterpret_cast<const volatile uint32_t *>(p.gather.epoch_ptr);
        gather_epoch = done + 1;
        if (p.x_copy_bytes == 0 && p.gather.wait_previous && done != 0) {
            // the activations are the output of the previous sharded layer: all its bands must be here
            // (when the producer copies the activations in, it has waited for the bands itself)
            if (warp == 0) wait_flags(p.gather.flag_peer[p.gather.rank], p.gather.world, done, lane, p.fault, p.poll_limit);
            named_bar_sync(1, NW * 32);
        }
    }
    if (threadIdx.x == 0) trace_stamp(p, 3);  // predecessor finished

    if (p.x_copy_bytes != 0) {
        if (!mbar_wait_bounded(x_full, 0u, p.fault, p.poll_limit)) return;
        if (threadIdx.x == 0) trace_fine(p, 0);  // the blocks have landed in shared memory
    } else {
        stage_activations<NW>(p, xs, x_ready, warp, lane, x_tag);
    }
    if (threadIdx.x == 0) trace_stamp(p, 4);  // activations staged

    // This lane's slices of X: slice i covers k in [128*(lane + 32 i), +128).
    int xq[NSB][M_T][32];
    float xd[NSB][M_T][4], xms[NSB][M_T][4];
#pragma unroll
    for (int i = 0; i < NSB; ++i) {
        const int sb = lane + 32 * i;
#pragma unroll
        for (int m = 0; m < M_T; ++m) {
            if (sb < p.n_super && m < p.M) {
                const uint4 *b = reinterpret_cast<const uint4 *>(xs + (size_t)m * p.x_pitch + (size_t)sb * Q8_BYTES);
                const uint4 ds = b[0];
                const uint32_t dsv[4] = {ds.x, ds.y, ds.z, ds.w};
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    xd[i][m][g] = 0.0625f * half_bits_to_float(dsv[g] & 0xFFFFu);  // d8 / 16, exact
                    xms[i][m][g] = -8.0f * half_bits_to_float(dsv[g] >> 16);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint4 v = b[1 + j];
                    xq[i][m][4 * j + 0] = (int)v.x;
                    xq[i][m][4 * j + 1] = (int)v.y;
                    xq[i][m][4 * j + 2] = (int)v.z;
                    xq[i][m][4 * j + 3] = (int)v.w;
                }
            } else {
#pragma unroll
                for (int g = 0; g < 4; ++g) xd[i][m][g] = xms[i][m][g] = 0.0f;
#pragma unroll
                for (int j = 0; j < 32; ++j) xq[i][m][j] = 0;
            }
        }
    }
    if (threadIdx.x == 0) trace_fine(p, 2 + (xq[0][0][0] == 0x7fffffff ? 1 : 0));  // activations in registers

    // Two stages (A, B) are taken per step, and everything a step needs besides the rows themselves is kept to
    // a few 32-bit operations: with one row per warp and stage, whatever is computed per stage is paid per row
    // (halving the number of steps took the fused cfg2 step from 8.4 to 7.2 us).  Rows are counted relative to
    // the CTA's first row.  When the whole slab has ring slots of its own (n_chunks <= stages) no slot is ever
    // refilled and nothing is handed back to the producer.
    const bool resident = n_chunks <= p.stages;
    const bool single_mat = p.n_mats <= 1;
    float *const y_cta = p.gather.world > 0 ? ybuf : (single_mat ? p.y + r_begin : nullptr);
    const size_t y_pitch = p.gather.world > 0 ? (size_t)p.y_rows : (size_t)p.N;
    // Tagged words leave as their rows finish: lane j of each half-warp stores to rank (rank + 1 + j) % world (the
    // ranks start on different peers; the local copy comes last), so the words are on their way while the rest of
    // the slab is still being multiplied, and nothing is left to push at the end.
    unsigned long long *word_dst = nullptr;
#ifdef JQ_BOUNDS_CHECK
    int word_peer = 0;
#endif
    if (tagged && (lane & 15) < p.gather.world) {
        const int q = (p.gather.rank + 1 + (lane & 15)) % p.gather.world;
        word_dst = reinterpret_cast<unsigned long long *>(reinterpret_cast<uint8_t *>(p.gather.y_peer[q]) +
                                                          (size_t)(gather_epoch & 1u) * p.gather.y_stride_bytes) +
                   p.gather.n_offset + r_begin;
#ifdef JQ_BOUNDS_CHECK
        word_peer = q;
#endif
    }
    const uint32_t row_off = (uint32_t)warp * p.row_bytes + (uint32_t)lane * 72u;
    int s = 0;
    uint32_t parity = 0;
    for (int c = 0; c < n_chunks; c += 2) {
        const bool two = c + 1 < n_chunks;
        const int sA = s;
        if (!mbar_wait_bounded(&full[sA], parity, p.fault, p.poll_limit)) return;
        if (tracing && c == 0) trace_stamp(p, 5);  // first stage landed
        if (++s == p.stages) {
            s = 0;
            parity ^= 1u;
        }
        const int sB = s;
        if (two) {
            if (!mbar_wait_bounded(&full[sB], parity, p.fault, p.poll_limit)) return;
            if (++s == p.stages) {
                s = 0;
                parity ^= 1u;
            }
        }
        if (tracing && c + 2 >= n_chunks) trace_stamp(p, 6);  // last stage landed
        const int rowsA = c < walk.n_main ? R : walk.tail_rows;
        const int rowsB = !two ? 0 : (c + 1 < walk.n_main ? R : walk.tail_rows);
        const uint32_t stageA = ring_addr + (uint32_t)sA * p.stage_bytes, stageB = ring_addr + (uint32_t)sB * p.stage_bytes;

        for (int r = warp; r < rowsA || r < rowsB; r += NW) {
            const bool hasA = r < rowsA, hasB = r < rowsB;  // warp-uniform; a missing row is computed on the other's bytes
            const uint32_t in_stage = row_off + (uint32_t)(r - warp) * p.row_bytes;
            const uint32_t rowA = (hasA ? stageA : stageB) + in_stage;
            const uint32_t rowB = (hasB ? stageB : stageA) + in_stage;
            float accA[M_T], accB[M_T];
#pragma unroll
            for (int m = 0; m < M_T; ++m) accA[m] = accB[m] = 0.0f;
#pragma unroll
            for (int i = 0; i < NSB; ++i) {
                if (lane + 32 * i < p.n_super) {  // lanes past the end of K hold no activations: their bytes are another row's
#ifdef JQ_BOUNDS_CHECK
                    {
                        const uint32_t base = smem_u32(gv_dynamic_smem) - (uint32_t)i * (32u * 72u);
                        if (!in_shared(rowA - base, 72, p.smem_total, p.fault) || !in_shared(rowB - base, 72, p.smem_total, p.fault)) continue;
                    }
#endif
                    uint32_t wA[18], wB[18];
#pragma unroll
                    for (int j = 0; j < 9; ++j) {
                        const uint2 a = lds_v2(rowA + (uint32_t)i * (32u * 72u) + 8u * j);
                        const uint2 b = lds_v2(rowB + (uint32_t)i * (32u * 72u) + 8u * j);
                        wA[2 * j] = a.x;
                        wA[2 * j + 1] = a.y;
                        wB[2 * j] = b.x;
                        wB[2 * j + 1] = b.y;
                    }
                    dp4a_slice<M_T>(wA, xq[i], xd[i], xms[i], accA);
                    if (two) dp4a_slice<M_T>(wB, xq[i], xd[i], xms[i], accB);
                }
            }
            // Both rows' lane sums reduced together: the first step leaves row A's halves in lanes 0-15 and row B's
            // in lanes 16-31, the other four run inside the halves.  Per row this adds the same pairs in the same
            // order as a plain xor-16, 8, 4, 2, 1 reduction.
            const bool upper = lane >= 16;
            const int rel = (upper ? c + 1 : c) * R + r;  // row relative to the CTA's first
#pragma unroll
            for (int m = 0; m < M_T; ++m) {
                const float give = upper ? accA[m] : accB[m];
                float v = (upper ? accB[m] : accA[m]) + __shfl_xor_sync(0xFFFFFFFFu, give, 16, 32);
#pragma unroll
                for (int off = 8; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off, 32);
                if (tagged) {
                    if (word_dst != nullptr && m < p.M && (upper ? hasB : hasA)) {
                        unsigned long long *dst = word_dst + (size_t)m * p.gather.N_total + (size_t)rel;
                        if (JQ_IN_EXTENT(p.ext_peer[word_peer], dst, sizeof(unsigned long long), p.fault)) st_word(dst, v, gather_epoch);
                    }
                } else if ((lane & 15) == 0 && m < p.M && (upper ? hasB : hasA)) {
                    if (y_cta != nullptr) {  // the band's staging buffer in shared memory, or a single matrix's output
#ifdef JQ_BOUNDS_CHECK
                        float *dst = y_cta + (size_t)m * y_pitch + (size_t)rel;
                        if (p.gather.world > 0 ? in_shared(dyn_offset(dst), sizeof(float), p.smem_total, p.fault)
                                               : in_extent(p.ext_y[0], dst, sizeof(float), p.fault))
                            *dst = v;
#else
                        y_cta[(size_t)m * y_pitch + (size_t)rel] = v;
#endif
                    } else {
                        store_y(p, m, r_begin + rel, v);
                    }
                }
            }
        }
        if (!resident) {
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&empty[sA]);
                if (two) mbar_arrive(&empty[sB]);
            }
        }
        if (threadIdx.x == 0 && c == 0) trace_fine(p, 4);  // warp 0: first stage pair computed
    }
    if (threadIdx.x == 0) trace_stamp(p, 7);  // warp 0 done
    if (threadIdx.x == (NW - 1) * 32) trace_fine(p, 5);  // last consumer warp done

    if (tagged) {
        // ---- all-gather epilogue, tagged words: each value and the number of this all-gather in one 8-byte store
        // to every rank's buffer.  Nothing follows the stores: no flag, no release, nobody waits here.
        // (the words went out row by row)
        if (threadIdx.x == 0) trace_fine(p, 6);  // warp 0: its stores are issued
        griddep_wait();  // a launch never ends before the one ahead of it
    } else if (p.gather.world > 0) {
        // ---- all-gather epilogue: this CTA's rows of the band go to every rank's buffer ----------
        const GatherArgs &ga = p.gather;
        if (!consumers_meet(meet, lane, p.fault, p.poll_limit)) return;  // the band of this CTA is complete in shared memory
        const int rows_cta = (int)(r_end - r_begin);
        for (int idx = warp; idx < ga.world * p.M; idx += NW) {
            const int q = idx / p.M, m = idx - q * p.M;
            float *dst = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(ga.y_peer[q]) +
                                                   (size_t)(gather_epoch & 1u) * ga.y_stride_bytes) +
                         (size_t)m * ga.N_total + ga.n_offset + r_begin;
            const float *src = ybuf + (size_t)m * p.y_rows;
            for (int i = lane; i < rows_cta; i += 32) {  // 128 contiguous bytes per warp store
                if (JQ_IN_EXTENT(p.ext_peer[q], dst + i, sizeof(float), p.fault)) dst[i] = src[i];
            }
        }
        if (!consumers_meet(meet + 1, lane, p.fault, p.poll_limit)) return;  // all of this CTA's peer stores have been issued
        if (warp == 0) {
            // Tell every rank that this CTA's part of the band is there: a release at system scope (cumulative
            // over the stores that the barrier ordered before it) adding this CTA's share to the count the
            // receiver keeps for this rank.  No CTA waits for another one and nobody waits here; the consumer
            // of the gathered output waits for the counts.
            if (lane < ga.world) {
                asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(ga.flag_peer[lane] + ga.rank), "r"(gather_share())
                             : "memory");
            }
            // bookkeeping off the critical path: the last CTA advances this rank's own step number, which
            // the next launch reads after the kernel boundary
            if (lane == 0) {
                const int prev = atomicAdd(ga.counter, 1);
                if (prev == (int)gridDim.x - 1) {
                    *ga.counter = 0;
                    *ga.epoch_ptr = gather_epoch;
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// mma variant (M <= 8): a stage holds 16 weight rows (one m16 tile), each copied separately so that
// the row distance in shared memory can be padded to an odd multiple of 16 bytes, which makes
// the fragment loads (8 rows x 4 consecutive words) bank-conflict free.  Warp w owns the K slice
// [w*KBW, (w+1)*KBW) of 32-wide blocks for all 16 rows: the activation fragments and scales of
// its slice stay in registers, and per block it issues one mma.m16n8k32 (u8 nibbles x s8
// activations -> exact s32 block sums for 16 rows x 8 columns).  Thread (g = lane/4, t = lane%4)
// feeds the tile with word t of the block: its low nibbles are weights 4t..4t+3 (fragment a0/a1),
// its high nibbles weights 16+4t.. (a2/a3) -- exactly the k ranges the fragment layout asks of it.
// Partial fp32 sums of the NW warps are added in a fixed order through shared memory.
// ------------------------------------------------------------------------------------------------
template <int KBW, int NW>
__global__ void __launch_bounds__((NW + 2) * 32, 1) gemv_mma_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + GV_MAX_STAGES;
    uint64_t *red_full = empty + GV_MAX_STAGES;
    uint64_t *red_empty = red_full + GV_RED_SLOTS;
    uint64_t *x_ready = full + 24;
    float *red = reinterpret_cast<float *>(smem + GV_BAR_BYTES);  // [GV_RED_SLOTS][NW][128]
    uint8_t *xs = smem + GV_BAR_BYTES + GV_RED_SLOTS * NW * 128 * sizeof(float);
    uint8_t *ring = xs + p.x_bytes;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], NW);
        }
        for (int s = 0; s < GV_RED_SLOTS; ++s) {
            mbar_init(&red_full[s], NW);
            mbar_init(&red_empty[s], 1);
        }
        mbar_init(x_ready, NW);
        fence_mbar_init();
    }
    __syncthreads();

    const RowWalk walk = cta_row_walk(p, 16);
    const int n_chunks = walk.n_chunks;

    if (threadIdx.x == 0) trace_stamp(p, 0);  // CTA started
    griddep_launch_dependents();
    if (warp == NW) {  // weight stream, issued by the whole warp
        if (!p.prefetch_early) griddep_wait();
        if (lane == 0) trace_stamp(p, 1);  // weight stream begins
        gemv_producer<true>(p, full, empty, x_ready, ring, lane);
        if (lane == 0) trace_stamp(p, 2);  // last copy issued
        return;
    }
    griddep_wait();
    if (threadIdx.x == 0) trace_stamp(p, 3);  // predecessor finished
    if (warp == NW + 1) {
        // Reducer: adds the NW partial tiles in a fixed order and writes the outputs, so that the
        // compute warps never wait for one another.
        for (int c = 0; c < n_chunks; ++c) {
            const int slot = c % GV_RED_SLOTS;
            const uint32_t round = (uint32_t)(c / GV_RED_SLOTS);
            if (!mbar_wait_bounded(&red_full[slot], round & 1u, p.fault, p.poll_limit)) return;
            int rows;
            const int64_t r0 = walk_stage(walk, c, 16, &rows);
            const float *src = red + (size_t)slot * NW * 128;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int idx = lane + 32 * j;  // idx = row * 8 + col
                float v = 0.0f;
#pragma unroll
                for (int w = 0; w < NW; ++w) v += src[w * 128 + idx];
                const int row = idx >> 3, col = idx & 7;
                if (row < rows && col < p.M) store_y(p, col, r0 + row, v);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&red_empty[slot]);
        }
        if (lane == 0) trace_stamp(p, 7);  // last outputs written
        return;
    }

    stage_activations<NW>(p, xs, x_ready, warp, lane);
    if (threadIdx.x == 0) trace_stamp(p, 4);  // activations staged

    const int g = lane >> 2, t = lane & 3;
    const int nb = p.K / QK;
    const int kb0 = warp * KBW;
    const uint32_t xs_addr = smem_u32(xs);
    const uint32_t ring_addr = smem_u32(ring);
    // B fragments (column g) and scales (columns 2t, 2t+1) of this warp's K slice.
    uint32_t xb0[KBW], xb1[KBW];
    float xd0[KBW], xd1[KBW], xm0[KBW], xm1[KBW];
#pragma unroll
    for (int j = 0; j < KBW; ++j) {
        const int kb = kb0 + j;
        xb0[j] = xb1[j] = 0u;
        xd0[j] = xd1[j] = xm0[j] = xm1[j] = 0.0f;
        if (kb < nb) {
            const int ks = kb >> 2, sub = kb & 3;
            if (g < p.M) {
                const uint32_t b = xs_addr + (uint32_t)g * p.x_pitch + (uint32_t)ks * Q8_BYTES + Q8_QS_OFFSET + sub * QK;
                xb0[j] = lds_u32(b + 4u * t);
                xb1[j] = lds_u32(b + 4u * (t + 4));
            }
            if (2 * t < p.M) {
                const uint32_t ds = lds_u32(xs_addr + (uint32_t)(2 * t) * p.x_pitch + (uint32_t)ks * Q8_BYTES + 4u * sub);
                xd0[j] = half_bits_to_float(ds & 0xFFFFu);
                xm0[j] = -8.0f * half_bits_to_float(ds >> 16);
            }
            if (2 * t + 1 < p.M) {
                const uint32_t ds = lds_u32(xs_addr + (uint32_t)(2 * t + 1) * p.x_pitch + (uint32_t)ks * Q8_BYTES + 4u * sub);
                xd1[j] = half_bits_to_float(ds & 0xFFFFu);
                xm1[j] = -8.0f * half_bits_to_float(ds >> 16);
            }
        }
    }

    const int zero4[4] = {0, 0, 0, 0};

    for (int c = 0; c < n_chunks; ++c) {
        const int s = c % p.stages;
        const uint32_t round = (uint32_t)(c / p.stages);
        if (!mbar_wait_bounded(&full[s], round & 1u, p.fault, p.poll_limit)) return;
        if (threadIdx.x == 0 && c == 0) trace_stamp(p, 5);  // first stage landed
        if (threadIdx.x == 0 && c == n_chunks - 1) trace_stamp(p, 6);  // last stage landed
        const uint32_t stage = ring_addr + (uint32_t)s * p.stage_bytes;

        float acc[4] = {0.f, 0.f, 0.f, 0.f};  // (row g, col 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1)
        const uint32_t row_lo = stage + (uint32_t)g * p.row_stride;
        const uint32_t row_hi = stage + (uint32_t)(g + 8) * p.row_stride;
#pragma unroll
        for (int jp = 0; jp < KBW / 2; ++jp) {
            const int kbe = kb0 + 2 * jp;  // even block, 4-byte aligned start at byte 18*kbe
            if (kbe < nb) {
                uint32_t a_even[4], a_odd[4];
                float d_even[2], d_odd[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t pr = (h == 0 ? row_lo : row_hi) + (uint32_t)kbe * Q4_BYTES;
                    const uint32_t u0 = lds_u32(pr + 4u * t), u1 = lds_u32(pr + 4u * t + 4u), u2 = lds_u32(pr + 4u * t + 20u);
                    const uint32_t we = __funnelshift_r(u0, u1, 16);  // word t of the even block
                    a_even[h] = we & MASK4;              // a0 / a1: weights 4t..4t+3
                    a_even[2 + h] = (we >> 4) & MASK4;   // a2 / a3: weights 16+4t..
                    a_odd[h] = u2 & MASK4;
                    a_odd[2 + h] = (u2 >> 4) & MASK4;
                    d_even[h] = half_bits_to_float(lds_u16(pr));
                    d_odd[h] = half_bits_to_float(lds_u16(pr + Q4_BYTES));
                }
                int ce[4], co[4];
                {
                    const uint32_t bfrag[2] = {xb0[2 * jp], xb1[2 * jp]};
                    mma_u8s8_16832(ce, a_even, bfrag, zero4);
                }
                acc[0] = fmaf(d_even[0], fmaf((float)ce[0], xd0[2 * jp], xm0[2 * jp]), acc[0]);
                acc[1] = fmaf(d_even[0], fmaf((float)ce[1], xd1[2 * jp], xm1[2 * jp]), acc[1]);
                acc[2] = fmaf(d_even[1], fmaf((float)ce[2], xd0[2 * jp], xm0[2 * jp]), acc[2]);
                acc[3] = fmaf(d_even[1], fmaf((float)ce[3], xd1[2 * jp], xm1[2 * jp]), acc[3]);
                if (kbe + 1 < nb) {
                    const uint32_t bfrag[2] = {xb0[2 * jp + 1], xb1[2 * jp + 1]};
                    mma_u8s8_16832(co, a_odd, bfrag, zero4);
                    acc[0] = fmaf(d_odd[0], fmaf((float)co[0], xd0[2 * jp + 1], xm0[2 * jp + 1]), acc[0]);
                    acc[1] = fmaf(d_odd[0], fmaf((float)co[1], xd1[2 * jp + 1], xm1[2 * jp + 1]), acc[1]);
                    acc[2] = fmaf(d_odd[1], fmaf((float)co[2], xd0[2 * jp + 1], xm0[2 * jp + 1]), acc[2]);
                    acc[3] = fmaf(d_odd[1], fmaf((float)co[3], xd1[2 * jp + 1], xm1[2 * jp + 1]), acc[3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);  // the stage's bytes have been consumed

        // hand the partial 16 x 8 tile to the reducer warp
        const int slot = c % GV_RED_SLOTS;
        const uint32_t rround = (uint32_t)(c / GV_RED_SLOTS);
        if (rround > 0 && !mbar_wait_bounded(&red_empty[slot], (rround - 1) & 1u, p.fault, p.poll_limit)) return;
        float *mine = red + ((size_t)slot * NW + warp) * 128;
        *reinterpret_cast<float2 *>(&mine[g * 8 + 2 * t]) = make_float2(acc[0], acc[1]);
        *reinterpret_cast<float2 *>(&mine[(g + 8) * 8 + 2 * t]) = make_float2(acc[2], acc[3]);
        __syncwarp();
        if (lane == 0) mbar_arrive(&red_full[slot]);
    }
}

// ---- host side ------------------------------------------------------------------------------------
// Raises a kernel's dynamic shared-memory limit and asks for the largest shared-memory carve-out, so that two
// CTAs of ~110 KB fit one SM.
int ensure_smem_attr(void (*kernel)(const GemvParams), int bytes) {
    return ensure_dynamic_smem(reinterpret_cast<const void *>(kernel), bytes, true);
}

inline uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

// Launch with programmatic stream serialization: the kernel may be scheduled while its
// predecessor in the stream drains; it orders itself with griddepcontrol.wait.
int launch_pdl(void (*kernel)(const GemvParams), int grid, int block, int smem, cudaStream_t st, const GemvParams &p) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)block);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    JQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p));
    return JQ_OK;
}

int fast_path_ok(const void *d_w, const void *d_xq, const float *d_x_f32, int64_t K, int64_t N) {
    if (K % 256 != 0) return set_error(JQ_ERR_UNSUPPORTED, "streaming GEMV needs K %% 256 == 0 (K = %lld)", (long long)K);
    if (((uintptr_t)d_w & 15u) != 0) return set_error(JQ_ERR_UNSUPPORTED, "streaming GEMV needs 16-byte aligned weights");
    if (d_x_f32 != nullptr && ((uintptr_t)d_x_f32 & 15u) != 0)
        return set_error(JQ_ERR_UNSUPPORTED, "streaming GEMV needs 16-byte aligned activations");
    if (d_x_f32 == nullptr && ((uintptr_t)d_xq & 15u) != 0)
        return set_error(JQ_ERR_UNSUPPORTED, "streaming GEMV needs 16-byte aligned Q8_1 blocks");
    if (K > (1 << 20) || N > (int64_t)1 << 31) return set_error(JQ_ERR_UNSUPPORTED, "shape too large for the streaming GEMV");
    return JQ_OK;
}

template <int M_T, int NSB, int NW, int MINB>
int run_dp4a(cudaStream_t st, GemvParams &p, const DeviceCaps &caps) {
    // MINB CTAs share an SM: each gets an equal slice of its shared memory (1 KB per CTA is reserved)
    const int64_t budget = min((int64_t)caps.smem_optin, (int64_t)caps.smem_per_sm / MINB - 1024);
    p.rows_per_stage = MINB > 1 ? 8 : NW;
    p.row_stride = p.row_bytes;
    p.y_bytes = 0;
    p.y_rows = 0;
    if (p.gather.world > 0) {
        // rows per CTA are at most ceil(N / grid) + 1 and the grid is at least min(SMs * MINB, N / rows_per_stage)
        const int64_t min_grid = max((int64_t)1, min((int64_t)caps.sm_count * MINB, (p.N + p.rows_per_stage - 1) / p.rows_per_stage));
        p.y_rows = (uint32_t)((p.N + min_grid - 1) / min_grid + 1);
        p.y_bytes = align_up((uint32_t)p.M * p.y_rows * 4u, 128);
    }
    for (;;) {
        p.stage_bytes = align_up((uint32_t)p.rows_per_stage * p.row_bytes, 128);
        const int64_t avail = budget - GV_BAR_BYTES - p.x_bytes - p.y_bytes;
        p.stages = (int)min((int64_t)GV_MAX_STAGES, avail / p.stage_bytes);
        if (p.stages >= 3 || p.rows_per_stage == 1) break;
        p.rows_per_stage = p.rows_per_stage > 2 ? p.rows_per_stage / 2 : 1;
    }
    if (p.stages < 2) return set_error(JQ_ERR_UNSUPPORTED, "row of %u bytes does not fit the shared-memory ring", p.row_bytes);
    const int smem = GV_BAR_BYTES + (int)p.y_bytes + (int)p.x_bytes + p.stages * (int)p.stage_bytes;
#ifdef JQ_BOUNDS_CHECK
    p.smem_total = (uint32_t)smem;
#endif
    auto kernel = p.gather.ticket != nullptr ? gemv_dp4a_kernel<M_T, NSB, NW, MINB, true> : gemv_dp4a_kernel<M_T, NSB, NW, MINB, false>;
    if (int rc = ensure_smem_attr(kernel, smem)) return rc;
    const int64_t want = (p.N + p.rows_per_stage - 1) / p.rows_per_stage;
    const int grid = (int)min((int64_t)caps.sm_count * MINB, max((int64_t)1, want));
    p.rows_q = (uint32_t)(p.N / grid);
    p.rows_r = (uint32_t)(p.N % grid);
    return launch_pdl(kernel, grid, (NW + 1) * 32, smem, st, p);
}

template <int KBW, int NW>
int run_mma(cudaStream_t st, GemvParams &p, const DeviceCaps &caps) {
    p.rows_per_stage = 16;
    // rows 16*odd bytes apart: 8 rows x 4 words hit 32 distinct banks
    p.row_stride = p.row_bytes + ((p.row_bytes / 16) % 2 == 0 ? 16 : 0);
    // the last warps may read a few blocks past the row end (their results are discarded)
    p.stage_bytes = align_up(16 * p.row_stride + KBW * Q4_BYTES + 64, 128);
    const int red_bytes = GV_RED_SLOTS * NW * 128 * (int)sizeof(float);
    const int64_t avail = (int64_t)caps.smem_optin - GV_BAR_BYTES - red_bytes - p.x_bytes;
    p.stages = (int)min((int64_t)GV_MAX_STAGES, avail / p.stage_bytes);
    if (p.stages < 2) return set_error(JQ_ERR_UNSUPPORTED, "16 rows of %u bytes do not fit the shared-memory ring", p.row_bytes);
    const int smem = GV_BAR_BYTES + red_bytes + (int)p.x_bytes + p.stages * (int)p.stage_bytes;
#ifdef JQ_BOUNDS_CHECK
    p.smem_total = (uint32_t)smem;
#endif
    auto kernel = gemv_mma_kernel<KBW, NW>;
    if (int rc = ensure_smem_attr(kernel, smem)) return rc;
    const int64_t want = (p.N + 15) / 16;
    const int grid = (int)min((int64_t)caps.sm_count, max((int64_t)1, want));
    p.rows_q = (uint32_t)(p.N / grid);
    p.rows_r = (uint32_t)(p.N % grid);
    return launch_pdl(kernel, grid, (NW + 2) * 32, smem, st, p);
}

int fill_params(GemvParams &p, const void *d_w, const void *d_xq, const float *d_x_f32, void *d_xq_out,
                float *d_y, int64_t K, int64_t N, int64_t M, int order, int s_mode) {
    p.n_mats = 1;
    p.w = static_cast<const uint8_t *>(d_w);
    p.xq = d_x_f32 ? nullptr : static_cast<const uint8_t *>(d_xq);
    p.x_f32 = d_x_f32;
    p.xq_out = d_x_f32 ? static_cast<uint8_t *>(d_xq_out) : nullptr;
    p.y = d_y;
    p.fault = device_fault_ptr();
    p.N = N;
    p.K = (int)K;
    p.M = (int)M;
    p.order = order;
    p.s_mode = s_mode;
    p.n_super = (int)(K / SUPER);
    p.row_bytes = (uint32_t)(K / QK * Q4_BYTES);
    // activation rows 16*odd bytes apart in shared memory: 8 columns x 4 consecutive words hit 32 banks
    p.x_pitch = (uint32_t)p.n_super * Q8_BYTES + (p.n_super % 2 == 0 ? 16u : 0u);
    p.x_bytes = align_up((uint32_t)M * p.x_pitch, 128);
    p.prefetch_early = option_value(JQ_OPT_STATIC_WEIGHTS) != 0;
    p.trace = static_cast<unsigned long long *>(next_trace_slot());
    // Ahead of the previous kernel's end only two stages are requested (more would delay the
    // activation loads that follow the wait).
    p.early_stages = p.prefetch_early ? 2 : (1 << 30);
    p.poll_limit = wait_poll_limit();
#ifdef JQ_BOUNDS_CHECK
    const unsigned long long blocks_bytes = (unsigned long long)M * (unsigned long long)p.n_super * Q8_BYTES;
    p.ext_w[0] = make_extent(d_w, (unsigned long long)N * p.row_bytes);
    p.ext_y[0] = make_extent(d_y, (unsigned long long)M * (unsigned long long)N * sizeof(float));
    p.ext_x = d_x_f32 ? make_extent(d_x_f32, (unsigned long long)M * (unsigned long long)K * sizeof(float)) : make_extent(d_xq, blocks_bytes);
    p.ext_xq_out = make_extent(p.xq_out, blocks_bytes);
#endif

    return JQ_OK;
}

}  // namespace

namespace {
int apply_multi(GemvParams &p, const MultiMat *multi, const GatherArgs *gather) {
    if (multi == nullptr) return JQ_OK;
    if (multi->n < 1 || multi->n > GV_MAX_MATS) return set_error(JQ_ERR_INVALID_ARG, "1 to %d weight matrices per launch", GV_MAX_MATS);
    if (gather != nullptr) return set_error(JQ_ERR_UNSUPPORTED, "the all-gather epilogue takes a single weight matrix");
    p.n_mats = multi->n;
    p.mat_begin[0] = 0;
    for (int i = 0; i < multi->n; ++i) {
        if (((uintptr_t)multi->w[i] & 15u) != 0) return set_error(JQ_ERR_UNSUPPORTED, "streaming GEMV needs 16-byte aligned weights");
        p.w_mat[i] = static_cast<const uint8_t *>(multi->w[i]);
        p.y_mat[i] = multi->y[i];
        p.mat_begin[i + 1] = p.mat_begin[i] + multi->rows[i];
#ifdef JQ_BOUNDS_CHECK
        p.ext_w[i] = make_extent(multi->w[i], (unsigned long long)multi->rows[i] * p.row_bytes);
        p.ext_y[i] = make_extent(multi->y[i], (unsigned long long)p.M * (unsigned long long)multi->rows[i] * sizeof(float));
#endif
    }
    if (p.mat_begin[multi->n] != p.N) return set_error(JQ_ERR_INVALID_ARG, "row counts of the matrices do not add up to N");
    p.w = p.w_mat[0];
    p.y = p.y_mat[0];
    return JQ_OK;
}
}  // namespace

int launch_allgather_wait(cudaStream_t st, const uint32_t *d_flags, int world, const uint32_t *d_epoch) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    JQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, allgather_wait_kernel, d_flags, world, d_epoch, device_fault_ptr(), wait_poll_limit()));
    return JQ_OK;
}

int launch_allgather_tagged_read(cudaStream_t st, const unsigned long long *d_words, uint64_t stride_bytes, int64_t M,
                                 int64_t N_total, const unsigned long long *d_ticket, float *d_out) {
    const int64_t n_words = M * N_total;
    DeviceCaps caps;
    if (int rc = device_caps(&caps)) return rc;
    const int grid = (int)max((int64_t)1, min((int64_t)caps.sm_count * 4, (n_words / 2 + 255) / 256));
    allgather_tagged_read_kernel<<<grid, 256, 0, st>>>(d_words, stride_bytes, n_words, d_ticket, d_out, device_fault_ptr(),
                                                       wait_poll_limit());
    JQ_CUDA_TRY(cudaGetLastError());
    return JQ_OK;
}

int launch_gemv_dp4a(cudaStream_t st, const void *d_w, const void *d_xq, const float *d_x_f32, void *d_xq_out,
                     float *d_y, int64_t K, int64_t N, int64_t M, int order, int s_mode, const GatherArgs *gather,
                     const MultiMat *multi) {
    if (multi != nullptr) d_w = multi->w[0];
    if (M < 1 || M > 2) return set_error(JQ_ERR_UNSUPPORTED, "dp4a GEMV handles M <= 2 (M = %lld)", (long long)M);
    if (int rc = fast_path_ok(d_w, d_xq, d_x_f32, K, N)) return rc;
    if (N == 0) return JQ_OK;
    DeviceCaps caps;
    if (int rc = device_caps(&caps)) return rc;
    GemvParams p{};
    fill_params(p, d_w, d_xq, d_x_f32, d_xq_out, d_y, K, N, M, order, s_mode);
    if (gather != nullptr) {
        p.gather = *gather;
#ifdef JQ_BOUNDS_CHECK
        const unsigned long long elem = gather->ticket != nullptr ? sizeof(unsigned long long) : sizeof(float);
        for (int q = 0; q < gather->world; ++q)
            p.ext_peer[q] = make_extent(gather->y_peer[q], gather->y_stride_bytes + (unsigned long long)M * (unsigned long long)gather->N_total * elem);
        if (gather->x_words != nullptr)
            p.ext_x_words = make_extent(gather->x_words, gather->x_stride_bytes + (unsigned long long)M * (unsigned long long)gather->x_row_words * 8ull);
#endif
    }
    if (int rc = apply_multi(p, multi, gather)) return rc;
    // Ready Q8_1 blocks whose columns are contiguous come in by bulk copy, queued by the producer thread ahead of
    // the rest of its weight stream, straight to their place in shared memory.  fp32 activations are loaded by
    // the consumer warps themselves (each its own pair of blocks, quantized in registers): their loads take the
    // load/store path and overtake the weight copies already queued, a bulk copy behind two stages of weights
    // does not.  Medians of 7 x 128 graph-replayed steps, cold weights, stages requested ahead of the previous
    // kernel's end 0 / 1 / 2 / 3: cfg2 fused, loads by the warps 7.19 / 6.88 / 6.19 / 6.66 us, by bulk copy
    // 7.16 / 7.39 / 7.36 / 7.41 us; cfg2 ready blocks by bulk copy 7.01 / 6.25 / 6.03 / 6.41 us; K = 11008 ready
    // blocks, bulk copy 9.34 / 8.18 / 7.63 / 7.98 us, loads by the warps 10.45 / 9.89 / 8.85 / 8.83 us.
    const bool x_words = p.gather.ticket != nullptr && p.gather.x_words != nullptr;
    if (p.x_f32 == nullptr && !x_words && (order == JQ_ORDER_COL_KSUPER || M == 1)) p.x_copy_bytes = (uint32_t)(M * p.n_super * Q8_BYTES);
    p.prefetch_early = option_value(JQ_OPT_STATIC_WEIGHTS) != 0;
    p.early_stages = p.prefetch_early ? 2 : (p.x_copy_bytes != 0 ? 0 : (1 << 30));
    // Activations that arrive as tagged words: two stages ahead as well.  Requesting the whole ring while the words
    // are still in flight delays the polling loads behind the weight traffic (two GPUs, every CTA's output sampled:
    // 9.15 us per step with two stages ahead, 10.1 with one, 9.6 with three, 10.4 with the whole ring).
    if (x_words) p.early_stages = 2;
    const int nsb = (p.n_super + 31) / 32;
    if (M == 1) {
        switch (nsb) {
            case 1:
                // Quantizing in the prologue is repeated by every CTA: one CTA of 16 warps per SM halves
                // that cost.  With ready-made Q8_1 input two CTAs of 8 warps per SM overlap better.
                // (20 consumer warps instead of 16 fit the register file and change nothing: 6.22 us either way)
                if (p.x_f32 != nullptr || x_words) return run_dp4a<1, 1, 16, 1>(st, p, caps);
                return run_dp4a<1, 1, 8, 2>(st, p, caps);
            case 2:
                // long slabs stream better with 12 consumer warps (K = 8192, N = 28672 on ready blocks: 22.9 -> 21.6 us),
                // short ones start faster with 8 (N = 4096: 6.56 against 7.01 us)
                if (N >= 16384) return run_dp4a<1, 2, 12, 1>(st, p, caps);
                return run_dp4a<1, 2, 8, 1>(st, p, caps);
            case 3: return run_dp4a<1, 3, 7, 1>(st, p, caps);  // (9 consumer warps: K = 11008, N = 4096 7.3 -> 9.6 us)
            case 4: return run_dp4a<1, 4, 7, 1>(st, p, caps);
            default: break;
        }
    } else {
        switch (nsb) {
            case 1:
                // two columns keep 64 activation words per lane: 12 + 1 warps of 128 registers fit the register file.
                // cfg2, medians of 5 x 128 steps, consumer warps 8 / 10 / 12 / 14: fused linear 9.41 / 9.12 / 8.71 /
                // 9.10 us, multiply on ready blocks 8.42 / 8.32 / 8.58 / 9.00 us
                if (p.x_f32 != nullptr) return run_dp4a<2, 1, 12, 1>(st, p, caps);
                return run_dp4a<2, 1, 10, 1>(st, p, caps);
            case 2: return run_dp4a<2, 2, 7, 1>(st, p, caps);
            default: break;
        }
    }
    return set_error(JQ_ERR_UNSUPPORTED, "dp4a GEMV: K = %lld too long to keep %lld activation columns in registers",
                     (long long)K, (long long)M);
}

int launch_gemv_mma(cudaStream_t st, const void *d_w, const void *d_xq, const float *d_x_f32, void *d_xq_out,
                    float *d_y, int64_t K, int64_t N, int64_t M, int order, int s_mode, const MultiMat *multi) {
    if (multi != nullptr) d_w = multi->w[0];
    if (M < 1 || M > 8) return set_error(JQ_ERR_UNSUPPORTED, "mma GEMV handles M <= 8 (M = %lld)", (long long)M);
    if (int rc = fast_path_ok(d_w, d_xq, d_x_f32, K, N)) return rc;
    if (N == 0) return JQ_OK;
    DeviceCaps caps;
    if (int rc = device_caps(&caps)) return rc;
    GemvParams p{};
    fill_params(p, d_w, d_xq, d_x_f32, d_xq_out, d_y, K, N, M, order, s_mode);
    if (d_x_f32 != nullptr) {
        // quantizing in the prologue: the stream starts at the wait for the previous kernel, where it overlaps the
        // quantization (cfg2 M = 4: 10.8 us; 11.0 us with two stages requested earlier)
        p.prefetch_early = 0;
        p.early_stages = 1 << 30;
    }
    // (ready blocks by the producer's bulk copies, as in the dp4a kernel, were measured slower here: cfg2 M = 8 on
    // ready blocks 10.5 against 9.3 us with the warps' own loads)
    if (int rc = apply_multi(p, multi, nullptr)) return rc;
    const int nb = (int)(K / QK);
    if (nb <= 8 * 8) return run_mma<8, 8>(st, p, caps);
    if (nb <= 16 * 8) return run_mma<8, 16>(st, p, caps);
    if (nb <= 16 * 12) return run_mma<12, 16>(st, p, caps);
    return set_error(JQ_ERR_UNSUPPORTED, "mma GEMV: K = %lld too long to keep the activation fragments in registers",
                     (long long)K);
}

}  // namespace jq
