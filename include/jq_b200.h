/*
 * jq_b200 -- C ABI of the B200 (sm_100a) Q4_0 x Q8_1 quantized-linear path.
 *
 * A drop-in for the two quantization operators of JJJetson_Ops:
 *   src/cuda/q8_1.cu            (activation quantizer, fp32 -> block_q8_1_mmq)
 *   src/cuda/mm_q4_0_q8_1.cu    (Q4_0 weights x Q8_1 activations -> fp32)
 * Every entry point is extern "C", takes plain pointers and sizes, returns a jq_status
 * (never exits the process, unlike CUDA_CHECK in the reference's include/cuda_utils.h:10-28)
 * and leaves a human-readable message in jq_last_error() when it fails.
 *
 * Data layouts are the reference's, byte for byte:
 *   Q4_0 block  (mm_q4_0_q8_1.cu:35-38): 18 bytes = fp16 d, then 16 bytes; byte j holds
 *               weight j in its low nibble and weight j+16 in its high nibble;
 *               value = (q - 8) * d.  W is N rows of K/32 consecutive blocks.
 *   Q8_1 block  (q8_1.cu:14-18, block_q8_1_mmq): 144 bytes = 4 x (fp16 d, fp16 s), then
 *               128 int8; four 32-value groups share one block.
 *   X is M rows of K floats (K fastest); Y is M rows of N floats (y[m*N + n],
 *   mm_q4_0_q8_1.cu:286).
 *
 * "Device" entry points are asynchronous on the given stream, allocate nothing and never
 * synchronise.  "Host" entry points take host pointers and do the allocate / copy / launch /
 * copy back / free round trip the reference's *_host style wrappers do.
 */
#ifndef JQ_B200_H_
#define JQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum jq_status {
    JQ_OK = 0,
    JQ_ERR_INVALID_ARG = 1, /* null pointer, negative size, unknown enum value */
    JQ_ERR_SHAPE = 2,       /* K not a multiple of 32 (quantize) or 128 (multiply) */
    JQ_ERR_ALIGN = 3,       /* a pointer lacks the alignment its layout needs */
    JQ_ERR_CUDA = 4,        /* a CUDA runtime call failed; jq_last_error() names it */
    JQ_ERR_UNSUPPORTED = 5, /* no kernel for this request on this device */
    JQ_ERR_TIMEOUT = 6,     /* a bounded device-side wait ran out (see jq_device_fault) */
    JQ_ERR_TOO_LARGE = 7    /* the request exceeds a stated fixed capacity */
} jq_status;

/* Order of the 144-byte activation blocks in memory for M > 1.  The two reference kernels
 * disagree: the quantizer writes block (k/128) * M + m (q8_1.cu:84-86, pinned by
 * tests/test_q8_1.py:33) while the multiply reads block m * (K/128) + k/128
 * (mm_q4_0_q8_1.cu:230,246).  They coincide for M == 1.  Both are supported. */
typedef enum jq_q8_order {
    JQ_ORDER_KSUPER_COL = 0, /* what q8_1() writes */
    JQ_ORDER_COL_KSUPER = 1  /* what mat_mul_q4_0_q8_1_device() reads */
} jq_q8_order;

/* Meaning of the second fp16 of each (d, s) pair. */
typedef enum jq_s_mode {
    JQ_S_SUM_X = 0,  /* s = fp16(sum of the 32 input floats): the reference, q8_1.cu:62-68,102 */
    JQ_S_D_SUM_Q = 1 /* s = fp16(fp16(d) * sum of the 32 int8): makes d4*(d8*sumi - 8*s) equal
                        dequantise-then-matmul up to fp16 rounding of s */
} jq_s_mode;

/* Kernel families of the multiply; JQ_KERNEL_AUTO picks by shape. */
typedef enum jq_kernel {
    JQ_KERNEL_AUTO = 0,
    JQ_KERNEL_GENERIC = 1,   /* any shape, plain loads; the safety net */
    JQ_KERNEL_GEMV_DP4A = 2, /* M <= 2: bulk-copy ring, dp4a, warp per row */
    JQ_KERNEL_GEMV_MMA = 3,  /* M <= 8: bulk-copy ring, int8 mma per block, K split over warps */
    JQ_KERNEL_GEMM_MMA = 4,  /* M > 8: tiled int8 mma.sync GEMM with per-block rescale */
    JQ_KERNEL_GEMM_TC = 5,   /* M > 8, K % 256 == 0: tcgen05.mma.kind::i8 GEMM, TMEM accumulators drained per block */
    JQ_KERNEL_GEMM_F16 = 6   /* M > 8, K % 256 == 0: operands dequantised to fp16, tcgen05.mma.kind::f16, fp32 accumulation.
                                Rounds every scaled operand to fp16 (about 2e-4 of the largest output); what
                                JQ_KERNEL_AUTO takes for 64 columns and more unless JQ_OPT_PREFILL_EXACT is set */
} jq_kernel;

/* Process-wide switches. */
typedef enum jq_option {
    /* 1: the caller promises that weight buffers are never written by work queued just ahead of a
     * multiply on the same stream (true for inference: weights are uploaded once).  The decode
     * kernels then start streaming weights while the previous kernel on the stream is still
     * draining, before they wait for it; activations and outputs are always ordered normally.
     * 0 (default): the weight stream, too, waits for the previous kernel. */
    JQ_OPT_STATIC_WEIGHTS = 0,
    /* What JQ_KERNEL_AUTO runs for prefill batches (64 activation columns and more).
     * 0 (default): the fp16-operand tcgen05 GEMM (JQ_KERNEL_GEMM_F16) when its shape rules hold (K % 256 == 0,
     * 16-byte aligned buffers), else an exact-integer kernel.  It is 2.5x as fast as the integer GEMMs; every
     * scaled operand is rounded to fp16 once, so results differ from the reference formula by about 2e-4 of the
     * largest output (inside the 1e-3 bound against dequantise-then-matmul that the path is held to), and the
     * activations must fit fp16's range.
     * 1: every automatic choice is an exact-integer kernel (int32 block sums as the reference forms them, fp32
     * results within 1e-6 of the reference formula).  Decode batches (fewer than 64 columns) always are. */
    JQ_OPT_PREFILL_EXACT = 1,
    /* Number of polls after which a bounded device-side wait (for a bulk copy, or for the bands of an
     * all-gather) gives up, sets the fault word read by jq_device_fault() and lets its kernel return.
     * It applies to the decode kernels' waits and to jq_allgather_wait_device.
     * 0 (default): 2^22 polls, far beyond any wait of a healthy run.  The value is read when a kernel is
     * launched.  There is no counterpart in the reference (its kernels never wait on one another). */
    JQ_OPT_WAIT_POLL_LIMIT = 2,
    JQ_OPT_COUNT_ = 3
} jq_option;
int jq_set_option(int option, int value);
int jq_get_option(int option, int *value_out);

/* Tracing aid for the decode kernels: after jq_trace_enable(d_buf, n), each of the next n launches
 * of a streaming GEMV writes 8 device-clock timestamps (ns, %globaltimer) per CTA into its own
 * 512 x 8 x uint64 slice of d_buf (CTA start, weight stream begins, last copy issued, predecessor
 * finished, activations staged, first stage landed, last stage landed, done).  d_buf must hold
 * n * 32768 bytes and be zeroed by the caller.  jq_trace_enable(NULL, 0) switches it off.
 * The tcgen05 GEMM uses its slice differently: SM clock stamps of CTA (0,0) for the first 128
 * blocks of K, four groups of 128 rows x 8 columns (accumulator seen complete / previous block
 * accumulated / buffer handed back, one column per drain warp; then MMA issue time in column 0
 * and stage publication per producer warp in columns 1-3).  The fp16-operand GEMM stamps SM clocks
 * of CTA (0,0) for the first 64 stages: rows 0-63 weight warp 0, rows 64-127 activation warp 4 (the
 * even stages, which the first producer group converts; columns: loop top, raw bytes landed, -,
 * operand stage free, converted, published), rows 128-191 the MMA thread (stage seen full, MMAs and
 * commit issued). */
int jq_trace_enable(void *d_buf, int64_t n_launches);

const char *jq_status_string(int status);
/* Message of the last failure on the calling thread ("" if none). */
const char *jq_last_error(void);
int jq_version(void);

/* Bytes of block_q8_1_mmq storage for M rows of K values: M * ceil(K/128) * 144
 * (the n_blocks rule of q8_1.cu:160). */
size_t jq_q8_1_bytes(int64_t K, int64_t M);
/* Bytes of Q4_0 storage for N rows of K values: N * K/32 * 18. */
size_t jq_q4_0_bytes(int64_t N, int64_t K);

/* ---- device entry points -------------------------------------------------------------- */

/* Replaces the kernel launch inside q8_1() (q8_1.cu:172-183, quantize_q8_1_kernel :20-104).
 * d_x: M*K floats.  d_xq: jq_q8_1_bytes(K, M) bytes, 16-byte aligned.  K % 32 == 0; groups of a
 * trailing partial 128-block are zero-filled.  An all-zero group stores d = 0 (the reference
 * stores fp16(1/0) = +inf there, which poisons the multiply with NaN). */
int jq_quantize_q8_1_device(void *stream, const float *d_x, void *d_xq, int64_t K, int64_t M,
                            int order, int s_mode);

/* Replaces mat_mul_q4_0_q8_1_device (mm_q4_0_q8_1.cu:394-398, contract :382-392).
 * d_w: N*K/32 Q4_0 blocks.  d_xq: activations already in block_q8_1_mmq form, in `order`.
 * d_y: M*N floats.  K % 128 == 0 (the check of mm_q4_0_q8_1.cu:335-340). */
int jq_mul_mat_q4_0_q8_1_device(void *stream, const void *d_w, const void *d_xq, float *d_y,
                                int64_t K, int64_t N, int64_t M, int order);

/* Same, with the kernel family forced (for tests and benchmarks). */
int jq_mul_mat_q4_0_q8_1_device_ex(void *stream, const void *d_w, const void *d_xq, float *d_y,
                                   int64_t K, int64_t N, int64_t M, int order, int kernel);

/* Quantize + multiply in one call: what mat_mul_q4_0_q8_1 (mm_q4_0_q8_1.cu:318-380) does
 * between its copies.  d_x: M*K floats.  d_ws: jq_q8_1_bytes(K, M) bytes of scratch that
 * receives the quantized activations (JQ_ORDER_COL_KSUPER) as a side effect, like the
 * reference's quant_workspace (:352).  For M <= 8 the quantization runs inside the multiply
 * kernel's prologue. */
int jq_linear_q4_0_device(void *stream, const void *d_w, const float *d_x, void *d_ws, float *d_y,
                          int64_t K, int64_t N, int64_t M, int s_mode);

/* Several linears that share their input, in one call: the separate q / k / v projections
 * (src/engine/transformer_runner.cpp:214-216) or gate / up (:319-321) of the reference's layer,
 * whose weights live in separate buffers (src/model/transformer_model.h:13-23).  Matrix i has
 * N[i] rows of K / 32 Q4_0 blocks and writes d_y[i] = [M][N[i]].  Give either d_x (fp32, then
 * d_ws receives the Q8_1 blocks as in jq_linear_q4_0_device) or d_xq (blocks in
 * JQ_ORDER_COL_KSUPER order, e.g. from jq_rms_norm_q8_1_device; d_ws unused).  For M <= 8 and
 * K within the decode kernels' reach the matrices are treated as one matrix of sum(N) rows and
 * multiplied by a single launch, with the same results as separate calls; other shapes quantize
 * once and run one multiply per matrix.  No counterpart in the reference (its linears are
 * separate cuBLAS calls). */
int jq_linear_q4_0_multi_device(void *stream, int n_mats, const void *const *d_w, const int64_t *N,
                                float *const *d_y, const float *d_x, const void *d_xq, void *d_ws,
                                int64_t K, int64_t M, int s_mode);

/* ---- producers of the quantized linear's input ---------------------------------------------
 * The two kernels that run just ahead of a linear in the reference's transformer layer
 * (src/engine/transformer_runner.cpp:208-216, 311-328), with the Q8_1 quantizer folded in: the
 * linear that follows then takes d_xq through jq_mul_mat_q4_0_q8_1_device and no fp32
 * activation has to be written, re-read and quantized by a launch of its own.  The fp32 values
 * are computed in the reference's own operation order, so both the fp32 outputs and the blocks
 * equal "reference kernel, then quantize_q8_1" bit for bit.
 *
 * jq_rms_norm_q8_1_device: rms_norm_fused_add_forward_device (src/cuda/rms_norm_fused_add.cu:
 * 85-105; z = input + residual, residual <- z, normed = z * rsqrt(mean(z^2) + eps) * weight)
 * when d_residual is given, rms_norm_forward_device (src/cuda/rms_norm.cu) when it is NULL.
 * Layout as there: [hidden_size] contiguous per token.  d_normed receives the fp32 result when
 * not NULL (pass d_input for the reference's in-place behaviour); d_xq receives
 * jq_q8_1_bytes(hidden_size, num_tokens) bytes of blocks when not NULL (hidden_size % 128 == 0).
 * d_input itself is only read unless it is also d_normed. */
int jq_rms_norm_q8_1_device(void *stream, float *d_input, float *d_residual, const float *d_weight,
                            float *d_normed, void *d_xq, int64_t hidden_size, int64_t num_tokens,
                            float epsilon, int order, int s_mode);

/* swiglu_silu_mul_launch_device (src/cuda/swiglu.cu:18-29): mid = silu(gate) * up over
 * [intermediate_size] contiguous values per token.  d_mid (fp32) and d_xq (Q8_1 blocks,
 * intermediate_size % 128 == 0) are each optional, at least one is required. */
int jq_swiglu_q8_1_device(void *stream, const float *d_gate, const float *d_up, float *d_mid, void *d_xq,
                          int64_t intermediate_size, int64_t num_tokens, int order, int s_mode);

/* ---- N-sharded decode (no counterpart in the reference, which is single-GPU) -------------------
 * One process per GPU owns a contiguous band of weight rows.  jq_linear_q4_0_allgather_device
 * runs this rank's quantize + multiply (M <= 2: one streaming kernel; larger M: a quantize launch
 * and the tensor-core GEMM, K % 256 == 0) and writes its band of the output directly into
 * every rank's [M][N_total] buffer through peer-mapped pointers (plain stores over NVLink); each
 * CTA then adds its share to the arrival count that every rank keeps for this rank (one
 * system-scope release-add per CTA and peer; a whole all-gather adds 65536).  The kernel does not
 * wait for the other ranks at its end:
 * whoever consumes the gathered output waits for the counts - the next sharded layer by passing
 * wait_epoch (its prologue then waits, while its weight stream is already running), anything
 * else by queueing jq_allgather_wait_device first.  All ranks must make the same sequence of calls.
 *   y_peers[q]     : rank q's pair of output buffers as mapped on this device (q == rank: local);
 *                    the second buffer starts y_stride_bytes after the first
 *   flag_peers[q]  : rank q's uint32[world] arrival counts, likewise; zero before the first call
 *   d_epoch        : a local uint32, zero before the first call: how many all-gathers this rank has
 *                    finished.  Call number e = *d_epoch + 1 stores into buffer (e & 1), brings the
 *                    counts to e * 65536 (mod 2^32) and sets *d_epoch = e (on the device, so CUDA
 *                    graphs can be replayed)
 *   wait_previous  : non-zero: the activations are the output of all-gather number *d_epoch; the
 *                    kernel waits for all its bands before reading them
 *   d_counter      : a local int, zero before the first call
 * The two buffers alternate, and with wait_previous (or a jq_allgather_wait_device between calls) a
 * fast rank cannot overwrite a band that a slow rank still has to read.
 * With M > 2, wait_previous is carried out by a jq_allgather_wait_device queued ahead of the launches.
 * Every wait inside the kernels is bounded; if one runs out jq_device_fault() reports 2.  Shapes
 * the kernels refuse return JQ_ERR_UNSUPPORTED: multiply locally and all-gather with NCCL.
 * jq_peer_alloc / jq_peer_open: device memory that other processes on the node can map
 * (cudaMalloc + cudaIpcGetMemHandle / cudaIpcOpenMemHandle); the 64-byte handle travels through any
 * host channel (e.g. torch.distributed all_gather_object). */
#define JQ_PEER_HANDLE_BYTES 64
int jq_peer_alloc(size_t bytes, void **d_ptr, unsigned char *handle_out);
int jq_peer_open(const unsigned char *handle, void **d_ptr);
int jq_peer_close(void *d_ptr);
int jq_peer_free(void *d_ptr);
int jq_linear_q4_0_allgather_device(void *stream, const void *d_w, const float *d_x, void *d_ws, int64_t K,
                                    int64_t N_local, int64_t M, int s_mode, void *const *y_peers,
                                    void *const *flag_peers, int world, int rank, int64_t n_offset,
                                    int64_t N_total, size_t y_stride_bytes, int wait_previous,
                                    unsigned *d_epoch, int *d_counter);
/* Blocks the stream (bounded) until all `world` counts at d_flags have reached *d_epoch * 65536,
 * i.e. until the bands of this rank's latest all-gather have arrived from every rank. */
int jq_allgather_wait_device(void *stream, const void *d_flags, int world, const unsigned *d_epoch);

/* The decode form of the fused all-gather (M <= 2), built for latency instead of flags: every output value
 * travels as one 8-byte word {fp32 bits, number of its all-gather} in a single store, which arrives whole.
 * The consumer polls the words it needs until they carry the number it expects: no arrival count, no
 * release and no acknowledgement round trip lies between a rank's last store and a peer's first use.
 *   word_peers[q]  : rank q's pair of [M][N_total] buffers of 8-byte words as mapped on this device (zero
 *                    before the first call); the second buffer starts y_stride_bytes after the first
 *   d_ticket       : a local 64-bit count, zero before the first call.  Every launch adds 65536 to it; the
 *                    launch that finds t is all-gather number e = (t >> 16) + 1, tags its words with e and
 *                    stores into buffer (e & 1).  Layers of a chain share one count.
 *   d_x            : plain fp32 activations [M][K]; or NULL and
 *   d_x_words      : this rank's own pair of word buffers whose all-gather number g = (t >> 16) - x_back is
 *                    this call's input (x_back = 0: the one launched just before this call, 1: the one before
 *                    that, e.g. the second of two projections fed by the same output): row m, activation k is
 *                    word m * x_row_words + (k / x_seg_len) * x_seg_stride + k % x_seg_len of buffer (g & 1).
 *                    x_seg_len = K takes the first K words of a row; K / world words from the start of every
 *                    rank's band make the call depend on all ranks.  x_seg_len is a multiple of 8, x_seg_stride
 *                    and x_row_words are even; when both are multiples of 4 (and the buffers 32-byte aligned)
 *                    the words are polled with 32-byte loads, which halves the polling time.
 * A call that consumes words needs no other ordering.  A call with plain d_x that follows other tagged calls
 * must come after a jq_allgather_tagged_read_device (or a stream synchronisation after one) so that no rank
 * overwrites a buffer another rank still reads.  All ranks make the same sequence of calls.  Waits are bounded
 * (JQ_OPT_WAIT_POLL_LIMIT); a wait that runs out sets jq_device_fault() to 2 and the kernel goes on. */
int jq_linear_q4_0_allgather_tagged_device(void *stream, const void *d_w, const float *d_x, const void *d_x_words,
                                           size_t x_stride_bytes, int64_t x_row_words, int64_t x_seg_len,
                                           int64_t x_seg_stride, int x_back, int64_t K, int64_t N_local, int64_t M, int s_mode,
                                           void *const *word_peers, int world, int rank, int64_t n_offset,
                                           int64_t N_total, size_t y_stride_bytes, unsigned long long *d_ticket);
/* Waits (bounded) for every word of the all-gather numbered *d_ticket >> 16 in this rank's pair of word
 * buffers and writes the values as plain fp32 [M][N_total] to d_out. */
int jq_allgather_tagged_read_device(void *stream, const void *d_words, size_t stride_bytes, int64_t M,
                                    int64_t N_total, const unsigned long long *d_ticket, float *d_out);

/* No counterpart in the reference.  jq_linear_q4_0_device() without the d_ws argument, for callers
 * that must not allocate device memory and have no spare buffer to lend: an inference server that
 * handed the whole device to its own arena at start-up (a later cudaMalloc fails or fragments),
 * or a latency-critical decode loop that cannot afford cudaMalloc's device-wide synchronisation.
 * The Q8_1 scratch lives in a fixed array inside the library image: JQ_NOALLOC_WS_BYTES bytes of
 * device memory on every GPU that loads the library, held until the process exits.
 *  - Capacity: jq_q8_1_bytes(K, M) <= JQ_NOALLOC_WS_BYTES (e.g. M = 512 at K = 4096, M = 128 at
 *    K = 11008); larger requests return JQ_ERR_TOO_LARGE and launch nothing.
 *  - The first call on each device looks up the array's device address (with that device current);
 *    make that first call outside any stream capture.  No call allocates or frees anything.
 *  - Every call on a device shares the one array and overwrites the part it uses, so nothing has to
 *    be cleared between calls; two calls whose kernels can overlap on the GPU (different streams
 *    without an ordering between them) race on it - order them, or use jq_linear_q4_0_device().
 *  - The quantized activations are not returned to the caller. */
#define JQ_NOALLOC_WS_BYTES (4u << 20)
int jq_linear_q4_0_device_noalloc(void *stream, const void *d_w, const float *d_x, float *d_y, int64_t K,
                                  int64_t N, int64_t M, int s_mode);

/* Parity aid: the exact int32 dot product of every (row n, 32-wide block kb, column m),
 * d_sums[(m*N + n)*(K/32) + kb], i.e. `sumi` of q4_0_q8_1_vec_dot_impl (mm_q4_0_q8_1.cu:71-93)
 * before any scale is applied.  The reference never exposes it. */
int jq_block_sums_q4_0_q8_1_device(void *stream, const void *d_w, const void *d_xq, int32_t *d_sums,
                                   int64_t K, int64_t N, int64_t M, int order);

/* fp32 [N][K] -> Q4_0.  The reference has no weight quantizer; this is the ggml rule its block
 * layout comes from (d = signed max-magnitude / -8, q = min(15, trunc(w/d + 8.5))). */
int jq_quantize_q4_0_device(void *stream, const float *d_w, void *d_wq, int64_t N, int64_t K);

/* *fault_out is non-zero after a kernel of this library gave up on a bounded wait on the current device
 * (1: a bulk copy or pipeline stage never completed; 2: the bands of an all-gather never arrived), or, in the
 * range-checked debug build, skipped an access that fell outside its buffer (3); the word keeps the highest
 * code.  The call then returns JQ_ERR_TIMEOUT, else JQ_OK.  The kernel has returned, its output is not
 * valid, and the device stays usable.  Synchronises the device.  `clear` != 0 resets the word. */
int jq_device_fault(int clear, int *fault_out);

/* The range-checked debug build (compiled with -DJQ_BOUNDS_CHECK, linked as libjq_b200_check.so) stands in
 * for a memory checker: its kernels check every global access against the extent that the entry point's
 * shape arguments give the buffer, and every dynamic shared-memory offset against the launch's size; an
 * access outside is skipped and jq_device_fault() reads 3.  (The reference's own hook is the sanitizer
 * option of its Debug configuration, src/cuda/CMakeLists.txt:127-129.)
 * jq_bounds_checked(): 1 in that build, 0 otherwise.  jq_debug_set_extent_shrink(n): every extent the
 * kernels are given from now on is n bytes shorter than the shapes say, so that a test can watch the checks
 * fire, and the accesses being skipped, on addresses that are in fact in range; 0 restores. */
int jq_bounds_checked(void);
int jq_debug_set_extent_shrink(unsigned long long bytes);

/* ---- host entry points (reference-facing) ------------------------------------------------ */

/* q8_1() (q8_1.cu:148-193) with a C signature: dims = {K, M, ne2, ne3}; writes
 * M*ceil(K/128) blocks in JQ_ORDER_KSUPER_COL order with s = sum(x). */
int jq_q8_1_host(const float *input, uint8_t *output, const int *dims, int ndims);

/* parse_q8_1_output (q8_1.cu:197-216). */
int jq_parse_q8_1_output(const uint8_t *input, int8_t *qs_out, float *scale_out, float *sum_out,
                         int64_t n_blocks);

/* mat_mul_q4_0_q8_1 (mm_q4_0_q8_1.cu:318-380): host weights, host activations, host outputs;
 * quant_workspace receives the quantized activations exactly as q8_1() writes them.
 * Unlike the reference, M > 1 gives the mathematically right product (the reference's two
 * kernels disagree on block order there). */
int jq_mat_mul_q4_0_q8_1_host(const void *weight_q4_0, const float *input, uint8_t *quant_workspace,
                              float *output, const int *input_dims, int ndims, int nrows_out,
                              int ncols_k);

/* Same with the meaning of the stored `s` chosen (the plain entry uses JQ_S_SUM_X like the reference). */
int jq_mat_mul_q4_0_q8_1_host_ex(const void *weight_q4_0, const float *input, uint8_t *quant_workspace,
                                 float *output, const int *input_dims, int ndims, int nrows_out,
                                 int ncols_k, int s_mode);

/* Weights kept resident on the current device, for callers that run many multiplies. */
typedef struct jq_weights jq_weights;
int jq_weights_create(const void *host_w_q4_0, int64_t N, int64_t K, jq_weights **out);
int jq_weights_destroy(jq_weights *w);
const void *jq_weights_device_ptr(const jq_weights *w);
/* x (host, M*K floats) -> y (host, M*N floats); pinned host buffers make the copies async.
 * quant_workspace may be NULL. */
int jq_linear_q4_0_host(jq_weights *w, const float *x, uint8_t *quant_workspace, float *y,
                        int64_t M, int s_mode);

/* ---- device description (include/device_hw_info.cuh:113-250 of the reference) ------------- */
typedef struct jq_device_hw_info {
    char name[256];
    int device_id, cc_major, cc_minor, sm_count;
    int sm_clock_khz, mem_clock_khz, mem_bus_width_bits;
    int fp32_cores_per_sm, warp_schedulers_per_sm, max_warps_per_sm;
    size_t smem_per_sm, smem_per_block_optin, l2_bytes, global_mem_bytes;
    double peak_fp32_tflops;      /* 2 * cores * clock */
    double peak_dram_gbs;         /* nominal, from the table for the chip when known */
    double peak_int8_dense_tops;  /* nominal dense int8 tensor throughput, 0 if unknown */
    double peak_bf16_dense_tflops;
    double ridge_int8_ops_per_byte;
} jq_device_hw_info;
int jq_query_device_hw_info(int device, jq_device_hw_info *out);

#ifdef __cplusplus
}
#endif
#endif /* JQ_B200_H_ */
