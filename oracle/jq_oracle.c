/*
 * CPU oracle for the Q4_0 x Q8_1 quantized-linear path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C on the host, the arithmetic of the reference's
 * two CUDA operators so that the CUDA kernels of this library can be checked
 * against it.  Nothing in the shipped library links, loads or calls this file;
 * only the test-suite, the smoke check and the CPU-baseline leg of the benchmark do.
 *
 * Parity status: the activation quantizer is pinned by the reference's own NumPy
 * restatement (tests/test_q8_1.py:5-62, seed 24 case, committed as a golden
 * fixture).  The reference holds no test, fixture or CPU implementation for the
 * matrix multiply, so for the multiply this oracle is pinned only by outputs of
 * the reference CUDA kernels themselves, rebuilt unmodified and run on a B200
 * (fixture tests/golden/ref_gpu_*.npz, made by tests/golden/make_ref_gpu_golden.py).
 *
 * Each function cites the reference lines (path inside the reference project)
 * whose behaviour it follows.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off: the fused operations
 * the CUDA compiler forms are written out with fmaf() by hand, everything else
 * must round once per operation exactly like the device code).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define JQO_QK 32          /* values per Q4_0 block and per Q8_1 sub-block */
#define JQO_Q4_BYTES 18    /* struct block_q4_0, src/cuda/mm_q4_0_q8_1.cu:35-38 */
#define JQO_SUPER 128      /* values per block_q8_1_mmq, src/cuda/q8_1.cu:14-18 */
#define JQO_Q8_BYTES 144

enum { JQO_ORDER_KSUPER_COL = 0, JQO_ORDER_COL_KSUPER = 1 };
enum { JQO_S_SUM_X = 0, JQO_S_D_SUM_Q = 1 };

/* ---- IEEE binary16 <-> binary32, round-to-nearest-even, like __float2half / __half2float ---- */
static uint16_t f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x0200u : 0u));
    }
    if (absx >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx < 0x33000001u) { /* <= 2^-25: rounds to zero (ties-to-even at exactly 2^-25) */
        return (uint16_t)sign;
    }
    int32_t exp = (int32_t)(absx >> 23) - 127;
    uint32_t man = (absx & 0x007FFFFFu) | 0x00800000u;
    uint32_t half;
    int shift;
    if (exp < -14) { /* subnormal half */
        shift = 13 + (-14 - exp);
        uint32_t q = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (q & 1u))) q++;
        half = q; /* may carry into the smallest normal, which is correct */
    } else {
        uint32_t q = man >> 13; /* 11 bits incl. hidden one */
        uint32_t rem = man & 0x1FFFu;
        if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++;
        half = ((uint32_t)(exp + 15) << 10) + (q - 0x400u); /* carry propagates into exponent */
    }
    return (uint16_t)(sign | half);
}

static float f16_to_f32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t x;
    if (exp == 0) {
        if (man == 0) {
            x = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400u));
            x = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        x = sign | 0x7F800000u | (man << 13);
    } else {
        x = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

uint16_t jqo_f32_to_f16(float f) { return f32_to_f16(f); }
float jqo_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

/* ------------------------------------------------------------------------------------------
 * Q4_0 weight quantizer.  The reference has none (its tests never build Q4_0 data); this is
 * the published ggml rule the block layout comes from (mm_q4_0_q8_1.cu:35-38,49): per 32
 * weights take the value of largest magnitude with its sign, d = max / -8,
 * q = min(15, trunc(w / d + 8.5)), byte j = q[j] | q[j+16] << 4, scale stored as fp16.
 * w: [n_rows][K] row-major fp32, K % 32 == 0.  out: n_rows * K/32 * 18 bytes.
 * ------------------------------------------------------------------------------------------ */
void jqo_quantize_q4_0(const float *w, int64_t n_rows, int64_t K, uint8_t *out) {
    const int64_t nb = K / JQO_QK;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n_rows; ++r) {
        for (int64_t b = 0; b < nb; ++b) {
            const float *x = w + r * K + b * JQO_QK;
            uint8_t *o = out + (r * nb + b) * JQO_Q4_BYTES;
            float amax = 0.0f, mx = 0.0f;
            for (int j = 0; j < JQO_QK; ++j) {
                const float v = x[j];
                if (amax < fabsf(v)) {
                    amax = fabsf(v);
                    mx = v;
                }
            }
            const float d = mx / -8.0f;
            const float id = d != 0.0f ? 1.0f / d : 0.0f;
            const uint16_t dh = f32_to_f16(d);
            memcpy(o, &dh, 2);
            for (int j = 0; j < JQO_QK / 2; ++j) {
                const float x0 = x[j] * id;
                const float x1 = x[j + JQO_QK / 2] * id;
                int q0 = (int)(int8_t)(x0 + 8.5f);
                int q1 = (int)(int8_t)(x1 + 8.5f);
                if (q0 > 15) q0 = 15;
                if (q1 > 15) q1 = 15;
                o[2 + j] = (uint8_t)(q0 | (q1 << 4));
            }
        }
    }
}

/* value = (q - 8) * d, mm_q4_0_q8_1.cu:71-93 (the "- 8 * s8" term is this zero point). */
static inline void dequant_row_q4_0(const uint8_t *row, int64_t nb, float *y) {
    for (int64_t b = 0; b < nb; ++b) {
        const uint8_t *o = row + b * JQO_Q4_BYTES;
        uint16_t dh;
        memcpy(&dh, o, 2);
        const float d = f16_to_f32(dh);
        for (int j = 0; j < 16; ++j) {
            y[b * JQO_QK + j] = (float)((int)(o[2 + j] & 0x0F) - 8) * d;
            y[b * JQO_QK + j + 16] = (float)((int)(o[2 + j] >> 4) - 8) * d;
        }
    }
}

void jqo_dequantize_q4_0(const uint8_t *wq, int64_t n_rows, int64_t K, float *w) {
    const int64_t nb = K / JQO_QK;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n_rows; ++r) {
        dequant_row_q4_0(wq + r * nb * JQO_Q4_BYTES, nb, w + r * K);
    }
}

static inline int64_t q8_block_index(int64_t ksuper, int64_t m, int64_t n_super, int64_t M,
                                     int order) {
    /* q8_1.cu:84-86 writes block (i0/128)*ne1 + col; mm_q4_0_q8_1.cu:230,246 reads
     * col*(K/128) + super.  Both orders are supported; they coincide for M == 1. */
    return order == JQO_ORDER_KSUPER_COL ? ksuper * M + m : m * n_super + ksuper;
}

/* ------------------------------------------------------------------------------------------
 * Activation quantizer, follows quantize_q8_1_kernel (src/cuda/q8_1.cu:20-104):
 *   - one thread owns 4 consecutive floats, 8 threads own a 32-value group;
 *   - amax by max over the group (:55-60), order does not matter;
 *   - sum: per-thread ((x+y)+z)+w (:62-63), then the xor butterfly with offsets 4,2,1
 *     (:65-68); lane 0 of a group ends with ((t0+t4)+(t2+t6))+((t1+t5)+(t3+t7));
 *   - d_inv = amax > 0 ? 127.0f / amax : 0 (:71), q = roundf(x * d_inv) (:73-79);
 *   - stores half2(1.0f / d_inv, sum) (:101-103).
 * Deviation, on purpose: for an all-zero group the reference stores fp16(1/0) = +inf,
 * which makes the multiply produce NaN; this oracle (like the reference's own NumPy
 * restatement, tests/test_q8_1.py:47-52) stores d = 0.
 * s_mode JQO_S_SUM_X stores s = fp16(sum of the 32 floats) as the reference does;
 * s_mode JQO_S_D_SUM_Q stores s = fp16(fp16(d) * sum of the 32 int8) (the ggml Q8_1
 * definition, which makes the multiply agree with dequantise-then-matmul).
 * x: [M][K] row-major (K fastest, "ne0 = K, ne1 = M").  K % 32 == 0.  A trailing partial
 * 128-block is zero-filled.  out: M * ceil(K/128) * 144 bytes.
 * ------------------------------------------------------------------------------------------ */
void jqo_quantize_q8_1_mmq(const float *x, int64_t K, int64_t M, int order, int s_mode,
                           uint8_t *out) {
    const int64_t n_super = (K + JQO_SUPER - 1) / JQO_SUPER;
    for (int64_t m = 0; m < M; ++m) {
        for (int64_t ks = 0; ks < n_super; ++ks) {
            uint8_t *blk = out + q8_block_index(ks, m, n_super, M, order) * JQO_Q8_BYTES;
            for (int g = 0; g < 4; ++g) {
                const int64_t k0 = ks * JQO_SUPER + g * JQO_QK;
                uint16_t dh = 0, sh = 0;
                int8_t *qs = (int8_t *)(blk + 16 + g * JQO_QK);
                if (k0 >= K) {
                    memset(qs, 0, JQO_QK);
                } else {
                    const float *v = x + m * K + k0;
                    float amax = 0.0f;
                    float t[8];
                    for (int l = 0; l < 8; ++l) {
                        const float a = v[4 * l], b = v[4 * l + 1], c = v[4 * l + 2],
                                    d4 = v[4 * l + 3];
                        amax = fmaxf(amax, fmaxf(fabsf(a), fmaxf(fabsf(b), fmaxf(fabsf(c), fabsf(d4)))));
                        t[l] = ((a + b) + c) + d4;
                    }
                    const float sum = ((t[0] + t[4]) + (t[2] + t[6])) + ((t[1] + t[5]) + (t[3] + t[7]));
                    const float d_inv = amax > 0.0f ? 127.0f / amax : 0.0f;
                    int isum = 0;
                    for (int j = 0; j < JQO_QK; ++j) {
                        const float q = roundf(v[j] * d_inv);
                        qs[j] = (int8_t)q;
                        isum += (int)qs[j];
                    }
                    dh = amax > 0.0f ? f32_to_f16(1.0f / d_inv) : 0;
                    if (s_mode == JQO_S_SUM_X) {
                        sh = f32_to_f16(sum);
                    } else {
                        sh = f32_to_f16(f16_to_f32(dh) * (float)isum);
                    }
                }
                memcpy(blk + 4 * g, &dh, 2);
                memcpy(blk + 4 * g + 2, &sh, 2);
            }
        }
    }
}

/* parse_q8_1_output (src/cuda/q8_1.cu:197-216): split raw blocks into qs / d / s arrays. */
void jqo_parse_q8_1(const uint8_t *raw, int64_t n_blocks, int8_t *qs, float *scale, float *sum) {
    for (int64_t b = 0; b < n_blocks; ++b) {
        const uint8_t *blk = raw + b * JQO_Q8_BYTES;
        memcpy(qs + b * JQO_SUPER, blk + 16, JQO_SUPER);
        for (int g = 0; g < 4; ++g) {
            uint16_t dh, sh;
            memcpy(&dh, blk + 4 * g, 2);
            memcpy(&sh, blk + 4 * g + 2, 2);
            scale[b * 4 + g] = f16_to_f32(dh);
            sum[b * 4 + g] = f16_to_f32(sh);
        }
    }
}

/* One Q4_0 block times one Q8_1 sub-block, integer part.  q4_0_q8_1_vec_dot_impl
 * (mm_q4_0_q8_1.cu:71-93) pairs the low nibbles of word i with X ints 2i (values 4i..4i+3)
 * and the high nibbles with 2i+1, and vec_dot (:141-161) feeds X ints l and l+4 there, so
 * weight j (low nibble of byte j) meets activation j and weight j+16 (high nibble) meets
 * activation j+16.  The nibbles are used unsigned (0..15). */
static inline int32_t block_sumi(const uint8_t *q4blk, const int8_t *q8) {
    int32_t s = 0;
    for (int j = 0; j < 16; ++j) {
        s += (int32_t)(q4blk[2 + j] & 0x0F) * (int32_t)q8[j];
        s += (int32_t)(q4blk[2 + j] >> 4) * (int32_t)q8[j + 16];
    }
    return s;
}

/* int32 block sums sumi[m][n][kb]; the bit-exact integer target of the multiply. */
void jqo_block_sums(const uint8_t *wq, const uint8_t *xq, int64_t K, int64_t N, int64_t M,
                    int order, int32_t *sums) {
    const int64_t nb = K / JQO_QK, n_super = K / JQO_SUPER;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t m = 0; m < M; ++m) {
            for (int64_t kb = 0; kb < nb; ++kb) {
                const uint8_t *xb =
                    xq + q8_block_index(kb / 4, m, n_super, M, order) * JQO_Q8_BYTES;
                sums[(m * N + n) * nb + kb] = block_sumi(
                    wq + (n * nb + kb) * JQO_Q4_BYTES, (const int8_t *)(xb + 16 + (kb % 4) * JQO_QK));
            }
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * The multiply with the reference formula and the reference accumulation order:
 *   y[m*N + n] = sum over kb ascending of  d4 * (sumi * d8 - 8 * s8)
 * (mm_q4_0_q8_1.cu:92 for the term, :206,256-269 for the ascending-kb fp32 accumulation,
 * :286 for the output index).  nvcc's default floating-point contraction turns the term into
 * fma(sumi, d8, -(8*s8)) and the accumulation into fma(d4, term, acc); both are written out.
 * ------------------------------------------------------------------------------------------ */
void jqo_mul_mat_ref(const uint8_t *wq, const uint8_t *xq, int64_t K, int64_t N, int64_t M,
                     int order, float *y) {
    const int64_t nb = K / JQO_QK, n_super = K / JQO_SUPER;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t m = 0; m < M; ++m) {
            float acc = 0.0f;
            for (int64_t kb = 0; kb < nb; ++kb) {
                const uint8_t *wb = wq + (n * nb + kb) * JQO_Q4_BYTES;
                const uint8_t *xb =
                    xq + q8_block_index(kb / 4, m, n_super, M, order) * JQO_Q8_BYTES;
                uint16_t h4, h8d, h8s;
                memcpy(&h4, wb, 2);
                memcpy(&h8d, xb + 4 * (kb % 4), 2);
                memcpy(&h8s, xb + 4 * (kb % 4) + 2, 2);
                const int32_t sumi = block_sumi(wb, (const int8_t *)(xb + 16 + (kb % 4) * JQO_QK));
                const float term = fmaf((float)sumi, f16_to_f32(h8d), -(8.0f * f16_to_f32(h8s)));
                acc = fmaf(f16_to_f32(h4), term, acc);
            }
            y[m * N + n] = acc;
        }
    }
}

/* Dequantise Q8_1 activations: value = q * fp16(d). */
void jqo_dequantize_q8_1(const uint8_t *xq, int64_t K, int64_t M, int order, float *x) {
    const int64_t n_super = K / JQO_SUPER;
    for (int64_t m = 0; m < M; ++m) {
        for (int64_t ks = 0; ks < n_super; ++ks) {
            const uint8_t *blk = xq + q8_block_index(ks, m, n_super, M, order) * JQO_Q8_BYTES;
            for (int g = 0; g < 4; ++g) {
                uint16_t dh;
                memcpy(&dh, blk + 4 * g, 2);
                const float d = f16_to_f32(dh);
                const int8_t *qs = (const int8_t *)(blk + 16 + g * JQO_QK);
                for (int j = 0; j < JQO_QK; ++j) {
                    x[m * K + ks * JQO_SUPER + g * JQO_QK + j] = (float)qs[j] * d;
                }
            }
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * Dequantise-then-matmul with float64 accumulation: the accuracy yardstick for the fp32
 * outputs (max |y - ref| / max |ref| <= 1e-3).  Build-authored: the reference has no CPU
 * implementation of the multiply.
 * ------------------------------------------------------------------------------------------ */
void jqo_mul_mat_deq_f64(const uint8_t *wq, const uint8_t *xq, int64_t K, int64_t N, int64_t M,
                         int order, float *y) {
    float *xf = (float *)malloc((size_t)M * K * sizeof(float));
    jqo_dequantize_q8_1(xq, K, M, order, xf);
#pragma omp parallel
    {
        float *wrow = (float *)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t n = 0; n < N; ++n) {
            dequant_row_q4_0(wq + n * (K / JQO_QK) * JQO_Q4_BYTES, K / JQO_QK, wrow);
            for (int64_t m = 0; m < M; ++m) {
                double acc = 0.0;
                const float *xr = xf + m * K;
                for (int64_t k = 0; k < K; ++k) acc += (double)wrow[k] * (double)xr[k];
                y[m * N + n] = (float)acc;
            }
        }
        free(wrow);
    }
    free(xf);
}

/* ------------------------------------------------------------------------------------------
 * The timed CPU baseline: fp32 activations -> Q8_1 -> dequantise both operands to fp32 ->
 * fp32 matmul, all host threads.  Same data flow as above but float accumulation, written
 * so that gcc vectorises the inner loop (8 independent partial sums).
 * Returns nothing; y[m*N + n].  xq_ws: caller's M*K/128*144-byte workspace.
 * ------------------------------------------------------------------------------------------ */
__attribute__((target_clones("avx512f", "avx2,fma", "default"))) static void
rows_times_x_f32(const float *wrow, const float *xf, int64_t K, int64_t M, int64_t N, int64_t n,
                 float *y) {
    for (int64_t m = 0; m < M; ++m) {
        const float *xr = xf + m * K;
        float p[16] = {0};
        for (int64_t k = 0; k < K; k += 16) {
            for (int l = 0; l < 16; ++l) p[l] += wrow[k + l] * xr[k + l];
        }
        float s = 0.0f;
        for (int l = 0; l < 16; ++l) s += p[l];
        y[m * N + n] = s;
    }
}

void jqo_linear_cpu_baseline(const uint8_t *wq, const float *x, uint8_t *xq_ws, int64_t K,
                             int64_t N, int64_t M, int s_mode, float *y) {
    jqo_quantize_q8_1_mmq(x, K, M, JQO_ORDER_COL_KSUPER, s_mode, xq_ws);
    float *xf = (float *)malloc((size_t)M * K * sizeof(float));
    jqo_dequantize_q8_1(xq_ws, K, M, JQO_ORDER_COL_KSUPER, xf);
#pragma omp parallel
    {
        float *wrow = (float *)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t n = 0; n < N; ++n) {
            dequant_row_q4_0(wq + n * (K / JQO_QK) * JQO_Q4_BYTES, K / JQO_QK, wrow);
            rows_times_x_f32(wrow, xf, K, M, N, n, y);
        }
        free(wrow);
    }
    free(xf);
}

/* ------------------------------------------------------------------------------------------------
 * Producers of the linear's input: RMSNorm (with or without the residual add) and SwiGLU.
 *
 * jqo_rms_norm follows rms_norm_fused_add_kernel (reference src/cuda/rms_norm_fused_add.cu:10-44) and
 * rms_norm_kernel (src/cuda/rms_norm.cu:12-41) including the order of the sum of squares: thread t of a
 * block of min(H, 256) threads adds z*z for i = t, t + block, ... with one fused multiply-add each
 * (nvcc contracts `sum += z * z`), then block_reduce_sum (include/cuda_utils.cuh:19-27, 49-65): a
 * shuffle-down tree inside each warp, one partial per warp, a second shuffle-down tree over the
 * partials.  The only step that cannot be restated exactly on a CPU is rsqrtf (:35), a hardware
 * approximation accurate to about 2 ulp; 1/sqrtf stands in for it, so fp32 results may differ from the
 * device's in the last bits.
 * residual may be NULL (plain RMSNorm); when given it is updated to z = input + residual. */
static float shuffle_down_tree(float *v) { /* v[32], clobbered; returns lane 0's result */
    for (int off = 16; off > 0; off >>= 1) {
        for (int i = 0; i < off; ++i) v[i] = v[i] + v[i + off];
    }
    return v[0];
}

void jqo_rms_norm(const float *input, float *residual, const float *weight, float *normed, int64_t H,
                  int64_t T, float epsilon) {
    const int block = (int)(H < 256 ? H : 256);
    const int n_warps = (block + 31) / 32;
    for (int64_t t = 0; t < T; ++t) {
        const float *in = input + t * H;
        float *res = residual ? residual + t * H : NULL;
        float partial[32 * 32];
        memset(partial, 0, sizeof(partial));
        for (int th = 0; th < block; ++th) {
            float acc = 0.0f;
            for (int64_t i = th; i < H; i += block) {
                float z = in[i];
                if (res) z = z + res[i];
                acc = fmaf(z, z, acc);
            }
            partial[th] = acc;
        }
        float warp_partial[32];
        memset(warp_partial, 0, sizeof(warp_partial));
        for (int w = 0; w < n_warps; ++w) warp_partial[w] = shuffle_down_tree(partial + 32 * w);
        const float sum_square = shuffle_down_tree(warp_partial);
        const float inv = 1.0f / sqrtf(sum_square / (float)H + epsilon);
        for (int64_t i = 0; i < H; ++i) {
            float z = in[i];
            if (res) {
                z = z + res[i];
            }
            const float y = (z * inv) * weight[i];
            if (res) res[i] = z;
            normed[t * H + i] = y;
        }
    }
}

/* swiglu_silu_mul_kernel (src/cuda/swiglu.cu:5-15): mid = (g * (1 / (1 + expf(-g)))) * u.  The device's
 * expf and this libm's may differ in the last bit. */
void jqo_swiglu(const float *gate, const float *up, float *mid, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        const float g = gate[i];
        const float s = g * (1.0f / (1.0f + expf(-g)));
        mid[i] = s * up[i];
    }
}

/* Thread count for the OpenMP loops above (launchers such as torchrun export OMP_NUM_THREADS=1). */
void jqo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int jqo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
