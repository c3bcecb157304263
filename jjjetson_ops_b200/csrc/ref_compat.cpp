// The reference's own symbols, kept so that code written against JJJetson_Ops links
// unchanged: q8_1 (src/cuda/q8_1.cu:148), parse_q8_1_output (:197), mat_mul_q4_0_q8_1
// (src/cuda/mm_q4_0_q8_1.cu:318) and mat_mul_q4_0_q8_1_device (:394).  They forward to the C ABI.
// Like the reference they return void; unlike it they never call exit(): a failure is printed
// to stderr and the outputs are left untouched (what the reference does for bad shapes,
// mm_q4_0_q8_1.cu:326-340).
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <vector>

#include "../../include/jq_b200.h"

static void report(const char *who, int rc) {
    if (rc != JQ_OK) std::fprintf(stderr, "%s: %s (%s)\n", who, jq_last_error(), jq_status_string(rc));
}

extern "C" void q8_1(float *input, uint8_t *output, std::vector<int> &input_dims) {
    report("q8_1", jq_q8_1_host(input, output, input_dims.data(), (int)input_dims.size()));
}

extern "C" void parse_q8_1_output(const uint8_t *input, int8_t *qs_out, float *scale_out, float *sum_out,
                                  int64_t n_blocks) {
    report("parse_q8_1_output", jq_parse_q8_1_output(input, qs_out, scale_out, sum_out, n_blocks));
}

extern "C" void mat_mul_q4_0_q8_1(const void *weight_q4_0, float *input, uint8_t *quant_workspace, float *output,
                                  std::vector<int> &input_dims, int nrows_out, int ncols_k) {
    report("mat_mul_q4_0_q8_1",
           jq_mat_mul_q4_0_q8_1_host(weight_q4_0, input, quant_workspace, output, input_dims.data(),
                                     (int)input_dims.size(), nrows_out, ncols_k));
}

// Device pointers in, kernel launch only; activations in the order the reference kernel reads
// them (block m * (K/128) + k/128, mm_q4_0_q8_1.cu:230).
extern "C" void mat_mul_q4_0_q8_1_device(const void *d_w_q4_0, const void *d_x_q8_1, float *d_y, const int ncols_k,
                                         const int nrows_out, const int batch, cudaStream_t stream) {
    report("mat_mul_q4_0_q8_1_device",
           jq_mul_mat_q4_0_q8_1_device(stream, d_w_q4_0, d_x_q8_1, d_y, ncols_k, nrows_out, batch,
                                       JQ_ORDER_COL_KSUPER));
}

// ---- the layer's neighbours of the quantized linear, under the reference's names ----------------
// rms_norm_fused_add_forward_device (src/cuda/rms_norm_fused_add.cu:85-105), rms_norm_forward_device
// (src/cuda/rms_norm.h:11-12) and swiglu_silu_mul_launch_device (src/cuda/swiglu.cu:18-29) keep their
// signatures and in-place behaviour; they run this library's kernels without the quantized output.
extern "C" int rms_norm_fused_add_forward_device(void *stream, float *d_input, float *d_residual, const float *d_weight,
                                                 int hidden_size, int num_tokens, float epsilon) {
    if (stream == nullptr || d_residual == nullptr) {  // the reference refuses both (rms_norm_fused_add.cu:91-101)
        std::fprintf(stderr, "rms_norm_fused_add_forward_device: stream or d_residual is null\n");
        return -1;
    }
    const int rc = jq_rms_norm_q8_1_device(stream, d_input, d_residual, d_weight, d_input, nullptr, hidden_size, num_tokens,
                                           epsilon, JQ_ORDER_COL_KSUPER, JQ_S_SUM_X);
    report("rms_norm_fused_add_forward_device", rc);
    return rc == JQ_OK ? 0 : -1;
}

extern "C" int rms_norm_forward_device(void *stream, const float *d_input, const float *d_weight, float *d_output,
                                       int hidden_size, int num_tokens, float epsilon) {
    const int rc = jq_rms_norm_q8_1_device(stream, const_cast<float *>(d_input), nullptr, d_weight, d_output, nullptr,
                                           hidden_size, num_tokens, epsilon, JQ_ORDER_COL_KSUPER, JQ_S_SUM_X);
    report("rms_norm_forward_device", rc);
    return rc == JQ_OK ? 0 : -1;
}

extern "C" void swiglu_silu_mul_launch_device(void *stream, const float *gate, const float *up, float *mid, int n_elem) {
    if (n_elem <= 0) return;
    report("swiglu_silu_mul_launch_device", jq_swiglu_q8_1_device(stream, gate, up, mid, nullptr, n_elem, 1, JQ_ORDER_COL_KSUPER, JQ_S_SUM_X));
}

// What linear_forward_device (src/cuda/linear.cu:9-24) is for fp32 weights, for Q4_0 weights: input
// [in_features] per token, weight out_features rows of in_features / 32 Q4_0 blocks, output
// [out_features] per token.  d_ws takes the place of the cuBLAS handle: jq_q8_1_bytes(in_features,
// num_tokens) bytes of scratch for the quantized activations.  Usable at the seven call sites of the
// layer (src/engine/transformer_runner.cpp:214-216, 294, 319-328).
extern "C" int linear_q4_0_forward_device(void *stream, const float *d_input, const void *d_weight_q4_0, void *d_ws,
                                          float *d_output, int in_features, int out_features, int num_tokens) {
    const int rc = jq_linear_q4_0_device(stream, d_weight_q4_0, d_input, d_ws, d_output, in_features, out_features, num_tokens,
                                         JQ_S_D_SUM_Q);
    report("linear_q4_0_forward_device", rc);
    return rc == JQ_OK ? 0 : -1;
}

// untied_lm_head_forward_device / tied_lm_head_forward_device (src/cuda/lm_head.cu:20-72) for a Q4_0 table:
// logits[vocab] per token = W[vocab][hidden] . hidden, W stored as vocab rows of hidden / 32 Q4_0 blocks
// (the tied layout, row = one token's embedding).  With d_hidden_q8_1 given, the final RMSNorm has already
// written the blocks (jq_rms_norm_q8_1_device with a NULL residual) and d_hidden / d_ws are not used.
extern "C" int lm_head_q4_0_forward_device(void *stream, const void *d_lm_head_q4_0, const float *d_hidden,
                                           const void *d_hidden_q8_1, void *d_ws, float *d_logits, int hidden_size,
                                           int vocab_size, int num_tokens) {
    int rc;
    if (d_hidden_q8_1 != nullptr) {
        rc = jq_mul_mat_q4_0_q8_1_device(stream, d_lm_head_q4_0, d_hidden_q8_1, d_logits, hidden_size, vocab_size, num_tokens,
                                         JQ_ORDER_COL_KSUPER);
    } else {
        rc = jq_linear_q4_0_device(stream, d_lm_head_q4_0, d_hidden, d_ws, d_logits, hidden_size, vocab_size, num_tokens,
                                   JQ_S_D_SUM_Q);
    }
    report("lm_head_q4_0_forward_device", rc);
    return rc == JQ_OK ? 0 : -1;
}
