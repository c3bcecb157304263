// The reference's own four symbols, kept so that code written against JJJetson_Ops links
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
