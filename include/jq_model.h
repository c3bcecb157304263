/* jq_model.h - the model's weights on the device with Q4_0 linears: the quantized counterpart of the
 * reference's weight container.
 *
 * The reference keeps, per decoder layer, nine fp32 device buffers (TransformerLayerWeights,
 * src/model/transformer_model.h:13-23) filled from a WeightLoadResult by transformer_model_load_weights
 * (src/model/transformer_model.cpp:327-373: "layer<i>.w_q" ... "layer<i>.w_post_attention_layernorm",
 * then "embed", "final_norm" and, when untied, "lm_head"), and its engine multiplies the seven linears one
 * cuBLAS call each (src/engine/transformer_runner.cpp:214-216, 294, 319-328).  This container takes a
 * jq_weight_set (fixture directory or safetensors file, jq_weights_io.h) whose seven linears per layer
 * are Q4_0 tensors and gives the engine the same view with block_q4_0 pointers in the linear slots.
 *
 * Layout in device memory: one allocation.  Per layer, in execution order: w_q, w_k, w_v back to back,
 * so that the three projections are also ONE [q_dim + 2 kv_dim, hidden] matrix (d_w_qkv) for a single
 * launch of jq_linear_q4_0_device; w_o; w_gate, w_up back to back (d_w_gate_up, [2 intermediate, hidden]);
 * w_down; the two norm vectors.  Then embed, final_norm, lm_head.  Every group starts on a 256-byte
 * boundary.
 *
 * Planning (names, shapes, offsets) is host-only and separate from the upload, so that a checkpoint can
 * be validated without a GPU.
 */
#ifndef JQ_MODEL_H_
#define JQ_MODEL_H_

#include <stddef.h>
#include <stdint.h>

#include "jq_weights_io.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ModelConfig (src/model/model_config.h), field for field. */
typedef struct jq_model_config {
    int hidden_size;
    int intermediate_size;
    int num_layers;
    int num_q_heads;
    int num_kv_heads;
    int head_dim;
    int vocab_size;
    int max_seq_len;
    float freq_base;
    float rms_norm_epsilon;
    int tie_word_embeddings;
} jq_model_config;

/* Reads the eleven "key=value" lines of a config.txt.  As the reference's loader
 * (src/model/weight_loader.cpp, parse_config_file) every key must be present, and the values must pass
 * model_config_validate (src/model/model_config.cpp): all sizes positive, num_kv_heads <= num_q_heads,
 * num_q_heads * head_dim == hidden_size, freq_base and rms_norm_epsilon positive, tie_word_embeddings
 * 0 or 1. */
int jq_model_config_parse(const char *config_text, jq_model_config *out);

/* One tensor of the plan: where the device copy lies and what it holds. */
typedef struct jq_model_slot {
    char name[96];
    int dtype;        /* jq_weight_dtype */
    int64_t rows, K;  /* Q4_0: [rows, K]; F32: rows = element count, K = 0 */
    size_t offset;    /* from the start of the device allocation */
    size_t nbytes;
} jq_model_slot;

typedef struct jq_model_plan {
    jq_model_config config;
    jq_model_slot *slots;  /* per layer the nine tensors in the order above, then embed, final_norm[, lm_head] */
    int num_slots;
    size_t total_bytes;
} jq_model_plan;

/* Validates `set` against its own config.txt and lays the model out.  Errors (status from jq_b200.h,
 * message in jq_last_error()): a key missing from config.txt or an invalid value; a tensor missing; a
 * linear that is still fp32 (JQ_ERR_UNSUPPORTED: run the offline quantizer first) or whose dims are not
 * the [out_features, in_features] the config implies; a norm, embed or lm_head of the wrong size.
 * embed may be F32 [vocab * hidden elements] or, when tied, Q4_0 [vocab, hidden] (it is then the
 * lm_head table of lm_head_q4_0_forward_device).  lm_head (untied only) is kept in the type it has. */
int jq_model_q4_0_plan(const jq_weight_set *set, jq_model_plan **out);
void jq_model_plan_destroy(jq_model_plan *plan);

/* TransformerLayerWeights (transformer_model.h:13-23) with Q4_0 linears, plus the two fused views. */
typedef struct jq_layer_weights_q4_0 {
    const void *d_w_q;      /* block_q4_0 [q_dim][hidden / 32] */
    const void *d_w_k;      /* [kv_dim][hidden / 32] */
    const void *d_w_v;
    const void *d_w_o;      /* [hidden][q_dim / 32] */
    const void *d_w_gate;   /* [intermediate][hidden / 32] */
    const void *d_w_up;
    const void *d_w_down;   /* [hidden][intermediate / 32] */
    const float *d_w_input_layernorm;
    const float *d_w_post_attention_layernorm;
    const void *d_w_qkv;      /* = d_w_q, read as [q_dim + 2 kv_dim][hidden / 32] */
    const void *d_w_gate_up;  /* = d_w_gate, read as [2 intermediate][hidden / 32] */
} jq_layer_weights_q4_0;

typedef struct jq_model_q4_0 jq_model_q4_0;

/* transformer_model_create + transformer_model_load_weights in one step: plans, allocates the model on
 * the current device and copies every tensor.  The model is immutable afterwards.  Fails with
 * JQ_ERR_CUDA (and allocates nothing) when there is no usable device. */
int jq_model_q4_0_create(const jq_weight_set *set, jq_model_q4_0 **out);
void jq_model_q4_0_destroy(jq_model_q4_0 *model);

const jq_model_config *jq_model_q4_0_config(const jq_model_q4_0 *model);
const jq_model_plan *jq_model_q4_0_layout(const jq_model_q4_0 *model);
/* transformer_model_get_layer_weights (transformer_model.h:45-46); NULL when layer is out of range. */
const jq_layer_weights_q4_0 *jq_model_q4_0_layer(const jq_model_q4_0 *model, int layer);
/* transformer_model_get_d_embed / _get_d_final_norm / _get_d_lm_head (transformer_model.h:48-52); the
 * table's jq_weight_dtype goes to *dtype (may be NULL).  Tied models return the embed table as lm_head. */
const void *jq_model_q4_0_embed(const jq_model_q4_0 *model, int *dtype);
const float *jq_model_q4_0_final_norm(const jq_model_q4_0 *model);
const void *jq_model_q4_0_lm_head(const jq_model_q4_0 *model, int *dtype);

#ifdef __cplusplus
}
#endif

#endif /* JQ_MODEL_H_ */
