// The model's weights on the device with Q4_0 linears (include/jq_model.h).
//
// Follows transformer_model_load_weights and its helpers (reference
// src/model/transformer_model.cpp:80-150, 327-373): the same tensor names, the same expected sizes
// (derived from the config, never from the file), one host-to-device copy per tensor.  What differs:
// the seven linears of a layer are block_q4_0 arrays, the model is one device allocation laid out in
// execution order, and the layout is computed (and checkable) without a GPU.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/jq_b200.h"
#include "../../include/jq_model.h"

namespace jq {
int set_error(int status, const char *fmt, ...);
int cuda_error(cudaError_t e, const char *what);
}  // namespace jq
using jq::set_error;

struct jq_model_q4_0 {
    jq_model_plan *plan = nullptr;
    uint8_t *d_base = nullptr;
    std::vector<jq_layer_weights_q4_0> layers;
    const void *d_embed = nullptr, *d_lm_head = nullptr;
    const float *d_final_norm = nullptr;
    int embed_dtype = JQ_WEIGHT_F32, lm_head_dtype = JQ_WEIGHT_F32;
};

namespace {

constexpr size_t kGroupAlign = 256;
constexpr int kLayerTensors = 9;
const char *const kLayerSuffix[kLayerTensors] = {"w_q",    "w_k",  "w_v",    "w_o",
                                                 "w_gate", "w_up", "w_down", "w_input_layernorm",
                                                 "w_post_attention_layernorm"};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int64_t numel_of(const jq_host_tensor &t) {
    int64_t n = 1;
    for (int d = 0; d < t.ndim; ++d) n *= t.dims[d];
    return n;
}

struct ConfigKey {
    const char *name;
    bool is_float;
    size_t offset;
};
const ConfigKey kConfigKeys[] = {
    {"hidden_size", false, offsetof(jq_model_config, hidden_size)},
    {"intermediate_size", false, offsetof(jq_model_config, intermediate_size)},
    {"num_layers", false, offsetof(jq_model_config, num_layers)},
    {"num_q_heads", false, offsetof(jq_model_config, num_q_heads)},
    {"num_kv_heads", false, offsetof(jq_model_config, num_kv_heads)},
    {"head_dim", false, offsetof(jq_model_config, head_dim)},
    {"vocab_size", false, offsetof(jq_model_config, vocab_size)},
    {"max_seq_len", false, offsetof(jq_model_config, max_seq_len)},
    {"freq_base", true, offsetof(jq_model_config, freq_base)},
    {"rms_norm_epsilon", true, offsetof(jq_model_config, rms_norm_epsilon)},
    {"tie_word_embeddings", false, offsetof(jq_model_config, tie_word_embeddings)},
};

// Adds one slot for tensor `name` of `set`: a Q4_0 matrix [rows, K] (K > 0) or `rows` fp32 values (K == 0,
// unless `q4_0_allowed`, where either form is taken).  `aligned` starts a new 256-byte group.
int add_slot(const jq_weight_set *set, const std::string &name, int64_t rows, int64_t K, bool must_be_q4_0, bool q4_0_allowed,
             bool aligned, std::vector<jq_model_slot> *slots, size_t *cursor) {
    const jq_host_tensor *t = jq_weight_set_find(set, name.c_str());
    if (t == nullptr) return set_error(JQ_ERR_INVALID_ARG, "missing tensor %s", name.c_str());
    if (name.size() >= sizeof(jq_model_slot::name)) return set_error(JQ_ERR_TOO_LARGE, "tensor name too long: %s", name.c_str());
    jq_model_slot s{};
    std::snprintf(s.name, sizeof(s.name), "%s", name.c_str());
    s.dtype = t->dtype;
    if (t->dtype == JQ_WEIGHT_Q4_0) {
        if (!must_be_q4_0 && !q4_0_allowed) return set_error(JQ_ERR_SHAPE, "%s must be fp32, found Q4_0", name.c_str());
        if (t->ndim != 2 || t->dims[0] != rows || t->dims[1] != K)
            return set_error(JQ_ERR_SHAPE, "%s: Q4_0 dims [%lld, %lld], the config implies [%lld, %lld] (out_features, in_features)",
                             name.c_str(), t->ndim == 2 ? (long long)t->dims[0] : -1LL, t->ndim == 2 ? (long long)t->dims[1] : -1LL,
                             (long long)rows, (long long)K);
        if (K % 32 != 0 || t->nbytes != jq_q4_0_bytes(rows, K))
            return set_error(JQ_ERR_SHAPE, "%s: %zu bytes, %zu expected for Q4_0 [%lld, %lld]", name.c_str(), t->nbytes,
                             jq_q4_0_bytes(rows, K), (long long)rows, (long long)K);
        s.rows = rows;
        s.K = K;
    } else if (t->dtype == JQ_WEIGHT_F32) {
        if (must_be_q4_0)
            return set_error(JQ_ERR_UNSUPPORTED, "%s is still fp32: quantize the weights first (jq_weights_quantize_fixture)", name.c_str());
        const int64_t want = K > 0 ? rows * K : rows;
        if (numel_of(*t) != want || t->nbytes != (size_t)want * sizeof(float))
            return set_error(JQ_ERR_SHAPE, "%s: %lld elements, the config implies %lld", name.c_str(), (long long)numel_of(*t),
                             (long long)want);
        s.rows = want;
        s.K = 0;
    } else {
        return set_error(JQ_ERR_INVALID_ARG, "%s: unknown dtype %d", name.c_str(), t->dtype);
    }
    if (aligned) *cursor = align_up(*cursor, kGroupAlign);
    s.offset = *cursor;
    s.nbytes = t->nbytes;
    *cursor += t->nbytes;
    slots->push_back(s);
    return JQ_OK;
}

}  // namespace

extern "C" int jq_model_config_parse(const char *config_text, jq_model_config *out) {
    if (!config_text || !out) return set_error(JQ_ERR_INVALID_ARG, "null argument");
    jq_weight_set probe{};
    probe.config_text = const_cast<char *>(config_text);
    jq_model_config cfg{};
    for (const ConfigKey &k : kConfigKeys) {
        double v = 0;
        if (!jq_weight_set_config_value(&probe, k.name, &v)) return set_error(JQ_ERR_INVALID_ARG, "config.txt: missing key %s", k.name);
        char *field = reinterpret_cast<char *>(&cfg) + k.offset;
        if (k.is_float) {
            *reinterpret_cast<float *>(field) = (float)v;
        } else {
            if (v != std::floor(v) || std::fabs(v) > 2147483647.0) return set_error(JQ_ERR_INVALID_ARG, "config.txt: %s is not an integer", k.name);
            *reinterpret_cast<int *>(field) = (int)v;
        }
    }
    if (cfg.hidden_size <= 0 || cfg.intermediate_size <= 0 || cfg.num_layers <= 0 || cfg.num_q_heads <= 0 || cfg.num_kv_heads <= 0 ||
        cfg.head_dim <= 0 || cfg.vocab_size <= 0 || cfg.max_seq_len <= 0)
        return set_error(JQ_ERR_INVALID_ARG, "config.txt: every size must be positive");
    if (cfg.num_kv_heads > cfg.num_q_heads) return set_error(JQ_ERR_INVALID_ARG, "config.txt: num_kv_heads exceeds num_q_heads");
    if ((int64_t)cfg.num_q_heads * cfg.head_dim != cfg.hidden_size)
        return set_error(JQ_ERR_INVALID_ARG, "config.txt: num_q_heads * head_dim must equal hidden_size");
    if (!(cfg.freq_base > 0.f) || !(cfg.rms_norm_epsilon > 0.f))
        return set_error(JQ_ERR_INVALID_ARG, "config.txt: freq_base and rms_norm_epsilon must be positive");
    if (cfg.tie_word_embeddings != 0 && cfg.tie_word_embeddings != 1)
        return set_error(JQ_ERR_INVALID_ARG, "config.txt: tie_word_embeddings must be 0 or 1");
    *out = cfg;
    return JQ_OK;
}

extern "C" void jq_model_plan_destroy(jq_model_plan *plan) {
    if (!plan) return;
    std::free(plan->slots);
    std::free(plan);
}

extern "C" int jq_model_q4_0_plan(const jq_weight_set *set, jq_model_plan **out) {
    if (!out) return set_error(JQ_ERR_INVALID_ARG, "null out pointer");
    *out = nullptr;
    if (!set) return set_error(JQ_ERR_INVALID_ARG, "null weight set");
    jq_model_config cfg{};
    if (int rc = jq_model_config_parse(set->config_text ? set->config_text : "", &cfg)) return rc;
    const int64_t H = cfg.hidden_size, I = cfg.intermediate_size, Q = (int64_t)cfg.num_q_heads * cfg.head_dim,
                  KV = (int64_t)cfg.num_kv_heads * cfg.head_dim, V = cfg.vocab_size;
    // out_features x in_features of the seven linears (compute_layer_weight_bytes, transformer_model.cpp:80-104)
    const int64_t rows[7] = {Q, KV, KV, H, I, I, H}, in_features[7] = {H, H, H, Q, H, H, I};
    // w_q, w_o, w_gate, w_down and the first norm start a 256-byte group; w_k, w_v and w_up follow their
    // predecessor directly, which makes q|k|v and gate|up single matrices
    const bool starts_group[kLayerTensors] = {true, false, false, true, true, false, true, true, false};
    std::vector<jq_model_slot> slots;
    size_t cursor = 0;
    for (int layer = 0; layer < cfg.num_layers; ++layer) {
        for (int i = 0; i < kLayerTensors; ++i) {
            std::ostringstream name;
            name << "layer" << layer << "." << kLayerSuffix[i];
            const int rc = i < 7 ? add_slot(set, name.str(), rows[i], in_features[i], true, true, starts_group[i], &slots, &cursor)
                                 : add_slot(set, name.str(), H, 0, false, false, starts_group[i], &slots, &cursor);
            if (rc) return rc;
        }
    }
    if (int rc = add_slot(set, "embed", V, H, false, cfg.tie_word_embeddings == 1, true, &slots, &cursor)) return rc;
    if (int rc = add_slot(set, "final_norm", H, 0, false, false, true, &slots, &cursor)) return rc;
    if (cfg.tie_word_embeddings == 0) {
        if (int rc = add_slot(set, "lm_head", V, H, false, true, true, &slots, &cursor)) return rc;
    }
    jq_model_plan *plan = static_cast<jq_model_plan *>(std::calloc(1, sizeof(jq_model_plan)));
    jq_model_slot *arr = static_cast<jq_model_slot *>(std::malloc(slots.size() * sizeof(jq_model_slot)));
    if (!plan || !arr) {
        std::free(plan);
        std::free(arr);
        return set_error(JQ_ERR_CUDA, "out of host memory");
    }
    std::memcpy(arr, slots.data(), slots.size() * sizeof(jq_model_slot));
    plan->config = cfg;
    plan->slots = arr;
    plan->num_slots = (int)slots.size();
    plan->total_bytes = align_up(cursor, kGroupAlign);
    *out = plan;
    return JQ_OK;
}

extern "C" void jq_model_q4_0_destroy(jq_model_q4_0 *model) {
    if (!model) return;
    if (model->d_base) cudaFree(model->d_base);
    jq_model_plan_destroy(model->plan);
    delete model;
}

extern "C" int jq_model_q4_0_create(const jq_weight_set *set, jq_model_q4_0 **out) {
    if (!out) return set_error(JQ_ERR_INVALID_ARG, "null out pointer");
    *out = nullptr;
    jq_model_plan *plan = nullptr;
    if (int rc = jq_model_q4_0_plan(set, &plan)) return rc;
    jq_model_q4_0 *m = new jq_model_q4_0();
    m->plan = plan;
    void *base = nullptr;
    cudaError_t e = cudaMalloc(&base, plan->total_bytes);
    if (e != cudaSuccess) {
        jq_model_q4_0_destroy(m);
        return jq::cuda_error(e, "cudaMalloc of the model");
    }
    m->d_base = static_cast<uint8_t *>(base);
    for (int i = 0; i < plan->num_slots; ++i) {
        const jq_model_slot &s = plan->slots[i];
        const jq_host_tensor *t = jq_weight_set_find(set, s.name);  // present: the plan was made from this set
        e = cudaMemcpy(m->d_base + s.offset, t->data, s.nbytes, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) {
            jq_model_q4_0_destroy(m);
            return jq::cuda_error(e, "cudaMemcpy of a model tensor");
        }
    }
    const int L = plan->config.num_layers;
    m->layers.resize((size_t)L);
    for (int layer = 0; layer < L; ++layer) {
        const jq_model_slot *s = plan->slots + (size_t)layer * kLayerTensors;
        const uint8_t *b = m->d_base;
        jq_layer_weights_q4_0 &w = m->layers[(size_t)layer];
        w.d_w_q = b + s[0].offset;
        w.d_w_k = b + s[1].offset;
        w.d_w_v = b + s[2].offset;
        w.d_w_o = b + s[3].offset;
        w.d_w_gate = b + s[4].offset;
        w.d_w_up = b + s[5].offset;
        w.d_w_down = b + s[6].offset;
        w.d_w_input_layernorm = reinterpret_cast<const float *>(b + s[7].offset);
        w.d_w_post_attention_layernorm = reinterpret_cast<const float *>(b + s[8].offset);
        w.d_w_qkv = w.d_w_q;
        w.d_w_gate_up = w.d_w_gate;
    }
    const jq_model_slot *tail = plan->slots + (size_t)L * kLayerTensors;
    m->d_embed = m->d_base + tail[0].offset;
    m->embed_dtype = tail[0].dtype;
    m->d_final_norm = reinterpret_cast<const float *>(m->d_base + tail[1].offset);
    if (plan->config.tie_word_embeddings) {
        m->d_lm_head = m->d_embed;
        m->lm_head_dtype = m->embed_dtype;
    } else {
        m->d_lm_head = m->d_base + tail[2].offset;
        m->lm_head_dtype = tail[2].dtype;
    }
    *out = m;
    return JQ_OK;
}

extern "C" const jq_model_config *jq_model_q4_0_config(const jq_model_q4_0 *model) { return model ? &model->plan->config : nullptr; }

extern "C" const jq_model_plan *jq_model_q4_0_layout(const jq_model_q4_0 *model) { return model ? model->plan : nullptr; }

extern "C" const jq_layer_weights_q4_0 *jq_model_q4_0_layer(const jq_model_q4_0 *model, int layer) {
    if (!model || layer < 0 || layer >= (int)model->layers.size()) return nullptr;
    return &model->layers[(size_t)layer];
}

extern "C" const void *jq_model_q4_0_embed(const jq_model_q4_0 *model, int *dtype) {
    if (!model) return nullptr;
    if (dtype) *dtype = model->embed_dtype;
    return model->d_embed;
}

extern "C" const float *jq_model_q4_0_final_norm(const jq_model_q4_0 *model) { return model ? model->d_final_norm : nullptr; }

extern "C" const void *jq_model_q4_0_lm_head(const jq_model_q4_0 *model, int *dtype) {
    if (!model) return nullptr;
    if (dtype) *dtype = model->lm_head_dtype;
    return model->d_lm_head;
}
