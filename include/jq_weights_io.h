/* jq_weights_io.h - Q4_0 tensors in the reference's two weight formats (fixture directory, safetensors
 * file): readers, writer and offline quantizer.
 *
 * The reference's loader (src/model/weight_loader.h:12-47) knows one tensor type, F32: a fixture is a
 * directory with config.txt ("key=value" lines), manifest.txt (one line per tensor:
 * "name ndim dim0 .. dimN-1 file") and one raw little-endian .f32 file per tensor
 * (src/model/weight_loader.cpp:193-260, tests/fixture_utils.py:74-103).  Its design notes list a
 * quantized type as future work (doc/design/phase2_lifecycle.md:84).  This header adds that type
 * without changing the format's grammar:
 *
 *   - a manifest entry whose file ends in ".q4_0" is a raw array of 18-byte block_q4_0
 *     (src/cuda/mm_q4_0_q8_1.cu:35-38; the ggml layout, so a GGUF Q4_0 tensor maps onto it byte for
 *     byte); its two dims are [rows, K]: `rows` output features, each K / 32 consecutive blocks;
 *   - everything else is read exactly as the reference reads it.
 *
 * jq_weight_set mirrors WeightLoadResult / HostTensor (weight_loader.h:17-30) with a dtype-tagged
 * void* payload.  Nothing here touches a GPU except jq_weights_quantize_fixture, which quantizes with
 * the library's own CUDA kernel (jq_quantize_q4_0_device): there is no CPU implementation of the
 * quantizer in the library.
 */
#ifndef JQ_WEIGHTS_IO_H_
#define JQ_WEIGHTS_IO_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum jq_weight_dtype {
    JQ_WEIGHT_F32 = 0,  /* WEIGHT_DTYPE_F32 (weight_loader.h:13) */
    JQ_WEIGHT_Q4_0 = 1  /* raw block_q4_0, dims = [rows, K] */
} jq_weight_dtype;

typedef struct jq_host_tensor {
    char *name;
    void *data;     /* float[numel] or block_q4_0[rows * K / 32] */
    int64_t *dims;
    int ndim;
    int dtype;      /* jq_weight_dtype */
    size_t nbytes;
} jq_host_tensor;

typedef struct jq_weight_set {
    jq_host_tensor *tensors;
    int num_tensors;
    char *config_text;  /* config.txt verbatim ("" when absent): parsing it is the engine's business */
} jq_weight_set;

/* weight_loader_load_fixture (weight_loader.h:40) with the extra tensor type.  Returns JQ_OK or a
 * status from jq_b200.h (message in jq_last_error()); *out is NULL on failure. */
int jq_weights_load_fixture(const char *dir, jq_weight_set **out);

/* weight_loader_load_safetensors (weight_loader.h:42-47; reader src/model/safetensors_reader.cpp:400-418)
 * with the extra tensor type.  `path` is one .safetensors file: 8 bytes of little-endian header length,
 * a JSON header {name: {"dtype", "shape", "data_offsets"}}, then the data.  As in the reference:
 * "__metadata__" is skipped, names are kept as they are, a config.txt in the file's directory is picked
 * up when there is one, a file without tensors and a dtype the loader does not know are errors.
 * F32 tensors are read as the reference reads them.  A Q4_0 tensor "w" is stored under the name
 * "w.q4_0" with dtype "U8" and shape [rows, K / 32, 18] (one innermost row per block_q4_0), so the
 * file stays readable by any safetensors tool; it is returned as "w" with dims [rows, K]. */
int jq_weights_load_safetensors(const char *path, jq_weight_set **out);

/* Writes a set as one .safetensors file in that convention: entries in name order with their data in
 * the same order (the layout of the reference's writer, tests/fixture_utils.py:30-53), no
 * "__metadata__", header padded with spaces to a multiple of 8 bytes.  config_text is not written:
 * config.txt stays a file of its own beside the weights. */
int jq_weights_save_safetensors(const jq_weight_set *set, const char *path);

/* weight_load_result_destroy / weight_load_result_find (weight_loader.h:34-36). */
void jq_weight_set_destroy(jq_weight_set *set);
const jq_host_tensor *jq_weight_set_find(const jq_weight_set *set, const char *name);

/* One value of config.txt as a number; returns 0 and leaves *value alone when the key is absent. */
int jq_weight_set_config_value(const jq_weight_set *set, const char *key, double *value);

/* Offline quantizer: copies the fixture at src_dir to dst_dir, replacing every linear weight by its
 * Q4_0 form.  A tensor is a linear weight when its name ends in one of w_q, w_k, w_v, w_o, w_gate,
 * w_up, w_down (the seven linears of transformer_runner.cpp:214-216, 294, 319-328) or is "embed" while
 * tie_word_embeddings=1.  The engine reads such a tensor as `out_features` rows of `in_features`
 * contiguous values (linear_forward_device, src/cuda/linear.cu:19-23: lda = in_features) whatever the
 * manifest's dims say, so K comes from config.txt (hidden_size; num_q_heads * head_dim for w_o;
 * intermediate_size for w_down) and rows = numel / K.  Tensors whose K is not a multiple of 32 are
 * left in F32.  *n_quantized (may be NULL) receives the number of tensors converted.
 * Needs a CUDA device: the conversion runs jq_quantize_q4_0_device. */
int jq_weights_quantize_fixture(const char *src_dir, const char *dst_dir, int *n_quantized);

#ifdef __cplusplus
}
#endif

#endif /* JQ_WEIGHTS_IO_H_ */
