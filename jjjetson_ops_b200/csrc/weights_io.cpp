// Q4_0 tensors in the reference's weight formats: fixture-directory reader and offline quantizer, then
// (second half of the file) the safetensors reader and writer.
//
// Follows weight_loader_load_fixture (reference src/model/weight_loader.cpp:193-260, 330-350): the
// same config.txt / manifest.txt grammar, the same limits in spirit (every dim positive, file size
// must match the dims exactly), plus one more tensor type selected by the file's ".q4_0" suffix.
#include <cuda_runtime.h>

#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include <sys/stat.h>

#include "../../include/jq_b200.h"
#include "../../include/jq_weights_io.h"

namespace jq {
int set_error(int status, const char *fmt, ...);
}
using jq::set_error;

namespace {

constexpr int kMaxNdim = 8;
constexpr int kMaxTensors = 1 << 16;

std::string trim(const std::string &s) {
    size_t a = 0, b = s.size();
    while (a < b && (s[a] == ' ' || s[a] == '\t' || s[a] == '\r' || s[a] == '\n')) ++a;
    while (b > a && (s[b - 1] == ' ' || s[b - 1] == '\t' || s[b - 1] == '\r' || s[b - 1] == '\n')) --b;
    return s.substr(a, b - a);
}

bool ends_with(const std::string &s, const char *suffix) {
    const size_t n = std::strlen(suffix);
    return s.size() >= n && s.compare(s.size() - n, n, suffix) == 0;
}

char *dup_c(const std::string &s) {
    char *p = static_cast<char *>(std::malloc(s.size() + 1));
    if (p) std::memcpy(p, s.c_str(), s.size() + 1);
    return p;
}

// Whole regular file -> bytes.  A directory opens as a stream too (and reports a nonsense length), so the
// path is checked first; a file too large for memory is a failed read, not an exception.
bool read_file(const std::string &path, std::vector<char> *out) {
    struct stat st;
    if (stat(path.c_str(), &st) != 0 || !S_ISREG(st.st_mode) || st.st_size < 0) return false;
    std::ifstream in(path, std::ios::binary);
    if (!in.is_open()) return false;
    const size_t n = (size_t)st.st_size;
    try {
        out->resize(n);
    } catch (const std::exception &) {
        return false;
    }
    return n == 0 || (bool)in.read(out->data(), (std::streamsize)n);
}

bool write_file(const std::string &path, const void *data, size_t n) {
    std::ofstream o(path, std::ios::binary | std::ios::trunc);
    if (!o.is_open()) return false;
    if (n) o.write(static_cast<const char *>(data), (std::streamsize)n);
    return (bool)o;
}

void free_tensor(jq_host_tensor *t) {
    std::free(t->name);
    std::free(t->data);
    std::free(t->dims);
    *t = jq_host_tensor{};
}

struct ManifestEntry {
    std::string name, file;
    std::vector<int64_t> dims;
};

int parse_manifest(const std::string &dir, std::vector<ManifestEntry> *entries) {
    std::ifstream in(dir + "/manifest.txt");
    if (!in.is_open()) return set_error(JQ_ERR_INVALID_ARG, "cannot open %s/manifest.txt", dir.c_str());
    std::string line;
    int lineno = 0;
    while (std::getline(in, line)) {
        ++lineno;
        line = trim(line);
        if (line.empty() || line[0] == '#') continue;
        if ((int)entries->size() >= kMaxTensors) return set_error(JQ_ERR_TOO_LARGE, "manifest.txt: too many tensors");
        std::istringstream iss(line);
        ManifestEntry e;
        int ndim = 0;
        if (!(iss >> e.name >> ndim) || ndim <= 0 || ndim > kMaxNdim)
            return set_error(JQ_ERR_SHAPE, "manifest.txt:%d: expected \"name ndim dims... file\"", lineno);
        for (int i = 0; i < ndim; ++i) {
            long long d = 0;
            if (!(iss >> d) || d <= 0) return set_error(JQ_ERR_SHAPE, "manifest.txt:%d: bad dimension %d", lineno, i);
            e.dims.push_back((int64_t)d);
        }
        if (!(iss >> e.file)) return set_error(JQ_ERR_SHAPE, "manifest.txt:%d: missing file name", lineno);
        if (e.file.find("..") != std::string::npos || (!e.file.empty() && e.file[0] == '/'))
            return set_error(JQ_ERR_INVALID_ARG, "manifest.txt:%d: file must be a path inside the fixture", lineno);
        entries->push_back(std::move(e));
    }
    return JQ_OK;
}

// product of the (positive) dims, or -1 when it would not fit a byte count
int64_t numel_of(const std::vector<int64_t> &dims) {
    int64_t n = 1;
    for (int64_t d : dims) {
        if (d <= 0 || n > (INT64_MAX / 64) / d) return -1;
        n *= d;
    }
    return n;
}

// bytes a tensor file must have, or -1 with the error recorded
int64_t expected_bytes(const ManifestEntry &e, int *dtype) {
    if (ends_with(e.file, ".q4_0")) {
        *dtype = JQ_WEIGHT_Q4_0;
        if (e.dims.size() != 2 || e.dims[1] % 32 != 0) {
            set_error(JQ_ERR_SHAPE, "%s: a Q4_0 tensor needs dims [rows, K] with K %% 32 == 0", e.name.c_str());
            return -1;
        }
        if (numel_of(e.dims) < 0) {
            set_error(JQ_ERR_TOO_LARGE, "%s: dims too large", e.name.c_str());
            return -1;
        }
        return (int64_t)jq_q4_0_bytes(e.dims[0], e.dims[1]);
    }
    *dtype = JQ_WEIGHT_F32;
    const int64_t n = numel_of(e.dims);
    if (n < 0) {
        set_error(JQ_ERR_TOO_LARGE, "%s: dims too large", e.name.c_str());
        return -1;
    }
    return n * (int64_t)sizeof(float);
}

bool config_lookup(const char *text, const char *key, double *value) {
    if (!text || !key) return false;
    std::istringstream in(text);
    std::string line;
    while (std::getline(in, line)) {
        line = trim(line);
        const size_t eq = line.find('=');
        if (line.empty() || line[0] == '#' || eq == std::string::npos) continue;
        if (trim(line.substr(0, eq)) != key) continue;
        char *end = nullptr;
        const std::string v = trim(line.substr(eq + 1));
        errno = 0;
        const double d = std::strtod(v.c_str(), &end);
        if (end == v.c_str() || errno != 0) return false;
        *value = d;
        return true;
    }
    return false;
}

// in_features of a linear weight by its name, 0 when the tensor is not a linear weight
int64_t linear_in_features(const std::string &name, const char *config) {
    double hidden = 0, inter = 0, qh = 0, hd = 0, tied = 0;
    config_lookup(config, "hidden_size", &hidden);
    config_lookup(config, "intermediate_size", &inter);
    config_lookup(config, "num_q_heads", &qh);
    config_lookup(config, "head_dim", &hd);
    config_lookup(config, "tie_word_embeddings", &tied);
    for (const char *s : {".w_q", ".w_k", ".w_v", ".w_gate", ".w_up"}) {
        if (ends_with(name, s)) return (int64_t)hidden;
    }
    if (ends_with(name, ".w_o")) return (int64_t)(qh * hd);
    if (ends_with(name, ".w_down")) return (int64_t)inter;
    if (name == "embed" && tied != 0) return (int64_t)hidden;  // the tied table doubles as lm_head: [vocab][hidden]
    return 0;
}

}  // namespace

extern "C" void jq_weight_set_destroy(jq_weight_set *set) {
    if (!set) return;
    for (int i = 0; i < set->num_tensors; ++i) free_tensor(&set->tensors[i]);
    std::free(set->tensors);
    std::free(set->config_text);
    std::free(set);
}

extern "C" const jq_host_tensor *jq_weight_set_find(const jq_weight_set *set, const char *name) {
    if (!set || !name) return nullptr;
    for (int i = 0; i < set->num_tensors; ++i) {
        if (std::strcmp(set->tensors[i].name, name) == 0) return &set->tensors[i];
    }
    return nullptr;
}

extern "C" int jq_weight_set_config_value(const jq_weight_set *set, const char *key, double *value) {
    double v = 0;
    if (!set || !value || !config_lookup(set->config_text, key, &v)) return 0;
    *value = v;
    return 1;
}

extern "C" int jq_weights_load_fixture(const char *dir, jq_weight_set **out) {
    if (!out) return set_error(JQ_ERR_INVALID_ARG, "null out pointer");
    *out = nullptr;
    if (!dir) return set_error(JQ_ERR_INVALID_ARG, "null path");
    std::vector<ManifestEntry> entries;
    if (int rc = parse_manifest(dir, &entries)) return rc;
    jq_weight_set *set = static_cast<jq_weight_set *>(std::calloc(1, sizeof(jq_weight_set)));
    if (!set) return set_error(JQ_ERR_CUDA, "out of host memory");
    std::vector<char> cfg;
    read_file(std::string(dir) + "/config.txt", &cfg);  // optional, as for the reference's safetensors path
    set->config_text = dup_c(std::string(cfg.begin(), cfg.end()));
    set->tensors = static_cast<jq_host_tensor *>(std::calloc(entries.empty() ? 1 : entries.size(), sizeof(jq_host_tensor)));
    if (!set->tensors || !set->config_text) {
        jq_weight_set_destroy(set);
        return set_error(JQ_ERR_CUDA, "out of host memory");
    }
    for (const ManifestEntry &e : entries) {
        int dtype = 0;
        const int64_t want = expected_bytes(e, &dtype);
        if (want < 0) {
            jq_weight_set_destroy(set);
            return JQ_ERR_SHAPE;
        }
        std::vector<char> blob;
        const std::string path = std::string(dir) + "/" + e.file;
        if (!read_file(path, &blob)) {
            jq_weight_set_destroy(set);
            return set_error(JQ_ERR_INVALID_ARG, "cannot read %s", path.c_str());
        }
        if ((int64_t)blob.size() != want) {
            jq_weight_set_destroy(set);
            return set_error(JQ_ERR_SHAPE, "%s: %lld bytes on disk, %lld expected from the manifest dims", path.c_str(),
                             (long long)blob.size(), (long long)want);
        }
        jq_host_tensor *t = &set->tensors[set->num_tensors];
        t->name = dup_c(e.name);
        t->dims = static_cast<int64_t *>(std::malloc(e.dims.size() * sizeof(int64_t)));
        t->data = std::malloc(blob.empty() ? 1 : blob.size());
        if (!t->name || !t->dims || !t->data) {
            free_tensor(t);
            jq_weight_set_destroy(set);
            return set_error(JQ_ERR_CUDA, "out of host memory");
        }
        std::memcpy(t->dims, e.dims.data(), e.dims.size() * sizeof(int64_t));
        std::memcpy(t->data, blob.data(), blob.size());
        t->ndim = (int)e.dims.size();
        t->dtype = dtype;
        t->nbytes = blob.size();
        ++set->num_tensors;
    }
    *out = set;
    return JQ_OK;
}

extern "C" int jq_weights_quantize_fixture(const char *src_dir, const char *dst_dir, int *n_quantized) {
    if (n_quantized) *n_quantized = 0;
    if (!src_dir || !dst_dir) return set_error(JQ_ERR_INVALID_ARG, "null path");
    jq_weight_set *set = nullptr;
    if (int rc = jq_weights_load_fixture(src_dir, &set)) return rc;
    if (mkdir(dst_dir, 0777) != 0 && errno != EEXIST) {
        jq_weight_set_destroy(set);
        return set_error(JQ_ERR_INVALID_ARG, "cannot create %s: %s", dst_dir, std::strerror(errno));
    }
    const std::string dst(dst_dir);
    std::string manifest;
    int rc = JQ_OK, converted = 0;
    cudaStream_t stream = nullptr;
    void *d_in = nullptr, *d_out = nullptr;
    size_t cap_in = 0, cap_out = 0;
    if (!write_file(dst + "/config.txt", set->config_text, std::strlen(set->config_text)))
        rc = set_error(JQ_ERR_INVALID_ARG, "cannot write %s/config.txt", dst_dir);
    for (int i = 0; rc == JQ_OK && i < set->num_tensors; ++i) {
        const jq_host_tensor &t = set->tensors[i];
        std::string base(t.name);
        for (char &ch : base) {
            if (ch == '.') ch = '_';  // the reference's file naming (tests/fixture_utils.py:95)
        }
        int64_t numel = 1;
        for (int d = 0; d < t.ndim; ++d) numel *= t.dims[d];
        const int64_t K = t.dtype == JQ_WEIGHT_F32 ? linear_in_features(t.name, set->config_text) : 0;
        std::ostringstream line;
        if (K > 0 && K % 32 == 0 && numel % K == 0) {
            const int64_t rows = numel / K;
            const size_t out_bytes = jq_q4_0_bytes(rows, K);
            std::vector<char> host_out(out_bytes);
            cudaError_t e = cudaSuccess;
            if (!stream) e = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
            if (e == cudaSuccess && t.nbytes > cap_in) {
                cudaFree(d_in);
                d_in = nullptr;
                e = cudaMalloc(&d_in, t.nbytes);
                cap_in = e == cudaSuccess ? t.nbytes : 0;
            }
            if (e == cudaSuccess && out_bytes > cap_out) {
                cudaFree(d_out);
                d_out = nullptr;
                e = cudaMalloc(&d_out, out_bytes);
                cap_out = e == cudaSuccess ? out_bytes : 0;
            }
            if (e == cudaSuccess) e = cudaMemcpyAsync(d_in, t.data, t.nbytes, cudaMemcpyHostToDevice, stream);
            if (e != cudaSuccess) {
                rc = set_error(JQ_ERR_CUDA, "%s: %s", t.name, cudaGetErrorString(e));
                break;
            }
            rc = jq_quantize_q4_0_device(stream, static_cast<const float *>(d_in), d_out, rows, K);
            if (rc != JQ_OK) break;
            e = cudaMemcpyAsync(host_out.data(), d_out, out_bytes, cudaMemcpyDeviceToHost, stream);
            if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
            if (e != cudaSuccess) {
                rc = set_error(JQ_ERR_CUDA, "%s: %s", t.name, cudaGetErrorString(e));
                break;
            }
            const std::string file = base + ".q4_0";
            if (!write_file(dst + "/" + file, host_out.data(), out_bytes)) {
                rc = set_error(JQ_ERR_INVALID_ARG, "cannot write %s/%s", dst_dir, file.c_str());
                break;
            }
            line << t.name << " 2 " << rows << " " << K << " " << file;
            ++converted;
        } else {
            const std::string file = base + (t.dtype == JQ_WEIGHT_Q4_0 ? ".q4_0" : ".f32");
            if (!write_file(dst + "/" + file, t.data, t.nbytes)) {
                rc = set_error(JQ_ERR_INVALID_ARG, "cannot write %s/%s", dst_dir, file.c_str());
                break;
            }
            line << t.name << " " << t.ndim;
            for (int d = 0; d < t.ndim; ++d) line << " " << t.dims[d];
            line << " " << file;
        }
        manifest += line.str() + "\n";
    }
    if (rc == JQ_OK && !write_file(dst + "/manifest.txt", manifest.data(), manifest.size()))
        rc = set_error(JQ_ERR_INVALID_ARG, "cannot write %s/manifest.txt", dst_dir);
    cudaFree(d_in);
    cudaFree(d_out);
    if (stream) cudaStreamDestroy(stream);
    jq_weight_set_destroy(set);
    if (n_quantized) *n_quantized = converted;
    return rc;
}

// ---------------------------------------------------------------------------------------------
// The single-file format: safetensors.
//
// Follows weight_loader_load_safetensors and safetensors_read_file (reference
// src/model/weight_loader.h:42-47, src/model/safetensors_reader.cpp:400-418): 8 bytes of little-endian
// header length, a JSON header {name: {dtype, shape, data_offsets}}, then the data the offsets point
// into; "__metadata__" is skipped, names are taken as they are, a config.txt beside the file is picked
// up when present, and a dtype the loader does not know is an error.  The extra tensor type keeps the
// file readable by any safetensors tool: a Q4_0 tensor "w" is stored under the name "w.q4_0" as U8
// with shape [rows, K / 32, 18], one innermost row per block_q4_0.
namespace {

constexpr size_t kMaxHeaderBytes = 100u << 20;

struct JsonCursor {
    const char *p, *end;
    void skip_ws() {
        while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) ++p;
    }
    bool eat(char c) {
        skip_ws();
        if (p < end && *p == c) {
            ++p;
            return true;
        }
        return false;
    }
};

void append_utf8(std::string *s, unsigned cp) {
    if (cp < 0x80) {
        s->push_back((char)cp);
    } else if (cp < 0x800) {
        s->push_back((char)(0xC0 | (cp >> 6)));
        s->push_back((char)(0x80 | (cp & 0x3F)));
    } else {
        s->push_back((char)(0xE0 | (cp >> 12)));
        s->push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
        s->push_back((char)(0x80 | (cp & 0x3F)));
    }
}

bool json_string(JsonCursor *c, std::string *out) {
    if (!c->eat('"')) return false;
    out->clear();
    while (c->p < c->end) {
        const char ch = *c->p++;
        if (ch == '"') return true;
        if (ch != '\\') {
            out->push_back(ch);
            continue;
        }
        if (c->p >= c->end) return false;
        const char e = *c->p++;
        switch (e) {
            case '"': case '\\': case '/': out->push_back(e); break;
            case 'b': out->push_back('\b'); break;
            case 'f': out->push_back('\f'); break;
            case 'n': out->push_back('\n'); break;
            case 'r': out->push_back('\r'); break;
            case 't': out->push_back('\t'); break;
            case 'u': {
                if (c->end - c->p < 4) return false;
                unsigned cp = 0;
                for (int i = 0; i < 4; ++i) {
                    const char h = *c->p++;
                    cp <<= 4;
                    if (h >= '0' && h <= '9') cp |= (unsigned)(h - '0');
                    else if (h >= 'a' && h <= 'f') cp |= (unsigned)(h - 'a' + 10);
                    else if (h >= 'A' && h <= 'F') cp |= (unsigned)(h - 'A' + 10);
                    else return false;
                }
                append_utf8(out, cp);
                break;
            }
            default: return false;
        }
    }
    return false;
}

bool json_uint(JsonCursor *c, int64_t *out) {
    c->skip_ws();
    if (c->p >= c->end || *c->p < '0' || *c->p > '9') return false;
    int64_t v = 0;
    while (c->p < c->end && *c->p >= '0' && *c->p <= '9') {
        if (v > (INT64_MAX - 9) / 10) return false;
        v = v * 10 + (*c->p++ - '0');
    }
    *out = v;
    return true;
}

bool json_uint_array(JsonCursor *c, std::vector<int64_t> *out) {
    out->clear();
    if (!c->eat('[')) return false;
    if (c->eat(']')) return true;
    for (;;) {
        int64_t v = 0;
        if (!json_uint(c, &v)) return false;
        out->push_back(v);
        if (c->eat(']')) return true;
        if (!c->eat(',')) return false;
    }
}

// skips one JSON value of any kind (used for "__metadata__" and for keys this reader does not need)
bool json_skip(JsonCursor *c, int depth = 0) {
    if (depth > 32) return false;
    c->skip_ws();
    if (c->p >= c->end) return false;
    if (*c->p == '"') {
        std::string s;
        return json_string(c, &s);
    }
    if (*c->p == '{' || *c->p == '[') {
        const char close = *c->p == '{' ? '}' : ']';
        const bool object = *c->p == '{';
        ++c->p;
        if (c->eat(close)) return true;
        for (;;) {
            if (object) {
                std::string key;
                if (!json_string(c, &key) || !c->eat(':')) return false;
            }
            if (!json_skip(c, depth + 1)) return false;
            if (c->eat(close)) return true;
            if (!c->eat(',')) return false;
        }
    }
    // number, true, false, null
    const char *start = c->p;
    while (c->p < c->end && *c->p != ',' && *c->p != '}' && *c->p != ']' && *c->p != ' ' && *c->p != '\n' && *c->p != '\t' &&
           *c->p != '\r')
        ++c->p;
    return c->p > start;
}

struct StEntry {
    std::string name, dtype;
    std::vector<int64_t> shape, offsets;
};

int parse_st_header(const char *json, size_t n, std::vector<StEntry> *entries) {
    JsonCursor c{json, json + n};
    if (!c.eat('{')) return set_error(JQ_ERR_SHAPE, "safetensors header is not a JSON object");
    if (c.eat('}')) return JQ_OK;
    for (;;) {
        StEntry e;
        if (!json_string(&c, &e.name) || !c.eat(':')) return set_error(JQ_ERR_SHAPE, "safetensors header: expected \"name\":");
        if (e.name == "__metadata__") {
            if (!json_skip(&c)) return set_error(JQ_ERR_SHAPE, "safetensors header: malformed __metadata__");
        } else {
            if ((int)entries->size() >= kMaxTensors) return set_error(JQ_ERR_TOO_LARGE, "safetensors header: too many tensors");
            if (!c.eat('{')) return set_error(JQ_ERR_SHAPE, "safetensors header: %s is not an object", e.name.c_str());
            if (!c.eat('}')) {
                for (;;) {
                    std::string key;
                    if (!json_string(&c, &key) || !c.eat(':')) return set_error(JQ_ERR_SHAPE, "safetensors header: malformed entry %s", e.name.c_str());
                    bool ok;
                    if (key == "dtype") ok = json_string(&c, &e.dtype);
                    else if (key == "shape") ok = json_uint_array(&c, &e.shape);
                    else if (key == "data_offsets") ok = json_uint_array(&c, &e.offsets);
                    else ok = json_skip(&c);
                    if (!ok) return set_error(JQ_ERR_SHAPE, "safetensors header: bad value of %s.%s", e.name.c_str(), key.c_str());
                    if (c.eat('}')) break;
                    if (!c.eat(',')) return set_error(JQ_ERR_SHAPE, "safetensors header: malformed entry %s", e.name.c_str());
                }
            }
            if (e.dtype.empty() || e.shape.empty() || e.shape.size() > (size_t)kMaxNdim || e.offsets.size() != 2 ||
                e.offsets[1] <= e.offsets[0])
                return set_error(JQ_ERR_SHAPE, "safetensors header: %s needs dtype, a shape of 1..%d dims and data_offsets [begin, end)",
                                 e.name.c_str(), kMaxNdim);
            entries->push_back(std::move(e));
        }
        if (c.eat('}')) break;
        if (!c.eat(',')) return set_error(JQ_ERR_SHAPE, "safetensors header: expected ',' or '}'");
    }
    return JQ_OK;
}

std::string json_quote(const char *s) {
    std::string q = "\"";
    for (; *s; ++s) {
        const unsigned char ch = (unsigned char)*s;
        if (ch == '"' || ch == '\\') {
            q.push_back('\\');
            q.push_back((char)ch);
        } else if (ch < 0x20) {
            char buf[8];
            std::snprintf(buf, sizeof(buf), "\\u%04x", ch);
            q += buf;
        } else {
            q.push_back((char)ch);
        }
    }
    q.push_back('"');
    return q;
}

std::string dir_of(const std::string &path) {
    const size_t slash = path.find_last_of('/');
    return slash == std::string::npos ? std::string(".") : (slash == 0 ? std::string("/") : path.substr(0, slash));
}

}  // namespace

extern "C" int jq_weights_load_safetensors(const char *path, jq_weight_set **out) {
    if (!out) return set_error(JQ_ERR_INVALID_ARG, "null out pointer");
    *out = nullptr;
    if (!path) return set_error(JQ_ERR_INVALID_ARG, "null path");
    std::vector<char> file;
    if (!read_file(path, &file)) return set_error(JQ_ERR_INVALID_ARG, "cannot read %s", path);
    if (file.size() < 8) return set_error(JQ_ERR_SHAPE, "%s: shorter than the 8-byte header length", path);
    uint64_t header_len = 0;
    for (int i = 7; i >= 0; --i) header_len = (header_len << 8) | (unsigned char)file[(size_t)i];
    if (header_len > kMaxHeaderBytes || header_len > file.size() - 8)
        return set_error(JQ_ERR_SHAPE, "%s: header length %llu exceeds the file", path, (unsigned long long)header_len);
    std::vector<StEntry> entries;
    if (int rc = parse_st_header(file.data() + 8, (size_t)header_len, &entries)) return rc;
    if (entries.empty()) return set_error(JQ_ERR_SHAPE, "%s: no tensors", path);
    const char *blob = file.data() + 8 + header_len;
    const uint64_t blob_size = file.size() - 8 - header_len;

    jq_weight_set *set = static_cast<jq_weight_set *>(std::calloc(1, sizeof(jq_weight_set)));
    if (!set) return set_error(JQ_ERR_CUDA, "out of host memory");
    std::vector<char> cfg;
    read_file(dir_of(path) + "/config.txt", &cfg);  // optional (weight_loader.h:44-45)
    set->config_text = dup_c(std::string(cfg.begin(), cfg.end()));
    set->tensors = static_cast<jq_host_tensor *>(std::calloc(entries.size(), sizeof(jq_host_tensor)));
    if (!set->tensors || !set->config_text) {
        jq_weight_set_destroy(set);
        return set_error(JQ_ERR_CUDA, "out of host memory");
    }
    for (const StEntry &e : entries) {
        std::string name = e.name;
        std::vector<int64_t> dims = e.shape;
        int dtype = JQ_WEIGHT_F32;
        int64_t want = 0;
        bool overflow = false;
        int64_t numel = 1;
        for (int64_t d : e.shape) {
            if (d != 0 && numel > INT64_MAX / 32 / d) {
                overflow = true;
                break;
            }
            numel *= d;
        }
        if (e.dtype == "F32") {
            want = numel * (int64_t)sizeof(float);
        } else if (e.dtype == "U8" && ends_with(e.name, ".q4_0") && e.name.size() > 5 && e.shape.size() == 3 && e.shape[2] == 18) {
            dtype = JQ_WEIGHT_Q4_0;
            name = e.name.substr(0, e.name.size() - 5);
            dims = {e.shape[0], e.shape[1] * 32};
            want = numel;
        } else {
            jq_weight_set_destroy(set);
            return set_error(JQ_ERR_UNSUPPORTED, "%s: unsupported dtype %s for tensor %s (F32, or U8 [rows, K/32, 18] named *.q4_0)", path,
                             e.dtype.c_str(), e.name.c_str());
        }
        const uint64_t begin = (uint64_t)e.offsets[0], end = (uint64_t)e.offsets[1];
        if (overflow || numel <= 0 || end > blob_size || (int64_t)(end - begin) != want) {
            jq_weight_set_destroy(set);
            return set_error(JQ_ERR_SHAPE, "%s: tensor %s: data_offsets [%llu, %llu) do not match its shape (%lld bytes) or the file", path,
                             e.name.c_str(), (unsigned long long)begin, (unsigned long long)end, (long long)want);
        }
        jq_host_tensor *t = &set->tensors[set->num_tensors];
        t->name = dup_c(name);
        t->dims = static_cast<int64_t *>(std::malloc(dims.size() * sizeof(int64_t)));
        t->data = std::malloc((size_t)want);
        if (!t->name || !t->dims || !t->data) {
            free_tensor(t);
            jq_weight_set_destroy(set);
            return set_error(JQ_ERR_CUDA, "out of host memory");
        }
        std::memcpy(t->dims, dims.data(), dims.size() * sizeof(int64_t));
        std::memcpy(t->data, blob + begin, (size_t)want);
        t->ndim = (int)dims.size();
        t->dtype = dtype;
        t->nbytes = (size_t)want;
        ++set->num_tensors;
    }
    *out = set;
    return JQ_OK;
}

extern "C" int jq_weights_save_safetensors(const jq_weight_set *set, const char *path) {
    if (!set || !path) return set_error(JQ_ERR_INVALID_ARG, "null argument");
    if (set->num_tensors <= 0) return set_error(JQ_ERR_INVALID_ARG, "a safetensors file needs at least one tensor");
    // entries in name order, data in the same order, as the reference's own writer lays a file out
    // (tests/fixture_utils.py:30-53)
    std::vector<int> order((size_t)set->num_tensors);
    for (int i = 0; i < set->num_tensors; ++i) order[(size_t)i] = i;
    for (size_t i = 1; i < order.size(); ++i) {  // insertion sort: a handful of tensors per layer
        const int v = order[i];
        size_t j = i;
        while (j > 0 && std::strcmp(set->tensors[order[j - 1]].name, set->tensors[v].name) > 0) {
            order[j] = order[j - 1];
            --j;
        }
        order[j] = v;
    }
    std::string header = "{";
    uint64_t offset = 0;
    for (size_t k = 0; k < order.size(); ++k) {
        const jq_host_tensor &t = set->tensors[order[k]];
        std::ostringstream e;
        if (t.dtype == JQ_WEIGHT_Q4_0) {
            if (t.ndim != 2 || t.dims[1] % 32 != 0 || t.nbytes != jq_q4_0_bytes(t.dims[0], t.dims[1]))
                return set_error(JQ_ERR_SHAPE, "%s: a Q4_0 tensor needs dims [rows, K] with K %% 32 == 0", t.name);
            e << json_quote((std::string(t.name) + ".q4_0").c_str()) << ":{\"dtype\":\"U8\",\"shape\":[" << t.dims[0] << "," << t.dims[1] / 32
              << ",18]";
        } else if (t.dtype == JQ_WEIGHT_F32) {
            e << json_quote(t.name) << ":{\"dtype\":\"F32\",\"shape\":[";
            for (int d = 0; d < t.ndim; ++d) e << (d ? "," : "") << t.dims[d];
            e << "]";
        } else {
            return set_error(JQ_ERR_INVALID_ARG, "%s: unknown dtype %d", t.name, t.dtype);
        }
        e << ",\"data_offsets\":[" << offset << "," << offset + t.nbytes << "]}";
        offset += t.nbytes;
        header += (k ? "," : "") + e.str();
    }
    header += "}";
    while (header.size() % 8 != 0) header.push_back(' ');  // the data starts on an 8-byte boundary
    std::ofstream o(path, std::ios::binary | std::ios::trunc);
    if (!o.is_open()) return set_error(JQ_ERR_INVALID_ARG, "cannot write %s", path);
    unsigned char len[8];
    for (int i = 0; i < 8; ++i) len[i] = (unsigned char)((uint64_t)header.size() >> (8 * i));
    o.write(reinterpret_cast<const char *>(len), 8);
    o.write(header.data(), (std::streamsize)header.size());
    for (int idx : order) {
        const jq_host_tensor &t = set->tensors[idx];
        if (t.nbytes) o.write(static_cast<const char *>(t.data), (std::streamsize)t.nbytes);
    }
    o.flush();
    if (!o) return set_error(JQ_ERR_INVALID_ARG, "short write to %s", path);
    return JQ_OK;
}
