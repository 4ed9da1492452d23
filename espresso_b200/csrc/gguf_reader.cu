// GGUF file front end: header, key/value metadata, tensor directory, aligned tensor data (GGUF versions 2 and 3),
// the model shape the reference derives from it, the GGUF -> Espresso tensor-name mapping, and an engine built
// straight from the file.  Replaces GGUFModelLoader.prepare (Sources/EspressoGGUF/GGUFModelLoader.swift:273-405),
// whose parsing and conversion live in the un-vendored Edgerunner package: quantised Q8_0 / Q4_0 blocks go to the
// device as they are (no fp16 materialisation, :341-369), the tied LM head reuses the embedding tensor (:224-263),
// the shape follows :297-326 and the published GGUF key names.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>

#include "engine.h"

namespace esp {

enum GgufValueType : uint32_t {
    GGUF_U8 = 0, GGUF_I8 = 1, GGUF_U16 = 2, GGUF_I16 = 3, GGUF_U32 = 4, GGUF_I32 = 5, GGUF_F32 = 6, GGUF_BOOL = 7,
    GGUF_STRING = 8, GGUF_ARRAY = 9, GGUF_U64 = 10, GGUF_I64 = 11, GGUF_F64 = 12
};

struct GgufValue {
    uint32_t type = 0;
    int64_t i = 0;          // integer and bool values
    double f = 0.0;         // floating-point values (integers are mirrored here)
    std::string s;          // string values
    uint64_t count = 0;     // arrays: element count (the elements themselves are skipped)
    uint32_t elem_type = 0;
};

struct GgufTensor {
    std::string name;
    uint32_t n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};  // dims[0] is the contiguous one (a matrix's columns)
    uint32_t type = 0;                // GGML type id
    uint64_t offset = 0;              // from the start of the data section
    uint64_t nbytes = 0;
};

static bool ggml_block(uint32_t type, uint64_t* elems, uint64_t* bytes) {
    switch (type) {
        case ESP_CUDA_F32: *elems = 1; *bytes = 4; return true;
        case ESP_CUDA_F16: case ESP_CUDA_BF16: *elems = 1; *bytes = 2; return true;
        case ESP_CUDA_Q4_0: *elems = 32; *bytes = 18; return true;
        case ESP_CUDA_Q8_0: *elems = 32; *bytes = 34; return true;
    }
    return false;
}

class GgufFile {
  public:
    ~GgufFile() {
        if (map_ && map_ != MAP_FAILED) munmap(map_, size_);
        if (fd_ >= 0) close(fd_);
    }
    int32_t open(const char* path);
    const GgufValue* find(const std::string& key) const {
        auto it = kv.find(key);
        return it == kv.end() ? nullptr : &it->second;
    }
    const GgufTensor* tensor(const std::string& name) const {
        for (auto& t : tensors)
            if (t.name == name) return &t;
        return nullptr;
    }
    const uint8_t* data_of(const GgufTensor& t) const { return static_cast<const uint8_t*>(map_) + data_start_ + t.offset; }

    uint32_t version = 0;
    uint64_t alignment = 32;
    std::map<std::string, GgufValue> kv;
    std::vector<GgufTensor> tensors;

  private:
    bool take(void* dst, size_t n) {
        if (cur_ + n > size_) return false;
        memcpy(dst, static_cast<const uint8_t*>(map_) + cur_, n);
        cur_ += n;
        return true;
    }
    bool take_string(std::string* s) {
        uint64_t n = 0;
        if (!take(&n, 8) || n > size_ - cur_) return false;
        s->assign(static_cast<const char*>(map_) + cur_, (size_t)n);
        cur_ += n;
        return true;
    }
    bool take_value(uint32_t type, GgufValue* v, bool in_array);

    int fd_ = -1;
    void* map_ = nullptr;
    size_t size_ = 0, cur_ = 0, data_start_ = 0;
};

bool GgufFile::take_value(uint32_t type, GgufValue* v, bool in_array) {
    v->type = type;
    switch (type) {
        case GGUF_U8: { uint8_t x; if (!take(&x, 1)) return false; v->i = x; break; }
        case GGUF_I8: { int8_t x; if (!take(&x, 1)) return false; v->i = x; break; }
        case GGUF_BOOL: { uint8_t x; if (!take(&x, 1)) return false; v->i = x != 0; break; }
        case GGUF_U16: { uint16_t x; if (!take(&x, 2)) return false; v->i = x; break; }
        case GGUF_I16: { int16_t x; if (!take(&x, 2)) return false; v->i = x; break; }
        case GGUF_U32: { uint32_t x; if (!take(&x, 4)) return false; v->i = x; break; }
        case GGUF_I32: { int32_t x; if (!take(&x, 4)) return false; v->i = x; break; }
        case GGUF_U64: { uint64_t x; if (!take(&x, 8)) return false; v->i = (int64_t)x; break; }
        case GGUF_I64: { int64_t x; if (!take(&x, 8)) return false; v->i = x; break; }
        case GGUF_F32: { float x; if (!take(&x, 4)) return false; v->f = x; v->i = (int64_t)x; return true; }
        case GGUF_F64: { double x; if (!take(&x, 8)) return false; v->f = x; v->i = (int64_t)x; return true; }
        case GGUF_STRING: return take_string(&v->s);
        case GGUF_ARRAY: {
            if (in_array) return false;  // nested arrays are not part of the format's use in model files
            uint32_t et = 0;
            uint64_t n = 0;
            if (!take(&et, 4) || !take(&n, 8)) return false;
            v->elem_type = et;
            v->count = n;
            GgufValue skip;
            for (uint64_t k = 0; k < n; k++)
                if (!take_value(et, &skip, true)) return false;
            return true;
        }
        default: return false;
    }
    v->f = (double)v->i;
    return true;
}

int32_t GgufFile::open(const char* path) {
    fd_ = ::open(path, O_RDONLY);
    if (fd_ < 0) return esp::fail(ESP_CUDA_ERR_IO, std::string("cannot open GGUF file ") + path);
    struct stat st;
    if (fstat(fd_, &st) != 0 || st.st_size < 24) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF file is too short");
    size_ = (size_t)st.st_size;
    map_ = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (map_ == MAP_FAILED) return esp::fail(ESP_CUDA_ERR_IO, "mmap of the GGUF file failed");
    uint32_t magic = 0;
    uint64_t n_tensors = 0, n_kv = 0;
    take(&magic, 4);
    take(&version, 4);
    if (magic != 0x46554747u) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "not a GGUF file (bad magic)");
    if (version != 2 && version != 3) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "unsupported GGUF version " + std::to_string(version));
    if (!take(&n_tensors, 8) || !take(&n_kv, 8)) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "truncated GGUF header");
    if (n_tensors > (1u << 20) || n_kv > (1u << 20)) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "implausible GGUF header counts");
    for (uint64_t k = 0; k < n_kv; k++) {
        std::string key;
        uint32_t type = 0;
        GgufValue v;
        if (!take_string(&key) || !take(&type, 4) || !take_value(type, &v, false))
            return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "truncated or malformed GGUF metadata near key '" + key + "'");
        kv[key] = v;
    }
    if (const GgufValue* a = find("general.alignment")) {
        if (a->i <= 0 || a->i > (1ll << 30)) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF alignment out of range");
        alignment = (uint64_t)a->i;
    }
    if (alignment == 0 || (alignment & (alignment - 1))) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF alignment is not a power of two");
    tensors.resize((size_t)n_tensors);
    for (auto& t : tensors) {
        if (!take_string(&t.name) || !take(&t.n_dims, 4) || t.n_dims < 1 || t.n_dims > 4)
            return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "malformed GGUF tensor directory");
        for (uint32_t d = 0; d < t.n_dims; d++)
            if (!take(&t.dims[d], 8)) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "truncated GGUF tensor directory");
        if (!take(&t.type, 4) || !take(&t.offset, 8)) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "truncated GGUF tensor directory");
        uint64_t be = 0, bb = 0;
        if (ggml_block(t.type, &be, &bb)) {
            // an untrusted file: the element count and the byte size are computed with overflow checks
            uint64_t n = 1;
            bool wrapped = false;
            for (int d = 0; d < 4; d++) wrapped = wrapped || __builtin_mul_overflow(n, t.dims[d], &n);
            if (wrapped) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF tensor " + t.name + ": dimensions overflow");
            if (t.dims[0] % be) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF tensor " + t.name + ": row length is not a multiple of the block size");
            if (__builtin_mul_overflow(n / be, bb, &t.nbytes)) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF tensor " + t.name + ": size overflows");
        }  // other GGML types are listed but cannot be uploaded
    }
    data_start_ = (cur_ + alignment - 1) / alignment * alignment;
    if (data_start_ > size_) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF file ends before its tensor data");
    for (auto& t : tensors)
        // written so that neither sum can wrap: offset and size are each compared with what is left of the file
        if (t.nbytes && (t.offset % alignment || t.offset > size_ - data_start_ || t.nbytes > size_ - data_start_ - t.offset))
            return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF tensor " + t.name + " lies outside the file or is misaligned");
    return ESP_CUDA_OK;
}

// "llama" family names the reference accepts (GGUFModelLoader.swift:299-305).
static bool gguf_arch(const std::string& name, int32_t* arch) {
    std::string a = name;
    for (auto& c : a) c = (char)tolower((unsigned char)c);
    if (a == "gpt2") { *arch = ESP_CUDA_ARCH_GPT2; return true; }
    for (const char* k : {"llama", "llama2", "llama3", "mistral", "qwen2", "qwen3"})
        if (a == k) { *arch = ESP_CUDA_ARCH_LLAMA; return true; }
    return false;
}

// llama.cpp's converter stores Wq / Wk of these architectures with each head's rows interleaved (row 2i+h of a head
// holds rotation half h, pair i) for its pairwise RoPE; the decode path here rotates half-split (row h*hd/2+i), so the
// rows are put back.  Qwen files keep the half-split order.
static bool gguf_rows_interleaved(const std::string& arch_name) {
    std::string a = arch_name;
    for (auto& c : a) c = (char)tolower((unsigned char)c);
    return a == "llama" || a == "llama2" || a == "llama3" || a == "mistral";
}

// Metadata integers are 64-bit in the file and 32-bit in the config: a value that does not fit is an invalid file,
// not something to truncate silently.
static bool fits_i32(long long v) { return v >= -2147483647LL - 1 && v <= 2147483647LL; }

static int32_t gguf_config(const GgufFile& f, esp_cuda_config* c, std::string* arch_name, int32_t* tied) {
    const GgufValue* an = f.find("general.architecture");
    if (!an || an->type != GGUF_STRING) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF metadata lacks general.architecture");
    *arch_name = an->s;
    int32_t arch = 0;
    if (!gguf_arch(an->s, &arch)) return esp::fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "unsupported GGUF architecture: " + an->s);
    const std::string p = an->s + ".";
    auto need = [&](const char* key, int32_t* dst) -> int32_t {
        const GgufValue* v = f.find(p + key);
        if (!v) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF metadata lacks " + p + key);
        if (!fits_i32((long long)v->i)) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF metadata value out of range: " + p + key);
        *dst = (int32_t)v->i;
        return ESP_CUDA_OK;
    };
    auto opt = [&](const GgufValue* v, int32_t fallback, int32_t* dst) -> int32_t {
        if (!v) { *dst = fallback; return ESP_CUDA_OK; }
        if (!fits_i32((long long)v->i)) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF metadata value out of range");
        *dst = (int32_t)v->i;
        return ESP_CUDA_OK;
    };
    *c = esp_cuda_config{};
    c->architecture = arch;
    int32_t rc;
    if ((rc = need("block_count", &c->n_layer))) return rc;
    if ((rc = need("attention.head_count", &c->n_head))) return rc;
    if ((rc = need("embedding_length", &c->d_model))) return rc;
    if ((rc = need("context_length", &c->max_seq))) return rc;
    const GgufValue* v;
    if ((rc = opt(f.find(p + "attention.head_count_kv"), c->n_head, &c->n_kv_head))) return rc;
    if (c->n_head <= 0) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF head count must be positive");
    if ((rc = opt(f.find(p + "attention.key_length"), c->d_model / c->n_head, &c->head_dim))) return rc;
    if ((v = f.find(p + "feed_forward_length"))) { if ((rc = opt(v, 0, &c->hidden_dim))) return rc; }
    else if (arch == ESP_CUDA_ARCH_GPT2) c->hidden_dim = 4 * c->d_model;
    else return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF metadata lacks " + p + "feed_forward_length");
    if ((v = f.find("tokenizer.ggml.tokens")) && v->type == GGUF_ARRAY) {
        if (v->count > 2147483647ull) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF vocabulary size out of range");
        c->vocab = (int32_t)v->count;
    } else if ((v = f.find(p + "vocab_size"))) { if ((rc = opt(v, 0, &c->vocab))) return rc; }
    else if (const GgufTensor* te = f.tensor("token_embd.weight")) {
        if (te->dims[1] > 2147483647ull) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF vocabulary size out of range");
        c->vocab = (int32_t)te->dims[1];
    }
    const char* eps_key = arch == ESP_CUDA_ARCH_GPT2 ? "attention.layer_norm_epsilon" : "attention.layer_norm_rms_epsilon";
    c->norm_eps = (v = f.find(p + eps_key)) ? (float)v->f : 1e-5f;
    c->rope_theta = (v = f.find(p + "rope.freq_base")) ? (float)v->f : 10000.0f;  // GGUFModelLoader.swift:307-308
    if ((rc = opt(f.find("tokenizer.ggml.eos_token_id"), -1, &c->eos_token))) return rc;
    c->max_batch = 1;
    c->tp_size = 1;
    *tied = f.tensor("output.weight") ? 0 : 1;
    return ESP_CUDA_OK;
}

// GGUF tensor name -> weight-directory path of the reference (Sources/ModelSupport/LayerWeightPaths.swift:22-77).
// Returns false for tensors the decode path has no slot for.  "attn_qkv" (GPT-2's fused projection) is reported as
// "layers/N/wqkv" / "layers/N/bqkv" and split by the caller.
static bool gguf_slot(int32_t arch, const std::string& name, std::string* slot) {
    const bool gpt2 = arch == ESP_CUDA_ARCH_GPT2;
    static const struct { const char* g; const char* llama; const char* gpt2; } top[] = {
        {"token_embd.weight", "embeddings/token", "embeddings/token"},
        {"position_embd.weight", nullptr, "embeddings/position"},
        {"output_norm.weight", "rms_final", "final_norm_gamma"},
        {"output_norm.bias", nullptr, "final_norm_beta"},
        {"output.weight", "lm_head", "lm_head"},
    };
    for (auto& e : top)
        if (name == e.g) {
            const char* s = gpt2 ? e.gpt2 : e.llama;
            if (!s) return false;
            *slot = s;
            return true;
        }
    if (name.compare(0, 4, "blk.") != 0) return false;
    const size_t dot = name.find('.', 4);
    if (dot == std::string::npos) return false;
    const std::string layer = name.substr(4, dot - 4), leaf = name.substr(dot + 1);
    for (char ch : layer)
        if (!isdigit((unsigned char)ch)) return false;
    static const struct { const char* g; const char* llama; const char* gpt2; } per_layer[] = {
        {"attn_norm.weight", "rms_att", "ln_1_gamma"}, {"attn_norm.bias", nullptr, "ln_1_beta"},
        {"attn_q.weight", "wq", "wq"}, {"attn_k.weight", "wk", "wk"}, {"attn_v.weight", "wv", "wv"},
        {"attn_q.bias", nullptr, "bq"}, {"attn_k.bias", nullptr, "bk"}, {"attn_v.bias", nullptr, "bv"},
        {"attn_qkv.weight", nullptr, "wqkv"}, {"attn_qkv.bias", nullptr, "bqkv"},
        {"attn_output.weight", "wo", "wo"}, {"attn_output.bias", nullptr, "bo"},
        {"attn_q_norm.weight", "q_norm", nullptr}, {"attn_k_norm.weight", "k_norm", nullptr},  // Qwen3 per-head q/k norm
        {"ffn_norm.weight", "rms_ffn", "ln_2_gamma"}, {"ffn_norm.bias", nullptr, "ln_2_beta"},
        {"ffn_gate.weight", "w1", nullptr}, {"ffn_up.weight", "w3", "w1"}, {"ffn_up.bias", nullptr, "b1"},
        {"ffn_down.weight", "w2", "w2"}, {"ffn_down.bias", nullptr, "b2"},
    };
    for (auto& e : per_layer)
        if (leaf == e.g) {
            const char* s = gpt2 ? e.gpt2 : e.llama;
            if (!s) return false;
            *slot = "layers/" + layer + "/" + s;
            return true;
        }
    return false;
}

// Undo the per-head row interleave of a [n_head * head_dim, cols] matrix stored in blocks of `row_bytes` per row.
static void deinterleave_rows(const uint8_t* src, uint8_t* dst, int n_head, int head_dim, size_t row_bytes) {
    const int half = head_dim / 2;
    for (int h = 0; h < n_head; h++)
        for (int i = 0; i < half; i++)
            for (int part = 0; part < 2; part++) {
                const size_t from = (size_t)h * head_dim + 2 * i + part, to = (size_t)h * head_dim + part * half + i;
                memcpy(dst + to * row_bytes, src + from * row_bytes, row_bytes);
            }
}

static float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// Any uploadable GGML type -> fp32 on the host (embedding tables and vectors that arrive quantised).
static void gguf_to_float(const uint8_t* src, uint32_t type, uint64_t n, float* dst) {
    if (type == ESP_CUDA_F32) { memcpy(dst, src, n * 4); return; }
    if (type == ESP_CUDA_F16) { for (uint64_t k = 0; k < n; k++) { uint16_t h; memcpy(&h, src + 2 * k, 2); dst[k] = half_bits_to_float(h); } return; }
    if (type == ESP_CUDA_BF16) { for (uint64_t k = 0; k < n; k++) { uint16_t h; memcpy(&h, src + 2 * k, 2); uint32_t u = (uint32_t)h << 16; memcpy(dst + k, &u, 4); } return; }
    for (uint64_t b = 0; b < n / 32; b++) {
        const uint8_t* s = src + b * (type == ESP_CUDA_Q8_0 ? 34 : 18);
        uint16_t hd; memcpy(&hd, s, 2);
        const float d = half_bits_to_float(hd);
        if (type == ESP_CUDA_Q8_0) {
            for (int k = 0; k < 32; k++) dst[b * 32 + k] = d * (float)(int8_t)s[2 + k];
        } else {
            for (int k = 0; k < 16; k++) {
                dst[b * 32 + k] = d * (float)((int)(s[2 + k] & 15) - 8);
                dst[b * 32 + 16 + k] = d * (float)((int)(s[2 + k] >> 4) - 8);
            }
        }
    }
}

int32_t gguf_load_into(Engine& eng, const GgufFile& f, const esp_cuda_config& c, const std::string& arch_name) {
    const bool interleaved = c.architecture == ESP_CUDA_ARCH_LLAMA && gguf_rows_interleaved(arch_name);
    std::vector<uint8_t> scratch;
    std::vector<float> floats;
    int loaded = 0;
    int32_t rc;
    for (const GgufTensor& t : f.tensors) {
        std::string slot;
        if (!gguf_slot(c.architecture, t.name, &slot)) {
            continue;  // rope tables and other tensors the decode path does not read
        }
        if (!t.nbytes) return esp::fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "GGUF tensor " + t.name + " has GGML type " + std::to_string(t.type) + "; supported: F32, F16, BF16, Q8_0, Q4_0");
        const uint8_t* data = f.data_of(t);
        const uint64_t n = t.dims[0] * t.dims[1] * t.dims[2] * t.dims[3];
        const std::string leaf = slot.substr(slot.rfind('/') + 1);
        const bool quant = t.type == ESP_CUDA_Q8_0 || t.type == ESP_CUDA_Q4_0;
        if (leaf == "wqkv" || leaf == "bqkv") {
            // GPT-2's fused projection: rows [0,d) q, [d,2d) k, [2d,3d) v
            const std::string base = slot.substr(0, slot.rfind('/') + 1);
            const char* names[3] = {leaf == "wqkv" ? "wq" : "bq", leaf == "wqkv" ? "wk" : "bk", leaf == "wqkv" ? "wv" : "bv"};
            if (t.nbytes % 3) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "fused qkv tensor " + t.name + " does not split in three");
            for (int k = 0; k < 3; k++)
                if ((rc = eng.load_tensor((base + names[k]).c_str(), (int32_t)t.type, data + (size_t)k * (t.nbytes / 3), t.nbytes / 3))) return rc;
            loaded += 3;
            continue;
        }
        if (slot == "embeddings/token" || slot == "embeddings/position" || (quant && t.n_dims == 1)) {
            if (quant) {  // the embedding lookup reads single elements: keep the table in 16-bit form
                floats.resize(n);
                gguf_to_float(data, t.type, n, floats.data());
                if ((rc = eng.load_tensor(slot.c_str(), ESP_CUDA_F32, floats.data(), n * 4))) return rc;
            } else if ((rc = eng.load_tensor(slot.c_str(), (int32_t)t.type, data, t.nbytes))) return rc;
            loaded++;
            continue;
        }
        if (interleaved && (leaf == "wq" || leaf == "wk")) {
            const int heads = leaf == "wq" ? c.n_head : c.n_kv_head;
            if (t.dims[1] != (uint64_t)heads * c.head_dim) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF tensor " + t.name + " has an unexpected row count");
            scratch.resize(t.nbytes);
            deinterleave_rows(data, scratch.data(), heads, c.head_dim, t.nbytes / t.dims[1]);
            data = scratch.data();
        }
        if ((rc = eng.load_tensor(slot.c_str(), (int32_t)t.type, data, t.nbytes))) return rc;
        loaded++;
    }
    if (!f.tensor("output.weight")) {  // tied head: the embedding matrix is the classifier (GGUFModelLoader.swift:224-263)
        const GgufTensor* te = f.tensor("token_embd.weight");
        if (!te || !te->nbytes) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "GGUF file has neither output.weight nor a usable token_embd.weight");
        if ((rc = eng.load_tensor("lm_head", (int32_t)te->type, f.data_of(*te), te->nbytes))) return rc;
        loaded++;
    }
    if (loaded == 0) return esp::fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "no tensors converted");  // noTensorsConverted
    return ESP_CUDA_OK;
}

}  // namespace esp

extern "C" {

int32_t esp_cuda_gguf_inspect(const char* path, esp_cuda_config* config, char* architecture_name, int32_t name_capacity,
                              int32_t* n_tensors, int32_t* tied_lm_head) {
    if (!path || !config) return esp::fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "esp_cuda_gguf_inspect: null argument");
    esp::GgufFile f;
    int32_t rc = f.open(path);
    if (rc) return rc;
    std::string arch;
    int32_t tied = 0;
    if ((rc = esp::gguf_config(f, config, &arch, &tied))) return rc;
    if (architecture_name && name_capacity > 0) snprintf(architecture_name, (size_t)name_capacity, "%s", arch.c_str());
    if (n_tensors) *n_tensors = (int32_t)f.tensors.size();
    if (tied_lm_head) *tied_lm_head = tied;
    return ESP_CUDA_OK;
}

int32_t esp_cuda_gguf_tensor_info(const char* path, int32_t index, char* name, int32_t name_capacity, char* slot, int32_t slot_capacity,
                                  int32_t* ggml_type, int64_t* dims4, uint64_t* data_offset, uint64_t* nbytes) {
    if (!path) return esp::fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "esp_cuda_gguf_tensor_info: null argument");
    esp::GgufFile f;
    int32_t rc = f.open(path);
    if (rc) return rc;
    if (index < 0 || index >= (int32_t)f.tensors.size()) return esp::fail(ESP_CUDA_ERR_OUT_OF_RANGE, "GGUF tensor index out of range");
    esp_cuda_config c;
    std::string arch;
    int32_t tied = 0;
    if ((rc = esp::gguf_config(f, &c, &arch, &tied))) return rc;
    const esp::GgufTensor& t = f.tensors[(size_t)index];
    std::string s;
    if (!esp::gguf_slot(c.architecture, t.name, &s)) s.clear();
    if (name && name_capacity > 0) snprintf(name, (size_t)name_capacity, "%s", t.name.c_str());
    if (slot && slot_capacity > 0) snprintf(slot, (size_t)slot_capacity, "%s", s.c_str());
    if (ggml_type) *ggml_type = (int32_t)t.type;
    if (dims4) for (int d = 0; d < 4; d++) dims4[d] = (int64_t)t.dims[d];
    if (data_offset) *data_offset = t.offset;
    if (nbytes) *nbytes = t.nbytes;
    return ESP_CUDA_OK;
}

int32_t esp_cuda_create_from_gguf(const char* path, int32_t max_batch, int32_t device, uint32_t flags, esp_cuda_engine** out) {
    if (!path || !out) return esp::fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "esp_cuda_create_from_gguf: null argument");
    *out = nullptr;
    esp::GgufFile f;
    int32_t rc = f.open(path);
    if (rc) return rc;
    esp_cuda_config c;
    std::string arch;
    int32_t tied = 0;
    if ((rc = esp::gguf_config(f, &c, &arch, &tied))) return rc;
    c.max_batch = max_batch; c.device = device; c.flags = (int32_t)flags;
    esp_cuda_engine* e = nullptr;
    if ((rc = esp_cuda_create(&c, nullptr, &e))) return rc;
    rc = esp::gguf_load_into(e->impl, f, c, arch);
    if (rc == ESP_CUDA_OK) rc = e->impl.finalize();
    if (rc != ESP_CUDA_OK) { esp_cuda_destroy(e); return rc; }
    *out = e;
    return ESP_CUDA_OK;
}

}  // extern "C"
