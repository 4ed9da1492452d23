/*
 * espresso_oracle.c -- TEST INFRASTRUCTURE, not part of the shipped library.
 *
 * A plain-C, fp32, CPU restatement of the transformer decode path of
 * christopherkarani/Espresso.  It exists only so that the CUDA library can be
 * checked against the reference's arithmetic; nothing in the product path may
 * link, import or execute this file.  Every function cites the reference
 * source (path inside the Espresso project : line) it follows.
 *
 * Parity pin status: the reference is Swift + Accelerate and cannot be built
 * on Linux, so this restatement is pinned against (a) the known-answer tests
 * of the reference's own test suite (RoPE, RMSNorm, decode attention, SiLU,
 * argmax tie rule, BLOBFILE header), restated in tests/test_oracle_kat.py, and
 * (b) logits of HuggingFace LlamaForCausalLM fed through the reference's own
 * Python weight bridge scripts/espresso_llama_weights.py (fixtures under
 * tests/golden/).  GGUF Q8_0/Q4_0 arithmetic lives in the reference's
 * un-vendored "Edgerunner" dependency (Package.swift:23-25, no version pin);
 * it is restated from the public GGUF block layout and pinned against the
 * `gguf` Python package's quantize/dequantize (fixtures under tests/golden/).
 *
 * Precision model (Sources/RealModelInference/RealModelInferenceEngine.swift:289-301):
 * fp32 weights (the fp16 file values widened), fp32 activations, fp32 KV cache,
 * no intermediate rounding by default; round_fp16 != 0 turns on the optional
 * fp16 rounding of q, k, v, RoPE outputs and residuals.
 *
 * Summation order: the reference calls vDSP (order unspecified).  Here every
 * dot product uses 16 interleaved partial sums folded at the end; that order is
 * deterministic and vectorisable without -ffast-math.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>

#if defined(_OPENMP)
#include <omp.h>
#endif

#define ESP_ORACLE_API __attribute__((visibility("default")))

enum { ESP_ARCH_LLAMA = 0, ESP_ARCH_GPT2 = 1 };

typedef struct {
    int32_t architecture;
    int32_t n_layer, n_head, n_kv_head, d_model, head_dim, hidden_dim, vocab, max_seq;
    float norm_eps, rope_theta;
    int32_t eos_token; /* -1 = none */
} esp_oracle_config;

/* ------------------------------------------------------------------ fp16 */

/* IEEE binary16 -> binary32, exact (BlobWeightLoader.swift:52 widens each payload element). */
ESP_ORACLE_API float esp_oracle_half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* binary32 -> binary16, round to nearest even (Swift Float16(x), WeightBlob.swift:36). */
ESP_ORACLE_API uint16_t esp_oracle_float_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t mant = x & 0x007FFFFFu;
    int32_t exp = (int32_t)((x >> 23) & 0xFFu);
    if (exp == 255) return (uint16_t)(sign | 0x7C00u | (mant ? 0x200u : 0));
    exp = exp - 127 + 15;
    if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        mant |= 0x00800000u;
        uint32_t shift = (uint32_t)(14 - exp);
        uint32_t half = mant >> shift;
        uint32_t rem = mant & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half & 1u))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)exp << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;
    return (uint16_t)(sign | half);
}

static inline float round_half(float v) { return esp_oracle_half_to_float(esp_oracle_float_to_half(v)); }

/* bf16 -> fp32 (config 5 keeps bf16 weights; the oracle widens them exactly). */
ESP_ORACLE_API float esp_oracle_bf16_to_float(uint16_t b) {
    uint32_t bits = (uint32_t)b << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* ------------------------------------------------------------ primitive ops */

static float dot16(const float* a, const float* b, int n) {
    float acc[16] = {0};
    int i = 0;
    for (; i + 16 <= n; i += 16)
        for (int j = 0; j < 16; j++) acc[j] += a[i + j] * b[i + j];
    float tail = 0.f;
    for (; i < n; i++) tail += a[i] * b[i];
    float s = 0.f;
    for (int j = 0; j < 16; j++) s += acc[j];
    return s + tail;
}

/* y = W[rows x cols] . x  -- multiplyRowMajorMatrix, RealModelInferenceEngine.swift:6674-6718 (vDSP_mmul). */
ESP_ORACLE_API void esp_oracle_gemv(const float* w, int rows, int cols, const float* x, float* y) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) y[r] = dot16(w + (size_t)r * cols, x, cols);
}

/* rmsNorm, RealModelInferenceEngine.swift:6724-6743: y = x * (1/sqrt(sum(x^2)/n + eps)) * w. */
ESP_ORACLE_API void esp_oracle_rmsnorm(const float* x, const float* w, int n, float eps, float* y) {
    float ss = dot16(x, x, n);
    float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = 0; i < n; i++) y[i] = (x[i] * inv) * w[i];
}

/* LayerNorm (GPT-2), graph layerNorm128 RealModelInferenceEngine.swift:8655-8685 and the CPU statement
 * normalizeHiddenForCoreMLReference (Sources/EspressoGenerate/GPT2DemoSupport.swift:150-187):
 * y = (x-mean) * (var_biased + eps)^-0.5 * gamma + beta. */
ESP_ORACLE_API void esp_oracle_layernorm(const float* x, const float* g, const float* b, int n, float eps, float* y) {
    float mean = 0.f;
    for (int i = 0; i < n; i++) mean += x[i];
    mean /= (float)n;
    float var = 0.f;
    for (int i = 0; i < n; i++) { float c = x[i] - mean; var += c * c; }
    var /= (float)n;
    float inv = 1.0f / sqrtf(var + eps);
    for (int i = 0; i < n; i++) y[i] = (x[i] - mean) * inv * g[i] + b[i];
}

/* applyPerHeadRMSNormInPlace, RealModelInferenceEngine.swift:6648-6672 (Qwen3 q/k norm). */
ESP_ORACLE_API void esp_oracle_per_head_rmsnorm(float* v, const float* w, int heads, int head_dim, float eps) {
    for (int h = 0; h < heads; h++) {
        float* p = v + (size_t)h * head_dim;
        float ss = 0.f;
        for (int i = 0; i < head_dim; i++) ss += p[i] * p[i];
        float inv = 1.0f / sqrtf(ss / (float)head_dim + eps);
        for (int i = 0; i < head_dim; i++) p[i] *= inv * w[i];
    }
}

/* applyHalfSplitRoPEPerHead, RealModelInferenceEngine.swift:6745-6772 (pairs (i, i+hd/2));
 * same rule as CPUOps RoPE.applyDecodeStep (Sources/CPUOps/RoPE.swift:56-110). */
ESP_ORACLE_API void esp_oracle_rope_half_split(float* v, int heads, int head_dim, int position, float theta) {
    int half = head_dim / 2;
    for (int h = 0; h < heads; h++) {
        float* p = v + (size_t)h * head_dim;
        for (int i = 0; i < half; i++) {
            float freq = 1.0f / powf(theta, (float)(2 * i) / (float)head_dim);
            float ang = (float)position * freq;
            float c = cosf(ang), s = sinf(ang);
            float v0 = p[i], v1 = p[i + half];
            p[i] = v0 * c - v1 * s;
            p[i + half] = v0 * s + v1 * c;
        }
    }
}

/* decodeContextFromCaches, RealModelInferenceEngine.swift:6774-6823; CPU twin
 * ForwardPass.cpuDecodeContext (Sources/Espresso/DecodeForwardPass.swift:683-756).
 * Caches are channel-major [kvDim, cache_stride]; kvHead = head / (heads/kvHeads) (grouped contiguous). */
ESP_ORACLE_API void esp_oracle_decode_context(const float* q, const float* k_cache, const float* v_cache, int heads,
                                              int kv_heads, int head_dim, int visible, int token_base,
                                              int cache_stride, float* ctx) {
    int qpk = heads / (kv_heads > 0 ? kv_heads : 1);
    if (qpk < 1) qpk = 1;
    float scale = 1.0f / sqrtf((float)head_dim);
#pragma omp parallel for schedule(static)
    for (int h = 0; h < heads; h++) {
        int kvh = h / qpk;
        if (kvh > kv_heads - 1) kvh = kv_heads - 1;
        const float* qh = q + (size_t)h * head_dim;
        float* scores = (float*)malloc(sizeof(float) * (size_t)visible);
        float mx = -INFINITY;
        for (int t = 0; t < visible; t++) {
            float dot = 0.f;
            for (int d = 0; d < head_dim; d++)
                dot += qh[d] * k_cache[((size_t)kvh * head_dim + d) * cache_stride + token_base + t];
            scores[t] = dot * scale;
            if (scores[t] > mx) mx = scores[t];
        }
        float denom = 0.f;
        for (int t = 0; t < visible; t++) { scores[t] = expf(scores[t] - mx); denom += scores[t]; }
        float inv = denom > 0.f ? 1.0f / denom : 0.f;
        for (int d = 0; d < head_dim; d++) {
            float acc = 0.f;
            const float* vrow = v_cache + ((size_t)kvh * head_dim + d) * cache_stride + token_base;
            for (int t = 0; t < visible; t++) acc += scores[t] * inv * vrow[t];
            ctx[(size_t)h * head_dim + d] = acc;
        }
        free(scores);
    }
}

/* silu, RealModelInferenceEngine.swift:6825-6827 (tanh form, equal to x/(1+e^-x), Sources/CPUOps/SiLU.swift:6-8). */
ESP_ORACLE_API float esp_oracle_silu(float x) { return 0.5f * x * (1.0f + tanhf(0.5f * x)); }

/* gelu128 tanh approximation, RealModelInferenceEngine.swift:8712-8729. */
ESP_ORACLE_API float esp_oracle_gelu(float x) {
    float inner = (x + 0.044715f * (x * x * x)) * 0.7978846f;
    return (0.5f * x) * (1.0f + tanhf(inner));
}

/* First index of the maximum (tie rule of neon_convert.c:61-83 and vDSP_maxvi). */
ESP_ORACLE_API int esp_oracle_argmax_first(const float* v, int n) {
    int best = 0;
    float bv = -INFINITY;
    for (int i = 0; i < n; i++)
        if (v[i] > bv) { bv = v[i]; best = i; }
    return best;
}

/* partitionedArgmax with Cauchy-Schwarz block pruning, RealModelInferenceEngine.swift:8182-8275
 * (block size 4000, :119).  Restated including the pruning so that it can be shown equal to the
 * naive argmax; block_size <= 0 disables blocking. */
ESP_ORACLE_API int esp_oracle_partitioned_argmax(const float* classifier, const float* input, int vocab, int dim,
                                                 int block_size) {
    if (block_size <= 0) block_size = vocab;
    int nblocks = (vocab + block_size - 1) / block_size;
    float* norms = (float*)malloc(sizeof(float) * (size_t)nblocks);
    for (int b = 0; b < nblocks; b++) {
        int s = b * block_size, e = s + block_size < vocab ? s + block_size : vocab;
        float bm = 0.f;
        for (int r = s; r < e; r++) {
            float n2 = dot16(classifier + (size_t)r * dim, classifier + (size_t)r * dim, dim);
            float nr = sqrtf(n2);
            if (nr > bm) bm = nr;
        }
        norms[b] = bm;
    }
    float in_norm = sqrtf(dot16(input, input, dim));
    float* scratch = (float*)malloc(sizeof(float) * (size_t)block_size);
    int best = 0;
    float bv = -INFINITY;
    for (int b = 0; b < nblocks; b++) {
        int s = b * block_size, e = s + block_size < vocab ? s + block_size : vocab;
        if (b > 0 && bv > -INFINITY && norms[b] * in_norm < bv) continue;
        esp_oracle_gemv(classifier + (size_t)s * dim, e - s, dim, input, scratch);
        int li = esp_oracle_argmax_first(scratch, e - s);
        if (scratch[li] > bv) { bv = scratch[li]; best = s + li; }
    }
    free(scratch);
    free(norms);
    return best;
}

/* ------------------------------------------------------------ GGUF Q8_0 / Q4_0 */
/* Public GGUF block layouts (the reference delegates these to its external Edgerunner package,
 * Sources/EspressoGGUF/GGUFModelLoader.swift:341-369):
 *   Q8_0: 34 bytes = fp16 d, 32 x int8 q;                value = d*q
 *   Q4_0: 18 bytes = fp16 d, 16 bytes; byte j low nibble = element j, high nibble = element j+16;
 *                                                         value = d*(nibble-8)
 * Quantisation follows the published reference quantisers: Q8_0 d = amax/127, q = round(x/d);
 * Q4_0 d = max_signed/-8 where max_signed is the element of largest magnitude, q = min(15, (int)(x/d + 8.5)). */

ESP_ORACLE_API void esp_oracle_quantize_q8_0(const float* x, int64_t n, uint8_t* out) {
    int64_t nb = n / 32;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; b++) {
        const float* p = x + b * 32;
        float amax = 0.f;
        for (int i = 0; i < 32; i++) { float a = fabsf(p[i]); if (a > amax) amax = a; }
        float d = amax / 127.0f;
        float id = d != 0.f ? 1.0f / d : 0.f;
        uint16_t dh = esp_oracle_float_to_half(d);
        uint8_t* o = out + b * 34;
        memcpy(o, &dh, 2);
        for (int i = 0; i < 32; i++) o[2 + i] = (uint8_t)(int8_t)roundf(p[i] * id);
    }
}

ESP_ORACLE_API void esp_oracle_dequantize_q8_0(const uint8_t* in, int64_t n, float* out) {
    int64_t nb = n / 32;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; b++) {
        const uint8_t* p = in + b * 34;
        uint16_t dh;
        memcpy(&dh, p, 2);
        float d = esp_oracle_half_to_float(dh);
        for (int i = 0; i < 32; i++) out[b * 32 + i] = d * (float)(int8_t)p[2 + i];
    }
}

ESP_ORACLE_API void esp_oracle_quantize_q4_0(const float* x, int64_t n, uint8_t* out) {
    int64_t nb = n / 32;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; b++) {
        const float* p = x + b * 32;
        float amax = 0.f, mx = 0.f;
        for (int i = 0; i < 32; i++) {
            float a = fabsf(p[i]);
            if (a > amax) { amax = a; mx = p[i]; }
        }
        float d = mx / -8.0f;
        float id = d != 0.f ? 1.0f / d : 0.f;
        uint16_t dh = esp_oracle_float_to_half(d);
        uint8_t* o = out + b * 18;
        memcpy(o, &dh, 2);
        for (int j = 0; j < 16; j++) {
            float x0 = p[j] * id, x1 = p[16 + j] * id;
            int q0 = (int)(int8_t)(x0 + 8.5f), q1 = (int)(int8_t)(x1 + 8.5f);
            if (q0 > 15) q0 = 15;
            if (q1 > 15) q1 = 15;
            o[2 + j] = (uint8_t)(q0 | (q1 << 4));
        }
    }
}

ESP_ORACLE_API void esp_oracle_dequantize_q4_0(const uint8_t* in, int64_t n, float* out) {
    int64_t nb = n / 32;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; b++) {
        const uint8_t* p = in + b * 18;
        uint16_t dh;
        memcpy(&dh, p, 2);
        float d = esp_oracle_half_to_float(dh);
        for (int j = 0; j < 16; j++) {
            out[b * 32 + j] = d * (float)((int)(p[2 + j] & 0x0F) - 8);
            out[b * 32 + 16 + j] = d * (float)((int)(p[2 + j] >> 4) - 8);
        }
    }
}

/* ------------------------------------------------------------ BLOBFILE */
/* WeightBlob.writeHeader (Sources/ANETypes/WeightBlob.swift:6-18) and BlobWeightLoader.load
 * (Sources/ModelSupport/BlobWeightLoader.swift:25-92): 128-byte header, byte0=1, byte4=2,
 * bytes 64..67 = EF BE AD DE, byte 68 = 1, u32 LE payload bytes @72, u32 LE data offset (=128) @80,
 * then little-endian fp16 payload. Error codes mirror BlobWeightLoaderError. */
enum {
    ESP_BLOB_OK = 0,
    ESP_BLOB_IO = -1,
    ESP_BLOB_TRUNCATED_HEADER = -2,
    ESP_BLOB_INVALID_MAGIC = -3,
    ESP_BLOB_INVALID_OFFSET = -4,
    ESP_BLOB_TRUNCATED_PAYLOAD = -5,
    ESP_BLOB_INVALID_PAYLOAD_SIZE = -6,
    ESP_BLOB_COUNT_MISMATCH = -7
};

ESP_ORACLE_API int esp_oracle_blob_write(const char* path, const uint16_t* fp16, uint32_t count) {
    uint8_t header[128];
    memset(header, 0, sizeof header);
    header[0] = 1;
    header[4] = 2;
    header[64] = 0xEF; header[65] = 0xBE; header[66] = 0xAD; header[67] = 0xDE;
    header[68] = 1;
    uint32_t bytes = count * 2u, off = 128u;
    memcpy(header + 72, &bytes, 4);
    memcpy(header + 80, &off, 4);
    FILE* f = fopen(path, "wb");
    if (!f) return ESP_BLOB_IO;
    int ok = fwrite(header, 1, 128, f) == 128 && (count == 0 || fwrite(fp16, 2, count, f) == count);
    fclose(f);
    return ok ? ESP_BLOB_OK : ESP_BLOB_IO;
}

/* Returns the element count (>= 0) or a negative error. out may be NULL to query the count. */
ESP_ORACLE_API int64_t esp_oracle_blob_read(const char* path, float* out, int64_t capacity) {
    FILE* f = fopen(path, "rb");
    if (!f) return ESP_BLOB_IO;
    uint8_t header[128];
    size_t got = fread(header, 1, 128, f);
    if (got < 128) { fclose(f); return ESP_BLOB_TRUNCATED_HEADER; }
    uint32_t magic, size, off;
    memcpy(&magic, header + 64, 4);
    memcpy(&size, header + 72, 4);
    memcpy(&off, header + 80, 4);
    if (magic != 0xDEADBEEFu) { fclose(f); return ESP_BLOB_INVALID_MAGIC; }
    if (off != 128u) { fclose(f); return ESP_BLOB_INVALID_OFFSET; }
    if (size % 2u) { fclose(f); return ESP_BLOB_INVALID_PAYLOAD_SIZE; }
    int64_t count = size / 2u;
    if (!out) { fclose(f); return count; }
    if (capacity < count) { fclose(f); return ESP_BLOB_COUNT_MISMATCH; }
    uint16_t* tmp = (uint16_t*)malloc(size ? size : 2);
    size_t n = fread(tmp, 1, size, f);
    fclose(f);
    if (n != size) { free(tmp); return ESP_BLOB_TRUNCATED_PAYLOAD; }
    for (int64_t i = 0; i < count; i++) out[i] = esp_oracle_half_to_float(tmp[i]);
    free(tmp);
    return count;
}

/* ------------------------------------------------------------ model */

typedef struct {
    float *rms_att, *ln1_beta, *wq, *wk, *wv, *wo, *bq, *bk, *bv, *bo;
    float *rms_ffn, *ln2_beta, *w1, *w2, *w3, *b1, *b2, *q_norm, *k_norm;
} layer_weights;

typedef struct esp_oracle_model {
    esp_oracle_config cfg;
    float *tok_emb, *pos_emb, *final_gamma, *final_beta, *lm_head;
    int lm_head_tied;
    layer_weights* layers;
} esp_oracle_model;

static int q_dim(const esp_oracle_config* c) { return c->n_head * c->head_dim; }
static int kv_dim(const esp_oracle_config* c) { return c->n_kv_head * c->head_dim; }

/* validateConfig, RealModelInferenceEngine.swift:7615-7634. */
ESP_ORACLE_API int esp_oracle_validate_config(const esp_oracle_config* c) {
    if (c->n_layer <= 0 || c->n_head <= 0 || c->n_kv_head <= 0 || c->d_model <= 0 || c->head_dim <= 0 ||
        c->hidden_dim <= 0 || c->vocab <= 0 || c->max_seq <= 0)
        return -1;
    if (c->n_head % c->n_kv_head != 0) return -1;
    if (c->architecture != ESP_ARCH_LLAMA && c->architecture != ESP_ARCH_GPT2) return -1;
    if (c->architecture == ESP_ARCH_LLAMA && (c->head_dim % 2)) return -1;
    return 0;
}

ESP_ORACLE_API esp_oracle_model* esp_oracle_model_create(const esp_oracle_config* cfg) {
    if (esp_oracle_validate_config(cfg) != 0) return NULL;
    esp_oracle_model* m = (esp_oracle_model*)calloc(1, sizeof *m);
    m->cfg = *cfg;
    m->layers = (layer_weights*)calloc((size_t)cfg->n_layer, sizeof(layer_weights));
    return m;
}

ESP_ORACLE_API void esp_oracle_model_destroy(esp_oracle_model* m) {
    if (!m) return;
    free(m->tok_emb); free(m->pos_emb); free(m->final_gamma); free(m->final_beta);
    if (!m->lm_head_tied) free(m->lm_head);
    for (int l = 0; l < m->cfg.n_layer; l++) {
        float** p = (float**)&m->layers[l];
        for (size_t i = 0; i < sizeof(layer_weights) / sizeof(float*); i++) free(p[i]);
    }
    free(m->layers);
    free(m);
}

/* Tensor names are the weight-directory relative paths without ".bin"
 * (LayerWeightPaths.forLayer, Sources/ModelSupport/LayerWeightPaths.swift:22-77; top-level names
 * RealModelInferenceEngine.swift:2066-2154). Returns the slot and expected element count. */
static float** model_slot(esp_oracle_model* m, const char* name, int64_t* expect) {
    const esp_oracle_config* c = &m->cfg;
    int64_t d = c->d_model, q = q_dim(c), kv = kv_dim(c), h = c->hidden_dim, V = c->vocab;
    if (!strcmp(name, "embeddings/token") || !strcmp(name, "embeddings/token_embeddings")) { *expect = V * d; return &m->tok_emb; }
    if (!strcmp(name, "embeddings/position") || !strcmp(name, "embeddings/position_embeddings")) { *expect = (int64_t)c->max_seq * d; return &m->pos_emb; }
    if (!strcmp(name, "rms_final") || !strcmp(name, "final_norm_gamma") || !strcmp(name, "final_norm") || !strcmp(name, "ln_f_gamma")) { *expect = d; return &m->final_gamma; }
    if (!strcmp(name, "final_norm_beta") || !strcmp(name, "ln_f_beta") || !strcmp(name, "rms_final_beta")) { *expect = d; return &m->final_beta; }
    if (!strcmp(name, "lm_head") || !strcmp(name, "classifier")) { *expect = V * d; return &m->lm_head; }
    int l = -1;
    char leaf[64];
    if (sscanf(name, "layers/%d/%63s", &l, leaf) == 2 && l >= 0 && l < c->n_layer) {
        layer_weights* L = &m->layers[l];
        struct { const char* n; float** p; int64_t cnt; } tab[] = {
            {"rms_att", &L->rms_att, d}, {"ln_1_gamma", &L->rms_att, d}, {"ln_1_beta", &L->ln1_beta, d},
            {"wq", &L->wq, q * d}, {"wk", &L->wk, kv * d}, {"wv", &L->wv, kv * d}, {"wo", &L->wo, d * q},
            {"bq", &L->bq, q}, {"bk", &L->bk, kv}, {"bv", &L->bv, kv}, {"bo", &L->bo, d},
            {"rms_ffn", &L->rms_ffn, d}, {"ln_2_gamma", &L->rms_ffn, d}, {"ln_2_beta", &L->ln2_beta, d},
            {"w1", &L->w1, h * d}, {"w2", &L->w2, d * h}, {"w3", &L->w3, h * d},
            {"b1", &L->b1, h}, {"b2", &L->b2, d}, {"q_norm", &L->q_norm, c->head_dim}, {"k_norm", &L->k_norm, c->head_dim},
        };
        for (size_t i = 0; i < sizeof tab / sizeof tab[0]; i++)
            if (!strcmp(leaf, tab[i].n)) { *expect = tab[i].cnt; return tab[i].p; }
    }
    return NULL;
}

ESP_ORACLE_API int esp_oracle_model_set_tensor(esp_oracle_model* m, const char* name, const float* data, int64_t count) {
    int64_t expect = 0;
    float** slot = model_slot(m, name, &expect);
    if (!slot) return -1;
    if (expect != count) return -2; /* invalidWeightCount, RealModelInferenceEngine.swift:85-115 */
    free(*slot);
    *slot = (float*)malloc(sizeof(float) * (size_t)count);
    memcpy(*slot, data, sizeof(float) * (size_t)count);
    return 0;
}

static int file_exists(const char* p) { struct stat st; return stat(p, &st) == 0; }

/* loadWeightTablePreferringFloat32Sidecar, RealModelInferenceEngine.swift:7830-7879:
 * "<name>.float32.bin" (raw LE fp32) wins over "<name>.bin" (BLOBFILE fp16). */
static int load_file_tensor(esp_oracle_model* m, const char* dir, const char* name, int required) {
    int64_t expect = 0;
    float** slot = model_slot(m, name, &expect);
    if (!slot) return -1;
    char path[4096];
    snprintf(path, sizeof path, "%s/%s.float32.bin", dir, name);
    float* buf = (float*)malloc(sizeof(float) * (size_t)expect);
    if (file_exists(path)) {
        FILE* f = fopen(path, "rb");
        if (!f) { free(buf); return -1; }
        fseek(f, 0, SEEK_END);
        long sz = ftell(f);
        fseek(f, 0, SEEK_SET);
        if (sz != (long)(expect * 4)) { fclose(f); free(buf); return -2; }
        size_t n = fread(buf, 4, (size_t)expect, f);
        fclose(f);
        if ((int64_t)n != expect) { free(buf); return -2; }
    } else {
        snprintf(path, sizeof path, "%s/%s.bin", dir, name);
        if (!file_exists(path)) { free(buf); return required ? -3 : 1; }
        int64_t cnt = esp_oracle_blob_read(path, NULL, 0);
        if (cnt < 0) { free(buf); return (int)cnt; }
        if (cnt != expect) { free(buf); return -2; }
        cnt = esp_oracle_blob_read(path, buf, expect);
        if (cnt < 0) { free(buf); return (int)cnt; }
    }
    free(*slot);
    *slot = buf;
    return 0;
}

static int load_first(esp_oracle_model* m, const char* dir, const char* const* cands, int n) {
    for (int i = 0; i < n; i++) {
        int rc = load_file_tensor(m, dir, cands[i], 0);
        if (rc == 0) return 0;
        if (rc < 0) return rc;
    }
    return -3;
}

/* Loads a weight directory in the reference layout (see model_slot). */
ESP_ORACLE_API int esp_oracle_model_load_dir(esp_oracle_model* m, const char* dir) {
    const esp_oracle_config* c = &m->cfg;
    int rc;
    const char* tok[] = {"embeddings/token", "embeddings/token_embeddings"};
    if ((rc = load_first(m, dir, tok, 2))) return rc;
    const char* head[] = {"lm_head", "classifier"};
    if ((rc = load_first(m, dir, head, 2))) return rc;
    if (c->architecture == ESP_ARCH_GPT2) {
        const char* pos[] = {"embeddings/position", "embeddings/position_embeddings"};
        if ((rc = load_first(m, dir, pos, 2))) return rc;
        const char* fg[] = {"final_norm_gamma", "ln_f_gamma", "rms_final"};
        if ((rc = load_first(m, dir, fg, 3))) return rc;
        const char* fb[] = {"final_norm_beta", "ln_f_beta", "rms_final_beta"};
        if ((rc = load_first(m, dir, fb, 3))) return rc;
    } else {
        const char* fg[] = {"rms_final", "final_norm_gamma", "final_norm"};
        if ((rc = load_first(m, dir, fg, 3))) return rc;
    }
    for (int l = 0; l < c->n_layer; l++) {
        const char* llama[] = {"rms_att", "wq", "wk", "wv", "wo", "rms_ffn", "w1", "w2", "w3"};
        const char* gpt2[] = {"ln_1_gamma", "ln_1_beta", "wq", "wk", "wv", "wo", "bq", "bk", "bv", "bo",
                              "ln_2_gamma", "ln_2_beta", "w1", "b1", "w2", "b2"};
        const char* const* names = c->architecture == ESP_ARCH_GPT2 ? gpt2 : llama;
        int n = c->architecture == ESP_ARCH_GPT2 ? 16 : 9;
        char name[128];
        for (int i = 0; i < n; i++) {
            snprintf(name, sizeof name, "layers/%d/%s", l, names[i]);
            if ((rc = load_file_tensor(m, dir, name, 1))) return rc;
        }
        if (c->architecture == ESP_ARCH_LLAMA) { /* optional, RealModelInferenceEngine.swift:6585-6607 */
            snprintf(name, sizeof name, "layers/%d/q_norm", l);
            if ((rc = load_file_tensor(m, dir, name, 0)) < 0) return rc;
            snprintf(name, sizeof name, "layers/%d/k_norm", l);
            if ((rc = load_file_tensor(m, dir, name, 0)) < 0) return rc;
        }
    }
    return 0;
}

static int model_complete(const esp_oracle_model* m) {
    const esp_oracle_config* c = &m->cfg;
    if (!m->tok_emb || !m->final_gamma || !m->lm_head) return 0;
    if (c->architecture == ESP_ARCH_GPT2 && (!m->pos_emb || !m->final_beta)) return 0;
    for (int l = 0; l < c->n_layer; l++) {
        const layer_weights* L = &m->layers[l];
        if (!L->rms_att || !L->wq || !L->wk || !L->wv || !L->wo || !L->rms_ffn || !L->w1 || !L->w2) return 0;
        if (c->architecture == ESP_ARCH_LLAMA && !L->w3) return 0;
        if (c->architecture == ESP_ARCH_GPT2 &&
            (!L->ln1_beta || !L->ln2_beta || !L->bq || !L->bk || !L->bv || !L->bo || !L->b1 || !L->b2))
            return 0;
    }
    return 1;
}

/* ------------------------------------------------------------ runtime */
/* CPUExactLlamaRuntime, RealModelInferenceEngine.swift:548-850 (state: lastHidden, K/V caches
 * [layer][kvDim*maxSeq] channel-major, visibleTokenCount); the GPT-2 variant restates the layer graph
 * of RealModelInferenceEngine.swift:7353-7541 with the same cache layout and cpuDecodeContext. */
typedef struct esp_oracle_runtime {
    const esp_oracle_model* m;
    int round_fp16;
    float** k_cache;
    float** v_cache;
    float* last_hidden;
    int visible;
    /* scratch */
    float *normed, *q, *k, *v, *ctx, *proj, *gate, *up, *act, *down, *logits;
    /* optional per-stage capture of the last advance() (mirrors the reference's testing dumps,
     * RealModelInferenceEngine.swift:419-484) */
    int capture_layer;
    float *cap_q, *cap_k, *cap_v, *cap_ctx, *cap_proj, *cap_act, *cap_hidden;
} esp_oracle_runtime;

typedef struct {
    int visible;
    float* last_hidden;
    float** k_cache;
    float** v_cache;
    int n_layer;
} esp_oracle_checkpoint;

static float* fzeros(size_t n) { return (float*)calloc(n ? n : 1, sizeof(float)); }

ESP_ORACLE_API esp_oracle_runtime* esp_oracle_runtime_create(const esp_oracle_model* m, int round_fp16) {
    if (!m || !model_complete(m)) return NULL;
    const esp_oracle_config* c = &m->cfg;
    esp_oracle_runtime* r = (esp_oracle_runtime*)calloc(1, sizeof *r);
    r->m = m;
    r->round_fp16 = round_fp16;
    r->k_cache = (float**)calloc((size_t)c->n_layer, sizeof(float*));
    r->v_cache = (float**)calloc((size_t)c->n_layer, sizeof(float*));
    size_t cs = (size_t)kv_dim(c) * c->max_seq;
    for (int l = 0; l < c->n_layer; l++) { r->k_cache[l] = fzeros(cs); r->v_cache[l] = fzeros(cs); }
    int d = c->d_model, q = q_dim(c), kv = kv_dim(c), h = c->hidden_dim;
    r->last_hidden = fzeros(d);
    r->normed = fzeros(d); r->q = fzeros(q); r->k = fzeros(kv); r->v = fzeros(kv); r->ctx = fzeros(q);
    r->proj = fzeros(d); r->gate = fzeros(h); r->up = fzeros(h); r->act = fzeros(h); r->down = fzeros(d);
    r->logits = fzeros(c->vocab);
    r->capture_layer = -1;
    r->cap_q = fzeros(q); r->cap_k = fzeros(kv); r->cap_v = fzeros(kv); r->cap_ctx = fzeros(q);
    r->cap_proj = fzeros(d); r->cap_act = fzeros(h); r->cap_hidden = fzeros(d);
    return r;
}

ESP_ORACLE_API void esp_oracle_runtime_destroy(esp_oracle_runtime* r) {
    if (!r) return;
    for (int l = 0; l < r->m->cfg.n_layer; l++) { free(r->k_cache[l]); free(r->v_cache[l]); }
    free(r->k_cache); free(r->v_cache); free(r->last_hidden);
    free(r->normed); free(r->q); free(r->k); free(r->v); free(r->ctx); free(r->proj);
    free(r->gate); free(r->up); free(r->act); free(r->down); free(r->logits);
    free(r->cap_q); free(r->cap_k); free(r->cap_v); free(r->cap_ctx); free(r->cap_proj); free(r->cap_act); free(r->cap_hidden);
    free(r);
}

/* reset, RealModelInferenceEngine.swift:613-635. */
ESP_ORACLE_API void esp_oracle_runtime_reset(esp_oracle_runtime* r) {
    const esp_oracle_config* c = &r->m->cfg;
    size_t cs = (size_t)kv_dim(c) * c->max_seq;
    for (int l = 0; l < c->n_layer; l++) {
        memset(r->k_cache[l], 0, cs * sizeof(float));
        memset(r->v_cache[l], 0, cs * sizeof(float));
    }
    memset(r->last_hidden, 0, sizeof(float) * (size_t)c->d_model);
    r->visible = 0;
}

static void maybe_round(const esp_oracle_runtime* r, float* v, int n) {
    if (!r->round_fp16) return;
    for (int i = 0; i < n; i++) v[i] = round_half(v[i]);
}

static void add_bias(float* y, const float* b, int n) { for (int i = 0; i < n; i++) y[i] += b[i]; }

/* forwardToken: Llama RealModelInferenceEngine.swift:686-823 (same body at :6221-6347);
 * GPT-2 layer graph :7353-7499 with embeddings :5435-5453. Writes the new hidden into `hidden`. */
static int forward_token(esp_oracle_runtime* r, uint32_t token, int position, float* hidden) {
    const esp_oracle_model* m = r->m;
    const esp_oracle_config* c = &m->cfg;
    if ((int64_t)token >= c->vocab) return -2;
    int d = c->d_model, q = q_dim(c), kv = kv_dim(c), h = c->hidden_dim, S = c->max_seq;
    int gpt2 = c->architecture == ESP_ARCH_GPT2;
    memcpy(hidden, m->tok_emb + (size_t)token * d, sizeof(float) * (size_t)d);
    if (gpt2)
        for (int i = 0; i < d; i++) hidden[i] += m->pos_emb[(size_t)position * d + i];
    for (int l = 0; l < c->n_layer; l++) {
        const layer_weights* L = &m->layers[l];
        if (gpt2) esp_oracle_layernorm(hidden, L->rms_att, L->ln1_beta, d, c->norm_eps, r->normed);
        else esp_oracle_rmsnorm(hidden, L->rms_att, d, c->norm_eps, r->normed);
        esp_oracle_gemv(L->wq, q, d, r->normed, r->q);
        esp_oracle_gemv(L->wk, kv, d, r->normed, r->k);
        esp_oracle_gemv(L->wv, kv, d, r->normed, r->v);
        if (gpt2) { add_bias(r->q, L->bq, q); add_bias(r->k, L->bk, kv); add_bias(r->v, L->bv, kv); }
        maybe_round(r, r->q, q); maybe_round(r, r->k, kv); maybe_round(r, r->v, kv);
        if (L->q_norm) esp_oracle_per_head_rmsnorm(r->q, L->q_norm, c->n_head, c->head_dim, c->norm_eps);
        if (L->k_norm) esp_oracle_per_head_rmsnorm(r->k, L->k_norm, c->n_kv_head, c->head_dim, c->norm_eps);
        if (!gpt2) {
            esp_oracle_rope_half_split(r->q, c->n_head, c->head_dim, position, c->rope_theta);
            esp_oracle_rope_half_split(r->k, c->n_kv_head, c->head_dim, position, c->rope_theta);
            maybe_round(r, r->q, q); maybe_round(r, r->k, kv);
        }
        for (int ch = 0; ch < kv; ch++) { /* KV append, :769-772 */
            r->k_cache[l][(size_t)ch * S + position] = r->k[ch];
            r->v_cache[l][(size_t)ch * S + position] = r->v[ch];
        }
        esp_oracle_decode_context(r->q, r->k_cache[l], r->v_cache[l], c->n_head, c->n_kv_head, c->head_dim,
                                  position + 1, 0, S, r->ctx);
        esp_oracle_gemv(L->wo, d, q, r->ctx, r->proj);
        if (gpt2) add_bias(r->proj, L->bo, d);
        for (int i = 0; i < d; i++) r->proj[i] += hidden[i];
        maybe_round(r, r->proj, d);
        if (gpt2) {
            esp_oracle_layernorm(r->proj, L->rms_ffn, L->ln2_beta, d, c->norm_eps, r->normed);
            esp_oracle_gemv(L->w1, h, d, r->normed, r->gate);
            add_bias(r->gate, L->b1, h);
            for (int i = 0; i < h; i++) r->act[i] = esp_oracle_gelu(r->gate[i]);
        } else {
            esp_oracle_rmsnorm(r->proj, L->rms_ffn, d, c->norm_eps, r->normed);
            esp_oracle_gemv(L->w1, h, d, r->normed, r->gate);
            esp_oracle_gemv(L->w3, h, d, r->normed, r->up);
            for (int i = 0; i < h; i++) r->act[i] = esp_oracle_silu(r->gate[i]) * r->up[i];
        }
        esp_oracle_gemv(L->w2, d, h, r->act, r->down);
        if (gpt2) add_bias(r->down, L->b2, d);
        for (int i = 0; i < d; i++) hidden[i] = r->proj[i] + r->down[i];
        maybe_round(r, hidden, d);
        if (l == r->capture_layer) {
            memcpy(r->cap_q, r->q, sizeof(float) * (size_t)q);
            memcpy(r->cap_k, r->k, sizeof(float) * (size_t)kv);
            memcpy(r->cap_v, r->v, sizeof(float) * (size_t)kv);
            memcpy(r->cap_ctx, r->ctx, sizeof(float) * (size_t)q);
            memcpy(r->cap_proj, r->proj, sizeof(float) * (size_t)d);
            memcpy(r->cap_act, r->act, sizeof(float) * (size_t)h);
            memcpy(r->cap_hidden, hidden, sizeof(float) * (size_t)d);
        }
    }
    return 0;
}

/* advance, RealModelInferenceEngine.swift:672-680: position guard, then forwardToken. */
ESP_ORACLE_API int esp_oracle_runtime_advance(esp_oracle_runtime* r, uint32_t token) {
    if (r->visible >= r->m->cfg.max_seq) return -1;
    float* hid = fzeros((size_t)r->m->cfg.d_model);
    int rc = forward_token(r, token, r->visible, hid);
    if (rc == 0) {
        maybe_round(r, hid, r->m->cfg.d_model);
        memcpy(r->last_hidden, hid, sizeof(float) * (size_t)r->m->cfg.d_model);
        r->visible += 1;
    }
    free(hid);
    return rc;
}

/* prefill = reset + advance per prompt token, RealModelInferenceEngine.swift:637-645. */
ESP_ORACLE_API int esp_oracle_runtime_prefill(esp_oracle_runtime* r, const uint32_t* tokens, int n) {
    if (n <= 0) return -3;
    esp_oracle_runtime_reset(r);
    for (int i = 0; i < n; i++) {
        int rc = esp_oracle_runtime_advance(r, tokens[i]);
        if (rc) return rc;
    }
    return 0;
}

static void final_norm(const esp_oracle_runtime* r, float* out) {
    const esp_oracle_model* m = r->m;
    if (m->cfg.architecture == ESP_ARCH_GPT2)
        esp_oracle_layernorm(r->last_hidden, m->final_gamma, m->final_beta, m->cfg.d_model, m->cfg.norm_eps, out);
    else
        esp_oracle_rmsnorm(r->last_hidden, m->final_gamma, m->cfg.d_model, m->cfg.norm_eps, out);
}

/* Full logits: projectLogits, RealModelInferenceEngine.swift:8154-8180, on the final-normed hidden. */
ESP_ORACLE_API void esp_oracle_runtime_logits(esp_oracle_runtime* r, float* out) {
    final_norm(r, r->normed);
    esp_oracle_gemv(r->m->lm_head, r->m->cfg.vocab, r->m->cfg.d_model, r->normed, out);
}

/* selectGreedyToken, RealModelInferenceEngine.swift:663-670 -> exactClassifierArgmax -> partitionedArgmax (4000-row blocks). */
ESP_ORACLE_API uint32_t esp_oracle_runtime_select_greedy(esp_oracle_runtime* r) {
    final_norm(r, r->normed);
    return (uint32_t)esp_oracle_partitioned_argmax(r->m->lm_head, r->normed, r->m->cfg.vocab, r->m->cfg.d_model, 4000);
}

ESP_ORACLE_API int esp_oracle_runtime_visible(const esp_oracle_runtime* r) { return r->visible; }
ESP_ORACLE_API const float* esp_oracle_runtime_last_hidden(const esp_oracle_runtime* r) { return r->last_hidden; }
ESP_ORACLE_API const float* esp_oracle_runtime_k_cache(const esp_oracle_runtime* r, int layer) { return r->k_cache[layer]; }
ESP_ORACLE_API const float* esp_oracle_runtime_v_cache(const esp_oracle_runtime* r, int layer) { return r->v_cache[layer]; }
ESP_ORACLE_API void esp_oracle_runtime_set_capture_layer(esp_oracle_runtime* r, int layer) { r->capture_layer = layer; }
/* stage: 0 q (post-RoPE), 1 k (post-RoPE), 2 v, 3 context, 4 projected (hidden + Wo.ctx), 5 activated, 6 layer output */
ESP_ORACLE_API const float* esp_oracle_runtime_captured(const esp_oracle_runtime* r, int stage) {
    switch (stage) {
        case 0: return r->cap_q; case 1: return r->cap_k; case 2: return r->cap_v; case 3: return r->cap_ctx;
        case 4: return r->cap_proj; case 5: return r->cap_act; case 6: return r->cap_hidden; default: return NULL;
    }
}

/* captureCheckpoint / rollback, RealModelInferenceEngine.swift:647-661 (full copies of the caches). */
ESP_ORACLE_API esp_oracle_checkpoint* esp_oracle_runtime_checkpoint(const esp_oracle_runtime* r) {
    const esp_oracle_config* c = &r->m->cfg;
    esp_oracle_checkpoint* cp = (esp_oracle_checkpoint*)calloc(1, sizeof *cp);
    size_t cs = (size_t)kv_dim(c) * c->max_seq;
    cp->visible = r->visible;
    cp->n_layer = c->n_layer;
    cp->last_hidden = fzeros((size_t)c->d_model);
    memcpy(cp->last_hidden, r->last_hidden, sizeof(float) * (size_t)c->d_model);
    cp->k_cache = (float**)calloc((size_t)c->n_layer, sizeof(float*));
    cp->v_cache = (float**)calloc((size_t)c->n_layer, sizeof(float*));
    for (int l = 0; l < c->n_layer; l++) {
        cp->k_cache[l] = (float*)malloc(cs * sizeof(float));
        cp->v_cache[l] = (float*)malloc(cs * sizeof(float));
        memcpy(cp->k_cache[l], r->k_cache[l], cs * sizeof(float));
        memcpy(cp->v_cache[l], r->v_cache[l], cs * sizeof(float));
    }
    return cp;
}

ESP_ORACLE_API void esp_oracle_runtime_rollback(esp_oracle_runtime* r, const esp_oracle_checkpoint* cp) {
    const esp_oracle_config* c = &r->m->cfg;
    size_t cs = (size_t)kv_dim(c) * c->max_seq;
    r->visible = cp->visible;
    memcpy(r->last_hidden, cp->last_hidden, sizeof(float) * (size_t)c->d_model);
    for (int l = 0; l < c->n_layer; l++) {
        memcpy(r->k_cache[l], cp->k_cache[l], cs * sizeof(float));
        memcpy(r->v_cache[l], cp->v_cache[l], cs * sizeof(float));
    }
}

ESP_ORACLE_API void esp_oracle_checkpoint_destroy(esp_oracle_checkpoint* cp) {
    if (!cp) return;
    for (int l = 0; l < cp->n_layer; l++) { free(cp->k_cache[l]); free(cp->v_cache[l]); }
    free(cp->k_cache); free(cp->v_cache); free(cp->last_hidden); free(cp);
}

/* ------------------------------------------------------------ generation loops */

/* Greedy generation from token ids (generateIncrementalExactCPULlama, RealModelInferenceEngine.swift:6349-6431;
 * limits :1419-1426). Llama: an EOS token is appended, then generation stops (:6385-6388). GPT-2: token 50256
 * stops generation without being appended (:1251, :4920-4922). Returns the number of generated tokens or < 0. */
ESP_ORACLE_API int esp_oracle_generate(esp_oracle_runtime* r, const uint32_t* prompt, int n_prompt, int max_tokens,
                                       uint32_t* out) {
    const esp_oracle_config* c = &r->m->cfg;
    if (n_prompt <= 0) return -3;
    if (n_prompt >= c->max_seq) return -4;
    if (max_tokens < 0) return -5;
    int remaining = c->max_seq - n_prompt;
    int eff = max_tokens < remaining ? max_tokens : remaining;
    if (eff == 0) return 0;
    int rc = esp_oracle_runtime_prefill(r, prompt, n_prompt);
    if (rc) return rc;
    int total = n_prompt, gen = 0;
    while (gen < eff) {
        uint32_t next = esp_oracle_runtime_select_greedy(r);
        if (c->architecture == ESP_ARCH_GPT2) {
            if (next == 50256u) break;
        } else if (c->eos_token >= 0 && next == (uint32_t)c->eos_token) {
            out[gen++] = next;
            break;
        }
        out[gen++] = next;
        total++;
        if (gen >= eff || total >= c->max_seq) break;
        rc = esp_oracle_runtime_advance(r, next);
        if (rc) return rc;
    }
    return gen;
}

typedef struct {
    int passes;
    int committed_exact_tokens;
    int accepted_future_tokens;
} esp_oracle_two_token_stats;

/* generateIncrementalExactTwoTokenDraftLlama, RealModelInferenceEngine.swift:6014-6190. */
ESP_ORACLE_API int esp_oracle_generate_two_token(esp_oracle_runtime* full, esp_oracle_runtime* draft,
                                                 const uint32_t* prompt, int n_prompt, int max_tokens, uint32_t* out,
                                                 esp_oracle_two_token_stats* stats) {
    const esp_oracle_config* c = &full->m->cfg;
    if (n_prompt <= 0) return -3;
    if (n_prompt >= c->max_seq) return -4;
    int remaining_ctx = c->max_seq - n_prompt;
    int eff = max_tokens < remaining_ctx ? max_tokens : remaining_ctx;
    if (stats) memset(stats, 0, sizeof *stats);
    if (eff <= 0) return 0;
    int rc;
    if ((rc = esp_oracle_runtime_prefill(full, prompt, n_prompt))) return rc;
    if ((rc = esp_oracle_runtime_prefill(draft, prompt, n_prompt))) return rc;
    int gen = 0, total = n_prompt, passes = 0, committed = 0, accepted = 0;
    int eos = c->eos_token;
    uint32_t first = esp_oracle_runtime_select_greedy(full);
    out[gen++] = first;
    if (eos >= 0 && first == (uint32_t)eos) return gen;
    total++;
    if (gen >= eff || total >= c->max_seq) return gen;
    if ((rc = esp_oracle_runtime_advance(full, first))) return rc;
    if ((rc = esp_oracle_runtime_advance(draft, first))) return rc;
    while (gen < eff && total < c->max_seq) {
        passes++;
        int budget = eff - gen < c->max_seq - total ? eff - gen : c->max_seq - total;
        esp_oracle_checkpoint* cp = esp_oracle_runtime_checkpoint(draft);
        uint32_t p0 = esp_oracle_runtime_select_greedy(draft);
        if ((rc = esp_oracle_runtime_advance(draft, p0))) { esp_oracle_checkpoint_destroy(cp); return rc; }
        uint32_t e0 = esp_oracle_runtime_select_greedy(full);
        int acc = 0, com = 0;
        if (e0 == p0) acc++;
        else esp_oracle_runtime_rollback(draft, cp);
        esp_oracle_checkpoint_destroy(cp);
        out[gen++] = e0; total++; com++;
        if (eos >= 0 && e0 == (uint32_t)eos) { committed += com; accepted += acc; break; }
        if ((rc = esp_oracle_runtime_advance(full, e0))) return rc;
        if (e0 != p0 && (rc = esp_oracle_runtime_advance(draft, e0))) return rc;
        if (gen >= eff || total >= c->max_seq || budget <= 1) { committed += com; accepted += acc; continue; }
        uint32_t p1 = esp_oracle_runtime_select_greedy(draft);
        uint32_t e1 = esp_oracle_runtime_select_greedy(full);
        if (e1 == p1) acc++;
        out[gen++] = e1; total++; com++;
        if (eos >= 0 && e1 == (uint32_t)eos) { committed += com; accepted += acc; break; }
        if ((rc = esp_oracle_runtime_advance(full, e1))) return rc;
        if ((rc = esp_oracle_runtime_advance(draft, e1))) return rc;
        committed += com; accepted += acc;
    }
    if (stats) { stats->passes = passes; stats->committed_exact_tokens = committed; stats->accepted_future_tokens = accepted; }
    return gen;
}

/* ExactTwoTokenBranchPromotionPlan.make, Sources/Espresso/GenerationHarness.swift:149-181.
 * committed[0..n) receives the tokens committed by this pass; *next_current is the token the next pass starts
 * from. Returns the number of committed tokens (1 or 2). */
ESP_ORACLE_API int esp_oracle_two_token_plan(uint32_t current, uint32_t proposed_future, uint32_t exact_next,
                                             uint32_t exact_future, int remaining, uint32_t* committed,
                                             uint32_t* next_current) {
    committed[0] = current;
    if (remaining > 1 && proposed_future == exact_next) {
        committed[1] = exact_next;
        *next_current = exact_future;
        return 2;
    }
    *next_current = exact_next;
    return 1;
}

ESP_ORACLE_API int esp_oracle_num_threads(void) {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ESP_ORACLE_API void esp_oracle_set_num_threads(int n) {
#if defined(_OPENMP)
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
