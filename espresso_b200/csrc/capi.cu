// extern "C" surface of libespresso_cuda.so (see include/espresso_cuda.h) and the host-side generation
// loops that mirror RealModelInferenceEngine's token-id entry points.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "engine.h"

namespace esp {
void set_force_failure(int on);
int32_t tp_unique_id(uint8_t* out, int32_t capacity);
int32_t gemv_bench(int32_t type, const void* weights, int32_t rows, int32_t cols, const float* x, float* y, int32_t warmup,
                   int32_t iterations, int32_t copies, float* avg_ms, int32_t device);
__global__ void k_dequant(const uint8_t* blocks, int type, int64_t n_blocks, float* out);
}

struct esp_cuda_engine {
    esp::Engine impl;
    explicit esp_cuda_engine(const esp_cuda_config& c) : impl(c) {}
};

static std::atomic<int> g_live_engines{0};

static int32_t fail(int32_t code, const std::string& msg) {
    esp::set_last_error(msg);
    return code;
}

#define ESP_GUARD(engine) \
    if (!(engine)) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "null engine handle")

// ---- metadata.json (Sources/ESPCompiler/ESPModelConfigIO.swift:12-59): a flat JSON object ------------

static bool json_find(const std::string& text, const char* key, std::string* raw) {
    std::string pat = std::string("\"") + key + "\"";
    size_t p = text.find(pat);
    if (p == std::string::npos) return false;
    p = text.find(':', p + pat.size());
    if (p == std::string::npos) return false;
    p++;
    while (p < text.size() && isspace((unsigned char)text[p])) p++;
    size_t e = p;
    if (p < text.size() && text[p] == '"') {
        e = text.find('"', p + 1);
        if (e == std::string::npos) return false;
        *raw = text.substr(p + 1, e - p - 1);
        return true;
    }
    while (e < text.size() && text[e] != ',' && text[e] != '}' && !isspace((unsigned char)text[e])) e++;
    *raw = text.substr(p, e - p);
    return *raw != "null";
}

static int32_t read_metadata(const std::string& dir, esp_cuda_config* c) {
    std::ifstream f(dir + "/metadata.json");
    if (!f) return fail(ESP_CUDA_ERR_IO, "missing metadata.json in " + dir);
    std::stringstream ss;
    ss << f.rdbuf();
    std::string t = ss.str(), v;
    struct { const char* k; int32_t* dst; } ints[] = {
        {"nLayer", &c->n_layer}, {"nHead", &c->n_head}, {"nKVHead", &c->n_kv_head}, {"dModel", &c->d_model},
        {"headDim", &c->head_dim}, {"hiddenDim", &c->hidden_dim}, {"vocab", &c->vocab}, {"maxSeq", &c->max_seq}};
    for (auto& e : ints) {
        if (!json_find(t, e.k, &v)) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, std::string("metadata.json: missing key ") + e.k);
        *e.dst = atoi(v.c_str());
    }
    if (!json_find(t, "normEps", &v)) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "metadata.json: missing key normEps");
    c->norm_eps = strtof(v.c_str(), nullptr);
    c->rope_theta = json_find(t, "ropeTheta", &v) ? strtof(v.c_str(), nullptr) : 10000.0f;  // default, ESPModelConfigIO.swift:53
    c->eos_token = json_find(t, "eosToken", &v) ? atoi(v.c_str()) : -1;
    if (!json_find(t, "architecture", &v)) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "metadata.json: missing key architecture");
    for (auto& ch : v) ch = (char)tolower((unsigned char)ch);
    if (v == "llama") c->architecture = ESP_CUDA_ARCH_LLAMA;
    else if (v == "gpt2") c->architecture = ESP_CUDA_ARCH_GPT2;
    else return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "Unsupported metadata architecture: " + v);
    return ESP_CUDA_OK;
}

extern "C" {

int32_t esp_cuda_create(const esp_cuda_config* config, const char* weight_dir, esp_cuda_engine** out) {
    if (!config || !out) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "esp_cuda_create: null argument");
    *out = nullptr;
    esp_cuda_engine* e = new (std::nothrow) esp_cuda_engine(*config);
    if (!e) return fail(ESP_CUDA_ERR_OUT_OF_MEMORY, "host allocation failed");
    int32_t rc = e->impl.init();
    if (rc == ESP_CUDA_OK && weight_dir) {
        rc = e->impl.load_directory(weight_dir);
        if (rc == ESP_CUDA_OK) rc = e->impl.finalize();
    }
    if (rc != ESP_CUDA_OK) { delete e; return rc; }
    g_live_engines.fetch_add(1);
    *out = e;
    return ESP_CUDA_OK;
}

int32_t esp_cuda_create_from_directory(const char* weight_dir, int32_t max_batch, int32_t device, uint32_t flags,
                                       esp_cuda_engine** out) {
    if (!weight_dir || !out) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "esp_cuda_create_from_directory: null argument");
    esp_cuda_config c{};
    int32_t rc = read_metadata(weight_dir, &c);
    if (rc) return rc;
    c.max_batch = max_batch; c.device = device; c.tp_rank = 0; c.tp_size = 1; c.flags = (int32_t)flags;
    return esp_cuda_create(&c, weight_dir, out);
}

int32_t esp_cuda_load_tensor(esp_cuda_engine* engine, const char* name, int32_t type, const void* data, uint64_t nbytes) {
    ESP_GUARD(engine);
    return engine->impl.load_tensor(name, type, data, nbytes);
}
int32_t esp_cuda_tp_unique_id(uint8_t* out, int32_t capacity) { return esp::tp_unique_id(out, capacity); }
int32_t esp_cuda_tp_init(esp_cuda_engine* engine, const uint8_t* unique_id, int32_t nbytes) {
    ESP_GUARD(engine);
    return engine->impl.tp_init(unique_id, nbytes);
}
int32_t esp_cuda_finalize(esp_cuda_engine* engine) { ESP_GUARD(engine); return engine->impl.finalize(); }
int32_t esp_cuda_destroy(esp_cuda_engine* engine) {
    ESP_GUARD(engine);
    delete engine;
    g_live_engines.fetch_sub(1);
    return ESP_CUDA_OK;
}
int32_t esp_cuda_get_config(const esp_cuda_engine* engine, esp_cuda_config* out) {
    ESP_GUARD(engine);
    if (!out) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "null output");
    *out = engine->impl.config();
    return ESP_CUDA_OK;
}

int32_t esp_cuda_reset(esp_cuda_engine* engine) { ESP_GUARD(engine); return engine->impl.reset(); }
int32_t esp_cuda_prefill(esp_cuda_engine* engine, const uint32_t* tokens, int32_t n) { ESP_GUARD(engine); return engine->impl.prefill(tokens, n); }
int32_t esp_cuda_advance(esp_cuda_engine* engine, uint32_t token) { ESP_GUARD(engine); return engine->impl.advance(token); }
int32_t esp_cuda_select_greedy(esp_cuda_engine* engine, uint32_t* token) { ESP_GUARD(engine); return engine->impl.select_greedy(token); }
int32_t esp_cuda_decode_step(esp_cuda_engine* engine, uint32_t token, uint32_t* next) { ESP_GUARD(engine); return engine->impl.decode_step(token, next); }
int32_t esp_cuda_visible_token_count(const esp_cuda_engine* engine, int32_t seq, int32_t* count) {
    ESP_GUARD(engine);
    if (!count || seq < 0 || seq >= engine->impl.config().max_batch) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "bad sequence index");
    *count = engine->impl.visible(seq);
    return ESP_CUDA_OK;
}
int32_t esp_cuda_get_logits(esp_cuda_engine* engine, int32_t seq, float* out, int32_t vocab) { ESP_GUARD(engine); return engine->impl.get_logits(seq, out, vocab); }
int32_t esp_cuda_checkpoint(esp_cuda_engine* engine, int32_t* id) { ESP_GUARD(engine); return engine->impl.checkpoint(id); }
int32_t esp_cuda_rollback(esp_cuda_engine* engine, int32_t id) { ESP_GUARD(engine); return engine->impl.rollback(id); }
int32_t esp_cuda_verify2(esp_cuda_engine* engine, uint32_t current, uint32_t proposed, uint32_t* exact_next, uint32_t* exact_future) {
    ESP_GUARD(engine);
    return engine->impl.verify2(current, proposed, exact_next, exact_future);
}
int32_t esp_cuda_commit(esp_cuda_engine* engine, int32_t steps) { ESP_GUARD(engine); return engine->impl.commit(steps); }
int32_t esp_cuda_prefill_batch(esp_cuda_engine* engine, const uint32_t* tokens, int32_t n_seq, int32_t len) {
    ESP_GUARD(engine);
    return engine->impl.prefill_batch(tokens, n_seq, len);
}
int32_t esp_cuda_decode_step_batch(esp_cuda_engine* engine, const uint32_t* tokens, int32_t n_seq, uint32_t* next) {
    ESP_GUARD(engine);
    return engine->impl.decode_step_batch(tokens, n_seq, next);
}

int32_t esp_cuda_generate(esp_cuda_engine* engine, const uint32_t* prompt, int32_t n_prompt, int32_t max_tokens,
                          uint32_t* out_tokens, int32_t* n_out, esp_cuda_generation_result* result) {
    ESP_GUARD(engine);
    return engine->impl.generate_batch(prompt, 1, n_prompt, max_tokens, out_tokens, n_out, result);
}
int32_t esp_cuda_generate_batch(esp_cuda_engine* engine, const uint32_t* prompts, int32_t n_seq, int32_t n_prompt,
                                int32_t max_tokens, uint32_t* out_tokens, int32_t* n_out, esp_cuda_generation_result* result) {
    ESP_GUARD(engine);
    return engine->impl.generate_batch(prompts, n_seq, n_prompt, max_tokens, out_tokens, n_out, result);
}

// Step-by-step generation with the caller's callback invoked inline after every token, as the reference's loop does
// with onStep (Engine.swift:6393-6405): prefill, select the first token, then one decode step per token.  Limits and
// stop rules as in generate (Llama: the EOS token is emitted, then the loop stops, :6385-6388; GPT-2: 50256 stops
// without being emitted, :4918-4922).
int32_t esp_cuda_generate_steps(esp_cuda_engine* engine, const uint32_t* prompt, int32_t n_prompt, int32_t max_tokens,
                                esp_cuda_step_callback on_step, void* user, uint32_t* out_tokens, int32_t* n_out,
                                esp_cuda_generation_result* result) {
    ESP_GUARD(engine);
    if (!prompt || !out_tokens || !n_out) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "generate_steps: null argument");
    esp::Engine& e = engine->impl;
    const esp_cuda_config& c = e.config();
    if (n_prompt <= 0) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "Prompt tokens must not be empty");
    if (max_tokens < 0) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "maxTokens must be >= 0");
    if (n_prompt >= c.max_seq) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "Prompt token count exceeds model context");
    const int eff = std::min(max_tokens, c.max_seq - n_prompt);
    if (result) { *result = esp_cuda_generation_result{}; result->prompt_tokens = n_prompt; }
    *n_out = 0;
    if (eff == 0) return ESP_CUDA_OK;
    auto now = [] { return std::chrono::steady_clock::now(); };
    auto ms = [](auto a, auto b) { return std::chrono::duration<double, std::milli>(b - a).count(); };
    auto t0 = now();
    int32_t rc;
    if ((rc = e.prefill(prompt, n_prompt))) return rc;
    auto t_prefill = now();
    auto t_last = t_prefill;
    std::vector<float> latencies;
    int gen = 0;
    bool hit_eos = false;
    double first_ms = 0.0;
    uint32_t tok = 0;
    if ((rc = e.select_greedy(&tok))) return rc;
    while (true) {
        if (c.architecture == ESP_CUDA_ARCH_GPT2 && tok == 50256u) { hit_eos = true; break; }
        auto t = now();
        const double lat = ms(t_last, t);
        t_last = t;
        if (gen == 0) first_ms = lat;
        out_tokens[gen] = tok;
        latencies.push_back((float)lat);
        if (on_step) on_step(user, tok, gen, lat);
        gen++;
        if (c.architecture != ESP_CUDA_ARCH_GPT2 && c.eos_token >= 0 && tok == (uint32_t)c.eos_token) { hit_eos = true; break; }
        if (gen >= eff || n_prompt + gen >= c.max_seq) break;
        uint32_t next = 0;
        if ((rc = e.decode_step(tok, &next))) return rc;
        tok = next;
    }
    auto t_end = now();
    *n_out = gen;
    e.set_token_latencies(latencies);
    if (result) {
        result->generated_tokens = gen;
        result->prefill_ms = ms(t0, t_prefill);
        result->first_token_latency_ms = first_ms;
        result->total_decode_ms = ms(t_prefill, t_end);
        result->tokens_per_second = gen / std::max(result->total_decode_ms / 1000.0, 1e-9);
        result->stopped_on_eos = hit_eos ? 1 : 0;
    }
    return ESP_CUDA_OK;
}

int32_t esp_cuda_token_latencies(esp_cuda_engine* engine, float* out_ms, int32_t capacity, int32_t* n) {
    ESP_GUARD(engine);
    return engine->impl.token_latencies(out_ms, capacity, n);
}

int32_t esp_cuda_decode(esp_cuda_engine* engine, int32_t n_seq, int32_t count, uint32_t* out_tokens, int32_t* n_out,
                        float* device_ms) {
    ESP_GUARD(engine);
    return engine->impl.decode_loop(n_seq, count, out_tokens, count, n_out, device_ms, nullptr);
}

// Exact two-token generation.  Each pass: the draft proposes the token that follows `current`; the target runs
// ONE forward over the two positions [current, proposed] (esp_cuda_verify2) and the pair is promoted by the
// rule of ExactTwoTokenBranchPromotionPlan.make (Sources/Espresso/GenerationHarness.swift:149-181): commit
// [current, exactNext] and continue from exactFuture iff proposed == exactNext and more than one token remains,
// else commit [current] and continue from exactNext.  Emission order, EOS handling and the per-pass statistics
// follow generateIncrementalExactTwoTokenDraftLlama (Engine.swift:6014-6190); the stream equals plain greedy
// decoding of the target.
int32_t esp_cuda_generate_two_token(esp_cuda_engine* engine, esp_cuda_engine* draft, const uint32_t* prompt,
                                    int32_t n_prompt, int32_t max_tokens, uint32_t* out_tokens, int32_t* n_out,
                                    esp_cuda_generation_result* result) {
    ESP_GUARD(engine);
    ESP_GUARD(draft);
    if (!prompt || !out_tokens || !n_out) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "generate_two_token: null argument");
    esp::Engine& full = engine->impl;
    esp::Engine& dr = draft->impl;
    const esp_cuda_config& c = full.config();
    if (c.architecture != ESP_CUDA_ARCH_LLAMA) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "two-token generation is defined for llama models");
    if (dr.config().vocab != c.vocab) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "draft and target must share one vocabulary");
    if (n_prompt <= 0) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "Prompt tokens must not be empty");
    if (max_tokens < 0) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "maxTokens must be >= 0");
    const int max_seq = std::min(c.max_seq, dr.config().max_seq);
    if (n_prompt >= max_seq) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "Prompt token count exceeds model context");
    const int eff = std::min(max_tokens, max_seq - n_prompt);
    if (result) { *result = esp_cuda_generation_result{}; result->prompt_tokens = n_prompt; }
    *n_out = 0;
    if (eff == 0) return ESP_CUDA_OK;
    auto now = [] { return std::chrono::steady_clock::now(); };
    auto ms = [](auto a, auto b) { return std::chrono::duration<double, std::milli>(b - a).count(); };
    auto t0 = now();
    int32_t rc;
    if ((rc = full.prefill(prompt, n_prompt))) return rc;
    if ((rc = dr.prefill(prompt, n_prompt))) return rc;
    auto t_prefill = now();
    int gen = 0, total = n_prompt, passes = 0, committed = 0, accepted = 0;
    const int eos = c.eos_token;
    bool hit_eos = false;
    uint32_t current;
    if ((rc = full.select_greedy(&current))) return rc;
    auto t_first = now();
    // `current` is always an exact target token that has been selected but not yet fed to either model.
    if (full.spec_compatible(dr) && !(eos >= 0 && current == (uint32_t)eos) && eff > 1 && n_prompt + 1 < max_seq) {
        // draft and target share one plan: the whole loop below runs as one device-driven launch
        out_tokens[0] = current;
        int stats[5] = {0, 0, 0, 0, 0};
        rc = full.run_spec(dr, prompt[n_prompt - 1], current, 1, eff, max_seq, out_tokens, stats);
        if (rc == ESP_CUDA_OK) {
            auto t_end = now();
            *n_out = stats[0];
            if (result) {
                result->generated_tokens = stats[0];
                result->prefill_ms = ms(t0, t_prefill);
                result->first_token_latency_ms = ms(t_prefill, t_first);
                result->total_decode_ms = ms(t_prefill, t_end);
                result->tokens_per_second = stats[0] / std::max(result->total_decode_ms / 1000.0, 1e-9);
                result->speculative_passes = stats[1];
                result->committed_exact_tokens_per_pass = stats[1] ? (double)stats[2] / stats[1] : 0.0;
                result->accepted_future_tokens_per_pass = stats[1] ? (double)stats[3] / stats[1] : 0.0;
                result->stopped_on_eos = stats[4];
            }
            return ESP_CUDA_OK;
        }
        // ERR_STATE: nothing ran (the two-position working set does not fit shared memory); the host loop below takes over
        if (rc != ESP_CUDA_ERR_STATE) return rc;
    }
    std::vector<uint32_t> draft_backlog;  // committed tokens the draft has not consumed yet
    while (true) {
        // emit `current`
        out_tokens[gen++] = current;
        total++;
        if (eos >= 0 && current == (uint32_t)eos) { hit_eos = true; break; }
        if (gen >= eff || total >= max_seq) break;
        const int remaining = std::min(eff - gen, max_seq - total);
        passes++;
        // draft: consume its backlog plus `current`, propose the token after `current`
        draft_backlog.push_back(current);
        std::vector<int> seq(draft_backlog.size(), 0);
        std::vector<uint32_t> dnext(draft_backlog.size());
        if ((rc = dr.feed((int)draft_backlog.size(), seq.data(), draft_backlog.data(), true, dnext.data()))) return rc;
        draft_backlog.clear();
        const uint32_t proposed = dnext.back();
        uint32_t exact_next, exact_future;
        if (remaining > 1 && total + 1 < max_seq) {
            if ((rc = full.verify2(current, proposed, &exact_next, &exact_future))) return rc;
            if (proposed == exact_next) {
                if ((rc = full.commit(2))) return rc;
                // second committed token of this pass
                out_tokens[gen++] = exact_next;
                total++;
                committed += 2; accepted += 1;
                if (eos >= 0 && exact_next == (uint32_t)eos) { hit_eos = true; break; }
                if (gen >= eff || total >= max_seq) break;
                draft_backlog.push_back(exact_next);
                current = exact_future;
                continue;
            }
            if ((rc = full.commit(1))) return rc;
            committed += 1;
            current = exact_next;
        } else {
            // one token left: a plain committed step (runCommittedSingleToken, GenerationHarness.swift:1296-1309)
            if ((rc = full.decode_step(current, &exact_next))) return rc;
            committed += 1;
            current = exact_next;
        }
    }
    auto t_end = now();
    *n_out = gen;
    if (result) {
        result->generated_tokens = gen;
        result->prefill_ms = ms(t0, t_prefill);
        result->first_token_latency_ms = ms(t_prefill, t_first);
        result->total_decode_ms = ms(t_prefill, t_end);
        result->tokens_per_second = gen / std::max(result->total_decode_ms / 1000.0, 1e-9);
        result->speculative_passes = passes;
        result->committed_exact_tokens_per_pass = passes ? (double)committed / passes : 0.0;
        result->accepted_future_tokens_per_pass = passes ? (double)accepted / passes : 0.0;
        result->stopped_on_eos = hit_eos ? 1 : 0;
    }
    return ESP_CUDA_OK;
}

int32_t esp_cuda_get_timings(esp_cuda_engine* engine, esp_cuda_timings* out) { ESP_GUARD(engine); return engine->impl.get_timings(out); }
int32_t esp_cuda_stage_trace(esp_cuda_engine* engine, int32_t cta, int64_t* out, int32_t capacity, int32_t* n) {
    ESP_GUARD(engine);
    return engine->impl.stage_trace(cta, reinterpret_cast<long long*>(out), capacity, n);
}
int32_t esp_cuda_token_times(esp_cuda_engine* engine, uint64_t* out_ns, int32_t capacity, int32_t* n) {
    ESP_GUARD(engine);
    return engine->impl.token_times(reinterpret_cast<unsigned long long*>(out_ns), capacity, n);
}
int32_t esp_cuda_set_debug_layer(esp_cuda_engine* engine, int32_t layer) { ESP_GUARD(engine); return engine->impl.set_debug_layer(layer); }
int32_t esp_cuda_debug_dump(esp_cuda_engine* engine, int32_t stage, float* out, int32_t capacity) { ESP_GUARD(engine); return engine->impl.debug_dump(stage, out, capacity); }
const char* esp_cuda_last_error_string(void) { return esp::last_error_cstr(); }
void esp_cuda_set_force_failure(int32_t enabled) { esp::set_force_failure(enabled); }
int32_t esp_cuda_set_wait_limit(esp_cuda_engine* engine, uint32_t spins) { ESP_GUARD(engine); return engine->impl.set_wait_limit(spins); }
int32_t esp_cuda_tp_sum_stats(esp_cuda_engine* engine, uint64_t* out3) {
    ESP_GUARD(engine);
    if (!out3) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "tp_sum_stats: null output");
    return engine->impl.tp_sum_stats(reinterpret_cast<unsigned long long*>(out3));
}
int32_t esp_cuda_live_engine_count(void) { return g_live_engines.load(); }
const char* esp_cuda_version(void) { return "espresso-cuda 0.1 (sm_100a)"; }

int32_t esp_cuda_dequantize(int32_t type, const void* blocks, int64_t n_elements, float* out, int32_t device) {
    if (!blocks || !out || n_elements < 0 || n_elements % 32) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "dequantize: bad arguments");
    if (type != ESP_CUDA_Q8_0 && type != ESP_CUDA_Q4_0) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "dequantize: type must be Q8_0 or Q4_0");
    if (esp::force_failure_enabled()) return fail(ESP_CUDA_ERR_FORCED_FAILURE, "forced failure is enabled");
    if (n_elements == 0) return ESP_CUDA_OK;
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return fail(ESP_CUDA_ERR_CUDA, cudaGetErrorString(e));
    const int64_t nb = n_elements / 32;
    const size_t in_bytes = (size_t)nb * (type == ESP_CUDA_Q8_0 ? 34 : 18);
    uint8_t* d_in = nullptr;
    float* d_out = nullptr;
    if ((e = cudaMalloc(&d_in, in_bytes)) != cudaSuccess) return fail(ESP_CUDA_ERR_OUT_OF_MEMORY, cudaGetErrorString(e));
    if ((e = cudaMalloc(&d_out, sizeof(float) * n_elements)) != cudaSuccess) { cudaFree(d_in); return fail(ESP_CUDA_ERR_OUT_OF_MEMORY, cudaGetErrorString(e)); }
    e = cudaMemcpy(d_in, blocks, in_bytes, cudaMemcpyDefault);
    if (e == cudaSuccess) {
        esp::k_dequant<<<(unsigned)((nb + 255) / 256), 256>>>(d_in, type, nb, d_out);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpy(out, d_out, sizeof(float) * n_elements, cudaMemcpyDefault);
    cudaFree(d_in);
    cudaFree(d_out);
    if (e != cudaSuccess) return fail(ESP_CUDA_ERR_CUDA, cudaGetErrorString(e));
    return ESP_CUDA_OK;
}

int32_t esp_cuda_gemv_bench(int32_t type, const void* weights, int32_t rows, int32_t cols, const float* x, float* y,
                            int32_t warmup, int32_t iterations, int32_t copies, float* avg_ms, int32_t device) {
    return esp::gemv_bench(type, weights, rows, cols, x, y, warmup, iterations, copies, avg_ms, device);
}

}  // extern "C"
