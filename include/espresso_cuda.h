/*
 * espresso_cuda.h -- C ABI of libespresso_cuda.so, the B200 (sm_100a) transformer-decode runtime
 * that stands in for Espresso's ANE/IOSurface/Metal dispatch.
 *
 * The reference's native boundary is Sources/ANEInterop/include/ane_interop.h (opaque ANEHandle,
 * ane_interop_compile / ane_interop_eval / ane_interop_free, bool-or-NULL results plus a global
 * last-error code, test hooks set_force_eval_failure / live_handle_count).  Above it the Swift engine
 * (Sources/RealModelInference/RealModelInferenceEngine.swift) owns one decoder object per model,
 * CPUExactLlamaRuntime (:548-850), with reset / prefill / advance / selectGreedyToken /
 * captureCheckpoint / rollback.  This header keeps that object model: one opaque engine handle
 * per model replica and device, plain pointers and sizes, an int32 status from every call.
 *
 * Conventions
 *  - Every function returns ESP_CUDA_OK (0) or an esp_cuda_status error; nothing aborts or traps.
 *    esp_cuda_last_error_string() describes the calling thread's last failure.
 *  - There is no CPU fallback: if the device or the kernels are unavailable the call fails.
 *  - One engine = one CUDA device + one stream.  Calls on one engine must be serialised by the
 *    caller (the reference has the same rule, Sources/ANERuntime/ANEKernel.swift:612-616);
 *    different engines may be driven from different host threads.
 *  - Token ids are uint32 (ANETypes/TokenID.swift:5).  Pointers are host pointers unless stated.
 */
#ifndef ESPRESSO_CUDA_H
#define ESPRESSO_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ESP_CUDA_API __attribute__((visibility("default")))

typedef struct esp_cuda_engine esp_cuda_engine;

typedef enum esp_cuda_status {
    ESP_CUDA_OK = 0,
    ESP_CUDA_ERR_INVALID_ARGUMENT = 1, /* RealModelInferenceError.invalidGenerationParameters / invalidConfig */
    ESP_CUDA_ERR_OUT_OF_RANGE = 2,     /* position >= maxSeq or token >= vocab (Engine.swift:673-689) */
    ESP_CUDA_ERR_CUDA = 3,             /* a CUDA runtime call failed (maps to ANEError.evaluationFailed) */
    ESP_CUDA_ERR_NCCL = 4,
    ESP_CUDA_ERR_TIMEOUT = 5,          /* a bounded device-side wait gave up */
    ESP_CUDA_ERR_OUT_OF_MEMORY = 6,
    ESP_CUDA_ERR_IO = 7,               /* weight directory / file problems (weightDirectoryNotFound, missingPath) */
    ESP_CUDA_ERR_INVALID_WEIGHTS = 8,  /* BlobWeightLoaderError.* and invalidWeightCount */
    ESP_CUDA_ERR_FORCED_FAILURE = 9,   /* esp_cuda_set_force_failure(1) is active */
    ESP_CUDA_ERR_STATE = 10            /* call not valid in the engine's current state */
} esp_cuda_status;

typedef enum esp_cuda_architecture { ESP_CUDA_ARCH_LLAMA = 0, ESP_CUDA_ARCH_GPT2 = 1 } esp_cuda_architecture;

/* Storage type of an uploaded tensor; the numeric values are the GGML type ids of a GGUF file. */
typedef enum esp_cuda_tensor_type {
    ESP_CUDA_F32 = 0,
    ESP_CUDA_F16 = 1,
    ESP_CUDA_Q4_0 = 2, /* 18-byte blocks: fp16 d + 16 bytes, low nibble = element j, high nibble = element j+16 */
    ESP_CUDA_Q8_0 = 8, /* 34-byte blocks: fp16 d + 32 x int8 */
    ESP_CUDA_BF16 = 30
} esp_cuda_tensor_type;

/* Model shape: the fields of MultiModelConfig (Sources/ModelSupport/MultiModelConfig.swift:3-55)
 * plus the placement of this replica. */
typedef struct esp_cuda_config {
    int32_t architecture; /* esp_cuda_architecture */
    int32_t n_layer, n_head, n_kv_head, d_model, head_dim, hidden_dim, vocab, max_seq;
    float norm_eps;
    float rope_theta;
    int32_t eos_token; /* -1 = none. GPT-2 always stops on 50256 (Engine.swift:1251) */
    int32_t max_batch; /* independent sequences decoded together by this engine, >= 1 */
    int32_t device;    /* CUDA device ordinal */
    int32_t tp_rank;   /* tensor-parallel rank and size; size <= 1 disables tensor parallelism */
    int32_t tp_size;
    int32_t flags;     /* ESP_CUDA_FLAG_* */
} esp_cuda_config;

#define ESP_CUDA_FLAG_KEEP_LOGITS 1u /* every step also stores the full fp32 logits (parity runs) */
#define ESP_CUDA_FLAG_NO_GRAPH 2u    /* launch kernels directly instead of replaying a CUDA graph */
#define ESP_CUDA_FLAG_NO_MEGAKERNEL 4u /* always use the per-stage kernels */
#define ESP_CUDA_FLAG_NO_TC_SHADOW 8u  /* quantised models: keep no fp16 expansion, batches use the row-wise kernels */

/* Result of a generate call: the numeric fields of GenerationResult (Engine.swift:17-55). */
typedef struct esp_cuda_generation_result {
    int32_t generated_tokens;
    int32_t prompt_tokens;
    double tokens_per_second;       /* generated / time since the end of prefill (Engine.swift:6355, 6415-6419) */
    double prefill_ms;              /* reported where the reference reports compileTimeMs */
    double first_token_latency_ms;
    double total_decode_ms;
    double committed_exact_tokens_per_pass; /* two-token path only, else 0 (Engine.swift:6170-6175) */
    double accepted_future_tokens_per_pass;
    int32_t speculative_passes;
    int32_t stopped_on_eos;
} esp_cuda_generation_result;

/* Device-time buckets of the most recent step, mirroring HybridDecodeTimingBreakdown
 * (Sources/Espresso/DecodeForwardPass.swift:322-339): projections, attention, FFN, head. */
typedef struct esp_cuda_timings {
    float qkv_ms, attention_ms, ffn_ms, head_ms, total_ms;
    int32_t kernel_launches; /* kernels of this library launched by the most recent step or decode loop */
} esp_cuda_timings;

/* ---- lifetime (replaces ane_interop_compile / ane_interop_free, ane_interop.h:24-35) ------------ */

/* Creates an engine.  weight_dir != NULL: loads every tensor from a weight directory in the
 * reference layout (BLOBFILE fp16 files; a "<name>.float32.bin" sidecar of exactly the tensor's element
 * count wins over "<name>.bin" as in Engine.swift:7830-7879 -- norm gains and biases keep its fp32
 * values, matrices and embeddings are rounded to the fp16 the device computes in; a sidecar of another
 * size is ESP_CUDA_ERR_INVALID_WEIGHTS;
 * layout: Sources/ModelSupport/LayerWeightPaths.swift:22-77, Engine.swift:2066-2154) and finalises.
 * weight_dir == NULL: the caller uploads tensors with esp_cuda_load_tensor and then calls
 * esp_cuda_finalize. */
ESP_CUDA_API int32_t esp_cuda_create(const esp_cuda_config* config, const char* weight_dir, esp_cuda_engine** out);

/* Reads <weight_dir>/metadata.json (schema of Sources/ESPCompiler/ESPModelConfigIO.swift:12-59), then
 * behaves like esp_cuda_create(config, weight_dir). */
ESP_CUDA_API int32_t esp_cuda_create_from_directory(const char* weight_dir, int32_t max_batch, int32_t device,
                                                   uint32_t flags, esp_cuda_engine** out);

/* ---- GGUF front end (replaces GGUFModelLoader.prepare, Sources/EspressoGGUF/GGUFModelLoader.swift:273-405; the
 * parser itself lives in the reference's un-vendored Edgerunner package) -------------------------------------- */

/* Parses a .gguf file (versions 2 and 3) on the host: fills the model shape the reference derives from the metadata
 * (GGUFModelLoader.swift:297-326: <arch>.block_count, attention.head_count[_kv], embedding_length,
 * feed_forward_length, context_length, attention.layer_norm[_rms]_epsilon, rope.freq_base (default 10000), vocab =
 * length of tokenizer.ggml.tokens, eos = tokenizer.ggml.eos_token_id), the architecture name, the tensor count and
 * whether the LM head is tied to the embedding (no "output.weight", :224-263).  Needs no GPU. */
ESP_CUDA_API int32_t esp_cuda_gguf_inspect(const char* path, esp_cuda_config* config, char* architecture_name, int32_t name_capacity,
                                           int32_t* n_tensors, int32_t* tied_lm_head);

/* One entry of the tensor directory: GGUF name, the weight-directory path it maps to ("" = not read by the decode
 * path; "layers/N/wqkv" = GPT-2's fused projection, split at upload), GGML type, dims (dims[0] = row length), offset
 * inside the data section and byte size (0 for GGML types that cannot be uploaded).  Needs no GPU. */
ESP_CUDA_API int32_t esp_cuda_gguf_tensor_info(const char* path, int32_t index, char* name, int32_t name_capacity, char* slot,
                                               int32_t slot_capacity, int32_t* ggml_type, int64_t* dims4, uint64_t* data_offset,
                                               uint64_t* nbytes);

/* Builds and finalises an engine from a .gguf file: F32/F16/BF16 tensors as they are, Q8_0/Q4_0 matrices as
 * quantised blocks (no fp16 materialisation, unlike GGUFModelLoader.swift:341-369), quantised embedding tables
 * expanded to fp16, Wq/Wk rows of llama/mistral files put back from llama.cpp's per-head interleave into the
 * half-split rotation order, a missing output.weight replaced by the embedding matrix. */
ESP_CUDA_API int32_t esp_cuda_create_from_gguf(const char* path, int32_t max_batch, int32_t device, uint32_t flags,
                                               esp_cuda_engine** out);

/* Uploads one tensor.  name is the weight-directory relative path without ".bin"
 * ("embeddings/token", "rms_final", "lm_head", "layers/3/wq", ...).  data may be a host or a device
 * pointer.  Matrices are row-major [out, in].  F16/BF16/F32 take raw elements; Q8_0/Q4_0 take GGUF
 * blocks in file order and are valid for the layer matrices and lm_head only.  This is the GGUF
 * upload path that replaces the reference's dequantise-to-fp16 conversion
 * (Sources/EspressoGGUF/GGUFModelLoader.swift:341-369): quantised blocks stay quantised on the device. */
ESP_CUDA_API int32_t esp_cuda_load_tensor(esp_cuda_engine* engine, const char* name, int32_t type, const void* data,
                                          uint64_t nbytes);

/* Tensor parallelism (no counterpart in the reference, which is single-device): one engine per GPU and process,
 * created with the GLOBAL model shape and tp_rank / tp_size in the config.  Rank r then expects its Megatron
 * shard from esp_cuda_load_tensor: rows [r*n/G, (r+1)*n/G) of wq, wk, wv, w1, w3, lm_head (n = that matrix's row
 * count), the matching COLUMNS of wo and w2 (stored row-major [d_model, n/G]), and full copies of the embedding
 * and the norm gains.  An all-reduce follows the Wo and W2 products (over IPC-mapped peer memory with this library's
 * own kernel; NCCL when a peer cannot be mapped or ESP_CUDA_TP_NCCL_ONLY is set), and the vocabulary-sharded argmax
 * is merged with an NCCL max-reduce.  esp_cuda_tp_unique_id (rank 0; share the 128 bytes with the other ranks) and
 * esp_cuda_tp_init (every rank; collective) must run before esp_cuda_finalize.  Every rank must then make the same
 * sequence of decode calls. */
ESP_CUDA_API int32_t esp_cuda_tp_unique_id(uint8_t* out, int32_t capacity);
ESP_CUDA_API int32_t esp_cuda_tp_init(esp_cuda_engine* engine, const uint8_t* unique_id, int32_t nbytes);
/* Diagnostics of the peer-memory all-reduce on this rank since the previous call: out3 = {all-reduces, device ns from
 * this rank's arrival to its last sum, device ns of that spent waiting for the peers' arrivals}; zeros under NCCL. */
ESP_CUDA_API int32_t esp_cuda_tp_sum_stats(esp_cuda_engine* engine, uint64_t* out3);

/* Checks that every required tensor is present and prepares the decode state. */
ESP_CUDA_API int32_t esp_cuda_finalize(esp_cuda_engine* engine);
ESP_CUDA_API int32_t esp_cuda_destroy(esp_cuda_engine* engine);
ESP_CUDA_API int32_t esp_cuda_get_config(const esp_cuda_engine* engine, esp_cuda_config* out);

/* ---- single-sequence decoder (CPUExactLlamaRuntime, Engine.swift:548-850); acts on sequence 0 --- */

ESP_CUDA_API int32_t esp_cuda_reset(esp_cuda_engine* engine);                                   /* reset() :613-635 */
ESP_CUDA_API int32_t esp_cuda_prefill(esp_cuda_engine* engine, const uint32_t* tokens, int32_t n); /* prefill :637-645 */
ESP_CUDA_API int32_t esp_cuda_advance(esp_cuda_engine* engine, uint32_t token);                 /* advance :672-680 */
ESP_CUDA_API int32_t esp_cuda_select_greedy(esp_cuda_engine* engine, uint32_t* token);          /* selectGreedyToken :663-670 */
/* advance(token) followed by selectGreedyToken() as one device submission. */
ESP_CUDA_API int32_t esp_cuda_decode_step(esp_cuda_engine* engine, uint32_t token, uint32_t* next_token);
ESP_CUDA_API int32_t esp_cuda_visible_token_count(const esp_cuda_engine* engine, int32_t seq, int32_t* count);
/* Full fp32 logits of sequence `seq` for its current state (projectLogits, Engine.swift:8154-8180). */
ESP_CUDA_API int32_t esp_cuda_get_logits(esp_cuda_engine* engine, int32_t seq, float* out, int32_t vocab);
/* captureCheckpoint / rollback (:647-661).  A checkpoint records (visible token count, last hidden);
 * KV slots beyond the count are overwritten by later steps, so no cache copy is needed. */
ESP_CUDA_API int32_t esp_cuda_checkpoint(esp_cuda_engine* engine, int32_t* checkpoint_id);
ESP_CUDA_API int32_t esp_cuda_rollback(esp_cuda_engine* engine, int32_t checkpoint_id);

/* Exact two-token verify (ANEExactTwoTokenBranchStatePromotionModel.performExactTwoTokenPass,
 * Sources/Espresso/GenerationHarness.swift:1281-1344): one forward over the two positions
 * [current, proposed_future]; returns the target's greedy token after each.  Nothing is committed
 * until esp_cuda_commit(engine, 1 or 2) (promotePreparedPair). */
ESP_CUDA_API int32_t esp_cuda_verify2(esp_cuda_engine* engine, uint32_t current, uint32_t proposed_future,
                                      uint32_t* exact_next, uint32_t* exact_future);
ESP_CUDA_API int32_t esp_cuda_commit(esp_cuda_engine* engine, int32_t steps);

/* ---- batched decoder: max_batch independent copies of the decoder above (no cross-sequence math) -- */

/* tokens is [n_seq][len] row-major; resets sequences 0..n_seq-1 and feeds len tokens to each. */
ESP_CUDA_API int32_t esp_cuda_prefill_batch(esp_cuda_engine* engine, const uint32_t* tokens, int32_t n_seq, int32_t len);
/* Feeds tokens[s] to sequence s and returns each sequence's next greedy token. */
ESP_CUDA_API int32_t esp_cuda_decode_step_batch(esp_cuda_engine* engine, const uint32_t* tokens, int32_t n_seq,
                                                uint32_t* next_tokens);

/* Greedy decode of up to `count` tokens for sequences 0..n_seq-1, continuing from their current state
 * (ESPRuntimeSession.decode(count:), Sources/ESPRuntime/ESPRuntimeContracts.swift:5-13).  The loop runs on
 * the device: each step's selected token is fed to the next step without a host round trip.  out_tokens is
 * [n_seq][count] (may be NULL), n_out[n_seq] (may be NULL); *device_ms (may be NULL) receives the device time
 * of the whole loop measured with CUDA events on the engine's stream.  The last emitted token of a sequence
 * has been selected but not yet fed. */
ESP_CUDA_API int32_t esp_cuda_decode(esp_cuda_engine* engine, int32_t n_seq, int32_t count, uint32_t* out_tokens,
                                     int32_t* n_out, float* device_ms);

/* ---- generation loops (token ids in, token ids out: generate*ForTesting, Engine.swift:1681-1876) - */

/* Greedy generation (generateIncrementalExactCPULlama, Engine.swift:6192-6431).  prompt must hold
 * 1..maxSeq-1 tokens; at most min(max_tokens, maxSeq - n_prompt) tokens are produced.  Llama: an EOS
 * token is emitted and then generation stops; GPT-2: token 50256 stops without being emitted.
 * out_tokens must have room for max_tokens entries. */
ESP_CUDA_API int32_t esp_cuda_generate(esp_cuda_engine* engine, const uint32_t* prompt, int32_t n_prompt,
                                       int32_t max_tokens, uint32_t* out_tokens, int32_t* n_out,
                                       esp_cuda_generation_result* result);
/* n_seq prompts of equal length, [n_seq][n_prompt]; out_tokens is [n_seq][max_tokens], n_out[n_seq]. */
ESP_CUDA_API int32_t esp_cuda_generate_batch(esp_cuda_engine* engine, const uint32_t* prompts, int32_t n_seq,
                                             int32_t n_prompt, int32_t max_tokens, uint32_t* out_tokens,
                                             int32_t* n_out, esp_cuda_generation_result* result);
/* The same generation, token by token, with `on_step(user, token, index, latency_ms)` called inline on the caller's
 * thread as each token becomes known: the reference's onStep callback (Engine.swift:6393-6405, GenerationStep
 * :57-83).  on_step may be NULL.  One host round trip per token, like the reference's loop. */
typedef void (*esp_cuda_step_callback)(void* user, uint32_t token, int32_t index, double latency_ms);
ESP_CUDA_API int32_t esp_cuda_generate_steps(esp_cuda_engine* engine, const uint32_t* prompt, int32_t n_prompt,
                                             int32_t max_tokens, esp_cuda_step_callback on_step, void* user,
                                             uint32_t* out_tokens, int32_t* n_out, esp_cuda_generation_result* result);
/* GenerationResult.tokenLatenciesMs (Engine.swift:17-55; the CLI's median / p95, Sources/EspressoGenerate/CLI.swift:
 * 1153-1165, 1283-1284) of sequence 0 for the most recent esp_cuda_generate / esp_cuda_generate_steps /
 * esp_cuda_decode: milliseconds between consecutive tokens (the first entry counts from the start of decoding).
 * Device timers inside the persistent kernel, CUDA events between the steps of the other kernels, the host clock for
 * esp_cuda_generate_steps. */
ESP_CUDA_API int32_t esp_cuda_token_latencies(esp_cuda_engine* engine, float* out_ms, int32_t capacity, int32_t* n);
/* Exact two-token speculative generation with a draft engine (Engine.swift:6014-6190); the emitted
 * stream equals plain greedy decoding of `engine`. */
ESP_CUDA_API int32_t esp_cuda_generate_two_token(esp_cuda_engine* engine, esp_cuda_engine* draft,
                                                 const uint32_t* prompt, int32_t n_prompt, int32_t max_tokens,
                                                 uint32_t* out_tokens, int32_t* n_out,
                                                 esp_cuda_generation_result* result);

/* ---- diagnostics ---------------------------------------------------------------------------------- */

ESP_CUDA_API int32_t esp_cuda_get_timings(esp_cuda_engine* engine, esp_cuda_timings* out);
/* Per-stage values of the most recent advance on sequence 0, for bisecting a mismatch by layer and stage
 * like the reference's testing dumps (Engine.swift:419-484).  stage: 0 q (post-RoPE), 1 k (post-RoPE, as
 * stored), 2 v (as stored), 3 attention context, 4 hidden after attention, 5 FFN activation, 6 layer
 * output.  Stages 0..5 are captured for `layer` only when esp_cuda_set_debug_layer(engine, layer) was called
 * before the step. */
/* SM clock stamps taken by one CTA of the persistent decode kernel during the last token of the most recent
 * decode loop (the fine-grained counterpart of the per-layer DecodeKernelProfile, DecodeForwardPass.swift:212-320).
 * Per layer 14 stamps: S1 begin, norm done, weights arrived, rows done, barrier passed; S2 weights arrived, done,
 * barrier passed; S3 norm done, weights arrived, gate/up done, weights arrived, down done, barrier passed; then
 * 4 for the head: begin, norm done, rows done, barrier passed.  *n = 0 when the model does not use that kernel.
 * `cta` selects which CTA records the NEXT loop. */
ESP_CUDA_API int32_t esp_cuda_stage_trace(esp_cuda_engine* engine, int32_t cta, int64_t* out, int32_t capacity, int32_t* n);
/* Emission time (GPU global timer, nanoseconds) of every token of the most recent decode loop that ran as the
 * persistent kernel; consecutive differences are the per-token latencies the reference's CLI summarises as median
 * and p95 (Sources/EspressoGenerate/CLI.swift:1153-1165, 1283-1284).  *n = 0 when that loop used other kernels. */
ESP_CUDA_API int32_t esp_cuda_token_times(esp_cuda_engine* engine, uint64_t* out_ns, int32_t capacity, int32_t* n);
ESP_CUDA_API int32_t esp_cuda_set_debug_layer(esp_cuda_engine* engine, int32_t layer);
ESP_CUDA_API int32_t esp_cuda_debug_dump(esp_cuda_engine* engine, int32_t stage, float* out, int32_t capacity);
ESP_CUDA_API const char* esp_cuda_last_error_string(void);
/* Test hooks with the meaning of ane_interop_set_force_eval_failure / ane_interop_live_handle_count
 * (ane_interop.h:37-41): while forced, every device submission returns ESP_CUDA_ERR_FORCED_FAILURE. */
ESP_CUDA_API void esp_cuda_set_force_failure(int32_t enabled);
/* Test hook for the failure path of the device-side waits (the reference has no device waits; its analogue is the
 * forced evaluation failure, ane_interop.m:2336-2338).  Every wait inside the persistent decode kernel polls at most
 * `spins` times (0 restores the default of about two million); a wait that runs out makes the kernel stop waiting
 * everywhere, finish, and the call return ESP_CUDA_ERR_TIMEOUT.  Nothing faults or hangs; the engine stays usable
 * after esp_cuda_reset once the limit is restored. */
ESP_CUDA_API int32_t esp_cuda_set_wait_limit(esp_cuda_engine* engine, uint32_t spins);
ESP_CUDA_API int32_t esp_cuda_live_engine_count(void);
ESP_CUDA_API const char* esp_cuda_version(void);

/* ---- stand-alone kernels (parity checks and kernel-level bandwidth measurement) ------------------- */

/* Dequantises GGUF blocks on the device: out[i] = fp32(d) * q, bit-exact.  blocks/out are host pointers. */
ESP_CUDA_API int32_t esp_cuda_dequantize(int32_t type, const void* blocks, int64_t n_elements, float* out, int32_t device);
/* y = W . x for one weight matrix of any storage type, timed on the device.  W is uploaded once,
 * the kernel runs `iterations` times after `warmup` runs; *avg_ms receives the mean kernel time. */
ESP_CUDA_API int32_t esp_cuda_gemv_bench(int32_t type, const void* weights, int32_t rows, int32_t cols, const float* x,
                                         float* y, int32_t warmup, int32_t iterations, int32_t copies, float* avg_ms,
                                         int32_t device);

/* Y[n][m] = sum_k W[m][k] * X[n][k] on the tensor cores (tcgen05 / TMEM): W [rows, cols] fp16 or bf16 row-major,
 * X [n, cols] fp32 (rounded to W's type on the device), Y [n, rows] fp32; 1 <= n <= 256, cols a multiple of 64.
 * This is the batched counterpart of esp_cuda_gemv_bench (the reference multiplies one vector at a time with
 * vDSP_mmul, Engine.swift:6674-6718, and uses cblas_sgemm for sequence verify, GenerationHarness.swift:2745-2761).
 * All pointers are host pointers; *avg_ms receives the mean kernel time. */
ESP_CUDA_API int32_t esp_cuda_gemm_tc_bench(int32_t type, const void* weights, int32_t rows, int32_t cols, const float* x,
                                            int32_t n, float* y, int32_t warmup, int32_t iterations, float* avg_ms,
                                            int32_t device);

/* ---- an entry point that allocates nothing --------------------------------------------------------- */

/* No counterpart in the reference.  Final RMSNorm (skipped when d_norm_gain is NULL) + fp16 LM head +
 * first-max greedy argmax for `rows` hidden vectors, for hosts that may not call the CUDA allocator while they
 * run: processes whose device-memory budget was fixed up front, plugins living in another framework's arena,
 * and latency-critical loops in which a cudaMalloc/cudaFree would stall the whole device.  Every pointer is a
 * DEVICE pointer owned by the caller: d_lm_head_f16 [vocab][d_model] fp16 row-major, d_hidden [rows][d_model]
 * fp32, d_norm_gain [d_model] fp32 or NULL, d_tokens [rows] uint32 (output).  The kernel's own working memory
 * (packed running maxima, completion counter, per-row control words) is a 4 KiB array compiled into the library,
 * which every GPU that loads the library holds until exit.  Limits: rows <= ESP_CUDA_STATIC_HEAD_MAX_ROWS,
 * d_model a multiple of 8 and <= 8192; anything larger is refused with ESP_CUDA_ERR_INVALID_ARGUMENT.  The work
 * is enqueued on `cuda_stream` (a cudaStream_t, NULL = default stream) and is complete when that stream reaches
 * this point.  All calls on a device share the array and it keeps the previous call's contents: the call resets
 * what it needs, and calls whose kernels overlap on the GPU race - serialise them.  The first call on a device
 * looks up the array's address and should be made before any stream capture begins.  The call itself performs
 * no cudaMalloc, cudaFree or other allocating routine.  d_lm_head_f16 must be 16-byte aligned and the other pointers
 * 4-byte aligned (a view that starts elsewhere is refused with ESP_CUDA_ERR_INVALID_ARGUMENT); the call runs on
 * `device` and leaves the caller's current device unchanged. */
#define ESP_CUDA_STATIC_HEAD_MAX_ROWS 64
ESP_CUDA_API int32_t esp_cuda_lm_head_argmax_static(const void* d_lm_head_f16, int32_t vocab, int32_t d_model,
                                                    const float* d_hidden, int32_t rows, const float* d_norm_gain,
                                                    float norm_eps, uint32_t* d_tokens, void* cuda_stream, int32_t device);

#ifdef __cplusplus
}
#endif
#endif /* ESPRESSO_CUDA_H */
