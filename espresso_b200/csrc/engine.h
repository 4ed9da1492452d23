// Host-side engine: owns the device copy of one model replica, the KV cache and the per-row decode
// state, and submits the decode kernels.  It is the CUDA counterpart of the reference's
// CPUExactLlamaRuntime (Sources/RealModelInference/RealModelInferenceEngine.swift:548-850) generalised to
// `max_batch` independent sequences and to GPT-2.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <map>
#include <string>
#include <vector>

#include "../../include/espresso_cuda.h"
#include "decode_kernels.cuh"
#include "mega_kernel.cuh"

namespace esp {

void set_last_error(const std::string& msg);
const char* last_error_cstr();
bool force_failure_enabled();

struct DeviceTensor {
    void* data = nullptr;       // matrix payload (see esp::Weight) or raw 16-bit elements (embeddings)
    __half* scales = nullptr;   // Q8_0 / Q4_0 scales
    float* f32 = nullptr;       // fp32 copy (norm gains, biases)
    int type = -1;
    int rows = 0, cols = 0;
    bool loaded = false;
    CUtensorMap map{};          // TMA map of a 16-bit matrix for the tensor-core path (128-row boxes)
    bool has_map = false;
    __half* shadow16 = nullptr; // fp16 expansion of a quantised matrix: what the tensor-core path multiplies by
};

struct Checkpoint {
    int visible = 0;
    float* hidden = nullptr;  // device copy of the last hidden state of sequence 0
};

class Engine {
public:
    explicit Engine(const esp_cuda_config& cfg);
    ~Engine();


    int32_t init();  // device buffers
    int32_t load_tensor(const char* name, int32_t type, const void* data, uint64_t nbytes);
    int32_t load_directory(const char* dir);
    int32_t finalize();
    int32_t tp_init(const uint8_t* unique_id, int32_t nbytes);  // tensor parallel: joins the NCCL communicator (collective call)

    int32_t reset();
    int32_t prefill(const uint32_t* tokens, int32_t n);
    int32_t advance(uint32_t token);
    int32_t select_greedy(uint32_t* token);
    int32_t decode_step(uint32_t token, uint32_t* next);
    int32_t get_logits(int32_t seq, float* out, int32_t vocab);
    int32_t checkpoint(int32_t* id);
    int32_t rollback(int32_t id);
    int32_t verify2(uint32_t current, uint32_t proposed, uint32_t* exact_next, uint32_t* exact_future);
    int32_t commit(int32_t steps);
    int32_t prefill_batch(const uint32_t* tokens, int32_t n_seq, int32_t len);
    int32_t decode_step_batch(const uint32_t* tokens, int32_t n_seq, uint32_t* next);
    // Feeds tok[r] to sequence seq[r] for every row (rows sharing a sequence take consecutive positions) and
    // optionally returns each row's next greedy token.
    int32_t feed(int rows, const int* seq, const uint32_t* tok, bool with_head, uint32_t* next_out);
    int32_t generate_batch(const uint32_t* prompts, int32_t n_seq, int32_t n_prompt, int32_t max_tokens,
                           uint32_t* out_tokens, int32_t* n_out, esp_cuda_generation_result* result);
    int32_t decode_loop(int32_t n_seq, int32_t count, uint32_t* out_tokens, int32_t out_stride, int32_t* n_out,
                        float* device_ms, double* first_token_ms);
    int32_t stage_trace(int32_t cta, long long* out, int32_t capacity, int32_t* n);
    int32_t token_times(unsigned long long* out_ns, int32_t capacity, int32_t* n);
    int32_t token_latencies(float* out_ms, int32_t capacity, int32_t* n);
    void set_token_latencies(const std::vector<float>& v) { latencies_ms_ = v; }
    int32_t set_debug_layer(int32_t layer);
    int32_t debug_dump(int32_t stage, float* out, int32_t capacity);
    int32_t get_timings(esp_cuda_timings* out);
    int32_t set_wait_limit(uint32_t spins);
    int32_t tp_sum_stats(unsigned long long* out3);
    // Exact two-token generation as one device-driven launch (spec_kernel.cuh).  `draft` must pass spec_compatible().
    // out_tokens[0 .. gen0) are already emitted (`current` is the newest of them, `prev` the token before it); the call
    // appends up to eff - gen0 more and fills stats[0..4] = tokens in total, passes, committed, accepted, stopped on EOS.
    bool spec_compatible(const Engine& draft) const;
    int32_t run_spec(Engine& draft, uint32_t prev, uint32_t current, int gen0, int eff, int max_seq, uint32_t* out_tokens, int* stats);

    const esp_cuda_config& config() const { return cfg_; }
    int visible(int seq) const { return h_visible_[seq]; }
    bool finalized() const { return finalized_; }

private:
    enum StepMode { STEP_FORWARD = 1, STEP_HEAD = 2, STEP_FEEDBACK = 4, STEP_TILED_ATT = 8 };  // TILED_ATT: prompt pass, tiled attention
    struct RowsHost {  // pinned mirror of the device row-control block
        int* base = nullptr;
    };

    int32_t check_ready(const char* what) const;
    DeviceTensor* slot(const std::string& name, int* rows, int* cols, bool* is_matrix, bool* is_embedding);
    int32_t load_file_tensor(const std::string& dir, const std::string& name);  // sidecar-first file loader; 1 = no such file
    int32_t upload_rows(int rows, const int* seq, const int* pos, const uint32_t* tok, const int* active,
                        const int* limit, bool zero_out_counts);
    int32_t submit(int rows, int mode);                  // graph replay or direct launch
    int32_t launch_step(int rows, int mode, cudaStream_t s, bool profile);
    int32_t launch_step_tc(int rows, int mode, cudaStream_t s);  // batched path: tensor-core GEMMs + element-wise stages
    int32_t build_tc();
    int32_t tc_operands();  // weight maps (and a quantised model's fp16 expansion), built on first use of the batched path
    int32_t all_reduce(const void* send, void* recv, size_t count, bool sum_f32, cudaStream_t s);
    const CUtensorMap* activation_map(const uint16_t* buf, int K, int tile);
    int32_t feed_rows(int rows, const int* seq, const uint32_t* tok, bool with_head, uint32_t* next_out);
    Weight weight_of(const DeviceTensor& t) const;
    LayerWeights layer_weights(int l) const;
    size_t gemv_smem(int type, int K, bool with_tmp) const;
    int32_t build_mega();   // packs the weights for the persistent decode kernel when the model qualifies
    int32_t run_mega(int n_steps, int* emitted, float* device_ms, double* first_token_ms);
    int32_t ensure_norms2();  // the gain vectors twice over, as the two-position kernel reads them
    int32_t spec_prepare();   // plan, arena and result block of the two-position kernel
    bool spec_verify_ok() const;  // verify2 can run as one launch of the two-position kernel
    int32_t run_spec_verify(uint32_t current, uint32_t proposed, uint32_t* exact_next, uint32_t* exact_future);

    esp_cuda_config cfg_;
    ModelDims m_{};
    cudaStream_t stream_ = nullptr;
    bool finalized_ = false;
    bool qk_norm_ = false;  // every layer has per-head q_norm / k_norm weights (Qwen3)
    int max_rows_ = 0;
    int n_splits_ = 1;
    int sm_count_ = 148;

    std::map<std::string, DeviceTensor> tensors_;
    std::vector<void*> owned_;  // every cudaMalloc'd pointer

    // device state
    Activations act_{};
    KvLayout kv_{};
    RowState rs_{};
    int* d_rows_block_ = nullptr;  // [6][max_rows] seq,pos,tok,active,n_out,limit
    int* h_rows_block_ = nullptr;  // pinned
    uint32_t* h_next_ = nullptr;   // pinned [max_rows]
    float2* d_rope_ = nullptr;
    float* d_debug_ = nullptr;
    int debug_layer_ = -1;
    int out_stride_ = 0;

    std::vector<int> h_visible_;   // per sequence
    std::vector<Checkpoint> checkpoints_;
    int pending_verify_ = 0;

    std::map<int, cudaGraphExec_t> graphs_;  // key = rows * 8 + mode
    std::map<int, int> launches_by_key_;
    std::vector<cudaEvent_t> prof_events_;
    cudaEvent_t ev_begin_ = nullptr, ev_end_ = nullptr;

    // tensor parallelism (Megatron column/row split, NCCL all-reduce after Wo and W2, max-reduce of the packed argmax)
    int tp_rank_ = 0, tp_size_ = 1;
    int vocab_global_ = 0;
    void* nccl_comm_ = nullptr;
    float* tp_partial_ = nullptr;  // [max_rows][d_model] partial projection before the all-reduce (NCCL path)
    // Peer-memory all-reduce: every rank maps every other rank's exchange block (two partial buffers + arrival flags)
    int32_t tp_peer_setup();
    int32_t tp_sum_peers(float* out, int rows, cudaStream_t s);  // out = sum over ranks of the current partial buffer
    float* tp_current_partial() const;  // where this rank's partial of the next all-reduce goes
    bool tp_peer_ready_ = false;
    uint8_t* tp_block_ = nullptr;               // this rank's exchange block (cudaMalloc, exported with cudaIpc)
    uint8_t* tp_peer_block_[8] = {};            // mapped exchange blocks, index = rank (own block at own index)
    size_t tp_buf_floats_ = 0;                  // floats per partial buffer
    unsigned int* tp_epoch_ = nullptr;          // [2] local: completed all-reduces, CTA ticket
    unsigned long long* tp_stats_ = nullptr;    // [4] local: count and device time of the peer-memory all-reduces
    int tp_parity_ = 0;                         // partial buffer of the next all-reduce (host side, fixed at graph capture)

    // batched tensor-core path (rows >= kTcMinRows, 16-bit weights)
    bool tc_ready_ = false;
    bool tc_operands_ready_ = false;
    std::vector<std::string> tc_mats_;
    int tc_bf16_ = 0;
    int tc_rows_alloc_ = 0;
    uint16_t *xh_d_ = nullptr, *xh_q_ = nullptr, *xh_h_ = nullptr;  // 16-bit operand rows [tc_rows_alloc_][K]
    float *kraw_ = nullptr, *vraw_ = nullptr, *up_ = nullptr;
    float* d_last_hidden_ = nullptr;  // [max_batch][d_model] last hidden state per sequence while a batch of prompts is fed
    int* d_tc_error_ = nullptr;
    std::map<std::pair<const void*, int>, CUtensorMap> act_maps_;

    // persistent decode kernel (single sequence, Llama fp16 models whose per-layer slice fits in shared memory)
    bool mega_ready_ = false;
    MegaPlan mega_plan_{};
    uint8_t* d_pack_ = nullptr;
    float* d_norms_ = nullptr;
    unsigned long long* d_mega_arena_ = nullptr;  // exchange words and counted sums of the persistent kernel (zeroed per launch)
    size_t mega_arena_words_ = 0;
    unsigned mega_spin_limit_ = kMegaSpinLimit;   // attempts per device-side wait (test hook: set_wait_limit)
    unsigned long long* d_mega_ctl_ = nullptr;  // [2] error (i32 in the upper half), [3..4] time stamps, [5] tokens emitted
    unsigned long long* h_mega_ctl_ = nullptr;  // pinned mirror
    long long* d_mega_trace_ = nullptr;
    unsigned long long* d_token_times_ = nullptr;  // [max_seq] emission time of every token of the last persistent loop
    int token_times_n_ = 0;
    std::vector<float> latencies_ms_;              // per-token latencies of sequence 0, most recent generation
    std::vector<cudaEvent_t> step_events_;         // one per step of a decode loop of the per-stage kernels
    int mega_trace_cta_ = 0;
    // two-token kernel (built on first use)
    bool spec_ready_ = false;
    MegaPlan spec_plan_{};
    float* d_norms2_ = nullptr;
    unsigned long long* d_spec_arena_ = nullptr;
    size_t spec_arena_words_ = 0;
    uint32_t* d_spec_out_ = nullptr;   // [max_seq + 1] emitted tokens
    int* d_spec_result_ = nullptr;     // [16]: results [0..7], error word [8]
    esp_cuda_timings timings_{};
    int launches_last_step_ = 0;
};

}  // namespace esp
