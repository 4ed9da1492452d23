// Engine implementation: device memory, weight upload (BLOBFILE directories and raw/GGUF tensors),
// kernel submission (direct or CUDA-graph replay, programmatic dependent launch between stages).
#include "engine.h"
#include "batch_kernels.cuh"
#include "tc_gemm.cuh"
#include "spec_kernel.cuh"
#include "prefill_attention.cuh"

#include <dlfcn.h>
#include <nccl.h>
#include <sys/stat.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <mutex>
#include <sstream>

namespace esp {

// ---------------------------------------------------------------------------------------------- errors

static thread_local std::string g_last_error;
static std::atomic<int> g_force_failure{0};

void set_last_error(const std::string& msg) { g_last_error = msg; }
const char* last_error_cstr() { return g_last_error.c_str(); }
bool force_failure_enabled() { return g_force_failure.load() != 0; }
void set_force_failure(int on) { g_force_failure.store(on ? 1 : 0); }

#define ESP_CUDA_TRY(expr)                                                                              \
    do {                                                                                                \
        cudaError_t _e = (expr);                                                                        \
        if (_e != cudaSuccess) {                                                                        \
            set_last_error(std::string(#expr) + ": " + cudaGetErrorString(_e));                         \
            return _e == cudaErrorMemoryAllocation ? ESP_CUDA_ERR_OUT_OF_MEMORY : ESP_CUDA_ERR_CUDA;    \
        }                                                                                               \
    } while (0)

static int32_t fail(int32_t code, const std::string& msg) {
    set_last_error(msg);
    return code;
}

int32_t tc_make_map(CUtensorMap* map, const void* base, bool bf16, uint64_t rows, uint64_t cols, uint32_t box_rows);
int tc_tile_for(int rows);
TcPlan tc_plan(int w_tiles, int rows, int kb, bool may_split_k, bool dual, int sms);
cudaError_t tc_launch(const TcPlan& plan, bool dual, const CUtensorMap* const* mw, const CUtensorMap& mx, TcArgs a, cudaStream_t s);
constexpr int kTcMinRows = 9;  // below this the row-batched GEMV stages are used
constexpr int kPrefillRows = 512;  // rows of a prefill pass on the batched path: every pass streams all the weights once

// ---------------------------------------------------------------------------------------------- kernels

template <int WT>
__global__ void __launch_bounds__(kThreads) k_qkv(const QkvArgs p) {
    extern __shared__ float smem[];
    // Before the previous stage has finished: pull this CTA's weight rows towards L2.
    {
        const int n_items = (p.m.q_dim + 2 * p.m.kv_dim) / 2;
        int begin, end;
        cta_range(n_items, blockIdx.x, gridDim.x, begin, end);
        const int half = p.m.head_dim / 2, q_items = p.m.q_dim / 2, k_items = p.m.kv_dim / 2;
        for (int item = begin + threadIdx.x; item < end; item += kThreads) {
            const Weight* W;
            int local, row0, row1;
            if (item < q_items) { W = &p.lw.wq; local = item; }
            else if (item < q_items + k_items) { W = &p.lw.wk; local = item - q_items; }
            else { W = &p.lw.wv; local = item - q_items - k_items; }
            if (item < q_items + k_items) { int h = local / half; row0 = h * p.m.head_dim + (local - h * half); row1 = row0 + half; }
            else { row0 = 2 * local; row1 = row0 + 1; }
            unsigned rb = (unsigned)weight_row_bytes(W->type, W->cols);
            l2_prefetch(weight_row(*W, row0), rb);
            l2_prefetch(weight_row(*W, row1), rb);
        }
    }
    stage_qkv<WT>(p, blockIdx.x, gridDim.x, smem + kRedFloats, smem);  // signals and waits for its neighbours inside
}

__global__ void __launch_bounds__(kAttThreads) k_attention(const AttArgs p) {
    __shared__ float sm[128 + kAttSplitTokens + 8 + (kAttThreads / 32) * 128];  // q, scores, reduction scratch, per-warp ctx
    pdl_launch_dependents();
    pdl_wait();
    stage_attention(p, blockIdx.y, blockIdx.x, blockIdx.z, sm);
}

template <int WT, int EPI>
__global__ void __launch_bounds__(kThreads) k_gemv(const GemvArgs p) {
    extern __shared__ float smem[];
    {
        const int n_items = EPI == EPI_SWIGLU ? p.w.rows : (p.w.rows + 1) / 2;
        int begin, end;
        cta_range(n_items, blockIdx.x, gridDim.x, begin, end);
        if (end > begin && threadIdx.x == 0) {
            // a CTA's rows are contiguous: bulk prefetches of at most 32 KiB each
            const size_t rb = weight_row_bytes(p.w.type, p.w.cols);
            const int r0 = EPI == EPI_SWIGLU ? begin : begin * 2;
            const int r1 = min(EPI == EPI_SWIGLU ? end : end * 2, p.w.rows);
            size_t bytes = (size_t)(r1 - r0) * rb;
            const uint8_t* b0 = weight_row(p.w, r0);
            const uint8_t* b1 = EPI == EPI_SWIGLU ? weight_row(p.w_up, r0) : nullptr;
            for (size_t off = 0; off < bytes; off += (32u << 10)) {
                unsigned n = (unsigned)min((size_t)(32u << 10), bytes - off);
                l2_prefetch(b0 + off, n);
                if (b1) l2_prefetch(b1 + off, n);
            }
        }
    }
    stage_gemv<WT, EPI>(p, blockIdx.x, gridDim.x, smem + kRedFloats, smem);
}

// Final norm + LM head + greedy argmax (a k_gemv<WT, EPI_HEAD> under its own name, so that profiles list it apart).
template <int WT>
__global__ void __launch_bounds__(kThreads) k_lm_head(const GemvArgs p) {
    extern __shared__ float smem[];
    {
        const int n_items = (p.w.rows + 1) / 2;
        int begin, end;
        cta_range(n_items, blockIdx.x, gridDim.x, begin, end);
        if (end > begin && threadIdx.x == 0) {
            const size_t rb = weight_row_bytes(p.w.type, p.w.cols);
            const int r0 = begin * 2, r1 = min(end * 2, p.w.rows);
            size_t bytes = (size_t)(r1 - r0) * rb;
            const uint8_t* b0 = weight_row(p.w, r0);
            for (size_t off = 0; off < bytes; off += (32u << 10)) l2_prefetch(b0 + off, (unsigned)min((size_t)(32u << 10), bytes - off));
        }
    }
    stage_gemv<WT, EPI_HEAD>(p, blockIdx.x, gridDim.x, smem + kRedFloats, smem);
}

__global__ void k_bump(RowState rs, int rows) {
    pdl_launch_dependents();
    pdl_wait();
    bump_positions(rs, rows);
}

// GGUF blocks (array of structs, file order) -> the split layout of esp::Weight.
__global__ void k_repack_q8_0(const uint8_t* __restrict__ blocks, int64_t n_blocks, int8_t* q, __half* scales) {
    int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const uint8_t* s = blocks + b * 34;
    scales[b] = __ushort_as_half((unsigned short)(s[0] | (s[1] << 8)));
    for (int i = 0; i < 32; i++) q[b * 32 + i] = (int8_t)s[2 + i];
}
__global__ void k_repack_q4_0(const uint8_t* __restrict__ blocks, int64_t n_blocks, uint8_t* q, __half* scales) {
    int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const uint8_t* s = blocks + b * 18;
    scales[b] = __ushort_as_half((unsigned short)(s[0] | (s[1] << 8)));
    for (int i = 0; i < 16; i++) q[b * 16 + i] = s[2 + i];
}

// out[i] = fp32(d) * q  (bit-exact GGUF dequantisation; used by the parity entry point)
__global__ void k_dequant(const uint8_t* __restrict__ blocks, int type, int64_t n_blocks, float* out) {
    int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    if (type == WT_Q8_0) {
        const uint8_t* s = blocks + b * 34;
        float d = __half2float(__ushort_as_half((unsigned short)(s[0] | (s[1] << 8))));
        for (int i = 0; i < 32; i++) out[b * 32 + i] = __fmul_rn(d, (float)(int8_t)s[2 + i]);
    } else {
        const uint8_t* s = blocks + b * 18;
        float d = __half2float(__ushort_as_half((unsigned short)(s[0] | (s[1] << 8))));
        for (int i = 0; i < 16; i++) {
            out[b * 32 + i] = __fmul_rn(d, (float)((int)(s[2 + i] & 15) - 8));
            out[b * 32 + 16 + i] = __fmul_rn(d, (float)((int)(s[2 + i] >> 4) - 8));
        }
    }
}

__global__ void k_to_f32(const void* src, int type, int64_t n, float* dst) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (type == ESP_CUDA_F32) dst[i] = static_cast<const float*>(src)[i];
    else dst[i] = emb_to_float(static_cast<const uint16_t*>(src)[i], type == ESP_CUDA_BF16 ? WT_BF16 : WT_F16);
}
__global__ void k_f32_to_f16(const float* src, int64_t n, __half* dst) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = __float2half_rn(src[i]);
}

// Split-layout Q8_0 / Q4_0 matrix -> fp16(d * q): the operand of the tensor-core path for batches.
__global__ void k_expand_quant(const void* __restrict__ q, const __half* __restrict__ scales, int type, int64_t n_blocks, __half* out) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 8 elements
    const int64_t b = t >> 2;
    const int part = (int)(t & 3);
    if (b >= n_blocks) return;
    const float d = __half2float(scales[b]);
    __half o[8];
    if (type == WT_Q8_0) {
        const int8_t* s = static_cast<const int8_t*>(q) + b * 32 + part * 8;
#pragma unroll
        for (int i = 0; i < 8; i++) o[i] = __float2half_rn(d * (float)s[i]);
    } else {
        // elements 0..15 are the low nibbles of the block's 16 bytes, 16..31 the high nibbles
        const uint8_t* s = static_cast<const uint8_t*>(q) + b * 16 + (part & 1) * 8;
#pragma unroll
        for (int i = 0; i < 8; i++) o[i] = __float2half_rn(d * (float)((int)((part & 2) ? (s[i] >> 4) : (s[i] & 15)) - 8));
    }
    *reinterpret_cast<uint4*>(out + b * 32 + part * 8) = *reinterpret_cast<const uint4*>(o);
}

// ---------------------------------------------------------------------------------------------- launch helpers

template <typename Kern, typename... Args>
static cudaError_t launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t s, const Args&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

template <int EPI>
static cudaError_t launch_gemv_typed(int type, dim3 grid, size_t smem, cudaStream_t s, const GemvArgs& a) {
    switch (type) {
        case WT_F16: return launch_pdl(k_gemv<WT_F16, EPI>, grid, dim3(kThreads), smem, s, a);
        case WT_BF16: return launch_pdl(k_gemv<WT_BF16, EPI>, grid, dim3(kThreads), smem, s, a);
        case WT_Q8_0: return launch_pdl(k_gemv<WT_Q8_0, EPI>, grid, dim3(kThreads), smem, s, a);
        case WT_Q4_0: return launch_pdl(k_gemv<WT_Q4_0, EPI>, grid, dim3(kThreads), smem, s, a);
    }
    return cudaErrorInvalidValue;
}
static cudaError_t launch_gemv(int epi, int type, dim3 grid, size_t smem, cudaStream_t s, const GemvArgs& a) {
    switch (epi) {
        case EPI_RESIDUAL: return launch_gemv_typed<EPI_RESIDUAL>(type, grid, smem, s, a);
        case EPI_SWIGLU: return launch_gemv_typed<EPI_SWIGLU>(type, grid, smem, s, a);
        case EPI_GELU: return launch_gemv_typed<EPI_GELU>(type, grid, smem, s, a);
        case EPI_HEAD:
            switch (type) {
                case WT_F16: return launch_pdl(k_lm_head<WT_F16>, grid, dim3(kThreads), smem, s, a);
                case WT_BF16: return launch_pdl(k_lm_head<WT_BF16>, grid, dim3(kThreads), smem, s, a);
                case WT_Q8_0: return launch_pdl(k_lm_head<WT_Q8_0>, grid, dim3(kThreads), smem, s, a);
                case WT_Q4_0: return launch_pdl(k_lm_head<WT_Q4_0>, grid, dim3(kThreads), smem, s, a);
            }
            return cudaErrorInvalidValue;
    }
    return cudaErrorInvalidValue;
}
static cudaError_t launch_qkv(int type, dim3 grid, size_t smem, cudaStream_t s, const QkvArgs& a) {
    switch (type) {
        case WT_F16: return launch_pdl(k_qkv<WT_F16>, grid, dim3(kThreads), smem, s, a);
        case WT_BF16: return launch_pdl(k_qkv<WT_BF16>, grid, dim3(kThreads), smem, s, a);
        case WT_Q8_0: return launch_pdl(k_qkv<WT_Q8_0>, grid, dim3(kThreads), smem, s, a);
        case WT_Q4_0: return launch_pdl(k_qkv<WT_Q4_0>, grid, dim3(kThreads), smem, s, a);
    }
    return cudaErrorInvalidValue;
}

static int epl_of(int type) { return type == WT_Q8_0 ? 16 : type == WT_Q4_0 ? 32 : 8; }
static int xs_floats_rt(int type, int K) { int e = 32 * epl_of(type); return ((K + e - 1) / e) * e; }

static void raise_smem_limits_on_current_device() {
    // allow the GEMV stages to stage long vectors (up to 200 KB of dynamic shared memory)
    const int bytes = 200 * 1024;
#define ESP_SET(k) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes)
#define ESP_SET_ALL(WT)                                                                 \
    ESP_SET((k_gemv<WT, EPI_RESIDUAL>)); ESP_SET((k_gemv<WT, EPI_SWIGLU>));             \
    ESP_SET((k_gemv<WT, EPI_GELU>)); ESP_SET((k_lm_head<WT>)); ESP_SET((k_qkv<WT>));
    ESP_SET_ALL(WT_F16) ESP_SET_ALL(WT_BF16) ESP_SET_ALL(WT_Q8_0) ESP_SET_ALL(WT_Q4_0)
#undef ESP_SET_ALL
#undef ESP_SET
    cudaFuncSetAttribute(k_attention_prefill<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, pf_smem_bytes<32>());
    cudaFuncSetAttribute(k_attention_prefill<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, pf_smem_bytes<64>());
    cudaFuncSetAttribute(k_attention_prefill<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, pf_smem_bytes<128>());
}
// Function attributes belong to a device: set them once per device ordinal.
static void raise_smem_limits(int device) {
    static std::mutex mu;
    static bool done[64] = {};
    std::lock_guard<std::mutex> lock(mu);
    if (device < 0 || device >= 64 || done[device]) return;
    raise_smem_limits_on_current_device();
    done[device] = true;
}

// ---------------------------------------------------------------------------------------------- engine

// NCCL is looked up at run time (the library loads without it on single-GPU hosts).  When torch.distributed has
// already brought up its bundled NCCL the soname resolves to that copy.
struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};
static NcclApi& nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(h, "ncclAllReduce"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(h, "ncclAllGather"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
        api.ok = api.GetUniqueId && api.CommInitRank && api.AllReduce && api.CommDestroy && api.GetErrorString;
    });
    return api;
}
static int32_t nccl_fail(ncclResult_t r, const char* what) {
    NcclApi& api = nccl_api();
    return fail(ESP_CUDA_ERR_NCCL, std::string(what) + ": " + (api.GetErrorString ? api.GetErrorString(r) : "NCCL error"));
}

Engine::Engine(const esp_cuda_config& cfg) : cfg_(cfg) {}

Engine::~Engine() {
    if (cfg_.device >= 0) cudaSetDevice(cfg_.device);
    if (stream_) cudaStreamSynchronize(stream_);
    for (auto& g : graphs_) cudaGraphExecDestroy(g.second);  // graphs hold captured collectives: they go first
    // Destroying a tensor-parallel engine is a collective call: a peer may still be reading this rank's exchange block
    // (its last k_tp_sum_peers of a forward-only pass), so the ranks meet once more before any mapping or block goes away.
    if (tp_peer_ready_ && nccl_comm_ && nccl_api().ok && tp_epoch_) {
        unsigned long long* d_sync = reinterpret_cast<unsigned long long*>(tp_epoch_);  // two words of scratch the kernels no longer use
        if (nccl_api().AllReduce(d_sync, d_sync, 1, ncclUint64, ncclMax, static_cast<ncclComm_t>(nccl_comm_), stream_) == ncclSuccess)
            cudaStreamSynchronize(stream_);
    }
    for (int p = 0; p < 8; p++)
        if (tp_peer_block_[p] && p != tp_rank_) cudaIpcCloseMemHandle(tp_peer_block_[p]);
    if (tp_block_) cudaFree(tp_block_);
    if (nccl_comm_ && nccl_api().ok) {
        cudaDeviceSynchronize();
        nccl_api().CommDestroy(static_cast<ncclComm_t>(nccl_comm_));
    }
    for (auto e : prof_events_) cudaEventDestroy(e);
    for (auto e : step_events_) cudaEventDestroy(e);
    if (ev_begin_) cudaEventDestroy(ev_begin_);
    if (ev_end_) cudaEventDestroy(ev_end_);
    for (void* p : owned_) cudaFree(p);
    if (h_rows_block_) cudaFreeHost(h_rows_block_);
    if (h_next_) cudaFreeHost(h_next_);
    if (h_mega_ctl_) cudaFreeHost(h_mega_ctl_);
    if (stream_) cudaStreamDestroy(stream_);
}

static int32_t validate_config(const esp_cuda_config& c) {
    // validateConfig, RealModelInferenceEngine.swift:7615-7634
    if (c.n_layer <= 0 || c.n_head <= 0 || c.n_kv_head <= 0 || c.d_model <= 0 || c.head_dim <= 0 || c.hidden_dim <= 0 ||
        c.vocab <= 0 || c.max_seq <= 0)
        return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "invalid config: every dimension must be > 0");
    if (c.n_head % c.n_kv_head != 0) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "invalid config: nHead must be a multiple of nKVHead");
    if (c.architecture != ESP_CUDA_ARCH_LLAMA && c.architecture != ESP_CUDA_ARCH_GPT2)
        return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "invalid config: unknown architecture");
    if (c.max_batch < 1) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "invalid config: max_batch must be >= 1");
    if (c.head_dim < 8 || c.head_dim > 128 || (c.head_dim & (c.head_dim - 1)))
        return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "invalid config: head_dim must be a power of two in [8, 128]");
    if (c.d_model % 8 != 0 || c.hidden_dim % 8 != 0)
        return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "invalid config: d_model and hidden_dim must be multiples of 8");
    if (c.tp_size > 1) {
        if (c.tp_rank < 0 || c.tp_rank >= c.tp_size) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "invalid config: tp_rank out of range");
        if (c.n_head % c.tp_size || c.n_kv_head % c.tp_size || c.hidden_dim % c.tp_size || c.vocab % c.tp_size)
            return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "invalid config: heads, kv heads, hidden_dim and vocab must divide by tp_size");
        if (c.architecture != ESP_CUDA_ARCH_LLAMA) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "tensor parallelism is implemented for llama models");
    }
    return ESP_CUDA_OK;
}

template <typename T>
static int32_t dev_alloc(std::vector<void*>& owned, T** out, size_t count, bool zero = true) {
    void* p = nullptr;
    size_t bytes = std::max<size_t>(count * sizeof(T), 16);
    ESP_CUDA_TRY(cudaMalloc(&p, bytes));
    owned.push_back(p);
    if (zero) ESP_CUDA_TRY(cudaMemset(p, 0, bytes));
    *out = static_cast<T*>(p);
    return ESP_CUDA_OK;
}

int32_t Engine::init() {
    int32_t rc = validate_config(cfg_);
    if (rc) return rc;
    int n_dev = 0;
    cudaError_t e = cudaGetDeviceCount(&n_dev);
    if (e != cudaSuccess || n_dev == 0)
        return fail(ESP_CUDA_ERR_CUDA, std::string("no CUDA device available: ") + cudaGetErrorString(e));
    if (cfg_.device < 0 || cfg_.device >= n_dev) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "device ordinal out of range");
    ESP_CUDA_TRY(cudaSetDevice(cfg_.device));
    cudaDeviceProp prop;
    ESP_CUDA_TRY(cudaGetDeviceProperties(&prop, cfg_.device));
    if (prop.major < 10) return fail(ESP_CUDA_ERR_CUDA, "this library is built for sm_100a (B200) only");
    sm_count_ = prop.multiProcessorCount;
    raise_smem_limits(cfg_.device);
    ESP_CUDA_TRY(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));

    m_.arch = cfg_.architecture; m_.n_layer = cfg_.n_layer; m_.n_head = cfg_.n_head; m_.n_kv_head = cfg_.n_kv_head;
    m_.d_model = cfg_.d_model; m_.head_dim = cfg_.head_dim; m_.hidden = cfg_.hidden_dim; m_.vocab = cfg_.vocab;
    vocab_global_ = cfg_.vocab;
    tp_size_ = std::max(cfg_.tp_size, 1);
    tp_rank_ = tp_size_ > 1 ? cfg_.tp_rank : 0;
    if (tp_size_ > 1) {  // this rank's shard: its heads, its slice of the FFN hidden units and of the vocabulary
        m_.n_head /= tp_size_; m_.n_kv_head /= tp_size_; m_.hidden /= tp_size_; m_.vocab /= tp_size_;
        m_.q_dim = m_.n_head * m_.head_dim;
        m_.kv_dim = m_.n_kv_head * m_.head_dim;
    }
    m_.max_seq = cfg_.max_seq; m_.q_dim = m_.n_head * m_.head_dim; m_.kv_dim = m_.n_kv_head * m_.head_dim;
    m_.n_seq = cfg_.max_batch; m_.eps = cfg_.norm_eps; m_.eos_token = cfg_.eos_token;

    max_rows_ = std::max(cfg_.max_batch, kPrefillRows);  // rows of one pass: sequences of a batch, or positions of a prefill chunk
    n_splits_ = (m_.max_seq + kAttSplitTokens - 1) / kAttSplitTokens;
    out_stride_ = m_.max_seq;

    if ((rc = dev_alloc(owned_, &act_.hidden, (size_t)max_rows_ * m_.d_model))) return rc;
    if ((rc = dev_alloc(owned_, &act_.q, (size_t)max_rows_ * m_.q_dim))) return rc;
    if ((rc = dev_alloc(owned_, &act_.ctx, (size_t)max_rows_ * m_.q_dim))) return rc;
    if ((rc = dev_alloc(owned_, &act_.act, (size_t)max_rows_ * m_.hidden))) return rc;
    if ((rc = dev_alloc(owned_, &act_.att_part, (size_t)max_rows_ * m_.n_head * n_splits_ * (m_.head_dim + 2)))) return rc;
    if ((rc = dev_alloc(owned_, &act_.att_ticket, (size_t)max_rows_ * m_.n_head))) return rc;
    act_.logits = nullptr;
    act_.debug = nullptr;
    act_.debug_layer = -1;
    size_t kv_elems = (size_t)m_.n_layer * m_.n_seq * m_.n_kv_head * m_.max_seq * m_.head_dim;
    if ((rc = dev_alloc(owned_, &kv_.k, kv_elems))) return rc;
    if ((rc = dev_alloc(owned_, &kv_.v, kv_elems))) return rc;

    if ((rc = dev_alloc(owned_, &d_rows_block_, (size_t)6 * max_rows_))) return rc;
    rs_.seq = d_rows_block_;
    rs_.pos = d_rows_block_ + max_rows_;
    rs_.tok = reinterpret_cast<uint32_t*>(d_rows_block_ + 2 * max_rows_);
    rs_.active = d_rows_block_ + 3 * max_rows_;
    rs_.n_out = d_rows_block_ + 4 * max_rows_;
    rs_.limit = d_rows_block_ + 5 * max_rows_;
    if ((rc = dev_alloc(owned_, &rs_.next, (size_t)max_rows_))) return rc;
    if ((rc = dev_alloc(owned_, &rs_.out, (size_t)max_rows_ * out_stride_))) return rc;
    rs_.out_stride = out_stride_;
    if ((rc = dev_alloc(owned_, &rs_.best, (size_t)max_rows_))) return rc;
    if ((rc = dev_alloc(owned_, &rs_.ticket, 4))) return rc;
    ESP_CUDA_TRY(cudaMallocHost(reinterpret_cast<void**>(&h_rows_block_), sizeof(int) * 6 * max_rows_));
    ESP_CUDA_TRY(cudaMallocHost(reinterpret_cast<void**>(&h_next_), sizeof(uint32_t) * max_rows_));
    h_visible_.assign(cfg_.max_batch, 0);

    if (m_.arch == ARCH_LLAMA) {
        // cos/sin of applyHalfSplitRoPEPerHead (Engine.swift:6745-6772), evaluated on the host in fp32
        int half = m_.head_dim / 2;
        std::vector<float2> tab((size_t)m_.max_seq * half);
        for (int pos = 0; pos < m_.max_seq; pos++)
            for (int i = 0; i < half; i++) {
                float freq = 1.0f / powf(cfg_.rope_theta, (float)(2 * i) / (float)m_.head_dim);
                float ang = (float)pos * freq;
                tab[(size_t)pos * half + i] = make_float2(cosf(ang), sinf(ang));
            }
        if ((rc = dev_alloc(owned_, &d_rope_, tab.size(), false))) return rc;
        ESP_CUDA_TRY(cudaMemcpy(d_rope_, tab.data(), tab.size() * sizeof(float2), cudaMemcpyHostToDevice));
    }
    ESP_CUDA_TRY(cudaDeviceSynchronize());  // the zero-fills above ran on the default stream
    return ESP_CUDA_OK;
}

// Canonical tensor names; aliases follow the candidate lists of Engine.swift:2066-2154.
static std::string canonical_name(const std::string& n, int arch) {
    if (n == "embeddings/token_embeddings") return "embeddings/token";
    if (n == "embeddings/position_embeddings") return "embeddings/position";
    if (n == "classifier") return "lm_head";
    if (arch == ARCH_LLAMA) {
        if (n == "final_norm_gamma" || n == "final_norm") return "rms_final";
    } else {
        if (n == "ln_f_gamma" || n == "rms_final") return "final_norm_gamma";
        if (n == "ln_f_beta" || n == "rms_final_beta") return "final_norm_beta";
    }
    return n;
}

DeviceTensor* Engine::slot(const std::string& raw, int* rows, int* cols, bool* is_matrix, bool* is_embedding) {
    std::string name = canonical_name(raw, m_.arch);
    const int d = m_.d_model, q = m_.q_dim, kv = m_.kv_dim, h = m_.hidden, V = m_.vocab;
    *is_matrix = false;
    *is_embedding = false;
    auto set = [&](int r, int c) { *rows = r; *cols = c; return &tensors_[name]; };
    if (name == "embeddings/token") { *is_embedding = true; return set(vocab_global_, d); }
    if (name == "embeddings/position" && m_.arch == ARCH_GPT2) { *is_embedding = true; return set(m_.max_seq, d); }
    if (name == "lm_head") { *is_matrix = true; return set(V, d); }
    if (name == "rms_final" && m_.arch == ARCH_LLAMA) return set(1, d);
    if ((name == "final_norm_gamma" || name == "final_norm_beta") && m_.arch == ARCH_GPT2) return set(1, d);
    int l = -1;
    char leaf[64];
    if (sscanf(name.c_str(), "layers/%d/%63s", &l, leaf) == 2 && l >= 0 && l < m_.n_layer) {
        std::string lf(leaf);
        struct E { const char* n; int r, c; bool mat; int arch; };
        const E tab[] = {
            {"wq", q, d, true, -1}, {"wk", kv, d, true, -1}, {"wv", kv, d, true, -1}, {"wo", d, q, true, -1},
            {"w1", h, d, true, -1}, {"w2", d, h, true, -1}, {"w3", h, d, true, ARCH_LLAMA},
            {"rms_att", 1, d, false, ARCH_LLAMA}, {"rms_ffn", 1, d, false, ARCH_LLAMA},
            {"q_norm", 1, m_.head_dim, false, ARCH_LLAMA}, {"k_norm", 1, m_.head_dim, false, ARCH_LLAMA},  // optional (Qwen3)
            {"ln_1_gamma", 1, d, false, ARCH_GPT2}, {"ln_1_beta", 1, d, false, ARCH_GPT2},
            {"ln_2_gamma", 1, d, false, ARCH_GPT2}, {"ln_2_beta", 1, d, false, ARCH_GPT2},
            {"bq", 1, q, false, ARCH_GPT2}, {"bk", 1, kv, false, ARCH_GPT2}, {"bv", 1, kv, false, ARCH_GPT2},
            {"bo", 1, d, false, ARCH_GPT2}, {"b1", 1, h, false, ARCH_GPT2}, {"b2", 1, d, false, ARCH_GPT2},
        };
        for (const E& e : tab)
            if (lf == e.n && (e.arch < 0 || e.arch == m_.arch)) { *is_matrix = e.mat; return set(e.r, e.c); }
    }
    return nullptr;
}

int32_t Engine::load_tensor(const char* name_c, int32_t type, const void* data, uint64_t nbytes) {
    if (!name_c || !data) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "load_tensor: null argument");
    if (finalized_) return fail(ESP_CUDA_ERR_STATE, "load_tensor: engine already finalized");
    ESP_CUDA_TRY(cudaSetDevice(cfg_.device));
    int rows = 0, cols = 0;
    bool is_matrix = false, is_embedding = false;
    DeviceTensor* t = slot(name_c, &rows, &cols, &is_matrix, &is_embedding);
    if (!t) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, std::string("load_tensor: unknown tensor name '") + name_c + "'");
    const uint64_t n = (uint64_t)rows * cols;
    uint64_t expect;
    switch (type) {
        case ESP_CUDA_F32: expect = n * 4; break;
        case ESP_CUDA_F16: case ESP_CUDA_BF16: expect = n * 2; break;
        case ESP_CUDA_Q8_0: expect = n / 32 * 34; break;
        case ESP_CUDA_Q4_0: expect = n / 32 * 18; break;
        default: return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "load_tensor: unsupported tensor type");
    }
    if (nbytes != expect) {  // invalidWeightCount(path, expected, actual), Engine.swift:85-115
        std::ostringstream os;
        os << "invalid weight count for " << name_c << ": expected " << expect << " bytes, got " << nbytes;
        return fail(ESP_CUDA_ERR_INVALID_WEIGHTS, os.str());
    }
    const bool quant = type == ESP_CUDA_Q8_0 || type == ESP_CUDA_Q4_0;
    if (quant && (!is_matrix || cols % 32 != 0))
        return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "load_tensor: Q8_0/Q4_0 are valid for matrices with cols % 32 == 0 only");
    if (t->loaded) return fail(ESP_CUDA_ERR_STATE, std::string("load_tensor: tensor loaded twice: ") + name_c);
    int32_t rc;
    t->rows = rows; t->cols = cols;
    void* staging = nullptr;
    if (quant || type == ESP_CUDA_F32 || (!is_matrix && !is_embedding)) {
        ESP_CUDA_TRY(cudaMalloc(&staging, std::max<uint64_t>(nbytes, 16)));
        cudaError_t e = cudaMemcpyAsync(staging, data, nbytes, cudaMemcpyDefault, stream_);
        if (e != cudaSuccess) { cudaFree(staging); ESP_CUDA_TRY(e); }
    }
    const int T = 256;
    if (!is_matrix && !is_embedding) {  // norm gains / biases: keep an fp32 copy
        if (quant) { cudaFree(staging); return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "vectors cannot be quantised"); }
        if ((rc = dev_alloc(owned_, &t->f32, n, false))) { cudaFree(staging); return rc; }
        k_to_f32<<<(unsigned)((n + T - 1) / T), T, 0, stream_>>>(staging, type, (int64_t)n, t->f32);
        t->type = ESP_CUDA_F32;
    } else if (quant) {
        uint64_t nb = n / 32;
        __half* sc = nullptr;
        if ((rc = dev_alloc(owned_, &sc, nb, false))) { cudaFree(staging); return rc; }
        t->scales = sc;
        if (type == ESP_CUDA_Q8_0) {
            int8_t* qd = nullptr;
            if ((rc = dev_alloc(owned_, &qd, n, false))) { cudaFree(staging); return rc; }
            k_repack_q8_0<<<(unsigned)((nb + T - 1) / T), T, 0, stream_>>>(static_cast<uint8_t*>(staging), (int64_t)nb, qd, sc);
            t->data = qd;
        } else {
            uint8_t* qd = nullptr;
            if ((rc = dev_alloc(owned_, &qd, n / 2, false))) { cudaFree(staging); return rc; }
            k_repack_q4_0<<<(unsigned)((nb + T - 1) / T), T, 0, stream_>>>(static_cast<uint8_t*>(staging), (int64_t)nb, qd, sc);
            t->data = qd;
        }
        t->type = type;
    } else if (type == ESP_CUDA_F32) {  // matrices and embeddings are stored as fp16
        __half* hd = nullptr;
        if ((rc = dev_alloc(owned_, &hd, n, false))) { cudaFree(staging); return rc; }
        k_f32_to_f16<<<(unsigned)((n + T - 1) / T), T, 0, stream_>>>(static_cast<float*>(staging), (int64_t)n, hd);
        t->data = hd;
        t->type = ESP_CUDA_F16;
    } else {
        uint16_t* hd = nullptr;
        if ((rc = dev_alloc(owned_, &hd, n, false))) return rc;
        ESP_CUDA_TRY(cudaMemcpyAsync(hd, data, nbytes, cudaMemcpyDefault, stream_));
        t->data = hd;
        t->type = type;
    }
    cudaError_t e = cudaStreamSynchronize(stream_);
    if (staging) cudaFree(staging);
    ESP_CUDA_TRY(e);
    ESP_CUDA_TRY(cudaGetLastError());
    t->loaded = true;
    return ESP_CUDA_OK;
}

static bool path_exists(const std::string& p) { struct stat st; return stat(p.c_str(), &st) == 0; }
static bool is_directory(const std::string& p) { struct stat st; return stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode); }

// BlobWeightLoader.load (Sources/ModelSupport/BlobWeightLoader.swift:25-92): header checks and payload read.
static int32_t read_blob(const std::string& path, std::vector<uint16_t>& out) {
    std::ifstream f(path, std::ios::binary);
    if (!f) return fail(ESP_CUDA_ERR_IO, "missing weight file: " + path);
    uint8_t header[128];
    f.read(reinterpret_cast<char*>(header), 128);
    if (f.gcount() < 128) return fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "truncatedHeader: " + path);
    uint32_t magic, size, off;
    memcpy(&magic, header + 64, 4); memcpy(&size, header + 72, 4); memcpy(&off, header + 80, 4);
    if (magic != 0xDEADBEEFu) return fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "invalidMagic: " + path);
    if (off != 128u) return fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "invalidDataOffset: " + path);
    if (size % 2u) return fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "invalidPayloadSize: " + path);
    out.resize(size / 2);
    f.read(reinterpret_cast<char*>(out.data()), size);
    if ((uint32_t)f.gcount() != size) return fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "truncatedPayload: " + path);
    return ESP_CUDA_OK;
}

// loadWeightTablePreferringFloat32Sidecar (Sources/RealModelInference/RealModelInferenceEngine.swift:7830-7879):
// "<name>.float32.bin" (raw little-endian fp32, exactly the tensor's element count) wins over "<name>.bin" (BLOBFILE
// fp16).  Norm gains and biases keep the fp32 values; matrices and embeddings are rounded to the fp16 the device
// computes in (load_tensor).  Returns -1 when neither file exists.
int32_t Engine::load_file_tensor(const std::string& dir, const std::string& name) {
    const std::string side = dir + "/" + name + ".float32.bin", blob = dir + "/" + name + ".bin";
    if (path_exists(side)) {
        std::ifstream f(side, std::ios::binary | std::ios::ate);
        if (!f) return fail(ESP_CUDA_ERR_IO, "Failed to read float32 sidecar " + side);
        const std::streamoff size = f.tellg();
        int rows = 0, cols = 0;
        bool is_matrix = false, is_embedding = false;
        if (!slot(name, &rows, &cols, &is_matrix, &is_embedding)) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "unknown tensor: " + name);
        const long long expect = (long long)rows * cols;
        if (size != (std::streamoff)(expect * 4)) {
            std::ostringstream os;
            os << "invalidWeightCount: " << side << " expected " << expect << " actual " << (long long)size / 4;
            return fail(ESP_CUDA_ERR_INVALID_WEIGHTS, os.str());
        }
        std::vector<float> buf((size_t)expect);
        f.seekg(0);
        f.read(reinterpret_cast<char*>(buf.data()), size);
        if (f.gcount() != size) return fail(ESP_CUDA_ERR_IO, "Failed to read float32 sidecar " + side);
        return load_tensor(name.c_str(), ESP_CUDA_F32, buf.data(), buf.size() * 4);
    }
    if (!path_exists(blob)) return -1;
    std::vector<uint16_t> buf;
    int32_t rc = read_blob(blob, buf);
    if (rc) return rc;
    return load_tensor(name.c_str(), ESP_CUDA_F16, buf.data(), buf.size() * 2);
}

int32_t Engine::load_directory(const char* dir_c) {
    std::string dir(dir_c ? dir_c : "");
    if (!is_directory(dir)) return fail(ESP_CUDA_ERR_IO, "weight directory not found: " + dir);
    auto load_first = [&](std::initializer_list<const char*> cands, const char* label) -> int32_t {
        for (const char* c : cands) {
            int32_t rc = load_file_tensor(dir, c);
            if (rc != -1) return rc;
        }
        return fail(ESP_CUDA_ERR_IO, std::string("missing ") + label + " in " + dir);
    };
    int32_t rc;
    if ((rc = load_first({"embeddings/token", "embeddings/token_embeddings"}, "token embedding"))) return rc;
    if ((rc = load_first({"lm_head", "classifier"}, "lm head"))) return rc;
    if (m_.arch == ARCH_GPT2) {
        if ((rc = load_first({"embeddings/position", "embeddings/position_embeddings"}, "position embedding"))) return rc;
        if ((rc = load_first({"final_norm_gamma", "ln_f_gamma", "rms_final"}, "final norm gamma"))) return rc;
        if ((rc = load_first({"final_norm_beta", "ln_f_beta", "rms_final_beta"}, "final norm beta"))) return rc;
    } else {
        if ((rc = load_first({"rms_final", "final_norm_gamma", "final_norm"}, "final norm gamma"))) return rc;
    }
    const char* llama[] = {"rms_att", "wq", "wk", "wv", "wo", "rms_ffn", "w1", "w2", "w3"};
    const char* gpt2[] = {"ln_1_gamma", "ln_1_beta", "wq", "wk", "wv", "wo", "bq", "bk", "bv", "bo",
                          "ln_2_gamma", "ln_2_beta", "w1", "b1", "w2", "b2"};
    for (int l = 0; l < m_.n_layer; l++) {
        const char* const* names = m_.arch == ARCH_GPT2 ? gpt2 : llama;
        int n = m_.arch == ARCH_GPT2 ? 16 : 9;
        for (int i = 0; i < n; i++) {
            std::string name = "layers/" + std::to_string(l) + "/" + names[i];
            rc = load_file_tensor(dir, name);
            if (rc == -1) return fail(ESP_CUDA_ERR_IO, "missing weight file: " + dir + "/" + name + ".bin");
            if (rc) return rc;
        }
        if (m_.arch == ARCH_LLAMA) {
            // optional per-head q/k norm weights: both or neither (Engine.swift:6589-6596)
            const std::string base = "layers/" + std::to_string(l) + "/";
            const int32_t rq = load_file_tensor(dir, base + "q_norm"), rk = load_file_tensor(dir, base + "k_norm");
            if (rq > 0) return rq;
            if (rk > 0) return rk;
            if ((rq == -1) != (rk == -1))
                return fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "Mismatched llama Q/K norm weights for " + dir + "/" + base + "; expected both q_norm.bin and k_norm.bin");
        }
    }
    return ESP_CUDA_OK;
}

int32_t Engine::finalize() {
    if (finalized_) return ESP_CUDA_OK;
    if (tp_size_ > 1 && !nccl_comm_) return fail(ESP_CUDA_ERR_STATE, "finalize: call esp_cuda_tp_init on every rank first");
    auto need = [&](const std::string& n) { auto it = tensors_.find(n); return it != tensors_.end() && it->second.loaded; };
    std::vector<std::string> req = {"embeddings/token", "lm_head"};
    if (m_.arch == ARCH_GPT2) { req.push_back("embeddings/position"); req.push_back("final_norm_gamma"); req.push_back("final_norm_beta"); }
    else req.push_back("rms_final");
    for (int l = 0; l < m_.n_layer; l++) {
        std::string p = "layers/" + std::to_string(l) + "/";
        if (m_.arch == ARCH_GPT2)
            for (const char* n : {"ln_1_gamma", "ln_1_beta", "wq", "wk", "wv", "wo", "bq", "bk", "bv", "bo", "ln_2_gamma", "ln_2_beta", "w1", "b1", "w2", "b2"}) req.push_back(p + n);
        else
            for (const char* n : {"rms_att", "wq", "wk", "wv", "wo", "rms_ffn", "w1", "w2", "w3"}) req.push_back(p + n);
    }
    for (auto& n : req)
        if (!need(n)) return fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "missing tensor: " + n);
    for (int l = 0; l < m_.n_layer; l++) {
        std::string p = "layers/" + std::to_string(l) + "/";
        int tq = tensors_[p + "wq"].type;
        if (tensors_[p + "wk"].type != tq || tensors_[p + "wv"].type != tq)
            return fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "wq/wk/wv of a layer must share one storage type");
        if (m_.arch == ARCH_LLAMA && tensors_[p + "w1"].type != tensors_[p + "w3"].type)
            return fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "w1/w3 of a layer must share one storage type");
    }
    if (m_.arch == ARCH_GPT2 && tensors_["embeddings/position"].type != tensors_["embeddings/token"].type)
        return fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "token and position embeddings must share one storage type");
    int32_t rc;
    // per-head q/k norm (Qwen3): every layer carries both vectors, or none does
    int n_qk = 0;
    for (int l = 0; l < m_.n_layer; l++) {
        const std::string p = "layers/" + std::to_string(l) + "/";
        const bool hq = need(p + "q_norm"), hk = need(p + "k_norm");
        if (hq != hk) return fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "Mismatched llama Q/K norm weights in layer " + std::to_string(l) + "; expected both q_norm and k_norm");
        n_qk += hq ? 1 : 0;
    }
    if (n_qk != 0 && n_qk != m_.n_layer) return fail(ESP_CUDA_ERR_INVALID_WEIGHTS, "q_norm/k_norm must be present in every layer or in none");
    qk_norm_ = n_qk > 0;
    if (qk_norm_ && tp_size_ > 1) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "per-head q/k norm is not available with tensor parallelism");
    // full logits are kept for rows that run the head: sequences of a batch (or the two rows of a verify pass), every
    // row of a pass only when the engine was asked to keep logits
    const int logit_rows = (cfg_.flags & ESP_CUDA_FLAG_KEEP_LOGITS) ? max_rows_ : std::max(cfg_.max_batch, 2);
    if ((rc = dev_alloc(owned_, &act_.logits, (size_t)logit_rows * m_.vocab))) return rc;
    size_t dbg = (size_t)m_.q_dim * 2 + 2 * m_.kv_dim + 2 * m_.d_model + m_.hidden;
    if ((rc = dev_alloc(owned_, &d_debug_, dbg))) return rc;
    ESP_CUDA_TRY(cudaDeviceSynchronize());
    if ((rc = build_tc())) return rc;
    if (qk_norm_ && !kraw_) {  // the per-stage q/k/v kernel hands k and v to the norm + RoPE + append kernel through these
        if ((rc = dev_alloc(owned_, &kraw_, (size_t)max_rows_ * m_.kv_dim))) return rc;
        if ((rc = dev_alloc(owned_, &vraw_, (size_t)max_rows_ * m_.kv_dim))) return rc;
    }
    if (tp_size_ > 1 && tc_ready_ && (rc = tp_peer_setup())) return rc;
    if ((rc = build_mega())) return rc;
    finalized_ = true;
    return reset();
}

Weight Engine::weight_of(const DeviceTensor& t) const {
    Weight w;
    w.data = t.data; w.scales = t.scales; w.rows = t.rows; w.cols = t.cols; w.type = t.type; w.pad = 0;
    return w;
}

LayerWeights Engine::layer_weights(int l) const {
    std::string p = "layers/" + std::to_string(l) + "/";
    auto T = [&](const char* n) -> const DeviceTensor& { return tensors_.at(p + n); };
    auto F = [&](const char* n) -> const float* { auto it = tensors_.find(p + n); return it == tensors_.end() ? nullptr : it->second.f32; };
    LayerWeights lw{};
    lw.wq = weight_of(T("wq")); lw.wk = weight_of(T("wk")); lw.wv = weight_of(T("wv")); lw.wo = weight_of(T("wo"));
    lw.w1 = weight_of(T("w1")); lw.w2 = weight_of(T("w2"));
    if (m_.arch == ARCH_LLAMA) {
        lw.w3 = weight_of(T("w3"));
        lw.norm1_g = F("rms_att"); lw.norm2_g = F("rms_ffn");
    } else {
        lw.w3 = Weight{nullptr, nullptr, 0, 0, 0, 0};
        lw.norm1_g = F("ln_1_gamma"); lw.norm1_b = F("ln_1_beta"); lw.norm2_g = F("ln_2_gamma"); lw.norm2_b = F("ln_2_beta");
        lw.bq = F("bq"); lw.bk = F("bk"); lw.bv = F("bv"); lw.bo = F("bo"); lw.b1 = F("b1"); lw.b2 = F("b2");
    }
    return lw;
}

size_t Engine::gemv_smem(int type, int K, bool with_tmp) const {
    return sizeof(float) * (size_t)(kRedFloats + xs_floats_rt(type, K) + (with_tmp ? m_.d_model : 0));
}

int32_t Engine::check_ready(const char* what) const {
    if (!finalized_) return fail(ESP_CUDA_ERR_STATE, std::string(what) + ": engine is not finalized");
    if (force_failure_enabled()) return fail(ESP_CUDA_ERR_FORCED_FAILURE, std::string(what) + ": forced failure is enabled");
    cudaError_t e = cudaSetDevice(cfg_.device);
    if (e != cudaSuccess) return fail(ESP_CUDA_ERR_CUDA, cudaGetErrorString(e));
    return ESP_CUDA_OK;
}

// One pass over the model for `rows` rows.  mode: STEP_FORWARD runs the layers on (tok, pos) of every active
// row; STEP_HEAD runs final norm + LM head + argmax; STEP_FEEDBACK makes the head emit and feed back its token.
int32_t Engine::launch_step(int rows, int mode, cudaStream_t s, bool profile) {
    if (tp_size_ > 1 && !tc_ready_) return fail(ESP_CUDA_ERR_STATE, "tensor parallelism needs 16-bit weights with 64-aligned shard sizes");
    if (tc_ready_ && (rows >= kTcMinRows || tp_size_ > 1)) return launch_step_tc(rows, mode, s);
    const bool gpt2 = m_.arch == ARCH_GPT2;
    const int cap = sm_count_ * 2;  // one wave: the stage kernels hold ~120 registers, two CTAs per SM
    int launches = 0;
    Activations a = act_;
    a.logits = nullptr;
    a.debug = debug_layer_ >= 0 ? d_debug_ : nullptr;
    a.debug_layer = debug_layer_;
    size_t ev = 0;
    auto mark = [&]() { if (profile && ev < prof_events_.size()) cudaEventRecord(prof_events_[ev++], s); };
    mark();
    if (mode & STEP_FORWARD) {
        const DeviceTensor& te = tensors_.at("embeddings/token");
        for (int l = 0; l < m_.n_layer; l++) {
            LayerWeights lw = layer_weights(l);
            QkvArgs qa{};
            qa.m = m_; qa.lw = lw; qa.layer = l; qa.rows = rows; qa.rs = rs_; qa.a = a; qa.kv = kv_;
            qa.tok_emb = static_cast<const uint16_t*>(te.data);
            qa.pos_emb = gpt2 ? static_cast<const uint16_t*>(tensors_.at("embeddings/position").data) : nullptr;
            qa.emb_type = te.type == ESP_CUDA_BF16 ? WT_BF16 : WT_F16;
            qa.rope = d_rope_;
            qa.from_embedding = l == 0;
            qa.k_raw = qk_norm_ ? kraw_ : nullptr;
            qa.v_raw = qk_norm_ ? vraw_ : nullptr;
            int items = (m_.q_dim + 2 * m_.kv_dim) / 2;
            int grid = std::max(1, std::min((items + kWarps - 1) / kWarps, cap));
            ESP_CUDA_TRY(launch_qkv(lw.wq.type, dim3(grid), gemv_smem(lw.wq.type, m_.d_model, true), s, qa));
            launches++;
            if (qk_norm_) {  // per-head norm, RoPE and the cache append need whole heads: one more small kernel
                RopeArgs ra{};
                ra.m = m_; ra.rs = rs_; ra.kv = kv_; ra.q = act_.q; ra.k_raw = kraw_; ra.v_raw = vraw_; ra.rope = d_rope_; ra.layer = l;
                ra.debug = (a.debug && l == debug_layer_) ? a.debug : nullptr;
                ra.q_norm = tensors_.at("layers/" + std::to_string(l) + "/q_norm").f32;
                ra.k_norm = tensors_.at("layers/" + std::to_string(l) + "/k_norm").f32;
                ESP_CUDA_TRY(launch_pdl(k_rope_append, dim3(rows, (m_.q_dim / 2 + m_.kv_dim + kThreads - 1) / kThreads), dim3(kThreads), 0, s, ra));
                launches++;
            }
            mark();
            AttArgs aa{};
            aa.m = m_; aa.layer = l; aa.rows = rows; aa.n_splits = n_splits_; aa.rs = rs_; aa.a = a; aa.kv = kv_;
            ESP_CUDA_TRY(launch_pdl(k_attention, dim3(m_.n_head, rows, n_splits_), dim3(kAttThreads), 0, s, aa));
            launches++;
            mark();
            GemvArgs ga{};
            ga.m = m_; ga.rows = rows; ga.rs = rs_; ga.a = a; ga.layer = l;
            // output projection + residual
            ga.w = lw.wo; ga.bias = lw.bo; ga.norm = NORM_NONE; ga.in = act_.ctx; ga.in_stride = m_.q_dim;
            ga.out = act_.hidden; ga.out_stride = m_.d_model; ga.debug_slot = 2 * m_.q_dim + 2 * m_.kv_dim;
            items = (m_.d_model + 1) / 2;
            grid = std::max(1, std::min((items + kWarps - 1) / kWarps, cap));
            ESP_CUDA_TRY(launch_gemv(EPI_RESIDUAL, lw.wo.type, dim3(grid), gemv_smem(lw.wo.type, m_.q_dim, false), s, ga));
            launches++;
            // FFN up (+gate) with the activation fused
            ga.w = lw.w1; ga.w_up = lw.w3; ga.bias = lw.b1; ga.norm = gpt2 ? NORM_LAYER : NORM_RMS;
            ga.norm_g = lw.norm2_g; ga.norm_b = lw.norm2_b; ga.in = act_.hidden; ga.in_stride = m_.d_model;
            ga.out = act_.act; ga.out_stride = m_.hidden; ga.debug_slot = 2 * m_.q_dim + 2 * m_.kv_dim + m_.d_model;
            items = gpt2 ? (m_.hidden + 1) / 2 : m_.hidden;
            grid = std::max(1, std::min((items + kWarps - 1) / kWarps, cap));
            ESP_CUDA_TRY(launch_gemv(gpt2 ? EPI_GELU : EPI_SWIGLU, lw.w1.type, dim3(grid), gemv_smem(lw.w1.type, m_.d_model, false), s, ga));
            launches++;
            // FFN down + residual
            ga.w = lw.w2; ga.w_up = Weight{nullptr, nullptr, 0, 0, 0, 0}; ga.bias = lw.b2; ga.norm = NORM_NONE;
            ga.norm_g = ga.norm_b = nullptr; ga.in = act_.act; ga.in_stride = m_.hidden; ga.out = act_.hidden;
            ga.out_stride = m_.d_model; ga.debug_slot = 2 * m_.q_dim + 2 * m_.kv_dim + m_.d_model + m_.hidden;
            items = (m_.d_model + 1) / 2;
            grid = std::max(1, std::min((items + kWarps - 1) / kWarps, cap));
            ESP_CUDA_TRY(launch_gemv(EPI_RESIDUAL, lw.w2.type, dim3(grid), gemv_smem(lw.w2.type, m_.hidden, false), s, ga));
            launches++;
            mark();
        }
    }
    if (mode & STEP_HEAD) {
        const DeviceTensor& lh = tensors_.at("lm_head");
        GemvArgs ga{};
        ga.m = m_; ga.rows = rows; ga.rs = rs_; ga.a = a; ga.layer = -1; ga.debug_slot = -1;
        if (cfg_.flags & ESP_CUDA_FLAG_KEEP_LOGITS) ga.a.logits = act_.logits;
        ga.w = weight_of(lh); ga.norm = gpt2 ? NORM_LAYER : NORM_RMS;
        ga.norm_g = tensors_.at(gpt2 ? "final_norm_gamma" : "rms_final").f32;
        ga.norm_b = gpt2 ? tensors_.at("final_norm_beta").f32 : nullptr;
        ga.in = act_.hidden; ga.in_stride = m_.d_model; ga.out = nullptr; ga.out_stride = 0;
        ga.finalize_mode = ((mode & STEP_FEEDBACK) ? 1 : 0) | ((mode & STEP_FORWARD) ? 2 : 0);
        int items = (m_.vocab + 1) / 2;
        int grid = std::max(1, std::min((items + kWarps - 1) / kWarps, cap));
        ESP_CUDA_TRY(launch_gemv(EPI_HEAD, lh.type, dim3(grid), gemv_smem(lh.type, m_.d_model, false), s, ga));
        launches++;
    } else if (mode & STEP_FORWARD) {
        ESP_CUDA_TRY(launch_pdl(k_bump, dim3(1), dim3(64), 0, s, rs_, rows));
        launches++;
    }
    mark();
    launches_last_step_ = launches;
    return ESP_CUDA_OK;
}

int32_t Engine::submit(int rows, int mode) {
    if (force_failure_enabled()) return fail(ESP_CUDA_ERR_FORCED_FAILURE, "forced failure is enabled");
    if (tc_ready_ && !tc_operands_ready_ && (rows >= kTcMinRows || tp_size_ > 1)) {
        int32_t rc = tc_operands();  // before any capture: it allocates
        if (rc) return rc;
    }
    const bool direct = (cfg_.flags & ESP_CUDA_FLAG_NO_GRAPH) || debug_layer_ >= 0;
    if (direct) {
        bool profile = (cfg_.flags & ESP_CUDA_FLAG_NO_GRAPH) && (mode & STEP_FORWARD) && (mode & STEP_HEAD);
        if (profile && prof_events_.empty()) {
            prof_events_.resize((size_t)3 * m_.n_layer + 2);
            for (auto& e : prof_events_) ESP_CUDA_TRY(cudaEventCreate(&e));
        }
        int32_t rc = launch_step(rows, mode, stream_, profile);
        if (rc) return rc;
        if (profile) {
            ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
            timings_ = esp_cuda_timings{};
            for (int l = 0; l < m_.n_layer; l++) {
                float t;
                cudaEventElapsedTime(&t, prof_events_[3 * l], prof_events_[3 * l + 1]); timings_.qkv_ms += t;
                cudaEventElapsedTime(&t, prof_events_[3 * l + 1], prof_events_[3 * l + 2]); timings_.attention_ms += t;
                cudaEventElapsedTime(&t, prof_events_[3 * l + 2], prof_events_[3 * l + 3]); timings_.ffn_ms += t;
            }
            float t;
            cudaEventElapsedTime(&t, prof_events_[3 * m_.n_layer], prof_events_[3 * m_.n_layer + 1]); timings_.head_ms = t;
            cudaEventElapsedTime(&t, prof_events_[0], prof_events_[3 * m_.n_layer + 1]); timings_.total_ms = t;
        }
        timings_.kernel_launches = launches_last_step_;
        return ESP_CUDA_OK;
    }
    const int key = rows * 16 + mode;
    auto it = graphs_.find(key);
    if (it == graphs_.end()) {
        cudaGraph_t graph = nullptr;
        ESP_CUDA_TRY(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
        int32_t rc = launch_step(rows, mode, stream_, false);
        cudaError_t e = cudaStreamEndCapture(stream_, &graph);
        if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
        ESP_CUDA_TRY(e);
        cudaGraphExec_t exec = nullptr;
        e = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        ESP_CUDA_TRY(e);
        it = graphs_.emplace(key, exec).first;
        launches_by_key_[key] = launches_last_step_;
    }
    launches_last_step_ = launches_by_key_[key];
    timings_.kernel_launches = launches_last_step_;
    ESP_CUDA_TRY(cudaGraphLaunch(it->second, stream_));
    return ESP_CUDA_OK;
}

int32_t Engine::upload_rows(int rows, const int* seq, const int* pos, const uint32_t* tok, const int* active,
                            const int* limit, bool zero_out_counts) {
    if (rows < 1 || rows > max_rows_) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "row count out of range");
    // the pinned block may still be in flight from the previous call
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    int* h = h_rows_block_;
    for (int r = 0; r < max_rows_; r++) {
        bool in = r < rows;
        h[r] = in ? seq[r] : 0;
        h[max_rows_ + r] = in ? pos[r] : 0;
        h[2 * max_rows_ + r] = in && tok ? (int)tok[r] : 0;
        h[3 * max_rows_ + r] = in ? (active ? active[r] : 1) : 0;
        h[4 * max_rows_ + r] = 0;
        h[5 * max_rows_ + r] = in && limit ? limit[r] : 0;
    }
    (void)zero_out_counts;
    ESP_CUDA_TRY(cudaMemcpyAsync(d_rows_block_, h, sizeof(int) * 6 * max_rows_, cudaMemcpyHostToDevice, stream_));
    return ESP_CUDA_OK;
}

int32_t Engine::reset() {
    int32_t rc = check_ready("reset");
    if (rc) return rc;
    // reset() zeroes the caches and the hidden state (Engine.swift:613-635)
    size_t kv_bytes = (size_t)m_.n_layer * m_.n_seq * m_.n_kv_head * m_.max_seq * m_.head_dim * sizeof(__half);
    ESP_CUDA_TRY(cudaMemsetAsync(kv_.k, 0, kv_bytes, stream_));
    ESP_CUDA_TRY(cudaMemsetAsync(kv_.v, 0, kv_bytes, stream_));
    ESP_CUDA_TRY(cudaMemsetAsync(act_.hidden, 0, sizeof(float) * (size_t)max_rows_ * m_.d_model, stream_));
    ESP_CUDA_TRY(cudaMemsetAsync(rs_.best, 0, sizeof(unsigned long long) * max_rows_, stream_));
    ESP_CUDA_TRY(cudaMemsetAsync(rs_.ticket, 0, 16, stream_));
    ESP_CUDA_TRY(cudaMemsetAsync(act_.att_ticket, 0, sizeof(unsigned int) * (size_t)max_rows_ * m_.n_head, stream_));
    // a bounded wait of the batched or tensor-parallel kernels that ran out left its code here and makes every later
    // kernel skip its waits: reset() is the documented way back (on a tensor-parallel group every rank must reset)
    if (d_tc_error_) ESP_CUDA_TRY(cudaMemsetAsync(d_tc_error_, 0, sizeof(int), stream_));
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    std::fill(h_visible_.begin(), h_visible_.end(), 0);
    for (auto& c : checkpoints_) c.visible = -1;
    pending_verify_ = 0;
    return ESP_CUDA_OK;
}

// Feeds one token to each of `rows` rows (row r = sequence seq[r] at its current position) and optionally
// selects the next greedy token of each row.
int32_t Engine::feed_rows(int rows, const int* seq, const uint32_t* tok, bool with_head, uint32_t* next_out) {
    std::vector<int> pos(rows);
    std::vector<int> extra(m_.n_seq, 0);
    for (int r = 0; r < rows; r++) {
        int s = seq[r];
        if (s < 0 || s >= m_.n_seq) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "sequence index out of range");
        pos[r] = h_visible_[s] + extra[s]++;
        if (pos[r] >= m_.max_seq) {  // advance guard, Engine.swift:673-677
            std::ostringstream os;
            os << "position " << pos[r] << " exceeds context " << m_.max_seq;
            return fail(ESP_CUDA_ERR_OUT_OF_RANGE, os.str());
        }
        if (tok[r] >= (uint32_t)vocab_global_) {  // token guard, Engine.swift:687-689
            std::ostringstream os;
            os << "token " << tok[r] << " is outside vocab " << vocab_global_;
            return fail(ESP_CUDA_ERR_OUT_OF_RANGE, os.str());
        }
    }
    int32_t rc = upload_rows(rows, seq, pos.data(), tok, nullptr, nullptr, true);
    if (rc) return rc;
    // A prompt pass whose 64-row tiles each hold consecutive positions of one sequence takes the tiled tensor-core
    // attention (prefill_attention.cuh); the choice is part of the graph key.
    int tiled = 0;
    if (tc_ready_ && rows >= 32 && !with_head && (m_.head_dim == 32 || m_.head_dim == 64 || m_.head_dim == 128)) {
        tiled = STEP_TILED_ATT;
        for (int r = 1; r < rows && tiled; r++)
            if (r % kPfRows != 0 && (seq[r] != seq[r - 1] || pos[r] != pos[r - 1] + 1)) tiled = 0;
    }
    if ((rc = submit(rows, STEP_FORWARD | (with_head ? STEP_HEAD : 0) | tiled))) return rc;
    if (with_head) ESP_CUDA_TRY(cudaMemcpyAsync(h_next_, rs_.next, sizeof(uint32_t) * rows, cudaMemcpyDeviceToHost, stream_));
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    if (tc_ready_ && (rows >= kTcMinRows || tp_size_ > 1)) {
        int herr = 0;
        ESP_CUDA_TRY(cudaMemcpy(&herr, d_tc_error_, sizeof(int), cudaMemcpyDeviceToHost));
        if (herr) return fail(ESP_CUDA_ERR_TIMEOUT, herr == 8 ? "peer all-reduce gave up waiting for another rank" : "tensor-core GEMM gave up waiting on a barrier");
    }
    for (int s = 0; s < m_.n_seq; s++) h_visible_[s] += extra[s];
    if (with_head && next_out) memcpy(next_out, h_next_, sizeof(uint32_t) * rows);
    return ESP_CUDA_OK;
}

int32_t Engine::feed(int rows, const int* seq, const uint32_t* tok, bool with_head, uint32_t* next_out) {
    int32_t rc = check_ready("feed");
    if (rc) return rc;
    if (!seq || !tok || rows < 1 || rows > max_rows_) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "feed: bad arguments");
    rc = feed_rows(rows, seq, tok, with_head, next_out);
    if (rc == ESP_CUDA_OK && rows > 1 && seq[rows - 1] == 0 && seq[0] == 0) {
        ESP_CUDA_TRY(cudaMemcpyAsync(act_.hidden, act_.hidden + (size_t)(rows - 1) * m_.d_model, sizeof(float) * m_.d_model,
                                     cudaMemcpyDeviceToDevice, stream_));
        ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    }
    return rc;
}

int32_t Engine::advance(uint32_t token) {
    int32_t rc = check_ready("advance");
    if (rc) return rc;
    int seq = 0;
    return feed_rows(1, &seq, &token, false, nullptr);
}

int32_t Engine::decode_step(uint32_t token, uint32_t* next) {
    int32_t rc = check_ready("decode_step");
    if (rc) return rc;
    if (!next) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "decode_step: null output");
    int seq = 0;
    return feed_rows(1, &seq, &token, true, next);
}

int32_t Engine::prefill(const uint32_t* tokens, int32_t n) {
    int32_t rc = check_ready("prefill");
    if (rc) return rc;
    if (!tokens || n <= 0) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "Prompt tokens must not be empty");
    if ((rc = reset())) return rc;
    // the prompt is processed in chunks of rows that share sequence 0 at consecutive positions
    const int chunk = std::min(max_rows_, tc_ready_ ? kPrefillRows : 8);
    std::vector<int> seq(chunk, 0);
    for (int i = 0; i < n; i += chunk) {
        int c = std::min(chunk, n - i);
        if ((rc = feed_rows(c, seq.data(), tokens + i, false, nullptr))) return rc;
        if (c > 1)  // the last row's hidden state is the sequence's lastHidden
            ESP_CUDA_TRY(cudaMemcpyAsync(act_.hidden, act_.hidden + (size_t)(c - 1) * m_.d_model, sizeof(float) * m_.d_model,
                                         cudaMemcpyDeviceToDevice, stream_));
    }
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    return ESP_CUDA_OK;
}

int32_t Engine::select_greedy(uint32_t* token) {
    int32_t rc = check_ready("select_greedy");
    if (rc) return rc;
    if (!token) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "select_greedy: null output");
    int seq = 0, pos = h_visible_[0];
    if ((rc = upload_rows(1, &seq, &pos, nullptr, nullptr, nullptr, true))) return rc;
    if ((rc = submit(1, STEP_HEAD))) return rc;
    ESP_CUDA_TRY(cudaMemcpyAsync(h_next_, rs_.next, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream_));
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    *token = h_next_[0];
    return ESP_CUDA_OK;
}

int32_t Engine::get_logits(int32_t seq, float* out, int32_t vocab) {
    int32_t rc = check_ready("get_logits");
    if (rc) return rc;
    if (tp_size_ > 1) return fail(ESP_CUDA_ERR_STATE, "get_logits: a tensor-parallel rank holds only its vocabulary shard");
    if (!out || vocab != m_.vocab) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "get_logits: output must hold exactly vocab floats");
    if (seq < 0 || seq >= m_.n_seq) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "sequence index out of range");
    int rows = seq + 1;
    std::vector<int> s(rows), p(rows), a(rows, 0);
    for (int r = 0; r < rows; r++) { s[r] = r; p[r] = h_visible_[r]; }
    a[seq] = 1;
    if ((rc = upload_rows(rows, s.data(), p.data(), nullptr, a.data(), nullptr, true))) return rc;
    uint32_t saved = cfg_.flags;
    int saved_dbg = debug_layer_;
    cfg_.flags |= ESP_CUDA_FLAG_KEEP_LOGITS | ESP_CUDA_FLAG_NO_GRAPH;
    rc = launch_step(rows, STEP_HEAD, stream_, false);
    cfg_.flags = saved;
    debug_layer_ = saved_dbg;
    if (rc) return rc;
    ESP_CUDA_TRY(cudaMemcpyAsync(out, act_.logits + (size_t)seq * m_.vocab, sizeof(float) * m_.vocab, cudaMemcpyDeviceToHost, stream_));
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    return ESP_CUDA_OK;
}

int32_t Engine::checkpoint(int32_t* id) {
    int32_t rc = check_ready("checkpoint");
    if (rc) return rc;
    if (!id) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "checkpoint: null output");
    Checkpoint c;
    c.visible = h_visible_[0];
    if ((rc = dev_alloc(owned_, &c.hidden, (size_t)m_.d_model, false))) return rc;
    ESP_CUDA_TRY(cudaMemcpyAsync(c.hidden, act_.hidden, sizeof(float) * m_.d_model, cudaMemcpyDeviceToDevice, stream_));
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    checkpoints_.push_back(c);
    *id = (int32_t)checkpoints_.size() - 1;
    return ESP_CUDA_OK;
}

int32_t Engine::rollback(int32_t id) {
    int32_t rc = check_ready("rollback");
    if (rc) return rc;
    if (id < 0 || id >= (int32_t)checkpoints_.size() || checkpoints_[id].visible < 0)
        return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "rollback: unknown checkpoint");
    const Checkpoint& c = checkpoints_[id];
    if (c.visible > h_visible_[0]) return fail(ESP_CUDA_ERR_STATE, "rollback: checkpoint is ahead of the current state");
    ESP_CUDA_TRY(cudaMemcpyAsync(act_.hidden, c.hidden, sizeof(float) * m_.d_model, cudaMemcpyDeviceToDevice, stream_));
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    h_visible_[0] = c.visible;
    return ESP_CUDA_OK;
}

int32_t Engine::verify2(uint32_t current, uint32_t proposed, uint32_t* exact_next, uint32_t* exact_future) {
    int32_t rc = check_ready("verify2");
    if (rc) return rc;
    if (!exact_next || !exact_future) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "verify2: null output");
    if (h_visible_[0] + 2 > m_.max_seq) return fail(ESP_CUDA_ERR_OUT_OF_RANGE, "verify2: two positions do not fit in the context");
    if (current >= (uint32_t)vocab_global_ || proposed >= (uint32_t)vocab_global_) return fail(ESP_CUDA_ERR_OUT_OF_RANGE, "verify2: token is outside the vocabulary");
    if (spec_verify_ok()) {
        rc = run_spec_verify(current, proposed, exact_next, exact_future);
        if (rc == ESP_CUDA_OK) { pending_verify_ = 2; return rc; }
        if (rc != ESP_CUDA_ERR_STATE) return rc;  // ERR_STATE: the two-position working set does not fit; the row-wise path below
    }
    int saved = h_visible_[0];
    int seq[2] = {0, 0};
    uint32_t tok[2] = {current, proposed};
    uint32_t next[2];
    if ((rc = feed_rows(2, seq, tok, true, next))) return rc;
    h_visible_[0] = saved;  // nothing is visible until commit()
    pending_verify_ = 2;
    *exact_next = next[0];
    *exact_future = next[1];
    return ESP_CUDA_OK;
}

int32_t Engine::commit(int32_t steps) {
    int32_t rc = check_ready("commit");
    if (rc) return rc;
    if (pending_verify_ != 2) return fail(ESP_CUDA_ERR_STATE, "commit: no verified pair is pending");
    if (steps < 1 || steps > 2) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "commit: steps must be 1 or 2");
    if (steps == 2)
        ESP_CUDA_TRY(cudaMemcpyAsync(act_.hidden, act_.hidden + m_.d_model, sizeof(float) * m_.d_model, cudaMemcpyDeviceToDevice, stream_));
    // No host wait: the copy is ordered before the next pass on the engine's stream, and verify2 has already
    // waited for the pair's tokens.
    h_visible_[0] += steps;
    pending_verify_ = 0;
    return ESP_CUDA_OK;
}

int32_t Engine::prefill_batch(const uint32_t* tokens, int32_t n_seq, int32_t len) {
    int32_t rc = check_ready("prefill_batch");
    if (rc) return rc;
    if (!tokens || len <= 0) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "Prompt tokens must not be empty");
    if (n_seq < 1 || n_seq > cfg_.max_batch) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "n_seq exceeds max_batch");
    if ((rc = reset())) return rc;
    // Rows are filled sequence by sequence: a pass of the tensor-core path holds up to kPrefillRows consecutive
    // positions, long runs of one sequence first (every pass streams all the weights once, and runs of consecutive
    // positions are what the tiled attention kernel wants).  Without that path a pass is one position of every sequence.
    if (!tc_ready_) {
        std::vector<int> seq(n_seq);
        std::vector<uint32_t> tok(n_seq);
        for (int s = 0; s < n_seq; s++) seq[s] = s;
        for (int t = 0; t < len; t++) {
            for (int s = 0; s < n_seq; s++) tok[s] = tokens[(size_t)s * len + t];
            if ((rc = feed_rows(n_seq, seq.data(), tok.data(), false, nullptr))) return rc;
        }
        return ESP_CUDA_OK;
    }
    const int budget = std::min(max_rows_, kPrefillRows);
    if (!d_last_hidden_ && (rc = dev_alloc(owned_, &d_last_hidden_, (size_t)cfg_.max_batch * m_.d_model))) return rc;
    std::vector<int> seq;
    std::vector<uint32_t> tok;
    std::vector<std::pair<int, int>> ends;  // (row, sequence) of every sequence that ends in the pass being built
    auto flush = [&]() -> int32_t {
        if (seq.empty()) return ESP_CUDA_OK;
        int32_t r = feed_rows((int)seq.size(), seq.data(), tok.data(), false, nullptr);
        if (r) return r;
        for (auto& e : ends)  // the sequence's last hidden state, before the next pass overwrites the rows
            ESP_CUDA_TRY(cudaMemcpyAsync(d_last_hidden_ + (size_t)e.second * m_.d_model, act_.hidden + (size_t)e.first * m_.d_model, sizeof(float) * m_.d_model,
                                         cudaMemcpyDeviceToDevice, stream_));
        seq.clear(); tok.clear(); ends.clear();
        return ESP_CUDA_OK;
    };
    for (int s = 0; s < n_seq; s++) {
        int t = 0;
        while (t < len) {
            const int take = std::min(len - t, budget - (int)seq.size());
            for (int j = 0; j < take; j++) { seq.push_back(s); tok.push_back(tokens[(size_t)s * len + t + j]); }
            t += take;
            if (t == len) ends.emplace_back((int)seq.size() - 1, s);
            if ((int)seq.size() == budget && (rc = flush())) return rc;
        }
    }
    if ((rc = flush())) return rc;
    // row s must hold the last hidden state of sequence s (decode passes have one row per sequence)
    ESP_CUDA_TRY(cudaMemcpyAsync(act_.hidden, d_last_hidden_, sizeof(float) * (size_t)n_seq * m_.d_model, cudaMemcpyDeviceToDevice, stream_));
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    return ESP_CUDA_OK;
}

int32_t Engine::decode_step_batch(const uint32_t* tokens, int32_t n_seq, uint32_t* next) {
    int32_t rc = check_ready("decode_step_batch");
    if (rc) return rc;
    if (!tokens || !next) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "decode_step_batch: null argument");
    if (n_seq < 1 || n_seq > cfg_.max_batch) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "n_seq exceeds max_batch");
    std::vector<int> seq(n_seq);
    for (int s = 0; s < n_seq; s++) seq[s] = s;
    return feed_rows(n_seq, seq.data(), tokens, true, next);
}

// Greedy generation for n_seq prompts of equal length.  After the prefill the loop is driven entirely from
// the device: each step's head feeds its token back as the next step's input, so the host only enqueues
// graph launches (generateIncrementalExactCPULlama, Engine.swift:6349-6431, with the limits of :1419-1426).
int32_t Engine::generate_batch(const uint32_t* prompts, int32_t n_seq, int32_t n_prompt, int32_t max_tokens,
                               uint32_t* out_tokens, int32_t* n_out, esp_cuda_generation_result* result) {
    int32_t rc = check_ready("generate");
    if (rc) return rc;
    if (!prompts || !out_tokens || !n_out) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "generate: null argument");
    if (n_prompt <= 0) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "Prompt tokens must not be empty");
    if (max_tokens < 0) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "maxTokens must be >= 0");
    if (n_prompt >= m_.max_seq) {
        std::ostringstream os;
        os << "Prompt token count " << n_prompt << " exceeds model context " << m_.max_seq - 1;
        return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, os.str());
    }
    if (n_seq < 1 || n_seq > cfg_.max_batch) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "n_seq exceeds max_batch");
    for (int64_t i = 0; i < (int64_t)n_seq * n_prompt; i++)
        if (prompts[i] >= (uint32_t)vocab_global_) return fail(ESP_CUDA_ERR_OUT_OF_RANGE, "prompt token outside vocab");
    const int eff = std::min(max_tokens, m_.max_seq - n_prompt);
    if (result) { *result = esp_cuda_generation_result{}; result->prompt_tokens = n_prompt; }
    for (int s = 0; s < n_seq; s++) n_out[s] = 0;
    if (eff == 0) return ESP_CUDA_OK;

    auto t_start = std::chrono::steady_clock::now();
    if (n_seq == 1) rc = prefill(prompts, n_prompt);
    else rc = prefill_batch(prompts, n_seq, n_prompt);
    if (rc) return rc;
    auto t_prefill = std::chrono::steady_clock::now();
    double first_ms = 0.0;
    if ((rc = decode_loop(n_seq, eff, out_tokens, max_tokens, n_out, nullptr, &first_ms))) return rc;
    auto t_end = std::chrono::steady_clock::now();
    if (result) {
        auto ms = [](auto a, auto b) { return std::chrono::duration<double, std::milli>(b - a).count(); };
        int total = 0;
        bool eos = false;
        for (int s = 0; s < n_seq; s++) { total += n_out[s]; if (n_out[s] < eff) eos = true; }
        result->generated_tokens = total;
        result->prefill_ms = ms(t_start, t_prefill);
        result->first_token_latency_ms = first_ms;
        result->total_decode_ms = ms(t_prefill, t_end);
        result->tokens_per_second = total > 0 ? total / std::max(result->total_decode_ms / 1000.0, 1e-9) : 0.0;
        result->stopped_on_eos = eos ? 1 : 0;
    }
    return ESP_CUDA_OK;
}

// Device-driven greedy decode of up to `count` tokens for sequences 0..n_seq-1, continuing from the current
// state (ESPRuntimeSession.decode(count:), Sources/ESPRuntime/ESPRuntimeContracts.swift:5-13).  The first token
// comes from the head alone (the state already holds the last hidden vector); each later token is one forward
// step whose head feeds its result back on the device, so the host only enqueues graph launches.
int32_t Engine::decode_loop(int32_t n_seq, int32_t count, uint32_t* out_tokens, int32_t out_stride, int32_t* n_out,
                            float* device_ms, double* first_token_ms) {
    int32_t rc = check_ready("decode");
    if (rc) return rc;
    if (n_seq < 1 || n_seq > cfg_.max_batch) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "n_seq exceeds max_batch");
    if (count < 0 || (out_tokens && out_stride < count)) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "decode: bad count");
    std::vector<int> seq(n_seq), pos(n_seq), lim(n_seq);
    int max_lim = 0;
    for (int s = 0; s < n_seq; s++) {
        if (h_visible_[s] <= 0) return fail(ESP_CUDA_ERR_STATE, "decode: sequence has no prefilled tokens");
        seq[s] = s; pos[s] = h_visible_[s];
        lim[s] = std::max(0, std::min(count, m_.max_seq - h_visible_[s]));
        max_lim = std::max(max_lim, lim[s]);
        if (n_out) n_out[s] = 0;
    }
    if (max_lim == 0) { if (device_ms) *device_ms = 0.f; return ESP_CUDA_OK; }
    if (mega_ready_ && n_seq == 1 && debug_layer_ < 0 && !(cfg_.flags & (ESP_CUDA_FLAG_NO_MEGAKERNEL | ESP_CUDA_FLAG_NO_GRAPH))) {
        int emitted = 0;
        if ((rc = run_mega(lim[0], &emitted, device_ms, first_token_ms))) return rc;
        if (n_out) n_out[0] = emitted;
        if (out_tokens) ESP_CUDA_TRY(cudaMemcpy(out_tokens, rs_.out, sizeof(uint32_t) * emitted, cudaMemcpyDeviceToHost));
        return ESP_CUDA_OK;
    }
    std::vector<int> active(n_seq);
    for (int s = 0; s < n_seq; s++) active[s] = lim[s] > 0;
    if ((rc = upload_rows(n_seq, seq.data(), pos.data(), nullptr, active.data(), lim.data(), true))) return rc;
    if (!ev_begin_) { ESP_CUDA_TRY(cudaEventCreate(&ev_begin_)); ESP_CUDA_TRY(cudaEventCreate(&ev_end_)); }
    auto t0 = std::chrono::steady_clock::now();
    ESP_CUDA_TRY(cudaEventRecord(ev_begin_, stream_));
    while ((int)step_events_.size() < max_lim) { cudaEvent_t ev; ESP_CUDA_TRY(cudaEventCreate(&ev)); step_events_.push_back(ev); }
    if ((rc = submit(n_seq, STEP_HEAD | STEP_FEEDBACK))) return rc;
    ESP_CUDA_TRY(cudaEventRecord(step_events_[0], stream_));  // one event per token: the per-token latencies
    if (first_token_ms) {
        ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
        *first_token_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    }
    const bool may_stop_early = m_.arch == ARCH_GPT2 || m_.eos_token >= 0;
    int steps_submitted = 1;
    for (int i = 1; i < max_lim; i++) {
        if ((rc = submit(n_seq, STEP_FORWARD | STEP_HEAD | STEP_FEEDBACK))) return rc;
        ESP_CUDA_TRY(cudaEventRecord(step_events_[i], stream_));
        steps_submitted = i + 1;
        if (may_stop_early && (i % 32) == 0) {
            ESP_CUDA_TRY(cudaMemcpyAsync(h_rows_block_ + 3 * max_rows_, rs_.active, sizeof(int) * n_seq, cudaMemcpyDeviceToHost, stream_));
            ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
            bool any = false;
            for (int s = 0; s < n_seq; s++) any |= h_rows_block_[3 * max_rows_ + s] != 0;
            if (!any) break;
        }
    }
    ESP_CUDA_TRY(cudaEventRecord(ev_end_, stream_));
    timings_.kernel_launches = launches_by_key_.count(n_seq * 16 + (STEP_HEAD | STEP_FEEDBACK)) ? launches_by_key_[n_seq * 16 + (STEP_HEAD | STEP_FEEDBACK)] : 1;
    if (max_lim > 1) timings_.kernel_launches += (max_lim - 1) * launches_last_step_;
    ESP_CUDA_TRY(cudaMemcpyAsync(h_rows_block_, d_rows_block_, sizeof(int) * 6 * max_rows_, cudaMemcpyDeviceToHost, stream_));
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    if (tc_ready_ && (n_seq >= kTcMinRows || tp_size_ > 1)) {  // bounded device waits report here
        int herr = 0;
        ESP_CUDA_TRY(cudaMemcpy(&herr, d_tc_error_, sizeof(int), cudaMemcpyDeviceToHost));
        if (herr) return fail(ESP_CUDA_ERR_TIMEOUT, herr == 8 ? "peer all-reduce gave up waiting for another rank" : "tensor-core GEMM gave up waiting on a barrier");
    }
    if (device_ms) ESP_CUDA_TRY(cudaEventElapsedTime(device_ms, ev_begin_, ev_end_));
    latencies_ms_.clear();
    {
        const int n0 = std::min(std::min(h_rows_block_[4 * max_rows_], lim[0]), steps_submitted);
        cudaEvent_t prev = ev_begin_;
        for (int i = 0; i < n0; i++) {
            float t = 0.f;
            ESP_CUDA_TRY(cudaEventElapsedTime(&t, prev, step_events_[i]));
            latencies_ms_.push_back(t);
            prev = step_events_[i];
        }
    }
    for (int s = 0; s < n_seq; s++) {
        int n = std::min(h_rows_block_[4 * max_rows_ + s], lim[s]);
        if (n_out) n_out[s] = n;
        h_visible_[s] = h_rows_block_[max_rows_ + s];
        if (n > 0 && out_tokens)
            ESP_CUDA_TRY(cudaMemcpy(out_tokens + (size_t)s * out_stride, rs_.out + (size_t)s * out_stride_, sizeof(uint32_t) * n, cudaMemcpyDeviceToHost));
    }
    return ESP_CUDA_OK;
}

// ---------------------------------------------------------------------------------------------- tensor parallelism

int32_t tp_unique_id(uint8_t* out, int32_t capacity) {
    NcclApi& api = nccl_api();
    if (!api.ok) return fail(ESP_CUDA_ERR_NCCL, "libnccl.so.2 could not be loaded");
    if (!out || capacity < (int32_t)sizeof(ncclUniqueId)) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "tp_unique_id: need 128 bytes");
    ncclUniqueId id;
    ncclResult_t r = api.GetUniqueId(&id);
    if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
    memcpy(out, &id, sizeof id);
    return ESP_CUDA_OK;
}

int32_t Engine::tp_init(const uint8_t* unique_id, int32_t nbytes) {
    if (tp_size_ <= 1) return fail(ESP_CUDA_ERR_STATE, "tp_init: the engine was created with tp_size <= 1");
    if (nccl_comm_) return fail(ESP_CUDA_ERR_STATE, "tp_init: already initialised");
    NcclApi& api = nccl_api();
    if (!api.ok) return fail(ESP_CUDA_ERR_NCCL, "libnccl.so.2 could not be loaded");
    if (!unique_id || nbytes != (int32_t)sizeof(ncclUniqueId)) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "tp_init: the unique id is 128 bytes");
    ESP_CUDA_TRY(cudaSetDevice(cfg_.device));
    ncclUniqueId id;
    memcpy(&id, unique_id, sizeof id);
    ncclComm_t comm = nullptr;
    ncclResult_t r = api.CommInitRank(&comm, tp_size_, id, tp_rank_);
    if (r != ncclSuccess) return nccl_fail(r, "ncclCommInitRank");
    nccl_comm_ = comm;
    return ESP_CUDA_OK;
}

// ---- all-reduce over peer memory (NVLink loads and stores; no multicast, no library kernel touches a peer) ----
// Exchange block of a rank: [partial buffer 0][partial buffer 1][arrival flags: one uint32 per rank].
// One all-reduce = one launch per rank: announce "my partial n is complete" in every peer's flag array, wait (bounded)
// until every peer has announced n, then read the peers' partials and add them in rank order (the same order on every
// rank, so all ranks hold bit-identical sums and keep choosing the same tokens).  Buffers alternate: a rank may
// overwrite buffer n%2 for all-reduce n+2 only after it passed the wait of n+1, which every peer reaches after it has
// finished reading n.  An even number of all-reduces per decode step keeps the parity of a captured graph fixed.
constexpr unsigned kTpSpinLimit = 1u << 22;  // a couple of seconds of polling

struct TpSumArgs {
    const float* partial[8];     // every rank's current partial buffer (own one included), index = rank
    unsigned int* peer_flags[8]; // every rank's arrival flags
    unsigned int* my_flags;
    unsigned int* epoch;         // [0] completed all-reduces, [1] CTA ticket (local)
    unsigned long long* stats;   // [0] all-reduces, [1] ns from this rank's arrival to its last sum, [2] ns of [1] spent waiting for the peers, [3] scratch
    float* out;                  // the residual stream: out += sum of the partials
    int world, rank, count4;
    int* error;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_peer_v4(const float* p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(256) k_tp_sum_peers(const TpSumArgs a) {
    pdl_launch_dependents();
    pdl_wait();  // this rank's partial (written by the previous kernels of the stream) is complete and visible
    __shared__ unsigned int s_epoch;
    if (threadIdx.x == 0) s_epoch = *reinterpret_cast<volatile unsigned int*>(a.epoch) + 1u;
    __syncthreads();
    const unsigned int epoch = s_epoch;
    const int p = threadIdx.x;
    unsigned long long t0 = 0;
    if (blockIdx.x == 0 && p == 0) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        a.stats[3] = t0;
    }
    if (p < a.world && p != a.rank) {
        if (blockIdx.x == 0) {
            __threadfence_system();
            st_release_sys(a.peer_flags[p] + a.rank, epoch);
        }
        unsigned spins = __ldcg(a.error) != 0 ? kTpSpinLimit : 0u;  // after a timeout nothing waits any more
        while ((int)(ld_acquire_sys(a.my_flags + p) - epoch) < 0) {  // peers may already be one all-reduce ahead
            if (++spins > kTpSpinLimit || ((spins & 0xfffu) == 0 && __ldcg(a.error) != 0)) {
                atomicCAS(a.error, 0, 8);
                break;
            }
        }
    }
    __syncthreads();
    if (blockIdx.x == 0 && p == 0) {
        unsigned long long t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        atomicAdd(a.stats + 2, t1 - t0);
    }
    // Every rank's 16 bytes are requested before the first addition: a peer load is a round trip over NVLink of a few
    // microseconds, and loads issued one after the other made an 8-rank sum take seven of them per element.
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < a.count4; i += gridDim.x * blockDim.x) {
        float4 v[8];
#pragma unroll
        for (int r = 0; r < 8; r++) {
            v[r] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r < a.world) v[r] = r == a.rank ? __ldcg(reinterpret_cast<const float4*>(a.partial[r]) + i) : ld_peer_v4(a.partial[r] + (size_t)i * 4);
        }
        float4 acc = reinterpret_cast<const float4*>(a.out)[i];  // the residual, then rank order: the same sum, bit for bit, on every rank
#pragma unroll
        for (int r = 0; r < 8; r++) {
            if (r < a.world) { acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w; }
        }
        reinterpret_cast<float4*>(a.out)[i] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(a.epoch + 1, 1u);
        if (t == gridDim.x - 1) {  // last CTA: this all-reduce is complete on this rank
            __threadfence();
            unsigned long long t2;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t2));
            atomicAdd(a.stats + 1, t2 - *reinterpret_cast<volatile unsigned long long*>(a.stats + 3));
            atomicAdd(a.stats, 1ull);
            a.epoch[1] = 0u;
            *reinterpret_cast<volatile unsigned int*>(a.epoch) = epoch;
            __threadfence();
        }
    }
}

// SiLU(gate) * up over fp32 rows -> the 16-bit operand rows of the W2 product.  Used where the gate and up products are
// cut along K (a narrow tensor-parallel shard), so that their sums are complete only after the product kernel.
struct SwigluArgs {
    const float* gate;  // [rows][hidden]
    const float* up;
    uint16_t* dst;      // [rows][hidden]
    float* debug;       // optional fp32 capture of row 0
    int hidden, n4, bf16;
};
__global__ void __launch_bounds__(256) k_swiglu_rows(const SwigluArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < a.n4; i += gridDim.x * blockDim.x) {
        const float4 g = __ldcg(reinterpret_cast<const float4*>(a.gate) + i), u = __ldcg(reinterpret_cast<const float4*>(a.up) + i);
        const float v0 = silu_fast(g.x) * u.x, v1 = silu_fast(g.y) * u.y, v2 = silu_fast(g.z) * u.z, v3 = silu_fast(g.w) * u.w;
        reinterpret_cast<uint2*>(a.dst)[i] = make_uint2(pack16x2(v0, v1, a.bf16), pack16x2(v2, v3, a.bf16));
        if (a.debug && 4 * i < a.hidden) *reinterpret_cast<float4*>(a.debug + 4 * i) = make_float4(v0, v1, v2, v3);
    }
}

// {all-reduces over peer memory, ns from arrival to the last sum, ns of that spent waiting for the peers} since the
// previous call (zeros when the group uses NCCL).
int32_t Engine::tp_sum_stats(unsigned long long* out3) {
    out3[0] = out3[1] = out3[2] = 0;
    if (!tp_peer_ready_ || !tp_stats_) return ESP_CUDA_OK;
    ESP_CUDA_TRY(cudaSetDevice(cfg_.device));
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    ESP_CUDA_TRY(cudaMemcpy(out3, tp_stats_, 3 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    ESP_CUDA_TRY(cudaMemset(tp_stats_, 0, 3 * sizeof(unsigned long long)));
    return ESP_CUDA_OK;
}

float* Engine::tp_current_partial() const {
    if (!tp_peer_ready_) return tp_partial_;
    return reinterpret_cast<float*>(tp_block_) + (size_t)tp_parity_ * tp_buf_floats_;
}

// Collective: every rank calls it once (from finalize).  On any failure the engine keeps the NCCL all-reduce.
// Collective: every rank runs the same two NCCL calls (handle exchange, vote) whatever happens locally, so a rank whose
// allocation or mapping fails cannot leave the others blocked inside a collective; one failure makes the whole group
// fall back to NCCL all-reduces.
int32_t Engine::tp_peer_setup() {
    tp_peer_ready_ = false;
    if (tp_size_ <= 1 || tp_size_ > 8 || !nccl_comm_ || getenv("ESP_CUDA_TP_NCCL_ONLY")) return ESP_CUDA_OK;
    NcclApi& api = nccl_api();
    if (!api.AllGather) return ESP_CUDA_OK;
    tp_buf_floats_ = ((size_t)max_rows_ * m_.d_model + 63) / 64 * 64;
    const size_t block_bytes = 2 * tp_buf_floats_ * sizeof(float) + 256;
    bool ok = true;  // this rank's part worked so far
    cudaIpcMemHandle_t mine{};
    if (cudaMalloc(reinterpret_cast<void**>(&tp_block_), block_bytes) != cudaSuccess) { cudaGetLastError(); tp_block_ = nullptr; ok = false; }
    if (ok && cudaMemset(tp_block_, 0, block_bytes) != cudaSuccess) { cudaGetLastError(); ok = false; }
    if (ok && dev_alloc(owned_, &tp_epoch_, 2) != ESP_CUDA_OK) ok = false;
    if (ok && dev_alloc(owned_, &tp_stats_, 4) != ESP_CUDA_OK) ok = false;
    if (ok && cudaIpcGetMemHandle(&mine, tp_block_) != cudaSuccess) { cudaGetLastError(); ok = false; }
    // exchange of the handles (a rank that failed sends zeros; nobody maps anything unless every rank voted "ok")
    uint8_t* d_handles = nullptr;
    ESP_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&d_handles), sizeof(mine) * (size_t)(tp_size_ + 1) + 16));
    std::vector<cudaIpcMemHandle_t> all((size_t)tp_size_);
    cudaError_t e = cudaMemcpy(d_handles + sizeof(mine) * tp_size_, &mine, sizeof(mine), cudaMemcpyHostToDevice);
    ncclResult_t r = api.AllGather(d_handles + sizeof(mine) * tp_size_, d_handles, sizeof(mine), ncclInt8, static_cast<ncclComm_t>(nccl_comm_), stream_);
    if (e == cudaSuccess && r == ncclSuccess) e = cudaStreamSynchronize(stream_);
    if (e == cudaSuccess && r == ncclSuccess) e = cudaMemcpy(all.data(), d_handles, sizeof(mine) * tp_size_, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess || r != ncclSuccess) ok = false;
    // first vote: did every rank export a block?
    auto vote = [&](bool mine_ok, bool* all_ok) -> int32_t {
        unsigned long long h = mine_ok ? 0ull : 1ull;  // max over ranks of "failed"
        unsigned long long* d_in = nullptr;
        ESP_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&d_in), 16));
        cudaError_t ce = cudaMemcpy(d_in, &h, 8, cudaMemcpyHostToDevice);
        ncclResult_t nr = api.AllReduce(d_in, d_in + 1, 1, ncclUint64, ncclMax, static_cast<ncclComm_t>(nccl_comm_), stream_);
        if (ce == cudaSuccess && nr == ncclSuccess) ce = cudaStreamSynchronize(stream_);
        if (ce == cudaSuccess && nr == ncclSuccess) ce = cudaMemcpy(&h, d_in + 1, 8, cudaMemcpyDeviceToHost);
        cudaFree(d_in);
        if (nr != ncclSuccess) return nccl_fail(nr, "ncclAllReduce");
        ESP_CUDA_TRY(ce);
        *all_ok = h == 0ull;
        return ESP_CUDA_OK;
    };
    bool everyone = false;
    int32_t rc = vote(ok, &everyone);
    cudaFree(d_handles);
    if (rc) return rc;
    if (everyone) {
        for (int p = 0; p < tp_size_; p++) {
            if (p == tp_rank_) { tp_peer_block_[p] = tp_block_; continue; }
            void* ptr = nullptr;
            if (cudaIpcOpenMemHandle(&ptr, all[(size_t)p], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); ok = false; break; }
            tp_peer_block_[p] = static_cast<uint8_t*>(ptr);
        }
    }
    // second vote: one rank that could not map a peer makes everybody fall back
    bool mapped = false;
    if ((rc = vote(ok && everyone, &mapped))) return rc;
    tp_peer_ready_ = mapped;
    tp_parity_ = 0;
    return ESP_CUDA_OK;
}

int32_t Engine::tp_sum_peers(float* out, int rows, cudaStream_t s) {
    TpSumArgs a{};
    for (int p = 0; p < tp_size_; p++) {
        a.partial[p] = reinterpret_cast<const float*>(tp_peer_block_[p]) + (size_t)tp_parity_ * tp_buf_floats_;
        a.peer_flags[p] = reinterpret_cast<unsigned int*>(tp_peer_block_[p] + 2 * tp_buf_floats_ * sizeof(float));
    }
    a.my_flags = a.peer_flags[tp_rank_];
    a.epoch = tp_epoch_;
    a.stats = tp_stats_;
    a.out = out;
    a.world = tp_size_; a.rank = tp_rank_;
    a.count4 = rows * m_.d_model / 4;
    a.error = d_tc_error_;
    const int grid = std::max(1, std::min(4 * sm_count_, (a.count4 + 255) / 256));  // one element per thread up to four CTAs per SM
    ESP_CUDA_TRY(launch_pdl(k_tp_sum_peers, dim3(grid), dim3(256), 0, s, a));
    tp_parity_ ^= 1;
    return ESP_CUDA_OK;
}

// sum of fp32 vectors, or maximum of packed 64-bit argmax keys
int32_t Engine::all_reduce(const void* send, void* recv, size_t count, bool sum_f32, cudaStream_t s) {
    NcclApi& api = nccl_api();
    ncclResult_t r = api.AllReduce(send, recv, count, sum_f32 ? ncclFloat32 : ncclUint64, sum_f32 ? ncclSum : ncclMax,
                                   static_cast<ncclComm_t>(nccl_comm_), s);
    if (r != ncclSuccess) return nccl_fail(r, "ncclAllReduce");
    return ESP_CUDA_OK;
}

// ---------------------------------------------------------------------------------------------- batched tensor-core path

int32_t Engine::build_tc() {
    tc_ready_ = false;
    if (max_rows_ > kPrefillRows) return ESP_CUDA_OK;
    if (m_.d_model % 64 || m_.q_dim % 64 || m_.hidden % 64 || m_.kv_dim % 16) return ESP_CUDA_OK;
    const int t0 = tensors_.at("lm_head").type;
    if (t0 != ESP_CUDA_F16 && t0 != ESP_CUDA_BF16 && t0 != ESP_CUDA_Q8_0 && t0 != ESP_CUDA_Q4_0) return ESP_CUDA_OK;
    std::vector<std::string> mats = {"lm_head"};
    for (int l = 0; l < m_.n_layer; l++)
        for (const char* n : {"wq", "wk", "wv", "wo", "w1", "w2", "w3"}) {
            if (m_.arch == ARCH_GPT2 && std::string(n) == "w3") continue;
            mats.push_back("layers/" + std::to_string(l) + "/" + n);
        }
    const bool quantised = t0 == ESP_CUDA_Q8_0 || t0 == ESP_CUDA_Q4_0;
    for (auto& n : mats) {
        const int t = tensors_.at(n).type;
        if (quantised ? (t != ESP_CUDA_Q8_0 && t != ESP_CUDA_Q4_0) : t != t0) return ESP_CUDA_OK;
    }
    if (quantised && (cfg_.flags & ESP_CUDA_FLAG_NO_TC_SHADOW)) return ESP_CUDA_OK;
    tc_bf16_ = t0 == ESP_CUDA_BF16;
    tc_mats_ = mats;
    tc_operands_ready_ = false;
    // 16-bit matrices get their TMA maps now.  A quantised model's fp16 expansion (what batches and prefill chunks
    // multiply by) is built by the first step that takes the batched path: an engine that only ever decodes one
    // sequence through the persistent kernel, which streams the GGUF blocks themselves, never allocates it.
    if (!quantised) {
        int32_t rc0 = tc_operands();
        if (rc0) return rc0;
    }
    tc_rows_alloc_ = (max_rows_ + 15) / 16 * 16;
    int32_t rc;
    if ((rc = dev_alloc(owned_, &xh_d_, (size_t)tc_rows_alloc_ * m_.d_model))) return rc;
    if ((rc = dev_alloc(owned_, &xh_q_, (size_t)tc_rows_alloc_ * m_.q_dim))) return rc;
    if ((rc = dev_alloc(owned_, &xh_h_, (size_t)tc_rows_alloc_ * m_.hidden))) return rc;
    if ((rc = dev_alloc(owned_, &kraw_, (size_t)max_rows_ * m_.kv_dim))) return rc;
    if ((rc = dev_alloc(owned_, &vraw_, (size_t)max_rows_ * m_.kv_dim))) return rc;
    if ((rc = dev_alloc(owned_, &up_, (size_t)max_rows_ * m_.hidden))) return rc;
    if ((rc = dev_alloc(owned_, &d_tc_error_, 4))) return rc;
    if (tp_size_ > 1 && (rc = dev_alloc(owned_, &tp_partial_, (size_t)max_rows_ * m_.d_model))) return rc;
    ESP_CUDA_TRY(cudaDeviceSynchronize());
    tc_ready_ = true;
    return ESP_CUDA_OK;
}

// TMA maps of the weight matrices for the batched path; for a quantised model first the fp16 expansion fp16(d * q) of
// every matrix.  Called outside stream capture (it allocates).
int32_t Engine::tc_operands() {
    if (tc_operands_ready_) return ESP_CUDA_OK;
    for (auto& n : tc_mats_) {
        DeviceTensor& t = tensors_.at(n);
        const void* base = t.data;
        if (t.type == ESP_CUDA_Q8_0 || t.type == ESP_CUDA_Q4_0) {
            const int64_t nb = (int64_t)t.rows * t.cols / 32;
            int32_t rc = dev_alloc(owned_, &t.shadow16, (size_t)t.rows * t.cols, false);
            if (rc) return rc;
            k_expand_quant<<<(unsigned)((nb * 4 + 255) / 256), 256, 0, stream_>>>(t.data, t.scales, t.type == ESP_CUDA_Q8_0 ? WT_Q8_0 : WT_Q4_0, nb, t.shadow16);
            ESP_CUDA_TRY(cudaGetLastError());
            base = t.shadow16;
        }
        int32_t rc = tc_make_map(&t.map, base, tc_bf16_, t.rows, t.cols, kTcHalf);
        if (rc) return rc;
        t.has_map = true;
    }
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    tc_operands_ready_ = true;
    return ESP_CUDA_OK;
}

const CUtensorMap* Engine::activation_map(const uint16_t* buf, int K, int tile) {
    auto key = std::make_pair(static_cast<const void*>(buf), tile);
    auto it = act_maps_.find(key);
    if (it == act_maps_.end()) {
        CUtensorMap m;
        if (tc_make_map(&m, buf, tc_bf16_, tc_rows_alloc_, K, tile)) return nullptr;
        it = act_maps_.emplace(key, m).first;
    }
    return &it->second;
}

// One pass over the model for `rows` rows with the matrix products on the tensor cores: every weight matrix is
// streamed once per pass whatever the row count.
int32_t Engine::launch_step_tc(int rows, int mode, cudaStream_t s) {
    const bool gpt2 = m_.arch == ARCH_GPT2;
    if (!tc_tile_for(rows)) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "too many rows for one tensor-core pass");
    tp_parity_ = 0;  // a step holds an even number of all-reduces: every step starts on partial buffer 0
    int launches = 0;
    float* dbg = debug_layer_ >= 0 ? d_debug_ : nullptr;
    const int q = m_.q_dim, kv = m_.kv_dim, d = m_.d_model, h = m_.hidden;
    auto tiles_of = [](int M) { return (M + kTcHalf - 1) / kTcHalf; };
    auto prep = [&](const float* src, int K, int norm, const float* g, const float* b, uint16_t* dst, bool from_emb, bool zero_qkv, bool zero_ffn = false,
                    float* zero_partial = nullptr) -> int32_t {
        PrepArgs p{};
        p.m = m_; p.rs = rs_; p.src = src; p.hidden_out = act_.hidden; p.K = K; p.norm = norm; p.g = g; p.b = b; p.dst = dst; p.bf16 = tc_bf16_;
        p.from_embedding = from_emb ? 1 : 0;
        if (from_emb) {
            const DeviceTensor& te = tensors_.at("embeddings/token");
            p.tok_emb = static_cast<const uint16_t*>(te.data);
            p.pos_emb = gpt2 ? static_cast<const uint16_t*>(tensors_.at("embeddings/position").data) : nullptr;
            p.emb_type = te.type == ESP_CUDA_BF16 ? WT_BF16 : WT_F16;
        }
        if (zero_qkv) {
            p.zero[0] = act_.q; p.zero_n[0] = q;
            p.zero[1] = kraw_; p.zero_n[1] = kv;
            p.zero[2] = vraw_; p.zero_n[2] = kv;
        }
        if (zero_ffn) {
            p.zero[0] = act_.act; p.zero_n[0] = h;
            p.zero[1] = up_; p.zero_n[1] = h;
        }
        if (zero_partial) { p.zero[3] = zero_partial; p.zero_n[3] = d; }
        ESP_CUDA_TRY(launch_pdl(k_prep_rows, dim3(rows), dim3(kThreads), 0, s, p));
        launches++;
        return ESP_CUDA_OK;
    };
    struct Part { const DeviceTensor* W; float* out; int ldo; const float* bias; };
    // one launch over up to three weight matrices that read the same operand rows
    auto gemm = [&](const TcPlan& plan, bool dual, std::initializer_list<Part> parts, const uint16_t* xbuf, int epi, uint16_t* out16, int ld16,
                    float* capture) -> int32_t {
        const int K = parts.begin()->W->cols;
        const CUtensorMap* mx = activation_map(xbuf, K, plan.x_rows);
        if (!mx) return fail(ESP_CUDA_ERR_CUDA, "tensor map missing for the batched path");
        TcArgs a{};
        const CUtensorMap* maps[3] = {&parts.begin()->W->map, &parts.begin()->W->map, &parts.begin()->W->map};
        int g = 0;
        for (const Part& pt : parts) {
            if (!pt.W->has_map || pt.W->cols != K) return fail(ESP_CUDA_ERR_CUDA, "tensor map missing for the batched path");
            maps[g] = &pt.W->map;
            a.g[g].M = pt.W->rows; a.g[g].out = pt.out; a.g[g].ldo = pt.ldo; a.g[g].bias = pt.bias;
            g++;
        }
        a.n_groups = dual ? 1 : g;
        a.K = K; a.n_valid = rows; a.epilogue = epi; a.active = rs_.active; a.error = d_tc_error_; a.bf16 = tc_bf16_;
        a.out16 = out16; a.ld16 = ld16; a.debug = capture;
        a.row_offset = epi == TC_HEAD ? tp_rank_ * m_.vocab : 0;
        if (epi == TC_HEAD) { a.best = rs_.best; a.logits = (cfg_.flags & ESP_CUDA_FLAG_KEEP_LOGITS) ? act_.logits : nullptr; }
        ESP_CUDA_TRY(tc_launch(plan, dual, maps, *mx, a, s));
        launches++;
        return ESP_CUDA_OK;
    };
    // hidden += W . x (+ bias).  Tensor parallel: W holds this rank's slice of the input dimension, so the product
    // is a partial sum; rank 0's partial also carries the residual and the bias, and one all-reduce leaves the
    // new residual stream on every rank.
    auto project = [&](const DeviceTensor& W, const uint16_t* xbuf, const float* bias) -> int32_t {
        const TcPlan plan = tc_plan(tiles_of(W.rows), rows, W.cols / kTcBlockK, true, false, sm_count_);
        if (tp_size_ <= 1) return gemm(plan, false, {{&W, act_.hidden, d, bias}}, xbuf, TC_RESIDUAL, nullptr, 0, nullptr);
        int32_t prc;
        float* partial = tp_current_partial();
        if (tp_peer_ready_) {
            // peer-memory sum: every rank's partial is the bare product (rank 0's carries the bias), cleared by the norm
            // kernel before it where K slices add into it; the sum kernel adds the partials to the residual stream
            if ((prc = gemm(plan, false, {{&W, partial, d, tp_rank_ == 0 ? bias : nullptr}}, xbuf, TC_STORE, nullptr, 0, nullptr))) return prc;
            launches++;
            return tp_sum_peers(act_.hidden, rows, s);
        }
        if (tp_rank_ == 0) {
            ESP_CUDA_TRY(cudaMemcpyAsync(partial, act_.hidden, sizeof(float) * (size_t)rows * d, cudaMemcpyDeviceToDevice, s));
            if ((prc = gemm(plan, false, {{&W, partial, d, bias}}, xbuf, TC_RESIDUAL, nullptr, 0, nullptr))) return prc;
        } else {
            if (plan.splits > 1) ESP_CUDA_TRY(cudaMemsetAsync(partial, 0, sizeof(float) * (size_t)rows * d, s));
            if ((prc = gemm(plan, false, {{&W, partial, d, nullptr}}, xbuf, TC_STORE, nullptr, 0, nullptr))) return prc;
        }
        return all_reduce(partial, act_.hidden, (size_t)rows * d, true, s);
    };
    auto copy_dbg = [&](const float* src, int offset, int n) {
        if (dbg) { k_copy_debug<<<(n + 255) / 256, 256, 0, s>>>(src, dbg + offset, n); launches++; }
    };
    // (row, head) pairs for every SM: one warp each (two below ~28 warps per SM); fewer: the split-KV kernel of the GEMV
    // path.  (Measured on 16 rows x 32 heads, contexts 128..384: 1.24 ms per step against 1.63 ms with the split-KV kernel
    // and its extra conversion pass.)
    const bool att_ok_hd = m_.head_dim == 32 || m_.head_dim == 64 || m_.head_dim == 128;
    // (a tensor-parallel rank holds 1/size of the heads: the choice follows the whole model's count, so that the ranks of a
    // group keep the kernel a single GPU would use)
    const bool att_rows = att_ok_hd && (long long)rows * m_.n_head * std::max(1, tp_size_) >= (long long)sm_count_;
    int32_t rc;
    if (mode & STEP_FORWARD) {
        const TcPlan plan_qkv = tc_plan(tiles_of(q) + 2 * tiles_of(kv), rows, d / kTcBlockK, true, false, sm_count_);
        const TcPlan plan_up = tc_plan(tiles_of(h), rows, d / kTcBlockK, false, !gpt2, sm_count_);
        // The fused gate/up product (activation in the epilogue) cannot be cut along K.  Where its weight tiles cover less
        // than half of the SMs (a narrow tensor-parallel shard, a small model) the rest would idle while each CTA streams
        // its tile at one SM's pace; there the two matrices run as a K-sliced grouped product into fp32 rows, and a small
        // kernel applies SiLU(gate) * up.
        const bool split_up = !gpt2 && 2 * tiles_of(h) * ((rows + kTcBatch - 1) / kTcBatch) <= sm_count_ && (h & 3) == 0;
        const TcPlan plan_up2 = tc_plan(2 * tiles_of(h), rows, d / kTcBlockK, true, false, sm_count_);
        for (int l = 0; l < m_.n_layer; l++) {
            const std::string pre = "layers/" + std::to_string(l) + "/";
            const LayerWeights lw = layer_weights(l);
            const bool cap = dbg && l == debug_layer_;
            if ((rc = prep(l == 0 ? nullptr : act_.hidden, d, gpt2 ? NORM_LAYER : NORM_RMS, lw.norm1_g, lw.norm1_b, xh_d_, l == 0, plan_qkv.splits > 1, false,
                           tp_peer_ready_ ? tp_current_partial() : nullptr)))
                return rc;
            if ((rc = gemm(plan_qkv, false,
                           {{&tensors_.at(pre + "wq"), act_.q, q, lw.bq}, {&tensors_.at(pre + "wk"), kraw_, kv, lw.bk}, {&tensors_.at(pre + "wv"), vraw_, kv, lw.bv}},
                           xh_d_, TC_STORE, nullptr, 0, nullptr)))
                return rc;
            RopeArgs ra{};
            ra.m = m_; ra.rs = rs_; ra.kv = kv_; ra.q = act_.q; ra.k_raw = kraw_; ra.v_raw = vraw_; ra.rope = gpt2 ? nullptr : d_rope_; ra.layer = l;
            ra.debug = cap ? dbg : nullptr;
            if (qk_norm_) { ra.q_norm = tensors_.at(pre + "q_norm").f32; ra.k_norm = tensors_.at(pre + "k_norm").f32; }
            ESP_CUDA_TRY(launch_pdl(k_rope_append, dim3(rows, (q / 2 + kv + kThreads - 1) / kThreads), dim3(kThreads), 0, s, ra));
            launches++;
            if ((mode & STEP_TILED_ATT) && att_ok_hd) {
                PrefillAttArgs pa{};
                pa.m = m_; pa.rs = rs_; pa.kv = kv_; pa.q = act_.q; pa.ctx16 = xh_q_; pa.bf16 = tc_bf16_; pa.layer = l; pa.rows = rows;
                pa.debug = cap ? dbg + q + 2 * kv : nullptr;
                const dim3 grid((rows + kPfRows - 1) / kPfRows, m_.n_head);
                if (m_.head_dim == 32) ESP_CUDA_TRY(launch_pdl(k_attention_prefill<32>, grid, dim3(kPfThreads), (size_t)pf_smem_bytes<32>(), s, pa));
                else if (m_.head_dim == 64) ESP_CUDA_TRY(launch_pdl(k_attention_prefill<64>, grid, dim3(kPfThreads), (size_t)pf_smem_bytes<64>(), s, pa));
                else ESP_CUDA_TRY(launch_pdl(k_attention_prefill<128>, grid, dim3(kPfThreads), (size_t)pf_smem_bytes<128>(), s, pa));
                launches++;
            } else if (att_rows) {
                AttRowsArgs ar{};
                ar.m = m_; ar.rs = rs_; ar.kv = kv_; ar.q = act_.q; ar.ctx16 = xh_q_; ar.bf16 = tc_bf16_; ar.layer = l; ar.rows = rows;
                ar.debug = cap ? dbg + q + 2 * kv : nullptr;
                const dim3 grid((rows * m_.n_head + kAttRowsWarps - 1) / kAttRowsWarps);
                // few (row, head) pairs (less than ~28 warps per SM): two warps per pair, on alternate position blocks
                const bool split2 = m_.n_head % kAttRowsWarps == 0 && (long long)rows * m_.n_head < 28LL * sm_count_;
                const dim3 block(kAttRowsWarps * 32 * (split2 ? 2 : 1));
#define ESP_ATT(HDV)                                                                                             \
    do {                                                                                                         \
        if (split2) ESP_CUDA_TRY(launch_pdl(k_attention_rows<HDV, 2>, grid, block, 0, s, ar));                   \
        else ESP_CUDA_TRY(launch_pdl(k_attention_rows<HDV, 1>, grid, block, 0, s, ar));                          \
    } while (0)
                if (m_.head_dim == 32) ESP_ATT(32);
                else if (m_.head_dim == 64) ESP_ATT(64);
                else ESP_ATT(128);
#undef ESP_ATT
                launches++;
            } else {
                AttArgs aa{};
                aa.m = m_; aa.layer = l; aa.rows = rows; aa.n_splits = n_splits_; aa.rs = rs_; aa.a = act_; aa.kv = kv_;
                aa.a.logits = nullptr; aa.a.debug = cap ? dbg : nullptr; aa.a.debug_layer = debug_layer_;
                ESP_CUDA_TRY(launch_pdl(k_attention, dim3(m_.n_head, rows, n_splits_), dim3(kAttThreads), 0, s, aa));
                launches++;
                if ((rc = prep(act_.ctx, q, NORM_NONE, nullptr, nullptr, xh_q_, false, false))) return rc;
            }
            if ((rc = project(tensors_.at(pre + "wo"), xh_q_, lw.bo))) return rc;
            if (cap) copy_dbg(act_.hidden, 2 * q + 2 * kv, d);
            if ((rc = prep(act_.hidden, d, gpt2 ? NORM_LAYER : NORM_RMS, lw.norm2_g, lw.norm2_b, xh_d_, false, false, split_up && plan_up2.splits > 1,
                           tp_peer_ready_ ? tp_current_partial() : nullptr)))
                return rc;
            // up projection with the activation in the epilogue: GELU(w1 x + b1), or SiLU(w1 x) * (w3 x) from two accumulators
            float* capture = cap ? dbg + 2 * q + 2 * kv + d : nullptr;
            if (gpt2) {
                if ((rc = gemm(plan_up, false, {{&tensors_.at(pre + "w1"), nullptr, 0, lw.b1}}, xh_d_, TC_GELU16, xh_h_, h, capture))) return rc;
            } else if (split_up) {
                if ((rc = gemm(plan_up2, false, {{&tensors_.at(pre + "w1"), act_.act, h, nullptr}, {&tensors_.at(pre + "w3"), up_, h, nullptr}}, xh_d_, TC_STORE,
                               nullptr, 0, nullptr)))
                    return rc;
                SwigluArgs sa{};
                sa.gate = act_.act; sa.up = up_; sa.dst = xh_h_; sa.debug = capture; sa.hidden = h; sa.n4 = rows * h / 4; sa.bf16 = tc_bf16_;
                ESP_CUDA_TRY(launch_pdl(k_swiglu_rows, dim3(std::max(1, std::min(4 * sm_count_, (sa.n4 + 255) / 256))), dim3(256), 0, s, sa));
                launches++;
            } else if ((rc = gemm(plan_up, true, {{&tensors_.at(pre + "w1"), nullptr, 0, nullptr}, {&tensors_.at(pre + "w3"), nullptr, 0, nullptr}}, xh_d_,
                                  TC_SWIGLU16, xh_h_, h, capture)))
                return rc;
            if ((rc = project(tensors_.at(pre + "w2"), xh_h_, lw.b2))) return rc;
            if (cap) copy_dbg(act_.hidden, 2 * q + 2 * kv + d + h, d);
        }
    }
    GemvArgs fin{};
    fin.m = m_; fin.rows = rows; fin.rs = rs_;
    if (mode & STEP_HEAD) {
        if ((rc = prep(act_.hidden, d, gpt2 ? NORM_LAYER : NORM_RMS, tensors_.at(gpt2 ? "final_norm_gamma" : "rms_final").f32,
                       gpt2 ? tensors_.at("final_norm_beta").f32 : nullptr, xh_d_, false, false))) return rc;
        const DeviceTensor& lh = tensors_.at("lm_head");
        const TcPlan plan_head = tc_plan(tiles_of(lh.rows), rows, d / kTcBlockK, false, false, sm_count_);
        if ((rc = gemm(plan_head, false, {{&lh, nullptr, 0, nullptr}}, xh_d_, TC_HEAD, nullptr, 0, nullptr))) return rc;
        if (tp_size_ > 1 && (rc = all_reduce(rs_.best, rs_.best, (size_t)rows, false, s))) return rc;  // max of (value, ~index) keys
        fin.m.vocab = vocab_global_;
        fin.finalize_mode = ((mode & STEP_FEEDBACK) ? 1 : 0) | ((mode & STEP_FORWARD) ? 2 : 0);
        ESP_CUDA_TRY(launch_pdl(k_head_done, dim3(1), dim3(256), 0, s, fin));
        launches++;
    } else if (mode & STEP_FORWARD) {
        ESP_CUDA_TRY(launch_pdl(k_bump, dim3(1), dim3(64), 0, s, rs_, rows));
        launches++;
    }
    ESP_CUDA_TRY(cudaGetLastError());
    launches_last_step_ = launches;
    return ESP_CUDA_OK;
}

static int pad128(long long v) { return (int)((v + 127) / 128 * 128); }

// Carves the exchange arena of a persistent kernel for `np` token positions: every array starts on a cache line.
// Returns the words needed; with `a` != null (a->x_words = arena base) it also sets the pointers.
static size_t mega_arena_layout(const ModelDims& m, const MegaPlan& p, int np, MegaArgs* a) {
    auto line = [](size_t words) { return (words + kMegaLineWords - 1) / kMegaLineWords * kMegaLineWords; };
    size_t o = 0;
    const size_t x_at = o;   o += line((size_t)np * m.d_model);
    const size_t act_at = o; o += line((size_t)np * (p.act_wpc ? (size_t)p.n_cta * p.act_wpc : (size_t)m.hidden));
    const size_t mid_at = o; o += line((size_t)np * m.d_model);
    const size_t qkv_at = o; o += line((size_t)np * m.n_kv_head * 2 * p.group_items);
    const size_t cand_at = o; o += line((size_t)np * p.n_cta * kMegaCandStride);
    if (a) {
        unsigned long long* base = a->x_words;
        a->x_words = base + x_at; a->act_words = base + act_at; a->mid_sums = base + mid_at; a->qkv_words = base + qkv_at; a->cand_words = base + cand_at;
    }
    return o + kMegaLineWords;
}

template <int WT>
static const void* mega_kernel_of(int head_dim) {
    if (head_dim == 64) return reinterpret_cast<const void*>(&k_decode_mega<64, WT>);
    if (head_dim == 128) return reinterpret_cast<const void*>(&k_decode_mega<128, WT>);
    return reinterpret_cast<const void*>(&k_decode_mega<32, WT>);
}
static const void* mega_kernel_for(int head_dim, int wt) {
    if (wt == WT_Q8_0) return mega_kernel_of<WT_Q8_0>(head_dim);
    if (wt == WT_Q4_0) return mega_kernel_of<WT_Q4_0>(head_dim);
    return mega_kernel_of<WT_F16>(head_dim);
}

// Plans and packs the persistent decode kernel.  Every CTA owns a contiguous share of the rows of every matrix;
// the model qualifies when one item of every stage fits a ring slot and the ring fits shared memory.
int32_t Engine::build_mega() {
    mega_ready_ = false;
    if ((cfg_.flags & ESP_CUDA_FLAG_NO_MEGAKERNEL) || tp_size_ > 1) return ESP_CUDA_OK;
    if (m_.arch != ARCH_LLAMA || qk_norm_) return ESP_CUDA_OK;  // (the per-head q/k norm lives in the per-stage and batched kernels)
    if (m_.head_dim != 32 && m_.head_dim != 64 && m_.head_dim != 128) return ESP_CUDA_OK;
    if (m_.d_model % 32 || m_.hidden % 32 || m_.n_head > sm_count_ || m_.n_head > 255 || m_.vocab >= (1 << 24)) return ESP_CUDA_OK;
    // The layer matrices share one storage type (fp16, or GGUF Q8_0 / Q4_0 blocks, which travel through the ring as they
    // are); the LM head has that type or fp16.  Anything else is left to the per-stage kernels.
    auto type_of = [&](const std::string& name) { return tensors_.at(name).type; };
    const int wt_layer = type_of("layers/0/wq");
    const int wt_head = type_of("lm_head");
    if (wt_layer != ESP_CUDA_F16 && wt_layer != ESP_CUDA_Q8_0 && wt_layer != ESP_CUDA_Q4_0) return ESP_CUDA_OK;
    if (wt_head != wt_layer && wt_head != ESP_CUDA_F16) return ESP_CUDA_OK;
    if (tensors_.at("embeddings/token").type != ESP_CUDA_F16) return ESP_CUDA_OK;
    for (int l = 0; l < m_.n_layer; l++)
        for (const char* n : {"wq", "wk", "wv", "wo", "w1", "w2", "w3"})
            if (type_of("layers/" + std::to_string(l) + "/" + n) != wt_layer) return ESP_CUDA_OK;
    const bool quant = wt_layer != ESP_CUDA_F16 || wt_head != ESP_CUDA_F16;
    if (quant && (m_.d_model % 256 || m_.hidden % 256)) return ESP_CUDA_OK;  // chunk sizes must stay multiples of 16 bytes
    int coop = 0, smem_max = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, cfg_.device);
    cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, cfg_.device);
    if (!coop) return ESP_CUDA_OK;
    MegaPlan p{};
    // every CTA must own at least one FFN unit and one row of W2 (it then takes part in every all-to-all exchange)
    const int P = std::min(sm_count_, std::min(m_.d_model, m_.hidden));
    if (P < m_.n_head) return ESP_CUDA_OK;
    p.n_cta = P;
    p.qpk = m_.n_head / m_.n_kv_head;
    p.group_items = (p.qpk + 2) * m_.head_dim / 2;
    p.cph = std::max(1, std::min(std::min(P / m_.n_head, m_.d_model), p.group_items / p.qpk));
    p.gsize = p.cph * p.qpk;
    p.n_group_cta = p.cph * m_.n_head;
    p.s1_max = (p.group_items + p.gsize - 1) / p.gsize;
    p.rpb = (m_.d_model + p.cph - 1) / p.cph;
    p.hpc_max = (m_.hidden + P - 1) / P;
    p.dpc_max = (m_.d_model + P - 1) / P;
    p.vpc_max = (m_.vocab + P - 1) / P;
    // Exchange arrays: the activation vector gets cache lines per CTA when every reader can poll all of it in one round
    // (four 16-byte loads per consumer thread); the layer output stays compact (see mega_kernel.cuh).
    p.act_wpc = (p.hpc_max + kMegaLineWords - 1) / kMegaLineWords * kMegaLineWords;
    if (P * ((p.hpc_max + 1) / 2) > 4 * kMegaConsumers) p.act_wpc = 0;
    if (quant) p.act_wpc = 0;  // the int8 staging of Q8_0 works on whole blocks of consecutive elements (and the wide quantised models need two polling rounds anyway)
    p.wt_layer = wt_layer;
    p.wt_head = wt_head;
    p.row_bytes = mega_row_bytes(wt_layer, m_.d_model);
    p.down_row_bytes = mega_row_bytes(wt_layer, m_.hidden);
    p.wo_row_bytes = mega_row_bytes(wt_layer, m_.head_dim);
    p.head_row_bytes = mega_row_bytes(wt_head, m_.d_model);
    // a quantised row of head_dim columns is 68 / 36 / ... bytes: chunks of the Wo stage must hold a multiple of `wo_rows`
    // rows to stay multiples of 16 bytes
    const int wo_rows = wt_layer == ESP_CUDA_F16 ? 1 : std::max(1, 8 / (m_.head_dim / 32));
    if (p.rpb % wo_rows) return ESP_CUDA_OK;
    p.s1_bytes = pad128((long long)2 * p.s1_max * p.row_bytes);
    p.s2_bytes = pad128((long long)p.rpb * p.wo_row_bytes);
    p.s3a_bytes = pad128((long long)2 * p.hpc_max * p.row_bytes);
    p.s3b_bytes = pad128((long long)p.dpc_max * p.down_row_bytes);
    p.layer_bytes = (long long)p.s1_bytes + p.s2_bytes + p.s3a_bytes + p.s3b_bytes;
    p.head_bytes = pad128((long long)p.vpc_max * p.head_row_bytes);
    p.cta_bytes = p.layer_bytes * m_.n_layer + p.head_bytes;
    // ring slots of 48 KB (more when one item of a stage is larger); a stage slice travels as chunks of whole items,
    // at most kMegaChunkRows rows each (the products of a chunk are spread over the warps as 8-row tiles)
    const int item_max = std::max(2 * p.row_bytes, p.down_row_bytes);
    p.slot_bytes = pad128(std::max(48 * 1024, item_max));
    p.s1_ipc = std::max(1, std::min(std::min(p.s1_max, kMegaChunkRows / 2), p.slot_bytes / (2 * p.row_bytes)));
    p.s3a_ipc = std::max(1, std::min(std::min(p.hpc_max, kMegaChunkRows / 2), p.slot_bytes / (2 * p.row_bytes)));
    p.s3b_rpc = std::max(1, std::min(std::min(p.dpc_max, kMegaChunkRows), p.slot_bytes / p.down_row_bytes));
    p.head_rpc = std::max(1, std::min(std::min(p.vpc_max, kMegaChunkRows), p.slot_bytes / p.head_row_bytes));
    p.s2_rpc = std::max(1, std::min(std::min(p.rpb, kMegaChunkRows), p.slot_bytes / p.wo_row_bytes));
    p.s2_rpc = std::max(wo_rows, p.s2_rpc / wo_rows * wo_rows);
    p.n_slots = 0;
    for (int ns = 8; ns >= 2; ns--) {
        MegaPlan probe = p;
        probe.n_slots = ns;
        mega_layout(m_, probe);
        if (probe.smem_bytes <= smem_max) { p = probe; break; }
    }
    if (p.n_slots == 0) return ESP_CUDA_OK;  // does not fit: the per-stage kernels serve this model
    const void* kern = mega_kernel_for(m_.head_dim, wt_layer);
    ESP_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, p.smem_bytes));
    int occ = 0;
    ESP_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kMegaThreads, p.smem_bytes));
    if (occ < 1) return ESP_CUDA_OK;

    int32_t rc;
    if ((rc = dev_alloc(owned_, &d_pack_, (size_t)P * p.cta_bytes, false))) return rc;
    if ((rc = dev_alloc(owned_, &d_norms_, (size_t)(2 * m_.n_layer + 1) * m_.d_model, false))) return rc;
    // exchange arena: x words, activation words, q/k/v words per KV head, counted sums, arg-max candidates
    mega_arena_words_ = mega_arena_layout(m_, p, 1, nullptr);
    if ((rc = dev_alloc(owned_, &d_mega_arena_, mega_arena_words_))) return rc;
    if ((rc = dev_alloc(owned_, &d_mega_ctl_, 8))) return rc;
    if ((rc = dev_alloc(owned_, &d_mega_trace_, (size_t)kMegaTraceLayer * m_.n_layer + kMegaTraceHead + 4 + 1024))) return rc;
    if ((rc = dev_alloc(owned_, &d_token_times_, (size_t)m_.max_seq + 1))) return rc;
    ESP_CUDA_TRY(cudaMallocHost(reinterpret_cast<void**>(&h_mega_ctl_), 8 * sizeof(unsigned long long)));
    // per-layer source matrices
    std::vector<PackMatrix> mats((size_t)7 * m_.n_layer);
    const char* names[7] = {"wq", "wk", "wv", "wo", "w1", "w2", "w3"};
    for (int k = 0; k < 7; k++)
        for (int l = 0; l < m_.n_layer; l++) {
            const DeviceTensor& t = tensors_.at("layers/" + std::to_string(l) + "/" + names[k]);
            mats[(size_t)k * m_.n_layer + l] = PackMatrix{t.data, t.scales};
        }
    PackMatrix* d_mats = nullptr;
    ESP_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&d_mats), mats.size() * sizeof(PackMatrix)));
    cudaError_t e = cudaMemcpy(d_mats, mats.data(), mats.size() * sizeof(PackMatrix), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) {
        PackSources src{};
        src.wq = d_mats; src.wk = d_mats + m_.n_layer; src.wv = d_mats + 2 * m_.n_layer; src.wo = d_mats + 3 * m_.n_layer;
        src.w1 = d_mats + 4 * m_.n_layer; src.w2 = d_mats + 5 * m_.n_layer; src.w3 = d_mats + 6 * m_.n_layer;
        const DeviceTensor& lh = tensors_.at("lm_head");
        src.lm_head = PackMatrix{lh.data, lh.scales};
        k_build_pack<<<P, 256, 0, stream_>>>(src, p, m_, d_pack_);
        e = cudaGetLastError();
    }
    for (int l = 0; l < m_.n_layer && e == cudaSuccess; l++) {
        std::string pre = "layers/" + std::to_string(l) + "/";
        e = cudaMemcpyAsync(d_norms_ + (size_t)(2 * l) * m_.d_model, tensors_.at(pre + "rms_att").f32, sizeof(float) * m_.d_model, cudaMemcpyDeviceToDevice, stream_);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(d_norms_ + (size_t)(2 * l + 1) * m_.d_model, tensors_.at(pre + "rms_ffn").f32, sizeof(float) * m_.d_model, cudaMemcpyDeviceToDevice, stream_);
    }
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(d_norms_ + (size_t)(2 * m_.n_layer) * m_.d_model, tensors_.at("rms_final").f32, sizeof(float) * m_.d_model, cudaMemcpyDeviceToDevice, stream_);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream_);
    cudaFree(d_mats);
    ESP_CUDA_TRY(e);
    mega_plan_ = p;
    mega_ready_ = true;
    return ESP_CUDA_OK;
}

// Runs the greedy loop (at most n_steps emitted tokens; fewer when the end-of-sequence token comes up) of sequence 0
// as one cooperative launch.  *emitted receives the number of tokens written to rs_.out.
int32_t Engine::run_mega(int n_steps, int* emitted, float* device_ms, double* first_token_ms) {
    MegaArgs a{};
    const MegaPlan& p = mega_plan_;
    a.m = m_; a.plan = p; a.pack = d_pack_; a.norms = d_norms_;
    a.tok_emb = static_cast<const uint16_t*>(tensors_.at("embeddings/token").data);
    a.rope = d_rope_; a.kv = kv_; a.hidden_io = act_.hidden;
    a.x_words = d_mega_arena_;
    mega_arena_layout(m_, p, 1, &a);
    a.error = reinterpret_cast<int*>(d_mega_ctl_ + 2) + 1;
    a.stamps = d_mega_ctl_ + 3;
    a.rs = rs_;
    a.trace = d_mega_trace_;
    a.token_times = n_steps <= m_.max_seq + 1 ? d_token_times_ : nullptr;
    token_times_n_ = 0;
    a.trace_cta = std::min(mega_trace_cta_, p.n_cta - 1);
    a.n_steps = n_steps;
    a.pos0 = h_visible_[0];
    a.spin_limit = mega_spin_limit_;
    if (!ev_begin_) { ESP_CUDA_TRY(cudaEventCreate(&ev_begin_)); ESP_CUDA_TRY(cudaEventCreate(&ev_end_)); }
    ESP_CUDA_TRY(cudaMemsetAsync(d_mega_ctl_, 0, 8 * sizeof(unsigned long long), stream_));
    ESP_CUDA_TRY(cudaMemsetAsync(d_mega_arena_, 0, mega_arena_words_ * sizeof(unsigned long long), stream_));
    ESP_CUDA_TRY(cudaEventRecord(ev_begin_, stream_));
    void* args[] = {&a};
    ESP_CUDA_TRY(cudaLaunchCooperativeKernel(mega_kernel_for(m_.head_dim, p.wt_layer), dim3(p.n_cta), dim3(kMegaThreads), args, (size_t)p.smem_bytes, stream_));
    ESP_CUDA_TRY(cudaEventRecord(ev_end_, stream_));
    ESP_CUDA_TRY(cudaMemcpyAsync(h_mega_ctl_, d_mega_ctl_, 8 * sizeof(unsigned long long), cudaMemcpyDeviceToHost, stream_));
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    launches_last_step_ = 1;
    timings_.kernel_launches = 1;
    const int err = reinterpret_cast<int*>(h_mega_ctl_ + 2)[1];
    if (err != 0) {
        std::ostringstream os;
        os << "persistent decode kernel gave up waiting (code " << err
           << ": 3 = weight chunk, 4 = ring slot, 5/9 = layer output words, 6 = q/k/v words, 7 = attention sums, 8 = activation words, 10 = arg-max words)";
        return fail(ESP_CUDA_ERR_TIMEOUT, os.str());
    }
    const int n = (int)h_mega_ctl_[5];
    if (n < 1 || n > n_steps) return fail(ESP_CUDA_ERR_CUDA, "persistent decode kernel reported an impossible token count");
    if (emitted) *emitted = n;
    token_times_n_ = a.token_times ? n : 0;
    if (device_ms) ESP_CUDA_TRY(cudaEventElapsedTime(device_ms, ev_begin_, ev_end_));
    if (first_token_ms) *first_token_ms = (double)(h_mega_ctl_[4] - h_mega_ctl_[3]) / 1e6;
    latencies_ms_.clear();
    if (a.token_times) {
        std::vector<unsigned long long> tt((size_t)n);
        ESP_CUDA_TRY(cudaMemcpy(tt.data(), d_token_times_, sizeof(unsigned long long) * n, cudaMemcpyDeviceToHost));
        unsigned long long prev = h_mega_ctl_[3];  // kernel start
        for (int i = 0; i < n; i++) { latencies_ms_.push_back((float)((double)(tt[i] - prev) / 1e6)); prev = tt[i]; }
    }
    h_visible_[0] += n - 1;
    return ESP_CUDA_OK;
}

static const void* spec_kernel_for(int head_dim) {
    if (head_dim == 64) return reinterpret_cast<const void*>(&k_spec_mega<64>);
    if (head_dim == 128) return reinterpret_cast<const void*>(&k_spec_mega<128>);
    return reinterpret_cast<const void*>(&k_spec_mega<32>);
}

int32_t Engine::ensure_norms2() {
    if (d_norms2_) return ESP_CUDA_OK;
    const size_t d = (size_t)m_.d_model, rows = (size_t)2 * m_.n_layer + 1;
    int32_t rc;
    if ((rc = dev_alloc(owned_, &d_norms2_, rows * 2 * d, false))) return rc;
    for (int copy = 0; copy < 2; copy++)
        ESP_CUDA_TRY(cudaMemcpy2DAsync(d_norms2_ + copy * d, 2 * d * sizeof(float), d_norms_, d * sizeof(float), d * sizeof(float), rows, cudaMemcpyDeviceToDevice, stream_));
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    return ESP_CUDA_OK;
}

// The two-token kernel serves a target and a draft that are both fp16 Llama models on the persistent-kernel path, on one
// device, with the same widths: they then share one plan (chunk sizes, work shares, ring) and differ in depth only.
bool Engine::spec_compatible(const Engine& draft) const {
    if (!mega_ready_ || !draft.mega_ready_ || tp_size_ > 1 || draft.tp_size_ > 1) return false;
    if ((cfg_.flags | draft.cfg_.flags) & (ESP_CUDA_FLAG_NO_MEGAKERNEL | ESP_CUDA_FLAG_NO_GRAPH)) return false;
    if (debug_layer_ >= 0 || draft.debug_layer_ >= 0 || cfg_.device != draft.cfg_.device) return false;
    const MegaPlan &a = mega_plan_, &b = draft.mega_plan_;
    if (a.wt_layer != ESP_CUDA_F16 || a.wt_head != ESP_CUDA_F16 || b.wt_layer != ESP_CUDA_F16 || b.wt_head != ESP_CUDA_F16) return false;
    const ModelDims &x = m_, &y = draft.m_;
    if (x.d_model != y.d_model || x.n_head != y.n_head || x.n_kv_head != y.n_kv_head || x.head_dim != y.head_dim || x.hidden != y.hidden || x.vocab != y.vocab ||
        x.eps != y.eps || cfg_.rope_theta != draft.cfg_.rope_theta)
        return false;
    return a.n_cta == b.n_cta && a.cph == b.cph && a.slot_bytes == b.slot_bytes && a.s1_ipc == b.s1_ipc && a.s2_rpc == b.s2_rpc && a.s3a_ipc == b.s3a_ipc &&
           a.s3b_rpc == b.s3b_rpc && a.head_rpc == b.head_rpc && a.layer_bytes == b.layer_bytes;
}

int32_t Engine::spec_prepare() {
    if (spec_ready_) return ESP_CUDA_OK;
    int smem_max = 0;
    cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, cfg_.device);
    MegaPlan p = mega_plan_;
    p.n_slots = 0;
    for (int ns = mega_plan_.n_slots; ns >= 3; ns--) {  // a stage holds back one slot past its exchange: fewer than three would stall the ring
        MegaPlan probe = mega_plan_;
        probe.n_slots = ns;
        spec_layout(m_, probe);
        if (probe.smem_bytes <= smem_max) { p = probe; break; }
    }
    if (p.n_slots == 0) return fail(ESP_CUDA_ERR_STATE, "two-token kernel: the model's working set does not fit shared memory");
    if (kSpecNP * p.n_cta * ((p.hpc_max + 1) / 2) > 4 * kMegaConsumers) p.act_wpc = 0;  // two positions no longer fit one polling round
    const void* kern = spec_kernel_for(m_.head_dim);
    ESP_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, p.smem_bytes));
    int occ = 0;
    ESP_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kMegaThreads, p.smem_bytes));
    if (occ < 1) return fail(ESP_CUDA_ERR_STATE, "two-token kernel: no CTA fits an SM");
    int32_t rc;
    spec_arena_words_ = mega_arena_layout(m_, p, kSpecNP, nullptr);
    if ((rc = dev_alloc(owned_, &d_spec_arena_, spec_arena_words_))) return rc;
    if ((rc = dev_alloc(owned_, &d_spec_out_, (size_t)m_.max_seq + 2))) return rc;
    if ((rc = dev_alloc(owned_, &d_spec_result_, 16))) return rc;
    spec_plan_ = p;
    spec_ready_ = true;
    return ESP_CUDA_OK;
}

bool Engine::spec_verify_ok() const {
    if (!mega_ready_ || tp_size_ > 1 || debug_layer_ >= 0) return false;
    if (cfg_.flags & (ESP_CUDA_FLAG_NO_MEGAKERNEL | ESP_CUDA_FLAG_NO_GRAPH | ESP_CUDA_FLAG_KEEP_LOGITS)) return false;
    return mega_plan_.wt_layer == ESP_CUDA_F16 && mega_plan_.wt_head == ESP_CUDA_F16;
}

// verify2 as one launch: both positions share one pass over the weights (the second rides in spare columns of the
// tensor-core products).  Leaves both rows' hidden states in act_.hidden as the row-wise path does, for commit().
int32_t Engine::run_spec_verify(uint32_t current, uint32_t proposed, uint32_t* exact_next, uint32_t* exact_future) {
    int32_t rc;
    if ((rc = spec_prepare())) return rc;
    if ((rc = ensure_norms2())) return rc;
    const MegaPlan& p = spec_plan_;
    SpecArgs sa{};
    MegaArgs& a = sa.base;
    a.m = m_; a.plan = p; a.rope = d_rope_;
    a.x_words = d_spec_arena_;
    mega_arena_layout(m_, p, kSpecNP, &a);
    a.error = d_spec_result_ + 8;
    a.spin_limit = mega_spin_limit_;
    SpecModel& M = sa.model[1];
    M.m = m_; M.pack = d_pack_; M.cta_bytes = mega_plan_.cta_bytes; M.norms2 = d_norms2_;
    M.tok_emb = static_cast<const uint16_t*>(tensors_.at("embeddings/token").data);
    M.kv = kv_;
    sa.model[0] = M;
    sa.out = d_spec_out_;
    sa.result = d_spec_result_;
    sa.hidden_out = act_.hidden;
    sa.prev = current; sa.current = proposed;
    sa.pos = h_visible_[0];
    sa.gen0 = 0; sa.eff = 1; sa.max_seq = m_.max_seq; sa.eos_token = -1;
    sa.verify_only = 1;
    ESP_CUDA_TRY(cudaMemsetAsync(d_spec_result_, 0, 16 * sizeof(int), stream_));
    ESP_CUDA_TRY(cudaMemsetAsync(d_spec_arena_, 0, spec_arena_words_ * sizeof(unsigned long long), stream_));
    void* args[] = {&sa};
    ESP_CUDA_TRY(cudaLaunchCooperativeKernel(spec_kernel_for(m_.head_dim), dim3(p.n_cta), dim3(kMegaThreads), args, (size_t)p.smem_bytes, stream_));
    int h[16];
    ESP_CUDA_TRY(cudaMemcpyAsync(h, d_spec_result_, sizeof(h), cudaMemcpyDeviceToHost, stream_));
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    launches_last_step_ = 1;
    timings_.kernel_launches = 1;
    if (h[8] != 0) {
        std::ostringstream os;
        os << "two-position verify kernel gave up waiting (code " << h[8] << ")";
        return fail(ESP_CUDA_ERR_TIMEOUT, os.str());
    }
    *exact_next = (uint32_t)h[0];
    *exact_future = (uint32_t)h[1];
    return ESP_CUDA_OK;
}

int32_t Engine::run_spec(Engine& draft, uint32_t prev, uint32_t current, int gen0, int eff, int max_seq, uint32_t* out_tokens, int* stats) {
    int32_t rc;
    if (!spec_compatible(draft)) return fail(ESP_CUDA_ERR_STATE, "two-token kernel: draft and target do not share one plan");
    if (gen0 < 1 || eff <= gen0 || h_visible_[0] < 1 || h_visible_[0] + 1 >= max_seq) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "two-token kernel: nothing left to generate");
    if ((rc = spec_prepare())) return rc;
    if ((rc = ensure_norms2())) return rc;
    if ((rc = draft.ensure_norms2())) return rc;
    ESP_CUDA_TRY(cudaStreamSynchronize(draft.stream_));  // the draft's prefill ran on its own stream
    const MegaPlan& p = spec_plan_;
    SpecArgs sa{};
    MegaArgs& a = sa.base;
    a.m = m_; a.plan = p; a.rope = d_rope_;
    a.x_words = d_spec_arena_;
    mega_arena_layout(m_, p, kSpecNP, &a);
    a.error = d_spec_result_ + 8;
    a.spin_limit = mega_spin_limit_;
    Engine* eng[2] = {&draft, this};
    for (int i = 0; i < 2; i++) {
        SpecModel& M = sa.model[i];
        M.m = eng[i]->m_;
        M.pack = eng[i]->d_pack_;
        M.cta_bytes = eng[i]->mega_plan_.cta_bytes;
        M.norms2 = eng[i]->d_norms2_;
        M.tok_emb = static_cast<const uint16_t*>(eng[i]->tensors_.at("embeddings/token").data);
        M.kv = eng[i]->kv_;
    }
    sa.out = d_spec_out_;
    sa.result = d_spec_result_;
    sa.hidden_out = act_.hidden;
    sa.prev = prev; sa.current = current;
    sa.pos = h_visible_[0];
    sa.gen0 = gen0; sa.eff = eff; sa.max_seq = max_seq;
    sa.eos_token = m_.eos_token;
    ESP_CUDA_TRY(cudaMemsetAsync(d_spec_result_, 0, 16 * sizeof(int), stream_));
    ESP_CUDA_TRY(cudaMemsetAsync(d_spec_arena_, 0, spec_arena_words_ * sizeof(unsigned long long), stream_));
    void* args[] = {&sa};
    ESP_CUDA_TRY(cudaLaunchCooperativeKernel(spec_kernel_for(m_.head_dim), dim3(p.n_cta), dim3(kMegaThreads), args, (size_t)p.smem_bytes, stream_));
    int h[16];
    ESP_CUDA_TRY(cudaMemcpyAsync(h, d_spec_result_, sizeof(h), cudaMemcpyDeviceToHost, stream_));
    ESP_CUDA_TRY(cudaStreamSynchronize(stream_));
    launches_last_step_ = 1;
    timings_.kernel_launches = 1;
    if (h[8] != 0) {
        std::ostringstream os;
        os << "two-token kernel gave up waiting (code " << h[8] << ": 3 = weight chunk, 4 = ring slot, 5/9 = layer output words, 6 = q/k/v words, 7 = attention sums, 8 = activation words, 10 = arg-max words)";
        return fail(ESP_CUDA_ERR_TIMEOUT, os.str());
    }
    const int n = h[0];
    if (n <= gen0 || n > eff) return fail(ESP_CUDA_ERR_CUDA, "two-token kernel reported an impossible token count");
    ESP_CUDA_TRY(cudaMemcpy(out_tokens + gen0, d_spec_out_ + gen0, sizeof(uint32_t) * (size_t)(n - gen0), cudaMemcpyDeviceToHost));
    for (int i = 0; i < 5; i++) stats[i] = h[i];
    h_visible_[0] = h[5];
    draft.h_visible_[0] = h[6];
    pending_verify_ = 0;
    return ESP_CUDA_OK;
}

int32_t Engine::stage_trace(int32_t cta, long long* out, int32_t capacity, int32_t* n) {
    if (!out || !n) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "stage_trace: null argument");
    *n = 0;
    if (!mega_ready_) return ESP_CUDA_OK;
#ifdef MEGA_FINE_TRACE
    const int count = 1000;
#else
    const int count = kMegaTraceLayer * m_.n_layer + kMegaTraceHead;
#endif
    if (capacity < count) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "stage_trace: capacity too small");
    ESP_CUDA_TRY(cudaSetDevice(cfg_.device));
    ESP_CUDA_TRY(cudaMemcpy(out, d_mega_trace_, sizeof(long long) * count, cudaMemcpyDeviceToHost));
    *n = count;
    mega_trace_cta_ = std::max(0, std::min(cta, mega_plan_.n_cta - 1));  // takes effect with the next decode loop
    return ESP_CUDA_OK;
}

// Emission time (GPU global timer, ns) of every token of the most recent persistent decode loop: the per-token gaps
// the reference's CLI reports as median / p95 latency (Sources/EspressoGenerate/CLI.swift:1153-1165).
int32_t Engine::token_times(unsigned long long* out_ns, int32_t capacity, int32_t* n) {
    if (!out_ns || !n) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "token_times: null argument");
    *n = 0;
    if (!mega_ready_ || token_times_n_ <= 0) return ESP_CUDA_OK;
    if (capacity < token_times_n_) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "token_times: capacity too small");
    ESP_CUDA_TRY(cudaSetDevice(cfg_.device));
    ESP_CUDA_TRY(cudaMemcpy(out_ns, d_token_times_, sizeof(unsigned long long) * token_times_n_, cudaMemcpyDeviceToHost));
    *n = token_times_n_;
    return ESP_CUDA_OK;
}

int32_t Engine::token_latencies(float* out_ms, int32_t capacity, int32_t* n) {
    if (!out_ms || !n) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "token_latencies: null argument");
    *n = 0;
    if (capacity < (int32_t)latencies_ms_.size()) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "token_latencies: capacity too small");
    std::copy(latencies_ms_.begin(), latencies_ms_.end(), out_ms);
    *n = (int32_t)latencies_ms_.size();
    return ESP_CUDA_OK;
}

int32_t Engine::set_debug_layer(int32_t layer) {
    if (layer >= m_.n_layer) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "debug layer out of range");
    debug_layer_ = layer < 0 ? -1 : layer;
    return ESP_CUDA_OK;
}

int32_t Engine::debug_dump(int32_t stage, float* out, int32_t capacity) {
    int32_t rc = check_ready("debug_dump");
    if (rc) return rc;
    const int q = m_.q_dim, kv = m_.kv_dim, d = m_.d_model, h = m_.hidden;
    const int offs[7] = {0, q, q + kv, q + 2 * kv, 2 * q + 2 * kv, 2 * q + 2 * kv + d, 2 * q + 2 * kv + d + h};
    const int sizes[7] = {q, kv, kv, q, d, h, d};
    if (stage < 0 || stage > 6 || !out || capacity < sizes[stage]) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "debug_dump: bad stage or capacity");
    ESP_CUDA_TRY(cudaMemcpy(out, d_debug_ + offs[stage], sizeof(float) * sizes[stage], cudaMemcpyDeviceToHost));
    return ESP_CUDA_OK;
}

int32_t Engine::set_wait_limit(uint32_t spins) {
    mega_spin_limit_ = spins == 0 ? kMegaSpinLimit : spins;
    return ESP_CUDA_OK;
}

int32_t Engine::get_timings(esp_cuda_timings* out) {
    if (!out) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "get_timings: null output");
    *out = timings_;
    return ESP_CUDA_OK;
}

}  // namespace esp

// ---------------------------------------------------------------------------------------------- stand-alone GEMV

namespace esp {

// y = W.x with the same inner loop as the decode stages: one warp per pair of rows, 16-byte weight loads.
// (Measured on B200: this plain loop - two rows per warp, four 16-byte slices per row requested together, three
// CTAs per SM - streams an LM-head sized fp16 matrix at 0.93 of the copy peak; the software-pipelined four-row
// loop of the decode stages is slower here (0.83) because its register footprint halves the resident warps.
// The Q4_0 instance sits right at 128 registers; small source changes pushed it to ~157 and one CTA per SM
// (Q4_0 20.6 -> 24.4 us on 32768 x 4096), hence the two-CTA launch bound.)
template <int WT>
__global__ void __launch_bounds__(kThreads, 2) k_gemv_plain(Weight w, const float* __restrict__ x, float* __restrict__ y) {
    extern __shared__ float smem[];
    float* xs = smem + kRedFloats;
    const float xdescale = stage_vector<WT>(x, w.cols, NORM_NONE, nullptr, nullptr, 0.f, xs, smem);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // rows per warp pass: the quantised types read 2-4x more staged activation bytes per weight byte than fp16, so
    // they share one activation read between four rows
    constexpr int NR = (WT == WT_Q8_0 || WT == WT_Q4_0) ? 4 : 2;
    const int n_items = (w.rows + NR - 1) / NR;
    int begin, end;
    cta_range(n_items, blockIdx.x, gridDim.x, begin, end);
    auto rows_of = [&](int item, const uint8_t* (&wr)[NR], const __half* (&sr)[NR]) {
#pragma unroll
        for (int r = 0; r < NR; r++) {
            const int row = min(item * NR + r, w.rows - 1);
            wr[r] = weight_row(w, row);
            sr[r] = scale_row(w, row);
        }
    };
    auto finish = [&](int item, float (&acc)[NR]) {
#pragma unroll
        for (int r = 0; r < NR; r++) {
            const float v = warp_sum(acc[r]) * xdescale;
            if (lane == 0 && item * NR + r < w.rows) y[item * NR + r] = v;
        }
    };
    for (int item = begin + warp; item < end; item += kWarps) {
        const uint8_t* wr[NR];
        const __half* sr[NR];
        float acc[NR];
        rows_of(item, wr, sr);
#pragma unroll
        for (int r = 0; r < NR; r++) acc[r] = 0.f;
        dot_rows<WT, NR>(wr, sr, w.cols, xs, lane, acc);
        finish(item, acc);
    }
}

int32_t gemv_bench(int32_t type, const void* weights, int32_t rows, int32_t cols, const float* x, float* y, int32_t warmup,
                   int32_t iterations, int32_t copies, float* avg_ms, int32_t device) {
    if (!weights || !x || !y || rows <= 0 || cols <= 0 || iterations < 1 || copies < 1)
        return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "gemv_bench: bad arguments");
    if (type != WT_F16 && type != WT_BF16 && type != WT_Q8_0 && type != WT_Q4_0)
        return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "gemv_bench: unsupported type");
    if (cols % epl_of(type)) return fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "gemv_bench: cols must be a multiple of the load width");
    if (force_failure_enabled()) return fail(ESP_CUDA_ERR_FORCED_FAILURE, "forced failure is enabled");
    ESP_CUDA_TRY(cudaSetDevice(device));
    {
        const int bytes = 200 * 1024;
        cudaFuncSetAttribute(k_gemv_plain<WT_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        cudaFuncSetAttribute(k_gemv_plain<WT_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        cudaFuncSetAttribute(k_gemv_plain<WT_Q8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        cudaFuncSetAttribute(k_gemv_plain<WT_Q4_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    }
    std::vector<void*> owned;
    auto cleanup = [&] { for (void* p : owned) cudaFree(p); };
    const size_t n = (size_t)rows * cols;
    const bool quant = type == WT_Q8_0 || type == WT_Q4_0;
    const size_t in_bytes = type == WT_Q8_0 ? n / 32 * 34 : type == WT_Q4_0 ? n / 32 * 18 : n * 2;
    const size_t data_bytes = weight_row_bytes(type, cols) * rows;
    void* staging = nullptr;
    int32_t rc = ESP_CUDA_OK;
    std::vector<Weight> ws(copies);
    float *dx = nullptr, *dy = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    auto body = [&]() -> int32_t {
        if (quant) {
            ESP_CUDA_TRY(cudaMalloc(&staging, in_bytes));
            owned.push_back(staging);
            ESP_CUDA_TRY(cudaMemcpy(staging, weights, in_bytes, cudaMemcpyDefault));
        }
        for (int c = 0; c < copies; c++) {
            void* d = nullptr;
            __half* sc = nullptr;
            ESP_CUDA_TRY(cudaMalloc(&d, data_bytes));
            owned.push_back(d);
            if (quant) {
                ESP_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&sc), n / 32 * 2));
                owned.push_back(sc);
                int64_t nb = (int64_t)(n / 32);
                if (type == WT_Q8_0) k_repack_q8_0<<<(unsigned)((nb + 255) / 256), 256>>>(static_cast<uint8_t*>(staging), nb, static_cast<int8_t*>(d), sc);
                else k_repack_q4_0<<<(unsigned)((nb + 255) / 256), 256>>>(static_cast<uint8_t*>(staging), nb, static_cast<uint8_t*>(d), sc);
            } else {
                ESP_CUDA_TRY(cudaMemcpy(d, weights, data_bytes, cudaMemcpyDefault));
            }
            ws[c] = Weight{d, sc, rows, cols, type, 0};
        }
        ESP_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&dx), sizeof(float) * cols));
        owned.push_back(dx);
        ESP_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&dy), sizeof(float) * rows));
        owned.push_back(dy);
        ESP_CUDA_TRY(cudaMemcpy(dx, x, sizeof(float) * cols, cudaMemcpyDefault));
        ESP_CUDA_TRY(cudaDeviceSynchronize());
        int sm = 148;
        cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, device);
        int items = (rows + 1) / 2;
        size_t smem = sizeof(float) * (size_t)(kRedFloats + xs_floats_rt(type, cols));
        // one wave of CTAs: every CTA stages the activation vector once and then streams many rows
        int occ = 1;
        switch (type) {
            case WT_F16: cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_gemv_plain<WT_F16>, kThreads, smem); break;
            case WT_BF16: cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_gemv_plain<WT_BF16>, kThreads, smem); break;
            case WT_Q8_0: cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_gemv_plain<WT_Q8_0>, kThreads, smem); break;
            default: cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_gemv_plain<WT_Q4_0>, kThreads, smem); break;
        }
        int grid = std::max(1, std::min((items + kWarps - 1) / kWarps, sm * std::max(occ, 1)));
        auto launch = [&](int c) {
            switch (type) {
                case WT_F16: k_gemv_plain<WT_F16><<<grid, kThreads, smem>>>(ws[c], dx, dy); break;
                case WT_BF16: k_gemv_plain<WT_BF16><<<grid, kThreads, smem>>>(ws[c], dx, dy); break;
                case WT_Q8_0: k_gemv_plain<WT_Q8_0><<<grid, kThreads, smem>>>(ws[c], dx, dy); break;
                default: k_gemv_plain<WT_Q4_0><<<grid, kThreads, smem>>>(ws[c], dx, dy); break;
            }
        };
        for (int i = 0; i < warmup; i++) launch(i % copies);
        ESP_CUDA_TRY(cudaEventCreate(&e0));
        ESP_CUDA_TRY(cudaEventCreate(&e1));
        ESP_CUDA_TRY(cudaDeviceSynchronize());
        ESP_CUDA_TRY(cudaEventRecord(e0));
        for (int i = 0; i < iterations; i++) launch((warmup + i) % copies);
        ESP_CUDA_TRY(cudaEventRecord(e1));
        ESP_CUDA_TRY(cudaEventSynchronize(e1));
        ESP_CUDA_TRY(cudaGetLastError());
        float total = 0.f;
        ESP_CUDA_TRY(cudaEventElapsedTime(&total, e0, e1));
        if (avg_ms) *avg_ms = total / iterations;
        launch(0);
        ESP_CUDA_TRY(cudaMemcpy(y, dy, sizeof(float) * rows, cudaMemcpyDefault));
        return ESP_CUDA_OK;
    };
    rc = body();
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cleanup();
    return rc;
}

}  // namespace esp
