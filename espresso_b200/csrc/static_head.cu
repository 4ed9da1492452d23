// esp_cuda_lm_head_argmax_static: final norm + LM head + greedy argmax for callers that must not allocate.
//
// Some hosts of this library run with a device-memory budget that is fixed before they start (a serving process
// whose pool was carved up front, a plugin living inside another framework's arena) or sit in a latency-critical
// loop where a cudaMalloc/cudaFree would synchronise the whole device.  They own device buffers for the inputs and
// the outputs already, but the head kernel also needs a little working memory of its own: the packed running
// maximum per row, the CTA completion counter and the per-row control words.  Here that working memory is a
// fixed array compiled into the library image, so the call itself never touches the CUDA allocator.
//
// Consequences of the fixed array, for users of the entry point:
//  * every GPU that loads the library holds the 4 KiB array until the process exits;
//  * at most ESP_CUDA_STATIC_HEAD_MAX_ROWS rows per call; larger requests are refused with an error;
//  * all calls on a device share the array and it keeps whatever the previous call left in it, so each call
//    re-initialises the words that must start from zero, and two calls whose kernels overlap on the GPU
//    (different streams, or different host threads) race with each other: serialise them;
//  * the first call on a device looks up the array's device address (cudaGetSymbolAddress); make that first
//    call before beginning any stream capture.
#include "engine.h"

namespace esp {

constexpr int kStaticHeadMaxRows = ESP_CUDA_STATIC_HEAD_MAX_ROWS;
constexpr int kStaticHeadMaxDModel = 8192;  // keeps the staged vector inside the default 48 KiB of shared memory
constexpr size_t kStaticHeadBytes = 4096;

// Layout (bytes): [0,512) packed maxima, [512,528) completion counter, then seven arrays of 64 32-bit words:
// seq, pos, tok, active, next, n_out, limit.
static __device__ __align__(256) unsigned char g_static_head_scratch[kStaticHeadBytes];

struct StaticHeadView {
    unsigned long long* best;
    unsigned int* ticket;
    int *seq, *pos, *active, *n_out, *limit;
    uint32_t *tok, *next;
};

__host__ __device__ inline StaticHeadView static_head_view(unsigned char* base) {
    StaticHeadView v;
    v.best = reinterpret_cast<unsigned long long*>(base);
    v.ticket = reinterpret_cast<unsigned int*>(base + 512);
    int* words = reinterpret_cast<int*>(base + 528);
    v.seq = words;
    v.pos = words + 64;
    v.tok = reinterpret_cast<uint32_t*>(words + 128);
    v.active = words + 192;
    v.next = reinterpret_cast<uint32_t*>(words + 256);
    v.n_out = words + 320;
    v.limit = words + 384;
    return v;
}

// Device code may name the array directly; this kernel resets the words a call depends on.
__global__ void k_static_head_init(int rows) {
    StaticHeadView v = static_head_view(g_static_head_scratch);
    const int t = threadIdx.x;
    if (t < kStaticHeadMaxRows) {
        v.best[t] = 0ull;
        v.seq[t] = 0; v.pos[t] = 0; v.tok[t] = 0u; v.next[t] = 0u; v.n_out[t] = 0; v.limit[t] = 0;
        v.active[t] = t < rows ? 1 : 0;
    }
    if (t == 0) *v.ticket = 0u;
}

// Host code needs the array's device address: the symbol's name in host code is only a stand-in.
static int32_t static_head_address(int device, unsigned char** out) {
    static std::mutex mu;
    static unsigned char* addr[64] = {};
    if (device < 0 || device >= 64) return esp::fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "device ordinal out of range");
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_head_scratch);  // the device must be current (it is: see caller)
        if (e != cudaSuccess) return esp::fail(ESP_CUDA_ERR_CUDA, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        addr[device] = static_cast<unsigned char*>(p);
    }
    *out = addr[device];
    return ESP_CUDA_OK;
}

int32_t lm_head_argmax_static(const void* d_lm_head_f16, int32_t vocab, int32_t d_model, const float* d_hidden, int32_t rows,
                              const float* d_norm_gain, float norm_eps, uint32_t* d_tokens, void* cuda_stream, int32_t device) {
    if (!d_lm_head_f16 || !d_hidden || !d_tokens) return esp::fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "lm_head_argmax_static: null pointer");
    if (rows < 1 || rows > kStaticHeadMaxRows) {
        std::ostringstream os;
        os << "lm_head_argmax_static: rows = " << rows << " is outside 1.." << kStaticHeadMaxRows
           << " (the working memory of this entry point is a fixed array)";
        return esp::fail(ESP_CUDA_ERR_INVALID_ARGUMENT, os.str());
    }
    if (vocab < 1 || d_model < 8 || d_model % 8 != 0 || d_model > kStaticHeadMaxDModel) {
        std::ostringstream os;
        os << "lm_head_argmax_static: d_model must be a multiple of 8 in [8, " << kStaticHeadMaxDModel << "] and vocab >= 1";
        return esp::fail(ESP_CUDA_ERR_INVALID_ARGUMENT, os.str());
    }
    // the kernel reads the matrix with 16-byte loads and the vectors as 4-byte words: a view that starts elsewhere would
    // fault on the device, so it is refused here
    if (reinterpret_cast<uintptr_t>(d_lm_head_f16) % 16 != 0)
        return esp::fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "lm_head_argmax_static: d_lm_head_f16 must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(d_hidden) % 4 != 0 || reinterpret_cast<uintptr_t>(d_norm_gain) % 4 != 0 || reinterpret_cast<uintptr_t>(d_tokens) % 4 != 0)
        return esp::fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "lm_head_argmax_static: d_hidden, d_norm_gain and d_tokens must be 4-byte aligned");
    if (force_failure_enabled()) return esp::fail(ESP_CUDA_ERR_FORCED_FAILURE, "forced failure is enabled");
    // the call runs on `device` and leaves the caller's current device as it found it
    struct DeviceGuard {
        int prev = -1;
        ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
    } guard;
    ESP_CUDA_TRY(cudaGetDevice(&guard.prev));
    if (guard.prev == device) guard.prev = -1;
    else ESP_CUDA_TRY(cudaSetDevice(device));
    unsigned char* base = nullptr;
    int32_t rc = static_head_address(device, &base);
    if (rc) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    const StaticHeadView v = static_head_view(base);

    k_static_head_init<<<1, 64, 0, stream>>>(rows);
    ESP_CUDA_TRY(cudaGetLastError());

    GemvArgs ga{};
    ga.m.arch = ARCH_LLAMA; ga.m.n_layer = 1; ga.m.n_head = 1; ga.m.n_kv_head = 1; ga.m.d_model = d_model; ga.m.head_dim = 8;
    ga.m.hidden = d_model; ga.m.vocab = vocab; ga.m.max_seq = 1; ga.m.q_dim = 8; ga.m.kv_dim = 8; ga.m.n_seq = rows;
    ga.m.eps = norm_eps; ga.m.eos_token = -1;
    ga.rows = rows;
    ga.rs.seq = v.seq; ga.rs.pos = v.pos; ga.rs.tok = v.tok; ga.rs.active = v.active; ga.rs.next = v.next;
    ga.rs.n_out = v.n_out; ga.rs.limit = v.limit; ga.rs.out = v.next; ga.rs.out_stride = 0;
    ga.rs.best = v.best; ga.rs.ticket = v.ticket;
    ga.w = Weight{d_lm_head_f16, nullptr, vocab, d_model, WT_F16, 0};
    ga.norm = d_norm_gain ? NORM_RMS : NORM_NONE;
    ga.norm_g = d_norm_gain;
    ga.in = d_hidden; ga.in_stride = d_model;
    ga.layer = -1; ga.debug_slot = -1; ga.finalize_mode = 0;
    int sm = 148;
    cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, device);
    const int items = (vocab + 1) / 2;
    const int grid = std::max(1, std::min((items + kWarps - 1) / kWarps, sm * 4));
    const size_t smem = sizeof(float) * (size_t)(kRedFloats + xs_floats_rt(WT_F16, d_model));
    ESP_CUDA_TRY(launch_pdl(k_lm_head<WT_F16>, dim3(grid), dim3(kThreads), smem, stream, ga));
    ESP_CUDA_TRY(cudaMemcpyAsync(d_tokens, v.next, sizeof(uint32_t) * rows, cudaMemcpyDeviceToDevice, stream));
    return ESP_CUDA_OK;
}

}  // namespace esp

extern "C" int32_t esp_cuda_lm_head_argmax_static(const void* d_lm_head_f16, int32_t vocab, int32_t d_model, const float* d_hidden,
                                                  int32_t rows, const float* d_norm_gain, float norm_eps, uint32_t* d_tokens,
                                                  void* cuda_stream, int32_t device) {
    return esp::lm_head_argmax_static(d_lm_head_f16, vocab, d_model, d_hidden, rows, d_norm_gain, norm_eps, d_tokens, cuda_stream, device);
}
