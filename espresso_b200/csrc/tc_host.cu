// Host side of the tensor-core GEMM: TMA tensor maps, launch dispatch over the batch tile width, and the
// stand-alone entry point used for parity checks and tensor-pipe measurements.
#include "engine.h"
#include "tc_gemm.cuh"

namespace esp {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D map over a row-major [rows, cols] matrix of 16-bit elements: boxes of 64 columns x box_rows rows, 128-byte
// swizzle, out-of-range elements read as zero.
int32_t tc_make_map(CUtensorMap* map, const void* base, bool bf16, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return esp::fail(ESP_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    if (cols % 8 != 0 || (reinterpret_cast<uintptr_t>(base) & 15)) return esp::fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "tensor map: base or row pitch not 16-byte aligned");
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)kTcBlockK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), gdim, gstride, box,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        std::ostringstream os;
        os << "cuTensorMapEncodeTiled failed with code " << (int)r;
        return esp::fail(ESP_CUDA_ERR_CUDA, os.str());
    }
    return ESP_CUDA_OK;
}

// Rows of the activation TMA box for `rows` batch rows (one batch tile holds at most 128).
int tc_tile_for(int rows) {
    if (rows > 4 * kTcBatch) return 0;
    for (int t : {16, 32, 64, 128})
        if (rows <= t) return t;
    return 128;
}

// Launch shape for a product with `w_tiles` 128-row weight tiles, `rows` batch rows and `kb` 64-wide K blocks on
// `sms` SMs.  A large matrix runs two weight tiles per CTA (256 weight rows per MMA) over all of K; a small one is
// cut along K (a slice keeps at least 3 K blocks; wide batches take fewer slices, measured), and goes to one tile
// per CTA, until the grid covers the SMs.
TcPlan tc_plan(int w_tiles, int rows, int kb, bool may_split_k, bool dual, int sms) {
    TcPlan p;
    p.x_rows = tc_tile_for(std::min(rows, kTcBatch));
    p.n_tiles = (rows + kTcBatch - 1) / kTcBatch;
    auto shape = [&](int halves) {
        p.halves = halves;
        const int ctas = (dual ? w_tiles : (w_tiles + halves - 1) / halves) * p.n_tiles;
        int want = may_split_k ? std::max(1, std::min(sms / std::max(1, ctas), kb / 3)) : 1;
        want = std::min(want, std::max(4, 1024 / std::max(1, rows)));  // every slice adds rows x M floats with atomics
        p.kb_per_split = (kb + want - 1) / want;
        p.splits = (kb + p.kb_per_split - 1) / p.kb_per_split;
        return ctas * p.splits;
    };
    if (shape(2) * 2 <= sms && !dual) shape(1);
    return p;
}

static cudaError_t tc_configure() {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_gemm_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemBytes);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    return cudaSuccess;
}

// mw: the weight maps of the group (unused slots repeat slot 0); map_x must have been built with box_rows ==
// plan.x_rows.  The argument block's tile list, K slicing and box size are filled in here.
cudaError_t tc_launch(const TcPlan& plan, bool dual, const CUtensorMap* const* mw, const CUtensorMap& mx, TcArgs a, cudaStream_t s) {
    cudaError_t e = tc_configure();
    if (e != cudaSuccess) return e;
    int tiles = 0;
    const int groups = dual ? 1 : a.n_groups;
    for (int g = 0; g < groups; g++) {
        a.g[g].tile0 = tiles;
        tiles += (a.g[g].M + kTcHalf - 1) / kTcHalf;
    }
    a.n_tiles = tiles;
    a.dual = dual ? 1 : 0;
    a.halves = dual ? 2 : plan.halves;
    a.x_rows = plan.x_rows;
    a.kb_per_split = plan.kb_per_split;
    a.atomic_out = plan.splits > 1 ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.n_tiles, dual ? tiles : (tiles + a.halves - 1) / a.halves, plan.splits);
    cfg.blockDim = dim3(kTcThreads);
    cfg.dynamicSmemBytes = kTcSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, k_gemm_tc, *mw[0], *mw[1], *mw[2], mx, a);
}

__global__ void k_f32_to_16(const float* src, int64_t n, uint16_t* dst, int bf16) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (bf16) dst[i] = __bfloat16_as_ushort(__float2bfloat16_rn(src[i]));
    else dst[i] = __half_as_ushort(__float2half_rn(src[i]));
}

// Y[n][m] = sum_k W[m][k] * X16[n][k], X16 = X rounded to the weights' 16-bit type.  W, X, Y are host pointers.
int32_t gemm_tc_bench(int32_t type, const void* w, int32_t M, int32_t K, const float* x, int32_t N, float* y, int32_t warmup,
                      int32_t iterations, float* avg_ms, int32_t device) {
    if (!w || !x || !y || M < 1 || N < 1 || N > 256 || K < kTcBlockK || K % kTcBlockK != 0 || iterations < 1)
        return esp::fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "gemm_tc_bench: need 1 <= N <= 256 and K a multiple of 64");
    if (type != WT_F16 && type != WT_BF16) return esp::fail(ESP_CUDA_ERR_INVALID_ARGUMENT, "gemm_tc_bench: fp16 or bf16 weights only");
    if (force_failure_enabled()) return esp::fail(ESP_CUDA_ERR_FORCED_FAILURE, "forced failure is enabled");
    ESP_CUDA_TRY(cudaSetDevice(device));
    const int alloc_rows = (N + 15) / 16 * 16;
    std::vector<void*> owned;
    auto cleanup = [&] { for (void* p : owned) cudaFree(p); };
    auto body = [&]() -> int32_t {
        void *dw = nullptr, *dx16 = nullptr;
        float *dx = nullptr, *dy = nullptr;
        int* derr = nullptr;
        ESP_CUDA_TRY(cudaMalloc(&dw, (size_t)M * K * 2)); owned.push_back(dw);
        ESP_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&dx), sizeof(float) * (size_t)N * K)); owned.push_back(dx);
        ESP_CUDA_TRY(cudaMalloc(&dx16, (size_t)alloc_rows * K * 2)); owned.push_back(dx16);
        ESP_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&dy), sizeof(float) * (size_t)N * M)); owned.push_back(dy);
        ESP_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&derr), sizeof(int))); owned.push_back(derr);
        ESP_CUDA_TRY(cudaMemcpy(dw, w, (size_t)M * K * 2, cudaMemcpyDefault));
        ESP_CUDA_TRY(cudaMemcpy(dx, x, sizeof(float) * (size_t)N * K, cudaMemcpyDefault));
        ESP_CUDA_TRY(cudaMemset(dx16, 0, (size_t)alloc_rows * K * 2));
        ESP_CUDA_TRY(cudaMemset(derr, 0, sizeof(int)));
        const int64_t nx = (int64_t)N * K;
        k_f32_to_16<<<(unsigned)((nx + 255) / 256), 256>>>(dx, nx, static_cast<uint16_t*>(dx16), type == WT_BF16);
        ESP_CUDA_TRY(cudaGetLastError());
        CUtensorMap mw, mx;
        int32_t rc;
        if ((rc = tc_make_map(&mw, dw, type == WT_BF16, M, K, kTcHalf))) return rc;
        int sms = 148;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        // the plan the decode engine would use for a product of this shape (K slices add into a zeroed output)
        const TcPlan plan = tc_plan((M + kTcHalf - 1) / kTcHalf, N, K / kTcBlockK, true, false, sms);
        if ((rc = tc_make_map(&mx, dx16, type == WT_BF16, alloc_rows, K, plan.x_rows))) return rc;
        const CUtensorMap* maps[3] = {&mw, &mw, &mw};
        TcArgs a{};
        a.n_groups = 1;
        a.g[0].M = M; a.g[0].out = dy; a.g[0].ldo = M;
        a.K = K; a.n_valid = N; a.epilogue = TC_STORE; a.error = derr; a.bf16 = type == WT_BF16;
        auto launch = [&]() -> cudaError_t {
            if (plan.splits > 1) {
                cudaError_t e = cudaMemsetAsync(dy, 0, sizeof(float) * (size_t)N * M, nullptr);
                if (e != cudaSuccess) return e;
            }
            return tc_launch(plan, false, maps, mx, a, nullptr);
        };
        for (int i = 0; i < warmup; i++) ESP_CUDA_TRY(launch());
        cudaEvent_t e0, e1;
        ESP_CUDA_TRY(cudaEventCreate(&e0));
        ESP_CUDA_TRY(cudaEventCreate(&e1));
        ESP_CUDA_TRY(cudaDeviceSynchronize());
        ESP_CUDA_TRY(cudaEventRecord(e0));
        for (int i = 0; i < iterations; i++) ESP_CUDA_TRY(launch());
        ESP_CUDA_TRY(cudaEventRecord(e1));
        cudaError_t e = cudaEventSynchronize(e1);
        float total = 0.f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&total, e0, e1);
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        ESP_CUDA_TRY(e);
        if (avg_ms) *avg_ms = total / iterations;
        int herr = 0;
        ESP_CUDA_TRY(cudaMemcpy(&herr, derr, sizeof(int), cudaMemcpyDeviceToHost));
        if (herr) return esp::fail(ESP_CUDA_ERR_TIMEOUT, "tensor-core GEMM gave up waiting on a barrier");
        ESP_CUDA_TRY(cudaMemcpy(y, dy, sizeof(float) * (size_t)N * M, cudaMemcpyDeviceToHost));
        return ESP_CUDA_OK;
    };
    int32_t rc = body();
    cleanup();
    return rc;
}

}  // namespace esp

extern "C" int32_t esp_cuda_gemm_tc_bench(int32_t type, const void* weights, int32_t rows, int32_t cols, const float* x, int32_t n, float* y,
                                          int32_t warmup, int32_t iterations, float* avg_ms, int32_t device) {
    return esp::gemm_tc_bench(type, weights, rows, cols, x, n, y, warmup, iterations, avg_ms, device);
}
