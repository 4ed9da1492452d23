// Dense "skinny" GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for the batched parts of the decode
// path: Y[n][m] = sum_k W[m][k] * X[n][k] for weight matrices W [M, K] (row-major, fp16 or bf16) and a batch of
// activation rows X [N, K] (the same 16-bit type), N = 1..256 rows.
//
// Mapping: the batch rows are the MMA's M dimension (one tile of up to 128 rows, TMEM lanes), the weight rows
// are its N dimension: a CTA owns 256 weight rows (two 128-row halves) and streams their K extent once.  One
// tcgen05.mma was measured at ~148 cycles whatever its shape, so the widest instruction (128 x 256 x 16) moves
// the most weight bytes per issue: 8 KB, about 55 bytes per cycle per SM, well above the SM's share of HBM.
// Operands are staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast); the fp32
// accumulator (128 lanes x 256 columns) lives in tensor memory and is read back with tcgen05.ld.
//
// Grid: x = batch tiles of 128 rows (fastest, so that the CTAs that share a weight tile run together and the second
// one finds it in L2), y = pairs of 128-row weight tiles, taken from up to three matrices that share X (a "group":
// the q, k and v projections run as one launch), z = slices of K.  The two halves of a CTA are
// independent (matrix, first row) pairs, so a pair may straddle two matrices.  A small matrix only goes faster
// with more CTAs: the host cuts K (and uses single-half CTAs) until the grid covers the SMs; K slices add their
// partial sums with fp32 vector atomics.
//
// DUAL (SwiGLU): half 0 holds 128 rows of the gate matrix, half 1 the same 128 rows of the up matrix, and the
// epilogue writes silu(gate) * up as 16-bit rows: the operand of the down projection, without an fp32 round trip.
//
// Warp roles (320 threads): warp 0 allocates tensor memory and issues the TMA loads, warp 1 issues the MMAs
// (one elected thread), warps 2..9 run the epilogue.  A warp may only touch the TMEM lanes 32*(warp%4)..+31, i.e.
// 32 batch rows, so two warps share a lane quadrant and split the columns.  tcgen05.ld hands a thread one batch
// row; written straight to global memory that is 32 different lines per store instruction (measured: 620 cycles
// per 16 columns), so the tile goes through shared memory (the idle pipeline stages) and leaves with the lanes
// along the weight rows: every global access is a contiguous 256-byte run per batch row.
// Every mbarrier wait is bounded; on a timeout the kernel records an error and unwinds normally.
// Programmatic dependent launch: the weight tiles of the first pipeline stages are requested before the wait on
// the previous kernel (weights never change); everything that depends on that kernel comes after the wait.
//
// Replaces, for batches, the per-row cblas/vDSP products of the reference (multiplyRowMajorMatrix,
// Sources/RealModelInference/RealModelInferenceEngine.swift:6674-6718) and the sequence-verify sgemm of
// Sources/Espresso/GenerationHarness.swift:2745-2761.
#pragma once
#include <cuda.h>

#include "mega_kernel.cuh"  // mbarrier helpers

namespace esp {

constexpr int kTcThreads = 320;  // TMA warp, MMA warp, 8 epilogue warps
constexpr int kTcHalf = 128;    // weight rows of one half tile (one TMA box)
constexpr int kTcBatch = 128;   // batch rows of one batch tile (the MMA's M)
constexpr int kTcBlockK = 64;   // 64 x 16-bit = one 128-byte swizzle row
constexpr int kTcStages = 4;
constexpr unsigned kTcSpinLimit = 1u << 22;
constexpr int kTcXBytes = kTcBatch * kTcBlockK * 2;       // 16 KB slot of the activation tile
constexpr int kTcHalfBytes = kTcHalf * kTcBlockK * 2;     // 16 KB per weight half
constexpr int kTcStageBytes = kTcXBytes + 2 * kTcHalfBytes;
constexpr size_t kTcSmemBytes = (size_t)kTcStages * kTcStageBytes + (2 * kTcStages + 1) * 8 + 16 + 1024;

enum TcEpilogue { TC_STORE = 0, TC_RESIDUAL = 1, TC_HEAD = 2, TC_GELU16 = 3, TC_SWIGLU16 = 4 };
constexpr int kTcMaxGroups = 3;

struct TcGroup {
    int M;              // weight rows of this matrix
    int tile0;          // index of its first 128-row tile in the launch's tile list
    float* out;         // [n][ldo] fp32 (TC_STORE: overwritten, TC_RESIDUAL: accumulated into)
    int ldo;
    const float* bias;  // [M] or null
};

struct TcArgs {
    int n_groups;
    TcGroup g[kTcMaxGroups];
    int n_tiles;                // 128-row weight tiles in the launch (all groups)
    int halves;                 // weight tiles per CTA: 1 or 2 (DUAL: 2 = gate and up)
    int dual;                   // SwiGLU pairing: half 0 from matrix 0, half 1 the same rows of matrix 1
    int K, n_valid;             // reduction length (multiple of 64), live batch rows
    int x_rows;                 // rows of the activation TMA box (16, 32, 64 or 128)
    int epilogue;               // TcEpilogue
    int kb_per_split;           // 64-wide K blocks per grid.z slice
    int atomic_out;             // K is sliced: TC_STORE / TC_RESIDUAL add into out (TC_STORE: out is zero beforehand)
    const int* active;          // [n] or null: rows with active == 0 are not written
    unsigned long long* best;   // TC_HEAD: packed running first-max per batch row
    float* logits;              // TC_HEAD: optional [n][M] logits store, or null
    uint16_t* out16;            // TC_GELU16 / TC_SWIGLU16: [n][ld16] operand rows of the next product
    int ld16;
    float* debug;               // TC_GELU16 / TC_SWIGLU16: optional fp32 capture of batch row 0
    int* error;                 // set to non-zero when a wait gave up
    int bf16;                   // operand type: 0 = fp16, 1 = bf16
    int row_offset;             // TC_HEAD: added to the row index (vocab shard of a tensor-parallel rank)
};

// Launch shape chosen by the host.
struct TcPlan {
    int x_rows = 16;       // activation box rows
    int n_tiles = 1;       // batch tiles (grid.y)
    int halves = 2;        // weight tiles per CTA
    int splits = 1;        // K slices (grid.z)
    int kb_per_split = 1;
};

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(smem_dst)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 x 16-bit) with the 128-byte
// swizzle: 8-row groups are 1024 bytes apart (stride byte offset), the leading byte offset is unused (1).
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(const void* smem_tile) {
    const uint32_t addr = smem_u32(smem_tile);
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFFu);   // start address, bits [0,14)
    d |= (uint64_t)1 << 16;                    // leading byte offset (ignored for swizzled K-major), bits [16,30)
    d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset, bits [32,46)
    d |= (uint64_t)1 << 46;                    // descriptor version of this architecture, bits [46,48)
    d |= (uint64_t)2 << 61;                    // layout type: 128-byte swizzle, bits [61,64)
    return d;
}

// Instruction descriptor of tcgen05.mma.kind::f16: fp32 accumulator, fp16 or bf16 operands, both K-major,
// M = 128 (batch rows), N = n (weight rows).
__device__ __forceinline__ uint32_t umma_idesc_f16(int n, int bf16) {
    uint32_t d = 0;
    d |= 1u << 4;                        // accumulator format: f32
    d |= (uint32_t)(bf16 ? 1 : 0) << 7;  // A format
    d |= (uint32_t)(bf16 ? 1 : 0) << 10; // B format
    d |= (uint32_t)(n >> 3) << 17;       // N / 8
    d |= (uint32_t)(kTcBatch >> 4) << 24;  // M / 16
    return d;
}

__device__ __forceinline__ bool tc_wait(uint64_t* bar, unsigned parity, int* error) {
    unsigned spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (++spins > kTcSpinLimit || ((spins & 0xfffu) == 0 && __ldcg(error) != 0)) {
            atomicCAS(error, 0, 7);
            return false;
        }
    }
    return true;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&f)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int j = 0; j < 16; j++) f[j] = __uint_as_float(r[j]);
}

// Activations of the batched epilogue.  The results are rounded to 16 bits right away, so the exponential may be
// the hardware approximation (relative error ~2^-21) instead of the exact tanhf of the single-row kernels.
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }
__device__ __forceinline__ float gelu_fast(float x) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    const float t = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * u));  // tanh(u)
    return 0.5f * x * (1.0f + t);
}

__device__ __forceinline__ uint32_t pack16x2(float a, float b, int bf16) {
    const uint32_t lo = bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(a)) : __half_as_ushort(__float2half_rn(a));
    const uint32_t hi = bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(b)) : __half_as_ushort(__float2half_rn(b));
    return lo | (hi << 16);
}

__global__ void __launch_bounds__(kTcThreads) k_gemm_tc(const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1,
                                                        const __grid_constant__ CUtensorMap map_w2, const __grid_constant__ CUtensorMap map_x,
                                                        const TcArgs a) {
    extern __shared__ __align__(1024) uint8_t tc_smem[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>(((uintptr_t)tc_smem + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)kTcStages * kTcStageBytes);
    uint64_t* empty = full + kTcStages;
    uint64_t* acc_ready = empty + kTcStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The (matrix, first row) of this CTA's weight halves.  Group fields are selected with constant indices: a
    // dynamically indexed parameter struct would be copied to local memory.
#define ESP_TC_G(gi, field) ((gi) == 0 ? a.g[0].field : (gi) == 1 ? a.g[1].field : a.g[2].field)
    int g_h0 = 0, g_h1 = 0, m0_h0 = 0, m0_h1 = 0;
    int n_halves = 0;
    if (a.dual) {
        g_h1 = 1;
        m0_h0 = m0_h1 = (int)blockIdx.y * kTcHalf;
        n_halves = 2;
    } else {
        const int t0 = (int)blockIdx.y * a.halves;
        if (t0 < a.n_tiles) {
            if (a.n_groups > 1 && t0 >= a.g[1].tile0) g_h0 = 1;
            if (a.n_groups > 2 && t0 >= a.g[2].tile0) g_h0 = 2;
            m0_h0 = (t0 - ESP_TC_G(g_h0, tile0)) * kTcHalf;
            n_halves = 1;
        }
        const int t1 = t0 + 1;
        if (a.halves == 2 && t1 < a.n_tiles) {
            if (a.n_groups > 1 && t1 >= a.g[1].tile0) g_h1 = 1;
            if (a.n_groups > 2 && t1 >= a.g[2].tile0) g_h1 = 2;
            m0_h1 = (t1 - ESP_TC_G(g_h1, tile0)) * kTcHalf;
            n_halves = 2;
        }
    }
    const CUtensorMap* const map_h0 = g_h0 == 0 ? &map_w0 : g_h0 == 1 ? &map_w1 : &map_w2;
    const CUtensorMap* const map_h1 = g_h1 == 0 ? &map_w0 : g_h1 == 1 ? &map_w1 : &map_w2;
    const int n0 = (int)blockIdx.x * kTcBatch;
    const int kb_total = a.K / kTcBlockK;
    const int kb0 = (int)blockIdx.z * a.kb_per_split;
    const int num_kb = n_halves > 0 ? min(a.kb_per_split, kb_total - kb0) : 0;
    const uint32_t stage_tx = (uint32_t)(a.x_rows * kTcBlockK * 2 + n_halves * kTcHalfBytes);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcStages; s++) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        mbar_init(acc_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // weight tiles of the first stages do not depend on the previous kernel
        const int pre = min(num_kb, kTcStages);
        for (int kb = 0; kb < pre; kb++) {
            uint8_t* sw = tiles + (size_t)kb * kTcStageBytes + kTcXBytes;
            mbar_expect_tx(full + kb, stage_tx);
            tma_load_2d(sw, map_h0, (kb0 + kb) * kTcBlockK, m0_h0, full + kb);
            if (n_halves == 2) tma_load_2d(sw + kTcHalfBytes, map_h1, (kb0 + kb) * kTcBlockK, m0_h1, full + kb);
        }
    }
    if (warp == 0) {  // the whole warp allocates the accumulator columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // The next kernel of the stream may be scheduled only after every CTA of this one holds its tensor memory:
    // a CTA of this kernel must never queue for columns behind a successor that is itself waiting for this kernel.
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t tmem_acc = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            for (int kb = 0; kb < num_kb; kb++) {
                const int s = kb % kTcStages;
                uint8_t* sx = tiles + (size_t)s * kTcStageBytes;
                if (kb >= kTcStages) {
                    if (!tc_wait(empty + s, ((kb / kTcStages) - 1) & 1, a.error)) break;
                    mbar_expect_tx(full + s, stage_tx);
                    tma_load_2d(sx + kTcXBytes, map_h0, (kb0 + kb) * kTcBlockK, m0_h0, full + s);
                    if (n_halves == 2) tma_load_2d(sx + kTcXBytes + kTcHalfBytes, map_h1, (kb0 + kb) * kTcBlockK, m0_h1, full + s);
                }
                tma_load_2d(sx, &map_x, (kb0 + kb) * kTcBlockK, n0, full + s);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(n_halves * kTcHalf, a.bf16);
            for (int kb = 0; kb < num_kb; kb++) {
                const int s = kb % kTcStages;
                if (!tc_wait(full + s, (kb / kTcStages) & 1, a.error)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint8_t* sx = tiles + (size_t)s * kTcStageBytes;
                const uint64_t da = umma_smem_desc_sw128(sx), db = umma_smem_desc_sw128(sx + kTcXBytes);
#pragma unroll
                for (int k = 0; k < kTcBlockK / 16; k++) {
                    // advancing 16 elements along K inside the swizzled row = 32 bytes = 2 descriptor units
                    umma_f16(tmem_acc, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                // the stage may be refilled once these MMAs have read it
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(empty + s)) : "memory");
            }
            // accumulator complete (or abandoned): release the epilogue either way
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(acc_ready)) : "memory");
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> shared -> global ----------------
        const int ew = warp - 2;            // 0..7
        const int lane_base = 32 * (warp & 3);
        const int sub = ew >> 2;            // which 64-column half of every 128-row weight tile this warp owns
        const int n = n0 + lane_base + lane;  // phase 1: this thread's batch row
        const bool warp_has_rows = n0 + lane_base < a.n_valid;
        const bool live = n < a.n_valid && (!a.active || a.active[n]);
        const bool ok = tc_wait(acc_ready, 0, a.error) && __ldcg(a.error) == 0 && num_kb > 0;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // kernel parameters used per chunk live in registers for the whole loop
        const int epilogue = a.epilogue, bf16 = a.bf16, ld16 = a.ld16, row_offset = a.row_offset;
        const bool atomic_out = a.atomic_out != 0, first_split = blockIdx.z == 0;
        float* const logits = a.logits;
        float* const debug = a.debug;
        uint16_t* const out16 = a.out16;
        const uint32_t trow = tmem_acc + ((uint32_t)lane_base << 16);
        if (ok && warp_has_rows && epilogue == TC_HEAD) {
            // a thread scans the weight rows of its batch row: first maximum, ascending, so a later equal value does not
            // replace an earlier one; the packed atomicMax (value, ~index) merges threads and CTAs with the same rule
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            const int M = a.g[0].M;
#pragma unroll 1
            for (int hh = 0; hh < n_halves; hh++) {
                const int mbase = (hh ? m0_h1 : m0_h0) + sub * 64;
#pragma unroll 1
                for (int c0 = 0; c0 < 64; c0 += 16) {
                    const int m = mbase + c0;
                    if (m >= M) break;
                    float v[16];
                    tmem_ld16(trow + (uint32_t)(hh * kTcHalf + sub * 64 + c0), v);
                    if (!live) continue;
                    const bool whole = m + 16 <= M;  // false only at a ragged vocabulary end
#pragma unroll
                    for (int j = 0; j < 16; j++)
                        if ((whole || m + j < M) && v[j] > bv) { bv = v[j]; bi = m + j + row_offset; }
                    if (logits) {
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (whole || m + j < M) logits[(size_t)n * M + m + j] = v[j];
                    }
                }
            }
            if (live && bi != 0x7fffffff) atomicMax(a.best + n, pack_best(bv, bi));
        } else if (ok && warp_has_rows) {
            // Phase 1: this warp's 32 batch rows x (64 columns of each weight half) go to its private staging rows.
            // Every MMA has completed, so the pipeline stages are idle and nothing else touches this memory.
            constexpr int kStride = 2 * 64 + 4;  // floats per staged row; the pad keeps the 16-byte row stores conflict-free
            float* const stg = reinterpret_cast<float*>(tiles) + (size_t)ew * 32 * kStride;
            {
                float* const mine = stg + (size_t)lane * kStride;
#pragma unroll 1
                for (int hh = 0; hh < n_halves; hh++) {
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        float v[16];
                        tmem_ld16(trow + (uint32_t)(hh * kTcHalf + sub * 64 + c * 16), v);
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            reinterpret_cast<float4*>(mine + hh * 64 + c * 16)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    }
                }
            }
            __syncwarp();
            // Phase 2: a half-warp per batch row, 16 lanes x 4 consecutive weight rows = one 256-byte run.
            const unsigned live_mask = __ballot_sync(0xffffffffu, live);
            const int nrow0 = n0 + lane_base;
            const int hl = lane >> 4, cl = (lane & 15) * 4;
            if (epilogue == TC_SWIGLU16) {
                const int m = m0_h0 + sub * 64 + cl;
                if (m < a.g[0].M) {
#pragma unroll 4
                    for (int r0 = 0; r0 < 32; r0 += 2) {
                        const int r = r0 + hl;
                        if (!((live_mask >> r) & 1u)) continue;
                        const float4 gt = *reinterpret_cast<const float4*>(stg + (size_t)r * kStride + cl);
                        const float4 up = *reinterpret_cast<const float4*>(stg + (size_t)r * kStride + 64 + cl);
                        const float v0 = silu_fast(gt.x) * up.x, v1 = silu_fast(gt.y) * up.y, v2 = silu_fast(gt.z) * up.z, v3 = silu_fast(gt.w) * up.w;
                        *reinterpret_cast<uint2*>(out16 + (size_t)(nrow0 + r) * ld16 + m) = make_uint2(pack16x2(v0, v1, bf16), pack16x2(v2, v3, bf16));
                        if (debug && nrow0 + r == 0) *reinterpret_cast<float4*>(debug + m) = make_float4(v0, v1, v2, v3);
                    }
                }
            } else {
#pragma unroll 1
                for (int hh = 0; hh < n_halves; hh++) {
                    const int gi = hh ? g_h1 : g_h0;
                    const int M = ESP_TC_G(gi, M), ldo = ESP_TC_G(gi, ldo);
                    const float* const bias = first_split ? ESP_TC_G(gi, bias) : nullptr;
                    float* const out = ESP_TC_G(gi, out);
                    const int m = (hh ? m0_h1 : m0_h0) + sub * 64 + cl;
                    if (m >= M) continue;
                    const bool vec = m + 4 <= M && ((ldo | ld16) & 3) == 0;
                    float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (bias) {
                        b4.x = bias[m];
                        if (m + 1 < M) b4.y = bias[m + 1];
                        if (m + 2 < M) b4.z = bias[m + 2];
                        if (m + 3 < M) b4.w = bias[m + 3];
                    }
#pragma unroll 4
                    for (int r0 = 0; r0 < 32; r0 += 2) {
                        const int r = r0 + hl;
                        if (!((live_mask >> r) & 1u)) continue;
                        float4 v = *reinterpret_cast<const float4*>(stg + (size_t)r * kStride + hh * 64 + cl);
                        v.x += b4.x; v.y += b4.y; v.z += b4.z; v.w += b4.w;
                        const size_t nr = (size_t)(nrow0 + r);
                        if (epilogue == TC_GELU16) {
                            const float g0 = gelu_fast(v.x), g1 = gelu_fast(v.y), g2 = gelu_fast(v.z), g3 = gelu_fast(v.w);
                            uint16_t* o = out16 + nr * ld16 + m;
                            if (vec) {
                                *reinterpret_cast<uint2*>(o) = make_uint2(pack16x2(g0, g1, bf16), pack16x2(g2, g3, bf16));
                            } else {
                                const float gl[4] = {g0, g1, g2, g3};
                                for (int j = 0; j < 4 && m + j < M; j++) o[j] = (uint16_t)(pack16x2(gl[j], 0.f, bf16) & 0xffffu);
                            }
                            if (debug && nr == 0) {
                                const float gl[4] = {g0, g1, g2, g3};
                                for (int j = 0; j < 4 && m + j < M; j++) debug[m + j] = gl[j];
                            }
                        } else {
                            float* o = out + nr * ldo + m;
                            if (vec) {
                                if (atomic_out) {
                                    red_add_v4(o, v.x, v.y, v.z, v.w);
                                } else {
                                    if (epilogue == TC_RESIDUAL) {
                                        const float4 pv = *reinterpret_cast<const float4*>(o);
                                        v.x += pv.x; v.y += pv.y; v.z += pv.z; v.w += pv.w;
                                    }
                                    *reinterpret_cast<float4*>(o) = v;
                                }
                            } else {
                                const float vv[4] = {v.x, v.y, v.z, v.w};
                                for (int j = 0; j < 4 && m + j < M; j++) {
                                    if (atomic_out) atomicAdd(o + j, vv[j]);
                                    else o[j] = epilogue == TC_RESIDUAL ? o[j] + vv[j] : vv[j];
                                }
                            }
                        }
                    }
                }
            }
        }
    }
#undef ESP_TC_G
    // tensor memory is released by the warp that allocated it, after everybody is done with it
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(256u) : "memory");
    }
}

}  // namespace esp
