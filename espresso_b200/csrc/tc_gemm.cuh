// Dense "skinny" GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for the batched parts of the decode
// path: Y[n][m] = sum_k W[m][k] * X[n][k] for weight matrices W [M, K] (row-major, fp16 or bf16) and a batch of
// activation rows X [N, K] (the same 16-bit type), N = 1..256 rows.
//
// Mapping: the weight rows are the MMA's M dimension (128 per CTA), the batch is its N dimension, so with one
// batch tile a CTA streams its 128 x K slice of W exactly once whatever the batch size.  Operands are staged in
// shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast), the fp32 accumulator lives in
// tensor memory (128 lanes x N columns) and is read back with tcgen05.ld for the epilogue.
//
// Grid: x = 128-row tiles of up to three weight matrices that share X (a "group": q, k and v projections run as one
// launch), y = batch tiles, z = slices of K.  One MMA of 128 x N x 16 occupies the tensor pipe for about 128
// cycles whatever N is (measured), so a small matrix only goes faster with more CTAs: the host splits the batch
// and K until the grid covers the SMs.  K slices add their partial sums with fp32 atomics.
//
// DUAL: the CTA keeps two accumulators, gate (W of group 0) and up (W of group 1) for the same 128 rows, and its
// epilogue writes silu(gate) * up as 16-bit rows: the operand of the down projection, without an fp32 round trip.
//
// Warp roles (192 threads): warp 0 allocates tensor memory and issues the TMA loads, warp 1 issues the MMAs
// (one elected thread), warps 2..5 run the epilogue (a warp may only touch the TMEM lanes 32*(warp%4)..+31).
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

constexpr int kTcThreads = 192;
constexpr int kTcBlockM = 128;
constexpr int kTcBlockK = 64;  // 64 x 16-bit = one 128-byte swizzle row
constexpr unsigned kTcSpinLimit = 1u << 22;

enum TcEpilogue { TC_STORE = 0, TC_RESIDUAL = 1, TC_HEAD = 2, TC_GELU16 = 3, TC_SWIGLU16 = 4 };
constexpr int kTcMaxGroups = 3;

struct TcGroup {
    int M;              // weight rows of this matrix
    int tile0;          // first blockIdx.x of this matrix
    float* out;         // [n][ldo] fp32 (TC_STORE: overwritten, TC_RESIDUAL: accumulated into)
    int ldo;
    const float* bias;  // [M] or null
};

struct TcArgs {
    int n_groups;
    TcGroup g[kTcMaxGroups];
    int K, n_valid;             // reduction length (multiple of 64), live batch rows
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

// Instruction descriptor of tcgen05.mma.kind::f16: fp32 accumulator, fp16 or bf16 operands, both K-major.
__device__ __forceinline__ uint32_t umma_idesc_f16(int n, int bf16) {
    uint32_t d = 0;
    d |= 1u << 4;                        // accumulator format: f32
    d |= (uint32_t)(bf16 ? 1 : 0) << 7;  // A format
    d |= (uint32_t)(bf16 ? 1 : 0) << 10; // B format
    d |= (uint32_t)(n >> 3) << 17;       // N / 8
    d |= (uint32_t)(kTcBlockM >> 4) << 24;  // M / 16
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

// Launch shape chosen by the host: batch tile width, batch tiles (grid.y), K slices (grid.z).
struct TcPlan {
    int tile = 16, n_tiles = 1, splits = 1, kb_per_split = 1;
};

template <int N_TILE, bool DUAL>
struct TcShape {
    static constexpr int A_BYTES = kTcBlockM * kTcBlockK * 2 * (DUAL ? 2 : 1);
    static constexpr int B_BYTES = N_TILE * kTcBlockK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + ((B_BYTES + 1023) / 1024) * 1024;
    static constexpr int STAGES = (200 * 1024 / STAGE_BYTES) > 6 ? 6 : (200 * 1024 / STAGE_BYTES);
    static constexpr int ACC_COLS = N_TILE * (DUAL ? 2 : 1);
    static constexpr int TMEM_COLS = ACC_COLS < 32 ? 32 : ACC_COLS;  // power of two >= 32 (N_TILE is 16/32/64/128/256)
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 1) * 8 + 16 + 1024;
};

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// N_TILE: accumulator columns (batch rows of one batch tile): 16, 32, 64, 128 or 256.  DUAL doubles the columns
// (two accumulators), up to the 512 columns of tensor memory.
template <int N_TILE, bool DUAL>
__global__ void __launch_bounds__(kTcThreads) k_gemm_tc(const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1,
                                                        const __grid_constant__ CUtensorMap map_w2, const __grid_constant__ CUtensorMap map_x,
                                                        const TcArgs a) {
    using S = TcShape<N_TILE, DUAL>;
    constexpr int STAGES = S::STAGES;
    constexpr int W_BYTES = kTcBlockM * kTcBlockK * 2;
    extern __shared__ __align__(1024) uint8_t tc_smem[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>(((uintptr_t)tc_smem + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * S::STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_ready = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
    __shared__ uint32_t s_live16[16];  // bit j of word c: batch row n0 + 16 c + j is written (live and active)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // which matrix of the group this CTA works on
    int gi = 0;
    if (!DUAL) {
        if (a.n_groups > 1 && (int)blockIdx.x >= a.g[1].tile0) gi = 1;
        if (a.n_groups > 2 && (int)blockIdx.x >= a.g[2].tile0) gi = 2;
    }
    const CUtensorMap* map_w = gi == 0 ? &map_w0 : gi == 1 ? &map_w1 : &map_w2;
    // (selected with constant indices: a dynamically indexed parameter struct would be copied to local memory)
#define ESP_TC_G(field) (gi == 0 ? a.g[0].field : gi == 1 ? a.g[1].field : a.g[2].field)
    const int m0 = ((int)blockIdx.x - ESP_TC_G(tile0)) * kTcBlockM;
    const int n0 = (int)blockIdx.y * N_TILE;
    const int kb_total = a.K / kTcBlockK;
    const int kb0 = (int)blockIdx.z * a.kb_per_split;
    const int num_kb = min(a.kb_per_split, kb_total - kb0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        mbar_init(acc_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // weight tiles of the first stages do not depend on the previous kernel
        const int pre = min(num_kb, STAGES);
        for (int kb = 0; kb < pre; kb++) {
            uint8_t* sa = tiles + (size_t)kb * S::STAGE_BYTES;
            mbar_expect_tx(full + kb, S::A_BYTES + S::B_BYTES);
            tma_load_2d(sa, map_w, (kb0 + kb) * kTcBlockK, m0, full + kb);
            if (DUAL) tma_load_2d(sa + W_BYTES, &map_w1, (kb0 + kb) * kTcBlockK, m0, full + kb);
        }
    }
    if (warp == 0) {  // the whole warp allocates the accumulator columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)S::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // The next kernel of the stream may be scheduled only after every CTA of this one holds its tensor memory:
    // a CTA of this kernel must never queue for columns behind a successor that is itself waiting for this kernel.
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x >= 32 && threadIdx.x < 48) {
        const int c = threadIdx.x - 32;
        uint32_t mask = 0;
        for (int j = 0; j < 16; j++) {
            const int n = n0 + c * 16 + j;
            if (c * 16 + j < N_TILE && n < a.n_valid && (!a.active || a.active[n])) mask |= 1u << j;
        }
        s_live16[c] = mask;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_acc = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            for (int kb = 0; kb < num_kb; kb++) {
                const int s = kb % STAGES;
                uint8_t* sa = tiles + (size_t)s * S::STAGE_BYTES;
                if (kb >= STAGES) {
                    if (!tc_wait(empty + s, ((kb / STAGES) - 1) & 1, a.error)) break;
                    mbar_expect_tx(full + s, S::A_BYTES + S::B_BYTES);
                    tma_load_2d(sa, map_w, (kb0 + kb) * kTcBlockK, m0, full + s);
                    if (DUAL) tma_load_2d(sa + W_BYTES, &map_w1, (kb0 + kb) * kTcBlockK, m0, full + s);
                }
                tma_load_2d(sa + S::A_BYTES, &map_x, (kb0 + kb) * kTcBlockK, n0, full + s);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(N_TILE, a.bf16);
            for (int kb = 0; kb < num_kb; kb++) {
                const int s = kb % STAGES;
                if (!tc_wait(full + s, (kb / STAGES) & 1, a.error)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint8_t* sa = tiles + (size_t)s * S::STAGE_BYTES;
                const uint64_t da = umma_smem_desc_sw128(sa), db = umma_smem_desc_sw128(sa + S::A_BYTES);
                const uint64_t da2 = DUAL ? umma_smem_desc_sw128(sa + W_BYTES) : 0;
#pragma unroll
                for (int k = 0; k < kTcBlockK / 16; k++) {
                    // advancing 16 elements along K inside the swizzled row = 32 bytes = 2 descriptor units
                    const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                    umma_f16(tmem_acc, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, accumulate);
                    if (DUAL) umma_f16(tmem_acc + (uint32_t)N_TILE, da2 + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, accumulate);
                }
                // the stage may be refilled once these MMAs have read it
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(empty + s)) : "memory");
            }
            // accumulator complete (or abandoned): release the epilogue either way
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(acc_ready)) : "memory");
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> global ----------------
        const bool ok = tc_wait(acc_ready, 0, a.error) && __ldcg(a.error) == 0 && num_kb > 0;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int lane_base = 32 * (warp & 3);
        const int m = m0 + lane_base + lane;
        // kernel parameters used per column live in registers for the whole loop
        const int epilogue = a.epilogue, M = ESP_TC_G(M), ldo = ESP_TC_G(ldo), row_offset = a.row_offset, ld16 = a.ld16, bf16 = a.bf16;
        const bool atomic_out = a.atomic_out != 0;
        const bool row_ok = ok && m < M;
        const float* const bias_p = ESP_TC_G(bias);
        const float bias = (row_ok && bias_p && blockIdx.z == 0) ? bias_p[m] : 0.f;
        float* const out = ESP_TC_G(out);
#undef ESP_TC_G
        float* const logits = a.logits;
        float* const debug = a.debug;
        uint16_t* const out16 = a.out16;
        unsigned long long* const best = a.best;
#pragma unroll 1
        for (int c0 = 0; c0 < N_TILE; c0 += 16) {
            const uint32_t live = s_live16[c0 >> 4];  // warp-uniform
            if (!live) continue;
            uint32_t r[16];
            const uint32_t taddr = tmem_acc + ((uint32_t)lane_base << 16) + (uint32_t)c0;
            tmem_ld16(taddr, r);
            uint32_t r2[16];
            if (DUAL) tmem_ld16(taddr + (uint32_t)N_TILE, r2);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const int nb = n0 + c0;
            if (epilogue == TC_HEAD) {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    if (!((live >> j) & 1u)) continue;
                    const int n = nb + j;
                    const float v = __uint_as_float(r[j]) + bias;
                    // first-max over the 32 rows of this warp, then one packed atomicMax per batch row
                    float bv = row_ok ? v : -INFINITY;
                    int bi = row_ok ? m + row_offset : 0x7fffffff;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
                    }
                    if (lane == 0 && bi != 0x7fffffff) atomicMax(best + n, pack_best(bv, bi));
                    if (logits && row_ok) logits[(size_t)n * M + m] = v;
                }
            } else if (epilogue == TC_GELU16 || epilogue == TC_SWIGLU16) {
                if (row_ok) {
                    uint16_t* o = out16 + (size_t)nb * ld16 + m;
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        if (!((live >> j) & 1u)) continue;
                        float v;
                        if (DUAL) v = silu_f(__uint_as_float(r[j])) * __uint_as_float(r2[j]);
                        else v = gelu_f(__uint_as_float(r[j]) + bias);
                        o[(size_t)j * ld16] = bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
                        if (debug && nb + j == 0) debug[m] = v;
                    }
                }
            } else if (row_ok) {
                float* o = out + (size_t)nb * ldo + m;
                if (atomic_out) {
#pragma unroll
                    for (int j = 0; j < 16; j++)
                        if ((live >> j) & 1u) atomicAdd(o + (size_t)j * ldo, __uint_as_float(r[j]) + bias);
                } else {
                    float prev[16];
                    if (epilogue == TC_RESIDUAL) {
#pragma unroll
                        for (int j = 0; j < 16; j++) prev[j] = ((live >> j) & 1u) ? o[(size_t)j * ldo] : 0.f;
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j++) prev[j] = 0.f;
                    }
#pragma unroll
                    for (int j = 0; j < 16; j++)
                        if ((live >> j) & 1u) o[(size_t)j * ldo] = prev[j] + (__uint_as_float(r[j]) + bias);
                }
            }
        }
    }
    // tensor memory is released by the warp that allocated it, after everybody is done with it
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)S::TMEM_COLS) : "memory");
    }
}

}  // namespace esp
