// Dense "skinny" GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for the batched parts of the decode
// path: Y[n][m] = sum_k W[m][k] * X[n][k] for a weight matrix W [M, K] (row-major, fp16 or bf16) and a batch of
// activation rows X [N, K] (the same 16-bit type), N = 16..256 rows per launch.
//
// Mapping: the weight rows are the MMA's M dimension (128 per CTA), the batch is its N dimension, so a CTA
// streams its 128 x K slice of W exactly once whatever the batch size.  Operands are staged in shared memory by
// TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast), the fp32 accumulator lives in tensor memory
// (128 lanes x N columns) and is read back with tcgen05.ld for the epilogue.
//
// Warp roles (192 threads): warp 0 allocates tensor memory and issues the TMA loads, warp 1 issues the MMAs
// (one elected thread), warps 2..5 run the epilogue (a warp may only touch the TMEM lanes 32*(warp%4)..+31).
// Every mbarrier wait is bounded; on a timeout the kernel records an error and unwinds normally.
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

enum TcEpilogue { TC_STORE = 0, TC_RESIDUAL = 1, TC_HEAD = 2 };

struct TcArgs {
    int M, K, n_valid;          // weight rows, reduction length (multiple of 64), live batch rows
    int epilogue;               // TcEpilogue
    float* out;                 // [n][ldo] fp32 (TC_STORE: overwritten, TC_RESIDUAL: accumulated into)
    int ldo;
    const float* bias;          // [M] or null
    const int* active;          // [n] or null: rows with active == 0 are not written
    unsigned long long* best;   // TC_HEAD: packed running first-max per batch row
    float* logits;              // TC_HEAD: optional [n][M] logits store, or null
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

// N_TILE: accumulator columns (batch rows covered by the launch), a multiple of 16 in [16, 256].
template <int N_TILE, int STAGES>
__global__ void __launch_bounds__(kTcThreads) k_gemm_tc(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                                                        const TcArgs a) {
    extern __shared__ __align__(1024) uint8_t tc_smem[];
    constexpr int A_BYTES = kTcBlockM * kTcBlockK * 2;
    constexpr int B_BYTES = N_TILE * kTcBlockK * 2;
    constexpr int STAGE_BYTES = A_BYTES + ((B_BYTES + 1023) / 1024) * 1024;
    constexpr int TMEM_COLS = N_TILE < 32 ? 32 : N_TILE;  // power of two >= 32 (N_TILE is 16/32/64/128/256)
    uint8_t* tiles = reinterpret_cast<uint8_t*>(((uintptr_t)tc_smem + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_ready = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);

    // which batch rows are written (live and active), fetched once: one 16-bit mask per group of 16 columns
    __shared__ uint32_t s_live16[16];
    if (threadIdx.x < 16) {
        uint32_t mask = 0;
        for (int j = 0; j < 16; j++) {
            const int n = threadIdx.x * 16 + j;
            if (n < N_TILE && n < a.n_valid && (!a.active || a.active[n])) mask |= 1u << j;
        }
        s_live16[threadIdx.x] = mask;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * kTcBlockM;
    const int num_kb = a.K / kTcBlockK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        mbar_init(acc_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {  // the whole warp allocates the accumulator columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
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
                if (kb >= STAGES && !tc_wait(empty + s, ((kb / STAGES) - 1) & 1, a.error)) break;
                uint8_t* sa = tiles + (size_t)s * STAGE_BYTES;
                mbar_expect_tx(full + s, A_BYTES + B_BYTES);
                tma_load_2d(sa, &map_w, kb * kTcBlockK, m0, full + s);
                tma_load_2d(sa + A_BYTES, &map_x, kb * kTcBlockK, 0, full + s);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(N_TILE, a.bf16);
            bool ok = true;
            for (int kb = 0; kb < num_kb && ok; kb++) {
                const int s = kb % STAGES;
                ok = tc_wait(full + s, (kb / STAGES) & 1, a.error);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint8_t* sa = tiles + (size_t)s * STAGE_BYTES;
                const uint64_t da = umma_smem_desc_sw128(sa), db = umma_smem_desc_sw128(sa + A_BYTES);
#pragma unroll
                for (int k = 0; k < kTcBlockK / 16; k++) {
                    // advancing 16 elements along K inside the swizzled row = 32 bytes = 2 descriptor units
                    const uint64_t dak = da + (uint64_t)(2 * k), dbk = db + (uint64_t)(2 * k);
                    const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                        ::"r"(tmem_acc), "l"(dak), "l"(dbk), "r"(idesc), "r"(accumulate)
                        : "memory");
                }
                // the stage may be refilled once these MMAs have read it
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(empty + s)) : "memory");
            }
            // accumulator complete (or abandoned): release the epilogue either way
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(acc_ready)) : "memory");
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> global ----------------
        const bool ok = tc_wait(acc_ready, 0, a.error) && __ldcg(a.error) == 0;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int lane_base = 32 * (warp & 3);
        const int m = m0 + lane_base + lane;
        const bool row_ok = ok && m < a.M;
        const float bias = (row_ok && a.bias) ? a.bias[m] : 0.f;
        // kernel parameters used per column live in registers for the whole loop
        const int epilogue = a.epilogue, ldo = a.ldo, M = a.M, row_offset = a.row_offset;
        float* const out = a.out;
        float* const logits = a.logits;
        unsigned long long* const best = a.best;
#pragma unroll 1
        for (int c0 = 0; c0 < N_TILE; c0 += 16) {
            const uint32_t live = s_live16[c0 >> 4];  // bit j: batch row c0 + j is written (warp-uniform)
            if (!live) continue;
            uint32_t r[16];
            const uint32_t taddr = tmem_acc + ((uint32_t)lane_base << 16) + (uint32_t)c0;
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                  "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                : "r"(taddr)
                : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (epilogue == TC_HEAD) {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    if (!((live >> j) & 1u)) continue;
                    const int n = c0 + j;
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
            } else if (row_ok) {
                float* o = out + (size_t)c0 * ldo + m;
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
    // tensor memory is released by the warp that allocated it, after everybody is done with it
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

template <int N_TILE, int STAGES>
constexpr size_t tc_smem_bytes() {
    return (size_t)STAGES * (kTcBlockM * kTcBlockK * 2 + ((N_TILE * kTcBlockK * 2 + 1023) / 1024) * 1024) + (2 * STAGES + 1) * 8 + 16 + 1024;
}

}  // namespace esp
