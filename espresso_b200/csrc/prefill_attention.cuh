// Causal attention for prompt passes: rows that are consecutive positions of one sequence, in tiles of 64 rows.
//
// The row-wise attention kernel gives every (row, head) a warp that streams the whole visible K/V range of its
// sequence; for a 256-row prompt pass at context 400 that is 1.8 GB of cache reads per layer out of L2 (half of the
// pass time on the 8B shape).  Here a CTA owns 64 query rows of one head: K and V travel once per tile of 64 positions
// through shared memory (cp.async, two stages) and the products QK^T and PV run on the tensor cores
// (mma.sync.m16n8k16, fp16 operands as the cache stores them, fp32 accumulation) with the online softmax of the
// reference's decode attention (max subtraction, Sources/CPUOps/Attention... restated in oracle/espresso_oracle.c) kept in
// registers.  One warp = 16 query rows; scores never leave the registers: the accumulator layout of QK^T is the A
// operand layout of PV.
//
// Shared-memory tiles are [row][HD] halves with the 16-byte chunks of a row XOR-swizzled by the row index, which makes
// both the cp.async stores and the ldmatrix loads conflict-free.
#pragma once
#include "batch_kernels.cuh"

namespace esp {

constexpr int kPfRows = 64;       // query rows per CTA
constexpr int kPfCols = 64;       // cache positions per step
constexpr int kPfThreads = 128;   // 4 warps x 16 rows

struct PrefillAttArgs {
    ModelDims m;
    RowState rs;
    KvLayout kv;
    const float* q;    // [rows][q_dim] fp32, RoPE applied
    uint16_t* ctx16;   // [rows][q_dim] fp16/bf16
    int bf16;
    int layer;
    int rows;
    float* debug;      // optional fp32 capture of row 0's context, or null
};

template <int HD>
__host__ __device__ constexpr int pf_smem_bytes() { return (kPfRows + 4 * kPfCols) * HD * 2; }  // Q + two stages of K and V

// Byte offset of 16-byte chunk `c` of row `r` in a swizzled [rows][HD] fp16 tile.
template <int HD>
__device__ __forceinline__ uint32_t pf_off(int r, int c) {
    constexpr int kChunks = HD / 8;
    constexpr int kMask = kChunks < 8 ? kChunks - 1 : 7;
    return (uint32_t)(r * (HD * 2) + ((c ^ (r & kMask)) << 4));
}

__device__ __forceinline__ void pf_cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void pf_ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void pf_ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void pf_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pf_pack(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// grid = (row tiles, query heads).  The host launches this kernel only for passes in which every tile's rows are
// active, belong to one sequence and sit at consecutive positions (Engine::upload_rows checks it).
template <int HD>
__global__ void __launch_bounds__(kPfThreads) k_attention_prefill(const PrefillAttArgs p) {
    extern __shared__ __align__(128) uint8_t pf_smem[];
    const ModelDims& m = p.m;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * kPfRows;
    const int n_rows = min(kPfRows, p.rows - row0);
    const int head = blockIdx.y;
    const int kvh = head / (m.n_head / m.n_kv_head);
    constexpr int kChunks = HD / 8;   // 16-byte chunks per row
    constexpr int kSteps = HD / 16;   // k-steps of QK^T
    constexpr int kOut = HD / 8;      // n-tiles of the output
    const uint32_t sQ = (uint32_t)__cvta_generic_to_shared(pf_smem);
    const uint32_t sK = sQ + kPfRows * HD * 2;                 // two stages
    const uint32_t sV = sK + 2 * kPfCols * HD * 2;             // two stages
    pdl_launch_dependents();
    pdl_wait();
    const int seq = p.rs.seq[row0], pos0 = p.rs.pos[row0];
    const int last_pos = pos0 + n_rows - 1;                    // newest visible position of the tile
    const int n_tiles = last_pos / kPfCols + 1;
    const __half* Kbase = p.kv.k + p.kv.offset(m, p.layer, seq, kvh, 0);
    const __half* Vbase = p.kv.v + p.kv.offset(m, p.layer, seq, kvh, 0);

    auto load_kv = [&](int tile, int stage) {
        const int n0 = tile * kPfCols;
        for (int i = tid; i < kPfCols * kChunks; i += kPfThreads) {
            const int r = i / kChunks, c = i - r * kChunks;
            const uint32_t off = (uint32_t)(stage * kPfCols * HD * 2) + pf_off<HD>(r, c);
            if (n0 + r <= last_pos) {
                pf_cp_async16(sK + off, Kbase + (size_t)(n0 + r) * HD + c * 8);
                pf_cp_async16(sV + off, Vbase + (size_t)(n0 + r) * HD + c * 8);
            } else {  // beyond the visible range: zeros (their scores are masked, but 0 * NaN must not reach the output)
                *reinterpret_cast<uint4*>(pf_smem + (sK - sQ) + off) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(pf_smem + (sV - sQ) + off) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    load_kv(0, 0);
    // the query tile, scaled by 1/sqrt(HD), as fp16
    {
        const float scale = 1.0f / sqrtf((float)HD);
        for (int i = tid; i < kPfRows * kChunks; i += kPfThreads) {
            const int r = i / kChunks, c = i - r * kChunks;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < n_rows) {
                const float4* src = reinterpret_cast<const float4*>(p.q + (size_t)(row0 + r) * m.q_dim + head * HD + c * 8);
                const float4 a = src[0], b = src[1];
                v.x = pf_pack(a.x * scale, a.y * scale); v.y = pf_pack(a.z * scale, a.w * scale);
                v.z = pf_pack(b.x * scale, b.y * scale); v.w = pf_pack(b.z * scale, b.w * scale);
            }
            *reinterpret_cast<uint4*>(pf_smem + pf_off<HD>(r, c)) = v;
        }
    }
    __syncthreads();
    // this warp's 16 query rows as A fragments, kept in registers for every tile
    uint32_t qa[kSteps][4];
#pragma unroll
    for (int ks = 0; ks < kSteps; ks++) {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = ks * 2 + (lane >> 4);
        pf_ldmatrix_x4(sQ + pf_off<HD>(r, c), qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
    }
    float o[kOut][4];
#pragma unroll
    for (int j = 0; j < kOut; j++) { o[j][0] = 0.f; o[j][1] = 0.f; o[j][2] = 0.f; o[j][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // rows g and g + 8 of the warp
    const int my_pos[2] = {pos0 + warp * 16 + g, pos0 + warp * 16 + g + 8};

    for (int tile = 0; tile < n_tiles; tile++) {
        const int stage = tile & 1;
        if (tile + 1 < n_tiles) {
            load_kv(tile + 1, stage ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const uint32_t kS = sK + stage * kPfCols * HD * 2, vS = sV + stage * kPfCols * HD * 2;
        const int n0 = tile * kPfCols;
        // a warp whose rows all lie before this tile has nothing to add (causal), but it still takes part in the barriers
        const bool active = n0 <= pos0 + warp * 16 + 15;
        if (active) {
            // ---- S = Q K^T for 16 rows x 64 positions
            float sc[8][4];
#pragma unroll
            for (int j = 0; j < 8; j++) { sc[j][0] = 0.f; sc[j][1] = 0.f; sc[j][2] = 0.f; sc[j][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < kSteps; ks++) {
#pragma unroll
                for (int jp = 0; jp < 4; jp++) {  // pairs of 8-position groups
                    uint32_t b0, b1, b2, b3;
                    const int r = jp * 16 + (lane & 7) + (lane >> 4) * 8, c = ks * 2 + ((lane >> 3) & 1);
                    pf_ldmatrix_x4(kS + pf_off<HD>(r, c), b0, b1, b2, b3);
                    pf_mma(sc[2 * jp], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
                    pf_mma(sc[2 * jp + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
                }
            }
            // ---- causal mask (only tiles that reach past the row's position need it) and the online softmax
            const bool diag = n0 + kPfCols - 1 > pos0 + warp * 16;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 8; j++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int col = n0 + j * 8 + 2 * t + (e & 1), rr = e >> 1;
                    if (diag && col > my_pos[rr]) sc[j][e] = -INFINITY;
                    mx[rr] = fmaxf(mx[rr], sc[j][e]);
                }
            }
            float corr[2];
#pragma unroll
            for (int rr = 0; rr < 2; rr++) {
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
                const float m_new = fmaxf(m_run[rr], mx[rr]);
                // position 0 is visible to every row, so m_new is finite from the first tile on
                corr[rr] = m_run[rr] == -INFINITY ? 0.f : __expf(m_run[rr] - m_new);
                m_run[rr] = m_new;
            }
            float rs[2] = {0.f, 0.f};
            uint32_t pa[4][4];  // P as A fragments: k-step kk covers positions 16 kk .. 16 kk + 15
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float p0 = __expf(sc[j][0] - m_run[0]), p1 = __expf(sc[j][1] - m_run[0]);
                const float p2 = __expf(sc[j][2] - m_run[1]), p3 = __expf(sc[j][3] - m_run[1]);
                rs[0] += p0 + p1;
                rs[1] += p2 + p3;
                pa[j >> 1][(j & 1) * 2] = pf_pack(p0, p1);
                pa[j >> 1][(j & 1) * 2 + 1] = pf_pack(p2, p3);
            }
#pragma unroll
            for (int rr = 0; rr < 2; rr++) {
                rs[rr] += __shfl_xor_sync(0xffffffffu, rs[rr], 1);
                rs[rr] += __shfl_xor_sync(0xffffffffu, rs[rr], 2);
                l_run[rr] = l_run[rr] * corr[rr] + rs[rr];
            }
#pragma unroll
            for (int j = 0; j < kOut; j++) { o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1]; }
            // ---- O += P V
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
#pragma unroll
                for (int jp = 0; jp < kOut / 2; jp++) {  // pairs of 8-channel groups
                    uint32_t b0, b1, b2, b3;
                    const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = jp * 2 + (lane >> 4);
                    pf_ldmatrix_x4_trans(vS + pf_off<HD>(r, c), b0, b1, b2, b3);
                    pf_mma(o[2 * jp], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                    pf_mma(o[2 * jp + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
                }
            }
        }
        __syncthreads();  // every warp is done with this stage before the next load overwrites it
    }
    // ---- normalise and store 16-bit context rows
#pragma unroll
    for (int rr = 0; rr < 2; rr++) {
        const int r = warp * 16 + g + rr * 8;
        if (r >= n_rows) continue;
        const float inv = l_run[rr] > 0.f ? 1.0f / l_run[rr] : 0.f;
        uint16_t* dst = p.ctx16 + (size_t)(row0 + r) * m.q_dim + head * HD;
#pragma unroll
        for (int j = 0; j < kOut; j++) {
            const float v0 = o[j][rr * 2] * inv, v1 = o[j][rr * 2 + 1] * inv;
            const uint32_t packed = (uint32_t)to_16bit(v0, p.bf16) | ((uint32_t)to_16bit(v1, p.bf16) << 16);
            *reinterpret_cast<uint32_t*>(dst + j * 8 + 2 * t) = packed;
            if (p.debug && row0 + r == 0) { p.debug[head * HD + j * 8 + 2 * t] = v0; p.debug[head * HD + j * 8 + 2 * t + 1] = v1; }
        }
    }
}

}  // namespace esp
