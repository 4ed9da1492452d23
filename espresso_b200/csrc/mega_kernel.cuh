// Persistent whole-loop decode kernel for one sequence of a Llama-style fp16 model.
//
// One cooperative launch runs an entire greedy decode loop: `n_steps` heads and `n_steps - 1` forward passes.
// The grid has one CTA per SM.  Inside a CTA one producer warp streams that CTA's weights from HBM into a
// shared-memory ring with bulk async copies (cp.async.bulk + mbarrier), always running ahead of the eight
// consumer warps, so HBM stays busy while the consumers wait on the activation dependencies of the step.
// Weights are re-laid out once ("pack") so that everything a CTA needs for one layer is contiguous.
//
// Per layer the consumers run three stages separated by grid barriers:
//   S1  norm -> rows of Wq/Wk/Wv -> RoPE -> q buffer / KV-cache append          (inner-product form)
//   S2  attention for one head (recomputed by the CTAs that share the head) -> partial Wo product for a
//       block of output rows -> atomic add into the residual stream             (per-head partial sums)
//   S3  norm -> gate/up rows -> SiLU*up -> partial W2 product (W2 stored transposed) -> atomic add
// and the LM head streams the CTA's vocab rows through the same ring and keeps a first-max argmax.
// The residual stream rotates through three buffers so that a stage never accumulates into a vector that
// other CTAs may still be reading.  Every wait (mbarrier, grid barrier) is bounded: when a limit is hit the
// kernel records an error code, stops waiting everywhere and runs to completion; the host reports a timeout.
#pragma once
#include "decode_kernels.cuh"

namespace esp {

constexpr int kMegaConsumerWarps = 8;
constexpr int kMegaConsumers = kMegaConsumerWarps * 32;
constexpr int kMegaThreads = kMegaConsumers + 32;  // + one producer warp
constexpr unsigned kMegaSpinLimit = 1u << 21;  // attempts per wait before the kernel gives up (a few seconds)

struct MegaPlan {
    int n_cta;
    int ppc;          // S1: RoPE row pairs per CTA
    int blocks, rpb;  // S2: output-row blocks per head, rows per block
    int hpc;          // S3: FFN hidden units per CTA
    int vpc;          // head: vocab rows per CTA
    int head_rows_per_chunk, head_chunks;
    int row_bytes;    // d_model * 2
    int s1_bytes, s2_bytes, s3a_bytes, s3b_bytes, head_chunk_bytes;  // packed bytes of a stage per layer / of a head chunk (multiples of 128)
    // A stage whose slice is larger than a ring slot arrives in several chunks of whole items:
    int s1_ipc;       // S1 row pairs per chunk
    int s2_rpc;       // S2 projection rows per chunk (a multiple of the rows one pass of the CTA covers)
    int s3a_ipc;      // S3 (gate, up) pairs per chunk
    int s3b_rpc;      // S3 down-projection rows per chunk
    int slot_bytes, n_slots;
    long long layer_bytes, cta_bytes;  // packed bytes per CTA: one layer, everything
    int smem_bytes;
};

struct MegaArgs {
    ModelDims m;
    MegaPlan plan;
    const uint8_t* pack;      // [n_cta][cta_bytes]
    const float* norms;       // [2*L + 1][d_model]: norm1(l), norm2(l), ..., final
    const uint16_t* tok_emb;  // fp16 [vocab][d_model]
    const float2* rope;       // [max_seq][head_dim/2]
    KvLayout kv;
    float* q;                 // [q_dim]
    float* xbuf;              // [3][d_model] rotating residual-stream buffers
    float* hidden_io;         // [d_model] last hidden state of the sequence (in and out)
    unsigned long long* best; // [2]
    unsigned int* barrier;    // [1] monotonic arrival counter, zero at launch
    int* error;               // [1] 0 = ok
    unsigned long long* stamps; // [2] globaltimer at kernel start and when the first token is known
    unsigned long long* token_times; // optional [n_steps] globaltimer (ns) at which each token became known, or null
    long long* trace;         // optional [14*L + 4] SM clock stamps of the last step taken by CTA `trace_cta`, or null
    int trace_cta;
    RowState rs;              // row 0 carries pos / tok / n_out / out
    int n_steps;              // tokens to emit (>= 1)
    int pos0;                 // visible tokens at launch
};

// ------------------------------------------------------------------------------------------------ PTX helpers

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(1000u)  // each attempt may sleep for at most about a microsecond
        : "memory");
    return ok != 0;
}
// Weight chunks carry an evict-first L2 policy: they are used once per token, and keeping them out of the way
// leaves the KV cache, the residual stream and the small per-layer vectors resident in L2.
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 lds128(const uint8_t* p) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(smem_u32(p)));
    return r;
}
__device__ __forceinline__ uint2 lds64(const uint8_t* p) {
    uint2 r;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "r"(smem_u32(p)));
    return r;
}
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kMegaConsumers) : "memory"); }

// ------------------------------------------------------------------------------------------------ shared state

struct MegaShared {
    uint8_t* slots;
    uint64_t* full;
    uint64_t* empty;
    float* xs;    // staged (normalised) activation vector, lane-major order (see xs_index)
    float* qs;    // [head_dim]
    float* ctx;   // [head_dim]
    float* sc;    // [max_seq] attention scores
    float* part;  // [warps][head_dim]
    float* red;   // [32]
    float* act;   // [hpc]
    int* abort;   // [1]
};

__device__ __forceinline__ MegaShared mega_carve(uint8_t* base, const MegaArgs& a) {
    MegaShared s;
    const MegaPlan& p = a.plan;
    s.slots = base;
    uint8_t* q = base + (size_t)p.n_slots * p.slot_bytes;
    s.full = reinterpret_cast<uint64_t*>(q); q += 8 * p.n_slots;
    s.empty = reinterpret_cast<uint64_t*>(q); q += 8 * p.n_slots;
    q = reinterpret_cast<uint8_t*>(((uintptr_t)q + 15) & ~(uintptr_t)15);
    s.xs = reinterpret_cast<float*>(q); q += sizeof(float) * xs_floats<8>(a.m.d_model);
    s.qs = reinterpret_cast<float*>(q); q += sizeof(float) * a.m.head_dim;
    s.ctx = reinterpret_cast<float*>(q); q += sizeof(float) * a.m.head_dim;
    s.sc = reinterpret_cast<float*>(q); q += sizeof(float) * a.m.max_seq;
    s.part = reinterpret_cast<float*>(q); q += sizeof(float) * kMegaConsumerWarps * a.m.head_dim;
    s.red = reinterpret_cast<float*>(q); q += sizeof(float) * 32;
    s.act = reinterpret_cast<float*>(q); q += sizeof(float) * ((p.hpc + 3) & ~3);
    s.abort = reinterpret_cast<int*>(q);
    return s;
}

__host__ __device__ inline int mega_smem_bytes(const ModelDims& m, const MegaPlan& p) {
    size_t b = (size_t)p.n_slots * p.slot_bytes + 16 * p.n_slots + 16;
    b += sizeof(float) * (size_t)(xs_floats<8>(m.d_model) + 2 * m.head_dim + m.max_seq + kMegaConsumerWarps * m.head_dim + 32 + ((p.hpc + 3) & ~3));
    return (int)(b + 64);
}

__device__ __forceinline__ void mega_fail(const MegaArgs& a, const MegaShared& s, int code) {
    *s.abort = 1;
    atomicCAS(a.error, 0, code);
}

// Bounded wait on an mbarrier phase.  Returns immediately once the kernel is aborting.
__device__ __forceinline__ void mega_wait(const MegaArgs& a, const MegaShared& s, uint64_t* bar, unsigned parity, int code) {
    if (*reinterpret_cast<volatile int*>(s.abort)) return;
    unsigned spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (++spins > kMegaSpinLimit || ((spins & 0xfffu) == 0 && (__ldcg(a.error) != 0 || *reinterpret_cast<volatile int*>(s.abort)))) {
            mega_fail(a, s, code);
            return;
        }
    }
}

// Grid-wide barrier of the consumer threads of all CTAs: arrivals are counted on one global counter.
// (A flag word per CTA polled by one thread each was measured slower on B200: 6 us against 2-3 us.)
__device__ __forceinline__ void mega_grid_sync(const MegaArgs& a, const MegaShared& s, unsigned& epoch) {
    consumer_sync();
    epoch++;
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(a.barrier, 1u);
        const unsigned target = epoch * (unsigned)a.plan.n_cta;
        if (!*reinterpret_cast<volatile int*>(s.abort)) {
            unsigned spins = 0;
            while (ld_acquire_u32(a.barrier) < target) {
                if (++spins > kMegaSpinLimit || ((spins & 0x3ffu) == 0 && __ldcg(a.error) != 0)) {
                    mega_fail(a, s, 2);
                    break;
                }
            }
        }
        __threadfence();
    }
    consumer_sync();
}

// Ring bookkeeping shared by the producer and the consumers: chunk c lives in slot c % n_slots.
struct ChunkCursor {
    unsigned c = 0;
};

__device__ __forceinline__ const uint8_t* mega_acquire(const MegaArgs& a, const MegaShared& s, unsigned c) {
    const unsigned slot = c % (unsigned)a.plan.n_slots;
    // one lane per warp polls the barrier (256 threads polling one shared-memory word serialise); the warp barrier
    // that follows orders the other lanes' reads of the chunk after the observed completion
    if ((threadIdx.x & 31) == 0) mega_wait(a, s, s.full + slot, (c / (unsigned)a.plan.n_slots) & 1u, 3);
    __syncwarp();
    return s.slots + (size_t)slot * a.plan.slot_bytes;
}
__device__ __forceinline__ void mega_release(const MegaArgs& a, const MegaShared& s, unsigned c) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(s.empty + (c % (unsigned)a.plan.n_slots));
}

// ------------------------------------------------------------------------------------------------ consumer pieces

__device__ __forceinline__ float mega_block_sum(float v, float* red) {
    v = warp_sum(v);
    consumer_sync();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    consumer_sync();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kMegaConsumerWarps; i++) t += red[i];
    return t;
}

// Loads a d_model vector (fp32 from L2, or an fp16 embedding row), RMS-normalises it and stages it.
__device__ __forceinline__ void mega_stage_norm(const MegaArgs& a, const MegaShared& s, const float* src, const uint16_t* emb_row,
                                                const float* gain) {
    constexpr int VMAX = 16;  // d_model <= 4096
    const int d = a.m.d_model;
    float xv[VMAX];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VMAX; i++) {
        const int k = threadIdx.x + i * kMegaConsumers;
        xv[i] = 0.f;
        if (k < d) xv[i] = emb_row ? __half2float(__ushort_as_half(emb_row[k])) : __ldcg(src + k);
        ss = fmaf(xv[i], xv[i], ss);
    }
    ss = mega_block_sum(ss, s.red);
    const float inv = 1.0f / sqrtf(ss / (float)d + a.m.eps);
#pragma unroll
    for (int i = 0; i < VMAX; i++) {
        const int k = threadIdx.x + i * kMegaConsumers;
        if (k < d) s.xs[xs_index<8>(k)] = (xv[i] * inv) * gain[k];
    }
    consumer_sync();
}

// Products of one 16-byte vector of fp16 weights with 8 activations, split over two accumulators so that the
// dependent FMA chain is 4 long instead of 8.
__device__ __forceinline__ void mega_fma8(const uint4& w, const float4& xa, const float4& xb, float& even, float& odd) {
    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
    const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&w.z));
    const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&w.w));
    even = fmaf(f0.x, xa.x, even); odd = fmaf(f0.y, xa.y, odd);
    even = fmaf(f1.x, xa.z, even); odd = fmaf(f1.y, xa.w, odd);
    even = fmaf(f2.x, xb.x, even); odd = fmaf(f2.y, xb.y, odd);
    even = fmaf(f3.x, xb.z, even); odd = fmaf(f3.y, xb.w, odd);
}

// Dot products of NR fp16 rows held in shared memory (row r at base + r * row_bytes) with the staged vector; the
// results are in every lane.  Two 256-element slices are in flight per pass: all of their shared-memory loads are
// issued before the first multiply, and every row has four independent accumulators (the consumer warps are too
// few to hide the load and FMA latencies of a one-slice-at-a-time loop: that form measured ~400 cycles per slice).
template <int NR>
__device__ __forceinline__ void mega_dot_rows(const uint8_t* base, int row_bytes, int K, const float* xs, int lane, float (&o)[NR]) {
    const float4* xs4 = reinterpret_cast<const float4*>(xs);
    float acc[NR][4];
#pragma unroll
    for (int r = 0; r < NR; r++) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
    const int iters = (K + 255) / 256;
    for (int it = 0; it < iters; it += 2) {
        const int k0 = it * 256 + lane * 8, k1 = k0 + 256;
        const bool in0 = k0 < K, in1 = k1 < K;
        uint4 w0[NR], w1[NR];
#pragma unroll
        for (int r = 0; r < NR; r++) {
            w0[r] = in0 ? lds128(base + (size_t)r * row_bytes + (size_t)k0 * 2) : make_uint4(0, 0, 0, 0);
            w1[r] = in1 ? lds128(base + (size_t)r * row_bytes + (size_t)k1 * 2) : make_uint4(0, 0, 0, 0);
        }
        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 xa0 = in0 ? xs4[(it * 2) * 32 + lane] : z, xb0 = in0 ? xs4[(it * 2 + 1) * 32 + lane] : z;
        const float4 xa1 = in1 ? xs4[(it * 2 + 2) * 32 + lane] : z, xb1 = in1 ? xs4[(it * 2 + 3) * 32 + lane] : z;
#pragma unroll
        for (int r = 0; r < NR; r++) {
            mega_fma8(w0[r], xa0, xb0, acc[r][0], acc[r][1]);
            mega_fma8(w1[r], xa1, xb1, acc[r][2], acc[r][3]);
        }
    }
    float t[NR];
#pragma unroll
    for (int r = 0; r < NR; r++) t[r] = (acc[r][0] + acc[r][1]) + (acc[r][2] + acc[r][3]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int r = 0; r < NR; r++) t[r] += __shfl_xor_sync(0xffffffffu, t[r], off);
    }
#pragma unroll
    for (int r = 0; r < NR; r++) o[r] = t[r];
}

// Two rows at arbitrary addresses (r1 - r0 is the row pitch).
__device__ __forceinline__ void mega_dot2(const uint8_t* r0, const uint8_t* r1, int K, const float* xs, int lane, float& o0, float& o1) {
    float o[2];
    mega_dot_rows<2>(r0, (int)(r1 - r0), K, xs, lane, o);
    o0 = o[0];
    o1 = o[1];
}

__device__ __forceinline__ void mega_dot4(const uint8_t* base, int row_bytes, int K, const float* xs, int lane, float (&o)[4]) {
    mega_dot_rows<4>(base, row_bytes, K, xs, lane, o);
}

// S1: q/k/v rows of this CTA (pairs that RoPE rotates together), RoPE, q store and KV-cache append.
__device__ __forceinline__ void mega_s1(const MegaArgs& a, const MegaShared& s, int layer, int pos, const uint8_t* chunk, int i0, int n_items) {
    const ModelDims& m = a.m;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half = m.head_dim / 2;
    const int q_items = m.q_dim / 2, k_items = m.kv_dim / 2, total = q_items + 2 * k_items;
    for (int i = warp; i < n_items; i += kMegaConsumerWarps) {  // i: item inside the chunk, i0 + i: item of this CTA
        const int item = blockIdx.x * a.plan.ppc + i0 + i;
        if (item >= total) break;
        float v0, v1;
        mega_dot2(chunk + (size_t)(2 * i) * a.plan.row_bytes, chunk + (size_t)(2 * i + 1) * a.plan.row_bytes, m.d_model, s.xs, lane, v0, v1);
        if (lane == 0) {
            int kind, local;
            if (item < q_items) { kind = 0; local = item; }
            else if (item < q_items + k_items) { kind = 1; local = item - q_items; }
            else { kind = 2; local = item - q_items - k_items; }
            int row0, row1;
            if (kind < 2) {
                const int head = local / half, idx = local - head * half;
                row0 = head * m.head_dim + idx; row1 = row0 + half;
                const float2 cs = a.rope[(size_t)pos * half + idx];
                const float r0 = v0 * cs.x - v1 * cs.y, r1 = v0 * cs.y + v1 * cs.x;
                v0 = r0; v1 = r1;
            } else { row0 = 2 * local; row1 = row0 + 1; }
            if (kind == 0) { a.q[row0] = v0; a.q[row1] = v1; }
            else {
                __half* base = kind == 1 ? a.kv.k : a.kv.v;
                const int kvh = row0 / m.head_dim;
                const size_t off = a.kv.offset(m, layer, 0, kvh, pos);
                base[off + (row0 - kvh * m.head_dim)] = __float2half_rn(v0);
                base[off + (row1 - kvh * m.head_dim)] = __float2half_rn(v1);
            }
        }
    }
}

// S2: attention of one head over positions [0, pos], then this CTA's block of the output projection.
// Each warp owns the positions t = warp + 8*i (i < 32 per round).  Four neighbouring lanes share one position:
// each loads a quarter of its K row with 16-byte vectors (a warp instruction touches 8 cache lines, not 32) and the
// score is completed with two shuffles.  The probabilities are then broadcast position by position while every
// lane accumulates its own channels of V.  K and V rows are requested before the query is even staged, and the
// eight per-warp (max, sum, ctx) triples are merged once.
template <int HD>
__device__ __forceinline__ void mega_s2_t(const MegaArgs& a, const MegaShared& s, int layer, int pos, unsigned& c, const float* x_in,
                                          const uint16_t* emb_row, float* x_mid) {
    const ModelDims& m = a.m;
    const MegaPlan& p = a.plan;
    const int units = m.n_head * p.blocks;
    if ((int)blockIdx.x >= units) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int hd = HD;
    constexpr int cpl = HD / 32;  // V channels per lane (head_dim 32/64/128 -> 1/2/4)
    constexpr int KV4 = HD / 32;  // 16-byte vectors of a K row quarter
    const int head = blockIdx.x / p.blocks, blk = blockIdx.x - head * p.blocks;
    const int kvh = head / (m.n_head / m.n_kv_head);
    const int visible = pos + 1;
    const __half* K = a.kv.k + a.kv.offset(m, layer, 0, kvh, 0);
    const __half* V = a.kv.v + a.kv.offset(m, layer, 0, kvh, 0);
    const float scale = 1.0f / sqrtf((float)hd);
    const int sub = lane & 3, tl = lane >> 2;
    if (tid < hd) s.qs[tid] = __ldcg(a.q + (size_t)head * hd + tid);
    // residual value this thread will add in the projection (head 0 only), requested early
    const int tpr = hd / 16;
    float resid = 0.f;
    {
        const int orow = blk * p.rpb + tid / tpr;
        if (head == 0 && (tid % tpr) == 0 && tid / tpr < p.rpb && orow < m.d_model)
            resid = emb_row ? __half2float(__ushort_as_half(emb_row[orow])) : __ldcg(x_in + orow);
    }
    float m_w = -INFINITY, l_w = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int base = 0; base < visible; base += kMegaConsumers) {
        // requests: K row quarters of the 4 x 8 positions of this round, V rows of the same positions
        uint4 kreg[4][KV4];
#pragma unroll
        for (int st = 0; st < 4; st++) {
            const int t = base + warp + kMegaConsumerWarps * (st * 8 + tl);
            const uint4* kr = reinterpret_cast<const uint4*>(K + (size_t)min(t, visible - 1) * hd + sub * (hd / 4));
#pragma unroll
            for (int c = 0; c < KV4; c++) kreg[st][c] = __ldcg(kr + c);
        }
        uint2 vreg[32];
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const int t = base + warp + kMegaConsumerWarps * j;
            vreg[j] = make_uint2(0, 0);
            if (t < visible) {
                const __half* vr = V + (size_t)t * hd + lane * cpl;
                if (cpl == 4) vreg[j] = __ldcg(reinterpret_cast<const uint2*>(vr));
                else if (cpl == 2) vreg[j].x = __ldcg(reinterpret_cast<const unsigned int*>(vr));
                else vreg[j].x = (unsigned int)__ldcg(reinterpret_cast<const unsigned short*>(vr));
            }
        }
        if (base == 0) consumer_sync();  // q is staged
        float sc[4];
        float mx = -INFINITY;
#pragma unroll
        for (int st = 0; st < 4; st++) {
            const int t = base + warp + kMegaConsumerWarps * (st * 8 + tl);
            float dot = 0.f;
#pragma unroll
            for (int c = 0; c < KV4; c++) {
                const uint32_t ww[4] = {kreg[st][c].x, kreg[st][c].y, kreg[st][c].z, kreg[st][c].w};
                const float* qv = s.qs + sub * (hd / 4) + c * 8;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&ww[i]));
                    dot = fmaf(f.x, qv[2 * i], dot);
                    dot = fmaf(f.y, qv[2 * i + 1], dot);
                }
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            sc[st] = t < visible ? dot * scale : -INFINITY;
            mx = fmaxf(mx, sc[st]);
        }
        const float m_new = fmaxf(m_w, warp_max(mx));
        float pr[4], psum = 0.f;
#pragma unroll
        for (int st = 0; st < 4; st++) {
            pr[st] = sc[st] == -INFINITY ? 0.f : expf(sc[st] - m_new);
            psum += pr[st];
        }
        const float corr = m_w == -INFINITY ? 0.f : expf(m_w - m_new);
        l_w = l_w * corr + 0.25f * warp_sum(psum);  // every probability sits in four lanes
#pragma unroll
        for (int c = 0; c < 4; c++) acc[c] *= corr;
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const float pj = __shfl_sync(0xffffffffu, pr[j >> 3], (j & 7) * 4);
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&vreg[j].x));
            const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&vreg[j].y));
            acc[0] = fmaf(pj, f0.x, acc[0]);
            if (cpl >= 2) acc[1] = fmaf(pj, f0.y, acc[1]);
            if (cpl == 4) { acc[2] = fmaf(pj, f1.x, acc[2]); acc[3] = fmaf(pj, f1.y, acc[3]); }
        }
        m_w = m_new;
    }
    // merge the per-warp partial results (a warp that saw no position carries max = -inf, sum = 0)
#pragma unroll
    for (int c = 0; c < 4; c++)
        if (c < cpl) s.part[warp * hd + lane * cpl + c] = acc[c];
    if (lane == 0) { s.red[warp] = m_w; s.red[8 + warp] = l_w; }
    consumer_sync();
    if (tid < hd) {
        float gm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kMegaConsumerWarps; w++) gm = fmaxf(gm, s.red[w]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < kMegaConsumerWarps; w++) {
            const float f = s.red[w] == -INFINITY ? 0.f : expf(s.red[w] - gm);
            num = fmaf(s.part[w * hd + tid], f, num);
            den = fmaf(s.red[8 + w], f, den);
        }
        s.ctx[tid] = den > 0.f ? num / den : 0.f;
    }
    consumer_sync();
    // partial output projection: rows [blk*rpb, ...) of Wo restricted to this head's columns
    const int psub = tid % tpr;  // tpr threads per row, 16 inputs each
    const int rows_per_pass = kMegaConsumers / tpr;
    for (int r0 = 0; r0 < p.rpb; r0 += p.s2_rpc) {  // the block's rows arrive in chunks of s2_rpc
        const uint8_t* chunk = mega_acquire(a, s, c);
        const int nr = min(p.s2_rpc, p.rpb - r0);
        for (int rb = 0; rb < nr; rb += rows_per_pass) {  // uniform trip count: the shuffles below need every lane
            const int r = rb + tid / tpr;
            const int orow = blk * p.rpb + r0 + r;
            const bool valid = r < nr;
            float v = 0.f;
            if (valid) {
                const uint8_t* wrow = chunk + (size_t)r * hd * 2 + psub * 32;
                const uint4 w0 = lds128(wrow), w1 = lds128(wrow + 16);
                fma_vec16<WT_F16>(w0, nullptr, 0, s.ctx + psub * 16, 0.f, v);
                fma_vec16<WT_F16>(w1, nullptr, 0, s.ctx + psub * 16 + 8, 0.f, v);
            }
            for (int o = tpr / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (valid && psub == 0 && orow < m.d_model) {
                if (head == 0)  // residual, added once
                    v += (r0 == 0 && rb == 0) ? resid : (emb_row ? __half2float(__ushort_as_half(emb_row[orow])) : __ldcg(x_in + orow));
                atomicAdd(x_mid + orow, v);
            }
        }
        mega_release(a, s, c);
        c++;
    }
}

// S3: gate/up rows of this CTA's hidden units, SiLU*up, then the partial down projection (W2 transposed).
__device__ __forceinline__ void mega_s3_up(const MegaArgs& a, const MegaShared& s, const uint8_t* chunk, int j0, int n_items) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int j = warp; j < n_items; j += kMegaConsumerWarps) {
        float g, u;
        mega_dot2(chunk + (size_t)(2 * j) * a.plan.row_bytes, chunk + (size_t)(2 * j + 1) * a.plan.row_bytes, a.m.d_model, s.xs, lane, g, u);
        if (lane == 0) s.act[j0 + j] = silu_f(g) * u;
    }
}
// Partial down projection: a thread owns up to four groups of 4 output columns (d_model <= 4096) and accumulates
// over the CTA's hidden units, whose rows of W2-transposed arrive in chunks of s3b_rpc.
constexpr int kMegaDownGroups = 4;
__device__ __forceinline__ void mega_s3_down(const MegaArgs& a, const MegaShared& s, unsigned& c, const float* x_mid, float* x_out) {
    const int d = a.m.d_model;
    const MegaPlan& p = a.plan;
    float acc[kMegaDownGroups][4];
#pragma unroll
    for (int g = 0; g < kMegaDownGroups; g++) acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
    for (int j0 = 0; j0 < p.hpc; j0 += p.s3b_rpc) {
        const uint8_t* chunk = mega_acquire(a, s, c);
        const int nj = min(p.s3b_rpc, p.hpc - j0);
#pragma unroll
        for (int g = 0; g < kMegaDownGroups; g++) {
            const int col = threadIdx.x * 4 + g * kMegaConsumers * 4;
            if (col < d) {
#pragma unroll 4
                for (int j = 0; j < nj; j++) {
                    const uint2 w = lds64(chunk + (size_t)j * p.row_bytes + (size_t)col * 2);
                    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
                    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
                    const float av = s.act[j0 + j];
                    acc[g][0] = fmaf(av, f0.x, acc[g][0]); acc[g][1] = fmaf(av, f0.y, acc[g][1]);
                    acc[g][2] = fmaf(av, f1.x, acc[g][2]); acc[g][3] = fmaf(av, f1.y, acc[g][3]);
                }
            }
        }
        mega_release(a, s, c);
        c++;
    }
#pragma unroll
    for (int g = 0; g < kMegaDownGroups; g++) {
        const int col = threadIdx.x * 4 + g * kMegaConsumers * 4;
        if (col < d) {
            if (blockIdx.x == 0) {  // residual, added once
                const float4 r = __ldcg(reinterpret_cast<const float4*>(x_mid + col));
                acc[g][0] += r.x; acc[g][1] += r.y; acc[g][2] += r.z; acc[g][3] += r.w;
            }
            red_add_v4(x_out + col, acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
        }
    }
}

// ------------------------------------------------------------------------------------------------ the kernel

__global__ void __launch_bounds__(kMegaThreads, 1) k_decode_mega(const MegaArgs a) {
    extern __shared__ __align__(128) uint8_t mega_smem[];
    const MegaShared s = mega_carve(mega_smem, a);
    const MegaPlan& p = a.plan;
    const ModelDims& m = a.m;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int L = m.n_layer;
    if (tid == 0) {
        for (int i = 0; i < p.n_slots; i++) { mbar_init(s.full + i, 1); mbar_init(s.empty + i, kMegaConsumerWarps); }
        *s.abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const uint8_t* blob = a.pack + (size_t)blockIdx.x * p.cta_bytes;
    const long long head_off = (long long)L * p.layer_bytes;

    if (warp == kMegaConsumerWarps) {
        // ---------------- producer: one thread streams this CTA's chunks in consumption order ----------------
        if (lane == 0) {
            unsigned c = 0;
            const uint64_t policy = l2_evict_first_policy();
            auto issue = [&](long long off, int bytes) {
                const unsigned slot = c % (unsigned)p.n_slots;
                if (*reinterpret_cast<volatile int*>(s.abort)) return;  // once aborting, nothing more is copied
                if (c >= (unsigned)p.n_slots) mega_wait(a, s, s.empty + slot, ((c / (unsigned)p.n_slots) - 1u) & 1u, 4);
                if (*reinterpret_cast<volatile int*>(s.abort)) return;
                mbar_expect_tx(s.full + slot, (unsigned)bytes);
                bulk_copy_g2s(s.slots + (size_t)slot * p.slot_bytes, blob + off, (unsigned)bytes, s.full + slot, policy);
                c++;
            };
            // a stage's slice: whole items, `per_chunk` at a time (the pack pads a CTA's last items with zero rows)
            auto issue_stage = [&](long long off, int items, int per_chunk, int item_bytes) {
                for (int i0 = 0; i0 < items; i0 += per_chunk) issue(off + (long long)i0 * item_bytes, min(per_chunk, items - i0) * item_bytes);
            };
            for (int step = 0; step < a.n_steps; step++) {
                if (step > 0) {
                    for (int l = 0; l < L; l++) {
                        long long off = (long long)l * p.layer_bytes;
                        issue_stage(off, p.ppc, p.s1_ipc, 2 * p.row_bytes); off += p.s1_bytes;
                        if ((int)blockIdx.x < m.n_head * p.blocks) issue_stage(off, p.rpb, p.s2_rpc, m.head_dim * 2);  // S2 runs on n_head * blocks CTAs
                        off += p.s2_bytes;
                        issue_stage(off, p.hpc, p.s3a_ipc, 2 * p.row_bytes); off += p.s3a_bytes;
                        issue_stage(off, p.hpc, p.s3b_rpc, p.row_bytes);
                    }
                }
                for (int hc = 0; hc < p.head_chunks; hc++) issue(head_off + (long long)hc * p.head_chunk_bytes, p.head_chunk_bytes);
            }
            // every copy that was issued must have landed before the CTA may exit
            const unsigned first = c > (unsigned)p.n_slots ? c - (unsigned)p.n_slots : 0u;
            for (unsigned k = first; k < c; k++) {
                unsigned spins = 0;
                while (!mbar_try_wait(s.full + (k % (unsigned)p.n_slots), (k / (unsigned)p.n_slots) & 1u) && ++spins < kMegaSpinLimit) {}
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    if (blockIdx.x == 0 && tid == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        a.stamps[0] = t;
    }
    int n_stamp = 0;
    auto stamp = [&](int step) {
        if (a.trace && (int)blockIdx.x == a.trace_cta && tid == 0 && step == a.n_steps - 1) a.trace[n_stamp++] = clock64();
    };
    unsigned c = 0;      // chunk counter, advances in lock step with the producer's
    unsigned epoch = 0;  // grid barrier epoch
    int pos = a.pos0;    // visible tokens
    uint32_t tok = 0;
    const float* fin_gain = a.norms + (size_t)(2 * L) * m.d_model;
    for (int step = 0; step < a.n_steps; step++) {
        const float* x_final = a.hidden_io;
        if (step > 0) {
            const uint16_t* emb_row = a.tok_emb + (size_t)tok * m.d_model;
            for (int l = 0; l < L; l++) {
                float* x_in = a.xbuf + (size_t)((2 * l) % 3) * m.d_model;
                float* x_mid = a.xbuf + (size_t)((2 * l + 1) % 3) * m.d_model;
                float* x_out = a.xbuf + (size_t)((2 * l + 2) % 3) * m.d_model;
                const uint16_t* er = l == 0 ? emb_row : nullptr;
                // S1
                stamp(step);
                mega_stage_norm(a, s, x_in, er, a.norms + (size_t)(2 * l) * m.d_model);
                stamp(step);
                if ((int)blockIdx.x == p.n_cta - 1)  // both accumulation targets of this layer start from zero
                    for (int k = tid; k < m.d_model; k += kMegaConsumers) { x_mid[k] = 0.f; x_out[k] = 0.f; }
                for (int i0 = 0; i0 < p.ppc; i0 += p.s1_ipc) {
                    const uint8_t* ch = mega_acquire(a, s, c);
                    if (i0 == 0) stamp(step);
                    mega_s1(a, s, l, pos, ch, i0, min(p.s1_ipc, p.ppc - i0));
                    mega_release(a, s, c); c++;
                }
                stamp(step);
                mega_grid_sync(a, s, epoch);
                stamp(step);
                // S2 (acquires its projection chunks itself, after the attention)
                stamp(step);
                if (m.head_dim == 64) mega_s2_t<64>(a, s, l, pos, c, x_in, er, x_mid);
                else if (m.head_dim == 128) mega_s2_t<128>(a, s, l, pos, c, x_in, er, x_mid);
                else mega_s2_t<32>(a, s, l, pos, c, x_in, er, x_mid);
                stamp(step);
                mega_grid_sync(a, s, epoch);
                stamp(step);
                // S3
                mega_stage_norm(a, s, x_mid, nullptr, a.norms + (size_t)(2 * l + 1) * m.d_model);
                stamp(step);
                for (int j0 = 0; j0 < p.hpc; j0 += p.s3a_ipc) {
                    const uint8_t* ch = mega_acquire(a, s, c);
                    if (j0 == 0) stamp(step);
                    mega_s3_up(a, s, ch, j0, min(p.s3a_ipc, p.hpc - j0));
                    mega_release(a, s, c); c++;
                }
                consumer_sync();
                stamp(step);
                stamp(step);
                mega_s3_down(a, s, c, x_mid, x_out);
                stamp(step);
                mega_grid_sync(a, s, epoch);
                stamp(step);
                x_final = x_out;
            }
            pos++;  // the token that was just processed is now visible
        }
        // LM head over this CTA's vocab rows, first-max argmax
        stamp(step);
        mega_stage_norm(a, s, x_final, nullptr, fin_gain);
        stamp(step);
        float best_v = -INFINITY;
        int best_i = 0x7fffffff;
        for (int hc = 0; hc < p.head_chunks; hc++) {
            const uint8_t* ch = mega_acquire(a, s, c);
            const int row_base = hc * p.head_rows_per_chunk;
            const int nrows = min(p.head_rows_per_chunk, p.vpc - row_base);
            // four rows per warp per pass; rows past the chunk's end are zero-filled in the pack and masked by `g < vocab`
            for (int r0 = 4 * warp; r0 < nrows; r0 += 4 * kMegaConsumerWarps) {
                float v[4];
                mega_dot4(ch + (size_t)r0 * p.row_bytes, p.row_bytes, m.d_model, s.xs, lane, v);
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    const int g = blockIdx.x * p.vpc + row_base + r0 + r;
                    if (r0 + r < nrows && g < m.vocab && v[r] > best_v) { best_v = v[r]; best_i = g; }
                }
            }
            mega_release(a, s, c); c++;
        }
        if (lane == 0 && best_i != 0x7fffffff) atomicMax(a.best + (step & 1), pack_best(best_v, best_i));
        stamp(step);
        mega_grid_sync(a, s, epoch);
        stamp(step);
        const unsigned long long key = __ldcg(a.best + (step & 1));
        tok = min(0xffffffffu - (uint32_t)(key & 0xffffffffull), (uint32_t)(m.vocab - 1));  // in range even if every logit was NaN
        if (blockIdx.x == 0 && tid == 0) {
            if (step == 0) {
                unsigned long long t;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                a.stamps[1] = t;
            }
            a.rs.out[step] = tok;
            if (a.token_times) {
                unsigned long long t;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                a.token_times[step] = t;
            }
            a.best[(step + 1) & 1] = 0ull;  // nobody reads that slot before the next head's barrier
        }
        if (step > 0 && step == a.n_steps - 1 && blockIdx.x == 0)  // keep the sequence's last hidden state
            for (int k = tid; k < m.d_model; k += kMegaConsumers) a.hidden_io[k] = __ldcg(x_final + k);
    }
    if (blockIdx.x == 0 && tid == 0) {
        a.rs.pos[0] = pos;
        a.rs.tok[0] = tok;
        a.rs.next[0] = tok;
        a.rs.n_out[0] = a.n_steps;
    }
}

// ------------------------------------------------------------------------------------------------ pack builder

struct PackSources {
    const __half* const* wq;  // per-layer device pointers (row-major [out, in] fp16)
    const __half* const* wk;
    const __half* const* wv;
    const __half* const* wo;
    const __half* const* w1;
    const __half* const* w2;
    const __half* const* w3;
    const __half* lm_head;
};

__device__ __forceinline__ void pack_copy(uint8_t* dst, const void* src, int bytes) {
    // bytes is a multiple of 16; src == nullptr writes zeros
    for (int o = threadIdx.x * 16; o < bytes; o += blockDim.x * 16) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (src) v = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(src) + o);
        *reinterpret_cast<uint4*>(dst + o) = v;
    }
}

// One CTA builds the blob of one megakernel CTA.
__global__ void k_build_pack(PackSources src, MegaPlan p, ModelDims m, uint8_t* pack) {
    const int cta = blockIdx.x;
    uint8_t* blob = pack + (size_t)cta * p.cta_bytes;
    const int d = m.d_model, hd = m.head_dim, half = hd / 2;
    const int q_items = m.q_dim / 2, k_items = m.kv_dim / 2, total = q_items + 2 * k_items;
    for (int l = 0; l < m.n_layer; l++) {
        uint8_t* base = blob + (size_t)l * p.layer_bytes;
        // S1: pairs of rows in RoPE order
        for (int i = 0; i < p.ppc; i++) {
            const int item = cta * p.ppc + i;
            const __half *r0 = nullptr, *r1 = nullptr;
            if (item < total) {
                const __half* W;
                int local, row0, row1;
                if (item < q_items) { W = src.wq[l]; local = item; }
                else if (item < q_items + k_items) { W = src.wk[l]; local = item - q_items; }
                else { W = src.wv[l]; local = item - q_items - k_items; }
                if (item < q_items + k_items) { int h = local / half; row0 = h * hd + (local - h * half); row1 = row0 + half; }
                else { row0 = 2 * local; row1 = row0 + 1; }
                r0 = W + (size_t)row0 * d; r1 = W + (size_t)row1 * d;
            }
            pack_copy(base + (size_t)(2 * i) * p.row_bytes, r0, p.row_bytes);
            pack_copy(base + (size_t)(2 * i + 1) * p.row_bytes, r1, p.row_bytes);
        }
        base += p.s1_bytes;
        // S2: rows [blk*rpb, +rpb) of Wo, columns of one head
        {
            const int units = m.n_head * p.blocks;
            const int head = cta / p.blocks, blk = cta - head * p.blocks;
            for (int r = 0; r < p.rpb; r++) {
                const int orow = blk * p.rpb + r;
                const __half* sp = (cta < units && orow < d) ? src.wo[l] + (size_t)orow * m.q_dim + (size_t)head * hd : nullptr;
                pack_copy(base + (size_t)r * hd * 2, sp, hd * 2);
            }
        }
        base += p.s2_bytes;
        // S3a: (gate_j, up_j) row pairs
        for (int j = 0; j < p.hpc; j++) {
            const int hrow = cta * p.hpc + j;
            pack_copy(base + (size_t)(2 * j) * p.row_bytes, hrow < m.hidden ? src.w1[l] + (size_t)hrow * d : nullptr, p.row_bytes);
            pack_copy(base + (size_t)(2 * j + 1) * p.row_bytes, hrow < m.hidden ? src.w3[l] + (size_t)hrow * d : nullptr, p.row_bytes);
        }
        base += p.s3a_bytes;
        // S3b: rows of W2 transposed: out[j][c] = W2[c][hrow]
        for (int j = 0; j < p.hpc; j++) {
            const int hrow = cta * p.hpc + j;
            __half* dst = reinterpret_cast<__half*>(base + (size_t)j * p.row_bytes);
            for (int c = threadIdx.x; c < d; c += blockDim.x)
                dst[c] = hrow < m.hidden ? src.w2[l][(size_t)c * m.hidden + hrow] : __float2half(0.f);
        }
    }
    uint8_t* hb = blob + (size_t)m.n_layer * p.layer_bytes;
    for (int i = 0; i < p.head_chunks * p.head_rows_per_chunk; i++) {
        const int v = cta * p.vpc + i;
        const int hc = i / p.head_rows_per_chunk, r = i - hc * p.head_rows_per_chunk;
        pack_copy(hb + (size_t)hc * p.head_chunk_bytes + (size_t)r * p.row_bytes, (i < p.vpc && v < m.vocab) ? src.lm_head + (size_t)v * d : nullptr,
                  p.row_bytes);
    }
}

}  // namespace esp
