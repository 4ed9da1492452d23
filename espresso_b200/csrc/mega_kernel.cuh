// Persistent whole-loop decode kernel for one sequence of a Llama-style fp16 model.
//
// One cooperative launch runs an entire greedy decode loop: `n_steps` heads and up to `n_steps - 1` forward
// passes.  The grid has one CTA per SM.  Inside a CTA one producer warp streams that CTA's weights from HBM into a
// shared-memory ring with bulk async copies (cp.async.bulk + mbarrier), always running ahead of the sixteen
// consumer warps, so HBM keeps streaming while the consumers wait on the activation dependencies of the step.
// Weights are re-laid out once ("pack") so that everything a CTA needs for one layer is contiguous.
//
// Batch-1 decode is bound by the chain of dependent vector exchanges between CTAs, not by bytes, so the kernel has
// no grid barrier at all.  Every vector that crosses CTAs is self-validating:
//   * "tagged words": an 8-byte word {fp32 value, 32-bit sequence tag} with a single writer.  A reader polls the
//     word itself until the tag is the one it expects: flag and data travel in one 8-byte access, so neither a
//     fence nor a separate arrival counter nor a second round trip for the data is needed.
//   * "counted sums": an 8-byte accumulator that several CTAs add into with one `red.add.u64` each; the addend is
//     (fixed-point value << 8) + 1, so the low byte counts contributions and the upper 56 bits carry their sum.
//     The accumulators are never cleared: a reader remembers the total it saw the last time and subtracts it
//     (all arithmetic is modulo 2^64, so neither field can overflow into a wrong result as long as one exchange's
//     sum fits 55 bits).  Integer addition is associative: the sums are bit-identical from run to run.
// Per layer the consumers run
//   S1  x (tagged words from the previous layer, or the embedding row) -> RMSNorm folded into the products ->
//       this CTA's rows of Wq/Wk/Wv -> RoPE -> tagged words for the CTAs that share the KV head, KV-cache append
//   S2  attention of one query head (recomputed by the CTAs that share the head) -> this CTA's block of rows of Wo
//       restricted to the head's columns -> counted sums (one contribution per head and row)
//   S3  x_mid -> norm -> this CTA's (gate, up) row pairs -> SiLU*up -> tagged words; then the whole activation
//       vector -> this CTA's rows of W2 (+ residual) -> tagged words = the next layer's x
// and the LM head streams the CTA's vocabulary rows through the same ring; every CTA publishes its best
// (logit, index) as tagged words and every CTA reduces all of them, so the token is known everywhere at once.
// Why single buffers suffice: each exchange is re-written only after an exchange of another kind that every
// reader of the old contents must have passed (see the notes at each stage).
// Every wait (mbarrier, tagged word, counted sum) is bounded: when a limit is hit the kernel records an error code,
// stops waiting everywhere and runs to completion; the host reports a timeout.
#pragma once
#include <type_traits>

#include "decode_kernels.cuh"

namespace esp {

constexpr int kMegaConsumerWarps = 16;
constexpr int kMegaConsumers = kMegaConsumerWarps * 32;
constexpr int kMegaThreads = kMegaConsumers + 32;  // + one producer warp
constexpr unsigned kMegaSpinLimit = 1u << 21;      // default attempts per wait before the kernel gives up (a few seconds)
constexpr int kMegaTraceLayer = 10;                // stamps per layer
constexpr int kMegaTraceHead = 4;                  // stamps of the head
constexpr float kMegaFix = 4294967296.0f;          // counted sums: fixed point with 32 fractional bits
constexpr float kMegaUnfix = 2.3283064365386963e-10f;

struct MegaPlan {
    int n_cta;
    int cph;          // CTAs per query head (S2 row blocks of Wo)
    int qpk;          // query heads per KV head
    int gsize;        // CTAs per KV-head group = cph * qpk
    int n_group_cta;  // CTAs that take part in S1/S2 = n_head * cph
    int group_items;  // S1 row pairs per KV-head group = (qpk + 2) * head_dim / 2
    int s1_max;       // largest number of S1 row pairs of a CTA
    int rpb;          // S2: output rows per block
    int hpc_max, dpc_max, vpc_max;  // largest number of FFN units / W2 rows / vocabulary rows of a CTA
    int row_bytes;    // d_model * 2
    int down_row_bytes;  // hidden * 2
    int s1_bytes, s2_bytes, s3a_bytes, s3b_bytes;  // packed bytes of a stage per layer (multiples of 128, sized for the largest CTA share)
    // A stage whose slice is larger than a ring slot arrives in several chunks of whole items:
    int s1_ipc;       // S1 row pairs per chunk
    int s2_rpc;       // S2 projection rows per chunk (a multiple of the rows one pass of the CTA covers)
    int s3a_ipc;      // S3 (gate, up) pairs per chunk
    int s3b_rpc;      // S3 down-projection rows per chunk
    int head_rpc;     // LM-head rows per chunk
    int slot_bytes, n_slots;
    long long layer_bytes, head_bytes, cta_bytes;  // packed bytes per CTA: one layer, the head, everything
    int smem_bytes;
    // byte offsets of the shared-memory areas behind the ring (see MegaShared)
    int off_bar, off_prev, off_key, off_xs, off_xraw, off_xmid, off_rope, off_qs, off_ctx, off_kn, off_vn, off_part, off_red, off_outv, off_flags, off_share;
};

// Contiguous share [begin, end) of `n` items owned by part `i` of `parts` (every part gets floor or ceil of n/parts).
// (n * parts stays far below 2^32 for every model size the plan accepts)
__host__ __device__ inline int mega_share_begin(int n, int parts, int i) { return (int)((unsigned)n * (unsigned)i / (unsigned)parts); }

struct MegaArgs {
    ModelDims m;
    MegaPlan plan;
    const uint8_t* pack;      // [n_cta][cta_bytes]
    const float* norms;       // [2*L + 1][d_model]: norm1(l), norm2(l), ..., final
    const uint16_t* tok_emb;  // fp16 [vocab][d_model]
    const float2* rope;       // [max_seq][head_dim/2]
    KvLayout kv;
    // exchange arena (zero at launch)
    unsigned long long* x_words;    // [d_model] tagged: output of a layer
    unsigned long long* act_words;  // [hidden] tagged: FFN activation
    unsigned long long* qkv_words;  // [n_kv_head][2 * group_items] tagged: post-RoPE q / k / v of one token
    unsigned long long* mid_sums;   // [d_model] counted: residual + attention projection
    unsigned long long* cand_words; // [n_cta][4] tagged: {logit bits, index} of each CTA's best row
    float* hidden_io;         // [d_model] last hidden state of the sequence (in and out)
    int* error;               // [1] 0 = ok
    unsigned long long* stamps; // [3] globaltimer at kernel start and when the first token is known; number of tokens emitted
    unsigned long long* token_times; // optional [n_steps] globaltimer (ns) at which each token became known, or null
    long long* trace;         // optional [kMegaTraceLayer*L + kMegaTraceHead] SM clock stamps of the last step taken by CTA `trace_cta`, or null
    int trace_cta;
    RowState rs;              // row 0 carries pos / tok / n_out / out
    int n_steps;              // tokens to emit at most (>= 1)
    int pos0;                 // visible tokens at launch
    unsigned spin_limit;      // attempts per wait
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
// Non-blocking test of a phase: the potentially blocking try_wait form costs about 0.25 us per call on this part even
// when the phase has already completed, which a chunk-by-chunk consumer cannot afford.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Weight chunks carry an evict-first L2 policy: they are used once per token, and keeping them out of the way
// leaves the KV cache and the exchange words resident in L2.
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ uint4 lds128(const uint8_t* p) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(smem_u32(p)));
    return r;
}
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kMegaConsumers) : "memory"); }

// 16 bytes = two exchange words; each word is validated on its own, so the pair needs no 16-byte atomicity.
__device__ __forceinline__ ulonglong2 ld_words2(const unsigned long long* p) {
    ulonglong2 v;
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_word(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_add_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long tagged(float v, unsigned tag) { return ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v); }
__device__ __forceinline__ unsigned long long counted(float v) { return ((unsigned long long)__float2ll_rn(v * kMegaFix) << 8) + 1ull; }

// ------------------------------------------------------------------------------------------------ work shares

struct MegaShare {
    bool in_group;       // takes part in S1 / S2
    int head, blk, kvh, hq, member;  // query head, Wo row block, KV head, head inside the KV group, CTA inside the KV group
    int s1_begin, s1_n;  // S1 row pairs inside the KV group
    int h_begin, h_n;    // FFN hidden units
    int d_begin, d_n;    // W2 rows
    int v_begin, v_n;    // vocabulary rows
};

__host__ __device__ inline MegaShare mega_share(const ModelDims& m, const MegaPlan& p, int cta) {
    MegaShare w{};
    w.in_group = cta < p.n_group_cta;
    if (w.in_group) {
        w.head = cta / p.cph;
        w.blk = cta - w.head * p.cph;
        w.kvh = w.head / p.qpk;
        w.hq = w.head - w.kvh * p.qpk;
        w.member = cta - w.kvh * p.gsize;
        w.s1_begin = mega_share_begin(p.group_items, p.gsize, w.member);
        w.s1_n = mega_share_begin(p.group_items, p.gsize, w.member + 1) - w.s1_begin;
    }
    w.h_begin = mega_share_begin(m.hidden, p.n_cta, cta);
    w.h_n = mega_share_begin(m.hidden, p.n_cta, cta + 1) - w.h_begin;
    w.d_begin = mega_share_begin(m.d_model, p.n_cta, cta);
    w.d_n = mega_share_begin(m.d_model, p.n_cta, cta + 1) - w.d_begin;
    w.v_begin = mega_share_begin(m.vocab, p.n_cta, cta);
    w.v_n = mega_share_begin(m.vocab, p.n_cta, cta + 1) - w.v_begin;
    return w;
}

// S1 row pair `item` of KV group `kvh`: which matrix (0 q, 1 k, 2 v) and which two rows.
__host__ __device__ inline void mega_s1_rows(const ModelDims& m, const MegaPlan& p, int kvh, int item, int& kind, int& row0, int& row1, int& idx) {
    const int half = m.head_dim / 2;
    if (item < p.qpk * half) {
        const int hq = item / half;
        idx = item - hq * half;
        kind = 0; row0 = (kvh * p.qpk + hq) * m.head_dim + idx; row1 = row0 + half;
    } else if (item < (p.qpk + 1) * half) {
        idx = item - p.qpk * half;
        kind = 1; row0 = kvh * m.head_dim + idx; row1 = row0 + half;
    } else {
        idx = item - (p.qpk + 1) * half;
        kind = 2; row0 = kvh * m.head_dim + 2 * idx; row1 = row0 + 1;
    }
}

// ------------------------------------------------------------------------------------------------ shared state

struct MegaShared {
    uint8_t* slots;
    uint64_t* full;
    uint64_t* empty;
    float* xs;     // staged activation vector (x * gain, or the FFN activation), lane-major order (see xs_index)
    float* xraw;   // [d_model] the residual stream entering the layer (also what the head reads)
    float* xmid;   // [d_model] the residual stream after the attention block
    float2* rope;  // [head_dim/2] (cos, sin) of the position being processed
    unsigned long long* prev;  // [d_model] totals of the counted sums seen at the previous exchange
    float* qs;     // [head_dim] query of this CTA's head
    float* ctx;    // [head_dim]
    __half* kn;    // [head_dim] the new token's key, rounded as the cache stores it
    __half* vn;    // [head_dim]
    float* part;   // [warps][head_dim]
    float* red;    // [64]
    float* outv;   // results of a stage before they are published: max(2*s1_max, hpc_max, dpc_max * kparts) floats
    unsigned long long* key;   // [32] arg-max keys
    struct MegaShare* share;  // this CTA's work shares, computed once
    int* abort;    // [1] a wait gave up: no more waiting in this CTA
    int* stop;     // [1] the loop ended early (EOS): the producer stops issuing
};

__host__ __device__ inline int mega_outv_floats(const MegaPlan& p) {
    int n = 2 * p.s1_max;
    if (p.hpc_max > n) n = p.hpc_max;
    if (p.dpc_max * kMegaConsumerWarps > n) n = p.dpc_max * kMegaConsumerWarps;
    return (n + 3) & ~3;
}
__host__ __device__ inline int mega_xs_floats(const ModelDims& m) { return xs_floats<8>(m.d_model > m.hidden ? m.d_model : m.hidden); }

// The areas sit at offsets the host computed once (mega_layout): an address is the base plus a kernel-argument
// constant, which costs no register to keep.
__device__ __forceinline__ MegaShared mega_carve(uint8_t* base, const MegaArgs& a) {
    MegaShared s;
    const MegaPlan& p = a.plan;
    s.slots = base;
    s.full = reinterpret_cast<uint64_t*>(base + p.off_bar);
    s.empty = s.full + p.n_slots;
    s.prev = reinterpret_cast<unsigned long long*>(base + p.off_prev);
    s.key = reinterpret_cast<unsigned long long*>(base + p.off_key);
    s.xs = reinterpret_cast<float*>(base + p.off_xs);
    s.xraw = reinterpret_cast<float*>(base + p.off_xraw);
    s.xmid = reinterpret_cast<float*>(base + p.off_xmid);
    s.rope = reinterpret_cast<float2*>(base + p.off_rope);
    s.qs = reinterpret_cast<float*>(base + p.off_qs);
    s.ctx = reinterpret_cast<float*>(base + p.off_ctx);
    s.kn = reinterpret_cast<__half*>(base + p.off_kn);
    s.vn = reinterpret_cast<__half*>(base + p.off_vn);
    s.part = reinterpret_cast<float*>(base + p.off_part);
    s.red = reinterpret_cast<float*>(base + p.off_red);
    s.outv = reinterpret_cast<float*>(base + p.off_outv);
    s.abort = reinterpret_cast<int*>(base + p.off_flags);
    s.stop = s.abort + 1;
    s.share = reinterpret_cast<MegaShare*>(base + p.off_share);
    return s;
}

// Fills the offsets and the total size (host side; p.n_slots and p.slot_bytes must be set).
inline void mega_layout(const ModelDims& m, MegaPlan& p) {
    size_t o = (size_t)p.n_slots * p.slot_bytes;
    auto take = [&](size_t bytes) { size_t at = (o + 15) & ~(size_t)15; o = at + bytes; return (int)at; };
    p.off_bar = take(16 * (size_t)p.n_slots);
    p.off_prev = take(8 * (size_t)m.d_model);
    p.off_key = take(8 * 32);
    p.off_xs = take(sizeof(float) * (size_t)mega_xs_floats(m));
    p.off_xraw = take(sizeof(float) * (size_t)m.d_model);
    p.off_xmid = take(sizeof(float) * (size_t)m.d_model);
    p.off_rope = take(sizeof(float2) * (size_t)(m.head_dim / 2));
    p.off_qs = take(sizeof(float) * (size_t)m.head_dim);
    p.off_ctx = take(sizeof(float) * (size_t)m.head_dim);
    p.off_kn = take(sizeof(__half) * (size_t)m.head_dim);
    p.off_vn = take(sizeof(__half) * (size_t)m.head_dim);
    p.off_part = take(sizeof(float) * (size_t)kMegaConsumerWarps * m.head_dim);
    p.off_red = take(sizeof(float) * 64);
    p.off_outv = take(sizeof(float) * (size_t)mega_outv_floats(p));
    p.off_flags = take(16);
    p.off_share = take(sizeof(MegaShare));
    p.smem_bytes = (int)((o + 127) & ~(size_t)127);
}

__device__ __forceinline__ void mega_fail(const MegaArgs& a, const MegaShared& s, int code) {
    *reinterpret_cast<volatile int*>(s.abort) = 1;
    atomicCAS(a.error, 0, code);
}
__device__ __forceinline__ bool mega_aborting(const MegaShared& s) { return *reinterpret_cast<volatile int*>(s.abort) != 0; }

// One failed attempt of a polling loop: true when the loop must give up (limit reached, or the kernel is aborting).
__device__ __forceinline__ bool mega_spin_out(const MegaArgs& a, const MegaShared& s, unsigned& spins, int code) {
    ++spins;
    if (spins > a.spin_limit) { mega_fail(a, s, code); return true; }
    if ((spins & 0x3ffu) == 0 && (__ldcg(a.error) != 0 || mega_aborting(s))) { *reinterpret_cast<volatile int*>(s.abort) = 1; return true; }
    return false;
}

// Bounded wait on an mbarrier phase.  Returns immediately once the kernel is aborting.
__device__ __forceinline__ void mega_wait(const MegaArgs& a, const MegaShared& s, uint64_t* bar, unsigned parity, int code) {
    if (mega_aborting(s)) return;
    unsigned spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (*reinterpret_cast<volatile int*>(s.stop)) return;
        if (mega_spin_out(a, s, spins, code)) return;
    }
}

// Ring bookkeeping shared by the producer and the consumers: chunk c lives in slot c % n_slots.
__device__ __forceinline__ const uint8_t* mega_acquire(const MegaArgs& a, const MegaShared& s, unsigned c) {
    const unsigned slot = c % (unsigned)a.plan.n_slots;
    // one lane per warp polls the barrier (many threads polling one shared-memory word serialise); the warp barrier
    // that follows orders the other lanes' reads of the chunk after the observed completion
    if ((threadIdx.x & 31) == 0) mega_wait(a, s, s.full + slot, (c / (unsigned)a.plan.n_slots) & 1u, 3);
    __syncwarp();
    return s.slots + (size_t)slot * a.plan.slot_bytes;
}
__device__ __forceinline__ void mega_release(const MegaArgs& a, const MegaShared& s, unsigned c) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(s.empty + (c % (unsigned)a.plan.n_slots));
}

// ------------------------------------------------------------------------------------------------ exchanges

// Reads `n` tagged words (n even, 16-byte aligned base) and hands (index, value, gain) to `sink`.  A thread keeps up to
// four 16-byte loads in flight; words that validated are not read again.  The gains (or 1 when `gain` is null) are
// requested before the polling starts, so they cost nothing once the words arrive.
template <class Sink>
__device__ __forceinline__ void mega_read_words(const MegaArgs& a, const MegaShared& s, const unsigned long long* base, int n, unsigned tag, int code,
                                                const float* gain, Sink sink) {
    const int n_pairs = n >> 1;
    for (int p0 = 0; p0 < n_pairs; p0 += 4 * kMegaConsumers) {
        ulonglong2 w[4];
        float2 g[4];
        bool ok[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int p = p0 + j * kMegaConsumers + (int)threadIdx.x;
            ok[j] = p >= n_pairs;
            w[j] = make_ulonglong2(0, 0);
            g[j] = (gain && !ok[j]) ? __ldg(reinterpret_cast<const float2*>(gain) + p) : make_float2(1.f, 1.f);
        }
        unsigned spins = 0;
        if (!mega_aborting(s)) {
            while (true) {
                bool all = true;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (!ok[j]) {
                        w[j] = ld_words2(base + 2 * (size_t)(p0 + j * kMegaConsumers + (int)threadIdx.x));
                        ok[j] = (unsigned)(w[j].x >> 32) == tag && (unsigned)(w[j].y >> 32) == tag;
                        all = all && ok[j];
                    }
                }
                if (all) break;
                if (mega_spin_out(a, s, spins, code)) break;
            }
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int p = p0 + j * kMegaConsumers + (int)threadIdx.x;
            if (p < n_pairs) {
                sink(2 * p, __uint_as_float((unsigned)w[j].x), g[j].x);
                sink(2 * p + 1, __uint_as_float((unsigned)w[j].y), g[j].y);
            }
        }
    }
}

// Reads the counted sums once each has received `n_contrib` contributions since the previous exchange.
template <class Sink>
__device__ __forceinline__ void mega_read_sums(const MegaArgs& a, const MegaShared& s, const unsigned long long* base, int n, int n_contrib, int code,
                                               const float* gain, Sink sink) {
    const int n_pairs = n >> 1;
    for (int p0 = 0; p0 < n_pairs; p0 += 2 * kMegaConsumers) {
        ulonglong2 w[2], pv[2];
        float2 g[2];
        bool ok[2];
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int p = p0 + j * kMegaConsumers + (int)threadIdx.x;
            ok[j] = p >= n_pairs;
            w[j] = make_ulonglong2(0, 0);
            pv[j] = ok[j] ? make_ulonglong2(0, 0) : *reinterpret_cast<const ulonglong2*>(s.prev + 2 * p);
            g[j] = (gain && !ok[j]) ? __ldg(reinterpret_cast<const float2*>(gain) + p) : make_float2(1.f, 1.f);
        }
        unsigned spins = 0;
        if (!mega_aborting(s)) {
            while (true) {
                bool all = true;
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    if (!ok[j]) {
                        w[j] = ld_words2(base + 2 * (size_t)(p0 + j * kMegaConsumers + (int)threadIdx.x));
                        ok[j] = ((w[j].x - pv[j].x) & 0xffull) == (unsigned long long)n_contrib && ((w[j].y - pv[j].y) & 0xffull) == (unsigned long long)n_contrib;
                        all = all && ok[j];
                    }
                }
                if (all) break;
                if (mega_spin_out(a, s, spins, code)) break;
            }
        }
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int p = p0 + j * kMegaConsumers + (int)threadIdx.x;
            if (p < n_pairs) {
                *reinterpret_cast<ulonglong2*>(s.prev + 2 * p) = w[j];
                const long long v0 = (long long)(w[j].x - pv[j].x - (unsigned long long)n_contrib) >> 8;
                const long long v1 = (long long)(w[j].y - pv[j].y - (unsigned long long)n_contrib) >> 8;
                sink(2 * p, (float)v0 * kMegaUnfix, g[j].x);
                sink(2 * p + 1, (float)v1 * kMegaUnfix, g[j].y);
            }
        }
    }
}

// Sum over the consumer threads of one float each; every thread receives the result.  One CTA barrier.
__device__ __forceinline__ float mega_block_sum(float v, float* red) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    consumer_sync();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kMegaConsumerWarps; i++) t += red[i];
    return t;
}

// ------------------------------------------------------------------------------------------------ dot products

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

// Dot products of NR fp16 rows held in shared memory (row r at base + r * row_bytes) with the staged vector over the
// 256-element slices [it_begin, it_end); the results are in every lane.  Two slices are in flight per pass: all of
// their shared-memory loads are issued before the first multiply, and every row has four independent accumulators.
template <int NR>
__device__ __forceinline__ void mega_dot_rows(const uint8_t* base, int row_bytes, int K, int it_begin, int it_end, const float* xs, int lane,
                                              float (&o)[NR]) {
    const float4* xs4 = reinterpret_cast<const float4*>(xs);
    float acc[NR][4];
#pragma unroll
    for (int r = 0; r < NR; r++) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
    for (int it = it_begin; it < it_end; it += 2) {
        const int k0 = it * 256 + lane * 8, k1 = k0 + 256;
        const bool in0 = k0 < K, in1 = it + 1 < it_end && k1 < K;
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

// ------------------------------------------------------------------------------------------------ consumer stages

// S1: q/k/v rows of this CTA (pairs that RoPE rotates together) from one ring chunk; results go to s.outv, k and v
// also to the KV cache.  `inv` is the RMSNorm scale of the staged vector (the gain is already in s.xs).
__device__ __forceinline__ void mega_s1(const MegaArgs& a, const MegaShared& s, const MegaShare& w, int layer, int pos, float inv,
                                        const uint8_t* chunk, int i0, int n_items) {
    const ModelDims& m = a.m;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int iters = (m.d_model + 255) / 256;
    for (int i = warp; i < n_items; i += kMegaConsumerWarps) {  // i: pair inside the chunk, i0 + i: pair of this CTA
        float v[2];
        mega_dot_rows<2>(chunk + (size_t)(2 * i) * a.plan.row_bytes, a.plan.row_bytes, m.d_model, 0, iters, s.xs, lane, v);
        if (lane == 0) {
            int kind, row0, row1, idx;
            mega_s1_rows(m, a.plan, w.kvh, w.s1_begin + i0 + i, kind, row0, row1, idx);
            float v0 = v[0] * inv, v1 = v[1] * inv;
            if (kind < 2) {
                const float2 cs = s.rope[idx];
                const float r0 = v0 * cs.x - v1 * cs.y, r1 = v0 * cs.y + v1 * cs.x;
                v0 = r0; v1 = r1;
            }
            s.outv[2 * (i0 + i)] = v0;
            s.outv[2 * (i0 + i) + 1] = v1;
            if (kind > 0) {
                __half* base = kind == 1 ? a.kv.k : a.kv.v;
                const size_t off = a.kv.offset(m, layer, 0, w.kvh, pos);
                base[off + (row0 - w.kvh * m.head_dim)] = __float2half_rn(v0);
                base[off + (row1 - w.kvh * m.head_dim)] = __float2half_rn(v1);
            }
        }
    }
}

// S2: attention of one head over the cached positions [0, pos) plus the new token (whose key and value are in
// shared memory), then this CTA's block of the output projection.
// Each warp owns the positions t = warp + 16*i (16 per round).  Four neighbouring lanes share one position: each loads
// a quarter of its K row with 16-byte vectors and the score is completed with two shuffles.  The probabilities are
// then broadcast position by position while every lane accumulates its own channels of V.  The K and V rows of the
// first round are requested by the caller's thread before the query is known (see `prefetch`), and the sixteen
// per-warp (max, sum, ctx) triples are merged once.
template <int HD>
struct MegaKvRound {
    uint4 kreg[2][HD / 32];
    uint2 vreg[16];
};

template <int HD>
__device__ __forceinline__ void mega_kv_load(MegaKvRound<HD>& r, const __half* K, const __half* V, int base, int n_cached, int warp, int lane) {
    constexpr int cpl = HD / 32, KV4 = HD / 32;
    const int sub = lane & 3, tl = lane >> 2;
#pragma unroll
    for (int st = 0; st < 2; st++) {
        const int t = base + warp + kMegaConsumerWarps * (st * 8 + tl);
#pragma unroll
        for (int c = 0; c < KV4; c++) {
            r.kreg[st][c] = make_uint4(0, 0, 0, 0);
            if (t < n_cached) r.kreg[st][c] = __ldcg(reinterpret_cast<const uint4*>(K + (size_t)t * HD + sub * (HD / 4)) + c);
        }
    }
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const int t = base + warp + kMegaConsumerWarps * j;
        r.vreg[j] = make_uint2(0, 0);
        if (t < n_cached) {
            const __half* vr = V + (size_t)t * HD + lane * cpl;
            if (cpl == 4) r.vreg[j] = __ldcg(reinterpret_cast<const uint2*>(vr));
            else if (cpl == 2) r.vreg[j].x = __ldcg(reinterpret_cast<const unsigned int*>(vr));
            else r.vreg[j].x = (unsigned int)__ldcg(reinterpret_cast<const unsigned short*>(vr));
        }
    }
}

template <int HD, class WaitQ>
__device__ __forceinline__ void mega_attention(const MegaArgs& a, const MegaShared& s, const MegaShare& w, int layer, int pos, WaitQ wait_q) {
    const ModelDims& m = a.m;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int cpl = HD / 32, KV4 = HD / 32;
    const int visible = pos + 1;
    const __half* K = a.kv.k + a.kv.offset(m, layer, 0, w.kvh, 0);
    const __half* V = a.kv.v + a.kv.offset(m, layer, 0, w.kvh, 0);
    const float scale = 1.0f / sqrtf((float)HD);
    const int sub = lane & 3, tl = lane >> 2;
    constexpr int kRound = kMegaConsumerWarps * 16;  // positions per round
    float m_w = -INFINITY, l_w = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int base = 0; base < visible - 1 || base == 0; base += kRound) {
        // cached rows of this round (the newest position is not in the cache: its key and value come with the query)
        MegaKvRound<HD> cur;
        mega_kv_load<HD>(cur, K, V, base, visible - 1, warp, lane);
        if (base == 0) wait_q();  // the loads above are in flight while the query is awaited
        float sc[2];
        float mx = -INFINITY;
#pragma unroll
        for (int st = 0; st < 2; st++) {
            const int t = base + warp + kMegaConsumerWarps * (st * 8 + tl);
            float dot = 0.f;
#pragma unroll
            for (int c = 0; c < KV4; c++) {
                const uint32_t ww[4] = {cur.kreg[st][c].x, cur.kreg[st][c].y, cur.kreg[st][c].z, cur.kreg[st][c].w};
                const float* qv = s.qs + sub * (HD / 4) + c * 8;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&ww[i]));
                    dot = fmaf(f.x, qv[2 * i], dot);
                    dot = fmaf(f.y, qv[2 * i + 1], dot);
                }
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            sc[st] = t < visible - 1 ? dot * scale : -INFINITY;
            mx = fmaxf(mx, sc[st]);
        }
        const float m_new = fmaxf(m_w, warp_max(mx));
        float pr[2], psum = 0.f;
#pragma unroll
        for (int st = 0; st < 2; st++) {
            pr[st] = sc[st] == -INFINITY ? 0.f : __expf(sc[st] - m_new);
            psum += pr[st];
        }
        const float corr = m_w == -INFINITY ? 0.f : __expf(m_w - m_new);
        l_w = l_w * corr + 0.25f * warp_sum(psum);  // every probability sits in four lanes
#pragma unroll
        for (int c = 0; c < 4; c++) acc[c] *= corr;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const float pj = __shfl_sync(0xffffffffu, pr[j >> 3], (j & 7) * 4);
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&cur.vreg[j].x));
            const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&cur.vreg[j].y));
            acc[0] = fmaf(pj, f0.x, acc[0]);
            if (cpl >= 2) acc[1] = fmaf(pj, f0.y, acc[1]);
            if (cpl == 4) { acc[2] = fmaf(pj, f1.x, acc[2]); acc[3] = fmaf(pj, f1.y, acc[3]); }
        }
        m_w = m_new;
    }
    // the newest position: key and value from shared memory, handled by one warp as a round of a single position
    if (warp == (visible - 1) % kMegaConsumerWarps) {
        float dot = 0.f;
#pragma unroll
        for (int c = 0; c < cpl; c++) dot = fmaf(s.qs[lane * cpl + c], __half2float(s.kn[lane * cpl + c]), dot);
        const float sn = warp_sum(dot) * scale;
        const float m_new = fmaxf(m_w, sn);
        const float corr = m_w == -INFINITY ? 0.f : __expf(m_w - m_new);
        const float pn = __expf(sn - m_new);
        l_w = l_w * corr + pn;
#pragma unroll
        for (int c = 0; c < 4; c++)
            if (c < cpl) acc[c] = fmaf(pn, __half2float(s.vn[lane * cpl + c]), acc[c] * corr);
        m_w = m_new;
    }
    // merge the per-warp partial results (a warp that saw no position carries max = -inf, sum = 0)
#pragma unroll
    for (int c = 0; c < 4; c++)
        if (c < cpl) s.part[warp * HD + lane * cpl + c] = acc[c];
    if (lane == 0) { s.red[warp] = m_w; s.red[kMegaConsumerWarps + warp] = l_w; }
    consumer_sync();
    if (tid < HD) {
        float gm = -INFINITY;
#pragma unroll
        for (int x = 0; x < kMegaConsumerWarps; x++) gm = fmaxf(gm, s.red[x]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int x = 0; x < kMegaConsumerWarps; x++) {
            const float f = s.red[x] == -INFINITY ? 0.f : __expf(s.red[x] - gm);
            num = fmaf(s.part[x * HD + tid], f, num);
            den = fmaf(s.red[kMegaConsumerWarps + x], f, den);
        }
        s.ctx[tid] = den > 0.f ? num / den : 0.f;
    }
    consumer_sync();
}

// Partial output projection: rows [blk*rpb, ...) of Wo restricted to this head's columns; every row's partial sum is
// one contribution to the counted sum of that row (head 0 also carries the residual).
template <int HD>
__device__ __forceinline__ void mega_wo_partial(const MegaArgs& a, const MegaShared& s, const MegaShare& w, unsigned& c) {
    const ModelDims& m = a.m;
    const MegaPlan& p = a.plan;
    const int tid = threadIdx.x;
    constexpr int ipt = HD <= 64 ? 8 : 16;  // inputs per thread
    constexpr int tpr = HD / ipt;           // threads per row
    const int psub = tid % tpr;
    constexpr int rows_per_pass = kMegaConsumers / tpr;
    for (int r0 = 0; r0 < p.rpb; r0 += p.s2_rpc) {  // the block's rows arrive in chunks of s2_rpc
        const uint8_t* chunk = mega_acquire(a, s, c);
        const int nr = min(p.s2_rpc, p.rpb - r0);
        for (int rb = 0; rb < nr; rb += rows_per_pass) {  // uniform trip count: the shuffles below need every lane
            const int r = rb + tid / tpr;
            const int orow = w.blk * p.rpb + r0 + r;
            const bool valid = r < nr;
            float v = 0.f;
            if (valid) {
                const uint8_t* wrow = chunk + (size_t)r * HD * 2 + psub * ipt * 2;
#pragma unroll
                for (int q = 0; q < ipt / 8; q++) fma_vec16<WT_F16>(lds128(wrow + 16 * q), nullptr, 0, s.ctx + psub * ipt + 8 * q, 0.f, v);
            }
#pragma unroll
            for (int o = tpr / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (valid && psub == 0 && orow < m.d_model) {
                if (w.head == 0) v += s.xraw[orow];  // residual, added once
                red_add_u64(a.mid_sums + orow, counted(v));
            }
        }
        mega_release(a, s, c);
        c++;
    }
}

// S3: gate/up rows of this CTA's hidden units, SiLU*up.
__device__ __forceinline__ void mega_s3_up(const MegaArgs& a, const MegaShared& s, float inv, const uint8_t* chunk, int j0, int n_items) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int iters = (a.m.d_model + 255) / 256;
    for (int j = warp; j < n_items; j += kMegaConsumerWarps) {
        float v[2];
        mega_dot_rows<2>(chunk + (size_t)(2 * j) * a.plan.row_bytes, a.plan.row_bytes, a.m.d_model, 0, iters, s.xs, lane, v);
        if (lane == 0) {
            const float g = v[0] * inv;
            s.outv[j0 + j] = g / (1.0f + __expf(-g)) * (v[1] * inv);  // silu(g) = g * sigmoid(g) = 0.5 g (1 + tanh(g / 2))
        }
    }
}

// ------------------------------------------------------------------------------------------------ the kernel

template <int HD>
__global__ void __launch_bounds__(kMegaThreads, 1) k_decode_mega(const MegaArgs a) {
    extern __shared__ __align__(128) uint8_t mega_smem[];
    const MegaShared s = mega_carve(mega_smem, a);
    const MegaPlan& p = a.plan;
    const ModelDims& m = a.m;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int L = m.n_layer;
    if (tid == 0) {
        *s.share = mega_share(m, p, (int)blockIdx.x);
        for (int i = 0; i < p.n_slots; i++) { mbar_init(s.full + i, 1); mbar_init(s.empty + i, kMegaConsumerWarps); }
        *s.abort = 0;
        *s.stop = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int k = tid; k < m.d_model; k += kMegaThreads) s.prev[k] = 0ull;  // the counted sums are zero at launch
    __syncthreads();
    const MegaShare& w = *s.share;  // read from shared memory wherever it is needed: no registers, no recomputation
    const uint8_t* blob = a.pack + (size_t)blockIdx.x * p.cta_bytes;
    const long long head_off = (long long)L * p.layer_bytes;

    if (warp == kMegaConsumerWarps) {
        // ---------------- producer: one thread streams this CTA's chunks in consumption order ----------------
        if (lane == 0) {
            unsigned c = 0;
#ifdef MEGA_FINE_TRACE
            int p_step = 0, p_n = 0;
#endif
            const uint64_t policy = l2_evict_first_policy();
            auto issue = [&](long long off, int bytes) {
                const unsigned slot = c % (unsigned)p.n_slots;
                if (mega_aborting(s) || *reinterpret_cast<volatile int*>(s.stop)) return;  // nothing more is copied
#ifdef MEGA_FINE_TRACE
                const bool tr = a.trace && (int)blockIdx.x == a.trace_cta && p_step == a.n_steps - 1 && p_n < 56;
                if (tr) a.trace[400 + 2 * p_n] = clock64();
#endif
                if (c >= (unsigned)p.n_slots) mega_wait(a, s, s.empty + slot, ((c / (unsigned)p.n_slots) - 1u) & 1u, 4);
                if (mega_aborting(s) || *reinterpret_cast<volatile int*>(s.stop)) return;
                mbar_expect_tx(s.full + slot, (unsigned)bytes);
                bulk_copy_g2s(s.slots + (size_t)slot * p.slot_bytes, blob + off, (unsigned)bytes, s.full + slot, policy);
#ifdef MEGA_FINE_TRACE
                if (tr) { a.trace[400 + 2 * p_n + 1] = clock64(); p_n++; }
#endif
                c++;
            };
            // a stage's slice: whole items, `per_chunk` at a time
            auto issue_stage = [&](long long off, int items, int per_chunk, int item_bytes) {
                for (int i0 = 0; i0 < items; i0 += per_chunk) issue(off + (long long)i0 * item_bytes, min(per_chunk, items - i0) * item_bytes);
            };
            for (int step = 0; step < a.n_steps; step++) {
#ifdef MEGA_FINE_TRACE
                p_step = step;
#endif
                if (step > 0) {
                    for (int l = 0; l < L; l++) {
                        long long off = (long long)l * p.layer_bytes;
                        if (w.in_group) issue_stage(off, w.s1_n, p.s1_ipc, 2 * p.row_bytes);
                        off += p.s1_bytes;
                        if (w.in_group) issue_stage(off, p.rpb, p.s2_rpc, m.head_dim * 2);
                        off += p.s2_bytes;
                        issue_stage(off, w.h_n, p.s3a_ipc, 2 * p.row_bytes); off += p.s3a_bytes;
                        issue_stage(off, w.d_n, p.s3b_rpc, p.down_row_bytes);
                    }
                }
                issue_stage(head_off, w.v_n, p.head_rpc, p.row_bytes);
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
#ifdef MEGA_FINE_TRACE
    int n_fine = 0;
    int fine_layer = -1, fine_step = -1;
#define FINE() do { if (a.trace && (int)blockIdx.x == a.trace_cta && tid == 0 && fine_step == a.n_steps - 1 && (fine_layer == 2 || fine_layer == 99) && n_fine < 120) a.trace[256 + n_fine++] = clock64(); } while (0)
#else
#define FINE() do {} while (0)
#endif
    int n_stamp = 0;
    auto stamp = [&](int step) {
        if (a.trace && (int)blockIdx.x == a.trace_cta && tid == 0 && step == a.n_steps - 1) a.trace[n_stamp++] = clock64();
    };
    unsigned c = 0;      // chunk counter, advances in lock step with the producer's
    int pos = a.pos0;    // visible tokens
    uint32_t tok = 0;
    int emitted = 0;
    constexpr int half = HD / 2;
    const int d = m.d_model;
    const float* fin_gain = a.norms + (size_t)(2 * L) * d;
    unsigned long long* my_qkv = a.qkv_words + (size_t)w.kvh * 2 * p.group_items;

    // Stages one value of the residual stream: raw copy, gained copy in the dot-product order, sum of squares.
    auto stage_x = [&](float* raw, int k, float v, float g, float& ss) {
        raw[k] = v;
        s.xs[xs_index<8>(k)] = v * g;
        ss = fmaf(v, v, ss);
    };

    for (int step = 0; step < a.n_steps; step++) {
        if (step > 0) {
            const uint16_t* emb_row = a.tok_emb + (size_t)tok * d;
            if (tid < half) s.rope[tid] = a.rope[(size_t)pos * half + tid];  // published by the barrier of the first norm
            for (int l = 0; l < L; l++) {
                const unsigned seq = (unsigned)((step - 1) * L + l + 1);  // tag of everything this layer publishes
                float inv = 0.f;
#ifdef MEGA_FINE_TRACE
                fine_layer = l; fine_step = step;
#endif
                stamp(step);
                if (w.in_group) {
                    // ---- S1: x of this layer.  x_words is re-written by the W2 stage of this layer, which starts only
                    // after every CTA has published its activation, i.e. after every group CTA has read x here.
                    const float* gain = a.norms + (size_t)(2 * l) * d;
                    float ss = 0.f;
                    if (l == 0) {
                        for (int k = tid; k < d; k += kMegaConsumers) stage_x(s.xraw, k, __half2float(__ushort_as_half(emb_row[k])), __ldg(gain + k), ss);
                    } else {
                        mega_read_words(a, s, a.x_words, d, seq - 1, 5, gain, [&](int k, float v, float g) { stage_x(s.xraw, k, v, g, ss); });
                    }
                    FINE();
                    ss = mega_block_sum(ss, s.red);
                    inv = 1.0f / sqrtf(ss / (float)d + m.eps);
                    FINE();
                    stamp(step);
                    for (int i0 = 0; i0 < w.s1_n; i0 += p.s1_ipc) {
                        const uint8_t* ch = mega_acquire(a, s, c);
                        FINE();
                        mega_s1(a, s, w, l, pos, inv, ch, i0, min(p.s1_ipc, w.s1_n - i0));
                        FINE();
                        mega_release(a, s, c); c++;
                    }
                    consumer_sync();
                    FINE();
                    // publish this CTA's pairs: one warp writes consecutive words.  qkv_words is re-written one layer
                    // later, after x_words of this layer is complete, which needs every CTA's W2 rows, hence the whole
                    // activation vector, hence every group CTA past its S2 of this layer.
                    for (int t = tid; t < 2 * w.s1_n; t += kMegaConsumers) st_word(my_qkv + 2 * w.s1_begin + t, tagged(s.outv[t], seq));
                    stamp(step);
                    {
                        FINE();
                        mega_attention<HD>(a, s, w, l, pos, [&]() {
                            // q of this CTA's head, k and v of the KV head: pairs in the order S1 published them
                            FINE();
                            if (tid < 3 * half) {
                                const int section = tid / half, idx = tid - section * half;
                                const int item = (section == 0 ? w.hq * half : section == 1 ? p.qpk * half : (p.qpk + 1) * half) + idx;
                                ulonglong2 v = make_ulonglong2(0, 0);
                                unsigned spins = 0;
                                if (!mega_aborting(s)) {
                                    while (true) {
                                        v = ld_words2(my_qkv + 2 * item);
                                        if ((unsigned)(v.x >> 32) == seq && (unsigned)(v.y >> 32) == seq) break;
                                        if (mega_spin_out(a, s, spins, 6)) break;
                                    }
                                }
                                const float v0 = __uint_as_float((unsigned)v.x), v1 = __uint_as_float((unsigned)v.y);
                                if (section == 0) { s.qs[idx] = v0; s.qs[idx + half] = v1; }
                                else if (section == 1) { s.kn[idx] = __float2half_rn(v0); s.kn[idx + half] = __float2half_rn(v1); }
                                else { s.vn[2 * idx] = __float2half_rn(v0); s.vn[2 * idx + 1] = __float2half_rn(v1); }
                            }
                            FINE();
                            consumer_sync();
                            FINE();
                            stamp(step);
                        });
                        stamp(step);
                        mega_wo_partial<HD>(a, s, w, c);
                    }
                    stamp(step);
                } else {
                    stamp(step); stamp(step); stamp(step); stamp(step); stamp(step);
                }
                // ---- S3: x_mid = residual + attention projection.  mid_sums receives the next layer's contributions
                // only after that layer's S1, which needs x_words of this layer complete, i.e. every CTA past this read.
                {
                    const float* gain = a.norms + (size_t)(2 * l + 1) * d;
                    float ss = 0.f;
                    FINE();
                    mega_read_sums(a, s, a.mid_sums, d, m.n_head, 7, gain, [&](int k, float v, float g) { stage_x(s.xmid, k, v, g, ss); });
                    FINE();
                    ss = mega_block_sum(ss, s.red);
                    inv = 1.0f / sqrtf(ss / (float)d + m.eps);
                }
                stamp(step);
                for (int j0 = 0; j0 < w.h_n; j0 += p.s3a_ipc) {
                    FINE();
                    const uint8_t* ch = mega_acquire(a, s, c);
                    FINE();
                    mega_s3_up(a, s, inv, ch, j0, min(p.s3a_ipc, w.h_n - j0));
                    FINE();
                    mega_release(a, s, c); c++;
                }
                consumer_sync();
                FINE();
                // act_words is re-written one layer later, after mid_sums of that layer is complete, which needs every group
                // CTA past x_words of this layer, i.e. every CTA past its W2 rows and so past this activation vector.
                for (int t = tid; t < w.h_n; t += kMegaConsumers) st_word(a.act_words + w.h_begin + t, tagged(s.outv[t], seq));
                stamp(step);
                // ---- the whole activation vector, then this CTA's rows of W2 (+ residual)
                FINE();
                mega_read_words(a, s, a.act_words, m.hidden, seq, 8, nullptr, [&](int k, float v, float) { s.xs[xs_index<8>(k)] = v; });
                FINE();
                consumer_sync();
                FINE();
                stamp(step);
                {
                    const int iters = (m.hidden + 255) / 256;
                    for (int r0 = 0; r0 < w.d_n; r0 += p.s3b_rpc) {
                        const uint8_t* ch = mega_acquire(a, s, c);
                        FINE();
                        const int nr = min(p.s3b_rpc, w.d_n - r0);
                        // each row is cut into `kparts` ranges of slices so that all warps work on few rows
                        const int kparts = max(1, min(kMegaConsumerWarps / nr, iters));
                        const int per = (iters + kparts - 1) / kparts;
                        for (int u = warp; u < nr * kparts; u += kMegaConsumerWarps) {
                            const int r = u % nr, part = u / nr;
                            float v[1];
                            mega_dot_rows<1>(ch + (size_t)r * p.down_row_bytes, p.down_row_bytes, m.hidden, part * per, min(iters, (part + 1) * per), s.xs, lane, v);
                            if (lane == 0) s.outv[(r0 + r) * kMegaConsumerWarps + part] = v[0];
                        }
                        FINE();
                        mega_release(a, s, c); c++;
                        consumer_sync();
                        FINE();
                        for (int t = tid; t < nr; t += kMegaConsumers) {
                            float v = s.xmid[w.d_begin + r0 + t];  // residual
                            for (int part = 0; part < kparts; part++) v += s.outv[(r0 + t) * kMegaConsumerWarps + part];
                            st_word(a.x_words + w.d_begin + r0 + t, tagged(v, seq));
                        }
                    }
                }
                stamp(step);
            }
            pos++;  // the token that was just processed is now visible
        }
        // ---- LM head over this CTA's vocabulary rows, first-max argmax
#ifdef MEGA_FINE_TRACE
        fine_layer = 99; fine_step = step;
#endif
        stamp(step);
        {
            float ss = 0.f;
            if (step == 0) {
                for (int k = tid; k < d; k += kMegaConsumers) stage_x(s.xraw, k, __ldcg(a.hidden_io + k), __ldg(fin_gain + k), ss);
            } else {
                mega_read_words(a, s, a.x_words, d, (unsigned)(step * L), 9, fin_gain, [&](int k, float v, float g) { stage_x(s.xraw, k, v, g, ss); });
            }
            consumer_sync();  // the RMSNorm scale is positive: the arg-max does not need it
        }
        stamp(step);
        float best_v = -INFINITY;
        int best_i = 0x7fffffff;
        {
            const int iters = (d + 255) / 256;
            for (int r0 = 0; r0 < w.v_n; r0 += p.head_rpc) {
                FINE();
                const uint8_t* ch = mega_acquire(a, s, c);
                FINE();
                const int nrows = min(p.head_rpc, w.v_n - r0);
                // two rows per warp per pass; a row past the chunk's end repeats the last one
                for (int r = 2 * warp; r < nrows; r += 2 * kMegaConsumerWarps) {
                    float v[2];
                    const int second = r + 1 < nrows ? 1 : 0;
                    mega_dot_rows<2>(ch + (size_t)r * p.row_bytes, second * p.row_bytes, d, 0, iters, s.xs, lane, v);
                    const int g = w.v_begin + r0 + r;
                    if (v[0] > best_v) { best_v = v[0]; best_i = g; }
                    if (second && v[1] > best_v) { best_v = v[1]; best_i = g + 1; }
                }
                mega_release(a, s, c); c++;
            }
        }
        // CTA-wide best (larger value first, then smaller index), published as two tagged words
        if (lane == 0) s.key[warp] = best_i != 0x7fffffff ? pack_best(best_v, best_i) : 0ull;
        consumer_sync();
        if (tid == 0) {
            unsigned long long k = 0ull;
#pragma unroll
            for (int x = 0; x < kMegaConsumerWarps; x++) k = max(k, s.key[x]);
            // Everything this CTA wrote with plain stores during the step (KV-cache rows) is ordered before the words
            // below, and a reader orders its later loads after seeing them: one fence pair per token.
            __threadfence();
            const unsigned tag = (unsigned)step + 1u;
            unsigned long long* mine = a.cand_words + 4 * (size_t)blockIdx.x;
            st_word(mine, ((unsigned long long)tag << 32) | (k >> 32));
            st_word(mine + 1, ((unsigned long long)tag << 32) | (k & 0xffffffffull));
        }
        stamp(step);
        {
            unsigned long long k = 0ull;
            if (tid < p.n_cta) {
                const unsigned tag = (unsigned)step + 1u;
                ulonglong2 v = make_ulonglong2(0, 0);
                unsigned spins = 0;
                if (!mega_aborting(s)) {
                    while (true) {
                        v = ld_words2(a.cand_words + 4 * (size_t)tid);
                        if ((unsigned)(v.x >> 32) == tag && (unsigned)(v.y >> 32) == tag) break;
                        if (mega_spin_out(a, s, spins, 10)) break;
                    }
                }
                __threadfence();
                k = ((v.x & 0xffffffffull) << 32) | (v.y & 0xffffffffull);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) k = max(k, __shfl_xor_sync(0xffffffffu, k, off));
            consumer_sync();  // s.key was read by thread 0 above
            if (lane == 0) s.key[warp] = k;
            if (tid == 0) s.red[63] = mega_aborting(s) ? 1.f : 0.f;  // one decision for the whole CTA
            consumer_sync();
            k = 0ull;
#pragma unroll
            for (int x = 0; x < kMegaConsumerWarps; x++) k = max(k, s.key[x]);
            tok = min(0xffffffffu - (uint32_t)(k & 0xffffffffull), (uint32_t)(m.vocab - 1));  // in range even if every logit was NaN
        }
        stamp(step);
        emitted = step + 1;
        if (blockIdx.x == 0 && tid == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (step == 0) a.stamps[1] = t;
            a.rs.out[step] = tok;
            if (a.token_times) a.token_times[step] = t;
        }
        // Llama rule: the end-of-sequence token is emitted, then the loop stops (every CTA sees the same token)
        const bool eos = m.eos_token >= 0 && tok == (uint32_t)m.eos_token;
        if (eos || s.red[63] != 0.f) {
            if (tid == 0) *reinterpret_cast<volatile int*>(s.stop) = 1;
            break;
        }
    }
    if (blockIdx.x == 0) {
        // the sequence's last hidden state (what the head just read)
        for (int k = tid; k < d; k += kMegaConsumers) a.hidden_io[k] = s.xraw[k];
        if (tid == 0) {
            a.rs.pos[0] = pos;
            a.rs.tok[0] = tok;
            a.rs.next[0] = tok;
            a.rs.n_out[0] = emitted;
            a.stamps[2] = (unsigned long long)emitted;
        }
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

// One CTA builds the blob of one CTA of the decode kernel.
__global__ void k_build_pack(PackSources src, MegaPlan p, ModelDims m, uint8_t* pack) {
    const int cta = blockIdx.x;
    uint8_t* blob = pack + (size_t)cta * p.cta_bytes;
    const int d = m.d_model, hd = m.head_dim;
    const MegaShare w = mega_share(m, p, cta);
    for (int l = 0; l < m.n_layer; l++) {
        uint8_t* base = blob + (size_t)l * p.layer_bytes;
        // S1: pairs of rows in RoPE order
        for (int i = 0; i < p.s1_max; i++) {
            const __half *r0 = nullptr, *r1 = nullptr;
            if (w.in_group && i < w.s1_n) {
                int kind, row0, row1, idx;
                mega_s1_rows(m, p, w.kvh, w.s1_begin + i, kind, row0, row1, idx);
                const __half* W = kind == 0 ? src.wq[l] : kind == 1 ? src.wk[l] : src.wv[l];
                r0 = W + (size_t)row0 * d; r1 = W + (size_t)row1 * d;
            }
            pack_copy(base + (size_t)(2 * i) * p.row_bytes, r0, p.row_bytes);
            pack_copy(base + (size_t)(2 * i + 1) * p.row_bytes, r1, p.row_bytes);
        }
        base += p.s1_bytes;
        // S2: rows [blk*rpb, +rpb) of Wo, columns of one head
        for (int r = 0; r < p.rpb; r++) {
            const int orow = w.blk * p.rpb + r;
            const __half* sp = (w.in_group && orow < d) ? src.wo[l] + (size_t)orow * m.q_dim + (size_t)w.head * hd : nullptr;
            pack_copy(base + (size_t)r * hd * 2, sp, hd * 2);
        }
        base += p.s2_bytes;
        // S3a: (gate_j, up_j) row pairs
        for (int j = 0; j < p.hpc_max; j++) {
            const int hrow = w.h_begin + j;
            pack_copy(base + (size_t)(2 * j) * p.row_bytes, j < w.h_n ? src.w1[l] + (size_t)hrow * d : nullptr, p.row_bytes);
            pack_copy(base + (size_t)(2 * j + 1) * p.row_bytes, j < w.h_n ? src.w3[l] + (size_t)hrow * d : nullptr, p.row_bytes);
        }
        base += p.s3a_bytes;
        // S3b: this CTA's rows of W2
        for (int r = 0; r < p.dpc_max; r++)
            pack_copy(base + (size_t)r * p.down_row_bytes, r < w.d_n ? src.w2[l] + (size_t)(w.d_begin + r) * m.hidden : nullptr, p.down_row_bytes);
    }
    uint8_t* hb = blob + (size_t)m.n_layer * p.layer_bytes;
    for (int i = 0; i < p.vpc_max; i++)
        pack_copy(hb + (size_t)i * p.row_bytes, i < w.v_n ? src.lm_head + (size_t)(w.v_begin + i) * d : nullptr, p.row_bytes);
}

}  // namespace esp
