// Persistent whole-loop decode kernel for one sequence of a Llama-style fp16 model.
//
// One cooperative launch runs an entire greedy decode loop: `n_steps` heads and up to `n_steps - 1` forward
// passes.  The grid has one CTA per SM.  Inside a CTA one producer warp streams that CTA's weights from HBM into a
// shared-memory ring with bulk async copies (cp.async.bulk + mbarrier), always running ahead of the sixteen
// consumer warps (a watcher warp turns the copies' completions into a counter the consumers can read cheaply), so HBM keeps streaming while the consumers wait on the activation dependencies of the step.
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
// Products.  The fp16->fp32 conversion rate of the CUDA cores (measured: 20-26 weights per clock per SM from shared
// memory) would make the row products the longest link of the chain, so they are issued as m16n8k16 tensor-core
// instructions: sixteen weight rows are the A operand, and the fp32 activation vector, split exactly into two fp16
// vectors (x = hi + lo, |error| <= 2^-22 |x|), occupies columns 0 and 1 of the B operand; the accumulators are fp32.  The
// pack stores every chunk in the order the A fragments are read: for each block of 32 columns, for each row, 64 bytes.
// GGUF Q8_0 / Q4_0 matrices travel through the ring as their blocks (32 or 16 bytes per row and block of 32 columns,
// the fp16 scales behind them): 34/32 or 18/32 bytes per weight from HBM, never an fp16 copy.  A block of 32 columns
// is exactly two m16n8k16 steps: the integers are widened to fp16 exactly in registers, the products of a block are
// accumulated from zero and multiplied by the block's scale in fp32 (value = fp32(d) * q as in the GGUF definition).
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
constexpr int kMegaThreads = kMegaConsumers + 64;  // + the producer warp and the watcher warp
constexpr unsigned kMegaSpinLimit = 1u << 21;      // default attempts per wait before the kernel gives up (a few seconds)
constexpr int kMegaTraceLayer = 10;                // stamps per layer
constexpr int kMegaTraceHead = 4;                  // stamps of the head
constexpr int kMegaChunkRows = 256;                // most rows of one chunk (16 tiles of 16 rows)
// Which exchanges give every CTA cache lines of its own (see mega_read_lines) is the plan's choice (act_wpc > 0).
// Measured on the 6-layer d768 model against compact arrays: arg-max candidates -4.6 us per token, activation vector
// -1.4 us, layer output x +0.3 us (five words per CTA: three times as many lines to poll for little contention saved).
// On the 22-layer d2048 model, whose activation vector needs two polling rounds either way, lines per CTA cost 1.8 us
// per layer.  So: candidates always, the activation vector when all of it is polled in one round, x never.
constexpr int kMegaLineWords = 16;  // 8-byte words of a 128-byte cache line
constexpr int kMegaCandStride = kMegaLineWords;  // 8-byte words between the arg-max candidates of two CTAs: a cache line each
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
    int act_wpc;  // exchange words reserved per CTA for its elements of the activation vector (whole cache lines); 0 = compact array
    int wt_layer, wt_head;  // storage type of the layer matrices and of the LM head: WT_F16, WT_Q8_0 or WT_Q4_0
    int row_bytes;       // packed bytes of a row of d_model columns of a layer matrix
    int down_row_bytes;  // ... of hidden columns (W2)
    int wo_row_bytes;    // ... of head_dim columns (this head's part of a row of Wo)
    int head_row_bytes;  // ... of d_model columns of the LM head
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
    int off_bar, off_prev, off_key, off_xs, off_xraw, off_xmid, off_rope, off_qs, off_ctx, off_kn, off_vn, off_part, off_red, off_outv, off_flags, off_share, off_beg;
};

// Packed bytes of K columns of one row: fp16, or GGUF blocks of 32 (int8 / nibbles) with one fp16 scale each.
__host__ __device__ inline int mega_row_bytes(int wt, int K) { return wt == WT_Q8_0 ? K + K / 16 : wt == WT_Q4_0 ? K / 2 + K / 16 : K * 2; }

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
    unsigned long long* act_words;  // [hidden] or [n_cta][act_wpc]; tagged: FFN activation
    unsigned long long* qkv_words;  // [n_kv_head][2 * group_items] tagged: post-RoPE q / k / v of one token
    unsigned long long* mid_sums;   // [d_model] counted: residual + attention projection
    unsigned long long* cand_words; // [n_cta][kMegaCandStride] {logit bits, index, 8-bit tag} of each CTA's best row in word 0
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
    const int half = m.head_dim / 2, lg_half = m.head_dim == 32 ? 4 : m.head_dim == 64 ? 5 : 6;  // head_dim is 32, 64 or 128
    if (item < p.qpk * half) {
        const int hq = item >> lg_half;
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

// Bytes of a staged vector of K values (hi and lo fp16 parts, see xa_index; or int8 digits, see qx_store_pair).
__host__ __device__ inline int xa_bytes(int K) { return (K / 32) * 128; }
// Bytes of the per-block scales that accompany a vector staged as int8 digits.
__host__ __device__ inline int qx_scale_bytes(int K) { return (K / 32) * 4; }

// ------------------------------------------------------------------------------------------------ shared state

struct MegaShared {
    uint8_t* slots;
    uint64_t* full;
    uint64_t* empty;
    uint8_t* xa;   // staged activation vector (x * gain, or the FFN activation) as the A operand: hi/lo fp16 (see xa_index)
    float* xraw;   // [d_model] the residual stream entering the layer (also what the head reads)
    float* xmid;   // [d_model] the residual stream after the attention block
    float2* rope;  // [head_dim/2] (cos, sin) of the position being processed
    unsigned long long* prev;  // [d_model] totals of the counted sums seen at the previous exchange
    float* qs;     // [head_dim] query of this CTA's head
    float* ctx;    // [head_dim] attention output of this CTA's head, staged like xa
    __half* kn;    // [head_dim] the new token's key, rounded as the cache stores it
    __half* vn;    // [head_dim]
    float* part;   // [warps][head_dim]
    float* red;    // [64]
    float* partial;  // [2][kMegaChunkRows] partial row sums of a chunk (alternating halves)
    unsigned long long* key;   // [32] arg-max keys
    struct MegaShare* share;  // this CTA's work shares, computed once
    int* hbeg;     // [n_cta + 1] first FFN unit (= element of the activation vector) of every CTA
    int* abort;    // [1] a wait gave up: no more waiting in this CTA
    int* stop;     // [1] the loop ended early (EOS): the producer stops issuing
    unsigned* landed;  // [1] number of chunks whose bytes have arrived (written by the producer warp's watcher lane)
};

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
    s.xa = base + p.off_xs;
    s.xraw = reinterpret_cast<float*>(base + p.off_xraw);
    s.xmid = reinterpret_cast<float*>(base + p.off_xmid);
    s.rope = reinterpret_cast<float2*>(base + p.off_rope);
    s.qs = reinterpret_cast<float*>(base + p.off_qs);
    s.ctx = reinterpret_cast<float*>(base + p.off_ctx);
    s.kn = reinterpret_cast<__half*>(base + p.off_kn);
    s.vn = reinterpret_cast<__half*>(base + p.off_vn);
    s.part = reinterpret_cast<float*>(base + p.off_part);
    s.red = reinterpret_cast<float*>(base + p.off_red);
    s.partial = reinterpret_cast<float*>(base + p.off_outv);
    s.abort = reinterpret_cast<int*>(base + p.off_flags);
    s.stop = s.abort + 1;
    s.landed = reinterpret_cast<unsigned*>(s.abort + 2);
    s.share = reinterpret_cast<MegaShare*>(base + p.off_share);
    s.hbeg = reinterpret_cast<int*>(base + p.off_beg);
    return s;
}

// Fills the offsets and the total size (host side; p.n_slots and p.slot_bytes must be set).
inline void mega_layout(const ModelDims& m, MegaPlan& p) {
    size_t o = (size_t)p.n_slots * p.slot_bytes;
    auto take = [&](size_t bytes) { size_t at = (o + 15) & ~(size_t)15; o = at + bytes; return (int)at; };
    p.off_bar = take(16 * (size_t)p.n_slots);
    p.off_prev = take(8 * (size_t)m.d_model);
    p.off_key = take(8 * 32);
    p.off_xs = take((size_t)xa_bytes(m.d_model > m.hidden ? m.d_model : m.hidden) + qx_scale_bytes(m.d_model > m.hidden ? m.d_model : m.hidden));
    p.off_xraw = take(sizeof(float) * (size_t)m.d_model);
    p.off_xmid = take(sizeof(float) * (size_t)m.d_model);
    p.off_rope = take(sizeof(float2) * (size_t)(m.head_dim / 2));
    p.off_qs = take(sizeof(float) * (size_t)m.head_dim);
    p.off_ctx = take((size_t)xa_bytes(m.head_dim) + qx_scale_bytes(m.head_dim));
    p.off_kn = take(sizeof(__half) * (size_t)m.head_dim);
    p.off_vn = take(sizeof(__half) * (size_t)m.head_dim);
    p.off_part = take(sizeof(float) * (size_t)kMegaConsumerWarps * m.head_dim);
    p.off_red = take(sizeof(float) * 64);
    p.off_outv = take(sizeof(float) * 2 * kMegaChunkRows);
    p.off_flags = take(16);
    p.off_share = take(sizeof(MegaShare));
    p.off_beg = take(sizeof(int) * ((size_t)p.n_cta + 1));
    p.smem_bytes = (int)((o + 127) & ~(size_t)127);
}

__device__ __forceinline__ void mega_fail(const MegaArgs& a, const MegaShared& s, int code) {
    *reinterpret_cast<volatile int*>(s.abort) = 1;
    atomicCAS(a.error, 0, code);
}
__device__ __forceinline__ bool mega_aborting(const MegaShared& s) { return *reinterpret_cast<volatile int*>(s.abort) != 0; }

#ifndef MEGA_POLL_NS
#define MEGA_POLL_NS 0
#endif
// Optional pause between two attempts of a poll of global memory.  Measured on the 6-layer d768 model: 0 and 100 ns
// give the same token time within 1 %, 300 ns costs 11 %, so the default polls back to back.
__device__ __forceinline__ void mega_backoff() {
    if (MEGA_POLL_NS > 0) __nanosleep(MEGA_POLL_NS);
}
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

// Ring bookkeeping shared by the producer and the consumers: chunk c lives in slot c % n_slots and completes phase
// (c / n_slots) & 1 of that slot's barriers.  Kept incrementally: a division by a run-time value on the critical path
// of every chunk costs a lone thread a quarter of a microsecond.
struct MegaCursor {
    unsigned slot = 0, phase = 0;
    __device__ __forceinline__ void next(unsigned n_slots) {
        if (++slot == n_slots) { slot = 0; phase ^= 1u; }
    }
};

// A consumer does not test the slot's mbarrier itself: that test costs ~280 cycles per call on this part even when the
// phase completed long ago.  The producer warp's second lane follows the chunks in order, waits on each barrier and
// publishes the count of landed chunks in a plain shared-memory word (release), which the consumers read (acquire).
__device__ __forceinline__ unsigned ld_acquire_cta_shared(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_cta_shared(unsigned* p, unsigned v) {
    asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ const uint8_t* mega_acquire(const MegaArgs& a, const MegaShared& s, const MegaCursor& c, unsigned index) {
    // one lane per warp polls; the warp barrier that follows orders the other lanes' reads of the chunk after it
    if ((threadIdx.x & 31) == 0 && !mega_aborting(s)) {
        unsigned spins = 0;
        while ((int)(ld_acquire_cta_shared(s.landed) - index) <= 0) {
            if (mega_spin_out(a, s, spins, 3)) break;
        }
    }
    __syncwarp();
    return s.slots + (size_t)c.slot * a.plan.slot_bytes;
}
__device__ __forceinline__ void mega_release(const MegaArgs& a, const MegaShared& s, MegaCursor& c) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(s.empty + c.slot);
    c.next((unsigned)a.plan.n_slots);
}
// Hands back `n` consecutive slots starting at `from` whose release was put off (see the kernel's chunk_products).
__device__ __forceinline__ void mega_release_deferred(const MegaArgs& a, const MegaShared& s, MegaCursor from, int n) {
    __syncwarp();
    for (int i = 0; i < n; i++) {
        if ((threadIdx.x & 31) == 0) mbar_arrive(s.empty + from.slot);
        from.next((unsigned)a.plan.n_slots);
    }
}

// ------------------------------------------------------------------------------------------------ exchanges

// Reads `n` tagged words (n even, 16-byte aligned base) and hands pairs (even index, two values, two gains) to `sink`
// (when n is a multiple of 64 every warp reaches the sink with all its lanes, consecutive pairs in consecutive lanes).  A thread keeps up to
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
                mega_backoff();
            }
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int p = p0 + j * kMegaConsumers + (int)threadIdx.x;
            if (p < n_pairs) sink(2 * p, __uint_as_float((unsigned)w[j].x), __uint_as_float((unsigned)w[j].y), g[j].x, g[j].y);
        }
    }
}

// Tagged words written line by line: the CTA that owns elements [beg[c], beg[c + 1]) of a vector writes them to the
// first words of slot c (`wpc` words per slot: whole cache lines, at least the largest share).  Cache lines with a single
// writer matter: a store to a line that every CTA is polling costs a round of invalidations, and the stores of several
// writers to one line queue up behind one another (sixteen writers per line made the arg-max exchange take 6 us).
// `lines` = positions x CTAs (position q's lines follow position q - 1's); the sink receives (q * n + element, value,
// gain).  `ppl` = pairs of words to read per line = ceil(largest share / 2); every thread takes up to four pairs.
template <class Sink>
__device__ __forceinline__ void mega_read_lines(const MegaArgs& a, const MegaShared& s, const unsigned long long* base, int wpc, const int* beg, int n, int lines, int ppl,
                                                unsigned tag, int code, const float* gain, Sink sink) {
    const int n_cta = a.plan.n_cta;
    const int slots = lines * ppl;
    for (int s0 = 0; s0 < slots; s0 += 4 * kMegaConsumers) {
        ulonglong2 w[4];
        float2 g[4];
        const unsigned long long* src[4];
        int k0[4], cnt[4];
        bool ok[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int slot = s0 + j * kMegaConsumers + (int)threadIdx.x;
            w[j] = make_ulonglong2(0, 0);
            g[j] = make_float2(1.f, 1.f);
            cnt[j] = 0; k0[j] = 0; src[j] = base;
            if (slot < slots) {
                const int line = (int)((unsigned)slot / (unsigned)ppl), jj = slot - line * ppl;
                const int q = line >= n_cta ? 1 : 0, cta = line - q * n_cta;  // at most two positions
                const int first = beg[cta] + 2 * jj;
                cnt[j] = max(0, min(2, beg[cta + 1] - first));
                k0[j] = q * n + first;
                src[j] = base + (size_t)line * wpc + 2 * jj;
                if (gain && cnt[j] > 0) {
                    g[j].x = __ldg(gain + k0[j]);
                    if (cnt[j] > 1) g[j].y = __ldg(gain + k0[j] + 1);
                }
            }
            ok[j] = cnt[j] == 0;
        }
        unsigned spins = 0;
        if (!mega_aborting(s)) {
            while (true) {
                bool all = true;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (!ok[j]) {
                        w[j] = ld_words2(src[j]);
                        ok[j] = (unsigned)(w[j].x >> 32) == tag && (cnt[j] < 2 || (unsigned)(w[j].y >> 32) == tag);
                        all = all && ok[j];
                    }
                }
                if (all) break;
                if (mega_spin_out(a, s, spins, code)) break;
                mega_backoff();
            }
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (cnt[j] > 0) sink(k0[j], __uint_as_float((unsigned)w[j].x), g[j].x);
            if (cnt[j] > 1) sink(k0[j] + 1, __uint_as_float((unsigned)w[j].y), g[j].y);
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
                mega_backoff();
            }
        }
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int p = p0 + j * kMegaConsumers + (int)threadIdx.x;
            if (p < n_pairs) {
                *reinterpret_cast<ulonglong2*>(s.prev + 2 * p) = w[j];
                const long long v0 = (long long)(w[j].x - pv[j].x - (unsigned long long)n_contrib) >> 8;
                const long long v1 = (long long)(w[j].y - pv[j].y - (unsigned long long)n_contrib) >> 8;
                sink(2 * p, (float)v0 * kMegaUnfix, (float)v1 * kMegaUnfix, g[j].x, g[j].y);
            }
        }
    }
}

// Sum over the consumer threads of one float each; every thread receives the result.  One CTA barrier.
__device__ __forceinline__ float mega_block_sum(float v, float* red) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    consumer_sync();
    // sixteen partial sums: four 16-byte loads and a tree of additions instead of a chain of sixteen
    const float4* r4 = reinterpret_cast<const float4*>(red);
    const float4 a = r4[0], b = r4[1], c = r4[2], e = r4[3];
    static_assert(kMegaConsumerWarps == 16, "mega_block_sum reads sixteen partial sums");
    return (((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w))) + (((c.x + c.y) + (c.z + c.w)) + ((e.x + e.y) + (e.z + e.w)));
}

// ------------------------------------------------------------------------------------------------ products

// Where element k of a staged vector lives (in halves): block of 32 columns kb, column c of the B operand (position q's
// hi part is column 2q, its lo part column 2q + 1; NP positions are staged side by side), piece t; the 16 bytes of a
// piece are the B registers of the two m16n8k16 steps of the block.
template <int NP = 1>
__device__ __forceinline__ int xa_index(int k, int c) {
    const int kb = k >> 5, kk = k & 31;
    return (((kb * 2 * NP + c) * 4 + ((kk & 7) >> 1)) << 3) + ((kk >> 3) << 1) + (kk & 1);
}

// Stores v as hi + lo (both fp16, hi saturating) at element k of position q of a staged vector.
template <int NP = 1>
__device__ __forceinline__ void xa_store(__half* xa, int k, float v, int q = 0) {
    __half hi;
    asm("cvt.rn.satfinite.f16.f32 %0, %1;" : "=h"(*reinterpret_cast<unsigned short*>(&hi)) : "f"(v));
    xa[xa_index<NP>(k, 2 * q)] = hi;
    xa[xa_index<NP>(k, 2 * q + 1)] = __float2half_rn(v - __half2float(hi));
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Partial products of the 16-row tile `tile` of a chunk of R rows with the staged vector over the column blocks
// [kb0, kb1).  The weights are the A operand (rows g and g + 8 of the tile: one 16-byte shared-memory load each per two
// m16n8k16 steps), the staged vector the B operand (column 0 = hi part, column 1 = lo part, held by lanes 0..7).  The
// lanes with lane % 4 == q < NP return the sums of position q for rows tile*16 + lane/4 (.x) and + 8 (.y); rows past R are
// meaningless.  With NP positions the staged vector holds 2 NP columns (lanes 0 .. 8 NP - 1 feed the B operand): the
// products of a second position ride in columns the instruction computes anyway.
template <int NP>
__device__ __forceinline__ float2 mega_tile_dot_f16(const uint8_t* chunk, int R, int n_kb, int tile, int kb0, int kb1, const uint8_t* xa, int lane) {
    // four independent accumulator sets: a dependent m16n8k16 costs ~40-60 cycles, and a warp has only a few blocks
    float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f}, c3[4] = {0.f, 0.f, 0.f, 0.f};
    const uint8_t* wp = chunk + ((size_t)(tile * 16 + (lane >> 2)) * 64 + (lane & 3) * 16);
    const size_t kstride = (size_t)R * 64;
    const uint8_t* xp = xa + lane * 16;
    // plain loads: the compiler may move them ahead of the previous block's products, never across a barrier
    auto block = [&](int kb, float (&ce)[4], float (&co)[4]) {
        const uint4 w0 = *reinterpret_cast<const uint4*>(wp + kb * kstride);
        const uint4 w8 = *reinterpret_cast<const uint4*>(wp + kb * kstride + 8 * 64);
        uint4 xv = make_uint4(0, 0, 0, 0);
        if (lane < 8 * NP) xv = *reinterpret_cast<const uint4*>(xp + kb * (128 * NP));
        mma_16816(ce, w0.x, w8.x, w0.y, w8.y, xv.x, xv.y);
        mma_16816(co, w0.z, w8.z, w0.w, w8.w, xv.z, xv.w);
    };
    int kb = kb0;
#pragma unroll 2
    for (; kb + 1 < kb1; kb += 2) {
        block(kb, c0, c1);
        block(kb + 1, c2, c3);
    }
    if (kb < kb1) block(kb, c0, c1);
    // column 0 of the product is w . x_hi, column 1 is w . x_lo
    return make_float2(((c0[0] + c1[0]) + (c2[0] + c3[0])) + ((c0[1] + c1[1]) + (c2[1] + c3[1])),
                       ((c0[2] + c1[2]) + (c2[2] + c3[2])) + ((c0[3] + c1[3]) + (c2[3] + c3[3])));
}

// ---- Q8_0: the activation as int8 digits, the products on the int8 tensor-core path ----
// A Q8_0 weight is an int8: instead of widening it to fp16 (eight byte permutes and subtractions per 32 weights and
// lane), the staged activation is turned into integers.  Per block of 32 columns: q = max|x| / 127 and
// x_i ~ q (d0 + d1 / 128 + d2 / 16384) with three int8 digits (22 bits relative to the block's largest value; the
// weights stay exact).  The digits are B columns 0..2 of one mma.sync.m16n8k32 (s8 x s8), the int32 results are combined
// and scaled by q and the weight block's scale in fp32.  (Q4_0 keeps the fp16 widening: its nibbles carry an offset of 8
// that has to be taken out through a per-block sum of the staged values, and the extra warp reduction per staged block
// cost more than the cheaper products gained: 492 against 460 us per token on the 22-layer d2048 model; Q8_0 gained 3 %.)
//
// Staged layout: block kb holds 128 bytes = [digit c][piece t][8 bytes: columns 4t..4t+3 then 16+4t..16+4t+3], the B
// registers of lane (g = c, t); the block scales q sit behind the vector (qx_scale_bytes).
__device__ __forceinline__ int qx_byte(int kb, int c, int e) { return kb * 128 + c * 32 + (((e & 15) >> 2) << 3) + ((e >> 4) << 2) + (e & 3); }

// Rounding and integer <-> float conversion without conversion instructions (they issue at a quarter of the rate of an
// addition, and this code runs once per staged element and four times per product block): adding 1.5 * 2^23 to a float
// of magnitude below 2^22 rounds it to the nearest integer and leaves that integer in the low mantissa bits.
constexpr float kRoundMagic = 12582912.0f;          // 1.5 * 2^23 = 0x4B400000
constexpr int kRoundMagicBits = 0x4B400000;
__device__ __forceinline__ float int_to_float_small(int v) { return __int_as_float(kRoundMagicBits + v) - kRoundMagic; }  // |v| < 2^22

// The three int8 digits of v * inv (|v * inv| <= 127); dg[c] carries digit c in its low 8 bits (two's complement).
__device__ __forceinline__ void qx_digits(float v, float inv, int (&dg)[3]) {
    const float s0 = v * inv, t0 = s0 + kRoundMagic, d0 = t0 - kRoundMagic;
    const float s1 = (s0 - d0) * 128.f, t1 = s1 + kRoundMagic, d1 = t1 - kRoundMagic;
    const float t2 = (s1 - d1) * 128.f + kRoundMagic;
    dg[0] = __float_as_int(t0); dg[1] = __float_as_int(t1); dg[2] = __float_as_int(t2);
}
// Stages elements k, k + 1 (k even).  Must be called by all 32 lanes of a warp with consecutive pairs: the 16 lanes of a
// half-warp hold one block of 32 columns.  The block's maximum comes from one warp reduction on integers (the bit
// pattern of a non-negative float orders like the float).
__device__ __forceinline__ void qx_store_pair(uint8_t* xq, float* qs, int k, float v0, float v1) {
    const unsigned half_mask = (threadIdx.x & 16) ? 0xffff0000u : 0x0000ffffu;
    const float mx = __uint_as_float(__reduce_max_sync(half_mask, __float_as_uint(fmaxf(fabsf(v0), fabsf(v1)))));
    const float inv = mx > 0.f ? __fdividef(127.0f, mx) : 0.f;
    int d0[3], d1[3];
    qx_digits(v0, inv, d0);
    qx_digits(v1, inv, d1);
    const int kb = k >> 5, e = k & 31;
#pragma unroll
    for (int c = 0; c < 3; c++)
        *reinterpret_cast<uint16_t*>(xq + qx_byte(kb, c, e)) = (uint16_t)__byte_perm((unsigned)d0[c], (unsigned)d1[c], 0x0040);
    if ((threadIdx.x & 15) == 0) qs[kb] = mx * (1.0f / 127.0f);
}
// Stages element k.  Must be called by all 32 lanes of a warp with consecutive k: the warp holds one block.
__device__ __forceinline__ void qx_store_elem(uint8_t* xq, float* qs, int k, float v) {
    const float mx = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(v))));
    const float inv = mx > 0.f ? __fdividef(127.0f, mx) : 0.f;
    int dg[3];
    qx_digits(v, inv, dg);
    const int kb = k >> 5, e = k & 31;
#pragma unroll
    for (int c = 0; c < 3; c++) xq[qx_byte(kb, c, e)] = (uint8_t)dg[c];
    if ((threadIdx.x & 31) == 0) qs[kb] = mx * (1.0f / 127.0f);
}

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Q8_0 chunk: [block][row][piece t: the int8 of columns 4t..4t+3 and 16+4t..16+4t+3], then the scales [block][row] fp16.
__device__ __forceinline__ float2 mega_tile_dot_q8(const uint8_t* chunk, int R, int n_kb, int tile, int kb0, int kb1, const uint8_t* xq, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const int row = tile * 16 + g;
    const uint8_t* wp = chunk + ((size_t)row * 32 + t * 8);
    const size_t kstride = (size_t)R * 32;
    const __half* sp = reinterpret_cast<const __half*>(chunk + (size_t)R * n_kb * 32) + row;
    const uint8_t* xp = xq + (g < 3 ? g * 32 + t * 8 : 0);
    const float* qs = reinterpret_cast<const float*>(xq + (size_t)n_kb * 128);
    // what this lane's two result columns mean: t = 0 holds digits 0 and 1, t = 1 digit 2, the others nothing
    const float k0 = t == 0 ? 1.0f : t == 1 ? (1.0f / 16384.0f) : 0.f, k1 = t == 0 ? (1.0f / 128.0f) : 0.f;
    float a0 = 0.f, a8 = 0.f;
#pragma unroll 4
    for (int kb = kb0; kb < kb1; kb++) {
        uint2 b = make_uint2(0, 0);
        if (g < 3) b = *reinterpret_cast<const uint2*>(xp + kb * 128);
        const float q = qs[kb];
        const float s0 = __half2float(sp[(size_t)kb * R]), s8 = __half2float(sp[(size_t)kb * R + 8]);
        const uint2 w0 = *reinterpret_cast<const uint2*>(wp + kb * kstride);
        const uint2 w8 = *reinterpret_cast<const uint2*>(wp + kb * kstride + 8 * 32);
        int c[4] = {0, 0, 0, 0};
        mma_s8(c, w0.x, w8.x, w0.y, w8.y, b.x, b.y);
        a0 = fmaf(s0 * q, fmaf(int_to_float_small(c[1]), k1, int_to_float_small(c[0]) * k0), a0);
        a8 = fmaf(s8 * q, fmaf(int_to_float_small(c[3]), k1, int_to_float_small(c[2]) * k0), a8);
    }
    // lanes t = 0 and t = 1 hold the two parts of every row's sum
    a0 += __shfl_xor_sync(0xffffffffu, a0, 1);
    a8 += __shfl_xor_sync(0xffffffffu, a8, 1);
    return make_float2(a0, a8);
}

// ---- Q4_0: widened to fp16 in registers (why not the int8 path: see the note above qx_byte) ----
__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
// Four bytes of a Q4_0 block (low nibble = element j, high nibble = element j + 16) -> four half2: the low nibbles of
// bytes (0,1), (2,3), then the high nibbles of (0,1), (2,3), each minus 8.
__device__ __forceinline__ void q4_widen(uint32_t w, uint32_t (&o)[4]) {
    const uint32_t x = w & 0x0F0F0F0Fu, y = (w >> 4) & 0x0F0F0F0Fu;
    const __half2 bias = __floats2half2_rn(1032.f, 1032.f);
    o[0] = h2_bits(__hsub2(u32_as_h2(__byte_perm(x, 0x64646464u, 0x4140)), bias));
    o[1] = h2_bits(__hsub2(u32_as_h2(__byte_perm(x, 0x64646464u, 0x4342)), bias));
    o[2] = h2_bits(__hsub2(u32_as_h2(__byte_perm(y, 0x64646464u, 0x4140)), bias));
    o[3] = h2_bits(__hsub2(u32_as_h2(__byte_perm(y, 0x64646464u, 0x4342)), bias));
}

// Q4_0 chunk: [block][row][16 bytes: piece t = bytes 2t, 2t+1, 2t+8, 2t+9 of the GGUF block], then the scales.
template <int NP>
__device__ __forceinline__ float2 mega_tile_dot_q4(const uint8_t* chunk, int R, int n_kb, int tile, int kb0, int kb1, const uint8_t* xa, int lane) {
    float a0 = 0.f, a8 = 0.f;
    const int row = tile * 16 + (lane >> 2);
    const uint8_t* wp = chunk + ((size_t)row * 16 + (lane & 3) * 4);
    const size_t kstride = (size_t)R * 16;
    const __half* sp = reinterpret_cast<const __half*>(chunk + (size_t)R * n_kb * 16) + row;
    const uint8_t* xp = xa + lane * 16;
#pragma unroll 2
    for (int kb = kb0; kb < kb1; kb++) {
        const uint32_t w0 = *reinterpret_cast<const uint32_t*>(wp + kb * kstride);
        const uint32_t w8 = *reinterpret_cast<const uint32_t*>(wp + kb * kstride + 8 * 16);
        const float s0 = __half2float(sp[(size_t)kb * R]), s8 = __half2float(sp[(size_t)kb * R + 8]);
        uint4 xv = make_uint4(0, 0, 0, 0);
        if (lane < 8 * NP) xv = *reinterpret_cast<const uint4*>(xp + kb * (128 * NP));
        uint32_t g[4], h[4];
        q4_widen(w0, g);
        q4_widen(w8, h);
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        mma_16816(c, g[0], h[0], g[1], h[1], xv.x, xv.y);
        mma_16816(c, g[2], h[2], g[3], h[3], xv.z, xv.w);
        a0 = fmaf(s0, c[0] + c[1], a0);
        a8 = fmaf(s8, c[2] + c[3], a8);
    }
    return make_float2(a0, a8);
}

template <int WT, int NP>
__device__ __forceinline__ float2 mega_tile_dot(const uint8_t* chunk, int R, int n_kb, int tile, int kb0, int kb1, const uint8_t* xa, int lane) {
    if constexpr (WT == WT_Q8_0) return mega_tile_dot_q8(chunk, R, n_kb, tile, kb0, kb1, xa, lane);
    else if constexpr (WT == WT_Q4_0) return mega_tile_dot_q4<NP>(chunk, R, n_kb, tile, kb0, kb1, xa, lane);
    else return mega_tile_dot_f16<NP>(chunk, R, n_kb, tile, kb0, kb1, xa, lane);
}

// All products of one chunk (R <= kMegaChunkRows rows over n_kb column blocks), spread over the consumer warps as
// (16-row tile, column range) units; the number of column ranges is a power of two so that a warp finds its unit with
// shifts (per chunk every scalar instruction of this set-up is on the critical path of the token).  Unit u = tile <<
// lg | range stores its sixteen partial sums at partial[u * 16 ...] (position q: + q * kMegaChunkRows); returns lg.  The
// caller synchronises before reading.
template <int WT, int NP = 1>
__device__ __forceinline__ int mega_chunk_dots(const uint8_t* chunk, int R, int n_kb, const uint8_t* xa, float* partial, int warp, int lane) {
    const int n_tiles = (R + 15) >> 4;
    // lg = log2(column ranges): the largest value with tiles << lg <= warps and 1 << lg <= n_kb
    const int lg_t = n_tiles > 1 ? 32 - __clz(n_tiles - 1) : 0;  // ceil(log2(tiles))
    const int lg = max(0, min(4 - lg_t, 31 - __clz(n_kb)));
    const int per = (n_kb + (1 << lg) - 1) >> lg;
    for (int u = warp; u < (n_tiles << lg); u += kMegaConsumerWarps) {
        const int tile = u >> lg, part = u & ((1 << lg) - 1);
        const float2 y = mega_tile_dot<WT, NP>(chunk, R, n_kb, tile, part * per, min(n_kb, (part + 1) * per), xa, lane);
        if ((lane & 3) < NP) {
            float* dst = partial + (NP > 1 ? (lane & 3) * kMegaChunkRows : 0) + u * 16 + (lane >> 2);
            dst[0] = y.x;
            dst[8] = y.y;
        }
    }
    return lg;
}
// Row r's sum over the column ranges: all loads are issued before the first addition.
__device__ __forceinline__ float mega_take_sum(const float* partial, int lg, int r) {
    const float* src = partial + ((r >> 4) << lg) * 16 + (r & 15);
    float v[16];
#pragma unroll
    for (int part = 0; part < 16; part++) v[part] = part < (1 << lg) ? src[part * 16] : 0.f;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
#pragma unroll
        for (int part = 0; part < o; part++) v[part] += v[part + o];
    }
    return v[0];
}

// ------------------------------------------------------------------------------------------------ consumer stages

// S2: attention of one head over the cached positions [0, pos) plus the new token (whose key and value are in
// shared memory), then this CTA's block of the output projection.
// Each warp owns the positions t = warp + 16*i (16 per round).  Four neighbouring lanes share one position: each loads
// a quarter of its K row with 16-byte vectors and the score is completed with two shuffles.  The probabilities are
// then broadcast position by position while every lane accumulates its own channels of V.  The K and V rows of the
// first round are requested by the caller's thread before the query is known (see `prefetch`), and the sixteen
// per-warp (max, sum, ctx) triples are merged once, by all threads: a few lanes per output channel, combined with
// shuffles (two warps walking all sixteen triples took 0.3 us longer per layer).
template <int HD>
struct MegaKvRound {
    uint4 kreg[2][HD / 32];
    uint2 vreg[16];
};

template <int HD, int NW = kMegaConsumerWarps>  // NW = warps that share one query (position t belongs to warp t % NW)
__device__ __forceinline__ void mega_kv_load(MegaKvRound<HD>& r, const __half* K, const __half* V, int base, int n_cached, int warp, int lane) {
    constexpr int cpl = HD / 32, KV4 = HD / 32;
    const int sub = lane & 3, tl = lane >> 2;
#pragma unroll
    for (int st = 0; st < 2; st++) {
        const int t = base + warp + NW * (st * 8 + tl);
#pragma unroll
        for (int c = 0; c < KV4; c++) {
            r.kreg[st][c] = make_uint4(0, 0, 0, 0);
            if (t < n_cached) r.kreg[st][c] = __ldcg(reinterpret_cast<const uint4*>(K + (size_t)t * HD + sub * (HD / 4)) + c);
        }
    }
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const int t = base + warp + NW * j;
        r.vreg[j] = make_uint2(0, 0);
        if (t < n_cached) {
            const __half* vr = V + (size_t)t * HD + lane * cpl;
            if (cpl == 4) r.vreg[j] = __ldcg(reinterpret_cast<const uint2*>(vr));
            else if (cpl == 2) r.vreg[j].x = __ldcg(reinterpret_cast<const unsigned int*>(vr));
            else r.vreg[j].x = (unsigned int)__ldcg(reinterpret_cast<const unsigned short*>(vr));
        }
    }
}

// With NP positions per pass the consumer warps split into NP teams of NW = 16 / NP warps, one team per query: query qi
// sees the n_cached cached positions and the new positions 0 .. qi, whose keys and values are rows of s.kn / s.vn; its
// context lands in position qi of the staged s.ctx.  The teams run side by side (each reads the cached rows itself).
template <int HD, int NP = 1, int QCTX = 0, class WaitQ>  // QCTX: 0 = fp16 context staging, 1 = int8 digits
__device__ __forceinline__ void mega_attention(const MegaArgs& a, const MegaShared& s, const MegaShare& w, const ModelDims& m, const KvLayout& kv, int layer, int n_cached,
                                               WaitQ wait_q) {
    constexpr int NW = kMegaConsumerWarps / NP;
    const int tid = threadIdx.x, lane = tid & 31;
    const int qi = (tid >> 5) / NW, warp = (tid >> 5) - qi * NW;  // this warp's query and its place in the team
    constexpr int cpl = HD / 32, KV4 = HD / 32;
    const int visible = n_cached + 1;
    const __half* K = kv.k + kv.offset(m, layer, 0, w.kvh, 0);
    const __half* V = kv.v + kv.offset(m, layer, 0, w.kvh, 0);
    const float* qs = s.qs + qi * HD;
    const float scale = 1.0f / sqrtf((float)HD);
    const int sub = lane & 3, tl = lane >> 2;
    constexpr int kRound = NW * 16;  // positions per round of a team
    float m_w = -INFINITY, l_w = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int base = 0; base < visible - 1 || base == 0; base += kRound) {
        // cached rows of this round (the newest position is not in the cache: its key and value come with the query)
        MegaKvRound<HD> cur;
        mega_kv_load<HD, NW>(cur, K, V, base, visible - 1, warp, lane);
        if (base == 0) wait_q();  // the loads above are in flight while the query is awaited
        float sc[2];
        float mx = -INFINITY;
#pragma unroll
        for (int st = 0; st < 2; st++) {
            const int t = base + warp + NW * (st * 8 + tl);
            float dot = 0.f;
#pragma unroll
            for (int c = 0; c < KV4; c++) {
                const uint32_t ww[4] = {cur.kreg[st][c].x, cur.kreg[st][c].y, cur.kreg[st][c].z, cur.kreg[st][c].w};
                const float* qv = qs + sub * (HD / 4) + c * 8;
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
    // the new positions: keys and values from shared memory, each handled by one warp as a round of a single position
#pragma unroll
    for (int j = 0; j < NP; j++) {
        if (j <= qi && warp == (n_cached + j) % NW) {
            const __half* kn = s.kn + j * HD;
            const __half* vn = s.vn + j * HD;
            float dot = 0.f;
#pragma unroll
            for (int c = 0; c < cpl; c++) dot = fmaf(qs[lane * cpl + c], __half2float(kn[lane * cpl + c]), dot);
            const float sn = warp_sum(dot) * scale;
            const float m_new = fmaxf(m_w, sn);
            const float corr = m_w == -INFINITY ? 0.f : __expf(m_w - m_new);
            const float pn = __expf(sn - m_new);
            l_w = l_w * corr + pn;
#pragma unroll
            for (int c = 0; c < 4; c++)
                if (c < cpl) acc[c] = fmaf(pn, __half2float(vn[lane * cpl + c]), acc[c] * corr);
            m_w = m_new;
        }
    }
    // merge the per-warp partial results of every team (a warp that saw no position carries max = -inf, sum = 0)
    const int gw = tid >> 5;  // warp index among all consumers
#pragma unroll
    for (int c = 0; c < 4; c++)
        if (c < cpl) s.part[gw * HD + lane * cpl + c] = acc[c];
    if (lane == 0) { s.red[gw] = m_w; s.red[kMegaConsumerWarps + gw] = l_w; }
    consumer_sync();
    {
        // G lanes per output channel, each with cpl of the team's NW partial results; the lanes combine with shuffles
        constexpr int G = kMegaConsumers / (NP * HD);
        static_assert(G >= 1 && G <= 32 && G * cpl == NW, "merge layout");
        const int o = tid / G, xr = tid - o * G;
        const int qq = o / HD, ch = o - qq * HD;
        float mv[cpl], gm = -INFINITY;
#pragma unroll
        for (int k = 0; k < cpl; k++) { mv[k] = s.red[qq * NW + xr * cpl + k]; gm = fmaxf(gm, mv[k]); }
#pragma unroll
        for (int off = G / 2; off > 0; off >>= 1) gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, off));
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int k = 0; k < cpl; k++) {
            const int x = qq * NW + xr * cpl + k;
            const float f = mv[k] == -INFINITY ? 0.f : __expf(mv[k] - gm);
            num = fmaf(s.part[x * HD + ch], f, num);
            den = fmaf(s.red[kMegaConsumerWarps + x], f, den);
        }
#pragma unroll
        for (int off = G / 2; off > 0; off >>= 1) {
            num += __shfl_xor_sync(0xffffffffu, num, off);
            den += __shfl_xor_sync(0xffffffffu, den, off);
        }
        // the staged operand of the Wo products
        const float cv = den > 0.f ? __fdividef(num, den) : 0.f;
        if constexpr (QCTX != 0) {
            // int8 digit staging works on whole warps of consecutive elements: the channel values are gathered first
            // (in the query's place: every warp is past its scores)
            static_assert(NP == 1, "int8 context staging handles one position");
            if (xr == 0) s.qs[ch] = cv;
            consumer_sync();
            if (tid < HD) qx_store_elem(reinterpret_cast<uint8_t*>(s.ctx), reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(s.ctx) + xa_bytes(HD)), tid, s.qs[tid]);
        } else {
            if (xr == 0) xa_store<NP>(reinterpret_cast<__half*>(s.ctx), ch, cv, qq);
        }
    }
    consumer_sync();
}

// ------------------------------------------------------------------------------------------------ the kernel

template <int HD, int WT>
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
        *s.landed = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int k = tid; k < m.d_model; k += kMegaThreads) s.prev[k] = 0ull;  // the counted sums are zero at launch
    for (int c = tid; c <= p.n_cta; c += kMegaThreads) {
        s.hbeg[c] = mega_share_begin(m.hidden, p.n_cta, c);
    }
    __syncthreads();
    const MegaShare& w = *s.share;  // read from shared memory wherever it is needed: no registers, no recomputation
    const uint8_t* blob = a.pack + (size_t)blockIdx.x * p.cta_bytes;
    const long long head_off = (long long)L * p.layer_bytes;

    if (warp == kMegaConsumerWarps) {
        // ---------------- producer: one thread streams this CTA's chunks in consumption order ----------------
        if (lane == 0) {
            MegaCursor c;
            unsigned issued = 0;
#ifdef MEGA_FINE_TRACE
            int p_step = 0, p_n = 0;
#endif
            const uint64_t policy = l2_evict_first_policy();
            uint64_t keep_policy;
            asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(keep_policy));
            // head rows behind the first (n_slots - 1) chunks: what still has to come from memory when the head begins
            const long long tail_off = (long long)min(w.v_n, (p.n_slots - 1) * p.head_rpc) * p.head_row_bytes;
            const long long tail_bytes = (long long)w.v_n * p.head_row_bytes - tail_off;
            auto issue = [&](long long off, int bytes) {
                if (mega_aborting(s) || *reinterpret_cast<volatile int*>(s.stop)) return;  // nothing more is copied
#ifdef MEGA_FINE_TRACE
                const bool tr = a.trace && (int)blockIdx.x == a.trace_cta && p_step == a.n_steps - 1 && p_n < 56;
                if (tr) a.trace[400 + 2 * p_n] = clock64();
#endif
                if (issued >= (unsigned)p.n_slots) mega_wait(a, s, s.empty + c.slot, c.phase ^ 1u, 4);  // the previous use of the slot was released
                if (mega_aborting(s) || *reinterpret_cast<volatile int*>(s.stop)) return;
                mbar_expect_tx(s.full + c.slot, (unsigned)bytes);
                bulk_copy_g2s(s.slots + (size_t)c.slot * p.slot_bytes, blob + off, (unsigned)bytes, s.full + c.slot, policy);
#ifdef MEGA_FINE_TRACE
                if (tr) { a.trace[400 + 2 * p_n + 1] = clock64(); p_n++; }
#endif
                c.next((unsigned)p.n_slots);
                issued++;
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
                        // HBM idles during the layers (their weights are a full layer ahead in the ring): the part of the head
                        // that the ring cannot hold before the head begins is brought into L2 now, a slice per layer
                        if (tail_bytes > 0 && !mega_aborting(s)) {
                            const long long b0 = tail_bytes * l / L / 16 * 16, b1 = l + 1 == L ? tail_bytes : tail_bytes * (l + 1) / L / 16 * 16;
                            if (b1 > b0)
                                asm volatile("cp.async.bulk.prefetch.L2.global.L2::cache_hint [%0], %1, %2;" ::"l"(blob + head_off + tail_off + b0), "r"((unsigned)(b1 - b0)),
                                             "l"(keep_policy)
                                             : "memory");
                        }
                        long long off = (long long)l * p.layer_bytes;
                        if (w.in_group) issue_stage(off, w.s1_n, p.s1_ipc, 2 * p.row_bytes);
                        off += p.s1_bytes;
                        if (w.in_group) issue_stage(off, p.rpb, p.s2_rpc, p.wo_row_bytes);
                        off += p.s2_bytes;
                        issue_stage(off, w.h_n, p.s3a_ipc, 2 * p.row_bytes); off += p.s3a_bytes;
                        issue_stage(off, w.d_n, p.s3b_rpc, p.down_row_bytes);
                    }
                }
                issue_stage(head_off, w.v_n, p.head_rpc, p.head_row_bytes);
            }
            // every copy that was issued must have landed before the CTA may exit: walk the last n_slots chunks backwards
            MegaCursor k = c;
            const unsigned back = issued < (unsigned)p.n_slots ? issued : (unsigned)p.n_slots;
            for (unsigned i = 0; i < back; i++) {
                if (k.slot == 0) { k.slot = (unsigned)p.n_slots - 1; k.phase ^= 1u; } else k.slot--;
                unsigned spins = 0;
                while (!mbar_try_wait(s.full + k.slot, k.phase) && ++spins < kMegaSpinLimit) {}
            }
        }
        return;
    }
    if (warp == kMegaConsumerWarps + 1) {
        // ---------------- watcher: follows the chunks in order and counts the ones whose bytes have arrived ----------------
        if (lane == 0) {
            auto chunks_of = [](int items, int per_chunk) { return (items + per_chunk - 1) / per_chunk; };
            const unsigned per_layer = (w.in_group ? chunks_of(w.s1_n, p.s1_ipc) + chunks_of(p.rpb, p.s2_rpc) : 0) + chunks_of(w.h_n, p.s3a_ipc) + chunks_of(w.d_n, p.s3b_rpc);
            const unsigned total = (unsigned)a.n_steps * chunks_of(w.v_n, p.head_rpc) + (unsigned)(a.n_steps - 1) * L * per_layer;
            MegaCursor k;
            for (unsigned i = 0; i < total; i++) {
                unsigned spins = 0;
                bool gone = false;
                while (!mbar_try_wait(s.full + k.slot, k.phase)) {
                    if (*reinterpret_cast<volatile int*>(s.stop) || mega_spin_out(a, s, spins, 3)) { gone = true; break; }
                }
                if (gone) break;
                st_release_cta_shared(s.landed, i + 1);
                k.next((unsigned)p.n_slots);
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
    MegaCursor c;        // ring position, advances in lock step with the producer's
    unsigned n_chunk = 0;  // chunks consumed so far
    int pos = a.pos0;    // visible tokens
    uint32_t tok = 0;
    int emitted = 0;
    int par = 0;         // which half of s.partial the next chunk's sums go to
    constexpr int half = HD / 2;
    const int d = m.d_model;
    const float inv_d = 1.0f / (float)d;
    const float* fin_gain = a.norms + (size_t)(2 * L) * d;
    unsigned long long* my_qkv = a.qkv_words + (size_t)w.kvh * 2 * p.group_items;
    __half* xa_h = reinterpret_cast<__half*>(s.xa);

    // Stages values of the residual stream: raw copy, gained copy as the products' staged operand (fp16 hi/lo parts, or
    // int8 digits for the quantised types; `K` = length of the vector being staged), sum of squares.
    constexpr bool kQuant = WT == WT_Q8_0;  // int8 digit staging (Q4_0 widens its nibbles to fp16 and reads the fp16 staging)
    auto stage_x = [&](float* raw, int K, bool digits, int k, float v, float g, float& ss) {  // one element per lane, consecutive k
        raw[k] = v;
        if (kQuant && digits) qx_store_elem(s.xa, reinterpret_cast<float*>(s.xa + xa_bytes(K)), k, v * g);
        else xa_store(xa_h, k, v * g);
        ss = fmaf(v, v, ss);
    };
    auto stage_x2 = [&](float* raw, int K, bool digits, int k, float v0, float v1, float g0, float g1, float& ss) {  // a pair per lane
        raw[k] = v0; raw[k + 1] = v1;
        if (kQuant && digits) {
            qx_store_pair(s.xa, reinterpret_cast<float*>(s.xa + xa_bytes(K)), k, v0 * g0, v1 * g1);
        } else {
            xa_store(xa_h, k, v0 * g0);
            xa_store(xa_h, k + 1, v1 * g1);
        }
        ss = fmaf(v0, v0, fmaf(v1, v1, ss));
    };
    const bool head_digits = kQuant && p.wt_head != WT_F16;  // an fp16 head on quantised layers reads the fp16 staging
    // One chunk of a stage: acquire, all products, release, CTA barrier; returns where the sums are.
    int lg_parts = 0;    // log2 of the column ranges of the chunk whose sums are being read
    // A freed slot makes the producer request the chunk that is n_slots ahead at once: megabytes of reads over all
    // CTAs, which would travel through L2 together with the words of the exchange that follows the stage and delay
    // them by microseconds.  The last chunk of a stage is therefore handed back only after that exchange (the chunk it
    // makes room for is needed a whole layer later).
    MegaCursor pend_from;
    int n_pend = 0;
    auto release_pending = [&]() {
        if (n_pend) mega_release_deferred(a, s, pend_from, n_pend);
        n_pend = 0;
    };
    auto chunk_products = [&](int rows, int n_kb, const uint8_t* xa, bool defer, bool is_head = false) {
        const uint8_t* ch = mega_acquire(a, s, c, n_chunk++);
        FINE();
        float* partial = s.partial + par * kMegaChunkRows;
        par ^= 1;
        if (WT != WT_F16 && is_head && p.wt_head == WT_F16) lg_parts = mega_chunk_dots<WT_F16>(ch, rows, n_kb, xa, partial, warp, lane);  // an fp16 head on quantised layers
        else lg_parts = mega_chunk_dots<WT>(ch, rows, n_kb, xa, partial, warp, lane);
        FINE();
        if (defer) {
            if (n_pend == 0) pend_from = c;
            n_pend++;
            c.next((unsigned)p.n_slots);
        } else {
            mega_release(a, s, c);
        }
        consumer_sync();
        FINE();
        return partial;
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
                        for (int k = tid; k < d; k += kMegaConsumers) stage_x(s.xraw, d, true, k, __half2float(__ushort_as_half(emb_row[k])), __ldg(gain + k), ss);
                    } else {
                        mega_read_words(a, s, a.x_words, d, seq - 1, 5, gain, [&](int k, float v0, float v1, float g0, float g1) { stage_x2(s.xraw, d, true, k, v0, v1, g0, g1, ss); });
                    }
                    FINE();
                    release_pending();  // the W2 chunk of the previous layer
                    ss = mega_block_sum(ss, s.red);
                    inv = rsqrtf(ss * inv_d + m.eps);  // (a correctly rounded division and square root cost ~200 cycles here)
                    FINE();
                    stamp(step);
                    // q/k/v row pairs of this CTA, RoPE, words for the CTAs that share the KV head, KV-cache append.
                    // qkv_words is re-written one layer later, after x_words of this layer is complete, which needs every
                    // CTA's W2 rows, hence the whole activation vector, hence every group CTA past its S2 of this layer.
                    for (int i0 = 0; i0 < w.s1_n; i0 += p.s1_ipc) {
                        const int n_items = min(p.s1_ipc, w.s1_n - i0);
                        // A chunk holds at most 128 row pairs: one per thread.  Where the pair goes (matrix, RoPE entry,
                        // exchange words, cache rows) does not depend on the products: worked out before them, it is off
                        // the path between the last product and the words the other CTAs are waiting for.
                        int kind = 0, row0 = 0, row1 = 0, idx = 0;
                        float2 cs = make_float2(1.f, 0.f);
                        unsigned long long* dst = my_qkv;
                        __half* kv_row = nullptr;
                        if (tid < n_items) {
                            mega_s1_rows(m, p, w.kvh, w.s1_begin + i0 + tid, kind, row0, row1, idx);
                            if (kind < 2) cs = s.rope[idx];
                            dst = my_qkv + 2 * (w.s1_begin + i0 + tid);
                            if (kind > 0) kv_row = (kind == 1 ? a.kv.k : a.kv.v) + a.kv.offset(m, l, 0, w.kvh, pos) - w.kvh * HD;
                        }
                        float* sums = chunk_products(2 * n_items, d >> 5, s.xa, i0 + p.s1_ipc >= w.s1_n);
                        if (tid < n_items) {
                            float v0 = mega_take_sum(sums, lg_parts, 2 * tid) * inv;
                            float v1 = mega_take_sum(sums, lg_parts, 2 * tid + 1) * inv;
                            const float r0 = v0 * cs.x - v1 * cs.y, r1 = v0 * cs.y + v1 * cs.x;  // (cos, sin) = (1, 0) for a value pair
                            st_word(dst, tagged(r0, seq));
                            st_word(dst + 1, tagged(r1, seq));
                            if (kind > 0) {
                                kv_row[row0] = __float2half_rn(r0);
                                kv_row[row1] = __float2half_rn(r1);
                            }
                        }
                    }
                    stamp(step);
                    // ---- S2: attention of this CTA's head (the cached K/V rows are requested before the query is awaited)
                    FINE();
                    mega_attention<HD, 1, WT == WT_Q8_0 ? 1 : 0>(a, s, w, m, a.kv, l, pos, [&]() {
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
                                    mega_backoff();
                                }
                            }
                            const float v0 = __uint_as_float((unsigned)v.x), v1 = __uint_as_float((unsigned)v.y);
                            if (section == 0) { s.qs[idx] = v0; s.qs[idx + half] = v1; }
                            else if (section == 1) { s.kn[idx] = __float2half_rn(v0); s.kn[idx + half] = __float2half_rn(v1); }
                            else { s.vn[2 * idx] = __float2half_rn(v0); s.vn[2 * idx + 1] = __float2half_rn(v1); }
                        }
                        release_pending();  // the q/k/v chunk
                        FINE();
                        consumer_sync();
                        FINE();
                        stamp(step);
                    });
                    stamp(step);
                    // ---- rows [blk*rpb, ...) of Wo restricted to this head's columns: every row's partial sum is one
                    // contribution to the counted sum of that row (head 0 also carries the residual)
                    for (int r0 = 0; r0 < p.rpb; r0 += p.s2_rpc) {
                        const int nr = min(p.s2_rpc, p.rpb - r0);
                        float* sums = chunk_products(nr, HD >> 5, reinterpret_cast<const uint8_t*>(s.ctx), r0 + p.s2_rpc >= p.rpb);
                        for (int r = tid; r < nr; r += kMegaConsumers) {
                            const int orow = w.blk * p.rpb + r0 + r;
                            float v = mega_take_sum(sums, lg_parts, r);
                            if (orow < d) {
                                if (w.head == 0) v += s.xraw[orow];
                                red_add_u64(a.mid_sums + orow, counted(v));
                            }
                        }
                    }
                    stamp(step);
                } else {
                    stamp(step); stamp(step); stamp(step); stamp(step); stamp(step);
                }
                // ---- S3: x_mid = residual + attention projection.  mid_sums receives the next layer's contributions
                // only after that layer's S1, which needs x_words of this layer complete, i.e. every CTA past this read.
                {
                    // The arg-max candidate words are used once per token; between two uses a whole model's worth of
                    // weights streams through L2.  Reading them once per layer keeps their lines resident, so that the
                    // token exchange does not start with a round trip to memory.
                    if (tid < p.n_cta) { unsigned long long keep; asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(keep) : "l"(a.cand_words + (size_t)tid * kMegaCandStride) : "memory"); }
                    const float* gain = a.norms + (size_t)(2 * l + 1) * d;
                    float ss = 0.f;
                    FINE();
                    mega_read_sums(a, s, a.mid_sums, d, m.n_head, 7, gain, [&](int k, float v0, float v1, float g0, float g1) { stage_x2(s.xmid, d, true, k, v0, v1, g0, g1, ss); });
                    FINE();
                    release_pending();  // the Wo chunk (CTAs outside the head groups: the W2 chunk of the previous layer)
                    ss = mega_block_sum(ss, s.red);
                    inv = rsqrtf(ss * inv_d + m.eps);  // (a correctly rounded division and square root cost ~200 cycles here)
                }
                stamp(step);
                // (gate, up) row pairs of this CTA's hidden units, SiLU(gate) * up.  act_words is re-written one layer later,
                // after mid_sums of that layer is complete, which needs every group CTA past x_words of this layer, i.e.
                // every CTA past its W2 rows and so past this activation vector.
                for (int j0 = 0; j0 < w.h_n; j0 += p.s3a_ipc) {
                    const int n_items = min(p.s3a_ipc, w.h_n - j0);
                    // (one item per thread; its word's address is known before the products)
                    unsigned long long* const dst = a.act_words + (p.act_wpc ? (size_t)blockIdx.x * p.act_wpc : (size_t)w.h_begin) + j0 + tid;
                    float* sums = chunk_products(2 * n_items, d >> 5, s.xa, j0 + p.s3a_ipc >= w.h_n);
                    if (tid < n_items) {
                        const float g = mega_take_sum(sums, lg_parts, 2 * tid) * inv;
                        const float u = mega_take_sum(sums, lg_parts, 2 * tid + 1) * inv;
                        // silu(g) = g * sigmoid(g) = 0.5 g (1 + tanh(g / 2))
                        st_word(dst, tagged(__fdividef(g, 1.0f + __expf(-g)) * u, seq));
                    }
                }
                stamp(step);
                // ---- the whole activation vector, then this CTA's rows of W2 (+ residual) = the next layer's x
                FINE();
                if (p.act_wpc) {  // (cache lines per CTA: fp16 models only, see the plan)
                    mega_read_lines(a, s, a.act_words, p.act_wpc, s.hbeg, m.hidden, p.n_cta, (p.hpc_max + 1) >> 1, seq, 8, nullptr, [&](int k, float v, float) { xa_store(xa_h, k, v); });
                } else {
                    mega_read_words(a, s, a.act_words, m.hidden, seq, 8, nullptr, [&](int k, float v0, float v1, float, float) {
                        if (kQuant) {
                            qx_store_pair(s.xa, reinterpret_cast<float*>(s.xa + xa_bytes(m.hidden)), k, v0, v1);
                        } else {
                            xa_store(xa_h, k, v0);
                            xa_store(xa_h, k + 1, v1);
                        }
                    });
                }
                FINE();
                release_pending();  // the gate/up chunk
                consumer_sync();
                FINE();
                stamp(step);
                for (int r0 = 0; r0 < w.d_n; r0 += p.s3b_rpc) {
                    const int nr = min(p.s3b_rpc, w.d_n - r0);
                    // (at most 256 rows per chunk: one per thread; residual and address are fetched before the products)
                    const float res = tid < nr ? s.xmid[w.d_begin + r0 + tid] : 0.f;
                    unsigned long long* const dst = a.x_words + w.d_begin + r0 + tid;
                    float* sums = chunk_products(nr, m.hidden >> 5, s.xa, r0 + p.s3b_rpc >= w.d_n);
                    if (tid < nr) st_word(dst, tagged(mega_take_sum(sums, lg_parts, tid) + res, seq));
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
        // Everything this CTA wrote with plain stores during the step (KV-cache rows; the CTA barriers since then order
        // them before this thread) is made visible before the candidate words that thread 0 publishes at the end of the
        // head.  Issued here, the fence overlaps the wait for the last layer's output.
        if (tid == 0) __threadfence();
        {
            float ss = 0.f;
            if (step == 0) {
                for (int k = tid; k < d; k += kMegaConsumers) stage_x(s.xraw, d, head_digits, k, __ldcg(a.hidden_io + k), __ldg(fin_gain + k), ss);
            } else {
                mega_read_words(a, s, a.x_words, d, (unsigned)(step * L), 9, fin_gain, [&](int k, float v0, float v1, float g0, float g1) { stage_x2(s.xraw, d, head_digits, k, v0, v1, g0, g1, ss); });
            }
            release_pending();  // the W2 chunk of the last layer
            consumer_sync();  // the RMSNorm scale is positive: the arg-max does not need it
        }
        stamp(step);
        float best_v = -INFINITY;
        int best_i = 0x7fffffff;
        for (int r0 = 0; r0 < w.v_n; r0 += p.head_rpc) {
            const int nrows = min(p.head_rpc, w.v_n - r0);
            FINE();
            float* sums = chunk_products(nrows, d >> 5, s.xa, r0 + 2 * p.head_rpc >= w.v_n, true);
            // thread r keeps the best of rows r0 + r over the chunks (ascending rows: '>' keeps the first maximum)
            if (tid < nrows) {
                const float v = mega_take_sum(sums, lg_parts, tid);
                if (v > best_v) { best_v = v; best_i = w.v_begin + r0 + tid; }
            }
        }
#ifdef MEGA_FINE_TRACE
        if (a.trace && tid == 0 && step == a.n_steps - 1) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); a.trace[600 + blockIdx.x] = (long long)t; }
#endif
        // CTA-wide best (larger value first, then smaller index), published as one word per CTA:
        // [ordered logit bits : 32][0xffffff - index : 24][tag : 8].  The tag is the same in every word of a step, so the
        // largest word is the best candidate; 148 consecutive words are ten cache lines for every reader.
        const unsigned long long tag8 = (unsigned long long)(step % 255 + 1);
        {
            unsigned long long k = best_i != 0x7fffffff ? ((unsigned long long)ordered_bits(best_v) << 32) | ((unsigned long long)(0xffffffu - (unsigned)best_i) << 8) : 0ull;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) k = max(k, __shfl_xor_sync(0xffffffffu, k, off));
            if (lane == 0) s.key[warp] = k;
        }
        consumer_sync();
        if (tid == 0) {
            unsigned long long k = 0ull;
#pragma unroll
            for (int x = 0; x < kMegaConsumerWarps; x++) k = max(k, s.key[x]);
            st_word(a.cand_words + (size_t)blockIdx.x * kMegaCandStride, k | tag8);
        }
        stamp(step);
        {
            unsigned long long k = 0ull;
            if (tid < p.n_cta) {
                unsigned spins = 0;
                if (!mega_aborting(s)) {
                    while (true) {
                        asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(k) : "l"(a.cand_words + (size_t)tid * kMegaCandStride) : "memory");
                        if ((k & 0xffull) == tag8) break;
                        if (mega_spin_out(a, s, spins, 10)) break;
                        mega_backoff();
                    }
                }
                // a reader orders its later loads (the KV-cache rows other CTAs appended during this step) after the
                // candidate words it saw; the writers' side of the pair is the fence at the start of the head
                __threadfence();
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
            tok = min(0xffffffu - (uint32_t)((k >> 8) & 0xffffffull), (uint32_t)(m.vocab - 1));  // in range even if every logit was NaN
        }
        release_pending();  // the last head chunks
        stamp(step);
#ifdef MEGA_FINE_TRACE
        if (a.trace && tid == 0 && step == a.n_steps - 1) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); a.trace[800 + blockIdx.x] = (long long)t; }
#endif
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

// One source matrix: row-major [rows][cols] fp16, or the split GGUF storage of the engine (Q8_0: int8 [rows][cols] +
// fp16 scales [rows][cols/32]; Q4_0: 16-byte nibble groups [rows][cols/32] + scales).
struct PackMatrix {
    const void* data;
    const __half* scales;
};
struct PackSources {
    const PackMatrix* wq;  // per-layer device arrays
    const PackMatrix* wk;
    const PackMatrix* wv;
    const PackMatrix* wo;
    const PackMatrix* w1;
    const PackMatrix* w2;
    const PackMatrix* w3;
    PackMatrix lm_head;
};

// Where a row starts: matrix `m` of `cols` columns, row `row`, first column `col0` (a multiple of 32).
struct PackRow {
    const uint8_t* data;     // null: a row of zeros
    const __half* scales;
};
__device__ __forceinline__ PackRow pack_row(int wt, const PackMatrix& m, int cols, size_t row, int col0) {
    PackRow r;
    const uint8_t* d = static_cast<const uint8_t*>(m.data);
    if (wt == WT_Q8_0) r.data = d + row * cols + col0;
    else if (wt == WT_Q4_0) r.data = d + (row * (cols / 32) + col0 / 32) * 16;
    else r.data = d + (row * cols + col0) * 2;
    r.scales = m.scales ? m.scales + row * (cols / 32) + col0 / 32 : nullptr;
    return r;
}

// Writes `nr` rows of K columns each in the order the products read them: for every block of 32 columns, for every row,
// four pieces.  fp16: piece t holds columns {2t, 2t+1, 2t+8, 2t+9, 16+2t, 17+2t, 24+2t, 25+2t} of the block (the A registers
// of two m16n8k16 steps for the lanes with that t).  Q8_0: the int8 of columns 4t..4t+3 and 16+4t..16+4t+3 (the A registers
// of one m16n8k32 step); Q4_0: bytes 2t, 2t+1, 2t+8, 2t+9 of the GGUF block, whose low and high nibbles are the fp16 piece's columns.
// The quantised types put the scales [block][row] behind the data.  row_of(r) names the row's source.
template <class RowOf>
__device__ __forceinline__ void pack_tiled(int wt, uint8_t* dst, int nr, int K, RowOf row_of) {
    const int n_kb = K >> 5;
    const int piece = wt == WT_Q8_0 ? 8 : wt == WT_Q4_0 ? 4 : 16;
    for (int i = threadIdx.x; i < n_kb * nr * 4; i += blockDim.x) {
        const int t = i & 3, q = i >> 2;
        const int kb = q / nr, r = q - kb * nr;
        const PackRow src = row_of(r);
        uint8_t* out = dst + ((size_t)q * 4 + t) * piece;
        if (wt == WT_F16) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (src.data) {
                const uint32_t* s32 = reinterpret_cast<const uint32_t*>(src.data + (size_t)kb * 64);
                v = make_uint4(s32[t], s32[t + 4], s32[t + 8], s32[t + 12]);
            }
            *reinterpret_cast<uint4*>(out) = v;
        } else if (wt == WT_Q8_0) {
            uint2 v = make_uint2(0, 0);
            if (src.data) {
                const uint32_t* s32 = reinterpret_cast<const uint32_t*>(src.data + (size_t)kb * 32);  // four columns each
                v.x = s32[t];      // columns 4t .. 4t+3
                v.y = s32[4 + t];  // columns 16+4t .. 16+4t+3
            }
            *reinterpret_cast<uint2*>(out) = v;
        } else {
            uint32_t v = 0x88888888u;  // nibble 8 = value 0
            if (src.data) {
                const uint16_t* s16 = reinterpret_cast<const uint16_t*>(src.data + (size_t)kb * 16);  // pairs of bytes
                v = (uint32_t)s16[t] | ((uint32_t)s16[t + 4] << 16);
            }
            *reinterpret_cast<uint32_t*>(out) = v;
        }
    }
    if (wt != WT_F16) {
        __half* sc = reinterpret_cast<__half*>(dst + (size_t)n_kb * nr * 4 * piece);
        for (int i = threadIdx.x; i < n_kb * nr; i += blockDim.x) {
            const int kb = i / nr, r = i - kb * nr;
            const PackRow src = row_of(r);
            sc[i] = src.data ? src.scales[kb] : __float2half(0.f);
        }
    }
}

// One CTA builds the blob of one CTA of the decode kernel: per layer [S1 | S2 | S3 gate/up | S3 W2], then the head;
// every stage is a sequence of chunks (the units the ring carries), each in the tiled order above.
__global__ void k_build_pack(PackSources src, MegaPlan p, ModelDims m, uint8_t* pack) {
    const int cta = blockIdx.x;
    uint8_t* blob = pack + (size_t)cta * p.cta_bytes;
    const int d = m.d_model, hd = m.head_dim;
    const int wt = p.wt_layer;
    const MegaShare w = mega_share(m, p, cta);
    for (int l = 0; l < m.n_layer; l++) {
        uint8_t* base = blob + (size_t)l * p.layer_bytes;
        // S1: pairs of rows in RoPE order
        if (w.in_group)
            for (int i0 = 0; i0 < w.s1_n; i0 += p.s1_ipc) {
                const int n = min(p.s1_ipc, w.s1_n - i0);
                pack_tiled(wt, base + (size_t)i0 * 2 * p.row_bytes, 2 * n, d, [&](int r) {
                    int kind, row0, row1, idx;
                    mega_s1_rows(m, p, w.kvh, w.s1_begin + i0 + (r >> 1), kind, row0, row1, idx);
                    const PackMatrix& W = kind == 0 ? src.wq[l] : kind == 1 ? src.wk[l] : src.wv[l];
                    return pack_row(wt, W, d, (size_t)((r & 1) ? row1 : row0), 0);
                });
            }
        base += p.s1_bytes;
        // S2: rows [blk*rpb, +rpb) of Wo, columns of one head
        if (w.in_group)
            for (int r0 = 0; r0 < p.rpb; r0 += p.s2_rpc) {
                const int n = min(p.s2_rpc, p.rpb - r0);
                pack_tiled(wt, base + (size_t)r0 * p.wo_row_bytes, n, hd, [&](int r) {
                    const int orow = w.blk * p.rpb + r0 + r;
                    return orow < d ? pack_row(wt, src.wo[l], m.q_dim, (size_t)orow, w.head * hd) : PackRow{nullptr, nullptr};
                });
            }
        base += p.s2_bytes;
        // S3: (gate_j, up_j) row pairs
        for (int j0 = 0; j0 < w.h_n; j0 += p.s3a_ipc) {
            const int n = min(p.s3a_ipc, w.h_n - j0);
            pack_tiled(wt, base + (size_t)j0 * 2 * p.row_bytes, 2 * n, d, [&](int r) {
                return pack_row(wt, (r & 1) ? src.w3[l] : src.w1[l], d, (size_t)(w.h_begin + j0 + (r >> 1)), 0);
            });
        }
        base += p.s3a_bytes;
        // S3: this CTA's rows of W2
        for (int r0 = 0; r0 < w.d_n; r0 += p.s3b_rpc) {
            const int n = min(p.s3b_rpc, w.d_n - r0);
            pack_tiled(wt, base + (size_t)r0 * p.down_row_bytes, n, m.hidden, [&](int r) { return pack_row(wt, src.w2[l], m.hidden, (size_t)(w.d_begin + r0 + r), 0); });
        }
    }
    uint8_t* hb = blob + (size_t)m.n_layer * p.layer_bytes;
    for (int r0 = 0; r0 < w.v_n; r0 += p.head_rpc) {
        const int n = min(p.head_rpc, w.v_n - r0);
        pack_tiled(p.wt_head, hb + (size_t)r0 * p.head_row_bytes, n, d, [&](int r) { return pack_row(p.wt_head, src.lm_head, d, (size_t)(w.v_begin + r0 + r), 0); });
    }
}

}  // namespace esp
