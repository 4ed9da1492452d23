// Exact two-token generation as ONE cooperative launch: a draft model proposes the token after `current`, the target
// model verifies `current` and the proposal in a single pass over its weights, and the commit rule of
// Sources/Espresso/GenerationHarness.swift:1281-1344 (commit two tokens when the proposal equals the target's own
// choice, otherwise one) runs inside the kernel, replicated in every CTA.  No host round trip separates the passes.
//
// The kernel is the persistent decode kernel (mega_kernel.cuh) widened to two token positions per pass:
//   * the products run on mma.sync with the weights as the A operand; the staged activations of the second position
//     occupy two more of the eight B columns the instruction computes anyway, so the weights are read from the ring
//     once for both positions and the per-position sums are bit-identical to the single-position kernel's;
//   * every exchange (tagged words, counted sums, arg-max candidates) carries one value per position;
//   * attention runs once per query; the second query also sees the first new position, whose key and value sit in
//     shared memory beside its own.
// Draft and target must have the same widths (d_model, heads, hidden, vocabulary, fp16 storage); they differ in depth
// only, so one plan and one ring serve both and a pass is a fixed sequence of weight chunks: draft layers, draft head,
// target layers, target head.  The draft always processes the two newest tokens (`prev`, `current`): when the
// previous pass committed one token the first of them was processed before, and writing the same key and value to the
// same cache row again is harmless; this keeps every pass the same shape.
#pragma once

#include "mega_kernel.cuh"

namespace esp {

constexpr int kSpecNP = 2;  // token positions per pass

struct SpecModel {
    ModelDims m;            // this model's dimensions (the KV-cache strides depend on its max_seq and sequence slots)
    const uint8_t* pack;    // [n_cta][cta_bytes] packed weights (see k_build_pack)
    long long cta_bytes;
    const float* norms2;    // [2 * n_layer + 1][2][d_model]: every gain vector twice (one copy per position)
    const uint16_t* tok_emb;
    KvLayout kv;
};

struct SpecArgs {
    MegaArgs base;          // target dimensions, the shared plan (shared-memory layout for two positions), rope table,
                            // exchange arena (every array holds two positions), error word, spin limit
    SpecModel model[2];     // 0 = draft, 1 = target
    uint32_t* out;          // emitted tokens; out[0 .. gen0) were written by the host
    int* result;            // [8]: tokens emitted in total, passes, committed, accepted, stopped on EOS, visible tokens of the
                            // target, visible tokens of the draft, row of the last target pass that produced the pending token
    float* hidden_out;      // [d_model] hidden state that produced the pending token (target), or null
    uint32_t prev, current; // the two newest tokens; `current` is emitted but not yet fed
    int pos;                // position of `current`
    int gen0;               // tokens emitted so far
    int eff;                // emission limit
    int max_seq;            // context limit (min over the two models)
    int eos_token;
    int verify_only;        // 1: a single target pass over (prev at pos, current at pos + 1), no draft, no loop: result[0..1] =
                            // the two greedy tokens, hidden_out[2][d_model] = both rows' hidden states (verify2 of the C ABI)
};

// Shared-memory layout for two positions (host side; p.n_slots and p.slot_bytes must be set).
inline void spec_layout(const ModelDims& m, MegaPlan& p) {
    constexpr int NP = kSpecNP;
    size_t o = (size_t)p.n_slots * p.slot_bytes;
    auto take = [&](size_t bytes) { size_t at = (o + 15) & ~(size_t)15; o = at + bytes; return (int)at; };
    p.off_bar = take(16 * (size_t)p.n_slots);
    p.off_prev = take(8 * (size_t)NP * m.d_model);
    p.off_key = take(8 * 32);
    p.off_xs = take((size_t)NP * xa_bytes(m.d_model > m.hidden ? m.d_model : m.hidden));
    p.off_xraw = take(sizeof(float) * (size_t)NP * m.d_model);
    p.off_xmid = take(sizeof(float) * (size_t)NP * m.d_model);
    p.off_rope = take(sizeof(float2) * (size_t)NP * (m.head_dim / 2));
    p.off_qs = take(sizeof(float) * (size_t)NP * m.head_dim);
    p.off_ctx = take((size_t)NP * xa_bytes(m.head_dim));
    p.off_kn = take(sizeof(__half) * (size_t)NP * m.head_dim);
    p.off_vn = take(sizeof(__half) * (size_t)NP * m.head_dim);
    p.off_part = take(sizeof(float) * (size_t)kMegaConsumerWarps * m.head_dim);
    p.off_red = take(sizeof(float) * 64);
    p.off_outv = take(sizeof(float) * 2 * NP * kMegaChunkRows);
    p.off_flags = take(16);
    p.off_share = take(sizeof(MegaShare));
    p.off_beg = take(sizeof(int) * ((size_t)p.n_cta + 1));
    p.smem_bytes = (int)((o + 127) & ~(size_t)127);
}

// Sums over the consumer threads of two floats each; every thread receives both.  One CTA barrier.
__device__ __forceinline__ float2 spec_block_sum2(float v0, float v1, float* red) {
    v0 = warp_sum(v0);
    v1 = warp_sum(v1);
    if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = v0; red[kMegaConsumerWarps + (threadIdx.x >> 5)] = v1; }
    consumer_sync();
    const float4* r4 = reinterpret_cast<const float4*>(red);
    float out[2];
#pragma unroll
    for (int q = 0; q < 2; q++) {
        const float4 a = r4[4 * q], b = r4[4 * q + 1], c = r4[4 * q + 2], e = r4[4 * q + 3];
        out[q] = (((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w))) + (((c.x + c.y) + (c.z + c.w)) + ((e.x + e.y) + (e.z + e.w)));
    }
    return make_float2(out[0], out[1]);
}

template <int HD>
__global__ void __launch_bounds__(kMegaThreads, 1) k_spec_mega(const SpecArgs sa) {
    constexpr int NP = kSpecNP;
    constexpr int WT = WT_F16;
    extern __shared__ __align__(128) uint8_t mega_smem[];
    const MegaArgs& a = sa.base;
    const MegaShared s = mega_carve(mega_smem, a);
    const MegaPlan& p = a.plan;
    const ModelDims& m = a.m;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        *s.share = mega_share(m, p, (int)blockIdx.x);
        for (int i = 0; i < p.n_slots; i++) { mbar_init(s.full + i, 1); mbar_init(s.empty + i, kMegaConsumerWarps); }
        *s.abort = 0;
        *s.stop = 0;
        *s.landed = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int k = tid; k < NP * m.d_model; k += kMegaThreads) s.prev[k] = 0ull;  // the counted sums are zero at launch
    for (int c = tid; c <= p.n_cta; c += kMegaThreads) {
        s.hbeg[c] = mega_share_begin(m.hidden, p.n_cta, c);
    }
    __syncthreads();
    const MegaShare& w = *s.share;
    const int max_passes = sa.verify_only ? 1 : sa.eff - sa.gen0;  // every pass emits at least one token
    const int first_model = sa.verify_only ? 1 : 0;
    auto chunks_of = [](int items, int per_chunk) { return (items + per_chunk - 1) / per_chunk; };

    if (warp == kMegaConsumerWarps) {
        // ---------------- producer: one thread streams this CTA's chunks in consumption order ----------------
        if (lane == 0) {
            MegaCursor c;
            unsigned issued = 0;
            const uint64_t policy = l2_evict_first_policy();
            auto stopped = [&]() { return mega_aborting(s) || *reinterpret_cast<volatile int*>(s.stop) != 0; };
            auto issue = [&](const uint8_t* src, int bytes) {
                if (stopped()) return;
                if (issued >= (unsigned)p.n_slots) mega_wait(a, s, s.empty + c.slot, c.phase ^ 1u, 4);  // the previous use of the slot was released
                if (stopped()) return;
                mbar_expect_tx(s.full + c.slot, (unsigned)bytes);
                bulk_copy_g2s(s.slots + (size_t)c.slot * p.slot_bytes, src, (unsigned)bytes, s.full + c.slot, policy);
                c.next((unsigned)p.n_slots);
                issued++;
            };
            auto issue_stage = [&](const uint8_t* src, int items, int per_chunk, int item_bytes) {
                for (int i0 = 0; i0 < items; i0 += per_chunk) issue(src + (long long)i0 * item_bytes, min(per_chunk, items - i0) * item_bytes);
            };
            for (int pass = 0; pass < max_passes && !stopped(); pass++) {
                for (int mi = first_model; mi < 2; mi++) {
                    // (fields picked one by one: a reference into the kernel parameters would force a local copy of all of them)
                    const uint8_t* blob = (mi ? sa.model[1].pack : sa.model[0].pack) + (size_t)blockIdx.x * (mi ? sa.model[1].cta_bytes : sa.model[0].cta_bytes);
                    const int n_layer = mi ? sa.model[1].m.n_layer : sa.model[0].m.n_layer;
                    for (int l = 0; l < n_layer; l++) {
                        const uint8_t* src = blob + (long long)l * p.layer_bytes;
                        if (w.in_group) issue_stage(src, w.s1_n, p.s1_ipc, 2 * p.row_bytes);
                        src += p.s1_bytes;
                        if (w.in_group) issue_stage(src, p.rpb, p.s2_rpc, p.wo_row_bytes);
                        src += p.s2_bytes;
                        issue_stage(src, w.h_n, p.s3a_ipc, 2 * p.row_bytes);
                        src += p.s3a_bytes;
                        issue_stage(src, w.d_n, p.s3b_rpc, p.down_row_bytes);
                    }
                    issue_stage(blob + (long long)n_layer * p.layer_bytes, w.v_n, p.head_rpc, p.head_row_bytes);
                }
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
            const unsigned per_layer = (w.in_group ? chunks_of(w.s1_n, p.s1_ipc) + chunks_of(p.rpb, p.s2_rpc) : 0) + chunks_of(w.h_n, p.s3a_ipc) + chunks_of(w.d_n, p.s3b_rpc);
            const unsigned per_pass = (unsigned)((first_model ? 0 : sa.model[0].m.n_layer) + sa.model[1].m.n_layer) * per_layer + (first_model ? 1u : 2u) * chunks_of(w.v_n, p.head_rpc);
            const unsigned total = (unsigned)max_passes * per_pass;
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
    MegaCursor c;          // ring position, advances in lock step with the producer's
    unsigned n_chunk = 0;  // chunks consumed so far
    int par = 0;           // which half of s.partial the next chunk's sums go to
    unsigned seq = 0;      // tag of everything the current layer publishes: layers are numbered through both models
    unsigned n_heads = 0;  // heads run so far (tag of the arg-max words)
    constexpr int half = HD / 2;
    const int d = m.d_model, hidden = m.hidden;
    const float inv_d = 1.0f / (float)d;
    const int gi2 = 2 * p.group_items;
    unsigned long long* my_qkv = a.qkv_words + (size_t)w.kvh * NP * gi2;
    __half* xa_h = reinterpret_cast<__half*>(s.xa);
    __half* ctx_h = reinterpret_cast<__half*>(s.ctx);
    (void)ctx_h;

    // Stages value v of element k (k in [0, NP * n): position k / n) of a residual stream: raw copy, gained copy as the
    // products' operand, sum of squares of its position.
    auto stage_x = [&](float* raw, int k, float v, float g, float (&ss)[NP]) {
        const int q = k >= d ? 1 : 0;
        raw[k] = v;
        xa_store<NP>(xa_h, k - q * d, v * g, q);
        if (q) ss[1] = fmaf(v, v, ss[1]); else ss[0] = fmaf(v, v, ss[0]);
    };
    auto stage_x2 = [&](float* raw, int k, float v0, float v1, float g0, float g1, float (&ss)[NP]) {  // k even: both in one position
        stage_x(raw, k, v0, g0, ss);
        stage_x(raw, k + 1, v1, g1, ss);
    };
    int lg_parts = 0;
    MegaCursor pend_from;
    int n_pend = 0;
    auto release_pending = [&]() {
        if (n_pend) mega_release_deferred(a, s, pend_from, n_pend);
        n_pend = 0;
    };
    // One chunk of a stage: acquire, all products of both positions, release (or defer it past the next exchange), CTA
    // barrier; returns where the sums are (position q at + q * kMegaChunkRows).
    auto chunk_products = [&](int rows, int n_kb, const uint8_t* xa, bool defer) {
        const uint8_t* ch = mega_acquire(a, s, c, n_chunk++);
        float* partial = s.partial + par * (NP * kMegaChunkRows);
        par ^= 1;
        lg_parts = mega_chunk_dots<WT, NP>(ch, rows, n_kb, xa, partial, warp, lane);
        if (defer) {
            if (n_pend == 0) pend_from = c;
            n_pend++;
            c.next((unsigned)p.n_slots);
        } else {
            mega_release(a, s, c);
        }
        consumer_sync();
        return partial;
    };

    // One pass of model M over the tokens (t0 at position pos0, t1 at pos0 + 1); every CTA learns both greedy tokens.
    // `row_sel` >= 0: CTA 0 keeps the hidden state of that row in sa.hidden_out.
    auto forward = [&](int mi, uint32_t t0, uint32_t t1, int pos0, uint32_t& o0, uint32_t& o1) {
        // the model's fields as scalars (a reference into the kernel parameters would force a local copy of all of them)
        const int L = mi ? sa.model[1].m.n_layer : sa.model[0].m.n_layer;
        const float* norms2 = mi ? sa.model[1].norms2 : sa.model[0].norms2;
        const uint16_t* tok_emb = mi ? sa.model[1].tok_emb : sa.model[0].tok_emb;
        KvLayout kv;
        kv.k = mi ? sa.model[1].kv.k : sa.model[0].kv.k;
        kv.v = mi ? sa.model[1].kv.v : sa.model[0].kv.v;
        ModelDims md = a.m;  // the widths are the target's; the cache strides are the model's own
        md.n_layer = L;
        md.n_seq = mi ? sa.model[1].m.n_seq : sa.model[0].m.n_seq;
        md.max_seq = mi ? sa.model[1].m.max_seq : sa.model[0].m.max_seq;
        if (tid < NP * half) {
            const int q = tid / half, i = tid - q * half;
            s.rope[tid] = a.rope[(size_t)min(pos0 + q, m.max_seq - 1) * half + i];  // published by the barrier of the first norm
        }
        for (int l = 0; l < L; l++) {
            ++seq;
            float inv[NP] = {0.f, 0.f};
            if (w.in_group) {
                // ---- S1: x of this layer for both positions, q/k/v row pairs, RoPE, words for the KV-head group, cache append
                const float* gain = norms2 + (size_t)(2 * l) * NP * d;
                float ss[NP] = {0.f, 0.f};
                if (l == 0) {
                    for (int k = tid; k < NP * d; k += kMegaConsumers) {
                        const int q = k >= d ? 1 : 0;
                        const uint16_t* emb_row = tok_emb + (size_t)(q ? t1 : t0) * d;
                        stage_x(s.xraw, k, __half2float(__ushort_as_half(emb_row[k - q * d])), __ldg(gain + k), ss);
                    }
                } else {
                    mega_read_words(a, s, a.x_words, NP * d, seq - 1, 5, gain, [&](int k, float v0, float v1, float g0, float g1) { stage_x2(s.xraw, k, v0, v1, g0, g1, ss); });
                }
                release_pending();  // the W2 chunk of the previous layer
                const float2 tot = spec_block_sum2(ss[0], ss[1], s.red);
                inv[0] = rsqrtf(tot.x * inv_d + m.eps);
                inv[1] = rsqrtf(tot.y * inv_d + m.eps);
                for (int i0 = 0; i0 < w.s1_n; i0 += p.s1_ipc) {
                    const int n_items = min(p.s1_ipc, w.s1_n - i0);
                    float* sums = chunk_products(2 * n_items, d >> 5, s.xa, i0 + p.s1_ipc >= w.s1_n);
                    for (int i = tid; i < NP * n_items; i += kMegaConsumers) {
                        const int q = i >= n_items ? 1 : 0, it = i - q * n_items;
                        int kind, row0, row1, idx;
                        mega_s1_rows(m, p, w.kvh, w.s1_begin + i0 + it, kind, row0, row1, idx);
                        const float* sq = sums + q * kMegaChunkRows;
                        float v0 = mega_take_sum(sq, lg_parts, 2 * it) * inv[q];
                        float v1 = mega_take_sum(sq, lg_parts, 2 * it + 1) * inv[q];
                        if (kind < 2) {
                            const float2 cs = s.rope[q * half + idx];
                            const float r0 = v0 * cs.x - v1 * cs.y, r1 = v0 * cs.y + v1 * cs.x;
                            v0 = r0; v1 = r1;
                        }
                        unsigned long long* dst = my_qkv + q * gi2 + 2 * (w.s1_begin + i0 + it);
                        st_word(dst, tagged(v0, seq));
                        st_word(dst + 1, tagged(v1, seq));
                        if (kind > 0 && pos0 + q < md.max_seq) {
                            __half* base = kind == 1 ? kv.k : kv.v;
                            const size_t off = kv.offset(md, l, 0, w.kvh, pos0 + q);
                            base[off + (row0 - w.kvh * HD)] = __float2half_rn(v0);
                            base[off + (row1 - w.kvh * HD)] = __float2half_rn(v1);
                        }
                    }
                }
                // ---- S2: attention of this CTA's head: the consumer warps split into one team per query (the cached rows are
                // requested before the queries are awaited)
                mega_attention<HD, NP, 0>(a, s, w, md, kv, l, pos0, [&]() {
                    if (tid < NP * 3 * half) {
                        const int q = tid / (3 * half), r = tid - q * 3 * half;
                        const int section = r / half, idx = r - section * half;
                        const int item = (section == 0 ? w.hq * half : section == 1 ? p.qpk * half : (p.qpk + 1) * half) + idx;
                        ulonglong2 v = make_ulonglong2(0, 0);
                        unsigned spins = 0;
                        if (!mega_aborting(s)) {
                            while (true) {
                                v = ld_words2(my_qkv + q * gi2 + 2 * item);
                                if ((unsigned)(v.x >> 32) == seq && (unsigned)(v.y >> 32) == seq) break;
                                if (mega_spin_out(a, s, spins, 6)) break;
                                mega_backoff();
                            }
                        }
                        const float v0 = __uint_as_float((unsigned)v.x), v1 = __uint_as_float((unsigned)v.y);
                        if (section == 0) { s.qs[q * HD + idx] = v0; s.qs[q * HD + idx + half] = v1; }
                        else if (section == 1) { s.kn[q * HD + idx] = __float2half_rn(v0); s.kn[q * HD + idx + half] = __float2half_rn(v1); }
                        else { s.vn[q * HD + 2 * idx] = __float2half_rn(v0); s.vn[q * HD + 2 * idx + 1] = __float2half_rn(v1); }
                    }
                    release_pending();  // the q/k/v chunk
                    consumer_sync();
                });
                // ---- rows [blk*rpb, ...) of Wo restricted to this head's columns: one contribution per position to the
                // counted sum of every row (head 0 also carries the residual)
                for (int r0 = 0; r0 < p.rpb; r0 += p.s2_rpc) {
                    const int nr = min(p.s2_rpc, p.rpb - r0);
                    float* sums = chunk_products(nr, HD >> 5, reinterpret_cast<const uint8_t*>(s.ctx), r0 + p.s2_rpc >= p.rpb);
                    for (int i = tid; i < NP * nr; i += kMegaConsumers) {
                        const int q = i >= nr ? 1 : 0, r = i - q * nr;
                        const int orow = w.blk * p.rpb + r0 + r;
                        float v = mega_take_sum(sums + q * kMegaChunkRows, lg_parts, r);
                        if (orow < d) {
                            if (w.head == 0) v += s.xraw[q * d + orow];
                            red_add_u64(a.mid_sums + q * d + orow, counted(v));
                        }
                    }
                }
            }
            // ---- S3: x_mid = residual + attention projection
            {
                if (tid < NP * p.n_cta) { unsigned long long keep; asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(keep) : "l"(a.cand_words + (size_t)tid * kMegaCandStride) : "memory"); }
                const float* gain = norms2 + (size_t)(2 * l + 1) * NP * d;
                float ss[NP] = {0.f, 0.f};
                mega_read_sums(a, s, a.mid_sums, NP * d, m.n_head, 7, gain, [&](int k, float v0, float v1, float g0, float g1) { stage_x2(s.xmid, k, v0, v1, g0, g1, ss); });
                release_pending();  // the Wo chunk (CTAs outside the head groups: the W2 chunk of the previous layer)
                const float2 tot = spec_block_sum2(ss[0], ss[1], s.red);
                inv[0] = rsqrtf(tot.x * inv_d + m.eps);
                inv[1] = rsqrtf(tot.y * inv_d + m.eps);
            }
            for (int j0 = 0; j0 < w.h_n; j0 += p.s3a_ipc) {
                const int n_items = min(p.s3a_ipc, w.h_n - j0);
                float* sums = chunk_products(2 * n_items, d >> 5, s.xa, j0 + p.s3a_ipc >= w.h_n);
                for (int i = tid; i < NP * n_items; i += kMegaConsumers) {
                    const int q = i >= n_items ? 1 : 0, j = i - q * n_items;
                    const float* sq = sums + q * kMegaChunkRows;
                    const float g = mega_take_sum(sq, lg_parts, 2 * j) * inv[q];
                    const float u = mega_take_sum(sq, lg_parts, 2 * j + 1) * inv[q];
                    st_word(a.act_words + (p.act_wpc ? (size_t)(q * p.n_cta + blockIdx.x) * p.act_wpc : (size_t)q * hidden + w.h_begin) + j0 + j, tagged(__fdividef(g, 1.0f + __expf(-g)) * u, seq));
                }
            }
            // ---- the whole activation vector of both positions, then this CTA's rows of W2 (+ residual) = the next layer's x
            auto stage_act = [&](int k, float v, float) {
                const int q = k >= hidden ? 1 : 0;
                xa_store<NP>(xa_h, k - q * hidden, v, q);
            };
            if (p.act_wpc) mega_read_lines(a, s, a.act_words, p.act_wpc, s.hbeg, hidden, NP * p.n_cta, (p.hpc_max + 1) >> 1, seq, 8, nullptr, stage_act);
            else mega_read_words(a, s, a.act_words, NP * hidden, seq, 8, nullptr, [&](int k, float v0, float v1, float, float) { stage_act(k, v0, 1.f); stage_act(k + 1, v1, 1.f); });
            release_pending();  // the gate/up chunk
            consumer_sync();
            for (int r0 = 0; r0 < w.d_n; r0 += p.s3b_rpc) {
                const int nr = min(p.s3b_rpc, w.d_n - r0);
                float* sums = chunk_products(nr, hidden >> 5, s.xa, r0 + p.s3b_rpc >= w.d_n);
                for (int i = tid; i < NP * nr; i += kMegaConsumers) {
                    const int q = i >= nr ? 1 : 0, r = i - q * nr;
                    const int row = w.d_begin + r0 + r;
                    st_word(a.x_words + (size_t)q * d + w.d_begin + r0 + r, tagged(mega_take_sum(sums + q * kMegaChunkRows, lg_parts, r) + s.xmid[q * d + row], seq));
                }
            }
        }
        // ---- LM head over this CTA's vocabulary rows for both positions, first-max argmax
        if (tid == 0) __threadfence();  // this CTA's cache rows of the pass, before the candidate words (see the decode kernel)
        {
            const float* gain = norms2 + (size_t)(2 * L) * NP * d;
            float ss[NP] = {0.f, 0.f};
            mega_read_words(a, s, a.x_words, NP * d, seq, 9, gain, [&](int k, float v0, float v1, float g0, float g1) { stage_x2(s.xraw, k, v0, v1, g0, g1, ss); });
            release_pending();  // the W2 chunk of the last layer
            consumer_sync();    // the RMSNorm scale is positive: the arg-max does not need it
        }
        // thread (q, r) = (tid / 256, tid % 256) keeps the best of rows r0 + r of position q over the chunks
        static_assert(kMegaConsumers == NP * kMegaChunkRows, "one thread per (position, chunk row)");
        const int hq = tid >> 8, hr = tid & (kMegaChunkRows - 1);
        float best_v = -INFINITY;
        int best_i = 0x7fffffff;
        for (int r0 = 0; r0 < w.v_n; r0 += p.head_rpc) {
            const int nrows = min(p.head_rpc, w.v_n - r0);
            float* sums = chunk_products(nrows, d >> 5, s.xa, r0 + p.head_rpc >= w.v_n);
            if (hr < nrows) {
                const float v = mega_take_sum(sums + hq * kMegaChunkRows, lg_parts, hr);
                if (v > best_v) { best_v = v; best_i = w.v_begin + r0 + hr; }
            }
        }
        const unsigned long long tag8 = (unsigned long long)(n_heads % 255 + 1);
        ++n_heads;
        {
            unsigned long long k = best_i != 0x7fffffff ? ((unsigned long long)ordered_bits(best_v) << 32) | ((unsigned long long)(0xffffffu - (unsigned)best_i) << 8) : 0ull;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) k = max(k, __shfl_xor_sync(0xffffffffu, k, off));
            if (lane == 0) s.key[warp] = k;  // warps 0..7 hold position 0, warps 8..15 position 1
        }
        consumer_sync();
        if (tid < NP) {
            unsigned long long k = 0ull;
#pragma unroll
            for (int x = 0; x < kMegaConsumerWarps / NP; x++) k = max(k, s.key[tid * (kMegaConsumerWarps / NP) + x]);
            st_word(a.cand_words + (size_t)(tid * p.n_cta + blockIdx.x) * kMegaCandStride, k | tag8);
        }
        {
            unsigned long long k = 0ull;
            if (tid < NP * p.n_cta) {
                unsigned spins = 0;
                if (!mega_aborting(s)) {
                    while (true) {
                        asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(k) : "l"(a.cand_words + (size_t)tid * kMegaCandStride) : "memory");
                        if ((k & 0xffull) == tag8) break;
                        if (mega_spin_out(a, s, spins, 10)) break;
                        mega_backoff();
                    }
                }
                __threadfence();  // later loads (cache rows other CTAs appended during this pass) after the words seen here
            }
            unsigned long long k0 = tid < p.n_cta ? k : 0ull, k1 = tid >= p.n_cta ? k : 0ull;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                k0 = max(k0, __shfl_xor_sync(0xffffffffu, k0, off));
                k1 = max(k1, __shfl_xor_sync(0xffffffffu, k1, off));
            }
            consumer_sync();  // s.key was read above
            if (lane == 0) { s.key[warp] = k0; s.key[kMegaConsumerWarps + warp] = k1; }
            if (tid == 0) s.red[63] = mega_aborting(s) ? 1.f : 0.f;  // one decision for the whole CTA
            consumer_sync();
            k0 = 0ull; k1 = 0ull;
#pragma unroll
            for (int x = 0; x < kMegaConsumerWarps; x++) { k0 = max(k0, s.key[x]); k1 = max(k1, s.key[kMegaConsumerWarps + x]); }
            o0 = min(0xffffffu - (uint32_t)((k0 >> 8) & 0xffffffull), (uint32_t)(m.vocab - 1));
            o1 = min(0xffffffu - (uint32_t)((k1 >> 8) & 0xffffffull), (uint32_t)(m.vocab - 1));
        }
        release_pending();  // the last head chunks
    };

    // ---- the generation loop (Sources/Espresso/GenerationHarness.swift:1281-1344; every CTA takes the same decisions)
    int gen = sa.gen0, total = sa.pos + 1;  // `current` sits at position sa.pos and has been emitted
    uint32_t prev = sa.prev, current = sa.current;
    int P = sa.pos;
    int passes = 0, committed = 0, accepted = 0, hit_eos = 0, row_sel = 0;
    int visible = sa.pos;  // tokens of the target's context that are committed
    int draft_visible = sa.pos;  // positions the draft has processed
    const bool writer = blockIdx.x == 0 && tid == 0;
    auto is_eos = [&](uint32_t t) { return sa.eos_token >= 0 && t == (uint32_t)sa.eos_token; };
    while (true) {
        const int remaining = min(sa.eff - gen, sa.max_seq - total);
        passes++;
        // verify-only launches (verify2 of the C ABI) take the target's pass alone: `prev` and `current` of the arguments
        // are then the two tokens to verify
        uint32_t proposed = sa.verify_only ? sa.current : 0u, next = 0, future = 0;
        if (sa.verify_only) current = sa.prev;
        bool gave_up = false;
        for (int mi = first_model; mi < 2 && !gave_up; mi++) {  // the only call site: the draft's pass, then the target's
            uint32_t o0, o1;
            forward(mi, mi ? current : prev, mi ? proposed : current, mi ? P : P - 1, o0, o1);
            if (mi == 0) { proposed = o1; draft_visible = P + 1; }
            else { next = o0; future = o1; }
            gave_up = s.red[63] != 0.f;
        }
        if (gave_up) break;
        if (sa.verify_only) {
            // both greedy tokens and both rows' hidden states; nothing is committed or emitted
            if (blockIdx.x == 0) {
                if (sa.hidden_out)
                    for (int k = tid; k < NP * d; k += kMegaConsumers) sa.hidden_out[k] = s.xraw[k];
                if (tid == 0) { sa.result[0] = (int)next; sa.result[1] = (int)future; }
            }
            if (tid == 0) *reinterpret_cast<volatile int*>(s.stop) = 1;
            return;
        }
        const bool two = remaining > 1 && total + 1 < sa.max_seq;
        if (two && proposed == next) {
            // both tokens are exact: the proposal is committed and emitted, the token after it becomes `current`
            if (writer) sa.out[gen] = next;
            gen++; total++;
            committed += 2; accepted += 1;
            visible = P + 2;
            row_sel = 1;
            if (is_eos(next)) { hit_eos = 1; break; }
            if (gen >= sa.eff || total >= sa.max_seq) break;
            prev = next; current = future; P += 2;
        } else {
            committed += 1;
            visible = P + 1;
            row_sel = 0;
            prev = current; current = next; P += 1;
        }
        if (writer) sa.out[gen] = current;
        gen++; total++;
        if (is_eos(current)) { hit_eos = 1; break; }
        if (gen >= sa.eff || total >= sa.max_seq) break;
    }
    if (tid == 0) *reinterpret_cast<volatile int*>(s.stop) = 1;
    if (blockIdx.x == 0) {
        if (sa.hidden_out)
            for (int k = tid; k < d; k += kMegaConsumers) sa.hidden_out[k] = s.xraw[row_sel * d + k];
        if (tid == 0) {
            sa.result[0] = gen;
            sa.result[1] = passes;
            sa.result[2] = committed;
            sa.result[3] = accepted;
            sa.result[4] = hit_eos;
            sa.result[5] = visible;
            sa.result[6] = draft_visible;
            sa.result[7] = row_sel;
        }
    }
}

}  // namespace esp
