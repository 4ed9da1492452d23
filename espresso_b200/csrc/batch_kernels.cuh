// Element-wise stages of the batched (tensor-core) decode path.  The matrix products run in k_gemm_tc; these
// kernels prepare its 16-bit operand rows and apply what the GEMV path fuses into its epilogues:
//   k_prep_rows    (embedding) -> RMSNorm / LayerNorm / none -> fp16 or bf16 operand rows
//   k_rope_append  half-split RoPE on q (in place) and k, KV-cache append of k and v
//   k_act_rows     SiLU(gate) * up  or  GELU(up)  -> 16-bit operand rows of the down projection
//   k_attention_rows  attention for many rows at once: one warp per (row, head), 16-bit context rows out
//   k_head_done    turns the packed per-row maxima of the LM-head GEMM into tokens (head_finalize)
// Every kernel here is launched with programmatic stream serialization: it lets its successor start early and
// waits for its predecessor before it touches global memory.
// Reference arithmetic: see decode_kernels.cuh.
#pragma once
#include "decode_kernels.cuh"

namespace esp {

__device__ __forceinline__ uint16_t to_16bit(float v, int bf16) {
    return bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
}

struct PrepArgs {
    ModelDims m;
    RowState rs;
    const float* src;         // [rows][K] fp32, or null when from_embedding
    float* hidden_out;        // from_embedding: the residual stream [rows][d_model] is initialised here
    const uint16_t* tok_emb;  // from_embedding
    const uint16_t* pos_emb;
    int emb_type;
    int from_embedding;
    int K;
    int norm;                 // NormKind
    const float* g;
    const float* b;
    uint16_t* dst;            // [rows][K] fp16/bf16
    int bf16;
    float* zero[4];           // optional fp32 rows to clear ([rows][zero_n[i]]): outputs that K-sliced products add into
    int zero_n[4];
};

// One CTA per row.  Rows of up to 8192 elements are held in registers (one global read, 16-byte accesses); longer
// rows are re-read for every pass.
__global__ void __launch_bounds__(kThreads) k_prep_rows(const PrepArgs p) {
    __shared__ float red[kRedFloats];
    const int r = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    // The row's state words and (when the row comes from the residual stream) its values are requested together;
    // the check for an inactive row comes after the requests, so the chain is one memory round trip shorter.
    const int row_active = p.rs.active[r];
    const int K = p.K;
    const float* src = p.src ? p.src + (size_t)r * K : nullptr;
    const uint16_t* te = nullptr;
    const uint16_t* pe = nullptr;
    if (p.from_embedding) {
        te = p.tok_emb + (size_t)p.rs.tok[r] * K;
        if (p.pos_emb) pe = p.pos_emb + (size_t)p.rs.pos[r] * K;
    }
    uint16_t* dst = p.dst + (size_t)r * K;
    constexpr int kVec = 8;  // float4 per thread held in registers
    const bool fast = K % 4 == 0 && K / 4 <= kVec * kThreads;
    float4 pre[kVec];
    if (fast && !p.from_embedding) {
#pragma unroll
        for (int i = 0; i < kVec; i++) {
            const int idx = threadIdx.x + i * kThreads;
            pre[i] = idx < K / 4 ? reinterpret_cast<const float4*>(src)[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    // (inactive rows are cleared too: a tensor-parallel sum reads every row of a partial buffer)
    for (int z = 0; z < 4; z++)
        if (p.zero[z]) {
            float4* zr = reinterpret_cast<float4*>(p.zero[z] + (size_t)r * p.zero_n[z]);  // row lengths are multiples of 16
            for (int k = threadIdx.x; k < p.zero_n[z] / 4; k += kThreads) zr[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    if (!row_active) return;
    if (fast) {
        const int nvec = K / 4;
        float4 v[kVec];
#pragma unroll
        for (int i = 0; i < kVec; i++) {
            const int idx = threadIdx.x + i * kThreads;
            v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (idx < nvec) {
                if (!p.from_embedding) {
                    v[i] = pre[i];
                } else {
                    const uint2 t = reinterpret_cast<const uint2*>(te)[idx];
                    v[i] = make_float4(emb_to_float((uint16_t)(t.x & 0xffffu), p.emb_type), emb_to_float((uint16_t)(t.x >> 16), p.emb_type),
                                       emb_to_float((uint16_t)(t.y & 0xffffu), p.emb_type), emb_to_float((uint16_t)(t.y >> 16), p.emb_type));
                    if (pe) {
                        const uint2 u = reinterpret_cast<const uint2*>(pe)[idx];
                        v[i].x += emb_to_float((uint16_t)(u.x & 0xffffu), p.emb_type);
                        v[i].y += emb_to_float((uint16_t)(u.x >> 16), p.emb_type);
                        v[i].z += emb_to_float((uint16_t)(u.y & 0xffffu), p.emb_type);
                        v[i].w += emb_to_float((uint16_t)(u.y >> 16), p.emb_type);
                    }
                    reinterpret_cast<float4*>(p.hidden_out + (size_t)r * K)[idx] = v[i];
                }
            }
        }
        float inv = 1.f, mean = 0.f;
        if (p.norm == NORM_RMS) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < kVec; i++) ss = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, ss))));
            ss = block_sum(ss, red);
            inv = 1.0f / sqrtf(ss / (float)K + p.m.eps);
        } else if (p.norm == NORM_LAYER) {
            float sm = 0.f;
#pragma unroll
            for (int i = 0; i < kVec; i++) sm += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            mean = block_sum(sm, red) / (float)K;
            float vs = 0.f;
#pragma unroll
            for (int i = 0; i < kVec; i++) {
                if (threadIdx.x + i * kThreads < nvec) {
                    const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
                    vs = fmaf(a, a, fmaf(b, b, fmaf(c, c, fmaf(d, d, vs))));
                }
            }
            vs = block_sum(vs, red);
            inv = 1.0f / sqrtf(vs / (float)K + p.m.eps);
        }
#pragma unroll
        for (int i = 0; i < kVec; i++) {
            const int idx = threadIdx.x + i * kThreads;
            if (idx >= nvec) continue;
            float4 o = v[i];
            if (p.norm == NORM_RMS) {
                const float4 g = reinterpret_cast<const float4*>(p.g)[idx];
                o = make_float4((o.x * inv) * g.x, (o.y * inv) * g.y, (o.z * inv) * g.z, (o.w * inv) * g.w);
            } else if (p.norm == NORM_LAYER) {
                const float4 g = reinterpret_cast<const float4*>(p.g)[idx];
                const float4 b = reinterpret_cast<const float4*>(p.b)[idx];
                o = make_float4((o.x - mean) * inv * g.x + b.x, (o.y - mean) * inv * g.y + b.y, (o.z - mean) * inv * g.z + b.z,
                                (o.w - mean) * inv * g.w + b.w);
            }
            reinterpret_cast<uint2*>(dst)[idx] =
                make_uint2((uint32_t)to_16bit(o.x, p.bf16) | ((uint32_t)to_16bit(o.y, p.bf16) << 16),
                           (uint32_t)to_16bit(o.z, p.bf16) | ((uint32_t)to_16bit(o.w, p.bf16) << 16));
        }
        return;
    }
    auto raw = [&](int k) {
        if (!p.from_embedding) return src[k];
        float v = emb_to_float(te[k], p.emb_type);
        if (pe) v += emb_to_float(pe[k], p.emb_type);
        return v;
    };
    float inv = 1.f, mean = 0.f;
    if (p.norm == NORM_RMS) {
        float ss = 0.f;
        for (int k = threadIdx.x; k < K; k += kThreads) { const float v = raw(k); ss = fmaf(v, v, ss); }
        ss = block_sum(ss, red);
        inv = 1.0f / sqrtf(ss / (float)K + p.m.eps);
    } else if (p.norm == NORM_LAYER) {
        float s = 0.f;
        for (int k = threadIdx.x; k < K; k += kThreads) s += raw(k);
        mean = block_sum(s, red) / (float)K;
        float vs = 0.f;
        for (int k = threadIdx.x; k < K; k += kThreads) { const float c = raw(k) - mean; vs = fmaf(c, c, vs); }
        vs = block_sum(vs, red);
        inv = 1.0f / sqrtf(vs / (float)K + p.m.eps);
    }
    for (int k = threadIdx.x; k < K; k += kThreads) {
        const float x = raw(k);
        if (p.from_embedding) p.hidden_out[(size_t)r * K + k] = x;
        float v = x;
        if (p.norm == NORM_RMS) v = (x * inv) * p.g[k];
        else if (p.norm == NORM_LAYER) v = (x - mean) * inv * p.g[k] + p.b[k];
        dst[k] = to_16bit(v, p.bf16);
    }
}

struct RopeArgs {
    ModelDims m;
    RowState rs;
    KvLayout kv;
    float* q;            // [rows][q_dim], rotated in place
    const float* k_raw;  // [rows][kv_dim]
    const float* v_raw;  // [rows][kv_dim]
    const float2* rope;  // [max_seq][head_dim/2] (cos, sin); null for GPT-2
    int layer;
    float* debug;        // optional capture of row 0 (q, k, v as stored)
    const float* q_norm; // [head_dim] per-head RMSNorm weights applied to q and k before RoPE (Qwen3), or null
    const float* k_norm;
};

// grid = (rows, chunks): one thread per rotation pair of q, per rotation pair of k, or per pair of v elements.
// The head_dim / 2 threads of a head are neighbours inside one CTA (256 is a multiple of 16, 32 and 64), which is what
// the optional per-head norm (applyPerHeadRMSNormInPlace, Sources/RealModelInference/RealModelInferenceEngine.swift:
// 6648-6672: v * rsqrt(mean(v^2) + eps) * w, before RoPE) uses for its sum of squares.
__global__ void __launch_bounds__(kThreads) k_rope_append(const RopeArgs p) {
    __shared__ float head_ss[kThreads / 32];
    const int r = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const int row_active = p.rs.active[r], pos = p.rs.pos[r], seq = p.rs.seq[r];  // one round trip for the three
    if (!row_active) return;
    const ModelDims& m = p.m;
    const int half = m.head_dim / 2;
    const int q_pairs = m.q_dim / 2, k_pairs = m.kv_dim / 2;
    const int i = blockIdx.y * kThreads + threadIdx.x;
    const bool rot = i < q_pairs + k_pairs;
    const bool is_q = i < q_pairs;
    const int local = is_q ? i : i - q_pairs;
    const int head = rot ? local / half : 0, idx = rot ? local - head * half : 0;
    const int i0 = head * m.head_dim + idx, i1 = i0 + half;
    float* q = p.q + (size_t)r * m.q_dim;
    const float* kr = p.k_raw + (size_t)r * m.kv_dim;
    float v0 = 0.f, v1 = 0.f;
    if (rot) { v0 = is_q ? q[i0] : kr[i0]; v1 = is_q ? q[i1] : kr[i1]; }
    if (p.q_norm) {  // uniform over the grid: every thread of the CTA takes part in the barrier
        float ss = v0 * v0 + v1 * v1;
        for (int o = (half < 32 ? half : 32) >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (half == 64) {  // a head spans two warps
            if ((threadIdx.x & 31) == 0) head_ss[threadIdx.x >> 5] = ss;
            __syncthreads();
            ss = head_ss[(threadIdx.x >> 5) & ~1] + head_ss[(threadIdx.x >> 5) | 1];
        }
        if (rot) {
            const float inv = 1.0f / sqrtf(ss / (float)m.head_dim + m.eps);
            const float* w = is_q ? p.q_norm : p.k_norm;
            v0 *= inv * w[idx];
            v1 *= inv * w[idx + half];
        }
    }
    if (i >= q_pairs + 2 * k_pairs) return;
    if (rot) {
        if (p.rope) {
            const float2 cs = p.rope[(size_t)pos * half + idx];
            const float r0 = v0 * cs.x - v1 * cs.y, r1 = v0 * cs.y + v1 * cs.x;
            v0 = r0; v1 = r1;
        }
        if (is_q) {
            q[i0] = v0; q[i1] = v1;
            if (p.debug && r == 0) { p.debug[i0] = v0; p.debug[i1] = v1; }
        } else {
            const size_t off = p.kv.offset(m, p.layer, seq, head, pos);
            p.kv.k[off + idx] = __float2half_rn(v0);
            p.kv.k[off + idx + half] = __float2half_rn(v1);
            if (p.debug && r == 0) {
                p.debug[m.q_dim + i0] = __half2float(__float2half_rn(v0));
                p.debug[m.q_dim + i1] = __half2float(__float2half_rn(v1));
            }
        }
    } else {
        const int e = 2 * (i - q_pairs - k_pairs);  // head_dim is even: both elements belong to one head
        const int head = e / m.head_dim, idx = e - head * m.head_dim;
        const float2 vv = *reinterpret_cast<const float2*>(p.v_raw + (size_t)r * m.kv_dim + e);
        const __half2 hv = __floats2half2_rn(vv.x, vv.y);
        *reinterpret_cast<__half2*>(p.kv.v + p.kv.offset(m, p.layer, seq, head, pos) + idx) = hv;
        if (p.debug && r == 0) {
            p.debug[m.q_dim + m.kv_dim + e] = __low2float(hv);
            p.debug[m.q_dim + m.kv_dim + e + 1] = __high2float(hv);
        }
    }
}

struct ActArgs {
    RowState rs;
    const float* gate;  // [rows][h] (GELU: the biased up projection)
    const float* up;    // [rows][h] or null for GELU
    uint16_t* dst;      // [rows][h]
    int h;
    int bf16;
    float* debug;       // optional fp32 capture of row 0
};

__global__ void __launch_bounds__(kThreads) k_act_rows(const ActArgs p) {
    const int r = blockIdx.y;
    pdl_launch_dependents();
    pdl_wait();
    if (!p.rs.active[r]) return;
    const int i = blockIdx.x * kThreads + threadIdx.x;
    if (i >= p.h) return;
    const float g = p.gate[(size_t)r * p.h + i];
    const float v = p.up ? silu_f(g) * p.up[(size_t)r * p.h + i] : gelu_f(g);
    p.dst[(size_t)r * p.h + i] = to_16bit(v, p.bf16);
    if (p.debug && r == 0) p.debug[i] = v;
}

__global__ void k_head_done(const GemvArgs p) {
    pdl_launch_dependents();
    pdl_wait();
    head_finalize(p);
}

struct AttRowsArgs {
    ModelDims m;
    RowState rs;
    KvLayout kv;
    const float* q;    // [rows][q_dim] fp32, RoPE applied
    uint16_t* ctx16;   // [rows][q_dim] fp16/bf16: operand rows of the output projection
    int bf16;
    int layer;
    int rows;
    float* debug;      // optional fp32 capture of row 0's context (already offset), or null
};

constexpr int kAttRowsWarps = 4;

__device__ __forceinline__ void halves16_to_float(const uint4& a, const uint4& b, float (&f)[16]) {
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

// Attention of one new token per row against its sequence's cache, for many rows: one warp per (row, head).
// HD / 16 lanes share a cache position (16 channels each), so a warp covers 32 / (HD / 16) positions per pass and
// every load instruction reads whole 128-byte (or longer) cache rows.  Each lane group keeps its own running
// (max, sum, context) over the positions it visits; the groups are merged once at the end.  Softmax in fp32 as in
// decodeContext (Sources/RealModelInference/RealModelInferenceEngine.swift:6560-6640), evaluated online.
// SPLIT = 2: two warps share one (row, head) and take alternate blocks of positions (twice the cache bytes in
// flight when there are few (row, head) pairs and long contexts); the second warp hands its (max, sum, context) to the
// first through shared memory.  Needs n_head % 4 == 0 so that a CTA (4 heads x SPLIT warps) never straddles two rows.
template <int HD, int SPLIT>
__global__ void __launch_bounds__(kAttRowsWarps * 32 * SPLIT) k_attention_rows(const AttRowsArgs p) {
    constexpr int LPP = HD / 16;   // lanes per position
    constexpr int G = 32 / LPP;    // positions per pass of one warp
    __shared__ float s_merge[SPLIT > 1 ? kAttRowsWarps * LPP * 18 : 1];
    pdl_launch_dependents();
    pdl_wait();
    const ModelDims& m = p.m;
    const int lane = threadIdx.x & 31;
    const int warp_in_cta = threadIdx.x >> 5;
    const int split = SPLIT > 1 ? warp_in_cta / kAttRowsWarps : 0;
    const int w = blockIdx.x * kAttRowsWarps + (SPLIT > 1 ? warp_in_cta % kAttRowsWarps : warp_in_cta);
    if (w >= p.rows * m.n_head) return;
    const int r = w / m.n_head, head = w - r * m.n_head;
    // the three row-state words are requested together (one memory round trip, not three)
    const int row_active = p.rs.active[r], row_pos = p.rs.pos[r], row_seq = p.rs.seq[r];
    const int sub = lane % LPP, slot = lane / LPP;
    float q[16];  // this lane's 16 channels of the query, requested with the row state
    {
        const float4* qp = reinterpret_cast<const float4*>(p.q + (size_t)r * m.q_dim + (size_t)head * HD + sub * 16);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 t = qp[i];
            q[4 * i] = t.x; q[4 * i + 1] = t.y; q[4 * i + 2] = t.z; q[4 * i + 3] = t.w;
        }
    }
    if (!row_active) return;
    const int visible = row_pos + 1;
    const int kvh = head / (m.n_head / m.n_kv_head);
    const size_t base = p.kv.offset(m, p.layer, row_seq, kvh, 0) + (size_t)sub * 16;
    const __half* K = p.kv.k + base;
    const __half* V = p.kv.v + base;
    const float scale = 1.0f / sqrtf((float)HD);
    float mx = -INFINITY, sum = 0.f, acc[16];
#pragma unroll
    for (int i = 0; i < 16; i++) acc[i] = 0.f;

    auto load = [&](int t0, uint4 (&k)[2][2], uint4 (&v)[2][2]) {
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const int t = t0 + u * G + slot;
            if (t < visible) {
                const uint4* kp = reinterpret_cast<const uint4*>(K + (size_t)t * HD);
                const uint4* vp = reinterpret_cast<const uint4*>(V + (size_t)t * HD);
                // through L1: with grouped-query attention the warps of a CTA are the query heads of one KV head and
                // walk the same rows almost in step, so three of four reads are L1 hits (the cache is only read here)
                k[u][0] = __ldg(kp); k[u][1] = __ldg(kp + 1);
                v[u][0] = __ldg(vp); v[u][1] = __ldg(vp + 1);
            } else {
                k[u][0] = k[u][1] = v[u][0] = v[u][1] = make_uint4(0, 0, 0, 0);
            }
        }
    };
    auto compute = [&](int t0, const uint4 (&k)[2][2], const uint4 (&v)[2][2]) {
        float s[2];
#pragma unroll
        for (int u = 0; u < 2; u++) {
            float kf[16];
            halves16_to_float(k[u][0], k[u][1], kf);
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < 16; i++) d = fmaf(kf[i], q[i], d);
#pragma unroll
            for (int o = 1; o < LPP; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
            s[u] = (t0 + u * G + slot < visible) ? d * scale : -INFINITY;
        }
        const float mn = fmaxf(mx, fmaxf(s[0], s[1]));
        if (mn == -INFINITY) return;  // nothing visible in this lane group yet
        const float corr = expf(mx - mn);  // exp(-inf) = 0 on the first visit
        const float p0 = expf(s[0] - mn), p1 = expf(s[1] - mn);
        mx = mn;
        sum = sum * corr + p0 + p1;
        float v0[16], v1[16];
        halves16_to_float(v[0][0], v[0][1], v0);
        halves16_to_float(v[1][0], v[1][1], v1);
#pragma unroll
        for (int i = 0; i < 16; i++) acc[i] = fmaf(p1, v1[i], fmaf(p0, v0[i], acc[i] * corr));
    };

    uint4 ka[2][2], va[2][2], kb[2][2], vb[2][2];
    const int first = split * 4 * G;  // warps of one (row, head) take alternate blocks of 4 G positions
    load(first, ka, va);
    for (int t0 = first; t0 < visible; t0 += 4 * G * SPLIT) {
        load(t0 + 2 * G, kb, vb);
        compute(t0, ka, va);
        load(t0 + 4 * G * SPLIT, ka, va);
        compute(t0 + 2 * G, kb, vb);
    }
    // merge the lane groups
#pragma unroll
    for (int o = LPP; o < 32; o <<= 1) {
        const float mo = __shfl_xor_sync(0xffffffffu, mx, o);
        const float so = __shfl_xor_sync(0xffffffffu, sum, o);
        const float mn = fmaxf(mx, mo);
        const float c1 = mx == -INFINITY ? 0.f : expf(mx - mn);
        const float c2 = mo == -INFINITY ? 0.f : expf(mo - mn);
        sum = sum * c1 + so * c2;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const float ao = __shfl_xor_sync(0xffffffffu, acc[i], o);
            acc[i] = acc[i] * c1 + ao * c2;
        }
        mx = mn;
    }
    if (SPLIT > 1) {  // (the whole CTA works on one row, so every warp reaches this barrier)
        float* mine = s_merge + ((warp_in_cta % kAttRowsWarps) * LPP + sub) * 18;
        if (split == 1 && slot == 0) {
            mine[0] = mx; mine[1] = sum;
#pragma unroll
            for (int i = 0; i < 16; i++) mine[2 + i] = acc[i];
        }
        __syncthreads();
        if (split == 0 && slot == 0) {
            const float mo = mine[0], so = mine[1];
            const float mn = fmaxf(mx, mo);
            const float c1 = mx == -INFINITY ? 0.f : expf(mx - mn);
            const float c2 = mo == -INFINITY ? 0.f : expf(mo - mn);
            sum = sum * c1 + so * c2;
#pragma unroll
            for (int i = 0; i < 16; i++) acc[i] = acc[i] * c1 + mine[2 + i] * c2;
        }
    }
    if (slot == 0 && split == 0) {
        const float inv = sum > 0.f ? 1.0f / sum : 0.f;
        uint32_t packed[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float a0 = acc[2 * i] * inv, a1 = acc[2 * i + 1] * inv;
            packed[i] = (uint32_t)to_16bit(a0, p.bf16) | ((uint32_t)to_16bit(a1, p.bf16) << 16);
            if (p.debug && r == 0) { p.debug[head * HD + sub * 16 + 2 * i] = a0; p.debug[head * HD + sub * 16 + 2 * i + 1] = a1; }
        }
        uint4* dst = reinterpret_cast<uint4*>(p.ctx16 + (size_t)r * m.q_dim + (size_t)head * HD + sub * 16);
        dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    }
}

__global__ void k_copy_debug(const float* src, float* dst, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src[i];
}

}  // namespace esp
