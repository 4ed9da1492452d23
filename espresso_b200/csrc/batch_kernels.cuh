// Element-wise stages of the batched (tensor-core) decode path.  The matrix products run in k_gemm_tc; these
// kernels prepare its 16-bit operand rows and apply what the GEMV path fuses into its epilogues:
//   k_prep_rows    (embedding) -> RMSNorm / LayerNorm / none -> fp16 or bf16 operand rows
//   k_rope_append  half-split RoPE on q (in place) and k, KV-cache append of k and v
//   k_act_rows     SiLU(gate) * up  or  GELU(up)  -> 16-bit operand rows of the down projection
//   k_head_done    turns the packed per-row maxima of the LM-head GEMM into tokens (head_finalize)
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
};

// One CTA per row.
__global__ void __launch_bounds__(kThreads) k_prep_rows(const PrepArgs p) {
    __shared__ float red[kRedFloats];
    const int r = blockIdx.x;
    if (!p.rs.active[r]) return;
    const int K = p.K;
    const float* src = p.src ? p.src + (size_t)r * K : nullptr;
    const uint16_t* te = nullptr;
    const uint16_t* pe = nullptr;
    if (p.from_embedding) {
        te = p.tok_emb + (size_t)p.rs.tok[r] * K;
        if (p.pos_emb) pe = p.pos_emb + (size_t)p.rs.pos[r] * K;
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
    uint16_t* dst = p.dst + (size_t)r * K;
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
};

// One CTA per row; threads stride over the rotation pairs of q and k and over the elements of v.
__global__ void __launch_bounds__(kThreads) k_rope_append(const RopeArgs p) {
    const int r = blockIdx.x;
    if (!p.rs.active[r]) return;
    const ModelDims& m = p.m;
    const int pos = p.rs.pos[r], seq = p.rs.seq[r];
    const int half = m.head_dim / 2;
    float* q = p.q + (size_t)r * m.q_dim;
    const float* kr = p.k_raw + (size_t)r * m.kv_dim;
    const float* vr = p.v_raw + (size_t)r * m.kv_dim;
    const int q_pairs = m.q_dim / 2, k_pairs = m.kv_dim / 2;
    for (int i = threadIdx.x; i < q_pairs + k_pairs; i += kThreads) {
        const bool is_q = i < q_pairs;
        const int local = is_q ? i : i - q_pairs;
        const int head = local / half, idx = local - head * half;
        const int i0 = head * m.head_dim + idx, i1 = i0 + half;
        float v0 = is_q ? q[i0] : kr[i0], v1 = is_q ? q[i1] : kr[i1];
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
    }
    for (int i = threadIdx.x; i < m.kv_dim; i += kThreads) {
        const int head = i / m.head_dim, idx = i - head * m.head_dim;
        const __half hv = __float2half_rn(vr[i]);
        p.kv.v[p.kv.offset(m, p.layer, seq, head, pos) + idx] = hv;
        if (p.debug && r == 0) p.debug[m.q_dim + m.kv_dim + i] = __half2float(hv);
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
    if (!p.rs.active[r]) return;
    const int i = blockIdx.x * kThreads + threadIdx.x;
    if (i >= p.h) return;
    const float g = p.gate[(size_t)r * p.h + i];
    const float v = p.up ? silu_f(g) * p.up[(size_t)r * p.h + i] : gelu_f(g);
    p.dst[(size_t)r * p.h + i] = to_16bit(v, p.bf16);
    if (p.debug && r == 0) p.debug[i] = v;
}

__global__ void k_head_done(const GemvArgs p) { head_finalize(p); }

__global__ void k_copy_debug(const float* src, float* dst, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src[i];
}

}  // namespace esp
