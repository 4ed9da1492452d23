// Device code of the decode path: weight-streaming GEMV stages with fused norm / RoPE / KV-append /
// activation / residual / argmax epilogues, and decode attention over the fp16 KV cache.
//
// Every stage is a __device__ function parameterised by (cta index, cta count) so that the same code
// runs either as one kernel per stage or inside the persistent whole-step kernel.
//
// Reference arithmetic restated here (paths inside the Espresso project):
//   rmsNorm / LayerNorm      Sources/RealModelInference/RealModelInferenceEngine.swift:6724-6743, :8655-8685
//   GEMV y = W.x             :6674-6718 (vDSP_mmul), biases for GPT-2 Sources/ANEBuilder/ANEBuilder+Composites.swift:27-36
//   half-split RoPE          :6745-6772
//   KV append                :769-772 (the cache layout here is token-major per head, see KvLayout)
//   decode attention         :6774-6823
//   SwiGLU / GELU FFN        :796-820, :8712-8729
//   final norm + LM head + first-max argmax   :663-670, :8182-8275
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace esp {

constexpr int WT_F16 = 1;
constexpr int WT_Q4_0 = 2;
constexpr int WT_Q8_0 = 8;
constexpr int WT_BF16 = 30;

constexpr int ARCH_LLAMA = 0;
constexpr int ARCH_GPT2 = 1;
constexpr uint32_t GPT2_EOS = 50256u;

constexpr int kThreads = 256;  // threads per CTA of every GEMV stage
constexpr int kWarps = kThreads / 32;

// One matrix [rows, cols], row-major.  F16/BF16: `data` holds the elements.  Q8_0: `data` holds int8
// [rows][cols] and `scales` fp16 [rows][cols/32].  Q4_0: `data` holds [rows][cols/32] 16-byte groups (byte j:
// low nibble = element j, high nibble = element j+16 of the group) and `scales` fp16 [rows][cols/32].
struct Weight {
    const void* data;
    const __half* scales;
    int rows, cols, type, pad;
};

struct LayerWeights {
    Weight wq, wk, wv, wo, w1, w2, w3;
    const float *norm1_g, *norm1_b, *norm2_g, *norm2_b;  // RMSNorm gain / LayerNorm gamma,beta (fp32 copies)
    const float *bq, *bk, *bv, *bo, *b1, *b2;             // GPT-2 biases (else null)
};

struct ModelDims {
    int arch, n_layer, n_head, n_kv_head, d_model, head_dim, hidden, vocab, max_seq, q_dim, kv_dim, n_seq;
    float eps;
    int eos_token;
};

// KV cache: fp16, [layer][sequence][kv_head][position][head_dim]; one token's head vector is contiguous.
struct KvLayout {
    __half* k;
    __half* v;
    __device__ __forceinline__ size_t offset(const ModelDims& m, int layer, int seq, int kvh, int pos) const {
        return ((((size_t)layer * m.n_seq + seq) * m.n_kv_head + kvh) * m.max_seq + pos) * (size_t)m.head_dim;
    }
};

// Per-row control state, resident on the device so that a decode loop needs no host round trip.
// A "row" is one token position being processed: for batched decode row r is sequence r; for prefill
// and two-token verify several rows share one sequence at consecutive positions.
struct RowState {
    int* seq;            // [rows] KV-cache sequence slot
    int* pos;            // [rows] position of the token being processed
    uint32_t* tok;       // [rows] token being fed
    int* active;         // [rows] 0 = skip this row
    uint32_t* next;      // [rows] greedy token selected by the last head pass
    int* n_out;          // [rows] tokens emitted so far
    int* limit;          // [rows] emission limit
    uint32_t* out;       // [rows][out_stride] emitted tokens
    int out_stride;
    unsigned long long* best;  // [rows] packed (ordered logit bits << 32 | ~index) running maximum
    unsigned int* ticket;      // [1] CTA completion counter of the head stage
};

struct Activations {
    float* hidden;   // [rows][d_model] residual stream
    float* q;        // [rows][q_dim] post-RoPE queries
    float* ctx;      // [rows][q_dim] attention output
    float* act;      // [rows][hidden] FFN activation
    float* logits;   // [rows][vocab] or null
    float* att_part; // split-KV partials [rows][n_head][splits][head_dim + 2]
    unsigned int* att_ticket;  // [rows][n_head]
    float* debug;    // optional per-stage capture, or null
    int debug_layer;
};

// ------------------------------------------------------------------------------------------------
// small helpers

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum of one float per thread; `red` has kWarps floats.  All threads receive the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kWarps; i++) t += red[i];
    return t;
}

// Weights are streamed once per token and would otherwise push the KV cache, the activations and the small
// per-layer vectors out of L2: they are read with an evict-first L2 policy and without L1 allocation.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint4 ld_weight16(const void* p) {
    uint4 r;
    const uint64_t pol = l2_evict_first_policy();
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p), "l"(pol));
    return r;
}

// Programmatic dependent launch: let the next kernel of the stream start its prologue, and wait until
// the previous kernel's writes are visible.  Both are no-ops when the launch carries no such dependency.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Ask L2 to fetch a contiguous byte range (16-byte aligned start, size multiple of 16).
__device__ __forceinline__ void l2_prefetch(const void* p, unsigned bytes) {
    if (bytes)
        asm volatile("cp.async.bulk.prefetch.L2.global.L2::cache_hint [%0], %1, %2;" ::"l"(p), "r"(bytes), "l"(l2_evict_first_policy()) : "memory");
}

__device__ __forceinline__ float emb_to_float(uint16_t bits, int type) {
    return type == WT_BF16 ? __uint_as_float((uint32_t)bits << 16) : __half2float(__ushort_as_half(bits));
}

template <int WT> struct WTraits;
template <> struct WTraits<WT_F16> { static constexpr int EPL = 8; };   // elements per lane per 16-byte load
template <> struct WTraits<WT_BF16> { static constexpr int EPL = 8; };
template <> struct WTraits<WT_Q8_0> { static constexpr int EPL = 16; };
template <> struct WTraits<WT_Q4_0> { static constexpr int EPL = 32; };

__host__ __device__ inline size_t weight_row_bytes(int type, int cols) {
    return type == WT_Q8_0 ? (size_t)cols : type == WT_Q4_0 ? (size_t)cols / 2 : (size_t)cols * 2;
}

// The activation vector is staged in shared memory in a lane-major order: element
// k = it*(32*EPL) + lane*EPL + j*4 + i lives at float index ((it*NJ + j)*32 + lane)*4 + i (NJ = EPL/4), so that
// the 32 lanes of a warp read 32 consecutive float4 (no bank conflicts) while each lane still owns the EPL
// consecutive elements that one 16-byte weight load covers.
template <int EPL>
__device__ __forceinline__ int xs_index(int k) {
    constexpr int NJ = EPL / 4;
    int it = k / (32 * EPL);
    int rem = k - it * (32 * EPL);
    int lane = rem / EPL;
    int e = rem - lane * EPL;
    return ((it * NJ + (e >> 2)) * 32 + lane) * 4 + (e & 3);
}
template <int EPL>
__host__ __device__ inline int xs_floats(int K) { return ((K + 32 * EPL - 1) / (32 * EPL)) * (32 * EPL); }

// Accumulates the products of one 16-byte vector of fp16/bf16 weights (8 elements) with 8 fp32 activations.
template <int WT>
__device__ __forceinline__ void fma_vec16(const uint4& w, const __half* srow, int k, const float* x, float sx, float& acc) {
    (void)srow; (void)k; (void)sx;
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
    if constexpr (WT == WT_F16) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float2 f = __half22float2(*reinterpret_cast<const __half2*>(&ww[i]));
            acc = fmaf(f.x, x[2 * i], acc);
            acc = fmaf(f.y, x[2 * i + 1], acc);
        }
    } else {
        static_assert(WT == WT_BF16, "fp32-activation path is for fp16/bf16 weights");
#pragma unroll
        for (int i = 0; i < 4; i++) {
            acc = fmaf(__uint_as_float(ww[i] << 16), x[2 * i], acc);
            acc = fmaf(__uint_as_float(ww[i] & 0xffff0000u), x[2 * i + 1], acc);
        }
    }
}

// --- GGUF block arithmetic on packed halves -------------------------------------------------------------
// Quantised weights are widened to fp16 exactly (an int8 or a nibble is an integer of at most 8 bits) with
// byte-permute / logic tricks instead of integer->float conversions, multiplied with activations that were
// staged as fp16 (scaled by a power of two so that |x| < 1, see stage_vector) and summed per 32-element block in
// packed fp16; each block sum is then widened and multiplied by the block scale in fp32.  The dequantised
// weight values themselves stay exactly fp32(d) * q.
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) | c
    return d;
}
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

// 16 bytes = 16 int8 of one Q8_0 block half; xh = the matching 16 staged activations (two 16-byte groups).
__device__ __forceinline__ float q8_block_dot(const uint4& w, const uint4& xa, const uint4& xb) {
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
    const uint32_t xx[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
    const __half2 bias = __floats2half2_rn(1152.f, 1152.f);  // 1024 + 128
    __half2 acc0 = __floats2half2_rn(0.f, 0.f), acc1 = acc0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t u = ww[i] ^ 0x80808080u;                       // int8 -> offset-128 unsigned
        const uint32_t lo = __byte_perm(u, 0x64646464u, 0x4140);      // halves 0x64b0, 0x64b1 = 1024 + b
        const uint32_t hi = __byte_perm(u, 0x64646464u, 0x4342);
        acc0 = __hfma2(__hsub2(u32_as_h2(lo), bias), u32_as_h2(xx[2 * i]), acc0);
        acc1 = __hfma2(__hsub2(u32_as_h2(hi), bias), u32_as_h2(xx[2 * i + 1]), acc1);
    }
    const float2 f = __half22float2(__hadd2(acc0, acc1));
    return f.x + f.y;
}

// 16 bytes = one Q4_0 block (byte j: low nibble = element j, high nibble = element j+16); x0..x3 = the staged
// activations of words 0..3 in the order {e, e+2}, {16+e, 16+e+2}, {e+1, e+3}, {16+e+1, 16+e+3} (e = 4*word).
// A masked nibble is used directly as the bit pattern of an fp16 subnormal: bits 0-3 read as n * 2^-24 and bits
// 4-7 as 16n * 2^-24, both exact, so no conversion instruction is needed at all.  The activations are staged with
// an extra factor 2^14 (see stage_vector) so that the products stay in the normal fp16 range, the "- 8" of the
// format is applied once per block through the block's activation sum, and the remaining powers of two are
// folded into the final de-scale factor.  Returns sum(n * 2^-24 * x'') over the 32 elements.
__device__ __forceinline__ float q4_block_dot(const uint4& w, const uint4& x0, const uint4& x1, const uint4& x2, const uint4& x3) {
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
    const uint4 xs4[4] = {x0, x1, x2, x3};
    __half2 acc_a = __floats2half2_rn(0.f, 0.f), acc_b = acc_a;  // acc_b carries the nibbles read at bit 4 (x16)
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t v = ww[i], t = v >> 8;
        acc_a = __hfma2(u32_as_h2(v & 0x000F000Fu), u32_as_h2(xs4[i].x), acc_a);
        acc_b = __hfma2(u32_as_h2(v & 0x00F000F0u), u32_as_h2(xs4[i].y), acc_b);
        acc_a = __hfma2(u32_as_h2(t & 0x000F000Fu), u32_as_h2(xs4[i].z), acc_a);
        acc_b = __hfma2(u32_as_h2(t & 0x00F000F0u), u32_as_h2(xs4[i].w), acc_b);
    }
    const float2 fa = __half22float2(acc_a), fb = __half22float2(acc_b);
    return (fa.x + fa.y) + (fb.x + fb.y) * 0.0625f;
}

// Per-block activation sums of the Q4_0 staging (pre-multiplied by 2^-21) live behind the staged halves.
__device__ __forceinline__ const float* q4_block_sums(const float* xs, int K) { return xs + xs_floats<32>(K) / 2; }

// Dot products of NR weight rows with the staged vector.  Each lane accumulates its slices; the caller
// reduces across the warp (and, for the quantised types, multiplies by the activation de-scale factor).
// K must be a multiple of EPL.  The loads of U consecutive 16-byte slices of all NR rows are issued before
// any arithmetic so that each lane keeps U*NR*16 bytes in flight.
// One "group" = U consecutive 16-byte slices of NR rows, with the block scales of the quantised types.
constexpr int kDotU = 4;
template <int WT, int NR>
struct DotGroup {
    uint4 w[kDotU][NR];
    __half sc[kDotU][NR];
};

template <int WT, int NR>
__device__ __forceinline__ void dot_load(DotGroup<WT, NR>& g, const uint8_t* const (&wrow)[NR], const __half* const (&srow)[NR], int K, int it0,
                                         int lane) {
    constexpr int EPL = WTraits<WT>::EPL;
#pragma unroll
    for (int u = 0; u < kDotU; u++) {
        const int k = (it0 + u) * 32 * EPL + lane * EPL;
        const size_t byte_off = WT == WT_Q8_0 ? (size_t)k : WT == WT_Q4_0 ? (size_t)k / 2 : (size_t)k * 2;
#pragma unroll
        for (int r = 0; r < NR; r++) {
            g.w[u][r] = k < K ? ld_weight16(wrow[r] + byte_off) : make_uint4(0, 0, 0, 0);
            if constexpr (WT == WT_Q8_0 || WT == WT_Q4_0) g.sc[u][r] = k < K ? srow[r][k >> 5] : __float2half(0.f);
        }
    }
}

template <int WT, int NR>
__device__ __forceinline__ void dot_compute(const DotGroup<WT, NR>& g, int K, int it0, const float* __restrict__ xs, int lane, float (&acc)[NR]) {
    constexpr int EPL = WTraits<WT>::EPL;
    const float4* xs4 = reinterpret_cast<const float4*>(xs);
    const uint4* xh4 = reinterpret_cast<const uint4*>(xs);  // quantised types: fp16 activations, 8 per 16-byte group
#pragma unroll
    for (int u = 0; u < kDotU; u++) {
        const int it = it0 + u;
        const int k = it * 32 * EPL + lane * EPL;
        if (k < K) {
            if constexpr (WT == WT_F16 || WT == WT_BF16) {
                const float4 va = xs4[(it * 2) * 32 + lane], vb = xs4[(it * 2 + 1) * 32 + lane];
                const float x[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
#pragma unroll
                for (int r = 0; r < NR; r++) fma_vec16<WT>(g.w[u][r], nullptr, 0, x, 0.f, acc[r]);
            } else if constexpr (WT == WT_Q8_0) {
                const uint4 xa = xh4[(it * 2) * 32 + lane], xb = xh4[(it * 2 + 1) * 32 + lane];
#pragma unroll
                for (int r = 0; r < NR; r++) acc[r] = fmaf(__half2float(g.sc[u][r]), q8_block_dot(g.w[u][r], xa, xb), acc[r]);
            } else {
                const uint4 x0 = xh4[(it * 4) * 32 + lane], x1 = xh4[(it * 4 + 1) * 32 + lane];
                const uint4 x2 = xh4[(it * 4 + 2) * 32 + lane], x3 = xh4[(it * 4 + 3) * 32 + lane];
                const float bs = q4_block_sums(xs, K)[k >> 5];
#pragma unroll
                for (int r = 0; r < NR; r++) acc[r] = fmaf(__half2float(g.sc[u][r]), q4_block_dot(g.w[u][r], x0, x1, x2, x3) - bs, acc[r]);
            }
        }
    }
}

template <int WT, int NR>
__device__ __forceinline__ void dot_rows(const uint8_t* const (&wrow)[NR], const __half* const (&srow)[NR], int K,
                                         const float* __restrict__ xs, int lane, float (&acc)[NR]) {
    constexpr int EPL = WTraits<WT>::EPL;
    const int iters = (K + 32 * EPL - 1) / (32 * EPL);
    for (int it0 = 0; it0 < iters; it0 += kDotU) {
        DotGroup<WT, NR> g;
        dot_load<WT, NR>(g, wrow, srow, K, it0, lane);
        dot_compute<WT, NR>(g, K, it0, xs, lane, acc);
    }
}

// --- software-pipelined variant ----------------------------------------------------------------------------
// A "batch" is two consecutive 16-byte slices of NR rows.  While one batch is being multiplied the next one (of
// the same rows, or the first batch of the rows the warp handles next) is already in flight, so a warp never
// waits with an empty memory queue between work items.  Weights are constants, which lets the very first batch
// be requested before the activation vector is staged, and even before the previous kernel has finished.
template <int WT, int NR>
struct WBatch {
    uint4 v[2][NR];
};

template <int WT, int NR>
__device__ __forceinline__ void load_batch(WBatch<WT, NR>& b, const uint8_t* const (&wrow)[NR], int K, int it0, int lane) {
    constexpr int EPL = WTraits<WT>::EPL;
#pragma unroll
    for (int u = 0; u < 2; u++) {
        const int k = (it0 + u) * 32 * EPL + lane * EPL;
        const size_t byte_off = WT == WT_Q8_0 ? (size_t)k : WT == WT_Q4_0 ? (size_t)k / 2 : (size_t)k * 2;
#pragma unroll
        for (int r = 0; r < NR; r++) b.v[u][r] = k < K ? ld_weight16(wrow[r] + byte_off) : make_uint4(0, 0, 0, 0);
    }
}

template <int WT, int NR>
__device__ __forceinline__ void compute_batch(const WBatch<WT, NR>& b, const __half* const (&srow)[NR], int K, int it0,
                                              const float* __restrict__ xs, int lane, float (&acc)[NR]) {
    constexpr int EPL = WTraits<WT>::EPL;
    const float4* xs4 = reinterpret_cast<const float4*>(xs);
    const uint4* xh4 = reinterpret_cast<const uint4*>(xs);
#pragma unroll
    for (int u = 0; u < 2; u++) {
        const int it = it0 + u;
        const int k = it * 32 * EPL + lane * EPL;
        if (k < K) {
            if constexpr (WT == WT_F16 || WT == WT_BF16) {
                const float4 va = xs4[(it * 2) * 32 + lane], vb = xs4[(it * 2 + 1) * 32 + lane];
                const float x[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
#pragma unroll
                for (int r = 0; r < NR; r++) fma_vec16<WT>(b.v[u][r], nullptr, 0, x, 0.f, acc[r]);
            } else if constexpr (WT == WT_Q8_0) {
                const uint4 xa = xh4[(it * 2) * 32 + lane], xb = xh4[(it * 2 + 1) * 32 + lane];
#pragma unroll
                for (int r = 0; r < NR; r++) acc[r] = fmaf(__half2float(srow[r][k >> 5]), q8_block_dot(b.v[u][r], xa, xb), acc[r]);
            } else {
                const uint4 x0 = xh4[(it * 4) * 32 + lane], x1 = xh4[(it * 4 + 1) * 32 + lane];
                const uint4 x2 = xh4[(it * 4 + 2) * 32 + lane], x3 = xh4[(it * 4 + 3) * 32 + lane];
#pragma unroll
                const float bs = q4_block_sums(xs, K)[k >> 5];
#pragma unroll
                for (int r = 0; r < NR; r++) acc[r] = fmaf(__half2float(srow[r][k >> 5]), q4_block_dot(b.v[u][r], x0, x1, x2, x3) - bs, acc[r]);
            }
        }
    }
}

// `cur` holds batch 0 of `wrow` on entry and batch 0 of `next` (when has_next) on return.
template <int WT, int NR>
__device__ __forceinline__ void dot_rows_pipelined(const uint8_t* const (&wrow)[NR], const __half* const (&srow)[NR], int K,
                                                   const float* __restrict__ xs, int lane, float (&acc)[NR], WBatch<WT, NR>& cur,
                                                   const uint8_t* const (&next)[NR], bool has_next) {
    constexpr int EPL = WTraits<WT>::EPL;
    const int iters = (K + 32 * EPL - 1) / (32 * EPL);
    for (int it0 = 0; it0 < iters; it0 += 2) {
        WBatch<WT, NR> nxt;
        const bool more = it0 + 2 < iters;
        if (more) load_batch<WT, NR>(nxt, wrow, K, it0 + 2, lane);
        else if (has_next) load_batch<WT, NR>(nxt, next, K, 0, lane);
        compute_batch<WT, NR>(cur, srow, K, it0, xs, lane, acc);
        if (more || has_next) cur = nxt;
    }
}

__device__ __forceinline__ const uint8_t* weight_row(const Weight& w, int row) {
    return static_cast<const uint8_t*>(w.data) + (size_t)row * weight_row_bytes(w.type, w.cols);
}
__device__ __forceinline__ const __half* scale_row(const Weight& w, int row) {
    return w.scales ? w.scales + (size_t)row * (w.cols >> 5) : nullptr;
}

enum NormKind { NORM_NONE = 0, NORM_RMS = 1, NORM_LAYER = 2 };

// Position (in halves) of element k of the fp16-staged vector used by the quantised types: the lane that owns
// the 16-byte weight vector holding k reads its activations as consecutive 16-byte groups, and inside a Q4_0
// group the order follows the nibble extraction of q4_block_dot.
template <int WT>
__device__ __forceinline__ int xh_index(int k) {
    constexpr int EPL = WTraits<WT>::EPL;
    const int it = k / (32 * EPL);
    const int rem = k - it * (32 * EPL);
    const int lane = rem / EPL;
    const int e = rem - lane * EPL;
    if constexpr (WT == WT_Q8_0) {
        return ((it * 2 + (e >> 3)) * 32 + lane) * 8 + (e & 7);
    } else {
        const int byte = e & 15, word = byte >> 2, r = byte & 3;
        const int slot = ((r & 1) ? 4 : 0) + ((r & 2) ? 1 : 0) + ((e & 16) ? 2 : 0);
        return ((it * 4 + word) * 32 + lane) * 8 + slot;
    }
}

__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = red[0];
#pragma unroll
    for (int i = 1; i < kWarps; i++) t = fmaxf(t, red[i]);
    return t;
}

// Stages `src` (K floats) into shared memory, optionally normalised:
//   RMSNorm   y = x * rsqrt(mean(x^2) + eps) * g          LayerNorm  y = (x-mean) * rsqrt(var + eps) * g + b
// fp16/bf16 weights: fp32 values in the lane-major order of xs_index; returns 1.
// Q8_0/Q4_0 weights: fp16 values scaled by a power of two 2^-e (so that |y| < 1) in the order of xh_index;
// returns 2^e, the factor that undoes the scaling after the dot product.
constexpr int kRedFloats = 16;  // reduction scratch in front of the staged vector

// Block-wide (sum, max) of one pair per thread in a single exchange; `red` has kRedFloats floats.
__device__ __forceinline__ void block_sum_max(float& sum, float& mx, float* red) {
    sum = warp_sum(sum);
    mx = warp_max(mx);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = sum; red[8 + (threadIdx.x >> 5)] = mx; }
    __syncthreads();
    float s = 0.f, m = red[8];
#pragma unroll
    for (int i = 0; i < kWarps; i++) { s += red[i]; m = fmaxf(m, red[8 + i]); }
    sum = s;
    mx = m;
}

template <int WT>
__device__ __forceinline__ float stage_vector(const float* __restrict__ src, int K, int norm, const float* g,
                                              const float* b, float eps, float* xs, float* red) {
    constexpr int EPL = WTraits<WT>::EPL;
    constexpr bool kHalf = WT == WT_Q8_0 || WT == WT_Q4_0;
    float inv = 1.f, mean = 0.f, amax = 0.f;
    if (norm == NORM_LAYER) {
        float s = 0.f;
        for (int k = threadIdx.x; k < K; k += kThreads) s += src[k];
        mean = block_sum(s, red) / (float)K;
        float vs = 0.f;
        for (int k = threadIdx.x; k < K; k += kThreads) { float c = src[k] - mean; vs = fmaf(c, c, vs); }
        vs = block_sum(vs, red);
        inv = 1.0f / sqrtf(vs / (float)K + eps);
        if (kHalf) {
            for (int k = threadIdx.x; k < K; k += kThreads) amax = fmaxf(amax, fabsf((src[k] - mean) * inv * g[k] + b[k]));
            amax = block_max(amax, red);
        }
    } else if (norm == NORM_RMS || kHalf) {
        // one pass: sum of squares and, for the fp16-staged types, the largest |x*g| (the norm scale is applied after)
        float ss = 0.f, mx = 0.f;
        for (int k = threadIdx.x; k < K; k += kThreads) {
            const float v = src[k];
            ss = fmaf(v, v, ss);
            if (kHalf) mx = fmaxf(mx, fabsf(norm == NORM_RMS ? v * g[k] : v));
        }
        block_sum_max(ss, mx, red);
        if (norm == NORM_RMS) inv = 1.0f / sqrtf(ss / (float)K + eps);
        amax = mx * inv;
    }
    auto value = [&](int k) {
        float v = src[k];
        if (norm == NORM_RMS) v = (v * inv) * g[k];
        else if (norm == NORM_LAYER) v = (v - mean) * inv * g[k] + b[k];
        return v;
    };
    float descale = 1.f;
    if constexpr (kHalf) {
        int e = 0;
        if (amax > 0.f && amax < 3.0e38f) frexpf(amax * 1.0001f, &e);  // amax = m * 2^e with m in [0.5, 1)
        // Q4_0 stages x * 2^(14-e) (see q4_block_dot) and owes a factor 2^10 at the end; Q8_0 stages x * 2^-e
        const float scale = ldexpf(1.0f, (WT == WT_Q4_0 ? 14 : 0) - e);
        descale = ldexpf(1.0f, e + (WT == WT_Q4_0 ? 10 : 0));
        __half* xh = reinterpret_cast<__half*>(xs);
        for (int k = threadIdx.x; k < K; k += kThreads) xh[xh_index<WT>(k)] = __float2half_rn(value(k) * scale);
        if constexpr (WT == WT_Q4_0) {
            __syncthreads();
            float* bsum = xs + xs_floats<32>(K) / 2;
            for (int blk = threadIdx.x; blk < K / 32; blk += kThreads) {
                float t = 0.f;
                for (int i = 0; i < 32; i++) t += __half2float(xh[xh_index<WT>(blk * 32 + i)]);
                bsum[blk] = t * 4.76837158203125e-07f;  // 2^-21: 8 * 2^-14 (staging) * 2^-10 (folded into the de-scale)
            }
        }
    } else {
        for (int k = threadIdx.x; k < K; k += kThreads) xs[xs_index<EPL>(k)] = value(k);
    }
    __syncthreads();
    return descale;
}

// Range of work items [begin, end) owned by CTA `cta` of `n_cta` (contiguous chunks, so that a CTA's weight
// rows are adjacent in memory).
__device__ __forceinline__ void cta_range(int n_items, int cta, int n_cta, int& begin, int& end) {
    int per = (n_items + n_cta - 1) / n_cta;
    begin = cta * per;
    end = min(begin + per, n_items);
    if (begin > end) begin = end;
}

// ------------------------------------------------------------------------------------------------
// Stage 1: (embedding) -> norm -> Wq,Wk,Wv (+bias) -> RoPE -> q buffer / KV-cache append.
// Work item = a pair of output rows that RoPE rotates together: for q and k the rows (head, i) and
// (head, i + head_dim/2); for v two consecutive rows.

struct QkvArgs {
    ModelDims m;
    LayerWeights lw;
    int layer;
    int rows;
    RowState rs;
    Activations a;
    KvLayout kv;
    const uint16_t* tok_emb; // [vocab][d] fp16 or bf16 bits (layer 0 reads the token row and writes the residual stream)
    const uint16_t* pos_emb; // GPT-2 [max_seq][d] or null
    int emb_type;            // WT_F16 or WT_BF16
    const float2* rope;      // [max_seq][head_dim/2] (cos, sin), Llama only
    int from_embedding;
    // Models with a per-head q/k norm (Qwen3): the norm needs a whole head, which no single work item holds, so this
    // stage stores the plain projections (q in place, k and v here) and k_rope_append applies norm, RoPE and the append.
    float* k_raw;            // [rows][kv_dim] or null
    float* v_raw;            // [rows][kv_dim] or null
};

template <int WT>
__device__ void stage_qkv(const QkvArgs& p, int cta, int n_cta, float* xs, float* red) {
    constexpr int EPL = WTraits<WT>::EPL;
    const ModelDims& m = p.m;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half = m.head_dim / 2;
    const int q_items = m.q_dim / 2, k_items = m.kv_dim / 2, v_items = m.kv_dim / 2;
    const int n_items = q_items + k_items + v_items;
    int begin, end;
    cta_range(n_items, cta, n_cta, begin, end);
    const bool gpt2 = m.arch == ARCH_GPT2;
    // the four weight rows of the two adjacent work items starting at item0
    struct Group {
        const uint8_t* wr[4];
        const __half* sr[4];
        int rows4[4], kinds[2], idx[2];
        const float* biases[2];
    };
    auto describe = [&](int item0, Group& gq) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int item = min(item0 + j, end - 1);
            const Weight* W;
            int local;
            if (item < q_items) { gq.kinds[j] = 0; local = item; W = &p.lw.wq; gq.biases[j] = p.lw.bq; }
            else if (item < q_items + k_items) { gq.kinds[j] = 1; local = item - q_items; W = &p.lw.wk; gq.biases[j] = p.lw.bk; }
            else { gq.kinds[j] = 2; local = item - q_items - k_items; W = &p.lw.wv; gq.biases[j] = p.lw.bv; }
            int row0, row1;
            gq.idx[j] = 0;
            if (gq.kinds[j] < 2) { int head = local / half; gq.idx[j] = local - head * half; row0 = head * m.head_dim + gq.idx[j]; row1 = row0 + half; }
            else { row0 = 2 * local; row1 = row0 + 1; }
            gq.rows4[2 * j] = row0; gq.rows4[2 * j + 1] = row1;
            gq.wr[2 * j] = weight_row(*W, row0); gq.wr[2 * j + 1] = weight_row(*W, row1);
            gq.sr[2 * j] = scale_row(*W, row0); gq.sr[2 * j + 1] = scale_row(*W, row1);
        }
    };
    const int first = begin + 2 * warp;
    Group cur_g, next_g;
    WBatch<WT, 4> batch;
    if (first < end) { describe(first, cur_g); load_batch<WT, 4>(batch, cur_g.wr, m.d_model, 0, lane); }  // weights: no dependency
    pdl_launch_dependents();
    pdl_wait();  // from here on the previous stage's outputs are visible
    for (int r = 0; r < p.rows; r++) {
        if (!p.rs.active[r]) continue;
        const int pos = p.rs.pos[r];
        float* hid = p.a.hidden + (size_t)r * m.d_model;
        float xdescale = 1.f;
        if (p.from_embedding) {
            // hidden = tokenEmbedding[token] (+ positionEmbedding[pos]); every CTA needs it, CTA 0 stores it.
            const uint16_t* te = p.tok_emb + (size_t)p.rs.tok[r] * m.d_model;
            const uint16_t* pe = p.pos_emb ? p.pos_emb + (size_t)pos * m.d_model : nullptr;
            float* tmp = xs + xs_floats<EPL>(m.d_model);  // scratch after the staged vector
            for (int k = threadIdx.x; k < m.d_model; k += kThreads) {
                float v = emb_to_float(te[k], p.emb_type);
                if (pe) v += emb_to_float(pe[k], p.emb_type);
                tmp[k] = v;
                if (cta == 0) hid[k] = v;
            }
            __syncthreads();
            xdescale = stage_vector<WT>(tmp, m.d_model, gpt2 ? NORM_LAYER : NORM_RMS, p.lw.norm1_g, p.lw.norm1_b, m.eps, xs, red);
        } else {
            xdescale = stage_vector<WT>(hid, m.d_model, gpt2 ? NORM_LAYER : NORM_RMS, p.lw.norm1_g, p.lw.norm1_b, m.eps, xs, red);
        }
        const int seq = p.rs.seq[r];
        if (r > 0 && first < end) { describe(first, cur_g); load_batch<WT, 4>(batch, cur_g.wr, m.d_model, 0, lane); }
        // each warp takes two adjacent work items (four weight rows) per iteration
        for (int item0 = first; item0 < end; item0 += 2 * kWarps) {
            const bool has_next = item0 + 2 * kWarps < end;
            if (has_next) describe(item0 + 2 * kWarps, next_g);
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            dot_rows_pipelined<WT, 4>(cur_g.wr, cur_g.sr, m.d_model, xs, lane, acc, batch, next_g.wr, has_next);
#pragma unroll
            for (int j = 0; j < 4; j++) acc[j] = warp_sum(acc[j]) * xdescale;
#pragma unroll
            for (int j = 0; j < 2; j++) {
                if (lane == j && item0 + j < end) {
                    const int kind = cur_g.kinds[j], row0 = cur_g.rows4[2 * j], row1 = cur_g.rows4[2 * j + 1];
                    float v0 = acc[2 * j], v1 = acc[2 * j + 1];
                    const float* bias = cur_g.biases[j];
                    if (bias) { v0 += bias[row0]; v1 += bias[row1]; }
                    if (p.k_raw) {
                        float* dst = kind == 0 ? p.a.q + (size_t)r * m.q_dim : (kind == 1 ? p.k_raw : p.v_raw) + (size_t)r * m.kv_dim;
                        dst[row0] = v0; dst[row1] = v1;
                        continue;
                    }
                    if (kind < 2 && !gpt2) {
                        float2 cs = p.rope[(size_t)pos * half + cur_g.idx[j]];
                        float r0 = v0 * cs.x - v1 * cs.y, r1 = v0 * cs.y + v1 * cs.x;
                        v0 = r0; v1 = r1;
                    }
                    if (kind == 0) {
                        float* q = p.a.q + (size_t)r * m.q_dim;
                        q[row0] = v0; q[row1] = v1;
                    } else {
                        __half* base = (kind == 1 ? p.kv.k : p.kv.v);
                        int kvh = row0 / m.head_dim;
                        size_t off = p.kv.offset(m, p.layer, seq, kvh, pos);
                        base[off + (row0 - kvh * m.head_dim)] = __float2half_rn(v0);
                        base[off + (row1 - kvh * m.head_dim)] = __float2half_rn(v1);
                    }
                    if (p.a.debug && p.layer == p.a.debug_layer && r == 0) {
                        float* dbg = p.a.debug + (kind == 0 ? 0 : kind == 1 ? m.q_dim : m.q_dim + m.kv_dim);
                        dbg[row0] = kind == 0 ? v0 : __half2float(__float2half_rn(v0));
                        dbg[row1] = kind == 0 ? v1 : __half2float(__float2half_rn(v1));
                    }
                }
            }
            if (has_next) cur_g = next_g;
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------------
// Stage 2: decode attention for one (row, query head, KV split).
// scores = q.K^T / sqrt(hd) over positions [0, pos], softmax with max subtraction, ctx = P.V.
// K/V rows are read as 16-byte vectors; softmax statistics use warp shuffles.  When the visible range is
// split across several CTAs each writes (m, l, unnormalised ctx) and the last to finish merges them.

constexpr int kAttThreads = 256;
constexpr int kAttSplitTokens = 256;  // positions handled by one CTA

struct AttArgs {
    ModelDims m;
    int layer, rows, n_splits;
    RowState rs;
    Activations a;
    KvLayout kv;
};

__device__ inline void stage_attention(const AttArgs& p, int r, int head, int split, float* sm) {
    const ModelDims& m = p.m;
    if (!p.rs.active[r]) return;
    const int hd = m.head_dim;
    const int visible = p.rs.pos[r] + 1;
    const int t0 = split * kAttSplitTokens;
    const int n_live_splits = (visible + kAttSplitTokens - 1) / kAttSplitTokens;
    if (t0 >= visible) return;
    const int nt = min(kAttSplitTokens, visible - t0);
    const int qpk = m.n_head / m.n_kv_head;
    const int kvh = head / qpk;
    const int seq = p.rs.seq[r];
    const __half* K = p.kv.k + p.kv.offset(m, p.layer, seq, kvh, t0);
    const __half* V = p.kv.v + p.kv.offset(m, p.layer, seq, kvh, t0);
    float* qs = sm;                       // [hd]
    float* sc = sm + hd;                  // [kAttSplitTokens]
    float* red = sc + kAttSplitTokens;    // [8]
    float* part = red + 8;                // [warps][hd]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = kAttThreads / 32;
    const float scale = 1.0f / sqrtf((float)hd);
    const float* q = p.a.q + (size_t)r * m.q_dim + (size_t)head * hd;
    for (int d = tid; d < hd; d += kAttThreads) qs[d] = q[d];
    __syncthreads();
    // scores: one thread per position, 16-byte loads along head_dim
    float lmax = -INFINITY;
    for (int t = tid; t < nt; t += kAttThreads) {
        const uint4* kr = reinterpret_cast<const uint4*>(K + (size_t)t * hd);
        uint4 kreg[16];  // the whole K row (head_dim <= 128) is requested before any arithmetic
#pragma unroll
        for (int c = 0; c < 16; c++) kreg[c] = c < hd / 8 ? __ldcg(kr + c) : make_uint4(0, 0, 0, 0);
        float dot = 0.f;
#pragma unroll
        for (int c = 0; c < 16; c++) {
            if (c < hd / 8) {
                const uint32_t ww[4] = {kreg[c].x, kreg[c].y, kreg[c].z, kreg[c].w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float2 f = __half22float2(*reinterpret_cast<const __half2*>(&ww[i]));
                    dot = fmaf(f.x, qs[c * 8 + 2 * i], dot);
                    dot = fmaf(f.y, qs[c * 8 + 2 * i + 1], dot);
                }
            }
        }
        dot *= scale;
        sc[t] = dot;
        lmax = fmaxf(lmax, dot);
    }
    lmax = warp_max(lmax);
    if (lane == 0) red[warp] = lmax;
    __syncthreads();
    float mx = red[0];
    for (int i = 1; i < nwarp; i++) mx = fmaxf(mx, red[i]);
    __syncthreads();
    float lsum = 0.f;
    for (int t = tid; t < nt; t += kAttThreads) {
        float e = expf(sc[t] - mx);
        sc[t] = e;
        lsum += e;
    }
    lsum = warp_sum(lsum);
    if (lane == 0) red[warp] = lsum;
    __syncthreads();
    float denom = 0.f;
    for (int i = 0; i < nwarp; i++) denom += red[i];
    // ctx: warps stride over positions; each lane owns head_dim/32 consecutive channels (2 or 4)
    const int cpl = hd / 32;  // channels per lane (head_dim 64 -> 2, 128 -> 4); smaller heads use lanes < hd
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (cpl >= 1) {
        constexpr int PU = 8;  // V rows requested together
        for (int tb = warp; tb < nt; tb += nwarp * PU) {
            uint2 vreg[PU];
#pragma unroll
            for (int u = 0; u < PU; u++) {
                const int t = tb + u * nwarp;
                vreg[u] = make_uint2(0, 0);
                if (t < nt) {
                    const __half* vr = V + (size_t)t * hd + lane * cpl;
                    if (cpl == 4) vreg[u] = __ldcg(reinterpret_cast<const uint2*>(vr));
                    else if (cpl == 2) vreg[u].x = __ldcg(reinterpret_cast<const unsigned int*>(vr));
                    else vreg[u].x = (unsigned int)__ldcg(reinterpret_cast<const unsigned short*>(vr));
                }
            }
#pragma unroll
            for (int u = 0; u < PU; u++) {
                const int t = tb + u * nwarp;
                if (t < nt) {
                    const float pt = sc[t];
                    float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&vreg[u].x));
                    float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&vreg[u].y));
                    acc[0] = fmaf(pt, f0.x, acc[0]);
                    if (cpl >= 2) acc[1] = fmaf(pt, f0.y, acc[1]);
                    if (cpl == 4) { acc[2] = fmaf(pt, f1.x, acc[2]); acc[3] = fmaf(pt, f1.y, acc[3]); }
                }
            }
        }
        for (int c = 0; c < cpl && c < 4; c++) part[warp * hd + lane * cpl + c] = acc[c];
    } else {  // head_dim < 32: lane d < hd owns channel d
        if (lane < hd) {
            for (int t = warp; t < nt; t += nwarp) acc[0] = fmaf(sc[t], __half2float(V[(size_t)t * hd + lane]), acc[0]);
            part[warp * hd + lane] = acc[0];
        }
    }
    __syncthreads();
    float* ctx = p.a.ctx + (size_t)r * m.q_dim + (size_t)head * hd;
    if (n_live_splits == 1) {
        const float inv = denom > 0.f ? 1.0f / denom : 0.f;
        for (int d = tid; d < hd; d += kAttThreads) {
            float s = 0.f;
            for (int w = 0; w < nwarp; w++) s += part[w * hd + d];
            ctx[d] = s * inv;
            if (p.a.debug && p.layer == p.a.debug_layer && r == 0) p.a.debug[m.q_dim + 2 * m.kv_dim + head * hd + d] = s * inv;
        }
        return;
    }
    // split-KV: publish this split's (max, sum, unnormalised ctx); the last CTA of the head merges
    float* mine = p.a.att_part + (((size_t)r * m.n_head + head) * p.n_splits + split) * (hd + 2);
    for (int d = tid; d < hd; d += kAttThreads) {
        float s = 0.f;
        for (int w = 0; w < nwarp; w++) s += part[w * hd + d];
        mine[2 + d] = s;
    }
    if (tid == 0) { mine[0] = mx; mine[1] = denom; }
    __threadfence();
    __syncthreads();
    __shared__ unsigned int s_last;
    unsigned int* ticket = p.a.att_ticket + (size_t)r * m.n_head + head;
    if (tid == 0) s_last = atomicAdd(ticket, 1u);
    __syncthreads();
    if (s_last != (unsigned)(n_live_splits - 1)) return;
    __threadfence();
    const float* all = p.a.att_part + ((size_t)r * m.n_head + head) * p.n_splits * (hd + 2);
    float gm = -INFINITY;
    for (int s = 0; s < n_live_splits; s++) gm = fmaxf(gm, all[(size_t)s * (hd + 2)]);
    float gl = 0.f;
    for (int s = 0; s < n_live_splits; s++) gl += all[(size_t)s * (hd + 2) + 1] * expf(all[(size_t)s * (hd + 2)] - gm);
    const float inv = gl > 0.f ? 1.0f / gl : 0.f;
    for (int d = tid; d < hd; d += kAttThreads) {
        float s = 0.f;
        for (int sp = 0; sp < n_live_splits; sp++)
            s += all[(size_t)sp * (hd + 2) + 2 + d] * expf(all[(size_t)sp * (hd + 2)] - gm);
        ctx[d] = s * inv;
        if (p.a.debug && p.layer == p.a.debug_layer && r == 0) p.a.debug[m.q_dim + 2 * m.kv_dim + head * hd + d] = s * inv;
    }
    if (tid == 0) *ticket = 0u;  // ready for the next launch
}

// ------------------------------------------------------------------------------------------------
// Generic "vector -> rows" stage used by the output projection, the FFN and the LM head.

enum Epilogue {
    EPI_RESIDUAL = 0,  // out[row] = resid[row] + y (+bias): Wo and W2
    EPI_SWIGLU = 1,    // act[i] = silu(W1.x)[i] * (W3.x)[i]
    EPI_GELU = 2,      // act[i] = gelu(W1.x + b1)[i]
    EPI_HEAD = 3       // logits (optional store) + running first-max argmax
};

struct GemvArgs {
    ModelDims m;
    int rows;
    RowState rs;
    Activations a;
    Weight w;          // main matrix (Wo, W1, W2 or lm_head)
    Weight w_up;       // W3 for SwiGLU
    const float* bias;
    const float *norm_g, *norm_b;
    int norm;          // NormKind applied to the input vector
    const float* in;   // [rows][in_stride]
    int in_stride;
    float* out;        // EPI_RESIDUAL: hidden (updated in place); EPI_SWIGLU/GELU: act
    int out_stride;
    int layer;
    int debug_slot;    // offset inside the debug capture buffer or -1
    int finalize_mode; // EPI_HEAD: bit 0 = emit the token and feed it back (device-driven decode loop);
                       //           bit 1 = the step processed a token: advance the row's position first
};

__device__ __forceinline__ float silu_f(float x) { return 0.5f * x * (1.0f + tanhf(0.5f * x)); }
__device__ __forceinline__ float gelu_f(float x) {
    float inner = (x + 0.044715f * (x * x * x)) * 0.7978846f;
    return (0.5f * x) * (1.0f + tanhf(inner));
}

// Monotonic mapping float -> uint32 (larger float => larger key).
__device__ __forceinline__ uint32_t ordered_bits(float f) {
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long pack_best(float v, int idx) {
    return ((unsigned long long)ordered_bits(v) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)idx);
}

// Runs once per head pass, by the last CTA to finish: turns the packed maxima into tokens and, in the
// device-driven loop, applies the reference's emission rules (Llama: emit EOS then stop, Engine.swift:6385-6388;
// GPT-2: stop on 50256 without emitting, :4920-4922; stop at the emission limit or when the context is full).
__device__ inline void head_finalize(const GemvArgs& p) {
    const ModelDims& m = p.m;
    for (int r = threadIdx.x; r < p.rows; r += blockDim.x) {
        unsigned long long key = p.rs.best[r];
        p.rs.best[r] = 0ull;
        if (!p.rs.active[r]) continue;
        uint32_t tokn = min(0xffffffffu - (uint32_t)(key & 0xffffffffull), (uint32_t)(m.vocab - 1));  // in range even if every logit was NaN
        p.rs.next[r] = tokn;
        int pos = p.rs.pos[r];
        if (p.finalize_mode & 2) { pos += 1; p.rs.pos[r] = pos; }
        if (p.finalize_mode & 1) {
            bool emit = true, stop = false;
            if (m.arch == ARCH_GPT2) { if (tokn == GPT2_EOS) { emit = false; stop = true; } }
            else if (m.eos_token >= 0 && tokn == (uint32_t)m.eos_token) stop = true;
            int n = p.rs.n_out[r];
            if (emit) { p.rs.out[(size_t)r * p.rs.out_stride + n] = tokn; n++; p.rs.n_out[r] = n; }
            // `pos` tokens are visible; with the token just emitted the sequence holds pos + 1 tokens
            if (n >= p.rs.limit[r] || pos + 1 >= m.max_seq) stop = true;
            p.rs.tok[r] = tokn;
            if (stop) p.rs.active[r] = 0;
        }
    }
}

template <int WT, int EPI>
__device__ void stage_gemv(const GemvArgs& p, int cta, int n_cta, float* xs, float* red) {
    constexpr int EPL = WTraits<WT>::EPL;
    constexpr int NR = 2;  // rows per work item
    const ModelDims& m = p.m;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = p.w.cols;
    const int n_out = p.w.rows;
    const int n_items = EPI == EPI_SWIGLU ? n_out : (n_out + NR - 1) / NR;
    int begin, end;
    cta_range(n_items, cta, n_cta, begin, end);
    struct Group {
        const uint8_t* wr[4];
        const __half* sr[4];
    };
    auto describe = [&](int item0, Group& gq) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int item = min(item0 + j, end - 1);
            if (EPI == EPI_SWIGLU) {
                gq.wr[2 * j] = weight_row(p.w, item); gq.wr[2 * j + 1] = weight_row(p.w_up, item);
                gq.sr[2 * j] = scale_row(p.w, item); gq.sr[2 * j + 1] = scale_row(p.w_up, item);
            } else {
                const int row0 = item * NR, row1 = min(row0 + 1, n_out - 1);
                gq.wr[2 * j] = weight_row(p.w, row0); gq.wr[2 * j + 1] = weight_row(p.w, row1);
                gq.sr[2 * j] = scale_row(p.w, row0); gq.sr[2 * j + 1] = scale_row(p.w, row1);
            }
        }
    };
    const int first = begin + 2 * warp;
    Group cur_g, next_g;
    WBatch<WT, 4> batch;
    if (first < end) { describe(first, cur_g); load_batch<WT, 4>(batch, cur_g.wr, K, 0, lane); }  // weights: no dependency
    pdl_launch_dependents();
    pdl_wait();  // from here on the previous stage's outputs are visible
    for (int r = 0; r < p.rows; r++) {
        if (!p.rs.active[r]) continue;
        const float xdescale = stage_vector<WT>(p.in + (size_t)r * p.in_stride, K, p.norm, p.norm_g, p.norm_b, m.eps, xs, red);
        float best_v = -INFINITY;
        int best_i = 0x7fffffff;
        if (r > 0 && first < end) { describe(first, cur_g); load_batch<WT, 4>(batch, cur_g.wr, K, 0, lane); }
        // each warp takes two adjacent work items (four weight rows) per iteration
        for (int item0 = first; item0 < end; item0 += 2 * kWarps) {
            const bool has_next = item0 + 2 * kWarps < end;
            if (has_next) describe(item0 + 2 * kWarps, next_g);
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            dot_rows_pipelined<WT, 4>(cur_g.wr, cur_g.sr, K, xs, lane, acc, batch, next_g.wr, has_next);
#pragma unroll
            for (int j = 0; j < 4; j++) acc[j] = warp_sum(acc[j]) * xdescale;
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int item = item0 + j;
                if (item >= end) break;
                float v0 = acc[2 * j], v1 = acc[2 * j + 1];
                const int row0 = EPI == EPI_SWIGLU ? item : item * NR;
                const int row1 = EPI == EPI_SWIGLU ? item : min(row0 + 1, n_out - 1);
                if (EPI == EPI_HEAD) {
                    // every lane holds the sums; keep a per-warp running first-max
                    if (v0 > best_v) { best_v = v0; best_i = row0; }
                    if (row1 != row0 && v1 > best_v) { best_v = v1; best_i = row1; }
                    if (lane == 0 && p.a.logits) {
                        float* lg = p.a.logits + (size_t)r * m.vocab;
                        lg[row0] = v0;
                        if (row1 != row0) lg[row1] = v1;
                    }
                } else if (lane == 0) {
                    if (EPI == EPI_RESIDUAL) {
                        float* o = p.out + (size_t)r * p.out_stride;
                        if (p.bias) { v0 += p.bias[row0]; v1 += p.bias[row1]; }
                        float o0 = o[row0] + v0;
                        o[row0] = o0;
                        float o1 = 0.f;
                        if (row1 != row0) { o1 = o[row1] + v1; o[row1] = o1; }
                        if (p.a.debug && p.debug_slot >= 0 && p.layer == p.a.debug_layer && r == 0) {
                            p.a.debug[p.debug_slot + row0] = o0;
                            if (row1 != row0) p.a.debug[p.debug_slot + row1] = o1;
                        }
                    } else if (EPI == EPI_SWIGLU) {
                        float av = silu_f(v0) * v1;
                        p.out[(size_t)r * p.out_stride + item] = av;
                        if (p.a.debug && p.debug_slot >= 0 && p.layer == p.a.debug_layer && r == 0) p.a.debug[p.debug_slot + item] = av;
                    } else {  // EPI_GELU
                        float* o = p.out + (size_t)r * p.out_stride;
                        if (p.bias) { v0 += p.bias[row0]; v1 += p.bias[row1]; }
                        float a0 = gelu_f(v0), a1 = gelu_f(v1);
                        o[row0] = a0;
                        if (row1 != row0) o[row1] = a1;
                        if (p.a.debug && p.debug_slot >= 0 && p.layer == p.a.debug_layer && r == 0) {
                            p.a.debug[p.debug_slot + row0] = a0;
                            if (row1 != row0) p.a.debug[p.debug_slot + row1] = a1;
                        }
                    }
                }
            }
            if (has_next) cur_g = next_g;
        }
        if (EPI == EPI_HEAD) {
            // rows grow with the item index, so within a warp the first maximum is kept by the strict '>' above;
            // across warps and CTAs the packed key (value, ~index) makes the smallest index win ties.
            if (lane == 0 && best_i != 0x7fffffff) atomicMax(p.rs.best + r, pack_best(best_v, best_i));
        }
        __syncthreads();
    }
    if (EPI == EPI_HEAD) {
        __shared__ unsigned int s_ticket;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) s_ticket = atomicAdd(p.rs.ticket, 1u);
        __syncthreads();
        if (s_ticket == (unsigned)(n_cta - 1)) {
            __threadfence();
            head_finalize(p);
            __syncthreads();
            if (threadIdx.x == 0) *p.rs.ticket = 0u;
        }
    }
}

// Advance the position of every active row by one (the token just processed becomes visible).
__device__ __forceinline__ void bump_positions(const RowState& rs, int rows) {
    for (int r = threadIdx.x; r < rows; r += blockDim.x)
        if (rs.active[r]) rs.pos[r] += 1;
}

}  // namespace esp
