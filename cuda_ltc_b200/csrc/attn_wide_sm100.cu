// Attention on the tensor pipe for head widths the streaming kernels do not cover (any multiple of 8, in
// particular the reference's TimeSelfAttention, where every head is as wide as the model:
// include/cuDNN_ops.h:166-169 of the reference gives qProjSize = kProjSize = vProjSize = input_dim).
//
// The streaming (flash) kernels keep a 128-row tile of O in tensor memory, which ends at 128 columns of head
// width.  Here the score matrix is written out instead, as cuDNN's multi-head attention does it
// (cudnnMultiHeadAttnForward keeps it in its reserve space, src/ml/cuDNN_ops.cu:203-226), and every contraction
// is one launch of the batched tcgen05 GEMM of gemm_sm100.cu over the (batch, head) pairs:
//   forward    S = Q K^T (fp32)  ->  P = softmax(mask(scale S)) (bf16, one warp per row)  ->  O = P V
//   backward   dP = dO V^T (fp32),  dV = P^T dO,  dS = scale P o (dP - rowsum(P o dP)) (bf16, over P),
//              dQ = dS K,  dK = dS^T Q
// No operand is transposed in memory: the GEMM takes both operand forms.
//
// Precision.  With optional low-order parts of Q and K (q = q_hi + q_lo, two bf16 terms, 16 significant bits)
// the scores are formed as q_hi k_hi + q_hi k_lo + q_lo k_hi in one accumulator.  The reference's configuration
// has no 1/sqrt(d) scale and heads as wide as the model, so scores of magnitude 10 - 20 are common and an 8-bit
// rounding of q and k alone would move a softmax weight by several per cent; the three-term form keeps the
// scores at fp32-class accuracy (tighter than the TF32 arithmetic cuDNN uses for the same products).
#include "host_common.h"
#include "gemm_sm100.h"
#include "attn_wide.h"
#include "sm100_ptx.cuh"

namespace ltca {

namespace {

__device__ __forceinline__ float wneg_inf() { return __int_as_float(0xff800000); }
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

struct SoftmaxArgs {
    int B, H, Sq, Sk, Skp;
    int causal, causal_off;
    float scale, clamp;          // clamp <= 0: none
    const float* keep_mask;      // [B, Sq, Sk] or null
    const int32_t* kv_len;       // [B] or null
    const float* scores;         // [B*H, Sq, Skp] raw Q K^T
    __nv_bfloat16* P;            // [B*H, Sq, Skp] normalised probabilities (pad columns zero)
    __nv_bfloat16* Plo;          // optional low-order term of P (and of dS)
    float* lse;                  // [B*H, Sq] or null
    // backward
    const float* dP;             // [B*H, Sq, Skp]
    __nv_bfloat16 *dS, *dSlo;    // where dS goes (P / Plo themselves when the caller gave no separate buffer)
};

// One warp per (batch, head, query) row: scale, clamp (the reference clamps scaled scores at 10,
// src/ml/flash_attention.cu:167), visibility (keep-mask value 0 hides, :161-164; causal; key lengths), softmax.
__global__ void __launch_bounds__(256) wide_softmax_fwd_kernel(const SoftmaxArgs a) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= (int64_t)a.B * a.H * a.Sq) return;
    const int i = (int)(row % a.Sq);
    const int b = (int)(row / ((int64_t)a.H * a.Sq));
    int lim = a.Sk;
    if (a.kv_len) lim = min(max(a.kv_len[b], 0), a.Sk);
    if (a.causal) lim = min(lim, i + a.causal_off + 1);
    const float* s = a.scores + row * a.Skp;
    const float* mrow = a.keep_mask ? a.keep_mask + ((int64_t)b * a.Sq + i) * a.Sk : nullptr;
    __nv_bfloat16* p = a.P + row * a.Skp;
    float m = wneg_inf();
    for (int j = lane; j < lim; j += 32) {
        if (mrow && mrow[j] == 0.0f) continue;
        float v = s[j] * a.scale;
        if (a.clamp > 0.f) v = fminf(v, a.clamp);
        m = fmaxf(m, v);
    }
    m = warp_max(m);
    float l = 0.f;
    if (m != wneg_inf()) {
        for (int j = lane; j < lim; j += 32) {
            if (mrow && mrow[j] == 0.0f) continue;
            float v = s[j] * a.scale;
            if (a.clamp > 0.f) v = fminf(v, a.clamp);
            l += __expf(v - m);
        }
    }
    l = warp_sum(l);
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    for (int j = lane; j < a.Skp; j += 32) {
        float pv = 0.f;
        if (j < lim && !(mrow && mrow[j] == 0.0f) && l > 0.f) {
            float v = s[j] * a.scale;
            if (a.clamp > 0.f) v = fminf(v, a.clamp);
            pv = __expf(v - m) * inv;
        }
        const __nv_bfloat16 hi = __float2bfloat16_rn(pv);
        p[j] = hi;
        if (a.Plo) a.Plo[row * a.Skp + j] = __float2bfloat16_rn(pv - __bfloat162float(hi));
    }
    if (lane == 0 && a.lse) a.lse[row] = l > 0.f ? m + __logf(l) : wneg_inf();
}

// dS = scale * P o (dP - sum_j P dP), zero where the score was clamped; written to dS (P itself by default).
__global__ void __launch_bounds__(256) wide_softmax_bwd_kernel(const SoftmaxArgs a) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= (int64_t)a.B * a.H * a.Sq) return;
    __nv_bfloat16* p = a.P + row * a.Skp;
    const float* dp = a.dP + row * a.Skp;
    const float* s = a.scores + row * a.Skp;
    __nv_bfloat16* plo = a.Plo ? a.Plo + row * a.Skp : nullptr;
    float delta = 0.f;
    for (int j = lane; j < a.Sk; j += 32) {
        const float pv = __bfloat162float(p[j]) + (plo ? __bfloat162float(plo[j]) : 0.f);
        delta = fmaf(pv, dp[j], delta);
    }
    delta = warp_sum(delta);
    for (int j = lane; j < a.Skp; j += 32) {
        float d = 0.f;
        if (j < a.Sk) {
            const float pv = __bfloat162float(p[j]) + (plo ? __bfloat162float(plo[j]) : 0.f);
            d = pv * (dp[j] - delta) * a.scale;
            if (a.clamp > 0.f && s[j] * a.scale >= a.clamp) d = 0.f;
        }
        const __nv_bfloat16 hi = __float2bfloat16_rn(d);
        a.dS[row * a.Skp + j] = hi;
        if (a.dSlo) a.dSlo[row * a.Skp + j] = __float2bfloat16_rn(d - __bfloat162float(hi));
    }
}

__device__ __forceinline__ uint2 pack4_bf16(const float* v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    return make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
}
__device__ __forceinline__ void unpack4_bf16(uint2 w, float* v) {
    v[0] = __uint_as_float(w.x << 16); v[1] = __uint_as_float(w.x & 0xffff0000u);
    v[2] = __uint_as_float(w.y << 16); v[3] = __uint_as_float(w.y & 0xffff0000u);
}

// The same two operations for rows of up to 128 * kChunks keys: a lane keeps its part of the row in registers
// (kChunks groups of four neighbouring columns), so every matrix is read once, 16 bytes per lane and access.
template <int kChunks>
__global__ void __launch_bounds__(256) wide_softmax_fwd_rows_kernel(const SoftmaxArgs a) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= (int64_t)a.B * a.H * a.Sq) return;
    const int i = (int)(row % a.Sq);
    const int b = (int)(row / ((int64_t)a.H * a.Sq));
    int lim = a.Sk;
    if (a.kv_len) lim = min(max(a.kv_len[b], 0), a.Sk);
    if (a.causal) lim = min(lim, i + a.causal_off + 1);
    const float* s = a.scores + row * a.Skp;
    const float* mrow = a.keep_mask ? a.keep_mask + ((int64_t)b * a.Sq + i) * a.Sk : nullptr;
    float x[kChunks][4];
    float m = wneg_inf();
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const int col = 4 * (lane + 32 * c);
        float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (col < a.Skp) v4 = *reinterpret_cast<const float4*>(s + col);
        const float v[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int j = col + e;
            float t = v[e] * a.scale;
            if (a.clamp > 0.f) t = fminf(t, a.clamp);
            if (j >= lim || (mrow && mrow[j] == 0.0f)) t = wneg_inf();
            x[c][e] = t;
            m = fmaxf(m, t);
        }
    }
    m = warp_max(m);
    float l = 0.f;
    if (m != wneg_inf()) {
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                x[c][e] = __expf(x[c][e] - m);          // hidden keys: exp(-inf) = 0
                l += x[c][e];
            }
    }
    l = warp_sum(l);
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const int col = 4 * (lane + 32 * c);
        if (col >= a.Skp) continue;
        float pv[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) pv[e] = l > 0.f ? x[c][e] * inv : 0.f;
        const uint2 hi = pack4_bf16(pv);
        *reinterpret_cast<uint2*>(a.P + row * a.Skp + col) = hi;
        if (a.Plo) {
            float back[4];
            unpack4_bf16(hi, back);
#pragma unroll
            for (int e = 0; e < 4; ++e) lo[e] = pv[e] - back[e];
            *reinterpret_cast<uint2*>(a.Plo + row * a.Skp + col) = pack4_bf16(lo);
        }
    }
    if (lane == 0 && a.lse) a.lse[row] = l > 0.f ? m + __logf(l) : wneg_inf();
}

template <int kChunks>
__global__ void __launch_bounds__(256) wide_softmax_bwd_rows_kernel(const SoftmaxArgs a) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= (int64_t)a.B * a.H * a.Sq) return;
    const int64_t base = row * a.Skp;
    float p[kChunks][4], dp[kChunks][4];
    float delta = 0.f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const int col = 4 * (lane + 32 * c);
#pragma unroll
        for (int e = 0; e < 4; ++e) p[c][e] = dp[c][e] = 0.f;
        if (col >= a.Skp) continue;
        unpack4_bf16(*reinterpret_cast<const uint2*>(a.P + base + col), p[c]);
        if (a.Plo) {
            float lo[4];
            unpack4_bf16(*reinterpret_cast<const uint2*>(a.Plo + base + col), lo);
#pragma unroll
            for (int e = 0; e < 4; ++e) p[c][e] += lo[e];
        }
        const float4 d4 = *reinterpret_cast<const float4*>(a.dP + base + col);
        dp[c][0] = d4.x; dp[c][1] = d4.y; dp[c][2] = d4.z; dp[c][3] = d4.w;
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (col + e < a.Sk) delta = fmaf(p[c][e], dp[c][e], delta);
    }
    delta = warp_sum(delta);
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const int col = 4 * (lane + 32 * c);
        if (col >= a.Skp) continue;
        float d[4], lo[4];
        float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (a.clamp > 0.f) s4 = *reinterpret_cast<const float4*>(a.scores + base + col);
        const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            d[e] = col + e < a.Sk ? p[c][e] * (dp[c][e] - delta) * a.scale : 0.f;
            if (a.clamp > 0.f && sv[e] * a.scale >= a.clamp) d[e] = 0.f;
        }
        const uint2 hi = pack4_bf16(d);
        *reinterpret_cast<uint2*>(a.dS + base + col) = hi;
        if (a.dSlo) {
            float back[4];
            unpack4_bf16(hi, back);
#pragma unroll
            for (int e = 0; e < 4; ++e) lo[e] = d[e] - back[e];
            *reinterpret_cast<uint2*>(a.dSlo + base + col) = pack4_bf16(lo);
        }
    }
}

// Four neighbouring values per thread when every row starts on 16 bytes.
__global__ void wide_split_vec_kernel(const float* __restrict__ src, int64_t ld_src, __nv_bfloat16* __restrict__ hi,
                                      __nv_bfloat16* __restrict__ lo, int64_t ld_dst, int64_t rows, int cols4) {
    const int64_t n = rows * cols4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cols4;
        const int c = 4 * (int)(i - r * cols4);
        const float4 x4 = *reinterpret_cast<const float4*>(src + r * ld_src + c);
        const float x[4] = {x4.x, x4.y, x4.z, x4.w};
        const uint2 h = pack4_bf16(x);
        *reinterpret_cast<uint2*>(hi + r * ld_dst + c) = h;
        if (lo) {
            float back[4], l[4];
            unpack4_bf16(h, back);
#pragma unroll
            for (int e = 0; e < 4; ++e) l[e] = x[e] - back[e];
            *reinterpret_cast<uint2*>(lo + r * ld_dst + c) = pack4_bf16(l);
        }
    }
}

// hi = bf16(x), lo = bf16(x - hi): two terms carry 16 significant bits of an fp32 value
__global__ void wide_split_kernel(const float* __restrict__ src, int64_t ld_src, __nv_bfloat16* __restrict__ hi,
                                  __nv_bfloat16* __restrict__ lo, int64_t ld_dst, int64_t rows, int cols) {
    const int64_t n = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cols;
        const int c = (int)(i - r * cols);
        const float x = src[r * ld_src + c];
        const __nv_bfloat16 h = __float2bfloat16_rn(x);
        hi[r * ld_dst + c] = h;
        if (lo) lo[r * ld_dst + c] = __float2bfloat16_rn(x - __bfloat162float(h));
    }
}

SoftmaxArgs softmax_args(const WideArgs& w) {
    SoftmaxArgs a;
    memset(&a, 0, sizeof(a));
    a.B = w.B; a.H = w.H; a.Sq = w.Sq; a.Sk = w.Sk; a.Skp = wide_padded_keys(w.Sk);
    a.causal = w.causal; a.causal_off = w.Sk - w.Sq;
    a.scale = w.scale; a.clamp = w.clamp;
    a.keep_mask = w.keep_mask; a.kv_len = w.kv_len;
    a.scores = w.scores; a.P = reinterpret_cast<__nv_bfloat16*>(w.P); a.lse = w.lse; a.dP = w.dP;
    a.Plo = reinterpret_cast<__nv_bfloat16*>(w.Plo);
    a.dS = reinterpret_cast<__nv_bfloat16*>(w.dS ? w.dS : w.P);
    a.dSlo = reinterpret_cast<__nv_bfloat16*>(w.dS ? w.dSlo : w.Plo);
    return a;
}

bool softmax_rows_aligned(const SoftmaxArgs& a) {
    const auto al = [](const void* p, uintptr_t n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; };
    return al(a.scores, 16) && al(a.P, 8) && al(a.Plo, 8);
}

// One batched product over the (head, batch) grid.  `a`/`b`: base pointer, row pitch, operand form and the
// (head, batch) strides of each operand; C likewise.
struct Mat { const void* ptr; int64_t ld; int mn_major; int64_t hs, bs; };
int batched(ltca_ctx* ctx, const WideArgs& w, int M, int N, int K, const Mat* a, const Mat* b, int n_sum, void* c,
            int64_t ldc, int64_t c_hs, int64_t c_bs, int out_bf16) {
    GemmProblem gp;
    gp.M = M; gp.N = N; gp.K = K;
    gp.n_sum = n_sum;
    for (int i = 0; i < n_sum; ++i) {
        gp.a[i] = GemmOperand{a[i].ptr, a[i].ld, a[i].mn_major};
        gp.b[i] = GemmOperand{b[i].ptr, b[i].ld, b[i].mn_major};
    }
    gp.a_bs[0] = a[0].hs; gp.a_bs[1] = a[0].bs;
    gp.b_bs[0] = b[0].hs; gp.b_bs[1] = b[0].bs;
    gp.c[0] = c;
    gp.ldc = ldc;
    gp.c_bs[0] = c_hs; gp.c_bs[1] = c_bs;
    gp.out_bf16 = out_bf16;
    gp.batch_h = w.H; gp.batch_b = w.B;
    return gemm_sm100(ctx, gp);
}

}  // namespace

int wide_split_bf16(ltca_ctx* ctx, const float* src, int64_t ld_src, void* hi, void* lo, int64_t ld_dst, int64_t rows,
                    int cols) {
    if (rows < 1 || cols < 1) return LTCA_OK;
    const int64_t n = rows * cols;
    const int64_t cap = (int64_t)(ctx->sm_count > 0 ? ctx->sm_count : kPlanSms) * 16;
    const int64_t blocks = (n + 255) / 256 < cap ? (n + 255) / 256 : cap;
    const auto al = [](const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; };
    if ((cols % 4) == 0 && (ld_src % 4) == 0 && (ld_dst % 4) == 0 && al(src, 16) && al(hi, 8) && al(lo, 8)) {
        const int64_t n4 = n / 4;
        const int64_t vblocks = (n4 + 255) / 256 < cap ? (n4 + 255) / 256 : cap;
        wide_split_vec_kernel<<<(unsigned)vblocks, 256, 0, ctx->stream>>>(
            src, ld_src, reinterpret_cast<__nv_bfloat16*>(hi), reinterpret_cast<__nv_bfloat16*>(lo), ld_dst, rows, cols / 4);
    } else {
        wide_split_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(
            src, ld_src, reinterpret_cast<__nv_bfloat16*>(hi), reinterpret_cast<__nv_bfloat16*>(lo), ld_dst, rows, cols);
    }
    LTCA_LAUNCH_OK(ctx, "wide_split_kernel");
    return LTCA_OK;
}

int wide_padded_keys(int Sk) { return (Sk + 7) / 8 * 8; }

size_t wide_matrix_elems(int B, int H, int Sq, int Sk) {
    return (size_t)B * H * Sq * wide_padded_keys(Sk);
}

bool wide_supported(int D, const ltca_strides& qs, const ltca_strides& ks, const ltca_strides& vs) {
    if (D < 8 || (D % 8)) return false;
    const ltca_strides* all[3] = {&qs, &ks, &vs};
    for (const ltca_strides* s : all)
        if ((s->seq % 8) || (s->head % 8) || (s->batch % 8)) return false;
    return true;
}

int wide_attn_fwd(ltca_ctx* ctx, const WideArgs& w) {
    const int Skp = wide_padded_keys(w.Sk);
    const int64_t mat = (int64_t)w.Sq * Skp;
    int rc;
    {   // scores = Q K^T, one or three terms
        Mat a[3] = {{w.qh, w.qs.seq, 0, w.qs.head, w.qs.batch},
                    {w.qh, w.qs.seq, 0, w.qs.head, w.qs.batch},
                    {w.ql, w.qs.seq, 0, w.qs.head, w.qs.batch}};
        Mat b[3] = {{w.kh, w.ks.seq, 0, w.ks.head, w.ks.batch},
                    {w.kl, w.ks.seq, 0, w.ks.head, w.ks.batch},
                    {w.kh, w.ks.seq, 0, w.ks.head, w.ks.batch}};
        const int terms = (w.ql && w.kl) ? 3 : 1;
        if ((rc = batched(ctx, w, w.Sq, w.Sk, w.D, a, b, terms, w.scores, Skp, mat, (int64_t)w.H * mat, 0))) return rc;
    }
    const SoftmaxArgs sa = softmax_args(w);
    const int64_t rows = (int64_t)w.B * w.H * w.Sq;
    const unsigned sblocks = (unsigned)((rows + 7) / 8);
    // rows of the scratch matrices start on 32 bytes (pitch a multiple of 8, bases from the 256-byte aligned carve)
    const bool vec = softmax_rows_aligned(sa);
    auto fwd_kernel = wide_softmax_fwd_kernel;
    if (vec && Skp <= 256) fwd_kernel = wide_softmax_fwd_rows_kernel<2>;
    else if (vec && Skp <= 512) fwd_kernel = wide_softmax_fwd_rows_kernel<4>;
    else if (vec && Skp <= 1024) fwd_kernel = wide_softmax_fwd_rows_kernel<8>;
    LTCA_CUDA_OK(ctx, launch_dependent(fwd_kernel, dim3(sblocks), dim3(256), 0, ctx->stream, sa));
    LTCA_LAUNCH_OK(ctx, "wide_softmax_fwd_kernel");
    if (!w.o) return LTCA_OK;
    // O = P V : P stored [Sq, Sk] (K-major), V stored [Sk, D] (N-major); terms hi hi, lo hi, hi lo
    Mat a[3] = {{w.P, Skp, 0, mat, (int64_t)w.H * mat}, {w.Plo, Skp, 0, mat, (int64_t)w.H * mat},
                {w.P, Skp, 0, mat, (int64_t)w.H * mat}};
    Mat b[3] = {{w.v, w.vs.seq, 1, w.vs.head, w.vs.batch}, {w.v, w.vs.seq, 1, w.vs.head, w.vs.batch},
                {w.vl, w.vs.seq, 1, w.vs.head, w.vs.batch}};
    const int terms = w.Plo ? (w.vl ? 3 : 2) : 1;
    return batched(ctx, w, w.Sq, w.D, w.Sk, a, b, terms, w.o, w.os.seq, w.os.head, w.os.batch, w.o_bf16);
}

int wide_attn_bwd(ltca_ctx* ctx, const WideArgs& w) {
    const int Skp = wide_padded_keys(w.Sk);
    const int64_t mat = (int64_t)w.Sq * Skp;
    const int64_t mat_b = (int64_t)w.H * mat;
    const int terms = w.Plo ? 2 : 1;                 // P (then dS) as one or two bf16 terms
    const bool full = w.Plo && w.vl && w.doutl && w.ql && w.kl;    // every operand in two terms: three-term products
    if ((w.vl || w.doutl) && !full)
        return fail(ctx, LTCA_ERR_INVALID, "low-order parts of V and dO come with those of Q, K and the probabilities");
    if (w.dS && w.Plo && !w.dSlo) return fail(ctx, LTCA_ERR_INVALID, "two-term probabilities need a two-term dS buffer");
    int rc;
    // (three-term products: hi hi, lo hi, hi lo)
    {   // dP = dO V^T : both K-major
        Mat a[3] = {{w.dout, w.dos.seq, 0, w.dos.head, w.dos.batch}, {w.doutl, w.dos.seq, 0, w.dos.head, w.dos.batch},
                    {w.dout, w.dos.seq, 0, w.dos.head, w.dos.batch}};
        Mat b[3] = {{w.v, w.vs.seq, 0, w.vs.head, w.vs.batch}, {w.v, w.vs.seq, 0, w.vs.head, w.vs.batch},
                    {w.vl, w.vs.seq, 0, w.vs.head, w.vs.batch}};
        if ((rc = batched(ctx, w, w.Sq, w.Sk, w.D, a, b, full ? 3 : 1, w.dP, Skp, mat, mat_b, 0))) return rc;
    }
    {   // dV = P^T dO : P stored [Sq, Sk] = [K, M], dO stored [Sq, D] = [K, N]
        Mat a[3] = {{w.P, Skp, 1, mat, mat_b}, {w.Plo, Skp, 1, mat, mat_b}, {w.P, Skp, 1, mat, mat_b}};
        Mat b[3] = {{w.dout, w.dos.seq, 1, w.dos.head, w.dos.batch}, {w.dout, w.dos.seq, 1, w.dos.head, w.dos.batch},
                    {w.doutl, w.dos.seq, 1, w.dos.head, w.dos.batch}};
        if ((rc = batched(ctx, w, w.Sk, w.D, w.Sq, a, b, full ? 3 : terms, w.dv, w.dvs.seq, w.dvs.head, w.dvs.batch,
                          w.grads_bf16)))
            return rc;
    }
    const SoftmaxArgs sa = softmax_args(w);
    const int64_t rows = (int64_t)w.B * w.H * w.Sq;
    const unsigned sblocks = (unsigned)((rows + 7) / 8);
    const bool vec = softmax_rows_aligned(sa) && (reinterpret_cast<uintptr_t>(sa.dP) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(sa.dS) & 7) == 0 && (reinterpret_cast<uintptr_t>(sa.dSlo) & 7) == 0;
    auto bwd_kernel = wide_softmax_bwd_kernel;
    if (vec && Skp <= 256) bwd_kernel = wide_softmax_bwd_rows_kernel<2>;
    else if (vec && Skp <= 512) bwd_kernel = wide_softmax_bwd_rows_kernel<4>;
    else if (vec && Skp <= 1024) bwd_kernel = wide_softmax_bwd_rows_kernel<8>;
    LTCA_CUDA_OK(ctx, launch_dependent(bwd_kernel, dim3(sblocks), dim3(256), 0, ctx->stream, sa));
    LTCA_LAUNCH_OK(ctx, "wide_softmax_bwd_kernel");
    {   // dQ = dS K : dS K-major, K stored [Sk, D] = [K, N]
        Mat a[3] = {{sa.dS, Skp, 0, mat, mat_b}, {sa.dSlo, Skp, 0, mat, mat_b}, {sa.dS, Skp, 0, mat, mat_b}};
        Mat b[3] = {{w.kh, w.ks.seq, 1, w.ks.head, w.ks.batch}, {w.kh, w.ks.seq, 1, w.ks.head, w.ks.batch},
                    {w.kl, w.ks.seq, 1, w.ks.head, w.ks.batch}};
        if ((rc = batched(ctx, w, w.Sq, w.D, w.Sk, a, b, full ? 3 : terms, w.dq, w.dqs.seq, w.dqs.head, w.dqs.batch,
                          w.grads_bf16)))
            return rc;
    }
    {   // dK = dS^T Q : dS stored [Sq, Sk] = [K, M], Q stored [Sq, D] = [K, N]
        Mat a[3] = {{sa.dS, Skp, 1, mat, mat_b}, {sa.dSlo, Skp, 1, mat, mat_b}, {sa.dS, Skp, 1, mat, mat_b}};
        Mat b[3] = {{w.qh, w.qs.seq, 1, w.qs.head, w.qs.batch}, {w.qh, w.qs.seq, 1, w.qs.head, w.qs.batch},
                    {w.ql, w.qs.seq, 1, w.qs.head, w.qs.batch}};
        if ((rc = batched(ctx, w, w.Sk, w.D, w.Sq, a, b, full ? 3 : terms, w.dk, w.dks.seq, w.dks.head, w.dks.batch,
                          w.grads_bf16)))
            return rc;
    }
    return LTCA_OK;
}

}  // namespace ltca
