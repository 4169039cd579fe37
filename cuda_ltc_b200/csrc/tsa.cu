// TimeSelfAttention module: out = LayerNorm(x + MHA(x)) and its backward, as the reference's
// CuDNNTimeSelfAttention computes them (reference src/ml/cudnn_time_self_attention.cu:211-368
// with the attention configured by include/cuDNN_ops.h:152-178).
//
// Data flow of the forward (all buffers fp32, row = one (batch, time) position):
//   x [rows,E] --Wq,Wk,Wv--> q,k,v [rows,H*W] --attention core--> ctx [rows,H*W] --Wo--> y [rows,E]
//   out = LayerNorm(y + x)        (residual and LayerNorm fused into one row pass)
// The attention core reads q/k/v and writes ctx through strided [B,H,S,W] views of the
// row-major projection buffers, so the reference's reshape kernels
// (src/ml/flash_attention.cu:402-455) have no counterpart here.
//
// Two pipelines:
//   - exact (LTCA_MODE_FP32, or shapes the tensor-pipe attention kernels do not cover): fp32 FMA GEMMs,
//     fp32 buffers between the kernels;
//   - tensor pipe (other modes): x, dy and the weights are rounded to bf16 once, every projection is
//     a tcgen05 GEMM (gemm_sm100.cu), q / k / v / ctx and their gradients stay in bf16 between the
//     kernels (the attention kernels read them through strides, nothing is packed or permuted), Q, K
//     and V share one launch, dx is one GEMM over the three (dq, W^T) pairs, the weight gradients
//     split their long contraction (batch x time) across CTAs and are summed in a fixed order.
// Backward follows the reference:
// the incoming gradient passes through LayerNorm and the residual unchanged
// (src/ml/cudnn_time_self_attention.cu:291-299), dx = dQ Wq^T + dK Wk^T + dV Wv^T.
#include "gemm_sm100.h"
#include "attn_wide.h"
#include "host_common.h"
#include "sm100_ptx.cuh"

namespace ltca {

namespace {

constexpr int kGT = 128;    // GEMM tile (M and N)
constexpr int kGK = 16;     // GEMM K step
constexpr int kGP = 4;      // row padding of the shared tiles (floats)

// C[M,N] (+)= op(A) op(B) (+ bias[N]); row-major storage.
//   ta == 0: A is [M,K] (lda = K-extent stride), ta == 1: A is stored [K,M].
//   tb == 0: B is [K,N],                          tb == 1: B is stored [N,K].
struct GemmArgs {
    const float *A, *B, *bias;
    float* C;
    int M, N, K;
    int lda, ldb, ldc;
    int ta, tb, accumulate;
    int kper;          // contraction extent one CTA covers (blockIdx.z selects the slice)
    float* partial;    // [gridDim.z][M][N] slice results when the contraction is split, else null
};

// Exact-mode projection GEMM (fp32 FMA, the arithmetic of the reference's cublasSgemm with tensor cores
// off, src/ml/flash_attention.cu:531-536): 128 x 128 tile per CTA, 16 x 16 threads with 8 x 8 outputs each
// (two 4-wide groups 64 apart per dimension, so shared-memory reads are conflict-free float4 loads), the
// next K slab is fetched from global memory into registers while the current one is multiplied.
__global__ void __launch_bounds__(256) gemm_fp32_kernel(const GemmArgs g) {
    __shared__ __align__(16) float As[kGK][kGT + kGP];
    __shared__ __align__(16) float Bs[kGK][kGT + kGP];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * kGT, n0 = blockIdx.x * kGT;
    const int kbeg = blockIdx.z * g.kper;
    const int kend = min(g.K, kbeg + g.kper);
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    // Each thread moves 8 elements of the A slab and 8 of the B slab.  With the contraction index
    // contiguous in memory (ta == 0 / tb == 1) a thread takes elements (r, k..k+7) of one row half; with the
    // M / N index contiguous (ta == 1 / tb == 0) it takes (k, c..c+7) of one K row.
    float ra[8], rb[8];
    auto fetch = [&](int k0) {
        if (!g.ta) {
            const int r = threadIdx.x >> 1, kk = (threadIdx.x & 1) * 8;
            const int gm = m0 + r;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int gk = k0 + kk + e;
                ra[e] = (gm < g.M && gk < kend) ? __ldg(g.A + (int64_t)gm * g.lda + gk) : 0.f;
            }
        } else {
            const int kk = threadIdx.x >> 4, c = (threadIdx.x & 15) * 8;
            const int gk = k0 + kk;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int gm = m0 + c + e;
                ra[e] = (gm < g.M && gk < kend) ? __ldg(g.A + (int64_t)gk * g.lda + gm) : 0.f;
            }
        }
        if (g.tb) {
            const int r = threadIdx.x >> 1, kk = (threadIdx.x & 1) * 8;
            const int gn = n0 + r;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int gk = k0 + kk + e;
                rb[e] = (gn < g.N && gk < kend) ? __ldg(g.B + (int64_t)gn * g.ldb + gk) : 0.f;
            }
        } else {
            const int kk = threadIdx.x >> 4, c = (threadIdx.x & 15) * 8;
            const int gk = k0 + kk;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int gn = n0 + c + e;
                rb[e] = (gn < g.N && gk < kend) ? __ldg(g.B + (int64_t)gk * g.ldb + gn) : 0.f;
            }
        }
    };
    auto stash = [&]() {
        if (!g.ta) {
            const int r = threadIdx.x >> 1, kk = (threadIdx.x & 1) * 8;
#pragma unroll
            for (int e = 0; e < 8; ++e) As[kk + e][r] = ra[e];
        } else {
            const int kk = threadIdx.x >> 4, c = (threadIdx.x & 15) * 8;
#pragma unroll
            for (int e = 0; e < 8; ++e) As[kk][c + e] = ra[e];
        }
        if (g.tb) {
            const int r = threadIdx.x >> 1, kk = (threadIdx.x & 1) * 8;
#pragma unroll
            for (int e = 0; e < 8; ++e) Bs[kk + e][r] = rb[e];
        } else {
            const int kk = threadIdx.x >> 4, c = (threadIdx.x & 15) * 8;
#pragma unroll
            for (int e = 0; e < 8; ++e) Bs[kk][c + e] = rb[e];
        }
    };

    fetch(kbeg);
    for (int k0 = kbeg; k0 < kend; k0 += kGK) {
        stash();
        __syncthreads();
        if (k0 + kGK < kend) fetch(k0 + kGK);
#pragma unroll
        for (int k = 0; k < kGK; ++k) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[k][4 * ty]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[k][64 + 4 * ty]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[k][4 * tx]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[k][64 + 4 * tx]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int gm = m0 + (i < 4 ? 4 * ty + i : 64 + 4 * ty + i - 4);
        if (gm >= g.M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int gn = n0 + (j < 4 ? 4 * tx + j : 64 + 4 * tx + j - 4);
            if (gn >= g.N) continue;
            float v = acc[i][j];
            if (g.partial) {
                g.partial[((int64_t)blockIdx.z * g.M + gm) * g.N + gn] = v;
                continue;
            }
            if (g.bias) v += g.bias[gn];
            float* c = g.C + (int64_t)gm * g.ldc + gn;
            *c = g.accumulate ? *c + v : v;
        }
    }
}

// C[m][n] = sum over slices, in slice order, of partial[z][m][n]: the second pass of a split contraction.
__global__ void gemm_fp32_reduce_kernel(const float* __restrict__ partial, float* __restrict__ C, int M,
                                        int N, int ldc, int slices) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)M * N) return;
    float v = 0.f;
    for (int z = 0; z < slices; ++z) v += partial[(int64_t)z * M * N + i];
    C[(i / N) * ldc + (i % N)] = v;
}

int gemm(ltca_ctx* ctx, const float* A, const float* B, const float* bias, float* C, int M, int N,
         int K, int lda, int ldb, int ldc, int ta, int tb, int accumulate) {
    GemmArgs g{A, B, bias, C, M, N, K, lda, ldb, ldc, ta, tb, accumulate, K, nullptr};
    dim3 grid((N + kGT - 1) / kGT, (M + kGT - 1) / kGT);
    gemm_fp32_kernel<<<grid, 256, 0, ctx->stream>>>(g);
    LTCA_LAUNCH_OK(ctx, "gemm_fp32_kernel");
    return LTCA_OK;
}

// A weight-gradient product (few output tiles, long contraction): the contraction is cut into slices, one
// CTA per (tile, slice), and the slices are summed in a fixed order, so the result does not depend on
// the launch.  `scratch` holds the slice results; with too little of it the product runs unsplit.
int gemm_long_k(ltca_ctx* ctx, const float* A, const float* B, float* C, int M, int N, int K, int lda,
                int ldb, int ldc, int ta, int tb, float* scratch, size_t scratch_bytes) {
    const int tiles = ((N + kGT - 1) / kGT) * ((M + kGT - 1) / kGT);
    int slices = (2 * ctx->sm_count + tiles - 1) / tiles;
    const size_t one = (size_t)M * N * sizeof(float);
    if ((size_t)slices * one > scratch_bytes) slices = (int)(scratch_bytes / one);
    if (slices > K / (4 * kGK)) slices = K / (4 * kGK);
    if (slices < 2) return gemm(ctx, A, B, nullptr, C, M, N, K, lda, ldb, ldc, ta, tb, 0);
    int kper = (K + slices - 1) / slices;
    kper = (kper + kGK - 1) / kGK * kGK;
    slices = (K + kper - 1) / kper;
    GemmArgs g{A, B, nullptr, C, M, N, K, lda, ldb, ldc, ta, tb, 0, kper, scratch};
    dim3 grid((N + kGT - 1) / kGT, (M + kGT - 1) / kGT, slices);
    gemm_fp32_kernel<<<grid, 256, 0, ctx->stream>>>(g);
    LTCA_LAUNCH_OK(ctx, "gemm_fp32_kernel");
    const int64_t n = (int64_t)M * N;
    gemm_fp32_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(scratch, C, M, N, ldc,
                                                                                  slices);
    LTCA_LAUNCH_OK(ctx, "gemm_fp32_reduce_kernel");
    return LTCA_OK;
}

// out[row] = LayerNorm(y[row] (+ x[row])) or just the sum / a copy; one warp per row.
__global__ void residual_layer_norm_kernel(const float* __restrict__ y, const float* __restrict__ x,
                                           const float* __restrict__ gamma,
                                           const float* __restrict__ beta, float* __restrict__ out,
                                           int64_t rows, int E, int use_res, int use_ln, float eps) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float* yr = y + row * E;
    const float* xr = x + row * E;
    float* outr = out + row * E;
    const uintptr_t align_bits = reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(x) |
                                 reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(gamma) |
                                 reinterpret_cast<uintptr_t>(beta);
    if (use_ln && (E & 127) == 0 && E <= 1024 && (align_bits & 15) == 0) {
        // the row stays in registers: one read of y and x, one write of the result
        float4 v[8];
        const int n4 = E >> 7;                        // float4 per lane
        float sum4 = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (i < n4) {
                v[i] = __ldg(reinterpret_cast<const float4*>(yr) + lane + 32 * i);
                if (use_res) {
                    const float4 r = __ldg(reinterpret_cast<const float4*>(xr) + lane + 32 * i);
                    v[i].x += r.x; v[i].y += r.y; v[i].z += r.z; v[i].w += r.w;
                }
                sum4 += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum4 += __shfl_xor_sync(0xffffffffu, sum4, o);
        const float mean4 = sum4 / E;
        float var4 = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (i < n4) {
                const float a = v[i].x - mean4, b = v[i].y - mean4, c = v[i].z - mean4, d = v[i].w - mean4;
                var4 = fmaf(a, a, var4); var4 = fmaf(b, b, var4); var4 = fmaf(c, c, var4); var4 = fmaf(d, d, var4);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) var4 += __shfl_xor_sync(0xffffffffu, var4, o);
        const float inv4 = rsqrtf(var4 / E + eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (i < n4) {
                float4 gm = make_float4(1.f, 1.f, 1.f, 1.f), bt = make_float4(0.f, 0.f, 0.f, 0.f);
                if (gamma) gm = __ldg(reinterpret_cast<const float4*>(gamma) + lane + 32 * i);
                if (beta) bt = __ldg(reinterpret_cast<const float4*>(beta) + lane + 32 * i);
                float4 o4;
                o4.x = (v[i].x - mean4) * inv4 * gm.x + bt.x;
                o4.y = (v[i].y - mean4) * inv4 * gm.y + bt.y;
                o4.z = (v[i].z - mean4) * inv4 * gm.z + bt.z;
                o4.w = (v[i].w - mean4) * inv4 * gm.w + bt.w;
                reinterpret_cast<float4*>(outr)[lane + 32 * i] = o4;
            }
        }
        return;
    }
    float sum = 0.f;
    for (int i = lane; i < E; i += 32) {
        const float v = yr[i] + (use_res ? xr[i] : 0.f);
        outr[i] = v;
        sum += v;
    }
    if (!use_ln) return;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / E;
    float var = 0.f;
    for (int i = lane; i < E; i += 32) {
        const float d = outr[i] - mean;
        var = fmaf(d, d, var);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
    const float inv_std = rsqrtf(var / E + eps);
    for (int i = lane; i < E; i += 32)
        outr[i] = (outr[i] - mean) * inv_std * (gamma ? gamma[i] : 1.f) + (beta ? beta[i] : 0.f);
}


// ---- pieces of the FlashAttention form: dropout, LayerNorm backward, column sums -----------------

// u in [0,1) from (seed, element index): splitmix64 finaliser, top 24 bits.  The same function runs on the host
// in the oracle, so masks can be compared element by element.
__host__ __device__ inline float dropout_uniform(uint64_t seed, uint64_t idx) {
    uint64_t z = seed + (idx + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// dst[i] = keep(i) ? src[i] / (1 - p) : 0   (inverted dropout, reference src/ml/flash_attention.cu:380-399;
// the reference draws from curand with a time-dependent offset, so only the distribution can match)
__global__ void dropout_kernel(const float* __restrict__ src, float* __restrict__ dst, int64_t n, float p,
                               uint64_t seed) {
    const float scale = 1.0f / (1.0f - p);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = dropout_uniform(seed, (uint64_t)i) >= p ? src[i] * scale : 0.f;
}

// LayerNorm backward, one warp per row.  g = gradient at the LayerNorm output, x = its input.
//   dx = inv_std * (g*gamma - mean(g*gamma) - xhat * mean(g*gamma*xhat))  (+ res[row] when res != null)
// prod (optional) receives g * xhat, whose column sums are dgamma.
__global__ void layer_norm_bwd_kernel(const float* __restrict__ g, const float* __restrict__ x,
                                      const float* __restrict__ gamma, const float* __restrict__ res,
                                      float* __restrict__ dx, float* __restrict__ prod, int64_t rows, int E,
                                      float eps) {
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float* xr = x + row * E;
    const float* gr = g + row * E;
    float sum = 0.f;
    for (int i = lane; i < E; i += 32) sum += xr[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / E;
    float var = 0.f;
    for (int i = lane; i < E; i += 32) { const float d = xr[i] - mean; var = fmaf(d, d, var); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
    const float inv_std = rsqrtf(var / E + eps);
    float m1 = 0.f, m2 = 0.f;
    for (int i = lane; i < E; i += 32) {
        const float xh = (xr[i] - mean) * inv_std;
        const float gg = gr[i] * gamma[i];
        m1 += gg;
        m2 = fmaf(gg, xh, m2);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        m1 += __shfl_xor_sync(0xffffffffu, m1, o);
        m2 += __shfl_xor_sync(0xffffffffu, m2, o);
    }
    m1 /= E; m2 /= E;
    for (int i = lane; i < E; i += 32) {
        const float xh = (xr[i] - mean) * inv_std;
        const float gi = gr[i];
        float v = inv_std * (gi * gamma[i] - m1 - xh * m2);
        if (res) v += res[row * E + i];
        if (prod) prod[row * E + i] = gi * xh;          // may alias g: each element is read before it is written
        dx[row * E + i] = v;
    }
}

// Column sums of a [rows, cols] matrix in two fixed-order stages (no atomics): kColChunks row chunks, then
// the chunks.
constexpr int kColChunks = 64;
__device__ __forceinline__ float ld_f(const float* p) { return *p; }
__device__ __forceinline__ float ld_f(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__global__ void column_sum_partial_kernel(const T* __restrict__ src, int64_t ld, int64_t rows, int cols,
                                          float* __restrict__ partial) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    const int64_t per = (rows + kColChunks - 1) / kColChunks;
    const int64_t r0 = blockIdx.y * per, r1 = r0 + per < rows ? r0 + per : rows;
    float acc = 0.f;
    for (int64_t r = r0; r < r1; ++r) acc += ld_f(src + r * ld + c);
    partial[(int64_t)blockIdx.y * cols + c] = acc;
}
__global__ void column_sum_final_kernel(const float* __restrict__ partial, int cols, float* __restrict__ dst) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float acc = 0.f;
    for (int k = 0; k < kColChunks; ++k) acc += partial[(int64_t)k * cols + c];
    dst[c] = acc;
}
template <typename T>
int column_sum(ltca_ctx* ctx, const T* src, int64_t ld, int64_t rows, int cols, float* dst, float* scratch) {
    dim3 grid((cols + 127) / 128, kColChunks);
    column_sum_partial_kernel<T><<<grid, 128, 0, ctx->stream>>>(src, ld, rows, cols, scratch);
    LTCA_LAUNCH_OK(ctx, "column_sum_partial_kernel");
    column_sum_final_kernel<<<(cols + 127) / 128, 128, 0, ctx->stream>>>(scratch, cols, dst);
    LTCA_LAUNCH_OK(ctx, "column_sum_final_kernel");
    return LTCA_OK;
}
size_t colsum_scratch_bytes(const ltca_tsa_params* t) {
    const int hw = t->H * t->head_width;
    return align_up((size_t)kColChunks * (hw > t->E ? hw : t->E) * sizeof(float), 256);
}

struct Plan {
    int64_t rows;
    int HW;
    size_t buf;          // bytes of one [rows, HW] fp32 buffer
    size_t lse;          // bytes of lse
    size_t y;            // bytes of one [rows, E] buffer
    size_t attn_fwd, attn_bwd;
};

void fill_attn(const ltca_tsa_params* t, ltca_attn_params* a) {
    memset(a, 0, sizeof(*a));
    const int HW = t->H * t->head_width;
    a->B = t->B; a->H = t->H; a->Sq = t->S; a->Sk = t->S; a->D = t->head_width;
    a->dtype = LTCA_F32;
    a->mode = t->mode == LTCA_MODE_SPLIT ? LTCA_MODE_AUTO : t->mode;     // the module has no split mode of its own
    a->causal = t->causal;
    a->scale = t->scale;
    a->score_clamp = t->score_clamp;
    ltca_strides st;
    st.head = t->head_width;
    if (t->time_major) { st.batch = HW; st.seq = (int64_t)t->B * HW; }
    else               { st.batch = (int64_t)t->S * HW; st.seq = HW; }
    a->q_strides = a->k_strides = a->v_strides = a->o_strides = st;
    a->do_strides = a->dq_strides = a->dk_strides = a->dv_strides = st;
    a->keep_mask = t->keep_mask;
    a->kv_len = t->kv_len;
    // the module's gradients stay bit-identical from run to run (the reference's tests pin backward
    // repeatability on the module, src/ml/time_self_attention_test.cu:799-838)
    a->bwd_deterministic = 1;
}

int make_plan(const ltca_tsa_params* t, Plan* pl) {
    pl->rows = (int64_t)t->B * t->S;
    pl->HW = t->H * t->head_width;
    pl->buf = align_up((size_t)pl->rows * pl->HW * sizeof(float), 256);
    pl->lse = align_up((size_t)t->B * t->H * t->S * sizeof(float), 256);
    pl->y = align_up((size_t)pl->rows * t->E * sizeof(float), 256);
    ltca_attn_params a;
    fill_attn(t, &a);
    // pointers only need to be non-null for the size queries
    int rc = ltca_attn_workspace_bytes(&a, 0, &pl->attn_fwd);
    if (rc) return rc;
    return ltca_attn_workspace_bytes(&a, 1, &pl->attn_bwd);
}

int check(ltca_ctx* ctx, const ltca_tsa_params* t) {
    if (!ctx) return LTCA_ERR_INVALID;
    if (!t) return fail(ctx, LTCA_ERR_INVALID, "null parameter block");
    if (t->B < 1 || t->S < 1 || t->E < 1 || t->H < 1 || t->head_width < 1)
        return fail(ctx, LTCA_ERR_INVALID, "B, S, E, H, head_width must be positive");
    // same validation as the reference constructor (src/ml/time_self_attention.cu:25-35)
    if (t->E % t->H != 0)
        return fail(ctx, LTCA_ERR_INVALID, "input_dim (%d) must be divisible by num_heads (%d)",
                    t->E, t->H);
    if (!t->x || !t->wq || !t->wk || !t->wv || !t->wo)
        return fail(ctx, LTCA_ERR_INVALID, "x and the four weight matrices must be non-null");
    if (!(t->scale > 0.f)) return fail(ctx, LTCA_ERR_INVALID, "scale must be positive");
    if (reinterpret_cast<uintptr_t>(t->workspace) & 255)
        return fail(ctx, LTCA_ERR_INVALID, "workspace must be 256-byte aligned");
    if (t->reuse_forward && !t->saved)
        return fail(ctx, LTCA_ERR_INVALID, "reuse_forward needs the saved block of the forward call");
    if (t->saved) {
        if (t->pre_norm)
            return fail(ctx, LTCA_ERR_UNSUPPORTED, "the saved block is not available in the pre_norm form");
        if (reinterpret_cast<uintptr_t>(t->saved) & 255)
            return fail(ctx, LTCA_ERR_INVALID, "saved must be 256-byte aligned");
        size_t need = 0;
        int rc = ltca_tsa_saved_bytes(t, &need);
        if (rc) return fail(ctx, rc, "bad shape for the saved block");
        if (t->saved_bytes < need)
            return fail(ctx, LTCA_ERR_WORKSPACE, "the saved block needs %zu bytes", need);
    }
    if (t->weight_cache) {
        if (reinterpret_cast<uintptr_t>(t->weight_cache) & 255)
            return fail(ctx, LTCA_ERR_INVALID, "weight_cache must be 256-byte aligned");
        size_t need = 0;
        int rc = ltca_tsa_weight_cache_bytes(t, &need);
        if (rc) return fail(ctx, rc, "bad shape for the weight cache");
        if (t->weight_cache_bytes < need)
            return fail(ctx, LTCA_ERR_WORKSPACE, "the weight cache needs %zu bytes", need);
    }
    return LTCA_OK;
}

// Projections + attention forward into workspace; returns pointers into it.
struct FwdBufs { float *q, *k, *v, *ctx, *lse; char* rest; };

// With a caller-kept `saved` block (ltca_tsa_params.saved) q, k, v, ctx and lse live there and the
// workspace only holds the attention scratch; with reuse_forward they are taken as they are.
int forward_core(ltca_ctx* ctx, const ltca_tsa_params* t, const Plan& pl, char* w, FwdBufs* fb,
                 size_t attn_ws_bytes) {
    char* rest = w;
    if (t->saved) w = reinterpret_cast<char*>(t->saved);
    fb->q = reinterpret_cast<float*>(w);   w += pl.buf;
    fb->k = reinterpret_cast<float*>(w);   w += pl.buf;
    fb->v = reinterpret_cast<float*>(w);   w += pl.buf;
    fb->ctx = reinterpret_cast<float*>(w); w += pl.buf;
    fb->lse = reinterpret_cast<float*>(w); w += pl.lse;
    fb->rest = t->saved ? rest : w;
    if (t->saved && t->reuse_forward) return LTCA_OK;
    const int rows = (int)pl.rows, E = t->E, HW = pl.HW;
    int rc;
    if ((rc = gemm(ctx, t->x, t->wq, t->bq, fb->q, rows, HW, E, E, HW, HW, 0, 0, 0))) return rc;
    if ((rc = gemm(ctx, t->x, t->wk, t->bk, fb->k, rows, HW, E, E, HW, HW, 0, 0, 0))) return rc;
    if ((rc = gemm(ctx, t->x, t->wv, t->bv, fb->v, rows, HW, E, E, HW, HW, 0, 0, 0))) return rc;
    ltca_attn_params a;
    fill_attn(t, &a);
    a.q = fb->q; a.k = fb->k; a.v = fb->v; a.o = fb->ctx; a.lse = fb->lse;
    a.workspace = attn_ws_bytes ? fb->rest : nullptr;
    a.workspace_bytes = attn_ws_bytes;
    rc = ltca_attn_fwd(ctx, &a);
    return rc;
}

// ---- tensor-pipe pipeline ---------------------------------------------------------------------

void fill_attn_bf16(const ltca_tsa_params* t, ltca_attn_params* a) {
    fill_attn(t, a);
    a->dtype = LTCA_BF16;
    a->mode = LTCA_MODE_BF16;
}

// A forward that leaves something for the backward (its intermediates, or the weights' copies) takes the pipeline
// the backward will take, so that both calls agree on what the blocks hold.
bool keeps_for_backward(const ltca_tsa_params* t) { return t->saved != nullptr || t->weight_cache != nullptr; }

// Whether the attention core of the tensor pipeline is the materialised-score path (attn_wide_sm100.cu): head
// widths the streaming kernels do not cover.  Taken for heads wider than 128 (the reference's configuration gives
// every head the model's width) and, on explicit request (LTCA_MODE_BF16), for any width that is a multiple of 8;
// narrow heads under LTCA_MODE_AUTO stay on the exact pipeline, whose handful of small kernels is faster there.
bool use_wide(const ltca_tsa_params* t, bool /*backward*/) {
    if (t->mode == LTCA_MODE_FP32) return false;
    if (t->head_width < 8 || (t->head_width % 8)) return false;
    ltca_attn_params a;
    fill_attn_bf16(t, &a);
    // one choice for forward and backward calls, so that a forward call computes what the backward recomputes
    // (width 128 has a streaming forward but no streaming backward: it takes this path for both)
    if (attn_fwd_sm100_supported(&a) && attn_bwd_sm100_supported(&a)) return false;
    return t->mode == LTCA_MODE_BF16 || t->head_width > 128;
}

// Whether the module runs on the tensor pipe: the caller allows it, an attention path on the tensor pipe covers
// the head width, and the bf16 rows keep the 16-byte pitch TMA needs.
bool use_tensor(const ltca_tsa_params* t, bool backward) {
    if (t->mode == LTCA_MODE_FP32) return false;
    if ((t->H * t->head_width) % 8) return false;
    if (use_wide(t, backward)) return true;
    ltca_attn_params a;
    fill_attn_bf16(t, &a);
    if (!attn_fwd_sm100_supported(&a)) return false;
    if (backward && !attn_bwd_sm100_supported(&a)) return false;
    return true;
}

struct TPlan {
    int64_t rows;
    int HW, Ep;
    size_t xb, w_in, w_out, act, lse, y;
    size_t attn_fwd, attn_bwd, partial;
    int ks_in, ks_out;
    // materialised-score path: low-order parts of x, Wq, Wk, q, k; fp32 projection scratch; score matrices
    bool wide;
    size_t mat32, mat16;
};

int make_tplan(const ltca_tsa_params* t, TPlan* pl, bool backward) {
    pl->rows = (int64_t)t->B * t->S;
    pl->HW = t->H * t->head_width;
    pl->Ep = (t->E + 7) / 8 * 8;
    pl->xb = align_up((size_t)pl->rows * pl->Ep * 2, 256);
    pl->w_in = align_up((size_t)t->E * pl->HW * 2, 256);
    pl->w_out = align_up((size_t)pl->HW * pl->Ep * 2, 256);
    pl->act = align_up((size_t)pl->rows * pl->HW * 2, 256);
    pl->lse = align_up((size_t)t->B * t->H * t->S * sizeof(float), 256);
    pl->y = align_up((size_t)pl->rows * t->E * sizeof(float), 256);
    pl->wide = use_wide(t, backward);
    pl->mat32 = pl->mat16 = 0;
    pl->attn_fwd = pl->attn_bwd = 0;
    int rc;
    if (pl->wide) {
        const size_t elems = wide_matrix_elems(t->B, t->H, t->S, t->S);
        pl->mat32 = align_up(elems * sizeof(float), 256);
        pl->mat16 = align_up(elems * 2, 256);
    } else {
        ltca_attn_params a;
        fill_attn_bf16(t, &a);
        if ((rc = ltca_attn_workspace_bytes(&a, 0, &pl->attn_fwd))) return rc;
        if ((rc = ltca_attn_workspace_bytes(&a, 1, &pl->attn_bwd))) return rc;
    }
    const int rows = (int)pl->rows;
    pl->ks_in = gemm_sm100_pick_ksplit(t->E, pl->HW, rows, 3, kPlanSms);
    pl->ks_out = gemm_sm100_pick_ksplit(pl->HW, t->E, rows, 1, kPlanSms);
    const size_t p_in = gemm_sm100_partial_bytes(t->E, pl->HW, 3, pl->ks_in);
    const size_t p_out = gemm_sm100_partial_bytes(pl->HW, t->E, 1, pl->ks_out);
    pl->partial = p_in > p_out ? p_in : p_out;
    return LTCA_OK;
}

// Extra scratch of the materialised-score path: x_lo, Wq_lo, Wk_lo, q_lo, k_lo, the fp32 projection result that is
// split into q (then k), the raw scores and the probabilities; the backward adds dP.
// What of it a forward keeps for the backward: the low-order parts, the raw scores and the probabilities.
size_t wide_kept(const TPlan& pl) { return pl.wide ? pl.xb + 2 * pl.w_in + 2 * pl.act + pl.mat32 + pl.mat16 : 0; }
size_t wide_extra(const TPlan& pl, int which) {
    if (!pl.wide) return 0;
    return wide_kept(pl) + (which == 0 ? 0 : pl.mat32 + pl.mat16);     // backward: dP and dS
}

size_t tensor_workspace(const TPlan& pl, int which) {
    // x, the four weight matrices, q, k, v, ctx, lse
    size_t n = pl.xb + 3 * pl.w_in + pl.w_out + 4 * pl.act + pl.lse + wide_extra(pl, which);
    if (which == 0) return n + pl.y + pl.attn_fwd;
    n += pl.xb + 4 * pl.act;                       // dy, dctx, dq, dk, dv
    n += pl.attn_fwd > pl.attn_bwd ? pl.attn_fwd : pl.attn_bwd;
    return n + pl.partial;
}

size_t tensor_saved_bytes(const TPlan& pl) {
    return pl.xb + 3 * pl.w_in + pl.w_out + 4 * pl.act + pl.lse + wide_kept(pl);
}

struct TBufs {
    void *xb, *wq, *wk, *wv, *wo, *q, *k, *v, *ctx;
    float* lse;
    char* rest;
    // materialised-score path
    void *xl, *wql, *wkl, *ql, *kl, *P, *dS;
    float *scores, *dP;
};

// The attention problem of the module for the materialised-score path (bf16 views of the projection outputs).
void fill_wide(const ltca_tsa_params* t, const TBufs& tb, WideArgs* w) {
    ltca_attn_params a;
    fill_attn_bf16(t, &a);
    w->B = t->B; w->H = t->H; w->Sq = t->S; w->Sk = t->S; w->D = t->head_width;
    w->causal = t->causal; w->scale = t->scale; w->clamp = t->score_clamp;
    w->keep_mask = t->keep_mask; w->kv_len = t->kv_len;
    w->qh = tb.q; w->ql = tb.ql; w->kh = tb.k; w->kl = tb.kl; w->v = tb.v;
    w->qs = w->ks = w->vs = w->os = a.q_strides;
    w->dos = w->dqs = w->dks = w->dvs = a.q_strides;
    w->o = tb.ctx; w->o_bf16 = 1; w->lse = tb.lse;
    w->scores = tb.scores; w->P = tb.P; w->dP = tb.dP; w->dS = tb.dS;
    w->grads_bf16 = 1;
}

// bf16 copies, fused Q/K/V projection, attention forward.
// `also_src` / `also_dst`: one more [rows, E] fp32 matrix (the backward's dy) to be rounded to bf16 by the same launch
// that rounds x and the weights; *also_done says whether that happened (not on the paths that convert otherwise
// or not at all).
int tensor_forward_core(ltca_ctx* ctx, const ltca_tsa_params* t, const TPlan& pl, char* w, TBufs* tb, int which,
                        const float* also_src = nullptr, void* also_dst = nullptr, bool* also_done = nullptr) {
    char* rest = w;
    const bool saved = t->saved != nullptr;
    if (saved) w = reinterpret_cast<char*>(t->saved);
    tb->xb = w;  w += pl.xb;
    tb->wq = w;  w += pl.w_in;
    tb->wk = w;  w += pl.w_in;
    tb->wv = w;  w += pl.w_in;
    tb->wo = w;  w += pl.w_out;
    tb->q = w;   w += pl.act;
    tb->k = w;   w += pl.act;
    tb->v = w;   w += pl.act;
    tb->ctx = w; w += pl.act;
    tb->lse = reinterpret_cast<float*>(w); w += pl.lse;
    if (pl.wide) {
        tb->xl = w;  w += pl.xb;
        tb->wql = w; w += pl.w_in;
        tb->wkl = w; w += pl.w_in;
        tb->ql = w;  w += pl.act;
        tb->kl = w;  w += pl.act;
        tb->scores = reinterpret_cast<float*>(w); w += pl.mat32;
        tb->P = w;   w += pl.mat16;
    }
    char* r = saved ? rest : w;                        // what follows is never kept
    if (pl.wide) {
        tb->dP = nullptr; tb->dS = nullptr;
        if (which != 0) {
            // dS gets its own buffer: the probabilities stay valid for the next backward call from the same forward
            tb->dP = reinterpret_cast<float*>(r); r += pl.mat32;
            tb->dS = r; r += pl.mat16;
        }
    }
    tb->rest = r;
    // the weights' copies live in the caller's cache when there is one
    const bool cached = t->weight_cache != nullptr;
    if (cached) {
        char* c = reinterpret_cast<char*>(t->weight_cache);
        tb->wq = c;  c += pl.w_in;
        tb->wk = c;  c += pl.w_in;
        tb->wv = c;  c += pl.w_in;
        tb->wo = c;  c += pl.w_out;
        if (pl.wide) { tb->wql = c; c += pl.w_in; tb->wkl = c; c += pl.w_in; }
    }
    const bool convert_weights = !(cached && t->weight_cache_valid);
    if (saved && t->reuse_forward) return LTCA_OK;
    const int E = t->E, HW = pl.HW, Ep = pl.Ep;
    int rc;
    {   // x, the four weight matrices unless their copies are kept, and the caller's extra matrix are rounded to
        // bf16 by one launch.  On the written-out-score path the operands of the products whose rounding would
        // reach the scores - x, Wq, Wk here, q and k below - get a second term.
        const float* src[6] = {t->x, t->wq, t->wk, t->wv, t->wo, nullptr};
        void* dst[6] = {tb->xb, tb->wq, tb->wk, tb->wv, tb->wo, nullptr};
        void* lo[6] = {pl.wide ? tb->xl : nullptr, pl.wide ? tb->wql : nullptr, pl.wide ? tb->wkl : nullptr,
                       nullptr, nullptr, nullptr};
        int64_t ld_src[6] = {E, HW, HW, HW, E, E}, ld_dst[6] = {Ep, HW, HW, HW, Ep, Ep};
        int64_t nrows[6] = {pl.rows, E, E, E, HW, pl.rows};
        int ncols[6] = {E, HW, HW, HW, E, E};
        int n = convert_weights ? 5 : 1;
        if (also_src) {
            src[n] = also_src; dst[n] = also_dst; lo[n] = nullptr;
            ld_src[n] = E; ld_dst[n] = Ep; nrows[n] = pl.rows; ncols[n] = E;
            ++n;
            if (also_done) *also_done = true;
        }
        if ((rc = convert_many_bf16(ctx, n, src, ld_src, dst, ld_dst, nrows, ncols, lo))) return rc;
    }
    if (pl.wide) {
        const void* whi[2] = {tb->wq, tb->wk};
        const void* wlo[2] = {tb->wql, tb->wkl};
        void* ohi[2] = {tb->q, tb->k};
        void* olo[2] = {tb->ql, tb->kl};
        const float* bias[2] = {t->bq, t->bk};
        for (int i = 0; i < 2; ++i) {
            // x W = x_hi W_hi + x_hi W_lo + x_lo W_hi in one fp32 accumulator, which the epilogue writes as two
            // bf16 terms
            GemmProblem gp;
            gp.M = (int)pl.rows; gp.N = HW; gp.K = E;
            gp.n_sum = 3;
            gp.a[0] = GemmOperand{tb->xb, Ep, 0}; gp.b[0] = GemmOperand{whi[i], HW, 1};
            gp.a[1] = GemmOperand{tb->xb, Ep, 0}; gp.b[1] = GemmOperand{wlo[i], HW, 1};
            gp.a[2] = GemmOperand{tb->xl, Ep, 0}; gp.b[2] = GemmOperand{whi[i], HW, 1};
            gp.c[0] = ohi[i];
            gp.c_lo = olo[i];
            gp.out_bf16 = 1;
            gp.bias[0] = bias[i];
            gp.ldc = HW;
            if ((rc = gemm_sm100(ctx, gp))) return rc;
        }
        {
            GemmProblem gp;
            gp.M = (int)pl.rows; gp.N = HW; gp.K = E;
            gp.a[0] = GemmOperand{tb->xb, Ep, 0};
            gp.b[0] = GemmOperand{tb->wv, HW, 1};
            gp.c[0] = tb->v;
            gp.bias[0] = t->bv;
            gp.ldc = HW;
            gp.out_bf16 = 1;
            if ((rc = gemm_sm100(ctx, gp))) return rc;
        }
        WideArgs wa;
        fill_wide(t, *tb, &wa);
        return wide_attn_fwd(ctx, wa);
    }
    GemmProblem gp;
    gp.M = (int)pl.rows; gp.N = HW; gp.K = E;
    gp.n_problems = 3;
    const void* wsrc[3] = {tb->wq, tb->wk, tb->wv};
    void* dst[3] = {tb->q, tb->k, tb->v};
    const float* bias[3] = {t->bq, t->bk, t->bv};
    for (int i = 0; i < 3; ++i) {
        gp.a[i] = GemmOperand{tb->xb, Ep, 0};
        gp.b[i] = GemmOperand{wsrc[i], HW, 1};           // stored [E, HW] = [K, N]
        gp.c[i] = dst[i];
        gp.bias[i] = bias[i];
    }
    gp.ldc = HW;
    gp.out_bf16 = 1;
    if ((rc = gemm_sm100(ctx, gp))) return rc;
    ltca_attn_params a;
    fill_attn_bf16(t, &a);
    a.q = tb->q; a.k = tb->k; a.v = tb->v; a.o = tb->ctx; a.lse = tb->lse;
    a.workspace = pl.attn_fwd ? tb->rest : nullptr;
    a.workspace_bytes = pl.attn_fwd;
    return ltca_attn_fwd(ctx, &a);
}

int tensor_forward(ltca_ctx* ctx, const ltca_tsa_params* t) {
    TPlan pl;
    int rc;
    if ((rc = make_tplan(t, &pl, keeps_for_backward(t)))) return rc;
    const size_t need = tensor_workspace(pl, 0);
    if (!t->workspace || t->workspace_bytes < need)
        return fail(ctx, LTCA_ERR_WORKSPACE, "forward needs %zu bytes of workspace", need);
    char* w = reinterpret_cast<char*>(t->workspace);
    float* y = reinterpret_cast<float*>(w);
    w += pl.y;
    TBufs tb;
    if ((rc = tensor_forward_core(ctx, t, pl, w, &tb, 0))) return rc;
    GemmProblem gp;
    gp.M = (int)pl.rows; gp.N = t->E; gp.K = pl.HW;
    gp.a[0] = GemmOperand{tb.ctx, pl.HW, 0};
    gp.b[0] = GemmOperand{tb.wo, pl.Ep, 1};              // stored [HW, E] = [K, N]
    gp.c[0] = y;
    gp.bias[0] = t->bo;
    gp.ldc = t->E;
    if ((rc = gemm_sm100(ctx, gp))) return rc;
    const int wpb = 8;
    LTCA_CUDA_OK(ctx, launch_dependent(residual_layer_norm_kernel, dim3((unsigned)((pl.rows + wpb - 1) / wpb)), dim3(wpb * 32),
                                       0, ctx->stream, (const float*)y, t->x, t->ln_gamma, t->ln_beta, t->out, pl.rows, t->E,
                                       t->use_residual, t->use_layer_norm, 1e-5f));
    LTCA_LAUNCH_OK(ctx, "residual_layer_norm_kernel");
    return LTCA_OK;
}

int tensor_backward(ltca_ctx* ctx, const ltca_tsa_params* t, bool want_dx, bool want_dw, float* colsum_scratch) {
    TPlan pl;
    int rc;
    if ((rc = make_tplan(t, &pl, true))) return rc;
    const size_t need = tensor_workspace(pl, 1);
    if (!t->workspace || t->workspace_bytes < need)
        return fail(ctx, LTCA_ERR_WORKSPACE, "backward needs %zu bytes of workspace", need);
    char* w = reinterpret_cast<char*>(t->workspace);
    void* dyb = w;   w += pl.xb;
    void* dctx = w;  w += pl.act;
    void* dq = w;    w += pl.act;
    void* dk = w;    w += pl.act;
    void* dv = w;    w += pl.act;
    float* partial = reinterpret_cast<float*>(w); w += pl.partial;
    TBufs tb;
    // the forward is recomputed, as the reference's caller does before each backward
    // (src/ml/ml_liquid_net.cu:715-721)
    bool dy_done = false;
    if ((rc = tensor_forward_core(ctx, t, pl, w, &tb, 1, t->dy, dyb, &dy_done))) return rc;
    const int rows = (int)pl.rows, E = t->E, HW = pl.HW, Ep = pl.Ep;
    if (!dy_done && (rc = convert_rows_bf16(ctx, t->dy, E, dyb, Ep, pl.rows, E))) return rc;
    {   // dctx = dy Wo^T : Wo is stored [HW, E] = [N, K]
        GemmProblem gp;
        gp.M = rows; gp.N = HW; gp.K = E;
        gp.a[0] = GemmOperand{dyb, Ep, 0};
        gp.b[0] = GemmOperand{tb.wo, Ep, 0};
        gp.c[0] = dctx;
        gp.ldc = HW;
        gp.out_bf16 = 1;
        if ((rc = gemm_sm100(ctx, gp))) return rc;
    }
    if (pl.wide) {
        WideArgs wa;
        fill_wide(t, tb, &wa);
        wa.dout = dctx; wa.dq = dq; wa.dk = dk; wa.dv = dv;
        if ((rc = wide_attn_bwd(ctx, wa))) return rc;
    } else {
        ltca_attn_params a;
        fill_attn_bf16(t, &a);
        a.q = tb.q; a.k = tb.k; a.v = tb.v; a.o = tb.ctx; a.lse = tb.lse;
        a.dout = dctx; a.dq = dq; a.dk = dk; a.dv = dv;
        a.workspace = pl.attn_bwd ? tb.rest : nullptr;
        a.workspace_bytes = pl.attn_bwd;
        if ((rc = ltca_attn_bwd(ctx, &a))) return rc;
    }
    const void* grads[3] = {dq, dk, dv};
    if (want_dw) {
        // bias gradients (FlashAttention form): column sums of the projection outputs' gradients
        float* db[3] = {t->dbq, t->dbk, t->dbv};
        for (int i = 0; i < 3; ++i)
            if (db[i] && (rc = column_sum(ctx, reinterpret_cast<const __nv_bfloat16*>(grads[i]), HW, pl.rows, HW, db[i],
                                          colsum_scratch))) return rc;
        if (t->dbo && (rc = column_sum(ctx, t->dy, E, pl.rows, E, t->dbo, colsum_scratch))) return rc;
    }
    if (want_dx) {
        // dx = dq Wq^T + dk Wk^T + dv Wv^T : each W is stored [E, HW] = [N, K]; one accumulator tile
        GemmProblem gp;
        gp.M = rows; gp.N = E; gp.K = HW;
        gp.n_sum = 3;
        const void* wsrc[3] = {tb.wq, tb.wk, tb.wv};
        for (int i = 0; i < 3; ++i) {
            gp.a[i] = GemmOperand{grads[i], HW, 0};
            gp.b[i] = GemmOperand{wsrc[i], HW, 0};
        }
        gp.c[0] = t->dx;
        gp.ldc = E;
        if ((rc = gemm_sm100(ctx, gp))) return rc;
    }
    if (want_dw) {
        {   // dW = x^T dq : x is stored [rows, E] = [K, M], dq [rows, HW] = [K, N]
            GemmProblem gp;
            gp.M = E; gp.N = HW; gp.K = rows;
            gp.n_problems = 3;
            gp.ksplit = pl.ks_in;
            void* dst[3] = {t->dwq, t->dwk, t->dwv};
            for (int i = 0; i < 3; ++i) {
                gp.a[i] = GemmOperand{tb.xb, Ep, 1};
                gp.b[i] = GemmOperand{grads[i], HW, 1};
                gp.c[i] = dst[i];
            }
            gp.ldc = HW;
            gp.partial = partial;
            if ((rc = gemm_sm100(ctx, gp))) return rc;
        }
        {   // dWo = ctx^T dy
            GemmProblem gp;
            gp.M = HW; gp.N = E; gp.K = rows;
            gp.ksplit = pl.ks_out;
            gp.a[0] = GemmOperand{tb.ctx, HW, 1};
            gp.b[0] = GemmOperand{dyb, Ep, 1};
            gp.c[0] = t->dwo;
            gp.ldc = E;
            gp.partial = partial;
            if ((rc = gemm_sm100(ctx, gp))) return rc;
        }
    }
    return LTCA_OK;
}

}  // namespace
}  // namespace ltca

using namespace ltca;

extern "C" {

// Workspace of the TimeSelfAttention form (no input LayerNorm, no dropout), without the column-sum scratch.
static int inner_workspace(const ltca_tsa_params* t, int which, size_t* bytes_out) {
    if (use_tensor(t, which != 0 || keeps_for_backward(t))) {
        TPlan tp;
        int trc = make_tplan(t, &tp, which != 0 || keeps_for_backward(t));
        if (trc) return trc;
        *bytes_out = tensor_workspace(tp, which);
        return LTCA_OK;
    }
    Plan pl;
    int rc = make_plan(t, &pl);
    if (rc) return rc;
    size_t n = 4 * pl.buf + pl.lse;                       // q, k, v, ctx, lse
    if (which == 0) {
        n += pl.y;                                        // y before residual / LayerNorm
        n += pl.attn_fwd;
    } else {
        n += 4 * pl.buf;                                  // dctx, dq, dk, dv
        n += pl.attn_fwd > pl.attn_bwd ? pl.attn_fwd : pl.attn_bwd;
    }
    *bytes_out = n;
    return LTCA_OK;
}

// The module without the FlashAttention-form steps: what the pre_norm wrappers run in the middle.
static ltca_tsa_params core_form(const ltca_tsa_params* t) {
    ltca_tsa_params c = *t;
    c.pre_norm = 0;
    c.use_residual = 0;
    c.use_layer_norm = 0;
    c.dropout_prob = 0.f;
    c.dgamma = nullptr;
    c.dbeta = nullptr;
    return c;
}
static size_t act_bytes(const ltca_tsa_params* t) {
    return align_up((size_t)t->B * t->S * t->E * sizeof(float), 256);
}

int ltca_tsa_saved_bytes(const ltca_tsa_params* t, size_t* bytes_out) {
    if (!t || !bytes_out) return LTCA_ERR_INVALID;
    if (t->pre_norm) return LTCA_ERR_UNSUPPORTED;
    ltca_tsa_params probe = *t;
    probe.saved = nullptr;
    if (use_tensor(&probe, true)) {
        TPlan tp;
        int rc = make_tplan(&probe, &tp, true);
        if (rc) return rc;
        *bytes_out = tensor_saved_bytes(tp);
        return LTCA_OK;
    }
    Plan pl;
    int rc = make_plan(&probe, &pl);
    if (rc) return rc;
    *bytes_out = 4 * pl.buf + pl.lse;
    return LTCA_OK;
}

int ltca_tsa_weight_cache_bytes(const ltca_tsa_params* t, size_t* bytes_out) {
    if (!t || !bytes_out) return LTCA_ERR_INVALID;
    *bytes_out = 0;
    // the cache serves the pipeline that the backward takes, which a forward with a cache takes too
    if (!use_tensor(t, true)) return LTCA_OK;
    TPlan tp;
    int rc = make_tplan(t, &tp, true);
    if (rc) return rc;
    *bytes_out = 3 * tp.w_in + tp.w_out + (tp.wide ? 2 * tp.w_in : 0);
    return LTCA_OK;
}

int ltca_tsa_workspace_bytes(const ltca_tsa_params* t, int which, size_t* bytes_out) {
    if (!t || !bytes_out || which < 0 || which > 3) return LTCA_ERR_INVALID;
    size_t n = 0;
    int rc;
    if (t->pre_norm) {
        const ltca_tsa_params c = core_form(t);
        if ((rc = inner_workspace(&c, which, &n))) return rc;
        n += (which == 0 ? 1 : 3) * act_bytes(t);         // LayerNorm(x); backward: + masked dy, gradient at LayerNorm(x)
    } else if ((rc = inner_workspace(t, which, &n))) {
        return rc;
    }
    if (which != 0) n += colsum_scratch_bytes(t);
    *bytes_out = n;
    return LTCA_OK;
}

static int tsa_backward(ltca_ctx* ctx, const ltca_tsa_params* t, bool want_dx, bool want_dw);

// FlashAttention form, forward: LayerNorm on the input, the core module, residual with the raw input, dropout.
static int prenorm_forward(ltca_ctx* ctx, const ltca_tsa_params* t) {
    size_t need = 0;
    int rc = ltca_tsa_workspace_bytes(t, 0, &need);
    if (rc) return rc;
    if (!t->workspace || t->workspace_bytes < need)
        return fail(ctx, LTCA_ERR_WORKSPACE, "forward needs %zu bytes of workspace", need);
    const int64_t rows = (int64_t)t->B * t->S;
    const int64_t n = rows * t->E;
    char* w = reinterpret_cast<char*>(t->workspace);
    float* xin = reinterpret_cast<float*>(w);
    w += act_bytes(t);
    ltca_tsa_params c = core_form(t);
    if (t->use_layer_norm) {
        const int wpb = 8;
        residual_layer_norm_kernel<<<(unsigned)((rows + wpb - 1) / wpb), wpb * 32, 0, ctx->stream>>>(
            t->x, t->x, t->ln_gamma, t->ln_beta, xin, rows, t->E, 0, 1, 1e-5f);
        LTCA_LAUNCH_OK(ctx, "residual_layer_norm_kernel");
        c.x = xin;
    }
    c.workspace = w;
    c.workspace_bytes = t->workspace_bytes - act_bytes(t);
    if ((rc = ltca_tsa_fwd(ctx, &c))) return rc;
    if (t->use_residual && (rc = ltca_add_tensors(ctx, t->out, t->x, t->out, (size_t)n))) return rc;
    if (t->dropout_prob > 0.f) {
        const unsigned blocks = (unsigned)((n + 255) / 256 < 2368 ? (n + 255) / 256 : 2368);
        dropout_kernel<<<blocks, 256, 0, ctx->stream>>>(t->out, t->out, n, t->dropout_prob, t->dropout_seed);
        LTCA_LAUNCH_OK(ctx, "dropout_kernel");
    }
    return LTCA_OK;
}

// FlashAttention form, backward (an extension: the reference class has no backward pass).
static int prenorm_backward(ltca_ctx* ctx, const ltca_tsa_params* t, bool want_dx, bool want_dw) {
    size_t need = 0;
    int rc = ltca_tsa_workspace_bytes(t, 1, &need);
    if (rc) return rc;
    if (!t->workspace || t->workspace_bytes < need)
        return fail(ctx, LTCA_ERR_WORKSPACE, "backward needs %zu bytes of workspace", need);
    if (t->use_layer_norm && !t->ln_gamma) return fail(ctx, LTCA_ERR_INVALID, "LayerNorm needs gamma");
    const int64_t rows = (int64_t)t->B * t->S;
    const int64_t n = rows * t->E;
    const size_t act = act_bytes(t);
    char* w = reinterpret_cast<char*>(t->workspace);
    float* xin = reinterpret_cast<float*>(w);   w += act;
    float* gbuf = reinterpret_cast<float*>(w);  w += act;
    float* dxin = reinterpret_cast<float*>(w);  w += act;
    float* colsum_scratch = reinterpret_cast<float*>(reinterpret_cast<char*>(t->workspace) + need - colsum_scratch_bytes(t));
    const int wpb = 8;
    const unsigned row_blocks = (unsigned)((rows + wpb - 1) / wpb);
    ltca_tsa_params c = core_form(t);
    if (t->use_layer_norm) {
        residual_layer_norm_kernel<<<row_blocks, wpb * 32, 0, ctx->stream>>>(
            t->x, t->x, t->ln_gamma, t->ln_beta, xin, rows, t->E, 0, 1, 1e-5f);
        LTCA_LAUNCH_OK(ctx, "residual_layer_norm_kernel");
        c.x = xin;
    }
    const float* g = t->dy;                      // gradient behind the dropout
    if (t->dropout_prob > 0.f) {
        const unsigned blocks = (unsigned)((n + 255) / 256 < 2368 ? (n + 255) / 256 : 2368);
        dropout_kernel<<<blocks, 256, 0, ctx->stream>>>(t->dy, gbuf, n, t->dropout_prob, t->dropout_seed);
        LTCA_LAUNCH_OK(ctx, "dropout_kernel");
        g = gbuf;
    }
    const bool want_ln_params = want_dw && t->use_layer_norm && (t->dgamma || t->dbeta);
    const bool need_dxin = want_dx || want_ln_params;
    c.dy = g;
    c.dx = dxin;
    c.workspace = w;
    c.workspace_bytes = t->workspace_bytes - 3 * act;
    if ((rc = tsa_backward(ctx, &c, need_dxin, want_dw))) return rc;
    if (!need_dxin) return LTCA_OK;
    if (!t->use_layer_norm) {
        if (want_dx) {
            if (t->use_residual) return ltca_add_tensors(ctx, dxin, g, t->dx, (size_t)n);
            LTCA_CUDA_OK(ctx, cudaMemcpyAsync(t->dx, dxin, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
        }
        return LTCA_OK;
    }
    if (want_ln_params && t->dbeta && (rc = column_sum(ctx, dxin, t->E, rows, t->E, t->dbeta, colsum_scratch))) return rc;
    // dx (or, when only parameter gradients are wanted, a dump into the no longer needed LayerNorm(x) buffer);
    // dxin is overwritten by dxin * xhat, whose column sums are dgamma
    float* dx_out = want_dx ? t->dx : xin;
    layer_norm_bwd_kernel<<<row_blocks, wpb * 32, 0, ctx->stream>>>(
        dxin, t->x, t->ln_gamma, (want_dx && t->use_residual) ? g : nullptr, dx_out,
        (want_ln_params && t->dgamma) ? dxin : nullptr, rows, t->E, 1e-5f);
    LTCA_LAUNCH_OK(ctx, "layer_norm_bwd_kernel");
    if (want_ln_params && t->dgamma && (rc = column_sum(ctx, dxin, t->E, rows, t->E, t->dgamma, colsum_scratch))) return rc;
    return LTCA_OK;
}

int ltca_tsa_fwd(ltca_ctx* ctx, const ltca_tsa_params* t) {
    int rc = check(ctx, t);
    if (rc) return rc;
    LTCA_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    if (!t->out) return fail(ctx, LTCA_ERR_INVALID, "out must be non-null");
    if (t->use_layer_norm && (!t->ln_gamma || !t->ln_beta))
        return fail(ctx, LTCA_ERR_INVALID, "LayerNorm needs gamma and beta");
    if (t->dropout_prob < 0.f || t->dropout_prob >= 1.f)
        return fail(ctx, LTCA_ERR_INVALID, "dropout_prob must be in [0, 1)");
    if (t->pre_norm) return prenorm_forward(ctx, t);
    if (use_tensor(t, keeps_for_backward(t))) return tensor_forward(ctx, t);
    Plan pl;
    if ((rc = make_plan(t, &pl))) return rc;
    size_t need = 0;
    ltca_tsa_workspace_bytes(t, 0, &need);
    if (!t->workspace || t->workspace_bytes < need)
        return fail(ctx, LTCA_ERR_WORKSPACE, "forward needs %zu bytes of workspace", need);
    char* w = reinterpret_cast<char*>(t->workspace);
    float* y = reinterpret_cast<float*>(w);
    w += pl.y;
    FwdBufs fb;
    if ((rc = forward_core(ctx, t, pl, w, &fb, pl.attn_fwd))) return rc;
    const int rows = (int)pl.rows;
    if ((rc = gemm(ctx, fb.ctx, t->wo, t->bo, y, rows, t->E, pl.HW, pl.HW, t->E, t->E, 0, 0, 0)))
        return rc;
    const int wpb = 8;
    residual_layer_norm_kernel<<<(unsigned)((pl.rows + wpb - 1) / wpb), wpb * 32, 0, ctx->stream>>>(
        y, t->x, t->ln_gamma, t->ln_beta, t->out, pl.rows, t->E, t->use_residual, t->use_layer_norm,
        1e-5f);
    LTCA_LAUNCH_OK(ctx, "residual_layer_norm_kernel");
    return LTCA_OK;
}

static int tsa_backward(ltca_ctx* ctx, const ltca_tsa_params* t, bool want_dx, bool want_dw) {
    int rc = check(ctx, t);
    if (rc) return rc;
    LTCA_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    if (!t->dy) return fail(ctx, LTCA_ERR_INVALID, "dy must be non-null");
    if (want_dx && !t->dx) return fail(ctx, LTCA_ERR_INVALID, "dx must be non-null");
    if (want_dw && (!t->dwq || !t->dwk || !t->dwv || !t->dwo))
        return fail(ctx, LTCA_ERR_INVALID, "dwq, dwk, dwv, dwo must be non-null");
    if (t->dropout_prob < 0.f || t->dropout_prob >= 1.f)
        return fail(ctx, LTCA_ERR_INVALID, "dropout_prob must be in [0, 1)");
    if (t->pre_norm) return prenorm_backward(ctx, t, want_dx, want_dw);
    size_t need = 0;
    ltca_tsa_workspace_bytes(t, 1, &need);
    if (!t->workspace || t->workspace_bytes < need)
        return fail(ctx, LTCA_ERR_WORKSPACE, "backward needs %zu bytes of workspace", need);
    float* colsum_scratch =
        reinterpret_cast<float*>(reinterpret_cast<char*>(t->workspace) + need - colsum_scratch_bytes(t));
    if (use_tensor(t, true)) return tensor_backward(ctx, t, want_dx, want_dw, colsum_scratch);
    Plan pl;
    if ((rc = make_plan(t, &pl))) return rc;
    if (!t->workspace || t->workspace_bytes < need)
        return fail(ctx, LTCA_ERR_WORKSPACE, "backward needs %zu bytes of workspace", need);
    char* w = reinterpret_cast<char*>(t->workspace);
    float* dctx = reinterpret_cast<float*>(w); w += pl.buf;
    float* dq = reinterpret_cast<float*>(w);   w += pl.buf;
    float* dk = reinterpret_cast<float*>(w);   w += pl.buf;
    float* dv = reinterpret_cast<float*>(w);   w += pl.buf;
    FwdBufs fb;
    // the forward is recomputed, as the reference's caller does before each backward
    // (src/ml/ml_liquid_net.cu:715-721)
    if ((rc = forward_core(ctx, t, pl, w, &fb, pl.attn_fwd))) return rc;
    const int rows = (int)pl.rows, E = t->E, HW = pl.HW;
    // dctx = dy Wo^T
    if ((rc = gemm(ctx, t->dy, t->wo, nullptr, dctx, rows, HW, E, E, E, HW, 0, 1, 0))) return rc;
    ltca_attn_params a;
    fill_attn(t, &a);
    a.q = fb.q; a.k = fb.k; a.v = fb.v; a.o = fb.ctx; a.lse = fb.lse;
    a.dout = dctx; a.dq = dq; a.dk = dk; a.dv = dv;
    a.workspace = pl.attn_bwd ? fb.rest : nullptr;
    a.workspace_bytes = pl.attn_bwd;
    if ((rc = ltca_attn_bwd(ctx, &a))) return rc;
    if (want_dw) {
        // bias gradients (FlashAttention form): column sums of the projection outputs' gradients
        if (t->dbq && (rc = column_sum(ctx, dq, HW, pl.rows, HW, t->dbq, colsum_scratch))) return rc;
        if (t->dbk && (rc = column_sum(ctx, dk, HW, pl.rows, HW, t->dbk, colsum_scratch))) return rc;
        if (t->dbv && (rc = column_sum(ctx, dv, HW, pl.rows, HW, t->dbv, colsum_scratch))) return rc;
        if (t->dbo && (rc = column_sum(ctx, t->dy, E, pl.rows, E, t->dbo, colsum_scratch))) return rc;
    }
    if (want_dx) {
        if ((rc = gemm(ctx, dq, t->wq, nullptr, t->dx, rows, E, HW, HW, HW, E, 0, 1, 0))) return rc;
        if ((rc = gemm(ctx, dk, t->wk, nullptr, t->dx, rows, E, HW, HW, HW, E, 0, 1, 1))) return rc;
        if ((rc = gemm(ctx, dv, t->wv, nullptr, t->dx, rows, E, HW, HW, HW, E, 0, 1, 1))) return rc;
    }
    if (want_dw) {
        // dW = x^T dQ  ([E, rows] x [rows, HW]),  dWo = ctx^T dy  ([HW, rows] x [rows, E])
        // dctx is dead once the attention backward has run: it holds the contraction slices
        if ((rc = gemm_long_k(ctx, t->x, dq, t->dwq, E, HW, rows, E, HW, HW, 1, 0, dctx, pl.buf))) return rc;
        if ((rc = gemm_long_k(ctx, t->x, dk, t->dwk, E, HW, rows, E, HW, HW, 1, 0, dctx, pl.buf))) return rc;
        if ((rc = gemm_long_k(ctx, t->x, dv, t->dwv, E, HW, rows, E, HW, HW, 1, 0, dctx, pl.buf))) return rc;
        if ((rc = gemm_long_k(ctx, fb.ctx, t->dy, t->dwo, HW, E, rows, HW, E, E, 1, 0, dctx, pl.buf)))
            return rc;
    }
    return LTCA_OK;
}

int ltca_tsa_bwd_data(ltca_ctx* ctx, const ltca_tsa_params* t) {
    return tsa_backward(ctx, t, true, false);
}
int ltca_tsa_bwd_weights(ltca_ctx* ctx, const ltca_tsa_params* t) {
    return tsa_backward(ctx, t, false, true);
}
int ltca_tsa_bwd(ltca_ctx* ctx, const ltca_tsa_params* t) {
    return tsa_backward(ctx, t, true, true);
}

}  // extern "C"
