// fp32 attention: the exact arithmetic mode (fp32 FMA, accurate expf) and the path for every
// shape the tensor-pipe kernels do not take (any head_dim up to 512, dense keep-masks, tiny
// sequences).  Forward, backward (two passes, no atomics, bit-reproducible) and the
// row-statistics helper shared with the tensor-pipe backward.
//
// Replaces flashAttentionKernel (reference src/ml/flash_attention.cu:18-272) on its own valid
// domain (head_dim <= 16, one key tile) and extends it to a true online softmax for longer
// sequences; the 16x16-thread tiling keeps one query row inside a half-warp so that row maxima
// and row sums are half-warp shuffle reductions.
#include <math.h>

#include "host_common.h"

namespace ltca {

namespace {

constexpr int kTM = 64;     // query rows per CTA
constexpr int kTN = 64;     // keys per step
constexpr int kThreads = 256;

__device__ __forceinline__ float ld_elem(const float* p) { return __ldg(p); }
__device__ __forceinline__ float ld_elem(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st_elem(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_elem(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

struct CoreArgs {
    int B, H, Sq, Sk, D;
    int causal, causal_off;
    float scale, clamp;
    int use_clamp;
    const void *q, *k, *v, *o_in, *dout;
    void *o, *dq, *dk, *dv;
    ltca_strides qs, ks, vs, os, dos, dqs, dks, dvs;
    float* lse;
    const float* lse_in;
    float* delta;
    const float* keep_mask;
    const int32_t* kv_len;
};

// Loads rows [r0, r0+64) x [0, D) of a [.., seq, D] tensor into smem [64][ld], zero padded.
template <typename T>
__device__ __forceinline__ void load_tile(float* dst, int ld, const T* base, int64_t row_stride,
                                          int r0, int rows_total, int D) {
    for (int idx = threadIdx.x; idx < kTM * D; idx += kThreads) {
        const int r = idx / D, d = idx - r * D;
        const int gr = r0 + r;
        dst[r * ld + d] = (gr < rows_total) ? ld_elem(base + (int64_t)gr * row_stride + d) : 0.f;
    }
}

__device__ __forceinline__ float half_warp_max(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ bool key_visible(const CoreArgs& a, int b, int qi, int kj, int kvlen) {
    if (kj >= kvlen) return false;
    if (a.causal && kj > qi + a.causal_off) return false;
    if (a.keep_mask && qi < a.Sq && a.keep_mask[((int64_t)b * a.Sq + qi) * a.Sk + kj] == 0.f)
        return false;
    return true;
}

// ----------------------------------------------------------------------------------------------
// forward
// thread (ty, tx) of a 16x16 grid owns query rows ty + 16 i and key columns tx + 16 j (i, j < 4)
// in the score step, and output columns tx + 16 c (c < DC) in the value step.
// ----------------------------------------------------------------------------------------------
template <typename T, int DC>
__global__ void __launch_bounds__(kThreads) attn_fwd_fp32_kernel(const CoreArgs a) {
    extern __shared__ float sm[];
    const int D = a.D;
    const int ld = D + 1;
    float* Qs = sm;
    float* Ks = Qs + kTM * ld;
    float* Vs = Ks + kTN * ld;
    float* Ps = Vs + kTN * ld;          // [64][65]

    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int q0 = blockIdx.x * kTM;
    const int h = blockIdx.y, b = blockIdx.z;
    int kvlen = a.Sk;
    if (a.kv_len) kvlen = min(max(a.kv_len[b], 0), a.Sk);

    const T* qb = reinterpret_cast<const T*>(a.q) + b * a.qs.batch + h * a.qs.head;
    const T* kb = reinterpret_cast<const T*>(a.k) + b * a.ks.batch + h * a.ks.head;
    const T* vb = reinterpret_cast<const T*>(a.v) + b * a.vs.batch + h * a.vs.head;

    load_tile(Qs, ld, qb, a.qs.seq, q0, a.Sq, D);

    float m_run[4], l_run[4], acc[4][DC];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m_run[i] = -INFINITY;
        l_run[i] = 0.f;
#pragma unroll
        for (int c = 0; c < DC; ++c) acc[i][c] = 0.f;
    }

    int k_end = kvlen;
    if (a.causal) k_end = min(k_end, min(q0 + kTM - 1, a.Sq - 1) + a.causal_off + 1);
    for (int k0 = 0; k0 < k_end; k0 += kTN) {
        __syncthreads();
        load_tile(Ks, ld, kb, a.ks.seq, k0, a.Sk, D);
        load_tile(Vs, ld, vb, a.vs.seq, k0, a.Sk, D);
        __syncthreads();

        float s[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
        for (int d = 0; d < D; ++d) {
            float qv[4], kv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) qv[i] = Qs[(ty + 16 * i) * ld + d];
#pragma unroll
            for (int j = 0; j < 4; ++j) kv[j] = Ks[(tx + 16 * j) * ld + d];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) s[i][j] = fmaf(qv[i], kv[j], s[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int qi = q0 + ty + 16 * i;
            float mt = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int kj = k0 + tx + 16 * j;
                float v = s[i][j] * a.scale;
                if (a.use_clamp) v = fminf(v, a.clamp);
                if (!key_visible(a, b, qi, kj, kvlen)) v = -INFINITY;
                s[i][j] = v;
                mt = fmaxf(mt, v);
            }
            mt = half_warp_max(mt);
            const float m_new = fmaxf(m_run[i], mt);
            const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = (m_run[i] == -INFINITY) ? 0.f : expf(m_run[i] - m_safe);
            float rs = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float p = expf(s[i][j] - m_safe);      // exp(-inf) = 0 for hidden keys
                Ps[(ty + 16 * i) * (kTN + 1) + tx + 16 * j] = p;
                rs += p;
            }
            rs = half_warp_sum(rs);
            l_run[i] = l_run[i] * corr + rs;
            m_run[i] = m_new;
#pragma unroll
            for (int c = 0; c < DC; ++c) acc[i][c] *= corr;
        }
        __syncthreads();
        for (int j = 0; j < kTN; ++j) {
            float pv[4], vv[DC];
#pragma unroll
            for (int i = 0; i < 4; ++i) pv[i] = Ps[(ty + 16 * i) * (kTN + 1) + j];
#pragma unroll
            for (int c = 0; c < DC; ++c) {
                const int d = tx + 16 * c;
                vv[c] = (d < D) ? Vs[j * ld + d] : 0.f;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int c = 0; c < DC; ++c) acc[i][c] = fmaf(pv[i], vv[c], acc[i][c]);
        }
    }

    T* ob = reinterpret_cast<T*>(a.o) + b * a.os.batch + h * a.os.head;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int qi = q0 + ty + 16 * i;
        if (qi >= a.Sq) continue;
        const float inv = l_run[i] > 0.f ? 1.f / l_run[i] : 0.f;
#pragma unroll
        for (int c = 0; c < DC; ++c) {
            const int d = tx + 16 * c;
            if (d < D) st_elem(ob + (int64_t)qi * a.os.seq + d, acc[i][c] * inv);
        }
        if (a.lse && tx == 0)
            a.lse[((int64_t)b * a.H + h) * a.Sq + qi] =
                l_run[i] > 0.f ? m_run[i] + logf(l_run[i]) : -INFINITY;
    }
}

// ----------------------------------------------------------------------------------------------
// backward helper: delta[b,h,i] = sum_d dO[i,d] * O[i,d]   (one warp per query row)
// ----------------------------------------------------------------------------------------------
template <typename T>
__global__ void attn_bwd_delta_kernel(const CoreArgs a) {
    const int warps_per_block = blockDim.x >> 5;
    const int64_t row = (int64_t)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int64_t total = (int64_t)a.B * a.H * a.Sq;
    if (row >= total) return;
    const int qi = (int)(row % a.Sq);
    const int64_t bh = row / a.Sq;
    const int h = (int)(bh % a.H), b = (int)(bh / a.H);
    const T* o = reinterpret_cast<const T*>(a.o_in) + b * a.os.batch + h * a.os.head + (int64_t)qi * a.os.seq;
    const T* g = reinterpret_cast<const T*>(a.dout) + b * a.dos.batch + h * a.dos.head + (int64_t)qi * a.dos.seq;
    float acc = 0.f;
    for (int d = lane; d < a.D; d += 32) acc = fmaf(ld_elem(o + d), ld_elem(g + d), acc);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) a.delta[row] = acc;
}

// ----------------------------------------------------------------------------------------------
// backward, pass 1: dQ.  One CTA per 64 query rows; loops over key tiles.
// ----------------------------------------------------------------------------------------------
template <typename T, int DC>
__global__ void __launch_bounds__(kThreads) attn_bwd_dq_fp32_kernel(const CoreArgs a) {
    extern __shared__ float sm[];
    const int D = a.D;
    const int ld = D + 1;
    float* Qs = sm;
    float* Gs = Qs + kTM * ld;          // dO
    float* Ks = Gs + kTM * ld;
    float* Vs = Ks + kTN * ld;
    float* Ss = Vs + kTN * ld;          // dS [64][65]

    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int q0 = blockIdx.x * kTM;
    const int h = blockIdx.y, b = blockIdx.z;
    int kvlen = a.Sk;
    if (a.kv_len) kvlen = min(max(a.kv_len[b], 0), a.Sk);

    const T* qb = reinterpret_cast<const T*>(a.q) + b * a.qs.batch + h * a.qs.head;
    const T* kb = reinterpret_cast<const T*>(a.k) + b * a.ks.batch + h * a.ks.head;
    const T* vb = reinterpret_cast<const T*>(a.v) + b * a.vs.batch + h * a.vs.head;
    const T* gb = reinterpret_cast<const T*>(a.dout) + b * a.dos.batch + h * a.dos.head;
    load_tile(Qs, ld, qb, a.qs.seq, q0, a.Sq, D);
    load_tile(Gs, ld, gb, a.dos.seq, q0, a.Sq, D);

    float lse[4], dlt[4], acc[4][DC];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int qi = q0 + ty + 16 * i;
        const int64_t r = ((int64_t)b * a.H + h) * a.Sq + qi;
        lse[i] = qi < a.Sq ? a.lse_in[r] : -INFINITY;
        dlt[i] = qi < a.Sq ? a.delta[r] : 0.f;
#pragma unroll
        for (int c = 0; c < DC; ++c) acc[i][c] = 0.f;
    }

    int k_end = kvlen;
    if (a.causal) k_end = min(k_end, min(q0 + kTM - 1, a.Sq - 1) + a.causal_off + 1);
    for (int k0 = 0; k0 < k_end; k0 += kTN) {
        __syncthreads();
        load_tile(Ks, ld, kb, a.ks.seq, k0, a.Sk, D);
        load_tile(Vs, ld, vb, a.vs.seq, k0, a.Sk, D);
        __syncthreads();
        float s[4][4], dp[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) { s[i][j] = 0.f; dp[i][j] = 0.f; }
        for (int d = 0; d < D; ++d) {
            float qv[4], gv[4], kv[4], vv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                qv[i] = Qs[(ty + 16 * i) * ld + d];
                gv[i] = Gs[(ty + 16 * i) * ld + d];
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                kv[j] = Ks[(tx + 16 * j) * ld + d];
                vv[j] = Vs[(tx + 16 * j) * ld + d];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    s[i][j] = fmaf(qv[i], kv[j], s[i][j]);
                    dp[i][j] = fmaf(gv[i], vv[j], dp[i][j]);
                }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int qi = q0 + ty + 16 * i;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int kj = k0 + tx + 16 * j;
                float v = s[i][j] * a.scale;
                bool clamped = false;
                if (a.use_clamp && v >= a.clamp) { v = a.clamp; clamped = true; }
                float ds = 0.f;
                if (key_visible(a, b, qi, kj, kvlen) && lse[i] != -INFINITY) {
                    const float p = expf(v - lse[i]);
                    ds = clamped ? 0.f : p * (dp[i][j] - dlt[i]) * a.scale;
                }
                Ss[(ty + 16 * i) * (kTN + 1) + tx + 16 * j] = ds;
            }
        }
        __syncthreads();
        for (int j = 0; j < kTN; ++j) {
            float pv[4], kk[DC];
#pragma unroll
            for (int i = 0; i < 4; ++i) pv[i] = Ss[(ty + 16 * i) * (kTN + 1) + j];
#pragma unroll
            for (int c = 0; c < DC; ++c) {
                const int d = tx + 16 * c;
                kk[c] = (d < D) ? Ks[j * ld + d] : 0.f;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int c = 0; c < DC; ++c) acc[i][c] = fmaf(pv[i], kk[c], acc[i][c]);
        }
    }
    T* dqb = reinterpret_cast<T*>(a.dq) + b * a.dqs.batch + h * a.dqs.head;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int qi = q0 + ty + 16 * i;
        if (qi >= a.Sq) continue;
#pragma unroll
        for (int c = 0; c < DC; ++c) {
            const int d = tx + 16 * c;
            if (d < D) st_elem(dqb + (int64_t)qi * a.dqs.seq + d, acc[i][c]);
        }
    }
}

// ----------------------------------------------------------------------------------------------
// backward, pass 2: dK and dV.  One CTA per 64 keys; loops over query tiles.
// In the accumulation step thread (ty, tx) owns key rows ty + 16 i and feature columns tx + 16 c.
// ----------------------------------------------------------------------------------------------
template <typename T, int DC>
__global__ void __launch_bounds__(kThreads) attn_bwd_dkv_fp32_kernel(const CoreArgs a) {
    extern __shared__ float sm[];
    const int D = a.D;
    const int ld = D + 1;
    float* Qs = sm;
    float* Gs = Qs + kTM * ld;
    float* Ks = Gs + kTM * ld;
    float* Vs = Ks + kTN * ld;
    float* Ps = Vs + kTN * ld;                  // P  [64 q][65]
    float* Ss = Ps + kTM * (kTN + 1);           // dS [64 q][65]

    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int k0 = blockIdx.x * kTN;
    const int h = blockIdx.y, b = blockIdx.z;
    int kvlen = a.Sk;
    if (a.kv_len) kvlen = min(max(a.kv_len[b], 0), a.Sk);

    const T* qb = reinterpret_cast<const T*>(a.q) + b * a.qs.batch + h * a.qs.head;
    const T* kb = reinterpret_cast<const T*>(a.k) + b * a.ks.batch + h * a.ks.head;
    const T* vb = reinterpret_cast<const T*>(a.v) + b * a.vs.batch + h * a.vs.head;
    const T* gb = reinterpret_cast<const T*>(a.dout) + b * a.dos.batch + h * a.dos.head;
    load_tile(Ks, ld, kb, a.ks.seq, k0, a.Sk, D);
    load_tile(Vs, ld, vb, a.vs.seq, k0, a.Sk, D);

    float acck[4][DC], accv[4][DC];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < DC; ++c) { acck[i][c] = 0.f; accv[i][c] = 0.f; }

    // first query row that can see key k0 (causal): qi >= k0 - causal_off
    int q_begin = 0;
    if (a.causal) q_begin = max(0, k0 - a.causal_off) / kTM * kTM;
    const bool tile_live = k0 < kvlen;
    for (int q0 = q_begin; q0 < a.Sq && tile_live; q0 += kTM) {
        __syncthreads();
        load_tile(Qs, ld, qb, a.qs.seq, q0, a.Sq, D);
        load_tile(Gs, ld, gb, a.dos.seq, q0, a.Sq, D);
        __syncthreads();
        float s[4][4], dp[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) { s[i][j] = 0.f; dp[i][j] = 0.f; }
        for (int d = 0; d < D; ++d) {
            float qv[4], gv[4], kv[4], vv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                qv[i] = Qs[(ty + 16 * i) * ld + d];
                gv[i] = Gs[(ty + 16 * i) * ld + d];
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                kv[j] = Ks[(tx + 16 * j) * ld + d];
                vv[j] = Vs[(tx + 16 * j) * ld + d];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    s[i][j] = fmaf(qv[i], kv[j], s[i][j]);
                    dp[i][j] = fmaf(gv[i], vv[j], dp[i][j]);
                }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int qi = q0 + ty + 16 * i;
            float lse = -INFINITY, dlt = 0.f;
            if (qi < a.Sq) {
                const int64_t r = ((int64_t)b * a.H + h) * a.Sq + qi;
                lse = a.lse_in[r];
                dlt = a.delta[r];
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int kj = k0 + tx + 16 * j;
                float v = s[i][j] * a.scale;
                bool clamped = false;
                if (a.use_clamp && v >= a.clamp) { v = a.clamp; clamped = true; }
                float p = 0.f, ds = 0.f;
                if (qi < a.Sq && key_visible(a, b, qi, kj, kvlen) && lse != -INFINITY) {
                    p = expf(v - lse);
                    ds = clamped ? 0.f : p * (dp[i][j] - dlt) * a.scale;
                }
                Ps[(ty + 16 * i) * (kTN + 1) + tx + 16 * j] = p;
                Ss[(ty + 16 * i) * (kTN + 1) + tx + 16 * j] = ds;
            }
        }
        __syncthreads();
        for (int r = 0; r < kTM; ++r) {
            float pp[4], dd[4], gg[DC], qq[DC];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                pp[i] = Ps[r * (kTN + 1) + ty + 16 * i];
                dd[i] = Ss[r * (kTN + 1) + ty + 16 * i];
            }
#pragma unroll
            for (int c = 0; c < DC; ++c) {
                const int d = tx + 16 * c;
                gg[c] = (d < D) ? Gs[r * ld + d] : 0.f;
                qq[c] = (d < D) ? Qs[r * ld + d] : 0.f;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int c = 0; c < DC; ++c) {
                    accv[i][c] = fmaf(pp[i], gg[c], accv[i][c]);
                    acck[i][c] = fmaf(dd[i], qq[c], acck[i][c]);
                }
        }
    }
    T* dkb = reinterpret_cast<T*>(a.dk) + b * a.dks.batch + h * a.dks.head;
    T* dvb = reinterpret_cast<T*>(a.dv) + b * a.dvs.batch + h * a.dvs.head;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int kj = k0 + ty + 16 * i;
        if (kj >= a.Sk) continue;
#pragma unroll
        for (int c = 0; c < DC; ++c) {
            const int d = tx + 16 * c;
            if (d < D) {
                st_elem(dkb + (int64_t)kj * a.dks.seq + d, acck[i][c]);
                st_elem(dvb + (int64_t)kj * a.dvs.seq + d, accv[i][c]);
            }
        }
    }
}

CoreArgs make_args(const ltca_attn_params* p) {
    CoreArgs a;
    memset(&a, 0, sizeof(a));
    a.B = p->B; a.H = p->H; a.Sq = p->Sq; a.Sk = p->Sk; a.D = p->D;
    a.causal = p->causal ? 1 : 0;
    a.causal_off = p->Sk - p->Sq;
    a.scale = p->scale;
    a.use_clamp = p->score_clamp > 0.f ? 1 : 0;
    a.clamp = p->score_clamp;
    a.q = p->q; a.k = p->k; a.v = p->v; a.o = p->o; a.o_in = p->o; a.dout = p->dout;
    a.dq = p->dq; a.dk = p->dk; a.dv = p->dv;
    a.qs = p->q_strides; a.ks = p->k_strides; a.vs = p->v_strides; a.os = p->o_strides;
    a.dos = p->do_strides; a.dqs = p->dq_strides; a.dks = p->dk_strides; a.dvs = p->dv_strides;
    a.lse = p->lse; a.lse_in = p->lse;
    a.keep_mask = p->keep_mask;
    a.kv_len = p->kv_len;
    return a;
}

template <typename K>
int set_smem(ltca_ctx* ctx, K kern, size_t bytes) {
    if (bytes > 48 * 1024)
        LTCA_CUDA_OK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)bytes));
    return LTCA_OK;
}

template <typename T, int DC>
int run_fwd(ltca_ctx* ctx, const CoreArgs& a) {
    const size_t smem = (size_t)(3 * kTM * (a.D + 1) + kTM * (kTN + 1)) * sizeof(float);
    auto kern = attn_fwd_fp32_kernel<T, DC>;
    int rc = set_smem(ctx, kern, smem);
    if (rc) return rc;
    dim3 grid((a.Sq + kTM - 1) / kTM, a.H, a.B);
    kern<<<grid, kThreads, smem, ctx->stream>>>(a);
    LTCA_LAUNCH_OK(ctx, "attn_fwd_fp32_kernel");
    return LTCA_OK;
}

template <typename T, int DC>
int run_bwd(ltca_ctx* ctx, const CoreArgs& a) {
    {
        const int wpb = 8;
        const int64_t rows = (int64_t)a.B * a.H * a.Sq;
        attn_bwd_delta_kernel<T><<<(unsigned)((rows + wpb - 1) / wpb), wpb * 32, 0, ctx->stream>>>(a);
        LTCA_LAUNCH_OK(ctx, "attn_bwd_delta_kernel");
    }
    {
        const size_t smem = (size_t)(4 * kTM * (a.D + 1) + kTM * (kTN + 1)) * sizeof(float);
        auto kern = attn_bwd_dq_fp32_kernel<T, DC>;
        int rc = set_smem(ctx, kern, smem);
        if (rc) return rc;
        dim3 grid((a.Sq + kTM - 1) / kTM, a.H, a.B);
        kern<<<grid, kThreads, smem, ctx->stream>>>(a);
        LTCA_LAUNCH_OK(ctx, "attn_bwd_dq_fp32_kernel");
    }
    {
        const size_t smem = (size_t)(4 * kTM * (a.D + 1) + 2 * kTM * (kTN + 1)) * sizeof(float);
        auto kern = attn_bwd_dkv_fp32_kernel<T, DC>;
        int rc = set_smem(ctx, kern, smem);
        if (rc) return rc;
        dim3 grid((a.Sk + kTN - 1) / kTN, a.H, a.B);
        kern<<<grid, kThreads, smem, ctx->stream>>>(a);
        LTCA_LAUNCH_OK(ctx, "attn_bwd_dkv_fp32_kernel");
    }
    return LTCA_OK;
}


// ----------------------------------------------------------------------------------------------
// Wide heads (128 < head_dim <= 512): the reference-compatible TimeSelfAttention gives every head
// the full model width (include/cuDNN_ops.h:166-169 of the reference), so a 512-wide model has
// 512-wide heads.  A tile of such rows no longer fits in shared memory next to its keys, so these
// kernels give one warp to one query row (or one key row in the dK/dV pass): the lanes split the
// feature dimension, a score is a warp reduction, and the row's accumulator lives in registers.
// Same arithmetic and the same masks as the tiled kernels above; no atomics.
// ----------------------------------------------------------------------------------------------
constexpr int kWideMaxD = 512;
constexpr int kWC = kWideMaxD / 32;        // feature columns per lane
constexpr int kWideWarps = 4;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename T>
__device__ __forceinline__ void load_row(float (&r)[kWC], const T* p, int D, int lane, float mul) {
#pragma unroll
    for (int c = 0; c < kWC; ++c) {
        const int d = lane + 32 * c;
        r[c] = d < D ? ld_elem(p + d) * mul : 0.f;
    }
}
__device__ __forceinline__ float dot_row(const float (&x)[kWC], const float (&y)[kWC]) {
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < kWC; ++c) s = fmaf(x[c], y[c], s);
    return warp_sum(s);
}

template <typename T>
__global__ void __launch_bounds__(kWideWarps * 32) attn_fwd_wide_kernel(const CoreArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWideWarps + (threadIdx.x >> 5);
    if (row >= (int64_t)a.B * a.H * a.Sq) return;
    const int qi = (int)(row % a.Sq);
    const int64_t bh = row / a.Sq;
    const int h = (int)(bh % a.H), b = (int)(bh / a.H);
    int kvlen = a.Sk;
    if (a.kv_len) kvlen = min(max(a.kv_len[b], 0), a.Sk);
    const T* kb = reinterpret_cast<const T*>(a.k) + b * a.ks.batch + h * a.ks.head;
    const T* vb = reinterpret_cast<const T*>(a.v) + b * a.vs.batch + h * a.vs.head;
    float q[kWC], acc[kWC];
    load_row(q, reinterpret_cast<const T*>(a.q) + b * a.qs.batch + h * a.qs.head + (int64_t)qi * a.qs.seq, a.D,
             lane, a.scale);
#pragma unroll
    for (int c = 0; c < kWC; ++c) acc[c] = 0.f;
    float m = -INFINITY, l = 0.f;
    int k_end = kvlen;
    if (a.causal) k_end = min(k_end, qi + a.causal_off + 1);
    for (int j = 0; j < k_end; ++j) {
        if (!key_visible(a, b, qi, j, kvlen)) continue;          // the same answer in every lane
        float kr[kWC];
        load_row(kr, kb + (int64_t)j * a.ks.seq, a.D, lane, 1.f);
        float v = dot_row(q, kr);
        if (a.use_clamp) v = fminf(v, a.clamp);
        const float m_new = fmaxf(m, v);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float p = expf(v - m_new);
        l = l * corr + p;
        m = m_new;
        load_row(kr, vb + (int64_t)j * a.vs.seq, a.D, lane, 1.f);
#pragma unroll
        for (int c = 0; c < kWC; ++c) acc[c] = fmaf(p, kr[c], acc[c] * corr);
    }
    T* op = reinterpret_cast<T*>(a.o) + b * a.os.batch + h * a.os.head + (int64_t)qi * a.os.seq;
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int c = 0; c < kWC; ++c) {
        const int d = lane + 32 * c;
        if (d < a.D) st_elem(op + d, acc[c] * inv);
    }
    if (a.lse && lane == 0) a.lse[row] = l > 0.f ? m + logf(l) : -INFINITY;
}

// dQ: one warp per query row.
template <typename T>
__global__ void __launch_bounds__(kWideWarps * 32) attn_bwd_dq_wide_kernel(const CoreArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWideWarps + (threadIdx.x >> 5);
    if (row >= (int64_t)a.B * a.H * a.Sq) return;
    const int qi = (int)(row % a.Sq);
    const int64_t bh = row / a.Sq;
    const int h = (int)(bh % a.H), b = (int)(bh / a.H);
    int kvlen = a.Sk;
    if (a.kv_len) kvlen = min(max(a.kv_len[b], 0), a.Sk);
    const T* kb = reinterpret_cast<const T*>(a.k) + b * a.ks.batch + h * a.ks.head;
    const T* vb = reinterpret_cast<const T*>(a.v) + b * a.vs.batch + h * a.vs.head;
    float q[kWC], g[kWC], acc[kWC];
    load_row(q, reinterpret_cast<const T*>(a.q) + b * a.qs.batch + h * a.qs.head + (int64_t)qi * a.qs.seq, a.D,
             lane, a.scale);
    load_row(g, reinterpret_cast<const T*>(a.dout) + b * a.dos.batch + h * a.dos.head + (int64_t)qi * a.dos.seq,
             a.D, lane, 1.f);
#pragma unroll
    for (int c = 0; c < kWC; ++c) acc[c] = 0.f;
    const float lse = a.lse_in[row], dlt = a.delta[row];
    int k_end = kvlen;
    if (a.causal) k_end = min(k_end, qi + a.causal_off + 1);
    if (lse == -INFINITY) k_end = 0;
    for (int j = 0; j < k_end; ++j) {
        if (!key_visible(a, b, qi, j, kvlen)) continue;
        float kr[kWC], vr[kWC];
        load_row(kr, kb + (int64_t)j * a.ks.seq, a.D, lane, 1.f);
        load_row(vr, vb + (int64_t)j * a.vs.seq, a.D, lane, 1.f);
        float v = dot_row(q, kr);
        const float dp = dot_row(g, vr);
        bool clamped = false;
        if (a.use_clamp && v >= a.clamp) { v = a.clamp; clamped = true; }
        const float ds = clamped ? 0.f : expf(v - lse) * (dp - dlt) * a.scale;
#pragma unroll
        for (int c = 0; c < kWC; ++c) acc[c] = fmaf(ds, kr[c], acc[c]);
    }
    T* dqp = reinterpret_cast<T*>(a.dq) + b * a.dqs.batch + h * a.dqs.head + (int64_t)qi * a.dqs.seq;
#pragma unroll
    for (int c = 0; c < kWC; ++c) {
        const int d = lane + 32 * c;
        if (d < a.D) st_elem(dqp + d, acc[c]);
    }
}

// dK and dV: one warp per key row, looping over the queries that see the key.
template <typename T>
__global__ void __launch_bounds__(kWideWarps * 32) attn_bwd_dkv_wide_kernel(const CoreArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kWideWarps + (threadIdx.x >> 5);
    if (row >= (int64_t)a.B * a.H * a.Sk) return;
    const int kj = (int)(row % a.Sk);
    const int64_t bh = row / a.Sk;
    const int h = (int)(bh % a.H), b = (int)(bh / a.H);
    int kvlen = a.Sk;
    if (a.kv_len) kvlen = min(max(a.kv_len[b], 0), a.Sk);
    const T* qb = reinterpret_cast<const T*>(a.q) + b * a.qs.batch + h * a.qs.head;
    const T* gb = reinterpret_cast<const T*>(a.dout) + b * a.dos.batch + h * a.dos.head;
    float kr[kWC], vr[kWC], dk[kWC], dv[kWC];
    load_row(kr, reinterpret_cast<const T*>(a.k) + b * a.ks.batch + h * a.ks.head + (int64_t)kj * a.ks.seq, a.D,
             lane, a.scale);
    load_row(vr, reinterpret_cast<const T*>(a.v) + b * a.vs.batch + h * a.vs.head + (int64_t)kj * a.vs.seq, a.D,
             lane, 1.f);
#pragma unroll
    for (int c = 0; c < kWC; ++c) { dk[c] = 0.f; dv[c] = 0.f; }
    int q_begin = 0;
    if (a.causal) q_begin = max(0, kj - a.causal_off);
    const int q_end = kj < kvlen ? a.Sq : 0;
    const int64_t stat0 = bh * a.Sq;
    for (int qi = q_begin; qi < q_end; ++qi) {
        if (!key_visible(a, b, qi, kj, kvlen)) continue;
        const float lse = a.lse_in[stat0 + qi];
        if (lse == -INFINITY) continue;
        float qr[kWC], gr[kWC];
        load_row(qr, qb + (int64_t)qi * a.qs.seq, a.D, lane, 1.f);
        load_row(gr, gb + (int64_t)qi * a.dos.seq, a.D, lane, 1.f);
        float v = dot_row(qr, kr);                     // kr carries the scale
        const float dp = dot_row(gr, vr);
        bool clamped = false;
        if (a.use_clamp && v >= a.clamp) { v = a.clamp; clamped = true; }
        const float p = expf(v - lse);
        const float ds = clamped ? 0.f : p * (dp - a.delta[stat0 + qi]) * a.scale;
#pragma unroll
        for (int c = 0; c < kWC; ++c) {
            dv[c] = fmaf(p, gr[c], dv[c]);
            dk[c] = fmaf(ds, qr[c], dk[c]);
        }
    }
    T* dkp = reinterpret_cast<T*>(a.dk) + b * a.dks.batch + h * a.dks.head + (int64_t)kj * a.dks.seq;
    T* dvp = reinterpret_cast<T*>(a.dv) + b * a.dvs.batch + h * a.dvs.head + (int64_t)kj * a.dvs.seq;
#pragma unroll
    for (int c = 0; c < kWC; ++c) {
        const int d = lane + 32 * c;
        if (d < a.D) { st_elem(dkp + d, dk[c]); st_elem(dvp + d, dv[c]); }
    }
}

template <typename T>
int run_wide(ltca_ctx* ctx, const CoreArgs& a, bool bwd) {
    const int64_t qrows = (int64_t)a.B * a.H * a.Sq, krows = (int64_t)a.B * a.H * a.Sk;
    const unsigned qblocks = (unsigned)((qrows + kWideWarps - 1) / kWideWarps);
    if (!bwd) {
        attn_fwd_wide_kernel<T><<<qblocks, kWideWarps * 32, 0, ctx->stream>>>(a);
        LTCA_LAUNCH_OK(ctx, "attn_fwd_wide_kernel");
        return LTCA_OK;
    }
    attn_bwd_delta_kernel<T><<<(unsigned)((qrows + 7) / 8), 256, 0, ctx->stream>>>(a);
    LTCA_LAUNCH_OK(ctx, "attn_bwd_delta_kernel");
    attn_bwd_dq_wide_kernel<T><<<qblocks, kWideWarps * 32, 0, ctx->stream>>>(a);
    LTCA_LAUNCH_OK(ctx, "attn_bwd_dq_wide_kernel");
    attn_bwd_dkv_wide_kernel<T><<<(unsigned)((krows + kWideWarps - 1) / kWideWarps), kWideWarps * 32, 0,
                                  ctx->stream>>>(a);
    LTCA_LAUNCH_OK(ctx, "attn_bwd_dkv_wide_kernel");
    return LTCA_OK;
}

template <typename T>
int dispatch(ltca_ctx* ctx, const CoreArgs& a, bool bwd) {
    if (a.D > 128) return run_wide<T>(ctx, a, bwd);
    const int dc = (a.D + 15) / 16;
#define LTCA_CASE(N) return bwd ? run_bwd<T, N>(ctx, a) : run_fwd<T, N>(ctx, a)
    if (dc <= 1) LTCA_CASE(1);
    if (dc <= 2) LTCA_CASE(2);
    if (dc <= 4) LTCA_CASE(4);
    LTCA_CASE(8);
#undef LTCA_CASE
}

}  // namespace

size_t attn_bwd_fp32_workspace(const ltca_attn_params* p) {
    return align_up((size_t)p->B * p->H * p->Sq * sizeof(float), 256);
}

int launch_attn_fwd_fp32(ltca_ctx* ctx, const ltca_attn_params* p) {
    if (p->D < 1 || p->D > kWideMaxD)
        return fail(ctx, LTCA_ERR_UNSUPPORTED, "fp32 attention supports head_dim 1..%d, got %d", kWideMaxD, p->D);
    CoreArgs a = make_args(p);
    return p->dtype == LTCA_BF16 ? dispatch<__nv_bfloat16>(ctx, a, false) : dispatch<float>(ctx, a, false);
}

int launch_attn_bwd_fp32(ltca_ctx* ctx, const ltca_attn_params* p) {
    if (p->D < 1 || p->D > kWideMaxD)
        return fail(ctx, LTCA_ERR_UNSUPPORTED, "fp32 attention supports head_dim 1..%d, got %d", kWideMaxD, p->D);
    if (p->workspace_bytes < attn_bwd_fp32_workspace(p) || !p->workspace)
        return fail(ctx, LTCA_ERR_WORKSPACE, "backward needs %zu bytes of workspace",
                    attn_bwd_fp32_workspace(p));
    CoreArgs a = make_args(p);
    a.delta = reinterpret_cast<float*>(p->workspace);
    return p->dtype == LTCA_BF16 ? dispatch<__nv_bfloat16>(ctx, a, true) : dispatch<float>(ctx, a, true);
}

}  // namespace ltca
