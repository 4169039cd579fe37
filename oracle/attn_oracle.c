/*
 * attn_oracle.c -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * An OpenMP fp64 host restatement of the attention path of Sirius437/CUDA_LTC.  Only the
 * test-suite, the smoke check and the CPU-baseline leg of the benchmark may load this
 * library; the shipped CUDA path never links, loads or calls it.
 *
 * What it restates (paths are inside the reference project):
 *   - attention core: scores = scale * Q K^T, keep-mask with "0 means masked"
 *     (src/ml/flash_attention.cu:151-164), optional upper clamp of the score
 *     (src/ml/flash_attention.cu:167), softmax over keys, O = P V
 *     (src/ml/flash_attention.cu:175-250, exact there for a single 16-key tile), the contract
 *     documented at include/flash_attention.h:213-230, scale = 1/sqrt(head_dim)
 *     (src/ml/flash_attention.cu:998), tensors [batch, heads, seq, head_dim]
 *     (src/ml/flash_attention.cu:19-23).
 *   - TimeSelfAttention module: per-head projections without bias, softmax(scale * Q K^T) V,
 *     output projection (include/cuDNN_ops.h:152-178), residual then post-LayerNorm with
 *     eps 1e-5 and biased variance (src/ml/cudnn_time_self_attention.cu:9-68, :211-252),
 *     backward = dQ-path + dK-path + dV-path input gradients with LayerNorm and residual
 *     treated as identity (src/ml/cudnn_time_self_attention.cu:254-302).
 *
 * Parity pin: the reference ships no golden vectors and no CPU path.  The oracle is pinned
 * against outputs of the reference's own flashAttentionKernel, built unmodified from the
 * reference sources and run on a GPU (see ref_driver.cu and tests/golden/ref_flash_case*), and
 * the module functions against the reference's own cuDNN TimeSelfAttention, linked from the
 * reference sources (see ref_tsa_driver.cu and tests/golden/ref_tsa_case*).
 *
 * Extensions beyond the reference (needed by the benchmark configurations): a causal flag,
 * per-sequence key lengths, a backward for the attention core, log-sum-exp output.
 *
 * Conventions
 *   - all tensors are float32 in memory with the head dimension contiguous and explicit
 *     element strides for (batch, head, sequence); results are float64.
 *   - causal: key j is visible to query i iff j <= i + (Sk - Sq).
 *   - kv_len[b] (optional): keys j >= kv_len[b] are invisible.
 *   - keep_mask[b, i, j] (optional, dense float [B, Sq, Sk]): value 0 hides key j from query i.
 *   - score_clamp > 0 applies s = min(s, score_clamp) to visible scores after scaling.
 *   - a query row that sees no key yields a zero output row, lse = -inf and zero gradients.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct {
    int32_t B, H, Sq, Sk, D;
    int32_t causal;
    float scale;
    float score_clamp;          /* <= 0: no clamp */
    const float* q;  int64_t q_sb, q_sh, q_ss;
    const float* k;  int64_t k_sb, k_sh, k_ss;
    const float* v;  int64_t v_sb, v_sh, v_ss;
    const float* keep_mask;     /* [B, Sq, Sk] or NULL */
    const int32_t* kv_len;      /* [B] or NULL */
} oracle_attn_desc;

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

static inline int visible(const oracle_attn_desc* a, int b, int i, int j) {
    if (a->kv_len && j >= a->kv_len[b]) return 0;
    if (a->causal && j > i + (a->Sk - a->Sq)) return 0;
    if (a->keep_mask && a->keep_mask[((int64_t)b * a->Sq + i) * a->Sk + j] == 0.0f) return 0;
    return 1;
}

/* Scores of one query row in fp64; hidden keys get -inf.  Returns the row maximum. */
static double score_row(const oracle_attn_desc* a, int b, int h, int i, double* s) {
    const float* qi = a->q + b * a->q_sb + h * a->q_sh + (int64_t)i * a->q_ss;
    const float* kb = a->k + b * a->k_sb + h * a->k_sh;
    double m = -INFINITY;
    for (int j = 0; j < a->Sk; ++j) {
        if (!visible(a, b, i, j)) { s[j] = -INFINITY; continue; }
        const float* kj = kb + (int64_t)j * a->k_ss;
        double acc = 0.0;
        for (int d = 0; d < a->D; ++d) acc += (double)qi[d] * (double)kj[d];
        acc *= (double)a->scale;
        if (a->score_clamp > 0.0f && acc > (double)a->score_clamp) acc = (double)a->score_clamp;
        s[j] = acc;
        if (acc > m) m = acc;
    }
    return m;
}

/*
 * Forward.  out [B,H,Sq,D] contiguous fp64, lse [B,H,Sq] fp64 (natural log).
 * Rows are processed only for (b,h) pairs with bh_begin <= b*H+h < bh_end so that a bounded
 * sample of a large problem can be evaluated.
 */
void oracle_attn_fwd(const oracle_attn_desc* a, double* out, double* lse,
                     int bh_begin, int bh_end) {
    const int B = a->B, H = a->H, Sq = a->Sq, Sk = a->Sk, D = a->D;
    if (bh_begin < 0) bh_begin = 0;
    if (bh_end > B * H) bh_end = B * H;
    const int64_t nrows = (int64_t)(bh_end - bh_begin) * Sq;
#pragma omp parallel
    {
        double* s = (double*)malloc(sizeof(double) * (size_t)(Sk > 0 ? Sk : 1));
#pragma omp for schedule(dynamic, 16)
        for (int64_t r = 0; r < nrows; ++r) {
            const int bh = bh_begin + (int)(r / Sq), i = (int)(r % Sq);
            const int b = bh / H, h = bh % H;
            double* o = out + ((int64_t)bh * Sq + i) * D;
            for (int d = 0; d < D; ++d) o[d] = 0.0;
            const double m = score_row(a, b, h, i, s);
            if (m == -INFINITY) { lse[(int64_t)bh * Sq + i] = -INFINITY; continue; }
            double l = 0.0;
            const float* vb = a->v + b * a->v_sb + h * a->v_sh;
            for (int j = 0; j < Sk; ++j) {
                if (s[j] == -INFINITY) continue;
                const double p = exp(s[j] - m);
                l += p;
                const float* vj = vb + (int64_t)j * a->v_ss;
                for (int d = 0; d < D; ++d) o[d] += p * (double)vj[d];
            }
            const double inv = 1.0 / l;
            for (int d = 0; d < D; ++d) o[d] *= inv;
            lse[(int64_t)bh * Sq + i] = m + log(l);
        }
        free(s);
    }
}

/*
 * Backward of the attention core.  dout [B,H,Sq,D] float32 with strides; dq [B,H,Sq,D],
 * dk/dv [B,H,Sk,D] contiguous fp64 (fully overwritten for the selected (b,h) range).
 * With P = softmax(S), dV = P^T dO, dP = dO V^T, dS = P o (dP - rowsum(dO o O)),
 * dQ = scale dS K, dK = scale dS^T Q.  A clamped score passes no gradient to Q and K.
 */
void oracle_attn_bwd(const oracle_attn_desc* a,
                     const float* dout, int64_t do_sb, int64_t do_sh, int64_t do_ss,
                     double* dq, double* dk, double* dv, int bh_begin, int bh_end) {
    const int B = a->B, H = a->H, Sq = a->Sq, Sk = a->Sk, D = a->D;
    if (bh_begin < 0) bh_begin = 0;
    if (bh_end > B * H) bh_end = B * H;
#pragma omp parallel
    {
        double* s  = (double*)malloc(sizeof(double) * (size_t)(Sk > 0 ? Sk : 1));
        double* dp = (double*)malloc(sizeof(double) * (size_t)(Sk > 0 ? Sk : 1));
        double* o  = (double*)malloc(sizeof(double) * (size_t)D);
#pragma omp for schedule(dynamic, 1)
        for (int bh = bh_begin; bh < bh_end; ++bh) {
            const int b = bh / H, h = bh % H;
            double* dqb = dq + (int64_t)bh * Sq * D;
            double* dkb = dk + (int64_t)bh * Sk * D;
            double* dvb = dv + (int64_t)bh * Sk * D;
            memset(dqb, 0, sizeof(double) * (size_t)Sq * D);
            memset(dkb, 0, sizeof(double) * (size_t)Sk * D);
            memset(dvb, 0, sizeof(double) * (size_t)Sk * D);
            const float* kb = a->k + b * a->k_sb + h * a->k_sh;
            const float* vb = a->v + b * a->v_sb + h * a->v_sh;
            for (int i = 0; i < Sq; ++i) {
                const double m = score_row(a, b, h, i, s);
                if (m == -INFINITY) continue;
                const float* qi  = a->q + b * a->q_sb + h * a->q_sh + (int64_t)i * a->q_ss;
                const float* doi = dout + b * do_sb + h * do_sh + (int64_t)i * do_ss;
                double l = 0.0;
                for (int j = 0; j < Sk; ++j) {
                    if (s[j] == -INFINITY) { dp[j] = 0.0; continue; }
                    l += exp(s[j] - m);
                }
                const double inv = 1.0 / l;
                for (int d = 0; d < D; ++d) o[d] = 0.0;
                for (int j = 0; j < Sk; ++j) {
                    if (s[j] == -INFINITY) continue;
                    const double p = exp(s[j] - m) * inv;
                    const float* vj = vb + (int64_t)j * a->v_ss;
                    double acc = 0.0;
                    for (int d = 0; d < D; ++d) {
                        o[d] += p * (double)vj[d];
                        acc += (double)doi[d] * (double)vj[d];
                    }
                    dp[j] = acc;
                }
                double delta = 0.0;
                for (int d = 0; d < D; ++d) delta += (double)doi[d] * o[d];
                for (int j = 0; j < Sk; ++j) {
                    if (s[j] == -INFINITY) continue;
                    const double p = exp(s[j] - m) * inv;
                    double* dvj = dvb + (int64_t)j * D;
                    for (int d = 0; d < D; ++d) dvj[d] += p * (double)doi[d];
                    double ds = p * (dp[j] - delta) * (double)a->scale;
                    if (a->score_clamp > 0.0f && s[j] >= (double)a->score_clamp) ds = 0.0;
                    const float* kj = kb + (int64_t)j * a->k_ss;
                    double* dkj = dkb + (int64_t)j * D;
                    double* dqi = dqb + (int64_t)i * D;
                    for (int d = 0; d < D; ++d) {
                        dqi[d] += ds * (double)kj[d];
                        dkj[d] += ds * (double)qi[d];
                    }
                }
            }
        }
        free(s); free(dp); free(o);
    }
}

/* ------------------------------------------------------------------------------------------
 * TimeSelfAttention module oracle.
 *
 * x [rows, E] float32, rows = B*S.  Row r holds (b, t) with r = b*S + t (batch-major) or
 * r = t*B + b (time_major != 0; the order the reference hands to cuDNN, include/cuDNN_ops.h:322-328).
 * Wq, Wk, Wv [E, H*W] row-major (y = x W), Wo [H*W, E]; W is the per-head width: E/H in the
 * benchmark form, E in the reference-compatible form (include/cuDNN_ops.h:152-178).
 * Optional biases bq,bk,bv [H*W], bo [E] (FlashAttention form, src/ml/flash_attention.cu:458-470).
 * ---------------------------------------------------------------------------------------- */
typedef struct {
    int32_t B, S, E, H, W;
    int32_t causal, time_major, use_residual, use_layer_norm;
    float scale, score_clamp, ln_eps;
    const float *x, *wq, *wk, *wv, *wo, *bq, *bk, *bv, *bo, *gamma, *beta;
    const float* keep_mask;     /* [B,S,S] or NULL */
    const int32_t* kv_len;      /* [B] or NULL */
} oracle_tsa_desc;

static inline int64_t tsa_row(const oracle_tsa_desc* t, int b, int s) {
    return t->time_major ? ((int64_t)s * t->B + b) : ((int64_t)b * t->S + s);
}

/* y[rows, N] = x[rows, K] * w[K, N] (+ bias[N]) in fp64 from float32 inputs. */
static void gemm_f32_in(const float* x, const float* w, const float* bias,
                        int64_t rows, int K, int N, double* y) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        double* yr = y + r * N;
        for (int n = 0; n < N; ++n) yr[n] = bias ? (double)bias[n] : 0.0;
        for (int k = 0; k < K; ++k) {
            const double xv = (double)x[r * K + k];
            const float* wr = w + (int64_t)k * N;
            for (int n = 0; n < N; ++n) yr[n] += xv * (double)wr[n];
        }
    }
}

/* y[rows, N] (+)= a[rows, K] * w[N, K]^T with fp64 a and float32 w. */
static void gemm_f64_wT(const double* a, const float* w, int64_t rows, int K, int N,
                        double* y, int accumulate) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const double* ar = a + r * K;
        double* yr = y + r * N;
        for (int n = 0; n < N; ++n) {
            const float* wn = w + (int64_t)n * K;
            double acc = 0.0;
            for (int k = 0; k < K; ++k) acc += ar[k] * (double)wn[k];
            yr[n] = accumulate ? yr[n] + acc : acc;
        }
    }
}

/*
 * Attention over fp64 projected tensors laid out [rows, H*W] (head-major inside a row).
 * Writes ctx [rows, H*W].  If dctx != NULL also computes dq, dk, dv [rows, H*W].
 */
static void tsa_core(const oracle_tsa_desc* t, const double* q, const double* k, const double* v,
                     double* ctx, const double* dctx, double* dq, double* dk, double* dv) {
    const int B = t->B, S = t->S, H = t->H, W = t->W;
    const int64_t HW = (int64_t)H * W;
    if (dctx) {
        memset(dq, 0, sizeof(double) * (size_t)B * S * HW);
        memset(dk, 0, sizeof(double) * (size_t)B * S * HW);
        memset(dv, 0, sizeof(double) * (size_t)B * S * HW);
    }
#pragma omp parallel
    {
        double* s  = (double*)malloc(sizeof(double) * (size_t)S);
        double* dp = (double*)malloc(sizeof(double) * (size_t)S);
#pragma omp for schedule(dynamic, 1)
        for (int bh = 0; bh < B * H; ++bh) {
            const int b = bh / H, h = bh % H;
            for (int i = 0; i < S; ++i) {
                const int64_t ri = tsa_row(t, b, i);
                const double* qi = q + ri * HW + (int64_t)h * W;
                double m = -INFINITY;
                for (int j = 0; j < S; ++j) {
                    int vis = 1;
                    if (t->kv_len && j >= t->kv_len[b]) vis = 0;
                    if (t->causal && j > i) vis = 0;
                    if (t->keep_mask && t->keep_mask[((int64_t)b * S + i) * S + j] == 0.0f) vis = 0;
                    if (!vis) { s[j] = -INFINITY; continue; }
                    const double* kj = k + tsa_row(t, b, j) * HW + (int64_t)h * W;
                    double acc = 0.0;
                    for (int d = 0; d < W; ++d) acc += qi[d] * kj[d];
                    acc *= (double)t->scale;
                    if (t->score_clamp > 0.0f && acc > (double)t->score_clamp) acc = (double)t->score_clamp;
                    s[j] = acc;
                    if (acc > m) m = acc;
                }
                double* ci = ctx + ri * HW + (int64_t)h * W;
                for (int d = 0; d < W; ++d) ci[d] = 0.0;
                if (m == -INFINITY) continue;
                double l = 0.0;
                for (int j = 0; j < S; ++j) if (s[j] != -INFINITY) l += exp(s[j] - m);
                const double inv = 1.0 / l;
                for (int j = 0; j < S; ++j) {
                    if (s[j] == -INFINITY) continue;
                    const double p = exp(s[j] - m) * inv;
                    const double* vj = v + tsa_row(t, b, j) * HW + (int64_t)h * W;
                    for (int d = 0; d < W; ++d) ci[d] += p * vj[d];
                }
                if (!dctx) continue;
                const double* doi = dctx + ri * HW + (int64_t)h * W;
                double delta = 0.0;
                for (int d = 0; d < W; ++d) delta += doi[d] * ci[d];
                for (int j = 0; j < S; ++j) {
                    if (s[j] == -INFINITY) continue;
                    const int64_t rj = tsa_row(t, b, j);
                    const double p = exp(s[j] - m) * inv;
                    const double* vj = v + rj * HW + (int64_t)h * W;
                    const double* kj = k + rj * HW + (int64_t)h * W;
                    double acc = 0.0;
                    for (int d = 0; d < W; ++d) acc += doi[d] * vj[d];
                    double ds = p * (acc - delta) * (double)t->scale;
                    if (t->score_clamp > 0.0f && s[j] >= (double)t->score_clamp) ds = 0.0;
                    double* dvj = dv + rj * HW + (int64_t)h * W;
                    double* dkj = dk + rj * HW + (int64_t)h * W;
                    double* dqi = dq + ri * HW + (int64_t)h * W;
                    for (int d = 0; d < W; ++d) {
                        dvj[d] += p * doi[d];
                        dqi[d] += ds * kj[d];
                        dkj[d] += ds * qi[d];
                    }
                }
            }
        }
        free(s); free(dp);
    }
}

/* fp64 -> float32 -> fp64 is NOT applied anywhere: intermediates stay fp64. */
static double* f64_alloc(int64_t n) { return (double*)calloc((size_t)(n > 0 ? n : 1), sizeof(double)); }

/*
 * Module forward: out [rows, E] fp64.  If attn_out != NULL it receives the pre-residual,
 * pre-LayerNorm projection output y.
 */
void oracle_tsa_fwd(const oracle_tsa_desc* t, double* out, double* attn_out) {
    const int64_t rows = (int64_t)t->B * t->S;
    const int E = t->E, HW = t->H * t->W;
    double *q = f64_alloc(rows * HW), *k = f64_alloc(rows * HW), *v = f64_alloc(rows * HW);
    double *ctx = f64_alloc(rows * HW);
    gemm_f32_in(t->x, t->wq, t->bq, rows, E, HW, q);
    gemm_f32_in(t->x, t->wk, t->bk, rows, E, HW, k);
    gemm_f32_in(t->x, t->wv, t->bv, rows, E, HW, v);
    tsa_core(t, q, k, v, ctx, NULL, NULL, NULL, NULL);
    /* y = ctx * Wo (+ bo) */
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        double* yr = out + r * E;
        for (int e = 0; e < E; ++e) yr[e] = t->bo ? (double)t->bo[e] : 0.0;
        for (int c = 0; c < HW; ++c) {
            const double cv = ctx[r * HW + c];
            const float* wr = t->wo + (int64_t)c * E;
            for (int e = 0; e < E; ++e) yr[e] += cv * (double)wr[e];
        }
        if (attn_out) memcpy(attn_out + r * E, yr, sizeof(double) * (size_t)E);
        if (t->use_residual) for (int e = 0; e < E; ++e) yr[e] += (double)t->x[r * E + e];
        if (t->use_layer_norm) {
            double mean = 0.0, var = 0.0;
            for (int e = 0; e < E; ++e) mean += yr[e];
            mean /= E;
            for (int e = 0; e < E; ++e) { const double dlt = yr[e] - mean; var += dlt * dlt; }
            var /= E;
            const double inv_std = 1.0 / sqrt(var + (double)t->ln_eps);
            for (int e = 0; e < E; ++e)
                yr[e] = (yr[e] - mean) * inv_std * (t->gamma ? (double)t->gamma[e] : 1.0)
                        + (t->beta ? (double)t->beta[e] : 0.0);
        }
    }
    free(q); free(k); free(v); free(ctx);
}

/*
 * Module backward.  dy [rows, E] float32 is the gradient w.r.t. the projection output y
 * (the reference passes the incoming gradient straight through LayerNorm and the residual,
 * src/ml/cudnn_time_self_attention.cu:291-299).  dx [rows, E] = dQ Wq^T + dK Wk^T + dV Wv^T.
 * Weight gradients (each may be NULL): dwq, dwk, dwv [E, H*W], dwo [H*W, E], overwritten
 * (the reference uses CUDNN_WGRAD_MODE_SET, src/ml/cuDNN_ops.cu:366-385).
 */
void oracle_tsa_bwd(const oracle_tsa_desc* t, const float* dy, double* dx,
                    double* dwq, double* dwk, double* dwv, double* dwo) {
    const int64_t rows = (int64_t)t->B * t->S;
    const int E = t->E, HW = t->H * t->W;
    double *q = f64_alloc(rows * HW), *k = f64_alloc(rows * HW), *v = f64_alloc(rows * HW);
    double *ctx = f64_alloc(rows * HW), *dctx = f64_alloc(rows * HW);
    double *dq = f64_alloc(rows * HW), *dk = f64_alloc(rows * HW), *dv = f64_alloc(rows * HW);
    gemm_f32_in(t->x, t->wq, t->bq, rows, E, HW, q);
    gemm_f32_in(t->x, t->wk, t->bk, rows, E, HW, k);
    gemm_f32_in(t->x, t->wv, t->bv, rows, E, HW, v);
    /* dctx = dy * Wo^T : [rows, HW] */
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int c = 0; c < HW; ++c) {
            const float* wr = t->wo + (int64_t)c * E;
            double acc = 0.0;
            for (int e = 0; e < E; ++e) acc += (double)dy[r * E + e] * (double)wr[e];
            dctx[r * HW + c] = acc;
        }
    tsa_core(t, q, k, v, ctx, dctx, dq, dk, dv);
    if (dx) {
        gemm_f64_wT(dq, t->wq, rows, HW, E, dx, 0);
        gemm_f64_wT(dk, t->wk, rows, HW, E, dx, 1);
        gemm_f64_wT(dv, t->wv, rows, HW, E, dx, 1);
    }
    const double* grads[3] = {dq, dk, dv};
    double* outs[3] = {dwq, dwk, dwv};
    for (int w = 0; w < 3; ++w) {
        if (!outs[w]) continue;
        double* dw = outs[w];
        const double* g = grads[w];
#pragma omp parallel for schedule(static)
        for (int e = 0; e < E; ++e)
            for (int c = 0; c < HW; ++c) {
                double acc = 0.0;
                for (int64_t r = 0; r < rows; ++r) acc += (double)t->x[r * E + e] * g[r * HW + c];
                dw[(int64_t)e * HW + c] = acc;
            }
    }
    if (dwo) {
#pragma omp parallel for schedule(static)
        for (int c = 0; c < HW; ++c)
            for (int e = 0; e < E; ++e) {
                double acc = 0.0;
                for (int64_t r = 0; r < rows; ++r) acc += ctx[r * HW + c] * (double)dy[r * E + e];
                dwo[(int64_t)c * E + e] = acc;
            }
    }
    free(q); free(k); free(v); free(ctx); free(dctx); free(dq); free(dk); free(dv);
}
