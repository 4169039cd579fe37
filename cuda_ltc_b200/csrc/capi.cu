// C-ABI entry points declared in include/ltc_attn.h: context handling, argument checks,
// dispatch between the tensor-pipe kernels and the fp32 kernels, and the small elementwise
// helpers that sit on the attention path of the reference (tensor add, LayerNorm, finite check).
#include <new>

#include "host_common.h"
#include "sm100_ptx.cuh"
#include "attn_wide.h"

namespace ltca {
int launch_attn_fwd_sm100_bf16in(ltca_ctx* ctx, const ltca_attn_params* p, const void* q,
                                 const void* k, const void* v, const ltca_strides& qs,
                                 const ltca_strides& ks, const ltca_strides& vs);

namespace {

// ---- elementwise kernels ----------------------------------------------------------------------
__global__ void add_kernel(const float* __restrict__ a, const float* __restrict__ b,
                           float* __restrict__ r, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t n4 = n / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 x = reinterpret_cast<const float4*>(a)[i];
        const float4 y = reinterpret_cast<const float4*>(b)[i];
        reinterpret_cast<float4*>(r)[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
    }
    for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        r[i] = a[i] + b[i];
}
__global__ void add_scalar_kernel(const float* a, const float* b, float* r, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) r[i] = a[i] + b[i];
}

// One warp per row: two-pass mean / biased variance in registers, shuffle reductions.
__global__ void layer_norm_kernel(float* x, const float* __restrict__ gamma,
                                  const float* __restrict__ beta, int64_t rows, int E, float eps) {
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    float* xr = x + row * E;
    float sum = 0.f;
    for (int i = lane; i < E; i += 32) sum += xr[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / E;
    float var = 0.f;
    for (int i = lane; i < E; i += 32) {
        const float d = xr[i] - mean;
        var = fmaf(d, d, var);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
    const float inv_std = rsqrtf(var / E + eps);
    for (int i = lane; i < E; i += 32)
        xr[i] = (xr[i] - mean) * inv_std * (gamma ? gamma[i] : 1.f) + (beta ? beta[i] : 0.f);
}

__global__ void validate_finite_kernel(const float* __restrict__ x, size_t n, int32_t* flag) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    bool bad = false;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = x[i];
        bad |= !(fabsf(v) <= 3.402823466e38f);      // false for NaN and Inf
    }
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicExch(flag, 1);
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ s, __nv_bfloat16* __restrict__ d, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        d[i] = __float2bfloat16_rn(s[i]);
}
__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ s, float* __restrict__ d, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        d[i] = __bfloat162float(s[i]);
}

// Strided fp32 [B,H,S,D] -> contiguous bf16 [B,H,S,D]; one thread per 4 elements (D % 4 == 0).  blockIdx.y picks
// the tensor, so the operands of one attention call are packed by one launch.
struct PackJobs {
    const float* src[kMaxPackJobs];
    __nv_bfloat16* dst[kMaxPackJobs];
    __nv_bfloat16* lo[kMaxPackJobs];
    ltca_strides st[kMaxPackJobs];
    int S[kMaxPackJobs];
};
__global__ void pack_bf16_kernel(const __grid_constant__ PackJobs jobs, int BH, int H, int D) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int j = blockIdx.y;
    const float* __restrict__ src = jobs.src[j];
    __nv_bfloat16* __restrict__ dst = jobs.dst[j];
    __nv_bfloat16* __restrict__ low = jobs.lo[j];
    const ltca_strides st = jobs.st[j];
    const int S = jobs.S[j];
    const int d4 = D / 4;
    const size_t n4 = (size_t)BH * S * d4;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const int dd = (int)(i % d4);
        size_t r = i / d4;
        const int s = (int)(r % S); r /= S;
        const int h = (int)(r % H);
        const int64_t b = (int64_t)(r / H);
        const float4 v = *reinterpret_cast<const float4*>(src + b * st.batch + h * st.head + (int64_t)s * st.seq + 4 * dd);
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&lo);
        u.y = *reinterpret_cast<uint32_t*>(&hi);
        reinterpret_cast<uint2*>(dst)[i] = u;
        if (low) {
            const __nv_bfloat162 l0 = __floats2bfloat162_rn(v.x - __low2float(lo), v.y - __high2float(lo));
            const __nv_bfloat162 l1 = __floats2bfloat162_rn(v.z - __low2float(hi), v.w - __high2float(hi));
            uint2 w;
            w.x = *reinterpret_cast<const uint32_t*>(&l0);
            w.y = *reinterpret_cast<const uint32_t*>(&l1);
            reinterpret_cast<uint2*>(low)[i] = w;
        }
    }
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// Half a warp per row i of the block (rows s0 .. s0+n of each of the BH accumulator slabs), four
// elements per lane and pass:
//   lse' = log(exp(lse_acc) + exp(lse_blk)),  o_acc = o_acc * exp(lse_acc - lse') + o_blk * exp(lse_blk - lse').
// A block row with no visible key carries lse_blk = -inf and leaves the accumulator as it is.
// D is a multiple of 4 and both tensors are 16-byte aligned (checked by the caller).
template <typename T>
__global__ void attn_merge_kernel(float* __restrict__ o_acc, float* __restrict__ lse_acc,
                                  const T* __restrict__ o_blk, const float* __restrict__ lse_blk,
                                  int64_t BH, int S_acc, int s0, int n, int D) {
    const int64_t row = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 2 + ((threadIdx.x >> 4) & 1);
    const bool live = row < BH * n;
    const int sub = threadIdx.x & 15;
    int64_t arow = 0;
    float wa = 1.f, wb = 0.f, lnew = 0.f;
    bool touch = false;
    if (live) {
        const int64_t bh = row / n;
        const int i = (int)(row % n);
        arow = bh * S_acc + s0 + i;
        const float la = lse_acc[arow], lb = lse_blk[row];
        if (lb != -INFINITY) {
            const float m = fmaxf(la, lb);
            const float ea = (la == -INFINITY) ? 0.f : __expf(la - m), eb = __expf(lb - m);
            const float inv = 1.f / (ea + eb);
            wa = ea * inv;
            wb = eb * inv;
            lnew = m + __logf(ea + eb);
            touch = true;
        }
    }
    if (touch) {
        float* oa = o_acc + arow * D;
        const T* ob = o_blk + row * D;
        for (int d = 4 * sub; d < D; d += 64) {
            float4 a = *reinterpret_cast<float4*>(oa + d);
            const float4 b = load4(ob + d);
            a.x = a.x * wa + b.x * wb;
            a.y = a.y * wa + b.y * wb;
            a.z = a.z * wa + b.z * wb;
            a.w = a.w * wa + b.w * wb;
            *reinterpret_cast<float4*>(oa + d) = a;
        }
    }
    __syncwarp();                        // every lane has read the old lse before it is replaced
    if (touch && sub == 0) lse_acc[arow] = lnew;
}

// acc[bh][s0 + i][d] += part[bh][i][d], four elements per thread (D is a multiple of 4)
template <typename T>
__global__ void accumulate_rows_kernel(float* __restrict__ acc, const T* __restrict__ part, int64_t total4,
                                       int S_acc, int s0, int n, int D) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int D4 = D >> 2;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total4; e += stride) {
        const int d = (int)(e % D4) * 4;
        const int64_t r = e / D4;
        const int64_t bh = r / n;
        const int i = (int)(r % n);
        float* dst = acc + (bh * S_acc + s0 + i) * D + d;
        float4 a = *reinterpret_cast<float4*>(dst);
        const float4 b = load4(part + e * 4);
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        *reinterpret_cast<float4*>(dst) = a;
    }
}

// One warp waits on a barrier that nothing ever arrives at: the path every bounded wait of the tensor-pipe
// kernels takes when its producer never shows up, with a limit short enough for a test.
__global__ void bounded_wait_selftest_kernel(uint32_t* status, unsigned long long limit_ns) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0u;
        mbar_init(smem_u32(&bar), 1);
        mbar_fence_init();
    }
    __syncthreads();
    const WaitCtx wc{&abort_flag, status, limit_ns};
    mbar_wait_warp(smem_u32(&bar), 0, wc, 0x7f);
}

inline int blocks_for(size_t n, int threads, int sm_count) {
    size_t b = (n + threads - 1) / threads;
    const size_t cap = (size_t)(sm_count > 0 ? sm_count : kPlanSms) * 16;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (int)b;
}

int check_common(ltca_ctx* ctx, const ltca_attn_params* p) {
    if (!ctx) return LTCA_ERR_INVALID;
    if (!p) return fail(ctx, LTCA_ERR_INVALID, "null parameter block");
    if (p->B < 1 || p->H < 1 || p->Sq < 1 || p->Sk < 1 || p->D < 1)
        return fail(ctx, LTCA_ERR_INVALID, "B, H, Sq, Sk, D must be positive (got %d %d %d %d %d)",
                    p->B, p->H, p->Sq, p->Sk, p->D);
    if (p->dtype != LTCA_F32 && p->dtype != LTCA_BF16)
        return fail(ctx, LTCA_ERR_INVALID, "unknown dtype %d", p->dtype);
    if (p->mode != LTCA_MODE_AUTO && p->mode != LTCA_MODE_BF16 && p->mode != LTCA_MODE_FP32 &&
        p->mode != LTCA_MODE_SPLIT)
        return fail(ctx, LTCA_ERR_INVALID, "unknown mode %d", p->mode);
    if (!p->q || !p->k || !p->v || !p->o)
        return fail(ctx, LTCA_ERR_INVALID, "q, k, v and o must be non-null");
    if (!(p->scale > 0.f) || !isfinite(p->scale))
        return fail(ctx, LTCA_ERR_INVALID, "scale must be positive and finite");
    return LTCA_OK;
}

// LTCA_MODE_SPLIT with fp32 storage: every operand in two bf16 terms, written-out scores (with bf16 storage there
// are no low-order bits to keep and the mode is LTCA_MODE_BF16).
bool split_mode(const ltca_attn_params* p) { return p->mode == LTCA_MODE_SPLIT && p->dtype == LTCA_F32; }

bool tensor_path(const ltca_attn_params* p, bool backward) {
    if (p->mode == LTCA_MODE_FP32 || split_mode(p)) return false;
    const bool ok = backward ? attn_bwd_sm100_supported(p) : attn_fwd_sm100_supported(p);
    if (!ok) return false;
    if (p->dtype == LTCA_F32 && (p->D % 4)) return false;
    return true;
}

size_t packed_bytes(const ltca_attn_params* p, int S) {
    return align_up((size_t)p->B * p->H * S * p->D * 2, 256);
}

ltca_strides contiguous_strides(int H, int S, int D) {
    ltca_strides s;
    s.seq = D;
    s.head = (int64_t)S * D;
    s.batch = (int64_t)H * S * D;
    return s;
}

// The materialised-score path (attn_wide_sm100.cu) behind the core entry points: on explicit request
// (LTCA_MODE_BF16) for head widths the streaming kernels do not cover, any multiple of 8.
bool wide_core_path(const ltca_attn_params* p, bool backward) {
    if (p->mode != LTCA_MODE_BF16 && !split_mode(p)) return false;
    // (the split mode takes this path at every head width: the streaming kernels carry single bf16 operands)
    if (!split_mode(p) && (backward ? attn_bwd_sm100_supported(p) : attn_fwd_sm100_supported(p))) return false;
    if (p->D < 8 || (p->D % 8) || p->Sq < 1 || p->Sk < 1 || !(p->scale > 0.f)) return false;
    if (p->dtype == LTCA_BF16) {
        if (!wide_supported(p->D, p->q_strides, p->k_strides, p->v_strides)) return false;
        if ((p->o_strides.seq % 8) || (p->o_strides.head % 8) || (p->o_strides.batch % 8)) return false;
    } else if ((p->o_strides.seq % 4) || (p->o_strides.head % 4) || (p->o_strides.batch % 4)) {
        return false;
    }
    return true;
}

size_t wide_core_workspace(const ltca_attn_params* p, bool backward) {
    size_t n = 0;
    if (p->dtype == LTCA_F32)
        n += (packed_bytes(p, p->Sq) * (backward ? 2 : 1) + 2 * packed_bytes(p, p->Sk)) * (split_mode(p) ? 2 : 1);
    const size_t elems = wide_matrix_elems(p->B, p->H, p->Sq, p->Sk);
    n += align_up(elems * 4, 256) + align_up(elems * 2, 256);       // raw scores, probabilities
    if (p->dtype == LTCA_F32) n += align_up(elems * 2, 256);         // second term of the probabilities (fp32 results)
    if (backward) n += align_up(elems * 4, 256);                     // dP
    return n;
}

int launch_wide_core(ltca_ctx* ctx, const ltca_attn_params* p, bool backward) {
    const size_t need = wide_core_workspace(p, backward);
    if (!p->workspace || p->workspace_bytes < need)
        return fail(ctx, LTCA_ERR_WORKSPACE, "this head width on the tensor pipe needs %zu bytes of workspace", need);
    if (reinterpret_cast<uintptr_t>(p->workspace) & 255)
        return fail(ctx, LTCA_ERR_INVALID, "workspace must be 256-byte aligned");
    char* w = reinterpret_cast<char*>(p->workspace);
    WideArgs a;
    a.B = p->B; a.H = p->H; a.Sq = p->Sq; a.Sk = p->Sk; a.D = p->D;
    a.causal = p->causal ? 1 : 0;
    a.scale = p->scale; a.clamp = p->score_clamp;
    a.keep_mask = p->keep_mask; a.kv_len = p->kv_len;
    a.qh = p->q; a.kh = p->k; a.v = p->v;
    a.qs = p->q_strides; a.ks = p->k_strides; a.vs = p->v_strides;
    a.dout = p->dout; a.dos = p->do_strides;
    int rc;
    if (split_mode(p)) {
        // q, k, v (and dO) as two bf16 terms each
        const size_t nq = packed_bytes(p, p->Sq), nk = packed_bytes(p, p->Sk);
        void* qh = w; w += nq;  void* ql = w; w += nq;
        void* kh = w; w += nk;  void* kl = w; w += nk;
        void* vh = w; w += nk;  void* vl = w; w += nk;
        PackJob jobs[kMaxPackJobs] = {{p->q, p->q_strides, qh, p->Sq, ql}, {p->k, p->k_strides, kh, p->Sk, kl},
                                      {p->v, p->v_strides, vh, p->Sk, vl}, {}};
        a.qh = qh; a.ql = ql; a.kh = kh; a.kl = kl; a.v = vh; a.vl = vl;
        a.qs = contiguous_strides(p->H, p->Sq, p->D);
        a.ks = a.vs = contiguous_strides(p->H, p->Sk, p->D);
        if (backward) {
            void* gh = w; w += nq;  void* gl = w; w += nq;
            jobs[3] = {p->dout, p->do_strides, gh, p->Sq, gl};
            a.dout = gh; a.doutl = gl; a.dos = a.qs;
        }
        if ((rc = pack_many_to_bf16(ctx, jobs, backward ? 4 : 3, p->B, p->H, p->D))) return rc;
    } else if (p->dtype == LTCA_F32) {
        void* qb = w; w += packed_bytes(p, p->Sq);
        void* kb = w; w += packed_bytes(p, p->Sk);
        void* vb = w; w += packed_bytes(p, p->Sk);
        PackJob jobs[kMaxPackJobs] = {{p->q, p->q_strides, qb, p->Sq}, {p->k, p->k_strides, kb, p->Sk},
                                      {p->v, p->v_strides, vb, p->Sk}, {}};
        a.qh = qb; a.kh = kb; a.v = vb;
        a.qs = contiguous_strides(p->H, p->Sq, p->D);
        a.ks = a.vs = contiguous_strides(p->H, p->Sk, p->D);
        if (backward) {
            void* gb = w; w += packed_bytes(p, p->Sq);
            jobs[3] = {p->dout, p->do_strides, gb, p->Sq};
            a.dout = gb; a.dos = a.qs;
        }
        if ((rc = pack_many_to_bf16(ctx, jobs, backward ? 4 : 3, p->B, p->H, p->D))) return rc;
    }
    const size_t elems = wide_matrix_elems(p->B, p->H, p->Sq, p->Sk);
    a.scores = reinterpret_cast<float*>(w); w += align_up(elems * 4, 256);
    a.P = w; w += align_up(elems * 2, 256);
    if (p->dtype == LTCA_F32) { a.Plo = w; w += align_up(elems * 2, 256); }
    const int bf16 = p->dtype == LTCA_BF16 ? 1 : 0;
    if (!backward) {
        a.o = p->o; a.os = p->o_strides; a.o_bf16 = bf16; a.lse = p->lse;
        return wide_attn_fwd(ctx, a);
    }
    // the probabilities are formed again from Q and K (the forward's result and lse are not needed for that)
    a.dP = reinterpret_cast<float*>(w);
    a.o = nullptr; a.lse = nullptr;
    if ((rc = wide_attn_fwd(ctx, a))) return rc;
    a.dq = p->dq; a.dk = p->dk; a.dv = p->dv;
    a.dqs = p->dq_strides; a.dks = p->dk_strides; a.dvs = p->dv_strides;
    a.grads_bf16 = bf16;
    return wide_attn_bwd(ctx, a);
}

}  // namespace

int pack_many_to_bf16(ltca_ctx* ctx, const PackJob* jobs, int count, int B, int H, int D) {
    if (count < 1 || count > kMaxPackJobs || (D % 4))
        return fail(ctx, LTCA_ERR_INVALID, "pack: %d tensors of head_dim %d", count, D);
    PackJobs k{};
    int s_max = 0;
    for (int j = 0; j < count; ++j) {
        const ltca_strides& st = jobs[j].st;
        if ((reinterpret_cast<uintptr_t>(jobs[j].src) & 15) || (st.seq % 4) || (st.head % 4) || (st.batch % 4))
            return fail(ctx, LTCA_ERR_INVALID, "fp32 tensors need 16-byte aligned rows for the tensor-pipe modes");
        k.src[j] = reinterpret_cast<const float*>(jobs[j].src);
        k.dst[j] = reinterpret_cast<__nv_bfloat16*>(jobs[j].dst);
        k.lo[j] = reinterpret_cast<__nv_bfloat16*>(jobs[j].lo);
        k.st[j] = st;
        k.S[j] = jobs[j].S;
        if (jobs[j].S > s_max) s_max = jobs[j].S;
    }
    // the grid is sized for the longest tensor; 16 blocks per SM over all the tensors together
    const size_t n4 = (size_t)B * H * s_max * D / 4;
    int bx = blocks_for(n4, 256, ctx->sm_count);
    const int cap = (ctx->sm_count > 0 ? ctx->sm_count : kPlanSms) * 16 / count;
    if (bx > cap) bx = cap;
    LTCA_CUDA_OK(ctx, launch_dependent(pack_bf16_kernel, dim3((unsigned)bx, (unsigned)count), dim3(256), 0, ctx->stream, k,
                                       B * H, H, D));
    LTCA_LAUNCH_OK(ctx, "pack_bf16_kernel");
    return LTCA_OK;
}
}  // namespace ltca

using namespace ltca;

extern "C" {

int ltca_version(void) { return LTCA_VERSION; }

int ltca_ctx_create(int device, void* stream, ltca_ctx** out) {
    if (!out) return LTCA_ERR_INVALID;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0 || device < 0 || device >= count) {
        cudaGetLastError();
        return LTCA_ERR_NO_DEVICE;
    }
    ltca_ctx* ctx = new (std::nothrow) ltca_ctx();
    if (!ctx) return LTCA_ERR_CUDA;
    ctx->device = device;
    ctx->stream = reinterpret_cast<cudaStream_t>(stream);
    cudaDeviceProp prop;
    if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
        delete ctx;
        return LTCA_ERR_CUDA;
    }
    ctx->sm_count = ctx->sm_device = prop.multiProcessorCount;
    ctx->cc_major = prop.major;
    ctx->cc_minor = prop.minor;
    if (prop.major != 10) {
        delete ctx;
        return LTCA_ERR_NO_DEVICE;       // the kernels are built for sm_100a only
    }
    // one small allocation: the status word, then the work-item counters of the persistent kernels
    if (cudaMalloc(&ctx->d_status, 16 * sizeof(uint32_t)) != cudaSuccess ||
        cudaMemset(ctx->d_status, 0, 16 * sizeof(uint32_t)) != cudaSuccess) {
        delete ctx;
        return LTCA_ERR_CUDA;
    }
    ctx->d_sched = reinterpret_cast<int*>(ctx->d_status + 4);
    *out = ctx;
    return LTCA_OK;
}

int ltca_ctx_enable_kernel_timing(ltca_ctx* ctx, int enable) {
    if (!ctx) return LTCA_ERR_INVALID;
    LTCA_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    if (enable && !ctx->kev[0])
        for (int i = 0; i < 4; ++i) LTCA_CUDA_OK(ctx, cudaEventCreate(&ctx->kev[i]));
    ctx->time_kernels = enable != 0;
    ctx->kev_recorded = 0;
    return LTCA_OK;
}

int ltca_ctx_last_bwd_kernel_ms(ltca_ctx* ctx, float* ms_out) {
    if (!ctx || !ms_out) return LTCA_ERR_INVALID;
    if (!ctx->time_kernels || ctx->kev_recorded < 4)
        return fail(ctx, LTCA_ERR_INVALID, "no timed tensor-pipe backward has run on this context");
    LTCA_CUDA_OK(ctx, cudaEventSynchronize(ctx->kev[3]));
    for (int i = 0; i < 3; ++i) LTCA_CUDA_OK(ctx, cudaEventElapsedTime(&ms_out[i], ctx->kev[i], ctx->kev[i + 1]));
    return LTCA_OK;
}

int ltca_ctx_set_stream(ltca_ctx* ctx, void* stream) {
    if (!ctx) return LTCA_ERR_INVALID;
    ctx->stream = reinterpret_cast<cudaStream_t>(stream);
    return LTCA_OK;
}

void ltca_ctx_destroy(ltca_ctx* ctx) {
    if (!ctx) return;
    for (int i = 0; i < 4; ++i)
        if (ctx->kev[i]) cudaEventDestroy(ctx->kev[i]);
    if (ctx->d_status) cudaFree(ctx->d_status);
    delete ctx;
}

const char* ltca_last_error(const ltca_ctx* ctx) { return ctx ? ctx->err : "null context"; }

int ltca_device_status(ltca_ctx* ctx, uint32_t* status_out) {
    if (!ctx || !status_out) return LTCA_ERR_INVALID;
    uint32_t v = 0;
    LTCA_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    LTCA_CUDA_OK(ctx, cudaMemcpyAsync(&v, ctx->d_status, sizeof(v), cudaMemcpyDeviceToHost, ctx->stream));
    LTCA_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    // a kernel that gave up may have left its work-item counters mid-count: clear everything
    if (v) LTCA_CUDA_OK(ctx, cudaMemsetAsync(ctx->d_status, 0, 16 * sizeof(uint32_t), ctx->stream));
    *status_out = v;
    if (v) return fail(ctx, LTCA_ERR_DEVICE, "device status word 0x%08x", v);
    return LTCA_OK;
}

int ltca_selftest_bounded_wait(ltca_ctx* ctx, uint32_t limit_us) {
    if (!ctx) return LTCA_ERR_INVALID;
    if (limit_us < 1 || limit_us > 1000000)
        return fail(ctx, LTCA_ERR_INVALID, "limit must be between 1 us and 1 s (got %u us)", limit_us);
    LTCA_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    bounded_wait_selftest_kernel<<<1, 32, 0, ctx->stream>>>(ctx->d_status, 1000ull * limit_us);
    LTCA_LAUNCH_OK(ctx, "bounded_wait_selftest_kernel");
    return LTCA_OK;
}

int ltca_attn_uses_tensor_pipe(const ltca_attn_params* p, int backward) {
    if (!p) return 0;
    return (tensor_path(p, backward != 0) || wide_core_path(p, backward != 0)) ? 1 : 0;
}

int ltca_attn_workspace_bytes(const ltca_attn_params* p, int backward, size_t* bytes_out) {
    if (!p || !bytes_out) return LTCA_ERR_INVALID;
    size_t n = 0;
    if (wide_core_path(p, backward != 0)) {
        n = wide_core_workspace(p, backward != 0);
    } else if (tensor_path(p, backward != 0)) {
        if (p->dtype == LTCA_F32) {
            n += packed_bytes(p, p->Sq) + 2 * packed_bytes(p, p->Sk);     // q, k, v as bf16
            if (backward) n += packed_bytes(p, p->Sq);                     // dO as bf16
        }
        if (backward) n += attn_bwd_sm100_workspace(p);
    } else if (backward) {
        n += attn_bwd_fp32_workspace(p);
    }
    *bytes_out = n;
    return LTCA_OK;
}

int ltca_attn_fwd(ltca_ctx* ctx, const ltca_attn_params* p) {
    int rc = check_common(ctx, p);
    if (rc) return rc;
    LTCA_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    if (wide_core_path(p, false)) return launch_wide_core(ctx, p, false);
    if (p->mode == LTCA_MODE_BF16 && !tensor_path(p, false))
        return fail(ctx, LTCA_ERR_UNSUPPORTED,
                    "the tensor-pipe forward needs a head_dim that is a multiple of 8 with 16-byte aligned rows (got %d)",
                    p->D);
    if (!tensor_path(p, false)) return launch_attn_fwd_fp32(ctx, p);
    if (p->dtype == LTCA_BF16)
        return launch_attn_fwd_sm100_bf16in(ctx, p, p->q, p->k, p->v, p->q_strides, p->k_strides,
                                            p->v_strides);
    size_t need = 0;
    ltca_attn_workspace_bytes(p, 0, &need);
    if (!p->workspace || p->workspace_bytes < need)
        return fail(ctx, LTCA_ERR_WORKSPACE, "forward needs %zu bytes of workspace", need);
    if (reinterpret_cast<uintptr_t>(p->workspace) & 255)
        return fail(ctx, LTCA_ERR_INVALID, "workspace must be 256-byte aligned");
    char* w = reinterpret_cast<char*>(p->workspace);
    void* qb = w;  w += packed_bytes(p, p->Sq);
    void* kb = w;  w += packed_bytes(p, p->Sk);
    void* vb = w;
    const PackJob jobs[3] = {{p->q, p->q_strides, qb, p->Sq}, {p->k, p->k_strides, kb, p->Sk},
                             {p->v, p->v_strides, vb, p->Sk}};
    if ((rc = pack_many_to_bf16(ctx, jobs, 3, p->B, p->H, p->D))) return rc;
    return launch_attn_fwd_sm100_bf16in(ctx, p, qb, kb, vb, contiguous_strides(p->H, p->Sq, p->D),
                                        contiguous_strides(p->H, p->Sk, p->D),
                                        contiguous_strides(p->H, p->Sk, p->D));
}

int ltca_attn_bwd(ltca_ctx* ctx, const ltca_attn_params* p) {
    int rc = check_common(ctx, p);
    if (rc) return rc;
    if (!p->dout || !p->dq || !p->dk || !p->dv || !p->lse)
        return fail(ctx, LTCA_ERR_INVALID, "backward needs dout, dq, dk, dv and lse");
    LTCA_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    if (p->workspace && (reinterpret_cast<uintptr_t>(p->workspace) & 255))
        return fail(ctx, LTCA_ERR_INVALID, "workspace must be 256-byte aligned");
    if (wide_core_path(p, true)) return launch_wide_core(ctx, p, true);
    if (p->mode == LTCA_MODE_BF16 && !tensor_path(p, true))
        return fail(ctx, LTCA_ERR_UNSUPPORTED, "the tensor-pipe backward does not cover this problem");
    if (!tensor_path(p, true)) return launch_attn_bwd_fp32(ctx, p);
    return launch_attn_bwd_sm100(ctx, p);
}

int ltca_attn_decode(ltca_ctx* ctx, const ltca_attn_params* p) {
    int rc = check_common(ctx, p);
    if (rc) return rc;
    LTCA_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    if (p->workspace && (reinterpret_cast<uintptr_t>(p->workspace) & 255))
        return fail(ctx, LTCA_ERR_INVALID, "workspace must be 256-byte aligned");
    return launch_attn_decode(ctx, p);
}

int ltca_attn_decode_workspace_bytes(const ltca_attn_params* p, size_t* bytes_out) {
    if (!p || !bytes_out) return LTCA_ERR_INVALID;
    *bytes_out = attn_decode_workspace(p);
    return LTCA_OK;
}

int ltca_ctx_set_sm_limit(ltca_ctx* ctx, int32_t n_sms) {
    if (!ctx) return LTCA_ERR_INVALID;
    ctx->sm_count = (n_sms <= 0 || n_sms > ctx->sm_device) ? ctx->sm_device : n_sms;
    return LTCA_OK;
}

int ltca_add_tensors(ltca_ctx* ctx, const float* a, const float* b, float* r, size_t n) {
    if (!ctx) return LTCA_ERR_INVALID;
    if (!a || !b || !r) return fail(ctx, LTCA_ERR_INVALID, "null tensor");
    if (n == 0) return LTCA_OK;
    LTCA_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    const bool aligned = !((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                            reinterpret_cast<uintptr_t>(r)) & 15);
    if (aligned)
        add_kernel<<<blocks_for(n / 4 + 1, 256, ctx->sm_count), 256, 0, ctx->stream>>>(a, b, r, n);
    else
        add_scalar_kernel<<<blocks_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(a, b, r, n);
    LTCA_LAUNCH_OK(ctx, "add_kernel");
    return LTCA_OK;
}

int ltca_attn_merge(ltca_ctx* ctx, float* o_acc, float* lse_acc, const void* o_blk, int32_t blk_dtype,
                    const float* lse_blk, int64_t BH, int32_t S_acc, int32_t s0, int32_t n, int32_t D) {
    if (!ctx) return LTCA_ERR_INVALID;
    if (!o_acc || !lse_acc || !o_blk || !lse_blk) return fail(ctx, LTCA_ERR_INVALID, "null tensor");
    if (BH < 0 || S_acc < 0 || s0 < 0 || n < 0 || D < 1 || s0 + n > S_acc)
        return fail(ctx, LTCA_ERR_INVALID, "bad row range %d + %d of %d", s0, n, S_acc);
    if (blk_dtype != LTCA_F32 && blk_dtype != LTCA_BF16) return fail(ctx, LTCA_ERR_INVALID, "bad dtype");
    if (BH * n == 0) return LTCA_OK;
    LTCA_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    if ((D & 3) || ((reinterpret_cast<uintptr_t>(o_acc) | reinterpret_cast<uintptr_t>(o_blk)) & 15))
        return fail(ctx, LTCA_ERR_INVALID, "head_dim must be a multiple of 4 and the tensors 16-byte aligned");
    const int wpb = 8;                                         // two rows per warp
    const unsigned grid = (unsigned)((BH * n + 2 * wpb - 1) / (2 * wpb));
    if (blk_dtype == LTCA_F32)
        attn_merge_kernel<float><<<grid, wpb * 32, 0, ctx->stream>>>(
            o_acc, lse_acc, static_cast<const float*>(o_blk), lse_blk, BH, S_acc, s0, n, D);
    else
        attn_merge_kernel<__nv_bfloat16><<<grid, wpb * 32, 0, ctx->stream>>>(
            o_acc, lse_acc, static_cast<const __nv_bfloat16*>(o_blk), lse_blk, BH, S_acc, s0, n, D);
    LTCA_LAUNCH_OK(ctx, "attn_merge_kernel");
    return LTCA_OK;
}

int ltca_accumulate_rows(ltca_ctx* ctx, float* acc, const void* part, int32_t part_dtype, int64_t BH,
                         int32_t S_acc, int32_t s0, int32_t n, int32_t D) {
    if (!ctx) return LTCA_ERR_INVALID;
    if (!acc || !part) return fail(ctx, LTCA_ERR_INVALID, "null tensor");
    if (BH < 0 || S_acc < 0 || s0 < 0 || n < 0 || D < 1 || s0 + n > S_acc)
        return fail(ctx, LTCA_ERR_INVALID, "bad row range %d + %d of %d", s0, n, S_acc);
    if (part_dtype != LTCA_F32 && part_dtype != LTCA_BF16) return fail(ctx, LTCA_ERR_INVALID, "bad dtype");
    if ((D & 3) || ((reinterpret_cast<uintptr_t>(acc) | reinterpret_cast<uintptr_t>(part)) & 15))
        return fail(ctx, LTCA_ERR_INVALID, "head_dim must be a multiple of 4 and the tensors 16-byte aligned");
    const int64_t total = BH * n * (D >> 2);
    if (total == 0) return LTCA_OK;
    LTCA_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    const int grid = blocks_for((size_t)total, 256, ctx->sm_count);
    if (part_dtype == LTCA_F32)
        accumulate_rows_kernel<float><<<grid, 256, 0, ctx->stream>>>(
            acc, static_cast<const float*>(part), total, S_acc, s0, n, D);
    else
        accumulate_rows_kernel<__nv_bfloat16><<<grid, 256, 0, ctx->stream>>>(
            acc, static_cast<const __nv_bfloat16*>(part), total, S_acc, s0, n, D);
    LTCA_LAUNCH_OK(ctx, "accumulate_rows_kernel");
    return LTCA_OK;
}

int ltca_layer_norm(ltca_ctx* ctx, float* x, const float* gamma, const float* beta, int64_t rows,
                    int32_t E) {
    if (!ctx) return LTCA_ERR_INVALID;
    if (!x || rows < 0 || E < 1) return fail(ctx, LTCA_ERR_INVALID, "bad LayerNorm arguments");
    if (rows == 0) return LTCA_OK;
    LTCA_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    const int wpb = 8;
    layer_norm_kernel<<<(unsigned)((rows + wpb - 1) / wpb), wpb * 32, 0, ctx->stream>>>(
        x, gamma, beta, rows, E, 1e-5f);
    LTCA_LAUNCH_OK(ctx, "layer_norm_kernel");
    return LTCA_OK;
}

int ltca_validate_finite(ltca_ctx* ctx, const float* x, size_t n, int32_t* flag_out) {
    if (!ctx) return LTCA_ERR_INVALID;
    if (!flag_out || (!x && n > 0)) return fail(ctx, LTCA_ERR_INVALID, "null argument");
    LTCA_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    LTCA_CUDA_OK(ctx, cudaMemsetAsync(flag_out, 0, sizeof(int32_t), ctx->stream));
    if (n == 0) return LTCA_OK;                 // nothing to check: clean
    validate_finite_kernel<<<blocks_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(x, n, flag_out);
    LTCA_LAUNCH_OK(ctx, "validate_finite_kernel");
    return LTCA_OK;
}

int ltca_f32_to_bf16(ltca_ctx* ctx, const float* src, void* dst, size_t n) {
    if (!ctx) return LTCA_ERR_INVALID;
    if (!src || !dst) return fail(ctx, LTCA_ERR_INVALID, "null argument");
    if (n == 0) return LTCA_OK;
    LTCA_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    f32_to_bf16_kernel<<<blocks_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(
        src, reinterpret_cast<__nv_bfloat16*>(dst), n);
    LTCA_LAUNCH_OK(ctx, "f32_to_bf16_kernel");
    return LTCA_OK;
}

int ltca_bf16_to_f32(ltca_ctx* ctx, const void* src, float* dst, size_t n) {
    if (!ctx) return LTCA_ERR_INVALID;
    if (!src || !dst) return fail(ctx, LTCA_ERR_INVALID, "null argument");
    if (n == 0) return LTCA_OK;
    LTCA_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    bf16_to_f32_kernel<<<blocks_for(n, 256, ctx->sm_count), 256, 0, ctx->stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(src), dst, n);
    LTCA_LAUNCH_OK(ctx, "bf16_to_f32_kernel");
    return LTCA_OK;
}

}  // extern "C"
