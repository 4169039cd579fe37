// Single-query attention over a key/value cache with per-sequence lengths.  The work is pure
// streaming of K and V (about 0.5 FLOP per byte), so the kernel is built around wide coalesced
// loads and keeps all arithmetic in fp32 registers:
//   - a group of D/4 lanes owns one key at a time (each lane a 16-byte slice of the row), the
//     score is a shuffle reduction inside the group, the value row is accumulated by the same
//     lanes without further communication;
//   - every group runs its own online softmax over the keys it visits; groups are merged once
//     per CTA through shared memory;
//   - when batch x heads cannot fill the GPU the key range is split across CTAs, partial
//     (max, sum, output) triples go to a caller-provided scratch buffer and a second small
//     kernel merges them;
//   - when batch x heads does fill the GPU but the sequences have different lengths, each
//     (batch, head) pair is a thread-block cluster of two or four CTAs that take alternate
//     32-key blocks of ITS keys and merge through distributed shared memory (no scratch, no
//     second kernel): the work per CTA is less uneven, which shortens the tail in which only
//     the CTAs of the longest sequences are still streaming.
// The reference has no counterpart: its cuDNN call always passes currIdx = -1
// (reference src/ml/cuDNN_ops.cu:206).
#include <cooperative_groups.h>
#include <math.h>

#include "host_common.h"

namespace ltca {

namespace {

constexpr int kDecThreads = 128;
constexpr int kUnroll = 4;

struct DecodeArgs {
    int B, H, Sk, D;
    float scale, clamp;
    int use_clamp;
    const void *q, *k, *v;
    void* o;
    ltca_strides qs, ks, vs, os;
    float* lse;
    const float* keep_mask;     // [B, 1, Sk]
    const int32_t* kv_len;
    int nsplit;
    float* partial;             // [B*H][nsplit][D + 2]; null when the splits are one cluster
};

__device__ __forceinline__ float4 ld4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st1(float* p, float v) { *p = v; }
__device__ __forceinline__ void st1(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// kCluster: the nsplit CTAs of one (batch, head) pair form a thread-block cluster (1, nsplit, 1).
template <typename T, int LPK, bool kCluster>
__global__ void __launch_bounds__(kDecThreads) attn_decode_kernel(const DecodeArgs a) {
    constexpr int D = 4 * LPK;
    constexpr int G = 32 / LPK;                         // key groups per warp
    constexpr int NG = (kDecThreads / 32) * G;          // key groups per CTA
    __shared__ float sm_o[NG][D];
    __shared__ float sm_m[NG], sm_l[NG];
    __shared__ float sm_part[D + 2];                    // this CTA's (max, sum, output) for the cluster merge

    const int bh = blockIdx.x;
    const int b = bh / a.H, h = bh % a.H;
    const int split = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = warp * G + lane / LPK;
    const int sub = lane % LPK;

    int kvlen = a.Sk;
    if (a.kv_len) kvlen = min(max(a.kv_len[b], 0), a.Sk);
    // the CTA's splits interleave at the granularity of one iteration (NG * kUnroll keys), so only
    // the sequence's last iteration is ragged, whatever the split count
    const int ks = 0, ke = kvlen;

    const T* qp = reinterpret_cast<const T*>(a.q) + b * a.qs.batch + h * a.qs.head + 4 * sub;
    const T* kp = reinterpret_cast<const T*>(a.k) + b * a.ks.batch + h * a.ks.head + 4 * sub;
    const T* vp = reinterpret_cast<const T*>(a.v) + b * a.vs.batch + h * a.vs.head + 4 * sub;
    const float* mrow = a.keep_mask ? a.keep_mask + (int64_t)b * a.Sk : nullptr;
    float4 q4 = ld4(qp);
    q4.x *= a.scale; q4.y *= a.scale; q4.z *= a.scale; q4.w *= a.scale;

    float m = -INFINITY, l = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    const int iters = (ke - ks + NG * kUnroll - 1) / (NG * kUnroll);
    for (int it = split; it < iters; it += a.nsplit) {
        float4 kk[kUnroll], vv[kUnroll];
        float s[kUnroll];
        bool live[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int j = ks + (it * kUnroll + u) * NG + g;
            live[u] = j < ke;
            const int jj = live[u] ? j : (ke - 1);            // in range: ke > ks here
            kk[u] = ld4(kp + (int64_t)jj * a.ks.seq);
            vv[u] = ld4(vp + (int64_t)jj * a.vs.seq);
            if (live[u] && mrow && mrow[j] == 0.f) live[u] = false;
        }
        float mt = m;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            float d = q4.x * kk[u].x + q4.y * kk[u].y + q4.z * kk[u].z + q4.w * kk[u].w;
#pragma unroll
            for (int off = LPK / 2; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
            if (a.use_clamp) d = fminf(d, a.clamp);
            s[u] = live[u] ? d : -INFINITY;
            mt = fmaxf(mt, s[u]);
        }
        const float m_safe = (mt == -INFINITY) ? 0.f : mt;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_safe);
        l *= corr;
        o.x *= corr; o.y *= corr; o.z *= corr; o.w *= corr;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const float p = expf(s[u] - m_safe);
            l += p;
            o.x = fmaf(p, vv[u].x, o.x);
            o.y = fmaf(p, vv[u].y, o.y);
            o.z = fmaf(p, vv[u].z, o.z);
            o.w = fmaf(p, vv[u].w, o.w);
        }
        m = mt;
    }
    sm_o[g][4 * sub + 0] = o.x;
    sm_o[g][4 * sub + 1] = o.y;
    sm_o[g][4 * sub + 2] = o.z;
    sm_o[g][4 * sub + 3] = o.w;
    if (sub == 0) { sm_m[g] = m; sm_l[g] = l; }
    __syncthreads();
    if (threadIdx.x < D) {
        const int d = threadIdx.x;
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < NG; ++i) M = fmaxf(M, sm_m[i]);
        const float Ms = (M == -INFINITY) ? 0.f : M;
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int i = 0; i < NG; ++i) {
            const float w = (sm_m[i] == -INFINITY) ? 0.f : expf(sm_m[i] - Ms);
            L = fmaf(sm_l[i], w, L);
            acc = fmaf(sm_o[i][d], w, acc);
        }
        if (kCluster) {
            sm_part[2 + d] = acc;
            if (d == 0) { sm_part[0] = M; sm_part[1] = L; }
        } else if (a.nsplit == 1) {
            T* op = reinterpret_cast<T*>(a.o) + b * a.os.batch + h * a.os.head;
            st1(op + d, L > 0.f ? acc / L : 0.f);
            if (d == 0 && a.lse) a.lse[bh] = L > 0.f ? M + logf(L) : -INFINITY;
        } else {
            float* part = a.partial + ((int64_t)bh * a.nsplit + split) * (D + 2);
            part[2 + d] = acc;
            if (d == 0) { part[0] = M; part[1] = L; }
        }
    }
    if (kCluster) {
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();                                  // every CTA's partial is in its shared memory
        if (cluster.block_rank() == 0 && threadIdx.x < D) {
            const int d = threadIdx.x;
            const int n = (int)cluster.num_blocks();
            float M = -INFINITY;
            for (int r = 0; r < n; ++r) M = fmaxf(M, cluster.map_shared_rank(sm_part, r)[0]);
            const float Ms = (M == -INFINITY) ? 0.f : M;
            float L = 0.f, acc = 0.f;
            for (int r = 0; r < n; ++r) {
                const float* ps = cluster.map_shared_rank(sm_part, r);
                const float w = (ps[0] == -INFINITY) ? 0.f : expf(ps[0] - Ms);
                L = fmaf(ps[1], w, L);
                acc = fmaf(ps[2 + d], w, acc);
            }
            T* op = reinterpret_cast<T*>(a.o) + b * a.os.batch + h * a.os.head;
            st1(op + d, L > 0.f ? acc / L : 0.f);
            if (d == 0 && a.lse) a.lse[bh] = L > 0.f ? M + logf(L) : -INFINITY;
        }
        cluster.sync();                                  // nobody leaves while its partial may still be read
    }
}

template <typename T>
__global__ void attn_decode_merge_kernel(const DecodeArgs a) {
    const int bh = blockIdx.x;
    const int b = bh / a.H, h = bh % a.H;
    const int d = threadIdx.x;
    if (d >= a.D) return;
    const float* part = a.partial + (int64_t)bh * a.nsplit * (a.D + 2);
    float M = -INFINITY;
    for (int s = 0; s < a.nsplit; ++s) M = fmaxf(M, part[s * (a.D + 2)]);
    const float Ms = (M == -INFINITY) ? 0.f : M;
    float L = 0.f, acc = 0.f;
    for (int s = 0; s < a.nsplit; ++s) {
        const float* ps = part + s * (a.D + 2);
        const float w = (ps[0] == -INFINITY) ? 0.f : expf(ps[0] - Ms);
        L = fmaf(ps[1], w, L);
        acc = fmaf(ps[2 + d], w, acc);
    }
    T* op = reinterpret_cast<T*>(a.o) + b * a.os.batch + h * a.os.head;
    st1(op + d, L > 0.f ? acc / L : 0.f);
    if (d == 0 && a.lse) a.lse[bh] = L > 0.f ? M + logf(L) : -INFINITY;
}

int pick_splits(const ltca_attn_params* p, int sm_count) {
    if (p->B < 1 || p->H < 1 || p->Sk < 1) return 1;      // nothing to split (and no division by zero below)
    const int64_t bh = (int64_t)p->B * p->H;
    if (sm_count <= 0) sm_count = kPlanSms;
    if (bh >= 2 * sm_count) return 1;
    int64_t want = (4 * (int64_t)sm_count + bh - 1) / bh;
    int64_t cap = (p->Sk + 255) / 256;
    int64_t n = want < cap ? want : cap;
    if (n < 1) n = 1;
    if (n > 64) n = 64;
    return (int)n;
}

// Splits of one (batch, head) pair that run as one cluster (0: none).  Used when batch x heads
// already fills the GPU (so the scratch path would not split) but the lengths differ.
int pick_cluster(const ltca_attn_params* p, int sm_count) {
#ifdef LTCA_DECODE_NO_CLUSTER
    return 0;
#endif
    if (pick_splits(p, sm_count) != 1) return 0;
    if (!p->kv_len || p->Sk < 512) return 0;
    // measured at B=256 H=8 lengths U{1..1024}: 2 CTAs 6112 GB/s, 4: 6011, 8: 4869 (1: 4820)
    return p->Sk < 2048 ? 2 : 4;
}

template <typename T, int LPK>
int run_decode(ltca_ctx* ctx, const DecodeArgs& a) {
    dim3 grid(a.B * a.H, a.nsplit);
    if (a.nsplit > 1 && !a.partial) {
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = grid;
        cfg.blockDim = dim3(kDecThreads);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = (unsigned)a.nsplit;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        LTCA_CUDA_OK(ctx, cudaLaunchKernelEx(&cfg, attn_decode_kernel<T, LPK, true>, a));
        return LTCA_OK;
    }
    attn_decode_kernel<T, LPK, false><<<grid, kDecThreads, 0, ctx->stream>>>(a);
    LTCA_LAUNCH_OK(ctx, "attn_decode_kernel");
    if (a.nsplit > 1) {
        attn_decode_merge_kernel<T><<<a.B * a.H, 128, 0, ctx->stream>>>(a);
        LTCA_LAUNCH_OK(ctx, "attn_decode_merge_kernel");
    }
    return LTCA_OK;
}

template <typename T>
int dispatch_decode(ltca_ctx* ctx, const DecodeArgs& a) {
    switch (a.D) {
        case 16: return run_decode<T, 4>(ctx, a);
        case 32: return run_decode<T, 8>(ctx, a);
        case 64: return run_decode<T, 16>(ctx, a);
        case 128: return run_decode<T, 32>(ctx, a);
    }
    return fail(ctx, LTCA_ERR_UNSUPPORTED, "decode supports head_dim 16, 32, 64, 128 (got %d)", a.D);
}

}  // namespace

// The split count must not depend on the context, so that the size query (which has no
// context) and the launch agree.  Non-positive shapes need no scratch (the launch refuses them).
size_t attn_decode_workspace(const ltca_attn_params* p) {
    if (p->B < 1 || p->H < 1 || p->Sk < 1 || p->D < 1) return 0;
    const int ns = pick_splits(p, kPlanSms);
    if (ns <= 1) return 0;
    return align_up((size_t)p->B * p->H * ns * (p->D + 2) * sizeof(float), 256);
}

int launch_attn_decode(ltca_ctx* ctx, const ltca_attn_params* p) {
    if (p->Sq != 1) return fail(ctx, LTCA_ERR_INVALID, "decode needs Sq == 1 (got %d)", p->Sq);
    const int es = elem_size(p->dtype);
    const int vec = 4 * es;     // bytes per lane load
    auto misaligned = [&](const void* ptr, const ltca_strides& s) {
        return (reinterpret_cast<uintptr_t>(ptr) % vec) || ((s.seq * es) % vec) ||
               ((s.head * es) % vec) || ((s.batch * es) % vec);
    };
    if (misaligned(p->q, p->q_strides) || misaligned(p->k, p->k_strides) ||
        misaligned(p->v, p->v_strides))
        return fail(ctx, LTCA_ERR_INVALID, "decode needs %d-byte aligned q/k/v rows", vec);
    DecodeArgs a;
    memset(&a, 0, sizeof(a));
    a.B = p->B; a.H = p->H; a.Sk = p->Sk; a.D = p->D;
    a.scale = p->scale;
    a.use_clamp = p->score_clamp > 0.f ? 1 : 0;
    a.clamp = p->score_clamp;
    a.q = p->q; a.k = p->k; a.v = p->v; a.o = p->o;
    a.qs = p->q_strides; a.ks = p->k_strides; a.vs = p->v_strides; a.os = p->o_strides;
    a.lse = p->lse;
    a.keep_mask = p->keep_mask;
    a.kv_len = p->kv_len;
    a.nsplit = pick_splits(p, kPlanSms);
    if (pick_cluster(p, kPlanSms) > 1) {
        a.nsplit = pick_cluster(p, kPlanSms);       // merged inside the cluster: a.partial stays null
    } else if (a.nsplit > 1) {
        const size_t need = attn_decode_workspace(p);
        if (!p->workspace || p->workspace_bytes < need)
            return fail(ctx, LTCA_ERR_WORKSPACE, "decode needs %zu bytes of workspace", need);
        a.partial = reinterpret_cast<float*>(p->workspace);
    }
    return p->dtype == LTCA_BF16 ? dispatch_decode<__nv_bfloat16>(ctx, a)
                                 : dispatch_decode<float>(ctx, a);
}

}  // namespace ltca

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the decode step.
//
// The regular entry point needs a context (whose creation makes one small device allocation)
// and, when the key range is split, a scratch buffer that the caller has to allocate.  Code
// that runs where device allocation is off limits -- a plug-in called from inside another
// framework's memory pool or arena, a real-time loop that forbids driver allocations after
// start-up, a host that hands out all device memory up front -- cannot provide either.  For
// those callers the split's partial results live in a fixed array that is part of the loaded
// library image, so the call touches no allocator at all.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = 256u << 10;   // 256 KiB, resident on every GPU that loads the library
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

// Device address of the array on each GPU, looked up on the first call there.  Host threads that make that
// first call at the same time all store the same value, hence relaxed atomics are enough.
constexpr int kMaxDevices = 64;
std::atomic<void*> g_static_scratch_ptr[kMaxDevices];

void set_err(char* buf, size_t len, const char* msg) {
    if (buf && len) snprintf(buf, len, "%s", msg);
}

}  // namespace

extern "C" int ltca_attn_decode_static(void* stream, const ltca_attn_params* p, char* err,
                                       size_t err_len) {
    if (!p) { set_err(err, err_len, "null parameter block"); return LTCA_ERR_INVALID; }
    // Arguments first: nothing below may divide by, or size a buffer from, a shape that is not positive.
    if (p->B < 1 || p->H < 1 || p->Sk < 1 || p->D < 1 || !p->q || !p->k || !p->v || !p->o ||
        !(p->scale > 0.f) || (p->dtype != LTCA_F32 && p->dtype != LTCA_BF16)) {
        set_err(err, err_len, "bad decode arguments (shape, null pointer, scale or dtype)");
        return LTCA_ERR_INVALID;
    }
    if (p->Sq != 1) {
        set_err(err, err_len, "decode needs Sq == 1");
        return LTCA_ERR_INVALID;
    }
    const size_t need = ltca::attn_decode_workspace(p);
    if (need > kStaticScratchBytes) {
        char msg[200];
        snprintf(msg, sizeof(msg),
                 "this decode shape needs %zu bytes of split scratch, the built-in array holds %zu; "
                 "use ltca_attn_decode with a caller-provided workspace", need, kStaticScratchBytes);
        set_err(err, err_len, msg);
        return LTCA_ERR_WORKSPACE;
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_err(err, err_len, "no current CUDA device (or device index above 63)");
        return LTCA_ERR_NO_DEVICE;
    }
    // One-time set-up per device, with that device current: in host code the array's name is
    // only a stand-in, the kernel needs the address the symbol has on THIS device.
    void* scratch = g_static_scratch_ptr[dev].load(std::memory_order_relaxed);
    if (!scratch) {
        cudaError_t e = cudaGetSymbolAddress(&scratch, g_decode_static_scratch);
        if (e != cudaSuccess || !scratch) {
            set_err(err, err_len, cudaGetErrorString(e));
            return LTCA_ERR_CUDA;
        }
        g_static_scratch_ptr[dev].store(scratch, std::memory_order_relaxed);
    }
    ltca_ctx tmp;                       // host-only bookkeeping: stream and error text
    tmp.device = dev;
    tmp.stream = reinterpret_cast<cudaStream_t>(stream);
    tmp.sm_count = tmp.sm_device = ltca::kPlanSms;    // only the split plan uses it, and that is fixed (see kPlanSms)
    ltca_attn_params q = *p;
    q.workspace = scratch;
    q.workspace_bytes = kStaticScratchBytes;
    const int rc = ltca::launch_attn_decode(&tmp, &q);
    if (rc) set_err(err, err_len, tmp.err);
    return rc;
}
