// Attention backward on the sm_100a tensor pipe (head_dim 64, bf16 operands, fp32 accumulation).
//
// With P = softmax(scale * Q K^T) recomputed from Q, K and the forward's log-sum-exp:
//   delta_i = sum_d dO[i,d] O[i,d]        dP = dO V^T        dS = P o (dP - delta)
//   dV = P^T dO        dK = scale * dS^T Q        dQ = scale * dS K
// The reference reaches this arithmetic through cudnnMultiHeadAttnBackwardData
// (reference src/ml/cuDNN_ops.cu:240-337); its FlashAttention class has no backward.
//
// Three launches, no atomics (two runs give identical bits; the reference's tests pin backward
// repeatability, src/ml/time_self_attention_test.cu:799-838):
//   1. attn_bwd_stats_kernel: delta and lse * log2(e) into padded [B*H, Sq_pad] fp32 rows
//      (padding and fully hidden rows get lse = +inf so that their P is exactly 0).
//   2. attn_bwd_dq_sm100_kernel: one CTA per 256 query rows; Q and dO tiles stay in shared
//      memory, K/V stream through a ring in 64-key steps.  Per step and 128-row tile:
//      S = Q K^T and dP = dO V^T into tensor memory, the elementwise warps (one query row per
//      thread) turn them into dS (bf16, written back over S), and dQ += dS K takes dS from
//      tensor memory and K as an MN-major operand from shared memory.
//   3. attn_bwd_dkv_sm100_kernel: the transposed problem, one CTA per 256 keys; K and V tiles
//      stay in shared memory, Q/dO (and the per-row statistics) stream in 64-query steps.
//      S^T = K Q^T and dP^T = V dO^T put one KEY per tensor-memory lane, so P^T and dS^T are
//      directly the A operands of dV += P^T dO and dK += dS^T Q.
// Both main kernels share the forward's structure: warps 0-3 / 4-7 elementwise for tile 0 / 1,
// warp 8 issues tcgen05.mma, warp 9 drives TMA; the two tiles are interleaved so one tile's
// elementwise work overlaps the other's contractions.  Every wait is bounded.
#include <type_traits>

#include "host_common.h"
#include "sm100_ptx.cuh"
#include "trace.cuh"


namespace ltca {

namespace {

constexpr int kTile = 128;          // rows of a resident tile (queries in dQ, keys in dKV)
constexpr int kStep = 64;           // streamed rows per step
constexpr int kD = 64;
constexpr int kThreads = 640;        // 16 elementwise warps + one warpgroup of control warps
constexpr int kMmaWarp0 = 16;        // issues the contractions of tile 0 (tile 1: the next warp)
constexpr int kTmaWarp = 18;
constexpr uint32_t kTmemCols = 512;
constexpr int kLaunchRegs = 96;      // registers per thread at launch (65536 / 640 rounded down to 8)
constexpr int kCtrlRegs = 56;        // kept by the TMA / MMA-issue warps
constexpr int kMathRegs = 104;       // taken by the elementwise warps
// setmaxnreg can only redistribute what the CTA was launched with; asking for more never returns
static_assert(512 * kMathRegs + 128 * kCtrlRegs <= kThreads * kLaunchRegs, "register budget");
constexpr int kBigTile = kTile * kD * 2;      // 16 KB
constexpr int kSmallTile = kStep * kD * 2;    // 8 KB

struct BwdArgs {
    int B, H, Sq, Sk, Sq_pad;
    int causal, causal_off;
    float scale, scale_log2;
    float clamp_raw, clamp_log2;     // clamp / scale ; clamp * log2(e)
    int use_clamp;
    const float* lse2;               // [B*H, Sq_pad]
    const float* delta;              // [B*H, Sq_pad]
    void *dq, *dk, *dv;
    ltca_strides dqs, dks, dvs;
    const float* keep_mask;
    const int32_t* kv_len;
    uint32_t* status;
};

__device__ __forceinline__ float neg_inf() { return __int_as_float(0xff800000); }
__device__ __forceinline__ float pos_inf() { return __int_as_float(0x7f800000); }

// ---------------------------------------------------------------------------------------------
// 1. statistics: 8 lanes per query row, 8 elements per lane (head_dim 64)
// ---------------------------------------------------------------------------------------------
struct StatsArgs {
    int B, H, Sq, Sq_pad;
    const void *o, *dout;
    ltca_strides os, dos;
    const float* lse;
    float *lse2, *delta;
    float* dq_acc;           // optional: fp32 [B*H, Sq_pad, 64] accumulator of the fused kernel, cleared here
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void load8(const float* p, float (&f)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

template <typename T>
__global__ void __launch_bounds__(256) attn_bwd_stats_kernel(const StatsArgs a) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int64_t row = (int64_t)blockIdx.x * 32 + (threadIdx.x >> 3);
    const int sub = threadIdx.x & 7;
    const int64_t total = (int64_t)a.B * a.H * a.Sq_pad;
    if (row >= total) return;                    // whole 8-lane groups leave together
    const int qi = (int)(row % a.Sq_pad);
    const int64_t bh = row / a.Sq_pad;
    const int h = (int)(bh % a.H), b = (int)(bh / a.H);
    if (a.dq_acc) {
        float4* z = reinterpret_cast<float4*>(a.dq_acc + row * kD + 8 * sub);
        z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
        z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float acc = 0.f;
    if (qi < a.Sq) {
        const T* o = reinterpret_cast<const T*>(a.o) + b * a.os.batch + h * a.os.head + (int64_t)qi * a.os.seq + 8 * sub;
        const T* g = reinterpret_cast<const T*>(a.dout) + b * a.dos.batch + h * a.dos.head + (int64_t)qi * a.dos.seq + 8 * sub;
        float fo[8], fg[8];
        load8(o, fo);
        load8(g, fg);
        // fp32 storage: the contractions see dO rounded to bf16, and sum_j P_ij dP_ij equals
        // delta_i only when delta is formed from the same rounded dO
        if constexpr (sizeof(T) == 4) {
#pragma unroll
            for (int i = 0; i < 8; ++i) fg[i] = __bfloat162float(__float2bfloat16_rn(fg[i]));
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = fmaf(fo[i], fg[i], acc);
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    if (sub == 0) {
        float l2 = pos_inf();
        if (qi < a.Sq) {
            const float l = a.lse[bh * a.Sq + qi];
            l2 = (l == neg_inf()) ? pos_inf() : l * 1.4426950408889634f;
        }
        a.lse2[row] = l2;
        a.delta[row] = acc;
    }
}

// ---------------------------------------------------------------------------------------------
// shared-memory plans
// ---------------------------------------------------------------------------------------------
struct DqSmem {
    static constexpr int kStages = 8;                         // ring of 8 KB K / V step tiles
    static constexpr int kQOff = 0;                           // Q0, Q1
    static constexpr int kDoOff = 2 * kBigTile;               // dO0, dO1
    static constexpr int kRingOff = 4 * kBigTile;
    static constexpr int kBarOff = kRingOff + kStages * kSmallTile;
    // bars: qdo_full, ring_full[S], ring_empty[S], sdp_full[2], sdp_free[2], ds_full[2], dq_done[2], stagger
    static constexpr int kNumBars = 1 + 2 * kStages + 9;
    static constexpr int kMiscOff = kBarOff + kNumBars * 8;
    static constexpr int kDynBytes = kMiscOff + 16 + 1024;
};

struct DkvSmem {
    static constexpr int kStages = 6;                         // ring of (Q_j, dO_j, lse2_j, delta_j)
    static constexpr int kStageBytes = 2 * kSmallTile + 1024; // stats padded to keep 1024-B alignment
    static constexpr int kKOff = 0;                           // K0, K1
    static constexpr int kVOff = 2 * kBigTile;                // V0, V1
    static constexpr int kRingOff = 4 * kBigTile;
    static constexpr int kBarOff = kRingOff + kStages * kStageBytes;
    // bars: kv_full, ring_full[S], ring_empty[S], sdp_full[2], pds_full[2], acc_done[2], stagger
    static constexpr int kNumBars = 1 + 2 * kStages + 7;
    static constexpr int kMiscOff = kBarOff + kNumBars * 8;
    static constexpr int kDynBytes = kMiscOff + 16 + 1024;
};

template <typename OutT>
__device__ __forceinline__ void store_row32(OutT* dst, const uint32_t (&o)[32], float mul) {
    if constexpr (sizeof(OutT) == 2) {
        uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]) * mul, __uint_as_float(o[8 * v + 1]) * mul);
            w.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]) * mul, __uint_as_float(o[8 * v + 3]) * mul);
            w.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]) * mul, __uint_as_float(o[8 * v + 5]) * mul);
            w.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]) * mul, __uint_as_float(o[8 * v + 7]) * mul);
            d[v] = w;
        }
    } else {
        float4* d = reinterpret_cast<float4*>(dst);
#pragma unroll
        for (int v = 0; v < 8; ++v)
            d[v] = make_float4(__uint_as_float(o[4 * v + 0]) * mul, __uint_as_float(o[4 * v + 1]) * mul,
                               __uint_as_float(o[4 * v + 2]) * mul, __uint_as_float(o[4 * v + 3]) * mul);
    }
}

// Packs 32 fp32 values into 16 bf16 pairs (and, for the split variants, the rounding residue).
template <bool kSplit>
__device__ __forceinline__ void pack32(const uint32_t (&v)[32], uint32_t (&hi)[16], uint32_t (&lo)[16]) {
#pragma unroll
    for (int cc = 0; cc < 32; cc += 2) {
        const float v0 = __uint_as_float(v[cc]), v1 = __uint_as_float(v[cc + 1]);
        const uint32_t h01 = pack_bf16x2(v0, v1);
        hi[cc / 2] = h01;
        if constexpr (kSplit)
            lo[cc / 2] = pack_bf16x2(v0 - __uint_as_float(h01 << 16), v1 - __uint_as_float(h01 & 0xffff0000u));
    }
}

// ---------------------------------------------------------------------------------------------
// 2. dQ
// tensor memory: tile t at t*192: S [0,64)  dP [64,128)  dQ [128,192);
// dS (bf16) of tile t at 384 + t*32, its low-order term (kSplit) at 448 + t*32.
// A query row belongs to two threads (warps w and w + 8), each owning 32 of the step's 64 keys.
// ---------------------------------------------------------------------------------------------
// kSplit (fp32 gradients out): dS is written as two bf16 terms and the dQ contraction runs once
// per term, so that the 2^-9 rounding of a single bf16 dS does not dominate the error of an fp32
// result.
template <typename OutT, bool kSplit>
__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_dq_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q,
                         const __grid_constant__ CUtensorMap tmap_do,
                         const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, const BwdArgs a) {
    using L = DqSmem;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t q_smem = smem_base + L::kQOff, do_smem = smem_base + L::kDoOff;
    const uint32_t ring_smem = smem_base + L::kRingOff, bar_base = smem_base + L::kBarOff;
    auto bar_qdo_full = [&]() { return bar_base; };
    auto bar_ring_full = [&](int s) { return bar_base + 8u * (1 + s); };
    auto bar_ring_empty = [&](int s) { return bar_base + 8u * (1 + L::kStages + s); };
    auto bar_sdp_full = [&](int t) { return bar_base + 8u * (1 + 2 * L::kStages + t); };
    auto bar_sdp_free = [&](int t) { return bar_base + 8u * (3 + 2 * L::kStages + t); };
    auto bar_ds_full = [&](int t) { return bar_base + 8u * (5 + 2 * L::kStages + t); };
    auto bar_dq_done = [&](int t) { return bar_base + 8u * (7 + 2 * L::kStages + t); };
    auto bar_stagger = [&]() { return bar_base + 8u * (9 + 2 * L::kStages); };
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_block = gridDim.x - 1 - blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;

    int kvlen = a.Sk;
    if (a.kv_len) {
        grid_dependency_wait();                // the lengths may come from the kernel before this one
        kvlen = min(max(a.kv_len[b], 0), a.Sk);
    }
    int n_steps[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int q0 = m_block * 2 * kTile + t * kTile;
        int lim = 0;
        if (q0 < a.Sq) {
            lim = kvlen;
            if (a.causal) lim = min(lim, min(q0 + kTile - 1, a.Sq - 1) + a.causal_off + 1);
        }
        n_steps[t] = lim > 0 ? (lim + kStep - 1) / kStep : 0;
    }
    const int n_max = max(n_steps[0], n_steps[1]);

    if (threadIdx.x == 0) {
        mbar_init(bar_qdo_full(), 1);
        for (int s = 0; s < L::kStages; ++s) { mbar_init(bar_ring_full(s), 1); mbar_init(bar_ring_empty(s), 2); }
        for (int t = 0; t < 2; ++t) {
            mbar_init(bar_sdp_full(t), 1);
            mbar_init(bar_sdp_free(t), 8);         // one arrival per elementwise warp of the tile
            mbar_init(bar_ds_full(t), 8);
            mbar_init(bar_dq_done(t), 1);
        }
        mbar_init(bar_stagger(), 8);
        misc[1] = 0u;
        mbar_fence_init();
    }
    if (warp == kMmaWarp0) { tmem_alloc(smem_u32(const_cast<uint32_t*>(&misc[0])), kTmemCols); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = misc[0];
    const WaitCtx wc{&misc[1], a.status};
    grid_launch_dependents();                  // (set up: the next kernel may place its CTAs)
    grid_dependency_wait();                    // the operands are complete once the kernel before this one has ended
    auto slot_of = [&](int item) { return item % L::kStages; };
    auto phase_of = [&](int item) { return (uint32_t)((item / L::kStages) & 1); };
    LTCA_TRACE_DECL(LTCA_TRACE_KERNEL == 1 && blockIdx.x == 0 && blockIdx.y == 5 && blockIdx.z == 0);
    LTCA_TRACE_EVT(0x01);

    if (warp >= 16) {
      reg_dealloc<kCtrlRegs>();
      if (warp == kTmaWarp) {
        if (lane == 0 && n_max > 0) {
            mbar_arrive_expect_tx(bar_qdo_full(), 4u * kBigTile);
            for (int t = 0; t < 2; ++t) {
                const int q0 = m_block * 2 * kTile + t * kTile;
                tma_load_4d(q_smem + t * kBigTile, &tmap_q, bar_qdo_full(), 0, q0, h, b);
                tma_load_4d(do_smem + t * kBigTile, &tmap_do, bar_qdo_full(), 0, q0, h, b);
            }
            bool ok = true;
            for (int j = 0; j < n_max && ok; ++j) {
#pragma unroll
                for (int which = 0; which < 2; ++which) {          // 0: K_j, 1: V_j
                    const int item = 2 * j + which;
                    ok = ok && mbar_wait(bar_ring_empty(slot_of(item)), phase_of(item) ^ 1u, wc, 0x40 + which);
                    if (!ok) break;
                    mbar_arrive_expect_tx(bar_ring_full(slot_of(item)), (uint32_t)kSmallTile);
                    tma_load_4d(ring_smem + slot_of(item) * kSmallTile, which == 0 ? &tmap_k : &tmap_v,
                                bar_ring_full(slot_of(item)), 0, j * kStep, h, b);
                }
            }
        }
      } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
        const int t = warp - kMmaWarp0;            // this thread issues the contractions of tile t
        if (lane == 0 && n_max > 0) {
            const int n_t = n_steps[t];
            constexpr uint32_t idesc_s = make_idesc_bf16(kTile, kStep, 0, 0);
            constexpr uint32_t idesc_dq = make_idesc_bf16(kTile, kD, 0, 1);
            const uint64_t q_desc = make_smem_desc_sw128(q_smem + t * kBigTile, 16, 1024);
            const uint64_t do_desc = make_smem_desc_sw128(do_smem + t * kBigTile, 16, 1024);
            const uint64_t ring_desc = make_smem_desc_sw128(ring_smem, 16, 1024);
            const uint64_t ring_desc_mn = make_smem_desc_sw128(ring_smem, 8192, 1024);
            const uint32_t tb = tmem_base + t * 192;
            const uint32_t ds_hi = tmem_base + 384 + t * 32, ds_lo = tmem_base + 448 + t * 32;
            // S_t = Q_t K_j^T and dP_t = dO_t V_j^T
            auto issue_sdp = [&](int slot_k, int slot_v) {
                const uint64_t kd = ring_desc + (uint64_t)((slot_k * kSmallTile) >> 4);
                const uint64_t vd = ring_desc + (uint64_t)((slot_v * kSmallTile) >> 4);
#pragma unroll
                for (int k = 0; k < kD / 16; ++k) mma_ss(tb, q_desc + 2 * k, kd + 2 * k, idesc_s, k > 0);
#pragma unroll
                for (int k = 0; k < kD / 16; ++k) mma_ss(tb + 64, do_desc + 2 * k, vd + 2 * k, idesc_s, k > 0);
            };
            // dQ_t += dS_t K_j   (dS from tensor memory, K_j rows as the contraction index)
            auto issue_dq = [&](int slot_k, bool acc) {
                const uint64_t kd = ring_desc_mn + (uint64_t)((slot_k * kSmallTile) >> 4);
#pragma unroll
                for (int k = 0; k < kStep / 16; ++k)
                    mma_ts(tb + 128, ds_hi + k * 8, kd + 128 * k, idesc_dq, (acc || k > 0) ? 1u : 0u);
                if constexpr (kSplit) {
#pragma unroll
                    for (int k = 0; k < kStep / 16; ++k)
                        mma_ts(tb + 128, ds_lo + k * 8, kd + 128 * k, idesc_dq, 1u);
                }
            };
            bool ok = mbar_wait(bar_qdo_full(), 0, wc, 0x50);
            ok = ok && mbar_wait(bar_ring_full(slot_of(0)), phase_of(0), wc, 0x51);
            ok = ok && mbar_wait(bar_ring_full(slot_of(1)), phase_of(1), wc, 0x52);
            if (ok) {
                tc_fence_after_sync();
                if (n_t > 0) { issue_sdp(slot_of(0), slot_of(1)); mma_commit(bar_sdp_full(t)); }
                mma_commit(bar_ring_empty(slot_of(1)));            // V_0 is consumed
            }
            for (int j = 0; j < n_max && ok; ++j) {
                const int item_k = 2 * j, item_k1 = 2 * j + 2, item_v1 = 2 * j + 3;
                if (j + 1 < n_max) {
                    ok = mbar_wait(bar_ring_full(slot_of(item_k1)), phase_of(item_k1), wc, 0x53);
                    ok = ok && mbar_wait(bar_ring_full(slot_of(item_v1)), phase_of(item_v1), wc, 0x54);
                    if (ok && j + 1 < n_t) {
                        // S and dP of step j are in registers: compute step j + 1 now
                        ok = mbar_wait(bar_sdp_free(t), (uint32_t)(j & 1), wc, 0x5a + t);
                        if (!ok) break;
                        tc_fence_after_sync();
                        LTCA_TRACE_EVT(0x20 + (j << 8));
                        issue_sdp(slot_of(item_k1), slot_of(item_v1));
                        mma_commit(bar_sdp_full(t));
                        LTCA_TRACE_EVT(0x21 + (j << 8));
                    }
                    if (!ok) break;
                    mma_commit(bar_ring_empty(slot_of(item_v1)));
                }
                if (j < n_t) {
                    ok = mbar_wait(bar_ds_full(t), (uint32_t)(j & 1), wc, 0x55 + t);
                    if (!ok) break;
                    tc_fence_after_sync();
                    LTCA_TRACE_EVT(0x22 + (j << 8));
                    issue_dq(slot_of(item_k), j > 0);
                    mma_commit(bar_dq_done(t));
                    LTCA_TRACE_EVT(0x23 + (j << 8));
                }
                mma_commit(bar_ring_empty(slot_of(item_k)));
            }
            if (ok && n_t > 0) ok = mbar_wait(bar_dq_done(t), (uint32_t)((n_t - 1) & 1), wc, 0x58 + t);
        }
      }
    } else {
        reg_alloc<kMathRegs>();
        const int t = (warp >> 2) & 1, half = warp >> 3, wq = warp & 3;
        const int row = wq * 32 + lane;
        const int q0 = m_block * 2 * kTile + t * kTile;
        const int qi = q0 + row;
        const int n_t = n_steps[t];
        const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
        const uint32_t tS = tmem_base + lane_base + t * 192 + half * 32;
        const uint32_t tDP = tS + 64;
        const uint32_t tDQ = tmem_base + lane_base + t * 192 + 128 + half * 32;
        const uint32_t tDS = tmem_base + lane_base + 384 + t * 32 + half * 16;
        const uint32_t tDSlo = tDS + 64;
        const float c2 = a.scale_log2;
        const bool general = (a.keep_mask != nullptr) || (a.use_clamp != 0);
        const int64_t srow = ((int64_t)b * a.H + h) * a.Sq_pad + qi;      // qi < Sq_pad by construction
        const float lse2 = a.lse2[srow];
        const float dlt = a.delta[srow];

        bool ok = true;
        for (int j = 0; j < n_t; ++j) {
            ok = mbar_wait_warp(bar_sdp_full(t), (uint32_t)(j & 1), wc, 0x60 + t);
            if (!ok) break;
            tc_fence_after_sync();
            LTCA_TRACE_EVT(0x10 + (j << 8));
            uint32_t s[32], dp[32];
            tmem_ld32(tS, s);
            tmem_ld32(tDP, dp);
            tmem_wait_ld();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sdp_free(t));
            LTCA_TRACE_EVT(0x11 + (j << 8));
            // One-time delay of tile 1: from then on one tile's exponentials overlap the other
            // tile's loads, stores and barrier traffic instead of all warps stalling together.
            if (t == 1 && j == 0 && n_steps[0] > 0) {
                ok = mbar_wait_warp(bar_stagger(), 0, wc, 0x66);
                if (!ok) break;
            }
            const int k0 = j * kStep;
            const bool edge = (k0 + kStep > kvlen) || (a.causal && (k0 + kStep - 1 > q0 + a.causal_off));
            // dS = P o (dP - delta), left in dp[]; the masked variant only runs on edge steps
            if (general) {
                int lim = kvlen;
                if (a.causal) lim = min(lim, qi + a.causal_off + 1);
                lim -= k0 + half * 32;
                const float* mrow = nullptr;
                if (a.keep_mask && qi < a.Sq)
                    mrow = a.keep_mask + ((int64_t)b * a.Sq + qi) * a.Sk + k0 + half * 32;
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const float sv = __uint_as_float(s[c]);
                    const float p = fast_exp2(fmaf(sv, c2, -lse2));
                    float d = p * (__uint_as_float(dp[c]) - dlt);
                    bool vis = c < lim;
                    if (mrow && vis) vis = (__ldg(mrow + c) != 0.0f);
                    if (a.use_clamp && sv >= a.clamp_raw) d = 0.f;
                    dp[c] = __float_as_uint(vis ? d : 0.f);
                }
            } else if (edge) {
                // causal diagonal or end of the keys, no dense mask: selects only, no branches
                int lim = kvlen;
                if (a.causal) lim = min(lim, qi + a.causal_off + 1);
                lim -= k0 + half * 32;
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const float p = fast_exp2(fmaf(__uint_as_float(s[c]), c2, -lse2));
                    dp[c] = __float_as_uint((c < lim) ? p * (__uint_as_float(dp[c]) - dlt) : 0.f);
                }
            } else {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const float p = fast_exp2(fmaf(__uint_as_float(s[c]), c2, -lse2));
                    dp[c] = __float_as_uint(p * (__uint_as_float(dp[c]) - dlt));
                }
            }
            uint32_t hi[16], lo[16];
            pack32<kSplit>(dp, hi, lo);
            if (t == 0 && j == 0) {
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_stagger());
            }
            LTCA_TRACE_EVT(0x12 + (j << 8));
            if (j > 0) {
                // the previous dS must have been consumed before it is overwritten
                ok = mbar_wait_warp(bar_dq_done(t), (uint32_t)((j - 1) & 1), wc, 0x64 + t);
                if (!ok) break;
            }
            tmem_st16(tDS, hi);
            if constexpr (kSplit) tmem_st16(tDSlo, lo);
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_ds_full(t));
            LTCA_TRACE_EVT(0x13 + (j << 8));
        }
        if (ok && q0 < a.Sq) {
            if (n_t > 0) {
                ok = mbar_wait_warp(bar_dq_done(t), (uint32_t)((n_t - 1) & 1), wc, 0x62 + t);
                tc_fence_after_sync();
            }
            OutT* drow = reinterpret_cast<OutT*>(a.dq) + b * a.dqs.batch + h * a.dqs.head +
                         (int64_t)qi * a.dqs.seq + half * 32;
            uint32_t o[32];
            if (n_t > 0 && ok) { tmem_ld32(tDQ, o); tmem_wait_ld(); }
            else {
#pragma unroll
                for (int c = 0; c < 32; ++c) o[c] = 0u;
            }
            if (qi < a.Sq) store_row32<OutT>(drow, o, a.scale);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp0) {
        __syncwarp();
        if (misc[1]) __nanosleep(200000);
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------
// 3. dK, dV (transposed problem: one KEY per tensor-memory lane)
// tensor memory per tile t (base t*256): S^T [0,64) dP^T [64,128) dV [128,192) dK [192,256).
// A key row belongs to two threads (warps w and w + 8); thread `half` owns query columns
// [32*half, 32*half + 32) of S^T and dP^T and writes its P^T / dS^T back INSIDE those columns
// (bf16 pairs in the first 16, the kSplit low-order term in the next 16), so neither thread
// ever overwrites scores the other has not read yet.
// ---------------------------------------------------------------------------------------------
template <typename OutT, bool kSplit>
__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_dkv_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q,
                          const __grid_constant__ CUtensorMap tmap_do,
                          const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_v, const BwdArgs a) {
    using L = DkvSmem;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t k_smem = smem_base + L::kKOff, v_smem = smem_base + L::kVOff;
    const uint32_t ring_smem = smem_base + L::kRingOff, bar_base = smem_base + L::kBarOff;
    auto bar_kv_full = [&]() { return bar_base; };
    auto bar_ring_full = [&](int s) { return bar_base + 8u * (1 + s); };
    auto bar_ring_empty = [&](int s) { return bar_base + 8u * (1 + L::kStages + s); };
    auto bar_sdp_full = [&](int t) { return bar_base + 8u * (1 + 2 * L::kStages + t); };
    auto bar_pds_full = [&](int t) { return bar_base + 8u * (3 + 2 * L::kStages + t); };
    auto bar_acc_done = [&](int t) { return bar_base + 8u * (5 + 2 * L::kStages + t); };
    auto bar_stagger = [&]() { return bar_base + 8u * (7 + 2 * L::kStages); };
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_block = blockIdx.x;                 // early key blocks carry the most causal work
    const int h = blockIdx.y, b = blockIdx.z;

    int kvlen = a.Sk;
    if (a.kv_len) {
        grid_dependency_wait();                // the lengths may come from the kernel before this one
        kvlen = min(max(a.kv_len[b], 0), a.Sk);
    }
    const int n_q = (a.Sq + kStep - 1) / kStep;     // query steps in total
    int j_begin[2];                                 // first query step that can see the tile's keys
    bool active[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int k0 = n_block * 2 * kTile + t * kTile;
        active[t] = (k0 < kvlen);
        int jb = 0;
        if (a.causal) jb = max(0, k0 - a.causal_off) / kStep;
        j_begin[t] = jb;
        if (jb >= n_q) active[t] = false;
    }
    const bool any_active = active[0] || active[1];
    const int j_first = min(active[0] ? j_begin[0] : n_q, active[1] ? j_begin[1] : n_q);

    if (threadIdx.x == 0) {
        mbar_init(bar_kv_full(), 1);
        for (int s = 0; s < L::kStages; ++s) { mbar_init(bar_ring_full(s), 1); mbar_init(bar_ring_empty(s), 2); }
        for (int t = 0; t < 2; ++t) {
            mbar_init(bar_sdp_full(t), 1);
            mbar_init(bar_pds_full(t), 8);         // one arrival per elementwise warp of the tile
            mbar_init(bar_acc_done(t), 1);
        }
        mbar_init(bar_stagger(), 8);
        misc[1] = 0u;
        mbar_fence_init();
    }
    if (warp == kMmaWarp0) { tmem_alloc(smem_u32(const_cast<uint32_t*>(&misc[0])), kTmemCols); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = misc[0];
    const WaitCtx wc{&misc[1], a.status};
    grid_launch_dependents();                  // (set up: the next kernel may place its CTAs)
    grid_dependency_wait();                    // the operands are complete once the kernel before this one has ended
    // ring items are numbered from the first streamed step of this CTA
    auto slot_of = [&](int j) { return (j - j_first) % L::kStages; };
    auto phase_of = [&](int j) { return (uint32_t)(((j - j_first) / L::kStages) & 1); };
    LTCA_TRACE_DECL(LTCA_TRACE_KERNEL == 2 && blockIdx.x == 0 && blockIdx.y == 5 && blockIdx.z == 0);
    LTCA_TRACE_EVT(0x01);

    if (warp >= 16) {
      reg_dealloc<kCtrlRegs>();
      if (warp == kTmaWarp) {
        if (lane == 0 && any_active) {
            mbar_arrive_expect_tx(bar_kv_full(), 4u * kBigTile);
            for (int t = 0; t < 2; ++t) {
                const int k0 = n_block * 2 * kTile + t * kTile;
                tma_load_4d(k_smem + t * kBigTile, &tmap_k, bar_kv_full(), 0, k0, h, b);
                tma_load_4d(v_smem + t * kBigTile, &tmap_v, bar_kv_full(), 0, k0, h, b);
            }
            const float* lse2_row = a.lse2 + ((int64_t)b * a.H + h) * a.Sq_pad;
            const float* dlt_row = a.delta + ((int64_t)b * a.H + h) * a.Sq_pad;
            bool ok = true;
            for (int j = j_first; j < n_q && ok; ++j) {
                ok = mbar_wait(bar_ring_empty(slot_of(j)), phase_of(j) ^ 1u, wc, 0x70);
                if (!ok) break;
                const uint32_t st = ring_smem + slot_of(j) * L::kStageBytes;
                mbar_arrive_expect_tx(bar_ring_full(slot_of(j)), 2u * kSmallTile + 512u);
                tma_load_4d(st, &tmap_q, bar_ring_full(slot_of(j)), 0, j * kStep, h, b);
                tma_load_4d(st + kSmallTile, &tmap_do, bar_ring_full(slot_of(j)), 0, j * kStep, h, b);
                asm volatile(
                    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 256, [%2];"
                    ::"r"(st + 2 * kSmallTile), "l"(reinterpret_cast<uint64_t>(lse2_row + j * kStep)),
                      "r"(bar_ring_full(slot_of(j))) : "memory");
                asm volatile(
                    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 256, [%2];"
                    ::"r"(st + 2 * kSmallTile + 256), "l"(reinterpret_cast<uint64_t>(dlt_row + j * kStep)),
                      "r"(bar_ring_full(slot_of(j))) : "memory");
            }
        }
      } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
        const int t = warp - kMmaWarp0;            // this thread issues the contractions of tile t
        if (lane == 0 && any_active) {
            constexpr uint32_t idesc_s = make_idesc_bf16(kTile, kStep, 0, 0);
            constexpr uint32_t idesc_acc = make_idesc_bf16(kTile, kD, 0, 1);
            const uint64_t k_desc = make_smem_desc_sw128(k_smem + t * kBigTile, 16, 1024);
            const uint64_t v_desc = make_smem_desc_sw128(v_smem + t * kBigTile, 16, 1024);
            const uint64_t ring_desc = make_smem_desc_sw128(ring_smem, 16, 1024);
            const uint64_t ring_desc_mn = make_smem_desc_sw128(ring_smem, 8192, 1024);
            const uint32_t tb = tmem_base + t * 256;
            const bool act = active[t];
            const int jb = j_begin[t];
            // S^T_t = K_t Q_j^T and dP^T_t = V_t dO_j^T
            auto issue_sdp = [&](int slot) {
                const uint64_t qd = ring_desc + (uint64_t)((slot * L::kStageBytes) >> 4);
                const uint64_t gd = qd + (uint64_t)(kSmallTile >> 4);
#pragma unroll
                for (int k = 0; k < kD / 16; ++k) mma_ss(tb, k_desc + 2 * k, qd + 2 * k, idesc_s, k > 0);
#pragma unroll
                for (int k = 0; k < kD / 16; ++k) mma_ss(tb + 64, v_desc + 2 * k, gd + 2 * k, idesc_s, k > 0);
            };
            // dV_t += P^T_t dO_j and dK_t += dS^T_t Q_j   (query rows are the contraction index);
            // queries [0,32) sit in columns [0,16) of their region, queries [32,64) in [32,48)
            auto issue_acc = [&](int slot, bool acc) {
                const uint64_t qd = ring_desc_mn + (uint64_t)((slot * L::kStageBytes) >> 4);
                const uint64_t gd = qd + (uint64_t)(kSmallTile >> 4);
#pragma unroll
                for (int k = 0; k < kStep / 16; ++k)
                    mma_ts(tb + 128, tb + (k / 2) * 32 + (k % 2) * 8, gd + 128 * k, idesc_acc,
                           (acc || k > 0) ? 1u : 0u);
#pragma unroll
                for (int k = 0; k < kStep / 16; ++k)
                    mma_ts(tb + 192, tb + 64 + (k / 2) * 32 + (k % 2) * 8, qd + 128 * k, idesc_acc,
                           (acc || k > 0) ? 1u : 0u);
                if constexpr (kSplit) {
#pragma unroll
                    for (int k = 0; k < kStep / 16; ++k)
                        mma_ts(tb + 128, tb + 16 + (k / 2) * 32 + (k % 2) * 8, gd + 128 * k, idesc_acc, 1u);
#pragma unroll
                    for (int k = 0; k < kStep / 16; ++k)
                        mma_ts(tb + 192, tb + 80 + (k / 2) * 32 + (k % 2) * 8, qd + 128 * k, idesc_acc, 1u);
                }
            };
            bool ok = mbar_wait(bar_kv_full(), 0, wc, 0x80);
            if (ok && j_first < n_q) {
                ok = mbar_wait(bar_ring_full(slot_of(j_first)), phase_of(j_first), wc, 0x81);
                if (ok && act && jb == j_first) {
                    tc_fence_after_sync();
                    issue_sdp(slot_of(j_first));
                    mma_commit(bar_sdp_full(t));
                }
            }
            for (int j = j_first; j < n_q && ok; ++j) {
                const bool have_next = (j + 1 < n_q);
                if (have_next) ok = mbar_wait(bar_ring_full(slot_of(j + 1)), phase_of(j + 1), wc, 0x82);
                if (!ok) break;
                if (act) {
                    if (j >= jb) {
                        ok = mbar_wait(bar_pds_full(t), (uint32_t)((j - jb) & 1), wc, 0x83 + t);
                        if (!ok) break;
                        tc_fence_after_sync();
                        LTCA_TRACE_EVT(0x22 + (j << 8));
                        issue_acc(slot_of(j), j > jb);
                        mma_commit(bar_acc_done(t));
                        LTCA_TRACE_EVT(0x23 + (j << 8));
                    }
                    if (have_next && j + 1 >= jb) {
                        issue_sdp(slot_of(j + 1));
                        mma_commit(bar_sdp_full(t));
                        LTCA_TRACE_EVT(0x21 + (j << 8));
                    }
                }
                mma_commit(bar_ring_empty(slot_of(j)));
            }
            if (ok && act) ok = mbar_wait(bar_acc_done(t), (uint32_t)((n_q - 1 - jb) & 1), wc, 0x88 + t);
        }
      }
    } else {
        reg_alloc<kMathRegs>();
        const int t = (warp >> 2) & 1, half = warp >> 3, wq = warp & 3;
        const int row = wq * 32 + lane;
        const int k0 = n_block * 2 * kTile + t * kTile;
        const int kj = k0 + row;                                   // this thread's key
        const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
        const uint32_t tS = tmem_base + lane_base + t * 256 + half * 32;
        const uint32_t tDP = tS + 64;
        const uint32_t tDV = tmem_base + lane_base + t * 256 + 128 + half * 32;
        const uint32_t tDK = tDV + 64;
        const float c2 = a.scale_log2;
        const bool general = (a.keep_mask != nullptr) || (a.use_clamp != 0);
        const bool key_live = kj < kvlen;

        bool ok = true;
        if (active[t]) {
            for (int j = j_begin[t]; j < n_q; ++j) {
                const int it = j - j_begin[t];
                ok = mbar_wait_warp(bar_sdp_full(t), (uint32_t)(it & 1), wc, 0x90 + t);
                if (!ok) break;
                tc_fence_after_sync();
                LTCA_TRACE_EVT(0x10 + (j << 8));
                uint32_t s[32], dp[32];
                tmem_ld32(tS, s);
                tmem_ld32(tDP, dp);
                tmem_wait_ld();
                LTCA_TRACE_EVT(0x11 + (j << 8));
                if (t == 1 && it == 0 && active[0] && j_begin[0] <= j_begin[1]) {
                    ok = mbar_wait_warp(bar_stagger(), 0, wc, 0x96);
                    if (!ok) break;
                }
                // lse2 and delta of this thread's 32 query columns (broadcast reads: every lane
                // of the warp reads the same address)
                const float4* st4 = reinterpret_cast<const float4*>(
                    smem_gen + L::kRingOff + slot_of(j) * L::kStageBytes + 2 * kSmallTile) + half * 8;
                const int q0 = j * kStep + half * 32;
                // a query column c is hidden from this key when q0 + c + off < kj
                const bool edge = !key_live || (k0 + kTile > kvlen) ||
                                  (a.causal && (j * kStep + a.causal_off < k0 + kTile - 1));
                // P^T into s[], dS^T = P^T o (dP^T - delta) into dp[]
                if (general) {
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const float4 l4 = st4[c4];
                        const float4 d4 = st4[16 + c4];
                        const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
                        const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = 4 * c4 + e;
                            const float sv = __uint_as_float(s[c]);
                            float p = fast_exp2(fmaf(sv, c2, -ls[e]));
                            float d = p * (__uint_as_float(dp[c]) - dl[e]);
                            bool vis = key_live && (!a.causal || (kj <= q0 + c + a.causal_off));
                            if (vis && a.keep_mask && (q0 + c) < a.Sq)
                                vis = a.keep_mask[((int64_t)b * a.Sq + q0 + c) * a.Sk + kj] != 0.0f;
                            if (a.use_clamp && sv >= a.clamp_raw) {
                                p = fast_exp2(a.clamp_log2 - ls[e]);
                                d = 0.f;
                            }
                            s[c] = __float_as_uint(vis ? p : 0.f);
                            dp[c] = __float_as_uint(vis ? d : 0.f);
                        }
                    }
                } else if (edge) {
                    // causal diagonal or end of the keys, no dense mask: selects only, no branches.
                    // Query column c is visible to this key when c >= cmin.
                    const int cmin = !key_live ? 0x7fffffff : (a.causal ? kj - a.causal_off - q0 : -0x7fffffff);
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const float4 l4 = st4[c4];
                        const float4 d4 = st4[16 + c4];
                        const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
                        const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = 4 * c4 + e;
                            const float p = fast_exp2(fmaf(__uint_as_float(s[c]), c2, -ls[e]));
                            const bool vis = c >= cmin;
                            s[c] = __float_as_uint(vis ? p : 0.f);
                            dp[c] = __float_as_uint(vis ? p * (__uint_as_float(dp[c]) - dl[e]) : 0.f);
                        }
                    }
                } else {
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const float4 l4 = st4[c4];
                        const float4 d4 = st4[16 + c4];
                        const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
                        const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = 4 * c4 + e;
                            const float p = fast_exp2(fmaf(__uint_as_float(s[c]), c2, -ls[e]));
                            s[c] = __float_as_uint(p);
                            dp[c] = __float_as_uint(p * (__uint_as_float(dp[c]) - dl[e]));
                        }
                    }
                }
                uint32_t pt[16], ptl[16], dst[16], dstl[16];
                pack32<kSplit>(s, pt, ptl);
                pack32<kSplit>(dp, dst, dstl);
                if (t == 0 && it == 0) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_stagger());
                }
                LTCA_TRACE_EVT(0x12 + (j << 8));
                tmem_st16(tS, pt);
                tmem_st16(tDP, dst);
                if constexpr (kSplit) {
                    tmem_st16(tS + 16, ptl);
                    tmem_st16(tDP + 16, dstl);
                }
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_pds_full(t));
                LTCA_TRACE_EVT(0x13 + (j << 8));
            }
        }
        // epilogue: dV and scale * dK (zeros for tiles that no query can see)
        if (ok && k0 < a.Sk) {
            if (active[t]) {
                ok = mbar_wait_warp(bar_acc_done(t), (uint32_t)((n_q - 1 - j_begin[t]) & 1), wc, 0x92 + t);
                tc_fence_after_sync();
            }
            OutT* dkrow = reinterpret_cast<OutT*>(a.dk) + b * a.dks.batch + h * a.dks.head +
                          (int64_t)kj * a.dks.seq + half * 32;
            OutT* dvrow = reinterpret_cast<OutT*>(a.dv) + b * a.dvs.batch + h * a.dvs.head +
                          (int64_t)kj * a.dvs.seq + half * 32;
            uint32_t o[32];
            if (active[t] && ok) { tmem_ld32(tDV, o); tmem_wait_ld(); }
            else {
#pragma unroll
                for (int c = 0; c < 32; ++c) o[c] = 0u;
            }
            if (kj < a.Sk) store_row32<OutT>(dvrow, o, 1.0f);
            if (active[t] && ok) { tmem_ld32(tDK, o); tmem_wait_ld(); }
            if (kj < a.Sk) store_row32<OutT>(dkrow, o, a.scale);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp0) {
        __syncwarp();
        if (misc[1]) __nanosleep(200000);
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------
// 4. dK, dV, single-tile persistent variant (bf16 operands and results).
// Work item = 128 keys of one (batch, head); query steps of 128.  Nothing in tensor memory is
// aliased, so the next step's S^T and dP^T are computed while this step's P^T and dS^T are being
// formed, and the contractions have N = 128 or K = 128:
//   S^T [0,128)  dP^T [128,256)  P^T bf16 [256,320)  dS^T bf16 [320,384)  dV [384,448)  dK [448,512)
// One CTA per SM takes items from the global counter (see ItemQueue); K and V are double-buffered
// so the next item's tiles and first query steps load while the current item drains, and the MMA
// threads issue the next item's first S^T / dP^T before the current item's last accumulation.
// 16 elementwise warps: warp w owns key rows 32 (w % 4) .. +31 and query columns 32 (w / 4) .. +31
// of the step.  Two MMA threads share the issue work: warp 16 issues S^T and dV, warp 17 dP^T
// and dK (each accumulator has one issuing thread, so the summation order is fixed).
// ---------------------------------------------------------------------------------------------
struct Dkv4Smem {
    static constexpr int kStages = 4;                         // ring of (Q_j, dO_j, lse2_j, delta_j)
    static constexpr int kStageBytes = 2 * kBigTile + 1024;
    static constexpr int kResOff = 0;                         // two (K, V) buffers
    static constexpr int kRingOff = 4 * kBigTile;
    static constexpr int kBarOff = kRingOff + kStages * kStageBytes;
    // bars: res_full[2], res_empty[2], ring_full[S], ring_empty[S], sdp_full, sdp_free, pds_full, acc_done,
    // acc_free, item_full[kItemSlots], item_empty[kItemSlots], staged[2]
    static constexpr int kNumBars = 4 + 2 * kStages + 5 + 2 * kItemSlots + 2;
    static constexpr int kMiscOff = kBarOff + kNumBars * 8;   // tmem base, abort flag, item slots
    static constexpr int kDynBytes = kMiscOff + 16 + 4 * kItemSlots + 1024;
};

__device__ __forceinline__ void store_row16_bf16(__nv_bfloat16* dst, const uint32_t (&o)[16], float mul) {
    uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int v = 0; v < 2; ++v) {
        uint4 w;
        w.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]) * mul, __uint_as_float(o[8 * v + 1]) * mul);
        w.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]) * mul, __uint_as_float(o[8 * v + 3]) * mul);
        w.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]) * mul, __uint_as_float(o[8 * v + 5]) * mul);
        w.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]) * mul, __uint_as_float(o[8 * v + 7]) * mul);
        d[v] = w;
    }
}

__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_dkv4_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q,
                           const __grid_constant__ CUtensorMap tmap_do,
                           const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v,
                           const __grid_constant__ CUtensorMap tmap_dk,
                           const __grid_constant__ CUtensorMap tmap_dv, const BwdArgs a, const ItemGrid grid) {
    using L = Dkv4Smem;
    constexpr int kQStep = 128;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t res_smem = smem_base + L::kResOff;
    const uint32_t ring_smem = smem_base + L::kRingOff, bar_base = smem_base + L::kBarOff;
    auto bar_res_full = [&](int r) { return bar_base + 8u * r; };
    auto bar_res_empty = [&](int r) { return bar_base + 8u * (2 + r); };
    auto bar_ring_full = [&](int s) { return bar_base + 8u * (4 + s); };
    auto bar_ring_empty = [&](int s) { return bar_base + 8u * (4 + L::kStages + s); };
    const uint32_t bar_sdp_full = bar_base + 8u * (4 + 2 * L::kStages);
    const uint32_t bar_sdp_free = bar_sdp_full + 8u;
    const uint32_t bar_pds_full = bar_sdp_full + 16u;
    const uint32_t bar_acc_done = bar_sdp_full + 24u;
    const uint32_t bar_acc_free = bar_sdp_full + 32u;
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);
    const ItemQueue iq{bar_sdp_full + 40u, bar_sdp_full + 40u + 8u * kItemSlots,
                       reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 16)};
    // dK and dV of an item staged in the item's own K / V buffer (one barrier per buffer)
    auto bar_staged = [&](int r) { return bar_sdp_full + 40u + 16u * kItemSlots + 8u * r; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_q = (a.Sq + kQStep - 1) / kQStep;   // query steps in total
    LTCA_TRACE_DECL(LTCA_TRACE_KERNEL == 4 && blockIdx.x == 5);
    LTCA_TRACE_EVT(0x01);

    if (threadIdx.x == 0) {
        // a K / V buffer is free again when both MMA threads are done with it and the item's dK / dV,
        // which are staged in it, have been read by their TMA stores
        for (int r = 0; r < 2; ++r) {
            mbar_init(bar_res_full(r), 1);
            mbar_init(bar_res_empty(r), 3);
            mbar_init(bar_staged(r), 16);
        }
        for (int s = 0; s < L::kStages; ++s) { mbar_init(bar_ring_full(s), 1); mbar_init(bar_ring_empty(s), 2); }
        mbar_init(bar_sdp_full, 2);                // one commit per MMA thread
        mbar_init(bar_sdp_free, 16);               // one arrival per elementwise warp
        mbar_init(bar_pds_full, 16);
        mbar_init(bar_acc_done, 2);
        mbar_init(bar_acc_free, 16);
        for (int i = 0; i < kItemSlots; ++i) { mbar_init(iq.full(i), 1); mbar_init(iq.empty(i), 19); }
        misc[1] = 0u;
        mbar_fence_init();
    }
    if (warp == kMmaWarp0) { tmem_alloc(smem_u32(const_cast<uint32_t*>(&misc[0])), kTmemCols); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = misc[0];
    const WaitCtx wc{&misc[1], a.status};
    grid_dependency_wait();                    // the operands are complete once the kernel before this one has ended
    auto slot_of = [&](int g) { return g % L::kStages; };
    auto phase_of = [&](int g) { return (uint32_t)((g / L::kStages) & 1); };
    // the item's key tile, first query step that can see it and number of query steps (0: none)
    auto item_steps = [&](int linear, int& k0, int& h, int& b, int& kvlen, int& j_begin) {
        int rank;
        sched_item(grid, linear, rank, h, b);
        k0 = rank * kTile;                          // early key blocks carry the most causal work
        kvlen = a.Sk;
        if (a.kv_len) kvlen = min(max(a.kv_len[b], 0), a.Sk);
        j_begin = 0;
        if (a.causal) j_begin = max(0, k0 - a.causal_off) / kQStep;
        const bool active = (k0 < kvlen) && (j_begin < n_q);
        return active ? n_q - j_begin : 0;
    };

    if (warp >= 16) {
      reg_dealloc<kCtrlRegs>();
      if (warp == kTmaWarp) {
        if (lane == 0) {
            int g = 0, na = 0;
            bool ok = true;
            for (int nq = 0; ok; ++nq) {
                const int linear = iq.produce(nq, grid.counters, grid.n_items, wc);
                if (linear < 0) break;
                int k0, h, b, kvlen, j_begin;
                const int n_it = item_steps(linear, k0, h, b, kvlen, j_begin);
                if (n_it == 0) continue;
                const int r = na & 1;
                ok = mbar_wait(bar_res_empty(r), (uint32_t)(((na >> 1) & 1) ^ 1), wc, 0xa1);
                if (!ok) break;
                mbar_arrive_expect_tx(bar_res_full(r), 2u * kBigTile);
                tma_load_4d(res_smem + r * 2 * kBigTile, &tmap_k, bar_res_full(r), 0, k0, h, b);
                tma_load_4d(res_smem + r * 2 * kBigTile + kBigTile, &tmap_v, bar_res_full(r), 0, k0, h, b);
                const float* lse2_row = a.lse2 + ((int64_t)b * a.H + h) * a.Sq_pad;
                const float* dlt_row = a.delta + ((int64_t)b * a.H + h) * a.Sq_pad;
                for (int it = 0; it < n_it && ok; ++it, ++g) {
                    const int j = j_begin + it;
                    ok = mbar_wait(bar_ring_empty(slot_of(g)), phase_of(g) ^ 1u, wc, 0xa0);
                    if (!ok) break;
                    const uint32_t st = ring_smem + slot_of(g) * L::kStageBytes;
                    const uint32_t bar = bar_ring_full(slot_of(g));
                    mbar_arrive_expect_tx(bar, 2u * kBigTile + 1024u);
                    tma_load_4d(st, &tmap_q, bar, 0, j * kQStep, h, b);
                    tma_load_4d(st + kBigTile, &tmap_do, bar, 0, j * kQStep, h, b);
                    asm volatile(
                        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 512, [%2];"
                        ::"r"(st + 2 * kBigTile), "l"(reinterpret_cast<uint64_t>(lse2_row + j * kQStep)), "r"(bar)
                        : "memory");
                    asm volatile(
                        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 512, [%2];"
                        ::"r"(st + 2 * kBigTile + 512), "l"(reinterpret_cast<uint64_t>(dlt_row + j * kQStep)),
                          "r"(bar)
                        : "memory");
                }
                ++na;
            }
        }
      } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
        // which == 0: S^T = K Q_j^T and dV += P^T dO_j;  which == 1: dP^T = V dO_j^T and dK += dS^T Q_j
        const int which = warp - kMmaWarp0;
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc_bf16(kTile, kQStep, 0, 0);
            constexpr uint32_t idesc_acc = make_idesc_bf16(kTile, kD, 0, 1);
            const uint64_t res_desc = make_smem_desc_sw128(res_smem + (which == 0 ? 0 : kBigTile), 16, 1024);
            // the streamed operand of the first contraction (Q for S^T, dO for dP^T), K-major
            const uint64_t b1_desc = make_smem_desc_sw128(ring_smem + (which == 0 ? 0 : kBigTile), 16, 1024);
            // the streamed operand of the accumulation (dO for dV, Q for dK), rows as the contraction index
            const uint64_t b2_desc = make_smem_desc_sw128(ring_smem + (which == 0 ? kBigTile : 0), 8192, 1024);
            const uint32_t d1 = tmem_base + (which == 0 ? 0 : 128);
            const uint32_t a2 = tmem_base + (which == 0 ? 256 : 320);
            const uint32_t d2 = tmem_base + (which == 0 ? 384 : 448);
            // the accumulation that is still to be issued (one step behind the first contraction)
            bool pending = false;
            int p_g = 0, p_na = 0;
            bool p_acc = false, p_first = false;
            bool ok = true;
            auto do_acc = [&]() {
                ok = mbar_wait(bar_pds_full, (uint32_t)(p_g & 1), wc, 0xb4);
                // the previous item's dV / dK must have left tensor memory before they are overwritten
                if (ok && p_first && p_na > 0) ok = mbar_wait(bar_acc_free, (uint32_t)((p_na - 1) & 1), wc, 0xb6);
                if (!ok) return;
                tc_fence_after_sync();
                const uint64_t bd = b2_desc + (uint64_t)((slot_of(p_g) * L::kStageBytes) >> 4);
#pragma unroll
                for (int k = 0; k < kQStep / 16; ++k)
                    mma_ts(d2, a2 + k * 8, bd + 128 * k, idesc_acc, (p_acc || k > 0) ? 1u : 0u);
                mma_commit(bar_acc_done);
                mma_commit(bar_ring_empty(slot_of(p_g)));
                LTCA_TRACE_EVT(0x22 + (p_g << 8));
                pending = false;
            };
            int g = 0, na = 0;
            for (int nq = 0; ok; ++nq) {
                const int linear = iq.consume(nq, wc);
                if (linear < 0) break;
                int k0, h, b, kvlen, j_begin;
                const int n_it = item_steps(linear, k0, h, b, kvlen, j_begin);
                if (n_it == 0) {
                    // An item without work does not carry the deferred accumulation along: the elementwise warps
                    // wait for it at the end of the item before, so they take no further queue entry, and after
                    // kItemSlots empty items in a row the queue would stand still with this thread waiting on it.
                    if (pending) do_acc();
                    continue;
                }
                const int r = na & 1;
                ok = mbar_wait(bar_res_full(r), (uint32_t)((na >> 1) & 1), wc, 0xb0);
                const uint64_t a_desc = res_desc + (uint64_t)((r * 2 * kBigTile) >> 4);
                for (int it = 0; it < n_it && ok; ++it, ++g) {
                    ok = mbar_wait(bar_ring_full(slot_of(g)), phase_of(g), wc, 0xb2);
                    if (g >= 1) ok = ok && mbar_wait(bar_sdp_free, (uint32_t)((g - 1) & 1), wc, 0xb3);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint64_t bd = b1_desc + (uint64_t)((slot_of(g) * L::kStageBytes) >> 4);
#pragma unroll
                    for (int k = 0; k < kD / 16; ++k) mma_ss(d1, a_desc + 2 * k, bd + 2 * k, idesc_s, k > 0);
                    mma_commit(bar_sdp_full);
                    LTCA_TRACE_EVT(0x20 + (g << 8));
                    if (it == n_it - 1) mma_commit(bar_res_empty(r));   // K (or V) of this item is no longer read
                    if (pending) do_acc();
                    if (!ok) break;
                    p_g = g; p_na = na; p_acc = it > 0; p_first = it == 0;
                    pending = true;
                }
                ++na;
            }
            if (ok && pending) do_acc();
            if (ok && g > 0) ok = mbar_wait(bar_acc_done, (uint32_t)((g - 1) & 1), wc, 0xb5);
        }
      } else {
        // warp 19: stores each item's dK and dV tiles (staged by the elementwise warps in the item's
        // K / V buffer, 128-byte swizzle) with TMA and hands the buffer back to the producer.  Rows
        // past the end of the keys are clipped by the tensor maps.
        if (lane == 0) {
            int na = 0;
            bool ok = true;
            for (int nq = 0; ok; ++nq) {
                const int linear = iq.consume(nq, wc);
                if (linear < 0) break;
                int k0, h, b, kvlen, j_begin;
                const int n_it = item_steps(linear, k0, h, b, kvlen, j_begin);
                if (n_it == 0) continue;
                const int r = na & 1;
                ok = mbar_wait(bar_staged(r), (uint32_t)((na >> 1) & 1), wc, 0xd8);
                if (ok) {
                    tma_store_4d(&tmap_dk, res_smem + r * 2 * kBigTile, 0, k0, h, b);
                    tma_store_4d(&tmap_dv, res_smem + r * 2 * kBigTile + kBigTile, 0, k0, h, b);
                    tma_store_commit();
                    tma_store_wait_read<0>();
                }
                mbar_arrive(bar_res_empty(r));
                ++na;
            }
        }
      }
    } else {
        reg_alloc<kMathRegs>();
        const int wq = warp & 3, cq = warp >> 2;
        const int row = wq * 32 + lane;
        const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
        const uint32_t tS = tmem_base + lane_base + 32 * cq;
        const uint32_t tDP = tS + 128;
        const uint32_t tP = tmem_base + lane_base + 256 + 16 * cq;
        const uint32_t tDS = tP + 64;
        const uint32_t tDV = tmem_base + lane_base + 384 + 16 * cq;
        const uint32_t tDK = tDV + 64;
        const float c2 = a.scale_log2;
        const bool general = (a.keep_mask != nullptr) || (a.use_clamp != 0);

        int g = 0, na = 0;
        bool ok = true;
        for (int nq = 0; ok; ++nq) {
            const int linear = iq.consume_warp(nq, wc);
            if (linear < 0) break;
            int k0, h, b, kvlen, j_begin;
            const int n_it = item_steps(linear, k0, h, b, kvlen, j_begin);
            const int kj = k0 + row;                                   // this thread's key
            const bool key_live = kj < kvlen;
            __nv_bfloat16* dkrow = reinterpret_cast<__nv_bfloat16*>(a.dk) + b * a.dks.batch + h * a.dks.head +
                                   (int64_t)kj * a.dks.seq + cq * 16;
            __nv_bfloat16* dvrow = reinterpret_cast<__nv_bfloat16*>(a.dv) + b * a.dvs.batch + h * a.dvs.head +
                                   (int64_t)kj * a.dvs.seq + cq * 16;
            if (n_it == 0) {
                if (kj < a.Sk) {                       // no query sees these keys: the gradients are zero
                    uint32_t z[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c) z[c] = 0u;
                    store_row16_bf16(dvrow, z, 0.f);
                    store_row16_bf16(dkrow, z, 0.f);
                }
                continue;
            }
            uint32_t s[32], dp[32];
            ok = mbar_wait_warp(bar_sdp_full, (uint32_t)(g & 1), wc, 0xc0);
            if (!ok) break;
            tc_fence_after_sync();
            tmem_ld32(tS, s);
            tmem_ld32(tDP, dp);
            tmem_wait_ld();
            // S^T and dP^T of this step are in registers: the next step's may be computed
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sdp_free);

            for (int it = 0; it < n_it && ok; ++it, ++g) {
                const int j = j_begin + it;
                LTCA_TRACE_EVT(0x11 + (g << 8));
                // lse2 and delta of this thread's 32 query columns (every lane reads the same address)
                const float4* st4 = reinterpret_cast<const float4*>(
                    smem_gen + L::kRingOff + slot_of(g) * L::kStageBytes + 2 * kBigTile) + cq * 8;
                const int q0 = j * kQStep + cq * 32;
                // a query column c is hidden from this key when q0 + c + off < kj
                const bool edge = !key_live || (k0 + kTile > kvlen) ||
                                  (a.causal && (j * kQStep + a.causal_off < k0 + kTile - 1));
                if (general) {
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const float4 l4 = st4[c4];
                        const float4 d4 = st4[32 + c4];
                        const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
                        const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = 4 * c4 + e;
                            const float sv = __uint_as_float(s[c]);
                            float p = fast_exp2(fmaf(sv, c2, -ls[e]));
                            float d = p * (__uint_as_float(dp[c]) - dl[e]);
                            bool vis = key_live && (!a.causal || (kj <= q0 + c + a.causal_off));
                            if (vis && a.keep_mask && (q0 + c) < a.Sq)
                                vis = a.keep_mask[((int64_t)b * a.Sq + q0 + c) * a.Sk + kj] != 0.0f;
                            if (a.use_clamp && sv >= a.clamp_raw) {
                                p = fast_exp2(a.clamp_log2 - ls[e]);
                                d = 0.f;
                            }
                            s[c] = __float_as_uint(vis ? p : 0.f);
                            dp[c] = __float_as_uint(vis ? d : 0.f);
                        }
                    }
                } else if (edge) {
                    // causal diagonal or end of the keys, no dense mask: selects only, no branches.
                    // Query column c is visible to this key when c >= cmin.
                    const int cmin = !key_live ? 0x7fffffff : (a.causal ? kj - a.causal_off - q0 : -0x7fffffff);
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const float4 l4 = st4[c4];
                        const float4 d4 = st4[32 + c4];
                        const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
                        const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = 4 * c4 + e;
                            const float p = fast_exp2(fmaf(__uint_as_float(s[c]), c2, -ls[e]));
                            const bool vis = c >= cmin;
                            s[c] = __float_as_uint(vis ? p : 0.f);
                            dp[c] = __float_as_uint(vis ? p * (__uint_as_float(dp[c]) - dl[e]) : 0.f);
                        }
                    }
                } else {
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const float4 l4 = st4[c4];
                        const float4 d4 = st4[32 + c4];
                        const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
                        const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = 4 * c4 + e;
                            const float p = fast_exp2(fmaf(__uint_as_float(s[c]), c2, -ls[e]));
                            s[c] = __float_as_uint(p);
                            dp[c] = __float_as_uint(p * (__uint_as_float(dp[c]) - dl[e]));
                        }
                    }
                }
                uint32_t pt[16], dst[16], unused[16];
                pack32<false>(s, pt, unused);
                pack32<false>(dp, dst, unused);
                LTCA_TRACE_EVT(0x12 + (g << 8));
                if (g > 0) {
                    // the accumulations of the previous step must have read P^T and dS^T
                    ok = mbar_wait_warp(bar_acc_done, (uint32_t)((g - 1) & 1), wc, 0xc1);
                    if (!ok) break;
                }
                LTCA_TRACE_EVT(0x15 + (g << 8));
                tmem_st16(tP, pt);
                tmem_st16(tDS, dst);
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_pds_full);
                LTCA_TRACE_EVT(0x13 + (g << 8));
                // (P^T and dS^T are announced before the next S^T / dP^T are awaited: the tensor pipe is
                // the busier unit in this kernel and must get this step's accumulations as early as possible)
                if (it + 1 < n_it) {
                    ok = mbar_wait_warp(bar_sdp_full, (uint32_t)((g + 1) & 1), wc, 0xc0);
                    if (!ok) break;
                    tc_fence_after_sync();
                    tmem_ld32(tS, s);
                    tmem_ld32(tDP, dp);
                    tmem_wait_ld();
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_sdp_free);
                }
            }
            if (!ok) break;
            // item epilogue: dV and scale * dK out of tensor memory, which is then free for the next item
            ok = mbar_wait_warp(bar_acc_done, (uint32_t)((g - 1) & 1), wc, 0xc2);
            if (!ok) break;
            LTCA_TRACE_EVT(0x18);
            tc_fence_after_sync();
            uint32_t ov[16], ok_[16];
            tmem_ld16(tDV, ov);
            tmem_ld16(tDK, ok_);
            tmem_wait_ld();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_free);
            {
                // this thread's 16 columns of dK (scaled) and dV, bf16, into the item's K and V buffers in
                // the layout of a 128-byte-swizzled TMA box; warp 19 stores the two tiles.  (Storing
                // 16-byte pieces of 128-byte rows straight from registers costs 32 L1 wavefronts per
                // instruction: measured, one item's 2048 wavefronts held up every shared-memory
                // operation of the SM for about 5000 cycles.)
                const int r = na & 1;
                ++na;
                uint8_t* st_k = smem_gen + L::kResOff + r * 2 * kBigTile + row * 128;
                uint8_t* st_v = st_k + kBigTile;
#pragma unroll
                for (int v = 0; v < 2; ++v) {
                    uint4 wk, wv;
                    wk.x = pack_bf16x2(__uint_as_float(ok_[8 * v + 0]) * a.scale, __uint_as_float(ok_[8 * v + 1]) * a.scale);
                    wk.y = pack_bf16x2(__uint_as_float(ok_[8 * v + 2]) * a.scale, __uint_as_float(ok_[8 * v + 3]) * a.scale);
                    wk.z = pack_bf16x2(__uint_as_float(ok_[8 * v + 4]) * a.scale, __uint_as_float(ok_[8 * v + 5]) * a.scale);
                    wk.w = pack_bf16x2(__uint_as_float(ok_[8 * v + 6]) * a.scale, __uint_as_float(ok_[8 * v + 7]) * a.scale);
                    wv.x = pack_bf16x2(__uint_as_float(ov[8 * v + 0]), __uint_as_float(ov[8 * v + 1]));
                    wv.y = pack_bf16x2(__uint_as_float(ov[8 * v + 2]), __uint_as_float(ov[8 * v + 3]));
                    wv.z = pack_bf16x2(__uint_as_float(ov[8 * v + 4]), __uint_as_float(ov[8 * v + 5]));
                    wv.w = pack_bf16x2(__uint_as_float(ov[8 * v + 6]), __uint_as_float(ov[8 * v + 7]));
                    const int pos = ((2 * cq + v) ^ (row & 7)) << 4;
                    *reinterpret_cast<uint4*>(st_k + pos) = wk;
                    *reinterpret_cast<uint4*>(st_v + pos) = wv;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_staged(r));
            }
            LTCA_TRACE_EVT(0x19);
        }
    }

    // Out of work: only now may the kernel after this one place its CTAs (released at the start, its blocks would
    // sit beside this kernel's CTAs for the whole run, waiting for it to end).
    grid_launch_dependents();
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) item_counters_release(grid.counters);
    if (warp == kMmaWarp0) {
        __syncwarp();
        if (misc[1]) __nanosleep(200000);
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------
// 4b. dK, dV and dQ in ONE persistent kernel (bf16 operands and results): five contractions per
// (128 keys x 128 queries) block instead of the seven of the two-kernel path, and every exponential once.
// The structure is that of the dK/dV kernel above (work item = 128 keys of one (batch, head), query steps of
// 128, one key per tensor-memory lane); on top of it every step forms this key block's share of
//   dQ_j = dS_j K          (M = 128 queries, N = 64, contraction over the 128 keys)
// and adds it into an fp32 accumulator [B*H, Sq_pad, 64] in global memory with a bulk tensor reduce
// (cp.reduce.async.bulk.tensor ... add: the addition is performed by the memory system, 4.4 - 5.9 TB/s of
// payload measured on B200 in this access pattern, no issue slots of the SM).  A conversion kernel then scales
// the accumulator and writes dQ in the caller's type.  The order in which the key blocks' shares arrive is not
// fixed, so dQ is reproducible only to fp32 rounding (before its conversion to bf16); dK and dV keep one issuing
// thread per accumulator and stay bit-reproducible.  Callers that need bit-identical dQ set
// ltca_attn_params.bwd_deterministic and get the two-kernel path.
//
// dS^T has to be an operand from SHARED memory for dQ (its A operand wants queries along M, and tensor memory
// holds keys along the lanes): the elementwise warps write it there too, in the 128-byte-swizzled layout of two
// [128 keys x 64 queries] blocks, which dQ_j = dS_j K reads as an M-major A operand.
// Tensor memory: S^T [0,128)  dP^T [128,256)  P^T bf16 [256,320)  dS^T bf16, then dQ_j [320,384)  dV [384,448)
// dK [448,512): dK takes dS^T from tensor memory (an operand from shared memory costs 4 KB of shared-memory reads
// per K step, and the contractions with N = 64 are already bound by that bandwidth), and the thread that issues dK
// issues dQ_j right behind it into the same columns.
// Shared memory: K, V (single buffer; released as soon as the item's last contraction has been issued, the
// elementwise warps are busy with the item's epilogue while the next item's tiles arrive) | ring of three
// (Q_j, dO_j, lse2_j, delta_j) stages | dS^T (32 KB; also the staging area of the item's dK / dV tiles) |
// dQ_j staging (fp32, two 128-byte-swizzled boxes of 32 columns).
// Warp 16 issues S^T and dV, warp 17 dP^T, dK and dQ_j, warp 18 is the TMA producer, warp 19 issues the
// reduces of dQ_j and the stores of dK / dV.
// ---------------------------------------------------------------------------------------------
struct FusedSmem {
    static constexpr int kStages = 3;                         // ring of (Q_j, dO_j, lse2_j, delta_j)
    static constexpr int kStageBytes = 2 * kBigTile + 1024;
    static constexpr int kResOff = 0;                         // K, V
    static constexpr int kRingOff = 2 * kBigTile;
    static constexpr int kDsOff = kRingOff + kStages * kStageBytes;
    static constexpr int kDsBytes = 2 * kBigTile;             // bf16 [2 blocks of 64 queries][128 keys][128 B]
    static constexpr int kDqOff = kDsOff + kDsBytes;
    static constexpr int kDqBytes = kTile * kD * 4;           // fp32 [2 boxes of 32 columns][128 queries][128 B]
    static constexpr int kBarOff = kDqOff + kDqBytes;
    // bars: res_full, res_empty, ring_full[S], ring_empty[S], sdp_full, sdp_free, pds_full, acc_done, acc_free,
    // dq_staged, dq_free, kv_staged, dsbuf_free, item_full[kItemSlots], item_empty[kItemSlots]
    static constexpr int kNumBars = 2 + 2 * kStages + 9 + 2 * kItemSlots;
    static constexpr int kMiscOff = kBarOff + kNumBars * 8;   // tmem base, abort flag, item slots
    static constexpr int kDynBytes = kMiscOff + 16 + 4 * kItemSlots + 1024;
};
static_assert(FusedSmem::kDynBytes <= 227 * 1024, "shared memory plan of the fused backward kernel");
constexpr int kFusedCtrlRegs = 64;   // the MMA thread of dP^T / dK / dQ_j holds three more operand descriptors
static_assert(512 * kMathRegs + 128 * kFusedCtrlRegs <= kThreads * kLaunchRegs, "register budget");

__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_fused_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q,
                            const __grid_constant__ CUtensorMap tmap_do,
                            const __grid_constant__ CUtensorMap tmap_k,
                            const __grid_constant__ CUtensorMap tmap_v,
                            const __grid_constant__ CUtensorMap tmap_dk,
                            const __grid_constant__ CUtensorMap tmap_dv,
                            const __grid_constant__ CUtensorMap tmap_dqacc, const BwdArgs a, const ItemGrid grid) {
    using L = FusedSmem;
    constexpr int kQStep = 128;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t res_smem = smem_base + L::kResOff;
    const uint32_t ring_smem = smem_base + L::kRingOff, bar_base = smem_base + L::kBarOff;
    const uint32_t ds_smem = smem_base + L::kDsOff, dq_smem = smem_base + L::kDqOff;
    const uint32_t bar_res_full = bar_base, bar_res_empty = bar_base + 8u;
    auto bar_ring_full = [&](int s) { return bar_base + 8u * (2 + s); };
    auto bar_ring_empty = [&](int s) { return bar_base + 8u * (2 + L::kStages + s); };
    const uint32_t bar_sdp_full = bar_base + 8u * (2 + 2 * L::kStages);
    const uint32_t bar_sdp_free = bar_sdp_full + 8u;
    const uint32_t bar_pds_full = bar_sdp_full + 16u;
    const uint32_t bar_acc_done = bar_sdp_full + 24u;
    const uint32_t bar_acc_free = bar_sdp_full + 32u;
    const uint32_t bar_dq_staged = bar_sdp_full + 40u;      // the 16 warps have written dQ_j into the staging area
    const uint32_t bar_dq_free = bar_sdp_full + 48u;        // the reduce has read the staging area
    const uint32_t bar_kv_staged = bar_sdp_full + 56u;      // the 16 warps have written dK / dV into the dS^T area
    const uint32_t bar_dsbuf_free = bar_sdp_full + 64u;     // the stores of dK / dV have read the dS^T area
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);
    const ItemQueue iq{bar_sdp_full + 72u, bar_sdp_full + 72u + 8u * kItemSlots,
                       reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 16)};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_q = (a.Sq + kQStep - 1) / kQStep;   // query steps in total
    LTCA_TRACE_DECL(LTCA_TRACE_KERNEL == 5 && blockIdx.x == 5);
    LTCA_TRACE_EVT(0x01);

    if (threadIdx.x == 0) {
        mbar_init(bar_res_full, 1);
        mbar_init(bar_res_empty, 2);               // both MMA threads are done with K and V
        for (int s = 0; s < L::kStages; ++s) { mbar_init(bar_ring_full(s), 1); mbar_init(bar_ring_empty(s), 2); }
        mbar_init(bar_sdp_full, 2);                // one commit per MMA thread
        mbar_init(bar_sdp_free, 16);               // one arrival per elementwise warp
        mbar_init(bar_pds_full, 16);
        mbar_init(bar_acc_done, 2);
        mbar_init(bar_acc_free, 16);
        mbar_init(bar_dq_staged, 16);
        mbar_init(bar_dq_free, 1);
        mbar_init(bar_kv_staged, 16);
        mbar_init(bar_dsbuf_free, 1);
        for (int i = 0; i < kItemSlots; ++i) { mbar_init(iq.full(i), 1); mbar_init(iq.empty(i), 19); }
        misc[1] = 0u;
        mbar_fence_init();
    }
    if (warp == kMmaWarp0) { tmem_alloc(smem_u32(const_cast<uint32_t*>(&misc[0])), kTmemCols); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = misc[0];
    const WaitCtx wc{&misc[1], a.status};
    grid_dependency_wait();                    // the operands are complete once the kernel before this one has ended
    auto slot_of = [&](int g) { return g % L::kStages; };
    auto phase_of = [&](int g) { return (uint32_t)((g / L::kStages) & 1); };
    // the item's key tile, first query step that can see it and number of query steps (0: none)
    auto item_steps = [&](int linear, int& k0, int& h, int& b, int& kvlen, int& j_begin) {
        int rank;
        sched_item(grid, linear, rank, h, b);
        k0 = rank * kTile;                          // early key blocks carry the most causal work
        kvlen = a.Sk;
        if (a.kv_len) kvlen = min(max(a.kv_len[b], 0), a.Sk);
        j_begin = 0;
        if (a.causal) j_begin = max(0, k0 - a.causal_off) / kQStep;
        const bool active = (k0 < kvlen) && (j_begin < n_q);
        return active ? n_q - j_begin : 0;
    };

    if (warp >= 16) {
      reg_dealloc<kFusedCtrlRegs>();
      if (warp == kTmaWarp) {
        if (lane == 0) {
            int g = 0, na = 0;
            bool ok = true;
            for (int nq = 0; ok; ++nq) {
                const int linear = iq.produce(nq, grid.counters, grid.n_items, wc);
                if (linear < 0) break;
                int k0, h, b, kvlen, j_begin;
                const int n_it = item_steps(linear, k0, h, b, kvlen, j_begin);
                if (n_it == 0) continue;
                ok = mbar_wait(bar_res_empty, (uint32_t)((na & 1) ^ 1), wc, 0xe1);
                if (!ok) break;
                mbar_arrive_expect_tx(bar_res_full, 2u * kBigTile);
                tma_load_4d(res_smem, &tmap_k, bar_res_full, 0, k0, h, b);
                tma_load_4d(res_smem + kBigTile, &tmap_v, bar_res_full, 0, k0, h, b);
                const float* lse2_row = a.lse2 + ((int64_t)b * a.H + h) * a.Sq_pad;
                const float* dlt_row = a.delta + ((int64_t)b * a.H + h) * a.Sq_pad;
                for (int it = 0; it < n_it && ok; ++it, ++g) {
                    const int j = j_begin + it;
                    ok = mbar_wait(bar_ring_empty(slot_of(g)), phase_of(g) ^ 1u, wc, 0xe0);
                    if (!ok) break;
                    const uint32_t st = ring_smem + slot_of(g) * L::kStageBytes;
                    const uint32_t bar = bar_ring_full(slot_of(g));
                    mbar_arrive_expect_tx(bar, 2u * kBigTile + 1024u);
                    tma_load_4d(st, &tmap_q, bar, 0, j * kQStep, h, b);
                    tma_load_4d(st + kBigTile, &tmap_do, bar, 0, j * kQStep, h, b);
                    asm volatile(
                        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 512, [%2];"
                        ::"r"(st + 2 * kBigTile), "l"(reinterpret_cast<uint64_t>(lse2_row + j * kQStep)), "r"(bar)
                        : "memory");
                    asm volatile(
                        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 512, [%2];"
                        ::"r"(st + 2 * kBigTile + 512), "l"(reinterpret_cast<uint64_t>(dlt_row + j * kQStep)),
                          "r"(bar)
                        : "memory");
                }
                ++na;
            }
        }
      } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
        // which == 0: S^T = K Q_j^T and dV += P^T dO_j
        // which == 1: dP^T = V dO_j^T, dK += dS^T Q_j and dQ_j = dS_j K
        // one instantiation per role, so that each thread's code only carries its own operand descriptors
        auto mma_role = [&](auto which_c) {
            constexpr int which = decltype(which_c)::value;
            constexpr uint32_t idesc_s = make_idesc_bf16(kTile, kQStep, 0, 0);
            constexpr uint32_t idesc_acc = make_idesc_bf16(kTile, kD, 0, 1);    // A K-major (or tensor memory), B N-major
            constexpr uint32_t idesc_dq = make_idesc_bf16(kQStep, kD, 1, 1);    // A M-major (dS^T read as dS), B N-major
            // (descriptors as low words, see mma_ss_lo: offsets are plain 32-bit additions of bytes >> 4.)
            // The bases pass through an opaque move inside the role, so that the compiler forms each role's
            // descriptors inside that role instead of hoisting both sets above the branch between the two roles
            // (which costs the control warps, at 64 registers, a spill on every step).
            uint32_t opaque_zero;
            asm volatile("mov.u32 %0, 0;" : "=r"(opaque_zero));
            const uint32_t res_b = res_smem + opaque_zero, ring_b = ring_smem + opaque_zero;
            const uint32_t ds_b = ds_smem + opaque_zero, tm_b = tmem_base + opaque_zero;
            const uint32_t a_desc = smem_desc_lo(res_b + (which == 0 ? 0 : kBigTile), 16);
            // the streamed operand of the first contraction (Q for S^T, dO for dP^T), K-major
            const uint32_t b1_desc = smem_desc_lo(ring_b + (which == 0 ? 0 : kBigTile), 16);
            // the streamed operand of the accumulation (dO for dV, Q for dK), rows as the contraction index
            const uint32_t b2_desc = smem_desc_lo(ring_b + (which == 0 ? kBigTile : 0), 8192);
            // dS^T in shared memory as the M-major A operand of dQ_j: blocks of 64 queries 16 KB apart, 16 key
            // rows = 2 KB per K step
            const uint32_t ds_m_desc = smem_desc_lo(ds_b, kBigTile);
            // K as the N-major B operand of dQ_j: 128 key rows of 128 bytes, 16 rows per K step
            const uint32_t kn_desc = smem_desc_lo(res_b, 8192);
            const uint32_t d1 = tm_b + (which == 0 ? 0 : 128);
            const uint32_t a2 = tm_b + 256;                      // P^T (which == 0 only)
            const uint32_t d2 = tm_b + (which == 0 ? 384 : 448);
            const uint32_t ds_tmem = tm_b + 320;                 // dS^T (bf16) of the step, then dQ_j (which == 1 only)
            // the accumulation that is still to be issued (one step behind the first contraction)
            bool pending = false;
            int p_g = 0, p_na = 0;
            bool p_acc = false, p_first = false, p_last = false;
            bool ok = true;
            auto do_acc = [&]() {
                ok = mbar_wait(bar_pds_full, (uint32_t)(p_g & 1), wc, 0xf4);
                LTCA_TRACE_EVT(0x21 + (p_g << 8));
                // the previous item's dV / dK must have left tensor memory before they are overwritten
                if (ok && p_first && p_na > 0) ok = mbar_wait(bar_acc_free, (uint32_t)((p_na - 1) & 1), wc, 0xf6);
                if (!ok) return;
                tc_fence_after_sync();
                const uint32_t bd = b2_desc + (uint32_t)((slot_of(p_g) * L::kStageBytes) >> 4);
                if constexpr (which == 0) {
#pragma unroll
                    for (int k = 0; k < kQStep / 16; ++k)
                        mma_ts_lo(d2, a2 + k * 8, bd + 128 * k, idesc_acc, (p_acc || k > 0) ? 1u : 0u);
                } else {
                    // dK takes dS^T from tensor memory; dQ_j then overwrites those very columns: one thread's
                    // contractions run in order, so dK has read them by then
#pragma unroll
                    for (int k = 0; k < kQStep / 16; ++k)
                        mma_ts_lo(d2, ds_tmem + k * 8, bd + 128 * k, idesc_acc, (p_acc || k > 0) ? 1u : 0u);
#pragma unroll
                    for (int k = 0; k < kTile / 16; ++k)
                        mma_ss_lo(ds_tmem, ds_m_desc + 128 * k, kn_desc + 128 * k, idesc_dq, k > 0 ? 1u : 0u);
                }
                mma_commit(bar_acc_done);
                mma_commit(bar_ring_empty(slot_of(p_g)));
                if (p_last) mma_commit(bar_res_empty);          // K (or V) of this item is no longer read
                LTCA_TRACE_EVT(0x22 + (p_g << 8));
                pending = false;
            };
            int g = 0, na = 0;
            for (int nq = 0; ok; ++nq) {
                const int linear = iq.consume(nq, wc);
                if (linear < 0) break;
                int k0, h, b, kvlen, j_begin;
                const int n_it = item_steps(linear, k0, h, b, kvlen, j_begin);
                // The previous item's last accumulation reads K / V of that item: it goes out before the wait
                // for this item's tiles, which arrive only after that accumulation has released the buffer - and
                // before an item without work is skipped: the elementwise warps wait for it at the end of the
                // item before, so they take no further queue entry, and after kItemSlots empty items in a row
                // the queue would stand still with this thread waiting on it.
                if (pending) do_acc();
                if (!ok) break;
                if (n_it == 0) continue;
                ok = mbar_wait(bar_res_full, (uint32_t)(na & 1), wc, 0xf0);
                for (int it = 0; it < n_it && ok; ++it, ++g) {
                    ok = mbar_wait(bar_ring_full(slot_of(g)), phase_of(g), wc, 0xf2);
                    if (g >= 1) ok = ok && mbar_wait(bar_sdp_free, (uint32_t)((g - 1) & 1), wc, 0xf3);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t bd = b1_desc + (uint32_t)((slot_of(g) * L::kStageBytes) >> 4);
#pragma unroll
                    for (int k = 0; k < kD / 16; ++k) mma_ss_lo(d1, a_desc + 2 * k, bd + 2 * k, idesc_s, k > 0);
                    mma_commit(bar_sdp_full);
                    LTCA_TRACE_EVT(0x20 + (g << 8));
                    if (pending) do_acc();
                    if (!ok) break;
                    p_g = g; p_na = na; p_acc = it > 0; p_first = it == 0; p_last = it == n_it - 1;
                    pending = true;
                }
                ++na;
            }
            if (ok && pending) do_acc();
            if (ok && g > 0) ok = mbar_wait(bar_acc_done, (uint32_t)((g - 1) & 1), wc, 0xf5);
        };
        if (lane == 0) {
            if (warp == kMmaWarp0) mma_role(std::integral_constant<int, 0>{});
            else mma_role(std::integral_constant<int, 1>{});
        }
      } else {
        // warp 19: adds every step's dQ_j tile into the fp32 accumulator (two boxes of 32 columns) and stores each
        // item's dK and dV tiles (staged by the elementwise warps in the dS^T area).  Rows past the end of the
        // keys are clipped by the tensor maps; the accumulator's rows are padded to whole steps.
        if (lane == 0) {
            int g = 0, na = 0;
            bool ok = true;
            for (int nq = 0; ok; ++nq) {
                const int linear = iq.consume(nq, wc);
                if (linear < 0) break;
                int k0, h, b, kvlen, j_begin;
                const int n_it = item_steps(linear, k0, h, b, kvlen, j_begin);
                if (n_it == 0) continue;
                for (int it = 0; it < n_it && ok; ++it, ++g) {
                    ok = mbar_wait(bar_dq_staged, (uint32_t)(g & 1), wc, 0xe8);
                    if (!ok) break;
                    LTCA_TRACE_EVT(0x30 + (g << 8));
                    const int q0 = (j_begin + it) * kQStep;
                    tma_reduce_add_4d(&tmap_dqacc, dq_smem, 0, q0, h, b);
                    tma_reduce_add_4d(&tmap_dqacc, dq_smem + kTile * 128, 32, q0, h, b);
                    tma_store_commit();
                    tma_store_wait_read<0>();
                    LTCA_TRACE_EVT(0x31 + (g << 8));
                    mbar_arrive(bar_dq_free);
                }
                if (!ok) break;
                ok = mbar_wait(bar_kv_staged, (uint32_t)(na & 1), wc, 0xe9);
                if (ok) {
                    tma_store_4d(&tmap_dk, ds_smem, 0, k0, h, b);
                    tma_store_4d(&tmap_dv, ds_smem + kBigTile, 0, k0, h, b);
                    tma_store_commit();
                    tma_store_wait_read<0>();
                }
                mbar_arrive(bar_dsbuf_free);
                ++na;
            }
            tma_store_wait_all<0>();                // every reduce and store has landed before the CTA ends
        }
      }
    } else {
        reg_alloc<kMathRegs>();
        const int wq = warp & 3, cq = warp >> 2;
        const int row = wq * 32 + lane;
        const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
        const uint32_t tS = tmem_base + lane_base + 32 * cq;
        const uint32_t tDP = tS + 128;
        const uint32_t tP = tmem_base + lane_base + 256 + 16 * cq;
        const uint32_t tDQ = tmem_base + lane_base + 320 + 16 * cq;
        const uint32_t tDV = tmem_base + lane_base + 384 + 16 * cq;
        const uint32_t tDK = tDV + 64;
        const float c2 = a.scale_log2;
        const bool general = (a.keep_mask != nullptr) || (a.use_clamp != 0);
        // this thread's 64 bytes of its dS^T row (32 query columns of key `row`): block cq / 2, 16-byte chunks
        // 4 (cq % 2) .. + 3, swizzled with the row; the dQ_j staging uses the same geometry with fp32 columns
        // 16 cq .. + 15 of query `row`: box cq / 2, chunks 4 (cq % 2) .. + 3
        // (both areas have the same size and geometry, so one 32-bit address serves both)
        static_assert(L::kDqBytes == L::kDsBytes && kTile * 128 == kBigTile, "dS^T and dQ staging share their geometry");
        const uint32_t ds_row = ds_smem + (uint32_t)((cq >> 1) * kBigTile + row * 128);
        const uint32_t chunk0 = (uint32_t)((cq & 1) * 4);
        const uint32_t sw = (uint32_t)(row & 7);

        int g = 0, na = 0;
        bool ok = true;
        // dQ_j of step g - 1: out of tensor memory, into the staging area, announced to the reducing thread
        // (the caller has already waited for the staging area: no loop in here, so that the 16 values are not kept
        // in registers across a wait)
        auto stage_dq = [&](const uint32_t (&dqv)[16], int gprev) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                st_shared_v4(ds_row + (uint32_t)L::kDsBytes + (((chunk0 + i) ^ sw) << 4), dqv[4 * i], dqv[4 * i + 1],
                             dqv[4 * i + 2], dqv[4 * i + 3]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_dq_staged);
            LTCA_TRACE_EVT(0x16 + (gprev << 8));
        };
        // the reduce of tile gprev - 1 has read the staging area
        auto wait_dq_stage = [&](int gprev) {
            if (gprev > 0) ok = mbar_wait_warp(bar_dq_free, (uint32_t)((gprev - 1) & 1), wc, 0xca);
        };
        for (int nq = 0; ok; ++nq) {
            const int linear = iq.consume_warp(nq, wc);
            if (linear < 0) break;
            int k0, h, b, kvlen, j_begin;
            const int n_it = item_steps(linear, k0, h, b, kvlen, j_begin);
            const int kj = k0 + row;                                   // this thread's key
            const bool key_live = kj < kvlen;
            if (n_it == 0) {
                if (kj < a.Sk) {                       // no query sees these keys: the gradients are zero
                    __nv_bfloat16* dkrow = reinterpret_cast<__nv_bfloat16*>(a.dk) + b * a.dks.batch +
                                           h * a.dks.head + (int64_t)kj * a.dks.seq + cq * 16;
                    __nv_bfloat16* dvrow = reinterpret_cast<__nv_bfloat16*>(a.dv) + b * a.dvs.batch +
                                           h * a.dvs.head + (int64_t)kj * a.dvs.seq + cq * 16;
                    uint32_t z[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c) z[c] = 0u;
                    store_row16_bf16(dvrow, z, 0.f);
                    store_row16_bf16(dkrow, z, 0.f);
                }
                continue;
            }
            for (int it = 0; it < n_it && ok; ++it, ++g) {
                const int j = j_begin + it;
                // S^T and dP^T of this step into registers (defined afresh in every iteration, so that they are
                // not carried round the loop); the next step's may then be computed
                uint32_t s[32], dp[32];
                ok = mbar_wait_warp(bar_sdp_full, (uint32_t)(g & 1), wc, 0xc0);
                if (!ok) break;
                LTCA_TRACE_EVT(0x10 + (g << 8));
                tc_fence_after_sync();
                tmem_ld32(tS, s);
                tmem_ld32(tDP, dp);
                tmem_wait_ld();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_sdp_free);
                LTCA_TRACE_EVT(0x11 + (g << 8));
                // lse2 and delta of this thread's 32 query columns (every lane reads the same address)
                const float4* st4 = reinterpret_cast<const float4*>(
                    smem_gen + L::kRingOff + slot_of(g) * L::kStageBytes + 2 * kBigTile) + cq * 8;
                const int q0 = j * kQStep + cq * 32;
                // a query column c is hidden from this key when q0 + c + off < kj
                const bool edge = !key_live || (k0 + kTile > kvlen) ||
                                  (a.causal && (j * kQStep + a.causal_off < k0 + kTile - 1));
                if (general) {
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const float4 l4 = st4[c4];
                        const float4 d4 = st4[32 + c4];
                        const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
                        const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = 4 * c4 + e;
                            const float sv = __uint_as_float(s[c]);
                            float pv = fast_exp2(fmaf(sv, c2, -ls[e]));
                            float d = pv * (__uint_as_float(dp[c]) - dl[e]);
                            bool vis = key_live && (!a.causal || (kj <= q0 + c + a.causal_off));
                            if (vis && a.keep_mask && (q0 + c) < a.Sq)
                                vis = a.keep_mask[((int64_t)b * a.Sq + q0 + c) * a.Sk + kj] != 0.0f;
                            if (a.use_clamp && sv >= a.clamp_raw) {
                                pv = fast_exp2(a.clamp_log2 - ls[e]);
                                d = 0.f;
                            }
                            s[c] = __float_as_uint(vis ? pv : 0.f);
                            dp[c] = __float_as_uint(vis ? d : 0.f);
                        }
                    }
                } else if (edge) {
                    // causal diagonal or end of the keys, no dense mask: selects only, no branches.
                    // Query column c is visible to this key when c >= cmin.
                    const int cmin = !key_live ? 0x7fffffff : (a.causal ? kj - a.causal_off - q0 : -0x7fffffff);
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const float4 l4 = st4[c4];
                        const float4 d4 = st4[32 + c4];
                        const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
                        const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = 4 * c4 + e;
                            const float pv = fast_exp2(fmaf(__uint_as_float(s[c]), c2, -ls[e]));
                            const bool vis = c >= cmin;
                            s[c] = __float_as_uint(vis ? pv : 0.f);
                            dp[c] = __float_as_uint(vis ? pv * (__uint_as_float(dp[c]) - dl[e]) : 0.f);
                        }
                    }
                } else {
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const float4 l4 = st4[c4];
                        const float4 d4 = st4[32 + c4];
                        const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
                        const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = 4 * c4 + e;
                            const float pv = fast_exp2(fmaf(__uint_as_float(s[c]), c2, -ls[e]));
                            s[c] = __float_as_uint(pv);
                            dp[c] = __float_as_uint(pv * (__uint_as_float(dp[c]) - dl[e]));
                        }
                    }
                }
                uint32_t pt[16], dst[16], unused[16];
                pack32<false>(s, pt, unused);
                pack32<false>(dp, dst, unused);
                LTCA_TRACE_EVT(0x12 + (g << 8));
                if (g > 0) {
                    // the contractions of the previous step have read P^T and dS^T, and its dQ_j is complete
                    ok = mbar_wait_warp(bar_acc_done, (uint32_t)((g - 1) & 1), wc, 0xc1);
                    if (!ok) break;
                }
                if (it > 0) {
                    wait_dq_stage(g - 1);
                    if (!ok) break;
                }
                // the first dS^T of an item goes where the previous item's dK / dV tiles were staged
                if (it == 0 && na > 0) {
                    ok = mbar_wait_warp(bar_dsbuf_free, (uint32_t)((na - 1) & 1), wc, 0xc3);
                    if (!ok) break;
                }
                LTCA_TRACE_EVT(0x13 + (g << 8));
                tc_fence_after_sync();
                // dQ_j of the previous step sits in the columns that take this step's dS^T: out first (read at an
                // item's first step too, where it is not used: a conditional load would keep 16 registers alive
                // round the loop)
                uint32_t dqv[16];
                tmem_ld16(tDQ, dqv);
                tmem_st16(tP, pt);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    st_shared_v4(ds_row + (((chunk0 + i) ^ sw) << 4), dst[4 * i], dst[4 * i + 1], dst[4 * i + 2],
                                 dst[4 * i + 3]);
                tmem_wait_ld();
                tmem_st16(tDQ, dst);                          // dS^T for dK (tensor memory) and for dQ_j (shared memory)
                if (it > 0) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        st_shared_v4(ds_row + (uint32_t)L::kDsBytes + (((chunk0 + i) ^ sw) << 4), dqv[4 * i],
                                     dqv[4 * i + 1], dqv[4 * i + 2], dqv[4 * i + 3]);
                }
                fence_proxy_async_smem();                     // one fence for dS^T and the staged dQ_j
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar_pds_full);
                    if (it > 0) mbar_arrive(bar_dq_staged);
                }
                LTCA_TRACE_EVT(0x14 + (g << 8));
            }
            if (!ok) break;
            // item epilogue: the last dQ_j, then dV and scale * dK out of tensor memory
            ok = mbar_wait_warp(bar_acc_done, (uint32_t)((g - 1) & 1), wc, 0xc2);
            if (!ok) break;
            tc_fence_after_sync();
            wait_dq_stage(g - 1);
            if (!ok) break;
            uint32_t ov[16], ok_[16];
            {
                uint32_t dqv[16];
                tmem_ld16(tDQ, dqv);
                tmem_ld16(tDV, ov);
                tmem_ld16(tDK, ok_);
                tmem_wait_ld();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_free);
                stage_dq(dqv, g - 1);
            }
            {
                // this thread's 16 columns of dK (scaled) and dV, bf16, into the dS^T area (the item's last
                // contractions have read it) in the layout of two 128-byte-swizzled TMA boxes
                const uint32_t st_k = ds_smem + (uint32_t)(row * 128);
#pragma unroll
                for (int v = 0; v < 2; ++v) {
                    const uint32_t pos = (((uint32_t)(2 * cq + v)) ^ sw) << 4;
                    st_shared_v4(st_k + pos,
                                 pack_bf16x2(__uint_as_float(ok_[8 * v + 0]) * a.scale, __uint_as_float(ok_[8 * v + 1]) * a.scale),
                                 pack_bf16x2(__uint_as_float(ok_[8 * v + 2]) * a.scale, __uint_as_float(ok_[8 * v + 3]) * a.scale),
                                 pack_bf16x2(__uint_as_float(ok_[8 * v + 4]) * a.scale, __uint_as_float(ok_[8 * v + 5]) * a.scale),
                                 pack_bf16x2(__uint_as_float(ok_[8 * v + 6]) * a.scale, __uint_as_float(ok_[8 * v + 7]) * a.scale));
                    st_shared_v4(st_k + (uint32_t)kBigTile + pos,
                                 pack_bf16x2(__uint_as_float(ov[8 * v + 0]), __uint_as_float(ov[8 * v + 1])),
                                 pack_bf16x2(__uint_as_float(ov[8 * v + 2]), __uint_as_float(ov[8 * v + 3])),
                                 pack_bf16x2(__uint_as_float(ov[8 * v + 4]), __uint_as_float(ov[8 * v + 5])),
                                 pack_bf16x2(__uint_as_float(ov[8 * v + 6]), __uint_as_float(ov[8 * v + 7])));
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_kv_staged);
                ++na;
            }
        }
    }

    // Out of work: only now may the kernel after this one place its CTAs (released at the start, its blocks would
    // sit beside this kernel's CTAs for the whole run, waiting for it to end).
    grid_launch_dependents();
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) item_counters_release(grid.counters);
    if (warp == kMmaWarp0) {
        __syncwarp();
        if (misc[1]) __nanosleep(200000);
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// The fp32 dQ accumulator of the fused kernel, scaled, into the caller's dQ (bf16, any strides); 8 lanes per row.
__global__ void __launch_bounds__(256) attn_bwd_dq_convert_kernel(const float* __restrict__ acc, void* dq,
                                                                  ltca_strides dqs, int B, int H, int Sq, int Sq_pad,
                                                                  float scale) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int64_t idx = (int64_t)blockIdx.x * 32 + (threadIdx.x >> 3);       // row among B * H * Sq
    const int sub = threadIdx.x & 7;
    if (idx >= (int64_t)B * H * Sq) return;
    const int qi = (int)(idx % Sq);
    const int64_t bh = idx / Sq;
    const int h = (int)(bh % H), b = (int)(bh / H);
    const float4* src = reinterpret_cast<const float4*>(acc + (bh * Sq_pad + qi) * kD + 8 * sub);
    const float4 x = __ldg(src), y = __ldg(src + 1);
    uint4 w;
    w.x = pack_bf16x2(x.x * scale, x.y * scale);
    w.y = pack_bf16x2(x.z * scale, x.w * scale);
    w.z = pack_bf16x2(y.x * scale, y.y * scale);
    w.w = pack_bf16x2(y.z * scale, y.w * scale);
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(dq) + b * dqs.batch + h * dqs.head + (int64_t)qi * dqs.seq + 8 * sub;
    *reinterpret_cast<uint4*>(dst) = w;
}

// ---------------------------------------------------------------------------------------------
// 5. dQ, single-tile persistent variant (bf16 operands and results).
// Work item = 128 queries of one (batch, head); key steps of 128; nothing aliased in tensor memory:
//   S [0,128)  dP [128,256)  dQ [320,384)  and three dS (bf16) buffers used in turn,
//   [256,320) [384,448) [448,512).
// One CTA per SM walks a list of items (item i of CTA c is entry c + i * gridDim.x of the
// grouped heavy-first order, so all CTAs get nearly the same work).  Barriers, tensor memory and
// tensor maps are set up once; the Q / dO tile is double-buffered, so the producer loads the next
// item's tile and first key steps while the current item drains, the MMA thread computes the next
// item's first S and dP while the elementwise warps write the current item's dQ.  Measured before
// this change: 4.5 us of prologue, pipeline fill and epilogue per 128-query tile, 20 % of the kernel.
// Elementwise warp w owns query rows 32 (w % 4) .. +31 and key columns 32 (w / 4) .. +31 of a
// step.  Warp 16 issues S and dP one step ahead, warp 17 issues dQ += dS K_j.
// ---------------------------------------------------------------------------------------------
struct Dq4Smem {
    static constexpr int kStages = 4;                         // ring of (K_j, V_j)
    static constexpr int kStageBytes = 2 * kBigTile;
    static constexpr int kResOff = 0;                         // two (Q, dO) buffers
    static constexpr int kRingOff = 4 * kBigTile;
    static constexpr int kBarOff = kRingOff + kStages * kStageBytes;
    // bars: res_full[2], res_empty[2], ring_full[S], ring_empty[S], sdp_full, sdp_free, ds_full[3],
    // ds_free[3], acc_free, item_full[kItemSlots], item_empty[kItemSlots], staged[2]
    static constexpr int kNumBars = 4 + 2 * kStages + 9 + 2 * kItemSlots + 2;
    static constexpr int kMiscOff = kBarOff + kNumBars * 8;        // tmem base, abort flag, item slots
    static constexpr int kDynBytes = kMiscOff + 16 + 4 * kItemSlots + 1024;
};

__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_dq4_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q,
                          const __grid_constant__ CUtensorMap tmap_do,
                          const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_dq, const BwdArgs a, const ItemGrid grid) {
    using L = Dq4Smem;
    constexpr int kKStep = 128;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t res_smem = smem_base + L::kResOff;
    const uint32_t ring_smem = smem_base + L::kRingOff, bar_base = smem_base + L::kBarOff;
    auto bar_res_full = [&](int r) { return bar_base + 8u * r; };
    auto bar_res_empty = [&](int r) { return bar_base + 8u * (2 + r); };
    auto bar_ring_full = [&](int s) { return bar_base + 8u * (4 + s); };
    auto bar_ring_empty = [&](int s) { return bar_base + 8u * (4 + L::kStages + s); };
    const uint32_t bar_sdp_full = bar_base + 8u * (4 + 2 * L::kStages);
    const uint32_t bar_sdp_free = bar_sdp_full + 8u;
    // One pair of barriers per dS buffer.  A barrier that is reused every step could complete
    // twice before a late waiter looks at it, and a parity wait cannot tell "not yet" from
    // "two phases ago"; with one barrier per buffer the next completion always depends on the
    // waiter itself.
    auto bar_ds_full = [&](int g) { return bar_sdp_full + 16u + 8u * (g % 3); };     // dS of step g stored
    auto bar_ds_free = [&](int g) { return bar_sdp_full + 40u + 8u * (g % 3); };     // dQ of step g done
    auto ds_parity = [&](int g) { return (uint32_t)((g / 3) & 1); };
    const uint32_t bar_acc_free = bar_sdp_full + 64u;
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);
    const ItemQueue iq{bar_sdp_full + 72u, bar_sdp_full + 72u + 8u * kItemSlots,
                       reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 16)};
    // dQ of an item staged in the item's own Q buffer (one barrier per buffer)
    auto bar_staged = [&](int r) { return bar_sdp_full + 72u + 16u * kItemSlots + 8u * r; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        // a Q / dO buffer is free again when the MMA thread is done with it and the item's dQ, which is
        // staged in its Q half, has been read by its TMA store
        for (int r = 0; r < 2; ++r) {
            mbar_init(bar_res_full(r), 1);
            mbar_init(bar_res_empty(r), 2);
            mbar_init(bar_staged(r), 16);
        }
        for (int s = 0; s < L::kStages; ++s) { mbar_init(bar_ring_full(s), 1); mbar_init(bar_ring_empty(s), 2); }
        mbar_init(bar_sdp_full, 1);
        mbar_init(bar_sdp_free, 16);               // one arrival per elementwise warp
        for (int r = 0; r < 3; ++r) { mbar_init(bar_ds_full(r), 16); mbar_init(bar_ds_free(r), 1); }
        mbar_init(bar_acc_free, 16);
        for (int i = 0; i < kItemSlots; ++i) { mbar_init(iq.full(i), 1); mbar_init(iq.empty(i), 19); }
        misc[1] = 0u;
        mbar_fence_init();
    }
    if (warp == kMmaWarp0) { tmem_alloc(smem_u32(const_cast<uint32_t*>(&misc[0])), kTmemCols); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = misc[0];
    const WaitCtx wc{&misc[1], a.status};
    grid_dependency_wait();                    // the operands are complete once the kernel before this one has ended
    auto slot_of = [&](int g) { return g % L::kStages; };
    auto phase_of = [&](int g) { return (uint32_t)((g / L::kStages) & 1); };
    // tensor-memory column of the dS buffer of step g: 256, 384, 448 in turn
    auto ds_col = [&](int g) { const int r = g % 3; return (uint32_t)(r == 0 ? 256 : (r == 1 ? 384 : 448)); };
    // the item's tile and its number of key steps (0: nothing visible, or rows beyond Sq)
    auto item_steps = [&](int linear, int& q0, int& h, int& b, int& kvlen) {
        int rank;
        sched_item(grid, linear, rank, h, b);
        q0 = (grid.nblk - 1 - rank) * kTile;           // heavy (late) causal blocks first
        kvlen = a.Sk;
        if (a.kv_len) kvlen = min(max(a.kv_len[b], 0), a.Sk);
        int lim = 0;
        if (q0 < a.Sq) {
            lim = kvlen;
            if (a.causal) lim = min(lim, min(q0 + kTile - 1, a.Sq - 1) + a.causal_off + 1);
        }
        return lim > 0 ? (lim + kKStep - 1) / kKStep : 0;
    };
    LTCA_TRACE_DECL(LTCA_TRACE_KERNEL == 3 && blockIdx.x == 5);
    LTCA_TRACE_EVT(0x01);

    if (warp >= 16) {
      reg_dealloc<kCtrlRegs>();
      if (warp == kTmaWarp) {
        if (lane == 0) {
            int g = 0, na = 0;
            bool ok = true;
            for (int nq = 0; ok; ++nq) {
                const int linear = iq.produce(nq, grid.counters, grid.n_items, wc);
                if (linear < 0) break;
                int q0, h, b, kvlen;
                const int n_it = item_steps(linear, q0, h, b, kvlen);
                if (n_it == 0) continue;
                const int r = na & 1;
                ok = mbar_wait(bar_res_empty(r), (uint32_t)(((na >> 1) & 1) ^ 1), wc, 0xd1);
                if (!ok) break;
                mbar_arrive_expect_tx(bar_res_full(r), 2u * kBigTile);
                tma_load_4d(res_smem + r * 2 * kBigTile, &tmap_q, bar_res_full(r), 0, q0, h, b);
                tma_load_4d(res_smem + r * 2 * kBigTile + kBigTile, &tmap_do, bar_res_full(r), 0, q0, h, b);
                for (int it = 0; it < n_it && ok; ++it, ++g) {
                    ok = mbar_wait(bar_ring_empty(slot_of(g)), phase_of(g) ^ 1u, wc, 0xd0);
                    if (!ok) break;
                    const uint32_t st = ring_smem + slot_of(g) * L::kStageBytes;
                    const uint32_t bar = bar_ring_full(slot_of(g));
                    mbar_arrive_expect_tx(bar, 2u * kBigTile);
                    tma_load_4d(st, &tmap_k, bar, 0, it * kKStep, h, b);
                    tma_load_4d(st + kBigTile, &tmap_v, bar, 0, it * kKStep, h, b);
                }
                ++na;
            }
        }
      } else if (warp == kMmaWarp0) {
        // S = Q K_j^T and dP = dO V_j^T, one step ahead of the elementwise warps
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc_bf16(kTile, kKStep, 0, 0);
            const uint64_t res_desc = make_smem_desc_sw128(res_smem, 16, 1024);
            const uint64_t ring_desc = make_smem_desc_sw128(ring_smem, 16, 1024);
            int g = 0, na = 0;
            bool ok = true;
            for (int nq = 0; ok; ++nq) {
                const int linear = iq.consume(nq, wc);
                if (linear < 0) break;
                int q0, h, b, kvlen;
                const int n_it = item_steps(linear, q0, h, b, kvlen);
                if (n_it == 0) continue;
                const int r = na & 1;
                ok = mbar_wait(bar_res_full(r), (uint32_t)((na >> 1) & 1), wc, 0xe0);
                const uint64_t q_desc = res_desc + (uint64_t)((r * 2 * kBigTile) >> 4);
                const uint64_t do_desc = q_desc + (uint64_t)(kBigTile >> 4);
                for (int it = 0; it < n_it && ok; ++it, ++g) {
                    ok = mbar_wait(bar_ring_full(slot_of(g)), phase_of(g), wc, 0xe2);
                    // S and dP of the previous step (of this or of the previous item) are in registers
                    if (g >= 1) ok = ok && mbar_wait(bar_sdp_free, (uint32_t)((g - 1) & 1), wc, 0xe3);
                    // dS lives in three buffers; step g reuses the one dQ(g-3) read.  Waiting for
                    // that contraction here keeps the check off the elementwise warps' path.
                    if (g >= 3) ok = ok && mbar_wait(bar_ds_free(g - 3), ds_parity(g - 3), wc, 0xe5);
                    if (!ok) break;
                    tc_fence_after_sync();
                    LTCA_TRACE_EVT(0x20 + (g << 8));
                    const uint64_t kd = ring_desc + (uint64_t)((slot_of(g) * L::kStageBytes) >> 4);
                    const uint64_t vd = kd + (uint64_t)(kBigTile >> 4);
#pragma unroll
                    for (int k = 0; k < kD / 16; ++k) mma_ss(tmem_base, q_desc + 2 * k, kd + 2 * k, idesc_s, k > 0);
#pragma unroll
                    for (int k = 0; k < kD / 16; ++k)
                        mma_ss(tmem_base + 128, do_desc + 2 * k, vd + 2 * k, idesc_s, k > 0);
                    mma_commit(bar_sdp_full);
                    mma_commit(bar_ring_empty(slot_of(g)));
                    LTCA_TRACE_EVT(0x21 + (g << 8));
                }
                if (ok) mma_commit(bar_res_empty(r));      // Q and dO of this item are no longer read
                ++na;
            }
            // all of this thread's contractions are complete once the last S / dP has been consumed
            if (ok && g > 0) ok = mbar_wait(bar_sdp_free, (uint32_t)((g - 1) & 1), wc, 0xe4);
        }
      } else if (warp == kMmaWarp0 + 1) {
        // dQ += dS K_j   (dS from tensor memory, K_j rows as the contraction index)
        if (lane == 0) {
            constexpr uint32_t idesc_dq = make_idesc_bf16(kTile, kD, 0, 1);
            const uint64_t ring_desc_mn = make_smem_desc_sw128(ring_smem, 8192, 1024);
            int g = 0, na = 0;
            bool ok = true;
            for (int nq = 0; ok; ++nq) {
                const int linear = iq.consume(nq, wc);
                if (linear < 0) break;
                int q0, h, b, kvlen;
                const int n_it = item_steps(linear, q0, h, b, kvlen);
                if (n_it == 0) continue;
                for (int it = 0; it < n_it && ok; ++it, ++g) {
                    ok = mbar_wait(bar_ring_full(slot_of(g)), phase_of(g), wc, 0xe8);
                    ok = ok && mbar_wait(bar_ds_full(g), ds_parity(g), wc, 0xe9);
                    // the previous item's dQ must have left tensor memory before it is overwritten
                    if (it == 0 && na > 0) ok = ok && mbar_wait(bar_acc_free, (uint32_t)((na - 1) & 1), wc, 0xeb);
                    if (!ok) break;
                    tc_fence_after_sync();
                    LTCA_TRACE_EVT(0x22 + (g << 8));
                    const uint64_t kd = ring_desc_mn + (uint64_t)((slot_of(g) * L::kStageBytes) >> 4);
#pragma unroll
                    for (int k = 0; k < kKStep / 16; ++k)
                        mma_ts(tmem_base + 320, tmem_base + ds_col(g) + k * 8, kd + 128 * k, idesc_dq,
                               (it > 0 || k > 0) ? 1u : 0u);
                    mma_commit(bar_ds_free(g));
                    mma_commit(bar_ring_empty(slot_of(g)));
                    LTCA_TRACE_EVT(0x23 + (g << 8));
                }
                ++na;
            }
            if (ok && g > 0) ok = mbar_wait(bar_ds_free(g - 1), ds_parity(g - 1), wc, 0xea);
        }
      } else {
        // warp 19: stores each item's dQ tile (staged by the elementwise warps in the item's Q buffer,
        // 128-byte swizzle) with TMA and hands the buffer back to the producer.  Rows past the end of
        // the queries are clipped by the tensor map.
        if (lane == 0) {
            int na = 0;
            bool ok = true;
            for (int nq = 0; ok; ++nq) {
                const int linear = iq.consume(nq, wc);
                if (linear < 0) break;
                int q0, h, b, kvlen;
                const int n_it = item_steps(linear, q0, h, b, kvlen);
                if (n_it == 0) continue;
                const int r = na & 1;
                ok = mbar_wait(bar_staged(r), (uint32_t)((na >> 1) & 1), wc, 0xd9);
                if (ok) {
                    tma_store_4d(&tmap_dq, res_smem + r * 2 * kBigTile, 0, q0, h, b);
                    tma_store_commit();
                    tma_store_wait_read<0>();
                }
                mbar_arrive(bar_res_empty(r));
                ++na;
            }
        }
      }
    } else {
        reg_alloc<kMathRegs>();
        const int wq = warp & 3, cq = warp >> 2;
        const int row = wq * 32 + lane;
        const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
        const uint32_t tS = tmem_base + lane_base + 32 * cq;
        const uint32_t tDP = tS + 128;
        const uint32_t tDQ = tmem_base + lane_base + 320 + 16 * cq;
        const float c2 = a.scale_log2;
        const bool general = (a.keep_mask != nullptr) || (a.use_clamp != 0);

        int g = 0, na = 0;
        bool ok = true;
        for (int nq = 0; ok; ++nq) {
            const int linear = iq.consume_warp(nq, wc);
            if (linear < 0) break;
            int q0, h, b, kvlen;
            const int n_it = item_steps(linear, q0, h, b, kvlen);
            const int qi = q0 + row;
            __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(a.dq) + b * a.dqs.batch + h * a.dqs.head +
                                  (int64_t)qi * a.dqs.seq + cq * 16;
            if (n_it == 0) {
                if (qi < a.Sq) {                       // nothing visible: the gradient is zero
                    uint32_t z[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c) z[c] = 0u;
                    store_row16_bf16(drow, z, 0.f);
                }
                continue;
            }
            const int64_t srow = ((int64_t)b * a.H + h) * a.Sq_pad + qi;      // qi < Sq_pad by construction
            const float lse2 = a.lse2[srow];
            const float dlt = a.delta[srow];

            uint32_t s[32], dp[32];
            ok = mbar_wait_warp(bar_sdp_full, (uint32_t)(g & 1), wc, 0xf0);
            if (!ok) break;
            tc_fence_after_sync();
            tmem_ld32(tS, s);
            tmem_ld32(tDP, dp);
            tmem_wait_ld();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sdp_free);

            for (int it = 0; it < n_it && ok; ++it, ++g) {
                LTCA_TRACE_EVT(0x11 + (g << 8));
                const int k0 = it * kKStep;
                const bool edge = (k0 + kKStep > kvlen) || (a.causal && (k0 + kKStep - 1 > q0 + a.causal_off));
                // dS = P o (dP - delta), left in dp[]; the masked variant only runs on edge steps
                if (general) {
                    int vis_lim = kvlen;
                    if (a.causal) vis_lim = min(vis_lim, qi + a.causal_off + 1);
                    vis_lim -= k0 + cq * 32;
                    const float* mrow = nullptr;
                    if (a.keep_mask && qi < a.Sq)
                        mrow = a.keep_mask + ((int64_t)b * a.Sq + qi) * a.Sk + k0 + cq * 32;
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const float sv = __uint_as_float(s[c]);
                        const float p = fast_exp2(fmaf(sv, c2, -lse2));
                        float d = p * (__uint_as_float(dp[c]) - dlt);
                        bool vis = c < vis_lim;
                        if (mrow && vis) vis = (__ldg(mrow + c) != 0.0f);
                        if (a.use_clamp && sv >= a.clamp_raw) d = 0.f;
                        dp[c] = __float_as_uint(vis ? d : 0.f);
                    }
                } else if (edge) {
                    // causal diagonal or end of the keys, no dense mask: selects only, no branches
                    int vis_lim = kvlen;
                    if (a.causal) vis_lim = min(vis_lim, qi + a.causal_off + 1);
                    vis_lim -= k0 + cq * 32;
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const float p = fast_exp2(fmaf(__uint_as_float(s[c]), c2, -lse2));
                        dp[c] = __float_as_uint((c < vis_lim) ? p * (__uint_as_float(dp[c]) - dlt) : 0.f);
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const float p = fast_exp2(fmaf(__uint_as_float(s[c]), c2, -lse2));
                        dp[c] = __float_as_uint(p * (__uint_as_float(dp[c]) - dlt));
                    }
                }
                uint32_t hi[16], unused[16];
                pack32<false>(dp, hi, unused);
                LTCA_TRACE_EVT(0x12 + (g << 8));
                // The next step's S and dP are requested now, so that their tensor-memory load runs
                // while this step's dS is stored and announced.  (No wait for dQ here: the dS buffer
                // written below was released before S and dP of this step were even issued.)
                const bool more = it + 1 < n_it;
                if (more) {
                    ok = mbar_wait_warp(bar_sdp_full, (uint32_t)((g + 1) & 1), wc, 0xf0);
                    if (!ok) break;
                    tc_fence_after_sync();
                    tmem_ld32(tS, s);
                    tmem_ld32(tDP, dp);
                }
                LTCA_TRACE_EVT(0x14 + (g << 8));
                tmem_st16(tmem_base + lane_base + ds_col(g) + 16 * cq, hi);
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_ds_full(g));
                if (more) {
                    tmem_wait_ld();
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_sdp_free);
                }
                LTCA_TRACE_EVT(0x13 + (g << 8));
            }
            if (!ok) break;
            // item epilogue: dQ out of tensor memory, which is then free for the next item
            ok = mbar_wait_warp(bar_ds_free(g - 1), ds_parity(g - 1), wc, 0xf2);
            if (!ok) break;
            tc_fence_after_sync();
            uint32_t o[16];
            tmem_ld16(tDQ, o);
            tmem_wait_ld();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_free);
            {
                // this thread's 16 columns of dQ (scaled), bf16, into the item's Q buffer in the layout of a
                // 128-byte-swizzled TMA box; warp 19 stores the tile
                const int r = na & 1;
                ++na;
                uint8_t* st_q = smem_gen + L::kResOff + r * 2 * kBigTile + row * 128;
#pragma unroll
                for (int v = 0; v < 2; ++v) {
                    uint4 w;
                    w.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]) * a.scale, __uint_as_float(o[8 * v + 1]) * a.scale);
                    w.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]) * a.scale, __uint_as_float(o[8 * v + 3]) * a.scale);
                    w.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]) * a.scale, __uint_as_float(o[8 * v + 5]) * a.scale);
                    w.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]) * a.scale, __uint_as_float(o[8 * v + 7]) * a.scale);
                    *reinterpret_cast<uint4*>(st_q + (((2 * cq + v) ^ (row & 7)) << 4)) = w;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_staged(r));
            }
        }
    }

    // Out of work: only now may the kernel after this one place its CTAs (released at the start, its blocks would
    // sit beside this kernel's CTAs for the whole run, waiting for it to end).
    grid_launch_dependents();
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) item_counters_release(grid.counters);
    if (warp == kMmaWarp0) {
        __syncwarp();
        if (misc[1]) __nanosleep(200000);
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace

#ifdef LTCA_TRACE
extern "C" int ltca_trace_read_bwd(unsigned long long* events, unsigned int* counts) {
    if (cudaMemcpyFromSymbol(events, g_trace, sizeof(g_trace)) != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(counts, g_trace_count, sizeof(g_trace_count)) != cudaSuccess) return -1;
    return 0;
}
#endif

namespace {

size_t stats_bytes(const ltca_attn_params* p) {
    const size_t sq_pad = align_up((size_t)p->Sq, 256);
    return align_up((size_t)p->B * p->H * sq_pad * sizeof(float), 256);
}

size_t dq_acc_bytes(const ltca_attn_params* p) {
    const size_t sq_pad = align_up((size_t)p->Sq, 256);
    return align_up((size_t)p->B * p->H * sq_pad * kD * sizeof(float), 256);
}

// The fused kernel serves bf16 storage unless the caller asks for bit-reproducible dQ.  (At 512 queries and fewer
// the two paths are within 5 % of each other, in the fused kernel's favour when the inputs come from HBM.)
bool use_fused(const ltca_attn_params* p) { return p->dtype == LTCA_BF16 && !p->bwd_deterministic; }

template <typename OutT>
int launch_main(ltca_ctx* ctx, const ltca_attn_params* p, const void* q, const void* k, const void* v,
                const void* dout, const ltca_strides& qs, const ltca_strides& ks, const ltca_strides& vs,
                const ltca_strides& dos, const float* lse2, const float* delta, float* dq_acc) {
    CUtensorMap tq128, tdo128, tk64, tv64, tq64, tdo64, tk128, tv128;
    int rc;
    if ((rc = make_tmap_bhsd(ctx, &tq128, q, 2, p->B, p->H, p->Sq, kD, qs, 64, kTile))) return rc;
    if ((rc = make_tmap_bhsd(ctx, &tdo128, dout, 2, p->B, p->H, p->Sq, kD, dos, 64, kTile))) return rc;
    if ((rc = make_tmap_bhsd(ctx, &tk64, k, 2, p->B, p->H, p->Sk, kD, ks, 64, kStep))) return rc;
    if ((rc = make_tmap_bhsd(ctx, &tv64, v, 2, p->B, p->H, p->Sk, kD, vs, 64, kStep))) return rc;
    if ((rc = make_tmap_bhsd(ctx, &tq64, q, 2, p->B, p->H, p->Sq, kD, qs, 64, kStep))) return rc;
    if ((rc = make_tmap_bhsd(ctx, &tdo64, dout, 2, p->B, p->H, p->Sq, kD, dos, 64, kStep))) return rc;
    if ((rc = make_tmap_bhsd(ctx, &tk128, k, 2, p->B, p->H, p->Sk, kD, ks, 64, kTile))) return rc;
    if ((rc = make_tmap_bhsd(ctx, &tv128, v, 2, p->B, p->H, p->Sk, kD, vs, 64, kTile))) return rc;

    BwdArgs a;
    memset(&a, 0, sizeof(a));
    a.B = p->B; a.H = p->H; a.Sq = p->Sq; a.Sk = p->Sk;
    a.Sq_pad = (int)align_up((size_t)p->Sq, 256);
    a.causal = p->causal ? 1 : 0;
    a.causal_off = p->Sk - p->Sq;
    a.scale = p->scale;
    a.scale_log2 = p->scale * 1.4426950408889634f;
    a.use_clamp = p->score_clamp > 0.f ? 1 : 0;
    a.clamp_raw = a.use_clamp ? p->score_clamp / p->scale : __builtin_inff();
    a.clamp_log2 = p->score_clamp * 1.4426950408889634f;
    a.lse2 = lse2; a.delta = delta;
    a.dq = p->dq; a.dk = p->dk; a.dv = p->dv;
    a.dqs = p->dq_strides; a.dks = p->dk_strides; a.dvs = p->dv_strides;
    a.keep_mask = p->keep_mask;
    a.kv_len = p->kv_len;
    a.status = ctx->d_status;

    if constexpr (sizeof(OutT) == 2) {
        if (dq_acc) {
            static SmemOptIn opt_fused;
            LTCA_CUDA_OK(ctx, opt_in_dynamic_smem(opt_fused, ctx->device, attn_bwd_fused_sm100_kernel,
                                                  FusedSmem::kDynBytes));
            ItemGrid ig;
            ig.nblk = (p->Sk + kTile - 1) / kTile;
            ig.H = p->H;
            ig.BH = p->H * p->B;
            ig.n_items = ig.nblk * ig.BH;
            ig.counters = ctx->d_sched + 4;             // ints 4,5: shared with the dK/dV kernel (never both in one call)
            const int n_cta = ig.n_items < ctx->sm_count ? ig.n_items : ctx->sm_count;
            CUtensorMap tdk, tdv, tacc;
            if ((rc = make_tmap_bhsd(ctx, &tdk, p->dk, 2, p->B, p->H, p->Sk, kD, p->dk_strides, 64, kTile))) return rc;
            if ((rc = make_tmap_bhsd(ctx, &tdv, p->dv, 2, p->B, p->H, p->Sk, kD, p->dv_strides, 64, kTile))) return rc;
            const ltca_strides accs{(int64_t)p->H * a.Sq_pad * kD, (int64_t)a.Sq_pad * kD, kD};
            if ((rc = make_tmap_bhsd(ctx, &tacc, dq_acc, 4, p->B, p->H, a.Sq_pad, kD, accs, 32, kTile))) return rc;
            LTCA_CUDA_OK(ctx, launch_dependent_if(small_attention_call(p), attn_bwd_fused_sm100_kernel, dim3(n_cta), dim3(kThreads), FusedSmem::kDynBytes,
                                               ctx->stream, tq128, tdo128, tk128, tv128, tdk, tdv, tacc, a, ig));
            LTCA_LAUNCH_OK(ctx, "attn_bwd_fused_sm100_kernel");
            kernel_timing_mark(ctx, 2);
            const int64_t rows = (int64_t)p->B * p->H * p->Sq;
            LTCA_CUDA_OK(ctx, launch_dependent_if(small_attention_call(p), attn_bwd_dq_convert_kernel, dim3((unsigned)((rows + 31) / 32)), dim3(256), 0,
                                               ctx->stream, (const float*)dq_acc, p->dq, p->dq_strides, p->B, p->H, p->Sq,
                                               a.Sq_pad, p->scale));
            LTCA_LAUNCH_OK(ctx, "attn_bwd_dq_convert_kernel");
            kernel_timing_mark(ctx, 3);
            return LTCA_OK;
        }
    }
    auto kdq = attn_bwd_dq_sm100_kernel<OutT, sizeof(OutT) == 4>;
    auto kdkv = attn_bwd_dkv_sm100_kernel<OutT, sizeof(OutT) == 4>;
    static SmemOptIn opt_dq, opt_dkv;         // one pair per template instantiation
    LTCA_CUDA_OK(ctx, opt_in_dynamic_smem(opt_dq, ctx->device, kdq, DqSmem::kDynBytes));
    LTCA_CUDA_OK(ctx, opt_in_dynamic_smem(opt_dkv, ctx->device, kdkv, DkvSmem::kDynBytes));
    bool dq_launched = false;
    if constexpr (sizeof(OutT) == 2) {
        {
            static SmemOptIn opt_dq4;
            LTCA_CUDA_OK(ctx, opt_in_dynamic_smem(opt_dq4, ctx->device, attn_bwd_dq4_sm100_kernel, Dq4Smem::kDynBytes));
            ItemGrid ig;
            ig.nblk = (p->Sq + kTile - 1) / kTile;
            ig.H = p->H;
            ig.BH = p->H * p->B;
            ig.n_items = ig.nblk * ig.BH;
            ig.counters = ctx->d_sched + 2;             // ints 2,3: the dQ kernel's item counters
            const int n_cta = ig.n_items < ctx->sm_count ? ig.n_items : ctx->sm_count;
            CUtensorMap tdq;
            if ((rc = make_tmap_bhsd(ctx, &tdq, p->dq, 2, p->B, p->H, p->Sq, kD, p->dq_strides, 64, kTile))) return rc;
            LTCA_CUDA_OK(ctx, launch_dependent_if(small_attention_call(p), attn_bwd_dq4_sm100_kernel, dim3(n_cta), dim3(kThreads), Dq4Smem::kDynBytes,
                                               ctx->stream, tq128, tdo128, tk128, tv128, tdq, a, ig));
            LTCA_LAUNCH_OK(ctx, "attn_bwd_dq4_sm100_kernel");
            dq_launched = true;
        }
    }
    if (!dq_launched) {
        dim3 gq((p->Sq + 2 * kTile - 1) / (2 * kTile), p->H, p->B);
        LTCA_CUDA_OK(ctx, launch_dependent_if(small_attention_call(p), kdq, gq, dim3(kThreads), DqSmem::kDynBytes, ctx->stream, tq128, tdo128, tk64, tv64, a));
        LTCA_LAUNCH_OK(ctx, "attn_bwd_dq_sm100_kernel");
    }
    kernel_timing_mark(ctx, 2);
    if constexpr (sizeof(OutT) == 2) {
        {
            static SmemOptIn opt_dkv4;
            LTCA_CUDA_OK(ctx, opt_in_dynamic_smem(opt_dkv4, ctx->device, attn_bwd_dkv4_sm100_kernel,
                                                  Dkv4Smem::kDynBytes));
            ItemGrid ig;
            ig.nblk = (p->Sk + kTile - 1) / kTile;
            ig.H = p->H;
            ig.BH = p->H * p->B;
            ig.n_items = ig.nblk * ig.BH;
            ig.counters = ctx->d_sched + 4;             // ints 4,5: the dK/dV kernel's item counters
            const int n_cta = ig.n_items < ctx->sm_count ? ig.n_items : ctx->sm_count;
            CUtensorMap tdk, tdv;
            if ((rc = make_tmap_bhsd(ctx, &tdk, p->dk, 2, p->B, p->H, p->Sk, kD, p->dk_strides, 64, kTile))) return rc;
            if ((rc = make_tmap_bhsd(ctx, &tdv, p->dv, 2, p->B, p->H, p->Sk, kD, p->dv_strides, 64, kTile))) return rc;
            LTCA_CUDA_OK(ctx, launch_dependent_if(small_attention_call(p), attn_bwd_dkv4_sm100_kernel, dim3(n_cta), dim3(kThreads), Dkv4Smem::kDynBytes,
                                               ctx->stream, tq128, tdo128, tk128, tv128, tdk, tdv, a, ig));
            LTCA_LAUNCH_OK(ctx, "attn_bwd_dkv4_sm100_kernel");
            kernel_timing_mark(ctx, 3);
            return LTCA_OK;
        }
    }
    dim3 gk((p->Sk + 2 * kTile - 1) / (2 * kTile), p->H, p->B);
    LTCA_CUDA_OK(ctx, launch_dependent_if(small_attention_call(p), kdkv, gk, dim3(kThreads), DkvSmem::kDynBytes, ctx->stream, tq64, tdo64, tk128, tv128, a));
    LTCA_LAUNCH_OK(ctx, "attn_bwd_dkv_sm100_kernel");
    kernel_timing_mark(ctx, 3);
    return LTCA_OK;
}

}  // namespace

bool attn_bwd_sm100_supported(const ltca_attn_params* p) {
    if (p->D != 64) return false;
    if (p->Sq < 1 || p->Sk < 1 || !(p->scale > 0.f)) return false;
    if (p->H > 65535 || p->B > 65535) return false;
    return true;
}

size_t attn_bwd_sm100_workspace(const ltca_attn_params* p) {
    return 2 * stats_bytes(p) + (use_fused(p) ? dq_acc_bytes(p) : 0);
}

int launch_attn_bwd_sm100(ltca_ctx* ctx, const ltca_attn_params* p) {
    size_t need = attn_bwd_sm100_workspace(p);
    const size_t pq = align_up((size_t)p->B * p->H * p->Sq * kD * 2, 256);
    const size_t pk = align_up((size_t)p->B * p->H * p->Sk * kD * 2, 256);
    if (p->dtype == LTCA_F32) need += 2 * pq + 2 * pk;
    if (!p->workspace || p->workspace_bytes < need)
        return fail(ctx, LTCA_ERR_WORKSPACE, "tensor-pipe backward needs %zu bytes of workspace", need);
    const int es = elem_size(p->dtype);
    auto bad16 = [&](const void* ptr, const ltca_strides& s) {
        return (reinterpret_cast<uintptr_t>(ptr) & 15) || ((s.seq * es) & 15) || ((s.head * es) & 15) ||
               ((s.batch * es) & 15);
    };
    if (bad16(p->o, p->o_strides) || bad16(p->dout, p->do_strides) || bad16(p->dq, p->dq_strides) ||
        bad16(p->dk, p->dk_strides) || bad16(p->dv, p->dv_strides))
        return fail(ctx, LTCA_ERR_INVALID, "o, dout, dq, dk, dv need 16-byte aligned bases and strides");

    char* w = reinterpret_cast<char*>(p->workspace);
    float* lse2 = reinterpret_cast<float*>(w);  w += stats_bytes(p);
    float* delta = reinterpret_cast<float*>(w); w += stats_bytes(p);
    float* dq_acc = nullptr;
    if (use_fused(p)) { dq_acc = reinterpret_cast<float*>(w); w += dq_acc_bytes(p); }

    StatsArgs s;
    s.B = p->B; s.H = p->H; s.Sq = p->Sq; s.Sq_pad = (int)align_up((size_t)p->Sq, 256);
    s.o = p->o; s.dout = p->dout; s.os = p->o_strides; s.dos = p->do_strides;
    s.lse = p->lse; s.lse2 = lse2; s.delta = delta; s.dq_acc = dq_acc;
    const int64_t rows = (int64_t)p->B * p->H * s.Sq_pad;
    const unsigned blocks = (unsigned)((rows + 31) / 32);
    kernel_timing_mark(ctx, 0);
    if (p->dtype == LTCA_BF16)
        LTCA_CUDA_OK(ctx, launch_dependent_if(small_attention_call(p), attn_bwd_stats_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, ctx->stream, s));
    else
        LTCA_CUDA_OK(ctx, launch_dependent_if(small_attention_call(p), attn_bwd_stats_kernel<float>, dim3(blocks), dim3(256), 0, ctx->stream, s));
    LTCA_LAUNCH_OK(ctx, "attn_bwd_stats_kernel");
    if (p->dtype == LTCA_BF16) kernel_timing_mark(ctx, 1);

    if (p->dtype == LTCA_BF16)
        return launch_main<__nv_bfloat16>(ctx, p, p->q, p->k, p->v, p->dout, p->q_strides, p->k_strides,
                                          p->v_strides, p->do_strides, lse2, delta, dq_acc);

    // fp32 storage: bf16 copies of the four operands, fp32 gradients out
    void* qb = w;  w += pq;
    void* kb = w;  w += pk;
    void* vb = w;  w += pk;
    void* gb = w;
    const PackJob jobs[4] = {{p->q, p->q_strides, qb, p->Sq}, {p->k, p->k_strides, kb, p->Sk},
                             {p->v, p->v_strides, vb, p->Sk}, {p->dout, p->do_strides, gb, p->Sq}};
    if (int rc = pack_many_to_bf16(ctx, jobs, 4, p->B, p->H, kD)) return rc;
    kernel_timing_mark(ctx, 1);
    ltca_strides cq{(int64_t)p->H * p->Sq * kD, (int64_t)p->Sq * kD, kD};
    ltca_strides ck{(int64_t)p->H * p->Sk * kD, (int64_t)p->Sk * kD, kD};
    return launch_main<float>(ctx, p, qb, kb, vb, gb, cq, ck, ck, cq, lse2, delta, nullptr);
}

}  // namespace ltca
