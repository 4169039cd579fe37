// Attention forward on the sm_100a tensor pipe.
//
//   O = softmax(mask(scale * Q K^T)) V,   lse = log sum exp of the masked, scaled scores
//
// replaces flashAttentionKernel of the reference (src/ml/flash_attention.cu:18-272): the same
// contract (scale, keep-mask with 0 = hidden, optional score clamp), plus a causal flag and
// per-sequence key lengths, computed as a true online softmax.
//
// Shape of the kernel
//   - one CTA per (256 query rows, head, batch): two 128-row query tiles share every K/V tile
//     that TMA brings in, which halves the L2 -> shared traffic per FLOP;
//   - 16 softmax warps: a query row belongs to TWO threads, each owning half of the step's key
//     columns (warps w and w + 8 read the same 32 tensor-memory lanes), so that every scheduler
//     holds four softmax warps and the special-function unit stays busy while other warps load,
//     reduce or wait.  The two threads of a row agree on the row maximum through shared memory;
//     row sums stay private until the epilogue.  Warps 0-3 / 8-11: tile 0, 4-7 / 12-15: tile 1;
//   - warps 16 / 17 issue the tcgen05.mma of tile 0 / 1 (one thread each), warp 18 is the TMA
//     producer.  The control warps give registers up for the softmax warps (setmaxnreg);
//   - S = Q K^T accumulates in tensor memory; the softmax warps read it with tcgen05.ld and
//     release it at once, so the next step's S is computed while this step's exponentials
//     run; P goes back to its OWN tensor-memory columns as packed bf16 (tcgen05.st) and the
//     second contraction O += P V takes it from there; O never leaves tensor memory until the
//     epilogue;
//   - K and V tiles travel through one ring of shared-memory slots in the order
//     K0 V0 K1 V1 ..., each slot guarded by a full/empty mbarrier pair.
//
// Keys per step (kBN): 128 for head_dim 64 with a bf16 result, else 64 (head_dim 128, or the
// split-P variant below), chosen so that everything fits the 512 tensor-memory columns:
//   S0 S1 (kBN each) | O0 O1 (D each) | P0 P1 (kBN/2 each) | split-P only: Plo0 Plo1 (kBN/2 each)
#include "host_common.h"
#include "sm100_ptx.cuh"
#include "trace.cuh"


namespace ltca {

namespace {

constexpr int kBlockM = 128;        // query rows per tile
constexpr int kFwd4MinSq = 256;     // queries above which the four-tile persistent kernel is used
// Two threads share one query row (each owns half of the step's key columns): 16 softmax warps, four per
// scheduler, row maxima exchanged through shared memory.  (One thread per row, 8 warps, hid no latency.)
constexpr int kRowSplit = 2;
constexpr int kMathWarps = 8 * kRowSplit;
constexpr int kFwdThreads = 32 * (kMathWarps + 4);   // + one warpgroup of control warps
constexpr int kMmaWarp0 = kMathWarps;                // issues the contractions of tile 0 (tile 1: the next warp)
constexpr int kTmaWarp = kMathWarps + 2;
constexpr int kLaunchRegs = 96;     // registers per thread at launch (65536 / threads, rounded down to 8)
constexpr int kCtrlRegs = 32;
constexpr int kMathRegs = 112;
// setmaxnreg can only redistribute what the CTA was launched with; asking for more never returns
static_assert(32 * kMathWarps * kMathRegs + 128 * kCtrlRegs <= kFwdThreads * kLaunchRegs, "register budget");
constexpr uint32_t kTmemCols = 512;

struct FwdArgs {
    int B, H, Sq, Sk;
    int causal, causal_off;
    float scale;            // score scale
    float scale_log2;       // scale * log2(e)
    float clamp_raw;        // score clamp divided by scale (raw QK^T units); +inf when unused
    int use_clamp;
    void* o;
    int64_t o_sb, o_sh, o_ss;
    float* lse;
    const float* keep_mask;
    const int32_t* kv_len;
    uint32_t* status;
};

template <int D, bool kSplitP>
struct FwdCfg {
    static constexpr int kBN = (D == 64 && !kSplitP) ? 128 : 64;   // keys per step
    static constexpr int kDimBlocks = D / 64;                      // 64-element (128 B) column blocks
    static constexpr int kQTileBytes = kBlockM * D * 2;
    static constexpr int kKvTileBytes = kBN * D * 2;
    static constexpr int kStages = 8;                              // ring slots
    // tensor-memory columns
    static constexpr int kColS = 0;
    static constexpr int kColO = 2 * kBN;
    static constexpr int kColP = kColO + 2 * D;
    static constexpr int kColPlo = kColP + kBN;
    static_assert(kColPlo + (kSplitP ? kBN : 0) <= 512, "tensor memory overflow");
    // shared memory
    static constexpr int kQOff = 0;
    static constexpr int kRingOff = 2 * kQTileBytes;
    static constexpr int kXchgOff = kRingOff + kStages * kKvTileBytes;   // float [3][2 tiles][2 halves][128]
    static constexpr int kBarOff = kXchgOff + 3 * 2 * 2 * kBlockM * 4;
    // barriers: q_full, kv_full[kStages], kv_empty[kStages], s_full[2], s_free[2], p_full[2], o_done[2],
    // pair[8] (one per pair of warps that share rows), turn[2]
    static constexpr int kNumBars = 1 + 2 * kStages + 8 + 8 + 2;
    static constexpr int kMiscOff = kBarOff + kNumBars * 8;        // tmem base, abort flag
    static constexpr int kBytes = kMiscOff + 16;
    static constexpr int kDynBytes = kBytes + 1024;                // room to align to 1024 B
};

__device__ __forceinline__ float neg_inf() { return __int_as_float(0xff800000); }

// kSplitP: P is written as two bf16 terms (p = hi + lo, 16 mantissa bits in total) and the
// second contraction runs once per term; used when the output is stored as fp32, where the
// 2^-9 rounding of a single bf16 P would be the largest error left.
template <int D, typename OutT, bool kSplitP>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q,
                      const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const FwdArgs a) {
    using L = FwdCfg<D, kSplitP>;
    constexpr int kBN = L::kBN;
    constexpr int kH = kBN / kRowSplit;  // key columns per thread and step
    constexpr int kDH = D / kRowSplit;   // output columns per thread
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t q_smem = smem_base + L::kQOff;
    const uint32_t ring_smem = smem_base + L::kRingOff;
    const uint32_t bar_base = smem_base + L::kBarOff;
    auto bar_q_full = [&]() { return bar_base; };
    auto bar_kv_full = [&](int s) { return bar_base + 8u * (1 + s); };
    auto bar_kv_empty = [&](int s) { return bar_base + 8u * (1 + L::kStages + s); };
    auto bar_s_full = [&](int t) { return bar_base + 8u * (1 + 2 * L::kStages + t); };
    auto bar_s_free = [&](int t) { return bar_base + 8u * (3 + 2 * L::kStages + t); };
    auto bar_p_full = [&](int t) { return bar_base + 8u * (5 + 2 * L::kStages + t); };
    auto bar_o_done = [&](int t) { return bar_base + 8u * (7 + 2 * L::kStages + t); };
    auto bar_pair = [&](int t, int wq) { return bar_base + 8u * (9 + 2 * L::kStages + t * 4 + wq); };
    auto bar_turn = [&](int t) { return bar_base + 8u * (17 + 2 * L::kStages + t); };
    float* xchg = reinterpret_cast<float*>(smem_gen + L::kXchgOff);
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);
    // misc[0] = tensor-memory base address, misc[1] = abort flag

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int m_block = gridDim.x - 1 - blockIdx.x;     // heavy (late) causal blocks first
    const int h = blockIdx.y;
    const int b = blockIdx.z;

    int kvlen = a.Sk;
    if (a.kv_len) {
        grid_dependency_wait();                // the lengths may come from the kernel before this one
        kvlen = min(max(a.kv_len[b], 0), a.Sk);
    }
    int n_tiles[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int q0 = m_block * 2 * kBlockM + t * kBlockM;
        int lim = 0;
        if (q0 < a.Sq) {
            lim = kvlen;
            if (a.causal) lim = min(lim, min(q0 + kBlockM - 1, a.Sq - 1) + a.causal_off + 1);
        }
        n_tiles[t] = lim > 0 ? (lim + kBN - 1) / kBN : 0;
    }
    const int n_max = max(n_tiles[0], n_tiles[1]);

    if (threadIdx.x == 0) {
        mbar_init(bar_q_full(), 1);
        for (int s = 0; s < L::kStages; ++s) {
            mbar_init(bar_kv_full(s), 1);
            mbar_init(bar_kv_empty(s), 2);     // both MMA issuers release a slot
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(bar_s_full(t), 1);
            mbar_init(bar_s_free(t), 4 * kRowSplit);   // one arrival per softmax warp of the tile
            mbar_init(bar_p_full(t), 4 * kRowSplit);
            mbar_init(bar_o_done(t), 1);
            for (int wq = 0; wq < 4; ++wq) mbar_init(bar_pair(t, wq), 2);
            mbar_init(bar_turn(t), 4 * kRowSplit);
        }
        misc[1] = 0u;
        mbar_fence_init();
    }
    if (warp == kMmaWarp0) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(&misc[0])), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = misc[0];
    const WaitCtx wc{&misc[1], a.status};
    LTCA_TRACE_DECL(blockIdx.x == 0 && blockIdx.y == 5 && blockIdx.z == 0);
    LTCA_TRACE_EVT(0x01);
    grid_launch_dependents();                  // (set up: the next kernel may place its CTAs)
    grid_dependency_wait();                    // q, k, v are complete once the kernel before this one has ended

    if (warp >= kMathWarps) {
        reg_dealloc<kCtrlRegs>();
        auto slot_of = [&](int item) { return item % L::kStages; };
        auto phase_of = [&](int item) { return (uint32_t)((item / L::kStages) & 1); };
        if (warp == kTmaWarp) {
            // ------------------------------ TMA producer --------------------------------------
            if (lane == 0 && n_max > 0) {
                tma_prefetch_desc(&tmap_q);
                tma_prefetch_desc(&tmap_k);
                tma_prefetch_desc(&tmap_v);
                mbar_arrive_expect_tx(bar_q_full(), 2u * L::kQTileBytes);
                for (int t = 0; t < 2; ++t)
                    for (int kb = 0; kb < L::kDimBlocks; ++kb)
                        tma_load_4d(q_smem + t * L::kQTileBytes + kb * (kBlockM * 128), &tmap_q,
                                    bar_q_full(), kb * 64, m_block * 2 * kBlockM + t * kBlockM, h, b);
                bool ok = true;
                for (int j = 0; j < n_max && ok; ++j) {
#pragma unroll
                    for (int which = 0; which < 2; ++which) {     // 0: K_j, 1: V_j
                        const int item = 2 * j + which;
                        const int slot = slot_of(item);
                        ok = ok && mbar_wait(bar_kv_empty(slot), phase_of(item) ^ 1u, wc, 0x10 + which);
                        if (!ok) break;
                        mbar_arrive_expect_tx(bar_kv_full(slot), (uint32_t)L::kKvTileBytes);
                        for (int kb = 0; kb < L::kDimBlocks; ++kb)
                            tma_load_4d(ring_smem + slot * L::kKvTileBytes + kb * (kBN * 128),
                                        which == 0 ? &tmap_k : &tmap_v, bar_kv_full(slot), kb * 64,
                                        j * kBN, h, b);
                    }
                }
            }
        } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
            // ------------------------------ MMA issuer of tile t ------------------------------
            const int t = warp - kMmaWarp0;
            if (lane == 0 && n_max > 0) {
                const int n_t = n_tiles[t];
                constexpr uint32_t idesc_qk = make_idesc_bf16(kBlockM, kBN, 0, 0);
                constexpr uint32_t idesc_pv = make_idesc_bf16(kBlockM, D, 0, 1);
                // descriptors are built once; a byte offset inside shared memory adds offset >> 4
                const uint64_t q_desc = make_smem_desc_sw128(q_smem + t * L::kQTileBytes, 16, 1024);
                const uint64_t k_desc = make_smem_desc_sw128(ring_smem, 16, 1024);
                const uint64_t v_desc = make_smem_desc_sw128(ring_smem, kBN * 128, 1024);
                const uint32_t s_tmem = tmem_base + L::kColS + t * kBN;
                const uint32_t o_tmem = tmem_base + L::kColO + t * D;
                const uint32_t p_tmem = tmem_base + L::kColP + t * (kBN / 2);
                const uint32_t plo_tmem = tmem_base + L::kColPlo + t * (kBN / 2);
                auto issue_qk = [&](int slot) {
                    const uint64_t kd = k_desc + (uint64_t)((slot * L::kKvTileBytes) >> 4);
#pragma unroll
                    for (int k = 0; k < D / 16; ++k) {
                        const uint32_t qoff = (k / 4) * (kBlockM * 128) + (k % 4) * 32;
                        const uint32_t koff = (k / 4) * (kBN * 128) + (k % 4) * 32;
                        mma_ss(s_tmem, q_desc + (qoff >> 4), kd + (koff >> 4), idesc_qk, k > 0 ? 1u : 0u);
                    }
                };
                auto issue_pv = [&](int slot, bool acc) {
                    const uint64_t vd = v_desc + (uint64_t)((slot * L::kKvTileBytes) >> 4);
#pragma unroll
                    for (int k = 0; k < kBN / 16; ++k)
                        mma_ts(o_tmem, p_tmem + k * 8, vd + ((k * 2048) >> 4), idesc_pv,
                               (acc || k > 0) ? 1u : 0u);
                    if constexpr (kSplitP) {
#pragma unroll
                        for (int k = 0; k < kBN / 16; ++k)
                            mma_ts(o_tmem, plo_tmem + k * 8, vd + ((k * 2048) >> 4), idesc_pv, 1u);
                    }
                };

                bool ok = mbar_wait(bar_q_full(), 0, wc, 0x20);
                ok = ok && mbar_wait(bar_kv_full(slot_of(0)), phase_of(0), wc, 0x21);
                if (ok) {
                    tc_fence_after_sync();
                    if (n_t > 0) {
                        issue_qk(slot_of(0));
                        mma_commit(bar_s_full(t));
                    }
                    mma_commit(bar_kv_empty(slot_of(0)));
                }
                for (int j = 0; j < n_max && ok; ++j) {
                    const int item_v = 2 * j + 1, item_k = 2 * j + 2;
                    // S of step j+1 as soon as the softmax warps have taken S of step j
                    if (j + 1 < n_max) {
                        ok = mbar_wait(bar_kv_full(slot_of(item_k)), phase_of(item_k), wc, 0x23);
                        if (ok && j + 1 < n_t) {
                            ok = mbar_wait(bar_s_free(t), (uint32_t)(j & 1), wc, 0x26 + t);
                            if (!ok) break;
                            tc_fence_after_sync();
                            LTCA_TRACE_EVT(0x20 + (j << 8));
                            issue_qk(slot_of(item_k));
                            mma_commit(bar_s_full(t));
                            LTCA_TRACE_EVT(0x22 + (j << 8));
                        }
                        if (!ok) break;
                        mma_commit(bar_kv_empty(slot_of(item_k)));
                    }
                    ok = mbar_wait(bar_kv_full(slot_of(item_v)), phase_of(item_v), wc, 0x22);
                    if (ok && j < n_t) {
                        ok = mbar_wait(bar_p_full(t), (uint32_t)(j & 1), wc, 0x24 + t);
                        if (!ok) break;
                        tc_fence_after_sync();
                        LTCA_TRACE_EVT(0x24 + (j << 8));
                        issue_pv(slot_of(item_v), j > 0);
                        mma_commit(bar_o_done(t));
                        LTCA_TRACE_EVT(0x26 + (j << 8));
                    }
                    if (!ok) break;
                    mma_commit(bar_kv_empty(slot_of(item_v)));
                }
                // everything this thread issued has to be complete before tensor memory is released
                if (ok && n_t > 0) ok = mbar_wait(bar_o_done(t), (uint32_t)((n_t - 1) & 1), wc, 0x28 + t);
            }
        }
    } else {
        // ------------------------------ softmax / correction / epilogue ------------------------
        reg_alloc<kMathRegs>();
        const int t = (warp >> 2) & 1;
        const int half = warp >> 3;          // which part of the key columns (and of the output columns)
        const int wq = warp & 3;
        const int row = wq * 32 + lane;
        const int q0 = m_block * 2 * kBlockM + t * kBlockM;
        const int qi = q0 + row;
        const int n_t = n_tiles[t];
        const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
        const uint32_t tS = tmem_base + lane_base + L::kColS + t * kBN + half * kH;
        const uint32_t tO = tmem_base + lane_base + L::kColO + t * D + half * kDH;
        const uint32_t tP = tmem_base + lane_base + L::kColP + t * (kBN / 2) + half * (kH / 2);
        const uint32_t tPlo = tmem_base + lane_base + L::kColPlo + t * (kBN / 2) + half * (kH / 2);
        const float c2 = a.scale_log2;
        const bool general = (a.keep_mask != nullptr) || (a.use_clamp != 0);
        // exchange slots: [buffer][tile][half][row]
        auto xslot = [&](int buf, int hf) { return xchg + ((buf * 2 + t) * 2 + hf) * kBlockM + row; };
        uint32_t pair_phase = 0;

        float m_run = neg_inf();
        float l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n_t; ++j) {
            ok = mbar_wait_warp(bar_s_full(t), (uint32_t)(j & 1), wc, 0x30 + t);
            if (!ok) break;
            tc_fence_after_sync();
            LTCA_TRACE_EVT(0x10 + (j << 8));
            uint32_t su[kH];
#pragma unroll
            for (int c0 = 0; c0 < kH; c0 += 32)
                tmem_ld32(tS + c0, reinterpret_cast<uint32_t(&)[32]>(su[c0]));
            tmem_wait_ld();
            // S is in registers: the next step's Q K^T may overwrite it
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_s_free(t));
            LTCA_TRACE_EVT(0x11 + (j << 8));
#define S_(c) __uint_as_float(su[(c)])
            const int k0 = j * kBN;
            const bool edge = (k0 + kBN > kvlen) || (a.causal && (k0 + kBN - 1 > q0 + a.causal_off));
            if (general) {
                int lim = kvlen;
                if (a.causal) lim = min(lim, qi + a.causal_off + 1);
                lim -= k0 + half * kH;                  // own columns c < lim are visible
                const float* mrow = nullptr;
                if (a.keep_mask && qi < a.Sq)
                    mrow = a.keep_mask + ((int64_t)b * a.Sq + qi) * a.Sk + k0 + half * kH;
#pragma unroll
                for (int c = 0; c < kH; ++c) {
                    float v = S_(c);
                    if (a.use_clamp) v = fminf(v, a.clamp_raw);
                    bool vis = c < lim;
                    if (mrow && vis) vis = (__ldg(mrow + c) != 0.0f);
                    su[c] = __float_as_uint(vis ? v : neg_inf());
                }
            } else if (edge) {
                // causal diagonal or end of the keys, no dense mask: a select per column, no branches
                int lim = kvlen;
                if (a.causal) lim = min(lim, qi + a.causal_off + 1);
                lim -= k0 + half * kH;
#pragma unroll
                for (int c = 0; c < kH; ++c) su[c] = (c < lim) ? su[c] : 0xff800000u;
            }
            float mx[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) mx[i] = fmaxf(S_(2 * i), S_(2 * i + 1));
#pragma unroll
            for (int c = 8; c < kH; c += 8)
#pragma unroll
                for (int i = 0; i < 4; ++i) mx[i] = fmax3(mx[i], S_(c + 2 * i), S_(c + 2 * i + 1));
            float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            {
                // the row's other half: both threads publish, meet, and read each other's maximum
                *xslot(j & 1, half) = mt;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_pair(t, wq));
                ok = mbar_wait_warp(bar_pair(t, wq), pair_phase, wc, 0x3a);
                pair_phase ^= 1u;
                if (!ok) break;
                mt = fmaxf(mt, *xslot(j & 1, half ^ 1));
            }
            LTCA_TRACE_EVT(0x12 + (j << 8));

            // Lazy rescale: keep the stale maximum while the new one exceeds it by less than
            // 2^8 in the exponent; P stays below 256 and fp32 sums keep their accuracy.
            float factor = 1.0f;
            bool need = false;
            if (j == 0) {
                m_run = mt;
            } else if ((mt - m_run) * c2 > 8.0f) {
                factor = fast_exp2((m_run - mt) * c2);
                m_run = mt;
                need = true;
            }
            bool o_waited = (j == 0);
            if (j > 0 && __any_sync(0xffffffffu, need)) {
                ok = mbar_wait_warp(bar_o_done(t), (uint32_t)((j - 1) & 1), wc, 0x32 + t);
                if (!ok) break;
                o_waited = true;
                tc_fence_after_sync();
#pragma unroll
                for (int c0 = 0; c0 < kDH; c0 += 32) {
                    uint32_t o[32];
                    tmem_ld32(tO + c0, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * factor);
                    tmem_st32(tO + c0, o);
                }
                l_run *= factor;
            }
            // One-time delay: tile 1 starts its first exponentials when tile 0 has finished its own, so that from
            // then on one tile exponentiates while the other loads its scores, finds its maxima and talks to the
            // barriers.  (Strict turn-taking at every step was slower.)
            if (t == 1 && j == 0 && n_tiles[0] > 0) {
                ok = mbar_wait_warp(bar_turn(0), 0, wc, 0x3e);
                if (!ok) break;
            }
            LTCA_TRACE_EVT(0x15 + (j << 8));
            const float m_safe = (m_run == neg_inf()) ? 0.f : m_run;
            const float mneg = -m_safe * c2;
            float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
            for (int ch = 0; ch < kH / 32; ++ch) {
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int cc = 0; cc < 32; cc += 4) {
                    const int c = ch * 32 + cc;
                    const float p0 = fast_exp2(fmaf(S_(c), c2, mneg));
                    const float p1 = fast_exp2(fmaf(S_(c + 1), c2, mneg));
                    const float p2 = fast_exp2(fmaf(S_(c + 2), c2, mneg));
                    const float p3 = fast_exp2(fmaf(S_(c + 3), c2, mneg));
                    sum0 += p0; sum1 += p1; sum2 += p2; sum3 += p3;
                    const uint32_t h01 = pack_bf16x2(p0, p1), h23 = pack_bf16x2(p2, p3);
                    hi[cc / 2] = h01;
                    hi[cc / 2 + 1] = h23;
                    if constexpr (kSplitP) {
                        lo[cc / 2] = pack_bf16x2(p0 - __uint_as_float(h01 << 16),
                                                 p1 - __uint_as_float(h01 & 0xffff0000u));
                        lo[cc / 2 + 1] = pack_bf16x2(p2 - __uint_as_float(h23 << 16),
                                                     p3 - __uint_as_float(h23 & 0xffff0000u));
                    }
                }
                if (ch == 0 && !o_waited) {
                    // P of the previous step must have been consumed before it is overwritten
                    ok = mbar_wait_warp(bar_o_done(t), (uint32_t)((j - 1) & 1), wc, 0x36 + t);
                    if (!ok) break;
                }
                tmem_st16(tP + ch * 16, hi);
                if constexpr (kSplitP) tmem_st16(tPlo + ch * 16, lo);
            }
            if (!ok) break;
            if (t == 0 && j == 0) {
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_turn(t));
            }
            l_run += (sum0 + sum1) + (sum2 + sum3);
            LTCA_TRACE_EVT(0x13 + (j << 8));
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p_full(t));
            LTCA_TRACE_EVT(0x14 + (j << 8));
#undef S_
        }

        // epilogue: O / l and lse; the row sum is the total of the two halves
        if (ok && q0 < a.Sq) {
            float inv = 0.f;
            float lse = neg_inf();
            if (n_t > 0) {
                {
                    *xslot(2, half) = l_run;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_pair(t, wq));
                    ok = mbar_wait_warp(bar_pair(t, wq), pair_phase, wc, 0x3b);
                    if (ok) l_run += *xslot(2, half ^ 1);
                }
                ok = ok && mbar_wait_warp(bar_o_done(t), (uint32_t)((n_t - 1) & 1), wc, 0x34 + t);
                tc_fence_after_sync();
                if (l_run > 0.f) {
                    inv = 1.0f / l_run;
                    lse = m_run * a.scale + __logf(l_run);
                }
            }
            OutT* orow = reinterpret_cast<OutT*>(a.o) + b * a.o_sb + h * a.o_sh + (int64_t)qi * a.o_ss +
                         half * kDH;
#pragma unroll
            for (int c0 = 0; c0 < kDH; c0 += 32) {
                uint32_t o[32];
                if (n_t > 0 && ok) {
                    tmem_ld32(tO + c0, o);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[c] = 0u;
                }
                if (qi < a.Sq) {
                    if constexpr (sizeof(OutT) == 2) {
                        uint4* dst = reinterpret_cast<uint4*>(orow + c0);
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            uint4 w;
                            w.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
                            w.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
                            w.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
                            w.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
                            dst[v] = w;
                        }
                    } else {
                        float4* dst = reinterpret_cast<float4*>(orow + c0);
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            dst[v] = make_float4(__uint_as_float(o[4 * v + 0]) * inv,
                                                 __uint_as_float(o[4 * v + 1]) * inv,
                                                 __uint_as_float(o[4 * v + 2]) * inv,
                                                 __uint_as_float(o[4 * v + 3]) * inv);
                    }
                }
            }
            if (half == 0 && a.lse && qi < a.Sq) a.lse[((int64_t)b * a.H + h) * a.Sq + qi] = lse;
        }
    }

    // ------------------------------ tear-down -------------------------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp0) {
        __syncwarp();
        if (misc[1]) __nanosleep(200000);    // aborted: give copies and MMAs in flight time to land
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------
// Four-tile persistent kernel (head_dim 64, bf16 result): the kernel used for long query ranges.
//
// Every scheduler of the SM holds four softmax warps that belong to four DIFFERENT query tiles;
// a tile's warps only ever wait for that tile's own barriers, so while one tile sits in a
// barrier round trip, a tensor-memory load or the tensor pipe's queue, the other three keep the
// special-function unit busy (measured on B200: four independent warps per scheduler hide every
// one of those latencies, two dependent ones hide almost none).
//   - steps of 64 keys; tile t: S_t = Q_t K_j^T in columns [64 t, 64 t + 64), O_t in
//     [256 + 64 t, 256 + 64 t + 64); P_t (bf16) overwrites the first 32 columns of S_t, so the
//     issuer queues O_t += P_t V_j and S_t = Q_t K_{j+1}^T back to back (the tensor pipe runs one
//     thread's MMAs in order) and one commit tells the tile both "S ready" and "O up to date";
//   - warps 0-15: softmax, one query row per thread (tile = warp / 4); warp 16 issues the
//     contractions of tiles 0 and 1, warp 17 those of tiles 2 and 3; warp 18: TMA producer.
//
// Persistent: one CTA per SM takes (512 query rows, head, batch)
// items from a global counter (ItemQueue; grouped heavy-first order).  Barriers, tensor memory
// and tensor maps are set up once per CTA; the Q tiles are double-buffered and the K/V ring runs
// straight from one item's last keys into the next item's first, so the pipeline never drains:
// a tile that has finished its rows of item i (the early tiles of a causal block have fewer key
// steps) writes its output and starts on item i+1 while the later tiles still work on item i.
// (A one-CTA-per-block version of this kernel spent 8.6 us per 512-row block on set-up, pipeline fill and drain.)
// Barrier phases run on per-role counters; every completion of a reused barrier depends on the
// waiter of the previous one, so a parity wait cannot alias:
//   s_full(t)    one commit per key step + one at the start and one at the end of an item
//   p_full(t)    one arrival per softmax warp per step
//   tile_free(t) the tile's warps have read O of the previous item out of tensor memory
//   q_full/q_empty[2], kv_full/kv_empty[8] as usual (both MMA threads release a slot).
// ---------------------------------------------------------------------------------------------
constexpr int kF4Tiles = 4;
constexpr int kF4BN = 64;
constexpr int kF4Threads = 640;
constexpr int kF4LaunchRegs = 96;
constexpr int kF4CtrlRegs = 56;
constexpr int kF4MathRegs = 104;
static_assert(512 * kF4MathRegs + 128 * kF4CtrlRegs <= kF4Threads * kF4LaunchRegs, "register budget");

struct F4PCfg {
    static constexpr int kQTileBytes = kBlockM * 64 * 2;       // 16 KB
    static constexpr int kKvTileBytes = kF4BN * 64 * 2;        // 8 KB
    static constexpr int kStages = 8;
    static constexpr int kQBufBytes = kF4Tiles * kQTileBytes;  // 64 KB, two of them
    static constexpr int kRingOff = 2 * kQBufBytes;
    static constexpr int kBarOff = kRingOff + kStages * kKvTileBytes;
    // q_full[2], q_empty[2], kv_full[S], kv_empty[S], s_full[4], p_full[4], tile_free[4], staged[4], item full/empty
    static constexpr int kNumBars = 4 + 2 * kStages + 4 * kF4Tiles + 2 * kItemSlots;
    static constexpr int kMiscOff = kBarOff + kNumBars * 8;
    static constexpr int kDynBytes = kMiscOff + 16 + 4 * kItemSlots + 1024;
};

template <bool kFold>
__global__ void __launch_bounds__(kF4Threads, 1)
attn_fwd4p_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q,
                        const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v,
                        const __grid_constant__ CUtensorMap tmap_o, const FwdArgs a, const ItemGrid grid) {
    using L = F4PCfg;
    constexpr int D = 64;
    constexpr int kBN = kF4BN;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t q_smem = smem_base;
    const uint32_t ring_smem = smem_base + L::kRingOff;
    const uint32_t bar_base = smem_base + L::kBarOff;
    auto bar_q_full = [&](int r) { return bar_base + 8u * r; };
    auto bar_q_empty = [&](int r) { return bar_base + 8u * (2 + r); };
    auto bar_kv_full = [&](int s) { return bar_base + 8u * (4 + s); };
    auto bar_kv_empty = [&](int s) { return bar_base + 8u * (4 + L::kStages + s); };
    auto bar_s_full = [&](int t) { return bar_base + 8u * (4 + 2 * L::kStages + t); };
    auto bar_p_full = [&](int t) { return bar_base + 8u * (4 + 2 * L::kStages + kF4Tiles + t); };
    auto bar_tile_free = [&](int t) { return bar_base + 8u * (4 + 2 * L::kStages + 2 * kF4Tiles + t); };
    auto bar_staged = [&](int t) { return bar_base + 8u * (4 + 2 * L::kStages + 3 * kF4Tiles + t); };
    const uint32_t bar_item0 = bar_base + 8u * (4 + 2 * L::kStages + 4 * kF4Tiles);
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOff);
    const ItemQueue iq{bar_item0, bar_item0 + 8u * kItemSlots,
                       reinterpret_cast<volatile int*>(smem_gen + L::kMiscOff + 16)};

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    LTCA_TRACE_DECL(blockIdx.x == 5);
    LTCA_TRACE_EVT(0x01);

    if (threadIdx.x == 0) {
        // a Q buffer is free again when both MMA threads are done with it and every tile's output,
        // which is staged in the tile's own Q slot, has been read by its TMA store
        for (int r = 0; r < 2; ++r) { mbar_init(bar_q_full(r), 1); mbar_init(bar_q_empty(r), 2 + kF4Tiles); }
        for (int s = 0; s < L::kStages; ++s) { mbar_init(bar_kv_full(s), 1); mbar_init(bar_kv_empty(s), 2); }
        for (int t = 0; t < kF4Tiles; ++t) {
            mbar_init(bar_s_full(t), 1);
            mbar_init(bar_p_full(t), 4);
            mbar_init(bar_tile_free(t), 4);
            mbar_init(bar_staged(t), 4);
        }
        for (int i = 0; i < kItemSlots; ++i) { mbar_init(iq.full(i), 1); mbar_init(iq.empty(i), 18); }
        misc[1] = 0u;
        mbar_fence_init();
    }
    if (warp == 16) { tmem_alloc(smem_u32(const_cast<uint32_t*>(&misc[0])), kTmemCols); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = misc[0];
    const WaitCtx wc{&misc[1], a.status};
    grid_dependency_wait();                    // the operands are complete once the kernel before this one has ended

    // the item's block, its (head, batch), and the number of 64-key steps of each tile
    struct Item { int m_block, h, b, kvlen, n_max; };
    // First query row of tile t of block m.  Plain: four neighbouring tiles.  Folded (a causal launch with no more
    // items than SMs, where the launch lasts as long as its heaviest item): tiles 2m and 2m + 1 from the start of
    // the padded tile range and the two tiles that mirror them at its end, so that every item carries the same
    // work; the early tiles finish their few key steps and wait, the late ones run on with the SM to themselves.
    auto tile_q0 = [&](int m, int t) {
        if (!kFold) return (m * kF4Tiles + t) * kBlockM;
        const int tile = t < 2 ? 2 * m + t : grid.nblk * kF4Tiles - 2 * m - 4 + t;
        return tile * kBlockM;
    };
    auto steps_of = [&](const Item& it, int t) {
        const int q0 = tile_q0(it.m_block, t);
        int lim = 0;
        if (q0 < a.Sq) {
            lim = it.kvlen;
            if (a.causal) lim = min(lim, min(q0 + kBlockM - 1, a.Sq - 1) + a.causal_off + 1);
        }
        return lim > 0 ? (lim + kBN - 1) / kBN : 0;
    };
    auto decode = [&](int linear, Item& it) {
        int rank;
        sched_item(grid, linear, rank, it.h, it.b);
        it.m_block = grid.nblk - 1 - rank;              // heavy (late) causal blocks first
        it.kvlen = a.Sk;
        if (a.kv_len) it.kvlen = min(max(a.kv_len[it.b], 0), a.Sk);
        it.n_max = 0;
#pragma unroll
        for (int t = 0; t < kF4Tiles; ++t) it.n_max = max(it.n_max, steps_of(it, t));
    };
    auto slot_of = [&](int e) { return e % L::kStages; };
    auto phase_of = [&](int e) { return (uint32_t)((e / L::kStages) & 1); };

    if (warp >= 16) {
        reg_dealloc<kF4CtrlRegs>();
        if (warp == 18) {
            // ------------------------------ TMA producer --------------------------------------
            if (lane == 0) {
                tma_prefetch_desc(&tmap_q);
                tma_prefetch_desc(&tmap_k);
                tma_prefetch_desc(&tmap_v);
                bool ok = true;
                int nq = 0, na = 0, kve = 0;
                auto load_q = [&](const Item& it, int use) {     // `use`: ordinal among the items that have keys
                    const int r = use & 1;
                    if (!mbar_wait(bar_q_empty(r), (uint32_t)(((use >> 1) & 1) ^ 1), wc, 0x11)) return false;
                    mbar_arrive_expect_tx(bar_q_full(r), (uint32_t)L::kQBufBytes);
                    for (int t = 0; t < kF4Tiles; ++t)
                        tma_load_4d(q_smem + r * L::kQBufBytes + t * L::kQTileBytes, &tmap_q, bar_q_full(r), 0,
                                    tile_q0(it.m_block, t), it.h, it.b);
                    LTCA_TRACE_EVT(0x31);
                    return true;
                };
                Item cur, nxt;
                int lin = iq.produce(nq++, grid.counters, grid.n_items, wc);
                bool cur_q = false;
                while (ok && lin >= 0) {
                    decode(lin, cur);
                    if (cur.n_max > 0 && !cur_q) ok = load_q(cur, na);
                    // the next item is fetched (a global atomic) towards the end of this item's key stream and
                    // its Q tiles are loaded under this item's last keys
                    int lin_next = -1;
                    bool have_lin_next = false;
                    bool nxt_q = false;
                    bool nxt_active = false;
                    auto fetch_next = [&]() {
                        lin_next = iq.produce(nq++, grid.counters, grid.n_items, wc);
                        have_lin_next = true;
                        if (lin_next == -2) { ok = false; return; }
                        LTCA_TRACE_EVT(0x32);
                        if (lin_next >= 0) { decode(lin_next, nxt); nxt_active = nxt.n_max > 0; }
                    };
                    if (cur.n_max > 0) {
                        const int use_next = na + 1;
                        for (int j = 0; j < cur.n_max && ok; ++j) {
#pragma unroll
                            for (int which = 0; which < 2; ++which, ++kve) {     // 0: K_j, 1: V_j
                                const int slot = slot_of(kve);
                                ok = ok && mbar_wait(bar_kv_empty(slot), phase_of(kve) ^ 1u, wc, 0x10);
                                if (!ok) break;
                                mbar_arrive_expect_tx(bar_kv_full(slot), (uint32_t)L::kKvTileBytes);
                                tma_load_4d(ring_smem + slot * L::kKvTileBytes, which == 0 ? &tmap_k : &tmap_v,
                                            bar_kv_full(slot), 0, j * kBN, cur.h, cur.b);
                            }
                            LTCA_TRACE_EVT(0x30 + (j << 8));
                            // (late: an item taken long before it is started is an item that an SM which
                            // becomes idle earlier can no longer take; two steps before the end of the key stream
                            // still leaves the consumers' four steps of ring depth to fetch it and load its Q)
                            if (ok && !have_lin_next && j + 2 >= cur.n_max) fetch_next();
                            // Q of the next item as soon as its buffer has been released, without
                            // ever holding up the key stream
                            if (ok && nxt_active && !nxt_q &&
                                mbar_try_wait(bar_q_empty(use_next & 1), (uint32_t)(((use_next >> 1) & 1) ^ 1))) {
                                ok = load_q(nxt, use_next);
                                nxt_q = true;
                            }
                        }
                        ++na;
                    }
                    if (ok && !have_lin_next) fetch_next();
                    cur_q = nxt_q;
                    lin = lin_next;
                }
            }
        } else if (warp == 16 || warp == 17) {
            // ------------------------------ MMA issuer of tiles 2i, 2i+1 ----------------------
            const int t0 = 2 * (warp - 16);
            if (lane == 0) {
                constexpr uint32_t idesc_qk = make_idesc_bf16(kBlockM, kBN, 0, 0);
                constexpr uint32_t idesc_pv = make_idesc_bf16(kBlockM, D, 0, 1);
                const uint64_t q_desc = make_smem_desc_sw128(q_smem, 16, 1024);
                const uint64_t k_desc = make_smem_desc_sw128(ring_smem, 16, 1024);
                const uint64_t v_desc = make_smem_desc_sw128(ring_smem, kBN * 128, 1024);
                auto issue_qk = [&](int t, int slot, int r) {
                    const uint64_t qd = q_desc + (uint64_t)((r * L::kQBufBytes + t * L::kQTileBytes) >> 4);
                    const uint64_t kd = k_desc + (uint64_t)((slot * L::kKvTileBytes) >> 4);
#pragma unroll
                    for (int k = 0; k < D / 16; ++k)
                        mma_ss(tmem_base + t * kBN, qd + 2 * k, kd + 2 * k, idesc_qk, k > 0 ? 1u : 0u);
                };
                auto issue_pv = [&](int t, int slot, bool acc) {
                    const uint64_t vd = v_desc + (uint64_t)((slot * L::kKvTileBytes) >> 4);
#pragma unroll
                    for (int k = 0; k < kBN / 16; ++k)
                        mma_ts(tmem_base + 256 + t * D, tmem_base + t * kBN + k * 8, vd + 128 * k, idesc_pv,
                               (acc || k > 0) ? 1u : 0u);
                };
                bool ok = true;
                int na = 0, kve = 0;
                int uses[2] = {0, 0};       // items in which tile t0 + i had keys
                int pcnt[2] = {0, 0};       // p_full phases consumed
                Item it;
                for (int nq = 0; ok; ++nq) {
                    const int lin = iq.consume(nq, wc);
                    if (lin < 0) break;
                    decode(lin, it);
                    if (it.n_max == 0) continue;
                    const int nt0 = steps_of(it, t0), nt1 = steps_of(it, t0 + 1);
                    const int r = na & 1;
                    ok = mbar_wait(bar_q_full(r), (uint32_t)((na >> 1) & 1), wc, 0x20);
                    ok = ok && mbar_wait(bar_kv_full(slot_of(kve)), phase_of(kve), wc, 0x21);
                    if (!ok) break;
                    LTCA_TRACE_EVT(0x28);
                    tc_fence_after_sync();
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int t = t0 + i;
                        if (ok && (i == 0 ? nt0 : nt1) > 0) {
                            // S and O of the tile's previous item must have been read out
                            if (uses[i] > 0) {
                                ok = mbar_wait(bar_tile_free(t), (uint32_t)((uses[i] - 1) & 1), wc, 0x2c + t);
                                if (!ok) break;
                                tc_fence_after_sync();
                            }
                            ++uses[i];
                            LTCA_TRACE_EVT(0x29 + (i << 8));
                            issue_qk(t, slot_of(kve), r);
                            mma_commit(bar_s_full(t));
                        }
                    }
                    if (!ok) break;
                    mma_commit(bar_kv_empty(slot_of(kve)));
                    for (int j = 0; j < it.n_max && ok; ++j) {
                        const int e_v = kve + 2 * j + 1, e_k = kve + 2 * j + 2;
                        const bool have_next = (j + 1 < it.n_max);
                        ok = mbar_wait(bar_kv_full(slot_of(e_v)), phase_of(e_v), wc, 0x22);
                        if (have_next) ok = ok && mbar_wait(bar_kv_full(slot_of(e_k)), phase_of(e_k), wc, 0x23);
                        LTCA_TRACE_EVT(0x24 + (j << 8));
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            const int t = t0 + i;
                            const int nt = i == 0 ? nt0 : nt1;
                            if (ok && j < nt) {
                                ok = mbar_wait(bar_p_full(t), (uint32_t)(pcnt[i] & 1), wc, 0x24 + t);
                                if (!ok) break;
                                ++pcnt[i];
                                LTCA_TRACE_EVT(0x20 + i + (j << 8));
                                tc_fence_after_sync();
                                issue_pv(t, slot_of(e_v), j > 0);
                                if (j + 1 < nt) issue_qk(t, slot_of(e_k), r);
                                mma_commit(bar_s_full(t));     // S of step j+1 ready, O holds steps 0..j
                                LTCA_TRACE_EVT(0x22 + i + (j << 8));
                            }
                        }
                        if (!ok) break;
                        mma_commit(bar_kv_empty(slot_of(e_v)));
                        if (have_next) mma_commit(bar_kv_empty(slot_of(e_k)));
                    }
                    if (!ok) break;
                    mma_commit(bar_q_empty(r));             // this thread's last read of the item's Q tiles
                    kve += 2 * it.n_max;
                    ++na;
                }
            }
        }
    } else {
        // ------------------------------ softmax / correction / epilogue ------------------------
        reg_alloc<kF4MathRegs>();
        const int t = warp >> 2;
        const int wq = warp & 3;
        const int row = wq * 32 + lane;
        const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
        const uint32_t tS = tmem_base + lane_base + t * kBN;
        const uint32_t tO = tmem_base + lane_base + 256 + t * D;
        const float c2 = a.scale_log2;
        const bool general = (a.keep_mask != nullptr) || (a.use_clamp != 0);
        int scnt = 0;                       // s_full phases consumed
        int na = 0;                         // items with keys so far (selects the Q buffer)
        int ecnt = 0;                       // outputs this tile has staged
        bool ok = true;
        Item it;
        for (int nq = 0; ok; ++nq) {
            const int lin = iq.consume_warp(nq, wc);
            if (lin < 0) break;
            decode(lin, it);
            const int n_t = steps_of(it, t);
            const int n_max = it.n_max;
            const int b_mask = it.b;
            // per row: number of visible keys; per tile: the first step that needs masking at all
            int lim_row, je = n_t;
            {
                const int q0 = tile_q0(it.m_block, t);
                lim_row = it.kvlen;
                if (a.causal) lim_row = min(lim_row, q0 + row + a.causal_off + 1);
                if (it.kvlen % kBN) je = min(je, it.kvlen / kBN);
                if (a.causal) {
                    const int v = q0 + a.causal_off - (kBN - 1);      // step j is cut by the diagonal when j * kBN > v
                    je = min(je, v < 0 ? 0 : v / kBN + 1);
                }
            }

            float m_run = neg_inf();
            float l_run = 0.f;
            for (int j = 0; j < n_t; ++j) {
                ok = mbar_wait_warp(bar_s_full(t), (uint32_t)(scnt & 1), wc, 0x30 + t);
                if (!ok) break;
                ++scnt;
                LTCA_TRACE_EVT(0x10 + (j << 8));
                tc_fence_after_sync();
                uint32_t su[kBN];
                tmem_ld32(tS, reinterpret_cast<uint32_t(&)[32]>(su[0]));
                tmem_ld32(tS + 32, reinterpret_cast<uint32_t(&)[32]>(su[32]));
                tmem_wait_ld();
                LTCA_TRACE_EVT(0x11 + (j << 8));
#define S_(c) __uint_as_float(su[(c)])
                if (general) {
                    const int k0 = j * kBN;
                    const int lim = lim_row - k0;           // columns c < lim are visible
                    const int qi = tile_q0(it.m_block, t) + row;
                    const float* mrow = nullptr;
                    if (a.keep_mask && qi < a.Sq)
                        mrow = a.keep_mask + ((int64_t)b_mask * a.Sq + qi) * a.Sk + k0;
#pragma unroll
                    for (int c = 0; c < kBN; ++c) {
                        float v = S_(c);
                        if (a.use_clamp) v = fminf(v, a.clamp_raw);
                        bool vis = c < lim;
                        if (mrow && vis) vis = (__ldg(mrow + c) != 0.0f);
                        su[c] = __float_as_uint(vis ? v : neg_inf());
                    }
                } else if (j >= je) {
                    // causal diagonal or end of the keys, no dense mask: a select per column, no branches
                    const int lim = lim_row - j * kBN;
#pragma unroll
                    for (int c = 0; c < kBN; ++c) su[c] = (c < lim) ? su[c] : 0xff800000u;
                }
                float mx[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) mx[i] = fmaxf(S_(2 * i), S_(2 * i + 1));
#pragma unroll
                for (int c = 8; c < kBN; c += 8)
#pragma unroll
                    for (int i = 0; i < 4; ++i) mx[i] = fmax3(mx[i], S_(c + 2 * i), S_(c + 2 * i + 1));
                const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));

                // Lazy rescale: keep the stale maximum while the new one exceeds it by less than
                // 2^8 in the exponent; P stays below 256 and fp32 sums keep their accuracy.
                float factor = 1.0f;
                bool need = false;
                if (j == 0) {
                    m_run = mt;
                } else if ((mt - m_run) * c2 > 8.0f) {
                    factor = fast_exp2((m_run - mt) * c2);
                    m_run = mt;
                    need = true;
                }
                if (j > 0 && __any_sync(0xffffffffu, need)) {
                    // O already holds every earlier step: the commit behind s_full covered it
                    // (rare: not unrolled, or its four 16-register pieces push the step's scores out of registers)
#pragma unroll 1
                    for (int c0 = 0; c0 < D; c0 += 16) {
                        uint32_t o[16];
                        tmem_ld16(tO + c0, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 16; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * factor);
                        tmem_st16(tO + c0, o);
                    }
                    l_run *= factor;
                }
                const float m_safe = (m_run == neg_inf()) ? 0.f : m_run;
                const float mneg = -m_safe * c2;
                float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
                for (int ch = 0; ch < kBN / 32; ++ch) {
                    uint32_t hi[16];
#pragma unroll
                    for (int cc = 0; cc < 32; cc += 4) {
                        const int c = ch * 32 + cc;
                        const float p0 = fast_exp2(fmaf(S_(c), c2, mneg));
                        const float p1 = fast_exp2(fmaf(S_(c + 1), c2, mneg));
                        const float p2 = fast_exp2(fmaf(S_(c + 2), c2, mneg));
                        const float p3 = fast_exp2(fmaf(S_(c + 3), c2, mneg));
                        sum0 += p0; sum1 += p1; sum2 += p2; sum3 += p3;
                        hi[cc / 2] = pack_bf16x2(p0, p1);
                        hi[cc / 2 + 1] = pack_bf16x2(p2, p3);
                    }
                    tmem_st16(tS + ch * 16, hi);      // P over the first columns of S (all of S is in registers)
                }
                l_run += (sum0 + sum1) + (sum2 + sum3);
                tmem_wait_st();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_p_full(t));
                LTCA_TRACE_EVT(0x12 + (j << 8));
#undef S_
            }
            if (!ok) break;

            // epilogue: O / l and lse; the tile's tensor memory is handed back before the stores
            decode(lin, it);                    // (re-derived here rather than kept in registers across the key loop)
            const int b = it.b, h = it.h;
            const int q0 = tile_q0(it.m_block, t);
            const int qi = q0 + row;
            if (it.n_max > 0) {
                const int r = na & 1;
                ++na;
                if (n_t > 0) {
                    ok = mbar_wait_warp(bar_s_full(t), (uint32_t)(scnt & 1), wc, 0x34 + t);
                    if (!ok) break;
                    ++scnt;
                    LTCA_TRACE_EVT(0x18);
                    tc_fence_after_sync();
                    uint32_t o[D];
                    tmem_ld32(tO, reinterpret_cast<uint32_t(&)[32]>(o[0]));
                    tmem_ld32(tO + 32, reinterpret_cast<uint32_t(&)[32]>(o[32]));
                    tmem_wait_ld();
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_tile_free(t));
                    LTCA_TRACE_EVT(0x19);
                    float inv = 0.f;
                    float lse = neg_inf();
                    if (l_run > 0.f) {
                        inv = 1.0f / l_run;
                        lse = m_run * a.scale + __logf(l_run);
                    }
                    // this row, bf16, into the tile's Q slot in the layout of a 128-byte-swizzled TMA box
                    uint8_t* stage = smem_gen + r * L::kQBufBytes + t * L::kQTileBytes + row * 128;
#pragma unroll
                    for (int v = 0; v < D / 8; ++v) {
                        uint4 w;
                        w.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
                        w.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
                        w.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
                        w.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
                        *reinterpret_cast<uint4*>(stage + ((v ^ (row & 7)) << 4)) = w;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_staged(t));
                    if (a.lse && qi < a.Sq) a.lse[((int64_t)b * a.H + h) * a.Sq + qi] = lse;
                    if (wq == 0 && lane == 0) {
                        // one thread stores the tile once all four warps have staged their rows
                        // (rows past the end of the sequence are clipped by the tensor map)
                        if (mbar_wait(bar_staged(t), (uint32_t)(ecnt & 1), wc, 0x38 + t)) {
                            tma_store_4d(&tmap_o, q_smem + r * L::kQBufBytes + t * L::kQTileBytes, 0, q0, h, b);
                            tma_store_commit();
                            tma_store_wait_read<0>();
                        }
                        mbar_arrive(bar_q_empty(r));
                    }
                    ++ecnt;
                } else {
                    // no key is visible to these rows: zeros and -inf
                    if (q0 < a.Sq && qi < a.Sq) {
                        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(a.o) + b * a.o_sb + h * a.o_sh +
                                              (int64_t)qi * a.o_ss;
                        uint4* dst = reinterpret_cast<uint4*>(orow);
#pragma unroll
                        for (int v = 0; v < D / 8; ++v) dst[v] = make_uint4(0u, 0u, 0u, 0u);
                        if (a.lse) a.lse[((int64_t)b * a.H + h) * a.Sq + qi] = neg_inf();
                    }
                    if (wq == 0 && lane == 0) mbar_arrive(bar_q_empty(r));
                }
            } else if (q0 < a.Sq && qi < a.Sq) {
                __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(a.o) + b * a.o_sb + h * a.o_sh +
                                      (int64_t)qi * a.o_ss;
                uint4* dst = reinterpret_cast<uint4*>(orow);
#pragma unroll
                for (int v = 0; v < D / 8; ++v) dst[v] = make_uint4(0u, 0u, 0u, 0u);
                if (a.lse) a.lse[((int64_t)b * a.H + h) * a.Sq + qi] = neg_inf();
            }
            LTCA_TRACE_EVT(0x1a);
        }
    }

    // ------------------------------ tear-down -------------------------------------------------
    // Out of work: only now may the kernel after this one place its CTAs (released at the start, its blocks would
    // sit beside this kernel's CTAs for the whole run, waiting for it to end).
    grid_launch_dependents();
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) item_counters_release(grid.counters);
    if (warp == 16) {
        __syncwarp();
        if (misc[1]) __nanosleep(200000);    // aborted: give copies and MMAs in flight time to land
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

int launch_fwd4(ltca_ctx* ctx, const ltca_attn_params* p, const void* q, const void* k, const void* v,
                const ltca_strides& qs, const ltca_strides& ks, const ltca_strides& vs, const FwdArgs& a) {
    using P = F4PCfg;
    CUtensorMap tq, tk, tv, to;
    int rc;
    if ((rc = make_tmap_bhsd(ctx, &tq, q, 2, p->B, p->H, p->Sq, 64, qs, 64, kBlockM))) return rc;
    if ((rc = make_tmap_bhsd(ctx, &tk, k, 2, p->B, p->H, p->Sk, 64, ks, 64, kF4BN))) return rc;
    if ((rc = make_tmap_bhsd(ctx, &tv, v, 2, p->B, p->H, p->Sk, 64, vs, 64, kF4BN))) return rc;
    if ((rc = make_tmap_bhsd(ctx, &to, p->o, 2, p->B, p->H, p->Sq, 64, p->o_strides, 64, kBlockM))) return rc;
    static SmemOptIn opt_in, opt_in_fold;
    LTCA_CUDA_OK(ctx, opt_in_dynamic_smem(opt_in, ctx->device, attn_fwd4p_sm100_kernel<false>, P::kDynBytes));
    LTCA_CUDA_OK(ctx, opt_in_dynamic_smem(opt_in_fold, ctx->device, attn_fwd4p_sm100_kernel<true>, P::kDynBytes));
    ItemGrid ig;
    ig.nblk = (p->Sq + kF4Tiles * kBlockM - 1) / (kF4Tiles * kBlockM);
    ig.H = p->H;
    ig.BH = p->B * p->H;
    ig.n_items = ig.nblk * ig.BH;
    ig.counters = ctx->d_sched + 6;             // ints 6,7: the forward kernel's item counters
    // (measured: B=1 H=16 S=4096, the bench workload dealt over eight GPUs: 92 us folded against 123 us)
    ig.fold = (a.causal && ig.nblk > 1 && ig.n_items <= ctx->sm_count) ? 1 : 0;
    const int n_cta = ig.n_items < ctx->sm_count ? ig.n_items : ctx->sm_count;
    if (ig.fold)
        LTCA_CUDA_OK(ctx, launch_dependent_if(small_attention_call(p), attn_fwd4p_sm100_kernel<true>, dim3(n_cta), dim3(kF4Threads), P::kDynBytes,
                                           ctx->stream, tq, tk, tv, to, a, ig));
    else
        LTCA_CUDA_OK(ctx, launch_dependent_if(small_attention_call(p), attn_fwd4p_sm100_kernel<false>, dim3(n_cta), dim3(kF4Threads), P::kDynBytes,
                                           ctx->stream, tq, tk, tv, to, a, ig));
    LTCA_LAUNCH_OK(ctx, "attn_fwd4p_sm100_kernel");
    return LTCA_OK;
}

template <int D, typename OutT>
int launch_fwd(ltca_ctx* ctx, const ltca_attn_params* p, const void* q, const void* k,
               const void* v, const ltca_strides& qs, const ltca_strides& ks,
               const ltca_strides& vs) {
    constexpr bool kSplitP = sizeof(OutT) == 4;
    using L = FwdCfg<D, kSplitP>;
    CUtensorMap tq, tk, tv;
    int rc;
    if ((rc = make_tmap_bhsd(ctx, &tq, q, 2, p->B, p->H, p->Sq, D, qs, 64, kBlockM))) return rc;
    if ((rc = make_tmap_bhsd(ctx, &tk, k, 2, p->B, p->H, p->Sk, D, ks, 64, L::kBN))) return rc;
    if ((rc = make_tmap_bhsd(ctx, &tv, v, 2, p->B, p->H, p->Sk, D, vs, 64, L::kBN))) return rc;

    FwdArgs a;
    a.B = p->B; a.H = p->H; a.Sq = p->Sq; a.Sk = p->Sk;
    a.causal = p->causal ? 1 : 0;
    a.causal_off = p->Sk - p->Sq;
    a.scale = p->scale;
    a.scale_log2 = p->scale * 1.4426950408889634f;
    a.use_clamp = (p->score_clamp > 0.f) ? 1 : 0;
    a.clamp_raw = a.use_clamp ? p->score_clamp / p->scale : __builtin_inff();
    a.o = p->o;
    a.o_sb = p->o_strides.batch; a.o_sh = p->o_strides.head; a.o_ss = p->o_strides.seq;
    a.lse = p->lse;
    a.keep_mask = p->keep_mask;
    a.kv_len = p->kv_len;
    a.status = ctx->d_status;

    if constexpr (D == 64 && sizeof(OutT) == 2) {
        // long query ranges: four independent tiles per CTA (see attn_fwd4p_sm100_kernel)
        // ... unless its work items (512 queries of one batch entry and head) leave SMs idle where the CTAs of the
        // two-tile kernel (256 queries) would fill them: B=4 H=16 Sq=512 Sk=4096 takes 129 us on 64 of 148 SMs
        // against 75 us on 128, B=1 H=8 S=4096 causal 92 against 70 us.  Per tile the four-tile kernel is the
        // faster one (16 pairs of S=4096, causal: 99 against 112 us), so it keeps the case unless the other fills
        // the SMs a quarter better.  The device's SM count decides, not a limit set on the context: the choice,
        // and with it the bits of the result, does not move with the launch width.
        bool four = p->Sq > kFwd4MinSq;
        const int64_t bh = (int64_t)p->B * p->H;
        const int64_t items4 = bh * ((p->Sq + 4 * kBlockM - 1) / (4 * kBlockM));
        const int64_t sms = ctx->sm_device > 0 ? ctx->sm_device : kPlanSms;
        if (four && items4 < sms) {
            const int64_t ctas2 = bh * ((p->Sq + 2 * kBlockM - 1) / (2 * kBlockM));
            const int64_t waves2 = (ctas2 + sms - 1) / sms;
            four = (double)ctas2 / (double)(waves2 * sms) < 1.25 * (double)items4 / (double)sms;
        }
        if (four) return launch_fwd4(ctx, p, q, k, v, qs, ks, vs, a);
    }

    auto kern = attn_fwd_sm100_kernel<D, OutT, kSplitP>;
    static SmemOptIn opt_in;                  // one per template instantiation
    LTCA_CUDA_OK(ctx, opt_in_dynamic_smem(opt_in, ctx->device, kern, L::kDynBytes));
    dim3 grid((p->Sq + 2 * kBlockM - 1) / (2 * kBlockM), p->H, p->B);
    LTCA_CUDA_OK(ctx, launch_dependent(kern, grid, dim3(kFwdThreads), L::kDynBytes, ctx->stream, tq, tk, tv, a));
    LTCA_LAUNCH_OK(ctx, "attn_fwd_sm100_kernel");
    return LTCA_OK;
}

}  // namespace

#ifdef LTCA_TRACE
extern "C" int ltca_trace_read_fwd(unsigned long long* events, unsigned int* counts) {
    if (cudaMemcpyFromSymbol(events, g_trace, sizeof(g_trace)) != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(counts, g_trace_count, sizeof(g_trace_count)) != cudaSuccess) return -1;
    return 0;
}
#endif

bool attn_fwd_sm100_supported(const ltca_attn_params* p) {
    if (p->D != 64 && p->D != 128) return false;
    if (p->Sq < 1 || p->Sk < 1) return false;
    if (!(p->scale > 0.f)) return false;
    if (p->H > 65535 || p->B > 65535) return false;
    return true;
}

// Expects bf16 Q, K, V (already converted when the caller's storage is fp32).
int launch_attn_fwd_sm100_bf16in(ltca_ctx* ctx, const ltca_attn_params* p, const void* q,
                                 const void* k, const void* v, const ltca_strides& qs,
                                 const ltca_strides& ks, const ltca_strides& vs) {
    const int oes = elem_size(p->dtype);
    if ((reinterpret_cast<uintptr_t>(p->o) & 15) || ((p->o_strides.seq * oes) & 15) ||
        ((p->o_strides.head * oes) & 15) || ((p->o_strides.batch * oes) & 15))
        return fail(ctx, LTCA_ERR_INVALID, "output base and strides must be 16-byte aligned");
    if (p->D == 64) {
        return p->dtype == LTCA_BF16 ? launch_fwd<64, __nv_bfloat16>(ctx, p, q, k, v, qs, ks, vs)
                                     : launch_fwd<64, float>(ctx, p, q, k, v, qs, ks, vs);
    }
    return p->dtype == LTCA_BF16 ? launch_fwd<128, __nv_bfloat16>(ctx, p, q, k, v, qs, ks, vs)
                                 : launch_fwd<128, float>(ctx, p, q, k, v, qs, ks, vs);
}

}  // namespace ltca
