// Projection GEMMs of the TimeSelfAttention module on the tcgen05 tensor pipe.
//
//   C[M,N] = sum over pairs p of op(A_p) op(B_p)  (+ bias[N]),   bf16 operands, fp32 accumulation
//
// replaces the reference's cublasSgemm + addBiasKernel calls
// (reference src/ml/flash_attention.cu:866-958, 1075-1104) and the projections that cuDNN performs
// inside cudnnMultiHeadAttnForward / BackwardData / BackwardWeights (src/ml/cuDNN_ops.cu:203, 301, 366).
//
// Operand forms (all row-major in HBM):
//   A "K-major":  stored [M, K]  (activations x, ctx, dy, dq ...)      -> one 128 x 64 TMA box
//   A "M-major":  stored [K, M]  (x^T, ctx^T of the weight gradients)  -> two 64 x 64 boxes
//   B "K-major":  stored [N, K]  (a weight matrix used transposed)     -> one 128 x 64 box
//   B "N-major":  stored [K, N]  (a weight matrix used as stored; dq of the weight gradients)
// so no operand is ever transposed in memory: the instruction descriptor's major bits select the
// form and the shared-memory descriptors follow the layout the TMA boxes produce.
//
// Persistent CTAs (one per SM) walk a list of 128 x 256 tiles of C: warp 0 is the TMA producer (ring of four
// 48 KB (A, B) stages), warp 1 issues the MMAs (M128 N256 K16) into one of two 256-column accumulators in tensor
// memory, warps 2-5 are the epilogue (one accumulator row per thread: tcgen05.ld, bias, convert; the tile is
// staged in shared memory as 128-byte-swizzled boxes and stored with TMA), which works on tile i while the MMAs
// of tile i+1 run.  Measured at the module's sizes (device time line of one CTA): a ring stage of 48 KB arrives
// every 600 - 700 cycles (about 80 bytes per cycle and SM from L2: every 128-row block of A is re-read once per
// N tile and every weight matrix once per M tile) against 512 cycles of MMAs, which is why the tile is 256 wide;
// the epilogue of a tile takes 4700 cycles (bf16) to 7200 (fp32) and is hidden behind the next tile's main loop
// except for the last tile of a CTA.
// The tile list runs over independent problems (Q, K and V projections share one launch) and/or splits of K
// (weight gradients: K = batch x time is long and M x N is small, so the K range is cut into
// slices whose partial tiles go to scratch and are summed in a fixed order by a second kernel).
// `n_sum` > 1 accumulates several operand pairs into one tile (dx = dq Wq^T + dk Wk^T + dv Wv^T).
#include "host_common.h"
#include "gemm_sm100.h"
#include "attn_wide.h"
#include "sm100_ptx.cuh"
#include "trace.cuh"
#ifndef LTCA_TRACE_GEMM_Z
#define LTCA_TRACE_GEMM_Z 1   // which launch of a module call records: the one with this many problems
#endif

namespace ltca {

namespace {

constexpr int kBM = 128, kBN = 256, kBK = 64;
constexpr int kStages = 4;                         // operand ring: 4 x (16 KB of A + 32 KB of B)
constexpr int kATileBytes = kBM * kBK * 2;         // 16 KB
constexpr int kBTileBytes = kBN * kBK * 2;         // 32 KB
constexpr int kStageBytes = kATileBytes + kBTileBytes;
// The result tile leaves through two staging boxes of 128 rows x 128 bytes (64 bf16 or 32 fp32 columns) that
// alternate.  A tiled TMA store reads shared memory at 32 bytes per cycle (513 cycles per box, measured with one
// and with 148 CTAs storing, whatever the number of stores in flight), so a second pair of boxes buys nothing,
// and a fourth ring stage measured 3 - 6 % faster at the module's sizes than three stages with four or five boxes.
constexpr int kStageBoxes = 2;
constexpr int kStageOutBytes = kBM * 128 * kStageBoxes;
constexpr int kGemmThreads = 192;
constexpr int kOutOff = kStages * kStageBytes;
constexpr int kBarOff = kOutOff + kStageOutBytes;
constexpr int kNumBars = 2 * kStages + 4;          // full[S], empty[S], acc_full[2], acc_empty[2]
constexpr int kMiscOff = kBarOff + kNumBars * 8;
constexpr int kDynBytes = kMiscOff + 16 + 1024;
constexpr uint32_t kAccCols = 2 * kBN;             // two accumulators

struct GemmKArgs {
    int M, N, K;
    int n_sum, ksplit;
    int tiles_x, tiles_y, tiles_z;   // N tiles, M tiles, problems x K slices
    int batch_h, batch_b;            // independent products of the same shape (slowest index of the tile list)
    int64_t c_bs[2];                 // element strides of C over (h, b)
    int64_t ldc;
    int out_bf16;
    int tma_store;           // results leave through shared memory and a TMA store (needs 16-byte aligned rows)
    void* C[3];
    void* c_lo;              // second bf16 term of the (single) result, or null; its tensor map is tc1
    const float* bias[3];
    float* partial;          // [problem][slice][M][N] when ksplit > 1
    uint32_t* status;
};

// One tile of the work list of a CTA.
struct GemmTile {
    int m0, n0, problem, slice, kb_begin, kb_end, pair_begin, n_pairs, n_iters;
    int bh, bb;                      // batch entry
};
__device__ __forceinline__ GemmTile gemm_tile(const GemmKArgs& g, int linear) {
    GemmTile t;
    const int x = linear % g.tiles_x;
    const int yz = linear / g.tiles_x;
    const int y = yz % g.tiles_y, zw = yz / g.tiles_y;
    const int z = zw % g.tiles_z, w = zw / g.tiles_z;
    t.bh = w % g.batch_h;
    t.bb = w / g.batch_h;
    t.n0 = x * kBN;
    t.m0 = y * kBM;
    t.problem = z / g.ksplit;
    t.slice = z % g.ksplit;
    const int nkb = (g.K + kBK - 1) / kBK;
    const int per = (nkb + g.ksplit - 1) / g.ksplit;
    t.kb_begin = min(t.slice * per, nkb);
    t.kb_end = min(t.kb_begin + per, nkb);
    t.pair_begin = g.n_sum > 1 ? 0 : t.problem;
    t.n_pairs = g.n_sum > 1 ? g.n_sum : 1;
    t.n_iters = t.n_pairs * (t.kb_end - t.kb_begin);
    return t;
}

// Persistent: CTA c computes tiles c, c + gridDim.x, ... of the list (N tiles fastest, so neighbouring CTAs
// share their rows of A in L2).  The two accumulators alternate: while the epilogue warps read tile i out of
// tensor memory, convert it and hand it to the TMA store, the MMA thread is already accumulating tile i+1 and
// the producer is loading tile i+2's operands.
template <bool kAMn, bool kBMn>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_sm100_kernel(const __grid_constant__ CUtensorMap ta0, const __grid_constant__ CUtensorMap ta1,
                       const __grid_constant__ CUtensorMap ta2, const __grid_constant__ CUtensorMap tb0,
                       const __grid_constant__ CUtensorMap tb1, const __grid_constant__ CUtensorMap tb2,
                       const __grid_constant__ CUtensorMap tc0, const __grid_constant__ CUtensorMap tc1,
                       const __grid_constant__ CUtensorMap tc2, const GemmKArgs g) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + kBarOff;
    auto a_smem = [&](int s) { return smem_base + (uint32_t)(s * kStageBytes); };
    auto b_smem = [&](int s) { return smem_base + (uint32_t)(s * kStageBytes + kATileBytes); };
    auto bar_full = [&](int s) { return bar_base + 8u * s; };
    auto bar_empty = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto bar_acc_full = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
    auto bar_acc_empty = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem_gen + kMiscOff);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = g.tiles_x * g.tiles_y * g.tiles_z * g.batch_h * g.batch_b;
    LTCA_TRACE_DECL(blockIdx.x == 5 && g.tiles_z == LTCA_TRACE_GEMM_Z);
    LTCA_TRACE_EVT(0x01);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar_acc_full(b), 1); mbar_init(bar_acc_empty(b), 4); }
        misc[1] = 0u;
        mbar_fence_init();
    }
    if (warp == 1) { tmem_alloc(smem_u32(const_cast<uint32_t*>(&misc[0])), kAccCols); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = misc[0];
    const WaitCtx wc{&misc[1], g.status};
    LTCA_TRACE_EVT(0x02);
    // barriers and tensor memory are set up: the kernel after this one may place its CTAs; this one's operands are
    // complete once the kernel before it has ended
    grid_launch_dependents();
    grid_dependency_wait();

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&ta0);
            tma_prefetch_desc(&tb0);
            bool ok = true;
            int it = 0;
            for (int lin = blockIdx.x; lin < n_tiles && ok; lin += gridDim.x) {
                const GemmTile t = gemm_tile(g, lin);
                for (int p = 0; p < t.n_pairs && ok; ++p) {
                    const int pair = t.pair_begin + p;
                    const CUtensorMap* ta = pair == 0 ? &ta0 : (pair == 1 ? &ta1 : &ta2);
                    const CUtensorMap* tb = pair == 0 ? &tb0 : (pair == 1 ? &tb1 : &tb2);
                    for (int kb = t.kb_begin; kb < t.kb_end; ++kb, ++it) {
                        const int s = it % kStages;
                        ok = mbar_wait(bar_empty(s), (uint32_t)(((it / kStages) & 1) ^ 1), wc, 0xd0);
                        if (!ok) break;
                        LTCA_TRACE_EVT(0x10 + (it << 8));
                        mbar_arrive_expect_tx(bar_full(s), (uint32_t)kStageBytes);
                        const int k0 = kb * kBK;
                        if (kAMn) {
                            tma_load_4d(a_smem(s), ta, bar_full(s), t.m0, k0, t.bh, t.bb);
                            tma_load_4d(a_smem(s) + 8192, ta, bar_full(s), t.m0 + 64, k0, t.bh, t.bb);
                        } else {
                            tma_load_4d(a_smem(s), ta, bar_full(s), k0, t.m0, t.bh, t.bb);
                        }
                        if (kBMn) {
#pragma unroll
                            for (int pn = 0; pn < kBN / 64; ++pn)     // 64-column blocks of 64 K rows, 8 KB each
                                tma_load_4d(b_smem(s) + pn * 8192, tb, bar_full(s), t.n0 + 64 * pn, k0, t.bh, t.bb);
                        } else {
                            // 256 rows of 128 bytes, as two boxes of 128 rows
                            tma_load_4d(b_smem(s), tb, bar_full(s), k0, t.n0, t.bh, t.bb);
                            tma_load_4d(b_smem(s) + kBTileBytes / 2, tb, bar_full(s), k0, t.n0 + 128, t.bh, t.bb);
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_bf16(kBM, kBN, kAMn ? 1 : 0, kBMn ? 1 : 0);
            // K-major tile: 128 rows of 128 bytes, 8-row groups 1024 bytes apart, 32 bytes per K step.
            // MN-major tile: two blocks of 64 columns, 8192 bytes apart, each 64 K rows of 128 bytes;
            // a K step of 16 rows advances 2048 bytes.
            const uint64_t a_desc0 = kAMn ? make_smem_desc_sw128(a_smem(0), 8192, 1024)
                                          : make_smem_desc_sw128(a_smem(0), 16, 1024);
            const uint64_t b_desc0 = kBMn ? make_smem_desc_sw128(b_smem(0), 8192, 1024)
                                          : make_smem_desc_sw128(b_smem(0), 16, 1024);
            constexpr uint64_t a_step = kAMn ? 128 : 2, b_step = kBMn ? 128 : 2;
            bool ok = true;
            int it = 0, na = 0;                         // ring position; tiles that used an accumulator
            for (int lin = blockIdx.x; lin < n_tiles && ok; lin += gridDim.x) {
                const GemmTile t = gemm_tile(g, lin);
                if (t.n_iters == 0) continue;
                const int buf = na & 1;
                // the epilogue has read this accumulator's previous tile out
                ok = mbar_wait(bar_acc_empty(buf), (uint32_t)(((na >> 1) & 1) ^ 1), wc, 0xd3);
                if (!ok) break;
                LTCA_TRACE_EVT(0x20 + (na << 8));
                const uint32_t acc = tmem_base + (uint32_t)kBN * buf;
                for (int i = 0; i < t.n_iters && ok; ++i, ++it) {
                    const int s = it % kStages;
                    ok = mbar_wait(bar_full(s), (uint32_t)((it / kStages) & 1), wc, 0xd1);
                    if (!ok) break;
                    LTCA_TRACE_EVT(0x21 + (it << 8));
                    tc_fence_after_sync();
                    const uint64_t ad = a_desc0 + (uint64_t)((s * kStageBytes) >> 4);
                    const uint64_t bd = b_desc0 + (uint64_t)((s * kStageBytes) >> 4);
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k)
                        mma_ss(acc, ad + a_step * k, bd + b_step * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    mma_commit(bar_empty(s));
                }
                if (ok) mma_commit(bar_acc_full(buf));
                LTCA_TRACE_EVT(0x22 + (na << 8));
                ++na;
            }
        }
    } else {
        // epilogue: warp w reads the 32 accumulator rows of its lane quarter (w % 4)
        const int qd = warp & 3;
        const int row = qd * 32 + lane;
        uint8_t* stage = smem_gen + kOutOff;
        const uint32_t stage_addr = smem_base + kOutOff;
        const int box_cols = g.out_bf16 ? 64 : 32;
        bool ok = true;
        int na = 0, pc = 0;                                 // accumulators used; boxes staged
        for (int lin = blockIdx.x; lin < n_tiles; lin += gridDim.x) {
            const GemmTile t = gemm_tile(g, lin);
            const int gm = t.m0 + row;
            const int buf = na & 1;
            const bool have = t.n_iters > 0;
            if (have) {
                if (ok) ok = mbar_wait_warp(bar_acc_full(buf), (uint32_t)((na >> 1) & 1), wc, 0xd2);
                tc_fence_after_sync();
                LTCA_TRACE_EVT(0x30 + (na << 8));
                ++na;
            }
            const uint32_t tacc = tmem_base + (uint32_t)kBN * buf + ((uint32_t)(qd * 32) << 16);
            const float* bias = (g.ksplit == 1) ? g.bias[t.problem] : nullptr;
            const bool staged = g.tma_store && g.ksplit == 1;
            if (staged) {
                // The tile leaves box by box: 128 rows of 128 bytes (64 bf16 or 32 fp32 columns) go to shared memory
                // in the layout of a 128-byte swizzled TMA box and one thread stores the box; the tensor map clips
                // rows and columns past the end of C.  (Storing a row's 16-byte pieces straight from registers costs
                // 32 L1 wavefronts per instruction, about as many cycles per tile as its MMAs.)  The two boxes of the
                // staging area alternate, so a box is filled while the store of the one before it is still reading,
                // and the columns of the next box are on their way out of tensor memory while this one is converted.
                // With a second term the low-order part takes the second box and the boxes do not alternate.
                const int n_pieces = kBN / box_cols;
                const bool two = g.out_bf16 != 0;              // a bf16 box holds two 32-column loads
                uint32_t va0[32], va1[32], vb0[32], vb1[32];
                auto load_piece = [&](int pi, uint32_t (&x0)[32], uint32_t (&x1)[32]) {
                    if (have && ok) {
                        tmem_ld32(tacc + pi * box_cols, x0);
                        if (two) tmem_ld32(tacc + pi * box_cols + 32, x1);
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; ++c) x0[c] = x1[c] = 0u;
                    }
                };
                auto put_bf16 = [&](uint8_t* box, int ch0, const uint32_t (&v)[32]) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint4 w;
                        w.x = pack_bf16x2(__uint_as_float(v[8 * c + 0]), __uint_as_float(v[8 * c + 1]));
                        w.y = pack_bf16x2(__uint_as_float(v[8 * c + 2]), __uint_as_float(v[8 * c + 3]));
                        w.z = pack_bf16x2(__uint_as_float(v[8 * c + 4]), __uint_as_float(v[8 * c + 5]));
                        w.w = pack_bf16x2(__uint_as_float(v[8 * c + 6]), __uint_as_float(v[8 * c + 7]));
                        *reinterpret_cast<uint4*>(box + (((ch0 + c) ^ (row & 7)) << 4)) = w;
                        if (g.c_lo) {
                            uint4 l;
                            l.x = pack_bf16x2(__uint_as_float(v[8 * c + 0]) - __uint_as_float(w.x << 16),
                                              __uint_as_float(v[8 * c + 1]) - __uint_as_float(w.x & 0xffff0000u));
                            l.y = pack_bf16x2(__uint_as_float(v[8 * c + 2]) - __uint_as_float(w.y << 16),
                                              __uint_as_float(v[8 * c + 3]) - __uint_as_float(w.y & 0xffff0000u));
                            l.z = pack_bf16x2(__uint_as_float(v[8 * c + 4]) - __uint_as_float(w.z << 16),
                                              __uint_as_float(v[8 * c + 5]) - __uint_as_float(w.z & 0xffff0000u));
                            l.w = pack_bf16x2(__uint_as_float(v[8 * c + 6]) - __uint_as_float(w.w << 16),
                                              __uint_as_float(v[8 * c + 7]) - __uint_as_float(w.w & 0xffff0000u));
                            *reinterpret_cast<uint4*>(box + kBM * 128 + (((ch0 + c) ^ (row & 7)) << 4)) = l;
                        }
                    }
                };
                auto add_bias = [&](int gn0, uint32_t (&v)[32]) {
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        if (gn0 + c < g.N) v[c] = __float_as_uint(__uint_as_float(v[c]) + __ldg(bias + gn0 + c));
                };
                auto put_piece = [&](int pi, uint32_t (&x0)[32], uint32_t (&x1)[32]) {
                    const int gn0 = t.n0 + pi * box_cols;
                    if (bias) {
                        add_bias(gn0, x0);
                        if (two) add_bias(gn0 + 32, x1);
                    }
                    const int hb = g.c_lo ? 2 * (pc % (kStageBoxes / 2)) : pc % kStageBoxes;
                    // the box is free: the storing thread waits for the store that last read it before it comes here
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    uint8_t* box = stage + hb * (kBM * 128) + row * 128;
                    if (two) {
                        put_bf16(box, 0, x0);
                        put_bf16(box, 4, x1);
                    } else {
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            *reinterpret_cast<uint4*>(box + ((c ^ (row & 7)) << 4)) =
                                make_uint4(x0[4 * c], x0[4 * c + 1], x0[4 * c + 2], x0[4 * c + 3]);
                    }
                    LTCA_TRACE_EVT(0x31 + (pi << 8));
                    fence_proxy_async_smem();
                    asm volatile("bar.sync 1, 128;" ::: "memory");    // the four epilogue warps have staged their rows
                    if (warp == 2 && lane == 0) {
                        const CUtensorMap* tc = t.problem == 0 ? &tc0 : (t.problem == 1 ? &tc1 : &tc2);
                        if (gn0 < g.N) {
                            tma_store_4d(tc, stage_addr + hb * (kBM * 128), gn0, t.m0, t.bh, t.bb);
                            if (g.c_lo) tma_store_4d(&tc1, stage_addr + (hb + 1) * (kBM * 128), gn0, t.m0, t.bh, t.bb);
                        }
                        tma_store_commit();
                        // the box that the next piece takes has been read
                        if (g.c_lo) tma_store_wait_read<kStageBoxes / 2 - 1>();
                        else tma_store_wait_read<kStageBoxes - 1>();
                        LTCA_TRACE_EVT(0x32 + (pi << 8));
                    }
                    ++pc;
                };
                load_piece(0, va0, va1);
#pragma unroll 1
                for (int pi = 0; pi < n_pieces; pi += 2) {
                    tmem_wait_ld();
                    tmem_ld_fence(va0);
                    tmem_ld_fence(va1);
                    load_piece(pi + 1, vb0, vb1);
                    put_piece(pi, va0, va1);
                    tmem_wait_ld();
                    tmem_ld_fence(vb0);
                    tmem_ld_fence(vb1);
                    if (pi + 2 < n_pieces) {
                        load_piece(pi + 2, va0, va1);
                    } else if (have) {
                        // the accumulator is in registers: the MMA thread may start the tile after next in it
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_acc_empty(buf));
                    }
                    put_piece(pi + 1, vb0, vb1);
                }
                continue;
            }
            // Direct stores: split-K partials and results whose rows are not 16-byte aligned.
#pragma unroll 1
            for (int c0 = 0; c0 < kBN; c0 += 32) {
                uint32_t v[32];
                __syncwarp();
                if (have && ok) {
                    tmem_ld32(tacc + c0, v);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] = 0u;
                }
                if (have && c0 + 32 == kBN) {
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_acc_empty(buf));
                }
                const int gn0 = t.n0 + c0;
                if (bias) {
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        if (gn0 + c < g.N) v[c] = __float_as_uint(__uint_as_float(v[c]) + __ldg(bias + gn0 + c));
                }
                if (gm >= g.M || gn0 >= g.N) continue;
                const bool full = gn0 + 32 <= g.N;
                if (g.ksplit > 1) {
                    float* dst = g.partial + (((int64_t)t.problem * g.ksplit + t.slice) * g.M + gm) * g.N + gn0;
                    if (full && (g.N & 3) == 0) {
#pragma unroll
                        for (int c = 0; c < 32; c += 4)
                            *reinterpret_cast<uint4*>(dst + c) = make_uint4(v[c], v[c + 1], v[c + 2], v[c + 3]);
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; ++c)
                            if (gn0 + c < g.N) dst[c] = __uint_as_float(v[c]);
                    }
                } else if (g.out_bf16) {
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(g.C[t.problem]) + t.bh * g.c_bs[0] +
                                         t.bb * g.c_bs[1] + (int64_t)gm * g.ldc + gn0;
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        if (gn0 + c < g.N) dst[c] = __float2bfloat16_rn(__uint_as_float(v[c]));
                    if (g.c_lo) {
                        __nv_bfloat16* lo = reinterpret_cast<__nv_bfloat16*>(g.c_lo) + (dst -
                                            reinterpret_cast<__nv_bfloat16*>(g.C[t.problem]));
#pragma unroll
                        for (int c = 0; c < 32; ++c)
                            if (gn0 + c < g.N)
                                lo[c] = __float2bfloat16_rn(__uint_as_float(v[c]) - __bfloat162float(dst[c]));
                    }
                } else {
                    float* dst = reinterpret_cast<float*>(g.C[t.problem]) + t.bh * g.c_bs[0] + t.bb * g.c_bs[1] +
                                 (int64_t)gm * g.ldc + gn0;
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        if (gn0 + c < g.N) dst[c] = __uint_as_float(v[c]);
                }
            }
        }
        if (warp == 2 && lane == 0) tma_store_wait_read<0>();    // the staging area outlives its last store
    }

    LTCA_TRACE_EVT(0x3e);
    tc_fence_before_sync();
    __syncthreads();
    LTCA_TRACE_EVT(0x3f);
    if (warp == 1) {
        __syncwarp();
        if (misc[1]) __nanosleep(200000);    // aborted: give copies and MMAs in flight time to land
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kAccCols);
    }
}

#ifdef LTCA_TRACE
}  // namespace
}  // namespace ltca
extern "C" int ltca_trace_read_gemm(unsigned long long* events, unsigned int* counts) {
    if (cudaMemcpyFromSymbol(events, ltca::g_trace, sizeof(ltca::g_trace)) != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(counts, ltca::g_trace_count, sizeof(ltca::g_trace_count)) != cudaSuccess) return -1;
    return 0;
}
namespace ltca {
namespace {
#endif

// C[problem][i] = sum over slices of partial[problem][slice][i], in slice order.
__global__ void gemm_splitk_reduce_kernel(const float* __restrict__ partial, float* c0, float* c1, float* c2,
                                          int64_t mn, int ksplit) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int problem = blockIdx.y;
    float* c = problem == 0 ? c0 : (problem == 1 ? c1 : c2);
    const float* p = partial + (int64_t)problem * ksplit * mn;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < mn; i += (int64_t)gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < ksplit; ++s) acc += p[(int64_t)s * mn + i];
        c[i] = acc;
    }
}

__global__ void cvt_rows_bf16_kernel(const float* __restrict__ src, int64_t ld_src, __nv_bfloat16* __restrict__ dst,
                                     int64_t ld_dst, int64_t rows, int cols) {
    const int64_t n = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cols;
        const int c = (int)(i - r * cols);
        dst[r * ld_dst + c] = __float2bfloat16_rn(src[r * ld_src + c]);
    }
}

__global__ void cvt_rows_bf16_vec_kernel(const float4* __restrict__ src, uint2* __restrict__ dst, int64_t n4) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const float4 v = __ldg(src + i);
        dst[i] = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
    }
}

// Several matrices of any sizes in ONE launch (the activations and the weights of a module call): the 16-byte
// pieces of all of them form one index range that the grid strides over.
constexpr int kMaxCvtMany = 6;
struct CvtMany {
    const float* src[kMaxCvtMany];
    __nv_bfloat16* dst[kMaxCvtMany];
    __nv_bfloat16* lo[kMaxCvtMany];         // second term bf16(x - bf16(x)), laid out like dst, or null
    int64_t ld_src[kMaxCvtMany], ld_dst[kMaxCvtMany];
    uint32_t cols4[kMaxCvtMany];
    uint32_t start4[kMaxCvtMany + 1];       // first piece of matrix m; start4[n] = all pieces
    int n;
};
__global__ void cvt_many_bf16_kernel(const __grid_constant__ CvtMany b) {
    grid_launch_dependents();
    grid_dependency_wait();
    const uint32_t total = b.start4[b.n];
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        int m = 0;
        while (m + 1 < b.n && i >= b.start4[m + 1]) ++m;
        const uint32_t j = i - b.start4[m];
        const uint32_t r = j / b.cols4[m], c4 = j - r * b.cols4[m];
        const float4 v = __ldg(reinterpret_cast<const float4*>(b.src[m] + (int64_t)r * b.ld_src[m]) + c4);
        const uint2 h = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
        reinterpret_cast<uint2*>(b.dst[m] + (int64_t)r * b.ld_dst[m])[c4] = h;
        if (b.lo[m]) {
            const uint2 l = make_uint2(pack_bf16x2(v.x - __uint_as_float(h.x << 16), v.y - __uint_as_float(h.x & 0xffff0000u)),
                                       pack_bf16x2(v.z - __uint_as_float(h.y << 16), v.w - __uint_as_float(h.y & 0xffff0000u)));
            reinterpret_cast<uint2*>(b.lo[m] + (int64_t)r * b.ld_dst[m])[c4] = l;
        }
    }
}

int make_operand_map(ltca_ctx* ctx, CUtensorMap* map, const GemmOperand& o, int mn_extent, int k_extent,
                     int batch_h, int batch_b, const int64_t* bs) {
    ltca_strides st;
    st.batch = bs[1]; st.head = bs[0]; st.seq = o.ld;
    if (o.mn_major)   // stored [K, MN]: rows are K, 64 x 64 boxes
        return make_tmap_bhsd(ctx, map, o.ptr, 2, batch_b, batch_h, k_extent, mn_extent, st, 64, 64);
    return make_tmap_bhsd(ctx, map, o.ptr, 2, batch_b, batch_h, mn_extent, k_extent, st, 64, 128);
}

}  // namespace

size_t gemm_sm100_partial_bytes(int M, int N, int n_problems, int ksplit) {
    if (ksplit <= 1) return 0;
    return align_up((size_t)n_problems * ksplit * M * N * sizeof(float), 256);
}

int gemm_sm100_pick_ksplit(int M, int N, int K, int n_problems, int sm_count) {
    const int tiles = ((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN) * n_problems;
    const int nkb = (K + kBK - 1) / kBK;
    if (sm_count <= 0) sm_count = kPlanSms;
    int ks = 1;
    // split while the tiles alone leave most SMs idle and every slice keeps at least 8 K blocks
    while (tiles * ks * 2 <= sm_count && nkb / (ks * 2) >= 8 && ks < 16) ks *= 2;
    return ks;
}

int gemm_sm100(ltca_ctx* ctx, const GemmProblem& gp) {
    if (gp.n_problems < 1 || gp.n_problems > 3 || gp.n_sum < 1 || gp.n_sum > 3 ||
        (gp.n_sum > 1 && gp.n_problems != 1))
        return fail(ctx, LTCA_ERR_INVALID, "gemm: between 1 and 3 problems, or one problem of up to 3 summed pairs");
    if (gp.M < 1 || gp.N < 1 || gp.K < 1) return fail(ctx, LTCA_ERR_INVALID, "gemm: empty problem");
    const bool batched = gp.batch_h > 1 || gp.batch_b > 1;
    if (gp.batch_h < 1 || gp.batch_b < 1 || (batched && (gp.n_problems != 1 || gp.ksplit > 1)))
        return fail(ctx, LTCA_ERR_INVALID, "gemm: a batch takes one problem (or one sum of pairs) and no split of K");
    const int n_pairs = gp.n_sum > 1 ? gp.n_sum : gp.n_problems;
    CUtensorMap ta[3], tb[3];
    int rc;
    for (int i = 0; i < 3; ++i) {
        const int j = i < n_pairs ? i : 0;
        if (gp.a[j].mn_major != gp.a[0].mn_major || gp.b[j].mn_major != gp.b[0].mn_major)
            return fail(ctx, LTCA_ERR_INVALID, "gemm: all pairs of one launch share the operand forms");
        if ((rc = make_operand_map(ctx, &ta[i], gp.a[j], gp.M, gp.K, gp.batch_h, gp.batch_b, gp.a_bs))) return rc;
        if ((rc = make_operand_map(ctx, &tb[i], gp.b[j], gp.N, gp.K, gp.batch_h, gp.batch_b, gp.b_bs))) return rc;
    }
    GemmKArgs g;
    g.M = gp.M; g.N = gp.N; g.K = gp.K;
    g.n_sum = gp.n_sum;
    g.ksplit = gp.ksplit > 1 ? gp.ksplit : 1;
    g.ldc = gp.ldc;
    g.out_bf16 = gp.out_bf16;
    g.c_lo = gp.c_lo;
    if (gp.c_lo && (!gp.out_bf16 || gp.n_problems != 1 || gp.ksplit > 1))
        return fail(ctx, LTCA_ERR_INVALID, "gemm: a second result term needs one bf16 problem and no split of K");
    for (int i = 0; i < 3; ++i) { g.C[i] = gp.c[i < gp.n_problems ? i : 0]; g.bias[i] = i < gp.n_problems ? gp.bias[i] : nullptr; }
    g.partial = gp.partial;
    g.status = ctx->d_status;
    g.batch_h = gp.batch_h; g.batch_b = gp.batch_b;
    g.c_bs[0] = gp.c_bs[0]; g.c_bs[1] = gp.c_bs[1];
    const int ces = gp.out_bf16 ? 2 : 4;
    g.tma_store = (g.ksplit == 1 && ((gp.ldc * ces) % 16) == 0 && ((gp.c_bs[0] * ces) % 16) == 0 &&
                   ((gp.c_bs[1] * ces) % 16) == 0) ? 1 : 0;
    for (int i = 0; i < gp.n_problems && g.tma_store; ++i)
        if (reinterpret_cast<uintptr_t>(gp.c[i]) & 15) g.tma_store = 0;
    if (reinterpret_cast<uintptr_t>(gp.c_lo) & 15) g.tma_store = 0;
    CUtensorMap tc[3];
    memset(tc, 0, sizeof(tc));
    if (g.tma_store) {
        ltca_strides cs;
        cs.batch = gp.c_bs[1]; cs.head = gp.c_bs[0]; cs.seq = gp.ldc;
        for (int i = 0; i < 3; ++i) {
            const int j = i < gp.n_problems ? i : 0;
            void* dst = (i == 1 && gp.c_lo) ? gp.c_lo : gp.c[j];
            if ((rc = make_tmap_bhsd(ctx, &tc[i], dst, ces, gp.batch_b, gp.batch_h, gp.M, gp.N, cs,
                                     gp.out_bf16 ? 64 : 32, kBM))) return rc;
        }
    }
    if (g.ksplit > 1) {
        if (!gp.partial) return fail(ctx, LTCA_ERR_WORKSPACE, "gemm: split K needs scratch");
        if (gp.out_bf16) return fail(ctx, LTCA_ERR_INVALID, "gemm: split K writes fp32 results");
        for (int i = 0; i < gp.n_problems; ++i)
            if (gp.bias[i]) return fail(ctx, LTCA_ERR_INVALID, "gemm: split K takes no bias");
    }
    g.tiles_x = (gp.N + kBN - 1) / kBN;
    g.tiles_y = (gp.M + kBM - 1) / kBM;
    g.tiles_z = gp.n_problems * g.ksplit;
    const int64_t n_tiles = (int64_t)g.tiles_x * g.tiles_y * g.tiles_z * g.batch_h * g.batch_b;
    if (n_tiles > 0x7fffffff) return fail(ctx, LTCA_ERR_UNSUPPORTED, "gemm: too many tiles");
    const int sms = ctx->sm_count > 0 ? ctx->sm_count : kPlanSms;
    dim3 grid((unsigned)(n_tiles < sms ? n_tiles : sms));
    const bool amn = gp.a[0].mn_major != 0, bmn = gp.b[0].mn_major != 0;
    auto launch = [&](auto kern) -> int {
        LTCA_CUDA_OK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kDynBytes));
        LTCA_CUDA_OK(ctx, launch_dependent(kern, grid, dim3(kGemmThreads), kDynBytes, ctx->stream, ta[0], ta[1], ta[2], tb[0],
                                           tb[1], tb[2], tc[0], tc[1], tc[2], g));
        LTCA_LAUNCH_OK(ctx, "gemm_bf16_sm100_kernel");
        return LTCA_OK;
    };
    if (!amn && !bmn) rc = launch(gemm_bf16_sm100_kernel<false, false>);
    else if (!amn && bmn) rc = launch(gemm_bf16_sm100_kernel<false, true>);
    else if (amn && bmn) rc = launch(gemm_bf16_sm100_kernel<true, true>);
    else return fail(ctx, LTCA_ERR_UNSUPPORTED, "gemm: A stored [K, M] with B stored [N, K] is not built");
    if (rc) return rc;
    if (g.ksplit > 1) {
        const int64_t mn = (int64_t)gp.M * gp.N;
        dim3 rg((unsigned)((mn + 255) / 256 < 1184 ? (mn + 255) / 256 : 1184), gp.n_problems);
        LTCA_CUDA_OK(ctx, launch_dependent(gemm_splitk_reduce_kernel, rg, dim3(256), 0, ctx->stream, (const float*)gp.partial,
                                           reinterpret_cast<float*>(gp.c[0]),
                                           reinterpret_cast<float*>(gp.c[gp.n_problems > 1 ? 1 : 0]),
                                           reinterpret_cast<float*>(gp.c[gp.n_problems > 2 ? 2 : 0]), mn, g.ksplit));
        LTCA_LAUNCH_OK(ctx, "gemm_splitk_reduce_kernel");
    }
    return LTCA_OK;
}

int convert_rows_bf16(ltca_ctx* ctx, const float* src, int64_t ld_src, void* dst, int64_t ld_dst, int64_t rows,
                      int cols) {
    if (rows < 1 || cols < 1) return LTCA_OK;
    const int64_t n = rows * cols;
    if (ld_src == cols && ld_dst == cols && (n & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
        const int64_t n4 = n / 4;
        const unsigned blocks = (unsigned)((n4 + 255) / 256 < 2368 ? (n4 + 255) / 256 : 2368);
        cvt_rows_bf16_vec_kernel<<<blocks, 256, 0, ctx->stream>>>(reinterpret_cast<const float4*>(src),
                                                                  reinterpret_cast<uint2*>(dst), n4);
    } else {
        const unsigned blocks = (unsigned)((n + 255) / 256 < 2368 ? (n + 255) / 256 : 2368);
        cvt_rows_bf16_kernel<<<blocks, 256, 0, ctx->stream>>>(src, ld_src, reinterpret_cast<__nv_bfloat16*>(dst),
                                                              ld_dst, rows, cols);
    }
    LTCA_LAUNCH_OK(ctx, "cvt_rows_bf16_kernel");
    return LTCA_OK;
}


int convert_many_bf16(ltca_ctx* ctx, int n, const float* const* src, const int64_t* ld_src, void* const* dst,
                      const int64_t* ld_dst, const int64_t* rows, const int* cols, void* const* lo) {
    if (n < 1 || n > kMaxCvtMany) return fail(ctx, LTCA_ERR_INVALID, "convert_many_bf16 takes 1 to %d matrices", kMaxCvtMany);
    CvtMany b;
    memset(&b, 0, sizeof(b));
    b.n = 0;
    uint64_t total = 0;
    bool vec = true;
    for (int i = 0; i < n; ++i) {
        if (rows[i] < 1 || cols[i] < 1) continue;
        if (lo && lo[i]) vec = vec && (reinterpret_cast<uintptr_t>(lo[i]) & 7) == 0;
        if (!vec || (cols[i] & 3) || (ld_src[i] & 3) || (ld_dst[i] & 3) || (reinterpret_cast<uintptr_t>(src[i]) & 15) ||
            (reinterpret_cast<uintptr_t>(dst[i]) & 7)) {
            vec = false;
            break;
        }
        const int m = b.n++;
        b.src[m] = src[i]; b.dst[m] = reinterpret_cast<__nv_bfloat16*>(dst[i]);
        b.lo[m] = lo ? reinterpret_cast<__nv_bfloat16*>(lo[i]) : nullptr;
        b.ld_src[m] = ld_src[i]; b.ld_dst[m] = ld_dst[i];
        b.cols4[m] = (uint32_t)(cols[i] / 4);
        b.start4[m] = (uint32_t)total;
        total += (uint64_t)rows[i] * (uint64_t)(cols[i] / 4);
    }
    if (!vec || total >= (1ull << 31)) {
        // odd shapes or alignments: one matrix at a time
        for (int i = 0; i < n; ++i) {
            int rc;
            if (lo && lo[i]) rc = wide_split_bf16(ctx, src[i], ld_src[i], dst[i], lo[i], ld_dst[i], rows[i], cols[i]);
            else rc = convert_rows_bf16(ctx, src[i], ld_src[i], dst[i], ld_dst[i], rows[i], cols[i]);
            if (rc) return rc;
        }
        return LTCA_OK;
    }
    if (b.n == 0) return LTCA_OK;
    b.start4[b.n] = (uint32_t)total;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 2368 ? (total + 255) / 256 : 2368);
    LTCA_CUDA_OK(ctx, launch_dependent(cvt_many_bf16_kernel, dim3(blocks), dim3(256), 0, ctx->stream, b));
    LTCA_LAUNCH_OK(ctx, "cvt_many_bf16_kernel");
    return LTCA_OK;
}

}  // namespace ltca
