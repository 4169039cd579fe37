// Thin inline-PTX wrappers for the sm_100a features the attention kernels use:
// mbarrier, TMA tile loads (cp.async.bulk.tensor, never multicast), tensor memory
// (tcgen05.alloc/ld/st) and the 5th-generation tensor-core MMA (tcgen05.mma) with its
// shared-memory and instruction descriptors.
//
// Every wait is bounded: a wait that runs out records a code in a device status word, raises
// a CTA-wide abort flag in shared memory and returns false, so that a kernel always reaches
// its tear-down (tensor-memory release) and the context stays usable.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace ltca {

// ---- device status codes (bit flags in the context's status word) -------------------------
enum : uint32_t {
    kStatusWaitTimeout   = 1u << 0,   // a bounded mbarrier wait ran out
    kStatusBadTmemBase   = 1u << 1,   // tcgen05.alloc returned an unexpected base
    kStatusInternal      = 1u << 2,
    kStatusWhereShift    = 8          // bits [8,24): which barrier gave up (role-specific code)
};

static constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // 2 s
// (No suspend-time hint on mbarrier.try_wait and no sleep between polls: measured on B200, a hint more than
// doubles the latency between an arrival and the waiter's wake-up, and a back-off changed nothing.)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier -------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Shared by all roles of a CTA: the abort flag lives in shared memory, the status word in
// global memory (one per context).
struct WaitCtx {
    volatile uint32_t* abort_flag;   // shared memory
    uint32_t* status;                // global memory
    unsigned long long limit_ns = kWaitLimitNs;   // only the wait self-test passes a shorter one
};

// Bounded wait.  Returns false if the CTA aborted or the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& w,
                                          uint32_t where) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = 0;
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 0xffu) == 0) {
            if (*w.abort_flag) return false;
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > w.limit_ns) {
                *w.abort_flag = 1u;
                atomicOr(w.status, kStatusWaitTimeout | (where << kStatusWhereShift));
                return false;
            }
        }
    }
}

// Whole-warp wait: every lane polls (measured on B200: electing one lane to poll and
// broadcasting the outcome is slower than letting the 32 lanes poll together).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const WaitCtx& w,
                                               uint32_t where) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, w, where));
}

// ---- programmatic dependent launch -----------------------------------------------------------
// A kernel launched with the stream-serialisation attribute (launch_dependent, host_common.h) may start while the
// kernel before it in the stream is still running.  grid_dependency_wait() holds the thread until that kernel has
// completed and its writes are visible: everything that reads or writes global memory comes after it (it does
// nothing in a launch without the attribute).  grid_launch_dependents() lets the kernel AFTER this one start its
// CTAs as soon as every CTA of this one has called it (or exited).
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- TMA ------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// 4-d tile load global -> shared (this CTA), completion counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_4d(uint32_t smem_dst, const void* tmap, uint32_t bar,
                                            int32_t c0, int32_t c1, int32_t c2, int32_t c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar),
          "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// 4-d tile store shared -> global (bulk group completion).
__device__ __forceinline__ void tma_store_4d(const void* tmap, uint32_t smem_src,
                                             int32_t c0, int32_t c1, int32_t c2, int32_t c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_src),
          "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// 4-d tile reduce-add shared -> global (fp32 add performed by the memory system).
__device__ __forceinline__ void tma_reduce_add_4d(const void* tmap, uint32_t smem_src,
                                                  int32_t c0, int32_t c1, int32_t c2, int32_t c3) {
    asm volatile(
        "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group "
        "[%0, {%2, %3, %4, %5}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_src),
          "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 16-byte store to shared memory through a 32-bit shared-window address (half the address registers of a
// generic pointer).
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// ---- tensor memory ----------------------------------------------------------------------------
// Whole-warp calls.  `ncols` is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result_addr, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_result_addr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// Compiler-only fence (no instruction): placed after tmem_wait_ld() it ties the registers of an earlier tmem_ld32
// to this point of the program, so that no use of them is scheduled before the wait.
__device__ __forceinline__ void tmem_ld_fence(uint32_t (&r)[32]) {
    asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]));
}
__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 columns of 32-bit: thread t of the warp receives row (lane base + t),
// columns [col, col+32).  The address carries the warp's lane quarter in bits [16,32).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
          "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
          "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// 16-column variants (smaller register footprint per call).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15])
        : "memory");
}

// ---- tcgen05.mma ------------------------------------------------------------------------------
// Shared-memory matrix descriptor for 128-byte-swizzled tiles whose rows are 128 bytes
// (64 bf16 / 32 fp32) as TMA writes them with CU_TENSOR_MAP_SWIZZLE_128B:
//   bits [0,14)  start address >> 4      bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4 bits [46,48) version = 1 on sm_100
//   bits [61,64) layout type, 2 = SWIZZLE_128B
// K-major operand (the contraction index is contiguous in a row): stride offset = 1024 B between
// groups of 8 rows; the leading offset is not used by the hardware for swizzled K-major tiles.
// MN-major operand (the M/N index is contiguous): stride offset = 1024 B between groups of 8
// contraction rows; leading offset = distance between successive 64-element blocks along M/N.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// Instruction descriptor for kind::f16 with bf16 operands and fp32 accumulation:
//   bits [4,6) D format (1 = f32), [7,10) A format (1 = bf16), [10,13) B format (1 = bf16),
//   bit 15 A major (0 = K, 1 = MN), bit 16 B major, bits [17,23) N >> 3, bits [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
           (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
           (static_cast<uint32_t>(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same two instructions with shared-memory descriptors given by their LOW words only.  Every descriptor of
// the kernels has the same high word (stride offset 1024 B, version, 128-byte swizzle), and the start address and
// the leading offset live in the low word, so a thread that juggles many operands keeps 32-bit values and lets
// the assembler materialise the high word: half the registers and 32-bit address arithmetic.
constexpr uint32_t kSmemDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
    return ((smem_addr & 0x3ffffu) >> 4) | (((lbo_bytes >> 4) & 0x3fffu) << 16);
}
__device__ __forceinline__ void mma_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %5};\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kSmemDescHiSw128)
        : "memory");
}
__device__ __forceinline__ void mma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t}\n"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kSmemDescHiSw128)
        : "memory");
}
// Arrives once on `bar` when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
        ::"r"(bar) : "memory");
}

// ---- register reallocation between warpgroups ---------------------------------------------------
// Every warp of a warpgroup (4 consecutive warps) must execute the same call.  The data-movement
// and MMA-issue warps give registers up so that the elementwise warps can hold whole score rows.
template <int N>
__device__ __forceinline__ void reg_alloc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dealloc() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// ---- CTA order for causal work ----------------------------------------------------------------
// Thread blocks start in the order of their linear index.  The (batch, head) pairs are taken in
// groups of kSchedGroup; inside a group every pair's heaviest block starts first, then every
// pair's second heaviest, and so on, so the long blocks of a launch never start last (short
// tail), while one group's K / V / Q / dO (a few tens of MB) stay resident in L2.
constexpr int kSchedGroup = 16;
__device__ __forceinline__ void sched_block(int& rank, int& h, int& b) {
    const int nblk = gridDim.x, H = gridDim.y, BH = gridDim.y * gridDim.z;
    const int linear = blockIdx.x + nblk * (blockIdx.y + H * blockIdx.z);
    const int g = linear / (kSchedGroup * nblk);
    const int n_in = min(kSchedGroup, BH - g * kSchedGroup);
    const int local = linear - g * kSchedGroup * nblk;
    rank = local / n_in;
    const int bh = g * kSchedGroup + local % n_in;
    h = bh % H;
    b = bh / H;
}

// ---- work items of a persistent kernel ----------------------------------------------------------
// One CTA per SM takes work items from a global counter (list order = grouped heavy-first order,
// so greedy hand-out balances the SMs to within one light item).  The producer thread fetches the
// next item while the current one is still in flight and publishes it through a small shared-
// memory queue; every consumer (MMA threads: one arrival each, elementwise warps: one arrival per
// warp) reads the same sequence.  Item -1 ends the sequence.  The last CTA to finish puts the two
// counters back to zero, so the next launch needs no memset.
constexpr int kItemSlots = 4;
struct ItemQueue {
    uint32_t bar_full0, bar_empty0;      // kItemSlots barriers each, consecutive
    volatile int* slots;                 // shared memory, kItemSlots ints
    __device__ __forceinline__ uint32_t full(int nq) const { return bar_full0 + 8u * (nq % kItemSlots); }
    __device__ __forceinline__ uint32_t empty(int nq) const { return bar_empty0 + 8u * (nq % kItemSlots); }
    __device__ __forceinline__ uint32_t parity(int nq) const { return (uint32_t)((nq / kItemSlots) & 1); }
    // producer thread: returns the item (or -1), -2 if a wait gave up
    __device__ __forceinline__ int produce(int nq, int* counter, int n_items, const WaitCtx& w) const {
        if (!mbar_wait(empty(nq), parity(nq) ^ 1u, w, 0xfa)) return -2;
        int item = atomicAdd(counter, 1);
        if (item >= n_items) item = -1;
        slots[nq % kItemSlots] = item;
        mbar_arrive(full(nq));           // release: the slot is written before the arrival is seen
        return item;
    }
    // single consumer thread
    __device__ __forceinline__ int consume(int nq, const WaitCtx& w) const {
        if (!mbar_wait(full(nq), parity(nq), w, 0xfb)) return -2;
        const int item = slots[nq % kItemSlots];
        mbar_arrive(empty(nq));
        return item;
    }
    // whole consumer warp (one arrival)
    __device__ __forceinline__ int consume_warp(int nq, const WaitCtx& w) const {
        if (!mbar_wait_warp(full(nq), parity(nq), w, 0xfc)) return -2;
        const int item = slots[nq % kItemSlots];
        __syncwarp();
        if ((threadIdx.x & 31) == 0) mbar_arrive(empty(nq));
        return item;
    }
};
// Called by one thread per CTA at the very end: counters[0] = item counter, counters[1] = CTAs done.
__device__ __forceinline__ void item_counters_release(int* counters) {
    __threadfence();
    if (atomicAdd(counters + 1, 1) == (int)gridDim.x - 1) {
        counters[0] = 0;
        counters[1] = 0;
        __threadfence();
    }
}

// The item list of a persistent kernel: nblk row blocks for each of BH (batch, head) pairs.
// fold (forward kernel only): an item takes two tiles from the start and the two that mirror them at the end of the
// block range instead of four neighbours, see attn_fwd4p_sm100_kernel.
struct ItemGrid { int nblk, H, BH, n_items; int* counters; int fold = 0; };

// Entry `linear` of the grouped heavy-first order (see sched_block): rank 0 is the heaviest block.
__device__ __forceinline__ void sched_item(const ItemGrid& g, int linear, int& rank, int& h, int& b) {
    const int grp = linear / (kSchedGroup * g.nblk);
    const int n_in = min(kSchedGroup, g.BH - grp * kSchedGroup);
    const int local = linear - grp * kSchedGroup * g.nblk;
    rank = local / n_in;
    const int bh = grp * kSchedGroup + local % n_in;
    h = bh % g.H;
    b = bh / g.H;
}

// ---- small math helpers -----------------------------------------------------------------------
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

}  // namespace ltca
