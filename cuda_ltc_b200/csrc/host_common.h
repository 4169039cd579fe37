// Host-side plumbing shared by the C-ABI translation units: the context object, error
// reporting, TMA tensor-map construction through the driver entry point, small helpers.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <utility>

#include "../../include/ltc_attn.h"

struct ltca_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 0;                 // SMs the persistent kernels spread over (ltca_ctx_set_sm_limit)
    int sm_device = 0;                // SMs of the device
    int cc_major = 0, cc_minor = 0;
    uint32_t* d_status = nullptr;     // device status word (allocated once at context creation)
    int* d_sched = nullptr;           // work-item counters of the persistent kernels (same allocation:
                                      // d_status + 4 .. ; two ints per kernel kind, kept at zero between launches)
    char err[512] = {0};
    // optional per-kernel timing of the backward pass (ltca_ctx_enable_kernel_timing)
    bool time_kernels = false;
    cudaEvent_t kev[4] = {nullptr, nullptr, nullptr, nullptr};
    int kev_recorded = 0;
};

namespace ltca {
// Marks a boundary between two kernels of the backward pass on the context's stream.
inline void kernel_timing_mark(ltca_ctx* ctx, int i) {
    if (ctx->time_kernels && i < 4 && ctx->kev[i]) {
        cudaEventRecord(ctx->kev[i], ctx->stream);
        ctx->kev_recorded = i + 1;
    }
}
}  // namespace ltca

namespace ltca {

inline int fail(ltca_ctx* ctx, int code, const char* fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

#define LTCA_CUDA_OK(ctx, expr)                                                             \
    do {                                                                                    \
        cudaError_t e__ = (expr);                                                           \
        if (e__ != cudaSuccess)                                                             \
            return ::ltca::fail((ctx), LTCA_ERR_CUDA, "%s failed: %s", #expr,               \
                                cudaGetErrorString(e__));                                   \
    } while (0)

#define LTCA_LAUNCH_OK(ctx, what)                                                           \
    do {                                                                                    \
        cudaError_t e__ = cudaGetLastError();                                               \
        if (e__ != cudaSuccess)                                                             \
            return ::ltca::fail((ctx), LTCA_ERR_CUDA, "launch of %s failed: %s", (what),    \
                                cudaGetErrorString(e__));                                   \
    } while (0)

// The opt-in to more than 48 KB of dynamic shared memory (cudaFuncSetAttribute) is a property of a kernel ON ONE
// DEVICE, so a process-wide "already done" flag would leave the second GPU of a process without it.  One bit per
// device and call site; two threads that race only repeat the call.
struct SmemOptIn { std::atomic<uint64_t> done{0}; };
template <typename Kernel>
inline cudaError_t opt_in_dynamic_smem(SmemOptIn& once, int device, Kernel kernel, int bytes) {
    const uint64_t bit = (device >= 0 && device < 64) ? (1ull << device) : 0ull;
    if (bit && (once.done.load(std::memory_order_acquire) & bit)) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess && bit) once.done.fetch_or(bit, std::memory_order_release);
    return e;
}

// SM count that size queries plan for.  Split counts (decode key ranges, the contraction of the weight-gradient
// products) fix how much scratch a call needs, and the size queries have no context to ask the device, so the plan
// is a function of the problem alone, laid out for the B200's 148 SMs.  Launch widths always come from the context.
constexpr int kPlanSms = 148;

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline int elem_size(int dtype) { return dtype == LTCA_BF16 ? 2 : 4; }

// cuTensorMapEncodeTiled fetched at run time, so the library links against the CUDA runtime only.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
                cudaSuccess || q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Tensor map over a [batch, head, seq, dim] tensor (dim contiguous) with a (box_dim x box_rows)
// tile, 128-byte swizzle.  `es` is the element size in bytes (2 = bf16, 4 = fp32).
inline int make_tmap_bhsd(ltca_ctx* ctx, CUtensorMap* map, const void* base, int es,
                          int B, int H, int S, int D, const ltca_strides& st,
                          int box_dim, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(ctx, LTCA_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
        return fail(ctx, LTCA_ERR_INVALID, "tensor base must be 16-byte aligned for TMA");
    const int64_t sb = st.batch * es, sh = st.head * es, ss = st.seq * es;
    if ((ss & 15) || (H > 1 && (sh & 15)) || (B > 1 && (sb & 15)))
        return fail(ctx, LTCA_ERR_INVALID, "tensor strides must be multiples of 16 bytes for TMA");
    cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
    // a stride of an extent-1 dimension is never used for addressing, but must still be valid
    cuuint64_t strides[3] = {(cuuint64_t)ss, (cuuint64_t)(H > 1 ? sh : ss * S),
                             (cuuint64_t)(B > 1 ? sb : (H > 1 ? sh * H : ss * S))};
    for (int i = 0; i < 3; ++i)
        if (strides[i] == 0 || (strides[i] & 15)) strides[i] = 16;
    cuuint32_t box[4] = {(cuuint32_t)box_dim, (cuuint32_t)box_rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, es == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                    4, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(ctx, LTCA_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return LTCA_OK;
}

}  // namespace ltca

// Launch with programmatic stream serialisation: the kernel's CTAs may be placed while the kernel before it in the
// stream is still running; the kernel itself waits (grid_dependency_wait) before it touches global memory.
namespace ltca {
// `dependent` false: an ordinary launch.  The attention-core kernels take it for large problems: there every launch
// runs for hundreds of microseconds, the set-up it could hide is nothing beside that, and with all four launches
// of a step dependent the step measured 3 % slower at the bench workload (1.47 against 1.43 ms) - while for short
// launches (the module at config 2, the core up to a few hundred (batch, head) pairs of a few hundred positions)
// the hidden set-up is a tenth of the call.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent_if(bool dependent, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                       cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
    return launch_dependent_if(true, kern, grid, block, smem, stream, std::forward<Args>(args)...);
}
// the attention-core launches of a call are dependent launches up to this many (batch, head, position) rows
constexpr int64_t kDependentLaunchRows = 131072;
inline bool small_attention_call(const ltca_attn_params* p) {
    return (int64_t)p->B * p->H * (p->Sq > p->Sk ? p->Sq : p->Sk) <= kDependentLaunchRows;
}
}  // namespace ltca

// Kernel launchers implemented in the .cu files of this directory (internal, not exported).
namespace ltca {
int launch_attn_fwd_sm100(ltca_ctx* ctx, const ltca_attn_params* p);
bool attn_fwd_sm100_supported(const ltca_attn_params* p);
int launch_attn_bwd_sm100(ltca_ctx* ctx, const ltca_attn_params* p);
bool attn_bwd_sm100_supported(const ltca_attn_params* p);
size_t attn_bwd_sm100_workspace(const ltca_attn_params* p);
int launch_attn_fwd_fp32(ltca_ctx* ctx, const ltca_attn_params* p);
int launch_attn_bwd_fp32(ltca_ctx* ctx, const ltca_attn_params* p);
size_t attn_bwd_fp32_workspace(const ltca_attn_params* p);
int launch_attn_decode(ltca_ctx* ctx, const ltca_attn_params* p);
size_t attn_decode_workspace(const ltca_attn_params* p);

// Strided fp32 [B,H,S,D] tensors -> contiguous bf16 copies, up to four tensors in ONE launch (capi.cu).  With a
// non-null `lo` the low-order term goes there as well: dst = bf16(x), lo = bf16(x - dst).
struct PackJob {
    const void* src;
    ltca_strides st;
    void* dst;
    int S;
    void* lo = nullptr;
};
constexpr int kMaxPackJobs = 4;
int pack_many_to_bf16(ltca_ctx* ctx, const PackJob* jobs, int count, int B, int H, int D);
}  // namespace ltca
