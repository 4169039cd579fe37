/*
 * ltc_attn.h -- C ABI of the B200 (sm_100a) attention path that replaces the attention
 * hot path of Sirius437/CUDA_LTC.
 *
 * The library is a plain C-ABI shared object (libltc_attn.so): pointers, sizes and status
 * codes only.  The C++ classes in ltc_attn_shim.hpp (cudatrader::FlashAttention,
 * cudatrader::TimeSelfAttention) are header-only wrappers over these entry points and keep
 * the reference's signatures.  Every entry point below names the reference interface it
 * replaces (paths are inside the reference project).
 *
 * General rules
 *   - All pointers are DEVICE pointers unless a comment says "host".
 *   - Outputs and workspace come from the caller (ltca_*_workspace_bytes tells how much); the
 *     only device allocation the library makes is the 4-byte status word of a context, made
 *     in ltca_ctx_create and released in ltca_ctx_destroy.  Work is enqueued on the context's
 *     stream; nothing synchronises the device unless stated.
 *   - Return value: 0 on success, a negative ltca_status otherwise; ltca_last_error() gives
 *     the text of the last failure on that context.  Nothing throws, prints or exits.
 *   - There is no CPU fallback: on a machine without an sm_100 GPU ltca_ctx_create fails.
 */
#ifndef LTC_ATTN_H_
#define LTC_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LTCA_VERSION 100

typedef enum {
    LTCA_OK              =  0,
    LTCA_ERR_INVALID     = -1,  /* bad argument (shape, null pointer, stride, alignment)      */
    LTCA_ERR_UNSUPPORTED = -2,  /* valid request outside what the kernels implement            */
    LTCA_ERR_CUDA        = -3,  /* a CUDA runtime/driver call failed                           */
    LTCA_ERR_WORKSPACE   = -4,  /* workspace missing or too small                              */
    LTCA_ERR_DEVICE      = -5,  /* a kernel reported a problem through its device status word  */
    LTCA_ERR_NO_DEVICE   = -6   /* no sm_100 device                                            */
} ltca_status;

/* Storage type of Q, K, V, O, dO, dQ, dK, dV. */
typedef enum { LTCA_F32 = 0, LTCA_BF16 = 1 } ltca_dtype;

/*
 * Arithmetic of the two contractions.
 *   LTCA_MODE_BF16 : bf16 operands on the tcgen05 tensor pipe, fp32 accumulation in tensor
 *                    memory, fp32 softmax.  fp32 storage is rounded to bf16 on the fly.  Head widths 64
 *                    (forward also 128) run on the streaming kernels; any other multiple of 8 runs through
 *                    written-out score matrices and batched tensor-pipe products (more workspace:
 *                    ltca_attn_workspace_bytes tells).
 *   LTCA_MODE_SPLIT: fp32 storage on the tensor pipe at fp32-class accuracy: Q, K, V, dO, the probabilities
 *                    and dS each travel as TWO bf16 terms (hi + lo, 16 significant bits - TF32 keeps 11) and
 *                    every contraction is evaluated as hi hi + hi lo + lo hi in one fp32 accumulator, through
 *                    written-out score matrices at every head width that is a multiple of 8.  Agreement with
 *                    an fp64 evaluation of the same fp32 inputs: 2e-5 + 2^-16 max|v| in the output, below 1e-5 in
 *                    relative L2 (tests/test_attn_gpu.py; the bf16 mode: 6e-3, the fp32 mode: 1e-6).  With
 *                    bf16 storage there are no low-order bits to keep and the mode equals LTCA_MODE_BF16.
 *                    The module entry points (ltca_tsa_*) treat it as LTCA_MODE_AUTO.
 *   LTCA_MODE_FP32 : fp32 FMA arithmetic end to end (the 1e-5 mode).
 *   LTCA_MODE_AUTO : BF16 when the streaming tensor-pipe kernels cover the shape, else FP32.
 */
typedef enum { LTCA_MODE_AUTO = 0, LTCA_MODE_BF16 = 1, LTCA_MODE_SPLIT = 2, LTCA_MODE_FP32 = 3 } ltca_mode;

typedef struct ltca_ctx ltca_ctx;

/* Element strides of a [batch, head, seq, head_dim] tensor; head_dim is contiguous.  This one
 * description covers the reference's [B,H,S,D] buffers (src/ml/flash_attention.cu:19-23) and
 * the un-permuted [B*S, H*D] projection outputs, so the reshape kernels
 * (src/ml/flash_attention.cu:402-455) are not needed. */
typedef struct {
    int64_t batch;
    int64_t head;
    int64_t seq;
} ltca_strides;

/*
 * One attention problem: O = softmax(mask(scale * Q K^T)) V per (batch, head).
 * Replaces the argument list of flashAttentionKernel / FlashAttention::flashAttention
 * (src/ml/flash_attention.cu:18-28, :994-1046; include/flash_attention.h:213-230).
 */
typedef struct {
    int32_t B, H, Sq, Sk, D;
    int32_t dtype;              /* ltca_dtype */
    int32_t mode;               /* ltca_mode */
    int32_t causal;             /* key j visible to query i iff j <= i + (Sk - Sq) */
    float   scale;              /* the reference uses 1/sqrt(D) (flash_attention.cu:998) */
    float   score_clamp;        /* > 0: s = min(s, score_clamp) after scaling; the reference
                                   clamps at 10 (flash_attention.cu:167).  <= 0: no clamp.  The gradient
                                   of a clamped score is zero: a score that lies within the mode's rounding
                                   of the threshold (1e-2 in the bf16 mode) can fall on either side of it,
                                   so with many scores AT the threshold the bf16 mode's gradients differ
                                   from an exact evaluation of unrounded inputs by whole terms */
    const void* q;  ltca_strides q_strides;    /* [B,H,Sq,D] */
    const void* k;  ltca_strides k_strides;    /* [B,H,Sk,D] */
    const void* v;  ltca_strides v_strides;    /* [B,H,Sk,D] */
    void*       o;  ltca_strides o_strides;    /* [B,H,Sq,D] */
    float*      lse;                           /* [B,H,Sq] natural-log sum-exp; required by
                                                  backward, may be NULL for forward only */
    const float*   keep_mask;   /* optional dense [B,Sq,Sk] fp32; value 0 hides the key
                                   (flash_attention.cu:161-164); NULL: none */
    const int32_t* kv_len;      /* optional [B]: keys j >= kv_len[b] are hidden; NULL: all Sk */
    /* backward only */
    const void* dout; ltca_strides do_strides; /* [B,H,Sq,D] */
    void* dq; ltca_strides dq_strides;         /* [B,H,Sq,D] */
    void* dk; ltca_strides dk_strides;         /* [B,H,Sk,D] */
    void* dv; ltca_strides dv_strides;         /* [B,H,Sk,D] */
    void*  workspace;           /* scratch, 256-byte aligned */
    size_t workspace_bytes;
    /* Backward on the tensor pipe with bf16 storage.  0 (default): one fused kernel forms dK, dV and dQ; the
     * key blocks' shares of dQ are added into an fp32 accumulator by the memory system in no fixed order, so
     * two runs can differ in dQ by fp32 rounding (dK and dV are bit-identical).  1: the two-kernel path, every
     * gradient bit-identical from run to run (the reference pins backward repeatability at 1e-6,
     * src/ml/time_self_attention_test.cu:799-838) at about 1.25 x the time for long sequences.  The workspace
     * size depends on it. */
    int32_t bwd_deterministic;
} ltca_attn_params;

/* ---- context ---------------------------------------------------------------------------- */

/* Binds a device and a stream (cudaStream_t passed as void*; NULL = default stream).
 * Replaces the per-object handle set-up of FlashAttention::FlashAttention
 * (src/ml/flash_attention.cu:485-549) and cudnn_ops::CuDNNHandle (include/cuDNN_ops.h:95-115). */
int ltca_ctx_create(int device, void* stream, ltca_ctx** out);
/* Rebinds the stream for the calls that follow.  A context is not thread-safe, and it keeps the work-item
 * counters of its persistent kernels: two launches of one context that overlap on the GPU (issued on two
 * streams with no ordering between them) would share those counters and corrupt each other.  Work that is
 * meant to overlap takes one context per stream; one process may hold contexts on several devices.
 * Stream order is kept: the kernels of a call are launched with programmatic stream serialisation, i.e. a kernel
 * may be placed on the GPU and set up its barriers while the kernel before it in the stream (this library's or the
 * caller's) is still running, but it touches no memory before that kernel has completed. */
int ltca_ctx_set_stream(ltca_ctx* ctx, void* stream);
void ltca_ctx_destroy(ltca_ctx* ctx);
/* Text of the last error on this context (host string, valid until the next call). */
const char* ltca_last_error(const ltca_ctx* ctx);
int ltca_version(void);

/* Optional timing of the kernels of the tensor-pipe backward (for benchmarks): when enabled,
 * ltca_attn_bwd records CUDA events on the context's stream around its three stages, and
 * ltca_ctx_last_bwd_kernel_ms waits for the last one and returns the durations in
 * milliseconds: ms_out[0] row statistics (delta, lse; plus the bf16 packing for fp32 storage, or the clearing of
 * the fused kernel's dQ accumulator), then for the fused backward ms_out[1] the fused kernel and ms_out[2] the
 * conversion of the dQ accumulator, for the two-kernel backward (bwd_deterministic, or fp32 storage) ms_out[1]
 * the dQ kernel and ms_out[2] the dK/dV kernel.  (No counterpart in the reference, whose
 * only timing is the per-stage event pair of ml::InferencePipeline::executeStage,
 * src/ml/ml_inference_pipeline.cu:42-80.) */
int ltca_ctx_enable_kernel_timing(ltca_ctx* ctx, int enable);
int ltca_ctx_last_bwd_kernel_ms(ltca_ctx* ctx, float* ms_out);

/* Reads and clears the device status word that kernels set when a bounded wait ran out or an
 * internal check failed.  Synchronises the context's stream.  0 = clean. */
int ltca_device_status(ltca_ctx* ctx, uint32_t* status_out);
/* Self-test of the bounded waits (no counterpart in the reference, whose only time limit,
 * InferencePipelineConfig::timeoutMs, is never read: include/inference_pipeline.h:28).  Launches one warp that
 * waits on a barrier nothing arrives at, with `limit_us` (1 .. 1 000 000) in place of the kernels' two seconds.
 * The kernel returns on its own; ltca_device_status then reports LTCA_ERR_DEVICE with the time-out bit
 * (status & 1) and barrier code 0x7f in bits 8..23, and the context stays usable. */
int ltca_selftest_bounded_wait(ltca_ctx* ctx, uint32_t limit_us);
/* The persistent kernels of this context launch one CTA per SM; n_sms caps that number so that other work
 * on the GPU (a communication library's copy kernels while slices are exchanged between GPUs) finds free SMs
 * at once instead of waiting for a whole kernel to end.  n_sms <= 0 or above the device's count restores the
 * default (all SMs).  Takes effect from the next launch. */
int ltca_ctx_set_sm_limit(ltca_ctx* ctx, int32_t n_sms);

/* ---- attention core --------------------------------------------------------------------- */

/* Scratch needed by ltca_attn_fwd (backward = 0) or ltca_attn_bwd (backward = 1). */
int ltca_attn_workspace_bytes(const ltca_attn_params* p, int backward, size_t* bytes_out);

/* 1 if the tensor-pipe (tcgen05) kernels cover this problem, 0 if it runs on the fp32 path. */
int ltca_attn_uses_tensor_pipe(const ltca_attn_params* p, int backward);

/* Forward.  Replaces flashAttentionKernel and its launch
 * (src/ml/flash_attention.cu:18-272, :994-1046). */
int ltca_attn_fwd(ltca_ctx* ctx, const ltca_attn_params* p);

/* Backward of the core: dQ, dK, dV from dO with recomputation of P from Q, K and lse.
 * The reference reaches this arithmetic through cudnnMultiHeadAttnBackwardData
 * (src/ml/cuDNN_ops.cu:240-337); FlashAttention itself has no backward. */
int ltca_attn_bwd(ltca_ctx* ctx, const ltca_attn_params* p);

/* Single-query step over a key/value cache: Sq must be 1, kv_len gives the live length of
 * each sequence.  The reference has no such call; the closest hook is the currIdx argument
 * of cudnnMultiHeadAttnForward, always -1 there (src/ml/cuDNN_ops.cu:206). */
int ltca_attn_decode(ltca_ctx* ctx, const ltca_attn_params* p);
/* Scratch needed by ltca_attn_decode: zero when batch x heads alone fills the GPU, otherwise
 * room for the partial results of the key-range split. */
int ltca_attn_decode_workspace_bytes(const ltca_attn_params* p, size_t* bytes_out);

/*
 * Decode step for callers that must not allocate.  (No counterpart in the reference.)
 *
 * Who needs it: code that runs where cudaMalloc is not an option -- a plug-in living inside
 * another framework's memory arena, a latency-critical loop that bans driver allocations once
 * it has started, a host process that has already handed out all device memory.  Such callers
 * can neither create an ltca_ctx (its creation allocates a status word) nor supply the scratch
 * buffer that the split over the key range wants.  This entry point takes no context, and the
 * split's partial results go to a 256 KiB array built into the library image (every GPU that
 * loads the library carries those 256 KiB until the process exits).  It calls no cudaMalloc,
 * cudaFree or any allocating routine.
 *
 *  - Works on the calling thread's CURRENT device and enqueues on `stream` (cudaStream_t as void*).
 *  - The first call on each device looks up the device address of the built-in array
 *    (cudaGetSymbolAddress); make that first call before starting any stream capture.
 *  - Shapes whose split scratch (ltca_attn_decode_workspace_bytes) exceeds 256 KiB are refused
 *    with LTCA_ERR_WORKSPACE and a message in `err`; nothing is launched.
 *  - All calls share the one array.  Each call overwrites every slot it later reads, so stale
 *    contents of an earlier call are harmless and nothing has to be cleared, but two calls
 *    that overlap on the GPU (different streams, no ordering between them) race on it.
 *  - Arguments as for ltca_attn_decode (Sq = 1; workspace fields of `p` are ignored).
 *    `err` (host buffer, may be NULL) receives the text of a failure.
 */
int ltca_attn_decode_static(void* stream, const ltca_attn_params* p, char* err, size_t err_len);

/* ---- TimeSelfAttention module ----------------------------------------------------------- */

/*
 * out = LayerNorm( x + MHA(x) ) as CuDNNTimeSelfAttention::forward computes it
 * (src/ml/cudnn_time_self_attention.cu:211-252) with the attention configured by
 * AttentionDescriptor::configure (include/cuDNN_ops.h:152-178).
 *
 * x, out, dy, dx : [rows = B*S, E] fp32.  Row r is (b, t): r = b*S + t, or r = t*B + b when
 * time_major is set (the order the reference gives cuDNN, include/cuDNN_ops.h:322-328).
 * wq, wk, wv : [E, H*W] row-major, y = x w.   wo : [H*W, E].   W = head_width:
 * E (reference-compatible, include/cuDNN_ops.h:166-169) or E/H (benchmark form).
 * Biases are optional (FlashAttention form, src/ml/flash_attention.cu:458-470).
 */
typedef struct {
    int32_t B, S, E, H;
    int32_t head_width;         /* W */
    int32_t causal;
    int32_t time_major;
    int32_t use_residual;       /* cudnn_time_self_attention.cu:240-243 */
    int32_t use_layer_norm;     /* cudnn_time_self_attention.cu:246-249, eps 1e-5 */
    int32_t mode;               /* ltca_mode for projections and attention */
    float   scale;              /* the reference passes 1.0 (cudnn_time_self_attention.cu:149) */
    float   score_clamp;
    const float* x;
    const float *wq, *wk, *wv, *wo;
    const float *bq, *bk, *bv, *bo;            /* optional */
    const float *ln_gamma, *ln_beta;           /* [E], required when use_layer_norm */
    const float*   keep_mask;                  /* optional [B,S,S], 0 hides */
    const int32_t* kv_len;                     /* optional [B] */
    float* out;                                /* forward output [rows, E] */
    /* backward */
    const float* dy;                           /* gradient at the module output; LayerNorm
                                                  and residual pass it through unchanged
                                                  (cudnn_time_self_attention.cu:291-299) */
    float* dx;                                 /* bwd_data output [rows, E] */
    float *dwq, *dwk, *dwv, *dwo;              /* bwd_weights outputs, overwritten
                                                  (CUDNN_WGRAD_MODE_SET, cuDNN_ops.cu:366-385) */
    void*  workspace;
    size_t workspace_bytes;
    /* FlashAttention form of the module (src/ml/flash_attention.cu:808-1150 of the reference):
     *   out = dropout( x + Wo·MHA(LayerNorm(x)) + bo )
     * i.e. LayerNorm on the INPUT (:822-834), residual with the raw input (:1107-1113), inverted dropout last
     * (:1117-1131).  Set pre_norm; use_layer_norm / use_residual then select those two steps, head_width is the
     * reference's head_dim, scale its 1/sqrt(head_dim) (:998), score_clamp its 10 (:167).  Zero keeps the
     * TimeSelfAttention form described above. */
    int32_t  pre_norm;
    float    dropout_prob;          /* 0 = none.  The keep decision of element i is a hash of (dropout_seed, i), */
    uint64_t dropout_seed;          /* so the backward pass regenerates the forward pass's mask. */
    /* optional outputs of the backward passes (the reference's FlashAttention has no backward; these complete it) */
    float *dbq, *dbk, *dbv, *dbo;   /* bias gradients [H*W], [H*W], [H*W], [E] */
    float *dgamma, *dbeta;          /* LayerNorm parameter gradients [E], pre_norm only */
    /* Optional: keep the forward's intermediates for the backward.  The reference's API carries nothing from
     * forward() to backward(), so its caller runs forward() again before every backward()
     * (src/ml/ml_liquid_net.cu:715-721) and the backward entry points here recompute it once more by default.
     * A caller that gives the SAME `saved` block (ltca_tsa_saved_bytes, 256-byte aligned) to ltca_tsa_fwd and
     * then, with x, the weights, the shape and the mode unchanged, to a backward call with reuse_forward = 1
     * skips that recomputation.  Not available with pre_norm.  With `saved` set the forward takes the pipeline
     * the backward will take. */
    void*   saved;
    size_t  saved_bytes;
    int32_t reuse_forward;
    /* Optional: keep the reduced-precision copies of the four weight matrices across calls.  The tensor-pipe
     * pipelines round wq, wk, wv, wo to bf16 (the materialised-score path also splits wq and wk into two terms)
     * at the start of every call; the reference's module never changes its projection weights after
     * construction or loadWeights (getParameters exposes the LayerNorm pair only,
     * src/ml/cudnn_time_self_attention.cu:436-450), so a caller can keep the copies.  With weight_cache set
     * (ltca_tsa_weight_cache_bytes, 256-byte aligned) a call with weight_cache_valid = 0 writes the copies there
     * and uses them; a call with weight_cache_valid = 1 uses them as they are and does not read wq..wo for the
     * projections.  The caller clears the flag whenever the weights, the shape, the head width or the mode
     * change.  Ignored by the exact pipeline. */
    void*   weight_cache;
    size_t  weight_cache_bytes;
    int32_t weight_cache_valid;
} ltca_tsa_params;

/* Size of the `saved` block for this shape and mode. */
int ltca_tsa_saved_bytes(const ltca_tsa_params* p, size_t* bytes_out);
/* Size of the `weight_cache` block for this shape and mode (0 where the call would not use one). */
int ltca_tsa_weight_cache_bytes(const ltca_tsa_params* p, size_t* bytes_out);

/* which: 0 forward, 1 backward-data, 2 backward-weights, 3 both backward passes. */
int ltca_tsa_workspace_bytes(const ltca_tsa_params* p, int which, size_t* bytes_out);
/* Replaces CuDNNTimeSelfAttention::forward (src/ml/cudnn_time_self_attention.cu:211-252). */
int ltca_tsa_fwd(ltca_ctx* ctx, const ltca_tsa_params* p);
/* Replaces CuDNNTimeSelfAttention::backward (src/ml/cudnn_time_self_attention.cu:254-302). */
int ltca_tsa_bwd_data(ltca_ctx* ctx, const ltca_tsa_params* p);
/* Replaces CuDNNTimeSelfAttention::backwardWeights (src/ml/cudnn_time_self_attention.cu:304-368). */
int ltca_tsa_bwd_weights(ltca_ctx* ctx, const ltca_tsa_params* p);
/* Both of the above in one pass (one recomputation of the forward instead of two); the order
 * backwardWeights-then-backward of the reference's training step
 * (src/ml/ml_liquid_net.cu:734-737) collapses into this call. */
int ltca_tsa_bwd(ltca_ctx* ctx, const ltca_tsa_params* p);

/* ---- small tensor helpers on the path ---------------------------------------------------- */

/* r = a + b, n fp32 elements.  Replaces cudatrader::addTensors (src/cuda_tensor_utils.cu:25-41). */
int ltca_add_tensors(ltca_ctx* ctx, const float* a, const float* b, float* r, size_t n);
/* Sequence sharding with key/value exchange (an extension: the reference is single-GPU and has no such
 * step).  A rank that holds a slice of the queries attends to one key/value shard at a time; each partial
 * result (o_blk [BH, n, D] contiguous, fp32 or bf16, with its natural-log sum-exp lse_blk [BH, n]) is
 * folded into fp32 accumulators o_acc [BH, S_acc, D], lse_acc [BH, S_acc] at rows s0 .. s0+n:
 *   lse' = log(exp(lse_acc) + exp(lse_blk)),  o_acc = o_acc e^(lse_acc - lse') + o_blk e^(lse_blk - lse').
 * Start from o_acc = 0, lse_acc = -inf.  Rows whose lse_blk is -inf leave the accumulator unchanged. */
int ltca_attn_merge(ltca_ctx* ctx, float* o_acc, float* lse_acc, const void* o_blk, int32_t blk_dtype,
                    const float* lse_blk, int64_t BH, int32_t S_acc, int32_t s0, int32_t n, int32_t D);
/* acc[bh][s0 + i][d] += part[bh][i][d]: partial dQ / dK / dV of one shard pair into fp32 accumulators
 * (acc [BH, S_acc, D] fp32, part [BH, n, D] contiguous, fp32 or bf16). */
int ltca_accumulate_rows(ltca_ctx* ctx, float* acc, const void* part, int32_t part_dtype, int64_t BH,
                         int32_t S_acc, int32_t s0, int32_t n, int32_t D);
/* In-place LayerNorm of [rows, E] fp32, biased variance, eps 1e-5.
 * Replaces applyLayerNorm / layerNormKernel (src/ml/cudnn_time_self_attention.cu:9-68, :496-508). */
int ltca_layer_norm(ltca_ctx* ctx, float* x, const float* gamma, const float* beta,
                    int64_t rows, int32_t E);
/* Sets *flag_out (device int) to 1 if any of n values is NaN or Inf, else 0.
 * Replaces validateGradientsKernel (src/cuda_tensor_utils.cu:14-22). */
int ltca_validate_finite(ltca_ctx* ctx, const float* x, size_t n, int32_t* flag_out);
/* fp32 <-> bf16 conversion of n elements (round to nearest even). */
int ltca_f32_to_bf16(ltca_ctx* ctx, const float* src, void* dst, size_t n);
int ltca_bf16_to_f32(ltca_ctx* ctx, const void* src, float* dst, size_t n);

#ifdef __cplusplus
}
#endif
#endif /* LTC_ATTN_H_ */
