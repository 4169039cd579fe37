// Internal interface of the tensor-pipe projection GEMM (gemm_sm100.cu).
#pragma once

#include "host_common.h"

namespace ltca {

// A bf16 matrix operand in HBM.  mn_major == 0: stored [M or N, K] (K contiguous);
// mn_major == 1: stored [K, M or N].  `ld` is the row pitch in elements, a multiple of 8.
struct GemmOperand {
    const void* ptr;
    int64_t ld;
    int mn_major;
};

// C_i[M,N] = A_i B_i (+ bias_i) for i < n_problems (n_sum == 1), or
// C_0[M,N] = sum_{p < n_sum} A_p B_p (+ bias_0)            (n_problems == 1).
struct GemmProblem {
    int M = 0, N = 0, K = 0;
    int n_problems = 1, n_sum = 1;
    int ksplit = 1;                 // > 1: K range cut into slices, summed in order from `partial`
    GemmOperand a[3] = {}, b[3] = {};
    void* c[3] = {nullptr, nullptr, nullptr};
    const float* bias[3] = {nullptr, nullptr, nullptr};
    int64_t ldc = 0;
    int out_bf16 = 0;               // result element type: bf16 or fp32
    void* c_lo = nullptr;           // with out_bf16, one problem, no split of K: also write bf16(x - bf16(x)) here,
                                    // laid out like C, so that C + c_lo carry 16 significant bits of the fp32 result
    float* partial = nullptr;       // gemm_sm100_partial_bytes() bytes when ksplit > 1
    // A grid of batch_h x batch_b independent products of the same shape (heads x sequences of the materialised
    // attention path): operand i of batch entry (h, b) starts h * bs[0] + b * bs[1] elements after its pointer.
    // Needs n_problems == 1 and ksplit == 1 (n_sum is allowed); strides must keep 16-byte alignment.
    int batch_h = 1, batch_b = 1;
    int64_t a_bs[2] = {0, 0}, b_bs[2] = {0, 0}, c_bs[2] = {0, 0};
};

int gemm_sm100(ltca_ctx* ctx, const GemmProblem& gp);
int gemm_sm100_pick_ksplit(int M, int N, int K, int n_problems, int sm_count);
size_t gemm_sm100_partial_bytes(int M, int N, int n_problems, int ksplit);
// dst[r, c] = bf16(src[r, c]) for a [rows, cols] block with row pitches ld_src / ld_dst (elements).
int convert_rows_bf16(ltca_ctx* ctx, const float* src, int64_t ld_src, void* dst, int64_t ld_dst, int64_t rows,
                      int cols);
// The same for up to six matrices of any sizes in one launch (16-byte aligned rows; otherwise one launch each).
// `lo` (or an entry of it) non-null: also the second term bf16(x - bf16(x)), laid out like the first.
int convert_many_bf16(ltca_ctx* ctx, int n, const float* const* src, const int64_t* ld_src, void* const* dst,
                      const int64_t* ld_dst, const int64_t* rows, const int* cols, void* const* lo = nullptr);

}  // namespace ltca
