// Internal interface of the materialised-score attention path (attn_wide_sm100.cu): attention on the tensor
// pipe for any head width that is a multiple of 8, built from batched launches of the tcgen05 GEMM.
#pragma once

#include "host_common.h"

namespace ltca {

// All matrices are bf16 views [batch, head, seq, width] given by element strides (multiples of 8).
struct WideArgs {
    int B = 0, H = 0, Sq = 0, Sk = 0, D = 0;
    int causal = 0;
    float scale = 1.f, clamp = 0.f;             // clamp <= 0: none
    const float* keep_mask = nullptr;           // dense [B, Sq, Sk], 0 hides
    const int32_t* kv_len = nullptr;            // [B]
    const void* qh = nullptr; const void* ql = nullptr;     // Q and, optionally, its low-order part
    const void* kh = nullptr; const void* kl = nullptr;
    const void* v = nullptr;
    const void* vl = nullptr;                   // optional low-order part of V (same strides): O = P V, dP = dO V^T
    ltca_strides qs{}, ks{}, vs{};              // and dK / dQ then run as three-term products as well
    void* o = nullptr; ltca_strides os{}; int o_bf16 = 1;   // forward result (null: probabilities only)
    float* lse = nullptr;                       // [B, H, Sq] natural-log sum-exp, optional
    float* scores = nullptr;                    // scratch fp32 [B*H, Sq, Skp]: raw Q K^T (kept for the backward's clamp test)
    void* P = nullptr;                          // scratch bf16 [B*H, Sq, Skp]: probabilities; the backward turns it into dS
    void* Plo = nullptr;                        // optional second term (p - bf16(p), later dS likewise) for fp32 results:
                                                // a single bf16 P would be the largest error left in an fp32 output
    // backward
    const void* dout = nullptr; ltca_strides dos{};
    const void* doutl = nullptr;                // optional low-order part of dO (same strides)
    void *dq = nullptr, *dk = nullptr, *dv = nullptr;
    ltca_strides dqs{}, dks{}, dvs{};
    int grads_bf16 = 1;
    float* dP = nullptr;                        // scratch fp32 [B*H, Sq, Skp]
    void* dS = nullptr;                         // optional bf16 [B*H, Sq, Skp] for dS (null: dS overwrites P, and Plo its
    void* dSlo = nullptr;                       // second term); with it the probabilities survive the backward
};

// hi[r, c] = bf16(src[r, c]), lo[r, c] = bf16(src[r, c] - hi[r, c]) (lo may be null); row pitches in elements.
int wide_split_bf16(ltca_ctx* ctx, const float* src, int64_t ld_src, void* hi, void* lo, int64_t ld_dst, int64_t rows,
                    int cols);
int wide_padded_keys(int Sk);                                  // row pitch of the score matrices (keys padded to 8)
size_t wide_matrix_elems(int B, int H, int Sq, int Sk);        // elements of one [B*H, Sq, Skp] scratch matrix
bool wide_supported(int D, const ltca_strides& qs, const ltca_strides& ks, const ltca_strides& vs);
// scores, probabilities (and lse), O = P V.
int wide_attn_fwd(ltca_ctx* ctx, const WideArgs& w);
// dQ, dK, dV from dO; expects `scores` and `P` as wide_attn_fwd left them for the same inputs.
int wide_attn_bwd(ltca_ctx* ctx, const WideArgs& w);

}  // namespace ltca
