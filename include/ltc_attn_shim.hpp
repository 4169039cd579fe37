// ltc_attn_shim.hpp -- header-only C++ binding of libltc_attn.so for the CUDA_LTC code base.
//
// Include it AFTER the reference's own headers "cuda_resources.h" and "time_self_attention.h"
// (it uses cudatrader::CudaMemory<float> and derives from cudatrader::TimeSelfAttention exactly
// as they are declared there, include/cuda_resources.h:531-770 and
// include/time_self_attention.h:19-165 of the reference).  It adds
//
//   cudatrader::B200TimeSelfAttention      a TimeSelfAttention whose forward / backward /
//                                          backwardWeights run on the sm_100a kernels,
//   cudatrader::createB200TimeSelfAttention the factory to call from TimeSelfAttention::create
//                                          (src/ml/time_self_attention.cu:41-56),
//   cudatrader::B200FlashAttention         the reference's FlashAttention module (same constructor, forward,
//                                          weight-file and getter signatures) plus a backward pass,
//   cudatrader::b200::flashAttention       the body of FlashAttention::flashAttention
//                                          (src/ml/flash_attention.cu:961-1046) on un-permuted
//                                          projection outputs, plus its backward.
//
// Error behaviour follows the reference: constructor argument errors are std::invalid_argument
// (src/ml/time_self_attention.cu:12-36), failures of the library are std::runtime_error (the type
// CHECK_CUDNN_ERROR throws, include/cuDNN_ops.h:42-49).  Nothing is swallowed.
#ifndef LTC_ATTN_SHIM_HPP_
#define LTC_ATTN_SHIM_HPP_

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <fstream>
#include <memory>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

#include "ltc_attn.h"

namespace cudatrader {

namespace b200 {

inline void check(ltca_ctx* ctx, int rc, const char* what) {
    if (rc != LTCA_OK)
        throw std::runtime_error(std::string(what) + ": " + (ctx ? ltca_last_error(ctx) : "no context"));
}

// One library context per (device, stream) user; the stream is rebound on every call because
// the reference passes it per call.
class Context {
public:
    explicit Context(int device = 0) {
        const int rc = ltca_ctx_create(device, nullptr, &ctx_);
        if (rc != LTCA_OK) throw std::runtime_error("ltca_ctx_create failed: no sm_100 device or CUDA error");
    }
    ~Context() { ltca_ctx_destroy(ctx_); }
    Context(const Context&) = delete;
    Context& operator=(const Context&) = delete;
    ltca_ctx* get(cudaStream_t stream) const {
        ltca_ctx_set_stream(ctx_, reinterpret_cast<void*>(stream));
        return ctx_;
    }
private:
    ltca_ctx* ctx_ = nullptr;
};

// Scaled-dot-product attention on projection outputs laid out [batch*seq, heads*head_dim]
// (batch-major rows), the layout FlashAttention::forward produces before its reshape kernels
// (src/ml/flash_attention.cu:866-958).  mask: optional dense [B,S,S] keep-mask, 0 hides
// (:161-164).  Returns [batch*seq, heads*head_dim]; `lse_out` (optional, [B,H,S]) receives the
// log-sum-exp needed by flashAttentionBackward.
inline CudaMemory<float> flashAttention(const Context& c, const CudaMemory<float>& query,
                                        const CudaMemory<float>& key, const CudaMemory<float>& value,
                                        int batch_size, int seq_len, int num_heads, int head_dim,
                                        const CudaMemory<float>* mask = nullptr, cudaStream_t stream = nullptr,
                                        CudaMemory<float>* lse_out = nullptr, float score_clamp = 10.0f) {
    const size_t n = (size_t)batch_size * seq_len * num_heads * head_dim;
    CudaMemory<float> out(n, stream);
    CudaMemory<float> ws;
    ltca_attn_params p = {};
    p.B = batch_size; p.H = num_heads; p.Sq = seq_len; p.Sk = seq_len; p.D = head_dim;
    p.dtype = LTCA_F32; p.mode = LTCA_MODE_AUTO; p.causal = 0;
    p.scale = 1.0f / std::sqrt((float)head_dim);                    // flash_attention.cu:998
    p.score_clamp = score_clamp;                                     // flash_attention.cu:167
    const ltca_strides st = {(int64_t)seq_len * num_heads * head_dim, (int64_t)head_dim,
                             (int64_t)num_heads * head_dim};
    p.q = query.get(); p.k = key.get(); p.v = value.get(); p.o = out.get();
    p.q_strides = p.k_strides = p.v_strides = p.o_strides = st;
    p.lse = lse_out ? lse_out->get() : nullptr;
    p.keep_mask = mask ? mask->get() : nullptr;
    size_t need = 0;
    ltca_attn_workspace_bytes(&p, 0, &need);
    if (need) { ws = CudaMemory<float>((need + 3) / 4, stream); p.workspace = ws.get(); p.workspace_bytes = need; }
    ltca_ctx* ctx = c.get(stream);
    check(ctx, ltca_attn_fwd(ctx, &p), "ltca_attn_fwd");
    return out;
}

// Gradients of flashAttention with respect to query, key and value (the reference's
// FlashAttention has no backward; this is the extension the attention path needs for training).
inline void flashAttentionBackward(const Context& c, const CudaMemory<float>& query,
                                   const CudaMemory<float>& key, const CudaMemory<float>& value,
                                   const CudaMemory<float>& out, const CudaMemory<float>& lse,
                                   const CudaMemory<float>& grad_out, CudaMemory<float>& grad_query,
                                   CudaMemory<float>& grad_key, CudaMemory<float>& grad_value,
                                   int batch_size, int seq_len, int num_heads, int head_dim,
                                   const CudaMemory<float>* mask = nullptr, cudaStream_t stream = nullptr,
                                   float score_clamp = 10.0f) {
    CudaMemory<float> ws;
    ltca_attn_params p = {};
    p.B = batch_size; p.H = num_heads; p.Sq = seq_len; p.Sk = seq_len; p.D = head_dim;
    p.dtype = LTCA_F32; p.mode = LTCA_MODE_AUTO; p.causal = 0;
    p.scale = 1.0f / std::sqrt((float)head_dim);
    p.score_clamp = score_clamp;
    const ltca_strides st = {(int64_t)seq_len * num_heads * head_dim, (int64_t)head_dim,
                             (int64_t)num_heads * head_dim};
    p.q = query.get(); p.k = key.get(); p.v = value.get(); p.o = out.get(); p.lse = lse.get();
    p.dout = grad_out.get(); p.dq = grad_query.get(); p.dk = grad_key.get(); p.dv = grad_value.get();
    p.q_strides = p.k_strides = p.v_strides = p.o_strides = st;
    p.do_strides = p.dq_strides = p.dk_strides = p.dv_strides = st;
    p.keep_mask = mask ? mask->get() : nullptr;
    size_t need = 0;
    ltca_attn_workspace_bytes(&p, 1, &need);
    if (need) { ws = CudaMemory<float>((need + 3) / 4, stream); p.workspace = ws.get(); p.workspace_bytes = need; }
    ltca_ctx* ctx = c.get(stream);
    check(ctx, ltca_attn_bwd(ctx, &p), "ltca_attn_bwd");
}

}  // namespace b200

// TimeSelfAttention on the sm_100a kernels.  `head_width` selects the arithmetic: input_dim
// reproduces the reference's cuDNN configuration (per-head projection width = input_dim, scale
// 1.0, no mask use, include/cuDNN_ops.h:152-178); input_dim / num_heads gives the compact form
// (scale 1/sqrt(head_dim)).  Rows are time-major, as the reference hands them to cuDNN
// (include/cuDNN_ops.h:322-328).
//
// The `mask` argument of forward / backward / backwardWeights is IGNORED by default, because the reference's
// module never reads it (src/ml/cudnn_time_self_attention.cu:211-237 passes no mask and a full attention window
// to cuDNN, src/ml/cuDNN_ops.cu:185-197) and its callers rely on that: its tests hand a 1 = keep / 0 = drop mask
// to forward and expect the unmasked result to stay finite (src/ml/time_self_attention_test.cu:452-457).
// setHonourMask(true) is the extension: the mask is then applied as a dense [B,S,S] keep-mask, 0 hides the key.
class B200TimeSelfAttention : public TimeSelfAttention {
public:
    B200TimeSelfAttention(int input_dim, int num_heads, bool use_layer_norm = true, bool use_residual = true,
                          float dropout_rate = 0.0f, unsigned long long seed = 42, bool compact_heads = false,
                          bool causal = false, int device = 0)
        : TimeSelfAttention(input_dim, num_heads, use_layer_norm, use_residual, dropout_rate, seed),
          ctx_(device),
          head_width_(compact_heads ? input_dim / num_heads : input_dim),
          scale_(compact_heads ? 1.0f / std::sqrt((float)(input_dim / num_heads)) : 1.0f),
          causal_(causal) {
        const size_t e = (size_t)input_dim_, hw = (size_t)num_heads_ * head_width_;
        wq_ = CudaMemory<float>(e * hw); wk_ = CudaMemory<float>(e * hw); wv_ = CudaMemory<float>(e * hw);
        wo_ = CudaMemory<float>(hw * e);
        ln_gamma_ = CudaMemory<float>(e); ln_beta_ = CudaMemory<float>(e);
        // Xavier-uniform in the reference's order Q, K, V, O from one mt19937(seed)
        // (src/ml/cuDNN_ops.cu:34-96): limit = sqrt(6 / (fan_in + fan_out)) of each matrix
        std::mt19937 gen((unsigned)seed_);
        auto fill = [&](CudaMemory<float>& w, size_t fan_in, size_t fan_out) {
            const float limit = std::sqrt(6.0f / (float)(fan_in + fan_out));
            std::uniform_real_distribution<float> dist(-limit, limit);
            std::vector<float> host(w.size());
            for (float& x : host) x = dist(gen);
            w.copyFromHost(host.data());
            cudaDeviceSynchronize();                  // `host` goes out of scope
        };
        fill(wq_, e, (size_t)head_width_); fill(wk_, e, (size_t)head_width_);
        fill(wv_, e, (size_t)head_width_); fill(wo_, (size_t)head_width_, e);
        std::vector<float> ones(e, 1.0f), zeros(e, 0.0f);
        ln_gamma_.copyFromHost(ones.data());
        ln_beta_.copyFromHost(zeros.data());
        cudaDeviceSynchronize();                      // the host vectors go out of scope
    }

    CudaMemory<float> forward(const CudaMemory<float>& x_seq, int batch_size, int seq_len,
                              const CudaMemory<float>* mask = nullptr, cudaStream_t stream = nullptr) override {
        CudaMemory<float> out((size_t)batch_size * seq_len * input_dim_, stream);
        ltca_tsa_params p = params(x_seq, batch_size, seq_len, mask);
        p.out = out.get();
        if (reuse_forward_) {
            size_t need = 0;
            b200::check(ctx_.get(stream), ltca_tsa_saved_bytes(&p, &need), "ltca_tsa_saved_bytes");
            if (need > saved_.bytes()) saved_ = CudaMemory<float>((need + 3) / 4, stream);
            p.saved = saved_.get();
            p.saved_bytes = saved_.bytes();
            saved_x_ = x_seq.get(); saved_mask_ = p.keep_mask; saved_b_ = batch_size; saved_s_ = seq_len;
        }
        run(p, 0, stream, ltca_tsa_fwd, "ltca_tsa_fwd");
        return out;
    }

    // forward() keeps its intermediates, and a backward() / backwardWeights() call for the same x_seq buffer, mask
    // and shape starts from them, as the reference's module does with cuDNN's reserve space
    // (src/ml/cudnn_time_self_attention.cu:254-302 hands the last forward's reserve_space_ to the backward calls;
    // its caller runs forward() right before them, src/ml/ml_liquid_net.cu:715-721).  Like there, the contents of
    // x_seq and the weights must not have changed in between; unlike there, a backward call for ANOTHER buffer,
    // mask or shape is noticed and recomputes the forward.  Off: every backward call recomputes.
    void setReuseForward(bool on) { reuse_forward_ = on; if (!on) saved_x_ = nullptr; }

    // Off (default): the mask argument is ignored, as in the reference.  On: dense keep-mask, 0 hides the key.
    void setHonourMask(bool on) { honour_mask_ = on; }

    // Extension.  The tensor-pipe pipelines round the four projection matrices to bf16 at the start of every
    // call.  With this switch on the copies are kept between calls; a caller that changes the matrices behind
    // the class's back (an optimizer working on getParameters()) calls weightsChanged() after every update.
    // loadWeights() does so itself.
    void setKeepWeightCopies(bool on) { keep_weight_copies_ = on; weight_copies_valid_ = false; }
    void weightsChanged() { weight_copies_valid_ = false; }

    CudaMemory<float> backward(const CudaMemory<float>& grad_output, const CudaMemory<float>& x_seq,
                               int batch_size, int seq_len, const CudaMemory<float>* mask = nullptr,
                               cudaStream_t stream = nullptr) override {
        CudaMemory<float> dx((size_t)batch_size * seq_len * input_dim_, stream);
        ltca_tsa_params p = params(x_seq, batch_size, seq_len, mask);
        p.dy = grad_output.get();
        p.dx = dx.get();
        attach_saved(p, x_seq, batch_size, seq_len);
        run(p, 1, stream, ltca_tsa_bwd_data, "ltca_tsa_bwd_data");
        return dx;
    }

    void backwardWeights(const CudaMemory<float>& grad_output, const CudaMemory<float>& x_seq,
                         int batch_size, int seq_len, const CudaMemory<float>* mask = nullptr,
                         cudaStream_t stream = nullptr) override {
        ensure_gradients(stream);
        ltca_tsa_params p = params(x_seq, batch_size, seq_len, mask);
        p.dy = grad_output.get();
        p.dwq = dwq_.get(); p.dwk = dwk_.get(); p.dwv = dwv_.get(); p.dwo = dwo_.get();
        attach_saved(p, x_seq, batch_size, seq_len);
        run(p, 2, stream, ltca_tsa_bwd_weights, "ltca_tsa_bwd_weights");
    }

    // LayerNorm scale and shift are the parameters the reference exposes
    // (src/ml/cudnn_time_self_attention.cu:436-450); the projection matrices follow them here so
    // that an optimizer can finally update them.
    std::vector<CudaMemory<float>*> getParameters() override {
        return {&ln_gamma_, &ln_beta_, &wq_, &wk_, &wv_, &wo_};
    }
    void initializeGradientStorage(cudaStream_t stream = nullptr) override {
        ensure_gradients(stream);
        dgamma_.memset(0, stream); dbeta_.memset(0, stream);
        dwq_.memset(0, stream); dwk_.memset(0, stream); dwv_.memset(0, stream); dwo_.memset(0, stream);
    }
    // gamma / beta gradients are zero placeholders, as in the reference
    // (src/ml/cudnn_time_self_attention.cu:357-364): LayerNorm is not differentiated there.
    std::vector<CudaMemory<float>*> getComputedGradients() override {
        ensure_gradients(nullptr);
        return {&dgamma_, &dbeta_, &dwq_, &dwk_, &dwv_, &dwo_};
    }

    // File layout: the reference's blob header (u32 0x43444E4E, u32 version, size_t byte count,
    // src/ml/cuDNN_ops.cu:391-420) followed by Wq, Wk, Wv [input_dim, heads * width] and Wo [heads * width,
    // input_dim] as fp32 row-major matrices, and `<path>.layernorm` with gamma then beta
    // (src/ml/cudnn_time_self_attention.cu:382-398).  In the reference's form (width = input_dim) this IS the
    // byte order of cuDNN's weight buffer on cuDNN 9.10: cudnnGetMultiHeadAttnWeights places the kinds Q, K, V, O
    // back to back and describes Q/K/V as [heads, width, input] with strides (width, 1, heads * width) and O as
    // [heads, output, width] with strides (output * width, 1, output), i.e. exactly those four row-major
    // matrices.  Files written by the reference's saveAttentionWeights therefore load here unchanged and files
    // written here load there, and since the constructor draws the matrices in that same order from one
    // mt19937(seed) with the reference's limits (src/ml/cuDNN_ops.cu:34-96), equal seeds give byte-identical
    // files.  A file of the compact form (width = input_dim / heads) has another byte count and is refused by
    // the other form.
    void saveWeights(const std::string& filepath) override {
        std::ofstream f(filepath, std::ios::binary);
        if (!f.is_open()) throw std::runtime_error("Failed to open file for writing: " + filepath);
        const uint32_t magic = 0x43444E4E, version = 1;
        const size_t nbytes = (wq_.size() + wk_.size() + wv_.size() + wo_.size()) * sizeof(float);
        f.write(reinterpret_cast<const char*>(&magic), sizeof(magic));
        f.write(reinterpret_cast<const char*>(&version), sizeof(version));
        f.write(reinterpret_cast<const char*>(&nbytes), sizeof(nbytes));
        for (const CudaMemory<float>* w : {&wq_, &wk_, &wv_, &wo_}) write_tensor(f, *w);
        if (f.fail()) throw std::runtime_error("Failed to write weights to file: " + filepath);
        std::ofstream g(filepath + ".layernorm", std::ios::binary);
        if (!g.is_open()) throw std::runtime_error("Failed to open file for writing: " + filepath + ".layernorm");
        write_tensor(g, ln_gamma_);
        write_tensor(g, ln_beta_);
    }
    void loadWeights(const std::string& filepath) override {
        std::ifstream f(filepath, std::ios::binary);
        if (!f.is_open()) throw std::runtime_error("Failed to open file for reading: " + filepath);
        uint32_t magic = 0, version = 0;
        size_t nbytes = 0;
        f.read(reinterpret_cast<char*>(&magic), sizeof(magic));
        f.read(reinterpret_cast<char*>(&version), sizeof(version));
        f.read(reinterpret_cast<char*>(&nbytes), sizeof(nbytes));
        const size_t want = (wq_.size() + wk_.size() + wv_.size() + wo_.size()) * sizeof(float);
        if (magic != 0x43444E4E || version != 1 || nbytes != want)
            throw std::runtime_error("Weight file does not match this module: " + filepath);
        for (CudaMemory<float>* w : {&wq_, &wk_, &wv_, &wo_}) read_tensor(f, *w);
        weight_copies_valid_ = false;
        if (f.fail()) throw std::runtime_error("Failed to read weights from file: " + filepath);
        std::ifstream g(filepath + ".layernorm", std::ios::binary);
        if (g.is_open()) { read_tensor(g, ln_gamma_); read_tensor(g, ln_beta_); }
    }

    int getHeadWidth() const { return head_width_; }

private:
    ltca_tsa_params params(const CudaMemory<float>& x, int B, int S, const CudaMemory<float>* mask) const {
        ltca_tsa_params p = {};
        p.B = B; p.S = S; p.E = input_dim_; p.H = num_heads_; p.head_width = head_width_;
        p.causal = causal_ ? 1 : 0;
        p.time_major = 1;
        p.use_residual = use_residual_ ? 1 : 0;
        p.use_layer_norm = use_layer_norm_ ? 1 : 0;
        p.mode = LTCA_MODE_AUTO;
        p.scale = scale_;
        p.x = x.get();
        p.wq = wq_.get(); p.wk = wk_.get(); p.wv = wv_.get(); p.wo = wo_.get();
        p.ln_gamma = ln_gamma_.get(); p.ln_beta = ln_beta_.get();
        p.keep_mask = (mask && honour_mask_) ? mask->get() : nullptr;
        return p;
    }
    void attach_saved(ltca_tsa_params& p, const CudaMemory<float>& x, int B, int S) const {
        if (!reuse_forward_ || saved_x_ != x.get() || saved_mask_ != p.keep_mask || saved_b_ != B || saved_s_ != S)
            return;
        p.saved = saved_.get();
        p.saved_bytes = saved_.bytes();
        p.reuse_forward = 1;
    }
    template <typename Fn>
    void run(ltca_tsa_params& p, int which, cudaStream_t stream, Fn fn, const char* what) {
        ltca_ctx* ctx = ctx_.get(stream);
        if (keep_weight_copies_) {              // before the workspace query: a call with a cache may take another pipeline
            size_t wneed = 0;
            b200::check(ctx, ltca_tsa_weight_cache_bytes(&p, &wneed), "ltca_tsa_weight_cache_bytes");
            if (wneed > weight_copies_.bytes()) {
                weight_copies_ = CudaMemory<float>((wneed + 3) / 4, stream);
                weight_copies_valid_ = false;
            }
            if (wneed) {
                p.weight_cache = weight_copies_.get();
                p.weight_cache_bytes = weight_copies_.bytes();
                p.weight_cache_valid = weight_copies_valid_ ? 1 : 0;
            }
        }
        size_t need = 0;
        ltca_tsa_workspace_bytes(&p, which, &need);
        if (need > workspace_.bytes()) workspace_ = CudaMemory<float>((need + 3) / 4, stream);
        p.workspace = workspace_.get();
        p.workspace_bytes = workspace_.bytes();
        b200::check(ctx, fn(ctx, &p), what);
        if (p.weight_cache) weight_copies_valid_ = true;
    }
    void ensure_gradients(cudaStream_t stream) {
        if (dwq_.size() == wq_.size() && dwq_.size() != 0) return;
        dwq_ = CudaMemory<float>(wq_.size(), stream); dwk_ = CudaMemory<float>(wk_.size(), stream);
        dwv_ = CudaMemory<float>(wv_.size(), stream); dwo_ = CudaMemory<float>(wo_.size(), stream);
        dgamma_ = CudaMemory<float>(ln_gamma_.size(), stream); dbeta_ = CudaMemory<float>(ln_beta_.size(), stream);
    }
    static void write_tensor(std::ofstream& f, const CudaMemory<float>& t) {
        std::vector<float> host(t.size());
        t.copyToHost(host.data());
        cudaDeviceSynchronize();
        f.write(reinterpret_cast<const char*>(host.data()), (std::streamsize)(host.size() * sizeof(float)));
    }
    static void read_tensor(std::ifstream& f, CudaMemory<float>& t) {
        std::vector<float> host(t.size());
        f.read(reinterpret_cast<char*>(host.data()), (std::streamsize)(host.size() * sizeof(float)));
        t.copyFromHost(host.data());
        cudaDeviceSynchronize();
    }

    b200::Context ctx_;
    int head_width_;
    float scale_;
    bool causal_;
    CudaMemory<float> wq_, wk_, wv_, wo_, ln_gamma_, ln_beta_;
    CudaMemory<float> dwq_, dwk_, dwv_, dwo_, dgamma_, dbeta_;
    CudaMemory<float> workspace_;
    bool reuse_forward_ = true;
    bool keep_weight_copies_ = false, weight_copies_valid_ = false;
    CudaMemory<float> weight_copies_;
    bool honour_mask_ = false;
    CudaMemory<float> saved_;
    const float* saved_x_ = nullptr;
    const float* saved_mask_ = nullptr;
    int saved_b_ = 0, saved_s_ = 0;
};

// The reference's FlashAttention module (include/flash_attention.h:19-260, src/ml/flash_attention.cu:485-1150)
// on the sm_100a kernels, with the constructor, forward, weight-file and getter signatures of that class:
//   out = dropout( x + Wo MHA(LayerNorm(x)) + bo ),  scale 1/sqrt(head_dim), scores clamped at 10,
//   optional dense keep-mask [B,S,S]; x is [batch*seq, input_dim] with batch-major rows.
// backward / backwardWeights are extensions with the signatures of TimeSelfAttention's
// (include/time_self_attention.h:84-106): the reference class is forward-only.
// Not reproduced: the reference swallows exceptions in forward and returns zeros
// (src/ml/flash_attention.cu:1058-1061, 1144-1147); failures here are std::runtime_error.  Dropout draws
// its mask from a hash of (seed, call counter, element index) instead of curand seeded with the wall clock
// (:1117-1131); backward(…) regenerates the mask of the latest forward call.
class B200FlashAttention {
public:
    B200FlashAttention(int input_dim, int head_dim, int num_heads, float dropout_prob = 0.0f,
                       bool use_layer_norm = true, bool use_residual = true, bool use_mixed_precision = false,
                       unsigned long long seed = 12345ULL, int device = 0)
        : ctx_(device), input_dim_(input_dim), head_dim_(head_dim), num_heads_(num_heads),
          model_dim_(head_dim * num_heads), dropout_prob_(dropout_prob), use_layer_norm_(use_layer_norm),
          use_residual_(use_residual), use_mixed_precision_(use_mixed_precision), seed_(seed) {
        if (input_dim <= 0 || head_dim <= 0 || num_heads <= 0)
            throw std::invalid_argument("FlashAttention: input_dim, head_dim and num_heads must be positive");
        if (dropout_prob < 0.0f || dropout_prob >= 1.0f)
            throw std::invalid_argument("FlashAttention: dropout_prob must be in [0, 1)");
        const size_t e = (size_t)input_dim_, m = (size_t)model_dim_;
        wq_ = CudaMemory<float>(e * m); wk_ = CudaMemory<float>(e * m); wv_ = CudaMemory<float>(e * m);
        wo_ = CudaMemory<float>(m * e);
        bq_ = CudaMemory<float>(m); bk_ = CudaMemory<float>(m); bv_ = CudaMemory<float>(m); bo_ = CudaMemory<float>(e);
        ln_gamma_ = CudaMemory<float>(e); ln_beta_ = CudaMemory<float>(e);
        initializeWeights(seed);
    }

    CudaMemory<float> forward(const CudaMemory<float>& x_seq, int batch_size, int seq_len,
                              const CudaMemory<float>* mask = nullptr, cudaStream_t stream = nullptr) {
        CudaMemory<float> out((size_t)batch_size * seq_len * input_dim_, stream);
        ++calls_;
        ltca_tsa_params p = params(x_seq, batch_size, seq_len, mask);
        p.out = out.get();
        run(p, 0, stream, ltca_tsa_fwd, "ltca_tsa_fwd");
        return out;
    }

    // Gradient with respect to x_seq of the latest forward call (same dropout mask).
    CudaMemory<float> backward(const CudaMemory<float>& grad_output, const CudaMemory<float>& x_seq,
                               int batch_size, int seq_len, const CudaMemory<float>* mask = nullptr,
                               cudaStream_t stream = nullptr) {
        CudaMemory<float> dx((size_t)batch_size * seq_len * input_dim_, stream);
        ltca_tsa_params p = params(x_seq, batch_size, seq_len, mask);
        p.dy = grad_output.get();
        p.dx = dx.get();
        run(p, 1, stream, ltca_tsa_bwd_data, "ltca_tsa_bwd_data");
        return dx;
    }

    // Gradients of every parameter, kept inside the object (getComputedGradients).
    void backwardWeights(const CudaMemory<float>& grad_output, const CudaMemory<float>& x_seq, int batch_size,
                         int seq_len, const CudaMemory<float>* mask = nullptr, cudaStream_t stream = nullptr) {
        ensure_gradients(stream);
        ltca_tsa_params p = params(x_seq, batch_size, seq_len, mask);
        p.dy = grad_output.get();
        p.dwq = dwq_.get(); p.dwk = dwk_.get(); p.dwv = dwv_.get(); p.dwo = dwo_.get();
        p.dbq = dbq_.get(); p.dbk = dbk_.get(); p.dbv = dbv_.get(); p.dbo = dbo_.get();
        if (use_layer_norm_) { p.dgamma = dgamma_.get(); p.dbeta = dbeta_.get(); }
        run(p, 2, stream, ltca_tsa_bwd_weights, "ltca_tsa_bwd_weights");
    }
    // Order: Wq, Wk, Wv, Wo, bq, bk, bv, bo, gamma, beta (the order of the weight file).
    std::vector<CudaMemory<float>*> getParameters() {
        return {&wq_, &wk_, &wv_, &wo_, &bq_, &bk_, &bv_, &bo_, &ln_gamma_, &ln_beta_};
    }
    std::vector<CudaMemory<float>*> getComputedGradients() {
        ensure_gradients(nullptr);
        return {&dwq_, &dwk_, &dwv_, &dwo_, &dbq_, &dbk_, &dbv_, &dbo_, &dgamma_, &dbeta_};
    }

    bool isTensorCoreOptimized() const {                       // src/ml/flash_attention.cu:613-615
        return (input_dim_ % 8 == 0) && (head_dim_ % 8 == 0) && (model_dim_ % 8 == 0);
    }

    // Xavier-uniform with one limit sqrt(6 / (input_dim + model_dim)), drawn from one mt19937(seed) in the
    // reference's order: (Wq[i], Wk[i], Wv[i]) interleaved, then Wo; biases zero, gamma one, beta zero
    // (src/ml/flash_attention.cu:548-611).
    void initializeWeights(unsigned long long seed = 12345ULL) {
        std::mt19937 gen((unsigned)seed);
        const size_t e = (size_t)input_dim_, m = (size_t)model_dim_;
        const float limit = std::sqrt(6.0f / (float)(input_dim_ + model_dim_));
        std::uniform_real_distribution<float> dist(-limit, limit);
        std::vector<float> q(e * m), k(e * m), v(e * m), o(m * e);
        for (size_t i = 0; i < e * m; ++i) { q[i] = dist(gen); k[i] = dist(gen); v[i] = dist(gen); }
        for (size_t i = 0; i < m * e; ++i) o[i] = dist(gen);
        std::vector<float> zm(m, 0.0f), ze(e, 0.0f), ones(e, 1.0f);
        wq_.copyFromHost(q.data()); wk_.copyFromHost(k.data()); wv_.copyFromHost(v.data()); wo_.copyFromHost(o.data());
        bq_.copyFromHost(zm.data()); bk_.copyFromHost(zm.data()); bv_.copyFromHost(zm.data()); bo_.copyFromHost(ze.data());
        ln_gamma_.copyFromHost(ones.data()); ln_beta_.copyFromHost(ze.data());
        cudaDeviceSynchronize();                      // the host vectors go out of scope
    }

    // The reference's file: input_dim, head_dim, num_heads, model_dim (int), dropout_prob (float),
    // use_layer_norm, use_residual (bool), then Wq, Wk, Wv, Wo, bq, bk, bv, bo and, with LayerNorm, gamma and
    // beta as fp32 (src/ml/flash_attention.cu:619-779).  Both return false on failure, as there.
    bool saveWeights(const std::string& path) const {
        std::ofstream f(path, std::ios::binary);
        if (!f.is_open()) return false;
        f.write(reinterpret_cast<const char*>(&input_dim_), sizeof(input_dim_));
        f.write(reinterpret_cast<const char*>(&head_dim_), sizeof(head_dim_));
        f.write(reinterpret_cast<const char*>(&num_heads_), sizeof(num_heads_));
        f.write(reinterpret_cast<const char*>(&model_dim_), sizeof(model_dim_));
        f.write(reinterpret_cast<const char*>(&dropout_prob_), sizeof(dropout_prob_));
        f.write(reinterpret_cast<const char*>(&use_layer_norm_), sizeof(use_layer_norm_));
        f.write(reinterpret_cast<const char*>(&use_residual_), sizeof(use_residual_));
        for (const CudaMemory<float>* w : {&wq_, &wk_, &wv_, &wo_, &bq_, &bk_, &bv_, &bo_}) write_tensor(f, *w);
        if (use_layer_norm_) { write_tensor(f, ln_gamma_); write_tensor(f, ln_beta_); }
        return !f.fail();
    }
    bool loadWeights(const std::string& path) {
        std::ifstream f(path, std::ios::binary);
        if (!f.is_open()) return false;
        int in = 0, hd = 0, nh = 0, md = 0;
        float dp = 0.0f;
        bool ln = false, res = false;
        f.read(reinterpret_cast<char*>(&in), sizeof(in));
        f.read(reinterpret_cast<char*>(&hd), sizeof(hd));
        f.read(reinterpret_cast<char*>(&nh), sizeof(nh));
        f.read(reinterpret_cast<char*>(&md), sizeof(md));
        f.read(reinterpret_cast<char*>(&dp), sizeof(dp));
        f.read(reinterpret_cast<char*>(&ln), sizeof(ln));
        f.read(reinterpret_cast<char*>(&res), sizeof(res));
        if (f.fail() || in != input_dim_ || hd != head_dim_ || nh != num_heads_ || md != model_dim_) return false;
        for (CudaMemory<float>* w : {&wq_, &wk_, &wv_, &wo_, &bq_, &bk_, &bv_, &bo_}) read_tensor(f, *w);
        if (use_layer_norm_ && ln) { read_tensor(f, ln_gamma_); read_tensor(f, ln_beta_); }
        return !f.fail();
    }

    int getNumHeads() const { return num_heads_; }
    int getHeadDim() const { return head_dim_; }
    bool getUseLayerNorm() const { return use_layer_norm_; }
    bool getUseResidual() const { return use_residual_; }
    int getInputDim() const { return input_dim_; }
    float getDropoutProb() const { return dropout_prob_; }
    int getModelDim() const { return model_dim_; }

private:
    ltca_tsa_params params(const CudaMemory<float>& x, int B, int S, const CudaMemory<float>* mask) const {
        ltca_tsa_params p = {};
        p.B = B; p.S = S; p.E = input_dim_; p.H = num_heads_; p.head_width = head_dim_;
        p.causal = 0;
        p.time_major = 0;                                          // rows are (batch, time), flash_attention.h:52
        p.pre_norm = 1;
        p.use_residual = use_residual_ ? 1 : 0;
        p.use_layer_norm = use_layer_norm_ ? 1 : 0;
        p.mode = LTCA_MODE_AUTO;
        p.scale = 1.0f / std::sqrt((float)head_dim_);              // flash_attention.cu:998
        p.score_clamp = 10.0f;                                     // flash_attention.cu:167
        p.dropout_prob = dropout_prob_;
        p.dropout_seed = (uint64_t)seed_ * 0x100000001B3ull + calls_;
        p.x = x.get();
        p.wq = wq_.get(); p.wk = wk_.get(); p.wv = wv_.get(); p.wo = wo_.get();
        p.bq = bq_.get(); p.bk = bk_.get(); p.bv = bv_.get(); p.bo = bo_.get();
        p.ln_gamma = ln_gamma_.get(); p.ln_beta = ln_beta_.get();
        p.keep_mask = mask ? mask->get() : nullptr;
        return p;
    }
    template <typename Fn>
    void run(ltca_tsa_params& p, int which, cudaStream_t stream, Fn fn, const char* what) {
        size_t need = 0;
        ltca_tsa_workspace_bytes(&p, which, &need);
        if (need > workspace_.bytes()) workspace_ = CudaMemory<float>((need + 3) / 4, stream);
        p.workspace = workspace_.get();
        p.workspace_bytes = workspace_.bytes();
        ltca_ctx* ctx = ctx_.get(stream);
        b200::check(ctx, fn(ctx, &p), what);
    }
    void ensure_gradients(cudaStream_t stream) {
        if (dwq_.size() == wq_.size() && dwq_.size() != 0) return;
        dwq_ = CudaMemory<float>(wq_.size(), stream); dwk_ = CudaMemory<float>(wk_.size(), stream);
        dwv_ = CudaMemory<float>(wv_.size(), stream); dwo_ = CudaMemory<float>(wo_.size(), stream);
        dbq_ = CudaMemory<float>(bq_.size(), stream); dbk_ = CudaMemory<float>(bk_.size(), stream);
        dbv_ = CudaMemory<float>(bv_.size(), stream); dbo_ = CudaMemory<float>(bo_.size(), stream);
        dgamma_ = CudaMemory<float>(ln_gamma_.size(), stream); dbeta_ = CudaMemory<float>(ln_beta_.size(), stream);
    }
    static void write_tensor(std::ofstream& f, const CudaMemory<float>& t) {
        std::vector<float> host(t.size());
        t.copyToHost(host.data());
        cudaDeviceSynchronize();
        f.write(reinterpret_cast<const char*>(host.data()), (std::streamsize)(host.size() * sizeof(float)));
    }
    static void read_tensor(std::ifstream& f, CudaMemory<float>& t) {
        std::vector<float> host(t.size());
        f.read(reinterpret_cast<char*>(host.data()), (std::streamsize)(host.size() * sizeof(float)));
        t.copyFromHost(host.data());
        cudaDeviceSynchronize();
    }

    b200::Context ctx_;
    int input_dim_, head_dim_, num_heads_, model_dim_;
    float dropout_prob_;
    bool use_layer_norm_, use_residual_, use_mixed_precision_;
    unsigned long long seed_;
    uint64_t calls_ = 0;
    CudaMemory<float> wq_, wk_, wv_, wo_, bq_, bk_, bv_, bo_, ln_gamma_, ln_beta_;
    CudaMemory<float> dwq_, dwk_, dwv_, dwo_, dbq_, dbk_, dbv_, dbo_, dgamma_, dbeta_;
    CudaMemory<float> workspace_;
};

// Returns nullptr when the machine has no sm_100 device, so that TimeSelfAttention::create can
// fall through to its existing branches.
inline std::unique_ptr<TimeSelfAttention> createB200TimeSelfAttention(int input_dim, int num_heads,
                                                                      bool use_layer_norm = true,
                                                                      bool use_residual = true,
                                                                      float dropout_rate = 0.0f,
                                                                      unsigned long long seed = 42) {
    try {
        return std::unique_ptr<TimeSelfAttention>(
            new B200TimeSelfAttention(input_dim, num_heads, use_layer_norm, use_residual, dropout_rate, seed));
    } catch (const std::invalid_argument&) {
        throw;                         // argument errors surface exactly as in the reference
    } catch (const std::runtime_error&) {
        return nullptr;
    }
}

}  // namespace cudatrader

#endif  // LTC_ATTN_SHIM_HPP_
