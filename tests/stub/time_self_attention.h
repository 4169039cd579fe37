// Test stand-in for the reference header of the same name: the abstract interface
// cudatrader::TimeSelfAttention as the reference declares it
// (include/time_self_attention.h:19-165), for the syntax check of ltc_attn_shim.hpp.
#pragma once
#include <memory>
#include <string>
#include <vector>
#include "cuda_resources.h"
namespace cudatrader {
class TimeSelfAttention {
public:
    TimeSelfAttention(int input_dim, int num_heads, bool use_layer_norm = true, bool use_residual = true,
                      float dropout_rate = 0.0f, unsigned long long seed = 42);
    virtual ~TimeSelfAttention();
    virtual CudaMemory<float> forward(const CudaMemory<float>& x_seq, int batch_size, int seq_len,
                                      const CudaMemory<float>* mask = nullptr, cudaStream_t stream = nullptr) = 0;
    virtual void saveWeights(const std::string& filepath) = 0;
    virtual void loadWeights(const std::string& filepath) = 0;
    virtual CudaMemory<float> backward(const CudaMemory<float>& grad_output, const CudaMemory<float>& x_seq,
                                       int batch_size, int seq_len, const CudaMemory<float>* mask = nullptr,
                                       cudaStream_t stream = nullptr) = 0;
    virtual void backwardWeights(const CudaMemory<float>& grad_output, const CudaMemory<float>& x_seq,
                                 int batch_size, int seq_len, const CudaMemory<float>* mask = nullptr,
                                 cudaStream_t stream = nullptr) = 0;
    static std::unique_ptr<TimeSelfAttention> create(int input_dim, int num_heads, bool use_layer_norm = true,
                                                     bool use_residual = true, float dropout_rate = 0.0f,
                                                     unsigned long long seed = 42, bool force_legacy = false);
    virtual std::vector<CudaMemory<float>*> getParameters() = 0;
    virtual void initializeGradientStorage(cudaStream_t stream = nullptr) = 0;
    virtual std::vector<CudaMemory<float>*> getComputedGradients() = 0;
protected:
    int input_dim_;
    int num_heads_;
    bool use_layer_norm_;
    bool use_residual_;
    float dropout_rate_;
    unsigned long long seed_;
};
}  // namespace cudatrader
