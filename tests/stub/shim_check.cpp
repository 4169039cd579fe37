// Translation unit of the syntax check: the reference's headers (real or stand-in, chosen by the
// include path) followed by the shim, and one instantiation of everything the shim offers.
#include "cuda_resources.h"
#include "time_self_attention.h"
#include "ltc_attn_shim.hpp"

using namespace cudatrader;

std::unique_ptr<TimeSelfAttention> make(int e, int h) { return createB200TimeSelfAttention(e, h); }

CudaMemory<float> step_without_recomputation(B200TimeSelfAttention& tsa, const CudaMemory<float>& x,
                                             const CudaMemory<float>& dy, int B, int S) {
    tsa.setReuseForward(true);
    CudaMemory<float> y = tsa.forward(x, B, S);
    tsa.backwardWeights(dy, x, B, S);
    return tsa.backward(dy, x, B, S);
}

CudaMemory<float> step(TimeSelfAttention& tsa, const CudaMemory<float>& x, const CudaMemory<float>& dy, int B, int S) {
    CudaMemory<float> y = tsa.forward(x, B, S);
    tsa.backwardWeights(dy, x, B, S);
    CudaMemory<float> dx = tsa.backward(dy, x, B, S);
    tsa.initializeGradientStorage();
    (void)tsa.getParameters();
    (void)tsa.getComputedGradients();
    tsa.saveWeights("w.bin");
    tsa.loadWeights("w.bin");
    return dx;
}

CudaMemory<float> core(const b200::Context& c, const CudaMemory<float>& q, const CudaMemory<float>& k,
                       const CudaMemory<float>& v, CudaMemory<float>& lse) {
    return b200::flashAttention(c, q, k, v, 2, 8, 2, 16, nullptr, nullptr, &lse);
}

CudaMemory<float> flash_module(const CudaMemory<float>& x, const CudaMemory<float>& dy, const CudaMemory<float>& mask) {
    B200FlashAttention fa(32, 16, 2, 0.1f, true, true, false, 12345ULL);
    CudaMemory<float> y = fa.forward(x, 2, 8, &mask);
    fa.backwardWeights(dy, x, 2, 8, &mask);
    CudaMemory<float> dx = fa.backward(dy, x, 2, 8, &mask);
    (void)fa.getParameters();
    (void)fa.getComputedGradients();
    (void)fa.isTensorCoreOptimized();
    if (!fa.saveWeights("fa.bin") || !fa.loadWeights("fa.bin")) return y;
    (void)(fa.getNumHeads() + fa.getHeadDim() + fa.getInputDim() + fa.getModelDim());
    (void)(fa.getUseLayerNorm() && fa.getUseResidual() && fa.getDropoutProb() > 0.f);
    return dx;
}
