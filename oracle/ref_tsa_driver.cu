// ref_tsa_driver.cu -- TEST INFRASTRUCTURE.  Drives the reference's OWN TimeSelfAttention
// (the cuDNN legacy multi-head-attention wrapper, src/ml/cudnn_time_self_attention.cu), linked
// from reference objects compiled where they lie (see the Makefile in this directory; nothing
// is copied).  It needs a GPU: it is built in advance, run once on a B200, and what it dumps
// becomes the golden vectors that pin the module oracle.
//
//   ref_tsa_driver dump <outdir>
//       For a list of seeded cases: create the module through TimeSelfAttention::create, run
//       forward and backward, save its weights through its own saveWeights, then read the four
//       projection matrices out of that blob exactly as the reference does
//       (cudnnGetMultiHeadAttnWeights + cudnnGetTensorNdDescriptor, src/ml/cuDNN_ops.cu:54-70)
//       and write x, dy, the matrices (with their dims and strides), out and dx as raw float32
//       plus a manifest.  The weight gradients come next: the reference class keeps them in a private byte
//       buffer that no accessor returns (src/ml/cudnn_time_self_attention.cu:340-356, :474-493), so this
//       file includes that source file textually (path given by the Makefile, nothing is copied) with its
//       `private:` sections opened, calls initializeGradientStorage + backwardWeights after backward (the
//       order cuDNN documents: weight gradients after data gradients) and dumps the buffer, whose layout is
//       the weight buffer's (same descriptors, src/ml/cuDNN_ops.cu:366-385).  The module's own weight file
//       is kept too (w<i>.bin): it is what saveWeights of the reference writes.
#include <cudnn.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <random>
#include <string>
#include <vector>

#include <iostream>
#include <memory>
#include <stdexcept>

#include "cuda_resources.h"
#include "time_self_attention.h"
#include "cuDNN_ops.h"

// every standard header the included file uses is already in; only its own class is affected
#define private public
#include REF_CUDNN_TSA_CU
#undef private

using namespace cudatrader;

namespace {

std::vector<float> random_tensor(size_t n, unsigned seed) {     // the reference tests' recipe
    std::mt19937 gen(seed);
    std::uniform_real_distribution<float> dist(-1.0f, 1.0f);
    std::vector<float> v(n);
    for (auto& x : v) x = dist(gen);
    return v;
}

void dump(const std::string& path, const float* p, size_t n) {
    FILE* f = fopen(path.c_str(), "wb");
    if (!f) { fprintf(stderr, "cannot write %s\n", path.c_str()); exit(2); }
    fwrite(p, sizeof(float), n, f);
    fclose(f);
}

struct Case { int E, H, B, S; bool ln, res; unsigned seed; };

}  // namespace

int main(int argc, char** argv) {
    if (argc < 3 || strcmp(argv[1], "dump") != 0) {
        fprintf(stderr, "usage: ref_tsa_driver dump <outdir>\n");
        return 1;
    }
    const std::string out = argv[2];
    const Case cases[] = {
        {8, 2, 2, 4, false, false, 42},          // the reference's backward fixture (time_self_attention_test.cu:659-709)
        {6, 2, 1, 3, false, false, 43},
        {64, 2, 2, 16, true, true, 12345},       // the reference's main fixture (:134-147)
        {64, 1, 1, 8, false, true, 7},
        {128, 4, 4, 32, true, false, 99},
    };
    FILE* mf = fopen((out + "/manifest.txt").c_str(), "w");
    int idx = 0;
    for (const Case& c : cases) {
        try {
            auto tsa = TimeSelfAttention::create(c.E, c.H, c.ln, c.res, 0.0f, c.seed);
            const size_t n = (size_t)c.B * c.S * c.E;
            std::vector<float> hx = random_tensor(n, c.seed + 1000), hdy = random_tensor(n, c.seed + 2000);
            CudaMemory<float> x(n), dy(n);
            x.copyFromHost(hx.data());
            dy.copyFromHost(hdy.data());
            cudaDeviceSynchronize();
            CudaMemory<float> y = tsa->forward(x, c.B, c.S);
            cudaDeviceSynchronize();
            std::vector<float> hy(n), hdx(n);
            y.copyToHost(hy.data());
            cudaDeviceSynchronize();
            bool have_dx = true;
            try {
                CudaMemory<float> dx = tsa->backward(dy, x, c.B, c.S);
                cudaDeviceSynchronize();
                dx.copyToHost(hdx.data());
                cudaDeviceSynchronize();
            } catch (const std::exception& e) {
                fprintf(stderr, "case %d backward: %s\n", idx, e.what());
                have_dx = false;
            }
            // weight gradients, after the data gradients as cuDNN asks
            bool have_dw = false;
            std::vector<uint8_t> hdw;
            if (have_dx) {
                try {
                    auto* impl = dynamic_cast<CuDNNTimeSelfAttention*>(tsa.get());
                    if (impl) {
                        impl->initializeGradientStorage();
                        cudaDeviceSynchronize();
                        impl->backwardWeights(dy, x, c.B, c.S);
                        cudaDeviceSynchronize();
                        if (impl->gradWeightBuffer_ && impl->gradWeightBuffer_->size() > 0) {
                            hdw.resize(impl->gradWeightBuffer_->size());
                            cudaMemcpy(hdw.data(), impl->gradWeightBuffer_->get(), hdw.size(), cudaMemcpyDeviceToHost);
                            have_dw = true;
                        }
                    }
                } catch (const std::exception& e) {
                    fprintf(stderr, "case %d backwardWeights: %s\n", idx, e.what());
                }
            }
            // weights: through the module's own file, then the reference's own query recipe
            const std::string wpath = out + "/w" + std::to_string(idx) + ".bin";
            tsa->saveWeights(wpath);
            std::ifstream wf(wpath, std::ios::binary);
            uint32_t magic = 0, version = 0;
            size_t nbytes = 0;
            wf.read(reinterpret_cast<char*>(&magic), 4);
            wf.read(reinterpret_cast<char*>(&version), 4);
            wf.read(reinterpret_cast<char*>(&nbytes), sizeof(nbytes));
            std::vector<uint8_t> blob(nbytes);
            wf.read(reinterpret_cast<char*>(blob.data()), (std::streamsize)nbytes);
            void* dblob = nullptr;
            cudaMalloc(&dblob, nbytes);
            cudaMemcpy(dblob, blob.data(), nbytes, cudaMemcpyHostToDevice);
            cudnn_ops::CuDNNHandle handle;
            cudnn_ops::AttentionDescriptor desc;
            cudnn_ops::AttentionConfig cfg;
            cfg.num_heads = c.H; cfg.input_dim = c.E; cfg.head_dim = c.E / c.H;
            cfg.data_type = CUDNN_DATA_FLOAT; cfg.dropout_prob = 0.0f; cfg.sm_scaler = 1.0f;
            cfg.batch_size = c.B; cfg.seq_len_q = c.S; cfg.seq_len_k = c.S;
            desc.configure(cfg);
            const cudnnMultiHeadAttnWeightKind_t kinds[4] = {CUDNN_MH_ATTN_Q_WEIGHTS, CUDNN_MH_ATTN_K_WEIGHTS,
                                                             CUDNN_MH_ATTN_V_WEIGHTS, CUDNN_MH_ATTN_O_WEIGHTS};
            const char* names[4] = {"wq", "wk", "wv", "wo"};
            fprintf(mf, "case %d E %d H %d B %d S %d ln %d res %d dx %d dw %d blob %zu\n", idx, c.E, c.H, c.B, c.S,
                    (int)c.ln, (int)c.res, (int)have_dx, (int)(have_dw && hdw.size() == nbytes), nbytes);
            if (have_dw && hdw.size() == nbytes) {
                FILE* f = fopen((out + "/dw" + std::to_string(idx) + ".bin").c_str(), "wb");
                if (f) { fwrite(hdw.data(), 1, hdw.size(), f); fclose(f); }
            }
            for (int k = 0; k < 4; ++k) {
                cudnnTensorDescriptor_t wd;
                cudnnCreateTensorDescriptor(&wd);
                void* wptr = nullptr;
                cudnnStatus_t st = cudnnGetMultiHeadAttnWeights(handle.get(), desc.get(), kinds[k], nbytes, dblob, wd, &wptr);
                if (st != CUDNN_STATUS_SUCCESS) { fprintf(mf, "  %s status %d\n", names[k], (int)st); continue; }
                cudnnDataType_t dt; int nd = 0, dims[8], strides[8];
                cudnnGetTensorNdDescriptor(wd, 8, &dt, &nd, dims, strides);
                size_t span = 1;
                for (int d = 0; d < nd; ++d) span += (size_t)(dims[d] - 1) * strides[d];
                std::vector<float> hw(span);
                cudaMemcpy(hw.data(), wptr, span * sizeof(float), cudaMemcpyDeviceToHost);
                fprintf(mf, "  %s nd %d dims", names[k], nd);
                for (int d = 0; d < nd; ++d) fprintf(mf, " %d", dims[d]);
                fprintf(mf, " strides");
                for (int d = 0; d < nd; ++d) fprintf(mf, " %d", strides[d]);
                fprintf(mf, " offset %zu span %zu\n", (size_t)((uint8_t*)wptr - (uint8_t*)dblob), span);
                dump(out + "/" + names[k] + std::to_string(idx) + ".f32", hw.data(), span);
                cudnnDestroyTensorDescriptor(wd);
            }
            cudaFree(dblob);
            dump(out + "/x" + std::to_string(idx) + ".f32", hx.data(), n);
            dump(out + "/dy" + std::to_string(idx) + ".f32", hdy.data(), n);
            dump(out + "/y" + std::to_string(idx) + ".f32", hy.data(), n);
            if (have_dx) dump(out + "/dx" + std::to_string(idx) + ".f32", hdx.data(), n);
        } catch (const std::exception& e) {
            fprintf(mf, "case %d failed: %s\n", idx, e.what());
            fprintf(stderr, "case %d failed: %s\n", idx, e.what());
        }
        ++idx;
    }
    fclose(mf);
    printf("done\n");
    return 0;
}
