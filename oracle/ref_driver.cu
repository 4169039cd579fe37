// ref_driver.cu -- TEST INFRASTRUCTURE.  Drives the reference's OWN attention code, compiled
// unmodified from the reference checkout at build time (see the Makefile in this directory;
// the reference file is pulled in by path through REF_ROOT_FLASH, nothing is copied here).
// It needs a GPU to run, so it is built in advance and executed by the GPU tests and by the
// golden-vector generator.
//
// Sub-commands
//   flash <outdir>         run the reference flashAttentionKernel on its valid domain
//                          (head_dim <= 16, one 16-key tile: src/ml/flash_attention.cu:1015-1017
//                          and the tile loop at :87) for a fixed list of seeded cases and dump
//                          q, k, v, mask, out as raw little-endian float32 plus a manifest.
//   flash_forward <outdir> call FlashAttention::forward at the benchmark's small shape
//                          (B=2 H=4 S=64 D=32) and record what it returns.
//   time_flash <B> <H> <S> <D> <iters>
//                          time the reference kernel with its own launch recipe
//                          (src/ml/flash_attention.cu:1001-1043); prints microseconds per launch.
#include REF_ROOT_FLASH   // the reference translation unit itself: kernels + FlashAttention class

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

using namespace cudatrader;

namespace {

// Same recipe as the reference tests' createRandomTensor: mt19937(seed), uniform(-1, 1)
// (src/ml/flash_attention_test.cu:15-32).
std::vector<float> random_tensor(size_t n, unsigned seed) {
    std::mt19937 gen(seed);
    std::uniform_real_distribution<float> dist(-1.0f, 1.0f);
    std::vector<float> v(n);
    for (auto& x : v) x = dist(gen);
    return v;
}

void dump(const std::string& path, const std::vector<float>& v) {
    FILE* f = fopen(path.c_str(), "wb");
    if (!f) { perror(path.c_str()); exit(2); }
    fwrite(v.data(), sizeof(float), v.size(), f);
    fclose(f);
}

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { \
    fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e)); exit(3); } } while (0)

// Launches the kernel exactly as FlashAttention::forward does (src/ml/flash_attention.cu:1001-1043).
void launch_reference_kernel(const float* q, const float* k, const float* v, const float* mask,
                             float* out, int B, int S, int H, int D, cudaStream_t stream) {
    const float scaling = 1.0f / sqrtf(static_cast<float>(D));
    dim3 grid((S + 15) / 16, (S + 15) / 16, B * H);
    const size_t smem = (16 * 16 + 16 * 16 + 16 * 16 + 16 * 16) * sizeof(float);
    flashAttentionKernel<<<grid, 256, smem, stream>>>(q, k, v, mask, out, B, S, H, D, scaling);
}

struct Case { int B, H, S, D, mask_kind; unsigned seed; };   // mask_kind: 0 none, 1 causal, 2 random

int cmd_flash(const char* outdir) {
    const Case cases[] = {
        {2, 2, 8, 16, 0, 12345},     // the reference test fixture (flash_attention_test.cu:97-104)
        {2, 4, 16, 16, 0, 12346},
        {2, 4, 16, 16, 1, 12347},
        {1, 2, 16, 8, 2, 12348},
        {4, 2, 8, 16, 1, 12349},
        {1, 1, 5, 4, 0, 12350},
    };
    FILE* man = fopen((std::string(outdir) + "/manifest.txt").c_str(), "w");
    if (!man) { perror("manifest"); return 2; }
    int idx = 0;
    for (const Case& c : cases) {
        const size_t n = (size_t)c.B * c.H * c.S * c.D;
        auto q = random_tensor(n, c.seed), k = random_tensor(n, c.seed + 100), v = random_tensor(n, c.seed + 200);
        std::vector<float> mask;
        if (c.mask_kind) {
            mask.assign((size_t)c.B * c.S * c.S, 1.0f);
            std::mt19937 gen(c.seed + 300);
            for (int b = 0; b < c.B; ++b)
                for (int i = 0; i < c.S; ++i)
                    for (int j = 0; j < c.S; ++j) {
                        bool keep = c.mask_kind == 1 ? (j <= i) : ((gen() % 10) < 7 || j == i);
                        mask[((size_t)b * c.S + i) * c.S + j] = keep ? 1.0f : 0.0f;
                    }
        }
        float *dq, *dk, *dv, *dm = nullptr, *dout;
        CK(cudaMalloc(&dq, n * 4)); CK(cudaMalloc(&dk, n * 4)); CK(cudaMalloc(&dv, n * 4));
        CK(cudaMalloc(&dout, n * 4));
        CK(cudaMemset(dout, 0, n * 4));     // the reference allocates zero-filled outputs
        CK(cudaMemcpy(dq, q.data(), n * 4, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(dk, k.data(), n * 4, cudaMemcpyHostToDevice));
        CK(cudaMemcpy(dv, v.data(), n * 4, cudaMemcpyHostToDevice));
        if (!mask.empty()) {
            CK(cudaMalloc(&dm, mask.size() * 4));
            CK(cudaMemcpy(dm, mask.data(), mask.size() * 4, cudaMemcpyHostToDevice));
        }
        launch_reference_kernel(dq, dk, dv, dm, dout, c.B, c.S, c.H, c.D, nullptr);
        CK(cudaGetLastError());
        CK(cudaDeviceSynchronize());
        std::vector<float> out(n);
        CK(cudaMemcpy(out.data(), dout, n * 4, cudaMemcpyDeviceToHost));
        const std::string base = std::string(outdir) + "/case" + std::to_string(idx);
        dump(base + "_q.bin", q); dump(base + "_k.bin", k); dump(base + "_v.bin", v);
        dump(base + "_out.bin", out);
        if (!mask.empty()) dump(base + "_mask.bin", mask);
        fprintf(man, "%d %d %d %d %d %d %.9g %.9g\n", idx, c.B, c.H, c.S, c.D, c.mask_kind,
                1.0 / sqrt((double)c.D), 10.0);
        cudaFree(dq); cudaFree(dk); cudaFree(dv); cudaFree(dout); if (dm) cudaFree(dm);
        ++idx;
    }
    fclose(man);
    printf("wrote %d cases to %s\n", idx, outdir);
    return 0;
}

int cmd_flash_forward(const char* outdir) {
    // B=2 H=4 S=64 D=32: the reference refuses head_dim > 16 and returns its zero-filled output.
    const int B = 2, H = 4, S = 64, D = 32, E = H * D;
    FlashAttention fa(E, D, H, 0.0f, false, false, false, 12345ULL);
    auto x = random_tensor((size_t)B * S * E, 777);
    CudaMemory<float> dx((size_t)B * S * E);
    CK(cudaMemcpy(dx.get(), x.data(), x.size() * 4, cudaMemcpyHostToDevice));
    CudaMemory<float> out = fa.forward(dx, B, S, nullptr, nullptr);
    CK(cudaDeviceSynchronize());
    std::vector<float> ho((size_t)B * S * E);
    CK(cudaMemcpy(ho.data(), out.get(), ho.size() * 4, cudaMemcpyDeviceToHost));
    double mx = 0;
    for (float f : ho) mx = std::max(mx, (double)fabsf(f));
    FILE* f = fopen((std::string(outdir) + "/flash_forward_c1.txt").c_str(), "w");
    if (f) { fprintf(f, "FlashAttention::forward B=2 H=4 S=64 D=32: max|out| = %.9g\n", mx); fclose(f); }
    printf("FlashAttention::forward B=2 H=4 S=64 D=32: max|out| = %.9g\n", mx);
    return 0;
}

int cmd_time_flash(int B, int H, int S, int D, int iters) {
    const size_t n = (size_t)B * H * S * D;
    float *dq, *dk, *dv, *dout;
    CK(cudaMalloc(&dq, n * 4)); CK(cudaMalloc(&dk, n * 4)); CK(cudaMalloc(&dv, n * 4)); CK(cudaMalloc(&dout, n * 4));
    auto q = random_tensor(n, 1);
    CK(cudaMemcpy(dq, q.data(), n * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dk, q.data(), n * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dv, q.data(), n * 4, cudaMemcpyHostToDevice));
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    for (int i = 0; i < 3; ++i) launch_reference_kernel(dq, dk, dv, nullptr, dout, B, S, H, D, nullptr);
    CK(cudaDeviceSynchronize());
    CK(cudaEventRecord(e0));
    for (int i = 0; i < iters; ++i) launch_reference_kernel(dq, dk, dv, nullptr, dout, B, S, H, D, nullptr);
    CK(cudaEventRecord(e1));
    CK(cudaDeviceSynchronize());
    float ms = 0;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    printf("{\"what\": \"reference flashAttentionKernel\", \"B\": %d, \"H\": %d, \"S\": %d, \"D\": %d, "
           "\"us_per_launch\": %.3f}\n", B, H, S, D, 1000.0 * ms / iters);
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc >= 3 && !strcmp(argv[1], "flash")) return cmd_flash(argv[2]);
    if (argc >= 3 && !strcmp(argv[1], "flash_forward")) return cmd_flash_forward(argv[2]);
    if (argc >= 7 && !strcmp(argv[1], "time_flash"))
        return cmd_time_flash(atoi(argv[2]), atoi(argv[3]), atoi(argv[4]), atoi(argv[5]), atoi(argv[6]));
    fprintf(stderr, "usage: ref_driver flash <outdir> | flash_forward <outdir> | time_flash B H S D iters\n");
    return 1;
}
