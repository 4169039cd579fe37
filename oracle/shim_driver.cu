// shim_driver.cu -- TEST INFRASTRUCTURE.  Runs the C++ binding of this library
// (include/ltc_attn_shim.hpp: cudatrader::B200TimeSelfAttention, createB200TimeSelfAttention,
// cudatrader::B200FlashAttention) on a GPU, compiled against the reference's OWN headers and linked
// with the reference's own objects (base-class constructor, cuDNN module; compiled where they lie, see
// the Makefile in this directory) and with libltc_attn.so.  Nothing here is on the product path.
//
//   shim_driver check <outdir>
//       The properties the reference's own tests pin for the class, reproduced on the binding
//       (src/ml/time_self_attention_test.cu of the reference):
//         construction errors :166-187, getters :160-165, DeterministicBehavior 1e-5 :521-558,
//         WeightSaveLoad 1e-4 :561-602, shape sweep :605-657, BackwardPassBasic :659-709,
//         BackwardPassWithMask :711-761, BackwardPassConsistency 1e-6 :799-838,
//       the call order of the reference's training step, forward -> backwardWeights -> backward
//       (src/ml/ml_liquid_net.cu:715-737), and drop-in checks against the reference's cuDNN module created
//       in the same process: same seed => byte-identical weight files; a file written by the reference
//       loads into the binding and both modules then give the same forward output and input gradient on
//       the same input (tolerance 2e-2 of the largest magnitude: cuDNN multiplies fp32 data in TF32, and with the
//       reference's scale of 1.0 and 64-wide heads the scores reach |s| ~ 10, so the 2^-11 rounding of q and k
//       moves a score by ~1e-2 and a softmax weight by that relative amount; the binding's exact path agrees
//       with the fp64 oracle to 1e-5 on the same function, tests/test_tsa_golden.py); the binding's output
//       equals a direct ltca_tsa_fwd call on its own parameters bit for bit.  The FlashAttention class is run
//       at the fixture of src/ml/flash_attention_test.cu:97-140 and its weight file is left in <outdir> for
//       the calling test to compare with the reference's initialisation recipe.
//       Prints one "CHECK <name> <value> <limit> PASS|FAIL" line per property; exit code 1 if any failed.
//
//   shim_driver time <B> <S> <E> <H> <iters>
//       Wall-clock (host, every device synchronisation of the callee included) and CUDA-event milliseconds
//       (medians over 3 * iters rounds) of forward, backwardWeights and backward, called in the order in which
//       the reference's model calls them, for the reference's
//       cuDNN module and for the binding in the reference's form (head width = E, scale 1, no mask: as
//       constructed, with setReuseForward(false), and with setKeepWeightCopies(true)) and in the compact
//       form (head width E/H, scale 1/sqrt(width), causal).  One JSON line.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <random>
#include <string>
#include <vector>

#include "cuda_resources.h"
#include "time_self_attention.h"
#include "cuDNN_ops.h"

#include "ltc_attn_shim.hpp"

using namespace cudatrader;

namespace {

int g_failed = 0;

void report(const char* name, double value, double limit, bool pass) {
    printf("CHECK %s %.9g %.9g %s\n", name, value, limit, pass ? "PASS" : "FAIL");
    if (!pass) ++g_failed;
}
void expect_le(const char* name, double value, double limit) { report(name, value, limit, value <= limit); }
void expect_true(const char* name, bool ok) { report(name, ok ? 1 : 0, 1, ok); }

std::vector<float> random_host(size_t n, unsigned seed) {     // createRandomTensor of the reference's tests
    std::mt19937 gen(seed);
    std::uniform_real_distribution<float> dist(-1.0f, 1.0f);
    std::vector<float> v(n);
    for (auto& x : v) x = dist(gen);
    return v;
}
CudaMemory<float> to_device(const std::vector<float>& h) {
    CudaMemory<float> d(h.size());
    d.copyFromHost(h.data());
    cudaDeviceSynchronize();
    return d;
}
std::vector<float> to_host(const CudaMemory<float>& d) {
    std::vector<float> h(d.size());
    cudaDeviceSynchronize();
    d.copyToHost(h.data());
    cudaDeviceSynchronize();
    return h;
}
double max_abs_diff(const std::vector<float>& a, const std::vector<float>& b) {
    if (a.size() != b.size()) return INFINITY;
    double m = 0;
    for (size_t i = 0; i < a.size(); ++i) m = std::fmax(m, std::fabs((double)a[i] - (double)b[i]));
    return m;
}
double max_abs(const std::vector<float>& a) {
    double m = 0;
    for (float x : a) m = std::fmax(m, std::fabs((double)x));
    return m;
}
bool all_finite(const std::vector<float>& a) {
    for (float x : a) if (!std::isfinite(x)) return false;
    return true;
}
std::vector<uint8_t> read_file(const std::string& p) {
    std::ifstream f(p, std::ios::binary);
    return std::vector<uint8_t>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

template <typename Fn>
bool throws_invalid_argument(Fn fn) {
    try { fn(); } catch (const std::invalid_argument&) { return true; } catch (...) { return false; }
    return false;
}

// ---------------------------------------------------------------------------------------------------------
int run_checks(const std::string& out) {
    const int E = 64, H = 2, B = 2, S = 16;
    const unsigned long long seed = 12345ULL;

    // construction (time_self_attention_test.cu:166-187) and getters (:160-165)
    expect_true("ctor_rejects_indivisible", throws_invalid_argument([] { createB200TimeSelfAttention(63, 2); }));
    expect_true("ctor_rejects_zero_heads", throws_invalid_argument([] { createB200TimeSelfAttention(64, 0); }));
    expect_true("ctor_rejects_negative_dim", throws_invalid_argument([] { createB200TimeSelfAttention(-64, 2); }));
    {
        auto a = createB200TimeSelfAttention(E, H, true, true, 0.0f, seed);
        expect_true("factory_returns_module", a != nullptr);
        if (!a) return 1;
        expect_true("getters", a->getInputDim() == E && a->getNumHeads() == H && a->getHeadDim() == E / H &&
                                   a->getUseLayerNorm() && a->getUseResidual() && a->getDropoutRate() == 0.0f);
    }

    const std::vector<float> hx = random_host((size_t)B * S * E, (unsigned)seed);
    CudaMemory<float> x = to_device(hx);

    // DeterministicBehavior (:521-558)
    {
        auto a1 = createB200TimeSelfAttention(E, H, true, true, 0.0f, seed);
        auto a2 = createB200TimeSelfAttention(E, H, true, true, 0.0f, seed);
        std::vector<float> o1 = to_host(a1->forward(x, B, S)), o2 = to_host(a2->forward(x, B, S));
        expect_le("deterministic_two_instances", max_abs_diff(o1, o2), 1e-5);
        expect_true("forward_finite", all_finite(o1));
        expect_le("forward_differs_from_input", -max_abs_diff(o1, hx), -1e-3);      // output != input (:441)
    }
    // WeightSaveLoad (:561-602)
    {
        auto a1 = createB200TimeSelfAttention(E, H, true, true, 0.0f, seed);
        std::vector<float> o1 = to_host(a1->forward(x, B, S));
        const std::string f = out + "/shim_tsa_weights.bin";
        a1->saveWeights(f);
        auto a2 = createB200TimeSelfAttention(E, H, true, true, 0.0f, seed + 1);
        std::vector<float> before = to_host(a2->forward(x, B, S));
        a2->loadWeights(f);
        std::vector<float> o2 = to_host(a2->forward(x, B, S));
        expect_le("save_load_same_output", max_abs_diff(o1, o2), 1e-4);
        expect_le("other_seed_differs", -max_abs_diff(o1, before), -1e-3);
        bool refused = false;
        try { auto a3 = createB200TimeSelfAttention(128, 4, true, true, 0.0f, seed); a3->loadWeights(f); }
        catch (const std::runtime_error&) { refused = true; }
        expect_true("load_refuses_other_shape", refused);
    }
    // shape sweep (:605-657): S in {8, 32}, B in {1, 4}, (E, H) in {(64,1), (128,4), (512,8)}, LN x residual
    {
        bool ok = true;
        const int shapes[][4] = {{B, 8, E, H}, {B, 32, E, H}, {1, S, E, H}, {4, S, E, H},
                                 {B, S, 64, 1}, {B, S, 128, 4}, {B, S, 512, 8}};
        for (const auto& sh : shapes) {
            for (int flags = 0; flags < 4; ++flags) {
                auto a = createB200TimeSelfAttention(sh[2], sh[3], (flags & 1) != 0, (flags & 2) != 0, 0.0f, seed);
                const size_t n = (size_t)sh[0] * sh[1] * sh[2];
                CudaMemory<float> xi = to_device(random_host(n, (unsigned)seed));
                std::vector<float> o = to_host(a->forward(xi, sh[0], sh[1]));
                ok = ok && o.size() == n && all_finite(o) && max_abs(o) > 0;
            }
        }
        expect_true("shape_sweep", ok);
    }
    // backward (:659-838) at the reference's backward fixtures, LayerNorm and residual off
    const int bw[][4] = {{2, 4, 8, 2}, {1, 3, 6, 2}};
    for (const auto& sh : bw) {
        const int b = sh[0], s = sh[1], e = sh[2], h = sh[3];
        auto a = createB200TimeSelfAttention(e, h, false, false, 0.0f, 42);
        const size_t n = (size_t)b * s * e;
        CudaMemory<float> xi = to_device(random_host(n, 1)), gy = to_device(random_host(n, 2));
        CudaMemory<float> mask = to_device(std::vector<float>((size_t)b * s * s, 1.0f));
        a->forward(xi, b, s);
        std::vector<float> g1 = to_host(a->backward(gy, xi, b, s));
        a->forward(xi, b, s);
        std::vector<float> g2 = to_host(a->backward(gy, xi, b, s));
        std::vector<float> gm = to_host(a->backward(gy, xi, b, s, &mask));
        char name[64];
        snprintf(name, sizeof(name), "backward_repeatable_e%d", e);
        expect_le(name, max_abs_diff(g1, g2), 1e-6);
        snprintf(name, sizeof(name), "backward_nonzero_finite_e%d", e);
        expect_true(name, all_finite(g1) && max_abs(g1) > 0 && all_finite(gm));
        bool threw = false;
        try { a->backwardWeights(gy, xi, b, s); } catch (...) { threw = true; }
        snprintf(name, sizeof(name), "backward_weights_no_throw_e%d", e);
        expect_true(name, !threw);
    }
    // the training step's order: forward -> backwardWeights -> backward (ml_liquid_net.cu:715-737), gradient
    // storage and parameter accessors (:919, :1160, :1181)
    {
        auto a = createB200TimeSelfAttention(E, H, true, true, 0.0f, seed);
        CudaMemory<float> gy = to_device(random_host((size_t)B * S * E, 7));
        a->initializeGradientStorage();
        a->forward(x, B, S);
        a->backwardWeights(gy, x, B, S);
        std::vector<float> dx = to_host(a->backward(gy, x, B, S));
        auto params = a->getParameters();
        auto grads = a->getComputedGradients();
        bool ok = params.size() == grads.size() && params.size() == 6 && all_finite(dx) && max_abs(dx) > 0;
        for (size_t i = 0; ok && i < params.size(); ++i) ok = params[i]->size() == grads[i]->size();
        for (size_t i = 2; ok && i < grads.size(); ++i) {           // the four projection matrices
            std::vector<float> g = to_host(*grads[i]);
            ok = all_finite(g) && max_abs(g) > 0;
        }
        expect_true("training_step_call_order", ok);
        // the mask argument: ignored, as by the reference's module (cudnn_time_self_attention.cu:211-237)
        std::vector<float> causal_mask((size_t)B * S * S, 0.0f);
        for (int b = 0; b < B; ++b)
            for (int i = 0; i < S; ++i)
                for (int j = 0; j <= i; ++j) causal_mask[((size_t)b * S + i) * S + j] = 1.0f;
        CudaMemory<float> mask = to_device(causal_mask);
        std::vector<float> o_plain = to_host(a->forward(x, B, S)), o_mask = to_host(a->forward(x, B, S, &mask));
        expect_le("mask_ignored_by_default", max_abs_diff(o_plain, o_mask), 0.0);
        auto* impl = dynamic_cast<B200TimeSelfAttention*>(a.get());
        impl->setHonourMask(true);
        std::vector<float> o_hon = to_host(a->forward(x, B, S, &mask));
        expect_le("mask_honoured_on_request", -max_abs_diff(o_plain, o_hon), -1e-4);
        impl->setHonourMask(false);
        // kept forward and kept weight copies: the same bits as the recomputing calls, over two rounds (the second
        // round runs on the copies made by the first)
        {
            impl->setReuseForward(false);
            std::vector<float> dx_plain = to_host(a->backward(gy, x, B, S));
            impl->setReuseForward(true);
            impl->setKeepWeightCopies(true);
            double worst = 0.0;
            for (int round = 0; round < 2; ++round) {
                std::vector<float> o_kept = to_host(a->forward(x, B, S));
                a->backwardWeights(gy, x, B, S);
                std::vector<float> dx_kept = to_host(a->backward(gy, x, B, S));
                worst = std::max(worst, std::max(max_abs_diff(o_plain, o_kept), max_abs_diff(dx_plain, dx_kept)));
            }
            expect_le("kept_forward_and_weight_copies_same_bits", worst, 0.0);
            impl->setKeepWeightCopies(false);
        }
        // the same numbers as a direct call of the C entry point on the module's own parameters
        ltca_ctx* ctx = nullptr;
        ltca_ctx_create(0, nullptr, &ctx);
        ltca_tsa_params p = {};
        p.B = B; p.S = S; p.E = E; p.H = H; p.head_width = E; p.time_major = 1;
        p.use_residual = 1; p.use_layer_norm = 1; p.mode = LTCA_MODE_AUTO; p.scale = 1.0f;
        p.x = x.get();
        p.ln_gamma = params[0]->get(); p.ln_beta = params[1]->get();
        p.wq = params[2]->get(); p.wk = params[3]->get(); p.wv = params[4]->get(); p.wo = params[5]->get();
        CudaMemory<float> direct((size_t)B * S * E);
        p.out = direct.get();
        size_t need = 0;
        ltca_tsa_workspace_bytes(&p, 0, &need);
        CudaMemory<float> ws((need + 3) / 4 + 64);
        p.workspace = ws.get(); p.workspace_bytes = ws.bytes();
        const int rc = ltca_tsa_fwd(ctx, &p);
        expect_true("direct_call_ok", rc == 0);
        expect_le("binding_equals_direct_call", max_abs_diff(o_plain, to_host(direct)), 0.0);
        uint32_t st = 1;
        ltca_device_status(ctx, &st);
        expect_true("device_status_clean", st == 0);
        ltca_ctx_destroy(ctx);
    }
    // drop-in against the reference's cuDNN module in the same process
    {
        bool have_ref = true;
        std::unique_ptr<TimeSelfAttention> ref, ref2;
        std::vector<float> y_ref, dx_ref;
        CudaMemory<float> gy = to_device(random_host((size_t)B * S * E, 9));
        try {
            ref = TimeSelfAttention::create(E, H, true, true, 0.0f, seed);
            y_ref = to_host(ref->forward(x, B, S));              // the first forward initialises the weights
            dx_ref = to_host(ref->backward(gy, x, B, S));
            ref->saveWeights(out + "/ref_same_seed.bin");
            ref2 = TimeSelfAttention::create(E, H, true, true, 0.0f, 777);
            ref2->forward(x, B, S);
            ref2->saveWeights(out + "/ref_other_seed.bin");
        } catch (const std::exception& e) {
            printf("NOTE reference cuDNN module unavailable: %s\n", e.what());
            have_ref = false;
        }
        if (have_ref) {
            auto a = createB200TimeSelfAttention(E, H, true, true, 0.0f, seed);
            a->saveWeights(out + "/shim_same_seed.bin");
            expect_true("same_seed_weight_file_is_byte_identical",
                        read_file(out + "/shim_same_seed.bin") == read_file(out + "/ref_same_seed.bin"));
            std::vector<float> y = to_host(a->forward(x, B, S)), dx = to_host(a->backward(gy, x, B, S));
            expect_le("forward_vs_reference_module", max_abs_diff(y, y_ref) / std::fmax(1.0, max_abs(y_ref)), 2e-2);
            expect_le("backward_vs_reference_module", max_abs_diff(dx, dx_ref) / std::fmax(1.0, max_abs(dx_ref)), 2e-2);
            a->loadWeights(out + "/ref_other_seed.bin");          // a file the reference wrote
            std::vector<float> y2 = to_host(a->forward(x, B, S)), y2_ref = to_host(ref2->forward(x, B, S));
            expect_le("reference_weight_file_loads", max_abs_diff(y2, y2_ref) / std::fmax(1.0, max_abs(y2_ref)), 2e-2);
            ref2->loadWeights(out + "/shim_same_seed.bin");       // and the other way round
            std::vector<float> y3_ref = to_host(ref2->forward(x, B, S));
            expect_le("reference_loads_binding_file", max_abs_diff(y3_ref, y_ref) / std::fmax(1.0, max_abs(y_ref)), 1e-5);
        }
    }
    // FlashAttention class at the fixture of flash_attention_test.cu:97-140
    {
        const int fe = 32, fd = 16, fh = 2, fb = 2, fs = 8;
        B200FlashAttention f1(fe, fd, fh, 0.0f, true, true, false, 12345ULL);
        B200FlashAttention f2(fe, fd, fh, 0.0f, true, true, false, 12345ULL);
        const std::vector<float> hxf = random_host((size_t)fb * fs * fe, 12345);
        CudaMemory<float> xf = to_device(hxf);
        std::vector<float> o1 = to_host(f1.forward(xf, fb, fs)), o2 = to_host(f2.forward(xf, fb, fs));
        expect_true("fa_forward_shape_finite", o1.size() == hxf.size() && all_finite(o1) && max_abs(o1) > 0);
        expect_le("fa_deterministic_two_instances", max_abs_diff(o1, o2), 1e-5);
        expect_true("fa_getters", f1.getNumHeads() == fh && f1.getHeadDim() == fd && f1.getInputDim() == fe &&
                                      f1.getModelDim() == fd * fh && f1.getUseLayerNorm() && f1.getUseResidual() &&
                                      f1.isTensorCoreOptimized());
        expect_true("fa_save", f1.saveWeights(out + "/shim_fa_weights.bin"));
        B200FlashAttention f3(fe, fd, fh, 0.0f, true, true, false, 999ULL);
        std::vector<float> o3 = to_host(f3.forward(xf, fb, fs));
        expect_le("fa_other_seed_differs", -max_abs_diff(o1, o3), -1e-4);
        expect_true("fa_load", f3.loadWeights(out + "/shim_fa_weights.bin"));
        expect_le("fa_save_load_same_output", max_abs_diff(o1, to_host(f3.forward(xf, fb, fs))), 1e-6);
        B200FlashAttention f4(fe, 8, fh, 0.0f, true, true, false, 1ULL);
        expect_true("fa_load_refuses_other_shape", !f4.loadWeights(out + "/shim_fa_weights.bin"));
        // keep-mask: 0 hides (flash_attention.cu:161-164); a causal mask changes the result, an all-ones mask does not
        std::vector<float> ones((size_t)fb * fs * fs, 1.0f), causal((size_t)fb * fs * fs, 0.0f);
        for (int b = 0; b < fb; ++b)
            for (int i = 0; i < fs; ++i)
                for (int j = 0; j <= i; ++j) causal[((size_t)b * fs + i) * fs + j] = 1.0f;
        CudaMemory<float> m1 = to_device(ones), mc = to_device(causal);
        expect_le("fa_all_ones_mask_is_no_mask", max_abs_diff(o1, to_host(f1.forward(xf, fb, fs, &m1))), 1e-6);
        std::vector<float> oc = to_host(f1.forward(xf, fb, fs, &mc));
        expect_true("fa_causal_mask_changes_output", all_finite(oc) && max_abs_diff(o1, oc) > 1e-4);
        // without LayerNorm and residual, with dropout (flash_attention_test.cu:215-312)
        B200FlashAttention f5(fe, fd, fh, 0.2f, false, false, false, 5ULL);
        std::vector<float> od = to_host(f5.forward(xf, fb, fs));
        size_t zeros = 0;
        for (float v : od) zeros += (v == 0.0f);
        expect_true("fa_dropout_drops_some", all_finite(od) && zeros > od.size() / 20 && zeros < od.size() / 2);
        // backward (extension): runs, finite, non-zero, repeatable
        CudaMemory<float> gy = to_device(random_host(hxf.size(), 3));
        f1.forward(xf, fb, fs);
        std::vector<float> g1 = to_host(f1.backward(gy, xf, fb, fs)), g2 = to_host(f1.backward(gy, xf, fb, fs));
        f1.backwardWeights(gy, xf, fb, fs);
        bool ok = all_finite(g1) && max_abs(g1) > 0 && max_abs_diff(g1, g2) <= 1e-6;
        for (CudaMemory<float>* g : f1.getComputedGradients()) ok = ok && all_finite(to_host(*g));
        expect_true("fa_backward", ok);
    }
    cudaDeviceSynchronize();
    const cudaError_t e = cudaGetLastError();
    expect_true("no_cuda_error", e == cudaSuccess);
    printf("%s (%d failed)\n", g_failed ? "FAILED" : "ALL PASS", g_failed);
    return g_failed ? 1 : 0;
}

// ---------------------------------------------------------------------------------------------------------
struct Timing { double fwd_wall = 0, bww_wall = 0, bwd_wall = 0, fwd_ev = 0, bww_ev = 0, bwd_ev = 0; bool ok = false;
                std::string note; };

Timing time_module(TimeSelfAttention& m, const CudaMemory<float>& x, const CudaMemory<float>& gy, int B, int S,
                   int iters) {
    Timing t;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    auto run = [&](int which) {
        if (which == 0) { CudaMemory<float> y = m.forward(x, B, S); }
        else if (which == 1) m.backwardWeights(gy, x, B, S);
        else { CudaMemory<float> dx = m.backward(gy, x, B, S); }
    };
    try {
        for (int w = 0; w < 10; ++w) { run(0); run(1); run(2); }         // forward -> backwardWeights -> backward
        cudaDeviceSynchronize();
        // The model's call order in every iteration, each call timed on its own; the median over the iterations
        // is reported: every call allocates and frees its result (the interface returns it by value), and the
        // allocator's cost jumps now and then on a fresh device.
        std::vector<double> wall[3], ev[3];
        for (int i = 0; i < 3 * iters; ++i) {
            for (int which = 0; which < 3; ++which) {
                cudaDeviceSynchronize();
                const auto t0 = std::chrono::steady_clock::now();
                cudaEventRecord(e0, nullptr);
                run(which);
                cudaEventRecord(e1, nullptr);
                cudaDeviceSynchronize();
                const auto t1 = std::chrono::steady_clock::now();
                float ms = 0;
                cudaEventElapsedTime(&ms, e0, e1);
                wall[which].push_back(std::chrono::duration<double, std::milli>(t1 - t0).count());
                ev[which].push_back(ms);
            }
        }
        auto median = [](std::vector<double>& v) { std::sort(v.begin(), v.end()); return v[v.size() / 2]; };
        t.fwd_wall = median(wall[0]); t.bww_wall = median(wall[1]); t.bwd_wall = median(wall[2]);
        t.fwd_ev = median(ev[0]); t.bww_ev = median(ev[1]); t.bwd_ev = median(ev[2]);
        t.ok = cudaGetLastError() == cudaSuccess;
    } catch (const std::exception& e) {
        t.note = e.what();
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return t;
}

void print_timing(const char* key, const Timing& t, bool last) {
    if (t.ok)
        printf("\"%s\": {\"fwd_ms\": %.4f, \"bwd_weights_ms\": %.4f, \"bwd_data_ms\": %.4f, \"fwd_event_ms\": %.4f, "
               "\"bwd_weights_event_ms\": %.4f, \"bwd_data_event_ms\": %.4f}%s",
               key, t.fwd_wall, t.bww_wall, t.bwd_wall, t.fwd_ev, t.bww_ev, t.bwd_ev, last ? "" : ", ");
    else
        printf("\"%s\": {\"unavailable\": \"%s\"}%s", key, t.note.c_str(), last ? "" : ", ");
}

int run_time(int B, int S, int E, int H, int iters) {
    const size_t n = (size_t)B * S * E;
    CudaMemory<float> x = to_device(random_host(n, 1)), gy = to_device(random_host(n, 2));
    Timing tr, ts, tn, tk, tc;
    try {
        auto ref = TimeSelfAttention::create(E, H, true, true, 0.0f, 42);
        tr = time_module(*ref, x, gy, B, S, iters);
    } catch (const std::exception& e) { tr.note = e.what(); }
    try {
        // as constructed: forward() keeps its intermediates for the two backward calls, which is what the cuDNN
        // module does with its reserve space
        B200TimeSelfAttention shim(E, H, true, true, 0.0f, 42, false, false);
        ts = time_module(shim, x, gy, B, S, iters);
    } catch (const std::exception& e) { ts.note = e.what(); }
    try {
        B200TimeSelfAttention shim(E, H, true, true, 0.0f, 42, false, false);
        shim.setReuseForward(false);        // every backward call recomputes the forward
        tn = time_module(shim, x, gy, B, S, iters);
    } catch (const std::exception& e) { tn.note = e.what(); }
    try {
        B200TimeSelfAttention shim(E, H, true, true, 0.0f, 42, false, false);
        shim.setKeepWeightCopies(true);     // the weights do not change between the timed calls
        tk = time_module(shim, x, gy, B, S, iters);
    } catch (const std::exception& e) { tk.note = e.what(); }
    try {
        B200TimeSelfAttention shim(E, H, true, true, 0.0f, 42, true, true);
        tc = time_module(shim, x, gy, B, S, iters);
    } catch (const std::exception& e) { tc.note = e.what(); }
    printf("{\"B\": %d, \"S\": %d, \"E\": %d, \"H\": %d, \"iters\": %d, \"cudnn\": \"%s\", ", B, S, E, H, iters,
           cudnn_ops::getCuDNNVersionString().c_str());
    print_timing("reference_cudnn_module", tr, false);
    print_timing("binding_reference_form", ts, false);
    print_timing("binding_reference_form_recomputing", tn, false);
    print_timing("binding_reference_form_kept_weight_copies", tk, false);
    print_timing("binding_compact_causal_form", tc, true);
    printf("}\n");
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc >= 3 && strcmp(argv[1], "check") == 0) return run_checks(argv[2]);
    if (argc >= 7 && strcmp(argv[1], "time") == 0)
        return run_time(atoi(argv[2]), atoi(argv[3]), atoi(argv[4]), atoi(argv[5]), atoi(argv[6]));
    fprintf(stderr, "usage: shim_driver check <outdir> | time <B> <S> <E> <H> <iters>\n");
    return 2;
}
