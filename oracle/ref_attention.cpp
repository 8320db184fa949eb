// TEST INFRASTRUCTURE ONLY -- not part of the shipped product path.
//
// Harness that drives the *reference's own* tensor ops (compiled from the
// reference sources where they lie, see oracle/Makefile) through causal
// attention forward and backward, so that the CUDA kernels in this repository
// can be compared with "Inferno's own attention path" on identical inputs.
//
// Forward follows the composition in InfernoApp/main.cpp:737-754
// (kt = k^T contiguous; matmul; * scale; triu mask; masked_fill -1e9; Softmax;
// matmul).  As shipped, the reference's autograd graph is cut at masked_fill
// (src/inferno/core/ops.cpp:1238, no backward node) and at contiguous()
// (ops.cpp:1308 + src/inferno/core/tensorimpl.cpp:389-396), so dQ/dK never
// arrive.  The backward here therefore runs the reference's own nodes in two
// stages, re-arming requires_grad on the two cut tensors:
//   stage 1: (y * dO).backward()   -> v.grad = dV, sm.grad = dS
//   stage 2: (s1 * dS).backward()  -> q.grad = dQ, k.grad = dK
// Engine::backward always seeds ones (src/inferno/gradengine/engine.cpp:59),
// which is why the upstream gradient enters through a multiply.
//
// With a fourth mode argument of 2 the same composition is run through the autograd additions of
// inferno_b200/inferno_shim/autograd_patches.h (masked_fill and contiguous that stay in the graph, a seeded backward)
// and a single backward pass; tests compare the two.
//
// Usage: ref_attention <cpu|cuda> B H T D q.bin k.bin v.bin do.bin out_prefix [mode: 0 fwd+bwd, 1 fwd only, 2 single-pass bwd]
// Files are raw little-endian fp32, dense row-major [B,H,T,D].
// Writes <out_prefix>.{o,dq,dk,dv}.bin and prints one JSON line with timings.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <inferno/inferno.h>
#include <inferno/core/ops.h>
#include "inferno/core/ops_impl.h"
#include "inferno/core/tensorimpl.h"
#include "../inferno_b200/inferno_shim/autograd_patches.h"

using Inferno::Tensor;

static std::vector<float> read_bin(const char* path, size_t n) {
    std::vector<float> v(n);
    FILE* f = std::fopen(path, "rb");
    if (!f) { std::fprintf(stderr, "cannot open %s\n", path); std::exit(2); }
    size_t got = std::fread(v.data(), sizeof(float), n, f);
    std::fclose(f);
    if (got != n) { std::fprintf(stderr, "short read %s: %zu of %zu\n", path, got, n); std::exit(2); }
    return v;
}

static void write_tensor(const std::string& path, const Tensor& t_in, size_t n) {
    Tensor t = t_in.contiguous().to(Inferno::Device::cpu());
    if (t.numel() != n) { std::fprintf(stderr, "numel mismatch for %s\n", path.c_str()); std::exit(2); }
    const float* p = Inferno::GetImpl(t)->data_as_ptr<float>() + t.offset();
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) { std::fprintf(stderr, "cannot write %s\n", path.c_str()); std::exit(2); }
    std::fwrite(p, sizeof(float), n, f);
    std::fclose(f);
}

static double now_ms() {
    using namespace std::chrono;
    return duration<double, std::milli>(steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char** argv) {
    if (argc < 11) {
        std::fprintf(stderr, "usage: %s <cpu|cuda> B H T D q k v do out_prefix [mode] [reps]\n", argv[0]);
        return 2;
    }
    const bool on_cuda = std::strcmp(argv[1], "cuda") == 0;
    const size_t B = std::strtoul(argv[2], nullptr, 10), H = std::strtoul(argv[3], nullptr, 10);
    const size_t T = std::strtoul(argv[4], nullptr, 10), D = std::strtoul(argv[5], nullptr, 10);
    const size_t n = B * H * T * D;
    const std::string prefix = argv[10];
    const int mode = argc > 11 ? std::atoi(argv[11]) : 0;
    const bool fwd_only = mode == 1, single_pass = mode == 2;
    // reps > 1 runs the whole pass that many times in this process and reports the last one: the first pays for the
    // CUDA context, the cuBLAS handle and the first launch of every kernel (what a timing wants to leave out)
    const int reps = argc > 12 ? std::max(1, std::atoi(argv[12])) : 1;
    Inferno::Device dev = on_cuda ? Inferno::Device::cuda(0) : Inferno::Device::cpu();

    std::vector<float> hq = read_bin(argv[6], n), hk = read_bin(argv[7], n), hv = read_bin(argv[8], n);
    std::vector<float> hdo = fwd_only ? std::vector<float>(n, 0.f) : read_bin(argv[9], n);

    for (int rep = 0; rep < reps; ++rep) {
    const bool last = rep + 1 == reps;
    Tensor q(Inferno::DType::Float32, hq, {B, H, T, D}, "q", dev, true);
    Tensor k(Inferno::DType::Float32, hk, {B, H, T, D}, "k", dev, true);
    Tensor v(Inferno::DType::Float32, hv, {B, H, T, D}, "v", dev, true);
    Tensor dO(Inferno::DType::Float32, hdo, {B, H, T, D}, "dO", dev, false);

    // ---- forward (InfernoApp/main.cpp:737-754) ----
    double t0 = now_ms();
    Tensor kt = single_pass ? Inferno::contiguous_with_grad(k.transpose(-1, -2)) : k.transpose(-1, -2).contiguous();
    kt.set_requires_grad(true);  // re-arm cut #1 (ContiguousBackward is attached but unreachable otherwise)
    Tensor s0 = Inferno::matmul(q, kt, "QK^T");
    const float scale = 1.0f / std::sqrt(static_cast<float>(D));
    Tensor s1 = s0 * scale;
    std::vector<int> ones_data(T * T, 1);
    Tensor ones(Inferno::DType::Int32, ones_data, {1, 1, T, T}, "causal_mask_ones", dev);
    Tensor mask = Inferno::triu(ones, 1);
    Tensor sm = single_pass ? Inferno::masked_fill_with_grad(s1, mask, -1e9f) : Inferno::masked_fill(s1, mask, -1e9f);
    if (!single_pass) sm.set_requires_grad(true);  // re-arm cut #2: sm becomes a leaf, stage boundary
    Tensor p = Inferno::Softmax(sm, -1);
    Tensor y = Inferno::matmul(p, v, "attn@V");
    if (on_cuda) { (void)y.to(Inferno::Device::cpu()); }  // device->host read = completion point
    double t1 = now_ms();
    if (last) write_tensor(prefix + ".o.bin", y, n);

    double t2 = t1, t3 = t1;
    if (!fwd_only) {
        t2 = now_ms();
        if (single_pass) {
            Inferno::backward_with_seed(y, dO);  // one pass through MaskedFillBackward and the re-armed ContiguousBackward
            if (!q.grad() || !k.grad() || !v.grad()) { std::fprintf(stderr, "missing gradient\n"); return 3; }
            write_tensor(prefix + ".dq.bin", q.Getgrad().contiguous(), n);
            write_tensor(prefix + ".dk.bin", k.Getgrad().contiguous(), n);
            write_tensor(prefix + ".dv.bin", v.Getgrad().contiguous(), n);
            t3 = now_ms();
            if (!last) continue;
            std::printf("{\"device\": \"%s\", \"B\": %zu, \"H\": %zu, \"T\": %zu, \"D\": %zu, \"fwd_ms\": %.3f, \"bwd_ms\": %.3f, \"single_pass\": true}\n",
                        argv[1], B, H, T, D, t1 - t0, t3 - t2);
            return 0;
        }
        Tensor l1 = y * dO;
        l1.backward();  // stage 1: dV and dS
        if (!sm.grad()) { std::fprintf(stderr, "stage 1 produced no dS\n"); return 3; }
        Tensor dS = sm.Getgrad();
        dS.set_requires_grad(false);
        Tensor l2 = s1 * dS;
        l2.backward();  // stage 2: scale, MMBackward(q, kt), contiguous/transpose backward
        if (!q.grad() || !k.grad() || !v.grad()) { std::fprintf(stderr, "missing gradient\n"); return 3; }
        Tensor dq = q.Getgrad().contiguous();
        Tensor dk = k.Getgrad().contiguous();
        Tensor dv = v.Getgrad().contiguous();
        if (on_cuda) { (void)dq.to(Inferno::Device::cpu()); (void)dk.to(Inferno::Device::cpu()); (void)dv.to(Inferno::Device::cpu()); }
        t3 = now_ms();
        if (last) {
            write_tensor(prefix + ".dq.bin", dq, n);
            write_tensor(prefix + ".dk.bin", dk, n);
            write_tensor(prefix + ".dv.bin", dv, n);
        }
    }
    if (!last) continue;
    std::printf("{\"device\": \"%s\", \"B\": %zu, \"H\": %zu, \"T\": %zu, \"D\": %zu, \"fwd_ms\": %.3f, \"bwd_ms\": %.3f}\n",
                argv[1], B, H, T, D, t1 - t0, t3 - t2);
    return 0;
    }
    return 0;
}
