// TEST INFRASTRUCTURE ONLY.  Proves that the fused op drops into the reference: it is compiled against
// the reference's own headers and objects, run on Device::cuda(0), and its gradients are produced by the
// reference's autograd Engine walking the AttentionBackward node (seeded through a multiply, because
// Engine::backward always seeds ones, src/inferno/gradengine/engine.cpp:59).
// Usage: shim_check B H T D q.bin k.bin v.bin do.bin out_prefix [bf16 | native16]   -> writes <prefix>.{o,dq,dk,dv}.bin
// With the trailing "bf16" the op runs in AttentionMath::BFloat16 (Float32 tensors, bf16 kernels).  With "native16"
// q, k, v are converted to BFloat16 TENSORS first (to_dtype, a graph op with its own backward node), the op receives
// those and hands their storage to the kernels, and its BFloat16 output is converted back for the loss: the Engine
// walks MultiplyBackward -> CastBackward -> AttentionBackward -> CastBackward x3.
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include <inferno/inferno.h>
#include "inferno/core/ops_impl.h"
#include "inferno/core/tensorimpl.h"

#include "../inferno_b200/inferno_shim/bf16_dtype.h"
#include "../inferno_b200/inferno_shim/causal_attention.h"

using Inferno::Tensor;

static std::vector<float> read_bin(const char* path, size_t n) {
    std::vector<float> v(n);
    FILE* f = std::fopen(path, "rb");
    if (!f || std::fread(v.data(), sizeof(float), n, f) != n) { std::fprintf(stderr, "cannot read %s\n", path); std::exit(2); }
    std::fclose(f);
    return v;
}
static void write_tensor(const std::string& path, const Tensor& t_in, size_t n) {
    Tensor t = t_in.contiguous().to(Inferno::Device::cpu());
    const float* p = Inferno::GetImpl(t)->data_as_ptr<float>() + t.offset();
    FILE* f = std::fopen(path.c_str(), "wb");
    std::fwrite(p, sizeof(float), n, f);
    std::fclose(f);
}

int main(int argc, char** argv) {
    if (argc < 10) { std::fprintf(stderr, "usage: %s B H T D q k v do out_prefix\n", argv[0]); return 2; }
    const size_t B = std::strtoul(argv[1], nullptr, 10), H = std::strtoul(argv[2], nullptr, 10);
    const size_t T = std::strtoul(argv[3], nullptr, 10), D = std::strtoul(argv[4], nullptr, 10);
    const size_t n = B * H * T * D;
    const std::string prefix = argv[9];
    Inferno::Device dev = Inferno::Device::cuda(0);
    std::vector<float> hq = read_bin(argv[5], n), hk = read_bin(argv[6], n), hv = read_bin(argv[7], n), hdo = read_bin(argv[8], n);
    Tensor q(Inferno::DType::Float32, hq, {B, H, T, D}, "q", dev, true);
    Tensor k(Inferno::DType::Float32, hk, {B, H, T, D}, "k", dev, true);
    Tensor v(Inferno::DType::Float32, hv, {B, H, T, D}, "v", dev, true);
    Tensor dO(Inferno::DType::Float32, hdo, {B, H, T, D}, "dO", dev, false);

    const bool bf16 = argc > 10 && std::string(argv[10]) == "bf16";
    const bool native16 = argc > 10 && std::string(argv[10]) == "native16";
    const float scale = 1.0f / std::sqrt(static_cast<float>(D));
    Tensor y;
    if (native16) {
        Tensor qb = Inferno::to_dtype(q, Inferno::DType::BFloat16), kb = Inferno::to_dtype(k, Inferno::DType::BFloat16),
               vb = Inferno::to_dtype(v, Inferno::DType::BFloat16);
        Tensor yb = Inferno::causal_attention(qb, kb, vb, scale);
        if (yb.dtype() != Inferno::DType::BFloat16) { std::fprintf(stderr, "output is not BFloat16\n"); return 4; }
        y = Inferno::to_dtype(yb, Inferno::DType::Float32);
    } else {
        y = Inferno::causal_attention(q, k, v, scale, bf16 ? Inferno::AttentionMath::BFloat16 : Inferno::AttentionMath::Float32);
    }
    write_tensor(prefix + ".o.bin", y, n);
    Tensor loss = y * dO;          // MultiplyBackward hands dO to AttentionBackward
    loss.backward();
    if (!q.grad() || !k.grad() || !v.grad()) { std::fprintf(stderr, "a gradient did not arrive\n"); return 3; }
    write_tensor(prefix + ".dq.bin", q.Getgrad(), n);
    write_tensor(prefix + ".dk.bin", k.Getgrad(), n);
    write_tensor(prefix + ".dv.bin", v.Getgrad(), n);
    Inferno::causal_attention_check();      // no bounded device-side wait expired in any of the calls above
    std::printf("shim_check ok\n");
    return 0;
}
