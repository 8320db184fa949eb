// See causal_attention.h.  The shape of this file follows the reference's ops: validate, make inputs
// dense, allocate the output Tensor, take raw device pointers from the TensorImpl, switch on the device
// type, call the launcher, attach the backward node (compare multiply(): src/inferno/core/ops.cpp:204-270).
#include "causal_attention.h"

#include <cstdlib>
#include <string>

#include "inferno/core/ops_impl.h"
#include "inferno/core/tensorimpl.h"
#include "inferno/util/logger.h"
#include "inferno_b200_attn.h"

namespace Inferno {

namespace {

[[noreturn]] void fail(const std::string& msg) {
    Logger::Append(Logger::LogLevel::LOGLEVEL_ERROR, "causal_attention: " + msg);
    std::exit(1);
}

float* dev_ptr(const Tensor& t) { return GetImpl(t)->data_as_ptr<float>() + t.offset(); }

// Scratch for the kernels, allocated like any other Inferno tensor (CUDAStorage = cudaMalloc RAII,
// src/inferno/storage/cudastorage.cpp:16-23) and released when it goes out of scope.
Tensor make_workspace(size_t bytes, const Device& dev) {
    return Tensor(DType::Float32, std::vector<size_t>{bytes / 4 + 64}, "attention_ws", dev);
}

void check(int rc, const char* what) {
    if (rc != IB200_OK) fail(std::string(what) + ": " + ib200_status_string(rc));
}

}  // namespace

Tensor causal_attention(const Tensor& q_in, const Tensor& k_in, const Tensor& v_in, float scale) {
    if (q_in.device() != k_in.device() || q_in.device() != v_in.device()) fail("tensors are on different devices");
    if (q_in.ndim() != 4 || q_in.shape() != k_in.shape() || q_in.shape() != v_in.shape()) fail("expects q, k, v of equal shape [B, H, T, D]");
    if (q_in.dtype() != DType::Float32 || k_in.dtype() != DType::Float32 || v_in.dtype() != DType::Float32) fail("expects Float32 tensors");

    switch (q_in.device().m_type) {
        case DeviceType::CUDA: break;
        default:
            // There is deliberately no CPU kernel: on the CPU device the stock composition of
            // matmul / masked_fill / Softmax (InfernoApp/main.cpp:737-754) is the implementation.
            fail("only the CUDA device is implemented");
    }

    Tensor q = q_in.contiguous(), k = k_in.contiguous(), v = v_in.contiguous();
    const auto& shp = q.shape();
    const int B = static_cast<int>(shp[0]), H = static_cast<int>(shp[1]), T = static_cast<int>(shp[2]), D = static_cast<int>(shp[3]);

    const bool gradreq = grad_enabled && (q_in.requires_grad() || k_in.requires_grad() || v_in.requires_grad());
    Tensor out(DType::Float32, shp, "attention", q.device(), gradreq);
    Tensor lse(DType::Float32, std::vector<size_t>{shp[0], shp[1], shp[2]}, "attention_lse", q.device());

    size_t ws_bytes = 0;
    check(ib200_attn_workspace_bytes(B, H, T, D, IB200_DTYPE_F32, IB200_PASS_FWD, &ws_bytes), "workspace query");
    Tensor ws = make_workspace(ws_bytes, q.device());
    // the reference launches everything on the legacy default stream
    check(ib200_attn_fwd(dev_ptr(q), dev_ptr(k), dev_ptr(v), dev_ptr(out), dev_ptr(lse), B, H, T, D, scale, /*causal=*/1,
                         IB200_DTYPE_F32, IB200_MATH_TF32, dev_ptr(ws), ws_bytes, nullptr),
          "forward");
    int code = 0;
    check(ib200_attn_check(dev_ptr(ws), nullptr, &code), "forward (device status)");

    if (gradreq) GetImpl(out)->gradfn() = std::make_shared<AttentionBackward>(q_in, k_in, v_in, out, lse, scale);
    return out;
}

AttentionBackward::AttentionBackward(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out, const Tensor& lse, float scale)
    : m_q(q), m_k(k), m_v(v), m_out(out), m_lse(lse), m_scale(scale) {
    set_name("AttentionBackward");
}

void AttentionBackward::backward() {
    NoGradGuard guard;
    Tensor g_out = Engine::grad_in(this, 0).contiguous();
    Tensor q = m_q.contiguous(), k = m_k.contiguous(), v = m_v.contiguous();
    const auto& shp = q.shape();
    const int B = static_cast<int>(shp[0]), H = static_cast<int>(shp[1]), T = static_cast<int>(shp[2]), D = static_cast<int>(shp[3]);

    Tensor dq(DType::Float32, shp, "attention_dq", q.device());
    Tensor dk(DType::Float32, shp, "attention_dk", q.device());
    Tensor dv(DType::Float32, shp, "attention_dv", q.device());
    size_t ws_bytes = 0;
    check(ib200_attn_workspace_bytes(B, H, T, D, IB200_DTYPE_F32, IB200_PASS_BWD, &ws_bytes), "workspace query");
    Tensor ws = make_workspace(ws_bytes, q.device());
    check(ib200_attn_bwd(dev_ptr(q), dev_ptr(k), dev_ptr(v), dev_ptr(m_out), dev_ptr(g_out), dev_ptr(m_lse), dev_ptr(dq), dev_ptr(dk),
                         dev_ptr(dv), B, H, T, D, m_scale, 1, IB200_DTYPE_F32, IB200_MATH_TF32, dev_ptr(ws), ws_bytes, nullptr),
          "backward");
    int code = 0;
    check(ib200_attn_check(dev_ptr(ws), nullptr, &code), "backward (device status)");

    // send gradients upstream (same pattern as MultiplyBackward::backward, src/inferno/gradfn/multiplybackward.cpp:34-57)
    auto nq = GetImpl(m_q)->grad_edge();
    auto nk = GetImpl(m_k)->grad_edge();
    auto nv = GetImpl(m_v)->grad_edge();
    if (nq) Engine::accumulate(nq.get(), 0, dq);
    if (nk) Engine::accumulate(nk.get(), 0, dk);
    if (nv) Engine::accumulate(nv.get(), 0, dv);
}

void AttentionBackward::release() {
    m_q = Tensor{};
    m_k = Tensor{};
    m_v = Tensor{};
    m_out = Tensor{};
    m_lse = Tensor{};
}

void AttentionBackward::get_inputs(std::vector<Tensor>& out) const {
    out.push_back(m_q);
    out.push_back(m_k);
    out.push_back(m_v);
}

}  // namespace Inferno
