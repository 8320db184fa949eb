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

// First element of the tensor (offset() counts elements of the tensor's own type).
void* dev_ptr(const Tensor& t) {
    auto impl = GetImpl(t);
    return t.dtype() == DType::BFloat16 ? static_cast<void*>(impl->data_as_ptr<unsigned short>() + t.offset())
                                        : static_cast<void*>(impl->data_as_ptr<float>() + t.offset());
}
float* dev_f32(const Tensor& t) { return static_cast<float*>(dev_ptr(t)); }

// Scratch for the kernels: one Inferno tensor (CUDAStorage = cudaMalloc RAII, src/inferno/storage/cudastorage.cpp:16-23)
// kept for the life of the process and grown on demand, so that a call neither allocates nor frees (cudaFree
// synchronises the device) and the sticky status word in its header survives from call to call.  The reference is
// single-threaded with one CUDA device (src/inferno/gradengine/engine.cpp:6), and so is this cache.
// The holder is never destroyed: at process exit the reference's own bookkeeping statics (node tracker, id broker) may
// already be gone when a Tensor destructor would reach for them.
Tensor& workspace_tensor() {
    static Tensor* t = new Tensor();
    return *t;
}
size_t g_workspace_bytes = 0;
void* workspace(size_t bytes, const Device& dev) {
    if (bytes > g_workspace_bytes) {
        causal_attention_check();                       // read the old buffer's status word before it goes
        workspace_tensor() = Tensor(DType::Float32, std::vector<size_t>{bytes / 4 + 64}, "attention_ws", dev);
        g_workspace_bytes = bytes;
    }
    return dev_ptr(workspace_tensor());
}

void check(int rc, const char* what) {
    if (rc != IB200_OK) fail(std::string(what) + ": " + ib200_status_string(rc));
}

// Raw device storage for n bf16 values, allocated like any other Inferno tensor (two bf16 per Float32 element).
Tensor make_bf16_buffer(size_t n, const char* name, const Device& dev) {
    return Tensor(DType::Float32, std::vector<size_t>{n / 2 + 8}, name, dev);
}

}  // namespace

void causal_attention_check() {
    if (g_workspace_bytes == 0) return;
    int code = 0;
    const int rc = ib200_attn_check(dev_ptr(workspace_tensor()), nullptr, &code);
    if (rc != IB200_OK) fail(std::string(ib200_status_string(rc)) + " (device code " + std::to_string(code) + ")");
}

Tensor causal_attention(const Tensor& q_in, const Tensor& k_in, const Tensor& v_in, float scale, AttentionMath math) {
    if (q_in.device() != k_in.device() || q_in.device() != v_in.device()) fail("tensors are on different devices");
    if (q_in.ndim() != 4 || q_in.shape() != k_in.shape() || q_in.shape() != v_in.shape()) fail("expects q, k, v of equal shape [B, H, T, D]");
    if (q_in.dtype() != k_in.dtype() || q_in.dtype() != v_in.dtype()) fail("q, k, v must have one dtype");
    if (q_in.dtype() != DType::Float32 && q_in.dtype() != DType::BFloat16) fail("expects Float32 or BFloat16 tensors");
    const bool native16 = q_in.dtype() == DType::BFloat16;      // the tensors' own storage is what the bf16 kernels read
    if (native16 && !(q_in.is_contiguous() && k_in.is_contiguous() && v_in.is_contiguous()))
        fail("BFloat16 tensors must be dense (contiguous() has no BFloat16 arm)");

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
    const size_t n = q.numel();
    const bool bf16 = !native16 && math == AttentionMath::BFloat16;      // Float32 tensors through bf16 copies
    const int dtype = (bf16 || native16) ? IB200_DTYPE_BF16 : IB200_DTYPE_F32;

    const bool gradreq = grad_enabled && (q_in.requires_grad() || k_in.requires_grad() || v_in.requires_grad());
    Tensor out(q.dtype(), shp, "attention", q.device(), gradreq);
    Tensor lse(DType::Float32, std::vector<size_t>{shp[0], shp[1], shp[2]}, "attention_lse", q.device());

    // what the kernels read and write: the tensors themselves, or bf16 copies of them
    Tensor sq = q, sk = k, sv = v, sout = out;
    if (bf16) {
        sq = make_bf16_buffer(n, "attention_q_bf16", q.device());
        sk = make_bf16_buffer(n, "attention_k_bf16", q.device());
        sv = make_bf16_buffer(n, "attention_v_bf16", q.device());
        sout = make_bf16_buffer(n, "attention_out_bf16", q.device());
        check(ib200_cast_f32_to_bf16(dev_f32(q), dev_ptr(sq), n, nullptr), "cast q");
        check(ib200_cast_f32_to_bf16(dev_f32(k), dev_ptr(sk), n, nullptr), "cast k");
        check(ib200_cast_f32_to_bf16(dev_f32(v), dev_ptr(sv), n, nullptr), "cast v");
    }

    size_t ws_bytes = 0;
    check(ib200_attn_workspace_bytes(B, H, T, D, dtype, IB200_PASS_FWD, &ws_bytes), "workspace query");
    void* ws = workspace(ws_bytes, q.device());
    // the reference launches everything on the legacy default stream
    check(ib200_attn_fwd(dev_ptr(sq), dev_ptr(sk), dev_ptr(sv), dev_ptr(sout), dev_f32(lse), B, H, T, D, scale, /*causal=*/1,
                         dtype, IB200_MATH_SPLIT_BF16, ws, g_workspace_bytes, nullptr),
          "forward");
    if (bf16) check(ib200_cast_bf16_to_f32(dev_ptr(sout), dev_f32(out), n, nullptr), "widen y");

    if (gradreq) GetImpl(out)->gradfn() = std::make_shared<AttentionBackward>(q_in, k_in, v_in, sq, sk, sv, sout, lse, scale, math);
    return out;
}

AttentionBackward::AttentionBackward(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& sq, const Tensor& sk, const Tensor& sv,
                                     const Tensor& sout, const Tensor& lse, float scale, AttentionMath math)
    : m_q(q), m_k(k), m_v(v), m_sq(sq), m_sk(sk), m_sv(sv), m_sout(sout), m_lse(lse), m_scale(scale), m_math(math) {
    set_name("AttentionBackward");
}

void AttentionBackward::backward() {
    NoGradGuard guard;
    Tensor g_out = Engine::grad_in(this, 0).contiguous();
    const auto& shp = m_q.shape();
    const int B = static_cast<int>(shp[0]), H = static_cast<int>(shp[1]), T = static_cast<int>(shp[2]), D = static_cast<int>(shp[3]);
    const size_t n = m_q.numel();
    const bool native16 = m_q.dtype() == DType::BFloat16;
    const bool bf16 = !native16 && m_math == AttentionMath::BFloat16;
    const int dtype = (bf16 || native16) ? IB200_DTYPE_BF16 : IB200_DTYPE_F32;
    const Device dev = m_q.device();
    if (g_out.dtype() != m_q.dtype()) fail("the upstream gradient must have the dtype of q, k, v");
    // Float32 math saved the inputs themselves; they may have been views, so make them dense again
    Tensor sq = bf16 ? m_sq : m_sq.contiguous(), sk = bf16 ? m_sk : m_sk.contiguous(), sv = bf16 ? m_sv : m_sv.contiguous();

    Tensor dq(m_q.dtype(), shp, "attention_dq", dev);
    Tensor dk(m_q.dtype(), shp, "attention_dk", dev);
    Tensor dv(m_q.dtype(), shp, "attention_dv", dev);
    Tensor sdo = g_out, sdq = dq, sdk = dk, sdv = dv;
    if (bf16) {
        sdo = make_bf16_buffer(n, "attention_do_bf16", dev);
        sdq = make_bf16_buffer(n, "attention_dq_bf16", dev);
        sdk = make_bf16_buffer(n, "attention_dk_bf16", dev);
        sdv = make_bf16_buffer(n, "attention_dv_bf16", dev);
        check(ib200_cast_f32_to_bf16(dev_f32(g_out), dev_ptr(sdo), n, nullptr), "cast dO");
    }
    size_t ws_bytes = 0;
    check(ib200_attn_workspace_bytes(B, H, T, D, dtype, IB200_PASS_BWD, &ws_bytes), "workspace query");
    void* ws = workspace(ws_bytes, dev);
    check(ib200_attn_bwd(dev_ptr(sq), dev_ptr(sk), dev_ptr(sv), dev_ptr(m_sout), dev_ptr(sdo), dev_f32(m_lse), dev_ptr(sdq), dev_ptr(sdk),
                         dev_ptr(sdv), B, H, T, D, m_scale, 1, dtype, IB200_MATH_SPLIT_BF16, ws, g_workspace_bytes, nullptr),
          "backward");
    if (bf16) {
        check(ib200_cast_bf16_to_f32(dev_ptr(sdq), dev_f32(dq), n, nullptr), "widen dq");
        check(ib200_cast_bf16_to_f32(dev_ptr(sdk), dev_f32(dk), n, nullptr), "widen dk");
        check(ib200_cast_bf16_to_f32(dev_ptr(sdv), dev_f32(dv), n, nullptr), "widen dv");
    }

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
    m_sq = Tensor{};
    m_sk = Tensor{};
    m_sv = Tensor{};
    m_sout = Tensor{};
    m_lse = Tensor{};
}

void AttentionBackward::get_inputs(std::vector<Tensor>& out) const {
    out.push_back(m_q);
    out.push_back(m_k);
    out.push_back(m_v);
}

}  // namespace Inferno
