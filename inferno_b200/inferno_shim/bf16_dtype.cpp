// See bf16_dtype.h.  Shaped like the reference's ops: validate, allocate the output Tensor, raw device pointers from the
// TensorImpl, call the launcher, attach the backward node (compare multiply(): src/inferno/core/ops.cpp:204-270).
#include "bf16_dtype.h"

#include <cstdlib>
#include <string>

#include "inferno/core/ops_impl.h"
#include "inferno/core/tensorimpl.h"
#include "inferno/util/logger.h"
#include "inferno_b200_attn.h"

namespace Inferno {

namespace {

[[noreturn]] void fail(const std::string& msg) {
    Logger::Append(Logger::LogLevel::LOGLEVEL_ERROR, "to_dtype: " + msg);
    std::exit(1);
}

// n elements of the tensor's own type starting at its offset
void* raw(const Tensor& t) {
    auto impl = GetImpl(t);
    return t.dtype() == DType::BFloat16 ? static_cast<void*>(impl->data_as_ptr<unsigned short>() + t.offset())
                                        : static_cast<void*>(impl->data_as_ptr<float>() + t.offset());
}

Tensor convert(const Tensor& t, DType dst) {
    const DType src = t.dtype();
    const bool down = src == DType::Float32 && dst == DType::BFloat16, up = src == DType::BFloat16 && dst == DType::Float32;
    if (!down && !up) fail("only Float32 <-> BFloat16 is implemented");
    if (!t.device().is_cuda()) fail("only the CUDA device is implemented");
    if (!t.is_contiguous()) fail("expects a dense tensor (contiguous() has no BFloat16 arm)");
    const size_t n = t.numel();
    if (n % 8) fail("element count must be a multiple of 8");
    Tensor out(dst, t.shape(), t.name() + (down ? "_bf16" : "_f32"), t.device());
    const int rc = down ? ib200_cast_f32_to_bf16(static_cast<const float*>(raw(t)), raw(out), n, nullptr)
                        : ib200_cast_bf16_to_f32(raw(t), static_cast<float*>(raw(out)), n, nullptr);
    if (rc != IB200_OK) fail(ib200_status_string(rc));
    return out;
}

}  // namespace

Tensor to_dtype(const Tensor& t, DType dst) {
    if (t.dtype() == dst) return t;
    Tensor out = convert(t, dst);
    if (grad_enabled && t.requires_grad()) {
        out.set_requires_grad(true);
        GetImpl(out)->gradfn() = std::make_shared<CastBackward>(t, t.dtype());
    }
    return out;
}

CastBackward::CastBackward(const Tensor& input, DType src) : m_input(input), m_src(src) { set_name("CastBackward"); }

void CastBackward::backward() {
    NoGradGuard guard;
    Tensor g_out = Engine::grad_in(this, 0);
    Tensor g_in = g_out.dtype() == m_src ? g_out : convert(g_out, m_src);
    if (auto edge = GetImpl(m_input)->grad_edge()) Engine::accumulate(edge.get(), 0, g_in);
}

void CastBackward::release() { m_input = Tensor{}; }

void CastBackward::get_inputs(std::vector<Tensor>& out) const { out.push_back(m_input); }

}  // namespace Inferno
