// See autograd_patches.h.  Shaped like the reference's own nodes (compare MultiplyBackward,
// src/inferno/gradfn/multiplybackward.cpp:34-57).
#include "autograd_patches.h"

#include <inferno/core/ops.h>

#include "inferno/core/ops_impl.h"
#include "inferno/core/tensorimpl.h"

namespace Inferno {

MaskedFillBackward::MaskedFillBackward(const Tensor& input, const Tensor& mask) : m_input(input), m_mask(mask) {
    set_name("MaskedFillBackward");
}

void MaskedFillBackward::backward() {
    NoGradGuard guard;
    Tensor g_out = Engine::grad_in(this, 0);
    // filled positions do not depend on the input: their gradient is zero
    Tensor g_in = masked_fill(g_out, m_mask, 0.0f);
    if (auto edge = GetImpl(m_input)->grad_edge()) Engine::accumulate(edge.get(), 0, g_in);
}

void MaskedFillBackward::release() {
    m_input = Tensor{};
    m_mask = Tensor{};
}

void MaskedFillBackward::get_inputs(std::vector<Tensor>& out) const { out.push_back(m_input); }

Tensor masked_fill_with_grad(const Tensor& input, const Tensor& mask, float value) {
    Tensor out = masked_fill(input, mask, value);
    if (grad_enabled && input.requires_grad()) {
        out.set_requires_grad(true);
        GetImpl(out)->gradfn() = std::make_shared<MaskedFillBackward>(input, mask);
    }
    return out;
}

Tensor contiguous_with_grad(const Tensor& input) {
    Tensor out = input.contiguous();
    // a dense input is returned as is; a copy carries a ContiguousBackward node that only becomes reachable once the
    // copy itself requires a gradient
    if (grad_enabled && input.requires_grad() && !out.requires_grad()) out.set_requires_grad(true);
    return out;
}

void backward_with_seed(const Tensor& t, const Tensor& grad) {
    Tensor seed = grad;
    seed.set_requires_grad(false);
    Tensor weighted = t * seed;
    weighted.backward();
}

}  // namespace Inferno
