// Autograd-correctness additions for the reference's composed attention path, written in the reference's own
// operator idiom and living beside it (nothing of the reference is modified).
//
// As shipped, the graph that InfernoApp/main.cpp:737-754 builds is cut in two places, so q and k never receive a
// gradient from the composed path:
//   * masked_fill returns a tensor with requires_grad = false and attaches no backward node
//     (src/inferno/core/ops.cpp:1235-1289);
//   * contiguous attaches a ContiguousBackward node but leaves requires_grad = false on its output, and
//     TensorImpl::grad_edge returns nullptr for such a tensor (src/inferno/core/ops.cpp:1302-1342,
//     src/inferno/core/tensorimpl.cpp:389-396), so the node is unreachable;
// and Engine::backward always seeds ones (src/inferno/gradengine/engine.cpp:59-60), so an upstream gradient cannot be
// injected.  The three functions below close those gaps; with them the stock composition is a valid end-to-end
// gradient oracle for the fused op (one backward pass instead of the two-stage workaround).
#pragma once

#include <inferno/core/tensor.h>

#include "inferno/gradengine/engine.h"

namespace Inferno {

// masked_fill with a backward node: out = value where mask != 0, else input; d(input) = d(out) where mask == 0, else 0.
Tensor masked_fill_with_grad(const Tensor& input, const Tensor& mask, float value);

// contiguous whose output stays part of the graph when the input requires a gradient.
Tensor contiguous_with_grad(const Tensor& input);

// Engine::backward with a caller-supplied upstream gradient: d(sum(t * grad)) = grad, so the stock ones-seeded
// engine delivers `grad` to t's producers.
void backward_with_seed(const Tensor& t, const Tensor& grad);

// Backward node of masked_fill_with_grad (interface: src/inferno/gradfn/node.h:23-45).
class MaskedFillBackward : public Node {
public:
    MaskedFillBackward(const Tensor& input, const Tensor& mask);
    void backward() override;
    void release() override;
    void get_inputs(std::vector<Tensor>& out) const override;

private:
    Tensor m_input, m_mask;
};

}  // namespace Inferno
