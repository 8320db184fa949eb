// A 16-bit floating-point DType for Inferno tensors, as far as the fused attention op needs one.
//
// The reference enumerates Float32 / Float64 / Int32 / Int8 / Bool (include/inferno/core/dtype.h:17-26) and its
// dispatch tags know int, float and double (src/inferno/core/dtype_dispatch.h:43-102, include/inferno/core/dtype_traits.h:6-20).
// Two edits inside the reference give it a BFloat16 tensor type (the recipe that applies them to a private mirror of
// the two files is in oracle/Makefile, target bf16 patches):
//   * include/inferno/core/dtype.h      one more enumerator, `BFloat16`, ahead of `Invalid`;
//   * src/inferno/core/tensorimpl.cpp   `case DType::BFloat16: return 2;` in TensorImpl::dtype_size (:321-329), which is
//                                        what the two TensorImpl constructors size their storage with (:38, :77).
// With those, `Tensor(DType::BFloat16, shape, name, Device::cuda(0))` allocates a bf16 tensor, it moves between
// devices (Tensor::to copies bytes, src/inferno/core/tensor.cpp:609-693), views of it work, and a dense bf16 tensor can
// be handed to Inferno::causal_attention, which passes its storage to the bf16 kernels as it is: no cast pass, no
// second copy of the activations.
// What is NOT added is a Tag<__nv_bfloat16> arm in dispatchAny / dispatchAnyTwo: such an arm instantiates every generic
// op of the reference (CPU loops over std:: math, SIMT kernels) for a type they were not written for.  Arithmetic on a
// BFloat16 tensor other than the ops declared here therefore still ends in the reference's "Unsupported dtype"
// error, and mixed-precision code moves between the types with to_dtype below -- the op a `Tensor::to(DType)` member
// would be.
#pragma once

#include <inferno/core/tensor.h>

#include "inferno/gradengine/engine.h"

namespace Inferno {

// Float32 <-> BFloat16 conversion of a dense tensor on the CUDA device (round to nearest even on the way down), through
// the library's cast kernels.  Differentiable: the result carries a CastBackward node that converts the incoming
// gradient back to the source type.  A tensor that already has the requested type is returned as it is.
Tensor to_dtype(const Tensor& t, DType dst);

// Backward node of to_dtype (interface: src/inferno/gradfn/node.h:23-45).
class CastBackward : public Node {
public:
    CastBackward(const Tensor& input, DType src);
    void backward() override;
    void release() override;
    void get_inputs(std::vector<Tensor>& out) const override;

private:
    Tensor m_input;
    DType m_src;
};

}  // namespace Inferno
