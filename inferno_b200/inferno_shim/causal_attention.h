// Fused causal attention as an Inferno op, written in the reference's own operator idiom.
//
// Stands where InfernoApp/main.cpp:737-754 composes
//     kt = k.transpose(-1,-2).contiguous(); matmul; * scale; masked_fill(triu mask, -1e9); Softmax; matmul
// and is used the same way as any other free op of namespace Inferno (src/inferno/core/ops.cpp):
//     Inferno::Tensor y = Inferno::causal_attention(q, k, v, scale);      // q, k, v: [B, H, T, D] on a CUDA device
// q, k, v are Float32 tensors, or -- where the reference has been given a 16-bit DType (bf16_dtype.h) -- BFloat16
// tensors, whose storage then goes to the bf16 kernels as it is and whose output and gradients are BFloat16 too.
// It needs the reference's headers (include/ and src/ of the Inferno tree) and links against
// libinferno_b200_attn.so.
#pragma once

#include <inferno/core/tensor.h>

#include "inferno/gradengine/engine.h"

namespace Inferno {

// Arithmetic of the fused op for Float32 tensors (the stock reference has no 16-bit DType,
// include/inferno/core/dtype.h:17-26; BFloat16 tensors always run the bf16 kernels and ignore this argument):
//   Float32   fp32 operands (carried as bf16 hi + lo pairs on the tensor cores, error ~1e-5); head dim 64
//   BFloat16  q, k, v and the upstream gradient are rounded to bf16 on the device, the bf16 kernels run (head dim 64
//             or 128, fp32 accumulation), and y / dq / dk / dv are widened back to Float32: the tolerance is the bf16
//             one (2e-2 normwise), the saved activations take half the memory and the kernels run several times faster
enum class AttentionMath { Float32, BFloat16 };

// y = softmax(mask(q k^T * scale)) v with a causal mask.  Attaches an AttentionBackward node to y
// when gradients are enabled and any input requires them.  Errors follow the reference's
// convention (log + exit(1), src/inferno/core/ops.cpp:44-47).
Tensor causal_attention(const Tensor& q, const Tensor& k, const Tensor& v, float scale, AttentionMath math = AttentionMath::Float32);

// The kernels report an expired device-side wait through a sticky status word in the op's scratch buffer instead of
// stopping the process.  This reads it (synchronising the default stream): call it where the reference would call
// check_cuda (src/inferno/cuda/cudaops.h:198-210), e.g. once per training step; on a recorded failure it logs and
// exits like every other error of the reference.  The op itself never synchronises.
void causal_attention_check();

// Backward node of causal_attention (interface: src/inferno/gradfn/node.h:23-45).
class AttentionBackward : public Node {
public:
    // q, k, v: the op's inputs (graph edges).  sq, sk, sv, sout: what the backward kernels read - the same tensors for
    // Float32 math and for BFloat16 tensors, bf16 copies (raw storage) for Float32 tensors in BFloat16 math.
    AttentionBackward(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& sq, const Tensor& sk, const Tensor& sv,
                      const Tensor& sout, const Tensor& lse, float scale, AttentionMath math);
    void backward() override;
    void release() override;
    void get_inputs(std::vector<Tensor>& out) const override;

private:
    Tensor m_q, m_k, m_v, m_sq, m_sk, m_sv, m_sout, m_lse;
    float m_scale;
    AttentionMath m_math;
};

}  // namespace Inferno
