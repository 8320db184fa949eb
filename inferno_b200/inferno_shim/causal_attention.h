// Fused causal attention as an Inferno op, written in the reference's own operator idiom.
//
// Stands where InfernoApp/main.cpp:737-754 composes
//     kt = k.transpose(-1,-2).contiguous(); matmul; * scale; masked_fill(triu mask, -1e9); Softmax; matmul
// and is used the same way as any other free op of namespace Inferno (src/inferno/core/ops.cpp):
//     Inferno::Tensor y = Inferno::causal_attention(q, k, v, scale);      // q, k, v: [B, H, T, D] Float32 on a CUDA device
// It needs the reference's headers (include/ and src/ of the Inferno tree) and links against
// libinferno_b200_attn.so; nothing of the reference is modified.
#pragma once

#include <inferno/core/tensor.h>

#include "inferno/gradengine/engine.h"

namespace Inferno {

// y = softmax(mask(q k^T * scale)) v with a causal mask.  Attaches an AttentionBackward node to y
// when gradients are enabled and any input requires them.  Errors follow the reference's
// convention (log + exit(1), src/inferno/core/ops.cpp:44-47).
Tensor causal_attention(const Tensor& q, const Tensor& k, const Tensor& v, float scale);

// Backward node of causal_attention (interface: src/inferno/gradfn/node.h:23-45).
class AttentionBackward : public Node {
public:
    AttentionBackward(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out, const Tensor& lse, float scale);
    void backward() override;
    void release() override;
    void get_inputs(std::vector<Tensor>& out) const override;

private:
    Tensor m_q, m_k, m_v, m_out, m_lse;
    float m_scale;
};

}  // namespace Inferno
