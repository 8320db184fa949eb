"""Drop-in proof: the fused op written in the reference's idiom (inferno_b200/inferno_shim), compiled against
the reference's own headers and objects (oracle/_ref/shim_check, built where the reference sources exist),
runs on the CUDA device and has its gradients delivered by the reference's autograd Engine."""
import os
import subprocess
import tempfile

import numpy as np
import pytest

from inferno_b200.synth import CONFIGS, make_config_inputs, make_inputs

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "oracle", "_ref", "shim_check")


def run_binary(binary, args, q, k, v, do, tail=()):
    B, H, T, D = q.shape
    with tempfile.TemporaryDirectory() as td:
        for name, arr in (("q", q), ("k", k), ("v", v), ("do", do)):
            np.ascontiguousarray(arr, dtype=np.float32).tofile(os.path.join(td, name + ".bin"))
        prefix = os.path.join(td, "out")
        cmd = [binary] + args + [str(B), str(H), str(T), str(D)] + [os.path.join(td, n + ".bin") for n in ("q", "k", "v", "do")] + [prefix] + list(tail)
        subprocess.run(cmd, check=True, cwd=td, capture_output=True, timeout=300)
        return [np.fromfile(f"{prefix}.{s}.bin", dtype=np.float32).reshape(B, H, T, D) for s in ("o", "dq", "dk", "dv")]


@pytest.mark.parametrize("shape", ["c1", (1, 2, 200, 64)])
def test_inferno_idiom_op_and_engine_backward(oracle_mod, shape):
    if not os.path.isfile(SHIM):
        pytest.skip("oracle/_ref/shim_check not built (reference sources absent at build time)")
    if shape == "c1":
        q, k, v, do = make_config_inputs(CONFIGS["c1"])
    else:
        q, k, v, do = make_inputs(*shape, 41)
    outs = run_binary(SHIM, [], q, k, v, do)
    refs = oracle_mod.oracle_f32(q, k, v, do)
    for name, x, r in zip(("O", "dQ", "dK", "dV"), outs, refs):
        err = oracle_mod.rel_err(x, r)
        assert err < 1e-3, f"{name}: rel err {err:.3e}"


@pytest.mark.parametrize("shape", [(1, 2, 200, 64), (2, 2, 384, 128)])
def test_inferno_idiom_op_bf16_math(oracle_mod, shape):
    """AttentionMath::BFloat16: Float32 Inferno tensors in and out, bf16 kernels in between (the only way the
    reference's tensors reach head dim 128); parity with the fp64 evaluator at the bf16 tolerance."""
    if not os.path.isfile(SHIM):
        pytest.skip("oracle/_ref/shim_check not built (reference sources absent at build time)")
    q, k, v, do = make_inputs(*shape, 43)
    outs = run_binary(SHIM, [], q, k, v, do, tail=["bf16"])
    refs = oracle_mod.attn_fp64(q, k, v, do)
    for name, x, r in zip(("O", "dQ", "dK", "dV"), outs, refs):
        err = oracle_mod.rel_err(x, r)
        assert err < 2e-2, f"{name}: rel err {err:.3e}"


@pytest.mark.parametrize("shape", [(1, 2, 200, 64), (2, 2, 384, 128)])
def test_inferno_idiom_op_on_bfloat16_tensors(oracle_mod, shape):
    """DType::BFloat16 tensors (the reference's dtype enum and dtype_size given one more entry): the op hands the tensors'
    own storage to the bf16 kernels, returns a BFloat16 tensor, and the reference's Engine delivers BFloat16 gradients
    through AttentionBackward; to_dtype (with its CastBackward node) sits either side only because the harness reads and
    writes fp32 files.  The operands are bf16-representable, so nothing but the kernels' own rounding separates the
    result from the float64 evaluation."""
    if not os.path.isfile(SHIM):
        pytest.skip("oracle/_ref/shim_check not built (reference sources absent at build time)")
    q, k, v, do = make_inputs(*shape, 47, 1.0, 0.5, "bf16")
    outs = run_binary(SHIM, [], q, k, v, do, tail=["native16"])
    refs = oracle_mod.attn_fp64(q, k, v, do)
    for name, x, r in zip(("O", "dQ", "dK", "dV"), outs, refs):
        err = oracle_mod.rel_err(x, r)
        assert err < 2e-2, f"{name}: rel err {err:.3e}"


def test_against_the_reference_cuda_path(oracle_mod):
    """The reference's own composed CUDA path (cuBLAS SGEMM + its SIMT kernels, compiled for sm_100a) on
    configuration 1, against this library through the C ABI."""
    if not oracle_mod.have_ref():
        pytest.skip("oracle/_ref/ref_attention not built")
    import torch
    from inferno_b200 import attention as A
    q, k, v, do = make_config_inputs(CONFIGS["c1"])
    refs = run_binary(oracle_mod.REF_BIN, ["cuda"], q, k, v, do)
    tq, tk, tv, tdo = (torch.from_numpy(a).cuda() for a in (q, k, v, do))
    o, lse = A.attention_forward(tq, tk, tv)
    grads = A.attention_backward(tq, tk, tv, o, tdo, lse)
    torch.cuda.synchronize()
    for name, x, r in zip(("O", "dQ", "dK", "dV"), (o,) + tuple(grads), refs):
        err = oracle_mod.rel_err(x.cpu().numpy(), r)
        assert err < 1e-3, f"{name}: rel err {err:.3e}"
