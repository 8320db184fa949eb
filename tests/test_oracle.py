"""The CPU checkers against the reference's own outputs (golden vectors) and against each other."""

import numpy as np
import pytest

from inferno_b200.synth import make_inputs
from golden_cases import MANIFEST, load_case


@pytest.mark.parametrize("name", sorted(MANIFEST))
def test_c_restatement_matches_reference_bit_exact(oracle_mod, name):
    """attn_oracle.c reproduces the compiled reference's outputs bit for bit."""
    _, (q, k, v, do), gold = load_case(name)
    out = oracle_mod.oracle_f32(q, k, v, do)
    for key, arr in zip(("o", "dq", "dk", "dv"), out):
        assert np.array_equal(arr, gold[key]), key


@pytest.mark.parametrize("name", sorted(MANIFEST))
def test_fp64_evaluator_agrees_with_reference(oracle_mod, name):
    _, (q, k, v, do), gold = load_case(name)
    out = oracle_mod.attn_fp64(q, k, v, do)
    for key, arr in zip(("o", "dq", "dk", "dv"), out):
        assert oracle_mod.rel_err(gold[key], arr) < 2e-6, key


@pytest.mark.parametrize("name", ["tiny_t32_d16", "single_t1_d64"])
def test_compiled_reference_reproduces_golden(oracle_mod, name):
    if not oracle_mod.have_ref():
        pytest.skip("oracle/_ref/ref_attention not built (reference sources absent)")
    _, (q, k, v, do), gold = load_case(name)
    out = oracle_mod.ref_attention(q, k, v, do)[:4]
    for key, arr in zip(("o", "dq", "dk", "dv"), out):
        assert np.array_equal(arr, gold[key]), key


@pytest.mark.parametrize("name", ["tiny_t32_d16", "single_t1_d64"])
def test_single_pass_backward_with_autograd_additions(oracle_mod, name):
    """The reference's composed path, run as ONE engine pass through the shim's autograd additions (MaskedFillBackward,
    contiguous that stays in the graph, seeded backward), gives the gradients of the two-stage workaround bit for bit."""
    if not oracle_mod.have_ref():
        pytest.skip("oracle/_ref/ref_attention not built (reference sources absent)")
    _, (q, k, v, do), gold = load_case(name)
    out = oracle_mod.ref_attention(q, k, v, do, single_pass=True)[:4]
    for key, arr in zip(("o", "dq", "dk", "dv"), out):
        assert np.array_equal(arr, gold[key]), key


def test_known_answers(oracle_mod):
    # T = 1: softmax over one key is 1, so O = V, dV = dO, dQ = dK = 0.
    q, k, v, do = make_inputs(1, 2, 1, 8, 3)
    o, dq, dk, dv = oracle_mod.oracle_f32(q, k, v, do)
    assert np.array_equal(o, v) and np.array_equal(dv, do)
    assert np.all(dq == 0) and np.all(dk == 0)
    # Row 0 of any causal attention sees only key 0.
    q, k, v, do = make_inputs(1, 1, 16, 8, 4)
    o = oracle_mod.oracle_f32(q, k, v)[0]
    assert np.array_equal(o[0, 0, 0], v[0, 0, 0])
    # T = 2 by hand, D = 1: row 1 = softmax([q1 k0, q1 k1] * scale) . [v0, v1]
    q = np.array([0.5, 2.0], np.float32).reshape(1, 1, 2, 1)
    k = np.array([1.0, -1.0], np.float32).reshape(1, 1, 2, 1)
    v = np.array([3.0, 7.0], np.float32).reshape(1, 1, 2, 1)
    o = oracle_mod.oracle_f32(q, k, v, scale=1.0)[0]
    w = np.exp(np.array([2.0, -2.0]) - 2.0)
    w /= w.sum()
    assert abs(o[0, 0, 1, 0] - (w[0] * 3.0 + w[1] * 7.0)) < 1e-6
    assert o[0, 0, 0, 0] == 3.0


def test_causality_of_oracle(oracle_mod):
    q, k, v, do = make_inputs(1, 1, 24, 8, 5)
    o1 = oracle_mod.oracle_f32(q, k, v)[0]
    k2, v2 = k.copy(), v.copy()
    k2[..., 12:, :] += 1.0
    v2[..., 12:, :] -= 2.0
    o2 = oracle_mod.oracle_f32(q, k2, v2)[0]
    assert np.array_equal(o1[..., :12, :], o2[..., :12, :])
    assert not np.array_equal(o1[..., 12:, :], o2[..., 12:, :])


def test_masked_entries_are_exact_zero(oracle_mod):
    """The -1e9 fill underflows to exactly 0 after softmax (reference numerics), so the last key
    receives gradient from the last query only: dV[T-1] = P[T-1,T-1] * dO[T-1]."""
    q, k, v, do = make_inputs(1, 1, 8, 4, 6)
    _, _, _, dv = oracle_mod.oracle_f32(q, k, v, do)
    ratio = dv[0, 0, -1].astype(np.float64) / do[0, 0, -1].astype(np.float64)
    assert 0.0 < ratio[0] < 1.0
    assert np.allclose(ratio, ratio[0], rtol=1e-6, atol=0)
