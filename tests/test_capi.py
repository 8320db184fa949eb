"""The C-ABI library: it loads, exports what the header declares, and validates arguments on the host.

No compute call is made here (there is no GPU); with valid arguments and no device the entry
points must fail loudly with IB200_ERR_NO_DEVICE rather than fall back to anything.
"""
import ctypes
import os
import re

import pytest

from inferno_b200 import _capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for fn in os.listdir(inc):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names.update(re.findall(r"\b(ib200_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol(built_lib):
    lib = ctypes.CDLL(built_lib)
    syms = declared_symbols()
    assert "ib200_attn_fwd" in syms and "ib200_attn_bwd" in syms and len(syms) >= 7
    for name in syms:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"


def test_binding_lists_match_header(built_lib):
    assert set(_capi.EXPORTS) <= set(declared_symbols())
    assert _capi.lib().ib200_version() >= 1000


def test_status_strings(built_lib):
    seen = set()
    for code in range(0, 8):
        s = _capi.status_string(code)
        assert s and s != "unknown status"
        seen.add(s)
    assert len(seen) == 8
    assert _capi.status_string(999) == "unknown status"


def test_workspace_query(built_lib):
    # bf16 forward needs only the status header; backward adds the fp32 dQ accumulator and delta
    assert _capi.workspace_bytes(2, 3, 100, 64, _capi.DTYPE_BF16, _capi.PASS_FWD) == 256
    n = 2 * 3 * 100 * 64
    bwd = _capi.workspace_bytes(2, 3, 100, 64, _capi.DTYPE_BF16, _capi.PASS_BWD)
    assert bwd >= 256 + 4 * n + 4 * 2 * 3 * 100
    # fp32 I/O carries hi/lo bf16 copies of the operands
    assert _capi.workspace_bytes(2, 3, 100, 64, _capi.DTYPE_F32, _capi.PASS_FWD) >= 256 + 6 * 2 * n
    assert _capi.workspace_bytes(2, 3, 100, 64, _capi.DTYPE_F32, _capi.PASS_BWD) >= bwd + 8 * 2 * n
    out = ctypes.c_size_t(0)
    L = _capi.lib()
    assert L.ib200_attn_workspace_bytes(1, 1, 16, 96, _capi.DTYPE_BF16, 0, ctypes.byref(out)) == _capi.ERR_UNSUPPORTED
    assert L.ib200_attn_workspace_bytes(1, 1, 16, 128, _capi.DTYPE_F32, 0, ctypes.byref(out)) == _capi.ERR_UNSUPPORTED
    assert L.ib200_attn_workspace_bytes(0, 1, 16, 64, _capi.DTYPE_BF16, 0, ctypes.byref(out)) == _capi.ERR_INVALID_ARGUMENT
    assert L.ib200_attn_workspace_bytes(1, 1, 16, 64, 7, 0, ctypes.byref(out)) == _capi.ERR_INVALID_ARGUMENT
    assert L.ib200_attn_workspace_bytes(1, 1, 16, 64, _capi.DTYPE_BF16, 2, ctypes.byref(out)) == _capi.ERR_INVALID_ARGUMENT
    assert L.ib200_attn_workspace_bytes(1, 1, 16, 64, _capi.DTYPE_BF16, 0, None) == _capi.ERR_INVALID_ARGUMENT
    # one head per grid row of the helper kernels: more than 65535 heads are refused here, before anything is launched
    assert L.ib200_attn_workspace_bytes(4096, 16, 16, 64, _capi.DTYPE_BF16, 1, ctypes.byref(out)) == _capi.ERR_UNSUPPORTED
    assert L.ib200_attn_workspace_bytes(4095, 16, 16, 64, _capi.DTYPE_BF16, 1, ctypes.byref(out)) == _capi.OK


def _fwd(L, ptrs, B=1, H=1, T=16, D=64, scale=0.125, causal=1, dtype=_capi.DTYPE_BF16, ws=0x1000, ws_bytes=1 << 20):
    q, k, v, o, lse = ptrs
    return L.ib200_attn_fwd(q, k, v, o, lse, B, H, T, D, scale, causal, dtype, 0, ws, ws_bytes, None)


def test_forward_argument_validation(built_lib):
    """Host-side rejection happens before any CUDA call; fake (never dereferenced) addresses suffice."""
    L = _capi.lib()
    good = (0x10000, 0x20000, 0x30000, 0x40000, 0x50000)
    assert _fwd(L, (None,) + good[1:]) == _capi.ERR_INVALID_ARGUMENT
    assert _fwd(L, good, T=0) == _capi.ERR_INVALID_ARGUMENT
    assert _fwd(L, good, causal=2) == _capi.ERR_INVALID_ARGUMENT
    assert _fwd(L, good, scale=0.0) == _capi.ERR_INVALID_ARGUMENT
    assert _fwd(L, good, scale=float("nan")) == _capi.ERR_INVALID_ARGUMENT
    assert _fwd(L, good, D=80) == _capi.ERR_UNSUPPORTED
    assert _fwd(L, (0x10004,) + good[1:]) == _capi.ERR_MISALIGNED
    assert _fwd(L, good, ws=None) == _capi.ERR_WORKSPACE
    assert _fwd(L, good, ws_bytes=16) == _capi.ERR_WORKSPACE
    # fp32 I/O has one arithmetic mode (split bf16); any other value is refused, not silently mapped onto it
    q, k, v, o, lse = good
    assert L.ib200_attn_fwd(q, k, v, o, lse, 1, 1, 16, 64, 0.125, 1, _capi.DTYPE_F32, 1, 0x1000, 1 << 20, None) == _capi.ERR_UNSUPPORTED


def test_selftest_and_static_check_argument_validation(built_lib):
    L = _capi.lib()
    assert L.ib200_selftest_wait_expiry(None, 256, 100, None) == _capi.ERR_WORKSPACE
    assert L.ib200_selftest_wait_expiry(0x1000, 64, 100, None) == _capi.ERR_WORKSPACE
    assert L.ib200_selftest_wait_expiry(0x1000, 256, 0, None) == _capi.ERR_INVALID_ARGUMENT
    assert L.ib200_selftest_wait_expiry(0x1000, 256, 10 ** 6, None) == _capi.ERR_INVALID_ARGUMENT
    assert L.ib200_attn_check(None, None, None) == _capi.ERR_INVALID_ARGUMENT
    import torch
    if not torch.cuda.is_available():
        assert L.ib200_attn_check_static(None, None) == _capi.ERR_NO_DEVICE
        assert L.ib200_selftest_wait_expiry(0x1000, 256, 100, None) == _capi.ERR_NO_DEVICE


def test_bounds_checked_build_has_the_same_abi(built_lib):
    """The range-checked build of the library exports exactly the same entry points."""
    from inferno_b200 import build
    lib = ctypes.CDLL(build.build(bounds=True))
    for name in declared_symbols():
        assert hasattr(lib, name)


def test_backward_argument_validation(built_lib):
    L = _capi.lib()
    p = [0x10000 * (i + 1) for i in range(9)]

    def bwd(ptrs, T=16, D=64, ws=0x1000, ws_bytes=1 << 20, dtype=_capi.DTYPE_BF16):
        return L.ib200_attn_bwd(*ptrs, 1, 1, T, D, 0.125, 1, dtype, 0, ws, ws_bytes, None)

    assert bwd([None] + p[1:]) == _capi.ERR_INVALID_ARGUMENT
    assert bwd(p[:8] + [None]) == _capi.ERR_INVALID_ARGUMENT
    assert bwd(p, D=32) == _capi.ERR_UNSUPPORTED
    assert bwd(p[:6] + [p[6] + 8] + p[7:]) == _capi.ERR_MISALIGNED
    assert bwd(p, ws_bytes=256) == _capi.ERR_WORKSPACE


def test_cast_argument_validation(built_lib):
    """fp32 <-> bf16 casts: host-side rejection before any CUDA call (fake addresses, never dereferenced)."""
    L = _capi.lib()
    assert L.ib200_cast_f32_to_bf16(None, 0x20000, 16, None) == _capi.ERR_INVALID_ARGUMENT
    assert L.ib200_cast_bf16_to_f32(0x10000, 0x20000, 0, None) == _capi.ERR_INVALID_ARGUMENT
    assert L.ib200_cast_f32_to_bf16(0x10000, 0x20000, 12, None) == _capi.ERR_UNSUPPORTED        # not a multiple of 8
    assert L.ib200_cast_bf16_to_f32(0x10004, 0x20000, 16, None) == _capi.ERR_MISALIGNED
    import torch
    if not torch.cuda.is_available():      # valid arguments: only ever issued where there is no GPU to run them on
        assert L.ib200_cast_f32_to_bf16(0x10000, 0x20000, 16, None) == _capi.ERR_NO_DEVICE


@pytest.mark.parametrize("case", [
    (0, 64, 16, 4096, 128, 148), (1, 64, 16, 4096, 128, 148), (1, 2, 16, 8192, 128, 148), (0, 16, 12, 1024, 64, 148),
    (1, 16, 16, 1024, 128, 148), (0, 1, 1, 1, 64, 148), (1, 3, 5, 777, 64, 132), (0, 37, 3, 300, 128, 7),
])
def test_item_order_of_persistent_kernels(built_lib, case):
    """The list the persistent kernels draw from: every (head, unit) exactly once; heads grouped into consecutive runs whose
    sizes differ by at most one; inside a group the heaviest unit of every head first; at least two rounds of items per group."""
    pass_, B, H, T, D, sms = case
    L = _capi.lib()
    per_head = (T + 255) // 256 if pass_ == 0 else (T + 127) // 128
    n = B * H * per_head
    heads, units, groups = (ctypes.c_int * n)(), (ctypes.c_int * n)(), ctypes.c_int(0)
    assert L.ib200_attn_item_order(pass_, B, H, T, D, sms, heads, units, n, ctypes.byref(groups)) == n
    items = list(zip(heads, units))
    assert sorted(items) == [(h, u) for h in range(B * H) for u in range(per_head)]
    g = groups.value
    assert 1 <= g <= B * H and (g == 1 or n // g >= 2 * sms)
    # walk the list group by group
    base, rem, pos, first_head = (B * H) // g, (B * H) % g, 0, 0
    for k in range(g):
        size = base + (1 if k < rem else 0)
        chunk = items[pos:pos + size * per_head]
        assert {h for h, _ in chunk} == set(range(first_head, first_head + size))
        work = [(u if pass_ == 0 else per_head - 1 - u) for _, u in chunk]          # longer walk = more work
        assert work == sorted(work, reverse=True)
        pos += size * per_head
        first_head += size
    assert pos == n
    assert L.ib200_attn_item_order(pass_, B, H, T, 96, sms, heads, units, n, None) == -_capi.ERR_UNSUPPORTED
    assert L.ib200_attn_item_order(7, B, H, T, D, sms, heads, units, n, None) == -_capi.ERR_INVALID_ARGUMENT


def test_no_device_fails_loudly(built_lib):
    """With well-formed arguments and no sm_100 device the call reports it; nothing else runs."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = _capi.lib()
    good = (0x10000, 0x20000, 0x30000, 0x40000, 0x50000)
    assert _fwd(L, good) == _capi.ERR_NO_DEVICE


def test_python_host_side_rejects_cpu_tensors(built_lib):
    import torch
    from inferno_b200 import attention as A
    q = torch.zeros(1, 1, 16, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        A.attention_forward(q, q, q)
    with pytest.raises(ValueError):
        A.attention_forward(q[0], q[0], q[0])
