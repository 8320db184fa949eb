"""TEST INFRASTRUCTURE ONLY -- CPU checkers for causal attention forward/backward.

Three independent evaluators, all taking dense row-major [B,H,T,D] numpy arrays:

* ``ref_attention``  -- the reference's own ops (its C++ sources compiled into
  ``oracle/_ref/ref_attention`` by ``oracle/Makefile``), composed exactly as
  ``InfernoApp/main.cpp:737-754`` with the two-stage backward described in
  ``oracle/ref_attention.cpp``.  Authoritative for "Inferno's own path".
* ``oracle_f32``     -- the plain-C restatement ``oracle/attn_oracle.c`` (fp32,
  same loop order); pinned bit-exact against ``ref_attention``.
* ``attn_fp64``      -- an independent float64 numpy evaluation, the only
  feasible checker at T >= 4096 (one head at a time).

Only tests, the smoke test and the CPU-baseline legs of the bench may import
this module.  The shipped library never does.
"""
from __future__ import annotations

import ctypes
import json
import os
import subprocess
import tempfile

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_BIN = os.path.join(_HERE, "_ref", "ref_attention")
ORACLE_SO = os.path.join(_HERE, "_build", "libattn_oracle.so")


def reference_root() -> str | None:
    """Where the reference's sources lie: the environment variable INFERNO_REF, else the Makefile's default REF."""
    root = os.environ.get("INFERNO_REF")
    if not root:
        with open(os.path.join(_HERE, "Makefile")) as f:
            for line in f:
                if line.startswith("REF") and "?=" in line:
                    root = line.split("?=", 1)[1].strip()
                    break
    return root if root and os.path.isdir(os.path.join(root, "src", "inferno")) else None


def build(ref: bool | None = None) -> None:
    """Compile the C restatement, and the reference harness when its sources are present."""
    subprocess.run(["make", "-s", "-C", _HERE, "oracle"], check=True)
    root = reference_root()
    if ref is None:
        ref = root is not None
    if ref:
        subprocess.run(["make", "-s", "-j8", "-C", _HERE, "ref", f"REF={root}"], check=True)


def have_ref() -> bool:
    return os.path.isfile(REF_BIN) and os.access(REF_BIN, os.X_OK)


def rel_err(x: np.ndarray, ref: np.ndarray) -> float:
    """Normwise relative error ||x - ref||_F / ||ref||_F in float64."""
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref.ravel())
    num = np.linalg.norm((x - ref).ravel())
    return float(num / den) if den > 0 else float(num)


def ref_attention(q, k, v, dO=None, device: str = "cpu", single_pass: bool = False, reps: int = 1):
    """Run the compiled reference.  Returns (o, dq, dk, dv, timings); grads are None if dO is None.

    ``single_pass`` runs the backward as one engine pass through the autograd additions of
    inferno_b200/inferno_shim/autograd_patches.h instead of the two-stage workaround.  ``reps`` > 1 repeats the
    whole pass in the one process and reports the timings of the last (warm) repetition."""
    if not have_ref():
        raise RuntimeError("oracle/_ref/ref_attention is not built (run `make -C oracle ref` where the reference is present)")
    B, H, T, D = q.shape
    with tempfile.TemporaryDirectory() as td:
        paths = {}
        for name, arr in (("q", q), ("k", k), ("v", v), ("do", dO)):
            paths[name] = os.path.join(td, name + ".bin")
            if arr is not None:
                np.ascontiguousarray(arr, dtype=np.float32).tofile(paths[name])
        prefix = os.path.join(td, "out")
        cmd = [REF_BIN, device, str(B), str(H), str(T), str(D), paths["q"], paths["k"], paths["v"], paths["do"], prefix,
               ("2" if single_pass else "0") if dO is not None else "1", str(int(reps))]
        res = subprocess.run(cmd, check=True, capture_output=True, text=True, cwd=td)
        timings = json.loads(res.stdout.strip().splitlines()[-1])
        rd = lambda s: np.fromfile(prefix + "." + s + ".bin", dtype=np.float32).reshape(B, H, T, D)
        o = rd("o")
        if dO is None:
            return o, None, None, None, timings
        return o, rd("dq"), rd("dk"), rd("dv"), timings


_lib = None


def _load():
    global _lib
    if _lib is None:
        if not os.path.isfile(ORACLE_SO):
            build(ref=False)
        lib = ctypes.CDLL(ORACLE_SO)
        fp = ctypes.POINTER(ctypes.c_float)
        lib.attn_oracle_f32.argtypes = [fp] * 8 + [ctypes.c_long] * 4 + [ctypes.c_float, ctypes.c_int, ctypes.c_int]
        lib.attn_oracle_f32.restype = ctypes.c_int
        lib.attn_oracle_max_threads.restype = ctypes.c_int
        _lib = lib
    return _lib


def max_threads() -> int:
    return int(_load().attn_oracle_max_threads())


def oracle_f32(q, k, v, dO=None, scale: float | None = None, threads: int = 0):
    """The C restatement.  Returns (o, dq, dk, dv); grads are None if dO is None."""
    lib = _load()
    B, H, T, D = q.shape
    if scale is None:
        scale = float(np.float32(1.0) / np.sqrt(np.float32(D)))
    q, k, v = (np.ascontiguousarray(a, dtype=np.float32) for a in (q, k, v))
    o = np.empty_like(q)
    fp = ctypes.POINTER(ctypes.c_float)
    ptr = lambda a: a.ctypes.data_as(fp)
    if dO is None:
        null = ctypes.cast(None, fp)
        rc = lib.attn_oracle_f32(ptr(q), ptr(k), ptr(v), null, ptr(o), null, null, null, B, H, T, D, scale, 0, threads)
        if rc != 0:
            raise MemoryError("attn_oracle_f32 failed")
        return o, None, None, None
    dO = np.ascontiguousarray(dO, dtype=np.float32)
    dq, dk, dv = np.empty_like(q), np.empty_like(q), np.empty_like(q)
    rc = lib.attn_oracle_f32(ptr(q), ptr(k), ptr(v), ptr(dO), ptr(o), ptr(dq), ptr(dk), ptr(dv), B, H, T, D, scale, 1, threads)
    if rc != 0:
        raise MemoryError("attn_oracle_f32 failed")
    return o, dq, dk, dv


def attn_fp64(q, k, v, dO=None, scale: float | None = None, want_lse: bool = False):
    """Independent float64 evaluation with -inf masking (result-equivalent to the -1e9 fill:
    both give exact zeros above the diagonal).  One head at a time, O(T^2) memory per head."""
    B, H, T, D = q.shape
    if scale is None:
        scale = 1.0 / np.sqrt(float(D))
    q64, k64, v64 = (np.asarray(a, dtype=np.float64).reshape(B * H, T, D) for a in (q, k, v))
    o = np.empty((B * H, T, D))
    lse = np.empty((B * H, T))
    grads = None
    if dO is not None:
        do64 = np.asarray(dO, dtype=np.float64).reshape(B * H, T, D)
        grads = [np.empty((B * H, T, D)) for _ in range(3)]
    upper = np.triu(np.ones((T, T), dtype=bool), 1)
    for i in range(B * H):
        s = (q64[i] @ k64[i].T) * scale
        s[upper] = -np.inf
        m = s.max(axis=1, keepdims=True)
        e = np.exp(s - m)
        z = e.sum(axis=1, keepdims=True)
        p = e / z
        lse[i] = (m + np.log(z))[:, 0]
        o[i] = p @ v64[i]
        if dO is not None:
            dp = do64[i] @ v64[i].T
            grads[2][i] = p.T @ do64[i]
            delta = (dp * p).sum(axis=1, keepdims=True)
            ds = p * (dp - delta) * scale
            grads[0][i] = ds @ k64[i]
            grads[1][i] = ds.T @ q64[i]
    shp = (B, H, T, D)
    out = [o.reshape(shp)] + ([g.reshape(shp) for g in grads] if grads else [None, None, None])
    if want_lse:
        out.append(lse.reshape(B, H, T))
    return tuple(out)
