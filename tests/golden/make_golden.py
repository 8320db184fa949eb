"""Generate the golden vectors under tests/golden/ by running the reference's own code.

Run where the reference sources are present (after ``make -C oracle ref``):
    python tests/golden/make_golden.py
Each ``<case>.npz`` holds the OUTPUTS (o, dq, dk, dv, float32) of
``oracle/_ref/ref_attention`` -- the reference's ops composed as in
InfernoApp/main.cpp:737-754 with the two-stage backward -- on inputs that
``inferno_b200.synth.make_inputs`` regenerates from the recorded seed, so only the
outputs are stored.  A case with a ``heads`` entry in the manifest ran the whole configuration through
the reference and stores those heads of the flattened batch*head axis, shaped [len(heads), 1, T, D].
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from inferno_b200.synth import CONFIGS, make_inputs  # noqa: E402
from oracle import oracle as orc  # noqa: E402

# name: (B, H, T, D, seed, qkv_std, do_std, dtype)
CASES = {
    "tiny_t32_d16": (1, 2, 32, 16, 0, 1.0, 1.0, "f32"),
    "tile_t128_d64": (1, 2, 128, 64, 10, 1.0, 1.0, "f32"),
    "ragged_t200_d64": (1, 1, 200, 64, 11, 1.0, 0.1, "f32"),
    "ragged_t160_d128_bf16": (1, 1, 160, 128, 12, 0.5, 0.1, "bf16"),
    "single_t1_d64": (2, 1, 1, 64, 13, 1.0, 1.0, "f32"),
}


# name: (configuration of inferno_b200.synth.CONFIGS, heads of its flattened batch*head axis that are stored)
CONFIG_CASES = {
    "c1_heads_0_15": ("c1", [0, 15]),       # configuration 1 (B4 H4 T128 D64 fp32, seed 0), first and last head
}


def main() -> None:
    here = os.path.dirname(os.path.abspath(__file__))
    manifest = {}
    for name, (B, H, T, D, seed, qs, ds, dt) in CASES.items():
        q, k, v, do = make_inputs(B, H, T, D, seed, qs, ds, dt)
        o, dq, dk, dv, _ = orc.ref_attention(q, k, v, do, device="cpu")
        np.savez_compressed(os.path.join(here, name + ".npz"), o=o, dq=dq, dk=dk, dv=dv)
        manifest[name] = dict(B=B, H=H, T=T, D=D, seed=seed, qkv_std=qs, do_std=ds, dtype=dt)
        print(name, "written")
    for name, (cfg_name, heads) in CONFIG_CASES.items():
        c = CONFIGS[cfg_name]
        # the whole configuration goes through the reference; the listed heads of its outputs are stored
        q, k, v, do = make_inputs(c.B, c.H, c.T, c.D, c.seed, c.qkv_std, c.do_std, c.dtype)
        outs = orc.ref_attention(q, k, v, do, device="cpu")[:4]
        sel = {key: a.reshape(c.B * c.H, 1, c.T, c.D)[heads] for key, a in zip(("o", "dq", "dk", "dv"), outs)}
        np.savez_compressed(os.path.join(here, name + ".npz"), **sel)
        manifest[name] = dict(B=c.B, H=c.H, T=c.T, D=c.D, seed=c.seed, qkv_std=c.qkv_std, do_std=c.do_std, dtype=c.dtype, heads=heads)
        print(name, "written")
    with open(os.path.join(here, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
