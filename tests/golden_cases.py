"""Loader of the golden cases under tests/golden/ (outputs of the compiled reference; see make_golden.py)."""
import json
import os

import numpy as np

from inferno_b200.synth import make_inputs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
with open(os.path.join(GOLDEN, "manifest.json")) as f:
    MANIFEST = json.load(f)


def load_case(name):
    """(manifest entry, (q, k, v, dO), golden outputs).  For a case that stores a subsample of a configuration's heads the
    inputs are the same heads, shaped [len(heads), 1, T, D] like the stored outputs."""
    c = MANIFEST[name]
    inputs = make_inputs(c["B"], c["H"], c["T"], c["D"], c["seed"], c["qkv_std"], c["do_std"], c["dtype"])
    if "heads" in c:
        inputs = tuple(a.reshape(c["B"] * c["H"], 1, c["T"], c["D"])[c["heads"]] for a in inputs)
    gold = np.load(os.path.join(GOLDEN, name + ".npz"))
    return c, inputs, gold
