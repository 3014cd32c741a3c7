"""Generates tests/golden/affine_golden.json: SHA-256 digests (plus a few leading values) of the CPU
checker's outputs on seeded inputs.  Inputs are never stored: tests regenerate them from the seed.

    python -m tests.golden.make_golden        (from the repository root)

The reference holds no fixture for its intgemm8 path and cannot be built here, so these vectors pin
the restatement against itself across machines and compilers, and give the GPU tests a committed
target that does not depend on the checker being rebuilt on the GPU box.
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def cases():
    """name -> (M, K, N, relu, bias, scale, seed).  The first is the single-affine benchmark configuration
    (X ~ N(0,1), W ~ N(0,0.02), bias ~ N(0,0.01), ReLU, seed 0); the others are points of the shape sweep."""
    return {
        "config1_256x512x2048_relu": dict(m=256, k=512, n=2048, relu=True, bias=True, scale=1.0, seed=0),
        "sweep_1x512x512": dict(m=1, k=512, n=512, relu=False, bias=True, scale=1.0, seed=11),
        "sweep_8x1024x2048_relu": dict(m=8, k=1024, n=2048, relu=True, bias=True, scale=1.0, seed=12),
        "sweep_64x4096x512_dot": dict(m=64, k=4096, n=512, relu=False, bias=False, scale=0.5, seed=13),
        "sweep_256x1024x4096": dict(m=256, k=1024, n=4096, relu=False, bias=True, scale=1.0, seed=14),
        "sweep_1024x512x2048_relu": dict(m=1024, k=512, n=2048, relu=True, bias=True, scale=1.0, seed=15),
        "ragged_33x1040x136": dict(m=33, k=1040, n=136, relu=True, bias=True, scale=1.0, seed=16),
        "vocab_16x1024x32000": dict(m=16, k=1024, n=32000, relu=False, bias=True, scale=1.0, seed=17),
    }


def inputs(spec):
    rng = np.random.default_rng(spec["seed"])
    a = rng.standard_normal((spec["m"], spec["k"])).astype(np.float32)
    w = (rng.standard_normal((spec["k"], spec["n"])) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(spec["n"]) * 0.01).astype(np.float32) if spec["bias"] else None
    return a, w, bias


def run_case(oracle, spec):
    a, w, bias = inputs(spec)
    bt, qb = oracle.prepare_b(w)
    out, acc, aq, qa = oracle.affine(a, bt, qb, bias, spec["scale"], spec["relu"], want_acc=True)
    return {"bt": bt, "qb": np.array([qb], np.float32), "aq": aq, "qa": np.array([qa], np.float32), "acc": acc, "out": out}


def digest(arr):
    return hashlib.sha256(np.ascontiguousarray(arr).tobytes()).hexdigest()


def main():
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle.oracle import COracle
    o = COracle()
    o.set_threads(o.max_threads())
    doc = {}
    for name, spec in cases().items():
        got = run_case(o, spec)
        doc[name] = {"spec": spec, "sha256": {k: digest(v) for k, v in got.items()},
                     "head": {"qa": float(got["qa"][0]), "qb": float(got["qb"][0]),
                              "acc": got["acc"].reshape(-1)[:6].tolist(), "out": [float(x) for x in got["out"].reshape(-1)[:6]]}}
    with open(os.path.join(HERE, "affine_golden.json"), "w") as f:
        json.dump(doc, f, indent=1)
    print("wrote", len(doc), "cases")


if __name__ == "__main__":
    main()
