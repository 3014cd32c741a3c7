"""Writes tests/golden/packed8_golden.npz from the REFERENCE's own packed-int8 GEMM.

Needs oracle/_ref/libref_mjdgemm.so (`make -C oracle ref`, which compiles src/tensors/cpu/mjdgemm of the reference
tree where it lies) on a host whose CPU takes the reference's AVX-512 route.  Run from the repository root:

    python tests/golden/make_packed8_golden.py

Contents: one case stored in full (the smallest weight shape the reference instantiates, N = K = 512: the
packed item, activations with ordinary, tiny-range, one-sided and large rows, the bias, the reference's outputs
with and without bias) and, for larger shapes, the SHA-256 of seeded inputs and of the reference's output.
The weights are packed by the checker's restatement of fbgemmPacked8Pack; the reference's own packB confirms the
block order before anything is written.
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.oracle import Packed8Oracle, RefMjdgemm  # noqa: E402


def inputs(seed: int, M: int, K: int, N: int):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    a = rng.standard_normal((M, K)).astype(np.float32)
    a *= np.exp(rng.uniform(-3, 3, size=(M, 1))).astype(np.float32)      # row ranges differ by orders of magnitude
    if M >= 4:
        a[1] = np.abs(a[1])                                              # one-sided row
        a[2] = 1.0 + a[2] * 1e-4                                         # tiny range away from zero
        a[3] *= 1000.0
    bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
    return w, a, bias


def sha(*arrays) -> str:
    h = hashlib.sha256()
    for x in arrays:
        h.update(np.ascontiguousarray(x).tobytes())
    return h.hexdigest()


def main():
    ref, chk = RefMjdgemm(), Packed8Oracle()
    assert ref.isa() in (5, 6), "the fixtures pin the AVX-512 route"
    out = {}
    w, a, bias = inputs(20, 6, 512, 512)
    item = chk.prepare_b(w)
    assert np.array_equal(ref.pack_b(np.ascontiguousarray(chk.unpack_bt(item).T)), item.packed[:512 * 512])
    out["full_packed"] = np.array(item.packed)
    out["full_a"] = a
    out["full_bias"] = bias
    out["full_c_bias"] = ref.gemm(a, item, bias)
    out["full_c_nobias"] = ref.gemm(a, item, None)
    cases = []
    for seed, (M, N, K) in enumerate([(3, 1024, 1024), (57, 4096, 1024), (9, 1024, 4096), (5, 32000, 512), (64, 512, 8192)], start=30):
        w, a, bias = inputs(seed, M, K, N)
        item = chk.prepare_b(w)
        c = ref.gemm(a, item, bias)
        cases.append((seed, M, N, K, sha(w, a, bias), sha(item.packed), sha(c)))
    out["hashed_cases"] = np.array([f"{s} {M} {N} {K} {hi} {hp} {hc}" for s, M, N, K, hi, hp, hc in cases])
    path = os.path.join(ROOT, "tests", "golden", "packed8_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
