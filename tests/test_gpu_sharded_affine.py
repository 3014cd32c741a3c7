"""Row-sharded affine on the GPU: the rows of A are split in two, each half is pushed through
parallel.sharded_affine with the exchanged maximum, and the halves equal the rows of the unsharded affine
bit for bit.  One process and one GPU: the two "ranks" run one after the other and the MAX all-reduce is
replaced by taking the maximum of their two abs-max tensors, which is what the collective computes."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_row_shards_equal_the_unsharded_affine(cuda_device):
    from marian_dev_b200 import ops, parallel
    rng = np.random.default_rng(11)
    m, k, n = 300, 256, 384
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(cuda_device)
    a[277, 5] = 7.25                                    # the global maximum sits in the second shard
    w = torch.from_numpy((rng.standard_normal((k, n)) * 0.02).astype(np.float32)).to(cuda_device)
    bias = torch.from_numpy((rng.standard_normal(n) * 0.01).astype(np.float32)).to(cuda_device)
    b = ops.prepareB(w)
    whole = ops.affine(a, b, bias)
    spans = [parallel.shard_rows(m, r, 2) for r in range(2)]
    maxima = [ops.max_absolute(a[s:e]) for s, e in spans]
    agreed = torch.maximum(maxima[0], maxima[1])
    assert float(agreed) == float(a.abs().max())
    for s, e in spans:
        aq = ops.quantize_with_absmax(a[s:e], agreed.clone())
        part = ops.multiply(aq, b, bias)
        assert torch.equal(part, whole[s:e])
    assert ops.poll_status() == 0


def test_sharded_affine_without_a_process_group_is_the_plain_affine(cuda_device):
    from marian_dev_b200 import ops, parallel
    a = torch.randn(64, 128, device=cuda_device)
    b = ops.prepareB(torch.randn(128, 256, device=cuda_device) * 0.02)
    assert torch.equal(parallel.sharded_affine(a, b, None, 1.0, True), ops.affineWithReluDropout(a, b, None))
