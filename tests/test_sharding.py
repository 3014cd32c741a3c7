"""Multi-GPU logic on CPU: mini-batches are dealt round-robin to one replica per rank
(src/translator/translator.h:154-167, graphs_[id % numDevices_]) and the outputs are gathered by
sentence id.  Two gloo ranks stand in for two GPUs; the decode itself is replaced by a deterministic
function of the mini-batch, so only the sharding / gathering code is under test."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from marian_dev_b200 import model, parallel
    corpus = model.synthetic_corpus(50, 100, seed=1, length_dist="uniform", lo=3, hi=9)
    batches = model.make_batches(corpus, 8)
    mine = parallel.shard_batches(batches, rank, world)

    def fake_decode(batch):                      # one "translation" per sentence: its reversed ids
        sent_ids, ids, mask = batch
        return {int(s): [int(t) for t, m in zip(ids[r][::-1], mask[r][::-1]) if m > 0] for r, s in enumerate(sent_ids)}

    local = {}
    for b in mine:
        local.update(fake_decode(b))
    merged = parallel.gather_outputs(local, max_len=16)
    if rank == 0:
        out.put(merged)
    dist.destroy_process_group()


def test_round_robin_sharding_and_gather_with_two_gloo_ranks():
    sys.path.insert(0, ROOT)
    from marian_dev_b200 import model
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29731, q)) for r in range(2)]
    for p in procs:
        p.start()
    merged = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    corpus = model.synthetic_corpus(50, 100, seed=1, length_dist="uniform", lo=3, hi=9)
    assert sorted(merged) == list(range(50))                      # every sentence exactly once
    for sid, toks in merged.items():
        assert toks == [int(t) for t in corpus[sid][::-1]]


def test_shard_batches_is_round_robin():
    sys.path.insert(0, ROOT)
    from marian_dev_b200 import parallel
    batches = list(range(10))
    assert parallel.shard_batches(batches, 0, 4) == [0, 4, 8]
    assert parallel.shard_batches(batches, 0, 4, snake=True) == [0, 7, 8]
    assert parallel.shard_batches(batches, 3, 4, snake=True) == [3, 4]
    assert sorted(sum((parallel.shard_batches(batches, r, 4, snake=True) for r in range(4)), [])) == batches
    assert parallel.shard_batches(batches, 3, 4) == [3, 7]
    assert sum((parallel.shard_batches(batches, r, 3) for r in range(3)), []).__len__() == 10


def _affine_worker(rank, world, port, out):
    """One rank of the row-sharded affine, with the CPU checker standing in for the device kernels: local
    abs-max, the MAX all-reduce of one float (the code under test), quantisation with the agreed multiplier."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from marian_dev_b200 import parallel
    from oracle.oracle import COracle
    o = COracle()
    rng = np.random.default_rng(5)
    m, k, n = 37, 64, 24
    a = rng.standard_normal((m, k)).astype(np.float32)
    a[30, 3] = 9.5                                   # the global maximum lives on the last rank only
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(n) * 0.01).astype(np.float32)
    bt, qb = o.prepare_b(w)
    b, e = parallel.shard_rows(m, rank, world)
    local_max = torch.tensor([np.abs(a[b:e]).max()], dtype=torch.float32)
    parallel.global_abs_max(local_max)
    qa = np.float32(127.0) / np.float32(local_max.item())
    aq = o.quantize(a[b:e], qa)
    acc = o.multiply_i32(aq, bt)
    unquant = np.float32(np.float32(1.0) / np.float32(np.float32(qa) * np.float32(qb))) * np.float32(1.0)
    c = o.unquantize(acc, unquant, bias, False)
    out.put((rank, b, e, c))
    dist.barrier()
    dist.destroy_process_group()


def test_row_sharded_affine_matches_unsharded_with_two_gloo_ranks():
    sys.path.insert(0, ROOT)
    from oracle.oracle import COracle
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_affine_worker, args=(r, 2, 29733, q)) for r in range(2)]
    for p in procs:
        p.start()
    parts = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    o = COracle()
    rng = np.random.default_rng(5)
    m, k, n = 37, 64, 24
    a = rng.standard_normal((m, k)).astype(np.float32)
    a[30, 3] = 9.5
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(n) * 0.01).astype(np.float32)
    bt, qb = o.prepare_b(w)
    want = o.affine(a, bt, qb, bias, 1.0, False)
    want = want[0] if isinstance(want, tuple) else want
    covered = np.zeros(m, dtype=bool)
    for _rank, b, e, c in parts:
        assert np.array_equal(c, want[b:e])           # bit-identical to the same rows of the unsharded affine
        covered[b:e] = True
    assert covered.all()


def test_shard_rows_covers_all_rows_once():
    sys.path.insert(0, ROOT)
    from marian_dev_b200 import parallel
    for m in (1, 7, 8, 37, 4096):
        for world in (1, 2, 3, 8):
            spans = [parallel.shard_rows(m, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == m
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert max(e - b for b, e in spans) - min(e - b for b, e in spans) <= 1


def _counter_worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from marian_dev_b200 import parallel
    take = parallel.shared_counter("test_counter")
    dist.barrier()
    mine = []
    while True:
        i = take()
        if i >= 23:
            break
        mine.append(i)
        if rank == 0:                            # a slow rank simply takes fewer
            import time
            time.sleep(0.01)
    merged = parallel.gather_outputs({i: [i, rank] for i in mine}, max_len=4)
    if rank == 0:
        out.put((mine, merged))
    dist.destroy_process_group()


def test_shared_counter_deals_every_mini_batch_to_exactly_one_rank():
    """Strong scaling deals from one counter: two gloo ranks draw until it runs out; together they hold every value once."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_counter_worker, args=(r, 2, 29741, q)) for r in range(2)]
    for p in procs:
        p.start()
    mine0, merged = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(merged) == list(range(23))
    owners = {i: v[1] for i, v in merged.items()}
    assert sorted(i for i, r in owners.items() if r == 0) == sorted(mine0)
    assert 0 < len(mine0) < 23                                   # both ranks took part


def test_shared_counter_without_a_process_group():
    from marian_dev_b200 import parallel
    take = parallel.shared_counter()
    assert [take() for _ in range(4)] == [0, 1, 2, 3]


def test_gather_refuses_to_truncate():
    import pytest
    from marian_dev_b200 import parallel
    assert parallel.gather_outputs({1: [1, 2, 3]}, max_len=2) == {1: [1, 2, 3]}      # single process: nothing to pack
    m = parallel.pack_outputs({4: [9, 8], 2: []}, rows=3, max_len=2)
    assert m.tolist() == [[2, 0, -1, -1], [4, 2, 9, 8], [-1, -1, -1, -1]]
    with pytest.raises(ValueError, match="3 tokens"):
        parallel.pack_outputs({1: [1, 2, 3]}, rows=1, max_len=2)


def test_output_matrices_round_trip_without_a_process_group():
    """gather_output_matrices (the exchange, what the benchmark times) and merge_output_matrices (the conversion to Python
    lists, done afterwards) together equal gather_outputs; empty hypotheses and empty ranks survive."""
    from marian_dev_b200 import parallel
    local = {7: [5, 6, 0], 2: [], 11: [9] * 6}
    mats = parallel.gather_output_matrices(local, max_len=6)
    assert len(mats) == 1 and mats[0].shape == (3, 8) and mats[0].dtype.name == "int32"
    assert parallel.merge_output_matrices(mats) == local
    assert parallel.merge_output_matrices(parallel.gather_output_matrices({}, max_len=4)) == {}
