"""Host-side logic of bench.py that needs no GPU: the fixed corpus and its mini-batches, the fixed shuffled order the
timed set is a prefix of, the dealing of mini-batches to ranks, the output digest."""
import numpy as np


def test_corpus_is_fixed_and_covers_the_named_workloads():
    import bench
    from marian_dev_b200 import model
    for name, n_batches in (("big", 64), ("base", 32)):
        wl = bench.WORKLOADS[name]
        batches = bench.corpus_batches(model, model.CONFIGS[name], wl)
        assert len(batches) == n_batches and all(b[1].shape[0] == wl["mini_batch"] for b in batches)
        widths = [b[1].shape[1] for b in batches]
        assert widths == sorted(widths, reverse=True)                       # maxi-batch order: longest first
        again = bench.corpus_batches(model, model.CONFIGS[name], wl)
        assert all(np.array_equal(a[1], b[1]) for a, b in zip(batches, again))
    big = bench.corpus_batches(model, model.CONFIGS["big"], bench.WORKLOADS["big"])
    lens = np.concatenate([b[2].sum(axis=1) for b in big]) - 1              # EOS excluded
    assert lens.min() >= 4 and lens.max() <= 128 and 28 < lens.mean() < 32  # clip(N(30,12),4,128)


def test_timed_set_is_a_prefix_of_one_fixed_order():
    import bench
    order = bench.batch_order(64)
    assert sorted(order) == list(range(64)) and order == bench.batch_order(64)
    widths = list(range(100, 36, -1))
    for world in (1, 2, 4, 8):
        steps = 5
        picked = [order[i % 64] for i in range(world * steps)]
        dealt = [bench.deal_batches(picked, widths, r, world) for r in range(world)]
        assert sorted(sum(dealt, [])) == sorted(picked) and all(len(d) == steps for d in dealt)
        cost = [sum(widths[b] for b in d) for d in dealt]
        assert max(cost) - min(cost) <= max(widths) - min(widths)           # equally long work per rank


def test_digest_depends_on_ids_lengths_and_tokens():
    import bench
    a = bench.tokens_digest([3, 1], [[5, 6, 0], [7, 0]])
    assert a == bench.tokens_digest([1, 3], [[7, 0], [5, 6, 0]])            # order of arrival does not matter
    assert a != bench.tokens_digest([3, 1], [[5, 6, 0], [7, 1]])
    assert a != bench.tokens_digest([3, 2], [[5, 6, 0], [7, 0]])
    assert a != bench.tokens_digest([3, 1], [[5, 6], [0, 7, 0]])


def test_worker_count_follows_the_number_of_timed_mini_batches():
    """bench.py runs several searches per GPU; the count is the caller's, or chosen so that few timed mini-batches are shared
    out evenly (never more searches than mini-batches), and four once there are enough to keep four busy."""
    import bench
    assert bench.pick_workers(3, 100) == 3 and bench.pick_workers(1, 2) == 1          # an explicit request stands
    assert [bench.pick_workers(0, k) for k in (1, 2, 3, 4)] == [1, 2, 3, 4]
    assert all(bench.pick_workers(0, k) == 4 for k in (8, 12, 16, 32, 64))
    assert all(1 <= bench.pick_workers(0, k) <= min(k, 6) for k in range(1, 40))
