"""Decode on several GPUs of one box: one process and one full model replica per GPU, mini-batches of
whole sentences dealt round-robin (src/translator/translator.h:154-167: ``graphs_[id % numDevices_]``).
Activation multipliers depend only on the mini-batch, so a mini-batch decodes to the same tokens on
any rank.  The only exchange is the gather of the outputs (the reference's OutputCollector orders them
by line number on the host, src/translator/output_collector.h:47-60)."""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_batches(batches, rank: int, world: int):
    """Mini-batch i goes to rank i % world."""
    return [b for i, b in enumerate(batches) if i % world == rank]


def gather_outputs(local: dict, max_len: int, device=None) -> dict:
    """All ranks contribute {sentence id: tokens}; every rank receives the union.  The payload is one
    int32 matrix [sentences, 2 + max_len] per rank (id, length, tokens), padded to the largest count."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size() == 1:
        return dict(local)
    world = dist.get_world_size()
    dev = device if device is not None else torch.device("cpu")
    n = torch.tensor([len(local)], dtype=torch.int64, device=dev)
    counts = [torch.zeros_like(n) for _ in range(world)]
    dist.all_gather(counts, n)
    rows = int(max(int(c.item()) for c in counts))
    mat = torch.full((max(rows, 1), 2 + max_len), -1, dtype=torch.int32)
    for r, (sid, toks) in enumerate(sorted(local.items())):
        toks = toks[:max_len]
        mat[r, 0], mat[r, 1] = sid, len(toks)
        if toks:
            mat[r, 2:2 + len(toks)] = torch.tensor(toks, dtype=torch.int32)
    mat = mat.to(dev)
    out = [torch.empty_like(mat) for _ in range(world)]
    dist.all_gather(out, mat)
    merged = {}
    for m in out:
        m = m.cpu()
        for row in m:
            sid = int(row[0])
            if sid >= 0:
                merged[sid] = [int(t) for t in row[2:2 + int(row[1])]]
    return merged
