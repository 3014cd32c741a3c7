"""Decode on several GPUs of one box: one process and one full model replica per GPU, mini-batches of
whole sentences dealt round-robin (src/translator/translator.h:154-167: ``graphs_[id % numDevices_]``).
Activation multipliers depend only on the mini-batch, so a mini-batch decodes to the same tokens on
any rank.  The only exchange is the gather of the outputs (the reference's OutputCollector orders them
by line number on the host, src/translator/output_collector.h:47-60).

A single affine can also be split by rows of the activation.  Its multiplier 127 / max|A| is a property of
the WHOLE tensor (src/tensors/cpu/integer_common.h:169-173), so the ranks exchange one float - the maximum
of their local maxima - between the abs-max and the quantisation; everything else is local, and the rows
a rank computes are bit-identical to the same rows of the unsharded affine."""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_batches(batches, rank: int, world: int, snake: bool = False):
    """Mini-batch i goes to rank i % world (the reference's rule).  With snake=True every second group of
    `world` mini-batches is dealt in reverse: for a length-sorted list (the maxi-batch order) the ranks then
    receive equally long work instead of rank 0 always getting the longest batch of each group."""
    if not snake:
        return [b for i, b in enumerate(batches) if i % world == rank]
    out = []
    for i, b in enumerate(batches):
        group, pos = divmod(i, world)
        if (pos if group % 2 == 0 else world - 1 - pos) == rank:
            out.append(b)
    return out


def shared_counter(key: str = "mi8_next_mini_batch"):
    """A counter shared by all ranks: the returned callable hands out 0, 1, 2, ... with every value going to exactly one
    rank (an atomic add on the process group's key-value store; a local counter without a process group).  It is how the
    reference's translator deals mini-batches - its thread pool gives the next one to whichever device is free
    (src/translator/translator.h:154-167) - when the ranks are processes instead of threads."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size() == 1:
        state = [0]

        def take_local() -> int:
            state[0] += 1
            return state[0] - 1
        return take_local
    store = dist.distributed_c10d._get_default_store()

    def take() -> int:
        return int(store.add(key, 1)) - 1
    return take


def pack_outputs(local: dict, rows: int, max_len: int):
    """{sentence id: tokens} as one int32 matrix [max(rows, 1), 2 + max_len] of (id, length, tokens), unused cells -1.
    A hypothesis longer than max_len is an error, never cut: outputs must not depend on the number of ranks."""
    import numpy as np
    mat = np.full((max(rows, 1), 2 + max_len), -1, dtype=np.int32)     # built and decoded with NumPy: no per-element tensor access
    for r, (sid, toks) in enumerate(sorted(local.items())):
        if len(toks) > max_len:
            raise ValueError(f"sentence {sid} has {len(toks)} tokens but the gather matrix holds {max_len}: "
                             "size max_len from the search's length limit (max_length_factor x the widest source)")
        mat[r, 0], mat[r, 1] = sid, len(toks)
        if toks:
            mat[r, 2:2 + len(toks)] = toks
    return mat


def gather_output_matrices(local: dict, max_len: int, device=None):
    """The exchange itself: every rank contributes {sentence id: tokens} as one int32 matrix [sentences, 2 + max_len]
    (id, length, tokens), padded to the largest count, and receives every rank's matrix as NumPy arrays (host memory).
    Without a process group: this rank's matrix alone."""
    import numpy as np
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size() == 1:
        return [pack_outputs(local, len(local), max_len)]
    world = dist.get_world_size()
    dev = device if device is not None else torch.device("cpu")
    n = torch.tensor([len(local)], dtype=torch.int64, device=dev)
    counts = [torch.zeros_like(n) for _ in range(world)]
    dist.all_gather(counts, n)
    rows = int(max(int(c.item()) for c in counts))
    mat_t = torch.from_numpy(pack_outputs(local, rows, max_len)).to(dev)
    out = [torch.empty_like(mat_t) for _ in range(world)]
    dist.all_gather(out, mat_t)
    return [m.cpu().numpy() for m in out]


def merge_output_matrices(mats) -> dict:
    """{sentence id: tokens} from the matrices gather_output_matrices returned."""
    merged = {}
    for m in mats:
        keep = m[m[:, 0] >= 0]
        for row, n in zip(keep.tolist(), keep[:, 1].tolist()):
            merged[row[0]] = row[2:2 + n]
    return merged


def gather_outputs(local: dict, max_len: int, device=None) -> dict:
    """All ranks contribute {sentence id: tokens}; every rank receives the union."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size() == 1:
        return dict(local)
    return merge_output_matrices(gather_output_matrices(local, max_len, device))


def shard_rows(m: int, rank: int, world: int):
    """Contiguous, near-even split of m rows: rank r owns [begin, end)."""
    per, extra = divmod(m, world)
    begin = rank * per + min(rank, extra)
    return begin, begin + per + (1 if rank < extra else 0)


def global_abs_max(local_max: torch.Tensor, group=None) -> torch.Tensor:
    """In-place MAX all-reduce of a one-element float32 tensor (4 bytes on the wire); a no-op without a
    process group.  Works on CPU tensors (gloo) and CUDA tensors (NCCL)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(local_max, op=dist.ReduceOp.MAX, group=group)
    return local_max


def sharded_affine(a_local: torch.Tensor, b, bias=None, scale: float = 1.0, relu: bool = False, out_dtype=torch.float32,
                   group=None, exchange: bool = True) -> torch.Tensor:
    """The int8 affine on this rank's rows of A: local abs-max, one MAX all-reduce of a float, quantisation
    with the agreed multiplier, GEMM with the fused write-back.  Returns this rank's rows of C.
    `exchange=False` leaves the all-reduce out (every rank then quantises with its own shard's multiplier, a
    different result): a timing aid that shows what the exchange costs, not a mode of the product."""
    from . import ops
    amax = ops.max_absolute(a_local)
    if exchange:
        global_abs_max(amax, group)
    aq = ops.quantize_with_absmax(a_local, amax)
    return ops.multiply(aq, b, bias, scale, relu, out_dtype=out_dtype)


def sharded_packed8_affine(a_local: torch.Tensor, w, bias=None) -> torch.Tensor:
    """The packed8avx512 affine on this rank's rows of A.  That scheme quantises every ROW of A with its own scale
    and zero point (src/tensors/cpu/mjdgemm/mjdgemm_avx512.cpp:195-228), so rows shard with no exchange at all:
    this rank's rows of C equal the same rows of the unsharded product bit for bit.  `w` is a packed8.Packed8Weight
    replicated on every rank."""
    from . import packed8
    return packed8.gemmInt8Packed(a_local, w, bias)
