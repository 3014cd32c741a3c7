#!/usr/bin/env python
"""Benchmark of the int8 decode path: transformer-big, beam 4, mini-batch 128, synthetic sentences.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is the decode of one mini-batch (128 synthetic sentences, beam 4) on one GPU: encoder,
then decoder steps until every hypothesis ended or 1.5 x the source width is reached, with every
weight multiplication on the int8 engine.  The workload's corpus is fixed (8192 sentences = 64
length-sorted mini-batches, whatever N is); the timed mini-batches are the first N x K of one fixed
shuffled order of them, so a run times a length-representative sample and `--steps 64` at N = 1 times
the whole corpus.  With N GPUs every rank holds a full model replica and decodes K of those
mini-batches (dealt so that the ranks get equally long work; the reference's translator hands the
next mini-batch to the next free device); the only collective is the gather of the output token
matrix.  Every decoded mini-batch is hashed and compared with the digest committed under
tests/golden/ (which the GPU tests tie to the CPU checker): a run whose output differs prints no
number.  Rank 0 prints one JSON line.

`value` is measured with the mini-batch's token ids and mask already resident in HBM; `e2e` is the
same decode called with host buffers (pinned host -> device copy of ids/mask inside the timed
region, device -> host reads of the n-best lists every step and of nothing else).
`--impl reference` times the CPU restatement of the reference's intgemm8 path (the reference itself
cannot be built: its int8 arithmetic lives in the un-vendored intgemm submodule).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

KERNEL_NAMES = ["mi8_gemm_pair_kernel", "mi8_gemm_kernel", "quantize_slot_kernel", "attention1_kernel", "attention_enc_kernel",
                "add_layernorm_kernel", "quantize_dual_kernel", "history_commit_kernel", "lse_topk_kernel",
                "lse_merge_kernel", "nbest_merge_kernel", "embed_kernel", "ancestors_update_kernel", "gather_rows_kernel",
                "ssru_cell_kernel", "mi8_absmax_kernel", "mi8_quantize_kernel", "mi8_transpose_quantize_kernel"]
METRIC = "int8_decode_tgt_tokens_per_sec"
UNIT = "tokens/s"
WORKLOAD = "transformer-big decode (6+6 layers, d=1024, ffn=4096, 16 heads, tied 32000 vocab, all affines int8), beam 4, mini-batch 128, lengths clip(N(30,12),4,128), max length 1.5x source"
MINI_BATCH = 128
BEAM = 4
# The benchmark line is the "big" workload; the others are the remaining named decode configurations,
# runnable with --model for parity-sized measurements (their lines carry their own workload string).
WORKLOADS = {
    "big": dict(desc=WORKLOAD, mini_batch=128, beam=4, sentences=8192, lengths=dict(length_dist="normal", lo=4, hi=128, mean=30.0, std=12.0)),
    "base": dict(desc="transformer-base decode (6+6 layers, d=512, ffn=2048, 8 heads, tied 32000 vocab, all affines int8), beam 4, "
                      "mini-batch 64, lengths U[8,64], max length 1.5x source",
                 mini_batch=64, beam=4, sentences=2048, lengths=dict(length_dist="uniform", lo=8, hi=64)),
    "student": dict(desc="student decode (12 encoder layers d=256 ffn=1536 8 heads, 2-layer SSRU decoder, 32000 vocab, all affines int8), "
                         "greedy, lengths U[5,40], max length 1.5x source",
                    mini_batch=16, beam=1, sentences=1024, lengths=dict(length_dist="uniform", lo=5, hi=40)),
}


def workload(args):
    w = dict(WORKLOADS.get(args.model, WORKLOADS["big"]))
    if args.model not in WORKLOADS:
        w["desc"] = f"{args.model} (debug workload)"
        w["sentences"] = 8 * w["mini_batch"]
    if args.mini_batch:
        w["mini_batch"] = args.mini_batch
    if args.beam:
        w["beam"] = args.beam
    if args.model != "big" or args.mini_batch or args.beam:
        w["desc"] += f" [mini-batch {w['mini_batch']}, beam {w['beam']}]"
    return w


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="big", help="big (the benchmark), base, student, tiny (debugging)")
    ap.add_argument("--mini-batch", type=int, default=0, help="override the workload's mini-batch (sentences)")
    ap.add_argument("--beam", type=int, default=0, help="override the workload's beam size")
    ap.add_argument("--cpu-sentences", type=int, default=16, help="sentences in the CPU-baseline sample")
    ap.add_argument("--affine", default=None, help="M,K,N: time one int8 affine (abs-max + quantise + GEMM with bias and ReLU) instead of the decode")
    ap.add_argument("--workers", type=int, default=0,
                    help="beam searches side by side on each GPU, each with its own step driver and stream (decoder.SearchPool); "
                         "0 = chosen from --steps (4 unless so few mini-batches are timed that another count shares them out better)")
    ap.add_argument("--sweep", action="store_true", help="time the affine shape sweep M x K x N instead of the decode")
    ap.add_argument("--write-digests", default=None, metavar="PATH",
                    help="decode the whole corpus of the big and base workloads and write the per-mini-batch output digests (the "
                         "file committed as tests/golden/decode_digests.json) instead of timing")
    ap.add_argument("--trace", default=None, metavar="PATH",
                    help="decode one mini-batch with the in-situ kernel timeline on and write its per-kernel summary to PATH")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="step-driver tuning switch (fuse_weights, quant_in_gemm, fused_output_max_rows, side_stream, attention_unroll)")
    ap.add_argument("--legacy-sample", action="store_true",
                    help="time what earlier versions of this benchmark timed (a corpus of (warmup + steps) mini-batches sorted longest first, "
                         "warm-up on the longest, the rest timed), for comparisons with their numbers; no digest check")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline sample (for quick A/B runs)")
    ap.add_argument("--strong", action="store_true",
                    help="strong scaling: the whole fixed corpus, mini-batches taken from a shared counter by whichever rank is free")
    ap.add_argument("--glue", default=None, metavar="KERNEL",
                    help="time one glue kernel at the benchmark's decode shapes (attention1_self, attention1_cross, quantize_slot, "
                         "add_layernorm, lse_topk, cluster_affine, cluster_affine_layernorm), the form the ncu captures use")
    ap.add_argument("--tile-sweep", default=None, metavar="M,K,N",
                    help="time the GEMM alone (operands already quantised) for every tile width and split-K factor the kernel offers")
    ap.add_argument("--packed8", action="store_true",
                    help="time the packed8avx512 affine on the weight shapes the reference's mjdgemm instantiates, the reference's own CPU code beside it")
    return ap.parse_args()


def corpus_batches(model_mod, cfg, wl):
    """The workload's whole corpus as length-sorted mini-batches (maxi-batch style): the same list for every N."""
    if wl.get("mini_batch") not in (None, 0) and wl.get("sentences", 0) % wl["mini_batch"] != 0:
        wl = dict(wl, sentences=(wl["sentences"] // wl["mini_batch"] + 1) * wl["mini_batch"])
    corpus = model_mod.synthetic_corpus(wl["sentences"], cfg.vocab, seed=1, **wl["lengths"])
    return model_mod.make_batches(corpus, wl["mini_batch"])


def batch_order(n_batches):
    """One fixed shuffled order of the corpus' mini-batches; the timed set is a prefix of it (cyclic when N x K exceeds it)."""
    import numpy as np
    return [int(i) for i in np.random.default_rng(7).permutation(n_batches)]


def deal_batches(picked, widths, rank, world):
    """The reference gives the next mini-batch to the next free device (src/translator/translator.h:154-167); for a
    pre-dealt list the equivalent is equally long work per rank: widest first, dealt in snake order."""
    ranked = sorted(picked, key=lambda b: -widths[b])
    mine = []
    for i, b in enumerate(ranked):
        group, pos = divmod(i, world)
        if (pos if group % 2 == 0 else world - 1 - pos) == rank:
            mine.append(b)
    return mine


def tokens_digest(sent_ids, results):
    """sha256 over (sentence id, length, tokens) of one mini-batch in sentence-id order."""
    import hashlib
    import numpy as np
    h = hashlib.sha256()
    for sid, toks in sorted(zip((int(x) for x in sent_ids), (list(t) for t in results))):
        h.update(np.asarray([sid, len(toks)] + toks, dtype=np.int32).tobytes())
    return h.hexdigest()


def load_digests(name):
    try:
        return json.load(open(os.path.join(ROOT, "tests", "golden", "decode_digests.json"))).get(name, {}).get("batches", {})
    except OSError:
        return {}


# DRAM read + write bytes of ONE launch of the decode's dominant GEMM shape (dram__bytes_read.sum + dram__bytes_write.sum),
# from the ncu captures summarised in profiles/decode_kernels_ncu_b200.md (key: M, N, K).  They are BELOW the algorithmic bytes:
# the fp32 output of these launches is still in the 126 MB L2 when the kernel ends, and part of the operands never left it.
NCU_DRAM_BYTES_PER_LAUNCH = {(512, 1024, 1024): 1.63e6, (512, 4096, 1024): 4.79e6, (512, 1024, 4096): 6.35e6, (512, 32000, 1024): 44.0e6}


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs (read-only queries)."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile(prefix="clocks_", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=f, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- GEMM attribution
class GemmTimer:
    """Has the library bracket every GEMM launch with CUDA events on the launching stream
    (mi8_profile_begin / mi8_profile_end), so the dominant kernel's achieved bandwidth / throughput is
    measured inside the timed region."""

    def __init__(self, capacity=200000):
        self.capacity = capacity
        self.records = []

    def __enter__(self):
        from marian_dev_b200.binding import check, lib
        check(lib().mi8_profile_begin(self.capacity))
        return self

    def __exit__(self, *exc):
        import ctypes
        from marian_dev_b200.binding import Mi8GemmRecord, check, lib
        buf = (Mi8GemmRecord * self.capacity)()
        n = ctypes.c_int(0)
        check(lib().mi8_profile_end(buf, self.capacity, ctypes.byref(n)))
        self.records = [(r.M, r.N, r.K, r.out_bytes, r.us, r.rows_computed) for r in buf[:n.value]]

    def summary(self):
        """Aggregate per shape class.  Bytes and operations are those of the rows a launch really computed
        (`rows_computed`, written by the kernel: launches over stored keys/values skip what is unchanged)."""
        total = {"launches": 0, "us": 0.0, "bytes": 0.0, "ops": 0.0}
        classes = {}
        for (m, n, k, ob, us, rows) in self.records:
            if rows > 0:
                by = rows * k + n * k + 4 * n + ob * rows * n + 8          # int8 A in, weights, bias, C out, two multipliers
                op = 2.0 * rows * n * k
                key = f"M={m if m <= 512 else '>512'},N={n},K={k}"
            else:
                by, op = 0.0, 0.0
                key = f"N={n},K={k}: earlier history slabs, nothing to recompute (launch exits)"
            c = classes.setdefault(key, {"launches": 0, "us": 0.0, "bytes": 0.0, "ops": 0.0, "m": m, "n": n, "k": k})
            for d in (c, total):
                d["launches"] += 1
                d["us"] += us
                d["bytes"] += by
                d["ops"] += op
        return total, classes


# ----------------------------------------------------------------------------- our arm
def _apply_options(stepper, args):
    for item in args.option:
        name, _, value = item.partition("=")
        stepper.set_option(name.strip(), int(value))


def _setup(args):
    import torch
    import torch.distributed as dist
    from marian_dev_b200 import decoder, model
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the int8 engine has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    cfg = model.CONFIGS[args.model]
    params = model.random_init(cfg, seed=0)
    net = decoder.Int8Transformer(cfg, params, dev, output_int8=True)
    del params
    wl = workload(args)
    batches = corpus_batches(model, cfg, wl)
    stepper = decoder.NativeStepper(net, max_batch=wl["mini_batch"], beam=wl["beam"], max_src=136, max_steps=208)
    _apply_options(stepper, args)
    search = decoder.BeamSearch(net, beam=wl["beam"], max_length_factor=1.5, normalize=1.0, native=stepper)
    return world, rank, local_rank, dev, cfg, wl, batches, stepper, search


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from marian_dev_b200 import ops, parallel

    world, rank, local_rank, dev, cfg, wl, batches, stepper, search = _setup(args)
    from marian_dev_b200 import decoder as decoder_mod
    pool = decoder_mod.SearchPool(search.m, pick_workers(args.workers, args.steps), beam=wl["beam"], max_length_factor=1.5, normalize=1.0,
                                  max_batch=wl["mini_batch"], max_src=136, max_steps=208, first=stepper)
    for st in pool.steppers:            # (after the pool set its own defaults)
        _apply_options(st, args)
    if args.legacy_sample:
        from marian_dev_b200 import model as model_mod
        per_rank = args.warmup + args.steps
        corpus = model_mod.synthetic_corpus(per_rank * world * wl["mini_batch"], cfg.vocab, seed=1, **wl["lengths"])
        batches = model_mod.make_batches(corpus, wl["mini_batch"])
    widths = [b[1].shape[1] for b in batches]
    order = batch_order(len(batches))
    need = world * args.steps
    if args.legacy_sample:
        own = parallel.shard_batches(list(range(len(batches))), rank, world, snake=True)
        warm, mine, picked = own[:args.warmup], own[args.warmup:args.warmup + args.steps], list(range(len(batches)))
        golden = {}
    else:
        picked = [order[i % len(order)] for i in range(need)]
        mine = deal_batches(picked, widths, rank, world)[:args.steps]
        warm = [order[(need + i) % len(order)] for i in range(args.warmup)]          # other mini-batches than the timed ones
        golden = load_digests(args.model) if not (args.mini_batch or args.beam) else {}
    max_len = int(np.ceil(1.5 * max(widths))) + 2

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def gather_outputs(collected):
        """The path's one collective, once per timed leg (the reference's OutputCollector also runs beside the
        decoding, not in lock-step with it): every rank contributes its {sentence id: tokens} as one int32 matrix and receives
        every rank's matrix in host memory.  (Turning the matrices into Python lists is parallel.merge_output_matrices, outside
        the timed region.)"""
        return parallel.gather_output_matrices(collected, max_len=max_len, device=dev)

    if world > 1:      # the collective's own set-up (communicator, kernels for this message size) stays out of the timed region
        gather_outputs({i: [0] * max_len for i in range(args.steps * wl["mini_batch"])})

    # warm-up (every worker decodes every warm-up mini-batch once)
    for b in warm:
        for srch in pool.searches:
            srch.search(batches[b][1], batches[b][2])
    if len(pool.searches) > 1:
        pool.run([(batches[b][1], batches[b][2]) for b in warm])
    torch.cuda.synchronize()

    # ---- leg 1: inputs resident in HBM ------------------------------------------------------
    leg1 = [batches[b] for b in mine]
    resident = [(sid, torch.from_numpy(ids.astype(np.int64)).to(dev), torch.from_numpy(mask).to(dev)) for sid, ids, mask in leg1]
    sampler = ClockSampler(local_rank)
    sampler.start()       # nvidia-smi takes a few hundred ms to come up (it opens the driver): it does so beside one more warm-up decode
    settle = batches[(warm or mine)[0]]
    pool.searches[0].search(settle[1], settle[2])
    torch.cuda.synchronize()
    time.sleep(0.25)
    launches_before = ops.launch_count()          # warm-up launches (lets a profiler skip them)
    ops.reset_launch_count()
    for st in pool.steppers:
        st.search_stats(reset=True)
    tokens = 0
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    collected = {}
    results1 = pool.run([(ids_t, mask_t) for _sid, ids_t, mask_t in resident], on_device=True)   # (orders this stream behind every worker)
    for (sid, _i, _m), res in zip(resident, results1):
        collected.update({int(i): toks for i, (toks, _s) in zip(sid, res)})
        tokens += sum(len(t) for t, _ in res)
    mats1 = gather_outputs(collected)
    e1.record()
    barrier()
    if world > 1 and not args.legacy_sample:       # every rank holds every timed sentence's tokens
        got_ids = parallel.merge_output_matrices(mats1)
        want_n = sum(len(batches[b][0]) for b in set(picked))
        if len(got_ids) != want_n:
            raise RuntimeError(f"rank {rank}: the gathered outputs hold {len(got_ids)} sentences, expected {want_n}")
    digests1 = [tokens_digest(sid, [t for t, _ in res]) for (sid, _i, _m), res in zip(resident, results1)]    # (hashed outside the timed region)
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    launches = ops.launch_count()
    host = {"issue_s": 0.0, "wait_s": 0.0, "host_s": 0.0, "steps": 0}
    for st in pool.steppers:
        for k, v in st.search_stats(reset=True).items():
            host[k] += v

    # the output of the timed leg against the committed digests (tests/golden/decode_digests.json)
    checked = mismatched = 0
    for b, dg in zip(mine, digests1):
        want = golden.get(str(b))
        if want is not None:
            checked += 1
            mismatched += int(want != dg)
    if mismatched:
        raise RuntimeError(f"rank {rank}: the decoded tokens of {mismatched} of {checked} timed mini-batches differ from "
                           "tests/golden/decode_digests.json: no number is reported for a wrong output")

    # ---- the same region once more with every GEMM launch bracketed by CUDA events (the events sit
    # between kernels and so cost some overlap: this pass attributes time, the pass above is the value)
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with GemmTimer() as gt:
        p0.record()
        for sid, ids_t, mask_t in resident:
            search.search_device(ids_t, mask_t)
        p1.record()
        barrier()
    ms_profiled = p0.elapsed_time(p1)
    gemm_total, gemm_classes = gt.summary()

    # ---- and once with every kernel bracketed (mi8_kernel_times_*): per kernel function its launches and device time
    kernel_table = None
    if rank == 0:
        import ctypes
        import re
        from marian_dev_b200.binding import Mi8KernelTime, check, lib
        check(lib().mi8_kernel_times_begin())
        for sid, ids_t, mask_t in resident[:max(1, min(3, len(resident) // 2))]:
            search.search_device(ids_t, mask_t)
        buf = (Mi8KernelTime * 64)()
        n = ctypes.c_int(0)
        check(lib().mi8_kernel_times_end(buf, 64, ctypes.byref(n)))
        rows = []
        for r in buf[:n.value]:
            nm = r.name.decode(errors="replace")
            short = max((b for b in KERNEL_NAMES if b in nm), key=len, default=nm[:40])        # readable part of the mangled symbol
            targs = re.findall(r"ILi(\d+)E|Li(\d+)E|Lb([01])E", nm[nm.find(short):])
            rows.append((short + ("<" + ",".join(x or y or z for x, y, z in targs) + ">" if targs else ""), int(r.launches), float(r.total_us)))
        tot = sum(us for _, _, us in rows) or 1.0
        merged = {}
        for nm, l, us in rows:
            a = merged.setdefault(nm, [0, 0.0])
            a[0] += l
            a[1] += us
        kernel_table = [{"kernel": k, "launches": v[0], "us": round(v[1], 1), "share": round(v[1] / tot, 4)}
                        for k, v in sorted(merged.items(), key=lambda kv: -kv[1][1])]
    barrier()

    # ---- leg 2: end to end through the public call with host buffers --------------------------
    pinned = [(sid, torch.from_numpy(ids.astype(np.int64)).pin_memory(), torch.from_numpy(mask).pin_memory()) for sid, ids, mask in leg1]
    pool.reset_counters()
    tokens2 = 0
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    collected = {}
    results2 = pool.run([(ids_p, mask_p) for _sid, ids_p, mask_p in pinned])
    for (sid, _i, _m), res in zip(pinned, results2):
        collected.update({int(i): toks for i, (toks, _s) in zip(sid, res)})
        tokens2 += sum(len(t) for t, _ in res)
    gather_outputs(collected)
    f1.record()
    barrier()
    digests2 = [tokens_digest(sid, [t for t, _ in res]) for (sid, _i, _m), res in zip(pinned, results2)]
    ms2 = f0.elapsed_time(f1)
    if digests2 != digests1:
        raise RuntimeError(f"rank {rank}: the end-to-end leg decoded different tokens than the device-resident leg")
    h2d, d2h = pool.h2d_bytes / max(1, len(pinned)), pool.d2h_bytes / max(1, len(pinned))
    status = ops.poll_status()
    int8_peak = round(ops.measure_int8_peak(), 1) if rank == 0 else None   # after the timed legs: it must not disturb them

    per_rank = None
    if world > 1:
        mine_ms = torch.tensor([ms, ms2], device=dev, dtype=torch.float64)
        every = [torch.zeros_like(mine_ms) for _ in range(world)]
        dist.all_gather(every, mine_ms)
        per_rank = [round(float(x[0]), 2) for x in every]
        ms, ms2 = max(float(x[0]) for x in every), max(float(x[1]) for x in every)
        c = torch.tensor([tokens, tokens2, launches, checked], device=dev, dtype=torch.float64)
        dist.all_reduce(c, op=dist.ReduceOp.SUM)
        tokens, tokens2, launches, checked = int(c[0]), int(c[1]), int(c[2]), int(c[3])

    if rank == 0:
        import hashlib
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        hbm_peak = peaks.get("hbm_gbs", 6650.0)
        peak_src = "measured" if "hbm_gbs" in peaks else "fallback"

        def rates(v):
            return {"launches": v["launches"], "us_total": round(v["us"], 1), "avg_us": round(v["us"] / max(1, v["launches"]), 2),
                    "GBps": round(v["bytes"] / max(v["us"], 1e-9) / 1e3, 1), "TOPS": round(v["ops"] / max(v["us"], 1e-9) / 1e6, 1)}

        by_shape = {k: rates(v) for k, v in sorted(gemm_classes.items(), key=lambda kv: -kv[1]["us"])}
        dom_key, dom = max(gemm_classes.items(), key=lambda kv: kv[1]["us"])       # the shape class the GEMM kernel spends most time in
        dom_rate = rates(dom)
        all_rate = rates(gemm_total)
        roofline = {
            "kernel": f"mi8_gemm_kernel, the decode's dominant shape class {dom_key} ({dom['launches']} launches, "
                      f"{round(100.0 * dom['us'] / max(gemm_total['us'], 1e-9), 1)} % of the GEMM time)",
            "bound": "hbm", "achieved": dom_rate["GBps"], "peak": hbm_peak, "unit": "GB/s",
            "frac": round(dom_rate["GBps"] / hbm_peak, 4), "peak_source": peak_src,
            "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get((dom["m"], dom["n"], dom["k"])),
            "avg_launch_us": dom_rate["avg_us"], "tops": dom_rate["TOPS"],
            "timing": "CUDA events around every GEMM launch of a repeat of the timed region (launch overlap off for that pass); "
                      "bytes and operations count the rows each launch really computed",
            "all_gemm_launches": dict(all_rate, frac=round(all_rate["GBps"] / hbm_peak, 4)),
            "int8_mma_peak_tops": int8_peak,   # a loop of the kernel's MMAs alone, measured on this GPU right after the timed legs
            "gemm_share_of_step_time": round(gemm_total["us"] / 1e3 / max(ms_profiled, 1e-9), 3),
            "profiled_pass_ms": round(ms_profiled, 2),
            "by_shape": by_shape,
        }
        steps_done = max(1, host["steps"])
        cpu = cpu_baseline(args, cfg_name=args.model) if world == 1 and not args.no_cpu_baseline else None
        line = {
            "metric": METRIC, "value": round(tokens / (ms / 1e3), 1), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / max(1, args.steps), 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 (s8 x s8 -> s32), fp32 epilogue",
            "data": "synthetic (random-init weights, uniform token ids, seeded)",
            "config": {"workload": wl["desc"], "mini_batch": wl["mini_batch"], "beam": wl["beam"],
                       "corpus": f"{wl['sentences']} sentences = {len(batches)} length-sorted mini-batches; timed: the first {need} of a fixed "
                                 f"shuffled order (widths {sorted(widths[b] for b in picked)[0]}..{sorted(widths[b] for b in picked)[-1]}, "
                                 f"mean {round(sum(widths[b] for b in picked) / len(picked), 1)}; corpus mean {round(sum(widths) / len(widths), 1)}), "
                                 "warm-up on other mini-batches",
                       "tokens_counted": "best hypothesis per sentence, EOS included", "parallelism": f"replicas x{world}",
                       "searches_side_by_side_per_gpu": len(pool.searches),
                       "gemm_tiles": ("256 activation rows per tile (several searches share the GPU: fewer fetches of every weight tile)"
                                      if len(pool.searches) > 1 and not any(o.startswith("gemm_tile_rows") for o in args.option)
                                      else "the plan's latency tiles unless an option says otherwise"),
                       "options": args.option, "legacy_sample": bool(args.legacy_sample),
                       "l2": "not flushed: one decode step streams ~0.2 GB of int8 weights plus fp32 logits and history, more than the 126 MB L2"},
            "e2e": {"value": round(tokens2 / (ms2 / 1e3), 1), "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": int(launches), "gpu_launches_before_timed_region": int(launches_before), "clocks": clocks,
            "outputs": {"digest": hashlib.sha256("".join(digests1).encode()).hexdigest()[:16], "mini_batches_checked_against_golden": checked,
                        "mismatches": 0, "e2e_leg_identical": True},
            # where the host thread of rank 0 spent the timed leg, per decoder step: issuing launches, waiting for the device
            # (the step's one synchronisation), beam bookkeeping
            "host_per_decoder_step_us": {"issue": round(1e6 * host["issue_s"] / steps_done, 1), "wait_for_device": round(1e6 * host["wait_s"] / steps_done, 1),
                                         "bookkeeping": round(1e6 * host["host_s"] / steps_done, 1), "decoder_steps": host["steps"],
                                         "launches_per_decoder_step": round(launches / world / steps_done, 1)},
            # per kernel: launches / device time / share, CUDA events around every launch of a few of the timed mini-batches;
            # launches serialise while timed, so every launch carries its ~4 us launch latency: compare shares
            "kernels": kernel_table, "roofline": roofline, "device_status": status,
        }
        if per_rank is not None:
            line["per_rank_ms"] = per_rank
            line["rank_spread"] = round(max(per_rank) / max(min(per_rank), 1e-9), 4)
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_write_digests(args):
    """Decodes the whole corpus of the big and base workloads on cuda:0 and writes the digest of every mini-batch."""
    import numpy as np
    import torch
    out = {"made_by": "python bench.py --write-digests PATH (on a B200); tests/test_gpu_decode_bench_config.py compares entries with the CPU checker",
           "digest": "sha256 over int32 (sentence id, length, tokens...) of the mini-batch's sentences in sentence-id order"}
    for name in ("big", "base"):
        a = argparse.Namespace(**vars(args))
        a.model, a.mini_batch, a.beam = name, 0, 0
        world, rank, local_rank, dev, cfg, wl, batches, stepper, search = _setup(a)
        d = {}
        tokens = 0
        for i, (sid, ids, mask) in enumerate(batches):
            res = search.search(ids, mask)
            d[str(i)] = tokens_digest(sid, [t for t, _ in res])
            tokens += sum(len(t) for t, _ in res)
        out[name] = {"sentences": wl["sentences"], "mini_batch": wl["mini_batch"], "beam": wl["beam"], "tokens": tokens, "batches": d}
        del stepper, search
        torch.cuda.empty_cache()
    with open(args.write_digests, "w") as f:
        json.dump(out, f, indent=1)
    print(json.dumps({"wrote": args.write_digests, "big_tokens": out["big"]["tokens"], "base_tokens": out["base"]["tokens"]}), flush=True)


# Beam searches side by side per GPU: measured speed-up over one search on transformer-big (wide GEMM tiles from 3 on).
WORKER_SPEEDUP = {1: 1.0, 2: 1.27, 3: 1.55, 4: 1.72, 5: 1.70, 6: 1.57}


def pick_workers(requested, n_batches):
    """The requested count, or the one that gets `n_batches` mini-batches done soonest under a simple model (rounds of w
    concurrent searches, each round w / speed-up(w) long): 4 once there are enough mini-batches to keep four busy."""
    if requested > 0:
        return requested
    if n_batches <= 0:
        return 4
    best = min(WORKER_SPEEDUP, key=lambda w: (-(-n_batches // w) * w / WORKER_SPEEDUP[w], abs(w - 4)))
    return min(best, n_batches)


TRACE_KERNELS = {1: "mi8_gemm_kernel", 2: "mi8_gemm_pair_kernel", 3: "quantize_slot_kernel", 4: "quantize_dual_kernel", 5: "add_layernorm_kernel",
                 6: "attention1_kernel", 7: "attention_enc_kernel", 8: "lse_topk_kernel", 9: "lse_merge_kernel", 10: "nbest_merge_kernel",
                 11: "embed_kernel", 12: "ancestors_update_kernel", 13: "history_commit_kernel", 14: "gather_rows_kernel", 15: "ssru_cell_kernel",
                 16: "mi8_absmax_kernel", 17: "mi8_quantize_kernel", 18: "mi8_gemm_kernel (output layer, reducing write-back)",
                 19: "mi8_gemm_kernel (quantising its activation)", 20: "mi8_gemm_cq_kernel"}


def run_trace(args):
    """One mini-batch (of median width) decoded with the in-situ timeline on: every kernel stamps the GPU's nanosecond timer at
    its entry, when its wait for the preceding kernel returns and when its block 0 ends, with launch overlap left on.  Written
    to PATH: per kernel (and GEMM shape) the launches, the time from `wait returned` to `end` (the kernel's own work), the time
    from the previous kernel's end to this kernel's `wait returned` (the hand-over gap) and their shares of the decoder steps."""
    import ctypes
    import numpy as np
    import torch
    from marian_dev_b200.binding import check, lib
    world, rank, local_rank, dev, cfg, wl, batches, stepper, search = _setup(args)
    widths = [b[1].shape[1] for b in batches]
    b = sorted(range(len(batches)), key=lambda i: widths[i])[len(batches) // 2]
    sid, ids, mask = batches[b]
    for _ in range(2):
        search.search(ids, mask)
    torch.cuda.synchronize()
    cap = 1000000
    buf = torch.zeros(2 + 2 * cap, dtype=torch.int64, device=dev)
    check(lib().mi8_trace_begin(buf.data_ptr(), cap))
    stepper.search_stats(reset=True)
    t0 = time.perf_counter()
    res = search.search(ids, mask)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    check(lib().mi8_trace_end())
    host = stepper.search_stats(reset=True)
    raw = buf.cpu().numpy()
    n = int(min(raw[0], cap))
    t = raw[2:2 + 2 * n:2].astype(np.int64)
    tag = raw[3:3 + 2 * n:2].astype(np.uint64)
    phase = (tag & np.uint64(0xff)).astype(np.int64)
    kern = ((tag >> np.uint64(8)) & np.uint64(0xff)).astype(np.int64)
    extra = (tag >> np.uint64(16)).astype(np.uint64)
    # pair the stamps of each launch: launches of one kernel (and GEMM shape) follow one another on the stream, so the n-th
    # stamp of a phase belongs to the n-th launch.  Phases: 0 entry, 1 wait returned, 2 end of block 0, 3 end of the last block;
    # GEMMs also 4 first operands landed, 5 first accumulator complete, 6 its write-back issued.
    per_key = {}
    for i in range(n):
        key = (int(kern[i]), int(extra[i]))
        per_key.setdefault(key, {}).setdefault(int(phase[i]), []).append(int(t[i]))
    launches = []
    for key, ph in per_key.items():
        for idx, t_in in enumerate(ph.get(0, [])):
            if idx >= len(ph.get(1, [])) or idx >= len(ph.get(2, [])):
                continue
            t_end = ph[2][idx]
            if idx < len(ph.get(3, [])) and len(ph[3]) == len(ph[0]):
                t_end = max(t_end, ph[3][idx])
            inner = tuple(ph[k][idx] if idx < len(ph.get(k, [])) and len(ph[k]) == len(ph[0]) else None for k in (4, 5, 6))
            launches.append((key, t_in, ph[1][idx], t_end, inner))
    launches.sort(key=lambda r: r[2])
    agg = {}
    prev_end = None
    for key, t_in, t_wait, t_end, inner in launches:
        k, ex = key
        name = TRACE_KERNELS.get(k, str(k))
        if k in (1, 2, 18, 19, 20):
            name += f" N={ex & 0xfffff},K={(ex >> 20) & 0xfffff}"
        a = agg.setdefault(name, {"launches": 0, "work_ns": 0, "gap_ns": 0, "pre_ns": 0, "inner": [0, 0, 0, 0], "inner_n": 0})
        a["launches"] += 1
        a["work_ns"] += t_end - t_wait
        a["pre_ns"] += t_wait - t_in                      # how long the kernel was resident before its predecessor finished
        if prev_end is not None:
            a["gap_ns"] += max(0, t_wait - prev_end)
        if all(x is not None for x in inner):
            a["inner"][0] += inner[0] - t_wait            # wait returned -> first operands in shared memory
            a["inner"][1] += inner[1] - inner[0]          # -> first accumulator complete (main loop)
            a["inner"][2] += inner[2] - inner[1]          # -> its write-back issued
            a["inner"][3] += t_end - inner[2]             # -> kernel end (remaining tiles, teardown)
            a["inner_n"] += 1
        prev_end = max(prev_end or 0, t_end)
    span = (launches[-1][3] - launches[0][1]) if launches else 1
    rows = [{"kernel": k, "launches": v["launches"], "work_us": round(v["work_ns"] / 1e3, 1), "avg_work_us": round(v["work_ns"] / 1e3 / v["launches"], 2),
             "gap_before_us": round(v["gap_ns"] / 1e3, 1), "avg_gap_us": round(v["gap_ns"] / 1e3 / v["launches"], 2),
             "avg_resident_before_wait_us": round(v["pre_ns"] / 1e3 / v["launches"], 2),
             "share_of_span": round((v["work_ns"] + v["gap_ns"]) / span, 4),
             **({"gemm_phases_avg_us": {"operands_landed": round(v["inner"][0] / 1e3 / v["inner_n"], 2), "main_loop": round(v["inner"][1] / 1e3 / v["inner_n"], 2),
                                        "write_back": round(v["inner"][2] / 1e3 / v["inner_n"], 2), "rest": round(v["inner"][3] / 1e3 / v["inner_n"], 2)}}
                if v["inner_n"] else {})}
            for k, v in sorted(agg.items(), key=lambda kv: -(kv[1]["work_ns"] + kv[1]["gap_ns"]))]
    out = {"workload": wl["desc"], "mini_batch_index": b, "width": widths[b], "tokens": sum(len(x) for x, _ in res), "decoder_steps": host["steps"],
           "wall_ms": round(wall * 1e3, 2), "device_span_ms": round(span / 1e6, 2), "stamps": n, "launches_paired": len(launches),
           "host_per_decoder_step_us": {"issue": round(1e6 * host["issue_s"] / max(1, host["steps"]), 1),
                                        "wait_for_device": round(1e6 * host["wait_s"] / max(1, host["steps"]), 1),
                                        "bookkeeping": round(1e6 * host["host_s"] / max(1, host["steps"]), 1)},
           "options": args.option, "kernels": rows,
           "note": "work = from the return of block 0's wait for the preceding kernel to the later of block 0's and the last block's end; "
                   "gap = from the end of the preceding kernels to that return (launch hand-over and memory flush)"}
    with open(args.trace, "w") as f:
        json.dump(out, f, indent=1)
    print(json.dumps({k: out[k] for k in ("wall_ms", "device_span_ms", "decoder_steps", "tokens", "host_per_decoder_step_us")}), flush=True)
    for r in rows[:24]:
        print(json.dumps(r), flush=True)


def run_strong(args):
    """Strong scaling as the reference's translator does it (src/translator/translator.h:154-167: a thread pool in which the
    next free device takes the next mini-batch): the whole fixed corpus, longest mini-batches first, dealt from one shared
    counter (the process group's key-value store) to whichever rank asks next.  Prints one JSON line with "scaling": "strong",
    the per-rank busy times and their spread."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from marian_dev_b200 import ops, parallel
    world, rank, local_rank, dev, cfg, wl, batches, stepper, search = _setup(args)
    widths = [b[1].shape[1] for b in batches]
    by_cost = sorted(range(len(batches)), key=lambda i: -widths[i])
    golden = load_digests(args.model)
    max_len = int(np.ceil(1.5 * max(widths))) + 2
    next_batch = parallel.shared_counter()
    order = batch_order(len(batches))
    from marian_dev_b200 import decoder as decoder_mod
    pool = decoder_mod.SearchPool(search.m, pick_workers(args.workers, len(batches)), beam=wl["beam"], max_length_factor=1.5, normalize=1.0,
                                  max_batch=wl["mini_batch"], max_src=136, max_steps=208, first=stepper)
    for st in pool.steppers:            # (after the pool set its own defaults)
        _apply_options(st, args)
    for i in range(args.warmup):
        for srch in pool.searches:
            srch.search(batches[order[i]][1], batches[order[i]][2])
    if len(pool.searches) > 1:
        pool.run([(batches[order[i]][1], batches[order[i]][2]) for i in range(args.warmup)])
    torch.cuda.synchronize()
    pinned = [(sid, torch.from_numpy(ids.astype(np.int64)).pin_memory(), torch.from_numpy(mask).pin_memory()) for sid, ids, mask in batches]
    torch.cuda.synchronize()
    if world > 1:      # the collective's own set-up (communicator, kernels for this message size) stays out of the timed region
        parallel.gather_output_matrices({i: [0] * max_len for i in range(-(-wl["sentences"] // world))}, max_len=max_len, device=dev)
        dist.barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()       # (comes up beside one more warm-up decode, see run_ours)
    pool.searches[0].search(batches[order[0]][1], batches[order[0]][2])
    torch.cuda.synchronize()
    time.sleep(0.25)
    if world > 1:
        dist.barrier()
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    e0.record()
    tokens, mine, bad = 0, [], 0
    collected = {}

    def source():                       # (called under the pool's lock: one worker at a time talks to the store)
        i = next_batch()
        if i >= len(by_cost):
            return None
        b = by_cost[i]
        return b, pinned[b][1], pinned[b][2]
    for b, res in pool.run_from(source).items():
        sid = pinned[b][0]
        collected.update({int(x): toks for x, (toks, _s) in zip(sid, res)})
        tokens += sum(len(t) for t, _ in res)
        mine.append(b)
        want = golden.get(str(b))
        bad += int(want is not None and want != tokens_digest(sid, [t for t, _ in res]))
    e1.record()
    mats = parallel.gather_output_matrices(collected, max_len=max_len, device=dev)   # every rank's tokens are in this rank's host memory
    e2.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    merged = parallel.merge_output_matrices(mats)                                     # (turning them into Python lists is not timed)
    busy, total = e0.elapsed_time(e1), e0.elapsed_time(e2)
    if bad:
        raise RuntimeError(f"rank {rank}: {bad} mini-batches decoded to tokens that differ from tests/golden/decode_digests.json")
    per_rank, counts = [busy], [len(mine)]
    if world > 1:
        v = torch.tensor([busy, total, tokens, len(mine)], device=dev, dtype=torch.float64)
        every = [torch.zeros_like(v) for _ in range(world)]
        dist.all_gather(every, v)
        per_rank = [round(float(x[0]), 2) for x in every]
        counts = [int(x[3]) for x in every]
        total = max(float(x[1]) for x in every)
        tokens = int(sum(float(x[2]) for x in every))
    if rank == 0:
        assert len(merged) == wl["sentences"]
        print(json.dumps({"metric": METRIC, "value": round(tokens / (total / 1e3), 1), "unit": UNIT, "n_gpus": world, "scaling": "strong",
                          "steps": len(batches), "ms_total": round(total, 2), "higher_is_better": True,
                          "config": {"workload": wl["desc"], "corpus": f"{wl['sentences']} sentences, {len(batches)} mini-batches, longest first, "
                                     "taken from a shared counter by the next free search (" + str(len(pool.searches)) + " per rank)"},
                          "per_rank_busy_ms": per_rank, "per_rank_mini_batches": counts,
                          "rank_spread": round(max(per_rank) / max(min(per_rank), 1e-9), 4), "tokens": tokens, "clocks": clocks,
                          "device_status": ops.poll_status()}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_glue(args):
    """One glue kernel of the decoder step at the benchmark's shapes (512 hypothesis rows, d = 1024, 16 heads, 32000 words), called
    through the C ABI on operand sets rotated through more than the L2 capacity, launch overlap on, CUDA events around 200 launches."""
    import torch
    from marian_dev_b200.binding import check, lib
    L = lib()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    st = torch.cuda.current_stream().cuda_stream
    R, d, heads, dh, V = 512, 1024, 16, 64, 32000
    kind = args.glue
    for item in args.option:                                   # process-wide kernel switches (attention_unroll, attention_block_heads)
        name, _, value = item.partition("=")
        from marian_dev_b200.decoder import NativeStepper
        check(L.mi8d_set_option(None, NativeStepper.OPTIONS[name.strip()], int(value)))
    slot = torch.zeros(64, dtype=torch.int32, device=dev)
    if kind in ("attention1_self", "attention1_cross"):
        length, batch, mode = (24, 128, 0) if kind == "attention1_self" else (32, 128, 1)
        kv_rows = length * R if mode == 0 else batch * length
        sets = max(2, int(200e6 // (2 * kv_rows * d * 4)) + 1)
        q = [torch.randn(R, d, device=dev) for _ in range(sets)]
        k = [torch.randn(kv_rows, d, device=dev) for _ in range(sets)]
        v = [torch.randn(kv_rows, d, device=dev) for _ in range(sets)]
        out = torch.empty(R, d, device=dev)
        mask = torch.zeros(batch, length, device=dev)
        by = 2 * kv_rows * d * 4 + 2 * R * d * 4

        def run(i):
            j = i % sets
            check(L.mi8g_attention1(q[j].data_ptr(), k[j].data_ptr(), v[j].data_ptr(), mask.data_ptr() if mode == 1 else None, R, heads, dh, length,
                                    batch, mode, out.data_ptr(), slot.data_ptr(), st))
        shape = f"{R} rows x {heads} heads x {dh}, {length} positions, mode {mode}"
    elif kind == "quantize_slot":
        sets = 64
        x = [torch.randn(R, d, device=dev) for _ in range(sets)]
        qo = torch.empty(R * d + 256, dtype=torch.int8, device=dev)
        slot.view(torch.float32)[0] = 5.0
        by = R * d * 5

        def run(i):
            check(L.mi8g_quantize_slot(x[i % sets].data_ptr(), R * d, slot.data_ptr(), qo.data_ptr(), qo[R * d:].data_ptr(), st))
        shape = f"{R} x {d} fp32 -> int8"
    elif kind == "add_layernorm":
        sets = 32
        a = [torch.randn(R, d, device=dev) for _ in range(sets)]
        r = [torch.randn(R, d, device=dev) for _ in range(sets)]
        g, b = torch.ones(d, device=dev), torch.zeros(d, device=dev)
        out = torch.empty(R, d, device=dev)
        by = R * d * 12

        def run(i):
            j = i % sets
            check(L.mi8g_add_layernorm(a[j].data_ptr(), r[j].data_ptr(), g.data_ptr(), b.data_ptr(), 1e-6, R, d, out.data_ptr(), None, slot.data_ptr(), st))
        shape = f"{R} rows x {d}"
    elif kind == "lse_topk":
        sets = 4
        lg = [torch.randn(R, V, device=dev) for _ in range(sets)]
        cs = torch.empty(R * 8, device=dev)
        cw = torch.empty(R * 8, dtype=torch.int32, device=dev)
        by = R * V * 4

        def run(i):
            check(L.mi8g_lse_topk(lg[i % sets].data_ptr(), R, V, 4, None, cs.data_ptr(), cw.data_ptr(), st))
        shape = f"{R} rows x {V} words, k = 4"
    elif kind in ("cluster_affine", "cluster_affine_layernorm"):
        # the optional cluster GEMM (mi8g_affine_slot*): Wo of an attention block, 512 x 1024 x 1024, from fp32 + abs-max slot
        from marian_dev_b200 import ops
        sets = 24
        x = [torch.randn(R, d, device=dev) for _ in range(sets)]
        slot.view(torch.float32)[0] = 6.0                      # max|x| of a standard normal tensor of this size, roughly; any bound works
        w = [ops.prepareB(torch.randn(d, d, device=dev) * 0.03) for _ in range(sets)]
        bias = torch.randn(d, device=dev) * 0.01
        res = [torch.randn(R, d, device=dev) for _ in range(sets)]
        g, b = torch.ones(d, device=dev), torch.zeros(d, device=dev)
        out = torch.empty(R, d, device=dev)
        by = R * d * 4 + d * d + 4 * d + R * d * 4 + (R * d * 4 if kind.endswith("layernorm") else 0)

        def run(i):
            j = i % sets
            if kind.endswith("layernorm"):
                check(L.mi8g_affine_slot_add_layernorm(x[j].data_ptr(), slot.data_ptr(), w[j].data.data_ptr(), w[j].quant_mult.data_ptr(), R, d, d, 1.0,
                                                       bias.data_ptr(), res[j].data_ptr(), g.data_ptr(), b.data_ptr(), 1e-6, out.data_ptr(), None,
                                                       slot[8:].data_ptr(), None, st))
            else:
                check(L.mi8g_affine_slot(x[j].data_ptr(), slot.data_ptr(), w[j].data.data_ptr(), w[j].quant_mult.data_ptr(), R, d, d, 1.0,
                                         bias.data_ptr(), 0, out.data_ptr(), slot[8:].data_ptr(), 0, 0, st))
        shape = f"{R} x {d} x {d}, fp32 activation + abs-max slot" + (" , + residual + LayerNorm" if kind.endswith("layernorm") else "")
    else:
        raise SystemExit(f"unknown kernel {kind}")
    iters = 200
    for i in range(10):
        run(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        run(i)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1000.0 / iters
    print(json.dumps({"metric": "glue_kernel", "kernel": kind, "shape": shape, "us_per_launch": round(us, 2), "algorithmic_bytes": by,
                      "GBps": round(by / us / 1e3, 1), "operand_sets": sets, "options": args.option,
                      "timing": f"{iters} back-to-back launches (programmatic dependent launch on), CUDA events"}), flush=True)


# ----------------------------------------------------------------------------- CPU baseline / reference arm
_CPU_NET = {}


def cpu_decode_sample(args, cfg_name):
    """Times the CPU restatement on a bounded sample of the same workload: one mini-batch of a few
    sentences, same beam, all host threads.  The model is built once per process."""
    from marian_dev_b200 import model
    from oracle.decode_oracle import OracleTransformer, beam_search
    from oracle.oracle import COracle
    cfg = model.CONFIGS[cfg_name]
    if cfg_name not in _CPU_NET:
        params = model.random_init(cfg, seed=0)
        o = COracle()
        _CPU_NET[cfg_name] = (OracleTransformer(cfg, params, oracle=o, output_int8=True, threads=o.max_threads()), o.max_threads())
        del params
    net, cores = _CPU_NET[cfg_name]
    wl = workload(args)
    corpus = model.synthetic_corpus(wl["mini_batch"], cfg.vocab, seed=1, **wl["lengths"])
    n = min(args.cpu_sentences, len(corpus))
    # a typical slice of the length-sorted batch (around the median length)
    order = sorted(range(len(corpus)), key=lambda i: len(corpus[i]))
    pick = [corpus[i] for i in order[len(order) // 2 - n // 2: len(order) // 2 - n // 2 + n]]
    batches = model.make_batches(pick, n)
    t0 = time.time()
    tokens = 0
    for _sid, ids, mask in batches:
        for toks, _s in beam_search(net, ids, mask, beam=wl["beam"], max_length_factor=1.5, normalize=1.0):
            tokens += len(toks)
    dt = time.time() - t0
    return tokens / dt, cores, (f"{n} sentences of median length from one mini-batch decoded as one batch of {n} (the GPU arm decodes {wl['mini_batch']} at a time: "
                                f"context, not a like-for-like comparison), beam {wl['beam']}, {dt:.1f} s of CPU work")


def cpu_baseline(args, cfg_name):
    try:
        v, cores, sample = cpu_decode_sample(args, cfg_name)
        return {"value": round(v, 2), "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
    except Exception as e:  # the baseline must not take the GPU line down with it
        return {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"failed: {e}"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    vals = []
    cores, sample = 0, ""
    t_all = time.time()
    for i in range(args.warmup + args.steps):
        v, cores, sample = cpu_decode_sample(args, args.model)
        if i >= args.warmup:
            vals.append(v)
        if time.time() - t_all > 240 and vals:       # keep the whole arm within a few minutes
            break
    value = statistics.mean(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": len(vals),
        "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 (s8 x s8 -> s32), fp32 epilogue", "data": "synthetic (random-init weights, uniform token ids, seeded)",
        "config": {"workload": workload(args)["desc"], "mini_batch": workload(args)["mini_batch"], "beam": workload(args)["beam"],
                   "note": "CPU restatement of the reference's intgemm8 path (the reference itself is unbuildable here: intgemm submodule absent)"},
        "cpu_baseline": {"value": round(value, 2), "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 2), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- single affines (parity-config shapes)
def time_affine(m, k, n, iters=40):
    """One affine = prepareA (abs-max + quantise) + GEMM with fused bias/ReLU, through the C ABI, on operand
    sets rotated through more than the L2 capacity; returns a dict for one JSON line."""
    import torch
    from marian_dev_b200 import ops
    dev = torch.device("cuda", torch.cuda.current_device())
    per_copy = 4 * m * k + n * k + 4 * m * n
    copies = max(2, min(32, int(300e6 // per_copy) + 1))
    xs = [torch.randn(m, k, device=dev) for _ in range(copies)]
    ws = [ops.prepareB(torch.randn(k, n, device=dev) * 0.02) for _ in range(copies)]
    bias = torch.randn(n, device=dev) * 0.01
    outs = [torch.empty(m, n, device=dev) for _ in range(copies)]
    aq = [ops.IntgemmTensor(m, k, dev) for _ in range(copies)]
    wsp = ops.Workspace(device=dev)          # one workspace for the warm-up and the captured stream alike

    def run(i):
        j = i % copies
        ops.prepareA(xs[j], out=aq[j], ws=wsp)
        ops.multiply(aq[j], ws[j], bias, 1.0, True, out=outs[j], ws=wsp)

    for i in range(5):
        run(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            for i in range(iters):
                run(i)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        g.replay()
        e1.record(s)
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1000.0 / iters
    by = 4 * m * k + k * n + 4 * n + 4 * m * n + 8
    return {"M": m, "K": k, "N": n, "us_per_affine": round(us, 2), "GBps": round(by / us / 1e3, 1), "TOPS": round(2.0 * m * n * k / us / 1e6, 2),
            "algorithmic_bytes": by, "launches_per_affine": 3, "operand_sets": copies}


def time_affine_sharded(m, k, n, rank, world, iters=40):
    """The same affine with the rows of A split over the ranks (one MAX all-reduce of a float between the
    abs-max and the quantisation).  Launched eagerly (the collective sits between the kernels), timed with
    CUDA events, maximum over the ranks; GB/s and TOPS are for the whole M x K x N problem."""
    import torch
    import torch.distributed as dist
    from marian_dev_b200 import ops, parallel
    dev = torch.device("cuda", torch.cuda.current_device())
    b, e = parallel.shard_rows(m, rank, world)
    ml = e - b
    per_copy = 4 * ml * k + n * k + 4 * ml * n
    copies = max(2, min(32, int(300e6 // max(per_copy, 1)) + 1))
    g = torch.Generator(device=dev).manual_seed(1234)          # the same weights on every rank
    ws = [ops.prepareB(torch.randn(k, n, device=dev, generator=g) * 0.02) for _ in range(copies)]
    bias = torch.randn(n, device=dev, generator=g) * 0.01
    xs = [torch.randn(max(ml, 1), k, device=dev)[:ml] for _ in range(copies)]
    for i in range(5):
        if ml > 0:
            parallel.sharded_affine(xs[i % copies], ws[i % copies], bias, 1.0, True)
        else:
            parallel.global_abs_max(torch.zeros(1, device=dev))
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    def timed(exchange):
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            if ml > 0:
                parallel.sharded_affine(xs[i % copies], ws[i % copies], bias, 1.0, True, exchange=exchange)
            elif exchange:                                      # fewer rows than ranks: still take part in the exchange
                parallel.global_abs_max(torch.zeros(1, device=dev))
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1000.0 / iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])
    us = timed(True)
    us_local = timed(False)       # the same launches without the all-reduce (per-shard multipliers): what the exchange costs
    by = 4 * m * k + k * n + 4 * n + 4 * m * n + 8
    return {"M": m, "K": k, "N": n, "us_per_affine": round(us, 2), "GBps": round(by / us / 1e3, 1), "TOPS": round(2.0 * m * n * k / us / 1e6, 2),
            "us_without_exchange": round(us_local, 2), "exchange_share": round(max(0.0, 1.0 - us_local / us), 3),
            "algorithmic_bytes": by, "n_gpus": world, "rows_per_rank": (m + world - 1) // world, "operand_sets": copies}


def time_packed8(m, k, n, iters=40):
    """One packed8avx512 affine = per-row uint8 quantisation + uint8 x int8 GEMM with the zero-point / scale / bias
    write-back (2 launches), through the C ABI, CUDA-graph replay over operand sets larger than L2."""
    import numpy as np
    import torch
    from marian_dev_b200 import ops, packed8
    from marian_dev_b200.binding import check, lib
    dev = torch.device("cuda", torch.cuda.current_device())
    L = lib()
    per_copy = 4 * m * k + n * k + 4 * m * n
    copies = max(2, min(32, int(300e6 // per_copy) + 1))
    rng = np.random.default_rng(0)
    host_item = np.zeros(int(L.mi8p_packed_bytes(k, n)), np.int8)
    host_item[:k * n] = rng.integers(-64, 64, size=k * n, dtype=np.int8)
    tail = host_item[k * n:]
    tail[:4 * n].view(np.float32)[:] = 0.001
    tail[4 * n:8 * n].view(np.int32)[:] = 3
    tail[8 * n:].view(np.int32)[:] = -7
    ws = [packed8.Packed8Weight(host_item, k, n, device=dev) for _ in range(copies)]
    xs = [torch.randn(m, k, device=dev) for _ in range(copies)]
    bias = torch.randn(n, device=dev) * 0.01
    outs = [torch.empty(m, n, device=dev) for _ in range(copies)]
    scratch = [torch.empty(max(256, int(L.mi8p_scratch_bytes(m, k))), dtype=torch.uint8, device=dev) for _ in range(copies)]
    wsp = ops.default_workspace(dev)

    def run(i, stream):
        j = i % copies
        w = ws[j]
        check(L.mi8p_gemm_int8_packed(xs[j].data_ptr(), w.bt.data_ptr(), w.scale_b.data_ptr(), w.zp_b.data_ptr(), w.off_b.data_ptr(),
                                      bias.data_ptr(), outs[j].data_ptr(), m, n, k, scratch[j].data_ptr(), scratch[j].numel(),
                                      wsp.ptr, wsp.nbytes, stream))

    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for i in range(5):
            run(i, s.cuda_stream)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for i in range(iters):
                run(i, s.cuda_stream)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        g.replay()
        e1.record(s)
        torch.cuda.synchronize()
    if ops.poll_status() != 0:
        raise RuntimeError("device status set during the packed8 timing")
    us = e0.elapsed_time(e1) * 1000.0 / iters
    by = 4 * m * k + k * n + 12 * n + 4 * n + 4 * m * n
    return {"M": m, "K": k, "N": n, "us_per_affine": round(us, 2), "GBps": round(by / us / 1e3, 1), "TOPS": round(2.0 * m * n * k / us / 1e6, 2),
            "algorithmic_bytes": by, "launches_per_affine": 2, "operand_sets": copies}


def time_packed8_reference(m, k, n, budget_s=0.6):
    """The reference's own gemmInt8Packed (compiled from its tree into oracle/_ref) on the host: one call on one
    thread, and one call per hardware thread at once (Marian runs one translation worker per core)."""
    import threading
    import numpy as np
    from oracle.oracle import Packed8Item, RefMjdgemm, aligned_copy, aligned_empty
    ref = RefMjdgemm()
    rng = np.random.default_rng(1)
    packed = aligned_empty((k * n + 12 * n,), np.int8)
    packed[:k * n] = rng.integers(-64, 64, size=k * n, dtype=np.int8)
    item = Packed8Item(packed, k, n)
    item.scale_b[:] = 0.001
    a = aligned_copy(rng.standard_normal((m, k)).astype(np.float32))
    bias = aligned_copy(rng.standard_normal(n).astype(np.float32))
    c = aligned_empty((m, n), np.float32)
    import ctypes

    def vp(x):
        return x.ctypes.data_as(ctypes.c_void_p)

    def call(out):
        ref.L.ref_mjd_gemm(vp(a), vp(packed), vp(bias), vp(out), m, n, k)

    call(c)
    t0 = time.perf_counter()
    reps = 0
    while reps < 3 or time.perf_counter() - t0 < budget_s / 2:
        call(c)
        reps += 1
    single_us = (time.perf_counter() - t0) / reps * 1e6
    cores = os.cpu_count() or 1
    outs = [aligned_empty((m, n), np.float32) for _ in range(cores)]
    per_thread = max(2, int(budget_s / 2 / (single_us * 1e-6)))

    def worker(o):
        for _ in range(per_thread):
            call(o)

    threads = [threading.Thread(target=worker, args=(o,)) for o in outs]
    t0 = time.perf_counter()
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    all_us = (time.perf_counter() - t0) / (per_thread * cores) * 1e6
    return {"us_per_affine_1_thread": round(single_us, 1), "us_per_affine_all_cores": round(all_us, 2), "cores": cores, "isa": ref.isa()}


def run_packed8(args):
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the int8 engine has no CPU path")
    torch.cuda.set_device(0)
    warm = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16)
    for _ in range(30):
        warm @ warm
    torch.cuda.synchronize()
    shapes_nk = [(512, 512), (1024, 1024), (4096, 1024), (3072, 1024), (1024, 4096), (8192, 512), (512, 8192), (1024, 512), (512, 1024),
                 (32000, 512)]
    if args.affine:                                     # one shape, GPU only (the form the ncu captures use)
        m, k, n = (int(v) for v in args.affine.split(","))
        r = time_packed8(m, k, n, iters=10)
        r.update({"metric": "packed8avx512_affine", "timing": "CUDA-graph replay of 10 affines, CUDA events"})
        print(json.dumps(r), flush=True)
        return
    for (n, k) in shapes_nk:
        for m in (1, 8, 64, 256, 1024):
            r = time_packed8(m, k, n)
            r.update({"metric": "packed8avx512_affine", "timing": "CUDA-graph replay of 40 affines, CUDA events, operand sets rotated through > L2"})
            try:
                cpu = time_packed8_reference(m, k, n)
                best_all = cpu["us_per_affine_all_cores"] < cpu["us_per_affine_1_thread"]
                r["cpu_baseline"] = {"value": cpu["us_per_affine_all_cores"] if best_all else cpu["us_per_affine_1_thread"], "unit": "us/affine",
                                     "cores": cpu["cores"] if best_all else 1, "kind": "reference",
                                     "sample": f"gemmInt8Packed of oracle/_ref (ISA {cpu['isa']}): single thread {cpu['us_per_affine_1_thread']} us, "
                                               f"one call per hardware thread at once {cpu['us_per_affine_all_cores']} us per affine"}
            except FileNotFoundError:
                r["cpu_baseline"] = None
            print(json.dumps(r), flush=True)


def run_tile_sweep(args):
    """The int8 GEMM alone on one shape under every plan the kernel accepts: tile widths 32..256 (and the two-CTA kernel) x split-K
    1..8, CUDA-graph replay of 40 launches over operand sets rotated through more than the L2 capacity.  The plan the library
    would pick by itself is marked."""
    import torch
    from marian_dev_b200 import multiply_plan, ops
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    m, k, n = (int(v) for v in args.tile_sweep.split(","))
    per_copy = m * k + n * k + 4 * m * n
    copies = max(2, min(32, int(300e6 // per_copy) + 1))
    aqs = [ops.prepareA(torch.randn(m, k, device=dev)) for _ in range(copies)]
    ws = [ops.prepareB(torch.randn(k, n, device=dev) * 0.02) for _ in range(copies)]
    bias = torch.randn(n, device=dev) * 0.01
    outs = [torch.empty(m, n, device=dev) for _ in range(copies)]
    wsp = ops.Workspace(device=dev)
    auto = multiply_plan(m, n, k)
    warm = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)
    for _ in range(20):
        warm @ warm
    for tile in (0, 16, 32, 64, 128, 256, 512):
        for splits in (0, 1, 2, 4, 8):
            if (tile == 0) != (splits == 0) or (tile == 512 and splits > 1) or (tile == 16 and m > 16):
                continue
            try:
                plan = multiply_plan(m, n, k, tile, splits)

                def run(i):
                    j = i % copies
                    ops.multiply(aqs[j], ws[j], bias, 1.0, False, out=outs[j], ws=wsp, tile_m=tile, splits=splits)
                for i in range(3):
                    run(i)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                st = torch.cuda.Stream()
                with torch.cuda.stream(st):
                    with torch.cuda.graph(g, stream=st):
                        for i in range(40):
                            run(i)
                    g.replay()
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(st)
                    g.replay()
                    e1.record(st)
                    torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1000.0 / 40
            except Exception as e:                      # a plan the kernel refuses for this shape
                print(json.dumps({"M": m, "K": k, "N": n, "tile": tile, "splits": splits, "refused": str(e)[:80]}), flush=True)
                continue
            by = m * k + k * n + 4 * n + 4 * m * n + 8
            print(json.dumps({"M": m, "K": k, "N": n, "tile": plan["tile_m"], "splits": plan["splits"], "ctas": plan["grid"],
                              "automatic": tile == 0, "us": round(us, 2), "GBps": round(by / us / 1e3, 1),
                              "TOPS": round(2.0 * m * n * k / us / 1e6, 1)}), flush=True)
    if ops.poll_status() != 0:
        raise RuntimeError("device status set during the tile sweep")


def run_affines(args):
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the int8 engine has no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    warm = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16)
    for _ in range(30):
        warm @ warm                                   # bring the clocks up before timing microsecond kernels
    if args.sweep and rank == 0:
        from marian_dev_b200 import ops
        print(json.dumps({"metric": "int8_mma_peak", "TOPS": round(ops.measure_int8_peak(), 1),
                          "how": "loop of tcgen05.mma kind::i8 128x256x32 on every SM, no loads or stores, CUDA events, best of 3"}), flush=True)
    torch.cuda.synchronize()
    if args.affine:
        shapes = [tuple(int(v) for v in args.affine.split(","))]
    else:
        shapes = [(m, k, n) for m in (1, 8, 64, 256, 1024, 4096) for k in (512, 1024, 4096) for n in (512, 2048, 4096, 32000)]
    for (m, k, n) in shapes:
        if world > 1:
            r = time_affine_sharded(m, k, n, rank, world)
            r.update({"metric": "int8_affine_rows_sharded",
                      "timing": "40 eager affines per rank (abs-max, MAX all-reduce of one float, quantise, GEMM), CUDA events, max over ranks; us_without_exchange = the same loop with the all-reduce left out"})
        else:
            r = time_affine(m, k, n)
            r.update({"metric": "int8_affine", "timing": "CUDA-graph replay of 40 affines, CUDA events, operand sets rotated through > L2"})
        if rank == 0:
            print(json.dumps(r), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    a = parse_args()
    if a.trace:      # the build of the library that carries the timeline stamps (the product library is built without them)
        os.environ["MARIAN_I8_LIBRARY"] = os.path.join(ROOT, "marian-dev_b200", "libmarian_i8_trace.so")
    if a.write_digests:
        run_write_digests(a)
    elif a.trace:
        run_trace(a)
    elif a.glue:
        run_glue(a)
    elif a.strong:
        run_strong(a)
    elif a.tile_sweep:
        run_tile_sweep(a)
    elif a.packed8:
        run_packed8(a)
    elif a.affine or a.sweep:
        run_affines(a)
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
