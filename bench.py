#!/usr/bin/env python
"""Benchmark of the int8 decode path: transformer-big, beam 4, mini-batch 128, synthetic sentences.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is the decode of one mini-batch (128 synthetic sentences, beam 4) on one GPU: encoder,
then decoder steps until every hypothesis ended or 1.5 x the source width is reached, with every
weight multiplication on the int8 engine.  With N GPUs every rank holds a full model replica and
decodes its own K mini-batches (mini-batches are dealt round-robin, as the reference's translator
does); the only collective is the gather of the output token matrix.  Rank 0 prints one JSON line.

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
                "add_layernorm_kernel", "history_quantize_kernel", "history_absmax_kernel", "history_commit_kernel", "lse_topk_kernel",
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
    "big": dict(desc=WORKLOAD, mini_batch=128, beam=4, lengths=dict(length_dist="normal", lo=4, hi=128, mean=30.0, std=12.0)),
    "base": dict(desc="transformer-base decode (6+6 layers, d=512, ffn=2048, 8 heads, tied 32000 vocab, all affines int8), beam 4, "
                      "mini-batch 64, lengths U[8,64], max length 1.5x source",
                 mini_batch=64, beam=4, lengths=dict(length_dist="uniform", lo=8, hi=64)),
    "student": dict(desc="student decode (12 encoder layers d=256 ffn=1536 8 heads, 2-layer SSRU decoder, 32000 vocab, all affines int8), "
                         "greedy, lengths U[5,40], max length 1.5x source",
                    mini_batch=16, beam=1, lengths=dict(length_dist="uniform", lo=5, hi=40)),
}


def workload(args):
    w = dict(WORKLOADS.get(args.model, WORKLOADS["big"]))
    if args.model not in WORKLOADS:
        w["desc"] = f"{args.model} (debug workload)"
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
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="big", help="big (the benchmark), base, student, tiny (debugging)")
    ap.add_argument("--mini-batch", type=int, default=0, help="override the workload's mini-batch (sentences)")
    ap.add_argument("--beam", type=int, default=0, help="override the workload's beam size")
    ap.add_argument("--cpu-sentences", type=int, default=16, help="sentences in the CPU-baseline sample")
    ap.add_argument("--affine", default=None, help="M,K,N: time one int8 affine (abs-max + quantise + GEMM with bias and ReLU) instead of the decode")
    ap.add_argument("--sweep", action="store_true", help="time the affine shape sweep M x K x N instead of the decode")
    ap.add_argument("--packed8", action="store_true",
                    help="time the packed8avx512 affine on the weight shapes the reference's mjdgemm instantiates, the reference's own CPU code beside it")
    return ap.parse_args()


def build_corpus(model_mod, cfg, n_batches, wl):
    n = n_batches * wl["mini_batch"]
    corpus = model_mod.synthetic_corpus(n, cfg.vocab, seed=1, **wl["lengths"])
    return model_mod.make_batches(corpus, wl["mini_batch"])


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
        self.records = [(r.M, r.N, r.K, r.out_bytes, r.us) for r in buf[:n.value]]

    def summary(self):
        """Aggregate per shape class."""
        total = {"launches": 0, "us": 0.0, "bytes": 0.0, "ops": 0.0}
        classes = {}
        for (m, n, k, ob, us) in self.records:
            by = m * k + n * k + 4 * n + ob * m * n + 8          # int8 A in, weights, bias, C out, two multipliers
            op = 2.0 * m * n * k
            key = ("history K/V re-projection (M = rows x steps)" if m > 1024 and n == k else f"N={n},K={k}")
            c = classes.setdefault(key, {"launches": 0, "us": 0.0, "bytes": 0.0, "ops": 0.0})
            for d in (c, total):
                d["launches"] += 1
                d["us"] += us
                d["bytes"] += by
                d["ops"] += op
        return total, classes


# ----------------------------------------------------------------------------- our arm
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from marian_dev_b200 import decoder, model, ops, parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the int8 engine has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = model.CONFIGS[args.model]
    params = model.random_init(cfg, seed=0)
    net = decoder.Int8Transformer(cfg, params, dev, output_int8=True)
    del params
    per_rank = args.warmup + args.steps                          # both timed legs decode the same mini-batches
    wl = workload(args)
    batches = build_corpus(model, cfg, per_rank * world, wl)
    mine = parallel.shard_batches(batches, rank, world, snake=True)[:per_rank]   # length-sorted list: snake order balances the ranks
    stepper = decoder.NativeStepper(net, max_batch=wl["mini_batch"], beam=wl["beam"], max_src=136, max_steps=208)
    search = decoder.BeamSearch(net, beam=wl["beam"], max_length_factor=1.5, normalize=1.0, native=stepper)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def gather_outputs(collected):
        """The path's one collective, once per timed leg (the reference's OutputCollector also runs beside the
        decoding, not in lock-step with it): every rank contributes its {sentence id: tokens}; all receive the union."""
        return parallel.gather_outputs(collected, max_len=192, device=dev)   # 192 = 1.5 x the longest source

    # warm-up
    for b in mine[:args.warmup]:
        search.search(b[1], b[2])
    torch.cuda.synchronize()

    # ---- leg 1: inputs resident in HBM ------------------------------------------------------
    leg1 = mine[args.warmup:args.warmup + args.steps]
    resident = [(sid, torch.from_numpy(ids.astype(np.int64)).to(dev), torch.from_numpy(mask).to(dev)) for sid, ids, mask in leg1]
    sampler = ClockSampler(local_rank)
    launches_before = ops.launch_count()          # warm-up launches (lets a profiler skip them)
    ops.reset_launch_count()
    tokens = 0
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    collected = {}
    for sid, ids_t, mask_t in resident:
        res = search.search_device(ids_t, mask_t)
        collected.update({int(i): toks for i, (toks, _s) in zip(sid, res)})
        tokens += sum(len(t) for t, _ in res)
    gather_outputs(collected)
    e1.record()
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    launches = ops.launch_count()

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
        for sid, ids_t, mask_t in resident[:max(1, len(resident) // 2)]:
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
    leg2 = leg1
    pinned = [(sid, torch.from_numpy(ids.astype(np.int64)).pin_memory(), torch.from_numpy(mask).pin_memory()) for sid, ids, mask in leg2]
    search.h2d_bytes = search.d2h_bytes = 0
    tokens2 = 0
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    collected = {}
    for sid, ids_p, mask_p in pinned:
        res = search.search(ids_p, mask_p)
        collected.update({int(i): toks for i, (toks, _s) in zip(sid, res)})
        tokens2 += sum(len(t) for t, _ in res)
    gather_outputs(collected)
    f1.record()
    barrier()
    ms2 = f0.elapsed_time(f1)
    h2d, d2h = search.h2d_bytes / max(1, len(pinned)), search.d2h_bytes / max(1, len(pinned))
    status = ops.poll_status()
    int8_peak = round(ops.measure_int8_peak(), 1) if rank == 0 else None   # after the timed legs: it must not disturb them

    if world > 1:
        t = torch.tensor([ms, ms2], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms2 = float(t[0]), float(t[1])
        c = torch.tensor([tokens, tokens2, launches], device=dev, dtype=torch.float64)
        dist.all_reduce(c, op=dist.ReduceOp.SUM)
        tokens, tokens2, launches = int(c[0]), int(c[1]), int(c[2])

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        hbm_peak = peaks.get("hbm_gbs", 6650.0)
        peak_src = "measured" if "hbm_gbs" in peaks else "fallback"
        achieved = gemm_total["bytes"] / max(gemm_total["us"], 1e-9) / 1e3          # GB/s
        roofline = {
            "kernel": "mi8_gemm_kernel (all launches of the timed region)",
            "bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
            "frac": round(achieved / hbm_peak, 4), "peak_source": peak_src,
            # DRAM read + write of one output-layer launch (M=512, K=1024, N=32000; algorithmic 98.9 MB, part of C stays in L2),
            # measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum) on one launch of that shape
            "traffic": 44.7e6, "traffic_unit": "bytes per launch of the 512x1024x32000 shape",
            "launches": gemm_total["launches"], "avg_launch_us": round(gemm_total["us"] / max(1, gemm_total["launches"]), 2),
            "tops": round(gemm_total["ops"] / max(gemm_total["us"], 1e-9) / 1e6, 1),
            "int8_mma_peak_tops": int8_peak,   # a loop of the kernel's MMAs alone, measured on this GPU right after the timed legs
            "gemm_share_of_step_time": round(gemm_total["us"] / 1e3 / max(ms_profiled, 1e-9), 3),
            "profiled_pass_ms": round(ms_profiled, 2),
            "by_shape": {k: {"launches": v["launches"], "us_total": round(v["us"], 1),
                             "GBps": round(v["bytes"] / max(v["us"], 1e-9) / 1e3, 1),
                             "TOPS": round(v["ops"] / max(v["us"], 1e-9) / 1e6, 1)} for k, v in sorted(gemm_classes.items(), key=lambda kv: -kv[1]["us"])},
        }
        cpu = cpu_baseline(args, cfg_name=args.model) if world == 1 else None
        line = {
            "metric": METRIC, "value": round(tokens / (ms / 1e3), 1), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / max(1, args.steps), 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 (s8 x s8 -> s32), fp32 epilogue",
            "data": "synthetic (random-init weights, uniform token ids, seeded)",
            "config": {"workload": wl["desc"], "mini_batch": wl["mini_batch"], "beam": wl["beam"],
                       "tokens_counted": "best hypothesis per sentence, EOS included", "parallelism": f"replicas x{world}",
                       "l2": "not flushed: one decode step streams ~0.2 GB of int8 weights plus fp32 logits and history, more than the 126 MB L2"},
            "e2e": {"value": round(tokens2 / (ms2 / 1e3), 1), "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": int(launches), "gpu_launches_before_timed_region": int(launches_before), "clocks": clocks,
            # per kernel: launches / device time / share, CUDA events around every launch of half the timed mini-batches;
            # launches serialise while timed, so every launch carries its ~4 us launch latency: compare shares
            "kernels": kernel_table, "roofline": roofline, "device_status": status,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


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
    return tokens / dt, cores, f"{n} sentences of median length from one mini-batch, beam {wl['beam']}, {dt:.1f} s of CPU work"


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

    def run(i):
        j = i % copies
        ops.prepareA(xs[j], out=aq[j])
        ops.multiply(aq[j], ws[j], bias, 1.0, True, out=outs[j])

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
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        if ml > 0:
            parallel.sharded_affine(xs[i % copies], ws[i % copies], bias, 1.0, True)
        else:                                                   # fewer rows than ranks: still take part in the exchange
            parallel.global_abs_max(torch.zeros(1, device=dev))
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1000.0 / iters], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    us = float(t[0])
    by = 4 * m * k + k * n + 4 * n + 4 * m * n + 8
    return {"M": m, "K": k, "N": n, "us_per_affine": round(us, 2), "GBps": round(by / us / 1e3, 1), "TOPS": round(2.0 * m * n * k / us / 1e6, 2),
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
                      "timing": "40 eager affines per rank (abs-max, MAX all-reduce of one float, quantise, GEMM), CUDA events, max over ranks"})
        else:
            r = time_affine(m, k, n)
            r.update({"metric": "int8_affine", "timing": "CUDA-graph replay of 40 affines, CUDA events, operand sets rotated through > L2"})
        if rank == 0:
            print(json.dumps(r), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    a = parse_args()
    if a.packed8:
        run_packed8(a)
    elif a.affine or a.sweep:
        run_affines(a)
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
