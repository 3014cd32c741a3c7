"""Decode parity at the configurations the benchmark runs, full-size mini-batches.

transformer-big, beam 4, mini-batch 128, lengths clip(N(30,12),4,128): with 512 hypothesis rows the 32-row tiles on 128
CTAs, the CTA-pair kernel for the history re-projection, the materialised-logits output route and the fused K|V
launches are the ones that run - none of which a small mini-batch reaches.  transformer-base, beam 4, mini-batch 64,
lengths U[8,64] likewise.  The corpora are the benchmark's own (same seeds, same batching); the CPU checker's decode
costs minutes per long mini-batch, so one full mini-batch of typical width is compared per model.  The bar is >= 99 %
identical sequences; the driver's float glue rounds like the checker's, so the assertion is 100 %.
The digests of tests/golden/decode_digests.json (what bench.py verifies its timed output against) are checked here
against the same GPU output, which ties them to the checker."""
import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench_batches(name):
    import bench
    from marian_dev_b200 import model
    wl = bench.WORKLOADS[name]
    cfg = model.CONFIGS[name]
    return cfg, wl, bench.corpus_batches(model, cfg, wl)


@pytest.mark.parametrize("name,batch_index", [("big", 48), ("base", 16)])
def test_full_mini_batch_identical_to_checker(cuda_device, name, batch_index):
    from marian_dev_b200 import decoder, model, ops
    from oracle.decode_oracle import OracleTransformer, beam_search
    from oracle.oracle import COracle
    cfg, wl, batches = _bench_batches(name)
    sid, ids, mask = batches[batch_index]
    assert ids.shape[0] == wl["mini_batch"]
    params = model.random_init(cfg, seed=0)
    gpu = decoder.Int8Transformer(cfg, params, cuda_device)
    stepper = decoder.NativeStepper(gpu, max_batch=wl["mini_batch"], beam=wl["beam"], max_src=136, max_steps=208)
    search = decoder.BeamSearch(gpu, beam=wl["beam"], max_length_factor=1.5, normalize=1.0, native=stepper)
    got = [t for t, _ in search.search(ids, mask)]
    assert ops.poll_status() == 0
    o = COracle()
    ref = OracleTransformer(cfg, params, oracle=o, output_int8=True, threads=o.max_threads())
    want = [t for t, _ in beam_search(ref, ids, mask, beam=wl["beam"], max_length_factor=1.5, normalize=1.0)]
    same = sum(1 for a, b in zip(got, want) if a == b)
    assert same == len(want), f"{name}: only {same}/{len(want)} sentences identical at mini-batch {wl['mini_batch']}"
    golden = json.load(open(os.path.join(ROOT, "tests", "golden", "decode_digests.json")))
    import bench
    assert golden[name]["batches"][str(batch_index)] == bench.tokens_digest(sid, got)


def test_options_do_not_change_the_output(cuda_device):
    """Every tuning switch of the step driver computes the same values: a width-128 model (where Wk|Wv, Wq|Wk|Wv and the
    SSRU's W|Wf run fused) decoded under each setting, against the checker and against each other."""
    from marian_dev_b200 import decoder, model, ops
    from oracle.decode_oracle import OracleTransformer, beam_search
    for cfg_name, beam in (("small", 4), ("small-ssru", 4), ("small", 1)):
        cfg = model.CONFIGS[cfg_name]
        params = model.random_init(cfg, 11)
        params["decoder_ff_logit_out_b"][0, cfg.eos_id] += 3.0          # hypotheses end at different steps
        corpus = model.synthetic_corpus(40, cfg.vocab, 12, "uniform", 4, 18)
        batches = model.make_batches(corpus, 20)
        ref = OracleTransformer(cfg, params, threads=8)
        want = {}
        for sent_ids, ids, mask in batches:
            for s, (toks, _s) in zip(sent_ids, beam_search(ref, ids, mask, beam=beam)):
                want[int(s)] = toks
        gpu = decoder.Int8Transformer(cfg, params, cuda_device)
        settings = [{}, {"fuse_weights": 0}, {"quant_in_gemm": 1}, {"fused_output_max_rows": 0}, {"fused_output_max_rows": 4096},
                    {"side_stream": 0}, {"attention_unroll": 16}, {"attention_block_heads": 2}, {"attention_block_heads": 0},
                    {"cluster_affine": 1}, {"cluster_affine": 1, "fused_layernorm": 0}, {"cluster_affine": 1, "cluster_size": 2},
                    {"cluster_affine": 1, "cluster_max_rows": 8}, {"cluster_affine": 1, "cluster_max_k": 256},
                    {"gemm_tile_rows": 64}, {"gemm_tile_rows": 256}, {"gemm_tile_rows": 512}, {"blocking_wait": 1}, {"blocking_wait": 2}]
        for opts in settings:
            stepper = decoder.NativeStepper(gpu, max_batch=20, beam=beam, max_src=24, max_steps=48)
            for k, v in opts.items():
                stepper.set_option(k, v)
            got, _ = decoder.decode_corpus(gpu, batches, beam=beam, native=stepper)
            stepper.set_option("attention_unroll", 8)                    # (these switches are process-wide: back to the defaults)
            stepper.set_option("attention_block_heads", 8)
            assert ops.poll_status() == 0
            diff = [k for k in want if want[k] != got[k]]
            assert not diff, f"{cfg_name} beam {beam} with {opts}: {len(diff)} of {len(want)} sentences differ"
