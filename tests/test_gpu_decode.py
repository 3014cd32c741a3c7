"""End-to-end decode parity: the GPU decoder (int8 engine + torch glue) against the independent
NumPy/C restatement, on random-init models and synthetic sentences.  Sequences must be identical
for at least 99 % of the sentences (float glue such as softmax and LayerNorm rounds differently on
the two sides, so exact agreement on every sentence is not required)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _decode_both(cfg_name, n_sent, mini_batch, beam, seed, lo=3, hi=12, output_int8=True):
    from marian_dev_b200 import decoder, model, ops
    from oracle.decode_oracle import OracleTransformer, beam_search
    cfg = model.CONFIGS[cfg_name]
    params = model.random_init(cfg, seed)
    corpus = model.synthetic_corpus(n_sent, cfg.vocab, seed + 1, "uniform", lo, hi)
    batches = model.make_batches(corpus, mini_batch)
    gpu = decoder.Int8Transformer(cfg, params, torch.device("cuda", 0), output_int8=output_int8)
    got, n_tok = decoder.decode_corpus(gpu, batches, beam=beam)
    assert ops.poll_status() == 0
    ref_model = OracleTransformer(cfg, params, output_int8=output_int8, threads=8)
    want = {}
    for sent_ids, ids, mask in batches:
        for sid, (toks, _s) in zip(sent_ids, beam_search(ref_model, ids, mask, beam=beam)):
            want[int(sid)] = toks
    same = sum(1 for k in want if want[k] == got[k])
    return same, len(want), got, want, n_tok


@pytest.mark.parametrize("cfg_name", ["tiny", "tiny-ssru"])
@pytest.mark.parametrize("beam", [1, 4])
def test_tiny_decode_matches_oracle(cuda_device, cfg_name, beam):
    same, total, got, want, n_tok = _decode_both(cfg_name, 48, 16, beam, seed=5)
    assert n_tok > 0
    assert same >= 0.99 * total, f"only {same}/{total} sentences identical"
    # every hypothesis ends by EOS or by reaching 1.5 x the batch width
    assert all(len(t) > 0 for t in got.values())


def test_decode_fp32_output_layer_mode(cuda_device):
    # reference-faithful mode: the tied output layer stays fp32 (Marian does not convert Wemb)
    same, total, *_ = _decode_both("tiny", 16, 8, 4, seed=9, output_int8=False)
    assert same >= 0.99 * total


def test_batch_purging_path(cuda_device):
    """A model whose output bias strongly favours EOS finishes hypotheses early, which exercises beam
    shrinking, dummy hypothesis slots and sentences leaving the batch."""
    from marian_dev_b200 import decoder, model, ops
    from oracle.decode_oracle import OracleTransformer, beam_search
    cfg = model.CONFIGS["tiny"]
    params = model.random_init(cfg, 3)
    params["decoder_ff_logit_out_b"][0, cfg.eos_id] += 4.0
    corpus = model.synthetic_corpus(40, cfg.vocab, 4, "uniform", 4, 14)
    batches = model.make_batches(corpus, 20)
    gpu = decoder.Int8Transformer(cfg, params, torch.device("cuda", 0))
    got, _ = decoder.decode_corpus(gpu, batches, beam=4)
    assert ops.poll_status() == 0
    ref_model = OracleTransformer(cfg, params, threads=8)
    want = {}
    for sent_ids, ids, mask in batches:
        for sid, (toks, _s) in zip(sent_ids, beam_search(ref_model, ids, mask, beam=4)):
            want[int(sid)] = toks
    lens = [len(t) for t in want.values()]
    assert min(lens) < max(lens), "the EOS-biased model should finish sentences at different times"
    assert any(t and t[-1] == cfg.eos_id for t in want.values())
    same = sum(1 for k in want if want[k] == got[k])
    assert same >= 0.99 * len(want), f"only {same}/{len(want)} identical"
