"""A packed8avx512 model through the decoder step driver (mi8d_set_packed8_weight + mi8d_search), against the CPU checker's decode
with every affine on the restatement of the reference's mjdgemm route (oracle_packed8.c, itself held to the reference's compiled
mjdgemm by tests/test_packed8_oracle.py).  The reference runs whole models on this format
(src/tensors/cpu/fbgemm/packed_gemm.cpp:566-592); activations are quantised per row there, so the driver keeps earlier
keys/values as a cache - the outputs must still equal the checker's, which recomputes them from the whole history every step."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _items(cfg, params):
    """Conversion on the CPU (marian-conv --gemm-type packed8avx512 restated): name -> Packed8Item, incl. the tied output matrix."""
    from marian_dev_b200.model import is_intgemm_param
    from oracle.oracle import Packed8Oracle
    chk = Packed8Oracle()
    items = {name: chk.prepare_b(np.ascontiguousarray(val, np.float32)) for name, val in params.items() if is_intgemm_param(name)}
    items["Wemb_packed8"] = chk.prepare_b(np.ascontiguousarray(params["Wemb"].T, dtype=np.float32))
    return items


@pytest.mark.parametrize("cfg_name,beam,upload_items", [("small", 4, True), ("small", 1, True), ("small-ssru", 4, True), ("small", 4, False)])
def test_packed8_model_decodes_like_the_checker(cuda_device, cfg_name, beam, upload_items):
    from marian_dev_b200 import decoder, model, ops, packed8
    from oracle.decode_oracle import OracleTransformer, beam_search
    cfg = model.CONFIGS[cfg_name]
    params = model.random_init(cfg, 21)
    params["decoder_ff_logit_out_b"][0, cfg.eos_id] += 3.0          # hypotheses end at different steps: beams shrink, sentences leave
    corpus = model.synthetic_corpus(36, cfg.vocab, 22, "uniform", 4, 16)
    batches = model.make_batches(corpus, 18)
    items = _items(cfg, params)
    ref = OracleTransformer(cfg, params, threads=8, scheme="packed8avx512", packed_items=items)
    want = {}
    for sent_ids, ids, mask in batches:
        for s, (toks, _s) in zip(sent_ids, beam_search(ref, ids, mask, beam=beam)):
            want[int(s)] = toks
    if upload_items:      # the model as read from a converted file: the same item bytes on both sides
        gpu_params = {k: v for k, v in params.items() if k not in items}
        gpu_params.update({k: packed8.Packed8Weight(it.packed, it.K, it.N, device=cuda_device) for k, it in items.items()})
    else:                 # a float model converted on the device
        gpu_params = params
    gpu = decoder.Int8Transformer(cfg, gpu_params, cuda_device, scheme="packed8avx512")
    stepper = decoder.NativeStepper(gpu, max_batch=18, beam=max(beam, 1), max_src=20, max_steps=40)
    got, n_tok = decoder.decode_corpus(gpu, batches, beam=beam, native=stepper)
    assert ops.poll_status() == 0 and n_tok > 0
    lens = [len(t) for t in want.values()]
    assert min(lens) < max(lens)
    diff = [k for k in want if want[k] != got[k]]
    assert not diff, f"{cfg_name} beam {beam}: {len(diff)} of {len(want)} sentences differ"


def test_mixing_schemes_is_refused(cuda_device):
    """A decoder with one packed8avx512 weight expects all of them in that format."""
    from marian_dev_b200 import decoder, model, ops, packed8
    cfg = model.CONFIGS["small"]
    params = model.random_init(cfg, 3)
    gpu = decoder.Int8Transformer(cfg, params, cuda_device)                      # an intgemm8 model
    stepper = decoder.NativeStepper(gpu, max_batch=4, beam=2, max_src=12, max_steps=24)
    w = packed8.prepareB(torch.from_numpy(params["decoder_l1_ffn_W1"]).to(cuda_device))
    from marian_dev_b200.binding import lib
    assert lib().mi8d_set_packed8_weight(stepper.h, b"decoder_l1_ffn_W1", w.bt.data_ptr(), w.scale_b.data_ptr(), w.zp_b.data_ptr(),
                                         w.off_b.data_ptr(), w.K, w.N) == 0
    corpus = model.synthetic_corpus(4, cfg.vocab, 5, "uniform", 4, 8)
    sid, ids, mask = model.make_batches(corpus, 4)[0]
    with pytest.raises(ops.Mi8Error) as e:
        decoder.BeamSearch(gpu, beam=2, native=stepper).search(ids, mask)
    assert e.value.status == 1
