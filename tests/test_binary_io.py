"""The binary model container, following the reference's own binary test
(src/tests/units/binary_tests.cpp:14-77: two items saved, reloaded, 256-byte padding, version word)
plus the intgemm8 item layout of marian-conv."""
import struct

import numpy as np
import pytest

from marian_dev_b200 import binary_io as bio


def test_two_items_roundtrip_like_the_reference_test(tmp_path):
    v1 = np.array([3.14, 2.71, 1.0, 0.0, 1.41], np.float32)
    v2 = np.array([5, 4, 3, 2, 1, 0], np.uint16)
    item1 = bio.Item("item1", [5, 1], bio.TYPE_FLOAT32, bio._pad256(v1.tobytes()))
    item2 = bio.Item("item2", [2, 3], 0x0200 + 2, bio._pad256(v2.tobytes()))     # Type::uint16
    path = str(tmp_path / "m.bin")
    bio.save_items(path, [item1, item2])
    raw = open(path, "rb").read()
    assert struct.unpack_from("<Q", raw, 0)[0] == bio.BINARY_FILE_VERSION      # magic number at the beginning of the file
    items = bio.load_items(path)
    assert [i.name for i in items] == ["item1", "item2"]
    assert items[0].shape == [5, 1] and items[1].shape == [2, 3]
    assert items[0].bytes[:v1.nbytes] == v1.tobytes() and items[1].bytes[:v2.nbytes] == v2.tobytes()
    assert all(len(i.bytes) % 256 == 0 for i in items)
    # payload starts on a 256-byte boundary
    assert (len(raw) - sum(len(i.bytes) for i in items)) % 256 == 0
    # loading from memory (what the reference does for mmap) gives the same
    again = bio.load_items(raw)
    assert again[1].bytes == items[1].bytes


def test_unaligned_item_is_rejected(tmp_path):
    with pytest.raises(ValueError, match="not 256-byte aligned"):
        bio.save_items(str(tmp_path / "x.bin"), [bio.Item("a", [3], bio.TYPE_FLOAT32, b"\0" * 12)])
    with pytest.raises(ValueError, match="Unknown binary file version"):
        bio.load_items(struct.pack("<QQ", 7, 0))


def test_intgemm8_item_layout_and_meta():
    bt = (np.arange(6 * 16).reshape(6, 16) % 200 - 100).astype(np.int8)       # Bt[N=6, K=16]
    it = bio.intgemm8_item("encoder_l1_ffn_W1", bt, 42.5, (16, 6))
    assert it.type == 0x10001 and it.shape == [16, 6]                          # logical [K,N], untransposed
    assert it.bytes[:96] == bt.tobytes()
    assert struct.unpack_from("<f", it.bytes, 96)[0] == 42.5                   # multiplier right behind the last element
    assert len(it.bytes) == 256
    meta = bio.meta_item("type: transformer\n")
    assert meta.type == 0x101 and meta.shape == [256] and meta.bytes.startswith(b"type: transformer\n\0")
    for name, want in [("decoder_l1_self_Wq", True), ("decoder_l2_rnn_W", True), ("decoder_l2_rnn_Wf", True), ("Wemb", False),
                       ("encoder_l1_self_bq", False), ("decoder_ff_logit_out_b", False), ("encoder_l1_ffn_W1", True)]:
        assert bio.is_intgemm_param(name) == want


def test_packed8avx512_item_layout(tmp_path):
    k, n = 256, 32
    packed = (np.arange(k * n + 12 * n) % 251 - 125).astype(np.int8)
    it = bio.packed8_item("encoder_l1_ffn_W1", packed, (k, n))
    assert it.type == 0x2801 and it.shape == [k, n]                            # Type::packed8avx512, logical [K,N]
    assert it.bytes[:packed.size] == packed.tobytes() and len(it.bytes) % 256 == 0
    path = str(tmp_path / "m.bin")
    bio.save_items(path, [it, bio.meta_item("type: transformer\n")])
    back = bio.load_items(path)[0]
    assert back.type == 0x2801 and back.shape == [k, n] and back.bytes[:packed.size] == packed.tobytes()
    assert bio.TYPE_NAMES[back.type] == "packed8avx512"


def test_hardware_specific_intgemm_items_are_refused():
    it = bio.Item("x_W", [16, 8], 0x10001 + 0x2000, b"\0" * 256)               # intgemm8avx512
    with pytest.raises(ValueError, match="hardware-specific"):
        bio.items_to_params([it], device="cpu")


@pytest.mark.gpu
def test_convert_save_load_decode_identical(cuda_device, tmp_path):
    import torch
    from marian_dev_b200 import decoder, model
    cfg = model.CONFIGS["tiny"]
    params = model.random_init(cfg, 2)
    items = bio.convert(params, cfg.to_yaml(), "intgemm8", device=cuda_device)
    path = str(tmp_path / "tiny.intgemm8.bin")
    bio.save_items(path, items)
    yaml_text, loaded = bio.items_to_params(bio.load_items(path), device=cuda_device)
    cfg2 = model.TransformerConfig.from_yaml(yaml_text)
    assert (cfg2.dim_emb, cfg2.dim_ffn, cfg2.heads, cfg2.enc_depth, cfg2.dec_depth, cfg2.vocab) == \
           (cfg.dim_emb, cfg.dim_ffn, cfg.heads, cfg.enc_depth, cfg.dec_depth, cfg.vocab)
    n_int8 = sum(1 for i in items if i.type == bio.TYPE_INTGEMM8)
    assert n_int8 == sum(1 for k in params if bio.is_intgemm_param(k)) and "Wemb" in loaded and isinstance(loaded["Wemb"], np.ndarray)
    corpus = model.synthetic_corpus(12, cfg.vocab, 3, "uniform", 3, 10)
    batches = model.make_batches(corpus, 6)
    outs = []
    for p in (params, loaded):
        net = decoder.Int8Transformer(cfg, p, cuda_device)
        st = decoder.NativeStepper(net, max_batch=6, beam=4, max_src=12, max_steps=32)
        outs.append(decoder.decode_corpus(net, batches, beam=4, native=st)[0])
    assert outs[0] == outs[1]
