"""Synthetic Marian transformer models and their intgemm8 conversion.

Parameter names and shapes follow the call sites of the reference's legacy transformer
(src/models/transformer.h:290-343 attention, :446-448 FFN via src/layers/generic.h:224-246,
src/rnn/cells.h:1007-1012 SSRU, src/layers/embedding.cpp:184-185 ``Wemb``,
src/layers/output.cpp:57-58 ``decoder_ff_logit_out_b``).  Conversion follows marian-conv
(src/tensors/cpu/expression_graph_packable.h:153-253): every float32 parameter whose name has
``_W`` two or three characters before its end becomes an ``intgemm8`` item; ``Wemb`` stays float.
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np


@dataclasses.dataclass
class TransformerConfig:
    dim_emb: int = 512
    dim_ffn: int = 2048
    heads: int = 8
    enc_depth: int = 6
    dec_depth: int = 6
    vocab: int = 32000
    decoder_autoreg: str = "self-attention"   # or "rnn" (SSRU cell), transformer-decoder-autoreg
    eos_id: int = 0                            # Marian's default vocabularies put </s> at 0, <unk> at 1
    unk_id: int = 1

    def to_yaml(self) -> str:
        """The ``special:model.yml`` item a converted model carries (src/tensors/cpu/expression_graph_packable.h:288-292)."""
        lines = [
            "type: transformer",
            f"dim-emb: {self.dim_emb}",
            f"dim-vocabs:\n  - {self.vocab}\n  - {self.vocab}",
            f"enc-depth: {self.enc_depth}",
            f"dec-depth: {self.dec_depth}",
            f"transformer-heads: {self.heads}",
            f"transformer-dim-ffn: {self.dim_ffn}",
            "transformer-ffn-activation: relu",
            "transformer-postprocess: dan",
            "transformer-postprocess-emb: d",
            "tied-embeddings-all: true",
            f"transformer-decoder-autoreg: {self.decoder_autoreg}",
        ]
        if self.decoder_autoreg == "rnn":
            lines.append("dec-cell: ssru")
        return "\n".join(lines) + "\n"

    @staticmethod
    def from_yaml(text: str) -> "TransformerConfig":
        kv = {}
        lines = text.splitlines()
        for i, ln in enumerate(lines):
            if ":" in ln and not ln.startswith(" "):
                k, v = ln.split(":", 1)
                kv[k.strip()] = v.strip()
            if ln.startswith("dim-vocabs"):
                kv["vocab"] = lines[i + 1].replace("-", "").strip()
        return TransformerConfig(dim_emb=int(kv["dim-emb"]), dim_ffn=int(kv["transformer-dim-ffn"]),
                                 heads=int(kv["transformer-heads"]), enc_depth=int(kv["enc-depth"]),
                                 dec_depth=int(kv["dec-depth"]), vocab=int(kv["vocab"]),
                                 decoder_autoreg=kv.get("transformer-decoder-autoreg", "self-attention"))


CONFIGS = {
    # the named workloads: transformer-base, transformer-big, the student with an SSRU decoder
    "base": TransformerConfig(512, 2048, 8, 6, 6, 32000),
    "big": TransformerConfig(1024, 4096, 16, 6, 6, 32000),
    "student": TransformerConfig(256, 1536, 8, 12, 2, 32000, decoder_autoreg="rnn"),
    "tiny": TransformerConfig(64, 128, 2, 2, 2, 512),
    "tiny-ssru": TransformerConfig(64, 128, 2, 2, 2, 512, decoder_autoreg="rnn"),
    # small models whose width is a multiple of 128 (the condition for multiplying Wk|Wv, Wq|Wk|Wv, W|Wf in one launch) and
    # whose heads are 64 wide and come in fours (the condition for the decoder attention that serves all beams per block)
    "small": TransformerConfig(256, 512, 4, 2, 2, 512),
    "small-ssru": TransformerConfig(256, 512, 4, 2, 2, 512, decoder_autoreg="rnn"),
}


def is_intgemm_param(name: str) -> bool:
    """marian-conv's name test: ``_W`` at length-3 or length-2 (expression_graph_packable.h:153-154)."""
    pos = name.find("_W")
    return pos != -1 and (pos == len(name) - 3 or pos == len(name) - 2)


def _glorot(rng, fan_in, fan_out):
    a = math.sqrt(6.0 / (fan_in + fan_out))
    return rng.uniform(-a, a, size=(fan_in, fan_out)).astype(np.float32)


def random_init(cfg: TransformerConfig, seed: int = 0) -> dict:
    """Random-init parameters: Glorot-uniform matrices, small N(0, 0.01) biases (so the bias path is
    exercised), unit LayerNorm scales, embeddings of roughly unit length."""
    rng = np.random.default_rng(seed)
    d, f, v = cfg.dim_emb, cfg.dim_ffn, cfg.vocab
    p: dict[str, np.ndarray] = {}

    def bias(n):
        return (rng.standard_normal((1, n)) * 0.01).astype(np.float32)

    def ln(prefix):
        p[prefix + "_ln_scale"] = np.ones((1, d), np.float32)
        p[prefix + "_ln_bias"] = np.zeros((1, d), np.float32)

    def attention(prefix):
        for w, b in (("Wq", "bq"), ("Wk", "bk"), ("Wv", "bv"), ("Wo", "bo")):
            p[f"{prefix}_{w}"] = _glorot(rng, d, d)
            p[f"{prefix}_{b}"] = bias(d)
        ln(prefix + "_Wo")

    def ffn(prefix):
        p[prefix + "_W1"] = _glorot(rng, d, f)
        p[prefix + "_b1"] = bias(f)
        p[prefix + "_W2"] = _glorot(rng, f, d)
        p[prefix + "_b2"] = bias(d)
        ln(prefix + "_ffn")

    p["Wemb"] = (rng.standard_normal((v, d)) / math.sqrt(d)).astype(np.float32)
    for i in range(1, cfg.enc_depth + 1):
        attention(f"encoder_l{i}_self")
        ffn(f"encoder_l{i}_ffn")
    for i in range(1, cfg.dec_depth + 1):
        if cfg.decoder_autoreg == "rnn":
            p[f"decoder_l{i}_rnn_W"] = _glorot(rng, d, d)
            p[f"decoder_l{i}_rnn_Wf"] = _glorot(rng, d, d)
            p[f"decoder_l{i}_rnn_bf"] = bias(d)
            ln(f"decoder_l{i}_rnn_ffn")
        else:
            attention(f"decoder_l{i}_self")
        attention(f"decoder_l{i}_context")
        ffn(f"decoder_l{i}_ffn")
    p["decoder_ff_logit_out_b"] = bias(v)
    return p


def synthetic_corpus(n_sentences: int, vocab: int, seed: int = 1, length_dist: str = "uniform", lo: int = 8, hi: int = 64,
                     mean: float = 30.0, std: float = 12.0, eos_id: int = 0):
    """Token IDs uniform over [4, vocab) and lengths either uniform over [lo, hi] or a clipped normal;
    EOS is appended to every sentence.  Returns a list of int32 arrays."""
    rng = np.random.default_rng(seed)
    if length_dist == "uniform":
        lens = rng.integers(lo, hi + 1, size=n_sentences)
    else:
        lens = np.clip(np.rint(rng.normal(mean, std, size=n_sentences)), lo, hi).astype(np.int64)
    out = []
    for n in lens:
        ids = rng.integers(4, vocab, size=int(n)).astype(np.int32)
        out.append(np.concatenate([ids, np.array([eos_id], np.int32)]))
    return out


def make_batches(corpus, mini_batch: int):
    """Maxi-batch style preparation: sort by length (longest first), cut into mini-batches of whole
    sentences, pad with EOS id and a 0/1 mask.  Returns [(sentence_ids, ids[B,S], mask[B,S])]."""
    order = sorted(range(len(corpus)), key=lambda i: -len(corpus[i]))
    batches = []
    for s in range(0, len(order), mini_batch):
        idx = order[s:s + mini_batch]
        width = max(len(corpus[i]) for i in idx)
        ids = np.zeros((len(idx), width), np.int32)
        mask = np.zeros((len(idx), width), np.float32)
        for r, i in enumerate(idx):
            n = len(corpus[i])
            ids[r, :n] = corpus[i]
            mask[r, :n] = 1.0
        batches.append((np.array(idx, np.int64), ids, mask))
    return batches


def sinusoidal_table(n: int, dim: int) -> np.ndarray:
    """Position table [n, dim] of gSinusoidalPositionEmbeddings (src/tensors/gpu/tensor_operators.cu:793-817):
    v = pos * exp(-(i mod dim/2) * ln(10000) / (dim/2 - 1)), sin for the first half, cos for the second.
    Computed once on the host in float32 so that every consumer sees the same bits."""
    half = dim // 2
    inc = np.float32(math.log(10000.0) / (half - 1.0))
    i = np.arange(dim)
    freq = np.exp((i % half).astype(np.float32) * -inc).astype(np.float32)
    pos = np.arange(n, dtype=np.float32)[:, None]
    v = (pos * freq[None, :]).astype(np.float32)
    return np.where(i[None, :] < half, np.sin(v), np.cos(v)).astype(np.float32)
