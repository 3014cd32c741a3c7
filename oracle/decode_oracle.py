"""CPU restatement of the int8 transformer decode: TEST INFRASTRUCTURE ONLY.

An independent NumPy implementation of what Marian does when it decodes an intgemm8 model on the CPU:
encoder and ``DecoderTransformer::step`` (src/models/transformer.h:581-637, 713-896), attention and
FFN blocks (:240-454), the SSRU cell (src/rnn/cells.h:983-1067) and ``BeamSearch::search`` with batch
purging (src/translator/beam_search.cpp:20-135, 224-245, 249-538; scoring in src/translator/history.h:27-35).
Every affine/dot goes through the C oracle (``oracle_i8.c``); nothing here touches the GPU engine.
It is written for clarity with explicit hypothesis objects, one sentence at a time where the reference
loops, so that it shares no code with the product's vectorised bookkeeping.

PARITY UNPINNED (see oracle_i8.c): there are no reference-held int8 decode outputs to compare with.
"""
from __future__ import annotations

import math

import numpy as np

from .oracle import COracle

NEG_MASK = np.float32(-99999999.0)


def _is_intgemm_param(name: str) -> bool:
    pos = name.find("_W")
    return pos != -1 and pos in (len(name) - 3, len(name) - 2)


def _positions(start, n, dim):
    half = dim // 2
    inc = np.float32(math.log(10000.0) / (half - 1.0))
    i = np.arange(dim)
    freq = np.exp((i % half).astype(np.float32) * -inc).astype(np.float32)
    pos = np.arange(start, start + n, dtype=np.float32)[:, None]
    v = (pos * freq[None, :]).astype(np.float32)
    return np.where(i[None, :] < half, np.sin(v), np.cos(v)).astype(np.float32)


def _layer_norm(x, scale, bias, eps=1e-6):
    mean = x.mean(axis=-1, keepdims=True, dtype=np.float32)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True, dtype=np.float32)
    return ((x - mean) / np.sqrt(var + np.float32(eps)) * scale.reshape(-1) + bias.reshape(-1)).astype(np.float32)


def _softmax(z):
    z = z - z.max(axis=-1, keepdims=True)
    e = np.exp(z, dtype=np.float32)
    return (e / e.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(np.float32)


def _log_softmax(z):
    m = z.max(axis=-1, keepdims=True)
    return (z - m - np.log(np.exp(z - m, dtype=np.float32).sum(axis=-1, keepdims=True, dtype=np.float32))).astype(np.float32)


class Hyp:
    __slots__ = ("prev", "word", "prev_state", "score")

    def __init__(self, prev=None, word=0, prev_state=0, score=0.0):
        self.prev, self.word, self.prev_state, self.score = prev, word, prev_state, score

    def words(self):
        out, h = [], self
        while h.prev is not None:
            out.append(h.word)
            h = h.prev
        return out[::-1]


class OracleTransformer:
    def __init__(self, cfg, params: dict, oracle: COracle | None = None, output_int8: bool = True, threads: int = 0):
        self.cfg = cfg
        self.o = oracle or COracle()
        if threads:
            self.o.set_threads(threads)
        self.w, self.p = {}, {}
        for name, val in params.items():
            val = np.ascontiguousarray(val, dtype=np.float32)
            if _is_intgemm_param(name):
                self.w[name] = self.o.prepare_b(val)          # (Bt int8 [N,K], quantMult)
            else:
                self.p[name] = val
        self.output_int8 = output_int8
        self.wemb = self.p["Wemb"]
        self.wemb_q = self.o.prepare_b(self.wemb, w_is_nk=True) if output_int8 else None
        self.d, self.h = cfg.dim_emb, cfg.heads
        self.dh = self.d // self.h

    def affine(self, x, wname, bname=None, relu=False):
        bt, qb = self.w[wname]
        bias = self.p[bname].reshape(-1) if bname else None
        return self.o.affine(x.reshape(-1, x.shape[-1]), bt, qb, bias, 1.0, relu)

    def ln(self, x, prefix):
        return _layer_norm(x, self.p[prefix + "_ln_scale"], self.p[prefix + "_ln_bias"])

    def heads(self, x, rows, steps):
        return x.reshape(rows, steps, self.h, self.dh).transpose(0, 2, 1, 3)

    def attention(self, q, k, v, log_mask):
        z = np.matmul(q, np.swapaxes(k, -1, -2)) * np.float32(1.0 / math.sqrt(self.dh))
        if log_mask is not None:
            z = z + log_mask
        return np.matmul(_softmax(z.astype(np.float32)), v).astype(np.float32)

    def ffn(self, x, prefix):
        h = self.affine(x, prefix + "_W1", prefix + "_b1", relu=True)
        out = self.affine(h, prefix + "_W2", prefix + "_b2")
        return self.ln(out.reshape(x.shape) + x, prefix + "_ffn")

    def encode(self, ids, mask):
        B, S = ids.shape
        x = (self.wemb[ids] * np.float32(math.sqrt(self.d)) + _positions(0, S, self.d)[None]).astype(np.float32)
        log_mask = ((1.0 - mask.astype(np.float32)) * NEG_MASK).reshape(B, 1, 1, S)
        for i in range(1, self.cfg.enc_depth + 1):
            pre = f"encoder_l{i}_self"
            q = self.heads(self.affine(x, pre + "_Wq", pre + "_bq"), B, S)
            k = self.heads(self.affine(x, pre + "_Wk", pre + "_bk"), B, S)
            v = self.heads(self.affine(x, pre + "_Wv", pre + "_bv"), B, S)
            a = self.attention(q, k, v, log_mask).transpose(0, 2, 1, 3).reshape(B * S, self.d)
            out = self.affine(a, pre + "_Wo", pre + "_bo")
            x = self.ln(out.reshape(B, S, self.d) + x, pre + "_Wo")
            x = self.ffn(x, f"encoder_l{i}_ffn")
        return x, log_mask

    def step(self, st, hyp_indices, prev_words, batch_indices, beam):
        cfg, t = self.cfg, st["pos"]
        if t > 0:
            if len(batch_indices) != st["ctx"].shape[0]:
                st["ctx"] = st["ctx"][batch_indices]
                st["mask"] = st["mask"][batch_indices]
            st["layer"] = [s[hyp_indices] for s in st["layer"]]
        B, S = st["ctx"].shape[:2]
        R = beam * B
        emb = np.zeros((R, self.d), np.float32) if t == 0 else self.wemb[prev_words]
        x = (emb * np.float32(math.sqrt(self.d)) + _positions(t, 1, self.d)).astype(np.float32)
        if st["cross_rows"] != B:
            st["ck"], st["cv"] = [], []
            for i in range(1, cfg.dec_depth + 1):
                pre = f"decoder_l{i}_context"
                st["ck"].append(self.heads(self.affine(st["ctx"], pre + "_Wk", pre + "_bk"), B, S))
                st["cv"].append(self.heads(self.affine(st["ctx"], pre + "_Wv", pre + "_bv"), B, S))
            st["cross_rows"] = B
        for i in range(1, cfg.dec_depth + 1):
            li = i - 1
            if cfg.decoder_autoreg == "rnn":
                pre = f"decoder_l{i}_rnn"
                xw = self.affine(x, pre + "_W")
                f = self.affine(x, pre + "_Wf", pre + "_bf")
                sig = (1.0 / (1.0 + np.exp(-f, dtype=np.float32))).astype(np.float32)
                cell = (st["layer"][li] * sig + xw * (1.0 - sig)).astype(np.float32)
                st["layer"][li] = cell
                x = self.ln(np.maximum(cell, 0) + x, pre + "_ffn")
            else:
                pre = f"decoder_l{i}_self"
                hist = x.reshape(R, 1, self.d) if st["layer"][li] is None else np.concatenate(
                    [st["layer"][li], x.reshape(R, 1, self.d)], axis=1)
                st["layer"][li] = hist
                steps = hist.shape[1]
                q = self.heads(self.affine(x, pre + "_Wq", pre + "_bq"), R, 1)
                k = self.heads(self.affine(hist, pre + "_Wk", pre + "_bk"), R, steps)
                v = self.heads(self.affine(hist, pre + "_Wv", pre + "_bv"), R, steps)
                a = self.attention(q, k, v, None).transpose(0, 2, 1, 3).reshape(R, self.d)
                x = self.ln(self.affine(a, pre + "_Wo", pre + "_bo") + x, pre + "_Wo")
            pre = f"decoder_l{i}_context"
            q = self.heads(self.affine(x, pre + "_Wq", pre + "_bq"), R, 1).reshape(beam, B, self.h, 1, self.dh)
            a = self.attention(q, st["ck"][li][None], st["cv"][li][None], st["mask"][None])
            a = a.transpose(0, 1, 3, 2, 4).reshape(R, self.d)
            x = self.ln(self.affine(a, pre + "_Wo", pre + "_bo") + x, pre + "_Wo")
            x = self.ffn(x, f"decoder_l{i}_ffn")
        st["pos"] = t + 1
        b = self.p["decoder_ff_logit_out_b"].reshape(-1)
        if self.output_int8:
            bt, qb = self.wemb_q
            return self.o.affine(x, bt, qb, b)
        return (x @ self.wemb.T + b).astype(np.float32)

    def start_state(self, ctx, mask):
        B = ctx.shape[0]
        layer = [np.zeros((B, self.d), np.float32) if self.cfg.decoder_autoreg == "rnn" else None
                 for _ in range(self.cfg.dec_depth)]
        return {"ctx": ctx, "mask": mask, "layer": layer, "cross_rows": -1, "pos": 0}


def beam_search(model: OracleTransformer, ids, mask, beam=4, max_length_factor=1.5, normalize=1.0, word_penalty=0.0):
    """Follows BeamSearch::search step by step with explicit beams of Hyp objects."""
    eos, V = model.cfg.eos_id, model.cfg.vocab
    B0, width = ids.shape
    ctx, log_mask = model.encode(ids.astype(np.int64), mask)
    st = model.start_state(ctx, log_mask)
    beams = [[Hyp() for _ in range(beam)] for _ in range(B0)]
    finals = [[] for _ in range(B0)]          # (normalised score, hyp)
    batch_map = list(range(B0))
    prev_map = list(batch_map)
    cur_dim = B0
    t = 0
    while True:
        max_beam = max(len(b) for b in beams)
        if max_beam == 0:
            break
        if t == 0:
            logits = model.step(st, None, None, None, 1)
            tensor_beam = 1
            active = list(range(B0))
            prev_scores = np.zeros((1, B0), np.float32)
        else:
            active = [o for o in range(B0) if beams[o]]
            batch_indices = np.array([prev_map[o] for o in active])
            hyp_idx, pw, ps = [], [], []
            for j in range(max_beam):
                for o in active:
                    if j < len(beams[o]):
                        h = beams[o][j]
                        hyp_idx.append(h.prev_state * cur_dim + prev_map[o])
                        pw.append(h.word)
                        ps.append(h.score)
                    else:
                        hyp_idx.append(0)
                        pw.append(eos)
                        ps.append(-np.inf)
            cur_dim = len(active)
            logits = model.step(st, np.array(hyp_idx), np.array(pw), batch_indices, max_beam)
            tensor_beam = max_beam
            prev_scores = np.array(ps, np.float32).reshape(max_beam, cur_dim)
        nb = len(active)
        logp = _log_softmax(logits).reshape(tensor_beam, nb, V)
        expanded = (prev_scores[:, :, None] + logp).transpose(1, 0, 2).reshape(nb, tensor_beam * V)
        n_best = max_beam
        new_beams = [[] for _ in range(B0)]
        for c, o in enumerate(active):
            row = expanded[c]
            keys = np.argpartition(-row, n_best)[:n_best] if row.size > n_best else np.arange(row.size)
            keys = keys[np.argsort(-row[keys], kind="stable")]
            for key in keys:
                if len(new_beams[o]) >= len(beams[o]):
                    break
                score = row[key]
                if score == -np.inf:
                    continue
                j, word = int(key) // V, int(key) % V
                new_beams[o].append(Hyp(beams[o][j], word, j, float(score)))
        prev_map = list(batch_map)
        # purge + history
        length = t + 1
        max_len_reached = length >= max_length_factor * width
        purged = [[h for h in new_beams[o] if h.word != eos] for o in range(B0)]
        for o in active:
            last = (not purged[o]) or max_len_reached
            for h in new_beams[o]:
                if h.word == eos or last:
                    finals[o].append(((h.score - word_penalty * length) / (length ** normalize), h))
        if max_len_reached:
            break
        beams = purged
        nxt = 0
        for o in range(B0):
            if beams[o]:
                batch_map[o] = nxt
                nxt += 1
        t += 1
    out = []
    for o in range(B0):
        if not finals[o]:
            out.append(([], float("-inf")))
            continue
        best = max(finals[o], key=lambda f: f[0])
        out.append((best[1].words(), float(best[0])))
    return out
