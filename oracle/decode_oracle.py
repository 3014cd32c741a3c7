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
    """All float glue (embedding, LayerNorm, attention, SSRU cell, log-softmax/top-k) runs through the
    fixed-order C functions of oracle_i8.c; all affines through its int8 path."""

    def __init__(self, cfg, params: dict, oracle: COracle | None = None, output_int8: bool = True, threads: int = 0,
                 scheme: str = "intgemm8", packed_items: dict | None = None):
        """scheme "packed8avx512": every affine goes through the restatement of the reference's mjdgemm route
        (oracle_packed8.c: per-row uint8 activations, per-column int8 weights) instead of the intgemm8 one; packed_items
        optionally supplies ready items (name -> Packed8Item, "Wemb_packed8" for the tied output matrix) so that a test can
        hand both sides the same bytes."""
        self.cfg = cfg
        self.o = oracle or COracle()
        self.scheme = scheme
        self.p8 = None
        if scheme == "packed8avx512":
            from .oracle import Packed8Oracle
            self.p8 = Packed8Oracle()
        if threads:
            self.o.set_threads(threads)
        self.w, self.p = {}, {}
        for name, val in params.items():
            val = np.ascontiguousarray(val, dtype=np.float32)
            if _is_intgemm_param(name):
                if self.p8 is not None:
                    self.w[name] = (packed_items or {}).get(name) or self.p8.prepare_b(val)
                else:
                    self.w[name] = self.o.prepare_b(val)          # (Bt int8 [N,K], quantMult)
            else:
                self.p[name] = val
        self.output_int8 = output_int8
        self.wemb = self.p["Wemb"]
        if not output_int8:
            self.wemb_q = None
        elif self.p8 is not None:
            self.wemb_q = (packed_items or {}).get("Wemb_packed8") or self.p8.prepare_b(np.ascontiguousarray(self.wemb.T))
        else:
            self.wemb_q = self.o.prepare_b(self.wemb, w_is_nk=True)
        self.d, self.h = cfg.dim_emb, cfg.heads
        self.dh = self.d // self.h
        self.pos = _positions(0, 512, self.d)
        self.scale = float(np.sqrt(np.float32(self.d)))

    def affine(self, x, wname, bname=None, relu=False):
        bias = self.p[bname].reshape(-1) if bname else None
        if self.p8 is not None:
            return self.p8.affine(np.ascontiguousarray(x.reshape(-1, x.shape[-1]), dtype=np.float32), self.w[wname], bias, relu)
        bt, qb = self.w[wname]
        return self.o.affine(x.reshape(-1, x.shape[-1]), bt, qb, bias, 1.0, relu)

    def add_ln(self, a, resid, prefix):
        return self.o.add_layernorm(a, resid, self.p[prefix + "_ln_scale"], self.p[prefix + "_ln_bias"], 1e-6)

    def ffn(self, x, prefix):
        h = self.affine(x, prefix + "_W1", prefix + "_b1", relu=True)
        out = self.affine(h, prefix + "_W2", prefix + "_b2")
        return self.add_ln(out, x, prefix + "_ffn")

    def encode(self, ids, mask):
        B, S = ids.shape
        M = B * S
        x = self.o.embed(self.wemb, ids.reshape(-1), self.pos, S, self.scale, M)
        log_mask = ((np.float32(1.0) - mask.astype(np.float32)) * NEG_MASK).astype(np.float32)      # [B, S]
        for i in range(1, self.cfg.enc_depth + 1):
            pre = f"encoder_l{i}_self"
            q = self.affine(x, pre + "_Wq", pre + "_bq")
            k = self.affine(x, pre + "_Wk", pre + "_bk")
            v = self.affine(x, pre + "_Wv", pre + "_bv")
            a = self.o.attention1(q, k, v, log_mask, M, self.h, self.dh, S, B, 2)
            x = self.add_ln(self.affine(a, pre + "_Wo", pre + "_bo"), x, pre + "_Wo")
            x = self.ffn(x, f"encoder_l{i}_ffn")
        return x.reshape(B, S, self.d), log_mask

    def start_state(self, ctx, mask):
        B = ctx.shape[0]
        layer = [np.zeros((B, self.d), np.float32) if self.cfg.decoder_autoreg == "rnn" else None
                 for _ in range(self.cfg.dec_depth)]
        return {"ctx": ctx, "mask": mask, "layer": layer, "cross_rows": -1, "pos": 0}

    def step(self, st, hyp_indices, prev_words, batch_indices, beam):
        """Returns the logits [beam*batch, V] of one decoder step (rows beam-major)."""
        cfg, t = self.cfg, st["pos"]
        if t > 0:
            if len(batch_indices) != st["ctx"].shape[0]:
                st["ctx"] = st["ctx"][batch_indices]
                st["mask"] = st["mask"][batch_indices]
            if cfg.decoder_autoreg == "rnn":
                st["layer"] = [s[hyp_indices] for s in st["layer"]]
            else:
                st["layer"] = [s[:, hyp_indices] for s in st["layer"]]           # history is time-major [T, R, d]
        B, S = st["ctx"].shape[:2]
        R = beam * B
        x = self.o.embed(self.wemb, None if t == 0 else prev_words, self.pos[t:t + 1], 0, self.scale, R)
        if st["cross_rows"] != B:
            st["ck"], st["cv"] = [], []
            for i in range(1, cfg.dec_depth + 1):
                pre = f"decoder_l{i}_context"
                st["ck"].append(self.affine(st["ctx"], pre + "_Wk", pre + "_bk"))      # [B*S, d]
                st["cv"].append(self.affine(st["ctx"], pre + "_Wv", pre + "_bv"))
            st["cross_rows"] = B
        for i in range(1, cfg.dec_depth + 1):
            li = i - 1
            if cfg.decoder_autoreg == "rnn":
                pre = f"decoder_l{i}_rnn"
                xw = self.affine(x, pre + "_W")
                f = self.affine(x, pre + "_Wf", pre + "_bf")
                cell, h = self.o.ssru_cell(st["layer"][li], xw, f)
                st["layer"][li] = cell
                x = self.add_ln(h, x, pre + "_ffn")
            else:
                pre = f"decoder_l{i}_self"
                hist = x[None] if st["layer"][li] is None else np.concatenate([st["layer"][li], x[None]], axis=0)
                st["layer"][li] = hist
                steps = hist.shape[0]
                q = self.affine(x, pre + "_Wq", pre + "_bq")
                k = self.affine(hist, pre + "_Wk", pre + "_bk")                          # one multiplier over the history
                v = self.affine(hist, pre + "_Wv", pre + "_bv")
                a = self.o.attention1(q, k, v, None, R, self.h, self.dh, steps, B, 0)
                x = self.add_ln(self.affine(a, pre + "_Wo", pre + "_bo"), x, pre + "_Wo")
            pre = f"decoder_l{i}_context"
            q = self.affine(x, pre + "_Wq", pre + "_bq")
            a = self.o.attention1(q, st["ck"][li], st["cv"][li], st["mask"], R, self.h, self.dh, S, B, 1)
            x = self.add_ln(self.affine(a, pre + "_Wo", pre + "_bo"), x, pre + "_Wo")
            x = self.ffn(x, f"decoder_l{i}_ffn")
        st["pos"] = t + 1
        b = self.p["decoder_ff_logit_out_b"].reshape(-1)
        if self.output_int8 and self.p8 is not None:
            return self.p8.affine(np.ascontiguousarray(x, dtype=np.float32), self.wemb_q, b)
        if self.output_int8:
            bt, qb = self.wemb_q
            return self.o.affine(x, bt, qb, b)
        return (x @ self.wemb.T + b).astype(np.float32)


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
        n_best = max_beam
        # log-softmax and top-N per row in the fixed order, then the N best of beam x N candidates per
        # sentence; ties go to the smaller flattened (beam, word) key
        cs, cw = model.o.lse_topk(logits, n_best, prev_scores.reshape(-1))
        cs = cs.reshape(tensor_beam, nb, n_best)
        cw = cw.reshape(tensor_beam, nb, n_best)
        new_beams = [[] for _ in range(B0)]
        for c, o in enumerate(active):
            cands = []
            for j in range(tensor_beam):
                for r in range(n_best):
                    if cs[j, c, r] != -np.inf:
                        cands.append((-float(cs[j, c, r]), j * V + int(cw[j, c, r]), float(cs[j, c, r])))
            cands.sort(key=lambda e: (e[0], e[1]))
            for _neg, key, score in cands[:n_best]:
                if len(new_beams[o]) >= len(beams[o]):
                    break
                j, word = key // V, key % V
                new_beams[o].append(Hyp(beams[o][j], word, j, score))
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
