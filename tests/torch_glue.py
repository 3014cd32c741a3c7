"""A second implementation of the decode with torch ops as glue: TEST INFRASTRUCTURE ONLY.

The product decodes through the C++ step driver (marian_dev_b200.decoder.NativeStepper).  This module restates the
encoder and ``DecoderTransformer::step`` (src/models/transformer.h:581-637, 713-896; ``MultiHead`` / ``LayerAttention`` /
``LayerFFN`` :279-454; the SSRU cell src/rnn/cells.h:983-1067) with torch for attention, softmax and LayerNorm and
``ops.prepareA`` + ``ops.multiply`` for every affine, so that the driver can be cross-checked against an independent
sequencing of the same int8 kernels.  Its float glue rounds differently from the driver's fixed-order kernels, so
random-init models occasionally pick another word; the tests hold it to a looser bar.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

from marian_dev_b200 import ops
from marian_dev_b200.decoder import NEG_MASK, BeamSearch, Int8Transformer


def sinusoidal_positions(start: int, n: int, dim: int, device) -> torch.Tensor:
    """gSinusoidalPositionEmbeddings (src/tensors/gpu/tensor_operators.cu:793-817)."""
    half = dim // 2
    inc = math.log(10000.0) / (half - 1.0)
    i = torch.arange(dim, device=device)
    freq = torch.exp((i % half).float() * -inc)
    pos = torch.arange(start, start + n, device=device, dtype=torch.float32)[:, None]
    v = pos * freq[None, :]
    return torch.where(i[None, :] < half, torch.sin(v), torch.cos(v))


class DecoderState:
    def __init__(self):
        self.layer = []          # per layer: self-attention history [R, t, d] or SSRU cell [R, d]
        self.cross_k = []        # per layer [B, h, S, dh]
        self.cross_v = []
        self.cross_rows = -1     # batch size the cross K/V were computed for
        self.context = None      # [B, S, d]
        self.log_mask = None     # [B, 1, 1, S]
        self.position = 0


class TorchGlueTransformer(Int8Transformer):
    """Int8Transformer (the weights) plus a forward pass sequenced from Python."""

    # ------------------------------------------------------------------ building blocks
    def quant(self, x: torch.Tensor) -> ops.IntgemmTensor:
        return ops.prepareA(x.reshape(-1, x.shape[-1]), ws=self.ws)

    def mul(self, aq, wname, bname=None, relu=False):
        bias = self.p[bname].view(-1) if bname else None
        return ops.multiply(aq, self.w[wname], bias, 1.0, relu, ws=self.ws)

    def layer_norm(self, x, prefix):
        return F.layer_norm(x, (self.d,), self.p[prefix + "_ln_scale"].view(-1), self.p[prefix + "_ln_bias"].view(-1), 1e-6)

    def split_heads(self, x, rows, steps):
        return x.view(rows, steps, self.h, self.dh).permute(0, 2, 1, 3)      # [rows, h, steps, dh]

    def attention(self, q, k, v, log_mask):
        """softmax(q k^T / sqrt(dh) + mask) v, all fp32 (transformer.h:240-277)."""
        z = torch.matmul(q, k.transpose(-1, -2)) * (1.0 / math.sqrt(self.dh))
        if log_mask is not None:
            z = z + log_mask
        return torch.matmul(torch.softmax(z, dim=-1), v)

    def ffn(self, x, prefix):
        """LayerFFN with relu: W1 + ReLU fused in the GEMM write-back, W2, then add & norm."""
        hq = self.quant(self.mul(self.quant(x), prefix + "_W1", prefix + "_b1", relu=True))
        out = self.mul(hq, prefix + "_W2", prefix + "_b2")
        return self.layer_norm(out.view_as(x) + x, prefix + "_ffn")

    # ------------------------------------------------------------------ encoder
    def encode(self, ids: torch.Tensor, mask: torch.Tensor):
        """ids [B,S] int64, mask [B,S] float 0/1 -> context [B,S,d], log_mask [B,1,1,S]."""
        B, S = ids.shape
        x = self.wemb[ids] * math.sqrt(self.d) + sinusoidal_positions(0, S, self.d, self.device)[None]
        log_mask = ((1.0 - mask) * NEG_MASK).view(B, 1, 1, S)
        for i in range(1, self.cfg.enc_depth + 1):
            pre = f"encoder_l{i}_self"
            xq = self.quant(x)  # q, keys and values are the same tensor: one quantisation serves all three
            q = self.split_heads(self.mul(xq, pre + "_Wq", pre + "_bq"), B, S)
            k = self.split_heads(self.mul(xq, pre + "_Wk", pre + "_bk"), B, S)
            v = self.split_heads(self.mul(xq, pre + "_Wv", pre + "_bv"), B, S)
            a = self.attention(q, k, v, log_mask).permute(0, 2, 1, 3).reshape(B * S, self.d)
            out = self.mul(self.quant(a), pre + "_Wo", pre + "_bo")
            x = self.layer_norm(out.view(B, S, self.d) + x, pre + "_Wo")
            x = self.ffn(x, f"encoder_l{i}_ffn")
        return x, log_mask

    def start_state(self, context, log_mask) -> DecoderState:
        st = DecoderState()
        st.context, st.log_mask = context, log_mask
        B = context.shape[0]
        for _ in range(self.cfg.dec_depth):
            if self.cfg.decoder_autoreg == "rnn":
                st.layer.append(torch.zeros(B, self.d, device=self.device))
            else:
                st.layer.append(None)
        return st

    # ------------------------------------------------------------------ one decoder step
    def step(self, st: DecoderState, hyp_indices, prev_words, batch_indices, beam: int) -> torch.Tensor:
        """Returns logits [beam * batch, V] (beam-major rows) and advances the state in place.

        hyp_indices / prev_words are None at t = 0 (one start hypothesis per sentence, zero embedding);
        batch_indices selects the sentences still active out of the previous step's batch."""
        t = st.position
        cfg = self.cfg
        if t > 0:
            if len(batch_indices) != st.context.shape[0]:
                st.context = st.context.index_select(0, batch_indices)
                st.log_mask = st.log_mask.index_select(0, batch_indices)
            st.layer = [s.index_select(0, hyp_indices) for s in st.layer]
        B, S = st.context.shape[0], st.context.shape[1]
        R = beam * B
        if t == 0:
            emb = torch.zeros(R, self.d, device=self.device)
        else:
            emb = self.wemb[prev_words]
        x = emb * math.sqrt(self.d) + sinusoidal_positions(t, 1, self.d, self.device)

        # cross-attention keys/values are cached per batch and recomputed when the batch shrinks
        if st.cross_rows != B:
            st.cross_k, st.cross_v = [], []
            cq = self.quant(st.context)
            for i in range(1, cfg.dec_depth + 1):
                pre = f"decoder_l{i}_context"
                st.cross_k.append(self.split_heads(self.mul(cq, pre + "_Wk", pre + "_bk"), B, S))
                st.cross_v.append(self.split_heads(self.mul(cq, pre + "_Wv", pre + "_bv"), B, S))
            st.cross_rows = B

        for i in range(1, cfg.dec_depth + 1):
            li = i - 1
            if cfg.decoder_autoreg == "rnn":
                pre = f"decoder_l{i}_rnn"
                xq = self.quant(x)
                xw = self.mul(xq, pre + "_W")                       # dot(input, W)
                f = self.mul(xq, pre + "_Wf", pre + "_bf")          # affine(input, Wf, bf)
                sig = torch.sigmoid(f)
                cell = st.layer[li] * sig + xw * (1.0 - sig)        # highway(cell, x, f)
                st.layer[li] = cell
                x = self.layer_norm(torch.relu(cell) + x, pre + "_ffn")
            else:
                pre = f"decoder_l{i}_self"
                hist = x.view(R, 1, self.d) if st.layer[li] is None else torch.cat([st.layer[li], x.view(R, 1, self.d)], dim=1)
                st.layer[li] = hist
                steps = hist.shape[1]
                q = self.split_heads(self.mul(self.quant(x), pre + "_Wq", pre + "_bq"), R, 1)
                # keys and values are re-projected from the whole history every step, with one
                # quantisation multiplier over all of it (transformer.h:401-417)
                hq = self.quant(hist)
                k = self.split_heads(self.mul(hq, pre + "_Wk", pre + "_bk"), R, steps)
                v = self.split_heads(self.mul(hq, pre + "_Wv", pre + "_bv"), R, steps)
                a = self.attention(q, k, v, None).permute(0, 2, 1, 3).reshape(R, self.d)
                out = self.mul(self.quant(a), pre + "_Wo", pre + "_bo")
                x = self.layer_norm(out + x, pre + "_Wo")

            pre = f"decoder_l{i}_context"
            q = self.split_heads(self.mul(self.quant(x), pre + "_Wq", pre + "_bq"), R, 1)   # [R, h, 1, dh]
            q = q.reshape(beam, B, self.h, 1, self.dh)
            a = self.attention(q, st.cross_k[li][None], st.cross_v[li][None], st.log_mask[None])
            a = a.permute(0, 1, 3, 2, 4).reshape(R, self.d)
            out = self.mul(self.quant(a), pre + "_Wo", pre + "_bo")
            x = self.layer_norm(out + x, pre + "_Wo")
            x = self.ffn(x, f"decoder_l{i}_ffn")

        st.position = t + 1
        out_b = self.p["decoder_ff_logit_out_b"].view(-1)
        if self.output_int8:
            return ops.multiply(self.quant(x), self.wemb_q, out_b, ws=self.ws)
        return torch.addmm(out_b, x, self.wemb.t())


class TorchGlueSearch(BeamSearch):
    """BeamSearch whose step runs through TorchGlueTransformer instead of the C++ driver."""

    def _begin(self, ids_t, mask_t):
        ctx, log_mask = self.m.encode(ids_t, mask_t)
        return self.m.start_state(ctx, log_mask)

    def _nbest(self, st, hyp_idx, pw, batch_indices, ps, tensor_beam, nb, n_best):
        return self._nbest_torch(st, hyp_idx, pw, batch_indices, ps, tensor_beam, nb, n_best)

    def _nbest_torch(self, st, hyp_idx, pw, batch_indices, ps, tensor_beam, nb, n_best):
        """One step through the torch-glue model, then n-best over beam x vocabulary per sentence:
        row-wise top-N of the logits, shifted by the row's log-sum-exp and previous path score, merged
        across the rows of a sentence (the same set as top-N over the flattened [beam * V] scores)."""
        m, dev = self.m, self.m.device
        if hyp_idx is None:
            logits = m.step(st, None, None, None, 1)
            prev_scores_t = torch.zeros(nb, device=dev)
        else:
            R = tensor_beam * nb
            host = torch.from_numpy(np.concatenate([hyp_idx, pw, batch_indices]).astype(np.int64)).to(dev)
            prev_scores_t = torch.from_numpy(ps).to(dev)
            self.h2d_bytes += host.numel() * 8 + ps.size * 4
            logits = m.step(st, host[:R], host[R:2 * R], host[2 * R:], tensor_beam)
        lse = torch.logsumexp(logits, dim=-1)
        top_v, top_i = torch.topk(logits, n_best, dim=-1)                              # [R, n_best]
        cand = (top_v - lse[:, None]) + prev_scores_t[:, None]
        cand = cand.view(tensor_beam, nb, n_best).permute(1, 0, 2).reshape(nb, tensor_beam * n_best)
        best_v, best_c = torch.topk(cand, n_best, dim=-1)                              # sorted, descending
        word_sel = top_i.view(tensor_beam, nb, n_best).permute(1, 0, 2).reshape(nb, -1).gather(1, best_c)
        out = torch.stack([best_v.double(), (best_c // n_best).double(), word_sel.double()]).cpu().numpy()  # the step's one sync
        self.d2h_bytes += out.size * 8
        return out[0].astype(np.float32), out[1].astype(np.int64), out[2].astype(np.int64)
