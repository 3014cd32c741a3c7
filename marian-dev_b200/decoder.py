"""Transformer / SSRU decode on the GPU with every affine running through the int8 engine.

This is the caller that drives the hot path for the tokens/sec metric; it restates
``DecoderTransformer::step`` (src/models/transformer.h:713-896), the encoder (:581-637),
``MultiHead`` / ``LayerAttention`` / ``LayerFFN`` (:279-454), the SSRU cell (src/rnn/cells.h:983-1067)
and ``BeamSearch::search`` (src/translator/beam_search.cpp:249-538).  Attention, softmax, LayerNorm
and the beam bookkeeping stay fp32 (torch ops and host code); all weight multiplications go through
``ops.prepareA`` + ``ops.multiply`` (libmarian_i8.so).

Row layout follows Marian: decoder tensors are ``[beam, batch, ...]`` flattened beam-major, so a
hypothesis lives in row ``beamHypIdx * batch + batchIdx`` (beam_search.cpp:398).
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

from . import ops
from .model import TransformerConfig, is_intgemm_param, sinusoidal_table

NEG_MASK = -99999999.0  # transposedLogMask (transformer.h:138-143)


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


class Int8Transformer:
    """Model replica on one GPU: converted (intgemm8) weights, fp32 biases / LayerNorm / embeddings."""

    def __init__(self, cfg: TransformerConfig, params: dict, device, output_int8: bool = True, ws=None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.ws = ws or ops.default_workspace(self.device)
        self.output_int8 = output_int8
        self.w = {}   # name -> IntgemmTensor
        self.p = {}   # name -> fp32 tensor
        for name, val in params.items():
            if isinstance(val, ops.IntgemmTensor):
                self.w[name] = val
            else:
                t = torch.as_tensor(np.ascontiguousarray(val), dtype=torch.float32).to(self.device)
                if is_intgemm_param(name):
                    self.w[name] = ops.prepareB(t, ws=self.ws)   # on-line conversion of a float model
                else:
                    self.p[name] = t
        self.wemb = self.p["Wemb"]                                 # [V, d] fp32, for the lookup
        # Tied output layer: affine(x, Wemb, b, transB=true).  The reference leaves Wemb in fp32
        # (its name test skips it); the int8 mode quantises the [V,d] matrix, which already is the
        # K-major Bt[N,K] layout.
        self.wemb_q = ops.prepareB(self.wemb, w_is_nk=True, ws=self.ws) if output_int8 else None
        self.d = cfg.dim_emb
        self.h = cfg.heads
        self.dh = cfg.dim_emb // cfg.heads

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


class NativeStepper:
    """The decoder time step as ONE call into the C++ driver (include/marian_i8_decode.h): all glue
    kernels and affines of a step are launched from native code, the caller only exchanges the small
    per-step index / n-best arrays.  Device memory (arena, outputs) is allocated here, once."""

    def __init__(self, model: "Int8Transformer", max_batch: int = 128, beam: int = 4, max_src: int = 136, max_steps: int = 208):
        import ctypes
        from .binding import Mi8dConfig, check, lib
        if not model.output_int8:
            raise ops.Mi8Error(3, "the native step driver runs the tied output layer in int8")
        self.m, self.L, self.check = model, lib(), check
        cfg = model.cfg
        max_steps = max(max_steps, max_src)        # the position table also serves the encoder
        self.cfg = Mi8dConfig(cfg.dim_emb, cfg.dim_ffn, cfg.heads, cfg.enc_depth, cfg.dec_depth, cfg.vocab,
                              int(cfg.decoder_autoreg == "rnn"), max_batch * beam, max_batch, max_steps, max_src)
        dev = model.device
        nbytes = int(self.L.mi8d_arena_bytes(ctypes.byref(self.cfg)))
        self.arena = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        handle = ctypes.c_void_p()
        check(self.L.mi8d_create(ctypes.byref(self.cfg), self.arena.data_ptr(), nbytes, model.ws.ptr, model.ws.nbytes,
                                 ctypes.byref(handle)))
        self.h = handle
        for name, w in model.w.items():
            check(self.L.mi8d_set_weight(self.h, name.encode(), w.data.data_ptr(), w.cols, w.rows))
        check(self.L.mi8d_set_weight(self.h, b"Wemb_intgemm8", model.wemb_q.data.data_ptr(), model.wemb_q.cols, model.wemb_q.rows))
        for name, p in model.p.items():
            check(self.L.mi8d_set_param(self.h, name.encode(), p.data_ptr()))
        self.pos = torch.from_numpy(sinusoidal_table(max_steps, cfg.dim_emb)).to(dev)
        check(self.L.mi8d_set_positions(self.h, self.pos.data_ptr()))
        self.max_batch, self.max_steps, self.max_src = max_batch, max_steps, max_src
        self.out = torch.empty(3, max_batch * 8, dtype=torch.int32, device=dev)       # score bits, beam, word
        self.host_out = torch.empty(3, max_batch * 8, dtype=torch.int32).pin_memory()
        self.ctrl = torch.empty(3 * max_batch * beam + max_batch, dtype=torch.int32, device=dev)
        self.host_ctrl = torch.empty(3 * max_batch * beam + max_batch, dtype=torch.int32).pin_memory()

    def __del__(self):
        try:
            self.L.mi8d_destroy(self.h)
        except Exception:
            pass

    def encode(self, ids_t: torch.Tensor, mask_t: torch.Tensor):
        """Encoder forward on the device (ids int64/int32 [B,S], mask float [B,S]) and start of the mini-batch."""
        B, S = ids_t.shape
        if B > self.max_batch or S > self.max_src:
            raise ops.Mi8Error(3, f"mini-batch {B}x{S} exceeds the driver's limits {self.max_batch}x{self.max_src}")
        ids32 = ids_t.to(torch.int32).contiguous()
        log_mask = ((1.0 - mask_t) * NEG_MASK).contiguous()     # exactly 0 or -99999999
        self.check(self.L.mi8d_encode(self.h, ids32.data_ptr(), log_mask.data_ptr(), B, S, torch.cuda.current_stream().cuda_stream))

    def search(self, ids_t: torch.Tensor, mask_t: torch.Tensor, beam: int, max_length_factor: float, normalize: float,
               word_penalty: float = 0.0, eos_id: int = 0):
        """mi8d_search: the whole beam search of one mini-batch (encoder, decoder steps, bookkeeping, traceback) in the
        C++ driver.  Returns [(tokens, score)] per sentence and the bytes moved host <-> device by the step loop."""
        import ctypes
        from .binding import Mi8dSearchConfig
        B, S = ids_t.shape
        if B > self.max_batch or S > self.max_src:
            raise ops.Mi8Error(3, f"mini-batch {B}x{S} exceeds the driver's limits {self.max_batch}x{self.max_src}")
        ids32 = ids_t.to(torch.int32).contiguous()
        log_mask = ((1.0 - mask_t) * NEG_MASK).contiguous()
        max_out = int(math.ceil(max_length_factor * S)) + 2
        toks = np.empty((B, max_out), np.int32)
        lens = np.empty(B, np.int32)
        scores = np.empty(B, np.float32)
        up, down = ctypes.c_ulonglong(0), ctypes.c_ulonglong(0)
        cfg = Mi8dSearchConfig(int(beam), float(max_length_factor), float(normalize), float(word_penalty), int(eos_id))
        self.check(self.L.mi8d_search(self.h, ids32.data_ptr(), log_mask.data_ptr(), B, S, ctypes.byref(cfg), toks.ctypes.data, max_out,
                                      lens.ctypes.data, scores.ctypes.data, ctypes.byref(up), ctypes.byref(down),
                                      torch.cuda.current_stream().cuda_stream))
        res = [(toks[b, :lens[b]].tolist(), float(scores[b])) for b in range(B)]
        return res, int(up.value), int(down.value)

    def history_reuse(self, reset: bool = False):
        """(reused, total) counts of (layer, step) pairs whose stored self-attention keys/values stayed valid."""
        import ctypes
        out = (ctypes.c_uint * 2)()
        self.check(self.L.mi8d_history_reuse(self.h, ctypes.byref(out), int(reset)))
        return int(out[0]), int(out[1])

    def start(self, ctx: torch.Tensor, log_mask: torch.Tensor):
        B, S = ctx.shape[0], ctx.shape[1]
        if B > self.max_batch or S > self.max_src:
            raise ops.Mi8Error(3, f"mini-batch {B}x{S} exceeds the driver's limits {self.max_batch}x{self.max_src}")
        self.check(self.L.mi8d_start(self.h, ctx.contiguous().data_ptr(), log_mask.contiguous().data_ptr(), B, S,
                                     torch.cuda.current_stream().cuda_stream))

    def step(self, hyp_idx, prev_words, batch_idx, prev_scores, beam: int, batch: int, n_best: int):
        """hyp_idx / prev_words / prev_scores: NumPy arrays of beam*batch entries (None at the first
        step); batch_idx: NumPy array of `batch` entries.  Returns NumPy (score, beam, word) [batch, n_best]."""
        stream = torch.cuda.current_stream().cuda_stream
        R = beam * batch
        if hyp_idx is None:
            ptrs = (None, None, None, None)
            up = 0
        else:
            hc = self.host_ctrl.numpy()
            hc[0:R] = hyp_idx
            hc[R:2 * R] = prev_words
            hc[2 * R:3 * R] = prev_scores.astype(np.float32).view(np.int32)
            hc[3 * R:3 * R + batch] = batch_idx
            up = 3 * R + batch
            self.ctrl[:up].copy_(self.host_ctrl[:up], non_blocking=True)
            base = self.ctrl.data_ptr()
            ptrs = (base, base + 4 * R, base + 12 * R, base + 8 * R)
        n = batch * n_best
        o = self.out
        self.check(self.L.mi8d_step(self.h, ptrs[0], ptrs[1], ptrs[2], ptrs[3], beam, batch, n_best,
                                    o[0].data_ptr(), o[1].data_ptr(), o[2].data_ptr(), stream))
        self.host_out[:, :n].copy_(o[:, :n], non_blocking=True)
        torch.cuda.current_stream().synchronize()                       # the step's one host sync
        ho = self.host_out.numpy()
        nv = ho[0, :n].view(np.float32).reshape(batch, n_best).copy()
        return nv, ho[1, :n].astype(np.int64).reshape(batch, n_best), ho[2, :n].astype(np.int64).reshape(batch, n_best), up * 4, 3 * n * 4


class BeamSearch:
    """Host-side bookkeeping of BeamSearch::search with batch purging (beam_search.cpp:249-538)."""

    def __init__(self, model: Int8Transformer, beam: int = 4, max_length_factor: float = 1.5, normalize: float = 1.0,
                 word_penalty: float = 0.0, native: "NativeStepper | None" = None, native_search: bool = True):
        self.m = model
        self.native = native      # None: torch glue ops per step; else the C++ step driver
        self.native_search = native_search   # with a native stepper: also run the bookkeeping in the C++ driver (mi8d_search)
        self.beam = beam
        self.factor = max_length_factor
        self.alpha = normalize
        self.wp = word_penalty
        self.h2d_bytes = 0    # bytes copied host -> device / device -> host by search(), for the benchmark
        self.d2h_bytes = 0

    def search(self, ids, mask):
        """ids/mask [B,S] on the HOST (NumPy arrays or, for asynchronous copies, pinned torch tensors).
        Returns per sentence (best token list incl. EOS, normalised score)."""
        dev = self.m.device
        if isinstance(ids, np.ndarray):
            ids = torch.from_numpy(ids.astype(np.int64))
            mask = torch.from_numpy(np.asarray(mask, dtype=np.float32))
        ids_t = ids.to(dev, non_blocking=True)
        mask_t = mask.to(dev, non_blocking=True)
        self.h2d_bytes += ids.numel() * ids.element_size() + mask.numel() * mask.element_size()
        return self.search_device(ids_t, mask_t)

    @torch.no_grad()
    def search_device(self, ids_t: torch.Tensor, mask_t: torch.Tensor):
        """Same with ids (int64) and mask (float32) already on the device."""
        if self.native is not None and self.native_search:
            res, up, down = self.native.search(ids_t, mask_t, self.beam, self.factor, self.alpha, self.wp, self.m.cfg.eos_id)
            self.h2d_bytes += up
            self.d2h_bytes += down
            return res
        m, dev, eos = self.m, self.m.device, self.m.cfg.eos_id
        B0, width = ids_t.shape
        if self.native is not None:
            self.native.encode(ids_t, mask_t)
            st = None
        else:
            ctx, log_mask = m.encode(ids_t, mask_t)
            st = m.start_state(ctx, log_mask)

        beam = self.beam
        col = np.arange(beam)[None, :]
        W = np.full(B0, beam, np.int64)                 # surviving hypotheses per original sentence
        words = np.zeros((B0, beam), np.int64)          # purged beam of the previous step
        scores = np.zeros((B0, beam), np.float32)
        prev_state = np.zeros((B0, beam), np.int64)     # beam row of the parent in the previous step's tensors
        step_map = np.arange(B0)                        # original sentence -> batch index in the previous step's tensors
        prev_dim = B0                                   # batch size of the previous step's tensors
        history = []                                    # per step: (words, parent beam row, purged->unpurged position)
        finals = [[] for _ in range(B0)]                # (normalised score, step, unpurged position)

        t = 0
        while True:
            max_beam = int(W.max())
            if max_beam == 0:
                break
            active = np.nonzero(W > 0)[0]
            nb = len(active)
            n_best = max_beam
            if t == 0:
                tensor_beam, hyp_idx, pw, ps, batch_indices = 1, None, None, None, None
            else:
                tensor_beam = max_beam
                batch_indices = step_map[active]
                valid = np.arange(max_beam)[:, None] < W[active][None, :]                  # [max_beam, nb]
                hyp_idx = np.where(valid, prev_state[active].T[:max_beam] * prev_dim + batch_indices[None, :], 0).reshape(-1)
                pw = np.where(valid, words[active].T[:max_beam], eos).reshape(-1)           # dummy slots carry EOS
                ps = np.where(valid, scores[active].T[:max_beam], -np.inf).astype(np.float32).reshape(-1)
            if self.native is not None:
                nv, nbm, nw, up, down = self.native.step(hyp_idx, pw, batch_indices, ps, tensor_beam, nb, n_best)
                self.h2d_bytes += up
                self.d2h_bytes += down
            else:
                nv, nbm, nw = self._nbest_torch(st, hyp_idx, pw, batch_indices, ps, tensor_beam, nb, n_best)

            # toHyps: every sentence keeps its current number of hypotheses, skipping invalid scores
            ok = nv > -np.inf
            rank = np.cumsum(ok, axis=1) - 1
            take = ok & (rank < W[active][:, None])
            rr, cc = np.nonzero(take)
            new_words = np.zeros((B0, beam), np.int64)
            new_scores = np.zeros((B0, beam), np.float32)
            new_prev = np.zeros((B0, beam), np.int64)
            new_n = np.zeros(B0, np.int64)
            new_words[active[rr], rank[rr, cc]] = nw[rr, cc]
            new_scores[active[rr], rank[rr, cc]] = nv[rr, cc]
            new_prev[active[rr], rank[rr, cc]] = nbm[rr, cc]
            new_n[active] = take.sum(axis=1)

            # purgeBeams: hypotheses that ended in EOS leave the beam; a sentence whose beam is empty
            # leaves the batch.  History::add scores the finished ones.
            length = t + 1                                       # history size when this step is added
            max_len_reached = length >= self.factor * width
            exists = col < new_n[:, None]
            is_eos = exists & (new_words == eos)
            surv = exists & ~is_eos
            new_W = surv.sum(axis=1)
            last = (new_W == 0) | max_len_reached
            fin_o, fin_p = np.nonzero(exists & (is_eos | last[:, None]))
            for o, pos in zip(fin_o, fin_p):
                norm = (float(new_scores[o, pos]) - self.wp * length) / (length ** self.alpha)
                finals[o].append((norm, t, int(pos)))
            rank2 = np.cumsum(surv, axis=1) - 1
            so, sp = np.nonzero(surv)
            unpurged_pos = np.zeros((B0, beam), np.int64)
            unpurged_pos[so, rank2[so, sp]] = sp
            history.append((new_words, new_prev, unpurged_pos))
            if max_len_reached:
                break
            words = np.zeros((B0, beam), np.int64)
            scores = np.zeros((B0, beam), np.float32)
            prev_state = np.zeros((B0, beam), np.int64)
            words[so, rank2[so, sp]] = new_words[so, sp]
            scores[so, rank2[so, sp]] = new_scores[so, sp]
            prev_state[so, rank2[so, sp]] = new_prev[so, sp]
            W = new_W
            step_map = np.full(B0, -1)
            step_map[active] = np.arange(nb)
            prev_dim = nb
            t += 1

        return self._traceback(history, finals, B0)

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

    @staticmethod
    def _traceback(history, finals, B0):
        results = []
        for o in range(B0):
            if not finals[o]:
                results.append(([], float("-inf")))
                continue
            score, t, pos = max(finals[o], key=lambda f: (f[0], -f[1], -f[2]))
            toks = []
            while True:
                words_t, prev_t, _ = history[t]
                toks.append(int(words_t[o, pos]))
                if t == 0:
                    break
                # the parent is addressed by its row in the previous step's (purged) beam; map that
                # back to its position in the previous step's unpurged list
                pos = int(history[t - 1][2][o, int(prev_t[o, pos])])
                t -= 1
            results.append((toks[::-1], score))
        return results


def decode_corpus(model: Int8Transformer, batches, beam=4, max_length_factor=1.5, normalize=1.0, native=None, native_search=True):
    """Translate all mini-batches on one replica; returns {sentence id: token list} and the token count."""
    bs = BeamSearch(model, beam, max_length_factor, normalize, native=native, native_search=native_search)
    out, n_tokens = {}, 0
    for sent_ids, ids, mask in batches:
        res = bs.search(ids, mask)
        for sid, (toks, _score) in zip(sent_ids, res):
            out[int(sid)] = toks
            n_tokens += len(toks)
    return out, n_tokens
