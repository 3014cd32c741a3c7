"""Transformer / SSRU decode on the GPU through the C++ step driver of libmarian_i8.so.

This is the caller that drives the hot path for the tokens/sec metric.  ``Int8Transformer`` holds one model
replica (converted intgemm8 weights, fp32 biases / LayerNorm / embeddings), ``NativeStepper`` owns the driver
object (include/marian_i8_decode.h) that runs the encoder (src/models/transformer.h:581-637) and
``DecoderTransformer::step`` (:713-896) as sm_100a kernels, and ``BeamSearch`` is ``BeamSearch::search``
(src/translator/beam_search.cpp:249-538): by default the whole search of a mini-batch is one call into the driver
(``mi8d_search``); with ``native_search=False`` the bookkeeping runs here in NumPy around ``mi8d_step``.
There is no other implementation behind these classes: without the library nothing runs.

Row layout follows Marian: decoder tensors are ``[beam, batch, ...]`` flattened beam-major, so a
hypothesis lives in row ``beamHypIdx * batch + batchIdx`` (beam_search.cpp:398).
"""
from __future__ import annotations

import math

import numpy as np
import torch

from . import ops
from .model import TransformerConfig, is_intgemm_param, sinusoidal_table

NEG_MASK = -99999999.0  # transposedLogMask (transformer.h:138-143)


class Int8Transformer:
    """Model replica on one GPU: converted (intgemm8) weights, fp32 biases / LayerNorm / embeddings."""

    def __init__(self, cfg: TransformerConfig, params: dict, device, output_int8: bool = True, ws=None, scheme: str = "intgemm8"):
        """scheme: "intgemm8" (per-tensor multipliers) or "packed8avx512" (per-column weight and per-row activation
        quantisation, the FBGEMM / mjdgemm format).  params may hold float arrays (converted here, as marian-conv would),
        ready IntgemmTensor objects or, for packed8avx512, packed8.Packed8Weight objects / their item bytes."""
        from . import packed8
        if scheme not in ("intgemm8", "packed8avx512"):
            raise ops.Mi8Error(1, f"unknown weight scheme {scheme}")
        self.cfg = cfg
        self.scheme = scheme
        self.device = torch.device(device)
        self.ws = ws or ops.default_workspace(self.device)
        self.output_int8 = output_int8
        self.w = {}   # name -> IntgemmTensor or Packed8Weight
        self.p = {}   # name -> fp32 tensor
        for name, val in params.items():
            if isinstance(val, (ops.IntgemmTensor, packed8.Packed8Weight)):
                self.w[name] = val
            else:
                t = torch.as_tensor(np.ascontiguousarray(val), dtype=torch.float32).to(self.device)
                if is_intgemm_param(name):     # on-line conversion of a float model
                    self.w[name] = ops.prepareB(t, ws=self.ws) if scheme == "intgemm8" else packed8.prepareB(t)
                else:
                    self.p[name] = t
        self.wemb = self.p["Wemb"]                                 # [V, d] fp32, for the lookup
        # Tied output layer: affine(x, Wemb, b, transB=true).  The reference leaves Wemb in fp32
        # (its name test skips it); the int8 mode quantises the [V,d] matrix, which already is the
        # K-major Bt[N,K] layout (for packed8avx512: the conversion of Wemb^T, unless the caller supplied "Wemb_packed8").
        if not output_int8:
            self.wemb_q = None
        elif scheme == "intgemm8":
            self.wemb_q = ops.prepareB(self.wemb, w_is_nk=True, ws=self.ws)
        else:
            self.wemb_q = self.w.pop("Wemb_packed8", None) or packed8.prepareB(self.wemb.t().contiguous())
        self.d = cfg.dim_emb
        self.h = cfg.heads
        self.dh = cfg.dim_emb // cfg.heads


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
        # every driver has a workspace of its own (split-K counters, abs-max partials): several drivers of one model may
        # run side by side on different streams (decode_corpus(workers=...))
        self.ws = ops.Workspace(dev)
        handle = ctypes.c_void_p()
        check(self.L.mi8d_create(ctypes.byref(self.cfg), self.arena.data_ptr(), nbytes, self.ws.ptr, self.ws.nbytes,
                                 ctypes.byref(handle)))
        self.h = handle
        if model.scheme == "packed8avx512":
            def reg(name, w):
                check(self.L.mi8d_set_packed8_weight(self.h, name.encode(), w.bt.data_ptr(), w.scale_b.data_ptr(), w.zp_b.data_ptr(),
                                                     w.off_b.data_ptr(), w.K, w.N))
            for name, w in model.w.items():
                reg(name, w)
            reg("Wemb_packed8", model.wemb_q)
        else:
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

    OPTIONS = {"fuse_weights": 1, "quant_in_gemm": 2, "fused_output_max_rows": 3, "side_stream": 4, "attention_unroll": 5, "attention_block_heads": 6,
               "cluster_affine": 7, "fused_layernorm": 8, "cluster_max_rows": 9, "cluster_size": 10, "cluster_max_k": 11, "gemm_tile_rows": 12, "blocking_wait": 13}

    def set_option(self, name: str, value: int):
        """mi8d_set_option: tuning switches of the step driver (every setting computes the same bits)."""
        self.check(self.L.mi8d_set_option(self.h, self.OPTIONS[name], int(value)))

    def search_stats(self, reset: bool = False):
        """Host-side timing of mi8d_search since the last reset: seconds issuing kernels, seconds waiting for the
        device, seconds of bookkeeping, decoder steps."""
        import ctypes
        out = (ctypes.c_double * 4)()
        self.check(self.L.mi8d_search_stats(self.h, ctypes.byref(out), int(reset)))
        return {"issue_s": out[0], "wait_s": out[1], "host_s": out[2], "steps": int(out[3])}

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
        self.native = native      # the C++ step driver
        self.native_search = native_search   # also run the bookkeeping in the C++ driver (mi8d_search)
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
        if self.native is not None and self.native_search and type(self)._nbest is BeamSearch._nbest:
            res, up, down = self.native.search(ids_t, mask_t, self.beam, self.factor, self.alpha, self.wp, self.m.cfg.eos_id)
            self.h2d_bytes += up
            self.d2h_bytes += down
            return res
        eos = self.m.cfg.eos_id
        B0, width = ids_t.shape
        st = self._begin(ids_t, mask_t)

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
            nv, nbm, nw = self._nbest(st, hyp_idx, pw, batch_indices, ps, tensor_beam, nb, n_best)

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

    def _begin(self, ids_t, mask_t):
        """Encoder forward and start of the mini-batch; returns the per-search state the step hook receives."""
        if self.native is None:
            raise ops.Mi8Error(1, "BeamSearch needs a NativeStepper: the decode has no implementation outside libmarian_i8.so")
        self.native.encode(ids_t, mask_t)
        return None

    def _nbest(self, st, hyp_idx, pw, batch_indices, ps, tensor_beam, nb, n_best):
        """One decoder step: (scores, parent beams, words), each [batch, n_best], from mi8d_step."""
        nv, nbm, nw, up, down = self.native.step(hyp_idx, pw, batch_indices, ps, tensor_beam, nb, n_best)
        self.h2d_bytes += up
        self.d2h_bytes += down
        return nv, nbm, nw

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


class SearchPool:
    """Several beam searches of one model side by side on one GPU, each with a step driver and a CUDA stream of its own,
    fed from one queue of mini-batches - the reference's translator with more than one worker on a device
    (src/translator/translator.h:100-167: one graph, scorer set and search per worker, the thread pool hands the next
    mini-batch to whichever worker is free).  A decode step is a chain of ~120 small dependent kernels that leaves most of
    the GPU idle most of the time; a second chain fills those gaps.  Results do not depend on the number of workers: every
    mini-batch is decoded on its own."""

    def __init__(self, model: Int8Transformer, workers: int = 2, beam: int = 4, max_length_factor: float = 1.5, normalize: float = 1.0,
                 max_batch: int = 128, max_src: int = 136, max_steps: int = 208, first: "NativeStepper | None" = None,
                 shared_gpu_tile_rows: int = 256):
        self.m = model
        self.steppers = [first if (i == 0 and first is not None) else NativeStepper(model, max_batch=max_batch, beam=beam, max_src=max_src,
                                                                                       max_steps=max_steps) for i in range(max(1, workers))]
        self.searches = [BeamSearch(model, beam, max_length_factor, normalize, native=st) for st in self.steppers]
        self.streams = [torch.cuda.Stream(device=model.device) for _ in self.steppers]
        if len(self.steppers) > 1 and shared_gpu_tile_rows:
            # With the GPU shared, an affine need not spread over every SM to be done soonest: wide tiles on few SMs read each
            # weight tile fewer times (measured on transformer-big, 4 workers: 187 k -> 218 k tokens/s).  Same values either way.
            for st in self.steppers:
                st.set_option("gemm_tile_rows", shared_gpu_tile_rows)
                st.set_option("blocking_wait", 2)     # the workers' host threads poll and yield instead of spinning on a core each

    @property
    def h2d_bytes(self):
        return sum(s.h2d_bytes for s in self.searches)

    @property
    def d2h_bytes(self):
        return sum(s.d2h_bytes for s in self.searches)

    def reset_counters(self):
        for s in self.searches:
            s.h2d_bytes = s.d2h_bytes = 0

    def run(self, items, on_device: bool = False):
        """items: list of (ids, mask) - host arrays / pinned tensors, or device tensors with on_device=True.  Returns the
        list of per-mini-batch results in the order of `items`.  The caller's current stream is ordered before the first
        and after the last kernel of every worker."""
        nxt = [0]

        def source():
            i = nxt[0]
            nxt[0] += 1
            return (i, items[i][0], items[i][1]) if i < len(items) else None
        got = self.run_from(source, on_device)
        return [got[i] for i in range(len(items))]

    def run_from(self, source, on_device: bool = False):
        """The same with the mini-batches drawn from `source()` -> (key, ids, mask) or None when there are no more (called
        under a lock, by whichever worker is free).  Returns {key: results}."""
        import threading
        dev = self.m.device
        results = {}
        errors = []
        lock = threading.Lock()
        caller = torch.cuda.current_stream(dev)
        start = torch.cuda.Event()
        start.record(caller)
        done = [torch.cuda.Event() for _ in self.searches]

        def work(w):
            try:
                torch.cuda.set_device(dev)
                with torch.cuda.stream(self.streams[w]):
                    self.streams[w].wait_event(start)
                    while not errors:
                        with lock:
                            item = source()
                        if item is None:
                            break
                        key, ids, mask = item
                        results[key] = self.searches[w].search_device(ids, mask) if on_device else self.searches[w].search(ids, mask)
                    done[w].record(self.streams[w])
            except Exception as e:      # surfaces in the caller
                errors.append(e)

        if len(self.searches) == 1:
            work(0)
        else:
            threads = [threading.Thread(target=work, args=(w,)) for w in range(len(self.searches))]
            for t in threads:
                t.start()
            for t in threads:
                t.join()
        if errors:
            raise errors[0]
        for ev in done:
            caller.wait_event(ev)
        return results


def decode_corpus(model: Int8Transformer, batches, beam=4, max_length_factor=1.5, normalize=1.0, native=None, native_search=True,
                  search_cls=None, workers: int = 1):
    """Translate all mini-batches on one replica; returns {sentence id: token list} and the token count.
    workers > 1 (native step driver only): that many searches side by side on the GPU (SearchPool)."""
    out, n_tokens = {}, 0
    if workers > 1:
        if native is None or not native_search or search_cls is not None:
            raise ValueError("workers > 1 needs the native step driver and its C++ search")
        widest = max(b[1].shape[1] for b in batches)
        pool = SearchPool(model, workers, beam, max_length_factor, normalize, max_batch=native.max_batch, max_src=native.max_src,
                          max_steps=native.max_steps, first=native)
        assert widest <= native.max_src
        all_res = pool.run([(ids, mask) for _sid, ids, mask in batches])
        torch.cuda.current_stream(model.device).synchronize()
        for (sent_ids, _ids, _mask), res in zip(batches, all_res):
            for sid, (toks, _score) in zip(sent_ids, res):
                out[int(sid)] = toks
                n_tokens += len(toks)
        return out, n_tokens
    bs = (search_cls or BeamSearch)(model, beam, max_length_factor, normalize, native=native, native_search=native_search)
    for sent_ids, ids, mask in batches:
        res = bs.search(ids, mask)
        for sid, (toks, _score) in zip(sent_ids, res):
            out[int(sid)] = toks
            n_tokens += len(toks)
    return out, n_tokens
