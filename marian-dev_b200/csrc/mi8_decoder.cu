// Host-side driver of one decoder time step (declared in include/marian_i8_decode.h): sequences the
// int8 affines and the glue kernels on one stream, with all buffers carved out of a caller-owned
// arena.  Restates DecoderTransformer::step (src/models/transformer.h:713-896): per layer
// self-attention over the re-projected history (or the SSRU cell), cross-attention over cached
// encoder keys/values, the ReLU feed-forward block, each followed by residual add + LayerNorm
// ("transformer-postprocess: dan"), then the tied output layer, log-softmax and n-best selection.
// mi8d_search adds the beam-search bookkeeping around the step (BeamSearch::search,
// src/translator/beam_search.cpp:249-538), so a mini-batch is translated by one call.
#include <cmath>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/marian_i8_decode.h"
#include "mi8_internal.h"

namespace mi8 {
namespace {

struct Weight {
  const int8_t* bt = nullptr;
  int K = 0, N = 0;
  const float* qm() const { return reinterpret_cast<const float*>(bt + static_cast<size_t>(K) * N); }
};

size_t align_up(size_t v, size_t a = 256) { return (v + a - 1) / a * a; }

struct Arena {
  uint8_t* base = nullptr;
  size_t size = 0, used = 0;
  template <typename T>
  T* take(size_t count) {
    size_t bytes = align_up(count * sizeof(T));
    T* p = base ? reinterpret_cast<T*>(base + used) : nullptr;
    used += bytes;
    return p;
  }
};

struct LayerBufs {
  float* slab = nullptr;     // [max_steps][slab_rows][d]  layer inputs (self-attention decoders), row order of each step
  float* rowmax = nullptr;   // [max_steps][slab_rows]     max|x| per slab row
  float* kslab = nullptr;    // [max_steps][slab_rows][d]  projected keys / values of the slabs, valid for the
  float* vslab = nullptr;    //                            history abs-max remembered in prev_bits
  int8_t* hq = nullptr;      // [max_steps][slab_rows][d]  quantised slabs + multiplier behind the last slab
  float* cross_k = nullptr;  // [max_batch * max_src, d]
  float* cross_v = nullptr;
  float* cell[2] = {nullptr, nullptr};  // SSRU state, double-buffered [max_rows, d]
};

}  // namespace
}  // namespace mi8

using namespace mi8;

struct mi8d_decoder {
  mi8d_config cfg;
  Arena arena;
  void* ws = nullptr;
  size_t ws_bytes = 0;
  std::unordered_map<std::string, Weight> weights;
  std::unordered_map<std::string, const float*> params;
  const float* positions = nullptr;

  std::vector<LayerBufs> layers;
  float* x_in = nullptr;                 // layer-0 input when there are no slabs (SSRU) and the final layer output
  float* x_final = nullptr;
  float *x1 = nullptr, *x2 = nullptr;    // after self / cross blocks
  float *qbuf = nullptr, *abuf = nullptr, *obuf = nullptr, *hbuf = nullptr, *fbuf = nullptr;
  int8_t *aq = nullptr, *cq = nullptr;
  unsigned* prev_bits = nullptr;   // per layer: history abs-max (bit pattern) the stored keys/values were computed with
  unsigned* reuse_stats = nullptr; // [0] (layer, step) pairs that reused stored keys/values, [1] all pairs
  int slab_rows = 0;               // rows reserved per history slab for the current mini-batch
  float* logits = nullptr;
  float* cand_score = nullptr;
  int* cand_word = nullptr;
  float* enc_x[2] = {nullptr, nullptr};
  float *enc_q = nullptr, *enc_k = nullptr, *enc_v = nullptr, *enc_h = nullptr;
  int8_t* enc_aq = nullptr;
  float* context[2] = {nullptr, nullptr};
  float* log_mask[2] = {nullptr, nullptr};
  int* anc[2] = {nullptr, nullptr};
  // beam-search bookkeeping (mi8d_search): per-step control words and n-best lists, device side and pinned host side
  int* s_ctrl = nullptr;            // [3 * max_rows + max_batch]: hypothesis rows, previous words, path scores (as bits), batch rows
  int* s_out = nullptr;             // [3][max_batch * 8]: scores (as bits), beams, words
  int* h_ctrl = nullptr;
  int* h_out = nullptr;
  float *blk_max = nullptr, *blk_sum = nullptr, *blk_topv = nullptr;   // per (row, 128-word block) partials of the output layer
  int* blk_topi = nullptr;
  bool keep_logits = false;
  unsigned* slots = nullptr;
  int n_slots = 0;
  // The history chain of a self-attention block (abs-max -> quantise -> key GEMM, value GEMM) does not depend on
  // the query projection, and the two GEMMs not on each other: they run on two internal streams, forked from
  // and joined to the caller's stream with events.
  cudaStream_t side[2] = {nullptr, nullptr};
  cudaEvent_t ev_x = nullptr, ev_hq = nullptr, ev_k = nullptr, ev_v = nullptr;
  bool overlap = false;

  int t = 0, batch = 0, src = 0, ctx_cur = 0, anc_cur = 0, cell_cur = 0;
  bool cross_valid = false;

  // lays the arena out; with a null base it only measures
  void layout() {
    const mi8d_config& c = cfg;
    const size_t d = c.dim_emb, f = c.dim_ffn, R = c.max_rows, T = c.max_steps, B = c.max_batch, S = c.max_src;
    arena.used = 0;
    layers.assign(c.dec_depth, LayerBufs());
    for(auto& L : layers) {
      if(!c.ssru) {
        L.slab = arena.take<float>(T * R * d);
        L.rowmax = arena.take<float>(T * R);
        L.kslab = arena.take<float>(T * R * d);
        L.vslab = arena.take<float>(T * R * d);
        L.hq = arena.take<int8_t>(T * R * d + 256);
      } else {
        L.cell[0] = arena.take<float>(R * d);
        L.cell[1] = arena.take<float>(R * d);
      }
      L.cross_k = arena.take<float>(B * S * d);
      L.cross_v = arena.take<float>(B * S * d);
    }
    x_in = arena.take<float>(R * d);
    x_final = arena.take<float>(R * d);
    x1 = arena.take<float>(R * d);
    x2 = arena.take<float>(R * d);
    qbuf = arena.take<float>(R * d);
    abuf = arena.take<float>(R * d);
    obuf = arena.take<float>(R * d);
    fbuf = arena.take<float>(R * d);
    hbuf = arena.take<float>(R * f);
    aq = arena.take<int8_t>(R * (f > d ? f : d) + 256);
    if(!c.ssru) {
      anc[0] = arena.take<int>(T * R);
      anc[1] = arena.take<int>(T * R);
      prev_bits = arena.take<unsigned>(c.dec_depth);
      reuse_stats = arena.take<unsigned>(2);
    }
    cq = arena.take<int8_t>(B * S * d + 256);
    logits = arena.take<float>(R * static_cast<size_t>(c.vocab));
    const size_t nb = (static_cast<size_t>(c.vocab) + 127) / 128;
    blk_max = arena.take<float>(R * nb);
    blk_sum = arena.take<float>(R * nb);
    blk_topv = arena.take<float>(R * nb * 8);
    blk_topi = arena.take<int>(R * nb * 8);
    s_ctrl = arena.take<int>(3 * R + B);
    s_out = arena.take<int>(3 * B * 8);
    cand_score = arena.take<float>(R * 8);
    cand_word = arena.take<int>(R * 8);
    for(int i = 0; i < 2; ++i) {
      context[i] = arena.take<float>(B * S * d);
      log_mask[i] = arena.take<float>(B * S);
    }
    if(c.enc_depth > 0) {
      const size_t M = B * S;
      for(int i = 0; i < 2; ++i)
        enc_x[i] = arena.take<float>(M * d);
      enc_q = arena.take<float>(M * d);
      enc_k = arena.take<float>(M * d);
      enc_v = arena.take<float>(M * d);
      enc_h = arena.take<float>(M * f);
      enc_aq = arena.take<int8_t>(M * (f > d ? f : d) + 256);
    }
    n_slots = 8 * c.dec_depth + 8 + 4 * c.enc_depth;
    slots = arena.take<unsigned>(n_slots);
  }

  const Weight* W(const std::string& name) const {
    auto it = weights.find(name);
    return it == weights.end() ? nullptr : &it->second;
  }
  const float* P(const std::string& name) const {
    auto it = params.find(name);
    return it == params.end() ? nullptr : it->second;
  }
};

namespace {

// aq (already quantised, multiplier behind the data) x weight -> c
int gemm(mi8d_decoder* d, const int8_t* a, int M, const std::string& wname, const std::string& bname, bool relu, float* c,
         cudaStream_t s, unsigned* absmax_out = nullptr, int force_splits = 0) {
  const Weight* w = d->W(wname);
  if(w == nullptr)
    return MI8_ERR_BAD_ARG;
  const float* bias = nullptr;
  if(!bname.empty()) {
    bias = d->P(bname);
    if(bias == nullptr)
      return MI8_ERR_BAD_ARG;
  }
  const float* qa = reinterpret_cast<const float*>(a + static_cast<size_t>(M) * w->K);
  return launch_gemm(a, w->bt, M, w->N, w->K, qa, w->qm(), 1.0f, bias, relu ? 1 : 0, c, MI8_F32, nullptr, d->ws, d->ws_bytes, s, 0,
                     force_splits, absmax_out);
}

int quant(mi8d_decoder* /*d*/, const float* x, size_t rows, size_t dim, const unsigned* slot, int8_t* q, cudaStream_t s) {
  return launch_quantize_slot(x, rows * dim, slot, q, reinterpret_cast<float*>(q + rows * dim), s);
}

int add_ln(mi8d_decoder* d, const float* a, const float* resid, const std::string& prefix, int rows, float* out, float* rowmax,
           unsigned* slot, cudaStream_t s) {
  const float* g = d->P(prefix + "_ln_scale");
  const float* b = d->P(prefix + "_ln_bias");
  if(g == nullptr || b == nullptr)
    return MI8_ERR_BAD_ARG;
  return launch_add_layernorm(a, resid, g, b, 1e-6f, rows, d->cfg.dim_emb, out, rowmax, slot, s);
}

#define MI8D_CUDA(expr)               \
  do {                                \
    cudaError_t ce_ = (expr);         \
    if(ce_ != cudaSuccess) {          \
      set_last_cuda_error(ce_);       \
      return MI8_ERR_LAUNCH;          \
    }                                 \
  } while(0)

#define MI8D_TRY(expr)      \
  do {                      \
    int rc_ = (expr);       \
    if(rc_ != MI8_OK)       \
      return rc_;           \
  } while(0)

}  // namespace

extern "C" {

size_t mi8d_arena_bytes(const mi8d_config* cfg) {
  if(cfg == nullptr)
    return 0;
  mi8d_decoder tmp;
  tmp.cfg = *cfg;
  tmp.layout();
  return tmp.arena.used + 4096;
}

int mi8d_create(const mi8d_config* cfg, void* arena, size_t arena_bytes, void* workspace, size_t workspace_bytes,
                mi8d_decoder** out) {
  if(cfg == nullptr || arena == nullptr || out == nullptr || workspace == nullptr)
    return MI8_ERR_BAD_ARG;
  if(cfg->enc_depth < 0 || cfg->dim_emb % 16 != 0 || cfg->dim_ffn % 16 != 0 || cfg->heads <= 0 || cfg->dim_emb % cfg->heads != 0 || cfg->dec_depth <= 0 ||
     cfg->max_rows <= 0 || cfg->max_steps <= 0 || cfg->max_batch <= 0 || cfg->max_src <= 0 || cfg->vocab <= 0)
    return MI8_ERR_BAD_ARG;
  const int dh = cfg->dim_emb / cfg->heads;
  if(dh != 64 && dh != 32)
    return MI8_ERR_UNSUPPORTED;
  if(reinterpret_cast<uintptr_t>(arena) & 255u)
    return MI8_ERR_MISALIGNED;
  if(arena_bytes < mi8d_arena_bytes(cfg) || workspace_bytes < mi8_workspace_bytes(0, 0, 0))
    return MI8_ERR_WORKSPACE;
  mi8d_decoder* d = new mi8d_decoder();
  d->cfg = *cfg;
  d->arena.base = static_cast<uint8_t*>(arena);
  d->arena.size = arena_bytes;
  d->layout();
  d->ws = workspace;
  d->ws_bytes = workspace_bytes;
  if(d->reuse_stats != nullptr)
    cudaMemset(d->reuse_stats, 0, 2 * sizeof(unsigned));
  {
    // pinned host staging for the beam search's per-step upload and download
    const size_t nc = 3 * static_cast<size_t>(cfg->max_rows) + cfg->max_batch, no = 3 * static_cast<size_t>(cfg->max_batch) * 8;
    if(cudaHostAlloc(reinterpret_cast<void**>(&d->h_ctrl), nc * sizeof(int), cudaHostAllocDefault) != cudaSuccess ||
       cudaHostAlloc(reinterpret_cast<void**>(&d->h_out), no * sizeof(int), cudaHostAllocDefault) != cudaSuccess) {
      cudaGetLastError();
      if(d->h_ctrl)
        cudaFreeHost(d->h_ctrl);
      d->h_ctrl = d->h_out = nullptr;   // mi8d_search then reports MI8_ERR_WORKSPACE; stepping by hand still works
    }
  }
  if(!cfg->ssru) {
    bool ok = cudaStreamCreateWithFlags(&d->side[0], cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&d->side[1], cudaStreamNonBlocking) == cudaSuccess;
    for(cudaEvent_t* e : {&d->ev_x, &d->ev_hq, &d->ev_k, &d->ev_v})
      ok = ok && cudaEventCreateWithFlags(e, cudaEventDisableTiming) == cudaSuccess;
    d->overlap = ok;   // without them the step simply runs on the caller's stream alone
    if(!ok)
      cudaGetLastError();
  }
  *out = d;
  return MI8_OK;
}

void mi8d_destroy(mi8d_decoder* d) {
  if(d == nullptr)
    return;
  for(cudaStream_t st : d->side)
    if(st != nullptr) {
      cudaStreamSynchronize(st);
      cudaStreamDestroy(st);
    }
  for(cudaEvent_t e : {d->ev_x, d->ev_hq, d->ev_k, d->ev_v})
    if(e != nullptr)
      cudaEventDestroy(e);
  if(d->h_ctrl)
    cudaFreeHost(d->h_ctrl);
  if(d->h_out)
    cudaFreeHost(d->h_out);
  delete d;
}

int mi8d_set_weight(mi8d_decoder* d, const char* name, const int8_t* bt, int K, int N) {
  if(d == nullptr || name == nullptr || bt == nullptr || K <= 0 || N <= 0)
    return MI8_ERR_BAD_ARG;
  if(K % 16 != 0 || (reinterpret_cast<uintptr_t>(bt) & 15u))
    return MI8_ERR_MISALIGNED;
  Weight w;
  w.bt = bt;
  w.K = K;
  w.N = N;
  d->weights[name] = w;
  return MI8_OK;
}

int mi8d_set_param(mi8d_decoder* d, const char* name, const float* p) {
  if(d == nullptr || name == nullptr || p == nullptr)
    return MI8_ERR_BAD_ARG;
  d->params[name] = p;
  return MI8_OK;
}

int mi8d_set_positions(mi8d_decoder* d, const float* table) {
  if(d == nullptr || table == nullptr)
    return MI8_ERR_BAD_ARG;
  d->positions = table;
  return MI8_OK;
}

const float* mi8d_last_logits(const mi8d_decoder* d) { return d ? d->logits : nullptr; }

int mi8d_keep_logits(mi8d_decoder* d, int keep) {
  if(d == nullptr)
    return MI8_ERR_BAD_ARG;
  d->keep_logits = keep != 0;
  return MI8_OK;
}

size_t mi8g_output_scratch_bytes(int rows, int vocab) {
  if(rows <= 0 || vocab <= 0)
    return 0;
  return static_cast<size_t>(rows) * ((static_cast<size_t>(vocab) + 127) / 128) * 18 * sizeof(float);
}

int mi8g_output_topk(const int8_t* aq, const float* d_qa, const int8_t* wq, const float* d_qw, int rows, int vocab, int K,
                     const float* bias, int k, const float* prev_scores, void* scratch, size_t scratch_bytes, float* logits_out,
                     float* cand_score, int* cand_word, void* stream) {
  if(rows <= 0 || vocab <= 0 || k < 1 || k > 8 || scratch == nullptr || cand_score == nullptr || cand_word == nullptr)
    return MI8_ERR_BAD_ARG;
  if(scratch_bytes < mi8g_output_scratch_bytes(rows, vocab))
    return MI8_ERR_WORKSPACE;
  const size_t cells = static_cast<size_t>(rows) * ((static_cast<size_t>(vocab) + 127) / 128);
  float* blk_max = static_cast<float*>(scratch);
  float* blk_sum = blk_max + cells;
  float* blk_topv = blk_sum + cells;
  int* blk_topi = reinterpret_cast<int*>(blk_topv + cells * 8);
  const int k_top = k <= 4 ? 4 : 8;
  int rc = launch_gemm_logits(aq, d_qa, wq, d_qw, rows, vocab, K, bias, 1.0f, k_top, blk_max, blk_sum, blk_topv, blk_topi, logits_out,
                              as_stream(stream));
  if(rc != MI8_OK)
    return rc;
  return launch_lse_merge(blk_max, blk_sum, blk_topv, blk_topi, rows, vocab, k_top, k, prev_scores, cand_score, cand_word, as_stream(stream));
}

int mi8d_history_reuse(mi8d_decoder* d, unsigned out[2], int reset) {
  if(d == nullptr || out == nullptr)
    return MI8_ERR_BAD_ARG;
  out[0] = out[1] = 0;
  if(d->reuse_stats == nullptr)
    return MI8_OK;
  cudaError_t e = cudaDeviceSynchronize();
  if(e == cudaSuccess)
    e = cudaMemcpy(out, d->reuse_stats, 2 * sizeof(unsigned), cudaMemcpyDeviceToHost);
  if(e == cudaSuccess && reset)
    e = cudaMemset(d->reuse_stats, 0, 2 * sizeof(unsigned));
  if(e != cudaSuccess) {
    set_last_cuda_error(e);
    return MI8_ERR_LAUNCH;
  }
  return MI8_OK;
}

int mi8g_embed(const float* wemb, const int* words, const float* pos, int pos_mod, float scale, int rows, int dim, float* out,
               float* rowmax, unsigned* absmax_slot, void* stream) {
  return launch_embed(wemb, words, pos, pos_mod, scale, rows, dim, out, rowmax, absmax_slot, as_stream(stream));
}
int mi8g_add_layernorm(const float* a, const float* resid, const float* gamma, const float* beta, float eps, int rows, int dim,
                       float* out, float* rowmax, unsigned* absmax_slot, void* stream) {
  if(gamma == nullptr || beta == nullptr)
    return MI8_ERR_BAD_ARG;
  return launch_add_layernorm(a, resid, gamma, beta, eps, rows, dim, out, rowmax, absmax_slot, as_stream(stream));
}
int mi8g_quantize_slot(const float* x, size_t n, const unsigned* absmax_slot, int8_t* q, float* d_quant_mult, void* stream) {
  return launch_quantize_slot(x, n, absmax_slot, q, d_quant_mult, as_stream(stream));
}
int mi8g_attention1(const float* q, const float* k, const float* v, const float* log_mask, int rows, int heads, int dim_head,
                    int len, int batch, int mode, float* out, unsigned* absmax_slot, void* stream) {
  if(q == nullptr || k == nullptr || v == nullptr || out == nullptr)
    return MI8_ERR_BAD_ARG;
  return launch_attention1(q, k, v, log_mask, rows, heads, dim_head, len, batch, mode, out, absmax_slot, as_stream(stream));
}
int mi8g_lse_topk(const float* logits, int rows, int vocab, int k, const float* prev_scores, float* cand_score, int* cand_word,
                  void* stream) {
  if(logits == nullptr || cand_score == nullptr || cand_word == nullptr)
    return MI8_ERR_BAD_ARG;
  return launch_lse_topk(logits, rows, vocab, k, prev_scores, cand_score, cand_word, as_stream(stream));
}
int mi8g_nbest_merge(const float* cand_score, const int* cand_word, int beam, int batch, int vocab, int k, float* out_score,
                     int* out_beam, int* out_word, void* stream) {
  if(cand_score == nullptr || cand_word == nullptr || out_score == nullptr || out_beam == nullptr || out_word == nullptr)
    return MI8_ERR_BAD_ARG;
  return launch_nbest_merge(cand_score, cand_word, beam, batch, vocab, k, out_score, out_beam, out_word, as_stream(stream));
}

int mi8d_start(mi8d_decoder* d, const float* context, const float* log_mask, int batch, int src, void* stream) {
  if(d == nullptr || context == nullptr || log_mask == nullptr || batch <= 0 || src <= 0)
    return MI8_ERR_BAD_ARG;
  if(batch > d->cfg.max_batch || src > d->cfg.max_src)
    return MI8_ERR_UNSUPPORTED;
  cudaStream_t s = as_stream(stream);
  const size_t dm = d->cfg.dim_emb;
  cudaError_t e = cudaMemcpyAsync(d->context[0], context, sizeof(float) * batch * src * dm, cudaMemcpyDeviceToDevice, s);
  if(e == cudaSuccess)
    e = cudaMemcpyAsync(d->log_mask[0], log_mask, sizeof(float) * batch * src, cudaMemcpyDeviceToDevice, s);
  if(e == cudaSuccess && d->cfg.ssru)
    for(auto& L : d->layers)
      if(e == cudaSuccess)
        e = cudaMemsetAsync(L.cell[0], 0, sizeof(float) * static_cast<size_t>(batch) * dm, s);
  if(e != cudaSuccess) {
    set_last_cuda_error(e);
    return MI8_ERR_LAUNCH;
  }
  d->t = 0;
  d->batch = batch;
  d->src = src;
  d->ctx_cur = 0;
  d->anc_cur = 0;
  d->cell_cur = 0;
  d->cross_valid = false;
  d->slab_rows = (d->cfg.max_rows / d->cfg.max_batch) * batch;
  return MI8_OK;
}

int mi8d_encode(mi8d_decoder* d, const int* ids, const float* log_mask, int batch, int src, void* stream) {
  if(d == nullptr || ids == nullptr || log_mask == nullptr || batch <= 0 || src <= 0)
    return MI8_ERR_BAD_ARG;
  const mi8d_config& c = d->cfg;
  if(c.enc_depth <= 0 || batch > c.max_batch || src > c.max_src || src > c.max_steps)
    return MI8_ERR_UNSUPPORTED;
  if(d->positions == nullptr || d->P("Wemb") == nullptr)
    return MI8_ERR_BAD_ARG;
  cudaStream_t s = as_stream(stream);
  const int dm = c.dim_emb, M = batch * src;
  cudaError_t e = cudaMemsetAsync(d->slots, 0, sizeof(unsigned) * d->n_slots, s);
  if(e == cudaSuccess)
    e = cudaMemcpyAsync(d->log_mask[0], log_mask, sizeof(float) * batch * src, cudaMemcpyDeviceToDevice, s);
  if(e != cudaSuccess) {
    set_last_cuda_error(e);
    return MI8_ERR_LAUNCH;
  }
  unsigned* slot = d->slots;
  auto next_slot = [&]() { return slot++; };
  // embeddings * sqrt(d) + positions 0..src-1 (src/models/transformer.h:93,110-114)
  float* x = d->enc_x[0];
  unsigned* x_slot = next_slot();
  MI8D_TRY(launch_embed(d->P("Wemb"), ids, d->positions, src, sqrtf(static_cast<float>(dm)), M, dm, x, nullptr, x_slot, s));
  for(int l = 0; l < c.enc_depth; ++l) {
    const std::string li = "encoder_l" + std::to_string(l + 1);
    const std::string pre = li + "_self", ffn = li + "_ffn";
    unsigned *sa = next_slot(), *s1 = next_slot(), *s3 = next_slot();
    // q, keys and values are the same tensor: one quantisation serves the three projections
    MI8D_TRY(launch_quantize_slot(x, static_cast<size_t>(M) * dm, x_slot, d->enc_aq, reinterpret_cast<float*>(d->enc_aq + static_cast<size_t>(M) * dm), s));
    MI8D_TRY(gemm(d, d->enc_aq, M, pre + "_Wq", pre + "_bq", false, d->enc_q, s));
    MI8D_TRY(gemm(d, d->enc_aq, M, pre + "_Wk", pre + "_bk", false, d->enc_k, s));
    MI8D_TRY(gemm(d, d->enc_aq, M, pre + "_Wv", pre + "_bv", false, d->enc_v, s));
    float* a = d->enc_x[1];   // attention output, then reused as x1
    MI8D_TRY(launch_attention1(d->enc_q, d->enc_k, d->enc_v, d->log_mask[0], M, c.heads, dm / c.heads, src, batch, 2, a, sa, s));
    MI8D_TRY(launch_quantize_slot(a, static_cast<size_t>(M) * dm, sa, d->enc_aq, reinterpret_cast<float*>(d->enc_aq + static_cast<size_t>(M) * dm), s));
    MI8D_TRY(gemm(d, d->enc_aq, M, pre + "_Wo", pre + "_bo", false, d->enc_q, s));
    MI8D_TRY(add_ln(d, d->enc_q, x, pre + "_Wo", M, a, nullptr, s1, s));                       // x1 = LN(Wo(a) + x)
    MI8D_TRY(launch_quantize_slot(a, static_cast<size_t>(M) * dm, s1, d->enc_aq, reinterpret_cast<float*>(d->enc_aq + static_cast<size_t>(M) * dm), s));
    MI8D_TRY(gemm(d, d->enc_aq, M, ffn + "_W1", ffn + "_b1", true, d->enc_h, s, s3));
    MI8D_TRY(launch_quantize_slot(d->enc_h, static_cast<size_t>(M) * c.dim_ffn, s3, d->enc_aq,
                                  reinterpret_cast<float*>(d->enc_aq + static_cast<size_t>(M) * c.dim_ffn), s));
    MI8D_TRY(gemm(d, d->enc_aq, M, ffn + "_W2", ffn + "_b2", false, d->enc_q, s));
    const bool last = l + 1 == c.enc_depth;
    float* nx = last ? d->context[0] : x;                                                     // the last layer writes the context
    x_slot = next_slot();
    MI8D_TRY(add_ln(d, d->enc_q, a, ffn + "_ffn", M, nx, nullptr, x_slot, s));
    x = nx;
  }
  if(c.ssru) {
    for(auto& L : d->layers) {
      e = cudaMemsetAsync(L.cell[0], 0, sizeof(float) * static_cast<size_t>(batch) * dm, s);
      if(e != cudaSuccess) {
        set_last_cuda_error(e);
        return MI8_ERR_LAUNCH;
      }
    }
  }
  d->t = 0;
  d->batch = batch;
  d->src = src;
  d->ctx_cur = 0;
  d->anc_cur = 0;
  d->cell_cur = 0;
  d->cross_valid = false;
  d->slab_rows = (c.max_rows / c.max_batch) * batch;
  return MI8_OK;
}

int mi8d_step(mi8d_decoder* d, const int* hyp_idx, const int* prev_words, const int* batch_idx, const float* prev_scores, int beam,
              int batch, int n_best, float* out_score, int* out_beam, int* out_word, void* stream) {
  if(d == nullptr || beam <= 0 || batch <= 0 || n_best <= 0 || n_best > 8 || out_score == nullptr || out_beam == nullptr ||
     out_word == nullptr)
    return MI8_ERR_BAD_ARG;
  const mi8d_config& c = d->cfg;
  const int t = d->t;
  const int R = beam * batch;
  if(R > c.max_rows || t >= c.max_steps || batch > d->batch || (!c.ssru && R > d->slab_rows))
    return MI8_ERR_UNSUPPORTED;
  if(t > 0 && (hyp_idx == nullptr || prev_words == nullptr))
    return MI8_ERR_BAD_ARG;
  if(t == 0 && beam != 1)
    return MI8_ERR_BAD_ARG;
  if(d->positions == nullptr || d->P("Wemb") == nullptr)
    return MI8_ERR_BAD_ARG;
  cudaStream_t s = as_stream(stream);
  const int dm = c.dim_emb, S = d->src;
  const int SR = d->slab_rows;
  const size_t slab_stride = static_cast<size_t>(SR) * dm;

  cudaError_t e = cudaMemsetAsync(d->slots, 0, sizeof(unsigned) * d->n_slots, s);
  if(e != cudaSuccess) {
    set_last_cuda_error(e);
    return MI8_ERR_LAUNCH;
  }
  unsigned* slot = d->slots;
  auto next_slot = [&]() { return slot++; };

  // sentences that finished leave the batch: compact the encoder context, recompute cross K/V
  if(batch != d->batch) {
    if(batch_idx == nullptr)
      return MI8_ERR_BAD_ARG;
    const int nxt = d->ctx_cur ^ 1;
    MI8D_TRY(launch_gather_rows(d->context[d->ctx_cur], batch_idx, batch, S * dm, d->context[nxt], s));
    MI8D_TRY(launch_gather_rows(d->log_mask[d->ctx_cur], batch_idx, batch, S, d->log_mask[nxt], s));
    d->ctx_cur = nxt;
    d->batch = batch;
    d->cross_valid = false;
  }
  const float* ctx = d->context[d->ctx_cur];
  const float* lmask = d->log_mask[d->ctx_cur];
  if(!d->cross_valid) {
    // one quantisation of the context serves the key and value projections of every layer
    const size_t n = static_cast<size_t>(batch) * S * dm;
    float* cq_tail = reinterpret_cast<float*>(d->cq + n);
    MI8D_TRY(launch_max_absolute(ctx, n, nullptr, cq_tail, d->ws, d->ws_bytes, s));
    MI8D_TRY(launch_quantize(ctx, n, cq_tail, d->cq, s));
    for(int l = 0; l < c.dec_depth; ++l) {
      const std::string pre = "decoder_l" + std::to_string(l + 1) + "_context";
      MI8D_TRY(gemm(d, d->cq, batch * S, pre + "_Wk", pre + "_bk", false, d->layers[l].cross_k, s));
      MI8D_TRY(gemm(d, d->cq, batch * S, pre + "_Wv", pre + "_bv", false, d->layers[l].cross_v, s));
    }
    d->cross_valid = true;
  }

  const int anc_new = d->anc_cur ^ 1;
  if(!c.ssru)
    MI8D_TRY(launch_ancestors_update(d->anc[d->anc_cur], d->anc[anc_new], hyp_idx, t, R, SR, s));

  // layer-0 input: scaled embedding of the previous word (zero at the first step) + position t
  float* x = c.ssru ? d->x_in : d->layers[0].slab + static_cast<size_t>(t) * slab_stride;
  float* x_rowmax = c.ssru ? nullptr : d->layers[0].rowmax + static_cast<size_t>(t) * SR;
  unsigned* x_slot = next_slot();
  MI8D_TRY(launch_embed(d->P("Wemb"), t == 0 ? nullptr : prev_words, d->positions + static_cast<size_t>(t) * dm, 0,
                        sqrtf(static_cast<float>(dm)), R, dm, x, x_rowmax, x_slot, s));

  const int cell_new = d->cell_cur ^ 1;
  for(int l = 0; l < c.dec_depth; ++l) {
    LayerBufs& L = d->layers[l];
    const std::string li = "decoder_l" + std::to_string(l + 1);
    unsigned* s1 = next_slot();
    if(c.ssru) {
      const std::string pre = li + "_rnn";
      MI8D_TRY(quant(d, x, R, dm, x_slot, d->aq, s));
      MI8D_TRY(gemm(d, d->aq, R, pre + "_W", "", false, d->qbuf, s));        // dot(input, W)
      MI8D_TRY(gemm(d, d->aq, R, pre + "_Wf", pre + "_bf", false, d->fbuf, s));  // affine(input, Wf, bf)
      MI8D_TRY(launch_ssru_cell(L.cell[d->cell_cur], t == 0 ? nullptr : hyp_idx, d->qbuf, d->fbuf, R, dm, L.cell[cell_new], d->abuf, s));
      MI8D_TRY(add_ln(d, d->abuf, x, pre + "_ffn", R, d->x1, nullptr, s1, s));
    } else {
      const std::string pre = li + "_self";
      unsigned* sh = next_slot();
      unsigned* sa = next_slot();
      // Keys and values are projections of the WHOLE history of layer inputs, quantised with one
      // multiplier over the live part of that history.  The projections of earlier steps are kept per slab
      // and stay valid as long as that multiplier's abs-max does not change (compared bit for bit on the
      // device); then only the newest slab is quantised and projected, otherwise everything is redone.
      // This chain only needs x and the ancestor table, so it runs beside the query projection.
      const bool ov = d->overlap;
      cudaStream_t sk = ov ? d->side[0] : s;   // abs-max, quantise, key GEMM
      cudaStream_t sv = ov ? d->side[1] : s;   // value GEMM
      if(ov) {
        MI8D_CUDA(cudaEventRecord(d->ev_x, s));
        MI8D_CUDA(cudaStreamWaitEvent(sk, d->ev_x, 0));
      }
      const int steps = t + 1;
      float* hq_tail = reinterpret_cast<float*>(L.hq + static_cast<size_t>(c.max_steps) * c.max_rows * dm);
      MI8D_TRY(launch_history_absmax(L.rowmax, d->anc[anc_new], steps, R, SR, sh, sk));
      MI8D_TRY(launch_history_quantize(L.slab, SR, steps, dm, sh, d->prev_bits + l, L.hq, hq_tail, sk));
      if(ov) {
        MI8D_CUDA(cudaEventRecord(d->ev_hq, sk));
        MI8D_CUDA(cudaStreamWaitEvent(sv, d->ev_hq, 0));
      }
      const Weight* wk = d->W(pre + "_Wk");
      const Weight* wv = d->W(pre + "_Wv");
      const float* bk = d->P(pre + "_bk");
      const float* bv = d->P(pre + "_bv");
      if(wk == nullptr || wv == nullptr || bk == nullptr || bv == nullptr)
        return MI8_ERR_BAD_ARG;
      // no split-K here (force_splits = 1): the three streams must not share the workspace's counters
      MI8D_TRY(launch_gemm(L.hq, wk->bt, steps * SR, wk->N, wk->K, hq_tail, wk->qm(), 1.0f, bk, 0, L.kslab, MI8_F32, nullptr, d->ws,
                           d->ws_bytes, sk, 0, 1, nullptr, d->prev_bits + l, sh, t * SR));
      MI8D_TRY(launch_gemm(L.hq, wv->bt, steps * SR, wv->N, wv->K, hq_tail, wv->qm(), 1.0f, bv, 0, L.vslab, MI8_F32, nullptr, d->ws,
                           d->ws_bytes, sv, 0, 1, nullptr, d->prev_bits + l, sh, t * SR));
      MI8D_TRY(quant(d, x, R, dm, x_slot, d->aq, s));
      MI8D_TRY(gemm(d, d->aq, R, pre + "_Wq", pre + "_bq", false, d->qbuf, s, nullptr, ov ? 1 : 0));
      if(ov) {
        MI8D_CUDA(cudaEventRecord(d->ev_k, sk));
        MI8D_CUDA(cudaEventRecord(d->ev_v, sv));
        MI8D_CUDA(cudaStreamWaitEvent(s, d->ev_k, 0));
        MI8D_CUDA(cudaStreamWaitEvent(s, d->ev_v, 0));
      }
      MI8D_TRY(launch_attention1(d->qbuf, L.kslab, L.vslab, nullptr, R, c.heads, dm / c.heads, steps, batch, 0, d->abuf, sa, s,
                                 d->anc[anc_new], SR, SR));
      MI8D_TRY(quant(d, d->abuf, R, dm, sa, d->aq, s));
      MI8D_TRY(gemm(d, d->aq, R, pre + "_Wo", pre + "_bo", false, d->obuf, s));
      MI8D_TRY(add_ln(d, d->obuf, x, pre + "_Wo", R, d->x1, nullptr, s1, s));
    }
    {
      const std::string pre = li + "_context";
      unsigned* sa = next_slot();
      unsigned* s2 = next_slot();
      MI8D_TRY(quant(d, d->x1, R, dm, s1, d->aq, s));
      MI8D_TRY(gemm(d, d->aq, R, pre + "_Wq", pre + "_bq", false, d->qbuf, s));
      MI8D_TRY(launch_attention1(d->qbuf, L.cross_k, L.cross_v, lmask, R, c.heads, dm / c.heads, S, batch, 1, d->abuf, sa, s));
      MI8D_TRY(quant(d, d->abuf, R, dm, sa, d->aq, s));
      MI8D_TRY(gemm(d, d->aq, R, pre + "_Wo", pre + "_bo", false, d->obuf, s));
      MI8D_TRY(add_ln(d, d->obuf, d->x1, pre + "_Wo", R, d->x2, nullptr, s2, s));

      const std::string ffn = li + "_ffn";
      unsigned* s3 = next_slot();
      MI8D_TRY(quant(d, d->x2, R, dm, s2, d->aq, s));
      MI8D_TRY(gemm(d, d->aq, R, ffn + "_W1", ffn + "_b1", true, d->hbuf, s, s3));   // ReLU and max|h| fused in the write-back
      MI8D_TRY(quant(d, d->hbuf, R, c.dim_ffn, s3, d->aq, s));
      MI8D_TRY(gemm(d, d->aq, R, ffn + "_W2", ffn + "_b2", false, d->obuf, s));
      // the block's output is the next layer's input: write it straight into that layer's history slab
      const bool last = l + 1 == c.dec_depth;
      float* nx = last ? d->x_final : (c.ssru ? d->x_in : d->layers[l + 1].slab + static_cast<size_t>(t) * slab_stride);
      float* nx_rowmax = (last || c.ssru) ? nullptr : d->layers[l + 1].rowmax + static_cast<size_t>(t) * SR;
      x_slot = next_slot();
      MI8D_TRY(add_ln(d, d->obuf, d->x2, ffn + "_ffn", R, nx, nx_rowmax, x_slot, s));
      x = nx;
    }
  }

  // tied output layer, then log-softmax + n-best per sentence over beam x vocabulary
  const float* out_b = d->P("decoder_ff_logit_out_b");
  const Weight* wout = d->W("Wemb_intgemm8");
  if(out_b == nullptr || wout == nullptr)
    return MI8_ERR_BAD_ARG;
  MI8D_TRY(quant(d, x, R, dm, x_slot, d->aq, s));
  // Below 512 rows the GEMM whose write-back reduces the 128-word blocks is faster than writing the logits and
  // reading them back (measured 49 vs 67 us at 256 rows, 33 vs 64 at 128); at 512 rows the two are equal (80 vs 78 us)
  // and for greedy search the plain GEMM followed by the log-softmax / top-k kernel wins.
  const bool fused_output = !d->keep_logits && R <= 480 && n_best >= 2;
  if(!fused_output) {
    MI8D_TRY(gemm(d, d->aq, R, "Wemb_intgemm8", "decoder_ff_logit_out_b", false, d->logits, s));
    MI8D_TRY(launch_lse_topk(d->logits, R, c.vocab, n_best, prev_scores, d->cand_score, d->cand_word, s));
  } else {
    // the GEMM's write-back reduces every 128-word block of a row; the logits never reach memory
    const int k_top = n_best <= 4 ? 4 : 8;
    const float* qa = reinterpret_cast<const float*>(d->aq + static_cast<size_t>(R) * dm);
    MI8D_TRY(launch_gemm_logits(d->aq, qa, wout->bt, wout->qm(), R, c.vocab, dm, out_b, 1.0f, k_top, d->blk_max, d->blk_sum, d->blk_topv,
                                d->blk_topi, nullptr, s));
    MI8D_TRY(launch_lse_merge(d->blk_max, d->blk_sum, d->blk_topv, d->blk_topi, R, c.vocab, k_top, n_best, prev_scores, d->cand_score,
                              d->cand_word, s));
  }
  MI8D_TRY(launch_nbest_merge(d->cand_score, d->cand_word, beam, batch, c.vocab, n_best, out_score, out_beam, out_word, s));

  if(!c.ssru)   // remember which abs-max the stored keys/values of every layer now belong to (slot 2 + 7*layer)
    MI8D_TRY(launch_history_commit(d->prev_bits, d->slots, 2, 7, c.dec_depth, d->reuse_stats, s));
  d->anc_cur = anc_new;
  d->cell_cur = cell_new;
  d->t = t + 1;
  return MI8_OK;
}

// Beam search over one mini-batch: the bookkeeping of BeamSearch::search (src/translator/beam_search.cpp:249-538)
// around mi8d_encode / mi8d_step.  Per step: every sentence still in the batch contributes its surviving
// hypotheses (beam-major rows, dummy slots with EOS and score -inf), the n-best lists come back, each sentence keeps
// as many candidates as it had hypotheses (toHyps, :24-210), hypotheses that ended in EOS are scored
// ((pathScore - wordPenalty * length) / length^normalize, src/translator/history.h:22-35) and leave the beam, a
// sentence whose beam is empty leaves the batch (purgeBeams, :224-245), and everything stops at
// length >= max_length_factor * width (:521-531).  The best finished hypothesis of every sentence is traced back
// through the per-step parent links.  One stream synchronisation per step (the n-best download).
int mi8d_search(mi8d_decoder* d, const int* ids, const float* log_mask, int batch, int width, const mi8d_search_config* sc,
                int* out_tokens, int max_out, int* out_len, float* out_score, unsigned long long* h2d_bytes, unsigned long long* d2h_bytes,
                void* stream) {
  if(d == nullptr || ids == nullptr || log_mask == nullptr || sc == nullptr || out_tokens == nullptr || out_len == nullptr || batch <= 0 ||
     width <= 0 || max_out <= 0 || sc->beam <= 0 || sc->beam > 8)
    return MI8_ERR_BAD_ARG;
  if(d->h_ctrl == nullptr || d->h_out == nullptr)
    return MI8_ERR_WORKSPACE;
  const mi8d_config& c = d->cfg;
  const int beam = sc->beam, eos = sc->eos_id, B0 = batch;
  if(beam * batch > c.max_rows || batch > c.max_batch)
    return MI8_ERR_UNSUPPORTED;
  cudaStream_t s = as_stream(stream);
  int rc = mi8d_encode(d, ids, log_mask, batch, width, stream);
  if(rc != MI8_OK)
    return rc;

  struct Final { double norm; int t, pos; };
  struct StepRecord { std::vector<int> words, prev, unpurged; };   // [B0 * beam] each
  std::vector<int> W(B0, beam), step_map(B0), new_n(B0), new_W(B0);
  std::vector<int> words(B0 * beam, 0), prev_state(B0 * beam, 0), new_words(B0 * beam), new_prev(B0 * beam);
  std::vector<float> scores(B0 * beam, 0.f), new_scores(B0 * beam);
  std::vector<std::vector<Final>> finals(B0);
  std::vector<StepRecord> history;
  std::vector<int> active;
  for(int o = 0; o < B0; ++o)
    step_map[o] = o;
  int prev_dim = B0;
  unsigned long long up_bytes = 0, down_bytes = 0;

  for(int t = 0;; ++t) {
    int max_beam = 0;
    active.clear();
    for(int o = 0; o < B0; ++o) {
      max_beam = W[o] > max_beam ? W[o] : max_beam;
      if(W[o] > 0)
        active.push_back(o);
    }
    if(max_beam == 0)
      break;
    const int nb = static_cast<int>(active.size());
    const int n_best = max_beam;
    const int tensor_beam = t == 0 ? 1 : max_beam;
    const int R = tensor_beam * nb;
    const int *hyp = nullptr, *pw = nullptr, *bidx = nullptr;
    const float* ps = nullptr;
    if(t > 0) {
      int* hc = d->h_ctrl;
      for(int j = 0; j < max_beam; ++j) {
        for(int a = 0; a < nb; ++a) {
          const int o = active[a];
          const bool valid = j < W[o];
          const int idx = j * nb + a;
          hc[idx] = valid ? prev_state[o * beam + j] * prev_dim + step_map[o] : 0;
          hc[R + idx] = valid ? words[o * beam + j] : eos;                       // dummy slots carry EOS
          const float sv = valid ? scores[o * beam + j] : -INFINITY;
          memcpy(&hc[2 * R + idx], &sv, sizeof(float));
        }
      }
      for(int a = 0; a < nb; ++a)
        hc[3 * R + a] = step_map[active[a]];
      const size_t n_up = static_cast<size_t>(3 * R + nb) * sizeof(int);
      MI8D_CUDA(cudaMemcpyAsync(d->s_ctrl, hc, n_up, cudaMemcpyHostToDevice, s));
      up_bytes += n_up;
      hyp = d->s_ctrl;
      pw = d->s_ctrl + R;
      ps = reinterpret_cast<const float*>(d->s_ctrl + 2 * R);
      bidx = d->s_ctrl + 3 * R;
    }
    const int cells = nb * n_best;
    float* o_score = reinterpret_cast<float*>(d->s_out);
    int* o_beam = d->s_out + cells;
    int* o_word = d->s_out + 2 * cells;
    rc = mi8d_step(d, hyp, pw, bidx, ps, tensor_beam, nb, n_best, o_score, o_beam, o_word, stream);
    if(rc != MI8_OK)
      return rc;
    MI8D_CUDA(cudaMemcpyAsync(d->h_out, d->s_out, static_cast<size_t>(3 * cells) * sizeof(int), cudaMemcpyDeviceToHost, s));
    MI8D_CUDA(cudaStreamSynchronize(s));
    down_bytes += static_cast<size_t>(3 * cells) * sizeof(int);
    const float* nv = reinterpret_cast<const float*>(d->h_out);
    const int* nbm = d->h_out + cells;
    const int* nw = d->h_out + 2 * cells;

    // toHyps: every sentence keeps its current number of hypotheses, skipping invalid scores
    std::fill(new_n.begin(), new_n.end(), 0);
    std::fill(new_words.begin(), new_words.end(), 0);
    std::fill(new_prev.begin(), new_prev.end(), 0);
    std::fill(new_scores.begin(), new_scores.end(), 0.f);
    for(int a = 0; a < nb; ++a) {
      const int o = active[a];
      int cnt = 0;
      for(int cidx = 0; cidx < n_best && cnt < W[o]; ++cidx) {
        const float v = nv[a * n_best + cidx];
        if(!(v > -INFINITY))
          continue;
        new_words[o * beam + cnt] = nw[a * n_best + cidx];
        new_scores[o * beam + cnt] = v;
        new_prev[o * beam + cnt] = nbm[a * n_best + cidx];
        ++cnt;
      }
      new_n[o] = cnt;
    }
    // purgeBeams and History::add
    const int length = t + 1;
    const bool max_len_reached = static_cast<double>(length) >= static_cast<double>(sc->max_length_factor) * width;
    StepRecord rec;
    rec.words = new_words;
    rec.prev = new_prev;
    rec.unpurged.assign(B0 * beam, 0);
    std::fill(new_W.begin(), new_W.end(), 0);
    for(int o = 0; o < B0; ++o) {
      int surv = 0;
      for(int j = 0; j < new_n[o]; ++j)
        if(new_words[o * beam + j] != eos)
          ++surv;
      new_W[o] = surv;
      const bool last = surv == 0 || max_len_reached;
      int rank = 0;
      for(int j = 0; j < new_n[o]; ++j) {
        const bool is_eos = new_words[o * beam + j] == eos;
        if(is_eos || last) {
          const double norm = (static_cast<double>(new_scores[o * beam + j]) - static_cast<double>(sc->word_penalty) * length) /
                              std::pow(static_cast<double>(length), static_cast<double>(sc->normalize));
          finals[o].push_back(Final{norm, t, j});
        }
        if(!is_eos)
          rec.unpurged[o * beam + rank++] = j;
      }
    }
    history.push_back(std::move(rec));
    if(max_len_reached)
      break;
    const StepRecord& cur = history.back();
    std::fill(words.begin(), words.end(), 0);
    std::fill(scores.begin(), scores.end(), 0.f);
    std::fill(prev_state.begin(), prev_state.end(), 0);
    for(int o = 0; o < B0; ++o) {
      for(int r2 = 0; r2 < new_W[o]; ++r2) {
        const int j = cur.unpurged[o * beam + r2];
        words[o * beam + r2] = new_words[o * beam + j];
        scores[o * beam + r2] = new_scores[o * beam + j];
        prev_state[o * beam + r2] = new_prev[o * beam + j];
      }
    }
    W = new_W;
    std::fill(step_map.begin(), step_map.end(), -1);
    for(int a = 0; a < nb; ++a)
      step_map[active[a]] = a;
    prev_dim = nb;
  }

  // best finished hypothesis per sentence (highest score; ties to the earlier step, then the earlier position), traced back
  for(int o = 0; o < B0; ++o) {
    out_len[o] = 0;
    if(out_score)
      out_score[o] = -INFINITY;
    if(finals[o].empty())
      continue;
    const Final* best = &finals[o][0];
    for(const Final& f : finals[o])
      if(f.norm > best->norm || (f.norm == best->norm && (f.t < best->t || (f.t == best->t && f.pos < best->pos))))
        best = &f;
    int t = best->t, pos = best->pos;
    const int len = t + 1;
    if(len > max_out)
      return MI8_ERR_WORKSPACE;
    for(;;) {
      out_tokens[static_cast<size_t>(o) * max_out + t] = history[t].words[o * beam + pos];
      if(t == 0)
        break;
      // the parent is addressed by its row in the previous step's purged beam: map it back to that step's unpurged list
      pos = history[t - 1].unpurged[o * beam + history[t].prev[o * beam + pos]];
      --t;
    }
    out_len[o] = len;
    if(out_score)
      out_score[o] = static_cast<float>(best->norm);
  }
  if(h2d_bytes)
    *h2d_bytes = up_bytes;
  if(d2h_bytes)
    *d2h_bytes = down_bytes;
  return MI8_OK;
}

}  // extern "C"
