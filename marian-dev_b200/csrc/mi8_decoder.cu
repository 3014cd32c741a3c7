// Host-side driver of one decoder time step (declared in include/marian_i8_decode.h): sequences the
// int8 affines and the glue kernels on one stream, with all buffers carved out of a caller-owned
// arena.  Restates DecoderTransformer::step (src/models/transformer.h:713-896): per layer
// self-attention over the re-projected history (or the SSRU cell), cross-attention over cached
// encoder keys/values, the ReLU feed-forward block, each followed by residual add + LayerNorm
// ("transformer-postprocess: dan"), then the tied output layer, log-softmax and n-best selection.
// mi8d_search adds the beam-search bookkeeping around the step (BeamSearch::search,
// src/translator/beam_search.cpp:249-538), so a mini-batch is translated by one call.
#include <thread>
#include <algorithm>
#include <chrono>
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

// One affine as the step loop uses it: everything resolved to pointers once (no name lookups per step).
struct Aff {
  const int8_t* bt = nullptr;
  const float* qm = nullptr;       // intgemm8: the weight's multiplier
  const float* bias = nullptr;
  int K = 0, N = 0;
  // packed8avx512: per-column scale, zero point and column offset instead of one multiplier
  bool p8 = false;
  const float* scale_b = nullptr;
  const int32_t* zp_b = nullptr;
  const int32_t* off_b = nullptr;
};
struct P8Weight {
  const int8_t* bt = nullptr;
  const float* scale_b = nullptr;
  const int32_t* zp_b = nullptr;
  const int32_t* off_b = nullptr;
  int K = 0, N = 0;
};
// Several weights of the same shape multiplied with the same activation in one launch (Wk|Wv, Wq|Wk|Wv,
// the SSRU's W|Wf): their int8 matrices copied one behind the other into the arena.
struct Fused {
  int8_t* bt = nullptr;   // [nseg * n, K] in the arena
  int nseg = 0, n = 0, K = 0;
  const float* qm[3] = {nullptr, nullptr, nullptr};
  const float* bias[3] = {nullptr, nullptr, nullptr};
  bool ready = false;
};
struct Norm {
  const float* g = nullptr;
  const float* b = nullptr;
};
struct EncLayerW {
  Aff q, k, v, o, w1, w2;
  Fused qkv;
  Norm ln_att, ln_ffn;
};
struct DecLayerW {
  Aff self_q, self_k, self_v, self_o, rnn_w, rnn_wf, ctx_q, ctx_k, ctx_v, ctx_o, w1, w2;
  Fused self_kv, rnn, ctx_kv;
  Norm ln_self, ln_ctx, ln_ffn;
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

// Slots of the per-step abs-max array: slot 0 belongs to the embedding (input of layer 0), then eight per layer.
enum LayerSlot { kSlotSelfLn = 0, kSlotHistory, kSlotSelfAtt, kSlotCtxAtt, kSlotCtxLn, kSlotRelu, kSlotOut, kSlotsPerLayer = 8 };

}  // namespace
}  // namespace mi8

using namespace mi8;

struct mi8d_decoder {
  mi8d_config cfg;
  Arena arena;
  void* ws = nullptr;
  size_t ws_bytes = 0;
  std::unordered_map<std::string, Weight> weights;
  std::unordered_map<std::string, P8Weight> p8_weights;   // packed8avx512 model: every affine's weight is registered here instead
  bool p8 = false;
  std::unordered_map<std::string, const float*> params;
  const float* positions = nullptr;
  // resolved model (rebuilt by resolve() after a parameter was registered)
  bool dirty = true;
  bool can_fuse = false;              // dim_emb is a multiple of 128: a weight tile never straddles two fused matrices
  std::vector<EncLayerW> enc_w;
  std::vector<DecLayerW> dec_w;
  const float* wemb = nullptr;
  const float* out_bias = nullptr;
  Aff out_w;
  std::vector<int8_t*> fused_enc, fused_self, fused_ctx;   // arena storage of the fused matrices

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
  // packed8avx512: scale, zero point and sum of every row of the activation quantised last
  float* p8_scale_a = nullptr;
  int32_t *p8_zp_a = nullptr, *p8_sum_a = nullptr;
  // Re-projecting the keys/values of the EARLIER history slabs (needed only when the history's abs-max changed) does
  // not depend on the query projection: it runs on an internal stream, forked from and joined to the caller's
  // stream with events, beside the query projection and the newest slab's keys/values.
  cudaStream_t side = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  cudaEvent_t ev_step = nullptr;   // blocking-sync event: the host thread sleeps instead of spinning while a step runs (opt_blocking_wait)
  int opt_blocking_wait = 0;
  bool overlap = false;
  // tuning switches (mi8d_set_option)
  int opt_fuse = 1, opt_quant_in_gemm = 0, opt_fused_out_rows = 480, opt_side_stream = 1;
  int opt_gemm_tile = 0;
  int opt_cluster = 0, opt_fused_ln = 1, opt_cluster_max_rows = 1024, opt_cluster_size = 0, opt_cluster_max_k = 2048;
  // host-side timing of mi8d_search
  double t_issue = 0, t_wait = 0, t_host = 0, n_steps = 0;

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
    n_slots = kSlotsPerLayer * c.dec_depth + 8 + 4 * c.enc_depth;
    slots = arena.take<unsigned>(n_slots);
    const size_t max_act_rows = R > B * S ? R : B * S;
    p8_scale_a = arena.take<float>(max_act_rows);
    p8_zp_a = arena.take<int32_t>(max_act_rows);
    p8_sum_a = arena.take<int32_t>(max_act_rows);
    // storage of the fused weight matrices (copies of the registered int8 matrices, made once by resolve())
    can_fuse = d % 128 == 0;
    fused_enc.assign(c.enc_depth, nullptr);
    fused_self.assign(c.dec_depth, nullptr);
    fused_ctx.assign(c.dec_depth, nullptr);
    if(can_fuse) {
      for(auto& p : fused_enc)
        p = arena.take<int8_t>(3 * d * d);
      for(auto& p : fused_self)
        p = arena.take<int8_t>(2 * d * d);
      for(auto& p : fused_ctx)
        p = arena.take<int8_t>(2 * d * d);
    }
  }

  unsigned* layer_slot(int l, int which) const { return slots + 1 + kSlotsPerLayer * l + which; }
  unsigned* input_slot(int l) const { return l == 0 ? slots : layer_slot(l - 1, kSlotOut); }
  unsigned* enc_slot(int l, int which) const { return slots + 1 + kSlotsPerLayer * cfg.dec_depth + 4 * l + which; }

  const Weight* W(const std::string& name) const {
    auto it = weights.find(name);
    return it == weights.end() ? nullptr : &it->second;
  }
  const float* P(const std::string& name) const {
    auto it = params.find(name);
    return it == params.end() ? nullptr : it->second;
  }
  bool aff(Aff& a, const std::string& wname, const std::string& bname) const {
    a = Aff();
    if(p8) {
      auto it = p8_weights.find(wname);
      if(it == p8_weights.end())
        return false;
      a.p8 = true;
      a.bt = it->second.bt;
      a.scale_b = it->second.scale_b;
      a.zp_b = it->second.zp_b;
      a.off_b = it->second.off_b;
      a.K = it->second.K;
      a.N = it->second.N;
    } else {
      const Weight* w = W(wname);
      if(w == nullptr)
        return false;
      a.bt = w->bt;
      a.qm = w->qm();
      a.K = w->K;
      a.N = w->N;
    }
    a.bias = nullptr;
    if(!bname.empty()) {
      a.bias = P(bname);
      if(a.bias == nullptr)
        return false;
    }
    return true;
  }
  bool norm(Norm& n, const std::string& prefix) const {
    n.g = P(prefix + "_ln_scale");
    n.b = P(prefix + "_ln_bias");
    return n.g != nullptr && n.b != nullptr;
  }
  // copies the matrices of `parts` one behind the other into `store` (stream-ordered on s)
  bool fuse(Fused& f, int8_t* store, std::initializer_list<const Aff*> parts, cudaStream_t s) {
    f = Fused();
    if(store == nullptr || p8)
      return true;   // not fusable for this model: the step falls back to one launch per matrix
    int i = 0;
    for(const Aff* a : parts) {
      if(i == 0) {
        f.n = a->N;
        f.K = a->K;
      } else if(a->N != f.n || a->K != f.K) {
        return true;
      }
      if(cudaMemcpyAsync(store + static_cast<size_t>(i) * f.n * f.K, a->bt, static_cast<size_t>(f.n) * f.K, cudaMemcpyDeviceToDevice, s) !=
         cudaSuccess)
        return false;
      f.qm[i] = a->qm;
      f.bias[i] = a->bias;
      ++i;
    }
    f.bt = store;
    f.nseg = i;
    f.ready = f.n % 128 == 0;
    return true;
  }

  // Looks every parameter up once and builds the fused matrices.  MI8_ERR_BAD_ARG names a missing parameter.
  int resolve(cudaStream_t s) {
    const mi8d_config& c = cfg;
    enc_w.assign(c.enc_depth, EncLayerW());
    dec_w.assign(c.dec_depth, DecLayerW());
    bool ok = true, copies = true;
    for(int l = 0; l < c.enc_depth; ++l) {
      EncLayerW& e = enc_w[l];
      const std::string pre = "encoder_l" + std::to_string(l + 1) + "_self", ffn = "encoder_l" + std::to_string(l + 1) + "_ffn";
      ok = ok && aff(e.q, pre + "_Wq", pre + "_bq") && aff(e.k, pre + "_Wk", pre + "_bk") && aff(e.v, pre + "_Wv", pre + "_bv") &&
           aff(e.o, pre + "_Wo", pre + "_bo") && aff(e.w1, ffn + "_W1", ffn + "_b1") && aff(e.w2, ffn + "_W2", ffn + "_b2") &&
           norm(e.ln_att, pre + "_Wo") && norm(e.ln_ffn, ffn + "_ffn");
      if(ok)
        copies = copies && fuse(e.qkv, fused_enc[l], {&e.q, &e.k, &e.v}, s);
    }
    for(int l = 0; l < c.dec_depth && ok; ++l) {
      DecLayerW& w = dec_w[l];
      const std::string li = "decoder_l" + std::to_string(l + 1);
      if(c.ssru) {
        const std::string pre = li + "_rnn";
        ok = ok && aff(w.rnn_w, pre + "_W", "") && aff(w.rnn_wf, pre + "_Wf", pre + "_bf") && norm(w.ln_self, pre + "_ffn");
        if(ok)
          copies = copies && fuse(w.rnn, fused_self[l], {&w.rnn_w, &w.rnn_wf}, s);
      } else {
        const std::string pre = li + "_self";
        ok = ok && aff(w.self_q, pre + "_Wq", pre + "_bq") && aff(w.self_k, pre + "_Wk", pre + "_bk") &&
             aff(w.self_v, pre + "_Wv", pre + "_bv") && aff(w.self_o, pre + "_Wo", pre + "_bo") && norm(w.ln_self, pre + "_Wo");
        if(ok)
          copies = copies && fuse(w.self_kv, fused_self[l], {&w.self_k, &w.self_v}, s);
      }
      const std::string pre = li + "_context", ffn = li + "_ffn";
      ok = ok && aff(w.ctx_q, pre + "_Wq", pre + "_bq") && aff(w.ctx_k, pre + "_Wk", pre + "_bk") && aff(w.ctx_v, pre + "_Wv", pre + "_bv") &&
           aff(w.ctx_o, pre + "_Wo", pre + "_bo") && norm(w.ln_ctx, pre + "_Wo") && aff(w.w1, ffn + "_W1", ffn + "_b1") &&
           aff(w.w2, ffn + "_W2", ffn + "_b2") && norm(w.ln_ffn, ffn + "_ffn");
      if(ok)
        copies = copies && fuse(w.ctx_kv, fused_ctx[l], {&w.ctx_k, &w.ctx_v}, s);
    }
    wemb = P("Wemb");
    ok = ok && wemb != nullptr && aff(out_w, p8 ? "Wemb_packed8" : "Wemb_intgemm8", "decoder_ff_logit_out_b");
    out_bias = out_w.bias;
    if(!ok)
      return MI8_ERR_BAD_ARG;
    if(!copies) {
      set_last_cuda_error(cudaGetLastError());
      return MI8_ERR_LAUNCH;
    }
    dirty = false;
    return MI8_OK;
  }
};

namespace {

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

// MI8D_OPT_GEMM_TILE_ROWS: the widest tile up to the option's value that M still fills more than half of (512 = the
// CTA-pair kernel, for more than 256 rows); 0 = leave the choice to the plan.
int wide_tile(const mi8d_decoder* d, int M) {
  int t = d->opt_gemm_tile;
  if(t <= 0 || M <= 16 || M > 1024)   // (encoder-sized products already fill the GPU: the plan's two-CTA kernel is the fastest there)
    return 0;
  if(t == 512 && M <= 256)
    t = 256;
  while(t > 32 && M <= t / 2)
    t >>= 1;
  return t;
}

// aq (already quantised, multiplier behind the data) x weight -> c
int gemm(mi8d_decoder* d, const int8_t* a, int M, const Aff& w, bool relu, float* c, cudaStream_t s, unsigned* absmax_out = nullptr,
         int force_splits = 0, int force_tile_m = 0) {
  const float* qa = reinterpret_cast<const float*>(a + static_cast<size_t>(M) * w.K);
  if(force_tile_m == 0 && w.N <= 8192 && wide_tile(d, M) != 0) {
    // several searches share the GPU: wider tiles on fewer SMs fetch every weight tile fewer times (throughput over latency)
    force_tile_m = wide_tile(d, M);
    force_splits = 1;
  }
  return launch_gemm(a, w.bt, M, w.N, w.K, qa, w.qm, 1.0f, w.bias, relu ? 1 : 0, c, MI8_F32, nullptr, d->ws, d->ws_bytes, s, force_tile_m,
                     force_splits, absmax_out);
}

// The narrowest tile (activation rows) that covers an M x N product with at most `budget` CTAs; 0 = leave it to the plan.
// Two GEMMs that run side by side on two streams each take half of the SMs this way (a CTA of this kernel fills an SM).
int tile_within(int M, int N, int budget) {
  if(M <= 64)
    return 0;
  for(int tm : {32, 64, 128, 256})
    if(((N + 127) / 128) * ((M + tm - 1) / tm) <= budget)
      return tm;
  return 0;
}

// the same activation against the matrices of a fused group, one launch; outs[i] receives [M, f.n]
int gemm_fused(mi8d_decoder* d, const int8_t* a, const float* qa, int M, const Fused& f, float* const* outs, cudaStream_t s,
               int force_splits = 0, int a_rows_cap = 0, int a_row0 = 0, const unsigned* skip_a = nullptr,
               const unsigned* skip_b = nullptr, int skip_rows_below = 0, int force_tile_m = 0) {
  GemmCall g;
  g.aq = a;
  g.bt = f.bt;
  g.M = M;
  g.N = f.nseg * f.n;
  g.K = f.K;
  g.d_qa = qa;
  g.nseg = f.nseg;
  for(int i = 0; i < f.nseg; ++i) {
    g.seg_qb[i] = f.qm[i];
    g.seg_bias[i] = f.bias[i];
    g.seg_c[i] = outs[i];
  }
  g.ws = d->ws;
  g.ws_bytes = d->ws_bytes;
  g.stream = s;
  g.force_splits = force_splits;
  g.force_tile_m = force_tile_m;
  g.a_rows_cap = a_rows_cap;
  g.a_row0 = a_row0;
  g.skip_a = skip_a;
  g.skip_b = skip_b;
  g.skip_rows_below = skip_rows_below;
  return launch_gemm_call(g);
}

// The activation quantisation of either scheme into `q`: intgemm8 - Int8::PrepareA with the multiplier 127 / max|x| from the
// slot the producer reduced (stored behind the data); packed8avx512 - uint8 per row with its own scale, zero point and sum
// (src/tensors/cpu/mjdgemm/mjdgemm_avx512.cpp:195-276), kept in the decoder's per-row arrays until the next quantisation.
int quantize_act(mi8d_decoder* d, const float* x, int M, int K, const unsigned* slot, int8_t* q, cudaStream_t s) {
  if(d->p8)
    return launch_p8_quantize_rows(x, M, K, reinterpret_cast<uint8_t*>(q), d->p8_scale_a, d->p8_zp_a, d->p8_sum_a, s);
  return launch_quantize_slot(x, static_cast<size_t>(M) * K, slot, q, reinterpret_cast<float*>(q + static_cast<size_t>(M) * K), s);
}

// ... and the product of that quantised activation with one weight
int gemm_act(mi8d_decoder* d, const int8_t* q, int M, const Aff& w, bool relu, float* c, cudaStream_t s, unsigned* absmax_out = nullptr,
             int force_splits = 0) {
  if(w.p8)
    return launch_gemm_p8(reinterpret_cast<const uint8_t*>(q), d->p8_scale_a, d->p8_zp_a, d->p8_sum_a, w.bt, w.scale_b, w.zp_b, w.off_b, M, w.N,
                          w.K, w.bias, relu ? 1 : 0, c, nullptr, d->ws, d->ws_bytes, s, 0, force_splits);
  return gemm(d, q, M, w, relu, c, s, absmax_out, force_splits);
}

// Int8::PrepareA of x (multiplier from the slot its producer reduced) followed by the affine: either the
// quantisation kernel and the GEMM, or - with the option set and a shape that gives every CTA one tile - the GEMM
// that quantises its operand while loading it.
int quant_gemm(mi8d_decoder* d, const float* x, int M, const unsigned* slot, const Aff& w, bool relu, float* c, cudaStream_t s,
               unsigned* absmax_out = nullptr) {
  float* qa = reinterpret_cast<float*>(d->aq + static_cast<size_t>(M) * w.K);
  if(!w.p8 && d->opt_cluster && M <= d->opt_cluster_max_rows && w.K <= d->opt_cluster_max_k && gemm_cq_supported(M, w.N, w.K, false)) {
    // the cluster GEMM: the CTAs of neighbouring weight tiles quantise the activation tile together (one launch, no int8 copy)
    CqCall g;
    g.a_f32 = x;
    g.a_slot = slot;
    g.bt = w.bt;
    g.d_qb = w.qm;
    g.M = M;
    g.N = w.N;
    g.K = w.K;
    g.bias = w.bias;
    g.relu = relu ? 1 : 0;
    g.c = c;
    g.absmax_out = absmax_out;
    g.force_cluster = d->opt_cluster_size;
    g.stream = s;
    return launch_gemm_cq(g);
  }
  if(!w.p8 && d->opt_quant_in_gemm && w.K <= 1024 && quant_a_tile(M, w.N) != 0)
    return launch_gemm_quant_a(x, slot, qa, w.bt, M, w.N, w.K, w.qm, 1.0f, w.bias, relu ? 1 : 0, c, MI8_F32, nullptr, s, absmax_out);
  MI8D_TRY(quantize_act(d, x, M, w.K, slot, d->aq, s));
  return gemm_act(d, d->aq, M, w, relu, c, s, absmax_out);
}

int add_ln(mi8d_decoder* d, const float* a, const float* resid, const Norm& n, int rows, float* out, float* rowmax, unsigned* slot,
           cudaStream_t s, unsigned* slot2 = nullptr) {
  return launch_add_layernorm(a, resid, n.g, n.b, 1e-6f, rows, d->cfg.dim_emb, out, rowmax, slot, s, slot2);
}

// out = LayerNorm(affine(x) + resid): the "dan" post-processing of a sub-layer's last affine (src/models/transformer.h:189-214).
// One launch when the row fits a cluster (the cluster GEMM's LayerNorm write-back), else affine (into `tmp`) and LayerNorm.
int quant_gemm_ln(mi8d_decoder* d, const float* x, int M, const unsigned* slot, const Aff& w, const float* resid, const Norm& n, float* tmp,
                  float* out, float* rowmax, unsigned* out_slot, cudaStream_t s, unsigned* out_slot2 = nullptr) {
  if(!w.p8 && d->opt_cluster && d->opt_fused_ln && M <= d->opt_cluster_max_rows && w.K <= d->opt_cluster_max_k && w.N == d->cfg.dim_emb &&
     gemm_cq_supported(M, w.N, w.K, true)) {
    CqCall g;
    g.a_f32 = x;
    g.a_slot = slot;
    g.bt = w.bt;
    g.d_qb = w.qm;
    g.M = M;
    g.N = w.N;
    g.K = w.K;
    g.bias = w.bias;
    g.ln = 1;
    g.ln_resid = resid;
    g.ln_gamma = n.g;
    g.ln_beta = n.b;
    g.ln_eps = 1e-6f;
    g.ln_out = out;
    g.ln_rowmax = rowmax;
    g.ln_slot = out_slot;
    g.ln_slot2 = out_slot2;
    g.stream = s;
    return launch_gemm_cq(g);
  }
  MI8D_TRY(quant_gemm(d, x, M, slot, w, false, tmp, s));
  return add_ln(d, tmp, resid, n, M, out, rowmax, out_slot, s, out_slot2);
}

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
  if(cfg->dec_depth > 16)
    return MI8_ERR_UNSUPPORTED;
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
    bool ok = cudaStreamCreateWithFlags(&d->side, cudaStreamNonBlocking) == cudaSuccess;
    for(cudaEvent_t* e : {&d->ev_fork, &d->ev_join})
      ok = ok && cudaEventCreateWithFlags(e, cudaEventDisableTiming) == cudaSuccess;
    d->overlap = ok;   // without them the step simply runs on the caller's stream alone
    if(!ok)
      cudaGetLastError();
  }
  if(cudaEventCreateWithFlags(&d->ev_step, cudaEventDisableTiming | cudaEventBlockingSync) != cudaSuccess) {
    d->ev_step = nullptr;
    cudaGetLastError();
  }
  *out = d;
  return MI8_OK;
}

void mi8d_destroy(mi8d_decoder* d) {
  if(d == nullptr)
    return;
  if(d->ev_step != nullptr)
    cudaEventDestroy(d->ev_step);
  if(d->side != nullptr) {
    cudaStreamSynchronize(d->side);
    cudaStreamDestroy(d->side);
  }
  for(cudaEvent_t e : {d->ev_fork, d->ev_join})
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
  d->dirty = true;
  return MI8_OK;
}

int mi8d_set_packed8_weight(mi8d_decoder* d, const char* name, const int8_t* bt, const float* scale_b, const int32_t* zp_b, const int32_t* off_b,
                            int K, int N) {
  if(d == nullptr || name == nullptr || bt == nullptr || scale_b == nullptr || zp_b == nullptr || off_b == nullptr || K <= 0 || N <= 0)
    return MI8_ERR_BAD_ARG;
  if(K % 16 != 0 || (reinterpret_cast<uintptr_t>(bt) & 15u))
    return MI8_ERR_MISALIGNED;
  P8Weight w;
  w.bt = bt;
  w.scale_b = scale_b;
  w.zp_b = zp_b;
  w.off_b = off_b;
  w.K = K;
  w.N = N;
  d->p8_weights[name] = w;
  d->p8 = true;
  d->dirty = true;
  return MI8_OK;
}

int mi8d_set_param(mi8d_decoder* d, const char* name, const float* p) {
  if(d == nullptr || name == nullptr || p == nullptr)
    return MI8_ERR_BAD_ARG;
  d->params[name] = p;
  d->dirty = true;
  return MI8_OK;
}

int mi8d_set_positions(mi8d_decoder* d, const float* table) {
  if(d == nullptr || table == nullptr)
    return MI8_ERR_BAD_ARG;
  d->positions = table;
  return MI8_OK;
}

int mi8d_set_option(mi8d_decoder* d, int option, int value) {
  if(d == nullptr && option != MI8D_OPT_ATTENTION_UNROLL && option != MI8D_OPT_ATTENTION_BLOCK_HEADS)
    return MI8_ERR_BAD_ARG;   // (the process-wide switches need no decoder)
  switch(option) {
    case MI8D_OPT_FUSE_WEIGHTS: d->opt_fuse = value != 0; break;
    case MI8D_OPT_QUANT_IN_GEMM: d->opt_quant_in_gemm = value != 0; break;
    case MI8D_OPT_FUSED_OUTPUT_MAX_ROWS: d->opt_fused_out_rows = value; break;
    case MI8D_OPT_SIDE_STREAM: d->opt_side_stream = value != 0; break;
    case MI8D_OPT_CLUSTER_AFFINE: d->opt_cluster = value != 0; break;
    case MI8D_OPT_FUSED_LAYERNORM: d->opt_fused_ln = value != 0; break;
    case MI8D_OPT_CLUSTER_MAX_ROWS: d->opt_cluster_max_rows = value; break;
    case MI8D_OPT_CLUSTER_SIZE:
      if(value != 0 && value != 1 && value != 2 && value != 4 && value != 8)
        return MI8_ERR_BAD_ARG;
      d->opt_cluster_size = value;
      break;
    case MI8D_OPT_CLUSTER_MAX_K: d->opt_cluster_max_k = value; break;
    case MI8D_OPT_BLOCKING_WAIT:
      if(value < 0 || value > 2)
        return MI8_ERR_BAD_ARG;
      d->opt_blocking_wait = value;
      break;
    case MI8D_OPT_GEMM_TILE_ROWS:
      if(value != 0 && value != 32 && value != 64 && value != 128 && value != 256 && value != 512)
        return MI8_ERR_BAD_ARG;
      d->opt_gemm_tile = value;
      break;
    case MI8D_OPT_ATTENTION_UNROLL:
      if(value != 8 && value != 16)
        return MI8_ERR_BAD_ARG;
      set_attention_unroll(value);
      break;
    case MI8D_OPT_ATTENTION_BLOCK_HEADS: set_attention_block_heads(value); break;
    default: return MI8_ERR_BAD_ARG;
  }
  return MI8_OK;
}

int mi8d_search_stats(mi8d_decoder* d, double out[4], int reset) {
  if(d == nullptr || out == nullptr)
    return MI8_ERR_BAD_ARG;
  out[0] = d->t_issue;
  out[1] = d->t_wait;
  out[2] = d->t_host;
  out[3] = d->n_steps;
  if(reset)
    d->t_issue = d->t_wait = d->t_host = d->n_steps = 0;
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
int mi8g_affine_slot(const float* a, const unsigned* absmax_slot, const int8_t* bt, const float* d_qb, int M, int N, int K,
                     float scale, const float* bias, int relu, float* c, unsigned* absmax_out, int tile_rows, int cluster,
                     void* stream) {
  CqCall g;
  g.a_f32 = a;
  g.a_slot = absmax_slot;
  g.bt = bt;
  g.d_qb = d_qb;
  g.M = M;
  g.N = N;
  g.K = K;
  g.scale = scale;
  g.bias = bias;
  g.relu = relu;
  g.c = c;
  g.absmax_out = absmax_out;
  g.force_tile_m = tile_rows;
  g.force_cluster = cluster;
  g.stream = as_stream(stream);
  return launch_gemm_cq(g);
}
int mi8g_affine_slot_add_layernorm(const float* a, const unsigned* absmax_slot, const int8_t* bt, const float* d_qb, int M,
                                   int N, int K, float scale, const float* bias, const float* resid, const float* gamma,
                                   const float* beta, float eps, float* out, float* rowmax, unsigned* out_slot,
                                   unsigned* out_slot2, void* stream) {
  CqCall g;
  g.a_f32 = a;
  g.a_slot = absmax_slot;
  g.bt = bt;
  g.d_qb = d_qb;
  g.M = M;
  g.N = N;
  g.K = K;
  g.scale = scale;
  g.bias = bias;
  g.ln = 1;
  g.ln_resid = resid;
  g.ln_gamma = gamma;
  g.ln_beta = beta;
  g.ln_eps = eps;
  g.ln_out = out;
  g.ln_rowmax = rowmax;
  g.ln_slot = out_slot;
  g.ln_slot2 = out_slot2;
  g.stream = as_stream(stream);
  return launch_gemm_cq(g);
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
  if(d->positions == nullptr)
    return MI8_ERR_BAD_ARG;
  cudaStream_t s = as_stream(stream);
  if(d->dirty)
    MI8D_TRY(d->resolve(s));
  const int dm = c.dim_emb, M = batch * src;
  const size_t n_d = static_cast<size_t>(M) * dm;
  cudaError_t e = cudaMemsetAsync(d->slots, 0, sizeof(unsigned) * d->n_slots, s);
  if(e == cudaSuccess)
    e = cudaMemcpyAsync(d->log_mask[0], log_mask, sizeof(float) * batch * src, cudaMemcpyDeviceToDevice, s);
  if(e != cudaSuccess) {
    set_last_cuda_error(e);
    return MI8_ERR_LAUNCH;
  }
  float* aq_tail = reinterpret_cast<float*>(d->enc_aq + n_d);
  // embeddings * sqrt(d) + positions 0..src-1 (src/models/transformer.h:93,110-114)
  float* x = d->enc_x[0];
  unsigned* x_slot = d->slots;
  MI8D_TRY(launch_embed(d->wemb, ids, d->positions, src, sqrtf(static_cast<float>(dm)), M, dm, x, nullptr, x_slot, s));
  for(int l = 0; l < c.enc_depth; ++l) {
    const EncLayerW& w = d->enc_w[l];
    unsigned *sa = d->enc_slot(l, 0), *s1 = d->enc_slot(l, 1), *s3 = d->enc_slot(l, 2);
    // q, keys and values are the same tensor: one quantisation serves the three projections, and with fused
    // weights one launch computes all three
    MI8D_TRY(quantize_act(d, x, M, dm, x_slot, d->enc_aq, s));
    if(d->opt_fuse && w.qkv.ready) {
      float* outs[3] = {d->enc_q, d->enc_k, d->enc_v};
      MI8D_TRY(gemm_fused(d, d->enc_aq, aq_tail, M, w.qkv, outs, s));
    } else {
      MI8D_TRY(gemm_act(d, d->enc_aq, M, w.q, false, d->enc_q, s));
      MI8D_TRY(gemm_act(d, d->enc_aq, M, w.k, false, d->enc_k, s));
      MI8D_TRY(gemm_act(d, d->enc_aq, M, w.v, false, d->enc_v, s));
    }
    float* a = d->enc_x[1];   // attention output, then reused as x1
    MI8D_TRY(launch_attention1(d->enc_q, d->enc_k, d->enc_v, d->log_mask[0], M, c.heads, dm / c.heads, src, batch, 2, a, sa, s));
    MI8D_TRY(quantize_act(d, a, M, dm, sa, d->enc_aq, s));
    MI8D_TRY(gemm_act(d, d->enc_aq, M, w.o, false, d->enc_q, s));
    MI8D_TRY(add_ln(d, d->enc_q, x, w.ln_att, M, a, nullptr, s1, s));                       // x1 = LN(Wo(a) + x)
    MI8D_TRY(quantize_act(d, a, M, dm, s1, d->enc_aq, s));
    MI8D_TRY(gemm_act(d, d->enc_aq, M, w.w1, true, d->enc_h, s, s3));                        // ReLU (and max|h|) in the write-back
    MI8D_TRY(quantize_act(d, d->enc_h, M, c.dim_ffn, s3, d->enc_aq, s));
    MI8D_TRY(gemm_act(d, d->enc_aq, M, w.w2, false, d->enc_q, s));
    const bool last = l + 1 == c.enc_depth;
    float* nx = last ? d->context[0] : x;                                                     // the last layer writes the context
    x_slot = d->enc_slot(l, 3);
    MI8D_TRY(add_ln(d, d->enc_q, a, w.ln_ffn, M, nx, nullptr, x_slot, s));
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
  if(d->positions == nullptr)
    return MI8_ERR_BAD_ARG;
  cudaStream_t s = as_stream(stream);
  if(d->dirty)
    MI8D_TRY(d->resolve(s));
  const int dm = c.dim_emb, S = d->src;
  const int SR = d->slab_rows;
  const size_t slab_stride = static_cast<size_t>(SR) * dm;
  const size_t n_d = static_cast<size_t>(R) * dm;

  MI8D_CUDA(cudaMemsetAsync(d->slots, 0, sizeof(unsigned) * d->n_slots, s));

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
    if(d->p8) {
      MI8D_TRY(quantize_act(d, ctx, batch * S, dm, nullptr, d->cq, s));
    } else {
      MI8D_TRY(launch_max_absolute(ctx, n, nullptr, cq_tail, d->ws, d->ws_bytes, s));
      MI8D_TRY(launch_quantize(ctx, n, cq_tail, d->cq, s));
    }
    for(int l = 0; l < c.dec_depth; ++l) {
      const DecLayerW& w = d->dec_w[l];
      if(d->opt_fuse && w.ctx_kv.ready) {
        float* outs[2] = {d->layers[l].cross_k, d->layers[l].cross_v};
        MI8D_TRY(gemm_fused(d, d->cq, cq_tail, batch * S, w.ctx_kv, outs, s));
      } else {
        MI8D_TRY(gemm_act(d, d->cq, batch * S, w.ctx_k, false, d->layers[l].cross_k, s));
        MI8D_TRY(gemm_act(d, d->cq, batch * S, w.ctx_v, false, d->layers[l].cross_v, s));
      }
    }
    d->cross_valid = true;
  }

  // Ancestor table of this step and, in the same launch, every layer's history abs-max over the earlier slabs; the
  // producer of a layer's newest slab (embedding / the previous layer's last LayerNorm) adds that slab's maximum.
  const int anc_new = d->anc_cur ^ 1;
  if(!c.ssru) {
    const float* rowmax[16];
    unsigned* hslot[16];
    for(int l = 0; l < c.dec_depth; ++l) {
      rowmax[l] = d->layers[l].rowmax;
      hslot[l] = d->layer_slot(l, kSlotHistory);
    }
    MI8D_TRY(launch_ancestors_update(d->anc[d->anc_cur], d->anc[anc_new], hyp_idx, t, R, SR, s, d->p8 ? 0 : c.dec_depth, rowmax, hslot));
  }

  // layer-0 input: scaled embedding of the previous word (zero at the first step) + position t
  float* x = c.ssru ? d->x_in : d->layers[0].slab + static_cast<size_t>(t) * slab_stride;
  float* x_rowmax = c.ssru ? nullptr : d->layers[0].rowmax + static_cast<size_t>(t) * SR;
  MI8D_TRY(launch_embed(d->wemb, t == 0 ? nullptr : prev_words, d->positions + static_cast<size_t>(t) * dm, 0, sqrtf(static_cast<float>(dm)), R,
                        dm, x, x_rowmax, d->input_slot(0), s, c.ssru ? nullptr : d->layer_slot(0, kSlotHistory)));

  const int cell_new = d->cell_cur ^ 1;
  float* aq_tail = reinterpret_cast<float*>(d->aq + n_d);
  for(int l = 0; l < c.dec_depth; ++l) {
    LayerBufs& L = d->layers[l];
    const DecLayerW& w = d->dec_w[l];
    unsigned* x_slot = d->input_slot(l);
    unsigned* s1 = d->layer_slot(l, kSlotSelfLn);
    if(c.ssru) {
      MI8D_TRY(quantize_act(d, x, R, dm, x_slot, d->aq, s));
      if(d->opt_fuse && w.rnn.ready) {
        float* outs[2] = {d->qbuf, d->fbuf};
        MI8D_TRY(gemm_fused(d, d->aq, aq_tail, R, w.rnn, outs, s));            // dot(input, W) and affine(input, Wf, bf)
      } else {
        MI8D_TRY(gemm_act(d, d->aq, R, w.rnn_w, false, d->qbuf, s));
        MI8D_TRY(gemm_act(d, d->aq, R, w.rnn_wf, false, d->fbuf, s));
      }
      MI8D_TRY(launch_ssru_cell(L.cell[d->cell_cur], t == 0 ? nullptr : hyp_idx, d->qbuf, d->fbuf, R, dm, L.cell[cell_new], d->abuf, s));
      MI8D_TRY(add_ln(d, d->abuf, x, w.ln_self, R, d->x1, nullptr, s1, s));
    } else if(d->p8) {
      // packed8avx512 quantises every ROW of an activation on its own, so the keys/values of earlier steps never change:
      // the newest slab is projected and stored, the rest is a plain key/value cache (what the reference recomputes from the
      // concatenated history, src/models/transformer.h:401-417, comes out identical row by row)
      unsigned* sa = d->layer_slot(l, kSlotSelfAtt);
      MI8D_TRY(quantize_act(d, x, R, dm, nullptr, d->aq, s));
      MI8D_TRY(gemm_act(d, d->aq, R, w.self_q, false, d->qbuf, s));
      MI8D_TRY(gemm_act(d, d->aq, R, w.self_k, false, L.kslab + static_cast<size_t>(t) * slab_stride, s));
      MI8D_TRY(gemm_act(d, d->aq, R, w.self_v, false, L.vslab + static_cast<size_t>(t) * slab_stride, s));
      MI8D_TRY(launch_attention1(d->qbuf, L.kslab, L.vslab, nullptr, R, c.heads, dm / c.heads, t + 1, batch, 0, d->abuf, sa, s, d->anc[anc_new],
                                 SR, SR));
      MI8D_TRY(quant_gemm_ln(d, d->abuf, R, sa, w.self_o, x, w.ln_self, d->obuf, d->x1, nullptr, s1, s));
    } else {
      unsigned* sh = d->layer_slot(l, kSlotHistory);
      unsigned* sa = d->layer_slot(l, kSlotSelfAtt);
      // Keys and values are projections of the WHOLE history of layer inputs, quantised with one multiplier over the
      // live part of that history.  The projections of earlier steps are kept per slab and stay valid as long as that
      // multiplier's abs-max does not change (compared bit for bit on the device): then only the newest slab is
      // quantised and projected, otherwise everything is.  One launch quantises the layer input twice - with its own
      // multiplier for the query projection and, as the newest history slab, with the history's.
      const int steps = t + 1;
      const int cap_rows = c.max_steps * c.max_rows;
      float* hq_tail = reinterpret_cast<float*>(L.hq + static_cast<size_t>(cap_rows) * dm);
      MI8D_TRY(launch_quantize_dual(x, n_d, x_slot, d->aq, aq_tail, L.slab, SR, steps, R, dm, sh, d->prev_bits + l, L.hq, hq_tail, s));
      const bool fused = d->opt_fuse && w.self_kv.ready;
      float* kv_new[2] = {L.kslab + static_cast<size_t>(t) * slab_stride, L.vslab + static_cast<size_t>(t) * slab_stride};
      float* kv_all[2] = {L.kslab, L.vslab};
      // The key/value projections do not depend on the query projection: they run on the internal stream beside it.  Both
      // sides then use tiles wide enough to fit half of the SMs each (a CTA of the GEMM fills an SM), so they really run
      // at the same time; no split-K on either side, the two streams must not share the workspace's counters.
      const bool side = d->overlap && d->opt_side_stream;
      cudaStream_t so = side ? d->side : s;
      const int half = sm_count() / 2;
      const int wide = wide_tile(d, R);
      const int tile_q = std::max(side ? tile_within(R, w.self_q.N, half) : 0, wide);
      const int tile_kv = std::max(side ? tile_within(R, 2 * w.self_k.N, half) : 0, wide);
      if(side) {
        MI8D_CUDA(cudaEventRecord(d->ev_fork, s));
        MI8D_CUDA(cudaStreamWaitEvent(so, d->ev_fork, 0));
      }
      if(t > 0) {
        // earlier slabs: recomputed only when the abs-max changed (all tiles skipped otherwise)
        if(fused) {
          MI8D_TRY(gemm_fused(d, L.hq, hq_tail, t * SR, w.self_kv, kv_all, so, 1, cap_rows, 0, d->prev_bits + l, sh, t * SR));
        } else {
          MI8D_TRY(launch_gemm(L.hq, w.self_k.bt, t * SR, w.self_k.N, w.self_k.K, hq_tail, w.self_k.qm, 1.0f, w.self_k.bias, 0, L.kslab, MI8_F32,
                               nullptr, d->ws, d->ws_bytes, so, 0, 1, nullptr, d->prev_bits + l, sh, t * SR));
          MI8D_TRY(launch_gemm(L.hq, w.self_v.bt, t * SR, w.self_v.N, w.self_v.K, hq_tail, w.self_v.qm, 1.0f, w.self_v.bias, 0, L.vslab, MI8_F32,
                               nullptr, d->ws, d->ws_bytes, so, 0, 1, nullptr, d->prev_bits + l, sh, t * SR));
        }
      }
      // newest slab: always projected, as a problem of its own (R live rows)
      if(fused) {
        MI8D_TRY(gemm_fused(d, L.hq, hq_tail, R, w.self_kv, kv_new, so, 1, cap_rows, t * SR, nullptr, nullptr, 0, tile_kv));
      } else {
        const int8_t* a_new = L.hq + static_cast<size_t>(t) * slab_stride;
        MI8D_TRY(launch_gemm(a_new, w.self_k.bt, R, w.self_k.N, w.self_k.K, hq_tail, w.self_k.qm, 1.0f, w.self_k.bias, 0, kv_new[0], MI8_F32,
                             nullptr, d->ws, d->ws_bytes, so, 0, 1));
        MI8D_TRY(launch_gemm(a_new, w.self_v.bt, R, w.self_v.N, w.self_v.K, hq_tail, w.self_v.qm, 1.0f, w.self_v.bias, 0, kv_new[1], MI8_F32,
                             nullptr, d->ws, d->ws_bytes, so, 0, 1));
      }
      if(side)
        MI8D_CUDA(cudaEventRecord(d->ev_join, so));
      MI8D_TRY(gemm(d, d->aq, R, w.self_q, false, d->qbuf, s, nullptr, side ? 1 : 0, tile_q));
      if(side)
        MI8D_CUDA(cudaStreamWaitEvent(s, d->ev_join, 0));
      MI8D_TRY(launch_attention1(d->qbuf, L.kslab, L.vslab, nullptr, R, c.heads, dm / c.heads, steps, batch, 0, d->abuf, sa, s,
                                 d->anc[anc_new], SR, SR));
      MI8D_TRY(quant_gemm_ln(d, d->abuf, R, sa, w.self_o, x, w.ln_self, d->obuf, d->x1, nullptr, s1, s));
    }
    {
      unsigned* sa = d->layer_slot(l, kSlotCtxAtt);
      unsigned* s2 = d->layer_slot(l, kSlotCtxLn);
      MI8D_TRY(quant_gemm(d, d->x1, R, s1, w.ctx_q, false, d->qbuf, s));
      MI8D_TRY(launch_attention1(d->qbuf, L.cross_k, L.cross_v, lmask, R, c.heads, dm / c.heads, S, batch, 1, d->abuf, sa, s));
      MI8D_TRY(quant_gemm_ln(d, d->abuf, R, sa, w.ctx_o, d->x1, w.ln_ctx, d->obuf, d->x2, nullptr, s2, s));

      unsigned* s3 = d->layer_slot(l, kSlotRelu);
      MI8D_TRY(quant_gemm(d, d->x2, R, s2, w.w1, true, d->hbuf, s, s3));   // ReLU and max|h| fused in the write-back

      // the block's output is the next layer's input: write it straight into that layer's history slab, and its
      // maximum into that layer's history abs-max as well
      const bool last = l + 1 == c.dec_depth;
      float* nx = last ? d->x_final : (c.ssru ? d->x_in : d->layers[l + 1].slab + static_cast<size_t>(t) * slab_stride);
      float* nx_rowmax = (last || c.ssru) ? nullptr : d->layers[l + 1].rowmax + static_cast<size_t>(t) * SR;
      unsigned* nx_hist = (last || c.ssru) ? nullptr : d->layer_slot(l + 1, kSlotHistory);
      MI8D_TRY(quant_gemm_ln(d, d->hbuf, R, s3, w.w2, d->x2, w.ln_ffn, d->obuf, nx, nx_rowmax, d->layer_slot(l, kSlotOut), s, nx_hist));
      x = nx;
    }
  }

  // tied output layer, then log-softmax + n-best per sentence over beam x vocabulary
  unsigned* x_slot = d->input_slot(c.dec_depth);
  MI8D_TRY(quantize_act(d, x, R, dm, x_slot, d->aq, s));
  // Up to opt_fused_out_rows rows the GEMM whose write-back reduces the 128-word blocks is faster than writing the logits
  // and reading them back; for greedy search the plain GEMM followed by the log-softmax / top-k kernel wins.
  const bool fused_output = !d->p8 && !d->keep_logits && R <= d->opt_fused_out_rows && n_best >= 2;
  if(!fused_output) {
    MI8D_TRY(gemm_act(d, d->aq, R, d->out_w, false, d->logits, s));
    MI8D_TRY(launch_lse_topk(d->logits, R, c.vocab, n_best, prev_scores, d->cand_score, d->cand_word, s));
  } else {
    // the GEMM's write-back reduces every 128-word block of a row; the logits never reach memory
    const int k_top = n_best <= 4 ? 4 : 8;
    MI8D_TRY(launch_gemm_logits(d->aq, aq_tail, d->out_w.bt, d->out_w.qm, R, c.vocab, dm, d->out_bias, 1.0f, k_top, d->blk_max, d->blk_sum,
                                d->blk_topv, d->blk_topi, nullptr, s));
    MI8D_TRY(launch_lse_merge(d->blk_max, d->blk_sum, d->blk_topv, d->blk_topi, R, c.vocab, k_top, n_best, prev_scores, d->cand_score,
                              d->cand_word, s));
  }
  MI8D_TRY(launch_nbest_merge(d->cand_score, d->cand_word, beam, batch, c.vocab, n_best, out_score, out_beam, out_word, s));

  if(!c.ssru && !d->p8)   // remember which abs-max the stored keys/values of every layer now belong to
    MI8D_TRY(launch_history_commit(d->prev_bits, d->slots, 1 + kSlotHistory, kSlotsPerLayer, c.dec_depth, d->reuse_stats, s));
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

  using clk = std::chrono::steady_clock;
  auto secs = [](clk::time_point a, clk::time_point b) { return std::chrono::duration<double>(b - a).count(); };
  clk::time_point mark = clk::now();
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
    const clk::time_point t_a = clk::now();
    rc = mi8d_step(d, hyp, pw, bidx, ps, tensor_beam, nb, n_best, o_score, o_beam, o_word, stream);
    if(rc != MI8_OK)
      return rc;
    MI8D_CUDA(cudaMemcpyAsync(d->h_out, d->s_out, static_cast<size_t>(3 * cells) * sizeof(int), cudaMemcpyDeviceToHost, s));
    const clk::time_point t_b = clk::now();
    if(d->opt_blocking_wait == 2 && d->ev_step != nullptr) {
      // several searches (and ranks) share the host's cores: poll, and hand the core to another thread between polls - as
      // quick as spinning while cores are free, fair when there are more waiting threads than cores
      MI8D_CUDA(cudaEventRecord(d->ev_step, s));
      cudaError_t qe;
      while((qe = cudaEventQuery(d->ev_step)) == cudaErrorNotReady)
        std::this_thread::yield();
      MI8D_CUDA(qe);
    } else if(d->opt_blocking_wait && d->ev_step != nullptr) {
      // sleep until the step's results have arrived (an interrupt wakes the thread: tens of microseconds later than polling)
      MI8D_CUDA(cudaEventRecord(d->ev_step, s));
      MI8D_CUDA(cudaEventSynchronize(d->ev_step));
    } else {
      MI8D_CUDA(cudaStreamSynchronize(s));
    }
    const clk::time_point t_c = clk::now();
    d->t_host += secs(mark, t_a);
    d->t_issue += secs(t_a, t_b);
    d->t_wait += secs(t_b, t_c);
    d->n_steps += 1;
    mark = t_c;
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
