/*
 * marian_i8_decode.h - C ABI of the decoder-step driver built on the int8 affine engine.
 *
 * One call runs the encoder, or a whole time step of Marian's transformer decoder on the device: what
 * DecoderTransformer::step builds as graph nodes (src/models/transformer.h:713-896) followed by the
 * log-softmax and n-best selection of BeamSearch::search (src/translator/beam_search.cpp:431-496).
 * Every affine goes through the int8 GEMM of marian_i8.h; the glue (embedding, LayerNorm, attention,
 * history handling, top-k) are sm_100a kernels of this library.  The beam bookkeeping stays with the
 * caller, exactly as in the reference: per step it uploads hypothesis indices / previous words /
 * path scores and downloads the n-best lists.
 *
 * Memory: the caller owns everything.  It passes one arena (mi8d_arena_bytes) for activations and
 * decoder state and one int8 workspace (mi8_workspace_bytes(0,0,0), zero-filled); parameters are
 * registered by pointer under Marian's parameter names and must stay alive.
 */
#ifndef MARIAN_I8_DECODE_H_
#define MARIAN_I8_DECODE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct mi8d_config {
  int dim_emb, dim_ffn, heads, enc_depth, dec_depth, vocab;   /* enc_depth 0: the caller supplies the encoder context */
  int ssru;        /* 0: self-attention decoder, 1: transformer-decoder-autoreg rnn with the SSRU cell */
  int max_rows;    /* beam * batch upper bound */
  int max_batch;   /* sentences per mini-batch upper bound */
  int max_steps;   /* target positions upper bound */
  int max_src;     /* source width upper bound */
} mi8d_config;

typedef struct mi8d_decoder mi8d_decoder;

/* Device bytes the arena must hold for this configuration. */
size_t mi8d_arena_bytes(const mi8d_config* cfg);
/* Creates the (host-side) driver object over caller-owned device memory. */
int mi8d_create(const mi8d_config* cfg, void* arena, size_t arena_bytes, void* workspace, size_t workspace_bytes,
                mi8d_decoder** out);
void mi8d_destroy(mi8d_decoder* d);

/* Registers an intgemm8 parameter (Bt[N,K] int8 followed by its fp32 multiplier) under Marian's name,
 * e.g. "decoder_l1_self_Wq"; "Wemb_intgemm8" is the quantised tied output matrix [vocab, dim_emb]. */
int mi8d_set_weight(mi8d_decoder* d, const char* name, const int8_t* bt, int K, int N);
/* Registers a packed8avx512 parameter under Marian's name: the row-major Bt[N,K] copy of its int8 matrix (mi8p_unpack_b)
 * and the per-column scale, zero point and column offset of the item's tail (src/tensors/cpu/fbgemm/packed_gemm.cpp:372-480).
 * A decoder that received one packed8avx512 weight runs EVERY affine through that scheme, as the reference does for a model
 * converted with marian-conv --gemm-type packed8avx512 (fbgemmPacked8Gemm -> mjdgemm::gemmInt8Packed,
 * src/tensors/cpu/fbgemm/packed_gemm.cpp:566-592): activations are quantised per row, so earlier keys/values of the decoder's
 * self-attention never change and are kept as a plain cache; the tied output matrix is registered as "Wemb_packed8"
 * (the conversion of Wemb^T [dim_emb, vocab]).  Mixing both kinds of weights is an error at the first step (MI8_ERR_BAD_ARG). */
int mi8d_set_packed8_weight(mi8d_decoder* d, const char* name, const int8_t* bt, const float* scale_b, const int32_t* zp_b,
                            const int32_t* off_b, int K, int N);
/* Registers a float32 parameter (biases, LayerNorm scale/bias, "Wemb", "decoder_ff_logit_out_b"). */
int mi8d_set_param(mi8d_decoder* d, const char* name, const float* p);
/* Sinusoidal position table [max_steps, dim_emb] (src/tensors/gpu/tensor_operators.cu:793-817). */
int mi8d_set_positions(mi8d_decoder* d, const float* table);

/* Starts a mini-batch: encoder context [batch, src, dim_emb] fp32 and log mask [batch, src]
 * ((1 - mask) * -99999999, src/models/transformer.h:138-143) are copied into the arena. */
int mi8d_start(mi8d_decoder* d, const float* context, const float* log_mask, int batch, int src, void* stream);

/* Runs the encoder on token ids [batch, src] (int32, device) with log mask [batch, src] and starts the
 * mini-batch with its output as the context (EncoderTransformer::apply, src/models/transformer.h:581-637);
 * needs enc_depth > 0 and the "encoder_l*" parameters registered. */
int mi8d_encode(mi8d_decoder* d, const int* ids, const float* log_mask, int batch, int src, void* stream);

/*
 * One decoder time step for beam * batch hypotheses (rows beam-major: row = beamHypIdx * batch + batchIdx).
 *   hyp_idx [beam*batch]    row of the previous step each hypothesis descends from   (NULL at the first step)
 *   prev_words [beam*batch] word each hypothesis ended in                            (NULL at the first step)
 *   batch_idx [batch]       previous-step batch positions of the sentences still active (NULL: unchanged)
 *   prev_scores [beam*batch] path scores (-inf for dummy slots); NULL = 0
 *   n_best                  candidates returned per sentence (Marian asks for the current beam width)
 * Outputs (device): out_score / out_beam / out_word [batch, n_best], sorted by descending path score.
 */
int mi8d_step(mi8d_decoder* d, const int* hyp_idx, const int* prev_words, const int* batch_idx, const float* prev_scores,
              int beam, int batch, int n_best, float* out_score, int* out_beam, int* out_word, void* stream);

/* Beam search over one mini-batch: the bookkeeping of BeamSearch::search (src/translator/beam_search.cpp:249-538,
 * hypothesis scoring src/translator/history.h:22-35) around mi8d_encode and mi8d_step, in C++ as in the reference.
 *   ids [batch, width] int32 and log_mask [batch, width] float on the device (as for mi8d_encode)
 *   out_tokens [batch, max_out] / out_len [batch] / out_score [batch] (optional) on the HOST: the best finished
 *   hypothesis of every sentence, EOS included, and its normalised score
 *   h2d_bytes / d2h_bytes (optional): bytes of per-step control words uploaded and n-best lists downloaded
 * One stream synchronisation per decoder step.  MI8_ERR_WORKSPACE if max_out is too small for a result. */
typedef struct mi8d_search_config {
  int beam;                  /* <= 8 */
  float max_length_factor;   /* stop at length >= factor * width */
  float normalize;           /* score / length^normalize */
  float word_penalty;
  int eos_id;
} mi8d_search_config;
int mi8d_search(mi8d_decoder* d, const int* ids, const float* log_mask, int batch, int width, const mi8d_search_config* cfg,
                int* out_tokens, int max_out, int* out_len, float* out_score, unsigned long long* h2d_bytes,
                unsigned long long* d2h_bytes, void* stream);

/* ---- the glue kernels on their own (what the driver sequences), exported for tests and for hosts that
 * build their own step.  All pointers are device pointers; `absmax_slot` is an optional 4-byte slot
 * (zeroed by the caller) into which the kernel reduces max|out| for a following mi8g_quantize_slot. ---- */

/* out[r,:] = wemb[words[r],:] * scale + pos[(pos_mod ? r % pos_mod : 0),:]; words NULL = zero embedding
 * (embedding scaling and sinusoidal positions, src/models/transformer.h:93,110-114). */
int mi8g_embed(const float* wemb, const int* words, const float* pos, int pos_mod, float scale, int rows, int dim,
               float* out, float* rowmax, unsigned* absmax_slot, void* stream);
/* out = gamma * (y - mean) / sqrt(var + eps) + beta with y = a + resid (resid may be NULL): the
 * "dan" post-processing (src/models/transformer.h:189-214, src/layers/generic.h:248-253). */
int mi8g_add_layernorm(const float* a, const float* resid, const float* gamma, const float* beta, float eps, int rows,
                       int dim, float* out, float* rowmax, unsigned* absmax_slot, void* stream);
/* One launch for "Int8::PrepareA + multiply + write-back" on decode shapes (the two lambda nodes of
 * src/tensors/cpu/intgemm_interface.h:17-32,46-99 together): `a` is the fp32 activation [M,K], `absmax_slot` the
 * device word holding the bit pattern of max|a| (as for mi8_multiply_f32_slot).  The CTAs of a thread-block cluster
 * work on neighbouring weight tiles of the same activation rows; each quantises a share of the activation tile and
 * stores it into the shared memory of all of them, so the fp32 values are read once per cluster.  c [M,N] fp32;
 * absmax_out (optional) receives max|c|.  K a multiple of 128 up to 4096, N a multiple of 128 (MI8_ERR_UNSUPPORTED
 * otherwise).  tile_rows (0, 32, 64, 128) and cluster (0, 1, 2, 4, 8) force the plan; 0 = chosen.  Bit-identical to
 * mi8g_quantize_slot + mi8_multiply_i8. */
int mi8g_affine_slot(const float* a, const unsigned* absmax_slot, const int8_t* bt, const float* d_qb, int M, int N, int K,
                     float scale, const float* bias, int relu, float* c, unsigned* absmax_out, int tile_rows, int cluster,
                     void* stream);
/* The same followed, in the same launch, by the transformer's "dan" post-processing of the result
 * (src/models/transformer.h:189-214): out = LayerNorm(affine(a) + resid) * gamma + beta, with the row maxima
 * (rowmax, optional) and max|out| (out_slot, out_slot2, optional) that mi8g_add_layernorm produces.  The cluster
 * spans the N / 128 <= 8 weight tiles of a row; the CTAs exchange per-row partial sums through distributed shared
 * memory.  Bit-identical to mi8g_affine_slot + mi8g_add_layernorm. */
int mi8g_affine_slot_add_layernorm(const float* a, const unsigned* absmax_slot, const int8_t* bt, const float* d_qb, int M,
                                   int N, int K, float scale, const float* bias, const float* resid, const float* gamma,
                                   const float* beta, float eps, float* out, float* rowmax, unsigned* out_slot,
                                   unsigned* out_slot2, void* stream);
/* Int8::PrepareA with the multiplier 127/max taken from an abs-max slot; writes the multiplier to d_quant_mult. */
int mi8g_quantize_slot(const float* x, size_t n, const unsigned* absmax_slot, int8_t* q, float* d_quant_mult, void* stream);
/* Single-query attention softmax(q.k/sqrt(dh) + mask).v (src/models/transformer.h:240-277); mode 0: decoder
 * self-attention over a time-major history [len, rows, dim]; 1: cross-attention over [batch, len, dim] with
 * rows beam-major; 2: encoder self-attention with rows ordered [batch, len]. */
int mi8g_attention1(const float* q, const float* k, const float* v, const float* log_mask, int rows, int heads,
                    int dim_head, int len, int batch, int mode, float* out, unsigned* absmax_slot, void* stream);
/* cand_score[r][j] = (j-th largest logit of row r - logsumexp(row r)) + prev_scores[r], cand_word[r][j]; k <= 8
 * (LogSoftmax + per-row part of the n-best search, src/translator/nth_element.cu:366-413). */
int mi8g_lse_topk(const float* logits, int rows, int vocab, int k, const float* prev_scores, float* cand_score,
                  int* cand_word, void* stream);
/* The output layer in two launches without logits in memory: the int8 GEMM of the quantised activation aq
 * [rows, K] (multiplier d_qa) with the quantised tied embedding matrix wq [vocab, K] (multiplier d_qw) reduces
 * value = float(acc) / (qa * qw) + bias[word] inside its write-back to, per (row, block of 128 words), the
 * block maximum, the block's sum of exponentials and its best entries; a second kernel combines the blocks.
 * Output as mi8g_lse_topk on the materialised logits, bit for bit.  scratch: mi8g_output_scratch_bytes()
 * bytes of device memory; logits_out (optional, [rows, vocab]) additionally receives the values (slow; for
 * checks).  (LogSoftmax + n-best of src/translator/beam_search.cpp:431-496 fused into the output affine.) */
size_t mi8g_output_scratch_bytes(int rows, int vocab);
int mi8g_output_topk(const int8_t* aq, const float* d_qa, const int8_t* wq, const float* d_qw, int rows, int vocab, int K,
                     const float* bias, int k, const float* prev_scores, void* scratch, size_t scratch_bytes, float* logits_out,
                     float* cand_score, int* cand_word, void* stream);

/* Per sentence: the k best of its beam x k row candidates, sorted; ties to the smaller (beam, word) key. */
int mi8g_nbest_merge(const float* cand_score, const int* cand_word, int beam, int batch, int vocab, int k,
                     float* out_score, int* out_beam, int* out_word, void* stream);

/* How often the stored self-attention keys/values could be kept: out[0] = (layer, step) pairs whose
 * history abs-max was bit-identical to the previous step's, out[1] = all pairs; reset != 0 clears the
 * counters.  Synchronises the device. */
int mi8d_history_reuse(mi8d_decoder* d, unsigned out[2], int reset);

/* Tuning switches of the step driver; every setting computes the same values, bit for bit.
 *   MI8D_OPT_FUSE_WEIGHTS (default 1): matrices that multiply the same activation (Wk|Wv of an attention block,
 *     Wq|Wk|Wv of an encoder layer, the SSRU's W|Wf) run as ONE GEMM launch over copies stored one behind the other;
 *   MI8D_OPT_QUANT_IN_GEMM (default 0): affines with K <= 1024 whose tiles fit one wave of CTAs quantise their
 *     activation while loading it (mi8_multiply_f32_slot) instead of through a quantisation launch;
 *   MI8D_OPT_FUSED_OUTPUT_MAX_ROWS (default 480): up to this many rows the output layer reduces its logits inside
 *     the GEMM's write-back, above it the logits are written and read back by the log-softmax / top-k kernel;
 *   MI8D_OPT_SIDE_STREAM (default 1): the re-projection of the earlier history slabs runs on an internal stream;
 *   MI8D_OPT_ATTENTION_UNROLL (8 or 16, default 8; process-wide): key/value rows a thread keeps in flight;
 *   MI8D_OPT_ATTENTION_BLOCK_HEADS (default 8, 0 = all; process-wide): heads one block of the decoder attention serves;
 *     a divisor of the head count splits every query row over several smaller blocks;
 *   MI8D_OPT_CLUSTER_AFFINE (default 0): affines whose activation comes with an abs-max slot run as ONE launch of the
 *     cluster GEMM (mi8g_affine_slot) instead of a quantisation launch and a GEMM launch.  Off by default: 74 to 98
 *     instead of 122 launches per step of the transformer-big decoder, but 5 to 20 % fewer tokens per second (the
 *     stores into the other CTAs' shared memory and the placement of whole clusters cost more than the launches saved);
 *   MI8D_OPT_FUSED_LAYERNORM (default 1; has an effect only with the above): the last affine of a sub-layer also applies the residual add and
 *     the LayerNorm that follow it (mi8g_affine_slot_add_layernorm) when the model width is at most 1024;
 *   MI8D_OPT_CLUSTER_MAX_ROWS (default 1024): activations with more rows than this take the two-launch route;
 *   MI8D_OPT_CLUSTER_SIZE (0 = chosen, 1, 2, 4, 8): CTAs per cluster of the plain cluster affine;
 *   MI8D_OPT_CLUSTER_MAX_K (default 2048): affines with a longer inner dimension take the two-launch route;
 *   MI8D_OPT_GEMM_TILE_ROWS (0 = the plan's choice, 32, 64, 128, 256, 512 = the two-CTA kernel): upper bound of the activation rows per
 *     tile of the decoder's plain affines (the widest tile that the live rows still fill more than half of is used).
 *     The plan spreads a small product over as many SMs as it can (lowest latency); when several searches share a GPU
 *     wider tiles on fewer SMs move fewer bytes from L2 for the same product;
 *   MI8D_OPT_BLOCKING_WAIT (default 0): how mi8d_search waits for a step's n-best lists.  0: cudaStreamSynchronize (spins on a
 *     core); 1: a blocking-sync event (the thread sleeps; woken tens of microseconds late: 5 % fewer tokens/s on one GPU);
 *     2: polls an event and yields the core between polls (for several searches per GPU and several GPUs per host). */
enum mi8d_option {
  MI8D_OPT_FUSE_WEIGHTS = 1,
  MI8D_OPT_QUANT_IN_GEMM = 2,
  MI8D_OPT_FUSED_OUTPUT_MAX_ROWS = 3,
  MI8D_OPT_SIDE_STREAM = 4,
  MI8D_OPT_ATTENTION_UNROLL = 5,
  MI8D_OPT_ATTENTION_BLOCK_HEADS = 6,
  MI8D_OPT_CLUSTER_AFFINE = 7,
  MI8D_OPT_FUSED_LAYERNORM = 8,
  MI8D_OPT_CLUSTER_MAX_ROWS = 9,
  MI8D_OPT_CLUSTER_SIZE = 10,
  MI8D_OPT_CLUSTER_MAX_K = 11,
  MI8D_OPT_GEMM_TILE_ROWS = 12,
  MI8D_OPT_BLOCKING_WAIT = 13
};
int mi8d_set_option(mi8d_decoder* d, int option, int value);   /* d may be NULL for the process-wide switches */

/* keep != 0: every step also writes its logits [beam*batch, vocab] (the output layer then runs unfused);
 * mi8d_last_logits returns them.  Off by default: the fused output layer never materialises them. */
int mi8d_keep_logits(mi8d_decoder* d, int keep);
/* Pointer to the last step's logits [beam*batch, vocab] (device); meaningful only with mi8d_keep_logits. */
const float* mi8d_last_logits(const mi8d_decoder* d);

#ifdef __cplusplus
}
#endif
#endif /* MARIAN_I8_DECODE_H_ */
