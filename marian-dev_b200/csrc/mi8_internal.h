// Internal declarations shared by the translation units of libmarian_i8.so.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/marian_i8.h"
#include "../../include/marian_i8_measure.h"

namespace mi8 {

// ------------------------------------------------------------------ workspace layout (bytes)
// [0, 256)            abs-max block counter (first 4 bytes) and reserved words
// [256, 16640)        split-K arrival counters, one uint32 per output tile
// [16640, 20736)      abs-max per-block partial maxima (1024 x uint32)
// [20736, ...)        split-K accumulation buffers, int32 [tile][column][128 rows]
// Everything except the abs-max partials must be zero between calls; kernels restore that.
constexpr size_t kWsOffAbsmaxCounter = 0;
constexpr size_t kWsOffTileCounters = 256;
constexpr int kWsMaxTileCounters = 4096;
constexpr size_t kWsOffAbsmaxPartials = kWsOffTileCounters + sizeof(uint32_t) * kWsMaxTileCounters;
constexpr int kWsMaxAbsmaxBlocks = 1024;
constexpr size_t kWsOffPartials = kWsOffAbsmaxPartials + sizeof(uint32_t) * kWsMaxAbsmaxBlocks;
constexpr size_t kWsHeaderBytes = kWsOffPartials;

// ------------------------------------------------------------------ per-thread error / launch bookkeeping
void set_last_cuda_error(cudaError_t e);
void count_launch();

// Device status word of the current device (address of a __device__ int, resolved once per device).
int* device_status_ptr();
int sm_count();

// Checks cudaGetLastError() after a launch; returns MI8_OK or MI8_ERR_LAUNCH.
int check_launch();

// ------------------------------------------------------------------ GEMM plan
struct GemmPlan {
  int tile_m;        // activation rows per tile (MMA N): 16, 32, 64, 128 or 256
  int pair;          // 1: CTA-pair kernel (256 weight rows x 256 activation rows per cluster of two CTAs)
  int stages;        // shared-memory pipeline depth
  int splits;        // split-K factor
  int n_tiles;       // tiles of 128 weight rows
  int m_tiles;       // tiles of tile_m activation rows
  int kb_total;      // 128-byte K blocks
  int kb_per_split;
  int grid;
  int smem_bytes;
  size_t partial_bytes;
};
int make_gemm_plan(int M, int N, int K, int force_tile_m, int force_splits, GemmPlan* plan);

// mi8_peak.cu: TOPS of a loop of this library's int8 MMAs alone (k_blocks 128-byte K blocks per SM).
int measure_int8_mma_peak(int k_blocks, float* tops_out, cudaStream_t stream);

int profile_begin(int max_records);
int profile_end(mi8_gemm_record* out, int capacity, int* count);

// quantisation kernels (mi8_quant.cu)
int launch_max_absolute(const float* x, size_t n, float* d_absmax, float* d_quant_mult, void* ws, size_t ws_bytes,
                        cudaStream_t stream);
int launch_quantize(const float* x, size_t n, const float* d_quant_mult, int8_t* q, cudaStream_t stream);
int launch_transpose_quantize(const float* w, int K, int N, const float* d_quant_mult, int8_t* bt, cudaStream_t stream);
int launch_transpose_f32(const float* in, int batch, int rows, int cols, float* out, cudaStream_t stream);

// GEMM (mi8_gemm.cu)
// absmax_out (optional): 4-byte slot that receives max|C| (unsigned bit pattern, atomicMax) for the
// quantisation of C as the next affine's input.
int launch_gemm(const int8_t* aq, const int8_t* bt, int M, int N, int K, const float* d_qa, const float* d_qb, float scale,
                const float* bias, int relu, void* c, int out_dtype, int32_t* acc_out, void* ws, size_t ws_bytes,
                cudaStream_t stream, int force_tile_m, int force_splits, unsigned* absmax_out = nullptr,
                const unsigned* skip_a = nullptr, const unsigned* skip_b = nullptr, int skip_rows_below = 0);

// The general form: one activation against up to three weight matrices of the same shape stored one behind the
// other (N = nseg * rows of one of them), each with its own multiplier, bias and output matrix [M, N / nseg].
struct GemmCall {
  const int8_t* aq = nullptr;
  const int8_t* bt = nullptr;
  int M = 0, N = 0, K = 0;
  const float* d_qa = nullptr;
  float scale = 1.0f;
  int relu = 0;
  int out_dtype = MI8_F32;
  int32_t* acc_out = nullptr;
  int nseg = 1;
  const float* seg_qb[3] = {nullptr, nullptr, nullptr};
  const float* seg_bias[3] = {nullptr, nullptr, nullptr};
  void* seg_c[3] = {nullptr, nullptr, nullptr};
  void* ws = nullptr;
  size_t ws_bytes = 0;
  cudaStream_t stream = nullptr;
  int force_tile_m = 0, force_splits = 0;
  unsigned* absmax_out = nullptr;
  const unsigned* skip_a = nullptr;
  const unsigned* skip_b = nullptr;
  int skip_rows_below = 0;
  int a_rows_cap = 0;   // rows the activation buffer holds (extent of its tensor map); 0 = M
  int a_row0 = 0;       // the M rows start at this row of the buffer `aq` points to (needs a_rows_cap >= a_row0 + M)
};
int launch_gemm_call(const GemmCall& g);

// Test hook behind mi8_test_wait_fault (marian_i8_measure.h).
void test_wait_fault(int withhold_item, unsigned spin_limit);

// The GEMM that quantises its activation itself: `a_f32` [M,K] fp32 and `a_slot`, the 4-byte slot its
// producer reduced max|A| into.  MI8_ERR_UNSUPPORTED when the shape does not give every CTA exactly one
// tile (quant_a_tile() == 0): the caller then quantises with a kernel of its own and calls launch_gemm.
int quant_a_tile(int M, int N);
int launch_gemm_quant_a(const float* a_f32, const unsigned* a_slot, float* qa_out, const int8_t* bt, int M, int N, int K,
                        const float* d_qb, float scale, const float* bias, int relu, void* c, int out_dtype, int32_t* acc_out,
                        cudaStream_t stream, unsigned* absmax_out = nullptr);

// The cluster GEMM for decode shapes: quantises the fp32 activation `a_f32` [M, K] itself with the multiplier of the abs-max
// slot `a_slot` (its CTAs share the quantised tile through distributed shared memory, so the fp32 values are read once
// per cluster), and with `ln` set writes LayerNorm(C + ln_resid) * ln_gamma + ln_beta (the arithmetic of
// add_layernorm_kernel, bit for bit) instead of C, with the row maxima and abs-max slots that kernel produces.
// gemm_cq_supported() says whether a shape can take this route (K a multiple of 128 up to 4096, N a multiple of 128;
// with `ln`: N <= 1024).
struct CqCall {
  const float* a_f32 = nullptr;
  const unsigned* a_slot = nullptr;
  float* qa_out = nullptr;
  const int8_t* bt = nullptr;
  const float* d_qb = nullptr;
  int M = 0, N = 0, K = 0;
  float scale = 1.0f;
  const float* bias = nullptr;
  int relu = 0;
  float* c = nullptr;
  unsigned* absmax_out = nullptr;
  int ln = 0;
  const float* ln_resid = nullptr;
  const float* ln_gamma = nullptr;
  const float* ln_beta = nullptr;
  float ln_eps = 0.0f;
  float* ln_out = nullptr;
  float* ln_rowmax = nullptr;
  unsigned* ln_slot = nullptr;
  unsigned* ln_slot2 = nullptr;
  cudaStream_t stream = nullptr;
  int force_tile_m = 0;     // 0 = chosen from M and N
  int force_cluster = 0;    // 0 = the largest of 8, 4, 2, 1 that divides N / 128 (ln: N / 128)
};
bool gemm_cq_supported(int M, int N, int K, bool ln);
int launch_gemm_cq(const CqCall& g);

// packed8avx512 scheme (mi8_packed8.cu, mi8_gemm.cu): weight item back to Bt[N,K]; per-row uint8 quantisation of
// the activation; uint8 x int8 GEMM whose write-back applies the zero points, the scales and the bias.
int launch_p8_prepare_b(const float* w, int K, int N, int8_t* packed, cudaStream_t stream);
int launch_p8_unpack_bt(const int8_t* packed, int K, int N, int8_t* bt, cudaStream_t stream);
int launch_p8_quantize_rows(const float* a, int M, int K, uint8_t* aq, float* scale_a, int32_t* zp_a, int32_t* sum_a, cudaStream_t stream);
int launch_gemm_p8(const uint8_t* aq, const float* scale_a, const int32_t* zp_a, const int32_t* sum_a, const int8_t* bt,
                   const float* scale_b, const int32_t* zp_b, const int32_t* off_b, int M, int N, int K, const float* bias, int relu,
                   float* c, int32_t* acc_out, void* ws, size_t ws_bytes, cudaStream_t stream, int force_tile_m, int force_splits);

// Output layer: GEMM whose write-back reduces every (row, block of 128 vocabulary entries) to its maximum, its sum
// of exponentials and its k_top (4 or 8) best entries (blk_* arrays: [rows][ceil(vocab/128)] (x k_top)); then
// launch_lse_merge turns those into the per-row candidates launch_lse_topk would have produced from the logits.
int launch_gemm_logits(const int8_t* aq, const float* d_qa, const int8_t* wq, const float* d_qw, int rows, int vocab, int K,
                       const float* bias, float scale, int k_top, float* blk_max, float* blk_sum, float* blk_topv, int* blk_topi,
                       float* logits_out, cudaStream_t stream);
int launch_lse_merge(const float* blk_max, const float* blk_sum, const float* blk_topv, const int* blk_topi, int rows, int vocab,
                     int k_top, int k, const float* prev_scores, float* cand_score, int* cand_word, cudaStream_t s);

// decode-step glue (mi8_glue.cu)
// slot2 (optional): a second 4-byte slot that receives the same maximum (the self-attention history's abs-max)
int launch_embed(const float* wemb, const int* words, const float* pos, int pos_mod, float scale, int rows, int dim, float* out,
                 float* rowmax, unsigned* slot, cudaStream_t s, unsigned* slot2 = nullptr);
int launch_add_layernorm(const float* a, const float* resid, const float* gamma, const float* beta, float eps, int rows, int dim,
                         float* out, float* rowmax, unsigned* slot, cudaStream_t s, unsigned* slot2 = nullptr);
int launch_quantize_slot(const float* x, size_t n, const unsigned* slot, int8_t* q, float* d_qm, cudaStream_t s);
// hist_layers > 0: also reduces, per layer, the maximum of rowmax over the earlier slabs' ancestor rows into hist_slot[l]
int launch_ancestors_update(const int* anc_old, int* anc_new, const int* hyp, int t, int rows, int stride, cudaStream_t s,
                            int hist_layers = 0, const float* const* hist_rowmax = nullptr, unsigned* const* hist_slot = nullptr);
// layer input x and the self-attention history quantised by one launch (see quantize_dual_kernel)
int launch_quantize_dual(const float* x, size_t n, const unsigned* slot_x, int8_t* q, float* qm_x, const float* slabs, int slab_rows,
                         int steps, int rows_new, int dim, const unsigned* slot_h, const unsigned* prev_bits, int8_t* hq, float* qm_h,
                         cudaStream_t s);
void set_attention_unroll(int u);
void set_attention_block_heads(int h);
// in-situ timeline: each translation unit with kernels installs the buffer in its own copy of the pointer
int trace_set_glue(unsigned long long* buf);
int trace_set_gemm(unsigned long long* buf);
int trace_set_quant(unsigned long long* buf);
int launch_history_commit(unsigned* prev_bits, const unsigned* slots, int first, int stride, int layers, unsigned* stats, cudaStream_t s);
int launch_attention1(const float* q, const float* k, const float* v, const float* log_mask, int rows, int heads, int dim_head,
                      int len, int batch, int mode, float* out, unsigned* slot, cudaStream_t s, const int* anc = nullptr,
                      int anc_stride = 0, int kv_rows = 0);
int launch_lse_topk(const float* logits, int rows, int vocab, int k, const float* prev_scores, float* cand_score, int* cand_word,
                    cudaStream_t s);
int launch_nbest_merge(const float* cand_score, const int* cand_word, int beam, int batch, int vocab, int k, float* out_score,
                       int* out_beam, int* out_word, cudaStream_t s);
int launch_gather_rows(const float* in, const int* idx, int rows, int dim, float* out, cudaStream_t s);
int launch_ssru_cell(const float* cell_old, const int* hyp, const float* xw, const float* f, int rows, int dim, float* cell_new,
                     float* h_out, cudaStream_t s);

// Whether kernels are launched with programmatic dependent launch (mi8_set_pdl; on by default).
bool pdl_enabled();
void set_pdl(bool on);

// Per-kernel device times (mi8_kernel_times_begin / _end): when on, every launch made through launch_kernel by
// the calling thread is bracketed by CUDA events on its stream and attributed to the kernel function.
bool kernel_times_on();
void kernel_times_before(const void* func, cudaStream_t stream);
void kernel_times_after(cudaStream_t stream);

// Launches `kernel` with or without the programmatic-stream-serialization attribute.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  if(kernel_times_on()) {
    kernel_times_before(reinterpret_cast<const void*>(kernel), stream);
    cudaLaunchConfig_t tcfg = {};
    tcfg.gridDim = grid;
    tcfg.blockDim = block;
    tcfg.dynamicSmemBytes = smem;
    tcfg.stream = stream;
    const cudaError_t te = cudaLaunchKernelEx(&tcfg, kernel, static_cast<KArgs>(args)...);   // no launch overlap while timing
    kernel_times_after(stream);
    return te;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline cudaStream_t as_stream(void* s) { return s ? reinterpret_cast<cudaStream_t>(s) : cudaStreamPerThread; }

}  // namespace mi8
