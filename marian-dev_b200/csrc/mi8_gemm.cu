// int8 x int8 -> int32 GEMM on the 5th-generation tensor cores (tcgen05, kind::i8) with TMEM
// accumulators, TMA-fed shared-memory ring and a fused dequantise + bias + ReLU epilogue.
//
// Orientation.  Marian's converted weight is Bt[N,K] (K contiguous) and the quantised activation
// is Aq[M,K] (K contiguous): both operands are K-major.  The kernel puts 128 rows of the WEIGHT on
// the MMA's M dimension (TMEM lanes) and a tile of `TM` activation rows on the MMA's N dimension
// (TMEM columns), i.e. it computes a tile of C^T.  Consequences:
//   * every weight byte is fetched from HBM exactly once per activation tile, whatever M is;
//   * skinny decode shapes (M = beam x batch) pick TM = 16..256 and waste no tensor work on padding;
//   * in the epilogue a thread owns one output column n and walks over rows m, so for a fixed m the
//     32 threads of a warp store 32 consecutive floats of C: fully coalesced without staging.
// When there are fewer tiles than SMs the K range is split across CTAs; every split adds its partial
// int32 accumulators into one buffer per tile in the workspace (red.global.add) and the last CTA to
// arrive reads the totals, zeroes the buffer again and runs the epilogue.  Integer addition is
// associative, so every split factor gives bit-identical accumulators.
//
// Roles inside a CTA of 320 threads: warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..9 = epilogue (two warps per TMEM lane quarter, alternating 32-column chunks).  Two TMEM
// accumulator buffers let the epilogue of one tile overlap the MMAs of the next.  CTAs are persistent
// over a static schedule.  The producer and MMA loops run warp-uniformly and issue from one elected lane.
//
// Variants in this file: the kernel that quantises its fp32 activation itself (kQuantA), the output-layer
// kernel whose write-back reduces every 128-word block to its maximum, sum of exponentials and best
// entries (kTopK), and the CTA-pair kernel (tcgen05.mma.cta_group::2, 256 x 256 tile per cluster of two
// CTAs) that the plan picks for large M.
#include <cfloat>
#include <cuda_fp16.h>

#include <vector>

#include "mi8_internal.h"
#include "mi8_math.cuh"
#include "mi8_ptx.cuh"

namespace mi8 {

namespace {

constexpr int kTileN = 128;     // weight rows per tile (MMA M)
constexpr int kTileKBytes = 128;  // K bytes per pipeline stage = one 128-byte swizzle row
constexpr int kMmaK = 32;       // K per tcgen05.mma kind::i8
constexpr int kThreads = 320;
constexpr int kEpilogueThreads = 256;
constexpr int kMaxStages = 8;
constexpr int kPairTileCode = 512;  // force_tile_m value that selects the CTA-pair kernel
constexpr int kMaxSegments = 3;

template <int TM>
struct TileCfg {
  static constexpr int kStages = TM == 256 ? 4 : (TM == 128 ? 6 : 8);
  static constexpr int kWBytes = kTileN * kTileKBytes;
  static constexpr int kABytes = TM * kTileKBytes;
  static constexpr int kStageBytes = kWBytes + kABytes;
  static constexpr int kAccStride = TM < 32 ? 32 : TM;  // TMEM columns between the two accumulators
  static constexpr int kTmemCols = 2 * kAccStride;
  static constexpr int kChunk = TM < 32 ? TM : 32;
};

struct Control {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  int abort;
  int is_last;
};

template <int TM>
constexpr int smem_bytes_for() {
  return TileCfg<TM>::kStages * TileCfg<TM>::kStageBytes + static_cast<int>(sizeof(Control)) + 1024;
}

struct GemmParams {
  int M, N, K;
  int n_tiles, m_tiles, splits, kb_total, kb_per_split, total_work;
  const float* d_qa;
  const float* d_qb;
  float scale;
  const float* bias;
  int relu;
  int out_f16;
  void* c;
  int32_t* acc_out;
  int32_t* partials;
  unsigned* tile_counters;
  unsigned* absmax_out;
  // output-layer variant (kTopK > 0): per (row, block of 128 columns) the block maximum, the block's sum of
  // exponentials and its kTopK largest values with their column indices, instead of (or besides) C
  float* lg_max;
  float* lg_sum;
  float* lg_topv;
  int* lg_topi;
  int lg_blocks;            // blocks of 128 columns per row
  float* lg_logits;         // optional [rows, columns] row-major copy of the values
  const float* a_f32;       // quantise-in-kernel variant: fp32 activation [M,K] and the 4-byte slot that
  const unsigned* a_slot;   // holds the bit pattern of max|A| (then aq / d_qa / the activation tensor map are unused)
  float* qa_out;            // optional: receives the activation multiplier 127 / max|A|
  const unsigned* skip_a;   // when both are set and *skip_a == *skip_b, tiles that lie entirely below
  const unsigned* skip_b;   // row skip_rows_below are not computed (their previous results still hold)
  int skip_rows_below;
  // packed8avx512 scheme (kP8): the activation is uint8 with a scale, zero point and row sum per ROW,
  // the weights int8 with a scale, zero point and column offset per COLUMN (d_qa / d_qb / scale unused)
  const float* p8_scale_a;
  const int32_t* p8_zp_a;
  const int32_t* p8_sum_a;
  const float* p8_scale_b;
  const int32_t* p8_zp_b;
  const int32_t* p8_off_b;
  int* status;
  // Several weight matrices of the same shape [seg_n, K] stored one behind the other and multiplied with the
  // same activation in one launch (Wk|Wv of an attention block, Wq|Wk|Wv of the encoder): segment s covers
  // weight rows [s * seg_n, (s + 1) * seg_n), has its own multiplier, bias and output matrix [M, seg_n].
  // seg_n is a multiple of 128, so a tile never straddles two segments.  nseg == 1: the plain call
  // (seg_n = N, seg_qb[0] = d_qb, seg_bias[0] = bias, seg_c[0] = c).
  int nseg, seg_n;
  const float* seg_qb[kMaxSegments];
  const float* seg_bias[kMaxSegments];
  void* seg_c[kMaxSegments];
  int a_row0;               // first row of the activation inside its tensor map (a slab of a larger buffer)
  int* rows_computed;       // optional (measurement): receives the number of activation rows this launch really computed
  int withhold_item;        // test hook: the producer leaves out the loads of this pipeline item (-1 = none)
  uint32_t spin_limit;      // bound of every barrier wait of this launch
};

struct WorkItem {
  int tile, split, n_tile, m_tile, kb_begin, kb_end;
};

__device__ __forceinline__ WorkItem decode_work(const GemmParams& p, int w) {
  WorkItem it;
  it.split = w % p.splits;
  it.tile = w / p.splits;
  it.n_tile = it.tile % p.n_tiles;
  it.m_tile = it.tile / p.n_tiles;
  it.kb_begin = it.split * p.kb_per_split;
  it.kb_end = min(p.kb_total, it.kb_begin + p.kb_per_split);
  return it;
}

__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

template <int N>
__device__ __forceinline__ void tmem_ld_chunk(uint32_t taddr, int32_t (&v)[N]);
template <>
__device__ __forceinline__ void tmem_ld_chunk<16>(uint32_t taddr, int32_t (&v)[16]) { tmem_ld_x16(taddr, v); }
template <>
__device__ __forceinline__ void tmem_ld_chunk<32>(uint32_t taddr, int32_t (&v)[32]) { tmem_ld_x32(taddr, v); }

// Int8::PrepareA on four values: round-to-nearest-even of x * qm, saturated to +-127, packed little-endian.
__device__ __forceinline__ unsigned pack4_i8(const float4& v, float qm) {
  const int a = max(-127, min(127, __float2int_rn(__fmul_rn(v.x, qm))));
  const int b = max(-127, min(127, __float2int_rn(__fmul_rn(v.y, qm))));
  const int c = max(-127, min(127, __float2int_rn(__fmul_rn(v.z, qm))));
  const int d = max(-127, min(127, __float2int_rn(__fmul_rn(v.w, qm))));
  return (static_cast<unsigned>(a) & 0xffu) | ((static_cast<unsigned>(b) & 0xffu) << 8) | ((static_cast<unsigned>(c) & 0xffu) << 16) |
         ((static_cast<unsigned>(d) & 0xffu) << 24);
}

// Dequantises one register chunk of accumulators of output column n (CH consecutive rows m starting at
// element `base` of C, of which `valid` exist; `valid` may exceed CH) and stores it:
// float(acc) * unquant (+ bias) as two separately rounded operations, then ReLU.  Each stage runs over
// the whole chunk so the columns overlap in the pipeline.  Returns the running max|C| bit pattern.
template <int CH>
__device__ __forceinline__ unsigned write_back_chunk(const GemmParams& p, const int32_t (&v)[CH], size_t base, int valid, float unquant,
                                                     float bias_n, unsigned out_max, void* c, int ldc, bool has_bias) {
  float f[CH];
#pragma unroll
  for(int j = 0; j < CH; ++j)
    f[j] = __fmul_rn(__int2float_rn(v[j]), unquant);
  if(has_bias) {
#pragma unroll
    for(int j = 0; j < CH; ++j)
      f[j] = __fadd_rn(f[j], bias_n);
  }
  if(p.relu) {
#pragma unroll
    for(int j = 0; j < CH; ++j)
      f[j] = f[j] > 0.0f ? f[j] : 0.0f;
  }
  if(p.absmax_out != nullptr) {
#pragma unroll
    for(int j = 0; j < CH; ++j)
      if(j < valid)
        out_max = max(out_max, __float_as_uint(f[j]) & 0x7fffffffu);
  }
  if(p.acc_out != nullptr) {   // (single-segment launches only: ldc == N)
    int32_t* dst = p.acc_out + base;
#pragma unroll
    for(int j = 0; j < CH; ++j)
      if(j < valid)
        dst[static_cast<size_t>(j) * ldc] = v[j];
  }
  if(p.out_f16) {
    __half* dst = reinterpret_cast<__half*>(c) + base;
#pragma unroll
    for(int j = 0; j < CH; ++j)
      if(j < valid)
        dst[static_cast<size_t>(j) * ldc] = __float2half_rn(f[j]);
  } else {
    float* dst = reinterpret_cast<float*>(c) + base;
    if(valid >= CH) {
#pragma unroll
      for(int j = 0; j < CH; ++j)
        dst[static_cast<size_t>(j) * ldc] = f[j];
    } else {
#pragma unroll
      for(int j = 0; j < CH; ++j)
        if(j < valid)
          dst[static_cast<size_t>(j) * ldc] = f[j];
    }
  }
  return out_max;
}

// Write-back of the packed8avx512 scheme (marian::cpu::mjdgemm dequantizeAndAdd, AVX-512 route,
// src/tensors/cpu/mjdgemm/mjdgemm_avx512.cpp:290-322): the thread owns weight column n, v[j] is the
// accumulator of activation row m_first + j.
//   xv = acc - zeroPointA[m] * colOffsetsB[n] - zeroPointB[n] * sumA[m]      (int32, wrapping)
//   out = (scaleA[m] * scaleB[n]) * float(xv), and with a bias one fused multiply-add of the same product,
// which is what the reference computes once GCC has contracted its multiply and add.
__device__ __forceinline__ float p8_value(int acc, int zp_a, int sum_a, float scale_a, float scale_b, int zp_b, int off_b, bool has_bias,
                                          float bias_n, int relu) {
  const unsigned xv = static_cast<unsigned>(acc) - static_cast<unsigned>(zp_a) * static_cast<unsigned>(off_b)
                      - static_cast<unsigned>(zp_b) * static_cast<unsigned>(sum_a);
  const float scale = __fmul_rn(scale_a, scale_b);
  const float xf = __int2float_rn(static_cast<int>(xv));
  float r = has_bias ? __fmaf_rn(scale, xf, bias_n) : __fmul_rn(scale, xf);
  if(relu)
    r = r > 0.0f ? r : 0.0f;
  return r;
}

// The per-row parameters of four consecutive activation rows come in with one 16-byte load per array
// (m_first is a multiple of 16 and the arrays are 16-byte aligned; a warp reads the same address, so each
// load is one broadcast transaction); the ragged last chunk of a tile takes the element-wise path.
template <int CH>
__device__ __forceinline__ void write_back_chunk_p8(const GemmParams& p, const int32_t (&v)[CH], size_t base, int valid, int m_first, float scale_b,
                                                    int zp_b, int off_b, float bias_n) {
  float* dst = reinterpret_cast<float*>(p.c) + base;
  int32_t* acc_dst = p.acc_out != nullptr ? p.acc_out + base : nullptr;
  const bool has_bias = p.bias != nullptr;
  if(valid >= CH) {
#pragma unroll
    for(int j = 0; j < CH; j += 4) {
      const int4 za = __ldg(reinterpret_cast<const int4*>(p.p8_zp_a + m_first + j));
      const int4 su = __ldg(reinterpret_cast<const int4*>(p.p8_sum_a + m_first + j));
      const float4 sa = __ldg(reinterpret_cast<const float4*>(p.p8_scale_a + m_first + j));
      dst[static_cast<size_t>(j + 0) * p.N] = p8_value(v[j + 0], za.x, su.x, sa.x, scale_b, zp_b, off_b, has_bias, bias_n, p.relu);
      dst[static_cast<size_t>(j + 1) * p.N] = p8_value(v[j + 1], za.y, su.y, sa.y, scale_b, zp_b, off_b, has_bias, bias_n, p.relu);
      dst[static_cast<size_t>(j + 2) * p.N] = p8_value(v[j + 2], za.z, su.z, sa.z, scale_b, zp_b, off_b, has_bias, bias_n, p.relu);
      dst[static_cast<size_t>(j + 3) * p.N] = p8_value(v[j + 3], za.w, su.w, sa.w, scale_b, zp_b, off_b, has_bias, bias_n, p.relu);
    }
  } else {
#pragma unroll
    for(int j = 0; j < CH; ++j)
      if(j < valid) {
        const int m = m_first + j;
        dst[static_cast<size_t>(j) * p.N] = p8_value(v[j], __ldg(p.p8_zp_a + m), __ldg(p.p8_sum_a + m), __ldg(p.p8_scale_a + m), scale_b, zp_b,
                                                     off_b, has_bias, bias_n, p.relu);
      }
  }
  if(acc_dst != nullptr) {
#pragma unroll
    for(int j = 0; j < CH; ++j)
      if(j < valid)
        acc_dst[static_cast<size_t>(j) * p.N] = v[j];
  }
}

// kQuantA: the activation arrives as fp32 plus the abs-max slot its producer reduced; the eight epilogue
// warps quantise the tile's rows (Int8::PrepareA: round(x * 127/max) saturated to +-127) straight into the
// shared-memory ring in the 128-byte-swizzled K-major layout the MMA reads, so no int8 copy of the
// activation and no quantisation launch exist.  Used when every CTA has one tile (they quantise before
// their write-back work begins).
// kTopK > 0 (the output layer, operands swapped by the host: the M-side tile holds 128 ACTIVATION rows, the
// N-side tile 256 rows of the tied embedding matrix): a thread owns one query row and 128 consecutive
// vocabulary entries of it per tile, so it can reduce them on its own - block maximum, sum of exponentials
// in ascending order, the kTopK best entries - and the [rows, vocabulary] logits never reach memory.
template <int TM, bool kQuantA, int kTopK = 0, bool kP8 = false>
__global__ void __launch_bounds__(kThreads, 1)
mi8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a, const GemmParams p) {
  using T = TileCfg<TM>;
  constexpr int kConvWarps = kEpilogueThreads / 32;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzled tiles must start on a 1024-byte boundary.
  const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  uint8_t* tiles = smem_raw + pad;
  Control* ctl = reinterpret_cast<Control*>(tiles + T::kStages * T::kStageBytes);
  volatile int* abort_flag = &ctl->abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  pdl_launch_dependents();  // the next kernel on the stream may begin its own set-up now
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  constexpr int kTraceId = kTopK > 0 ? kTrGemmLogits : (kQuantA ? kTrGemmQuantA : kTrGemm);
  const unsigned long long trace_extra = static_cast<unsigned long long>(p.N) | (static_cast<unsigned long long>(p.K) << 20) |
                                         (static_cast<unsigned long long>(p.M) << 40);
  if(threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_a);
    for(int s = 0; s < T::kStages; ++s) {
      mbar_init(&ctl->full[s], kQuantA ? 1 + kConvWarps : 1);   // producer (+ one arrival per quantising warp)
      mbar_init(&ctl->empty[s], 1);
    }
    for(int b = 0; b < 2; ++b) {
      mbar_init(&ctl->tmem_full[b], 1);
      mbar_init(&ctl->tmem_empty[b], kEpilogueThreads);
    }
    mbar_init(&ctl->drain, 1);
    ctl->abort = 0;
    ctl->is_last = 0;
    fence_mbar_init();
  }
  if(warp == 1) {
    tmem_alloc(&ctl->tmem_base, T::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);

  bool ok = true;

  if(warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // The weights do not depend on the previous kernel: the weight tiles of the first pipeline fill
    // are requested before waiting for it, the activation tiles (its output) after.
    uint32_t it = 0;
    uint32_t prefetched = 0;  // stages whose weight tile is already in flight
    if(p.skip_a == nullptr && kTopK == 0 && p.withhold_item < 0) {   // (output-layer variant: the M-side operand is the activation, nothing to prefetch)
      const WorkItem w0 = decode_work(p, blockIdx.x);
      const int n_pre = min(T::kStages, w0.kb_end - w0.kb_begin);
      if(elect_one()) {
        for(int i = 0; i < n_pre; ++i) {
          uint8_t* st = tiles + i * T::kStageBytes;
          mbar_arrive_expect_tx(&ctl->full[i], kQuantA ? T::kWBytes : T::kStageBytes);
          tma_load_2d(st, &tmap_w, (w0.kb_begin + i) * kTileKBytes, w0.n_tile * kTileN, &ctl->full[i]);
        }
      }
      __syncwarp();
      prefetched = n_pre;
    }
    pdl_wait();
    const bool skip_on = p.skip_a != nullptr && *p.skip_a == *p.skip_b;
    if(p.rows_computed != nullptr && blockIdx.x == 0 && lane == 0)
      *p.rows_computed = p.M - (skip_on ? min(p.M, (p.skip_rows_below / TM) * TM) : 0);
    for(int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x) {
      const WorkItem wi = decode_work(p, w);
      if(skip_on && (wi.m_tile + 1) * TM <= p.skip_rows_below)
        continue;
      for(int kb = wi.kb_begin; kb < wi.kb_end; ++kb, ++it) {
        const uint32_t s = it % T::kStages;
        const uint32_t ph = (it / T::kStages) & 1u;
        const bool pre = it < prefetched;
        if(!pre)
          ok = mbar_wait_bounded(&ctl->empty[s], ph ^ 1u, abort_flag, p.spin_limit);   // every lane polls: the branch stays warp-uniform
        ok = __all_sync(0xffffffffu, ok);
        if(!ok)
          break;
        // (test hook: a withheld item's operands never arrive, so the roles that wait for them run out of patience)
        if(elect_one() && static_cast<int>(it) != p.withhold_item) {
          uint8_t* st = tiles + s * T::kStageBytes;
          if(!pre) {
            mbar_arrive_expect_tx(&ctl->full[s], kQuantA ? T::kWBytes : T::kStageBytes);
            tma_load_2d(st, &tmap_w, kb * kTileKBytes, wi.n_tile * kTileN, &ctl->full[s]);
          }
          if(!kQuantA)
            tma_load_2d(st + T::kWBytes, &tmap_a, kb * kTileKBytes, p.a_row0 + wi.m_tile * TM, &ctl->full[s]);
        }
        __syncwarp();
      }
    }
    if(!ok) {
      *abort_flag = 1;
      if(lane == 0) {
        atomicMax(p.status, static_cast<int>(kDevTimeoutProducer));
        // Wait (bounded) for the copies already issued, so none lands after the CTA has gone.
        const uint32_t first = it > static_cast<uint32_t>(T::kStages) ? it - T::kStages : 0u;
        int no_abort = 0;
        for(uint32_t j = first; j < it; ++j)
          mbar_wait_bounded(&ctl->full[j % T::kStages], (j / T::kStages) & 1u, &no_abort, p.spin_limit);
      }
      __syncwarp();
    }
  } else if(warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = kP8 ? make_idesc_i8_ub(TM) : make_idesc_i8(TM);
    uint32_t it = 0, acc_it = 0;
    // No MMA can be issued before the activation tiles arrive, and those are requested after the producer's
    // pdl_wait(): waiting here as well costs nothing and keeps the predecessor's run time out of the bounded
    // waits below (it also orders the read of the skip words, which earlier kernels of the stream write).
    pdl_wait();
    const bool skip_on = p.skip_a != nullptr && *p.skip_a == *p.skip_b;
    for(int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x) {
      const WorkItem wi = decode_work(p, w);
      if(skip_on && (wi.m_tile + 1) * TM <= p.skip_rows_below)
        continue;
      const uint32_t as = acc_it & 1u;
      const uint32_t aph = (acc_it >> 1) & 1u;
      // The whole warp walks the loop and polls the barriers, so every value below is warp-uniform;
      // one elected lane issues the MMAs and commits.
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctl->tmem_empty[as], aph ^ 1u, abort_flag, p.spin_limit));
      if(!ok)
        break;
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + as * T::kAccStride;
      for(int kb = wi.kb_begin; kb < wi.kb_end; ++kb, ++it) {
        const uint32_t s = it % T::kStages;
        const uint32_t ph = (it / T::kStages) & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctl->full[s], ph, abort_flag, p.spin_limit));
        if(!ok)
          break;
        tc_fence_after_sync();
        const uint32_t w_addr = smem_u32(tiles + s * T::kStageBytes);
        const uint32_t a_addr = w_addr + T::kWBytes;
        if(elect_one()) {
#pragma unroll
          for(int k = 0; k < kTileKBytes / kMmaK; ++k) {
            tc_mma_i8(d_tmem, make_kmajor_sw128_desc(w_addr + k * kMmaK), make_kmajor_sw128_desc(a_addr + k * kMmaK), idesc,
                      (kb > wi.kb_begin || k > 0) ? 1u : 0u);
          }
          tc_commit(&ctl->empty[s]);  // frees the smem slot once these MMAs have read it
        }
        __syncwarp();
      }
      if(!ok)
        break;
      if(elect_one())
        tc_commit(&ctl->tmem_full[as]);  // accumulator complete
      __syncwarp();
      ++acc_it;
    }
    if(!ok) {
      *abort_flag = 1;
      if(lane == 0)
        atomicMax(p.status, static_cast<int>(kDevTimeoutMma));
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    // A warp may only read the TMEM lane quarter (warp % 4); two warps share each quarter and take
    // alternate 32-column chunks, so every scheduler has two epilogue warps to hide latency with.
    const int quarter = warp & 3;
    const int group = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int epi_tid = threadIdx.x - 64;
    constexpr int kChunks = TM / T::kChunk;
    constexpr int kChunkStep = kChunks > 1 ? 2 : 1;
    const bool has_chunks = kChunks > 1 || group == 0;
    pdl_wait();  // the activation multiplier (or abs-max slot) is written by the previous kernel
    trace_stamp_start(th, kTraceId, trace_extra);
    // kQuantA: the multiplier comes from the abs-max slot, which is read only after the first fp32 loads of the
    // activation have been issued (below), so the two round trips to L2 overlap instead of following one another.
    float qa = 1.0f;
    bool qa_ready = !kQuantA;
    if(!kQuantA && !kP8)
      qa = *p.d_qa;
    float unquant = (kP8 || kQuantA) ? 1.0f : __fmul_rn(__fdiv_rn(1.0f, __fmul_rn(qa, *p.seg_qb[0])), p.scale);
    uint32_t acc_it = 0;
    uint32_t conv_it = 0;
    const bool skip_on = p.skip_a != nullptr && *p.skip_a == *p.skip_b;
    for(int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x) {
      const WorkItem wi = decode_work(p, w);
      if(skip_on && (wi.m_tile + 1) * TM <= p.skip_rows_below)
        continue;
      if(kQuantA) {
        // Quantise this tile's activation rows, one 128-byte K block per pipeline stage.  A thread
        // converts 16 consecutive K values (four 16-byte loads) into one 16-byte chunk and stores it where
        // the 128-byte swizzle puts chunk c of row r: byte r * 128 + ((c ^ (r & 7)) << 4) of the tile.
        // The fp32 loads of several K blocks are issued together (they do not depend on the ring), so a
        // tile costs about one L2 round trip per batch instead of one per K block.
        constexpr int kCpt = (TM * 8 + kEpilogueThreads - 1) / kEpilogueThreads;   // chunks per thread and K block
        constexpr int kBatch = 8 / kCpt;   // 32 16-byte loads in flight per thread: all of K = 1024 in one round trip
        for(int kb0 = wi.kb_begin; kb0 < wi.kb_end && ok; kb0 += kBatch) {
          float4 f[kBatch][kCpt][4];
#pragma unroll
          for(int b = 0; b < kBatch; ++b) {
#pragma unroll
            for(int q = 0; q < kCpt; ++q) {
              const int c = epi_tid + q * kEpilogueThreads;
              const int gm = wi.m_tile * TM + (c >> 3);
              const int gk = (kb0 + b) * kTileKBytes + (c & 7) * 16;
              const bool in = c < TM * 8 && kb0 + b < wi.kb_end && gm < p.M && gk < p.K;   // K % 16 == 0: whole chunk in or out
              const float4* src = reinterpret_cast<const float4*>(p.a_f32 + static_cast<size_t>(in ? gm : 0) * p.K + (in ? gk : 0));
#pragma unroll
              for(int e = 0; e < 4; ++e)
                f[b][q][e] = in ? src[e] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
          }
          if(!qa_ready) {
            const unsigned bits = *p.a_slot;
            qa = bits == 0u ? 1.0f : __fdiv_rn(127.0f, __uint_as_float(bits));
            unquant = __fmul_rn(__fdiv_rn(1.0f, __fmul_rn(qa, *p.seg_qb[0])), p.scale);
            if(blockIdx.x == 0 && epi_tid == 0) {
              if(p.qa_out != nullptr)
                *p.qa_out = qa;
              if(bits >= 0x7f800000u)
                atomicMax(p.status, static_cast<int>(kDevNonFinite));
            }
            qa_ready = true;
          }
#pragma unroll
          for(int b = 0; b < kBatch; ++b) {
            if(kb0 + b < wi.kb_end && ok) {
              const uint32_t s = conv_it % T::kStages;
              const uint32_t ph = (conv_it / T::kStages) & 1u;
              ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctl->empty[s], ph ^ 1u, abort_flag, p.spin_limit));
              if(ok) {
                uint8_t* a_tile = tiles + s * T::kStageBytes + T::kWBytes;
#pragma unroll
                for(int q = 0; q < kCpt; ++q) {
                  const int c = epi_tid + q * kEpilogueThreads;
                  if(c < TM * 8) {
                    const int r = c >> 3, ch = c & 7;
                    uint4 o;
                    o.x = pack4_i8(f[b][q][0], qa);
                    o.y = pack4_i8(f[b][q][1], qa);
                    o.z = pack4_i8(f[b][q][2], qa);
                    o.w = pack4_i8(f[b][q][3], qa);
                    *reinterpret_cast<uint4*>(a_tile + r * 128 + ((ch ^ (r & 7)) << 4)) = o;
                  }
                }
                fence_proxy_async_smem();   // the tensor core reads these bytes through the async proxy
                __syncwarp();
                if(lane == 0)
                  mbar_arrive(&ctl->full[s]);
                ++conv_it;
              }
            }
          }
        }
        if(!ok)
          break;
      }
      const uint32_t as = acc_it & 1u;
      const uint32_t aph = (acc_it >> 1) & 1u;
      if(lane == 0)
        ok = mbar_wait_bounded(&ctl->tmem_full[as], aph, abort_flag, p.spin_limit);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if(!ok)
        break;
      tc_fence_after_sync();

      const uint32_t t_addr = tmem_base + as * T::kAccStride + (static_cast<uint32_t>(quarter * 32) << 16);
      const int n = wi.n_tile * kTileN + row;
      const bool n_ok = n < p.N;
      const int m0 = wi.m_tile * TM;
      const int cols_valid = min(TM, p.M - m0);  // activation rows of this tile that exist
      // the weight segment this tile belongs to: its multiplier, bias, output matrix and the column inside it
      int seg = 0, n_loc = n;
      if(!kP8 && kTopK == 0 && p.nseg > 1) {
        seg = (wi.n_tile * kTileN) / p.seg_n;
        n_loc = n - seg * p.seg_n;
        unquant = __fmul_rn(__fdiv_rn(1.0f, __fmul_rn(qa, *p.seg_qb[seg])), p.scale);
      }
      const float* seg_bias = p.seg_bias[seg];
      void* seg_c = p.seg_c[seg];
      const int ldc = p.seg_n;
      if constexpr(kTopK > 0) {
        // Output layer: lane = query row n, columns = vocabulary entries m0 .. m0 + TM - 1; warp group g takes
        // the 128-column block g of the tile.  Value = float(acc) * unquant + bias[column], rounded as in the
        // plain write-back.  Two sweeps over the block's accumulators (TMEM reads are cheap): maximum and best
        // entries first, then the exponentials against that maximum, added in ascending column order.
        static_assert(TM == 256, "the output-layer write-back assumes 256-column tiles");
        const int blk_col0 = group * 128;
        const int cnt = min(128, cols_valid - blk_col0);           // columns of this block that exist (may be <= 0)
        const int v0 = m0 + blk_col0;
        TopK best;
#pragma unroll
        for(int j = 0; j < kTopK; ++j) {
          best.v[j] = -FLT_MAX;
          best.i[j] = 0x7fffffff;
        }
        float bmax = -FLT_MAX;
        float bsum = 0.f;
        // Whole blocks (all but the vocabulary's last one) run without per-column tests, so the 32 columns of a
        // chunk form one straight-line region and their conversions / exponentials overlap in the pipeline.
        const bool whole = cnt == 128;
#pragma unroll 1
        for(int c = 0; c < 4; ++c) {
          int32_t v[32];
          tmem_ld_chunk<32>(t_addr + blk_col0 + c * 32, v);
          const float4* b4 = reinterpret_cast<const float4*>(p.bias + v0 + c * 32);
          float x[32];
          if(whole) {
            float bb[32];
            if((reinterpret_cast<uintptr_t>(b4) & 15u) == 0) {
#pragma unroll
              for(int j = 0; j < 8; ++j) {
                const float4 t4 = __ldg(b4 + j);
                bb[4 * j] = t4.x; bb[4 * j + 1] = t4.y; bb[4 * j + 2] = t4.z; bb[4 * j + 3] = t4.w;
              }
            } else {
#pragma unroll
              for(int j = 0; j < 32; ++j)
                bb[j] = __ldg(p.bias + v0 + c * 32 + j);
            }
            tc_wait_ld();
#pragma unroll
            for(int j = 0; j < 32; ++j)
              x[j] = __fadd_rn(__fmul_rn(__int2float_rn(v[j]), unquant), bb[j]);
            float cm = x[0];
#pragma unroll
            for(int j = 1; j < 32; ++j)
              cm = fmaxf(cm, x[j]);
            bmax = fmaxf(bmax, cm);
            if(cm >= best.v[kTopK - 1]) {   // only chunks that can change the list are scanned for candidates
#pragma unroll
              for(int j = 0; j < 32; ++j)
                topk_insert<kTopK>(best, x[j], v0 + c * 32 + j);
            }
          } else {
            tc_wait_ld();
#pragma unroll
            for(int j = 0; j < 32; ++j) {
              const int col = c * 32 + j;
              x[j] = -FLT_MAX;
              if(col < cnt) {
                x[j] = __fadd_rn(__fmul_rn(__int2float_rn(v[j]), unquant), __ldg(p.bias + v0 + col));
                bmax = fmaxf(bmax, x[j]);
                topk_insert<kTopK>(best, x[j], v0 + col);
              }
            }
          }
          if(p.lg_logits != nullptr && n_ok) {
#pragma unroll
            for(int j = 0; j < 32; ++j)
              if(c * 32 + j < cnt)
                p.lg_logits[static_cast<size_t>(n) * p.M + v0 + c * 32 + j] = x[j];
          }
        }
#pragma unroll 1
        for(int c = 0; c < 4; ++c) {
          int32_t v[32];
          tmem_ld_chunk<32>(t_addr + blk_col0 + c * 32, v);
          tc_wait_ld();
          if(whole) {
            float e[32];
#pragma unroll
            for(int j = 0; j < 32; ++j) {
              const float x = __fadd_rn(__fmul_rn(__int2float_rn(v[j]), unquant), __ldg(p.bias + v0 + c * 32 + j));
              e[j] = det_expf(__fadd_rn(x, -bmax));
            }
#pragma unroll
            for(int j = 0; j < 32; ++j)
              bsum = __fadd_rn(bsum, e[j]);
          } else {
#pragma unroll
            for(int j = 0; j < 32; ++j) {
              const int col = c * 32 + j;
              if(col < cnt) {
                const float x = __fadd_rn(__fmul_rn(__int2float_rn(v[j]), unquant), __ldg(p.bias + v0 + col));
                bsum = __fadd_rn(bsum, det_expf(__fadd_rn(x, -bmax)));
              }
            }
          }
        }
        if(n_ok && cnt > 0) {
          const size_t slot = static_cast<size_t>(n) * p.lg_blocks + (v0 >> 7);
          p.lg_max[slot] = bmax;
          p.lg_sum[slot] = bsum;
#pragma unroll
          for(int j = 0; j < kTopK; ++j) {
            p.lg_topv[slot * kTopK + j] = best.v[j];
            p.lg_topi[slot * kTopK + j] = best.i[j];
          }
        }
        tc_fence_before_sync();
        mbar_arrive(&ctl->tmem_empty[as]);
        ++acc_it;
        continue;
      }
      const float bias_n = (seg_bias != nullptr && n_ok) ? __ldg(seg_bias + n_loc) : 0.0f;
      float p8_scale_b = 0.0f;
      int p8_zp_b = 0, p8_off_b = 0;
      if constexpr(kP8) {
        if(n_ok) {
          p8_scale_b = __ldg(p.p8_scale_b + n);
          p8_zp_b = __ldg(p.p8_zp_b + n);
          p8_off_b = __ldg(p.p8_off_b + n);
        }
      }
      // Split-K: every split adds its partial accumulators into one int32 buffer per tile with
      // fire-and-forget reductions (layout [column][128 rows], coalesced); the last split to arrive
      // reads the totals back, zeroes the buffer again and runs the write-back.
      int32_t* tile_acc = p.partials + static_cast<size_t>(wi.tile) * (kTileN * TM);
      bool finalize = true;

      if(p.splits > 1) {
        if(has_chunks) {
#pragma unroll 1
          for(int c = group * (kChunkStep - 1); c < kChunks; c += kChunkStep) {
            int32_t v[T::kChunk];
            tmem_ld_chunk<T::kChunk>(t_addr + c * T::kChunk, v);
            tc_wait_ld();
#pragma unroll
            for(int j = 0; j < T::kChunk; ++j)
              if(c * T::kChunk + j < cols_valid)
                atomicAdd(tile_acc + (c * T::kChunk + j) * kTileN + row, v[j]);
          }
        }
        __threadfence();
        named_bar_sync(1, kEpilogueThreads);
        if(epi_tid == 0) {
          const unsigned old = atomicAdd(&p.tile_counters[wi.tile], 1u);
          const int last = (old == static_cast<unsigned>(p.splits - 1)) ? 1 : 0;
          if(last)
            p.tile_counters[wi.tile] = 0u;  // leave the workspace zeroed for the next call
          *reinterpret_cast<volatile int*>(&ctl->is_last) = last;
        }
        named_bar_sync(1, kEpilogueThreads);
        finalize = *reinterpret_cast<volatile int*>(&ctl->is_last) != 0;
        if(finalize)
          __threadfence();
      }

      unsigned out_max = 0u;  // max|C| over what this thread writes, for the next affine's quantisation
      if(finalize && has_chunks) {
#pragma unroll 1
        for(int c = group * (kChunkStep - 1); c < kChunks; c += kChunkStep) {
          int32_t v[T::kChunk];
          const int col0 = c * T::kChunk;
          if(p.splits > 1) {
            int32_t* src = tile_acc + col0 * kTileN + row;
#pragma unroll
            for(int j = 0; j < T::kChunk; ++j)
              v[j] = (col0 + j < cols_valid) ? __ldcg(src + j * kTileN) : 0;
#pragma unroll
            for(int j = 0; j < T::kChunk; ++j)
              if(col0 + j < cols_valid)
                src[j * kTileN] = 0;
          } else {
            tmem_ld_chunk<T::kChunk>(t_addr + col0, v);
            tc_wait_ld();
          }
          if constexpr(kP8) {
            if(n_ok)
              write_back_chunk_p8<T::kChunk>(p, v, static_cast<size_t>(m0 + col0) * p.N + n, cols_valid - col0, m0 + col0, p8_scale_b, p8_zp_b,
                                             p8_off_b, bias_n);
          } else if(n_ok)
            out_max = write_back_chunk<T::kChunk>(p, v, static_cast<size_t>(m0 + col0) * ldc + n_loc, cols_valid - col0, unquant, bias_n,
                                                  out_max, seg_c, ldc, seg_bias != nullptr);
        }
      }
      if(p.absmax_out != nullptr) {
        out_max = __reduce_max_sync(0xffffffffu, out_max);
        if(lane == 0 && out_max != 0u)
          atomicMax(p.absmax_out, out_max);
      }
      // hand the accumulator buffer back to the MMA warp
      tc_fence_before_sync();
      mbar_arrive(&ctl->tmem_empty[as]);
      ++acc_it;
    }
    if(!ok) {
      *abort_flag = 1;
      if(lane == 0)
        atomicMax(p.status, static_cast<int>(kDevTimeoutEpilogue));
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if(warp == 1) {
    if(*abort_flag) {
      // Something gave up: make sure no MMA is still running before the accumulators are released.
      bool drained = true;
      if(lane == 0) {
        int no_abort = 0;
        tc_commit(&ctl->drain);
        drained = mbar_wait_bounded(&ctl->drain, 0u, &no_abort, p.spin_limit);
        if(!drained)
          atomicMax(p.status, static_cast<int>(kDevTimeoutDrain));
      }
      __syncwarp();
    }
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, T::kTmemCols);
  }
  trace_stamp(tb, kTraceId, 2, trace_extra);
  trace_stamp(th.last, kTraceId, 3, trace_extra);
}

// ------------------------------------------------------------------ CTA-pair variant (large M)
// A cluster of two CTAs computes a tile of 256 weight rows x 256 activation rows with one
// tcgen05.mma.cta_group::2 per 32 bytes of K.  CTA `rank` of the pair loads weight rows
// [256 * pair_n + 128 * rank, +128) and activation rows [256 * m_tile + 128 * rank, +128) into its own
// shared memory (32 KB per stage instead of 48 KB for the same 128 x 256 outputs per CTA) and owns the
// accumulators of its 128 weight rows x all 256 activation rows in its TMEM, so its epilogue is the
// one of the single-CTA kernel.  Per CTA the tensor core reads 64 instead of 96 bytes of shared
// memory per clock at full rate, which leaves the shared-memory port room for the TMA writes.
//   * full[s] lives in the rank-0 CTA: its producer announces the bytes of both CTAs, both CTAs'
//     copies are credited to it; empty[s] and tmem_full[b] exist in both CTAs and are signalled by
//     commits of the rank-0 MMA thread addressed to both; tmem_empty[b] of rank 0 collects one
//     arrival per CTA (after that CTA's epilogue warps met at a named barrier).
//   * The cluster barrier brackets the kernel: no remote arrival before the barriers exist, no CTA
//     leaves (or frees TMEM) while its peer may still read its shared memory.
struct PairCfg {
  static constexpr int kTM = 256;             // activation rows per pair tile (MMA N)
  static constexpr int kHalfRows = 128;       // activation rows each CTA loads
  static constexpr int kStages = 6;
  static constexpr int kWBytes = kTileN * kTileKBytes;
  static constexpr int kABytes = kHalfRows * kTileKBytes;
  static constexpr int kStageBytes = kWBytes + kABytes;
  static constexpr int kAccStride = 256;
  static constexpr int kTmemCols = 512;
  static constexpr int kChunk = 32;
};
constexpr int smem_bytes_pair() { return PairCfg::kStages * PairCfg::kStageBytes + static_cast<int>(sizeof(Control)) + 1024; }

template <bool kP8>
__global__ void __launch_bounds__(kThreads, 1)
mi8_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a, const GemmParams p) {
  using T = PairCfg;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;  // same in both CTAs
  uint8_t* tiles = smem_raw + pad;
  Control* ctl = reinterpret_cast<Control*>(tiles + T::kStages * T::kStageBytes);
  volatile int* abort_flag = &ctl->abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  const uint32_t peer_abort = mapa_shared(smem_u32(&ctl->abort), rank ^ 1u);

  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  const unsigned long long trace_extra = static_cast<unsigned long long>(p.N) | (static_cast<unsigned long long>(p.K) << 20) |
                                         (static_cast<unsigned long long>(p.M) << 40);
  if(threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_a);
    for(int s = 0; s < T::kStages; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    for(int b = 0; b < 2; ++b) {
      mbar_init(&ctl->tmem_full[b], 1);
      mbar_init(&ctl->tmem_empty[b], 2);  // one arrival per CTA of the pair
    }
    mbar_init(&ctl->drain, 1);
    ctl->abort = 0;
    ctl->is_last = 0;
    fence_mbar_init();
  }
  if(warp == 1) {
    tmem_alloc_pair(&ctl->tmem_base, T::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);

  bool ok = true;

  if(warp == 0) {
    // ------------------------------------------------------------ TMA producer (one per CTA)
    uint32_t it = 0;
    uint32_t prefetched = 0;
    // copies of both CTAs are credited to full[s] of the rank-0 CTA
    auto full_addr = [&](uint32_t s) { return mapa_shared(smem_u32(&ctl->full[s]), 0u); };
    if(p.skip_a == nullptr && pair_id < p.total_work && p.withhold_item < 0) {
      // weights do not depend on the previous kernel: request the first pipeline fill before waiting for it
      const WorkItem w0 = decode_work(p, pair_id);
      const int n_pre = min(T::kStages, w0.kb_end - w0.kb_begin);
      if(elect_one()) {
        for(int i = 0; i < n_pre; ++i) {
          uint8_t* st = tiles + i * T::kStageBytes;
          if(leader)
            mbar_arrive_expect_tx(&ctl->full[i], 2 * T::kStageBytes);
          tma_load_2d_pair(st, &tmap_w, (w0.kb_begin + i) * kTileKBytes, (2 * w0.n_tile + static_cast<int>(rank)) * kTileN, full_addr(i));
        }
      }
      __syncwarp();
      prefetched = n_pre;
    }
    pdl_wait();
    const bool skip_on = p.skip_a != nullptr && *p.skip_a == *p.skip_b;
    if(p.rows_computed != nullptr && blockIdx.x == 0 && lane == 0)
      *p.rows_computed = p.M - (skip_on ? min(p.M, (p.skip_rows_below / T::kTM) * T::kTM) : 0);
    for(int w = pair_id; w < p.total_work && ok; w += n_pairs) {
      const WorkItem wi = decode_work(p, w);
      if(skip_on && (wi.m_tile + 1) * T::kTM <= p.skip_rows_below)
        continue;
      for(int kb = wi.kb_begin; kb < wi.kb_end; ++kb, ++it) {
        const uint32_t s = it % T::kStages;
        const uint32_t ph = (it / T::kStages) & 1u;
        const bool pre = it < prefetched;
        if(!pre)
          ok = mbar_wait_bounded(&ctl->empty[s], ph ^ 1u, abort_flag, p.spin_limit);
        ok = __all_sync(0xffffffffu, ok);
        if(!ok)
          break;
        if(elect_one() && static_cast<int>(it) != p.withhold_item) {   // (test hook: both CTAs of the pair leave a withheld item out)
          uint8_t* st = tiles + s * T::kStageBytes;
          if(!pre) {
            if(leader)
              mbar_arrive_expect_tx(&ctl->full[s], 2 * T::kStageBytes);
            tma_load_2d_pair(st, &tmap_w, kb * kTileKBytes, (2 * wi.n_tile + static_cast<int>(rank)) * kTileN, full_addr(s));
          }
          tma_load_2d_pair(st + T::kWBytes, &tmap_a, kb * kTileKBytes,
                           p.a_row0 + wi.m_tile * T::kTM + static_cast<int>(rank) * T::kHalfRows, full_addr(s));
        }
        __syncwarp();
      }
    }
    if(!ok) {
      *abort_flag = 1;
      if(lane == 0) {
        st_cluster_u32(peer_abort, 1u);
        atomicMax(p.status, static_cast<int>(kDevTimeoutProducer));
        if(leader) {
          // Wait (bounded) for the copies of both CTAs already announced, so none lands after the pair has gone.
          const uint32_t first = it > static_cast<uint32_t>(T::kStages) ? it - T::kStages : 0u;
          int no_abort = 0;
          for(uint32_t j = first; j < it; ++j)
            mbar_wait_bounded(&ctl->full[j % T::kStages], (j / T::kStages) & 1u, &no_abort, p.spin_limit);
        }
      }
      __syncwarp();
    }
  } else if(warp == 1) {
    // ------------------------------------------------------------ MMA issuer (rank 0 only; rank 1 owns its TMEM half)
    if(leader) {
      constexpr uint32_t idesc = kP8 ? make_idesc_i8_ub(T::kTM, 256) : make_idesc_i8(T::kTM, 256);
      uint32_t it = 0, acc_it = 0;
      pdl_wait();   // as in the single-CTA kernel: keeps the predecessor's run time out of the bounded waits
      const bool skip_on = p.skip_a != nullptr && *p.skip_a == *p.skip_b;
      for(int w = pair_id; w < p.total_work && ok; w += n_pairs) {
        const WorkItem wi = decode_work(p, w);
        if(skip_on && (wi.m_tile + 1) * T::kTM <= p.skip_rows_below)
          continue;
        const uint32_t as = acc_it & 1u;
        const uint32_t aph = (acc_it >> 1) & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctl->tmem_empty[as], aph ^ 1u, abort_flag, p.spin_limit));
        if(!ok)
          break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + as * T::kAccStride;
        for(int kb = wi.kb_begin; kb < wi.kb_end; ++kb, ++it) {
          const uint32_t s = it % T::kStages;
          const uint32_t ph = (it / T::kStages) & 1u;
          ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctl->full[s], ph, abort_flag, p.spin_limit));
          if(!ok)
            break;
          tc_fence_after_sync();
          const uint32_t w_addr = smem_u32(tiles + s * T::kStageBytes);
          const uint32_t a_addr = w_addr + T::kWBytes;
          if(elect_one()) {
#pragma unroll
            for(int k = 0; k < kTileKBytes / kMmaK; ++k) {
              tc_mma_i8_pair(d_tmem, make_kmajor_sw128_desc(w_addr + k * kMmaK), make_kmajor_sw128_desc(a_addr + k * kMmaK), idesc,
                             (kb > wi.kb_begin || k > 0) ? 1u : 0u);
            }
            tc_commit_pair(&ctl->empty[s], 3);  // frees this slot in both CTAs once the MMAs have read it
          }
          __syncwarp();
        }
        if(!ok)
          break;
        if(elect_one())
          tc_commit_pair(&ctl->tmem_full[as], 3);  // accumulator complete in both CTAs
        __syncwarp();
        ++acc_it;
      }
      if(!ok) {
        *abort_flag = 1;
        if(lane == 0) {
          st_cluster_u32(peer_abort, 1u);
          atomicMax(p.status, static_cast<int>(kDevTimeoutMma));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9 of both CTAs)
    const int quarter = warp & 3;
    const int group = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int epi_tid = threadIdx.x - 64;
    constexpr int kChunks = T::kTM / T::kChunk;
    pdl_wait();
    trace_stamp_start(th, kTrGemmPair, trace_extra);
    const float qa = kP8 ? 1.0f : *p.d_qa;
    float unquant = kP8 ? 1.0f : __fmul_rn(__fdiv_rn(1.0f, __fmul_rn(qa, *p.seg_qb[0])), p.scale);
    uint32_t acc_it = 0;
    const bool skip_on = p.skip_a != nullptr && *p.skip_a == *p.skip_b;
    for(int w = pair_id; w < p.total_work && ok; w += n_pairs) {
      const WorkItem wi = decode_work(p, w);
      if(skip_on && (wi.m_tile + 1) * T::kTM <= p.skip_rows_below)
        continue;
      const uint32_t as = acc_it & 1u;
      const uint32_t aph = (acc_it >> 1) & 1u;
      if(lane == 0)
        ok = mbar_wait_bounded(&ctl->tmem_full[as], aph, abort_flag, p.spin_limit);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if(!ok)
        break;
      tc_fence_after_sync();

      const uint32_t t_addr = tmem_base + as * T::kAccStride + (static_cast<uint32_t>(quarter * 32) << 16);
      const int n = (2 * wi.n_tile + static_cast<int>(rank)) * kTileN + row;
      const bool n_ok = n < p.N;
      const int m0 = wi.m_tile * T::kTM;
      const int cols_valid = min(T::kTM, p.M - m0);
      int seg = 0, n_loc = n;
      if(!kP8 && p.nseg > 1) {
        seg = ((2 * wi.n_tile + static_cast<int>(rank)) * kTileN) / p.seg_n;
        n_loc = n - seg * p.seg_n;
        unquant = __fmul_rn(__fdiv_rn(1.0f, __fmul_rn(qa, *p.seg_qb[seg])), p.scale);
      }
      const float* seg_bias = p.seg_bias[seg];
      void* seg_c = p.seg_c[seg];
      const int ldc = p.seg_n;
      const float bias_n = (seg_bias != nullptr && n_ok) ? __ldg(seg_bias + n_loc) : 0.0f;
      float p8_scale_b = 0.0f;
      int p8_zp_b = 0, p8_off_b = 0;
      if constexpr(kP8) {
        if(n_ok) {
          p8_scale_b = __ldg(p.p8_scale_b + n);
          p8_zp_b = __ldg(p.p8_zp_b + n);
          p8_off_b = __ldg(p.p8_off_b + n);
        }
      }
      unsigned out_max = 0u;
#pragma unroll 1
      for(int c = group; c < kChunks; c += 2) {
        const int col0 = c * T::kChunk;
        if(col0 >= cols_valid)
          break;
        int32_t v[T::kChunk];
        tmem_ld_chunk<T::kChunk>(t_addr + col0, v);
        tc_wait_ld();
        if constexpr(kP8) {
          if(n_ok)
            write_back_chunk_p8<T::kChunk>(p, v, static_cast<size_t>(m0 + col0) * p.N + n, cols_valid - col0, m0 + col0, p8_scale_b, p8_zp_b,
                                           p8_off_b, bias_n);
        } else if(n_ok)
          out_max = write_back_chunk<T::kChunk>(p, v, static_cast<size_t>(m0 + col0) * ldc + n_loc, cols_valid - col0, unquant, bias_n, out_max,
                                                seg_c, ldc, seg_bias != nullptr);
      }
      if(p.absmax_out != nullptr) {
        out_max = __reduce_max_sync(0xffffffffu, out_max);
        if(lane == 0 && out_max != 0u)
          atomicMax(p.absmax_out, out_max);
      }
      // hand the accumulator buffer back: all epilogue warps of this CTA meet, then one arrival per CTA
      tc_fence_before_sync();
      named_bar_sync(1, kEpilogueThreads);
      if(epi_tid == 0)
        mbar_arrive_cluster(mapa_shared(smem_u32(&ctl->tmem_empty[as]), 0u));
      ++acc_it;
    }
    if(!ok) {
      *abort_flag = 1;
      if(lane == 0) {
        st_cluster_u32(peer_abort, 1u);
        atomicMax(p.status, static_cast<int>(kDevTimeoutEpilogue));
      }
    }
  }

  // ------------------------------------------------------------ teardown
  if(warp == 1 && leader && *abort_flag) {
    // Something gave up: make sure no MMA is still running in either CTA before the accumulators are released.
    if(lane == 0) {
      int no_abort = 0;
      tc_commit_pair(&ctl->drain, 1);
      if(!mbar_wait_bounded(&ctl->drain, 0u, &no_abort, p.spin_limit))
        atomicMax(p.status, static_cast<int>(kDevTimeoutDrain));
    }
    __syncwarp();
  }
  tc_fence_before_sync();
  cluster_sync_all();
  if(warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, T::kTmemCols);
  }
  trace_stamp(tb, kTrGemmPair, 2, trace_extra);
  trace_stamp(th.last, kTrGemmPair, 3, trace_extra);
}

// ------------------------------------------------------------------ cluster variant (decode shapes)
// One launch = "quantise the fp32 activation with the multiplier of its abs-max slot" + GEMM + write-back, and
// optionally the residual add + LayerNorm that follows.  A cluster holds the CTAs of `csize` neighbouring weight
// tiles of ONE activation tile.  Every CTA needs the whole quantised activation tile [TM, K]; CTA `rank`
// quantises the 128-byte K blocks kb = rank, rank + csize, ... (fp32 read once per cluster) and stores each
// 16-byte chunk into the shared memory of all CTAs of the cluster at the place the 128-byte swizzle gives it,
// then arrives on a_full[kb] in each of them.  The activation tile stays resident (K <= 4096), only the weight
// tiles run through a TMA ring.  One tile per CTA, no split-K.
//   LayerNorm mode (TM = 32, the cluster covers the whole row: csize = N / 128 <= 8): the write-back keeps
//   y = C + residual in shared memory, every CTA reduces its 128 columns per row exactly as one warp of
//   add_layernorm_kernel does (lane l owns columns 4l..4l+3, butterfly), the per-row partial sums travel to all
//   CTAs of the cluster, and are added in ascending block order starting from 0 - the arithmetic of
//   add_layernorm_kernel for rows of up to 1024 values, bit for bit.  Three cluster barriers separate the phases;
//   every thread of every CTA reaches them whatever happened before (all other waits are bounded).
constexpr int kCqMaxKb = 32;        // K <= 4096
constexpr int kCqMaxCluster = 8;
constexpr int kCqLnRows = 64;      // activation rows per tile in LayerNorm mode: 32 or 64

struct CqControl {
  uint64_t w_full[kMaxStages];
  uint64_t w_empty[kMaxStages];
  uint64_t a_full[kCqMaxKb];
  uint64_t tmem_full;
  uint64_t drain;
  uint32_t tmem_base;
  int abort;
  float part_sum[kCqMaxCluster][kCqLnRows];
  float part_sq[kCqMaxCluster][kCqLnRows];
  unsigned part_max[kCqMaxCluster][kCqLnRows];
};

struct CqParams {
  int M, N, K, kb_total, stages;
  const float* a_f32;       // [M, K] fp32
  const unsigned* a_slot;   // bit pattern of max|A|
  float* qa_out;            // optional: receives 127 / max|A|
  const float* d_qb;
  float scale;
  const float* bias;
  int relu;
  float* c;                 // [M, N] fp32 (plain mode)
  unsigned* absmax_out;     // plain mode: max|C| reduced into this slot
  int ln;                   // 1: out = LayerNorm(C + resid) * gamma + beta instead of C
  const float* ln_resid;
  const float* ln_gamma;
  const float* ln_beta;
  float ln_eps;
  float* ln_out;
  float* ln_rowmax;         // optional [M]
  unsigned* ln_slot;        // optional abs-max slots of the output
  unsigned* ln_slot2;
  int* status;
  uint32_t spin_limit;
  int withhold_item;
  int* rows_computed;
};

__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, const uint4& v) {
  asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
// try_wait whose acquire reaches writes released at cluster scope (shared memory written by another CTA)
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint32_t limit) {
  for(uint32_t i = 0; i < limit; ++i) {
    if(mbar_try_wait_cluster(bar, parity))
      return true;
    if((i & 0xff) == 0xff && *abort_flag)
      return false;
  }
  return false;
}

template <int TM>
constexpr int cq_smem_bytes(int kb_total, int stages) {
  return kb_total * TM * kTileKBytes + stages * kTileN * kTileKBytes + static_cast<int>(sizeof(CqControl)) + 1024;
}

template <int TM>
__global__ void __launch_bounds__(kThreads, 1)
mi8_gemm_cq_kernel(const __grid_constant__ CUtensorMap tmap_w, const CqParams p) {
  constexpr int kWBytes = kTileN * kTileKBytes;
  constexpr int kABlock = TM * kTileKBytes;          // one K block of the activation tile
  constexpr int kTmemCols = TM < 32 ? 32 : TM;
  constexpr int kConvWarps = kEpilogueThreads / 32;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;   // the same in every CTA of the kernel
  uint8_t* a_region = smem_raw + pad;
  uint8_t* w_ring = a_region + p.kb_total * kABlock;
  CqControl* ctl = reinterpret_cast<CqControl*>(w_ring + p.stages * kWBytes);
  volatile int* abort_flag = &ctl->abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const uint32_t csize = cluster_nctarank();
  const int n_tile = blockIdx.x;
  const int m0 = blockIdx.y * TM;

  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  const unsigned long long trace_extra = static_cast<unsigned long long>(p.N) | (static_cast<unsigned long long>(p.K) << 20);
  if(threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_w);
    for(int s = 0; s < p.stages; ++s) {
      mbar_init(&ctl->w_full[s], 1);
      mbar_init(&ctl->w_empty[s], 1);
    }
    for(int kb = 0; kb < p.kb_total; ++kb)
      mbar_init(&ctl->a_full[kb], kConvWarps);    // one arrival per quantising warp of the CTA that owns the K block
    mbar_init(&ctl->tmem_full, 1);
    mbar_init(&ctl->drain, 1);
    ctl->abort = 0;
    fence_mbar_init();
  }
  if(warp == 1) {
    tmem_alloc(&ctl->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
  cluster_sync_all();   // the barriers of every CTA of the cluster exist before anything is stored or signalled remotely

  bool ok = true;
  float unquant = 1.0f;

  if(warp == 0) {
    // ------------------------------------------------------------ weight producer (weights never depend on the preceding kernel)
    for(int kb = 0; kb < p.kb_total; ++kb) {
      const uint32_t s = kb % p.stages;
      const uint32_t ph = (kb / p.stages) & 1u;
      if(kb >= p.stages)
        ok = mbar_wait_bounded(&ctl->w_empty[s], ph ^ 1u, abort_flag, p.spin_limit);
      ok = __all_sync(0xffffffffu, ok);
      if(!ok)
        break;
      if(elect_one() && kb != p.withhold_item) {
        mbar_arrive_expect_tx(&ctl->w_full[s], kWBytes);
        tma_load_2d(w_ring + s * kWBytes, &tmap_w, kb * kTileKBytes, n_tile * kTileN, &ctl->w_full[s]);
      }
      __syncwarp();
    }
    if(!ok) {
      *abort_flag = 1;
      if(lane == 0)
        atomicMax(p.status, static_cast<int>(kDevTimeoutProducer));
    }
  } else if(warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc_i8(TM);
    for(int kb = 0; kb < p.kb_total; ++kb) {
      const uint32_t s = kb % p.stages;
      const uint32_t ph = (kb / p.stages) & 1u;
      ok = mbar_wait_cluster_bounded(&ctl->a_full[kb], 0u, abort_flag, p.spin_limit) && mbar_wait_bounded(&ctl->w_full[s], ph, abort_flag, p.spin_limit);
      ok = __all_sync(0xffffffffu, ok);
      if(!ok)
        break;
      fence_proxy_async_smem();
      tc_fence_after_sync();
      const uint32_t w_addr = smem_u32(w_ring + s * kWBytes);
      const uint32_t a_addr = smem_u32(a_region + kb * kABlock);
      if(elect_one()) {
#pragma unroll
        for(int k = 0; k < kTileKBytes / kMmaK; ++k)
          tc_mma_i8(tmem_base, make_kmajor_sw128_desc(w_addr + k * kMmaK), make_kmajor_sw128_desc(a_addr + k * kMmaK), idesc, (kb > 0 || k > 0) ? 1u : 0u);
        tc_commit(&ctl->w_empty[s]);
      }
      __syncwarp();
    }
    if(ok) {
      if(elect_one())
        tc_commit(&ctl->tmem_full);
      __syncwarp();
    } else {
      *abort_flag = 1;
      if(lane == 0)
        atomicMax(p.status, static_cast<int>(kDevTimeoutMma));
    }
  } else {
    // ------------------------------------------------------------ quantisers, then write-back (warps 2..9)
    const int epi_tid = threadIdx.x - 64;
    const int quarter = warp & 3;
    const int group = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    pdl_wait();   // the activation and its abs-max slot are the preceding kernel's output
    trace_stamp_start(th, kTrGemmCq, trace_extra);
    if(p.rows_computed != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && epi_tid == 0)
      *p.rows_computed = p.M;
    constexpr int kCpt = TM * 8 / kEpilogueThreads;     // 16-byte chunks per thread and K block (1, 2, 4)
    constexpr int kBatch = 4 / kCpt;                    // K blocks per batch: 16 loads of 16 bytes in flight per thread
    const uint32_t a_base = smem_u32(a_region);
    const uint32_t bar_base = smem_u32(&ctl->a_full[0]);
    float qa = 1.0f;
    bool qa_ready = false;
    for(int kb0 = static_cast<int>(rank); kb0 < p.kb_total; kb0 += static_cast<int>(csize) * kBatch) {
      float4 f[kBatch][kCpt][4];
#pragma unroll
      for(int b = 0; b < kBatch; ++b) {
        const int kb = kb0 + b * static_cast<int>(csize);
#pragma unroll
        for(int q = 0; q < kCpt; ++q) {
          const int c = epi_tid + q * kEpilogueThreads;
          const int gm = m0 + (c >> 3);
          const bool in = kb < p.kb_total && gm < p.M;
          const float4* src = reinterpret_cast<const float4*>(p.a_f32 + static_cast<size_t>(in ? gm : 0) * p.K + (in ? kb * kTileKBytes + (c & 7) * 16 : 0));
#pragma unroll
          for(int e = 0; e < 4; ++e)
            f[b][q][e] = in ? src[e] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      if(!qa_ready) {   // (read after the loads above were issued: the two round trips overlap)
        const unsigned bits = *p.a_slot;
        qa = bits == 0u ? 1.0f : __fdiv_rn(127.0f, __uint_as_float(bits));
        unquant = __fmul_rn(__fdiv_rn(1.0f, __fmul_rn(qa, *p.d_qb)), p.scale);
        if(blockIdx.x == 0 && blockIdx.y == 0 && epi_tid == 0) {
          if(p.qa_out != nullptr)
            *p.qa_out = qa;
          if(bits >= 0x7f800000u)
            atomicMax(p.status, static_cast<int>(kDevNonFinite));
        }
        qa_ready = true;
      }
#pragma unroll
      for(int b = 0; b < kBatch; ++b) {
        const int kb = kb0 + b * static_cast<int>(csize);
        if(kb < p.kb_total) {
#pragma unroll
          for(int q = 0; q < kCpt; ++q) {
            const int c = epi_tid + q * kEpilogueThreads;
            const int r = c >> 3, ch = c & 7;
            uint4 o;
            o.x = pack4_i8(f[b][q][0], qa);
            o.y = pack4_i8(f[b][q][1], qa);
            o.z = pack4_i8(f[b][q][2], qa);
            o.w = pack4_i8(f[b][q][3], qa);
            const uint32_t off = static_cast<uint32_t>(kb * kABlock + r * 128 + ((ch ^ (r & 7)) << 4));
            for(uint32_t j = 0; j < csize; ++j)
              st_cluster_v4(mapa_shared(a_base + off, j), o);
          }
          fence_proxy_async_all();   // the tensor cores read these bytes through the async proxy
          __syncwarp();
          if(lane < csize)
            mbar_arrive_cluster(mapa_shared(bar_base + static_cast<uint32_t>(kb) * 8u, lane));
        }
      }
    }
    trace_stamp(tb, kTrGemmCq, 4, trace_extra);   // this CTA's share of the activation tile is stored and signalled
    if(!qa_ready) {   // (more CTAs in the cluster than K blocks: this one quantised nothing)
      const unsigned bits = *p.a_slot;
      qa = bits == 0u ? 1.0f : __fdiv_rn(127.0f, __uint_as_float(bits));
      unquant = __fmul_rn(__fdiv_rn(1.0f, __fmul_rn(qa, *p.d_qb)), p.scale);
    }

    if(lane == 0)
      ok = mbar_wait_bounded(&ctl->tmem_full, 0u, abort_flag, p.spin_limit);
    ok = __shfl_sync(0xffffffffu, ok, 0);
    trace_stamp(tb, kTrGemmCq, 5, trace_extra);   // accumulator complete
    if(ok) {
      tc_fence_after_sync();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      const int n = n_tile * kTileN + row;
      const bool n_ok = n < p.N;
      const float bias_n = (p.bias != nullptr && n_ok) ? __ldg(p.bias + n) : 0.0f;
      constexpr int kChunks = TM / 32;
      constexpr int kChunkStep = kChunks > 1 ? 2 : 1;
      const bool has_chunks = kChunks > 1 || group == 0;
      unsigned out_max = 0u;
      if(has_chunks) {
#pragma unroll 1
        for(int c = group * (kChunkStep - 1); c < kChunks; c += kChunkStep) {
          int32_t v[32];
          tmem_ld_chunk<32>(t_addr + c * 32, v);
          tc_wait_ld();
          const int valid = min(32, p.M - (m0 + c * 32));
          float fv[32];
#pragma unroll
          for(int j = 0; j < 32; ++j)
            fv[j] = __fmul_rn(__int2float_rn(v[j]), unquant);
          if(p.bias != nullptr) {
#pragma unroll
            for(int j = 0; j < 32; ++j)
              fv[j] = __fadd_rn(fv[j], bias_n);
          }
          if(p.relu) {
#pragma unroll
            for(int j = 0; j < 32; ++j)
              fv[j] = fv[j] > 0.0f ? fv[j] : 0.0f;
          }
          if(p.ln) {
            // y = C + residual, parked row-major [TM rows][128 columns] where the weight ring was (all its tiles are consumed)
            float* tile = reinterpret_cast<float*>(w_ring) + c * 32 * 128;
            const float* res = p.ln_resid + static_cast<size_t>(m0 + c * 32) * p.N + n;
#pragma unroll
            for(int j = 0; j < 32; ++j) {
              float y = 0.0f;
              if(j < valid && n_ok)
                y = p.ln_resid != nullptr ? __fadd_rn(fv[j], res[static_cast<size_t>(j) * p.N]) : fv[j];
              tile[j * 128 + row] = y;
            }
          } else if(n_ok) {
            float* dst = p.c + static_cast<size_t>(m0 + c * 32) * p.N + n;
#pragma unroll
            for(int j = 0; j < 32; ++j)
              if(j < valid) {
                dst[static_cast<size_t>(j) * p.N] = fv[j];
                out_max = max(out_max, __float_as_uint(fv[j]) & 0x7fffffffu);
              }
          }
        }
      }
      trace_stamp(tb, kTrGemmCq, 6, trace_extra);   // write-back (or the LayerNorm tile) done
      if(!p.ln && p.absmax_out != nullptr) {
        out_max = __reduce_max_sync(0xffffffffu, out_max);
        if(lane == 0 && out_max != 0u)
          atomicMax(p.absmax_out, out_max);
      }
    } else {
      *abort_flag = 1;
      if(lane == 0)
        atomicMax(p.status, static_cast<int>(kDevTimeoutEpilogue));
    }
  }

  if(p.ln) {
    // ------------------------------------------------------------ LayerNorm over the cluster (TM = 32 or 64): warp e of the eight takes rows kRpw * e .. + kRpw - 1
    const bool worker = warp >= 2;
    const int e = warp - 2;
    const float* tile = reinterpret_cast<const float*>(w_ring);
    const float dimf = static_cast<float>(p.N);
    constexpr int kRpw = TM >= 64 ? 8 : 4;   // rows per warp (TM = 128 never runs this mode)
    float4 x[kRpw];
    float mean[kRpw];
    if(worker) {
      named_bar_sync(1, kEpilogueThreads);   // the tile is complete
#pragma unroll
      for(int i = 0; i < kRpw; ++i) {
        const int m = kRpw * e + i;
        x[i] = *reinterpret_cast<const float4*>(tile + m * 128 + 4 * lane);
        const float s = warp_sum_det(__fadd_rn(0.0f, __fadd_rn(__fadd_rn(x[i].x, x[i].y), __fadd_rn(x[i].z, x[i].w))));
        if(lane < csize)
          asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(mapa_shared(smem_u32(&ctl->part_sum[rank][m]), lane)), "f"(s) : "memory");
      }
    }
    cluster_sync_all();
    if(worker) {
#pragma unroll
      for(int i = 0; i < kRpw; ++i) {
        const int m = kRpw * e + i;
        float t = 0.0f;
#pragma unroll
        for(int w = 0; w < kCqMaxCluster; ++w)
          t = __fadd_rn(t, w < static_cast<int>(csize) ? ctl->part_sum[w][m] : 0.0f);
        mean[i] = __fdiv_rn(t, dimf);
        const float dx = __fadd_rn(x[i].x, -mean[i]), dy = __fadd_rn(x[i].y, -mean[i]), dz = __fadd_rn(x[i].z, -mean[i]), dw = __fadd_rn(x[i].w, -mean[i]);
        const float q = warp_sum_det(__fadd_rn(0.0f, __fmaf_rn(dx, dx, __fmaf_rn(dy, dy, __fmaf_rn(dz, dz, __fmul_rn(dw, dw))))));
        if(lane < csize)
          asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(mapa_shared(smem_u32(&ctl->part_sq[rank][m]), lane)), "f"(q) : "memory");
      }
    }
    cluster_sync_all();
    if(worker) {
      const int ncol = n_tile * kTileN + 4 * lane;
      const float4 g = __ldg(reinterpret_cast<const float4*>(p.ln_gamma + ncol));
      const float4 b = __ldg(reinterpret_cast<const float4*>(p.ln_beta + ncol));
      unsigned wmax = 0u;
#pragma unroll
      for(int i = 0; i < kRpw; ++i) {
        const int m = kRpw * e + i;
        float t = 0.0f;
#pragma unroll
        for(int w = 0; w < kCqMaxCluster; ++w)
          t = __fadd_rn(t, w < static_cast<int>(csize) ? ctl->part_sq[w][m] : 0.0f);
        const float var = __fdiv_rn(t, dimf);
        const float denom = __fsqrt_rn(__fadd_rn(var, p.ln_eps));
        float4 o;
        o.x = __fadd_rn(__fmul_rn(__fdiv_rn(__fadd_rn(x[i].x, -mean[i]), denom), g.x), b.x);
        o.y = __fadd_rn(__fmul_rn(__fdiv_rn(__fadd_rn(x[i].y, -mean[i]), denom), g.y), b.y);
        o.z = __fadd_rn(__fmul_rn(__fdiv_rn(__fadd_rn(x[i].z, -mean[i]), denom), g.z), b.z);
        o.w = __fadd_rn(__fmul_rn(__fdiv_rn(__fadd_rn(x[i].w, -mean[i]), denom), g.w), b.w);
        unsigned rmax = 0u;
        if(m0 + m < p.M) {
          *reinterpret_cast<float4*>(p.ln_out + static_cast<size_t>(m0 + m) * p.N + ncol) = o;
          rmax = max(max(__float_as_uint(o.x) & 0x7fffffffu, __float_as_uint(o.y) & 0x7fffffffu),
                     max(__float_as_uint(o.z) & 0x7fffffffu, __float_as_uint(o.w) & 0x7fffffffu));
        }
        rmax = __reduce_max_sync(0xffffffffu, rmax);
        wmax = max(wmax, rmax);
        if(lane == 0 && p.ln_rowmax != nullptr)   // the row maximum is put together by the CTA of rank 0
          asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(mapa_shared(smem_u32(&ctl->part_max[rank][m]), 0)), "r"(rmax) : "memory");
      }
      if(lane == 0 && wmax != 0u) {
        if(p.ln_slot != nullptr)
          atomicMax(p.ln_slot, wmax);
        if(p.ln_slot2 != nullptr)
          atomicMax(p.ln_slot2, wmax);
      }
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before_sync();
  cluster_sync_all();   // no CTA leaves while a peer may still store into its shared memory or signal its barriers
  if(p.ln && p.ln_rowmax != nullptr && rank == 0 && (warp == 2 || warp == 3)) {
    const int m = (warp - 2) * 32 + lane;
    if(m < TM && m0 + m < p.M) {
      unsigned r = 0u;
      for(uint32_t w = 0; w < csize; ++w)
        r = max(r, ctl->part_max[w][m]);
      p.ln_rowmax[m0 + m] = __uint_as_float(r);
    }
  }
  if(warp == 1) {
    if(*abort_flag) {
      bool drained = true;
      if(lane == 0) {
        int no_abort = 0;
        tc_commit(&ctl->drain);
        drained = mbar_wait_bounded(&ctl->drain, 0u, &no_abort, p.spin_limit);
        if(!drained)
          atomicMax(p.status, static_cast<int>(kDevTimeoutDrain));
      }
      __syncwarp();
    }
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  trace_stamp(tb, kTrGemmCq, 2, trace_extra);
  trace_stamp(th.last, kTrGemmCq, 3, trace_extra);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    if(e != cudaSuccess || qres != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// Tensor map over a row-major int8 matrix [rows, K] with a box of 128 K-bytes x box_rows rows,
// 128-byte swizzle, zero fill outside the matrix.
int encode_kmajor_map(CUtensorMap* map, const int8_t* base, int rows, int K, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if(fn == nullptr)
    return MI8_ERR_DRIVER;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(K)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kTileKBytes), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(base), dims, strides, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MI8_OK : MI8_ERR_DRIVER;
}

// A tensor map only describes an address range and a box shape, so it can be reused for as long as the same
// (pointer, rows, K, box) comes back - which a decoder that multiplies the same weights and the same activation
// buffers every step does about a hundred times per step.  Per-thread table, open addressing; when it fills up
// it is emptied and rebuilt (descriptors never go stale: they hold no data).
struct MapCache {
  static constexpr int kSlots = 2048;   // power of two
  struct Entry {
    const void* base;
    int rows, K, box;
    bool used;
  };
  Entry keys[kSlots];
  alignas(64) CUtensorMap maps[kSlots];
  int count = 0;
  MapCache() { clear(); }
  void clear() {
    for(int i = 0; i < kSlots; ++i)
      keys[i].used = false;
    count = 0;
  }
};
thread_local MapCache* t_map_cache = nullptr;

int get_kmajor_map(CUtensorMap* out, const int8_t* base, int rows, int K, int box_rows) {
  if(t_map_cache == nullptr)
    t_map_cache = new MapCache();
  MapCache& mc = *t_map_cache;
  uint64_t h = reinterpret_cast<uintptr_t>(base) >> 4;
  h ^= static_cast<uint64_t>(rows) * 0x9E3779B97F4A7C15ull;
  h ^= (static_cast<uint64_t>(K) << 21) ^ (static_cast<uint64_t>(static_cast<uint32_t>(box_rows)) << 40);
  h ^= h >> 29;
  int slot = static_cast<int>(h & (MapCache::kSlots - 1));
  for(int probe = 0; probe < 16; ++probe, slot = (slot + 1) & (MapCache::kSlots - 1)) {
    MapCache::Entry& e = mc.keys[slot];
    if(!e.used)
      break;
    if(e.base == base && e.rows == rows && e.K == K && e.box == box_rows) {
      *out = mc.maps[slot];
      return MI8_OK;
    }
  }
  int rc = encode_kmajor_map(out, base, rows, K, box_rows);
  if(rc != MI8_OK)
    return rc;
  if(mc.count > MapCache::kSlots / 2)
    mc.clear();
  slot = static_cast<int>(h & (MapCache::kSlots - 1));
  for(int probe = 0; probe < 16; ++probe, slot = (slot + 1) & (MapCache::kSlots - 1)) {
    MapCache::Entry& e = mc.keys[slot];
    if(!e.used) {
      e.base = base;
      e.rows = rows;
      e.K = K;
      e.box = box_rows;
      e.used = true;
      mc.maps[slot] = *out;
      ++mc.count;
      break;
    }
  }
  return MI8_OK;
}

// Test hook (mi8_test_wait_fault): the next launches withhold one pipeline item and wait with a short limit.
int g_test_withhold_item = -1;
uint32_t g_test_spin_limit = 0;

// Optional bracketing of every GEMM launch with CUDA events on the launching stream (mi8_profile_begin /
// mi8_profile_end), so a benchmark can attribute device time to this kernel inside its timed region.  The
// kernel itself reports how many activation rows it computed (launches that reuse stored rows skip most).
struct ProfileRecord {
  int M, N, K, out_bytes;
  cudaEvent_t start, stop;
};
struct ProfileState {
  bool on = false;
  size_t capacity = 0;
  std::vector<ProfileRecord> records;
  std::vector<cudaEvent_t> pool;   // events are created once and reused
  size_t pool_used = 0;
  int* d_rows = nullptr;           // [capacity] rows computed per recorded launch (device memory held while profiling)
  cudaEvent_t take() {
    if(pool_used == pool.size()) {
      cudaEvent_t e;
      if(cudaEventCreate(&e) != cudaSuccess)
        return nullptr;
      pool.push_back(e);
    }
    return pool[pool_used++];
  }
};
thread_local ProfileState t_profile;

// Fields every launcher sets the same way.
void finish_params(GemmParams& p) {
  p.withhold_item = g_test_withhold_item;
  p.spin_limit = g_test_spin_limit != 0 ? g_test_spin_limit : kSpinLimit;
  p.rows_computed = nullptr;
  if(t_profile.on && t_profile.d_rows != nullptr && t_profile.records.size() < t_profile.capacity)
    p.rows_computed = t_profile.d_rows + t_profile.records.size();
}
void single_segment(GemmParams& p) {
  p.a_row0 = 0;
  p.nseg = 1;
  p.seg_n = p.N;
  for(int i = 0; i < kMaxSegments; ++i) {
    p.seg_qb[i] = p.d_qb;
    p.seg_bias[i] = p.bias;
    p.seg_c[i] = p.c;
  }
}

template <int TM, bool kQuantA = false, int kTopK = 0, bool kP8 = false>
int launch_cfg(const CUtensorMap& tw, const CUtensorMap& ta, const GemmParams& p, const GemmPlan& plan, cudaStream_t stream) {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  constexpr int smem = smem_bytes_for<TM>();
  if(dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(mi8_gemm_kernel<TM, kQuantA, kTopK, kP8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if(e != cudaSuccess) {
      set_last_cuda_error(e);
      return MI8_ERR_LAUNCH;
    }
    attr_set[dev] = true;
  }
  ProfileRecord rec{};
  const bool profiled = t_profile.on && t_profile.records.size() < t_profile.capacity;
  if(profiled) {
    // (the output-layer variant runs with swapped operands: report the problem as the caller sees it)
    rec = ProfileRecord{kTopK > 0 ? p.N : p.M, kTopK > 0 ? p.M : p.N, p.K, p.out_f16 ? 2 : 4, t_profile.take(), t_profile.take()};
    if(rec.start != nullptr && rec.stop != nullptr)
      cudaEventRecord(rec.start, stream);
  }
  cudaError_t le = launch_kernel(mi8_gemm_kernel<TM, kQuantA, kTopK, kP8>, dim3(plan.grid), dim3(kThreads), smem, stream, tw, ta, p);
  if(le != cudaSuccess) {
    set_last_cuda_error(le);
    return MI8_ERR_LAUNCH;
  }
  if(profiled && rec.start != nullptr && rec.stop != nullptr) {
    cudaEventRecord(rec.stop, stream);
    t_profile.records.push_back(rec);
  }
  count_launch();
  return check_launch();
}

// Launch of the CTA-pair kernel: clusters of two CTAs, as many as can be resident at once.
template <bool kP8 = false>
int launch_pair(const CUtensorMap& tw, const CUtensorMap& ta, const GemmParams& p, const GemmPlan& plan, cudaStream_t stream) {
  static bool attr_set[64] = {};
  static int max_clusters[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if(dev < 0 || dev >= 64)
    return MI8_ERR_UNSUPPORTED;
  constexpr int smem = smem_bytes_pair();
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  if(!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(mi8_gemm_pair_kernel<kP8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if(e != cudaSuccess) {
      set_last_cuda_error(e);
      return MI8_ERR_LAUNCH;
    }
    // how many CTA pairs the device can hold at once (bounds the persistent grid)
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, mi8_gemm_pair_kernel<kP8>, &cfg);
    if(e != cudaSuccess || n <= 0) {
      set_last_cuda_error(e);
      cudaGetLastError();
      return MI8_ERR_LAUNCH;
    }
    max_clusters[dev] = n;
    attr_set[dev] = true;
  }
  const int pairs = plan.grid / 2 < max_clusters[dev] ? plan.grid / 2 : max_clusters[dev];
  cfg.gridDim = dim3(2 * pairs);
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  ProfileRecord rec{};
  const bool profiled = t_profile.on && t_profile.records.size() < t_profile.capacity;
  if(profiled) {
    rec = ProfileRecord{p.M, p.N, p.K, p.out_f16 ? 2 : 4, t_profile.take(), t_profile.take()};
    if(rec.start != nullptr && rec.stop != nullptr)
      cudaEventRecord(rec.start, stream);
  }
  const bool timed = kernel_times_on();
  if(timed) {
    cfg.numAttrs = 1;   // no launch overlap while per-kernel times are taken
    kernel_times_before(reinterpret_cast<const void*>(mi8_gemm_pair_kernel<kP8>), stream);
  }
  cudaError_t le = cudaLaunchKernelEx(&cfg, mi8_gemm_pair_kernel<kP8>, tw, ta, p);
  if(timed)
    kernel_times_after(stream);
  if(le != cudaSuccess) {
    set_last_cuda_error(le);
    return MI8_ERR_LAUNCH;
  }
  if(profiled && rec.start != nullptr && rec.stop != nullptr) {
    cudaEventRecord(rec.stop, stream);
    t_profile.records.push_back(rec);
  }
  count_launch();
  return check_launch();
}

}  // namespace

MI8_DEFINE_TRACE_SETTER(trace_set_gemm)

void test_wait_fault(int withhold_item, unsigned spin_limit) {
  g_test_withhold_item = withhold_item;
  g_test_spin_limit = spin_limit;
}

int profile_begin(int max_records) {
  if(max_records <= 0)
    return MI8_ERR_BAD_ARG;
  if(t_profile.d_rows != nullptr) {
    cudaFree(t_profile.d_rows);
    t_profile.d_rows = nullptr;
  }
  // the one allocation of the library, made by this measurement aid for the time profiling is on
  if(cudaMalloc(reinterpret_cast<void**>(&t_profile.d_rows), sizeof(int) * static_cast<size_t>(max_records)) != cudaSuccess) {
    cudaGetLastError();
    t_profile.d_rows = nullptr;
  } else {
    cudaMemset(t_profile.d_rows, 0xff, sizeof(int) * static_cast<size_t>(max_records));   // -1: "not reported"
  }
  t_profile.on = true;
  t_profile.capacity = static_cast<size_t>(max_records);
  t_profile.records.clear();
  t_profile.pool_used = 0;
  return MI8_OK;
}

int profile_end(mi8_gemm_record* out, int capacity, int* count) {
  t_profile.on = false;
  int n = 0;
  std::vector<int> rows(t_profile.records.size(), -1);
  if(t_profile.d_rows != nullptr && !rows.empty()) {
    if(cudaDeviceSynchronize() != cudaSuccess ||
       cudaMemcpy(rows.data(), t_profile.d_rows, sizeof(int) * rows.size(), cudaMemcpyDeviceToHost) != cudaSuccess) {
      cudaGetLastError();
      std::fill(rows.begin(), rows.end(), -1);
    }
  }
  for(size_t i = 0; i < t_profile.records.size(); ++i) {
    const ProfileRecord& r = t_profile.records[i];
    if(n >= capacity || out == nullptr)
      break;
    float ms = 0.f;
    if(cudaEventSynchronize(r.stop) != cudaSuccess || cudaEventElapsedTime(&ms, r.start, r.stop) != cudaSuccess) {
      cudaGetLastError();
      continue;
    }
    out[n].M = r.M;
    out[n].N = r.N;
    out[n].K = r.K;
    out[n].out_bytes = r.out_bytes;
    out[n].us = ms * 1000.f;
    out[n].rows_computed = rows[i] >= 0 ? rows[i] : r.M;
    ++n;
  }
  if(count != nullptr)
    *count = n;
  t_profile.records.clear();
  t_profile.pool_used = 0;
  if(t_profile.d_rows != nullptr) {
    cudaFree(t_profile.d_rows);
    t_profile.d_rows = nullptr;
  }
  return MI8_OK;
}

int make_gemm_plan(int M, int N, int K, int force_tile_m, int force_splits, GemmPlan* plan) {
  if(M <= 0 || N <= 0 || K <= 0)
    return MI8_ERR_BAD_ARG;
  const int sms = sm_count();
  int tm = force_tile_m;
  plan->pair = 0;
  if(tm == 0 && force_splits <= 1 && M > 64) {
    // Enough 128 x 256 tiles for every SM and at least eight K blocks per tile: the CTA-pair kernel
    // moves a third less operand data from L2 into shared memory per output and measured 10-20 % faster
    // there; with shorter K its extra per-tile synchronisation costs more than that saves.
    const long long tiles256 = static_cast<long long>((N + kTileN - 1) / kTileN) * ((M + 255) / 256);
    if(tiles256 >= sms && (K + kTileKBytes - 1) / kTileKBytes >= 8 && N > kTileN)
      tm = kPairTileCode;
  }
  if(tm == kPairTileCode) {
    // CTA-pair variant: tiles of 256 weight rows x 256 activation rows, one per cluster of two CTAs.
    if(force_splits > 1)
      return MI8_ERR_BAD_ARG;
    plan->pair = 1;
    plan->tile_m = PairCfg::kTM;
    plan->stages = PairCfg::kStages;
    plan->n_tiles = (N + 2 * kTileN - 1) / (2 * kTileN);
    plan->m_tiles = (M + PairCfg::kTM - 1) / PairCfg::kTM;
    plan->kb_total = (K + kTileKBytes - 1) / kTileKBytes;
    plan->kb_per_split = plan->kb_total;
    plan->splits = 1;
    const long long pair_tiles = static_cast<long long>(plan->n_tiles) * plan->m_tiles;
    if(pair_tiles > 0x7fffffffLL / 64)
      return MI8_ERR_UNSUPPORTED;
    const long long pairs = pair_tiles < sms / 2 ? pair_tiles : sms / 2;
    plan->grid = static_cast<int>(2 * pairs);
    plan->smem_bytes = smem_bytes_pair();
    plan->partial_bytes = 0;
    return MI8_OK;
  }
  if(tm == 0) {
    // Tile width along M.  Up to 64 rows: the smallest tile that holds them.  Above that, 256-row tiles
    // only when they already give every SM a tile; otherwise narrower tiles spread the work over more SMs.
    if(M <= 64) {
      tm = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    } else {
      const long long tiles256 = static_cast<long long>((N + kTileN - 1) / kTileN) * ((M + 255) / 256);
      if(tiles256 >= sms) {
        tm = 256;
      } else {
        // The main loop of a CTA is bound by what one SM can pull from L2 (~64 bytes per clock), so the
        // narrowest tile that still gives every tile its own SM finishes first (512 x 1024 x 1024: 5.2 us
        // with 32-row tiles on 128 CTAs, 6.1 us with 128-row tiles on 32 CTAs).
        tm = 128;
        for(int cand : {32, 64}) {
          if(static_cast<long long>((N + kTileN - 1) / kTileN) * ((M + cand - 1) / cand) <= sms) {
            tm = cand;
            break;
          }
        }
      }
    }
  }
  if(tm != 16 && tm != 32 && tm != 64 && tm != 128 && tm != 256)
    return MI8_ERR_BAD_ARG;
  plan->tile_m = tm;
  plan->stages = tm == 256 ? 4 : (tm == 128 ? 6 : 8);
  plan->n_tiles = (N + kTileN - 1) / kTileN;
  plan->m_tiles = (M + tm - 1) / tm;
  plan->kb_total = (K + kTileKBytes - 1) / kTileKBytes;
  const long long tiles = static_cast<long long>(plan->n_tiles) * plan->m_tiles;
  if(tiles > 0x7fffffffLL / 64)
    return MI8_ERR_UNSUPPORTED;
  int splits = force_splits;
  if(splits == 0) {
    splits = 1;
    if(tiles < sms) {
      // Split K across idle SMs, but leave every split at least eight 128-byte K blocks: below that
      // the fence + arrival counter of the split path costs more than the shorter stream saves.
      int by_sms = static_cast<int>(sms / tiles);
      int by_depth = plan->kb_total / 8 > 1 ? plan->kb_total / 8 : 1;
      splits = by_sms < by_depth ? by_sms : by_depth;
      if(splits > plan->kb_total)
        splits = plan->kb_total;
      if(splits < 1)
        splits = 1;
    }
  }
  if(splits < 1 || splits > plan->kb_total)
    return MI8_ERR_BAD_ARG;
  plan->kb_per_split = (plan->kb_total + splits - 1) / splits;
  splits = (plan->kb_total + plan->kb_per_split - 1) / plan->kb_per_split;  // no empty split
  plan->splits = splits;
  if(splits > 1 && tiles > kWsMaxTileCounters)
    return MI8_ERR_UNSUPPORTED;
  const long long work = tiles * splits;
  plan->grid = static_cast<int>(work < sms ? work : sms);
  plan->smem_bytes = tm == 256 ? smem_bytes_for<256>()
                               : tm == 128 ? smem_bytes_for<128>()
                                           : tm == 64 ? smem_bytes_for<64>() : tm == 32 ? smem_bytes_for<32>() : smem_bytes_for<16>();
  plan->partial_bytes = splits > 1 ? static_cast<size_t>(tiles) * kTileN * tm * sizeof(int32_t) : 0;
  return MI8_OK;
}

int launch_gemm_call(const GemmCall& g) {
  const int M = g.M, N = g.N, K = g.K;
  if(M < 0 || N <= 0 || K <= 0)
    return MI8_ERR_BAD_ARG;
  if(M == 0)
    return MI8_OK;
  if(g.aq == nullptr || g.bt == nullptr || g.d_qa == nullptr || g.nseg < 1 || g.nseg > kMaxSegments)
    return MI8_ERR_BAD_ARG;
  for(int i = 0; i < g.nseg; ++i)
    if(g.seg_qb[i] == nullptr || g.seg_c[i] == nullptr)
      return MI8_ERR_BAD_ARG;
  if(g.nseg > 1 && (N % g.nseg != 0 || (N / g.nseg) % kTileN != 0 || g.acc_out != nullptr))
    return MI8_ERR_UNSUPPORTED;   // a tile of 128 weight rows must not straddle two segments
  if(g.out_dtype != MI8_F32 && g.out_dtype != MI8_F16)
    return MI8_ERR_BAD_ARG;
  if(K % 16 != 0 || (reinterpret_cast<uintptr_t>(g.aq) & 15u) || (reinterpret_cast<uintptr_t>(g.bt) & 15u))
    return MI8_ERR_MISALIGNED;
  GemmPlan plan;
  int rc = make_gemm_plan(M, N, K, g.force_tile_m, g.force_splits, &plan);
  if(rc != MI8_OK)
    return rc;
  if(plan.splits > 1) {
    if(g.ws == nullptr || g.ws_bytes < kWsHeaderBytes + plan.partial_bytes)
      return MI8_ERR_WORKSPACE;
  }
  CUtensorMap tw, ta;
  rc = get_kmajor_map(&tw, g.bt, N, K, kTileN);
  if(rc != MI8_OK)
    return rc;
  // a_rows_cap: the activation buffer is known to hold that many rows, so one descriptor serves every M up to
  // it (rows past M inside the last tile are then real bytes instead of zero fill; their products are never stored)
  if(g.a_row0 < 0 || (g.a_row0 > 0 && g.a_rows_cap < g.a_row0 + M))
    return MI8_ERR_BAD_ARG;
  rc = get_kmajor_map(&ta, g.aq, g.a_rows_cap > M ? g.a_rows_cap : M, K, plan.pair ? PairCfg::kHalfRows : plan.tile_m);
  if(rc != MI8_OK)
    return rc;

  GemmParams p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.n_tiles = plan.n_tiles;
  p.m_tiles = plan.m_tiles;
  p.splits = plan.splits;
  p.kb_total = plan.kb_total;
  p.kb_per_split = plan.kb_per_split;
  p.total_work = plan.n_tiles * plan.m_tiles * plan.splits;
  p.d_qa = g.d_qa;
  p.d_qb = g.seg_qb[0];
  p.scale = g.scale;
  p.bias = g.seg_bias[0];
  p.relu = g.relu ? 1 : 0;
  p.out_f16 = g.out_dtype == MI8_F16 ? 1 : 0;
  p.c = g.seg_c[0];
  p.acc_out = g.acc_out;
  uint8_t* wsb = static_cast<uint8_t*>(g.ws);
  p.partials = wsb ? reinterpret_cast<int32_t*>(wsb + kWsOffPartials) : nullptr;
  p.tile_counters = wsb ? reinterpret_cast<unsigned*>(wsb + kWsOffTileCounters) : nullptr;
  p.absmax_out = g.absmax_out;
  p.lg_max = p.lg_sum = p.lg_topv = nullptr;
  p.lg_topi = nullptr;
  p.lg_blocks = 0;
  p.lg_logits = nullptr;
  p.a_f32 = nullptr;
  p.a_slot = nullptr;
  p.qa_out = nullptr;
  p.skip_a = g.skip_a;
  p.skip_b = g.skip_b;
  p.skip_rows_below = g.skip_rows_below;
  p.p8_scale_a = p.p8_scale_b = nullptr;
  p.p8_zp_a = p.p8_sum_a = p.p8_zp_b = p.p8_off_b = nullptr;
  p.status = device_status_ptr();
  if(p.status == nullptr)
    return MI8_ERR_LAUNCH;
  single_segment(p);
  p.nseg = g.nseg;
  p.seg_n = N / g.nseg;
  for(int i = 0; i < g.nseg; ++i) {
    p.seg_qb[i] = g.seg_qb[i];
    p.seg_bias[i] = g.seg_bias[i];
    p.seg_c[i] = g.seg_c[i];
  }
  p.a_row0 = g.a_row0;
  finish_params(p);

  if(plan.pair)
    return launch_pair(tw, ta, p, plan, g.stream);
  switch(plan.tile_m) {
    case 16: return launch_cfg<16>(tw, ta, p, plan, g.stream);
    case 32: return launch_cfg<32>(tw, ta, p, plan, g.stream);
    case 64: return launch_cfg<64>(tw, ta, p, plan, g.stream);
    case 128: return launch_cfg<128>(tw, ta, p, plan, g.stream);
    default: return launch_cfg<256>(tw, ta, p, plan, g.stream);
  }
}

int launch_gemm(const int8_t* aq, const int8_t* bt, int M, int N, int K, const float* d_qa, const float* d_qb, float scale,
                const float* bias, int relu, void* c, int out_dtype, int32_t* acc_out, void* ws, size_t ws_bytes,
                cudaStream_t stream, int force_tile_m, int force_splits, unsigned* absmax_out, const unsigned* skip_a,
                const unsigned* skip_b, int skip_rows_below) {
  if(M > 0 && (d_qb == nullptr || c == nullptr))
    return MI8_ERR_BAD_ARG;
  GemmCall g;
  g.aq = aq;
  g.bt = bt;
  g.M = M;
  g.N = N;
  g.K = K;
  g.d_qa = d_qa;
  g.scale = scale;
  g.relu = relu;
  g.out_dtype = out_dtype;
  g.acc_out = acc_out;
  g.nseg = 1;
  g.seg_qb[0] = d_qb;
  g.seg_bias[0] = bias;
  g.seg_c[0] = c;
  g.ws = ws;
  g.ws_bytes = ws_bytes;
  g.stream = stream;
  g.force_tile_m = force_tile_m;
  g.force_splits = force_splits;
  g.absmax_out = absmax_out;
  g.skip_a = skip_a;
  g.skip_b = skip_b;
  g.skip_rows_below = skip_rows_below;
  return launch_gemm_call(g);
}

// ------------------------------------------------------------------ cluster GEMM (quantising, optional LayerNorm write-back)
bool gemm_cq_supported(int M, int N, int K, bool ln) {
  if(M <= 0 || N <= 0 || K <= 0 || N % kTileN != 0 || K % kTileKBytes != 0 || K / kTileKBytes > kCqMaxKb)
    return false;
  if(ln && N / kTileN > kCqMaxCluster)
    return false;
  return true;
}

namespace {
template <int TM>
int launch_cq_tile(const CUtensorMap& tw, CqParams& p, int n_tiles, int cluster, cudaStream_t stream) {
  static int attr_smem[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if(dev < 0 || dev >= 64)
    return MI8_ERR_UNSUPPORTED;
  constexpr int kSmemMax = 232448;   // 227 KB opt-in limit per CTA
  const int fixed = p.kb_total * TM * kTileKBytes + static_cast<int>(sizeof(CqControl)) + 1024;
  int stages = (kSmemMax - fixed) / (kTileN * kTileKBytes);
  if(stages > kMaxStages)
    stages = kMaxStages;
  const int min_stages = p.ln ? TM / 32 : 1;   // (LayerNorm mode parks its [TM][128] fp32 tile where the ring was)
  if(stages > p.kb_total)
    stages = p.kb_total > min_stages ? p.kb_total : min_stages;
  if(stages < min_stages)
    return MI8_ERR_UNSUPPORTED;
  p.stages = stages;
  const int smem = cq_smem_bytes<TM>(p.kb_total, stages);
  if(attr_smem[dev] < smem) {
    cudaError_t e = cudaFuncSetAttribute(mi8_gemm_cq_kernel<TM>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
    if(e != cudaSuccess) {
      set_last_cuda_error(e);
      return MI8_ERR_LAUNCH;
    }
    attr_smem[dev] = kSmemMax;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_tiles, (p.M + TM - 1) / TM);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  ProfileRecord rec{};
  const bool profiled = t_profile.on && t_profile.records.size() < t_profile.capacity;
  if(profiled) {
    rec = ProfileRecord{p.M, p.N, p.K, 4, t_profile.take(), t_profile.take()};
    if(rec.start != nullptr && rec.stop != nullptr)
      cudaEventRecord(rec.start, stream);
  }
  const bool timed = kernel_times_on();
  if(timed) {
    cfg.numAttrs = 1;
    kernel_times_before(reinterpret_cast<const void*>(mi8_gemm_cq_kernel<TM>), stream);
  }
  cudaError_t le = cudaLaunchKernelEx(&cfg, mi8_gemm_cq_kernel<TM>, tw, p);
  if(timed)
    kernel_times_after(stream);
  if(le != cudaSuccess) {
    set_last_cuda_error(le);
    return MI8_ERR_LAUNCH;
  }
  if(profiled && rec.start != nullptr && rec.stop != nullptr) {
    cudaEventRecord(rec.stop, stream);
    t_profile.records.push_back(rec);
  }
  count_launch();
  return check_launch();
}
}  // namespace

int launch_gemm_cq(const CqCall& g) {
  if(g.a_f32 == nullptr || g.a_slot == nullptr || g.bt == nullptr || g.d_qb == nullptr)
    return MI8_ERR_BAD_ARG;
  if(!gemm_cq_supported(g.M, g.N, g.K, g.ln != 0))
    return MI8_ERR_UNSUPPORTED;
  if(g.ln ? (g.ln_out == nullptr || g.ln_gamma == nullptr || g.ln_beta == nullptr) : g.c == nullptr)
    return MI8_ERR_BAD_ARG;
  if((reinterpret_cast<uintptr_t>(g.a_f32) & 15u) != 0)
    return MI8_ERR_BAD_ARG;
  const int n_tiles = g.N / kTileN;
  int cluster = g.force_cluster;
  if(g.ln)
    cluster = n_tiles;
  else if(cluster <= 0) {
    cluster = 4;     // larger clusters share the quantisation further but are placed fewer at a time (measured slower)
    while(n_tiles % cluster != 0)
      cluster >>= 1;
  }
  if(cluster < 1 || cluster > kCqMaxCluster || n_tiles % cluster != 0)
    return MI8_ERR_BAD_ARG;
  // the narrowest tile that still gives every tile its own SM (as the plain kernel's plan does)
  int tm = g.force_tile_m;
  if(g.ln) {
    // Clusters of eight are placed a few at a time (measured: about eight fit at once), so rows go in tiles of 64 as soon
    // as 32-row tiles would need more clusters than that and the 64-row activation tile still fits in shared memory.
    if(tm != 32 && tm != 64)
      tm = ((g.M + 31) / 32 > 8 && g.K <= 2048) ? 64 : 32;
    if(tm == 64 && g.K > 2048)
      return MI8_ERR_UNSUPPORTED;
  } else if(tm <= 0) {
    const int sms = sm_count();
    tm = 32;
    while(tm < 128 && n_tiles * ((g.M + tm - 1) / tm) > sms)
      tm <<= 1;
  }
  if(tm != 32 && tm != 64 && tm != 128)
    return MI8_ERR_BAD_ARG;
  CqParams p{};
  p.M = g.M;
  p.N = g.N;
  p.K = g.K;
  p.kb_total = g.K / kTileKBytes;
  p.a_f32 = g.a_f32;
  p.a_slot = g.a_slot;
  p.qa_out = g.qa_out;
  p.d_qb = g.d_qb;
  p.scale = g.scale;
  p.bias = g.bias;
  p.relu = g.relu;
  p.c = g.c;
  p.absmax_out = g.absmax_out;
  p.ln = g.ln;
  p.ln_resid = g.ln_resid;
  p.ln_gamma = g.ln_gamma;
  p.ln_beta = g.ln_beta;
  p.ln_eps = g.ln_eps;
  p.ln_out = g.ln_out;
  p.ln_rowmax = g.ln_rowmax;
  p.ln_slot = g.ln_slot;
  p.ln_slot2 = g.ln_slot2;
  p.status = device_status_ptr();
  p.withhold_item = g_test_withhold_item;
  p.spin_limit = g_test_spin_limit != 0 ? g_test_spin_limit : kSpinLimit;
  p.rows_computed = nullptr;
  if(t_profile.on && t_profile.d_rows != nullptr && t_profile.records.size() < t_profile.capacity)
    p.rows_computed = t_profile.d_rows + t_profile.records.size();
  CUtensorMap tw;
  int rc = get_kmajor_map(&tw, g.bt, g.N, g.K, kTileN);
  if(rc != MI8_OK)
    return rc;
  switch(tm) {
    case 32: return launch_cq_tile<32>(tw, p, n_tiles, cluster, g.stream);
    case 64: return launch_cq_tile<64>(tw, p, n_tiles, cluster, g.stream);
    default: return launch_cq_tile<128>(tw, p, n_tiles, cluster, g.stream);
  }
}

// The packed8avx512 multiply: the plan of launch_gemm (CTA-pair kernel included); the accumulators and the
// split-K machinery are the same, only the operand signedness and the write-back differ.
int launch_gemm_p8(const uint8_t* aq, const float* scale_a, const int32_t* zp_a, const int32_t* sum_a, const int8_t* bt,
                   const float* scale_b, const int32_t* zp_b, const int32_t* off_b, int M, int N, int K, const float* bias, int relu,
                   float* c, int32_t* acc_out, void* ws, size_t ws_bytes, cudaStream_t stream, int force_tile_m, int force_splits) {
  if(M < 0 || N <= 0 || K <= 0 || force_tile_m < 0 || force_splits < 0)
    return MI8_ERR_BAD_ARG;
  if(M == 0)
    return MI8_OK;
  if(aq == nullptr || bt == nullptr || c == nullptr || scale_a == nullptr || zp_a == nullptr || sum_a == nullptr || scale_b == nullptr
     || zp_b == nullptr || off_b == nullptr)
    return MI8_ERR_BAD_ARG;
  if(K % 16 != 0 || (reinterpret_cast<uintptr_t>(aq) & 15u) || (reinterpret_cast<uintptr_t>(bt) & 15u))
    return MI8_ERR_MISALIGNED;
  if((reinterpret_cast<uintptr_t>(scale_a) & 15u) || (reinterpret_cast<uintptr_t>(zp_a) & 15u) || (reinterpret_cast<uintptr_t>(sum_a) & 15u))
    return MI8_ERR_MISALIGNED;   // the write-back reads the per-row arrays four rows at a time
  GemmPlan plan;
  int rc = make_gemm_plan(M, N, K, force_tile_m, force_splits, &plan);
  if(rc != MI8_OK)
    return rc;
  if(plan.splits > 1 && (ws == nullptr || ws_bytes < kWsHeaderBytes + plan.partial_bytes))
    return MI8_ERR_WORKSPACE;
  CUtensorMap tw, ta;
  rc = get_kmajor_map(&tw, bt, N, K, kTileN);
  if(rc != MI8_OK)
    return rc;
  rc = get_kmajor_map(&ta, reinterpret_cast<const int8_t*>(aq), M, K, plan.pair ? PairCfg::kHalfRows : plan.tile_m);
  if(rc != MI8_OK)
    return rc;
  GemmParams p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.n_tiles = plan.n_tiles;
  p.m_tiles = plan.m_tiles;
  p.splits = plan.splits;
  p.kb_total = plan.kb_total;
  p.kb_per_split = plan.kb_per_split;
  p.total_work = plan.n_tiles * plan.m_tiles * plan.splits;
  p.scale = 1.0f;
  p.bias = bias;
  p.relu = relu ? 1 : 0;
  p.c = c;
  p.acc_out = acc_out;
  uint8_t* wsb = static_cast<uint8_t*>(ws);
  p.partials = wsb ? reinterpret_cast<int32_t*>(wsb + kWsOffPartials) : nullptr;
  p.tile_counters = wsb ? reinterpret_cast<unsigned*>(wsb + kWsOffTileCounters) : nullptr;
  p.p8_scale_a = scale_a;
  p.p8_zp_a = zp_a;
  p.p8_sum_a = sum_a;
  p.p8_scale_b = scale_b;
  p.p8_zp_b = zp_b;
  p.p8_off_b = off_b;
  p.status = device_status_ptr();
  if(p.status == nullptr)
    return MI8_ERR_LAUNCH;
  single_segment(p);
  finish_params(p);
  if(plan.pair)
    return launch_pair<true>(tw, ta, p, plan, stream);
  switch(plan.tile_m) {
    case 16: return launch_cfg<16, false, 0, true>(tw, ta, p, plan, stream);
    case 32: return launch_cfg<32, false, 0, true>(tw, ta, p, plan, stream);
    case 64: return launch_cfg<64, false, 0, true>(tw, ta, p, plan, stream);
    case 128: return launch_cfg<128, false, 0, true>(tw, ta, p, plan, stream);
    default: return launch_cfg<256, false, 0, true>(tw, ta, p, plan, stream);
  }
}

// Tile width for the quantise-in-kernel variant: one tile per CTA, tiles as narrow as still fit on the
// SMs (each CTA reads its rows of the fp32 activation, so narrow tiles keep that read short).  0 = none fits.
int quant_a_tile(int M, int N) {
  const int sms = sm_count();
  const int n_tiles = (N + kTileN - 1) / kTileN;
  if(M <= 64)
    return n_tiles <= sms ? (M <= 16 ? 16 : (M <= 32 ? 32 : 64)) : 0;
  for(int tm : {32, 64})
    if(static_cast<long long>(n_tiles) * ((M + tm - 1) / tm) <= sms)
      return tm;
  return 0;
}

int launch_gemm_quant_a(const float* a_f32, const unsigned* a_slot, float* qa_out, const int8_t* bt, int M, int N, int K,
                        const float* d_qb, float scale, const float* bias, int relu, void* c, int out_dtype, int32_t* acc_out,
                        cudaStream_t stream, unsigned* absmax_out) {
  if(M < 0 || N <= 0 || K <= 0)
    return MI8_ERR_BAD_ARG;
  if(M == 0)
    return MI8_OK;
  if(a_f32 == nullptr || a_slot == nullptr || bt == nullptr || d_qb == nullptr || c == nullptr)
    return MI8_ERR_BAD_ARG;
  if(out_dtype != MI8_F32 && out_dtype != MI8_F16)
    return MI8_ERR_BAD_ARG;
  if(K % 16 != 0 || (reinterpret_cast<uintptr_t>(a_f32) & 15u) || (reinterpret_cast<uintptr_t>(bt) & 15u))
    return MI8_ERR_MISALIGNED;
  const int tm = quant_a_tile(M, N);
  if(tm == 0)
    return MI8_ERR_UNSUPPORTED;
  GemmPlan plan;
  int rc = make_gemm_plan(M, N, K, tm, 1, &plan);
  if(rc != MI8_OK)
    return rc;
  CUtensorMap tw;
  rc = get_kmajor_map(&tw, bt, N, K, kTileN);
  if(rc != MI8_OK)
    return rc;
  GemmParams p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.n_tiles = plan.n_tiles;
  p.m_tiles = plan.m_tiles;
  p.splits = 1;
  p.kb_total = plan.kb_total;
  p.kb_per_split = plan.kb_per_split;
  p.total_work = plan.n_tiles * plan.m_tiles;
  p.d_qa = nullptr;
  p.d_qb = d_qb;
  p.scale = scale;
  p.bias = bias;
  p.relu = relu ? 1 : 0;
  p.out_f16 = out_dtype == MI8_F16 ? 1 : 0;
  p.c = c;
  p.acc_out = acc_out;
  p.partials = nullptr;
  p.tile_counters = nullptr;
  p.absmax_out = absmax_out;
  p.lg_max = p.lg_sum = p.lg_topv = nullptr;
  p.lg_topi = nullptr;
  p.lg_blocks = 0;
  p.lg_logits = nullptr;
  p.a_f32 = a_f32;
  p.a_slot = a_slot;
  p.qa_out = qa_out;
  p.skip_a = nullptr;
  p.skip_b = nullptr;
  p.skip_rows_below = 0;
  p.status = device_status_ptr();
  if(p.status == nullptr)
    return MI8_ERR_LAUNCH;
  single_segment(p);
  finish_params(p);
  switch(tm) {   // the weight map stands in for the unused activation map
    case 16: return launch_cfg<16, true>(tw, tw, p, plan, stream);
    case 32: return launch_cfg<32, true>(tw, tw, p, plan, stream);
    default: return launch_cfg<64, true>(tw, tw, p, plan, stream);
  }
}

// Output layer without logits in memory: values[r][v] = float(acc) * unquant + bias[v] are reduced inside the
// write-back to, per (row, block of 128 vocabulary entries), the block maximum, the block's sum of exponentials
// and its k_top (4 or 8) best entries.  The host swaps the operands: the activation is the M-side operand of the
// kernel (128 rows per tile, one TMEM lane per query row) and the weight matrix the N-side operand (256 rows
// per tile), so a thread owns a row and walks 128 consecutive vocabulary entries.
int launch_gemm_logits(const int8_t* aq, const float* d_qa, const int8_t* wq, const float* d_qw, int rows, int vocab, int K,
                       const float* bias, float scale, int k_top, float* blk_max, float* blk_sum, float* blk_topv, int* blk_topi,
                       float* logits_out, cudaStream_t stream) {
  if(rows < 0 || vocab <= 0 || K <= 0 || (k_top != 4 && k_top != 8))
    return MI8_ERR_BAD_ARG;
  if(rows == 0)
    return MI8_OK;
  if(aq == nullptr || wq == nullptr || d_qa == nullptr || d_qw == nullptr || bias == nullptr || blk_max == nullptr || blk_sum == nullptr ||
     blk_topv == nullptr || blk_topi == nullptr)
    return MI8_ERR_BAD_ARG;
  if(K % 16 != 0 || (reinterpret_cast<uintptr_t>(aq) & 15u) || (reinterpret_cast<uintptr_t>(wq) & 15u))
    return MI8_ERR_MISALIGNED;
  GemmPlan plan;
  // in the kernel's terms: "weights" = the activation (N = rows), "activation" = the weight matrix (M = vocab)
  int rc = make_gemm_plan(vocab, rows, K, 256, 1, &plan);
  if(rc != MI8_OK)
    return rc;
  CUtensorMap tw, ta;
  rc = get_kmajor_map(&tw, aq, rows, K, kTileN);
  if(rc != MI8_OK)
    return rc;
  rc = get_kmajor_map(&ta, wq, vocab, K, 256);
  if(rc != MI8_OK)
    return rc;
  GemmParams p;
  p.M = vocab;
  p.N = rows;
  p.K = K;
  p.n_tiles = plan.n_tiles;
  p.m_tiles = plan.m_tiles;
  p.splits = 1;
  p.kb_total = plan.kb_total;
  p.kb_per_split = plan.kb_per_split;
  p.total_work = plan.n_tiles * plan.m_tiles;
  p.d_qa = d_qw;
  p.d_qb = d_qa;
  p.scale = scale;
  p.bias = bias;
  p.relu = 0;
  p.out_f16 = 0;
  p.c = nullptr;
  p.acc_out = nullptr;
  p.partials = nullptr;
  p.tile_counters = nullptr;
  p.absmax_out = nullptr;
  p.lg_max = blk_max;
  p.lg_sum = blk_sum;
  p.lg_topv = blk_topv;
  p.lg_topi = blk_topi;
  p.lg_blocks = (vocab + 127) / 128;
  p.lg_logits = logits_out;
  p.a_f32 = nullptr;
  p.a_slot = nullptr;
  p.qa_out = nullptr;
  p.skip_a = nullptr;
  p.skip_b = nullptr;
  p.skip_rows_below = 0;
  p.status = device_status_ptr();
  if(p.status == nullptr)
    return MI8_ERR_LAUNCH;
  single_segment(p);
  finish_params(p);
  p.rows_computed = nullptr;   // (in this launch p.M counts vocabulary entries, not activation rows)
  return k_top == 4 ? launch_cfg<256, false, 4>(tw, ta, p, plan, stream) : launch_cfg<256, false, 8>(tw, ta, p, plan, stream);
}

}  // namespace mi8
