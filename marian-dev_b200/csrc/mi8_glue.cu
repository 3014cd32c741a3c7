// Decode-step glue kernels around the int8 affines: embedding + position, residual add + LayerNorm,
// quantisation from a pre-reduced abs-max, single-query attention over a key/value history,
// history bookkeeping for the per-step re-projection of self-attention keys/values, and the
// log-softmax + top-k of the output layer.  All fp32, all HBM/latency-bound streaming kernels.
//
// Abs-max fusion: every producer of a tensor that is quantised next (embedding, LayerNorm, attention,
// the ReLU GEMM) reduces max|x| on the fly into a 4-byte slot (unsigned bit pattern, atomicMax), so
// the quantisation needs one launch instead of two.  Slots are zeroed once per step by the driver.
#include <cfloat>

#include "mi8_internal.h"
#include "mi8_math.cuh"
#include "mi8_ptx.cuh"

namespace mi8 {
namespace {

constexpr int kRowThreads = 256;
constexpr int kMaxVec = 4;  // float4 per thread: rows of up to 4096 floats
constexpr int kMaxHistLayers = 16;

__device__ __forceinline__ unsigned abs_bits(float v) { return __float_as_uint(v) & 0x7fffffffu; }

__device__ __forceinline__ unsigned block_max_u(unsigned v, unsigned* red) {
  v = __reduce_max_sync(0xffffffffu, v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if(lane == 0)
    red[warp] = v;
  __syncthreads();
  unsigned t = 0u;
#pragma unroll
  for(int w = 0; w < kRowThreads / 32; ++w)
    t = max(t, red[w]);
  return t;
}

__device__ __forceinline__ unsigned max4u(unsigned m, const float4& v) {
  return max(max(max(m, abs_bits(v.x)), max(abs_bits(v.y), abs_bits(v.z))), abs_bits(v.w));
}

// out[r,:] = wemb[words[r],:] * scale + pos[(pos_mod ? r % pos_mod : 0),:]
// (words == nullptr: zero embedding, the start symbol; pos_mod = source width for the encoder, 0 for a decoder step)
__global__ void __launch_bounds__(kRowThreads)
embed_kernel(const float* __restrict__ wemb, const int* __restrict__ words, const float* __restrict__ pos, int pos_mod, float scale,
             int dim, float* __restrict__ out, float* __restrict__ rowmax, unsigned* absmax_slot, unsigned* absmax_slot2) {
  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  pdl_wait();
  trace_stamp_start(th, kTrEmbed);
  __shared__ unsigned red[kRowThreads / 32];
  const int r = blockIdx.x;
  const float4* src = words ? reinterpret_cast<const float4*>(wemb + static_cast<size_t>(words[r]) * dim) : nullptr;
  const float4* p4 = reinterpret_cast<const float4*>(pos + static_cast<size_t>(pos_mod ? r % pos_mod : 0) * dim);
  float4* dst = reinterpret_cast<float4*>(out + static_cast<size_t>(r) * dim);
  unsigned m = 0u;
  for(int i = threadIdx.x; i < dim / 4; i += kRowThreads) {
    float4 e = src ? __ldg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 p = __ldg(p4 + i);
    float4 o;
    o.x = __fadd_rn(__fmul_rn(e.x, scale), p.x);
    o.y = __fadd_rn(__fmul_rn(e.y, scale), p.y);
    o.z = __fadd_rn(__fmul_rn(e.z, scale), p.z);
    o.w = __fadd_rn(__fmul_rn(e.w, scale), p.w);
    dst[i] = o;
    m = max4u(m, o);
  }
  m = block_max_u(m, red);
  if(threadIdx.x == 0) {
    if(rowmax)
      rowmax[r] = __uint_as_float(m);
    if(absmax_slot)
      atomicMax(absmax_slot, m);
    if(absmax_slot2)
      atomicMax(absmax_slot2, m);
  }
  trace_stamp(tb, kTrEmbed, 2);
  trace_stamp(th.last, kTrEmbed, 3);
}

// out = LayerNorm(a + resid) * gamma + beta, one block of 256 threads per row; biased variance
// (gamma * (x - mean) / sqrt(var + eps) + beta, src/tensors/cpu/tensor_operators.cpp:1087-1124).
// Arithmetic order (all operations rounded to nearest, restated identically by the CPU checker):
//   thread t owns the float4 chunks c = t + 256*j;  y = a + resid;
//   s_t = sum_j ((y0 + y1) + (y2 + y3));  mean = block256_sum(s) / dim;
//   q_t = sum_j fma(d0,d0, fma(d1,d1, fma(d2,d2, d3*d3))), d = y - mean;  var = block256_sum(q) / dim;
//   out = ((y - mean) / sqrt(var + eps)) * gamma + beta.
__global__ void __launch_bounds__(kRowThreads)
add_layernorm_kernel(const float* __restrict__ a, const float* __restrict__ resid, const float* __restrict__ gamma,
                     const float* __restrict__ beta, float eps, int dim, float* __restrict__ out, float* __restrict__ rowmax,
                     unsigned* absmax_slot, unsigned* absmax_slot2) {
  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  pdl_wait();
  trace_stamp_start(th, kTrAddLn);
  __shared__ float redf[kRowThreads / 32];
  __shared__ unsigned redu[kRowThreads / 32];
  const int r = blockIdx.x;
  const float4* a4 = reinterpret_cast<const float4*>(a + static_cast<size_t>(r) * dim);
  const float4* r4 = resid ? reinterpret_cast<const float4*>(resid + static_cast<size_t>(r) * dim) : nullptr;
  float4 v[kMaxVec];
  float s = 0.f;
#pragma unroll
  for(int j = 0; j < kMaxVec; ++j) {
    const int i = threadIdx.x + j * kRowThreads;
    if(i < dim / 4) {
      float4 x = a4[i];
      if(r4) {
        const float4 y = r4[i];
        x.x = __fadd_rn(x.x, y.x); x.y = __fadd_rn(x.y, y.y); x.z = __fadd_rn(x.z, y.z); x.w = __fadd_rn(x.w, y.w);
      }
      v[j] = x;
      s = __fadd_rn(s, __fadd_rn(__fadd_rn(x.x, x.y), __fadd_rn(x.z, x.w)));
    }
  }
  const float mean = __fdiv_rn(block256_sum_det(s, redf), static_cast<float>(dim));
  float q = 0.f;
#pragma unroll
  for(int j = 0; j < kMaxVec; ++j) {
    const int i = threadIdx.x + j * kRowThreads;
    if(i < dim / 4) {
      const float dx = __fadd_rn(v[j].x, -mean), dy = __fadd_rn(v[j].y, -mean), dz = __fadd_rn(v[j].z, -mean), dw = __fadd_rn(v[j].w, -mean);
      q = __fadd_rn(q, __fmaf_rn(dx, dx, __fmaf_rn(dy, dy, __fmaf_rn(dz, dz, __fmul_rn(dw, dw)))));
    }
  }
  const float var = __fdiv_rn(block256_sum_det(q, redf), static_cast<float>(dim));
  const float denom = __fsqrt_rn(__fadd_rn(var, eps));
  const float4* g4 = reinterpret_cast<const float4*>(gamma);
  const float4* b4 = reinterpret_cast<const float4*>(beta);
  float4* o4 = reinterpret_cast<float4*>(out + static_cast<size_t>(r) * dim);
  unsigned m = 0u;
#pragma unroll
  for(int j = 0; j < kMaxVec; ++j) {
    const int i = threadIdx.x + j * kRowThreads;
    if(i < dim / 4) {
      const float4 g = __ldg(g4 + i), b = __ldg(b4 + i);
      float4 o;
      o.x = __fadd_rn(__fmul_rn(__fdiv_rn(__fadd_rn(v[j].x, -mean), denom), g.x), b.x);
      o.y = __fadd_rn(__fmul_rn(__fdiv_rn(__fadd_rn(v[j].y, -mean), denom), g.y), b.y);
      o.z = __fadd_rn(__fmul_rn(__fdiv_rn(__fadd_rn(v[j].z, -mean), denom), g.z), b.z);
      o.w = __fadd_rn(__fmul_rn(__fdiv_rn(__fadd_rn(v[j].w, -mean), denom), g.w), b.w);
      o4[i] = o;
      m = max4u(m, o);
    }
  }
  m = block_max_u(m, redu);
  if(threadIdx.x == 0) {
    if(rowmax)
      rowmax[r] = __uint_as_float(m);
    if(absmax_slot)
      atomicMax(absmax_slot, m);
    if(absmax_slot2)
      atomicMax(absmax_slot2, m);
  }
  trace_stamp(tb, kTrAddLn, 2);
  trace_stamp(th.last, kTrAddLn, 3);
}

__device__ __forceinline__ int quantize_one(float v, float qm) {
  int r = __float2int_rn(__fmul_rn(v, qm));
  return max(-127, min(127, r));
}
__device__ __forceinline__ unsigned pack4(const float4& v, float qm) {
  return (static_cast<unsigned>(quantize_one(v.x, qm)) & 0xffu) | ((static_cast<unsigned>(quantize_one(v.y, qm)) & 0xffu) << 8) |
         ((static_cast<unsigned>(quantize_one(v.z, qm)) & 0xffu) << 16) | ((static_cast<unsigned>(quantize_one(v.w, qm)) & 0xffu) << 24);
}
__device__ __forceinline__ float quant_mult_from_bits(unsigned bits) {
  return bits == 0u ? 1.0f : __fdiv_rn(127.0f, __uint_as_float(bits));
}

// Quantise with the multiplier derived from an abs-max slot that a producer kernel already reduced.
// Optional row gather: source row of output row i is src_rows[i] (rows of `row_len` floats).
__global__ void __launch_bounds__(256)
quantize_slot_kernel(const float* __restrict__ x, size_t n, const unsigned* __restrict__ absmax_slot, int8_t* __restrict__ q,
                     float* __restrict__ d_quant_mult, int* status) {
  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  pdl_wait();
  trace_stamp_start(th, kTrQuantSlot);
  const unsigned bits = *absmax_slot;
  const float qm = quant_mult_from_bits(bits);
  if(blockIdx.x == 0 && threadIdx.x == 0) {
    *d_quant_mult = qm;
    if(bits >= 0x7f800000u)
      atomicMax(status, static_cast<int>(kDevNonFinite));
  }
  const size_t n16 = n / 16;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  uint4* q16 = reinterpret_cast<uint4*>(q);
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for(size_t i = tid; i < n16; i += stride) {
    const float4 a = __ldg(x4 + 4 * i), b = __ldg(x4 + 4 * i + 1), c = __ldg(x4 + 4 * i + 2), d = __ldg(x4 + 4 * i + 3);
    uint4 o;
    o.x = pack4(a, qm); o.y = pack4(b, qm); o.z = pack4(c, qm); o.w = pack4(d, qm);
    q16[i] = o;
  }
  for(size_t i = n16 * 16 + tid; i < n; i += stride)
    q[i] = static_cast<int8_t>(quantize_one(x[i], qm));
  trace_stamp(tb, kTrQuantSlot, 2);
  trace_stamp(th.last, kTrQuantSlot, 3);
}

// Two quantisations in one launch, for the start of a decoder self-attention block: blocks [0, blocks_x)
// quantise the layer input x with its own multiplier (the query projection's operand), the others the
// self-attention history with the multiplier of the whole live history (the key/value projections' operand):
// one slab row per block and iteration, only the newest slab (`rows_new` live rows) when the history's abs-max
// still has the bits the stored keys/values were computed with (*prev_bits), everything otherwise.
__global__ void __launch_bounds__(256)
quantize_dual_kernel(const float* __restrict__ x, size_t n, const unsigned* __restrict__ slot_x, int8_t* __restrict__ q,
                     float* __restrict__ qm_x, int* status, int blocks_x, const float* __restrict__ slabs, int slab_rows, int steps,
                     int rows_new, int dim, const unsigned* __restrict__ slot_h, const unsigned* __restrict__ prev_bits,
                     int8_t* __restrict__ hq, float* __restrict__ qm_h) {
  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  pdl_wait();
  trace_stamp_start(th, kTrQuantDual);
  if(static_cast<int>(blockIdx.x) < blocks_x) {
    const unsigned bits = *slot_x;
    const float qm = quant_mult_from_bits(bits);
    if(blockIdx.x == 0 && threadIdx.x == 0) {
      *qm_x = qm;
      if(bits >= 0x7f800000u)
        atomicMax(status, static_cast<int>(kDevNonFinite));
    }
    const size_t n16 = n / 16;   // (rows * dim with dim % 16 == 0: no tail)
    const float4* x4 = reinterpret_cast<const float4*>(x);
    uint4* q16 = reinterpret_cast<uint4*>(q);
    const size_t stride = static_cast<size_t>(blocks_x) * blockDim.x;
    for(size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += stride) {
      const float4 a = __ldg(x4 + 4 * i), b = __ldg(x4 + 4 * i + 1), c = __ldg(x4 + 4 * i + 2), d = __ldg(x4 + 4 * i + 3);
      uint4 o;
      o.x = pack4(a, qm); o.y = pack4(b, qm); o.z = pack4(c, qm); o.w = pack4(d, qm);
      q16[i] = o;
    }
  } else {
    const int hb = static_cast<int>(blockIdx.x) - blocks_x, nhb = static_cast<int>(gridDim.x) - blocks_x;
    const unsigned bits = *slot_h;
    const float qm = quant_mult_from_bits(bits);
    if(hb == 0 && threadIdx.x == 0)
      *qm_h = qm;
    const int total = (steps - 1) * slab_rows + rows_new;
    const int first = (*prev_bits == bits) ? (steps - 1) * slab_rows : 0;   // unchanged abs-max: only the newest slab
    for(int out_row = first + hb; out_row < total; out_row += nhb) {
      const float4* src = reinterpret_cast<const float4*>(slabs + static_cast<size_t>(out_row) * dim);
      uint4* dst = reinterpret_cast<uint4*>(hq + static_cast<size_t>(out_row) * dim);
      for(int i = threadIdx.x; i < dim / 16; i += blockDim.x) {
        const float4 a = __ldg(src + 4 * i), b = __ldg(src + 4 * i + 1), c = __ldg(src + 4 * i + 2), d = __ldg(src + 4 * i + 3);
        uint4 o;
        o.x = pack4(a, qm); o.y = pack4(b, qm); o.z = pack4(c, qm); o.w = pack4(d, qm);
        dst[i] = o;
      }
    }
  }
  trace_stamp(tb, kTrQuantDual, 2);
  trace_stamp(th.last, kTrQuantDual, 3);
}

// ---- self-attention history ------------------------------------------------------------------
// The decoder re-projects keys/values from the whole history of layer inputs every step, quantised
// with ONE multiplier over that history (src/models/transformer.h:401-417).  The history is kept as
// per-step slabs slab[t'][row][dim] in the row order of step t', plus an ancestor table
// anc[t'][r] = row of slab t' that current hypothesis r descends from, so a beam reorder only
// rewrites the small table.  rowmax[t'][row] holds max|x| of each slab row.

// anc_new[t'][r] = anc_old[t'][hyp[r]] (t' < t), anc_new[t][r] = r.
// With hist.layers > 0 the kernel also starts every layer's history abs-max of this step: for each layer l the
// maximum of rowmax_l[t'][anc_new[t'][r]] over the EARLIER slabs t' < t is reduced into hist.slot[l]; the producer
// of the layer's newest slab adds that slab's maximum to the same slot, which then holds what
// history_absmax_kernel computes in a launch of its own.
struct HistMaxArgs {
  int layers;
  const float* rowmax[kMaxHistLayers];
  unsigned* slot[kMaxHistLayers];
};
__global__ void __launch_bounds__(256)
ancestors_update_kernel(const int* __restrict__ anc_old, int* __restrict__ anc_new, const int* __restrict__ hyp,
                        int t, int rows, int stride, const HistMaxArgs hist) {
  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  pdl_wait();
  trace_stamp_start(th, kTrAncestors);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const bool in = i < (t + 1) * rows;
  int tp = 0, src = 0;
  if(in) {
    tp = i / rows;
    const int r = i - tp * rows;
    src = tp == t ? r : anc_old[tp * stride + hyp[r]];
    anc_new[tp * stride + r] = src;
  }
  for(int l = 0; l < hist.layers; ++l) {
    unsigned m = (in && tp < t) ? abs_bits(hist.rowmax[l][tp * stride + src]) : 0u;
    m = __reduce_max_sync(0xffffffffu, m);
    if((threadIdx.x & 31) == 0 && m != 0u)
      atomicMax(hist.slot[l], m);
  }
  trace_stamp(tb, kTrAncestors, 2);
  trace_stamp(th.last, kTrAncestors, 3);
}

// prev_bits[l] = slots[first + l * stride]: remembers, per layer, the abs-max the stored keys/values belong to.
// stats[0] counts (layer, step) pairs whose abs-max was unchanged, stats[1] all pairs.
__global__ void history_commit_kernel(unsigned* __restrict__ prev_bits, const unsigned* __restrict__ slots, int first, int stride, int layers,
                                      unsigned* __restrict__ stats) {
  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  pdl_wait();
  trace_stamp_start(th, kTrCommit);
  const int l = threadIdx.x;
  if(l < layers) {
    const unsigned now = slots[first + l * stride];
    if(stats) {
      if(prev_bits[l] == now)
        atomicAdd(stats, 1u);
      atomicAdd(stats + 1, 1u);
    }
    prev_bits[l] = now;
  }
  trace_stamp(tb, kTrCommit, 2);
  trace_stamp(th.last, kTrCommit, 3);
}

// ---- single-query attention --------------------------------------------------------------------
// One block per query row; thread i owns elements 4i..4i+3 of the model dimension, i.e. a quarter-row
// slice of head i / G with G = DH/4 threads per head.  For every key position the block reads the whole
// key row (all heads) with one 16-byte load per thread - fully coalesced whatever the layout of the
// history - and the G threads of a head combine their partial dot products with a butterfly.
// Key/value row of position p for query row r is  kv_base(r) + p * kv_stride:
//   mode 0, decoder self-attention over the time-major history:  base = r,              stride = rows
//   mode 1, cross-attention over the context [batch, len, dim]:   base = (r % batch)*len, stride = 1, log mask row r % batch
//   mode 2, encoder self-attention, rows ordered [batch, len]:    base = (r / len)*len,   stride = 1, log mask row r / len
// softmax(q.k / sqrt(dh) + mask) . v in fp32 (src/models/transformer.h:240-277).
// Arithmetic order per (row, head), restated identically by the CPU checker:
//   thread j of the head: d_j = fma(q3,k3, fma(q2,k2, fma(q1,k1, q0*k0))) over its four elements
//   s_p = butterfly over the G threads (d_j + d_{j^o}, o = G/2 .. 1);  s_p = s_p * scale;  s_p = s_p + mask_p
//   mx = max_p s_p;  e_p = det_expf(s_p - mx)
//   thread j accumulates e_p for p = j, j+G, ... ascending; sum = butterfly over the G threads
//   w_p = e_p / sum;  out_i = fma-chain over p ascending of w_p * v_{p,i}, starting from 0.
template <int DH, int U>
__global__ void __launch_bounds__(256)
attention1_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                  const float* __restrict__ log_mask, int heads, int len, int rows, int batch, int mode, float scale,
                  float* __restrict__ out, unsigned* absmax_slot, const int* __restrict__ anc, int anc_stride, int kv_rows) {
  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  pdl_wait();
  trace_stamp_start(th, kTrAttention1);
  extern __shared__ float sc_smem[];  // [heads][len] scores, then probabilities
  constexpr int G = DH / 4;
  const int r = blockIdx.x;
  // blockIdx.y selects the group of heads this block serves (blockDim.x / G heads, all of them when gridDim.y == 1);
  // `tid` is the thread's position in the row (quarter-row slice tid of the model dimension)
  const int hb = gridDim.y == 1 ? heads : static_cast<int>(blockDim.x) / G;
  const int tid = blockIdx.y * hb * G + threadIdx.x;
  const int dim = heads * DH;
  const bool active = tid < dim / 4;
  const int head = threadIdx.x / G, j = threadIdx.x % G;   // head inside the block's group
  const int group = mode == 1 ? r % batch : (mode == 2 ? r / len : 0);
  const size_t base = mode == 0 ? static_cast<size_t>(r) : static_cast<size_t>(group) * len;
  const size_t stride = (mode == 0 ? static_cast<size_t>(rows) : 1) * dim;
  const float* mask = (mode != 0 && log_mask) ? log_mask + static_cast<size_t>(group) * len : nullptr;
  const float4 qv = active ? __ldg(reinterpret_cast<const float4*>(q + static_cast<size_t>(r) * dim) + tid) : make_float4(0.f, 0.f, 0.f, 0.f);
  float* srow = sc_smem + (active ? head : 0) * len;
  // mode 0 with an ancestor table: keys/values are stored per step in that step's row order, and the row
  // of position p that query row r descends from is anc[p][r]
  const bool indirect = mode == 0 && anc != nullptr;
  int* anc_s = reinterpret_cast<int*>(sc_smem + hb * len);   // [len] ancestor rows of this query row
  if(indirect) {
    for(int p = threadIdx.x; p < len; p += blockDim.x)
      anc_s[p] = anc[static_cast<size_t>(p) * anc_stride + r];
    __syncthreads();
  }
  auto row_offset = [&](int p) -> size_t {
    if(indirect)
      return (static_cast<size_t>(p) * kv_rows + anc_s[p]) * dim + 4 * tid;
    return base * dim + 4 * tid + p * stride;
  };

  // scores: U key rows in flight per thread (the loads do not depend on one another; the arithmetic per
  // position is the same whatever U is)
  for(int p0 = 0; p0 < len; p0 += U) {
    float4 kk[U];
#pragma unroll
    for(int u = 0; u < U; ++u)
      kk[u] = (active && p0 + u < len) ? __ldg(reinterpret_cast<const float4*>(k + row_offset(p0 + u))) : make_float4(0.f, 0.f, 0.f, 0.f);
    float d[U];
#pragma unroll
    for(int u = 0; u < U; ++u) {
      d[u] = __fmul_rn(qv.x, kk[u].x);
      d[u] = __fmaf_rn(qv.y, kk[u].y, d[u]);
      d[u] = __fmaf_rn(qv.z, kk[u].z, d[u]);
      d[u] = __fmaf_rn(qv.w, kk[u].w, d[u]);
    }
    // The butterfly of the G threads of a head, for U positions at once: at the level that pairs lanes j and j ^ o the two
    // lanes split the positions still held between them - each sends the partial sums of the half it gives up and adds
    // what it receives to the half it keeps - so a level costs half as many shuffles and additions as the one before,
    // instead of one of each per position.  Every sum is "own + partner's" of the same two operands as in the plain
    // butterfly, hence the same bits.  Once a lane holds a single position the remaining levels are the plain butterfly.
    int pos = 0;
#pragma unroll
    for(int lvl = 0; ((G / 2) >> lvl) > 0; ++lvl) {
      const int o = (G / 2) >> lvl;
      const int c = (U >> lvl) > 1 ? (U >> lvl) : 1;   // positions a lane holds before this level
      if(c > 1) {
        const bool upper = (j & o) != 0;
#pragma unroll
        for(int i = 0; i < c / 2; ++i) {
          const float send = upper ? d[i] : d[i + c / 2];
          const float keep = upper ? d[i + c / 2] : d[i];
          d[i] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, o));
        }
        pos += upper ? c / 2 : 0;
      } else {
        d[0] = __fadd_rn(d[0], __shfl_xor_sync(0xffffffffu, d[0], o));
      }
    }
    // lanes that differ only in the bits of the plain levels hold the same position: the one with those bits clear writes
    // (with more positions than lanes a lane ends up holding U / G neighbouring positions)
    constexpr int kPlainMask = (U >= G) ? 0 : (G / U) - 1;
    constexpr int kHeld = U > G ? U / G : 1;
    if(active && (j & kPlainMask) == 0) {
#pragma unroll
      for(int i = 0; i < kHeld; ++i) {
        if(p0 + pos + i < len) {
          float sc = __fmul_rn(d[i], scale);
          if(mask)
            sc = __fadd_rn(sc, mask[p0 + pos + i]);
          srow[p0 + pos + i] = sc;
        }
      }
    }
  }
  __syncthreads();
  // softmax over the positions of this thread's head (the G threads of a head work together)
  float mx = -FLT_MAX;
  if(active)
    for(int p = j; p < len; p += G)
      mx = fmaxf(mx, srow[p]);
#pragma unroll
  for(int o = G / 2; o > 0; o >>= 1)
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float part = 0.f;
  if(active)
    for(int p = j; p < len; p += G) {
      const float e = det_expf(__fadd_rn(srow[p], -mx));
      srow[p] = e;
      part = __fadd_rn(part, e);
    }
#pragma unroll
  for(int o = G / 2; o > 0; o >>= 1)
    part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, o));
  if(active)
    for(int p = j; p < len; p += G)
      srow[p] = __fdiv_rn(srow[p], part);
  __syncthreads();
  // weighted sum of the value rows, strictly in position order, loads U rows ahead
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for(int p0 = 0; p0 < len; p0 += U) {
    float4 vv[U];
#pragma unroll
    for(int u = 0; u < U; ++u)
      vv[u] = (active && p0 + u < len) ? __ldg(reinterpret_cast<const float4*>(v + row_offset(p0 + u))) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for(int u = 0; u < U; ++u) {
      if(p0 + u < len) {
        const float w = srow[p0 + u];
        acc.x = __fmaf_rn(w, vv[u].x, acc.x);
        acc.y = __fmaf_rn(w, vv[u].y, acc.y);
        acc.z = __fmaf_rn(w, vv[u].z, acc.z);
        acc.w = __fmaf_rn(w, vv[u].w, acc.w);
      }
    }
  }
  unsigned m_abs = 0u;
  if(active) {
    reinterpret_cast<float4*>(out + static_cast<size_t>(r) * dim)[tid] = acc;
    m_abs = max4u(0u, acc);
  }
  if(absmax_slot) {
    m_abs = __reduce_max_sync(0xffffffffu, m_abs);
    if((threadIdx.x & 31) == 0 && m_abs != 0u)
      atomicMax(absmax_slot, m_abs);
  }
  trace_stamp(tb, kTrAttention1, 2);
  trace_stamp(th.last, kTrAttention1, 3);
}

// Encoder self-attention (mode 2) with the keys and values of one (sentence, head) staged in shared memory: block
// (b, h), thread = one query position (128 at a time).  attention1_kernel re-reads every key/value row once per
// query; here they cross L2 -> SM once per sentence and head.  The arithmetic per (row, head) is that of
// attention1_kernel restated for one thread: the G = DH/4 four-element partial dot products are combined in the
// butterfly's order (pairs G/2 apart first), the softmax sum as G interleaved partial sums combined the same way,
// the output as a fused-multiply-add chain over the positions in ascending order.
template <int G>
__device__ __forceinline__ float butterfly_order_sum(float (&a)[G]) {
#pragma unroll
  for(int o = G / 2; o > 0; o >>= 1) {
#pragma unroll
    for(int j = 0; j < o; ++j)
      a[j] = __fadd_rn(a[j], a[j + o]);
  }
  return a[0];
}

template <int DH>
__global__ void __launch_bounds__(128)
attention_enc_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                     const float* __restrict__ log_mask, int heads, int len, float scale, float* __restrict__ out,
                     unsigned* absmax_slot) {
  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  pdl_wait();
  trace_stamp_start(th, kTrAttentionEnc);
  extern __shared__ float enc_smem[];
  constexpr int G = DH / 4;
  const int b = blockIdx.x, h = blockIdx.y;
  const int dim = heads * DH;
  float* ks = enc_smem;                     // [len][DH]
  float* vs = ks + static_cast<size_t>(len) * DH;
  float* sc = vs + static_cast<size_t>(len) * DH;   // [len][128] scores / probabilities, position-major
  const size_t row0 = static_cast<size_t>(b) * len;
  for(int i = threadIdx.x; i < len * (DH / 4); i += blockDim.x) {
    const int p = i / (DH / 4), c = i % (DH / 4);
    const size_t off = (row0 + p) * dim + h * DH + 4 * c;
    reinterpret_cast<float4*>(ks)[i] = __ldg(reinterpret_cast<const float4*>(k + off));
    reinterpret_cast<float4*>(vs)[i] = __ldg(reinterpret_cast<const float4*>(v + off));
  }
  __syncthreads();
  const float* mask = log_mask ? log_mask + row0 : nullptr;
  unsigned m_abs = 0u;
  for(int q0 = 0; q0 < len; q0 += 128) {
    const int qi = q0 + threadIdx.x;
    const bool active = qi < len;
    float qv[DH];
    {
      const float4* q4 = reinterpret_cast<const float4*>(q + (row0 + (active ? qi : 0)) * dim + h * DH);
#pragma unroll
      for(int c = 0; c < DH / 4; ++c) {
        const float4 t = __ldg(q4 + c);
        qv[4 * c] = t.x; qv[4 * c + 1] = t.y; qv[4 * c + 2] = t.z; qv[4 * c + 3] = t.w;
      }
    }
    float mx = -FLT_MAX;
    for(int p = 0; p < len; ++p) {
      const float* kr = ks + p * DH;
      float a[G];
#pragma unroll
      for(int j = 0; j < G; ++j) {
        float d = __fmul_rn(qv[4 * j], kr[4 * j]);
        d = __fmaf_rn(qv[4 * j + 1], kr[4 * j + 1], d);
        d = __fmaf_rn(qv[4 * j + 2], kr[4 * j + 2], d);
        d = __fmaf_rn(qv[4 * j + 3], kr[4 * j + 3], d);
        a[j] = d;
      }
      float sv = __fmul_rn(butterfly_order_sum<G>(a), scale);
      if(mask)
        sv = __fadd_rn(sv, mask[p]);
      sc[p * 128 + threadIdx.x] = sv;
      mx = fmaxf(mx, sv);
    }
    float part[G];
#pragma unroll
    for(int j = 0; j < G; ++j)
      part[j] = 0.f;
    for(int p0 = 0; p0 < len; p0 += G) {
#pragma unroll
      for(int j = 0; j < G; ++j) {
        if(p0 + j < len) {
          const float e = det_expf(__fadd_rn(sc[(p0 + j) * 128 + threadIdx.x], -mx));
          sc[(p0 + j) * 128 + threadIdx.x] = e;
          part[j] = __fadd_rn(part[j], e);
        }
      }
    }
    const float total = butterfly_order_sum<G>(part);
    float acc[DH];
#pragma unroll
    for(int e = 0; e < DH; ++e)
      acc[e] = 0.f;
    for(int p = 0; p < len; ++p) {
      const float w = __fdiv_rn(sc[p * 128 + threadIdx.x], total);
      const float* vr = vs + p * DH;
#pragma unroll
      for(int e = 0; e < DH; ++e)
        acc[e] = __fmaf_rn(w, vr[e], acc[e]);
    }
    if(active) {
      float4* o4 = reinterpret_cast<float4*>(out + (row0 + qi) * dim + h * DH);
#pragma unroll
      for(int c = 0; c < DH / 4; ++c) {
        const float4 t = make_float4(acc[4 * c], acc[4 * c + 1], acc[4 * c + 2], acc[4 * c + 3]);
        o4[c] = t;
        m_abs = max4u(m_abs, t);
      }
    }
  }
  if(absmax_slot) {
    m_abs = __reduce_max_sync(0xffffffffu, m_abs);
    if((threadIdx.x & 31) == 0 && m_abs != 0u)
      atomicMax(absmax_slot, m_abs);
  }
  trace_stamp(tb, kTrAttentionEnc, 2);
  trace_stamp(th.last, kTrAttentionEnc, 3);
}

// ---- output layer: log-softmax + per-row top-k --------------------------------------------------
// Tree merge of the 256 per-thread sorted candidate lists in shared memory; the result is in list 0.
template <int K>
__device__ __forceinline__ void topk_block_merge(float* s_v, int* s_i) {
  for(int active = 128; active >= 1; active >>= 1) {
    if(threadIdx.x < active) {
      TopK a;
#pragma unroll
      for(int j = 0; j < K; ++j) {
        a.v[j] = s_v[threadIdx.x * K + j];
        a.i[j] = s_i[threadIdx.x * K + j];
      }
#pragma unroll
      for(int j = 0; j < K; ++j)
        topk_insert<K>(a, s_v[(threadIdx.x + active) * K + j], s_i[(threadIdx.x + active) * K + j]);
#pragma unroll
      for(int j = 0; j < K; ++j) {
        s_v[threadIdx.x * K + j] = a.v[j];
        s_i[threadIdx.x * K + j] = a.i[j];
      }
    }
    __syncthreads();
  }
}

// Combines the per-block pairs (m_b, s_b) of one row, held in shared memory, into the row's log-sum-exp:
// M = max_b m_b;  S = sum over b ascending of s_b * exp(m_b - M), product and sum rounded separately;
// lse = M + log(S).  bm/bs: nb entries each; red: 9 floats.  Every thread returns the same value.
__device__ __forceinline__ float lse_from_blocks(float* bm, float* bs, int nb, float* red) {
  float mx = -FLT_MAX;
  for(int b = threadIdx.x; b < nb; b += blockDim.x)
    mx = fmaxf(mx, bm[b]);
  for(int o = 16; o > 0; o >>= 1)
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  __syncthreads();
  if((threadIdx.x & 31) == 0)
    red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
  for(int w = 1; w < static_cast<int>(blockDim.x >> 5); ++w)
    mx = fmaxf(mx, red[w]);
  for(int b = threadIdx.x; b < nb; b += blockDim.x)
    bs[b] = __fmul_rn(bs[b], det_expf(__fadd_rn(bm[b], -mx)));
  __syncthreads();
  if(threadIdx.x == 0) {
    float total = 0.f;
    for(int b = 0; b < nb; ++b)
      total = __fadd_rn(total, bs[b]);
    red[8] = __fadd_rn(mx, det_logf(total));
  }
  __syncthreads();
  return red[8];
}

// One block per row: cand_score[r][j] = (j-th largest logit - logsumexp(row)) + prev_score[r], cand_word[r][j].
// The log-sum-exp is defined over blocks of 128 consecutive entries (the unit the output GEMM's write-back
// owns): per block its maximum m_b and s_b = sum of det_expf(x - m_b) with the entries added one after the
// other in ascending order; the blocks are combined by lse_from_blocks.  Thread t takes blocks t, t + 256, ...
template <int K>
__global__ void __launch_bounds__(256)
lse_topk_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ prev_scores, float* __restrict__ cand_score,
                int* __restrict__ cand_word) {
  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  pdl_wait();
  trace_stamp_start(th, kTrLseTopk);
  extern __shared__ float lse_blocks[];   // [nb] block maxima, [nb] block sums
  __shared__ float s_v[256 * K];
  __shared__ int s_i[256 * K];
  __shared__ float red[9];
  const int r = blockIdx.x;
  const float* row = logits + static_cast<size_t>(r) * vocab;
  const int nb = (vocab + 127) / 128;
  float* bm = lse_blocks;
  float* bs = lse_blocks + nb;
  const bool vec = (vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15u) == 0;
  TopK t;
#pragma unroll
  for(int j = 0; j < K; ++j) {
    t.v[j] = -FLT_MAX;
    t.i[j] = 0x7fffffff;
  }
  for(int b = threadIdx.x; b < nb; b += 256) {
    const int lo = b * 128, cnt = min(128, vocab - lo);
    float m = -FLT_MAX;
    if(vec && cnt == 128) {
      // whole block, 16-byte loads: 32 values at a time in registers, no per-value tests, so the conversions and
      // exponentials of a chunk overlap; only chunks that can change the candidate list are scanned
      const float4* p4 = reinterpret_cast<const float4*>(row + lo);
#pragma unroll 1
      for(int c = 0; c < 4; ++c) {
        float x[32];
#pragma unroll
        for(int j = 0; j < 8; ++j) {
          const float4 q = __ldg(p4 + c * 8 + j);
          x[4 * j] = q.x; x[4 * j + 1] = q.y; x[4 * j + 2] = q.z; x[4 * j + 3] = q.w;
        }
        float cm = x[0];
#pragma unroll
        for(int j = 1; j < 32; ++j)
          cm = fmaxf(cm, x[j]);
        m = fmaxf(m, cm);
        if(cm >= t.v[K - 1]) {
#pragma unroll
          for(int j = 0; j < 32; ++j)
            topk_insert<K>(t, x[j], lo + c * 32 + j);
        }
      }
      float sum = 0.f;
#pragma unroll 1
      for(int c = 0; c < 4; ++c) {
        float e[32];
#pragma unroll
        for(int j = 0; j < 8; ++j) {
          const float4 q = __ldg(p4 + c * 8 + j);
          e[4 * j] = det_expf(__fadd_rn(q.x, -m));
          e[4 * j + 1] = det_expf(__fadd_rn(q.y, -m));
          e[4 * j + 2] = det_expf(__fadd_rn(q.z, -m));
          e[4 * j + 3] = det_expf(__fadd_rn(q.w, -m));
        }
#pragma unroll
        for(int j = 0; j < 32; ++j)
          sum = __fadd_rn(sum, e[j]);
      }
      bs[b] = sum;
    } else if(vec) {
      const float4* p4 = reinterpret_cast<const float4*>(row + lo);
      for(int c = 0; c < cnt / 4; ++c) {
        const float4 x = __ldg(p4 + c);
        const int i = lo + 4 * c;
        m = fmaxf(m, fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w)));
        topk_insert<K>(t, x.x, i);
        topk_insert<K>(t, x.y, i + 1);
        topk_insert<K>(t, x.z, i + 2);
        topk_insert<K>(t, x.w, i + 3);
      }
      float sum = 0.f;
      for(int c = 0; c < cnt / 4; ++c) {
        const float4 x = __ldg(p4 + c);
        sum = __fadd_rn(sum, det_expf(__fadd_rn(x.x, -m)));
        sum = __fadd_rn(sum, det_expf(__fadd_rn(x.y, -m)));
        sum = __fadd_rn(sum, det_expf(__fadd_rn(x.z, -m)));
        sum = __fadd_rn(sum, det_expf(__fadd_rn(x.w, -m)));
      }
      bs[b] = sum;
    } else {
      for(int i = 0; i < cnt; ++i) {
        const float x = row[lo + i];
        m = fmaxf(m, x);
        topk_insert<K>(t, x, lo + i);
      }
      float sum = 0.f;
      for(int i = 0; i < cnt; ++i)
        sum = __fadd_rn(sum, det_expf(__fadd_rn(row[lo + i], -m)));
      bs[b] = sum;
    }
    bm[b] = m;
  }
#pragma unroll
  for(int j = 0; j < K; ++j) {
    s_v[threadIdx.x * K + j] = t.v[j];
    s_i[threadIdx.x * K + j] = t.i[j];
  }
  __syncthreads();
  const float lse = lse_from_blocks(bm, bs, nb, red);
  topk_block_merge<K>(s_v, s_i);
  if(threadIdx.x < K) {
    const float ps = prev_scores ? prev_scores[r] : 0.f;
    cand_score[r * K + threadIdx.x] = __fadd_rn(__fadd_rn(s_v[threadIdx.x], -lse), ps);
    cand_word[r * K + threadIdx.x] = s_i[threadIdx.x];
  }
  trace_stamp(tb, kTrLseTopk, 2);
  trace_stamp(th.last, kTrLseTopk, 3);
}

// Second half of the fused output layer: the GEMM's write-back left, per (row, block of 128 vocabulary entries),
// the block maximum, the block's sum of exponentials and its KT best entries; one block per row combines them
// into the row's log-sum-exp (lse_from_blocks) and its k best entries overall, exactly what lse_topk_kernel
// computes from materialised logits.
template <int KT>
__global__ void __launch_bounds__(256)
lse_merge_kernel(const float* __restrict__ blk_max, const float* __restrict__ blk_sum, const float* __restrict__ blk_topv,
                 const int* __restrict__ blk_topi, int nb, int k, const float* __restrict__ prev_scores, float* __restrict__ cand_score,
                 int* __restrict__ cand_word) {
  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  pdl_wait();
  trace_stamp_start(th, kTrLseMerge);
  extern __shared__ float lse_blocks[];
  __shared__ float s_v[256 * KT];
  __shared__ int s_i[256 * KT];
  __shared__ float red[9];
  const int r = blockIdx.x;
  float* bm = lse_blocks;
  float* bs = lse_blocks + nb;
  TopK t;
#pragma unroll
  for(int j = 0; j < KT; ++j) {
    t.v[j] = -FLT_MAX;
    t.i[j] = 0x7fffffff;
  }
  for(int b = threadIdx.x; b < nb; b += 256) {
    const size_t slot = static_cast<size_t>(r) * nb + b;
    bm[b] = blk_max[slot];
    bs[b] = blk_sum[slot];
#pragma unroll
    for(int j = 0; j < KT; ++j)
      topk_insert<KT>(t, blk_topv[slot * KT + j], blk_topi[slot * KT + j]);
  }
#pragma unroll
  for(int j = 0; j < KT; ++j) {
    s_v[threadIdx.x * KT + j] = t.v[j];
    s_i[threadIdx.x * KT + j] = t.i[j];
  }
  __syncthreads();
  const float lse = lse_from_blocks(bm, bs, nb, red);
  topk_block_merge<KT>(s_v, s_i);
  if(threadIdx.x < k) {
    const float ps = prev_scores ? prev_scores[r] : 0.f;
    cand_score[r * k + threadIdx.x] = __fadd_rn(__fadd_rn(s_v[threadIdx.x], -lse), ps);
    cand_word[r * k + threadIdx.x] = s_i[threadIdx.x];
  }
  trace_stamp(tb, kTrLseMerge, 2);
  trace_stamp(th.last, kTrLseMerge, 3);
}

// Per sentence b: merge the beam x K row candidates (rows beam-major: row = j * batch + b) into the
// K best, sorted; key order on ties = (beam j, rank) ascending, i.e. smaller flattened key first.
// out_score[b][n], out_beam[b][n], out_word[b][n].
template <int K>
__global__ void nbest_merge_kernel(const float* __restrict__ cand_score, const int* __restrict__ cand_word, int beam, int batch,
                                   int vocab, float* __restrict__ out_score, int* __restrict__ out_beam, int* __restrict__ out_word) {
  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  pdl_wait();
  trace_stamp_start(th, kTrNbest);
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if(b >= batch) {
    trace_stamp(tb, kTrNbest, 2);
    trace_stamp(th.last, kTrNbest, 3);
    return;
  }
  TopK t;
#pragma unroll
  for(int j = 0; j < K; ++j) {
    t.v[j] = -FLT_MAX;
    t.i[j] = 0x7fffffff;
  }
  for(int j = 0; j < beam; ++j) {
    const int row = j * batch + b;
    for(int c = 0; c < K; ++c) {
      const float s = cand_score[row * K + c];
      const int key = j * vocab + cand_word[row * K + c];  // the reference's flattened (beam, word) key
      // -inf candidates (dummy hypotheses) must stay behind every real one but keep a defined order
      topk_insert<K>(t, s == -INFINITY ? -FLT_MAX : s, key);
    }
  }
#pragma unroll
  for(int n = 0; n < K; ++n) {
    const bool valid = t.i[n] != 0x7fffffff && t.v[n] > -FLT_MAX;
    out_score[b * K + n] = valid ? t.v[n] : -INFINITY;
    out_beam[b * K + n] = valid ? t.i[n] / vocab : 0;
    out_word[b * K + n] = valid ? t.i[n] % vocab : 0;
  }
  trace_stamp(tb, kTrNbest, 2);
  trace_stamp(th.last, kTrNbest, 3);
}

// rows gather: out[i,:] = in[idx[i],:]  (16-byte copies when the row length allows it)
__global__ void gather_rows_kernel(const float* __restrict__ in, const int* __restrict__ idx, int dim, float* __restrict__ out) {
  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  pdl_wait();
  trace_stamp_start(th, kTrGather);
  const int r = blockIdx.x;
  const float* src = in + static_cast<size_t>(idx[r]) * dim;
  float* dst = out + static_cast<size_t>(r) * dim;
  if((dim & 3) == 0) {
    const float4* s4 = reinterpret_cast<const float4*>(src);
    float4* d4 = reinterpret_cast<float4*>(dst);
    for(int i = threadIdx.x; i < dim / 4; i += blockDim.x)
      d4[i] = __ldg(s4 + i);
  } else {
    for(int i = threadIdx.x; i < dim; i += blockDim.x)
      dst[i] = __ldg(src + i);
  }
  trace_stamp(tb, kTrGather, 2);
  trace_stamp(th.last, kTrGather, 3);
}

// SSRU cell (src/rnn/cells.h:1052-1066): c' = c[hyp] * sigmoid(f) + x * (1 - sigmoid(f)); h = relu(c').
// Writes the new cell state and y = LayerNorm(h + resid) * gamma + beta is done by add_layernorm on h.
__global__ void ssru_cell_kernel(const float* __restrict__ cell_old, const int* __restrict__ hyp, const float* __restrict__ xw,
                                 const float* __restrict__ f, int dim, float* __restrict__ cell_new, float* __restrict__ h_out) {
  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  pdl_wait();
  trace_stamp_start(th, kTrSsru);
  const int r = blockIdx.x;
  const float* c = cell_old + static_cast<size_t>(hyp ? hyp[r] : r) * dim;
  for(int i = threadIdx.x; i < dim; i += blockDim.x) {
    const size_t o = static_cast<size_t>(r) * dim + i;
    // sigmoid and highway with every rounding explicit: sig = 1 / (1 + det_expf(-f));
    // c' = fma(x, 1 - sig, c * sig)
    const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, det_expf(-f[o])));
    const float cn = __fmaf_rn(xw[o], __fadd_rn(1.0f, -sig), __fmul_rn(c[i], sig));
    cell_new[o] = cn;
    h_out[o] = cn > 0.f ? cn : 0.f;
  }
  trace_stamp(tb, kTrSsru, 2);
  trace_stamp(th.last, kTrSsru, 3);
}

int g_attention_block_heads = 8;   // heads one block of attention1_kernel serves (0 = all heads of the row)
int g_attention_unroll = 8;   // key/value rows a thread of attention1_kernel keeps in flight (8 or 16; 16 costs a block per SM and measured 7 % slower)

}  // namespace

MI8_DEFINE_TRACE_SETTER(trace_set_glue)
void set_attention_unroll(int u) { g_attention_unroll = u; }
void set_attention_block_heads(int h) { g_attention_block_heads = h; }

// ------------------------------------------------------------------------------------------------ launchers
int launch_embed(const float* wemb, const int* words, const float* pos, int pos_mod, float scale, int rows, int dim, float* out,
                 float* rowmax, unsigned* slot, cudaStream_t s, unsigned* slot2) {
  if(rows <= 0 || dim <= 0 || dim % 4 != 0 || dim > kRowThreads * 4 * kMaxVec || out == nullptr || pos == nullptr)
    return MI8_ERR_BAD_ARG;
  launch_kernel(embed_kernel, dim3(rows), dim3(kRowThreads), 0, s, wemb, words, pos, pos_mod, scale, dim, out, rowmax, slot, slot2);
  count_launch();
  return check_launch();
}

int launch_add_layernorm(const float* a, const float* resid, const float* gamma, const float* beta, float eps, int rows, int dim,
                         float* out, float* rowmax, unsigned* slot, cudaStream_t s, unsigned* slot2) {
  if(rows <= 0 || dim <= 0 || dim % 4 != 0 || dim > kRowThreads * 4 * kMaxVec || a == nullptr || out == nullptr)
    return MI8_ERR_BAD_ARG;
  launch_kernel(add_layernorm_kernel, dim3(rows), dim3(kRowThreads), 0, s, a, resid, gamma, beta, eps, dim, out, rowmax, slot, slot2);
  count_launch();
  return check_launch();
}

int launch_quantize_slot(const float* x, size_t n, const unsigned* slot, int8_t* q, float* d_qm, cudaStream_t s) {
  if(x == nullptr || q == nullptr || slot == nullptr || d_qm == nullptr || n == 0)
    return MI8_ERR_BAD_ARG;
  if((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(q) & 15u))
    return MI8_ERR_MISALIGNED;
  int* status = device_status_ptr();
  if(status == nullptr)
    return MI8_ERR_LAUNCH;
  size_t blocks = (n / 16 + 255) / 256;
  const size_t cap = static_cast<size_t>(sm_count()) * 8;
  blocks = blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
  launch_kernel(quantize_slot_kernel, dim3(static_cast<int>(blocks)), dim3(256), 0, s, x, n, slot, q, d_qm, status);
  count_launch();
  return check_launch();
}

int launch_ancestors_update(const int* anc_old, int* anc_new, const int* hyp, int t, int rows, int stride, cudaStream_t s,
                            int hist_layers, const float* const* hist_rowmax, unsigned* const* hist_slot) {
  if(hist_layers < 0 || hist_layers > kMaxHistLayers)
    return MI8_ERR_UNSUPPORTED;
  HistMaxArgs hist;
  hist.layers = hist_layers;
  for(int l = 0; l < kMaxHistLayers; ++l) {
    hist.rowmax[l] = l < hist_layers ? hist_rowmax[l] : nullptr;
    hist.slot[l] = l < hist_layers ? hist_slot[l] : nullptr;
  }
  const int n = (t + 1) * rows;
  launch_kernel(ancestors_update_kernel, dim3((n + 255) / 256), dim3(256), 0, s, anc_old, anc_new, hyp, t, rows, stride, hist);
  count_launch();
  return check_launch();
}

int launch_quantize_dual(const float* x, size_t n, const unsigned* slot_x, int8_t* q, float* qm_x, const float* slabs, int slab_rows,
                         int steps, int rows_new, int dim, const unsigned* slot_h, const unsigned* prev_bits, int8_t* hq, float* qm_h,
                         cudaStream_t s) {
  if(x == nullptr || q == nullptr || slot_x == nullptr || qm_x == nullptr || slabs == nullptr || slot_h == nullptr || prev_bits == nullptr ||
     hq == nullptr || qm_h == nullptr || n == 0 || steps <= 0 || rows_new <= 0 || rows_new > slab_rows)
    return MI8_ERR_BAD_ARG;
  if(dim % 16 != 0 || n % 16 != 0 || (reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(q) & 15u))
    return MI8_ERR_MISALIGNED;
  int* status = device_status_ptr();
  if(status == nullptr)
    return MI8_ERR_LAUNCH;
  size_t bx = (n / 16 + 255) / 256;
  const size_t cap = static_cast<size_t>(sm_count()) * 4;
  bx = bx < 1 ? 1 : (bx > cap ? cap : bx);
  // history part: one block per row of the newest slab (the common case); a full requantisation strides over the rest
  int bh = rows_new;
  const int hcap = sm_count() * 8;
  bh = bh > hcap ? hcap : bh;
  launch_kernel(quantize_dual_kernel, dim3(static_cast<unsigned>(bx) + bh), dim3(256), 0, s, x, n, slot_x, q, qm_x, status,
                static_cast<int>(bx), slabs, slab_rows, steps, rows_new, dim, slot_h, prev_bits, hq, qm_h);
  count_launch();
  return check_launch();
}

int launch_history_commit(unsigned* prev_bits, const unsigned* slots, int first, int stride, int layers, unsigned* stats, cudaStream_t s) {
  if(layers > 64)
    return MI8_ERR_UNSUPPORTED;
  launch_kernel(history_commit_kernel, dim3(1), dim3(64), 0, s, prev_bits, slots, first, stride, layers, stats);
  count_launch();
  return check_launch();
}

int launch_attention1(const float* q, const float* k, const float* v, const float* log_mask, int rows, int heads, int dim_head,
                      int len, int batch, int mode, float* out, unsigned* slot, cudaStream_t s, const int* anc, int anc_stride,
                      int kv_rows) {
  if(rows <= 0 || heads <= 0 || len <= 0)
    return MI8_ERR_BAD_ARG;
  if(mode < 0 || mode > 2)
    return MI8_ERR_BAD_ARG;
  const float scale = 1.0f / sqrtf(static_cast<float>(dim_head));
  const int dim = heads * dim_head;
  if(dim > 1024)
    return MI8_ERR_UNSUPPORTED;
  if(mode == 2 && batch > 0 && rows == batch * len && anc == nullptr && (dim_head == 64 || dim_head == 32)) {
    // encoder: keys/values of a (sentence, head) staged in shared memory, one thread per query position
    const size_t esmem = (static_cast<size_t>(len) * dim_head * 2 + static_cast<size_t>(len) * 128) * sizeof(float);
    if(esmem <= 200 * 1024) {
      static bool attr_set[64][2] = {};
      int dev = 0;
      cudaGetDevice(&dev);
      const int which = dim_head == 64 ? 0 : 1;
      if(dev >= 0 && dev < 64 && !attr_set[dev][which]) {
        cudaError_t e = which == 0 ? cudaFuncSetAttribute(attention_enc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                                   : cudaFuncSetAttribute(attention_enc_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if(e != cudaSuccess) {
          set_last_cuda_error(e);
          return MI8_ERR_LAUNCH;
        }
        attr_set[dev][which] = true;
      }
      if(which == 0)
        launch_kernel(attention_enc_kernel<64>, dim3(batch, heads), dim3(128), esmem, s, q, k, v, log_mask, heads, len, scale, out, slot);
      else
        launch_kernel(attention_enc_kernel<32>, dim3(batch, heads), dim3(128), esmem, s, q, k, v, log_mask, heads, len, scale, out, slot);
      count_launch();
      return check_launch();
    }
  }
  // A block serves `hb` heads of one query row.  Splitting a row over several smaller blocks changes nothing in the
  // arithmetic (heads are independent) and lets the SMs share the rows out evenly: 512 rows of 256 threads are 3.46
  // blocks per SM - some SMs get four, the others three - while halves or quarters of rows balance to within a few per cent.
  const int G = dim_head / 4;
  int hb = heads;
  if(g_attention_block_heads > 0 && heads % g_attention_block_heads == 0 && (g_attention_block_heads * G) % 32 == 0)
    hb = g_attention_block_heads;
  const int threads = ((hb * G + 31) / 32) * 32;
  const dim3 agrid(rows, heads / hb);
  const size_t smem = (static_cast<size_t>(hb) + 1) * len * sizeof(float);
  if(smem > 48 * 1024)
    return MI8_ERR_UNSUPPORTED;
  const bool wide = g_attention_unroll >= 16;
  if(dim_head == 64 && wide)
    launch_kernel(attention1_kernel<64, 16>, agrid, dim3(threads), smem, s, q, k, v, log_mask, heads, len, rows, batch, mode, scale, out, slot, anc, anc_stride, kv_rows);
  else if(dim_head == 64)
    launch_kernel(attention1_kernel<64, 8>, agrid, dim3(threads), smem, s, q, k, v, log_mask, heads, len, rows, batch, mode, scale, out, slot, anc, anc_stride, kv_rows);
  else if(dim_head == 32 && wide)
    launch_kernel(attention1_kernel<32, 16>, agrid, dim3(threads), smem, s, q, k, v, log_mask, heads, len, rows, batch, mode, scale, out, slot, anc, anc_stride, kv_rows);
  else if(dim_head == 32)
    launch_kernel(attention1_kernel<32, 8>, agrid, dim3(threads), smem, s, q, k, v, log_mask, heads, len, rows, batch, mode, scale, out, slot, anc, anc_stride, kv_rows);
  else
    return MI8_ERR_UNSUPPORTED;
  count_launch();
  return check_launch();
}

int launch_lse_topk(const float* logits, int rows, int vocab, int k, const float* prev_scores, float* cand_score, int* cand_word,
                    cudaStream_t s) {
  if(rows <= 0 || vocab <= 0 || k < 1 || k > kMaxK)
    return MI8_ERR_BAD_ARG;
  const size_t smem = 2 * static_cast<size_t>((vocab + 127) / 128) * sizeof(float);
  if(smem > 32 * 1024)
    return MI8_ERR_UNSUPPORTED;
  switch(k) {
    case 1: launch_kernel(lse_topk_kernel<1>, dim3(rows), dim3(256), smem, s, logits, vocab, prev_scores, cand_score, cand_word); break;
    case 2: launch_kernel(lse_topk_kernel<2>, dim3(rows), dim3(256), smem, s, logits, vocab, prev_scores, cand_score, cand_word); break;
    case 3: launch_kernel(lse_topk_kernel<3>, dim3(rows), dim3(256), smem, s, logits, vocab, prev_scores, cand_score, cand_word); break;
    case 4: launch_kernel(lse_topk_kernel<4>, dim3(rows), dim3(256), smem, s, logits, vocab, prev_scores, cand_score, cand_word); break;
    case 5: launch_kernel(lse_topk_kernel<5>, dim3(rows), dim3(256), smem, s, logits, vocab, prev_scores, cand_score, cand_word); break;
    case 6: launch_kernel(lse_topk_kernel<6>, dim3(rows), dim3(256), smem, s, logits, vocab, prev_scores, cand_score, cand_word); break;
    case 7: launch_kernel(lse_topk_kernel<7>, dim3(rows), dim3(256), smem, s, logits, vocab, prev_scores, cand_score, cand_word); break;
    default: launch_kernel(lse_topk_kernel<8>, dim3(rows), dim3(256), smem, s, logits, vocab, prev_scores, cand_score, cand_word); break;
  }
  count_launch();
  return check_launch();
}

int launch_lse_merge(const float* blk_max, const float* blk_sum, const float* blk_topv, const int* blk_topi, int rows, int vocab,
                     int k_top, int k, const float* prev_scores, float* cand_score, int* cand_word, cudaStream_t s) {
  if(rows <= 0 || vocab <= 0 || k < 1 || k > k_top || (k_top != 4 && k_top != 8))
    return MI8_ERR_BAD_ARG;
  const int nb = (vocab + 127) / 128;
  const size_t smem = 2 * static_cast<size_t>(nb) * sizeof(float);
  if(smem > 32 * 1024)
    return MI8_ERR_UNSUPPORTED;
  if(k_top == 4)
    launch_kernel(lse_merge_kernel<4>, dim3(rows), dim3(256), smem, s, blk_max, blk_sum, blk_topv, blk_topi, nb, k, prev_scores, cand_score,
                  cand_word);
  else
    launch_kernel(lse_merge_kernel<8>, dim3(rows), dim3(256), smem, s, blk_max, blk_sum, blk_topv, blk_topi, nb, k, prev_scores, cand_score,
                  cand_word);
  count_launch();
  return check_launch();
}

int launch_nbest_merge(const float* cand_score, const int* cand_word, int beam, int batch, int vocab, int k, float* out_score,
                       int* out_beam, int* out_word, cudaStream_t s) {
  if(k < 1 || k > kMaxK || beam < 1 || batch < 1)
    return MI8_ERR_BAD_ARG;
  const int blocks = (batch + 127) / 128;
  switch(k) {
    case 1: launch_kernel(nbest_merge_kernel<1>, dim3(blocks), dim3(128), 0, s, cand_score, cand_word, beam, batch, vocab, out_score, out_beam, out_word); break;
    case 2: launch_kernel(nbest_merge_kernel<2>, dim3(blocks), dim3(128), 0, s, cand_score, cand_word, beam, batch, vocab, out_score, out_beam, out_word); break;
    case 3: launch_kernel(nbest_merge_kernel<3>, dim3(blocks), dim3(128), 0, s, cand_score, cand_word, beam, batch, vocab, out_score, out_beam, out_word); break;
    case 4: launch_kernel(nbest_merge_kernel<4>, dim3(blocks), dim3(128), 0, s, cand_score, cand_word, beam, batch, vocab, out_score, out_beam, out_word); break;
    case 5: launch_kernel(nbest_merge_kernel<5>, dim3(blocks), dim3(128), 0, s, cand_score, cand_word, beam, batch, vocab, out_score, out_beam, out_word); break;
    case 6: launch_kernel(nbest_merge_kernel<6>, dim3(blocks), dim3(128), 0, s, cand_score, cand_word, beam, batch, vocab, out_score, out_beam, out_word); break;
    case 7: launch_kernel(nbest_merge_kernel<7>, dim3(blocks), dim3(128), 0, s, cand_score, cand_word, beam, batch, vocab, out_score, out_beam, out_word); break;
    default: launch_kernel(nbest_merge_kernel<8>, dim3(blocks), dim3(128), 0, s, cand_score, cand_word, beam, batch, vocab, out_score, out_beam, out_word); break;
  }
  count_launch();
  return check_launch();
}

int launch_gather_rows(const float* in, const int* idx, int rows, int dim, float* out, cudaStream_t s) {
  if(rows <= 0 || dim <= 0)
    return MI8_ERR_BAD_ARG;
  launch_kernel(gather_rows_kernel, dim3(rows), dim3(128), 0, s, in, idx, dim, out);
  count_launch();
  return check_launch();
}

int launch_ssru_cell(const float* cell_old, const int* hyp, const float* xw, const float* f, int rows, int dim, float* cell_new,
                     float* h_out, cudaStream_t s) {
  launch_kernel(ssru_cell_kernel, dim3(rows), dim3(256), 0, s, cell_old, hyp, xw, f, dim, cell_new, h_out);
  count_launch();
  return check_launch();
}

}  // namespace mi8
