// Float arithmetic of the glue kernels, written so that every rounding step is explicit.
//
// An int8 pipeline is chaotic at the 1/127 level: a one-ulp difference in a LayerNorm or softmax
// output flips a few quantised values, and two affines later the activations differ by a full
// quantisation step.  Two implementations of the decode therefore only agree if their float glue is
// bit-identical.  Everything here uses only correctly rounded IEEE operations (add, mul, fma, div,
// sqrt, rint) in a fixed order, so a CPU restatement with fmaf() reproduces it bit for bit; the
// library exp/log (whose last bits differ between CUDA and libm) are replaced by the fixed
// polynomials below.
#pragma once
#include <cuda_runtime.h>

namespace mi8 {

// exp(x): n = rint(x*log2(e)), r = x - n*ln2 (two-term), degree-6 Taylor polynomial, scaled by 2^n.
__device__ __forceinline__ float det_expf(float x) {
  if(x < -87.0f)
    return 0.0f;
  if(x > 88.0f)
    x = 88.0f;
  const float n = rintf(__fmul_rn(x, 1.44269504f));
  float r = __fmaf_rn(n, -0.693145752f, x);
  r = __fmaf_rn(n, -1.42860677e-06f, r);
  float p = 1.3888889e-3f;
  p = __fmaf_rn(p, r, 8.3333338e-3f);
  p = __fmaf_rn(p, r, 4.1666668e-2f);
  p = __fmaf_rn(p, r, 1.6666667e-1f);
  p = __fmaf_rn(p, r, 0.5f);
  p = __fmaf_rn(p, r, 1.0f);
  p = __fmaf_rn(p, r, 1.0f);
  const int e = static_cast<int>(n);
  return __fmul_rn(p, __int_as_float((e + 127) << 23));
}

// log(x) for finite x > 0 (normal numbers): x = m * 2^e with m in [sqrt(1/2), sqrt(2)),
// log(m) = 2 atanh(s), s = (m-1)/(m+1), odd series up to s^11.
__device__ __forceinline__ float det_logf(float x) {
  int bits = __float_as_int(x);
  int e = ((bits >> 23) & 0xff) - 127;
  float m = __int_as_float((bits & 0x007fffff) | 0x3f800000);
  if(m > 1.41421354f) {
    m = __fmul_rn(m, 0.5f);
    e += 1;
  }
  const float s = __fdiv_rn(__fadd_rn(m, -1.0f), __fadd_rn(m, 1.0f));
  const float s2 = __fmul_rn(s, s);
  float t = 0.181818187f;               // 2/11
  t = __fmaf_rn(t, s2, 0.222222224f);   // 2/9
  t = __fmaf_rn(t, s2, 0.285714298f);   // 2/7
  t = __fmaf_rn(t, s2, 0.400000006f);   // 2/5
  t = __fmaf_rn(t, s2, 0.666666687f);   // 2/3
  t = __fmul_rn(t, s2);
  const float lm = __fmaf_rn(s, t, __fmul_rn(2.0f, s));
  return __fmaf_rn(static_cast<float>(e), 0.693147182f, lm);
}

// Butterfly all-reduce over the 32 lanes of a warp: v <- v + v[lane ^ o] for o = 16, 8, 4, 2, 1.
// Floating-point addition is commutative, so every lane ends with the same bits.
__device__ __forceinline__ float warp_sum_det(float v) {
#pragma unroll
  for(int o = 16; o > 0; o >>= 1)
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of 256 threads: butterfly inside each warp, then the 8 warp totals added in
// ascending warp order starting from 0.  `red` is 8 floats of shared memory.
__device__ __forceinline__ float block256_sum_det(float v, float* red) {
  v = warp_sum_det(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if(lane == 0)
    red[warp] = v;
  __syncthreads();
  float t = 0.0f;
#pragma unroll
  for(int w = 0; w < 8; ++w)
    t = __fadd_rn(t, red[w]);
  return t;
}

// ---- small sorted candidate lists (value descending, ties to the smaller index), kept in registers
constexpr int kMaxK = 8;

struct TopK {
  float v[kMaxK];
  int i[kMaxK];
};

// larger value first; ties: smaller index first
__device__ __forceinline__ bool better(float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia < ib); }

// Inserts (v, idx) into the sorted list without branches: the K comparisons against the current entries are
// independent of one another (the list is sorted, so they form a prefix of false followed by true), then every
// entry either stays, takes its predecessor or takes the new value.  The only chain from one insertion to the
// next is a compare and a select, which keeps a scan over many values short on the critical path.
template <int K>
__device__ __forceinline__ void topk_insert(TopK& t, float v, int idx) {
  bool c[K];
#pragma unroll
  for(int j = 0; j < K; ++j)
    c[j] = better(v, idx, t.v[j], t.i[j]);
#pragma unroll
  for(int j = K - 1; j > 0; --j) {
    t.v[j] = c[j - 1] ? t.v[j - 1] : (c[j] ? v : t.v[j]);
    t.i[j] = c[j - 1] ? t.i[j - 1] : (c[j] ? idx : t.i[j]);
  }
  t.v[0] = c[0] ? v : t.v[0];
  t.i[0] = c[0] ? idx : t.i[0];
}

}  // namespace mi8
