// Abs-max reduction, fp32 -> int8 quantisation and the one-off weight conversion.
// All three are plain HBM-bound streaming kernels: 16-byte loads, several in flight per thread,
// grids sized from the SM count.
#include "mi8_internal.h"
#include "mi8_ptx.cuh"

namespace mi8 {

namespace {

constexpr int kBlock = 256;

__device__ __forceinline__ unsigned abs_bits(float v) { return __float_as_uint(v) & 0x7fffffffu; }

__device__ __forceinline__ unsigned max4(unsigned m, const float4& v) {
  m = max(m, abs_bits(v.x));
  m = max(m, abs_bits(v.y));
  m = max(m, abs_bits(v.z));
  m = max(m, abs_bits(v.w));
  return m;
}

// Block-wide maximum of an unsigned value; result valid in thread 0.
__device__ __forceinline__ unsigned block_max(unsigned m, unsigned* smem) {
  m = __reduce_max_sync(0xffffffffu, m);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if(lane == 0)
    smem[warp] = m;
  __syncthreads();
  if(warp == 0) {
    m = lane < (kBlock / 32) ? smem[lane] : 0u;
    m = __reduce_max_sync(0xffffffffu, m);
  }
  return m;
}

// |x| of non-negative IEEE floats orders like the unsigned integer of its bits, and Inf/NaN sort
// above every finite value, so one unsigned max finds both the maximum and non-finite input.
// Every block parks its maximum in `partials`; the last block to arrive reduces them, writes the
// results and resets the arrival counter.
__global__ void __launch_bounds__(kBlock)
mi8_absmax_kernel(const float* __restrict__ x, size_t n, unsigned* partials, unsigned* counter, float* d_absmax,
                  float* d_quant_mult, int* status) {
  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  pdl_wait();
  trace_stamp_start(th, kTrAbsmax);
  __shared__ unsigned red[kBlock / 32];
  __shared__ int is_last;
  unsigned m = 0u;
  const size_t n4 = n / 4;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  const size_t stride = static_cast<size_t>(gridDim.x) * kBlock;
  size_t i = static_cast<size_t>(blockIdx.x) * kBlock + threadIdx.x;
  for(; i + 3 * stride < n4; i += 4 * stride) {
    const float4 a = __ldg(x4 + i);
    const float4 b = __ldg(x4 + i + stride);
    const float4 c = __ldg(x4 + i + 2 * stride);
    const float4 d = __ldg(x4 + i + 3 * stride);
    m = max4(max4(max4(max4(m, a), b), c), d);
  }
  for(; i < n4; i += stride)
    m = max4(m, __ldg(x4 + i));
  if(blockIdx.x == 0 && threadIdx.x < (n & 3))
    m = max(m, abs_bits(x[n4 * 4 + threadIdx.x]));

  m = block_max(m, red);
  if(threadIdx.x == 0) {
    partials[blockIdx.x] = m;
    __threadfence();
    const unsigned old = atomicAdd(counter, 1u);
    is_last = (old == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if(!is_last) {
    trace_stamp(tb, kTrAbsmax, 2);
    trace_stamp(th.last, kTrAbsmax, 3);
    return;
  }
  __threadfence();
  m = 0u;
  for(unsigned b = threadIdx.x; b < gridDim.x; b += kBlock)
    m = max(m, __ldcg(partials + b));
  __syncthreads();  // `red` is reused
  m = block_max(m, red);
  if(threadIdx.x == 0) {
    *counter = 0u;  // leave the workspace zeroed for the next call
    if(m >= 0x7f800000u)
      atomicMax(status, static_cast<int>(kDevNonFinite));
    const float mx = __uint_as_float(m);
    if(d_absmax != nullptr)
      *d_absmax = mx;
    if(d_quant_mult != nullptr)
      *d_quant_mult = (m == 0u) ? 1.0f : __fdiv_rn(127.0f, mx);
  }
  trace_stamp(tb, kTrAbsmax, 2);
  trace_stamp(th.last, kTrAbsmax, 3);
}

__device__ __forceinline__ int quantize_one(float v, float qm) {
  int r = __float2int_rn(__fmul_rn(v, qm));  // round half to even; NaN -> 0
  return max(-127, min(127, r));              // -128 is never produced
}

__device__ __forceinline__ unsigned pack4(const float4& v, float qm) {
  return (static_cast<unsigned>(quantize_one(v.x, qm)) & 0xffu) | ((static_cast<unsigned>(quantize_one(v.y, qm)) & 0xffu) << 8) |
         ((static_cast<unsigned>(quantize_one(v.z, qm)) & 0xffu) << 16) | ((static_cast<unsigned>(quantize_one(v.w, qm)) & 0xffu) << 24);
}

// 16 floats in (four 16-byte loads), 16 int8 out (one 16-byte store) per thread and iteration.
__global__ void __launch_bounds__(kBlock)
mi8_quantize_kernel(const float* __restrict__ x, size_t n, const float* __restrict__ d_quant_mult, int8_t* __restrict__ q) {
  pdl_launch_dependents();
  const TraceHandles th = trace_open_all();
  unsigned long long* const tb = th.first;
  pdl_wait();
  trace_stamp_start(th, kTrQuantize);
  const float qm = *d_quant_mult;
  const size_t n16 = n / 16;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  uint4* q16 = reinterpret_cast<uint4*>(q);
  const size_t stride = static_cast<size_t>(gridDim.x) * kBlock;
  const size_t tid = static_cast<size_t>(blockIdx.x) * kBlock + threadIdx.x;
  for(size_t i = tid; i < n16; i += stride) {
    const float4 a = __ldg(x4 + 4 * i);
    const float4 b = __ldg(x4 + 4 * i + 1);
    const float4 c = __ldg(x4 + 4 * i + 2);
    const float4 d = __ldg(x4 + 4 * i + 3);
    uint4 o;
    o.x = pack4(a, qm);
    o.y = pack4(b, qm);
    o.z = pack4(c, qm);
    o.w = pack4(d, qm);
    q16[i] = o;
  }
  for(size_t i = n16 * 16 + tid; i < n; i += stride)
    q[i] = static_cast<int8_t>(quantize_one(x[i], qm));
  trace_stamp(tb, kTrQuantize, 2);
  trace_stamp(th.last, kTrQuantize, 3);
}

// W fp32 [K,N] row-major -> Bt int8 [N,K] row-major.  A block moves a 32(k) x 32(n) tile through
// shared memory so that both the fp32 reads (along n) and the int8 writes (along k) are contiguous.
__global__ void __launch_bounds__(256)
mi8_transpose_quantize_kernel(const float* __restrict__ w, int K, int N, const float* __restrict__ d_quant_mult,
                              int8_t* __restrict__ bt) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float tile[32][33];
  const float qm = *d_quant_mult;
  const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
  for(int r = 0; r < 32; r += 8) {
    const int k = k0 + ty + r, n = n0 + tx;
    tile[ty + r][tx] = (k < K && n < N) ? w[static_cast<size_t>(k) * N + n] : 0.0f;
  }
  __syncthreads();
#pragma unroll
  for(int r = 0; r < 32; r += 8) {
    const int n = n0 + ty + r, k = k0 + tx;
    if(n < N && k < K)
      bt[static_cast<size_t>(n) * K + k] = static_cast<int8_t>(quantize_one(tile[tx][ty + r], qm));
  }
}

// out[b][c][r] = in[b][r][c]: the last two axes of a float tensor swapped, 32 x 32 tiles through shared memory so that
// reads and writes are both contiguous.  (Serves affine / dot with transA, which the reference resolves by a transpose
// node in front of the quantisation, src/tensors/cpu/intgemm_interface.h:52.)
__global__ void __launch_bounds__(256)
mi8_transpose_f32_kernel(const float* __restrict__ in, int rows, int cols, float* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float tile[32][33];
  const size_t plane = static_cast<size_t>(rows) * cols;
  const float* src = in + blockIdx.z * plane;
  float* dst = out + blockIdx.z * plane;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for(int i = 0; i < 32; i += 8) {
    const int r = r0 + ty + i, c = c0 + tx;
    tile[ty + i][tx] = (r < rows && c < cols) ? src[static_cast<size_t>(r) * cols + c] : 0.0f;
  }
  __syncthreads();
#pragma unroll
  for(int i = 0; i < 32; i += 8) {
    const int c = c0 + ty + i, r = r0 + tx;
    if(c < cols && r < rows)
      dst[static_cast<size_t>(c) * rows + r] = tile[tx][ty + i];
  }
}

int stream_grid(size_t work_items) {
  const size_t per_block = static_cast<size_t>(kBlock) * 4;
  size_t blocks = (work_items + per_block - 1) / per_block;
  const size_t cap = static_cast<size_t>(sm_count()) * 8;
  if(blocks > cap)
    blocks = cap;
  if(blocks < 1)
    blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace

MI8_DEFINE_TRACE_SETTER(trace_set_quant)

int launch_max_absolute(const float* x, size_t n, float* d_absmax, float* d_quant_mult, void* ws, size_t ws_bytes,
                        cudaStream_t stream) {
  if(x == nullptr || n == 0)
    return MI8_ERR_BAD_ARG;
  if(ws == nullptr || ws_bytes < kWsHeaderBytes)
    return MI8_ERR_WORKSPACE;
  if(reinterpret_cast<uintptr_t>(x) & 15u)
    return MI8_ERR_MISALIGNED;
  int* status = device_status_ptr();
  if(status == nullptr)
    return MI8_ERR_LAUNCH;
  uint8_t* wsb = static_cast<uint8_t*>(ws);
  int grid = stream_grid(n / 4 + 1);
  if(grid > kWsMaxAbsmaxBlocks)
    grid = kWsMaxAbsmaxBlocks;
  launch_kernel(mi8_absmax_kernel, dim3(grid), dim3(kBlock), 0, stream, x, n, reinterpret_cast<unsigned*>(wsb + kWsOffAbsmaxPartials),
                                                 reinterpret_cast<unsigned*>(wsb + kWsOffAbsmaxCounter), d_absmax,
                                                 d_quant_mult, status);
  count_launch();
  return check_launch();
}

int launch_quantize(const float* x, size_t n, const float* d_quant_mult, int8_t* q, cudaStream_t stream) {
  if(x == nullptr || q == nullptr || d_quant_mult == nullptr || n == 0)
    return MI8_ERR_BAD_ARG;
  if((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(q) & 15u))
    return MI8_ERR_MISALIGNED;
  const int grid = stream_grid(n / 16 + 1);
  launch_kernel(mi8_quantize_kernel, dim3(grid), dim3(kBlock), 0, stream, x, n, d_quant_mult, q);
  count_launch();
  return check_launch();
}

int launch_transpose_quantize(const float* w, int K, int N, const float* d_quant_mult, int8_t* bt, cudaStream_t stream) {
  if(w == nullptr || bt == nullptr || d_quant_mult == nullptr || K <= 0 || N <= 0)
    return MI8_ERR_BAD_ARG;
  dim3 grid((N + 31) / 32, (K + 31) / 32);
  if(grid.y > 65535)
    return MI8_ERR_UNSUPPORTED;
  launch_kernel(mi8_transpose_quantize_kernel, dim3(grid), dim3(256), 0, stream, w, K, N, d_quant_mult, bt);
  count_launch();
  return check_launch();
}

int launch_transpose_f32(const float* in, int batch, int rows, int cols, float* out, cudaStream_t stream) {
  if(in == nullptr || out == nullptr || batch <= 0 || rows <= 0 || cols <= 0)
    return MI8_ERR_BAD_ARG;
  dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch);
  if(grid.y > 65535 || grid.z > 65535)
    return MI8_ERR_UNSUPPORTED;
  launch_kernel(mi8_transpose_f32_kernel, grid, dim3(256), 0, stream, in, rows, cols, out);
  count_launch();
  return check_launch();
}

}  // namespace mi8
