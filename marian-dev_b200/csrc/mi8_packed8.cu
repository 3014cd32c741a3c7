// packed8avx512 items (the FBGEMM / mjdgemm int8 scheme of the reference) on the same tcgen05 GEMM:
//   * the block-ordered weight item is put back into Bt[N,K] row-major once, at load time;
//   * the activation is quantised per ROW to uint8 with a scale, a zero point and the row's sum
//     (marian::cpu::mjdgemm computeQuantizationParams + quantize, AVX-512 route,
//      src/tensors/cpu/mjdgemm/mjdgemm_avx512.cpp:195-276);
//   * the GEMM runs uint8 x int8 and its write-back applies the zero-point corrections (mi8_gemm.cu).
// Both kernels here are HBM-bound streaming kernels.
#include <algorithm>

#include "mi8_internal.h"
#include "mi8_ptx.cuh"

namespace mi8 {

namespace {

constexpr int kBlock = 256;
constexpr int kKcb = 256;   // rows of one weight block (BlockingFactors::KCB, src/tensors/cpu/mjdgemm/mjdgemm_utils.h:33-43)
constexpr int kNcb = 32;    // columns of one weight block
constexpr int kRi = 4;      // consecutive rows stored together (row interleave)

// packB (src/tensors/cpu/mjdgemm/mjdgemm_utils.h:136-165) stores the weights as
// [K/256][N/32][64 row groups][32 columns][4 rows].  A thread moves one 4-byte row group: consecutive
// threads read consecutive words of the item and write bt[n][4 * kq .. 4 * kq + 3].
__global__ void __launch_bounds__(kBlock)
p8_unpack_bt_kernel(const uint32_t* __restrict__ packed, int K, int N, uint32_t* __restrict__ bt) {
  pdl_wait();
  const size_t words = static_cast<size_t>(K) * N / kRi;
  const size_t stride = static_cast<size_t>(gridDim.x) * kBlock;
  constexpr int kBlockWords = kKcb * kNcb / kRi;
  const int n_blocks = N / kNcb;
  for(size_t w = static_cast<size_t>(blockIdx.x) * kBlock + threadIdx.x; w < words; w += stride) {
    const size_t blk = w / kBlockWords;
    const int in = static_cast<int>(w % kBlockWords);
    const int kb = static_cast<int>(blk / n_blocks), nb = static_cast<int>(blk % n_blocks);
    const int group = in / kNcb, nc = in % kNcb;
    const int n = nb * kNcb + nc;
    const int k = kb * kKcb + group * kRi;
    bt[(static_cast<size_t>(n) * K + k) / kRi] = __ldg(packed + w);
  }
}

// Offline conversion of one fp32 weight [K,N] into a packed8avx512 item (fbgemmPacked8Pack with min/max ranges,
// src/tensors/cpu/fbgemm/packed_gemm.cpp:372-480): per column scaleB = (max - min) / 127,
// zeroPointB = trunc(63 - max / scaleB), q = nearest_even(clamp(zeroPointB + x / scaleB, -64, 63)) (7-bit range),
// colOffsetsB = sum of the column's q - zeroPointB * K; weights in the block order of the item, the three arrays behind them.
// One block converts the 32 columns of one block column: warp w takes the row groups w, w + 8, ... (four
// consecutive rows each), lane = column, so every load is one 128-byte line and every store one 128-byte run.
__global__ void __launch_bounds__(kBlock)
p8_prepare_b_kernel(const float* __restrict__ w, int K, int N, uint32_t* __restrict__ packed, float* __restrict__ scale_b,
                    int32_t* __restrict__ zp_b, int32_t* __restrict__ off_b) {
  pdl_wait();
  __shared__ float s_min[kBlock / 32][kNcb], s_max[kBlock / 32][kNcb];
  __shared__ int s_sum[kBlock / 32][kNcb];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nb = blockIdx.x, n = nb * kNcb + lane;
  float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
  for(int k = warp; k < K; k += kBlock / 32) {
    const float v = __ldg(w + static_cast<size_t>(k) * N + n);
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
  s_min[warp][lane] = mn;
  s_max[warp][lane] = mx;
  __syncthreads();
#pragma unroll
  for(int i = 0; i < kBlock / 32; ++i) {
    mn = fminf(mn, s_min[i][lane]);
    mx = fmaxf(mx, s_max[i][lane]);
  }
  float s = __fdiv_rn(__fsub_rn(mx, mn), 127.0f);
  if(!(s > 0.0f))
    s = 1.0f;   // constant column
  const int z = __float2int_rz(__fsub_rn(63.0f, __fdiv_rn(mx, s)));
  const float zf = __int2float_rn(z);
  int sum = 0;
  const int n_blocks = N / kNcb;
  for(int g = warp; g < K / kRi; g += kBlock / 32) {
    uint32_t word = 0;
#pragma unroll
    for(int r = 0; r < kRi; ++r) {
      const float x = __ldg(w + static_cast<size_t>(g * kRi + r) * N + n);
      const float t = fminf(fmaxf(__fadd_rn(zf, __fdiv_rn(x, s)), -64.0f), 63.0f);
      const int q = __float2int_rn(t);
      sum += q;
      word |= (static_cast<uint32_t>(q) & 0xffu) << (8 * r);
    }
    const int kb = (g * kRi) / kKcb, group = (g * kRi % kKcb) / kRi;
    packed[(static_cast<size_t>(kb) * n_blocks + nb) * (kKcb * kNcb / kRi) + group * kNcb + lane] = word;
  }
  s_sum[warp][lane] = sum;
  __syncthreads();
  if(warp == 0) {
    int total = 0;
#pragma unroll
    for(int i = 0; i < kBlock / 32; ++i)
      total += s_sum[i][lane];
    scale_b[n] = s;
    zp_b[n] = z;
    off_b[n] = total - z * K;
  }
}

__device__ __forceinline__ float block_reduce(float v, float* smem, bool is_max) {
#pragma unroll
  for(int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, other) : fminf(v, other);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();   // smem may still be read from the previous use
  if(lane == 0)
    smem[warp] = v;
  __syncthreads();
  v = smem[0];
#pragma unroll
  for(int i = 1; i < kBlock / 32; ++i)
    v = is_max ? fmaxf(v, smem[i]) : fminf(v, smem[i]);
  return v;
}

// One block per activation row: minimum and maximum, then
//   scaleA = (max - min) / 255, zeroPointA = trunc(255 - max / scaleA),
//   q = nearest_even(min(max(fma(x, 1 / scaleA, zeroPointA), 0), 255)), sumA = sum of q.
// A row whose values are all equal (the reference divides by zero there) first widens its range to
// contain 0; an all-zero row takes scaleA = 1.  Inf or NaN in the row raises the non-finite status.
__global__ void __launch_bounds__(kBlock)
p8_quantize_rows_kernel(const float* __restrict__ a, int K, uint8_t* __restrict__ aq, float* __restrict__ scale_a, int32_t* __restrict__ zp_a,
                        int32_t* __restrict__ sum_a, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[kBlock / 32];
  __shared__ int red_i[kBlock / 32];
  const int m = blockIdx.x;
  const float4* row = reinterpret_cast<const float4*>(a + static_cast<size_t>(m) * K);
  const int k4 = K / 4;
  float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
  unsigned bits = 0u;
  for(int i = threadIdx.x; i < k4; i += kBlock) {
    const float4 v = __ldg(row + i);
    mn = fminf(fminf(mn, v.x), fminf(v.y, fminf(v.z, v.w)));
    mx = fmaxf(fmaxf(mx, v.x), fmaxf(v.y, fmaxf(v.z, v.w)));
    bits = max(max(bits, __float_as_uint(v.x) & 0x7fffffffu), max(__float_as_uint(v.y) & 0x7fffffffu,
               max(__float_as_uint(v.z) & 0x7fffffffu, __float_as_uint(v.w) & 0x7fffffffu)));
  }
  mn = block_reduce(mn, red, false);
  mx = block_reduce(mx, red, true);
  if(bits >= 0x7f800000u)
    atomicMax(status, static_cast<int>(kDevNonFinite));
  if(mn == mx) {
    mn = fminf(mn, 0.0f);
    mx = fmaxf(mx, 0.0f);
  }
  float s = __fdiv_rn(__fsub_rn(mx, mn), 255.0f);
  if(mn == mx)
    s = 1.0f;
  const int z = __float2int_rz(__fsub_rn(255.0f, __fdiv_rn(mx, s)));
  const float inv = __fdiv_rn(1.0f, s), zf = __int2float_rn(z);
  int sum = 0;
  uint32_t* out = reinterpret_cast<uint32_t*>(aq + static_cast<size_t>(m) * K);
  for(int i = threadIdx.x; i < k4; i += kBlock) {
    const float4 v = __ldg(row + i);
    const int q0 = __float2int_rn(fminf(fmaxf(__fmaf_rn(v.x, inv, zf), 0.0f), 255.0f));
    const int q1 = __float2int_rn(fminf(fmaxf(__fmaf_rn(v.y, inv, zf), 0.0f), 255.0f));
    const int q2 = __float2int_rn(fminf(fmaxf(__fmaf_rn(v.z, inv, zf), 0.0f), 255.0f));
    const int q3 = __float2int_rn(fminf(fmaxf(__fmaf_rn(v.w, inv, zf), 0.0f), 255.0f));
    sum += q0 + q1 + q2 + q3;
    out[i] = static_cast<uint32_t>(q0) | (static_cast<uint32_t>(q1) << 8) | (static_cast<uint32_t>(q2) << 16) | (static_cast<uint32_t>(q3) << 24);
  }
  sum = __reduce_add_sync(0xffffffffu, sum);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if(lane == 0)
    red_i[warp] = sum;
  __syncthreads();
  if(threadIdx.x == 0) {
    int total = 0;
#pragma unroll
    for(int i = 0; i < kBlock / 32; ++i)
      total += red_i[i];
    scale_a[m] = s;
    zp_a[m] = z;
    sum_a[m] = total;
  }
}

__device__ __forceinline__ int p8_q(float x, float inv, float zf) {
  return __float2int_rn(fminf(fmaxf(__fmaf_rn(x, inv, zf), 0.0f), 255.0f));
}

// The same for rows of at most 128 * kVec values: one WARP per row, the row held in registers (kVec 16-byte loads per
// lane, all issued before the first use), statistics by shuffles - one pass over global memory and no block barrier.
template <int kVec>
__global__ void __launch_bounds__(kBlock)
p8_quantize_rows_warp_kernel(const float* __restrict__ a, int M, int K, uint8_t* __restrict__ aq, float* __restrict__ scale_a,
                             int32_t* __restrict__ zp_a, int32_t* __restrict__ sum_a, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int m = blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5);
  if(m >= M)
    return;
  const float4* row = reinterpret_cast<const float4*>(a + static_cast<size_t>(m) * K);
  const int k4 = K / 4;
  float4 v[kVec];
#pragma unroll
  for(int i = 0; i < kVec; ++i) {
    const int idx = lane + 32 * i;
    v[i] = idx < k4 ? __ldg(row + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
  unsigned bits = 0u;
#pragma unroll
  for(int i = 0; i < kVec; ++i) {
    if(lane + 32 * i < k4) {
      mn = fminf(fminf(mn, v[i].x), fminf(v[i].y, fminf(v[i].z, v[i].w)));
      mx = fmaxf(fmaxf(mx, v[i].x), fmaxf(v[i].y, fmaxf(v[i].z, v[i].w)));
      bits = max(max(bits, __float_as_uint(v[i].x) & 0x7fffffffu), max(__float_as_uint(v[i].y) & 0x7fffffffu,
                 max(__float_as_uint(v[i].z) & 0x7fffffffu, __float_as_uint(v[i].w) & 0x7fffffffu)));
    }
  }
#pragma unroll
  for(int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if(bits >= 0x7f800000u)
    atomicMax(status, static_cast<int>(kDevNonFinite));
  if(mn == mx) {
    mn = fminf(mn, 0.0f);
    mx = fmaxf(mx, 0.0f);
  }
  float s = __fdiv_rn(__fsub_rn(mx, mn), 255.0f);
  if(mn == mx)
    s = 1.0f;
  const int z = __float2int_rz(__fsub_rn(255.0f, __fdiv_rn(mx, s)));
  const float inv = __fdiv_rn(1.0f, s), zf = __int2float_rn(z);
  int sum = 0;
  uint32_t* out = reinterpret_cast<uint32_t*>(aq + static_cast<size_t>(m) * K);
#pragma unroll
  for(int i = 0; i < kVec; ++i) {
    const int idx = lane + 32 * i;
    if(idx < k4) {
      const int q0 = p8_q(v[i].x, inv, zf), q1 = p8_q(v[i].y, inv, zf), q2 = p8_q(v[i].z, inv, zf), q3 = p8_q(v[i].w, inv, zf);
      sum += q0 + q1 + q2 + q3;
      out[idx] = static_cast<uint32_t>(q0) | (static_cast<uint32_t>(q1) << 8) | (static_cast<uint32_t>(q2) << 16) | (static_cast<uint32_t>(q3) << 24);
    }
  }
  sum = __reduce_add_sync(0xffffffffu, sum);
  if(lane == 0) {
    scale_a[m] = s;
    zp_a[m] = z;
    sum_a[m] = sum;
  }
}

}  // namespace

int launch_p8_unpack_bt(const int8_t* packed, int K, int N, int8_t* bt, cudaStream_t stream) {
  if(packed == nullptr || bt == nullptr || K <= 0 || N <= 0)
    return MI8_ERR_BAD_ARG;
  if(K % kKcb != 0 || N % kNcb != 0)
    return MI8_ERR_UNSUPPORTED;   // the reference's packB has no padding either
  if((reinterpret_cast<uintptr_t>(packed) & 3u) || (reinterpret_cast<uintptr_t>(bt) & 15u))
    return MI8_ERR_MISALIGNED;
  const size_t words = static_cast<size_t>(K) * N / kRi;
  const int grid = static_cast<int>(std::min<size_t>((words + kBlock - 1) / kBlock, static_cast<size_t>(sm_count()) * 16));
  cudaError_t e = launch_kernel(p8_unpack_bt_kernel, dim3(grid), dim3(kBlock), 0, stream, reinterpret_cast<const uint32_t*>(packed), K, N,
                                reinterpret_cast<uint32_t*>(bt));
  if(e != cudaSuccess) {
    set_last_cuda_error(e);
    return MI8_ERR_LAUNCH;
  }
  count_launch();
  return check_launch();
}

int launch_p8_prepare_b(const float* w, int K, int N, int8_t* packed, cudaStream_t stream) {
  if(w == nullptr || packed == nullptr || K <= 0 || N <= 0)
    return MI8_ERR_BAD_ARG;
  if(K % kKcb != 0 || N % kNcb != 0)
    return MI8_ERR_UNSUPPORTED;
  if(reinterpret_cast<uintptr_t>(packed) & 3u)
    return MI8_ERR_MISALIGNED;
  int8_t* tail = packed + static_cast<size_t>(K) * N;
  cudaError_t e = launch_kernel(p8_prepare_b_kernel, dim3(N / kNcb), dim3(kBlock), 0, stream, w, K, N, reinterpret_cast<uint32_t*>(packed),
                                reinterpret_cast<float*>(tail), reinterpret_cast<int32_t*>(tail + static_cast<size_t>(N) * 4),
                                reinterpret_cast<int32_t*>(tail + static_cast<size_t>(N) * 8));
  if(e != cudaSuccess) {
    set_last_cuda_error(e);
    return MI8_ERR_LAUNCH;
  }
  count_launch();
  return check_launch();
}

int launch_p8_quantize_rows(const float* a, int M, int K, uint8_t* aq, float* scale_a, int32_t* zp_a, int32_t* sum_a, cudaStream_t stream) {
  if(M < 0 || K <= 0)
    return MI8_ERR_BAD_ARG;
  if(M == 0)
    return MI8_OK;
  if(a == nullptr || aq == nullptr || scale_a == nullptr || zp_a == nullptr || sum_a == nullptr)
    return MI8_ERR_BAD_ARG;
  if(K % 16 != 0 || (reinterpret_cast<uintptr_t>(a) & 15u) || (reinterpret_cast<uintptr_t>(aq) & 15u))
    return MI8_ERR_MISALIGNED;
  int* status = device_status_ptr();
  if(status == nullptr)
    return MI8_ERR_LAUNCH;
  const int warp_grid = (M + kBlock / 32 - 1) / (kBlock / 32);
  cudaError_t e;
  if(K <= 512)
    e = launch_kernel(p8_quantize_rows_warp_kernel<4>, dim3(warp_grid), dim3(kBlock), 0, stream, a, M, K, aq, scale_a, zp_a, sum_a, status);
  else if(K <= 1024)
    e = launch_kernel(p8_quantize_rows_warp_kernel<8>, dim3(warp_grid), dim3(kBlock), 0, stream, a, M, K, aq, scale_a, zp_a, sum_a, status);
  else if(K <= 2048)
    e = launch_kernel(p8_quantize_rows_warp_kernel<16>, dim3(warp_grid), dim3(kBlock), 0, stream, a, M, K, aq, scale_a, zp_a, sum_a, status);
  else
    e = launch_kernel(p8_quantize_rows_kernel, dim3(M), dim3(kBlock), 0, stream, a, K, aq, scale_a, zp_a, sum_a, status);
  if(e != cudaSuccess) {
    set_last_cuda_error(e);
    return MI8_ERR_LAUNCH;
  }
  count_launch();
  return check_launch();
}

}  // namespace mi8
