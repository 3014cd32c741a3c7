// Measurement aid: the rate at which this GPU's tensor cores retire tcgen05.mma kind::i8 (128 x 256 x 32)
// when nothing else happens - no loads, no write-back.  Every CTA allocates one accumulator and issues the
// same MMA on one shared-memory tile over and over; the host times the launch with CUDA events.  The figure
// is the denominator for "fraction of the int8 tensor pipe" (no vendor-measured int8 peak exists for the
// power-capped clocks these GPUs run at).
#include "mi8_internal.h"
#include "mi8_ptx.cuh"

namespace mi8 {
namespace {

constexpr int kPeakThreads = 64;
constexpr int kPeakN = 256;
constexpr int kPeakTileBytes = (128 + kPeakN) * 128;   // one 128-byte K block of both operands

struct PeakControl {
  uint64_t done;
  uint32_t tmem_base;
  int abort;
};

__global__ void __launch_bounds__(kPeakThreads, 1) mi8_mma_peak_kernel(int k_blocks, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  uint8_t* tile = smem_raw + pad;
  PeakControl* ctl = reinterpret_cast<PeakControl*>(tile + kPeakTileBytes);
  const int warp = threadIdx.x >> 5;
  for(int i = threadIdx.x; i < kPeakTileBytes / 4; i += kPeakThreads)   // pseudo-random operand bytes (data toggling costs power)
    reinterpret_cast<uint32_t*>(tile)[i] = (static_cast<uint32_t>(i) * 2654435761u) ^ (static_cast<uint32_t>(blockIdx.x) * 40503u);
  if(threadIdx.x == 0) {
    mbar_init(&ctl->done, 1);
    ctl->abort = 0;
    fence_mbar_init();
  }
  fence_proxy_async_smem();
  if(warp == 1) {
    tmem_alloc(&ctl->tmem_base, kPeakN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
  if(warp == 1) {
    constexpr uint32_t idesc = make_idesc_i8(kPeakN);
    const uint32_t w_addr = smem_u32(tile);
    const uint32_t a_addr = w_addr + 128 * 128;
    if(elect_one()) {
      for(int kb = 0; kb < k_blocks; ++kb) {
#pragma unroll
        for(int k = 0; k < 4; ++k)
          tc_mma_i8(tmem_base, make_kmajor_sw128_desc(w_addr + k * 32), make_kmajor_sw128_desc(a_addr + k * 32), idesc,
                    (kb > 0 || k > 0) ? 1u : 0u);
      }
      tc_commit(&ctl->done);
    }
    __syncwarp();
    // one wait for everything issued; bounded like every wait of this library (the limit scales with the work)
    bool ok = false;
    for(int round = 0; round < 64 && !ok; ++round)
      ok = mbar_wait_bounded(&ctl->done, 0u, &ctl->abort);
    ok = __all_sync(0xffffffffu, ok);
    if(!ok && (threadIdx.x & 31) == 0)
      atomicMax(status, static_cast<int>(kDevTimeoutMma));
    tc_fence_after_sync();
  }
  tc_fence_before_sync();
  __syncthreads();
  if(warp == 1)
    tmem_dealloc(tmem_base, kPeakN);
}

}  // namespace

int measure_int8_mma_peak(int k_blocks, float* tops_out, cudaStream_t stream) {
  if(k_blocks <= 0 || k_blocks > (1 << 16) || tops_out == nullptr)
    return MI8_ERR_BAD_ARG;
  int* status = device_status_ptr();
  if(status == nullptr)
    return MI8_ERR_LAUNCH;
  const int smem = kPeakTileBytes + static_cast<int>(sizeof(PeakControl)) + 1024;
  cudaError_t e = cudaFuncSetAttribute(mi8_mma_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if(e == cudaSuccess)
    e = cudaEventCreate(&e0);
  if(e == cudaSuccess)
    e = cudaEventCreate(&e1);
  const int grid = sm_count();
  float best_ms = 0.f;
  for(int rep = 0; rep < 4 && e == cudaSuccess; ++rep) {   // first repetition warms up; best of the rest
    cudaEventRecord(e0, stream);
    mi8_mma_peak_kernel<<<grid, kPeakThreads, smem, stream>>>(k_blocks, status);
    cudaEventRecord(e1, stream);
    e = cudaEventSynchronize(e1);
    float ms = 0.f;
    if(e == cudaSuccess)
      e = cudaEventElapsedTime(&ms, e0, e1);
    if(rep > 0 && (best_ms == 0.f || ms < best_ms))
      best_ms = ms;
    count_launch();
  }
  if(e0)
    cudaEventDestroy(e0);
  if(e1)
    cudaEventDestroy(e1);
  if(e != cudaSuccess || best_ms <= 0.f) {
    set_last_cuda_error(e);
    cudaGetLastError();
    return MI8_ERR_LAUNCH;
  }
  const double ops = 2.0 * 128.0 * kPeakN * 128.0 * static_cast<double>(k_blocks) * grid;
  *tops_out = static_cast<float>(ops / (best_ms * 1e-3) / 1e12);
  return MI8_OK;
}

}  // namespace mi8
