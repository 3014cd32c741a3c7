// mi8_multiply_i8_static: the int8 multiply for callers that cannot hand the library a workspace.
//
// Who that is.  Marian reserves almost all device memory for its own arena at start-up
// (--workspace), so once a graph is running a cudaMalloc from inside an operator can fail outright;
// and a serving thread that must never stall cannot afford cudaMalloc either, because it
// synchronises the whole device.  Such callers own their inputs and outputs but have nowhere to
// put the split-K scratch (arrival counters + int32 accumulation buffers) that mi8_multiply_i8
// takes as `workspace`.  For them the scratch lives in a fixed array inside this library.
//
// Cost and limits.  Every GPU that loads the library carries the array (kStaticScratchBytes, a
// little over 2 MiB) until the process exits.  A problem whose split-K plan needs more than the
// array holds is refused with MI8_ERR_WORKSPACE; use mi8_multiply_i8 with a caller-owned workspace
// for those.  All calls share the one array and it keeps whatever the last call left, so each call
// first clears the part it is about to use (stream-ordered), and two calls that overlap on the
// device (different streams, no dependency) race on it.
//
// First call on a device.  Host code cannot use the array's name as a pointer: on the host it is
// only a handle for the device symbol.  The first call made while a device is current asks the
// runtime for that device's address of the array (cudaGetSymbolAddress) and remembers it; make that
// first call outside of any stream capture.  Two host threads that make the first call on the same device
// at the same time both store the same address, which is harmless.  Nothing here calls cudaMalloc,
// cudaFree or any allocating library routine.
#include "mi8_internal.h"

namespace mi8 {
namespace {

constexpr size_t kStaticAccumBytes = size_t(2) << 20;                       // split-K accumulation buffers
constexpr size_t kStaticScratchBytes = kWsHeaderBytes + kStaticAccumBytes;  // same layout as a caller workspace

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

unsigned char* g_scratch_ptr[64] = {};

// Device address of the array for the current device; resolved once per device.
int static_scratch(unsigned char** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if(e != cudaSuccess || dev < 0 || dev >= 64) {
    set_last_cuda_error(e);
    return MI8_ERR_LAUNCH;
  }
  if(g_scratch_ptr[dev] == nullptr) {
    unsigned char* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if(e != cudaSuccess || p == nullptr) {
      set_last_cuda_error(e);
      return MI8_ERR_LAUNCH;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return MI8_OK;
}

}  // namespace
}  // namespace mi8

using namespace mi8;

extern "C" int mi8_multiply_i8_static(const int8_t* aq, const int8_t* bt, int M, int N, int K, const float* d_qa,
                                      const float* d_qb, float scale, const float* bias, int relu, void* c, int out_dtype,
                                      void* stream) {
  if(M < 0 || N <= 0 || K <= 0)
    return MI8_ERR_BAD_ARG;
  if(M == 0)
    return MI8_OK;
  // every argument is checked before anything is queued on the stream, so a refused call leaves the array untouched
  if(aq == nullptr || bt == nullptr || d_qa == nullptr || d_qb == nullptr || c == nullptr || (out_dtype != MI8_F32 && out_dtype != MI8_F16))
    return MI8_ERR_BAD_ARG;
  if(K % 16 != 0 || (reinterpret_cast<uintptr_t>(aq) & 15u) || (reinterpret_cast<uintptr_t>(bt) & 15u))
    return MI8_ERR_MISALIGNED;
  GemmPlan plan;
  int rc = make_gemm_plan(M, N, K, 0, 0, &plan);
  if(rc != MI8_OK)
    return rc;
  if(plan.partial_bytes > kStaticAccumBytes)
    return MI8_ERR_WORKSPACE;  // beyond the built-in scratch: this shape needs a caller-owned workspace
  unsigned char* scratch = nullptr;
  rc = static_scratch(&scratch);
  if(rc != MI8_OK)
    return rc;
  cudaStream_t s = as_stream(stream);
  if(plan.splits > 1) {
    // The array still holds what the previous call left: zero this call's arrival counters and
    // accumulation buffers before the kernel adds into them.
    const size_t tiles = static_cast<size_t>(plan.n_tiles) * plan.m_tiles;
    cudaError_t e = cudaMemsetAsync(scratch + kWsOffTileCounters, 0, tiles * sizeof(uint32_t), s);
    if(e == cudaSuccess)
      e = cudaMemsetAsync(scratch + kWsOffPartials, 0, plan.partial_bytes, s);
    if(e != cudaSuccess) {
      set_last_cuda_error(e);
      return MI8_ERR_LAUNCH;
    }
  }
  return launch_gemm(aq, bt, M, N, K, d_qa, d_qb, scale, bias, relu, c, out_dtype, nullptr, scratch, kStaticScratchBytes, s,
                     0, 0);
}
