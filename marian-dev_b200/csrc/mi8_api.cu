// The extern "C" surface of libmarian_i8.so: argument checks, bookkeeping and the sequencing of
// the kernels.  No call here allocates device memory or synchronises with the host, except
// mi8_poll_status which exists to do exactly that.
#include <atomic>
#include <cstring>
#include <vector>

#include "../../include/marian_packed8.h"
#include "mi8_internal.h"
#include "mi8_ptx.cuh"

namespace mi8 {

// One status word per device (each device that loads the module gets its own instance).
__device__ int g_status_word = 0;

namespace {
thread_local cudaError_t t_last_error = cudaSuccess;
std::atomic<unsigned long long> g_launches{0};   // all threads of the process: searches may run on several threads at once
int* g_status_ptr[64] = {};
int g_sm_count[64] = {};
}  // namespace

namespace {
bool g_pdl = true;
}
bool pdl_enabled() { return g_pdl; }
void set_pdl(bool on) { g_pdl = on; }

// ---- per-kernel device times -------------------------------------------------------------------------
struct KernelTimeState {
  bool on = false;
  std::vector<const void*> funcs;
  std::vector<cudaEvent_t> pool;     // two events per launch, created once and reused
  size_t used = 0;
  cudaEvent_t take() {
    if(used == pool.size()) {
      cudaEvent_t e = nullptr;
      if(cudaEventCreate(&e) != cudaSuccess)
        return nullptr;
      pool.push_back(e);
    }
    return pool[used++];
  }
};
thread_local KernelTimeState t_ktimes;

bool kernel_times_on() { return t_ktimes.on; }
void kernel_times_before(const void* func, cudaStream_t stream) {
  cudaEvent_t e = t_ktimes.take();
  t_ktimes.funcs.push_back(func);
  if(e != nullptr)
    cudaEventRecord(e, stream);
}
void kernel_times_after(cudaStream_t stream) {
  cudaEvent_t e = t_ktimes.take();
  if(e != nullptr)
    cudaEventRecord(e, stream);
}

void set_last_cuda_error(cudaError_t e) { t_last_error = e; }
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int check_launch() {
  cudaError_t e = cudaGetLastError();
  if(e != cudaSuccess) {
    t_last_error = e;
    return MI8_ERR_LAUNCH;
  }
  return MI8_OK;
}

int* device_status_ptr() {
  int dev = 0;
  if(cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return nullptr;
  if(g_status_ptr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_status_word);
    if(e != cudaSuccess) {
      t_last_error = e;
      return nullptr;
    }
    g_status_ptr[dev] = static_cast<int*>(p);
  }
  return g_status_ptr[dev];
}

int sm_count() {
  int dev = 0;
  if(cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return 148;  // B200; also what plan queries answer on a host without a GPU
  if(g_sm_count[dev] == 0) {
    int n = 0;
    if(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 148;
    }
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

}  // namespace mi8

using namespace mi8;

extern "C" {

int mi8_version(void) { return 10200; }

const char* mi8_strerror(int status) {
  switch(status) {
    case MI8_OK: return "ok";
    case MI8_ERR_BAD_ARG: return "bad argument (null pointer, negative size or unknown enum value)";
    case MI8_ERR_MISALIGNED: return "pointer not 16-byte aligned or K not a multiple of 16";
    case MI8_ERR_UNSUPPORTED: return "shape not supported";
    case MI8_ERR_WORKSPACE: return "workspace missing or too small";
    case MI8_ERR_LAUNCH: return "CUDA error at kernel launch";
    case MI8_ERR_DEVICE: return "a kernel raised the device status word";
    case MI8_ERR_DRIVER: return "tensor-map encoding unavailable (driver entry point)";
    default: return "unknown status";
  }
}

int mi8_last_cuda_error(void) { return static_cast<int>(t_last_error); }
const char* mi8_last_cuda_error_string(void) { return cudaGetErrorString(t_last_error); }

unsigned long long mi8_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
void mi8_launch_count_reset(void) { g_launches.store(0, std::memory_order_relaxed); }

size_t mi8_workspace_bytes(int M, int N, int K) {
  // Upper bound over every plan: only problems with fewer tiles than SMs are split, and each tile
  // accumulates into 128 x 256 int32 at most.
  const size_t upper = kWsHeaderBytes + static_cast<size_t>(160) * 128 * 256 * sizeof(int32_t);
  if(M <= 0 || N <= 0 || K <= 0)
    return upper;
  GemmPlan plan;
  if(make_gemm_plan(M, N, K, 0, 0, &plan) != MI8_OK)
    return upper;
  return kWsHeaderBytes + plan.partial_bytes;
}

int mi8_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  if(workspace == nullptr || workspace_bytes < kWsHeaderBytes)
    return MI8_ERR_WORKSPACE;
  cudaError_t e = cudaMemsetAsync(workspace, 0, workspace_bytes, as_stream(stream));
  if(e != cudaSuccess) {
    set_last_cuda_error(e);
    return MI8_ERR_LAUNCH;
  }
  return MI8_OK;
}

int mi8_poll_status(int* status) {
  int* p = device_status_ptr();
  if(p == nullptr)
    return MI8_ERR_LAUNCH;
  int v = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if(e == cudaSuccess)
    e = cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
  if(e != cudaSuccess) {
    set_last_cuda_error(e);
    return MI8_ERR_LAUNCH;
  }
  if(status != nullptr)
    *status = v;
  return v == 0 ? MI8_OK : MI8_ERR_DEVICE;
}

int mi8_clear_status(void* stream) {
  int* p = device_status_ptr();
  if(p == nullptr)
    return MI8_ERR_LAUNCH;
  cudaError_t e = cudaMemsetAsync(p, 0, sizeof(int), as_stream(stream));
  if(e != cudaSuccess) {
    set_last_cuda_error(e);
    return MI8_ERR_LAUNCH;
  }
  return MI8_OK;
}

int mi8_max_absolute_f32(const float* x, size_t n, float* d_absmax, float* d_quant_mult, void* workspace,
                         size_t workspace_bytes, void* stream) {
  return launch_max_absolute(x, n, d_absmax, d_quant_mult, workspace, workspace_bytes, as_stream(stream));
}

int mi8_quantize_f32_i8(const float* x, size_t n, const float* d_quant_mult, int8_t* q, void* stream) {
  return launch_quantize(x, n, d_quant_mult, q, as_stream(stream));
}

int mi8_prepare_a_f32(const float* a, int rows, int cols, int8_t* q, float* d_quant_mult, void* workspace,
                      size_t workspace_bytes, void* stream) {
  if(rows < 0 || cols <= 0 || d_quant_mult == nullptr)
    return MI8_ERR_BAD_ARG;
  if(rows == 0)
    return MI8_OK;
  const size_t n = static_cast<size_t>(rows) * static_cast<size_t>(cols);
  int rc = launch_max_absolute(a, n, nullptr, d_quant_mult, workspace, workspace_bytes, as_stream(stream));
  if(rc != MI8_OK)
    return rc;
  return launch_quantize(a, n, d_quant_mult, q, as_stream(stream));
}

int mi8_prepare_b_f32(const float* w, int K, int N, int w_is_nk, int8_t* bt, float* d_quant_mult, void* workspace,
                      size_t workspace_bytes, void* stream) {
  if(K <= 0 || N <= 0 || d_quant_mult == nullptr)
    return MI8_ERR_BAD_ARG;
  const size_t n = static_cast<size_t>(K) * static_cast<size_t>(N);
  int rc = launch_max_absolute(w, n, nullptr, d_quant_mult, workspace, workspace_bytes, as_stream(stream));
  if(rc != MI8_OK)
    return rc;
  if(w_is_nk)
    return launch_quantize(w, n, d_quant_mult, bt, as_stream(stream));
  return launch_transpose_quantize(w, K, N, d_quant_mult, bt, as_stream(stream));
}

int mi8_transpose_f32(const float* in, int batch, int rows, int cols, float* out, void* stream) {
  return launch_transpose_f32(in, batch, rows, cols, out, as_stream(stream));
}

int mi8_multiply_i8(const int8_t* aq, const int8_t* bt, int M, int N, int K, const float* d_qa, const float* d_qb,
                    float scale, const float* bias, int relu, void* c, int out_dtype, int32_t* acc_out, void* workspace,
                    size_t workspace_bytes, void* stream) {
  return launch_gemm(aq, bt, M, N, K, d_qa, d_qb, scale, bias, relu, c, out_dtype, acc_out, workspace, workspace_bytes,
                     as_stream(stream), 0, 0);
}

int mi8_multiply_i8_ex(const int8_t* aq, const int8_t* bt, int M, int N, int K, const float* d_qa, const float* d_qb,
                       float scale, const float* bias, int relu, void* c, int out_dtype, int32_t* acc_out, void* workspace,
                       size_t workspace_bytes, void* stream, int force_tile_m, int force_splits) {
  if(force_tile_m < 0 || force_splits < 0)
    return MI8_ERR_BAD_ARG;
  return launch_gemm(aq, bt, M, N, K, d_qa, d_qb, scale, bias, relu, c, out_dtype, acc_out, workspace, workspace_bytes,
                     as_stream(stream), force_tile_m, force_splits);
}

int mi8_multiply_i8_multi(const int8_t* aq, const int8_t* bt_all, int M, int n_each, int K, int count, const float* d_qa,
                          const float* const* d_qb, float scale, const float* const* bias, int relu, void* const* c, int out_dtype,
                          void* workspace, size_t workspace_bytes, void* stream) {
  if(count < 1 || count > 3 || n_each <= 0 || d_qb == nullptr || c == nullptr)
    return MI8_ERR_BAD_ARG;
  GemmCall g;
  g.aq = aq;
  g.bt = bt_all;
  g.M = M;
  g.N = n_each * count;
  g.K = K;
  g.d_qa = d_qa;
  g.scale = scale;
  g.relu = relu;
  g.out_dtype = out_dtype;
  g.nseg = count;
  for(int i = 0; i < count; ++i) {
    g.seg_qb[i] = d_qb[i];
    g.seg_bias[i] = bias != nullptr ? bias[i] : nullptr;
    g.seg_c[i] = c[i];
  }
  g.ws = workspace;
  g.ws_bytes = workspace_bytes;
  g.stream = as_stream(stream);
  return launch_gemm_call(g);
}

int mi8_multiply_f32_slot(const float* a, const unsigned* absmax_slot, float* qa_out, const int8_t* bt, int M, int N, int K,
                          const float* d_qb, float scale, const float* bias, int relu, void* c, int out_dtype, int32_t* acc_out,
                          void* stream) {
  return launch_gemm_quant_a(a, absmax_slot, qa_out, bt, M, N, K, d_qb, scale, bias, relu, c, out_dtype, acc_out, as_stream(stream));
}

int mi8_multiply_i8_rows_from(const int8_t* aq, const int8_t* bt, int M, int N, int K, const float* d_qa, const float* d_qb,
                              float scale, const float* bias, int relu, void* c, int out_dtype, void* workspace,
                              size_t workspace_bytes, void* stream, const unsigned* same_a, const unsigned* same_b,
                              int rows_unchanged_below, int force_tile_m) {
  if(force_tile_m < 0 || same_a == nullptr || same_b == nullptr || rows_unchanged_below < 0)
    return MI8_ERR_BAD_ARG;
  return launch_gemm(aq, bt, M, N, K, d_qa, d_qb, scale, bias, relu, c, out_dtype, nullptr, workspace, workspace_bytes,
                     as_stream(stream), force_tile_m, 0, nullptr, same_a, same_b, rows_unchanged_below);
}

int mi8_affine_f32(const float* a, int M, int K, const int8_t* bt, const float* d_qb, int N, const float* bias, float scale,
                   int relu, void* c, int out_dtype, int8_t* aq_scratch, void* workspace, size_t workspace_bytes,
                   void* stream) {
  if(M < 0 || K <= 0 || N <= 0 || aq_scratch == nullptr)
    return MI8_ERR_BAD_ARG;
  if(M == 0)
    return MI8_OK;
  if(K % 16 != 0)
    return MI8_ERR_MISALIGNED;
  float* d_qa = reinterpret_cast<float*>(aq_scratch + static_cast<size_t>(M) * K);
  int rc = mi8_prepare_a_f32(a, M, K, aq_scratch, d_qa, workspace, workspace_bytes, stream);
  if(rc != MI8_OK)
    return rc;
  return launch_gemm(aq_scratch, bt, M, N, K, d_qa, d_qb, scale, bias, relu, c, out_dtype, nullptr, workspace,
                     workspace_bytes, as_stream(stream), 0, 0);
}

void mi8_set_pdl(int enabled) { set_pdl(enabled != 0); }

void mi8_test_wait_fault(int withhold_item, unsigned spin_limit) { test_wait_fault(withhold_item, spin_limit); }

int mi8_trace_begin(unsigned long long* device_buf, int capacity) {
  if(device_buf == nullptr || capacity <= 0)
    return MI8_ERR_BAD_ARG;
#ifdef MI8_NO_TRACE
  return MI8_ERR_UNSUPPORTED;   // this build carries no timeline code (libmarian_i8_trace.so does)
#endif
  const unsigned long long head[2] = {0ull, static_cast<unsigned long long>(capacity)};
  cudaError_t e = cudaDeviceSynchronize();
  if(e == cudaSuccess)
    e = cudaMemcpy(device_buf, head, sizeof(head), cudaMemcpyHostToDevice);
  if(e != cudaSuccess) {
    set_last_cuda_error(e);
    return MI8_ERR_LAUNCH;
  }
  if(trace_set_glue(device_buf) != 0 || trace_set_gemm(device_buf) != 0 || trace_set_quant(device_buf) != 0) {
    set_last_cuda_error(cudaGetLastError());
    return MI8_ERR_LAUNCH;
  }
  return MI8_OK;
}

int mi8_trace_end(void) {
  cudaError_t e = cudaDeviceSynchronize();
  const int rc = trace_set_glue(nullptr) | trace_set_gemm(nullptr) | trace_set_quant(nullptr);
  if(e != cudaSuccess || rc != 0) {
    set_last_cuda_error(e != cudaSuccess ? e : cudaGetLastError());
    return MI8_ERR_LAUNCH;
  }
  return MI8_OK;
}

int mi8_kernel_times_begin(void) {
  t_ktimes.on = true;
  t_ktimes.funcs.clear();
  t_ktimes.used = 0;
  return MI8_OK;
}

int mi8_kernel_times_end(mi8_kernel_time* out, int capacity, int* count) {
  t_ktimes.on = false;
  int n = 0;
  cudaError_t e = cudaDeviceSynchronize();
  std::vector<const void*> slot_func;   // launches are merged per kernel FUNCTION (names are only labels and may be truncated)
  for(size_t i = 0; e == cudaSuccess && i < t_ktimes.funcs.size() && 2 * i + 1 < t_ktimes.used; ++i) {
    float ms = 0.f;
    if(cudaEventElapsedTime(&ms, t_ktimes.pool[2 * i], t_ktimes.pool[2 * i + 1]) != cudaSuccess) {
      cudaGetLastError();
      continue;
    }
    int slot = -1;
    for(int j = 0; j < n; ++j)
      if(slot_func[j] == t_ktimes.funcs[i]) {
        slot = j;
        break;
      }
    if(slot < 0) {
      if(out == nullptr || n >= capacity)
        continue;
      const char* name = nullptr;
      if(cudaFuncGetName(&name, t_ktimes.funcs[i]) != cudaSuccess || name == nullptr) {
        cudaGetLastError();
        name = "?";
      }
      slot = n++;
      slot_func.push_back(t_ktimes.funcs[i]);
      memset(&out[slot], 0, sizeof(out[slot]));
      strncpy(out[slot].name, name, sizeof(out[slot].name) - 1);
    }
    out[slot].launches += 1;
    out[slot].total_us += ms * 1000.0;
  }
  t_ktimes.funcs.clear();
  t_ktimes.used = 0;
  if(count != nullptr)
    *count = n;
  if(e != cudaSuccess) {
    set_last_cuda_error(e);
    return MI8_ERR_LAUNCH;
  }
  return MI8_OK;
}

int mi8_measure_int8_peak(int k_blocks, float* tops_out, void* stream) { return measure_int8_mma_peak(k_blocks, tops_out, as_stream(stream)); }

int mi8_profile_begin(int max_records) { return profile_begin(max_records); }
int mi8_profile_end(mi8_gemm_record* records, int capacity, int* count) { return profile_end(records, capacity, count); }

int mi8_multiply_plan(int M, int N, int K, int force_tile_m, int force_splits, int out[8]) {
  if(out == nullptr)
    return MI8_ERR_BAD_ARG;
  GemmPlan plan;
  int rc = make_gemm_plan(M, N, K, force_tile_m, force_splits, &plan);
  if(rc != MI8_OK)
    return rc;
  out[0] = plan.pair ? 512 : plan.tile_m;
  out[1] = plan.stages;
  out[2] = plan.splits;
  out[3] = plan.n_tiles;
  out[4] = plan.m_tiles;
  out[5] = plan.grid;
  out[6] = plan.smem_bytes;
  out[7] = sm_count();
  return MI8_OK;
}

// ------------------------------------------------------------------ packed8avx512 scheme (marian_packed8.h)
size_t mi8p_packed_bytes(int K, int N) {
  return K > 0 && N > 0 ? static_cast<size_t>(K) * N + static_cast<size_t>(N) * 12 : 0;
}

int mi8p_prepare_b_f32(const float* w, int K, int N, int8_t* packed, void* stream) {
  return launch_p8_prepare_b(w, K, N, packed, as_stream(stream));
}

int mi8p_unpack_b(const int8_t* packed, int K, int N, int8_t* bt, void* stream) {
  return launch_p8_unpack_bt(packed, K, N, bt, as_stream(stream));
}

int mi8p_quantize_rows(const float* a, int M, int K, uint8_t* aq, float* scale_a, int32_t* zp_a, int32_t* sum_a, void* stream) {
  return launch_p8_quantize_rows(a, M, K, aq, scale_a, zp_a, sum_a, as_stream(stream));
}

int mi8p_multiply(const uint8_t* aq, const float* scale_a, const int32_t* zp_a, const int32_t* sum_a, const int8_t* bt,
                  const float* scale_b, const int32_t* zp_b, const int32_t* off_b, int M, int N, int K, const float* bias, int relu,
                  float* c, int32_t* acc_out, void* workspace, size_t workspace_bytes, void* stream, int force_tile_m,
                  int force_splits) {
  return launch_gemm_p8(aq, scale_a, zp_a, sum_a, bt, scale_b, zp_b, off_b, M, N, K, bias, relu, c, acc_out, workspace, workspace_bytes,
                        as_stream(stream), force_tile_m, force_splits);
}

size_t mi8p_scratch_bytes(int M, int K) {
  if(M <= 0 || K <= 0)
    return 0;
  const size_t aq = (static_cast<size_t>(M) * K + 255) / 256 * 256;
  const size_t per_row = (static_cast<size_t>(M) * 4 + 255) / 256 * 256;
  return aq + 3 * per_row;
}

int mi8p_gemm_int8_packed(const float* a, const int8_t* bt, const float* scale_b, const int32_t* zp_b, const int32_t* off_b,
                          const float* bias, float* c, int M, int N, int K, void* scratch, size_t scratch_bytes, void* workspace,
                          size_t workspace_bytes, void* stream) {
  if(M < 0 || N <= 0 || K <= 0)
    return MI8_ERR_BAD_ARG;
  if(M == 0)
    return MI8_OK;
  if(scratch == nullptr || scratch_bytes < mi8p_scratch_bytes(M, K))
    return MI8_ERR_WORKSPACE;
  if(reinterpret_cast<uintptr_t>(scratch) & 255u)
    return MI8_ERR_MISALIGNED;
  uint8_t* base = static_cast<uint8_t*>(scratch);
  const size_t aq_bytes = (static_cast<size_t>(M) * K + 255) / 256 * 256;
  const size_t per_row = (static_cast<size_t>(M) * 4 + 255) / 256 * 256;
  uint8_t* aq = base;
  float* scale_a = reinterpret_cast<float*>(base + aq_bytes);
  int32_t* zp_a = reinterpret_cast<int32_t*>(base + aq_bytes + per_row);
  int32_t* sum_a = reinterpret_cast<int32_t*>(base + aq_bytes + 2 * per_row);
  int rc = launch_p8_quantize_rows(a, M, K, aq, scale_a, zp_a, sum_a, as_stream(stream));
  if(rc != MI8_OK)
    return rc;
  return launch_gemm_p8(aq, scale_a, zp_a, sum_a, bt, scale_b, zp_b, off_b, M, N, K, bias, 0, c, nullptr, workspace, workspace_bytes,
                        as_stream(stream), 0, 0);
}

}  // extern "C"
