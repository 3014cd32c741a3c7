// Inline-PTX building blocks for the sm_100a int8 affine engine: mbarrier, TMA loads into this CTA only,
// tcgen05 (TMEM allocation, kind::i8 MMA, commit, TMEM loads).  Every wait is bounded.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace mi8 {

// Status words the kernels can raise in the device status slot (see mi8_poll_status()).
enum DeviceStatus : int {
  kDevOk = 0,
  kDevTimeoutProducer = 101,  // TMA producer gave up waiting for a free smem slot
  kDevTimeoutMma = 102,       // MMA issuer gave up waiting for operands or a free accumulator
  kDevTimeoutEpilogue = 103,  // epilogue gave up waiting for a finished accumulator
  kDevTimeoutDrain = 104,     // teardown gave up waiting for copies / MMAs still in flight
  kDevNonFinite = 110,        // abs-max saw Inf or NaN
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-stream-serialization attribute may start while its
// predecessor on the stream is still running.  pdl_launch_dependents() lets the successor start
// launching; pdl_wait() blocks until the predecessor has completed and its writes are visible.
// Everything a kernel does before pdl_wait() must not depend on (or disturb) the predecessor:
// barrier/TMEM set-up and loads of constant weights qualify.  Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- in-situ timeline (measurement aid)
// While a trace buffer is installed (mi8_trace_begin), one thread of block 0 of every kernel stamps the
// global nanosecond timer at kernel entry (phase 0), after pdl_wait() (1) and at its exit (2; 3 = the last block's exit) into the buffer
// ([0] = entries used, [1] = capacity, then pairs (time, extra << 16 | kernel << 8 | phase); the GEMMs put
// N | K << 20 | M << 40 into `extra`).  Unlike events between
// launches this leaves programmatic dependent launch undisturbed, so it shows what a kernel costs inside the
// running decoder step.  Every translation unit holds its own copy of the pointer (set by its
// MI8_DEFINE_TRACE_SETTER function); it is null outside a trace, which costs one load per kernel.
static __device__ unsigned long long* s_trace_buf = nullptr;
enum TraceKernel : int {
  kTrGemm = 1, kTrGemmPair, kTrQuantSlot, kTrQuantDual, kTrAddLn, kTrAttention1, kTrAttentionEnc, kTrLseTopk, kTrLseMerge,
  kTrNbest, kTrEmbed, kTrAncestors, kTrCommit, kTrGather, kTrSsru, kTrAbsmax, kTrQuantize, kTrGemmLogits, kTrGemmQuantA, kTrGemmCq
};
// Every kernel reads the pointer ONCE, at its entry (before its wait for the preceding kernel, so the load overlaps that
// kernel's tail), in the two threads that stamp: the last thread of block 0 and the last thread of the last block.  All other
// threads get null.  The stamps sit outside every hot loop (a store the compiler cannot see through would hold it back there).  Nothing else of the timeline runs when it is off.
struct TraceHandles {
  unsigned long long* first;     // block 0: phases 0, 1, 2
  unsigned long long* last;      // last block of the grid: phase 3
  unsigned long long t_entry;    // the timer at kernel entry (phase 0 is written together with phase 1, see trace_stamp_start)
};
__device__ __forceinline__ TraceHandles trace_open_all() {
  TraceHandles h;
  h.first = nullptr;
  h.last = nullptr;
  h.t_entry = 0ull;
#ifdef MI8_NO_TRACE
  return h;
#endif
  if(threadIdx.x == blockDim.x - 1) {
    const bool b0 = blockIdx.x == 0 && blockIdx.y == 0;
    const bool bl = blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1 && (gridDim.x > 1 || gridDim.y > 1);
    if(b0 || bl) {
      // The load is only ISSUED here; nothing may depend on it before the kernel's wait for its predecessor, or the
      // thread (and, through the next block-wide barrier, its whole block) would sit out an L2 round trip at start-up.
      unsigned long long* t = s_trace_buf;
      h.first = b0 ? t : nullptr;
      h.last = bl ? t : nullptr;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(h.t_entry));
    }
  }
  return h;
}
__device__ __forceinline__ void trace_stamp(unsigned long long* tb, int kernel, int phase, unsigned long long extra = 0ull) {
  if(tb != nullptr) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    const unsigned long long idx = atomicAdd(tb, 1ull);
    if(idx < tb[1]) {
      tb[2 + 2 * idx] = t;
      tb[3 + 2 * idx] = (extra << 16) | (static_cast<unsigned long long>(kernel) << 8) | static_cast<unsigned long long>(phase);
    }
  }
}
// Phases 0 (entry, with the time taken then) and 1 (now: the wait for the preceding kernel has returned), written together.
__device__ __forceinline__ void trace_stamp_start(const TraceHandles& h, int kernel, unsigned long long extra = 0ull) {
  unsigned long long* tb = h.first;
  if(tb != nullptr) {
    const unsigned long long idx = atomicAdd(tb, 1ull);
    if(idx < tb[1]) {
      tb[2 + 2 * idx] = h.t_entry;
      tb[3 + 2 * idx] = (extra << 16) | (static_cast<unsigned long long>(kernel) << 8);
    }
    trace_stamp(tb, kernel, 1, extra);
  }
}
#define MI8_DEFINE_TRACE_SETTER(name)                                                         \
  int name(unsigned long long* buf) {                                                         \
    return cudaMemcpyToSymbol(s_trace_buf, &buf, sizeof(buf)) == cudaSuccess ? 0 : 5;         \
  }

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Default spin limit of a barrier wait.  A healthy pipeline completes a wait in well under a
// microsecond (every role first waits for the preceding kernel with pdl_wait(), so the limit only
// measures this kernel's own pipeline); it exists so that a broken one returns an error instead of hanging.
constexpr uint32_t kSpinLimit = 1u << 20;

// Bounded wait.  `abort_flag` (shared memory) lets the other roles leave early once one gave up.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint32_t limit = kSpinLimit) {
  for(uint32_t i = 0; i < limit; ++i) {
    if(mbar_try_wait(bar, parity))
      return true;
    if((i & 0xff) == 0xff && *abort_flag)
      return false;
  }
  return false;
}

// ---------------------------------------------------------------- one elected lane
// True in exactly one lane of a fully active warp.  Unlike a test of the lane index, the compiler
// knows the guarded code runs in one lane with warp-uniform operands, so descriptors and coordinates
// of the TMA / tcgen05 instructions inside stay in uniform registers instead of being moved there one
// by one (measured: ~100 cycles per tcgen05.mma issued under `lane == 0`, far less under elect.sync).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- TMA (tiled 2-D load, this CTA only)
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// x = innermost coordinate in elements (bytes here; callers keep it a multiple of 16), y = row.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// ---------------------------------------------------------------- tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive once on `bar` when every tcgen05 operation this thread issued so far has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], int8 x int8 -> int32, shape 128 x N x 32 per instruction.
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---------------------------------------------------------------- CTA pairs (cluster of two, tcgen05 cta_group::2)
// The two CTAs of a cluster of size two run on one TPC and can issue one MMA of 256 rows together:
// each holds its 128 rows of the M-side operand and half of the N-side operand in its own shared
// memory, the accumulators land in both CTAs' TMEM (128 lanes each).  One thread of the CTA with
// cluster rank 0 issues the MMAs and the commits for both.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in the CTA with rank `rank`.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t cta_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
  return r;
}
// Hardware barrier over all threads of the cluster (cannot time out; every path of a kernel reaches it).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// TMA load into this CTA's shared memory whose byte count is credited to an mbarrier that may live in
// the peer CTA (`bar_cluster_addr` is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar_cluster_addr)
      : "memory");
}
// TMEM management for a CTA pair: the same warp index of both CTAs executes these.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrive once on the barrier at this shared-memory offset in every CTA of `cta_mask` when all
// tcgen05 operations issued so far by this thread (for both CTAs) have completed.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(cta_mask)
               : "memory");
}
// D[tmem of both CTAs] (+)= A * B, 256 x N x 32 per instruction (128 rows of A and N/2 rows of B per CTA).
__device__ __forceinline__ void tc_mma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Each thread of the warp reads its own TMEM lane (lane = 32*(warp%4) + threadIdx%32), N consecutive
// 32-bit columns starting at the column in `taddr`.
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, int32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, int32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (what a TMA box of 128 bytes x rows with SWIZZLE_128B produces):
//   bits [0,14)  start address >> 4          bits [16,30) leading byte offset >> 4 (unused for swizzled K-major; 1)
//   bits [32,46) stride byte offset >> 4 = 1024 >> 4 (distance between 8-row groups)
//   bits [46,48) descriptor version 1        bits [61,64) layout type 2 = 128-byte swizzle
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fffu);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::i8: signed 8-bit A and B, both K-major, int32 accumulator,
// M rows (128 for one CTA, 256 for a CTA pair), N columns.
//   bits [4,6) accumulator format 2 = S32; bits [7,10) A format 1 = signed; bits [10,13) B format 1 = signed;
//   bit 15 / 16 A / B major 0 = K; bits [17,23) N >> 3; bits [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_i8(int n, int m = 128) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// The same with an UNSIGNED 8-bit B operand (bits [10,13) = 0): uint8 activations against int8 weights.
__host__ __device__ constexpr uint32_t make_idesc_i8_ub(int n, int m = 128) {
  return (2u << 4) | (1u << 7) | (0u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

}  // namespace mi8
