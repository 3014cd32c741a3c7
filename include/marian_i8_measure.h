/*
 * marian_i8_measure.h - measurement and test aids of libmarian_i8.so.
 *
 * None of these has a counterpart in the reference and none is part of the drop-in surface
 * (marian_i8.h, marian_i8_decode.h, marian_packed8.h): a benchmark uses them to attribute device time to
 * kernels and to count launches, a test uses the last one to make a bounded device wait run out.
 */
#ifndef MARIAN_I8_MEASURE_H_
#define MARIAN_I8_MEASURE_H_

#include "marian_i8.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Runs, on every SM, a loop of `k_blocks` x 4
 * tcgen05.mma kind::i8 instructions (128 x 256 x 32 each) on one resident shared-memory tile, without loads
 * or write-back, times it with CUDA events (best of three) and returns the rate in TOPS (host float).
 * This is the int8 tensor-pipe figure the roofline fractions of the large-M shapes are quoted against;
 * synchronises the stream. */
int mi8_measure_int8_peak(int k_blocks, float* tops_out, void* stream);

/* Measurement aid: between mi8_profile_begin and mi8_profile_end every GEMM launch made by the calling
 * thread is bracketed by CUDA events on its stream; mi8_profile_end waits for them and returns one record
 * per launch (at most `capacity`).  Off by default; costs two cudaEventRecord calls per launch when on.  While it is on the library holds one
 * device array of max_records ints (the only device allocation the library ever makes; freed by mi8_profile_end). */
typedef struct mi8_gemm_record {
  int M, N, K;        /* problem size of the launch */
  int out_bytes;      /* bytes per output element (4 or 2) */
  float us;           /* device time between the two events, microseconds */
  int rows_computed;  /* activation rows the kernel really computed: M, less the rows of tiles it skipped
                         (mi8_multiply_i8_rows_from and the decoder's stored keys/values); written by the kernel */
} mi8_gemm_record;
int mi8_profile_begin(int max_records);
int mi8_profile_end(mi8_gemm_record* records, int capacity, int* count);

/* Measurement aid: between mi8_kernel_times_begin and mi8_kernel_times_end every kernel the calling thread
 * launches through the library is bracketed by CUDA events on its stream (launch overlap is off meanwhile, so
 * the launches serialise); _end waits for the device and returns, per kernel function, its launches and
 * total device time.  `name` is the function's (mangled) symbol name, truncated. */
typedef struct mi8_kernel_time {
  char name[160];
  long long launches;
  double total_us;
} mi8_kernel_time;
int mi8_kernel_times_begin(void);
int mi8_kernel_times_end(mi8_kernel_time* out, int capacity, int* count);

/* Number of kernels the process (all its threads) has launched through the library since the last reset. */
unsigned long long mi8_launch_count(void);
void mi8_launch_count_reset(void);

/* In-situ timeline of the kernels of this library.  Between mi8_trace_begin and mi8_trace_end one thread of block 0
 * of every kernel writes the GPU's global nanosecond timer into `device_buf` at three points: phase 0 at kernel entry,
 * phase 1 when its wait for the preceding kernel returns, phase 2 at the end of block 0 (phase 3: the end of the last block).  Unlike events placed between
 * launches this leaves programmatic dependent launch as it is, so the stamps show what each kernel costs inside a
 * running decoder step.  device_buf: caller-owned device memory of 2 + 2 * capacity 64-bit words; on return from
 * mi8_trace_end word 0 holds the number of stamps taken (those beyond `capacity` are dropped), followed by pairs
 * (time in ns, extra << 16 | kernel << 8 | phase) in arrival order.  kernel: 1 GEMM, 2 CTA-pair GEMM, 3 quantize_slot,
 * 4 quantize_dual, 5 add_layernorm, 6 attention1, 7 attention_enc, 8 lse_topk, 9 lse_merge, 10 nbest_merge, 11 embed,
 * 12 ancestors_update, 13 history_commit, 14 gather_rows, 15 ssru_cell, 16 absmax, 17 quantize, 18 output-layer GEMM,
 * 19 quantising GEMM; the GEMMs put N | K << 20 into `extra`.  Both calls synchronise the device.
 * The stamps cost about 2 % of a decode even while no buffer is installed, so the product library is built without them
 * (mi8_trace_begin then returns MI8_ERR_UNSUPPORTED); libmarian_i8_trace.so, built from the same sources, carries them. */
int mi8_trace_begin(unsigned long long* device_buf, int capacity);
int mi8_trace_end(void);

/* Test aid: makes a bounded wait inside the GEMM kernels run out on purpose, without faulting anything.
 * While withhold_item >= 0, every CTA's TMA producer leaves out the loads of its pipeline item number
 * `withhold_item` (0 = its first 128-byte K block), so the roles waiting for those bytes give up after
 * `spin_limit` polls (0 = the default of about a million), raise a status word 101..104 (mi8_poll_status),
 * drain what is in flight, release their tensor memory and return; the output of such a launch is undefined.
 * mi8_test_wait_fault(-1, 0) restores normal operation; afterwards mi8_workspace_init + mi8_clear_status make
 * the next call exact again.  Process-wide; not for use beside production calls. */
void mi8_test_wait_fault(int withhold_item, unsigned spin_limit);

/* Host-side timing of mi8d_search (marian_i8_decode.h), accumulated per decoder since the last reset:
 * out[0] = seconds spent issuing the steps' kernels (inside mi8d_step), out[1] = seconds spent waiting for the
 * step's n-best lists (stream synchronisation), out[2] = seconds of host bookkeeping between steps,
 * out[3] = decoder steps taken.  Tells whether a decode is bound by the host's launch rate or by the device. */
struct mi8d_decoder;
int mi8d_search_stats(struct mi8d_decoder* d, double out[4], int reset);

#ifdef __cplusplus
}
#endif
#endif /* MARIAN_I8_MEASURE_H_ */
