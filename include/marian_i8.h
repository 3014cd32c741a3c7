/*
 * marian_i8.h - C ABI of the B200 (sm_100a) int8 affine engine for Marian.
 *
 * Every entry point replaces one piece of Marian's CPU intgemm8 path (paths below are inside the
 * Marian source tree).  Conventions shared by all calls:
 *   - all pointers are DEVICE pointers unless a parameter is named host_*;
 *   - the library never allocates or frees device memory: outputs, the int8 copy of A and the
 *     workspace are supplied by the caller (Marian's graph allocator hands out 256-byte aligned
 *     pieces, src/tensors/tensor_allocator.h:17);
 *   - quantisation multipliers stay on the device (Marian keeps them in the 4 bytes behind the last
 *     int8 element, src/tensors/cpu/integer_common.h:101-111), so no call synchronises with the host;
 *   - `stream` is a cudaStream_t passed as void*; NULL selects the per-thread default stream, the
 *     stream Marian's kernels run on (CMakeLists.txt:548-550, --default-stream per-thread);
 *   - the return value is an mi8_status; nothing aborts or throws across this boundary.  A host
 *     wrapper turns non-zero into Marian's ABORT (src/common/logging.h:100-140).
 *
 * Workspace contract: the caller passes a workspace of at least mi8_workspace_bytes() bytes that was
 * zero-filled once (mi8_workspace_init).  Kernels use it for arrival counters, abs-max partials and
 * split-K accumulation buffers and put every word they need zeroed back to zero before they finish,
 * so one workspace serves every later call on the same stream.  Calls that share a workspace must
 * not overlap on the device.
 *
 * Measurement and test aids (launch counters, per-kernel timers, the MMA-rate probe, the wait-fault hook)
 * are declared separately in marian_i8_measure.h; nothing of this header needs them.
 */
#ifndef MARIAN_I8_H_
#define MARIAN_I8_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum mi8_status {
  MI8_OK = 0,
  MI8_ERR_BAD_ARG = 1,        /* null pointer, negative size, unknown enum value */
  MI8_ERR_MISALIGNED = 2,     /* a pointer or K breaks the 16-byte rule of the TMA loads */
  MI8_ERR_UNSUPPORTED = 3,    /* shape outside what the kernels cover */
  MI8_ERR_WORKSPACE = 4,      /* workspace missing or too small */
  MI8_ERR_LAUNCH = 5,         /* CUDA reported an error at launch; see mi8_last_cuda_error() */
  MI8_ERR_DEVICE = 6,         /* a kernel raised a status word (bounded wait ran out, non-finite input) */
  MI8_ERR_DRIVER = 7          /* the driver entry point for tensor-map encoding is unavailable */
} mi8_status;

/* Output element type of the fused epilogue. */
typedef enum mi8_dtype { MI8_F32 = 0, MI8_F16 = 1 } mi8_dtype;

/* Library version (major*10000 + minor*100 + patch). */
int mi8_version(void);
/* Text for an mi8_status. */
const char* mi8_strerror(int status);
/* Last cudaError_t seen by this thread inside the library, as an int, and its text. */
int mi8_last_cuda_error(void);
const char* mi8_last_cuda_error_string(void);

/* Bytes of workspace a call with exactly these dimensions needs; mi8_workspace_bytes(0,0,0) is the
 * upper bound that covers every shape (about 21 MB). */
size_t mi8_workspace_bytes(int M, int N, int K);
/* Zero-fills the whole workspace (stream-ordered).  Needed once after allocation, and again after a
 * call that ended with MI8_ERR_DEVICE. */
int mi8_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/* Reads the device status word of the current device (synchronises the device).  0 = healthy;
 * 1xx values say which bounded wait ran out or that an input held Inf/NaN.  *status may be NULL. */
int mi8_poll_status(int* status);
/* Resets the device status word of the current device to 0 (stream-ordered on `stream`). */
int mi8_clear_status(void* stream);

/*
 * max|x| over n floats -> *d_absmax, and 127/max|x| -> *d_quant_mult (either may be NULL).
 * Replaces intgemm::MaxAbsolute + computeQuantMult<intgemm8> (src/tensors/cpu/integer_common.h:169-173).
 * An all-zero input gives quant_mult = 1 (the reference divides by zero there).
 */
int mi8_max_absolute_f32(const float* x, size_t n, float* d_absmax, float* d_quant_mult,
                         void* workspace, size_t workspace_bytes, void* stream);

/*
 * q[i] = saturate_[-127,127](round_half_even(x[i] * *d_quant_mult)).
 * Replaces intgemm::Int8::PrepareA as called at src/tensors/cpu/intgemm_interface.h:23-27.
 */
int mi8_quantize_f32_i8(const float* x, size_t n, const float* d_quant_mult, int8_t* q, void* stream);

/*
 * The whole prepareA node (src/tensors/cpu/intgemm_interface.h:17-32): multiplier from max|A| over
 * the whole [rows, cols] tensor, quantise, store the multiplier in *d_quant_mult (Marian's
 * getQuantMult(out) slot: pass (float*)(q + rows*cols) to keep the reference layout).
 */
int mi8_prepare_a_f32(const float* a, int rows, int cols, int8_t* q, float* d_quant_mult,
                      void* workspace, size_t workspace_bytes, void* stream);

/*
 * Weight conversion of marian-conv --gemm-type intgemm8
 * (src/tensors/cpu/expression_graph_packable.h:160-201): W fp32 [K,N] row-major ->
 * Bt int8 [N,K] row-major (K contiguous), multiplier 127/max|W| -> *d_quant_mult.
 * w_is_nk != 0: W already is [N,K] (a tied embedding used with transB) and is only quantised.
 */
int mi8_prepare_b_f32(const float* w, int K, int N, int w_is_nk, int8_t* bt, float* d_quant_mult,
                      void* workspace, size_t workspace_bytes, void* stream);

/*
 * out[b][c][r] = in[b][r][c] for `batch` matrices [rows, cols] of fp32: the transpose the reference puts in front of
 * prepareA when affine / dot are called with transA (src/tensors/cpu/intgemm_interface.h:52,
 * `transpose(a)` of src/graph/expression_operators.cpp).
 */
int mi8_transpose_f32(const float* in, int batch, int rows, int cols, float* out, void* stream);

/*
 * C[M,N] = relu?( float(Aq . Bt^T) * (1/(qa*qb) * scale) + bias ), the forward step of the
 * multiply node of affineOrDotTyped (src/tensors/cpu/intgemm_interface.h:60-88: Multiply with
 * callbacks::UnquantizeAndAddBiasAndWrite / UnquantizeAndWrite) with the ReLU of
 * affineWithReluDropout (src/graph/expression_operators.cpp:721-731) fused in.
 *   aq [M,K] int8 row-major, bt [N,K] int8 row-major, d_qa / d_qb device floats,
 *   bias fp32 [N] or NULL (dot), c [M,N] row-major of out_dtype,
 *   acc_out int32 [M,N] or NULL: raw accumulators for bit-exact checks.
 * Requirements: K % 16 == 0; aq, bt 16-byte aligned.
 */
int mi8_multiply_i8(const int8_t* aq, const int8_t* bt, int M, int N, int K,
                    const float* d_qa, const float* d_qb, float scale,
                    const float* bias, int relu, void* c, int out_dtype, int32_t* acc_out,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Same, with the tile width along M (16/32/64/128/256, 0 = automatic; 512 = the two-CTA kernel: one
 * tcgen05.mma.cta_group::2 tile of 256 weight rows x 256 activation rows per cluster of two CTAs, no
 * split-K) and the split-K factor (0 = automatic) forced.  Any choice gives bit-identical results. */
int mi8_multiply_i8_ex(const int8_t* aq, const int8_t* bt, int M, int N, int K,
                       const float* d_qa, const float* d_qb, float scale,
                       const float* bias, int relu, void* c, int out_dtype, int32_t* acc_out,
                       void* workspace, size_t workspace_bytes, void* stream,
                       int force_tile_m, int force_splits);

/* One quantised activation against `count` (1..3) converted weights of the same shape in ONE launch: what
 * MultiHead builds as separate affines over the same input - kh = affine(keys, Wk, bk) and vh = affine(values, Wv, bv)
 * with keys == values (src/models/transformer.h:305-327), or q / k / v of encoder self-attention (:290-327) - and the
 * SSRU's dot(input, W) and affine(input, Wf, bf) (src/rnn/cells.h:1029-1050).  bt_all holds the `count` matrices
 * Bt[n_each, K] one behind the other; matrix i has its own multiplier *d_qb[i], bias bias[i] (bias or bias[i] NULL =
 * dot) and output c[i] [M, n_each] row-major.  d_qb / bias / c are HOST arrays of device pointers.  n_each must be a
 * multiple of 128 for count > 1 (MI8_ERR_UNSUPPORTED otherwise: the caller then multiplies one by one).  Each
 * output is bit-identical to the mi8_multiply_i8 call it replaces. */
int mi8_multiply_i8_multi(const int8_t* aq, const int8_t* bt_all, int M, int n_each, int K, int count, const float* d_qa,
                          const float* const* d_qb, float scale, const float* const* bias, int relu, void* const* c, int out_dtype,
                          void* workspace, size_t workspace_bytes, void* stream);

/* The multiply that performs Int8::PrepareA itself (src/tensors/cpu/intgemm_interface.h:17-32 followed by
 * :97-147 in one launch): `a` is the fp32 activation [M,K], `absmax_slot` a device word holding the bit
 * pattern of max|a| that the activation's producer (or mi8_max_absolute_f32) left there.  The kernel
 * derives quantMult = 127 / max|a|, quantises the rows it needs on the fly into shared memory and runs the
 * same tcgen05 GEMM and write-back; no int8 copy of the activation is written.  qa_out (optional) receives
 * the multiplier.  Results are bit-identical to mi8_quantize_f32_i8 + mi8_multiply_i8.  Only shapes that
 * give every CTA one tile qualify (M * N small enough: the decode shapes); others return
 * MI8_ERR_UNSUPPORTED and the caller takes the two-call route.  Every CTA reads its rows of the fp32
 * activation (four times the int8 bytes), so with back-to-back launches overlapped by programmatic
 * dependent launch the two-call route measured slightly faster (8.3 vs 8.9 us for 512 x 1024 x 1024);
 * this entry saves a launch and the int8 buffer where that matters more. */
int mi8_multiply_f32_slot(const float* a, const unsigned* absmax_slot, float* qa_out, const int8_t* bt,
                          int M, int N, int K, const float* d_qb, float scale,
                          const float* bias, int relu, void* c, int out_dtype, int32_t* acc_out, void* stream);

/* The multiply for an activation whose leading rows did not change since the previous call (no
 * counterpart in the reference, which recomputes; used for the decoder's stored keys/values).  When the
 * two device words *same_a and *same_b are equal at the time the kernel runs, tiles of activation rows
 * that lie entirely below row `rows_unchanged_below` are left as they are in c (the caller guarantees
 * they hold the result of the same operands); everything else is computed.  When the words differ
 * the whole product is computed.  The decision is taken on the device, so no host synchronisation. */
int mi8_multiply_i8_rows_from(const int8_t* aq, const int8_t* bt, int M, int N, int K,
                              const float* d_qa, const float* d_qb, float scale,
                              const float* bias, int relu, void* c, int out_dtype,
                              void* workspace, size_t workspace_bytes, void* stream,
                              const unsigned* same_a, const unsigned* same_b, int rows_unchanged_below,
                              int force_tile_m);

/*
 * affine / dot / affineWithReluDropout on a float A and a converted weight in one call
 * (src/graph/expression_operators.cpp:554-731 dispatching to
 * src/tensors/cpu/intgemm_interface.h:46-99): prepareA into aq_scratch (M*K + 4 bytes, multiplier
 * in the last 4), then the multiply with the fused epilogue.  bias NULL = dot.
 */
int mi8_affine_f32(const float* a, int M, int K, const int8_t* bt, const float* d_qb, int N,
                   const float* bias, float scale, int relu, void* c, int out_dtype,
                   int8_t* aq_scratch, void* workspace, size_t workspace_bytes, void* stream);

/*
 * mi8_multiply_i8 for callers that cannot allocate device memory and so have no workspace to pass:
 * code running inside Marian's forward pass after the graph arena has taken the device memory
 * (a cudaMalloc there can fail), or a serving thread that cannot tolerate cudaMalloc's device-wide
 * synchronisation.  This entry point has no counterpart in the reference.
 * The split-K scratch lives in a fixed array inside the library (about 2 MiB per GPU that loads the
 * library, held until the process exits).  Shapes whose split-K plan needs more than 2 MiB of
 * accumulation buffers are refused with MI8_ERR_WORKSPACE (use mi8_multiply_i8 for them).
 * The first call made on a device resolves the array's device address; make that first call outside
 * of any stream capture.  Every call shares the array and clears the part it uses first; calls that
 * overlap on the device race on it, so keep them ordered on one stream.  Inputs, outputs and the
 * meaning of the arguments are those of mi8_multiply_i8; nothing is allocated or freed.
 */
int mi8_multiply_i8_static(const int8_t* aq, const int8_t* bt, int M, int N, int K,
                           const float* d_qa, const float* d_qb, float scale,
                           const float* bias, int relu, void* c, int out_dtype, void* stream);

/* How mi8_multiply_i8 would tile a problem on the current device:
 * out[0]=tile_m, out[1]=pipeline stages, out[2]=splits, out[3]=tiles along N, out[4]=tiles along M,
 * out[5]=CTAs launched, out[6]=dynamic shared memory bytes, out[7]=SM count. */
int mi8_multiply_plan(int M, int N, int K, int force_tile_m, int force_splits, int out[8]);

/* Programmatic dependent launch: when enabled (the default) every kernel of the library is launched so
 * that its set-up (and, in the GEMM, the first weight tiles) overlaps the tail of the previous kernel on
 * the stream; each kernel waits for its predecessor before touching dependent data.  Process-wide switch. */
void mi8_set_pdl(int enabled);


#ifdef __cplusplus
}
#endif
#endif /* MARIAN_I8_H_ */
