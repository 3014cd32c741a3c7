/*
 * C ABI for Marian's packed-int8 affine (weight type packed8avx512) on a B200.
 *
 * The reference runs this scheme on the CPU only: fbgemmPacked8Gemm
 * (src/tensors/cpu/fbgemm/packed_gemm.cpp:566-671) and, without FBGEMM or when forced, its own
 * marian::cpu::mjdgemm::gemmInt8Packed(A, B, bias, C, M, N, K) (src/tensors/cpu/mjdgemm/mjdgemm.h:38,
 * called from packed_gemm.cpp:18-31).  The entry points below are the device-side counterpart of the
 * mjdgemm route and reproduce its AVX-512 path bit for bit:
 *   per activation ROW   scaleA = (max - min) / 255, zeroPointA = (int32)(255 - max / scaleA),
 *                        q = nearest_even(clamp(fma(x, 1/scaleA, zeroPointA), 0, 255)), sumA = sum of q
 *                        (src/tensors/cpu/mjdgemm/mjdgemm_avx512.cpp:195-276)
 *   multiply             acc = sum_k uint8 q[m][k] * int8 B[k][n]           (mjdgemm_avx512.cpp:21-170)
 *   write-back           xv = acc - zeroPointA * colOffsetsB[n] - zeroPointB[n] * sumA
 *                        C = (scaleA * scaleB[n]) * float(xv) (+ bias[n], fused)   (mjdgemm_avx512.cpp:290-322)
 * A packed8avx512 item is K*N block-ordered int8 weights followed by N floats scaleB, N int32 zeroPointB and
 * N int32 colOffsetsB (mjdgemm_avx512.cpp:222-227; written by fbgemmPacked8Pack, packed_gemm.cpp:372-480).
 *
 * Conventions are those of marian_i8.h: device pointers, caller-owned memory, stream-ordered, status codes,
 * no allocation inside the library.  All-equal rows, where the reference divides by zero, are defined here:
 * the row's range is widened to contain 0, an all-zero row takes scaleA = 1.
 */
#ifndef MARIAN_PACKED8_H_
#define MARIAN_PACKED8_H_

#include "marian_i8.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Bytes of a packed8avx512 item for a [K,N] weight: K*N + 12*N. */
size_t mi8p_packed_bytes(int K, int N);

/* Offline conversion, the packed8avx512 branch of marian-conv (ExpressionGraphPackable::pack,
 * src/tensors/cpu/expression_graph_packable.h:49-95 -> fbgemmPacked8Pack, src/tensors/cpu/fbgemm/packed_gemm.cpp:372-480,
 * min/max ranges): w fp32 [K,N] row-major -> item of mi8p_packed_bytes(K, N) bytes.  Per column
 * scaleB = (max - min) / 127, zeroPointB = (int32)(63 - max / scaleB), q = nearest_even(clamp(zeroPointB + x / scaleB, -64, 63)),
 * colOffsetsB = sum(q) - zeroPointB * K.  K % 256 == 0 and N % 32 == 0, else MI8_ERR_UNSUPPORTED. */
int mi8p_prepare_b_f32(const float* w, int K, int N, int8_t* packed, void* stream);

/* Load-time step: the block order of packB (src/tensors/cpu/mjdgemm/mjdgemm_utils.h:136-165:
 * [K/256][N/32][64][32 columns][4 rows]) back to bt[N,K] row-major, the K-major layout the GEMM reads.
 * Requires K % 256 == 0 and N % 32 == 0 (the reference pads neither); MI8_ERR_UNSUPPORTED otherwise.
 * The per-column arrays need no conversion: they are packed + K*N, + K*N + 4*N and + K*N + 8*N. */
int mi8p_unpack_b(const int8_t* packed, int K, int N, int8_t* bt, void* stream);

/* computeQuantizationParams + quantize of every row of a [M,K] (mjdgemm_avx512.cpp:195-276):
 * aq uint8 [M,K], scale_a float [M], zp_a int32 [M], sum_a int32 [M].  K % 16 == 0, a and aq 16-byte aligned. */
int mi8p_quantize_rows(const float* a, int M, int K, uint8_t* aq, float* scale_a, int32_t* zp_a, int32_t* sum_a,
                       void* stream);

/* computeBlock + dequantizeAndAdd (mjdgemm_avx512.cpp:21-170, 290-322) on the tcgen05 GEMM: c fp32 [M,N];
 * bias fp32 [N] or NULL; relu != 0 applies max(0, .) (affineWithReluDropout, src/graph/expression_operators.cpp:721-731);
 * acc_out int32 [M,N] or NULL receives the raw uint8 x int8 sums.  workspace as for mi8_multiply_i8.
 * aq, bt and the three per-row arrays must be 16-byte aligned, K % 16 == 0.
 * force_tile_m / force_splits: 0 = automatic (test hooks, as in mi8_multiply_i8_ex). */
int mi8p_multiply(const uint8_t* aq, const float* scale_a, const int32_t* zp_a, const int32_t* sum_a,
                  const int8_t* bt, const float* scale_b, const int32_t* zp_b, const int32_t* off_b,
                  int M, int N, int K, const float* bias, int relu, float* c, int32_t* acc_out,
                  void* workspace, size_t workspace_bytes, void* stream, int force_tile_m, int force_splits);

/* Scratch for mi8p_gemm_int8_packed: the uint8 activation (rounded up to 256 bytes) and the three per-row arrays. */
size_t mi8p_scratch_bytes(int M, int K);

/* gemmInt8Packed(A, B, bias, C, M, N, K) (src/tensors/cpu/mjdgemm/mjdgemm.h:38) in one call: quantise the rows
 * of `a` into `scratch`, then multiply against the unpacked weight `bt` and the item's per-column arrays. */
int mi8p_gemm_int8_packed(const float* a, const int8_t* bt, const float* scale_b, const int32_t* zp_b,
                          const int32_t* off_b, const float* bias, float* c, int M, int N, int K,
                          void* scratch, size_t scratch_bytes, void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MARIAN_PACKED8_H_ */
