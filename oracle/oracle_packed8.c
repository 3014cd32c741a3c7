/*
 * CPU restatement of Marian's packed-int8 affine (type packed8avx512, the mjdgemm route).
 * TEST INFRASTRUCTURE ONLY: the checker for the CUDA path of the same scheme; nothing shipped in the
 * product library links, loads or calls it.
 *
 * PARITY PINNED for the multiply: the reference's own implementation of this route
 * (the files of src/tensors/cpu/mjdgemm) compiles on its own (Makefile target `ref`), and the tests compare every
 * function below that has a counterpart there bit for bit against it, and against fixtures it produced.
 * The restatement follows the AVX-512 route, the one gemmInt8Packed selects on an AVX-512 host
 * (mjdgemm.cpp:50-77), as GCC compiles it with the flags of the reference's src/CMakeLists.txt:
 *
 *   per ROW of A (mjdgemm_avx512.cpp:195-228):
 *       scaleA = (max - min) / 255;  zeroPointA = (int32)(255 - max / scaleA)        (truncation)
 *   quantise (mjdgemm_avx512.cpp:241-276):
 *       q = cvt_nearest_even(min(max(fma(x, 1.0f / scaleA, (float)zeroPointA), 0), 255));  sumA = sum of q
 *   multiply (mjdgemm_avx512.cpp:21-170):   acc[m][n] = sum_k uint8 q[m][k] * int8 B[k][n]   (exact int32)
 *   write-back (mjdgemm_avx512.cpp:290-322):
 *       xv  = acc - zeroPointA * colOffsetsB[n] - zeroPointB[n] * sumA               (int32, wrapping)
 *       out = (scaleA * scaleB[n]) * (float)xv  (+ bias[n])
 *     The add of the bias follows the multiply in the source; GCC contracts the pair into one fused
 *     multiply-add under its default -ffp-contract=fast, and that is what the compiled reference computes.
 *   packed layout of B (mjdgemm_utils.h:136-165): [K/256][N/32][64][32 columns][4 rows], then N floats
 *       scaleB, N int32 zeroPointB, N int32 colOffsetsB (mjdgemm_avx512.cpp:222-227).
 *
 * UNPINNED part: the weight statistics.  packed8avx512 items are produced by fbgemmPacked8Pack
 * (src/tensors/cpu/fbgemm/packed_gemm.cpp:372-480), whose per-column range, scale (max-min)/127 and zero
 * point (int32)(63 - max/scale) are Marian's own lines (:391-431), but whose rounding
 * (fbgemm::Quantize with precision 7: zero_point + x/scale, clamp to [-64,63], nearbyint) and column
 * offsets (sum of the column's int8 values - zero_point * K) live in the un-vendored FBGEMM submodule and
 * are restated from its published behaviour.  The multiply does not depend on them: it reads whatever the
 * packed item holds.
 *
 * Rows whose values are all equal make the reference divide by zero (scaleA = 0); here the range is first
 * widened to contain 0, and an all-zero row takes scaleA = 1.
 */
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define P8_KCB 256
#define P8_NCB 32
#define P8_RI 4

static int p8_threads = 1;
void mo_p8_set_threads(int n) { p8_threads = n > 0 ? n : 1; }

size_t mo_p8_packed_bytes(int K, int N) { return (size_t)K * N + (size_t)N * 12; }

/* byte offset of element (k, n) inside the packed block layout */
static inline size_t p8_offset(int k, int n, int N) {
  int kb = k / P8_KCB, kr = k % P8_KCB, nb = n / P8_NCB, nc = n % P8_NCB;
  return ((size_t)kb * (N / P8_NCB) + nb) * (P8_KCB * P8_NCB) + (size_t)(kr / P8_RI) * (P8_NCB * P8_RI) + (size_t)nc * P8_RI
         + (size_t)(kr % P8_RI);
}

/* W fp32 [K,N] row-major -> packed8avx512 item (weights + scaleB + zeroPointB + colOffsetsB). */
int mo_p8_prepare_b(const float* w, int K, int N, int8_t* packed) {
  if(K <= 0 || N <= 0 || K % P8_KCB || N % P8_NCB)
    return 1;
  float* scale = (float*)(packed + (size_t)K * N);
  int32_t* zp = (int32_t*)(packed + (size_t)K * N + (size_t)N * 4);
  int32_t* off = (int32_t*)(packed + (size_t)K * N + (size_t)N * 8);
  for(int n = 0; n < N; ++n) {
    float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
    for(int k = 0; k < K; ++k) {
      float v = w[(size_t)k * N + n];
      if(mn > v) mn = v;
      if(mx < v) mx = v;
    }
    float s = (mx - mn) / 127;
    if(!(s > 0.0f)) { /* constant column: representable exactly with any scale that maps it to an integer */
      s = 1.0f;
    }
    int32_t z = (int32_t)(63 - mx / s);
    int32_t sum = 0;
    for(int k = 0; k < K; ++k) {
      float t = (float)z + w[(size_t)k * N + n] / s;
      t = t < -64.0f ? -64.0f : (t > 63.0f ? 63.0f : t);
      int32_t q = (int32_t)nearbyintf(t);
      packed[p8_offset(k, n, N)] = (int8_t)q;
      sum += q;
    }
    scale[n] = s;
    zp[n] = z;
    off[n] = sum - z * K;
  }
  return 0;
}

/* plain int8 B [K,N] row-major -> the block layout (the reference's packB) */
int mo_p8_pack_b(const int8_t* b, int K, int N, int8_t* packed) {
  if(K <= 0 || N <= 0 || K % P8_KCB || N % P8_NCB)
    return 1;
  for(int k = 0; k < K; ++k)
    for(int n = 0; n < N; ++n)
      packed[p8_offset(k, n, N)] = b[(size_t)k * N + n];
  return 0;
}

/* block layout -> Bt [N,K] row-major (K contiguous), the layout the GPU GEMM reads */
int mo_p8_unpack_bt(const int8_t* packed, int K, int N, int8_t* bt) {
  if(K <= 0 || N <= 0 || K % P8_KCB || N % P8_NCB)
    return 1;
  for(int n = 0; n < N; ++n)
    for(int k = 0; k < K; ++k)
      bt[(size_t)n * K + k] = packed[p8_offset(k, n, N)];
  return 0;
}

/* Per-row statistics and quantisation of A fp32 [M,K]. */
void mo_p8_quantize_rows(const float* a, int M, int K, uint8_t* aq, float* scale_a, int32_t* zp_a, int32_t* sum_a) {
  for(int m = 0; m < M; ++m) {
    const float* row = a + (size_t)m * K;
    float mn = 3.402823466e+38f, mx = -3.402823466e+38f;
    for(int k = 0; k < K; ++k) {
      mn = row[k] < mn ? row[k] : mn;
      mx = row[k] > mx ? row[k] : mx;
    }
    if(mn == mx) { /* the reference divides by zero here */
      mn = mn < 0.0f ? mn : 0.0f;
      mx = mx > 0.0f ? mx : 0.0f;
    }
    float s = (mx - mn) / 255;
    if(mn == mx)
      s = 1.0f;
    int32_t z = (int32_t)(255 - mx / s);
    float inv = 1.0f / s, zf = (float)z;
    int32_t sum = 0;
    for(int k = 0; k < K; ++k) {
      float t = fmaf(row[k], inv, zf);
      t = t > 0.0f ? t : 0.0f;
      t = t < 255.0f ? t : 255.0f;
      int32_t q = (int32_t)nearbyintf(t);
      aq[(size_t)m * K + k] = (uint8_t)q;
      sum += q;
    }
    scale_a[m] = s;
    zp_a[m] = z;
    sum_a[m] = sum;
  }
}

typedef struct {
  const uint8_t* aq; const int8_t* bt; const float* scale_a; const int32_t* zp_a; const int32_t* sum_a;
  const float* scale_b; const int32_t* zp_b; const int32_t* off_b; const float* bias;
  float* c; int32_t* acc; int M, N, K, relu, r0, r1;
} p8_job;

static void* p8_rows(void* arg) {
  p8_job* j = (p8_job*)arg;
  for(int m = j->r0; m < j->r1; ++m) {
    const uint8_t* ar = j->aq + (size_t)m * j->K;
    for(int n = 0; n < j->N; ++n) {
      const int8_t* br = j->bt + (size_t)n * j->K;
      int32_t acc = 0;
      for(int k = 0; k < j->K; ++k)
        acc += (int32_t)ar[k] * (int32_t)br[k];
      if(j->acc)
        j->acc[(size_t)m * j->N + n] = acc;
      uint32_t xv = (uint32_t)acc;
      xv -= (uint32_t)j->zp_a[m] * (uint32_t)j->off_b[n];
      xv -= (uint32_t)j->zp_b[n] * (uint32_t)j->sum_a[m];
      float scale = j->scale_a[m] * j->scale_b[n];
      float xf = (float)(int32_t)xv;
      float r = j->bias ? fmaf(scale, xf, j->bias[n]) : scale * xf;
      if(j->relu)
        r = r > 0.0f ? r : 0.0f;
      j->c[(size_t)m * j->N + n] = r;
    }
  }
  return NULL;
}

/* The whole affine on an already-unpacked Bt [N,K] plus the three per-column arrays. */
int mo_p8_affine_bt(const float* a, const int8_t* bt, const float* scale_b, const int32_t* zp_b, const int32_t* off_b, const float* bias,
                    int relu, float* c, int32_t* acc_out, int M, int N, int K) {
  if(M < 0 || N <= 0 || K <= 0)
    return 1;
  if(M == 0)
    return 0;
  uint8_t* aq = (uint8_t*)malloc((size_t)M * K);
  float* sa = (float*)malloc(sizeof(float) * M);
  int32_t* za = (int32_t*)malloc(sizeof(int32_t) * M);
  int32_t* su = (int32_t*)malloc(sizeof(int32_t) * M);
  if(!aq || !sa || !za || !su) {
    free(aq); free(sa); free(za); free(su);
    return 1;
  }
  mo_p8_quantize_rows(a, M, K, aq, sa, za, su);
  int T = p8_threads < M ? p8_threads : M;
  if(T > 64) T = 64;
  p8_job jobs[64];
  pthread_t th[64];
  for(int t = 0; t < T; ++t) {
    p8_job j = {aq, bt, sa, za, su, scale_b, zp_b, off_b, bias, c, acc_out, M, N, K, relu, (int)((long long)M * t / T),
                (int)((long long)M * (t + 1) / T)};
    jobs[t] = j;
    if(t + 1 < T)
      pthread_create(&th[t], NULL, p8_rows, &jobs[t]);
  }
  p8_rows(&jobs[T - 1]);
  for(int t = 0; t + 1 < T; ++t)
    pthread_join(th[t], NULL);
  free(aq); free(sa); free(za); free(su);
  return 0;
}

/* Same call shape as the reference's gemmInt8Packed(A, B, bias, C, M, N, K) on a packed item. */
int mo_p8_gemm_packed(const float* a, const int8_t* packed, const float* bias, float* c, int M, int N, int K) {
  if(K <= 0 || N <= 0 || K % P8_KCB || N % P8_NCB)
    return 1;
  int8_t* bt = (int8_t*)malloc((size_t)K * N);
  if(!bt)
    return 1;
  mo_p8_unpack_bt(packed, K, N, bt);
  const float* scale_b = (const float*)(packed + (size_t)K * N);
  const int32_t* zp_b = (const int32_t*)(packed + (size_t)K * N + (size_t)N * 4);
  const int32_t* off_b = (const int32_t*)(packed + (size_t)K * N + (size_t)N * 8);
  int rc = mo_p8_affine_bt(a, bt, scale_b, zp_b, off_b, bias, 0, c, NULL, M, N, K);
  free(bt);
  return rc;
}
