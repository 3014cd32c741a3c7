/*
 * CPU restatement of Marian's intgemm8 affine/dot path.  TEST INFRASTRUCTURE ONLY:
 * this file is the checker for the CUDA engine and the timed CPU baseline; nothing
 * shipped in the product library links, loads or calls it.
 *
 * PARITY UNPINNED.  The arithmetic Marian runs on this path lives in the third-party
 * module marian-nmt/intgemm (git submodule src/3rd_party/intgemm, no recoverable pin),
 * whose sources are not part of the reference tree, and no test of the reference
 * exercises an intgemm-typed operand.  The functions below therefore follow the
 * reference's own call sites and the published behaviour of the intgemm entry points
 * they call:
 *
 *   MaxAbsolute            : max over |x|                              (call site src/tensors/cpu/integer_common.h:173)
 *   computeQuantMult       : 127.0f / MaxAbsolute                      (src/tensors/cpu/integer_common.h:169-182)
 *   Int8::PrepareA         : x*quantMult, round to nearest even, saturate to [-127,127]
 *                                                                      (call site src/tensors/cpu/intgemm_interface.h:23)
 *   getQuantMult           : the multiplier is stored as a float right after the last int8 element
 *                                                                      (src/tensors/cpu/integer_common.h:101-111, src/common/types.cpp:32-37)
 *   Multiply               : acc[i][j] = sum_k A[i][k]*B[k][j] in int32 (the AVX512-VNNI route; an optional
 *                            saturating-int16 emulation documents the pre-VNNI kernels)
 *                                                                      (call site src/tensors/cpu/intgemm_interface.h:74-87)
 *   UnquantizeAndWrite / UnquantizeAndAddBiasAndWrite : out = float(acc)*unquant (+ bias[col])
 *                                                                      (src/tensors/cpu/intgemm_interface.h:66-87)
 *   ReLU afterwards, in place                                          (src/graph/expression_operators.cpp:721-731,
 *                                                                       src/graph/node_operators_unary.h:1053-1068)
 *   weight conversion      : Transpose10, 127/max|W|, plain quantise -> Bt[N,K] row-major + scale tail
 *                                                                      (src/tensors/cpu/expression_graph_packable.h:153-253)
 *
 * Build with -ffp-contract=off so that "multiply then add" stays two rounded operations.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

#define MO_OK 0
#define MO_BAD_ARG 1

int mo_version(void) { return 1; }

/* Row-parallel helper on POSIX threads: the GEMM and the write-back split their M rows over the
 * worker count set with mo_set_threads (default 1, as Marian runs one GEMM per worker thread,
 * src/common/config.cpp:245-248; the timed baseline raises it to the host's core count). */
static int g_threads = 1;

int mo_max_threads(void) {
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n > 0 ? (int)n : 1;
}

void mo_set_threads(int n) { g_threads = n > 0 ? n : 1; }

typedef void (*mo_row_fn)(int row_begin, int row_end, void* ctx);
typedef struct { mo_row_fn fn; int b, e; void* ctx; } mo_job;

static void* mo_job_main(void* p) {
  mo_job* j = (mo_job*)p;
  j->fn(j->b, j->e, j->ctx);
  return NULL;
}

static void mo_parallel_rows(int m, mo_row_fn fn, void* ctx) {
  int t = g_threads;
  if(t > m) t = m;
  if(t <= 1) { fn(0, m, ctx); return; }
  pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)t);
  mo_job* jobs = (mo_job*)malloc(sizeof(mo_job) * (size_t)t);
  int per = (m + t - 1) / t;
  for(int i = 0; i < t; ++i) {
    jobs[i].fn = fn; jobs[i].ctx = ctx;
    jobs[i].b = i * per < m ? i * per : m;
    jobs[i].e = (i + 1) * per < m ? (i + 1) * per : m;
    if(i > 0) pthread_create(&th[i], NULL, mo_job_main, &jobs[i]);
  }
  mo_job_main(&jobs[0]);
  for(int i = 1; i < t; ++i) pthread_join(th[i], NULL);
  free(th); free(jobs);
}

/* intgemm::MaxAbsolute(begin, end) as used by computeQuantMult (integer_common.h:173). */
static float mo_max_absolute_portable(const float* x, size_t n) {
  float m = 0.0f;
  for(size_t i = 0; i < n; ++i) {
    float a = fabsf(x[i]);
    if(a > m) m = a;   /* NaN never wins the comparison */
  }
  return m;
}

#if defined(__x86_64__)
#include <immintrin.h>
__attribute__((target("avx2")))
static float mo_max_absolute_avx2(const float* x, size_t n) {
  const __m256 sign = _mm256_set1_ps(-0.0f);
  __m256 m = _mm256_setzero_ps();
  size_t i = 0;
  for(; i + 8 <= n; i += 8)
    m = _mm256_max_ps(_mm256_andnot_ps(sign, _mm256_loadu_ps(x + i)), m);   /* a NaN operand yields m, as in the scalar loop */
  float t[8];
  _mm256_storeu_ps(t, m);
  float r = 0.0f;
  for(int j = 0; j < 8; ++j) if(t[j] > r) r = t[j];
  for(; i < n; ++i) { float a = fabsf(x[i]); if(a > r) r = a; }
  return r;
}
#endif

static int mo_has_avx2(void) {
#if defined(__x86_64__)
  static int cached = -1;
  if(cached < 0) { __builtin_cpu_init(); cached = __builtin_cpu_supports("avx2") ? 1 : 0; }
  return cached;
#else
  return 0;
#endif
}

typedef struct { const float* x; size_t n; size_t per; float part[64]; } mo_absmax_ctx;
static void mo_absmax_chunk(int b, int e, void* p) {
  mo_absmax_ctx* c = (mo_absmax_ctx*)p;
  for(int u = b; u < e; ++u) {
    const size_t lo = (size_t)u * c->per, hi = lo + c->per < c->n ? lo + c->per : c->n;
#if defined(__x86_64__)
    c->part[u] = mo_has_avx2() ? mo_max_absolute_avx2(c->x + lo, hi - lo) : mo_max_absolute_portable(c->x + lo, hi - lo);
#else
    c->part[u] = mo_max_absolute_portable(c->x + lo, hi - lo);
#endif
  }
}

/* intgemm::MaxAbsolute(begin, end) as used by computeQuantMult (integer_common.h:173).  A maximum does not
 * depend on the order it is taken in, so large inputs are split over the worker threads. */
float mo_max_absolute(const float* x, size_t n) {
  mo_absmax_ctx c;
  c.x = x; c.n = n;
  int units = (g_threads > 1 && n >= ((size_t)1 << 18)) ? (g_threads < 64 ? g_threads : 64) : 1;
  c.per = (n + (size_t)units - 1) / (size_t)units;
  if(units == 1) mo_absmax_chunk(0, 1, &c); else mo_parallel_rows(units, mo_absmax_chunk, &c);
  float m = 0.0f;
  for(int u = 0; u < units; ++u) if(c.part[u] > m) m = c.part[u];
  return m;
}

/* computeQuantMult<intgemm8> (integer_common.h:169-173).  The reference divides by zero for an
 * all-zero tensor; this restatement defines that case as quantMult = 1 (all quantised values 0). */
float mo_compute_quant_mult(const float* x, size_t n) {
  float m = mo_max_absolute(x, n);
  if(m == 0.0f) return 1.0f;
  return 127.0f / m;
}

static inline int8_t mo_quantize_one(float x, float quant_mult) {
  float r = rintf(x * quant_mult); /* default rounding mode: to nearest, ties to even */
  if(r > 127.0f) r = 127.0f;
  if(r < -127.0f) r = -127.0f;   /* -128 is never produced */
  if(r != r) r = 0.0f;
  return (int8_t)r;
}

/* Int8::PrepareA(in, out, quantMult, rows, cols): element-wise quantise, same layout
 * (intgemm_interface.h:23-27).  `tail`, when non-null, receives the multiplier the way
 * getQuantMult(out) = quantMult does (intgemm_interface.h:28). */
#if defined(__x86_64__)
/* Same arithmetic as mo_quantize_one on 32 values at a time: one rounded multiply, round to nearest even,
 * clamp to +-127, NaN -> 0, convert (exact for integral values), pack to bytes in order. */
__attribute__((target("avx2")))
static void mo_quantize_avx2(const float* in, int8_t* out, float qm, size_t n) {
  const __m256 vq = _mm256_set1_ps(qm), hi = _mm256_set1_ps(127.0f), lo = _mm256_set1_ps(-127.0f);
  const __m256i order = _mm256_setr_epi32(0, 4, 1, 5, 2, 6, 3, 7);
  size_t i = 0;
  for(; i + 32 <= n; i += 32) {
    __m256i v[4];
    for(int j = 0; j < 4; ++j) {
      const __m256 prod = _mm256_mul_ps(_mm256_loadu_ps(in + i + 8 * j), vq);
      __m256 r = _mm256_round_ps(prod, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
      r = _mm256_max_ps(_mm256_min_ps(r, hi), lo);
      r = _mm256_and_ps(r, _mm256_cmp_ps(prod, prod, _CMP_ORD_Q));
      v[j] = _mm256_cvtps_epi32(r);
    }
    const __m256i b = _mm256_packs_epi16(_mm256_packs_epi32(v[0], v[1]), _mm256_packs_epi32(v[2], v[3]));
    _mm256_storeu_si256((__m256i*)(out + i), _mm256_permutevar8x32_epi32(b, order));
  }
  for(; i < n; ++i) out[i] = mo_quantize_one(in[i], qm);
}
#endif

typedef struct { const float* in; int8_t* out; float qm; size_t n, per; } mo_quant_ctx;
static void mo_quant_chunk(int b, int e, void* p) {
  mo_quant_ctx* c = (mo_quant_ctx*)p;
  for(int u = b; u < e; ++u) {
    const size_t lo = (size_t)u * c->per, hi = lo + c->per < c->n ? lo + c->per : c->n;
#if defined(__x86_64__)
    if(mo_has_avx2()) { mo_quantize_avx2(c->in + lo, c->out + lo, c->qm, hi - lo); continue; }
#endif
    for(size_t i = lo; i < hi; ++i) c->out[i] = mo_quantize_one(c->in[i], c->qm);
  }
}

void mo_prepare_a(const float* in, int8_t* out, float quant_mult, int rows, int cols, float* tail) {
  mo_quant_ctx c = {in, out, quant_mult, (size_t)rows * (size_t)cols, 0};
  int units = (g_threads > 1 && c.n >= ((size_t)1 << 18)) ? g_threads : 1;
  c.per = ((c.n + (size_t)units - 1) / (size_t)units + 31) & ~(size_t)31;
  if(units == 1) mo_quant_chunk(0, 1, &c); else mo_parallel_rows(units, mo_quant_chunk, &c);
  if(tail) memcpy(tail, &quant_mult, sizeof(float));
}

/* marian-conv's intgemm8 branch (expression_graph_packable.h:160-201): tmp = Transpose10(W),
 * quantMult = 127/max|W|, Int8::PrepareA(tmp) -> Bt[N,K] row-major; returns quantMult.
 * With w_is_nk != 0 the input already is [N,K] (a tied embedding matrix used with transB) and
 * is only quantised. */
float mo_prepare_b(const float* w, int k, int n, int w_is_nk, int8_t* bt) {
  size_t total = (size_t)k * (size_t)n;
  float qm = mo_compute_quant_mult(w, total);
  if(w_is_nk) {
    for(size_t i = 0; i < total; ++i) bt[i] = mo_quantize_one(w[i], qm);
  } else {
    for(int j = 0; j < n; ++j)
      for(int i = 0; i < k; ++i)
        bt[(size_t)j * k + i] = mo_quantize_one(w[(size_t)i * n + j], qm);
  }
  return qm;
}

/* Multiply(A, B, rowsA, colsA, colsB, callback) with exact 32-bit accumulation
 * (intgemm_interface.h:74-87).  A is [M,K] row-major int8, Bt is [N,K] row-major int8, so every output is a
 * dot product of two K-contiguous rows.  Three routes, chosen once at run time; all give the same exact sums:
 *   AVX512-VNNI  vpdpbusd (u8 x s8 -> s32, no saturation) on A + 128, corrected by 128 * sum_k Bt[j][k]
 *                (the unsigned-shift trick intgemm's "Shifted" kernels use); 4 x 4 register blocking
 *   AVX2         sign-extend to 16 bits, vpmaddwd (exact, unlike the saturating vpmaddubsw)
 *   portable C   */
#if defined(__x86_64__)
#include <immintrin.h>

__attribute__((target("avx512f,avx512bw,avx512vnni")))
static void mo_rows_vnni(const int8_t* a, const int8_t* bt, int k, int n, int32_t* acc, int row_b, int row_e, int col_b, int col_e,
                         uint8_t* au /* 4 * kp bytes */) {
  const int kp = (k + 63) & ~63;
  for(int i0 = row_b; i0 < row_e; i0 += 4) {
    const int mi = row_e - i0 < 4 ? row_e - i0 : 4;
    for(int r = 0; r < 4; ++r) {              /* A + 128 as unsigned bytes, zero padded to a multiple of 64 */
      uint8_t* d = au + (size_t)r * kp;
      if(r < mi) {
        const int8_t* sr = a + (size_t)(i0 + r) * k;
        for(int p = 0; p < k; ++p) d[p] = (uint8_t)(sr[p] + 128);
        for(int p = k; p < kp; ++p) d[p] = 0;
      } else {
        memset(d, 0, (size_t)kp);
      }
    }
    for(int j0 = col_b; j0 < col_e; j0 += 4) {
      const int nj = col_e - j0 < 4 ? col_e - j0 : 4;
      __m512i c[4][4];
      for(int r = 0; r < 4; ++r)
        for(int q = 0; q < 4; ++q) c[r][q] = _mm512_setzero_si512();
      for(int p = 0; p < k; p += 64) {
        const __mmask64 mk = (k - p) >= 64 ? ~(__mmask64)0 : (((__mmask64)1 << (k - p)) - 1);
        __m512i vb[4];
        for(int q = 0; q < 4; ++q)
          vb[q] = q < nj ? _mm512_maskz_loadu_epi8(mk, bt + (size_t)(j0 + q) * k + p) : _mm512_setzero_si512();
        for(int r = 0; r < 4; ++r) {
          const __m512i va = _mm512_loadu_si512((const void*)(au + (size_t)r * kp + p));
          for(int q = 0; q < 4; ++q) c[r][q] = _mm512_dpbusd_epi32(c[r][q], va, vb[q]);
        }
      }
      for(int q = 0; q < nj; ++q) {
        /* 128 * sum_k Bt[j][k] undoes the shift of A; vpdpbusd of all-ones bytes against Bt gives that sum */
        __m512i sb = _mm512_setzero_si512();
        const __m512i ones = _mm512_set1_epi8(1);
        for(int p = 0; p < k; p += 64) {
          const __mmask64 mk = (k - p) >= 64 ? ~(__mmask64)0 : (((__mmask64)1 << (k - p)) - 1);
          sb = _mm512_dpbusd_epi32(sb, ones, _mm512_maskz_loadu_epi8(mk, bt + (size_t)(j0 + q) * k + p));
        }
        const int32_t corr = 128 * _mm512_reduce_add_epi32(sb);
        for(int r = 0; r < mi; ++r)
          acc[(size_t)(i0 + r) * n + j0 + q] = _mm512_reduce_add_epi32(c[r][q]) - corr;
      }
    }
  }
}

__attribute__((target("avx2")))
static void mo_rows_avx2(const int8_t* a, const int8_t* bt, int k, int n, int32_t* acc, int row_b, int row_e, int col_b, int col_e) {
  const int k16 = k & ~15;
  for(int i = row_b; i < row_e; ++i) {
    const int8_t* ar = a + (size_t)i * k;
    for(int j = col_b; j < col_e; ++j) {
      const int8_t* br = bt + (size_t)j * k;
      __m256i c = _mm256_setzero_si256();
      for(int p = 0; p < k16; p += 16) {
        const __m256i va = _mm256_cvtepi8_epi16(_mm_loadu_si128((const __m128i*)(ar + p)));
        const __m256i vb = _mm256_cvtepi8_epi16(_mm_loadu_si128((const __m128i*)(br + p)));
        c = _mm256_add_epi32(c, _mm256_madd_epi16(va, vb));
      }
      __m128i h = _mm_add_epi32(_mm256_castsi256_si128(c), _mm256_extracti128_si256(c, 1));
      h = _mm_add_epi32(h, _mm_shuffle_epi32(h, 0x4e));
      h = _mm_add_epi32(h, _mm_shuffle_epi32(h, 0xb1));
      int32_t sum = _mm_cvtsi128_si32(h);
      for(int p = k16; p < k; ++p) sum += (int32_t)ar[p] * (int32_t)br[p];
      acc[(size_t)i * n + j] = sum;
    }
  }
}
#endif

static void mo_rows_portable(const int8_t* a, const int8_t* bt, int k, int n, int32_t* acc, int row_b, int row_e, int col_b, int col_e) {
  for(int i = row_b; i < row_e; ++i)
    for(int j = col_b; j < col_e; ++j) {
      const int8_t* ar = a + (size_t)i * k;
      const int8_t* b = bt + (size_t)j * k;
      int32_t sum = 0;
      for(int p = 0; p < k; ++p) sum += (int32_t)ar[p] * (int32_t)b[p];
      acc[(size_t)i * n + j] = sum;
    }
}

/* 0 portable, 1 AVX2, 2 AVX512-VNNI; mo_set_isa(-1) picks the best the host has (the default). */
static int g_isa = -1;
static int mo_best_isa(void) {
#if defined(__x86_64__)
  __builtin_cpu_init();
  if(__builtin_cpu_supports("avx512vnni") && __builtin_cpu_supports("avx512bw")) return 2;
  if(__builtin_cpu_supports("avx2")) return 1;
#endif
  return 0;
}
int mo_set_isa(int isa) {
  const int best = mo_best_isa();
  g_isa = (isa < 0 || isa > best) ? best : isa;
  return g_isa;
}

/* Work is dealt to the threads in units of 4 rows when there are enough rows, otherwise (the skinny decode
 * shapes) in units of 16 weight rows, every thread then walking all activation rows. */
typedef struct { const int8_t* a; const int8_t* bt; int m, k, n; int32_t* acc; int isa; int by_cols; } mo_mul_ctx;

static void mo_mul_range(const mo_mul_ctx* c, int rb, int re, int cb, int ce) {
#if defined(__x86_64__)
  if(c->isa == 2) {
    const int kp = (c->k + 63) & ~63;
    uint8_t* au = (uint8_t*)aligned_alloc(64, (size_t)4 * kp);
    if(au != NULL) {
      mo_rows_vnni(c->a, c->bt, c->k, c->n, c->acc, rb, re, cb, ce, au);
      free(au);
      return;
    }
  }
  if(c->isa >= 1) {
    mo_rows_avx2(c->a, c->bt, c->k, c->n, c->acc, rb, re, cb, ce);
    return;
  }
#endif
  mo_rows_portable(c->a, c->bt, c->k, c->n, c->acc, rb, re, cb, ce);
}

static void mo_mul_units(int b, int e, void* p) {
  const mo_mul_ctx* c = (const mo_mul_ctx*)p;
  if(c->by_cols) {
    const int cb = b * 16, ce = e * 16 < c->n ? e * 16 : c->n;
    mo_mul_range(c, 0, c->m, cb, ce);
  } else {
    const int rb = b * 4, re = e * 4 < c->m ? e * 4 : c->m;
    mo_mul_range(c, rb, re, 0, c->n);
  }
}

int mo_multiply_i32(const int8_t* a, const int8_t* bt, int m, int k, int n, int32_t* acc) {
  if(m < 0 || k <= 0 || n <= 0) return MO_BAD_ARG;
  if(m == 0) return MO_OK;
  if(g_isa < 0) mo_set_isa(-1);
  mo_mul_ctx c = {a, bt, m, k, n, acc, g_isa, 0};
  const int row_units = (m + 3) / 4, col_units = (n + 15) / 16;
  c.by_cols = row_units < 2 * g_threads && col_units > row_units;
  mo_parallel_rows(c.by_cols ? col_units : row_units, mo_mul_units, &c);
  return MO_OK;
}

static inline int16_t mo_sat16(int32_t v) {
  if(v > 32767) return 32767;
  if(v < -32768) return -32768;
  return (int16_t)v;
}

/* The pre-VNNI intgemm kernels multiply with pmaddubsw: |a| (unsigned) times sign-adjusted b,
 * adjacent pairs summed with signed 16-bit saturation, then pairs of those sums added again with
 * 16-bit saturation before widening to 32 bits.  This emulation keeps that structure so the
 * "reference's saturation behaviour" can be compared against; it is not the primary oracle. */
int mo_multiply_sat16(const int8_t* a, const int8_t* bt, int m, int k, int n, int32_t* acc) {
  if(m < 0 || k <= 0 || n <= 0 || (k % 4) != 0) return MO_BAD_ARG;
  for(int i = 0; i < m; ++i) {
    const int8_t* ar = a + (size_t)i * k;
    for(int j = 0; j < n; ++j) {
      const int8_t* b = bt + (size_t)j * k;
      int32_t s = 0;
      for(int p = 0; p < k; p += 4) {
        int16_t pair[2];
        for(int h = 0; h < 2; ++h) {
          int a0 = ar[p + 2 * h], a1 = ar[p + 2 * h + 1];
          int b0 = b[p + 2 * h], b1 = b[p + 2 * h + 1];
          int ua0 = a0 < 0 ? -a0 : a0, ua1 = a1 < 0 ? -a1 : a1;
          int sb0 = a0 < 0 ? -b0 : (a0 == 0 ? 0 : b0);
          int sb1 = a1 < 0 ? -b1 : (a1 == 0 ? 0 : b1);
          pair[h] = mo_sat16(ua0 * sb0 + ua1 * sb1);
        }
        s += (int32_t)mo_sat16((int32_t)pair[0] + (int32_t)pair[1]);
      }
      acc[(size_t)i * n + j] = s;
    }
  }
  return MO_OK;
}

/* unquant_mult = 1.0f / (aQuantMult * bQuantMult); unquant_mult *= scale (intgemm_interface.h:69-70). */
float mo_unquant_mult(float qa, float qb, float scale) {
  float u = 1.0f / (qa * qb);
  u = u * scale;
  return u;
}

/* callbacks::UnquantizeAndWrite / UnquantizeAndAddBiasAndWrite followed by the separate in-place
 * ReLU of affineWithReluDropout on this path (expression_operators.cpp:721-731). */
typedef struct { const int32_t* acc; int n; float unquant; const float* bias; int relu; float* out; } mo_wr_ctx;

static void mo_wr_rows(int b, int e, void* p) {
  mo_wr_ctx* c = (mo_wr_ctx*)p;
  for(int i = b; i < e; ++i) {
    for(int j = 0; j < c->n; ++j) {
      float v = (float)c->acc[(size_t)i * c->n + j] * c->unquant;
      if(c->bias) v = v + c->bias[j];
      if(c->relu && !(v > 0.0f)) v = 0.0f;
      c->out[(size_t)i * c->n + j] = v;
    }
  }
}

void mo_unquantize_write(const int32_t* acc, int m, int n, float unquant, const float* bias, int relu, float* out) {
  mo_wr_ctx c = {acc, n, unquant, bias, relu, out};
  if((size_t)m * n < ((size_t)1 << 17))
    mo_wr_rows(0, m, &c);            /* too little work to pay for starting threads */
  else
    mo_parallel_rows(m, mo_wr_rows, &c);
}

/* The whole affineOrDotTyped sequence (intgemm_interface.h:46-99) for float A [M,K] and a converted
 * weight Bt [N,K] with multiplier qb.  aq (M*K), acc (M*N) are optional outputs. */
int mo_affine(const float* a, int m, int k, const int8_t* bt, float qb, int n, const float* bias, float scale,
              int relu, float* out, int8_t* aq_out, int32_t* acc_out, float* qa_out) {
  if(m < 0 || k <= 0 || n <= 0) return MO_BAD_ARG;
  if(m == 0) return MO_OK;
  int8_t* aq = aq_out ? aq_out : (int8_t*)malloc((size_t)m * k);
  int32_t* acc = acc_out ? acc_out : (int32_t*)malloc((size_t)m * n * sizeof(int32_t));
  if(!aq || !acc) return MO_BAD_ARG;
  float qa = mo_compute_quant_mult(a, (size_t)m * k);
  mo_prepare_a(a, aq, qa, m, k, NULL);
  mo_multiply_i32(aq, bt, m, k, n, acc);
  mo_unquantize_write(acc, m, n, mo_unquant_mult(qa, qb, scale), bias, relu, out);
  if(qa_out) *qa_out = qa;
  if(!aq_out) free(aq);
  if(!acc_out) free(acc);
  return MO_OK;
}

/* ===================================================================================================
 * Float glue of the decode (LayerNorm, attention, log-softmax/top-k, embedding, SSRU cell).
 *
 * The reference leaves the order of its float reductions to whatever BLAS / SIMD kernels it is built
 * with, so no particular order is "the" reference order.  An int8 pipeline amplifies a one-ulp
 * difference in these ops to a full quantisation step within two affines, therefore the checker and
 * the engine must round identically to be comparable at all.  The functions below fix one order
 * (thread-strided partial sums, a 32-wide butterfly, eight partials added in ascending order; fma
 * chains in ascending index order) and fixed polynomials for exp and log, built from correctly
 * rounded IEEE operations only.
 *   LayerNorm: gamma * (x - mean) / sqrt(var + eps) + beta, biased variance
 *              (src/tensors/cpu/tensor_operators.cpp:1087-1124, eps 1e-6 src/layers/generic.h:248-253)
 *   attention: softmax(q.k / sqrt(dh) + mask) . v   (src/models/transformer.h:240-277)
 *   SSRU:      c' = c*sigmoid(f) + x*(1 - sigmoid(f)), h = relu(c')   (src/rnn/cells.h:1052-1066)
 *   n-best:    log-softmax + top-N over beam x vocabulary (src/translator/beam_search.cpp:469-496)
 * =================================================================================================== */
#include <float.h>

#define MO_FMA_CLONES __attribute__((target_clones("arch=haswell", "default")))

static inline float mo_det_expf_i(float x) {
  if(x < -87.0f) return 0.0f;
  if(x > 88.0f) x = 88.0f;
  const float n = rintf(x * 1.44269504f);
  float r = fmaf(n, -0.693145752f, x);
  r = fmaf(n, -1.42860677e-06f, r);
  float p = 1.3888889e-3f;
  p = fmaf(p, r, 8.3333338e-3f);
  p = fmaf(p, r, 4.1666668e-2f);
  p = fmaf(p, r, 1.6666667e-1f);
  p = fmaf(p, r, 0.5f);
  p = fmaf(p, r, 1.0f);
  p = fmaf(p, r, 1.0f);
  const int e = (int)n;
  union { int32_t i; float f; } s;
  s.i = (e + 127) << 23;
  return p * s.f;
}

static inline float mo_det_logf_i(float x) {
  union { int32_t i; float f; } u;
  u.f = x;
  int e = ((u.i >> 23) & 0xff) - 127;
  u.i = (u.i & 0x007fffff) | 0x3f800000;
  float m = u.f;
  if(m > 1.41421354f) { m = m * 0.5f; e += 1; }
  const float s = (m + -1.0f) / (m + 1.0f);
  const float s2 = s * s;
  float t = 0.181818187f;
  t = fmaf(t, s2, 0.222222224f);
  t = fmaf(t, s2, 0.285714298f);
  t = fmaf(t, s2, 0.400000006f);
  t = fmaf(t, s2, 0.666666687f);
  t = t * s2;
  const float lm = fmaf(s, t, 2.0f * s);
  return fmaf((float)e, 0.693147182f, lm);
}

MO_FMA_CLONES float mo_det_expf(float x) { return mo_det_expf_i(x); }
MO_FMA_CLONES float mo_det_logf(float x) { return mo_det_logf_i(x); }

/* v[i] <- v[i] + v[i ^ o] for o = 16, 8, 4, 2, 1; every entry ends with the same bits */
static inline float mo_warp_sum(const float* v32) {
  float a[32], b[32];
  memcpy(a, v32, sizeof(a));
  for(int o = 16; o > 0; o >>= 1) {
    for(int i = 0; i < 32; ++i) b[i] = a[i] + a[i ^ o];
    memcpy(a, b, sizeof(a));
  }
  return a[0];
}

static inline float mo_block256_sum(const float* v256) {
  float t = 0.0f;
  for(int w = 0; w < 8; ++w) t = t + mo_warp_sum(v256 + 32 * w);
  return t;
}

/* out = LayerNorm(a + resid) * gamma + beta per row (resid may be NULL) */
MO_FMA_CLONES void mo_add_layernorm(const float* a, const float* resid, const float* gamma, const float* beta, float eps, int rows,
                                    int dim, float* out) {
  const int chunks = dim / 4;
  float* y = (float*)malloc(sizeof(float) * (size_t)dim);
  for(int r = 0; r < rows; ++r) {
    const float* ar = a + (size_t)r * dim;
    const float* rr = resid ? resid + (size_t)r * dim : NULL;
    for(int i = 0; i < dim; ++i) y[i] = rr ? ar[i] + rr[i] : ar[i];
    float part[256];
    for(int t = 0; t < 256; ++t) {
      float s = 0.0f;
      for(int c = t; c < chunks; c += 256) s = s + ((y[4 * c] + y[4 * c + 1]) + (y[4 * c + 2] + y[4 * c + 3]));
      part[t] = s;
    }
    const float mean = mo_block256_sum(part) / (float)dim;
    for(int t = 0; t < 256; ++t) {
      float q = 0.0f;
      for(int c = t; c < chunks; c += 256) {
        const float dx = y[4 * c] + -mean, dy = y[4 * c + 1] + -mean, dz = y[4 * c + 2] + -mean, dw = y[4 * c + 3] + -mean;
        q = q + fmaf(dx, dx, fmaf(dy, dy, fmaf(dz, dz, dw * dw)));
      }
      part[t] = q;
    }
    const float var = mo_block256_sum(part) / (float)dim;
    const float denom = sqrtf(var + eps);
    float* o = out + (size_t)r * dim;
    for(int i = 0; i < dim; ++i) o[i] = ((y[i] + -mean) / denom) * gamma[i] + beta[i];
  }
  free(y);
}

/* v[j] <- v[j] + v[j ^ o] for o = g/2 .. 1 over a group of g entries (g a power of two <= 32) */
static inline float mo_group_sum(const float* v, int g) {
  float a[32], b[32];
  memcpy(a, v, sizeof(float) * (size_t)g);
  for(int o = g / 2; o > 0; o >>= 1) {
    for(int i = 0; i < g; ++i) b[i] = a[i] + a[i ^ o];
    memcpy(a, b, sizeof(float) * (size_t)g);
  }
  return a[0];
}

/* Single-query attention; key/value row of position p for query row r is base(r) + p*stride:
 * mode 0: base = r, stride = rows (time-major history); mode 1: base = (r % batch)*len (cross-attention);
 * mode 2: base = (r / len)*len (encoder self-attention, rows ordered [batch, len]).
 * A head is handled by g = dh/4 workers, worker j owning elements 4j..4j+3 of the head. */
typedef struct { const float *q, *k, *v, *log_mask; int rows, heads, dh, len, batch, mode; float* out; } mo_att_ctx;

MO_FMA_CLONES static void mo_attention_rows(int rb, int re, void* ctx) {
  const mo_att_ctx* c = (const mo_att_ctx*)ctx;
  const float *q = c->q, *k = c->k, *v = c->v, *log_mask = c->log_mask;
  const int rows = c->rows, heads = c->heads, dh = c->dh, len = c->len, batch = c->batch, mode = c->mode;
  float* out = c->out;
  const int dim = heads * dh;
  const int g = dh / 4;
  const float scale = 1.0f / sqrtf((float)dh);
  float* p = (float*)malloc(sizeof(float) * (size_t)len);
  for(int r = rb; r < re; ++r) {
    const int group = mode == 1 ? r % batch : (mode == 2 ? r / len : 0);
    const size_t base = mode == 0 ? (size_t)r : (size_t)group * len;
    const size_t stride = mode == 0 ? (size_t)rows : 1;
    const float* mask = (mode != 0 && log_mask) ? log_mask + (size_t)group * len : NULL;
    for(int h = 0; h < heads; ++h) {
      const float* qh = q + (size_t)r * dim + h * dh;
      float mx = -FLT_MAX;
      for(int pos = 0; pos < len; ++pos) {
        const float* kr = k + (base + pos * stride) * dim + h * dh;
        float d[32];
        for(int j = 0; j < g; ++j) {
          float t = qh[4 * j] * kr[4 * j];
          t = fmaf(qh[4 * j + 1], kr[4 * j + 1], t);
          t = fmaf(qh[4 * j + 2], kr[4 * j + 2], t);
          t = fmaf(qh[4 * j + 3], kr[4 * j + 3], t);
          d[j] = t;
        }
        float s = mo_group_sum(d, g);
        s = s * scale;
        if(mask) s = s + mask[pos];
        p[pos] = s;
        if(s > mx) mx = s;
      }
      float part[32];
      for(int j = 0; j < g; ++j) part[j] = 0.0f;
      for(int pos = 0; pos < len; ++pos) {
        const float e = mo_det_expf_i(p[pos] + -mx);
        p[pos] = e;
        part[pos % g] = part[pos % g] + e;
      }
      const float sum = mo_group_sum(part, g);
      for(int pos = 0; pos < len; ++pos) p[pos] = p[pos] / sum;
      /* every output element is the fma chain over the positions in ascending order, starting from 0;
       * walking position-major keeps that order per element and reads each value row contiguously */
      float* o = out + (size_t)r * dim + h * dh;
      float acc[128];
      for(int i = 0; i < dh; ++i) acc[i] = 0.0f;
      for(int pos = 0; pos < len; ++pos) {
        const float w = p[pos];
        const float* vr = v + (base + pos * stride) * dim + h * dh;
        for(int i = 0; i < dh; ++i) acc[i] = fmaf(w, vr[i], acc[i]);
      }
      for(int i = 0; i < dh; ++i) o[i] = acc[i];
    }
  }
  free(p);
}

void mo_attention1(const float* q, const float* k, const float* v, const float* log_mask, int rows, int heads, int dh, int len, int batch,
                   int mode, float* out) {
  mo_att_ctx c = {q, k, v, log_mask, rows, heads, dh, len, batch, mode, out};
  mo_parallel_rows(rows, mo_attention_rows, &c);
}

/* larger value first; ties: smaller index first */
static inline int mo_better(float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia < ib); }
/* cand_score[r][j] = (j-th largest logit - lse(row)) + prev_score[r]; cand_word[r][j]; k <= 8 */
typedef struct { const float* logits; int vocab, k; const float* prev_scores; float* cand_score; int32_t* cand_word; } mo_lse_ctx;

MO_FMA_CLONES static void mo_lse_rows(int rb, int re, void* ctx) {
  const mo_lse_ctx* c = (const mo_lse_ctx*)ctx;
  const float* logits = c->logits;
  const int vocab = c->vocab, k = c->k;
  const float* prev_scores = c->prev_scores;
  float* cand_score = c->cand_score;
  int32_t* cand_word = c->cand_word;
  for(int r = rb; r < re; ++r) {
    const float* row = logits + (size_t)r * vocab;
    float tv[8];
    int ti[8];
    for(int j = 0; j < k; ++j) { tv[j] = -FLT_MAX; ti[j] = 0x7fffffff; }
    for(int i = 0; i < vocab; ++i) {
      const float x = row[i];
      if(mo_better(x, i, tv[k - 1], ti[k - 1])) {
        int pos = k - 1;
        while(pos > 0 && mo_better(x, i, tv[pos - 1], ti[pos - 1])) { tv[pos] = tv[pos - 1]; ti[pos] = ti[pos - 1]; --pos; }
        tv[pos] = x;
        ti[pos] = i;
      }
    }
    /* log-sum-exp over blocks of 128 consecutive entries (the last one may be short): per block its maximum m_b
     * and s_b = sum of exp(x - m_b), entries added one after the other in ascending order starting from 0;
     * then M = max_b m_b, S = sum over the blocks in ascending order of s_b * exp(m_b - M) (product and sum
     * rounded separately), lse = M + log(S).  A producer that owns one block of a row at a time (the output
     * GEMM's write-back) can compute the per-block pairs without seeing the rest of the row. */
    const int nb = (vocab + 127) / 128;
    float big = -FLT_MAX;
    float* bm = (float*)malloc(sizeof(float) * (size_t)nb * 2);
    float* bs = bm + nb;
    for(int b = 0; b < nb; ++b) {
      const int lo = b * 128, hi = lo + 128 < vocab ? lo + 128 : vocab;
      float m = -FLT_MAX;
      for(int i = lo; i < hi; ++i) if(row[i] > m) m = row[i];
      float sb = 0.0f;
      for(int i = lo; i < hi; ++i) sb = sb + mo_det_expf_i(row[i] + -m);
      bm[b] = m;
      bs[b] = sb;
      if(m > big) big = m;
    }
    float total = 0.0f;
    for(int b = 0; b < nb; ++b) {
      const float term = bs[b] * mo_det_expf_i(bm[b] + -big);
      total = total + term;
    }
    free(bm);
    const float lse = big + mo_det_logf_i(total);
    const float ps = prev_scores ? prev_scores[r] : 0.0f;
    for(int j = 0; j < k; ++j) {
      cand_score[(size_t)r * k + j] = (tv[j] + -lse) + ps;
      cand_word[(size_t)r * k + j] = ti[j];
    }
  }
}

void mo_lse_topk(const float* logits, int rows, int vocab, int k, const float* prev_scores, float* cand_score, int32_t* cand_word) {
  mo_lse_ctx c = {logits, vocab, k, prev_scores, cand_score, cand_word};
  mo_parallel_rows(rows, mo_lse_rows, &c);
}

/* out[r,:] = wemb[words[r],:] * scale + pos[(pos_mod ? r % pos_mod : 0),:]   (words NULL: zero embedding) */
void mo_embed(const float* wemb, const int32_t* words, const float* pos, int pos_mod, float scale, int rows, int dim, float* out) {
  for(int r = 0; r < rows; ++r) {
    const float* e = words ? wemb + (size_t)words[r] * dim : NULL;
    const float* p = pos + (size_t)(pos_mod ? r % pos_mod : 0) * dim;
    for(int i = 0; i < dim; ++i) out[(size_t)r * dim + i] = (e ? e[i] : 0.0f) * scale + p[i];
  }
}

/* SSRU cell on already gathered state: sig = 1/(1+exp(-f)); c' = fma(x, 1 - sig, c*sig); h = relu(c') */
MO_FMA_CLONES void mo_ssru_cell(const float* cell, const float* xw, const float* f, size_t n, float* cell_new, float* h) {
  for(size_t i = 0; i < n; ++i) {
    const float sig = 1.0f / (1.0f + mo_det_expf_i(-f[i]));
    const float cn = fmaf(xw[i], 1.0f + -sig, cell[i] * sig);
    cell_new[i] = cn;
    h[i] = cn > 0.0f ? cn : 0.0f;
  }
}
