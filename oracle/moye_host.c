/*
 * TEST INFRASTRUCTURE -- CPU restatement of MoYe.jl's host `gemm!` / `copyto!` path.
 *
 * This file is the checker the CUDA kernels are compared with, and the timed CPU baseline.
 * Nothing in the product library links it.  The reference is Julia and cannot run where
 * this is built, so the functions below restate its algorithms in plain C; each one names
 * the reference source it follows (paths inside the MoYe.jl project).
 *
 * Arithmetic rule (the parity definition).  MoYe's host GEMM is the `gemm!` rank tower
 * (src/algorithm/blas.jl:11-88) over the 1x1x1 atom `UniversalFMA`, whose `fma!` is
 * `d .= a .* b .+ c` (src/arch/mma/mma.jl:64): one multiply, one add, two roundings, k
 * ascending, accumulator starting at zero (`zeros!`, examples/gemm.jl:39) and finally
 * overwriting C (examples/gemm.jl:62).  Julia never contracts `a*b+c` into an FMA on the
 * host, so this file must be compiled with -ffp-contract=off.  The product is formed in
 * promote_type(TA,TB): literally, Int8*Int8 wraps in Int8 and Float16*Float16 rounds to
 * Float16 before the add.  The meaningful reference ("fp32-accumulated", "Int32") therefore
 * widens the inputs first (exact) and runs the same tower in Float32 / Int32; both forms are
 * provided, the widened one is what the GPU is compared with.
 *
 * Parity pin: the reference holds no stored numeric GEMM vectors (test/host/tiling_matmul.jl:41
 * checks `C ≈ A*B'`, test/device/matmul.jl:81 runs only on a GPU); this restatement is pinned
 * by (i) the bit-exact copy goldens of test/copy.jl, (ii) agreement of its three GEMM forms
 * (tower, emulated kernel, plain triple loop) with each other and with an fp64 product.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ scalar codecs */
static float half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h >> 15) << 31;
  uint32_t exp = (h >> 10) & 0x1f;
  uint32_t man = h & 0x3ff;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static uint16_t float_to_half_rne(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint16_t sign = (uint16_t)((x >> 16) & 0x8000);
  uint32_t ax = x & 0x7fffffffu;
  if (ax >= 0x7f800000u) return (uint16_t)(sign | (ax > 0x7f800000u ? 0x7e00 : 0x7c00));
  if (ax >= 0x477ff000u) return (uint16_t)(sign | 0x7c00); /* rounds to inf */
  if (ax < 0x33000001u) return sign;                       /* rounds to zero */
  int e = (int)(ax >> 23) - 127;
  uint32_t m = (ax & 0x7fffffu) | 0x800000u;
  int shift = e < -14 ? 13 + (-14 - e) : 13;
  uint32_t half_m = m >> shift;
  uint32_t rem = m & ((1u << shift) - 1);
  uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (half_m & 1))) ++half_m;
  uint16_t out;
  if (e < -14) out = (uint16_t)half_m; /* subnormal (may carry into the normal range) */
  else out = (uint16_t)(((uint32_t)(e + 15) << 10) + (half_m - 0x400u));
  return (uint16_t)(sign | out);
}

static float bf16_to_float(uint16_t b) {
  uint32_t bits = (uint32_t)b << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static uint16_t float_to_bf16_rne(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40);
  uint32_t lsb = (x >> 16) & 1;
  x += 0x7fffu + lsb;
  return (uint16_t)(x >> 16);
}

static float e4m3_to_float(uint8_t v) {
  int sign = v >> 7, exp = (v >> 3) & 0xf, man = v & 7;
  float r;
  if (exp == 0) r = ldexpf((float)man, -9);
  else if (exp == 15 && man == 7) r = NAN;
  else r = ldexpf(1.0f + (float)man / 8.0f, exp - 7);
  return sign ? -r : r;
}

/* round-to-nearest-even with saturation to +-448 (the "satfinite" conversion) */
static uint8_t float_to_e4m3_rne_sat(float f) {
  if (isnan(f)) return 0x7f;
  uint8_t sign = signbit(f) ? 0x80 : 0;
  float a = fabsf(f);
  if (a >= 448.0f) return (uint8_t)(sign | 0x7e);
  if (a < ldexpf(1.0f, -10)) return sign; /* below half the smallest subnormal */
  int e;
  frexpf(a, &e); /* a = m * 2^e, m in [0.5,1) */
  int exp = e - 1;
  if (exp < -6) exp = -6; /* subnormal range shares the scale 2^-6 */
  float scaled = ldexpf(a, 3 - exp); /* units of the last mantissa bit */
  float r = nearbyintf(scaled);      /* default rounding mode: nearest even */
  int q = (int)r;
  int biased;
  if (exp == -6 && q < 8) {
    biased = 0; /* subnormal */
  } else {
    if (q == 16) { q = 8; ++exp; }
    biased = exp + 7;
    q -= 8;
  }
  if (biased > 15 || (biased == 15 && q > 6)) return (uint8_t)(sign | 0x7e);
  return (uint8_t)(sign | (biased << 3) | q);
}

void moye_oracle_half_to_float(const uint16_t* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = half_to_float(in[i]);
}
void moye_oracle_float_to_half(const float* in, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = float_to_half_rne(in[i]);
}
void moye_oracle_bf16_to_float(const uint16_t* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = bf16_to_float(in[i]);
}
void moye_oracle_float_to_bf16(const float* in, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = float_to_bf16_rne(in[i]);
}
void moye_oracle_e4m3_to_float(const uint8_t* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = e4m3_to_float(in[i]);
}
void moye_oracle_float_to_e4m3(const float* in, uint8_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = float_to_e4m3_rne_sat(in[i]);
}

/* ------------------------------------------------------------------ UniversalFMA, literally
 * `d .= a .* b .+ c` with Julia's promotion (src/arch/mma/mma.jl:64): the product is formed
 * in the operand type before it meets the accumulator. */
int32_t moye_oracle_fma_literal_s8(int8_t a, int8_t b, int32_t c) {
  int8_t p = (int8_t)((int)a * (int)b); /* Int8*Int8 wraps modulo 256 */
  return (int32_t)p + c;
}
float moye_oracle_fma_literal_f16(uint16_t a, uint16_t b, float c) {
  float p = half_to_float(a) * half_to_float(b);
  p = half_to_float(float_to_half_rne(p)); /* Float16*Float16 rounds to Float16 */
  return p + c;
}

/* ------------------------------------------------------------------ layout function
 * layout(i) for a flattened layout: colexicographic split of the 0-based index, every mode
 * wrapping (`%`) including the last; a rank-1 layout multiplies without wrapping
 * (src/stride.jl:1-31). */
static int64_t layout_offset0(int rank, const int64_t* shape, const int64_t* stride, int64_t idx0) {
  if (rank == 1) return idx0 * stride[0];
  int64_t off = 0;
  for (int k = 0; k < rank; ++k) {
    off += (idx0 % shape[k]) * stride[k];
    idx0 /= shape[k];
  }
  return off;
}

void moye_oracle_layout_eval(int rank, const int64_t* shape, const int64_t* stride, int64_t first, int64_t n,
                             int64_t* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = 1 + layout_offset0(rank, shape, stride, first + i - 1);
}

/* Elementwise `copyto!(dst, src)`: i = 1:size(src) through both layouts
 * (src/algorithm/copy.jl:4-16,42-64). */
void moye_oracle_copy_layout(void* dst, int drank, const int64_t* dshape, const int64_t* dstride, const void* src,
                             int srank, const int64_t* sshape, const int64_t* sstride, int64_t n, int elem_bytes) {
  for (int64_t i = 0; i < n; ++i) {
    int64_t so = layout_offset0(srank, sshape, sstride, i);
    int64_t dofs = layout_offset0(drank, dshape, dstride, i);
    memcpy((char*)dst + dofs * elem_bytes, (const char*)src + so * elem_bytes, (size_t)elem_bytes);
  }
}

/* `copy_kernel` (test/host/copy_async.jl:3-25) run sequentially over blocks and threads
 * (the reference's own host emulation of a kernel, test/copy.jl:23-30): every block takes a
 * (bm, bn) tile of the column-major (m, n) matrix, every thread of the (tm, tn) thread
 * layout copies its interleaved partition global -> "shared" tile, then after the barrier
 * shared -> global.  m % bm == 0, n % bn == 0, bm % tm == 0, bn % tn == 0. */
int moye_oracle_copy_kernel(void* dst, int64_t dst_ld, const void* src, int64_t src_ld, int64_t m, int64_t n,
                            int bm, int bn, int tm, int tn, int elem_bytes) {
  if (m % bm || n % bn || bm % tm || bn % tn) return -1;
  char* smem = (char*)malloc((size_t)bm * bn * elem_bytes);
  if (!smem) return -2;
  for (int64_t by = 0; by < n / bn; ++by)
    for (int64_t bx = 0; bx < m / bm; ++bx) {
      const char* gs = (const char*)src + (bx * bm + by * bn * src_ld) * elem_bytes;
      char* gd = (char*)dst + (bx * bm + by * bn * dst_ld) * elem_bytes;
      for (int pass = 0; pass < 2; ++pass) /* pass 0: gmem->smem ; barrier ; pass 1: smem->gmem */
        for (int t = 0; t < tm * tn; ++t) {
          int ti = t % tm, tj = t / tm; /* get_congr_coord of a compact (tm,tn) thread layout */
          for (int j = 0; j < bn / tn; ++j)
            for (int i = 0; i < bm / tm; ++i) {
              int r = ti + i * tm, c = tj + j * tn;
              if (pass == 0)
                memcpy(smem + ((size_t)r + (size_t)c * bm) * elem_bytes, gs + ((int64_t)r + c * src_ld) * elem_bytes,
                       (size_t)elem_bytes);
              else
                memcpy(gd + ((int64_t)r + c * dst_ld) * elem_bytes, smem + ((size_t)r + (size_t)c * bm) * elem_bytes,
                       (size_t)elem_bytes);
            }
        }
    }
  free(smem);
  return 0;
}

/* ------------------------------------------------------------------ host GEMM, three forms
 * All take general element strides: A[m*a_sm + k*a_sk], B[n*b_sn + k*b_sk], C[m*c_sm + n*c_sn]
 * and compute C = A.B^T, overwriting C. */

/* (1) plain sequential-k triple loop. */
void moye_oracle_gemm_f32(const float* A, int64_t a_sm, int64_t a_sk, const float* B, int64_t b_sn, int64_t b_sk,
                          float* C, int64_t c_sm, int64_t c_sn, int64_t M, int64_t N, int64_t K) {
  for (int64_t n = 0; n < N; ++n)
    for (int64_t m = 0; m < M; ++m) {
      float acc = 0.0f;
      for (int64_t k = 0; k < K; ++k) {
        float p = A[m * a_sm + k * a_sk] * B[n * b_sn + k * b_sk];
        acc = p + acc;
      }
      C[m * c_sm + n * c_sn] = acc;
    }
}

void moye_oracle_gemm_s32(const int32_t* A, int64_t a_sm, int64_t a_sk, const int32_t* B, int64_t b_sn, int64_t b_sk,
                          int32_t* C, int64_t c_sm, int64_t c_sn, int64_t M, int64_t N, int64_t K) {
  for (int64_t n = 0; n < N; ++n)
    for (int64_t m = 0; m < M; ++m) {
      int32_t acc = 0;
      for (int64_t k = 0; k < K; ++k) acc = A[m * a_sm + k * a_sk] * B[n * b_sn + k * b_sk] + acc;
      C[m * c_sm + n * c_sn] = acc;
    }
}

void moye_oracle_gemm_f64(const double* A, int64_t a_sm, int64_t a_sk, const double* B, int64_t b_sn, int64_t b_sk,
                          double* C, int64_t c_sm, int64_t c_sn, int64_t M, int64_t N, int64_t K) {
  for (int64_t n = 0; n < N; ++n)
    for (int64_t m = 0; m < M; ++m) {
      double acc = 0.0;
      for (int64_t k = 0; k < K; ++k) {
        double p = A[m * a_sm + k * a_sk] * B[n * b_sn + k * b_sk];
        acc = p + acc;
      }
      C[m * c_sm + n * c_sn] = acc;
    }
}

/* (2) the `gemm!` rank tower on one thread's fragments (src/algorithm/blas.jl:39-88):
 *     for k (3,3,3,3 -> 3,2,2,3), for n, for m in serpentine order (:65), D = a*b + C. */
static void gemm_tower_f32(float* acc, int tM, int tN, const float* sA, int64_t sa_m, int64_t sa_k, const float* sB,
                           int64_t sb_n, int64_t sb_k, int bK) {
  for (int k = 0; k < bK; ++k)
    for (int n = 1; n <= tN; ++n)
      for (int m = 1; m <= tM; ++m) {
        int ms = (n & 1) ? m : tM + 1 - m;
        float p = sA[(ms - 1) * sa_m + k * sa_k] * sB[(n - 1) * sb_n + k * sb_k];
        acc[(ms - 1) + (n - 1) * tM] = p + acc[(ms - 1) + (n - 1) * tM];
      }
}

/* (3) `matmul_kernel` (examples/gemm.jl:4-64; gemm! form test/device/matmul.jl:3-53) run
 *     sequentially over blocks and threads: local_tile (bM,bK)/(bN,bK)/(bM,bN), gmem->smem
 *     copies by the (tAm,tAk) thread layout, barrier, per-thread accumulation over its
 *     (tCm,tCn)-interleaved partition, C overwritten at the end.  use_tower selects the gemm!
 *     tower (test/device/matmul.jl:46) or the explicit loop nest (examples/gemm.jl:51-57).
 *     M % bM == 0, N % bN == 0, K % bK == 0 as the reference requires. */
int moye_oracle_matmul_kernel_f32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int bM,
                                  int bN, int bK, int tAm, int tAk, int tCm, int tCn, int use_tower) {
  if (M % bM || N % bN || K % bK || bM % tAm || bN % tAm || bK % tAk || bM % tCm || bN % tCn) return -1;
  if (tAm * tAk != tCm * tCn) return -1;
  const int nthr = tCm * tCn, tM = bM / tCm, tN = bN / tCn;
  float* sA = (float*)malloc(sizeof(float) * bM * bK);
  float* sB = (float*)malloc(sizeof(float) * bN * bK);
  float* frg = (float*)malloc(sizeof(float) * nthr * tM * tN);
  if (!sA || !sB || !frg) return -2;
  for (int64_t by = 0; by < N / bN; ++by)
    for (int64_t bx = 0; bx < M / bM; ++bx) {
      memset(frg, 0, sizeof(float) * nthr * tM * tN); /* zeros!(frg_c) */
      for (int64_t kt = 0; kt < K / bK; ++kt) {
        /* copyto!(threadtile_sA, view(threadtile_gA, :, :, kt)) for every thread */
        for (int t = 0; t < nthr; ++t) {
          int ti = t % tAm, tj = t / tAm;
          for (int j = 0; j < bK / tAk; ++j) {
            int kk = tj + j * tAk;
            for (int i = 0; i < bM / tAm; ++i) {
              int r = ti + i * tAm;
              sA[r + kk * bM] = A[(bx * bM + r) + (kt * bK + kk) * M];
            }
            for (int i = 0; i < bN / tAm; ++i) {
              int r = ti + i * tAm;
              sB[r + kk * bN] = B[(by * bN + r) + (kt * bK + kk) * N];
            }
          }
        }
        /* cp_async_wait(); sync_threads() */
        for (int t = 0; t < nthr; ++t) {
          int ti = t % tCm, tj = t / tCm;
          float* acc = frg + (size_t)t * tM * tN;
          const float* cA = sA + ti; /* rows ti, ti+tCm, ... : stride tCm */
          const float* cB = sB + tj;
          if (use_tower) {
            gemm_tower_f32(acc, tM, tN, cA, tCm, bM, cB, tCn, bN, bK);
          } else {
            for (int k = 0; k < bK; ++k)
              for (int m = 0; m < tM; ++m)
                for (int n = 0; n < tN; ++n) {
                  float p = cA[m * tCm + k * bM] * cB[n * tCn + k * bN];
                  acc[m + n * tM] = acc[m + n * tM] + p;
                }
          }
        }
        /* sync_threads() */
      }
      for (int t = 0; t < nthr; ++t) { /* copyto!(computetile_gC, frg_c) */
        int ti = t % tCm, tj = t / tCm;
        const float* acc = frg + (size_t)t * tM * tN;
        for (int n = 0; n < tN; ++n)
          for (int m = 0; m < tM; ++m)
            C[(bx * bM + ti + m * tCm) + (by * bN + tj + n * tCn) * M] = acc[m + n * tM];
      }
    }
  free(sA);
  free(sB);
  free(frg);
  return 0;
}

/* ------------------------------------------------------------------ widened-input GEMM on samples
 * dtype: 1 = f16, 2 = bf16, 3 = s8, 5 = e4m3 (the values of moye_dtype_t).  A and B are
 * K-major (row stride lda / ldb elements).  Output element (m, n) goes to
 * out[i*N + n] for the i-th listed row (rows != NULL), for all n; or, when cols != NULL,
 * out[j*M + m] for the j-th listed column, for all m.  Float path: inputs widened to
 * Float32 (exact), sequential-k tower arithmetic.  Integer path: Int32. */
static float load_as_float(const void* p, int dtype, int64_t i) {
  switch (dtype) {
    case 1: return half_to_float(((const uint16_t*)p)[i]);
    case 2: return bf16_to_float(((const uint16_t*)p)[i]);
    case 5: return e4m3_to_float(((const uint8_t*)p)[i]);
    default: return ((const float*)p)[i];
  }
}

static void widen_row(const void* p, int dtype, int64_t row, int64_t ld, int64_t K, float* out) {
  for (int64_t k = 0; k < K; ++k) out[k] = load_as_float(p, dtype, row * ld + k);
}

static float dot_seq_f32(const float* a, const float* b, int64_t K) {
  float acc = 0.0f;
  for (int64_t k = 0; k < K; ++k) {
    float p = a[k] * b[k];
    acc = p + acc;
  }
  return acc;
}

static int32_t dot_seq_s8(const int8_t* a, const int8_t* b, int64_t K) {
  int32_t acc = 0;
  for (int64_t k = 0; k < K; ++k) acc = (int32_t)a[k] * (int32_t)b[k] + acc;
  return acc;
}

typedef struct {
  const void *A, *B;
  int dtype;
  int64_t lda, ldb, M, N, K;
  const int32_t* idx;
  int64_t nidx;
  int by_rows;
  void* out;
  int tid, nthreads;
} sample_job_t;

static void* sample_worker(void* arg) {
  sample_job_t* j = (sample_job_t*)arg;
  const int64_t other = j->by_rows ? j->N : j->M;
  if (j->dtype == 3) {
    const int8_t* A = (const int8_t*)j->A;
    const int8_t* B = (const int8_t*)j->B;
    int32_t* out = (int32_t*)j->out;
    for (int64_t i = j->tid; i < j->nidx; i += j->nthreads)
      for (int64_t o = 0; o < other; ++o) {
        int64_t m = j->by_rows ? j->idx[i] : o, n = j->by_rows ? o : j->idx[i];
        out[i * other + o] = dot_seq_s8(A + m * j->lda, B + n * j->ldb, j->K);
      }
    return NULL;
  }
  float* fixed = (float*)malloc(sizeof(float) * j->K);
  float* moving = (float*)malloc(sizeof(float) * j->K);
  float* out = (float*)j->out;
  for (int64_t i = j->tid; i < j->nidx; i += j->nthreads) {
    if (j->by_rows) widen_row(j->A, j->dtype, j->idx[i], j->lda, j->K, fixed);
    else widen_row(j->B, j->dtype, j->idx[i], j->ldb, j->K, fixed);
    for (int64_t o = 0; o < other; ++o) {
      if (j->by_rows) widen_row(j->B, j->dtype, o, j->ldb, j->K, moving);
      else widen_row(j->A, j->dtype, o, j->lda, j->K, moving);
      out[i * other + o] = j->by_rows ? dot_seq_f32(fixed, moving, j->K) : dot_seq_f32(moving, fixed, j->K);
    }
  }
  free(fixed);
  free(moving);
  return NULL;
}

int moye_oracle_gemm_samples(const void* A, int64_t lda, const void* B, int64_t ldb, int dtype, int64_t M, int64_t N,
                             int64_t K, const int32_t* idx, int64_t nidx, int by_rows, void* out, int nthreads) {
  if (nthreads < 1) nthreads = 1;
  if (nthreads > 256) nthreads = 256;
  pthread_t th[256];
  sample_job_t jobs[256];
  for (int t = 0; t < nthreads; ++t) {
    sample_job_t j = {A, B, dtype, lda, ldb, M, N, K, idx, nidx, by_rows, out, t, nthreads};
    jobs[t] = j;
    if (pthread_create(&th[t], NULL, sample_worker, &jobs[t]) != 0) return -1;
  }
  for (int t = 0; t < nthreads; ++t) pthread_join(th[t], NULL);
  return 0;
}

/* ------------------------------------------------------------------ threaded host GEMM
 * The reference's multi-threaded host path (test/host/tiling_matmul.jl:20-39): thread
 * `tid` of a (tr, tc) thread layout owns the interleaved partition of C (rows = ti mod tr,
 * columns = tj mod tc) and runs `for k, for m, for n: C[m,n] += A[m,k]*B[n,k]` on it.
 * A:(M,K), B:(N,K), C:(M,N), all column-major; C is zeroed first.  Only the rows
 * [0, m_limit) of every thread's partition are computed when m_limit < M (a bounded sample
 * for timing). */
typedef struct {
  const float *A, *B;
  float* C;
  int64_t M, N, K, m_limit;
  int tr, tc, tid;
} mt_job_t;

static void* mt_worker(void* arg) {
  mt_job_t* j = (mt_job_t*)arg;
  const int ti = j->tid % j->tr, tj = j->tid / j->tr;
  for (int64_t k = 0; k < j->K; ++k)
    for (int64_t m = ti; m < j->m_limit; m += j->tr) {
      const float a = j->A[m + k * j->M];
      for (int64_t n = tj; n < j->N; n += j->tc) {
        float p = a * j->B[n + k * j->N];
        j->C[m + n * j->M] = j->C[m + n * j->M] + p;
      }
    }
  return NULL;
}

int moye_oracle_matmul_threads_f32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int tr,
                                   int tc, int64_t m_limit) {
  const int nthreads = tr * tc;
  if (nthreads < 1 || nthreads > 256) return -1;
  if (m_limit <= 0 || m_limit > M) m_limit = M;
  for (int64_t n = 0; n < N; ++n) memset(C + n * M, 0, sizeof(float) * (size_t)m_limit);
  pthread_t th[256];
  mt_job_t jobs[256];
  for (int t = 0; t < nthreads; ++t) {
    mt_job_t j = {A, B, C, M, N, K, m_limit, tr, tc, t};
    jobs[t] = j;
    if (pthread_create(&th[t], NULL, mt_worker, &jobs[t]) != 0) return -1;
  }
  for (int t = 0; t < nthreads; ++t) pthread_join(th[t], NULL);
  return 0;
}
