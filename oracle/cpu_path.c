/* TEST INFRASTRUCTURE -- not part of the product.
 *
 * CPU restatement ("port") of the reference's CPU branches for the dense-contraction path,
 * in the reference's own arithmetic (fp32 storage and accumulation for Real; fp16 storage with
 * fp32 accumulation for Half).  It exists to (1) cross-check the fp64 numpy oracle in
 * oracle/oracle.py, and (2) be timed on the host cores as the CPU baseline.  Nothing in the
 * shipped library links or calls it.
 *
 * What it follows (paths inside the ginn source tree):
 *   cpu_gemm            ginn/node/prod.h:30-32,41-47  (C = A*B, dB += A^T*dC, dA += dC*B^T)
 *   cpu_gemm_batched    ginn/node/prod.h:108-117,129-147 (serial loop over the batch)
 *   cpu_affine_forward  ginn/node/affine.h:48-54,74-76 + ginn/nonlin.h:93-95,116-118,136-145
 *   cpu_affine_backward ginn/node/affine.h:79-102     + ginn/nonlin.h:96-106,119-126,146-152
 * The reference evaluates these with Eigen expressions; Eigen is not vendored with the
 * reference (empty submodule, pinned at libeigen/eigen 87300c93), so the dense product is
 * restated here as a packed, register-blocked GEMM with the same operation order at the
 * level the reference fixes it: products accumulate into the destination (`+=`), bias is
 * added per row across all columns, gradients of inputs without has_grad are skipped.
 *
 * Column-major everywhere; dtype 0 = float, 1 = IEEE half (uint16 bit patterns).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define MR 16
#define NR 8
#define KC 256
#define MC 256 /* multiple of MR */
#define NC 1024 /* multiple of NR */

typedef _Float16 half_t;

static inline float ld_elem(int dtype, const void* p, long i) {
  return dtype == 0 ? ((const float*)p)[i] : (float)((const half_t*)p)[i];
}
static inline void st_elem(int dtype, void* p, long i, float v) {
  if (dtype == 0)
    ((float*)p)[i] = v;
  else
    ((half_t*)p)[i] = (half_t)v;
}

/* op(A)(i, p): A stored column-major with leading dimension lda; ta = stored as k x m. */
static inline float a_at(int dtype, const void* A, long lda, int ta, long i, long p) {
  return ta ? ld_elem(dtype, A, p + i * lda) : ld_elem(dtype, A, i + p * lda);
}
static inline float b_at(int dtype, const void* B, long ldb, int tb, long p, long j) {
  return tb ? ld_elem(dtype, B, j + p * ldb) : ld_elem(dtype, B, p + j * ldb);
}

/* acc(MR x NR) += Apanel(MR x kc, p-major) * Bpanel(kc x NR, p-major).
 * One MR-wide vector per column of the register tile; the compiler lowers it to the widest
 * SIMD of each clone (one zmm, two ymm, four xmm). */
typedef float vmr_t __attribute__((vector_size(MR * 4), aligned(4)));
__attribute__((target_clones("avx512f", "avx2", "default"))) static void
micro_kernel(long kc, const float* restrict ap, const float* restrict bp, float* restrict acc) {
  vmr_t c[NR];
  for (int j = 0; j < NR; ++j) c[j] = (vmr_t){0};
  for (long p = 0; p < kc; ++p) {
    const vmr_t a = *(const vmr_t*)(ap + p * MR);
    const float* b = bp + p * NR;
#pragma GCC unroll 8
    for (int j = 0; j < NR; ++j) c[j] += a * b[j];
  }
  for (int j = 0; j < NR; ++j) *(vmr_t*)(acc + j * MR) = c[j];
}

/* C(m x n) = op(A) * op(B) + (accumulate ? C : 0), fp32 accumulation, threads over column blocks. */
void cpu_gemm(int dtype, int ta, int tb, long m, long n, long k, const void* A, long lda,
              const void* B, long ldb, void* C, long ldc, int accumulate, int threads) {
  if (m <= 0 || n <= 0) return;
  const long njc = (n + NC - 1) / NC;
  const long nic = (m + MC - 1) / MC;
  const long ntasks = njc * nic;
  (void)threads;
#ifdef _OPENMP
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
#endif
  {
    float* apack = (float*)aligned_alloc(64, sizeof(float) * MC * KC);
    float* bpack = (float*)aligned_alloc(64, sizeof(float) * KC * NC);
    float* ctile = (float*)aligned_alloc(64, sizeof(float) * MC * NC);
    float acc[MR * NR] __attribute__((aligned(64)));
#ifdef _OPENMP
#pragma omp for schedule(dynamic)
#endif
    for (long task = 0; task < ntasks; ++task) {
      const long jc = (task / nic) * NC, ic = (task % nic) * MC;
      const long nb = n - jc < NC ? n - jc : NC;
      const long mb = m - ic < MC ? m - ic : MC;
      for (long j = 0; j < nb; ++j)
        for (long i = 0; i < mb; ++i)
          ctile[j * MC + i] = accumulate ? ld_elem(dtype, C, (ic + i) + (jc + j) * ldc) : 0.f;
      for (long pc = 0; pc < k; pc += KC) {
        const long kb = k - pc < KC ? k - pc : KC;
        /* pack B block: panels of NR columns, p-major, zero padded */
        for (long jr = 0; jr < nb; jr += NR) {
          float* dst = bpack + jr * KC;
          for (int jj = 0; jj < NR; ++jj) {
            if (jr + jj >= nb) {
              for (long p = 0; p < kb; ++p) dst[p * NR + jj] = 0.f;
            } else if (dtype == 0) {
              const float* src = (const float*)B + (tb ? (jc + jr + jj) + pc * ldb : pc + (jc + jr + jj) * ldb);
              const long st = tb ? ldb : 1;
              for (long p = 0; p < kb; ++p) dst[p * NR + jj] = src[p * st];
            } else {
              const half_t* src = (const half_t*)B + (tb ? (jc + jr + jj) + pc * ldb : pc + (jc + jr + jj) * ldb);
              const long st = tb ? ldb : 1;
              for (long p = 0; p < kb; ++p) dst[p * NR + jj] = (float)src[p * st];
            }
          }
        }
        /* pack A block: panels of MR rows, p-major, zero padded */
        for (long ir = 0; ir < mb; ir += MR) {
          float* dst = apack + ir * KC;
          const int rows = mb - ir < MR ? (int)(mb - ir) : MR;
          for (long p = 0; p < kb; ++p) {
            if (dtype == 0) {
              const float* src = (const float*)A + (ta ? (pc + p) + (ic + ir) * lda : (ic + ir) + (pc + p) * lda);
              const long st = ta ? lda : 1;
              for (int ii = 0; ii < rows; ++ii) dst[p * MR + ii] = src[ii * st];
            } else {
              const half_t* src = (const half_t*)A + (ta ? (pc + p) + (ic + ir) * lda : (ic + ir) + (pc + p) * lda);
              const long st = ta ? lda : 1;
              for (int ii = 0; ii < rows; ++ii) dst[p * MR + ii] = (float)src[ii * st];
            }
            for (int ii = rows; ii < MR; ++ii) dst[p * MR + ii] = 0.f;
          }
        }
        for (long jr = 0; jr < nb; jr += NR)
          for (long ir = 0; ir < mb; ir += MR) {
            micro_kernel(kb, apack + ir * KC, bpack + jr * KC, acc);
            for (int jj = 0; jj < NR && jr + jj < nb; ++jj)
              for (int ii = 0; ii < MR && ir + ii < mb; ++ii)
                ctile[(jr + jj) * MC + ir + ii] += acc[jj * MR + ii];
          }
      }
      for (long j = 0; j < nb; ++j)
        for (long i = 0; i < mb; ++i)
          st_elem(dtype, C, (ic + i) + (jc + j) * ldc, ctile[j * MC + i]);
    }
    free(apack);
    free(bpack);
    free(ctile);
  }
}

/* Serial loop over the batch, as the reference's CPU branch does. */
void cpu_gemm_batched(int dtype, int ta, int tb, long m, long n, long k, const void* A, long lda,
                      long sa, const void* B, long ldb, long sb, void* C, long ldc, long sc,
                      long batches, int accumulate, int threads) {
  const long es = dtype == 0 ? 4 : 2;
  for (long i = 0; i < batches; ++i)
    cpu_gemm(dtype, ta, tb, m, n, k, (const char*)A + i * sa * es, lda,
             (const char*)B + i * sb * es, ldb, (char*)C + i * sc * es, ldc, accumulate, threads);
}

static float act_forward(int dtype, int act, float x) {
  switch (act) {
    case 1: return tanhf(x);
    case 2:
      if (dtype == 1) {
        if (x > 0.f) return 1.f / (1.f + expf(-x));
        return expf(x) / (1.f + expf(x));
      }
      return 0.5f * tanhf(0.5f * x) + 0.5f;
    case 3: return x > 0.f ? x : 0.f;
    default: return x;
  }
}
static float act_backward(int dtype, int act, float y, float dy) {
  switch (act) {
    case 1: return dtype == 1 ? dy - y * y * dy : (1.f - y * y) * dy;
    case 2: return y * (1.f - y) * dy;
    case 3: return y > 0.f ? dy : 0.f;
    default: return dy;
  }
}

/* out = act( sum_i A_i * B_i + bias ): first product assigned with the bias added per row,
 * further products accumulated, activation applied last. */
void cpu_affine_forward(int dtype, int npairs, const void* const* A, const long* lda,
                        const void* const* B, const long* ldb, const long* ks, long m, long n,
                        const void* bias, int act, void* out, long ldo, int threads) {
  if (npairs == 0)
    for (long j = 0; j < n; ++j)
      for (long i = 0; i < m; ++i) st_elem(dtype, out, i + j * ldo, 0.f);
  for (int p = 0; p < npairs || p == 0; ++p) {
    if (p < npairs)
      cpu_gemm(dtype, 0, 0, m, n, ks[p], A[p], lda[p], B[p], ldb[p], out, ldo, p > 0, threads);
    if (p == 0 && bias)
      for (long j = 0; j < n; ++j)
        for (long i = 0; i < m; ++i)
          st_elem(dtype, out, i + j * ldo, ld_elem(dtype, out, i + j * ldo) + ld_elem(dtype, bias, i));
  }
  if (act)
    for (long j = 0; j < n; ++j)
      for (long i = 0; i < m; ++i)
        st_elem(dtype, out, i + j * ldo, act_forward(dtype, act, ld_elem(dtype, out, i + j * ldo)));
}

/* dA = dout (.) act'(out) into `scratch` (the node's dpreactiv_), then
 * dbias += rowsum(dA); dB_i += A_i^T dA; dA_i += dA B_i^T, each only when the slot is non-null. */
void cpu_affine_backward(int dtype, int npairs, const void* const* A, const long* lda,
                         const void* const* B, const long* ldb, const long* ks, void* const* dA,
                         const long* ldda, void* const* dB, const long* lddb, long m, long n,
                         const void* dout, long lddout, const void* out, long ldout, int act,
                         void* dbias, void* scratch, int threads) {
  for (long j = 0; j < n; ++j)
    for (long i = 0; i < m; ++i) {
      const float dy = ld_elem(dtype, dout, i + j * lddout);
      const float y = act ? ld_elem(dtype, out, i + j * ldout) : 0.f;
      st_elem(dtype, scratch, i + j * m, act_backward(dtype, act, y, dy));
    }
  if (dbias)
    for (long i = 0; i < m; ++i) {
      float s = 0.f;
      for (long j = 0; j < n; ++j) s += ld_elem(dtype, scratch, i + j * m);
      st_elem(dtype, dbias, i, ld_elem(dtype, dbias, i) + s);
    }
  for (int p = 0; p < npairs; ++p) {
    if (dB && dB[p])
      cpu_gemm(dtype, 1, 0, ks[p], n, m, A[p], lda[p], scratch, m, dB[p], lddb[p], 1, threads);
    if (dA && dA[p])
      cpu_gemm(dtype, 0, 1, m, ks[p], n, scratch, m, B[p], ldb[p], dA[p], ldda[p], 1, threads);
  }
}

int cpu_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
