// CUDA-core kernels for the shapes the tensor-core tiles do not fit:
//   * products with a tiny result (m*n of a few elements), e.g. the batched 1x1 dot products
//     that SoftmaxOp::backward and LayerNormNode::backward send through gpu_batched_prod
//     (ginn/nonlin.h:180-183, ginn/node/layernorm.h:61-64), and k == 0;
//   * the bias gradient alone (row sums of dY (.) act'(Y)) when no weight gradient is wanted.
//   * "skinny" products, where one extent is at most 16 (a 10-class output layer: W 10 x 1024 on
//     4096 columns, and its two gradients).  A 128 x 128 tensor-core tile would be 8 % full and
//     the product is bound by reading or writing the large operand once, so CUDA cores at HBM
//     speed win by a wide margin.  Three mappings, chosen so that the large operand is read or
//     written coalesced:
//       skinny_m_kernel   m <= 16, B contraction-contiguous: one warp per column of C, lanes
//                         along k, up to 16 running sums, warp reduction
//       skinny_mt_kernel  m <= 16, B outer-contiguous (weight gradients): lanes along n, one
//                         k-chunk per CTA row, partial sums added to C with atomics (fp32,
//                         accumulating products only)
//       skinny_k_kernel   k <= 32 in total: one thread per element of C, lanes along m
// fp32 accumulation throughout; the tiny-result kernel uses one warp per output element, lanes
// strided along the contraction.
#include <cuda_fp16.h>
#include "ptx.cuh"
#include "math.cuh"
#include "launch.h"

namespace gb {

namespace {

__device__ __forceinline__ float ld_f(const float* p) { return __ldg(p); }
__device__ __forceinline__ float ld_f(const __half* p) { return __half2float(ldg1(p)); }
// Plain (coherent) loads for locations this kernel also writes.
__device__ __forceinline__ float ld_rw(const float* p) { return *p; }
__device__ __forceinline__ float ld_rw(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ void st_f(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_f(__half* p, float v) { *p = __float2half_rn(v); }
// Value of v after one rounding to the storage type T (in registers; no memory access).
template <typename T>
__device__ __forceinline__ float round_to(float v) {
  return sizeof(T) == 2 ? __half2float(__float2half_rn(v)) : v;
}

template <typename T>
__device__ __forceinline__ float fetch(const Operand& op, long long boff, long long o,
                                       long long kk) {
  const long long col = op.k_contig ? o : kk;
  const long long row = op.k_contig ? kk : o;
  const T* p = (op.cols ? static_cast<const T*>(op.cols[col])
                        : static_cast<const T*>(op.base) + boff + col * op.ld) + row;
  float v = ld_f(p);
  if (op.dact != ACT_NONE) {
    const T* py = (op.ycols ? static_cast<const T*>(op.ycols[col])
                            : static_cast<const T*>(op.ybase) + boff + col * op.ld) + row;
    // The staged kernel rounds dY (.) act'(Y) to T before the product; do the same here.
    v = round_to<T>(act_backward<T>(op.dact, ld_f(py), v));
  }
  return v;
}

template <typename T>
__global__ void small_gemm_kernel(const __grid_constant__ Problem P) {
  const long long warp_global = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long per_batch = static_cast<long long>(P.M) * P.N;
  const long long total = per_batch * P.batches;
  if (warp_global >= total) return;
  const long long batch = warp_global / per_batch;
  const long long rem = warp_global % per_batch;
  const long long row = rem % P.M;
  const long long col = rem / P.M;
  float acc = 0.f;
  for (int p = 0; p < P.npairs; ++p) {
    const long long ab = batch * P.a[p].batch_stride, bb = batch * P.b[p].batch_stride;
    for (long long kk = lane; kk < P.k[p]; kk += 32)
      acc += fetch<T>(P.a[p], ab, row, kk) * fetch<T>(P.b[p], bb, col, kk);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    T* cp = (P.ccols ? static_cast<T*>(P.ccols[col])
                     : static_cast<T*>(P.c) + batch * P.c_batch_stride + col * P.ldc) + row;
    float x = acc;
    if (P.bias) x += ld_f(static_cast<const T*>(P.bias) + row);
    if (P.accumulate) x += ld_rw(cp);
    st_f(cp, act_forward<T>(P.act, x));
  }
}

constexpr int kSkinny = 16;

// Writes one element of C: bias, previous value, activation, one rounding.
template <typename T>
__device__ __forceinline__ void finish(const Problem& P, long long batch, long long row,
                                       long long col, float x) {
  T* cp = (P.ccols ? static_cast<T*>(P.ccols[col])
                   : static_cast<T*>(P.c) + batch * P.c_batch_stride + col * P.ldc) + row;
  if (P.bias) x += ld_f(static_cast<const T*>(P.bias) + row);
  if (P.accumulate) x += ld_rw(cp);
  st_f(cp, act_forward<T>(P.act, x));
}

// m <= 16: one warp per (column, batch); lanes strided along the contraction.
template <typename T>
__global__ void __launch_bounds__(256) skinny_m_kernel(const __grid_constant__ Problem P) {
  const long long warp_global = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp_global >= static_cast<long long>(P.N) * P.batches) return;
  const long long batch = warp_global / P.N;
  const long long col = warp_global % P.N;
  float acc[kSkinny];
#pragma unroll
  for (int m = 0; m < kSkinny; ++m) acc[m] = 0.f;
  for (int p = 0; p < P.npairs; ++p) {
    const long long ab = batch * P.a[p].batch_stride, bb = batch * P.b[p].batch_stride;
    for (long long kk = lane; kk < P.k[p]; kk += 32) {
      const float b = fetch<T>(P.b[p], bb, col, kk);
#pragma unroll
      for (int m = 0; m < kSkinny; ++m)
        if (m < P.M) acc[m] += fetch<T>(P.a[p], ab, m, kk) * b;
    }
  }
#pragma unroll
  for (int m = 0; m < kSkinny; ++m) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], off);
  }
  // lane m keeps row m (every lane holds every sum after the butterfly)
  float mine = 0.f;
#pragma unroll
  for (int m = 0; m < kSkinny; ++m)
    if (lane == m) mine = acc[m];
  if (lane < P.M) finish<T>(P, batch, lane, col, mine);
}

// m <= 16, accumulating, B outer-contiguous: thread = column n, blockIdx.y = k-chunk of 128.
__global__ void __launch_bounds__(128) skinny_mt_kernel(const __grid_constant__ Problem P) {
  const long long col = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long batch = blockIdx.z;
  if (col >= P.N) return;
  float acc[kSkinny];
#pragma unroll
  for (int m = 0; m < kSkinny; ++m) acc[m] = 0.f;
  // chunks are numbered over the concatenated contraction of all pairs
  long long chunk = blockIdx.y;
  for (int p = 0; p < P.npairs; ++p) {
    const long long nchunks = (P.k[p] + 127) / 128;
    if (chunk >= nchunks) {
      chunk -= nchunks;
      continue;
    }
    const long long ab = batch * P.a[p].batch_stride, bb = batch * P.b[p].batch_stride;
    const long long k1 = chunk * 128 + 128 < P.k[p] ? chunk * 128 + 128 : P.k[p];
    for (long long kk = chunk * 128; kk < k1; ++kk) {
      const float b = fetch<float>(P.b[p], bb, col, kk);
#pragma unroll
      for (int m = 0; m < kSkinny; ++m)
        if (m < P.M) acc[m] += fetch<float>(P.a[p], ab, m, kk) * b;
    }
    break;
  }
#pragma unroll
  for (int m = 0; m < kSkinny; ++m)
    if (m < P.M) {
      float* cp = (P.ccols ? static_cast<float*>(P.ccols[col])
                           : static_cast<float*>(P.c) + batch * P.c_batch_stride + col * P.ldc) + m;
      atomicAdd(cp, acc[m]);
    }
}

// total k <= 32: one thread per element of C, consecutive threads along m.
template <typename T>
__global__ void __launch_bounds__(256) skinny_k_kernel(const __grid_constant__ Problem P) {
  const long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long per_batch = static_cast<long long>(P.M) * P.N;
  if (e >= per_batch * P.batches) return;
  const long long batch = e / per_batch;
  const long long rem = e - batch * per_batch;
  const long long col = rem / P.M;
  const long long row = rem - col * P.M;
  float acc = 0.f;
  for (int p = 0; p < P.npairs; ++p) {
    const long long ab = batch * P.a[p].batch_stride, bb = batch * P.b[p].batch_stride;
    for (long long kk = 0; kk < P.k[p]; ++kk)
      acc += fetch<T>(P.a[p], ab, row, kk) * fetch<T>(P.b[p], bb, col, kk);
  }
  finish<T>(P, batch, row, col, acc);
}

// ---- lean variants for plain operands (no pointer tables, no fused derivative, one pair): the
// generic fetch() above costs some thirty instructions per element, which would bound these
// kernels; here an element is one load from base + o * so + k * sk. ----
template <typename T>
struct Plain {
  const T* p;
  long long so, sk;  // element strides along the outer index and along the contraction
  __device__ __forceinline__ Plain(const Operand& op, long long batch)
      : p(static_cast<const T*>(op.base) + batch * op.batch_stride),
        so(op.k_contig ? op.ld : 1),
        sk(op.k_contig ? 1 : op.ld) {}
};

// m <= 16, B contraction-contiguous.  A CTA owns 16 columns of C (two per warp).  The small
// operand A is staged, 512 contraction indices at a time, in shared memory as [m][k], so that
// lanes running along k read it without bank conflicts whatever its layout in memory is (read
// straight from global memory, an outer-contiguous A costs ten cache lines per load: lanes are
// 4 m bytes apart).  Every staged value is used for both columns of the warp.
__device__ __forceinline__ void ld4(const float* p, float (&x)[4]) {
  const float4 v = __ldg(reinterpret_cast<const float4*>(p));
  x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
}
__device__ __forceinline__ void ld4(const __half* p, float (&x)[4]) {
  const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
  x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
}

constexpr int kSkinnyKC = 512;
constexpr int kSkinnyCols = 2;  // columns of C per warp
template <typename T>
__global__ void __launch_bounds__(256) skinny_m_plain_kernel(const __grid_constant__ Problem P) {
  __shared__ __align__(16) float As[kSkinny * kSkinnyKC];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long batch = blockIdx.y;
  const Plain<T> A(P.a[0], batch), Bm(P.b[0], batch);
  const int M = P.M;
  const long long K = P.k[0];
  const long long col0 = static_cast<long long>(blockIdx.x) * (8 * kSkinnyCols) + warp * kSkinnyCols;
  const T* bp[kSkinnyCols];
  bool live[kSkinnyCols];
#pragma unroll
  for (int c = 0; c < kSkinnyCols; ++c) {
    live[c] = col0 + c < P.N;
    bp[c] = Bm.p + (live[c] ? col0 + c : 0) * Bm.so;  // contraction-contiguous: sk = 1
  }
  float acc[kSkinnyCols][kSkinny];
#pragma unroll
  for (int c = 0; c < kSkinnyCols; ++c)
#pragma unroll
    for (int m = 0; m < kSkinny; ++m) acc[c][m] = 0.f;
  // every column of B starts on a boundary of four elements
  const unsigned va = sizeof(T) * 4;
  const bool vec = (reinterpret_cast<uintptr_t>(Bm.p) & (va - 1)) == 0 && (Bm.so * sizeof(T)) % va == 0;
  for (long long k0 = 0; k0 < K; k0 += kSkinnyKC) {
    const int kc = K - k0 < kSkinnyKC ? static_cast<int>(K - k0) : kSkinnyKC;
    __syncthreads();
    for (int kk = threadIdx.x; kk < kc; kk += 256) {
      const T* ak = A.p + (k0 + kk) * A.sk;
#pragma unroll
      for (int m = 0; m < kSkinny; ++m)
        if (m < M) As[m * kSkinnyKC + kk] = ld_f(ak + m * A.so);
    }
    __syncthreads();
    if (vec) {
      // four consecutive contraction indices per lane: 16-byte loads of B and of the staged A
#pragma unroll 2
      for (int kk = 4 * lane; kk + 3 < kc; kk += 128) {
        float b[kSkinnyCols][4];
#pragma unroll
        for (int c = 0; c < kSkinnyCols; ++c) {
          if (live[c]) {
            ld4(bp[c] + k0 + kk, b[c]);
          } else {
            b[c][0] = b[c][1] = b[c][2] = b[c][3] = 0.f;
          }
        }
#pragma unroll
        for (int m = 0; m < kSkinny; ++m)
          if (m < M) {
            const float4 a = *reinterpret_cast<const float4*>(&As[m * kSkinnyKC + kk]);
#pragma unroll
            for (int c = 0; c < kSkinnyCols; ++c)
              acc[c][m] += (a.x * b[c][0] + a.y * b[c][1]) + (a.z * b[c][2] + a.w * b[c][3]);
          }
      }
    }
    // scalar path: everything when unaligned, else the last kc % 4 indices of the chunk
    for (int kk = (vec ? (kc & ~3) : 0) + lane; kk < kc; kk += 32) {
      float b[kSkinnyCols];
#pragma unroll
      for (int c = 0; c < kSkinnyCols; ++c) b[c] = live[c] ? ld_f(bp[c] + k0 + kk) : 0.f;
#pragma unroll
      for (int m = 0; m < kSkinny; ++m)
        if (m < M) {
          const float a = As[m * kSkinnyKC + kk];
#pragma unroll
          for (int c = 0; c < kSkinnyCols; ++c) acc[c][m] += a * b[c];
        }
    }
  }
#pragma unroll
  for (int c = 0; c < kSkinnyCols; ++c) {
    float mine = 0.f;
#pragma unroll
    for (int m = 0; m < kSkinny; ++m) {
      float v = acc[c][m];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      if (lane == m) mine = v;
    }
    if (live[c] && lane < M) finish<T>(P, batch, lane, col0 + c, mine);
  }
}

// m <= 16, accumulating, B outer-contiguous (weight gradients), plain operands.  A CTA of 32 x 8
// threads owns 32 columns of C and 256 contraction indices: warp ty sums its 32 indices for the
// 32 columns (lanes along n: coalesced reads of B; A is a broadcast), the eight warps meet in
// shared memory and one atomic add per element and CTA goes to memory.  (Atomics on the same
// cache line serialise in L2 at some 30 cycles each: one per thread and chunk, as a first version
// did, made 1.3 M of them the whole run time.)  The thread of column 0 also sums A along the
// contraction: the bias gradient, for free.
constexpr int kSkinnyMtChunk = 256;
__global__ void __launch_bounds__(256) skinny_mt_plain_kernel(const __grid_constant__ Problem P) {
  __shared__ float red[8][kSkinny][33];
  __shared__ float rsred[8][kSkinny];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const long long col = static_cast<long long>(blockIdx.x) * 32 + tx;
  const long long batch = blockIdx.z;
  const bool live = col < P.N;
  const Plain<float> A(P.a[0], batch), Bm(P.b[0], batch);
  const float* bp = Bm.p + (live ? col : 0) * Bm.so;
  const int M = P.M;
  const long long k0 = static_cast<long long>(blockIdx.y) * kSkinnyMtChunk + ty * 32;
  const long long k1 = k0 + 32 < P.k[0] ? k0 + 32 : P.k[0];
  // the CTA's slice of A (256 contraction indices x m) through shared memory: every thread
  // needs every value of it
  __shared__ float As[kSkinnyMtChunk][kSkinny + 1];
  {
    const long long kb = static_cast<long long>(blockIdx.y) * kSkinnyMtChunk;
    const int tid = ty * 32 + tx;
    const int kn = P.k[0] - kb < kSkinnyMtChunk ? static_cast<int>(P.k[0] - kb) : kSkinnyMtChunk;
    // storage order: index = k * M + m when m is contiguous, else m * kn + k
    for (int idx = tid; idx < kn * M; idx += 256) {
      const int kl = A.so == 1 ? idx / M : idx % kn;
      const int m = A.so == 1 ? idx % M : idx / kn;
      As[kl][m] = __ldg(A.p + (kb + kl) * A.sk + m * A.so);
    }
  }
  __syncthreads();
  float acc[kSkinny], rs[kSkinny];
#pragma unroll
  for (int m = 0; m < kSkinny; ++m) acc[m] = rs[m] = 0.f;
#pragma unroll 8
  for (long long kk = k0; kk < k1; ++kk) {
    const float b = live ? __ldg(bp + kk * Bm.sk) : 0.f;
    const float* ak = As[ty * 32 + static_cast<int>(kk - k0)];  // the same word in every lane
#pragma unroll
    for (int m = 0; m < kSkinny; ++m)
      if (m < M) {
        const float a = ak[m];
        acc[m] += a * b;
        rs[m] += a;
      }
  }
#pragma unroll
  for (int m = 0; m < kSkinny; ++m) {
    red[ty][m][tx] = acc[m];
    if (tx == 0) rsred[ty][m] = rs[m];
  }
  __syncthreads();
  if (ty == 0 && live) {
    float* cp = static_cast<float*>(P.c) + batch * P.c_batch_stride + col * P.ldc;
    const bool sums = P.rowsum != nullptr && blockIdx.x == 0 && tx == 0;
#pragma unroll
    for (int m = 0; m < kSkinny; ++m)
      if (m < M) {
        float v = 0.f, r = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
          v += red[w][m][tx];
          r += rsred[w][m];
        }
        atomicAdd(cp + m, v);
        if (sums) atomicAdd(static_cast<float*>(P.rowsum) + m, r);
      }
  }
}

// k <= 32: a CTA owns 256 rows x 16 columns of C (small tiles: many CTAs, so that enough loads
// and stores are in flight); thread = one row, its row of A in registers.
// Both operand tiles pass through shared memory so that global memory is read in the order it
// is stored (a contraction-contiguous A read row by row from the threads would again cost one
// cache line per lane).
constexpr int kSkinnyKCols = 16;
template <typename T, int KMAX>
__global__ void __launch_bounds__(256) skinny_k_plain_kernel(const __grid_constant__ Problem P) {
  __shared__ float Bs[kSkinnyKCols][KMAX + 1];
  __shared__ float As[256][KMAX + 1];
  const long long batch = blockIdx.z;
  const Plain<T> A(P.a[0], batch), Bm(P.b[0], batch);
  const int K = static_cast<int>(P.k[0]);
  const long long row0 = static_cast<long long>(blockIdx.x) * 256;
  const long long col0 = static_cast<long long>(blockIdx.y) * kSkinnyKCols;
  const int rows = P.M - row0 < 256 ? static_cast<int>(P.M - row0) : 256;
  const int cols = P.N - col0 < kSkinnyKCols ? static_cast<int>(P.N - col0) : kSkinnyKCols;
  // tiles in storage order: index = outer * K + k when the contraction is contiguous, else
  // k * extent + outer
  for (int idx = threadIdx.x; idx < cols * K; idx += 256) {
    const int c = Bm.sk == 1 ? idx / K : idx % cols;
    const int kk = Bm.sk == 1 ? idx % K : idx / cols;
    Bs[c][kk] = ld_f(Bm.p + (col0 + c) * Bm.so + kk * Bm.sk);
  }
  for (int idx = threadIdx.x; idx < rows * K; idx += 256) {
    const int r = A.sk == 1 ? idx / K : idx % rows;
    const int kk = A.sk == 1 ? idx % K : idx / rows;
    As[r][kk] = ld_f(A.p + (row0 + r) * A.so + kk * A.sk);
  }
  __syncthreads();
  if (static_cast<int>(threadIdx.x) >= rows) return;
  float a[KMAX];
#pragma unroll
  for (int kk = 0; kk < KMAX; ++kk) a[kk] = kk < K ? As[threadIdx.x][kk] : 0.f;
  const long long row = row0 + threadIdx.x;
  const float bias = P.bias ? ld_f(static_cast<const T*>(P.bias) + row) : 0.f;
  T* crow = static_cast<T*>(P.c) + batch * P.c_batch_stride + row;
  // eight columns at a time: the previous values of C (for +=) are requested together, so that
  // their latency is paid once per eight elements and not once per element
  for (int c0 = 0; c0 < cols; c0 += 8) {
    float x[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      x[j] = (P.accumulate && c0 + j < cols) ? ld_rw(crow + (col0 + c0 + j) * P.ldc) : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float acc = 0.f;
      const int c = c0 + j < cols ? c0 + j : 0;
#pragma unroll
      for (int kk = 0; kk < KMAX; ++kk)
        if (kk < K) acc += a[kk] * Bs[c][kk];  // the same word in every lane: a broadcast
      x[j] += acc + bias;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (c0 + j < cols) st_f(crow + (col0 + c0 + j) * P.ldc, act_forward<T>(P.act, x[j]));
  }
}

// ---- streaming variants: the same three mappings for the case that matters in practice, a
// large fp32 operand that is read or written exactly once (the ten-class output layer of the MLP
// configuration: logits, its weight gradient, the gradient of its input).  Measured at those
// shapes the kernels above ran at 0.7-1.4 TB/s whether or not the large operand was in L2: a CTA
// is a chain of dependent round trips to memory (a staging loop of scalar loads, a few loads per
// thread and trip), so it is latency that bounds them.  These variants bring the small operand
// in with one round of independent loads, move 16 bytes per thread and access with eight or more
// loads in flight, keep every CTA resident at once, and send few, wide atomics. ----

// Copies `count` floats of the small operand into shared memory, up to ROUNDS x 256 elements per
// round trip: all loads of a round are issued before its first store.  Element i is described by
// (q, r) = (i / d, i % d) for a divisor d the caller picks (the extent along which the operand is
// contiguous); `src_of(q, r)` gives its address and `pos(q, r)` its place.  The pair is advanced
// incrementally -- an integer division per element (a runtime divisor costs some twenty
// instructions) had made the copy two thirds of a kernel's instructions.
template <int ROUNDS, typename SrcFn, typename PosFn>
__device__ __forceinline__ void stage_small(float* dst, int count, int d, SrcFn src_of, PosFn pos) {
  int q = static_cast<int>(threadIdx.x) / d, r = static_cast<int>(threadIdx.x) % d;
  const int dq = 256 / d, dr = 256 % d;
  for (int base = 0; base < count; base += ROUNDS * 256) {
    float v[ROUNDS];
    int qq = q, rr = r;
#pragma unroll
    for (int t = 0; t < ROUNDS; ++t) {
      v[t] = base + t * 256 + static_cast<int>(threadIdx.x) < count ? __ldg(src_of(qq, rr)) : 0.f;
      qq += dq;
      rr += dr;
      if (rr >= d) {
        rr -= d;
        ++qq;
      }
    }
#pragma unroll
    for (int t = 0; t < ROUNDS; ++t) {
      if (base + t * 256 + static_cast<int>(threadIdx.x) < count) dst[pos(q, r)] = v[t];
      q += dq;
      r += dr;
      if (r >= d) {
        r -= d;
        ++q;
      }
    }
  }
}

// The same for a source that is one contiguous, 16-byte aligned run of `count` floats (count a
// multiple of four): 16-byte loads, up to ROUNDS x 1024 floats per round trip.
template <int ROUNDS, typename PosFn>
__device__ __forceinline__ void stage_run(float* dst, const float* src, int count, int d, PosFn pos) {
  const float4* src4 = reinterpret_cast<const float4*>(src);
  const int count4 = count >> 2;
  int q = 4 * static_cast<int>(threadIdx.x) / d, r = 4 * static_cast<int>(threadIdx.x) % d;
  const int dq = 1024 / d, dr = 1024 % d;
  for (int base = 0; base < count4; base += ROUNDS * 256) {
    float4 v[ROUNDS];
#pragma unroll
    for (int t = 0; t < ROUNDS; ++t) {
      const int i = base + t * 256 + threadIdx.x;
      v[t] = i < count4 ? __ldg(src4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int t = 0; t < ROUNDS; ++t) {
      if (base + t * 256 + static_cast<int>(threadIdx.x) < count4) {
        const float e[4] = {v[t].x, v[t].y, v[t].z, v[t].w};
        int qq = q, rr = r;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          dst[pos(qq, rr)] = e[j];
          if (++rr == d) {
            rr = 0;
            ++qq;
          }
        }
      }
      q += dq;
      r += dr;
      if (r >= d) {
        r -= d;
        ++q;
      }
    }
  }
}
__device__ __forceinline__ bool run_ok(const float* p, long long count) {
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0 && count % 4 == 0;
}

// m <= 16, fp32, B contraction-contiguous with 16-byte aligned columns, the whole of A (m x K)
// resident in shared memory as [m][kpad]; a CTA owns sixteen columns of C (two per warp), every
// CTA of the grid is resident at once.
__global__ void __launch_bounds__(256) skinny_m_stream_kernel(const __grid_constant__ Problem P,
                                                              int kpad) {
  extern __shared__ __align__(16) float As_dyn[];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long batch = blockIdx.y;
  const Plain<float> A(P.a[0], batch), Bm(P.b[0], batch);
  const int M = P.M;
  const int K = static_cast<int>(P.k[0]);
  // A in the order it is stored: element i = (q, r) with r the fast index -- m when m is
  // contiguous (q = k), else k (q = m)
  const bool m_fast = A.so == 1;
  const int d = m_fast ? M : K;
  auto a_pos = [&](int q, int r) { return m_fast ? r * kpad + q : q * kpad + r; };
  if ((m_fast ? A.sk == M : A.so == K) && run_ok(A.p, static_cast<long long>(M) * K))
    stage_run<10>(As_dyn, A.p, M * K, d, a_pos);  // A is one run: 10 K floats per round trip
  else
    stage_small<16>(
        As_dyn, M * K, d,
        [&](int q, int r) { return A.p + (m_fast ? static_cast<long long>(q) * A.sk + r
                                                 : static_cast<long long>(q) * A.so + r); },
        a_pos);
  if (kpad > K && threadIdx.x < M)  // the padding is read by the last 16-byte load of each row
    for (int k = K; k < kpad; ++k) As_dyn[threadIdx.x * kpad + k] = 0.f;
  __syncthreads();
  const long long col0 = static_cast<long long>(blockIdx.x) * 16 + warp * 2;
  const bool live0 = col0 < P.N, live1 = col0 + 1 < P.N;
  const float* b0 = Bm.p + (live0 ? col0 : 0) * Bm.so;
  const float* b1 = Bm.p + (live1 ? col0 + 1 : 0) * Bm.so;
  float acc0[kSkinny], acc1[kSkinny];
#pragma unroll
  for (int m = 0; m < kSkinny; ++m) acc0[m] = acc1[m] = 0.f;
#pragma unroll 4
  for (int kk = 4 * lane; kk < K; kk += 128) {
    float x0[4], x1[4];
    if (kk + 3 < K) {
      ld4(b0 + kk, x0);
      ld4(b1 + kk, x1);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        x0[e] = kk + e < K ? __ldg(b0 + kk + e) : 0.f;
        x1[e] = kk + e < K ? __ldg(b1 + kk + e) : 0.f;
      }
    }
#pragma unroll
    for (int m = 0; m < kSkinny; ++m)
      if (m < M) {
        const float4 a = *reinterpret_cast<const float4*>(&As_dyn[m * kpad + kk]);
        // one fused multiply-add per product (the kernel is bound by instruction issue)
        acc0[m] = fmaf(a.w, x0[3], fmaf(a.z, x0[2], fmaf(a.y, x0[1], fmaf(a.x, x0[0], acc0[m]))));
        acc1[m] = fmaf(a.w, x1[3], fmaf(a.z, x1[2], fmaf(a.y, x1[1], fmaf(a.x, x1[0], acc1[m]))));
      }
  }
  float mine0 = 0.f, mine1 = 0.f;
#pragma unroll
  for (int m = 0; m < kSkinny; ++m)
    if (m < M) {
      float v0 = acc0[m], v1 = acc1[m];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        v0 += __shfl_xor_sync(0xffffffffu, v0, off);
        v1 += __shfl_xor_sync(0xffffffffu, v1, off);
      }
      if (lane == m) {
        mine0 = v0;
        mine1 = v1;
      }
    }
  if (live0 && lane < M) finish<float>(P, batch, lane, col0, mine0);
  if (live1 && lane < M) finish<float>(P, batch, lane, col0 + 1, mine1);
}

// m <= 16, fp32, accumulating, B outer-contiguous with 16-byte aligned rows (a weight gradient).
// A CTA owns 128 columns of C and 128 contraction indices: a lane reads four neighbouring columns
// of B in one load, the eight warps interleave along the contraction (sixteen loads per lane,
// eight in flight), A's slice sits in shared memory as [k][16] (read as broadcasts), the warps
// meet in shared memory through conflict-free shared atomics and the CTA sends its 128 x m sums
// to C -- as 16-byte vector atomics when C is one contiguous, aligned run (ldc = m).
// blockIdx.x = 0 also sums A along k (bias gradient).
__global__ void __launch_bounds__(256, 2) skinny_mt_stream_kernel(const __grid_constant__ Problem P) {
  __shared__ __align__(16) float As[128 * kSkinny];
  __shared__ __align__(16) float red[kSkinny * 128];  // [m][j][lane]: column 4 * lane + j
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long batch = blockIdx.z;
  const Plain<float> A(P.a[0], batch), Bm(P.b[0], batch);
  const int M = P.M;
  const long long K = P.k[0];
  const long long kb = static_cast<long long>(blockIdx.y) * 128;
  const int kn = K - kb < 128 ? static_cast<int>(K - kb) : 128;
  const long long col = static_cast<long long>(blockIdx.x) * 128 + 4 * lane;
  const bool live = col < P.N;  // N is a multiple of four: a lane's columns live or die together
  // A's slice in the order it is stored: (q, r) = (k, m) when m is contiguous, else (m, k)
  const bool m_fast = A.so == 1;
  stage_small<8>(
      As, kn * M, m_fast ? M : kn,
      [&](int q, int r) { return A.p + (m_fast ? (kb + q) * A.sk + r
                                               : (kb + r) * A.sk + static_cast<long long>(q) * A.so); },
      [&](int q, int r) { return m_fast ? q * kSkinny + r : r * kSkinny + q; });
  for (int idx = threadIdx.x; idx < kSkinny * 128; idx += 256) red[idx] = 0.f;
  __syncthreads();
  float acc[4][kSkinny];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int m = 0; m < kSkinny; ++m) acc[j][m] = 0.f;
  const float* bp = Bm.p + (live ? col : 0);  // outer-contiguous: so = 1
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    float4 b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int kl = warp + 8 * (half * 8 + i);
      b[i] = (live && kl < kn) ? __ldg(reinterpret_cast<const float4*>(bp + (kb + kl) * Bm.sk))
                               : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int kl = warp + 8 * (half * 8 + i);
      if (kl >= kn) continue;
#pragma unroll
      for (int m = 0; m < kSkinny; ++m)
        if (m < M) {
          const float a = As[kl * kSkinny + m];  // the same word in every lane
          acc[0][m] += a * b[i].x;
          acc[1][m] += a * b[i].y;
          acc[2][m] += a * b[i].z;
          acc[3][m] += a * b[i].w;
        }
    }
  }
#pragma unroll
  for (int m = 0; m < kSkinny; ++m)
    if (m < M) {
#pragma unroll
      for (int j = 0; j < 4; ++j) atomicAdd(&red[(m * 4 + j) * 32 + lane], acc[j][m]);
    }
  __syncthreads();
  float* cbase = static_cast<float*>(P.c) + batch * P.c_batch_stride;
  const long long cfirst = static_cast<long long>(blockIdx.x) * 128;
  const int ncols = P.N - cfirst < 128 ? static_cast<int>(P.N - cfirst) : 128;
  const bool flat = P.ldc == M && (reinterpret_cast<uintptr_t>(cbase + cfirst * P.ldc) & 15u) == 0 &&
                    (ncols * M) % 4 == 0;
  if (flat) {
    // the CTA's part of C is the run [cfirst * m, (cfirst + ncols) * m): element e is row e % m of
    // column e / m
    float* run = cbase + cfirst * P.ldc;
    for (int e4 = threadIdx.x * 4; e4 < ncols * M; e4 += 1024) {
      float v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int e = e4 + i, c = e / M, m = e - c * M;
        v[i] = red[(m * 4 + (c & 3)) * 32 + (c >> 2)];
      }
      atomicAdd(reinterpret_cast<float4*>(run + e4), make_float4(v[0], v[1], v[2], v[3]));
    }
  } else {
    for (int e = threadIdx.x; e < ncols * M; e += 256) {
      const int c = e / M, m = e - c * M;
      atomicAdd(cbase + (cfirst + c) * P.ldc + m, red[(m * 4 + (c & 3)) * 32 + (c >> 2)]);
    }
  }
  if (P.rowsum != nullptr && blockIdx.x == 0 && threadIdx.x < M) {
    float r = 0.f;
    for (int kl = 0; kl < kn; ++kl) r += As[kl * kSkinny + threadIdx.x];
    atomicAdd(static_cast<float*>(P.rowsum) + threadIdx.x, r);
  }
}

// k <= 16, fp32, M a multiple of four, C 16-byte aligned: a thread owns four consecutive rows
// (their rows of A in registers), a CTA 1024 rows and sixteen columns; C is read (for +=) and
// written with 16-byte accesses, eight columns of loads in flight per thread, two CTAs per SM.
constexpr int kSkinnyKS = 16;  // largest contraction of the streaming variant
__global__ void __launch_bounds__(256, 2) skinny_k_stream_kernel(const __grid_constant__ Problem P) {
  __shared__ __align__(16) float Bs[kSkinnyKCols * kSkinnyKS];
  extern __shared__ __align__(16) float Ak_dyn[];  // [1024][K + 1]
  pdl_wait();
  pdl_launch_dependents();
  const long long batch = blockIdx.z;
  const Plain<float> A(P.a[0], batch), Bm(P.b[0], batch);
  const int K = static_cast<int>(P.k[0]);
  const long long row0 = static_cast<long long>(blockIdx.x) * 1024;
  const long long col0 = static_cast<long long>(blockIdx.y) * kSkinnyKCols;
  const int rows = P.M - row0 < 1024 ? static_cast<int>(P.M - row0) : 1024;
  const int cols = P.N - col0 < kSkinnyKCols ? static_cast<int>(P.N - col0) : kSkinnyKCols;
  for (int idx = threadIdx.x; idx < kSkinnyKCols * kSkinnyKS; idx += 256) {
    const int c = idx / kSkinnyKS, kk = idx % kSkinnyKS;
    Bs[idx] = (c < cols && kk < K) ? __ldg(Bm.p + (col0 + c) * Bm.so + kk * Bm.sk) : 0.f;
  }
  // A tile in the order it is stored: (q, r) = (row, k) when the contraction is contiguous, else
  // (k, row)
  const bool k_fast = A.sk == 1;
  auto a_pos = [&](int q, int r) { return k_fast ? q * (K + 1) + r : r * (K + 1) + q; };
  if (k_fast && A.so == K && run_ok(A.p + row0 * K, static_cast<long long>(rows) * K))
    stage_run<10>(Ak_dyn, A.p + row0 * K, rows * K, K, a_pos);  // the rows are one run
  else
    stage_small<16>(
        Ak_dyn, rows * K, k_fast ? K : rows,
        [&](int q, int r) { return A.p + (k_fast ? (row0 + q) * A.so + r
                                                 : (row0 + r) * A.so + static_cast<long long>(q) * A.sk); },
        a_pos);
  __syncthreads();
  const int r4 = threadIdx.x * 4;
  if (r4 >= rows) return;  // M is a multiple of four: the thread's rows exist together
  float a[4][kSkinnyKS];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int kk = 0; kk < kSkinnyKS; ++kk) a[i][kk] = kk < K ? Ak_dyn[(r4 + i) * (K + 1) + kk] : 0.f;
  const long long row = row0 + r4;
  float4 bias = make_float4(0.f, 0.f, 0.f, 0.f);
  if (P.bias) {
    const float* bp = static_cast<const float*>(P.bias) + row;
    bias = make_float4(__ldg(bp), __ldg(bp + 1), __ldg(bp + 2), __ldg(bp + 3));
  }
  float* crow = static_cast<float*>(P.c) + batch * P.c_batch_stride + row;
  for (int c0 = 0; c0 < cols; c0 += 8) {
    float4 x[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      x[j] = (P.accumulate && c0 + j < cols)
                 ? *reinterpret_cast<const float4*>(crow + (col0 + c0 + j) * P.ldc)
                 : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = c0 + j < cols ? c0 + j : 0;
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
      for (int kk = 0; kk < kSkinnyKS; kk += 4) {
        // the same words in every lane (zero beyond K)
        const float4 b = *reinterpret_cast<const float4*>(&Bs[c * kSkinnyKS + kk]);
        s0 = fmaf(a[0][kk + 3], b.w, fmaf(a[0][kk + 2], b.z, fmaf(a[0][kk + 1], b.y, fmaf(a[0][kk], b.x, s0))));
        s1 = fmaf(a[1][kk + 3], b.w, fmaf(a[1][kk + 2], b.z, fmaf(a[1][kk + 1], b.y, fmaf(a[1][kk], b.x, s1))));
        s2 = fmaf(a[2][kk + 3], b.w, fmaf(a[2][kk + 2], b.z, fmaf(a[2][kk + 1], b.y, fmaf(a[2][kk], b.x, s2))));
        s3 = fmaf(a[3][kk + 3], b.w, fmaf(a[3][kk + 2], b.z, fmaf(a[3][kk + 1], b.y, fmaf(a[3][kk], b.x, s3))));
      }
      x[j].x = act_forward<float>(P.act, x[j].x + s0 + bias.x);
      x[j].y = act_forward<float>(P.act, x[j].y + s1 + bias.y);
      x[j].z = act_forward<float>(P.act, x[j].z + s2 + bias.z);
      x[j].w = act_forward<float>(P.act, x[j].w + s3 + bias.w);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (c0 + j < cols) *reinterpret_cast<float4*>(crow + (col0 + c0 + j) * P.ldc) = x[j];
  }
}

__device__ __forceinline__ void atomic_add_t(float* p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add_t(__half* p, float v) { atomicAdd(p, __float2half_rn(v)); }

// rowsum[o] += sum_n dY[o,n] * act'(Y[o,n]).  Threads of a block cover 32 consecutive rows
// (coalesced along a column) and blockDim.y slices of the block's range of columns (blockIdx.y);
// the slices meet in shared memory, the blocks in an atomic add.
template <typename T>
__global__ void rowsum_kernel(const T* __restrict__ dy, const T* __restrict__ y, int dact,
                              long long ld, int M, long long N, T* __restrict__ rowsum) {
  __shared__ float part[8][33];
  const int row = blockIdx.x * 32 + threadIdx.x;
  const long long per = (N + gridDim.y - 1) / gridDim.y;
  const long long n0 = blockIdx.y * per;
  const long long n1 = n0 + per < N ? n0 + per : N;
  float acc = 0.f;
  if (row < M) {
#pragma unroll 4
    for (long long n = n0 + threadIdx.y; n < n1; n += blockDim.y) {
      float v = ld_f(dy + n * ld + row);
      if (dact != ACT_NONE) v = round_to<T>(act_backward<T>(dact, ld_f(y + n * ld + row), v));
      acc += v;
    }
  }
  part[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && row < M) {
    float s = 0.f;
    for (int j = 0; j < blockDim.y; ++j) s += part[j][threadIdx.x];
    atomic_add_t(rowsum + row, s);
  }
}

// The same sum at memory speed for aligned matrices: a thread owns V = 16 / sizeof(T) consecutive
// rows (one 16-byte load per column), 16 such threads cover 16 V rows of a column and 16 slices
// share the block's range of columns; the slices meet in shared memory, the blocks in an atomic
// add.  (The scalar kernel above reads 64 bytes per warp and load: 160 GB/s on a 1024 x 4096 Half
// matrix, 49 us of a 110 us layer step.)  Requires ld, M multiples of V and 16-byte aligned bases.
// With `partials` set the block writes its fp32 sums to partials[blockIdx.y][row] instead of
// adding them to `rowsum`: atomics from many blocks onto the few cache lines of a short vector
// serialise (16 k fp16 atomics onto the 16 lines of a 1024-row bias gradient took 20 us; the sums
// themselves take 3), so large fp16 bias gradients are finished by rowsum_finish_kernel.
template <typename T>
__global__ void __launch_bounds__(256)
rowsum_vec_kernel(const T* __restrict__ dy, const T* __restrict__ y, int dact, long long ld, int M,
                  long long N, T* __restrict__ rowsum, float* __restrict__ partials) {
  constexpr int V = 16 / sizeof(T);
  __shared__ float part[16][16 * V + 1];
  pdl_wait();
  pdl_launch_dependents();
  const int row = (blockIdx.x * 16 + threadIdx.x) * V;
  const long long per = (N + gridDim.y - 1) / gridDim.y;
  const long long n0 = blockIdx.y * per;
  const long long n1 = n0 + per < N ? n0 + per : N;
  float acc[V];
#pragma unroll
  for (int e = 0; e < V; ++e) acc[e] = 0.f;
  if (row < M) {
#pragma unroll 4
    for (long long n = n0 + threadIdx.y; n < n1; n += 16) {
      const uint4 dv = __ldg(reinterpret_cast<const uint4*>(dy + n * ld + row));
      const T* d = reinterpret_cast<const T*>(&dv);
      if (dact != ACT_NONE) {
        const uint4 yv = __ldg(reinterpret_cast<const uint4*>(y + n * ld + row));
        const T* yy = reinterpret_cast<const T*>(&yv);
#pragma unroll
        for (int e = 0; e < V; ++e)
          acc[e] += round_to<T>(act_backward<T>(dact, to_f(yy[e]), to_f(d[e])));
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] += to_f(d[e]);
      }
    }
  }
#pragma unroll
  for (int e = 0; e < V; ++e) part[threadIdx.y][threadIdx.x * V + e] = acc[e];
  __syncthreads();
  // 256 threads, 16 V rows: thread t sums row t (and t + 256 ... when V > 16) over the slices
  for (int r = threadIdx.y * 16 + threadIdx.x; r < 16 * V; r += 256) {
    const int grow = blockIdx.x * 16 * V + r;
    if (grow >= M) continue;
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) sum += part[j][r];
    if (partials != nullptr)
      partials[static_cast<long long>(blockIdx.y) * M + grow] = sum;
    else
      atomic_add_t(rowsum + grow, sum);
  }
}

// rowsum[row] += sum over `parts` fp32 partial vectors of length M stored back to back.
template <typename T>
__global__ void __launch_bounds__(256)
rowsum_finish_kernel(const float* __restrict__ partials, int parts, int M, T* __restrict__ rowsum) {
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  float sum = 0.f;
  for (int q = 0; q < parts; ++q) sum += partials[static_cast<long long>(q) * M + row];
  rowsum[row] = from_f<T>(to_f(rowsum[row]) + sum);
}

// Self test of the bounded-wait machinery: one thread waits on an mbarrier on which nothing ever
// arrives, with a short limit, and must come back with DEV_TIMEOUT_SELFTEST in the status word.
// Nothing faults and nothing hangs: the wait simply runs out.
__global__ void wait_selftest_kernel(int* status, long long limit_cycles, int* returned) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
    const bool ok = mbar_wait(smem_u32(&bar), 0, status, DEV_TIMEOUT_SELFTEST, 0x5e1f, limit_cycles);
    *returned = ok ? 1 : 2;
    mbar_inval(smem_u32(&bar));
  }
}

}  // namespace

cudaError_t launch_wait_selftest(int* status, long long limit_cycles, int* returned,
                                 cudaStream_t stream) {
  wait_selftest_kernel<<<1, 32, 0, stream>>>(status, limit_cycles, returned);
  return cudaGetLastError();
}

cudaError_t set_smem_limit_once(const void* kern, int bytes, unsigned long long* done) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const unsigned long long bit = dev >= 0 && dev < 64 ? 1ull << dev : 0ull;
  // a plain read-modify-write: at worst two threads both set the attribute, which is harmless
  if (bit != 0 && (__atomic_load_n(done, __ATOMIC_RELAXED) & bit)) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && bit != 0) __atomic_fetch_or(done, bit, __ATOMIC_RELAXED);
  return e;
}

cudaError_t launch_small(int dtype, const Problem& p, cudaStream_t stream) {
  const long long total = static_cast<long long>(p.M) * p.N * p.batches;
  if (total <= 0) return cudaSuccess;
  const int threads = 128;  // 4 warps = 4 outputs per block
  const long long blocks = (total + 3) / 4;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
  if (dtype == 0)
    small_gemm_kernel<float><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(p);
  else
    small_gemm_kernel<__half><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(p);
  return cudaGetLastError();
}

// 0: not a skinny problem (or a form the skinny kernels do not take); otherwise the mapping.
int skinny_kind(int dtype, const Problem& p) {
  if (p.rowsum != nullptr) return 0;  // the caller decides how the bias gradient is formed
  long long ktot = 0;
  for (int i = 0; i < p.npairs; ++i) ktot += p.k[i];
  if (ktot <= 0 || p.M <= 0 || p.N <= 0) return 0;
  if (p.M <= kSkinny) {
    bool b_kc = true;
    for (int i = 0; i < p.npairs; ++i) b_kc = b_kc && p.b[i].k_contig;
    if (b_kc) return 1;
    if (dtype == 0 && p.accumulate && p.act == ACT_NONE && p.bias == nullptr && ktot >= 512 &&
        ktot <= 2000000 && p.batches <= 65535)
      return 2;
  }
  if (ktot <= 32 && static_cast<long long>(p.M) * p.N >= 4096) return 3;
  return 0;
}

cudaError_t launch_skinny(int dtype, int kind, const Problem& p, cudaStream_t stream) {
  bool plain = p.npairs == 1 && p.ccols == nullptr;
  for (int i = 0; i < p.npairs; ++i)
    plain = plain && p.a[i].cols == nullptr && p.b[i].cols == nullptr &&
            p.a[i].dact == ACT_NONE && p.b[i].dact == ACT_NONE;
  if (kind == 1) {
    const long long warps = static_cast<long long>(p.N) * p.batches;
    const long long blocks = (warps + 7) / 8;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
    const unsigned g = static_cast<unsigned>(blocks);
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    const long long kpad = (p.k[0] + 3) / 4 * 4;
    const long long a_bytes = static_cast<long long>(p.M) * kpad * 4;
    if (plain && dtype == 0 && p.batches <= 65535 && a_bytes <= 64 * 1024 && p.N >= 256 &&
        al16(p.b[0].base) && p.b[0].ld % 4 == 0 && p.b[0].batch_stride % 4 == 0) {
      dim3 grid(static_cast<unsigned>((p.N + 15) / 16), static_cast<unsigned>(p.batches));
      static unsigned long long set_f = 0;
      cudaError_t e = set_smem_limit_once(reinterpret_cast<const void*>(skinny_m_stream_kernel),
                                          64 * 1024, &set_f);
      if (e != cudaSuccess) return e;
      return launch_kernel(skinny_m_stream_kernel, grid, dim3(256), static_cast<size_t>(a_bytes),
                           stream, pdl_enabled(), p, static_cast<int>(kpad));
    }
    if (plain && p.batches <= 65535) {
      dim3 grid(static_cast<unsigned>((p.N + 15) / 16), static_cast<unsigned>(p.batches));
      if (dtype == 0) skinny_m_plain_kernel<float><<<grid, 256, 0, stream>>>(p);
      else skinny_m_plain_kernel<__half><<<grid, 256, 0, stream>>>(p);
    } else if (dtype == 0) {
      skinny_m_kernel<float><<<g, 256, 0, stream>>>(p);
    } else {
      skinny_m_kernel<__half><<<g, 256, 0, stream>>>(p);
    }
  } else if (kind == 2) {
    const int chunk = plain ? kSkinnyMtChunk : 128;
    long long chunks = 0;
    for (int i = 0; i < p.npairs; ++i) chunks += (p.k[i] + chunk - 1) / chunk;
    if (chunks > 65535) return cudaErrorInvalidValue;
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    if (plain && !p.b[0].k_contig && p.N % 4 == 0 && p.N >= 128 && al16(p.b[0].base) &&
        p.b[0].ld % 4 == 0 && p.b[0].batch_stride % 4 == 0 && (p.k[0] + 127) / 128 <= 65535) {
      dim3 grid(static_cast<unsigned>((p.N + 127) / 128), static_cast<unsigned>((p.k[0] + 127) / 128),
                static_cast<unsigned>(p.batches));
      return launch_kernel(skinny_mt_stream_kernel, grid, dim3(256), 0, stream, pdl_enabled(), p);
    }
    if (plain) {
      dim3 grid(static_cast<unsigned>((p.N + 31) / 32), static_cast<unsigned>(chunks),
                static_cast<unsigned>(p.batches));
      skinny_mt_plain_kernel<<<grid, dim3(32, 8), 0, stream>>>(p);
    } else {
      dim3 grid(static_cast<unsigned>((p.N + 127) / 128), static_cast<unsigned>(chunks),
                static_cast<unsigned>(p.batches));
      skinny_mt_kernel<<<grid, 128, 0, stream>>>(p);
    }
  } else if (plain && dtype == 0 && p.batches <= 65535 && p.M % 4 == 0 && p.M >= 1024 &&
             p.k[0] <= kSkinnyKS &&
             p.ldc % 4 == 0 && p.c_batch_stride % 4 == 0 &&
             (reinterpret_cast<uintptr_t>(p.c) & 15u) == 0 &&
             (p.bias == nullptr || (reinterpret_cast<uintptr_t>(p.bias) & 3u) == 0) &&
             (p.N + kSkinnyKCols - 1) / kSkinnyKCols <= 65535) {
    dim3 grid(static_cast<unsigned>((p.M + 1023) / 1024),
              static_cast<unsigned>((p.N + kSkinnyKCols - 1) / kSkinnyKCols),
              static_cast<unsigned>(p.batches));
    const size_t smem = 1024 * (static_cast<size_t>(p.k[0]) + 1) * 4;  // at most 68 KiB
    static unsigned long long set16 = 0;
    cudaError_t e = set_smem_limit_once(reinterpret_cast<const void*>(skinny_k_stream_kernel),
                                        1024 * 17 * 4, &set16);
    if (e != cudaSuccess) return e;
    return launch_kernel(skinny_k_stream_kernel, grid, dim3(256), smem, stream, pdl_enabled(), p);
  } else if (plain && p.batches <= 65535 && (p.N + kSkinnyKCols - 1) / kSkinnyKCols <= 65535) {
    dim3 grid(static_cast<unsigned>((p.M + 255) / 256),
              static_cast<unsigned>((p.N + kSkinnyKCols - 1) / kSkinnyKCols),
              static_cast<unsigned>(p.batches));
    const bool k16 = p.k[0] <= 16;
    if (dtype == 0) {
      if (k16) skinny_k_plain_kernel<float, 16><<<grid, 256, 0, stream>>>(p);
      else skinny_k_plain_kernel<float, 32><<<grid, 256, 0, stream>>>(p);
    } else {
      if (k16) skinny_k_plain_kernel<__half, 16><<<grid, 256, 0, stream>>>(p);
      else skinny_k_plain_kernel<__half, 32><<<grid, 256, 0, stream>>>(p);
    }
  } else {
    const long long total = static_cast<long long>(p.M) * p.N * p.batches;
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
    if (dtype == 0) skinny_k_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
    else skinny_k_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
  }
  return cudaGetLastError();
}

// fp16 bias gradient of an aligned matrix in two launches and no atomics: fp32 partial sums of
// `rowsum_ws_parts(M, N)` column chunks into `ws` (that many vectors of M floats), then one pass
// that adds their sum to rowsum.  Returns cudaErrorInvalidValue when the shape does not qualify
// (the caller then uses launch_rowsum).
int rowsum_ws_parts(int M, long long N) {
  if (M % 8 != 0 || N < 1024) return 0;
  long long chunks = N / 64;
  return static_cast<int>(chunks > 64 ? 64 : chunks);
}
cudaError_t launch_rowsum_half_ws(const void* dy, long long ld, int M, long long N, void* rowsum,
                                  float* ws, cudaStream_t stream) {
  const int parts = rowsum_ws_parts(M, N);
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  if (parts == 0 || ld % 8 != 0 || !al(dy)) return cudaErrorInvalidValue;
  dim3 grid((M + 127) / 128, static_cast<unsigned>(parts)), block(16, 16);
  cudaError_t e = launch_kernel(rowsum_vec_kernel<__half>, grid, block, 0, stream, pdl_enabled(),
                                static_cast<const __half*>(dy), static_cast<const __half*>(nullptr),
                                static_cast<int>(ACT_NONE), ld, M, N, static_cast<__half*>(rowsum), ws);
  if (e != cudaSuccess) return e;
  return launch_kernel(rowsum_finish_kernel<__half>, dim3((M + 255) / 256), dim3(256), 0, stream,
                       pdl_enabled(), static_cast<const float*>(ws), parts, M,
                       static_cast<__half*>(rowsum));
}

cudaError_t launch_rowsum(int dtype, const void* dy, const void* y, int dact, long long ld, int M,
                          long long N, void* rowsum, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return cudaSuccess;
  {
    const int esize = dtype == 0 ? 4 : 2, V = 16 / esize;
    auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    if (M % V == 0 && ld % V == 0 && al(dy) && (dact == ACT_NONE || al(y)) && N >= 64) {
      const int row_blocks = (M + 16 * V - 1) / (16 * V);
      long long chunks = 592 / row_blocks;  // about four blocks of 256 threads per SM
      if (chunks > (N + 63) / 64) chunks = (N + 63) / 64;
      // every block adds its part to the fp16 sum with one more rounding: keep them few
      if (dtype != 0 && chunks > 16) chunks = 16;
      if (chunks < 1) chunks = 1;
      dim3 vgrid(row_blocks, static_cast<unsigned>(chunks)), vblock(16, 16);
      if (dtype == 0)
        return launch_kernel(rowsum_vec_kernel<float>, vgrid, vblock, 0, stream, pdl_enabled(),
                             static_cast<const float*>(dy), static_cast<const float*>(y), dact, ld,
                             M, N, static_cast<float*>(rowsum), static_cast<float*>(nullptr));
      return launch_kernel(rowsum_vec_kernel<__half>, vgrid, vblock, 0, stream, pdl_enabled(),
                           static_cast<const __half*>(dy), static_cast<const __half*>(y), dact, ld, M,
                           N, static_cast<__half*>(rowsum), static_cast<float*>(nullptr));
    }
  }
  dim3 block(32, 8);
  // enough blocks along the columns to fill the GPU when there are few rows (at least 64
  // columns per block)
  long long chunks = 1184 / ((M + 31) / 32);
  if (chunks > (N + 63) / 64) chunks = (N + 63) / 64;
  if (chunks < 1) chunks = 1;
  if (chunks > 65535) chunks = 65535;
  dim3 grid((M + 31) / 32, static_cast<unsigned>(chunks));
  if (dtype == 0)
    rowsum_kernel<float><<<grid, block, 0, stream>>>(static_cast<const float*>(dy),
                                                     static_cast<const float*>(y), dact, ld, M, N,
                                                     static_cast<float*>(rowsum));
  else
    rowsum_kernel<__half><<<grid, block, 0, stream>>>(static_cast<const __half*>(dy),
                                                      static_cast<const __half*>(y), dact, ld, M,
                                                      N, static_cast<__half*>(rowsum));
  return cudaGetLastError();
}

}  // namespace gb
