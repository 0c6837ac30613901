// CUDA-core kernels for the shapes the tensor-core tiles do not fit:
//   * products with a tiny result (m*n of a few elements), e.g. the batched 1x1 dot products
//     that SoftmaxOp::backward and LayerNormNode::backward send through gpu_batched_prod
//     (ginn/nonlin.h:180-183, ginn/node/layernorm.h:61-64), and k == 0;
//   * the bias gradient alone (row sums of dY (.) act'(Y)) when no weight gradient is wanted.
// fp32 accumulation, one warp per output element, lanes strided along the contraction.
#include <cuda_fp16.h>
#include "ptx.cuh"
#include "math.cuh"
#include "launch.h"

namespace gb {

namespace {

__device__ __forceinline__ float ld_f(const float* p) { return __ldg(p); }
__device__ __forceinline__ float ld_f(const __half* p) { return __half2float(__ldg(p)); }
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

// One warp per row: rowsum[o] += sum_n dY[o,n] * act'(Y[o,n]).
template <typename T>
__global__ void rowsum_kernel(const T* __restrict__ dy, const T* __restrict__ y, int dact,
                              long long ld, int M, long long N, T* __restrict__ rowsum) {
  // Threads of a block cover 32 consecutive rows (coalesced along the column) and
  // blockDim.y slices of the columns; partial sums meet in shared memory.
  __shared__ float part[8][33];
  const int row = blockIdx.x * 32 + threadIdx.x;
  float acc = 0.f;
  if (row < M) {
    for (long long n = threadIdx.y; n < N; n += blockDim.y) {
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
    st_f(rowsum + row, ld_rw(rowsum + row) + s);
  }
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

cudaError_t launch_rowsum(int dtype, const void* dy, const void* y, int dact, long long ld, int M,
                          long long N, void* rowsum, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return cudaSuccess;
  dim3 block(32, 8);
  dim3 grid((M + 31) / 32);
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
