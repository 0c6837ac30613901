// The elementwise neighbours of the GEMMs on a training step: the picked negative log softmax
// loss (forward and backward) and the Adam update.  All three are bound by HBM bandwidth; each
// is one pass over its operands.
//
//   pick_nll_forward : per column j of X (rows x cols, column-major)
//                        smax[:, j] = softmax(X[:, j]),  value[j] = -log(smax[index[j], j])
//                      (SoftmaxOp::forward, ginn/nonlin.h:162-168: subtract the column maximum,
//                      exponentiate, divide by the column sum; the pick of ginn/node/pick.h:60-84;
//                      the -log of PickNegLogSoftmaxNode::forward_, pick.h:209-216)
//   pick_nll_backward: dX[i, j] += (smax[i, j] - [i == index[j]]) * g[j]
//                      (PickNegLogSoftmaxNode::backward_, pick.h:218-224, and pick_grad with
//                      negate, pick.h:87-131, in one pass instead of gather + scatter + add)
//   softmax_forward  : the same kernel without the pick (SoftmaxOp::forward alone)
//   softmax_backward : dX (+)= Y (.) (dY - colsum(Y (.) dY))   (SoftmaxOp::backward,
//                      ginn/nonlin.h:169-190: a batched 1 x 1 product plus a broadcast expression)
//   adam_update      : d = clip(d); m = b1 m + (1 - b1) d; v = b2 v + (1 - b2) d^2;
//                      w += -lr / (1 - b1^t) * m / (eps + sqrt(v / (1 - b2^t)))
//                      (Adam::update, ginn/update/update.h:115-133; m and v are always fp32)
#include <cuda_fp16.h>
#include "math.cuh"
#include "ptx.cuh"
#include "launch.h"

namespace gb {

namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Four consecutive elements of storage type T as floats.
__device__ __forceinline__ void load4(const float* p, float (&x)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
}
__device__ __forceinline__ void load4(const __half* p, float (&x)[4]) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
  x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, const float (&x)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
}
__device__ __forceinline__ void store4(__half* p, const float (&x)[4]) {
  uint2 v;
  *reinterpret_cast<__half2*>(&v.x) = __floats2half2_rn(x[0], x[1]);
  *reinterpret_cast<__half2*>(&v.y) = __floats2half2_rn(x[2], x[3]);
  *reinterpret_cast<uint2*>(p) = v;
}

// One group of G threads (G = 32: a warp, G = blockDim.x: the whole CTA) per column.  Lanes run
// along the column, which is contiguous in memory.
template <typename T, bool BLOCK, bool VEC>
__global__ void __launch_bounds__(256)
pick_nll_forward_kernel(const T* __restrict__ x, long long ldx, const int* __restrict__ index,
                        T* __restrict__ smax, long long lds, T* __restrict__ value, int rows,
                        long long cols) {
  __shared__ float red[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = BLOCK ? blockDim.x : 32;
  const int g = BLOCK ? threadIdx.x : lane;
  const long long j = BLOCK ? blockIdx.x : static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp;
  if (j >= cols) return;  // BLOCK: uniform per CTA; warp mode: uniform per warp (no CTA barrier used)
  const T* xc = x + j * ldx;
  T* sc = smax + j * lds;

  auto reduce = [&](float v, bool is_max) -> float {
    v = is_max ? warp_max(v) : warp_sum(v);
    if (!BLOCK) return v;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < (blockDim.x >> 5); ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
  };

  // VEC: columns start on 16-byte (fp16: 8-byte) boundaries; four elements per lane and pass,
  // the last rows % 4 by the scalar tail.
  const int rows4 = VEC ? rows / 4 : 0;
  float m = -INFINITY;
  for (int q = g; q < rows4; q += G) {
    float v[4];
    load4(xc + 4 * q, v);
    m = fmaxf(fmaxf(m, fmaxf(v[0], v[1])), fmaxf(v[2], v[3]));
  }
  for (int i = 4 * rows4 + g; i < rows; i += G) m = fmaxf(m, to_f(xc[i]));
  m = reduce(m, true);
  float s = 0.f;
  for (int q = g; q < rows4; q += G) {
    float v[4];
    load4(xc + 4 * q, v);
    s += (expf(v[0] - m) + expf(v[1] - m)) + (expf(v[2] - m) + expf(v[3] - m));
  }
  for (int i = 4 * rows4 + g; i < rows; i += G) s += expf(to_f(xc[i]) - m);
  s = reduce(s, false);
  const float inv = 1.f / s;
  for (int q = g; q < rows4; q += G) {
    float v[4];
    load4(xc + 4 * q, v);
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = expf(v[e] - m) * inv;
    store4(sc + 4 * q, v);
  }
  for (int i = 4 * rows4 + g; i < rows; i += G) sc[i] = from_f<T>(expf(to_f(xc[i]) - m) * inv);
  if (g == 0 && index != nullptr) {  // plain softmax: no pick
    const int p = index[j];
    // the reference takes the log of the stored (rounded) probability
    const float picked = (p >= 0 && p < rows) ? to_f(from_f<T>(expf(to_f(xc[p]) - m) * inv)) : 0.f;
    value[j] = from_f<T>(-logf(picked));
  }
}

// Softmax backward (SoftmaxOp::backward, ginn/nonlin.h:169-190): per column
//   m = sum_i y_i dy_i,   dx_i (+)= y_i (dy_i - m)
// in one kernel: the reference forms m with a batched 1 x 1 product and then runs a broadcast
// expression.  One warp per column (one CTA above 2048 rows); the column is read twice, the
// second time from cache.
template <typename T, bool BLOCK, bool VEC>
__global__ void __launch_bounds__(256)
softmax_backward_kernel(const T* __restrict__ y, long long ldy, const T* __restrict__ dy,
                        long long lddy, T* __restrict__ dx, long long lddx, int rows,
                        long long cols, int accumulate) {
  __shared__ float red[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = BLOCK ? blockDim.x : 32;
  const int g = BLOCK ? threadIdx.x : lane;
  const long long j = BLOCK ? blockIdx.x : static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp;
  if (j >= cols) return;
  const T* yc = y + j * ldy;
  const T* dc = dy + j * lddy;
  T* xc = dx + j * lddx;
  const int rows4 = VEC ? rows / 4 : 0;
  float m = 0.f;
  for (int q = g; q < rows4; q += G) {
    float a[4], b[4];
    load4(yc + 4 * q, a);
    load4(dc + 4 * q, b);
    m += (a[0] * b[0] + a[1] * b[1]) + (a[2] * b[2] + a[3] * b[3]);
  }
  for (int i = 4 * rows4 + g; i < rows; i += G) m += to_f(yc[i]) * to_f(dc[i]);
  m = warp_sum(m);
  if (BLOCK) {
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) m += red[w];
  }
  m = to_f(from_f<T>(m));  // the reference keeps m in a tensor of the storage type
  for (int q = g; q < rows4; q += G) {
    float a[4], b[4], o[4] = {0.f, 0.f, 0.f, 0.f};
    load4(yc + 4 * q, a);
    load4(dc + 4 * q, b);
    if (accumulate) load4(xc + 4 * q, o);
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] += a[e] * (b[e] - m);
    store4(xc + 4 * q, o);
  }
  for (int i = 4 * rows4 + g; i < rows; i += G) {
    const float v = to_f(yc[i]) * (to_f(dc[i]) - m);
    xc[i] = from_f<T>(accumulate ? to_f(xc[i]) + v : v);
  }
}

// One warp per column (eight columns per CTA), lanes along the column; no index arithmetic per
// element.  VEC as above.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
pick_nll_backward_kernel(const T* __restrict__ smax, long long lds, const int* __restrict__ index,
                         const T* __restrict__ grad, T* __restrict__ dx, long long lddx, int rows,
                         long long cols) {
  const int lane = threadIdx.x & 31;
  const long long j = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (j >= cols) return;
  const float g = to_f(grad[j]);
  const int pick = index[j];
  const T* sc = smax + j * lds;
  T* dc = dx + j * lddx;
  // two rounded steps, as the reference's two statements are: dX -= g at the pick, dX += y * g
  auto one = [&](int i, float d, float y) {
    if (i == pick) d = to_f(from_f<T>(d - g));
    return to_f(from_f<T>(d + to_f(from_f<T>(y * g))));
  };
  const int rows4 = VEC ? rows / 4 : 0;
  for (int q = lane; q < rows4; q += 32) {
    float y[4], d[4];
    load4(sc + 4 * q, y);
    load4(dc + 4 * q, d);
#pragma unroll
    for (int e = 0; e < 4; ++e) d[e] = one(4 * q + e, d[e], y[e]);
    store4(dc + 4 * q, d);
  }
  for (int i = 4 * rows4 + lane; i < rows; i += 32) dc[i] = from_f<T>(one(i, to_f(dc[i]), to_f(sc[i])));
}

// dA = dY (.) act'(Y) in fp16, every operation rounded to fp16 as the reference's Half expressions
// are (ginn/nonlin.h:96-106 tanh, :119-126 relu, :146-152 sigmoid): the tensor AffineNode::backward_
// calls dpreactiv_ (ginn/node/affine.h:82-88), materialised once so that both gradient products
// can run on the TMA-fed kernels.  dA is m x n with leading dimension m.
__device__ __forceinline__ __half2 dact_h2(int act, __half2 y, __half2 d) {
  const __half2 one = __float2half2_rn(1.f), zero = __float2half2_rn(0.f);
  if (act == ACT_TANH) return __hsub2(d, __hmul2(__hmul2(y, y), d));
  if (act == ACT_SIGMOID) return __hmul2(__hmul2(y, __hsub2(one, y)), d);
  if (act == ACT_RELU) return __hmul2(__hgt2(y, zero), d);
  return d;
}

template <bool VEC>
__global__ void __launch_bounds__(256)
dact_half_kernel(const __half* __restrict__ dy, long long lddy, const __half* __restrict__ y,
                 long long ldy, int act, __half* __restrict__ da, int m, long long n) {
  pdl_wait();
  pdl_launch_dependents();
  const long long col = blockIdx.y;
  const int per = VEC ? 8 : 1;
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) * per;
  if (r >= m || col >= n) return;
  const __half* dp = dy + col * lddy + r;
  const __half* yp = y + col * ldy + r;
  __half* op = da + col * static_cast<long long>(m) + r;
  if (VEC) {
    uint4 dv = *reinterpret_cast<const uint4*>(dp);
    const uint4 yv = *reinterpret_cast<const uint4*>(yp);
    __half2* d2 = reinterpret_cast<__half2*>(&dv);
    const __half2* y2 = reinterpret_cast<const __half2*>(&yv);
#pragma unroll
    for (int e = 0; e < 4; ++e) d2[e] = dact_h2(act, y2[e], d2[e]);
    *reinterpret_cast<uint4*>(op) = dv;
  } else {
    const __half2 v = dact_h2(act, __half2half2(*yp), __half2half2(*dp));
    *op = __low2half(v);
  }
}

// C (m x n, leading dimension ldc) += sum over `parts` dense m x n fp16 matrices stored back to
// back: the partial products of a contraction split into chunks.  Summed in fp32, rounded once.
template <bool VEC>
__global__ void __launch_bounds__(256)
add_partials_half_kernel(__half* __restrict__ c, long long ldc, const __half* __restrict__ ws,
                         int parts, int m, long long n) {
  pdl_wait();
  pdl_launch_dependents();
  const long long col = blockIdx.y;
  const int per = VEC ? 8 : 1;
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) * per;
  if (r >= m || col >= n) return;
  __half* cp = c + col * ldc + r;
  const __half* wp = ws + col * static_cast<long long>(m) + r;
  const long long part_stride = static_cast<long long>(m) * n;
  if (VEC) {
    uint4 cv = *reinterpret_cast<const uint4*>(cp);
    __half2* c2 = reinterpret_cast<__half2*>(&cv);
    float2 acc[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[e] = __half22float2(c2[e]);
    for (int q = 0; q < parts; ++q) {
      const uint4 wv = *reinterpret_cast<const uint4*>(wp + q * part_stride);
      const __half2* w2 = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 w = __half22float2(w2[e]);
        acc[e].x += w.x;
        acc[e].y += w.y;
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) c2[e] = __floats2half2_rn(acc[e].x, acc[e].y);
    *reinterpret_cast<uint4*>(cp) = cv;
  } else {
    float acc = __half2float(*cp);
    for (int q = 0; q < parts; ++q) acc += __half2float(wp[q * part_stride]);
    *cp = __float2half_rn(acc);
  }
}

// Y = act(Y + bias) in place, fp16 (bias per row, broadcast over columns): the epilogue of a large
// Half Affine whose product ran on a TMA-fed kernel that has no fused epilogue of its own.
template <bool VEC>
__global__ void __launch_bounds__(256)
bias_act_half_kernel(__half* __restrict__ y, long long ldy, const __half* __restrict__ bias, int act,
                     int m, long long n) {
  pdl_wait();
  pdl_launch_dependents();
  const long long col = blockIdx.y;
  const int per = VEC ? 8 : 1;
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) * per;
  if (r >= m || col >= n) return;
  __half* yp = y + col * ldy + r;
  if (VEC) {
    uint4 v = *reinterpret_cast<const uint4*>(yp);
    uint4 bv = make_uint4(0, 0, 0, 0);
    if (bias) bv = *reinterpret_cast<const uint4*>(bias + r);
    __half2* v2 = reinterpret_cast<__half2*>(&v);
    const __half2* b2 = reinterpret_cast<const __half2*>(&bv);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = __half22float2(v2[e]), b = __half22float2(b2[e]);
      v2[e] = __floats2half2_rn(act_forward_half(act, x.x + b.x), act_forward_half(act, x.y + b.y));
    }
    *reinterpret_cast<uint4*>(yp) = v;
  } else {
    const float b = bias ? __half2float(bias[r]) : 0.f;
    *yp = __float2half_rn(act_forward_half(act, __half2float(*yp) + b));
  }
}

__device__ __forceinline__ float sigmoid_f(float x) { return 0.5f * tanhf(0.5f * x) + 0.5f; }

// The same cell update for cells that each live in tensors of their own (one column per graph
// node, as ginn allocates them): `tab` holds tables of `n` device pointers each, one entry per
// cell.  forward tables: gates (4H, overwritten with the activations), c_prev (H; entry may be
// null), c (H), h (H).  backward tables: gates, c, c_prev (may be null), dh (H: gradient of h),
// dc (H: gradient of c gathered from the next step), dgates (4H, +=), dc_prev (H, +=; null
// where c_prev is).  Gradients accumulate, as every gradient write in ginn does.
__global__ void __launch_bounds__(256)
lstm_cells_forward_kernel(const void* const* __restrict__ tab, int H, long long n) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  const long long col = blockIdx.y;
  if (r >= H || col >= n) return;
  float* g = static_cast<float*>(const_cast<void*>(tab[col])) + r;
  const float* cprev = static_cast<const float*>(tab[n + col]);
  float* c = static_cast<float*>(const_cast<void*>(tab[2 * n + col]));
  float* h = static_cast<float*>(const_cast<void*>(tab[3 * n + col]));
  const long long Hl = H;
  const float i = sigmoid_f(g[0]), f = sigmoid_f(g[Hl]), gg = tanhf(g[2 * Hl]), o = sigmoid_f(g[3 * Hl]);
  g[0] = i;
  g[Hl] = f;
  g[2 * Hl] = gg;
  g[3 * Hl] = o;
  const float cv = f * (cprev ? cprev[r] : 0.f) + i * gg;
  c[r] = cv;
  h[r] = o * tanhf(cv);
}

__global__ void __launch_bounds__(256)
lstm_cells_backward_kernel(const void* const* __restrict__ tab, int H, long long n) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  const long long col = blockIdx.y;
  if (r >= H || col >= n) return;
  const float* g = static_cast<const float*>(tab[col]) + r;
  const float* c = static_cast<const float*>(tab[n + col]);
  const float* cprev = static_cast<const float*>(tab[2 * n + col]);
  const float* dhp = static_cast<const float*>(tab[3 * n + col]);
  const float* dcp = static_cast<const float*>(tab[4 * n + col]);
  float* dg = static_cast<float*>(const_cast<void*>(tab[5 * n + col])) + r;
  float* dcprev = static_cast<float*>(const_cast<void*>(tab[6 * n + col]));
  const long long Hl = H;
  const float i = g[0], f = g[Hl], gg = g[2 * Hl], o = g[3 * Hl];
  const float tc = tanhf(c[r]);
  const float cp = cprev ? cprev[r] : 0.f;
  const float dh = dhp[r];
  const float dc = dcp[r] + dh * o * (1.f - tc * tc);
  dg[0] += dc * gg * i * (1.f - i);
  dg[Hl] += dc * cp * f * (1.f - f);
  dg[2 * Hl] += dc * i * (1.f - gg * gg);
  dg[3 * Hl] += dh * tc * o * (1.f - o);
  if (dcprev) dcprev[r] += dc * f;
}

// x[i] = value for n elements (what Tensor::fill / setConstant do on the device).
template <typename T>
__global__ void __launch_bounds__(256) fill_kernel(T* __restrict__ x, long long n, float value) {
  const T v = from_f<T>(value);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    x[i] = v;
}

// S = scale * S in place over a strided batch of T x T score matrices (row = key position,
// column = query position); with `causal`, keys after the query (row > column) become -inf, as
// min-GPT's InPlaceMask does before the softmax (examples/min-gpt.cu.cpp:133-137).
__global__ void __launch_bounds__(256)
scale_mask_f32_kernel(float* __restrict__ s, long long ld, long long stride, int T, float scale,
                      int causal) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  const int col = blockIdx.y;
  if (r >= T) return;
  float* q = s + blockIdx.z * stride + col * ld + r;
  *q = (causal && r > col) ? -INFINITY : *q * scale;
}

// C = act(C) in place, fp32: the activation of a product whose contraction was split over
// several CTAs (their partial sums meet in C, so the nonlinearity cannot ride on any of them).
__global__ void __launch_bounds__(256)
act_inplace_f32_kernel(float* __restrict__ c, long long ldc, long long stride, int act, int m, int n) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= m) return;
  float* p = c + blockIdx.z * stride + r;
  for (int col = blockIdx.y; col < n; col += gridDim.y) {
    float* q = p + col * ldc;
    *q = act_forward<float>(act, *q);
  }
}

// ---- LSTM cell glue of the autobatch benchmark -------------------------------------------
// The gates of one level arrive as one 4H x n matrix (rows i | f | g | o, the order of the
// benchmark's shared gate weight); the cell update the reference composes from CwiseProd, Tanh
// and Add nodes (ginn/model/lstm.h:97-100) is one pass here.  fp32 only.
//   forward : i, f, o = sigmoid, g = tanh (written back over the pre-activations, the backward
//             pass needs them), c = f c_prev + i g, h = o tanh(c); h of the columns that live on
//             is also copied into the next level's input block.
//   backward: dh = upstream (next level's input gradient for columns that live on, `dh_end` for
//             those that end here), dc = dc_next + dh o (1 - tanh(c)^2), the four gate gradients
//             through their nonlinearities, and dc f carried to the previous level.

__global__ void __launch_bounds__(256)
lstm_cell_forward_kernel(float* __restrict__ gates, long long ldg, const float* __restrict__ c_prev,
                         long long ldcp, float* __restrict__ c, long long ldc, float* __restrict__ h,
                         long long ldh, float* __restrict__ xh_next, long long ldx, int H,
                         long long n, long long n_next) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  const long long col = blockIdx.y;
  if (r >= H || col >= n) return;
  float* g = gates + col * ldg + r;
  const float i = sigmoid_f(g[0]), f = sigmoid_f(g[H]), gg = tanhf(g[2 * static_cast<long long>(H)]),
              o = sigmoid_f(g[3 * static_cast<long long>(H)]);
  g[0] = i;
  g[H] = f;
  g[2 * static_cast<long long>(H)] = gg;
  g[3 * static_cast<long long>(H)] = o;
  const float cp = c_prev ? c_prev[col * ldcp + r] : 0.f;
  const float cv = f * cp + i * gg;
  const float hv = o * tanhf(cv);
  c[col * ldc + r] = cv;
  h[col * ldh + r] = hv;
  if (xh_next != nullptr && col < n_next) xh_next[col * ldx + r] = hv;
}

__global__ void __launch_bounds__(256)
lstm_cell_backward_kernel(const float* __restrict__ gates, long long ldg, const float* __restrict__ c,
                          long long ldc, const float* __restrict__ c_prev, long long ldcp,
                          const float* __restrict__ dh_next, long long lddh,
                          const float* __restrict__ dc_next, long long lddc, float dh_end,
                          float* __restrict__ dgates, long long lddg, float* __restrict__ dc_out,
                          long long lddo, int H, long long n, long long n_next) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  const long long col = blockIdx.y;
  if (r >= H || col >= n) return;
  const float* g = gates + col * ldg + r;
  const long long Hl = H;
  const float i = g[0], f = g[Hl], gg = g[2 * Hl], o = g[3 * Hl];
  const float tc = tanhf(c[col * ldc + r]);
  const float cp = c_prev ? c_prev[col * ldcp + r] : 0.f;
  const bool lives = col < n_next;
  const float dh = lives ? dh_next[col * lddh + r] : dh_end;
  const float dc = (lives ? dc_next[col * lddc + r] : 0.f) + dh * o * (1.f - tc * tc);
  float* dg = dgates + col * lddg + r;
  dg[0] = dc * gg * i * (1.f - i);
  dg[Hl] = dc * cp * f * (1.f - f);
  dg[2 * Hl] = dc * i * (1.f - gg * gg);
  dg[3 * Hl] = dh * tc * o * (1.f - o);
  dc_out[col * lddo + r] = dc * f;
}

// One element of the update; returns the new weight and leaves d, m, v updated.
template <typename T>
__device__ __forceinline__ float adam_one(float w, float& d, float& m, float& v, float clip,
                                          float b1, float b2, float step, float vscale, float eps) {
  d = to_f(from_f<T>(fmaxf(fminf(d, clip), -clip)));  // the reference clips the gradient in place
  m = b1 * m + (1.f - b1) * d;
  v = b2 * v + (1.f - b2) * d * d;
  // w += cast<Scalar>( step * m / (eps + sqrt(vscale * v)) ),  step = -lr / (1 - b1^t)
  const float upd = to_f(from_f<T>(step * m / (eps + sqrtf(vscale * v))));
  return to_f(from_f<T>(w + upd));
}

// VEC: all four arrays are 16-byte aligned (8-byte for fp16 w and d); four elements per thread and
// pass, the last n % 4 elements by the scalar tail.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
adam_kernel(T* __restrict__ w, T* __restrict__ d, float* __restrict__ m, float* __restrict__ v,
            long long n, float clip, float b1, float b2, float step, float vscale, float eps) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long n4 = VEC ? n / 4 : 0;
  for (long long q = tid; q < n4; q += stride) {
    float wi[4], di[4], mi[4], vi[4];
    load4(w + 4 * q, wi);
    load4(d + 4 * q, di);
    load4(m + 4 * q, mi);
    load4(v + 4 * q, vi);
#pragma unroll
    for (int e = 0; e < 4; ++e)
      wi[e] = adam_one<T>(wi[e], di[e], mi[e], vi[e], clip, b1, b2, step, vscale, eps);
    store4(w + 4 * q, wi);
    store4(d + 4 * q, di);
    store4(m + 4 * q, mi);
    store4(v + 4 * q, vi);
  }
  for (long long i = 4 * n4 + tid; i < n; i += stride) {
    float di = to_f(d[i]), mi = m[i], vi = v[i];
    const float wn = adam_one<T>(to_f(w[i]), di, mi, vi, clip, b1, b2, step, vscale, eps);
    w[i] = from_f<T>(wn);
    d[i] = from_f<T>(di);
    m[i] = mi;
    v[i] = vi;
  }
}

}  // namespace

namespace {
// Every column of a matrix with leading dimension ld starts on a boundary of `bytes`.
bool cols_aligned(const void* p, long long ld, int esize, unsigned bytes) {
  return (reinterpret_cast<uintptr_t>(p) & (bytes - 1)) == 0 && (ld * esize) % bytes == 0;
}

template <typename T>
void pick_forward_t(const void* x, long long ldx, const int* index, void* smax, long long lds,
                    void* value, int rows, long long cols, cudaStream_t stream) {
  const unsigned a = sizeof(T) * 4;
  const bool vec = cols_aligned(x, ldx, sizeof(T), a) && cols_aligned(smax, lds, sizeof(T), a);
  const bool block = rows > 2048;
  const unsigned grid = block ? static_cast<unsigned>(cols) : static_cast<unsigned>((cols + 7) / 8);
  const T* xp = static_cast<const T*>(x);
  T* sp = static_cast<T*>(smax);
  T* vp = static_cast<T*>(value);
  if (block && vec) pick_nll_forward_kernel<T, true, true><<<grid, 256, 0, stream>>>(xp, ldx, index, sp, lds, vp, rows, cols);
  else if (block) pick_nll_forward_kernel<T, true, false><<<grid, 256, 0, stream>>>(xp, ldx, index, sp, lds, vp, rows, cols);
  else if (vec) pick_nll_forward_kernel<T, false, true><<<grid, 256, 0, stream>>>(xp, ldx, index, sp, lds, vp, rows, cols);
  else pick_nll_forward_kernel<T, false, false><<<grid, 256, 0, stream>>>(xp, ldx, index, sp, lds, vp, rows, cols);
}

template <typename T>
void softmax_backward_t(const void* y, long long ldy, const void* dy, long long lddy, void* dx,
                        long long lddx, int rows, long long cols, int accumulate,
                        cudaStream_t stream) {
  const unsigned a = sizeof(T) * 4;
  const bool vec = cols_aligned(y, ldy, sizeof(T), a) && cols_aligned(dy, lddy, sizeof(T), a) &&
                   cols_aligned(dx, lddx, sizeof(T), a);
  const bool block = rows > 2048;
  const unsigned grid = block ? static_cast<unsigned>(cols) : static_cast<unsigned>((cols + 7) / 8);
  const T* yp = static_cast<const T*>(y);
  const T* dp = static_cast<const T*>(dy);
  T* xp = static_cast<T*>(dx);
  if (block && vec) softmax_backward_kernel<T, true, true><<<grid, 256, 0, stream>>>(yp, ldy, dp, lddy, xp, lddx, rows, cols, accumulate);
  else if (block) softmax_backward_kernel<T, true, false><<<grid, 256, 0, stream>>>(yp, ldy, dp, lddy, xp, lddx, rows, cols, accumulate);
  else if (vec) softmax_backward_kernel<T, false, true><<<grid, 256, 0, stream>>>(yp, ldy, dp, lddy, xp, lddx, rows, cols, accumulate);
  else softmax_backward_kernel<T, false, false><<<grid, 256, 0, stream>>>(yp, ldy, dp, lddy, xp, lddx, rows, cols, accumulate);
}

template <typename T>
void pick_backward_t(const void* smax, long long lds, const int* index, const void* grad, void* dx,
                     long long lddx, int rows, long long cols, cudaStream_t stream) {
  const unsigned a = sizeof(T) * 4;
  const bool vec = cols_aligned(smax, lds, sizeof(T), a) && cols_aligned(dx, lddx, sizeof(T), a);
  const unsigned grid = static_cast<unsigned>((cols + 7) / 8);
  const T* sp = static_cast<const T*>(smax);
  const T* gp = static_cast<const T*>(grad);
  T* dp = static_cast<T*>(dx);
  if (vec) pick_nll_backward_kernel<T, true><<<grid, 256, 0, stream>>>(sp, lds, index, gp, dp, lddx, rows, cols);
  else pick_nll_backward_kernel<T, false><<<grid, 256, 0, stream>>>(sp, lds, index, gp, dp, lddx, rows, cols);
}
}  // namespace

cudaError_t launch_pick_nll_forward(int dtype, const void* x, long long ldx, const int* index,
                                    void* smax, long long lds, void* value, int rows,
                                    long long cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  if (cols > 0x7fffffffLL) return cudaErrorInvalidValue;
  if (dtype == 0) pick_forward_t<float>(x, ldx, index, smax, lds, value, rows, cols, stream);
  else pick_forward_t<__half>(x, ldx, index, smax, lds, value, rows, cols, stream);
  return cudaGetLastError();
}

cudaError_t launch_softmax_backward(int dtype, const void* y, long long ldy, const void* dy,
                                    long long lddy, void* dx, long long lddx, int rows,
                                    long long cols, int accumulate, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  if (cols > 0x7fffffffLL) return cudaErrorInvalidValue;
  if (dtype == 0) softmax_backward_t<float>(y, ldy, dy, lddy, dx, lddx, rows, cols, accumulate, stream);
  else softmax_backward_t<__half>(y, ldy, dy, lddy, dx, lddx, rows, cols, accumulate, stream);
  return cudaGetLastError();
}

cudaError_t launch_pick_nll_backward(int dtype, const void* smax, long long lds, const int* index,
                                     const void* grad, void* dx, long long lddx, int rows,
                                     long long cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  if (cols > 0x7fffffffLL) return cudaErrorInvalidValue;
  if (dtype == 0) pick_backward_t<float>(smax, lds, index, grad, dx, lddx, rows, cols, stream);
  else pick_backward_t<__half>(smax, lds, index, grad, dx, lddx, rows, cols, stream);
  return cudaGetLastError();
}

cudaError_t launch_bias_act_half(void* y, long long ldy, const void* bias, int act, int m,
                                 long long n, cudaStream_t stream) {
  if (m <= 0 || n <= 0 || (bias == nullptr && act == ACT_NONE)) return cudaSuccess;
  if (n > 65535) return cudaErrorInvalidValue;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  const bool vec = m % 8 == 0 && ldy % 8 == 0 && al(y) && (bias == nullptr || al(bias));
  const int per = vec ? 8 : 1;
  dim3 grid(((m + per - 1) / per + 255) / 256, static_cast<unsigned>(n));
  return launch_kernel(vec ? bias_act_half_kernel<true> : bias_act_half_kernel<false>, grid, dim3(256), 0,
                       stream, pdl_enabled(), static_cast<__half*>(y), ldy,
                       static_cast<const __half*>(bias), act, m, n);
}

cudaError_t launch_add_partials_half(void* c, long long ldc, const void* ws, int parts, int m,
                                     long long n, cudaStream_t stream) {
  if (m <= 0 || n <= 0 || parts <= 0) return cudaSuccess;
  if (n > 65535) return cudaErrorInvalidValue;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  const bool vec = m % 8 == 0 && ldc % 8 == 0 && al(c) && al(ws);
  const int per = vec ? 8 : 1;
  dim3 grid(((m + per - 1) / per + 255) / 256, static_cast<unsigned>(n));
  return launch_kernel(vec ? add_partials_half_kernel<true> : add_partials_half_kernel<false>, grid,
                       dim3(256), 0, stream, pdl_enabled(), static_cast<__half*>(c), ldc,
                       static_cast<const __half*>(ws), parts, m, n);
}

cudaError_t launch_dact_half(const void* dy, long long lddy, const void* y, long long ldy, int act,
                             void* da, int m, long long n, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return cudaSuccess;
  if (n > 65535) return cudaErrorInvalidValue;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  const bool vec = m % 8 == 0 && lddy % 8 == 0 && ldy % 8 == 0 && al(dy) && al(y) && al(da);
  const int per = vec ? 8 : 1;
  dim3 grid(((m + per - 1) / per + 255) / 256, static_cast<unsigned>(n));
  const __half *d = static_cast<const __half*>(dy), *yy = static_cast<const __half*>(y);
  return launch_kernel(vec ? dact_half_kernel<true> : dact_half_kernel<false>, grid, dim3(256), 0, stream,
                       pdl_enabled(), d, lddy, yy, ldy, act, static_cast<__half*>(da), m, n);
}

cudaError_t launch_act_inplace_f32(float* c, long long ldc, long long stride, int act, int m, int n,
                                   int batches, cudaStream_t stream) {
  if (m <= 0 || n <= 0 || batches <= 0 || act == ACT_NONE) return cudaSuccess;
  if (batches > 65535) return cudaErrorInvalidValue;
  dim3 grid((m + 255) / 256, n < 65535 ? n : 65535, batches);
  return launch_kernel(act_inplace_f32_kernel, grid, dim3(256), 0, stream, pdl_enabled(), c, ldc,
                       stride, act, m, n);
}

cudaError_t launch_lstm_cell_forward(float* gates, long long ldg, const float* c_prev,
                                     long long ldcp, float* c, long long ldc, float* h,
                                     long long ldh, float* xh_next, long long ldx, int H,
                                     long long n, long long n_next, cudaStream_t stream) {
  if (H <= 0 || n <= 0) return cudaSuccess;
  if (n > 65535) return cudaErrorInvalidValue;
  dim3 grid((H + 255) / 256, static_cast<unsigned>(n));
  return launch_kernel(lstm_cell_forward_kernel, grid, dim3(256), 0, stream, pdl_enabled(), gates,
                       ldg, c_prev, ldcp, c, ldc, h, ldh, xh_next, ldx, H, n, n_next);
}

cudaError_t launch_fill(int dtype, void* x, long long n, float value, int num_sms, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  long long blocks = (n + 255) / 256;
  if (blocks > static_cast<long long>(num_sms) * 8) blocks = static_cast<long long>(num_sms) * 8;
  if (dtype == 0)
    fill_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<float*>(x), n, value);
  else
    fill_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<__half*>(x), n, value);
  return cudaGetLastError();
}

cudaError_t launch_scale_mask_f32(float* s, long long ld, long long stride, int T, int batches,
                                  float scale, int causal, cudaStream_t stream) {
  if (T <= 0 || batches <= 0) return cudaSuccess;
  if (T > 65535 || batches > 65535) return cudaErrorInvalidValue;
  dim3 grid((T + 255) / 256, T, batches);
  scale_mask_f32_kernel<<<grid, 256, 0, stream>>>(s, ld, stride, T, scale, causal);
  return cudaGetLastError();
}

cudaError_t launch_lstm_cells(bool backward, const void* const* dtab, int H, long long n,
                              cudaStream_t stream) {
  if (H <= 0 || n <= 0) return cudaSuccess;
  if (n > 65535) return cudaErrorInvalidValue;
  dim3 grid((H + 255) / 256, static_cast<unsigned>(n));
  return launch_kernel(backward ? lstm_cells_backward_kernel : lstm_cells_forward_kernel, grid,
                       dim3(256), 0, stream, pdl_enabled(), dtab, H, n);
}

cudaError_t launch_lstm_cell_backward(const float* gates, long long ldg, const float* c,
                                      long long ldc, const float* c_prev, long long ldcp,
                                      const float* dh_next, long long lddh, const float* dc_next,
                                      long long lddc, float dh_end, float* dgates, long long lddg,
                                      float* dc_out, long long lddo, int H, long long n,
                                      long long n_next, cudaStream_t stream) {
  if (H <= 0 || n <= 0) return cudaSuccess;
  if (n > 65535) return cudaErrorInvalidValue;
  dim3 grid((H + 255) / 256, static_cast<unsigned>(n));
  return launch_kernel(lstm_cell_backward_kernel, grid, dim3(256), 0, stream, pdl_enabled(), gates,
                       ldg, c, ldc, c_prev, ldcp, dh_next, lddh, dc_next, lddc, dh_end, dgates, lddg,
                       dc_out, lddo, H, n, n_next);
}

cudaError_t launch_adam(int dtype, void* w, void* d, float* m, float* v, long long n, float clip,
                        float b1, float b2, float step, float vscale, float eps, int num_sms,
                        cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  auto al = [](const void* p, unsigned a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; };
  const bool vec = al(m, 16) && al(v, 16) && al(w, dtype == 0 ? 16 : 8) && al(d, dtype == 0 ? 16 : 8);
  const long long work = vec ? (n + 3) / 4 : n;
  long long blocks = (work + 255) / 256;
  const long long cap = static_cast<long long>(num_sms) * 8;  // grid-stride beyond eight CTAs per SM
  if (blocks > cap) blocks = cap;
  const unsigned g = static_cast<unsigned>(blocks);
  if (dtype == 0) {
    float *wf = static_cast<float*>(w), *df = static_cast<float*>(d);
    if (vec) adam_kernel<float, true><<<g, 256, 0, stream>>>(wf, df, m, v, n, clip, b1, b2, step, vscale, eps);
    else adam_kernel<float, false><<<g, 256, 0, stream>>>(wf, df, m, v, n, clip, b1, b2, step, vscale, eps);
  } else {
    __half *wh = static_cast<__half*>(w), *dh = static_cast<__half*>(d);
    if (vec) adam_kernel<__half, true><<<g, 256, 0, stream>>>(wh, dh, m, v, n, clip, b1, b2, step, vscale, eps);
    else adam_kernel<__half, false><<<g, 256, 0, stream>>>(wh, dh, m, v, n, clip, b1, b2, step, vscale, eps);
  }
  return cudaGetLastError();
}

}  // namespace gb
