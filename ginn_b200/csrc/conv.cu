// Conv2d through the matrix-product kernels (ginn/node/conv.h:28-79, ginn/eigenop/eigen_conv.h):
// the reference forms image patches with Eigen's extract_image_patches and contracts them with
// the filters reshaped to a matrix.  Same decomposition here, on ginn's column-major layout
//   input   (channels C, rows R, cols W, batch B)      index c + C (r + R (w + W b))
//   filters (filters F, channels C, KR, KC)            index f + F (c + C (kr + KR kc))
//   output  (F, OR, OC, B),  OR = ceil(R / row_stride), OC = ceil(W / col_stride)   ("SAME")
// with patch matrix P of shape (C KR KC) x (OR OC B), inner index c + C (kr + KR kc), column
// index or + OR (oc + OC b):
//   forward          Y  = K * P                      (F x CKK) (CKK x N)
//   filter gradient  dK += dY * P^T
//   input gradient   dP = K^T * dY,  dX += col2im(dP)
// The patch matrix is written once by an HBM-bound kernel (coalesced along the channel index,
// or along the output row when C is small) into a workspace; the products run on the tensor-core
// kernels of this library.  Padding follows Eigen's PADDING_SAME: total = max(0, (O - 1) stride
// + K - I), the smaller half in front.
#include <cuda_fp16.h>
#include "launch.h"
#include "math.cuh"

namespace gb {

namespace {

struct ConvGeom {
  int C, R, W, B, F, KR, KC, sr, sc;
  int OR, OC, pt, pl;  // output extents, top / left padding
  long long inner;     // C KR KC
  long long ncols;     // OR OC B
};

// One thread per element of the patch matrix, inner index fastest (coalesced writes; reads are
// contiguous along c, and along r for consecutive kr when C == 1).
template <typename T>
__global__ void __launch_bounds__(256)
im2col_kernel(const T* __restrict__ x, T* __restrict__ p, ConvGeom g) {
  const long long total = g.inner * g.ncols;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long col = i / g.inner;
    int in = static_cast<int>(i - col * g.inner);
    const int c = in % g.C;
    in /= g.C;
    const int kr = in % g.KR, kc = in / g.KR;
    const int orow = static_cast<int>(col % g.OR);
    const long long t = col / g.OR;
    const int ocol = static_cast<int>(t % g.OC);
    const long long b = t / g.OC;
    const int r = orow * g.sr - g.pt + kr, w = ocol * g.sc - g.pl + kc;
    T v = from_f<T>(0.f);
    if (r >= 0 && r < g.R && w >= 0 && w < g.W)
      v = x[c + static_cast<long long>(g.C) * (r + static_cast<long long>(g.R) * (w + g.W * b))];
    p[i] = v;
  }
}

// dX += col2im(dP): one thread per input element gathers the (kr, kc) patch entries that read
// it in the forward pass (no atomics; fp32 sum, one rounding).
template <typename T>
__global__ void __launch_bounds__(256)
col2im_add_kernel(const T* __restrict__ dp, T* __restrict__ dx, ConvGeom g) {
  const long long total = static_cast<long long>(g.C) * g.R * g.W * g.B;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % g.C);
    long long t = i / g.C;
    const int r = static_cast<int>(t % g.R);
    t /= g.R;
    const int w = static_cast<int>(t % g.W);
    const long long b = t / g.W;
    float sum = 0.f;
    for (int kc = 0; kc < g.KC; ++kc) {
      const int wn = w + g.pl - kc;
      if (wn < 0 || wn % g.sc != 0) continue;
      const int ocol = wn / g.sc;
      if (ocol >= g.OC) continue;
      for (int kr = 0; kr < g.KR; ++kr) {
        const int rn = r + g.pt - kr;
        if (rn < 0 || rn % g.sr != 0) continue;
        const int orow = rn / g.sr;
        if (orow >= g.OR) continue;
        const long long col = orow + static_cast<long long>(g.OR) * (ocol + g.OC * b);
        const long long in = c + static_cast<long long>(g.C) * (kr + g.KR * kc);
        sum += to_f(dp[in + g.inner * col]);
      }
    }
    dx[i] = from_f<T>(to_f(dx[i]) + sum);
  }
}

unsigned grid_for(long long total, int num_sms) {
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(num_sms) * 16;
  if (blocks > cap) blocks = cap;
  return static_cast<unsigned>(blocks < 1 ? 1 : blocks);
}

}  // namespace

bool conv2d_geometry(long long C, long long R, long long W, long long B, long long F, long long KR,
                     long long KC, long long sr, long long sc, ConvShape* out) {
  if (C <= 0 || R <= 0 || W <= 0 || B <= 0 || F <= 0 || KR <= 0 || KC <= 0 || sr <= 0 || sc <= 0)
    return false;
  const long long OR = (R + sr - 1) / sr, OC = (W + sc - 1) / sc;
  const long long pr = (OR - 1) * sr + KR - R, pc = (OC - 1) * sc + KC - W;
  out->out_rows = OR;
  out->out_cols = OC;
  out->pad_top = pr > 0 ? pr / 2 : 0;
  out->pad_left = pc > 0 ? pc / 2 : 0;
  out->inner = C * KR * KC;
  out->ncols = OR * OC * B;
  const long long lim = 0x7fffffffLL;
  return C <= lim && R <= lim && W <= lim && B <= lim && F <= lim && out->inner <= lim &&
         out->ncols <= lim && KR <= lim && KC <= lim;
}

static ConvGeom make_geom(long long C, long long R, long long W, long long B, long long F,
                          long long KR, long long KC, long long sr, long long sc,
                          const ConvShape& s) {
  ConvGeom g;
  g.C = (int)C; g.R = (int)R; g.W = (int)W; g.B = (int)B; g.F = (int)F;
  g.KR = (int)KR; g.KC = (int)KC; g.sr = (int)sr; g.sc = (int)sc;
  g.OR = (int)s.out_rows; g.OC = (int)s.out_cols; g.pt = (int)s.pad_top; g.pl = (int)s.pad_left;
  g.inner = s.inner;
  g.ncols = s.ncols;
  return g;
}

cudaError_t launch_im2col(int dtype, const void* x, void* patches, long long C, long long R,
                          long long W, long long B, long long F, long long KR, long long KC,
                          long long sr, long long sc, const ConvShape& s, int num_sms,
                          cudaStream_t stream) {
  const ConvGeom g = make_geom(C, R, W, B, F, KR, KC, sr, sc, s);
  const unsigned grid = grid_for(g.inner * g.ncols, num_sms);
  if (dtype == 0)
    im2col_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(x),
                                                    static_cast<float*>(patches), g);
  else
    im2col_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(x),
                                                     static_cast<__half*>(patches), g);
  return cudaGetLastError();
}

cudaError_t launch_col2im_add(int dtype, const void* dpatches, void* dx, long long C, long long R,
                              long long W, long long B, long long F, long long KR, long long KC,
                              long long sr, long long sc, const ConvShape& s, int num_sms,
                              cudaStream_t stream) {
  const ConvGeom g = make_geom(C, R, W, B, F, KR, KC, sr, sc, s);
  const unsigned grid = grid_for(C * R * W * B, num_sms);
  if (dtype == 0)
    col2im_add_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(dpatches),
                                                        static_cast<float*>(dx), g);
  else
    col2im_add_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(dpatches),
                                                         static_cast<__half*>(dx), g);
  return cudaGetLastError();
}

}  // namespace gb
