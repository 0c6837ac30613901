// Host-side launch entry points of the individual kernels (internal; the public surface is
// the C ABI in include/ginn_b200.h).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include "problem.h"

struct CUtensorMap_st;  // CUDA driver tensor-map descriptor (cuda.h)

namespace gb {

// Whether kernels that support it are launched with programmatic dependent launch (option
// "pdl" of the calling thread, default on).
bool pdl_enabled();
// Large fp32 products split their operands into hi / lo planes once, in a scratch allocation,
// instead of in every tile that reads them (option "presplit"; 0 = never).
bool presplit_enabled();
// Cap on the K split of fp32 products (option "max_split" of the calling thread; 0 = no cap).
int max_split();
// SMs the persistent kernels leave free (option "sm_margin" of the calling thread).
int sm_margin();
// fp32 TMA kernel: products whose tiles have at most this many k-blocks (and outnumber the SMs)
// run with one CTA per SM walking the tiles (option "walk_kblocks"; 0 = never).
int walk_kblocks();

// Launch with the programmatic-stream-serialization attribute when `pdl` is set: the kernel may
// begin while its predecessor in the stream drains; it must call pdl_wait() before it touches
// global memory.  Kernel arguments must have the kernel's exact parameter types.
template <typename... KArgs>
cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, bool pdl, KArgs... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

// Raises a kernel's dynamic shared-memory limit once per device instead of on every launch (the
// attribute call costs about as much host time as the launch itself).  `done` is a bit mask per
// call site: one bit per device ordinal below 64.
cudaError_t set_smem_limit_once(const void* kern, int bytes, unsigned long long* done);

// Allocation-free grouped launch (grouped_static.cu): descriptors live in a fixed array inside
// the library image, and so does the status word its kernels report to.
constexpr size_t kGroupedStaticBytes = 256 * 1024;
cudaError_t grouped_static_scratch(int device, void** scratch, int** status);
cudaError_t launch_grouped_static(int dtype, const void* host_image, size_t bytes, void* scratch,
                                  int* status, int nprobs, int total_tiles, bool with_y,
                                  cudaStream_t stream);

// --- TMA-fed persistent fp16 kernel (hgemm_tma.cu) ---
struct HgemmArgs {
  const void* A;
  const void* B;
  void* C;
  long long lda, ldb, ldc;
  long long strideA, strideB, strideC;  // elements
  int transA, transB;
  int M, N, K, batches;
  int accumulate;
  // Affine epilogue out = act(fp16(product [+ C]) + bias[row]); batches must be 1 when set.
  const void* bias = nullptr;
  int act = 0;
};
// Returns true when the TMA path can take the problem (alignment and size rules).
bool hgemm_tma_supported(const HgemmArgs& a);
cudaError_t launch_hgemm_tma(const HgemmArgs& a, int num_sms, cudaStream_t stream, int* status);

// --- fp16 kernel on CTA pairs, 256 x 256 tiles (hgemm_pair.cu) ---
bool hgemm_pair_supported(const HgemmArgs& a);
// `counter`: two ints of device memory for the launch's tile queue, zero when the kernel starts;
// the kernel leaves them zero again.  Launches that may run at the same time need different
// counters.  group_m: m-tiles per rasterisation group (0 = default).  l2_hint: bit 0 = eviction
// policies on the operand loads, bit 1 = streaming accesses to C.
cudaError_t launch_hgemm_pair(const HgemmArgs& a, int num_sms, int group_m, int l2_hint,
                              int* counter, cudaStream_t stream, int* status);

// --- general fp16 kernel with a cp.async front end (hgemm_gather.cu) ---
bool hgemm_gather_supported(const Problem& p);
cudaError_t launch_hgemm_gather(Problem& p, cudaStream_t stream, int* status);
cudaError_t launch_hgemm_gather_grouped(const Problem* dprobs, int nprobs, int total_tiles,
                                        cudaStream_t stream, int* status);

// --- tensor maps (defined in hgemm_tma.cu) ---
bool encode_tmap(::CUtensorMap_st* out, int esize, const void* ptr, unsigned long long d0,
                 unsigned long long d1, unsigned long long d2, unsigned long long ld,
                 unsigned long long batch_stride, unsigned b0, unsigned b1, bool swizzle128);
bool tmap_encoder_available();

// --- TMA-fed fp32 (3xTF32) kernel (sgemm3x_tma.cu) ---
// True when every operand of the problem can be described by a tensor map (16-byte aligned
// bases, leading dimensions and batch strides; no column tables) and the problem has k > 0.
bool sgemm3x_supported(const Problem& p);
cudaError_t launch_sgemm3x(const Problem& p, cudaStream_t stream, int* status);

// K split for a problem with `tiles` output tiles (see the definition for the rules).
int sgemm3x_pick_split(const Problem& p, long long tiles, int num_sms, bool tma_path = false);
// Same pipeline with a cp.async gather front end: any alignment, column tables, grouped launches.
bool sgemm3x_gather_supported(const Problem& p);
cudaError_t launch_sgemm3x_gather(Problem& p, cudaStream_t stream, int* status);
// with_y: some problem of the level carries a derivative operand (dy (.) act'(y) on the fly).
cudaError_t launch_sgemm3x_gather_grouped(const Problem* dprobs, int nprobs, int total_tiles,
                                          bool with_y, cudaStream_t stream, int* status);

// One thread waits (bounded by limit_cycles) on a barrier nobody arrives on; writes 2 to *returned
// and DEV_TIMEOUT_SELFTEST to *status when the wait ran out as it must.
cudaError_t launch_wait_selftest(int* status, long long limit_cycles, int* returned,
                                 cudaStream_t stream);

// --- CUDA-core kernels for degenerate shapes and elementwise helpers (small.cu) ---
// One warp per output element; used for tiny m*n (batched dot products) and k == 0.
cudaError_t launch_small(int dtype, const Problem& p, cudaStream_t stream);
// Products with one extent of at most 16 (or a total contraction of at most 32) on CUDA cores.
// skinny_kind: 0 = not taken, else the mapping to pass to launch_skinny.  Problems with a bias
// gradient are not taken: the caller issues launch_rowsum first and clears `rowsum`.
int skinny_kind(int dtype, const Problem& p);
cudaError_t launch_skinny(int dtype, int kind, const Problem& p, cudaStream_t stream);
// rowsum[o] += sum_n dY[o, n] * act'(Y[o, n])   (bias gradient when no weight gradient is wanted)
cudaError_t launch_rowsum(int dtype, const void* dy, const void* y, int dact, long long ld, int M,
                          long long N, void* rowsum, cudaStream_t stream);

// --- fused attention forward, fp32 (attention.cu) ---
struct AttentionArgs {
  const void* K;  // T x hs per batch (key index contiguous)
  const void* Q;  // hs x T
  const void* V;  // hs x T
  void* O;        // hs x T
  void* P;        // T x T softmax output, or null when the caller does not need it
  long long ldk, ldq, ldv, ldo, ldp;
  long long strideK, strideQ, strideV, strideO, strideP;  // elements between batches
  int T, hs, batches;
  float scale;
  int causal;
};
// True when the one-kernel path can take the problem (T <= 256, hs in {32, 64, 128}, 16-byte
// aligned operands and strides).
bool attention_fused_supported(const AttentionArgs& a);
cudaError_t launch_attention_fwd(const AttentionArgs& a, cudaStream_t stream, int* status);
// s = scale * s in place over a strided batch of T x T matrices; with `causal`, entries with
// row > column (keys after the query) become -inf.
cudaError_t launch_scale_mask_f32(float* s, long long ld, long long stride, int T, int batches,
                                  float scale, int causal, cudaStream_t stream);

// --- Conv2d as patch extraction + matrix products (conv.cu) ---
struct ConvShape {
  long long out_rows, out_cols, pad_top, pad_left;
  long long inner;  // channels * kernel rows * kernel cols: rows of the patch matrix
  long long ncols;  // out_rows * out_cols * batch: its columns
};
// Output extents and padding of a SAME convolution; false for non-positive or oversized extents.
bool conv2d_geometry(long long C, long long R, long long W, long long B, long long F, long long KR,
                     long long KC, long long sr, long long sc, ConvShape* out);
cudaError_t launch_im2col(int dtype, const void* x, void* patches, long long C, long long R,
                          long long W, long long B, long long F, long long KR, long long KC,
                          long long sr, long long sc, const ConvShape& s, int num_sms,
                          cudaStream_t stream);
cudaError_t launch_col2im_add(int dtype, const void* dpatches, void* dx, long long C, long long R,
                              long long W, long long B, long long F, long long KR, long long KC,
                              long long sr, long long sc, const ConvShape& s, int num_sms,
                              cudaStream_t stream);

// --- elementwise neighbours of the products on a training step (step_ops.cu) ---
cudaError_t launch_pick_nll_forward(int dtype, const void* x, long long ldx, const int* index,
                                    void* smax, long long lds, void* value, int rows,
                                    long long cols, cudaStream_t stream);
// index == nullptr in launch_pick_nll_forward: plain column softmax, `value` unused.
cudaError_t launch_softmax_backward(int dtype, const void* y, long long ldy, const void* dy,
                                    long long lddy, void* dx, long long lddx, int rows,
                                    long long cols, int accumulate, cudaStream_t stream);
cudaError_t launch_pick_nll_backward(int dtype, const void* smax, long long lds, const int* index,
                                     const void* grad, void* dx, long long lddx, int rows,
                                     long long cols, cudaStream_t stream);
// c = act(c) in place, fp32, every matrix of a strided batch (the activation of a product whose
// contraction was split over CTAs).
cudaError_t launch_act_inplace_f32(float* c, long long ldc, long long stride, int act, int m, int n,
                                   int batches, cudaStream_t stream);
// y = act(y + bias) in place, fp16, n <= 65535.
cudaError_t launch_bias_act_half(void* y, long long ldy, const void* bias, int act, int m,
                                 long long n, cudaStream_t stream);
// da (m x n, leading dimension m) = dy (.) act'(y), fp16, n <= 65535.
// fp16 bias gradient without atomics (small.cu): `ws` holds rowsum_ws_parts(M, N) vectors of M
// floats; 0 parts = the shape does not qualify.
int rowsum_ws_parts(int M, long long N);
cudaError_t launch_rowsum_half_ws(const void* dy, long long ld, int M, long long N, void* rowsum,
                                  float* ws, cudaStream_t stream);
// c (m x n, ld ldc) += the sum of `parts` dense m x n fp16 matrices stored back to back at ws.
cudaError_t launch_add_partials_half(void* c, long long ldc, const void* ws, int parts, int m,
                                     long long n, cudaStream_t stream);
cudaError_t launch_dact_half(const void* dy, long long lddy, const void* y, long long ldy, int act,
                             void* da, int m, long long n, cudaStream_t stream);
cudaError_t launch_lstm_cell_forward(float* gates, long long ldg, const float* c_prev,
                                     long long ldcp, float* c, long long ldc, float* h,
                                     long long ldh, float* xh_next, long long ldx, int H,
                                     long long n, long long n_next, cudaStream_t stream);
cudaError_t launch_lstm_cell_backward(const float* gates, long long ldg, const float* c,
                                      long long ldc, const float* c_prev, long long ldcp,
                                      const float* dh_next, long long lddh, const float* dc_next,
                                      long long lddc, float dh_end, float* dgates, long long lddg,
                                      float* dc_out, long long lddo, int H, long long n,
                                      long long n_next, cudaStream_t stream);
// Cell update over per-cell tensors: `dtab` = 4 (forward) or 7 (backward) device tables of n
// pointers each (step_ops.cu describes them).
cudaError_t launch_lstm_cells(bool backward, const void* const* dtab, int H, long long n,
                              cudaStream_t stream);
cudaError_t launch_fill(int dtype, void* x, long long n, float value, int num_sms, cudaStream_t stream);
cudaError_t launch_adam(int dtype, void* w, void* d, float* m, float* v, long long n, float clip,
                        float b1, float b2, float step, float vscale, float eps, int num_sms,
                        cudaStream_t stream);

}  // namespace gb
