/* ginn_b200 -- C ABI of the B200 (sm_100a) back end for ginn's dense-contraction path.
 *
 * All matrices are column-major, as in ginn (ginn/tensor.h).  Pointers are device pointers on
 * GPU `device`; `stream` is a cudaStream_t (NULL = legacy default stream).  Calls enqueue work
 * and return; they never synchronise the device and never allocate from a ginn Device (the
 * library keeps small internal buffers of its own).  The one host-side wait: ginn_b200_grouped
 * recycles an 8 MiB descriptor ring in halves and, before it reuses a half, waits for its own
 * earlier launches that read that half.  Every function returns a ginn_b200_status; on a
 * non-zero status ginn_b200_last_error() describes the failure for the calling thread.
 *
 * Scratch memory: a few entry points take scratch for the duration of a call from the device's
 * default stream-ordered memory pool (cudaMallocAsync / cudaFreeAsync on the caller's stream):
 * large fp16 Affine backward passes (documented at ginn_b200_affine_backward), convolutions
 * without a caller workspace, and large fp32 products (option "presplit": 8 * (m + n) * k bytes).
 * On the first call for a device the library gives that pool a release threshold of 4 GiB, so
 * that freed scratch stays cached instead of going back to the driver at every synchronisation.
 * ginn_b200_grouped_static is the entry point that allocates nothing.
 *
 * Streams: every call orders its work on `stream`.  ginn_b200_affine_backward,
 * ginn_b200_prod_backward and ginn_b200_attention_backward run part of their launches on one
 * extra stream per device that the library owns, forked from and joined back into `stream`
 * inside the call (option "fork_streams").
 *
 * dtype: GINN_B200_F32 computes with three TF32 tensor-core products per term (fp32-level
 * accuracy, fp32 accumulation); GINN_B200_F16 uses fp16 inputs/outputs with fp32 accumulation.
 */
#ifndef GINN_B200_H
#define GINN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  GINN_B200_OK = 0,
  GINN_B200_BAD_ARGUMENT = 1,  /* shape / pointer / leading-dimension check failed            */
  GINN_B200_UNSUPPORTED = 2,   /* dtype or option not supported                               */
  GINN_B200_CUDA_ERROR = 3,    /* a CUDA runtime call failed (text in ginn_b200_last_error)   */
  GINN_B200_DEVICE_TIMEOUT = 4 /* a kernel gave up on a bounded wait (ginn_b200_device_status) */
} ginn_b200_status;

typedef enum { GINN_B200_F32 = 0, GINN_B200_F16 = 1 } ginn_b200_dtype;

/* Nonlinearities that are fused into the kernels (ginn/nonlin.h:67-155). */
typedef enum {
  GINN_B200_ACT_NONE = 0,
  GINN_B200_ACT_TANH = 1,
  GINN_B200_ACT_SIGMOID = 2,
  GINN_B200_ACT_RELU = 3
} ginn_b200_act;

/* C = op(A) * op(B) + (accumulate ? C : 0).   op(A) is m x k, op(B) is k x n.
 * Replaces internal::gpu_gemm (ginn/prod.h:32-66) as called by internal::gpu_prod
 * (ginn/prod.h:211-253): trans_a/trans_b are ProdTranspose First/Second, accumulate is
 * ProdResult::Add, lda/ldb/ldc are the stored row counts. */
int ginn_b200_gemm(int device, void* stream, int dtype, int trans_a, int trans_b, int64_t m,
                   int64_t n, int64_t k, const void* a, int64_t lda, const void* b, int64_t ldb,
                   void* c, int64_t ldc, int accumulate);

/* Strided-batched form: matrix i of each operand starts stride_* elements after matrix i-1.
 * Replaces internal::gpu_batched_gemm (ginn/prod.h:68-135) as called by
 * internal::gpu_batched_prod (ginn/prod.h:255-310), including the m = n = 1 batched dot
 * products of SoftmaxOp::backward (ginn/nonlin.h:180-183). */
int ginn_b200_gemm_batched(int device, void* stream, int dtype, int trans_a, int trans_b,
                           int64_t m, int64_t n, int64_t k, const void* a, int64_t lda,
                           int64_t stride_a, const void* b, int64_t ldb, int64_t stride_b, void* c,
                           int64_t ldc, int64_t stride_c, int64_t batches, int accumulate);

/* Both gradient products of a ProdNode / BatchedProdNode whose forward pass was
 * C (m x n) = A (m x k) * B (k x n), per batch:
 *     da (m x k) += dc (m x n) * B^T      (skipped when da is NULL)
 *     db (k x n) += A^T * dc (m x n)      (skipped when db is NULL)
 * Replaces the two gpu_prod / gpu_batched_prod calls of ProdNode::backward_ and
 * BatchedProdNode::backward_ (ginn/node/prod.h:51-66, 118-130).  The two products share only
 * read-only operands; when their outputs do not overlap they run side by side (the second on
 * a stream of the library's own, forked from and joined back into `stream` inside the call;
 * option "fork_streams").  batches = 1 with strides 0 is the plain product. */
int ginn_b200_prod_backward(int device, void* stream, int dtype, int64_t m, int64_t n, int64_t k,
                            int64_t batches, const void* a, int64_t lda, int64_t stride_a,
                            const void* b, int64_t ldb, int64_t stride_b, const void* dc,
                            int64_t lddc, int64_t stride_dc, void* da, int64_t ldda,
                            int64_t stride_da, void* db, int64_t lddb, int64_t stride_db);

/* One (A_i, B_i) term of an Affine node: A_i is m x k (leading dimension lda), B_i is k x n. */
typedef struct {
  const void* a;
  int64_t lda;
  const void* b;
  int64_t ldb;
  int64_t k;
} ginn_b200_pair;

/* out(m x n) = act( sum_i A_i * B_i + bias ), bias broadcast over columns; one kernel.
 * Replaces the GPU branch of AffineNode::forward_ (ginn/node/affine.h:56-64,74-76): the bias
 * broadcast kernel, the accumulating GEMMs and the separate nonlinearity kernel.
 * npairs <= 4; bias may be NULL. */
int ginn_b200_affine_forward(int device, void* stream, int dtype, int npairs,
                             const ginn_b200_pair* pairs, int64_t m, int64_t n, const void* bias,
                             int act, void* out, int64_t ldo);

/* Gradient slots of one Affine term; NULL means "input has no gradient". */
typedef struct {
  const void* a; /* A_i value, m x k */
  int64_t lda;
  const void* b; /* B_i value, k x n */
  int64_t ldb;
  int64_t k;
  void* da; /* += dA * B_i^T   (m x k, leading dimension ldda) */
  int64_t ldda;
  void* db; /* += A_i^T * dA   (k x n, leading dimension lddb) */
  int64_t lddb;
} ginn_b200_pair_grad;

/* Backward of the Affine node, with dA = dout (.) act'(out):
 *   dbias += rowsum(dA);   db_i += A_i^T * dA;   da_i += dA * B_i^T.
 * fp32: dA is formed on the fly inside the operand loaders (no dpreactiv_ tensor is written).
 * fp16 with m * n >= 65536: dA is materialised once in a stream-ordered scratch allocation of the
 * library's own (cudaMallocAsync / cudaFreeAsync on `stream`), as the reference materialises
 * dpreactiv_, so that both products run on the TMA-fed kernels.  Large layers also take two small
 * stream-ordered buffers from the same pool: fp32 partial sums of the bias gradient (at most
 * 64 * m floats) and, when a weight gradient has few output tiles and n >= 1024, fp16 partial
 * products of its column chunks (at most 8 * m * k elements), which one pass adds to da.
 * Replaces the GPU branch of AffineNode::backward_ (ginn/node/affine.h:79-87,103-125).
 * `out` is the node's value (needed for tanh/sigmoid/relu derivatives; may be NULL for
 * ACT_NONE); dbias may be NULL. */
int ginn_b200_affine_backward(int device, void* stream, int dtype, int npairs,
                              const ginn_b200_pair_grad* pairs, int64_t m, int64_t n,
                              const void* dout, int64_t lddout, const void* out, int64_t ldout,
                              int act, void* dbias);

/* The same with the scratch tensor supplied by the caller: `scratch` holds m * n elements of
 * `dtype` (16-byte aligned, leading dimension m) and is what AffineNode keeps as dpreactiv_
 * (ginn/node/affine.h:82-88), so a node that passes its own tensor keeps dA out of the library's
 * pool and its device's accounting (PreallocGpuDevice::used()) exactly as the reference has it;
 * the two small partial-sum buffers described above still come from the stream-ordered pool
 * (which hands the same blocks back call after call: the device's free memory does not move).
 * Only large Half Affines with a nonlinearity write it; NULL = as ginn_b200_affine_backward. */
int ginn_b200_affine_backward_scratch(int device, void* stream, int dtype, int npairs,
                                      const ginn_b200_pair_grad* pairs, int64_t m, int64_t n,
                                      const void* dout, int64_t lddout, const void* out,
                                      int64_t ldout, int act, void* dbias, void* scratch);

/* One group of an autobatch level: `ncols` products that share the left operand W (m x k).
 * Column j of the right-hand side lives at x_cols[j] (k contiguous elements), column j of
 * the result at y_cols[j] (m contiguous elements) -- the addresses of the individual nodes'
 * tensors, so the concatenation copy of RowwiseCat and the bias broadcast of ColBroadcast
 * (ginn/autobatch.h:80-113,149-183; ginn/node/layout.h:227-241,870-887) disappear.
 * x_cols / y_cols are HOST arrays of DEVICE pointers; the library stages them. */
typedef struct {
  const void* w;
  int64_t ldw;
  int64_t m, k;
  const void* bias; /* forward: added to every column (may be NULL); dW mode: unused */
  int64_t ncols;
  const void* const* x_cols; /* forward/dW: inputs x_j (k);  dX mode: unused              */
  void* const* y_cols;       /* forward: outputs y_j (m);    dX/dW mode: upstream dy_j (m) */
  void* const* dx_cols;      /* dX mode: dx_j (k), accumulated                              */
  void* dw;                  /* dW mode: m x k, accumulated (leading dimension lddw)        */
  int64_t lddw;
  void* dbias;               /* dW mode: m, accumulated (may be NULL)                       */
  int accumulate;            /* forward: y_j += W * x_j (+ bias) instead of y_j = ...       */
  /* Affines with a fused nonlinearity (ginn/autobatch.h:30-38 leaves them unbatched):
   * forward: y_j = act(W x_j + bias [+ y_j]) -- set it on the launch that adds a node's last
   * product;  dX / dW mode: the upstream gradient is taken as dy_j (.) act'(out_j), where
   * out_cols[j] is the node's forward value (m elements).  GINN_B200_ACT_NONE = identity. */
  int act;
  const void* const* out_cols; /* dX / dW mode with act != NONE: node values out_j (m)       */
} ginn_b200_group;

typedef enum {
  GINN_B200_GROUPED_FORWARD = 0, /* y_j  = W * x_j + bias  (+= when the group says accumulate) */
  GINN_B200_GROUPED_DX = 1,      /* dx_j += W^T * dy_j               */
  GINN_B200_GROUPED_DW = 2       /* dW  += sum_j dy_j x_j^T, dbias += sum_j dy_j */
} ginn_b200_grouped_mode;

/* All groups of one autobatch level in ONE launch (device-side tile table lookup).
 * The descriptors travel through a host ring that later calls reuse, so the call refuses
 * (GINN_B200_UNSUPPORTED) a stream that is being captured into a CUDA graph; prepared levels
 * (ginn_b200_level_*) are the form to capture. */
int ginn_b200_grouped(int device, void* stream, int dtype, int mode, int ngroups,
                      const ginn_b200_group* groups);

/* ginn_b200_grouped for callers that must not allocate.  No counterpart in the reference.
 *
 * ginn_b200_grouped keeps the per-level problem descriptors and column-pointer tables in
 * buffers it obtains from cudaMalloc / cudaMallocHost on first use.  A host that runs with a
 * fixed GPU-memory budget -- for example a ginn program built around PreallocGpuDevice, whose
 * tests account for every byte taken from the device (ginn/dev.h:214-261, test/dev.cu.cpp) --
 * or one that calls from a place where the CUDA allocator must not be entered, can use this
 * entry point instead.  It computes exactly the same thing with the same kernel, but the
 * descriptors live in a fixed 256 KiB array that is part of the library itself (each GPU that
 * loads the library carries it until the process ends), and the call makes no cudaMalloc,
 * cudaFree or other allocating call.
 *
 * Limit: descriptors plus tables of one call must fit in 256 KiB -- about 640 bytes per group
 * and 16 bytes per column, e.g. 32 groups with 15000 columns in total.  Larger levels are
 * refused with GINN_B200_BAD_ARGUMENT; split them or use ginn_b200_grouped.
 * The first call on each device looks up the array's device address; make that first call
 * outside any stream capture.  Every call copies its descriptors from one host buffer that the
 * next call overwrites, so a call on a stream that is being captured is refused with
 * GINN_B200_UNSUPPORTED.  Because that buffer is ordinary host memory, the call may wait for
 * work already queued on `stream`.  All calls on a GPU share the one array, and it keeps what
 * the last call wrote; the part a call uses is rewritten in full, so nothing has to be
 * cleared, but two calls whose GPU work overlaps (different streams without an event between
 * them) would corrupt each other -- keep these calls on one stream.  A kernel that gives up on
 * a bounded wait records it in a status word that also lives inside the library image; read
 * it with ginn_b200_grouped_static_status (ginn_b200_device_status does not see it). */
int ginn_b200_grouped_static(int device, void* stream, int dtype, int mode, int ngroups,
                             const ginn_b200_group* groups);

/* Status word of the kernels launched by ginn_b200_grouped_static on `device` (same layout as
 * ginn_b200_device_status; 0 = healthy).  Allocates nothing; synchronises the device. */
int ginn_b200_grouped_static_status(int device, int reset);

/* A level prepared once and launched many times -- the schedule cache ginn's Autobatch lacks: the
 * reference rebuilds RowwiseCat / Prod / RowwiseUncat nodes and re-copies every column on each
 * evaluation (ginn/autobatch.h:149-183, ginn/node/layout.h:227-241).  ginn_b200_level_create
 * validates the groups and keeps descriptors and column tables resident in device memory;
 * ginn_b200_level_run is then a single kernel launch with no host-to-device copy, so it can
 * also be captured in a CUDA graph.  The tensors named by the groups must stay where they are
 * while the level is in use (the nodes of a re-evaluated ginn graph do).  Create and destroy
 * synchronise with the device; run does not. */
typedef struct ginn_b200_level ginn_b200_level;
int ginn_b200_level_create(int device, int dtype, int mode, int ngroups,
                           const ginn_b200_group* groups, ginn_b200_level** out);
int ginn_b200_level_run(ginn_b200_level* level, void* stream);
int ginn_b200_level_destroy(ginn_b200_level* level);

/* ---- The elementwise neighbours of the products on a training step ------------------------ */

/* Picked negative log softmax, forward: for every column j of x (rows x cols, column-major)
 *   smax[:, j] = softmax(x[:, j]),   value[j] = -log(smax[index[j], j]).
 * Replaces PickNegLogSoftmaxNode::forward_ (ginn/node/pick.h:209-216) with its SoftmaxOp::forward
 * (ginn/nonlin.h:162-168: maximum, exp, sum, divide as four statements and two temporaries) and
 * the thrust gather of PickNode::pick (pick.h:60-84).  `index` is a device array of `cols` ints;
 * an index outside [0, rows) yields value = +inf (the reference asserts on the CPU only,
 * pick.h:133-142).  smax is kept by the caller for the backward pass, as the node keeps smax_. */
int ginn_b200_pick_nll_forward(int device, void* stream, int dtype, int64_t rows, int64_t cols,
                               const void* x, int64_t ldx, const int* index, void* smax,
                               int64_t ldsmax, void* value);

/* Backward of the above: dx[i, j] += (smax[i, j] - [i == index[j]]) * grad[j], one pass.
 * Replaces PickNegLogSoftmaxNode::backward_ (pick.h:218-224) and pick_grad(negate) (pick.h:87-131:
 * gather, subtract, scatter through a temporary). */
int ginn_b200_pick_nll_backward(int device, void* stream, int dtype, int64_t rows, int64_t cols,
                                const void* smax, int64_t ldsmax, const int* index,
                                const void* grad, void* dx, int64_t lddx);

/* Column softmax y[:, j] = softmax(x[:, j]) of a rows x cols column-major matrix (any number of
 * trailing dimensions folded into cols).  Replaces SoftmaxOp::forward (ginn/nonlin.h:162-168). */
int ginn_b200_softmax_forward(int device, void* stream, int dtype, int64_t rows, int64_t cols,
                              const void* x, int64_t ldx, void* y, int64_t ldy);

/* dx (+)= y (.) (dy - colsum(y (.) dy)), `+=` when accumulate != 0.  Replaces SoftmaxOp::backward
 * (ginn/nonlin.h:169-190), including the batched 1 x 1 products its GPU branch sends through
 * gpu_batched_prod (:177-184). */
int ginn_b200_softmax_backward(int device, void* stream, int dtype, int64_t rows, int64_t cols,
                               const void* y, int64_t ldy, const void* dy, int64_t lddy, void* dx,
                               int64_t lddx, int accumulate);

/* LSTM cell glue for the autobatch benchmark (fp32).  No single reference counterpart: ginn
 * composes the cell from CwiseProd, Tanh and Add nodes (ginn/model/lstm.h:97-100), i.e. several
 * elementwise kernels per step; with one merged gate product per level (rows i | f | g | o of a
 * 4*hidden x n matrix) the whole update is one pass.
 * forward: gates are replaced by their activations (sigmoid, sigmoid, tanh, sigmoid);
 *   c = f c_prev + i g (c_prev NULL: zeros), h = o tanh(c); when xh_next is not NULL the first
 *   n_next columns of h are also written there (the next level's input block, leading dim ldx). */
int ginn_b200_lstm_cell_forward(int device, void* stream, int64_t hidden, int64_t n, int64_t n_next,
                                float* gates, int64_t ldg, const float* c_prev, int64_t ldcp,
                                float* c, int64_t ldc, float* h, int64_t ldh, float* xh_next,
                                int64_t ldx);
/* backward: columns < n_next take dh from dh_next and dc from dc_next (the next level's results),
 * the others end here and take dh = dh_end, dc = 0;  dc += dh o (1 - tanh(c)^2);
 *   dgates = [dc g i(1-i) | dc c_prev f(1-f) | dc i (1-g^2) | dh tanh(c) o(1-o)],  dc_out = dc f. */
int ginn_b200_lstm_cell_backward(int device, void* stream, int64_t hidden, int64_t n,
                                 int64_t n_next, const float* gates, int64_t ldg, const float* c,
                                 int64_t ldc, const float* c_prev, int64_t ldcp,
                                 const float* dh_next, int64_t lddh, const float* dc_next,
                                 int64_t lddc, float dh_end, float* dgates, int64_t lddg,
                                 float* dc_out, int64_t lddo);

/* The same cell update for cells whose tensors are separate allocations -- one graph node per
 * sequence and step, as ginn builds an LSTM -- so that all cells of one autobatch level are one
 * launch.  `tables` is a HOST array of 4 (forward) or 7 (backward) tables of `n` DEVICE pointers
 * each, table after table:
 *   forward : gates (4*hidden, replaced by the activations), c_prev (hidden; an entry may be
 *             NULL = zeros), c (hidden, written), h (hidden, written)
 *   backward: gates, c, c_prev (entry may be NULL), dh (gradient of h), dc (gradient of c),
 *             dgates (4*hidden, +=), dc_prev (hidden, +=; NULL where c_prev is NULL)
 * ginn_b200_lstm_cells stages the tables and launches (not capturable, like ginn_b200_grouped);
 * ginn_b200_lstm_cells_level_create keeps them on the device for ginn_b200_level_run /
 * ginn_b200_level_destroy.  No reference counterpart (ginn/model/lstm.h:97-100 as node-wise ops). */
int ginn_b200_lstm_cells(int device, void* stream, int backward, int64_t hidden, int64_t n,
                         const void* const* tables);
int ginn_b200_lstm_cells_level_create(int device, int backward, int64_t hidden, int64_t n,
                                      const void* const* tables, ginn_b200_level** out);

/* One Adam step on n elements: d is clipped to [-clip, clip] in place, then
 *   m = beta1 m + (1 - beta1) d,  v = beta2 v + (1 - beta2) d^2,
 *   w += -lr / (1 - beta1_t) * m / (eps + sqrt(v / (1 - beta2_t))),
 * with beta1_t = beta1^t, beta2_t = beta2^t already advanced by the caller for this step.
 * Replaces Adam::update (ginn/update/update.h:115-133: six tensor statements).  w and d have
 * type `dtype`; m and v are always fp32, as the reference's History keeps them. */
int ginn_b200_adam_update(int device, void* stream, int dtype, int64_t n, void* w, void* d,
                          float* m, float* v, float lr, float clip, float eps, float beta1,
                          float beta2, float beta1_t, float beta2_t);

/* ---- Attention as min-GPT composes it from BatchedProd, mask and Softmax ------------------- */

/* For every batch b (min-GPT folds batch and heads into it):
 *   S = scale * K'_b * Q_b;  causal: S[i, j] = -inf for key i > query j;
 *   P = column softmax of S;  O_b = V_b * P
 * with ginn's layouts (examples/min-gpt.cu.cpp:108-157): K' is T x hs, Q and V are hs x T, P is
 * T x T, O is hs x T, all column-major with the given leading dimensions and batch strides.
 * Replaces BatchedProd -> InPlaceProdScalar -> InPlaceMask -> Softmax -> BatchedProd, which
 * writes and re-reads two T x T tensors per batch.  fp32 with T <= 256, hs in {32, 64, 128} and
 * 16-byte aligned operands runs as ONE kernel that keeps the scores in tensor memory; `p` is then
 * written only because SoftmaxOp's backward needs it and may be NULL when no backward follows.
 * Other shapes (and fp16) take the unfused sequence inside the library and need `p` as their
 * score buffer. */
int ginn_b200_attention_forward(int device, void* stream, int dtype, int64_t t, int64_t hs,
                                int64_t batches, const void* k, int64_t ldk, int64_t stride_k,
                                const void* q, int64_t ldq, int64_t stride_q, const void* v,
                                int64_t ldv, int64_t stride_v, float scale, int causal, void* o,
                                int64_t ldo, int64_t stride_o, void* p, int64_t ldp,
                                int64_t stride_p);
/* Gradients of the above from the kept softmax output `p` and the upstream gradient `d_o`, all
 * accumulated (`+=`), NULL = input without gradient:
 *   dv += d_o * P^T;   dP = V^T * d_o;   dS = scale * P (.) (dP - colsum(P (.) dP));
 *   dk += dS * Q^T;    dq += K'^T * dS.
 * `ds` is a caller-owned T x T x batches scratch with p's layout (it holds dP, then dS).
 * Replaces the backward passes of the five nodes (ginn/node/prod.h:129-169, ginn/nonlin.h:
 * 169-190): four batched products and one softmax-backward pass, without the mask / scale
 * tensors. */
int ginn_b200_attention_backward(int device, void* stream, int dtype, int64_t t, int64_t hs,
                                 int64_t batches, const void* k, int64_t ldk, int64_t stride_k,
                                 const void* q, int64_t ldq, int64_t stride_q, const void* v,
                                 int64_t ldv, int64_t stride_v, float scale, const void* p,
                                 int64_t ldp, int64_t stride_p, const void* d_o, int64_t ldo,
                                 int64_t stride_o, void* ds, void* dk, void* dq, void* dv);

/* ---- Conv2d through the same products ------------------------------------------------------ */

/* 2-d convolution with "SAME" padding, as Conv2dNode computes it (ginn/node/conv.h:28-79 over
 * ginn/eigenop/eigen_conv.h:28-74): cross-correlation of
 *   x (channels, rows, cols, batch)  with  k (filters, channels, krows, kcols)
 * into y (filters, ceil(rows / row_stride), ceil(cols / col_stride), batch), all column-major and
 * contiguous.  The reference extracts image patches and contracts them with the reshaped filters
 * (Eigen::contract); here the patch matrix ((channels krows kcols) x (out_rows out_cols batch))
 * is written into `workspace` by one pass over x and the contraction runs on the tensor-core
 * kernels.  `workspace` must hold ginn_b200_conv2d_workspace(...) bytes and be 16-byte aligned;
 * NULL makes the call take it from the stream-ordered allocator for the duration of the call. */
size_t ginn_b200_conv2d_workspace(int dtype, int64_t channels, int64_t rows, int64_t cols,
                                  int64_t batch, int64_t filters, int64_t krows, int64_t kcols,
                                  int64_t row_stride, int64_t col_stride);
int ginn_b200_conv2d_forward(int device, void* stream, int dtype, int64_t channels, int64_t rows,
                             int64_t cols, int64_t batch, int64_t filters, int64_t krows,
                             int64_t kcols, int64_t row_stride, int64_t col_stride, const void* x,
                             const void* k, void* y, void* workspace);
/* Gradients of the above (ginn/node/conv.h:52-64, eigen_conv.h:76-190), both accumulated:
 *   dk += dy * patches(x)^T          (when dk != NULL)
 *   dx += col2im(k^T * dy)           (when dx != NULL)
 * `workspace` as for the forward call (the patch matrix, then the patch gradients). */
int ginn_b200_conv2d_backward(int device, void* stream, int dtype, int64_t channels, int64_t rows,
                              int64_t cols, int64_t batch, int64_t filters, int64_t krows,
                              int64_t kcols, int64_t row_stride, int64_t col_stride, const void* x,
                              const void* k, const void* dy, void* dx, void* dk, void* workspace);

/* x[i] = value for n elements of type `dtype`, enqueued on `stream` (Tensor::fill on a GPU tensor,
 * ginn/tensor.h fill / setConstant; also how Graph::backward seeds the sink's gradient without a
 * host copy that would wait for the forward pass). */
int ginn_b200_fill(int device, void* stream, int dtype, int64_t n, void* x, float value);

/* Text of the last failure on the calling thread ("" if none). */
const char* ginn_b200_last_error(void);

/* Reads (and, if reset != 0, clears) the device status word that kernels write when a bounded
 * wait expires.  0 = healthy.  Synchronises the device. Returns -1 if the query itself fails. */
int ginn_b200_device_status(int device, int reset);

/* Exercises the kernels' bounded-wait machinery on `device`: a one-thread kernel waits, with a
 * limit of about 0.1 ms, on a barrier nothing arrives on, and must come back with the time-out
 * code in a status word (the library's own status word is not touched).  Returns GINN_B200_OK
 * when the wait ran out and was reported as designed.  Nothing faults or hangs.
 * Status word layout, also for ginn_b200_device_status: (code << 16) | detail with code
 * 1 = a filled stage never came, 2 = a free stage never came, 3 = an accumulator never completed,
 * 4 = an accumulator was never drained, 5 = self test. */
int ginn_b200_selftest(int device);

/* Library version: major * 10000 + minor * 100 + patch. */
int ginn_b200_version(void);   /* 200: ginn_b200_group gained `act` and `out_cols` */

/* Test / benchmark knobs.  They belong to the calling host thread: a value set here affects
 * the calls this thread makes afterwards and nobody else's.
 * "force_path": 0 = automatic, 2 = one-CTA TMA fp16 kernel, 4 = CTA-pair fp16 kernel (both fall
 * back to automatic when not applicable), 3 = CUDA-core kernel, 5 = cp.async gather kernels
 * (the fallbacks for operands a tensor map cannot describe).
 * "sm_margin": number of SMs the persistent kernels (fp16, and fp32 products whose CTAs walk
 * their tiles) leave unoccupied (default 0), so that a
 * collective running beside them (NCCL) finds free SMs instead of delaying the last tiles; set
 * it around the one product that overlaps the collective and back to 0 afterwards.
 * "pair_group_m": m-tiles per rasterisation group of the CTA-pair kernel (0 = default).
 * "fork_streams": 1 (default) lets ginn_b200_affine_backward, ginn_b200_prod_backward and
 * ginn_b200_attention_backward run the products of a call that do not depend on each other
 * (input gradient beside weight gradient; dA beside dB; dV and dQ beside dP -> dS -> dK') on a second stream of the library's own, forked
 * from and joined back into the caller's stream inside the call (also under stream capture);
 * 0 keeps every launch on the caller's stream.
 * "presplit": 1 (default) lets large fp32 products (at least four 128-wide tiles along both
 * extents, no batch; a full wave of tiles and a contraction of 256 or more, or fewer tiles with
 * a split contraction of 2048 or more) split both operands into
 * hi / lo planes once, in a stream-ordered scratch allocation of 8 * (m + n) * k bytes taken from
 * the device's default memory pool, instead of in every tile that reads them (a product whose
 * scratch cannot be allocated runs on the ordinary path); 0 turns it off.
 * "pair_l2_hint": L2 eviction hints of the CTA-pair kernel: bit 0 = A slices loaded evict-last
 * and B slices evict-first, bit 1 = streaming reads and writes of C (default 3; 0 = none).
 * "max_split": cap on the number of CTAs an fp32 product's contraction is split over, and on the
 * column chunks of a large fp16 weight gradient (0 = the library's choice, 1 = never split).
 * "walk_kblocks": fp32 products whose tiles have at most this many 32-deep k-blocks (and
 * outnumber the SMs) run with one CTA per SM walking the tiles (default 16; 0 = one CTA per tile).
 * "pdl": 1 (default) launches the tensor-core kernels (fp32, one-CTA fp16) and the small
 * elementwise kernels around them with programmatic dependent launch, so that a kernel's set-up overlaps the end of the kernel before
 * it in the stream (chains of small dependent launches, e.g. autobatch levels); 0 turns it off.
 * Returns GINN_B200_UNSUPPORTED for unknown names. */
int ginn_b200_set_option(const char* name, int value);

/* Number of kernels this library has launched since load (all threads, all devices). */
int64_t ginn_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* GINN_B200_H */
