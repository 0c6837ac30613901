// Problem description shared by the host dispatch code and the kernels.
//
// Every matrix product on ginn's Affine / Prod / BatchedProd / autobatch path is expressed as
//     C(M x N) = act( sum_p  A_p(M x K_p) * B_p(K_p x N)  + bias(M) [+ C] )
// on column-major storage.  An operand is addressed through `Operand`, which can describe a
// plain strided matrix, a transposed one, a strided batch of them, or a matrix whose columns
// live at unrelated addresses (the rhs columns autobatch would otherwise concatenate).
#pragma once
#include <stdint.h>

namespace gb {

enum Act : int { ACT_NONE = 0, ACT_TANH = 1, ACT_SIGMOID = 2, ACT_RELU = 3 };

constexpr int kMaxPairs = 4;

// Logical operand X(o, kk): o = outer index (row of C for A, column of C for B), kk = index
// along the contraction.  The stored matrix S is column-major: S[row, col] lives at
//   (cols ? cols[col] : base + batch * batch_stride + col * ld) + row.
//   k_contig = 1 :  X(o, kk) = S[row = kk, col = o]   (contraction index contiguous)
//   k_contig = 0 :  X(o, kk) = S[row = o,  col = kk]  (outer index contiguous)
// When `ybase`/`ycols` is set the operand is the product dY (.) act'(Y) formed on the fly: `base`
// addresses dY, `ybase` addresses Y with the same geometry, `dact` names the nonlinearity.
struct Operand {
  const void* base;
  const void* ybase;
  const void* const* cols;
  const void* const* ycols;
  long long ld;
  long long batch_stride;
  int k_contig;
  int vec;   // 1: 16-byte vector loads along the contraction are legal (k_contig = 1 only)
  int dact;  // Act of the fused derivative, ACT_NONE when ybase is null
  int pad_;
};

struct Problem {
  Operand a[kMaxPairs];
  Operand b[kMaxPairs];
  long long k[kMaxPairs];
  int npairs;
  int M, N;
  int batches;
  void* c;                // output
  void* const* ccols;     // optional per-column output pointers
  long long ldc;
  long long c_batch_stride;
  const void* bias;       // per-row bias or null
  void* rowsum;           // when set: rowsum[o] += sum_kk A_0(o, kk)  (bias gradient), A_0.k_contig = 0
  int act;                // activation applied to the result
  int accumulate;         // 1: C += ..., 0: C = ...
  // tile bookkeeping (filled by the launcher)
  int tiles_m, tiles_n;
  int tile_start;         // first linear tile index of this problem inside a grouped launch
  // Split of the contraction over `split_k` CTAs per output tile (fp32 tensor-core kernels only,
  // one pair): every CTA adds its partial sum to C with atomic adds, the first one of a tile
  // also the bias.  0 or 1 = no split.  The gather kernels split only products that add and have
  // no activation; the TMA-fed launcher handles the rest around the kernel.
  int split_k;
};

}  // namespace gb
