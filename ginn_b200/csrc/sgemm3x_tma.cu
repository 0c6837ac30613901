// TMA-fed fp32 GEMM with three TF32 tensor-core products per term ("3xTF32") for ginn's
// column-major tensors:  C = act( sum_p A_p * B_p + bias [+ C] ), optionally strided-batched,
// optionally with one operand formed on the fly as dY (.) act'(Y) and with the bias gradient
// (row sums of the A operand) accumulated on the side.
//
// Pipeline inside a CTA (one 128 x 128 tile of C):
//   warp 0     TMA producer: raw fp32 slices (128 rows x 32 k) of A, B (and Y) into a ring.
//   warps 2-9  transform A, warps 10-17 transform B: raw slice -> registers -> (derivative) ->
//              hi = rna_tf32(x), lo = x - hi -> two K-major, 128-byte-swizzled planes.  Operands
//              whose outer index is contiguous in memory are transposed here, for free.
//   warp 1     MMA issuer: per 8-wide k-step  cross += lo*hi, cross += hi*lo, main[j] += hi*hi.
//   warps 2-17 epilogue: sum the accumulators, bias / previous C / activation, store.
//
// Accuracy: the tensor core truncates when it adds into its fp32 accumulator, which biases a
// long accumulation chain (measured: relative error grows linearly with K, about 7e-9 per unit
// of K with one accumulator).  The chain is therefore cut: the large hi*hi terms rotate over
// three accumulators (k-block j goes to accumulator j mod 3), the small cross terms use a
// fourth, and the epilogue adds the four in fp32 with round-to-nearest.
#include <cuda.h>
#include <cstdio>
#include <cstring>
#include "ptx.cuh"
#include "math.cuh"
#include "launch.h"

namespace gb {

namespace {

constexpr int SBM = 128, SBN = 128, SBK = 32;
constexpr int RAW_TILE = SBM * SBK * 4;   // 16 KiB: one raw operand slice
constexpr int PLANE = 16384;              // one 128-row K-major plane
constexpr int PLANE_STAGE = 4 * PLANE;    // A hi, A lo, B hi, B lo
constexpr int PLANE_STAGES = 2;
constexpr int RAW_BYTES_TOTAL = 96 * 1024;  // 3 stages of (A,B) or 2 stages of (A,B,Y)
constexpr int XFORM_THREADS = 512;   // 8 warps per operand
constexpr int NTHREADS = 64 + XFORM_THREADS;
constexpr uint32_t CROSS_COL = 384;

struct SParams {
  CUtensorMap tmA[kMaxPairs];
  CUtensorMap tmB[kMaxPairs];
  CUtensorMap tmY;
  int k[kMaxPairs];
  int a_kc[kMaxPairs];
  int b_kc[kMaxPairs];
  int npairs;
  int dop;   // 0: none, 1: A operand carries the derivative, 2: B operand
  int dact;
  int M, N;
  int tiles_m, tiles_n;
  float* C;
  long long ldc, strideC;
  const float* bias;
  float* rowsum;
  int act;
  int accumulate;
  int split_k;  // CTAs per output tile along K (1 = none): partial sums are added atomically
  int batches;
  int total_tiles;  // tiles_m * tiles_n * batches * split_k: a CTA takes tiles blockIdx.x, + gridDim.x, ...
  int bn;       // columns of C per tile: 128, or 64 for narrow results (half the B-side work)
  // Element (row, col) of the tile's result lives at C + row * c_rs + col * c_cs: (1, ldc) for
  // C itself, (ldc, 1) when the launcher computes the transposed product (see launch_sgemm3x).
  long long c_rs, c_cs;
};

// Inline: with the short tanh of math.cuh eight copies per pass are cheaper than eight calls
// (measured on a 128 x 128 tile: 7.5 against 11.4 thousand cycles for the tanh epilogue).
__device__ __forceinline__ float act_forward_f32(int act, float x) { return act_forward<float>(act, x); }

// Sum of the four accumulators for eight consecutive columns of this thread's row (warp
// collective: every lane takes part in the tensor-memory loads).
__device__ __forceinline__ void load_acc8(uint32_t taddr, int nkb, float (&acc)[8]) {
  uint32_t v0[8], v1[8], v2[8], v3[8];
  if (nkb > 0) tmem_ld8(taddr + CROSS_COL, v0);
  if (nkb > 0) tmem_ld8(taddr, v1);
  if (nkb > 1) tmem_ld8(taddr + SBN, v2);
  if (nkb > 2) tmem_ld8(taddr + 2 * SBN, v3);
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float t = 0.f;
    if (nkb > 0) t = __uint_as_float(v0[j]) + __uint_as_float(v1[j]);
    if (nkb > 1) t += __uint_as_float(v2[j]);
    if (nkb > 2) t += __uint_as_float(v3[j]);
    acc[j] = t;
  }
}

// Eight results of one row into C: `dst` addresses the first, consecutive columns are `cs`
// elements apart, the first `nvalid` exist.  mode 0: store, 1: add to the previous C, 2: atomic
// add (partial sum of a split contraction).  The bounds test is compiled out for full groups.
template <bool FULL>
__device__ __forceinline__ void store_acc8(float* dst, long long cs, int nvalid, float (&acc)[8],
                                           float bias, int mode, int act) {
  if (FULL && cs == 1 && mode != 2 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
    // transposed result: this thread's eight columns are contiguous in memory
    float4* d4 = reinterpret_cast<float4*>(dst);
    float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
    if (mode == 1) {
      lo = d4[0];
      hi = d4[1];
    }
    float v[8] = {acc[0] + lo.x, acc[1] + lo.y, acc[2] + lo.z, acc[3] + lo.w,
                  acc[4] + hi.x, acc[5] + hi.y, acc[6] + hi.z, acc[7] + hi.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[j] += bias;
      if (act != ACT_NONE) v[j] = act_forward_f32(act, v[j]);
    }
    d4[0] = make_float4(v[0], v[1], v[2], v[3]);
    d4[1] = make_float4(v[4], v[5], v[6], v[7]);
    return;
  }
  if (mode == 1) {
    float old[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) old[j] = (FULL || j < nvalid) ? dst[j * cs] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += old[j];
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float v = acc[j] + bias;
    if (mode != 2 && act != ACT_NONE) v = act_forward_f32(act, v);
    if (FULL || j < nvalid) {
      if (mode == 2)
        atomicAdd(dst + j * cs, v);
      else
        dst[j * cs] = v;
    }
  }
}

// Transform of a k-contiguous raw slice: it already is K-major and swizzled (TMA box 32 k x 128
// outer with the 128-byte swizzle), so hi and lo go to the same offsets of their planes.
// 256 threads, 4 pieces of 16 bytes each (2 when the slice has 64 rows: its first half).  The
// guard of the split is tested once for the thread's sixteen values (math.cuh).
template <bool HAS_Y>
__device__ __forceinline__ void transform_kc(const uint8_t* src, const uint8_t* ysrc,
                                             uint8_t* dst_hi, uint8_t* dst_lo, int t, int dact,
                                             int rows = 128) {
  const int np = rows > 64 ? 4 : 2;
  float4 x[4];
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (i >= np) break;
    const int off = (t + 256 * i) * 16;
    x[i] = *reinterpret_cast<const float4*>(src + off);
    if (HAS_Y) {
      const float4 y = *reinterpret_cast<const float4*>(ysrc + off);
      x[i].x = act_backward<float>(dact, y.x, x[i].x);
      x[i].y = act_backward<float>(dact, y.y, x[i].y);
      x[i].z = act_backward<float>(dact, y.z, x[i].z);
      x[i].w = act_backward<float>(dact, y.w, x[i].w);
    }
    m = fmaxf(m, absmax4(x[i]));
  }
  if (guard_ok(m)) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (i >= np) break;
      const int off = (t + 256 * i) * 16;
      float4 h, l;
      split4<false>(x[i], h, l);
      *reinterpret_cast<float4*>(dst_hi + off) = h;
      *reinterpret_cast<float4*>(dst_lo + off) = l;
    }
  } else {
#pragma unroll  // (a rolled loop would index x dynamically and push it to local memory)
    for (int i = 0; i < 4; ++i) {
      if (i >= np) break;
      const int off = (t + 256 * i) * 16;
      float4 h, l;
      split4<true>(x[i], h, l);
      *reinterpret_cast<float4*>(dst_hi + off) = h;
      *reinterpret_cast<float4*>(dst_lo + off) = l;
    }
  }
}

// Transform of an outer-contiguous raw slice [atom][k][32 outer] (four unswizzled TMA boxes):
// thread t owns outer index t % 128 and half of the 32 k values, reads them with
// conflict-free scalar loads (lanes = consecutive outer indices) and writes the transposed,
// swizzled K-major chunks.  Returns the sum of the values it handled (bias gradient).
template <bool HAS_Y>
__device__ __forceinline__ float transform_oc(const uint8_t* src, const uint8_t* ysrc,
                                              uint8_t* dst_hi, uint8_t* dst_lo, int t, int dact,
                                              int rows = 128) {
  const int o = t & 127;
  if (o >= rows) return 0.f;  // a 64-row slice: the other rows of the tile do not exist
  const int kbase = (t >> 7) * 16;
  const float* col = reinterpret_cast<const float*>(src + (o >> 5) * 4096) + (o & 31);
  const float* ycol = reinterpret_cast<const float*>(ysrc + (o >> 5) * 4096) + (o & 31);
  float sum = 0.f, m = 0.f;
  float4 x[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    float v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      v[e] = col[(kbase + 4 * c + e) * 32];
      if (HAS_Y) v[e] = act_backward<float>(dact, ycol[(kbase + 4 * c + e) * 32], v[e]);
    }
    sum += (v[0] + v[1]) + (v[2] + v[3]);
    x[c] = make_float4(v[0], v[1], v[2], v[3]);
    m = fmaxf(m, absmax4(x[c]));
  }
  if (guard_ok(m)) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float4 h, l;
      split4<false>(x[c], h, l);
      const uint32_t off = sw128_offset(o, (kbase >> 2) + c);
      *reinterpret_cast<float4*>(dst_hi + off) = h;
      *reinterpret_cast<float4*>(dst_lo + off) = l;
    }
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float4 h, l;
      split4<true>(x[c], h, l);
      const uint32_t off = sw128_offset(o, (kbase >> 2) + c);
      *reinterpret_cast<float4*>(dst_hi + off) = h;
      *reinterpret_cast<float4*>(dst_lo + off) = l;
    }
  }
  return sum;
}

// PERSISTENT: the CTA walks tiles blockIdx.x, + gridDim.x, ...; otherwise it serves exactly one
// (the loops below then run once and compile to straight-line code, which the long-tile launches
// need: the walking form cost them 3-5 %).
template <bool PERSISTENT>
__global__ void __launch_bounds__(NTHREADS, 1)
sgemm3x_tma_kernel(const __grid_constant__ SParams p, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t raw_full[3];
  __shared__ __align__(8) uint64_t raw_empty[3];
  __shared__ __align__(8) uint64_t plane_full[PLANE_STAGES];
  __shared__ __align__(8) uint64_t plane_empty[PLANE_STAGES];
  __shared__ __align__(8) uint64_t acc_full;
  __shared__ __align__(8) uint64_t acc_empty;
  __shared__ uint32_t tmem_slot;
#ifdef GB_PHASE_TIMES  // instrumented build (-DGB_PHASE_TIMES): CTA 0 prints its phase durations
  __shared__ long long ph_t[12];
  if (threadIdx.x == 0) ph_t[0] = clock64();
#define PH(i) do { ph_t[i] = clock64(); } while (0)
#else
#define PH(i) do { } while (0)
#endif

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t planes_base = base;                               // PLANE_STAGES * 64 KiB
  const uint32_t raws_base = base + PLANE_STAGES * PLANE_STAGE;    // 96 KiB
  const int raw_stages = p.dop ? 2 : 3;
  const int raw_stage_bytes = p.dop ? 3 * RAW_TILE : 2 * RAW_TILE;

  // A CTA works through tiles blockIdx.x, blockIdx.x + gridDim.x, ...: the barriers, the raw and
  // plane rings and the tensor-memory allocation are set up once, the producer runs ahead into
  // the next tile's slices while this tile's accumulator is written out (one prologue and one
  // first round trip to memory per CTA instead of per tile: 6-7 of the ~17 thousand cycles a
  // two-k-block tile costs).
  int nkb_total = 0;
  for (int i = 0; i < p.npairs; ++i) nkb_total += (p.k[i] + SBK - 1) / SBK;
  struct Tile {
    int m0, n0, n_tile, batch, split, kb_begin, nkb;
  };
  auto decode = [&](int tile) {
    Tile t;
    const int m_tile = tile % p.tiles_m;
    tile /= p.tiles_m;
    t.n_tile = tile % p.tiles_n;
    tile /= p.tiles_n;
    t.batch = tile % p.batches;
    t.split = tile / p.batches;
    t.m0 = m_tile * SBM;
    t.n0 = t.n_tile * p.bn;
    // k-blocks [kb_begin, kb_begin + nkb) belong to this tile (single pair when split)
    t.kb_begin = static_cast<int>(static_cast<long long>(nkb_total) * t.split / p.split_k);
    t.nkb = static_cast<int>(static_cast<long long>(nkb_total) * (t.split + 1) / p.split_k) - t.kb_begin;
    return t;
  };

  if (warp == 0 && lane == 0) {
    for (int i = 0; i < p.npairs; ++i) {
      prefetch_tmap(&p.tmA[i]);
      prefetch_tmap(&p.tmB[i]);
    }
    if (p.dop) prefetch_tmap(&p.tmY);
  }
  if (warp == 1) {
    if (lane == 0) {
      for (int s = 0; s < 3; ++s) {
        mbar_init(smem_u32(&raw_full[s]), 1);
        mbar_init(smem_u32(&raw_empty[s]), XFORM_THREADS);
      }
      for (int s = 0; s < PLANE_STAGES; ++s) {
        mbar_init(smem_u32(&plane_full[s]), XFORM_THREADS);
        mbar_init(smem_u32(&plane_empty[s]), 1);
      }
      mbar_init(smem_u32(&acc_full), 1);
      mbar_init(smem_u32(&acc_empty), XFORM_THREADS);
      fence_mbar_init();
    }
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  // Everything above touched only shared and tensor memory; from here on the kernel reads what
  // its predecessor in the stream may have written.
  if (threadIdx.x == 0) PH(1);
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x == 0) PH(2);

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
      const Tile tl = decode(tile);
      const int m0 = tl.m0, n0 = tl.n0, batch = tl.batch, nkb = tl.nkb;
      int pair = 0, k0 = tl.kb_begin * SBK;
      for (int it = 0; it < nkb; ++it) {
        if (!mbar_wait(smem_u32(&raw_empty[s]), ph ^ 1u, status, DEV_TIMEOUT_EMPTY, it)) {
          ok = false;
          break;
        }
        const uint32_t bar = smem_u32(&raw_full[s]);
        const uint32_t dst = raws_base + s * raw_stage_bytes;
        // bytes of this stage: A (and a derivative partner of A) always 128 rows, B (and its
        // partner) p.bn rows of 128 bytes
        const int b_bytes = p.bn * 128;
        mbar_arrive_expect_tx(bar, RAW_TILE + b_bytes + (p.dop == 1 ? RAW_TILE : p.dop == 2 ? b_bytes : 0));
        // k-contiguous operand: one 32(k) x 128(outer) box, 128-byte swizzle (32 x bn for B).
        // outer-contiguous operand: boxes of 32(outer) x 32(k), unswizzled.
        if (p.a_kc[pair]) {
          tma_load_3d(dst, &p.tmA[pair], bar, k0, m0, batch);
        } else {
#pragma unroll
          for (int a = 0; a < 4; ++a)
            tma_load_3d(dst + a * 4096, &p.tmA[pair], bar, m0 + 32 * a, k0, batch);
        }
        if (p.b_kc[pair]) {
          tma_load_3d(dst + RAW_TILE, &p.tmB[pair], bar, k0, n0, batch);
        } else {
#pragma unroll
          for (int a = 0; a < 4; ++a)
            if (32 * a < p.bn)
              tma_load_3d(dst + RAW_TILE + a * 4096, &p.tmB[pair], bar, n0 + 32 * a, k0, batch);
        }
        if (p.dop) {
          const int kc = p.dop == 1 ? p.a_kc[0] : p.b_kc[0];
          const int o0 = p.dop == 1 ? m0 : n0;
          const int orows = p.dop == 1 ? SBM : p.bn;
          if (kc) {
            tma_load_3d(dst + 2 * RAW_TILE, &p.tmY, bar, k0, o0, batch);
          } else {
#pragma unroll
            for (int a = 0; a < 4; ++a)
              if (32 * a < orows)
                tma_load_3d(dst + 2 * RAW_TILE + a * 4096, &p.tmY, bar, o0 + 32 * a, k0, batch);
          }
        }
        if (++s == raw_stages) {
          s = 0;
          ph ^= 1u;
        }
        k0 += SBK;
        if (k0 >= p.k[pair]) {
          ++pair;
          k0 = 0;
        }
      }
      if (!PERSISTENT) break;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (elect_one()) {
      const uint32_t IDESC = make_idesc(2, 0, 0, SBM, static_cast<uint32_t>(p.bn));
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int local = 0;  // tiles this CTA has started
      for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, ++local) {
      const int nkb = decode(tile).nkb;
      // the epilogue of the previous tile has read the accumulators
      if (PERSISTENT && local > 0 &&
          !mbar_wait(smem_u32(&acc_empty), (local - 1) & 1u, status, DEV_TIMEOUT_TMEM_FREE, local)) {
        ok = false;
        break;
      }
      tc_fence_after();
      for (int it = 0; it < nkb; ++it) {
        if (!mbar_wait(smem_u32(&plane_full[s]), ph, status, DEV_TIMEOUT_FULL, it)) {
          ok = false;
          break;
        }
        if (it == 0) PH(4);
        tc_fence_after();
        const uint32_t a_hi = planes_base + s * PLANE_STAGE;
        const uint32_t a_lo = a_hi + PLANE;
        const uint32_t b_hi = a_hi + 2 * PLANE;
        const uint32_t b_lo = a_hi + 3 * PLANE;
        const uint32_t d_main = tmem + (it % 3) * SBN;
        const uint32_t d_cross = tmem + CROSS_COL;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t dah = make_smem_desc(a_hi + ks * 32, 16, 1024);
          const uint64_t dal = make_smem_desc(a_lo + ks * 32, 16, 1024);
          const uint64_t dbh = make_smem_desc(b_hi + ks * 32, 16, 1024);
          const uint64_t dbl = make_smem_desc(b_lo + ks * 32, 16, 1024);
          mma_tf32(d_cross, dal, dbh, IDESC, (it > 0 || ks > 0) ? 1u : 0u);
          mma_tf32(d_cross, dah, dbl, IDESC, 1u);
          mma_tf32(d_main, dah, dbh, IDESC, (it >= 3 || ks > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&plane_empty[s]));
        if (++s == PLANE_STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
      if (ok) tc_commit(smem_u32(&acc_full));
      PH(5);
      if (!PERSISTENT) break;
      }
    }
    __syncwarp();
  } else {
    // ===================== transform (warps 2-9: A, warps 10-17: B) =====================
    const int xt = threadIdx.x - 64;
    const int grp = xt >> 8;  // 0 = A operand, 1 = B operand
    const int t = xt & 255;
    bool ok = true;
    int rs_i = 0, ps_i = 0;
    uint32_t rph = 0, pph = 0;
    int local = 0;  // tiles this CTA has started
    for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, ++local) {
    const Tile tl = decode(tile);
    const int m0 = tl.m0, n0 = tl.n0, batch = tl.batch, split = tl.split, nkb = tl.nkb;
    const bool want_rowsum = grp == 0 && p.rowsum != nullptr && tl.n_tile == 0;
    float rs = 0.f;
    int pair = 0, k0 = tl.kb_begin * SBK;
    for (int it = 0; it < nkb; ++it) {
      if (!mbar_wait(smem_u32(&raw_full[rs_i]), rph, status, DEV_TIMEOUT_FULL, 0x100 + it) ||
          !mbar_wait(smem_u32(&plane_empty[ps_i]), pph ^ 1u, status, DEV_TIMEOUT_EMPTY,
                     0x100 + it)) {
        ok = false;
        break;
      }
      if (it == 0 && threadIdx.x == 64) PH(3);
      const uint8_t* raw_stage = base_ptr + PLANE_STAGES * PLANE_STAGE + rs_i * raw_stage_bytes;
      const uint8_t* src = raw_stage + grp * RAW_TILE;
      const uint8_t* ysrc = raw_stage + 2 * RAW_TILE;
      uint8_t* dst_hi = base_ptr + ps_i * PLANE_STAGE + grp * 2 * PLANE;
      uint8_t* dst_lo = dst_hi + PLANE;
      const int kc = grp ? p.b_kc[pair] : p.a_kc[pair];
      const bool has_y = p.dop == grp + 1;
      const int rows = grp ? p.bn : SBM;
      if (kc) {
        if (has_y)
          transform_kc<true>(src, ysrc, dst_hi, dst_lo, t, p.dact, rows);
        else
          transform_kc<false>(src, ysrc, dst_hi, dst_lo, t, p.dact, rows);
      } else {
        const float part = has_y ? transform_oc<true>(src, ysrc, dst_hi, dst_lo, t, p.dact, rows)
                                 : transform_oc<false>(src, ysrc, dst_hi, dst_lo, t, p.dact, rows);
        if (want_rowsum && pair == 0) rs += part;
      }
      // (One elected arrival per warp after a warp barrier was measured: 7 % slower than every
      // thread arriving for itself.)
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&plane_full[ps_i]));
      mbar_arrive(smem_u32(&raw_empty[rs_i]));
      if (++rs_i == raw_stages) {
        rs_i = 0;
        rph ^= 1u;
      }
      if (++ps_i == PLANE_STAGES) {
        ps_i = 0;
        pph ^= 1u;
      }
      k0 += SBK;
      if (k0 >= p.k[pair]) {
        ++pair;
        k0 = 0;
      }
    }
    // two threads share a row (one per k half): both add their part
    if (want_rowsum && ok && m0 + (t & 127) < p.M) atomicAdd(p.rowsum + m0 + (t & 127), rs);

    // ===================== epilogue (all sixteen warps; 32 columns each) =====================
    const int q = warp & 3;
    const int cgrp = (warp - 2) >> 2;  // 0..3
    const int row = m0 + q * 32 + lane;
    const bool row_ok = row < p.M;
    // fetched before the wait for the accumulator, so that its latency hides behind the MMAs
    const float bias = (p.bias != nullptr && row_ok && split == 0) ? p.bias[row] : 0.f;  // once per tile
    const bool epi_ok =
        ok && mbar_wait(smem_u32(&acc_full), local & 1u, status, DEV_TIMEOUT_ACCUM, local);
    if (threadIdx.x == 64) PH(6);
    float* crow = p.C + static_cast<long long>(batch) * p.strideC + row * p.c_rs;
    const int c0 = cgrp * 32;
    const bool split_k = p.split_k > 1;
    if (epi_ok) {
      tc_fence_after();
      const uint32_t tbase = tmem + (static_cast<uint32_t>(q * 32) << 16) + c0;
      const long long ldc = p.c_cs;  // distance between consecutive columns of the result
      const int mode = split_k ? 2 : (p.accumulate ? 1 : 0);
      const int act = p.act;  // none when the contraction is split: a pass over C follows
      // columns of this warp's group that exist (may be <= 0): inside the matrix and the tile
      const int ncols = (p.N - n0 < p.bn ? p.N - n0 : p.bn) - c0;
      float* dst = crow + static_cast<long long>(n0 + c0) * ldc;
      // eight columns per pass, not unrolled (code size: a CTA runs this once, from a cold
      // instruction cache); the per-element work is a pointer increment, an add and a store.
      // (Issuing the next pass's tensor-memory loads ahead of this pass's stores was tried and
      // made a pass half as long again.)
#pragma unroll 1
      for (int c = 0; c < 32 && c < ncols; c += 8, dst += 8 * ldc) {
        float acc[8];
        load_acc8(tbase + c, nkb, acc);
        if (row_ok) {
          if (ncols - c >= 8)
            store_acc8<true>(dst, ldc, 8, acc, bias, mode, act);
          else
            store_acc8<false>(dst, ldc, ncols - c, acc, bias, mode, act);
        }
      }
    }
    if (threadIdx.x == 64) PH(7);
    if (!PERSISTENT || !epi_ok) break;
    // this thread has read its part of the accumulators: the next tile's MMAs may overwrite them
    tc_fence_before();
    mbar_arrive(smem_u32(&acc_empty));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
#ifdef GB_PHASE_TIMES
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const long long t9 = clock64();
    printf("phase cycles: prologue %lld pdl_wait %lld first_raw %lld first_plane %lld mma_issued %lld "
           "acc_ready %lld epilogue %lld exit %lld  (nkb %d)\n",
           ph_t[1] - ph_t[0], ph_t[2] - ph_t[1], ph_t[3] - ph_t[2], ph_t[4] - ph_t[3],
           ph_t[5] - ph_t[4], ph_t[6] - ph_t[5], ph_t[7] - ph_t[6], t9 - ph_t[7], nkb);
  }
#endif
}


// ===========================================================================================
// Operands split once in HBM.  A large product re-reads every operand slice from many tiles (a
// row panel of A from every column tile, a column panel of B from every row tile) and the kernel
// above splits it into hi and lo planes again each time: that transform, not the tensor pipe,
// bounds it.  For products with at least four tiles along both extents the launcher therefore
// splits both operands ONCE, into K-major hi / lo planes in a stream-ordered scratch allocation
// (rows padded with zeros to a multiple of 32 along the contraction), and runs the kernel below,
// whose producer lets TMA drop the four planes of a k-block straight into the layout the MMA
// descriptors read: no transform warps, three 64 KiB stages.  The derivative of a fused
// nonlinearity is applied by the split pass.
// ===========================================================================================
constexpr int PRE_STAGES = 3;

// Both operands X(o, kk) (see Operand) -> hi[o * kp + kk], lo[o * kp + kk] in one launch:
// blockIdx.z = operand, blockIdx.x = 32-wide tile along o, blockIdx.y = along kk; 256 threads,
// 16 bytes each way per thread.  Bases are 16-byte aligned and leading dimensions multiples of
// four elements (what the tensor maps of the unsplit path need as well).
struct SplitJob {
  const float* base;
  const float* ybase;
  long long ld;
  int k_contig, dact, O;
  float* hi;
  float* lo;
};
struct SplitJobs {
  SplitJob op[2];
  int K, kp;
  float* rowsum;  // when set: rowsum[o] += sum over kk of operand 0 (outer-contiguous only)
};

__device__ __forceinline__ float4 load4_guarded(const float* p0, int valid) {
  if (valid >= 4) return *reinterpret_cast<const float4*>(p0);
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (valid > 0) v.x = p0[0];
  if (valid > 1) v.y = p0[1];
  if (valid > 2) v.z = p0[2];
  return v;
}

__global__ void __launch_bounds__(256)
presplit_kernel(const SplitJobs jobs) {
  __shared__ float th[32][33], tl[32][33];
  // field by field: indexing the parameter with blockIdx.z would copy it to local memory
  const bool second = blockIdx.z != 0;
  SplitJob jb;
  jb.base = second ? jobs.op[1].base : jobs.op[0].base;
  jb.ybase = second ? jobs.op[1].ybase : jobs.op[0].ybase;
  jb.ld = second ? jobs.op[1].ld : jobs.op[0].ld;
  jb.k_contig = second ? jobs.op[1].k_contig : jobs.op[0].k_contig;
  jb.dact = second ? jobs.op[1].dact : jobs.op[0].dact;
  jb.O = second ? jobs.op[1].O : jobs.op[0].O;
  jb.hi = second ? jobs.op[1].hi : jobs.op[0].hi;
  jb.lo = second ? jobs.op[1].lo : jobs.op[0].lo;
  const int o0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  if (o0 >= jb.O) return;
  const int q = threadIdx.x & 7, r = threadIdx.x >> 3;  // 8 quads x 32 rows
  const int K = jobs.K, kp = jobs.kp;
  pdl_wait();
  if (jb.k_contig) {
    const int o = o0 + r, kk = k0 + 4 * q;
    if (o >= jb.O) return;
    const long long off = static_cast<long long>(o) * jb.ld + kk;
    float4 v = load4_guarded(jb.base + off, K - kk);
    if (jb.ybase) {
      const float4 y = load4_guarded(jb.ybase + off, K - kk);
      v.x = act_backward<float>(jb.dact, y.x, v.x);
      v.y = act_backward<float>(jb.dact, y.y, v.y);
      v.z = act_backward<float>(jb.dact, y.z, v.z);
      v.w = act_backward<float>(jb.dact, y.w, v.w);
      // beyond K the planes must hold zeros whatever act'(0) is
      if (K - kk < 4) {
        if (K - kk < 1) v.x = 0.f;
        if (K - kk < 2) v.y = 0.f;
        if (K - kk < 3) v.z = 0.f;
        v.w = 0.f;
      }
    }
    float4 h, l;
    split4<true>(v, h, l);
    *reinterpret_cast<float4*>(jb.hi + static_cast<long long>(o) * kp + kk) = h;
    *reinterpret_cast<float4*>(jb.lo + static_cast<long long>(o) * kp + kk) = l;
  } else {
    {
      const int kk = k0 + r, o = o0 + 4 * q;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (kk < K) {
        const long long off = static_cast<long long>(kk) * jb.ld + o;
        v = load4_guarded(jb.base + off, jb.O - o);
        if (jb.ybase) {
          const float4 y = load4_guarded(jb.ybase + off, jb.O - o);
          v.x = act_backward<float>(jb.dact, y.x, v.x);
          v.y = act_backward<float>(jb.dact, y.y, v.y);
          v.z = act_backward<float>(jb.dact, y.z, v.z);
          v.w = act_backward<float>(jb.dact, y.w, v.w);
        }
      }
      float4 h, l;
      split4<true>(v, h, l);
      th[r][4 * q] = h.x; th[r][4 * q + 1] = h.y; th[r][4 * q + 2] = h.z; th[r][4 * q + 3] = h.w;
      tl[r][4 * q] = l.x; tl[r][4 * q + 1] = l.y; tl[r][4 * q + 2] = l.z; tl[r][4 * q + 3] = l.w;
    }
    __syncthreads();
    const int o = o0 + r, kk = k0 + 4 * q;
    // rows of the tile beyond K were filled with zeros above
    const float4 h = make_float4(th[4 * q][r], th[4 * q + 1][r], th[4 * q + 2][r], th[4 * q + 3][r]);
    const float4 l = make_float4(tl[4 * q][r], tl[4 * q + 1][r], tl[4 * q + 2][r], tl[4 * q + 3][r]);
    if (!second && jobs.rowsum != nullptr) {
      // hi + lo is the value itself; the eight threads of a row add up their quads
      float part = (h.x + l.x) + (h.y + l.y) + (h.z + l.z) + (h.w + l.w);
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      part += __shfl_xor_sync(0xffffffffu, part, 4);
      if (q == 0 && o < jb.O) atomicAdd(jobs.rowsum + o, part);
    }
    if (o >= jb.O) return;
    *reinterpret_cast<float4*>(jb.hi + static_cast<long long>(o) * kp + kk) = h;
    *reinterpret_cast<float4*>(jb.lo + static_cast<long long>(o) * kp + kk) = l;
  }
}

// C tile = A_hi B_hi + (A_hi B_lo + A_lo B_hi) from planes TMA loads directly; p.tmA[0] / [1]
// describe A's hi / lo planes, p.tmB[0] / [1] B's; one CTA per tile and part of the contraction
// (p.split_k parts: partial sums are added atomically, as in the kernel above), one pair.
// Warp 0: producer, warp 1: MMA issuer, warps 2-17: epilogue (as in sgemm3x_tma_kernel).
__global__ void __launch_bounds__(NTHREADS, 1)
sgemm3x_pre_kernel(const __grid_constant__ SParams p, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full[PRE_STAGES];
  __shared__ __align__(8) uint64_t empty[PRE_STAGES];
  __shared__ __align__(8) uint64_t acc_full;
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int tiles = p.tiles_m * p.tiles_n;
  const int tile = static_cast<int>(blockIdx.x) % tiles;
  const int split = static_cast<int>(blockIdx.x) / tiles;  // part of the contraction (p.split_k parts)
  const int m0 = (tile % p.tiles_m) * SBM;
  const int n0 = (tile / p.tiles_m) * p.bn;
  const int nkb_total = (p.k[0] + SBK - 1) / SBK;
  const int kb_begin = static_cast<int>(static_cast<long long>(nkb_total) * split / p.split_k);
  const int nkb =
      static_cast<int>(static_cast<long long>(nkb_total) * (split + 1) / p.split_k) - kb_begin;

  if (warp == 0 && lane == 0) {
    prefetch_tmap(&p.tmA[0]);
    prefetch_tmap(&p.tmA[1]);
    prefetch_tmap(&p.tmB[0]);
    prefetch_tmap(&p.tmB[1]);
  }
  if (warp == 1) {
    if (lane == 0) {
      for (int s = 0; s < PRE_STAGES; ++s) {
        mbar_init(smem_u32(&full[s]), 1);
        mbar_init(smem_u32(&empty[s]), 1);
      }
      mbar_init(smem_u32(&acc_full), 1);
      fence_mbar_init();
    }
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  pdl_wait();  // the planes are written by the launches before this one
  pdl_launch_dependents();

  bool ok = true;
  if (warp == 0) {
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      const int b_bytes = p.bn * 128;
      for (int it = 0; it < nkb; ++it) {
        if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1u, status, DEV_TIMEOUT_EMPTY, it)) break;
        const uint32_t bar = smem_u32(&full[s]);
        const uint32_t dst = base + s * PLANE_STAGE;
        mbar_arrive_expect_tx(bar, 2 * RAW_TILE + 2 * b_bytes);
        const int k0 = (kb_begin + it) * SBK;
        tma_load_3d(dst, &p.tmA[0], bar, k0, m0, 0);
        tma_load_3d(dst + PLANE, &p.tmA[1], bar, k0, m0, 0);
        tma_load_3d(dst + 2 * PLANE, &p.tmB[0], bar, k0, n0, 0);
        tma_load_3d(dst + 3 * PLANE, &p.tmB[1], bar, k0, n0, 0);
        if (++s == PRE_STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t IDESC = make_idesc(2, 0, 0, SBM, static_cast<uint32_t>(p.bn));
      int s = 0;
      uint32_t ph = 0;
      bool mok = true;
      for (int it = 0; it < nkb; ++it) {
        if (!mbar_wait(smem_u32(&full[s]), ph, status, DEV_TIMEOUT_FULL, it)) {
          mok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_hi = base + s * PLANE_STAGE;
        const uint32_t a_lo = a_hi + PLANE;
        const uint32_t b_hi = a_hi + 2 * PLANE;
        const uint32_t b_lo = a_hi + 3 * PLANE;
        const uint32_t d_main = tmem + (it % 3) * SBN;
        const uint32_t d_cross = tmem + CROSS_COL;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t dah = make_smem_desc(a_hi + ks * 32, 16, 1024);
          const uint64_t dal = make_smem_desc(a_lo + ks * 32, 16, 1024);
          const uint64_t dbh = make_smem_desc(b_hi + ks * 32, 16, 1024);
          const uint64_t dbl = make_smem_desc(b_lo + ks * 32, 16, 1024);
          mma_tf32(d_cross, dal, dbh, IDESC, (it > 0 || ks > 0) ? 1u : 0u);
          mma_tf32(d_cross, dah, dbl, IDESC, 1u);
          mma_tf32(d_main, dah, dbh, IDESC, (it >= 3 || ks > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&empty[s]));
        if (++s == PRE_STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
      if (mok) tc_commit(smem_u32(&acc_full));
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    const int cgrp = (warp - 2) >> 2;  // 0..3
    const int row = m0 + q * 32 + lane;
    const bool row_ok = row < p.M;
    const float bias = (p.bias != nullptr && row_ok && split == 0) ? p.bias[row] : 0.f;
    ok = mbar_wait(smem_u32(&acc_full), 0u, status, DEV_TIMEOUT_ACCUM, 0);
    if (ok) {
      tc_fence_after();
      const int c0 = cgrp * 32;
      const uint32_t tbase = tmem + (static_cast<uint32_t>(q * 32) << 16) + c0;
      const int mode = p.split_k > 1 ? 2 : (p.accumulate ? 1 : 0);  // 2: atomic partial sums
      const int ncols = (p.N - n0 < p.bn ? p.N - n0 : p.bn) - c0;
      float* dst = p.C + row + static_cast<long long>(n0 + c0) * p.ldc;
#pragma unroll 1
      for (int c = 0; c < 32 && c < ncols; c += 8, dst += 8 * p.ldc) {
        float acc[8];
        load_acc8(tbase + c, nkb, acc);
        if (row_ok) {
          if (ncols - c >= 8)
            store_acc8<true>(dst, p.ldc, 8, acc, bias, mode, p.act);
          else
            store_acc8<false>(dst, p.ldc, ncols - c, acc, bias, mode, p.act);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ===========================================================================================
// Gather front end: the same transform / MMA / epilogue pipeline, but the raw slices are
// brought in by the transform threads themselves with cp.async (4- or 16-byte pieces, zero
// filled outside the matrix) instead of TMA.  It takes what a tensor map cannot describe:
// unaligned bases and leading dimensions, and operands whose columns live at unrelated
// addresses (the per-node tensors of an autobatch level), and it reads its problem either from
// the kernel parameters or, for a grouped launch, from a device array of descriptors.
// ===========================================================================================
constexpr int GNTHREADS = 32 + XFORM_THREADS;  // warp 0: MMA issuer; warps 1-8: A; warps 9-16: B

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
// Arrive on `bar` once all cp.async issued so far by this thread have landed (the barrier's
// expected count already includes this arrival).
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// A 16-byte piece whose source is only 4-byte aligned: element by element.  Out of line: the
// fill loop has to stay short (its length is what bounds a k-block once the tensor core is fed).
__device__ __noinline__ void fill_piece_slow(uint32_t dst, const float* src, int valid,
                                             const void* safe) {
#pragma unroll
  for (int e = 0; e < 4; ++e)
    cp_async4(dst + 4 * e, e < valid ? static_cast<const void*>(src + e) : safe, e < valid ? 4 : 0);
}

// 16 bytes (4 floats) from src to dst, of which `valid` (0..4) elements exist; the rest is zero.
__device__ __forceinline__ void fill_piece(uint32_t dst, const float* src, int valid,
                                           const void* safe) {
  if (valid > 0 && (reinterpret_cast<uintptr_t>(src) & 15u) != 0)
    fill_piece_slow(dst, src, valid, safe);
  else
    cp_async16(dst, valid > 0 ? static_cast<const void*>(src) : safe, valid * 4);
}

// Per-thread geometry of one raw slice (128 outer x 32 k) of an operand, in the two layouts the
// TMA front end produces, worked out once per (tile, pair) and kept in registers: the copies'
// "memory" clobbers would otherwise force every operand field to be re-read before each piece.
//   k-contiguous : piece i = row (t/8 + 32 i), k offset 4 (t%8)    -> offset off0 + 4096 i
//   outer-contig.: piece i = k (t/32 + 8 i), outer offset 4 (t%32) -> offset off0 + 1024 i
struct RawFeeder {
  const void* const* cols;
  const float* p0;    // untabled: element of piece 0 at k = 0
  const void* safe;
  long long ld, K;
  uint32_t off0;
  int o_first, O, sub, valid_o;
  bool kc;

  __device__ __forceinline__ void init(const Operand& op, bool y, long long boff, int o0, int O_,
                                       long long K_, int t) {
    const float* base = static_cast<const float*>(y ? op.ybase : op.base);
    cols = y ? op.ycols : op.cols;
    safe = cols ? static_cast<const void*>(cols) : static_cast<const void*>(base);
    ld = op.ld;
    K = K_;
    O = O_;
    kc = op.k_contig != 0;
    p0 = nullptr;
    if (kc) {
      sub = t & 7;
      const int row0 = t >> 3;
      off0 = sw128_offset(row0, sub);
      o_first = o0 + row0;
      valid_o = 4;
      if (!cols) p0 = base + boff + static_cast<long long>(o_first) * ld + 4 * sub;
    } else {
      sub = t >> 5;
      const int oc = t & 31;
      off0 = (oc >> 3) * 4096u + sub * 128u + (oc & 7) * 16u;
      o_first = o0 + 4 * oc;
      valid_o = O_ - o_first >= 4 ? 4 : (O_ - o_first > 0 ? O_ - o_first : 0);
      if (!cols) p0 = base + boff + o_first;
    }
  }

  __device__ __forceinline__ void fill(uint32_t dst_tile, long long k0) const {
    uint32_t d = dst_tile + off0;
    if (kc) {
      const long long kk = k0 + 4 * sub;
      const int kv = K - kk >= 4 ? 4 : (K - kk > 0 ? static_cast<int>(K - kk) : 0);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int o = o_first + 32 * i;
        const int valid = o < O ? kv : 0;
        const float* src = nullptr;
        if (valid > 0)
          src = cols ? static_cast<const float*>(cols[o]) + kk : p0 + static_cast<long long>(32 * i) * ld + k0;
        fill_piece(d, src, valid, safe);
        d += 4096u;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const long long kk = k0 + sub + 8 * i;
        const int valid = kk < K ? valid_o : 0;
        const float* src = nullptr;
        if (valid > 0) src = cols ? static_cast<const float*>(cols[kk]) + o_first : p0 + kk * ld;
        fill_piece(d, src, valid, safe);
        d += 1024u;
      }
    }
  }
};

// WITH_Y: the instantiation that can take a derivative operand.  Grouped levels never have one
// (autobatch merges identity Affines only) and most single products do not either; leaving the
// second feeder and the derivative transforms out makes their kernel a fifth smaller, which is
// run time for tiles of a few k-blocks (the code is fetched once per CTA, cold).
template <bool GROUPED, bool WITH_Y>
__global__ void __launch_bounds__(GNTHREADS, 1)
sgemm3x_gather_kernel(const __grid_constant__ Problem p0, const Problem* __restrict__ probs,
                      int nprobs, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t raw_full[2][3];   // [operand group][stage]: slice landed
  __shared__ __align__(8) uint64_t raw_empty[2][3];  // [operand group][stage]: slice consumed
  __shared__ __align__(8) uint64_t plane_full[PLANE_STAGES];
  __shared__ __align__(8) uint64_t plane_empty[PLANE_STAGES];
  __shared__ __align__(8) uint64_t acc_full;
  __shared__ uint32_t tmem_slot;
  __shared__ Problem sprob;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t planes_base = base;
  const uint32_t raws_base = base + PLANE_STAGES * PLANE_STAGE;

  // Barrier set-up and the TMEM allocation need nothing from global memory: they run before
  // the wait for the preceding kernel.
  if (warp == 0) {
    if (lane == 0) {
      for (int g = 0; g < 2; ++g)
        for (int s = 0; s < 3; ++s) {
          mbar_init(smem_u32(&raw_full[g][s]), 256);
          mbar_init(smem_u32(&raw_empty[g][s]), 256);
        }
      for (int s = 0; s < PLANE_STAGES; ++s) {
        mbar_init(smem_u32(&plane_full[s]), XFORM_THREADS);
        mbar_init(smem_u32(&plane_empty[s]), 1);
      }
      mbar_init(smem_u32(&acc_full), 1);
      fence_mbar_init();
    }
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
    tc_fence_before();
  }
  pdl_wait();
  pdl_launch_dependents();

  int tile = blockIdx.x;
  if (GROUPED) {
    int g = 0;
    for (int i = 0; i < nprobs; ++i)
      if (tile >= probs[i].tile_start) g = i;
    const int nwords = sizeof(Problem) / 4;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(probs + g);
    uint32_t* dst = reinterpret_cast<uint32_t*>(&sprob);
    for (int i = threadIdx.x; i < nwords; i += blockDim.x) dst[i] = src[i];
    __syncthreads();
  }
  const Problem& P = GROUPED ? sprob : p0;
  tile -= P.tile_start;
  const int m_tile = tile % P.tiles_m;
  int rest = tile / P.tiles_m;
  const int n_tile = rest % P.tiles_n;
  rest /= P.tiles_n;
  const long long batch = rest % P.batches;
  const int split = rest / P.batches;
  const int nsplit = P.split_k > 1 ? P.split_k : 1;
  const int m0 = m_tile * SBM, n0 = n_tile * SBN;

  int nkb_total = 0;
  for (int i = 0; i < P.npairs; ++i) nkb_total += static_cast<int>((P.k[i] + SBK - 1) / SBK);
  const int kb_begin = static_cast<int>(static_cast<long long>(nkb_total) * split / nsplit);
  const int nkb =
      static_cast<int>(static_cast<long long>(nkb_total) * (split + 1) / nsplit) - kb_begin;
  const int dop = !WITH_Y ? 0 : (P.a[0].dact != ACT_NONE ? 1 : (P.b[0].dact != ACT_NONE ? 2 : 0));
  const int dact = dop == 1 ? P.a[0].dact : (dop == 2 ? P.b[0].dact : ACT_NONE);
  const int raw_stages = dop ? 2 : 3;
  const int raw_stage_bytes = dop ? 3 * RAW_TILE : 2 * RAW_TILE;

  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 0) {
    // ===================== MMA issuer =====================
    if (elect_one()) {
      constexpr uint32_t IDESC = make_idesc(2, 0, 0, SBM, SBN);
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0; it < nkb; ++it) {
        if (!mbar_wait(smem_u32(&plane_full[s]), ph, status, DEV_TIMEOUT_FULL, it)) break;
        tc_fence_after();
        const uint32_t a_hi = planes_base + s * PLANE_STAGE;
        const uint32_t a_lo = a_hi + PLANE;
        const uint32_t b_hi = a_hi + 2 * PLANE;
        const uint32_t b_lo = a_hi + 3 * PLANE;
        const uint32_t d_main = tmem + (it % 3) * SBN;
        const uint32_t d_cross = tmem + CROSS_COL;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t dah = make_smem_desc(a_hi + ks * 32, 16, 1024);
          const uint64_t dal = make_smem_desc(a_lo + ks * 32, 16, 1024);
          const uint64_t dbh = make_smem_desc(b_hi + ks * 32, 16, 1024);
          const uint64_t dbl = make_smem_desc(b_lo + ks * 32, 16, 1024);
          mma_tf32(d_cross, dal, dbh, IDESC, (it > 0 || ks > 0) ? 1u : 0u);
          mma_tf32(d_cross, dah, dbl, IDESC, 1u);
          mma_tf32(d_main, dah, dbh, IDESC, (it >= 3 || ks > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&plane_empty[s]));
        if (++s == PLANE_STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
      tc_commit(smem_u32(&acc_full));
    }
    __syncwarp();
  } else {
    // ============ fill + transform (warps 1-8: A operand, warps 9-16: B operand) ============
    const int xt = threadIdx.x - 32;
    const int grp = xt >> 8;
    const int t = xt & 255;
    const int o0 = grp ? n0 : m0;
    const int O = grp ? P.N : P.M;
    const bool has_y = WITH_Y && dop == grp + 1;
    const bool want_rowsum = grp == 0 && P.rowsum != nullptr && n_tile == 0;
    float rs = 0.f;
    bool ok = true;

    // Fill side of the pipeline: k-blocks are filled in order, raw_stages - 1 ahead of the
    // transform; its position (pair, k0), ring stage and use count advance incrementally.
    RawFeeder fx, fy;
    int f_pair = 0, f_stage = 0;
    uint32_t f_use = 0;  // how often the ring has wrapped
    long long f_k0 = static_cast<long long>(kb_begin) * SBK;  // kb_begin > 0 only with one pair
    auto f_setup = [&]() {
      const Operand& op = grp ? P.b[f_pair] : P.a[f_pair];
      fx.init(op, false, batch * op.batch_stride, o0, O, P.k[f_pair], t);
      if (has_y) fy.init(op, true, batch * op.batch_stride, o0, O, P.k[f_pair], t);
    };
    if (nkb > 0) f_setup();
    auto fill = [&](int j) -> bool {
      if (!mbar_wait(smem_u32(&raw_empty[grp][f_stage]), (f_use & 1u) ^ 1u, status,
                     DEV_TIMEOUT_EMPTY, 0x300 + j))
        return false;
      const uint32_t dst = raws_base + f_stage * raw_stage_bytes;
      fx.fill(dst + grp * RAW_TILE, f_k0);
      if (has_y) fy.fill(dst + 2 * RAW_TILE, f_k0);
      cp_async_arrive(smem_u32(&raw_full[grp][f_stage]));
      if (++f_stage == raw_stages) {
        f_stage = 0;
        ++f_use;
      }
      f_k0 += SBK;
      if (f_k0 >= P.k[f_pair] && f_pair + 1 < P.npairs) {
        ++f_pair;
        f_k0 = 0;
        f_setup();
      }
      return true;
    };

    int rs_i = 0, ps_i = 0;
    uint32_t rph = 0, pph = 0;
    int pair = 0;
    long long k0 = static_cast<long long>(kb_begin) * SBK;  // kb_begin > 0 only with one pair
    // One loop, one copy of the fill code: step j fills k-block j and transforms k-block
    // j - (raw_stages - 1).
    for (int it = 1 - raw_stages; it < nkb; ++it) {
      const int ahead = it + raw_stages - 1;
      if (ok && ahead < nkb) ok = fill(ahead);
      if (it < 0) continue;
      if (!ok ||
          !mbar_wait(smem_u32(&raw_full[grp][rs_i]), rph, status, DEV_TIMEOUT_FULL, 0x200 + it) ||
          !mbar_wait(smem_u32(&plane_empty[ps_i]), pph ^ 1u, status, DEV_TIMEOUT_EMPTY,
                     0x200 + it)) {
        ok = false;
        break;
      }
      const uint8_t* raw_stage = base_ptr + PLANE_STAGES * PLANE_STAGE + rs_i * raw_stage_bytes;
      const uint8_t* src = raw_stage + grp * RAW_TILE;
      const uint8_t* ysrc = raw_stage + 2 * RAW_TILE;
      uint8_t* dst_hi = base_ptr + ps_i * PLANE_STAGE + grp * 2 * PLANE;
      uint8_t* dst_lo = dst_hi + PLANE;
      const int kc = grp ? P.b[pair].k_contig : P.a[pair].k_contig;
      if (kc) {
        if (has_y)
          transform_kc<true>(src, ysrc, dst_hi, dst_lo, t, dact);
        else
          transform_kc<false>(src, ysrc, dst_hi, dst_lo, t, dact);
      } else {
        const float part = has_y ? transform_oc<true>(src, ysrc, dst_hi, dst_lo, t, dact)
                                 : transform_oc<false>(src, ysrc, dst_hi, dst_lo, t, dact);
        if (want_rowsum && pair == 0) rs += part;
      }
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&plane_full[ps_i]));
      mbar_arrive(smem_u32(&raw_empty[grp][rs_i]));  // this thread is done reading the raw stage
      if (++rs_i == raw_stages) {
        rs_i = 0;
        rph ^= 1u;
      }
      if (++ps_i == PLANE_STAGES) {
        ps_i = 0;
        pph ^= 1u;
      }
      k0 += SBK;
      if (k0 >= P.k[pair]) {
        ++pair;
        k0 = 0;
      }
    }
    if (want_rowsum && ok && m0 + (t & 127) < P.M)
      atomicAdd(static_cast<float*>(P.rowsum) + m0 + (t & 127), rs);

    // ===================== epilogue (sixteen warps; 32 columns each) =====================
    const int q = warp & 3;
    const int c0 = ((warp - 1) >> 2) * 32;
    const int row = m0 + q * 32 + lane;
    const bool row_ok = row < P.M;
    // fetched before the wait for the accumulator, so that its latency hides behind the MMAs
    const float bias = (P.bias != nullptr && row_ok && split == 0)
                           ? static_cast<const float*>(P.bias)[row] : 0.f;  // once per tile
    if (ok && mbar_wait(smem_u32(&acc_full), 0, status, DEV_TIMEOUT_ACCUM, 0)) {
      tc_fence_after();
      const uint32_t tbase = tmem + (static_cast<uint32_t>(q * 32) << 16) + c0;
      const int mode = nsplit > 1 ? 2 : (P.accumulate ? 1 : 0);
      void* const* ccols = P.ccols;
      const long long ldc = P.ldc;
      const int act = P.act;
      const int ncols = P.N - (n0 + c0);
      float* dst = static_cast<float*>(P.c) + batch * P.c_batch_stride +
                   static_cast<long long>(n0 + c0) * ldc + row;
      // Eight columns per pass, not unrolled: a kernel that serves 2-k-block tiles runs its code
      // once per CTA, from a cold instruction cache.
#pragma unroll 1
      for (int c = 0; c < 32 && c < ncols; c += 8, dst += 8 * ldc) {
        float acc[8];
        load_acc8(tbase + c, nkb, acc);
        if (!row_ok) continue;
        if (ccols == nullptr) {
          if (ncols - c >= 8)
            store_acc8<true>(dst, ldc, 8, acc, bias, mode, act);
          else
            store_acc8<false>(dst, ldc, ncols - c, acc, bias, mode, act);
        } else {
          // every column at its own address: the table entries first, then the same three steps
          float* cp[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            cp[j] = c + j < ncols ? static_cast<float*>(ccols[n0 + c0 + c + j]) + row : nullptr;
          if (mode == 1) {
            float old[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) old[j] = cp[j] ? *cp[j] : 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += old[j];
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float v = acc[j] + bias;
            if (mode != 2 && act != ACT_NONE) v = act_forward_f32(act, v);
            if (cp[j]) {
              if (mode == 2)
                atomicAdd(cp[j], v);
              else
                *cp[j] = v;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

template <bool GROUPED, bool WITH_Y>
cudaError_t launch_gather(const Problem& p, const Problem* dprobs, int nprobs, int total_tiles,
                          cudaStream_t stream, int* status) {
  auto kern = sgemm3x_gather_kernel<GROUPED, WITH_Y>;
  const int smem = PLANE_STAGES * PLANE_STAGE + RAW_BYTES_TOTAL + 1024;
  static unsigned long long smem_set = 0;  // per template instantiation: per kernel
  cudaError_t e = set_smem_limit_once(reinterpret_cast<const void*>(kern), smem, &smem_set);
  if (e != cudaSuccess) return e;
  return launch_kernel(kern, dim3(total_tiles), dim3(GNTHREADS), smem, stream, pdl_enabled(), p,
                       dprobs, nprobs, status);
}

bool operand_tma_ok(const Operand& o, int batches) {
  if (o.cols != nullptr || o.ycols != nullptr) return false;
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  if (!al(o.base) || (o.ybase && !al(o.ybase))) return false;
  if (o.ld % 4 != 0) return false;
  if (batches > 1 && o.batch_stride % 4 != 0) return false;
  return true;
}

// Stored extents of operand X(outer O, inner K): k-contiguous -> K rows x O columns.
// `tile_outer` is the tile's extent along O: 128, or 64 for the B side of a narrow tile.
bool encode_operand(CUtensorMap* out, const void* ptr, const Operand& o, long long O, long long K,
                    int batches, int tile_outer = SBM) {
  const unsigned long long rows = o.k_contig ? K : O, cols = o.k_contig ? O : K;
  const unsigned long long bs = batches > 1 ? o.batch_stride : o.ld * cols;
  return encode_tmap(out, 4, ptr, rows, cols, batches, o.ld, bs ? bs : 4, 32,
                     o.k_contig ? tile_outer : SBK, o.k_contig != 0);
}

}  // namespace

// SM count of the current device (queried once per device).
static int device_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  int n = __atomic_load_n(&cached[dev], __ATOMIC_RELAXED);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    __atomic_store_n(&cached[dev], n, __ATOMIC_RELAXED);
  }
  return n;
}

bool sgemm3x_supported(const Problem& p) {
  if (p.npairs < 1 || p.ccols != nullptr || !tmap_encoder_available()) return false;
  int nderiv = 0;
  for (int i = 0; i < p.npairs; ++i) {
    if (p.k[i] <= 0 || p.k[i] > 0x7fffffffLL) return false;
    if (!operand_tma_ok(p.a[i], p.batches) || !operand_tma_ok(p.b[i], p.batches)) return false;
    nderiv += (p.a[i].dact != ACT_NONE) + (p.b[i].dact != ACT_NONE);
  }
  if (nderiv > 1 || (nderiv == 1 && p.npairs != 1)) return false;
  if (p.rowsum != nullptr && p.a[0].k_contig) return false;
  return true;
}

// Tile shape.  The tile is 128 rows of C by `bn` columns, bn = 64 when C has at most 64 columns
// (half of a 128-column tile would be computed and thrown away).  A plain product (no bias, row
// sums, activation or derivative operand) with at most 64 rows and more columns than that is run
// as its transpose, C^T = B^T A^T, the operands exchanged and the tile written through strides
// (ldc, 1): the short extent then lies along the 64-wide side.
// Operands split once (see sgemm3x_pre_kernel): a single unsplit product without a batch, a bias
// gradient or column tables, at least four tiles along both extents and a full wave of tiles, so
// that every plane is read several times and no SM idles for lack of a split contraction.
static bool presplit_wanted(const Problem& p) {
  if (!presplit_enabled() || p.npairs != 1 || p.batches != 1 || p.ccols != nullptr) return false;
  if (p.rowsum != nullptr && p.a[0].k_contig) return false;
  if (p.M < 4 * SBM || p.N < 4 * SBN || p.k[0] < 256 || p.k[0] > (1LL << 20)) return false;
  const long long tiles = static_cast<long long>((p.M + SBM - 1) / SBM) * ((p.N + SBN - 1) / SBN);
  const int split = p.split_k > 1 ? p.split_k : 1;
  // a full wave of tiles, or a split contraction long enough to pay for the split pass
  if (split == 1 ? tiles < device_sm_count() : (tiles * split * 2 < device_sm_count() || p.k[0] < 2048))
    return false;
  const long long kp = (p.k[0] + SBK - 1) / SBK * SBK;
  return 2 * (static_cast<long long>(p.M) + p.N) * kp * 4 <= (2LL << 30);  // scratch of at most 2 GiB
}

static cudaError_t launch_sgemm3x_pre(const Problem& p, cudaStream_t stream, int* status) {
  const long long K = p.k[0], kp = (K + SBK - 1) / SBK * SBK;
  const size_t a_plane = static_cast<size_t>(p.M) * kp * 4, b_plane = static_cast<size_t>(p.N) * kp * 4;
  void* ws = nullptr;
  cudaError_t e = cudaMallocAsync(&ws, 2 * (a_plane + b_plane), stream);
  if (e != cudaSuccess) return e;
  float* a_hi = static_cast<float*>(ws);
  float* a_lo = a_hi + a_plane / 4;
  float* b_hi = a_lo + a_plane / 4;
  float* b_lo = b_hi + b_plane / 4;
  {
    SplitJobs jobs;
    jobs.op[0] = SplitJob{static_cast<const float*>(p.a[0].base), static_cast<const float*>(p.a[0].ybase),
                          p.a[0].ld, p.a[0].k_contig, p.a[0].dact, p.M, a_hi, a_lo};
    jobs.op[1] = SplitJob{static_cast<const float*>(p.b[0].base), static_cast<const float*>(p.b[0].ybase),
                          p.b[0].ld, p.b[0].k_contig, p.b[0].dact, p.N, b_hi, b_lo};
    jobs.K = static_cast<int>(K);
    jobs.kp = static_cast<int>(kp);
    jobs.rowsum = static_cast<float*>(p.rowsum);
    const int omax = p.M > p.N ? p.M : p.N;
    const dim3 grid(static_cast<unsigned>((omax + 31) / 32), static_cast<unsigned>(kp / 32), 2);
    e = launch_kernel(presplit_kernel, grid, dim3(256), 0, stream, pdl_enabled(), jobs);
  }
  SParams sp;
  std::memset(&sp, 0, sizeof(sp));
  if (e == cudaSuccess) {
    const unsigned long long ukp = static_cast<unsigned long long>(kp);
    const bool enc =
        encode_tmap(&sp.tmA[0], 4, a_hi, ukp, p.M, 1, ukp, ukp * p.M, 32, SBM, true) &&
        encode_tmap(&sp.tmA[1], 4, a_lo, ukp, p.M, 1, ukp, ukp * p.M, 32, SBM, true) &&
        encode_tmap(&sp.tmB[0], 4, b_hi, ukp, p.N, 1, ukp, ukp * p.N, 32, SBN, true) &&
        encode_tmap(&sp.tmB[1], 4, b_lo, ukp, p.N, 1, ukp, ukp * p.N, 32, SBN, true);
    if (!enc) e = cudaErrorInvalidValue;
  }
  if (e == cudaSuccess) {
    sp.npairs = 1;
    sp.k[0] = static_cast<int>(kp);
    sp.M = p.M;
    sp.N = p.N;
    sp.bn = SBN;
    sp.tiles_m = (p.M + SBM - 1) / SBM;
    sp.tiles_n = (p.N + SBN - 1) / SBN;
    sp.C = static_cast<float*>(p.c);
    sp.ldc = p.ldc;
    sp.c_rs = 1;
    sp.c_cs = p.ldc;
    sp.bias = static_cast<const float*>(p.bias);
    sp.act = p.act;
    sp.accumulate = p.accumulate;
    sp.split_k = p.split_k > 1 ? p.split_k : 1;
    sp.batches = 1;
    sp.total_tiles = sp.tiles_m * sp.tiles_n * sp.split_k;
    if (sp.split_k > 1) {
      sp.act = ACT_NONE;  // applied by a pass over the summed C after the kernel
      if (!p.accumulate)  // partial sums are added onto zeros
        e = cudaMemset2DAsync(p.c, p.ldc * 4, 0, static_cast<size_t>(p.M) * 4, p.N, stream);
    }
    const int smem = PRE_STAGES * PLANE_STAGE + 1024;
    static unsigned long long smem_set = 0;
    if (e == cudaSuccess)
      e = set_smem_limit_once(reinterpret_cast<const void*>(sgemm3x_pre_kernel), smem, &smem_set);
    if (e == cudaSuccess)
      e = launch_kernel(sgemm3x_pre_kernel, dim3(static_cast<unsigned>(sp.total_tiles)),
                        dim3(NTHREADS), smem, stream, pdl_enabled(), sp, status);
    if (e == cudaSuccess && sp.split_k > 1 && p.act != ACT_NONE)
      e = launch_act_inplace_f32(sp.C, sp.ldc, 0, p.act, p.M, p.N, 1, stream);
  }
  const cudaError_t fe = cudaFreeAsync(ws, stream);
  return e != cudaSuccess ? e : fe;
}

cudaError_t launch_sgemm3x(const Problem& p_in, cudaStream_t stream, int* status) {
  if (presplit_wanted(p_in)) {
    const cudaError_t e = launch_sgemm3x_pre(p_in, stream, status);
    if (e != cudaErrorMemoryAllocation) return e;
    cudaGetLastError();  // no scratch to be had: nothing was queued, take the path below
  }
  Problem p = p_in;
  bool transposed = false;
  if (p.M <= 64 && p.N > 64 && p.bias == nullptr && p.rowsum == nullptr && p.act == ACT_NONE) {
    bool plain = true;
    for (int i = 0; i < p.npairs; ++i)
      plain = plain && p.a[i].dact == ACT_NONE && p.b[i].dact == ACT_NONE;
    if (plain) {
      for (int i = 0; i < p.npairs; ++i) std::swap(p.a[i], p.b[i]);
      std::swap(p.M, p.N);
      transposed = true;
    }
  }
  const int bn = p.N <= 64 ? 64 : SBN;
  SParams sp;
  std::memset(&sp, 0, sizeof(sp));
  sp.npairs = p.npairs;
  for (int i = 0; i < p.npairs; ++i) {
    sp.k[i] = static_cast<int>(p.k[i]);
    sp.a_kc[i] = p.a[i].k_contig;
    sp.b_kc[i] = p.b[i].k_contig;
    if (!encode_operand(&sp.tmA[i], p.a[i].base, p.a[i], p.M, p.k[i], p.batches) ||
        !encode_operand(&sp.tmB[i], p.b[i].base, p.b[i], p.N, p.k[i], p.batches, bn))
      return cudaErrorInvalidValue;
  }
  if (p.a[0].dact != ACT_NONE) {
    sp.dop = 1;
    sp.dact = p.a[0].dact;
    if (!encode_operand(&sp.tmY, p.a[0].ybase, p.a[0], p.M, p.k[0], p.batches))
      return cudaErrorInvalidValue;
  } else if (p.b[0].dact != ACT_NONE) {
    sp.dop = 2;
    sp.dact = p.b[0].dact;
    if (!encode_operand(&sp.tmY, p.b[0].ybase, p.b[0], p.N, p.k[0], p.batches, bn))
      return cudaErrorInvalidValue;
  }
  sp.M = p.M;
  sp.N = p.N;
  sp.bn = bn;
  sp.c_rs = transposed ? p.ldc : 1;
  sp.c_cs = transposed ? 1 : p.ldc;
  sp.tiles_m = (p.M + SBM - 1) / SBM;
  sp.tiles_n = (p.N + bn - 1) / bn;
  sp.C = static_cast<float*>(p.c);
  sp.ldc = p.ldc;
  sp.strideC = p.c_batch_stride;
  sp.bias = static_cast<const float*>(p.bias);
  sp.rowsum = static_cast<float*>(p.rowsum);
  sp.act = p.act;
  sp.accumulate = p.accumulate;
  sp.split_k = p.split_k > 1 ? p.split_k : 1;
  sp.batches = p.batches;
  if (sp.split_k > 1) {
    if (p.npairs != 1) return cudaErrorInvalidValue;
    sp.act = ACT_NONE;  // applied by a pass over the summed C after the kernel
    if (!p.accumulate) {  // partial sums are added onto zeros
      cudaError_t ze = cudaSuccess;
      // C as the caller stores it: p_in.M rows by p_in.N columns, whatever the tile orientation
      if (p.batches == 1 || p.c_batch_stride == p.ldc * p_in.N)
        ze = cudaMemset2DAsync(p.c, p.ldc * 4, 0, static_cast<size_t>(p_in.M) * 4,
                               static_cast<size_t>(p_in.N) * p.batches, stream);
      else
        for (int b = 0; b < p.batches && ze == cudaSuccess; ++b)
          ze = cudaMemset2DAsync(static_cast<float*>(p.c) + b * p.c_batch_stride, p.ldc * 4, 0,
                                 static_cast<size_t>(p_in.M) * 4, p_in.N, stream);
      if (ze != cudaSuccess) return ze;
    }
  }
  const long long total = static_cast<long long>(sp.tiles_m) * sp.tiles_n * p.batches * sp.split_k;
  if (total <= 0) return cudaSuccess;
  if (total > 0x7fffffffLL) return cudaErrorInvalidValue;
  sp.total_tiles = static_cast<int>(total);
  const int smem = PLANE_STAGES * PLANE_STAGE + RAW_BYTES_TOTAL + 1024;
  // Tiles with few k-blocks (the batched products of attention: two to eight) are walked by one
  // CTA per SM, which saves the per-CTA prologue and first round trip to memory (256 x
  // (256 x 64 x 256): 57 -> 46 us).  Long tiles gain nothing from that and lose the hardware's
  // dynamic placement of CTAs (4096^3: 3-5 % slower), so they keep one CTA per tile.
  long long nkb_tile = 0;
  for (int i = 0; i < p.npairs; ++i) nkb_tile += (p.k[i] + SBK - 1) / SBK;
  nkb_tile = (nkb_tile + sp.split_k - 1) / sp.split_k;
  int sms = device_sm_count() - sm_margin();
  if (sms < 1) sms = 1;
  const bool walk = nkb_tile <= walk_kblocks() && total > sms;
  static unsigned long long smem_set[2] = {0, 0};  // per kernel
  auto kern = walk ? sgemm3x_tma_kernel<true> : sgemm3x_tma_kernel<false>;
  cudaError_t e = set_smem_limit_once(reinterpret_cast<const void*>(kern), smem, &smem_set[walk ? 1 : 0]);
  if (e != cudaSuccess) return e;
  e = launch_kernel(kern, dim3(static_cast<unsigned>(walk ? sms : total)), dim3(NTHREADS), smem,
                    stream, pdl_enabled(), sp, status);
  if (e != cudaSuccess || sp.split_k == 1 || p.act == ACT_NONE) return e;
  // an activated product is never run transposed, so (p.M, p.N) are the caller's here
  return launch_act_inplace_f32(sp.C, sp.ldc, sp.strideC, p.act, p.M, p.N, p.batches, stream);
}

// Number of K splits for a problem of `tiles` output tiles (batches included): when the tiles
// alone leave most SMs idle, one pair, and never below two k-blocks per CTA.  Partial sums are
// added to C atomically (a bias by the first CTA of a tile).  The gather front end only splits
// products that add without an activation; the TMA-fed launcher (`tma_path`) splits any product:
// it zeroes C first when the product assigns and applies an activation in a pass over the
// summed C afterwards (measured on 512 x 128 x 784: 10 + 2.5 us against 25 us unsplit; letting
// the last CTA of each tile apply it in the same kernel cost 8 us in fences and re-reads).
int sgemm3x_pick_split(const Problem& p, long long tiles, int num_sms, bool tma_path) {
  if (p.npairs != 1 || max_split() == 1) return 1;
  const bool plain_add = p.accumulate && p.act == ACT_NONE;
  if (!plain_add && !tma_path) return 1;
  const long long nkb = (p.k[0] + SBK - 1) / SBK;
  if (tiles <= 0 || tiles * 2 > num_sms || nkb < 4) return 1;
  long long s = num_sms / tiles;
  if (s > nkb / 2) s = nkb / 2;
  if (s > 32) s = 32;
  if (max_split() > 0 && s > max_split()) s = max_split();
  return s < 1 ? 1 : static_cast<int>(s);
}

// fp32 problems a tensor map cannot describe (any alignment, column tables); k > 0, at most one
// derivative operand and then a single pair; the bias gradient needs an outer-contiguous A.
bool sgemm3x_gather_supported(const Problem& p) {
  if (p.npairs < 1) return false;
  int nderiv = 0;
  for (int i = 0; i < p.npairs; ++i) {
    if (p.k[i] <= 0 || p.k[i] > 0x7fffffffLL) return false;
    nderiv += (p.a[i].dact != ACT_NONE) + (p.b[i].dact != ACT_NONE);
  }
  if (nderiv > 1 || (nderiv == 1 && p.npairs != 1)) return false;
  if (p.rowsum != nullptr && p.a[0].k_contig) return false;
  return true;
}

cudaError_t launch_sgemm3x_gather(Problem& p, cudaStream_t stream, int* status) {
  p.tiles_m = (p.M + SBM - 1) / SBM;
  p.tiles_n = (p.N + SBN - 1) / SBN;
  p.tile_start = 0;
  const long long total = static_cast<long long>(p.tiles_m) * p.tiles_n * p.batches *
                          (p.split_k > 1 ? p.split_k : 1);
  if (total <= 0) return cudaSuccess;
  if (total > 0x7fffffffLL) return cudaErrorInvalidValue;
  const bool with_y = p.a[0].dact != ACT_NONE || p.b[0].dact != ACT_NONE;
  return with_y ? launch_gather<false, true>(p, nullptr, 1, static_cast<int>(total), stream, status)
                : launch_gather<false, false>(p, nullptr, 1, static_cast<int>(total), stream, status);
}

// Descriptors in device memory, tiles_m / tiles_n / tile_start filled for 128 x 128 tiles.
cudaError_t launch_sgemm3x_gather_grouped(const Problem* dprobs, int nprobs, int total_tiles,
                                          bool with_y, cudaStream_t stream, int* status) {
  if (total_tiles <= 0) return cudaSuccess;
  Problem dummy{};
  return with_y ? launch_gather<true, true>(dummy, dprobs, nprobs, total_tiles, stream, status)
                : launch_gather<true, false>(dummy, dprobs, nprobs, total_tiles, stream, status);
}

}  // namespace gb
