// General tcgen05 GEMM for ginn's column-major tensors ("staged" kernel).
//
// Producer warps read the operands with ordinary global loads, so any alignment, any
// leading dimension, transposed operands, strided batches and gathered columns (pointer
// tables) all go through one code path.  While a tile slice sits in registers the
// producers
//   * multiply by the derivative of the nonlinearity (dY (.) act'(Y)) when asked to,
//   * accumulate the bias gradient (row sums of the A operand),
//   * split fp32 values into two TF32 planes (hi = rna(x), lo = x - hi),
// and then write K-major, 128-byte-swizzled tiles to shared memory.  One elected thread
// issues tcgen05.mma into TMEM; the epilogue reads TMEM with tcgen05.ld, adds bias / previous
// C, applies the activation and stores coalesced along rows, which are contiguous in
// column-major storage.
//
// fp32 uses kind::tf32 three times per k-step.  The tensor core truncates when it adds into
// its fp32 accumulator, which biases long accumulation chains, so the chain is cut: the small
// cross terms lo*hi + hi*lo go to one accumulator, the hi*hi terms rotate over three more
// (k-block j -> accumulator j mod 3) and the epilogue adds the four with round-to-nearest.
// fp16 uses kind::f16 once per k-step and a single accumulator.
//
// Role layout of a CTA (288 threads): warps 0-3 produce the A slice, warps 4-7 the B slice,
// then all eight run the epilogue (TMEM lane quarter = warp index mod 4, half of the columns
// each); warp 8 allocates TMEM and issues the MMAs.
#include <mutex>
#include "ptx.cuh"
#include "math.cuh"
#include "problem.h"
#include "launch.h"

namespace gb {

template <typename T>
struct TT;
template <>
struct TT<float> {
  static constexpr int EPC = 4;     // elements per 16-byte chunk
  static constexpr int PLANES = 2;  // hi and lo TF32 planes
  static constexpr int ACCS = 4;    // cross + three rotating main accumulators
  static constexpr uint32_t FMT = 2;
};
template <>
struct TT<__half> {
  static constexpr int EPC = 8;
  static constexpr int PLANES = 1;
  static constexpr int ACCS = 1;
  static constexpr uint32_t FMT = 0;
};

constexpr int kBM = 128;           // rows of C per tile == TMEM lanes
constexpr int kRowBytes = 128;     // bytes of K per tile row == swizzle span
constexpr int kKSteps = 4;         // MMAs (per plane combination) per k-block: 32 bytes of K each
constexpr int kGroupThreads = 128; // producer threads per operand
constexpr int kStagedThreads = 2 * kGroupThreads + 32;

// Per-thread view of one operand for one tile.  Everything that does not change along K is
// worked out once in init(); load() then only adds the k offset.
//   k_contig : slot i covers row i*16 + t/8, 16-byte chunk t%8 (8 threads read one 128-byte row)
//   else     : the thread owns one row (t % ROWS) and slot i covers chunk (i*128 + t) / ROWS;
//              consecutive threads read consecutive rows, which are contiguous in memory.
template <typename T, int ROWS>
struct TileLoader {
  static constexpr int NS = ROWS / 16;
  static constexpr int E = TT<T>::EPC;
  const Operand* op;
  const T* ptr[NS];   // k_contig: column base of each slot's row (nullptr = outside the matrix)
  const T* yptr[NS];
  const T* rowp;      // outer-contiguous: base + row (nullptr = outside)
  const T* yrowp;
  int t;
  int row;            // outer-contiguous: row inside the tile
  int o;              // outer-contiguous: global outer index
  bool has_y;

  __device__ __forceinline__ void init(const Operand& op_, long long boff, int o0, int O, int t_) {
    op = &op_;
    t = t_;
    has_y = op_.dact != ACT_NONE;
    rowp = yrowp = nullptr;
    row = t_ % ROWS;
    o = o0 + row;
    if (op_.k_contig) {
#pragma unroll
      for (int i = 0; i < NS; ++i) {
        const int oi = o0 + i * 16 + (t_ >> 3);
        ptr[i] = yptr[i] = nullptr;
        if (oi < O) {
          ptr[i] = op_.cols ? static_cast<const T*>(op_.cols[oi])
                            : static_cast<const T*>(op_.base) + boff + static_cast<long long>(oi) * op_.ld;
          if (has_y)
            yptr[i] = op_.ycols ? static_cast<const T*>(op_.ycols[oi])
                                : static_cast<const T*>(op_.ybase) + boff + static_cast<long long>(oi) * op_.ld;
        }
      }
    } else if (o < O && op_.cols == nullptr) {
      rowp = static_cast<const T*>(op_.base) + boff + o;
      if (has_y) yrowp = static_cast<const T*>(op_.ybase) + boff + o;
    }
    if (!op_.k_contig) {
#pragma unroll
      for (int i = 0; i < NS; ++i) ptr[i] = yptr[i] = nullptr;
    }
  }

  __device__ __forceinline__ void load(long long k0, long long K, int O, uint4 (&r)[NS]) const {
    const Operand& P = *op;
    if (P.k_contig) {
      const long long kk = k0 + (t & 7) * E;
#pragma unroll
      for (int i = 0; i < NS; ++i) {
        uint4 du = make_uint4(0, 0, 0, 0), yu = make_uint4(0, 0, 0, 0);
        if (ptr[i] != nullptr && kk < K) {
          T* d = reinterpret_cast<T*>(&du);
          T* y = reinterpret_cast<T*>(&yu);
          if (P.vec && kk + E <= K) {
            du = __ldg(reinterpret_cast<const uint4*>(ptr[i] + kk));
            if (has_y) yu = __ldg(reinterpret_cast<const uint4*>(yptr[i] + kk));
          } else {
#pragma unroll
            for (int e = 0; e < E; ++e) {
              if (kk + e < K) {
                d[e] = ldg1(ptr[i] + kk + e);
                if (has_y) y[e] = ldg1(yptr[i] + kk + e);
              }
            }
          }
          if (has_y) {
#pragma unroll
            for (int e = 0; e < E; ++e)
              d[e] = from_f<T>(act_backward<T>(P.dact, to_f(y[e]), to_f(d[e])));
          }
        }
        r[i] = du;
      }
    } else {
      const bool row_ok = o < O;
#pragma unroll
      for (int i = 0; i < NS; ++i) {
        const int chunk = (i * kGroupThreads + t) / ROWS;
        const long long kk = k0 + chunk * E;
        uint4 du = make_uint4(0, 0, 0, 0);
        T* d = reinterpret_cast<T*>(&du);
        if (row_ok) {
#pragma unroll
          for (int e = 0; e < E; ++e) {
            if (kk + e < K) {
              float yv = 0.f;
              if (P.cols != nullptr) {
                d[e] = ldg1(static_cast<const T*>(P.cols[kk + e]) + o);
                if (has_y) yv = to_f(ldg1(static_cast<const T*>(P.ycols[kk + e]) + o));
              } else {
                d[e] = ldg1(rowp + (kk + e) * P.ld);
                if (has_y) yv = to_f(ldg1(yrowp + (kk + e) * P.ld));
              }
              if (has_y) d[e] = from_f<T>(act_backward<T>(P.dact, yv, to_f(d[e])));
            }
          }
        }
        r[i] = du;
      }
    }
  }

  // Writes the slots into the swizzled K-major plane(s); optionally adds the values to *rowsum
  // (meaningful for outer-contiguous operands, where the thread owns one row).
  __device__ __forceinline__ void store(const uint4 (&r)[NS], uint8_t* plane0, uint8_t* plane1,
                                        float* rowsum) const {
    const int kc = op->k_contig;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
      const int srow = kc ? i * 16 + (t >> 3) : row;
      const int chunk = kc ? (t & 7) : (i * kGroupThreads + t) / ROWS;
      const uint32_t off = sw128_offset(srow, chunk);
      if (TT<T>::PLANES == 2) {
        const float* x = reinterpret_cast<const float*>(&r[i]);
        float4 h, l;
        split_tf32(x[0], h.x, l.x);
        split_tf32(x[1], h.y, l.y);
        split_tf32(x[2], h.z, l.z);
        split_tf32(x[3], h.w, l.w);
        if (rowsum) *rowsum += (x[0] + x[1]) + (x[2] + x[3]);
        *reinterpret_cast<float4*>(plane0 + off) = h;
        *reinterpret_cast<float4*>(plane1 + off) = l;
      } else {
        if (rowsum) {
          const __half* x = reinterpret_cast<const __half*>(&r[i]);
#pragma unroll
          for (int e = 0; e < 8; ++e) *rowsum += __half2float(x[e]);
        }
        *reinterpret_cast<uint4*>(plane0 + off) = r[i];
      }
    }
  }
};

template <typename T, int BN>
struct StageLayout {
  static constexpr int A_PLANE = kBM * kRowBytes;
  static constexpr int B_PLANE = BN * kRowBytes;
  static constexpr int A_BYTES = A_PLANE * TT<T>::PLANES;
  static constexpr int B_BYTES = B_PLANE * TT<T>::PLANES;
  static constexpr int BYTES = A_BYTES + B_BYTES;
};

template <typename T, int ROWS>
__device__ __forceinline__ bool produce(const Problem& P, bool is_a, int o0, int O, long long batch,
                                        int tg, int nkb, int stages, int stage_bytes,
                                        uint8_t* tiles_ptr, int plane_off, int plane_bytes,
                                        uint64_t* full_bar, uint64_t* empty_bar, float* rowsum,
                                        int* status) {
  constexpr int E = TT<T>::EPC;
  constexpr int BK = 8 * E;
  TileLoader<T, ROWS> ld;
  uint4 r[ROWS / 16];
  int pair = 0;
  long long k0 = 0;
  const Operand* op = is_a ? &P.a[0] : &P.b[0];
  ld.init(*op, batch * op->batch_stride, o0, O, tg);
  if (nkb > 0) ld.load(0, P.k[0], O, r);
  int s = 0;
  uint32_t ph = 0;
  for (int it = 0; it < nkb; ++it) {
    if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, status, DEV_TIMEOUT_EMPTY, it)) return false;
    uint8_t* st = tiles_ptr + s * stage_bytes + plane_off;
    ld.store(r, st, st + plane_bytes, (rowsum != nullptr && pair == 0) ? rowsum : nullptr);
    fence_proxy_async_smem();
    mbar_arrive(smem_u32(&full_bar[s]));
    if (++s == stages) {
      s = 0;
      ph ^= 1u;
    }
    k0 += BK;
    if (k0 >= P.k[pair]) {
      ++pair;
      k0 = 0;
      if (it + 1 < nkb) {
        op = is_a ? &P.a[pair] : &P.b[pair];
        ld.init(*op, batch * op->batch_stride, o0, O, tg);
      }
    }
    if (it + 1 < nkb) ld.load(k0, P.k[pair], O, r);
  }
  return true;
}

template <typename T, int BN, int STAGES, bool GROUPED>
__global__ void __launch_bounds__(kStagedThreads, 1)
gemm_staged_kernel(const __grid_constant__ Problem p0, const Problem* __restrict__ probs,
                   int nprobs, int* __restrict__ status) {
  using L = StageLayout<T, BN>;
  constexpr int E = TT<T>::EPC;
  constexpr int BK = 8 * E;  // elements of K per k-block
  constexpr int ACCS = TT<T>::ACCS;
  constexpr uint32_t NCOLS = (ACCS * BN) < 32 ? 32 : (ACCS * BN);
  constexpr uint32_t IDESC = make_idesc(TT<T>::FMT, 0, 0, kBM, BN);
  constexpr uint32_t CROSS_COL = 3 * BN;  // fp32 only: accumulator of the lo*hi + hi*lo terms

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ Problem sprob;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // ---- which problem / tile ----
  int tile = blockIdx.x;
  if (GROUPED) {
    int g = 0;
    for (int i = 0; i < nprobs; ++i)
      if (tile >= probs[i].tile_start) g = i;
    const int nwords = sizeof(Problem) / 4;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(probs + g);
    uint32_t* dst = reinterpret_cast<uint32_t*>(&sprob);
    for (int i = tid; i < nwords; i += blockDim.x) dst[i] = src[i];
    __syncthreads();
  }
  const Problem& P = GROUPED ? sprob : p0;
  tile -= P.tile_start;
  const int m_tile = tile % P.tiles_m;
  const int rest = tile / P.tiles_m;
  const int n_tile = rest % P.tiles_n;
  const long long batch = rest / P.tiles_n;
  const int m0 = m_tile * kBM;
  const int n0 = n_tile * BN;

  int nkb = 0;
  for (int p = 0; p < P.npairs; ++p) nkb += static_cast<int>((P.k[p] + BK - 1) / BK);

  const uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* tiles_ptr = smem_raw + (tiles_base - smem_u32(smem_raw));

  // ---- setup ----
  if (warp == 8) {
    if (lane == 0) {
      for (int s = 0; s < STAGES; ++s) {
        mbar_init(smem_u32(&full_bar[s]), 2 * kGroupThreads);
        mbar_init(smem_u32(&empty_bar[s]), 1);
      }
      mbar_init(smem_u32(&accum_bar), 1);
      fence_mbar_init();
    }
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_slot), NCOLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp < 8) {
    // ================= producers =================
    const bool is_a = warp < 4;
    const int tg = tid & (kGroupThreads - 1);
    float rs = 0.f;
    const bool want_rowsum = is_a && P.rowsum != nullptr && n_tile == 0;
    bool ok;
    if (is_a)
      ok = produce<T, kBM>(P, true, m0, P.M, batch, tg, nkb, STAGES, L::BYTES, tiles_ptr, 0,
                           L::A_PLANE, full_bar, empty_bar, want_rowsum ? &rs : nullptr, status);
    else
      ok = produce<T, BN>(P, false, n0, P.N, batch, tg, nkb, STAGES, L::BYTES, tiles_ptr,
                          L::A_BYTES, L::B_PLANE, full_bar, empty_bar, nullptr, status);
    if (want_rowsum && ok) {
      const int row = m0 + tg;
      if (row < P.M) {
        if (sizeof(T) == 4)
          atomicAdd(static_cast<float*>(P.rowsum) + row, rs);
        else
          atomicAdd(static_cast<__half*>(P.rowsum) + row, __float2half_rn(rs));
      }
    }

    // ================= epilogue =================
    constexpr int COLS_PER_HALF = BN >= 64 ? BN / 2 : BN;
    const int half = warp >> 2;
    const bool has_cols = BN >= 64 || half == 0;
    if (ok && has_cols && mbar_wait(smem_u32(&accum_bar), 0, status, DEV_TIMEOUT_ACCUM, 0)) {
      tc_fence_after();
      const int q = warp & 3;
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < P.M;
      float bias = 0.f;
      if (P.bias != nullptr && row_ok) bias = to_f(static_cast<const T*>(P.bias)[row]);
      T* cbase = static_cast<T*>(P.c) + batch * P.c_batch_stride;
      const uint32_t tbase = tmem + (static_cast<uint32_t>(q * 32) << 16);
      const int cbeg = BN >= 64 ? half * COLS_PER_HALF : 0;
#pragma unroll 1
      for (int c0 = cbeg; c0 < cbeg + COLS_PER_HALF; c0 += 32) {
        float acc[32];
        // previous C first, so the loads are in flight while TMEM is read
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = n0 + c0 + j;
          float v = bias;
          if (P.accumulate && row_ok && col < P.N) {
            const T* src = (P.ccols ? static_cast<const T*>(P.ccols[col])
                                    : cbase + static_cast<long long>(col) * P.ldc) + row;
            v += to_f(*src);
          }
          acc[j] = v;
        }
        uint32_t v[32];
        if (nkb > 0) {
          if (ACCS == 4) {
            tmem_ld32(tbase + CROSS_COL + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] += __uint_as_float(v[j]);
#pragma unroll 1
            for (int a = 0; a < 3 && a < nkb; ++a) {
              tmem_ld32(tbase + a * BN + c0, v);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) acc[j] += __uint_as_float(v[j]);
            }
          } else {
            tmem_ld32(tbase + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] += __uint_as_float(v[j]);
          }
        }
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = n0 + c0 + j;
            if (col < P.N) {
              T* dst = (P.ccols ? static_cast<T*>(P.ccols[col])
                                : cbase + static_cast<long long>(col) * P.ldc) + row;
              *dst = from_f<T>(act_forward<T>(P.act, acc[j]));
            }
          }
        }
      }
    }
  } else {
    // ================= MMA issuer =================
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0; it < nkb; ++it) {
        if (!mbar_wait(smem_u32(&full_bar[s]), ph, status, DEV_TIMEOUT_FULL, it)) break;
        tc_fence_after();
        const uint32_t a0 = tiles_base + s * L::BYTES;
        const uint32_t b0 = a0 + L::A_BYTES;
#pragma unroll
        for (int ks = 0; ks < kKSteps; ++ks) {
          if (TT<T>::PLANES == 2) {
            const uint64_t a_hi = make_smem_desc(a0 + ks * 32, 16, 1024);
            const uint64_t a_lo = make_smem_desc(a0 + L::A_PLANE + ks * 32, 16, 1024);
            const uint64_t b_hi = make_smem_desc(b0 + ks * 32, 16, 1024);
            const uint64_t b_lo = make_smem_desc(b0 + L::B_PLANE + ks * 32, 16, 1024);
            mma_tf32(tmem + CROSS_COL, a_lo, b_hi, IDESC, (it > 0 || ks > 0) ? 1u : 0u);
            mma_tf32(tmem + CROSS_COL, a_hi, b_lo, IDESC, 1u);
            mma_tf32(tmem + (it % 3) * BN, a_hi, b_hi, IDESC, (it >= 3 || ks > 0) ? 1u : 0u);
          } else {
            const uint64_t a = make_smem_desc(a0 + ks * 32, 16, 1024);
            const uint64_t b = make_smem_desc(b0 + ks * 32, 16, 1024);
            mma_f16(tmem, a, b, IDESC, (it > 0 || ks > 0) ? 1u : 0u);
          }
        }
        tc_commit(smem_u32(&empty_bar[s]));
        if (++s == STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
      tc_commit(smem_u32(&accum_bar));
    }
    __syncwarp();
  }

  // ---- teardown ----
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem, NCOLS);
  }
}

// -------------------------------------------------------------------------------------------
// Host side
// -------------------------------------------------------------------------------------------
template <typename T, int BN>
constexpr int stages_for() {
  constexpr int per = StageLayout<T, BN>::BYTES;
  constexpr int budget = 200 * 1024;
  return (budget / per) > 6 ? 6 : (budget / per);
}

template <typename T, int BN, bool GROUPED>
static cudaError_t launch_one(const Problem& p, const Problem* dprobs, int nprobs, int total_tiles,
                              cudaStream_t stream, int* status) {
  constexpr int STAGES = stages_for<T, BN>();
  static_assert(STAGES >= 2, "need at least two stages");
  auto kern = gemm_staged_kernel<T, BN, STAGES, GROUPED>;
  const int smem = STAGES * StageLayout<T, BN>::BYTES + 1024;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  kern<<<total_tiles, kStagedThreads, smem, stream>>>(p, dprobs, nprobs, status);
  return cudaGetLastError();
}

int staged_pick_bn(int dtype, long long M, long long N, long long batches, int num_sms) {
  (void)dtype;
  if (N <= 32) return 32;
  if (N <= 64) return 64;
  // Prefer the widest tile that still gives every SM a CTA.
  const long long tm = (M + kBM - 1) / kBM;
  if (tm * ((N + 127) / 128) * batches >= num_sms) return 128;
  if (tm * ((N + 63) / 64) * batches >= num_sms || N % 64 == 0) return 64;
  return 128;
}

template <typename T>
static cudaError_t launch_staged_t(Problem& p, int bn, cudaStream_t stream, int* status) {
  p.tiles_m = (p.M + kBM - 1) / kBM;
  p.tiles_n = (p.N + bn - 1) / bn;
  p.tile_start = 0;
  const long long total = static_cast<long long>(p.tiles_m) * p.tiles_n * p.batches;
  if (total <= 0) return cudaSuccess;
  if (total > 0x7fffffffLL) return cudaErrorInvalidValue;
  const int tt = static_cast<int>(total);
  switch (bn) {
    case 32: return launch_one<T, 32, false>(p, nullptr, 1, tt, stream, status);
    case 64: return launch_one<T, 64, false>(p, nullptr, 1, tt, stream, status);
    default: return launch_one<T, 128, false>(p, nullptr, 1, tt, stream, status);
  }
}

cudaError_t launch_staged(int dtype, Problem& p, int bn, cudaStream_t stream, int* status) {
  return dtype == 0 ? launch_staged_t<float>(p, bn, stream, status)
                    : launch_staged_t<__half>(p, bn, stream, status);
}

template <typename T>
static cudaError_t launch_grouped_t(const Problem* dprobs, int nprobs, int total_tiles, int bn,
                                    cudaStream_t stream, int* status) {
  Problem dummy{};
  if (total_tiles <= 0) return cudaSuccess;
  switch (bn) {
    case 32: return launch_one<T, 32, true>(dummy, dprobs, nprobs, total_tiles, stream, status);
    case 64: return launch_one<T, 64, true>(dummy, dprobs, nprobs, total_tiles, stream, status);
    default: return launch_one<T, 128, true>(dummy, dprobs, nprobs, total_tiles, stream, status);
  }
}

cudaError_t launch_staged_grouped(int dtype, const Problem* dprobs, int nprobs, int total_tiles,
                                  int bn, cudaStream_t stream, int* status) {
  return dtype == 0 ? launch_grouped_t<float>(dprobs, nprobs, total_tiles, bn, stream, status)
                    : launch_grouped_t<__half>(dprobs, nprobs, total_tiles, bn, stream, status);
}

// -------------------------------------------------------------------------------------------
// Grouped launch that allocates nothing.
//
// The ordinary grouped launch keeps its problem descriptors and column-pointer tables in a
// cudaMalloc'ed ring.  Some hosts cannot allocate at the point where they call: a caller that
// runs inside a memory pool it must not disturb, or one that has pledged a fixed footprint
// (ginn's PreallocGpuDevice style of accounting, where every byte taken from the GPU is counted).
// For them the same kernel reads its descriptors from a fixed array that is part of the
// library image, so nothing is requested from the CUDA allocator at call time.
//
// The array exists once per GPU that loads the library and stays until the process exits.
// All calls on a GPU share it, and it always holds whatever the last call put there; the part a
// call uses is completely rewritten by that call, so nothing in it needs clearing.  Two calls
// whose GPU work overlaps (different streams) would overwrite each other's descriptors: keep
// calls of this variant on one stream, or order them with events.
// -------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_grouped_static_scratch[kGroupedStaticBytes];

namespace {
struct StaticScratchSlot {
  void* ptr = nullptr;
  bool ready = false;
};
StaticScratchSlot g_static_slots[64];
std::mutex g_static_mu;
}  // namespace

// `device` must be current.  In host code the array's name is only a handle, not a device
// address, so the address is looked up once per device and cached.
cudaError_t grouped_static_scratch(int device, void** ptr) {
  if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> g(g_static_mu);
  StaticScratchSlot& slot = g_static_slots[device];
  if (!slot.ready) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_grouped_static_scratch);
    if (e != cudaSuccess) return e;
    slot.ptr = p;
    slot.ready = true;
  }
  *ptr = slot.ptr;
  return cudaSuccess;
}

// Copies the host image (descriptors followed by pointer tables, already holding device
// addresses inside the static array) and launches the grouped kernel on it.
cudaError_t launch_staged_grouped_static(int dtype, const void* host_image, size_t bytes,
                                         void* scratch, int nprobs, int total_tiles, int bn,
                                         bool fp32_gather, cudaStream_t stream) {
  if (bytes > kGroupedStaticBytes) return cudaErrorInvalidValue;
  cudaError_t e = cudaMemcpyAsync(scratch, host_image, bytes, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return e;
  // No status word: a wait that runs out still ends the kernel, it is just not recorded.
  // Same kernels as the allocating entry point: the gather kernels unless the staged one is forced.
  if (fp32_gather && dtype == 0)
    return launch_sgemm3x_gather_grouped(static_cast<const Problem*>(scratch), nprobs,
                                         total_tiles, stream, nullptr);
  if (fp32_gather)
    return launch_hgemm_gather_grouped(static_cast<const Problem*>(scratch), nprobs, total_tiles,
                                       stream, nullptr);
  return launch_staged_grouped(dtype, static_cast<const Problem*>(scratch), nprobs, total_tiles,
                               bn, stream, nullptr);
}

}  // namespace gb
