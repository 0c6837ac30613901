// General fp16 GEMM (fp32 accumulation) for ginn's column-major tensors:
//   C = act( sum_p A_p * B_p + bias [+ C] ), any alignment, any leading dimension, transposed
//   operands, strided batches, gathered columns (pointer tables), grouped launches, the
//   derivative dY (.) act'(Y) and the bias gradient fused into the operand path.
//
// Half operands need no transformation before the tensor core: tcgen05 reads K-contiguous and
// M/N-contiguous fp16 tiles alike, so the producers copy 16-byte pieces from global memory
// straight into the 128-byte-swizzled layout of the matching major with cp.async (zero filled
// outside the matrix).  Only an operand that carries a derivative or a bias-gradient sum, or
// whose addresses are not even 4-byte aligned, goes through registers, prefetched one k-block
// ahead.  A slice is announced to the MMA warp by one arrival per producer warp, a k-block after
// it was issued (cp.async groups), so two slices of copies are in flight per thread.  One 128 x 128 tile of C per CTA, BK = 64, three stages, two CTAs per SM.
//
//   warp 0       TMEM allocation and MMA issue (kind::f16, M = 128, N = 128, K = 16)
//   warps 1-4    producers of the A slice, warps 5-8 of the B slice; then the epilogue
#include "ptx.cuh"
#include "math.cuh"
#include "launch.h"

namespace gb {

namespace {

constexpr int GBM = 128, GBN = 128, GBK = 64;
constexpr int GSTAGES = 3;
constexpr int GTILE = 128 * GBK * 2;  // 16 KiB per operand slice
constexpr int GSTAGE = 2 * GTILE;
constexpr int GPROD = 128;            // producer threads per operand
constexpr int GTHREADS = 32 + 2 * GPROD;
constexpr int GPIECES = GTILE / 16 / GPROD;  // 16-byte pieces per thread per slice = 8

__device__ __forceinline__ void hcp16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void hcp4(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
struct PieceSrc {
  const __half* p;   // first element (nullptr: nothing valid)
  const __half* y;   // same position in Y (derivative operands)
  int valid;         // number of valid elements (0..8) along the contiguous direction
};

// The kernel's code has to stay small: the k loop of a tile runs at the speed of instruction
// fetch once the code outgrows the instruction caches, so everything off the common path
// (unaligned pieces, edges, the nonlinearities) is an out-of-line call.
struct Piece2 {
  uint4 d, y;
};

// Any alignment, partial pieces: element by element.
__device__ __noinline__ Piece2 load_piece_slow(const __half* p, const __half* y, int valid) {
  Piece2 r;
  r.d = make_uint4(0, 0, 0, 0);
  r.y = make_uint4(0, 0, 0, 0);
  __half* dh = reinterpret_cast<__half*>(&r.d);
  __half* yh = reinterpret_cast<__half*>(&r.y);
#pragma unroll
  for (int e = 0; e < 8; ++e)
    if (e < valid) {
      dh[e] = ldg1(p + e);
      if (y) yh[e] = ldg1(y + e);
    }
  return r;
}

// dY (.) act'(Y) on 8 halves in packed fp16 arithmetic, every operation rounded to fp16 as the
// reference's Half expressions are (ginn/nonlin.h:96-106 tanh, :119-126 relu, :146-152 sigmoid).
__device__ __forceinline__ uint4 apply_dact(uint4 d, uint4 y, int dact) {
  __half2* dh = reinterpret_cast<__half2*>(&d);
  const __half2* yh = reinterpret_cast<const __half2*>(&y);
  const __half2 one = __float2half2_rn(1.f), zero = __float2half2_rn(0.f);
  if (dact == ACT_TANH) {
#pragma unroll
    for (int e = 0; e < 4; ++e) dh[e] = __hsub2(dh[e], __hmul2(__hmul2(yh[e], yh[e]), dh[e]));
  } else if (dact == ACT_SIGMOID) {
#pragma unroll
    for (int e = 0; e < 4; ++e) dh[e] = __hmul2(__hmul2(yh[e], __hsub2(one, yh[e])), dh[e]);
  } else if (dact == ACT_RELU) {
#pragma unroll
    for (int e = 0; e < 4; ++e) dh[e] = __hmul2(__hgt2(yh[e], zero), dh[e]);
  }
  return d;
}

// A piece whose source is not 16-byte aligned: 4-byte asynchronous copies, or through registers
// when even those are impossible.
__device__ __noinline__ void copy_piece_slow(uint32_t d, const __half* p, int valid, const void* safe) {
  if ((reinterpret_cast<uintptr_t>(p) & 3u) == 0) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int left = valid - 2 * e;
      hcp4(d + 4 * e, left > 0 ? static_cast<const void*>(p + 2 * e) : safe,
           left >= 2 ? 4 : (left == 1 ? 2 : 0));
    }
  } else {
    const Piece2 r = load_piece_slow(p, nullptr, valid);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(d), "r"(r.d.x), "r"(r.d.y),
                 "r"(r.d.z), "r"(r.d.w)
                 : "memory");
  }
}

// Per-thread geometry of one operand slice, worked out once per (tile, pair): which eight
// 16-byte pieces the thread moves, where they come from and where they go.  Per k-block only a
// pointer advance and a bounds test remain.
//   k-contiguous : piece i = row (t/8 + 16 i), k offset 8 (t%8)    -> smem offset off0 + 2048 i
//   outer-contig.: piece i = k (t/16 + 8 i), outer offset 8 (t%16) -> smem offset off0 + 1024 i
struct Feeder {
  const void* const* cols;   // operand fields held in registers: the copies' "memory" clobbers
  const void* const* ycols;  // would otherwise force a reload of each before every piece
  const void* safe;          // any valid address, for zero-length copies
  long long ld;
  int dact;
  const __half* p0;   // untabled: element of piece 0 at k-block 0
  const __half* y0;
  long long K;
  uint32_t off0;
  int o_first;        // first outer index this thread touches
  int O, sub, valid_o;
  bool kc, has_y;
  // Fast path (plain operand, 16-byte aligned base, leading dimension and batch offset): the
  // eight sources are p0 + k-block * kadv + i * pstep (bytes) and only the edges need a test.
  bool fast;
  long long pstep, kadv, qoff, ydelta;
  uint32_t omask;     // k-contiguous: bit i set when piece i's row is inside the matrix

  __device__ __forceinline__ void init(const Operand& o, long long K_, long long boff, int o0,
                                       int O_, int t) {
    cols = o.cols;
    ycols = o.ycols;
    safe = o.cols ? static_cast<const void*>(o.cols) : o.base;
    ld = o.ld;
    dact = o.dact;
    K = K_;
    O = O_;
    kc = o.k_contig != 0;
    has_y = o.dact != ACT_NONE;
    p0 = y0 = nullptr;
    fast = o.cols == nullptr &&
           ((reinterpret_cast<uintptr_t>(o.base) | static_cast<uintptr_t>(o.ld * 2) |
             static_cast<uintptr_t>(boff * 2) | (has_y ? reinterpret_cast<uintptr_t>(o.ybase) : 0)) &
            15u) == 0;
    ydelta = has_y ? static_cast<const char*>(o.ybase) - static_cast<const char*>(o.base) : 0;
    pstep = (o.k_contig ? 16 : 8) * o.ld * 2;
    kadv = o.k_contig ? GBK * 2 : GBK * o.ld * 2;
    omask = 0;
    qoff = o.k_contig ? 0 : (t >> 4) * o.ld * 2;  // outer-contiguous: piece 0 sits at k = t / 16
    if (kc) {
#pragma unroll
      for (int i = 0; i < GPIECES; ++i) omask |= (o0 + (t >> 3) + 16 * i < O_) ? (1u << i) : 0u;
      sub = t & 7;
      const int row0 = t >> 3;
      off0 = sw128_offset(row0, sub);
      o_first = o0 + row0;
      valid_o = 8;
      if (o.cols == nullptr) {
        const long long e = boff + static_cast<long long>(o_first) * o.ld + 8 * sub;
        p0 = static_cast<const __half*>(o.base) + e;
        if (has_y) y0 = static_cast<const __half*>(o.ybase) + e;
      }
    } else {
      sub = t >> 4;  // k index of piece 0 inside the slice
      const int oc = t & 15;
      off0 = (oc >> 3) * 8192u + sw128_offset(sub, oc & 7);
      o_first = o0 + 8 * oc;
      valid_o = O_ - o_first >= 8 ? 8 : (O_ - o_first > 0 ? O_ - o_first : 0);
      if (o.cols == nullptr) {
        p0 = static_cast<const __half*>(o.base) + boff + o_first;
        if (has_y) y0 = static_cast<const __half*>(o.ybase) + boff + o_first;
      }
    }
  }

  __device__ __forceinline__ uint32_t offset(int i) const { return off0 + (kc ? 2048u : 1024u) * i; }

  // All eight pieces of the k-block starting at k0 (a multiple of GBK), fast path.
  __device__ __forceinline__ void fill_fast(uint32_t dst, long long k0) const {
    const char* q = reinterpret_cast<const char*>(p0) + (k0 / GBK) * kadv + qoff;
    uint32_t d = dst + off0;
    if (kc) {
      const long long rem = K - (k0 + 8 * sub);
      const uint32_t kb = rem >= 8 ? 16u : (rem > 0 ? static_cast<uint32_t>(rem) * 2u : 0u);
#pragma unroll
      for (int i = 0; i < GPIECES; ++i) {
        const uint32_t nb = ((omask >> i) & 1u) ? kb : 0u;
        hcp16(d, nb ? static_cast<const void*>(q) : safe, nb);
        q += pstep;
        d += 2048u;
      }
    } else {
      long long kg = k0 + sub;
      const uint32_t ob = static_cast<uint32_t>(valid_o) * 2u;
#pragma unroll
      for (int i = 0; i < GPIECES; ++i) {
        const uint32_t nb = kg < K ? ob : 0u;
        hcp16(d, nb ? static_cast<const void*>(q) : safe, nb);
        q += pstep;
        d += 1024u;
        kg += 8;
      }
    }
  }

  // Pieces h .. h+3 of the k-block starting at k0 into registers (and their Y values), fast path.
  __device__ __forceinline__ void load4_fast(long long k0, int h, uint4* d, uint4* y) const {
    const char* q = reinterpret_cast<const char*>(p0) + (k0 / GBK) * kadv + qoff + h * pstep;
    const long long rem = K - (k0 + 8 * sub);
    const int kv = rem >= 8 ? 8 : (rem > 0 ? static_cast<int>(rem) : 0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int valid;
      if (kc) valid = ((omask >> (h + i)) & 1u) ? kv : 0;
      else valid = (k0 + sub + 8 * (h + i) < K) ? valid_o : 0;
      d[i] = make_uint4(0, 0, 0, 0);
      y[i] = make_uint4(0, 0, 0, 0);
      if (valid == 8) {
        d[i] = __ldg(reinterpret_cast<const uint4*>(q));
        if (has_y) y[i] = __ldg(reinterpret_cast<const uint4*>(q + ydelta));
      } else if (valid > 0) {
        const Piece2 r = load_piece_slow(reinterpret_cast<const __half*>(q),
                                         has_y ? reinterpret_cast<const __half*>(q + ydelta) : nullptr, valid);
        d[i] = r.d;
        y[i] = r.y;
      }
      q += pstep;
    }
  }

  // Source of piece i for the k-block starting at k0.
  __device__ __forceinline__ PieceSrc src(int i, long long k0) const {
    PieceSrc s{nullptr, nullptr, 0};
    if (kc) {
      const long long kg = k0 + 8 * sub;
      const int og = o_first + 16 * i;
      if (og >= O || kg >= K) return s;
      if (cols) {
        s.p = static_cast<const __half*>(cols[og]) + kg;
        if (has_y) s.y = static_cast<const __half*>(ycols[og]) + kg;
      } else {
        const long long e = static_cast<long long>(16 * i) * ld + k0;
        s.p = p0 + e;
        if (has_y) s.y = y0 + e;
      }
      s.valid = K - kg >= 8 ? 8 : static_cast<int>(K - kg);
    } else {
      const long long kg = k0 + sub + 8 * i;
      if (valid_o <= 0 || kg >= K) return s;
      if (cols) {
        s.p = static_cast<const __half*>(cols[kg]) + o_first;
        if (has_y) s.y = static_cast<const __half*>(ycols[kg]) + o_first;
      } else {
        s.p = p0 + kg * ld;
        if (has_y) s.y = y0 + kg * ld;
      }
      s.valid = valid_o;
    }
    return s;
  }
};

// WITH_REGS: the instantiation that can route an operand through registers (fused derivative,
// bias-gradient sums).  That machinery is 60 % of the kernel's code; products that need none of
// it (plain products, Affine forward) run an instantiation without it.
template <bool GROUPED, bool WITH_REGS>
__global__ void __launch_bounds__(GTHREADS, 2)
hgemm_gather_kernel(const __grid_constant__ Problem p0, const Problem* __restrict__ probs,
                    int nprobs, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[GSTAGES];
  __shared__ __align__(8) uint64_t empty_bar[GSTAGES];
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ Problem sprob;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

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
  const int rest = tile / P.tiles_m;
  const int n_tile = rest % P.tiles_n;
  const long long batch = rest / P.tiles_n;
  const int m0 = m_tile * GBM, n0 = n_tile * GBN;

  int nkb = 0;
  for (int i = 0; i < P.npairs; ++i) nkb += static_cast<int>((P.k[i] + GBK - 1) / GBK);

  if (warp == 0) {
    if (lane == 0) {
      for (int s = 0; s < GSTAGES; ++s) {
        mbar_init(smem_u32(&full_bar[s]), 2 * GPROD / 32);  // one arrival per producer warp
        mbar_init(smem_u32(&empty_bar[s]), 1);
      }
      mbar_init(smem_u32(&acc_bar), 1);
      fence_mbar_init();
    }
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_slot), GBN);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 0) {
    // ===================== MMA issuer =====================
    if (elect_one()) {
      int s = 0, pair = 0;
      uint32_t ph = 0;
      long long k0 = 0;
      for (int it = 0; it < nkb; ++it) {
        if (!mbar_wait(smem_u32(&full_bar[s]), ph, status, DEV_TIMEOUT_FULL, it)) break;
        // The slices were written through the generic proxy (cp.async or plain stores).
        fence_proxy_async_smem();
        tc_fence_after();
        const uint32_t a_s = tiles_base + s * GSTAGE;
        const uint32_t b_s = a_s + GTILE;
        const uint32_t a_mn = P.a[pair].k_contig ? 0u : 1u, b_mn = P.b[pair].k_contig ? 0u : 1u;
        const uint32_t idesc = make_idesc(0, a_mn, b_mn, GBM, GBN);
#pragma unroll
        for (int ks = 0; ks < GBK / 16; ++ks) {
          const uint64_t ad = a_mn ? make_smem_desc(a_s + ks * 2048, 8192, 1024)
                                   : make_smem_desc(a_s + ks * 32, 16, 1024);
          const uint64_t bd = b_mn ? make_smem_desc(b_s + ks * 2048, 8192, 1024)
                                   : make_smem_desc(b_s + ks * 32, 16, 1024);
          mma_f16(tmem, ad, bd, idesc, (it > 0 || ks > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&empty_bar[s]));
        if (++s == GSTAGES) {
          s = 0;
          ph ^= 1u;
        }
        k0 += GBK;
        if (k0 >= P.k[pair]) {
          ++pair;
          k0 = 0;
        }
      }
      tc_commit(smem_u32(&acc_bar));
    }
    __syncwarp();
  } else {
    // ===================== producers (warps 1-4: A, warps 5-8: B) =====================
    const int pt = threadIdx.x - 32;
    const int grp = pt >> 7;  // 0 = A, 1 = B
    const int t = pt & (GPROD - 1);
    const int o0 = grp ? n0 : m0;
    const int O = grp ? P.N : P.M;
    const bool want_rowsum = WITH_REGS && grp == 0 && P.rowsum != nullptr && n_tile == 0;
    float rs[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    bool ok = true;
    int s = 0, pair = 0;
    uint32_t ph = 0;
    long long k0 = 0;
    uint4 regs[GPIECES];
    bool regs_loaded = false;

    auto operand = [&](int pr) -> const Operand& { return grp ? P.b[pr] : P.a[pr]; };
    // Register path: this operand carries a derivative or feeds the bias gradient.
    auto via_regs = [&](int pr) {
      return WITH_REGS && (operand(pr).dact != ACT_NONE || (want_rowsum && pr == 0));
    };
    Feeder fd;
    auto setup = [&](int pr) {
      const Operand& op = operand(pr);
      fd.init(op, P.k[pr], batch * op.batch_stride, o0, O, t);
    };
    auto load_regs = [&](long long kk0) {
#pragma unroll
      for (int h = 0; h < GPIECES; h += 4) {  // four pieces at a time: their Y values need registers too
        uint4 y[4];
        if (fd.fast) {
          fd.load4_fast(kk0, h, &regs[h], y);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {  // tables or unaligned operands: element by element
            const PieceSrc ps = fd.src(h + i, kk0);
            regs[h + i] = make_uint4(0, 0, 0, 0);
            y[i] = make_uint4(0, 0, 0, 0);
            if (ps.valid > 0) {
              const Piece2 r = load_piece_slow(ps.p, ps.y, ps.valid);
              regs[h + i] = r.d;
              y[i] = r.y;
            }
          }
        }
        if (fd.has_y) {
#pragma unroll
          for (int i = 0; i < 4; ++i) regs[h + i] = apply_dact(regs[h + i], y[i], fd.dact);
        }
      }
    };

    // Slice `stage` is complete for this warp: its copies have landed (cp.async groups waited
    // for by every lane, ordinary stores in program order), made visible to the tensor core's
    // proxy, then one lane arrives for the warp.
    int sig = 0;
    auto announce = [&](int stage) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&full_bar[stage]));
    };

    if (nkb > 0) setup(0);
    // The pass it = -1 only prefetches (one copy of the register loads in the code, not two).
    for (int it = -1; it < nkb; ++it) {
      if (it >= 0) {
      if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, status, DEV_TIMEOUT_EMPTY, it)) {
        ok = false;
        break;
      }
      const uint32_t dst = tiles_base + s * GSTAGE + grp * GTILE;
      if (via_regs(pair)) {
#pragma unroll
        for (int i = 0; i < GPIECES; ++i) {
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + fd.offset(i)),
                       "r"(regs[i].x), "r"(regs[i].y), "r"(regs[i].z), "r"(regs[i].w)
                       : "memory");
          if (want_rowsum && pair == 0) {
            const __half2* h = reinterpret_cast<const __half2*>(&regs[i]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __half22float2(h[e]);
              rs[2 * e] += f.x;
              rs[2 * e + 1] += f.y;
            }
          }
        }
        regs_loaded = false;
      } else {
        const void* safe = fd.safe;
        if (fd.fast) fd.fill_fast(dst, k0);
        else
#pragma unroll
        for (int i = 0; i < GPIECES; ++i) {
          const PieceSrc src = fd.src(i, k0);
          const uint32_t d = dst + fd.offset(i);
          if (src.valid > 0 && (reinterpret_cast<uintptr_t>(src.p) & 15u) != 0)
            copy_piece_slow(d, src.p, src.valid, safe);
          else
            hcp16(d, src.valid > 0 ? static_cast<const void*>(src.p) : safe, src.valid * 2);
        }
      }
      // The slice just issued is announced one k-block later, when its copies have landed;
      // the copies of the next slice are in flight meanwhile.
      asm volatile("cp.async.commit_group;" ::: "memory");
      if (it > 0) {
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        announce(sig);
        if (++sig == GSTAGES) sig = 0;
      }
      if (++s == GSTAGES) {
        s = 0;
        ph ^= 1u;
      }
      k0 += GBK;
      if (k0 >= P.k[pair]) {
        ++pair;
        k0 = 0;
        if (it + 1 < nkb) setup(pair);
      }
      }  // it >= 0
      if (it + 1 < nkb && via_regs(pair)) {  // prefetch the next slice while this one is consumed
        load_regs(k0);
        regs_loaded = true;
      }
    }
    if (ok && nkb > 0) {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      announce(sig);
    }
    if (want_rowsum && ok) {
      // Outer-contiguous A: every piece of this thread covers the same 8 rows.
      const int row = m0 + 8 * (t & 15);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (row + e < P.M)
          atomicAdd(static_cast<__half*>(P.rowsum) + row + e, __float2half_rn(rs[e]));
    }

    // ===================== epilogue (eight warps, 64 columns each) =====================
    if (ok && mbar_wait(smem_u32(&acc_bar), 0, status, DEV_TIMEOUT_ACCUM, 0)) {
      tc_fence_after();
      const int q = warp & 3;
      const int cbeg = ((warp - 1) >> 2) * 64;
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < P.M;
      const float bias = (P.bias != nullptr && row_ok)
                             ? __half2float(static_cast<const __half*>(P.bias)[row]) : 0.f;
      __half* cbase = static_cast<__half*>(P.c) + batch * P.c_batch_stride;
      const uint32_t tbase = tmem + (static_cast<uint32_t>(q * 32) << 16);
      void* const* ccols = P.ccols;
      const long long ldc = P.ldc;
      const int N = P.N, act = P.act;
      const bool load_c = P.accumulate && row_ok;
      // eight columns per pass, not unrolled: the epilogue runs once per CTA, so its code size
      // is pure instruction-fetch time
#pragma unroll 1
      for (int c0 = cbeg; c0 < cbeg + 64; c0 += 8) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int col = n0 + c0 + j;
          float v = bias;
          if (load_c && col < N)
            v += __half2float((ccols ? static_cast<const __half*>(ccols[col])
                                     : cbase + static_cast<long long>(col) * ldc)[row]);
          acc[j] = v;
        }
        if (nkb > 0) {
          uint32_t v[8];
          tmem_ld8(tbase + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += __uint_as_float(v[j]);
        }
        if (act != ACT_NONE) {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = act_forward_half(act, acc[j]);
        }
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int col = n0 + c0 + j;
            if (col < N)
              (ccols ? static_cast<__half*>(ccols[col]) : cbase + static_cast<long long>(col) * ldc)[row] =
                  __float2half_rn(acc[j]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, GBN);
  }
}

template <bool GROUPED, bool WITH_REGS>
cudaError_t launch_hgather(const Problem& p, const Problem* dprobs, int nprobs, int total_tiles,
                           cudaStream_t stream, int* status) {
  auto kern = hgemm_gather_kernel<GROUPED, WITH_REGS>;
  const int smem = GSTAGES * GSTAGE + 1024;
  static unsigned long long smem_set = 0;  // per template instantiation: per kernel
  cudaError_t e = set_smem_limit_once(reinterpret_cast<const void*>(kern), smem, &smem_set);
  if (e != cudaSuccess) return e;
  kern<<<total_tiles, GTHREADS, smem, stream>>>(p, dprobs, nprobs, status);
  return cudaGetLastError();
}

}  // namespace

// Any fp16 problem with k > 0; the bias gradient needs an outer-contiguous A operand.
bool hgemm_gather_supported(const Problem& p) {
  if (p.npairs < 1) return false;
  for (int i = 0; i < p.npairs; ++i)
    if (p.k[i] <= 0 || p.k[i] > 0x7fffffffLL) return false;
  if (p.rowsum != nullptr && p.a[0].k_contig) return false;
  return true;
}

cudaError_t launch_hgemm_gather(Problem& p, cudaStream_t stream, int* status) {
  p.tiles_m = (p.M + GBM - 1) / GBM;
  p.tiles_n = (p.N + GBN - 1) / GBN;
  p.tile_start = 0;
  const long long total = static_cast<long long>(p.tiles_m) * p.tiles_n * p.batches;
  if (total <= 0) return cudaSuccess;
  if (total > 0x7fffffffLL) return cudaErrorInvalidValue;
  bool regs = p.rowsum != nullptr;
  for (int i = 0; i < p.npairs; ++i) regs = regs || p.a[i].dact != ACT_NONE || p.b[i].dact != ACT_NONE;
  return regs ? launch_hgather<false, true>(p, nullptr, 1, static_cast<int>(total), stream, status)
              : launch_hgather<false, false>(p, nullptr, 1, static_cast<int>(total), stream, status);
}

cudaError_t launch_hgemm_gather_grouped(const Problem* dprobs, int nprobs, int total_tiles,
                                        cudaStream_t stream, int* status) {
  if (total_tiles <= 0) return cudaSuccess;
  Problem dummy{};
  return launch_hgather<true, true>(dummy, dprobs, nprobs, total_tiles, stream, status);
}

}  // namespace gb
