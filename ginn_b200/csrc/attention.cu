// Fused attention forward for ginn's min-GPT pattern (examples/min-gpt.cu.cpp:124-157), fp32:
//   S = K' * Q * scale  ->  causal mask  ->  column softmax  ->  O = V * P
// per (batch, head), with ginn's layouts: K' is T x hs, Q and V are hs x T, S / P are T x T (row
// = key position, column = query position; Softmax normalises over rows), O is hs x T.  The
// reference materialises S (BatchedProd), scales and masks it in place, runs Softmax into a
// second T x T tensor and feeds that to another BatchedProd; here the scores never leave the
// SM: they are accumulated in tensor memory, normalised by the threads that own their rows, and
// re-staged in shared memory as the left operand of the second product.  P is written to HBM
// only when the caller asks for it (the backward pass of SoftmaxOp needs it).
//
// One CTA serves 128 query positions j of one (batch, head).  Transposed problem, so that a
// softmax column is one TMEM lane:
//   phase A   S^T[j, i] = sum_h Q[h, j] K'[i, h]      M = 128 (j), N = T (i), K = hs
//   phase B   per lane j: m = max_i s, l = sum_i exp(s - m)          (s = scale * S, masked)
//   phase C   O^T[j, h] = sum_i P^T[j, i] V[h, i]      M = 128 (j), N = hs,   K = T
// Both products use three TF32 tensor-core products per term (hi*hi, hi*lo, lo*hi of values
// split as hi = rna_tf32(x), lo = x - hi), the same scheme as sgemm3x_tma.cu; the contractions
// are short (hs and T <= 256), so one fp32 accumulator per product keeps the error far below
// the 1e-5 bound.
//   warp 0      TMA producer: raw slices of Q, K' (phase A) and V (phase C)
//   warp 1      MMA issuer
//   warps 2-17  phase A: split Q / K' slices into hi / lo planes; phase B: softmax statistics;
//               phase C: P = exp(s - m) / l for one 32-key block at a time, split into planes
//               (and stored to HBM if wanted), V slices split alongside; then the epilogue.
// Limits: T <= 256, T % 4 == 0, hs in {32, 64, 128}, 16-byte aligned operands.
#include <cuda.h>
#include <cstdio>
#include <cstring>
#include "ptx.cuh"
#include "math.cuh"
#include "launch.h"

namespace gb {

namespace {

constexpr int ATM = 128;                 // query positions per CTA
constexpr int ABK = 32;                  // contraction slice
constexpr int ARAW_TILE = 128 * ABK * 4; // 16 KiB raw slice of a 128-row operand
constexpr int ARAW_STAGE = 2 * ARAW_TILE;
constexpr int ARAW_STAGES = 2;
constexpr int APLANE = 16384;
constexpr int APLANE_STAGE = 4 * APLANE; // A hi, A lo, B hi, B lo
constexpr int APLANE_STAGES = 2;
constexpr int AXFORM = 512;
constexpr int ATHREADS = 64 + AXFORM;
constexpr uint32_t O_COL = 256;          // TMEM: S^T in columns [0, 256), O^T from 256

struct AttParams {
  CUtensorMap tmQ, tmK, tmV;
  float* O;
  long long ldo, strideO;
  float* P;  // may be null
  long long ldp, strideP;
  int T, hs, nb;
  float scale;
  int causal;
};

// k-contiguous raw slice (TMA box 32 k x 128 rows, 128-byte swizzle) -> hi / lo planes.
// One guard for the thread's sixteen values (see math.cuh).
__device__ __forceinline__ void split_kc(const uint8_t* src, uint8_t* dst_hi, uint8_t* dst_lo, int t) {
  float4 x[4];
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[i] = *reinterpret_cast<const float4*>(src + (t + 256 * i) * 16);
    m = fmaxf(m, absmax4(x[i]));
  }
  if (guard_ok(m)) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float4 h, l;
      split4<false>(x[i], h, l);
      *reinterpret_cast<float4*>(dst_hi + (t + 256 * i) * 16) = h;
      *reinterpret_cast<float4*>(dst_lo + (t + 256 * i) * 16) = l;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float4 h, l;
      split4<true>(x[i], h, l);
      *reinterpret_cast<float4*>(dst_hi + (t + 256 * i) * 16) = h;
      *reinterpret_cast<float4*>(dst_lo + (t + 256 * i) * 16) = l;
    }
  }
}

// Outer-contiguous raw slice [box of 32 outer][32 k][32 outer] (unswizzled TMA boxes) ->
// transposed, swizzled K-major planes.  `outer` rows (32, 64 or 128) are shared by `nthreads`
// threads (a power of two with 32 * outer / nthreads >= 4): thread t owns row t % outer and
// 32 * outer / nthreads consecutive k values.
__device__ __forceinline__ void split_oc(const uint8_t* src, uint8_t* dst_hi, uint8_t* dst_lo, int t,
                                         int outer, int nthreads = 256) {
  const int o = t & (outer - 1);
  const int kper = 32 * outer / nthreads;  // 4, 8 or 16
  const int kbase = (t / outer) * kper;
  const float* col = reinterpret_cast<const float*>(src + (o >> 5) * 4096) + (o & 31);
  for (int c = 0; c < kper; c += 4) {
    float4 x;
    x.x = col[(kbase + c) * 32];
    x.y = col[(kbase + c + 1) * 32];
    x.z = col[(kbase + c + 2) * 32];
    x.w = col[(kbase + c + 3) * 32];
    float4 h, l;
    if (guard_ok(absmax4(x)))
      split4<false>(x, h, l);
    else
      split4<true>(x, h, l);
    const uint32_t off = sw128_offset(o, (kbase + c) >> 2);
    *reinterpret_cast<float4*>(dst_hi + off) = h;
    *reinterpret_cast<float4*>(dst_lo + off) = l;
  }
}

// hi / lo split of a finite value of moderate size (softmax outputs): the rounding of
// split_tf32 without its guard for infinities.
__device__ __forceinline__ void split_finite(float x, float& hi, float& lo) {
  hi = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
  lo = x - hi;
}

__global__ void __launch_bounds__(ATHREADS, 1)
attention_fwd_kernel(const __grid_constant__ AttParams p, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t raw_full[ARAW_STAGES];
  __shared__ __align__(8) uint64_t raw_empty[ARAW_STAGES];
  __shared__ __align__(8) uint64_t plane_full[APLANE_STAGES];
  __shared__ __align__(8) uint64_t plane_empty[APLANE_STAGES];
  __shared__ __align__(8) uint64_t s_full, o_full;
  __shared__ uint32_t tmem_slot;
  __shared__ float red[4][ATM];  // per column group: row maxima, then row sums
#ifdef GB_PHASE_TIMES  // instrumented build (-DGB_PHASE_TIMES): two CTAs print their phase durations
  __shared__ long long ph_t[12];
  if (threadIdx.x == 0) ph_t[0] = clock64();
#define APH(i) do { if (threadIdx.x == 64) ph_t[i] = clock64(); } while (0)
#else
#define APH(i) do { } while (0)
#endif

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t planes_base = base;
  const uint32_t raws_base = base + APLANE_STAGES * APLANE_STAGE;

  const int jblocks = (p.T + ATM - 1) / ATM;
  const int batch = blockIdx.x / jblocks;
  const int j0 = (blockIdx.x % jblocks) * ATM;
  const int nkbA = p.hs / ABK;              // k-blocks of phase A
  const int halves = (p.T + 127) / 128;     // 128-key groups of S^T
  const int nA = nkbA * halves;
  const int nC = (p.T + ABK - 1) / ABK;     // k-blocks of phase C

  if (warp == 0 && lane == 0) {
    prefetch_tmap(&p.tmQ);
    prefetch_tmap(&p.tmK);
    prefetch_tmap(&p.tmV);
  }
  if (warp == 1) {
    if (lane == 0) {
      for (int s = 0; s < ARAW_STAGES; ++s) {
        mbar_init(smem_u32(&raw_full[s]), 1);
        mbar_init(smem_u32(&raw_empty[s]), AXFORM);
      }
      for (int s = 0; s < APLANE_STAGES; ++s) {
        mbar_init(smem_u32(&plane_full[s]), AXFORM);
        mbar_init(smem_u32(&plane_empty[s]), 1);
      }
      mbar_init(smem_u32(&s_full), 1);
      mbar_init(smem_u32(&o_full), 1);
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
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0; it < nA + nC; ++it) {
        if (!mbar_wait(smem_u32(&raw_empty[s]), ph ^ 1u, status, DEV_TIMEOUT_EMPTY, 0x500 + it)) break;
        const uint32_t bar = smem_u32(&raw_full[s]);
        const uint32_t dst = raws_base + s * ARAW_STAGE;
        if (it < nA) {
          const int half = it / nkbA, k0 = (it % nkbA) * ABK;
          mbar_arrive_expect_tx(bar, ARAW_STAGE);
          tma_load_3d(dst, &p.tmQ, bar, k0, j0, batch);  // Q^T slice: 32 h x 128 j, swizzled
#pragma unroll
          for (int a = 0; a < 4; ++a)                    // K' slice: 128 i x 32 h as four boxes
            tma_load_3d(dst + ARAW_TILE + a * 4096, &p.tmK, bar, half * 128 + 32 * a, k0, batch);
        } else {
          const int i0 = (it - nA) * ABK;
          mbar_arrive_expect_tx(bar, (p.hs / 32) * 4096);
          for (int a = 0; a < p.hs / 32; ++a)            // V slice: hs x 32 i as boxes of 32 h
            tma_load_3d(dst + a * 4096, &p.tmV, bar, 32 * a, i0, batch);
        }
        if (++s == ARAW_STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (elect_one()) {
      constexpr uint32_t IDESC_A = make_idesc(2, 0, 0, ATM, 128);
      const uint32_t idesc_c = make_idesc(2, 0, 0, ATM, static_cast<uint32_t>(p.hs));
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0; it < nA + nC; ++it) {
        if (!mbar_wait(smem_u32(&plane_full[s]), ph, status, DEV_TIMEOUT_FULL, 0x500 + it)) break;
        tc_fence_after();
        const uint32_t a_hi = planes_base + s * APLANE_STAGE;
        const uint32_t a_lo = a_hi + APLANE;
        const uint32_t b_hi = a_hi + 2 * APLANE;
        const uint32_t b_lo = a_hi + 3 * APLANE;
        const bool phase_a = it < nA;
        const int kb = phase_a ? it % nkbA : it - nA;
        const uint32_t d = phase_a ? tmem + (it / nkbA) * 128 : tmem + O_COL;
        const uint32_t idesc = phase_a ? IDESC_A : idesc_c;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t dah = make_smem_desc(a_hi + ks * 32, 16, 1024);
          const uint64_t dal = make_smem_desc(a_lo + ks * 32, 16, 1024);
          const uint64_t dbh = make_smem_desc(b_hi + ks * 32, 16, 1024);
          const uint64_t dbl = make_smem_desc(b_lo + ks * 32, 16, 1024);
          mma_tf32(d, dal, dbh, idesc, (kb > 0 || ks > 0) ? 1u : 0u);
          mma_tf32(d, dah, dbl, idesc, 1u);
          mma_tf32(d, dah, dbh, idesc, 1u);
        }
        tc_commit(smem_u32(&plane_empty[s]));
        if (it == nA - 1) tc_commit(smem_u32(&s_full));
        if (++s == APLANE_STAGES) {
          s = 0;
          ph ^= 1u;
        }
      }
      tc_commit(smem_u32(&o_full));
    }
    __syncwarp();
  } else {
    // ===================== transform / softmax / epilogue warps =====================
    const int xt = threadIdx.x - 64;
    const int grp = xt >> 8;  // phase A: 0 = Q slices, 1 = K' slices
    const int t = xt & 255;
    const int q = warp & 3;            // TMEM lane quarter this warp may read
    const int cg = (warp - 2) >> 2;    // column group 0..3
    const int row = q * 32 + lane;     // query position inside the block = TMEM lane
    const int j = j0 + row;
    bool ok = true;
    int rs_i = 0, ps_i = 0;
    uint32_t rph = 0, pph = 0;
    auto advance = [&]() {
      if (++rs_i == ARAW_STAGES) {
        rs_i = 0;
        rph ^= 1u;
      }
      if (++ps_i == APLANE_STAGES) {
        ps_i = 0;
        pph ^= 1u;
      }
    };

    APH(1);
    // ---- phase A: split the raw Q and K' slices ----
    for (int it = 0; it < nA && ok; ++it) {
      if (!mbar_wait(smem_u32(&raw_full[rs_i]), rph, status, DEV_TIMEOUT_FULL, 0x600 + it) ||
          !mbar_wait(smem_u32(&plane_empty[ps_i]), pph ^ 1u, status, DEV_TIMEOUT_EMPTY, 0x600 + it)) {
        ok = false;
        break;
      }
      const uint8_t* src = base_ptr + APLANE_STAGES * APLANE_STAGE + rs_i * ARAW_STAGE + grp * ARAW_TILE;
      uint8_t* dst_hi = base_ptr + ps_i * APLANE_STAGE + grp * 2 * APLANE;
      if (grp == 0)
        split_kc(src, dst_hi, dst_hi + APLANE, t);
      else
        split_oc(src, dst_hi, dst_hi + APLANE, t, 128);
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&plane_full[ps_i]));
      mbar_arrive(smem_u32(&raw_empty[rs_i]));
      advance();
    }

    APH(2);
    // ---- phase B: softmax statistics of this thread's row over its share of the keys ----
    // For the statistics thread (row, cg) takes a contiguous quarter of the keys (32 columns per
    // tensor-memory load); for phase C it owns keys i with (i % 32) / 8 == cg, eight consecutive
    // keys of every 32-key block.  Any partition serves for a maximum and a sum.
    ok = ok && mbar_wait(smem_u32(&s_full), 0, status, DEV_TIMEOUT_ACCUM, 0x700);
    tc_fence_after();
    APH(3);
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t tbase = lane_base + cg * 8;
    const int last_key = p.causal ? (j < p.T - 1 ? j : p.T - 1) : p.T - 1;  // keys i <= last_key count
    // exp(scale * (S - Smax)) = 2^(S * c1 - Smax * c1) with c1 = scale * log2(e): one fused
    // multiply-add and one hardware exponential per key (scale > 0, as 1 / sqrt(hs) is).  The
    // hardware exponential is good to about 2e-7 relative, against 1e-5 allowed; libm's expf and
    // a per-key mask test made this phase and the next instruction-bound.
    const float c1 = p.scale * 1.44269502f;
    const int quarter = nC * 8;  // keys per column group (nC blocks of 32 keys in all)
    float m = -INFINITY;         // maximum of the raw scores of this row
    if (ok) {
      for (int c = 0; c < quarter; c += 32) {
        uint32_t v[32];
        tmem_ld32(lane_base + cg * quarter + c, v);
        tmem_ld_wait();
        const int i0 = cg * quarter + c;
        if (i0 + 31 <= last_key && c + 32 <= quarter) {  // the usual case: nothing masked
#pragma unroll
          for (int e = 0; e < 32; ++e) m = fmaxf(m, __uint_as_float(v[e]));
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (c + e < quarter && i0 + e <= last_key) m = fmaxf(m, __uint_as_float(v[e]));
        }
      }
    }
    red[cg][row] = m;
    asm volatile("bar.sync 1, %0;" ::"n"(AXFORM) : "memory");
    m = fmaxf(fmaxf(red[0][row], red[1][row]), fmaxf(red[2][row], red[3][row]));
    asm volatile("bar.sync 1, %0;" ::"n"(AXFORM) : "memory");  // everyone has read the maxima
    const float c0 = -m * c1;
    auto expo = [&](uint32_t bits) -> float {
      float y;
      asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(fmaf(__uint_as_float(bits), c1, c0)));
      return y;
    };
    float l = 0.f;
    if (ok) {
      for (int c = 0; c < quarter; c += 32) {
        uint32_t v[32];
        tmem_ld32(lane_base + cg * quarter + c, v);
        tmem_ld_wait();
        const int i0 = cg * quarter + c;
        if (i0 + 31 <= last_key && c + 32 <= quarter) {
#pragma unroll
          for (int e = 0; e < 32; ++e) l += expo(v[e]);
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (c + e < quarter && i0 + e <= last_key) l += expo(v[e]);
        }
      }
    }
    red[cg][row] = l;
    asm volatile("bar.sync 1, %0;" ::"n"(AXFORM) : "memory");
    l = (red[0][row] + red[1][row]) + (red[2][row] + red[3][row]);
    const float inv = 1.f / l;  // key 0 always counts, so l > 0

    APH(4);
    // ---- phase C: P for one 32-key block at a time, V slices alongside ----
    float* prow = p.P ? p.P + static_cast<long long>(batch) * p.strideP + static_cast<long long>(j) * p.ldp
                      : nullptr;
    for (int kb = 0; kb < nC && ok; ++kb) {
      if (!mbar_wait(smem_u32(&raw_full[rs_i]), rph, status, DEV_TIMEOUT_FULL, 0x800 + kb) ||
          !mbar_wait(smem_u32(&plane_empty[ps_i]), pph ^ 1u, status, DEV_TIMEOUT_EMPTY, 0x800 + kb)) {
        ok = false;
        break;
      }
      uint32_t v[8];
      tmem_ld8(tbase + kb * 32, v);
      tmem_ld_wait();
      float pv[8];
      const int i0 = kb * 32 + cg * 8;
      if (i0 + 7 <= last_key) {
#pragma unroll
        for (int e = 0; e < 8; ++e) pv[e] = expo(v[e]) * inv;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) pv[e] = i0 + e <= last_key ? expo(v[e]) * inv : 0.f;
      }
      uint8_t* a_hi = base_ptr + ps_i * APLANE_STAGE;
      uint8_t* a_lo = a_hi + APLANE;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float4 h, lo4;
        split_finite(pv[4 * c + 0], h.x, lo4.x);
        split_finite(pv[4 * c + 1], h.y, lo4.y);
        split_finite(pv[4 * c + 2], h.z, lo4.z);
        split_finite(pv[4 * c + 3], h.w, lo4.w);
        const uint32_t off = sw128_offset(row, cg * 2 + c);
        *reinterpret_cast<float4*>(a_hi + off) = h;
        *reinterpret_cast<float4*>(a_lo + off) = lo4;
      }
      if (prow != nullptr && j < p.T) {
        if (i0 + 8 <= p.T) {
          *reinterpret_cast<float4*>(prow + i0) = make_float4(pv[0], pv[1], pv[2], pv[3]);
          *reinterpret_cast<float4*>(prow + i0 + 4) = make_float4(pv[4], pv[5], pv[6], pv[7]);
        } else {
          for (int e = 0; e < 8 && i0 + e < p.T; ++e) prow[i0 + e] = pv[e];
        }
      }
      {  // V slice (hs x 32 keys) -> B planes, shared by all threads (by half of them when hs = 32)
        const uint8_t* src = base_ptr + APLANE_STAGES * APLANE_STAGE + rs_i * ARAW_STAGE;
        const int nthr = p.hs >= 64 ? AXFORM : 256;
        if (xt < nthr) split_oc(src, a_hi + 2 * APLANE, a_hi + 3 * APLANE, xt, p.hs, nthr);
      }
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&plane_full[ps_i]));
      mbar_arrive(smem_u32(&raw_empty[rs_i]));
      advance();
    }

    APH(5);
    // ---- epilogue: O^T[j, h] -> O[h, j]; this thread writes hs / 4 consecutive h of column j ----
    if (ok && mbar_wait(smem_u32(&o_full), 0, status, DEV_TIMEOUT_ACCUM, 0x900)) {
      tc_fence_after();
      APH(6);
      const int per = p.hs >> 2;  // 8, 16 or 32 values
      const uint32_t obase = tmem + (static_cast<uint32_t>(q * 32) << 16) + O_COL + cg * per;
      float* ocol = p.O + static_cast<long long>(batch) * p.strideO + static_cast<long long>(j) * p.ldo + cg * per;
      for (int c = 0; c < per; c += 8) {
        uint32_t v[8];
        tmem_ld8(obase + c, v);
        tmem_ld_wait();
        if (j < p.T) {
          *reinterpret_cast<float4*>(ocol + c) = make_float4(__uint_as_float(v[0]), __uint_as_float(v[1]),
                                                             __uint_as_float(v[2]), __uint_as_float(v[3]));
          *reinterpret_cast<float4*>(ocol + c + 4) = make_float4(__uint_as_float(v[4]), __uint_as_float(v[5]),
                                                                 __uint_as_float(v[6]), __uint_as_float(v[7]));
        }
      }
    }
  }

  APH(7);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
#ifdef GB_PHASE_TIMES
  if (threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == 300))
    printf("attention phases (cycles): prologue %lld  A(split) %lld  wait S %lld  stats %lld  C %lld  "
           "wait O %lld  epilogue %lld  total %lld\n",
           ph_t[1] - ph_t[0], ph_t[2] - ph_t[1], ph_t[3] - ph_t[2], ph_t[4] - ph_t[3], ph_t[5] - ph_t[4],
           ph_t[6] - ph_t[5], ph_t[7] - ph_t[6], clock64() - ph_t[0]);
#endif
}

}  // namespace

bool attention_fused_supported(const AttentionArgs& a) {
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  if (!tmap_encoder_available()) return false;
  if (a.T < 1 || a.T > 256 || a.T % 4 != 0) return false;
  if (a.hs != 32 && a.hs != 64 && a.hs != 128) return false;
  if (a.batches < 1) return false;
  if (!al(a.K) || !al(a.Q) || !al(a.V) || !al(a.O) || (a.P && !al(a.P))) return false;
  // leading dimensions and batch strides in multiples of four elements (16 bytes)
  const long long lds[] = {a.ldk, a.ldq, a.ldv, a.ldo, a.strideK, a.strideQ, a.strideV, a.strideO,
                           a.P ? a.ldp : 4, a.P ? a.strideP : 4};
  for (long long x : lds)
    if (x % 4 != 0) return false;
  return a.ldk >= a.T && a.ldq >= a.hs && a.ldv >= a.hs && a.ldo >= a.hs && (!a.P || a.ldp >= a.T);
}

cudaError_t launch_attention_fwd(const AttentionArgs& a, cudaStream_t stream, int* status) {
  AttParams p;
  std::memset(&p, 0, sizeof(p));
  const unsigned long long T = a.T, hs = a.hs, nb = a.batches;
  // Q (hs x T): contraction index h contiguous -> one swizzled box of 32 h x 128 j
  if (!encode_tmap(&p.tmQ, 4, a.Q, hs, T, nb, a.ldq, nb > 1 ? a.strideQ : a.ldq * T, 32, 128, true))
    return cudaErrorInvalidValue;
  // K' (T x hs): key index contiguous -> unswizzled boxes of 32 i x 32 h
  if (!encode_tmap(&p.tmK, 4, a.K, T, hs, nb, a.ldk, nb > 1 ? a.strideK : a.ldk * hs, 32, 32, false))
    return cudaErrorInvalidValue;
  // V (hs x T): h contiguous, contraction over the key index -> unswizzled boxes of 32 h x 32 i
  if (!encode_tmap(&p.tmV, 4, a.V, hs, T, nb, a.ldv, nb > 1 ? a.strideV : a.ldv * T, 32, 32, false))
    return cudaErrorInvalidValue;
  p.O = static_cast<float*>(a.O);
  p.ldo = a.ldo;
  p.strideO = a.strideO;
  p.P = static_cast<float*>(a.P);
  p.ldp = a.ldp;
  p.strideP = a.strideP;
  p.T = a.T;
  p.hs = a.hs;
  p.nb = a.batches;
  p.scale = a.scale;
  p.causal = a.causal;
  const long long blocks = static_cast<long long>((a.T + ATM - 1) / ATM) * a.batches;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
  const int smem = APLANE_STAGES * APLANE_STAGE + ARAW_STAGES * ARAW_STAGE + 1024;
  static unsigned long long smem_set = 0;  // per template instantiation: per kernel
  cudaError_t e = set_smem_limit_once(reinterpret_cast<const void*>(attention_fwd_kernel), smem, &smem_set);
  if (e != cudaSuccess) return e;
  return launch_kernel(attention_fwd_kernel, dim3(static_cast<unsigned>(blocks)), dim3(ATHREADS), smem,
                       stream, pdl_enabled(), p, status);
}

}  // namespace gb
