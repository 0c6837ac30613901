// fp16 GEMM on CTA pairs (tcgen05 cta_group::2) for large, 16-byte-aligned problems:
//   C = op(A) * op(B) [+ C], column-major, optionally strided-batched.
//
// Two CTAs of a cluster work on one 256 x 256 tile of C.  CTA r of the pair holds rows
// [128 r, 128 r + 128) of the A slice, columns [128 r, 128 r + 128) of the B slice and the
// matching 128 accumulator lanes (256 fp32 columns, double buffered = all 512 TMEM columns).
// The even CTA issues one tcgen05.mma (M = 256, N = 256, K = 16) for both; the tensor cores read
// the two B halves from both CTAs' shared memory, so each SM stages only half of B: per k-block
// 32 KiB per CTA instead of 48 KiB, which is what lets the ring run six stages deep and keeps
// shared-memory traffic off the tensor pipe's critical path.
//
//   warp 0      TMA producer (in both CTAs): its own A rows and B half, completion counted on
//               the even CTA's "full" barrier.  Plain loads, no multicast.
//   warp 1      TMEM allocation (both CTAs); MMA issue (even CTA only).  tcgen05.commit releases
//               the ring stage in both CTAs and publishes the accumulator to both epilogues.
//   warps 2..5  epilogue of the CTA's own 128 rows, overlapped with the next tile's main loop.
#include <cuda.h>
#include <cstring>
#include "ptx.cuh"
#include "math.cuh"
#include "launch.h"

namespace gb {

namespace {

constexpr int PBM = 256, PBN = 256, PBK = 64;   // tile of the CTA pair
constexpr int PSTAGES = 6;
constexpr int PA_BYTES = 128 * PBK * 2;          // 16 KiB: this CTA's A rows
constexpr int PB_BYTES = 128 * PBK * 2;          // 16 KiB: this CTA's half of B
constexpr int PSTAGE_BYTES = PA_BYTES + PB_BYTES;
constexpr int PATOM_BYTES = 64 * PBK * 2;        // one 64 x 64 box of an MN-major operand
constexpr int PEPI_PITCH = 36;
constexpr int PEPI_WARP_BYTES = 32 * PEPI_PITCH * 4;
constexpr int PEPI_BYTES = 4 * PEPI_WARP_BYTES;
// Ring through which the even CTA's producer announces tile numbers to every other role of the
// pair.  Depth: with at least two k-blocks per tile (K > 64, which hgemm_pair_supported requires)
// the six-stage ring holds at most three tiles, and the MMA warp runs at most two accumulators
// ahead of the epilogues, so the producer is never more than five tiles ahead of the slowest
// reader and eight slots cannot be overrun.
constexpr int PSCHED = 8;

struct PParams {
  __half* C;
  long long ldc, strideC;
  int M, N, K, batches;
  int accumulate;
  int vec_c;
  int tiles_m, tiles_n, total_tiles;
  int group_m;  // m-tiles per rasterisation group (L2 reuse of the A rows across waves)
  // L2 eviction hints.  Bit 0: the A slices (re-read by every column of a rasterisation group)
  // are loaded evict-last, the B slices (used by one wave) evict-first; bit 1: C is read and
  // written with streaming accesses.
  int l2_hint;
  // Fused Affine epilogue: out = act(fp16(acc [+ C]) + bias[row]); bias may be null, act NONE.
  const __half* bias;
  int act;
  int vec_bias;  // bias allows 16-byte loads
  // Work queue: tiles [0, #pairs) are taken statically, every further tile is claimed with an
  // atomic add on counter[0].  A pair that starts late -- because another kernel, e.g. an NCCL
  // collective, holds its SMs for a while -- then simply finds fewer tiles left instead of
  // delaying the end of the launch.  counter[1] counts the pairs that have finished; the last
  // one puts both words back to zero, so the next launch needs no memset of its own (a memset
  // queued on another stream could otherwise clear the counter of a launch that is running).
  int* counter;
};

__device__ __forceinline__ void pair_decode_tile(const PParams& p, int t, int& m_idx, int& n_idx,
                                                 int& batch) {
  const int per_batch = p.tiles_m * p.tiles_n;
  batch = t / per_batch;
  const int r = t % per_batch;
  const int group_span = p.group_m * p.tiles_n;
  const int g = r / group_span;
  const int first_m = g * p.group_m;
  const int gm = min(p.group_m, p.tiles_m - first_m);
  const int in_g = r % group_span;
  m_idx = first_m + in_g % gm;
  n_idx = in_g / gm;
}

template <int A_MN, int B_MN>
__global__ void __launch_bounds__(192, 1)
hgemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const PParams p, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[PSTAGES];   // used in the even CTA
  __shared__ __align__(8) uint64_t empty_bar[PSTAGES];  // one per CTA
  __shared__ __align__(8) uint64_t acc_full[2];         // one per CTA
  __shared__ __align__(8) uint64_t acc_empty[2];        // used in the even CTA (8 arrivals)
  __shared__ __align__(8) uint64_t sched_full[PSCHED];  // one per CTA: tile number announced
  __shared__ int tile_ring[PSCHED];
  __shared__ uint32_t tmem_slot;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = issues the MMAs
  const int cluster_id = blockIdx.x >> 1;
  const int nclusters = gridDim.x >> 1;
  const uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int nkb = (p.K + PBK - 1) / PBK;
  constexpr uint32_t IDESC = make_idesc(0, A_MN, B_MN, PBM, PBN);

  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    if (lane == 0) {
      for (int s = 0; s < PSTAGES; ++s) {
        mbar_init(smem_u32(&full_bar[s]), 1);
        mbar_init(smem_u32(&empty_bar[s]), 1);
      }
      for (int a = 0; a < 2; ++a) {
        mbar_init(smem_u32(&acc_full[a]), 1);
        mbar_init(smem_u32(&acc_empty[a]), 8);
      }
      for (int i = 0; i < PSCHED; ++i) mbar_init(smem_u32(&sched_full[i]), 1);
      fence_mbar_init();
    }
    __syncwarp();
    tmem_alloc_pair(smem_u32(&tmem_slot), 512);
    tmem_relinquish_pair();
    tc_fence_before();
  }
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them remotely
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  // Tile number of this pair's i-th tile, as announced by the even CTA's producer (-1 = none).
  auto announced_tile = [&](int i) -> int {
    const int slot = i % PSCHED;
    if (!mbar_wait_cluster(smem_u32(&sched_full[slot]), (i / PSCHED) & 1u, status,
                           DEV_TIMEOUT_FULL, 0x400 + (i & 0xff)))
      return -1;
    return *reinterpret_cast<volatile int*>(&tile_ring[slot]);
  };
  // Even CTA's producer: claim the i-th tile and announce it to both CTAs.
  auto claim_tile = [&](int i) -> int {
    int t = cluster_id;
    if (i > 0) t = nclusters + atomicAdd(p.counter, 1);
    if (t >= p.total_tiles) t = -1;
    const int slot = i % PSCHED;
    *reinterpret_cast<volatile int*>(&tile_ring[slot]) = t;
    st_shared_remote(mapa_shared(smem_u32(&tile_ring[slot]), 1), static_cast<uint32_t>(t));
    mbar_arrive(smem_u32(&sched_full[slot]));
    mbar_arrive_remote(mapa_shared(smem_u32(&sched_full[slot]), 1));
    return t;
  };

  if (warp == 0) {
    // ===================== TMA producer (both CTAs) =====================
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      const uint64_t pol_a = make_l2_policy(true), pol_b = make_l2_policy(false);
      for (int i = 0; ok; ++i) {
        const int t = rank == 0 ? claim_tile(i) : announced_tile(i);
        if (t < 0) break;
        int m_idx, n_idx, batch;
        pair_decode_tile(p, t, m_idx, n_idx, batch);
        const int m0 = m_idx * PBM + static_cast<int>(rank) * 128;
        const int n0 = n_idx * PBN + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, status, DEV_TIMEOUT_EMPTY, kb)) {
            ok = false;
            break;
          }
          const uint32_t bar = mapa_shared(smem_u32(&full_bar[s]), 0);
          const uint32_t a_s = tiles_base + s * PSTAGE_BYTES;
          const uint32_t b_s = a_s + PA_BYTES;
          const int k0 = kb * PBK;
          // The even CTA announces the bytes of both CTAs for this stage.
          if (rank == 0) mbar_arrive_expect_tx(smem_u32(&full_bar[s]), 2 * PSTAGE_BYTES);
          if (p.l2_hint & 1) {
            if (A_MN) {
              tma_load_3d_pair_hint(a_s, &tmA, bar, m0, k0, batch, pol_a);
              tma_load_3d_pair_hint(a_s + PATOM_BYTES, &tmA, bar, m0 + 64, k0, batch, pol_a);
            } else {
              tma_load_3d_pair_hint(a_s, &tmA, bar, k0, m0, batch, pol_a);
            }
            if (B_MN) {
              tma_load_3d_pair_hint(b_s, &tmB, bar, n0, k0, batch, pol_b);
              tma_load_3d_pair_hint(b_s + PATOM_BYTES, &tmB, bar, n0 + 64, k0, batch, pol_b);
            } else {
              tma_load_3d_pair_hint(b_s, &tmB, bar, k0, n0, batch, pol_b);
            }
          } else {
            if (A_MN) {
              tma_load_3d_pair(a_s, &tmA, bar, m0, k0, batch);
              tma_load_3d_pair(a_s + PATOM_BYTES, &tmA, bar, m0 + 64, k0, batch);
            } else {
              tma_load_3d_pair(a_s, &tmA, bar, k0, m0, batch);
            }
            if (B_MN) {
              tma_load_3d_pair(b_s, &tmB, bar, n0, k0, batch);
              tma_load_3d_pair(b_s + PATOM_BYTES, &tmB, bar, n0 + 64, k0, batch);
            } else {
              tma_load_3d_pair(b_s, &tmB, bar, k0, n0, batch);
            }
          }
          if (++s == PSTAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer (even CTA only) =====================
    if (rank == 0 && elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (; ok; ++it) {
        if (announced_tile(it) < 0) break;
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1u;
        if (!mbar_wait(smem_u32(&acc_empty[acc]), acc_ph ^ 1u, status, DEV_TIMEOUT_TMEM_FREE, it)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d = tmem + acc * PBN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, status, DEV_TIMEOUT_FULL, kb)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_s = tiles_base + s * PSTAGE_BYTES;
          const uint32_t b_s = a_s + PA_BYTES;
#pragma unroll
          for (int ks = 0; ks < PBK / 16; ++ks) {
            const uint64_t ad = A_MN ? make_smem_desc(a_s + ks * 2048, PATOM_BYTES, 1024)
                                     : make_smem_desc(a_s + ks * 32, 16, 1024);
            const uint64_t bd = B_MN ? make_smem_desc(b_s + ks * 2048, PATOM_BYTES, 1024)
                                     : make_smem_desc(b_s + ks * 32, 16, 1024);
            mma_f16_pair(d, ad, bd, IDESC, (kb > 0 || ks > 0) ? 1u : 0u);
          }
          // free this ring stage in both CTAs
          tc_commit_pair(smem_u32(&empty_bar[s]));
          tc_commit_pair(mapa_shared(smem_u32(&empty_bar[s]), 1));
          if (++s == PSTAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
        // publish the accumulator to both epilogues
        tc_commit_pair(smem_u32(&acc_full[acc]));
        tc_commit_pair(mapa_shared(smem_u32(&acc_full[acc]), 1));
      }
    }
    __syncwarp();
  } else {
    // ===================== epilogue (both CTAs, own 128 rows) =====================
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int it = 0;
    bool ok = true;
    const bool fused = p.bias != nullptr || p.act != ACT_NONE;
    for (; ok; ++it) {
      const int t = announced_tile(it);
      if (t < 0) break;
      int m_idx, n_idx, batch;
      pair_decode_tile(p, t, m_idx, n_idx, batch);
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1u;
      if (!mbar_wait(smem_u32(&acc_full[acc]), acc_ph, status, DEV_TIMEOUT_ACCUM, it)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row0 = m_idx * PBM + static_cast<int>(rank) * 128 + q * 32;
      const int n0 = n_idx * PBN;
      __half* cbase = p.C + static_cast<long long>(batch) * p.strideC;
      const uint32_t taddr = tmem + (static_cast<uint32_t>(q * 32) << 16) + acc * PBN;
      float* stage = reinterpret_cast<float*>(smem_raw + (tiles_base - smem_u32(smem_raw)) +
                                              PSTAGES * PSTAGE_BYTES + q * PEPI_WARP_BYTES);
#pragma unroll 1
      for (int c0 = 0; c0 < PBN; c0 += 32) {
        // Each lane owns 4 pieces of the 32x32 chunk: 8 consecutive rows of one column (16 B of C).
        uint4 cold[4];
        if (p.accumulate && p.vec_c) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int piece = lane + 32 * i;
            const int col = n0 + c0 + (piece >> 2), row = row0 + (piece & 3) * 8;
            cold[i] = make_uint4(0, 0, 0, 0);
            if (col < p.N && row + 8 <= p.M)
              {
                const uint4* src = reinterpret_cast<const uint4*>(cbase + static_cast<long long>(col) * p.ldc + row);
                cold[i] = (p.l2_hint & 2) ? __ldcs(src) : *src;
              }
          }
        }
        uint32_t v[32];
        tmem_ld32(taddr + c0, v);
        tmem_ld_wait();
        if (c0 + 32 == PBN) {
          // Accumulator drained into registers: hand it back to the MMA warp of the even CTA.
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(mapa_shared(smem_u32(&acc_empty[acc]), 0));
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) stage[j * PEPI_PITCH + lane] = __uint_as_float(v[j]);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int piece = lane + 32 * i;
          const int cl = piece >> 2, rg = piece & 3;
          const int col = n0 + c0 + cl, row = row0 + rg * 8;
          if (col >= p.N || row >= p.M) continue;
          const float4 x0 = *reinterpret_cast<const float4*>(stage + cl * PEPI_PITCH + rg * 8);
          const float4 x1 = *reinterpret_cast<const float4*>(stage + cl * PEPI_PITCH + rg * 8 + 4);
          float x[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
          __half* cp = cbase + static_cast<long long>(col) * p.ldc + row;
          if (fused) {
            // The reference rounds the product (and the sum with the previous pairs) to fp16,
            // adds the bias and applies the nonlinearity to that: the same roundings here.
            const bool vec = p.vec_c && row + 8 <= p.M;
            if (p.accumulate) {
              if (vec) {
                const __half* o = reinterpret_cast<const __half*>(&cold[i]);
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] += __half2float(o[e]);
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e)
                  if (row + e < p.M) x[e] += __half2float(cp[e]);
              }
            }
            float b[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) b[e] = 0.f;
            if (p.bias != nullptr) {
              if (p.vec_bias && row + 8 <= p.M) {
                const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + row);
                const __half* bh = reinterpret_cast<const __half*>(&bv);
#pragma unroll
                for (int e = 0; e < 8; ++e) b[e] = __half2float(bh[e]);
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e)
                  if (row + e < p.M) b[e] = __half2float(p.bias[row + e]);
              }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e)
              x[e] = act_forward_half(p.act, __half2float(__float2half_rn(x[e])) + b[e]);
            if (vec) {
              uint4 out;
              __half2* oh = reinterpret_cast<__half2*>(&out);
#pragma unroll
              for (int e = 0; e < 4; ++e) oh[e] = __floats2half2_rn(x[2 * e], x[2 * e + 1]);
              if (p.l2_hint & 2) __stcs(reinterpret_cast<uint4*>(cp), out);
              else *reinterpret_cast<uint4*>(cp) = out;
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e)
                if (row + e < p.M) cp[e] = __float2half_rn(x[e]);
            }
            continue;
          }
          if (p.vec_c && row + 8 <= p.M) {
            if (p.accumulate) {
              const __half* o = reinterpret_cast<const __half*>(&cold[i]);
#pragma unroll
              for (int e = 0; e < 8; ++e) x[e] += __half2float(o[e]);
            }
            uint4 out;
            __half2* oh = reinterpret_cast<__half2*>(&out);
#pragma unroll
            for (int e = 0; e < 4; ++e) oh[e] = __floats2half2_rn(x[2 * e], x[2 * e + 1]);
            if (p.l2_hint & 2) __stcs(reinterpret_cast<uint4*>(cp), out);
              else *reinterpret_cast<uint4*>(cp) = out;
          } else {
            for (int e = 0; e < 8 && row + e < p.M; ++e) {
              float y = x[e];
              if (p.accumulate) y += __half2float(cp[e]);
              cp[e] = __float2half_rn(y);
            }
          }
        }
        __syncwarp();
      }
    }
  }

  // Neither CTA may leave while the other can still touch its shared memory or barriers.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem, 512);
  }
  // This pair has made its last claim (the even CTA's producer left its loop before the
  // barriers above).  The last pair to get here re-arms the queue for the next launch.
  if (rank == 0 && threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.counter + 1, 1) == nclusters - 1) {
      p.counter[0] = 0;
      p.counter[1] = 0;
      __threadfence();
    }
  }
}

template <int A_MN, int B_MN>
cudaError_t launch_pair_variant(const CUtensorMap& ta, const CUtensorMap& tb, const PParams& p,
                                int num_sms, cudaStream_t stream, int* status) {
  auto kern = hgemm_pair_kernel<A_MN, B_MN>;
  const int smem = PSTAGES * PSTAGE_BYTES + PEPI_BYTES + 1024;
  static unsigned long long smem_set = 0;  // per template instantiation: per kernel
  cudaError_t e = set_smem_limit_once(reinterpret_cast<const void*>(kern), smem, &smem_set);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // How many CTA pairs can be resident at once (one CTA per SM, pairs inside a GPC).
  cfg.gridDim = dim3(2 * (num_sms / 2), 1, 1);
  int max_clusters = 0;
  e = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);
  if (e != cudaSuccess) return e;
  if (max_clusters < 1) return cudaErrorLaunchOutOfResources;
  int clusters = p.total_tiles < max_clusters ? p.total_tiles : max_clusters;
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  return cudaLaunchKernelEx(&cfg, kern, ta, tb, p, status);
}

}  // namespace

bool hgemm_pair_supported(const HgemmArgs& a) {
  if (!hgemm_tma_supported(a)) return false;
  // At least two k-blocks per tile: the tile-announcement ring's depth is sized for that.
  if (a.K <= PBK) return false;
  // 16-byte accesses to C keep the two epilogues cheap; fall back to the one-CTA kernel otherwise.
  return (reinterpret_cast<uintptr_t>(a.C) & 15u) == 0 && a.ldc % 8 == 0 &&
         (a.batches == 1 || a.strideC % 8 == 0);
}

cudaError_t launch_hgemm_pair(const HgemmArgs& a, int num_sms, int group_m, int l2_hint,
                              int* counter, cudaStream_t stream, int* status) {
  const unsigned long long a_rows = a.transA ? a.K : a.M, a_cols = a.transA ? a.M : a.K;
  const unsigned long long b_rows = a.transB ? a.N : a.K, b_cols = a.transB ? a.K : a.N;
  const unsigned long long sa = a.batches > 1 ? a.strideA : a.lda * a_cols;
  const unsigned long long sb = a.batches > 1 ? a.strideB : a.ldb * b_cols;
  CUtensorMap ta, tb;
  // Every box covers this CTA's 128 rows (A) or 128 columns (B) of the pair's tile.
  if (!encode_tmap(&ta, 2, a.A, a_rows, a_cols, a.batches, a.lda, sa, 64, a.transA ? 128 : PBK, true))
    return cudaErrorInvalidValue;
  if (!encode_tmap(&tb, 2, a.B, b_rows, b_cols, a.batches, a.ldb, sb, 64, a.transB ? PBK : 128, true))
    return cudaErrorInvalidValue;
  PParams p;
  p.C = static_cast<__half*>(a.C);
  p.ldc = a.ldc;
  p.strideC = a.strideC;
  p.M = a.M; p.N = a.N; p.K = a.K; p.batches = a.batches;
  p.accumulate = a.accumulate;
  p.vec_c = 1;
  p.tiles_m = (a.M + PBM - 1) / PBM;
  p.tiles_n = (a.N + PBN - 1) / PBN;
  const long long total = static_cast<long long>(p.tiles_m) * p.tiles_n * a.batches;
  if (total > 0x7fffffffLL) return cudaErrorInvalidValue;
  p.total_tiles = static_cast<int>(total);
  p.l2_hint = l2_hint & 3;
  p.group_m = group_m > 0 ? group_m : 8;
  p.counter = counter;
  if ((a.bias != nullptr || a.act != ACT_NONE) && a.batches != 1) return cudaErrorInvalidValue;
  p.bias = static_cast<const __half*>(a.bias);
  p.act = a.act;
  p.vec_bias = (reinterpret_cast<uintptr_t>(a.bias) & 15u) == 0 ? 1 : 0;
  if (!a.transA && !a.transB) return launch_pair_variant<1, 0>(ta, tb, p, num_sms, stream, status);
  if (a.transA && !a.transB) return launch_pair_variant<0, 0>(ta, tb, p, num_sms, stream, status);
  return launch_pair_variant<1, 1>(ta, tb, p, num_sms, stream, status);
}

}  // namespace gb
