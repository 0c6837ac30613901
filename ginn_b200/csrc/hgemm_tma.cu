// Persistent, warp-specialised fp16 GEMM (fp32 accumulation) for large, 16-byte-aligned
// problems on column-major storage:  C = op(A) * op(B) [+ C], optionally strided-batched.
//
//   warp 0      : TMA producer.  One elected thread streams 128x64 A slices and 256x64 B slices
//                 into a 4-stage ring of 128-byte-swizzled shared-memory tiles.
//   warp 1      : allocates all 512 TMEM columns (two 128x256 fp32 accumulators) and issues
//                 tcgen05.mma kind::f16; tcgen05.commit frees ring stages and publishes finished
//                 accumulators.
//   warps 2..5  : epilogue.  tcgen05.ld -> fp16 -> global, coalesced along rows; runs while the
//                 MMA warp fills the other accumulator for the next tile.
//
// Column-major operands map onto the tensor core without any transposition copy:
//   A not transposed (m x k, m contiguous)  -> MN-major operand, loaded as two 64(m) x 64(k) boxes
//   A transposed     (k x m, k contiguous)  -> K-major operand, one 64(k) x 128(m) box
//   B not transposed (k x n, k contiguous)  -> K-major operand, one 64(k) x 256(n) box
//   B transposed     (n x k, n contiguous)  -> MN-major operand, four 64(n) x 64(k) boxes
// Every CTA loads its own tiles; no cluster multicast is used anywhere.
#include <cuda.h>
#include <mutex>
#include <unordered_map>
#include <string>
#include <cstring>
#include "ptx.cuh"
#include "math.cuh"
#include "launch.h"

namespace gb {

namespace {

constexpr int TBM = 128, TBN = 256, TBK = 64, TSTAGES = 4;
constexpr int TA_BYTES = TBM * TBK * 2;  // 16 KiB
constexpr int TB_BYTES = TBN * TBK * 2;  // 32 KiB
constexpr int TSTAGE_BYTES = TA_BYTES + TB_BYTES;
constexpr int TMN_ATOM_BYTES = 64 * TBK * 2;  // one 64(mn) x 64(k) box of an MN-major operand
constexpr int TGROUP_M = 16;                  // m-tiles per rasterisation group (L2 reuse)
// Epilogue staging: per epilogue warp a 32(col) x 32(row) fp32 tile, column pitch 36 floats so
// that both the row-per-lane writes and the 8-rows-per-lane reads are bank-conflict free.
constexpr int TEPI_PITCH = 36;
constexpr int TEPI_WARP_BYTES = 32 * TEPI_PITCH * 4;
constexpr int TEPI_BYTES = 4 * TEPI_WARP_BYTES;

struct HParams {
  __half* C;
  long long ldc, strideC;
  int M, N, K, batches;
  int accumulate;
  int vec_c;  // 1: C allows 16-byte accesses (base, ldc and batch stride multiples of 8 halves)
  int tiles_m, tiles_n, total_tiles;
  // Fused Affine epilogue: out = act(fp16(acc [+ C]) + bias[row]); bias may be null, act NONE.
  const __half* bias;
  int act;
  int vec_bias;  // bias allows 16-byte loads
};

__device__ __forceinline__ void decode_tile(const HParams& p, int t, int& m_idx, int& n_idx,
                                            int& batch) {
  const int per_batch = p.tiles_m * p.tiles_n;
  batch = t / per_batch;
  const int r = t % per_batch;
  const int group_span = TGROUP_M * p.tiles_n;
  const int g = r / group_span;
  const int first_m = g * TGROUP_M;
  const int gm = min(TGROUP_M, p.tiles_m - first_m);
  const int in_g = r % group_span;
  m_idx = first_m + in_g % gm;
  n_idx = in_g / gm;
}

template <int A_MN, int B_MN>
__global__ void __launch_bounds__(192, 1)
hgemm_tma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const HParams p, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[TSTAGES];
  __shared__ __align__(8) uint64_t empty_bar[TSTAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_slot;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int nkb = (p.K + TBK - 1) / TBK;
  constexpr uint32_t IDESC = make_idesc(0, A_MN, B_MN, TBM, TBN);

  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    if (lane == 0) {
      for (int s = 0; s < TSTAGES; ++s) {
        mbar_init(smem_u32(&full_bar[s]), 1);
        mbar_init(smem_u32(&empty_bar[s]), 1);
      }
      for (int a = 0; a < 2; ++a) {
        mbar_init(smem_u32(&acc_full[a]), 1);
        mbar_init(smem_u32(&acc_empty[a]), 4);
      }
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
  // Everything above touched only shared and tensor memory and overlaps the tail of the kernel
  // before this one in the stream when launched as its programmatic dependent; from here on the
  // kernel reads what that kernel may have written.
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
        int m_idx, n_idx, batch;
        decode_tile(p, t, m_idx, n_idx, batch);
        const int m0 = m_idx * TBM, n0 = n_idx * TBN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, status, DEV_TIMEOUT_EMPTY, kb)) {
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(&full_bar[s]);
          const uint32_t a_s = tiles_base + s * TSTAGE_BYTES;
          const uint32_t b_s = a_s + TA_BYTES;
          const int k0 = kb * TBK;
          mbar_arrive_expect_tx(bar, TSTAGE_BYTES);
          if (A_MN) {
            tma_load_3d(a_s, &tmA, bar, m0, k0, batch);
            tma_load_3d(a_s + TMN_ATOM_BYTES, &tmA, bar, m0 + 64, k0, batch);
          } else {
            tma_load_3d(a_s, &tmA, bar, k0, m0, batch);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tma_load_3d(b_s + j * TMN_ATOM_BYTES, &tmB, bar, n0 + 64 * j, k0, batch);
          } else {
            tma_load_3d(b_s, &tmB, bar, k0, n0, batch);
          }
          if (++s == TSTAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1u;
        if (!mbar_wait(smem_u32(&acc_empty[acc]), acc_ph ^ 1u, status, DEV_TIMEOUT_TMEM_FREE, it)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d = tmem + acc * TBN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, status, DEV_TIMEOUT_FULL, kb)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_s = tiles_base + s * TSTAGE_BYTES;
          const uint32_t b_s = a_s + TA_BYTES;
#pragma unroll
          for (int ks = 0; ks < TBK / 16; ++ks) {
            // K-major: 16 elements of K = 32 bytes inside the 128-byte row.
            // MN-major: 16 elements of K = two groups of eight 128-byte rows = 2048 bytes.
            const uint64_t ad = A_MN ? make_smem_desc(a_s + ks * 2048, TMN_ATOM_BYTES, 1024)
                                     : make_smem_desc(a_s + ks * 32, 16, 1024);
            const uint64_t bd = B_MN ? make_smem_desc(b_s + ks * 2048, TMN_ATOM_BYTES, 1024)
                                     : make_smem_desc(b_s + ks * 32, 16, 1024);
            mma_f16(d, ad, bd, IDESC, (kb > 0 || ks > 0) ? 1u : 0u);
          }
          tc_commit(smem_u32(&empty_bar[s]));
          if (++s == TSTAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
        tc_commit(smem_u32(&acc_full[acc]));
      }
    }
    __syncwarp();
  } else {
    // ===================== epilogue =====================
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int it = 0;
    bool ok = true;
    const bool fused = p.bias != nullptr || p.act != ACT_NONE;
    for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++it) {
      int m_idx, n_idx, batch;
      decode_tile(p, t, m_idx, n_idx, batch);
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1u;
      if (!mbar_wait(smem_u32(&acc_full[acc]), acc_ph, status, DEV_TIMEOUT_ACCUM, it)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row0 = m_idx * TBM + q * 32;  // first row of this warp's TMEM lane quarter
      const int n0 = n_idx * TBN;
      __half* cbase = p.C + static_cast<long long>(batch) * p.strideC;
      const uint32_t taddr = tmem + (static_cast<uint32_t>(q * 32) << 16) + acc * TBN;
      float* stage = reinterpret_cast<float*>(smem_raw + (tiles_base - smem_u32(smem_raw)) +
                                              TSTAGES * TSTAGE_BYTES + q * TEPI_WARP_BYTES);
#pragma unroll 1
      for (int c0 = 0; c0 < TBN; c0 += 32) {
        // Each lane owns 4 pieces of the 32x32 chunk: 8 consecutive rows of one column (16 B of C).
        uint4 cold[4];
        if (p.accumulate && p.vec_c) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int piece = lane + 32 * i;
            const int col = n0 + c0 + (piece >> 2), row = row0 + (piece & 3) * 8;
            cold[i] = make_uint4(0, 0, 0, 0);
            if (col < p.N && row + 8 <= p.M)
              cold[i] = *reinterpret_cast<const uint4*>(cbase + static_cast<long long>(col) * p.ldc + row);
          }
        }
        uint32_t v[32];
        tmem_ld32(taddr + c0, v);
        tmem_ld_wait();
        if (c0 + 32 == TBN) {
          // Accumulator drained into registers: hand it back to the MMA warp.
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&acc_empty[acc]));
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) stage[j * TEPI_PITCH + lane] = __uint_as_float(v[j]);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int piece = lane + 32 * i;
          const int cl = piece >> 2, rg = piece & 3;
          const int col = n0 + c0 + cl, row = row0 + rg * 8;
          if (col >= p.N || row >= p.M) continue;
          const float4 x0 = *reinterpret_cast<const float4*>(stage + cl * TEPI_PITCH + rg * 8);
          const float4 x1 = *reinterpret_cast<const float4*>(stage + cl * TEPI_PITCH + rg * 8 + 4);
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
              *reinterpret_cast<uint4*>(cp) = out;
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
            *reinterpret_cast<uint4*>(cp) = out;
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

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------
// Tensor maps
// ------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
  static EncodeFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      sym = nullptr;
    return reinterpret_cast<EncodeFn>(sym);
  }();
  return fn;
}

struct MapKey {
  const void* ptr;
  unsigned long long d0, d1, d2, s1, s2;
  unsigned b0, b1;
  int dev;
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    const unsigned long long* w = reinterpret_cast<const unsigned long long*>(&k);
    size_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(MapKey) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
    return h;
  }
};

}  // namespace

// 3-D tiled map: dim0 = contiguous extent, dim1 = number of stored columns, dim2 = batches.
// esize 2 = fp16, 4 = fp32.  Boxes are b0 x b1 x 1; swizzle128 selects the 128-byte swizzle
// (otherwise none).  Maps are cached per (device, pointer, geometry).
bool encode_tmap(CUtensorMap* out, int esize, const void* ptr, unsigned long long d0,
                 unsigned long long d1, unsigned long long d2, unsigned long long ld,
                 unsigned long long batch_stride, unsigned b0, unsigned b1, bool swizzle128) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  key.ptr = ptr;
  key.d0 = d0; key.d1 = d1; key.d2 = d2;
  key.s1 = ld * esize; key.s2 = batch_stride * esize;
  key.b0 = b0; key.b1 = b1 | (swizzle128 ? 0x10000u : 0u) | (static_cast<unsigned>(esize) << 20);
  cudaGetDevice(&key.dev);
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  EncodeFn enc = get_encode();
  if (!enc) return false;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {key.s1, key.s2};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                   3, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return true;
}

bool tmap_encoder_available() { return get_encode() != nullptr; }

namespace {

bool encode_map(CUtensorMap* out, const void* ptr, unsigned long long d0, unsigned long long d1,
                unsigned long long d2, unsigned long long ld, unsigned long long batch_stride,
                unsigned b0, unsigned b1) {
  return encode_tmap(out, 2, ptr, d0, d1, d2, ld, batch_stride, b0, b1, true);
}

template <int A_MN, int B_MN>
cudaError_t launch_variant(const CUtensorMap& ta, const CUtensorMap& tb, const HParams& p, int grid,
                           cudaStream_t stream, int* status) {
  auto kern = hgemm_tma_kernel<A_MN, B_MN>;
  const int smem = TSTAGES * TSTAGE_BYTES + TEPI_BYTES + 1024;
  static unsigned long long smem_set = 0;  // per template instantiation: per kernel
  cudaError_t e = set_smem_limit_once(reinterpret_cast<const void*>(kern), smem, &smem_set);
  if (e != cudaSuccess) return e;
  return launch_kernel(kern, dim3(grid), dim3(192), smem, stream, pdl_enabled(), ta, tb, p, status);
}

}  // namespace

bool hgemm_tma_supported(const HgemmArgs& a) {
  if (a.transA && a.transB) return false;
  if (a.M < 1 || a.N < 1 || a.K < 1 || a.batches < 1) return false;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!al16(a.A) || !al16(a.B)) return false;
  if (a.lda % 8 || a.ldb % 8) return false;
  if (a.batches > 1 && (a.strideA % 8 || a.strideB % 8)) return false;
  return get_encode() != nullptr;
}

cudaError_t launch_hgemm_tma(const HgemmArgs& a, int num_sms, cudaStream_t stream, int* status) {
  // Stored extents: A is (transA ? K x M : M x K), B is (transB ? N x K : K x N).
  const unsigned long long a_rows = a.transA ? a.K : a.M, a_cols = a.transA ? a.M : a.K;
  const unsigned long long b_rows = a.transB ? a.N : a.K, b_cols = a.transB ? a.K : a.N;
  const unsigned long long sa = a.batches > 1 ? a.strideA : a.lda * a_cols;
  const unsigned long long sb = a.batches > 1 ? a.strideB : a.ldb * b_cols;
  CUtensorMap ta, tb;
  // A: MN-major boxes are 64(m) x 64(k); K-major box is 64(k) x 128(m).
  if (!encode_map(&ta, a.A, a_rows, a_cols, a.batches, a.lda, sa, 64, a.transA ? TBM : TBK))
    return cudaErrorInvalidValue;
  // B: K-major box is 64(k) x 256(n); MN-major boxes are 64(n) x 64(k).
  if (!encode_map(&tb, a.B, b_rows, b_cols, a.batches, a.ldb, sb, 64, a.transB ? TBK : TBN))
    return cudaErrorInvalidValue;
  HParams p;
  p.C = static_cast<__half*>(a.C);
  p.ldc = a.ldc;
  p.strideC = a.strideC;
  p.M = a.M; p.N = a.N; p.K = a.K; p.batches = a.batches;
  p.accumulate = a.accumulate;
  p.vec_c = ((reinterpret_cast<uintptr_t>(a.C) & 15u) == 0 && a.ldc % 8 == 0 &&
             (a.batches == 1 || a.strideC % 8 == 0)) ? 1 : 0;
  p.tiles_m = (a.M + TBM - 1) / TBM;
  p.tiles_n = (a.N + TBN - 1) / TBN;
  const long long total = static_cast<long long>(p.tiles_m) * p.tiles_n * a.batches;
  if (total > 0x7fffffffLL) return cudaErrorInvalidValue;
  p.total_tiles = static_cast<int>(total);
  if ((a.bias != nullptr || a.act != ACT_NONE) && a.batches != 1) return cudaErrorInvalidValue;
  p.bias = static_cast<const __half*>(a.bias);
  p.act = a.act;
  p.vec_bias = (reinterpret_cast<uintptr_t>(a.bias) & 15u) == 0 ? 1 : 0;
  const int grid = static_cast<int>(total < num_sms ? total : num_sms);
  if (!a.transA && !a.transB) return launch_variant<1, 0>(ta, tb, p, grid, stream, status);
  if (a.transA && !a.transB) return launch_variant<0, 0>(ta, tb, p, grid, stream, status);
  return launch_variant<1, 1>(ta, tb, p, grid, stream, status);
}

}  // namespace gb
