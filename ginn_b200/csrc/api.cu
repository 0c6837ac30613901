// extern "C" layer: argument validation, path selection, per-device state.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/ginn_b200.h"
#include "launch.h"
#include "ptx.cuh"

namespace {

using gb::Operand;
using gb::Problem;

thread_local std::string t_error;
std::atomic<long long> g_launches{0};
// Options set through ginn_b200_set_option belong to the calling host thread (ginn's model is
// one thread per GPU, or several threads that share one): a margin set by the thread that
// overlaps a collective with a product does not slow the products of another thread.
thread_local int t_force_path = 0;
thread_local int t_sm_margin = 0;     // SMs the persistent kernels leave free (e.g. for NCCL)
thread_local int t_pair_group_m = 0;  // rasterisation group of the CTA-pair kernel (0 = default)
thread_local int t_fork_streams = 1;  // backward entries: independent products side by side
thread_local int t_presplit = 1;  // large fp32 products: operands split once in a scratch allocation
thread_local int t_pair_l2_hint = 3;  // L2 eviction hints of the CTA-pair kernel (bits, see PParams)
thread_local int t_max_split = 0;     // cap on the K split of fp32 products (0 = none, 1 = no split)
thread_local int t_pdl = 1;           // programmatic dependent launch for the kernels that support it

}  // namespace
bool gb::pdl_enabled() { return t_pdl != 0; }
bool gb::presplit_enabled() { return t_presplit != 0; }
int gb::max_split() { return t_max_split; }
int gb::sm_margin() { return t_sm_margin; }
thread_local int t_walk_kblocks = 16;  // fp32: CTAs walk the tiles of products with at most this many k-blocks per tile
int gb::walk_kblocks() { return t_walk_kblocks; }
namespace {

int fail(int status, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  t_error = buf;
  return status;
}

#define CU_TRY(expr)                                                                      \
  do {                                                                                    \
    cudaError_t e_ = (expr);                                                              \
    if (e_ != cudaSuccess)                                                                \
      return fail(GINN_B200_CUDA_ERROR, "%s failed: %s (%s:%d)", #expr,                   \
                  cudaGetErrorString(e_), __FILE__, __LINE__);                            \
  } while (0)

constexpr int kMaxDevices = 64;
constexpr size_t kStageBytes = 8u << 20;
constexpr unsigned kCounters = 64;  // tile queues (two ints each) handed out round robin

struct DevCtx {
  std::mutex mu;
  bool ready = false;
  int num_sms = 0;
  int* d_status = nullptr;
  int* d_counters = nullptr;     // tile queues of the CTA-pair kernel: zero between launches
  unsigned next_counter = 0;
  // Staging ring for grouped launches (problem descriptors + pointer tables), used in two
  // halves.  A half is reused only after the launches that read it have finished: every stream
  // that used a half leaves an event behind, and the host waits for those before it writes
  // into that half again.
  unsigned char* h_stage = nullptr;
  unsigned char* d_stage = nullptr;
  size_t stage_off = 0;
  struct StageUser {
    cudaStream_t stream;
    cudaEvent_t done;
  };
  std::vector<StageUser> stage_users[2];
  // Prepared levels (ginn_b200_level_create) take their device images from slabs instead of one
  // cudaMalloc each, and upload them asynchronously on a stream of the library's own: a graph
  // with hundreds of levels is prepared in the time of a few allocations.
  struct Slab {
    unsigned char* base = nullptr;
    size_t cap = 0, off = 0;
    int refs = 0;
  };
  Slab* slab = nullptr;           // the slab new levels are carved from
  cudaStream_t prep_stream = nullptr;
  // Second stream for entry points that run independent products side by side (the Affine and
  // attention backward passes): forked from and joined back into the caller's stream with these
  // events.
  // `fork_mu` keeps one call's record/wait pairs together.
  std::mutex fork_mu;
  cudaStream_t side_stream = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_mid = nullptr, ev_join = nullptr;
};
DevCtx g_ctx[kMaxDevices];

int get_ctx(int device, DevCtx** out) {
  if (device < 0 || device >= kMaxDevices)
    return fail(GINN_B200_BAD_ARGUMENT, "device index %d out of range", device);
  CU_TRY(cudaSetDevice(device));
  DevCtx& c = g_ctx[device];
  std::lock_guard<std::mutex> g(c.mu);
  if (!c.ready) {
    int major = 0;
    CU_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    if (major != 10)
      return fail(GINN_B200_UNSUPPORTED,
                  "device %d has compute capability %d.x; this library is built for sm_100a only",
                  device, major);
    CU_TRY(cudaDeviceGetAttribute(&c.num_sms, cudaDevAttrMultiProcessorCount, device));
    CU_TRY(cudaMalloc(&c.d_status, sizeof(int)));
    CU_TRY(cudaMemset(c.d_status, 0, sizeof(int)));
    CU_TRY(cudaMalloc(&c.d_counters, 2 * kCounters * sizeof(int)));
    CU_TRY(cudaMemset(c.d_counters, 0, 2 * kCounters * sizeof(int)));
    {
      // Scratch of the entry points that need one comes from the device's stream-ordered pool;
      // without a release threshold the pool hands its memory back to the driver at every
      // synchronisation and the next call pays for a fresh allocation (tens of microseconds).
      cudaMemPool_t pool = nullptr;
      if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess && pool != nullptr) {
        unsigned long long keep = 1ull << 32;  // keep up to 4 GiB cached
        cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
      }
    }
    CU_TRY(cudaStreamCreateWithFlags(&c.side_stream, cudaStreamNonBlocking));
    CU_TRY(cudaEventCreateWithFlags(&c.ev_fork, cudaEventDisableTiming));
    CU_TRY(cudaEventCreateWithFlags(&c.ev_mid, cudaEventDisableTiming));
    CU_TRY(cudaEventCreateWithFlags(&c.ev_join, cudaEventDisableTiming));
    c.ready = true;
  }
  *out = &c;
  return GINN_B200_OK;
}

int esize(int dtype) { return dtype == GINN_B200_F32 ? 4 : 2; }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

Operand make_operand(int dtype, const void* base, long long ld, long long batch_stride,
                     int batches, int k_contig, const void* ybase = nullptr,
                     int dact = gb::ACT_NONE) {
  Operand o;
  std::memset(&o, 0, sizeof(o));
  o.base = base;
  o.ybase = dact != gb::ACT_NONE ? ybase : nullptr;
  o.ld = ld;
  o.batch_stride = batch_stride;
  o.k_contig = k_contig;
  o.dact = o.ybase ? dact : gb::ACT_NONE;
  const long long es = esize(dtype);
  bool v = k_contig && aligned16(base) && (ld * es) % 16 == 0;
  if (batches > 1) v = v && (batch_stride * es) % 16 == 0;
  if (o.ybase) v = v && aligned16(o.ybase);
  o.vec = v ? 1 : 0;
  return o;
}

// Fork of the caller's stream onto the library's second stream for one entry point: products
// that do not depend on each other run side by side, so that the CTAs of one take the SMs the
// other leaves idle in its last wave.  begin() makes the second stream wait for everything
// queued on the caller's stream so far; join() (also run by the destructor, on every path out)
// makes the caller's stream wait for the second one.  Both are legal inside a stream capture.
struct Fork {
  DevCtx* ctx = nullptr;
  cudaStream_t main = nullptr, side = nullptr;
  std::unique_lock<std::mutex> lock;
  bool active = false;
  cudaError_t begin(DevCtx* c, cudaStream_t caller) {
    ctx = c;
    main = caller;
    lock = std::unique_lock<std::mutex>(c->fork_mu);  // keeps this call's record/wait pairs together
    // the stream and the events exist since the device's first call (never created in a capture)
    cudaError_t e = cudaEventRecord(c->ev_fork, main);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(c->side_stream, c->ev_fork, 0);
    if (e != cudaSuccess) return e;
    side = c->side_stream;
    active = true;
    return cudaSuccess;
  }
  // The second stream also waits for what the caller's stream has queued since begin().
  cudaError_t sync_side() {
    cudaError_t e = cudaEventRecord(ctx->ev_mid, main);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(side, ctx->ev_mid, 0);
    return e;
  }
  cudaError_t join() {
    if (!active) return cudaSuccess;
    active = false;
    cudaError_t e = cudaEventRecord(ctx->ev_join, side);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(main, ctx->ev_join, 0);
    lock.unlock();
    return e;
  }
  ~Fork() { join(); }
};

// SMs a persistent kernel may occupy: all of them minus the margin the host asked to keep free.
int persistent_sms(const DevCtx* ctx) {
  const int n = ctx->num_sms - t_sm_margin;
  return n < 2 ? 2 : n;
}

// Value 1 named a kernel that no longer exists.
enum Path { PATH_AUTO = 0, PATH_TMA = 2, PATH_SMALL = 3, PATH_PAIR = 4, PATH_GATHER = 5 };

// Runs one Problem on a tensor-core kernel or the CUDA-core kernel.
int run_problem_once(DevCtx* ctx, int dtype, Problem& p, cudaStream_t stream) {
  if (p.M <= 0 || p.N <= 0 || p.batches <= 0) return GINN_B200_OK;
  long long ktot = 0;
  for (int i = 0; i < p.npairs; ++i) ktot += p.k[i];
  const int force = t_force_path;
  bool small = (static_cast<long long>(p.M) * p.N <= 16) || ktot == 0;
  if (force == PATH_SMALL) small = true;
  if (p.rowsum != nullptr && ktot > 0) small = false;
  if (small) {
    CU_TRY(gb::launch_small(dtype, p, stream));
  } else if (dtype == GINN_B200_F32 &&
             (gb::sgemm3x_supported(p) || gb::sgemm3x_gather_supported(p))) {
    const long long tiles = static_cast<long long>((p.M + 127) / 128) * ((p.N + 127) / 128) * p.batches;
    if (force != PATH_GATHER && gb::sgemm3x_supported(p)) {
      // The TMA-fed launcher can split any single-pair product: it zeroes C for an assignment
      // and applies an activation in a pass of its own.
      p.split_k = gb::sgemm3x_pick_split(p, tiles, ctx->num_sms, true);
      CU_TRY(gb::launch_sgemm3x(p, stream, ctx->d_status));
      if (p.split_k > 1 && p.act != gb::ACT_NONE) g_launches.fetch_add(1);
    } else {
      p.split_k = gb::sgemm3x_pick_split(p, tiles, ctx->num_sms);
      CU_TRY(gb::launch_sgemm3x_gather(p, stream, ctx->d_status));
    }
  } else if (dtype == GINN_B200_F16 && gb::hgemm_gather_supported(p)) {
    CU_TRY(gb::launch_hgemm_gather(p, stream, ctx->d_status));
  } else {
    // Not reachable through the entry points of this file: they build one pair per gradient
    // product and hang the bias gradient on an outer-contiguous operand.
    return fail(GINN_B200_UNSUPPORTED, "no kernel takes this combination of operands");
  }
  g_launches.fetch_add(1);
  return GINN_B200_OK;
}

// Operand restricted to contraction indices [k0, ...): only for operands without column tables.
Operand shift_k(const Operand& o, int dtype, long long k0) {
  Operand r = o;
  const long long step = (o.k_contig ? 1 : o.ld) * k0 * esize(dtype);
  r.base = static_cast<const char*>(o.base) + step;
  if (o.ybase) r.ybase = static_cast<const char*>(o.ybase) + step;
  if (r.vec && !aligned16(r.base)) r.vec = 0;
  return r;
}

// fp32 accuracy guard.  The 3xTF32 kernels keep the 1e-5 bound for contractions of up to
// kMaxChainK per launch (their accumulation chain is cut four ways, but the tensor core still
// truncates on every add).  Longer contractions are issued as several launches that accumulate
// into C, so each partial result is rounded to nearest in memory; bias goes with the first
// launch, the activation with the last.
constexpr long long kMaxChainK = 8192;

// Products with one extent of at most 16 go to the CUDA-core kernels of small.cu (automatic
// path choice only); a bias gradient riding on such a product is issued as its own launch.
// Sets *done when the problem was taken.
int try_skinny(int dtype, Problem& p, cudaStream_t stream, bool* done) {
  *done = false;
  if (p.M <= 0 || p.N <= 0 || p.batches <= 0) return GINN_B200_OK;
  Problem q = p;
  q.rowsum = nullptr;
  const bool rowsum_ok = p.rowsum == nullptr || (p.a[0].cols == nullptr && p.a[0].ycols == nullptr &&
                                                 p.batches == 1 && !p.a[0].k_contig);
  const int kind = rowsum_ok ? gb::skinny_kind(dtype, q) : 0;
  if (kind == 0) return GINN_B200_OK;
  // The weight-gradient mapping (2) of plain operands sums the rows of A on the way; otherwise
  // the bias gradient is a launch of its own.
  const bool fold = kind == 2 && p.rowsum != nullptr && p.npairs == 1 && p.a[0].dact == gb::ACT_NONE &&
                    p.b[0].cols == nullptr && p.b[0].dact == gb::ACT_NONE && p.ccols == nullptr;
  if (fold) {
    q.rowsum = p.rowsum;
  } else if (p.rowsum != nullptr) {
    CU_TRY(gb::launch_rowsum(dtype, p.a[0].base, p.a[0].ybase, p.a[0].dact, p.a[0].ld, p.M, p.k[0],
                             p.rowsum, stream));
    g_launches.fetch_add(1);
  }
  CU_TRY(gb::launch_skinny(dtype, kind, q, stream));
  g_launches.fetch_add(1);
  *done = true;
  return GINN_B200_OK;
}

int run_problem(DevCtx* ctx, int dtype, Problem& p, cudaStream_t stream) {
  if (t_force_path == PATH_AUTO) {
    bool done = false;
    if (int s = try_skinny(dtype, p, stream, &done)) return s;
    if (done) return GINN_B200_OK;
  }
  bool chain = dtype == GINN_B200_F32 && t_force_path != PATH_SMALL;
  long long kmax = 0, ktot = 0;
  for (int i = 0; i < p.npairs; ++i) {
    kmax = p.k[i] > kmax ? p.k[i] : kmax;
    ktot += p.k[i];
    if (p.a[i].cols || p.b[i].cols) chain = false;
  }
  if (!chain || ktot <= kMaxChainK) return run_problem_once(ctx, dtype, p, stream);
  struct Piece { int pair; long long k0, k; };
  std::vector<Piece> pieces;
  for (int i = 0; i < p.npairs; ++i)
    for (long long k0 = 0; k0 < p.k[i]; k0 += kMaxChainK)
      pieces.push_back({i, k0, p.k[i] - k0 < kMaxChainK ? p.k[i] - k0 : kMaxChainK});
  size_t at = 0;
  bool first = true;
  while (at < pieces.size()) {
    Problem q = p;
    q.npairs = 0;
    long long ksum = 0;
    while (at < pieces.size() && q.npairs < gb::kMaxPairs && ksum + pieces[at].k <= kMaxChainK &&
           !(pieces[at].pair == 0 && q.npairs > 0)) {  // pair 0 leads a launch: it carries rowsum
      const Piece& pc = pieces[at];
      q.a[q.npairs] = shift_k(p.a[pc.pair], dtype, pc.k0);
      q.b[q.npairs] = shift_k(p.b[pc.pair], dtype, pc.k0);
      q.k[q.npairs] = pc.k;
      ksum += pc.k;
      ++q.npairs;
      ++at;
    }
    const bool last = at == pieces.size();
    q.rowsum = (pieces[at - q.npairs].pair == 0) ? p.rowsum : nullptr;
    q.bias = first ? p.bias : nullptr;
    q.accumulate = first ? p.accumulate : 1;
    q.act = last ? p.act : gb::ACT_NONE;
    if (int s = run_problem_once(ctx, dtype, q, stream)) return s;
    first = false;
  }
  return GINN_B200_OK;
}

int check_common(int dtype, int64_t m, int64_t n, int64_t k) {
  if (dtype != GINN_B200_F32 && dtype != GINN_B200_F16)
    return fail(GINN_B200_UNSUPPORTED, "dtype %d is not fp32 (0) or fp16 (1)", dtype);
  if (m < 0 || n < 0 || k < 0)
    return fail(GINN_B200_BAD_ARGUMENT, "negative dimension m=%lld n=%lld k=%lld", (long long)m,
                (long long)n, (long long)k);
  if (m > 0x7fffffffLL || n > 0x7fffffffLL || k > 0x7fffffffLL)
    return fail(GINN_B200_BAD_ARGUMENT, "dimension exceeds 2^31-1");
  return GINN_B200_OK;
}

// Half product on the TMA-fed kernels.  Returns -1 when launched, 0 when neither kernel takes
// the problem (the caller goes on to the general path), or an error status.  `h.bias` / `h.act`
// ask for the Affine epilogue on the result; both kernels fuse it.
// Measured on B200 (Half, us): the one-CTA TMA kernel beats the cp.async kernel on every
// aligned shape tried, down to 512 x 128 x 784 (12 against 21), and the CTA-pair kernel until
// the pairs have about two waves of 256 x 256 tiles (1024 x 4096 x 1024: 16.5 against 19.9;
// 2048^3: 21 against 25; 8192^3: 786 against 732).  Shapes with a tiny extent go on to the
// CUDA-core kernels.
static int half_tma_dispatch(DevCtx* ctx, const gb::HgemmArgs& h, cudaStream_t stream, int force) {
  const long long m = h.M, n = h.N, k = h.K, batches = h.batches;
  const bool big = m > 16 && n > 16 && k > 32;
  const bool big_pair = m >= 256 && n >= 256 && k >= 128 &&
                        ((m + 255) / 256) * ((n + 255) / 256) * batches >= ctx->num_sms;
  if ((force == PATH_PAIR || (force == PATH_AUTO && big_pair)) && gb::hgemm_pair_supported(h)) {
    int* counter;
    {
      std::lock_guard<std::mutex> g(ctx->mu);
      counter = ctx->d_counters + 2 * (ctx->next_counter++ % kCounters);
    }
    CU_TRY(gb::launch_hgemm_pair(h, persistent_sms(ctx), t_pair_group_m, t_pair_l2_hint, counter,
                                 stream, ctx->d_status));
    g_launches.fetch_add(1);
    return -1;
  }
  if ((big || force == PATH_TMA) && gb::hgemm_tma_supported(h)) {
    CU_TRY(gb::launch_hgemm_tma(h, persistent_sms(ctx), stream, ctx->d_status));
    g_launches.fetch_add(1);
    return -1;
  }
  return 0;
}

int gemm_impl(int device, void* stream_, int dtype, int trans_a, int trans_b, int64_t m, int64_t n,
              int64_t k, const void* a, int64_t lda, int64_t stride_a, const void* b, int64_t ldb,
              int64_t stride_b, void* c, int64_t ldc, int64_t stride_c, int64_t batches,
              int accumulate) {
  if (int s = check_common(dtype, m, n, k)) return s;
  if (batches < 0 || batches > 0x7fffffffLL)
    return fail(GINN_B200_BAD_ARGUMENT, "bad batch count %lld", (long long)batches);
  if (m == 0 || n == 0 || batches == 0) return GINN_B200_OK;
  const int64_t a_rows = trans_a ? k : m, b_rows = trans_b ? n : k;
  if (c == nullptr || (k > 0 && (a == nullptr || b == nullptr)))
    return fail(GINN_B200_BAD_ARGUMENT, "null matrix pointer");
  if (lda < (a_rows > 1 ? a_rows : 1) || ldb < (b_rows > 1 ? b_rows : 1) || ldc < m)
    return fail(GINN_B200_BAD_ARGUMENT,
                "leading dimension too small: lda=%lld (rows %lld) ldb=%lld (rows %lld) ldc=%lld "
                "(rows %lld)",
                (long long)lda, (long long)a_rows, (long long)ldb, (long long)b_rows,
                (long long)ldc, (long long)m);
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int force = t_force_path;

  if (dtype == GINN_B200_F16 && k > 0 &&
      (force == PATH_AUTO || force == PATH_TMA || force == PATH_PAIR)) {
    gb::HgemmArgs h;
    h.A = a; h.B = b; h.C = c;
    h.lda = lda; h.ldb = ldb; h.ldc = ldc;
    h.strideA = stride_a; h.strideB = stride_b; h.strideC = stride_c;
    h.transA = trans_a ? 1 : 0; h.transB = trans_b ? 1 : 0;
    h.M = (int)m; h.N = (int)n; h.K = (int)k; h.batches = (int)batches;
    h.accumulate = accumulate ? 1 : 0;
    const int r = half_tma_dispatch(ctx, h, stream, force);
    if (r != 0) return r < 0 ? GINN_B200_OK : r;
  }

  Problem p;
  std::memset(&p, 0, sizeof(p));
  p.npairs = 1;
  p.a[0] = make_operand(dtype, a, lda, stride_a, (int)batches, trans_a ? 1 : 0);
  p.b[0] = make_operand(dtype, b, ldb, stride_b, (int)batches, trans_b ? 0 : 1);
  p.k[0] = k;
  p.M = (int)m; p.N = (int)n; p.batches = (int)batches;
  p.c = c; p.ldc = ldc; p.c_batch_stride = stride_c;
  p.act = gb::ACT_NONE;
  p.accumulate = accumulate ? 1 : 0;
  return run_problem(ctx, dtype, p, stream);
}

// Reserves `bytes` in the staging ring for a launch on `stream`; returns host and device
// addresses of the slot.  Call stage_mark after the launch has been queued.
int stage_alloc(DevCtx* ctx, size_t bytes, cudaStream_t stream, unsigned char** h,
                unsigned char** d, int* half_out) {
  bytes = (bytes + 255) & ~size_t(255);
  constexpr size_t kHalf = kStageBytes / 2;
  if (bytes > kHalf)
    return fail(GINN_B200_BAD_ARGUMENT, "grouped launch needs %zu staging bytes (limit %zu)",
                bytes, kHalf);
  std::lock_guard<std::mutex> g(ctx->mu);
  if (!ctx->h_stage) {
    CU_TRY(cudaMallocHost(&ctx->h_stage, kStageBytes));
    CU_TRY(cudaMalloc(&ctx->d_stage, kStageBytes));
  }
  int half = ctx->stage_off < kHalf ? 0 : 1;
  if (ctx->stage_off + bytes > static_cast<size_t>(half + 1) * kHalf) {
    // Moving on to the other half: the launches that read it last time round must be done.
    // The host waits for their events only -- other work on the device is left alone.
    half ^= 1;
    for (const DevCtx::StageUser& u : ctx->stage_users[half]) CU_TRY(cudaEventSynchronize(u.done));
    ctx->stage_off = half * kHalf;
  }
  *h = ctx->h_stage + ctx->stage_off;
  *d = ctx->d_stage + ctx->stage_off;
  *half_out = half;
  ctx->stage_off += bytes;
  (void)stream;
  return GINN_B200_OK;
}

// Leaves (or moves) the event that tells when `stream` is done with `half` of the ring.
int stage_mark(DevCtx* ctx, int half, cudaStream_t stream) {
  std::lock_guard<std::mutex> g(ctx->mu);
  for (DevCtx::StageUser& u : ctx->stage_users[half])
    if (u.stream == stream) {
      CU_TRY(cudaEventRecord(u.done, stream));
      return GINN_B200_OK;
    }
  cudaEvent_t ev;
  CU_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  CU_TRY(cudaEventRecord(ev, stream));
  ctx->stage_users[half].push_back({stream, ev});
  return GINN_B200_OK;
}

// Entry points that copy descriptors from a host buffer they reuse cannot be recorded into a
// CUDA graph: a replay would copy whatever the buffer holds by then.
int refuse_capture(cudaStream_t stream, const char* who) {
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  CU_TRY(cudaStreamIsCapturing(stream, &cs));
  if (cs != cudaStreamCaptureStatusNone)
    return fail(GINN_B200_UNSUPPORTED,
                "%s was called on a stream that is being captured; its descriptors are copied "
                "from a host buffer that later calls overwrite.  Prepare the level with "
                "ginn_b200_level_create and capture ginn_b200_level_run instead",
                who);
  return GINN_B200_OK;
}


// ---- grouped levels: validation, image layout, launch (shared by the three entry points) ----
struct LevelPlan {
  size_t desc_bytes = 0;  // descriptors, padded to 16 bytes
  size_t bytes = 0;       // descriptors + both pointer tables of every live group
  int live = 0;           // groups with m, k, ncols > 0
  long long max_n = 0, sum_tiles128 = 0;
};
struct LevelLaunch {
  int nprobs = 0, tiles = 0;
  bool with_y = false;  // some group forms dy (.) act'(out) on the fly
};

int plan_level(int dtype, int mode, int ngroups, const ginn_b200_group* groups, LevelPlan* plan) {
  if (dtype != GINN_B200_F32 && dtype != GINN_B200_F16)
    return fail(GINN_B200_UNSUPPORTED, "dtype %d is not fp32 (0) or fp16 (1)", dtype);
  if (mode < GINN_B200_GROUPED_FORWARD || mode > GINN_B200_GROUPED_DW)
    return fail(GINN_B200_BAD_ARGUMENT, "unknown grouped mode %d", mode);
  if (ngroups < 0 || (ngroups > 0 && groups == nullptr))
    return fail(GINN_B200_BAD_ARGUMENT, "bad group list");
  size_t table_bytes = 0;
  for (int g = 0; g < ngroups; ++g) {
    const ginn_b200_group& q = groups[g];
    if (q.m < 0 || q.k < 0 || q.ncols < 0 || q.m > 0x7fffffffLL || q.k > 0x7fffffffLL ||
        q.ncols > 0x7fffffffLL)
      return fail(GINN_B200_BAD_ARGUMENT, "group %d: bad dimensions", g);
    if (q.m == 0 || q.k == 0 || q.ncols == 0) continue;
    if (!q.w || q.ldw < q.m || !q.y_cols)
      return fail(GINN_B200_BAD_ARGUMENT, "group %d: bad W or column table", g);
    if ((mode != GINN_B200_GROUPED_DX && !q.x_cols) || (mode == GINN_B200_GROUPED_DX && !q.dx_cols))
      return fail(GINN_B200_BAD_ARGUMENT, "group %d: missing column table for mode %d", g, mode);
    if (mode == GINN_B200_GROUPED_DW && (!q.dw || q.lddw < q.m))
      return fail(GINN_B200_BAD_ARGUMENT, "group %d: bad dW", g);
    if (q.act < GINN_B200_ACT_NONE || q.act > GINN_B200_ACT_RELU)
      return fail(GINN_B200_UNSUPPORTED, "group %d: activation %d cannot be fused", g, q.act);
    const bool deriv = mode != GINN_B200_GROUPED_FORWARD && q.act != GINN_B200_ACT_NONE;
    if (deriv && !q.out_cols)
      return fail(GINN_B200_BAD_ARGUMENT,
                  "group %d: the nodes' values (out_cols) are needed for the derivative", g);
    table_bytes += (deriv ? 3 : 2) * static_cast<size_t>(q.ncols) * sizeof(void*);
    const long long N = mode == GINN_B200_GROUPED_DW ? q.k : q.ncols;
    const long long M = mode == GINN_B200_GROUPED_DX ? q.k : q.m;
    plan->max_n = N > plan->max_n ? N : plan->max_n;
    plan->sum_tiles128 += ((M + 127) / 128) * ((N + 127) / 128);
    ++plan->live;
  }
  plan->desc_bytes = (static_cast<size_t>(plan->live) * sizeof(Problem) + 15) & ~size_t(15);
  plan->bytes = plan->desc_bytes + table_bytes;
  return GINN_B200_OK;
}

// Writes descriptors and pointer tables into the host image `h`; `d` is the device address the
// image will have, so that the descriptors can point at their tables.
LevelLaunch fill_level_image(int dtype, int mode, int ngroups, const ginn_b200_group* groups,
                             const LevelPlan& plan, int num_sms, unsigned char* h,
                             unsigned char* d) {
  LevelLaunch ll;
  // Levels run on the gather kernels (128 x 128 tiles): the cp.async front end of the 3xTF32
  // kernel for fp32, the cp.async fp16 kernel for Half.
  Problem* hp = reinterpret_cast<Problem*>(h);
  size_t off = plan.desc_bytes;
  for (int g = 0; g < ngroups; ++g) {
    const ginn_b200_group& q = groups[g];
    if (q.m == 0 || q.k == 0 || q.ncols == 0) continue;
    const size_t tb = static_cast<size_t>(q.ncols) * sizeof(void*);
    const void** t0 = reinterpret_cast<const void**>(h + off);
    const void* const* d_t0 = reinterpret_cast<const void* const*>(d + off);
    off += tb;
    const void** t1 = reinterpret_cast<const void**>(h + off);
    void* const* d_t1 = reinterpret_cast<void* const*>(d + off);
    off += tb;
    const bool deriv = mode != GINN_B200_GROUPED_FORWARD && q.act != GINN_B200_ACT_NONE;
    const void* const* d_t2 = nullptr;
    if (deriv) {
      const void** t2 = reinterpret_cast<const void**>(h + off);
      d_t2 = reinterpret_cast<const void* const*>(d + off);
      off += tb;
      for (int64_t j = 0; j < q.ncols; ++j) t2[j] = q.out_cols[j];
      ll.with_y = true;
    }
    Problem& p = hp[ll.nprobs];
    std::memset(&p, 0, sizeof(p));
    p.npairs = 1;
    p.batches = 1;
    bool al = true;
    if (mode == GINN_B200_GROUPED_FORWARD) {
      for (int64_t j = 0; j < q.ncols; ++j) {
        t0[j] = q.x_cols[j];
        t1[j] = q.y_cols[j];
        al = al && aligned16(q.x_cols[j]);
      }
      p.a[0] = make_operand(dtype, q.w, q.ldw, 0, 1, 0);
      p.b[0] = make_operand(dtype, nullptr, 0, 0, 1, 1);
      p.b[0].cols = d_t0;
      p.b[0].vec = al ? 1 : 0;
      p.k[0] = q.k;
      p.M = (int)q.m; p.N = (int)q.ncols;
      p.ccols = d_t1;
      p.bias = q.bias;
      p.act = q.act;
      p.accumulate = q.accumulate ? 1 : 0;
    } else if (mode == GINN_B200_GROUPED_DX) {
      for (int64_t j = 0; j < q.ncols; ++j) {
        t0[j] = q.y_cols[j];
        t1[j] = q.dx_cols[j];
        al = al && aligned16(q.y_cols[j]) && (!deriv || aligned16(q.out_cols[j]));
      }
      p.a[0] = make_operand(dtype, q.w, q.ldw, 0, 1, 1);  // W^T: contraction over m
      p.b[0] = make_operand(dtype, nullptr, 0, 0, 1, 1);
      p.b[0].cols = d_t0;
      p.b[0].vec = al ? 1 : 0;
      if (deriv) {
        p.b[0].ycols = d_t2;
        p.b[0].dact = q.act;
      }
      p.k[0] = q.m;
      p.M = (int)q.k; p.N = (int)q.ncols;
      p.ccols = d_t1;
      p.accumulate = 1;
    } else {
      for (int64_t j = 0; j < q.ncols; ++j) {
        t0[j] = q.y_cols[j];
        t1[j] = q.x_cols[j];
      }
      p.a[0] = make_operand(dtype, nullptr, 0, 0, 1, 0);  // dy columns, contraction over j
      p.a[0].cols = d_t0;
      if (deriv) {
        p.a[0].ycols = d_t2;
        p.a[0].dact = q.act;
      }
      p.b[0] = make_operand(dtype, nullptr, 0, 0, 1, 0);  // x columns
      p.b[0].cols = reinterpret_cast<const void* const*>(d_t1);
      p.k[0] = q.ncols;
      p.M = (int)q.m; p.N = (int)q.k;
      p.c = q.dw; p.ldc = q.lddw;
      p.rowsum = q.dbias;
      p.accumulate = 1;
    }
    p.tiles_m = (p.M + 127) / 128;
    p.tiles_n = (p.N + 127) / 128;
    p.tile_start = ll.tiles;
    if (dtype == GINN_B200_F32)
      p.split_k = gb::sgemm3x_pick_split(p, plan.sum_tiles128, num_sms);
    ll.tiles += p.tiles_m * p.tiles_n * (p.split_k > 1 ? p.split_k : 1);
    ++ll.nprobs;
  }
  return ll;
}

// Stride (in elements) of a column table whose entries are equally spaced, i.e. the columns of
// one strided matrix; -1 otherwise.  A single column fits any stride.
long long table_stride(const void* const* t, int64_t n, int es, int64_t rows) {
  if (n <= 1) return rows;
  const char* p0 = static_cast<const char*>(t[0]);
  const long long step = static_cast<const char*>(t[1]) - p0;
  if (step < rows * es || step % es != 0) return -1;
  for (int64_t j = 2; j < n; ++j)
    if (static_cast<const char*>(t[j]) - p0 != step * j) return -1;
  return step / es;
}

// A level whose column tables all describe plain strided matrices -- the nodes' tensors happen
// to be the columns of one allocation, as with a bump allocator or a batched input -- needs no
// tables at all: each group is an ordinary product, and an fp32 one whose operands a tensor map
// can describe runs on the TMA-fed kernel (about twice the throughput of the cp.async front
// end).  Returns true and the per-group problems when the whole level qualifies.
bool direct_level(int dtype, int mode, int ngroups, const ginn_b200_group* groups, int num_sms,
                  std::vector<Problem>* out) {
  if (dtype != GINN_B200_F32 || t_force_path != PATH_AUTO) return false;
  out->clear();
  for (int g = 0; g < ngroups; ++g) {
    const ginn_b200_group& q = groups[g];
    if (q.m == 0 || q.k == 0 || q.ncols == 0) continue;
    if (out->size() == 4) return false;  // many groups: one grouped launch serves them better
    Problem p;
    std::memset(&p, 0, sizeof(p));
    p.npairs = 1;
    p.batches = 1;
    if (mode == GINN_B200_GROUPED_FORWARD || mode == GINN_B200_GROUPED_DX) {
      const bool fwd = mode == GINN_B200_GROUPED_FORWARD;
      const void* const* in = fwd ? q.x_cols : reinterpret_cast<const void* const*>(q.y_cols);
      void* const* outc = fwd ? q.y_cols : q.dx_cols;
      const int64_t in_rows = fwd ? q.k : q.m, out_rows = fwd ? q.m : q.k;
      const long long ldi = table_stride(in, q.ncols, 4, in_rows);
      const long long ldo = table_stride(reinterpret_cast<const void* const*>(outc), q.ncols, 4, out_rows);
      if (ldi < 0 || ldo < 0) return false;
      p.a[0] = make_operand(dtype, q.w, q.ldw, 0, 1, fwd ? 0 : 1);
      p.b[0] = make_operand(dtype, in[0], ldi, 0, 1, 1);
      p.k[0] = in_rows;
      p.M = (int)out_rows; p.N = (int)q.ncols;
      p.c = outc[0]; p.ldc = ldo;
      p.bias = fwd ? q.bias : nullptr;
      p.accumulate = fwd ? (q.accumulate ? 1 : 0) : 1;
      if (fwd) {
        p.act = q.act;
      } else if (q.act != GINN_B200_ACT_NONE) {  // dy (.) act'(out): out must share dy's stride
        if (!q.out_cols || table_stride(q.out_cols, q.ncols, 4, q.m) != ldi) return false;
        p.b[0] = make_operand(dtype, in[0], ldi, 0, 1, 1, q.out_cols[0], q.act);
      }
    } else {
      const long long ldy = table_stride(reinterpret_cast<const void* const*>(q.y_cols), q.ncols, 4, q.m);
      const long long ldx = table_stride(q.x_cols, q.ncols, 4, q.k);
      if (ldy < 0 || ldx < 0) return false;
      p.a[0] = make_operand(dtype, q.y_cols[0], ldy, 0, 1, 0);
      if (q.act != GINN_B200_ACT_NONE) {
        if (!q.out_cols || table_stride(q.out_cols, q.ncols, 4, q.m) != ldy) return false;
        p.a[0] = make_operand(dtype, q.y_cols[0], ldy, 0, 1, 0, q.out_cols[0], q.act);
      }
      p.b[0] = make_operand(dtype, q.x_cols[0], ldx, 0, 1, 0);
      p.k[0] = q.ncols;
      p.M = (int)q.m; p.N = (int)q.k;
      p.c = q.dw; p.ldc = q.lddw;
      p.rowsum = q.dbias;
      p.accumulate = 1;
    }
    if (p.k[0] > kMaxChainK || !gb::sgemm3x_supported(p)) return false;
    const long long tiles = static_cast<long long>((p.M + 127) / 128) * ((p.N + 127) / 128);
    p.split_k = gb::sgemm3x_pick_split(p, tiles, num_sms);
    out->push_back(p);
  }
  return !out->empty();
}

int launch_direct_level(const std::vector<Problem>& probs, cudaStream_t stream, int* status) {
  for (const Problem& p : probs) {
    CU_TRY(gb::launch_sgemm3x(p, stream, status));
    g_launches.fetch_add(1);
  }
  return GINN_B200_OK;
}

cudaError_t launch_level(int dtype, const LevelLaunch& ll, const Problem* dprobs,
                         cudaStream_t stream, int* status) {
  if (dtype == GINN_B200_F32)
    return gb::launch_sgemm3x_gather_grouped(dprobs, ll.nprobs, ll.tiles, ll.with_y, stream, status);
  return gb::launch_hgemm_gather_grouped(dprobs, ll.nprobs, ll.tiles, stream, status);
}

}  // namespace

extern "C" {

int ginn_b200_gemm(int device, void* stream, int dtype, int trans_a, int trans_b, int64_t m,
                   int64_t n, int64_t k, const void* a, int64_t lda, const void* b, int64_t ldb,
                   void* c, int64_t ldc, int accumulate) {
  return gemm_impl(device, stream, dtype, trans_a, trans_b, m, n, k, a, lda, 0, b, ldb, 0, c, ldc,
                   0, 1, accumulate);
}

int ginn_b200_gemm_batched(int device, void* stream, int dtype, int trans_a, int trans_b,
                           int64_t m, int64_t n, int64_t k, const void* a, int64_t lda,
                           int64_t stride_a, const void* b, int64_t ldb, int64_t stride_b, void* c,
                           int64_t ldc, int64_t stride_c, int64_t batches, int accumulate) {
  return gemm_impl(device, stream, dtype, trans_a, trans_b, m, n, k, a, lda, stride_a, b, ldb,
                   stride_b, c, ldc, stride_c, batches, accumulate);
}

int ginn_b200_affine_forward(int device, void* stream_, int dtype, int npairs,
                             const ginn_b200_pair* pairs, int64_t m, int64_t n, const void* bias,
                             int act, void* out, int64_t ldo) {
  if (int s = check_common(dtype, m, n, 0)) return s;
  if (npairs < 1 || npairs > gb::kMaxPairs || pairs == nullptr)
    return fail(GINN_B200_BAD_ARGUMENT, "npairs=%d must be in 1..%d", npairs, gb::kMaxPairs);
  if (act < GINN_B200_ACT_NONE || act > GINN_B200_ACT_RELU)
    return fail(GINN_B200_UNSUPPORTED, "activation %d cannot be fused", act);
  if (m == 0 || n == 0) return GINN_B200_OK;
  if (out == nullptr || ldo < m) return fail(GINN_B200_BAD_ARGUMENT, "bad output (ldo=%lld)", (long long)ldo);
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  Problem p;
  std::memset(&p, 0, sizeof(p));
  int np = 0;
  for (int i = 0; i < npairs; ++i) {
    const ginn_b200_pair& q = pairs[i];
    if (q.k < 0 || q.k > 0x7fffffffLL) return fail(GINN_B200_BAD_ARGUMENT, "pair %d: bad k", i);
    if (q.k == 0) continue;
    if (!q.a || !q.b || q.lda < m || q.ldb < q.k)
      return fail(GINN_B200_BAD_ARGUMENT, "pair %d: null pointer or leading dimension too small", i);
    p.a[np] = make_operand(dtype, q.a, q.lda, 0, 1, 0);
    p.b[np] = make_operand(dtype, q.b, q.ldb, 0, 1, 1);
    p.k[np] = q.k;
    ++np;
  }
  p.npairs = np;
  p.M = (int)m; p.N = (int)n; p.batches = 1;
  p.c = out; p.ldc = ldo;
  p.bias = bias;
  p.act = act;
  p.accumulate = 0;
  // Half with every pair on the TMA kernels: one product per pair (the first assigns, the others
  // accumulate) and the bias and activation in the epilogue of the last one.
  // 16 us for a 1024 x 1024 layer on 4096 columns against 29 us for the fused cp.async kernel.
  // The product is rounded to fp16 before the bias and the nonlinearity, as the reference's is.
  if (dtype == GINN_B200_F16 && t_force_path == PATH_AUTO && np > 0 && m > 16 && n > 16 &&
      n <= 65535) {
    gb::HgemmArgs h[gb::kMaxPairs];
    bool tma = true;
    for (int i = 0; i < np && tma; ++i) {
      h[i].A = p.a[i].base; h[i].B = p.b[i].base; h[i].C = out;
      h[i].lda = p.a[i].ld; h[i].ldb = p.b[i].ld; h[i].ldc = ldo;
      h[i].strideA = h[i].strideB = h[i].strideC = 0;
      h[i].transA = h[i].transB = 0;
      h[i].M = (int)m; h[i].N = (int)n; h[i].K = (int)p.k[i]; h[i].batches = 1;
      h[i].accumulate = i > 0;
      tma = p.k[i] > 32 && gb::hgemm_tma_supported(h[i]);
    }
    if (tma) {
      h[np - 1].bias = bias;
      h[np - 1].act = act;
      for (int i = 0; i < np; ++i) {
        const int r = half_tma_dispatch(ctx, h[i], static_cast<cudaStream_t>(stream_), PATH_AUTO);
        if (r > 0) return r;
        if (r == 0) return fail(GINN_B200_CUDA_ERROR, "Half TMA dispatch declined a checked problem");
      }
      return GINN_B200_OK;
    }
  }
  return run_problem(ctx, dtype, p, static_cast<cudaStream_t>(stream_));
}

int ginn_b200_affine_backward(int device, void* stream_, int dtype, int npairs,
                              const ginn_b200_pair_grad* pairs, int64_t m, int64_t n,
                              const void* dout, int64_t lddout, const void* out, int64_t ldout,
                              int act, void* dbias) {
  return ginn_b200_affine_backward_scratch(device, stream_, dtype, npairs, pairs, m, n, dout, lddout,
                                           out, ldout, act, dbias, nullptr);
}

// Byte range of a column-major matrix.
struct ByteRange {
  const char* lo;
  const char* hi;
};
static ByteRange range_of(const void* p, int64_t rows, int64_t cols, int64_t ld, int es) {
  const char* lo = static_cast<const char*>(p);
  if (p == nullptr || rows <= 0 || cols <= 0) return ByteRange{lo, lo};
  return ByteRange{lo, lo + ((cols - 1) * ld + rows) * es};
}
static bool overlap(const ByteRange& a, const ByteRange& b) { return a.lo < b.hi && b.lo < a.hi; }

// True when a backward call has both an input gradient and a weight gradient to form and no
// input gradient shares memory with a weight or bias gradient (the two kinds then run on
// different streams).
static bool wants_both(int dtype, int npairs, const ginn_b200_pair_grad* pairs, int64_t m, int64_t n,
                       const void* dbias) {
  const int es = dtype == GINN_B200_F32 ? 4 : 2;
  int n_dx = 0, n_dw = 0;
  for (int i = 0; i < npairs; ++i) {
    if (pairs[i].k <= 0) continue;
    n_dx += pairs[i].db != nullptr;
    n_dw += pairs[i].da != nullptr;
  }
  if (n_dx == 0 || n_dw == 0) return false;
  const ByteRange bias = range_of(dbias, m, 1, m, es);
  for (int i = 0; i < npairs; ++i) {
    if (pairs[i].k <= 0 || pairs[i].db == nullptr) continue;
    const ByteRange dx = range_of(pairs[i].db, pairs[i].k, n, pairs[i].lddb, es);
    if (overlap(dx, bias)) return false;
    for (int j = 0; j < npairs; ++j) {
      if (pairs[j].k <= 0 || pairs[j].da == nullptr) continue;
      if (overlap(dx, range_of(pairs[j].da, m, pairs[j].k, pairs[j].ldda, es))) return false;
    }
  }
  return true;
}

int ginn_b200_affine_backward_scratch(int device, void* stream_, int dtype, int npairs,
                                      const ginn_b200_pair_grad* pairs, int64_t m, int64_t n,
                                      const void* dout, int64_t lddout, const void* out,
                                      int64_t ldout, int act, void* dbias, void* caller_scratch) {
  if (int s = check_common(dtype, m, n, 0)) return s;
  if (npairs < 0 || (npairs > 0 && pairs == nullptr))
    return fail(GINN_B200_BAD_ARGUMENT, "bad pair list");
  if (act < GINN_B200_ACT_NONE || act > GINN_B200_ACT_RELU)
    return fail(GINN_B200_UNSUPPORTED, "activation %d cannot be fused", act);
  if (m == 0 || n == 0) return GINN_B200_OK;
  if (dout == nullptr || lddout < m) return fail(GINN_B200_BAD_ARGUMENT, "bad upstream gradient");
  if (act != GINN_B200_ACT_NONE && (out == nullptr || ldout != lddout))
    return fail(GINN_B200_BAD_ARGUMENT,
                "the node value is required for the derivative and must share the gradient's "
                "leading dimension (ldout=%lld, lddout=%lld)", (long long)ldout, (long long)lddout);
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  bool dbias_done = dbias == nullptr;

  // Half, large: materialise dA = dout (.) act'(out) once, as the reference does in dpreactiv_
  // (ginn/node/affine.h:82-88), and send both gradient products through the plain product entry,
  // i.e. to the TMA-fed kernels.  Fusing the derivative into the operand loaders recomputes it
  // once per output tile that reads the element and keeps those products on the register path
  // of the general kernel: 82 + 239 us against about 90 us for a 1024 x 1024 layer on 4096
  // columns.  The scratch is a stream-ordered allocation of the library's own.
  if (dtype == GINN_B200_F16 && t_force_path == PATH_AUTO && m * n >= 65536 && n <= 65535) {
    void* scratch = nullptr;  // the library's own allocation, when the caller gave none
    const void* dA = dout;
    int64_t ldA = lddout;
    if (act != GINN_B200_ACT_NONE && caller_scratch != nullptr) {
      if (!aligned16(caller_scratch))
        return fail(GINN_B200_BAD_ARGUMENT, "the scratch tensor must be 16-byte aligned");
      cudaError_t e = gb::launch_dact_half(dout, lddout, out, ldout, act, caller_scratch, (int)m, n, stream);
      if (e != cudaSuccess)
        return fail(GINN_B200_CUDA_ERROR, "derivative kernel: %s", cudaGetErrorString(e));
      g_launches.fetch_add(1);
      dA = caller_scratch;
      ldA = m;
    } else if (act != GINN_B200_ACT_NONE) {
      CU_TRY(cudaMallocAsync(&scratch, static_cast<size_t>(m) * n * 2, stream));
      cudaError_t e = gb::launch_dact_half(dout, lddout, out, ldout, act, scratch, (int)m, n, stream);
      if (e != cudaSuccess) {
        cudaFreeAsync(scratch, stream);
        return fail(GINN_B200_CUDA_ERROR, "derivative kernel: %s", cudaGetErrorString(e));
      }
      g_launches.fetch_add(1);
      dA = scratch;
      ldA = m;
    }
    int status = GINN_B200_OK;
    // The input gradients go to the second stream (after the derivative pass above), the weight
    // and bias gradients stay on the caller's: they only share read-only operands.
    Fork fk;
    cudaStream_t dx_stream = stream;
    if (t_fork_streams && wants_both(dtype, npairs, pairs, m, n, dbias)) {
      cudaError_t e = fk.begin(ctx, stream);
      if (e != cudaSuccess) {
        if (scratch) cudaFreeAsync(scratch, stream);
        return fail(GINN_B200_CUDA_ERROR, "second stream: %s", cudaGetErrorString(e));
      }
      dx_stream = fk.side;
    }
    if (dbias != nullptr) {
      // large aligned matrices: fp32 partial sums in a stream-ordered allocation, then one pass
      // (atomics from many blocks onto the few lines of the bias gradient serialise)
      const int parts = gb::rowsum_ws_parts((int)m, n);
      cudaError_t e = cudaErrorInvalidValue;
      if (parts > 0 && ldA % 8 == 0 && aligned16(dA)) {
        void* rws = nullptr;
        e = cudaMallocAsync(&rws, static_cast<size_t>(parts) * m * 4, stream);
        if (e == cudaSuccess) {
          e = gb::launch_rowsum_half_ws(dA, ldA, (int)m, n, dbias, static_cast<float*>(rws), stream);
          cudaFreeAsync(rws, stream);
          g_launches.fetch_add(1);
        }
      } else {
        e = gb::launch_rowsum(dtype, dA, nullptr, gb::ACT_NONE, ldA, (int)m, n, dbias, stream);
      }
      if (e != cudaSuccess) status = fail(GINN_B200_CUDA_ERROR, "bias gradient: %s", cudaGetErrorString(e));
      g_launches.fetch_add(1);
    }
    for (int i = 0; i < npairs && status == GINN_B200_OK; ++i) {
      const ginn_b200_pair_grad& q = pairs[i];
      if (q.k < 0 || q.k > 0x7fffffffLL) status = fail(GINN_B200_BAD_ARGUMENT, "pair %d: bad k", i);
      if (status != GINN_B200_OK || q.k == 0) continue;
      if (q.db) {  // db (k x n) += A^T (k x m) * dA (m x n)
        if (!q.a || q.lda < m || q.lddb < q.k)
          status = fail(GINN_B200_BAD_ARGUMENT, "pair %d: bad A / db", i);
        else
          status = gemm_impl(device, dx_stream, dtype, 1, 0, q.k, n, m, q.a, q.lda, 0, dA, ldA, 0, q.db,
                             q.lddb, 0, 1, 1);
      }
      if (status == GINN_B200_OK && q.da) {  // da (m x k) += dA (m x n) * B^T (n x k)
        if (!q.b || q.ldb < q.k || q.ldda < m) {
          status = fail(GINN_B200_BAD_ARGUMENT, "pair %d: bad B / da", i);
          continue;
        }
        // A weight gradient has few output tiles and contracts over all n columns (1024 x 1024
        // over 4096 columns: 32 tiles of 128 x 256 on 148 SMs, 36 us).  Split the columns into
        // chunks that run as one strided-batched product into fp16 partial matrices and add
        // those to da in one pass (fp32 sum, one rounding): 4 x 32 CTAs, about 14 us.  The
        // partials live in a stream-ordered allocation.
        const long long tiles = ((m + 127) / 128) * ((q.k + 255) / 256);
        long long parts = 1;
        if (t_max_split != 1 && tiles * 2 <= ctx->num_sms && n >= 1024 && q.k <= 65535) {
          parts = ctx->num_sms / tiles;
          if (parts > 8) parts = 8;
          if (parts > n / 512) parts = n / 512;
          if (t_max_split > 0 && parts > t_max_split) parts = t_max_split;
          while (parts > 1 && (n % parts != 0 || (n / parts) % 8 != 0)) --parts;
        }
        if (parts > 1) {
          void* ws = nullptr;
          const long long chunk = n / parts;
          cudaError_t e = cudaMallocAsync(&ws, static_cast<size_t>(parts) * m * q.k * 2, stream);
          if (e != cudaSuccess) {
            status = fail(GINN_B200_CUDA_ERROR, "partial products: %s", cudaGetErrorString(e));
            continue;
          }
          status = gemm_impl(device, stream_, dtype, 0, 1, m, q.k, chunk, dA, ldA, chunk * ldA, q.b,
                             q.ldb, chunk * q.ldb, ws, m, m * q.k, parts, 0);
          if (status == GINN_B200_OK) {
            e = gb::launch_add_partials_half(q.da, q.ldda, ws, (int)parts, (int)m, q.k, stream);
            if (e != cudaSuccess)
              status = fail(GINN_B200_CUDA_ERROR, "partial sums: %s", cudaGetErrorString(e));
            g_launches.fetch_add(1);
          }
          cudaFreeAsync(ws, stream);
        } else {
          status = gemm_impl(device, stream_, dtype, 0, 1, m, q.k, n, dA, ldA, 0, q.b, q.ldb, 0, q.da,
                             q.ldda, 0, 1, 1);
        }
      }
    }
    const cudaError_t je = fk.join();
    if (je != cudaSuccess && status == GINN_B200_OK)
      status = fail(GINN_B200_CUDA_ERROR, "joining the second stream failed: %s", cudaGetErrorString(je));
    if (scratch) cudaFreeAsync(scratch, stream);
    return status;
  }

  // Input gradients on the second stream, weight and bias gradients on the caller's: they only
  // share read-only operands, and the CTAs of one fill the SMs the other leaves idle.
  Fork fk;
  cudaStream_t dx_stream = stream;
  if (t_fork_streams && wants_both(dtype, npairs, pairs, m, n, dbias)) {
    CU_TRY(fk.begin(ctx, stream));
    dx_stream = fk.side;
  }
  for (int i = 0; i < npairs; ++i) {
    const ginn_b200_pair_grad& q = pairs[i];
    if (q.k < 0 || q.k > 0x7fffffffLL) return fail(GINN_B200_BAD_ARGUMENT, "pair %d: bad k", i);
    if (q.k == 0) continue;
    if (q.db) {  // db (k x n) += A^T (k x m) * dA (m x n)
      if (!q.a || q.lda < m || q.lddb < q.k)
        return fail(GINN_B200_BAD_ARGUMENT, "pair %d: bad A / db", i);
      Problem p;
      std::memset(&p, 0, sizeof(p));
      p.npairs = 1;
      p.a[0] = make_operand(dtype, q.a, q.lda, 0, 1, 1);
      p.b[0] = make_operand(dtype, dout, lddout, 0, 1, 1, out, act);
      p.k[0] = m;
      p.M = (int)q.k; p.N = (int)n; p.batches = 1;
      p.c = q.db; p.ldc = q.lddb;
      p.accumulate = 1;
      if (int s = run_problem(ctx, dtype, p, dx_stream)) return s;
    }
    if (q.da) {  // da (m x k) += dA (m x n) * B^T (n x k)
      if (!q.b || q.ldb < q.k || q.ldda < m)
        return fail(GINN_B200_BAD_ARGUMENT, "pair %d: bad B / da", i);
      Problem p;
      std::memset(&p, 0, sizeof(p));
      p.npairs = 1;
      p.a[0] = make_operand(dtype, dout, lddout, 0, 1, 0, out, act);
      p.b[0] = make_operand(dtype, q.b, q.ldb, 0, 1, 0);
      p.k[0] = n;
      p.M = (int)m; p.N = (int)q.k; p.batches = 1;
      p.c = q.da; p.ldc = q.ldda;
      p.accumulate = 1;
      if (!dbias_done) {
        p.rowsum = dbias;  // bias gradient rides on the loader of dA
        dbias_done = true;
      }
      if (int s = run_problem(ctx, dtype, p, stream)) return s;
    }
  }
  if (!dbias_done) {
    CU_TRY(gb::launch_rowsum(dtype, dout, act != GINN_B200_ACT_NONE ? out : nullptr, act, lddout,
                             (int)m, n, dbias, stream));
    g_launches.fetch_add(1);
  }
  CU_TRY(fk.join());
  return GINN_B200_OK;
}

int ginn_b200_grouped(int device, void* stream_, int dtype, int mode, int ngroups,
                      const ginn_b200_group* groups) {
  LevelPlan plan;
  if (int s = plan_level(dtype, mode, ngroups, groups, &plan)) return s;
  if (plan.live == 0) return GINN_B200_OK;
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  std::vector<Problem> direct;
  if (direct_level(dtype, mode, ngroups, groups, ctx->num_sms, &direct))
    return launch_direct_level(direct, stream, ctx->d_status);
  if (int s = refuse_capture(stream, "ginn_b200_grouped")) return s;
  unsigned char *h, *d;
  int half = 0;
  if (int s = stage_alloc(ctx, plan.bytes, stream, &h, &d, &half)) return s;
  LevelLaunch ll = fill_level_image(dtype, mode, ngroups, groups, plan, ctx->num_sms, h, d);
  CU_TRY(cudaMemcpyAsync(d, h, plan.bytes, cudaMemcpyHostToDevice, stream));
  CU_TRY(launch_level(dtype, ll, reinterpret_cast<const Problem*>(d), stream, ctx->d_status));
  g_launches.fetch_add(1);
  return stage_mark(ctx, half, stream);
}

// Same work as ginn_b200_grouped, for callers that may not allocate (see include/ginn_b200.h).
// Nothing here calls cudaMalloc, cudaMallocHost, cudaFree or any allocating library routine:
// the device-side descriptors go into a fixed array inside the library image
// (grouped_static.cu), the host-side image is assembled in a fixed buffer below.
int ginn_b200_grouped_static(int device, void* stream_, int dtype, int mode, int ngroups,
                             const ginn_b200_group* groups) {
  static std::mutex image_mu;
  alignas(16) static unsigned char image[gb::kGroupedStaticBytes];
  LevelPlan plan;
  if (int s = plan_level(dtype, mode, ngroups, groups, &plan)) return s;
  if (plan.live == 0) return GINN_B200_OK;
  if (device < 0 || device >= kMaxDevices)
    return fail(GINN_B200_BAD_ARGUMENT, "device index %d out of range", device);
  CU_TRY(cudaSetDevice(device));
  int major = 0, num_sms = 0;
  CU_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  if (major != 10)
    return fail(GINN_B200_UNSUPPORTED, "device %d is not an sm_100 GPU", device);
  CU_TRY(cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, device));
  if (plan.bytes > gb::kGroupedStaticBytes)
    return fail(GINN_B200_BAD_ARGUMENT,
                "level too large for the allocation-free entry point: %zu bytes of descriptors "
                "and column tables, limit %zu (%d groups, 16 bytes per column); split the level "
                "or use ginn_b200_grouped",
                plan.bytes, gb::kGroupedStaticBytes, plan.live);
  // The host image below is one buffer shared by all calls: a captured copy would read it at
  // replay time, after later calls have overwritten it.
  if (int s = refuse_capture(static_cast<cudaStream_t>(stream_), "ginn_b200_grouped_static"))
    return s;
  void* scratch = nullptr;
  int* status = nullptr;
  CU_TRY(gb::grouped_static_scratch(device, &scratch, &status));
  std::lock_guard<std::mutex> lock(image_mu);
  LevelLaunch ll = fill_level_image(dtype, mode, ngroups, groups, plan, num_sms, image,
                                    static_cast<unsigned char*>(scratch));
  CU_TRY(gb::launch_grouped_static(dtype, image, plan.bytes, scratch, status, ll.nprobs, ll.tiles,
                                   ll.with_y, static_cast<cudaStream_t>(stream_)));
  g_launches.fetch_add(1);
  return GINN_B200_OK;
}

// A level whose descriptors stay resident on the device: built once, launched many times.
struct ginn_b200_level {
  int device;
  int dtype;
  LevelLaunch ll;
  unsigned char* d_image;
  DevCtx::Slab* slab = nullptr;     // where d_image lives
  cudaEvent_t uploaded = nullptr;   // the image's upload on the preparation stream
  bool upload_seen = false;
  std::vector<Problem> direct;  // table-free form of the level (then d_image is null)
  // cells level (ginn_b200_lstm_cells_level_create): d_image holds the pointer tables
  int cells = 0;                // 0: grouped products, 1: cell forward, 2: cell backward
  int hidden = 0;
  long long ncells = 0;
};

namespace {
constexpr size_t kSlabBytes = 4u << 20;

// Device memory for a level image plus its upload from `host` (pinned staging, asynchronous).
// The level must wait for `uploaded` before its first launch.
int level_upload(DevCtx* ctx, ginn_b200_level* lv, const void*, size_t bytes) {
  bytes = (bytes + 255) & ~size_t(255);
  {
    std::lock_guard<std::mutex> g(ctx->mu);
    if (!ctx->prep_stream) CU_TRY(cudaStreamCreateWithFlags(&ctx->prep_stream, cudaStreamNonBlocking));
    if (!ctx->slab || ctx->slab->off + bytes > ctx->slab->cap) {
      if (ctx->slab && ctx->slab->refs == 0) {  // nobody lives in the old slab any more
        cudaFree(ctx->slab->base);
        delete ctx->slab;
      }
      ctx->slab = new DevCtx::Slab();
      ctx->slab->cap = bytes > kSlabBytes ? bytes : kSlabBytes;
      cudaError_t e = cudaMalloc(&ctx->slab->base, ctx->slab->cap);
      if (e != cudaSuccess) {
        delete ctx->slab;
        ctx->slab = nullptr;
        return fail(GINN_B200_CUDA_ERROR, "preparing a level failed: %s", cudaGetErrorString(e));
      }
    }
    lv->slab = ctx->slab;
    lv->d_image = ctx->slab->base + ctx->slab->off;
    ctx->slab->off += bytes;
    ++ctx->slab->refs;
  }
  return GINN_B200_OK;
}

// Drops a level's claim on its slab; the slab goes when its last level does (unless it is the
// one new levels are still carved from).
void level_release(ginn_b200_level* lv) {
  if (!lv->slab) return;
  DevCtx& c = g_ctx[lv->device];
  std::lock_guard<std::mutex> g(c.mu);
  if (--lv->slab->refs == 0 && lv->slab != c.slab) {
    cudaSetDevice(lv->device);
    cudaFree(lv->slab->base);
    delete lv->slab;
  }
  lv->slab = nullptr;
}

// Copies `bytes` of `image` (a host vector) into the level's device image: through the pinned
// staging ring on the preparation stream, leaving an event behind.
int level_copy(DevCtx* ctx, ginn_b200_level* lv, const unsigned char* image, size_t bytes) {
  unsigned char *h, *d_ring;
  int half = 0;
  if (int s = stage_alloc(ctx, bytes, ctx->prep_stream, &h, &d_ring, &half)) return s;
  std::memcpy(h, image, bytes);
  CU_TRY(cudaMemcpyAsync(lv->d_image, h, bytes, cudaMemcpyHostToDevice, ctx->prep_stream));
  CU_TRY(cudaEventCreateWithFlags(&lv->uploaded, cudaEventDisableTiming));
  CU_TRY(cudaEventRecord(lv->uploaded, ctx->prep_stream));
  return stage_mark(ctx, half, ctx->prep_stream);
}

// Before a level's first launch: its image must have arrived.  A host-side wait (the upload was
// queued at preparation time and is normally long done), so it is also legal under capture.
int level_ready(ginn_b200_level* lv) {
  if (lv->uploaded && !lv->upload_seen) {
    CU_TRY(cudaEventSynchronize(lv->uploaded));
    lv->upload_seen = true;
  }
  return GINN_B200_OK;
}
}  // namespace

int ginn_b200_level_create(int device, int dtype, int mode, int ngroups,
                           const ginn_b200_group* groups, ginn_b200_level** out) {
  if (out == nullptr) return fail(GINN_B200_BAD_ARGUMENT, "null output handle");
  *out = nullptr;
  LevelPlan plan;
  if (int s = plan_level(dtype, mode, ngroups, groups, &plan)) return s;
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  ginn_b200_level* lv = new ginn_b200_level{device, dtype, LevelLaunch{}, nullptr, {}};
  const bool direct =
      plan.live > 0 && direct_level(dtype, mode, ngroups, groups, ctx->num_sms, &lv->direct);
  if (!direct) lv->direct.clear();
  if (plan.live > 0 && !direct) {
    std::vector<unsigned char> h(plan.bytes);
    int s = level_upload(ctx, lv, nullptr, plan.bytes);
    if (s == GINN_B200_OK) {
      lv->ll = fill_level_image(dtype, mode, ngroups, groups, plan, ctx->num_sms, h.data(),
                                lv->d_image);
      s = level_copy(ctx, lv, h.data(), plan.bytes);
    }
    if (s != GINN_B200_OK) {
      ginn_b200_level_destroy(lv);
      return s;
    }
  }
  *out = lv;
  return GINN_B200_OK;
}

int ginn_b200_level_run(ginn_b200_level* level, void* stream) {
  if (level == nullptr) return fail(GINN_B200_BAD_ARGUMENT, "null level");
  if (level->d_image == nullptr && level->direct.empty()) return GINN_B200_OK;
  DevCtx* ctx;
  if (int s = get_ctx(level->device, &ctx)) return s;
  if (int s = level_ready(level)) return s;
  if (level->cells) {
    CU_TRY(gb::launch_lstm_cells(level->cells == 2,
                                 reinterpret_cast<const void* const*>(level->d_image),
                                 level->hidden, level->ncells, static_cast<cudaStream_t>(stream)));
    g_launches.fetch_add(1);
    return GINN_B200_OK;
  }
  if (!level->direct.empty())
    return launch_direct_level(level->direct, static_cast<cudaStream_t>(stream), ctx->d_status);
  CU_TRY(launch_level(level->dtype, level->ll, reinterpret_cast<const Problem*>(level->d_image),
                      static_cast<cudaStream_t>(stream), ctx->d_status));
  g_launches.fetch_add(1);
  return GINN_B200_OK;
}

namespace {
int check_cells(int64_t hidden, int64_t n, const void* const* tables, int ntab) {
  if (hidden < 0 || n < 0 || hidden > 0x7fffffffLL || n > 65535)
    return fail(GINN_B200_BAD_ARGUMENT, "bad extents hidden=%lld n=%lld (n <= 65535)",
                (long long)hidden, (long long)n);
  if (hidden == 0 || n == 0) return GINN_B200_OK;
  if (!tables) return fail(GINN_B200_BAD_ARGUMENT, "null tables");
  for (int t = 0; t < ntab; ++t)
    for (int64_t j = 0; j < n; ++j) {
      const bool optional = (ntab == 4 && t == 1) || (ntab == 7 && (t == 2 || t == 6));
      if (!optional && tables[t * n + j] == nullptr)
        return fail(GINN_B200_BAD_ARGUMENT, "table %d, cell %lld: null pointer", t, (long long)j);
    }
  return GINN_B200_OK;
}
}  // namespace

int ginn_b200_lstm_cells(int device, void* stream_, int backward, int64_t hidden, int64_t n,
                         const void* const* tables) {
  const int ntab = backward ? 7 : 4;
  if (int s = check_cells(hidden, n, tables, ntab)) return s;
  if (hidden == 0 || n == 0) return GINN_B200_OK;
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (int s = refuse_capture(stream, "ginn_b200_lstm_cells")) return s;
  const size_t bytes = static_cast<size_t>(ntab) * n * sizeof(void*);
  unsigned char *h, *d;
  int half = 0;
  if (int s = stage_alloc(ctx, bytes, stream, &h, &d, &half)) return s;
  std::memcpy(h, tables, bytes);
  CU_TRY(cudaMemcpyAsync(d, h, bytes, cudaMemcpyHostToDevice, stream));
  CU_TRY(gb::launch_lstm_cells(backward != 0, reinterpret_cast<const void* const*>(d), (int)hidden, n,
                               stream));
  g_launches.fetch_add(1);
  return stage_mark(ctx, half, stream);
}

int ginn_b200_lstm_cells_level_create(int device, int backward, int64_t hidden, int64_t n,
                                      const void* const* tables, ginn_b200_level** out) {
  if (out == nullptr) return fail(GINN_B200_BAD_ARGUMENT, "null output handle");
  *out = nullptr;
  const int ntab = backward ? 7 : 4;
  if (int s = check_cells(hidden, n, tables, ntab)) return s;
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  ginn_b200_level* lv = new ginn_b200_level{device, GINN_B200_F32, LevelLaunch{}, nullptr, {}};
  lv->cells = backward ? 2 : 1;
  lv->hidden = (int)hidden;
  lv->ncells = n;
  if (hidden > 0 && n > 0) {
    const size_t bytes = static_cast<size_t>(ntab) * n * sizeof(void*);
    int s = level_upload(ctx, lv, nullptr, bytes);
    if (s == GINN_B200_OK)
      s = level_copy(ctx, lv, reinterpret_cast<const unsigned char*>(tables), bytes);
    if (s != GINN_B200_OK) {
      ginn_b200_level_destroy(lv);
      return s;
    }
  }
  *out = lv;
  return GINN_B200_OK;
}

int ginn_b200_level_destroy(ginn_b200_level* level) {
  if (level == nullptr) return GINN_B200_OK;
  if (level->uploaded) {
    cudaSetDevice(level->device);
    cudaEventSynchronize(level->uploaded);  // the upload must not outlive the slab
    cudaEventDestroy(level->uploaded);
  }
  level_release(level);
  delete level;
  return GINN_B200_OK;
}

int ginn_b200_attention_forward(int device, void* stream_, int dtype, int64_t t, int64_t hs,
                                int64_t batches, const void* k, int64_t ldk, int64_t stride_k,
                                const void* q, int64_t ldq, int64_t stride_q, const void* v,
                                int64_t ldv, int64_t stride_v, float scale, int causal, void* o,
                                int64_t ldo, int64_t stride_o, void* p, int64_t ldp,
                                int64_t stride_p) {
  if (int s = check_common(dtype, t, hs, batches)) return s;
  if (t == 0 || hs == 0 || batches == 0) return GINN_B200_OK;
  if (!k || !q || !v || !o) return fail(GINN_B200_BAD_ARGUMENT, "null tensor pointer");
  if (ldk < t || ldq < hs || ldv < hs || ldo < hs || (p && ldp < t))
    return fail(GINN_B200_BAD_ARGUMENT, "leading dimension smaller than the matrix it describes");
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  gb::AttentionArgs a;
  a.K = k; a.Q = q; a.V = v; a.O = o; a.P = p;
  a.ldk = ldk; a.ldq = ldq; a.ldv = ldv; a.ldo = ldo; a.ldp = ldp;
  a.strideK = stride_k; a.strideQ = stride_q; a.strideV = stride_v; a.strideO = stride_o;
  a.strideP = stride_p;
  a.T = (int)t; a.hs = (int)hs; a.batches = (int)batches;
  a.scale = scale;
  a.causal = causal ? 1 : 0;
  if (!(scale > 0.f)) return fail(GINN_B200_BAD_ARGUMENT, "attention scale must be positive");
  if (dtype == GINN_B200_F32 && t_force_path == PATH_AUTO && gb::attention_fused_supported(a)) {
    CU_TRY(gb::launch_attention_fwd(a, stream, ctx->d_status));
    g_launches.fetch_add(1);
    return GINN_B200_OK;
  }
  // The sequence the reference runs, with `p` as the score tensor.
  if (!p) return fail(GINN_B200_BAD_ARGUMENT,
                      "this shape takes the unfused path, which needs `p` as its score buffer");
  if (int s = gemm_impl(device, stream_, dtype, 0, 0, t, t, hs, k, ldk, stride_k, q, ldq, stride_q, p,
                        ldp, stride_p, batches, 0))
    return s;
  if (scale != 1.f || causal) {
    if (dtype != GINN_B200_F32)
      return fail(GINN_B200_UNSUPPORTED, "scale / causal mask on the unfused path are fp32 only");
    CU_TRY(gb::launch_scale_mask_f32(static_cast<float*>(p), ldp, stride_p, (int)t, (int)batches, scale,
                                     a.causal, stream));
    g_launches.fetch_add(1);
  }
  if (stride_p != ldp * t)
    return fail(GINN_B200_UNSUPPORTED, "the unfused path needs densely packed score matrices");
  CU_TRY(gb::launch_pick_nll_forward(dtype, p, ldp, nullptr, p, ldp, nullptr, (int)t, t * batches,
                                     stream));
  g_launches.fetch_add(1);
  return gemm_impl(device, stream_, dtype, 0, 0, hs, t, t, v, ldv, stride_v, p, ldp, stride_p, o, ldo,
                   stride_o, batches, 0);
}

int ginn_b200_attention_backward(int device, void* stream_, int dtype, int64_t t, int64_t hs,
                                 int64_t batches, const void* k, int64_t ldk, int64_t stride_k,
                                 const void* q, int64_t ldq, int64_t stride_q, const void* v,
                                 int64_t ldv, int64_t stride_v, float scale, const void* p,
                                 int64_t ldp, int64_t stride_p, const void* d_o, int64_t ldo,
                                 int64_t stride_o, void* ds, void* dk, void* dq, void* dv) {
  if (int s = check_common(dtype, t, hs, batches)) return s;
  if (t == 0 || hs == 0 || batches == 0) return GINN_B200_OK;
  if (!k || !q || !v || !p || !d_o || !ds) return fail(GINN_B200_BAD_ARGUMENT, "null tensor pointer");
  if (stride_p != ldp * t)
    return fail(GINN_B200_UNSUPPORTED, "the score matrices must be densely packed (stride = ld * t)");
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  // dV and dQ do not depend on the chain dP -> dS -> dK': they run on a second stream, where
  // their CTAs take the SMs the other products leave idle at the end of their last wave and
  // during the softmax pass (256 x (256, 64): 0.33 -> 0.31 ms per forward + backward step).
  Fork fk;
  bool fork = t_fork_streams && (dv != nullptr) + (dq != nullptr) + (dk != nullptr) >= 2;
  if (fork && dk) {  // gradients that share memory (tied inputs) stay on one stream
    const int es = dtype == GINN_B200_F32 ? 4 : 2;
    auto span = [&](const void* p0, int64_t rows, int64_t cols, int64_t ld, int64_t stride) {
      ByteRange r = range_of(p0, rows, cols, ld, es);
      if (p0) r.hi += (batches - 1) * stride * es;
      return r;
    };
    const ByteRange rk = span(dk, t, hs, ldk, stride_k);
    if (overlap(rk, span(dv, hs, t, ldv, stride_v)) || overlap(rk, span(dq, hs, t, ldq, stride_q)))
      fork = false;
  }
  cudaStream_t side = stream;
  if (fork) {
    CU_TRY(fk.begin(ctx, stream));
    side = fk.side;
  }
  auto join = [&](int status) {
    cudaError_t e = fk.join();
    if (e != cudaSuccess && status == GINN_B200_OK)
      return fail(GINN_B200_CUDA_ERROR, "joining the second stream failed: %s", cudaGetErrorString(e));
    return status;
  };
  // dv (hs x T) += d_o (hs x T) * P^T
  if (dv)
    if (int s = gemm_impl(device, side, dtype, 0, 1, hs, t, t, d_o, ldo, stride_o, p, ldp, stride_p,
                          dv, ldv, stride_v, batches, 1))
      return join(s);
  if (!dk && !dq) return join(GINN_B200_OK);
  // dP (T x T) = V^T * d_o, then dS = P (.) (dP - colsum(P (.) dP)) in place
  if (int s = gemm_impl(device, stream_, dtype, 1, 0, t, t, hs, v, ldv, stride_v, d_o, ldo, stride_o, ds,
                        ldp, stride_p, batches, 0))
    return join(s);
  cudaError_t e = gb::launch_softmax_backward(dtype, p, ldp, ds, ldp, ds, ldp, (int)t, t * batches, 0, stream);
  if (e != cudaSuccess)
    return join(fail(GINN_B200_CUDA_ERROR, "softmax backward launch failed: %s", cudaGetErrorString(e)));
  g_launches.fetch_add(1);
  if (scale != 1.f) {
    if (dtype != GINN_B200_F32) return join(fail(GINN_B200_UNSUPPORTED, "scale != 1 is fp32 only"));
    e = gb::launch_scale_mask_f32(static_cast<float*>(ds), ldp, stride_p, (int)t, (int)batches, scale, 0,
                                  stream);
    if (e != cudaSuccess)
      return join(fail(GINN_B200_CUDA_ERROR, "scale launch failed: %s", cudaGetErrorString(e)));
    g_launches.fetch_add(1);
  }
  // dk (T x hs) += dS * Q^T;  dq (hs x T) += K'^T * dS (on the second stream once dS is there)
  if (fork && dq && dk) {
    e = fk.sync_side();
    if (e != cudaSuccess)
      return join(fail(GINN_B200_CUDA_ERROR, "forking the second stream failed: %s", cudaGetErrorString(e)));
  }
  cudaStream_t dq_stream = (fork && dq && dk) ? side : stream;
  if (dk)
    if (int s = gemm_impl(device, stream_, dtype, 0, 1, t, hs, t, ds, ldp, stride_p, q, ldq, stride_q, dk,
                          ldk, stride_k, batches, 1))
      return join(s);
  if (dq)
    if (int s = gemm_impl(device, dq_stream, dtype, 1, 0, hs, t, t, k, ldk, stride_k, ds, ldp, stride_p, dq,
                          ldq, stride_q, batches, 1))
      return join(s);
  return join(GINN_B200_OK);
}

int ginn_b200_prod_backward(int device, void* stream_, int dtype, int64_t m, int64_t n, int64_t k,
                            int64_t batches, const void* a, int64_t lda, int64_t stride_a,
                            const void* b, int64_t ldb, int64_t stride_b, const void* dc,
                            int64_t lddc, int64_t stride_dc, void* da, int64_t ldda,
                            int64_t stride_da, void* db, int64_t lddb, int64_t stride_db) {
  if (int s = check_common(dtype, m, n, k)) return s;
  if (batches < 0) return fail(GINN_B200_BAD_ARGUMENT, "negative batch count");
  if (!da && !db) return GINN_B200_OK;
  if (m == 0 || n == 0 || k == 0 || batches == 0) return GINN_B200_OK;  // nothing to add
  if (!dc || (da && !b) || (db && !a)) return fail(GINN_B200_BAD_ARGUMENT, "null tensor pointer");
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  Fork fk;
  cudaStream_t db_stream = stream;
  if (t_fork_streams && da && db) {
    const int es = dtype == GINN_B200_F32 ? 4 : 2;
    ByteRange ra = range_of(da, m, k, ldda, es), rb = range_of(db, k, n, lddb, es);
    ra.hi += (batches - 1) * stride_da * es;
    rb.hi += (batches - 1) * stride_db * es;
    if (!overlap(ra, rb)) {  // Prod(x, x) adds both gradients into one tensor: one stream then
      CU_TRY(fk.begin(ctx, stream));
      db_stream = fk.side;
    }
  }
  int status = GINN_B200_OK;
  if (da)  // da (m x k) += dc (m x n) * b^T (n x k)
    status = gemm_impl(device, stream_, dtype, 0, 1, m, k, n, dc, lddc, stride_dc, b, ldb, stride_b, da,
                       ldda, stride_da, batches, 1);
  if (db && status == GINN_B200_OK)  // db (k x n) += a^T (k x m) * dc (m x n)
    status = gemm_impl(device, db_stream, dtype, 1, 0, k, n, m, a, lda, stride_a, dc, lddc, stride_dc,
                       db, lddb, stride_db, batches, 1);
  const cudaError_t je = fk.join();
  if (je != cudaSuccess && status == GINN_B200_OK)
    status = fail(GINN_B200_CUDA_ERROR, "joining the second stream failed: %s", cudaGetErrorString(je));
  return status;
}

size_t ginn_b200_conv2d_workspace(int dtype, int64_t C, int64_t R, int64_t W, int64_t B, int64_t F,
                                  int64_t KR, int64_t KC, int64_t sr, int64_t sc) {
  gb::ConvShape s;
  if ((dtype != GINN_B200_F32 && dtype != GINN_B200_F16) ||
      !gb::conv2d_geometry(C, R, W, B, F, KR, KC, sr, sc, &s))
    return 0;
  return (static_cast<size_t>(s.inner) * s.ncols * esize(dtype) + 255) & ~size_t(255);
}

namespace {
// Shared set-up of the two convolution entry points: geometry, context, workspace.
struct ConvCall {
  gb::ConvShape shape;
  DevCtx* ctx = nullptr;
  void* ws = nullptr;
  bool own_ws = false;
};
int conv_begin(int device, cudaStream_t stream, int dtype, int64_t C, int64_t R, int64_t W,
               int64_t B, int64_t F, int64_t KR, int64_t KC, int64_t sr, int64_t sc,
               void* workspace, ConvCall* call) {
  if (dtype != GINN_B200_F32 && dtype != GINN_B200_F16)
    return fail(GINN_B200_UNSUPPORTED, "dtype %d is not fp32 (0) or fp16 (1)", dtype);
  if (!gb::conv2d_geometry(C, R, W, B, F, KR, KC, sr, sc, &call->shape))
    return fail(GINN_B200_BAD_ARGUMENT,
                "bad convolution extents: input %lld x %lld x %lld x %lld, filters %lld x %lld x "
                "%lld, strides %lld, %lld", (long long)C, (long long)R, (long long)W, (long long)B,
                (long long)F, (long long)KR, (long long)KC, (long long)sr, (long long)sc);
  if (int s = get_ctx(device, &call->ctx)) return s;
  call->ws = workspace;
  if (workspace == nullptr) {
    const size_t bytes = static_cast<size_t>(call->shape.inner) * call->shape.ncols * esize(dtype);
    CU_TRY(cudaMallocAsync(&call->ws, bytes, stream));
    call->own_ws = true;
  } else if (!aligned16(workspace)) {
    return fail(GINN_B200_BAD_ARGUMENT, "the convolution workspace must be 16-byte aligned");
  }
  return GINN_B200_OK;
}
void conv_end(ConvCall* call, cudaStream_t stream) {
  if (call->own_ws && call->ws) cudaFreeAsync(call->ws, stream);
}
}  // namespace

int ginn_b200_conv2d_forward(int device, void* stream_, int dtype, int64_t C, int64_t R, int64_t W,
                             int64_t B, int64_t F, int64_t KR, int64_t KC, int64_t sr, int64_t sc,
                             const void* x, const void* k, void* y, void* workspace) {
  if (!x || !k || !y) return fail(GINN_B200_BAD_ARGUMENT, "null tensor pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  ConvCall call;
  if (int s = conv_begin(device, stream, dtype, C, R, W, B, F, KR, KC, sr, sc, workspace, &call))
    return s;
  const gb::ConvShape& g = call.shape;
  int status = GINN_B200_OK;
  cudaError_t e = gb::launch_im2col(dtype, x, call.ws, C, R, W, B, F, KR, KC, sr, sc, g,
                                    call.ctx->num_sms, stream);
  if (e != cudaSuccess) status = fail(GINN_B200_CUDA_ERROR, "patch extraction: %s", cudaGetErrorString(e));
  g_launches.fetch_add(1);
  if (status == GINN_B200_OK)  // y (F x N) = k (F x CKK) * patches (CKK x N)
    status = gemm_impl(device, stream_, dtype, 0, 0, F, g.ncols, g.inner, k, F, 0, call.ws, g.inner,
                       0, y, F, 0, 1, 0);
  conv_end(&call, stream);
  return status;
}

int ginn_b200_conv2d_backward(int device, void* stream_, int dtype, int64_t C, int64_t R, int64_t W,
                              int64_t B, int64_t F, int64_t KR, int64_t KC, int64_t sr, int64_t sc,
                              const void* x, const void* k, const void* dy, void* dx, void* dk,
                              void* workspace) {
  if (!dy || (dk && !x) || (dx && !k)) return fail(GINN_B200_BAD_ARGUMENT, "null tensor pointer");
  if (!dx && !dk) return GINN_B200_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  ConvCall call;
  if (int s = conv_begin(device, stream, dtype, C, R, W, B, F, KR, KC, sr, sc, workspace, &call))
    return s;
  const gb::ConvShape& g = call.shape;
  int status = GINN_B200_OK;
  if (dk) {  // dk (F x CKK) += dy (F x N) * patches^T (N x CKK)
    cudaError_t e = gb::launch_im2col(dtype, x, call.ws, C, R, W, B, F, KR, KC, sr, sc, g,
                                      call.ctx->num_sms, stream);
    if (e != cudaSuccess) status = fail(GINN_B200_CUDA_ERROR, "patch extraction: %s", cudaGetErrorString(e));
    g_launches.fetch_add(1);
    if (status == GINN_B200_OK)
      status = gemm_impl(device, stream_, dtype, 0, 1, F, g.inner, g.ncols, dy, F, 0, call.ws, g.inner,
                         0, dk, F, 0, 1, 1);
  }
  if (dx && status == GINN_B200_OK) {  // dpatches (CKK x N) = k^T (CKK x F) * dy (F x N)
    status = gemm_impl(device, stream_, dtype, 1, 0, g.inner, g.ncols, F, k, F, 0, dy, F, 0, call.ws,
                       g.inner, 0, 1, 0);
    if (status == GINN_B200_OK) {
      cudaError_t e = gb::launch_col2im_add(dtype, call.ws, dx, C, R, W, B, F, KR, KC, sr, sc, g,
                                            call.ctx->num_sms, stream);
      if (e != cudaSuccess) status = fail(GINN_B200_CUDA_ERROR, "patch scatter: %s", cudaGetErrorString(e));
      g_launches.fetch_add(1);
    }
  }
  conv_end(&call, stream);
  return status;
}

int ginn_b200_fill(int device, void* stream, int dtype, int64_t n, void* x, float value) {
  if (dtype != GINN_B200_F32 && dtype != GINN_B200_F16)
    return fail(GINN_B200_UNSUPPORTED, "dtype %d is not fp32 (0) or fp16 (1)", dtype);
  if (n < 0) return fail(GINN_B200_BAD_ARGUMENT, "negative element count");
  if (n == 0) return GINN_B200_OK;
  if (!x) return fail(GINN_B200_BAD_ARGUMENT, "null pointer");
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  CU_TRY(gb::launch_fill(dtype, x, n, value, ctx->num_sms, static_cast<cudaStream_t>(stream)));
  g_launches.fetch_add(1);
  return GINN_B200_OK;
}

const char* ginn_b200_last_error(void) { return t_error.c_str(); }

int ginn_b200_device_status(int device, int reset) {
  DevCtx* ctx = nullptr;
  if (get_ctx(device, &ctx) != GINN_B200_OK || ctx == nullptr) return -1;
  int v = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpy(&v, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (reset && v != 0) {
    cudaMemset(ctx->d_status, 0, sizeof(int));
    // a kernel that gave up may have left its tile queue half used
    cudaMemset(ctx->d_counters, 0, 2 * kCounters * sizeof(int));
  }
  return v;
}

int ginn_b200_grouped_static_status(int device, int reset) {
  if (device < 0 || device >= kMaxDevices) return -1;
  if (cudaSetDevice(device) != cudaSuccess) return -1;
  void* scratch = nullptr;
  int* status = nullptr;
  if (gb::grouped_static_scratch(device, &scratch, &status) != cudaSuccess) return -1;
  int v = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpy(&v, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (reset && v != 0) cudaMemset(status, 0, sizeof(int));
  return v;
}

int ginn_b200_pick_nll_forward(int device, void* stream, int dtype, int64_t rows, int64_t cols,
                               const void* x, int64_t ldx, const int* index, void* smax,
                               int64_t ldsmax, void* value) {
  if (int s = check_common(dtype, rows, cols, 0)) return s;
  if (rows == 0 || cols == 0) return GINN_B200_OK;
  if (!x || !index || !smax || !value) return fail(GINN_B200_BAD_ARGUMENT, "null pointer");
  if (ldx < rows || ldsmax < rows)
    return fail(GINN_B200_BAD_ARGUMENT, "leading dimension smaller than %lld rows", (long long)rows);
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  CU_TRY(gb::launch_pick_nll_forward(dtype, x, ldx, index, smax, ldsmax, value, (int)rows, cols,
                                     static_cast<cudaStream_t>(stream)));
  g_launches.fetch_add(1);
  return GINN_B200_OK;
}

int ginn_b200_softmax_forward(int device, void* stream, int dtype, int64_t rows, int64_t cols,
                              const void* x, int64_t ldx, void* y, int64_t ldy) {
  if (int s = check_common(dtype, rows, cols, 0)) return s;
  if (rows == 0 || cols == 0) return GINN_B200_OK;
  if (!x || !y) return fail(GINN_B200_BAD_ARGUMENT, "null pointer");
  if (ldx < rows || ldy < rows)
    return fail(GINN_B200_BAD_ARGUMENT, "leading dimension smaller than %lld rows", (long long)rows);
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  CU_TRY(gb::launch_pick_nll_forward(dtype, x, ldx, nullptr, y, ldy, nullptr, (int)rows, cols,
                                     static_cast<cudaStream_t>(stream)));
  g_launches.fetch_add(1);
  return GINN_B200_OK;
}

int ginn_b200_softmax_backward(int device, void* stream, int dtype, int64_t rows, int64_t cols,
                               const void* y, int64_t ldy, const void* dy, int64_t lddy, void* dx,
                               int64_t lddx, int accumulate) {
  if (int s = check_common(dtype, rows, cols, 0)) return s;
  if (rows == 0 || cols == 0) return GINN_B200_OK;
  if (!y || !dy || !dx) return fail(GINN_B200_BAD_ARGUMENT, "null pointer");
  if (ldy < rows || lddy < rows || lddx < rows)
    return fail(GINN_B200_BAD_ARGUMENT, "leading dimension smaller than %lld rows", (long long)rows);
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  CU_TRY(gb::launch_softmax_backward(dtype, y, ldy, dy, lddy, dx, lddx, (int)rows, cols,
                                     accumulate ? 1 : 0, static_cast<cudaStream_t>(stream)));
  g_launches.fetch_add(1);
  return GINN_B200_OK;
}

int ginn_b200_pick_nll_backward(int device, void* stream, int dtype, int64_t rows, int64_t cols,
                                const void* smax, int64_t ldsmax, const int* index,
                                const void* grad, void* dx, int64_t lddx) {
  if (int s = check_common(dtype, rows, cols, 0)) return s;
  if (rows == 0 || cols == 0) return GINN_B200_OK;
  if (!smax || !index || !grad || !dx) return fail(GINN_B200_BAD_ARGUMENT, "null pointer");
  if (ldsmax < rows || lddx < rows)
    return fail(GINN_B200_BAD_ARGUMENT, "leading dimension smaller than %lld rows", (long long)rows);
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  CU_TRY(gb::launch_pick_nll_backward(dtype, smax, ldsmax, index, grad, dx, lddx, (int)rows, cols,
                                      static_cast<cudaStream_t>(stream)));
  g_launches.fetch_add(1);
  return GINN_B200_OK;
}

int ginn_b200_lstm_cell_forward(int device, void* stream, int64_t hidden, int64_t n, int64_t n_next,
                                float* gates, int64_t ldg, const float* c_prev, int64_t ldcp,
                                float* c, int64_t ldc, float* h, int64_t ldh, float* xh_next,
                                int64_t ldx) {
  if (hidden < 0 || n < 0 || n_next < 0 || n_next > n || hidden > 0x7fffffffLL)
    return fail(GINN_B200_BAD_ARGUMENT, "bad extents hidden=%lld n=%lld n_next=%lld",
                (long long)hidden, (long long)n, (long long)n_next);
  if (hidden == 0 || n == 0) return GINN_B200_OK;
  if (!gates || !c || !h || (n_next > 0 && xh_next == nullptr && ldx != 0))
    return fail(GINN_B200_BAD_ARGUMENT, "null pointer");
  if (ldg < 4 * hidden || ldc < hidden || ldh < hidden || (c_prev && ldcp < hidden) ||
      (xh_next && ldx < hidden))
    return fail(GINN_B200_BAD_ARGUMENT, "leading dimension too small");
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  CU_TRY(gb::launch_lstm_cell_forward(gates, ldg, c_prev, ldcp, c, ldc, h, ldh, xh_next, ldx,
                                      (int)hidden, n, xh_next ? n_next : 0,
                                      static_cast<cudaStream_t>(stream)));
  g_launches.fetch_add(1);
  return GINN_B200_OK;
}

int ginn_b200_lstm_cell_backward(int device, void* stream, int64_t hidden, int64_t n,
                                 int64_t n_next, const float* gates, int64_t ldg, const float* c,
                                 int64_t ldc, const float* c_prev, int64_t ldcp,
                                 const float* dh_next, int64_t lddh, const float* dc_next,
                                 int64_t lddc, float dh_end, float* dgates, int64_t lddg,
                                 float* dc_out, int64_t lddo) {
  if (hidden < 0 || n < 0 || n_next < 0 || n_next > n || hidden > 0x7fffffffLL)
    return fail(GINN_B200_BAD_ARGUMENT, "bad extents hidden=%lld n=%lld n_next=%lld",
                (long long)hidden, (long long)n, (long long)n_next);
  if (hidden == 0 || n == 0) return GINN_B200_OK;
  if (!gates || !c || !dgates || !dc_out || (n_next > 0 && (!dh_next || !dc_next)))
    return fail(GINN_B200_BAD_ARGUMENT, "null pointer");
  if (ldg < 4 * hidden || lddg < 4 * hidden || ldc < hidden || lddo < hidden ||
      (c_prev && ldcp < hidden) || (n_next > 0 && (lddh < hidden || lddc < hidden)))
    return fail(GINN_B200_BAD_ARGUMENT, "leading dimension too small");
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  CU_TRY(gb::launch_lstm_cell_backward(gates, ldg, c, ldc, c_prev, ldcp, dh_next, lddh, dc_next,
                                       lddc, dh_end, dgates, lddg, dc_out, lddo, (int)hidden, n,
                                       n_next, static_cast<cudaStream_t>(stream)));
  g_launches.fetch_add(1);
  return GINN_B200_OK;
}

int ginn_b200_adam_update(int device, void* stream, int dtype, int64_t n, void* w, void* d,
                          float* m, float* v, float lr, float clip, float eps, float beta1,
                          float beta2, float beta1_t, float beta2_t) {
  if (dtype != GINN_B200_F32 && dtype != GINN_B200_F16)
    return fail(GINN_B200_UNSUPPORTED, "dtype %d is not fp32 (0) or fp16 (1)", dtype);
  if (n < 0) return fail(GINN_B200_BAD_ARGUMENT, "negative element count");
  if (n == 0) return GINN_B200_OK;
  if (!w || !d || !m || !v) return fail(GINN_B200_BAD_ARGUMENT, "null pointer");
  if (!(beta1_t < 1.f) || !(beta2_t < 1.f))
    return fail(GINN_B200_BAD_ARGUMENT, "beta powers must be below 1 (got %g, %g)", beta1_t, beta2_t);
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  const float step = -lr * (1.f / (1.f - beta1_t));
  const float vscale = 1.f / (1.f - beta2_t);
  CU_TRY(gb::launch_adam(dtype, w, d, m, v, n, clip, beta1, beta2, step, vscale, eps, ctx->num_sms,
                         static_cast<cudaStream_t>(stream)));
  g_launches.fetch_add(1);
  return GINN_B200_OK;
}

int ginn_b200_selftest(int device) {
  DevCtx* ctx;
  if (int s = get_ctx(device, &ctx)) return s;
  // Run on scratch words of our own so that the device status word keeps its meaning.
  int* d = nullptr;
  CU_TRY(cudaMalloc(&d, 2 * sizeof(int)));
  CU_TRY(cudaMemset(d, 0, 2 * sizeof(int)));
  cudaError_t e = gb::launch_wait_selftest(d, 200000, d + 1, nullptr);  // ~0.1 ms limit
  int h[2] = {0, 0};
  if (e == cudaSuccess) e = cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
  cudaFree(d);
  if (e != cudaSuccess)
    return fail(GINN_B200_CUDA_ERROR, "self test failed to run: %s", cudaGetErrorString(e));
  const int want = (gb::DEV_TIMEOUT_SELFTEST << 16) | 0x5e1f;
  if (h[0] != want || h[1] != 2)
    return fail(GINN_B200_DEVICE_TIMEOUT,
                "bounded wait did not report as expected: status %#x (want %#x), flag %d", h[0],
                want, h[1]);
  return GINN_B200_OK;
}

int ginn_b200_version(void) { return 200; }

int ginn_b200_set_option(const char* name, int value) {
  if (name && std::strcmp(name, "force_path") == 0) {
    if (value < 0 || value > 5 || value == 1)
      return fail(GINN_B200_BAD_ARGUMENT, "force_path must be 0, 2, 3, 4 or 5");
    t_force_path = value;
    return GINN_B200_OK;
  }
  if (name && std::strcmp(name, "pair_group_m") == 0) {
    if (value < 0 || value > 1024) return fail(GINN_B200_BAD_ARGUMENT, "pair_group_m must be 0..1024");
    t_pair_group_m = value;
    return GINN_B200_OK;
  }
  if (name && std::strcmp(name, "fork_streams") == 0) {
    if (value < 0 || value > 1) return fail(GINN_B200_BAD_ARGUMENT, "fork_streams must be 0 or 1");
    t_fork_streams = value;
    return GINN_B200_OK;
  }
  if (name && std::strcmp(name, "presplit") == 0) {
    if (value < 0 || value > 1) return fail(GINN_B200_BAD_ARGUMENT, "presplit must be 0 or 1");
    t_presplit = value;
    return GINN_B200_OK;
  }
  if (name && std::strcmp(name, "pair_l2_hint") == 0) {
    if (value < 0 || value > 3) return fail(GINN_B200_BAD_ARGUMENT, "pair_l2_hint must be 0..3");
    t_pair_l2_hint = value;
    return GINN_B200_OK;
  }
  if (name && std::strcmp(name, "max_split") == 0) {
    if (value < 0 || value > 32) return fail(GINN_B200_BAD_ARGUMENT, "max_split must be 0..32");
    t_max_split = value;
    return GINN_B200_OK;
  }
  if (name && std::strcmp(name, "walk_kblocks") == 0) {
    if (value < 0 || value > 4096) return fail(GINN_B200_BAD_ARGUMENT, "walk_kblocks must be 0..4096");
    t_walk_kblocks = value;
    return GINN_B200_OK;
  }
  if (name && std::strcmp(name, "pdl") == 0) {
    t_pdl = value != 0;
    return GINN_B200_OK;
  }
  if (name && std::strcmp(name, "sm_margin") == 0) {
    if (value < 0 || value > 128) return fail(GINN_B200_BAD_ARGUMENT, "sm_margin must be 0..128");
    t_sm_margin = value;
    return GINN_B200_OK;
  }
  return fail(GINN_B200_UNSUPPORTED, "unknown option '%s'", name ? name : "(null)");
}

int64_t ginn_b200_launch_count(void) { return g_launches.load(); }

}  // extern "C"
