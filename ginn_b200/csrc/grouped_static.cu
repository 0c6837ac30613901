// Grouped launch that allocates nothing.
//
// The ordinary grouped launch keeps its problem descriptors and column-pointer tables in a
// cudaMalloc'ed ring.  Some hosts cannot allocate at the point where they call: a caller that
// runs inside a memory pool it must not disturb, or one that has pledged a fixed footprint
// (ginn's PreallocGpuDevice style of accounting, where every byte taken from the GPU is counted).
// For them the same kernels read their descriptors from a fixed array that is part of the
// library image, so nothing is requested from the CUDA allocator at call time.
//
// The array exists once per GPU that loads the library and stays until the process exits.
// All calls on a GPU share it, and it always holds whatever the last call put there; the part a
// call uses is completely rewritten by that call, so nothing in it needs clearing.  Two calls
// whose GPU work overlaps (different streams) would overwrite each other's descriptors: keep
// calls of this variant on one stream, or order them with events.
#include <mutex>
#include "launch.h"

namespace gb {

static __device__ __align__(256) unsigned char g_grouped_static_scratch[kGroupedStaticBytes];
// Status word of the kernels launched through this variant: a bounded wait that runs out
// records its code here (the ordinary entry points use a cudaMalloc'ed word instead).
static __device__ int g_grouped_static_status;

namespace {
struct StaticSlot {
  void* scratch = nullptr;
  int* status = nullptr;
  bool ready = false;
};
StaticSlot g_static_slots[64];
std::mutex g_static_mu;
}  // namespace

// `device` must be current.  In host code the arrays' names are only handles, not device
// addresses, so the addresses are looked up once per device and cached.
cudaError_t grouped_static_scratch(int device, void** scratch, int** status) {
  if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> g(g_static_mu);
  StaticSlot& slot = g_static_slots[device];
  if (!slot.ready) {
    void* p = nullptr;
    void* s = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_grouped_static_scratch);
    if (e != cudaSuccess) return e;
    e = cudaGetSymbolAddress(&s, g_grouped_static_status);
    if (e != cudaSuccess) return e;
    slot.scratch = p;
    slot.status = static_cast<int*>(s);
    slot.ready = true;
  }
  *scratch = slot.scratch;
  *status = slot.status;
  return cudaSuccess;
}

// Copies the host image (descriptors followed by pointer tables, already holding device
// addresses inside the static array) and launches the grouped kernel on it.
cudaError_t launch_grouped_static(int dtype, const void* host_image, size_t bytes, void* scratch,
                                  int* status, int nprobs, int total_tiles, bool with_y,
                                  cudaStream_t stream) {
  if (bytes > kGroupedStaticBytes) return cudaErrorInvalidValue;
  cudaError_t e = cudaMemcpyAsync(scratch, host_image, bytes, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return e;
  // Same kernels as the allocating entry point.
  if (dtype == 0)
    return launch_sgemm3x_gather_grouped(static_cast<const Problem*>(scratch), nprobs,
                                         total_tiles, with_y, stream, status);
  return launch_hgemm_gather_grouped(static_cast<const Problem*>(scratch), nprobs, total_tiles,
                                     stream, status);
}

}  // namespace gb
