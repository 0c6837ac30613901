// Devices: the part of ginn/dev.h the matrix-product path touches.
//   Device          alloc / realloc / free / kind / id / precedence / copy   (ginn/dev.h:63-75)
//   CpuDevice       host storage only -- this back end computes nothing on the CPU
//   GpuDevice       per-GPU singleton with its own blocking stream            (ginn/dev.h:149-212)
//   PreallocGpuDevice  bump allocator without padding, used()/clear()         (ginn/dev.h:214-261)
// There is no cuBLAS handle: products go through libginn_b200.so.
#ifndef GINN_B200_HOST_DEV_H
#define GINN_B200_HOST_DEV_H

#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <vector>

#include <ginn/def.h>
#include <ginn/except.h>

namespace ginn {

enum DeviceKind { CPU, GPU, NULL_DEV };

struct DeviceId {
  DeviceKind kind;
  size_t idx = 0;
  bool operator==(const DeviceId& o) const { return kind == o.kind && idx == o.idx; }
};

class Device {
 public:
  virtual ~Device() = default;
  virtual void* alloc(size_t bytes) = 0;
  virtual void* realloc(void* data, size_t bytes) = 0;
  virtual void free(void* data) = 0;
  virtual DeviceKind kind() const = 0;
  virtual DeviceId id() const = 0;
  virtual short precedence() const { return 0; }
  // Copies `bytes` from `other_data` on `other` into `data` on this device.
  void copy(const Device& other, void* data, const void* other_data, size_t bytes);
};
using DevPtr = std::shared_ptr<Device>;

class CpuDevice : public Device {
 public:
  void* alloc(size_t bytes) override { return std::malloc(bytes); }
  void* realloc(void* data, size_t bytes) override { return std::realloc(data, bytes); }
  void free(void* data) override { std::free(data); }
  DeviceKind kind() const override { return CPU; }
  DeviceId id() const override { return {CPU, 0}; }
};

inline DevPtr& cpu() {
  static DevPtr dev = std::make_shared<CpuDevice>();
  return dev;
}

class GpuDevice : public Device {
  size_t idx_;
  cudaStream_t stream_ = nullptr;

 public:
  explicit GpuDevice(size_t idx) : idx_(idx) {
    GINN_CUDA_CALL(cudaSetDevice(static_cast<int>(idx_)));
    GINN_CUDA_CALL(cudaStreamCreate(&stream_));  // blocking stream, like ginn's
  }
  void* alloc(size_t bytes) override {
    void* p = nullptr;
    GINN_CUDA_CALL(cudaSetDevice(static_cast<int>(idx_)));
    GINN_CUDA_CALL(cudaMalloc(&p, bytes));
    return p;
  }
  void* realloc(void* data, size_t bytes) override {  // contents are not preserved
    free(data);
    return alloc(bytes);
  }
  void free(void* data) override {
    if (data) {
      GINN_CUDA_CALL(cudaSetDevice(static_cast<int>(idx_)));
      GINN_CUDA_CALL(cudaFree(data));
    }
  }
  DeviceKind kind() const override { return GPU; }
  DeviceId id() const override { return {GPU, idx_}; }
  cudaStream_t stream() const { return stream_; }
};

inline DevPtr& gpu(size_t idx = 0) {
  static std::mutex mu;
  static std::vector<DevPtr> devs;
  std::lock_guard<std::mutex> g(mu);
  if (devs.size() <= idx) devs.resize(idx + 1);
  if (!devs[idx]) devs[idx] = std::make_shared<GpuDevice>(idx);
  return devs[idx];
}

inline int gpus() {
  int n = 0;
  return cudaGetDeviceCount(&n) == cudaSuccess ? n : 0;
}

class PreallocGpuDevice : public Device {
  size_t idx_, size_, used_ = 0;
  char* storage_ = nullptr;

 public:
  PreallocGpuDevice(size_t idx, size_t bytes) : idx_(idx), size_(bytes) {
    GINN_CUDA_CALL(cudaSetDevice(static_cast<int>(idx_)));
    GINN_CUDA_CALL(cudaMalloc(reinterpret_cast<void**>(&storage_), bytes));
  }
  ~PreallocGpuDevice() override { cudaFree(storage_); }
  void* alloc(size_t bytes) override {
    GINN_ASSERT(used_ + bytes <= size_, "Not enough memory on PreallocGpuDevice!");
    void* p = storage_ + used_;  // no alignment padding: byte accounting stays exact
    used_ += bytes;
    return p;
  }
  void* realloc(void*, size_t bytes) override { return alloc(bytes); }
  void free(void*) override {}
  void clear() { used_ = 0; }
  size_t used() const { return used_; }
  size_t size() const { return size_; }
  DeviceKind kind() const override { return GPU; }
  DeviceId id() const override { return {GPU, idx_}; }
  short precedence() const override { return 1; }
};

inline std::shared_ptr<PreallocGpuDevice> PreallocGpu(size_t idx, size_t bytes) {
  return std::make_shared<PreallocGpuDevice>(idx, bytes);
}

// The stream products for tensors of `dev` are enqueued on.
inline cudaStream_t stream_of(const Device& dev) {
  GINN_ASSERT(dev.kind() == GPU);
  auto g = std::dynamic_pointer_cast<GpuDevice>(gpu(dev.id().idx));
  return g->stream();
}

inline void Device::copy(const Device& other, void* data, const void* other_data, size_t bytes) {
  if (bytes == 0) return;
  if (kind() == CPU && other.kind() == CPU) {
    std::memcpy(data, other_data, bytes);
    return;
  }
  // Any transfer that involves a GPU: order it after the work queued on that GPU's stream.
  const Device& g = kind() == GPU ? *this : other;
  GINN_CUDA_CALL(cudaSetDevice(static_cast<int>(g.id().idx)));
  GINN_CUDA_CALL(cudaMemcpyAsync(data, other_data, bytes, cudaMemcpyDefault, stream_of(g)));
  GINN_CUDA_CALL(cudaStreamSynchronize(stream_of(g)));
}

}  // namespace ginn
#endif
