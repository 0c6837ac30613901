// Tensor<Scalar>: column-major storage plus shape, the members ginn's product path relies on
// (ginn/tensor.h:76-86, 247-256, 268-324, 439-444).  No expression machinery: this layer only
// moves data and calls the GPU library.
#ifndef GINN_B200_HOST_TENSOR_H
#define GINN_B200_HOST_TENSOR_H

#include <initializer_list>
#include <vector>

#include <ginn_b200.h>

#include <ginn/dev.h>

namespace ginn {

inline float to_float(float x) { return x; }
inline float to_float(Half x) { return __half2float(x); }

template <typename ScalarType = Real>
class Tensor {
 public:
  using Scalar = ScalarType;

 private:
  DevPtr dev_;
  Shape shape_ = {0};
  Scalar* data_ = nullptr;
  bool owns_ = true;

  void release() {
    if (owns_ && data_) dev_->free(data_);
    data_ = nullptr;
  }

 public:
  Tensor(DevPtr dev = cpu()) : dev_(std::move(dev)) {}
  Tensor(DevPtr dev, const Shape& shape) : dev_(std::move(dev)) { resize(shape); }
  Tensor(DevPtr dev, const Shape& shape, const std::vector<Scalar>& column_major)
      : dev_(std::move(dev)) {
    resize(shape);
    set(column_major);
  }
  Tensor(const Tensor& o) : dev_(o.dev_) { *this = o; }
  Tensor(Tensor&& o) noexcept
      : dev_(o.dev_), shape_(o.shape_), data_(o.data_), owns_(o.owns_) {
    o.data_ = nullptr;
    o.shape_ = {0};
  }
  ~Tensor() { release(); }

  // Deep copy; keeps this tensor's device (ginn's assignment copies across devices).
  Tensor& operator=(const Tensor& o) {
    if (this == &o) return *this;
    resize(o.shape_);
    dev_->copy(*o.dev_, data_, o.data_, size() * sizeof(Scalar));
    return *this;
  }

  const DevPtr& dev() const { return dev_; }  // (by reference: a copy is two atomic operations)
  const Shape& shape() const { return shape_; }
  Scalar* data() { return data_; }
  const Scalar* data() const { return data_; }

  static Size size(const Shape& s) {
    Size n = 1;
    for (Size d : s) n *= d;
    return n;
  }
  Size size() const { return size(shape_); }

  // Shape with exactly `dim` entries: trailing dims multiplied into the last one, or padded with 1.
  static Shape reduce(const Shape& s, Size dim) {
    Shape out(s.begin(), s.begin() + std::min<size_t>(s.size(), dim));
    for (size_t i = dim; i < s.size(); ++i) out[dim - 1] *= s[i];
    while (static_cast<Size>(out.size()) < dim) out.push_back(1);
    return out;
  }
  Shape shape2() const { return reduce(shape_, 2); }
  // (computed in place: the host side of an autobatched graph asks these tens of thousands of
  // times per pass, and shape2() builds a vector)
  Size rows() const { return shape_.empty() ? 1 : shape_[0]; }
  Size cols() const {
    Size n = 1;
    for (size_t i = 1; i < shape_.size(); ++i) n *= shape_[i];
    return n;
  }

  // Reallocates only when the element count changes; GPU contents are then lost.
  void resize(const Shape& s) {
    GINN_ASSERT(owns_ || size(s) == size(), "cannot resize a mapped tensor");
    if (size(s) != size() || (data_ == nullptr && size(s) > 0)) {
      const Size n = size(s);
      if (data_ == nullptr) {
        data_ = n > 0 ? static_cast<Scalar*>(dev_->alloc(n * sizeof(Scalar))) : nullptr;
      } else if (n == 0) {
        release();
      } else {
        data_ = static_cast<Scalar*>(dev_->realloc(data_, n * sizeof(Scalar)));
      }
    }
    shape_ = s;
  }

  // Non-owning alias of (part of) another tensor.
  Tensor& map(Tensor& other, const Shape& s, Size offset = 0) {
    GINN_ASSERT(size(s) + offset <= other.size());
    release();
    dev_ = other.dev_;
    data_ = other.data_ + offset;
    shape_ = s;
    owns_ = false;
    return *this;
  }
  Tensor& map(Tensor& other) { return map(other, other.shape_); }
  bool is_mapped() const { return !owns_; }
  // Ends an alias: the tensor becomes an empty one that owns (nothing) again and can be resized.
  // No effect on a tensor that owns its memory.
  void unmap() {
    if (owns_) return;
    data_ = nullptr;
    shape_ = {0};
    owns_ = true;
  }
  Tensor reshaped(const Shape& s) {
    GINN_ASSERT(size(s) == size());
    Tensor t(dev_);
    t.map(*this, s);
    return t;
  }

  // Host <-> device helpers (values in column-major order).
  void set(const std::vector<Scalar>& v) {
    GINN_ASSERT(static_cast<Size>(v.size()) == size(), "set(): size mismatch");
    dev_->copy(*cpu(), data_, v.data(), v.size() * sizeof(Scalar));
  }
  // Rows written one after the other, as ginn's Values<2>({{...},{...}}) does.
  void set2(std::initializer_list<std::initializer_list<double>> rows_) {
    const Size r = rows_.size(), c = r ? rows_.begin()->size() : 0;
    resize({r, c});
    std::vector<Scalar> v(r * c);
    Size i = 0;
    for (auto& row : rows_) {
      Size j = 0;
      for (double x : row) v[i + (j++) * r] = Scalar(static_cast<float>(x));
      ++i;
    }
    set(v);
  }
  std::vector<Scalar> vector() const {
    std::vector<Scalar> v(size());
    cpu()->copy(*dev_, v.data(), data_, v.size() * sizeof(Scalar));
    return v;
  }
  void fill(Scalar value) {
    if (size() == 0) return;
    if (dev_->kind() == GPU) {  // on the device's stream, no host copy and no wait
      const int status = ginn_b200_fill(static_cast<int>(dev_->id().idx), stream_of(*dev_),
                                        sizeof(Scalar) == 4 ? GINN_B200_F32 : GINN_B200_F16, size(),
                                        data_, to_float(value));
      if (status != GINN_B200_OK) GINN_CUDA_THROW(ginn_b200_last_error());
    } else {
      set(std::vector<Scalar>(size(), value));
    }
  }
  void set_zero() {
    if (size() == 0) return;
    if (dev_->kind() == GPU) {
      GINN_CUDA_CALL(cudaSetDevice(static_cast<int>(dev_->id().idx)));
      GINN_CUDA_CALL(cudaMemsetAsync(data_, 0, size() * sizeof(Scalar), stream_of(*dev_)));
    } else {
      std::memset(data_, 0, size() * sizeof(Scalar));
    }
  }
  Tensor copy_to(const DevPtr& to) const {
    Tensor t(to, shape_);
    to->copy(*dev_, t.data_, data_, size() * sizeof(Scalar));
    return t;
  }
};

}  // namespace ginn
#endif
