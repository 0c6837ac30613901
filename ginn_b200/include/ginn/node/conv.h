// Conv2dNode: 2-d convolution with SAME padding (ginn/node/conv.h:22-81).
//   input   (channels, rows, cols, others...)   trailing dimensions fold into the batch
//   filters (filters, channels, kernel rows, kernel cols)
//   value   (filters, ceil(rows / row_stride), ceil(cols / col_stride), others...)
// The reference contracts Eigen image patches with the reshaped filters; here the patch matrix
// is written once into a scratch tensor on the node's device and the contraction runs on the
// library's tensor-core products (ginn_b200_conv2d_forward / _backward).
#ifndef GINN_B200_HOST_NODE_CONV_H
#define GINN_B200_HOST_NODE_CONV_H

#include <ginn/node/data.h>
#include <ginn/prod.h>

namespace ginn {

template <typename Scalar = Real>
class Conv2dNode : public BaseDataNode<Scalar> {
  NodePtr<Scalar> in_, filter_;
  size_t row_stride_ = 1, col_stride_ = 1;
  Tensor<Scalar> patches_;  // scratch: (channels * krows * kcols) x (out_rows * out_cols * batch)

  static Size dim(Size len, size_t stride) { return (len + stride - 1) / stride; }

  void* workspace(const Shape& s, const Shape& f) {
    const size_t bytes = ginn_b200_conv2d_workspace(internal::b200_dtype<Scalar>(), s[0], s[1], s[2],
                                                    s[3], f[0], f[2], f[3], row_stride_, col_stride_);
    const Size n = static_cast<Size>((bytes + sizeof(Scalar) - 1) / sizeof(Scalar));
    if (patches_.size() != n) patches_.resize({n});
    return patches_.data();
  }

  void forward_() override {
    GINN_ASSERT(this->dev()->kind() == GPU, "ginn_b200 serves GPU devices only");
    const Shape s = Tensor<Scalar>::reduce(in_->shape(), 4), f = filter_->shape();
    GINN_ASSERT(f.size() == 4, "Conv2d expects rank-4 filters!");
    GINN_ASSERT(f[1] == s[0], "Mismatching channel counts in Conv2d!");
    Shape out = in_->shape();
    while (out.size() < 4) out.push_back(1);
    out[0] = f[0];
    out[1] = dim(s[1], row_stride_);
    out[2] = dim(s[2], col_stride_);
    this->value().resize(out);
    internal::b200_check(ginn_b200_conv2d_forward(
        internal::b200_device(this->dev()), stream_of(*this->dev()), internal::b200_dtype<Scalar>(),
        s[0], s[1], s[2], s[3], f[0], f[2], f[3], row_stride_, col_stride_, in_->value().data(),
        filter_->value().data(), this->value().data(), workspace(s, f)));
  }

  void backward_() override {
    const Shape s = Tensor<Scalar>::reduce(in_->shape(), 4), f = filter_->shape();
    internal::b200_check(ginn_b200_conv2d_backward(
        internal::b200_device(this->dev()), stream_of(*this->dev()), internal::b200_dtype<Scalar>(),
        s[0], s[1], s[2], s[3], f[0], f[2], f[3], row_stride_, col_stride_, in_->value().data(),
        filter_->value().data(), this->grad().data(),
        in_->has_grad() ? in_->grad().data() : nullptr,
        filter_->has_grad() ? filter_->grad().data() : nullptr, workspace(s, f)));
  }

 public:
  Conv2dNode(const NodePtr<Scalar>& input, const NodePtr<Scalar>& filters, size_t row_stride = 1,
             size_t col_stride = 1)
      : BaseDataNode<Scalar>(std::vector<BaseNodePtr>{input, filters}), in_(input), filter_(filters),
        row_stride_(row_stride), col_stride_(col_stride), patches_(this->value().dev()) {}
  std::string name() const override { return "Conv2d"; }
};

template <typename In, typename Filt>
auto Conv2d(const Ptr<In>& input, const Ptr<Filt>& filters, size_t row_stride = 1,
            size_t col_stride = 1) {
  using Scalar = typename In::Scalar;
  return make_ptr<Conv2dNode<Scalar>>(NodePtr<Scalar>(input), NodePtr<Scalar>(filters), row_stride,
                                      col_stride);
}

}  // namespace ginn
#endif
