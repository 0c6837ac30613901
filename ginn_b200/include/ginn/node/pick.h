// PickNegLogSoftmaxNode with ginn's forward/backward protocol (ginn/node/pick.h:28-248):
//   forward   smax = column softmax of the input, value = -log(smax[index[j], j]), shape {1, cols}
//   backward  in.grad += (smax - onehot(index)) * grad, only if the input has_grad()
// GPU devices only: both passes are one kernel of libginn_b200.so each.
#ifndef GINN_B200_HOST_NODE_PICK_H
#define GINN_B200_HOST_NODE_PICK_H

#include <ginn/node/data.h>
#include <ginn/prod.h>

namespace ginn {

template <typename Scalar = Real>
class PickNegLogSoftmaxNode : public BaseDataNode<Scalar> {
  NodePtr<Scalar> in_;
  DataPtr<Int> index_;
  Tensor<Scalar> smax_;

  void forward_() override {
    GINN_ASSERT(this->dev()->kind() == GPU, "ginn_b200 serves GPU devices only");
    auto& x = in_->value();
    auto& index = index_->value();
    GINN_ASSERT(x.cols() == index.size(), "Index size does not match input columns! (" +
                                              std::to_string(index.size()) + "≠" +
                                              std::to_string(x.cols()));
    this->value().resize({1, x.cols()});
    GINN_ASSERT(smax_.dev()->kind() == GPU && x.dev()->kind() == GPU && index.dev()->kind() == GPU,
                "PickNegLogSoftmax needs its input, index and buffers on a GPU device");
    smax_.resize(x.shape());
    const int dev = static_cast<int>(this->dev()->id().idx);
    internal::b200_check(ginn_b200_pick_nll_forward(
        dev, stream_of(*this->dev()), internal::b200_dtype<Scalar>(), x.rows(), x.cols(), x.data(),
        x.rows(), index.data(), smax_.data(), x.rows(), this->value().data()));
  }

  void backward_() override {
    if (!in_->has_grad()) return;
    const int dev = static_cast<int>(this->dev()->id().idx);
    internal::b200_check(ginn_b200_pick_nll_backward(
        dev, stream_of(*this->dev()), internal::b200_dtype<Scalar>(), smax_.rows(), smax_.cols(),
        smax_.data(), smax_.rows(), index_->value().data(), this->grad().data(),
        in_->grad().data(), smax_.rows()));
  }

 public:
  PickNegLogSoftmaxNode(const NodePtr<Scalar>& in, const DataPtr<Int>& index)
      : BaseDataNode<Scalar>(std::vector<BaseNodePtr>{in, index}),
        in_(in),
        index_(index),
        smax_(this->value_.dev()) {  // a default-constructed Tensor would live on the CPU
    this->set_has_grad(in->has_grad());
  }
  PickNegLogSoftmaxNode(const NodePtr<Scalar>& in, const std::vector<Int>& index)
      : PickNegLogSoftmaxNode(in, make_index(in->dev(), index)) {}

  static DataPtr<Int> make_index(DevPtr dev, const std::vector<Int>& index) {
    auto n = Data<Int>(std::move(dev), {static_cast<Size>(index.size())});
    n->value().set(index);
    n->set_has_grad(false);
    return n;
  }
  const Tensor<Scalar>& softmax() const { return smax_; }
  std::string name() const override { return "PickNegLogSoftmax"; }
};

template <typename Scalar>
auto PickNegLogSoftmax(const NodePtr<Scalar>& in, const DataPtr<Int>& index) {
  return make_ptr<PickNegLogSoftmaxNode<Scalar>>(in, index);
}
template <typename Scalar>
auto PickNegLogSoftmax(const NodePtr<Scalar>& in, const std::vector<Int>& index) {
  return make_ptr<PickNegLogSoftmaxNode<Scalar>>(in, index);
}

}  // namespace ginn
#endif
