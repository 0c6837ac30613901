// SoftmaxNode with ginn's forward/backward protocol (ginn/node/nlnode.h:66 with SoftmaxOp,
// ginn/nonlin.h:157-190): softmax over dimension 0, trailing dimensions folded into columns;
//   backward  in.grad += y (.) (dy - colsum(y (.) dy)).
// GPU devices only; one kernel of libginn_b200.so per pass (the reference's GPU branch sends a
// batched 1 x 1 product through gpu_batched_prod and then evaluates a broadcast expression).
#ifndef GINN_B200_HOST_NODE_NLNODE_H
#define GINN_B200_HOST_NODE_NLNODE_H

#include <ginn/node/data.h>
#include <ginn/prod.h>

namespace ginn {

template <typename Scalar = Real>
class SoftmaxNode : public BaseDataNode<Scalar> {
  NodePtr<Scalar> in_;

  void forward_() override {
    GINN_ASSERT(this->dev()->kind() == GPU, "ginn_b200 serves GPU devices only");
    auto& x = in_->value();
    this->value().resize(x.shape());
    internal::b200_check(ginn_b200_softmax_forward(
        internal::b200_device(this->dev()), stream_of(*this->dev()), internal::b200_dtype<Scalar>(),
        x.rows(), x.cols(), x.data(), x.rows(), this->value().data(), x.rows()));
  }
  void backward_() override {
    if (!in_->has_grad()) return;
    auto& y = this->value();
    internal::b200_check(ginn_b200_softmax_backward(
        internal::b200_device(this->dev()), stream_of(*this->dev()), internal::b200_dtype<Scalar>(),
        y.rows(), y.cols(), y.data(), y.rows(), this->grad().data(), y.rows(), in_->grad().data(),
        y.rows(), /*accumulate=*/1));
  }

 public:
  explicit SoftmaxNode(const NodePtr<Scalar>& in)
      : BaseDataNode<Scalar>(std::vector<BaseNodePtr>{in}), in_(in) {}
  std::string name() const override { return "Softmax"; }
};

template <typename Scalar>
auto Softmax(const NodePtr<Scalar>& in) {
  return make_ptr<SoftmaxNode<Scalar>>(in);
}

}  // namespace ginn
#endif
