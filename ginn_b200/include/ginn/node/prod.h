// ProdNode and BatchedProdNode with ginn's forward/backward protocol (ginn/node/prod.h:22-169):
//   forward   C = A*B                      (per trailing-dimension batch for BatchedProd)
//   backward  dB += A^T*dC,  dA += dC*B^T  each only for inputs with has_grad()
// GPU devices only: the products go to libginn_b200.so through internal::gpu_prod.
#ifndef GINN_B200_HOST_NODE_PROD_H
#define GINN_B200_HOST_NODE_PROD_H

#include <ginn/node/data.h>
#include <ginn/prod.h>

namespace ginn {

template <typename Scalar = Real>
class ProdNode : public BaseDataNode<Scalar> {
  NodePtr<Scalar> a_, b_;

  void forward_() override {
    GINN_ASSERT(this->dev()->kind() == GPU, "ginn_b200 serves GPU devices only");
    this->value().resize({a_->value().rows(), b_->value().cols()});
    internal::gpu_prod(this->value(), a_->value(), b_->value());
  }
  void backward_() override {
    // db += a^T * d and da += d * b^T in one call: the library runs them side by side
    if (a_->has_grad() || b_->has_grad())
      internal::gpu_prod_backward(a_->has_grad() ? &a_->grad() : nullptr,
                                  b_->has_grad() ? &b_->grad() : nullptr, this->grad(),
                                  a_->value(), b_->value());
  }

 public:
  ProdNode(const NodePtr<Scalar>& a, const NodePtr<Scalar>& b)
      : BaseDataNode<Scalar>(std::vector<BaseNodePtr>{a, b}), a_(a), b_(b) {}
  const NodePtr<Scalar>& lhs() const { return a_; }
  const NodePtr<Scalar>& rhs() const { return b_; }
  int batch_kind() const override {
    return std::is_same<Scalar, Real>::value ? BaseNode::kProd : BaseNode::kPlain;
  }
  std::string name() const override { return "Prod"; }
};

template <typename Scalar = Real>
class BatchedProdNode : public BaseDataNode<Scalar> {
  NodePtr<Scalar> a_, b_;

  void forward_() override {
    GINN_ASSERT(this->dev()->kind() == GPU, "ginn_b200 serves GPU devices only");
    const Shape sa = a_->shape(), sb = b_->shape();
    GINN_ASSERT(sa.size() >= 3 && sb.size() >= 3, "BatchedProd expects at least rank 3 inputs!");
    GINN_ASSERT(sa[1] == sb[0], "Mismatching inner dimensions in BatchedProd!");
    GINN_ASSERT(sa.size() == sb.size(), "Mismatching batch dimensions in BatchedProd!");
    for (size_t i = 2; i < sa.size(); ++i)
      GINN_ASSERT(sa[i] == sb[i], "Mismatching batch dimensions in BatchedProd!");
    Shape s = sb;
    s[0] = sa[0];
    this->value().resize(s);
    internal::gpu_batched_prod(this->value(), a_->value(), b_->value());
  }
  void backward_() override {
    if (a_->has_grad() || b_->has_grad())
      internal::gpu_batched_prod_backward(a_->has_grad() ? &a_->grad() : nullptr,
                                          b_->has_grad() ? &b_->grad() : nullptr, this->grad(),
                                          a_->value(), b_->value());
  }

 public:
  BatchedProdNode(const NodePtr<Scalar>& a, const NodePtr<Scalar>& b)
      : BaseDataNode<Scalar>(std::vector<BaseNodePtr>{a, b}), a_(a), b_(b) {}
  std::string name() const override { return "BatchedProd"; }
};

template <typename NodeA, typename NodeB>
auto Prod(const Ptr<NodeA>& a, const Ptr<NodeB>& b) {
  using Scalar = typename NodeA::Scalar;
  return make_ptr<ProdNode<Scalar>>(NodePtr<Scalar>(a), NodePtr<Scalar>(b));
}
template <typename NodeA, typename NodeB>
auto BatchedProd(const Ptr<NodeA>& a, const Ptr<NodeB>& b) {
  using Scalar = typename NodeA::Scalar;
  return make_ptr<BatchedProdNode<Scalar>>(NodePtr<Scalar>(a), NodePtr<Scalar>(b));
}
template <typename NodeA, typename NodeB>
auto operator*(const Ptr<NodeA>& a, const Ptr<NodeB>& b) {
  return Prod(a, b);
}

}  // namespace ginn
#endif
