// AffineNode: value = f( sum_i A_i * B_i + bias ), inputs given as A_1, B_1, A_2, B_2, ..., bias
// (ginn/node/affine.h:28-246).  Forward and backward are one library call each: bias, the
// nonlinearity, its derivative and the bias gradient are fused into the products, so neither a
// pre-activation nor a d-pre-activation tensor is materialised.
#ifndef GINN_B200_HOST_NODE_AFFINE_H
#define GINN_B200_HOST_NODE_AFFINE_H

#include <ginn/node/data.h>
#include <ginn/nonlin.h>
#include <ginn/prod.h>

namespace ginn {

template <typename Scalar = Real>
class AffineNode : public BaseDataNode<Scalar> {
  std::vector<NodePtr<Scalar>> in_;
  std::unique_ptr<NonlinOp<Scalar>> nonlin_;
  Tensor<Scalar> dpreactiv_;  // Half with a nonlinearity: dY (.) f'(Y), as in ginn/node/affine.h:82

  size_t npairs() const { return (in_.size() - 1) / 2; }

  void forward_() override {
    GINN_ASSERT(this->dev()->kind() == GPU, "ginn_b200 serves GPU devices only");
    auto& a = in_[0]->value();
    auto& b = in_[1]->value();
    auto& bias = in_.back()->value();
    GINN_ASSERT(a.shape().size() == 2);
    GINN_ASSERT(npairs() <= 4, "ginn_b200 fuses at most four (A, B) pairs per Affine");
    Shape s = b.shape();  // output rank follows the right operand
    s[0] = a.rows();
    this->value().resize(s);
    ginn_b200_pair pairs[4];
    for (size_t p = 0; p < npairs(); ++p) {
      auto& ap = in_[2 * p]->value();
      auto& bp = in_[2 * p + 1]->value();
      GINN_ASSERT(ap.shape().size() == 2);
      GINN_ASSERT(ap.rows() == a.rows() && bp.cols() == b.cols() && ap.cols() == bp.rows());
      pairs[p] = {ap.data(), ap.rows(), bp.data(), bp.rows(), ap.cols()};
    }
    GINN_ASSERT(bias.size() == a.rows());
    internal::b200_check(ginn_b200_affine_forward(
        internal::b200_device(this->dev()), stream_of(*this->dev()),
        internal::b200_dtype<Scalar>(), static_cast<int>(npairs()), pairs, a.rows(), b.cols(),
        bias.data(), nonlin_->fused_act(), this->value().data(), this->value().rows()));
  }

  void backward_() override {
    ginn_b200_pair_grad g[4];
    for (size_t p = 0; p < npairs(); ++p) {
      auto &an = in_[2 * p], &bn = in_[2 * p + 1];
      auto &ap = an->value(), &bp = bn->value();
      g[p] = {ap.data(), ap.rows(), bp.data(), bp.rows(), ap.cols(),
              an->has_grad() ? an->grad().data() : nullptr, ap.rows(),
              bn->has_grad() ? bn->grad().data() : nullptr, bp.rows()};
    }
    auto& bias = in_.back();
    // Half Affines with a nonlinearity hand the library their own d-pre-activation tensor, as
    // the reference's node owns one; fp32 forms the derivative inside the operand split.
    void* scratch = nullptr;
    if (std::is_same<Scalar, Half>::value && !nonlin_->is_identity()) {
      dpreactiv_.resize(this->value().shape());
      scratch = dpreactiv_.data();
    }
    internal::b200_check(ginn_b200_affine_backward_scratch(
        internal::b200_device(this->dev()), stream_of(*this->dev()),
        internal::b200_dtype<Scalar>(), static_cast<int>(npairs()), g, this->value().rows(),
        this->value().cols(), this->grad().data(), this->grad().rows(), this->value().data(),
        this->value().rows(), nonlin_->fused_act(),
        bias->has_grad() ? bias->grad().data() : nullptr, scratch));
  }

  static std::vector<BaseNodePtr> base(const std::vector<NodePtr<Scalar>>& v) {
    return std::vector<BaseNodePtr>(v.begin(), v.end());
  }

 public:
  AffineNode(std::unique_ptr<NonlinOp<Scalar>> nonlin, const std::vector<NodePtr<Scalar>>& ins)
      : BaseDataNode<Scalar>(base(ins)), in_(ins), nonlin_(std::move(nonlin)),
        dpreactiv_(this->value().dev()) {
    GINN_ASSERT(ins.size() >= 3 && ins.size() % 2 == 1,
                "Affine expects pairs of (A, B) inputs followed by a bias");
  }
  explicit AffineNode(const std::vector<NodePtr<Scalar>>& ins)
      : AffineNode(std::make_unique<IdentityOp<Scalar>>(), ins) {}

  const std::vector<NodePtr<Scalar>>& affine_ins() const { return in_; }
  const NonlinOp<Scalar>& nonlin() const { return *nonlin_; }
  int batch_kind() const override {
    return std::is_same<Scalar, Real>::value ? BaseNode::kAffine : BaseNode::kPlain;
  }
  std::string name() const override { return "Affine"; }
};

namespace internal {
template <typename Scalar, typename... Ns>
std::vector<NodePtr<Scalar>> node_list(const Ns&... ns) {
  return {NodePtr<Scalar>(ns)...};
}
}  // namespace internal

// Affine(W, x, b), Affine(W, x, V, h, b), ...
template <typename First, typename... Rest>
auto Affine(const Ptr<First>& first, const Rest&... rest) {
  using Scalar = typename First::Scalar;
  return make_ptr<AffineNode<Scalar>>(internal::node_list<Scalar>(first, rest...));
}
// Affine<TanhOp>(W, x, b)
template <template <typename> class Op, typename First, typename... Rest>
auto Affine(const Ptr<First>& first, const Rest&... rest) {
  using Scalar = typename First::Scalar;
  return make_ptr<AffineNode<Scalar>>(std::make_unique<Op<Scalar>>(),
                                      internal::node_list<Scalar>(first, rest...));
}
// Affine(TanhOp<Real>(), W, x, b)
template <template <typename> class Op, typename Scalar, typename... Rest>
auto Affine(const Op<Scalar>& op, const Rest&... rest) {
  return make_ptr<AffineNode<Scalar>>(op.copy(), internal::node_list<Scalar>(rest...));
}

}  // namespace ginn
#endif
