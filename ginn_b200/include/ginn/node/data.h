// Storage nodes: BaseDataNode (value + gradient + has_grad flag) and the leaf DataNode with its
// factories (ginn/node/data.h:27-71 and the Data/Values/Random helpers used by ginn's tests).
#ifndef GINN_B200_HOST_NODE_DATA_H
#define GINN_B200_HOST_NODE_DATA_H

#include <random>

#include <ginn/node.h>

namespace ginn {

template <typename Scalar = Real>
class BaseDataNode : public Node<Scalar> {
 protected:
  Tensor<Scalar> value_, grad_;
  bool has_grad_ = true;

 public:
  BaseDataNode(DevPtr dev, const Shape& shape) : value_(dev, shape), grad_(dev) {}
  explicit BaseDataNode(const std::vector<BaseNodePtr>& ins)
      : Node<Scalar>(ins), value_(best_dev(ins)), grad_(best_dev(ins)) {
    has_grad_ = false;
    for (auto& in : ins) has_grad_ = has_grad_ || in->has_grad();
  }
  // Highest-precedence device among the inputs (a preallocated device wins), ginn/dev.h:350-359.
  static DevPtr best_dev(const std::vector<BaseNodePtr>& ins) {
    GINN_ASSERT(!ins.empty());
    DevPtr best = ins.front()->dev();
    for (auto& in : ins)
      if (in->dev()->precedence() > best->precedence()) best = in->dev();
    return best;
  }
  Tensor<Scalar>& value() override { return value_; }
  Tensor<Scalar>& grad() override { return grad_; }
  bool has_grad() const override { return has_grad_; }
  void set_has_grad(bool g) { has_grad_ = g; }
};

template <typename Scalar = Real>
class DataNode : public BaseDataNode<Scalar> {
 public:
  DataNode(DevPtr dev, const Shape& shape) : BaseDataNode<Scalar>(std::move(dev), shape) {
    this->forwarded = true;
  }
  void reset_forwarded() override {}  // leaves always hold their value
  std::string name() const override { return "Data"; }
};
template <typename Scalar = Real>
using DataPtr = Ptr<DataNode<Scalar>>;

template <typename Scalar = Real>
DataPtr<Scalar> Data(DevPtr dev, const Shape& shape) {
  return make_ptr<DataNode<Scalar>>(std::move(dev), shape);
}
template <typename Scalar = Real>
DataPtr<Scalar> FixedData(DevPtr dev, const Shape& shape) {
  auto n = Data<Scalar>(std::move(dev), shape);
  n->set_has_grad(false);
  return n;
}
// Matrix literal, rows written one after the other: Values<Real>(dev, {{1,2,3},{4,5,6}}).
template <typename Scalar = Real>
DataPtr<Scalar> Values(DevPtr dev, std::initializer_list<std::initializer_list<double>> rows) {
  auto n = Data<Scalar>(std::move(dev), {0, 0});
  n->value().set2(rows);
  return n;
}
// Uniform(-1, 1) entries from a seeded host generator.
template <typename Scalar = Real>
DataPtr<Scalar> Random(DevPtr dev, const Shape& shape, unsigned seed = 1234) {
  auto n = Data<Scalar>(std::move(dev), shape);
  std::mt19937 gen(seed);
  std::uniform_real_distribution<float> u(-1.f, 1.f);
  std::vector<Scalar> v(n->value().size());
  for (auto& x : v) x = Scalar(u(gen));
  n->value().set(v);
  return n;
}

}  // namespace ginn
#endif
