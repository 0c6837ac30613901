// Graph core, reduced to what drives the matrix-product nodes: BaseNode / Node<Scalar> /
// Graph with ginn's names and call protocol (ginn/node.h:113-273): forward() runs forward_()
// once, backward() runs backward_() when the node has a gradient, Graph walks a topological
// list, reset_grad() zero-fills every gradient, and all gradient writes accumulate.
#ifndef GINN_B200_HOST_NODE_H
#define GINN_B200_HOST_NODE_H

#include <memory>
#include <string>
#include <unordered_set>
#include <vector>

#include <ginn/tensor.h>

namespace ginn {

template <typename T>
using Ptr = std::shared_ptr<T>;
template <typename T, typename... Args>
Ptr<T> make_ptr(Args&&... args) {
  return std::make_shared<T>(std::forward<Args>(args)...);
}
template <typename To, typename From>
Ptr<To> dynamic_ptr_cast(const Ptr<From>& p) {
  return std::dynamic_pointer_cast<To>(p);
}

class BaseNode;
using BaseNodePtr = Ptr<BaseNode>;

class BaseNode {
 protected:
  std::vector<BaseNodePtr> ins_;
  virtual void forward_() {}
  virtual void backward_() {}

 public:
  bool forwarded = false;
  BaseNode() = default;
  explicit BaseNode(std::vector<BaseNodePtr> ins) : ins_(std::move(ins)) {}
  virtual ~BaseNode() = default;

  const std::vector<BaseNodePtr>& ins() const { return ins_; }
  const BaseNodePtr& in(size_t i = 0) const { return ins_.at(i); }

  virtual DevPtr dev() const = 0;
  virtual Shape shape() const = 0;
  Size rows() const { return Tensor<>::reduce(shape(), 2)[0]; }
  Size cols() const { return Tensor<>::reduce(shape(), 2)[1]; }

  void forward() {
    if (!forwarded) {
      forward_();
      forwarded = true;
    }
  }
  void backward() {
    if (has_grad()) backward_();
  }
  virtual bool has_grad() const { return false; }
  // What Autobatch may do with this node: 0 = run it on its own, otherwise one of the kinds
  // BatchedGraph merges per level (it then casts statically; no RTTI on the rewrite path).
  enum BatchKind { kPlain = 0, kProd = 1, kAffine = 2, kLstmCell = 3 };
  virtual int batch_kind() const { return kPlain; }
  // Scratch slot for graph passes (index of the node in the pass's own flat arrays).
  mutable int pass_index = -1;
  virtual void init_grad() {}
  virtual void reset_grad() {}
  virtual void reset_forwarded() { forwarded = false; }
  virtual std::string name() const = 0;
};

template <typename ScalarType = Real>
class Node : public BaseNode {
 public:
  using Scalar = ScalarType;
  using BaseNode::BaseNode;
  virtual Tensor<Scalar>& value() = 0;
  virtual Tensor<Scalar>& grad() = 0;
  DevPtr dev() const override { return const_cast<Node*>(this)->value().dev(); }
  Shape shape() const override { return const_cast<Node*>(this)->value().shape(); }
  void init_grad() override {
    GINN_ASSERT(forwarded, "Cannot init grad on non-forwarded nodes!");
    if (has_grad() && value().size() != grad().size()) grad().resize(value().shape());
  }
  void reset_grad() override {
    init_grad();
    if (has_grad()) grad().set_zero();
  }
};
template <typename Scalar = Real>
using NodePtr = Ptr<Node<Scalar>>;

class Graph {
  std::vector<BaseNodePtr> list_;

  void traverse(const BaseNodePtr& e, std::unordered_set<BaseNode*>& seen) {
    if (seen.count(e.get())) return;
    for (auto& in : e->ins()) traverse(in, seen);
    seen.insert(e.get());
    list_.push_back(e);
  }

 public:
  explicit Graph(const BaseNodePtr& sink) {
    std::unordered_set<BaseNode*> seen;
    traverse(sink, seen);
  }
  Graph& forward() {
    for (auto& e : list_) e->forward();
    return *this;
  }
  // Seeds the sink's gradient with `loss_coeff` and walks the list backwards.
  Graph& backward(double loss_coeff = 1) {
    if (auto s = dynamic_ptr_cast<Node<Real>>(list_.back())) {
      GINN_ASSERT(s->has_grad());
      s->grad().fill(static_cast<Real>(loss_coeff));
    } else if (auto h = dynamic_ptr_cast<Node<Half>>(list_.back())) {
      GINN_ASSERT(h->has_grad());
      h->grad().fill(__float2half(static_cast<float>(loss_coeff)));
    } else {
      GINN_THROW("Unexpected scalar type in sink node!");
    }
    for (auto e = list_.rbegin(); e != list_.rend(); ++e) (*e)->backward();
    return *this;
  }
  Graph& init_grad() {
    for (auto& e : list_) e->init_grad();
    return *this;
  }
  Graph& reset_grad() {
    for (auto& e : list_) e->reset_grad();
    return *this;
  }
  Graph& reset_forwarded() {
    for (auto& e : list_) e->reset_forwarded();
    return *this;
  }
  const std::vector<BaseNodePtr>& nodes() const { return list_; }
  BaseNodePtr sink() const { return list_.back(); }
};

}  // namespace ginn
#endif
