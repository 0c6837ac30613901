// LstmCellNode: the elementwise part of an LSTM step as ONE node.
//
// ginn composes a cell from CwiseProd, Tanh and Add nodes around four Affines
// (ginn/model/lstm.h:94-100).  With the four gate pre-activations produced by a single Affine
// (rows i | f | g | o of a 4H x n matrix) the rest of the step is one pass:
//   i, f, o = sigmoid, g = tanh;  c = f * c_prev + i * g;  h = o * tanh(c)
// value() is h; c is kept inside the node for the next step's cell.  The gate node's value is
// overwritten with the activations (the backward pass needs them, and an identity Affine does
// not need its own value).  No single reference counterpart: harness node of the autobatch
// benchmark and tests; Autobatch runs all cells of a level as one launch.
#ifndef GINN_B200_HOST_NODE_LSTMCELL_H
#define GINN_B200_HOST_NODE_LSTMCELL_H

#include <ginn/node/data.h>
#include <ginn/prod.h>

namespace ginn {

class LstmCellNode : public BaseDataNode<Real> {
  NodePtr<Real> gates_;
  Ptr<LstmCellNode> prev_;  // previous step's cell, or null at the start of a sequence
  Tensor<Real> c_, dc_;

  static std::vector<BaseNodePtr> ins_of(const NodePtr<Real>& g, const Ptr<LstmCellNode>& p) {
    std::vector<BaseNodePtr> v{g};
    if (p) v.push_back(p);
    return v;
  }
  // Column pointers of a contiguous rows x n tensor.
  static void cols(std::vector<const void*>& t, Tensor<Real>* x, Size n) {
    for (Size j = 0; j < n; ++j) t.push_back(x ? x->data() + j * x->rows() : nullptr);
  }

  void forward_() override {
    GINN_ASSERT(this->dev()->kind() == GPU, "ginn_b200 serves GPU devices only");
    prepare_forward();
    const Size n = value().cols();
    std::vector<const void*> t;
    cols(t, &gates_->value(), n);
    cols(t, prev_ ? &prev_->c_ : nullptr, n);
    cols(t, &c_, n);
    cols(t, &value(), n);
    internal::b200_check(ginn_b200_lstm_cells(internal::b200_device(this->dev()),
                                              stream_of(*this->dev()), 0, hidden(), n, t.data()));
  }
  void backward_() override {
    const Size n = value().cols();
    std::vector<const void*> t;
    cols(t, &gates_->value(), n);
    cols(t, &c_, n);
    cols(t, prev_ ? &prev_->c_ : nullptr, n);
    cols(t, &grad(), n);
    cols(t, &dc_, n);
    cols(t, &gates_->grad(), n);
    cols(t, prev_ ? &prev_->dc_ : nullptr, n);
    internal::b200_check(ginn_b200_lstm_cells(internal::b200_device(this->dev()),
                                              stream_of(*this->dev()), 1, hidden(), n, t.data()));
  }

 public:
  LstmCellNode(const NodePtr<Real>& gates, const Ptr<LstmCellNode>& prev = nullptr)
      : BaseDataNode<Real>(ins_of(gates, prev)), gates_(gates), prev_(prev), c_(this->value().dev()),
        dc_(this->value().dev()) {}

  Size hidden() const { return gates_->value().rows() / 4; }
  // Sizes h and c for the gates' current shape (what forward_() does before it computes).
  void prepare_forward() {
    GINN_ASSERT(gates_->value().rows() % 4 == 0, "gate matrix must have 4 * hidden rows");
    const Shape s{hidden(), gates_->value().cols()};
    GINN_ASSERT(!prev_ || prev_->c_.shape() == s, "previous cell has another shape");
    value().resize(s);
    c_.resize(s);
  }
  const NodePtr<Real>& gates() const { return gates_; }
  const Ptr<LstmCellNode>& prev() const { return prev_; }
  Tensor<Real>& c() { return c_; }
  Tensor<Real>& dc() { return dc_; }
  void init_grad() override {
    BaseDataNode<Real>::init_grad();
    if (has_grad() && dc_.size() != c_.size()) dc_.resize(c_.shape());
  }
  void reset_grad() override {
    BaseDataNode<Real>::reset_grad();
    if (has_grad()) dc_.set_zero();
  }
  int batch_kind() const override { return BaseNode::kLstmCell; }
  std::string name() const override { return "LstmCell"; }
};

inline Ptr<LstmCellNode> LstmCell(const NodePtr<Real>& gates, const Ptr<LstmCellNode>& prev = nullptr) {
  return make_ptr<LstmCellNode>(gates, prev);
}

}  // namespace ginn
#endif
