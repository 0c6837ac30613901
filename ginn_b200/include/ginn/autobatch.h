// Autobatch for the B200 back end.
//
// ginn's Autobatch (ginn/autobatch.h:57-202) rewrites the graph: every Affine becomes a sum of
// products plus a broadcast bias, products that share their left operand and their height are
// replaced by RowwiseCat -> Prod -> RowwiseUncat, and the new graph is evaluated node by node.
// Here the same grouping -- key (left operand, height) -- drives a level executor instead: the
// nodes keep their own value / gradient tensors, and each level is ONE grouped launch for the
// forward products, one for the right-operand gradients and one for the weight and bias
// gradients, reading and writing the nodes' tensors through column-pointer tables.  No
// concatenation copy, no bias broadcast, no Add node.
//
// Batched: ProdNode<Real> and AffineNode<Real> with the identity nonlinearity (ginn's rewrite is
// only valid for identity Affines, ginn/autobatch.h:30-38); an Affine with several (W, x) pairs
// contributes one product per pair, the later pairs accumulating onto the first.  Every other
// node runs through its own forward()/backward(), level by level, so results equal Graph's.
#ifndef GINN_B200_HOST_AUTOBATCH_H
#define GINN_B200_HOST_AUTOBATCH_H

#include <algorithm>
#include <map>
#include <unordered_map>

#include <ginn/node/affine.h>
#include <ginn/node/prod.h>

namespace ginn {

class BatchedGraph {
  // One product of a batchable node: out (+)= W * x, with the bias riding on the first product.
  struct Item {
    Node<Real>* out;
    Node<Real>* w;
    Node<Real>* x;
    Node<Real>* bias;  // only on pair 0 of an Affine
    int pair;          // index of the (W, x) pair inside its node
  };
  struct Level {
    std::vector<BaseNode*> plain;  // nodes that are not batched: run one by one
    std::vector<Item> items;
    std::vector<Node<Real>*> outs;  // batched nodes of this level
  };

  std::vector<BaseNodePtr> list_;
  std::vector<Level> levels_;
  DevPtr dev_;

  static bool batchable(BaseNode* n, std::vector<Item>& items) {
    if (auto p = dynamic_cast<ProdNode<Real>*>(n)) {
      items.push_back({p, p->lhs().get(), p->rhs().get(), nullptr, 0});
      return true;
    }
    if (auto a = dynamic_cast<AffineNode<Real>*>(n)) {
      if (!a->nonlin().is_identity()) return false;
      auto& ins = a->affine_ins();
      for (size_t i = 0; i + 1 < ins.size(); i += 2)
        items.push_back({a, ins[i].get(), ins[i + 1].get(), i == 0 ? ins.back().get() : nullptr,
                         static_cast<int>(i / 2)});
      return true;
    }
    return false;
  }

  void build() {
    std::unordered_map<BaseNode*, size_t> height;
    size_t max_h = 0;
    for (auto& n : list_) {  // list_ is topological: inputs come first
      size_t h = 0;
      for (auto& in : n->ins()) h = std::max(h, height.at(in.get()));
      height[n.get()] = h + 1;
      max_h = std::max(max_h, h + 1);
    }
    levels_.assign(max_h + 1, Level{});
    for (auto& n : list_) {
      Level& lv = levels_[height[n.get()]];
      if (n->dev()->kind() == GPU && batchable(n.get(), lv.items)) {
        lv.outs.push_back(dynamic_cast<Node<Real>*>(n.get()));
        if (!dev_) dev_ = n->dev();
      } else {
        lv.plain.push_back(n.get());
      }
    }
  }

  static Real* col(Tensor<Real>& t, Size j) { return t.data() + j * t.rows(); }

  // One grouped launch over `items` (all must be safe to run concurrently), grouped by
  // (W, bias): the library computes every group in the same launch.
  void launch(const std::vector<const Item*>& items, int mode, bool accumulate) {
    if (items.empty()) return;
    struct Tables {
      std::vector<const void*> x;
      std::vector<void*> y, dx;
    };
    std::map<std::pair<Node<Real>*, Node<Real>*>, Tables> groups;
    for (const Item* it : items) {
      Tables& t = groups[{it->w, it->bias}];
      Tensor<Real>& outv = mode == GINN_B200_GROUPED_FORWARD ? it->out->value() : it->out->grad();
      for (Size j = 0; j < it->x->value().cols(); ++j) {
        t.x.push_back(col(it->x->value(), j));
        t.y.push_back(col(outv, j));
        if (mode == GINN_B200_GROUPED_DX) t.dx.push_back(col(it->x->grad(), j));
      }
    }
    std::vector<ginn_b200_group> gs;
    for (auto& kv : groups) {
      Node<Real>* w = kv.first.first;
      Node<Real>* bias = kv.first.second;
      ginn_b200_group g{};
      g.w = w->value().data();
      g.ldw = w->value().rows();
      g.m = w->value().rows();
      g.k = w->value().cols();
      g.ncols = static_cast<int64_t>(kv.second.y.size());
      g.x_cols = kv.second.x.data();
      g.y_cols = kv.second.y.data();
      g.dx_cols = kv.second.dx.data();
      g.accumulate = accumulate ? 1 : 0;
      if (mode == GINN_B200_GROUPED_FORWARD) g.bias = bias ? bias->value().data() : nullptr;
      if (mode == GINN_B200_GROUPED_DW) {
        g.dw = w->grad().data();
        g.lddw = w->grad().rows();
        g.dbias = (bias && bias->has_grad()) ? bias->grad().data() : nullptr;
      }
      gs.push_back(g);
    }
    internal::b200_check(ginn_b200_grouped(internal::b200_device(dev_), stream_of(*dev_),
                                           GINN_B200_F32, mode, static_cast<int>(gs.size()),
                                           gs.data()));
  }

  void forward_level(Level& lv) {
    int max_pair = -1;
    for (auto& it : lv.items) max_pair = std::max(max_pair, it.pair);
    // Pair p of every node in one launch; later pairs accumulate onto the first.
    for (int p = 0; p <= max_pair; ++p) {
      std::vector<const Item*> wave;
      for (auto& it : lv.items)
        if (it.pair == p && !it.out->forwarded) wave.push_back(&it);
      launch(wave, GINN_B200_GROUPED_FORWARD, p > 0);
    }
  }

  void backward_level(Level& lv) {
    // dX: two products that feed the same x would both add into x.grad; such items go to
    // successive launches (wave = how many earlier items already write that x).
    std::unordered_map<Node<Real>*, int> seen;
    std::vector<std::vector<const Item*>> waves;
    std::vector<const Item*> dw_items, db_only;
    for (auto& it : lv.items) {
      if (!it.out->has_grad()) continue;
      if (it.x->has_grad()) {
        const size_t w = seen[it.x]++;
        if (waves.size() <= w) waves.resize(w + 1);
        waves[w].push_back(&it);
      }
      if (it.w->has_grad())
        dw_items.push_back(&it);
      else if (it.bias && it.bias->has_grad())
        db_only.push_back(&it);
    }
    for (auto& wv : waves) launch(wv, GINN_B200_GROUPED_DX, true);
    // dW: a launch may hold only one group per W (groups are keyed by (W, bias), and two groups
    // with the same W would both add into W.grad), so groups that differ only in their bias go
    // to successive launches.
    std::unordered_map<Node<Real>*, std::vector<Node<Real>*>> biases_of;
    std::vector<std::vector<const Item*>> dw_waves;
    for (const Item* it : dw_items) {
      auto& seen_bias = biases_of[it->w];
      size_t w = 0;
      while (w < seen_bias.size() && seen_bias[w] != it->bias) ++w;
      if (w == seen_bias.size()) seen_bias.push_back(it->bias);
      if (dw_waves.size() <= w) dw_waves.resize(w + 1);
      dw_waves[w].push_back(it);
    }
    for (auto& wv : dw_waves) launch(wv, GINN_B200_GROUPED_DW, true);
    GINN_ASSERT(db_only.empty(),
                "autobatch: a bias gradient without its weight gradient is not batched; use Graph");
  }

 public:
  explicit BatchedGraph(const Graph& g) : list_(g.nodes()) { build(); }

  BatchedGraph& forward() {
    for (auto& lv : levels_) {
      for (auto* n : lv.plain) n->forward();
      for (auto& it : lv.items) {
        if (it.out->forwarded || it.pair != 0) continue;
        GINN_ASSERT(it.w->value().shape().size() == 2);
        Shape s = it.x->value().shape();
        s[0] = it.w->value().rows();
        it.out->value().resize(s);
      }
      for (auto& it : lv.items)
        if (!it.out->forwarded) GINN_ASSERT(it.w->value().cols() == it.x->value().rows());
      forward_level(lv);
      for (auto* o : lv.outs) o->forwarded = true;
    }
    return *this;
  }

  BatchedGraph& backward(double loss_coeff = 1) {
    auto sink = dynamic_ptr_cast<Node<Real>>(list_.back());
    GINN_ASSERT(sink && sink->has_grad(), "autobatched graphs need a Real sink with a gradient");
    sink->grad().fill(static_cast<Real>(loss_coeff));
    for (auto lv = levels_.rbegin(); lv != levels_.rend(); ++lv) {
      // Plain nodes of a level only depend on lower levels, so the order inside a level is free.
      for (auto n = lv->plain.rbegin(); n != lv->plain.rend(); ++n) (*n)->backward();
      backward_level(*lv);
    }
    return *this;
  }
  BatchedGraph& reset_grad() {
    for (auto& e : list_) e->reset_grad();
    return *this;
  }
  BatchedGraph& reset_forwarded() {
    for (auto& e : list_) e->reset_forwarded();
    return *this;
  }
  const std::vector<BaseNodePtr>& nodes() const { return list_; }
  BaseNodePtr sink() const { return list_.back(); }
  size_t levels() const { return levels_.size(); }
};

inline BatchedGraph Autobatch(const Graph& g) { return BatchedGraph(g); }

}  // namespace ginn
#endif
