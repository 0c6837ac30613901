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
// Batched: ProdNode<Real>; AffineNode<Real> with the identity or a fused nonlinearity (tanh,
// sigmoid, relu -- the reference leaves Affines with nonlinearities unbatched,
// ginn/autobatch.h:30-38): an Affine with several (W, x) pairs contributes one product per pair,
// the later pairs accumulating onto the first, the nonlinearity riding on the last; and
// LstmCellNode (all cells of a level in one launch).  Every other node runs through its own
// forward()/backward(), level by level, so results equal Graph's.
//
// Host cost (the part ginn pays per graph, ginn/autobatch.h:57-147 with an unordered_map and a
// dynamic_cast per node): heights live in a flat array indexed through BaseNode::pass_index,
// node kinds come from a virtual call, groups are formed by sorting a flat item array.  The
// launch descriptors of every level are prepared once (ginn_b200_level_create) and replayed by
// later forward()/backward() calls on the same BatchedGraph -- the schedule cache for graphs
// that are evaluated more than once; tensors must then stay in place (they do unless a node is
// resized to another element count).
#ifndef GINN_B200_HOST_AUTOBATCH_H
#define GINN_B200_HOST_AUTOBATCH_H

#include <algorithm>
#include <tuple>

#include <ginn/node/affine.h>
#include <ginn/node/lstmcell.h>
#include <ginn/node/prod.h>

namespace ginn {

class BatchedGraph {
  // One product of a batchable node: out (+)= W * x, with the bias riding on the first product
  // and the nonlinearity on the last.
  struct Item {
    Node<Real>* out;
    Node<Real>* w;
    Node<Real>* x;
    Node<Real>* bias;  // only on pair 0 of an Affine
    int pair;          // index of the (W, x) pair inside its node
    int act;           // the node's fused nonlinearity (ginn_b200_act)
    bool last;         // last pair of its node: the forward launch applies `act`
  };
  // One prepared library launch: the group array, the pointer tables it refers to, and the
  // handle of the resident copy.
  struct Launch {
    int mode = 0;
    std::vector<ginn_b200_group> groups;
    std::vector<std::vector<const void*>> tables;  // stable storage for the groups' tables
    ginn_b200_level* handle = nullptr;
  };
  struct Level {
    std::vector<BaseNode*> plain;  // nodes that are not batched: run one by one
    std::vector<Item> items;
    std::vector<Node<Real>*> outs;     // batched product nodes of this level
    std::vector<LstmCellNode*> cells;  // batched cells of this level
    std::vector<Launch> fwd, bwd;
    ginn_b200_level* cells_fwd = nullptr;
    ginn_b200_level* cells_bwd = nullptr;
    bool fwd_ready = false, bwd_ready = false;
  };

  std::vector<BaseNodePtr> list_;
  std::vector<Level> levels_;
  DevPtr dev_;
  // reset_grad: the gradient tensors as merged byte ranges (built on first use)
  std::vector<std::pair<char*, size_t>> zero_ranges_;
  bool zero_ready_ = false;

  void add_items(BaseNode* n, Level& lv) {
    if (n->batch_kind() == BaseNode::kProd) {
      auto p = static_cast<ProdNode<Real>*>(n);
      lv.items.push_back({p, p->lhs().get(), p->rhs().get(), nullptr, 0, GINN_B200_ACT_NONE, true});
      lv.outs.push_back(p);
    } else {
      auto a = static_cast<AffineNode<Real>*>(n);
      auto& ins = a->affine_ins();
      const int npairs = static_cast<int>((ins.size() - 1) / 2);
      for (int p = 0; p < npairs; ++p)
        lv.items.push_back({a, ins[2 * p].get(), ins[2 * p + 1].get(),
                            p == 0 ? ins.back().get() : nullptr, p, a->nonlin().fused_act(),
                            p + 1 == npairs});
      lv.outs.push_back(a);
    }
  }

  void build() {
    // list_ is topological (inputs first): heights in one pass over a flat array
    std::vector<int> height(list_.size(), 0);
    for (size_t i = 0; i < list_.size(); ++i) list_[i]->pass_index = static_cast<int>(i);
    int max_h = 0;
    for (size_t i = 0; i < list_.size(); ++i) {
      int h = 0;
      for (auto& in : list_[i]->ins()) h = std::max(h, height[in->pass_index]);
      height[i] = h + 1;
      max_h = std::max(max_h, h + 1);
    }
    levels_.clear();
    levels_.resize(max_h + 1);
    for (size_t i = 0; i < list_.size(); ++i) {
      BaseNode* n = list_[i].get();
      Level& lv = levels_[height[i]];
      const bool on_gpu = n->dev()->kind() == GPU;
      const int kind = on_gpu ? n->batch_kind() : BaseNode::kPlain;
      if (on_gpu && !dev_) dev_ = n->dev();
      if (kind == BaseNode::kProd || kind == BaseNode::kAffine) {
        add_items(n, lv);
      } else if (kind == BaseNode::kLstmCell) {
        lv.cells.push_back(static_cast<LstmCellNode*>(n));
      } else {
        lv.plain.push_back(n);
      }
    }
  }

  static Real* col(Tensor<Real>& t, Size j) { return t.data() + j * t.rows(); }

  // Prepares one grouped launch over `items` (all safe to run concurrently).  Items with the
  // same (W, bias, nonlinearity) form a group; the library computes all groups in one launch.
  void prepare(std::vector<Launch>& out, std::vector<const Item*> items, int mode, bool accumulate) {
    if (items.empty()) return;
    const bool fwd = mode == GINN_B200_GROUPED_FORWARD;
    auto key = [&](const Item* it) {
      const int act = fwd ? (it->last ? it->act : GINN_B200_ACT_NONE) : it->act;
      return std::make_tuple(static_cast<const void*>(it->w), static_cast<const void*>(it->bias), act);
    };
    std::stable_sort(items.begin(), items.end(),
                     [&](const Item* a, const Item* b) { return key(a) < key(b); });
    out.emplace_back();
    Launch& L = out.back();
    L.mode = mode;
    size_t ngroups = 0;
    for (size_t i = 0; i < items.size(); ++i)
      if (i == 0 || key(items[i]) != key(items[i - 1])) ++ngroups;
    L.tables.reserve(4 * ngroups);  // the groups keep pointers into these vectors
    for (size_t i = 0; i < items.size();) {
      size_t j = i;
      while (j < items.size() && key(items[j]) == key(items[i])) ++j;
      const Item* first = items[i];
      const int act = std::get<2>(key(first));
      L.tables.emplace_back();
      auto& tx = L.tables.back();
      L.tables.emplace_back();
      auto& ty = L.tables.back();
      L.tables.emplace_back();
      auto& tdx = L.tables.back();
      L.tables.emplace_back();
      auto& tout = L.tables.back();
      for (size_t q = i; q < j; ++q) {
        const Item* it = items[q];
        Tensor<Real>& outv = fwd ? it->out->value() : it->out->grad();
        for (Size c = 0; c < it->x->value().cols(); ++c) {
          tx.push_back(col(it->x->value(), c));
          ty.push_back(col(outv, c));
          if (mode == GINN_B200_GROUPED_DX) tdx.push_back(col(it->x->grad(), c));
          if (!fwd && act != GINN_B200_ACT_NONE) tout.push_back(col(it->out->value(), c));
        }
      }
      ginn_b200_group g{};
      g.w = first->w->value().data();
      g.ldw = first->w->value().rows();
      g.m = first->w->value().rows();
      g.k = first->w->value().cols();
      g.ncols = static_cast<int64_t>(ty.size());
      g.x_cols = tx.data();
      g.y_cols = const_cast<void* const*>(reinterpret_cast<const void* const*>(ty.data()));
      g.dx_cols = const_cast<void* const*>(reinterpret_cast<const void* const*>(tdx.data()));
      g.accumulate = accumulate ? 1 : 0;
      g.act = act;
      g.out_cols = tout.empty() ? nullptr : tout.data();
      if (fwd) g.bias = first->bias ? first->bias->value().data() : nullptr;
      if (mode == GINN_B200_GROUPED_DW) {
        g.dw = first->w->grad().data();
        g.lddw = first->w->grad().rows();
        g.dbias = (first->bias && first->bias->has_grad()) ? first->bias->grad().data() : nullptr;
      }
      L.groups.push_back(g);
      i = j;
    }
    internal::b200_check(ginn_b200_level_create(internal::b200_device(dev_), GINN_B200_F32, mode,
                                                static_cast<int>(L.groups.size()), L.groups.data(),
                                                &L.handle));
  }

  void run(std::vector<Launch>& ls) {
    for (auto& L : ls) internal::b200_check(ginn_b200_level_run(L.handle, stream_of(*dev_)));
  }

  void prepare_forward(Level& lv) {
    int max_pair = -1;
    for (auto& it : lv.items) max_pair = std::max(max_pair, it.pair);
    // Pair p of every node in one launch; later pairs accumulate onto the first.
    for (int p = 0; p <= max_pair; ++p) {
      std::vector<const Item*> wave;
      for (auto& it : lv.items)
        if (it.pair == p) wave.push_back(&it);
      prepare(lv.fwd, wave, GINN_B200_GROUPED_FORWARD, p > 0);
    }
    if (!lv.cells.empty()) {
      const Size n = static_cast<Size>(lv.cells.size());
      std::vector<const void*> t(4 * n);
      Size hidden = lv.cells[0]->hidden();
      for (Size j = 0; j < n; ++j) {
        LstmCellNode* c = lv.cells[j];
        GINN_ASSERT(c->hidden() == hidden && c->value().cols() == 1,
                    "autobatch: cells of a level must share their size and hold one column");
        t[j] = c->gates()->value().data();
        t[n + j] = c->prev() ? c->prev()->c().data() : nullptr;
        t[2 * n + j] = c->c().data();
        t[3 * n + j] = c->value().data();
      }
      internal::b200_check(ginn_b200_lstm_cells_level_create(internal::b200_device(dev_), 0, hidden,
                                                             n, t.data(), &lv.cells_fwd));
    }
    lv.fwd_ready = true;
  }

  void prepare_backward(Level& lv) {
    // dX: two products that feed the same x would both add into x.grad; such items go to
    // successive launches (wave = how many earlier items already write that x).  The count
    // lives in the x node's pass_index while this level is prepared.
    std::vector<std::vector<const Item*>> waves;
    std::vector<const Item*> dw_items;
    for (auto& it : lv.items) it.x->pass_index = 0;
    for (auto& it : lv.items) {
      if (!it.out->has_grad()) continue;
      if (it.x->has_grad()) {
        const size_t w = static_cast<size_t>(it.x->pass_index++);
        if (waves.size() <= w) waves.resize(w + 1);
        waves[w].push_back(&it);
      }
      if (it.w->has_grad())
        dw_items.push_back(&it);
      else
        GINN_ASSERT(!(it.bias && it.bias->has_grad()),
                    "autobatch: a bias gradient without its weight gradient is not batched; use Graph");
    }
    for (auto& wv : waves) prepare(lv.bwd, wv, GINN_B200_GROUPED_DX, true);
    // dW: a launch may hold only one group per W (two groups with the same W would both add
    // into W.grad), so groups that differ only in bias or nonlinearity go to successive launches.
    std::stable_sort(dw_items.begin(), dw_items.end(), [](const Item* a, const Item* b) {
      return std::make_tuple((const void*)a->w, (const void*)a->bias, a->act) <
             std::make_tuple((const void*)b->w, (const void*)b->bias, b->act);
    });
    std::vector<std::vector<const Item*>> dw_waves;
    size_t variant = 0;
    for (size_t i = 0; i < dw_items.size(); ++i) {
      if (i > 0) {
        const Item *a = dw_items[i - 1], *b = dw_items[i];
        if (a->w != b->w)
          variant = 0;
        else if (a->bias != b->bias || a->act != b->act)
          ++variant;
      }
      if (dw_waves.size() <= variant) dw_waves.resize(variant + 1);
      dw_waves[variant].push_back(dw_items[i]);
    }
    for (auto& wv : dw_waves) prepare(lv.bwd, wv, GINN_B200_GROUPED_DW, true);
    if (!lv.cells.empty()) {
      std::vector<LstmCellNode*> live;
      for (auto* c : lv.cells)
        if (c->has_grad()) live.push_back(c);
      const Size n = static_cast<Size>(live.size());
      if (n > 0) {
        std::vector<const void*> t(7 * n);
        for (Size j = 0; j < n; ++j) {
          LstmCellNode* c = live[j];
          GINN_ASSERT(c->gates()->has_grad(), "autobatch: a cell with a gradient needs gates with one");
          t[j] = c->gates()->value().data();
          t[n + j] = c->c().data();
          t[2 * n + j] = c->prev() ? c->prev()->c().data() : nullptr;
          t[3 * n + j] = c->grad().data();
          t[4 * n + j] = c->dc().data();
          t[5 * n + j] = c->gates()->grad().data();
          t[6 * n + j] = (c->prev() && c->prev()->has_grad()) ? c->prev()->dc().data() : nullptr;
        }
        internal::b200_check(ginn_b200_lstm_cells_level_create(
            internal::b200_device(dev_), 1, live[0]->hidden(), n, t.data(), &lv.cells_bwd));
      }
    }
    lv.bwd_ready = true;
  }

  void destroy() {
    for (auto& lv : levels_) {
      for (auto* ls : {&lv.fwd, &lv.bwd})
        for (auto& L : *ls)
          if (L.handle) ginn_b200_level_destroy(L.handle);
      if (lv.cells_fwd) ginn_b200_level_destroy(lv.cells_fwd);
      if (lv.cells_bwd) ginn_b200_level_destroy(lv.cells_bwd);
    }
    levels_.clear();
  }

 public:
  explicit BatchedGraph(const Graph& g) : list_(g.nodes()) { build(); }
  BatchedGraph(const BatchedGraph&) = delete;
  BatchedGraph& operator=(const BatchedGraph&) = delete;
  BatchedGraph(BatchedGraph&& o) noexcept
      : list_(std::move(o.list_)), levels_(std::move(o.levels_)), dev_(std::move(o.dev_)),
        zero_ranges_(std::move(o.zero_ranges_)), zero_ready_(o.zero_ready_) {
    o.levels_.clear();
  }
  ~BatchedGraph() { destroy(); }

  BatchedGraph& forward() {
    for (auto& lv : levels_) {
      for (auto* n : lv.plain) n->forward();
      bool todo = false;
      for (auto* o : lv.outs) todo = todo || !o->forwarded;
      for (auto* c : lv.cells) todo = todo || !c->forwarded;
      if (!todo) continue;
      if (!lv.fwd_ready) {
        for (auto& it : lv.items) {
          if (it.pair != 0) continue;
          GINN_ASSERT(it.w->value().shape().size() == 2);
          Shape s = it.x->value().shape();
          s[0] = it.w->value().rows();
          it.out->value().resize(s);
        }
        for (auto& it : lv.items) GINN_ASSERT(it.w->value().cols() == it.x->value().rows());
        for (auto* c : lv.cells) c->prepare_forward();
        prepare_forward(lv);
      }
      run(lv.fwd);
      if (lv.cells_fwd)
        internal::b200_check(ginn_b200_level_run(lv.cells_fwd, stream_of(*dev_)));
      for (auto* o : lv.outs) o->forwarded = true;
      for (auto* c : lv.cells) c->forwarded = true;
    }
    return *this;
  }

  BatchedGraph& backward(double loss_coeff = 1) {
    auto sink = dynamic_ptr_cast<Node<Real>>(list_.back());
    GINN_ASSERT(sink && sink->has_grad(), "autobatched graphs need a Real sink with a gradient");
    sink->grad().fill(static_cast<Real>(loss_coeff));
    for (auto lv = levels_.rbegin(); lv != levels_.rend(); ++lv) {
      // Nodes of a level only depend on lower levels, so the order inside a level is free.
      for (auto n = lv->plain.rbegin(); n != lv->plain.rend(); ++n) (*n)->backward();
      if (!lv->bwd_ready) prepare_backward(*lv);
      if (lv->cells_bwd)
        internal::b200_check(ginn_b200_level_run(lv->cells_bwd, stream_of(*dev_)));
      run(lv->bwd);
    }
    return *this;
  }

  // Zero-fills every gradient, as Graph::reset_grad does node by node (ginn/node.h:197-200,
  // 261-264) -- but gradients that sit back to back in memory (a bump allocator hands them out
  // that way) are cleared with one fill per contiguous range.
  BatchedGraph& reset_grad() {
    if (!zero_ready_) {
      for (auto& e : list_) e->init_grad();
      // (address, bytes, owner): ranges are merged only inside one preallocated device -- its
      // tensors are pieces of a single allocation; two cudaMalloc'ed tensors may be neighbours
      // in the address space and still not be one region a fill may cross.
      struct Range {
        char* p;
        size_t bytes;
        Device* owner;  // null: not mergeable
        bool operator<(const Range& o) const { return p < o.p; }
      };
      std::vector<Range> r;
      bool all_gpu = true;
      auto add = [&](Tensor<Real>& t) {
        if (t.size() == 0) return;
        Device* d = t.dev().get();
        r.push_back({reinterpret_cast<char*>(t.data()), t.size() * sizeof(Real),
                     d->precedence() > 0 ? d : nullptr});
      };
      for (auto& e : list_) {
        if (!e->has_grad()) continue;
        auto n = dynamic_cast<Node<Real>*>(e.get());
        if (!n || n->dev()->kind() != GPU) {
          all_gpu = false;
          break;
        }
        add(n->grad());
        if (e->batch_kind() == BaseNode::kLstmCell) add(static_cast<LstmCellNode*>(e.get())->dc());
      }
      if (!all_gpu) {  // mixed graph: leave it to the nodes
        for (auto& e : list_) e->reset_grad();
        return *this;
      }
      std::sort(r.begin(), r.end());
      zero_ranges_.clear();
      Device* last_owner = nullptr;
      for (auto& x : r) {
        if (!zero_ranges_.empty() && x.owner != nullptr && x.owner == last_owner &&
            zero_ranges_.back().first + zero_ranges_.back().second >= x.p) {
          char* end = std::max(zero_ranges_.back().first + zero_ranges_.back().second, x.p + x.bytes);
          zero_ranges_.back().second = static_cast<size_t>(end - zero_ranges_.back().first);
        } else {
          zero_ranges_.emplace_back(x.p, x.bytes);
        }
        last_owner = x.owner;
      }
      zero_ready_ = true;
    }
    if (dev_) {
      GINN_CUDA_CALL(cudaSetDevice(internal::b200_device(dev_)));
      for (auto& x : zero_ranges_)
        GINN_CUDA_CALL(cudaMemsetAsync(x.first, 0, x.second, stream_of(*dev_)));
    }
    return *this;
  }
  BatchedGraph& reset_forwarded() {
    for (auto& e : list_) e->reset_forwarded();
    return *this;
  }
  const std::vector<BaseNodePtr>& nodes() const { return list_; }
  BaseNodePtr sink() const { return list_.back(); }
  size_t levels() const { return levels_.size(); }
  // Number of library launches a forward + backward pass makes (after preparation).
  size_t launches() const {
    size_t n = 0;
    for (auto& lv : levels_)
      n += lv.fwd.size() + lv.bwd.size() + (lv.cells_fwd ? 1 : 0) + (lv.cells_bwd ? 1 : 0);
    return n;
  }
};

inline BatchedGraph Autobatch(const Graph& g) { return BatchedGraph(g); }

}  // namespace ginn
#endif
