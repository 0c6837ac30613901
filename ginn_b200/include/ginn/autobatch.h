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

#include <memory>
#ifdef GINN_AUTOBATCH_TIMES
#include <chrono>
#include <cstdio>
#endif
#include <algorithm>
#include <tuple>

#include <ginn/node/affine.h>
#include <ginn/node/lstmcell.h>
#include <ginn/node/prod.h>

namespace ginn {

#ifdef GINN_AUTOBATCH_TIMES  // host-time breakdown of the preparation (bench builds only)
struct AbTimes {
  double t[8] = {0};
  ~AbTimes() {
    std::fprintf(stderr, "autobatch host ms: size %.2f build_launch %.2f level_create %.2f cells_create %.2f "
                 "grad_prep %.2f\n", t[0], t[1], t[2], t[3], t[4]);
  }
};
inline AbTimes& ab_times() { static AbTimes x; return x; }
struct AbScope {
  int i;
  std::chrono::steady_clock::time_point t0 = std::chrono::steady_clock::now();
  explicit AbScope(int i_) : i(i_) {}
  ~AbScope() {
    ab_times().t[i] += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
  }
};
#define GINN_AB_TIME(i) AbScope ab_scope_##i(i)
#else
#define GINN_AB_TIME(i) do { } while (0)
#endif

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
    bool hoisted;      // runs in the launches of hoisted_ instead of its level's (see build())
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
    bool fwd_ready = false, bwd_ready = false, sized = false;
    cudaEvent_t ready = nullptr;  // the level's output gradients are final (run_backward)
    // Storage the level's batched nodes are moved into (see place()), and the tensors that alias
    // it: they are detached again (left empty) when the BatchedGraph goes, since the storage goes
    // with it -- copy out what should outlive the BatchedGraph.
    std::vector<std::unique_ptr<Tensor<Real>>> slabs;
    std::vector<Tensor<Real>*> placed;
  };

  std::vector<BaseNodePtr> list_;
  std::vector<Level> levels_;
  Level hoisted_;  // launches over the hoisted items of all levels (items stay in their levels)
  bool sized_ = false, hoist_ = false;
  cudaGraphExec_t pass_exec_ = nullptr;  // capture_pass()
  cudaStream_t side_ = nullptr;          // weight-gradient launches (run_backward)
  cudaEvent_t join_ = nullptr;
  bool side_used_ = false;

  void release_capture() {
    if (pass_exec_) cudaGraphExecDestroy(pass_exec_);
    pass_exec_ = nullptr;
  }
  DevPtr dev_;
  // reset_grad: the gradient tensors as merged byte ranges (built on first use)
  std::vector<std::pair<char*, size_t>> zero_ranges_;
  bool zero_ready_ = false;

  void add_items(BaseNode* n, Level& lv) {
    if (n->batch_kind() == BaseNode::kProd) {
      auto p = static_cast<ProdNode<Real>*>(n);
      lv.items.push_back({p, p->lhs().get(), p->rhs().get(), nullptr, 0, GINN_B200_ACT_NONE, true, false});
      lv.outs.push_back(p);
    } else {
      auto a = static_cast<AffineNode<Real>*>(n);
      auto& ins = a->affine_ins();
      const int npairs = static_cast<int>((ins.size() - 1) / 2);
      for (int p = 0; p < npairs; ++p)
        lv.items.push_back({a, ins[2 * p].get(), ins[2 * p + 1].get(),
                            p == 0 ? ins.back().get() : nullptr, p, a->nonlin().fused_act(),
                            p + 1 == npairs,
                            // The first product of a multi-pair Affine on a graph input that
                            // needs no gradient (the input projection W_x x_t of a recurrent
                            // step) depends on nothing the graph computes: all of them, from every
                            // level, run as one launch before the first level, and their weight
                            // gradients as one launch after the last.
                            p == 0 && npairs > 1 && ins[1]->ins().empty() && !ins[1]->has_grad()});
      lv.outs.push_back(a);
    }
  }

  static int kind_of(BaseNode* n) {
    return n->dev()->kind() == GPU ? n->batch_kind() : BaseNode::kPlain;
  }

  void build() {
    // list_ is topological (inputs first): heights in one pass over a flat array
    const size_t N = list_.size();
    std::vector<int> height(N, 0);
    for (size_t i = 0; i < N; ++i) list_[i]->pass_index = static_cast<int>(i);
    int max_h = 0;
    for (size_t i = 0; i < N; ++i) {
      int h = 0;
      for (auto& in : list_[i]->ins()) h = std::max(h, height[in->pass_index]);
      height[i] = h + 1;
      max_h = std::max(max_h, h + 1);
    }
    // reach[i]: the highest level a chain of batched nodes starting at node i gets to.  Inside a
    // level the batched nodes are ordered by it (longest-lived first, then by position in the
    // graph), the same rule on every level: in a recurrence over sequences of different lengths
    // the nodes a level hands on to the next then form a prefix of the level, in the next
    // level's own order -- so once rehome() has laid a level's tensors out back to back in that
    // order, both the outputs and the recurrent inputs of every level are equally spaced
    // columns and the library runs the level as plain TMA-fed products instead of following
    // pointer tables.
    std::vector<int> kind(N);
    for (size_t i = 0; i < N; ++i) kind[i] = kind_of(list_[i].get());
    std::vector<int> reach(height);
    for (size_t i = N; i-- > 0;) {
      if (kind[i] == BaseNode::kPlain) continue;
      for (auto& in : list_[i]->ins())
        reach[in->pass_index] = std::max(reach[in->pass_index], reach[i]);
    }
    std::vector<size_t> order(N);
    for (size_t i = 0; i < N; ++i) order[i] = i;
    // (level, plain nodes first, longest reach first); the sort is stable, so nodes that tie
    // keep their order in the graph
    std::vector<int> rank(N);
    for (size_t i = 0; i < N; ++i)
      rank[i] = kind[i] == BaseNode::kPlain ? -1 : static_cast<int>(N) - reach[i];
    std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) {
      if (height[a] != height[b]) return height[a] < height[b];
      return rank[a] < rank[b];
    });
    levels_.clear();
    levels_.resize(max_h + 1);
    for (size_t i : order) {
      BaseNode* n = list_[i].get();
      Level& lv = levels_[height[i]];
      const int k = kind[i];
      if (!dev_ && n->dev()->kind() == GPU) dev_ = n->dev();
      if (k == BaseNode::kProd || k == BaseNode::kAffine) {
        add_items(n, lv);
      } else if (k == BaseNode::kLstmCell) {
        lv.cells.push_back(static_cast<LstmCellNode*>(n));
      } else {
        lv.plain.push_back(n);
      }
    }
  }

  // Gives the tensors `ts` the shapes `shapes` in ONE allocation, back to back in the given
  // order (what they held is dropped: values are about to be computed, gradients about to be
  // zeroed).  Tensors of one shape on one device only; otherwise each is resized on its own.
  // The reference's Autobatch gives its batched nodes the same layout: their values are column
  // views (RowwiseUncat) of one merged result.
  void place(Level& lv, const std::vector<Tensor<Real>*>& ts, const std::vector<Shape>& shapes) {
    if (ts.empty()) return;
    bool same = ts.size() > 1 && Tensor<Real>::size(shapes[0]) > 0;
    for (size_t i = 1; i < ts.size() && same; ++i)
      same = shapes[i] == shapes[0] && ts[i]->dev() == ts[0]->dev();
    if (!same) {
      for (size_t i = 0; i < ts.size(); ++i) ts[i]->resize(shapes[i]);
      return;
    }
    const Size n = Tensor<Real>::size(shapes[0]);
    // A bump allocator hands out unaligned pointers (ginn/dev.h:237-245); three spare elements
    // let the run start on a 16-byte boundary, which the TMA-fed kernels need.
    lv.slabs.emplace_back(new Tensor<Real>(ts[0]->dev(), Shape{n * static_cast<Size>(ts.size()) + 3}));
    Tensor<Real>& slab = *lv.slabs.back();
    Size off = static_cast<Size>(((16 - (reinterpret_cast<uintptr_t>(slab.data()) & 15u)) & 15u) / sizeof(Real));
    for (auto* t : ts) {
      t->map(slab, shapes[0], off);
      lv.placed.push_back(t);
      off += n;
    }
  }

  static Real* col(Tensor<Real>& t, Size j) { return t.data() + j * t.rows(); }

  // Builds the groups and pointer tables of one grouped launch over `items` (all safe to run
  // concurrently).  Items with the same (W, bias, nonlinearity) form a group; `first_of[g]` is
  // the index (into the sorted `items`) of group g's first item.
  Launch build_launch(std::vector<const Item*>& items, int mode, bool accumulate,
                      std::vector<size_t>* first_of) {
    GINN_AB_TIME(1);
    const bool fwd = mode == GINN_B200_GROUPED_FORWARD;
    auto key = [&](const Item* it) {
      const int act = fwd ? (it->last ? it->act : GINN_B200_ACT_NONE) : it->act;
      return std::make_tuple(static_cast<const void*>(it->w), static_cast<const void*>(it->bias), act);
    };
    bool one_key = true;  // the common case (one W per level): nothing to sort
    for (size_t i = 1; i < items.size() && one_key; ++i) one_key = key(items[i]) == key(items[0]);
    if (!one_key)
      std::stable_sort(items.begin(), items.end(),
                       [&](const Item* a, const Item* b) { return key(a) < key(b); });
    Launch L;
    L.mode = mode;
    size_t ngroups = 0;
    for (size_t i = 0; i < items.size(); ++i)
      if (i == 0 || key(items[i]) != key(items[i - 1])) ++ngroups;
    L.tables.reserve(4 * ngroups);  // the groups keep pointers into these vectors
    for (size_t i = 0; i < items.size();) {
      size_t j = i;
      while (j < items.size() && key(items[j]) == key(items[i])) ++j;
      if (first_of) first_of->push_back(i);
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
      tx.reserve(j - i);
      ty.reserve(j - i);
      if (mode == GINN_B200_GROUPED_DX) tdx.reserve(j - i);
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
    return L;
  }

  void create(std::vector<Launch>& out, Launch&& L) {
    GINN_AB_TIME(2);
    out.push_back(std::move(L));  // moving keeps the tables' storage where the groups point
    Launch& X = out.back();
    internal::b200_check(ginn_b200_level_create(internal::b200_device(dev_), GINN_B200_F32, X.mode,
                                                static_cast<int>(X.groups.size()), X.groups.data(),
                                                &X.handle));
  }

  // Prepares the launch (or two) over `items`.  Groups whose column tables are equally spaced
  // run as plain products on the TMA-fed kernel when their launch holds nothing else (the library
  // decides per launch), so they are kept apart from groups that need their tables.
  void prepare(std::vector<Launch>& out, std::vector<const Item*> items, int mode, bool accumulate) {
    if (items.empty()) return;
    std::vector<size_t> first_of;
    Launch L = build_launch(items, mode, accumulate, &first_of);
    size_t nplain = 0;
    for (auto& g : L.groups) nplain += strided(g, mode) ? 1 : 0;
    if (nplain == 0 || nplain == L.groups.size()) {
      create(out, std::move(L));
      return;
    }
    std::vector<const Item*> plain_items, table_items;
    for (size_t g = 0; g < L.groups.size(); ++g) {
      const size_t end = g + 1 < first_of.size() ? first_of[g + 1] : items.size();
      auto& dst = strided(L.groups[g], mode) ? plain_items : table_items;
      dst.insert(dst.end(), items.begin() + first_of[g], items.begin() + end);
    }
    create(out, build_launch(plain_items, mode, accumulate, nullptr));
    create(out, build_launch(table_items, mode, accumulate, nullptr));
  }

  static bool equally_spaced(const void* const* t, int64_t n, int64_t rows) {
    if (t == nullptr) return false;
    if (n <= 1) return true;
    const char* p0 = static_cast<const char*>(t[0]);
    const long long step = static_cast<const char*>(t[1]) - p0;
    if (step < rows * static_cast<long long>(sizeof(Real))) return false;
    for (int64_t j = 2; j < n; ++j)
      if (static_cast<const char*>(t[j]) - p0 != step * j) return false;
    return true;
  }
  // Mirrors the library's test for a table-free group.
  static bool strided(const ginn_b200_group& g, int mode) {
    auto y = reinterpret_cast<const void* const*>(g.y_cols);
    if (mode == GINN_B200_GROUPED_FORWARD)
      return equally_spaced(g.x_cols, g.ncols, g.k) && equally_spaced(y, g.ncols, g.m);
    if (mode == GINN_B200_GROUPED_DX)
      return equally_spaced(y, g.ncols, g.m) &&
             equally_spaced(reinterpret_cast<const void* const*>(g.dx_cols), g.ncols, g.k);
    return equally_spaced(y, g.ncols, g.m) && equally_spaced(g.x_cols, g.ncols, g.k);
  }

  void run(std::vector<Launch>& ls) {
    for (auto& L : ls) internal::b200_check(ginn_b200_level_run(L.handle, stream_of(*dev_)));
  }

  // Backward launches of a level.  Nothing in the pass waits for a weight gradient before its
  // end, so those launches go to a second stream, off the chain cell update -> input gradient ->
  // next level (they wait for `ready`, recorded once the level's output gradients are final,
  // and keep their own order, which serialises the additions into W.grad).
  void run_backward(std::vector<Launch>& ls, cudaEvent_t ready) {
    cudaStream_t main = stream_of(*dev_);
    bool forked = false;
    for (auto& L : ls) {
      cudaStream_t st = main;
      if (L.mode == GINN_B200_GROUPED_DW) {
        if (!forked) {
          GINN_CUDA_CALL(cudaEventRecord(ready, main));
          GINN_CUDA_CALL(cudaStreamWaitEvent(side(), ready, 0));
          forked = true;
        }
        st = side_;
      }
      internal::b200_check(ginn_b200_level_run(L.handle, st));
    }
    side_used_ = side_used_ || forked;
  }
  cudaStream_t side() {
    if (side_ == nullptr) {
      GINN_CUDA_CALL(cudaSetDevice(internal::b200_device(dev_)));
      GINN_CUDA_CALL(cudaStreamCreateWithFlags(&side_, cudaStreamNonBlocking));
      GINN_CUDA_CALL(cudaEventCreateWithFlags(&join_, cudaEventDisableTiming));
    }
    return side_;
  }
  cudaEvent_t event_of(Level& lv) {
    if (lv.ready == nullptr) GINN_CUDA_CALL(cudaEventCreateWithFlags(&lv.ready, cudaEventDisableTiming));
    return lv.ready;
  }

  void prepare_forward(Level& lv) {
    int max_pair = -1;
    for (auto& it : lv.items) max_pair = std::max(max_pair, it.pair);
    // Pair p of every node in one launch; later pairs accumulate onto the first.
    for (int p = 0; p <= max_pair; ++p) {
      std::vector<const Item*> wave;
      for (auto& it : lv.items)
        if (it.pair == p && !it.hoisted) wave.push_back(&it);
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
      GINN_AB_TIME(3);
      internal::b200_check(ginn_b200_lstm_cells_level_create(internal::b200_device(dev_), 0, hidden,
                                                             n, t.data(), &lv.cells_fwd));
    }
    lv.fwd_ready = true;
  }

  // dW launches: one may hold only one group per W (two groups with the same W would both add
  // into W.grad), so groups that differ only in bias or nonlinearity go to successive launches.
  void prepare_dw(std::vector<Launch>& out, std::vector<const Item*> dw_items) {
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
    for (auto& wv : dw_waves) prepare(out, wv, GINN_B200_GROUPED_DW, true);
  }

  // Gives the level's batched nodes their shapes and their place in the level's storage.
  void size_level(Level& lv) {
    GINN_AB_TIME(0);
    std::vector<Tensor<Real>*> v, h, cc;
    std::vector<Shape> vs, hs;
    for (auto& it : lv.items) {
      GINN_ASSERT(it.w->value().cols() == it.x->value().rows());
      if (it.pair != 0) continue;
      GINN_ASSERT(it.w->value().shape().size() == 2);
      Shape s = it.x->value().shape();
      s[0] = it.w->value().rows();
      v.push_back(&it.out->value());
      vs.push_back(s);
    }
    place(lv, v, vs);
    for (auto* c : lv.cells) {
      Tensor<Real>& g = c->gates()->value();
      GINN_ASSERT(g.rows() % 4 == 0, "gate matrix must have 4 * hidden rows");
      h.push_back(&c->value());
      cc.push_back(&c->c());
      hs.push_back(Shape{g.rows() / 4, g.cols()});  // as LstmCellNode::prepare_forward shapes them
    }
    place(lv, h, hs);
    place(lv, cc, hs);
    for (auto* c : lv.cells) c->prepare_forward();  // its own checks; the sizes already fit
    lv.sized = true;
  }

  // First forward pass: decides whether the hoisted items can run ahead of the levels.  They
  // write into tensors of every level, so every level must get its shapes and storage before
  // anything runs -- possible when no batched node reads a node that only sizes its value while
  // it computes (a plain node of the graph); otherwise nothing is hoisted.
  void decide_hoist() {
    bool any = false;
    for (auto& lv : levels_)
      for (auto& it : lv.items) any = any || it.hoisted;
    hoist_ = any;
    for (auto& lv : levels_) {
      if (!hoist_) break;
      for (auto& it : lv.items)
        if (it.x->value().size() == 0 || it.w->value().size() == 0) hoist_ = false;
      for (auto* c : lv.cells)
        if (c->gates()->value().size() == 0 && kind_of(c->gates().get()) == BaseNode::kPlain) hoist_ = false;
      if (hoist_ && !lv.sized && (!lv.items.empty() || !lv.cells.empty())) size_level(lv);
    }
    if (!hoist_) {
      for (auto& lv : levels_)
        for (auto& it : lv.items) it.hoisted = false;
      return;
    }
    std::vector<const Item*> items;
    for (auto& lv : levels_)
      for (auto& it : lv.items)
        if (it.hoisted) items.push_back(&it);
    prepare(hoisted_.fwd, items, GINN_B200_GROUPED_FORWARD, false);
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
      if (it.w->has_grad()) {
        if (!it.hoisted) dw_items.push_back(&it);
      } else {
        GINN_ASSERT(!(it.bias && it.bias->has_grad()),
                    "autobatch: a bias gradient without its weight gradient is not batched; use Graph");
      }
    }
    for (auto& wv : waves) prepare(lv.bwd, wv, GINN_B200_GROUPED_DX, true);
    prepare_dw(lv.bwd, dw_items);
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
        GINN_AB_TIME(3);
        internal::b200_check(ginn_b200_lstm_cells_level_create(
            internal::b200_device(dev_), 1, live[0]->hidden(), n, t.data(), &lv.cells_bwd));
      }
    }
    lv.bwd_ready = true;
  }

  void destroy() {
    release_capture();
    if (side_) {
      cudaStreamSynchronize(side_);
      cudaStreamDestroy(side_);
      cudaEventDestroy(join_);
      side_ = nullptr;
      join_ = nullptr;
    }
    for (auto& lv : levels_) {  // the nodes outlive this object: end their aliases of its storage
      for (auto* t : lv.placed) t->unmap();
      lv.placed.clear();
    }
    if (hoisted_.ready) cudaEventDestroy(hoisted_.ready);
    hoisted_.ready = nullptr;
    for (auto& lv : levels_)
      if (lv.ready) {
        cudaEventDestroy(lv.ready);
        lv.ready = nullptr;
      }
    for (auto* ls : {&hoisted_.fwd, &hoisted_.bwd})
      for (auto& L : *ls)
        if (L.handle) ginn_b200_level_destroy(L.handle);
    hoisted_.fwd.clear();
    hoisted_.bwd.clear();
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
      : list_(std::move(o.list_)), levels_(std::move(o.levels_)), hoisted_(std::move(o.hoisted_)),
        sized_(o.sized_), hoist_(o.hoist_), pass_exec_(o.pass_exec_), side_(o.side_), join_(o.join_),
        side_used_(o.side_used_), dev_(std::move(o.dev_)),
        zero_ranges_(std::move(o.zero_ranges_)), zero_ready_(o.zero_ready_) {
    o.levels_.clear();
    o.hoisted_.fwd.clear();
    o.hoisted_.bwd.clear();
    o.pass_exec_ = nullptr;
    o.side_ = nullptr;
    o.join_ = nullptr;
    o.hoisted_.ready = nullptr;
  }
  ~BatchedGraph() { destroy(); }

  BatchedGraph& forward() {
    if (!sized_) {
      decide_hoist();
      sized_ = true;
    }
    if (hoist_) {
      bool todo = false;
      for (auto& lv : levels_)
        for (auto& it : lv.items) todo = todo || (it.hoisted && !it.out->forwarded);
      if (todo) run(hoisted_.fwd);
    }
    for (auto& lv : levels_) {
      for (auto* n : lv.plain) n->forward();
      bool todo = false;
      for (auto* o : lv.outs) todo = todo || !o->forwarded;
      for (auto* c : lv.cells) todo = todo || !c->forwarded;
      if (!todo) continue;
      if (!lv.fwd_ready) {
        if (!lv.sized) size_level(lv);
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
      if (!lv->bwd.empty()) run_backward(lv->bwd, event_of(*lv));
    }
    if (hoist_) {  // the hoisted items' weight (and bias) gradients: every out.grad is final now
      if (!hoisted_.bwd_ready) {
        std::vector<const Item*> dw_items;
        for (auto& lv : levels_)
          for (auto& it : lv.items)
            if (it.hoisted && it.out->has_grad() && it.w->has_grad()) dw_items.push_back(&it);
        prepare_dw(hoisted_.bwd, dw_items);
        hoisted_.bwd_ready = true;
      }
      if (!hoisted_.bwd.empty()) run_backward(hoisted_.bwd, event_of(hoisted_));
    }
    if (side_used_) {  // the pass ends when the weight gradients are in as well
      GINN_CUDA_CALL(cudaEventRecord(join_, side_));
      GINN_CUDA_CALL(cudaStreamWaitEvent(stream_of(*dev_), join_, 0));
      side_used_ = false;
    }
    return *this;
  }

  // Zero-fills every gradient, as Graph::reset_grad does node by node (ginn/node.h:197-200,
  // 261-264) -- but gradients that sit back to back in memory (a bump allocator hands them out
  // that way) are cleared with one fill per contiguous range.
  BatchedGraph& reset_grad() {
    if (!zero_ready_) {
      GINN_AB_TIME(4);
      // gradients of a level's batched nodes: one allocation per kind, laid out like the values
      // (init_grad then finds them in place and allocates nothing for them)
      std::vector<std::pair<char*, size_t>> slab_ranges;  // the gradient storage placed below
      for (auto& lv : levels_) {
        const size_t first_slab = lv.slabs.size();
        std::vector<Tensor<Real>*> g, gh, gc;
        std::vector<Shape> gs, hs;
        for (auto* o : lv.outs)
          if (o->has_grad()) {
            g.push_back(&o->grad());
            gs.push_back(o->value().shape());
          }
        for (auto* c : lv.cells)
          if (c->has_grad()) {
            gh.push_back(&c->grad());
            gc.push_back(&c->dc());
            hs.push_back(c->value().shape());
          }
        place(lv, g, gs);
        place(lv, gh, hs);
        place(lv, gc, hs);
        for (size_t i = first_slab; i < lv.slabs.size(); ++i)
          slab_ranges.emplace_back(reinterpret_cast<char*>(lv.slabs[i]->data()),
                                   static_cast<size_t>(lv.slabs[i]->size()) * sizeof(Real));
      }
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
        if (t.size() == 0 || t.is_mapped()) return;  // aliases: covered by what they alias
        Device* d = t.dev().get();
        r.push_back({reinterpret_cast<char*>(t.data()), t.size() * sizeof(Real),
                     d->precedence() > 0 ? d : nullptr});
      };
      for (auto& e : list_) {
        if (!e->has_grad()) continue;
        // the batched kinds are Node<Real>s by construction: no run-time cast needed for them
        auto n = e->batch_kind() != BaseNode::kPlain ? static_cast<Node<Real>*>(e.get())
                                                     : dynamic_cast<Node<Real>*>(e.get());
        if (!n || n->value().dev()->kind() != GPU) {
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
      for (auto& sr : slab_ranges) r.push_back({sr.first, sr.second, nullptr});
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

  // A graph that is evaluated many times with the same structure (an epoch over fixed-shape
  // batches, a benchmark) pays ~200 host-side launches per pass; on B200 the pass itself is
  // shorter than the time the host needs to issue them.  capture_pass() runs one full pass
  // (forward, reset_grad, backward) eagerly -- which prepares every level -- and then records a
  // second one into a CUDA graph; replay_pass() launches the recording.  Every launch of a
  // prepared level is capturable (no host-to-device copies); plain nodes of the graph must be
  // capturable too (no synchronous copies in their forward_/backward_).  Inputs may be rewritten
  // in place between replays; shapes and tensor addresses may not change.
  BatchedGraph& capture_pass(double loss_coeff = 1) {
    GINN_ASSERT(dev_, "capture_pass: the graph has no GPU nodes");
    release_capture();
    reset_forwarded().forward().reset_grad().backward(loss_coeff);
    cudaStream_t st = stream_of(*dev_);
    GINN_CUDA_CALL(cudaStreamSynchronize(st));
    reset_forwarded();
    GINN_CUDA_CALL(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    forward().reset_grad().backward(loss_coeff);
    cudaGraph_t g = nullptr;
    GINN_CUDA_CALL(cudaStreamEndCapture(st, &g));
    GINN_CUDA_CALL(cudaGraphInstantiate(&pass_exec_, g, 0));
    GINN_CUDA_CALL(cudaGraphDestroy(g));
    return *this;
  }
  BatchedGraph& replay_pass() {
    GINN_ASSERT(pass_exec_ != nullptr, "replay_pass: call capture_pass first");
    GINN_CUDA_CALL(cudaGraphLaunch(pass_exec_, stream_of(*dev_)));
    return *this;
  }
  const std::vector<BaseNodePtr>& nodes() const { return list_; }
  BaseNodePtr sink() const { return list_.back(); }
  size_t levels() const { return levels_.size(); }
  // How many of the prepared product launches have equally spaced column tables throughout
  // (the library runs those as plain TMA-fed products).
  size_t strided_launches() const {
    size_t n = 0;
    auto count = [&](const std::vector<Launch>& ls) {
      for (auto& L : ls) {
        bool all = !L.groups.empty();
        for (auto& g : L.groups) all = all && strided(g, L.mode);
        n += all ? 1 : 0;
      }
    };
    count(hoisted_.fwd);
    count(hoisted_.bwd);
    for (auto& lv : levels_) {
      count(lv.fwd);
      count(lv.bwd);
    }
    return n;
  }
  // Number of library launches a forward + backward pass makes (after preparation).
  size_t launches() const {
    size_t n = hoisted_.fwd.size() + hoisted_.bwd.size();
    for (auto& lv : levels_)
      n += lv.fwd.size() + lv.bwd.size() + (lv.cells_fwd ? 1 : 0) + (lv.cells_bwd ? 1 : 0);
    return n;
  }
};

inline BatchedGraph Autobatch(const Graph& g) { return BatchedGraph(g); }

}  // namespace ginn
#endif
