// Benchmark of the host-side autobatch path (ginn_b200/include/ginn/autobatch.h) on config 2:
// 256 sequences of length U{5..40}, per sequence and step
//     gates = Affine(W_x[4H x E], x_t, W_h[4H x H], h_{t-1}, b);  (h_t, c_t) = LstmCell(gates, ...)
// with H = 256, E = 128 and shared weights, one graph node per sequence and step as a ginn
// program builds it (ginn/model/lstm.h, examples/sum-lstm.cu.cpp), node tensors taken from a
// PreallocGpuDevice that is cleared between graphs.
//
// Timed with the host clock around device synchronisation, per graph:
//   build     constructing the nodes (ginn's own cost, not Autobatch's)
//   rewrite   Autobatch(g): heights, kinds, items                       (ginn/autobatch.h:57-147)
//   first     forward + reset_grad + backward including the one-time preparation of the levels
//   replay    the same pass again on the prepared schedule (a graph evaluated more than once)
//   graph     the same pass replayed from a CUDA graph (BatchedGraph::capture_pass / replay_pass)
// Prints one JSON object.  nodes = number of gate Affines (the unit of "autobatched nodes/s").
#include <chrono>
#include <cstdio>
#include <cstring>
#include <random>

#include <ginn/ginn.h>

using namespace ginn;
using Clock = std::chrono::steady_clock;

static double ms_since(Clock::time_point t0) {
  return std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
}

// Loss = sum over the given cells of sum_i h_i.  Only its gradient is produced (one grouped
// launch adds the sink's gradient to every element of every cell's dh); value() stays 0.
class SumOfCellsNode : public BaseDataNode<Real> {
  std::vector<Ptr<LstmCellNode>> cells_;
  Tensor<Real> ones_;  // 1 x H

  static std::vector<BaseNodePtr> base(const std::vector<Ptr<LstmCellNode>>& c) {
    return std::vector<BaseNodePtr>(c.begin(), c.end());
  }
  void forward_() override {
    value().resize({1, 1});
    value().set_zero();
    const Size H = cells_[0]->value().rows();  // known once the cells have run
    if (ones_.size() != H) {
      ones_.resize({1, H});
      ones_.set(std::vector<Real>(H, 1.f));
    }
  }
  // Prepared once (the cells' gradient tensors do not move after the first pass) and run from
  // then on: a prepared level copies nothing from the host at run time, so the pass can be
  // recorded into a CUDA graph.
  ginn_b200_level* level_ = nullptr;
  void backward_() override {
    if (level_ == nullptr) {
      const Size H = cells_[0]->value().rows();
      std::vector<void*> dy, dx;
      for (auto& c : cells_) {
        dy.push_back(grad().data());
        dx.push_back(c->grad().data());
      }
      ginn_b200_group g{};
      g.w = ones_.data();
      g.ldw = 1;
      g.m = 1;
      g.k = H;
      g.ncols = static_cast<int64_t>(cells_.size());
      g.y_cols = dy.data();
      g.dx_cols = dx.data();
      internal::b200_check(ginn_b200_level_create(internal::b200_device(dev()), GINN_B200_F32,
                                                  GINN_B200_GROUPED_DX, 1, &g, &level_));
    }
    internal::b200_check(ginn_b200_level_run(level_, stream_of(*dev())));
  }

 public:
  SumOfCellsNode(DevPtr weights_dev, const std::vector<Ptr<LstmCellNode>>& cells)
      : BaseDataNode<Real>(base(cells)), cells_(cells), ones_(std::move(weights_dev)) {}
  ~SumOfCellsNode() override {
    if (level_) ginn_b200_level_destroy(level_);
  }
  std::string name() const override { return "SumOfCells"; }
};

int main(int argc, char** argv) {
  const int graphs = argc > 1 ? std::atoi(argv[1]) : 5;
  const int replays = argc > 2 ? std::atoi(argv[2]) : 20;
  const Size H = 256, E = 128, nseq = 256;
  if (gpus() < 1) {
    std::printf("{\"error\": \"no GPU\"}\n");
    return 2;
  }
  std::mt19937 gen(20242);
  std::uniform_int_distribution<int> len_dist(5, 40);
  std::vector<int> lens(nseq);
  Size total = 0;
  for (auto& l : lens) {
    l = len_dist(gen);
    total += l;
  }
  // Weights and the input data live on the ordinary device; everything a graph creates comes
  // from the preallocated one and is dropped with clear().
  auto Wx = Random<Real>(gpu(), {4 * H, E}, 1), Wh = Random<Real>(gpu(), {4 * H, H}, 2);
  auto b = Random<Real>(gpu(), {4 * H}, 3);
  {
    // Xavier-sized weights keep the recurrence in range (ginn/init/init.h:45-51)
    auto scale = [](DataPtr<Real>& w, Size rows, Size cols) {
      auto v = w->value().vector();
      const float a = std::sqrt(6.f / (0.5f * (rows + cols)));
      for (auto& x : v) x *= a;
      w->value().set(v);
    };
    scale(Wx, 4 * H, E + H);
    scale(Wh, 4 * H, E + H);
  }
  auto X = Random<Real>(gpu(), {E, total}, 4);   // every x_t is a column of this matrix
  X->set_has_grad(false);
  auto pre = PreallocGpu(0, size_t(768) << 20);

  double build_ms = 0, rewrite_ms = 0, first_ms = 0, replay_ms = 0, graph_ms = 0;
  size_t levels = 0, launches = 0, strided = 0;
  for (int it = 0; it < graphs + 1; ++it) {  // the first graph warms the library up, untimed
    pre->clear();
    GINN_CUDA_CALL(cudaDeviceSynchronize());
    auto t0 = Clock::now();
    auto h0 = Data<Real>(pre, {H});
    h0->value().set_zero();
    h0->set_has_grad(false);
    std::vector<Ptr<LstmCellNode>> finals;
    Size col = 0;
    for (Size q = 0; q < nseq; ++q) {
      NodePtr<Real> h = h0;
      Ptr<LstmCellNode> cell;
      for (int t = 0; t < lens[q]; ++t, ++col) {
        auto x = make_ptr<DataNode<Real>>(pre, Shape{0});
        x->value().map(X->value(), {E}, col * E);
        x->set_has_grad(false);
        NodePtr<Real> gates = Affine(Wx, x, Wh, h, b);
        cell = LstmCell(gates, cell);
        h = cell;
      }
      finals.push_back(cell);
    }
    NodePtr<Real> loss = make_ptr<SumOfCellsNode>(gpu(), finals);
    Graph g(loss);
    const double t_build = ms_since(t0);

    t0 = Clock::now();
    auto bg = Autobatch(g);
    const double t_rewrite = ms_since(t0);

    t0 = Clock::now();
    bg.forward().reset_grad().backward(1.);
    GINN_CUDA_CALL(cudaDeviceSynchronize());
    const double t_first = ms_since(t0);

    GINN_CUDA_CALL(cudaDeviceSynchronize());
    t0 = Clock::now();
    for (int r = 0; r < replays; ++r) bg.reset_forwarded().forward().reset_grad().backward(1.);
    GINN_CUDA_CALL(cudaDeviceSynchronize());
    const double t_replay = ms_since(t0) / replays;
    bg.capture_pass(1.);
    for (int r = 0; r < 3; ++r) bg.replay_pass();
    GINN_CUDA_CALL(cudaDeviceSynchronize());
    t0 = Clock::now();
    for (int r = 0; r < replays; ++r) bg.replay_pass();
    GINN_CUDA_CALL(cudaDeviceSynchronize());
    const double t_graph = ms_since(t0) / replays;
    if (it > 0) {
      graph_ms += t_graph;
      build_ms += t_build;
      rewrite_ms += t_rewrite;
      first_ms += t_first;
      replay_ms += t_replay;
    }
    levels = bg.levels();
    launches = bg.launches();
    strided = bg.strided_launches();
  }
  build_ms /= graphs;
  rewrite_ms /= graphs;
  first_ms /= graphs;
  replay_ms /= graphs;
  graph_ms /= graphs;
  const int status = ginn_b200_device_status(0, 1);
  std::printf(
      "{\"nodes\": %ld, \"levels\": %zu, \"launches_per_pass\": %zu, \"table_free_launches\": %zu, "
      "\"graphs\": %d, \"build_ms\": %.3f, \"rewrite_ms\": %.3f, \"first_pass_ms\": %.3f, "
      "\"replay_pass_ms\": %.3f, \"graph_pass_ms\": %.3f, \"nodes_per_s_with_rewrite\": %.1f, "
      "\"nodes_per_s_replay\": %.1f, \"nodes_per_s_graph\": %.1f, \"device_status\": %d}\n",
      (long)total, levels, launches, strided, graphs, build_ms, rewrite_ms,
      first_ms, replay_ms, graph_ms, total / ((rewrite_ms + first_ms) * 1e-3),
      total / (replay_ms * 1e-3), total / (graph_ms * 1e-3), status);
  return status == 0 ? 0 : 1;
}
