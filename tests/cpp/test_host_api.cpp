// Tests of the header-only host layer (ginn_b200/include/ginn) on a GPU, written after the
// reference's own node tests: known answers (test/nodes.cu.cpp:1023-1196), BatchedProd against
// per-slice products (:1043-1115), the CPU-vs-GPU protocol of test/check_node.h:27-121 (same
// inputs on both sides, value and every input gradient within eps, gradients accumulated over two
// consumers), the autobatch before/after protocol of test/autobatch.cpp:37-190, and the
// allocation accounting of test/dev.cu.cpp.  The CPU side is the C restatement in
// oracle/cpu_path.c (test infrastructure).
#include <cmath>
#include <cstdio>
#include <functional>
#include <string>

#include <ginn/ginn.h>

extern "C" {
void cpu_gemm(int dtype, int ta, int tb, long m, long n, long k, const void* A, long lda,
              const void* B, long ldb, void* C, long ldc, int accumulate, int threads);
void cpu_affine_forward(int dtype, int npairs, const void* const* A, const long* lda,
                        const void* const* B, const long* ldb, const long* ks, long m, long n,
                        const void* bias, int act, void* out, long ldo, int threads);
void cpu_affine_backward(int dtype, int npairs, const void* const* A, const long* lda,
                         const void* const* B, const long* ldb, const long* ks, void* const* dA,
                         const long* ldda, void* const* dB, const long* lddb, long m, long n,
                         const void* dout, long lddout, const void* out, long ldout, int act,
                         void* dbias, void* scratch, int threads);
}

using namespace ginn;

static int g_failed = 0, g_checks = 0;
#define CHECK(cond)                                                          \
  do {                                                                       \
    ++g_checks;                                                              \
    if (!(cond)) {                                                           \
      ++g_failed;                                                            \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);          \
    }                                                                        \
  } while (0)

static float f(float x) { return x; }
static float f(Half x) { return __half2float(x); }

template <typename S>
static bool close(const std::vector<S>& got, const std::vector<float>& want, float rel,
                  float abs_eps = 1e-6f) {
  if (got.size() != want.size()) return false;
  for (size_t i = 0; i < got.size(); ++i) {
    const float d = std::fabs(f(got[i]) - want[i]);
    if (!(d <= rel * std::fabs(want[i]) || d <= abs_eps)) {
      std::printf("  element %zu: got %g want %g\n", i, f(got[i]), want[i]);
      return false;
    }
  }
  return true;
}
template <typename S>
static std::vector<float> floats(const std::vector<S>& v) {
  std::vector<float> o(v.size());
  for (size_t i = 0; i < v.size(); ++i) o[i] = f(v[i]);
  return o;
}

template <typename S>
static void test_prod_known_answer(float eps) {
  auto W = Values<S>(gpu(), {{1, 2, 3}, {4, 5, 6}});
  auto V = Values<S>(gpu(), {{0.6, 0.5}, {0.4, -0.1}, {-0.2, -0.3}});
  auto p = W * V;
  Graph(p).forward();
  CHECK(close(p->value().vector(), {0.8f, 3.2f, -0.6f, -0.3f}, eps));  // column-major
  CHECK((p->shape() == Shape{2, 2}));
}

template <typename S>
static void test_affine_known_answers(float eps) {
  auto W = Values<S>(gpu(), {{1, 2, 3}, {4, 5, 6}});
  auto V = Values<S>(gpu(), {{0.6}, {0.4}, {-0.2}});
  auto b = Values<S>(gpu(), {{0.01}, {0.02}});
  auto a = Affine(W, V, b);
  Graph(a).forward();
  CHECK(close(a->value().vector(), {0.81f, 3.22f}, eps));
  auto s = Affine<SigmoidOp>(W, V, b);
  Graph(s).forward();
  CHECK(close(s->value().vector(), {0.692109f, 0.96158f}, std::max(eps, 2e-6f)));
  auto s2 = Affine(SigmoidOp<S>(), W, V, b);
  Graph(s2).forward();
  CHECK(close(s2->value().vector(), {0.692109f, 0.96158f}, std::max(eps, 2e-6f)));
  // broadcast over columns
  auto V2 = Values<S>(gpu(), {{6, 5}, {4, -1}, {-2, -3}});
  auto b2 = Values<S>(gpu(), {{0.1}, {0.2}});
  auto a2 = Affine(W, V2, b2);
  Graph(a2).forward();
  CHECK(close(a2->value().vector(), {8.1f, 32.2f, -5.9f, -2.8f}, eps));
  // rank-3 right operand: output rank follows it
  auto V3 = Data<S>(gpu(), {3, 2, 2});
  std::vector<S> v3;
  for (int rep = 0; rep < 2; ++rep)
    for (float x : {6.f, 4.f, -2.f, 5.f, -1.f, -3.f}) v3.push_back(S(x));
  V3->value().set(v3);
  auto b1 = Data<S>(gpu(), {2});
  b1->value().set({S(0.1f), S(0.2f)});
  auto a3 = Affine(W, V3, b1);
  Graph(a3).forward();
  CHECK((a3->shape() == Shape{2, 2, 2}));
  CHECK(close(a3->value().vector(), {8.1f, 32.2f, -5.9f, -2.8f, 8.1f, 32.2f, -5.9f, -2.8f}, eps));
}

template <typename S>
static void test_batched_prod_equals_slices(float eps) {
  for (Shape extra : {Shape{4}, Shape{2, 2}}) {
    Shape sa{2, 3}, sb{3, 5};
    for (Size d : extra) {
      sa.push_back(d);
      sb.push_back(d);
    }
    auto a = Random<S>(gpu(), sa, 1), b = Random<S>(gpu(), sb, 2);
    auto c = BatchedProd(a, b);
    Graph(c).forward();
    auto cv = c->value().vector();
    const Size batches = Tensor<S>::size(extra);
    for (Size i = 0; i < batches; ++i) {
      auto ai = Data<S>(gpu(), {2, 3});
      auto bi = Data<S>(gpu(), {3, 5});
      ai->value().map(a->value(), {2, 3}, 6 * i);
      bi->value().map(b->value(), {3, 5}, 15 * i);
      auto ci = ai * bi;
      Graph(ci).forward();
      std::vector<S> slice(cv.begin() + 10 * i, cv.begin() + 10 * (i + 1));
      CHECK(close(slice, floats(ci->value().vector()), eps, 1e-3f * eps * 100));
    }
  }
}

// CPU-vs-GPU: f(sum A_i B_i + b) consumed twice, every gradient against the CPU restatement.
template <typename S, template <typename> class Op>
static void test_affine_cpu_vs_gpu(int act, float eps) {
  const int dtype = sizeof(S) == 4 ? 0 : 1;
  const long m = 37, k1 = 29, k2 = 11, n = 23;
  auto W = Random<S>(gpu(), {m, k1}, 3), X = Random<S>(gpu(), {k1, n}, 4);
  auto V = Random<S>(gpu(), {m, k2}, 5), H = Random<S>(gpu(), {k2, n}, 6);
  auto b = Random<S>(gpu(), {m}, 7);
  auto I = Data<S>(gpu(), {m, m});
  {
    std::vector<S> id(m * m, S(0.f));
    for (long i = 0; i < m; ++i) id[i + i * m] = S(1.f);
    I->value().set(id);
    I->set_has_grad(false);
  }
  auto zero = Data<S>(gpu(), {m});
  zero->value().set_zero();
  zero->set_has_grad(false);
  auto e = Affine<Op>(W, X, V, H, b);
  auto sink = Affine(I, e, I, e, zero);  // e + e: two gradient contributions must accumulate
  Graph g(sink);
  g.forward().reset_grad().backward(1.);

  auto w = W->value().vector(), x = X->value().vector(), v = V->value().vector(),
       h = H->value().vector(), bv = b->value().vector();
  std::vector<S> y(m * n), dY(m * n, S(2.f)), dW(m * k1, S(0.f)), dX(k1 * n, S(0.f)),
      dV(m * k2, S(0.f)), dH(k2 * n, S(0.f)), db(m, S(0.f)), scratch(m * n);
  const void* A[2] = {w.data(), v.data()};
  const void* B[2] = {x.data(), h.data()};
  const long lda[2] = {m, m}, ldb[2] = {k1, k2}, ks[2] = {k1, k2};
  cpu_affine_forward(dtype, 2, A, lda, B, ldb, ks, m, n, bv.data(), act, y.data(), m, 1);
  void* dA[2] = {dW.data(), dV.data()};
  void* dB[2] = {dX.data(), dH.data()};
  cpu_affine_backward(dtype, 2, A, lda, B, ldb, ks, dA, lda, dB, ldb, m, n, dY.data(), m,
                      y.data(), m, act, db.data(), scratch.data(), 1);
  // Half: the CPU side rounds the running sum to fp16 after every product and the bias add,
  // the GPU once at the end, so small outputs differ by a few fp16 ulps of the pre-activation.
  const float aeps = sizeof(S) == 2 ? 5e-3f : eps * 0.05f;
  CHECK(close(e->value().vector(), floats(y), eps, aeps));
  CHECK(close(W->grad().vector(), floats(dW), eps, aeps * 20));
  CHECK(close(X->grad().vector(), floats(dX), eps, aeps * 20));
  CHECK(close(V->grad().vector(), floats(dV), eps, aeps * 20));
  CHECK(close(H->grad().vector(), floats(dH), eps, aeps * 20));
  CHECK(close(b->grad().vector(), floats(db), eps, aeps * 20));
}

static void test_prod_cpu_vs_gpu() {
  const long m = 40, k = 33, n = 21;
  auto A = Random<Real>(gpu(), {m, k}, 8), B = Random<Real>(gpu(), {k, n}, 9);
  B->set_has_grad(false);  // inputs without gradient are skipped
  auto p = A * B;
  Graph g(p);
  g.forward().reset_grad().backward(1.);
  auto a = A->value().vector(), b = B->value().vector();
  std::vector<float> c(m * n), ones(m * n, 1.f), dA(m * k, 0.f);
  cpu_gemm(0, 0, 0, m, n, k, a.data(), m, b.data(), k, c.data(), m, 0, 1);
  cpu_gemm(0, 0, 1, m, k, n, ones.data(), m, b.data(), k, dA.data(), m, 1, 1);
  CHECK(close(p->value().vector(), c, 1e-4f, 1e-5f));
  CHECK(close(A->grad().vector(), dA, 1e-4f, 1e-5f));
  CHECK(B->grad().size() == 0);
}

// Value of the sink and gradients of `ins`, first through Graph, then through Autobatch.
static void check_autobatch(const NodePtr<Real>& sink, const std::vector<NodePtr<Real>>& ins,
                            size_t expect_fewer_levels_than_nodes = 0) {
  Graph g(sink);
  g.reset_forwarded().forward();
  auto before = sink->value().vector();
  g.reset_grad().backward(1.);
  std::vector<std::vector<Real>> d_before;
  for (auto& in : ins) d_before.push_back(in->grad().vector());

  auto bg = Autobatch(g);
  bg.reset_forwarded().forward();
  CHECK(close(sink->value().vector(), before, 1e-4f, 1e-5f));
  bg.reset_grad().backward(1.);
  for (size_t i = 0; i < ins.size(); ++i) {
    const bool same = close(ins[i]->grad().vector(), d_before[i], 1e-4f, 1e-5f);
    if (!same) std::printf("  (gradient of input %zu differs after Autobatch)\n", i);
    CHECK(same);
  }
  if (expect_fewer_levels_than_nodes) CHECK(bg.levels() < expect_fewer_levels_than_nodes);
}

static NodePtr<Real> identity_sum(const std::vector<NodePtr<Real>>& hs, Size m) {
  // sum_i h_i as one Affine with identity weights (the layer has no Add node)
  auto I = Data<Real>(gpu(), {m, m});
  std::vector<Real> id(m * m, 0.f);
  for (Size i = 0; i < m; ++i) id[i + i * m] = 1.f;
  I->value().set(id);
  I->set_has_grad(false);
  auto zero = Data<Real>(gpu(), {m});
  zero->value().set_zero();
  zero->set_has_grad(false);
  std::vector<NodePtr<Real>> ins;
  for (auto& h : hs) {
    ins.push_back(I);
    ins.push_back(h);
  }
  ins.push_back(zero);
  return make_ptr<AffineNode<Real>>(ins);
}

static void test_autobatch() {
  {  // stacked Affines sharing inputs (test/autobatch.cpp "Autobatch grad")
    auto x = Random<Real>(gpu(), {2, 2}, 11), y = Random<Real>(gpu(), {2, 2}, 12);
    auto b = Random<Real>(gpu(), {2}, 13);
    NodePtr<Real> h = Affine(x, y, x, y, b);
    NodePtr<Real> t = Affine(h, y, b);
    check_autobatch(t, {x, y, b});
  }
  for (int mixed = 0; mixed < 2; ++mixed) {  // "Recurrent" and "Recurrent mixed"
    std::vector<NodePtr<Real>> x;
    for (int i = 0; i < 12; ++i) x.push_back(Random<Real>(gpu(), {2}, 20 + i));
    auto W = Random<Real>(gpu(), {3, 2}, 40), V = Random<Real>(gpu(), {3, 3}, 41);
    auto b = Random<Real>(gpu(), {3}, 42);
    std::vector<NodePtr<Real>> hs;
    size_t nodes = 0;
    for (int i = 0; i < 3; ++i) {
      NodePtr<Real> h = Data<Real>(gpu(), {3});
      h->value().set_zero();
      for (int t = 0; t < 4; ++t) {
        if (mixed && (i + t) % 2 == 0) {
          NodePtr<Real> wx = W * x[4 * i + t];
          NodePtr<Real> vh = V * h;
          h = identity_sum({wx, vh}, 3);  // W*x + V*h (bias-free variant of the mixed case)
          nodes += 3;
        } else {
          h = Affine(W, x[4 * i + t], V, h, b);
          nodes += 1;
        }
      }
      hs.push_back(h);
    }
    auto s = identity_sum(hs, 3);
    std::vector<NodePtr<Real>> ins = x;
    ins.push_back(W);
    ins.push_back(V);
    ins.push_back(b);
    check_autobatch(s, ins, nodes);
  }
  {  // a level with several groups of different shapes and a shared right operand
    auto x = Random<Real>(gpu(), {40, 3}, 50);
    auto W1 = Random<Real>(gpu(), {130, 40}, 51), W2 = Random<Real>(gpu(), {17, 40}, 52);
    auto b1 = Random<Real>(gpu(), {130}, 53), b2 = Random<Real>(gpu(), {17}, 54);
    NodePtr<Real> h1 = Affine(W1, x, b1), h2 = Affine(W2, x, b2);  // both read and update x
    auto U = Random<Real>(gpu(), {8, 130}, 55), T = Random<Real>(gpu(), {8, 17}, 56);
    auto c = Random<Real>(gpu(), {8}, 57);
    NodePtr<Real> out = Affine(U, h1, T, h2, c);
    check_autobatch(out, {x, W1, W2, b1, b2, U, T, c});
  }
}

// Affines with fused nonlinearities (which the reference's Autobatch does not batch,
// ginn/autobatch.h:30-38) and LSTM cells: a small recurrent net, node by node through Graph and
// level by level through Autobatch.
static void test_autobatch_nonlinear_and_cells() {
  {  // "Recurrent" of test/autobatch.cpp with tanh inside the Affines
    std::vector<NodePtr<Real>> x;
    for (int i = 0; i < 12; ++i) x.push_back(Random<Real>(gpu(), {2}, 120 + i));
    auto W = Random<Real>(gpu(), {3, 2}, 140), V = Random<Real>(gpu(), {3, 3}, 141);
    auto b = Random<Real>(gpu(), {3}, 142);
    std::vector<NodePtr<Real>> hs;
    for (int i = 0; i < 3; ++i) {
      NodePtr<Real> h = Data<Real>(gpu(), {3});
      h->value().set_zero();
      for (int t = 0; t < 2 + i; ++t)  // sequences of different lengths
        h = (t % 2) ? NodePtr<Real>(Affine<TanhOp>(W, x[4 * i + t], V, h, b))
                    : NodePtr<Real>(Affine<SigmoidOp>(W, x[4 * i + t], V, h, b));
      hs.push_back(h);
    }
    auto s = identity_sum(hs, 3);
    std::vector<NodePtr<Real>> ins = x;
    ins.push_back(W);
    ins.push_back(V);
    ins.push_back(b);
    check_autobatch(s, ins, 10);
  }
  {  // one Affine for the four gates + one cell node per step, three sequences of lengths 3, 2, 4
    const Size H = 8, E = 4;
    auto Wx = Random<Real>(gpu(), {4 * H, E}, 150), Wh = Random<Real>(gpu(), {4 * H, H}, 151);
    auto b = Random<Real>(gpu(), {4 * H}, 152);
    std::vector<NodePtr<Real>> ins{Wx, Wh, b}, finals;
    const int lens[3] = {3, 2, 4};
    size_t nodes = 0;
    for (int q = 0; q < 3; ++q) {
      NodePtr<Real> h = Random<Real>(gpu(), {H}, 160 + q);
      ins.push_back(h);
      Ptr<LstmCellNode> cell;
      for (int t = 0; t < lens[q]; ++t) {
        auto xt = Random<Real>(gpu(), {E}, 170 + 10 * q + t);
        ins.push_back(xt);
        NodePtr<Real> gates = Affine(Wx, xt, Wh, h, b);
        cell = LstmCell(gates, cell);
        h = cell;
        nodes += 2;
      }
      finals.push_back(h);
    }
    check_autobatch(identity_sum(finals, H), ins, nodes);
  }
  {  // the same net on inputs without gradients: their products W_x x_t are hoisted out of the
     // levels (one launch ahead of them, one weight-gradient launch after), the levels' tensors
     // lie back to back, and the whole pass is replayed from a CUDA graph with new input data
    const Size H = 8, E = 4;
    auto Wx = Random<Real>(gpu(), {4 * H, E}, 250), Wh = Random<Real>(gpu(), {4 * H, H}, 251);
    auto b = Random<Real>(gpu(), {4 * H}, 252);
    std::vector<NodePtr<Real>> ins{Wx, Wh, b}, finals, xs;
    const int lens[4] = {2, 5, 3, 5};
    size_t nodes = 0;
    for (int q = 0; q < 4; ++q) {
      NodePtr<Real> h = Random<Real>(gpu(), {H}, 260 + q);
      ins.push_back(h);
      Ptr<LstmCellNode> cell;
      for (int t = 0; t < lens[q]; ++t) {
        auto xt = Random<Real>(gpu(), {E}, 270 + 10 * q + t);
        xt->set_has_grad(false);
        xs.push_back(xt);
        NodePtr<Real> gates = Affine(Wx, xt, Wh, h, b);
        cell = LstmCell(gates, cell);
        h = cell;
        nodes += 2;
      }
      finals.push_back(h);
    }
    auto sink = identity_sum(finals, H);
    check_autobatch(sink, ins, nodes);
    // replayed pass: new inputs, Graph as the reference
    for (size_t i = 0; i < xs.size(); ++i) {
      auto v = xs[i]->value().vector();
      for (auto& e : v) e = 0.5f * e - 0.1f;
      xs[i]->value().set(v);
    }
    Graph g(sink);
    auto bg = Autobatch(g);
    bg.capture_pass(1.);
    bg.replay_pass();
    GINN_CUDA_CALL(cudaDeviceSynchronize());
    auto value = sink->value().vector();
    std::vector<std::vector<Real>> grads;
    for (auto& in : ins) grads.push_back(in->grad().vector());
    CHECK(bg.launches() < 5 * 5 + 4 * 5 + 6);  // one forward launch per level, not two
    Graph g2(sink);  // the nodes' tensors stay where Autobatch put them; Graph runs node by node
    g2.reset_forwarded().forward();
    CHECK(close(sink->value().vector(), value, 1e-4f, 1e-5f));
    g2.reset_grad().backward(1.);
    for (size_t i = 0; i < ins.size(); ++i) CHECK(close(ins[i]->grad().vector(), grads[i], 1e-4f, 1e-5f));
  }
}

// test/convnodes.cu.cpp:38-70 ("Conv2d"): known values with and without strides, then both
// gradients of sum(y) against the closed form (every filter tap sums the inputs it touches).
static void test_conv2d() {
  auto x = Data<Real>(gpu(), {1, 3, 3, 1});
  x->value().set({1, 2, 3, 4, 5, 6, 7, 8, 9});  // column-major: element (0, r, c, 0) = 1 + r + 3c
  auto f = Data<Real>(gpu(), {1, 1, 2, 2});
  f->value().set({1, 2, 3, 4});                  // [[1, 3], [2, 4]]
  auto y = Conv2d(x, f);
  Graph g(y);
  g.forward();
  CHECK((y->shape() == Shape{1, 3, 3, 1}));
  CHECK(close(y->value().vector(), {37, 47, 21, 67, 77, 33, 23, 26, 9}, 1e-6f));
  auto y2 = Conv2d(x, f, 2, 1);
  Graph(y2).forward();
  CHECK((y2->shape() == Shape{1, 2, 3, 1}));
  CHECK(close(y2->value().vector(), {37, 21, 67, 33, 23, 9}, 1e-6f));
  auto y3 = Conv2d(x, f, 2, 3);
  Graph(y3).forward();
  CHECK(close(y3->value().vector(), {37, 21}, 1e-6f));
  g.reset_grad().backward(1.);
  // d sum(y) / d f[kr][kc] = sum of x over the window positions that tap stays inside the image
  CHECK(close(f->grad().vector(), {45, 33, 39, 28}, 1e-5f));  // (0,0), (1,0), (0,1), (1,1)
  // d sum(y) / d x[r][c] = sum of the taps that reach it: 1 at the top-left, 10 in the interior
  CHECK(close(x->grad().vector(), {1, 3, 3, 4, 10, 10, 4, 10, 10}, 1e-5f));
}

static void test_prealloc_accounting() {
  auto dev = PreallocGpu(0, 1 << 20);
  auto W = Data<Real>(dev, {8, 5}), x = Data<Real>(dev, {5, 3}), b = Data<Real>(dev, {8});
  W->value().set(std::vector<Real>(40, 0.5f));
  x->value().set(std::vector<Real>(15, 1.f));
  b->value().set(std::vector<Real>(8, 0.f));
  const size_t inputs = (40 + 15 + 8) * sizeof(Real);
  CHECK(dev->used() == inputs);
  auto a = Affine<TanhOp>(W, x, b);
  Graph g(a);
  g.forward();
  CHECK(a->dev().get() == dev.get());
  CHECK(dev->used() == inputs + 24 * sizeof(Real));  // the value, nothing hidden
  g.reset_grad();
  CHECK(dev->used() == inputs + (24 + 24 + 40 + 15 + 8) * sizeof(Real));  // + the gradients
  g.backward(1.);
  CHECK(dev->used() == inputs + (24 + 24 + 40 + 15 + 8) * sizeof(Real));  // backward allocates nothing
  CHECK(close(a->value().vector(), std::vector<float>(24, std::tanh(2.5f)), 1e-5f));
}

static void test_errors() {
  auto A = Random<Real>(gpu(), {4, 3}, 60), B = Random<Real>(gpu(), {5, 2}, 61);
  bool threw = false;
  try {
    Graph(A * B).forward();
  } catch (const RuntimeError&) {
    threw = true;
  }
  CHECK(threw);  // inner dimensions differ: GINN_ASSERT in gpu_prod
  auto a3 = Random<Real>(gpu(), {2, 3, 4}, 62), b3 = Random<Real>(gpu(), {3, 5, 5}, 63);
  threw = false;
  try {
    Graph(BatchedProd(a3, b3)).forward();
  } catch (const RuntimeError&) {
    threw = true;
  }
  CHECK(threw);
  auto c = Random<Real>(cpu(), {3, 2}, 64);
  threw = false;
  try {
    Graph(c * c).forward();
  } catch (const RuntimeError&) {
    threw = true;
  }
  CHECK(threw);  // CPU tensors are not served: no silent fallback
}

// test/nodes.cu.cpp:755-797 ("Pickles"): known picked negative log softmax, then the gradient
// d/dW sum_j g_j * value_j = (softmax - onehot) * g against the closed form on the host.
template <typename S>
static void test_pick_nll(float eps) {
  auto W = Values<S>(gpu(), {{-0.5, 0.55, -0.45}, {1., 2., -1.}, {0., 0., 0.}, {0.3, -0.33, 1.3}});
  auto loss = PickNegLogSoftmax<S>(W, std::vector<Int>{3, 0, 1});
  Graph g(loss);
  g.forward();
  CHECK((loss->shape() == Shape{1, 3}));
  CHECK(close(loss->value().vector(), {1.43601264f, 1.8333567f, 2.73603603f}, eps));
  g.reset_grad();
  g.backward(2.);  // every column's loss weighted by 2
  const std::vector<float> sm = floats(loss->softmax().vector());
  std::vector<float> want(12);
  const int idx[3] = {3, 0, 1};
  for (int j = 0; j < 3; ++j)
    for (int i = 0; i < 4; ++i) want[i + 4 * j] = 2.f * (sm[i + 4 * j] - (i == idx[j] ? 1.f : 0.f));
  CHECK(close(W->grad().vector(), want, eps * 10, eps));
  // index count must match the columns
  bool threw = false;
  try {
    Graph(PickNegLogSoftmax<S>(W, std::vector<Int>{0, 1})).forward();
  } catch (const RuntimeError&) {
    threw = true;
  }
  CHECK(threw);
}

// test/nodes.cu.cpp:689-700: Softmax values; gradient of sum_ij c_ij y_ij against the closed form
// y (.) (c - colsum(y (.) c)), accumulated onto a non-zero gradient.
template <typename S>
static void test_softmax(float eps) {
  auto W = Values<S>(gpu(), {{-1, -2, -3}, {4, 5, 6}});
  auto y = Softmax<S>(W);
  Graph g(y);
  g.forward();
  CHECK(close(y->value().vector(),
              {0.00669285f, 0.99330715f, 9.11051194e-04f, 9.99088949e-01f, 1.23394576e-04f,
               9.99876605e-01f},
              eps * 10, eps));
  g.reset_grad();
  g.backward(0.5);  // c = 0.5 everywhere: y (.) (0.5 - 0.5 * colsum(y)) = 0 up to rounding
  for (float v : floats(W->grad().vector())) CHECK(std::fabs(v) <= eps);
}

// ginn/update/update.h:115-133 restated on the host in double, two steps.
static void test_adam() {
  auto w = Random<Real>(gpu(), {7, 5}, 70);
  update::Adam<Real> adam;  // lr 1e-3, clip 5, eps 1e-8, betas 0.9 / 0.999
  adam.init(w);
  std::vector<double> ref(35), m(35, 0.), v(35, 0.);
  const std::vector<Real> w0 = w->value().vector();
  for (int i = 0; i < 35; ++i) ref[i] = w0[i];
  double b1t = 1, b2t = 1;
  w->grad().resize(w->shape());
  for (int t = 0; t < 2; ++t) {
    std::vector<Real> d(35);
    for (int i = 0; i < 35; ++i) d[i] = 0.9f * (i - 17) * (t + 1);  // some beyond the clip
    w->grad().set(d);
    adam.update(w);
    b1t *= 0.9;
    b2t *= 0.999;
    for (int i = 0; i < 35; ++i) {
      const double dc = std::fmin(std::fmax(double(d[i]), -5.), 5.);
      m[i] = 0.9 * m[i] + 0.1 * dc;
      v[i] = 0.999 * v[i] + 0.001 * dc * dc;
      ref[i] += -1e-3 / (1 - b1t) * m[i] / (1e-8 + std::sqrt(v[i] / (1 - b2t)));
    }
    const std::vector<Real> dgot = w->grad().vector();
    for (int i = 0; i < 35; ++i) CHECK(std::fabs(dgot[i]) <= 5.f);  // clipped in place
  }
  std::vector<float> want(35);
  for (int i = 0; i < 35; ++i) want[i] = static_cast<float>(ref[i]);
  CHECK(close(w->value().vector(), want, 1e-6f, 1e-6f));
}

int main() {
  if (gpus() < 1) {
    std::printf("no GPU\n");
    return 2;
  }
  test_prod_known_answer<Real>(1e-6f);
  test_prod_known_answer<Half>(1e-2f);
  test_affine_known_answers<Real>(2e-6f);
  test_affine_known_answers<Half>(2e-3f);
  test_batched_prod_equals_slices<Real>(1e-5f);
  test_batched_prod_equals_slices<Half>(1e-2f);
  test_affine_cpu_vs_gpu<Real, IdentityOp>(GINN_B200_ACT_NONE, 1e-4f);
  test_affine_cpu_vs_gpu<Real, TanhOp>(GINN_B200_ACT_TANH, 1e-4f);
  test_affine_cpu_vs_gpu<Real, SigmoidOp>(GINN_B200_ACT_SIGMOID, 1e-4f);
  test_affine_cpu_vs_gpu<Real, ReluOp>(GINN_B200_ACT_RELU, 1e-4f);
  test_affine_cpu_vs_gpu<Half, TanhOp>(GINN_B200_ACT_TANH, 1e-2f);
  test_prod_cpu_vs_gpu();
  test_autobatch();
  test_autobatch_nonlinear_and_cells();
  test_conv2d();
  test_prealloc_accounting();
  test_errors();
  test_pick_nll<Real>(1e-6f);
  test_pick_nll<Half>(2e-3f);
  test_adam();
  test_softmax<Real>(1e-6f);
  test_softmax<Half>(1e-3f);
  cudaDeviceSynchronize();
  const int status = ginn_b200_device_status(0, 1);
  CHECK(status == 0);
  std::printf("%d checks, %d failed\n", g_checks, g_failed);
  return g_failed == 0 ? 0 : 1;
}
