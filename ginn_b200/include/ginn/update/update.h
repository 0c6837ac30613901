// Adam with ginn's interface (ginn/update/update.h:85-155): per-weight histories m, v (always
// Real) keyed by an id, the bias-correction powers advanced once per update, the gradient
// clipped in place.  The whole update of one weight is one kernel of libginn_b200.so.
#ifndef GINN_B200_HOST_UPDATE_H
#define GINN_B200_HOST_UPDATE_H

#include <mutex>
#include <unordered_map>

#include <ginn/node/data.h>
#include <ginn/prod.h>

namespace ginn {
namespace update {

template <typename Scalar = Real>
class Adam {
 public:
  struct History {
    Tensor<Real> m, v;
    Real beta_1_t = 1, beta_2_t = 1;
  };

  std::unordered_map<size_t, History> weight_histories;
  std::mutex history_access;
  Real lr_, eps_, beta_1_, beta_2_, clip_;

  Adam(Real lr = 1e-3, Real clip = 5., Real eps = 1e-8, Real beta_1 = 0.9, Real beta_2 = 0.999)
      : lr_(lr), eps_(eps), beta_1_(beta_1), beta_2_(beta_2), clip_(clip) {}

  // Zeroed histories for the weight `id` (the reference keys them by WeightNode::id()).
  void init(const Tensor<Scalar>& w, size_t id) {
    GINN_ASSERT(w.size() > 0);
    History h{Tensor<Real>(w.dev(), w.shape()), Tensor<Real>(w.dev(), w.shape()), 1, 1};
    h.m.set_zero();
    h.v.set_zero();
    std::lock_guard<std::mutex> l(history_access);
    weight_histories.erase(id);
    weight_histories.emplace(id, std::move(h));
  }

  void update(Tensor<Scalar>& w, Tensor<Scalar>& d, size_t id) {
    GINN_ASSERT(w.dev()->kind() == GPU, "ginn_b200 serves GPU devices only");
    GINN_ASSERT(w.size() == d.size(), "weight and gradient differ in size");
    History* h;
    {
      std::lock_guard<std::mutex> l(history_access);
      auto it = weight_histories.find(id);
      GINN_ASSERT(it != weight_histories.end(), "Adam::update before Adam::init for this weight");
      h = &it->second;
    }
    h->beta_1_t *= beta_1_;
    h->beta_2_t *= beta_2_;
    internal::b200_check(ginn_b200_adam_update(
        static_cast<int>(w.dev()->id().idx), stream_of(*w.dev()), internal::b200_dtype<Scalar>(),
        w.size(), w.data(), d.data(), h->m.data(), h->v.data(), lr_, clip_, eps_, beta_1_, beta_2_,
        h->beta_1_t, h->beta_2_t));
  }

  // A node that owns value and gradient; its address is the history key.
  void init(const DataPtr<Scalar>& w) { init(w->value(), reinterpret_cast<size_t>(w.get())); }
  void update(const DataPtr<Scalar>& w) {
    if (w->has_grad()) update(w->value(), w->grad(), reinterpret_cast<size_t>(w.get()));
  }
};

}  // namespace update
}  // namespace ginn
#endif
