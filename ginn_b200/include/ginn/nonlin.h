// Nonlinearity tags for Affine nodes.  The four ops ginn marks backward_requires_input() == false
// and that the GPU library fuses (ginn/nonlin.h:67-155) are represented; each knows the
// activation code of the C ABI.  Ops that need their input (Softmax, Log, Gelu...) are not part
// of this layer: an Affine with such an op passes ACT_NONE and runs ginn's own op afterwards.
#ifndef GINN_B200_HOST_NONLIN_H
#define GINN_B200_HOST_NONLIN_H

#include <memory>

#include <ginn_b200.h>

#include <ginn/def.h>

namespace ginn {

template <typename Scalar>
class NonlinOp {
 public:
  virtual ~NonlinOp() = default;
  virtual bool backward_requires_input() const { return false; }
  virtual bool is_identity() const { return false; }
  virtual int fused_act() const = 0;  // ginn_b200_act
  virtual std::unique_ptr<NonlinOp<Scalar>> copy() const = 0;
};

#define GINN_B200_FUSED_OP(NAME, ACT, IDENT)                                  \
  template <typename Scalar = Real>                                           \
  class NAME : public NonlinOp<Scalar> {                                      \
   public:                                                                    \
    bool is_identity() const override { return IDENT; }                       \
    int fused_act() const override { return ACT; }                            \
    std::unique_ptr<NonlinOp<Scalar>> copy() const override {                 \
      return std::make_unique<NAME<Scalar>>(*this);                           \
    }                                                                         \
  }

GINN_B200_FUSED_OP(IdentityOp, GINN_B200_ACT_NONE, true);
GINN_B200_FUSED_OP(TanhOp, GINN_B200_ACT_TANH, false);
GINN_B200_FUSED_OP(ReluOp, GINN_B200_ACT_RELU, false);
GINN_B200_FUSED_OP(SigmoidOp, GINN_B200_ACT_SIGMOID, false);

}  // namespace ginn
#endif
