// internal::gpu_prod / gpu_batched_prod with ginn's signatures, shape algebra and assertions
// (ginn/prod.h:207-310), routed to libginn_b200.so instead of cuBLAS.
#ifndef GINN_B200_HOST_PROD_H
#define GINN_B200_HOST_PROD_H

#include <type_traits>

#include <ginn_b200.h>

#include <ginn/tensor.h>

namespace ginn {
namespace internal {

enum class ProdResult { Assign, Add };
enum class ProdTranspose { None, First, Second, Both };

template <typename Scalar>
constexpr int b200_dtype() {
  static_assert(std::is_same<Scalar, Real>::value || std::is_same<Scalar, Half>::value,
                "Unexpected Scalar type in gpu_gemm!");
  return std::is_same<Scalar, Real>::value ? GINN_B200_F32 : GINN_B200_F16;
}

inline void b200_check(int status) {
  if (status == GINN_B200_BAD_ARGUMENT) GINN_THROW(ginn_b200_last_error());
  if (status != GINN_B200_OK) GINN_CUDA_THROW(ginn_b200_last_error());
}

inline int b200_device(const DevPtr& dev) {
  GINN_ASSERT(dev->kind() == GPU, "gpu_prod needs tensors on a GPU device");
  return static_cast<int>(dev->id().idx);
}

// C = A * B
template <typename Scalar>
inline void gpu_prod(Tensor<Scalar>& c, Tensor<Scalar>& a, Tensor<Scalar>& b,
                     ProdResult res = ProdResult::Assign,
                     ProdTranspose tra = ProdTranspose::None) {
  const bool ta = tra == ProdTranspose::First || tra == ProdTranspose::Both;
  const bool tb = tra == ProdTranspose::Second || tra == ProdTranspose::Both;
  const Size a_outer = ta ? a.cols() : a.rows(), a_inner = ta ? a.rows() : a.cols();
  const Size b_outer = tb ? b.rows() : b.cols(), b_inner = tb ? b.cols() : b.rows();
  GINN_ASSERT(a_inner == b_inner);
  GINN_ASSERT(a_outer == c.rows());
  GINN_ASSERT(b_outer == c.cols());
  const int dev = b200_device(c.dev());
  b200_check(ginn_b200_gemm(dev, stream_of(*c.dev()), b200_dtype<Scalar>(), ta, tb, a_outer,
                            b_outer, a_inner, a.data(), a.rows(), b.data(), b.rows(), c.data(),
                            c.rows(), res == ProdResult::Add));
}

// C[:,:,i] = A[:,:,i] * B[:,:,i] for every i; ranks above 3 fold into the batch index.
template <typename Scalar>
inline void gpu_batched_prod(Tensor<Scalar>& c, Tensor<Scalar>& a, Tensor<Scalar>& b,
                             ProdResult res = ProdResult::Assign,
                             ProdTranspose tra = ProdTranspose::None) {
  const Shape as = Tensor<Scalar>::reduce(a.shape(), 3), bs = Tensor<Scalar>::reduce(b.shape(), 3),
              cs = Tensor<Scalar>::reduce(c.shape(), 3);
  const bool ta = tra == ProdTranspose::First || tra == ProdTranspose::Both;
  const bool tb = tra == ProdTranspose::Second || tra == ProdTranspose::Both;
  const Size a_outer = ta ? as[1] : as[0], a_inner = ta ? as[0] : as[1];
  const Size b_outer = tb ? bs[0] : bs[1], b_inner = tb ? bs[1] : bs[0];
  GINN_ASSERT(a_inner == b_inner);
  GINN_ASSERT(a_outer == cs[0]);
  GINN_ASSERT(b_outer == cs[1]);
  const int dev = b200_device(c.dev());
  b200_check(ginn_b200_gemm_batched(dev, stream_of(*c.dev()), b200_dtype<Scalar>(), ta, tb,
                                    a_outer, b_outer, a_inner, a.data(), as[0], as[0] * as[1],
                                    b.data(), bs[0], bs[0] * bs[1], c.data(), cs[0],
                                    a_outer * b_outer, as[2], res == ProdResult::Add));
}

// Both gradient products of C = A * B in one call (ProdNode::backward_, ginn/node/prod.h:51-66):
// da += dc * B^T and db += A^T * dc; a null `da` / `db` skips that product.  The library runs the
// two side by side when their outputs do not overlap.
template <typename Scalar>
inline void gpu_prod_backward(Tensor<Scalar>* da, Tensor<Scalar>* db, Tensor<Scalar>& dc,
                              Tensor<Scalar>& a, Tensor<Scalar>& b) {
  GINN_ASSERT(a.cols() == b.rows());
  GINN_ASSERT(a.rows() == dc.rows());
  GINN_ASSERT(b.cols() == dc.cols());
  if (da) GINN_ASSERT(da->rows() == a.rows() && da->cols() == a.cols());
  if (db) GINN_ASSERT(db->rows() == b.rows() && db->cols() == b.cols());
  const int dev = b200_device(dc.dev());
  b200_check(ginn_b200_prod_backward(dev, stream_of(*dc.dev()), b200_dtype<Scalar>(), a.rows(),
                                     b.cols(), a.cols(), 1, a.data(), a.rows(), 0, b.data(),
                                     b.rows(), 0, dc.data(), dc.rows(), 0,
                                     da ? da->data() : nullptr, a.rows(), 0,
                                     db ? db->data() : nullptr, b.rows(), 0));
}

// The batched form (BatchedProdNode::backward_, ginn/node/prod.h:118-130); ranks above 3 fold
// into the batch index.
template <typename Scalar>
inline void gpu_batched_prod_backward(Tensor<Scalar>* da, Tensor<Scalar>* db, Tensor<Scalar>& dc,
                                      Tensor<Scalar>& a, Tensor<Scalar>& b) {
  const Shape as = Tensor<Scalar>::reduce(a.shape(), 3), bs = Tensor<Scalar>::reduce(b.shape(), 3),
              cs = Tensor<Scalar>::reduce(dc.shape(), 3);
  GINN_ASSERT(as[1] == bs[0]);
  GINN_ASSERT(as[0] == cs[0]);
  GINN_ASSERT(bs[1] == cs[1]);
  GINN_ASSERT(as[2] == bs[2] && as[2] == cs[2]);
  if (da) GINN_ASSERT(da->size() == a.size());
  if (db) GINN_ASSERT(db->size() == b.size());
  const int dev = b200_device(dc.dev());
  b200_check(ginn_b200_prod_backward(dev, stream_of(*dc.dev()), b200_dtype<Scalar>(), as[0], bs[1],
                                     as[1], as[2], a.data(), as[0], as[0] * as[1], b.data(), bs[0],
                                     bs[0] * bs[1], dc.data(), cs[0], cs[0] * cs[1],
                                     da ? da->data() : nullptr, as[0], as[0] * as[1],
                                     db ? db->data() : nullptr, bs[0], bs[0] * bs[1]));
}

}  // namespace internal
}  // namespace ginn
#endif
