// Error types and assertion macros with ginn's names and behaviour (ginn/except.h:23-54,
// ginn/cudef.h:23-59): failed assertions throw ginn::RuntimeError, CUDA failures ginn::CudaError.
#ifndef GINN_B200_HOST_EXCEPT_H
#define GINN_B200_HOST_EXCEPT_H

#include <cuda_runtime.h>
#include <stdexcept>
#include <string>

namespace ginn {

struct RuntimeError : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct CudaError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

}  // namespace ginn

#define GINN_B200_PICK(_1, _2, NAME, ...) NAME
#define GINN_ASSERT(...) GINN_B200_PICK(__VA_ARGS__, GINN_ASSERT_MSG, GINN_ASSERT_PLAIN)(__VA_ARGS__)
#define GINN_ASSERT_MSG(cond, msg)                  \
  do {                                              \
    if (!(cond)) throw ::ginn::RuntimeError(msg);   \
  } while (0)
#define GINN_ASSERT_PLAIN(cond) GINN_ASSERT_MSG(cond, "Assertion " #cond " failed!")
#define GINN_THROW(msg) throw ::ginn::RuntimeError(msg)
#define GINN_CUDA_THROW(msg) throw ::ginn::CudaError(msg)
#define GINN_CUDA_CALL(expr)                                                                   \
  do {                                                                                         \
    cudaError_t ginn_err_ = (expr);                                                            \
    if (ginn_err_ != cudaSuccess)                                                              \
      GINN_CUDA_THROW(std::string(#expr " failed: ") + cudaGetErrorString(ginn_err_) + " (" + \
                      __FILE__ + ":" + std::to_string(__LINE__) + ")");                        \
  } while (0)

#endif
