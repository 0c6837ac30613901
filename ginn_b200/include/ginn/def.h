// Scalar and shape vocabulary of the host layer (mirrors ginn/def.h:31-39 of ginn).
#ifndef GINN_B200_HOST_DEF_H
#define GINN_B200_HOST_DEF_H

#include <cuda_fp16.h>
#include <cstddef>
#include <vector>

namespace ginn {

using Real = float;   // ginn's GINN_DOUBLE_PRECISION mode never reaches a GPU (ginn/prod.h:63-65)
using Half = __half;  // bit-compatible with Eigen::half, which ginn reinterprets as __half
using Int = int;
using Size = long;
using Shape = std::vector<Size>;

}  // namespace ginn
#endif
