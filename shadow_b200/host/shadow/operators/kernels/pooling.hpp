// Same include path as the reference (shadow/operators/kernels/pooling.hpp); the abstract kernel
// interfaces live in op_kernels.hpp.
#include "../../op_kernels.hpp"
