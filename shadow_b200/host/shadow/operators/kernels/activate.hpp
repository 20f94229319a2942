// Same include path as the reference (shadow/operators/kernels/activate.hpp); the abstract kernel
// interfaces of the six operators live in op_kernels.hpp.
#include "../../op_kernels.hpp"
