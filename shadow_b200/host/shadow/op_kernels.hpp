// Abstract kernel interfaces of the six operators and their operation codes.  These are the
// reference's own signatures (the drop-in boundary): a class deriving one of them and registered
// under "<Op>GPU(Default)" is what an operator front-end obtains from CreateKernel.
//   BinaryKernel    shadow/operators/kernels/binary.hpp:23-35
//   UnaryKernel     shadow/operators/kernels/unary.hpp:9-32
//   ActivateKernel  shadow/operators/kernels/activate.hpp:24-42
//   ScaleKernel     shadow/operators/kernels/scale.hpp:29-39
//   ReduceKernel    shadow/operators/kernels/reduce.hpp:21-36
//   SoftmaxKernel   shadow/operators/kernels/softmax.hpp:20-24
// Output blobs arrive already reshaped by the operator front-end.
#ifndef SHADOW_B200_HOST_OP_KERNELS_HPP_
#define SHADOW_B200_HOST_OP_KERNELS_HPP_

#include "shadow_api.hpp"

namespace Shadow {

// Binary and Reduce both define kMax / kMin with different values in the reference (each in its
// own translation unit); here they are scoped to keep one header.
namespace BinaryCode { enum { kAdd = 0, kSub = 1, kMul = 2, kDiv = 3, kPow = 4, kMax = 5, kMin = 6 }; }
namespace UnaryCode {
enum { kAbs = 0, kSquare, kSqrt, kLog, kExp, kSin, kCos, kTan, kAsin, kAcos, kAtan, kFloor, kCeil, kNeg, kReciprocal };
}
namespace ActivateCode {
enum { kPRelu = 0, kRelu, kLeaky, kSigmoid, kSoftPlus, kTanh, kRelu6, kHardSwish, kGelu };
}
namespace ReduceCode { enum { kProd = 0, kSum, kMax, kMin, kAvg, kLpNorm1, kLpNorm2 }; }

using BlobPtr = std::shared_ptr<Blob>;

class BinaryKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, int operation, float scalar_value) = 0;
  virtual void Run(const BlobPtr& input, const BlobPtr& scalar, BlobPtr& output, Workspace* ws, int operation,
                   bool need_broadcast) = 0;
};

class UnaryKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, int operation) = 0;
};

class ActivateKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, const BlobPtr& slope, BlobPtr& output, Workspace* ws, int activate_type,
                   float slope_val) = 0;
};

class ScaleKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, const BlobPtr& scale, const BlobPtr& bias, BlobPtr& output, Workspace* ws,
                   int axis) = 0;
  virtual void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, int axis, const VecFloat& scale_value,
                   const VecFloat& bias_value) = 0;
};

class ReduceKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, int operation, const VecInt& axes) = 0;
};

// shadow/operators/kernels/eltwise.hpp:11-17 (codes Prod 0, Sum 1, Max 2, Min 3)
class EltwiseKernel : public Kernel {
 public:
  virtual void Run(const std::vector<BlobPtr>& inputs, BlobPtr& output, Workspace* ws, int operation,
                   const VecFloat& coeff) = 0;
};

// shadow/operators/kernels/axpy.hpp:20-27
class AxpyKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& alpha, const BlobPtr& x, const BlobPtr& y, BlobPtr& output, Workspace* ws) = 0;
};

// shadow/operators/kernels/concat.hpp:19-24, stack.hpp:18-23
class ConcatKernel : public Kernel {
 public:
  virtual void Run(const std::vector<BlobPtr>& inputs, BlobPtr& output, Workspace* ws, int axis) = 0;
};
class StackKernel : public Kernel {
 public:
  virtual void Run(const std::vector<BlobPtr>& inputs, BlobPtr& output, Workspace* ws, int axis) = 0;
};
// shadow/operators/kernels/slice.hpp:19-25
class SliceKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, std::vector<BlobPtr>& outputs, Workspace* ws, int axis) = 0;
};
// shadow/operators/kernels/permute.hpp:18-23
class PermuteKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, const VecInt& order_value) = 0;
};
// shadow/operators/kernels/gather.hpp:16-22
class GatherKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, const BlobPtr& indexes, BlobPtr& output, Workspace* ws, int axis) = 0;
};
// shadow/operators/kernels/pad.hpp:18-24
class PadKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, const VecInt& paddings, float value) = 0;
};

// shadow/operators/kernels/pooling.hpp:29-42
class PoolingKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, int pool_type, int kernel_size_h, int kernel_size_w,
                   int stride_h, int stride_w, int pad_h, int pad_w, bool full_pooling) = 0;
  virtual void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, int pool_type, int kernel_size_d, int kernel_size_h,
                   int kernel_size_w, int stride_d, int stride_h, int stride_w, int pad_d, int pad_h, int pad_w,
                   bool full_pooling) = 0;
};

// shadow/operators/kernels/ssd_normalize.hpp:24-30
class SSDNormalizeKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, const BlobPtr& scale, BlobPtr& output, Workspace* ws, bool across_spatial,
                   bool channel_shared, float eps) = 0;
};

// shadow/operators/kernels/group_norm.hpp:30-37 (also used by InstanceNorm with group = channels)
class GroupNormKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, const BlobPtr& scale, const BlobPtr& bias, BlobPtr& output, Workspace* ws,
                   int group, float eps) = 0;
};

// shadow/operators/kernels/layer_norm.hpp:8-16
class LayerNormKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, const BlobPtr& scale, const BlobPtr& bias, BlobPtr& output, Workspace* ws,
                   const VecInt& normalized_shape, float eps) = 0;
};

// shadow/operators/kernels/normalize.hpp:20-25
class NormalizeKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, float p, int axis, float eps) = 0;
};

// shadow/operators/kernels/batch_norm.hpp:20-28
class BatchNormKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, const BlobPtr& mean, const BlobPtr& variance, BlobPtr& output, Workspace* ws,
                   float scale_factor, float eps) = 0;
};

class SoftmaxKernel : public Kernel {
 public:
  virtual void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, int axis) = 0;
};

}  // namespace Shadow

#endif  // SHADOW_B200_HOST_OP_KERNELS_HPP_
