// The GPU kernel classes (every operator except Reduce and Eltwise, which sit in gpu_kernels_reduce.cpp and
// gpu_kernels_eltwise.cpp), registered as "<Op>GPU(Default)".  Each Run translates blobs into
// the raw pointers / sizes of the sb200 C ABI and enqueues on the workspace's stream.  A non-zero
// status becomes a LOG(FATAL) (print + std::runtime_error), the reference's error convention.
// There is no other implementation behind these classes: without libsb200 this file does not link.
//
// The file uses only what the reference's own headers offer (shadow/core/{blob,workspace,kernel}.hpp
// and shadow/operators/kernels/<op>.hpp: the abstract XxxKernel classes, Blob::count/shape/data,
// Workspace::Ctx/GrowTempBuffer/CreateTempBlob, Context::stream, REGISTER_OP_KERNEL_DEFAULT), so the
// same translation unit compiles inside the reference's tree (-I<reference>/shadow) and registers
// there under the same keys; tests/test_reference_binding.py compiles it both ways.
#include "operators/kernels/activate.hpp"
#include "operators/kernels/axpy.hpp"
#include "operators/kernels/batch_norm.hpp"
#include "operators/kernels/binary.hpp"
#include "operators/kernels/concat.hpp"
#include "operators/kernels/gather.hpp"
#include "operators/kernels/group_norm.hpp"
#include "operators/kernels/layer_norm.hpp"
#include "operators/kernels/normalize.hpp"
#include "operators/kernels/pad.hpp"
#include "operators/kernels/permute.hpp"
#include "operators/kernels/pooling.hpp"
#include "operators/kernels/scale.hpp"
#include "operators/kernels/slice.hpp"
#include "operators/kernels/softmax.hpp"
#include "operators/kernels/ssd_normalize.hpp"
#include "operators/kernels/stack.hpp"
#include "operators/kernels/unary.hpp"

#include "gpu_kernels_common.hpp"

namespace Shadow {

namespace {

class BinaryKernelB200 : public BinaryKernel {
 public:
  void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, int operation, float scalar_value) override {
    expect_ok(sb200_binary_scalar(input->data<float>(), scalar_value, output->mutable_data<float>(),
                                  count64(input), operation, stream_of(ws)),
              "sb200_binary_scalar");
  }
  void Run(const BlobPtr& input, const BlobPtr& scalar, BlobPtr& output, Workspace* ws, int operation,
           bool need_broadcast) override {
    if (need_broadcast) {
      // shapes stay on the host: no temp buffer, no upload
      expect_ok(sb200_binary_broadcast(input->data<float>(), input->shape().data(), scalar->data<float>(),
                                       scalar->shape().data(), output->shape().data(), input->num_axes(),
                                       output->mutable_data<float>(), operation, stream_of(ws)),
                "sb200_binary_broadcast");
    } else {
      expect_ok(sb200_binary(input->data<float>(), scalar->data<float>(), output->mutable_data<float>(),
                             count64(input), operation, stream_of(ws)),
                "sb200_binary");
    }
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

class UnaryKernelB200 : public UnaryKernel {
 public:
  void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, int operation) override {
    expect_ok(sb200_unary(input->data<float>(), output->mutable_data<float>(),
                          count64(input), operation, stream_of(ws)),
              "sb200_unary");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

class ActivateKernelB200 : public ActivateKernel {
 public:
  void Run(const BlobPtr& input, const BlobPtr& slope, BlobPtr& output, Workspace* ws, int activate_type,
           float slope_val) override {
    if (activate_type == 0 /* kPRelu, shadow/operators/kernels/activate.hpp:25 */) {
      CHECK_GE(input->num_axes(), 2);
      CHECK_NOTNULL(slope);
      const bool channel_shared = slope->count() == 1;
      if (!channel_shared) CHECK_EQ(slope->count(), input->shape(1));
      int64_t dim = 1;
      for (int n = 2; n < input->num_axes(); ++n) dim *= input->shape(n);
      expect_ok(sb200_prelu(input->data<float>(), output->mutable_data<float>(), input->shape(0), input->shape(1),
                            dim, slope->data<float>(), channel_shared ? 1 : 0, stream_of(ws)),
                "sb200_prelu");
    } else {
      expect_ok(sb200_activate(input->data<float>(), output->mutable_data<float>(),
                               count64(output), activate_type, slope_val, stream_of(ws)),
                "sb200_activate");
    }
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

class ScaleKernelB200 : public ScaleKernel {
 public:
  void Run(const BlobPtr& input, const BlobPtr& scale, const BlobPtr& bias, BlobPtr& output, Workspace* ws,
           int axis) override {
    CHECK(scale != nullptr || bias != nullptr);
    if (scale != nullptr && bias != nullptr) CHECK(scale->shape() == bias->shape());
    const BlobPtr& ref = scale != nullptr ? scale : bias;
    const int inner = input->count(axis + ref->num_axes());
    expect_ok(sb200_scale_bias(input->data<float>(), output->mutable_data<float>(),
                               count64(input), scale ? scale->data<float>() : nullptr,
                               bias ? bias->data<float>() : nullptr, ref->count(), inner, stream_of(ws)),
              "sb200_scale_bias");
  }

  // Value form: the vectors are uploaded into the workspace temp buffer on every call, as the
  // reference does (shadow/operators/kernels/scale.hpp:73-110).
  void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, int axis, const VecFloat& scale_value,
           const VecFloat& bias_value) override {
    const int dim = input->shape(axis), inner = input->count(axis + 1);
    CHECK(!scale_value.empty() || !bias_value.empty());
    if (!scale_value.empty()) CHECK_EQ(static_cast<int>(scale_value.size()), dim);
    if (!bias_value.empty()) CHECK_EQ(static_cast<int>(bias_value.size()), dim);
    ws->GrowTempBuffer(2 * (static_cast<size_t>(dim) * sizeof(float) + 256));
    BlobPtr scale, bias;
    if (!scale_value.empty()) {
      scale = ws->CreateTempBlob({dim}, DataType::kF32);
      scale->set_data<float>(scale_value.data(), dim);
    }
    if (!bias_value.empty()) {
      bias = ws->CreateTempBlob({dim}, DataType::kF32);
      bias->set_data<float>(bias_value.data(), dim);
    }
    expect_ok(sb200_scale_bias(input->data<float>(), output->mutable_data<float>(),
                               count64(input), scale ? scale->data<float>() : nullptr,
                               bias ? bias->data<float>() : nullptr, dim, inner, stream_of(ws)),
              "sb200_scale_bias");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

class SoftmaxKernelB200 : public SoftmaxKernel {
 public:
  void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, int axis) override {
    const int64_t outer = input->count(0, axis), dim = input->shape(axis), inner = input->count(axis + 1);
    expect_ok(sb200_softmax(input->data<float>(), output->mutable_data<float>(), outer, dim, inner, stream_of(ws)),
              "sb200_softmax");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

class AxpyKernelB200 : public AxpyKernel {
 public:
  void Run(const BlobPtr& alpha, const BlobPtr& x, const BlobPtr& y, BlobPtr& output, Workspace* ws) override {
    expect_ok(sb200_axpy(alpha->data<float>(), x->data<float>(), y->data<float>(), output->mutable_data<float>(),
                         count64(alpha), x->count(2), stream_of(ws)),
              "sb200_axpy");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

// ---- data movement: one launch moves every part (the reference launches once per input/output)
class ConcatKernelB200 : public ConcatKernel {
 public:
  void Run(const std::vector<BlobPtr>& inputs, BlobPtr& output, Workspace* ws, int axis) override {
    std::vector<const float*> ptrs;
    std::vector<int64_t> widths;
    const int64_t inner = output->count(axis + 1);
    for (const auto& in : inputs) {
      ptrs.push_back(in->data<float>());
      widths.push_back(in->shape(axis) * inner);
    }
    expect_ok(sb200_concat(ptrs.data(), widths.data(), static_cast<int>(ptrs.size()), output->mutable_data<float>(),
                           output->count(0, axis), stream_of(ws)),
              "sb200_concat");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

class StackKernelB200 : public StackKernel {
 public:
  void Run(const std::vector<BlobPtr>& inputs, BlobPtr& output, Workspace* ws, int axis) override {
    std::vector<const float*> ptrs;
    const int64_t size = output->count(axis + 1);
    for (const auto& in : inputs) ptrs.push_back(in->data<float>());
    std::vector<int64_t> widths(ptrs.size(), size);
    expect_ok(sb200_concat(ptrs.data(), widths.data(), static_cast<int>(ptrs.size()), output->mutable_data<float>(),
                           output->count(0, axis), stream_of(ws)),
              "sb200_concat");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

class SliceKernelB200 : public SliceKernel {
 public:
  void Run(const BlobPtr& input, std::vector<BlobPtr>& outputs, Workspace* ws, int axis) override {
    std::vector<float*> ptrs;
    std::vector<int64_t> widths;
    const int64_t inner = input->count(axis + 1);
    for (auto& out : outputs) {
      ptrs.push_back(out->mutable_data<float>());
      widths.push_back(out->shape(axis) * inner);
    }
    expect_ok(sb200_slice(input->data<float>(), ptrs.data(), widths.data(), static_cast<int>(ptrs.size()),
                          input->count(0, axis), stream_of(ws)),
              "sb200_slice");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

class PermuteKernelB200 : public PermuteKernel {
 public:
  // shapes and order stay on the host: no temporary blobs
  void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, const VecInt& order_value) override {
    expect_ok(sb200_permute(input->data<float>(), output->mutable_data<float>(), input->shape().data(), order_value.data(),
                            input->num_axes(), stream_of(ws)),
              "sb200_permute");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

class GatherKernelB200 : public GatherKernel {
 public:
  void Run(const BlobPtr& input, const BlobPtr& indexes, BlobPtr& output, Workspace* ws, int axis) override {
    expect_ok(sb200_gather(input->data<float>(), indexes->data<int>(), indexes->count(), input->count(0, axis),
                           input->shape(axis), input->count(axis + 1), output->mutable_data<float>(), stream_of(ws)),
              "sb200_gather");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

class PadKernelB200 : public PadKernel {
 public:
  void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, const VecInt& paddings, float value) override {
    CHECK_EQ(input->num_axes(), 4);
    CHECK_EQ(paddings.size(), 4u);
    expect_ok(sb200_pad(input->data<float>(), output->mutable_data<float>(),
                        static_cast<int64_t>(input->shape(0)) * input->shape(1), input->shape(2), input->shape(3),
                        paddings.data(), value, stream_of(ws)),
              "sb200_pad");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

class PoolingKernelB200 : public PoolingKernel {
 public:
  void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, int pool_type, int kernel_size_h, int kernel_size_w,
           int stride_h, int stride_w, int pad_h, int pad_w, bool) override {
    const int in[3] = {1, input->shape(2), input->shape(3)}, out[3] = {1, output->shape(2), output->shape(3)};
    const int k[3] = {1, kernel_size_h, kernel_size_w}, st[3] = {1, stride_h, stride_w}, pd[3] = {0, pad_h, pad_w};
    expect_ok(sb200_pooling(input->data<float>(), output->mutable_data<float>(),
                            static_cast<int64_t>(input->shape(0)) * input->shape(1), in, out, k, st, pd, pool_type, stream_of(ws)),
              "sb200_pooling");
  }
  void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, int pool_type, int kernel_size_d, int kernel_size_h,
           int kernel_size_w, int stride_d, int stride_h, int stride_w, int pad_d, int pad_h, int pad_w, bool) override {
    const int in[3] = {input->shape(2), input->shape(3), input->shape(4)};
    const int out[3] = {output->shape(2), output->shape(3), output->shape(4)};
    const int k[3] = {kernel_size_d, kernel_size_h, kernel_size_w}, st[3] = {stride_d, stride_h, stride_w};
    const int pd[3] = {pad_d, pad_h, pad_w};
    expect_ok(sb200_pooling(input->data<float>(), output->mutable_data<float>(),
                            static_cast<int64_t>(input->shape(0)) * input->shape(1), in, out, k, st, pd, pool_type, stream_of(ws)),
              "sb200_pooling");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

// One launch; the shared scale is read on the device (the reference copies it to the host first).
class SSDNormalizeKernelB200 : public SSDNormalizeKernel {
 public:
  void Run(const BlobPtr& input, const BlobPtr& scale, BlobPtr& output, Workspace* ws, bool across_spatial,
           bool channel_shared, float eps) override {
    const int channel = input->shape(1);
    if (scale != nullptr) CHECK_EQ(scale->count(), channel_shared ? 1 : channel);
    expect_ok(sb200_ssd_normalize(input->data<float>(), output->mutable_data<float>(), input->shape(0), channel,
                                  input->count(2), across_spatial ? 1 : 0, eps,
                                  scale != nullptr ? scale->data<float>() : nullptr, channel_shared ? 1 : 0, stream_of(ws)),
              "sb200_ssd_normalize");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

// One fused launch and no temporary blobs (the reference grows the workspace by count + inner +
// 2*rows floats and makes six launches).
class GroupNormKernelB200 : public GroupNormKernel {
 public:
  void Run(const BlobPtr& input, const BlobPtr& scale, const BlobPtr& bias, BlobPtr& output, Workspace* ws, int group,
           float eps) override {
    const int64_t count = count64(input);
    const int64_t rows = static_cast<int64_t>(input->shape(0)) * group, inner = count / rows;
    const bool affine = scale != nullptr && bias != nullptr;
    const int channel = input->shape(1);
    if (affine) {
      CHECK_EQ(scale->count(), channel);
      CHECK_EQ(bias->count(), channel);
    }
    expect_ok(sb200_row_norm(input->data<float>(), output->mutable_data<float>(), rows, inner, eps,
                             affine ? scale->data<float>() : nullptr, affine ? bias->data<float>() : nullptr,
                             affine ? 2 : 0, group, channel / group, input->count(2), stream_of(ws)),
              "sb200_row_norm");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

class LayerNormKernelB200 : public LayerNormKernel {
 public:
  void Run(const BlobPtr& input, const BlobPtr& scale, const BlobPtr& bias, BlobPtr& output, Workspace* ws,
           const VecInt& normalized_shape, float eps) override {
    const int64_t inner = input->count(input->num_axes() - static_cast<int>(normalized_shape.size()));
    const int64_t rows = count64(input) / inner;
    const bool affine = scale != nullptr && bias != nullptr;
    if (affine) {
      CHECK(scale->shape() == normalized_shape);
      CHECK(bias->shape() == normalized_shape);
    }
    expect_ok(sb200_row_norm(input->data<float>(), output->mutable_data<float>(), rows, inner, eps,
                             affine ? scale->data<float>() : nullptr, affine ? bias->data<float>() : nullptr,
                             affine ? 1 : 0, 1, 1, 1, stream_of(ws)),
              "sb200_row_norm");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

class NormalizeKernelB200 : public NormalizeKernel {
 public:
  // no temporary blob: the norms stay on chip (the reference grows the workspace by outer*inner floats)
  void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, float p, int axis, float eps) override {
    const int64_t outer = input->count(0, axis), dim = input->shape(axis), inner = input->count(axis + 1);
    expect_ok(sb200_normalize(input->data<float>(), output->mutable_data<float>(), outer, dim, inner, p, eps,
                              stream_of(ws)),
              "sb200_normalize");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

class BatchNormKernelB200 : public BatchNormKernel {
 public:
  void Run(const BlobPtr& input, const BlobPtr& mean, const BlobPtr& variance, BlobPtr& output, Workspace* ws,
           float scale_factor, float eps) override {
    const int channel = input->shape(1);
    CHECK_EQ(channel, mean->count());
    CHECK_EQ(channel, variance->count());
    expect_ok(sb200_batch_norm(input->data<float>(), output->mutable_data<float>(),
                               count64(input), mean->data<float>(), variance->data<float>(),
                               channel, input->count(2), scale_factor, eps, stream_of(ws)),
              "sb200_batch_norm");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

}  // namespace

REGISTER_OP_KERNEL_DEFAULT(BatchNormGPU, BatchNormKernelB200);
REGISTER_OP_KERNEL_DEFAULT(NormalizeGPU, NormalizeKernelB200);
REGISTER_OP_KERNEL_DEFAULT(ConcatGPU, ConcatKernelB200);
REGISTER_OP_KERNEL_DEFAULT(StackGPU, StackKernelB200);
REGISTER_OP_KERNEL_DEFAULT(SliceGPU, SliceKernelB200);
REGISTER_OP_KERNEL_DEFAULT(PermuteGPU, PermuteKernelB200);
REGISTER_OP_KERNEL_DEFAULT(GatherGPU, GatherKernelB200);
REGISTER_OP_KERNEL_DEFAULT(PadGPU, PadKernelB200);
REGISTER_OP_KERNEL_DEFAULT(PoolingGPU, PoolingKernelB200);
REGISTER_OP_KERNEL_DEFAULT(SSDNormalizeGPU, SSDNormalizeKernelB200);
REGISTER_OP_KERNEL_DEFAULT(GroupNormGPU, GroupNormKernelB200);
REGISTER_OP_KERNEL_DEFAULT(LayerNormGPU, LayerNormKernelB200);
REGISTER_OP_KERNEL_DEFAULT(AxpyGPU, AxpyKernelB200);
REGISTER_OP_KERNEL_DEFAULT(BinaryGPU, BinaryKernelB200);
REGISTER_OP_KERNEL_DEFAULT(UnaryGPU, UnaryKernelB200);
REGISTER_OP_KERNEL_DEFAULT(ActivateGPU, ActivateKernelB200);
REGISTER_OP_KERNEL_DEFAULT(ScaleGPU, ScaleKernelB200);
REGISTER_OP_KERNEL_DEFAULT(SoftmaxGPU, SoftmaxKernelB200);

}  // namespace Shadow
