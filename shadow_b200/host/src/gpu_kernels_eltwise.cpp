// The Eltwise kernel class, registered as "EltwiseGPU(Default)".  A translation unit of its own because the
// reference's eltwise.hpp declares unscoped operation codes (kMax, kMin, ...) that clash with those of
// binary.hpp and reduce.hpp, exactly as in the reference's tree, where every kernel source includes
// only its own header.  See gpu_kernels.cpp.
#include "operators/kernels/eltwise.hpp"

#include "gpu_kernels_common.hpp"

namespace Shadow {

namespace {

class EltwiseKernelB200 : public EltwiseKernel {
 public:
  void Run(const std::vector<BlobPtr>& inputs, BlobPtr& output, Workspace* ws, int operation,
           const VecFloat& coeff) override {
    std::vector<const float*> ptrs;
    for (const auto& in : inputs) ptrs.push_back(in->data<float>());
    // the front-end always passes one coefficient per input (1 by default); only Sum uses them
    const float* cf = (operation == 1 && coeff.size() == inputs.size()) ? coeff.data() : nullptr;
    expect_ok(sb200_eltwise(ptrs.data(), static_cast<int>(ptrs.size()), cf, output->mutable_data<float>(),
                            count64(inputs[0]), operation, stream_of(ws)),
              "sb200_eltwise");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

}  // namespace

REGISTER_OP_KERNEL_DEFAULT(EltwiseGPU, EltwiseKernelB200);

}  // namespace Shadow
