// The Reduce kernel class, registered as "ReduceGPU(Default)".  A translation unit of its own because the
// reference's reduce.hpp declares unscoped operation codes (kMax, kMin, ...) that clash with those of
// binary.hpp and eltwise.hpp, exactly as in the reference's tree, where every kernel source includes
// only its own header.  See gpu_kernels.cpp.
#include "operators/kernels/reduce.hpp"

#include "gpu_kernels_common.hpp"

namespace Shadow {

namespace {

class ReduceKernelB200 : public ReduceKernel {
 public:
  void Run(const BlobPtr& input, BlobPtr& output, Workspace* ws, int operation, const VecInt& axes) override {
    CHECK(!axes.empty());
    const int rank = input->num_axes();
    const int64_t need = sb200_reduce_scratch_bytes(input->shape().data(), rank, axes.data(),
                                                    static_cast<int>(axes.size()), operation);
    CHECK_GE(need, 0) << "Reduce: bad axes";
    void* scratch = nullptr;
    if (need > 0) {
      ws->GrowTempBuffer(static_cast<size_t>(need) + 256);
      const int64_t ints = (need + 3) / 4;
      CHECK_LE(ints, 0x7fffffff);
      scratch = ws->CreateTempBlob({static_cast<int>(ints)}, DataType::kI32)->mutable_data<int>();
    }
    expect_ok(sb200_reduce(input->data<float>(), input->shape().data(), rank, axes.data(),
                           static_cast<int>(axes.size()), operation, output->mutable_data<float>(), scratch, need,
                           stream_of(ws)),
              "sb200_reduce");
  }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  std::string kernel_type() const override { return "Default"; }
};

}  // namespace

REGISTER_OP_KERNEL_DEFAULT(ReduceGPU, ReduceKernelB200);

}  // namespace Shadow
