// Operator front-ends of the six tensor operators (+ Input): argument parsing, shape inference and
// the checks the reference makes, then one call into the registered kernel.  Argument names,
// defaults and failure conditions follow shadow/operators/{binary,unary,activate,scale,reduce,
// softmax,input}_op.cpp.
#include <algorithm>
#include <cmath>

#include "op_kernels.hpp"

namespace Shadow {

namespace {

template <typename K>
std::shared_ptr<K> kernel_for(const shadow::OpParam& op_param, Workspace* ws) {
  auto kernel = std::dynamic_pointer_cast<K>(CreateKernel(op_param.type(), ws->Ctx()->device_type()));
  CHECK_NOTNULL(kernel);
  return kernel;
}

// Input: a pure placeholder; the backend shapes its tops from the v_i arguments named after them
// (shadow/operators/input_op.cpp:7-17).
class InputOp : public Operator {
 public:
  using Operator::Operator;
  void Run(const std::vector<BlobPtr>&, std::vector<BlobPtr>&) override {}
};

// Binary (shadow/operators/binary_op.cpp:9-65): `operation` 0..6 is required; the presence of a
// `scalar` argument selects the one-input form.  Two-input form: NumPy-style broadcast with the
// lower rank left-padded by 1s; each dim must match or be 1; output dim is the larger.
class BinaryOp : public Operator {
 public:
  BinaryOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    operation_ = get_single_argument<int>("operation", -1);
    CHECK_GE(operation_, 0);
    CHECK_LE(operation_, 6);
    has_scalar_ = has_argument("scalar");
    if (has_scalar_) scalar_value_ = get_single_argument<float>("scalar", 0);
    kernel_ = kernel_for<BinaryKernel>(op_param, ws_);
  }

  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    CHECK_EQ(inputs.size(), has_scalar_ ? 1u : 2u);
    const auto& lhs = inputs[0];
    auto& out = outputs[0];
    if (has_scalar_) {
      out->reshape(lhs->shape());
      kernel_->Run(lhs, out, ws_, operation_, scalar_value_);
      return;
    }
    const auto& rhs = inputs[1];
    if (lhs->shape() == rhs->shape()) {
      out->reshape(lhs->shape());
      kernel_->Run(lhs, rhs, out, ws_, operation_, false);
      return;
    }
    // The kernel reads rank-aligned shapes from the blobs, so the shorter shape is padded for the
    // duration of the call and restored afterwards, also when the call throws.
    const VecInt lhs_shape = lhs->shape(), rhs_shape = rhs->shape();
    struct Restore {
      const BlobPtr &a, &b;
      VecInt sa, sb;
      ~Restore() { a->set_shape(sa), b->set_shape(sb); }
    } restore{lhs, rhs, lhs_shape, rhs_shape};
    const size_t rank = std::max(lhs_shape.size(), rhs_shape.size());
    VecInt pl(rank - lhs_shape.size(), 1), pr(rank - rhs_shape.size(), 1);
    pl.insert(pl.end(), lhs_shape.begin(), lhs_shape.end());
    pr.insert(pr.end(), rhs_shape.begin(), rhs_shape.end());
    lhs->set_shape(pl), rhs->set_shape(pr);
    CHECK_EQ(lhs->num_axes(), rhs->num_axes());
    VecInt out_shape;
    for (size_t n = 0; n < rank; ++n) {
      const int dl = pl[n], dr = pr[n];
      CHECK(dl == dr || dl == 1 || dr == 1);
      out_shape.push_back(std::max(dl, dr));
    }
    out->reshape(out_shape);
    kernel_->Run(lhs, rhs, out, ws_, operation_, true);
  }

 private:
  int operation_ = -1;
  float scalar_value_ = 0.f;
  bool has_scalar_ = false;
  std::shared_ptr<BinaryKernel> kernel_;
};

// Unary (shadow/operators/unary_op.cpp:9-28): `operation` 0..14 required.
class UnaryOp : public Operator {
 public:
  UnaryOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    operation_ = get_single_argument<int>("operation", -1);
    CHECK_GE(operation_, 0);
    CHECK_LE(operation_, 14);
    kernel_ = kernel_for<UnaryKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    outputs[0]->reshape(inputs[0]->shape());
    kernel_->Run(inputs[0], outputs[0], ws_, operation_);
  }

 private:
  int operation_;
  std::shared_ptr<UnaryKernel> kernel_;
};

// Activate (shadow/operators/activate_op.cpp:9-34): `type` default 1 (ReLU), `slope` default 0.1;
// PReLU (type 0) takes the slope blob as a second input.
class ActivateOp : public Operator {
 public:
  ActivateOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    type_ = get_single_argument<int>("type", 1);
    slope_ = get_single_argument<float>("slope", 0.1f);
    CHECK_GE(type_, 0);
    CHECK_LE(type_, 8);
    kernel_ = kernel_for<ActivateKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    const bool prelu = type_ == ActivateCode::kPRelu;
    CHECK_EQ(inputs.size(), prelu ? 2u : 1u);
    outputs[0]->reshape(inputs[0]->shape());
    kernel_->Run(inputs[0], prelu ? inputs[1] : BlobPtr(), outputs[0], ws_, type_, slope_);
  }

 private:
  int type_;
  float slope_;
  std::shared_ptr<ActivateKernel> kernel_;
};

// Scale (shadow/operators/scale_op.cpp:9-52): `axis` default 1; has_scale / has_bias (default
// false) select blob inputs; otherwise scale_value / bias_value vectors (a single value is
// repeated over the axis).
class ScaleOp : public Operator {
 public:
  ScaleOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    axis_ = get_single_argument<int>("axis", 1);
    has_scale_ = get_single_argument<bool>("has_scale", false);
    has_bias_ = get_single_argument<bool>("has_bias", false);
    scale_value_ = get_repeated_argument<float>("scale_value");
    bias_value_ = get_repeated_argument<float>("bias_value");
    kernel_ = kernel_for<ScaleKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    const auto& in = inputs[0];
    auto& out = outputs[0];
    out->reshape(in->shape());
    if (has_scale_ || has_bias_) {
      CHECK_EQ(inputs.size(), (has_scale_ && has_bias_) ? 3u : 2u);
      const BlobPtr none;
      const BlobPtr& scale = has_scale_ ? inputs[1] : none;
      const BlobPtr& bias = has_bias_ ? inputs[has_scale_ ? 2 : 1] : none;
      kernel_->Run(in, scale, bias, out, ws_, axis_);
      return;
    }
    const int dim = in->shape(axis_);
    auto widen = [dim](VecFloat* v) {
      if (v->size() > 1) {
        CHECK_EQ(static_cast<int>(v->size()), dim);
      } else if (v->size() == 1) {
        *v = VecFloat(dim, (*v)[0]);
      }
    };
    widen(&scale_value_), widen(&bias_value_);
    kernel_->Run(in, out, ws_, axis_, scale_value_, bias_value_);
  }

 private:
  int axis_;
  bool has_scale_, has_bias_;
  VecFloat scale_value_, bias_value_;
  std::shared_ptr<ScaleKernel> kernel_;
};

// Reduce (shadow/operators/reduce_op.cpp:9-65): `operation` default 0 (Prod), `axes` (empty = all),
// `keep_dims` default true.  In-place is refused.  Reduced dims become 1; with keep_dims false they
// are squeezed after the kernel ran (all axes -> shape [] with one element).
class ReduceOp : public Operator {
 public:
  ReduceOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    operation_ = get_single_argument<int>("operation", 0);
    CHECK_GE(operation_, 0);
    CHECK_LE(operation_, 6);
    axes_ = get_repeated_argument<int>("axes");
    keep_dims_ = get_single_argument<bool>("keep_dims", true);
    kernel_ = kernel_for<ReduceKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    const auto& in = inputs[0];
    auto& out = outputs[0];
    CHECK_NE(in, out);
    const int rank = in->num_axes();
    VecInt axes = axes_;
    if (axes.empty()) {
      for (int n = 0; n < rank; ++n) axes.push_back(n);
    }
    VecInt out_shape = in->shape();
    for (int axis : axes) out_shape[in->canonical_index(axis)] = 1;
    out->reshape(out_shape);
    kernel_->Run(in, out, ws_, operation_, axes);
    if (!keep_dims_) {
      VecInt squeezed;
      for (int n = 0; n < rank; ++n) {
        const bool reduced = std::find(axes.begin(), axes.end(), n) != axes.end();
        if (reduced) {
          CHECK_EQ(out->shape(n), 1);
        } else {
          squeezed.push_back(out->shape(n));
        }
      }
      out->set_shape(squeezed);
    }
  }

 private:
  int operation_;
  bool keep_dims_;
  VecInt axes_;
  std::shared_ptr<ReduceKernel> kernel_;
};

// Softmax (shadow/operators/softmax_op.cpp:9-28): `axis` default 1, negative values count from
// the end.
class SoftmaxOp : public Operator {
 public:
  SoftmaxOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    axis_ = get_single_argument<int>("axis", 1);
    kernel_ = kernel_for<SoftmaxKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    axis_ = inputs[0]->canonical_index(axis_);
    outputs[0]->reshape(inputs[0]->shape());
    kernel_->Run(inputs[0], outputs[0], ws_, axis_);
  }

 private:
  int axis_;
  std::shared_ptr<SoftmaxKernel> kernel_;
};

// Eltwise (shadow/operators/eltwise_op.cpp:7-56): `operation` 0..3 required (Prod, Sum, Max, Min);
// `coeff` (optional, Sum only) holds one coefficient per input; all inputs share one shape.
class EltwiseOp : public Operator {
 public:
  EltwiseOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    operation_ = get_single_argument<int>("operation", -1);
    CHECK_GE(operation_, 0);
    CHECK_LE(operation_, 3);
    coeff_ = get_repeated_argument<float>("coeff");
    kernel_ = kernel_for<EltwiseKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    CHECK_GE(inputs.size(), 2u);
    for (size_t n = 1; n < inputs.size(); ++n) CHECK(inputs[n]->shape() == inputs[0]->shape());
    outputs[0]->reshape(inputs[0]->shape());
    CHECK(coeff_.empty() || coeff_.size() == inputs.size()) << "Eltwise op takes one coefficient per input blob.";
    CHECK(!(operation_ != 1 && !coeff_.empty())) << "Eltwise op only takes coefficients for summation.";
    VecFloat coeff(inputs.size(), 1.f);
    for (size_t n = 0; n < coeff_.size(); ++n) coeff[n] = coeff_[n];
    kernel_->Run(inputs, outputs[0], ws_, operation_, coeff);
  }

 private:
  int operation_;
  VecFloat coeff_;
  std::shared_ptr<EltwiseKernel> kernel_;
};

// Axpy (shadow/operators/axpy_op.cpp:16-51): F = a * X + Y with a of shape [N, C] (or [N, C, 1, 1]).
class AxpyOp : public Operator {
 public:
  AxpyOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    kernel_ = kernel_for<AxpyKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    CHECK_EQ(inputs.size(), 3u) << "This op must have three inputs: alpha, x and y";
    const auto &alpha = inputs[0], &x = inputs[1], &y = inputs[2];
    CHECK_EQ(alpha->shape(0), x->shape(0));
    CHECK_EQ(alpha->shape(1), x->shape(1));
    if (alpha->num_axes() == 4) {
      CHECK_EQ(alpha->shape(2), 1);
      CHECK_EQ(alpha->shape(3), 1);
    }
    CHECK(x->shape() == y->shape());
    outputs[0]->reshape(x->shape());
    kernel_->Run(alpha, x, y, outputs[0], ws_);
  }

 private:
  std::shared_ptr<AxpyKernel> kernel_;
};

// ---- zero-copy shape operators: the output aliases the input's memory (Blob::share_data) --------
// Reshape (shadow/operators/reshape_op.cpp:9-80): the dims [axis, axis + num_axes) of the input are
// replaced by `shape`, where 0 keeps the input's extent at that position and one -1 is inferred.
class ReshapeOp : public Operator {
 public:
  ReshapeOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    axis_ = get_single_argument<int>("axis", 0);
    num_axes_ = get_single_argument<int>("num_axes", -1);
    CHECK_GE(num_axes_, -1);
    shape_ = get_repeated_argument<int>("shape");
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    const auto& input = inputs[0];
    auto& output = outputs[0];
    CHECK_NE(input, output);
    const int start = input->canonical_index(axis_);
    CHECK_GE(start, 0);
    CHECK_LT(start, input->num_axes());
    const int end = num_axes_ == -1 ? input->num_axes() : start + num_axes_;
    CHECK_LE(end, input->num_axes());
    VecInt out_shape;
    for (int d = 0; d < start; ++d) out_shape.push_back(input->shape(d));
    int inferred = -1;
    long long known = 1;
    for (size_t k = 0; k < shape_.size(); ++k) {
      int dim = shape_[k];
      if (dim == 0) {
        CHECK_GT(input->num_axes(), start + static_cast<int>(k));
        dim = input->shape(start + static_cast<int>(k));
      }
      if (dim == -1) {
        CHECK_EQ(inferred, -1);
        inferred = start + static_cast<int>(k);
      } else {
        known *= dim;
      }
      out_shape.push_back(dim);
    }
    for (int d = end; d < input->num_axes(); ++d) out_shape.push_back(input->shape(d));
    if (inferred >= 0) {
      known *= input->count(0, start);
      known *= input->count(end);
      CHECK_EQ(0, input->count() % known);
      out_shape[inferred] = static_cast<int>(input->count() / known);
    }
    output->share_data(input->data<void>(), out_shape);
    CHECK_EQ(output->count(), input->count());
  }

 private:
  int axis_, num_axes_;
  VecInt shape_;
};

// Flatten (shadow/operators/flatten_op.cpp:9-45): dims [axis, end_axis] become one; `axis` default 1,
// `end_axis` default -1 = last.
class FlattenOp : public Operator {
 public:
  FlattenOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    axis_ = get_single_argument<int>("axis", 1);
    CHECK_GE(axis_, 0);
    end_axis_ = get_single_argument<int>("end_axis", -1);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    const auto& input = inputs[0];
    auto& output = outputs[0];
    CHECK_NE(input, output);
    const int n = input->num_axes();
    if (end_axis_ == -1) end_axis_ = n - 1;
    CHECK_LT(end_axis_, n);
    CHECK_LE(axis_, end_axis_);
    VecInt out_shape;
    for (int d = 0; d < axis_; ++d) out_shape.push_back(input->shape(d));
    out_shape.push_back(input->count(axis_, end_axis_ + 1));
    for (int d = end_axis_ + 1; d < n; ++d) out_shape.push_back(input->shape(d));
    output->share_data(input->data<void>(), out_shape);
    CHECK_EQ(output->count(), input->count());
  }

 private:
  int axis_, end_axis_;
};

// Squeeze (shadow/operators/squeeze_op.cpp:9-55): drops the listed axes (each must have extent 1),
// or every extent-1 axis when `axes` is empty.
class SqueezeOp : public Operator {
 public:
  SqueezeOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    axes_ = get_repeated_argument<int>("axes");
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    const auto& input = inputs[0];
    auto& output = outputs[0];
    CHECK_NE(input, output);
    VecInt out_shape;
    for (int n = 0; n < input->num_axes(); ++n) {
      const int dim = input->shape(n);
      const bool listed = std::find(axes_.begin(), axes_.end(), n) != axes_.end();
      if (axes_.empty()) {
        if (dim > 1) out_shape.push_back(dim);
        else CHECK_EQ(dim, 1);
      } else if (listed) {
        CHECK_EQ(dim, 1);
      } else {
        out_shape.push_back(dim);
      }
    }
    output->share_data(input->data<void>(), out_shape);
    CHECK_EQ(output->count(), input->count());
  }

 private:
  VecInt axes_;
};

// Unsqueeze (shadow/operators/unsqueeze_op.cpp:9-45): inserts extent-1 axes at the listed output
// positions (negative positions count from the end of the output).
class UnsqueezeOp : public Operator {
 public:
  UnsqueezeOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    axes_ = get_repeated_argument<int>("axes");
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    const auto& input = inputs[0];
    auto& output = outputs[0];
    CHECK_NE(input, output);
    const int n = input->num_axes();
    VecInt out_shape(n + axes_.size(), 0);
    for (int axis : axes_) out_shape[axis < 0 ? axis + n + 1 : axis] = 1;
    int d = 0;
    for (auto& dim : out_shape)
      if (dim == 0) dim = input->shape(d++);
    CHECK_EQ(d, n);
    output->share_data(input->data<void>(), out_shape);
    CHECK_EQ(output->count(), input->count());
  }

 private:
  VecInt axes_;
};

// ---- data movement -------------------------------------------------------------------------------
// Concat (shadow/operators/concat_op.cpp:9-45): `axis` default 1; inputs agree on every other axis.
class ConcatOp : public Operator {
 public:
  ConcatOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    axis_ = get_single_argument<int>("axis", 1);
    kernel_ = kernel_for<ConcatKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    CHECK_GE(inputs.size(), 2u);
    axis_ = inputs[0]->canonical_index(axis_);
    auto shape = inputs[0]->shape();
    const int n = inputs[0]->num_axes();
    for (size_t k = 1; k < inputs.size(); ++k) {
      CHECK_EQ(n, inputs[k]->num_axes()) << "Inputs must have the same axes!";
      for (int d = 0; d < n; ++d)
        if (d != axis_) CHECK_EQ(shape[d], inputs[k]->shape(d)) << "Inputs must have the same shape, except at concat_axis!";
      shape[axis_] += inputs[k]->shape(axis_);
    }
    outputs[0]->reshape(shape);
    kernel_->Run(inputs, outputs[0], ws_, axis_);
  }

 private:
  int axis_;
  std::shared_ptr<ConcatKernel> kernel_;
};

// Slice (shadow/operators/slice_op.cpp:9-60): `axis` default 1; `slice_point` lists the cut
// positions (strictly increasing); without it the axis is split evenly over the outputs.
class SliceOp : public Operator {
 public:
  SliceOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    axis_ = get_single_argument<int>("axis", 1);
    slice_point_ = get_repeated_argument<int>("slice_point");
    kernel_ = kernel_for<SliceKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    CHECK_GE(outputs.size(), 2u);
    const auto& input = inputs[0];
    axis_ = input->canonical_index(axis_);
    const int pieces = static_cast<int>(outputs.size()), extent = input->shape(axis_);
    VecInt sizes;
    if (slice_point_.empty()) {
      CHECK_EQ(extent % pieces, 0);
      sizes.assign(pieces, extent / pieces);
    } else {
      CHECK_EQ(static_cast<int>(slice_point_.size()), pieces - 1);
      int prev = 0;
      for (int point : slice_point_) {
        CHECK_GT(point, prev);
        sizes.push_back(point - prev);
        prev = point;
      }
      CHECK_GT(extent, prev);
      sizes.push_back(extent - prev);
    }
    int total = 0;
    auto shape = input->shape();
    for (int k = 0; k < pieces; ++k) {
      shape[axis_] = sizes[k];
      outputs[k]->reshape(shape);
      total += outputs[k]->count();
    }
    CHECK_EQ(total, input->count());
    kernel_->Run(input, outputs, ws_, axis_);
  }

 private:
  int axis_;
  VecInt slice_point_;
  std::shared_ptr<SliceKernel> kernel_;
};

// Stack (shadow/operators/stack_op.cpp:9-40): a new axis of extent #inputs at `axis` (default 0,
// negative values count from the end of the output).
class StackOp : public Operator {
 public:
  StackOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    axis_ = get_single_argument<int>("axis", 0);
    kernel_ = kernel_for<StackKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    CHECK_GE(inputs.size(), 2u);
    const int n = inputs[0]->num_axes();
    CHECK(axis_ >= -(n + 1) && axis_ < n + 1) << "axis out of bound.";
    if (axis_ < 0) axis_ += n + 1;
    auto shape = inputs[0]->shape();
    shape.insert(shape.begin() + axis_, static_cast<int>(inputs.size()));
    outputs[0]->reshape(shape);
    kernel_->Run(inputs, outputs[0], ws_, axis_);
  }

 private:
  int axis_;
  std::shared_ptr<StackKernel> kernel_;
};

// Permute (shadow/operators/permute_op.cpp:9-35): `order` lists, per output axis, the input axis.
class PermuteOp : public Operator {
 public:
  PermuteOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    order_ = get_repeated_argument<int>("order");
    kernel_ = kernel_for<PermuteKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    const auto& input = inputs[0];
    CHECK_NE(input, outputs[0]);
    CHECK_EQ(input->num_axes(), static_cast<int>(order_.size()));
    VecInt shape;
    for (int axis : order_) shape.push_back(input->shape(axis));
    outputs[0]->reshape(shape);
    kernel_->Run(input, outputs[0], ws_, order_);
  }

 private:
  VecInt order_;
  std::shared_ptr<PermuteKernel> kernel_;
};

// Gather (shadow/operators/gather_op.cpp:9-50): `axis` default 0; the indexes come from the
// `indexes` argument (uploaded into a temporary int blob) or from a second, 1-d int input.
class GatherOp : public Operator {
 public:
  GatherOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    axis_ = get_single_argument<int>("axis", 0);
    indexes_ = get_repeated_argument<int>("indexes");
    kernel_ = kernel_for<GatherKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    const auto& input = inputs[0];
    CHECK_NE(input, outputs[0]);
    axis_ = input->canonical_index(axis_);
    BlobPtr indexes;
    if (indexes_.empty()) {
      CHECK_EQ(inputs.size(), 2u);
      indexes = inputs[1];
      CHECK_EQ(indexes->num_axes(), 1);
    } else {
      const int n = static_cast<int>(indexes_.size());
      ws_->GrowTempBuffer(n * sizeof(int));
      indexes = ws_->CreateTempBlob({n}, DataType::kI32);
      indexes->set_data<int>(indexes_.data(), indexes->count());
    }
    const int n = indexes->count();
    CHECK_GT(n, 0);
    auto shape = input->shape();
    shape[axis_] = n;
    outputs[0]->reshape(shape);
    kernel_->Run(input, indexes, outputs[0], ws_, axis_);
  }

 private:
  int axis_;
  VecInt indexes_;
  std::shared_ptr<GatherKernel> kernel_;
};

// Pad (shadow/operators/pad_op.cpp:9-40): `paddings` = [top, bottom, left, right] on axes 2 and 3,
// `value` default 0.
class PadOp : public Operator {
 public:
  PadOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    paddings_ = get_repeated_argument<int>("paddings");
    CHECK_EQ(paddings_.size(), 4u);
    value_ = get_single_argument<float>("value", 0);
    kernel_ = kernel_for<PadKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    const auto& input = inputs[0];
    CHECK_NE(input, outputs[0]);
    auto shape = input->shape();
    shape[2] = input->shape(2) + paddings_[0] + paddings_[1];
    shape[3] = input->shape(3) + paddings_[2] + paddings_[3];
    outputs[0]->reshape(shape);
    kernel_->Run(input, outputs[0], ws_, paddings_, value_);
  }

 private:
  float value_;
  VecInt paddings_;
  std::shared_ptr<PadKernel> kernel_;
};

// Pooling (shadow/operators/pooling_op.cpp:7-100): `pool` 0 = max, 1 = average; `global_pooling`
// makes the kernel the whole spatial extent (stride 1, pad 0); otherwise `kernel_size`, `stride`
// (default 1), `pad` (default 0) hold one value or one per spatial axis; `full_pooling` (default
// true) rounds the output size up instead of down.  2 or 3 spatial axes.
class PoolingOp : public Operator {
 public:
  PoolingOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    pool_type_ = get_single_argument<int>("pool", 0);
    CHECK_GE(pool_type_, 0);
    CHECK_LE(pool_type_, 1);
    global_pooling_ = get_single_argument<bool>("global_pooling", false);
    if (global_pooling_) {
      stride_ = VecInt(1, 1), pad_ = VecInt(1, 0);
    } else {
      kernel_size_ = get_repeated_argument<int>("kernel_size", 0);
      stride_ = get_repeated_argument<int>("stride", 1);
      pad_ = get_repeated_argument<int>("pad", 0);
    }
    full_pooling_ = get_single_argument<bool>("full_pooling", true);
    kernel_ = kernel_for<PoolingKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    const auto& input = inputs[0];
    CHECK_NE(input, outputs[0]);
    const int ns = input->num_axes() - 2;
    CHECK(ns == 2 || ns == 3) << "Only support 2D or 3D Pooling";
    if (global_pooling_ && static_cast<int>(kernel_size_.size()) != ns) {
      for (int n = 0; n < ns; ++n) kernel_size_.push_back(input->shape(n + 2));
    }
    const VecInt k = per_axis(kernel_size_, ns), st = per_axis(stride_, ns), pd = per_axis(pad_, ns);
    auto shape = input->shape();
    for (int n = 0; n < ns; ++n) {
      // float arithmetic, as the reference: (dim + 2.f*pad - kernel) / stride, rounded up or down, plus 1
      const float q = (input->shape(n + 2) + 2.f * pd[n] - k[n]) / st[n];
      shape[n + 2] = static_cast<int>(full_pooling_ ? std::ceil(q) : std::floor(q)) + 1;
    }
    outputs[0]->reshape(shape);
    if (ns == 2) kernel_->Run(input, outputs[0], ws_, pool_type_, k[0], k[1], st[0], st[1], pd[0], pd[1], full_pooling_);
    else kernel_->Run(input, outputs[0], ws_, pool_type_, k[0], k[1], k[2], st[0], st[1], st[2], pd[0], pd[1], pd[2], full_pooling_);
  }

 private:
  static VecInt per_axis(const VecInt& v, int n) {
    if (v.size() == 1) return VecInt(n, v[0]);
    CHECK_EQ(static_cast<int>(v.size()), n);
    return v;
  }
  int pool_type_;
  bool global_pooling_, full_pooling_;
  VecInt kernel_size_, stride_, pad_;
  std::shared_ptr<PoolingKernel> kernel_;
};

// SSDNormalize (shadow/operators/ssd_normalize_op.cpp:9-45): `across_spatial` default true,
// `channel_shared` default true, `eps` default 1e-5; one input, or two (x, scale).
class SSDNormalizeOp : public Operator {
 public:
  SSDNormalizeOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    across_spatial_ = get_single_argument<bool>("across_spatial", true);
    channel_shared_ = get_single_argument<bool>("channel_shared", true);
    eps_ = get_single_argument<float>("eps", 1e-5f);
    kernel_ = kernel_for<SSDNormalizeKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    outputs[0]->reshape(inputs[0]->shape());
    if (inputs.size() == 1) {
      kernel_->Run(inputs[0], nullptr, outputs[0], ws_, across_spatial_, channel_shared_, eps_);
    } else {
      CHECK_EQ(inputs.size(), 2u);
      kernel_->Run(inputs[0], inputs[1], outputs[0], ws_, across_spatial_, channel_shared_, eps_);
    }
  }

 private:
  float eps_;
  bool across_spatial_, channel_shared_;
  std::shared_ptr<SSDNormalizeKernel> kernel_;
};

// GroupNorm (shadow/operators/group_norm_op.cpp:9-45): `group` default 1, `eps` default 1e-5; one
// input, or three (x, per-channel scale, per-channel bias).
class GroupNormOp : public Operator {
 public:
  GroupNormOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    group_ = get_single_argument<int>("group", 1);
    eps_ = get_single_argument<float>("eps", 1e-5f);
    kernel_ = kernel_for<GroupNormKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    outputs[0]->reshape(inputs[0]->shape());
    CHECK_EQ(inputs[0]->shape(1) % group_, 0);
    if (inputs.size() == 1) {
      kernel_->Run(inputs[0], nullptr, nullptr, outputs[0], ws_, group_, eps_);
    } else {
      CHECK_EQ(inputs.size(), 3u);
      kernel_->Run(inputs[0], inputs[1], inputs[2], outputs[0], ws_, group_, eps_);
    }
  }

 private:
  int group_;
  float eps_;
  std::shared_ptr<GroupNormKernel> kernel_;
};

// InstanceNorm (shadow/operators/instance_norm_op.cpp:9-40): the GroupNorm kernel with one channel
// per group.
class InstanceNormOp : public Operator {
 public:
  InstanceNormOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    eps_ = get_single_argument<float>("eps", 1e-5f);
    kernel_ = std::dynamic_pointer_cast<GroupNormKernel>(CreateKernel("GroupNorm", ws_->Ctx()->device_type()));
    CHECK_NOTNULL(kernel_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    outputs[0]->reshape(inputs[0]->shape());
    const int channel = inputs[0]->shape(1);
    if (inputs.size() == 1) {
      kernel_->Run(inputs[0], nullptr, nullptr, outputs[0], ws_, channel, eps_);
    } else {
      CHECK_EQ(inputs.size(), 3u);
      kernel_->Run(inputs[0], inputs[1], inputs[2], outputs[0], ws_, channel, eps_);
    }
  }

 private:
  float eps_;
  std::shared_ptr<GroupNormKernel> kernel_;
};

// LayerNorm (shadow/operators/layer_norm_op.cpp:9-50): `normalized_shape` (required) must equal
// the trailing dims of the input; `eps` default 1e-5; one input, or three (x, scale, bias).
class LayerNormOp : public Operator {
 public:
  LayerNormOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    normalized_shape_ = get_repeated_argument<int>("normalized_shape");
    CHECK(!normalized_shape_.empty());
    eps_ = get_single_argument<float>("eps", 1e-5f);
    kernel_ = kernel_for<LayerNormKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    const auto& input = inputs[0];
    outputs[0]->reshape(input->shape());
    const int k = static_cast<int>(normalized_shape_.size());
    for (int n = 0; n < k; ++n) CHECK_EQ(input->shape(n - k), normalized_shape_[n]);
    if (inputs.size() == 1) {
      kernel_->Run(input, nullptr, nullptr, outputs[0], ws_, normalized_shape_, eps_);
    } else {
      CHECK_EQ(inputs.size(), 3u);
      kernel_->Run(input, inputs[1], inputs[2], outputs[0], ws_, normalized_shape_, eps_);
    }
  }

 private:
  float eps_;
  VecInt normalized_shape_;
  std::shared_ptr<LayerNormKernel> kernel_;
};

// Normalize (shadow/operators/normalize_op.cpp:9-37): `p` default 2, `axis` default 1 (negative
// values count from the end), `eps` default 1e-12.
class NormalizeOp : public Operator {
 public:
  NormalizeOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    p_ = get_single_argument<float>("p", 2);
    axis_ = get_single_argument<int>("axis", 1);
    eps_ = get_single_argument<float>("eps", 1e-12f);
    kernel_ = kernel_for<NormalizeKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    outputs[0]->reshape(inputs[0]->shape());
    kernel_->Run(inputs[0], outputs[0], ws_, p_, inputs[0]->canonical_index(axis_), eps_);
  }

 private:
  float p_, eps_;
  int axis_;
  std::shared_ptr<NormalizeKernel> kernel_;
};

// BatchNorm, inference only (shadow/operators/batch_norm_op.cpp:9-43): `use_global_stats` must be
// true, `eps` default 1e-5; inputs x, mean, variance and optionally a one-element scale blob whose
// reciprocal (0 if the scale is 0) multiplies mean and variance.  The scale is read back from the
// device on every Run, as in the reference.
class BatchNormOp : public Operator {
 public:
  BatchNormOp(const shadow::OpParam& op_param, Workspace* ws) : Operator(op_param, ws) {
    CHECK(get_single_argument<bool>("use_global_stats", true));
    eps_ = get_single_argument<float>("eps", 1e-5f);
    kernel_ = kernel_for<BatchNormKernel>(op_param, ws_);
  }
  void Run(const std::vector<BlobPtr>& inputs, std::vector<BlobPtr>& outputs) override {
    CHECK_GE(inputs.size(), 3u);
    outputs[0]->reshape(inputs[0]->shape());
    float scale_factor = 1;
    if (inputs.size() == 4) {
      float scale = 1;
      CHECK_EQ(inputs[3]->count(), 1);
      inputs[3]->get_data<float>(&scale, 1);
      scale_factor = scale == 0 ? 0 : 1 / scale;
    }
    kernel_->Run(inputs[0], inputs[1], inputs[2], outputs[0], ws_, scale_factor, eps_);
  }

 private:
  float eps_;
  std::shared_ptr<BatchNormKernel> kernel_;
};

}  // namespace

REGISTER_OPERATOR(BatchNorm, BatchNormOp);
REGISTER_OPERATOR(Normalize, NormalizeOp);
REGISTER_OPERATOR(Reshape, ReshapeOp);
REGISTER_OPERATOR(Flatten, FlattenOp);
REGISTER_OPERATOR(Squeeze, SqueezeOp);
REGISTER_OPERATOR(Unsqueeze, UnsqueezeOp);
REGISTER_OPERATOR(Concat, ConcatOp);
REGISTER_OPERATOR(Slice, SliceOp);
REGISTER_OPERATOR(Stack, StackOp);
REGISTER_OPERATOR(Permute, PermuteOp);
REGISTER_OPERATOR(Gather, GatherOp);
REGISTER_OPERATOR(Pad, PadOp);
REGISTER_OPERATOR(Pooling, PoolingOp);
REGISTER_OPERATOR(SSDNormalize, SSDNormalizeOp);
REGISTER_OPERATOR(GroupNorm, GroupNormOp);
REGISTER_OPERATOR(InstanceNorm, InstanceNormOp);
REGISTER_OPERATOR(LayerNorm, LayerNormOp);
REGISTER_OPERATOR(Eltwise, EltwiseOp);
REGISTER_OPERATOR(Axpy, AxpyOp);
REGISTER_OPERATOR(Input, InputOp);
REGISTER_OPERATOR(Binary, BinaryOp);
REGISTER_OPERATOR(Unary, UnaryOp);
REGISTER_OPERATOR(Activate, ActivateOp);
REGISTER_OPERATOR(Scale, ScaleOp);
REGISTER_OPERATOR(Reduce, ReduceOp);
REGISTER_OPERATOR(Softmax, SoftmaxOp);

}  // namespace Shadow
