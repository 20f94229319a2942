// Kernel / operator / backend registries, the sequential Native backend and the Network facade.
#include <algorithm>

#include "shadow_api.hpp"

namespace Shadow {

// ---- kernel registry ----------------------------------------------------------------------------
SHADOW_DEFINE_REGISTRY(KernelRegistry, Kernel);

namespace {

const char* device_suffix(DeviceType device_type) {
  switch (device_type) {
    case DeviceType::kCPU: return "CPU";
    case DeviceType::kGPU: return "GPU";
    default: return "NPU";
  }
}

// Preference order of kernel flavours per device, best first (shadow/core/kernel.cpp:8-10).
const std::vector<std::string>& flavour_order(DeviceType device_type) {
  static const std::vector<std::string> cpu = {"DNNL", "NNPACK", "Default"}, gpu = {"CUDNN", "Default"};
  return device_type == DeviceType::kGPU ? gpu : cpu;
}

VecString keys_containing(const std::string& hint) {
  VecString out;
  for (const auto& key : KernelRegistry()->Keys())
    if (key.find(hint) != std::string::npos) out.push_back(key);
  return out;
}

}  // namespace

VecString GetKernelKeys(DeviceType device_type) { return keys_containing(device_suffix(device_type)); }

VecString GetKernelKeys(const std::string& op_type, DeviceType device_type) {
  return keys_containing(op_type + device_suffix(device_type));
}

std::shared_ptr<Kernel> CreateKernel(const std::string& op_type, DeviceType device_type,
                                     const std::string& kernel_type) {
  std::string flavour = kernel_type;
  if (flavour.empty()) {
    flavour = "None";
    const auto keys = GetKernelKeys(op_type, device_type);
    for (const auto& candidate : flavour_order(device_type)) {
      const bool found = std::any_of(keys.begin(), keys.end(), [&](const std::string& k) {
        return k.find(candidate) != std::string::npos;
      });
      if (found) {
        flavour = candidate;
        break;
      }
    }
  }
  const std::string key = op_type + device_suffix(device_type) + "(" + flavour + ")";
  std::shared_ptr<Kernel> kernel(KernelRegistry()->Create(key));
  LOG_IF(FATAL, kernel == nullptr) << "Kernel type: " << key << " is not registered";
  return kernel;
}

// ---- operator -----------------------------------------------------------------------------------
SHADOW_DEFINE_REGISTRY(OperatorRegistry, Operator, const shadow::OpParam&, Workspace*);

Operator::Operator(const shadow::OpParam& op_param, Workspace* ws)
    : ws_(ws), op_param_(op_param), arg_helper_(op_param) {
  // every top blob is created up front; its element type comes from an optional "<top>_type"
  // argument and defaults to float
  for (const auto& top : op_param_.top()) {
    const auto type = get_single_argument<std::string>(top + "_type", "float");
    CHECK_NOTNULL(ws->CreateBlob(top, type))
        << name() << ": Failed to create output blob " << top << ", asked for type " << type;
  }
}

std::string Operator::debug_log(const std::vector<std::shared_ptr<Blob>>& inputs,
                                const std::vector<std::shared_ptr<Blob>>& outputs) const {
  auto describe = [](const std::vector<std::shared_ptr<Blob>>& blobs) {
    std::stringstream ss;
    for (size_t i = 0; i < blobs.size(); ++i) {
      ss << (i ? " + " : "") << blobs[i]->name() << "(";
      for (int d = 0; d < blobs[i]->num_axes(); ++d) ss << (d ? "," : "") << blobs[i]->shape(d);
      ss << ")";
    }
    return ss.str();
  };
  return name() + "(" + type() + "): " + describe(inputs) + " -> " + describe(outputs);
}

std::shared_ptr<Operator> CreateOperator(const shadow::OpParam& op_param, Workspace* ws) {
  std::shared_ptr<Operator> op(OperatorRegistry()->Create(op_param.type(), op_param, ws));
  CHECK_NOTNULL(op) << "Op type: " << op_param.type() << " is not registered";
  return op;
}

// ---- backend: the sequential "Native" runner ----------------------------------------------------
SHADOW_DEFINE_REGISTRY(BackendRegistry, Backend, const ArgumentHelper&);

namespace {

// Runs the operators of a NetParam in order on one Workspace (device + stream).  Mirrors
// shadow/backends/native/native.cpp: weight blobs from NetParam.blob, `Input` tops shaped by
// their v_i arguments, host inputs uploaded per Run (or copied device to device when the
// backend argument device_input is set), mandatory net argument out_blob.
class Native : public Backend {
 public:
  explicit Native(const ArgumentHelper& arguments) {
    device_input_ = arguments.GetSingleArgument<bool>("device_input", false);
    debug_ = arguments.GetSingleArgument<bool>("debug", false);
    ws_ = std::make_shared<Workspace>(arguments);
  }

  void LoadModel(const shadow::NetParam& net_param) override {
    for (const auto& blob : net_param.blob()) {
      const std::string type = blob.has_type() ? blob.type() : std::string("float");
      auto dst = ws_->CreateBlob(blob.name(), type);
      CHECK_NOTNULL(dst) << "Failed to create blob " << blob.name() << ", asked for type " << type;
      dst->reshape(blob.shape());
      if (dst->data_type() == DataType::kF32 && blob.data_f_size() > 0) {
        CHECK_EQ(static_cast<size_t>(blob.data_f_size()), dst->count64());
        dst->set_data<float>(blob.data_f().data(), blob.data_f_size());
        // the source vector lives in the caller's NetParam: finish the upload before returning
        ws_->Ctx()->synchronize();
      } else if (dst->data_type() != DataType::kF32 && blob.data_b_size() > 0 && !blob.data_b(0).empty()) {
        // non-float blobs (an int32 index list for Gather, ...) travel as raw bytes in data_b(0)
        // (shadow/backends/native/native.cpp:158-167)
        CHECK_EQ(blob.data_b(0).size(), dst->raw_size());
        ws_->Ctx()->allocator()->write(dst->raw_size(), blob.data_b(0).data(), dst->mutable_data<unsigned char>());
        ws_->Ctx()->synchronize();
      }
    }
    ops_.clear(), in_blob_.clear();
    for (const auto& op_param : net_param.op()) {
      ops_.push_back(CreateOperator(op_param, ws_.get()));
      if (op_param.type() == "Input") {
        CHECK(in_blob_.empty());
        for (const auto& top : op_param.top()) {
          ws_->GetBlob(top)->reshape(ops_.back()->get_repeated_argument<int>(top));
          in_blob_.push_back(top);
        }
      }
    }
    arg_helper_ = ArgumentHelper(net_param);
    CHECK(arg_helper_.HasArgument("out_blob")) << "Network must have out_blob argument";
    out_blob_ = arg_helper_.GetRepeatedArgument<std::string>("out_blob");
  }

  void Run(const std::map<std::string, void*>& data_map,
           const std::map<std::string, std::vector<int>>& shape_map) override {
    if (ops_.empty()) return;
    for (const auto& in : data_map) {
      CHECK_NOTNULL(in.second) << in.first << " has null data";
      auto blob = ws_->GetBlob(in.first);
      CHECK_NOTNULL(blob) << "Can not find blob " << in.first;
      auto shape_it = shape_map.find(in.first);
      if (shape_it != shape_map.end() && !shape_it->second.empty()) blob->reshape(shape_it->second);
      if (device_input_) {
        ws_->Ctx()->allocator()->copy(blob->raw_size(), in.second, blob->mutable_data<unsigned char>());
      } else {
        ws_->Ctx()->allocator()->write(blob->raw_size(), in.second, blob->mutable_data<unsigned char>());
      }
    }
    for (auto& op : ops_) {
      std::vector<std::shared_ptr<Blob>> inputs, outputs;
      for (const auto& name : op->op_param().bottom()) {
        CHECK(ws_->HasBlob(name)) << op->name() << ": Can not find input blob " << name;
        inputs.push_back(ws_->GetBlob(name));
      }
      for (const auto& name : op->op_param().top()) {
        CHECK(ws_->HasBlob(name)) << op->name() << ":  Can not find output blob " << name;
        outputs.push_back(ws_->GetBlob(name));
      }
      op->Run(inputs, outputs);
      LOG_IF(INFO, debug_) << op->debug_log(inputs, outputs);
    }
  }

  void SaveEngine(const std::string&, std::map<std::string, std::vector<char>>*) override {}

 private:
  bool device_input_ = false, debug_ = false;
  std::vector<std::shared_ptr<Operator>> ops_;
};

}  // namespace

REGISTER_BACKEND(Native, Native);

std::shared_ptr<Backend> CreateBackend(const ArgumentHelper& arguments) {
  CHECK(arguments.HasArgument("backend_type"));
  const auto type = arguments.GetSingleArgument<std::string>("backend_type", "");
  CHECK(!type.empty());
  std::shared_ptr<Backend> backend(BackendRegistry()->Create(type, arguments));
  CHECK_NOTNULL(backend) << "Backend type: " << type << " is not registered";
  return backend;
}

// ---- Network ------------------------------------------------------------------------------------
Network::Network() = default;

void Network::LoadXModel(const shadow::NetParam& net_param, const ArgumentHelper& arguments) {
  backend_ = CreateBackend(arguments);
  backend_->LoadModel(net_param);
}

void Network::Forward(const std::map<std::string, void*>& data_map,
                      const std::map<std::string, std::vector<int>>& shape_map) {
  CHECK_NOTNULL(backend_);
  backend_->ws()->Ctx()->switch_device();
  backend_->Run(data_map, shape_map);
  backend_->ws()->Ctx()->synchronize();
}

#define SB_NETWORK_BLOB(T)                                                                              \
  template <>                                                                                           \
  const T* Network::GetBlobDataByName<T>(const std::string& blob_name, const std::string& locate) {     \
    auto blob = backend_->ws()->GetBlob(blob_name);                                                     \
    CHECK_NOTNULL(blob) << "Unknown blob: " + blob_name;                                                \
    return locate == "host" ? blob->cpu_data<T>() : blob->data<T>();                                    \
  }                                                                                                     \
  template <>                                                                                           \
  std::vector<int> Network::GetBlobShapeByName<T>(const std::string& blob_name) const {                 \
    return backend_->ws()->GetBlobShape(blob_name);                                                     \
  }
SB_NETWORK_BLOB(std::int64_t)
SB_NETWORK_BLOB(std::int32_t)
SB_NETWORK_BLOB(std::int16_t)
SB_NETWORK_BLOB(std::int8_t)
SB_NETWORK_BLOB(std::uint64_t)
SB_NETWORK_BLOB(std::uint32_t)
SB_NETWORK_BLOB(std::uint16_t)
SB_NETWORK_BLOB(std::uint8_t)
SB_NETWORK_BLOB(float)
SB_NETWORK_BLOB(bool)
#undef SB_NETWORK_BLOB

const std::vector<std::string>& Network::in_blob() const { return backend_->in_blob(); }
const std::vector<std::string>& Network::out_blob() const { return backend_->out_blob(); }
bool Network::has_argument(const std::string& name) const { return backend_->arg_helper().HasArgument(name); }

#define SB_NETWORK_ARG(T)                                                                               \
  template <>                                                                                           \
  T Network::get_single_argument<T>(const std::string& name, const T& default_value) const {            \
    return backend_->arg_helper().GetSingleArgument<T>(name, default_value);                            \
  }                                                                                                     \
  template <>                                                                                           \
  std::vector<T> Network::get_repeated_argument<T>(const std::string& name,                             \
                                                   const std::vector<T>& default_value) const {         \
    return backend_->arg_helper().GetRepeatedArgument<T>(name, default_value);                          \
  }
SB_NETWORK_ARG(float)
SB_NETWORK_ARG(int)
SB_NETWORK_ARG(bool)
SB_NETWORK_ARG(std::string)
#undef SB_NETWORK_ARG

}  // namespace Shadow
