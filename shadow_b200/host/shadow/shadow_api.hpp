// Host-side mirror of the Shadow plugin API for the tensor-operator path, in one header.
//
// A Shadow op graph is a shadow::NetParam (ops + arguments) executed by a Backend over named
// Blobs in a Workspace; every operator delegates its arithmetic to a Kernel looked up in a
// string-keyed registry.  This header re-creates exactly that surface - same namespaces, class
// names, method signatures, argument names, registry keys and error behaviour - so that code
// written against the reference's headers compiles and runs unchanged:
//   shadow::{Argument,Blob,OpParam,NetParam}     shadow/core/params.hpp:14-249 (protobuf-free form)
//   Shadow::ArgumentHelper, add_s_i ...          shadow/core/helper.hpp:10-58
//   CHECK* / LOG(FATAL) -> std::runtime_error    shadow/util/log.hpp:22-118
//   Registry / SHADOW_REGISTER_CLASS             shadow/core/registry.hpp:15-103
//   Allocator, Context, Blob, Workspace          shadow/core/{allocator,context,blob,workspace}.hpp
//   Kernel / CreateKernel / REGISTER_OP_KERNEL_* shadow/core/kernel.hpp:13-41, kernel.cpp:5-56
//   Operator / CreateOperator / REGISTER_OPERATOR shadow/core/operator.hpp:19-79
//   Backend / CreateBackend / REGISTER_BACKEND   shadow/core/backend.hpp:12-41
//   Network                                      shadow/core/network.hpp:15-43
// Only the GPU device exists here: a Context is a CUDA device + stream, an Allocator is
// cudaMalloc/cudaMemcpyAsync; there is no CPU context and no CPU kernel.
#ifndef SHADOW_B200_HOST_SHADOW_API_HPP_
#define SHADOW_B200_HOST_SHADOW_API_HPP_

#include <cstddef>
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

// ---------------------------------------------------------------------------------------------
// Model description (the protobuf-free classes of the reference, accessor for accessor)
// ---------------------------------------------------------------------------------------------
namespace shadow {

#define SB_SCALAR_FIELD(name, type)                                  \
 public:                                                             \
  const type& name() const { return name##_; }                       \
  void set_##name(const type& v) { name##_ = v, has_##name##_ = true; } \
  bool has_##name() const { return has_##name##_; }                  \
  void clear_##name() { name##_ = type(), has_##name##_ = false; }   \
                                                                     \
 private:                                                            \
  type name##_{};                                                    \
  bool has_##name##_ = false;

#define SB_LIST_FIELD(name, type)                                        \
 public:                                                                 \
  const std::vector<type>& name() const { return name##_; }              \
  std::vector<type>* mutable_##name() { return &name##_; }               \
  const type& name(int i) const { return name##_[i]; }                   \
  type* mutable_##name(int i) { return &name##_[i]; }                    \
  void set_##name(int i, const type& v) { name##_[i] = v; }              \
  type* add_##name() { name##_.emplace_back(); return &name##_.back(); } \
  void add_##name(const type& v) { name##_.push_back(v); }               \
  int name##_size() const { return static_cast<int>(name##_.size()); }   \
  bool has_##name() const { return !name##_.empty(); }                   \
  void clear_##name() { name##_.clear(); }                               \
                                                                         \
 private:                                                                \
  std::vector<type> name##_;

class Blob {
  SB_SCALAR_FIELD(name, std::string)
  SB_SCALAR_FIELD(type, std::string)
  SB_LIST_FIELD(shape, int)
  SB_LIST_FIELD(data_f, float)
  SB_LIST_FIELD(data_i, int)
  SB_LIST_FIELD(data_b, std::vector<char>)
};

class Argument {
  SB_SCALAR_FIELD(name, std::string)
  SB_SCALAR_FIELD(s_f, float)
  SB_SCALAR_FIELD(s_i, int)
  SB_SCALAR_FIELD(s_s, std::string)
  SB_LIST_FIELD(v_f, float)
  SB_LIST_FIELD(v_i, int)
  SB_LIST_FIELD(v_s, std::string)
};

class OpParam {
  SB_SCALAR_FIELD(name, std::string)
  SB_SCALAR_FIELD(type, std::string)
  SB_LIST_FIELD(bottom, std::string)
  SB_LIST_FIELD(top, std::string)
  SB_LIST_FIELD(arg, Argument)
};

class NetParam {
  SB_SCALAR_FIELD(name, std::string)
  SB_LIST_FIELD(blob, Blob)
  SB_LIST_FIELD(op, OpParam)
  SB_LIST_FIELD(arg, Argument)
};

// shadow/proto/shadow.proto:41-47: several networks in one file
class MetaNetParam {
  SB_SCALAR_FIELD(name, std::string)
  SB_LIST_FIELD(network, NetParam)
  SB_LIST_FIELD(arg, Argument)
};

#undef SB_SCALAR_FIELD
#undef SB_LIST_FIELD

}  // namespace shadow

namespace Shadow {

using VecInt = std::vector<int>;
using VecFloat = std::vector<float>;
using VecString = std::vector<std::string>;

// ---------------------------------------------------------------------------------------------
// Logging / checks: a failed CHECK or LOG(FATAL) prints "FATAL: file:line] message" to stderr and
// throws std::runtime_error(message), like shadow/util/log.hpp:84-118 (without the backtrace).
// ---------------------------------------------------------------------------------------------
class LogMessage {
 public:
  LogMessage(const char* severity, const char* file, int line);
  ~LogMessage() noexcept(false);
  std::stringstream& stream() { return stream_; }

 private:
  std::string severity_;
  std::stringstream stream_;
};

#define LOG(severity) ::Shadow::LogMessage(#severity, __FILE__, __LINE__).stream()
#define LOG_IF(severity, condition) \
  if ((condition)) LOG(severity)
#define CHECK(condition) \
  if (!(condition)) LOG(FATAL) << "Check Failed: " #condition << " "
#define CHECK_NOTNULL(ptr) \
  if ((ptr) == nullptr) LOG(FATAL) << "Check Failed: '" #ptr << "' Must be non NULL "
#define SB_CHECK_OP(op, a, b) \
  if (!((a)op(b))) LOG(FATAL) << "Check Failed: " #a " " #op " " #b " (" << (a) << " vs " << (b) << ") "
#define CHECK_EQ(a, b) SB_CHECK_OP(==, a, b)
#define CHECK_NE(a, b) SB_CHECK_OP(!=, a, b)
#define CHECK_LE(a, b) SB_CHECK_OP(<=, a, b)
#define CHECK_LT(a, b) SB_CHECK_OP(<, a, b)
#define CHECK_GE(a, b) SB_CHECK_OP(>=, a, b)
#define CHECK_GT(a, b) SB_CHECK_OP(>, a, b)

// ---------------------------------------------------------------------------------------------
// ArgumentHelper (shadow/core/helper.hpp:10-34) and the add_* helpers (:36-58)
// ---------------------------------------------------------------------------------------------
class ArgumentHelper {
 public:
  ArgumentHelper() = default;
  explicit ArgumentHelper(const shadow::NetParam& def) { Absorb(def.arg(), def.name()); }
  explicit ArgumentHelper(const shadow::OpParam& def) { Absorb(def.arg(), def.name()); }

  bool HasArgument(const std::string& name) const { return arguments_.count(name) > 0; }

  template <typename T>
  T GetSingleArgument(const std::string& name, const T& default_value) const;
  template <typename T>
  std::vector<T> GetRepeatedArgument(const std::string& name,
                                     const std::vector<T>& default_value = std::vector<T>()) const;
  template <typename T>
  void AddSingleArgument(const std::string& name, const T& value);
  template <typename T>
  void AddRepeatedArgument(const std::string& name, const std::vector<T>& value);

 private:
  void Absorb(const std::vector<shadow::Argument>& args, const std::string& owner);
  std::map<std::string, shadow::Argument> arguments_;
};

void add_s_f(shadow::NetParam* p, const std::string& name, const float& v);
void add_s_i(shadow::NetParam* p, const std::string& name, const int& v);
void add_s_i(shadow::NetParam* p, const std::string& name, const bool& v);
void add_s_s(shadow::NetParam* p, const std::string& name, const std::string& v);
void add_v_f(shadow::NetParam* p, const std::string& name, const std::vector<float>& v);
void add_v_i(shadow::NetParam* p, const std::string& name, const std::vector<int>& v);
void add_v_i(shadow::NetParam* p, const std::string& name, const std::vector<bool>& v);
void add_v_s(shadow::NetParam* p, const std::string& name, const std::vector<std::string>& v);
void add_s_f(shadow::OpParam* p, const std::string& name, const float& v);
void add_s_i(shadow::OpParam* p, const std::string& name, const int& v);
void add_s_i(shadow::OpParam* p, const std::string& name, const bool& v);
void add_s_s(shadow::OpParam* p, const std::string& name, const std::string& v);
void add_v_f(shadow::OpParam* p, const std::string& name, const std::vector<float>& v);
void add_v_i(shadow::OpParam* p, const std::string& name, const std::vector<int>& v);
void add_v_i(shadow::OpParam* p, const std::string& name, const std::vector<bool>& v);
void add_v_s(shadow::OpParam* p, const std::string& name, const std::vector<std::string>& v);

// ---------------------------------------------------------------------------------------------
// Registry (shadow/core/registry.hpp): string key -> factory; a duplicate key ends the process.
// ---------------------------------------------------------------------------------------------
template <typename Key, typename Object, typename... Args>
class Registry {
 public:
  using Creator = std::function<Object*(Args...)>;
  void Register(const Key& key, Creator creator, const std::string& help = "");
  Object* Create(const Key& key, Args... args) {
    auto it = table_.find(key);
    return it == table_.end() ? nullptr : it->second(args...);
  }
  bool Has(const Key& key) const { return table_.count(key) > 0; }
  std::vector<Key> Keys() const {
    std::vector<Key> keys;
    for (const auto& kv : table_) keys.push_back(kv.first);
    return keys;
  }
  std::string HelpMessage(const Key& key) const {
    auto it = help_.find(key);
    return it == help_.end() ? std::string() : it->second;
  }

 private:
  std::map<Key, Creator> table_;
  std::map<Key, std::string> help_;
};

void registry_duplicate_key(const std::string& key);  // prints and std::exit(1)

template <typename Key, typename Object, typename... Args>
void Registry<Key, Object, Args...>::Register(const Key& key, Creator creator, const std::string& help) {
  if (Has(key)) registry_duplicate_key(key);
  table_[key] = creator;
  help_[key] = help;
}

template <typename Key, typename Object, typename... Args>
class Register {
 public:
  Register(const Key& key, Registry<Key, Object, Args...>* registry,
           typename Registry<Key, Object, Args...>::Creator creator, const std::string& help = "") {
    registry->Register(key, creator, help);
  }
  template <typename Derived>
  static Object* DefaultCreator(Args... args) {
    return new Derived(args...);
  }
};

#define SB_CONCAT_IMPL(a, b) a##b
#define SB_CONCAT(a, b) SB_CONCAT_IMPL(a, b)
#define SHADOW_DECLARE_REGISTRY(RegistryName, ObjectType, ...)              \
  ::Shadow::Registry<std::string, ObjectType, ##__VA_ARGS__>* RegistryName(); \
  using Register##RegistryName = ::Shadow::Register<std::string, ObjectType, ##__VA_ARGS__>;
#define SHADOW_DEFINE_REGISTRY(RegistryName, ObjectType, ...)                           \
  ::Shadow::Registry<std::string, ObjectType, ##__VA_ARGS__>* RegistryName() {          \
    static auto* registry = new ::Shadow::Registry<std::string, ObjectType, ##__VA_ARGS__>(); \
    return registry;                                                                    \
  }
#define SHADOW_REGISTER_CLASS(RegistryName, key, ...)                             \
  namespace {                                                                     \
  static Register##RegistryName SB_CONCAT(g_sb_registrar_, __COUNTER__)(          \
      #key, RegistryName(), Register##RegistryName::DefaultCreator<__VA_ARGS__>); \
  }

// ---------------------------------------------------------------------------------------------
// Device runtime: Allocator, Context (shadow/core/allocator.hpp:10-27, context.hpp:11-29)
// ---------------------------------------------------------------------------------------------
enum class DeviceType { kCPU, kGPU, kNPU };

class Allocator {
 public:
  virtual ~Allocator() = default;
  virtual DeviceType device_type() const = 0;
  virtual void* malloc(size_t size, const void* host_ptr) const = 0;
  virtual void read(size_t size, const void* src, void* dst) const = 0;   // device -> host
  virtual void write(size_t size, const void* src, void* dst) const = 0;  // host -> device
  virtual void copy(size_t size, const void* src, void* dst) const = 0;   // device -> device
  virtual void free(void* ptr) const = 0;
  virtual void set_stream(void* stream) = 0;
};

class Context {
 public:
  virtual ~Context() = default;
  virtual Allocator* allocator() const = 0;
  virtual DeviceType device_type() const = 0;
  virtual int device_id() const = 0;
  virtual void switch_device() = 0;
  virtual void synchronize() = 0;
  virtual void* stream() const { return nullptr; }
  virtual void* cublas_handle() const { return nullptr; }
  virtual void* cudnn_handle() const { return nullptr; }
  virtual void* nnpack_handle() const { return nullptr; }
  virtual void* dnnl_handle() const { return nullptr; }
};

template <DeviceType D>
std::shared_ptr<Allocator> GetAllocator();
template <DeviceType D>
std::shared_ptr<Context> GetContext(const ArgumentHelper& arguments);

// ---------------------------------------------------------------------------------------------
// Blob (shadow/core/blob.hpp:28-223): typed dense N-d buffer owned through an Allocator
// ---------------------------------------------------------------------------------------------
enum class DataType { kI64, kI32, kI16, kI8, kU64, kU32, kU16, kU8, kF32, kBool };

size_t data_type_size(DataType type);
template <typename T>
DataType data_type_of();

class Blob {
 public:
  Blob(std::string name, DataType data_type, Allocator* allocator);
  ~Blob();
  Blob(const Blob&) = delete;
  Blob& operator=(const Blob&) = delete;

  template <typename T>
  const T* data() const { return static_cast<const T*>(data_); }
  template <typename T>
  T* mutable_data() { return static_cast<T*>(data_); }

  // Host copy of the contents (device -> host, then the stream is synchronised so the returned
  // pointer is valid immediately).
  template <typename T>
  const T* cpu_data() {
    require_type(data_type_of<T>());
    host_copy_.resize(raw_size());
    download(host_copy_.data(), raw_size(), 0);
    return reinterpret_cast<const T*>(host_copy_.data());
  }
  template <typename T>
  void set_data(const void* cpu_data, int set_count, int offset = 0) {
    require_type(data_type_of<T>());
    upload(cpu_data, static_cast<size_t>(set_count) * elem_size(), static_cast<size_t>(offset) * elem_size(),
           static_cast<size_t>(set_count) + offset);
  }
  template <typename T>
  void get_data(void* cpu_data, int get_count, int offset = 0) const {
    require_type(data_type_of<T>());
    CHECK_NOTNULL(cpu_data);
    CHECK_LE(static_cast<size_t>(get_count) + offset, count64());
    download(cpu_data, static_cast<size_t>(get_count) * elem_size(), static_cast<size_t>(offset) * elem_size());
  }

  void share_data(const void* data, const std::vector<int>& shape);
  void reshape(const std::vector<int>& shape);

  const std::string& name() const { return name_; }
  const DataType& data_type() const { return data_type_; }
  size_t capacity() const { return capacity_; }
  bool shared() const { return shared_; }
  void set_name(const std::string& name) { name_ = name; }

  const std::vector<int>& shape() const { return shape_; }
  int shape(int index) const { return shape_[canonical_index(index)]; }
  void set_shape(int index, int value) { shape_[canonical_index(index)] = value; }
  void set_shape(const std::vector<int>& shape) { shape_ = shape; }
  void add_shape(int value) { shape_.push_back(value); }
  int num_axes() const { return static_cast<int>(shape_.size()); }
  int num() const { return count() / shape(0); }
  int count() const { return count(0); }
  int count(int start_axis) const { return count(start_axis, num_axes()); }
  int count(int start_axis, int end_axis) const;
  size_t count64() const;
  size_t raw_size() const { return count64() * elem_size(); }
  size_t max_size() const { return capacity_ * elem_size(); }
  size_t elem_size() const { return data_type_size(data_type_); }
  int canonical_index(int index) const;

 private:
  void require_type(DataType asked) const;
  void upload(const void* host, size_t bytes, size_t byte_offset, size_t end_elem);
  void download(void* host, size_t bytes, size_t byte_offset) const;

  std::string name_;
  DataType data_type_;
  Allocator* allocator_;
  void* data_ = nullptr;
  std::vector<int> shape_;
  size_t capacity_ = 0;  // elements
  bool shared_ = false;
  std::vector<unsigned char> host_copy_;
};

// ---------------------------------------------------------------------------------------------
// Workspace (shadow/core/workspace.hpp:13-51): name -> Blob map, device context, and one grow-only
// temp buffer handed out as a bump allocator (valid until the next GrowTempBuffer).
// ---------------------------------------------------------------------------------------------
class Workspace {
 public:
  explicit Workspace(const ArgumentHelper& arguments);
  Workspace(const Workspace&) = delete;

  std::shared_ptr<Context>& Ctx() { return context_; }
  bool HasBlob(const std::string& name) const { return blobs_.count(name) > 0; }
  DataType GetBlobDataType(const std::string& name) const;
  std::vector<int> GetBlobShape(const std::string& name) const;
  std::shared_ptr<Blob> GetBlob(const std::string& name) const;
  std::shared_ptr<Blob> CreateBlob(const std::string& name, DataType data_type, Allocator* allocator = nullptr);
  std::shared_ptr<Blob> CreateBlob(const std::string& name, const std::string& data_type_str,
                                   Allocator* allocator = nullptr);
  std::shared_ptr<Blob> CreateTempBlob(const std::vector<int>& shape, DataType data_type);
  void GrowTempBuffer(size_t raw_size);
  size_t GetWorkspaceSize() const;
  size_t GetWorkspaceTempSize() const;

 private:
  std::shared_ptr<Context> context_;
  std::map<std::string, std::shared_ptr<Blob>> blobs_;
  size_t temp_offset_ = 0;
};

// ---------------------------------------------------------------------------------------------
// Kernel registry (shadow/core/kernel.hpp:13-41, kernel.cpp:5-56)
// ---------------------------------------------------------------------------------------------
class Kernel {
 public:
  virtual ~Kernel() = default;
  virtual DeviceType device_type() const = 0;
  virtual std::string kernel_type() const = 0;
};

VecString GetKernelKeys(DeviceType device_type);
VecString GetKernelKeys(const std::string& op_type, DeviceType device_type);
std::shared_ptr<Kernel> CreateKernel(const std::string& op_type, DeviceType device_type,
                                     const std::string& kernel_type = "");
SHADOW_DECLARE_REGISTRY(KernelRegistry, Kernel);

#define REGISTER_OP_KERNEL(name, ...) SHADOW_REGISTER_CLASS(KernelRegistry, name, __VA_ARGS__)
#define REGISTER_OP_KERNEL_DEFAULT(name, ...) REGISTER_OP_KERNEL(name(Default), __VA_ARGS__)
#define REGISTER_OP_KERNEL_DNNL(name, ...) REGISTER_OP_KERNEL(name(DNNL), __VA_ARGS__)
#define REGISTER_OP_KERNEL_CUDNN(name, ...) REGISTER_OP_KERNEL(name(CUDNN), __VA_ARGS__)

// ---------------------------------------------------------------------------------------------
// Operator (shadow/core/operator.hpp:19-79, operator.cpp:5-46)
// ---------------------------------------------------------------------------------------------
class Operator {
 public:
  Operator(const shadow::OpParam& op_param, Workspace* ws);
  virtual ~Operator() = default;

  virtual void Run(const std::vector<std::shared_ptr<Blob>>& inputs,
                   std::vector<std::shared_ptr<Blob>>& outputs) = 0;

  bool has_argument(const std::string& name) const { return arg_helper_.HasArgument(name); }
  template <typename T>
  T get_single_argument(const std::string& name, const T& default_value) const {
    return arg_helper_.GetSingleArgument<T>(name, default_value);
  }
  template <typename T>
  std::vector<T> get_repeated_argument(const std::string& name, const std::vector<T>& default_value = {}) const {
    return arg_helper_.GetRepeatedArgument<T>(name, default_value);
  }
  template <typename T>
  std::vector<T> get_repeated_argument(const std::string& name, const T& default_value) const {
    const auto& val = arg_helper_.GetRepeatedArgument<T>(name);
    return val.empty() ? std::vector<T>(1, arg_helper_.GetSingleArgument<T>(name, default_value)) : val;
  }

  Workspace* ws() const { return ws_; }
  const shadow::OpParam& op_param() const { return op_param_; }
  const std::string& name() const { return op_param_.name(); }
  const std::string& type() const { return op_param_.type(); }
  std::string debug_log(const std::vector<std::shared_ptr<Blob>>& inputs,
                        const std::vector<std::shared_ptr<Blob>>& outputs) const;

 protected:
  Workspace* ws_ = nullptr;

 private:
  shadow::OpParam op_param_;
  ArgumentHelper arg_helper_;
};

std::shared_ptr<Operator> CreateOperator(const shadow::OpParam& op_param, Workspace* ws);
SHADOW_DECLARE_REGISTRY(OperatorRegistry, Operator, const shadow::OpParam&, Workspace*);
#define REGISTER_OPERATOR(name, ...) SHADOW_REGISTER_CLASS(OperatorRegistry, name, __VA_ARGS__)

// ---------------------------------------------------------------------------------------------
// Backend and Network (shadow/core/backend.hpp:12-41, network.hpp:15-43)
// ---------------------------------------------------------------------------------------------
class Backend {
 public:
  virtual ~Backend() = default;
  virtual void LoadModel(const shadow::NetParam& net_param) = 0;
  virtual void Run(const std::map<std::string, void*>& data_map,
                   const std::map<std::string, std::vector<int>>& shape_map) = 0;
  virtual void SaveEngine(const std::string& save_path, std::map<std::string, std::vector<char>>* save_data) = 0;
  const ArgumentHelper& arg_helper() const { return arg_helper_; }
  const std::shared_ptr<Workspace>& ws() const { return ws_; }
  const std::vector<std::string>& in_blob() const { return in_blob_; }
  const std::vector<std::string>& out_blob() const { return out_blob_; }

 protected:
  ArgumentHelper arg_helper_;
  std::shared_ptr<Workspace> ws_;
  std::vector<std::string> in_blob_, out_blob_;
};

std::shared_ptr<Backend> CreateBackend(const ArgumentHelper& arguments);
SHADOW_DECLARE_REGISTRY(BackendRegistry, Backend, const ArgumentHelper&);
#define REGISTER_BACKEND(name, ...) SHADOW_REGISTER_CLASS(BackendRegistry, name, __VA_ARGS__)

class Network {
 public:
  Network();
  void LoadXModel(const shadow::NetParam& net_param, const ArgumentHelper& arguments);
  void Forward(const std::map<std::string, void*>& data_map,
               const std::map<std::string, std::vector<int>>& shape_map = {});
  template <typename T>
  const T* GetBlobDataByName(const std::string& blob_name, const std::string& locate = "host");
  template <typename T>
  std::vector<int> GetBlobShapeByName(const std::string& blob_name) const;
  const std::vector<std::string>& in_blob() const;
  const std::vector<std::string>& out_blob() const;
  bool has_argument(const std::string& name) const;
  template <typename T>
  T get_single_argument(const std::string& name, const T& default_value) const;
  template <typename T>
  std::vector<T> get_repeated_argument(const std::string& name, const std::vector<T>& default_value = {}) const;

 private:
  std::shared_ptr<Backend> backend_;
};

// ---------------------------------------------------------------------------------------------
// Model text format (shadow/util/io.hpp:47-52 in a build without protobuf; format in
// shadow/core/parser.cpp:1034-1917).  Throws (CHECK) on malformed text or on an operator type
// this library does not have; ReadProtoFromTextFile returns false when the file cannot be opened.
// ---------------------------------------------------------------------------------------------
namespace IO {
// ReadProtoFromText takes either text form: the line-based one (it starts with '[') or protobuf text
// format (`.shadowtxt`, what TextFormat prints for shadow/proto/shadow.proto; shadow/util/io.hpp:20-22).
bool ReadProtoFromText(const std::string& proto_text, shadow::NetParam* proto);
bool ReadProtoFromTextFile(const std::string& proto_file, shadow::NetParam* proto);
// protobuf text format only, for either top-level message
bool ReadProtoFromProtoText(const std::string& proto_text, shadow::NetParam* proto);
bool ReadProtoFromProtoText(const std::string& proto_text, shadow::MetaNetParam* proto);
// Protobuf binary models (shadow/util/io.hpp:20-27; messages of shadow/proto/shadow.proto), decoded
// without a protobuf runtime.  Throw (CHECK) on malformed input; the file forms return false when the
// file cannot be opened.
bool ReadProtoFromArray(const void* proto_data, int proto_size, shadow::NetParam* proto);
bool ReadProtoFromArray(const void* proto_data, int proto_size, shadow::MetaNetParam* proto);
bool ReadProtoFromBinaryFile(const std::string& proto_file, shadow::NetParam* proto);
bool ReadProtoFromBinaryFile(const std::string& proto_file, shadow::MetaNetParam* proto);
}  // namespace IO

}  // namespace Shadow

#endif  // SHADOW_B200_HOST_SHADOW_API_HPP_
