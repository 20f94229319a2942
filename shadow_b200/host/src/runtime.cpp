// Data runtime behind the Shadow API: logging, arguments, CUDA allocator/context, Blob, Workspace.
#include <cuda_runtime.h>

#include <cstdlib>
#include <iostream>
#include <numeric>

#include "shadow_api.hpp"

namespace Shadow {

// ---- logging ------------------------------------------------------------------------------------
LogMessage::LogMessage(const char* severity, const char* file, int line) : severity_(severity) {
  std::string path(file);
  const auto slash = path.find_last_of("/\\");
  stream_ << severity << ": " << (slash == std::string::npos ? path : path.substr(slash + 1)) << ":" << line
          << "] ";
}

LogMessage::~LogMessage() noexcept(false) {
  const std::string msg = stream_.str();
  (severity_ == "INFO" ? std::cout : std::cerr) << msg << std::endl;
  if (severity_ == "FATAL") throw std::runtime_error(msg);
}

#define CUDA_CHECK(expr)                                                        \
  do {                                                                          \
    cudaError_t sb_err = (expr);                                                \
    CHECK_EQ(sb_err, cudaSuccess) << #expr << ": " << cudaGetErrorString(sb_err); \
  } while (0)

void registry_duplicate_key(const std::string& key) {
  std::cerr << "Key: " << key << " is already registered" << std::endl;
  std::exit(1);
}

// ---- arguments ----------------------------------------------------------------------------------
void ArgumentHelper::Absorb(const std::vector<shadow::Argument>& args, const std::string& owner) {
  for (const auto& arg : args) {
    CHECK(!HasArgument(arg.name())) << "Duplicated argument name: " << arg.name() << " found in def: " << owner;
    arguments_[arg.name()] = arg;
  }
}

#define SB_SINGLE_ARG(field, T)                                                                        \
  template <>                                                                                          \
  T ArgumentHelper::GetSingleArgument<T>(const std::string& name, const T& default_value) const {      \
    auto it = arguments_.find(name);                                                                   \
    if (it == arguments_.end()) return default_value;                                                  \
    CHECK(it->second.has_##field());                                                                   \
    return static_cast<T>(it->second.field());                                                         \
  }                                                                                                    \
  template <>                                                                                          \
  void ArgumentHelper::AddSingleArgument<T>(const std::string& name, const T& value) {                 \
    CHECK(!HasArgument(name)) << "Duplicated argument name: " << name;                                 \
    shadow::Argument arg;                                                                              \
    arg.set_name(name);                                                                                \
    arg.set_##field(value);                                                                            \
    arguments_[name] = arg;                                                                            \
  }
SB_SINGLE_ARG(s_f, float)
SB_SINGLE_ARG(s_i, int)
SB_SINGLE_ARG(s_i, bool)
SB_SINGLE_ARG(s_s, std::string)
#undef SB_SINGLE_ARG

#define SB_REPEATED_ARG(field, T)                                                                       \
  template <>                                                                                           \
  std::vector<T> ArgumentHelper::GetRepeatedArgument<T>(const std::string& name,                        \
                                                        const std::vector<T>& default_value) const {    \
    auto it = arguments_.find(name);                                                                    \
    if (it == arguments_.end()) return default_value;                                                   \
    std::vector<T> out;                                                                                 \
    for (const auto& v : it->second.field()) out.push_back(static_cast<T>(v));                          \
    return out;                                                                                         \
  }                                                                                                     \
  template <>                                                                                           \
  void ArgumentHelper::AddRepeatedArgument<T>(const std::string& name, const std::vector<T>& value) {   \
    CHECK(!HasArgument(name)) << "Duplicated argument name: " << name;                                  \
    shadow::Argument arg;                                                                               \
    arg.set_name(name);                                                                                 \
    for (const auto& v : value) arg.add_##field(v);                                                     \
    arguments_[name] = arg;                                                                             \
  }
SB_REPEATED_ARG(v_f, float)
SB_REPEATED_ARG(v_i, int)
SB_REPEATED_ARG(v_i, bool)
SB_REPEATED_ARG(v_s, std::string)
#undef SB_REPEATED_ARG

namespace {
template <typename P>
shadow::Argument* new_arg(P* p, const std::string& name) {
  auto* arg = p->add_arg();
  arg->set_name(name);
  return arg;
}
}  // namespace

#define SB_ADD_HELPERS(P)                                                                              \
  void add_s_f(P* p, const std::string& n, const float& v) { new_arg(p, n)->set_s_f(v); }               \
  void add_s_i(P* p, const std::string& n, const int& v) { new_arg(p, n)->set_s_i(v); }                 \
  void add_s_i(P* p, const std::string& n, const bool& v) { new_arg(p, n)->set_s_i(v ? 1 : 0); }        \
  void add_s_s(P* p, const std::string& n, const std::string& v) { new_arg(p, n)->set_s_s(v); }         \
  void add_v_f(P* p, const std::string& n, const std::vector<float>& v) {                               \
    auto* a = new_arg(p, n);                                                                            \
    for (float x : v) a->add_v_f(x);                                                                    \
  }                                                                                                     \
  void add_v_i(P* p, const std::string& n, const std::vector<int>& v) {                                 \
    auto* a = new_arg(p, n);                                                                            \
    for (int x : v) a->add_v_i(x);                                                                      \
  }                                                                                                     \
  void add_v_i(P* p, const std::string& n, const std::vector<bool>& v) {                                \
    auto* a = new_arg(p, n);                                                                            \
    for (bool x : v) a->add_v_i(x ? 1 : 0);                                                             \
  }                                                                                                     \
  void add_v_s(P* p, const std::string& n, const std::vector<std::string>& v) {                         \
    auto* a = new_arg(p, n);                                                                            \
    for (const auto& x : v) a->add_v_s(x);                                                              \
  }
SB_ADD_HELPERS(shadow::NetParam)
SB_ADD_HELPERS(shadow::OpParam)
#undef SB_ADD_HELPERS

// ---- data types ---------------------------------------------------------------------------------
size_t data_type_size(DataType type) {
  switch (type) {
    case DataType::kI64: case DataType::kU64: return 8;
    case DataType::kI32: case DataType::kU32: case DataType::kF32: return 4;
    case DataType::kI16: case DataType::kU16: return 2;
    case DataType::kI8: case DataType::kU8: return 1;
    case DataType::kBool: return sizeof(bool);
  }
  return 0;
}

template <> DataType data_type_of<std::int64_t>() { return DataType::kI64; }
template <> DataType data_type_of<std::int32_t>() { return DataType::kI32; }
template <> DataType data_type_of<std::int16_t>() { return DataType::kI16; }
template <> DataType data_type_of<std::int8_t>() { return DataType::kI8; }
template <> DataType data_type_of<std::uint64_t>() { return DataType::kU64; }
template <> DataType data_type_of<std::uint32_t>() { return DataType::kU32; }
template <> DataType data_type_of<std::uint16_t>() { return DataType::kU16; }
template <> DataType data_type_of<std::uint8_t>() { return DataType::kU8; }
template <> DataType data_type_of<float>() { return DataType::kF32; }
template <> DataType data_type_of<bool>() { return DataType::kBool; }

// ---- CUDA allocator and context -----------------------------------------------------------------
namespace {

// Device memory through the CUDA runtime; copies are asynchronous on the context stream.  A
// device -> host read is followed by a stream synchronisation so that the host buffer is valid
// when read() returns (the reference leaves this to the pageable-memory staging of
// cudaMemcpyAsync, shadow/core/allocator.cu:20-27).
class GpuAllocator : public Allocator {
 public:
  DeviceType device_type() const override { return DeviceType::kGPU; }
  void* malloc(size_t size, const void* host_ptr) const override {
    void* ptr = nullptr;
    CUDA_CHECK(cudaMalloc(&ptr, size));
    if (host_ptr != nullptr) write(size, host_ptr, ptr);
    return ptr;
  }
  void read(size_t size, const void* src, void* dst) const override {
    CUDA_CHECK(cudaMemcpyAsync(dst, src, size, cudaMemcpyDeviceToHost, stream_));
    CUDA_CHECK(cudaStreamSynchronize(stream_));
  }
  void write(size_t size, const void* src, void* dst) const override {
    CUDA_CHECK(cudaMemcpyAsync(dst, src, size, cudaMemcpyHostToDevice, stream_));
  }
  void copy(size_t size, const void* src, void* dst) const override {
    CUDA_CHECK(cudaMemcpyAsync(dst, src, size, cudaMemcpyDeviceToDevice, stream_));
  }
  void free(void* ptr) const override {
    // frees are ordered after work already queued on the stream
    CUDA_CHECK(cudaStreamSynchronize(stream_));
    CUDA_CHECK(cudaFree(ptr));
  }
  void set_stream(void* stream) override { stream_ = static_cast<cudaStream_t>(stream); }

 private:
  cudaStream_t stream_ = nullptr;
};

class GpuContext : public Context {
 public:
  explicit GpuContext(const ArgumentHelper& arguments) {
    device_id_ = arguments.GetSingleArgument<int>("device_id", 0);
    per_thread_stream_ = arguments.GetSingleArgument<bool>("default_cuda_stream", false);
    int num_devices = 0;
    CUDA_CHECK(cudaGetDeviceCount(&num_devices));
    CHECK_GE(device_id_, 0);
    CHECK_LT(device_id_, num_devices);
    CUDA_CHECK(cudaSetDevice(device_id_));
    if (per_thread_stream_) {
      stream_ = cudaStreamPerThread;
    } else {
      CUDA_CHECK(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    }
    allocator_ = std::make_shared<GpuAllocator>();
    allocator_->set_stream(stream_);
  }
  ~GpuContext() override {
    if (stream_ != nullptr && !per_thread_stream_) cudaStreamDestroy(stream_);
  }
  Allocator* allocator() const override { return allocator_.get(); }
  DeviceType device_type() const override { return DeviceType::kGPU; }
  int device_id() const override { return device_id_; }
  void switch_device() override { CUDA_CHECK(cudaSetDevice(device_id_)); }
  void synchronize() override { CUDA_CHECK(cudaStreamSynchronize(stream_)); }
  void* stream() const override { return stream_; }

 private:
  int device_id_ = 0;
  bool per_thread_stream_ = false;
  cudaStream_t stream_ = nullptr;
  std::shared_ptr<GpuAllocator> allocator_;
};

}  // namespace

template <>
std::shared_ptr<Allocator> GetAllocator<DeviceType::kGPU>() {
  return std::make_shared<GpuAllocator>();
}
template <>
std::shared_ptr<Context> GetContext<DeviceType::kGPU>(const ArgumentHelper& arguments) {
  return std::make_shared<GpuContext>(arguments);
}

// ---- Blob ---------------------------------------------------------------------------------------
Blob::Blob(std::string name, DataType data_type, Allocator* allocator)
    : name_(std::move(name)), data_type_(data_type), allocator_(allocator) {
  CHECK_NOTNULL(allocator_);
}

Blob::~Blob() {
  try {
    if (data_ != nullptr && !shared_) allocator_->free(data_);
  } catch (const std::exception&) {
    // a failing cudaFree while tearing down must not escape a destructor
  }
  data_ = nullptr;
}

size_t Blob::count64() const {
  size_t n = 1;
  for (int d : shape_) n *= static_cast<size_t>(d);
  return n;
}

int Blob::count(int start_axis, int end_axis) const {
  CHECK_LE(start_axis, end_axis);
  CHECK_GE(start_axis, 0);
  CHECK_LE(end_axis, num_axes());
  int n = 1;
  for (int i = start_axis; i < end_axis; ++i) n *= shape_[i];
  return n;
}

int Blob::canonical_index(int index) const {
  CHECK_GE(index, -num_axes());
  CHECK_LT(index, num_axes());
  return index < 0 ? index + num_axes() : index;
}

void Blob::require_type(DataType asked) const { CHECK(asked == data_type_) << "blob " << name_ << " type mismatch"; }

void Blob::upload(const void* host, size_t bytes, size_t byte_offset, size_t end_elem) {
  CHECK_NOTNULL(host);
  CHECK_LE(end_elem, count64());
  CHECK_NOTNULL(data_);
  allocator_->write(bytes, host, static_cast<unsigned char*>(data_) + byte_offset);
}

void Blob::download(void* host, size_t bytes, size_t byte_offset) const {
  CHECK_NOTNULL(data_);
  allocator_->read(bytes, static_cast<const unsigned char*>(data_) + byte_offset, host);
}

void Blob::share_data(const void* data, const std::vector<int>& shape) {
  CHECK_NOTNULL(data);
  if (data_ != nullptr && !shared_) allocator_->free(data_);
  data_ = const_cast<void*>(data);
  shape_ = shape;
  capacity_ = 0;
  shared_ = true;
  CHECK_GT(count64(), 0u);
}

// Grow-only: a larger shape frees and reallocates, a smaller one keeps the buffer.
void Blob::reshape(const std::vector<int>& shape) {
  size_t n = 1;
  for (int d : shape) {
    CHECK_GT(d, 0);
    n *= static_cast<size_t>(d);
  }
  if (data_ != nullptr && !shared_ && n > capacity_) {
    allocator_->free(data_);
    data_ = nullptr;
  }
  if (data_ == nullptr || shared_) {
    data_ = allocator_->malloc(n * elem_size(), nullptr);
    capacity_ = n;
  }
  shape_ = shape;
  shared_ = false;
}

// ---- Workspace ----------------------------------------------------------------------------------
Workspace::Workspace(const ArgumentHelper& arguments) {
  // Every backend type runs on the GPU here; the reference picks the GPU context for "Native"
  // (shadow/core/workspace.cpp:5-17) and there is no CPU context in this library.
  context_ = GetContext<DeviceType::kGPU>(arguments);
}

DataType Workspace::GetBlobDataType(const std::string& name) const {
  CHECK(HasBlob(name)) << "Unknown blob: " + name;
  return blobs_.at(name)->data_type();
}

std::vector<int> Workspace::GetBlobShape(const std::string& name) const {
  CHECK(HasBlob(name)) << "Unknown blob: " + name;
  return blobs_.at(name)->shape();
}

std::shared_ptr<Blob> Workspace::GetBlob(const std::string& name) const {
  auto it = blobs_.find(name);
  return it == blobs_.end() ? nullptr : it->second;
}

std::shared_ptr<Blob> Workspace::CreateBlob(const std::string& name, DataType data_type, Allocator* allocator) {
  auto it = blobs_.find(name);
  if (it != blobs_.end()) return it->second;
  auto blob = std::make_shared<Blob>(name, data_type, allocator != nullptr ? allocator : context_->allocator());
  blobs_[name] = blob;
  return blob;
}

std::shared_ptr<Blob> Workspace::CreateBlob(const std::string& name, const std::string& type, Allocator* allocator) {
  static const std::map<std::string, DataType> kTypes = {
      {"int64", DataType::kI64}, {"int32", DataType::kI32}, {"int16", DataType::kI16}, {"int8", DataType::kI8},
      {"uint64", DataType::kU64}, {"uint32", DataType::kU32}, {"uint16", DataType::kU16}, {"uint8", DataType::kU8},
      {"float", DataType::kF32}, {"bool", DataType::kBool}};
  auto it = kTypes.find(type);
  return it == kTypes.end() ? nullptr : CreateBlob(name, it->second, allocator);
}

// The temp buffer is one I32 blob named "temp_blob" (as in the reference, so GetWorkspaceTempSize
// and blob listings agree); CreateTempBlob hands out 256-byte aligned slices of it.
void Workspace::GrowTempBuffer(size_t raw_size) {
  auto temp = CreateBlob("temp_blob", DataType::kI32);
  const size_t ints = raw_size / sizeof(int) + 1;
  CHECK_LE(ints, static_cast<size_t>(0x7fffffff));
  temp->reshape({static_cast<int>(ints)});
  temp_offset_ = 0;
}

std::shared_ptr<Blob> Workspace::CreateTempBlob(const std::vector<int>& shape, DataType data_type) {
  size_t n = 1;
  for (int d : shape) n *= static_cast<size_t>(d);
  CHECK_GT(n, 0u);
  auto temp = GetBlob("temp_blob");
  CHECK_NOTNULL(temp);
  auto blob = std::make_shared<Blob>("temp", data_type, context_->allocator());
  const size_t bytes = n * blob->elem_size();
  // keep slices 256-byte aligned when the buffer has room for the padding, else pack them
  size_t offset = (temp_offset_ + 255) / 256 * 256;
  if (offset + bytes > temp->max_size()) offset = temp_offset_;
  CHECK_LE(offset + bytes, temp->max_size());
  blob->share_data(temp->data<unsigned char>() + offset, shape);
  temp_offset_ = offset + bytes;
  return blob;
}

size_t Workspace::GetWorkspaceSize() const {
  size_t bytes = 0;
  for (const auto& kv : blobs_) bytes += kv.second->max_size();
  return bytes;
}

size_t Workspace::GetWorkspaceTempSize() const {
  auto temp = GetBlob("temp_blob");
  return temp != nullptr ? temp->max_size() : 0;
}

}  // namespace Shadow
