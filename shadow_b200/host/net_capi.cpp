// C adapter over the Shadow Network / NetParam C++ API (see include/shadow_net_capi.h).
//
// The only Shadow headers it needs are the public ones: core/network.hpp
// (Network, shadow/core/network.hpp:15-43) and core/helper.hpp (ArgumentHelper and the
// add_* helpers, shadow/core/helper.hpp:10-58).  It therefore compiles unchanged against
// this repository's host library and against the reference's own headers, which is how
// the same op graph is driven on both sides of a parity test.
#include "shadow_net_capi.h"

#include "core/helper.hpp"
#include "core/network.hpp"
#include "util/io.hpp"

#include <cstdio>
#include <cstring>
#include <exception>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

thread_local std::string g_last_error;

struct NetHandle {
  shadow::NetParam param;
  std::unique_ptr<Shadow::Network> network;
};

template <typename F>
int guarded(F&& body) {
  try {
    body();
    return 0;
  } catch (const std::exception& e) {
    g_last_error = e.what();
  } catch (...) {
    g_last_error = "unknown C++ exception";
  }
  return 1;
}

}  // namespace

extern "C" {

void* SHADOW_CAPI(net_create)(const char* net_name) {
  auto* handle = new NetHandle;
  handle->param.set_name(net_name != nullptr ? net_name : "net");
  return handle;
}

void SHADOW_CAPI(net_destroy)(void* net) { delete static_cast<NetHandle*>(net); }

int SHADOW_CAPI(net_add_op)(void* net, const char* type, const char* name, int n_bottom,
                            const char* const* bottoms, int n_top, const char* const* tops,
                            int n_arg, const char* const* arg_names, const int* arg_kinds,
                            const int* arg_counts, const double* arg_values,
                            const char* const* arg_strings) {
  return guarded([&] {
    auto* op = static_cast<NetHandle*>(net)->param.add_op();
    op->set_type(type);
    op->set_name(name);
    for (int i = 0; i < n_bottom; ++i) op->add_bottom(bottoms[i]);
    for (int i = 0; i < n_top; ++i) op->add_top(tops[i]);
    int vpos = 0, spos = 0;
    for (int a = 0; a < n_arg; ++a) {
      const std::string key(arg_names[a]);
      const int cnt = arg_counts[a];
      switch (arg_kinds[a]) {
        case SHADOW_ARG_S_I:
          Shadow::add_s_i(op, key, static_cast<int>(arg_values[vpos]));
          vpos += 1;
          break;
        case SHADOW_ARG_S_F:
          Shadow::add_s_f(op, key, static_cast<float>(arg_values[vpos]));
          vpos += 1;
          break;
        case SHADOW_ARG_V_I: {
          std::vector<int> v;
          for (int k = 0; k < cnt; ++k) v.push_back(static_cast<int>(arg_values[vpos + k]));
          Shadow::add_v_i(op, key, v);
          vpos += cnt;
          break;
        }
        case SHADOW_ARG_V_F: {
          std::vector<float> v;
          for (int k = 0; k < cnt; ++k) v.push_back(static_cast<float>(arg_values[vpos + k]));
          Shadow::add_v_f(op, key, v);
          vpos += cnt;
          break;
        }
        case SHADOW_ARG_S_S:
          Shadow::add_s_s(op, key, std::string(arg_strings[spos]));
          spos += 1;
          break;
        case SHADOW_ARG_V_S: {
          std::vector<std::string> v;
          for (int k = 0; k < cnt; ++k) v.emplace_back(arg_strings[spos + k]);
          Shadow::add_v_s(op, key, v);
          spos += cnt;
          break;
        }
        default:
          throw std::runtime_error("net_add_op: unknown argument kind");
      }
    }
  });
}

int SHADOW_CAPI(net_add_blob)(void* net, const char* name, int ndim, const int* shape,
                              const float* data) {
  return guarded([&] {
    auto* blob = static_cast<NetHandle*>(net)->param.add_blob();
    blob->set_name(name);
    blob->set_type("float");
    size_t count = 1;
    for (int i = 0; i < ndim; ++i) {
      blob->add_shape(shape[i]);
      count *= static_cast<size_t>(shape[i]);
    }
    if (data != nullptr) {
      for (size_t i = 0; i < count; ++i) blob->add_data_f(data[i]);
    }
  });
}

int SHADOW_CAPI(net_parse_text)(void* net, const char* text) {
  return guarded([&] {
    auto* handle = static_cast<NetHandle*>(net);
    if (handle == nullptr || text == nullptr) throw std::runtime_error("net_parse_text: null argument");
    shadow::NetParam parsed;
    if (!Shadow::IO::ReadProtoFromText(text, &parsed)) throw std::runtime_error("net_parse_text: the text could not be parsed");
    handle->param = parsed;
  });
}

#ifdef SHADOW_CAPI_PRODUCT_EXTENSIONS
int SHADOW_CAPI(net_parse_binary)(void* net, const void* data, int size, int network) {
  return guarded([&] {
    auto* handle = static_cast<NetHandle*>(net);
    if (handle == nullptr || data == nullptr || size < 0) throw std::runtime_error("net_parse_binary: bad argument");
    if (network < 0) {
      shadow::NetParam parsed;
      Shadow::IO::ReadProtoFromArray(data, size, &parsed);
      handle->param = parsed;
    } else {
      shadow::MetaNetParam meta;
      Shadow::IO::ReadProtoFromArray(data, size, &meta);
      if (network >= meta.network_size()) throw std::runtime_error("net_parse_binary: the file holds fewer networks");
      handle->param = meta.network(network);
    }
  });
}

int SHADOW_CAPI(net_dump)(void* net, char* buf, int cap) {
  auto* handle = static_cast<NetHandle*>(net);
  if (handle == nullptr) return -1;
  std::string out;
  char num[64];
  auto hexf = [&](float v) { std::snprintf(num, sizeof(num), " %a", static_cast<double>(v)); out += num; };
  auto dump_arg = [&](const char* word, const shadow::Argument& a) {
    out += std::string(word) + " " + a.name();
    if (a.has_s_f()) { out += " s_f"; hexf(a.s_f()); }
    else if (a.has_s_i()) out += " s_i " + std::to_string(a.s_i());
    else if (a.has_s_s()) out += " s_s " + a.s_s();
    else if (a.v_f_size() > 0) { out += " v_f"; for (float v : a.v_f()) hexf(v); }
    else if (a.v_s_size() > 0) { out += " v_s"; for (const auto& v : a.v_s()) out += " " + v; }
    else { out += " v_i"; for (int v : a.v_i()) out += " " + std::to_string(v); }
    out += "\n";
  };
  const auto& p = handle->param;
  out += "net " + p.name() + "\n";
  for (const auto& a : p.arg()) dump_arg("netarg", a);
  for (const auto& b : p.blob()) {
    out += "blob " + b.name() + " " + (b.has_type() ? b.type() : std::string("float")) + " " + std::to_string(b.shape_size());
    for (int d : b.shape()) out += " " + std::to_string(d);
    out += " " + std::to_string(b.data_f_size());
    for (float v : b.data_f()) hexf(v);
    out += "\n";
  }
  for (const auto& op : p.op()) {
    out += "op " + op.type() + " " + op.name() + " " + std::to_string(op.bottom_size());
    for (const auto& s : op.bottom()) out += " " + s;
    out += " " + std::to_string(op.top_size());
    for (const auto& s : op.top()) out += " " + s;
    out += " " + std::to_string(op.arg_size()) + "\n";
    for (const auto& a : op.arg()) dump_arg("arg", a);
  }
  if (buf != nullptr && cap > 0) {
    const size_t n = out.size() < static_cast<size_t>(cap - 1) ? out.size() : static_cast<size_t>(cap - 1);
    std::memcpy(buf, out.data(), n);
    buf[n] = 0;
  }
  return static_cast<int>(out.size() + 1);
}
#endif

int SHADOW_CAPI(net_load)(void* net, const char* backend_type, int device_id, int n_out,
                          const char* const* out_blobs) {
  return guarded([&] {
    auto* handle = static_cast<NetHandle*>(net);
    std::vector<std::string> outs;
    for (int i = 0; i < n_out; ++i) outs.emplace_back(out_blobs[i]);
    Shadow::add_v_s(&handle->param, "out_blob", outs);
    Shadow::ArgumentHelper backend_args;
    backend_args.AddSingleArgument<std::string>("backend_type", backend_type);
    backend_args.AddSingleArgument<int>("device_id", device_id);
    handle->network.reset(new Shadow::Network());
    handle->network->LoadXModel(handle->param, backend_args);
  });
}

int SHADOW_CAPI(net_forward)(void* net, int n_in, const char* const* names,
                             const void* const* host_ptrs) {
  return guarded([&] {
    auto* handle = static_cast<NetHandle*>(net);
    if (!handle->network) throw std::runtime_error("net_forward: net is not loaded");
    std::map<std::string, void*> data_map;
    for (int i = 0; i < n_in; ++i) data_map[names[i]] = const_cast<void*>(host_ptrs[i]);
    handle->network->Forward(data_map);
  });
}

int SHADOW_CAPI(net_blob_shape)(void* net, const char* name, int* shape, int cap) {
  int ndim = -1;
  guarded([&] {
    auto* handle = static_cast<NetHandle*>(net);
    if (!handle->network) throw std::runtime_error("net_blob_shape: net is not loaded");
    const auto dims = handle->network->GetBlobShapeByName<float>(name);
    for (int i = 0; i < static_cast<int>(dims.size()) && i < cap; ++i) shape[i] = dims[i];
    ndim = static_cast<int>(dims.size());
  });
  return ndim;
}

const float* SHADOW_CAPI(net_blob_data)(void* net, const char* name, int on_host) {
  const float* ptr = nullptr;
  guarded([&] {
    auto* handle = static_cast<NetHandle*>(net);
    if (!handle->network) throw std::runtime_error("net_blob_data: net is not loaded");
    ptr = handle->network->GetBlobDataByName<float>(name, on_host ? "host" : "device");
  });
  return ptr;
}

const char* SHADOW_CAPI(last_error)(void) { return g_last_error.c_str(); }

}  // extern "C"
