/*
 * C view of the Shadow `Network` / `NetParam` public API, for callers that cannot
 * include C++ headers (the Python tests and the benchmark bind it with ctypes).
 *
 * It is NOT the kernel boundary (that is sb200.h); it is a thin adapter over the
 * C++ API declared in shadow/core/network.hpp:15-43 (Network::LoadXModel, Forward,
 * GetBlobDataByName, GetBlobShapeByName) and shadow/core/helper.hpp:36-58
 * (add_s_i / add_s_f / add_v_i / add_v_f / add_s_s / add_v_s on OpParam and NetParam).
 *
 * One source file implements it (shadow_b200/host/net_capi.cpp).  Compiled against
 * this repository's host library it exports the symbols with the prefix `sb200net_`;
 * compiled against the reference's own headers (the oracle build does that) it
 * exports the same functions with the prefix `sref_`.  The prefix is chosen with
 * -DSHADOW_CAPI_PREFIX=<prefix>.
 *
 * Error convention: the C++ API reports errors by throwing std::runtime_error
 * (shadow/util/log.hpp:111-117).  Every function here catches, stores the message in
 * a thread-local buffer readable through <prefix>last_error(), and returns non-zero
 * (or NULL).
 */
#ifndef SHADOW_NET_CAPI_H_
#define SHADOW_NET_CAPI_H_

#ifdef __cplusplus
extern "C" {
#endif

#ifndef SHADOW_CAPI_PREFIX
#define SHADOW_CAPI_PREFIX sb200net_
#endif
#define SHADOW_CAPI_CAT2(a, b) a##b
#define SHADOW_CAPI_CAT(a, b) SHADOW_CAPI_CAT2(a, b)
#define SHADOW_CAPI(name) SHADOW_CAPI_CAT(SHADOW_CAPI_PREFIX, name)

/* Argument kinds: which field of shadow::Argument (shadow/proto/shadow.proto:14-22)
 * the values go to.  Numeric values travel as doubles (every int and float is exact
 * in a double); strings travel in `arg_strings`. */
enum {
  SHADOW_ARG_S_I = 0, /* one int (bools ride here, shadow/core/helper.cpp:50-51) */
  SHADOW_ARG_S_F = 1, /* one float */
  SHADOW_ARG_V_I = 2, /* repeated int */
  SHADOW_ARG_V_F = 3, /* repeated float */
  SHADOW_ARG_S_S = 4, /* one string  */
  SHADOW_ARG_V_S = 5  /* repeated string */
};

/* A net under construction (shadow::NetParam) that becomes a loaded Shadow::Network. */
void* SHADOW_CAPI(net_create)(const char* net_name);
void SHADOW_CAPI(net_destroy)(void* net);

/* Append one shadow::OpParam.  `arg_counts[i]` values of argument i are taken from the
 * running position in `arg_values` (kinds 0..3) or `arg_strings` (kinds 4..5). */
int SHADOW_CAPI(net_add_op)(void* net, const char* type, const char* name, int n_bottom,
                            const char* const* bottoms, int n_top, const char* const* tops,
                            int n_arg, const char* const* arg_names, const int* arg_kinds,
                            const int* arg_counts, const double* arg_values,
                            const char* const* arg_strings);

/* Append one weight blob (shadow::Blob with data_f) to the NetParam. */
int SHADOW_CAPI(net_add_blob)(void* net, const char* name, int ndim, const int* shape,
                              const float* data);

/* Replace the NetParam under construction by the one IO::ReadProtoFromText parses from `text`
 * (the protobuf-free model text format, shadow/util/io.hpp:47-52, shadow/core/parser.cpp:1844-1917). */
int SHADOW_CAPI(net_parse_text)(void* net, const char* text);

#ifdef SHADOW_CAPI_PRODUCT_EXTENSIONS
/* Only in this repository's build of the adapter (the reference's protobuf-free build has no binary
 * reader to compare with).
 * net_parse_binary: replace the NetParam under construction by the one decoded from a protobuf
 * binary model (IO::ReadProtoFromArray); with `network` >= 0 the bytes are a MetaNetParam and that
 * network of it is taken.
 * net_dump: write a line-based description of the NetParam under construction into `buf` (at most
 * `cap` bytes including the terminator) and return the length it needs; floats are written as C99
 * hexadecimal literals so that they compare exactly.  Lines:
 *   net <name> / netarg|arg <name> <kind> <values...> / blob <name> <type> <ndim> <dims...> <n data_f> <values...>
 *   / op <type> <name> <n bottoms> <bottoms...> <n tops> <tops...> <n args>  (its arg lines follow). */
int SHADOW_CAPI(net_parse_binary)(void* net, const void* data, int size, int network);
int SHADOW_CAPI(net_dump)(void* net, char* buf, int cap);
#endif

/* Network::LoadXModel with backend arguments backend_type / device_id and the net
 * argument out_blob (mandatory, shadow/backends/native/native.cpp:186-188). */
int SHADOW_CAPI(net_load)(void* net, const char* backend_type, int device_id, int n_out,
                          const char* const* out_blobs);

/* Network::Forward(data_map): copies each named host buffer into its input blob, runs
 * every operator in order, synchronises.  n_in == 0 re-runs the operators on the data
 * already in the blobs. */
int SHADOW_CAPI(net_forward)(void* net, int n_in, const char* const* names,
                             const void* const* host_ptrs);

/* Network::GetBlobShapeByName; writes at most `cap` dims, returns the number of axes
 * (or -1 on error). */
int SHADOW_CAPI(net_blob_shape)(void* net, const char* name, int* shape, int cap);

/* Network::GetBlobDataByName<float>(name, on_host ? "host" : "device"). */
const float* SHADOW_CAPI(net_blob_data)(void* net, const char* name, int on_host);

const char* SHADOW_CAPI(last_error)(void);

#ifdef __cplusplus
}
#endif
#endif /* SHADOW_NET_CAPI_H_ */
