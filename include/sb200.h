/*
 * sb200 - C ABI of the B200 (sm_100a) tensor-operator kernels.
 *
 * These are the entry points a Shadow kernel class (`<Op>GPU(Default)` in the kernel registry,
 * shadow/core/kernel.hpp:31-35) calls instead of the reference's `Blas::` / `Vision::` device
 * functions.  Each declaration names the reference interface it replaces.
 *
 * Conventions
 *  - every pointer is a DEVICE pointer to dense row-major float32 data unless it is documented
 *    as a host array (shapes, axes);
 *  - `stream` is a cudaStream_t passed as void* (Context::stream(), shadow/core/context.cu:69-72);
 *    work is enqueued asynchronously on it and the call returns without synchronising;
 *  - the caller's CUDA device must be current (the reference does cudaSetDevice in
 *    Context::switch_device before running operators, shadow/core/context.cu:63);
 *  - nothing here allocates or frees device memory; kernels that need scratch take a
 *    caller-provided buffer (Workspace::GrowTempBuffer / CreateTempBlob,
 *    shadow/core/workspace.cpp:83-123) whose size a *_scratch_bytes query returns;
 *  - in-place operation (y == x) is allowed for the elementwise entry points, as in the
 *    reference (Vision::Activate(out, out, ...), shadow/operators/kernels/conv.hpp:129), and
 *    forbidden for reduce (shadow/operators/reduce_op.cpp:27); softmax also accepts y == x;
 *  - return value: SB200_OK or an error code; bad arguments are rejected before any launch.
 *    Launch errors are read with cudaGetLastError (the reference uses cudaPeekAtLastError in
 *    CUDA_CHECK, shadow/core/external.hpp:39-43); asynchronous faults surface at the caller's
 *    next synchronisation, as in the reference.
 *  - element counts are 64-bit; a single call handles up to 2^40 elements.
 */
#ifndef SB200_H_
#define SB200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  SB200_OK = 0,
  SB200_ERR_BAD_ARGUMENT = 1, /* null pointer, negative size, unknown operation code, bad axis */
  SB200_ERR_UNSUPPORTED = 2,  /* geometry outside what the kernels cover (more than 8 collapsed axes) */
  SB200_ERR_CUDA = 3,         /* a CUDA runtime call or a launch failed; see sb200_last_cuda_error */
  SB200_ERR_SCRATCH = 4       /* scratch buffer missing, misaligned or too small */
};

#define SB200_MAX_AXES 16 /* raw axes accepted; at most 8 remain after collapsing */

const char* sb200_status_string(int status);
/* Text of the CUDA error behind the calling thread's last SB200_ERR_CUDA ("" if none). */
const char* sb200_last_cuda_error(void);
/* Multiprocessor count of the current device (grid sizing uses it); -1 on error. */
int sb200_device_sm_count(void);
/* Number of kernels this library has launched so far in the calling process. */
long long sb200_launch_count(void);

/* Operation codes are the reference's own enums. */
enum { SB200_ADD = 0, SB200_SUB = 1, SB200_MUL = 2, SB200_DIV = 3, SB200_POW = 4, SB200_MAX = 5, SB200_MIN = 6 };
enum {
  SB200_ABS = 0, SB200_SQUARE = 1, SB200_SQRT = 2, SB200_LOG = 3, SB200_EXP = 4, SB200_SIN = 5,
  SB200_COS = 6, SB200_TAN = 7, SB200_ASIN = 8, SB200_ACOS = 9, SB200_ATAN = 10, SB200_FLOOR = 11,
  SB200_CEIL = 12, SB200_NEG = 13, SB200_RECIPROCAL = 14
};
enum {
  SB200_PRELU = 0, SB200_RELU = 1, SB200_LEAKY = 2, SB200_SIGMOID = 3, SB200_SOFTPLUS = 4,
  SB200_TANH = 5, SB200_RELU6 = 6, SB200_HARDSWISH = 7, SB200_GELU = 8
};
enum {
  SB200_RED_PROD = 0, SB200_RED_SUM = 1, SB200_RED_MAX = 2, SB200_RED_MIN = 3, SB200_RED_AVG = 4,
  SB200_RED_L1 = 5, SB200_RED_L2 = 6
};

/* y[i] = val.  Replaces Blas::Set<kGPU,float>(n, val, y, offy, ctx)
 * (shadow/core/blas.hpp:10-11, shadow/core/blas.cu:11-21). */
int sb200_fill(float* y, int64_t n, float val, void* stream);

/* y[i] = f(x[i]), f by SB200_ABS..SB200_RECIPROCAL.  Replaces the fifteen
 * Blas::{Abs..Reciprocal}<kGPU,float>(n, a, offa, y, offy, ctx)
 * (shadow/core/blas.hpp:31-49, shadow/core/blas.cu:77-108), called from
 * UnaryKernelDefault::Run (shadow/operators/kernels/unary.hpp:35-97). */
int sb200_unary(const float* x, float* y, int64_t n, int operation, void* stream);

/* y[i] = act(x[i]) for SB200_RELU..SB200_GELU.  Replaces
 * Vision::Activate<kGPU,float>(in, out, count, type, slope, ctx)
 * (shadow/operators/kernels/activate.hpp:10-12, activate.cu:7-45). */
int sb200_activate(const float* x, float* y, int64_t n, int type, float slope, void* stream);

/* PReLU over x viewed as [outer, channels, dim]: y = x > 0 ? x : x * slope[c], c = channel index,
 * or slope[0] when channel_shared.  Replaces Vision::PRelu<kGPU,float>(in, out, in_shape,
 * channel_shared, slope, ctx) (shadow/operators/kernels/activate.hpp:14-16, activate.cu:47-71);
 * outer = shape[0], channels = shape[1], dim = product of shape[2:]. */
int sb200_prelu(const float* x, float* y, int64_t outer, int64_t channels, int64_t dim,
                const float* slope, int channel_shared, void* stream);

/* y[i] = a[i] op alpha.  Replaces Blas::{Add..Min}<kGPU,float>(n, a, offa, float alpha, y, offy, ctx)
 * (shadow/core/blas.hpp:13-28, shadow/core/blas.cu:50-75). */
int sb200_binary_scalar(const float* a, float alpha, float* y, int64_t n, int operation, void* stream);

/* y[i] = a[i] op b[i].  Replaces Blas::{Add..Min}<kGPU,float>(n, a, offa, b, offb, y, offy, ctx)
 * (shadow/core/blas.hpp:13-28, shadow/core/blas.cu:23-48). */
int sb200_binary(const float* a, const float* b, float* y, int64_t n, int operation, void* stream);

/* N-d broadcast binary.  a_shape, b_shape, out_shape are HOST arrays of num_axes ints (already
 * rank-aligned: each input dim equals the output dim or is 1).  Replaces
 * Vision::BroadcastBinary<kGPU,float>(in, in_shape, scalar, scalar_shape, operation, num_axes, count,
 * out_shape, out, ctx) (shadow/operators/kernels/binary.hpp:11-15, binary.cu:7-64), which takes
 * the three shapes as DEVICE arrays uploaded per call (binary.hpp:84-92); here they are collapsed
 * on the host into strides passed by value, so no temp buffer and no upload is needed. */
int sb200_binary_broadcast(const float* a, const int* a_shape, const float* b, const int* b_shape,
                           const int* out_shape, int num_axes, float* y, int operation, void* stream);

/* y[i] = x[i] * scale[c] + bias[c] with c = (i / inner_num) % scale_num; multiply and add are
 * rounded separately (not fused), as the reference CPU build does.  scale == NULL gives
 * y = x + bias[c], bias == NULL gives y = x * scale[c].  Replaces Vision::ScaleBias / Scale / Bias
 * <kGPU,float>(in, count, scale, bias, scale_num, inner_num, out, ctx)
 * (shadow/operators/kernels/scale.hpp:10-25, scale.cu:7-69). */
int sb200_scale_bias(const float* x, float* y, int64_t n, const float* scale, const float* bias,
                     int64_t scale_num, int64_t inner_num, void* stream);

/* ---- data movement ---------------------------------------------------------------------------
 * Concat / Stack: y viewed as [outer, sum(widths)] receives, side by side in every row, the rows of
 * n_inputs tensors viewed as [outer, widths[k]] (Concat on `axis`: outer = count(0, axis),
 * widths[k] = shape_k(axis) * count(axis + 1); Stack: widths[k] = count(axis) of an input).
 * `inputs` and `widths` are HOST arrays.  One launch per 16 inputs instead of one per input.
 * Replaces Vision::Concat<kGPU,float> / Vision::Stack<kGPU,float> called once per input
 * (shadow/operators/kernels/concat.hpp:30-47, stack.hpp:29-42). */
int sb200_concat(const float* const* inputs, const int64_t* widths, int n_inputs, float* y, int64_t outer,
                 void* stream);

/* Slice: the inverse - x viewed as [outer, sum(widths)] is split into n_outputs tensors
 * [outer, widths[k]].  `outputs` and `widths` are HOST arrays.
 * Replaces Vision::Slice<kGPU,float> called once per output (shadow/operators/kernels/slice.hpp:30-48). */
int sb200_slice(const float* x, float* const* outputs, const int64_t* widths, int n_outputs, int64_t outer,
                void* stream);

/* Permute: y has shape in_shape[order[0]], in_shape[order[1]], ...; y[...] = x[...] with the axes
 * reordered.  in_shape and order are HOST arrays; no index tables are uploaded.  x != y.
 * Replaces Vision::Permute<kGPU,float>(in, count, num_axes, order, old_steps, new_steps, out, ctx)
 * and the three temp blobs of PermuteKernelDefault::Run (shadow/operators/kernels/permute.hpp:27-58). */
int sb200_permute(const float* x, float* y, const int* in_shape, const int* order, int num_axes, void* stream);

/* Gather along one axis: x viewed as [outer, gather_dim, inner], y as [outer, num_indexes, inner],
 * y[o, k, :] = x[o, indexes[k], :].  `indexes` is a DEVICE array of int.  An index outside
 * [0, gather_dim) yields zeros (the reference reads out of bounds).
 * Replaces Vision::Gather<kGPU,float>(in, indexes, num_indexes, gather_dim, inner_num, count, out, ctx)
 * (shadow/operators/kernels/gather.hpp:24-33). */
int sb200_gather(const float* x, const int* indexes, int64_t num_indexes, int64_t outer, int64_t gather_dim,
                 int64_t inner, float* y, void* stream);

/* Pad the last two axes: x viewed as [planes, in_h, in_w], paddings = {top, bottom, left, right}
 * (HOST array; negative values crop), y as [planes, in_h + top + bottom, in_w + left + right];
 * positions outside the input hold `value`.  One pass over y (the reference fills y, then copies rows).
 * Replaces PadKernelDefault<kGPU>::Run = Blas::Set + Vision::Pad (shadow/operators/kernels/pad.hpp:27-44). */
int sb200_pad(const float* x, float* y, int64_t planes, int in_h, int in_w, const int* paddings, float value,
              void* stream);

/* Max (pool_type 0) or average (1) pooling of x viewed as [planes, in_dhw] into y [planes, out_dhw];
 * in_dhw, out_dhw, kernel, stride, pad are HOST arrays of three ints (depth, height, width; 2-D
 * pooling passes depth 1, kernel 1, stride 1, pad 0).  The window of an output starts at
 * index*stride - pad and ends at min(start + kernel, in + pad); the average divides by that size
 * before clipping to the tensor.  The caller supplies out_dhw (the operator front-end's rounding
 * rule decides it).
 * Replaces Vision::Pooling2D<kGPU,float> and Vision::Pooling3D<kGPU,float>
 * (shadow/operators/kernels/pooling.hpp:10-27, pooling.cu). */
int sb200_pooling(const float* x, float* y, int64_t planes, const int* in_dhw, const int* out_dhw, const int* kernel,
                  const int* stride, const int* pad, int pool_type, void* stream);

/* SSD-style L2 normalisation of x[batch, channels, spatial].  across_spatial != 0: one norm per
 * sample, y = x * (1 / sqrt(sum(x*x) + eps)); else one norm per (sample, position) over the
 * channels, y = x / (float)sqrt(sum(x*x) + eps) with the square root taken in double.  Squares are
 * float products accumulated in double.  scale (may be NULL): one value when channel_shared != 0,
 * else one per channel; multiplied in last.  It is read on the device, so no host copy of the
 * shared scale is needed.  No scratch.
 * Replaces SSDNormalizeKernelDefault<kGPU>::Run (shadow/operators/kernels/ssd_normalize.hpp:33-82):
 * Blas::Square + BlasSasum/Mul per sample or Vision::SSDNormalize + BlasSscal / Vision::Scale. */
int sb200_ssd_normalize(const float* x, float* y, int64_t batch, int64_t channels, int64_t spatial,
                        int across_spatial, float eps, const float* scale, int channel_shared, void* stream);

/* Row normalisation of x viewed as [rows, inner] (contiguous rows): mean = sum(x/inner),
 * v = x - mean, var = sum(v*v/inner), y = v / sqrt(var + eps); then, unless affine_mode is 0,
 * y*scale[k] + bias[k] with k = position in the row (affine_mode 1: LayerNorm) or the channel
 * (affine_mode 2: row r belongs to group r % groups of channels_per_group channels of `spatial`
 * elements each, inner == channels_per_group*spatial: GroupNorm; InstanceNorm is groups = channels,
 * channels_per_group = 1).  Terms are accumulated in double as by the reference's CPU Sgemv.
 * No scratch (the reference uses count + inner + 2*rows floats and six launches).
 * Replaces the Default GPU kernels LayerNormKernelDefault<kGPU>::Run
 * (shadow/operators/kernels/layer_norm.hpp:20-75) and GroupNormKernelDefault<kGPU>::Run
 * (shadow/operators/kernels/group_norm.hpp:41-87), i.e. Blas::Set + Blas::BlasSgemv x2 +
 * Vision::SubtractMeanAndSquare + Vision::DivideVariance + Vision::ScaleBias. */
int sb200_row_norm(const float* x, float* y, int64_t rows, int64_t inner, float eps, const float* scale,
                   const float* bias, int affine_mode, int64_t groups, int64_t channels_per_group,
                   int64_t spatial, void* stream);

/* y = x / max(||x||_p, eps), the p-norm over the middle axis of x viewed as [outer, dim, inner];
 * terms accumulated in double as on the reference CPU, quotients correctly rounded.  No scratch:
 * the reference's temporary blob of outer*inner norms is not needed.
 * Replaces Vision::Normalize<kGPU,float>(in, outer_num, dim, inner_num, val, p, eps, out, ctx)
 * (shadow/operators/kernels/normalize.hpp:10-13, normalize.cu). */
int sb200_normalize(const float* x, float* y, int64_t outer, int64_t dim, int64_t inner, float p, float eps,
                    void* stream);

/* Inference batch normalisation: y[i] = (x[i] - mean[c]*scale_factor) / sqrt(|variance[c]*scale_factor| + eps)
 * with c = (i / inner_num) % channels, each step one IEEE float operation as on the reference CPU.
 * Replaces Vision::BatchNorm<kGPU,float>(in, count, mean, variance, channel, inner_num, scale_factor,
 * eps, out, ctx) (shadow/operators/kernels/batch_norm.hpp:10-15, batch_norm.cu). */
int sb200_batch_norm(const float* x, float* y, int64_t n, const float* mean, const float* variance,
                     int64_t channels, int64_t inner_num, float scale_factor, float eps, void* stream);

/* Reduce x (HOST shape in_shape[num_axes]) over the HOST list `axes` (non-negative, distinct,
 * n_axes >= 1) with SB200_RED_*; y receives one float per kept position, row-major over the
 * kept axes.  Prod/Sum/Avg/L1/L2 accumulate in double, Max/Min in float starting from
 * -FLT_MAX/+FLT_MAX with NaNs skipped, as shadow/operators/kernels/reduce.cpp:9-65.
 * Replaces ReduceKernelDefault::Run's table building plus
 * Vision::Reduce<kGPU,float>(in, list, offset, num_list, operation, count, out, ctx)
 * (shadow/operators/kernels/reduce.hpp:10-13,41-90, reduce.cu:7-85): the reference uploads an
 * int offset list with one entry per reduced element on every call; here the geometry is
 * collapsed on the host and no index table exists.
 * `scratch` (256-byte aligned, sb200_reduce_scratch_bytes() bytes, may be NULL when that is 0)
 * holds cross-block partials; its previous contents are ignored. */
int64_t sb200_reduce_scratch_bytes(const int* in_shape, int num_axes, const int* axes, int n_axes,
                                   int operation);
int sb200_reduce(const float* x, const int* in_shape, int num_axes, const int* axes, int n_axes,
                 int operation, float* y, void* scratch, int64_t scratch_bytes, void* stream);

/* Same reduction as sb200_reduce for callers that have no scratch buffer to pass and must not
 * allocate one.  It has no counterpart in the reference (whose kernels always take their temp
 * memory from the Workspace).  Who needs it: code running after all device memory has been handed
 * out for good - a serving loop that sizes every buffer at start-up and forbids allocation on the
 * request path - and callers that hold only the input and output pointers, with no Workspace to
 * grow.  The cross-block partials go to a buffer of SB200_STATIC_SCRATCH_BYTES that is built into
 * the library (a static device array; every GPU that loads the library holds it until the process
 * exits).  Rules that follow from that:
 *  - a reduction whose scratch need (sb200_reduce_scratch_bytes) exceeds the built-in buffer is
 *    refused with SB200_ERR_SCRATCH before anything is launched (sb200_last_cuda_error() says how
 *    many bytes were needed); use sb200_reduce for those;
 *  - the FIRST call on each device looks up the buffer's device address (cudaGetSymbolAddress, no
 *    allocation); make that first call before starting any stream capture on that device;
 *  - all calls on a device share the one buffer and find the previous call's partials in it.
 *    Nothing has to start at zero: every slot a call reads was written by that call's own first
 *    kernel.  But two calls that can run at the same time on one GPU (different streams) would
 *    overwrite each other's partials: keep calls on a device ordered on one stream;
 *  - no cudaMalloc/cudaFree and no allocating library routine is called. */
#define SB200_STATIC_SCRATCH_BYTES (1 << 20)
int sb200_reduce_static(const float* x, const int* in_shape, int num_axes, const int* axes, int n_axes,
                        int operation, float* y, void* stream);

/* Two-step form for a tensor sharded over several GPUs on an axis that is being reduced: step 1
 * writes one DOUBLE partial per kept position (sum for Sum/Avg/L1, sum of squares for L2, product
 * for Prod, max/min value for Max/Min) so the caller can combine the shards' partials (sum, product,
 * max or min across ranks); step 2 turns combined partials into the float result:
 * cast (Sum, Prod, L1, Max, Min), divide by total_reduced_count then cast (Avg),
 * sqrtf((float)p) (L2).  No counterpart in the reference, which is single-device. */
int sb200_reduce_partial(const float* x, const int* in_shape, int num_axes, const int* axes,
                         int n_axes, int operation, double* partial, void* scratch,
                         int64_t scratch_bytes, void* stream);
int sb200_reduce_finalize(const double* partial, float* y, int64_t count, int operation,
                          int64_t total_reduced_count, void* stream);
/* Finalize from SEVERAL partial records without a reducing collective: part p of output o is
 * parts[p * part_stride + o] (for instance the all-gathered records of n_parts ranks); the parts
 * are merged in index order (sum / product / max / min by `operation`) and finished as above.
 * part_stride > count lets one gathered buffer carry the partials of several reductions. */
int sb200_reduce_combine(const double* parts, int64_t n_parts, int64_t part_stride, float* y, int64_t count,
                         int operation, int64_t total_reduced_count, void* stream);

/* Eltwise: y = fold of n_inputs same-size tensors, operation 0 Prod, 1 Sum, 2 Max, 3 Min, folded left
 * to right; Sum computes ((0 + coeff[0]*x0) + coeff[1]*x1) + ... with separately rounded multiply
 * and add (coeff NULL = all ones; coeff is only allowed for Sum).  `inputs` is a HOST array of
 * n_inputs DEVICE pointers, `coeff` a HOST array.  One launch per 8 inputs (the reference makes one
 * pass over the output per input).  Replaces EltwiseKernelDefault<kGPU>::Run
 * (shadow/operators/kernels/eltwise.hpp:19-71) with its Blas::Mul/Max/Min/Set/BlasSaxpy calls. */
int sb200_eltwise(const float* const* inputs, int n_inputs, const float* coeff, float* y, int64_t n,
                  int operation, void* stream);

/* Axpy: out[r*inner + i] = y[...] + alpha[r] * x[...] for r < outer (alpha has one value per
 * (n, c) pair; inner = H*W); multiply and add rounded separately.  Replaces
 * Vision::Axpy<kGPU,float>(alpha, x, y, outer_num, inner_num, out, ctx)
 * (shadow/operators/kernels/axpy.hpp:10-13, axpy.cu). */
int sb200_axpy(const float* alpha, const float* x, const float* y, float* out, int64_t outer, int64_t inner,
               void* stream);

/* Softmax over the middle axis of x viewed as [outer, dim, inner]: max, exp(x - max), sum,
 * divide, all in float.  Replaces Vision::Softmax<kGPU,float>(in, outer, dim, inner, val, out, ctx)
 * (shadow/operators/kernels/softmax.hpp:10-12, softmax.cu:9-70); the reference's `val` scratch of
 * outer*inner floats and its four launches are not needed. */
int sb200_softmax(const float* x, float* y, int64_t outer, int64_t dim, int64_t inner, void* stream);
/* How many blocks of the resident-plane Softmax kernel (planes of about 100..200 KB kept in shared memory
 * and filled by bulk asynchronous copies) have ever given up a bounded wait for their own copies on the
 * current device: 0 on a healthy run; -1 if the counter cannot be read.  Synchronises the device.  A
 * diagnostic of this implementation; no counterpart in the reference. */
long long sb200_softmax_ring_timeouts(void);

#ifdef __cplusplus
}
#endif
#endif /* SB200_H_ */
