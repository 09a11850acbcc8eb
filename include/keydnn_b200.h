/*
 * keydnn_b200.h - C ABI of libkeydnn_b200.so, the sm_100a (B200) operator library
 * that stands in for KeyDNN's KeyDNNV2CudaNative DLL on the pool / reduce /
 * elementwise / optimizer path.
 *
 * Conventions (those of the reference library):
 *   - plain C symbols, default visibility, opened once per process with ctypes.CDLL;
 *   - device pointers cross as T* or as uint64_t integers;
 *   - every function returns int: 0 = ok, > 0 = cudaError_t (mul family: 1/2/3,
 *     memcpy_d2d: 1/2, broadcast_to: 1..4, transpose2d: 1/2/3), < 0 = argument guard;
 *   - tensors are dense, contiguous, row-major (NCHW for pooling);
 *   - all work is enqueued on one stream (the legacy default stream unless
 *     keydnn_cuda_set_stream is called); nothing synchronises unless stated.
 *
 * "ref:" names the reference declaration each entry replaces, as a path inside
 * the reference project.  NC/ = src/keydnn/infrastructure/native_cuda/
 * keydnn_v2_cuda_native/KeyDNNV2CudaNative/.  Entries marked "additive" have no
 * counterpart in the reference library.
 */
#ifndef KEYDNN_B200_H
#define KEYDNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------- */
/* Runtime: device, memory, copies, stream, events                            */
/* ref: NC/keydnn_cuda_utils.hpp:30-42, NC/keydnn_cuda_ops.hpp:18             */
/* ------------------------------------------------------------------------- */
int keydnn_cuda_set_device(int device);
/* malloc/free go through a per-device caching pool (no cudaFree sync per op). */
int keydnn_cuda_malloc(uint64_t* out_dev_ptr, size_t nbytes);
int keydnn_cuda_free(uint64_t dev_ptr);
/* h2d / d2h return when the copy is complete. */
int keydnn_cuda_memcpy_h2d(uint64_t dst_dev_ptr, const void* src_host_ptr, size_t nbytes);
int keydnn_cuda_memcpy_d2h(void* dst_host_ptr, uint64_t src_dev_ptr, size_t nbytes);
int keydnn_cuda_memcpy_d2d(void* dst, const void* src, size_t nbytes);
int keydnn_cuda_memset(uint64_t dev_ptr, int value, size_t nbytes);
int keydnn_cuda_synchronize(void);
/* additive */
int keydnn_cuda_memcpy_h2d_async(uint64_t dst_dev_ptr, const void* src_host_ptr, size_t nbytes);
int keydnn_cuda_memcpy_d2h_async(void* dst_host_ptr, uint64_t src_dev_ptr, size_t nbytes);
int keydnn_cuda_empty_cache(void);
int keydnn_cuda_pool_stats(uint64_t* out4); /* reserved, in use, driver mallocs, requests */
/* reduction scratch of the current device: partial bytes, ticket slots, driver allocations made for them,
 * outgrown buffers parked for a recorded graph */
int keydnn_cuda_scratch_stats(uint64_t* out4);
int keydnn_cuda_mem_info(uint64_t* out2);   /* cudaMemGetInfo: free, total */
int keydnn_cuda_host_alloc(void** out, size_t nbytes); /* pinned host memory */
int keydnn_cuda_host_free(void* p);
int keydnn_cuda_get_stream(uint64_t* out);
int keydnn_cuda_set_stream(uint64_t stream);
int keydnn_cuda_stream_create(uint64_t* out);
int keydnn_cuda_stream_destroy(uint64_t stream);
int keydnn_cuda_stream_synchronize(void);
/* additive; the names the reference's backward profiler looks up
 * (src/keydnn/infrastructure/tensor/_tensor.py:1619-1629) */
int keydnn_cuda_event_create(uint64_t* out);
int keydnn_cuda_event_record(uint64_t ev);
int keydnn_cuda_event_synchronize(uint64_t ev);
int keydnn_cuda_stream_wait_event(uint64_t ev); /* later work on the library stream waits for ev */
int keydnn_cuda_event_elapsed_ms(uint64_t start, uint64_t stop, float* out_ms);
int keydnn_cuda_event_destroy(uint64_t ev);
/* additive: record what is enqueued on the library stream (a created stream, not the default one) between
 * begin and end into a CUDA graph; replay with one launch.  Warm the work up eagerly on that stream first.
 * Blocks allocated during the recording stay reserved for the graph until graph_destroy.
 * -3: library stream is the default stream; -4: a recording or a graph already exists on this device. */
int keydnn_cuda_graph_capture_begin(void);
int keydnn_cuda_graph_capture_end(uint64_t* out_exec);
int keydnn_cuda_graph_launch(uint64_t exec);
int keydnn_cuda_graph_destroy(uint64_t exec);
int keydnn_cuda_device_count(int* out);
int keydnn_cuda_sm_count(int* out);
const char* keydnn_cuda_error_string(int code);
int keydnn_b200_abi_version(void);

/* ------------------------------------------------------------------------- */
/* Pooling, reference signatures (planes already padded by the caller)         */
/* ref: NC/keydnn_maxpool2d_cuda.hpp:28-72                                     */
/* ------------------------------------------------------------------------- */
int keydnn_cuda_maxpool2d_forward_f32(const float* x_pad, float* y, int64_t* argmax_idx, int N, int C, int H_pad,
                                      int W_pad, int H_out, int W_out, int k_h, int k_w, int s_h, int s_w);
int keydnn_cuda_maxpool2d_forward_f64(const double* x_pad, double* y, int64_t* argmax_idx, int N, int C, int H_pad,
                                      int W_pad, int H_out, int W_out, int k_h, int k_w, int s_h, int s_w);
/* grad_x_pad[argmax] += grad_out; the caller zero-fills grad_x_pad first. */
int keydnn_cuda_maxpool2d_backward_f32(const float* grad_out, const int64_t* argmax_idx, float* grad_x_pad, int N,
                                       int C, int H_out, int W_out, int H_pad, int W_pad);
int keydnn_cuda_maxpool2d_backward_f64(const double* grad_out, const int64_t* argmax_idx, double* grad_x_pad, int N,
                                       int C, int H_out, int W_out, int H_pad, int W_pad);
/* ref: NC/keydnn_avgpool2d_cuda.hpp:38-76 */
int keydnn_cuda_avgpool2d_forward_f32(const float* x_pad, float* y, int N, int C, int H_pad, int W_pad, int H_out,
                                      int W_out, int k_h, int k_w, int s_h, int s_w);
int keydnn_cuda_avgpool2d_forward_f64(const double* x_pad, double* y, int N, int C, int H_pad, int W_pad, int H_out,
                                      int W_out, int k_h, int k_w, int s_h, int s_w);
/* grad_x_pad += gathered gradient; the caller zero-fills grad_x_pad first. */
int keydnn_cuda_avgpool2d_backward_f32(const float* grad_out, float* grad_x_pad, int N, int C, int H_out, int W_out,
                                       int H_pad, int W_pad, int k_h, int k_w, int s_h, int s_w);
int keydnn_cuda_avgpool2d_backward_f64(const double* grad_out, double* grad_x_pad, int N, int C, int H_out, int W_out,
                                       int H_pad, int W_pad, int k_h, int k_w, int s_h, int s_w);
/* ref: NC/keydnn_global_avgpool2d_cuda.hpp:34-60 */
int keydnn_cuda_global_avgpool2d_forward_f32(const float* x, float* y, int N, int C, int H, int W);
int keydnn_cuda_global_avgpool2d_forward_f64(const double* x, double* y, int N, int C, int H, int W);
int keydnn_cuda_global_avgpool2d_backward_f32(const float* grad_out, float* grad_x, int N, int C, int H, int W);
int keydnn_cuda_global_avgpool2d_backward_f64(const double* grad_out, double* grad_x, int N, int C, int H, int W);
/* ref: NC/keydnn_pad2d_cuda.hpp (pad2d / crop2d declarations) */
int keydnn_cuda_pad2d_f32(const float* x, float* y_pad, int N, int C, int H, int W, int p_h, int p_w, float pad_value);
int keydnn_cuda_pad2d_f64(const double* x, double* y_pad, int N, int C, int H, int W, int p_h, int p_w,
                          double pad_value);
int keydnn_cuda_crop2d_f32(const float* x_pad, float* y, int N, int C, int H_pad, int W_pad, int p_h, int p_w, int H,
                           int W);
int keydnn_cuda_crop2d_f64(const double* x_pad, double* y, int N, int C, int H_pad, int W_pad, int p_h, int p_w, int H,
                           int W);

/* additive, host-only (no device work): how the row-band pooling kernels (any window / stride / padding / alignment)
 * would split one (H, W) plane.  kind 0 = forward (rows = output rows per band), 1 = AvgPool backward, 2 = MaxPool
 * backward (rows = input rows per band); out5 = usable (0 = the one-thread-per-element kernels run instead), rows per
 * band, bands per plane, dynamic shared memory in bytes, elements of one arrival buffer. */
int keydnn_cuda_debug_pool_band_plan(int kind, int elem_size, int H, int W, int H_out, int W_out, int k_h, int k_w, int s_h,
                                     int s_w, int p_h, int p_w, int64_t* out5);

/* ------------------------------------------------------------------------- */
/* Pooling, fused entries (additive): un-padded tensors, explicit padding.      */
/* Replace the pad->pool and memset->pool-backward->crop call sequences of      */
/* src/keydnn/infrastructure/ops/pool2d_cuda_ext.py:56-522.  argmax keeps the   */
/* reference encoding h*W_pad + w in the padded plane.  Backward overwrites     */
/* every element of grad_x.                                                     */
/* ------------------------------------------------------------------------- */
int keydnn_cuda_maxpool2d_forward_ex_f32(const float* x, float* y, int64_t* argmax_idx, int N, int C, int H, int W,
                                         int H_out, int W_out, int k_h, int k_w, int s_h, int s_w, int p_h, int p_w);
int keydnn_cuda_maxpool2d_forward_ex_f64(const double* x, double* y, int64_t* argmax_idx, int N, int C, int H, int W,
                                         int H_out, int W_out, int k_h, int k_w, int s_h, int s_w, int p_h, int p_w);
int keydnn_cuda_maxpool2d_backward_ex_f32(const float* grad_out, const int64_t* argmax_idx, float* grad_x, int N,
                                          int C, int H, int W, int H_out, int W_out, int k_h, int k_w, int s_h,
                                          int s_w, int p_h, int p_w);
int keydnn_cuda_maxpool2d_backward_ex_f64(const double* grad_out, const int64_t* argmax_idx, double* grad_x, int N,
                                          int C, int H, int W, int H_out, int W_out, int k_h, int k_w, int s_h,
                                          int s_w, int p_h, int p_w);
int keydnn_cuda_avgpool2d_forward_ex_f32(const float* x, float* y, int N, int C, int H, int W, int H_out, int W_out,
                                         int k_h, int k_w, int s_h, int s_w, int p_h, int p_w);
int keydnn_cuda_avgpool2d_forward_ex_f64(const double* x, double* y, int N, int C, int H, int W, int H_out, int W_out,
                                         int k_h, int k_w, int s_h, int s_w, int p_h, int p_w);
int keydnn_cuda_avgpool2d_backward_ex_f32(const float* grad_out, float* grad_x, int N, int C, int H, int W, int H_out,
                                          int W_out, int k_h, int k_w, int s_h, int s_w, int p_h, int p_w);
int keydnn_cuda_avgpool2d_backward_ex_f64(const double* grad_out, double* grad_x, int N, int C, int H, int W,
                                          int H_out, int W_out, int k_h, int k_w, int s_h, int s_w, int p_h, int p_w);

/* ------------------------------------------------------------------------- */
/* Reductions.  ref: NC/keydnn_reduce_cuda.hpp:56-140                          */
/* ------------------------------------------------------------------------- */
int keydnn_cuda_sum_all_f32(const float* x, float* y, int64_t numel);
int keydnn_cuda_sum_all_f64(const double* x, double* y, int64_t numel);
int keydnn_cuda_mean_all_f32(const float* x, float* y, int64_t numel);
int keydnn_cuda_mean_all_f64(const double* x, double* y, int64_t numel);
int keydnn_cuda_sum_backward_fill_f32(const float* grad_out, float* grad_x, int64_t numel);
int keydnn_cuda_sum_backward_fill_f64(const double* grad_out, double* grad_x, int64_t numel);
int keydnn_cuda_mean_backward_fill_f32(const float* grad_out, float* grad_x, int64_t numel);
int keydnn_cuda_mean_backward_fill_f64(const double* grad_out, double* grad_x, int64_t numel);
int keydnn_cuda_max_axis2d_forward_f32(const float* x, float* y, int64_t* idx, int rows, int cols, int axis);
int keydnn_cuda_max_axis2d_forward_f64(const double* x, double* y, int64_t* idx, int rows, int cols, int axis);
/* grad_x[argmax] += grad_out; the caller zero-fills grad_x first. */
int keydnn_cuda_max_axis2d_backward_f32(const float* grad_out, const int64_t* idx, float* grad_x, int rows, int cols,
                                        int axis);
int keydnn_cuda_max_axis2d_backward_f64(const double* grad_out, const int64_t* idx, double* grad_x, int rows,
                                        int cols, int axis);
int keydnn_cuda_sum_axis2d_forward_f32(const float* x, float* y, int rows, int cols, int axis);
int keydnn_cuda_sum_axis2d_forward_f64(const double* x, double* y, int rows, int cols, int axis);
int keydnn_cuda_sum_axis2d_backward_f32(const float* grad_out, float* grad_x, int rows, int cols, int axis);
int keydnn_cuda_sum_axis2d_backward_f64(const double* grad_out, double* grad_x, int rows, int cols, int axis);
/* in_shape / out_shape are HOST arrays of ndim extents (out extent is 1 or the in extent). */
int keydnn_cuda_sum_to_shape_f32(const float* x, float* y, const int64_t* in_shape, const int64_t* out_shape,
                                 int ndim);
int keydnn_cuda_sum_to_shape_f64(const double* x, double* y, const int64_t* in_shape, const int64_t* out_shape,
                                 int ndim);
/* No counterpart in the reference.  Column sums (axis 0) of a float32 (rows, cols) matrix for
 * callers that may not allocate device memory at call time (hosts whose own allocator owns the
 * device heap, latency-critical loops, fixed-budget processes): no cudaMalloc / cudaFree; partials
 * live in a static 2,113,536-byte device array that each GPU holds while the library is loaded.
 * cols <= KEYDNN_NOALLOC_MAX_COLS, else -20.  First call per device resolves the array's address
 * (do it outside stream capture).  Calls that overlap on the GPU race on the shared array. */
#define KEYDNN_NOALLOC_MAX_COLS 65536
int keydnn_cuda_sum_axis0_noalloc_f32(const float* x, float* y, int rows, int cols);
/* additive, host-only (no device work): launch shape of the axis-0 reductions for a (rows, cols) matrix of
 * elem_size-byte elements: out3 = rows per chunk, chunks, column stripes; -2 where the entry points return -2
 * (row indices are 32-bit in the kernels: chunks * rows-per-chunk must stay below 2^31). */
int keydnn_cuda_debug_col_chunks(int rows, int cols, int elem_size, int ctas_per_sm, int64_t* out3);
/* additive: the reference has no axis-wise mean (tensor/mixins/reduction/_tensor_mean.py:91-192
 * is all-elements only), no all-elements max (_tensor_max.py:70-85 is 2-D, axis 0/1), and its max
 * backward needs a zero-fill pass before it (ops/reduce_cuda.py:409-414). */
int keydnn_cuda_max_axis2d_backward_ex_f32(const float* grad_out, const int64_t* idx, float* grad_x, int rows,
                                           int cols, int axis);
int keydnn_cuda_max_axis2d_backward_ex_f64(const double* grad_out, const int64_t* idx, double* grad_x, int rows,
                                           int cols, int axis);
int keydnn_cuda_mean_axis2d_forward_f32(const float* x, float* y, int rows, int cols, int axis);
int keydnn_cuda_mean_axis2d_forward_f64(const double* x, double* y, int rows, int cols, int axis);
int keydnn_cuda_mean_axis2d_backward_f32(const float* grad_out, float* grad_x, int rows, int cols, int axis);
int keydnn_cuda_mean_axis2d_backward_f64(const double* grad_out, double* grad_x, int rows, int cols, int axis);
int keydnn_cuda_max_all_forward_f32(const float* x, float* y, int64_t* idx, int64_t numel);
int keydnn_cuda_max_all_forward_f64(const double* x, double* y, int64_t* idx, int64_t numel);
int keydnn_cuda_max_all_backward_f32(const float* grad_out, const int64_t* idx, float* grad_x, int64_t numel);
int keydnn_cuda_max_all_backward_f64(const double* grad_out, const int64_t* idx, double* grad_x, int64_t numel);

/* ------------------------------------------------------------------------- */
/* Elementwise.  ref: NC/keydnn_tensor_arithmetic.hpp:19-108,164-183           */
/* Compares write float32 1.0/0.0 masks for both input types.                  */
/* ------------------------------------------------------------------------- */
int keydnn_cuda_neg_f32(const float* x, float* y, int64_t n);
int keydnn_cuda_neg_f64(const double* x, double* y, int64_t n);
int keydnn_cuda_add_f32(const float* a, const float* b, float* y, int64_t n);
int keydnn_cuda_add_f64(const double* a, const double* b, double* y, int64_t n);
int keydnn_cuda_sub_f32(const float* a, const float* b, float* y, int64_t n);
int keydnn_cuda_sub_f64(const double* a, const double* b, double* y, int64_t n);
int keydnn_cuda_div_f32(const float* a, const float* b, float* y, int64_t n);
int keydnn_cuda_div_f64(const double* a, const double* b, double* y, int64_t n);
int keydnn_cuda_gt_f32(const float* a, const float* b, float* y, int64_t n);
int keydnn_cuda_gt_f64(const double* a, const double* b, float* y, int64_t n);
int keydnn_cuda_ge_f32(const float* a, const float* b, float* y, int64_t n);
int keydnn_cuda_ge_f64(const double* a, const double* b, float* y, int64_t n);
int keydnn_cuda_lt_f32(const float* a, const float* b, float* y, int64_t n);
int keydnn_cuda_lt_f64(const double* a, const double* b, float* y, int64_t n);
int keydnn_cuda_le_f32(const float* a, const float* b, float* y, int64_t n);
int keydnn_cuda_le_f64(const double* a, const double* b, float* y, int64_t n);
int keydnn_cuda_eq_f32(const float* a, const float* b, float* y, int64_t n);
int keydnn_cuda_eq_f64(const double* a, const double* b, float* y, int64_t n);
int keydnn_cuda_ne_f32(const float* a, const float* b, float* y, int64_t n);
int keydnn_cuda_ne_f64(const double* a, const double* b, float* y, int64_t n);
int keydnn_cuda_add_scalar_f32(const float* a, float alpha, float* y, int64_t n);
int keydnn_cuda_add_scalar_f64(const double* a, double alpha, double* y, int64_t n);
int keydnn_cuda_sub_scalar_f32(const float* a, float alpha, float* y, int64_t n);
int keydnn_cuda_sub_scalar_f64(const double* a, double alpha, double* y, int64_t n);
int keydnn_cuda_div_scalar_f32(const float* a, float alpha, float* y, int64_t n);
int keydnn_cuda_div_scalar_f64(const double* a, double alpha, double* y, int64_t n);
int keydnn_cuda_gt_scalar_f32(const float* a, float alpha, float* y, int64_t n);
int keydnn_cuda_gt_scalar_f64(const double* a, double alpha, float* y, int64_t n);
int keydnn_cuda_ge_scalar_f32(const float* a, float alpha, float* y, int64_t n);
int keydnn_cuda_ge_scalar_f64(const double* a, double alpha, float* y, int64_t n);
int keydnn_cuda_lt_scalar_f32(const float* a, float alpha, float* y, int64_t n);
int keydnn_cuda_lt_scalar_f64(const double* a, double alpha, float* y, int64_t n);
int keydnn_cuda_le_scalar_f32(const float* a, float alpha, float* y, int64_t n);
int keydnn_cuda_le_scalar_f64(const double* a, double alpha, float* y, int64_t n);
int keydnn_cuda_eq_scalar_f32(const float* a, float alpha, float* y, int64_t n);
int keydnn_cuda_eq_scalar_f64(const double* a, double alpha, float* y, int64_t n);
int keydnn_cuda_ne_scalar_f32(const float* a, float alpha, float* y, int64_t n);
int keydnn_cuda_ne_scalar_f64(const double* a, double alpha, float* y, int64_t n);
int keydnn_cuda_add_inplace_f32(float* a, const float* b, int64_t n);
int keydnn_cuda_add_inplace_f64(double* a, const double* b, int64_t n);
int keydnn_cuda_sub_inplace_f32(float* a, const float* b, int64_t n);
int keydnn_cuda_sub_inplace_f64(double* a, const double* b, int64_t n);
int keydnn_cuda_div_inplace_f32(float* a, const float* b, int64_t n);
int keydnn_cuda_div_inplace_f64(double* a, const double* b, int64_t n);
int keydnn_cuda_add_scalar_inplace_f32(float* a, float alpha, int64_t n);
int keydnn_cuda_add_scalar_inplace_f64(double* a, double alpha, int64_t n);
int keydnn_cuda_sub_scalar_inplace_f32(float* a, float alpha, int64_t n);
int keydnn_cuda_sub_scalar_inplace_f64(double* a, double alpha, int64_t n);
int keydnn_cuda_div_scalar_inplace_f32(float* a, float alpha, int64_t n);
int keydnn_cuda_div_scalar_inplace_f64(double* a, double alpha, int64_t n);
/* mul family: `int numel`, status 0/1/2/3.  ref: NC/keydnn_cuda_ops.hpp:33-46 */
int keydnn_cuda_mul_f32(const float* a, const float* b, float* y, int numel);
int keydnn_cuda_mul_f64(const double* a, const double* b, double* y, int numel);
int keydnn_cuda_mul_scalar_f32(const float* a, float alpha, float* y, int numel);
int keydnn_cuda_mul_scalar_f64(const double* a, double alpha, double* y, int numel);
int keydnn_cuda_mul_inplace_f32(float* a, const float* b, int numel);
int keydnn_cuda_mul_inplace_f64(double* a, const double* b, int numel);
int keydnn_cuda_mul_scalar_inplace_f32(float* a, float alpha, int numel);
int keydnn_cuda_mul_scalar_inplace_f64(double* a, double alpha, int numel);
/* additive: 64-bit element counts for mul */
int keydnn_cuda_mul64_f32(const float* a, const float* b, float* y, int64_t n);
int keydnn_cuda_mul64_f64(const double* a, const double* b, double* y, int64_t n);
/* additive: both gradients of y = a*b (ga = g*b, gb = g*a) or y = a/b (ga = g/b, gb = (-(g*a))/(b*b)) in
 * one pass, each operation rounded as in the reference closures
 * (src/keydnn/infrastructure/tensor/mixins/arithmetic/_tensor_multiplication.py:98-103,
 * _tensor_division.py:104-114); ga or gb may be NULL. */
int keydnn_cuda_mul_backward_f32(const float* g, const float* a, const float* b, float* ga, float* gb, int64_t n);
int keydnn_cuda_mul_backward_f64(const double* g, const double* a, const double* b, double* ga, double* gb, int64_t n);
int keydnn_cuda_div_backward_f32(const float* g, const float* a, const float* b, float* ga, float* gb, int64_t n);
int keydnn_cuda_div_backward_f64(const double* g, const double* a, const double* b, double* ga, double* gb, int64_t n);
/* ref: NC/keydnn_fill_cuda.hpp:36-46 */
int keydnn_cuda_fill_f32(float* y, int64_t numel, float value);
int keydnn_cuda_fill_f64(double* y, int64_t numel, double value);
/* additive: fused optimizer step.  Replaces the five tensor passes of
 * src/keydnn/infrastructure/optimizers/_sgd.py:119-140 with one; v may be NULL
 * (no momentum).  Separately rounded ops in the reference order:
 * g' = g*grad_scale (skipped when 1); g' += p*wd (skipped when 0);
 * v = v*mu + g'; p -= (v or g')*lr. */
int keydnn_cuda_sgd_momentum_step_f32(float* p, const float* g, float* v, int64_t n, float lr, float momentum,
                                      float weight_decay, float grad_scale);
int keydnn_cuda_sgd_momentum_step_f64(double* p, const double* g, double* v, int64_t n, double lr, double momentum,
                                      double weight_decay, double grad_scale);

/* ------------------------------------------------------------------------- */
/* Layer glue.  ref: NC/keydnn_cuda_ops.hpp:20-21,57-67;                       */
/*              NC/keydnn_tensor_arithmetic.hpp:130-159                        */
/* ------------------------------------------------------------------------- */
int keydnn_cuda_broadcast_to_f32(const float* x, float* y, const int64_t* in_shape, int in_ndim,
                                 const int64_t* out_shape, int out_ndim);
int keydnn_cuda_broadcast_to_f64(const double* x, double* y, const int64_t* in_shape, int in_ndim,
                                 const int64_t* out_shape, int out_ndim);
int keydnn_cuda_bias_add_f32(const float* x, const float* b, float* y, int64_t batch, int64_t out);
int keydnn_cuda_bias_add_f64(const double* x, const double* b, double* y, int64_t batch, int64_t out);
int keydnn_cuda_bias_add_inplace_f32(float* y, const float* b, int64_t batch, int64_t out);
int keydnn_cuda_bias_add_inplace_f64(double* y, const double* b, int64_t batch, int64_t out);
int keydnn_cuda_transpose2d_f32(const float* x, float* y, int rows, int cols);
int keydnn_cuda_transpose2d_f64(const double* x, double* y, int rows, int cols);

/* ------------------------------------------------------------------------- */
/* BatchNorm2d (additive).  The reference composes the layer from ~25 tensor-op launches and
 * rejects CUDA tensors (src/keydnn/infrastructure/layers/_batchnorm.py:543-544, body :562-700);
 * these entries run the same formulas in two kernels per direction.  x, y, grad_* are
 * (N, C, HW) contiguous; gamma/beta (both or neither) may be NULL; mean / invstd receive the
 * statistics used (saved for backward); training != 0 uses batch statistics and updates
 * running_mean / running_var (may be NULL) with `momentum`.  relu != 0 fuses the mask-and-multiply
 * ReLU that follows the layer (src/keydnn/infrastructure/_function.py:291-293) into both directions. */
/* ------------------------------------------------------------------------- */
int keydnn_cuda_bn2d_forward_f32(const float* x, const float* gamma, const float* beta, float* y, float* mean,
                                 float* invstd, float* running_mean, float* running_var, int N, int C, int64_t HW,
                                 float eps, float momentum, int training, int relu);
int keydnn_cuda_bn2d_forward_f64(const double* x, const double* gamma, const double* beta, double* y, double* mean,
                                 double* invstd, double* running_mean, double* running_var, int N, int C, int64_t HW,
                                 double eps, double momentum, int training, int relu);
int keydnn_cuda_bn2d_backward_f32(const float* x, const float* gamma, const float* beta, const float* grad_out,
                                  const float* mean, const float* invstd, float* grad_x, float* grad_gamma,
                                  float* grad_beta, int N, int C, int64_t HW, int relu);
int keydnn_cuda_bn2d_backward_f64(const double* x, const double* gamma, const double* beta, const double* grad_out,
                                  const double* mean, const double* invstd, double* grad_x, double* grad_gamma,
                                  double* grad_beta, int N, int C, int64_t HW, int relu);

/* The layer in front adds a per-channel bias (a convolution's): pre_bias (C values) is added to every element of x as
 * it is read, one rounded addition, so the separate bias pass over the activation disappears; statistics, output and
 * gradients are those of x + pre_bias. */
int keydnn_cuda_bn2d_forward_bias_f32(const float* x, const float* pre_bias, const float* gamma, const float* beta,
                                      float* y, float* mean, float* invstd, float* running_mean, float* running_var,
                                      int N, int C, int64_t HW, float eps, float momentum, int training, int relu);
int keydnn_cuda_bn2d_forward_bias_f64(const double* x, const double* pre_bias, const double* gamma, const double* beta,
                                      double* y, double* mean, double* invstd, double* running_mean,
                                      double* running_var, int N, int C, int64_t HW, double eps, double momentum,
                                      int training, int relu);
int keydnn_cuda_bn2d_backward_bias_f32(const float* x, const float* pre_bias, const float* gamma, const float* beta,
                                       const float* grad_out, const float* mean, const float* invstd, float* grad_x,
                                       float* grad_gamma, float* grad_beta, int N, int C, int64_t HW, int relu);
int keydnn_cuda_bn2d_backward_bias_f64(const double* x, const double* pre_bias, const double* gamma, const double* beta,
                                       const double* grad_out, const double* mean, const double* invstd,
                                       double* grad_x, double* grad_gamma, double* grad_beta, int N, int C, int64_t HW,
                                       int relu);

/* BatchNorm2d (+ ReLU) followed by MaxPool2d(2): forward writes only the pooled tensor and its int64 positions
 * (h * W + w, as keydnn_cuda_maxpool2d_forward_ex_* records them); backward takes the gradient of the pooled tensor
 * and derives each element's gradient on the fly.  Same bits as the separate entries; the (N, C, H, W) activation
 * and its gradient are never stored.  H even, W a multiple of 8, else -6 (use the separate entries). */
int keydnn_cuda_bn2d_maxpool2x2_forward_f32(const float* x, const float* pre_bias, const float* gamma, const float* beta,
                                            float* y_pool, int64_t* argmax_idx, float* mean, float* invstd,
                                            float* running_mean, float* running_var, int N, int C, int H, int W,
                                            float eps, float momentum, int training, int relu);
int keydnn_cuda_bn2d_maxpool2x2_forward_f64(const double* x, const double* pre_bias, const double* gamma,
                                            const double* beta, double* y_pool, int64_t* argmax_idx, double* mean,
                                            double* invstd, double* running_mean, double* running_var, int N, int C,
                                            int H, int W, double eps, double momentum, int training, int relu);
int keydnn_cuda_bn2d_maxpool2x2_backward_f32(const float* x, const float* pre_bias, const float* gamma, const float* beta,
                                             const float* grad_pool, const int64_t* argmax_idx, const float* mean,
                                             const float* invstd, float* grad_x, float* grad_gamma, float* grad_beta,
                                             int N, int C, int H, int W, int relu);
int keydnn_cuda_bn2d_maxpool2x2_backward_f64(const double* x, const double* pre_bias, const double* gamma,
                                             const double* beta, const double* grad_pool, const int64_t* argmax_idx,
                                             const double* mean, const double* invstd, double* grad_x,
                                             double* grad_gamma, double* grad_beta, int N, int C, int H, int W, int relu);

/* BatchNorm2d (+ ReLU) followed by GlobalAvgPool2d: forward writes only the (N, C) plane means, backward takes their
 * gradient (every element of plane (n, c) receives grad_mean[n, c] * (1 / HW)).  Same bits as the separate entries.
 * HW a multiple of 4 and above 64, else -6. */
int keydnn_cuda_bn2d_global_avgpool_forward_f32(const float* x, const float* pre_bias, const float* gamma,
                                                const float* beta, float* y_mean, float* mean, float* invstd,
                                                float* running_mean, float* running_var, int N, int C, int64_t HW,
                                                float eps, float momentum, int training, int relu);
int keydnn_cuda_bn2d_global_avgpool_forward_f64(const double* x, const double* pre_bias, const double* gamma,
                                                const double* beta, double* y_mean, double* mean, double* invstd,
                                                double* running_mean, double* running_var, int N, int C, int64_t HW,
                                                double eps, double momentum, int training, int relu);
int keydnn_cuda_bn2d_global_avgpool_backward_f32(const float* x, const float* pre_bias, const float* gamma,
                                                 const float* beta, const float* grad_mean, const float* mean,
                                                 const float* invstd, float* grad_x, float* grad_gamma,
                                                 float* grad_beta, int N, int C, int64_t HW, int relu);
int keydnn_cuda_bn2d_global_avgpool_backward_f64(const double* x, const double* pre_bias, const double* gamma,
                                                 const double* beta, const double* grad_mean, const double* mean,
                                                 const double* invstd, double* grad_x, double* grad_gamma,
                                                 double* grad_beta, int N, int C, int64_t HW, int relu);

/* ------------------------------------------------------------------------- */
/* exp / log / sqrt, activations, losses, Adam.                                 */
/* ref: NC/keydnn_cuda_ops.hpp (keydnn_cuda_exp_*; kernel keydnn_cuda_exp.cu:5-40) is the only unary
 * export of the reference.  Everything else here is additive: the reference builds these from chains of
 * one-op tensor kernels (src/keydnn/infrastructure/_function.py:54-612, _losses.py:44-408,
 * optimizers/_adam.py:170-220) or on the host (tensor/mixins/unary/_tensor_log.py:77,
 * _tensor_sqrt.py:81-91); each entry is one pass with the same separately rounded operations.        */
/* ------------------------------------------------------------------------- */
/* status as in the reference: 1 numel < 0, 2 null pointer, 3 launch failure */
int keydnn_cuda_exp_f32(const float* x, float* y, int numel);
int keydnn_cuda_exp_f64(const double* x, double* y, int numel);
/* additive */
int keydnn_cuda_log_f32(const float* x, float* y, int64_t n);
int keydnn_cuda_sqrt_f32(const float* x, float* y, int64_t n);
int keydnn_cuda_sqrt_backward_f32(const float* grad_out, const float* y, float* grad_x, int64_t n);          /* g * (0.5 / y) */
int keydnn_cuda_sigmoid_forward_f32(const float* x, float* y, int64_t n);                                  /* 1 / (exp(-x) + 1) */
int keydnn_cuda_sigmoid_backward_f32(const float* grad_out, const float* y, float* grad_x, int64_t n);        /* (g*y) * ((-y) + 1) */
int keydnn_cuda_tanh_forward_f32(const float* x, float* y, int64_t n);                                     /* (e^x - e^-x) / (e^x + e^-x) */
int keydnn_cuda_tanh_backward_f32(const float* grad_out, const float* y, float* grad_x, int64_t n);           /* g - (y*y)*g */
int keydnn_cuda_relu_forward_f32(const float* x, float* y, float* mask_or_null, int64_t n);                   /* mask = x > 0; y = x*mask */
int keydnn_cuda_relu_backward_f32(const float* grad_out, const float* x, float* grad_x, int64_t n);           /* g * (x > 0) */
int keydnn_cuda_leaky_relu_forward_f32(const float* x, float* y, float alpha, int64_t n);
int keydnn_cuda_leaky_relu_backward_f32(const float* grad_out, const float* x, float* grad_x, float alpha, int64_t n);
int keydnn_cuda_log_f64(const double* x, double* y, int64_t n);
int keydnn_cuda_sqrt_f64(const double* x, double* y, int64_t n);
int keydnn_cuda_sqrt_backward_f64(const double* grad_out, const double* y, double* grad_x, int64_t n);          /* g * (0.5 / y) */
int keydnn_cuda_sigmoid_forward_f64(const double* x, double* y, int64_t n);                                  /* 1 / (exp(-x) + 1) */
int keydnn_cuda_sigmoid_backward_f64(const double* grad_out, const double* y, double* grad_x, int64_t n);        /* (g*y) * ((-y) + 1) */
int keydnn_cuda_tanh_forward_f64(const double* x, double* y, int64_t n);                                     /* (e^x - e^-x) / (e^x + e^-x) */
int keydnn_cuda_tanh_backward_f64(const double* grad_out, const double* y, double* grad_x, int64_t n);           /* g - (y*y)*g */
int keydnn_cuda_relu_forward_f64(const double* x, double* y, double* mask_or_null, int64_t n);                   /* mask = x > 0; y = x*mask */
int keydnn_cuda_relu_backward_f64(const double* grad_out, const double* x, double* grad_x, int64_t n);           /* g * (x > 0) */
int keydnn_cuda_leaky_relu_forward_f64(const double* x, double* y, double alpha, int64_t n);
int keydnn_cuda_leaky_relu_backward_f64(const double* grad_out, const double* x, double* grad_x, double alpha, int64_t n);
/* softmax along the middle axis of a dense (outer, len, inner) view; inner = 1 for the last axis */
int keydnn_cuda_softmax_forward_f32(const float* x, float* y, int64_t outer, int64_t len, int64_t inner);
int keydnn_cuda_softmax_backward_f32(const float* grad_out, const float* y, float* grad_x, int64_t outer, int64_t len,
                                     int64_t inner);
int keydnn_cuda_softmax_forward_f64(const double* x, double* y, int64_t outer, int64_t len, int64_t inner);
int keydnn_cuda_softmax_backward_f64(const double* grad_out, const double* y, double* grad_x, int64_t outer, int64_t len,
                                     int64_t inner);
/* Adam with coupled L2 decay, in place on p, m, v.  one_minus_beta* = 1 - beta*, bias* = 1 - beta*^t, all
 * computed by the caller in double and narrowed here, as the reference's Python scalars are at its call
 * boundary; grad_scale multiplies g first (1 skips it). */
int keydnn_cuda_adam_step_f32(float* p, const float* g, float* m, float* v, int64_t n, float lr, float beta1, float beta2, float eps,
                              float weight_decay, float one_minus_beta1, float one_minus_beta2, float bias1, float bias2,
                              float grad_scale);
int keydnn_cuda_adam_step_f64(double* p, const double* g, double* m, double* v, int64_t n, double lr, double beta1, double beta2, double eps,
                              double weight_decay, double one_minus_beta1, double one_minus_beta2, double bias1, double bias2,
                              double grad_scale);
/* Adam whose step count lives on the device (step_counter: one int64, zero before the first step): entry i of
 * bias_table holds {1 - beta1^(i+1), 1 - beta2^(i+1)} as the caller computed them, table_len entries, the last one
 * used for every later step (build the table until both values are exactly 1).  bias_now: 2 elements of scratch.
 * No argument changes between steps, so a step recorded in a CUDA graph can be replayed. */
int keydnn_cuda_adam_step_counted_f32(float* p, const float* g, float* m, float* v, int64_t n, float lr, float beta1,
                                      float beta2, float eps, float weight_decay, float one_minus_beta1,
                                      float one_minus_beta2, const float* bias_table, int64_t table_len,
                                      int64_t* step_counter, float* bias_now, float grad_scale);
int keydnn_cuda_adam_step_counted_f64(double* p, const double* g, double* m, double* v, int64_t n, double lr,
                                      double beta1, double beta2, double eps, double weight_decay,
                                      double one_minus_beta1, double one_minus_beta2, const double* bias_table,
                                      int64_t table_len, int64_t* step_counter, double* bias_now, double grad_scale);
/* Losses.  loss is one device scalar.  sqdiff: diff = pred - target (written when diff is not null), loss =
 * sum(diff*diff), times 1/n when mean.  In the backward entries g is the upstream gradient as a DEVICE
 * scalar (null = 1); it is combined with the host factor in double on the device, where the reference reads
 * it to the host first: sqdiff grad_pred = diff * (scale*g), grad_target (nullable) = grad_pred * -1;
 * bce grad_pred = ((p - t) / (p*(1 - p))) * (g/n); cce grad_pred = (t/p) * -(g/batch). */
int keydnn_cuda_sqdiff_forward_f32(const float* pred, const float* target, float* diff, float* loss, int64_t n, int mean);
int keydnn_cuda_sqdiff_backward_f32(const float* diff, const float* g, double scale, float* grad_pred, float* grad_target,
                                    int64_t n);
int keydnn_cuda_bce_forward_f32(const float* pred, const float* target, float* loss, int64_t n);
int keydnn_cuda_bce_backward_f32(const float* pred, const float* target, const float* g, float* grad_pred, int64_t n);
int keydnn_cuda_cce_forward_f32(const float* pred, const float* target, float* loss, int64_t n, int64_t batch);
int keydnn_cuda_cce_backward_f32(const float* pred, const float* target, const float* g, float* grad_pred, int64_t n,
                                 int64_t batch);
int keydnn_cuda_sqdiff_forward_f64(const double* pred, const double* target, double* diff, double* loss, int64_t n, int mean);
int keydnn_cuda_sqdiff_backward_f64(const double* diff, const double* g, double scale, double* grad_pred, double* grad_target,
                                    int64_t n);
int keydnn_cuda_bce_forward_f64(const double* pred, const double* target, double* loss, int64_t n);
int keydnn_cuda_bce_backward_f64(const double* pred, const double* target, const double* g, double* grad_pred, int64_t n);
int keydnn_cuda_cce_forward_f64(const double* pred, const double* target, double* loss, int64_t n, int64_t batch);
int keydnn_cuda_cce_backward_f64(const double* pred, const double* target, const double* g, double* grad_pred, int64_t n,
                                 int64_t batch);

/* ------------------------------------------------------------------------- */
/* Multi-GPU (additive; the reference has no distributed code).  One process   */
/* per GPU; NCCL is opened with dlopen at first use; collectives run on the    */
/* library stream.  Status: -10 not initialised, -11 NCCL not loadable,        */
/* 200000 + ncclResult_t on NCCL errors.                                       */
/* ------------------------------------------------------------------------- */
int keydnn_nccl_unique_id(void* out128);                       /* 128-byte id, made on rank 0 */
int keydnn_nccl_init(const void* id128, int world, int rank);
int keydnn_nccl_destroy(void);
int keydnn_nccl_world(int* world, int* rank);
int keydnn_nccl_allreduce_sum_f32(float* buf, int64_t count);  /* in place */
int keydnn_nccl_allreduce_sum_f64(double* buf, int64_t count);
int keydnn_nccl_allgather(const void* send, void* recv, int64_t nbytes);
int keydnn_nccl_broadcast(void* buf, int64_t nbytes, int root);
/* out[i] = sum over the `world` gathered blocks, in rank order (double accumulation, one rounding), of element i,
 * times seg_scale[k] where seg_begin[k] <= i < seg_end[k] (HOST arrays, nseg <= 8; the 1/count of a mean).
 * stride = elements between two ranks' blocks.  Behind keydnn_nccl_allgather this is an all-reduce whose result
 * does not depend on the collective's internal order. */
int keydnn_cuda_rank_sum_f32(const float* blocks, int world, int64_t stride, int64_t n, float* out,
                             const int64_t* seg_begin, const int64_t* seg_end, const float* seg_scale, int nseg);
int keydnn_cuda_rank_sum_f64(const double* blocks, int world, int64_t stride, int64_t n, double* out,
                             const int64_t* seg_begin, const int64_t* seg_end, const double* seg_scale, int nseg);
/* Winner per column among `world` per-rank (value, local position) maxima; rank r's n values start at
 * vals + r*val_stride and its n positions at idx + r*idx_stride (strides in elements, so both can live
 * in one gathered block per rank): greater value, else lower rank; global position = rank*span + local;
 * out_local is the position inside this rank's shard or -1 when another rank owns the maximum. */
int keydnn_cuda_argmax_select_f32(const float* vals, const int64_t* idx, int world, int rank, int64_t span, int64_t n,
                                  int64_t val_stride, int64_t idx_stride, float* out_val, int64_t* out_global,
                                  int64_t* out_local);
int keydnn_cuda_argmax_select_f64(const double* vals, const int64_t* idx, int world, int rank, int64_t span, int64_t n,
                                  int64_t val_stride, int64_t idx_stride, double* out_val, int64_t* out_global,
                                  int64_t* out_local);

#ifdef __cplusplus
}
#endif
#endif /* KEYDNN_B200_H */
