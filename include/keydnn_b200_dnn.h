/*
 * keydnn_b200_dnn.h - C ABI of libkeydnn_b200_dnn.so: the library GEMM / convolution entries of
 * KeyDNN's CUDA DLL (cuBLAS, cuDNN), kept as library calls but with cached plans, a persistent
 * workspace and entries that take un-padded tensors.  Same conventions as keydnn_b200.h; status
 * 100000 + cudnnStatus_t on cuDNN errors (ref: NC/keydnn_cuda_conv2d.cu:16-19), matmul 0/1/2/3/4.
 * NC/ = src/keydnn/infrastructure/native_cuda/keydnn_v2_cuda_native/KeyDNNV2CudaNative/.
 */
#ifndef KEYDNN_B200_DNN_H
#define KEYDNN_B200_DNN_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* additive: the stream of the cuBLAS / cuDNN calls.  bind_stream_source takes the address of
 * libkeydnn_b200.so's keydnn_cuda_get_stream (int f(uint64_t* out)); from then on every call asks it, so both
 * libraries always share one stream (the reference has one: the default stream, NC/keydnn_cuda_conv2d.cu:53-61).
 * set_stream sets an explicit stream and drops a bound source (default: legacy default stream). */
int keydnn_dnn_set_stream(uint64_t stream);
int keydnn_dnn_bind_stream_source(uint64_t get_stream_fn);
int keydnn_dnn_get_stream(uint64_t* out);

/* ref: NC/keydnn_cuda_conv2d.hpp:17-99 (planes already padded by the caller) */
int keydnn_cuda_conv2d_forward_f32(const float* x_pad, const float* w, const float* b, float* y, int N, int C_in,
                                   int H_pad, int W_pad, int C_out, int H_out, int W_out, int K_h, int K_w, int s_h,
                                   int s_w);
int keydnn_cuda_conv2d_forward_f64(const double* x_pad, const double* w, const double* b, double* y, int N, int C_in,
                                   int H_pad, int W_pad, int C_out, int H_out, int W_out, int K_h, int K_w, int s_h,
                                   int s_w);
int keydnn_cuda_conv2d_backward_f32(const float* x_pad, const float* w, const float* grad_out, float* grad_x_pad,
                                    float* grad_w, int N, int C_in, int H_pad, int W_pad, int C_out, int H_out,
                                    int W_out, int K_h, int K_w, int s_h, int s_w);
int keydnn_cuda_conv2d_backward_f64(const double* x_pad, const double* w, const double* grad_out, double* grad_x_pad,
                                    double* grad_w, int N, int C_in, int H_pad, int W_pad, int C_out, int H_out,
                                    int W_out, int K_h, int K_w, int s_h, int s_w);
/* additive: un-padded x / grad_x, cuDNN pads; grad_x or grad_w may be NULL.  Replace the host round trips of
 * src/keydnn/infrastructure/ops/conv2d_cuda_ext.py:279-513. */
int keydnn_cuda_conv2d_forward_ex_f32(const float* x, const float* w, const float* b, float* y, int N, int C_in, int H,
                                      int W, int C_out, int H_out, int W_out, int K_h, int K_w, int s_h, int s_w,
                                      int p_h, int p_w);
int keydnn_cuda_conv2d_forward_ex_f64(const double* x, const double* w, const double* b, double* y, int N, int C_in,
                                      int H, int W, int C_out, int H_out, int W_out, int K_h, int K_w, int s_h, int s_w,
                                      int p_h, int p_w);
int keydnn_cuda_conv2d_backward_ex_f32(const float* x, const float* w, const float* grad_out, float* grad_x,
                                       float* grad_w, int N, int C_in, int H, int W, int C_out, int H_out, int W_out,
                                       int K_h, int K_w, int s_h, int s_w, int p_h, int p_w);
int keydnn_cuda_conv2d_backward_ex_f64(const double* x, const double* w, const double* grad_out, double* grad_x,
                                       double* grad_w, int N, int C_in, int H, int W, int C_out, int H_out, int W_out,
                                       int K_h, int K_w, int s_h, int s_w, int p_h, int p_w);
/* ref: NC/keydnn_cuda_ops.hpp:25-26; row-major C[M,N] = A[M,K] * B[K,N] */
int keydnn_cuda_matmul_f32(const float* A, const float* B, float* C, int M, int N, int K);
int keydnn_cuda_matmul_f64(const double* A, const double* B, double* C, int M, int N, int K);
/* additive: C[M,N] = op(A) * op(B); trans_a: A is stored (K,M); trans_b: B is stored (N,K) */
int keydnn_cuda_matmul_ex_f32(const float* A, const float* B, float* C, int M, int N, int K, int trans_a, int trans_b);
int keydnn_cuda_matmul_ex_f64(const double* A, const double* B, double* C, int M, int N, int K, int trans_a,
                              int trans_b);

#ifdef __cplusplus
}
#endif
#endif /* KEYDNN_B200_DNN_H */
