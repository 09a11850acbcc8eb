// Library GEMM and convolution for the layers around the pool / reduce / elementwise path:
// cuBLAS (Linear) and cuDNN (Conv2d).  These stay library calls, as in the reference
// (KeyDNNV2CudaNative/keydnn_matmul.cu:46-93, keydnn_cuda_conv2d.cu:100-340); what changes is the
// plumbing around them:
//   * the `_ex` convolution entries take the un-padded tensors and let cuDNN pad, so the reference
//     wrapper's device->host copy, np.pad on the CPU and host->device copy
//     (src/keydnn/infrastructure/ops/conv2d_cuda_ext.py:353-373, ops/conv2d_cuda.py:345-374) disappear;
//   * descriptors, algorithm choice and workspace size are cached per problem shape instead of
//     being rebuilt on every call (keydnn_cuda_conv2d.cu:116-168), and the workspace is one
//     grow-only buffer instead of a cudaMalloc/cudaFree pair per call (:168,187,290,305,336-337);
//   * `matmul_ex` takes transpose flags, so Linear's W.T needs no transpose kernel.
// Built into its own shared library so that the main operator library keeps no cuBLAS / cuDNN
// dependency.
#include <cublas_v2.h>
#include <cuda_runtime.h>
#include <cudnn.h>

#include <cstdint>
#include <map>
#include <tuple>
#include <type_traits>

#define KD_API extern "C" __attribute__((visibility("default")))

namespace {

// One source of truth for the stream.  The operator library (libkeydnn_b200.so) owns "the library stream";
// its keydnn_cuda_get_stream is bound here once (keydnn_dnn_bind_stream_source) and asked before every
// cuDNN / cuBLAS call, so a convolution is always enqueued on the stream the BatchNorm / pooling / loss /
// optimizer kernels around it use and program order is stream order, as on the reference's single default
// stream (KeyDNNV2CudaNative/keydnn_cuda_conv2d.cu:53-61).  Without a bound source the stream is whatever
// keydnn_dnn_set_stream last set (default: the legacy default stream).
using StreamSource = int (*)(std::uint64_t*);
StreamSource g_stream_source = nullptr;
cudaStream_t g_stream = nullptr;
cudaStream_t g_last_stream = nullptr;      // stream of the previous call (compared, never dereferenced)
bool g_have_last = false;
cublasHandle_t g_blas = nullptr;
cudnnHandle_t g_dnn = nullptr;
void* g_ws = nullptr;
size_t g_ws_bytes = 0;

inline int cudnn_status(cudnnStatus_t s) { return s == CUDNN_STATUS_SUCCESS ? 0 : 100000 + static_cast<int>(s); }

cudaStream_t current_stream() {
    cudaStream_t s = g_stream;
    if (g_stream_source) {
        std::uint64_t v = 0;
        if (g_stream_source(&v) == 0) s = reinterpret_cast<cudaStream_t>(v);
    }
    if (g_have_last && s != g_last_stream) {
        // Calls enqueued under the previous stream may still use the shared workspace (and cuDNN's handle state):
        // let them finish before the first call on the new stream.  The old handle itself is not touched (its
        // owner may have destroyed it since), so the whole device is waited for; stream changes are rare.
        // While the new stream is being recorded into a graph nothing may block: the caller has run the step
        // eagerly on that stream before recording it.
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        if (s == nullptr || cudaStreamIsCapturing(s, &cs) != cudaSuccess) cs = cudaStreamCaptureStatusNone;
        if (cs == cudaStreamCaptureStatusNone) cudaDeviceSynchronize();
        (void)cudaGetLastError();
    }
    g_last_stream = s;
    g_have_last = true;
    return s;
}

cudnnHandle_t dnn() {
    if (!g_dnn && cudnnCreate(&g_dnn) != CUDNN_STATUS_SUCCESS) g_dnn = nullptr;
    if (g_dnn) cudnnSetStream(g_dnn, current_stream());
    return g_dnn;
}
cublasHandle_t blas() {
    if (!g_blas && cublasCreate(&g_blas) != CUBLAS_STATUS_SUCCESS) g_blas = nullptr;
    if (g_blas) cublasSetStream(g_blas, current_stream());
    return g_blas;
}
void* workspace(size_t bytes) {
    if (bytes <= g_ws_bytes) return g_ws;
    if (g_ws) cudaFree(g_ws);
    g_ws = nullptr;
    g_ws_bytes = 0;
    if (cudaMalloc(&g_ws, bytes) != cudaSuccess) return nullptr;
    g_ws_bytes = bytes;
    return g_ws;
}

struct ConvPlan {
    cudnnTensorDescriptor_t x = nullptr, y = nullptr, b = nullptr;
    cudnnFilterDescriptor_t w = nullptr;
    cudnnConvolutionDescriptor_t conv = nullptr;
    cudnnConvolutionFwdAlgo_t fwd{};
    cudnnConvolutionBwdDataAlgo_t bwd_data{};
    cudnnConvolutionBwdFilterAlgo_t bwd_filter{};
    size_t ws_fwd = 0, ws_data = 0, ws_filter = 0;
    bool have_fwd = false, have_bwd = false;
    int status = 0;
};

using ConvKey = std::tuple<int, int, int, int, int, int, int, int, int, int, int, int, int, int>;
std::map<ConvKey, ConvPlan> g_plans;

#define KD_DNN(call)                                        \
    do {                                                    \
        cudnnStatus_t st_ = (call);                         \
        if (st_ != CUDNN_STATUS_SUCCESS) { p.status = cudnn_status(st_); return p; } \
    } while (0)

ConvPlan& conv_plan(int dtype, int N, int Cin, int H, int W, int Cout, int Ho, int Wo, int Kh, int Kw, int sh, int sw,
                    int ph, int pw) {
    const ConvKey key{dtype, N, Cin, H, W, Cout, Ho, Wo, Kh, Kw, sh, sw, ph, pw};
    auto it = g_plans.find(key);
    if (it != g_plans.end()) return it->second;
    ConvPlan& p = g_plans[key];
    const cudnnDataType_t dt = dtype == 0 ? CUDNN_DATA_FLOAT : CUDNN_DATA_DOUBLE;
    KD_DNN(cudnnCreateTensorDescriptor(&p.x));
    KD_DNN(cudnnCreateTensorDescriptor(&p.y));
    KD_DNN(cudnnCreateTensorDescriptor(&p.b));
    KD_DNN(cudnnCreateFilterDescriptor(&p.w));
    KD_DNN(cudnnCreateConvolutionDescriptor(&p.conv));
    KD_DNN(cudnnSetTensor4dDescriptor(p.x, CUDNN_TENSOR_NCHW, dt, N, Cin, H, W));
    KD_DNN(cudnnSetFilter4dDescriptor(p.w, dt, CUDNN_TENSOR_NCHW, Cout, Cin, Kh, Kw));
    KD_DNN(cudnnSetConvolution2dDescriptor(p.conv, ph, pw, sh, sw, 1, 1, CUDNN_CROSS_CORRELATION, dt));
    int oN = 0, oC = 0, oH = 0, oW = 0;
    KD_DNN(cudnnGetConvolution2dForwardOutputDim(p.conv, p.x, p.w, &oN, &oC, &oH, &oW));
    if (oN != N || oC != Cout || oH != Ho || oW != Wo) { p.status = static_cast<int>(cudaErrorInvalidValue); return p; }
    KD_DNN(cudnnSetTensor4dDescriptor(p.y, CUDNN_TENSOR_NCHW, dt, N, Cout, Ho, Wo));
    KD_DNN(cudnnSetTensor4dDescriptor(p.b, CUDNN_TENSOR_NCHW, dt, 1, Cout, 1, 1));
    return p;
}

// Algorithm choice: measured once per problem shape (cudnnFind*, which times the candidates on the
// device), falling back to the heuristic the reference uses on every call (cudnnGet*_v7).
// One search times every candidate once, and two candidates a few percent apart swap places from run to
// run; the search is therefore repeated and the candidate with the lowest time seen in any round wins.
// `find(perf, &n)` runs one search; on return perf[0] holds the winner.  Returns -1 when no round succeeded.
template <typename Perf, typename Find>
int pick_fastest(Perf (&perf)[8], Find find) {
    constexpr int kRounds = 3;
    Perf best{};
    bool have = false;
    for (int r = 0; r < kRounds; ++r) {
        int n = 0;
        if (find(perf, &n) != CUDNN_STATUS_SUCCESS) continue;
        for (int i = 0; i < n; ++i)
            if (perf[i].status == CUDNN_STATUS_SUCCESS && perf[i].time >= 0.f && (!have || perf[i].time < best.time)) {
                best = perf[i];
                have = true;
            }
    }
    if (!have) return -1;
    perf[0] = best;
    return 0;
}

int plan_fwd(ConvPlan& p) {
    if (p.have_fwd) return 0;
    cudnnConvolutionFwdAlgoPerf_t perf[8];
    int n = 0;
    cudnnStatus_t s;
    int pick = pick_fastest(perf, [&](cudnnConvolutionFwdAlgoPerf_t* out, int* cnt) {
        return cudnnFindConvolutionForwardAlgorithm(dnn(), p.x, p.w, p.conv, p.y, 8, cnt, out);
    });
    if (pick < 0) {
        s = cudnnGetConvolutionForwardAlgorithm_v7(dnn(), p.x, p.w, p.conv, p.y, 1, &n, perf);
        if (s != CUDNN_STATUS_SUCCESS) return cudnn_status(s);
        pick = 0;
    }
    p.fwd = perf[pick].algo;
    s = cudnnGetConvolutionForwardWorkspaceSize(dnn(), p.x, p.w, p.conv, p.y, p.fwd, &p.ws_fwd);
    if (s != CUDNN_STATUS_SUCCESS) return cudnn_status(s);
    p.have_fwd = true;
    return 0;
}

int plan_bwd(ConvPlan& p) {
    if (p.have_bwd) return 0;
    int n = 0, pick = -1;
    cudnnConvolutionBwdDataAlgoPerf_t pd[8];
    cudnnStatus_t s;
    pick = pick_fastest(pd, [&](cudnnConvolutionBwdDataAlgoPerf_t* out, int* cnt) {
        return cudnnFindConvolutionBackwardDataAlgorithm(dnn(), p.w, p.y, p.conv, p.x, 8, cnt, out);
    });
    if (pick < 0) {
        s = cudnnGetConvolutionBackwardDataAlgorithm_v7(dnn(), p.w, p.y, p.conv, p.x, 1, &n, pd);
        if (s != CUDNN_STATUS_SUCCESS) return cudnn_status(s);
        pick = 0;
    }
    p.bwd_data = pd[pick].algo;
    s = cudnnGetConvolutionBackwardDataWorkspaceSize(dnn(), p.w, p.y, p.conv, p.x, p.bwd_data, &p.ws_data);
    if (s != CUDNN_STATUS_SUCCESS) return cudnn_status(s);
    cudnnConvolutionBwdFilterAlgoPerf_t pf[8];
    pick = pick_fastest(pf, [&](cudnnConvolutionBwdFilterAlgoPerf_t* out, int* cnt) {
        return cudnnFindConvolutionBackwardFilterAlgorithm(dnn(), p.x, p.y, p.conv, p.w, 8, cnt, out);
    });
    if (pick < 0) {
        s = cudnnGetConvolutionBackwardFilterAlgorithm_v7(dnn(), p.x, p.y, p.conv, p.w, 1, &n, pf);
        if (s != CUDNN_STATUS_SUCCESS) return cudnn_status(s);
        pick = 0;
    }
    p.bwd_filter = pf[pick].algo;
    s = cudnnGetConvolutionBackwardFilterWorkspaceSize(dnn(), p.x, p.y, p.conv, p.w, p.bwd_filter, &p.ws_filter);
    if (s != CUDNN_STATUS_SUCCESS) return cudnn_status(s);
    p.have_bwd = true;
    return 0;
}

template <typename T>
int conv_forward(const T* x, const T* w, const T* b, T* y, int N, int Cin, int H, int W, int Cout, int Ho, int Wo, int Kh,
                 int Kw, int sh, int sw, int ph, int pw) {
    if (!x || !w || !y) return -1;
    if (N < 0 || Cin <= 0 || H <= 0 || W <= 0 || Cout < 0 || Ho < 0 || Wo < 0) return -2;
    if (Kh <= 0 || Kw <= 0 || sh <= 0 || sw <= 0 || ph < 0 || pw < 0) return -3;
    if (N == 0 || Cout == 0 || Ho == 0 || Wo == 0) return 0;
    if (!dnn()) return cudnn_status(CUDNN_STATUS_INTERNAL_ERROR);
    ConvPlan& p = conv_plan(std::is_same<T, float>::value ? 0 : 1, N, Cin, H, W, Cout, Ho, Wo, Kh, Kw, sh, sw, ph, pw);
    if (p.status) return p.status;
    if (int st = plan_fwd(p)) return st;
    void* ws = p.ws_fwd ? workspace(p.ws_fwd) : nullptr;
    if (p.ws_fwd && !ws) return static_cast<int>(cudaErrorMemoryAllocation);
    const T one = T(1), zero = T(0);
    cudnnStatus_t s = cudnnConvolutionForward(dnn(), &one, p.x, x, p.w, w, p.conv, p.fwd, ws, p.ws_fwd, &zero, p.y, y);
    if (s != CUDNN_STATUS_SUCCESS) return cudnn_status(s);
    if (b) {
        s = cudnnAddTensor(dnn(), &one, p.b, b, &one, p.y, y);
        if (s != CUDNN_STATUS_SUCCESS) return cudnn_status(s);
    }
    return 0;
}

template <typename T>
int conv_backward(const T* x, const T* w, const T* go, T* gx, T* gw, int N, int Cin, int H, int W, int Cout, int Ho, int Wo,
                  int Kh, int Kw, int sh, int sw, int ph, int pw) {
    if (!x || !w || !go) return -1;
    if (N < 0 || Cin <= 0 || H <= 0 || W <= 0 || Cout < 0 || Ho < 0 || Wo < 0) return -2;
    if (Kh <= 0 || Kw <= 0 || sh <= 0 || sw <= 0 || ph < 0 || pw < 0) return -3;
    if (N == 0 || Cout == 0 || Ho == 0 || Wo == 0) return 0;
    if (!dnn()) return cudnn_status(CUDNN_STATUS_INTERNAL_ERROR);
    ConvPlan& p = conv_plan(std::is_same<T, float>::value ? 0 : 1, N, Cin, H, W, Cout, Ho, Wo, Kh, Kw, sh, sw, ph, pw);
    if (p.status) return p.status;
    if (int st = plan_bwd(p)) return st;
    const size_t need = p.ws_data > p.ws_filter ? p.ws_data : p.ws_filter;
    void* ws = need ? workspace(need) : nullptr;
    if (need && !ws) return static_cast<int>(cudaErrorMemoryAllocation);
    const T one = T(1), zero = T(0);
    if (gx) {
        cudnnStatus_t s = cudnnConvolutionBackwardData(dnn(), &one, p.w, w, p.y, go, p.conv, p.bwd_data, ws, p.ws_data, &zero,
                                                       p.x, gx);
        if (s != CUDNN_STATUS_SUCCESS) return cudnn_status(s);
    }
    if (gw) {
        cudnnStatus_t s = cudnnConvolutionBackwardFilter(dnn(), &one, p.x, x, p.y, go, p.conv, p.bwd_filter, ws, p.ws_filter,
                                                         &zero, p.w, gw);
        if (s != CUDNN_STATUS_SUCCESS) return cudnn_status(s);
    }
    return 0;
}

// Row-major C[M,N] = op(A) * op(B) through column-major cuBLAS: C^T = op(B)^T * op(A)^T.
template <typename T>
int matmul(const T* A, const T* B, T* C, int M, int N, int K, int transA, int transB) {
    if (M < 0 || N < 0 || K < 0) return 1;
    if (M == 0 || N == 0) return 0;
    if (!A || !B || !C) return 2;
    if (!blas()) return 3;
    const T one = T(1), zero = T(0);
    const cublasOperation_t opB = transB ? CUBLAS_OP_T : CUBLAS_OP_N;
    const cublasOperation_t opA = transA ? CUBLAS_OP_T : CUBLAS_OP_N;
    const int ldb = transB ? K : N, lda = transA ? M : K;
    cublasStatus_t s;
    if (std::is_same<T, float>::value)
        s = cublasSgemm(blas(), opB, opA, N, M, K, reinterpret_cast<const float*>(&one), reinterpret_cast<const float*>(B), ldb,
                        reinterpret_cast<const float*>(A), lda, reinterpret_cast<const float*>(&zero),
                        reinterpret_cast<float*>(C), N);
    else
        s = cublasDgemm(blas(), opB, opA, N, M, K, reinterpret_cast<const double*>(&one), reinterpret_cast<const double*>(B),
                        ldb, reinterpret_cast<const double*>(A), lda, reinterpret_cast<const double*>(&zero),
                        reinterpret_cast<double*>(C), N);
    return s == CUBLAS_STATUS_SUCCESS ? 0 : 4;
}

}  // namespace

// An explicit stream for callers that use this library on its own; it also drops a bound source.
KD_API int keydnn_dnn_set_stream(std::uint64_t stream) {
    g_stream_source = nullptr;
    g_stream = reinterpret_cast<cudaStream_t>(stream);
    return 0;
}

// `get_stream_fn` is the address of a function `int f(uint64_t* out)` that stores the stream every call of
// this library must be enqueued on (libkeydnn_b200.so's keydnn_cuda_get_stream); 0 unbinds.
KD_API int keydnn_dnn_bind_stream_source(std::uint64_t get_stream_fn) {
    g_stream_source = reinterpret_cast<StreamSource>(get_stream_fn);
    return 0;
}

// The stream the next call would be enqueued on (tests; diagnostics).
KD_API int keydnn_dnn_get_stream(std::uint64_t* out) {
    if (!out) return -1;
    cudaStream_t s = g_stream;
    if (g_stream_source) {
        std::uint64_t v = 0;
        if (g_stream_source(&v) == 0) s = reinterpret_cast<cudaStream_t>(v);
    }
    *out = reinterpret_cast<std::uint64_t>(s);
    return 0;
}

#define KD_DNN_EXPORTS(T, SUF)                                                                                          \
    KD_API int keydnn_cuda_conv2d_forward_##SUF(const T* x_pad, const T* w, const T* b, T* y, int N, int C_in, int H_pad,  \
                                                int W_pad, int C_out, int H_out, int W_out, int K_h, int K_w, int s_h,   \
                                                int s_w) {                                                              \
        return conv_forward<T>(x_pad, w, b, y, N, C_in, H_pad, W_pad, C_out, H_out, W_out, K_h, K_w, s_h, s_w, 0, 0);    \
    }                                                                                                                   \
    KD_API int keydnn_cuda_conv2d_backward_##SUF(const T* x_pad, const T* w, const T* grad_out, T* grad_x_pad, T* grad_w,  \
                                                 int N, int C_in, int H_pad, int W_pad, int C_out, int H_out, int W_out, \
                                                 int K_h, int K_w, int s_h, int s_w) {                                   \
        return conv_backward<T>(x_pad, w, grad_out, grad_x_pad, grad_w, N, C_in, H_pad, W_pad, C_out, H_out, W_out, K_h,  \
                                K_w, s_h, s_w, 0, 0);                                                                   \
    }                                                                                                                   \
    KD_API int keydnn_cuda_conv2d_forward_ex_##SUF(const T* x, const T* w, const T* b, T* y, int N, int C_in, int H, int W, \
                                                   int C_out, int H_out, int W_out, int K_h, int K_w, int s_h, int s_w,  \
                                                   int p_h, int p_w) {                                                  \
        return conv_forward<T>(x, w, b, y, N, C_in, H, W, C_out, H_out, W_out, K_h, K_w, s_h, s_w, p_h, p_w);            \
    }                                                                                                                   \
    KD_API int keydnn_cuda_conv2d_backward_ex_##SUF(const T* x, const T* w, const T* grad_out, T* grad_x, T* grad_w, int N, \
                                                    int C_in, int H, int W, int C_out, int H_out, int W_out, int K_h,    \
                                                    int K_w, int s_h, int s_w, int p_h, int p_w) {                       \
        return conv_backward<T>(x, w, grad_out, grad_x, grad_w, N, C_in, H, W, C_out, H_out, W_out, K_h, K_w, s_h, s_w,  \
                                p_h, p_w);                                                                              \
    }                                                                                                                   \
    KD_API int keydnn_cuda_matmul_##SUF(const T* A, const T* B, T* C, int M, int N, int K) {                             \
        return matmul<T>(A, B, C, M, N, K, 0, 0);                                                                       \
    }                                                                                                                   \
    KD_API int keydnn_cuda_matmul_ex_##SUF(const T* A, const T* B, T* C, int M, int N, int K, int trans_a, int trans_b) { \
        return matmul<T>(A, B, C, M, N, K, trans_a, trans_b);                                                           \
    }

KD_DNN_EXPORTS(float, f32)
KD_DNN_EXPORTS(double, f64)
