// exp / log / sqrt, the activation functions built on them, the loss functions and Adam.
//
// Reference: keydnn_cuda_exp.cu:5-40 is the only unary kernel of the reference library; its
// activations (_function.py:54-612), losses (_losses.py:44-408) and Adam (optimizers/_adam.py:170-220)
// are chains of one-op tensor kernels with a temporary between each pair, and log / sqrt copy the
// tensor to the host and back (tensor/mixins/unary/_tensor_log.py:77, _tensor_sqrt.py:81-91).
// Each chain is one pass here.  Every product, sum and quotient is rounded on its own in the
// order the reference applies them (kd::Rn), so a fused result equals the chained one bit for bit.
//
// This file is compiled with nvcc's default FMA contraction (the reference library's setting) so
// that expf / exp / logf / log expand to the same instruction sequence as in the reference build;
// all arithmetic written here goes through explicitly rounded intrinsics and cannot be contracted.
#include "map.cuh"

namespace {

using kd::MapArgs;
using kd::Rn;

template <typename T> __device__ __forceinline__ T t_exp(T x);
template <> __device__ __forceinline__ float t_exp<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ double t_exp<double>(double x) { return exp(x); }
template <typename T> __device__ __forceinline__ T t_log(T x);
template <> __device__ __forceinline__ float t_log<float>(float x) { return logf(x); }
template <> __device__ __forceinline__ double t_log<double>(double x) { return log(x); }
template <typename T> __device__ __forceinline__ T t_sqrt(T x);
template <> __device__ __forceinline__ float t_sqrt<float>(float x) { return __fsqrt_rn(x); }
template <> __device__ __forceinline__ double t_sqrt<double>(double x) { return __dsqrt_rn(x); }
template <typename T> __device__ __forceinline__ T t_div(T a, T b);
template <> __device__ __forceinline__ float t_div<float>(float a, float b) { return __fdiv_rn(a, b); }
template <> __device__ __forceinline__ double t_div<double>(double a, double b) { return __ddiv_rn(a, b); }

// ---- unary --------------------------------------------------------------------------------------
template <typename T> struct FExp { __device__ void operator()(const T (&x)[1], T (&y)[1]) const { y[0] = t_exp(x[0]); } };
template <typename T> struct FLog { __device__ void operator()(const T (&x)[1], T (&y)[1]) const { y[0] = t_log(x[0]); } };
template <typename T> struct FSqrt { __device__ void operator()(const T (&x)[1], T (&y)[1]) const { y[0] = t_sqrt(x[0]); } };
// _tensor_sqrt.py:108: grad_out * (0.5 / out)
template <typename T> struct FSqrtBwd {
    __device__ void operator()(const T (&in)[2], T (&o)[1]) const { o[0] = Rn<T>::mul(in[0], t_div(T(0.5), in[1])); }
};

// ---- sigmoid: _function.py:203-212 (t = exp(-x); t += 1; out = 1 / t), :236-252 -------------------
template <typename T> struct FSigmoid {
    __device__ void operator()(const T (&x)[1], T (&y)[1]) const { y[0] = t_div(T(1), Rn<T>::add(t_exp(-x[0]), T(1))); }
};
template <typename T> struct FSigmoidBwd {   // in: g, y   tmp = g*y; om = (-y) + 1; tmp *= om
    __device__ void operator()(const T (&in)[2], T (&o)[1]) const {
        o[0] = Rn<T>::mul(Rn<T>::mul(in[0], in[1]), Rn<T>::add(-in[1], T(1)));
    }
};

// ---- tanh: _function.py:459-471 ((e^x - e^-x) / (e^x + e^-x)), :490-493 (g - (y*y)*g) -------------
template <typename T> struct FTanh {
    __device__ void operator()(const T (&x)[1], T (&y)[1]) const {
        const T ep = t_exp(x[0]), en = t_exp(-x[0]);
        y[0] = t_div(Rn<T>::sub(ep, en), Rn<T>::add(ep, en));
    }
};
template <typename T> struct FTanhBwd {      // in: g, y
    __device__ void operator()(const T (&in)[2], T (&o)[1]) const {
        o[0] = Rn<T>::sub(in[0], Rn<T>::mul(Rn<T>::mul(in[1], in[1]), in[0]));
    }
};

// ---- relu: _function.py:291-293 (mask = x > 0; x * mask), :311-312 (g * mask) ----------------------
template <typename T> struct FRelu {         // out: y, mask
    __device__ void operator()(const T (&x)[1], T (&o)[2]) const {
        const T m = x[0] > T(0) ? T(1) : T(0);
        o[0] = Rn<T>::mul(x[0], m);
        o[1] = m;
    }
};
template <typename T> struct FReluBwd {      // in: g, x
    __device__ void operator()(const T (&in)[2], T (&o)[1]) const { o[0] = Rn<T>::mul(in[0], in[1] > T(0) ? T(1) : T(0)); }
};

// ---- leaky relu: _function.py:366-377, :401-409 ----------------------------------------------------
//   pos = x > 0; neg = (-pos) + 1; out = x*pos; tmp = x*neg; tmp *= alpha; out += tmp   (same with g for backward)
template <typename T> struct FLeaky {        // in: v (x or g), x
    T alpha;
    __device__ void operator()(const T (&in)[2], T (&o)[1]) const {
        const T pos = in[1] > T(0) ? T(1) : T(0);
        const T neg = Rn<T>::add(-pos, T(1));
        o[0] = Rn<T>::add(Rn<T>::mul(in[0], pos), Rn<T>::mul(Rn<T>::mul(in[0], neg), alpha));
    }
};
template <typename T> struct FLeaky1 {       // forward: v == x, one load
    T alpha;
    __device__ void operator()(const T (&x)[1], T (&o)[1]) const {
        const T in2[2] = {x[0], x[0]};
        FLeaky<T>{alpha}(in2, o);
    }
};

// ---- Adam: optimizers/_adam.py:190-219, every scalar narrowed to T before use --------------------
template <typename T> struct FAdam {         // in: p, g, m, v   out: p, m, v
    T lr, b1, b2, eps, wd, c1, c2, bias1, bias2, gscale;
    bool use_wd, use_scale;
    const T* dev_bias;                       // when set: {bias1, bias2} of this step, left there by adam_tick_kernel
    __device__ void prepare() {
        if (dev_bias) {
            bias1 = __ldg(dev_bias);
            bias2 = __ldg(dev_bias + 1);
        }
    }
    __device__ void operator()(const T (&in)[4], T (&o)[3]) const {
        const T p = in[0];
        T g = in[1];
        if (use_scale) g = Rn<T>::mul(g, gscale);
        if (use_wd) g = Rn<T>::add(g, Rn<T>::mul(wd, p));
        const T m = Rn<T>::add(Rn<T>::mul(b1, in[2]), Rn<T>::mul(c1, g));
        const T v = Rn<T>::add(Rn<T>::mul(b2, in[3]), Rn<T>::mul(c2, Rn<T>::mul(g, g)));
        const T m_hat = t_div(m, bias1);
        const T v_hat = t_div(v, bias2);
        const T denom = Rn<T>::add(t_sqrt(v_hat), eps);
        o[0] = Rn<T>::sub(p, Rn<T>::mul(lr, t_div(m_hat, denom)));
        o[1] = m;
        o[2] = v;
    }
};

// ---- losses ---------------------------------------------------------------------------------------
// _losses.py:86-88 / :173-176: diff = pred - target (kept for backward); sum or mean of diff*diff
template <typename T> struct FSub2 {
    __device__ void operator()(const T (&in)[2], T (&o)[1]) const { o[0] = Rn<T>::sub(in[0], in[1]); }
};
template <typename T> struct FSqDiff {
    __device__ T operator()(const T (&in)[2]) const { const T d = Rn<T>::sub(in[0], in[1]); return Rn<T>::mul(d, d); }
};
// _losses.py:271-272: -(t*log(p) + (1 - t)*log(1 - p))
template <typename T> struct FBce {
    __device__ T operator()(const T (&in)[2]) const {
        const T p = in[0], t = in[1];
        return -Rn<T>::add(Rn<T>::mul(t, t_log(p)), Rn<T>::mul(Rn<T>::sub(T(1), t), t_log(Rn<T>::sub(T(1), p))));
    }
};
// _losses.py:371: -(t*log(p))
template <typename T> struct FCce {
    __device__ T operator()(const T (&in)[2]) const { return -Rn<T>::mul(in[1], t_log(in[0])); }
};

// Upstream scalar of a loss gradient.  The reference reads the scalar to the host (`item()`),
// combines it with the element count in Python doubles and narrows the result at the call
// boundary; the same double arithmetic runs here on the device, so no host read is needed.
//   mode 0: a * g     mode 1: g / a     mode 2: -(g / a)         (g = 1 when `g` is null)
template <typename T>
__device__ __forceinline__ T upstream_scale(const T* g, double a, int mode) {
    const double gv = g ? static_cast<double>(__ldg(g)) : 1.0;
    const double s = mode == 0 ? __dmul_rn(a, gv) : (mode == 1 ? __ddiv_rn(gv, a) : -__ddiv_rn(gv, a));
    return static_cast<T>(s);
}
// _losses.py:122-126 / :211-215: grad_pred = diff * scale; grad_target = grad_pred * -1
template <typename T> struct FScale2 {
    const T* g; double a; int mode;
    __device__ void operator()(const T (&in)[1], T (&o)[2]) const {
        const T s = upstream_scale<T>(g, a, mode);
        o[0] = Rn<T>::mul(in[0], s);
        o[1] = Rn<T>::mul(o[0], T(-1));
    }
};
// _losses.py:305-317: gp = p - t; denom = p * (1 - p); gp /= denom; gp *= g / n
template <typename T> struct FBceBwd {
    const T* g; double a;
    __device__ void operator()(const T (&in)[2], T (&o)[1]) const {
        const T p = in[0], t = in[1];
        const T q = t_div(Rn<T>::sub(p, t), Rn<T>::mul(p, Rn<T>::sub(T(1), p)));
        o[0] = Rn<T>::mul(q, upstream_scale<T>(g, a, 1));
    }
};
// _losses.py:402-405: gp = t / p; gp *= -(g / n)
template <typename T> struct FCceBwd {
    const T* g; double a;
    __device__ void operator()(const T (&in)[2], T (&o)[1]) const {
        o[0] = Rn<T>::mul(t_div(in[1], in[0]), upstream_scale<T>(g, a, 2));
    }
};

template <typename T, typename F>
int unary(const T* x, T* y, int64_t n, F f) {
    if (!x || !y) return -1;
    if (n < 0) return -2;
    if (n == 0) return 0;
    MapArgs<T, 1, 1> a{{x}, {y}};
    return kd::launch_map<T, 1, 1>(a, n, f);
}
template <typename T, typename F>
int binary(const T* u, const T* v, T* y, int64_t n, F f) {
    if (!u || !v || !y) return -1;
    if (n < 0) return -2;
    if (n == 0) return 0;
    MapArgs<T, 2, 1> a{{u, v}, {y}};
    return kd::launch_map<T, 2, 1>(a, n, f);
}

// keydnn_cuda_exp.cu:19-31: 1 for a negative count, 0 for an empty tensor, 2 for a null pointer, 3 for a failed launch
template <typename T>
int exp_reference_abi(const T* x, T* y, int numel) {
    if (numel < 0) return 1;
    if (numel == 0) return 0;
    if (!x || !y) return 2;
    MapArgs<T, 1, 1> a{{x}, {y}};
    return kd::launch_map<T, 1, 1>(a, numel, FExp<T>{}) == 0 ? 0 : 3;
}

// The step count lives on the device: entry i of `table` holds {1 - beta1^(i+1), 1 - beta2^(i+1)} as the caller
// computed them (clamped to the last entry, where both have reached 1); this kernel hands the entry of the current
// step to the update kernel behind it and advances the count.  No launch argument changes from step to step, so a
// recorded step can be replayed.
template <typename T>
__global__ void adam_tick_kernel(const T* __restrict__ table, long long table_len, long long* step, T* bias_now) {
    kd::pdl_prologue();
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        const long long t = *step;
        const long long i = t < table_len ? t : table_len - 1;
        bias_now[0] = table[2 * i];
        bias_now[1] = table[2 * i + 1];
        *step = t + 1;
    }
}

template <typename T>
int adam_step(T* p, const T* g, T* m, T* v, int64_t n, T lr, T b1, T b2, T eps, T wd, T c1, T c2, T bias1, T bias2,
              T gscale, const T* dev_bias = nullptr) {
    if (!p || !g || !m || !v) return -1;
    if (n < 0) return -2;
    if (n == 0) return 0;
    MapArgs<T, 4, 3> a{{p, g, m, v}, {p, m, v}};
    FAdam<T> f{lr, b1, b2, eps, wd, c1, c2, bias1, bias2, gscale, wd != T(0), gscale != T(1), dev_bias};
    // one packet per tensor in flight per thread: the update's long dependent chain (three divisions, a square
    // root) wants resident warps more than it wants loads per thread (measured on B200: 107 us against 186 us
    // with two packets for 25 M parameters)
    return kd::launch_map<T, 4, 3, 1>(a, n, f, 16);
}

template <typename T, typename F>
int loss_sum(const T* pred, const T* target, T* loss, int64_t n, T scale, int finish, F f) {
    if (!pred || !target || !loss) return -1;
    if (n <= 0) return -2;
    MapArgs<T, 2, 1> a{{pred, target}, {loss}};
    return kd::launch_map_sum<T, 2>(a, n, scale, finish, f);
}

}  // namespace

#define KD_ACT_EXPORTS(T, SUF)                                                                                         \
    KD_API int keydnn_cuda_exp_##SUF(const T* x, T* y, int numel) { return exp_reference_abi<T>(x, y, numel); }        \
    KD_API int keydnn_cuda_log_##SUF(const T* x, T* y, int64_t n) { return unary<T>(x, y, n, FLog<T>{}); }             \
    KD_API int keydnn_cuda_sqrt_##SUF(const T* x, T* y, int64_t n) { return unary<T>(x, y, n, FSqrt<T>{}); }           \
    KD_API int keydnn_cuda_sqrt_backward_##SUF(const T* g, const T* y, T* gx, int64_t n) {                             \
        return binary<T>(g, y, gx, n, FSqrtBwd<T>{});                                                                  \
    }                                                                                                                  \
    KD_API int keydnn_cuda_sigmoid_forward_##SUF(const T* x, T* y, int64_t n) { return unary<T>(x, y, n, FSigmoid<T>{}); } \
    KD_API int keydnn_cuda_sigmoid_backward_##SUF(const T* g, const T* y, T* gx, int64_t n) {                          \
        return binary<T>(g, y, gx, n, FSigmoidBwd<T>{});                                                               \
    }                                                                                                                  \
    KD_API int keydnn_cuda_tanh_forward_##SUF(const T* x, T* y, int64_t n) { return unary<T>(x, y, n, FTanh<T>{}); }   \
    KD_API int keydnn_cuda_tanh_backward_##SUF(const T* g, const T* y, T* gx, int64_t n) {                             \
        return binary<T>(g, y, gx, n, FTanhBwd<T>{});                                                                  \
    }                                                                                                                  \
    KD_API int keydnn_cuda_relu_forward_##SUF(const T* x, T* y, T* mask, int64_t n) {                                  \
        if (!x || !y) return -1;                                                                                       \
        if (n < 0) return -2;                                                                                          \
        if (n == 0) return 0;                                                                                          \
        MapArgs<T, 1, 2> a{{x}, {y, mask}};                                                                            \
        return kd::launch_map<T, 1, 2>(a, n, FRelu<T>{});                                                              \
    }                                                                                                                  \
    KD_API int keydnn_cuda_relu_backward_##SUF(const T* g, const T* x, T* gx, int64_t n) {                             \
        return binary<T>(g, x, gx, n, FReluBwd<T>{});                                                                  \
    }                                                                                                                  \
    KD_API int keydnn_cuda_leaky_relu_forward_##SUF(const T* x, T* y, T alpha, int64_t n) {                            \
        return unary<T>(x, y, n, FLeaky1<T>{alpha});                                                                   \
    }                                                                                                                  \
    KD_API int keydnn_cuda_leaky_relu_backward_##SUF(const T* g, const T* x, T* gx, T alpha, int64_t n) {              \
        return binary<T>(g, x, gx, n, FLeaky<T>{alpha});                                                               \
    }                                                                                                                  \
    KD_API int keydnn_cuda_adam_step_##SUF(T* p, const T* g, T* m, T* v, int64_t n, T lr, T beta1, T beta2, T eps,     \
                                           T weight_decay, T one_minus_beta1, T one_minus_beta2, T bias1, T bias2,     \
                                           T grad_scale) {                                                             \
        return adam_step<T>(p, g, m, v, n, lr, beta1, beta2, eps, weight_decay, one_minus_beta1, one_minus_beta2,      \
                            bias1, bias2, grad_scale);                                                                 \
    }                                                                                                                  \
    KD_API int keydnn_cuda_adam_step_counted_##SUF(T* p, const T* g, T* m, T* v, int64_t n, T lr, T beta1, T beta2,    \
                                                   T eps, T weight_decay, T one_minus_beta1, T one_minus_beta2,        \
                                                   const T* bias_table, int64_t table_len, int64_t* step_counter,      \
                                                   T* bias_now, T grad_scale) {                                        \
        if (!bias_table || !step_counter || !bias_now) return -1;                                                      \
        if (table_len <= 0) return -2;                                                                                 \
        (void)cudaGetLastError();                                                                                      \
        (void)kd::launch(adam_tick_kernel<T>, dim3(1), 32, 0, bias_table, static_cast<long long>(table_len),           \
                         reinterpret_cast<long long*>(step_counter), bias_now);                                        \
        if (int st = kd::launch_status()) return st;                                                                   \
        return adam_step<T>(p, g, m, v, n, lr, beta1, beta2, eps, weight_decay, one_minus_beta1, one_minus_beta2,      \
                            T(1), T(1), grad_scale, bias_now);                                                         \
    }                                                                                                                  \
    KD_API int keydnn_cuda_sqdiff_forward_##SUF(const T* pred, const T* target, T* diff, T* loss, int64_t n, int mean) { \
        if (diff) {                                                                                                    \
            const int st = binary<T>(pred, target, diff, n, FSub2<T>{});                                               \
            if (st) return st;                                                                                         \
        }                                                                                                              \
        return loss_sum<T>(pred, target, loss, n, T(1) / static_cast<T>(n), mean ? 1 : 0, FSqDiff<T>{});               \
    }                                                                                                                  \
    KD_API int keydnn_cuda_sqdiff_backward_##SUF(const T* diff, const T* g, double scale, T* grad_pred,                \
                                                 T* grad_target, int64_t n) {                                          \
        if (!diff || !grad_pred) return -1;                                                                            \
        if (n < 0) return -2;                                                                                          \
        if (n == 0) return 0;                                                                                          \
        MapArgs<T, 1, 2> a{{diff}, {grad_pred, grad_target}};                                                          \
        return kd::launch_map<T, 1, 2>(a, n, FScale2<T>{g, scale, 0});                                                 \
    }                                                                                                                  \
    KD_API int keydnn_cuda_bce_forward_##SUF(const T* pred, const T* target, T* loss, int64_t n) {                     \
        return loss_sum<T>(pred, target, loss, n, T(1) / static_cast<T>(n), 1, FBce<T>{});                             \
    }                                                                                                                  \
    KD_API int keydnn_cuda_bce_backward_##SUF(const T* pred, const T* target, const T* g, T* grad_pred, int64_t n) {   \
        return binary<T>(pred, target, grad_pred, n, FBceBwd<T>{g, static_cast<double>(n)});                           \
    }                                                                                                                  \
    KD_API int keydnn_cuda_cce_forward_##SUF(const T* pred, const T* target, T* loss, int64_t n, int64_t batch) {      \
        if (batch <= 0) return -2;                                                                                     \
        return loss_sum<T>(pred, target, loss, n, static_cast<T>(batch), 2, FCce<T>{});                                \
    }                                                                                                                  \
    KD_API int keydnn_cuda_cce_backward_##SUF(const T* pred, const T* target, const T* g, T* grad_pred, int64_t n,     \
                                              int64_t batch) {                                                         \
        if (batch <= 0) return -2;                                                                                     \
        return binary<T>(pred, target, grad_pred, n, FCceBwd<T>{g, static_cast<double>(batch)});                       \
    }

KD_ACT_EXPORTS(float, f32)
KD_ACT_EXPORTS(double, f64)
