// Elementwise family: neg, add/sub/mul/div, six compares, scalar and in-place
// variants, fill, and the fused SGD(-momentum) update.
//
// Replaces the reference kernels of
//   KeyDNNV2CudaNative/keydnn_tensor_arithmetic.cu:25-254 (one element per
//   thread, 4-byte accesses, launch_1d :65-77), keydnn_mul.cu:8-131 and
//   keydnn_fill_cuda.cu:19-53,
// with one streaming kernel template: every thread moves UNROLL independent
// 4-element packets (16-byte accesses for float, 32-byte for double) per trip of a grid-stride loop, all loads
// of a trip issued before the first use.  Arithmetic is one correctly rounded
// IEEE operation per element exactly as in the reference (no fast-math, no FMA
// contraction), so results are bit-identical to it.
#include "common.cuh"

namespace {

using kd::Pack4;

constexpr int kThreads = 256;

enum Mode { kUnary = 0, kBinary = 1, kScalar = 2 };

struct OpNeg { template <typename T> __device__ T operator()(T a, T) const { return -a; } };
struct OpAdd { template <typename T> __device__ T operator()(T a, T b) const { return a + b; } };
struct OpSub { template <typename T> __device__ T operator()(T a, T b) const { return a - b; } };
struct OpMul { template <typename T> __device__ T operator()(T a, T b) const { return a * b; } };
struct OpDiv { template <typename T> __device__ T operator()(T a, T b) const { return a / b; } };
struct OpGt { template <typename T> __device__ float operator()(T a, T b) const { return a > b ? 1.0f : 0.0f; } };
struct OpGe { template <typename T> __device__ float operator()(T a, T b) const { return a >= b ? 1.0f : 0.0f; } };
struct OpLt { template <typename T> __device__ float operator()(T a, T b) const { return a < b ? 1.0f : 0.0f; } };
struct OpLe { template <typename T> __device__ float operator()(T a, T b) const { return a <= b ? 1.0f : 0.0f; } };
struct OpEq { template <typename T> __device__ float operator()(T a, T b) const { return a == b ? 1.0f : 0.0f; } };
struct OpNe { template <typename T> __device__ float operator()(T a, T b) const { return a != b ? 1.0f : 0.0f; } };

// Packet path: all pointers aligned to one packet (16 bytes for float, 32 for double). `a` may alias `y` (in-place ops):
// a thread reads its own packets before it writes them and nobody else touches
// them, and the loads are ordinary coherent loads.
template <typename TI, typename TO, int MODE, int UNROLL, typename Op>
__global__ void __launch_bounds__(kThreads)
ew_packet_kernel(const TI* a, const TI* b, TI alpha, TO* y, int64_t n, Op op) {
    kd::pdl_prologue();
    const int64_t n4 = n >> 2;
    const int64_t tile = static_cast<int64_t>(kThreads) * UNROLL;
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * tile; base < n4;
         base += static_cast<int64_t>(gridDim.x) * tile) {
        Pack4<TI> va[UNROLL], vb[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t p = base + u * kThreads + threadIdx.x;
            if (p < n4) {
                va[u] = kd::load4_stream(a + 4 * p);
                if (MODE == kBinary) vb[u] = kd::load4_stream(b + 4 * p);
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t p = base + u * kThreads + threadIdx.x;
            if (p < n4) {
                Pack4<TO> r;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    r.v[k] = op(va[u].v[k], MODE == kBinary ? vb[u].v[k] : alpha);
                kd::store4(y + 4 * p, r);
            }
        }
    }
    // ragged tail (n % 4 elements)
    if (blockIdx.x == 0) {
        const int64_t i = (n4 << 2) + threadIdx.x;
        if (threadIdx.x < 4 && i < n) y[i] = op(a[i], MODE == kBinary ? b[i] : alpha);
    }
}

// Any alignment: one element per thread per trip, still coalesced.
template <typename TI, typename TO, int MODE, typename Op>
__global__ void __launch_bounds__(kThreads)
ew_scalar_kernel(const TI* a, const TI* b, TI alpha, TO* y, int64_t n, Op op) {
    kd::pdl_prologue();
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * kThreads)
        y[i] = op(a[i], MODE == kBinary ? b[i] : alpha);
}

template <typename TI, typename TO, int MODE, typename Op>
int launch_ew(const TI* a, const TI* b, TI alpha, TO* y, int64_t n, Op op) {
    (void)cudaGetLastError();   // report this launch, not a stale error
    const bool vec = kd::aligned_pack<TI>(a) && kd::aligned_pack<TO>(y) && (MODE != kBinary || kd::aligned_pack<TI>(b));
    if (vec) {
        constexpr int UNROLL = (MODE == kBinary) ? 4 : 8;
        const int64_t tiles = ((n >> 2) + kThreads * UNROLL - 1) / (kThreads * UNROLL);
        KD_LAUNCH_W((ew_packet_kernel<TI, TO, MODE, UNROLL, Op>), 64, tiles, kThreads, 0, a, b, alpha, y, n, op);
    } else {
        const unsigned grid = kd::grid_for((n + kThreads - 1) / kThreads, 16);
        (void)kd::launch(ew_scalar_kernel<TI, TO, MODE, Op>, dim3(grid), kThreads, 0, a, b, alpha, y, n, op);
    }
    return kd::launch_status();
}

// --- fill -------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads) fill_kernel(T* y, int64_t n, T value, int head) {
    kd::pdl_prologue();
    // `head` elements bring y up to a packet boundary; packets follow; tail last.
    const int64_t body = n - head;
    const int64_t n4 = body >> 2;
    T* yb = y + head;
    Pack4<T> r;
    r.v[0] = r.v[1] = r.v[2] = r.v[3] = value;
    for (int64_t p = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; p < n4;
         p += static_cast<int64_t>(gridDim.x) * kThreads)
        kd::store4(yb + 4 * p, r);
    if (blockIdx.x == 0) {
        if (threadIdx.x < head) y[threadIdx.x] = value;
        const int64_t i = head + (n4 << 2) + (threadIdx.x - 32);
        if (threadIdx.x >= 32 && threadIdx.x < 36 && i < n) y[i] = value;
    }
}

template <typename T>
int launch_fill(T* y, int64_t n, T value) {
    if (!y) return -1;
    if (n < 0) return -2;
    if (n == 0) return 0;
    (void)cudaGetLastError();
    const uintptr_t addr = reinterpret_cast<uintptr_t>(y);
    if (addr % sizeof(T)) return static_cast<int>(cudaErrorMisalignedAddress);
    constexpr uintptr_t kA = sizeof(T) * 4;   // packet alignment
    int head = static_cast<int>(((kA - (addr & (kA - 1))) & (kA - 1)) / sizeof(T));
    if (head > n) head = static_cast<int>(n);
    KD_LAUNCH_W(fill_kernel<T>, 16, ((n >> 2) + kThreads - 1) / kThreads + 1, kThreads, 0, y, n, value, head);
    return kd::launch_status();
}

// --- fused SGD / SGD-momentum -------------------------------------------------
// Op order of the reference optimizer step (optimizers/_sgd.py:130-140), each
// product and sum rounded on its own:
//   t1 = p * wd ; g2 = g + t1 ; [v = v * mu + g2] ; t2 = (v or g2) * lr ; p = p - t2
// `gscale` pre-multiplies g (1/world after a gradient all-reduce); 1 skips it.
using kd::Rn;

template <typename T>
__device__ __forceinline__ void sgd_one(T& p, T g, T* v, T lr, T mu, T wd, T gscale, bool use_scale, bool use_wd) {
    if (use_scale) g = Rn<T>::mul(g, gscale);
    if (use_wd) g = Rn<T>::add(g, Rn<T>::mul(p, wd));
    if (v) {
        *v = Rn<T>::add(Rn<T>::mul(*v, mu), g);
        g = *v;
    }
    p = Rn<T>::sub(p, Rn<T>::mul(g, lr));
}

template <typename T, bool MOMENTUM, bool VEC>
__global__ void __launch_bounds__(kThreads)
sgd_kernel(T* p, const T* g, T* v, int64_t n, T lr, T mu, T wd, T gscale, bool use_scale, bool use_wd) {
    kd::pdl_prologue();
    if (VEC) {
        constexpr int UNROLL = 2;
        const int64_t n4 = n >> 2;
        const int64_t tile = static_cast<int64_t>(kThreads) * UNROLL;
        for (int64_t base = static_cast<int64_t>(blockIdx.x) * tile; base < n4;
             base += static_cast<int64_t>(gridDim.x) * tile) {
            Pack4<T> vp[UNROLL], vg[UNROLL], vv[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int64_t q = base + u * kThreads + threadIdx.x;
                if (q < n4) {
                    vp[u] = kd::load4_stream(p + 4 * q);
                    vg[u] = kd::load4_stream(g + 4 * q);
                    if (MOMENTUM) vv[u] = kd::load4_stream(v + 4 * q);
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int64_t q = base + u * kThreads + threadIdx.x;
                if (q < n4) {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        sgd_one<T>(vp[u].v[k], vg[u].v[k], MOMENTUM ? &vv[u].v[k] : nullptr, lr, mu, wd, gscale,
                                   use_scale, use_wd);
                    kd::store4(p + 4 * q, vp[u]);
                    if (MOMENTUM) kd::store4(v + 4 * q, vv[u]);
                }
            }
        }
        if (blockIdx.x == 0) {
            const int64_t i = (n4 << 2) + threadIdx.x;
            if (threadIdx.x < 4 && i < n) {
                T pi = p[i];
                T vi = MOMENTUM ? v[i] : T(0);
                sgd_one<T>(pi, g[i], MOMENTUM ? &vi : nullptr, lr, mu, wd, gscale, use_scale, use_wd);
                p[i] = pi;
                if (MOMENTUM) v[i] = vi;
            }
        }
    } else {
        for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n;
             i += static_cast<int64_t>(gridDim.x) * kThreads) {
            T pi = p[i];
            T vi = MOMENTUM ? v[i] : T(0);
            sgd_one<T>(pi, g[i], MOMENTUM ? &vi : nullptr, lr, mu, wd, gscale, use_scale, use_wd);
            p[i] = pi;
            if (MOMENTUM) v[i] = vi;
        }
    }
}

// --- fused backward of mul and div ----------------------------------------------
// The reference's closures run one kernel per product (tensor/mixins/arithmetic/
// _tensor_multiplication.py:98-103: g*b, g*a; _tensor_division.py:104-114: g/b, then g*a, neg,
// b*b, div), re-reading g, a, b for each.  One pass computes both gradients with the same
// separately rounded operations: DIV == false: ga = g*b, gb = g*a;
// DIV == true: ga = g/b, gb = (-(g*a)) / (b*b).  Either output may be null.
template <typename T, bool DIV>
__global__ void __launch_bounds__(kThreads)
muldiv_backward_kernel(const T* __restrict__ g, const T* __restrict__ a, const T* __restrict__ b, T* ga, T* gb, int64_t n,
                       bool vec) {
    kd::pdl_prologue();
    if (vec) {
        constexpr int UNROLL = 2;
        const int64_t n4 = n >> 2;
        const int64_t tile = static_cast<int64_t>(kThreads) * UNROLL;
        for (int64_t base = static_cast<int64_t>(blockIdx.x) * tile; base < n4;
             base += static_cast<int64_t>(gridDim.x) * tile) {
            Pack4<T> vg[UNROLL], va[UNROLL], vb[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int64_t p = base + u * kThreads + threadIdx.x;
                if (p < n4) {
                    vg[u] = kd::load4_stream(g + 4 * p);
                    va[u] = kd::load4_stream(a + 4 * p);
                    vb[u] = kd::load4_stream(b + 4 * p);
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int64_t p = base + u * kThreads + threadIdx.x;
                if (p < n4) {
                    Pack4<T> ra, rb;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (DIV) {
                            ra.v[k] = vg[u].v[k] / vb[u].v[k];
                            rb.v[k] = (-Rn<T>::mul(vg[u].v[k], va[u].v[k])) / Rn<T>::mul(vb[u].v[k], vb[u].v[k]);
                        } else {
                            ra.v[k] = Rn<T>::mul(vg[u].v[k], vb[u].v[k]);
                            rb.v[k] = Rn<T>::mul(vg[u].v[k], va[u].v[k]);
                        }
                    }
                    if (ga) kd::store4(ga + 4 * p, ra);
                    if (gb) kd::store4(gb + 4 * p, rb);
                }
            }
        }
    }
    const int64_t done = vec ? ((n >> 2) << 2) : 0;
    for (int64_t i = done + static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * kThreads) {
        if (DIV) {
            if (ga) ga[i] = g[i] / b[i];
            if (gb) gb[i] = (-Rn<T>::mul(g[i], a[i])) / Rn<T>::mul(b[i], b[i]);
        } else {
            if (ga) ga[i] = Rn<T>::mul(g[i], b[i]);
            if (gb) gb[i] = Rn<T>::mul(g[i], a[i]);
        }
    }
}

template <typename T, bool DIV>
int launch_muldiv_backward(const T* g, const T* a, const T* b, T* ga, T* gb, int64_t n) {
    if (!g || !a || !b || (!ga && !gb)) return static_cast<int>(cudaErrorInvalidDevicePointer);
    if (n <= 0) return 0;
    (void)cudaGetLastError();
    const bool vec = kd::aligned_pack<T>(g) && kd::aligned_pack<T>(a) && kd::aligned_pack<T>(b) &&
                     (!ga || kd::aligned_pack<T>(ga)) && (!gb || kd::aligned_pack<T>(gb));
    const int64_t tiles = vec ? ((n >> 2) + kThreads * 2 - 1) / (kThreads * 2) : (n + kThreads - 1) / kThreads;
    KD_LAUNCH_W((muldiv_backward_kernel<T, DIV>), 64, tiles, kThreads, 0, g, a, b, ga, gb, n, vec);
    return kd::launch_status();
}

template <typename T>
int launch_sgd(T* p, const T* g, T* v, int64_t n, T lr, T mu, T wd, T gscale) {
    if (!p || !g) return -1;
    if (n < 0) return -2;
    if (n == 0) return 0;
    (void)cudaGetLastError();
    const bool vec = kd::aligned_pack<T>(p) && kd::aligned_pack<T>(g) && (!v || kd::aligned_pack<T>(v));
    const bool use_scale = !(gscale == T(1));
    const bool use_wd = !(wd == T(0));
    const int64_t tiles = vec ? ((n >> 2) + kThreads * 2 - 1) / (kThreads * 2) : (n + kThreads - 1) / kThreads;
    if (v) {
        if (vec) KD_LAUNCH_W((sgd_kernel<T, true, true>), 16, tiles, kThreads, 0, p, g, v, n, lr, mu, wd, gscale, use_scale, use_wd);
        else KD_LAUNCH_W((sgd_kernel<T, true, false>), 16, tiles, kThreads, 0, p, g, v, n, lr, mu, wd, gscale, use_scale, use_wd);
    } else {
        if (vec) KD_LAUNCH_W((sgd_kernel<T, false, true>), 16, tiles, kThreads, 0, p, g, v, n, lr, mu, wd, gscale, use_scale, use_wd);
        else KD_LAUNCH_W((sgd_kernel<T, false, false>), 16, tiles, kThreads, 0, p, g, v, n, lr, mu, wd, gscale, use_scale, use_wd);
    }
    return kd::launch_status();
}

constexpr int kBadPtr = static_cast<int>(cudaErrorInvalidDevicePointer);

}  // namespace

// ---------------------------------------------------------------------------
// C ABI.  Guards follow the reference: null pointer -> cudaErrorInvalidDevicePointer,
// n <= 0 -> 0 without a launch (keydnn_tensor_arithmetic.cu:65-77, 265-571).
// ---------------------------------------------------------------------------
#define KD_EW_UNARY(NAME, OP)                                                                     \
    KD_API int keydnn_cuda_##NAME##_f32(const float* x, float* y, int64_t n) {                    \
        if (!x || !y) return kBadPtr;                                                             \
        if (n <= 0) return 0;                                                                     \
        return launch_ew<float, float, kUnary>(x, nullptr, 0.0f, y, n, OP{});                     \
    }                                                                                             \
    KD_API int keydnn_cuda_##NAME##_f64(const double* x, double* y, int64_t n) {                  \
        if (!x || !y) return kBadPtr;                                                             \
        if (n <= 0) return 0;                                                                     \
        return launch_ew<double, double, kUnary>(x, nullptr, 0.0, y, n, OP{});                    \
    }

#define KD_EW_BINARY(NAME, OP, TO32, TO64)                                                        \
    KD_API int keydnn_cuda_##NAME##_f32(const float* a, const float* b, TO32* y, int64_t n) {     \
        if (!a || !b || !y) return kBadPtr;                                                       \
        if (n <= 0) return 0;                                                                     \
        return launch_ew<float, TO32, kBinary>(a, b, 0.0f, y, n, OP{});                           \
    }                                                                                             \
    KD_API int keydnn_cuda_##NAME##_f64(const double* a, const double* b, TO64* y, int64_t n) {   \
        if (!a || !b || !y) return kBadPtr;                                                       \
        if (n <= 0) return 0;                                                                     \
        return launch_ew<double, TO64, kBinary>(a, b, 0.0, y, n, OP{});                           \
    }

#define KD_EW_SCALAR(NAME, OP, TO32, TO64)                                                        \
    KD_API int keydnn_cuda_##NAME##_f32(const float* a, float alpha, TO32* y, int64_t n) {        \
        if (!a || !y) return kBadPtr;                                                             \
        if (n <= 0) return 0;                                                                     \
        return launch_ew<float, TO32, kScalar>(a, nullptr, alpha, y, n, OP{});                    \
    }                                                                                             \
    KD_API int keydnn_cuda_##NAME##_f64(const double* a, double alpha, TO64* y, int64_t n) {      \
        if (!a || !y) return kBadPtr;                                                             \
        if (n <= 0) return 0;                                                                     \
        return launch_ew<double, TO64, kScalar>(a, nullptr, alpha, y, n, OP{});                   \
    }

#define KD_EW_INPLACE(NAME, OP)                                                                   \
    KD_API int keydnn_cuda_##NAME##_f32(float* a, const float* b, int64_t n) {                    \
        if (!a || !b) return kBadPtr;                                                             \
        if (n <= 0) return 0;                                                                     \
        return launch_ew<float, float, kBinary>(a, b, 0.0f, a, n, OP{});                          \
    }                                                                                             \
    KD_API int keydnn_cuda_##NAME##_f64(double* a, const double* b, int64_t n) {                  \
        if (!a || !b) return kBadPtr;                                                             \
        if (n <= 0) return 0;                                                                     \
        return launch_ew<double, double, kBinary>(a, b, 0.0, a, n, OP{});                         \
    }

#define KD_EW_SCALAR_INPLACE(NAME, OP)                                                            \
    KD_API int keydnn_cuda_##NAME##_f32(float* a, float alpha, int64_t n) {                       \
        if (!a) return kBadPtr;                                                                   \
        if (n <= 0) return 0;                                                                     \
        return launch_ew<float, float, kScalar>(a, nullptr, alpha, a, n, OP{});                   \
    }                                                                                             \
    KD_API int keydnn_cuda_##NAME##_f64(double* a, double alpha, int64_t n) {                     \
        if (!a) return kBadPtr;                                                                   \
        if (n <= 0) return 0;                                                                     \
        return launch_ew<double, double, kScalar>(a, nullptr, alpha, a, n, OP{});                 \
    }

KD_EW_UNARY(neg, OpNeg)

KD_EW_BINARY(add, OpAdd, float, double)
KD_EW_BINARY(sub, OpSub, float, double)
KD_EW_BINARY(div, OpDiv, float, double)
KD_EW_BINARY(gt, OpGt, float, float)
KD_EW_BINARY(ge, OpGe, float, float)
KD_EW_BINARY(lt, OpLt, float, float)
KD_EW_BINARY(le, OpLe, float, float)
KD_EW_BINARY(eq, OpEq, float, float)
KD_EW_BINARY(ne, OpNe, float, float)

KD_EW_SCALAR(add_scalar, OpAdd, float, double)
KD_EW_SCALAR(sub_scalar, OpSub, float, double)
KD_EW_SCALAR(div_scalar, OpDiv, float, double)
KD_EW_SCALAR(gt_scalar, OpGt, float, float)
KD_EW_SCALAR(ge_scalar, OpGe, float, float)
KD_EW_SCALAR(lt_scalar, OpLt, float, float)
KD_EW_SCALAR(le_scalar, OpLe, float, float)
KD_EW_SCALAR(eq_scalar, OpEq, float, float)
KD_EW_SCALAR(ne_scalar, OpNe, float, float)

KD_EW_INPLACE(add_inplace, OpAdd)
KD_EW_INPLACE(sub_inplace, OpSub)
KD_EW_INPLACE(div_inplace, OpDiv)

KD_EW_SCALAR_INPLACE(add_scalar_inplace, OpAdd)
KD_EW_SCALAR_INPLACE(sub_scalar_inplace, OpSub)
KD_EW_SCALAR_INPLACE(div_scalar_inplace, OpDiv)

// mul family: `int numel` and the 0/1/2/3 status convention of keydnn_mul.cu:64-131
// (1 = negative count, 2 = null pointer, 3 = launch failure).
#define KD_MUL_STATUS(expr) ((expr) == 0 ? 0 : 3)

KD_API int keydnn_cuda_mul_f32(const float* a, const float* b, float* y, int numel) {
    if (numel < 0) return 1;
    if (numel == 0) return 0;
    if (!a || !b || !y) return 2;
    return KD_MUL_STATUS((launch_ew<float, float, kBinary>(a, b, 0.0f, y, numel, OpMul{})));
}
KD_API int keydnn_cuda_mul_f64(const double* a, const double* b, double* y, int numel) {
    if (numel < 0) return 1;
    if (numel == 0) return 0;
    if (!a || !b || !y) return 2;
    return KD_MUL_STATUS((launch_ew<double, double, kBinary>(a, b, 0.0, y, numel, OpMul{})));
}
KD_API int keydnn_cuda_mul_scalar_f32(const float* a, float alpha, float* y, int numel) {
    if (numel < 0) return 1;
    if (numel == 0) return 0;
    if (!a || !y) return 2;
    return KD_MUL_STATUS((launch_ew<float, float, kScalar>(a, nullptr, alpha, y, numel, OpMul{})));
}
KD_API int keydnn_cuda_mul_scalar_f64(const double* a, double alpha, double* y, int numel) {
    if (numel < 0) return 1;
    if (numel == 0) return 0;
    if (!a || !y) return 2;
    return KD_MUL_STATUS((launch_ew<double, double, kScalar>(a, nullptr, alpha, y, numel, OpMul{})));
}
KD_API int keydnn_cuda_mul_inplace_f32(float* a, const float* b, int numel) {
    if (numel < 0) return 1;
    if (numel == 0) return 0;
    if (!a || !b) return 2;
    return KD_MUL_STATUS((launch_ew<float, float, kBinary>(a, b, 0.0f, a, numel, OpMul{})));
}
KD_API int keydnn_cuda_mul_inplace_f64(double* a, const double* b, int numel) {
    if (numel < 0) return 1;
    if (numel == 0) return 0;
    if (!a || !b) return 2;
    return KD_MUL_STATUS((launch_ew<double, double, kBinary>(a, b, 0.0, a, numel, OpMul{})));
}
KD_API int keydnn_cuda_mul_scalar_inplace_f32(float* a, float alpha, int numel) {
    if (numel < 0) return 1;
    if (numel == 0) return 0;
    if (!a) return 2;
    return KD_MUL_STATUS((launch_ew<float, float, kScalar>(a, nullptr, alpha, a, numel, OpMul{})));
}
KD_API int keydnn_cuda_mul_scalar_inplace_f64(double* a, double alpha, int numel) {
    if (numel < 0) return 1;
    if (numel == 0) return 0;
    if (!a) return 2;
    return KD_MUL_STATUS((launch_ew<double, double, kScalar>(a, nullptr, alpha, a, numel, OpMul{})));
}

// Additive: 64-bit counts for the mul family (the reference's `int numel`
// stops at 2^31-1 elements).
KD_API int keydnn_cuda_mul64_f32(const float* a, const float* b, float* y, int64_t n) {
    if (!a || !b || !y) return kBadPtr;
    if (n <= 0) return 0;
    return launch_ew<float, float, kBinary>(a, b, 0.0f, y, n, OpMul{});
}
KD_API int keydnn_cuda_mul64_f64(const double* a, const double* b, double* y, int64_t n) {
    if (!a || !b || !y) return kBadPtr;
    if (n <= 0) return 0;
    return launch_ew<double, double, kBinary>(a, b, 0.0, y, n, OpMul{});
}

// fill: keydnn_fill_cuda.cu:28-62 (-1 null, -2 negative count, 0 for empty).
KD_API int keydnn_cuda_fill_f32(float* y, int64_t numel, float value) { return launch_fill<float>(y, numel, value); }
KD_API int keydnn_cuda_fill_f64(double* y, int64_t numel, double value) { return launch_fill<double>(y, numel, value); }

// Additive: one pass over (p, g[, v]) instead of the reference's five tensor
// passes and four temporaries per parameter (optimizers/_sgd.py:119-140 driven
// through tensor/mixins/arithmetic/_base.py:459-536).  `v` may be null (plain
// SGD).  Momentum has no counterpart in the reference optimizer.
KD_API int keydnn_cuda_sgd_momentum_step_f32(float* p, const float* g, float* v, int64_t n, float lr, float momentum,
                                             float weight_decay, float grad_scale) {
    return launch_sgd<float>(p, g, v, n, lr, momentum, weight_decay, grad_scale);
}
KD_API int keydnn_cuda_sgd_momentum_step_f64(double* p, const double* g, double* v, int64_t n, double lr,
                                             double momentum, double weight_decay, double grad_scale) {
    return launch_sgd<double>(p, g, v, n, lr, momentum, weight_decay, grad_scale);
}

// Additive: both gradients of a product / a quotient in one pass (see muldiv_backward_kernel).
KD_API int keydnn_cuda_mul_backward_f32(const float* g, const float* a, const float* b, float* ga, float* gb, int64_t n) {
    return launch_muldiv_backward<float, false>(g, a, b, ga, gb, n);
}
KD_API int keydnn_cuda_mul_backward_f64(const double* g, const double* a, const double* b, double* ga, double* gb, int64_t n) {
    return launch_muldiv_backward<double, false>(g, a, b, ga, gb, n);
}
KD_API int keydnn_cuda_div_backward_f32(const float* g, const float* a, const float* b, float* ga, float* gb, int64_t n) {
    return launch_muldiv_backward<float, true>(g, a, b, ga, gb, n);
}
KD_API int keydnn_cuda_div_backward_f64(const double* g, const double* a, const double* b, double* ga, double* gb, int64_t n) {
    return launch_muldiv_backward<double, true>(g, a, b, ga, gb, n);
}
