// Softmax forward / backward along one axis of a dense tensor viewed as (outer, len, inner).
//
// Reference: SoftmaxFn (_function.py:547-575, :604-610) runs max -> broadcast_to -> sub -> exp ->
// sum -> broadcast_to -> div (forward) and mul -> sum -> broadcast_to -> sub -> mul (backward), seven
// and five kernels with as many temporaries.  Here each direction is one kernel: one HBM read of
// every operand, one write.  Element arithmetic is the reference's, separately rounded:
//   forward   m = max over the axis (strict >, from -inf; a NaN never wins)
//             e = exp(x - m);  y = e / sum(e)
//   backward  gy = g * y;  dx = y * (g - sum(gy))
// The sums are tree sums (the reference adds serially), hence equal only to rounding.
//
// Compiled with nvcc's default FMA contraction so that exp expands as in the reference build; all
// arithmetic written here uses explicitly rounded intrinsics.
#include "common.cuh"

namespace {

using kd::Rn;

template <typename T> __device__ __forceinline__ T t_exp(T x);
template <> __device__ __forceinline__ float t_exp<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ double t_exp<double>(double x) { return exp(x); }
template <typename T> __device__ __forceinline__ T t_div(T a, T b);
template <> __device__ __forceinline__ float t_div<float>(float a, float b) { return __fdiv_rn(a, b); }
template <> __device__ __forceinline__ double t_div<double>(double a, double b) { return __ddiv_rn(a, b); }
template <typename T> __device__ __forceinline__ T neg_inf() { return -std::numeric_limits<T>::infinity(); }

template <typename T> __device__ __forceinline__ T warp_max(T v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const T w = __shfl_xor_sync(0xffffffffu, v, o);
        v = w > v ? w : v;
    }
    return v;
}
template <typename T> __device__ __forceinline__ T warp_add(T v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = Rn<T>::add(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// ---- rows that fit in the registers of one warp: len <= 32 * R -----------------------------------
// A warp owns a row; lane l holds elements l, l+32, ...  Loads of the R elements are independent.
template <typename T, int R, bool BWD>
__global__ void __launch_bounds__(kThreads)
softmax_warp_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t rows, int len) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kWarps;
    for (int64_t row = warp0; row < rows; row += stride) {
        const T* pa = a + row * len;
        T va[R], vb[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int c = lane + 32 * r;
            if (BWD) {
                va[r] = c < len ? __ldcs(pa + c) : T(0);                  // g
                vb[r] = c < len ? __ldcs(b + row * len + c) : T(0);       // y
            } else {
                va[r] = c < len ? __ldcs(pa + c) : neg_inf<T>();
            }
        }
        if (BWD) {
            T dot = T(0);
#pragma unroll
            for (int r = 0; r < R; ++r) dot = Rn<T>::add(dot, Rn<T>::mul(va[r], vb[r]));
            dot = warp_add(dot);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int c = lane + 32 * r;
                if (c < len) __stcs(out + row * len + c, Rn<T>::mul(vb[r], Rn<T>::sub(va[r], dot)));
            }
        } else {
            T m = neg_inf<T>();
#pragma unroll
            for (int r = 0; r < R; ++r) m = va[r] > m ? va[r] : m;
            m = warp_max(m);
            T s = T(0);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int c = lane + 32 * r;
                va[r] = c < len ? t_exp(Rn<T>::sub(va[r], m)) : T(0);
                s = Rn<T>::add(s, va[r]);
            }
            s = warp_add(s);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int c = lane + 32 * r;
                if (c < len) __stcs(out + row * len + c, t_div(va[r], s));
            }
        }
    }
}

// ---- long rows: one CTA per row, the row staged in shared memory (or re-read from L2 when it
// does not fit: `staged` false) -------------------------------------------------------------------
template <typename T> __device__ __forceinline__ T block_max(T v, T* sm) {
    v = warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    T r = sm[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) r = sm[w] > r ? sm[w] : r;
    return r;
}
template <typename T> __device__ __forceinline__ T block_add(T v, T* sm) {
    v = warp_add(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    T r = sm[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) r = Rn<T>::add(r, sm[w]);
    return r;
}

template <typename T, bool BWD>
__global__ void __launch_bounds__(kThreads)
softmax_block_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t rows, int len,
                     bool staged) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* buf = reinterpret_cast<T*>(smem_raw);          // forward: e;  backward: g*y
    __shared__ T red[kWarps];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* pa = a + row * len;
        const T* pb = BWD ? b + row * len : nullptr;
        T* po = out + row * len;
        if (BWD) {
            T dot = T(0);
            for (int c = threadIdx.x; c < len; c += kThreads) dot = Rn<T>::add(dot, Rn<T>::mul(pa[c], pb[c]));
            dot = block_add(dot, red);
            for (int c = threadIdx.x; c < len; c += kThreads)
                __stcs(po + c, Rn<T>::mul(pb[c], Rn<T>::sub(pa[c], dot)));
        } else {
            T m = neg_inf<T>();
            for (int c = threadIdx.x; c < len; c += kThreads) {
                const T v = pa[c];
                if (staged) buf[c] = v;
                m = v > m ? v : m;
            }
            m = block_max(m, red);
            T s = T(0);
            for (int c = threadIdx.x; c < len; c += kThreads) {
                const T e = t_exp(Rn<T>::sub(staged ? buf[c] : pa[c], m));
                if (staged) buf[c] = e;
                s = Rn<T>::add(s, e);
            }
            s = block_add(s, red);
            for (int c = threadIdx.x; c < len; c += kThreads)
                __stcs(po + c, t_div(staged ? buf[c] : t_exp(Rn<T>::sub(pa[c], m)), s));
        }
        __syncthreads();
    }
}

// ---- axis is not the last one: a thread owns one (outer, inner) line; neighbouring threads are
// neighbouring `inner`, so every access of a warp is contiguous ---------------------------------------
template <typename T, bool BWD>
__global__ void __launch_bounds__(kThreads)
softmax_strided_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t outer, int len,
                       int64_t inner) {
    const int64_t lines = outer * inner;
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; t < lines;
         t += static_cast<int64_t>(gridDim.x) * kThreads) {
        const int64_t o = t / inner, i = t - o * inner;
        const int64_t base = o * len * inner + i;
        if (BWD) {
            T dot = T(0);
            for (int k = 0; k < len; ++k) dot = Rn<T>::add(dot, Rn<T>::mul(a[base + k * inner], b[base + k * inner]));
            for (int k = 0; k < len; ++k)
                out[base + k * inner] = Rn<T>::mul(b[base + k * inner], Rn<T>::sub(a[base + k * inner], dot));
        } else {
            T m = neg_inf<T>();
            for (int k = 0; k < len; ++k) {
                const T v = a[base + k * inner];
                m = v > m ? v : m;
            }
            T s = T(0);
            for (int k = 0; k < len; ++k) s = Rn<T>::add(s, t_exp(Rn<T>::sub(a[base + k * inner], m)));
            for (int k = 0; k < len; ++k) out[base + k * inner] = t_div(t_exp(Rn<T>::sub(a[base + k * inner], m)), s);
        }
    }
}

template <typename T, int R, bool BWD>
void launch_warp(const T* a, const T* b, T* out, int64_t rows, int len) {
    KD_LAUNCH_W((softmax_warp_kernel<T, R, BWD>), 8, (rows + kWarps - 1) / kWarps, kThreads, 0, a, b, out, rows, len);
}

template <typename T, bool BWD>
int softmax(const T* a, const T* b, T* out, int64_t outer, int64_t len, int64_t inner) {
    if (!a || !out || (BWD && !b)) return -1;
    if (outer < 0 || len <= 0 || inner <= 0 || len > 0x7fffffff) return -2;
    if (outer == 0) return 0;
    (void)cudaGetLastError();
    const int n = static_cast<int>(len);
    if (inner > 1) {
        KD_LAUNCH_W((softmax_strided_kernel<T, BWD>), 8, (outer * inner + kThreads - 1) / kThreads, kThreads, 0, a, b, out,
                    outer, n, inner);
        return kd::launch_status();
    }
    if (n <= 32) launch_warp<T, 1, BWD>(a, b, out, outer, n);
    else if (n <= 64) launch_warp<T, 2, BWD>(a, b, out, outer, n);
    else if (n <= 128) launch_warp<T, 4, BWD>(a, b, out, outer, n);
    else if (n <= 256) launch_warp<T, 8, BWD>(a, b, out, outer, n);
    else if (n <= 512) launch_warp<T, 16, BWD>(a, b, out, outer, n);
    else if (n <= 1024 && (!BWD || sizeof(T) == 4)) launch_warp<T, 32, BWD>(a, b, out, outer, n);
    else {
        // stage the row when it fits the opt-in shared memory of one CTA (two CTAs per SM stay resident up to 96 KiB)
        size_t smem = BWD ? 0 : static_cast<size_t>(n) * sizeof(T);
        bool staged = !BWD && smem <= 200 * 1024;
        if (!staged) smem = 0;
        auto kernel = softmax_block_kernel<T, BWD>;
        if (smem > 48 * 1024) {
            static size_t granted = 0;      // per template instance
            if (smem > granted) {
                if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) {
                    (void)cudaGetLastError();
                    staged = false;
                    smem = 0;
                } else {
                    granted = 200 * 1024;
                }
            }
        }
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem) != cudaSuccess || per_sm < 1)
            per_sm = 1;
        const int64_t cap = static_cast<int64_t>(kd::sm_count()) * per_sm * 4;
        const unsigned grid = static_cast<unsigned>(outer < cap ? outer : cap);
        kernel<<<grid, kThreads, smem, kd::stream()>>>(a, b, out, outer, n, staged);
    }
    return kd::launch_status();
}

}  // namespace

#define KD_SOFTMAX_EXPORTS(T, SUF)                                                                                    \
    KD_API int keydnn_cuda_softmax_forward_##SUF(const T* x, T* y, int64_t outer, int64_t len, int64_t inner) {       \
        return softmax<T, false>(x, nullptr, y, outer, len, inner);                                                   \
    }                                                                                                                 \
    KD_API int keydnn_cuda_softmax_backward_##SUF(const T* grad_out, const T* y, T* grad_x, int64_t outer, int64_t len, \
                                                  int64_t inner) {                                                    \
        return softmax<T, true>(grad_out, y, grad_x, outer, len, inner);                                              \
    }

KD_SOFTMAX_EXPORTS(float, f32)
KD_SOFTMAX_EXPORTS(double, f64)
