// Shared device/host helpers for the sm_100a KeyDNN operator library.
//
// Everything in this library is HBM-bound: kernels are written around 16-byte
// global accesses, enough independent loads per thread to cover DRAM latency,
// and grids sized from the SM count of the device the call runs on.
#pragma once

#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>
#include <limits>

#define KD_API extern "C" __attribute__((visibility("default")))

namespace kd {

// ---------------------------------------------------------------------------
// Runtime state owned by runtime.cu
// ---------------------------------------------------------------------------
cudaStream_t stream();          // stream every kernel of the library launches on
int sm_count();                 // SMs of the current device (148 on B200)
// Device scratch for two-stage reductions (partials + completion counters).
// Grows on demand; counters start at zero and every kernel leaves them at zero.
void* scratch(size_t nbytes);
unsigned int* counters(size_t count);

inline int status(cudaError_t e) { return e == cudaSuccess ? 0 : static_cast<int>(e); }

// Launch status of the kernel just enqueued (clears the sticky-free last error).
inline int launch_status() { return status(cudaGetLastError()); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Grid for a grid-stride kernel: enough CTAs to fill every SM `per_sm` times,
// never more than the work available.
inline unsigned grid_for(int64_t work_items, int per_sm) {
    int64_t cap = static_cast<int64_t>(sm_count()) * per_sm;
    int64_t g = work_items < cap ? work_items : cap;
    return static_cast<unsigned>(g < 1 ? 1 : g);
}

// ---------------------------------------------------------------------------
// 4-element packets: one 16-byte access for float, two for double.
// ---------------------------------------------------------------------------
template <typename T> struct Pack4 { T v[4]; };

template <typename T> __device__ __forceinline__ Pack4<T> load4(const T* p);
template <> __device__ __forceinline__ Pack4<float> load4<float>(const float* p) {
    float4 t = __ldg(reinterpret_cast<const float4*>(p));
    Pack4<float> r; r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w; return r;
}
template <> __device__ __forceinline__ Pack4<double> load4<double>(const double* p) {
    double2 a = __ldg(reinterpret_cast<const double2*>(p));
    double2 b = __ldg(reinterpret_cast<const double2*>(p) + 1);
    Pack4<double> r; r.v[0] = a.x; r.v[1] = a.y; r.v[2] = b.x; r.v[3] = b.y; return r;
}
template <> __device__ __forceinline__ Pack4<long long> load4<long long>(const long long* p) {
    longlong2 a = __ldg(reinterpret_cast<const longlong2*>(p));
    longlong2 b = __ldg(reinterpret_cast<const longlong2*>(p) + 1);
    Pack4<long long> r; r.v[0] = a.x; r.v[1] = a.y; r.v[2] = b.x; r.v[3] = b.y; return r;
}

// Streaming loads: data that is touched once (evict-first in L1/L2).
template <typename T> __device__ __forceinline__ Pack4<T> load4_stream(const T* p);
template <> __device__ __forceinline__ Pack4<float> load4_stream<float>(const float* p) {
    float4 t = __ldcs(reinterpret_cast<const float4*>(p));
    Pack4<float> r; r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w; return r;
}
template <> __device__ __forceinline__ Pack4<double> load4_stream<double>(const double* p) {
    double2 a = __ldcs(reinterpret_cast<const double2*>(p));
    double2 b = __ldcs(reinterpret_cast<const double2*>(p) + 1);
    Pack4<double> r; r.v[0] = a.x; r.v[1] = a.y; r.v[2] = b.x; r.v[3] = b.y; return r;
}
template <> __device__ __forceinline__ Pack4<long long> load4_stream<long long>(const long long* p) {
    longlong2 a = __ldcs(reinterpret_cast<const longlong2*>(p));
    longlong2 b = __ldcs(reinterpret_cast<const longlong2*>(p) + 1);
    Pack4<long long> r; r.v[0] = a.x; r.v[1] = a.y; r.v[2] = b.x; r.v[3] = b.y; return r;
}

template <typename T> __device__ __forceinline__ void store4(T* p, const Pack4<T>& r);
template <> __device__ __forceinline__ void store4<float>(float* p, const Pack4<float>& r) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(r.v[0], r.v[1], r.v[2], r.v[3]));
}
template <> __device__ __forceinline__ void store4<double>(double* p, const Pack4<double>& r) {
    __stcs(reinterpret_cast<double2*>(p), make_double2(r.v[0], r.v[1]));
    __stcs(reinterpret_cast<double2*>(p) + 1, make_double2(r.v[2], r.v[3]));
}
template <> __device__ __forceinline__ void store4<long long>(long long* p, const Pack4<long long>& r) {
    __stcs(reinterpret_cast<longlong2*>(p), make_longlong2(r.v[0], r.v[1]));
    __stcs(reinterpret_cast<longlong2*>(p) + 1, make_longlong2(r.v[2], r.v[3]));
}

template <typename T> __device__ __forceinline__ T neg_inf();
template <> __device__ __forceinline__ float neg_inf<float>() { return __int_as_float(0xff800000); }
template <> __device__ __forceinline__ double neg_inf<double>() {
    return __longlong_as_double(static_cast<long long>(0xfff0000000000000ULL));
}

// ---------------------------------------------------------------------------
// Warp / block reductions (sum in double; arg-max pairs)
// ---------------------------------------------------------------------------
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}

// Block-wide sum, result valid in thread 0. `sm` holds one double per warp.
__device__ __forceinline__ double block_sum(double v, double* sm) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) sm[warp] = v;
    __syncthreads();
    double r = 0.0;
    if (warp == 0) {
        r = (lane < nwarps) ? sm[lane] : 0.0;
        r = warp_sum(r);
    }
    __syncthreads();
    return r;
}

// Running maximum with the position of its first occurrence. Selection rule of
// the serial scan it replaces: start from -inf, replace only on strictly
// greater, so NaN never wins and ties keep the smaller index. `idx` stays at
// the sentinel while nothing exceeded -inf; callers map the sentinel to their
// "nothing selected" position.
constexpr long long kNoIndex = std::numeric_limits<long long>::max();

template <typename T> struct ArgMax {
    T val;
    long long idx;
};

template <typename T> __device__ __forceinline__ ArgMax<T> argmax_init() {
    ArgMax<T> a; a.val = neg_inf<T>(); a.idx = kNoIndex; return a;
}

// Serial step: candidate positions are visited in increasing order.
template <typename T> __device__ __forceinline__ void argmax_step(ArgMax<T>& a, T v, long long i) {
    if (v > a.val) { a.val = v; a.idx = i; }
}

// Merge of two partial scans over disjoint index sets.
template <typename T> __device__ __forceinline__ void argmax_merge(ArgMax<T>& a, T v, long long i) {
    if (v > a.val || (v == a.val && i < a.idx)) { a.val = v; a.idx = i; }
}

template <typename T> __device__ __forceinline__ ArgMax<T> warp_argmax(ArgMax<T> a) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        T v = __shfl_down_sync(0xffffffffu, a.val, o);
        long long i = __shfl_down_sync(0xffffffffu, a.idx, o);
        argmax_merge(a, v, i);
    }
    return a;
}

}  // namespace kd
