// Streaming map over flat tensors with several inputs and outputs, and its reducing twin.
//
// The reference builds activations, losses and optimizer steps out of one-op elementwise kernels
// (keydnn_tensor_arithmetic.cu:25-254) with a temporary tensor between each pair.  `map_kernel`
// runs a whole chain per element in registers: NIN tensors in, NOUT tensors out, one 4-element
// packet per access (16 bytes for float, 32 for double), UNROLL packets in flight per thread.
// An output may alias an input: a thread reads all of its packets before it writes any, and no
// other thread touches them.
#pragma once
#include "common.cuh"

namespace kd {

constexpr int kMapThreads = 256;

template <typename T, int NIN, int NOUT>
struct MapArgs {
    const T* in[NIN];
    T* out[NOUT];
};

// A functor may define prepare(): it runs once per thread behind the dependency wait and before the first
// element, e.g. to fetch launch-invariant scalars that an earlier kernel of the stream left in device memory.
template <typename F> __device__ __forceinline__ auto map_prepare(F& f, int) -> decltype(f.prepare(), void()) { f.prepare(); }
template <typename F> __device__ __forceinline__ void map_prepare(F&, long) {}

template <typename T, int NIN, int NOUT, int UNROLL, bool VEC, typename F>
__global__ void __launch_bounds__(kMapThreads)
map_kernel(MapArgs<T, NIN, NOUT> a, int64_t n, F f) {
    kd::pdl_prologue();
    map_prepare(f, 0);
    if (VEC) {
        const int64_t n4 = n >> 2;
        const int64_t tile = static_cast<int64_t>(kMapThreads) * UNROLL;
        for (int64_t base = static_cast<int64_t>(blockIdx.x) * tile; base < n4;
             base += static_cast<int64_t>(gridDim.x) * tile) {
            Pack4<T> vin[UNROLL][NIN];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int64_t p = base + u * kMapThreads + threadIdx.x;
                if (p < n4) {
#pragma unroll
                    for (int i = 0; i < NIN; ++i) vin[u][i] = load4_stream(a.in[i] + 4 * p);
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int64_t p = base + u * kMapThreads + threadIdx.x;
                if (p < n4) {
                    Pack4<T> vout[NOUT];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        T xi[NIN], yo[NOUT];
#pragma unroll
                        for (int i = 0; i < NIN; ++i) xi[i] = vin[u][i].v[k];
                        f(xi, yo);
#pragma unroll
                        for (int o = 0; o < NOUT; ++o) vout[o].v[k] = yo[o];
                    }
#pragma unroll
                    for (int o = 0; o < NOUT; ++o)
                        if (a.out[o]) store4(a.out[o] + 4 * p, vout[o]);
                }
            }
        }
        if (blockIdx.x == 0 && threadIdx.x < 4) {          // ragged tail (n % 4 elements)
            const int64_t i = (n4 << 2) + threadIdx.x;
            if (i < n) {
                T xi[NIN], yo[NOUT];
#pragma unroll
                for (int j = 0; j < NIN; ++j) xi[j] = a.in[j][i];
                f(xi, yo);
#pragma unroll
                for (int o = 0; o < NOUT; ++o)
                    if (a.out[o]) a.out[o][i] = yo[o];
            }
        }
    } else {
        for (int64_t i = static_cast<int64_t>(blockIdx.x) * kMapThreads + threadIdx.x; i < n;
             i += static_cast<int64_t>(gridDim.x) * kMapThreads) {
            T xi[NIN], yo[NOUT];
#pragma unroll
            for (int j = 0; j < NIN; ++j) xi[j] = a.in[j][i];
            f(xi, yo);
#pragma unroll
            for (int o = 0; o < NOUT; ++o)
                if (a.out[o]) a.out[o][i] = yo[o];
        }
    }
}

// All non-null pointers packet-aligned?
template <typename T, int NIN, int NOUT>
inline bool map_aligned(const MapArgs<T, NIN, NOUT>& a) {
    for (int i = 0; i < NIN; ++i)
        if (!aligned_pack<T>(a.in[i])) return false;
    for (int o = 0; o < NOUT; ++o)
        if (a.out[o] && !aligned_pack<T>(a.out[o])) return false;
    return true;
}

// Launches the map; inputs must be non-null, outputs may be null (skipped).  Returns a cudaError_t.
// UNROLL_ = 0 picks the packets in flight per thread from the number of inputs; compute-heavy maps pass a
// smaller value to trade registers for resident warps.
template <typename T, int NIN, int NOUT, int UNROLL_ = 0, typename F>
inline int launch_map(const MapArgs<T, NIN, NOUT>& a, int64_t n, F f, int waves = 0) {
    (void)cudaGetLastError();
    constexpr int UNROLL = UNROLL_ > 0 ? UNROLL_ : ((NIN <= 1) ? 8 : (NIN == 2 ? 4 : 2));
    const int WAVES = waves > 0 ? waves : ((NIN + NOUT <= 3) ? 64 : 16);
    if (map_aligned(a)) {
        const int64_t tiles = ((n >> 2) + kMapThreads * UNROLL - 1) / (kMapThreads * UNROLL);
        KD_LAUNCH_W((map_kernel<T, NIN, NOUT, UNROLL, true, F>), WAVES, tiles > 0 ? tiles : 1, kMapThreads, 0, a, n, f);
    } else {
        KD_LAUNCH_W((map_kernel<T, NIN, NOUT, 1, false, F>), 16, (n + kMapThreads - 1) / kMapThreads, kMapThreads, 0, a, n,
                    f);
    }
    return launch_status();
}

// ---------------------------------------------------------------------------
// map + sum: out[0] = finish(sum_i f(in_0[i], ..., in_{NIN-1}[i])); finish 0: the sum, 1: sum * scale, 2: sum / scale
// (each applied in T after the double sum is narrowed).  Deterministic: every CTA owns an
// equal contiguous share, publishes one double, and the CTA that takes the last ticket folds them
// in index order.  `counter` must be zero on entry and is zero again on exit.
// ---------------------------------------------------------------------------
template <typename T, int NIN, bool VEC, typename F>
__global__ void __launch_bounds__(kMapThreads)
map_sum_kernel(MapArgs<T, NIN, 1> a, int64_t n, double* partials, unsigned int* counter, T scale, int finish, F f) {
    kd::pdl_prologue();
    __shared__ double sm[kMapThreads / 32];
    __shared__ bool last;
    constexpr int U = (NIN == 1) ? 8 : 4;
    constexpr int A = 4;
    T acc[A];
#pragma unroll
    for (int k = 0; k < A; ++k) acc[k] = T(0);
    if (VEC) {
        const int64_t n4 = n >> 2;
        const int64_t share = ((n4 + gridDim.x - 1) / gridDim.x + kMapThreads - 1) / kMapThreads * kMapThreads;
        const int64_t begin = static_cast<int64_t>(blockIdx.x) * share;
        const int64_t end = begin + share < n4 ? begin + share : n4;
        for (int64_t base = begin; base < end; base += static_cast<int64_t>(kMapThreads) * U) {
            Pack4<T> v[U][NIN];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t p = base + u * kMapThreads + threadIdx.x;
                if (p < end) {
#pragma unroll
                    for (int i = 0; i < NIN; ++i) v[u][i] = load4_stream(a.in[i] + 4 * p);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t p = base + u * kMapThreads + threadIdx.x;
                if (p < end) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        T xi[NIN];
#pragma unroll
                        for (int i = 0; i < NIN; ++i) xi[i] = v[u][i].v[k];
                        acc[k] += f(xi);
                    }
                }
            }
        }
        if (blockIdx.x == 0 && threadIdx.x < 4) {
            const int64_t i = (n4 << 2) + threadIdx.x;
            if (i < n) {
                T xi[NIN];
#pragma unroll
                for (int j = 0; j < NIN; ++j) xi[j] = a.in[j][i];
                acc[0] += f(xi);
            }
        }
    } else {
        for (int64_t i = static_cast<int64_t>(blockIdx.x) * kMapThreads + threadIdx.x; i < n;
             i += static_cast<int64_t>(gridDim.x) * kMapThreads) {
            T xi[NIN];
#pragma unroll
            for (int j = 0; j < NIN; ++j) xi[j] = a.in[j][i];
            acc[0] += f(xi);
        }
    }
    double s = 0.0;
#pragma unroll
    for (int k = 0; k < A; ++k) s += static_cast<double>(acc[k]);
    s = block_sum(s, sm);
    if (threadIdx.x == 0) partials[blockIdx.x] = s;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = (atomicAdd(counter, 1u) == gridDim.x - 1);
    __syncthreads();
    if (last) {
        __threadfence();
        double v = 0.0;
        for (unsigned i = threadIdx.x; i < gridDim.x; i += kMapThreads) v += __ldcg(partials + i);
        v = block_sum(v, sm);
        if (threadIdx.x == 0) {
            T r = static_cast<T>(v);
            if (finish == 1) r = r * scale;
            else if (finish == 2) r = r / scale;
            a.out[0][0] = r;
            *counter = 0u;
        }
    }
}

template <typename T, int NIN, typename F>
inline int launch_map_sum(const MapArgs<T, NIN, 1>& a, int64_t n, T scale, int finish, F f) {
    (void)cudaGetLastError();
    bool vec = true;
    for (int i = 0; i < NIN; ++i) vec = vec && aligned_pack<T>(a.in[i]);
    constexpr int U = (NIN == 1) ? 8 : 4;
    const int64_t tiles = vec ? ((n >> 2) + kMapThreads * U - 1) / (kMapThreads * U) : (n + kMapThreads - 1) / kMapThreads;
    const unsigned grid = vec ? grid_fit(map_sum_kernel<T, NIN, true, F>, kMapThreads, tiles > 0 ? tiles : 1)
                              : grid_fit(map_sum_kernel<T, NIN, false, F>, kMapThreads, tiles > 0 ? tiles : 1);
    double* partials = static_cast<double*>(scratch(grid * sizeof(double)));
    unsigned int* counter = counters(1);
    if (!partials || !counter) return static_cast<int>(cudaErrorMemoryAllocation);
    if (vec) (void)kd::launch(map_sum_kernel<T, NIN, true, F>, dim3(grid), kMapThreads, 0, a, n, partials, counter, scale, finish, f);
    else (void)kd::launch(map_sum_kernel<T, NIN, false, F>, dim3(grid), kMapThreads, 0, a, n, partials, counter, scale, finish, f);
    return launch_status();
}

}  // namespace kd
