// Shared device/host helpers for the sm_100a KeyDNN operator library.
//
// Everything in this library is HBM-bound: kernels are written around 16- and
// 32-byte global accesses, enough independent loads per thread to cover DRAM
// latency, and grids sized from the SM count and the measured occupancy of the
// device the call runs on.
#pragma once

#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <limits>
#include <mutex>
#include <unordered_map>

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
// A 4-element packet is one access: 16 bytes for float, 32 bytes for double / int64.
template <typename T> inline bool aligned_pack(const void* p) {
    return (reinterpret_cast<uintptr_t>(p) & (sizeof(T) * 4 - 1)) == 0;
}

// Grid for a grid-stride kernel: enough CTAs to fill every SM `per_sm` times,
// never more than the work available.
inline unsigned grid_for(int64_t work_items, int per_sm) {
    int64_t cap = static_cast<int64_t>(sm_count()) * per_sm;
    int64_t g = work_items < cap ? work_items : cap;
    return static_cast<unsigned>(g < 1 ? 1 : g);
}

// CTAs of `kernel` that one SM holds at once (cached per kernel).
template <typename K> inline int occupancy(K kernel, int threads, size_t smem = 0) {
    // kernels of one signature share this map: the key is the kernel's address mixed with the launch shape
    static std::unordered_map<uint64_t, int> cache;
    static std::mutex mu;
    const uint64_t key = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(kernel)) * 0x9E3779B97F4A7C15ull ^
                         (static_cast<uint64_t>(smem) << 12) ^ static_cast<uint64_t>(threads);
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, smem) != cudaSuccess || n < 1) n = 1;
    cache.emplace(key, n);
    return n;
}

// Grid for a grid-stride kernel: `waves` times what the machine holds at once (every SM
// holds as many CTAs of this kernel as fit), or fewer when there is less work.
//   waves = 1: all CTAs resident from start to end; for kernels whose CTAs split the work
//              evenly themselves and publish one partial each.
//   waves >> 1: pure streaming kernels; the hardware scheduler hands out the many small CTAs
//              as SMs free up, which evens out the last trips (measured on B200: element-wise
//              kernels gain 5% from 1 to 8 waves and 5% more up to 64; write-only fills peak
//              at 8-16 and collapse when a CTA has less than a few packets per thread).
constexpr int kStreamWaves = 8;
inline int stream_waves() { return kStreamWaves; }
template <typename K>
inline unsigned grid_fit(K kernel, int threads, int64_t work_ctas, size_t smem = 0, int waves = 1) {
    const int64_t cap = static_cast<int64_t>(sm_count()) * occupancy(kernel, threads, smem) * waves;
    const int64_t g = work_ctas < cap ? work_ctas : cap;
    return static_cast<unsigned>(g < 1 ? 1 : g);
}

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of the library opens with pdl_prologue(): it lets the next
// kernel of the stream be scheduled while this one is still running, then waits until everything the stream
// holds in front of this kernel has completed and its writes are visible.  A dependent kernel's CTAs are
// therefore already resident, parked at the wait, when the last CTA of its predecessor retires: launch latency
// and the ramp-up of a grid are hidden behind the tail of the kernel before it (the short reductions of this
// library spend 2-4 us of a 20-45 us run in ramp and tail).  Nothing is read or written before the wait, so
// stream order is kept exactly.  Launched without the attribute both instructions do nothing.
// ---------------------------------------------------------------------------
bool pdl_enabled();             // runtime.cu: on unless the environment sets KEYDNN_PDL=0
__device__ __forceinline__ void pdl_prologue() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, unsigned threads, size_t smem, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Launch with the CTAs of one grid column (gridDim.y) grouped into thread-block clusters of `cluster_y`: they are
// co-scheduled on one GPC, synchronise with the hardware cluster barrier and read each other's shared memory.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_cluster_y(void (*kernel)(KArgs...), dim3 grid, unsigned threads, unsigned cluster_y, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream();
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = cluster_y;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define KD_LAUNCH(KERNEL, WORK, THREADS, SMEM, ...)                                                           \
    do {                                                                                                      \
        auto kd_fn_ = (KERNEL);                                                                               \
        (void)kd::launch(kd_fn_, dim3(kd::grid_fit(kd_fn_, (THREADS), (WORK), (SMEM), kd::stream_waves())), (THREADS), \
                         (SMEM), __VA_ARGS__);                                                                \
    } while (0)

// Same with an explicit number of waves.
#define KD_LAUNCH_W(KERNEL, WAVES, WORK, THREADS, SMEM, ...)                                                  \
    do {                                                                                                      \
        auto kd_fn_ = (KERNEL);                                                                               \
        (void)kd::launch(kd_fn_, dim3(kd::grid_fit(kd_fn_, (THREADS), (WORK), (SMEM), (WAVES))), (THREADS), (SMEM), __VA_ARGS__); \
    } while (0)

// Same with exactly one resident wave.
#define KD_LAUNCH1(KERNEL, WORK, THREADS, SMEM, ...)                                                          \
    do {                                                                                                      \
        auto kd_fn_ = (KERNEL);                                                                               \
        (void)kd::launch(kd_fn_, dim3(kd::grid_fit(kd_fn_, (THREADS), (WORK), (SMEM), 1)), (THREADS), (SMEM), __VA_ARGS__); \
    } while (0)

// Separately rounded IEEE operations: never contracted into an FMA, whatever -fmad says.
template <typename T> struct Rn;
template <> struct Rn<float> {
    static __device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
    static __device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
    static __device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
};
template <> struct Rn<double> {
    static __device__ __forceinline__ double mul(double a, double b) { return __dmul_rn(a, b); }
    static __device__ __forceinline__ double add(double a, double b) { return __dadd_rn(a, b); }
    static __device__ __forceinline__ double sub(double a, double b) { return __dsub_rn(a, b); }
};

// ---------------------------------------------------------------------------
// 4-element packets: one 16-byte access for float, one 32-byte access (256-bit
// ld/st, sm_100) for double and int64, so that a warp always touches whole,
// contiguous sectors with a single instruction.
// ---------------------------------------------------------------------------
template <typename T> struct Pack4 { T v[4]; };

template <typename T> __device__ __forceinline__ Pack4<T> load4(const T* p);
template <> __device__ __forceinline__ Pack4<float> load4<float>(const float* p) {
    float4 t = __ldg(reinterpret_cast<const float4*>(p));
    Pack4<float> r; r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w; return r;
}
template <> __device__ __forceinline__ Pack4<double> load4<double>(const double* p) {
    Pack4<double> r;
    asm volatile("ld.global.nc.v4.f64 {%0,%1,%2,%3}, [%4];"
                 : "=d"(r.v[0]), "=d"(r.v[1]), "=d"(r.v[2]), "=d"(r.v[3]) : "l"(p));
    return r;
}
template <> __device__ __forceinline__ Pack4<long long> load4<long long>(const long long* p) {
    Pack4<long long> r;
    asm volatile("ld.global.nc.v4.s64 {%0,%1,%2,%3}, [%4];"
                 : "=l"(r.v[0]), "=l"(r.v[1]), "=l"(r.v[2]), "=l"(r.v[3]) : "l"(p));
    return r;
}

// Streaming loads: data that is touched once (evict-first in L1/L2).
template <typename T> __device__ __forceinline__ Pack4<T> load4_stream(const T* p);
template <> __device__ __forceinline__ Pack4<float> load4_stream<float>(const float* p) {
    float4 t = __ldcs(reinterpret_cast<const float4*>(p));
    Pack4<float> r; r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w; return r;
}
template <> __device__ __forceinline__ Pack4<double> load4_stream<double>(const double* p) {
    Pack4<double> r;
    asm volatile("ld.global.cs.v4.f64 {%0,%1,%2,%3}, [%4];"
                 : "=d"(r.v[0]), "=d"(r.v[1]), "=d"(r.v[2]), "=d"(r.v[3]) : "l"(p));
    return r;
}
template <> __device__ __forceinline__ Pack4<long long> load4_stream<long long>(const long long* p) {
    Pack4<long long> r;
    asm volatile("ld.global.cs.v4.s64 {%0,%1,%2,%3}, [%4];"
                 : "=l"(r.v[0]), "=l"(r.v[1]), "=l"(r.v[2]), "=l"(r.v[3]) : "l"(p));
    return r;
}

template <typename T> __device__ __forceinline__ void store4(T* p, const Pack4<T>& r);
template <> __device__ __forceinline__ void store4<float>(float* p, const Pack4<float>& r) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(r.v[0], r.v[1], r.v[2], r.v[3]));
}
template <> __device__ __forceinline__ void store4<double>(double* p, const Pack4<double>& r) {
    asm volatile("st.global.cs.v4.f64 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "d"(r.v[0]), "d"(r.v[1]), "d"(r.v[2]), "d"(r.v[3]) : "memory");
}
template <> __device__ __forceinline__ void store4<long long>(long long* p, const Pack4<long long>& r) {
    asm volatile("st.global.cs.v4.s64 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "l"(r.v[0]), "l"(r.v[1]), "l"(r.v[2]), "l"(r.v[3]) : "memory");
}

// 8 contiguous elements of one row owned by one thread.  For float this is a single
// 256-bit access, so a warp instruction covers 1 KiB of whole sectors instead of
// every other half sector; for double it is two 256-bit accesses.
template <typename T> struct Row8 { T v[8]; };
template <typename T> inline bool aligned_row8(const void* p) {
    return (reinterpret_cast<uintptr_t>(p) & 31u) == 0;
}

template <typename T> __device__ __forceinline__ Row8<T> load8(const T* p);          // read-only, cached
template <typename T> __device__ __forceinline__ Row8<T> load8_stream(const T* p);   // touched once
template <typename T> __device__ __forceinline__ void store8(T* p, const Row8<T>& r);

template <> __device__ __forceinline__ Row8<float> load8<float>(const float* p) {
    Row8<float> r;
    asm volatile("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]),
                   "=f"(r.v[7]) : "l"(p));
    return r;
}
template <> __device__ __forceinline__ Row8<float> load8_stream<float>(const float* p) {
    Row8<float> r;
    asm volatile("ld.global.cs.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]),
                   "=f"(r.v[7]) : "l"(p));
    return r;
}
template <> __device__ __forceinline__ void store8<float>(float* p, const Row8<float>& r) {
    asm volatile("st.global.cs.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :: "l"(p), "f"(r.v[0]), "f"(r.v[1]), "f"(r.v[2]), "f"(r.v[3]), "f"(r.v[4]), "f"(r.v[5]), "f"(r.v[6]),
                    "f"(r.v[7]) : "memory");
}
template <> __device__ __forceinline__ Row8<double> load8<double>(const double* p) {
    const Pack4<double> a = load4(p), b = load4(p + 4);
    Row8<double> r;
#pragma unroll
    for (int k = 0; k < 4; ++k) { r.v[k] = a.v[k]; r.v[4 + k] = b.v[k]; }
    return r;
}
template <> __device__ __forceinline__ Row8<double> load8_stream<double>(const double* p) {
    const Pack4<double> a = load4_stream(p), b = load4_stream(p + 4);
    Row8<double> r;
#pragma unroll
    for (int k = 0; k < 4; ++k) { r.v[k] = a.v[k]; r.v[4 + k] = b.v[k]; }
    return r;
}
template <> __device__ __forceinline__ void store8<double>(double* p, const Row8<double>& r) {
    Pack4<double> a, b;
#pragma unroll
    for (int k = 0; k < 4; ++k) { a.v[k] = r.v[k]; b.v[k] = r.v[4 + k]; }
    store4(p, a);
    store4(p + 4, b);
}

template <typename T> __device__ __forceinline__ T neg_inf();
template <> __device__ __forceinline__ float neg_inf<float>() { return __int_as_float(0xff800000); }
template <> __device__ __forceinline__ double neg_inf<double>() {
    return __longlong_as_double(static_cast<long long>(0xfff0000000000000ULL));
}

// ---------------------------------------------------------------------------
// Division of a 31-bit index by a launch-invariant divisor: one multiply-high and
// one shift instead of the ~20 (32-bit) or ~100 (64-bit) instruction division
// sequence.  q = floor(n / d) for every 0 <= n < 2^31, 1 <= d < 2^31.
// ---------------------------------------------------------------------------
struct FastDiv {
    unsigned d, mul, shr;
    FastDiv() : d(1), mul(0), shr(0) {}
    explicit FastDiv(unsigned divisor) : d(divisor), mul(0), shr(0) {
        if (d > 1) {
            unsigned lg = 0;
            while ((1ull << lg) < d) ++lg;                 // ceil(log2(d))
            const unsigned p = 31 + lg;
            mul = static_cast<unsigned>(((1ull << p) + d - 1) / d);
            shr = p - 32;
        }
    }
    __host__ __device__ __forceinline__ unsigned div(unsigned n) const {
#ifdef __CUDA_ARCH__
        return d == 1 ? n : (__umulhi(n, mul) >> shr);
#else
        return d == 1 ? n : static_cast<unsigned>((static_cast<unsigned long long>(n) * mul) >> 32) >> shr;
#endif
    }
    __host__ __device__ __forceinline__ void divmod(unsigned n, unsigned& q, unsigned& r) const {
        q = div(n);
        r = n - q * d;
    }
};

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
