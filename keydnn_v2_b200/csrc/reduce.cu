// Reductions over flat vectors and 2-D matrices, their gradient broadcast / mask
// kernels, and the N-D un-broadcast sum.
//
// Reference kernels replaced (KeyDNNV2CudaNative/keydnn_reduce_cuda.cu):
//   sum_all_kernel :58-70          one atomicAdd per element onto one address
//   scale_scalar_kernel :98-101    <<<1,1>>> mean scale
//   fill_with_scalar_kernel :122-132
//   max_axis2d_forward_axis{1,0} :156-205   one thread per row / per column, serial
//   max_axis2d_backward_axis{1,0} :235-263  scatter onto a caller-zeroed matrix
//   sum_axis2d_forward_axis{1,0} :292-323   one thread per row / per column, serial
//   sum_axis2d_backward_axis{1,0} :355-381  int64 div/mod per element
//   sum_to_shape_kernel :418-458   one atomicAdd per input element, 4 cudaMalloc per call
//
// Design: every forward reduction is a streaming pass with 16-byte loads and
// per-thread partials, then warp shuffles, then a block tree in shared memory.
// Cross-CTA combination is deterministic: each CTA publishes its partial to a
// scratch array and the last CTA to arrive (an atomic ticket) folds the partials
// in a fixed order; the counter is returned to zero for the next call.  Sums are
// accumulated in the element type per thread (a few dozen terms) and combined in
// double.  Maxima carry the position of the first occurrence through every merge.
#include "common.cuh"

#include <cooperative_groups.h>

#include <mutex>

namespace {

namespace cg = cooperative_groups;

using kd::ArgMax;
using kd::Pack4;

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

template <typename T> __device__ __forceinline__ T ld_cg(const T* p) { return __ldcg(p); }

// ---------------------------------------------------------------------------
// Full reductions: sum / mean / max over all elements
// ---------------------------------------------------------------------------
// Folds the partials published by all CTAs; runs in the last CTA only.
__device__ __forceinline__ bool take_ticket(unsigned int* counter, unsigned int expected) {
    __shared__ bool last;
    __threadfence();            // publish this thread's partials device-wide
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(counter, 1u);
        last = (t == expected - 1);
    }
    __syncthreads();
    if (last) __threadfence();
    return last;
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads)
sum_all_kernel(const T* __restrict__ x, int64_t n, double* partials, unsigned int* counter, T* out, T scale,
               bool apply_scale) {
    kd::pdl_prologue();
    __shared__ double sm[kWarps];
    constexpr int U = 8;     // packets in flight per thread and trip
    constexpr int A = 8;     // independent accumulators
    T acc[A];
#pragma unroll
    for (int k = 0; k < A; ++k) acc[k] = T(0);
    if (VEC) {
        // every CTA owns an equal, contiguous share of the packets (a multiple of the CTA width)
        const int64_t n4 = n >> 2;
        const int64_t share = ((n4 + gridDim.x - 1) / gridDim.x + kThreads - 1) / kThreads * kThreads;
        const int64_t begin = static_cast<int64_t>(blockIdx.x) * share;
        const int64_t end = begin + share < n4 ? begin + share : n4;
        const int64_t tile = static_cast<int64_t>(kThreads) * U;
        for (int64_t base = begin; base < end; base += tile) {
            Pack4<T> v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t p = base + u * kThreads + threadIdx.x;
                if (p < end) v[u] = kd::load4_stream(x + 4 * p);
                else v[u].v[0] = v[u].v[1] = v[u].v[2] = v[u].v[3] = T(0);
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[(4 * u + k) % A] += v[u].v[k];
        }
        if (blockIdx.x == 0 && threadIdx.x < 4) {
            const int64_t i = (n4 << 2) + threadIdx.x;
            if (i < n) acc[0] += x[i];
        }
    } else {
        for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n;
             i += static_cast<int64_t>(gridDim.x) * kThreads)
            acc[0] += x[i];
    }
    double s = 0.0;
#pragma unroll
    for (int k = 0; k < A; ++k) s += static_cast<double>(acc[k]);
    s = kd::block_sum(s, sm);
    if (threadIdx.x == 0) partials[blockIdx.x] = s;
    if (take_ticket(counter, gridDim.x)) {
        double v = 0.0;
        for (unsigned i = threadIdx.x; i < gridDim.x; i += kThreads) v += ld_cg(partials + i);
        v = kd::block_sum(v, sm);
        if (threadIdx.x == 0) {
            T r = static_cast<T>(v);
            if (apply_scale) r = r * scale;
            out[0] = r;
            *counter = 0u;
        }
    }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads)
max_all_kernel(const T* __restrict__ x, int64_t n, T* pval, long long* pidx, unsigned int* counter, T* out,
               long long* out_idx) {
    kd::pdl_prologue();
    __shared__ T smv[kWarps];
    __shared__ long long smi[kWarps];
    ArgMax<T> a = kd::argmax_init<T>();
    if (VEC) {
        constexpr int U = 4;
        const int64_t n4 = n >> 2;
        const int64_t share = ((n4 + gridDim.x - 1) / gridDim.x + kThreads - 1) / kThreads * kThreads;
        const int64_t begin = static_cast<int64_t>(blockIdx.x) * share;
        const int64_t end = begin + share < n4 ? begin + share : n4;
        for (int64_t base = begin; base < end; base += static_cast<int64_t>(kThreads) * U) {
            Pack4<T> v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t p = base + u * kThreads + threadIdx.x;
                if (p < end) v[u] = kd::load4_stream(x + 4 * p);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t p = base + u * kThreads + threadIdx.x;
                if (p < end) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) kd::argmax_step(a, v[u].v[k], 4 * p + k);
                }
            }
        }
        if (blockIdx.x == 0 && threadIdx.x < 4) {
            const int64_t i = (n4 << 2) + threadIdx.x;
            if (i < n) kd::argmax_merge(a, x[i], static_cast<long long>(i));
        }
    } else {
        for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n;
             i += static_cast<int64_t>(gridDim.x) * kThreads)
            kd::argmax_step(a, x[i], static_cast<long long>(i));
    }
    auto block_reduce = [&](ArgMax<T> v) {
        v = kd::warp_argmax(v);
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        if (lane == 0) { smv[warp] = v.val; smi[warp] = v.idx; }
        __syncthreads();
        if (warp == 0) {
            ArgMax<T> w = kd::argmax_init<T>();
            if (lane < kWarps) { w.val = smv[lane]; w.idx = smi[lane]; }
            v = kd::warp_argmax(w);
        }
        __syncthreads();
        return v;
    };
    a = block_reduce(a);
    if (threadIdx.x == 0) { pval[blockIdx.x] = a.val; pidx[blockIdx.x] = a.idx; }
    if (take_ticket(counter, gridDim.x)) {
        ArgMax<T> v = kd::argmax_init<T>();
        for (unsigned i = threadIdx.x; i < gridDim.x; i += kThreads)
            kd::argmax_merge(v, ld_cg(pval + i), ld_cg(pidx + i));
        v = block_reduce(v);
        if (threadIdx.x == 0) {
            out[0] = v.val;
            out_idx[0] = (v.idx == kd::kNoIndex) ? 0 : v.idx;
            *counter = 0u;
        }
    }
}

// Ticket for kernels in which only thread 0 of a CTA publishes a partial: thread 0's store is ordered before its
// own acq_rel atomic (release), the CTA that draws the last ticket acquires with the same atomic, and the barrier
// behind it hands that ordering to the other threads of the CTA (which read the partials with ld.cg, from L2).
// No fence is executed by the other 255 threads.
__device__ __forceinline__ bool take_ticket_t0(unsigned int* counter, unsigned int expected) {
    __shared__ bool last;
    if (threadIdx.x == 0) {
        unsigned int t;
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(t) : "l"(counter) : "memory");
        last = (t == expected - 1);
    }
    __syncthreads();
    return last;
}

// Full reductions over aligned data: many short CTAs (one per tile of Tile<T>::kPackets packets, every thread with
// Tile<T>::U independent 16 / 32-byte loads in flight), handed out by the hardware scheduler as SMs free up, each
// leaving one partial; the CTA that draws the last ticket folds the partials with all its loads issued at once.
// Measured on B200 against one resident wave of grid-stride CTAs (fp64, 134 MB): 22.6 us instead of 25.2 us;
// the streaming part alone runs at the copy peak (20.7 us), the ticket and the fold are the remaining 2 us.
// A trip is 32 KiB per CTA (measured best on B200 for both element sizes): 8 packets of 16 bytes per thread for
// float, 4 packets of 32 bytes for double.
template <typename T> struct Tile {
    static constexpr int U = 128 / static_cast<int>(sizeof(T) * 4);
    static constexpr int kPackets = kThreads * U;
};
constexpr int kFoldBatch = 16;                       // partials per thread and fold round: 4096 per round
constexpr int kMaxFoldBatch = 8;                     // the arg-max fold holds a value and a position per partial
constexpr unsigned kMaxTileGrid = 2 * kFoldBatch * kThreads;   // at most two fold rounds

// U: packets per thread and trip.  SINGLE: every CTA makes exactly one trip (per_cta == kThreads * U): no loop
// around the loads.
template <typename T, int U, bool SINGLE>
__global__ void __launch_bounds__(kThreads)
sum_all_tiles_kernel(const T* __restrict__ x, int64_t n, int64_t per_cta, double* partials, unsigned int* counter, T* out,
                     T scale, bool apply_scale) {
    kd::pdl_prologue();
    __shared__ double sm[kWarps];
    const int64_t n4 = n >> 2;
    const int64_t begin = static_cast<int64_t>(blockIdx.x) * (SINGLE ? static_cast<int64_t>(kThreads) * U : per_cta);
    const int64_t end = SINGLE ? n4 : (begin + per_cta < n4 ? begin + per_cta : n4);
    double s = 0.0;
    for (int64_t base = begin; base < end; base += static_cast<int64_t>(kThreads) * U) {
        Pack4<T> v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t p = base + u * kThreads + threadIdx.x;
            if (p < end) v[u] = kd::load4_stream(x + 4 * p);
            else v[u].v[0] = v[u].v[1] = v[u].v[2] = v[u].v[3] = T(0);
        }
        T a[4] = {T(0), T(0), T(0), T(0)};          // U terms each in the element type, then double
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int k = 0; k < 4; ++k) a[k] += v[u].v[k];
        s += (static_cast<double>(a[0]) + static_cast<double>(a[1])) + (static_cast<double>(a[2]) + static_cast<double>(a[3]));
        if (SINGLE) break;
    }
    if (blockIdx.x == 0 && threadIdx.x < 4) {
        const int64_t i = (n4 << 2) + threadIdx.x;
        if (i < n) s += static_cast<double>(x[i]);
    }
    s = kd::block_sum(s, sm);
    if (threadIdx.x == 0) partials[blockIdx.x] = s;
    if (take_ticket_t0(counter, gridDim.x)) {
        double v = 0.0;
        for (unsigned base = 0; base < gridDim.x; base += kFoldBatch * kThreads) {
            double t[kFoldBatch];
#pragma unroll
            for (int k = 0; k < kFoldBatch; ++k) {
                const unsigned i = base + k * kThreads + threadIdx.x;
                t[k] = i < gridDim.x ? ld_cg(partials + i) : 0.0;
            }
#pragma unroll
            for (int k = 0; k < kFoldBatch; ++k) v += t[k];
        }
        v = kd::block_sum(v, sm);
        if (threadIdx.x == 0) {
            T r = static_cast<T>(v);
            if (apply_scale) r = r * scale;
            out[0] = r;
            *counter = 0u;
        }
    }
}

template <typename T, int U, bool SINGLE>
__global__ void __launch_bounds__(kThreads)
max_all_tiles_kernel(const T* __restrict__ x, int64_t n, int64_t per_cta, T* pval, long long* pidx, unsigned int* counter,
                     T* out, long long* out_idx) {
    kd::pdl_prologue();
    __shared__ T smv[kWarps];
    __shared__ long long smi[kWarps];
    const int64_t n4 = n >> 2;
    const int64_t begin = static_cast<int64_t>(blockIdx.x) * (SINGLE ? static_cast<int64_t>(kThreads) * U : per_cta);
    const int64_t end = SINGLE ? n4 : (begin + per_cta < n4 ? begin + per_cta : n4);
    // inside a trip the position is a 32-bit offset from the trip's first element; widened once per trip
    ArgMax<T> a = kd::argmax_init<T>();
    for (int64_t base = begin; base < end; base += static_cast<int64_t>(kThreads) * U) {
        Pack4<T> v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t p = base + u * kThreads + threadIdx.x;
            if (p < end) v[u] = kd::load4_stream(x + 4 * p);
            else v[u].v[0] = v[u].v[1] = v[u].v[2] = v[u].v[3] = kd::neg_inf<T>();
        }
        T best = kd::neg_inf<T>();
        int where = -1;
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (v[u].v[k] > best) { best = v[u].v[k]; where = 4 * (u * kThreads + static_cast<int>(threadIdx.x)) + k; }
        if (where >= 0) kd::argmax_step(a, best, 4 * base + where);      // trips come in increasing position order
        if (SINGLE) break;
    }
    if (blockIdx.x == 0 && threadIdx.x < 4) {
        const int64_t i = (n4 << 2) + threadIdx.x;
        if (i < n) kd::argmax_merge(a, x[i], static_cast<long long>(i));
    }
    auto block_reduce = [&](ArgMax<T> v) {
        v = kd::warp_argmax(v);
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        if (lane == 0) { smv[warp] = v.val; smi[warp] = v.idx; }
        __syncthreads();
        if (warp == 0) {
            ArgMax<T> w = kd::argmax_init<T>();
            if (lane < kWarps) { w.val = smv[lane]; w.idx = smi[lane]; }
            v = kd::warp_argmax(w);
        }
        __syncthreads();
        return v;
    };
    a = block_reduce(a);
    if (threadIdx.x == 0) { pval[blockIdx.x] = a.val; pidx[blockIdx.x] = a.idx; }
    if (take_ticket_t0(counter, gridDim.x)) {
        ArgMax<T> v = kd::argmax_init<T>();
        for (unsigned base = 0; base < gridDim.x; base += kMaxFoldBatch * kThreads) {
            T tv[kMaxFoldBatch];
            long long ti[kMaxFoldBatch];
#pragma unroll
            for (int k = 0; k < kMaxFoldBatch; ++k) {
                const unsigned i = base + k * kThreads + threadIdx.x;
                tv[k] = i < gridDim.x ? ld_cg(pval + i) : kd::neg_inf<T>();
                ti[k] = i < gridDim.x ? ld_cg(pidx + i) : kd::kNoIndex;
            }
#pragma unroll
            for (int k = 0; k < kMaxFoldBatch; ++k) kd::argmax_merge(v, tv[k], ti[k]);
        }
        v = block_reduce(v);
        if (threadIdx.x == 0) {
            out[0] = v.val;
            out_idx[0] = (v.idx == kd::kNoIndex) ? 0 : v.idx;
            *counter = 0u;
        }
    }
}

// Packets per CTA for the tile kernels: one trip of Tile<T>::kPackets where that keeps the grid within two fold rounds,
// more trips (a multiple of the trip size) for larger inputs.
inline int64_t tile_packets_per_cta(int64_t n4, int trip) {
    int64_t per = trip;
    const int64_t need = (n4 + kMaxTileGrid - 1) / kMaxTileGrid;
    if (need > per) per = (need + trip - 1) / trip * trip;
    return per;
}

// ---------------------------------------------------------------------------
// Row reductions (axis = 1): y[r] = reduce over c of x[r, c]
// ---------------------------------------------------------------------------
// TPR threads cooperate on a row (32 = one warp, 256 = the CTA).
template <typename T, int TPR, bool VEC>
__global__ void __launch_bounds__(kThreads)
sum_rows_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int cols, T scale, bool apply_scale) {
    kd::pdl_prologue();
    __shared__ double sm[kWarps];
    constexpr int RPB = kThreads / TPR;              // rows per CTA trip
    const int t = threadIdx.x % TPR;
    const int sub = threadIdx.x / TPR;
    for (int64_t r0 = static_cast<int64_t>(blockIdx.x) * RPB; r0 < rows; r0 += static_cast<int64_t>(gridDim.x) * RPB) {
        const int64_t r = r0 + sub;
        T a0 = T(0), a1 = T(0), a2 = T(0), a3 = T(0);
        if (r < rows) {
            const T* src = x + r * cols;
            if (VEC) {
                const int c4 = cols >> 2;
                int p = t;
                for (; p + 3 * TPR < c4; p += 4 * TPR) {
                    const Pack4<T> v0 = kd::load4_stream(src + 4 * p);
                    const Pack4<T> v1 = kd::load4_stream(src + 4 * (p + TPR));
                    const Pack4<T> v2 = kd::load4_stream(src + 4 * (p + 2 * TPR));
                    const Pack4<T> v3 = kd::load4_stream(src + 4 * (p + 3 * TPR));
                    a0 += v0.v[0]; a1 += v0.v[1]; a2 += v0.v[2]; a3 += v0.v[3];
                    a0 += v1.v[0]; a1 += v1.v[1]; a2 += v1.v[2]; a3 += v1.v[3];
                    a0 += v2.v[0]; a1 += v2.v[1]; a2 += v2.v[2]; a3 += v2.v[3];
                    a0 += v3.v[0]; a1 += v3.v[1]; a2 += v3.v[2]; a3 += v3.v[3];
                }
                for (; p < c4; p += TPR) {
                    const Pack4<T> v0 = kd::load4_stream(src + 4 * p);
                    a0 += v0.v[0]; a1 += v0.v[1]; a2 += v0.v[2]; a3 += v0.v[3];
                }
            } else {
                for (int c = t; c < cols; c += TPR) a0 += src[c];
            }
        }
        double s = (static_cast<double>(a0) + static_cast<double>(a1)) +
                   (static_cast<double>(a2) + static_cast<double>(a3));
        if (TPR == 32) {
            s = kd::warp_sum(s);
        } else {
            s = kd::block_sum(s, sm);
        }
        if (t == 0 && r < rows) {
            T out = static_cast<T>(s);
            if (apply_scale) out = out * scale;
            y[r] = out;
        }
    }
}

template <typename T, int TPR, bool VEC>
__global__ void __launch_bounds__(kThreads)
max_rows_kernel(const T* __restrict__ x, T* __restrict__ y, long long* __restrict__ idx, int64_t rows, int cols) {
    kd::pdl_prologue();
    __shared__ T smv[kWarps];
    __shared__ long long smi[kWarps];
    constexpr int RPB = kThreads / TPR;
    const int t = threadIdx.x % TPR;
    const int sub = threadIdx.x / TPR;
    for (int64_t r0 = static_cast<int64_t>(blockIdx.x) * RPB; r0 < rows; r0 += static_cast<int64_t>(gridDim.x) * RPB) {
        const int64_t r = r0 + sub;
        ArgMax<T> a = kd::argmax_init<T>();
        if (r < rows) {
            const T* src = x + r * cols;
            if (VEC) {
                const int c4 = cols >> 2;
                int p = t;
                for (; p + 3 * TPR < c4; p += 4 * TPR) {
                    Pack4<T> v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) v[u] = kd::load4_stream(src + 4 * (p + u * TPR));
#pragma unroll
                    for (int u = 0; u < 4; ++u)
#pragma unroll
                        for (int k = 0; k < 4; ++k) kd::argmax_step(a, v[u].v[k], 4 * (p + u * TPR) + k);
                }
                for (; p < c4; p += TPR) {
                    const Pack4<T> v0 = kd::load4_stream(src + 4 * p);
#pragma unroll
                    for (int k = 0; k < 4; ++k) kd::argmax_step(a, v0.v[k], 4 * p + k);
                }
            } else {
                for (int c = t; c < cols; c += TPR) kd::argmax_step(a, src[c], static_cast<long long>(c));
            }
        }
        a = kd::warp_argmax(a);
        if (TPR != 32) {
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
            if (lane == 0) { smv[warp] = a.val; smi[warp] = a.idx; }
            __syncthreads();
            if (warp == 0) {
                ArgMax<T> w = kd::argmax_init<T>();
                if (lane < kWarps) { w.val = smv[lane]; w.idx = smi[lane]; }
                a = kd::warp_argmax(w);
            }
            __syncthreads();
        }
        if (t == 0 && r < rows) {
            y[r] = a.val;
            idx[r] = (a.idx == kd::kNoIndex) ? 0 : a.idx;
        }
    }
}

// ---------------------------------------------------------------------------
// Column reductions (axis = 0): y[c] = reduce over r of x[r, c]
// ---------------------------------------------------------------------------
// A CTA is 32 lanes x 8 row phases and owns a tile of 32*V columns by `rch`
// rows.  Lanes read V adjacent columns (16 bytes when V = 4), so a warp reads a
// contiguous 512-byte (f32) or 1-KiB (f64) piece of a row.  Each tile leaves one
// partial per column in scratch; the last tile of a column stripe to finish folds
// the stripe's partials in row order.
template <typename T, int V> struct ColLoad {
    static __device__ __forceinline__ void get(const T* p, T* out) {
        if (V == 8) {
            const kd::Row8<T> v = kd::load8_stream(p);
#pragma unroll
            for (int k = 0; k < 8; ++k) out[k] = v.v[k];
        } else if (V == 4) {
            const Pack4<T> v = kd::load4_stream(p);
#pragma unroll
            for (int k = 0; k < 4; ++k) out[k] = v.v[k];
        } else {
            out[0] = *p;
        }
    }
};

// Columns per lane: 32 bytes when the matrix allows it (8 floats / 4 doubles, one
// 256-bit load, 1 KiB contiguous per warp and row), else one packet, else one element.
template <typename T> inline int col_vector_width(const void* x, int cols) {
    constexpr int kWide = 32 / static_cast<int>(sizeof(T));
    if ((reinterpret_cast<uintptr_t>(x) & 31u) == 0 && cols % kWide == 0) return kWide;
    if (kd::aligned_pack<T>(x) && cols % 4 == 0) return 4;
    return 1;
}

template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
sum_cols_kernel(const T* __restrict__ x, T* __restrict__ y, int rows, int cols, int rch, T* partials,
                unsigned int* counters, T scale, bool apply_scale) {
    kd::pdl_prologue();
    __shared__ T sm[kWarps][32 * V + 1];
    const int lane = threadIdx.x & 31, phase = threadIdx.x >> 5;
    const int stripe = blockIdx.x;                    // column stripe
    const int chunk = blockIdx.y;                     // row chunk
    const int nchunks = gridDim.y;
    const int c0 = (stripe * 32 + lane) * V;
    const int r_begin = chunk * rch;
    const int r_end = min(rows, r_begin + rch);
    T acc[V];
#pragma unroll
    for (int k = 0; k < V; ++k) acc[k] = T(0);
    if (c0 < cols) {
        const T* src = x + c0;
        int r = r_begin + phase;
        for (; r + 3 * kWarps < r_end; r += 4 * kWarps) {
            T v[4][V];
#pragma unroll
            for (int u = 0; u < 4; ++u) ColLoad<T, V>::get(src + static_cast<int64_t>(r + u * kWarps) * cols, v[u]);
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int k = 0; k < V; ++k) acc[k] += v[u][k];
        }
        for (; r < r_end; r += kWarps) {
            T v[V];
            ColLoad<T, V>::get(src + static_cast<int64_t>(r) * cols, v);
#pragma unroll
            for (int k = 0; k < V; ++k) acc[k] += v[k];
        }
    }
#pragma unroll
    for (int k = 0; k < V; ++k) sm[phase][lane * V + k] = acc[k];
    __syncthreads();
    // fold the 8 row phases; thread j (< 32*V) owns column stripe*32*V + j
    const int ncol_tile = 32 * V;
    for (int j = threadIdx.x; j < ncol_tile; j += kThreads) {
        const int c = stripe * ncol_tile + j;
        if (c < cols) {
            double s = 0.0;
#pragma unroll
            for (int p = 0; p < kWarps; ++p) s += static_cast<double>(sm[p][j]);
            if (nchunks == 1) {
                T out = static_cast<T>(s);
                if (apply_scale) out = out * scale;
                y[c] = out;
            } else {
                partials[static_cast<int64_t>(chunk) * cols + c] = static_cast<T>(s);
            }
        }
    }
    if (nchunks == 1) return;
    if (take_ticket(counters + stripe, nchunks)) {
        for (int j = threadIdx.x; j < ncol_tile; j += kThreads) {
            const int c = stripe * ncol_tile + j;
            if (c < cols) {
                double s = 0.0;
                for (int q = 0; q < nchunks; ++q) s += static_cast<double>(ld_cg(partials + static_cast<int64_t>(q) * cols + c));
                T out = static_cast<T>(s);
                if (apply_scale) out = out * scale;
                y[c] = out;
            }
        }
        if (threadIdx.x == 0) counters[stripe] = 0u;
    }
}

template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
max_cols_kernel(const T* __restrict__ x, T* __restrict__ y, long long* __restrict__ idx, int rows, int cols, int rch,
                T* pval, int* pidx, unsigned int* counters) {
    kd::pdl_prologue();
    __shared__ T smv[kWarps][32 * V + 1];
    __shared__ int smi[kWarps][32 * V + 1];
    constexpr int kNone = std::numeric_limits<int>::max();
    const int lane = threadIdx.x & 31, phase = threadIdx.x >> 5;
    const int stripe = blockIdx.x, chunk = blockIdx.y, nchunks = gridDim.y;
    const int c0 = (stripe * 32 + lane) * V;
    const int r_begin = chunk * rch;
    const int r_end = min(rows, r_begin + rch);
    T best[V];
    int brow[V];
#pragma unroll
    for (int k = 0; k < V; ++k) { best[k] = kd::neg_inf<T>(); brow[k] = kNone; }
    if (c0 < cols) {
        const T* src = x + c0;
        int r = r_begin + phase;
        for (; r + 3 * kWarps < r_end; r += 4 * kWarps) {
            T v[4][V];
#pragma unroll
            for (int u = 0; u < 4; ++u) ColLoad<T, V>::get(src + static_cast<int64_t>(r + u * kWarps) * cols, v[u]);
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int k = 0; k < V; ++k)
                    if (v[u][k] > best[k]) { best[k] = v[u][k]; brow[k] = r + u * kWarps; }
        }
        for (; r < r_end; r += kWarps) {
            T v[V];
            ColLoad<T, V>::get(src + static_cast<int64_t>(r) * cols, v);
#pragma unroll
            for (int k = 0; k < V; ++k)
                if (v[k] > best[k]) { best[k] = v[k]; brow[k] = r; }
        }
    }
#pragma unroll
    for (int k = 0; k < V; ++k) { smv[phase][lane * V + k] = best[k]; smi[phase][lane * V + k] = brow[k]; }
    __syncthreads();
    const int ncol_tile = 32 * V;
    for (int j = threadIdx.x; j < ncol_tile; j += kThreads) {
        const int c = stripe * ncol_tile + j;
        if (c < cols) {
            T bv = kd::neg_inf<T>();
            int bi = kNone;
#pragma unroll
            for (int p = 0; p < kWarps; ++p) {
                const T v = smv[p][j];
                const int i = smi[p][j];
                if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
            }
            if (nchunks == 1) {
                y[c] = bv;
                idx[c] = (bi == kNone) ? 0 : bi;
            } else {
                pval[static_cast<int64_t>(chunk) * cols + c] = bv;
                pidx[static_cast<int64_t>(chunk) * cols + c] = bi;
            }
        }
    }
    if (nchunks == 1) return;
    if (take_ticket(counters + stripe, nchunks)) {
        for (int j = threadIdx.x; j < ncol_tile; j += kThreads) {
            const int c = stripe * ncol_tile + j;
            if (c < cols) {
                T bv = kd::neg_inf<T>();
                int bi = kNone;
                for (int q = 0; q < nchunks; ++q) {
                    const T v = ld_cg(pval + static_cast<int64_t>(q) * cols + c);
                    const int i = ld_cg(pidx + static_cast<int64_t>(q) * cols + c);
                    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
                }
                y[c] = bv;
                idx[c] = (bi == kNone) ? 0 : bi;
            }
        }
        if (threadIdx.x == 0) counters[stripe] = 0u;
    }
}

// Column reductions whose row chunks form one thread-block cluster.  grid = (stripes, CS), cluster = (1, CS, 1):
// the CS chunks of a column stripe are co-scheduled, every CTA pushes its per-column partials into the shared
// memory of the CTA that finishes that column (distributed shared memory stores), and after ONE hardware cluster
// barrier each CTA adds the CS values it received for its 32*V/CS columns (a fixed shuffle tree, so the result is
// reproducible).  No global partials, no atomics, no scratch: what is left of the tail is one cluster barrier.
// Measured on B200, fp64 4096 x 4096: sum 22.4 us against 24.1 us for the ticketed kernel above, max 22.9 us against
// 26.4 us.  For fp32 8192 x 8192 the ticketed sum is as fast (42.0 against 41.8 us), so fp32 sums stay there; the
// fp32 arg-max gains (43.0 against 44.1 us) once its registers are held to 48, i.e. five CTAs per SM: at four per SM
// the thirty-two 16-CTA clusters of the grid fit at once only if every GPC has sixteen SMs to give, and a second
// wave costs 40 % (60 us measured).
constexpr int kClusterChunks = 16;      // CTAs per cluster (above 8: needs the non-portable size attribute)

template <typename T, int V>
__global__ void __launch_bounds__(kThreads)         // 44-48 registers: five CTAs per SM without asking
sum_cols_cluster_kernel(const T* __restrict__ x, T* __restrict__ y, int rows, int cols, int rch, T scale, bool apply_scale) {
    kd::pdl_prologue();
    cg::cluster_group cluster = cg::this_cluster();
    cluster.barrier_arrive();                          // "this CTA runs": awaited before anybody stores into its shared memory
    constexpr int TC = 32 * V;
    __shared__ T sm[kWarps][TC + 1];
    __shared__ double recv[TC];                        // [chunk q][column slot]: what the chunks of the stripe push to this CTA
    const int lane = threadIdx.x & 31, phase = threadIdx.x >> 5;
    const int stripe = blockIdx.x, chunk = blockIdx.y;
    const int c0 = (stripe * 32 + lane) * V;
    const int r_begin = chunk * rch;
    const int r_end = min(rows, r_begin + rch);
    T acc[V];
#pragma unroll
    for (int k = 0; k < V; ++k) acc[k] = T(0);
    if (c0 < cols) {
        const T* src = x + c0;
        int r = r_begin + phase;
        for (; r + 3 * kWarps < r_end; r += 4 * kWarps) {
            T v[4][V];
#pragma unroll
            for (int u = 0; u < 4; ++u) ColLoad<T, V>::get(src + static_cast<int64_t>(r + u * kWarps) * cols, v[u]);
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int k = 0; k < V; ++k) acc[k] += v[u][k];
        }
        for (; r < r_end; r += kWarps) {
            T v[V];
            ColLoad<T, V>::get(src + static_cast<int64_t>(r) * cols, v);
#pragma unroll
            for (int k = 0; k < V; ++k) acc[k] += v[k];
        }
    }
#pragma unroll
    for (int k = 0; k < V; ++k) sm[phase][lane * V + k] = acc[k];
    __syncthreads();
    // Column j of the stripe is finished by the CTA of rank j / W: every chunk pushes its partial there (a remote
    // shared-memory store, nothing waits for it), one cluster barrier makes the pushes visible, and each CTA adds
    // the CS values it received from its own shared memory.  Nobody touches remote memory after the barrier, so
    // CTAs leave as they finish.
    const unsigned cs = cluster.num_blocks(), rank = cluster.block_rank();
    const unsigned W = TC / cs;
    cluster.barrier_wait();                            // every CTA of the cluster has started (long ago)
    for (int j = threadIdx.x; j < TC; j += kThreads) {
        double s = 0.0;
#pragma unroll
        for (int p = 0; p < kWarps; ++p) s += static_cast<double>(sm[p][j]);
        cluster.map_shared_rank(recv, j / W)[rank * W + j % W] = s;
    }
    cluster.sync();
    if (threadIdx.x < TC) {                            // whole warps: TC is a multiple of 32
        const unsigned q = threadIdx.x % cs, slot = threadIdx.x / cs;      // (chunk, column slot)
        double v = recv[q * W + slot];
        for (unsigned o = cs >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        const int c = stripe * TC + static_cast<int>(rank * W + slot);
        if (q == 0 && c < cols) {
            T out = static_cast<T>(v);
            if (apply_scale) out = out * scale;
            y[c] = out;
        }
    }
}

template <typename T, int V>
__global__ void __launch_bounds__(kThreads, 5)      // five CTAs per SM: 32 clusters of 16 then fit whatever the GPC sizes
max_cols_cluster_kernel(const T* __restrict__ x, T* __restrict__ y, long long* __restrict__ idx, int rows, int cols, int rch) {
    kd::pdl_prologue();
    cg::cluster_group cluster = cg::this_cluster();
    cluster.barrier_arrive();                          // "this CTA runs": awaited before anybody stores into its shared memory
    constexpr int TC = 32 * V;
    constexpr int kNone = std::numeric_limits<int>::max();
    __shared__ T smv[kWarps][TC + 1];
    __shared__ int smi[kWarps][TC + 1];
    __shared__ T rv[TC];                               // [chunk q][column slot] pushed here by the chunks of the stripe
    __shared__ int ri[TC];
    const int lane = threadIdx.x & 31, phase = threadIdx.x >> 5;
    const int stripe = blockIdx.x, chunk = blockIdx.y;
    const int c0 = (stripe * 32 + lane) * V;
    const int r_begin = chunk * rch;
    const int r_end = min(rows, r_begin + rch);
    T best[V];
    int brow[V];
#pragma unroll
    for (int k = 0; k < V; ++k) { best[k] = kd::neg_inf<T>(); brow[k] = kNone; }
    if (c0 < cols) {
        const T* src = x + c0;
        int r = r_begin + phase;
        for (; r + kWarps < r_end; r += 2 * kWarps) {
            T v[2][V];
#pragma unroll
            for (int u = 0; u < 2; ++u) ColLoad<T, V>::get(src + static_cast<int64_t>(r + u * kWarps) * cols, v[u]);
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int k = 0; k < V; ++k)
                    if (v[u][k] > best[k]) { best[k] = v[u][k]; brow[k] = r + u * kWarps; }
        }
        for (; r < r_end; r += kWarps) {
            T v[V];
            ColLoad<T, V>::get(src + static_cast<int64_t>(r) * cols, v);
#pragma unroll
            for (int k = 0; k < V; ++k)
                if (v[k] > best[k]) { best[k] = v[k]; brow[k] = r; }
        }
    }
#pragma unroll
    for (int k = 0; k < V; ++k) { smv[phase][lane * V + k] = best[k]; smi[phase][lane * V + k] = brow[k]; }
    __syncthreads();
    const unsigned cs = cluster.num_blocks(), rank = cluster.block_rank();
    const unsigned W = TC / cs;
    cluster.barrier_wait();
    for (int j = threadIdx.x; j < TC; j += kThreads) {
        T bv = kd::neg_inf<T>();
        int bi = kNone;
#pragma unroll
        for (int p = 0; p < kWarps; ++p) {
            const T v = smv[p][j];
            const int i = smi[p][j];
            if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
        }
        cluster.map_shared_rank(rv, j / W)[rank * W + j % W] = bv;     // pushed to the CTA that finishes column j
        cluster.map_shared_rank(ri, j / W)[rank * W + j % W] = bi;
    }
    cluster.sync();
    if (threadIdx.x < TC) {
        const unsigned q = threadIdx.x % cs, slot = threadIdx.x / cs;
        T bv = rv[q * W + slot];
        int bi = ri[q * W + slot];
        for (unsigned o = cs >> 1; o > 0; o >>= 1) {
            const T v = __shfl_xor_sync(0xffffffffu, bv, o);
            const int i = __shfl_xor_sync(0xffffffffu, bi, o);
            if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
        }
        const int c = stripe * TC + static_cast<int>(rank * W + slot);
        if (q == 0 && c < cols) {
            y[c] = bv;
            idx[c] = (bi == kNone) ? 0 : bi;
        }
    }
}

// ---------------------------------------------------------------------------
// Gradient kernels (pure writes)
// ---------------------------------------------------------------------------
// gx[i] = go[0] * scale   (keydnn_reduce_cuda.cu:122-149; scale is 1 for sum)
template <typename T>
__global__ void __launch_bounds__(kThreads)
bcast_scalar_kernel(const T* __restrict__ go, T* __restrict__ gx, int64_t n, T scale, int head) {
    kd::pdl_prologue();
    const T v = __ldg(go) * scale;
    const int64_t body = n - head;
    const int64_t n4 = body >> 2;
    T* gb = gx + head;
    Pack4<T> r;
    r.v[0] = r.v[1] = r.v[2] = r.v[3] = v;
    for (int64_t p = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; p < n4;
         p += static_cast<int64_t>(gridDim.x) * kThreads)
        kd::store4(gb + 4 * p, r);
    if (blockIdx.x == 0) {
        if (threadIdx.x < head) gx[threadIdx.x] = v;
        const int64_t i = head + (n4 << 2) + (threadIdx.x - 32);
        if (threadIdx.x >= 32 && threadIdx.x < 36 && i < n) gx[i] = v;
    }
}

// gx[i] = (i == idx[0]) ? 0 + go[0] : 0   (gradient of max over all elements)
template <typename T>
__global__ void __launch_bounds__(kThreads)
onehot_kernel(const T* __restrict__ go, const long long* __restrict__ idx, T* __restrict__ gx, int64_t n, int head) {
    kd::pdl_prologue();
    const T g = T(0) + __ldg(go);
    const long long target = __ldg(idx);
    const int64_t body = n - head;
    const int64_t n4 = body >> 2;
    T* gb = gx + head;
    for (int64_t p = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; p < n4;
         p += static_cast<int64_t>(gridDim.x) * kThreads) {
        const long long i0 = head + 4 * p;
        Pack4<T> r;
#pragma unroll
        for (int k = 0; k < 4; ++k) r.v[k] = (i0 + k == target) ? g : T(0);
        kd::store4(gb + 4 * p, r);
    }
    if (blockIdx.x == 0) {
        if (threadIdx.x < head) gx[threadIdx.x] = (threadIdx.x == target) ? g : T(0);
        const int64_t i = head + (n4 << 2) + (threadIdx.x - 32);
        if (threadIdx.x >= 32 && threadIdx.x < 36 && i < n) gx[i] = (i == target) ? g : T(0);
    }
}

// Matrix-shaped gradients.  MODE selects the value written at (r, c):
//   0: go[r]                      sum over axis 1
//   1: go[c]                      sum over axis 0
//   2: idx[r] == c ? 0+go[r] : 0  max over axis 1
//   3: idx[c] == r ? 0+go[c] : 0  max over axis 0
// `scale` multiplies modes 0/1 when apply_scale (mean over an axis).
// blockIdx.x / threadIdx.x walk 4-column packets of a row, blockIdx.y walks
// blocks of consecutive rows, so column-indexed operands are loaded once per
// thread and no division is needed.
template <typename T, int MODE, int V>
__global__ void __launch_bounds__(kThreads)
grad_matrix_kernel(const T* __restrict__ go, const long long* __restrict__ idx, T* __restrict__ gx, int rows, int cols,
                   T scale, bool apply_scale) {
    kd::pdl_prologue();
    const int ppr = (cols + V - 1) / V;
    for (int p = blockIdx.x * kThreads + threadIdx.x; p < ppr; p += gridDim.x * kThreads) {
        const int c0 = p * V;
        T gcol[V];
        long long icol[V];
        if (MODE == 1 || MODE == 3) {
#pragma unroll
            for (int k = 0; k < V; ++k) {
                gcol[k] = __ldg(go + c0 + k);
                if (MODE == 1 && apply_scale) gcol[k] = gcol[k] * scale;
                if (MODE == 3) { icol[k] = __ldg(idx + c0 + k); gcol[k] = T(0) + gcol[k]; }
            }
        }
        // blockIdx.y owns a block of consecutive rows: the grid writes the matrix front to back
        const int rpb = (rows + gridDim.y - 1) / gridDim.y;
        const int r_begin = blockIdx.y * rpb;
        const int r_end = min(rows, r_begin + rpb);
        for (int r = r_begin; r < r_end; ++r) {
            T out[V];
            if (MODE == 0) {
                T g = __ldg(go + r);
                if (apply_scale) g = g * scale;
#pragma unroll
                for (int k = 0; k < V; ++k) out[k] = g;
            } else if (MODE == 1) {
#pragma unroll
                for (int k = 0; k < V; ++k) out[k] = gcol[k];
            } else if (MODE == 2) {
                const long long target = __ldg(idx + r);
                const T g = T(0) + __ldg(go + r);
#pragma unroll
                for (int k = 0; k < V; ++k) out[k] = (target == c0 + k) ? g : T(0);
            } else {
#pragma unroll
                for (int k = 0; k < V; ++k) out[k] = (icol[k] == r) ? gcol[k] : T(0);
            }
            T* dst = gx + static_cast<int64_t>(r) * cols + c0;
            if (V == 4) {
                Pack4<T> pk;
#pragma unroll
                for (int k = 0; k < 4; ++k) pk.v[k] = out[k];
                kd::store4(dst, pk);
            } else {
                dst[0] = out[0];
            }
        }
    }
}

// Reference-signature max backward: grad_x[argmax] += grad_out onto the caller's
// (zero-filled) matrix (keydnn_reduce_cuda.cu:235-263).
template <typename T>
__global__ void __launch_bounds__(kThreads)
max_scatter_kernel(const T* __restrict__ go, const long long* __restrict__ idx, T* gx, int rows, int cols, int axis) {
    kd::pdl_prologue();
    const int n = axis == 1 ? rows : cols;
    for (int i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads) {
        const long long k = idx[i];
        if (axis == 1) {
            if (k >= 0 && k < cols) gx[static_cast<int64_t>(i) * cols + k] += go[i];
        } else {
            if (k >= 0 && k < rows) gx[k * cols + i] += go[i];
        }
    }
}

// ---------------------------------------------------------------------------
// sum_to_shape: out[k] = sum over (a, b) of x[a, k, b]   (outer A, kept K, inner B)
// ---------------------------------------------------------------------------
// One CTA per (k, slice of a): reads `ach` contiguous runs of B elements, leaves
// one partial; the last slice of k folds them in order.
template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads)
sum_akb_kernel(const T* __restrict__ x, T* __restrict__ y, int A, int K, int64_t B, int ach, double* partials,
               unsigned int* counters) {
    kd::pdl_prologue();
    __shared__ double sm[kWarps];
    const int k = blockIdx.x, slice = blockIdx.y, nslices = gridDim.y;
    const int a_begin = slice * ach;
    const int a_end = min(A, a_begin + ach);
    T a0 = T(0), a1 = T(0), a2 = T(0), a3 = T(0);
    for (int a = a_begin; a < a_end; ++a) {
        const T* src = x + (static_cast<int64_t>(a) * K + k) * B;
        if (VEC) {
            const int64_t b4 = B >> 2;
            for (int64_t p = threadIdx.x; p < b4; p += kThreads) {
                const Pack4<T> v = kd::load4_stream(src + 4 * p);
                a0 += v.v[0]; a1 += v.v[1]; a2 += v.v[2]; a3 += v.v[3];
            }
        } else {
            for (int64_t b = threadIdx.x; b < B; b += kThreads) a0 += src[b];
        }
    }
    double s = (static_cast<double>(a0) + static_cast<double>(a1)) +
               (static_cast<double>(a2) + static_cast<double>(a3));
    s = kd::block_sum(s, sm);
    if (nslices == 1) {
        if (threadIdx.x == 0) y[k] = static_cast<T>(s);
        return;
    }
    if (threadIdx.x == 0) partials[static_cast<int64_t>(slice) * K + k] = s;
    if (take_ticket_t0(counters + k, nslices)) {
        double v = 0.0;
        for (int q = threadIdx.x; q < nslices; q += kThreads) v += ld_cg(partials + static_cast<int64_t>(q) * K + k);
        v = kd::block_sum(v, sm);
        if (threadIdx.x == 0) { y[k] = static_cast<T>(v); counters[k] = 0u; }
    }
}

constexpr int kMaxDims = 8;
struct ShapeMeta {
    int ndim;
    int64_t in_stride[kMaxDims];
    int64_t out_stride[kMaxDims];   // 0 where the dimension is reduced
};

// Fallback for arbitrary kept/reduced interleavings: atomics onto a zeroed y.
template <typename T>
__global__ void __launch_bounds__(kThreads)
sum_to_shape_atomic_kernel(const T* __restrict__ x, T* y, int64_t n, ShapeMeta m) {
    kd::pdl_prologue();
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * kThreads) {
        int64_t rem = i, off = 0;
#pragma unroll
        for (int d = 0; d < kMaxDims; ++d) {
            if (d >= m.ndim) break;
            const int64_t q = rem / m.in_stride[d];
            rem -= q * m.in_stride[d];
            off += q * m.out_stride[d];
        }
        atomicAdd(y + off, x[i]);
    }
}

// ---------------------------------------------------------------------------
// Host-side launchers
// ---------------------------------------------------------------------------
template <typename T>
int sum_all(const T* x, T* y, int64_t n, bool mean) {
    if (!x || !y) return -1;
    if (n <= 0) return -2;
    (void)cudaGetLastError();
    const T scale = T(1) / static_cast<T>(n);
    if (kd::aligned_pack<T>(x) && (n >> 2) > 0) {
        const int64_t n4 = n >> 2;
        const int64_t per_cta = tile_packets_per_cta(n4, Tile<T>::kPackets);
        const unsigned grid = static_cast<unsigned>((n4 + per_cta - 1) / per_cta);
        double* partials = static_cast<double*>(kd::scratch(grid * sizeof(double)));
        unsigned int* counter = kd::counters(1);
        if (!partials || !counter) return static_cast<int>(cudaErrorMemoryAllocation);
        if (per_cta == Tile<T>::kPackets)
            (void)kd::launch(sum_all_tiles_kernel<T, Tile<T>::U, true>, dim3(grid), kThreads, 0, x, n, per_cta, partials, counter, y, scale, mean);
        else
            (void)kd::launch(sum_all_tiles_kernel<T, Tile<T>::U, false>, dim3(grid), kThreads, 0, x, n, per_cta, partials, counter, y, scale, mean);
        return kd::launch_status();
    }
    const int64_t tiles = (n + kThreads - 1) / kThreads;   // one wave of grid-stride CTAs
    const unsigned grid = kd::grid_fit(sum_all_kernel<T, false>, kThreads, tiles);
    double* partials = static_cast<double*>(kd::scratch(grid * sizeof(double)));
    unsigned int* counter = kd::counters(1);
    if (!partials || !counter) return static_cast<int>(cudaErrorMemoryAllocation);
    (void)kd::launch(sum_all_kernel<T, false>, dim3(grid), kThreads, 0, x, n, partials, counter, y, scale, mean);
    return kd::launch_status();
}

template <typename T>
int max_all(const T* x, T* y, long long* idx, int64_t n) {
    if (!x || !y || !idx) return -1;
    if (n <= 0) return -2;
    (void)cudaGetLastError();
    const bool vec = kd::aligned_pack<T>(x) && (n >> 2) > 0;
    int64_t per_cta = 0;
    unsigned grid;
    if (vec) {
        const int64_t n4 = n >> 2;
        // two trips of 32 KiB per CTA: measured best for the arg-max kernel, whose registers let four CTAs share an SM
        per_cta = tile_packets_per_cta(n4, 2 * Tile<T>::kPackets);
        grid = static_cast<unsigned>((n4 + per_cta - 1) / per_cta);
    } else {
        grid = kd::grid_fit(max_all_kernel<T, false>, kThreads, (n + kThreads - 1) / kThreads);
    }
    char* buf = static_cast<char*>(kd::scratch(static_cast<size_t>(grid) * 16));
    unsigned int* counter = kd::counters(1);
    if (!buf || !counter) return static_cast<int>(cudaErrorMemoryAllocation);
    long long* pidx = reinterpret_cast<long long*>(buf);
    T* pval = reinterpret_cast<T*>(buf + static_cast<size_t>(grid) * 8);
    if (vec)
        (void)kd::launch(max_all_tiles_kernel<T, Tile<T>::U, false>, dim3(grid), kThreads, 0, x, n, per_cta, pval, pidx, counter, y, idx);
    else (void)kd::launch(max_all_kernel<T, false>, dim3(grid), kThreads, 0, x, n, pval, pidx, counter, y, idx);
    return kd::launch_status();
}

template <typename T>
int sum_rows(const T* x, T* y, int64_t rows, int cols, T scale, bool apply_scale) {
    const bool vec = kd::aligned_pack<T>(x) && (cols % 4 == 0);
    cudaStream_t s = kd::stream();
    if (cols >= 2048) {
        if (vec) KD_LAUNCH((sum_rows_kernel<T, kThreads, true>), rows, kThreads, 0, x, y, rows, cols, scale, apply_scale);
        else KD_LAUNCH((sum_rows_kernel<T, kThreads, false>), rows, kThreads, 0, x, y, rows, cols, scale, apply_scale);
    } else {
        if (vec) KD_LAUNCH((sum_rows_kernel<T, 32, true>), (rows + kWarps - 1) / kWarps, kThreads, 0, x, y, rows, cols, scale, apply_scale);
        else KD_LAUNCH((sum_rows_kernel<T, 32, false>), (rows + kWarps - 1) / kWarps, kThreads, 0, x, y, rows, cols, scale, apply_scale);
    }
    return kd::launch_status();
}

template <typename T>
int max_rows(const T* x, T* y, long long* idx, int64_t rows, int cols) {
    const bool vec = kd::aligned_pack<T>(x) && (cols % 4 == 0);
    cudaStream_t s = kd::stream();
    if (cols >= 2048) {
        if (vec) KD_LAUNCH((max_rows_kernel<T, kThreads, true>), rows, kThreads, 0, x, y, idx, rows, cols);
        else KD_LAUNCH((max_rows_kernel<T, kThreads, false>), rows, kThreads, 0, x, y, idx, rows, cols);
    } else {
        if (vec) KD_LAUNCH((max_rows_kernel<T, 32, true>), (rows + kWarps - 1) / kWarps, kThreads, 0, x, y, idx, rows, cols);
        else KD_LAUNCH((max_rows_kernel<T, 32, false>), (rows + kWarps - 1) / kWarps, kThreads, 0, x, y, idx, rows, cols);
    }
    return kd::launch_status();
}

// Row-chunk height for column reductions.  The (stripe, chunk) grid is sized to
// what the machine holds at once, so every CTA is resident from the start, all do
// the same amount of work and there is no partial last wave; partial traffic is
// nchunks * cols elements (under 1% of the input at the benchmark sizes).
// All of this arithmetic is 64-bit: `rows` may be close to 2^31 for a narrow matrix.
inline int64_t pick_row_chunk(int rows, int stripes, int ctas_per_sm) {
    const int64_t slots = static_cast<int64_t>(kd::sm_count()) * ctas_per_sm;
    int64_t nchunks = slots / stripes;
    const int64_t max_chunks = (static_cast<int64_t>(rows) + 4 * kWarps - 1) / (4 * kWarps);   // at least 32 rows per chunk
    if (nchunks > max_chunks) nchunks = max_chunks;
    if (nchunks < 1) nchunks = 1;
    int64_t rch = (static_cast<int64_t>(rows) + nchunks - 1) / nchunks;
    rch = ((rch + kWarps - 1) / kWarps) * kWarps;
    return rch;
}

// The (stripe, chunk) launch shape of a column reduction, or false when it cannot be launched: the kernels
// index rows with 32-bit integers, so chunk * rch, r_begin + rch and the unrolled look-ahead of the row loop
// (r + 3 * kWarps) must all stay below 2^31, and gridDim.y is limited to 65,535.
struct ColChunks {
    int rch = 0, nchunks = 0;
};
inline bool col_chunks(int rows, int64_t rch, ColChunks* out) {
    if (rch < 1) return false;
    const int64_t nchunks = (static_cast<int64_t>(rows) + rch - 1) / rch;
    const int64_t reach = nchunks * rch + 4 * kWarps;       // largest row index any thread computes
    if (nchunks > 65535 || reach > std::numeric_limits<int>::max()) return false;
    out->rch = static_cast<int>(rch);
    out->nchunks = static_cast<int>(nchunks);
    return true;
}

// Whether a column reduction of (rows, cols) takes the cluster path, and with which chunk height: 8-byte elements,
// 32-byte lanes, a shape for which about kClusterChunks chunks per stripe fill the machine (that is what the
// ticketed kernels would use), and a device that can hold at least one such cluster.  `kernel` must be the
// instantiation that will be launched; the non-portable cluster size is enabled on it once.
template <typename K>
inline bool cluster_cols_plan(K kernel, size_t elem_size, int V, int rows, int stripes, int ctas_per_sm, bool f32_too,
                              int* rch_out) {
    if (!((elem_size == 8 && V == 4) || (f32_too && elem_size == 4 && V == 8))) return false;     // 32 bytes per lane
    const int64_t slots = static_cast<int64_t>(kd::sm_count()) * ctas_per_sm;
    const int64_t wanted = slots / stripes;
    if (wanted < 12 || wanted > 32) return false;
    if (rows < kClusterChunks * 4 * kWarps) return false;           // at least 32 rows per chunk
    static std::unordered_map<const void*, int> usable;             // kernel -> 1 usable, 0 not (per process)
    const void* key = reinterpret_cast<const void*>(kernel);
    auto it = usable.find(key);
    if (it == usable.end()) {
        int ok = 0;
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(1, kClusterChunks);
            cfg.blockDim = dim3(kThreads);
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1;
            attr[0].val.clusterDim.y = kClusterChunks;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) == cudaSuccess && n >= 1) ok = 1;
        }
        (void)cudaGetLastError();
        it = usable.emplace(key, ok).first;
    }
    if (!it->second) return false;
    int64_t rch = (static_cast<int64_t>(rows) + kClusterChunks - 1) / kClusterChunks;
    rch = (rch + kWarps - 1) / kWarps * kWarps;
    if ((static_cast<int64_t>(rows) + rch - 1) / rch != kClusterChunks) return false;   // every rank of the cluster gets rows
    ColChunks cc;
    if (!col_chunks(rows, rch, &cc)) return false;
    *rch_out = cc.rch;
    return true;
}

template <typename T, int V>
int sum_cols_v(const T* x, T* y, int rows, int cols, T scale, bool apply_scale) {
    const int stripes = (cols + 32 * V - 1) / (32 * V);
    int crch = 0;
    // fp32 sums stay on the ticketed kernel: measured equal there (41.8 against 42.0 us), and the allocation-free
    // entry then keeps giving the regular entry's bits
    if (cluster_cols_plan(sum_cols_cluster_kernel<T, V>, sizeof(T), V, rows, stripes, kd::occupancy(sum_cols_kernel<T, V>, kThreads), false,
                          &crch)) {
        if (kd::launch_cluster_y(sum_cols_cluster_kernel<T, V>, dim3(stripes, kClusterChunks), kThreads, kClusterChunks, x, y, rows, cols,
                                 crch, scale, apply_scale) == cudaSuccess)
            return kd::launch_status();
        (void)cudaGetLastError();          // could not be launched as a cluster: the ticketed kernel below
    }
    ColChunks cc;
    if (!col_chunks(rows, pick_row_chunk(rows, stripes, kd::occupancy(sum_cols_kernel<T, V>, kThreads)), &cc)) return -2;
    const int rch = cc.rch, nchunks = cc.nchunks;
    T* partials = nullptr;
    unsigned int* counters = nullptr;
    if (nchunks > 1) {
        partials = static_cast<T*>(kd::scratch(static_cast<size_t>(nchunks) * cols * sizeof(T)));
        counters = kd::counters(stripes);
        if (!partials || !counters) return static_cast<int>(cudaErrorMemoryAllocation);
    }
    (void)kd::launch(sum_cols_kernel<T, V>, dim3(stripes, nchunks), kThreads, 0, x, y, rows, cols, rch, partials, counters,
                                                                               scale, apply_scale);
    return kd::launch_status();
}

template <typename T>
int sum_cols(const T* x, T* y, int rows, int cols, T scale, bool apply_scale) {
    const int V = col_vector_width<T>(x, cols);
    if (sizeof(T) == 4 && V == 8) return sum_cols_v<T, (sizeof(T) == 4 ? 8 : 4)>(x, y, rows, cols, scale, apply_scale);
    if (V >= 4) return sum_cols_v<T, 4>(x, y, rows, cols, scale, apply_scale);
    return sum_cols_v<T, 1>(x, y, rows, cols, scale, apply_scale);
}

template <typename T, int V>
int max_cols_v(const T* x, T* y, long long* idx, int rows, int cols) {
    const int stripes = (cols + 32 * V - 1) / (32 * V);
    int crch = 0;
    if (cluster_cols_plan(max_cols_cluster_kernel<T, V>, sizeof(T), V, rows, stripes, kd::occupancy(max_cols_kernel<T, V>, kThreads), true,
                          &crch)) {
        if (kd::launch_cluster_y(max_cols_cluster_kernel<T, V>, dim3(stripes, kClusterChunks), kThreads, kClusterChunks, x, y, idx, rows,
                                 cols, crch) == cudaSuccess)
            return kd::launch_status();
        (void)cudaGetLastError();
    }
    ColChunks cc;
    if (!col_chunks(rows, pick_row_chunk(rows, stripes, kd::occupancy(max_cols_kernel<T, V>, kThreads)), &cc)) return -2;
    const int rch = cc.rch, nchunks = cc.nchunks;
    T* pval = nullptr;
    int* pidx = nullptr;
    unsigned int* counters = nullptr;
    if (nchunks > 1) {
        const size_t cells = static_cast<size_t>(nchunks) * cols;
        char* buf = static_cast<char*>(kd::scratch(cells * (sizeof(T) + sizeof(int))));
        counters = kd::counters(stripes);
        if (!buf || !counters) return static_cast<int>(cudaErrorMemoryAllocation);
        pval = reinterpret_cast<T*>(buf);
        pidx = reinterpret_cast<int*>(buf + cells * sizeof(T));
    }
    (void)kd::launch(max_cols_kernel<T, V>, dim3(stripes, nchunks), kThreads, 0, x, y, idx, rows, cols, rch, pval, pidx,
                                                                               counters);
    return kd::launch_status();
}

template <typename T>
int max_cols(const T* x, T* y, long long* idx, int rows, int cols) {
    const int V = col_vector_width<T>(x, cols);
    if (sizeof(T) == 4 && V == 8) return max_cols_v<T, (sizeof(T) == 4 ? 8 : 4)>(x, y, idx, rows, cols);
    if (V >= 4) return max_cols_v<T, 4>(x, y, idx, rows, cols);
    return max_cols_v<T, 1>(x, y, idx, rows, cols);
}

template <typename T>
int reduce_axis2d_sum(const T* x, T* y, int rows, int cols, int axis, bool mean) {
    if (!x || !y) return -1;
    if (rows <= 0 || cols <= 0) return -2;
    if (!(axis == 0 || axis == 1)) return -3;
    (void)cudaGetLastError();
    const T scale = T(1) / static_cast<T>(axis == 1 ? cols : rows);
    return axis == 1 ? sum_rows<T>(x, y, rows, cols, scale, mean) : sum_cols<T>(x, y, rows, cols, scale, mean);
}

template <typename T>
int reduce_axis2d_max(const T* x, T* y, long long* idx, int rows, int cols, int axis) {
    if (!x || !y || !idx) return -1;
    if (rows <= 0 || cols <= 0) return -2;
    if (!(axis == 0 || axis == 1)) return -3;
    (void)cudaGetLastError();
    return axis == 1 ? max_rows<T>(x, y, idx, rows, cols) : max_cols<T>(x, y, idx, rows, cols);
}

template <typename T>
int bcast_scalar(const T* go, T* gx, int64_t n, T scale) {
    if (!go || !gx) return -1;
    if (n <= 0) return -2;
    (void)cudaGetLastError();
    const uintptr_t addr = reinterpret_cast<uintptr_t>(gx);
    if (addr % sizeof(T)) return static_cast<int>(cudaErrorMisalignedAddress);
    constexpr uintptr_t kA = sizeof(T) * 4;   // packet alignment
    int head = static_cast<int>(((kA - (addr & (kA - 1))) & (kA - 1)) / sizeof(T));
    if (head > n) head = static_cast<int>(n);
    KD_LAUNCH_W(bcast_scalar_kernel<T>, 16, ((n >> 2) + kThreads - 1) / kThreads + 1, kThreads, 0, go, gx, n, scale, head);
    return kd::launch_status();
}

template <typename T, int MODE>
int grad_matrix(const T* go, const long long* idx, T* gx, int rows, int cols, T scale, bool apply_scale) {
    const bool vec = kd::aligned_pack<T>(gx) && (cols % 4 == 0);
    const int V = vec ? 4 : 1;
    const int ppr = (cols + V - 1) / V;
    int gx_dim = (ppr + kThreads - 1) / kThreads;
    if (gx_dim > 64) gx_dim = 64;
    int64_t want = static_cast<int64_t>(kd::sm_count()) * 8 * 16;     // many small CTAs: see grid_fit
    int gy = static_cast<int>((want + gx_dim - 1) / gx_dim);
    if (gy > (rows + 3) / 4) gy = (rows + 3) / 4;      // at least four rows per CTA: column operands amortise
    if (gy > 65535) gy = 65535;
    if (gy < 1) gy = 1;
    dim3 grid(gx_dim, gy);
    cudaStream_t s = kd::stream();
    if (vec) (void)kd::launch(grad_matrix_kernel<T, MODE, 4>, dim3(grid), kThreads, 0, go, idx, gx, rows, cols, scale, apply_scale);
    else (void)kd::launch(grad_matrix_kernel<T, MODE, 1>, dim3(grid), kThreads, 0, go, idx, gx, rows, cols, scale, apply_scale);
    return kd::launch_status();
}

template <typename T>
int sum_axis2d_backward(const T* go, T* gx, int rows, int cols, int axis, bool mean) {
    if (!go || !gx) return -1;
    if (rows <= 0 || cols <= 0) return -2;
    if (!(axis == 0 || axis == 1)) return -3;
    (void)cudaGetLastError();
    const T scale = T(1) / static_cast<T>(axis == 1 ? cols : rows);
    return axis == 1 ? grad_matrix<T, 0>(go, nullptr, gx, rows, cols, scale, mean)
                     : grad_matrix<T, 1>(go, nullptr, gx, rows, cols, scale, mean);
}

template <typename T>
int max_axis2d_backward_full(const T* go, const long long* idx, T* gx, int rows, int cols, int axis) {
    if (!go || !idx || !gx) return -1;
    if (rows <= 0 || cols <= 0) return -2;
    if (!(axis == 0 || axis == 1)) return -3;
    (void)cudaGetLastError();
    return axis == 1 ? grad_matrix<T, 2>(go, idx, gx, rows, cols, T(1), false)
                     : grad_matrix<T, 3>(go, idx, gx, rows, cols, T(1), false);
}

template <typename T>
int max_axis2d_backward_legacy(const T* go, const long long* idx, T* gx, int rows, int cols, int axis) {
    if (!go || !idx || !gx) return -1;
    if (rows <= 0 || cols <= 0) return -2;
    if (!(axis == 0 || axis == 1)) return -3;
    (void)cudaGetLastError();
    const int n = axis == 1 ? rows : cols;
    const unsigned grid = kd::grid_for((n + kThreads - 1) / kThreads, 8);
    (void)kd::launch(max_scatter_kernel<T>, dim3(grid), kThreads, 0, go, idx, gx, rows, cols, axis);
    return kd::launch_status();
}

template <typename T>
int max_all_backward(const T* go, const long long* idx, T* gx, int64_t n) {
    if (!go || !idx || !gx) return -1;
    if (n <= 0) return -2;
    (void)cudaGetLastError();
    const uintptr_t addr = reinterpret_cast<uintptr_t>(gx);
    if (addr % sizeof(T)) return static_cast<int>(cudaErrorMisalignedAddress);
    constexpr uintptr_t kA = sizeof(T) * 4;   // packet alignment
    int head = static_cast<int>(((kA - (addr & (kA - 1))) & (kA - 1)) / sizeof(T));
    if (head > n) head = static_cast<int>(n);
    KD_LAUNCH_W(onehot_kernel<T>, 16, ((n >> 2) + kThreads - 1) / kThreads + 1, kThreads, 0, go, idx, gx, n, head);
    return kd::launch_status();
}

template <typename T>
int sum_to_shape(const T* x, T* y, const int64_t* in_shape, const int64_t* out_shape, int ndim) {
    if (!x || !y || !in_shape || !out_shape) return -1;
    if (ndim <= 0) return -2;
    if (ndim > kMaxDims) return -3;
    int64_t numel_in = 1, numel_out = 1;
    for (int d = 0; d < ndim; ++d) {
        const int64_t id = in_shape[d], od = out_shape[d];
        if (id < 0 || od < 0) return -4;
        if (!(od == 1 || od == id)) return -5;
        numel_in *= id;
        numel_out *= od;
    }
    if (numel_out == 0) return 0;
    (void)cudaGetLastError();
    cudaStream_t s = kd::stream();
    if (numel_in == 0) return kd::status(cudaMemsetAsync(y, 0, numel_out * sizeof(T), s));

    // Collapse to alternating groups of reduced (R) / kept (K) extents.
    int64_t ext[kMaxDims];
    bool red[kMaxDims];
    int ng = 0;
    for (int d = 0; d < ndim; ++d) {
        if (in_shape[d] == 1) continue;
        const bool r = (out_shape[d] == 1);
        if (ng > 0 && red[ng - 1] == r) ext[ng - 1] *= in_shape[d];
        else { ext[ng] = in_shape[d]; red[ng] = r; ++ng; }
    }
    const int64_t imax = std::numeric_limits<int>::max();
    if (ng == 0 || (ng == 1 && !red[0]))
        return kd::status(cudaMemcpyAsync(y, x, numel_in * sizeof(T), cudaMemcpyDeviceToDevice, s));
    if (ng == 1) return sum_all<T>(x, y, numel_in, false);
    if (ng == 2 && red[0] && ext[0] <= imax && ext[1] <= imax)
        return sum_cols<T>(x, y, static_cast<int>(ext[0]), static_cast<int>(ext[1]), T(1), false);
    if (ng == 2 && !red[0] && ext[1] <= imax)
        return sum_rows<T>(x, y, ext[0], static_cast<int>(ext[1]), T(1), false);
    if (ng == 3 && red[0] && ext[0] <= imax && ext[1] <= imax) {
        const int A = static_cast<int>(ext[0]), K = static_cast<int>(ext[1]);
        const int64_t B = ext[2];
        // Short CTAs (about 32 KiB of input each, as for the full reductions) handed out as SMs free up; at most
        // kThreads slices per kept index so that the CTA that draws the last ticket folds them in one round, and
        // never fewer CTAs than cover the machine a few times.
        int64_t ach64 = (int64_t(32) << 10) / static_cast<int64_t>(sizeof(T)) / (B > 0 ? B : 1);
        if (ach64 < 1) ach64 = 1;
        const int64_t fill = (static_cast<int64_t>(kd::sm_count()) * 8 + K - 1) / K;      // slices that fill the machine
        if ((A + ach64 - 1) / ach64 < fill) ach64 = (A + fill - 1) / fill;
        if (ach64 < 1) ach64 = 1;
        if ((A + ach64 - 1) / ach64 > kThreads) ach64 = (A + kThreads - 1) / kThreads;
        const int ach = static_cast<int>(ach64);
        int nslices = (A + ach - 1) / ach;
        double* partials = nullptr;
        unsigned int* counters = nullptr;
        if (nslices > 1) {
            partials = static_cast<double*>(kd::scratch(static_cast<size_t>(nslices) * K * sizeof(double)));
            counters = kd::counters(K);
            if (!partials || !counters) return static_cast<int>(cudaErrorMemoryAllocation);
        }
        dim3 grid(K, nslices);
        const bool vec = kd::aligned_pack<T>(x) && (B % 4 == 0);
        if (vec) (void)kd::launch(sum_akb_kernel<T, true>, dim3(grid), kThreads, 0, x, y, A, K, B, ach, partials, counters);
        else (void)kd::launch(sum_akb_kernel<T, false>, dim3(grid), kThreads, 0, x, y, A, K, B, ach, partials, counters);
        return kd::launch_status();
    }
    // general interleaving
    ShapeMeta m;
    m.ndim = ndim;
    int64_t si = 1, so = 1;
    for (int d = ndim - 1; d >= 0; --d) {
        m.in_stride[d] = si;
        m.out_stride[d] = (out_shape[d] == 1) ? 0 : so;
        si *= in_shape[d];
        so *= out_shape[d];
    }
    cudaError_t st = cudaMemsetAsync(y, 0, numel_out * sizeof(T), s);
    if (st != cudaSuccess) return kd::status(st);
    const unsigned grid = kd::grid_for((numel_in + kThreads - 1) / kThreads, 8);
    (void)kd::launch(sum_to_shape_atomic_kernel<T>, dim3(grid), kThreads, 0, x, y, numel_in, m);
    return kd::launch_status();
}

}  // namespace

// ---------------------------------------------------------------------------
// C ABI: reference signatures (keydnn_reduce_cuda.hpp:56-140).  Guards: -1 null
// pointer, -2 non-positive extent, -3 bad axis (keydnn_reduce_cuda.cu:74-75,
// 209-211); sum_to_shape -1..-5 (:467-489).
// ---------------------------------------------------------------------------
#define KD_REDUCE(T, SUF)                                                                                           \
    KD_API int keydnn_cuda_sum_all_##SUF(const T* x, T* y, int64_t numel) { return sum_all<T>(x, y, numel, false); } \
    KD_API int keydnn_cuda_mean_all_##SUF(const T* x, T* y, int64_t numel) { return sum_all<T>(x, y, numel, true); } \
    KD_API int keydnn_cuda_sum_backward_fill_##SUF(const T* grad_out, T* grad_x, int64_t numel) {                   \
        return bcast_scalar<T>(grad_out, grad_x, numel, T(1));                                                      \
    }                                                                                                               \
    KD_API int keydnn_cuda_mean_backward_fill_##SUF(const T* grad_out, T* grad_x, int64_t numel) {                  \
        if (numel <= 0) return (!grad_out || !grad_x) ? -1 : -2;                                                    \
        return bcast_scalar<T>(grad_out, grad_x, numel, T(1) / static_cast<T>(numel));                              \
    }                                                                                                               \
    KD_API int keydnn_cuda_max_axis2d_forward_##SUF(const T* x, T* y, int64_t* idx, int rows, int cols, int axis) { \
        return reduce_axis2d_max<T>(x, y, reinterpret_cast<long long*>(idx), rows, cols, axis);                     \
    }                                                                                                               \
    KD_API int keydnn_cuda_max_axis2d_backward_##SUF(const T* grad_out, const int64_t* idx, T* grad_x, int rows,    \
                                                     int cols, int axis) {                                          \
        return max_axis2d_backward_legacy<T>(grad_out, reinterpret_cast<const long long*>(idx), grad_x, rows, cols, \
                                             axis);                                                                 \
    }                                                                                                               \
    KD_API int keydnn_cuda_sum_axis2d_forward_##SUF(const T* x, T* y, int rows, int cols, int axis) {               \
        return reduce_axis2d_sum<T>(x, y, rows, cols, axis, false);                                                 \
    }                                                                                                               \
    KD_API int keydnn_cuda_sum_axis2d_backward_##SUF(const T* grad_out, T* grad_x, int rows, int cols, int axis) {  \
        return sum_axis2d_backward<T>(grad_out, grad_x, rows, cols, axis, false);                                   \
    }                                                                                                               \
    KD_API int keydnn_cuda_sum_to_shape_##SUF(const T* x, T* y, const int64_t* in_shape, const int64_t* out_shape,  \
                                              int ndim) {                                                           \
        return sum_to_shape<T>(x, y, in_shape, out_shape, ndim);                                                    \
    }                                                                                                               \
    /* ---- additive entries (no counterpart in the reference library) ---- */                                      \
    /* max backward that writes the whole matrix: no zero-fill pass before it */                                    \
    KD_API int keydnn_cuda_max_axis2d_backward_ex_##SUF(const T* grad_out, const int64_t* idx, T* grad_x, int rows, \
                                                        int cols, int axis) {                                       \
        return max_axis2d_backward_full<T>(grad_out, reinterpret_cast<const long long*>(idx), grad_x, rows, cols,   \
                                           axis);                                                                   \
    }                                                                                                               \
    /* mean over one axis of a matrix: sum * (1/extent), and its gradient */                                        \
    KD_API int keydnn_cuda_mean_axis2d_forward_##SUF(const T* x, T* y, int rows, int cols, int axis) {              \
        return reduce_axis2d_sum<T>(x, y, rows, cols, axis, true);                                                  \
    }                                                                                                               \
    KD_API int keydnn_cuda_mean_axis2d_backward_##SUF(const T* grad_out, T* grad_x, int rows, int cols, int axis) { \
        return sum_axis2d_backward<T>(grad_out, grad_x, rows, cols, axis, true);                                    \
    }                                                                                                               \
    /* max over all elements with the flat position of its first occurrence */                                      \
    KD_API int keydnn_cuda_max_all_forward_##SUF(const T* x, T* y, int64_t* idx, int64_t numel) {                   \
        return max_all<T>(x, y, reinterpret_cast<long long*>(idx), numel);                                          \
    }                                                                                                               \
    KD_API int keydnn_cuda_max_all_backward_##SUF(const T* grad_out, const int64_t* idx, T* grad_x, int64_t numel) { \
        return max_all_backward<T>(grad_out, reinterpret_cast<const long long*>(idx), grad_x, numel);               \
    }

KD_REDUCE(float, f32)
KD_REDUCE(double, f64)

// Additive, host-only: the launch shape the column reductions would use for a (rows, cols) matrix of
// `elem_size`-byte elements with `ctas_per_sm` resident CTAs per SM: out3 = {rows per chunk, chunks, stripes}.
// Returns -2 where the entry points return -2 (the shape cannot be indexed with 32-bit rows).  No device work.
KD_API int keydnn_cuda_debug_col_chunks(int rows, int cols, int elem_size, int ctas_per_sm, int64_t* out3) {
    if (!out3) return -1;
    if (rows <= 0 || cols <= 0 || ctas_per_sm <= 0 || !(elem_size == 4 || elem_size == 8)) return -2;
    const int V = 32 / elem_size;
    const int stripes = (cols + 32 * V - 1) / (32 * V);
    ColChunks cc;
    if (!col_chunks(rows, pick_row_chunk(rows, stripes, ctas_per_sm), &cc)) return -2;
    out3[0] = cc.rch;
    out3[1] = cc.nchunks;
    out3[2] = stripes;
    return 0;
}

// ---------------------------------------------------------------------------
// Column sums without any device allocation
// ---------------------------------------------------------------------------
// For callers that must not allocate device memory when they call in: code running inside a
// framework that owns the whole device heap (its caching allocator has reserved the memory and a
// stray cudaMalloc can fail or fragment it), latency-critical serving loops where an allocation
// would stall every stream of the process, and processes that run under a fixed memory budget
// checked at start-up.  The regular column-sum entry may grow the library's scratch buffer with
// cudaMalloc the first time a shape needs it; this one never does: its partial sums and completion
// tickets live in the file-scope array below, which every GPU that loads the library holds from
// load to exit (kNoAllocCounterBytes + kNoAllocPartialBytes = 2,113,536 bytes).
namespace {

constexpr size_t kNoAllocCounterBytes = 16 * 1024;        // 4096 completion tickets
constexpr size_t kNoAllocPartialBytes = size_t(2) << 20;  // per-chunk column partials
constexpr int kNoAllocMaxCols = 65536;
constexpr int kNoAllocTooLarge = -20;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocCounterBytes + kNoAllocPartialBytes];

// In host code `g_noalloc_scratch` is only a handle for the runtime, not a device address; the
// address the kernel needs comes from cudaGetSymbolAddress, once per device, with that device current.
struct NoAllocDevice {
    bool ready = false;
    unsigned char* base = nullptr;
};
NoAllocDevice g_noalloc_device[16];
std::mutex g_noalloc_mu;           // the first call per device may come from any host thread

int noalloc_base(unsigned char** out) {
    int dev = -1;
    cudaError_t st = cudaGetDevice(&dev);
    if (st != cudaSuccess) return static_cast<int>(st);
    if (dev < 0 || dev >= 16) return static_cast<int>(cudaErrorInvalidDevice);
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    NoAllocDevice& d = g_noalloc_device[dev];
    if (!d.ready) {
        void* p = nullptr;
        st = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (st != cudaSuccess) return static_cast<int>(st);
        if (!p) return static_cast<int>(cudaErrorInvalidSymbol);
        d.base = static_cast<unsigned char*>(p);
        d.ready = true;
    }
    *out = d.base;
    return 0;
}

template <int V>
int noalloc_sum_cols(const float* x, float* y, int rows, int cols, unsigned char* base) {
    const int stripes = (cols + 32 * V - 1) / (32 * V);
    if (static_cast<size_t>(stripes) * sizeof(unsigned int) > kNoAllocCounterBytes) return kNoAllocTooLarge;
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, sum_cols_kernel<float, V>, kThreads, 0) != cudaSuccess || occ < 1)
        occ = 1;
    int64_t rch64 = pick_row_chunk(rows, stripes, occ);
    // fewer, taller chunks until the partials fit the static array
    while (static_cast<size_t>((rows + rch64 - 1) / rch64) * cols * sizeof(float) > kNoAllocPartialBytes) rch64 *= 2;
    ColChunks cc;
    if (!col_chunks(rows, rch64, &cc)) return kNoAllocTooLarge;
    const int rch = cc.rch, nchunks = cc.nchunks;
    unsigned int* counters = reinterpret_cast<unsigned int*>(base);
    float* partials = reinterpret_cast<float*>(base + kNoAllocCounterBytes);
    cudaStream_t s = kd::stream();
    // the array keeps whatever the previous call left: tickets must start at zero
    cudaError_t st = cudaMemsetAsync(counters, 0, static_cast<size_t>(stripes) * sizeof(unsigned int), s);
    if (st != cudaSuccess) return static_cast<int>(st);
    (void)kd::launch(sum_cols_kernel<float, V>, dim3(stripes, nchunks), kThreads, 0, x, y, rows, cols, rch, partials, counters, 1.0f,
                                                                       false);
    return kd::launch_status();
}

}  // namespace

// y[c] = sum over r of x[r, c] for a dense row-major float32 (rows, cols) matrix, same result
// contract as keydnn_cuda_sum_axis2d_forward_f32(x, y, rows, cols, 0), but this call allocates
// nothing: no cudaMalloc / cudaFree, no allocating library routine.
//   * limits: cols <= 65,536 (KEYDNN_NOALLOC_MAX_COLS); larger returns -20 and launches nothing.
//   * the first call on a device looks up the array's device address (cudaGetSymbolAddress); make
//     that first call outside any stream capture.
//   * every call uses the same array: calls that overlap on the GPU (two streams, two host
//     threads) race on it.  Calls on the library's one stream are ordered and safe.
KD_API int keydnn_cuda_sum_axis0_noalloc_f32(const float* x, float* y, int rows, int cols) {
    if (!x || !y) return -1;
    if (rows <= 0 || cols <= 0) return -2;
    if (cols > kNoAllocMaxCols) return kNoAllocTooLarge;
    unsigned char* base = nullptr;
    const int st = noalloc_base(&base);
    if (st != 0) return st;
    (void)cudaGetLastError();
    const int V = col_vector_width<float>(x, cols);
    if (V == 8) return noalloc_sum_cols<8>(x, y, rows, cols, base);
    if (V == 4) return noalloc_sum_cols<4>(x, y, rows, cols, base);
    return noalloc_sum_cols<1>(x, y, rows, cols, base);
}
