// Softmax forward / backward along one axis of a dense tensor viewed as (outer, len, inner).
//
// Reference: SoftmaxFn (_function.py:547-575, :604-610) runs max -> broadcast_to -> sub -> exp ->
// sum -> broadcast_to -> div (forward) and mul -> sum -> broadcast_to -> sub -> mul (backward), seven
// and five kernels with as many temporaries.  Here each direction is one kernel: one HBM read of
// every operand, one write.  Element arithmetic is the reference's, separately rounded:
//   forward   m = max over the axis (strict >, from -inf; a NaN never wins)
//             e = exp(x - m);  y = e * (1 / sum(e))
//   backward  gy = g * y;  dx = y * (g - sum(gy))
// Rows of at most 32 elements are walked serially by one thread, in the reference's order and with its
// division: bit-identical to the reference chain.  Longer rows use tree sums (the reference adds serially),
// so their results equal the reference's only to rounding in any case; their forward therefore multiplies
// by the correctly rounded reciprocal of the sum (one division per row) instead of dividing every element,
// which halves its instruction count.
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

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// Reductions inside groups of G neighbouring lanes (G a power of two).
template <typename T, int G> __device__ __forceinline__ T group_max(T v) {
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) {
        const T w = __shfl_xor_sync(0xffffffffu, v, o);
        v = w > v ? w : v;
    }
    return v;
}
template <typename T, int G> __device__ __forceinline__ T group_add(T v) {
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) v = Rn<T>::add(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---- rows of up to G*R elements: G lanes own a row, lane l of the group holds elements l, l+G, ...;
// a warp works on K groups of 32/G rows at once so that K*R independent loads are in flight per lane.
template <typename T, int G, int R, int K, bool BWD>
__global__ void __launch_bounds__(kThreads, (R * sizeof(T) * (BWD ? 2 : 1) >= 128 ? 3 : 1))
softmax_warp_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t rows, int len) {
    kd::pdl_prologue();
    constexpr int RPG = 32 / G;                 // rows per group of a warp
    constexpr int RPW = RPG * K;                // rows per warp and trip
    const int lane = threadIdx.x & 31;
    const int sub = lane / G, col0 = lane % G;
    const int64_t warp0 = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kWarps;
    const int64_t trips = (rows + RPW - 1) / RPW;
    for (int64_t trip = warp0; trip < trips; trip += stride) {
        T va[K][R], vb[K][R];
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const int64_t row = trip * RPW + k * RPG + sub;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int c = col0 + G * r;
                const bool ok = row < rows && c < len;
                if (BWD) {
                    va[k][r] = ok ? __ldcs(a + row * len + c) : T(0);                  // g
                    vb[k][r] = ok ? __ldcs(b + row * len + c) : T(0);                  // y
                } else {
                    va[k][r] = ok ? __ldcs(a + row * len + c) : neg_inf<T>();
                }
            }
        }
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const int64_t row = trip * RPW + k * RPG + sub;
            if (BWD) {
                T dot = T(0);
#pragma unroll
                for (int r = 0; r < R; ++r) dot = Rn<T>::add(dot, Rn<T>::mul(va[k][r], vb[k][r]));
                dot = group_add<T, G>(dot);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int c = col0 + G * r;
                    if (row < rows && c < len)
                        __stcs(out + row * len + c, Rn<T>::mul(vb[k][r], Rn<T>::sub(va[k][r], dot)));
                }
            } else {
                T m = neg_inf<T>();
#pragma unroll
                for (int r = 0; r < R; ++r) m = va[k][r] > m ? va[k][r] : m;
                m = group_max<T, G>(m);
                T s = T(0);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int c = col0 + G * r;
                    va[k][r] = (row < rows && c < len) ? t_exp(Rn<T>::sub(va[k][r], m)) : T(0);
                    s = Rn<T>::add(s, va[k][r]);
                }
                const T inv = t_div(T(1), group_add<T, G>(s));
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int c = col0 + G * r;
                    if (row < rows && c < len) __stcs(out + row * len + c, Rn<T>::mul(va[k][r], inv));
                }
            }
        }
    }
}

// ---- rows of at most 32 elements (classifier heads): one thread owns a row and walks it in index order,
// which is the reference's own order for the row maximum and the row sums (keydnn_reduce_cuda.cu:301-306,
// :167-179 are serial loops), and the forward divides every element by the sum as the reference does: the
// result equals the reference's kernel chain bit for bit.  LEN is the row length rounded up to 4, 8, 16 or 32;
// VEC: len % 4 == 0 and packet-aligned pointers.  Neighbouring lanes read neighbouring rows, so the 16-byte
// pieces a warp asks for in one instruction lie len*sizeof(T) apart; the other pieces of the same sectors
// follow in the next instructions and are served by L1.
template <typename T, int LEN, bool VEC, bool BWD>
__global__ void __launch_bounds__(kThreads)
softmax_thread_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t rows, int len) {
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; row < rows;
         row += static_cast<int64_t>(gridDim.x) * kThreads) {
        const T* pa = a + row * len;
        const T* pb = BWD ? b + row * len : nullptr;
        T* po = out + row * len;
        T va[LEN], vb[LEN];
        if (VEC) {
#pragma unroll
            for (int j = 0; j < LEN; j += 4) {
                if (j < len) {
                    const kd::Pack4<T> p = kd::load4(pa + j);
#pragma unroll
                    for (int k = 0; k < 4; ++k) va[j + k] = p.v[k];
                    if (BWD) {
                        const kd::Pack4<T> q = kd::load4(pb + j);
#pragma unroll
                        for (int k = 0; k < 4; ++k) vb[j + k] = q.v[k];
                    }
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < LEN; ++j) {
                if (j < len) {
                    va[j] = __ldg(pa + j);
                    if (BWD) vb[j] = __ldg(pb + j);
                }
            }
        }
        if (BWD) {
            T dot = T(0);
#pragma unroll
            for (int j = 0; j < LEN; ++j)
                if (j < len) dot = Rn<T>::add(dot, Rn<T>::mul(va[j], vb[j]));
#pragma unroll
            for (int j = 0; j < LEN; ++j)
                if (j < len) va[j] = Rn<T>::mul(vb[j], Rn<T>::sub(va[j], dot));
        } else {
            T m = neg_inf<T>();
#pragma unroll
            for (int j = 0; j < LEN; ++j)
                if (j < len) m = va[j] > m ? va[j] : m;
            T s = T(0);
#pragma unroll
            for (int j = 0; j < LEN; ++j)
                if (j < len) {
                    va[j] = t_exp(Rn<T>::sub(va[j], m));
                    s = Rn<T>::add(s, va[j]);
                }
#pragma unroll
            for (int j = 0; j < LEN; ++j)
                if (j < len) va[j] = t_div(va[j], s);
        }
        if (VEC) {
#pragma unroll
            for (int j = 0; j < LEN; j += 4) {
                if (j < len) {
                    kd::Pack4<T> p;
#pragma unroll
                    for (int k = 0; k < 4; ++k) p.v[k] = va[j + k];
                    kd::store4(po + j, p);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < LEN; ++j)
                if (j < len) po[j] = va[j];
        }
    }
}

// Same walk for rows whose pieces do not line up with 16-byte packets (len % 4 != 0 or an unaligned base): a CTA
// copies TPB consecutive rows - one
// contiguous piece of memory - into shared memory with coalesced accesses, every thread then walks its own row there
// (row pitch len | 1 words: odd, so the lanes of a warp hit 32 different banks), and the results go back the same way.
template <typename T, int LEN, int TPB, bool BWD>
__global__ void __launch_bounds__(TPB)
softmax_thread_staged_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t rows, int len,
                             kd::FastDiv by_len) {
    kd::pdl_prologue();
    extern __shared__ __align__(32) unsigned char smem_raw[];
    const int pitch = len | 1;
    T* sa = reinterpret_cast<T*>(smem_raw);
    T* sb = sa + TPB * pitch;
    const int64_t tiles = (rows + TPB - 1) / TPB;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t row0 = tile * TPB;
        const int nrows = static_cast<int>(rows - row0 < TPB ? rows - row0 : TPB);
        const int count = nrows * len;
        const T* pa = a + row0 * len;
        const T* pb = BWD ? b + row0 * len : nullptr;
        for (int i = threadIdx.x; i < count; i += TPB) {
            const unsigned r = by_len.div(static_cast<unsigned>(i));
            const int at = static_cast<int>(r) * pitch + (i - static_cast<int>(r) * len);
            sa[at] = __ldcs(pa + i);
            if (BWD) sb[at] = __ldcs(pb + i);
        }
        __syncthreads();
        if (static_cast<int>(threadIdx.x) < nrows) {
            T* ra = sa + threadIdx.x * pitch;
            const T* rb = sb + threadIdx.x * pitch;
            T va[LEN];
#pragma unroll
            for (int j = 0; j < LEN; ++j)
                if (j < len) va[j] = ra[j];
            if (BWD) {
                T dot = T(0);
#pragma unroll
                for (int j = 0; j < LEN; ++j)
                    if (j < len) dot = Rn<T>::add(dot, Rn<T>::mul(va[j], rb[j]));
#pragma unroll
                for (int j = 0; j < LEN; ++j)
                    if (j < len) ra[j] = Rn<T>::mul(rb[j], Rn<T>::sub(va[j], dot));
            } else {
                T m = neg_inf<T>();
#pragma unroll
                for (int j = 0; j < LEN; ++j)
                    if (j < len) m = va[j] > m ? va[j] : m;
                T s = T(0);
#pragma unroll
                for (int j = 0; j < LEN; ++j)
                    if (j < len) {
                        va[j] = t_exp(Rn<T>::sub(va[j], m));
                        s = Rn<T>::add(s, va[j]);
                    }
#pragma unroll
                for (int j = 0; j < LEN; ++j)
                    if (j < len) ra[j] = t_div(va[j], s);
            }
        }
        __syncthreads();
        T* po = out + row0 * len;
        for (int i = threadIdx.x; i < count; i += TPB) {
            const unsigned r = by_len.div(static_cast<unsigned>(i));
            __stcs(po + i, sa[static_cast<int>(r) * pitch + (i - static_cast<int>(r) * len)]);
        }
        __syncthreads();
    }
}

// ---- long rows: one CTA per row, operands staged in shared memory while they stream in (or re-read
// through L2 when they do not fit: `staged` false).  VEC: rows start on packet boundaries and len % 4 == 0.
template <typename T, int kBlockWarps> __device__ __forceinline__ T block_max(T v, T* sm) {
    v = group_max<T, 32>(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    T r = sm[0];
#pragma unroll
    for (int w = 1; w < kBlockWarps; ++w) r = sm[w] > r ? sm[w] : r;
    return r;
}
template <typename T, int kBlockWarps> __device__ __forceinline__ T block_add(T v, T* sm) {
    v = group_add<T, 32>(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
    __syncthreads();
    T r = sm[0];
#pragma unroll
    for (int w = 1; w < kBlockWarps; ++w) r = Rn<T>::add(r, sm[w]);
    return r;
}

template <typename T, bool BWD, bool VEC, int kBlockThreads>
__global__ void __launch_bounds__(kBlockThreads)
softmax_block_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t rows, int len,
                     bool staged) {
    kd::pdl_prologue();
    extern __shared__ __align__(32) unsigned char smem_raw[];
    T* buf = reinterpret_cast<T*>(smem_raw);          // forward: x then e;  backward: g
    T* buf2 = buf + len;                              // backward: y
    constexpr int kBlockWarps = kBlockThreads / 32;
    __shared__ T red[kBlockWarps];
    constexpr int V = VEC ? 4 : 1;
    const int step = kBlockThreads * V;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* pa = a + row * len;
        const T* pb = BWD ? b + row * len : nullptr;
        T* po = out + row * len;
        if (BWD) {
            T dot[V];
#pragma unroll
            for (int k = 0; k < V; ++k) dot[k] = T(0);
#pragma unroll 2
            for (int c = threadIdx.x * V; c < len; c += step) {
                kd::Pack4<T> g, y;
                if (VEC) {          // rows that are not staged are read again below: keep them in L2
                    g = staged ? kd::load4_stream(pa + c) : kd::load4(pa + c);
                    y = staged ? kd::load4_stream(pb + c) : kd::load4(pb + c);
                }
                else { g.v[0] = pa[c]; y.v[0] = pb[c]; }
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    dot[k] = Rn<T>::add(dot[k], Rn<T>::mul(g.v[k], y.v[k]));
                    if (staged) { buf[c + k] = g.v[k]; buf2[c + k] = y.v[k]; }
                }
            }
            T d = dot[0];
#pragma unroll
            for (int k = 1; k < V; ++k) d = Rn<T>::add(d, dot[k]);
            d = block_add<T, kBlockWarps>(d, red);
#pragma unroll 2
            for (int c = threadIdx.x * V; c < len; c += step) {
                kd::Pack4<T> r;
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    const T g = staged ? buf[c + k] : pa[c + k], y = staged ? buf2[c + k] : pb[c + k];
                    r.v[k] = Rn<T>::mul(y, Rn<T>::sub(g, d));
                }
                if (VEC) kd::store4(po + c, r);
                else po[c] = r.v[0];
            }
        } else {
            T m = neg_inf<T>();
#pragma unroll 2
            for (int c = threadIdx.x * V; c < len; c += step) {
                kd::Pack4<T> x;
                if (VEC) x = staged ? kd::load4_stream(pa + c) : kd::load4(pa + c);
                else x.v[0] = pa[c];
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    if (staged) buf[c + k] = x.v[k];
                    m = x.v[k] > m ? x.v[k] : m;
                }
            }
            m = block_max<T, kBlockWarps>(m, red);
            T s = T(0);
            for (int c = threadIdx.x * V; c < len; c += step) {
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    const T e = t_exp(Rn<T>::sub(staged ? buf[c + k] : pa[c + k], m));
                    if (staged) buf[c + k] = e;
                    s = Rn<T>::add(s, e);
                }
            }
            const T inv = t_div(T(1), block_add<T, kBlockWarps>(s, red));
            for (int c = threadIdx.x * V; c < len; c += step) {
                kd::Pack4<T> r;
#pragma unroll
                for (int k = 0; k < V; ++k)
                    r.v[k] = Rn<T>::mul(staged ? buf[c + k] : t_exp(Rn<T>::sub(pa[c + k], m)), inv);
                if (VEC) kd::store4(po + c, r);
                else po[c] = r.v[0];
            }
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
    kd::pdl_prologue();
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
            const T inv = t_div(T(1), s);
            for (int k = 0; k < len; ++k) out[base + k * inner] = Rn<T>::mul(t_exp(Rn<T>::sub(a[base + k * inner], m)), inv);
        }
    }
}

// Forward for long packet-aligned rows, the row kept in registers: every thread requests its PER packets of the row at
// once (all of the row's loads are in flight together, nothing is staged in shared memory and nothing is read twice),
// then the block maximum, the exponentials with their block sum, and the normalised row go out.  Same assignment of
// elements to threads, same order of additions and same block reductions as softmax_block_kernel: same bits.
template <typename T, int kBlockThreads, int PER>
__global__ void __launch_bounds__(kBlockThreads)
softmax_fwd_regs_kernel(const T* __restrict__ a, T* __restrict__ out, int64_t rows, int len) {
    kd::pdl_prologue();
    constexpr int kBlockWarps = kBlockThreads / 32;
    __shared__ T red[kBlockWarps];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* pa = a + row * len;
        T* po = out + row * len;
        kd::Pack4<T> x[PER];
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int c = (threadIdx.x + i * kBlockThreads) * 4;
            if (c < len) x[i] = kd::load4_stream(pa + c);
        }
        T m = neg_inf<T>();
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            if ((threadIdx.x + i * kBlockThreads) * 4 < len) {
#pragma unroll
                for (int k = 0; k < 4; ++k) m = x[i].v[k] > m ? x[i].v[k] : m;
            }
        }
        m = block_max<T, kBlockWarps>(m, red);
        T s = T(0);
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            if ((threadIdx.x + i * kBlockThreads) * 4 < len) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    x[i].v[k] = t_exp(Rn<T>::sub(x[i].v[k], m));
                    s = Rn<T>::add(s, x[i].v[k]);
                }
            }
        }
        const T inv = t_div(T(1), block_add<T, kBlockWarps>(s, red));
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int c = (threadIdx.x + i * kBlockThreads) * 4;
            if (c < len) {
#pragma unroll
                for (int k = 0; k < 4; ++k) x[i].v[k] = Rn<T>::mul(x[i].v[k], inv);
                kd::store4(po + c, x[i]);
            }
        }
    }
}

// Backward of the same rows: g and y in registers (PER packets each), dot = sum g*y with one accumulator per packet
// lane over the thread's packets in order, lanes combined, block sum; grad_x = y * (g - dot).  The arithmetic and the
// order inside a thread are those of softmax_block_kernel.
template <typename T, int kBlockThreads, int PER>
__global__ void __launch_bounds__(kBlockThreads)
softmax_bwd_regs_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t rows, int len) {
    kd::pdl_prologue();
    constexpr int kBlockWarps = kBlockThreads / 32;
    __shared__ T red[kBlockWarps];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* pa = a + row * len;
        const T* pb = b + row * len;
        T* po = out + row * len;
        kd::Pack4<T> g[PER], y[PER];
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int c = (threadIdx.x + i * kBlockThreads) * 4;
            if (c < len) { g[i] = kd::load4_stream(pa + c); y[i] = kd::load4_stream(pb + c); }
        }
        T dot[4] = {T(0), T(0), T(0), T(0)};
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            if ((threadIdx.x + i * kBlockThreads) * 4 < len) {
#pragma unroll
                for (int k = 0; k < 4; ++k) dot[k] = Rn<T>::add(dot[k], Rn<T>::mul(g[i].v[k], y[i].v[k]));
            }
        }
        T d = dot[0];
#pragma unroll
        for (int k = 1; k < 4; ++k) d = Rn<T>::add(d, dot[k]);
        d = block_add<T, kBlockWarps>(d, red);
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int c = (threadIdx.x + i * kBlockThreads) * 4;
            if (c < len) {
                kd::Pack4<T> r;
#pragma unroll
                for (int k = 0; k < 4; ++k) r.v[k] = Rn<T>::mul(y[i].v[k], Rn<T>::sub(g[i].v[k], d));
                kd::store4(po + c, r);
            }
        }
    }
}

template <typename T, int THREADS, int PER>
int launch_bwd_regs(const T* a, const T* b, T* out, int64_t rows, int len) {
    auto kernel = softmax_bwd_regs_kernel<T, THREADS, PER>;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, THREADS, 0) != cudaSuccess || per_sm < 1) per_sm = 1;
    const int64_t cap = static_cast<int64_t>(kd::sm_count()) * per_sm * 4;
    (void)kd::launch(kernel, dim3(static_cast<unsigned>(rows < cap ? rows : cap)), THREADS, 0, a, b, out, rows, len);
    return kd::launch_status();
}

template <typename T, int THREADS, int PER>
int launch_fwd_regs(const T* a, T* out, int64_t rows, int len) {
    auto kernel = softmax_fwd_regs_kernel<T, THREADS, PER>;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, THREADS, 0) != cudaSuccess || per_sm < 1) per_sm = 1;
    const int64_t cap = static_cast<int64_t>(kd::sm_count()) * per_sm * 4;
    (void)kd::launch(kernel, dim3(static_cast<unsigned>(rows < cap ? rows : cap)), THREADS, 0, a, out, rows, len);
    return kd::launch_status();
}

template <typename T, int G, int R, int K, bool BWD>
void launch_warp(const T* a, const T* b, T* out, int64_t rows, int len) {
    constexpr int RPW = (32 / G) * K;
    const int64_t trips = (rows + RPW - 1) / RPW;
    KD_LAUNCH_W((softmax_warp_kernel<T, G, R, K, BWD>), 8, (trips + kWarps - 1) / kWarps, kThreads, 0, a, b, out, rows, len);
}

// Rows are staged while at least two CTAs stay resident per SM; longer rows are re-read through L2.
template <typename T, bool BWD, bool VEC, int THREADS>
int launch_block(const T* a, const T* b, T* out, int64_t rows, int len) {
    auto kernel = softmax_block_kernel<T, BWD, VEC, THREADS>;
    constexpr size_t kMaxSmem = 100 * 1024;
    size_t smem = static_cast<size_t>(len) * sizeof(T) * (BWD ? 2 : 1);
    bool staged = smem <= kMaxSmem;
    if (staged && smem > 48 * 1024) {
        static bool opted = false;                    // per template instance
        if (!opted) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kMaxSmem)) !=
                cudaSuccess) {
                (void)cudaGetLastError();
                staged = false;
            } else {
                opted = true;
            }
        }
    }
    if (!staged) smem = 0;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, THREADS, smem) != cudaSuccess || per_sm < 1)
        per_sm = 1;
    const int64_t cap = static_cast<int64_t>(kd::sm_count()) * per_sm * 4;
    const unsigned grid = static_cast<unsigned>(rows < cap ? rows : cap);
    (void)kd::launch(kernel, dim3(grid), THREADS, smem, a, b, out, rows, len, staged);
    return kd::launch_status();
}

// CTA width: wide enough that a row gives every thread work and that the staged bytes per thread stay near
// what lets 1,536-2,048 threads share an SM's shared memory (about 112 bytes each).
template <typename T, bool BWD, bool VEC>
int launch_block_for(const T* a, const T* b, T* out, int64_t rows, int len) {
    const size_t bytes = static_cast<size_t>(len) * sizeof(T) * (BWD ? 2 : 1);
    if constexpr (BWD && VEC && sizeof(T) == 4) {
        // backward rows of up to 16384 elements: g and y in registers, two to four packets of each per thread
        if (len <= 256 * 4 * 2) return launch_bwd_regs<T, 256, 2>(a, b, out, rows, len);
        if (len <= 256 * 4 * 4) return launch_bwd_regs<T, 256, 4>(a, b, out, rows, len);
        if (len <= 512 * 4 * 4) return launch_bwd_regs<T, 512, 4>(a, b, out, rows, len);
        if (len <= 1024 * 4 * 4) return launch_bwd_regs<T, 1024, 4>(a, b, out, rows, len);
    }
    if constexpr (!BWD && VEC) {
        // rows of 1024 to 16384 elements: in registers, two to eight packets per thread
        if (len >= 1024 && len <= 512 * 4 * 8) {
            if (len <= 128 * 4 * 2) return launch_fwd_regs<T, 128, 2>(a, out, rows, len);
            if (len <= 128 * 4 * 4) return launch_fwd_regs<T, 128, 4>(a, out, rows, len);
            if (len <= 256 * 4 * 4) return launch_fwd_regs<T, 256, 4>(a, out, rows, len);
            if (len <= 512 * 4 * 4) return launch_fwd_regs<T, 512, 4>(a, out, rows, len);
            if constexpr (sizeof(T) == 4) return launch_fwd_regs<T, 512, 8>(a, out, rows, len);
        }
    }
    int threads = len <= 256 ? 32 : (len <= 512 ? 64 : 128);
    if (bytes <= 100 * 1024) {
        while (threads < 512 && static_cast<size_t>(threads) * 112 < bytes) threads *= 2;
    } else {
        threads = 1024;                                 // not staged: re-read through L2
    }
    switch (threads) {
        case 32: return launch_block<T, BWD, VEC, 32>(a, b, out, rows, len);
        case 64: return launch_block<T, BWD, VEC, 64>(a, b, out, rows, len);
        case 128: return launch_block<T, BWD, VEC, 128>(a, b, out, rows, len);
        case 256: return launch_block<T, BWD, VEC, 256>(a, b, out, rows, len);
        case 512: return launch_block<T, BWD, VEC, 512>(a, b, out, rows, len);
        default: return launch_block<T, BWD, VEC, 1024>(a, b, out, rows, len);
    }
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
    // Measured on B200 (2^27 elements): the forward pass (an exp per element between two reductions) runs faster
    // from shared memory with many small CTAs once a row has 256 elements; the backward pass stays in registers
    // up to 1024 (float) / 512 (double) elements.
    const int block_min = BWD ? (sizeof(T) == 4 ? 1025 : 513) : 256;
    if (n >= block_min) {
        const bool vec = (n % 4 == 0) && kd::aligned_pack<T>(a) && kd::aligned_pack<T>(out) && (!BWD || kd::aligned_pack<T>(b));
        return vec ? launch_block_for<T, BWD, true>(a, b, out, outer, n) : launch_block_for<T, BWD, false>(a, b, out, outer, n);
    }
    if (n <= 32) {
        const bool vec = (n % 4 == 0) && kd::aligned_pack<T>(a) && kd::aligned_pack<T>(out) && (!BWD || kd::aligned_pack<T>(b));
        const int64_t ctas = (outer + kThreads - 1) / kThreads;
#define KD_SOFTMAX_THREAD(LEN)                                                                                            \
    do {                                                                                                                  \
        KD_LAUNCH_W((softmax_thread_kernel<T, LEN, true, BWD>), 8, ctas, kThreads, 0, a, b, out, outer, n);                \
    } while (0)
#define KD_SOFTMAX_STAGED(LEN)                                                                                            \
    do {                                                                                                                  \
        constexpr int TPB = (BWD && sizeof(T) == 8) ? 64 : 128;                                                           \
        const size_t smem = static_cast<size_t>(TPB) * (n | 1) * sizeof(T) * (BWD ? 2 : 1);                               \
        KD_LAUNCH_W((softmax_thread_staged_kernel<T, LEN, TPB, BWD>), 8, (outer + TPB - 1) / TPB, TPB, smem, a, b, out,   \
                    outer, n, kd::FastDiv(static_cast<unsigned>(n)));                                                     \
    } while (0)
        if (vec) {                   // measured: packet-aligned rows are faster straight from global memory, up to 32
            if (n <= 4) KD_SOFTMAX_THREAD(4);
            else if (n <= 8) KD_SOFTMAX_THREAD(8);
            else if (n <= 16) KD_SOFTMAX_THREAD(16);
            else KD_SOFTMAX_THREAD(32);
        } else if (n <= 4) KD_SOFTMAX_STAGED(4);
        else if (n <= 8) KD_SOFTMAX_STAGED(8);
        else if (n <= 16) KD_SOFTMAX_STAGED(16);
        else KD_SOFTMAX_STAGED(32);
#undef KD_SOFTMAX_STAGED
#undef KD_SOFTMAX_THREAD
    } else if (n <= 64) launch_warp<T, 32, 2, 4, BWD>(a, b, out, outer, n);
    else if (n <= 128) launch_warp<T, 32, 4, 2, BWD>(a, b, out, outer, n);
    else if (n <= 256) launch_warp<T, 32, 8, 1, BWD>(a, b, out, outer, n);
    else if (n <= 512) launch_warp<T, 32, 16, 1, BWD>(a, b, out, outer, n);
    else if constexpr (sizeof(T) == 4) launch_warp<T, 32, 32, 1, BWD>(a, b, out, outer, n);
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
