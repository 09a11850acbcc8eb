// BatchNorm2d on (N, C, H, W) tensors, training and inference, forward and backward.
//
// The reference composes BatchNorm2d from ~25 tensor-op launches (two sum_to_shape, four
// broadcast_to, sub, mul, add, a host-side sqrt, ...) and refuses CUDA tensors altogether
// (src/keydnn/infrastructure/layers/_batchnorm.py:543-544; body :562-700).  Here the layer is
// four kernels with the same formulas:
//   forward   stats : per-channel sum and sum of squares in double -> mean, biased variance,
//                     inv_std = 1 / sqrt(var + eps) and the running-average update
//                     running = running * (1 - momentum) + batch * momentum          (:46-83)
//             apply : y = gamma * ((x - mean) * inv_std) + beta                      (:590-600)
//   backward  reduce: sum(g), sum(g * x_hat) per channel  (= dbeta, dgamma)
//             apply : dx = (1/m) * inv_std * (m*dxhat - sum(dxhat) - x_hat * sum(dxhat*x_hat)),
//                     dxhat = g * gamma                                               (:640-655)
// x_hat is recomputed from x, mean and inv_std instead of being stored.
// No counterpart in the reference's CUDA library (additive entries).
#include "common.cuh"

namespace {

using kd::Pack4;

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ bool bn_take_ticket(unsigned int* counter, unsigned int expected) {
    __shared__ bool last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = (atomicAdd(counter, 1u) == expected - 1);
    __syncthreads();
    if (last) __threadfence();
    return last;
}

// Two sums per channel over the (n, hw) extent.  F(v, w) maps an element of the first (and
// second) tensor to the two summands.  grid = (C, slices); slice s owns images [s*ach, ...).
// MODE 0: s0 = sum x, s1 = sum x*x.   MODE 1: s0 = sum g, s1 = sum g * x_hat.
// RELU: the layer output was relu(gamma * x_hat + beta) computed as z * (z > 0 ? 1 : 0); the
// upstream gradient is first multiplied by that mask, which is recomputed from x here.
template <typename T> __device__ __forceinline__ T relu_mask(T z) { return z > T(0) ? T(1) : T(0); }

__device__ __forceinline__ void load_pair(const float* p, float& a, float& b) {
    const float2 v = __ldg(reinterpret_cast<const float2*>(p));
    a = v.x; b = v.y;
}
__device__ __forceinline__ void load_pair(const double* p, double& a, double& b) {
    const double2 v = __ldg(reinterpret_cast<const double2*>(p));
    a = v.x; b = v.y;
}

// Gradient of four neighbouring elements (e .. e+3 of one input row, e % 4 == 0) of a plane that went through a
// 2x2 / stride 2 max pooling: the pooled gradient where the recorded position says so, zero elsewhere - exactly
// the values the separate pooling backward writes (`0 + go`: it accumulates onto a zeroed buffer).  `pool_go` /
// `pool_idx` are the (H/2, W/2) planes of this (n, c); positions are h * W + w.
template <typename T>
__device__ __forceinline__ Pack4<T> pooled_grad4(const T* __restrict__ pool_go, const long long* __restrict__ pool_idx,
                                                 int64_t pooled_plane_base, unsigned e, kd::FastDiv by_w) {
    const unsigned h = by_w.div(e), w0 = e - h * by_w.d;
    const int64_t at = pooled_plane_base + static_cast<int64_t>(h >> 1) * (by_w.d >> 1) + (w0 >> 1);
    // `at` is even (w0 % 4 == 0, W % 4 == 0): the two gradients and the two positions come as one access each
    T g0, g1;
    load_pair(pool_go + at, g0, g1);
    const longlong2 ii = __ldg(reinterpret_cast<const longlong2*>(pool_idx + at));
    const long long i0 = ii.x, i1 = ii.y;
    Pack4<T> r;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const long long want = (k < 2) ? i0 : i1;
        const T go = (k < 2) ? g0 : g1;
        r.v[k] = (want == static_cast<long long>(e + k)) ? T(0) + go : T(0);
    }
    return r;
}

// Where the upstream gradient of the layer output comes from:
//   0  a dense (N, C, H, W) tensor;
//   1  the (N, C, H/2, W/2) gradient and positions of a 2x2 / stride 2 max pooling of the output (pooled_grad4);
//   2  the (N, C) gradient of a global average pooling of the output: every element of plane (n, c) gets
//      g[n, c] * (1 / HW), the product the pooling backward stores (its reciprocal is rounded first).
template <typename T>
struct GradSrc {
    int mode;
    const long long* pool_idx;
    kd::FastDiv by_w;
    T gap_scale;
};

template <typename T>
__device__ __forceinline__ Pack4<T> grad4(const GradSrc<T>& gs, const T* __restrict__ g, int64_t dense_off, int64_t plane,
                                          int64_t HW, unsigned e) {
    if (gs.mode == 1) return pooled_grad4<T>(g, gs.pool_idx, plane * (HW >> 2), e, gs.by_w);
    if (gs.mode == 2) {
        const T v = __ldg(g + plane) * gs.gap_scale;
        Pack4<T> r;
        r.v[0] = r.v[1] = r.v[2] = r.v[3] = v;
        return r;
    }
    return kd::load4_stream(g + dense_off);
}

template <typename T, int MODE, bool VEC, bool RELU>
__global__ void __launch_bounds__(kThreads)
bn_channel_sums(const T* __restrict__ x, const T* __restrict__ g, const T* __restrict__ mean,
                const T* __restrict__ invstd, const T* __restrict__ gamma, const T* __restrict__ beta,
                const T* __restrict__ pre_bias, int N, int C, int64_t HW, int ach, double* partials,
                unsigned int* counters, double* sums /* [2][C] */, GradSrc<T> gsrc) {
    kd::pdl_prologue();
    __shared__ double sm[kWarps];
    const int c = blockIdx.x, slice = blockIdx.y, nslices = gridDim.y;
    const int n_begin = slice * ach;
    const int n_end = min(N, n_begin + ach);
    T mu = T(0), is = T(0), ga = T(1), be = T(0);
    const bool biased = pre_bias != nullptr;            // the layer input is x + pre_bias[c], rounded once
    const T pb = biased ? __ldg(pre_bias + c) : T(0);
    if (MODE == 1) { mu = __ldg(mean + c); is = __ldg(invstd + c); }
    if (RELU) { ga = gamma ? __ldg(gamma + c) : T(1); be = beta ? __ldg(beta + c) : T(0); }
    double a0 = 0.0, a1 = 0.0;
    for (int n = n_begin; n < n_end; ++n) {
        const int64_t base = (static_cast<int64_t>(n) * C + c) * HW;
        T p0 = T(0), p1 = T(0), q0 = T(0), q1 = T(0);      // short per-image partials in T
        if (VEC) {
            const int64_t b4 = HW >> 2;
#pragma unroll 2
            for (int64_t p = threadIdx.x; p < b4; p += kThreads) {
                Pack4<T> vx = kd::load4_stream(x + base + 4 * p);
                if (biased) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) vx.v[k] = vx.v[k] + pb;
                }
                if (MODE == 0) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (k & 1) { p1 += vx.v[k]; q1 += vx.v[k] * vx.v[k]; }
                        else { p0 += vx.v[k]; q0 += vx.v[k] * vx.v[k]; }
                    }
                } else {
                    const Pack4<T> vg = grad4<T>(gsrc, g, base + 4 * p, static_cast<int64_t>(n) * C + c, HW,
                                                 static_cast<unsigned>(4 * p));
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const T xh = (vx.v[k] - mu) * is;
                        const T gk = RELU ? vg.v[k] * relu_mask<T>(ga * xh + be) : vg.v[k];
                        if (k & 1) { p1 += gk; q1 += gk * xh; }
                        else { p0 += gk; q0 += gk * xh; }
                    }
                }
            }
        } else {
            for (int64_t b = threadIdx.x; b < HW; b += kThreads) {
                const T vx = biased ? x[base + b] + pb : x[base + b];
                if (MODE == 0) { p0 += vx; q0 += vx * vx; }
                else {
                    const T xh = (vx - mu) * is;
                    const T vg = RELU ? g[base + b] * relu_mask<T>(ga * xh + be) : g[base + b];
                    p0 += vg;
                    q0 += vg * xh;
                }
            }
        }
        a0 += static_cast<double>(p0) + static_cast<double>(p1);
        a1 += static_cast<double>(q0) + static_cast<double>(q1);
    }
    a0 = kd::block_sum(a0, sm);
    a1 = kd::block_sum(a1, sm);
    if (threadIdx.x == 0) {
        partials[(static_cast<int64_t>(slice) * C + c) * 2 + 0] = a0;
        partials[(static_cast<int64_t>(slice) * C + c) * 2 + 1] = a1;
    }
    if (bn_take_ticket(counters + c, nslices)) {
        double v0 = 0.0, v1 = 0.0;
        for (int q = threadIdx.x; q < nslices; q += kThreads) {
            v0 += __ldcg(partials + (static_cast<int64_t>(q) * C + c) * 2 + 0);
            v1 += __ldcg(partials + (static_cast<int64_t>(q) * C + c) * 2 + 1);
        }
        v0 = kd::block_sum(v0, sm);
        v1 = kd::block_sum(v1, sm);
        if (threadIdx.x == 0) {
            sums[c] = v0;
            sums[C + c] = v1;
            counters[c] = 0u;
        }
    }
}

// mean, biased variance, inv_std and the running averages, one thread per channel.
template <typename T>
__global__ void bn_finalize_stats(const double* __restrict__ sums, int C, double m, T eps, T momentum, T* mean, T* var,
                                  T* invstd, T* running_mean, T* running_var) {
    kd::pdl_prologue();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const double mu = sums[c] / m;
    double v = sums[C + c] / m - mu * mu;
    if (v < 0.0) v = 0.0;
    const T mu_t = static_cast<T>(mu), v_t = static_cast<T>(v);
    mean[c] = mu_t;
    if (var) var[c] = v_t;
    invstd[c] = T(1) / sqrt(v_t + eps);
    if (running_mean) running_mean[c] = running_mean[c] * (T(1) - momentum) + mu_t * momentum;
    if (running_var) running_var[c] = running_var[c] * (T(1) - momentum) + v_t * momentum;
}

template <typename T>
__global__ void bn_invstd_from_var(const T* __restrict__ var, int C, T eps, T* invstd) {
    kd::pdl_prologue();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < C) invstd[c] = T(1) / sqrt(var[c] + eps);
}

// y = gamma * ((x - mean) * inv_std) + beta.  blockIdx.x walks (n, c) rows of HW elements,
// blockIdx.y splits a row.
template <typename T, bool VEC, bool RELU>
__global__ void __launch_bounds__(kThreads)
bn_apply_fwd(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
             const T* __restrict__ mean, const T* __restrict__ invstd, const T* __restrict__ pre_bias, T* __restrict__ y,
             int64_t rows, int C, int64_t HW) {
    kd::pdl_prologue();
    const bool biased = pre_bias != nullptr;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const int c = static_cast<int>(r % C);
        const T mu = __ldg(mean + c), is = __ldg(invstd + c);
        const T pb = biased ? __ldg(pre_bias + c) : T(0);
        const T ga = gamma ? __ldg(gamma + c) : T(1), be = beta ? __ldg(beta + c) : T(0);
        const bool affine = gamma != nullptr;
        const T* src = x + r * HW;
        T* dst = y + r * HW;
        if (VEC) {
            const int64_t b4 = HW >> 2;
            for (int64_t p = static_cast<int64_t>(blockIdx.y) * kThreads + threadIdx.x; p < b4;
                 p += static_cast<int64_t>(gridDim.y) * kThreads) {
                Pack4<T> v = kd::load4_stream(src + 4 * p);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const T xv = biased ? v.v[k] + pb : v.v[k];
                    const T xh = (xv - mu) * is;
                    const T z = affine ? ga * xh + be : xh;
                    v.v[k] = RELU ? z * relu_mask<T>(z) : z;
                }
                kd::store4(dst + 4 * p, v);
            }
        } else {
            for (int64_t b = static_cast<int64_t>(blockIdx.y) * kThreads + threadIdx.x; b < HW;
                 b += static_cast<int64_t>(gridDim.y) * kThreads) {
                const T xv = biased ? src[b] + pb : src[b];
                const T xh = (xv - mu) * is;
                const T z = affine ? ga * xh + be : xh;
                dst[b] = RELU ? z * relu_mask<T>(z) : z;
            }
        }
    }
}

// BatchNorm apply (+ ReLU) and the 2x2 / stride 2 max pooling that follows it, in one pass: the normalised
// activation is never written.  A thread owns four adjacent windows of one output row: two rows of eight inputs
// come in as 32-byte loads, each is normalised exactly as bn_apply_fwd does, and the four maxima leave with
// their int64 positions (h * W + w; strict `>` from -inf in (0,0), (0,1), (1,0), (1,1) order, as the pooling
// kernel scans).  Needs H even, W % 8 == 0.
template <typename T, int U, bool RELU>
__global__ void __launch_bounds__(kThreads)
bn_relu_maxpool2x2_fwd(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                       const T* __restrict__ mean, const T* __restrict__ invstd, const T* __restrict__ pre_bias,
                       T* __restrict__ y, long long* __restrict__ idx, int H, int W, int Wo, int64_t groups,
                       kd::FastDiv by_gpr, kd::FastDiv by_ho, kd::FastDiv by_c) {
    kd::pdl_prologue();
    const bool affine = gamma != nullptr, biased = pre_bias != nullptr;
    const int64_t tile = static_cast<int64_t>(kThreads) * U;
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * tile; base < groups;
         base += static_cast<int64_t>(gridDim.x) * tile) {
        kd::Row8<T> top8[U], bot8[U];
        int64_t row[U];
        int jg[U], i2[U], ch[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t gi = base + u * kThreads + threadIdx.x;
            if (gi < groups) {
                unsigned rw, j4, nc, i, n_;
                by_gpr.divmod(static_cast<unsigned>(gi), rw, j4);
                by_ho.divmod(rw, nc, i);
                n_ = by_c.div(nc);
                row[u] = rw;
                jg[u] = static_cast<int>(j4);
                i2[u] = 2 * static_cast<int>(i);
                ch[u] = static_cast<int>(nc - n_ * by_c.d);
                const T* r0 = x + (static_cast<int64_t>(nc) * H + i2[u]) * W + 8 * jg[u];
                top8[u] = kd::load8_stream(r0);
                bot8[u] = kd::load8_stream(r0 + W);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t gi = base + u * kThreads + threadIdx.x;
            if (gi < groups) {
                const int c = ch[u];
                const T mu = __ldg(mean + c), is = __ldg(invstd + c);
                const T ga = affine ? __ldg(gamma + c) : T(1), be = affine ? __ldg(beta + c) : T(0);
                const T pb = biased ? __ldg(pre_bias + c) : T(0);
                T top[8], bot[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const T a = biased ? top8[u].v[k] + pb : top8[u].v[k];
                    const T b = biased ? bot8[u].v[k] + pb : bot8[u].v[k];
                    const T xa = (a - mu) * is, xb = (b - mu) * is;
                    const T za = affine ? ga * xa + be : xa, zb = affine ? ga * xb + be : xb;
                    top[k] = RELU ? za * relu_mask<T>(za) : za;
                    bot[k] = RELU ? zb * relu_mask<T>(zb) : zb;
                }
                Pack4<T> out;
                Pack4<long long> pos;
                const long long origin = static_cast<long long>(i2[u]) * W + 8 * jg[u];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    T best = -std::numeric_limits<T>::infinity();
                    long long off = 0;
                    if (top[2 * q] > best) { best = top[2 * q]; off = 0; }
                    if (top[2 * q + 1] > best) { best = top[2 * q + 1]; off = 1; }
                    if (bot[2 * q] > best) { best = bot[2 * q]; off = W; }
                    if (bot[2 * q + 1] > best) { best = bot[2 * q + 1]; off = W + 1; }
                    out.v[q] = best;
                    pos.v[q] = origin + 2 * q + off;
                }
                const int64_t o = row[u] * Wo + 4 * jg[u];
                kd::store4(y + o, out);
                kd::store4(idx + o, pos);
            }
        }
    }
}

// BatchNorm apply (+ ReLU) and the global average pooling that follows it, in one pass: a warp owns a plane, every
// lane normalises its packets as bn_apply_fwd does and adds them up exactly as the pooling kernel for long planes
// does (four running sums per lane in T, combined in double, a shuffle tree, one division by HW), so the mean has
// the bits of the two separate layers and the normalised activation is never written.  HW % 4 == 0, HW > 64.
template <typename T, bool RELU>
__global__ void __launch_bounds__(kThreads)
bn_relu_gap_fwd(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                const T* __restrict__ mean, const T* __restrict__ invstd, const T* __restrict__ pre_bias,
                T* __restrict__ y, int64_t rows, int C, int L) {
    kd::pdl_prologue();
    const bool affine = gamma != nullptr, biased = pre_bias != nullptr;
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * (kThreads / 32);
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5); r < rows; r += nwarps) {
        const int c = static_cast<int>(r % C);
        const T mu = __ldg(mean + c), is = __ldg(invstd + c);
        const T ga = affine ? __ldg(gamma + c) : T(1), be = affine ? __ldg(beta + c) : T(0);
        const T pb = biased ? __ldg(pre_bias + c) : T(0);
        const T* src = x + r * L;
        T s[4] = {T(0), T(0), T(0), T(0)};
        const int c4 = L >> 2;
        for (int p = lane; p < c4; p += 32) {
            const Pack4<T> v = kd::load4_stream(src + 4 * p);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const T xv = biased ? v.v[k] + pb : v.v[k];
                const T xh = (xv - mu) * is;
                const T z = affine ? ga * xh + be : xh;
                s[k] += RELU ? z * relu_mask<T>(z) : z;
            }
        }
        double t = (static_cast<double>(s[0]) + static_cast<double>(s[1])) + (static_cast<double>(s[2]) + static_cast<double>(s[3]));
        t = kd::warp_sum(t);
        if (lane == 0) y[r] = static_cast<T>(t) / static_cast<T>(L);
    }
}

// dx = (1/m) * inv_std * (m*dxhat - sum_dxhat - x_hat * sum_dxhat_xhat), dxhat = g * gamma;
// sums[c] = sum g, sums[C + c] = sum g * x_hat (so sum_dxhat = gamma * sums[c], ...).
template <typename T, bool VEC, bool RELU>
__global__ void __launch_bounds__(kThreads)
bn_apply_bwd(const T* __restrict__ x, const T* __restrict__ g, const T* __restrict__ gamma, const T* __restrict__ beta,
             const T* __restrict__ mean, const T* __restrict__ invstd, const T* __restrict__ pre_bias,
             const double* __restrict__ sums, T* __restrict__ dx, int64_t rows, int C, int64_t HW, T m, GradSrc<T> gsrc) {
    kd::pdl_prologue();
    const bool biased = pre_bias != nullptr;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const int c = static_cast<int>(r % C);
        const T mu = __ldg(mean + c), is = __ldg(invstd + c);
        const T pb = biased ? __ldg(pre_bias + c) : T(0);
        const T ga = gamma ? __ldg(gamma + c) : T(1);
        const T be = (RELU && beta) ? __ldg(beta + c) : T(0);
        const T s1 = static_cast<T>(sums[c]) * ga;
        const T s2 = static_cast<T>(sums[C + c]) * ga;
        const T k0 = (T(1) / m) * is;
        const T* xs = x + r * HW;
        const T* gs = g + r * HW;
        T* dst = dx + r * HW;
        if (VEC) {
            const int64_t b4 = HW >> 2;
            for (int64_t p = static_cast<int64_t>(blockIdx.y) * kThreads + threadIdx.x; p < b4;
                 p += static_cast<int64_t>(gridDim.y) * kThreads) {
                const Pack4<T> vx = kd::load4_stream(xs + 4 * p);
                const Pack4<T> vg = grad4<T>(gsrc, g, r * HW + 4 * p, r, HW, static_cast<unsigned>(4 * p));
                Pack4<T> out;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const T xv = biased ? vx.v[k] + pb : vx.v[k];
                    const T xh = (xv - mu) * is;
                    const T gk = RELU ? vg.v[k] * relu_mask<T>(ga * xh + be) : vg.v[k];
                    out.v[k] = k0 * (m * (gk * ga) - s1 - xh * s2);
                }
                kd::store4(dst + 4 * p, out);
            }
        } else {
            for (int64_t b = static_cast<int64_t>(blockIdx.y) * kThreads + threadIdx.x; b < HW;
                 b += static_cast<int64_t>(gridDim.y) * kThreads) {
                const T xv = biased ? xs[b] + pb : xs[b];
                const T xh = (xv - mu) * is;
                const T gk = RELU ? gs[b] * relu_mask<T>(ga * xh + be) : gs[b];
                dst[b] = k0 * (m * (gk * ga) - s1 - xh * s2);
            }
        }
    }
}

template <typename T>
__global__ void bn_param_grads(const double* __restrict__ sums, int C, T* dgamma, T* dbeta) {
    kd::pdl_prologue();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    if (dbeta) dbeta[c] = static_cast<T>(sums[c]);
    if (dgamma) dgamma[c] = static_cast<T>(sums[C + c]);
}

struct SumsPlan {
    int nslices, ach;
    double* partials;
    unsigned int* counters;
    double* sums;
};

// scratch layout: [2*C doubles of sums][nslices*C*2 doubles of partials]
// plane_bytes = 0: one resident wave of CTAs that hold eight per SM (the forward statistics: 32 registers).
// plane_bytes > 0: many short CTAs of about 32 KiB of x each, handed out as SMs free up - for the backward sums, whose
// registers let five CTAs share an SM, so that a grid sized for eight ran as 1.6 waves.
inline bool plan_sums(int N, int C, SumsPlan& p, int64_t plane_bytes = 0) {
    int nslices = static_cast<int>((static_cast<int64_t>(kd::sm_count()) * 8 + C - 1) / C);
    if (plane_bytes > 0) {
        const int64_t images = std::max<int64_t>(1, (32 * 1024) / plane_bytes);
        nslices = static_cast<int>(std::min<int64_t>((N + images - 1) / images, 1024));
    }
    if (nslices > N) nslices = N;
    if (nslices < 1) nslices = 1;
    p.ach = (N + nslices - 1) / nslices;
    p.nslices = (N + p.ach - 1) / p.ach;
    double* buf = static_cast<double*>(kd::scratch((static_cast<size_t>(p.nslices) + 1) * C * 2 * sizeof(double)));
    p.counters = kd::counters(C);
    if (!buf || !p.counters) return false;
    p.sums = buf;
    p.partials = buf + 2 * static_cast<size_t>(C);
    return true;
}

inline dim3 row_grid(int64_t rows, int64_t HW) {
    const int64_t cap = static_cast<int64_t>(kd::sm_count()) * 64;
    const unsigned gx = static_cast<unsigned>(rows < cap ? rows : cap);
    const int64_t per_row = (HW / 4 + kThreads - 1) / kThreads;
    int64_t gy = (cap + gx - 1) / gx;
    if (gy > per_row) gy = per_row;
    if (gy < 1) gy = 1;
    if (gy > 65535) gy = 65535;
    return dim3(gx, static_cast<unsigned>(gy));
}

template <typename T>
int bn_forward(const T* x, const T* gamma, const T* beta, T* y, T* mean, T* invstd, T* running_mean, T* running_var,
               int N, int C, int64_t HW, T eps, T momentum, int training, int relu, const T* pre_bias) {
    if (!x || !y || !mean || !invstd) return -1;
    if (N <= 0 || C <= 0 || HW <= 0) return -2;
    if ((gamma == nullptr) != (beta == nullptr)) return -3;
    if (!training && (!running_mean || !running_var)) return -4;
    (void)cudaGetLastError();
    cudaStream_t s = kd::stream();
    const bool vec = kd::aligned_pack<T>(x) && kd::aligned_pack<T>(y) && (HW % 4 == 0);
    if (training) {
        SumsPlan p;
        if (!plan_sums(N, C, p)) return static_cast<int>(cudaErrorMemoryAllocation);
        dim3 grid(C, p.nslices);
        if (vec) (void)kd::launch(bn_channel_sums<T, 0, true, false>, dim3(grid), kThreads, 0, x, nullptr, nullptr, nullptr, nullptr, nullptr, pre_bias, N, C, HW, p.ach, p.partials, p.counters, p.sums, GradSrc<T>{0, nullptr, kd::FastDiv(), T(0)});
        else (void)kd::launch(bn_channel_sums<T, 0, false, false>, dim3(grid), kThreads, 0, x, nullptr, nullptr, nullptr, nullptr, nullptr, pre_bias, N, C, HW, p.ach, p.partials, p.counters, p.sums, GradSrc<T>{0, nullptr, kd::FastDiv(), T(0)});
        (void)kd::launch(bn_finalize_stats<T>, dim3((C + 127) / 128), 128, 0, p.sums, C, static_cast<double>(N) * static_cast<double>(HW), eps,
                                                          momentum, mean, static_cast<T*>(nullptr), invstd, running_mean,
                                                          running_var);
    } else {
        (void)kd::launch(bn_invstd_from_var<T>, dim3((C + 127) / 128), 128, 0, running_var, C, eps, invstd);
        cudaMemcpyAsync(mean, running_mean, C * sizeof(T), cudaMemcpyDeviceToDevice, s);
    }
    const int64_t rows = static_cast<int64_t>(N) * C;
    const dim3 g2 = row_grid(rows, HW);
    if (relu) {
        if (vec) (void)kd::launch(bn_apply_fwd<T, true, true>, dim3(g2), kThreads, 0, x, gamma, beta, mean, invstd, pre_bias, y, rows, C, HW);
        else (void)kd::launch(bn_apply_fwd<T, false, true>, dim3(g2), kThreads, 0, x, gamma, beta, mean, invstd, pre_bias, y, rows, C, HW);
    } else {
        if (vec) (void)kd::launch(bn_apply_fwd<T, true, false>, dim3(g2), kThreads, 0, x, gamma, beta, mean, invstd, pre_bias, y, rows, C, HW);
        else (void)kd::launch(bn_apply_fwd<T, false, false>, dim3(g2), kThreads, 0, x, gamma, beta, mean, invstd, pre_bias, y, rows, C, HW);
    }
    return kd::launch_status();
}

// Statistics as bn_forward, then the fused apply + ReLU + pooling kernel.  -6: geometry the fused kernel does not take.
template <typename T>
int bn_pool_forward(const T* x, const T* gamma, const T* beta, T* y_pool, long long* idx, T* mean, T* invstd,
                    T* running_mean, T* running_var, int N, int C, int H, int W, T eps, T momentum, int training, int relu,
                    const T* pre_bias) {
    if (!x || !y_pool || !idx || !mean || !invstd) return -1;
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0) return -2;
    if ((gamma == nullptr) != (beta == nullptr)) return -3;
    if (!training && (!running_mean || !running_var)) return -4;
    const int64_t HW = static_cast<int64_t>(H) * W;
    const int64_t total = static_cast<int64_t>(N) * C * (HW / 4);
    if ((H & 1) || (W % 8) || !kd::aligned_row8<T>(x) || !kd::aligned_pack<T>(y_pool) || !kd::aligned_pack<long long>(idx) ||
        total >= (int64_t(1) << 32))
        return -6;
    (void)cudaGetLastError();
    cudaStream_t s = kd::stream();
    if (training) {
        SumsPlan p;
        if (!plan_sums(N, C, p)) return static_cast<int>(cudaErrorMemoryAllocation);
        dim3 grid(C, p.nslices);
        (void)kd::launch(bn_channel_sums<T, 0, true, false>, dim3(grid), kThreads, 0, x, nullptr, nullptr, nullptr, nullptr, nullptr,
                         pre_bias, N, C, HW, p.ach, p.partials, p.counters, p.sums, GradSrc<T>{0, nullptr, kd::FastDiv(), T(0)});
        (void)kd::launch(bn_finalize_stats<T>, dim3((C + 127) / 128), 128, 0, p.sums, C, static_cast<double>(N) * static_cast<double>(HW),
                         eps, momentum, mean, static_cast<T*>(nullptr), invstd, running_mean, running_var);
    } else {
        (void)kd::launch(bn_invstd_from_var<T>, dim3((C + 127) / 128), 128, 0, running_var, C, eps, invstd);
        cudaMemcpyAsync(mean, running_mean, C * sizeof(T), cudaMemcpyDeviceToDevice, s);
    }
    constexpr int U = 2;
    const int Ho = H / 2, Wo = W / 2;
    const int64_t groups = total >> 2;
    const int64_t work = (groups + kThreads * U - 1) / (kThreads * U);
    if (relu) KD_LAUNCH((bn_relu_maxpool2x2_fwd<T, U, true>), work, kThreads, 0, x, gamma, beta, mean, invstd, pre_bias, y_pool, idx,
                        H, W, Wo, groups, kd::FastDiv(Wo / 4), kd::FastDiv(Ho), kd::FastDiv(C));
    else KD_LAUNCH((bn_relu_maxpool2x2_fwd<T, U, false>), work, kThreads, 0, x, gamma, beta, mean, invstd, pre_bias, y_pool, idx,
                   H, W, Wo, groups, kd::FastDiv(Wo / 4), kd::FastDiv(Ho), kd::FastDiv(C));
    return kd::launch_status();
}

// Statistics as bn_forward, then the fused apply + ReLU + global average pooling kernel.
template <typename T>
int bn_gap_forward(const T* x, const T* gamma, const T* beta, T* y_gap, T* mean, T* invstd, T* running_mean, T* running_var,
                   int N, int C, int64_t HW, T eps, T momentum, int training, int relu, const T* pre_bias) {
    if (!x || !y_gap || !mean || !invstd) return -1;
    if (N <= 0 || C <= 0 || HW <= 0) return -2;
    if ((gamma == nullptr) != (beta == nullptr)) return -3;
    if (!training && (!running_mean || !running_var)) return -4;
    if (HW % 4 != 0 || HW <= 64 || HW > std::numeric_limits<int>::max() || !kd::aligned_pack<T>(x)) return -6;
    (void)cudaGetLastError();
    cudaStream_t s = kd::stream();
    if (training) {
        SumsPlan p;
        if (!plan_sums(N, C, p)) return static_cast<int>(cudaErrorMemoryAllocation);
        dim3 grid(C, p.nslices);
        (void)kd::launch(bn_channel_sums<T, 0, true, false>, dim3(grid), kThreads, 0, x, nullptr, nullptr, nullptr, nullptr, nullptr,
                         pre_bias, N, C, HW, p.ach, p.partials, p.counters, p.sums, GradSrc<T>{0, nullptr, kd::FastDiv(), T(0)});
        (void)kd::launch(bn_finalize_stats<T>, dim3((C + 127) / 128), 128, 0, p.sums, C, static_cast<double>(N) * static_cast<double>(HW),
                         eps, momentum, mean, static_cast<T*>(nullptr), invstd, running_mean, running_var);
    } else {
        (void)kd::launch(bn_invstd_from_var<T>, dim3((C + 127) / 128), 128, 0, running_var, C, eps, invstd);
        cudaMemcpyAsync(mean, running_mean, C * sizeof(T), cudaMemcpyDeviceToDevice, s);
    }
    const int64_t rows = static_cast<int64_t>(N) * C;
    const unsigned grid = kd::grid_for((rows + 7) / 8, 8);
    if (relu) (void)kd::launch(bn_relu_gap_fwd<T, true>, dim3(grid), kThreads, 0, x, gamma, beta, mean, invstd, pre_bias, y_gap, rows, C,
                               static_cast<int>(HW));
    else (void)kd::launch(bn_relu_gap_fwd<T, false>, dim3(grid), kThreads, 0, x, gamma, beta, mean, invstd, pre_bias, y_gap, rows, C,
                          static_cast<int>(HW));
    return kd::launch_status();
}

template <typename T>
int bn_backward(const T* x, const T* gamma, const T* beta, const T* go, const T* mean, const T* invstd, T* dx, T* dgamma,
                T* dbeta, int N, int C, int64_t HW, int relu, const T* pre_bias, const long long* pool_idx = nullptr,
                int W = 0, bool gap = false) {
    if (!x || !go || !mean || !invstd || !dx) return -1;
    if (N <= 0 || C <= 0 || HW <= 0) return -2;
    (void)cudaGetLastError();
    cudaStream_t s = kd::stream();
    bool vec = kd::aligned_pack<T>(x) && kd::aligned_pack<T>(dx) && (HW % 4 == 0);
    kd::FastDiv by_w;
    if (pool_idx) {
        // `go` and `pool_idx` are the (H/2, W/2) planes behind a 2x2 / stride 2 max pooling of this layer's output
        if (W <= 0 || W % 4 != 0 || HW % W != 0 || ((HW / W) & 1) || HW >= (int64_t(1) << 32) || !vec) return -6;
        if ((reinterpret_cast<uintptr_t>(go) & (2 * sizeof(T) - 1)) || (reinterpret_cast<uintptr_t>(pool_idx) & 15u)) return -6;
        by_w = kd::FastDiv(static_cast<unsigned>(W));
    } else if (gap) {
        if (!vec || HW >= (int64_t(1) << 32)) return -6;        // `go` is the (N, C) gradient behind a global average pooling
    } else {
        vec = vec && kd::aligned_pack<T>(go);
    }
    const GradSrc<T> gsrc{pool_idx ? 1 : (gap ? 2 : 0), pool_idx, by_w, T(1) / static_cast<T>(HW)};
    SumsPlan p;
    if (!plan_sums(N, C, p, HW * static_cast<int64_t>(sizeof(T)))) return static_cast<int>(cudaErrorMemoryAllocation);
    dim3 grid(C, p.nslices);
#define KD_BN_SUMS(V, R) (void)kd::launch(bn_channel_sums<T, 1, V, R>, dim3(grid), kThreads, 0, x, go, mean, invstd, gamma, beta, pre_bias, N, C, HW, p.ach, p.partials, p.counters, p.sums, gsrc)
    if (relu) { if (vec) KD_BN_SUMS(true, true); else KD_BN_SUMS(false, true); }
    else { if (vec) KD_BN_SUMS(true, false); else KD_BN_SUMS(false, false); }
#undef KD_BN_SUMS
    if (dgamma || dbeta) (void)kd::launch(bn_param_grads<T>, dim3((C + 127) / 128), 128, 0, p.sums, C, dgamma, dbeta);
    const int64_t rows = static_cast<int64_t>(N) * C;
    const dim3 g2 = row_grid(rows, HW);
    const T m = static_cast<T>(static_cast<double>(N) * static_cast<double>(HW));
#define KD_BN_APPLY(V, R) (void)kd::launch(bn_apply_bwd<T, V, R>, dim3(g2), kThreads, 0, x, go, gamma, beta, mean, invstd, pre_bias, p.sums, dx, rows, C, HW, m, gsrc)
    if (relu) { if (vec) KD_BN_APPLY(true, true); else KD_BN_APPLY(false, true); }
    else { if (vec) KD_BN_APPLY(true, false); else KD_BN_APPLY(false, false); }
#undef KD_BN_APPLY
    return kd::launch_status();
}

}  // namespace

// `relu` != 0 fuses the activation that follows the layer in a Conv-BN-ReLU stack: forward writes
// z * (z > 0 ? 1 : 0) with z = gamma * x_hat + beta (the reference's mask-and-multiply ReLU,
// _function.py:291-293, bit for bit), backward multiplies grad_out by the same mask, recomputed from x.
KD_API int keydnn_cuda_bn2d_forward_f32(const float* x, const float* gamma, const float* beta, float* y, float* mean,
                                        float* invstd, float* running_mean, float* running_var, int N, int C, int64_t HW,
                                        float eps, float momentum, int training, int relu) {
    return bn_forward<float>(x, gamma, beta, y, mean, invstd, running_mean, running_var, N, C, HW, eps, momentum, training,
                             relu, nullptr);
}
KD_API int keydnn_cuda_bn2d_forward_f64(const double* x, const double* gamma, const double* beta, double* y, double* mean,
                                        double* invstd, double* running_mean, double* running_var, int N, int C,
                                        int64_t HW, double eps, double momentum, int training, int relu) {
    return bn_forward<double>(x, gamma, beta, y, mean, invstd, running_mean, running_var, N, C, HW, eps, momentum, training,
                              relu, nullptr);
}
KD_API int keydnn_cuda_bn2d_backward_f32(const float* x, const float* gamma, const float* beta, const float* grad_out,
                                         const float* mean, const float* invstd, float* grad_x, float* grad_gamma,
                                         float* grad_beta, int N, int C, int64_t HW, int relu) {
    return bn_backward<float>(x, gamma, beta, grad_out, mean, invstd, grad_x, grad_gamma, grad_beta, N, C, HW, relu, nullptr);
}
KD_API int keydnn_cuda_bn2d_backward_f64(const double* x, const double* gamma, const double* beta, const double* grad_out,
                                         const double* mean, const double* invstd, double* grad_x, double* grad_gamma,
                                         double* grad_beta, int N, int C, int64_t HW, int relu) {
    return bn_backward<double>(x, gamma, beta, grad_out, mean, invstd, grad_x, grad_gamma, grad_beta, N, C, HW, relu, nullptr);
}

// The layer in front adds a per-channel bias (a convolution's): `pre_bias` (C values) is added to every element of x
// as it is read - one rounded addition, what the separate bias pass would have stored - so that pass and its
// read + write of the whole activation disappear.  Statistics, output and gradients are those of x + pre_bias.
#define KD_BN_BIAS_EXPORTS(T, SUF)                                                                                      \
    KD_API int keydnn_cuda_bn2d_forward_bias_##SUF(const T* x, const T* pre_bias, const T* gamma, const T* beta, T* y,   \
                                                   T* mean, T* invstd, T* running_mean, T* running_var, int N, int C,    \
                                                   int64_t HW, T eps, T momentum, int training, int relu) {              \
        return bn_forward<T>(x, gamma, beta, y, mean, invstd, running_mean, running_var, N, C, HW, eps, momentum,        \
                             training, relu, pre_bias);                                                                  \
    }                                                                                                                    \
    KD_API int keydnn_cuda_bn2d_backward_bias_##SUF(const T* x, const T* pre_bias, const T* gamma, const T* beta,        \
                                                    const T* grad_out, const T* mean, const T* invstd, T* grad_x,        \
                                                    T* grad_gamma, T* grad_beta, int N, int C, int64_t HW, int relu) {   \
        return bn_backward<T>(x, gamma, beta, grad_out, mean, invstd, grad_x, grad_gamma, grad_beta, N, C, HW, relu,     \
                              pre_bias);                                                                                 \
    }
KD_BN_BIAS_EXPORTS(float, f32)
KD_BN_BIAS_EXPORTS(double, f64)

// BatchNorm2d (+ ReLU) followed by MaxPool2d(2): forward writes only the pooled tensor and its int64 positions
// (h * W + w, the pooling kernels' encoding); backward takes the gradient of the pooled tensor and those positions
// and derives each element's gradient on the fly.  Same bits as the separate layers; the (N, C, H, W) activation and
// its gradient are never stored.  H even, W a multiple of 8 (else -6: use the separate entries).
#define KD_BN_POOL_EXPORTS(T, SUF)                                                                                      \
    KD_API int keydnn_cuda_bn2d_maxpool2x2_forward_##SUF(const T* x, const T* pre_bias, const T* gamma, const T* beta,   \
                                                         T* y_pool, int64_t* argmax_idx, T* mean, T* invstd,             \
                                                         T* running_mean, T* running_var, int N, int C, int H, int W,    \
                                                         T eps, T momentum, int training, int relu) {                    \
        return bn_pool_forward<T>(x, gamma, beta, y_pool, reinterpret_cast<long long*>(argmax_idx), mean, invstd,        \
                                  running_mean, running_var, N, C, H, W, eps, momentum, training, relu, pre_bias);       \
    }                                                                                                                    \
    KD_API int keydnn_cuda_bn2d_maxpool2x2_backward_##SUF(const T* x, const T* pre_bias, const T* gamma, const T* beta,  \
                                                          const T* grad_pool, const int64_t* argmax_idx, const T* mean,  \
                                                          const T* invstd, T* grad_x, T* grad_gamma, T* grad_beta,       \
                                                          int N, int C, int H, int W, int relu) {                        \
        if (!argmax_idx) return -1;                                                                                      \
        if (H <= 0 || W <= 0 || (H & 1)) return -6;                                                                      \
        return bn_backward<T>(x, gamma, beta, grad_pool, mean, invstd, grad_x, grad_gamma, grad_beta, N, C,              \
                              static_cast<int64_t>(H) * W, relu, pre_bias,                                               \
                              reinterpret_cast<const long long*>(argmax_idx), W);                                        \
    }
KD_BN_POOL_EXPORTS(float, f32)
KD_BN_POOL_EXPORTS(double, f64)

// BatchNorm2d (+ ReLU) followed by GlobalAvgPool2d: forward writes only the (N, C) means, backward takes their
// gradient; every element of plane (n, c) receives grad[n, c] * (1 / HW) as the pooling backward would have stored it.
// Same bits as the separate layers.  HW a multiple of 4 and above 64, else -6 (use the separate entries).
#define KD_BN_GAP_EXPORTS(T, SUF)                                                                                        \
    KD_API int keydnn_cuda_bn2d_global_avgpool_forward_##SUF(const T* x, const T* pre_bias, const T* gamma, const T* beta, \
                                                             T* y_mean, T* mean, T* invstd, T* running_mean,              \
                                                             T* running_var, int N, int C, int64_t HW, T eps, T momentum, \
                                                             int training, int relu) {                                    \
        return bn_gap_forward<T>(x, gamma, beta, y_mean, mean, invstd, running_mean, running_var, N, C, HW, eps, momentum, \
                                 training, relu, pre_bias);                                                               \
    }                                                                                                                     \
    KD_API int keydnn_cuda_bn2d_global_avgpool_backward_##SUF(const T* x, const T* pre_bias, const T* gamma,              \
                                                              const T* beta, const T* grad_mean, const T* mean,           \
                                                              const T* invstd, T* grad_x, T* grad_gamma, T* grad_beta,    \
                                                              int N, int C, int64_t HW, int relu) {                       \
        return bn_backward<T>(x, gamma, beta, grad_mean, mean, invstd, grad_x, grad_gamma, grad_beta, N, C, HW, relu,     \
                              pre_bias, nullptr, 0, true);                                                                \
    }
KD_BN_GAP_EXPORTS(float, f32)
KD_BN_GAP_EXPORTS(double, f64)
