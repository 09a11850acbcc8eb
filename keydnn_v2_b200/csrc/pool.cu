// 2-D pooling on NCHW planes: MaxPool2d, AvgPool2d, GlobalAvgPool2d (forward and
// backward), plus the pad2d / crop2d passes the reference runs around them.
//
// Reference kernels replaced (all one element per thread, 4-byte accesses,
// N*C planes in gridDim.z, which stops at 65,535 planes):
//   KeyDNNV2CudaNative/kernel.cu:97-185               max forward / backward
//   keydnn_avgpool2d_cuda.cu:55-92, 143-198           avg forward / gather backward
//   keydnn_global_avgpool2d_cuda.cu:32-97             global average
//   keydnn_pad2d_cuda.cu:30-97                        pad / crop
//
// Two entry styles are exported:
//   * the reference signatures (pre-padded planes; backward accumulates into a
//     caller-zeroed padded buffer), and
//   * `_ex` entries that take the un-padded tensor with explicit padding, so the
//     pad pass before and the memset + crop passes after disappear: forward
//     treats out-of-range taps as the pad value, backward writes every element of
//     the un-padded gradient exactly once.
// Planes are flattened into the x dimension of a grid-stride loop, so any
// N*C works.
#include "common.cuh"

namespace {

using kd::Pack4;

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

struct PoolGeom {
    int H, W;        // un-padded input plane
    int Ho, Wo;      // output plane
    int kh, kw, sh, sw;
    int ph, pw;      // symmetric zero / -inf padding
};

// ===========================================================================
// MaxPool
// ===========================================================================
// Selection rule (kernel.cu:122-145): best starts at -inf and the recorded
// position at the window origin; taps are scanned row-major and replace the best
// only when strictly greater.  NaN therefore never wins, ties keep the first
// tap, and a window without any tap above -inf reports (-inf, origin).  Taps
// that fall into the padding hold -inf in the reference and can never win, so
// they are skipped here.  The index is h*W_pad + w in the padded plane.

template <typename T>
__global__ void __launch_bounds__(kThreads)
maxpool_fwd_generic(const T* __restrict__ x, T* __restrict__ y, long long* __restrict__ idx, PoolGeom g,
                    int64_t total) {
    kd::pdl_prologue();
    const int Wp = g.W + 2 * g.pw;
    for (int64_t o = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; o < total;
         o += static_cast<int64_t>(gridDim.x) * kThreads) {
        const int j = static_cast<int>(o % g.Wo);
        const int64_t t = o / g.Wo;
        const int i = static_cast<int>(t % g.Ho);
        const int64_t nc = t / g.Ho;
        const T* plane = x + nc * g.H * g.W;
        const int hp0 = i * g.sh, wp0 = j * g.sw;
        T best = kd::neg_inf<T>();
        int bh = hp0, bw = wp0;
        for (int a = 0; a < g.kh; ++a) {
            const int h = hp0 + a - g.ph;
            if (h < 0 || h >= g.H) continue;
            for (int b = 0; b < g.kw; ++b) {
                const int w = wp0 + b - g.pw;
                if (w < 0 || w >= g.W) continue;
                const T v = __ldg(plane + static_cast<int64_t>(h) * g.W + w);
                if (v > best) { best = v; bh = hp0 + a; bw = wp0 + b; }
            }
        }
        y[o] = best;
        idx[o] = static_cast<long long>(bh) * Wp + bw;
    }
}

// kernel 2x2, stride 2, no padding, W % 8 == 0.  A thread owns four adjacent
// windows: two rows of eight inputs come in as four 16-byte loads, the four
// maxima leave as one 16-byte store and the four int64 positions as two.
template <typename T, int U>
__global__ void __launch_bounds__(kThreads)
maxpool2x2_fwd(const T* __restrict__ x, T* __restrict__ y, long long* __restrict__ idx, int H, int W, int Ho, int Wo,
               int64_t groups, kd::FastDiv by_gpr, kd::FastDiv by_ho) {
    kd::pdl_prologue();
    const int64_t tile = static_cast<int64_t>(kThreads) * U;
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * tile; base < groups;
         base += static_cast<int64_t>(gridDim.x) * tile) {
        kd::Row8<T> top8[U], bot8[U];
        int64_t row[U];
        int jg[U], i2[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t gi = base + u * kThreads + threadIdx.x;
            if (gi < groups) {
                unsigned rw, j4, nc, i;
                by_gpr.divmod(static_cast<unsigned>(gi), rw, j4);     // groups < 2^31 (checked by the launcher)
                by_ho.divmod(rw, nc, i);
                row[u] = rw;
                jg[u] = static_cast<int>(j4);
                i2[u] = 2 * static_cast<int>(i);
                const T* r0 = x + (static_cast<int64_t>(nc) * H + i2[u]) * W + 8 * jg[u];
                top8[u] = kd::load8_stream(r0);
                bot8[u] = kd::load8_stream(r0 + W);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t gi = base + u * kThreads + threadIdx.x;
            if (gi < groups) {
                const T* top = top8[u].v;
                const T* bot = bot8[u].v;
                Pack4<T> out;
                Pack4<long long> pos;
                const long long origin = static_cast<long long>(i2[u]) * W + 8 * jg[u];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    T best = kd::neg_inf<T>();
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

// Backward for kernel 2x2, stride 2, no padding, H even, W % 8 == 0: windows tile the plane.
// A thread owns eight adjacent gradient elements of ONE input row (one 32-byte store), so a
// warp writes one contiguous kilobyte and the grid writes the tensor front to back; the four
// windows above/below them come in as one packet of grad_out and one of positions (the thread
// of the neighbouring row reads the same two packets: an L1 hit).  The routed value lands
// where the recorded position says, zero elsewhere: no memset, no atomics.  `0 + go`
// reproduces the reference's accumulation onto a zeroed buffer (it turns -0 into +0).
template <typename T, int U>
__global__ void __launch_bounds__(kThreads)
maxpool2x2_bwd(const T* __restrict__ go, const long long* __restrict__ idx, T* __restrict__ gx, int H, int W, int Ho,
               int Wo, int64_t blocks, kd::FastDiv by_bpr, kd::FastDiv by_h) {
    kd::pdl_prologue();
    const int64_t tile = static_cast<int64_t>(kThreads) * U;
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * tile; base < blocks;
         base += static_cast<int64_t>(gridDim.x) * tile) {
        Pack4<T> gv[U];
        Pack4<long long> pv[U];
        long long want[U];      // position of this thread's first element inside the plane
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t bi = base + u * kThreads + threadIdx.x;
            if (bi < blocks) {
                unsigned rowflat, jg, nc, h;                      // rowflat = nc * H + h
                by_bpr.divmod(static_cast<unsigned>(bi), rowflat, jg);
                by_h.divmod(rowflat, nc, h);
                const int64_t o = (static_cast<int64_t>(nc) * Ho + (h >> 1)) * Wo + 4 * jg;
                gv[u] = kd::load4(go + o);
                pv[u] = kd::load4(idx + o);
                want[u] = static_cast<long long>(h) * W + 8 * jg;
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t bi = base + u * kThreads + threadIdx.x;
            if (bi < blocks) {
                kd::Row8<T> out;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const T g = T(0) + gv[u].v[q];
                    const long long off = pv[u].v[q] - want[u];
                    out.v[2 * q] = (off == 2 * q) ? g : T(0);
                    out.v[2 * q + 1] = (off == 2 * q + 1) ? g : T(0);
                }
                kd::store8(gx + 8 * bi, out);
            }
        }
    }
}

// kernel 3x3, stride 2, padding 1, W % 8 == 0: the register layout of avgpool3x3s2p1_fwd (four adjacent outputs per
// thread, three rows of eight aligned inputs plus the one left of them) with the selection rule above.  A tap in the
// padding is held as -inf, which can never replace the best.
// (fp32: six CTAs per SM, which costs two spilled registers and gains 8 % - the kernel waits on its loads.)
template <typename T>
__global__ void __launch_bounds__(kThreads, sizeof(T) == 4 ? 6 : 1)
maxpool3x3s2p1_fwd(const T* __restrict__ x, T* __restrict__ y, long long* __restrict__ idx, int H, int W, int Ho, int Wo,
                   int64_t groups, kd::FastDiv by_gpr, kd::FastDiv by_ho) {
    kd::pdl_prologue();
    const int Wp = W + 2;
    for (int64_t gi = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; gi < groups;
         gi += static_cast<int64_t>(gridDim.x) * kThreads) {
        unsigned row, ujg, nc, ui;
        by_gpr.divmod(static_cast<unsigned>(gi), row, ujg);
        by_ho.divmod(row, nc, ui);
        const int jg = static_cast<int>(ujg), i = static_cast<int>(ui);
        const T* plane = x + static_cast<int64_t>(nc) * H * W;
        T c[3][9];
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            const int h = 2 * i - 1 + r;
            if (h >= 0 && h < H) {
                const T* p = plane + static_cast<int64_t>(h) * W + 8 * jg;
                const kd::Row8<T> a = kd::load8(p);
                c[r][0] = jg > 0 ? __ldg(p - 1) : kd::neg_inf<T>();
#pragma unroll
                for (int k = 0; k < 8; ++k) c[r][1 + k] = a.v[k];
            } else {
#pragma unroll
                for (int k = 0; k < 9; ++k) c[r][k] = kd::neg_inf<T>();
            }
        }
        Pack4<T> out;
        Pack4<long long> pos;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            T best = kd::neg_inf<T>();
            int bt = 0;                                            // a * 4 + b of the best tap
#pragma unroll
            for (int r = 0; r < 3; ++r)
#pragma unroll
                for (int b = 0; b < 3; ++b) {
                    const T v = c[r][2 * q + b];
                    if (v > best) { best = v; bt = r * 4 + b; }
                }
            out.v[q] = best;
            pos.v[q] = static_cast<long long>(2 * i + (bt >> 2)) * Wp + (2 * (4 * jg + q) + (bt & 3));
        }
        kd::store4(y + static_cast<int64_t>(row) * Wo + 4 * jg, out);
        kd::store4(idx + static_cast<int64_t>(row) * Wo + 4 * jg, pos);
    }
}

// Backward of the same geometry: the 2x8 block of gradient rows (2m, 2m+1) x [8jg, 8jg+8) per thread, as in
// avgpool3x3s2p1_bwd.  Each of the ten windows that touch the block (five per output row) is reduced to
// tap = recorded position - position of the window origin (a * Wp + b for a position inside the window, -1 otherwise);
// an element takes the gradient of a covering window when the tap is the element's own offset in that window.
// Windows are visited in ascending (i, j) as in maxpool_bwd_gather.
template <typename T>
__global__ void __launch_bounds__(kThreads)
maxpool3x3s2p1_bwd(const T* __restrict__ go, const long long* __restrict__ idx, T* __restrict__ gx, int H, int W, int Ho, int Wo,
                   int64_t blocks, kd::FastDiv by_bpr, kd::FastDiv by_hh) {
    kd::pdl_prologue();
    const int Wp = W + 2;
    for (int64_t bi = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; bi < blocks;
         bi += static_cast<int64_t>(gridDim.x) * kThreads) {
        unsigned rowp, ujg, nc, um;                    // rowp = nc * ceil(H/2) + m
        by_bpr.divmod(static_cast<unsigned>(bi), rowp, ujg);
        by_hh.divmod(rowp, nc, um);
        const int jg = static_cast<int>(ujg), m = static_cast<int>(um);
        const int64_t p0 = (static_cast<int64_t>(nc) * Ho + m) * Wo + 4 * jg;
        const bool has_fifth = 4 * jg + 4 < Wo;        // the fifth window exists
        const bool second = m + 1 < Ho;                // output row m+1 exists
        T g[2][5];
        int tap[2][5];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const bool live = r == 0 || second;
            Pack4<T> a;
            Pack4<long long> p;
            a.v[0] = a.v[1] = a.v[2] = a.v[3] = T(0);
            p.v[0] = p.v[1] = p.v[2] = p.v[3] = -1;
            T e = T(0);
            long long pe = -1;
            if (live) {
                a = kd::load4(go + p0 + r * Wo);
                p = kd::load4(idx + p0 + r * Wo);
                if (has_fifth) { e = __ldg(go + p0 + r * Wo + 4); pe = __ldg(idx + p0 + r * Wo + 4); }
            }
            const long long origin = static_cast<long long>(2 * (m + r)) * Wp + 8 * jg;      // of the first window
#pragma unroll
            for (int k = 0; k < 5; ++k) {
                const long long d = (k < 4 ? p.v[k] : pe) - (origin + 2 * k);
                g[r][k] = k < 4 ? a.v[k] : e;
                tap[r][k] = (d >= 0 && d < 3 * static_cast<long long>(Wp)) ? static_cast<int>(d) : -1;
            }
            if (!live || !has_fifth) tap[r][4] = -1;
            if (!live) {
#pragma unroll
                for (int k = 0; k < 4; ++k) tap[r][k] = -1;
            }
        }
        T* r0 = gx + (static_cast<int64_t>(nc) * H + 2 * m) * W + 8 * jg;
        {   // row 2m (padded row 2m+1): a = 1 in output row m
            kd::Row8<T> out;
#pragma unroll
            for (int cidx = 0; cidx < 8; ++cidx) {
                const int k = cidx >> 1;
                T acc = T(0);
                if (cidx & 1) {
                    acc += tap[0][k] == Wp + 2 ? g[0][k] : T(0);
                    acc += tap[0][k + 1] == Wp ? g[0][k + 1] : T(0);
                } else {
                    acc += tap[0][k] == Wp + 1 ? g[0][k] : T(0);
                }
                out.v[cidx] = acc;
            }
            kd::store8(r0, out);
        }
        if (2 * m + 1 < H) {   // row 2m+1 (padded row 2m+2): a = 2 in output row m, a = 0 in output row m+1
            kd::Row8<T> out;
#pragma unroll
            for (int cidx = 0; cidx < 8; ++cidx) {
                const int k = cidx >> 1;
                T acc = T(0);
                if (cidx & 1) {
                    acc += tap[0][k] == 2 * Wp + 2 ? g[0][k] : T(0);
                    acc += tap[0][k + 1] == 2 * Wp ? g[0][k + 1] : T(0);
                    acc += tap[1][k] == 2 ? g[1][k] : T(0);
                    acc += tap[1][k + 1] == 0 ? g[1][k + 1] : T(0);
                } else {
                    acc += tap[0][k] == 2 * Wp + 1 ? g[0][k] : T(0);
                    acc += tap[1][k] == 1 ? g[1][k] : T(0);
                }
                out.v[cidx] = acc;
            }
            kd::store8(r0 + W, out);
        }
    }
}

// Any geometry: one thread per un-padded input element gathers, in ascending
// (i, j) order, the gradients of the windows that recorded it.  Writes every
// element once.  (The reference sums overlapping windows with float atomics in
// arbitrary order, kernel.cu:173-184, so only non-overlapping results are
// bit-comparable.)
template <typename T>
__global__ void __launch_bounds__(kThreads)
maxpool_bwd_gather(const T* __restrict__ go, const long long* __restrict__ idx, T* __restrict__ gx, PoolGeom g,
                   int64_t total) {
    kd::pdl_prologue();
    const int Wp = g.W + 2 * g.pw;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; e < total;
         e += static_cast<int64_t>(gridDim.x) * kThreads) {
        const int w = static_cast<int>(e % g.W);
        const int64_t t = e / g.W;
        const int h = static_cast<int>(t % g.H);
        const int64_t nc = t / g.H;
        const int hp = h + g.ph, wp = w + g.pw;
        const long long target = static_cast<long long>(hp) * Wp + wp;
        const int a0 = hp - g.kh + 1, c0 = wp - g.kw + 1;
        const int i_lo = a0 <= 0 ? 0 : (a0 + g.sh - 1) / g.sh;
        const int j_lo = c0 <= 0 ? 0 : (c0 + g.sw - 1) / g.sw;
        const int i_hi = min(g.Ho - 1, hp / g.sh);
        const int j_hi = min(g.Wo - 1, wp / g.sw);
        const int64_t obase = nc * g.Ho * g.Wo;
        T acc = T(0);
        for (int i = i_lo; i <= i_hi; ++i)
            for (int j = j_lo; j <= j_hi; ++j) {
                const int64_t o = obase + static_cast<int64_t>(i) * g.Wo + j;
                if (__ldg(idx + o) == target) acc += __ldg(go + o);
            }
        gx[e] = acc;
    }
}

// Reference-signature backward (kernel.cu:153-185): grad_x_pad[idx] += go with
// atomics on whatever the caller put in grad_x_pad (it zero-fills it).
template <typename T>
__global__ void __launch_bounds__(kThreads)
maxpool_bwd_scatter(const T* __restrict__ go, const long long* __restrict__ idx, T* gx_pad, int Ho, int Wo, int Hp,
                    int Wp, int64_t total) {
    kd::pdl_prologue();
    const int64_t plane_o = static_cast<int64_t>(Ho) * Wo;
    const int64_t plane_i = static_cast<int64_t>(Hp) * Wp;
    for (int64_t o = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; o < total;
         o += static_cast<int64_t>(gridDim.x) * kThreads) {
        const long long p = idx[o];
        if (p < 0 || p >= plane_i) continue;
        const int64_t nc = o / plane_o;
        atomicAdd(gx_pad + nc * plane_i + p, go[o]);
    }
}

// ===========================================================================
// AvgPool (count_include_pad: divisor is always kh*kw)
// ===========================================================================
// Reference arithmetic (keydnn_avgpool2d_cuda.cu:79-91): sum = 0; sum += tap in
// row-major order over the zero-padded window; y = sum / T(kh*kw).  A padded tap
// adds +0, which never changes the running sum (it starts at +0 and so is never
// -0), so skipping those taps is bit-identical.

template <typename T>
__global__ void __launch_bounds__(kThreads)
avgpool_fwd_generic(const T* __restrict__ x, T* __restrict__ y, PoolGeom g, int64_t total) {
    kd::pdl_prologue();
    const T denom = static_cast<T>(g.kh * g.kw);
    for (int64_t o = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; o < total;
         o += static_cast<int64_t>(gridDim.x) * kThreads) {
        const int j = static_cast<int>(o % g.Wo);
        const int64_t t = o / g.Wo;
        const int i = static_cast<int>(t % g.Ho);
        const int64_t nc = t / g.Ho;
        const T* plane = x + nc * g.H * g.W;
        const int h0 = i * g.sh - g.ph, w0 = j * g.sw - g.pw;
        T sum = T(0);
        for (int a = 0; a < g.kh; ++a) {
            const int h = h0 + a;
            if (h < 0 || h >= g.H) continue;
            for (int b = 0; b < g.kw; ++b) {
                const int w = w0 + b;
                if (w < 0 || w >= g.W) continue;
                sum += __ldg(plane + static_cast<int64_t>(h) * g.W + w);
            }
        }
        y[o] = sum / denom;
    }
}

// kernel 2x2, stride 2, no padding, W % 8 == 0: the layout of maxpool2x2_fwd (four adjacent windows per thread, two
// rows of eight inputs as 32-byte loads, one 16-byte store).  sum = 0; sum += the four taps row-major; the division
// by four is an exact scaling.
template <typename T, int U>
__global__ void __launch_bounds__(kThreads)
avgpool2x2_fwd(const T* __restrict__ x, T* __restrict__ y, int H, int W, int Ho, int Wo, int64_t groups, kd::FastDiv by_gpr,
               kd::FastDiv by_ho) {
    kd::pdl_prologue();
    const int64_t tile = static_cast<int64_t>(kThreads) * U;
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * tile; base < groups;
         base += static_cast<int64_t>(gridDim.x) * tile) {
        kd::Row8<T> top8[U], bot8[U];
        int64_t o[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t gi = base + u * kThreads + threadIdx.x;
            if (gi < groups) {
                unsigned rw, j4, nc, i;
                by_gpr.divmod(static_cast<unsigned>(gi), rw, j4);     // groups < 2^31 (checked by the launcher)
                by_ho.divmod(rw, nc, i);
                o[u] = static_cast<int64_t>(rw) * Wo + 4 * j4;
                const T* r0 = x + (static_cast<int64_t>(nc) * H + 2 * i) * W + 8 * j4;
                top8[u] = kd::load8_stream(r0);
                bot8[u] = kd::load8_stream(r0 + W);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t gi = base + u * kThreads + threadIdx.x;
            if (gi < groups) {
                Pack4<T> out;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    T sum = T(0);
                    sum += top8[u].v[2 * q];
                    sum += top8[u].v[2 * q + 1];
                    sum += bot8[u].v[2 * q];
                    sum += bot8[u].v[2 * q + 1];
                    out.v[q] = sum * T(0.25);
                }
                kd::store4(y + o[u], out);
            }
        }
    }
}

// Backward of the same geometry: eight adjacent gradient elements of one input row per thread (one 32-byte store, and
// with ACCUM one 32-byte load), from one packet of grad_out; acc = 0; acc += go / 4.  Rows below the last window
// (odd H) receive +0.
template <typename T, bool ACCUM, int U>
__global__ void __launch_bounds__(kThreads)
avgpool2x2_bwd(const T* __restrict__ go, T* __restrict__ gx, int H, int W, int Ho, int Wo, int64_t blocks, kd::FastDiv by_bpr,
               kd::FastDiv by_h) {
    kd::pdl_prologue();
    const int64_t tile = static_cast<int64_t>(kThreads) * U;
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * tile; base < blocks;
         base += static_cast<int64_t>(gridDim.x) * tile) {
        Pack4<T> gv[U];
        kd::Row8<T> held[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t bi = base + u * kThreads + threadIdx.x;
            if (bi < blocks) {
                unsigned rowflat, jg, nc, h;                      // rowflat = nc * H + h
                by_bpr.divmod(static_cast<unsigned>(bi), rowflat, jg);
                by_h.divmod(rowflat, nc, h);
                if (static_cast<int>(h >> 1) < Ho) {
                    gv[u] = kd::load4(go + (static_cast<int64_t>(nc) * Ho + (h >> 1)) * Wo + 4 * jg);
                } else {
                    gv[u].v[0] = gv[u].v[1] = gv[u].v[2] = gv[u].v[3] = T(0);
                }
                if (ACCUM) held[u] = kd::load8_stream(gx + 8 * bi);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t bi = base + u * kThreads + threadIdx.x;
            if (bi < blocks) {
                kd::Row8<T> out;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    T acc = T(0);
                    acc += gv[u].v[q] * T(0.25);
                    out.v[2 * q] = ACCUM ? held[u].v[2 * q] + acc : acc;
                    out.v[2 * q + 1] = ACCUM ? held[u].v[2 * q + 1] + acc : acc;
                }
                kd::store8(gx + 8 * bi, out);
            }
        }
    }
}

// x / 9, correctly rounded.  For float inside [2^-100, 2^100] the quotient comes from the
// rounded reciprocal and one exact FMA residual (q0 = x*r; e = fma(-q0, 9, x); q = fma(e, r, q0)),
// three instructions instead of the division sequence; this equals RN(x / 9) for every float
// in that range (checked exhaustively on a CPU: 3,355,443,202 values, no mismatch).  Anything
// else (zeros, subnormal-range, huge, inf, NaN, and double) takes the true division.
template <typename T> __device__ __forceinline__ T div9(T x) { return x / T(9); }
__device__ __noinline__ float div9_by_division(float x) { return x / 9.0f; }   // a call, so that the rare path is not if-converted
template <> __device__ __forceinline__ float div9<float>(float x) {
    constexpr float r = 1.0f / 9.0f;
    const float q0 = __fmul_rn(x, r);
    const float e = __fmaf_rn(-q0, 9.0f, x);
    const float q = __fmaf_rn(e, r, q0);
    const float ax = fabsf(x);
    if (__builtin_expect(ax >= 0x1p-100f && ax <= 0x1p100f, 1)) return q;
    return div9_by_division(x);
}

// kernel 3x3, stride 2, padding 1, W % 8 == 0 (so Wo = W/2, Wo % 4 == 0).
// A thread owns four adjacent outputs of one output row: from each of the three
// input rows it takes eight aligned inputs (two 16-byte loads) plus the one
// input left of them, which the neighbouring thread also loads (an L1 hit).
// Odd input rows serve two output rows; the second read comes from L1/L2.
template <typename T>
__global__ void __launch_bounds__(kThreads)
avgpool3x3s2p1_fwd(const T* __restrict__ x, T* __restrict__ y, int H, int W, int Ho, int Wo, int64_t groups,
                   kd::FastDiv by_gpr, kd::FastDiv by_ho) {
    kd::pdl_prologue();
    for (int64_t gi = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; gi < groups;
         gi += static_cast<int64_t>(gridDim.x) * kThreads) {
        unsigned row, ujg, nc, ui;
        by_gpr.divmod(static_cast<unsigned>(gi), row, ujg);
        by_ho.divmod(row, nc, ui);
        const int jg = static_cast<int>(ujg), i = static_cast<int>(ui);
        const T* plane = x + static_cast<int64_t>(nc) * H * W;
        T c[3][9];
        bool live[3];
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            const int h = 2 * i - 1 + r;
            live[r] = (h >= 0 && h < H);
            if (live[r]) {
                const T* p = plane + static_cast<int64_t>(h) * W + 8 * jg;
                const kd::Row8<T> a = kd::load8(p);
                c[r][0] = jg > 0 ? __ldg(p - 1) : T(0);
#pragma unroll
                for (int k = 0; k < 8; ++k) c[r][1 + k] = a.v[k];
            }
        }
        Pack4<T> out;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            T sum = T(0);
#pragma unroll
            for (int r = 0; r < 3; ++r) {
                if (live[r]) {
                    sum += c[r][2 * q];
                    sum += c[r][2 * q + 1];
                    sum += c[r][2 * q + 2];
                }
            }
            out.v[q] = div9<T>(sum);
        }
        kd::store4(y + static_cast<int64_t>(row) * Wo + 4 * jg, out);
    }
}

// Reference backward arithmetic (keydnn_avgpool2d_cuda.cu:164-197): for each
// input, acc = 0; acc += go[i,j] / T(kh*kw) over the covering windows in
// ascending (i, j); result = 0 + acc.  Each term is divided on its own.
// `ACCUM` keeps the reference-signature behaviour of adding onto the buffer.
template <typename T, bool ACCUM>
__global__ void __launch_bounds__(kThreads)
avgpool_bwd_gather(const T* __restrict__ go, T* __restrict__ gx, PoolGeom g, int64_t total) {
    kd::pdl_prologue();
    const T denom = static_cast<T>(g.kh * g.kw);
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; e < total;
         e += static_cast<int64_t>(gridDim.x) * kThreads) {
        const int w = static_cast<int>(e % g.W);
        const int64_t t = e / g.W;
        const int h = static_cast<int>(t % g.H);
        const int64_t nc = t / g.H;
        const int hp = h + g.ph, wp = w + g.pw;
        const int a0 = hp - g.kh + 1, c0 = wp - g.kw + 1;
        const int i_lo = a0 <= 0 ? 0 : (a0 + g.sh - 1) / g.sh;
        const int j_lo = c0 <= 0 ? 0 : (c0 + g.sw - 1) / g.sw;
        const int i_hi = min(g.Ho - 1, hp / g.sh);
        const int j_hi = min(g.Wo - 1, wp / g.sw);
        const int64_t obase = nc * g.Ho * g.Wo;
        T acc = T(0);
        for (int i = i_lo; i <= i_hi; ++i)
            for (int j = j_lo; j <= j_hi; ++j)
                acc += __ldg(go + obase + static_cast<int64_t>(i) * g.Wo + j) / denom;
        if (ACCUM) gx[e] += acc;
        else gx[e] = acc;
    }
}

// ---------------------------------------------------------------------------
// Band kernels: any window, stride and padding, any alignment.
// A CTA takes a band of whole rows of one plane.  Everything the band reads is one contiguous
// span of memory (rows are complete), so it is staged in shared memory with 16-byte cp.async
// copies (two buffers: the next item's span arrives while the current one is worked on) and the
// stencil reads shared memory; global traffic is fully coalesced whatever the stride of the
// window.  A thread then owns one column of the band (backward: 1, 2 or 4 adjacent columns) and
// walks down its rows, so that everything that depends on the column only is computed once and a
// row costs a pointer increment: these kernels are bound by instruction issue before they are
// bound by memory, and index arithmetic per element is what has to go.  The arithmetic on the
// data is that of the one-thread-per-element kernels above, tap for tap.  `lanes` (a power of
// two, 8 .. the CTA) threads share a row; a CTA has 32, 64 or 128 threads by the size of an item.
// ---------------------------------------------------------------------------
constexpr int kBandBytes = 16 * 1024;          // staged span per band
constexpr int kBandRowsMax = 512;              // backward: rows of a band (one table entry each)

template <typename T> struct BandVec { static constexpr int value = 16 / static_cast<int>(sizeof(T)); };

struct BandPlan {
    bool ok;
    int rows;        // rows of the band (output rows forward, input rows backward)
    int bands;       // bands per plane
    int buffer;      // elements of one arrival buffer (forward: the input span; backward: the gradients)
    size_t smem;
};

constexpr int kBandThreads = 128;

// Threads of a CTA for items of `work` thread-iterations (outputs forward, column groups x rows backward): a warp for
// the smallest planes, so that an SM holds more of them and a barrier stops fewer threads.
inline int band_threads(int64_t work) { return work <= 64 ? 32 : (work <= 384 ? 64 : kBandThreads); }

// log2 of the threads that share a row: the smallest power of two >= width, 8..threads
inline int band_lane_bits(int width, int threads) {
    int bits = 3;
    while ((1 << bits) < width && (1 << bits) < threads) ++bits;
    return bits;
}

// Forward: `rows` output rows need (rows-1)*sh + kh input rows.
template <typename T> inline BandPlan band_plan_fwd(const PoolGeom& g) {
    BandPlan p = {false, 0, 0, 0, 0};
    const int64_t cap = kBandBytes / static_cast<int64_t>(sizeof(T));
    if (static_cast<int64_t>(g.kh) * g.W > cap) return p;
    int64_t r = (cap / g.W - g.kh) / g.sh + 1;
    if (r > g.Ho) r = g.Ho;
    if (r < 1) return p;
    p.bands = static_cast<int>((g.Ho + r - 1) / r);
    p.rows = (g.Ho + p.bands - 1) / p.bands;
    // two staging buffers, each a whole number of 16-byte packets
    p.buffer = (((p.rows - 1) * g.sh + g.kh) * g.W + 2 * BandVec<T>::value - 1) / BandVec<T>::value * BandVec<T>::value;
    p.smem = 2 * static_cast<size_t>(p.buffer) * sizeof(T);
    p.ok = true;
    return p;
}

// Backward: `rows` input rows are covered by at most (rows + kh - 2) / sh + 1 output rows; they are staged
// with one more column and one more row, both zero.
inline __host__ __device__ int64_t band_go_rows(const PoolGeom& g, int64_t r) { return (r + g.kh - 2) / g.sh + 1; }
inline __host__ __device__ size_t band_bwd_table_bytes(int rows) { return static_cast<size_t>(rows) * sizeof(int4); }
template <typename T> inline __host__ __device__ size_t band_bwd_quotient_bytes(const PoolGeom& g, int rows) {
    return (static_cast<size_t>((band_go_rows(g, rows) + 1) * (g.Wo + 1)) * sizeof(T) + 15) & ~size_t(15);
}

template <typename T> inline BandPlan band_plan_bwd(const PoolGeom& g) {
    BandPlan p = {false, 0, 0, 0, 0};
    const int64_t cap = kBandBytes / 2 / static_cast<int64_t>(sizeof(T));
    const int64_t pitch = g.Wo + 1;
    if ((band_go_rows(g, 1) + 1) * pitch > cap) return p;
    int64_t r = (cap / pitch - 2) * g.sh - g.kh + 2;
    if (r < 1) r = 1;
    while (r > 1 && (band_go_rows(g, r) + 1) * pitch > cap) --r;
    const int64_t most = (8192 + g.W - 1) / g.W;             // and at most ~8192 elements a band
    if (r > most) r = most;
    if (r > kBandRowsMax) r = kBandRowsMax;
    if (r > g.H) r = g.H;
    p.bands = static_cast<int>((g.H + r - 1) / r);
    p.rows = (g.H + p.bands - 1) / p.bands;
    // the row table, the quotients (rows of Wo + 1, one more row), two buffers for the gradients as they arrive
    constexpr int V = BandVec<T>::value;
    p.buffer = static_cast<int>((band_go_rows(g, p.rows) * g.Wo + 2 * V - 1) / V * V);
    p.smem = band_bwd_table_bytes(p.rows) + band_bwd_quotient_bytes<T>(g, p.rows) + 2 * static_cast<size_t>(p.buffer) * sizeof(T);
    p.ok = true;
    return p;
}

// mis: the element offset of a span inside its first 16-byte packet; element e is staged at s[mis + e], which keeps
// the packets aligned on both sides.
template <typename T> __device__ __forceinline__ int band_misalign(const T* p) {
    return static_cast<int>((reinterpret_cast<uintptr_t>(p) / sizeof(T)) & (BandVec<T>::value - 1));
}

// x / taps: the exact short forms where they exist.  TAPS > 0: known when the kernel is compiled.
template <typename T, int TAPS> struct WindowDiv {
    T d, inv;
    int kind;                                                     // 0: division, 1: nine, 2: power of two
    __device__ explicit WindowDiv(int taps) : d(static_cast<T>(taps)), inv(T(1) / static_cast<T>(taps)),
                                              kind(taps == 9 ? 1 : ((taps & (taps - 1)) == 0 ? 2 : 0)) {}
    __device__ __forceinline__ T operator()(T x) const {
        if (TAPS == 9) return div9<T>(x);
        if (TAPS > 0 && (TAPS & (TAPS - 1)) == 0) return x * (T(1) / T(TAPS > 0 ? TAPS : 1));
        if (kind == 1) return div9<T>(x);
        if (kind == 2) return x * inv;                            // exact scaling, gradual underflow included
        return x / d;
    }
};

// Forward kernels.  KH, KW: the window when the kernel is compiled for it, 0 = taken from g.  EDGES: a window may
// reach outside the plane (padding, or an output size that lets the last window hang over); such taps contribute +0
// to an average, which leaves the running sum as it is (it starts at +0 and is therefore never -0), and are no
// candidates for a maximum.  Only the outputs on the rim of the plane have such windows: the rectangle of outputs
// whose windows lie inside runs through the unchecked loop, the rim (a few rows and columns) through a checked one
// spread over all threads, so that no warp executes both.
// The staging is asynchronous (cp.async, 16 bytes each, no registers) into one of two buffers: the span of the CTA's
// next item is requested before the stencil of the current one runs, so its loads are in flight under the arithmetic
// and a CTA never waits for a full memory round trip between items.
struct BandItem {
    unsigned nc;
    int nout, nrows, in_off, out_off, top;      // top: staged row of the first tap of the band's first output row
    int i0;
};

__device__ __forceinline__ BandItem band_item(const PoolGeom& g, int kh, int rows, const kd::FastDiv& by_bands, unsigned item) {
    BandItem it;
    unsigned band;
    by_bands.divmod(item, it.nc, band);
    it.i0 = static_cast<int>(band) * rows;
    it.nout = min(g.Ho, it.i0 + rows) - it.i0;
    const int h_lo = max(0, it.i0 * g.sh - g.ph);
    it.nrows = min(g.H, (it.i0 + it.nout - 1) * g.sh - g.ph + kh) - h_lo;
    it.in_off = h_lo * g.W;
    it.out_off = it.i0 * g.Wo;
    it.top = it.i0 * g.sh - g.ph - h_lo;
    return it;
}

// Requests src[0, n) into s[mis, mis + n): cp.async for the 16-byte packets, plain loads for the elements before the
// first and after the last boundary.  The caller commits the group and waits for it.
template <typename T>
__device__ __forceinline__ void band_stage_async(const T* __restrict__ src, int n, T* s, int mis) {
    constexpr int V = BandVec<T>::value;
    int head = (V - mis) & (V - 1);
    if (head > n) head = n;
    const int nv = (n - head) / V;
    if (static_cast<int>(threadIdx.x) < head) s[mis + threadIdx.x] = __ldg(src + threadIdx.x);
    const T* body = src + head;
    const unsigned sbody = static_cast<unsigned>(__cvta_generic_to_shared(s + mis + head));   // a multiple of 16 bytes
    for (int v = threadIdx.x; v < nv; v += blockDim.x)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sbody + 16u * v), "l"(body + static_cast<size_t>(v) * V) : "memory");
    const int done = head + nv * V;
    if (static_cast<int>(threadIdx.x) < n - done) s[mis + done + threadIdx.x] = __ldg(src + done + threadIdx.x);
}
__device__ __forceinline__ void band_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void band_wait_all_but_newest() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

template <typename T, int KH, int KW, bool EDGES>
__global__ void __launch_bounds__(kBandThreads)
avgpool_fwd_band(const T* __restrict__ x, T* __restrict__ y, PoolGeom g, int rows, unsigned items, kd::FastDiv by_bands,
                 int lane_bits, int buffer_elems, kd::FastDiv by_wo, kd::FastDiv by_edge_cols) {
    extern __shared__ __align__(16) unsigned char band_smem[];
    T* const buf = reinterpret_cast<T*>(band_smem);
    kd::pdl_prologue();
    const int kh = KH ? KH : g.kh, kw = KW ? KW : g.kw;
    const WindowDiv<T, KH * KW> divide(kh * kw);
    const int lanes = 1 << lane_bits;
    const int group = threadIdx.x >> lane_bits, lig = threadIdx.x & (lanes - 1), ngroups = blockDim.x >> lane_bits;
    const int step = ngroups * g.sh;
    const int64_t plane_in = static_cast<int64_t>(g.H) * g.W, plane_out = static_cast<int64_t>(g.Ho) * g.Wo;
    unsigned item = blockIdx.x;
    if (item >= items) return;
    BandItem it = band_item(g, kh, rows, by_bands, item);
    const T* src = x + it.nc * plane_in + it.in_off;
    int mis = band_misalign(src);
    int cur = 0;
    if (it.nrows > 0) band_stage_async(src, it.nrows * g.W, buf, mis);
    band_commit();
    for (; item < items; item += gridDim.x) {
        const unsigned next = item + gridDim.x;
        BandItem nx = it;
        int nmis = 0;
        if (next < items) {
            nx = band_item(g, kh, rows, by_bands, next);
            const T* nsrc = x + nx.nc * plane_in + nx.in_off;
            nmis = band_misalign(nsrc);
            if (nx.nrows > 0) band_stage_async(nsrc, nx.nrows * g.W, buf + (cur ^ 1) * buffer_elems, nmis);
        }
        band_commit();
        band_wait_all_but_newest();
        __syncthreads();
        const T* s = buf + cur * buffer_elems;
        const int nrows = it.nrows;
        T* const dst = y + it.nc * plane_out + it.out_off;
        // one output whose window may reach outside the plane: every tap checked
        auto checked = [&](int ii, int j) {
            const int hh = it.top + ii * g.sh, w0 = j * g.sw - g.pw;
            const T* t = s + mis + hh * g.W + w0;
            T sum = T(0);
            for (int a = 0; a < kh; ++a) {
                if (hh + a < 0 || hh + a >= nrows) continue;
                for (int b = 0; b < kw; ++b) {
                    if (w0 + b < 0 || w0 + b >= g.W) continue;
                    sum += t[a * g.W + b];
                }
            }
            dst[ii * g.Wo + j] = divide(sum);
        };
        // the outputs whose windows lie inside the staged rows and inside the plane: rows [ia, ib], columns [ja, jb]
        int ia = 0, ib = it.nout - 1, ja = 0, jb = g.Wo - 1;
        if (EDGES) {
            ia = it.top >= 0 ? 0 : (-it.top + g.sh - 1) / g.sh;
            ib = nrows - kh - it.top >= 0 ? min(it.nout - 1, (nrows - kh - it.top) / g.sh) : -1;
            ja = (g.pw + g.sw - 1) / g.sw;
            jb = g.W - kw + g.pw >= 0 ? min(g.Wo - 1, (g.W - kw + g.pw) / g.sw) : -1;
            if (ib < ia || jb < ja) { ia = it.nout; ib = it.nout - 1; ja = 0; jb = -1; }      // none: everything is an edge
        }
        for (int j = ja + lig; j <= jb; j += lanes) {
            const int w0 = j * g.sw - g.pw;
            const T* t = s + mis + (it.top + (ia + group) * g.sh) * g.W + w0;
            T* out = dst + (ia + group) * g.Wo + j;
            for (int ii = ia + group; ii <= ib; ii += ngroups, t += step * g.W, out += ngroups * g.Wo) {
                T sum = T(0);
                if (KH > 0) {
#pragma unroll
                    for (int a = 0; a < KH; ++a)
#pragma unroll
                        for (int b = 0; b < KW; ++b) sum += t[a * g.W + b];
                } else {
                    for (int a = 0; a < kh; ++a)
                        for (int b = 0; b < kw; ++b) sum += t[a * g.W + b];
                }
                *out = divide(sum);
            }
        }
        if (EDGES) {
            // the rows above ia and below ib, all columns; then the columns left of ja and right of jb in the rows between
            const int inner_rows = max(0, ib - ia + 1);
            const int edge_rows = it.nout - inner_rows;
            for (int e = threadIdx.x; e < edge_rows * g.Wo; e += blockDim.x) {
                unsigned r, j;
                by_wo.divmod(static_cast<unsigned>(e), r, j);
                checked(static_cast<int>(r) < ia ? static_cast<int>(r) : ib + 1 + (static_cast<int>(r) - ia), static_cast<int>(j));
            }
            const int edge_cols = inner_rows > 0 ? ja + (g.Wo - 1 - jb) : 0;
            for (int e = threadIdx.x; e < inner_rows * edge_cols; e += blockDim.x) {
                unsigned r, k;
                by_edge_cols.divmod(static_cast<unsigned>(e), r, k);
                checked(ia + static_cast<int>(r), static_cast<int>(k) < ja ? static_cast<int>(k) : jb + 1 + (static_cast<int>(k) - ja));
            }
        }
        __syncthreads();
        it = nx;
        mis = nmis;
        cur ^= 1;
    }
}

// MaxPool forward on the same bands: the selection rule of maxpool_fwd_generic tap for tap (row-major scan, strictly
// greater replaces, taps outside the plane are never candidates), the position as h * (W + 2 pw) + w in the padded plane.
template <typename T, int KH, int KW, bool EDGES>
__global__ void __launch_bounds__(kBandThreads)
maxpool_fwd_band(const T* __restrict__ x, T* __restrict__ y, long long* __restrict__ idx, PoolGeom g, int rows, unsigned items,
                 kd::FastDiv by_bands, int lane_bits, int buffer_elems, kd::FastDiv by_wo, kd::FastDiv by_edge_cols) {
    extern __shared__ __align__(16) unsigned char band_smem[];
    T* const buf = reinterpret_cast<T*>(band_smem);
    kd::pdl_prologue();
    const int kh = KH ? KH : g.kh, kw = KW ? KW : g.kw;
    const int lanes = 1 << lane_bits;
    const int group = threadIdx.x >> lane_bits, lig = threadIdx.x & (lanes - 1), ngroups = blockDim.x >> lane_bits;
    const int step = ngroups * g.sh;
    const int Wp = g.W + 2 * g.pw;
    const int64_t plane_in = static_cast<int64_t>(g.H) * g.W, plane_out = static_cast<int64_t>(g.Ho) * g.Wo;
    unsigned item = blockIdx.x;
    if (item >= items) return;
    BandItem it = band_item(g, kh, rows, by_bands, item);
    const T* src = x + it.nc * plane_in + it.in_off;
    int mis = band_misalign(src);
    int cur = 0;
    if (it.nrows > 0) band_stage_async(src, it.nrows * g.W, buf, mis);
    band_commit();
    for (; item < items; item += gridDim.x) {
        const unsigned next = item + gridDim.x;
        BandItem nx = it;
        int nmis = 0;
        if (next < items) {
            nx = band_item(g, kh, rows, by_bands, next);
            const T* nsrc = x + nx.nc * plane_in + nx.in_off;
            nmis = band_misalign(nsrc);
            if (nx.nrows > 0) band_stage_async(nsrc, nx.nrows * g.W, buf + (cur ^ 1) * buffer_elems, nmis);
        }
        band_commit();
        band_wait_all_but_newest();
        __syncthreads();
        const T* s = buf + cur * buffer_elems;
        const int nrows = it.nrows;
        const int64_t obase = it.nc * plane_out + it.out_off;
        auto checked = [&](int ii, int j) {
            const int hh = it.top + ii * g.sh, wp0 = j * g.sw, w0 = wp0 - g.pw;
            const T* t = s + mis + hh * g.W + w0;
            T best = kd::neg_inf<T>();
            int ba = 0, bb = 0;
            for (int a = 0; a < kh; ++a) {
                if (hh + a < 0 || hh + a >= nrows) continue;
                for (int b = 0; b < kw; ++b) {
                    if (w0 + b < 0 || w0 + b >= g.W) continue;
                    const T v = t[a * g.W + b];
                    if (v > best) { best = v; ba = a; bb = b; }
                }
            }
            const int64_t o = obase + static_cast<int64_t>(ii) * g.Wo + j;
            y[o] = best;
            idx[o] = static_cast<long long>((it.i0 + ii) * g.sh + ba) * Wp + (wp0 + bb);
        };
        int ia = 0, ib = it.nout - 1, ja = 0, jb = g.Wo - 1;
        if (EDGES) {
            ia = it.top >= 0 ? 0 : (-it.top + g.sh - 1) / g.sh;
            ib = nrows - kh - it.top >= 0 ? min(it.nout - 1, (nrows - kh - it.top) / g.sh) : -1;
            ja = (g.pw + g.sw - 1) / g.sw;
            jb = g.W - kw + g.pw >= 0 ? min(g.Wo - 1, (g.W - kw + g.pw) / g.sw) : -1;
            if (ib < ia || jb < ja) { ia = it.nout; ib = it.nout - 1; ja = 0; jb = -1; }      // none: everything is an edge
        }
        for (int j = ja + lig; j <= jb; j += lanes) {
            const int wp0 = j * g.sw;
            const int w0 = wp0 - g.pw;
            int hp0 = (it.i0 + ia + group) * g.sh;                             // padded-plane row of the first tap
            const T* t = s + mis + (it.top + (ia + group) * g.sh) * g.W + w0;
            int64_t o = obase + static_cast<int64_t>(ia + group) * g.Wo + j;
            for (int ii = ia + group; ii <= ib; ii += ngroups, hp0 += step, t += step * g.W, o += ngroups * g.Wo) {
                T best = kd::neg_inf<T>();
                int ba = 0, bb = 0;
                if (KH > 0) {
#pragma unroll
                    for (int a = 0; a < KH; ++a)
#pragma unroll
                        for (int b = 0; b < KW; ++b) {
                            const T v = t[a * g.W + b];
                            if (v > best) { best = v; ba = a; bb = b; }
                        }
                } else {
                    for (int a = 0; a < kh; ++a)
                        for (int b = 0; b < kw; ++b) {
                            const T v = t[a * g.W + b];
                            if (v > best) { best = v; ba = a; bb = b; }
                        }
                }
                y[o] = best;
                idx[o] = static_cast<long long>(hp0 + ba) * Wp + (wp0 + bb);
            }
        }
        if (EDGES) {
            const int inner_rows = max(0, ib - ia + 1);
            const int edge_rows = it.nout - inner_rows;
            for (int e = threadIdx.x; e < edge_rows * g.Wo; e += blockDim.x) {
                unsigned r, j;
                by_wo.divmod(static_cast<unsigned>(e), r, j);
                checked(static_cast<int>(r) < ia ? static_cast<int>(r) : ib + 1 + (static_cast<int>(r) - ia), static_cast<int>(j));
            }
            const int edge_cols = inner_rows > 0 ? ja + (g.Wo - 1 - jb) : 0;
            for (int e = threadIdx.x; e < inner_rows * edge_cols; e += blockDim.x) {
                unsigned r, k;
                by_edge_cols.divmod(static_cast<unsigned>(e), r, k);
                checked(ia + static_cast<int>(r), static_cast<int>(k) < ja ? static_cast<int>(k) : jb + 1 + (static_cast<int>(k) - ja));
            }
        }
        __syncthreads();
        it = nx;
        mis = nmis;
        cur ^= 1;
    }
}

// Backward.  The quotients go / (kh*kw) of the output rows that cover the band are staged once, in rows of Wo + 1
// with a zero in the extra column, followed by a row of zeros.  What depends on the column only (the first covering
// output column and how many there are) is computed once per thread; what depends on the row only comes from a table
// that is refilled when the CTA moves to a different band (with one band per plane: once).  MAXW = 2 or 3: no element is
// covered by more than MAXW windows along either axis (kh <= MAXW sh, kw <= MAXW sw: 3x3 / 2, 2x2 / 2 ... and 3x3 / 1,
// 5x5 / 2 ...); the table holds the staged (byte) offsets of the covering rows and the thread those of the covering
// columns, a window that does not exist being replaced by the zero row / zero column, so the MAXW x MAXW taps are taken
// without a branch or a predicate.  A zero tap leaves the running
// sum as it is (it starts at +0 and is therefore never -0).  MAXW = 0: the table holds {offset of the first covering
// row, number of covering rows} and the taps are counted loops.  A thread owns V adjacent columns, moved with one
// access of 4 to 16 bytes, and has 8 / V rows in flight.
template <typename T> struct BandColumn { int j_lo, nj, a, b, c; };   // a, b, c: the first three covering columns, Wo where there is none

template <typename T>
__device__ __forceinline__ BandColumn<T> band_column(const PoolGeom& g, int w, const kd::FastDiv& by_sw) {
    const int wp = w + g.pw;
    const int c0 = wp - g.kw + 1;
    BandColumn<T> c;
    c.j_lo = c0 <= 0 ? 0 : static_cast<int>(by_sw.div(static_cast<unsigned>(c0 + g.sw - 1)));
    c.nj = min(g.Wo - 1, static_cast<int>(by_sw.div(static_cast<unsigned>(wp)))) - c.j_lo + 1;
    c.a = c.nj >= 1 ? c.j_lo : g.Wo;
    c.b = c.nj >= 2 ? c.j_lo + 1 : g.Wo;
    c.c = c.nj >= 3 ? c.j_lo + 2 : g.Wo;
    return c;
}

// V adjacent elements with one access (V * sizeof(T) = 4, 8 or 16 bytes, the address aligned to that); touched once.
template <typename T, int V> __device__ __forceinline__ void band_load(const T* p, T (&v)[V]) {
    if constexpr (V == 1) {
        v[0] = __ldcs(p);
    } else if constexpr (sizeof(T) * V == 8) {
        const float2 t = __ldcs(reinterpret_cast<const float2*>(p));
        v[0] = t.x; v[1] = t.y;
    } else if constexpr (sizeof(T) == 4) {
        const float4 t = __ldcs(reinterpret_cast<const float4*>(p));
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
        const double2 t = __ldcs(reinterpret_cast<const double2*>(p));
        v[0] = t.x; v[1] = t.y;
    }
}
template <typename T, int V> __device__ __forceinline__ void band_store(T* p, const T (&v)[V]) {
    if constexpr (V == 1) __stcs(p, v[0]);
    else if constexpr (sizeof(T) * V == 8) __stcs(reinterpret_cast<float2*>(p), make_float2(v[0], v[1]));
    else if constexpr (sizeof(T) == 4) __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
    else __stcs(reinterpret_cast<double2*>(p), make_double2(v[0], v[1]));
}

// V: adjacent columns per thread, moved with one access (W % V == 0 and the tensor aligned to V elements).
// The gradients of the covering output rows arrive asynchronously (cp.async into one of two buffers; those of the
// CTA's next item are requested before the current one is worked on) and are turned into the staged quotients by a
// short shared-to-shared pass.
struct BandBwdItem { unsigned nc, band; int h0, nrows, i_first, ngo; };

__device__ __forceinline__ BandBwdItem band_bwd_item(const PoolGeom& g, int rows, const kd::FastDiv& by_bands,
                                                     const kd::FastDiv& by_sh, unsigned item) {
    BandBwdItem it;
    by_bands.divmod(item, it.nc, it.band);
    it.h0 = static_cast<int>(it.band) * rows;
    it.nrows = min(g.H, it.h0 + rows) - it.h0;
    const int a_first = it.h0 + g.ph - g.kh + 1;
    it.i_first = a_first <= 0 ? 0 : static_cast<int>(by_sh.div(static_cast<unsigned>(a_first + g.sh - 1)));
    const int i_last = min(g.Ho - 1, static_cast<int>(by_sh.div(static_cast<unsigned>(it.h0 + it.nrows - 1 + g.ph))));
    it.ngo = max(0, i_last - it.i_first + 1);
    return it;
}

template <typename T, bool ACCUM, int MAXW, int V>
__global__ void __launch_bounds__(kBandThreads)
avgpool_bwd_band(const T* __restrict__ go, T* __restrict__ gx, PoolGeom g, int rows, unsigned items, kd::FastDiv by_bands,
                 int lane_bits, kd::FastDiv by_sh, kd::FastDiv by_sw, kd::FastDiv by_wo, int buffer_elems) {
    extern __shared__ __align__(16) unsigned char band_smem[];
    int4* rowinfo = reinterpret_cast<int4*>(band_smem);
    T* q = reinterpret_cast<T*>(band_smem + band_bwd_table_bytes(rows));
    T* const raw = reinterpret_cast<T*>(band_smem + band_bwd_table_bytes(rows) + band_bwd_quotient_bytes<T>(g, rows));
    kd::pdl_prologue();
    const WindowDiv<T, 0> divide(g.kh * g.kw);
    const int lanes = 1 << lane_bits;
    const int group = threadIdx.x >> lane_bits, lig = threadIdx.x & (lanes - 1), ngroups = blockDim.x >> lane_bits;
    const int pitch = g.Wo + 1;
    constexpr int U = 8 / V;                   // rows in flight per thread
    const int wv = g.W / V;                    // column groups
    const int64_t stride = static_cast<int64_t>(ngroups) * g.W;
    const int64_t plane_in = static_cast<int64_t>(g.H) * g.W, plane_out = static_cast<int64_t>(g.Ho) * g.Wo;
    BandColumn<T> mine[V];
#pragma unroll
    for (int k = 0; k < V; ++k) mine[k] = band_column<T>(g, lig * V + k, by_sw);
    unsigned item = blockIdx.x;
    if (item >= items) return;
    BandBwdItem it = band_bwd_item(g, rows, by_bands, by_sh, item);
    const T* src = go + it.nc * plane_out + static_cast<int64_t>(it.i_first) * g.Wo;
    int mis = band_misalign(src);
    int cur = 0;
    unsigned tabled = ~0u;                     // the band the row table and the zero row are filled for
    if (it.ngo > 0) band_stage_async(src, it.ngo * g.Wo, raw, mis);
    band_commit();
    for (; item < items; item += gridDim.x) {
        const unsigned next = item + gridDim.x;
        BandBwdItem nx = it;
        int nmis = 0;
        if (next < items) {
            nx = band_bwd_item(g, rows, by_bands, by_sh, next);
            const T* nsrc = go + nx.nc * plane_out + static_cast<int64_t>(nx.i_first) * g.Wo;
            nmis = band_misalign(nsrc);
            if (nx.ngo > 0) band_stage_async(nsrc, nx.ngo * g.Wo, raw + (cur ^ 1) * buffer_elems, nmis);
        }
        band_commit();
        const int nrows = it.nrows, ngo = it.ngo;
        T* plane = gx + it.nc * plane_in + static_cast<int64_t>(it.h0 + group) * g.W;     // this thread's first row of the band
        // what the buffer holds in this thread's first rows is requested now, so that the reads are under way
        // while the quotients are prepared
        T held[U][V];
        if (ACCUM && lig < wv) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (group + u * ngroups < nrows) band_load<T, V>(plane + lig * V + u * stride, held[u]);
            }
        }
        band_wait_all_but_newest();
        __syncthreads();
        const T* arrived = raw + cur * buffer_elems + mis;
        const int n = ngo * g.Wo;
        auto prepare = [&](auto quotient) {
#pragma unroll 4
            for (int e = threadIdx.x; e < n; e += blockDim.x) {
                unsigned r, c;
                by_wo.divmod(static_cast<unsigned>(e), r, c);
                q[r * pitch + c] = quotient(arrived[e]);
            }
        };
        if (divide.kind == 1) prepare([](T v) { return div9<T>(v); });
        else if (divide.kind == 2) prepare([&](T v) { return v * divide.inv; });
        else prepare([&](T v) { return v / divide.d; });
        if (it.band != tabled) {
            tabled = it.band;
            for (int r = threadIdx.x; r < ngo; r += blockDim.x) q[r * pitch + g.Wo] = T(0);
            for (int c = threadIdx.x; c < pitch; c += blockDim.x) q[ngo * pitch + c] = T(0);
            for (int hh = threadIdx.x; hh < nrows; hh += blockDim.x) {
                const int hp = it.h0 + hh + g.ph;
                const int a0 = hp - g.kh + 1;
                const int i_lo = a0 <= 0 ? 0 : static_cast<int>(by_sh.div(static_cast<unsigned>(a0 + g.sh - 1)));
                const int ni = min(g.Ho - 1, static_cast<int>(by_sh.div(static_cast<unsigned>(hp)))) - i_lo + 1;
                const int first = (i_lo - it.i_first) * pitch;
                constexpr int B = static_cast<int>(sizeof(T));                 // MAXW > 0: byte offsets
                const int none = ngo * pitch;
                if (MAXW > 0)
                    rowinfo[hh] = make_int4((ni >= 1 ? first : none) * B, (ni >= 2 ? first + pitch : none) * B,
                                            (ni >= 3 ? first + 2 * pitch : none) * B, 0);
                else rowinfo[hh] = make_int4(first, max(0, ni), 0, 0);
            }
        }
        __syncthreads();
        for (int c = lig; c < wv; c += lanes) {
            BandColumn<T> col[V];
#pragma unroll
            for (int k = 0; k < V; ++k) col[k] = c == lig ? mine[k] : band_column<T>(g, c * V + k, by_sw);
            const char* pa[V];
            const char* pb[V];
            const char* pc[V];
#pragma unroll
            for (int k = 0; k < V; ++k) {
                pa[k] = reinterpret_cast<const char*>(q + col[k].a);
                pb[k] = reinterpret_cast<const char*>(q + col[k].b);
                pc[k] = reinterpret_cast<const char*>(q + col[k].c);
            }
            T* out = plane + c * V;
            for (int hb = group; hb < nrows; hb += U * ngroups, out += U * stride) {
                if (ACCUM && (c != lig || hb != group)) {
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        if (hb + u * ngroups < nrows) band_load<T, V>(out + u * stride, held[u]);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int hh = hb + u * ngroups;
                    if (hh >= nrows) break;
                    const int4 ro = rowinfo[hh];
                    T res[V];
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        T acc = T(0);
                        if (MAXW > 0) {
                            const int row_at[3] = {ro.x, ro.y, ro.z};
#pragma unroll
                            for (int r = 0; r < MAXW; ++r) {
                                acc += *reinterpret_cast<const T*>(pa[k] + row_at[r]);
                                acc += *reinterpret_cast<const T*>(pb[k] + row_at[r]);
                                if (MAXW == 3) acc += *reinterpret_cast<const T*>(pc[k] + row_at[r]);
                            }
                        } else {
                            for (int a = 0; a < ro.y; ++a)
                                for (int b = 0; b < col[k].nj; ++b) acc += q[ro.x + a * pitch + col[k].j_lo + b];
                        }
                        res[k] = ACCUM ? held[u][k] + acc : acc;
                    }
                    band_store<T, V>(out + u * stride, res);
                }
            }
        }
        it = nx;
        mis = nmis;
        cur ^= 1;
    }
}

// MaxPool backward on bands of input rows: every element of gx is written once with the sum, in ascending (i, j), of
// the gradients of the windows that recorded it (the rule of maxpool_bwd_gather).  The covering output rows are staged
// as {gradient, tap}: tap = a * kw + b of the recorded position inside its own window, -1 when the position is not
// inside it; an element at window offset (a, b) takes the gradient when the staged tap equals a * kw + b.  Rows of
// Wo + 1 with {0, -1} in the extra column and a last row of {0, -1} stand in for windows that do not exist, as in the
// AvgPool kernel; the row table holds {offsets of the covering rows (MAXW = 2, 3) or first offset and number of rows
// (MAXW = 0), a * kw of the element in the first covering row}.  Gradients and positions arrive asynchronously
// (cp.async, two buffers each; the next item's are requested before the current one is worked on) and a short
// shared-to-shared pass turns them into the staged pairs.
struct BandPlanMax { bool ok; int rows, bands, staged, buffer; size_t smem; };

inline __host__ __device__ size_t band_round16(size_t bytes) { return (bytes + 15) & ~size_t(15); }

template <typename T> inline BandPlanMax band_plan_maxbwd(const PoolGeom& g) {
    BandPlanMax p = {false, 0, 0, 0, 0, 0};
    const int64_t cap = 1024;                                // staged outputs per band (32 bytes of shared memory each)
    const int64_t pitch = g.Wo + 1;
    if ((band_go_rows(g, 1) + 1) * pitch > cap) return p;
    int64_t r = (cap / pitch - 2) * g.sh - g.kh + 2;
    if (r < 1) r = 1;
    while (r > 1 && (band_go_rows(g, r) + 1) * pitch > cap) --r;
    const int64_t most = (8192 + g.W - 1) / g.W;
    if (r > most) r = most;
    if (r > kBandRowsMax) r = kBandRowsMax;
    if (r > g.H) r = g.H;
    p.bands = static_cast<int>((g.H + r - 1) / r);
    p.rows = (g.H + p.bands - 1) / p.bands;
    p.staged = static_cast<int>((band_go_rows(g, p.rows) + 1) * pitch);
    p.buffer = static_cast<int>((band_go_rows(g, p.rows) * g.Wo + 7) / 4 * 4);        // whole packets for both element sizes
    p.smem = static_cast<size_t>(p.rows) * sizeof(int4) + band_round16(p.staged * sizeof(T)) + band_round16(p.staged * sizeof(int)) +
             2 * band_round16(p.buffer * sizeof(long long)) + 2 * band_round16(p.buffer * sizeof(T));
    p.ok = true;
    return p;
}

template <typename T, int MAXW, int V>
__global__ void __launch_bounds__(kBandThreads)
maxpool_bwd_band(const T* __restrict__ go, const long long* __restrict__ idx, T* __restrict__ gx, PoolGeom g, int rows,
                 unsigned items, kd::FastDiv by_bands, int lane_bits, kd::FastDiv by_sh, kd::FastDiv by_sw, kd::FastDiv by_wo,
                 kd::FastDiv by_wp, int staged, int buffer_elems) {
    extern __shared__ __align__(16) unsigned char band_smem[];
    unsigned char* at = band_smem;
    int4* rowinfo = reinterpret_cast<int4*>(at);
    at += static_cast<size_t>(rows) * sizeof(int4);
    T* q = reinterpret_cast<T*>(at);
    at += band_round16(static_cast<size_t>(staged) * sizeof(T));
    int* tap = reinterpret_cast<int*>(at);
    at += band_round16(static_cast<size_t>(staged) * sizeof(int));
    long long* const raw_idx = reinterpret_cast<long long*>(at);
    at += 2 * band_round16(static_cast<size_t>(buffer_elems) * sizeof(long long));
    T* const raw_go = reinterpret_cast<T*>(at);
    const int idx_stride = static_cast<int>(band_round16(static_cast<size_t>(buffer_elems) * sizeof(long long)) / sizeof(long long));
    const int go_stride = static_cast<int>(band_round16(static_cast<size_t>(buffer_elems) * sizeof(T)) / sizeof(T));
    kd::pdl_prologue();
    const int lanes = 1 << lane_bits;
    const int group = threadIdx.x >> lane_bits, lig = threadIdx.x & (lanes - 1), ngroups = blockDim.x >> lane_bits;
    const int pitch = g.Wo + 1;
    constexpr int U = 8 / V;
    const int wv = g.W / V;
    const int Wp = g.W + 2 * g.pw;
    const long long padded = static_cast<long long>(g.H + 2 * g.ph) * Wp;
    const int64_t stride = static_cast<int64_t>(ngroups) * g.W;
    const int64_t plane_in = static_cast<int64_t>(g.H) * g.W, plane_out = static_cast<int64_t>(g.Ho) * g.Wo;
    const int row_step = g.sh * g.kw;
    BandColumn<T> mine[V];
#pragma unroll
    for (int k = 0; k < V; ++k) mine[k] = band_column<T>(g, lig * V + k, by_sw);
    unsigned item = blockIdx.x;
    if (item >= items) return;
    BandBwdItem it = band_bwd_item(g, rows, by_bands, by_sh, item);
    int64_t first_out = it.nc * plane_out + static_cast<int64_t>(it.i_first) * g.Wo;
    int mis_go = band_misalign(go + first_out), mis_idx = band_misalign(idx + first_out);
    int cur = 0;
    unsigned tabled = ~0u;
    if (it.ngo > 0) {
        band_stage_async(go + first_out, it.ngo * g.Wo, raw_go, mis_go);
        band_stage_async(idx + first_out, it.ngo * g.Wo, raw_idx, mis_idx);
    }
    band_commit();
    for (; item < items; item += gridDim.x) {
        const unsigned next = item + gridDim.x;
        BandBwdItem nx = it;
        int nmis_go = 0, nmis_idx = 0;
        if (next < items) {
            nx = band_bwd_item(g, rows, by_bands, by_sh, next);
            const int64_t nfirst = nx.nc * plane_out + static_cast<int64_t>(nx.i_first) * g.Wo;
            nmis_go = band_misalign(go + nfirst);
            nmis_idx = band_misalign(idx + nfirst);
            if (nx.ngo > 0) {
                band_stage_async(go + nfirst, nx.ngo * g.Wo, raw_go + (cur ^ 1) * go_stride, nmis_go);
                band_stage_async(idx + nfirst, nx.ngo * g.Wo, raw_idx + (cur ^ 1) * idx_stride, nmis_idx);
            }
        }
        band_commit();
        band_wait_all_but_newest();
        __syncthreads();
        const int nrows = it.nrows, ngo = it.ngo;
        const T* go_in = raw_go + cur * go_stride + mis_go;
        const long long* idx_in = raw_idx + cur * idx_stride + mis_idx;
        const int n = ngo * g.Wo;
#pragma unroll 4
        for (int e = threadIdx.x; e < n; e += blockDim.x) {
            unsigned r, c;
            by_wo.divmod(static_cast<unsigned>(e), r, c);
            const long long p = idx_in[e];
            int code = -1;
            if (p >= 0 && p < padded) {
                unsigned hb, wb;
                by_wp.divmod(static_cast<unsigned>(p), hb, wb);
                const int a = static_cast<int>(hb) - (it.i_first + static_cast<int>(r)) * g.sh;
                const int b = static_cast<int>(wb) - static_cast<int>(c) * g.sw;
                if (a >= 0 && a < g.kh && b >= 0 && b < g.kw) code = a * g.kw + b;
            }
            q[r * pitch + c] = go_in[e];
            tap[r * pitch + c] = code;
        }
        if (it.band != tabled) {
            tabled = it.band;
            for (int r = threadIdx.x; r < ngo; r += blockDim.x) { q[r * pitch + g.Wo] = T(0); tap[r * pitch + g.Wo] = -1; }
            for (int c = threadIdx.x; c < pitch; c += blockDim.x) { q[ngo * pitch + c] = T(0); tap[ngo * pitch + c] = -1; }
            for (int hh = threadIdx.x; hh < nrows; hh += blockDim.x) {
                const int hp = it.h0 + hh + g.ph;
                const int a0 = hp - g.kh + 1;
                const int i_lo = a0 <= 0 ? 0 : static_cast<int>(by_sh.div(static_cast<unsigned>(a0 + g.sh - 1)));
                const int ni = min(g.Ho - 1, static_cast<int>(by_sh.div(static_cast<unsigned>(hp)))) - i_lo + 1;
                const int first = (i_lo - it.i_first) * pitch;
                const int rp = (hp - i_lo * g.sh) * g.kw;
                const int none = ngo * pitch;
                if (MAXW > 0)
                    rowinfo[hh] = make_int4(ni >= 1 ? first : none, ni >= 2 ? first + pitch : none, ni >= 3 ? first + 2 * pitch : none, rp);
                else rowinfo[hh] = make_int4(first, max(0, ni), 0, rp);
            }
        }
        __syncthreads();
        T* plane = gx + it.nc * plane_in + static_cast<int64_t>(it.h0 + group) * g.W;     // this thread's first row of the band
        for (int c = lig; c < wv; c += lanes) {
            BandColumn<T> col[V];
            int cp[V];                                                // b of the element in its first covering column
#pragma unroll
            for (int k = 0; k < V; ++k) {
                col[k] = c == lig ? mine[k] : band_column<T>(g, c * V + k, by_sw);
                cp[k] = c * V + k + g.pw - col[k].j_lo * g.sw;
            }
            T* out = plane + c * V;
            for (int hb = group; hb < nrows; hb += U * ngroups, out += U * stride) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int hh = hb + u * ngroups;
                    if (hh >= nrows) break;
                    const int4 ro = rowinfo[hh];
                    T res[V];
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        T acc = T(0);
                        if (MAXW > 0) {
                            const int row_at[3] = {ro.x, ro.y, ro.z};
                            const int col_at[3] = {col[k].a, col[k].b, col[k].c};
#pragma unroll
                            for (int r = 0; r < MAXW; ++r)
#pragma unroll
                                for (int b = 0; b < MAXW; ++b) {
                                    const int at_ = row_at[r] + col_at[b];
                                    acc += tap[at_] == ro.w - r * row_step + cp[k] - b * g.sw ? q[at_] : T(0);
                                }
                        } else {
                            for (int a = 0; a < ro.y; ++a)
                                for (int b = 0; b < col[k].nj; ++b) {
                                    const int at_ = ro.x + a * pitch + col[k].j_lo + b;
                                    if (tap[at_] == ro.w - a * row_step + cp[k] - b * g.sw) acc += q[at_];
                                }
                        }
                        res[k] = acc;
                    }
                    band_store<T, V>(out + u * stride, res);
                }
            }
        }
        it = nx;
        mis_go = nmis_go;
        mis_idx = nmis_idx;
        cur ^= 1;
    }
}

// kernel 3x3, stride 2, padding 1, W % 8 == 0.  A thread owns the 2x8 block of gradient rows
// (2m, 2m+1), columns [8jg, 8jg+8): two 32-byte stores.  Row 2m is covered by output row m
// only, row 2m+1 by rows m and m+1; even columns by one output column, odd columns by two.
// Ten quotients go/9 (five per output row) feed all sixteen sums, which are added in
// ascending (i, j) as the reference does.  The kernel is bound by instruction issue as much
// as by memory, hence the two rows per thread (index arithmetic and quotients are shared).
template <typename T>
__global__ void __launch_bounds__(kThreads)
avgpool3x3s2p1_bwd(const T* __restrict__ go, T* __restrict__ gx, int H, int W, int Ho, int Wo, int64_t blocks,
                   kd::FastDiv by_bpr, kd::FastDiv by_hh) {
    kd::pdl_prologue();
    for (int64_t bi = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; bi < blocks;
         bi += static_cast<int64_t>(gridDim.x) * kThreads) {
        unsigned rowp, ujg, nc, um;                    // rowp = nc * ceil(H/2) + m
        by_bpr.divmod(static_cast<unsigned>(bi), rowp, ujg);
        by_hh.divmod(rowp, nc, um);
        const int jg = static_cast<int>(ujg), m = static_cast<int>(um);
        const T* gplane = go + static_cast<int64_t>(nc) * Ho * Wo;
        const bool has_fifth = 4 * jg + 4 < Wo;        // the fifth quotient has a window
        const bool second = m + 1 < Ho;                // output row m+1 exists
        const T* p0 = gplane + static_cast<int64_t>(m) * Wo + 4 * jg;
        const Pack4<T> a0 = kd::load4(p0);
        const T e0 = has_fifth ? __ldg(p0 + 4) : T(0);
        Pack4<T> a1;
        a1.v[0] = a1.v[1] = a1.v[2] = a1.v[3] = T(0);
        T e1 = T(0);
        if (second) {
            a1 = kd::load4(p0 + Wo);
            e1 = has_fifth ? __ldg(p0 + Wo + 4) : T(0);
        }
        T q[2][5];
#pragma unroll
        for (int k = 0; k < 4; ++k) { q[0][k] = div9<T>(a0.v[k]); q[1][k] = div9<T>(a1.v[k]); }
        q[0][4] = div9<T>(e0);
        q[1][4] = div9<T>(e1);
        T* r0 = gx + (static_cast<int64_t>(nc) * H + 2 * m) * W + 8 * jg;
        {   // row 2m: output row m
            kd::Row8<T> out;
#pragma unroll
            for (int cidx = 0; cidx < 8; ++cidx) {
                T acc = T(0);
                acc += q[0][cidx >> 1];
                if ((cidx & 1) && (has_fifth || cidx != 7)) acc += q[0][(cidx >> 1) + 1];
                out.v[cidx] = acc;
            }
            kd::store8(r0, out);
        }
        if (2 * m + 1 < H) {   // row 2m+1: output rows m and m+1
            kd::Row8<T> out;
#pragma unroll
            for (int cidx = 0; cidx < 8; ++cidx) {
                const bool two = (cidx & 1) && (has_fifth || cidx != 7);
                T acc = T(0);
                acc += q[0][cidx >> 1];
                if (two) acc += q[0][(cidx >> 1) + 1];
                if (second) {
                    acc += q[1][cidx >> 1];
                    if (two) acc += q[1][(cidx >> 1) + 1];
                }
                out.v[cidx] = acc;
            }
            kd::store8(r0 + W, out);
        }
    }
}

// ===========================================================================
// Global average pool
// ===========================================================================
// Short rows (L = H*W <= 64): a warp stages 32 consecutive rows (one contiguous,
// 16-byte aligned span) in shared memory with coalesced 16-byte loads, then lane
// r adds row r serially in (h, w) order and divides by T(L): the arithmetic of the
// reference's one-thread-per-row loop (keydnn_global_avgpool2d_cuda.cu:47-60),
// bit for bit, but with coalesced traffic.  Odd L makes the per-lane stride
// conflict-free; even L is padded by one word per row.
template <typename T, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
gap_fwd_short(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int L, int Ls) {
    kd::pdl_prologue();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* sm = reinterpret_cast<T*>(smem_raw) + static_cast<size_t>(threadIdx.x >> 5) * 32 * Ls;
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * WARPS;
    const int64_t chunks = (rows + 31) >> 5;
    for (int64_t ch = static_cast<int64_t>(blockIdx.x) * WARPS + (threadIdx.x >> 5); ch < chunks; ch += nwarps) {
        const int64_t r0 = ch << 5;
        const int nrow = (rows - r0 < 32) ? static_cast<int>(rows - r0) : 32;
        const int count = nrow * L;
        const T* src = x + r0 * L;
        const int c4 = count >> 2;
        if (Ls == L) {
            // Shared layout == global layout: asynchronous 16-byte copies straight into shared
            // memory, every piece of the span in flight at once, no register staging.
            const int pieces = static_cast<int>((static_cast<size_t>(count) * sizeof(T)) >> 4);
            const char* gsrc = reinterpret_cast<const char*>(src);
            const unsigned sdst = static_cast<unsigned>(__cvta_generic_to_shared(sm));
            for (int q = lane; q < pieces; q += 32)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(sdst + 16u * q), "l"(gsrc + 16 * q) : "memory");
            asm volatile("cp.async.commit_group;" ::: "memory");
            const int done = static_cast<int>((static_cast<size_t>(pieces) << 4) / sizeof(T));
            for (int e = done + lane; e < count; e += 32) sm[e] = src[e];
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        } else {
            // padded rows: stage through registers, four packets per lane in flight per trip
            for (int p0 = lane; p0 < c4; p0 += 128) {
                Pack4<T> v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (p0 + 32 * u < c4) v[u] = kd::load4_stream(src + 4 * (p0 + 32 * u));
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int p = p0 + 32 * u;
                    if (p < c4) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int e = 4 * p + k;
                            const int rr = e / L;
                            sm[rr * Ls + (e - rr * L)] = v[u].v[k];
                        }
                    }
                }
            }
            for (int e = (c4 << 2) + lane; e < count; e += 32) {
                const int rr = e / L;
                sm[rr * Ls + (e - rr * L)] = src[e];
            }
        }
        __syncwarp();
        if (lane < nrow) {
            const T* rp = sm + lane * Ls;
            T sum = T(0);
            for (int k = 0; k < L; ++k) sum += rp[k];
            y[r0 + lane] = sum / static_cast<T>(L);
        }
        __syncwarp();
    }
}

// Long rows: one warp per row, 16-byte loads when rows are aligned, partial sums
// in T per lane, combined in double.
template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads)
gap_fwd_long(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int L) {
    kd::pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * (kThreads / 32);
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5); r < rows; r += nwarps) {
        const T* src = x + r * L;
        T s0 = T(0), s1 = T(0), s2 = T(0), s3 = T(0);
        if (VEC) {
            const int c4 = L >> 2;
            for (int p = lane; p < c4; p += 32) {
                const Pack4<T> v = kd::load4_stream(src + 4 * p);
                s0 += v.v[0]; s1 += v.v[1]; s2 += v.v[2]; s3 += v.v[3];
            }
        } else {
            for (int e = lane; e < L; e += 32) s0 += src[e];
        }
        double s = (static_cast<double>(s0) + static_cast<double>(s1)) +
                   (static_cast<double>(s2) + static_cast<double>(s3));
        s = kd::warp_sum(s);
        if (lane == 0) y[r] = static_cast<T>(s) / static_cast<T>(L);
    }
}

// Backward (keydnn_global_avgpool2d_cuda.cu:69-97): gx = go[row] * (T(1)/T(L)),
// a multiply by the rounded reciprocal.
template <typename T>
__global__ void __launch_bounds__(kThreads)
gap_bwd(const T* __restrict__ go, T* __restrict__ gx, int64_t total, int L, bool vec) {
    kd::pdl_prologue();
    const T scale = T(1) / static_cast<T>(L);
    if (vec) {
        const int64_t n4 = total >> 2;
        const bool small = total < (int64_t(1) << 31);      // 32-bit index arithmetic is enough
        for (int64_t p = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; p < n4;
             p += static_cast<int64_t>(gridDim.x) * kThreads) {
            const int64_t e0 = p << 2;
            int64_t row;
            int rem;
            if (small) {
                const unsigned e32 = static_cast<unsigned>(e0);
                const unsigned r32 = e32 / static_cast<unsigned>(L);
                row = r32;
                rem = static_cast<int>(e32 - r32 * static_cast<unsigned>(L));
            } else {
                row = e0 / L;
                rem = static_cast<int>(e0 - row * L);
            }
            Pack4<T> out;
            if (L >= 4) {
                // a packet touches at most two rows
                const T g0 = __ldg(go + row) * scale;
                const bool spill = rem + 3 >= L;
                const T g1 = spill ? __ldg(go + row + 1) * scale : g0;
#pragma unroll
                for (int k = 0; k < 4; ++k) out.v[k] = (rem + k >= L) ? g1 : g0;
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    while (rem >= L) { rem -= L; ++row; }
                    out.v[k] = __ldg(go + row) * scale;
                    ++rem;
                }
            }
            kd::store4(gx + e0, out);
        }
        if (blockIdx.x == 0 && threadIdx.x < 4) {
            const int64_t e = (n4 << 2) + threadIdx.x;
            if (e < total) gx[e] = go[e / L] * scale;
        }
    } else {
        for (int64_t e = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; e < total;
             e += static_cast<int64_t>(gridDim.x) * kThreads)
            gx[e] = __ldg(go + e / L) * scale;
    }
}

// ===========================================================================
// pad / crop
// ===========================================================================
template <typename T>
__global__ void __launch_bounds__(kThreads)
pad2d_kernel(const T* __restrict__ x, T* __restrict__ y, int H, int W, int ph, int pw, T value, int64_t total) {
    kd::pdl_prologue();
    const int Hp = H + 2 * ph, Wp = W + 2 * pw;
    for (int64_t o = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; o < total;
         o += static_cast<int64_t>(gridDim.x) * kThreads) {
        const int wp = static_cast<int>(o % Wp);
        const int64_t t = o / Wp;
        const int hp = static_cast<int>(t % Hp);
        const int64_t nc = t / Hp;
        const int h = hp - ph, w = wp - pw;
        y[o] = (h >= 0 && h < H && w >= 0 && w < W) ? x[(nc * H + h) * W + w] : value;
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
crop2d_kernel(const T* __restrict__ xp, T* __restrict__ y, int Hp, int Wp, int ph, int pw, int H, int W,
              int64_t total) {
    kd::pdl_prologue();
    for (int64_t o = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; o < total;
         o += static_cast<int64_t>(gridDim.x) * kThreads) {
        const int w = static_cast<int>(o % W);
        const int64_t t = o / W;
        const int h = static_cast<int>(t % H);
        const int64_t nc = t / H;
        const int hp = h + ph, wp = w + pw;
        if (hp < Hp && wp < Wp) y[o] = xp[(nc * Hp + hp) * Wp + wp];
    }
}

// Row-wise forms: a warp owns four consecutive rows of the output (one multiply-high per ROW instead of four 64-bit
// divisions per ELEMENT), its lanes walk the rows, so loads and stores are contiguous; the loads of the four rows are
// issued before the first store, which keeps enough bytes in flight for rows as short as 56 elements.  rows < 2^31.
constexpr int kRowsPerWarp = 4;

template <typename T>
__global__ void __launch_bounds__(kThreads)
pad2d_rows_kernel(const T* __restrict__ x, T* __restrict__ y, int H, int W, int ph, int pw, T value, unsigned rows,
                  kd::FastDiv by_hp) {
    kd::pdl_prologue();
    const int Hp = H + 2 * ph, Wp = W + 2 * pw;
    const int lane = threadIdx.x & 31;
    for (unsigned r0 = (blockIdx.x * kWarps + (threadIdx.x >> 5)) * kRowsPerWarp; r0 < rows; r0 += gridDim.x * kWarps * kRowsPerWarp) {
        const T* src[kRowsPerWarp];
        bool live[kRowsPerWarp], data[kRowsPerWarp];
#pragma unroll
        for (int u = 0; u < kRowsPerWarp; ++u) {
            const unsigned r = r0 + u;
            live[u] = r < rows;
            const unsigned nc = by_hp.div(live[u] ? r : 0u);
            const int h = static_cast<int>((live[u] ? r : 0u) - nc * static_cast<unsigned>(Hp)) - ph;
            data[u] = live[u] && h >= 0 && h < H;
            src[u] = x + (static_cast<int64_t>(nc) * H + (data[u] ? h : 0)) * W - pw;
        }
        T* dst = y + static_cast<int64_t>(r0) * Wp;
#pragma unroll 1
        for (int w = lane; w < Wp; w += 32) {
            const bool inside = w >= pw && w < pw + W;
            T v[kRowsPerWarp];
#pragma unroll
            for (int u = 0; u < kRowsPerWarp; ++u) v[u] = (data[u] && inside) ? __ldcs(src[u] + w) : value;
#pragma unroll
            for (int u = 0; u < kRowsPerWarp; ++u)
                if (live[u]) __stcs(dst + static_cast<int64_t>(u) * Wp + w, v[u]);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
crop2d_rows_kernel(const T* __restrict__ xp, T* __restrict__ y, int Hp, int Wp, int ph, int pw, int H, int W, unsigned rows,
                   kd::FastDiv by_h) {
    kd::pdl_prologue();
    const int lane = threadIdx.x & 31;
    for (unsigned r0 = (blockIdx.x * kWarps + (threadIdx.x >> 5)) * kRowsPerWarp; r0 < rows; r0 += gridDim.x * kWarps * kRowsPerWarp) {
        const T* src[kRowsPerWarp];
        bool live[kRowsPerWarp];
#pragma unroll
        for (int u = 0; u < kRowsPerWarp; ++u) {
            const unsigned r = r0 + u;
            const bool in_range = r < rows;
            const unsigned nc = by_h.div(in_range ? r : 0u);
            const int hp = static_cast<int>((in_range ? r : 0u) - nc * static_cast<unsigned>(H)) + ph;
            live[u] = in_range && hp < Hp;            // rows the padded plane does not have stay untouched, as in the flat kernel
            src[u] = xp + (static_cast<int64_t>(nc) * Hp + (live[u] ? hp : 0)) * Wp + pw;
        }
        T* dst = y + static_cast<int64_t>(r0) * W;
#pragma unroll 1
        for (int w = lane; w < W; w += 32) {
            const bool inside = w + pw < Wp;
            T v[kRowsPerWarp];
#pragma unroll
            for (int u = 0; u < kRowsPerWarp; ++u) v[u] = (live[u] && inside) ? __ldcs(src[u] + w) : T(0);
#pragma unroll
            for (int u = 0; u < kRowsPerWarp; ++u)
                if (live[u] && inside) __stcs(dst + static_cast<int64_t>(u) * W + w, v[u]);
        }
    }
}

// ===========================================================================
// Host-side dispatch
// ===========================================================================
inline unsigned flat_grid(int64_t items, int per_sm = 8) {
    return kd::grid_for((items + kThreads - 1) / kThreads, per_sm);
}

inline bool out_dims_ok(const PoolGeom& g) {
    // every window must start inside the padded plane
    return (static_cast<int64_t>(g.Ho - 1) * g.sh < g.H + 2 * g.ph) &&
           (static_cast<int64_t>(g.Wo - 1) * g.sw < g.W + 2 * g.pw);
}

// the geometry of the 3x3 / stride 2 / padding 1 kernels: rows of a multiple of eight elements, every output present
inline bool is_3x3s2p1(const PoolGeom& g) {
    return g.kh == 3 && g.kw == 3 && g.sh == 2 && g.sw == 2 && g.ph == 1 && g.pw == 1 && (g.W % 8 == 0) && g.Wo == g.W / 2 &&
           g.Ho == (g.H - 1) / 2 + 1;
}

// the geometry of the 2x2 / stride 2 AvgPool kernels: no padding, rows of a multiple of eight elements, every window present
inline bool is_2x2s2p0(const PoolGeom& g) {
    return g.kh == 2 && g.kw == 2 && g.sh == 2 && g.sw == 2 && g.ph == 0 && g.pw == 0 && (g.W % 8 == 0) && g.Wo == g.W / 2 &&
           g.Ho == g.H / 2;
}

// most windows that cover one element along an axis, as far as the branch-free backward kernels go: 2, 3, or 0 (more)
inline int band_max_windows(const PoolGeom& g) {
    if (g.kh <= 2 * g.sh && g.kw <= 2 * g.sw) return 2;
    if (g.kh <= 3 * g.sh && g.kw <= 3 * g.sw) return 3;
    return 0;
}

// forward bands: the number of output columns whose windows reach over the left or right edge of the plane (a divisor)
inline kd::FastDiv band_edge_cols(const PoolGeom& g) {
    const int ja = (g.pw + g.sw - 1) / g.sw;
    const int jb = g.W - g.kw + g.pw >= 0 ? std::min(g.Wo - 1, (g.W - g.kw + g.pw) / g.sw) : -1;
    const int n = jb < ja ? 0 : ja + (g.Wo - 1 - jb);
    return kd::FastDiv(static_cast<unsigned>(n > 0 ? n : 1));
}

// the band kernels index inside a plane with 32-bit integers
inline bool band_indexable(const PoolGeom& g) {
    return static_cast<int64_t>(g.H) * g.W < (int64_t(1) << 31) && static_cast<int64_t>(g.Ho) * g.Wo < (int64_t(1) << 31);
}

// no window reaches outside the plane: no padding, and the last window ends inside
inline bool windows_inside(const PoolGeom& g) {
    return g.ph == 0 && g.pw == 0 && static_cast<int64_t>(g.Ho - 1) * g.sh + g.kh <= g.H &&
           static_cast<int64_t>(g.Wo - 1) * g.sw + g.kw <= g.W;
}

template <typename T>
int maxpool_forward(const T* x, T* y, long long* idx, int N, int C, PoolGeom g) {
    if (!x || !y || !idx) return -1;
    if (N <= 0 || C <= 0 || g.H <= 0 || g.W <= 0) return -2;
    if (g.Ho <= 0 || g.Wo <= 0 || g.kh <= 0 || g.kw <= 0) return -3;
    if (g.sh <= 0 || g.sw <= 0) return -4;
    if (g.ph < 0 || g.pw < 0 || !out_dims_ok(g)) return -5;
    (void)cudaGetLastError();
    const int64_t nc = static_cast<int64_t>(N) * C;
    const int64_t total = nc * g.Ho * g.Wo;
    const bool fast = g.kh == 2 && g.kw == 2 && g.sh == 2 && g.sw == 2 && g.ph == 0 && g.pw == 0 &&
                      (g.W % 8 == 0) && g.Wo == g.W / 2 && g.Ho <= g.H / 2 && kd::aligned_row8<T>(x) &&
                      kd::aligned_pack<T>(y) && kd::aligned_pack<long long>(idx) && total < (int64_t(1) << 32);
    if (fast) {
        constexpr int U = 2;
        const int64_t groups = total >> 2;
        KD_LAUNCH((maxpool2x2_fwd<T, U>), (groups + kThreads * U - 1) / (kThreads * U), kThreads, 0, x, y, idx, g.H, g.W,
                  g.Ho, g.Wo, groups, kd::FastDiv(g.Wo / 4), kd::FastDiv(g.Ho));
        return kd::launch_status();
    }
    if (is_3x3s2p1(g) && kd::aligned_row8<T>(x) && kd::aligned_pack<T>(y) && kd::aligned_pack<long long>(idx) &&
        total < (int64_t(1) << 32)) {
        const int64_t groups = total >> 2;
        KD_LAUNCH1(maxpool3x3s2p1_fwd<T>, (groups + kThreads - 1) / kThreads, kThreads, 0, x, y, idx, g.H, g.W, g.Ho, g.Wo, groups,
                   kd::FastDiv(g.Wo / 4), kd::FastDiv(g.Ho));
        return kd::launch_status();
    }
    const BandPlan plan = band_plan_fwd<T>(g);
    if (plan.ok && nc * plan.bands < (int64_t(1) << 31) && band_indexable(g)) {
        const unsigned items = static_cast<unsigned>(nc * plan.bands);
        const kd::FastDiv by_bands(plan.bands);
        const int threads = band_threads(static_cast<int64_t>(plan.rows) * g.Wo);
        const int lanes = band_lane_bits(g.Wo, threads);
        const bool inside = windows_inside(g);
#define KD_FWD_BAND(KH_, KW_, EDGES_)                                                                               \
    KD_LAUNCH_W((maxpool_fwd_band<T, KH_, KW_, EDGES_>), 2, items, threads, plan.smem, x, y, idx, g, plan.rows, items, \
                by_bands, lanes, plan.buffer, kd::FastDiv(g.Wo), band_edge_cols(g))
        if (g.kh == 3 && g.kw == 3) { if (inside) KD_FWD_BAND(3, 3, false); else KD_FWD_BAND(3, 3, true); }
        else if (g.kh == 2 && g.kw == 2) { if (inside) KD_FWD_BAND(2, 2, false); else KD_FWD_BAND(2, 2, true); }
        else if (inside) KD_FWD_BAND(0, 0, false);
        else KD_FWD_BAND(0, 0, true);
#undef KD_FWD_BAND
    } else {
        (void)kd::launch(maxpool_fwd_generic<T>, dim3(flat_grid(total)), kThreads, 0, x, y, idx, g, total);
    }
    return kd::launch_status();
}

template <typename T>
int maxpool_backward_ex(const T* go, const long long* idx, T* gx, int N, int C, PoolGeom g) {
    if (!go || !idx || !gx) return -1;
    if (N <= 0 || C <= 0 || g.H <= 0 || g.W <= 0) return -2;
    if (g.Ho <= 0 || g.Wo <= 0 || g.kh <= 0 || g.kw <= 0) return -3;
    if (g.sh <= 0 || g.sw <= 0) return -4;
    if (g.ph < 0 || g.pw < 0 || !out_dims_ok(g)) return -5;
    (void)cudaGetLastError();
    const int64_t nc = static_cast<int64_t>(N) * C;
    const bool fast = g.kh == 2 && g.kw == 2 && g.sh == 2 && g.sw == 2 && g.ph == 0 && g.pw == 0 &&
                      (g.W % 8 == 0) && (g.H % 2 == 0) && g.Wo == g.W / 2 && g.Ho == g.H / 2 &&
                      kd::aligned_pack<T>(go) && kd::aligned_row8<T>(gx) && kd::aligned_pack<long long>(idx) &&
                      nc * g.H * g.W < (int64_t(1) << 33);
    if (fast) {
        constexpr int U = 2;
        const int64_t blocks = (nc * g.H * g.W) >> 3;
        KD_LAUNCH((maxpool2x2_bwd<T, U>), (blocks + kThreads * U - 1) / (kThreads * U), kThreads, 0, go, idx, gx, g.H,
                  g.W, g.Ho, g.Wo, blocks, kd::FastDiv(g.W / 8), kd::FastDiv(g.H));
        return kd::launch_status();
    }
    if (is_3x3s2p1(g) && kd::aligned_pack<T>(go) && kd::aligned_pack<long long>(idx) && kd::aligned_row8<T>(gx) &&
        nc * g.H * g.W < (int64_t(1) << 33)) {
        const int64_t blocks = nc * ((g.H + 1) / 2) * (g.W / 8);
        KD_LAUNCH(maxpool3x3s2p1_bwd<T>, (blocks + kThreads - 1) / kThreads, kThreads, 0, go, idx, gx, g.H, g.W, g.Ho, g.Wo, blocks,
                  kd::FastDiv(g.W / 8), kd::FastDiv((g.H + 1) / 2));
        return kd::launch_status();
    }
    const BandPlanMax plan = band_plan_maxbwd<T>(g);
    const int64_t padded = static_cast<int64_t>(g.H + 2 * g.ph) * (g.W + 2 * g.pw);
    if (plan.ok && nc * plan.bands < (int64_t(1) << 31) && padded < (int64_t(1) << 31) && band_indexable(g)) {
        const unsigned items = static_cast<unsigned>(nc * plan.bands);
        const kd::FastDiv by_bands(plan.bands), by_sh(g.sh), by_sw(g.sw), by_wo(g.Wo), by_wp(g.W + 2 * g.pw);
        const int maxw = band_max_windows(g);
        int v = 16 / static_cast<int>(sizeof(T));
        while (v > 1 && (g.W % v != 0 || (reinterpret_cast<uintptr_t>(gx) % (v * sizeof(T))) != 0)) v /= 2;
        const int threads = band_threads(static_cast<int64_t>(plan.rows) * (g.W / v) / (8 / v));
        const int lanes = band_lane_bits(g.W / v, threads);
#define KD_BWD_BAND_V(MAXW_, V_)                                                                                     \
    KD_LAUNCH_W((maxpool_bwd_band<T, MAXW_, V_>), 2, items, threads, plan.smem, go, idx, gx, g, plan.rows, items, by_bands, \
                lanes, by_sh, by_sw, by_wo, by_wp, plan.staged, plan.buffer)
#define KD_BWD_BAND(MAXW_)                                                                                          \
    do {                                                                                                            \
        if (v == 4) { if constexpr (sizeof(T) == 4) KD_BWD_BAND_V(MAXW_, 4); }                                      \
        else if (v == 2) KD_BWD_BAND_V(MAXW_, 2);                                                                   \
        else KD_BWD_BAND_V(MAXW_, 1);                                                                               \
    } while (0)
        if (maxw == 2) KD_BWD_BAND(2);
        else if (maxw == 3) KD_BWD_BAND(3);
        else KD_BWD_BAND(0);
#undef KD_BWD_BAND_V
#undef KD_BWD_BAND
    } else {
        const int64_t total = nc * g.H * g.W;
        (void)kd::launch(maxpool_bwd_gather<T>, dim3(flat_grid(total)), kThreads, 0, go, idx, gx, g, total);
    }
    return kd::launch_status();
}

template <typename T>
int maxpool_backward_legacy(const T* go, const long long* idx, T* gx_pad, int N, int C, int Ho, int Wo, int Hp,
                            int Wp) {
    if (!go || !idx || !gx_pad) return -1;
    if (N <= 0 || C <= 0) return -2;
    if (Ho <= 0 || Wo <= 0 || Hp <= 0 || Wp <= 0) return -3;
    (void)cudaGetLastError();
    const int64_t total = static_cast<int64_t>(N) * C * Ho * Wo;
    (void)kd::launch(maxpool_bwd_scatter<T>, dim3(flat_grid(total)), kThreads, 0, go, idx, gx_pad, Ho, Wo, Hp, Wp, total);
    return kd::launch_status();
}

template <typename T>
int avgpool_forward(const T* x, T* y, int N, int C, PoolGeom g) {
    if (!x || !y) return -1;
    if (N <= 0 || C <= 0) return -2;
    if (g.H <= 0 || g.W <= 0 || g.Ho <= 0 || g.Wo <= 0) return -3;
    if (g.kh <= 0 || g.kw <= 0 || g.sh <= 0 || g.sw <= 0) return -4;
    if (g.ph < 0 || g.pw < 0 || !out_dims_ok(g)) return -5;
    (void)cudaGetLastError();
    const int64_t nc = static_cast<int64_t>(N) * C;
    const int64_t total = nc * g.Ho * g.Wo;
    const bool fast = g.kh == 3 && g.kw == 3 && g.sh == 2 && g.sw == 2 && g.ph == 1 && g.pw == 1 &&
                      (g.W % 8 == 0) && g.Wo == g.W / 2 && g.Ho == (g.H - 1) / 2 + 1 && kd::aligned_row8<T>(x) &&
                      kd::aligned_pack<T>(y) && total < (int64_t(1) << 32);
    if (fast) {
        const int64_t groups = total >> 2;
        KD_LAUNCH1(avgpool3x3s2p1_fwd<T>, (groups + kThreads - 1) / kThreads, kThreads, 0, x, y, g.H, g.W, g.Ho, g.Wo, groups,
                   kd::FastDiv(g.Wo / 4), kd::FastDiv(g.Ho));
        return kd::launch_status();
    }
    if (is_2x2s2p0(g) && kd::aligned_row8<T>(x) && kd::aligned_pack<T>(y) && total < (int64_t(1) << 32)) {
        constexpr int U = 2;
        const int64_t groups = total >> 2;
        KD_LAUNCH((avgpool2x2_fwd<T, U>), (groups + kThreads * U - 1) / (kThreads * U), kThreads, 0, x, y, g.H, g.W, g.Ho, g.Wo,
                  groups, kd::FastDiv(g.Wo / 4), kd::FastDiv(g.Ho));
        return kd::launch_status();
    }
    const BandPlan plan = band_plan_fwd<T>(g);
    if (plan.ok && nc * plan.bands < (int64_t(1) << 31) && band_indexable(g)) {
        const unsigned items = static_cast<unsigned>(nc * plan.bands);
        const kd::FastDiv by_bands(plan.bands);
        const int threads = band_threads(static_cast<int64_t>(plan.rows) * g.Wo);
        const int lanes = band_lane_bits(g.Wo, threads);
        const bool inside = windows_inside(g);
#define KD_FWD_BAND(KH_, KW_, EDGES_)                                                                               \
    KD_LAUNCH_W((avgpool_fwd_band<T, KH_, KW_, EDGES_>), 2, items, threads, plan.smem, x, y, g, plan.rows, items, by_bands, lanes, \
                plan.buffer, kd::FastDiv(g.Wo), band_edge_cols(g))
        if (g.kh == 3 && g.kw == 3) { if (inside) KD_FWD_BAND(3, 3, false); else KD_FWD_BAND(3, 3, true); }
        else if (g.kh == 2 && g.kw == 2) { if (inside) KD_FWD_BAND(2, 2, false); else KD_FWD_BAND(2, 2, true); }
        else if (inside) KD_FWD_BAND(0, 0, false);
        else KD_FWD_BAND(0, 0, true);
#undef KD_FWD_BAND
    } else {
        (void)kd::launch(avgpool_fwd_generic<T>, dim3(flat_grid(total)), kThreads, 0, x, y, g, total);
    }
    return kd::launch_status();
}

template <typename T>
int avgpool_backward(const T* go, T* gx, int N, int C, PoolGeom g, bool accumulate) {
    if (!go || !gx) return -1;
    if (N <= 0 || C <= 0) return -2;
    if (g.Ho <= 0 || g.Wo <= 0 || g.H <= 0 || g.W <= 0) return -3;
    if (g.kh <= 0 || g.kw <= 0 || g.sh <= 0 || g.sw <= 0) return -4;
    if (g.ph < 0 || g.pw < 0) return -5;
    (void)cudaGetLastError();
    const int64_t nc = static_cast<int64_t>(N) * C;
    const int64_t total = nc * g.H * g.W;
    const bool fast = !accumulate && g.kh == 3 && g.kw == 3 && g.sh == 2 && g.sw == 2 && g.ph == 1 && g.pw == 1 &&
                      (g.W % 8 == 0) && g.Wo == g.W / 2 && g.Ho == (g.H - 1) / 2 + 1 && kd::aligned_pack<T>(go) &&
                      kd::aligned_row8<T>(gx) && total < (int64_t(1) << 33);
    if (fast) {
        const int64_t blocks = nc * ((g.H + 1) / 2) * (g.W / 8);
        KD_LAUNCH(avgpool3x3s2p1_bwd<T>, (blocks + kThreads - 1) / kThreads, kThreads, 0, go, gx, g.H, g.W, g.Ho, g.Wo, blocks,
                  kd::FastDiv(g.W / 8), kd::FastDiv((g.H + 1) / 2));
        return kd::launch_status();
    }
    if (is_2x2s2p0(g) && kd::aligned_pack<T>(go) && kd::aligned_row8<T>(gx) && total < (int64_t(1) << 33)) {
        constexpr int U = 2;
        const int64_t blocks = total >> 3;
        const kd::FastDiv by_bpr(g.W / 8), by_h(g.H);
        if (accumulate)
            KD_LAUNCH((avgpool2x2_bwd<T, true, U>), (blocks + kThreads * U - 1) / (kThreads * U), kThreads, 0, go, gx, g.H, g.W,
                      g.Ho, g.Wo, blocks, by_bpr, by_h);
        else
            KD_LAUNCH((avgpool2x2_bwd<T, false, U>), (blocks + kThreads * U - 1) / (kThreads * U), kThreads, 0, go, gx, g.H, g.W,
                      g.Ho, g.Wo, blocks, by_bpr, by_h);
        return kd::launch_status();
    }
    const BandPlan plan = band_plan_bwd<T>(g);
    if (plan.ok && nc * plan.bands < (int64_t(1) << 31) && band_indexable(g)) {
        const unsigned items = static_cast<unsigned>(nc * plan.bands);
        const kd::FastDiv by_bands(plan.bands), by_sh(g.sh), by_sw(g.sw);
        const kd::FastDiv by_wo(g.Wo);
        const int maxw = band_max_windows(g);
        // columns per thread: as many as one aligned access of up to 16 bytes holds, for every row of every plane
        int v = 16 / static_cast<int>(sizeof(T));
        while (v > 1 && (g.W % v != 0 || (reinterpret_cast<uintptr_t>(gx) % (v * sizeof(T))) != 0)) v /= 2;
        const int threads = band_threads(static_cast<int64_t>(plan.rows) * (g.W / v) / (8 / v));
        const int lanes = band_lane_bits(g.W / v, threads);
#define KD_BWD_BAND_V(ACC, MAXW_, V_)                                                                                \
    KD_LAUNCH_W((avgpool_bwd_band<T, ACC, MAXW_, V_>), 2, items, threads, plan.smem, go, gx, g, plan.rows, items, by_bands, \
                lanes, by_sh, by_sw, by_wo, plan.buffer)
#define KD_BWD_BAND(ACC, MAXW_)                                                                                     \
    do {                                                                                                            \
        if (v == 4) { if constexpr (sizeof(T) == 4) KD_BWD_BAND_V(ACC, MAXW_, 4); }                                 \
        else if (v == 2) KD_BWD_BAND_V(ACC, MAXW_, 2);                                                              \
        else KD_BWD_BAND_V(ACC, MAXW_, 1);                                                                          \
    } while (0)
        if (accumulate) {
            if (maxw == 2) KD_BWD_BAND(true, 2);
            else if (maxw == 3) KD_BWD_BAND(true, 3);
            else KD_BWD_BAND(true, 0);
        } else {
            if (maxw == 2) KD_BWD_BAND(false, 2);
            else if (maxw == 3) KD_BWD_BAND(false, 3);
            else KD_BWD_BAND(false, 0);
        }
#undef KD_BWD_BAND_V
#undef KD_BWD_BAND
    } else if (accumulate) {
        (void)kd::launch(avgpool_bwd_gather<T, true>, dim3(flat_grid(total)), kThreads, 0, go, gx, g, total);
    } else {
        (void)kd::launch(avgpool_bwd_gather<T, false>, dim3(flat_grid(total)), kThreads, 0, go, gx, g, total);
    }
    return kd::launch_status();
}

template <typename T>
int gap_forward(const T* x, T* y, int N, int C, int H, int W) {
    if (!x || !y) return -1;
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0) return -2;
    (void)cudaGetLastError();
    const int64_t rows = static_cast<int64_t>(N) * C;
    const int64_t L64 = static_cast<int64_t>(H) * W;
    if (L64 > std::numeric_limits<int>::max()) return -2;
    const int L = static_cast<int>(L64);
    if (L <= 64 && kd::aligned_pack<T>(x)) {
        constexpr int WARPS = 4;
        const int Ls = (L & 1) ? L : L + 1;
        const size_t smem = static_cast<size_t>(WARPS) * 32 * Ls * sizeof(T);   // <= 66,560 bytes
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(gap_fwd_short<T, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);
        const int64_t chunks = (rows + 31) / 32;
        KD_LAUNCH1((gap_fwd_short<T, WARPS>), (chunks + WARPS - 1) / WARPS, WARPS * 32, smem, x, y, rows, L, Ls);
    } else {
        const unsigned grid = kd::grid_for((rows + 7) / 8, 8);
        const bool vec = kd::aligned_pack<T>(x) && (L % 4 == 0);
        if (vec) (void)kd::launch(gap_fwd_long<T, true>, dim3(grid), kThreads, 0, x, y, rows, L);
        else (void)kd::launch(gap_fwd_long<T, false>, dim3(grid), kThreads, 0, x, y, rows, L);
    }
    return kd::launch_status();
}

template <typename T>
int gap_backward(const T* go, T* gx, int N, int C, int H, int W) {
    if (!go || !gx) return -1;
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0) return -2;
    (void)cudaGetLastError();
    const int64_t L64 = static_cast<int64_t>(H) * W;
    if (L64 > std::numeric_limits<int>::max()) return -2;
    const int64_t total = static_cast<int64_t>(N) * C * L64;
    const bool vec = kd::aligned_pack<T>(gx);
    const int64_t items = vec ? (total >> 2) + 1 : total;
    KD_LAUNCH_W(gap_bwd<T>, 4, (items + kThreads - 1) / kThreads, kThreads, 0, go, gx, total, static_cast<int>(L64), vec);
    return kd::launch_status();
}

template <typename T>
int pad2d(const T* x, T* y, int N, int C, int H, int W, int ph, int pw, T value) {
    if (!x || !y) return -1;
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0) return -2;
    if (ph < 0 || pw < 0) return -3;
    (void)cudaGetLastError();
    const int64_t total = static_cast<int64_t>(N) * C * (H + 2 * ph) * (W + 2 * pw);
    if (ph == 0 && pw == 0)         // nothing to add: the reference pads even then (ops/pool2d_cuda_ext.py:56-184)
        return kd::status(cudaMemcpyAsync(y, x, static_cast<size_t>(total) * sizeof(T), cudaMemcpyDeviceToDevice, kd::stream()));
    const int64_t rows = static_cast<int64_t>(N) * C * (H + 2 * ph);
    if (rows < (int64_t(1) << 31)) {
        KD_LAUNCH_W(pad2d_rows_kernel<T>, 8, (rows + kWarps * kRowsPerWarp - 1) / (kWarps * kRowsPerWarp), kThreads, 0, x, y, H, W, ph, pw, value,
                    static_cast<unsigned>(rows), kd::FastDiv(static_cast<unsigned>(H + 2 * ph)));
        return kd::launch_status();
    }
    (void)kd::launch(pad2d_kernel<T>, dim3(flat_grid(total)), kThreads, 0, x, y, H, W, ph, pw, value, total);
    return kd::launch_status();
}

template <typename T>
int crop2d(const T* xp, T* y, int N, int C, int Hp, int Wp, int ph, int pw, int H, int W) {
    if (!xp || !y) return -1;
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0) return -2;
    if (Hp <= 0 || Wp <= 0) return -3;
    if (ph < 0 || pw < 0) return -4;
    (void)cudaGetLastError();
    const int64_t total = static_cast<int64_t>(N) * C * H * W;
    if (ph == 0 && pw == 0 && Hp == H && Wp == W)
        return kd::status(cudaMemcpyAsync(y, xp, static_cast<size_t>(total) * sizeof(T), cudaMemcpyDeviceToDevice, kd::stream()));
    const int64_t rows = static_cast<int64_t>(N) * C * H;
    if (rows < (int64_t(1) << 31)) {
        KD_LAUNCH_W(crop2d_rows_kernel<T>, 8, (rows + kWarps * kRowsPerWarp - 1) / (kWarps * kRowsPerWarp), kThreads, 0, xp, y, Hp, Wp, ph, pw, H, W,
                    static_cast<unsigned>(rows), kd::FastDiv(static_cast<unsigned>(H)));
        return kd::launch_status();
    }
    (void)kd::launch(crop2d_kernel<T>, dim3(flat_grid(total)), kThreads, 0, xp, y, Hp, Wp, ph, pw, H, W, total);
    return kd::launch_status();
}

inline PoolGeom geom(int H, int W, int Ho, int Wo, int kh, int kw, int sh, int sw, int ph, int pw) {
    PoolGeom g;
    g.H = H; g.W = W; g.Ho = Ho; g.Wo = Wo; g.kh = kh; g.kw = kw; g.sh = sh; g.sw = sw; g.ph = ph; g.pw = pw;
    return g;
}

}  // namespace

// ---------------------------------------------------------------------------
// C ABI: reference signatures (keydnn_maxpool2d_cuda.hpp:28-72,
// keydnn_avgpool2d_cuda.hpp:38-76, keydnn_global_avgpool2d_cuda.hpp:34-60,
// keydnn_pad2d_cuda.hpp).  The plane handed in is already padded, so these run
// the same kernels with padding 0 on (H_pad, W_pad).
// ---------------------------------------------------------------------------
#define KD_POOL_LEGACY(T, SUF)                                                                                     \
    KD_API int keydnn_cuda_maxpool2d_forward_##SUF(const T* x_pad, T* y, std::int64_t* argmax_idx, int N, int C,   \
                                                   int H_pad, int W_pad, int H_out, int W_out, int k_h, int k_w,   \
                                                   int s_h, int s_w) {                                             \
        return maxpool_forward<T>(x_pad, y, reinterpret_cast<long long*>(argmax_idx), N, C,                        \
                                  geom(H_pad, W_pad, H_out, W_out, k_h, k_w, s_h, s_w, 0, 0));                     \
    }                                                                                                              \
    KD_API int keydnn_cuda_maxpool2d_backward_##SUF(const T* grad_out, const std::int64_t* argmax_idx,             \
                                                    T* grad_x_pad, int N, int C, int H_out, int W_out, int H_pad,  \
                                                    int W_pad) {                                                   \
        return maxpool_backward_legacy<T>(grad_out, reinterpret_cast<const long long*>(argmax_idx), grad_x_pad, N, \
                                          C, H_out, W_out, H_pad, W_pad);                                          \
    }                                                                                                              \
    KD_API int keydnn_cuda_avgpool2d_forward_##SUF(const T* x_pad, T* y, int N, int C, int H_pad, int W_pad,       \
                                                   int H_out, int W_out, int k_h, int k_w, int s_h, int s_w) {     \
        return avgpool_forward<T>(x_pad, y, N, C, geom(H_pad, W_pad, H_out, W_out, k_h, k_w, s_h, s_w, 0, 0));     \
    }                                                                                                              \
    KD_API int keydnn_cuda_avgpool2d_backward_##SUF(const T* grad_out, T* grad_x_pad, int N, int C, int H_out,     \
                                                    int W_out, int H_pad, int W_pad, int k_h, int k_w, int s_h,    \
                                                    int s_w) {                                                     \
        return avgpool_backward<T>(grad_out, grad_x_pad, N, C,                                                     \
                                   geom(H_pad, W_pad, H_out, W_out, k_h, k_w, s_h, s_w, 0, 0), true);              \
    }                                                                                                              \
    KD_API int keydnn_cuda_global_avgpool2d_forward_##SUF(const T* x, T* y, int N, int C, int H, int W) {          \
        return gap_forward<T>(x, y, N, C, H, W);                                                                   \
    }                                                                                                              \
    KD_API int keydnn_cuda_global_avgpool2d_backward_##SUF(const T* grad_out, T* grad_x, int N, int C, int H,      \
                                                           int W) {                                                \
        return gap_backward<T>(grad_out, grad_x, N, C, H, W);                                                      \
    }                                                                                                              \
    KD_API int keydnn_cuda_pad2d_##SUF(const T* x, T* y_pad, int N, int C, int H, int W, int p_h, int p_w,         \
                                       T pad_value) {                                                              \
        return pad2d<T>(x, y_pad, N, C, H, W, p_h, p_w, pad_value);                                                \
    }                                                                                                              \
    KD_API int keydnn_cuda_crop2d_##SUF(const T* x_pad, T* y, int N, int C, int H_pad, int W_pad, int p_h,         \
                                        int p_w, int H, int W) {                                                   \
        return crop2d<T>(x_pad, y, N, C, H_pad, W_pad, p_h, p_w, H, W);                                            \
    }

KD_POOL_LEGACY(float, f32)
KD_POOL_LEGACY(double, f64)

// Host-only: how the row-band kernels would split a plane (nothing is launched).  kind 0: forward (rows = output rows
// of a band), 1: AvgPool backward, 2: MaxPool backward (rows = input rows of a band).  out5 = {usable, rows per band,
// bands per plane, dynamic shared memory in bytes, elements of one arrival buffer}.
KD_API int keydnn_cuda_debug_pool_band_plan(int kind, int elem_size, int H, int W, int H_out, int W_out, int k_h, int k_w, int s_h,
                                            int s_w, int p_h, int p_w, std::int64_t* out5) {
    if (!out5) return -1;
    if ((elem_size != 4 && elem_size != 8) || kind < 0 || kind > 2) return -2;
    if (H <= 0 || W <= 0 || H_out <= 0 || W_out <= 0 || k_h <= 0 || k_w <= 0 || s_h <= 0 || s_w <= 0 || p_h < 0 || p_w < 0) return -3;
    const PoolGeom g = geom(H, W, H_out, W_out, k_h, k_w, s_h, s_w, p_h, p_w);
    if (kind == 2) {
        const BandPlanMax p = elem_size == 4 ? band_plan_maxbwd<float>(g) : band_plan_maxbwd<double>(g);
        out5[0] = p.ok && band_indexable(g); out5[1] = p.rows; out5[2] = p.bands; out5[3] = static_cast<std::int64_t>(p.smem);
        out5[4] = p.buffer;
        return 0;
    }
    const BandPlan p = kind == 0 ? (elem_size == 4 ? band_plan_fwd<float>(g) : band_plan_fwd<double>(g))
                                 : (elem_size == 4 ? band_plan_bwd<float>(g) : band_plan_bwd<double>(g));
    out5[0] = p.ok && band_indexable(g); out5[1] = p.rows; out5[2] = p.bands; out5[3] = static_cast<std::int64_t>(p.smem);
    out5[4] = p.buffer;
    return 0;
}

// ---------------------------------------------------------------------------
// C ABI: fused entries (additive).  x / grad_x are the un-padded (N,C,H,W)
// tensors; argmax positions keep the reference encoding h*W_pad + w in the padded
// plane, W_pad = W + 2*p_w.  Backward overwrites grad_x (no zero-fill needed).
// They replace the pad -> pool and memset -> pool-backward -> crop sequences of
// ops/pool2d_cuda_ext.py:56-522.
// ---------------------------------------------------------------------------
#define KD_POOL_EX(T, SUF)                                                                                         \
    KD_API int keydnn_cuda_maxpool2d_forward_ex_##SUF(const T* x, T* y, std::int64_t* argmax_idx, int N, int C,    \
                                                      int H, int W, int H_out, int W_out, int k_h, int k_w,        \
                                                      int s_h, int s_w, int p_h, int p_w) {                        \
        return maxpool_forward<T>(x, y, reinterpret_cast<long long*>(argmax_idx), N, C,                            \
                                  geom(H, W, H_out, W_out, k_h, k_w, s_h, s_w, p_h, p_w));                         \
    }                                                                                                              \
    KD_API int keydnn_cuda_maxpool2d_backward_ex_##SUF(const T* grad_out, const std::int64_t* argmax_idx,          \
                                                       T* grad_x, int N, int C, int H, int W, int H_out,           \
                                                       int W_out, int k_h, int k_w, int s_h, int s_w, int p_h,     \
                                                       int p_w) {                                                  \
        return maxpool_backward_ex<T>(grad_out, reinterpret_cast<const long long*>(argmax_idx), grad_x, N, C,      \
                                      geom(H, W, H_out, W_out, k_h, k_w, s_h, s_w, p_h, p_w));                     \
    }                                                                                                              \
    KD_API int keydnn_cuda_avgpool2d_forward_ex_##SUF(const T* x, T* y, int N, int C, int H, int W, int H_out,     \
                                                      int W_out, int k_h, int k_w, int s_h, int s_w, int p_h,      \
                                                      int p_w) {                                                   \
        return avgpool_forward<T>(x, y, N, C, geom(H, W, H_out, W_out, k_h, k_w, s_h, s_w, p_h, p_w));             \
    }                                                                                                              \
    KD_API int keydnn_cuda_avgpool2d_backward_ex_##SUF(const T* grad_out, T* grad_x, int N, int C, int H, int W,   \
                                                       int H_out, int W_out, int k_h, int k_w, int s_h, int s_w,   \
                                                       int p_h, int p_w) {                                         \
        return avgpool_backward<T>(grad_out, grad_x, N, C,                                                         \
                                   geom(H, W, H_out, W_out, k_h, k_w, s_h, s_w, p_h, p_w), false);                 \
    }

KD_POOL_EX(float, f32)
KD_POOL_EX(double, f64)
