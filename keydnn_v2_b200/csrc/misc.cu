// Data-movement helpers either side of the pool / reduce kernels in a layer:
// broadcast_to (the backward of sum_to_shape and BatchNorm's per-channel
// expansion), bias_add (Linear) and transpose2d (Linear's W.T).
//
// Reference kernels replaced:
//   KeyDNNV2CudaNative/keydnn_cuda_broadcast_to.cu:58-131   N-D gather, no grid-stride
//   keydnn_tensor_bias_add.cu:30-47                         y = x + b[i % out]
//   keydnn_transpose2d.cu:4-12                              un-tiled transpose
#include "common.cuh"

namespace {

using kd::Pack4;

constexpr int kThreads = 256;
constexpr int kMaxDims = 8;

// status codes of the reference's broadcast_to (keydnn_cuda_broadcast_to.cu:6-10)
constexpr int ST_OK = 0, ST_BAD_PTR = 1, ST_CUDA_ERR = 2, ST_BAD_DIMS = 3, ST_BAD_SHAPE = 4;

struct GatherMeta {
    int ndim;
    int64_t out_stride[kMaxDims];
    int64_t in_stride[kMaxDims];   // 0 where the input extent is 1
};

template <typename T>
__global__ void __launch_bounds__(kThreads)
broadcast_gather_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t n, GatherMeta m) {
    kd::pdl_prologue();
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * kThreads) {
        int64_t rem = i, off = 0;
#pragma unroll
        for (int d = 0; d < kMaxDims; ++d) {
            if (d >= m.ndim) break;
            const int64_t q = rem / m.out_stride[d];
            rem -= q * m.out_stride[d];
            off += q * m.in_stride[d];
        }
        y[i] = __ldg(x + off);
    }
}

// y[(a*K + k)*B + b] = x[k]: every output row of B elements holds one value.
template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads)
broadcast_rows_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int K, int64_t B) {
    kd::pdl_prologue();
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const T v = __ldg(x + (r % K));
        T* dst = y + r * B;
        if (VEC) {
            Pack4<T> pk;
            pk.v[0] = pk.v[1] = pk.v[2] = pk.v[3] = v;
            const int64_t b4 = B >> 2;
            for (int64_t p = static_cast<int64_t>(blockIdx.y) * kThreads + threadIdx.x; p < b4;
                 p += static_cast<int64_t>(gridDim.y) * kThreads)
                kd::store4(dst + 4 * p, pk);
        } else {
            for (int64_t b = static_cast<int64_t>(blockIdx.y) * kThreads + threadIdx.x; b < B;
                 b += static_cast<int64_t>(gridDim.y) * kThreads)
                dst[b] = v;
        }
    }
}

// y[a, k] = x[k]: every output row is a copy of x.
template <typename T>
__global__ void __launch_bounds__(kThreads)
broadcast_cols_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t A, int64_t K) {
    kd::pdl_prologue();
    for (int64_t k = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; k < K;
         k += static_cast<int64_t>(gridDim.x) * kThreads) {
        const T v = __ldg(x + k);
        for (int64_t a = blockIdx.y; a < A; a += gridDim.y) y[a * K + k] = v;
    }
}

template <typename T>
int broadcast_to(const T* x, T* y, const int64_t* in_shape, int in_ndim, const int64_t* out_shape, int out_ndim) {
    if (!x || !y || !in_shape || !out_shape) return ST_BAD_PTR;
    if (out_ndim < 0 || in_ndim < 0) return ST_BAD_DIMS;
    if (out_ndim > kMaxDims) return ST_BAD_DIMS;
    if (in_ndim > out_ndim) return ST_BAD_SHAPE;
    int64_t in_p[kMaxDims], out_p[kMaxDims];
    const int pad = out_ndim - in_ndim;
    for (int i = 0; i < out_ndim; ++i) {
        out_p[i] = out_shape[i];
        in_p[i] = i < pad ? 1 : in_shape[i - pad];
        if (out_p[i] < 0 || in_p[i] < 0) return ST_BAD_SHAPE;
        const bool ok = (in_p[i] == out_p[i]) || (in_p[i] == 1);
        if (!ok) return ST_BAD_SHAPE;
    }
    int64_t n = 1;
    for (int i = 0; i < out_ndim; ++i) n *= out_p[i];
    if (n == 0) return ST_OK;
    (void)cudaGetLastError();
    cudaStream_t s = kd::stream();

    // collapse into alternating broadcast (B) / kept (K) groups
    int64_t ext[kMaxDims];
    bool bc[kMaxDims];
    int ng = 0;
    for (int d = 0; d < out_ndim; ++d) {
        if (out_p[d] == 1) continue;
        const bool b = (in_p[d] == 1);
        if (ng > 0 && bc[ng - 1] == b) ext[ng - 1] *= out_p[d];
        else { ext[ng] = out_p[d]; bc[ng] = b; ++ng; }
    }
    const int64_t imax = std::numeric_limits<int>::max();
    if (ng == 0 || (ng == 1 && !bc[0])) {
        cudaError_t st = cudaMemcpyAsync(y, x, n * sizeof(T), cudaMemcpyDeviceToDevice, s);
        return st == cudaSuccess ? ST_OK : ST_CUDA_ERR;
    }
    int64_t A = 1, K = 1, B = 1;
    bool pattern = false;
    if (ng == 1) { B = ext[0]; pattern = true; }                                   // [B]
    else if (ng == 2 && bc[0]) { A = ext[0]; K = ext[1]; pattern = true; }         // [B,K]
    else if (ng == 2 && !bc[0]) { K = ext[0]; B = ext[1]; pattern = true; }        // [K,B]
    else if (ng == 3 && bc[0]) { A = ext[0]; K = ext[1]; B = ext[2]; pattern = true; }   // [B,K,B]
    if (pattern && K <= imax) {
        if (B == 1) {
            unsigned gx = kd::grid_for((K + kThreads - 1) / kThreads, 8);
            int64_t gy = (static_cast<int64_t>(kd::sm_count()) * 8 + gx - 1) / gx;
            if (gy > A) gy = A;
            if (gy > 65535) gy = 65535;
            dim3 grid(gx, static_cast<unsigned>(gy));
            (void)kd::launch(broadcast_cols_kernel<T>, dim3(grid), kThreads, 0, x, y, A, K);
        } else {
            const int64_t rows = A * K;
            // few long rows: split each row over blockIdx.y so the machine stays full
            const unsigned gx = kd::grid_for(rows, 16);
            const int64_t per_row = (B / 4 + kThreads - 1) / kThreads;
            int64_t gy = (static_cast<int64_t>(kd::sm_count()) * 16 + gx - 1) / gx;
            if (gy > per_row) gy = per_row;
            if (gy < 1) gy = 1;
            if (gy > 65535) gy = 65535;
            const dim3 grid(gx, static_cast<unsigned>(gy));
            const bool vec = kd::aligned_pack<T>(y) && (B % 4 == 0);
            if (vec) (void)kd::launch(broadcast_rows_kernel<T, true>, dim3(grid), kThreads, 0, x, y, rows, static_cast<int>(K), B);
            else (void)kd::launch(broadcast_rows_kernel<T, false>, dim3(grid), kThreads, 0, x, y, rows, static_cast<int>(K), B);
        }
        return cudaGetLastError() == cudaSuccess ? ST_OK : ST_CUDA_ERR;
    }
    GatherMeta m;
    m.ndim = out_ndim;
    int64_t so = 1, si = 1;
    for (int d = out_ndim - 1; d >= 0; --d) {
        m.out_stride[d] = so;
        m.in_stride[d] = (in_p[d] == 1) ? 0 : si;
        so *= out_p[d];
        si *= in_p[d];
    }
    const unsigned grid = kd::grid_for((n + kThreads - 1) / kThreads, 8);
    (void)kd::launch(broadcast_gather_kernel<T>, dim3(grid), kThreads, 0, x, y, n, m);
    return cudaGetLastError() == cudaSuccess ? ST_OK : ST_CUDA_ERR;
}

// y[i] = x[i] + b[i % out]; x may alias y (the in-place form).
template <typename T>
__global__ void __launch_bounds__(kThreads)
bias_add_kernel(const T* x, const T* __restrict__ b, T* y, int64_t out, int64_t n) {
    kd::pdl_prologue();
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * kThreads)
        y[i] = x[i] + __ldg(b + (i % out));
}

// Packet path: `out` a multiple of 4 and every pointer packet-aligned, so a 4-element packet never straddles a
// row and its bias packet is b[4*(p % (out/4)) ...]; the row of packet p comes from a multiply-high division.
template <typename T, int UNROLL>
__global__ void __launch_bounds__(kThreads)
bias_add_packet_kernel(const T* x, const T* __restrict__ b, T* y, kd::FastDiv per_row, int64_t n4) {
    kd::pdl_prologue();
    const int64_t tile = static_cast<int64_t>(kThreads) * UNROLL;
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * tile; base < n4; base += static_cast<int64_t>(gridDim.x) * tile) {
        kd::Pack4<T> vx[UNROLL], vb[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t p = base + u * kThreads + threadIdx.x;
            if (p < n4) {
                vx[u] = kd::load4_stream(x + 4 * p);
                const unsigned q = static_cast<unsigned>(p);
                vb[u] = kd::load4(b + 4 * static_cast<int64_t>(q - per_row.div(q) * per_row.d));
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t p = base + u * kThreads + threadIdx.x;
            if (p < n4) {
#pragma unroll
                for (int k = 0; k < 4; ++k) vx[u].v[k] = vx[u].v[k] + vb[u].v[k];
                kd::store4(y + 4 * p, vx[u]);
            }
        }
    }
}

template <typename T>
int bias_add(const T* x, const T* b, T* y, int64_t batch, int64_t out) {
    if (!x || !b || !y) return static_cast<int>(cudaErrorInvalidDevicePointer);
    if (batch < 0 || out < 0) return static_cast<int>(cudaErrorInvalidValue);
    const int64_t n = batch * out;
    if (n <= 0) return 0;
    (void)cudaGetLastError();
    if (out % 4 == 0 && (n >> 2) < (1ll << 31) && kd::aligned_pack<T>(x) && kd::aligned_pack<T>(y) && kd::aligned_pack<T>(b)) {
        constexpr int UNROLL = 4;
        const int64_t n4 = n >> 2;
        KD_LAUNCH_W((bias_add_packet_kernel<T, UNROLL>), 64, (n4 + kThreads * UNROLL - 1) / (kThreads * UNROLL), kThreads, 0, x, b,
                    y, kd::FastDiv(static_cast<unsigned>(out >> 2)), n4);
        return kd::launch_status();
    }
    const unsigned grid = kd::grid_for((n + kThreads - 1) / kThreads, 8);
    (void)kd::launch(bias_add_kernel<T>, dim3(grid), kThreads, 0, x, b, y, out, n);
    return kd::launch_status();
}

// 32x32 tiles through shared memory: both the read and the write are coalesced.
template <typename T>
__global__ void __launch_bounds__(kThreads)
transpose_kernel(const T* __restrict__ x, T* __restrict__ y, int rows, int cols) {
    kd::pdl_prologue();
    __shared__ T tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
    const int tiles_c = (cols + 31) / 32, tiles_r = (rows + 31) / 32;
    for (int64_t t = blockIdx.x; t < static_cast<int64_t>(tiles_c) * tiles_r; t += gridDim.x) {
        const int tr = static_cast<int>(t / tiles_c), tc = static_cast<int>(t % tiles_c);
#pragma unroll
        for (int k = 0; k < 32; k += 8) {
            const int r = tr * 32 + ty + k, c = tc * 32 + tx;
            if (r < rows && c < cols) tile[ty + k][tx] = x[static_cast<int64_t>(r) * cols + c];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 32; k += 8) {
            const int c = tc * 32 + ty + k, r = tr * 32 + tx;
            if (r < rows && c < cols) y[static_cast<int64_t>(c) * rows + r] = tile[tx][ty + k];
        }
        __syncthreads();
    }
}

// 64x64 tiles, one packet (4 elements) per access on both sides: rows and cols multiples of 4, both pointers
// packet-aligned.  A thread reads 4 packets along the input rows and writes 4 packets along the output rows,
// gathering each output packet from one tile column (row stride 65 words: at most 2-way bank conflicts).
template <typename T>
__global__ void __launch_bounds__(kThreads)
transpose_packet_kernel(const T* __restrict__ x, T* __restrict__ y, int rows, int cols) {
    kd::pdl_prologue();
    __shared__ T tile[64][65];
    const int tiles_c = (cols + 63) / 64, tiles_r = (rows + 63) / 64;
    for (int64_t t = blockIdx.x; t < static_cast<int64_t>(tiles_c) * tiles_r; t += gridDim.x) {
        const int r0 = static_cast<int>(t / tiles_c) * 64, c0 = static_cast<int>(t % tiles_c) * 64;
        kd::Pack4<T> v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int idx = threadIdx.x + kThreads * k, r = r0 + (idx >> 4), c = c0 + 4 * (idx & 15);
            if (r < rows && c < cols) v[k] = kd::load4_stream(x + static_cast<int64_t>(r) * cols + c);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int idx = threadIdx.x + kThreads * k;
#pragma unroll
            for (int j = 0; j < 4; ++j) tile[idx >> 4][4 * (idx & 15) + j] = v[k].v[j];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int idx = threadIdx.x + kThreads * k, oc = idx >> 4, r4 = 4 * (idx & 15);
            const int c = c0 + oc, r = r0 + r4;
            if (c < cols && r < rows) {
                kd::Pack4<T> o;
#pragma unroll
                for (int j = 0; j < 4; ++j) o.v[j] = tile[r4 + j][oc];
                kd::store4(y + static_cast<int64_t>(c) * rows + r, o);
            }
        }
        __syncthreads();
    }
}

template <typename T>
int transpose2d(const T* x, T* y, int rows, int cols) {
    if (rows < 0 || cols < 0) return 1;
    if (rows == 0 || cols == 0) return 0;
    if (!x || !y) return 2;
    (void)cudaGetLastError();
    if (rows % 4 == 0 && cols % 4 == 0 && kd::aligned_pack<T>(x) && kd::aligned_pack<T>(y)) {
        const int64_t tiles = static_cast<int64_t>((cols + 63) / 64) * ((rows + 63) / 64);
        KD_LAUNCH_W(transpose_packet_kernel<T>, 8, tiles, kThreads, 0, x, y, rows, cols);
    } else {
        const int64_t tiles = static_cast<int64_t>((cols + 31) / 32) * ((rows + 31) / 32);
        (void)kd::launch(transpose_kernel<T>, dim3(kd::grid_for(tiles, 8)), kThreads, 0, x, y, rows, cols);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace

// C ABI: reference signatures (keydnn_cuda_ops.hpp:20-21,57-67; keydnn_tensor_arithmetic.hpp:130-159).
KD_API int keydnn_cuda_broadcast_to_f32(const float* x, float* y, const int64_t* in_shape, int in_ndim,
                                        const int64_t* out_shape, int out_ndim) {
    return broadcast_to<float>(x, y, in_shape, in_ndim, out_shape, out_ndim);
}
KD_API int keydnn_cuda_broadcast_to_f64(const double* x, double* y, const int64_t* in_shape, int in_ndim,
                                        const int64_t* out_shape, int out_ndim) {
    return broadcast_to<double>(x, y, in_shape, in_ndim, out_shape, out_ndim);
}
KD_API int keydnn_cuda_bias_add_f32(const float* x, const float* b, float* y, int64_t batch, int64_t out) {
    return bias_add<float>(x, b, y, batch, out);
}
KD_API int keydnn_cuda_bias_add_f64(const double* x, const double* b, double* y, int64_t batch, int64_t out) {
    return bias_add<double>(x, b, y, batch, out);
}
KD_API int keydnn_cuda_bias_add_inplace_f32(float* y, const float* b, int64_t batch, int64_t out) {
    return bias_add<float>(y, b, y, batch, out);
}
KD_API int keydnn_cuda_bias_add_inplace_f64(double* y, const double* b, int64_t batch, int64_t out) {
    return bias_add<double>(y, b, y, batch, out);
}
KD_API int keydnn_cuda_transpose2d_f32(const float* x, float* y, int rows, int cols) {
    return transpose2d<float>(x, y, rows, cols);
}
KD_API int keydnn_cuda_transpose2d_f64(const double* x, double* y, int rows, int cols) {
    return transpose2d<double>(x, y, rows, cols);
}
