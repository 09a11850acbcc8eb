/*
 * CPU restatement of the reference's pooling arithmetic.  TEST INFRASTRUCTURE
 * ONLY: it is the checker for the CUDA kernels (tests/, the smoke check and the
 * CPU-baseline leg of the benchmark); nothing in the product path calls it.
 *
 * Each function restates, step by step, the call sequence the reference runs for
 * one op on its CUDA path (src/keydnn/infrastructure/ops/pool2d_cuda_ext.py):
 *   maxpool forward : pad with -inf (:94-122)  -> window scan (:133-151)
 *   maxpool backward: zero padded grad (:221-223) -> scatter-add (:255-268) -> crop (:270-284)
 *   avgpool forward : pad with 0 -> window sum / (kh*kw)
 *   avgpool backward: zero padded grad -> gather of go/(kh*kw) -> crop
 *   global avgpool  : serial row sum / (H*W); backward go * (1/(H*W))
 * with the per-element arithmetic of the kernels those steps launch:
 *   NC/kernel.cu:97-185, NC/keydnn_avgpool2d_cuda.cu:55-92,143-198,
 *   NC/keydnn_global_avgpool2d_cuda.cu:32-97, NC/keydnn_pad2d_cuda.cu:30-97
 *   (NC/ = src/keydnn/infrastructure/native_cuda/keydnn_v2_cuda_native/KeyDNNV2CudaNative/),
 * and the CPU kernels native/src/keydnn_maxpool2d.cpp:18-123,
 * native/src/keydnn_avgpool2d.cpp:18-103, which share that arithmetic.
 * The padded planes are materialised exactly as the reference does.
 *
 * Where the reference sums with atomics in arbitrary order (maxpool backward
 * with overlapping windows) this file adds in ascending output order.
 *
 * Build: gcc -O2 -fPIC -shared -ffp-contract=off pool_oracle.c -o libkeydnn_oracle.so
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define DEFINE_POOL(T, SUF)                                                                                          \
    static T* pad_plane_##SUF(const T* x, int H, int W, int ph, int pw, T value) {                                   \
        const int Hp = H + 2 * ph, Wp = W + 2 * pw;                                                                  \
        T* p = (T*)malloc(sizeof(T) * (size_t)Hp * Wp);                                                              \
        for (int h = 0; h < Hp; ++h)                                                                                 \
            for (int w = 0; w < Wp; ++w) {                                                                           \
                const int hi = h - ph, wi = w - pw;                                                                  \
                p[(size_t)h * Wp + w] = (hi >= 0 && hi < H && wi >= 0 && wi < W) ? x[(size_t)hi * W + wi] : value;   \
            }                                                                                                        \
        return p;                                                                                                    \
    }                                                                                                                \
                                                                                                                     \
    int oracle_maxpool2d_forward_##SUF(const T* x, T* y, int64_t* idx, int N, int C, int H, int W, int Ho, int Wo,   \
                                       int kh, int kw, int sh, int sw, int ph, int pw) {                             \
        const int Hp = H + 2 * ph, Wp = W + 2 * pw;                                                                  \
        for (int64_t nc = 0; nc < (int64_t)N * C; ++nc) {                                                            \
            T* xp = pad_plane_##SUF(x + nc * H * W, H, W, ph, pw, (T)(-INFINITY));                                   \
            for (int i = 0; i < Ho; ++i)                                                                             \
                for (int j = 0; j < Wo; ++j) {                                                                       \
                    const int h0 = i * sh, w0 = j * sw;                                                              \
                    T best = (T)(-INFINITY);                                                                         \
                    int bh = h0, bw = w0;                                                                            \
                    for (int a = 0; a < kh; ++a)                                                                     \
                        for (int b = 0; b < kw; ++b) {                                                               \
                            const int h = h0 + a, w = w0 + b;                                                        \
                            if (h >= Hp || w >= Wp) continue;                                                        \
                            const T v = xp[(size_t)h * Wp + w];                                                      \
                            if (v > best) { best = v; bh = h; bw = w; }                                              \
                        }                                                                                            \
                    y[(nc * Ho + i) * Wo + j] = best;                                                                \
                    idx[(nc * Ho + i) * Wo + j] = (int64_t)bh * Wp + bw;                                             \
                }                                                                                                    \
            free(xp);                                                                                                \
        }                                                                                                            \
        return 0;                                                                                                    \
    }                                                                                                                \
                                                                                                                     \
    int oracle_maxpool2d_backward_##SUF(const T* go, const int64_t* idx, T* gx, int N, int C, int H, int W, int Ho,  \
                                        int Wo, int ph, int pw) {                                                    \
        const int Hp = H + 2 * ph, Wp = W + 2 * pw;                                                                  \
        T* gp = (T*)malloc(sizeof(T) * (size_t)Hp * Wp);                                                             \
        for (int64_t nc = 0; nc < (int64_t)N * C; ++nc) {                                                            \
            memset(gp, 0, sizeof(T) * (size_t)Hp * Wp);                                                              \
            for (int i = 0; i < Ho; ++i)                                                                             \
                for (int j = 0; j < Wo; ++j) {                                                                       \
                    const int64_t p = idx[(nc * Ho + i) * Wo + j];                                                   \
                    const int h = (int)(p / Wp), w = (int)(p % Wp);                                                  \
                    if (h < 0 || h >= Hp || w < 0 || w >= Wp) continue;                                              \
                    gp[(size_t)h * Wp + w] += go[(nc * Ho + i) * Wo + j];                                            \
                }                                                                                                    \
            for (int h = 0; h < H; ++h)                                                                              \
                for (int w = 0; w < W; ++w) gx[(nc * H + h) * W + w] = gp[(size_t)(h + ph) * Wp + (w + pw)];         \
        }                                                                                                            \
        free(gp);                                                                                                    \
        return 0;                                                                                                    \
    }                                                                                                                \
                                                                                                                     \
    int oracle_avgpool2d_forward_##SUF(const T* x, T* y, int N, int C, int H, int W, int Ho, int Wo, int kh, int kw, \
                                       int sh, int sw, int ph, int pw) {                                             \
        const int Hp = H + 2 * ph, Wp = W + 2 * pw;                                                                  \
        const T denom = (T)(kh * kw);                                                                                \
        for (int64_t nc = 0; nc < (int64_t)N * C; ++nc) {                                                            \
            T* xp = pad_plane_##SUF(x + nc * H * W, H, W, ph, pw, (T)0);                                             \
            for (int i = 0; i < Ho; ++i)                                                                             \
                for (int j = 0; j < Wo; ++j) {                                                                       \
                    T sum = (T)0;                                                                                    \
                    for (int a = 0; a < kh; ++a)                                                                     \
                        for (int b = 0; b < kw; ++b) {                                                               \
                            const int h = i * sh + a, w = j * sw + b;                                                \
                            if (h >= Hp || w >= Wp) continue;                                                        \
                            sum += xp[(size_t)h * Wp + w];                                                           \
                        }                                                                                            \
                    y[(nc * Ho + i) * Wo + j] = sum / denom;                                                         \
                }                                                                                                    \
            free(xp);                                                                                                \
        }                                                                                                            \
        return 0;                                                                                                    \
    }                                                                                                                \
                                                                                                                     \
    int oracle_avgpool2d_backward_##SUF(const T* go, T* gx, int N, int C, int H, int W, int Ho, int Wo, int kh,      \
                                        int kw, int sh, int sw, int ph, int pw) {                                    \
        const int Hp = H + 2 * ph, Wp = W + 2 * pw;                                                                  \
        const T denom = (T)(kh * kw);                                                                                \
        T* gp = (T*)malloc(sizeof(T) * (size_t)Hp * Wp);                                                             \
        for (int64_t nc = 0; nc < (int64_t)N * C; ++nc) {                                                            \
            memset(gp, 0, sizeof(T) * (size_t)Hp * Wp);                                                              \
            for (int h = 0; h < Hp; ++h)                                                                             \
                for (int w = 0; w < Wp; ++w) {                                                                       \
                    T acc = (T)0;                                                                                    \
                    for (int i = 0; i < Ho; ++i) {                                                                   \
                        if (h < i * sh || h >= i * sh + kh) continue;                                                \
                        for (int j = 0; j < Wo; ++j) {                                                               \
                            if (w < j * sw || w >= j * sw + kw) continue;                                            \
                            acc += go[(nc * Ho + i) * Wo + j] / denom;                                               \
                        }                                                                                            \
                    }                                                                                                \
                    gp[(size_t)h * Wp + w] += acc;                                                                   \
                }                                                                                                    \
            for (int h = 0; h < H; ++h)                                                                              \
                for (int w = 0; w < W; ++w) gx[(nc * H + h) * W + w] = gp[(size_t)(h + ph) * Wp + (w + pw)];         \
        }                                                                                                            \
        free(gp);                                                                                                    \
        return 0;                                                                                                    \
    }                                                                                                                \
                                                                                                                     \
    int oracle_global_avgpool2d_forward_##SUF(const T* x, T* y, int N, int C, int H, int W) {                        \
        const int HW = H * W;                                                                                        \
        for (int64_t nc = 0; nc < (int64_t)N * C; ++nc) {                                                            \
            T sum = (T)0;                                                                                            \
            for (int k = 0; k < HW; ++k) sum += x[nc * HW + k];                                                      \
            y[nc] = sum / (T)HW;                                                                                     \
        }                                                                                                            \
        return 0;                                                                                                    \
    }                                                                                                                \
                                                                                                                     \
    int oracle_global_avgpool2d_backward_##SUF(const T* go, T* gx, int N, int C, int H, int W) {                     \
        const int HW = H * W;                                                                                        \
        const T scale = (T)1 / (T)HW;                                                                                \
        for (int64_t nc = 0; nc < (int64_t)N * C; ++nc)                                                              \
            for (int k = 0; k < HW; ++k) gx[nc * HW + k] = go[nc] * scale;                                           \
        return 0;                                                                                                    \
    }

DEFINE_POOL(float, f32)
DEFINE_POOL(double, f64)
