// Cross-GPU plumbing for row-sharded workloads: one process per GPU, NCCL over
// NVLink / NVSwitch, every collective enqueued on the library stream right behind
// the kernel that produced its operand (no host synchronisation in between).
//
// Additive: the reference has no distributed code at all (cross-device copy_from
// is rejected, src/keydnn/infrastructure/tensor/mixins/memory/_base.py:970-975).
// NCCL is opened with dlopen at first use, so the library loads on machines
// without it and shares the copy a host framework has already loaded.
#include "common.cuh"

#include <dlfcn.h>
#include <cstring>
#include <nccl.h>

namespace {

struct Api {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
};

Api g_api;
ncclComm_t g_comm = nullptr;
int g_world = 1, g_rank = 0;

constexpr int kNotInit = -10, kNoLib = -11;
inline int nstat(ncclResult_t r) { return r == ncclSuccess ? 0 : 200000 + static_cast<int>(r); }

bool load_api() {
    if (g_api.handle) return true;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* n : names) {
        h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
    }
    if (!h) return false;
#define KD_SYM(field, sym)                                                 \
    g_api.field = reinterpret_cast<decltype(g_api.field)>(dlsym(h, sym));  \
    if (!g_api.field) return false;
    KD_SYM(GetUniqueId, "ncclGetUniqueId")
    KD_SYM(CommInitRank, "ncclCommInitRank")
    KD_SYM(CommDestroy, "ncclCommDestroy")
    KD_SYM(AllReduce, "ncclAllReduce")
    KD_SYM(AllGather, "ncclAllGather")
    KD_SYM(Broadcast, "ncclBroadcast")
#undef KD_SYM
    g_api.handle = h;
    return true;
}

// Picks, per column, the winner among `world` per-rank maxima (rank r's values start at
// vals + r*val_stride, its positions at idx + r*idx_stride, strides in elements): greater value wins,
// equal values keep the lower rank (= the smaller global row), and a column whose
// maximum is -inf keeps global position 0, the single-GPU rule.  `local_idx`
// receives the position inside this rank's shard, or -1 when another rank owns it.
template <typename T>
__global__ void argmax_select_kernel(const T* __restrict__ vals, const long long* __restrict__ idx, int world, int rank,
                                     long long span, int64_t n, int64_t val_stride, int64_t idx_stride,
                                     T* __restrict__ out_val,
                                     long long* __restrict__ out_global, long long* __restrict__ out_local) {
    kd::pdl_prologue();
    for (int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < n;
         c += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        T best = kd::neg_inf<T>();
        long long g = 0;
        int owner = 0;
        for (int r = 0; r < world; ++r) {
            const T v = vals[r * val_stride + c];
            if (v > best) { best = v; g = static_cast<long long>(r) * span + idx[r * idx_stride + c]; owner = r; }
        }
        out_val[c] = best;
        out_global[c] = g;
        out_local[c] = (owner == rank) ? g - static_cast<long long>(rank) * span : -1;
    }
}

template <typename T>
int argmax_select(const T* vals, const long long* idx, int world, int rank, long long span, int64_t n,
                  int64_t val_stride, int64_t idx_stride, T* out_val, long long* out_global, long long* out_local) {
    if (!vals || !idx || !out_val || !out_global || !out_local) return -1;
    if (world <= 0 || rank < 0 || rank >= world || n <= 0 || val_stride < n || idx_stride < n) return -2;
    (void)cudaGetLastError();
    const unsigned grid = kd::grid_for((n + 255) / 256, 8);
    (void)kd::launch(argmax_select_kernel<T>, dim3(grid), 256, 0, vals, idx, world, rank, span, n, val_stride, idx_stride, out_val,
                                                          out_global, out_local);
    return kd::launch_status();
}

// out[i] = (sum over ranks r = 0 .. world-1, in that order, of blocks[r * stride + i]) [* scale of the segment i
// lies in].  The sum of one element is formed in double and rounded once; up to kMaxSegments index ranges carry
// a scale (a mean's 1/count), applied as one multiplication in the element type.  With an all-gather in front
// this is an all-reduce whose result does not depend on the collective's internal order.
constexpr int kMaxSegments = 8;
template <typename T> struct Segments {
    int n;
    long long begin[kMaxSegments], end[kMaxSegments];
    T scale[kMaxSegments];
};

template <typename T>
__global__ void rank_sum_kernel(const T* __restrict__ blocks, int world, int64_t stride, int64_t n, T* __restrict__ out,
                                Segments<T> seg) {
    kd::pdl_prologue();
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        double s = 0.0;
        for (int r = 0; r < world; ++r) s += static_cast<double>(blocks[r * stride + i]);
        T v = static_cast<T>(s);
        for (int k = 0; k < seg.n; ++k)
            if (i >= seg.begin[k] && i < seg.end[k]) v = v * seg.scale[k];
        out[i] = v;
    }
}

template <typename T>
int rank_sum(const T* blocks, int world, int64_t stride, int64_t n, T* out, const int64_t* seg_begin, const int64_t* seg_end,
             const T* seg_scale, int nseg) {
    if (!blocks || !out) return -1;
    if (world <= 0 || n <= 0 || stride < n || nseg < 0 || nseg > kMaxSegments) return -2;
    if (nseg > 0 && (!seg_begin || !seg_end || !seg_scale)) return -1;
    Segments<T> seg;
    seg.n = nseg;
    for (int k = 0; k < nseg; ++k) {
        seg.begin[k] = seg_begin[k];
        seg.end[k] = seg_end[k];
        seg.scale[k] = seg_scale[k];
    }
    (void)cudaGetLastError();
    const unsigned grid = kd::grid_for((n + 255) / 256, 8);
    (void)kd::launch(rank_sum_kernel<T>, dim3(grid), 256, 0, blocks, world, stride, n, out, seg);
    return kd::launch_status();
}

}  // namespace

KD_API int keydnn_nccl_unique_id(void* out128) {
    if (!out128) return -1;
    if (!load_api()) return kNoLib;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
    return nstat(g_api.GetUniqueId(static_cast<ncclUniqueId*>(out128)));
}

KD_API int keydnn_nccl_init(const void* id128, int world, int rank) {
    if (!id128) return -1;
    if (world <= 0 || rank < 0 || rank >= world) return -2;
    if (!load_api()) return kNoLib;
    if (g_comm) { g_api.CommDestroy(g_comm); g_comm = nullptr; }
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclResult_t r = g_api.CommInitRank(&g_comm, world, id, rank);
    if (r != ncclSuccess) { g_comm = nullptr; return nstat(r); }
    g_world = world;
    g_rank = rank;
    return 0;
}

KD_API int keydnn_nccl_destroy() {
    if (g_comm && g_api.CommDestroy) {
        cudaStreamSynchronize(kd::stream());
        g_api.CommDestroy(g_comm);
    }
    g_comm = nullptr;
    g_world = 1;
    g_rank = 0;
    return 0;
}

KD_API int keydnn_nccl_world(int* world, int* rank) {
    if (world) *world = g_world;
    if (rank) *rank = g_rank;
    return g_comm ? 0 : kNotInit;
}

// In-place sum across ranks.
KD_API int keydnn_nccl_allreduce_sum_f32(float* buf, int64_t count) {
    if (!buf || count <= 0) return -1;
    if (!g_comm) return kNotInit;
    return nstat(g_api.AllReduce(buf, buf, static_cast<size_t>(count), ncclFloat32, ncclSum, g_comm, kd::stream()));
}
KD_API int keydnn_nccl_allreduce_sum_f64(double* buf, int64_t count) {
    if (!buf || count <= 0) return -1;
    if (!g_comm) return kNotInit;
    return nstat(g_api.AllReduce(buf, buf, static_cast<size_t>(count), ncclFloat64, ncclSum, g_comm, kd::stream()));
}
// recv holds world * nbytes; rank r's block lands at offset r * nbytes.
KD_API int keydnn_nccl_allgather(const void* send, void* recv, int64_t nbytes) {
    if (!send || !recv || nbytes <= 0) return -1;
    if (!g_comm) return kNotInit;
    return nstat(g_api.AllGather(send, recv, static_cast<size_t>(nbytes), ncclInt8, g_comm, kd::stream()));
}
KD_API int keydnn_nccl_broadcast(void* buf, int64_t nbytes, int root) {
    if (!buf || nbytes <= 0) return -1;
    if (!g_comm) return kNotInit;
    return nstat(g_api.Broadcast(buf, buf, static_cast<size_t>(nbytes), ncclInt8, root, g_comm, kd::stream()));
}

KD_API int keydnn_cuda_argmax_select_f32(const float* vals, const int64_t* idx, int world, int rank, int64_t span,
                                         int64_t n, int64_t val_stride, int64_t idx_stride, float* out_val,
                                         int64_t* out_global, int64_t* out_local) {
    return argmax_select<float>(vals, reinterpret_cast<const long long*>(idx), world, rank, span, n, val_stride,
                              idx_stride, out_val,
                                reinterpret_cast<long long*>(out_global), reinterpret_cast<long long*>(out_local));
}
KD_API int keydnn_cuda_argmax_select_f64(const double* vals, const int64_t* idx, int world, int rank, int64_t span,
                                         int64_t n, int64_t val_stride, int64_t idx_stride, double* out_val,
                                         int64_t* out_global, int64_t* out_local) {
    return argmax_select<double>(vals, reinterpret_cast<const long long*>(idx), world, rank, span, n, val_stride,
                              idx_stride, out_val,
                                 reinterpret_cast<long long*>(out_global), reinterpret_cast<long long*>(out_local));
}

// out[i] = sum over the `world` gathered blocks (rank order, double accumulation, one rounding) of element i,
// times seg_scale[k] where seg_begin[k] <= i < seg_end[k] (host arrays, nseg <= 8).  stride: elements between
// two ranks' blocks.  Behind keydnn_nccl_allgather it replaces an all-reduce.
KD_API int keydnn_cuda_rank_sum_f32(const float* blocks, int world, int64_t stride, int64_t n, float* out,
                                    const int64_t* seg_begin, const int64_t* seg_end, const float* seg_scale, int nseg) {
    return rank_sum<float>(blocks, world, stride, n, out, seg_begin, seg_end, seg_scale, nseg);
}
KD_API int keydnn_cuda_rank_sum_f64(const double* blocks, int world, int64_t stride, int64_t n, double* out,
                                    const int64_t* seg_begin, const int64_t* seg_end, const double* seg_scale, int nseg) {
    return rank_sum<double>(blocks, world, stride, n, out, seg_begin, seg_end, seg_scale, nseg);
}
