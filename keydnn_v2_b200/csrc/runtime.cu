// Device runtime behind the C ABI: device selection, the caching allocator,
// host<->device copies, the library stream, events and reduction scratch.
//
// Replaces the reference exports defined in
// native_cuda/.../KeyDNNV2CudaNative/keydnn_cuda_utils.cu:13-54 and
// keydnn_memcpy_d2d.cu:4-9 (raw cudaMalloc / cudaFree / cudaMemcpy wrappers).
//
// Differences that callers can observe only as speed:
//  * keydnn_cuda_malloc / keydnn_cuda_free go through a per-device caching pool.
//    Work of this library is ordered on the library stream, so a block handed
//    back by `free` can be handed out again at once: work that still reads it was
//    enqueued earlier on the same stream.  Every cached block remembers the
//    stream that was current when it was freed; when it is handed out while
//    another stream is current, that stream first waits (an event, on the device)
//    for the work enqueued on the old one.  cudaFree's implicit device
//    synchronisation disappears from the per-op path.
//  * copies are enqueued on the library stream and the host waits on that
//    stream only.
#include "common.cuh"

#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

constexpr int kMaxDevices = 16;
constexpr size_t kGranule = 512;             // allocation granularity (bytes)
constexpr size_t kSmallLimit = 1u << 20;     // below this, round up to a power of two

struct DevicePool {
    std::multimap<size_t, void*> free_blocks;          // size -> block
    std::unordered_map<void*, size_t> live;            // block -> rounded size
    std::map<uintptr_t, size_t> requested;             // live block -> bytes the caller asked for (bounds of copies)
    size_t bytes_reserved = 0;                         // total held from the driver
    size_t bytes_in_use = 0;
    size_t n_driver_mallocs = 0;
    size_t n_requests = 0;
    // Stream capture: blocks handed out while a graph is being recorded belong to that graph.
    // They may be recycled among the tensors of the recording (the graph keeps their order),
    // but never leave it: a replay writes to these addresses whoever holds them.
    bool capturing = false;
    std::multimap<size_t, void*> capture_free;         // freed during the recording, reusable inside it
    std::unordered_map<void*, size_t> graph_blocks;    // every block owned by a recorded graph
    int live_graphs = 0;                               // recorded graphs not yet destroyed
    std::unordered_map<void*, cudaStream_t> freed_on;  // cached block -> stream that was current at its free
    cudaEvent_t handover = nullptr;                    // orders a block's old stream before its new one
};

struct DeviceState {
    bool inited = false;
    int sm_count = 0;
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    unsigned int* counters = nullptr;
    size_t counters_len = 0;
    size_t scratch_allocs = 0;     // driver allocations made for scratch / counters
    std::vector<void*> parked;     // outgrown scratch / counter buffers a recorded graph may still write to
    cudaStream_t stream = nullptr; // the library stream of this device: legacy default stream unless the caller sets one
    DevicePool pool;
};

std::mutex g_mu;
DeviceState g_dev[kMaxDevices];
bool g_pool_enabled = true;
size_t g_scratch_min = size_t(8) << 20;   // first size of the reduction scratch (KEYDNN_B200_SCRATCH_MIN, bytes)

int current_device() {
    int d = 0;
    cudaGetDevice(&d);
    return (d >= 0 && d < kMaxDevices) ? d : 0;
}

DeviceState& state() {
    DeviceState& s = g_dev[current_device()];
    if (!s.inited) {
        int d = current_device();
        cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, d);
        if (s.sm_count <= 0) s.sm_count = 148;
        const char* e = std::getenv("KEYDNN_B200_NO_POOL");
        if (e && e[0] == '1') g_pool_enabled = false;
        if (const char* m = std::getenv("KEYDNN_B200_SCRATCH_MIN")) {
            const long long v = std::atoll(m);
            if (v >= 256) g_scratch_min = static_cast<size_t>(v);
        }
        s.inited = true;
    }
    return s;
}

size_t round_size(size_t n) {
    if (n == 0) n = 1;
    if (n < kSmallLimit) {
        size_t p = kGranule;
        while (p < n) p <<= 1;
        return p;
    }
    // large blocks: 2 MiB granularity keeps reuse likely without doubling.
    const size_t big = size_t(2) << 20;
    return (n + big - 1) / big * big;
}

void release_cached(DevicePool& p) {
    for (auto& kv : p.free_blocks) {
        cudaFree(kv.second);
        p.bytes_reserved -= kv.first;
    }
    p.free_blocks.clear();
    p.freed_on.clear();
}

// Copies and memsets are checked against the size the caller asked for, not the rounded block: cudaMemcpy
// rejects a device range that leaves its allocation (cudaErrorInvalidValue), and the reference's wrappers rely on
// that to catch buffers that are too small (ops/matmul_cuda.py probes the last byte of every operand).  With
// size classes the driver would let such a copy through; this keeps the answer the caller would have got from
// a plain cudaMalloc.  Pointers that are not inside a live pool block are left to the driver.
bool range_ok(const void* p, size_t n) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    std::lock_guard<std::mutex> lk(g_mu);
    const auto& req = g_dev[current_device()].pool.requested;
    auto it = req.upper_bound(a);
    if (it == req.begin()) return true;
    --it;
    const auto& live = g_dev[current_device()].pool.live;
    auto lt = live.find(reinterpret_cast<void*>(it->first));
    if (lt == live.end() || a >= it->first + lt->second) return true;      // beyond the block: not ours to judge
    return a + n <= it->first + it->second;
}

// The library stream of the current device (the fast path of every launch: no lock, one TLS read).
inline cudaStream_t& dev_stream() { return g_dev[current_device()].stream; }

// A cached block leaves the pool: if it was freed while another stream was current, work enqueued on that
// stream may still touch it, so the current stream waits for it on the device.  Not while a graph is being
// recorded (the recording's blocks are recycled inside it, in the recorded order).
void hand_over(DevicePool& p, void* q, cudaStream_t now) {
    auto it = p.freed_on.find(q);
    if (it == p.freed_on.end()) return;
    const cudaStream_t then = it->second;
    p.freed_on.erase(it);
    if (then == now || p.capturing) return;
    if (!p.handover && cudaEventCreateWithFlags(&p.handover, cudaEventDisableTiming) != cudaSuccess) {
        p.handover = nullptr;
        (void)cudaGetLastError();
        cudaStreamSynchronize(then);
        return;
    }
    if (cudaEventRecord(p.handover, then) != cudaSuccess || cudaStreamWaitEvent(now, p.handover, 0) != cudaSuccess) {
        (void)cudaGetLastError();
        cudaStreamSynchronize(then);
    }
}

// Outgrown scratch buffers: freed at once unless a recorded graph (or a recording in progress) holds their address.
void retire(DeviceState& s, void* old) {
    if (!old) return;
    if (s.pool.live_graphs > 0 || s.pool.capturing) s.parked.push_back(old);
    else cudaFree(old);     // synchronises with earlier kernels that still use it
}

}  // namespace

namespace kd {

cudaStream_t stream() { return dev_stream(); }

bool pdl_enabled() {
    static const bool on = [] {
        const char* e = std::getenv("KEYDNN_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

int sm_count() {
    std::lock_guard<std::mutex> lk(g_mu);
    return state().sm_count;
}

// Growth rules (both buffers):
//  * while a graph is being recorded nothing may be allocated: a reduction whose shape needs more than the
//    buffer holds fails (nullptr -> cudaErrorMemoryAllocation from the entry point); run the step eagerly
//    once before recording it, as keydnn_cuda_graph_capture_begin asks.
//  * while a recorded graph is alive its launches hold the old address: the outgrown buffer is parked until
//    keydnn_cuda_graph_destroy instead of being freed, so a later, larger eager reduction cannot pull the
//    memory from under a replay.
void* scratch(size_t nbytes) {
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& s = state();
    if (nbytes > s.scratch_bytes) {
        if (s.pool.capturing) return nullptr;
        size_t want = nbytes < g_scratch_min ? g_scratch_min : nbytes;
        void* fresh = nullptr;
        if (cudaMalloc(&fresh, want) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        retire(s, s.scratch);
        s.scratch_allocs++;
        s.scratch = fresh;
        s.scratch_bytes = want;
    }
    return s.scratch;
}

unsigned int* counters(size_t count) {
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& s = state();
    if (count > s.counters_len) {
        if (s.pool.capturing) return nullptr;
        size_t want = count < 4096 ? 4096 : count;
        void* fresh = nullptr;
        if (cudaMalloc(&fresh, want * sizeof(unsigned int)) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        cudaMemset(fresh, 0, want * sizeof(unsigned int));
        retire(s, s.counters);
        s.scratch_allocs++;
        s.counters = static_cast<unsigned int*>(fresh);
        s.counters_len = want;
    }
    return s.counters;
}

}  // namespace kd

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------

KD_API int keydnn_cuda_set_device(int device) {
    return kd::status(cudaSetDevice(device));
}

KD_API int keydnn_cuda_malloc(std::uint64_t* out_ptr, std::size_t nbytes) {
    if (!out_ptr) return -1;
    *out_ptr = 0;
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& s = state();
    DevicePool& p = s.pool;
    p.n_requests++;
    if (!g_pool_enabled) {
        void* q = nullptr;
        cudaError_t st = cudaMalloc(&q, nbytes);
        if (st != cudaSuccess) return static_cast<int>(st);
        *out_ptr = reinterpret_cast<std::uint64_t>(q);
        return 0;
    }
    const size_t want = round_size(nbytes);
    if (p.capturing) {
        auto ct = p.capture_free.lower_bound(want);
        if (ct != p.capture_free.end() && ct->first <= want + want / 2 + kGranule) {
            void* q = ct->second;
            size_t sz = ct->first;
            p.capture_free.erase(ct);
            p.live.emplace(q, sz);
            p.requested[reinterpret_cast<uintptr_t>(q)] = nbytes;
            p.bytes_in_use += sz;
            *out_ptr = reinterpret_cast<std::uint64_t>(q);
            return 0;
        }
    }
    auto it = p.free_blocks.lower_bound(want);
    // Accept a cached block only if it wastes less than half of itself.
    if (it != p.free_blocks.end() && it->first <= want + want / 2 + kGranule) {
        void* q = it->second;
        size_t sz = it->first;
        p.free_blocks.erase(it);
        hand_over(p, q, s.stream);
        p.live.emplace(q, sz);
        p.requested[reinterpret_cast<uintptr_t>(q)] = nbytes;
        p.bytes_in_use += sz;
        if (p.capturing) p.graph_blocks.emplace(q, sz);
        *out_ptr = reinterpret_cast<std::uint64_t>(q);
        return 0;
    }
    void* q = nullptr;
    cudaError_t st = cudaMalloc(&q, want);
    if (st != cudaSuccess) {
        // Give cached memory back to the driver and try once more.
        (void)cudaGetLastError();
        release_cached(p);
        st = cudaMalloc(&q, want);
        if (st != cudaSuccess) {
            (void)cudaGetLastError();
            return static_cast<int>(st);
        }
    }
    p.n_driver_mallocs++;
    p.bytes_reserved += want;
    p.bytes_in_use += want;
    p.live.emplace(q, want);
    p.requested[reinterpret_cast<uintptr_t>(q)] = nbytes;
    if (p.capturing) p.graph_blocks.emplace(q, want);
    *out_ptr = reinterpret_cast<std::uint64_t>(q);
    return 0;
}

KD_API int keydnn_cuda_free(std::uint64_t ptr) {
    if (ptr == 0) return 0;
    void* q = reinterpret_cast<void*>(ptr);
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& s = state();
    DevicePool& p = s.pool;
    auto it = p.live.find(q);
    if (it == p.live.end()) {
        // Not one of ours (pool disabled, or allocated on another device).
        for (int d = 0; d < kMaxDevices; ++d) {
            auto jt = g_dev[d].pool.live.find(q);
            if (jt != g_dev[d].pool.live.end()) {
                size_t sz = jt->second;
                g_dev[d].pool.live.erase(jt);
                g_dev[d].pool.requested.erase(reinterpret_cast<uintptr_t>(q));
                g_dev[d].pool.bytes_in_use -= sz;
                g_dev[d].pool.free_blocks.emplace(sz, q);
                g_dev[d].pool.freed_on[q] = g_dev[d].stream;
                return 0;
            }
        }
        return kd::status(cudaFree(q));
    }
    size_t sz = it->second;
    p.live.erase(it);
    p.requested.erase(reinterpret_cast<uintptr_t>(q));
    p.bytes_in_use -= sz;
    if (p.graph_blocks.count(q)) {
        // owned by a recorded graph: reusable only inside the recording, never by anybody else
        if (p.capturing) p.capture_free.emplace(sz, q);
        return 0;
    }
    p.free_blocks.emplace(sz, q);
    p.freed_on[q] = s.stream;
    return 0;
}

// Additive: hand every cached block back to the driver.
KD_API int keydnn_cuda_empty_cache() {
    cudaError_t st = cudaDeviceSynchronize();       // blocks may have been freed under any stream
    std::lock_guard<std::mutex> lk(g_mu);
    release_cached(state().pool);
    return kd::status(st);
}

// Additive: out[0]=bytes reserved from the driver, out[1]=bytes handed out,
// out[2]=driver allocations made, out[3]=allocation requests served.
KD_API int keydnn_cuda_pool_stats(std::uint64_t* out4) {
    if (!out4) return -1;
    std::lock_guard<std::mutex> lk(g_mu);
    DevicePool& p = state().pool;
    out4[0] = p.bytes_reserved;
    out4[1] = p.bytes_in_use;
    out4[2] = p.n_driver_mallocs;
    out4[3] = p.n_requests;
    return 0;
}

// Additive: the reduction scratch of the current device.  out[0] = bytes of the partials buffer, out[1] =
// completion-ticket slots, out[2] = driver allocations made for either so far, out[3] = outgrown buffers
// parked for a recorded graph.
KD_API int keydnn_cuda_scratch_stats(std::uint64_t* out4) {
    if (!out4) return -1;
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& s = state();
    out4[0] = s.scratch_bytes;
    out4[1] = s.counters_len;
    out4[2] = s.scratch_allocs;
    out4[3] = s.parked.size();
    return 0;
}

// Additive: free and total bytes of the current device as the driver sees them (cudaMemGetInfo).
KD_API int keydnn_cuda_mem_info(std::uint64_t* out2) {
    if (!out2) return -1;
    size_t f = 0, t = 0;
    cudaError_t st = cudaMemGetInfo(&f, &t);
    out2[0] = f;
    out2[1] = t;
    return kd::status(st);
}

KD_API int keydnn_cuda_memcpy_h2d(std::uint64_t dst_dev, const void* src_host, std::size_t nbytes) {
    if (nbytes == 0) return 0;
    if (!range_ok(reinterpret_cast<const void*>(dst_dev), nbytes)) return static_cast<int>(cudaErrorInvalidValue);
    cudaError_t st = cudaMemcpyAsync(reinterpret_cast<void*>(dst_dev), src_host, nbytes,
                                     cudaMemcpyHostToDevice, dev_stream());
    if (st != cudaSuccess) return static_cast<int>(st);
    // Pageable sources are staged before the call returns; pinned sources are
    // read by the DMA engine, so wait for it: the caller may reuse the buffer.
    return kd::status(cudaStreamSynchronize(dev_stream()));
}

KD_API int keydnn_cuda_memcpy_d2h(void* dst_host, std::uint64_t src_dev, std::size_t nbytes) {
    if (nbytes == 0) return 0;
    if (!range_ok(reinterpret_cast<const void*>(src_dev), nbytes)) return static_cast<int>(cudaErrorInvalidValue);
    cudaError_t st = cudaMemcpyAsync(dst_host, reinterpret_cast<const void*>(src_dev), nbytes,
                                     cudaMemcpyDeviceToHost, dev_stream());
    if (st != cudaSuccess) return static_cast<int>(st);
    return kd::status(cudaStreamSynchronize(dev_stream()));
}

// Additive: host->device copy that returns as soon as it is enqueued (the
// source must stay valid and, to overlap, be pinned).
KD_API int keydnn_cuda_memcpy_h2d_async(std::uint64_t dst_dev, const void* src_host, std::size_t nbytes) {
    if (nbytes == 0) return 0;
    if (!range_ok(reinterpret_cast<const void*>(dst_dev), nbytes)) return static_cast<int>(cudaErrorInvalidValue);
    return kd::status(cudaMemcpyAsync(reinterpret_cast<void*>(dst_dev), src_host, nbytes,
                                      cudaMemcpyHostToDevice, dev_stream()));
}

// Additive: device->host copy that returns as soon as it is enqueued; the destination (pinned, to be
// asynchronous) may be read after an event recorded behind the copy has completed.
KD_API int keydnn_cuda_memcpy_d2h_async(void* dst_host, std::uint64_t src_dev, std::size_t nbytes) {
    if (nbytes == 0) return 0;
    if (!range_ok(reinterpret_cast<const void*>(src_dev), nbytes)) return static_cast<int>(cudaErrorInvalidValue);
    return kd::status(cudaMemcpyAsync(dst_host, reinterpret_cast<const void*>(src_dev), nbytes,
                                      cudaMemcpyDeviceToHost, dev_stream()));
}

KD_API int keydnn_cuda_memcpy_d2d(void* dst, const void* src, std::size_t nbytes) {
    if (nbytes == 0) return 0;
    if (!dst || !src) return 1;
    if (!range_ok(dst, nbytes) || !range_ok(src, nbytes)) return 2;
    cudaError_t st = cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToDevice, dev_stream());
    return st == cudaSuccess ? 0 : 2;
}

KD_API int keydnn_cuda_memset(std::uint64_t dev_ptr, int value, std::size_t nbytes) {
    if (nbytes == 0) return 0;
    if (!range_ok(reinterpret_cast<const void*>(dev_ptr), nbytes)) return static_cast<int>(cudaErrorInvalidValue);
    return kd::status(cudaMemsetAsync(reinterpret_cast<void*>(dev_ptr), value, nbytes, dev_stream()));
}

KD_API int keydnn_cuda_synchronize() {
    return kd::status(cudaDeviceSynchronize());
}

// Additive: pinned host buffers for the end-to-end path.
KD_API int keydnn_cuda_host_alloc(void** out, std::size_t nbytes) {
    if (!out) return -1;
    *out = nullptr;
    return kd::status(cudaMallocHost(out, nbytes ? nbytes : 1));
}
KD_API int keydnn_cuda_host_free(void* p) {
    if (!p) return 0;
    return kd::status(cudaFreeHost(p));
}

// Additive: the stream all work of this library is enqueued on.
// The stream belongs to the current device (keydnn_cuda_set_device): each device keeps its own.
KD_API int keydnn_cuda_get_stream(std::uint64_t* out) {
    if (!out) return -1;
    *out = reinterpret_cast<std::uint64_t>(dev_stream());
    return 0;
}
KD_API int keydnn_cuda_set_stream(std::uint64_t s) {
    dev_stream() = reinterpret_cast<cudaStream_t>(s);
    return 0;
}
KD_API int keydnn_cuda_stream_create(std::uint64_t* out) {
    if (!out) return -1;
    cudaStream_t s = nullptr;
    cudaError_t st = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    *out = reinterpret_cast<std::uint64_t>(s);
    return kd::status(st);
}
KD_API int keydnn_cuda_stream_destroy(std::uint64_t s) {
    if (!s) return 0;
    const cudaStream_t dead = reinterpret_cast<cudaStream_t>(s);
    {
        std::lock_guard<std::mutex> lk(g_mu);
        bool synced = false;
        for (int d = 0; d < kMaxDevices; ++d) {
            if (g_dev[d].stream == dead) g_dev[d].stream = nullptr;
            // cached blocks freed under this stream: let its work finish now, the handle is about to go
            auto& tags = g_dev[d].pool.freed_on;
            for (auto it = tags.begin(); it != tags.end();) {
                if (it->second != dead) { ++it; continue; }
                if (!synced) { cudaStreamSynchronize(dead); synced = true; }
                it = tags.erase(it);
            }
        }
    }
    return kd::status(cudaStreamDestroy(dead));
}
KD_API int keydnn_cuda_stream_synchronize() {
    return kd::status(cudaStreamSynchronize(dev_stream()));
}

// Additive: CUDA events on the library stream.  These are the names the
// reference's backward profiler probes for (tensor/_tensor.py:1619-1629) and
// never finds in its own DLL.
KD_API int keydnn_cuda_event_create(std::uint64_t* out) {
    if (!out) return -1;
    cudaEvent_t e = nullptr;
    cudaError_t st = cudaEventCreate(&e);
    *out = reinterpret_cast<std::uint64_t>(e);
    return kd::status(st);
}
KD_API int keydnn_cuda_event_record(std::uint64_t ev) {
    return kd::status(cudaEventRecord(reinterpret_cast<cudaEvent_t>(ev), dev_stream()));
}
// Work enqueued on the library stream after this call starts only once `ev` has completed.
KD_API int keydnn_cuda_stream_wait_event(std::uint64_t ev) {
    return kd::status(cudaStreamWaitEvent(dev_stream(), reinterpret_cast<cudaEvent_t>(ev), 0));
}
KD_API int keydnn_cuda_event_synchronize(std::uint64_t ev) {
    return kd::status(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(ev)));
}
KD_API int keydnn_cuda_event_elapsed_ms(std::uint64_t start, std::uint64_t stop, float* out_ms) {
    if (!out_ms) return -1;
    return kd::status(cudaEventElapsedTime(out_ms, reinterpret_cast<cudaEvent_t>(start),
                                           reinterpret_cast<cudaEvent_t>(stop)));
}
KD_API int keydnn_cuda_event_destroy(std::uint64_t ev) {
    if (!ev) return 0;
    return kd::status(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(ev)));
}

// Additive: record everything enqueued on the library stream between begin and end into a CUDA
// graph and replay it with one launch.  The library stream must be a created stream (not the
// legacy default stream); run the work eagerly on that stream a few times first so that plans,
// scratch and the allocator are warm: the recording itself must not need cudaMalloc.  Device
// blocks allocated during the recording stay reserved for the graph until graph_destroy.
// One recording at a time, one graph alive per device.
KD_API int keydnn_cuda_graph_capture_begin() {
    if (!dev_stream()) return -3;                       // the legacy default stream cannot be captured
    {
        std::lock_guard<std::mutex> lk(g_mu);
        DevicePool& p = state().pool;
        if (p.capturing || !p.graph_blocks.empty()) return -4;
        p.capturing = true;
    }
    cudaError_t st = cudaStreamBeginCapture(dev_stream(), cudaStreamCaptureModeRelaxed);
    if (st != cudaSuccess) {
        std::lock_guard<std::mutex> lk(g_mu);
        state().pool.capturing = false;
    }
    return kd::status(st);
}

KD_API int keydnn_cuda_graph_capture_end(std::uint64_t* out_exec) {
    if (!out_exec) return -1;
    *out_exec = 0;
    cudaGraph_t graph = nullptr;
    cudaError_t st = cudaStreamEndCapture(dev_stream(), &graph);
    {
        std::lock_guard<std::mutex> lk(g_mu);
        DevicePool& p = state().pool;
        p.capturing = false;
        p.capture_free.clear();                      // those blocks stay in graph_blocks
        if (st != cudaSuccess || !graph) {           // failed recording: give its blocks back
            for (auto& kv : p.graph_blocks)
                if (!p.live.count(kv.first)) p.free_blocks.emplace(kv.second, kv.first);
            p.graph_blocks.clear();
        }
    }
    if (st != cudaSuccess) { (void)cudaGetLastError(); return kd::status(st); }
    cudaGraphExec_t exec = nullptr;
    st = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (st != cudaSuccess) return kd::status(st);
    {
        std::lock_guard<std::mutex> lk(g_mu);
        state().pool.live_graphs++;
    }
    *out_exec = reinterpret_cast<std::uint64_t>(exec);
    return 0;
}

KD_API int keydnn_cuda_graph_launch(std::uint64_t exec) {
    if (!exec) return -1;
    return kd::status(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(exec), dev_stream()));
}

KD_API int keydnn_cuda_graph_destroy(std::uint64_t exec) {
    cudaError_t st = cudaSuccess;
    if (exec) {
        cudaStreamSynchronize(dev_stream());
        st = cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(exec));
    }
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState& ds = state();
    DevicePool& p = ds.pool;
    for (auto& kv : p.graph_blocks)
        if (!p.live.count(kv.first)) p.free_blocks.emplace(kv.second, kv.first);   // live ones return on their free
    p.graph_blocks.clear();
    if (exec && p.live_graphs > 0) p.live_graphs--;
    if (p.live_graphs == 0) {
        for (void* q : ds.parked) cudaFree(q);      // outgrown scratch the graph could still have written to
        ds.parked.clear();
    }
    return kd::status(st);
}

// Additive: device facts for the harness.
KD_API int keydnn_cuda_device_count(int* out) {
    if (!out) return -1;
    return kd::status(cudaGetDeviceCount(out));
}
KD_API int keydnn_cuda_sm_count(int* out) {
    if (!out) return -1;
    *out = kd::sm_count();
    return 0;
}
KD_API const char* keydnn_cuda_error_string(int code) {
    if (code <= 0) return code == 0 ? "ok" : "argument guard";
    return cudaGetErrorString(static_cast<cudaError_t>(code));
}
KD_API int keydnn_b200_abi_version() { return 1; }
