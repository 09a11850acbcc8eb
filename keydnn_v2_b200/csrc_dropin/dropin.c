/*
 * libkeydnn_b200_dropin.so - the one file that takes the place of KeyDNNV2CudaNative.dll.
 *
 * KeyDNN opens a single native CUDA library (src/keydnn/infrastructure/native_cuda/python/_native_loader.py:79-150,
 * ctypes.CDLL on a fixed path) and resolves every keydnn_cuda_* symbol in it, by attribute
 * (reduce_ctypes.py:32-176) or by address (GetProcAddress, ops/tensor_arithmetic_ctypes.py:54-120).  Here the
 * symbols live in two libraries: libkeydnn_b200.so (the hand-written kernels and the runtime) and
 * libkeydnn_b200_dnn.so (matmul / conv2d, kept on cuBLAS / cuDNN).  This object depends on both, so a lookup
 * through its handle (dlsym searches the object and its dependencies) finds every export of either, and its
 * load-time constructor gives both libraries one stream state: the cuDNN / cuBLAS library asks the operator
 * library for the stream before every call.  Placed (or linked) at the path the reference loader hard-codes,
 * it makes the reference's own bindings run unchanged.
 */
#include <stdint.h>

extern int keydnn_cuda_get_stream(uint64_t* out);
extern int keydnn_dnn_bind_stream_source(uint64_t get_stream_fn);

__attribute__((constructor)) static void keydnn_b200_dropin_bind(void) {
    (void)keydnn_dnn_bind_stream_source((uint64_t)(uintptr_t)&keydnn_cuda_get_stream);
}

/* 1 = both libraries are loaded and share the operator library's stream. */
__attribute__((visibility("default"))) int keydnn_b200_dropin_version(void) { return 1; }
