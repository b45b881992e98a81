// Status codes and the thread-local error message behind mlk_last_error().
#pragma once

#include <cuda_runtime.h>

namespace mlk {

// Weight/activation type tags (also the dtype codes of the C ABI); used as template arguments.
constexpr int kBF16 = 0;  // bf16 weights, bf16 activations
constexpr int kFP16 = 1;  // fp16 weights, fp16 activations
constexpr int kE4M3 = 2;  // e4m3 weights decoded to bf16 in registers, bf16 activations

enum Status : int {
    kOk = 0,
    kInvalidArg = 1,    // a precondition of the reference API is violated (shape, divisibility, null)
    kUnsupported = 2,   // valid request that no kernel of this build implements
    kCudaError = 3,     // a CUDA runtime call failed (message holds cudaGetErrorString)
    kIoError = 4,       // dispatch table file could not be read / parsed
};

// printf-style; returns `code` so call sites can `return fail(kInvalidArg, "...", ...)`.
int fail(int code, const char* fmt, ...);
const char* last_error();
void clear_error();

// Library-wide options (mlk_set_option).
enum Option : int {
    kOptPdl = 0,            // launch kernels with programmatic stream serialization (default 1)
    kOptStaticWeights = 1,  // weight tensors are never written by kernels of the calling stream (default 0)
    kOptFullScales = 2,     // tcgen05 e4m3 kernels: block scales with 16 significant bits instead of 8 (default 0)
    kOptWaitLog2 = 3,       // log2 of the poll budget of the waits on OTHER GPUs (peer-memory combine); 0 = built-in (24)
    kNumOptions = 4,
};
int option(int which);
void set_option(int which, int value);

// Number of SMs of the current device (queried once per device); 148 if the query fails.
int sm_count();

// Fills the launch attributes common to the streaming kernels: cluster split-K and programmatic dependent launch.
inline int launch_attrs(cudaLaunchAttribute* attr, int cluster_y) {
    int n = 0;
    if (cluster_y > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = cluster_y;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (option(kOptPdl)) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    return n;
}

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(kCudaError, "%s: %s", what, cudaGetErrorString(e));
    return kOk;
}

}  // namespace mlk
