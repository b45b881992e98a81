// Expert-parallel combine across GPUs: the ranks' fp32 shares of the layer output are added and rounded once, in one
// kernel per rank over peer memory (NVLink / NVSwitch loads and stores), instead of an NCCL all-reduce plus a cast.
//
//   every rank holds   share_r [T, H] fp32   (its experts' un-rounded contribution, written by the expert compute)
//   rank i owns rows [T i / N, T (i + 1) / N): it reads those rows of every rank's share (its own from local memory,
//   the others through peer pointers), adds them in rank order (the same bits whichever rank computes), rounds to the
//   16-bit type and stores the finished rows into EVERY rank's output [T, H].
// A reduce-scatter and an all-gather in one pass: (N - 1) / N of the shares cross the links once as fp32, the result
// once as 16 bits.  The reference is single-GPU (its only hook is experts_map, csrc/moe_kernels/moe_align_tokens.h:44-49);
// this replaces the collective a caller of that hook would issue.
//
// Synchronisation.  CTA b of rank i exchanges flags with CTA b of every peer (same grid on all ranks):
//   A  "my share is complete" (the CTA has started, so the kernels before it in its stream have finished) -- waited for
//      before the peers' rows are read;
//   B  "my stores into your output are done" (after a system-scope fence) -- waited for before the CTA ends, so that
//      the kernel's completion on rank i means every peer's rows have arrived, and so that no rank's share is overwritten
//      by its next layer call while a peer still reads it.
// Flags carry an epoch kept in device memory (incremented by the last CTA of each launch), so a CUDA graph can replay the
// launch.  Every wait is bounded; on expiry the CTA records a status code and carries on (the output of that call is
// then incomplete, the kernel still ends).  No load uses TMA or multicast: plain ld / st on peer pointers.
#include <algorithm>

#include "common.cuh"
#include "moe.cuh"
#include "status.h"

namespace mlk {

namespace {

constexpr int kEpGrid = 128;            // CTAs per rank, the same on every rank
constexpr int kEpMaxWorld = 16;
constexpr int kEpFlagBase = 64;         // words 0 / 1: epoch, finished-CTA counter
constexpr unsigned kEpSpinLimit = 1u << 24;
constexpr int kEpExpired = 0x0E000001;
// Shares up to this many elements take the one-pass form; it moves world x the data of the two-exchange form, so the
// bound shrinks with the rank count (256 K elements up to four ranks, 128 K at eight).
constexpr long long kEpLlMaxElems = 256 * 1024;
constexpr long long kEpLlMaxWorldElems = 1024 * 1024;
inline bool ep_one_pass(int world, long long n) {
    return world > 1 && n > 0 && n <= std::min(kEpLlMaxElems, kEpLlMaxWorldElems / world);
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_peer16(const float* p) {
    float4 r;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(p) : "memory");
    return r;
}

// flag word of (phase, cta, source rank) inside a rank's flag block
__device__ __forceinline__ int flag_index(int phase, int cta, int src) {
    return kEpFlagBase + (phase * kEpGrid + cta) * kEpMaxWorld + src;
}

// Signals this CTA's flag to every rank and waits for every rank's flag (threads 0 .. world - 1 take one peer each).
__device__ __forceinline__ void exchange_flags(unsigned* const* flags, int rank, int world, int phase, unsigned epoch,
                                               unsigned spin_limit, int* status) {
    __syncthreads();
    const int t = threadIdx.x;
    if (t < world) {
        st_release_sys(flags[t] + flag_index(phase, blockIdx.x, rank), epoch);
        const unsigned* mine = flags[rank] + flag_index(phase, blockIdx.x, t);
        unsigned polls = 0;
        // epochs only grow; a flag from a later launch also means this one was passed
        while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
            if (++polls > spin_limit) {
                if (status != nullptr) atomicCAS(status, 0, kEpExpired);
                break;
            }
            __nanosleep(40);
        }
    }
    __syncthreads();
}

template <int WT>
__global__ void __launch_bounds__(256) ep_reduce_kernel(const float* const* __restrict__ shares, uint8_t* const* __restrict__ outs,
                                                       unsigned* const* __restrict__ flags, int rank, int world, long long T,
                                                       int H, unsigned spin_limit, int* status) {
    // the share comes from the kernels before this one in the stream: only past this wait may the peers be told that it is
    // complete (and the epoch of the previous launch has been written)
    pdl_wait();
    pdl_launch_dependents();
    unsigned* const my_flags = flags[rank];
    const unsigned epoch = *reinterpret_cast<volatile unsigned*>(my_flags) + 1u;    // read by every CTA before the last one of this launch moves it on

    exchange_flags(flags, rank, world, 0, epoch, spin_limit, status);

    const long long r0 = T * rank / world, r1 = T * (rank + 1) / world;
    const int quads = H >> 2;
    const long long total = (r1 - r0) * quads;
    const size_t base = (size_t)r0 * H;
    const long long stride = (long long)gridDim.x * blockDim.x;
    // peer loads take microseconds: kUnroll of them per rank are in flight per thread before the first is used
    constexpr int kUnroll = 4;
    for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < total; i0 += kUnroll * stride) {
        float4 acc[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < world; ++j) {             // rank order: the sum does not depend on who computes it
            float4 v[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const long long i = i0 + u * stride;
                v[u] = (i < total) ? ld_peer16(shares[j] + base + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w;
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const long long i = i0 + u * stride;
            if (i < total) {
                uint2 w;
                w.x = pack2<WT>(acc[u].x, acc[u].y);
                w.y = pack2<WT>(acc[u].z, acc[u].w);
                for (int j = 0; j < world; ++j) *reinterpret_cast<uint2*>(outs[j] + (base + 4 * i) * 2) = w;
            }
        }
    }
    __threadfence_system();

    exchange_flags(flags, rank, world, 1, epoch, spin_limit, status);

    // the last CTA out moves the epoch on for the next launch
    if (threadIdx.x == 0) {
        if (atomicAdd(&my_flags[1], 1u) == gridDim.x - 1) {
            my_flags[1] = 0;
            my_flags[0] = epoch;
            __threadfence();
        }
    }
}

// Small shares (decode batches): one pass, no barrier.  Every rank stores its whole share into every peer's receive
// buffer as 8-byte (value, epoch) pairs -- an aligned 8-byte store arrives whole, so the epoch says that the value
// next to it is this call's -- and adds what it receives in rank order as the pairs land; every rank computes the full
// output itself.  Receive buffers: [2 sets][world sources][T * H] pairs per rank, the set alternates with the epoch: a
// rank can be one call ahead of a peer (it needs the peer's data of call k + 1 to finish call k + 1) but not two.
template <int WT>
__global__ void __launch_bounds__(256) ep_reduce_ll_kernel(const float* const* __restrict__ shares, uint8_t* const* __restrict__ outs,
                                                          unsigned* const* __restrict__ flags, uint2* const* __restrict__ recv,
                                                          int rank, int world, long long n, unsigned spin_limit, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    unsigned* const my_flags = flags[rank];
    const unsigned epoch = *reinterpret_cast<volatile unsigned*>(my_flags) + 1u;
    const size_t set = (size_t)(epoch & 1u) * world * n;
    const float* const mine = shares[rank];
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long first = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    for (long long i = first; i < n; i += stride) {
        const uint2 pair = make_uint2(__float_as_uint(mine[i]), epoch);
        for (int j = 0; j < world; ++j)
            if (j != rank) {
                uint2* dst = recv[j] + set + (size_t)rank * n + i;
                asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(pair.x), "r"(pair.y) : "memory");
            }
    }
    uint16_t* const out = reinterpret_cast<uint16_t*>(outs[rank]);
    bool expired = false;
    for (long long i = first; i < n; i += stride) {
        float acc = 0.f;
        for (int j = 0; j < world; ++j) {            // rank order: every rank forms the same sum
            if (j == rank) {
                acc += mine[i];
                continue;
            }
            const uint2* src = recv[rank] + set + (size_t)j * n + i;
            uint2 pair;
            unsigned polls = 0;
            for (;;) {
                asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(pair.x), "=r"(pair.y) : "l"(src) : "memory");
                if (pair.y == epoch || expired) break;
                if (++polls > spin_limit) {
                    expired = true;
                    if (status != nullptr) atomicCAS(status, 0, kEpExpired);
                    break;
                }
            }
            acc += __uint_as_float(pair.x);
        }
        out[i] = (uint16_t)(pack2<WT>(acc, 0.f) & 0xFFFFu);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(&my_flags[1], 1u) == gridDim.x - 1) {
            my_flags[1] = 0;
            my_flags[0] = epoch;
            __threadfence();
        }
    }
}

}  // namespace

long long ep_reduce_flag_bytes() { return (long long)(kEpFlagBase + 2 * kEpGrid * kEpMaxWorld) * 4; }

long long ep_reduce_recv_bytes(int world, long long T, int H) {
    const long long n = T * H;
    return ep_one_pass(world, n) ? 2LL * world * n * 8 : 0;
}

int launch_ep_reduce(const void* const* shares_dev, void* const* outs_dev, void* const* flags_dev, void* const* recv_dev,
                     int rank, int world, long long T, int H, int dtype, int* status, cudaStream_t s) {
    if (!shares_dev || !outs_dev || !flags_dev) return fail(kInvalidArg, "ep_reduce_shares: null pointer");
    if (world < 1 || world > kEpMaxWorld || rank < 0 || rank >= world) return fail(kInvalidArg, "ep_reduce_shares: rank %d of %d", rank, world);
    if (T < 0 || H <= 0 || H % 4 != 0) return fail(kInvalidArg, "ep_reduce_shares: need hidden %% 4 == 0");
    if (dtype != kBF16 && dtype != kFP16) return fail(kInvalidArg, "ep_reduce_shares: output type must be bf16 or fp16");
    auto sh = reinterpret_cast<const float* const*>(shares_dev);
    auto ou = reinterpret_cast<uint8_t* const*>(outs_dev);
    auto fl = reinterpret_cast<unsigned* const*>(flags_dev);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kEpGrid);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = launch_attrs(attr, 1);
    cudaError_t e;
    const long long n = T * H;
    const int wl = option(kOptWaitLog2);
    const unsigned spin = (wl >= 4 && wl <= 30) ? (1u << wl) : kEpSpinLimit;      // poll budget of the waits on peers
    if (recv_dev != nullptr && ep_one_pass(world, n)) {
        // small share: the one-pass form
        auto rv = reinterpret_cast<uint2* const*>(recv_dev);
        cfg.gridDim = dim3((unsigned)std::min<long long>(kEpGrid, (n + 255) / 256));
        e = dtype == kFP16 ? cudaLaunchKernelEx(&cfg, ep_reduce_ll_kernel<kFP16>, sh, ou, fl, rv, rank, world, n, spin, status)
                           : cudaLaunchKernelEx(&cfg, ep_reduce_ll_kernel<kBF16>, sh, ou, fl, rv, rank, world, n, spin, status);
    } else {
        e = dtype == kFP16 ? cudaLaunchKernelEx(&cfg, ep_reduce_kernel<kFP16>, sh, ou, fl, rank, world, T, H, spin, status)
                           : cudaLaunchKernelEx(&cfg, ep_reduce_kernel<kBF16>, sh, ou, fl, rank, world, T, H, spin, status);
    }
    if (e != cudaSuccess) return fail(kCudaError, "ep_reduce_shares launch: %s", cudaGetErrorString(e));
    return kOk;
}

}  // namespace mlk
