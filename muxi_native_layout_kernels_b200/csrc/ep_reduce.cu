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
#include "common.cuh"
#include "moe.cuh"
#include "status.h"

namespace mlk {

namespace {

constexpr int kEpGrid = 96;             // CTAs per rank, the same on every rank
constexpr int kEpMaxWorld = 16;
constexpr int kEpFlagBase = 64;         // words 0 / 1: epoch, finished-CTA counter
constexpr unsigned kEpSpinLimit = 1u << 24;
constexpr int kEpExpired = 0x0E000001;

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
                                               int* status) {
    __syncthreads();
    const int t = threadIdx.x;
    if (t < world) {
        st_release_sys(flags[t] + flag_index(phase, blockIdx.x, rank), epoch);
        const unsigned* mine = flags[rank] + flag_index(phase, blockIdx.x, t);
        unsigned polls = 0;
        // epochs only grow; a flag from a later launch also means this one was passed
        while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
            if (++polls > kEpSpinLimit) {
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
                                                       int H, int* status) {
    unsigned* const my_flags = flags[rank];
    const unsigned epoch = my_flags[0] + 1u;          // every CTA reads it before the last one of this launch moves it on

    exchange_flags(flags, rank, world, 0, epoch, status);

    const long long r0 = T * rank / world, r1 = T * (rank + 1) / world;
    const int quads = H >> 2;
    const long long total = (r1 - r0) * quads;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long row = r0 + i / quads;
        const int q = (int)(i % quads);
        const size_t off = (size_t)row * H + 4 * q;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < world; ++j) {             // rank order: the sum does not depend on who computes it
            const float4 v = ld_peer16(shares[j] + off);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        uint2 w;
        w.x = pack2<WT>(acc.x, acc.y);
        w.y = pack2<WT>(acc.z, acc.w);
        for (int j = 0; j < world; ++j) *reinterpret_cast<uint2*>(outs[j] + off * 2) = w;
    }
    __threadfence_system();

    exchange_flags(flags, rank, world, 1, epoch, status);

    // the last CTA out moves the epoch on for the next launch
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

int launch_ep_reduce(const void* const* shares_dev, void* const* outs_dev, void* const* flags_dev, int rank, int world,
                     long long T, int H, int dtype, int* status, cudaStream_t s) {
    if (!shares_dev || !outs_dev || !flags_dev) return fail(kInvalidArg, "ep_reduce_shares: null pointer");
    if (world < 1 || world > kEpMaxWorld || rank < 0 || rank >= world) return fail(kInvalidArg, "ep_reduce_shares: rank %d of %d", rank, world);
    if (T < 0 || H <= 0 || H % 4 != 0) return fail(kInvalidArg, "ep_reduce_shares: need hidden %% 4 == 0");
    if (dtype != kBF16 && dtype != kFP16) return fail(kInvalidArg, "ep_reduce_shares: output type must be bf16 or fp16");
    // launched without programmatic serialization: its start must mean that the kernels before it have finished
    auto sh = reinterpret_cast<const float* const*>(shares_dev);
    auto ou = reinterpret_cast<uint8_t* const*>(outs_dev);
    auto fl = reinterpret_cast<unsigned* const*>(flags_dev);
    if (dtype == kFP16) ep_reduce_kernel<kFP16><<<kEpGrid, 256, 0, s>>>(sh, ou, fl, rank, world, T, H, status);
    else ep_reduce_kernel<kBF16><<<kEpGrid, 256, 0, s>>>(sh, ou, fl, rank, world, T, H, status);
    return check_launch("ep_reduce_shares");
}

}  // namespace mlk
