// MoE token alignment: flat slots i = token*topk + j grouped by expert, each expert's run padded to a
// multiple of the micro batch, one expert id per block -- all in one single-CTA kernel (the problem is
// a few thousand integers; latency, not bandwidth, is what counts).
//
// Contract kept from the reference (csrc/moe_kernels/moe_align_tokens.h:9-94, moe_align_tokens.cu:5-21):
//   experts_ids_out[0..max_blocks) is zero-filled, then [b] = e for every block of expert e
//   padded_num_experts[0] = number of blocks
//   sorted_token_ids[start_e + r] = i for the r-th slot routed to e (order inside an expert is unspecified);
//     every other position holds the sentinel T*topk (written here, so the caller need not pre-fill)
//   cumsum_buffer: [e] = start_e + count_e for e < E, [E] = padded total -- the state the reference leaves
//     behind after its second kernel has used the buffer as per-expert cursors
//   experts_map: global id -> local id, -1 = not on this rank (slot is skipped)
// Optionally the kernel also emits the expert-compute work list (see MoeWorkHeader in moe.cuh) and, with it, the slot of
// every compact position (cpos_slot: the routed slots numbered expert by expert without the padding).
#include "common.cuh"
#include "moe.cuh"
#include "status.h"

namespace mlk {

namespace {

constexpr int kMaxExperts = 1024;

__global__ void __launch_bounds__(1024) moe_align_kernel(const int32_t* __restrict__ topk_ids, int numel, int E,
                                                        int mbs, int max_blocks, int max_padded, int32_t* __restrict__ sorted,
                                                        int32_t* __restrict__ cumsum, int32_t* __restrict__ nblocks,
                                                        int32_t* __restrict__ block_expert,
                                                        const int32_t* __restrict__ experts_map, int n_global,
                                                        int4* __restrict__ worklist, int block_slots,
                                                        int32_t* __restrict__ cpos_slot) {
    __shared__ int cnt[kMaxExperts];
    __shared__ int cursor[kMaxExperts];
    __shared__ int pad_before[kMaxExperts];     // padding in front of expert e: position minus compact position
    __shared__ int warp_tot[32], warp_tot2[32], warp_tot3[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // the routing comes from the preceding kernel of the stream (and the buffers written here may still be read by it
    // or its predecessors); the kernels behind this one may become resident meanwhile
    pdl_wait();
    pdl_launch_dependents();
    for (int e = tid; e < E; e += blockDim.x) cnt[e] = 0;
    for (int b = tid; b < max_blocks; b += blockDim.x) block_expert[b] = 0;
    for (int i = tid; i < max_padded; i += blockDim.x) sorted[i] = numel;   // sentinel everywhere; slots overwrite it below
    __syncthreads();

    for (int i = tid; i < numel; i += blockDim.x) {
        int e = topk_ids[i];
        if (experts_map != nullptr) e = (e >= 0 && e < n_global) ? experts_map[e] : -1;
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();

    // block-wide exclusive scans over experts (E <= 1024 = blockDim): padded counts and work items
    const int c = (tid < E) ? cnt[tid] : 0;
    const int padded = ((c + mbs - 1) / mbs) * mbs;
    const int items = (block_slots > 0) ? (c + block_slots - 1) / block_slots : 0;
    int incl = padded, incl2 = items, incl3 = c;      // incl3: unpadded ("compact") positions
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
        const int v2 = __shfl_up_sync(0xFFFFFFFFu, incl2, o);
        const int v3 = __shfl_up_sync(0xFFFFFFFFu, incl3, o);
        if (lane >= o) { incl += v; incl2 += v2; incl3 += v3; }
    }
    if (lane == 31) { warp_tot[warp] = incl; warp_tot2[warp] = incl2; warp_tot3[warp] = incl3; }
    __syncthreads();
    if (warp == 0) {
        int w = warp_tot[lane], w2 = warp_tot2[lane], w3 = warp_tot3[lane];
        const int nw = blockDim.x >> 5;
        if (lane >= nw) { w = 0; w2 = 0; w3 = 0; }
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xFFFFFFFFu, w, o);
            const int v2 = __shfl_up_sync(0xFFFFFFFFu, w2, o);
            const int v3 = __shfl_up_sync(0xFFFFFFFFu, w3, o);
            if (lane >= o) { w += v; w2 += v2; w3 += v3; }
        }
        warp_tot[lane] = w;
        warp_tot2[lane] = w2;
        warp_tot3[lane] = w3;
    }
    __syncthreads();
    const int base = (warp > 0) ? warp_tot[warp - 1] : 0;
    const int base2 = (warp > 0) ? warp_tot2[warp - 1] : 0;
    const int excl = base + incl - padded;
    const int excl2 = base2 + incl2 - items;
    const int excl3 = ((warp > 0) ? warp_tot3[warp - 1] : 0) + incl3 - c;
    if (tid < E) {
        cursor[tid] = excl;
        pad_before[tid] = excl - excl3;
        cumsum[tid] = excl + c;
        for (int b = excl / mbs; b < (excl + padded) / mbs; ++b) block_expert[b] = tid;
        if (worklist != nullptr)
            for (int j = 0; j < items; ++j)
                worklist[1 + excl2 + j] = make_int4(tid, excl + j * block_slots, min(block_slots, c - j * block_slots),
                                                    excl3 + j * block_slots);
    }
    if (tid == E - 1) {
        cumsum[E] = excl + padded;
        nblocks[0] = (excl + padded) / mbs;
        if (worklist != nullptr) worklist[0] = make_int4(excl2 + items, excl3 + c, 0, 0);
    }
    __syncthreads();

    for (int i = tid; i < numel; i += blockDim.x) {
        int e = topk_ids[i];
        if (experts_map != nullptr) e = (e >= 0 && e < n_global) ? experts_map[e] : -1;
        if (e >= 0 && e < E) {
            const int pos = atomicAdd(&cursor[e], 1);
            sorted[pos] = i;
            if (cpos_slot != nullptr) cpos_slot[pos - pad_before[e]] = i;
        }
    }
}

}  // namespace

int launch_moe_align(int T, int E, int topk, int mbs, const int32_t* topk_ids, int32_t* sorted_token_ids,
                     int32_t* cumsum, int32_t* padded_num_experts, int32_t* experts_ids_out,
                     const int32_t* experts_map, int experts_map_len, cudaStream_t s, void* worklist,
                     int block_slots, int32_t* cpos_slot) {
    if (!topk_ids || !sorted_token_ids || !cumsum || !padded_num_experts || !experts_ids_out)
        return fail(kInvalidArg, "moe_align: null pointer");
    if (T < 0 || topk <= 0) return fail(kInvalidArg, "moe_align: bad batch size / topK");
    if (E <= 0 || E > kMaxExperts) return fail(kUnsupported, "moe_align: 1 <= expertCount <= %d (got %d)", kMaxExperts, E);
    if (mbs <= 0) return fail(kInvalidArg, "moe_align: microBatchSize must be positive");
    const long long numel = (long long)T * topk;
    if (numel > 0x3FFFFFFF) return fail(kInvalidArg, "moe_align: too many slots");
    const int max_padded = (int)numel + E * (mbs - 1);
    const int max_blocks = (max_padded + mbs - 1) / mbs;
    if (experts_map != nullptr && experts_map_len <= 0) return fail(kInvalidArg, "moe_align: experts_map needs its length");
    const int n_global = experts_map_len;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(1024);
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = launch_attrs(attr, 1);
    const cudaError_t e = cudaLaunchKernelEx(&cfg, moe_align_kernel, topk_ids, (int)numel, E, mbs, max_blocks, max_padded,
                                             sorted_token_ids, cumsum, padded_num_experts, experts_ids_out, experts_map, n_global,
                                             reinterpret_cast<int4*>(worklist), block_slots, cpos_slot);
    if (e != cudaSuccess) return fail(kCudaError, "moe_align launch: %s", cudaGetErrorString(e));
    return kOk;
}

}  // namespace mlk
