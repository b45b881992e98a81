// Fused-MoE expert compute for decode batches (at most 8 tokens and 64 routed slots) as ONE persistent kernel, one
// CTA per SM:  work list -> gather-GEMM1 with SiLU*up -> grid barrier -> GEMM2 x routing weight -> per-token sum.
//
// At one token the layer's weights are a few tens of megabytes spread over a handful of experts; what limits a
// chain of small launches is not bandwidth but how many bytes each SM has in flight and how often the chain starts
// over.  Here every SM's whole share of the weights is requested up front: a producer warp walks the CTA's task list
// and issues one bulk copy (cp.async.bulk, completion on an mbarrier) per 8 KB segment of layout A into a 192 KB
// shared-memory ring, without waiting for the routing-dependent activations; eight consumer warps multiply the
// segments as they land (mma.sync m16n8k16 straight from the layout-A bytes in shared memory, the same fragment
// mapping as the streaming core: a [16 rows][8 k] block of layout A is the A fragment of two lanes' 16-byte loads).
// The second GEMM's weights follow in the same ring while the first is still being multiplied.
//
// Decomposition.  Phase 1: a unit is (work item, 16 gate rows + the 16 matching up rows), K = H split into segments;
// the CTA owns a contiguous range of units.  Phase 2: a unit is (16-row tile of H, work item), K = I; the CTA owns
// whole tiles, so every slot's rows of a tile are produced in one CTA and each token's top-k rows are added there in
// slot order (fp32, one rounding) -- no combine scratch, no atomics on the output.
// The only cross-CTA wait is the grid barrier between the phases: the launch is cooperative (all CTAs resident), the
// spin is bounded, and on expiry the CTA records a status code and carries on, so the kernel always ends.
//
// Replaces, for small batches, the launch sequence of fused_experts_compute
// (csrc/moe_kernels/fused_experts_compute.cu:50-296; muxi_layout_kernels/muxi_moe_planC.py:56-149).
#include <algorithm>
#include <atomic>

#include "moe.cuh"
#include "moe_route.cuh"
#include "status.h"
#include "umma_common.cuh"

namespace mlk {

namespace {

using umma::mbar_init;
using umma::mbar_expect_tx;
using umma::mbar_try_wait;

constexpr int kDecSlots = 64;          // T * topk at most
constexpr int kDecTokens = 8;          // T at most
constexpr int kDecPool = 64;           // independent sets of counters, handed out round-robin per launch
constexpr int kRing = 24;              // ring slots
constexpr int kSegBytes = 8192;        // one slot: 16 rows x (512 e4m3 | 256 16-bit) k values of layout A
constexpr int kConsumers = 16;         // consumer warps; the warp after them is the producer
constexpr int kThreads = (kConsumers + 1) * 32;
constexpr unsigned kDecSpinLimit = 1u << 22;       // polls of the grid barrier before giving up
constexpr uint32_t kDecWaitLimit = 1u << 22;       // try_wait attempts on a ring barrier before giving up
constexpr int kDecBarrierExpired = 0x0D000001;
constexpr int kDecRingExpired = 0x0D000002;

struct DecodeSync {
    unsigned barrier;            // CTAs that finished the first GEMM
    unsigned done;               // CTAs that finished the kernel
};
__device__ DecodeSync g_decode_sync[kDecPool];

#ifdef MLK_DECODE_TIMELINE
// Developer instrumentation (compiled out by default): per-CTA %globaltimer stamps of the phases.
__device__ long long g_dec_timeline[512 * 16];
#define MLK_DTL(slot, who)                                                                                \
    do {                                                                                                  \
        if (threadIdx.x == (who) && blockIdx.x < 512) {                                                   \
            long long t_;                                                                                 \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                        \
            g_dec_timeline[blockIdx.x * 16 + (slot)] = t_;                                                 \
        }                                                                                                 \
    } while (0)
#else
#define MLK_DTL(slot, who) do { } while (0)
#endif

struct DecodeParams {
    const uint8_t* w1;
    const uint8_t* w2;
    long long w1_expert_bytes, w2_expert_bytes;
    const float* s1;
    const float* s2;
    long long s1_expert, s2_expert;
    const uint8_t* x;            // [T, H]
    uint8_t* act;                // [slots, I] 16-bit
    void* y;                     // [T, H] 16-bit or fp32
    const int32_t* topk_ids;
    const void* topk_weights;
    const int32_t* experts_map;
    int map_len;
    int T, E, topk, H, I;
    int fp8_order, y_fp32, mbs;
    int32_t* sorted;             // alignment outputs of the reference contract, written by the last CTA
    int32_t* cumsum;
    int32_t* nblocks;
    int32_t* block_expert;
    int max_blocks, max_padded;
    // routing fused in front: logits != nullptr; topk_ids / topk_weights then receive the routing (written by CTA 0)
    const void* logits;          // [T, n_global]
    const void* route_bias;
    int n_global, score_fun, n_groups, topk_groups, renormalize;
    int sync_slot;
    int* status;
};

// Bookkeeping in static shared memory.
struct DecodeShared {
    int cnt[1024];                   // routed slots per expert (then: first item of the expert)
    int expert_of_slot[kDecSlots];   // local expert id or -1
    int rank_of_slot[kDecSlots];     // position of the slot among its expert's slots
    int item_expert[kDecSlots];
    int item_n[kDecSlots];
    int item_slot[kDecSlots][8];
    int warp_tot[8];
    int n_items;
    volatile int abort;
    float slot_weight[kDecSlots];    // routing weight of every slot
    int32_t route_ids[kDecSlots];    // fused routing: the ids and (16-bit) weights of every slot
    uint16_t route_wts[kDecSlots];
    int released[kRing];             // how many uses of each ring slot its consumers have finished with
};

// One GEMM phase as every role sees it.
struct Phase {
    int unit0, unit1;        // this CTA's units
    int nseg;                // K segments per unit
    int seg_chunks;          // 32-k chunks per segment (the last one may be shorter)
    int chunks;              // K / 32
    int upr;                 // units per round of the eight consumer warps
    int planes;              // ring slots per task: 2 (gate, up) or 1
    int g0;                  // ring sequence number of the phase's first slot
};

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory"); }
// weights are read once: their L2 lines are marked evict-first
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(pol)
                 : "memory");
}
__device__ __forceinline__ uint4 ldg_l2_16(const void* p) {
    uint4 r;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
    return r;
}

// Bounded wait on a ring barrier; gives up at once when another role already has.
__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity, DecodeShared& ds, int* status) {
    if (ds.abort) return false;
    for (uint32_t i = 0; i < kDecWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023) == 1023 && ds.abort) return false;
    }
    ds.abort = 1;
    if (status != nullptr) atomicCAS(status, 0, kDecRingExpired);
    return false;
}

// Work list in shared memory, built by every CTA for itself (at most 64 integers of routing): items of at most 8 slots
// of one expert, experts ascending.  All threads of the CTA take part.
__device__ __forceinline__ void build_items(const DecodeParams& p, DecodeShared& ds, bool wt_is_fp16, const int32_t* ids,
                                            const void* wts) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int numel = p.T * p.topk;
    if (tid == 0) ds.abort = 0;
    if (tid < kRing) ds.released[tid] = 0;
    if (tid >= 64 && tid < 64 + numel)
        ds.slot_weight[tid - 64] = wt_is_fp16 ? load_scalar16<kFP16>(wts, tid - 64) : load_scalar16<kBF16>(wts, tid - 64);
    if (p.T == 1 && numel <= 32) {
        // one token: every routed slot is its own item (its experts differ), no counting or scanning
        if (warp == 0) {
            int e = -1;
            if (lane < numel) {
                e = ids[lane];
                if (p.experts_map != nullptr) e = (e >= 0 && e < p.map_len) ? p.experts_map[e] : -1;
                if (e < 0 || e >= p.E) e = -1;
            }
            const unsigned valid = __ballot_sync(0xFFFFFFFFu, e >= 0);
            const unsigned same = __match_any_sync(0xFFFFFFFFu, e);
            const unsigned lt = (1u << lane) - 1u;
            ds.expert_of_slot[lane] = e;
            ds.rank_of_slot[lane] = __popc(same & lt);
            if (e >= 0) {
                const int item = __popc(valid & lt);
                ds.item_expert[item] = e;
                ds.item_n[item] = 1;
                ds.item_slot[item][0] = lane;
            }
            if (lane == 0) ds.n_items = __popc(valid);
        }
        __syncthreads();
        return;
    }
    for (int e = tid; e < p.E; e += kThreads) ds.cnt[e] = 0;
    __syncthreads();
    // rank of a slot among the slots of its expert, in slot order (the same in every CTA): inside a warp by matching
    // lanes, the second warp of slots on top of the first one's counts
    int e_mine = -1, r_mine = 0;
    unsigned same = 0;
    if (tid < kDecSlots) {
        if (tid < numel) {
            e_mine = ids[tid];
            if (p.experts_map != nullptr) e_mine = (e_mine >= 0 && e_mine < p.map_len) ? p.experts_map[e_mine] : -1;
            if (e_mine < 0 || e_mine >= p.E) e_mine = -1;
        }
        ds.expert_of_slot[tid] = e_mine;
        same = __match_any_sync(0xFFFFFFFFu, e_mine);
        r_mine = __popc(same & ((1u << lane) - 1u));
        if (warp == 0 && e_mine >= 0 && r_mine == 0) ds.cnt[e_mine] = __popc(same);
    }
    __syncthreads();
    int base = 0;
    if (warp == 1 && e_mine >= 0) base = ds.cnt[e_mine];
    if (warp == 1) __syncwarp();
    if (warp == 1 && e_mine >= 0) {
        if (r_mine == 0) ds.cnt[e_mine] = base + __popc(same);
        r_mine += base;
    }
    if (tid < kDecSlots) ds.rank_of_slot[tid] = r_mine;
    __syncthreads();
    // exclusive scan of the items per expert (ceil(count / 8)): thread t < 256 owns experts 4t .. 4t+3
    int c[4] = {0, 0, 0, 0}, mine = 0;
    if (tid < 256) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid * 4 + i;
            c[i] = (e < p.E) ? ds.cnt[e] : 0;
            mine += (c[i] + 7) >> 3;
        }
    }
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31 && warp < 8) ds.warp_tot[warp] = incl;
    __syncthreads();
    if (tid < 256) {
        int first = incl - mine;
        for (int w = 0; w < warp; ++w) first += ds.warp_tot[w];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid * 4 + i;
            if (e < p.E) ds.cnt[e] = first;
            for (int k = 0; k * 8 < c[i]; ++k) {
                ds.item_expert[first] = e;
                ds.item_n[first] = min(8, c[i] - 8 * k);
                ++first;
            }
        }
        if (tid == 255) ds.n_items = first;
    }
    __syncthreads();
    if (e_mine >= 0) ds.item_slot[ds.cnt[e_mine] + (r_mine >> 3)][r_mine & 7] = tid;
    __syncthreads();
}

// The alignment outputs the reference's entry point leaves behind (moe_align.cu states the contract), from the expert
// of every slot in shared memory.  One warp (the producer warp of the last CTA, once its copies are issued: off the
// critical path); nothing in this kernel reads the outputs.  ds.cnt is free by then (the items are built).
__device__ __forceinline__ void write_alignment(const DecodeParams& p, DecodeShared& ds) {
    const int lane = threadIdx.x & 31;
    const int numel = p.T * p.topk;
    const int mbs = p.mbs;
    int* cnt = ds.cnt;
    for (int e = lane; e < p.E; e += 32) cnt[e] = 0;
    for (int b = lane; b < p.max_blocks; b += 32) p.block_expert[b] = 0;
    for (int i = lane; i < p.max_padded; i += 32) p.sorted[i] = numel;
    __syncwarp();
    for (int i = lane; i < numel; i += 32)
        if (ds.expert_of_slot[i] >= 0) atomicAdd(&cnt[ds.expert_of_slot[i]], 1);
    __syncwarp();
    // lane l owns experts [l * per, (l + 1) * per): padded counts scanned across the warp, then serially inside
    const int per = (p.E + 31) / 32;
    int mine = 0;
    for (int e = lane * per; e < min(p.E, (lane + 1) * per); ++e) mine += ((cnt[e] + mbs - 1) / mbs) * mbs;
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
        if (lane >= o) incl += v;
    }
    int start = incl - mine;
    for (int e = lane * per; e < min(p.E, (lane + 1) * per); ++e) {
        const int c = cnt[e];
        const int padded = ((c + mbs - 1) / mbs) * mbs;
        p.cumsum[e] = start + c;
        for (int b = start / mbs; b < (start + padded) / mbs; ++b) p.block_expert[b] = e;
        cnt[e] = start;            // becomes the expert's first position
        start += padded;
    }
    const int total = __shfl_sync(0xFFFFFFFFu, incl, 31);
    if (lane == 0) {
        p.cumsum[p.E] = total;
        p.nblocks[0] = total / mbs;
    }
    __syncwarp();
    for (int i = lane; i < numel; i += 32)
        if (ds.expert_of_slot[i] >= 0) p.sorted[cnt[ds.expert_of_slot[i]] + ds.rank_of_slot[i]] = i;
}

template <int WT>
struct DecShape {
    static constexpr int ESZ = (WT == kE4M3) ? 1 : 2;
    static constexpr int CB = 512 * ESZ;                 // bytes of one 32-k chunk of a 16-row group
    static constexpr int MAXC = kSegBytes / CB;          // chunks per ring slot: 16 (e4m3) or 8 (16-bit)
};

// Splits K (in 32-k chunks) into the fewest segments that fit a ring slot; with block scales a segment is a whole
// number of 128-k blocks.
template <int WT, bool SCALE>
__device__ __forceinline__ void split_k(int chunks, int& nseg, int& seg_chunks) {
    constexpr int MAXC = DecShape<WT>::MAXC;
    nseg = (chunks + MAXC - 1) / MAXC;
    seg_chunks = (chunks + nseg - 1) / nseg;
    if (SCALE) seg_chunks = (seg_chunks + 3) & ~3;
    nseg = (chunks + seg_chunks - 1) / seg_chunks;
}

// A ring slot is free for its use number `use` once `use` earlier uses have been released.  A counter, not an
// mbarrier: parity waits cannot tell phases two apart, and neither the producer lanes nor the consumer warps are
// bound to be less than two uses of a slot apart.
__device__ __forceinline__ bool slot_wait_released(DecodeShared& ds, int slot, int use, int* status) {
    if (ds.abort) return false;
    const uint32_t addr = smem_u32(&ds.released[slot]);
    for (uint32_t i = 0; i < kDecWaitLimit; ++i) {
        int v;
        asm volatile("ld.acquire.cta.shared.s32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
        if (v >= use) return true;
        if ((i & 1023) == 1023 && ds.abort) return false;
    }
    ds.abort = 1;
    if (status != nullptr) atomicCAS(status, 0, kDecRingExpired);
    return false;
}
__device__ __forceinline__ void slot_release(DecodeShared& ds, int slot) {
    const uint32_t addr = smem_u32(&ds.released[slot]);
    asm volatile("red.release.cta.shared.add.s32 [%0], 1;" ::"r"(addr) : "memory");
}

// ---- producer warp: one bulk copy per ring slot, both phases back to back.  Lane l owns ring slot l and issues the
// sequence numbers l, l + 24, ...: every lane finds its task in closed form, so 24 copies are issued at a time. ------
template <int WT>
__device__ __forceinline__ void produce(const DecodeParams& p, DecodeShared& ds, const Phase& p1, const Phase& p2,
                                        uint32_t ring, uint32_t full0) {
    constexpr int ESZ = DecShape<WT>::ESZ, CB = DecShape<WT>::CB;
    const int lane = threadIdx.x & 31;
    const int n_items = ds.n_items;
    const int groups1 = p.I >> 4;
    const int G1 = 2 * (p1.unit1 - p1.unit0) * p1.nseg;
    const int GT = G1 + (p2.unit1 - p2.unit0) * p2.nseg;
    bool ok = true;
    int issued = -1;
    // One lane per ring slot: the uses of a slot are then issued in order by one thread, which waits for use n - 1 to
    // be released only after it issued it (a parity wait cannot tell phases two apart).
    for (int g = lane; lane < kRing && g < GT && ok; g += kRing) {
        const uint8_t* src;
        uint32_t bytes;
        if (g < G1) {
            const int q = g >> 1, pl = g & 1;
            const int u = p1.unit0 + q / p1.nseg, s = q % p1.nseg;
            const int item = u / groups1, rg = u - item * groups1;
            const int c0 = s * p1.seg_chunks, c1 = min(p1.chunks, c0 + p1.seg_chunks);
            bytes = (uint32_t)(c1 - c0) * CB;
            src = p.w1 + (long long)ds.item_expert[item] * p.w1_expert_bytes +
                  ((size_t)(rg + pl * groups1) * 16 * p.H) * ESZ + (size_t)c0 * CB;         // gate rows, then up rows
        } else {
            const int q = g - G1;
            const int v = p2.unit0 + q / p2.nseg, s = q % p2.nseg;
            const int tile = v / n_items, item = v - tile * n_items;
            const int c0 = s * p2.seg_chunks, c1 = min(p2.chunks, c0 + p2.seg_chunks);
            bytes = (uint32_t)(c1 - c0) * CB;
            src = p.w2 + (long long)ds.item_expert[item] * p.w2_expert_bytes + ((size_t)tile * 16 * p.I) * ESZ + (size_t)c0 * CB;
        }
        const int slot = g % kRing, use = g / kRing;
        if (use > 0) ok = slot_wait_released(ds, slot, use, p.status);
        if (ok) {
            mbar_expect_tx(full0 + 8 * slot, bytes);
            bulk_load(ring + slot * kSegBytes, src, bytes, full0 + 8 * slot);
            issued = g;
        }
    }
    if (ds.abort && issued >= 0) {
        // someone gave up: no copy of this lane may still be in flight when the CTA leaves
        const uint32_t bar = full0 + 8 * (issued % kRing), parity = (uint32_t)(issued / kRing) & 1u;
        for (uint32_t i = 0; i < kDecWaitLimit; ++i)
            if (mbar_try_wait(bar, parity)) break;
    }
}

// ---- consumer: one task = the PL slots of (unit, segment); fp32 sums of 16 rows x 8 token columns per plane ---------
// xrow: this lane's token row (token = lane / 4) at k = 0, or null; L2: read it past L1 (rows other CTAs just wrote).
template <int WT, bool SCALE, int PL, bool L2, bool XALL>
__device__ __forceinline__ void consume_task(float (&acc)[PL][4], const DecodeParams& p, DecodeShared& ds, uint32_t ring,
                                             uint32_t full0, int g, int c0, int nch, const uint8_t* xrow,
                                             const float* const (&scale_row)[PL]) {
    constexpr int ESZ = DecShape<WT>::ESZ, CB = DecShape<WT>::CB, MAXC = DecShape<WT>::MAXC;
    const int lane = threadIdx.x & 31, gq = lane >> 2, t = lane & 3;
    // token fragments four chunks (128 k) at a time, one block ahead; the first block before the weights have arrived
    auto load_x = [&](uint4 (&dst)[4], int cb) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            dst[i] = make_uint4(0, 0, 0, 0);
            if (xrow != nullptr && cb + i < nch) {
                const uint8_t* src = xrow + (size_t)(c0 + cb + i) * 64 + t * 16;
                dst[i] = L2 ? ldg_l2_16(src) : __ldg(reinterpret_cast<const uint4*>(src));
            }
        }
    };
    // XALL: all of the segment's fragments at once (phase 2: they come from L2, one round trip instead of one per block)
    constexpr int NB = XALL ? MAXC / 4 : 1;
    uint4 xn[NB][4];
#pragma unroll
    for (int bq = 0; bq < NB; ++bq) load_x(xn[bq], 4 * bq);
    uint32_t sb[PL];
    bool ok = true;
#pragma unroll
    for (int pl = 0; pl < PL; ++pl) {
        const int slot = (g + pl) % kRing, use = (g + pl) / kRing;
        sb[pl] = ring + slot * kSegBytes + t * (128 * ESZ) + gq * 16;
        // A round can span more slots than the ring has, so the slot's previous use may not even have landed: first
        // wait until that use has been released (then the barrier is in this use's phase), then for this use's bytes.
        if (use > 0) ok = slot_wait_released(ds, slot, use, p.status) && ok;
        ok = ok && ring_wait(full0 + 8 * slot, (uint32_t)use & 1u, ds, p.status);
    }
    if (ok) {
        const uint32_t sel01 = p.fp8_order ? kSelRep01 : kSelNat01, sel23 = p.fp8_order ? kSelRep23 : kSelNat23;
        float blk[SCALE ? PL : 1][4];
        float sc[PL];
#pragma unroll
        for (int cb = 0; cb < MAXC; cb += 4) {
            if (cb < nch) {
                uint4 xf[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) xf[i] = xn[XALL ? cb / 4 : 0][i];
                if constexpr (!XALL) {
                    if (cb + 4 < nch) load_x(xn[0], cb + 4);
                }
                if constexpr (SCALE) {
#pragma unroll
                    for (int pl = 0; pl < PL; ++pl) {
                        sc[pl] = __ldg(scale_row[pl] + ((c0 + cb) >> 2));
                        blk[pl][0] = blk[pl][1] = blk[pl][2] = blk[pl][3] = 0.f;
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c = cb + i;
                    if (c < nch) {
#pragma unroll
                        for (int pl = 0; pl < PL; ++pl) {
                            uint32_t p0, p1, p2, p3, q0, q1, q2, q3;
                            if constexpr (WT == kE4M3) {
                                const uint4 w = lds16(sb[pl] + c * CB);
                                p0 = e4m3x2_to_bf16x2(w.x, sel01); p1 = e4m3x2_to_bf16x2(w.x, sel23);
                                p2 = e4m3x2_to_bf16x2(w.y, sel01); p3 = e4m3x2_to_bf16x2(w.y, sel23);
                                q0 = e4m3x2_to_bf16x2(w.z, sel01); q1 = e4m3x2_to_bf16x2(w.z, sel23);
                                q2 = e4m3x2_to_bf16x2(w.w, sel01); q3 = e4m3x2_to_bf16x2(w.w, sel23);
                            } else {
                                const uint4 lo = lds16(sb[pl] + c * CB), hi = lds16(sb[pl] + c * CB + 128);
                                p0 = lo.x; p1 = lo.y; p2 = lo.z; p3 = lo.w;
                                q0 = hi.x; q1 = hi.y; q2 = hi.z; q3 = hi.w;
                            }
                            if constexpr (SCALE) {
                                mma16816<WT>(blk[pl], p0, q0, p1, q1, xf[i].x, xf[i].y);
                                mma16816<WT>(blk[pl], p2, q2, p3, q3, xf[i].z, xf[i].w);
                            } else {
                                mma16816<WT>(acc[pl], p0, q0, p1, q1, xf[i].x, xf[i].y);
                                mma16816<WT>(acc[pl], p2, q2, p3, q3, xf[i].z, xf[i].w);
                            }
                        }
                    }
                }
                if constexpr (SCALE) {
#pragma unroll
                    for (int pl = 0; pl < PL; ++pl)
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[pl][i] = fmaf(sc[pl], blk[pl][i], acc[pl][i]);
                }
            }
        }
    }
    __syncwarp();
    if (lane == 0 && ok)
#pragma unroll
        for (int pl = 0; pl < PL; ++pl) slot_release(ds, (g + pl) % kRing);
}

// ---- consumer: one phase.  PHASE 1: units (item, gate/up row group pair) -> act;  PHASE 2: units (tile, item) ->
// weighted rows of the tile in shared memory, and after a tile's last item the per-token sums -> y. ----------------
template <int WT, bool SCALE, int PHASE>
__device__ __forceinline__ void consume_phase(const DecodeParams& p, DecodeShared& ds, const Phase& ph, uint32_t ring,
                                              uint32_t full0, float* partial, float* out_s) {
    constexpr int PL = (PHASE == 1) ? 2 : 1;
    constexpr int AT = (WT == kFP16) ? kFP16 : kBF16;     // activation type
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, t = lane & 3;
    const int n_items = ds.n_items;
    const int groups1 = p.I >> 4;
    const int K = (PHASE == 1) ? p.H : p.I;
    const int ldscale = (K + 127) >> 7;
    constexpr int NT = kConsumers * 32;
    for (int u = ph.unit0; u < ph.unit1;) {
        int nu = min(ph.upr, ph.unit1 - u);
        if (PHASE == 2) nu = min(nu, n_items - u % n_items);       // a round stays inside one tile
        // this warp's unit of the round and its segments: with 8 or more segments per unit all warps share one unit
        const int ui = (ph.nseg >= kConsumers) ? 0 : warp / ph.nseg;
        const int s_first = (ph.nseg >= kConsumers) ? warp : warp % ph.nseg;
        const int s_step = (ph.nseg >= kConsumers) ? kConsumers : ph.nseg;
        const bool active = ui < nu;
        float acc[PL][4];
#pragma unroll
        for (int pl = 0; pl < PL; ++pl) acc[pl][0] = acc[pl][1] = acc[pl][2] = acc[pl][3] = 0.f;
        if (active) {
            const int unit = u + ui;
            const int item = (PHASE == 1) ? unit / groups1 : unit % n_items;
            const int rgidx = (PHASE == 1) ? unit - item * groups1 : unit / n_items;       // row group / tile
            const int nt = ds.item_n[item];
            const uint8_t* xrow = nullptr;
            if (gq < nt) {
                const int slot = ds.item_slot[item][gq];
                xrow = (PHASE == 1) ? p.x + (size_t)(slot / p.topk) * p.H * 2 : p.act + (size_t)slot * p.I * 2;
            }
            const float* srow[PL];
#pragma unroll
            for (int pl = 0; pl < PL; ++pl) {
                srow[pl] = nullptr;
                if constexpr (SCALE) {
                    const int row = (rgidx + pl * groups1) * 16;
                    srow[pl] = ((PHASE == 1) ? p.s1 + (long long)ds.item_expert[item] * p.s1_expert
                                             : p.s2 + (long long)ds.item_expert[item] * p.s2_expert) + (size_t)(row >> 7) * ldscale;
                }
            }
            for (int s = s_first; s < ph.nseg; s += s_step) {
                const int q = (unit - ph.unit0) * ph.nseg + s;
                const int c0 = s * ph.seg_chunks, nch = min(ph.chunks, c0 + ph.seg_chunks) - c0;
                consume_task<WT, SCALE, PL, PHASE == 2, PHASE == 2>(acc, p, ds, ring, full0, ph.g0 + q * PL, c0, nch, xrow, srow);
            }
            // fp32 sums -> partial[warp][plane][token * 16 + row]; e4m3 fragments hold rows 2g, 2g+1
            const int ra = (WT == kE4M3) ? 2 * gq : gq, rb = (WT == kE4M3) ? 2 * gq + 1 : gq + 8;
#pragma unroll
            for (int pl = 0; pl < PL; ++pl) {
                float* dst = partial + (warp * 2 + pl) * 128;
                dst[(2 * t) * 16 + ra] = acc[pl][0];
                dst[(2 * t + 1) * 16 + ra] = acc[pl][1];
                dst[(2 * t) * 16 + rb] = acc[pl][2];
                dst[(2 * t + 1) * 16 + rb] = acc[pl][3];
            }
        }
        consumer_sync();
        // reduction over the warps of each unit, in warp order
        const int wpu = (ph.nseg >= kConsumers) ? kConsumers : ph.nseg;       // warps per unit
        if constexpr (PHASE == 1) {
            for (int idx = tid; idx < nu * 64; idx += NT) {
                const int uj = idx >> 6, tok = (idx >> 3) & 7, rp = idx & 7;
                const int unit = u + uj, item = unit / groups1, rg = unit - item * groups1;
                if (tok >= ds.item_n[item]) continue;
                float gt0 = 0.f, gt1 = 0.f, up0 = 0.f, up1 = 0.f;
                for (int w = 0; w < wpu; ++w) {
                    const float* src = partial + ((uj * wpu + w) * 2) * 128 + tok * 16 + 2 * rp;
                    gt0 += src[0]; gt1 += src[1];
                    up0 += src[128]; up1 += src[129];
                }
                const float o0 = (gt0 / (1.f + __expf(-gt0))) * up0, o1 = (gt1 / (1.f + __expf(-gt1))) * up1;
                const int slot = ds.item_slot[item][tok];
                *reinterpret_cast<uint32_t*>(p.act + ((size_t)slot * p.I + rg * 16 + 2 * rp) * 2) = pack2<AT>(o0, o1);
            }
        } else {
            for (int idx = tid; idx < nu * 128; idx += NT) {
                const int uj = idx >> 7, tok = (idx >> 4) & 7, row = idx & 15;
                const int item = (u + uj) % n_items;
                if (tok >= ds.item_n[item]) continue;
                float v = 0.f;
                for (int w = 0; w < wpu; ++w) v += partial[((uj * wpu + w) * 2) * 128 + tok * 16 + row];
                const int slot = ds.item_slot[item][tok];
                out_s[slot * 16 + row] = ds.slot_weight[slot] * v;
            }
            if ((u + nu) % n_items == 0) {
                // the tile's last item: every token's rows, in slot order, one rounding
                consumer_sync();
                const int tile = u / n_items;
                for (int idx = tid; idx < p.T * 8; idx += NT) {
                    const int tk = idx >> 3, rp = idx & 7;
                    float s0 = 0.f, s1 = 0.f;
                    for (int j = 0; j < p.topk; ++j) {
                        const int slot = tk * p.topk + j;
                        if (ds.expert_of_slot[slot] < 0) continue;
                        s0 += out_s[slot * 16 + 2 * rp];
                        s1 += out_s[slot * 16 + 2 * rp + 1];
                    }
                    const size_t o = (size_t)tk * p.H + tile * 16 + 2 * rp;
                    if (p.y_fp32) *reinterpret_cast<float2*>(reinterpret_cast<float*>(p.y) + o) = make_float2(s0, s1);
                    else *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(p.y) + o * 2) = pack2<AT>(s0, s1);
                }
            }
        }
        u += nu;
        consumer_sync();      // the partial sums are free for the next round
    }
}

constexpr size_t kDecRingBytes = (size_t)kRing * kSegBytes;
constexpr size_t kDecPartialBytes = kConsumers * 2 * 128 * sizeof(float);
constexpr size_t kDecOutBytes = kDecSlots * 16 * sizeof(float);
constexpr size_t kDecSmem = kDecRingBytes + kDecPartialBytes + kDecOutBytes + kRing * 8;

template <int WT, bool SCALE>
__global__ void __launch_bounds__(kThreads, 1) moe_decode_kernel(const DecodeParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ DecodeShared ds;
    const int tid = threadIdx.x, warp = tid >> 5;
    const uint32_t ring = smem_u32(smem);
    float* partial = reinterpret_cast<float*>(smem + kDecRingBytes);
    float* out_s = reinterpret_cast<float*>(smem + kDecRingBytes + kDecPartialBytes);
    const uint32_t full0 = smem_u32(smem + kDecRingBytes + kDecPartialBytes + kDecOutBytes);
    DecodeSync& sync = g_decode_sync[p.sync_slot];

    if (tid == 0) {
        for (int i = 0; i < kRing; ++i) {
            mbar_init(full0 + 8 * i, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // the routing comes from the preceding kernel of the stream
    MLK_DTL(0, 0);
    pdl_wait();
    pdl_launch_dependents();
    MLK_DTL(1, 0);
    const int32_t* ids = p.topk_ids;
    const void* wts = p.topk_weights;
    if (p.logits != nullptr) {
        // routing fused in front: warp t routes token t (every CTA for itself: a few hundred numbers), scratch in the
        // partial-sum buffer; CTA 0 also hands the routing to the caller
        constexpr int AT = (WT == kFP16) ? kFP16 : kBF16;
        if (warp < p.T) {
            const int lane = tid & 31;
            float* ssel = partial + warp * (p.n_global + 2 * p.n_groups);
            float xl[kVPT];
#pragma unroll
            for (int i = 0; i < kVPT; ++i) {
                const int e = lane + 32 * i;
                xl[i] = (e < p.n_global) ? load_scalar16<AT>(p.logits, (int64_t)warp * p.n_global + e) : -INFINITY;
            }
            route_token<AT>(xl, warp, lane, p.score_fun, p.n_global, p.n_groups, p.topk_groups, ds.route_ids, ds.route_wts, p.topk,
                            p.route_bias, p.renormalize, ssel, ssel + p.n_global, reinterpret_cast<int*>(ssel + p.n_global + p.n_groups));
        }
        __syncthreads();
        if (blockIdx.x == 0 && tid < p.T * p.topk) {
            const_cast<int32_t*>(p.topk_ids)[tid] = ds.route_ids[tid];
            reinterpret_cast<uint16_t*>(const_cast<void*>(p.topk_weights))[tid] = ds.route_wts[tid];
        }
        ids = ds.route_ids;
        wts = ds.route_wts;
    }
    build_items(p, ds, WT == kFP16, ids, wts);          // starts with a CTA-wide barrier: the mbarriers are visible to every role after it
    const int n_items = ds.n_items;

    // both phases as every role sees them
    const long long G = gridDim.x, b = blockIdx.x;
    Phase p1, p2;
    {
        const long long U1 = (long long)n_items * (p.I >> 4);
        p1.unit0 = (int)(U1 * b / G);
        p1.unit1 = (int)(U1 * (b + 1) / G);
        p1.chunks = p.H >> 5;
        split_k<WT, SCALE>(p1.chunks, p1.nseg, p1.seg_chunks);
        p1.upr = (p1.nseg >= kConsumers) ? 1 : kConsumers / p1.nseg;
        p1.planes = 2;
        p1.g0 = 0;
        const long long T2 = p.H >> 4;
        p2.unit0 = (int)(T2 * b / G) * n_items;
        p2.unit1 = (int)(T2 * (b + 1) / G) * n_items;
        p2.chunks = p.I >> 5;
        split_k<WT, SCALE>(p2.chunks, p2.nseg, p2.seg_chunks);
        p2.upr = (p2.nseg >= kConsumers) ? 1 : kConsumers / p2.nseg;
        p2.planes = 1;
        p2.g0 = 2 * (p1.unit1 - p1.unit0) * p1.nseg;
    }

    MLK_DTL(2, 0);
    if (warp == kConsumers) {
        produce<WT>(p, ds, p1, p2, ring, full0);
        if (blockIdx.x == gridDim.x - 1) {
            __syncwarp();
            write_alignment(p, ds);
        }
        MLK_DTL(7, kConsumers * 32);
    } else {
        consume_phase<WT, SCALE, 1>(p, ds, p1, ring, full0, partial, out_s);
        MLK_DTL(3, 0);
        // every CTA's activation rows must be in memory before anyone multiplies them
        consumer_sync();
        if (tid == 0) {
            __threadfence();
            atomicAdd(&sync.barrier, 1u);
            unsigned polls = 0;
            while (ld_acquire_u32(&sync.barrier) < gridDim.x) {
                if (++polls > kDecSpinLimit) {
                    if (p.status != nullptr) atomicCAS(p.status, 0, kDecBarrierExpired);
                    break;
                }
                __nanosleep(20);
            }
            __threadfence();
            // nobody touches the barrier counter after passing it: the last CTA through puts the counters back for the
            // next launch that gets this set
            if (atomicAdd(&sync.done, 1u) == gridDim.x - 1) {
                sync.barrier = 0;
                sync.done = 0;
                __threadfence();
            }
        }
        consumer_sync();
        MLK_DTL(4, 0);
        consume_phase<WT, SCALE, 2>(p, ds, p2, ring, full0, partial, out_s);
        MLK_DTL(5, 0);
        if (n_items == 0) {
            // nothing routed to this rank: y is all zeros (the fp32 form is not zeroed by the caller)
            const int t0 = (int)((long long)(p.H >> 4) * b / G), t1 = (int)((long long)(p.H >> 4) * (b + 1) / G);
            for (int idx = tid; idx < p.T * (t1 - t0) * 16; idx += kConsumers * 32) {
                const int tk = idx / ((t1 - t0) * 16), col = t0 * 16 + idx % ((t1 - t0) * 16);
                if (p.y_fp32) reinterpret_cast<float*>(p.y)[(size_t)tk * p.H + col] = 0.f;
                else reinterpret_cast<uint16_t*>(p.y)[(size_t)tk * p.H + col] = 0;
            }
        }
    }
    __syncthreads();
    MLK_DTL(6, 0);
}

template <int WT, bool SCALE>
int launch_decode_inst(DecodeParams p, cudaStream_t s) {
    auto kern = moe_decode_kernel<WT, SCALE>;
    static bool prepared[64] = {};
    static int pdl_state[64] = {};     // 0 = not tried, 1 = accepted together with the cooperative attribute, -1 = refused
    static std::atomic<unsigned> next_slot{0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!prepared[dev & 63]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDecSmem) != cudaSuccess) {
            cudaGetLastError();
            return fail(kCudaError, "moe decode: %zu bytes of shared memory refused", kDecSmem);
        }
        int occ = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kThreads, kDecSmem) != cudaSuccess || occ < 1) {
            cudaGetLastError();
            return fail(kCudaError, "moe decode: the kernel does not fit an SM");
        }
        prepared[dev & 63] = true;
    }
    // One CTA per SM, all resident together (the launch is cooperative).  A few SMs are left out so that the grid can
    // become resident while the small kernels before it in the stream still hold theirs (programmatic dependent launch).
    const int grid = std::max(1, sm_count() - 4);
    p.sync_slot = (int)(next_slot.fetch_add(1) % kDecPool);

    int& pdl = pdl_state[dev & 63];
    for (int attempt = 0; attempt < 2; ++attempt) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kDecSmem;
        cfg.stream = s;
        cudaLaunchAttribute attr[2];
        int n = 0;
        // all CTAs wait for one another at the grid barrier: the launch must make them resident together
        attr[n].id = cudaLaunchAttributeCooperative;
        attr[n].val.cooperative = 1;
        ++n;
        const bool with_pdl = option(kOptPdl) && pdl >= 0;
        if (with_pdl) {
            attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[n].val.programmaticStreamSerializationAllowed = 1;
            ++n;
        }
        cfg.attrs = attr;
        cfg.numAttrs = n;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
        if (e == cudaSuccess) {
            if (with_pdl) pdl = 1;
            return kOk;
        }
        if (with_pdl && pdl == 0) {
            // the two attributes together were refused: remember it and launch cooperatively only
            cudaGetLastError();
            pdl = -1;
            continue;
        }
        return fail(kCudaError, "moe decode launch: %s", cudaGetErrorString(e));
    }
    return fail(kCudaError, "moe decode launch failed");
}

}  // namespace

bool moe_decode_supported(const MoeParams& m) {
    const long long slots = (long long)m.T * m.topk;
    const bool scale = m.dtype == kE4M3 && m.w1_scale && m.w2_scale;
    const bool routed_ok = m.gating == nullptr ||
                           (m.n_global >= 1 && m.n_global <= 32 * kVPT && m.n_groups >= 1 && m.n_global % m.n_groups == 0 &&
                            m.topk_groups >= 1 && m.topk_groups <= m.n_groups && m.topk <= 32 && m.topk <= m.n_global &&
                            (m.score_fun == 0 || m.score_fun == 1) &&
                            (size_t)m.T * (m.n_global + 2 * m.n_groups) * sizeof(float) <= kDecPartialBytes);
    return m.T >= 1 && m.T <= kDecTokens && slots <= kDecSlots && m.E <= 1024 && m.H % 32 == 0 && m.I % 32 == 0 &&
           (!scale || (m.H % 128 == 0 && m.I % 128 == 0)) && routed_ok;
}

int launch_moe_decode(const MoeParams& m, cudaStream_t s) {
    if (!moe_decode_supported(m)) return fail(kInvalidArg, "moe decode: unsupported call");
    const int wt = m.dtype;
    const int esz = (wt == kE4M3) ? 1 : 2;
    const bool scale = wt == kE4M3 && m.w1_scale && m.w2_scale;
    const int mbs = m.mbs > 0 ? m.mbs : 16;
    DecodeParams p{};
    p.w1 = reinterpret_cast<const uint8_t*>(m.w1);
    p.w2 = reinterpret_cast<const uint8_t*>(m.w2);
    p.w1_expert_bytes = 2LL * m.I * m.H * esz;
    p.w2_expert_bytes = (long long)m.H * m.I * esz;
    p.s1 = m.w1_scale;
    p.s2 = m.w2_scale;
    p.s1_expert = (long long)((2 * m.I + 127) / 128) * ((m.H + 127) / 128);
    p.s2_expert = (long long)((m.H + 127) / 128) * ((m.I + 127) / 128);
    p.x = reinterpret_cast<const uint8_t*>(m.x);
    p.act = reinterpret_cast<uint8_t*>(m.C);
    p.y = m.y;
    p.topk_ids = m.topk_ids;
    p.topk_weights = m.topk_weights;
    p.experts_map = m.experts_map;
    p.map_len = m.experts_map_len;
    p.T = m.T; p.E = m.E; p.topk = m.topk; p.H = m.H; p.I = m.I;
    p.fp8_order = m.fp8_order;
    p.y_fp32 = m.y_fp32;
    p.mbs = mbs;
    p.sorted = m.sorted_token_ids;
    p.cumsum = m.cumsum;
    p.nblocks = m.padded_num_experts;
    p.block_expert = m.experts_ids;
    p.max_padded = m.T * m.topk + m.E * (mbs - 1);
    p.max_blocks = (p.max_padded + mbs - 1) / mbs;
    p.status = m.status;
    p.logits = m.gating;
    p.route_bias = m.gating_bias;
    p.n_global = m.n_global; p.score_fun = m.score_fun; p.n_groups = m.n_groups; p.topk_groups = m.topk_groups;
    p.renormalize = m.renormalize;
    switch (wt) {
        case kBF16: return launch_decode_inst<kBF16, false>(p, s);
        case kFP16: return launch_decode_inst<kFP16, false>(p, s);
        case kE4M3: return scale ? launch_decode_inst<kE4M3, true>(p, s) : launch_decode_inst<kE4M3, false>(p, s);
    }
    return fail(kUnsupported, "moe decode: unknown weight type %d", wt);
}

}  // namespace mlk

#ifdef MLK_DECODE_TIMELINE
extern "C" int mlk_decode_timeline_read(long long* host) {
    return (int)cudaMemcpyFromSymbol(host, mlk::g_dec_timeline, sizeof(long long) * 512 * 16);
}
#endif
