// Narrow GEMM for 16..64 tokens on the 5th-generation tensor cores: C[n,m] = alpha * X[n,k] * A[m,k]^T (+ bias).
//
// "Swap-AB" tile: the 128 weight rows are the UMMA M dimension, the (padded) tokens the N dimension, the fp32
// accumulator [128 x N] lives in tensor memory.  Why the native weight layout fits without any shuffle: one
// layout-A block [16 rows][8 k] is 256 contiguous bytes = two K-major, no-swizzle UMMA core matrices (8 rows x 16
// bytes each).  A 4-D TMA tensor map over global memory (128-byte core matrix, k-octet, row group, half) lands a
// 128 x 64 weight tile in shared memory as [half][row group][k-octet][128 B], which one shared-memory descriptor
// addresses with uniform strides (8-row step 1024 B, k-octet step 128 B); accumulator rows are a fixed permutation
// of the tile's weight rows, undone when the output is written.
// Activations are row-major; a 2-D tensor map with the 128-byte swizzle delivers the [N x 64] tile in the
// canonical K-major SW128 layout (rows beyond n are zero-filled by the TMA unit).
//
// Structure per CTA (192 threads): lane 0 of warp 0 issues TMA loads into a ring of stages, lane 0 of warp 1
// issues tcgen05.mma (4 per stage, K = 16 each) and releases stages with tcgen05.commit, four epilogue warps read
// the accumulator with tcgen05.ld, stage the tile in shared memory and write C with 16-byte stores.  The grid is
// persistent (a multiple of the SM count) and splits the work stream-K fashion; tiles shared by several CTAs are
// combined through an fp32 workspace in a fixed order (no CTA ever waits for another one, bit-reproducible).
// Every wait is bounded: on expiry the kernel records a code in *status, stops, waits (bounded) for its own TMA
// copies, frees its tensor memory and returns.
//
// Role in the reference: the CTA-tile kernel GemmMmaJustLayoutAKernel2 (csrc/gemm_layout_A.cu:296) -- weights and
// tokens staged through shared memory, tile_m in {64,128}, tile_k 128 -- selected by kernelId 2 in the tables.
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "dense.cuh"
#include "status.h"
#include "umma_common.cuh"

namespace mlk {

namespace {

using namespace umma;


struct UmmaParams {
    void* C;
    const void* bias;
    float alpha;
    int m, n, k;
    int c_layout;
    int x_layout;      // 0 row-major activations, 1 layout B
    int kblocks;       // k / 64
    float* ws;         // [tiles][max_parts][NP][128] fp32 partial tiles
    int max_parts;     // workspace slots per tile
    int* counters;     // [tiles], zero between launches
    int* status;       // sticky error word (0 = ok), may be null
};

// ---- kernel ---------------------------------------------------------------------------------------------
//
// Work decomposition ("stream-K"): the unit of work is (128-row tile, 64-wide k block); units are numbered
// tile-major and split into gridDim.x contiguous, equally long ranges, one per CTA, so every SM streams the same
// number of weight bytes whatever the shape.  A CTA's range decomposes into segments (one tile each).  A segment
// that covers all k blocks of its tile is written straight to C.  Otherwise the tile is shared by `parts` CTAs;
// part j = CTA index minus the first CTA that touches the tile, so part 0 owns the head of the k range and is the
// last thing its CTA computes, while the other parts are finished earlier in their CTAs' runs.  Protocol:
//   * a CTA parks its fp32 partial tile in workspace slot (tile, j) and bumps the tile's counter; the CTA that
//     arrives last adds the slots in descending j and writes C (no spinning, bit-reproducible);
//   * shortcut for part 0: while its MMAs are still running, its epilogue warps watch the counter; once all other
//     parts have arrived they are summed (descending j) into registers ahead of time, and when the accumulator is
//     ready the result is own + sum -- the same additions in the same order, without the store / atomic / load
//     round trips at the very end of the kernel, where nothing else hides them.
//
// Warp roles (192 threads): warp 0 lane 0 = TMA producer, warp 1 = tensor-memory owner and (lane 0) MMA issuer,
// warps 2..5 = epilogue (warp w reads TMEM lanes 32*(w%4)...).  Two accumulators in tensor memory alternate
// between segments so the MMAs of the next segment overlap the epilogue of the previous one.
//
// Overlap with the preceding kernel of the stream: under the static-weights promise the producer fills the whole
// ring with weight tiles before it waits for the preceding kernel (griddepcontrol.wait); activations are only
// touched after that wait.  With a ring of at most about 110 KB two consecutive launches are resident on an SM at
// the same time, so this start-up runs under the predecessor's tail.  (Asking L2 to prefetch further ahead with
// cp.async.bulk.prefetch.tensor was measured and made every case slower; it is not used.)

#ifdef MLK_UMMA_TIMELINE
// Developer instrumentation (compiled out by default): per-CTA %globaltimer stamps of the pipeline milestones.
__device__ long long g_timeline[1024 * 16];
#define MLK_TL(slot)                                                                        \
    do {                                                                                    \
        long long t_;                                                                       \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                              \
        const unsigned b_ = blockIdx.x * gridDim.y + blockIdx.y;                            \
        if (b_ < 1024) g_timeline[b_ * 16 + (slot)] = t_;                                   \
    } while (0)
#define MLK_TLV(slot, v) do { const unsigned b_ = blockIdx.x * gridDim.y + blockIdx.y; if (b_ < 1024) g_timeline[b_ * 16 + (slot)] = (v); } while (0)
#else
#define MLK_TL(slot) do { } while (0)
#define MLK_TLV(slot, v) do { } while (0)
#endif

__device__ __forceinline__ int cta_of_unit(long long u, long long U, int G) {
    // the g with floor(U*g/G) <= u < floor(U*(g+1)/G)
    return (int)(((u + 1) * G - 1) / U);
}

__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

constexpr uint32_t kPollLimit = 1u << 22;   // counter polls (64 ns apart) before the early fix-up gives up

// CLUSTER = false: persistent stream-K grid; true: one cluster per tile (gridDim.y = cluster size), which needs none of
// the workspace code paths and so fits two 64-token CTAs per SM.
// (CLUSTER = 2: clusters of up to 16 CTAs, a non-portable size that needs its own kernel attribute; kept apart
// because the attribute and the longer reduction loop cost the ordinary cluster kernel 0.3-1 us per launch)
template <int WT, int NP, int STAGES, int CLUSTER>
__global__ void __launch_bounds__(192, CLUSTER ? 2 : 1) dense_umma_kernel(const __grid_constant__ CUtensorMap map_a,
                                                         const __grid_constant__ CUtensorMap map_x, const UmmaParams p,
                                                         const int static_weights) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int kBBytes = NP * 128;
    constexpr uint32_t kTmemCols = 2 * NP < 32 ? 32 : 2 * NP;
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
    __shared__ uint32_t tmem_slot;
    __shared__ int last_flag;
    __shared__ volatile int ep_mode;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint64_t wpol = l2_evict_first_policy();       // weights are read once: first out of L2
    const int G = gridDim.x, g = blockIdx.x;
    const int KB = p.kblocks;
    const long long U = (long long)(p.m / kTileM) * KB;
    const int SK = CLUSTER ? (int)gridDim.y : 1;   // cluster split-K: blockIdx.x = tile, blockIdx.y = rank in the cluster
    const long long u0 = CLUSTER ? (long long)g * KB + (long long)KB * blockIdx.y / SK : U * g / G;
    const long long u1 = CLUSTER ? (long long)g * KB + (long long)KB * (blockIdx.y + 1) / SK : U * (g + 1) / G;
    if (tid == 0) MLK_TL(0);

    // 1024-byte aligned operand ring (all A stages, then all B stages), then the output staging tile
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_base = base, b_base = base + STAGES * kABytes;
    uint8_t* const out_stage = smem_raw + (base - smem_u32(smem_raw)) + STAGES * (kABytes + kBBytes);
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto acc_full = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
    auto acc_empty = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 4);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    if (tid == 0) MLK_TL(1);

    int issued = 0;
    if (warp == 0 && lane == 0) {
        // ---- TMA producer: one stage per unit, running ahead of the MMAs by up to STAGES units ----
        // (tile, k block) advance by increment: a 64-bit division per stage in this single thread would cost more
        // than the stage's memory time.
        const int tile0 = (int)(u0 / KB), kb0 = (int)(u0 - (long long)tile0 * KB);
        const int nunits = (int)(u1 - u0);
        int lt = tile0, lk = kb0;     // next unit whose weights are loaded
        auto load_a = [&](int s) {
            tma_load_4d_hint(a_base + s * kABytes, &map_a, full_bar(s), 0, lk * (kBlockK / 8), lt * (kTileM / 16), 0, wpol);
        };
        int i = 0;
        if (static_weights) {
            // weights may stream before the preceding kernel has finished; activations never do
            pdl_launch_dependents();
            const int pre = nunits < STAGES ? nunits : STAGES;
            for (; i < pre; ++i) {
                mbar_expect_tx(full_bar(i), kABytes + kBBytes);
                load_a(i);
                if (++lk == KB) { lk = 0; ++lt; }
            }
            pdl_wait();
            int bk = kb0;
            for (int j = 0; j < pre; ++j) {
                if (p.x_layout == 0) tma_load_2d(b_base + j * kBBytes, &map_x, full_bar(j), bk * kBlockK, 0);
                else tma_load_5d(b_base + j * kBBytes, &map_x, full_bar(j), 0, 0, 0, 0, bk * (kBlockK / 32));
                if (++bk == KB) bk = 0;
            }
            issued = pre;
            MLK_TL(2);
        } else {
            pdl_wait();
            pdl_launch_dependents();
        }
        for (; i < nunits; ++i) {
            const int s = i % STAGES;
            if (i >= STAGES && !mbar_wait(empty_bar(s), ((i / STAGES) - 1) & 1)) {
                abort_flag = 1;
                if (p.status) atomicExch(p.status, 1);
            }
            if (abort_flag) break;
            mbar_expect_tx(full_bar(s), kABytes + kBBytes);
            load_a(s);
            if (p.x_layout == 0) tma_load_2d(b_base + s * kBBytes, &map_x, full_bar(s), lk * kBlockK, 0);
            else tma_load_5d(b_base + s * kBBytes, &map_x, full_bar(s), 0, 0, 0, 0, lk * (kBlockK / 32));
            if (++lk == KB) { lk = 0; ++lt; }
            ++issued;
        }
        MLK_TL(3);
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        // Its bounded waits must not start counting while the producer still waits for the preceding kernel of the
        // stream (the token tiles are only requested after that): wait for it here as well.
        pdl_wait();
        constexpr uint32_t idesc = instr_desc<WT, NP>();
        int i = 0, seg = 0;
        for (long long u = u0; u < u1 && !abort_flag; ++seg) {
            const int tile = (int)(u / KB), kb_begin = (int)(u - (long long)tile * KB);
            const int kb_end = (int)min((long long)KB, kb_begin + (u1 - u));
            const int b = seg & 1;
            if (seg >= 2 && !mbar_wait(acc_empty(b), ((seg >> 1) - 1) & 1)) {
                abort_flag = 1;
                if (p.status) atomicExch(p.status, 4);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int kb = kb_begin; kb < kb_end; ++kb, ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(full_bar(s), (i / STAGES) & 1)) {
                    abort_flag = 1;
                    if (p.status) atomicExch(p.status, 2);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int kk = 0; kk < kBlockK / 16; ++kk) {
                    // A: no swizzle, [half][row group][k-octet][8 rows x 16 B]: 8-row step 1024 B, k-octet step 128 B;
                    // one MMA consumes two k-octets
                    const uint64_t da = smem_desc(a_base + s * kABytes + kk * 256, 128, 1024, 0);
                    // B: 128-byte swizzle, 8-token step 1024 B; one MMA consumes 32 bytes of each 128-byte row
                    // (layout-B activations: no swizzle, k-octet step NP * 16 bytes, 8-token step 128 bytes)
                    const uint64_t db = p.x_layout == 0 ? smem_desc(b_base + s * kBBytes + kk * 32, 16, 1024, 2)
                                                        : smem_desc(b_base + s * kBBytes + kk * (NP * 32), NP * 16, 128, 0);
                    umma_f16(tmem + b * NP, da, db, idesc, (kb > kb_begin || kk > 0) ? 1u : 0u);
                }
                umma_commit(empty_bar(s));     // arrives when the MMAs above have finished reading the stage
            }
            if (abort_flag) break;
            umma_commit(acc_full(b));          // arrives when this segment's accumulation is complete
            u += kb_end - kb_begin;
        }
        MLK_TL(4);
    } else if (warp >= 2) {
        // ---- epilogue warps ----
        const int quad = warp & 3;
        const int lrow = quad * 32 + lane;          // accumulator row = TMEM lane
        // accumulator row rho holds weight row 16*(rho%64 / 8) + 8*(rho / 64) + rho%8 of the tile (see make_map_a16)
        const int wrow = ((lrow & 63) >> 3) * 16 + (lrow >> 6) * 8 + (lrow & 7);
        const int etid = tid - 64;
        const size_t part_elems = (size_t)NP * kTileM;
        // counters and workspace belong to the preceding kernel of the stream until it has finished, and the bounded
        // waits below must not run out while that kernel is still at work
        pdl_wait();
        if constexpr (CLUSTER) {
            // cluster split-K: park the fp32 partial tile [token][accumulator row] in this CTA's (now idle) ring
            if (lane == 0 && !mbar_wait(acc_full(0), 0)) {
                abort_flag = 1;
                if (p.status) atomicExch(p.status, 3);
            }
            __syncwarp();
            if (!abort_flag) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                float* const red = reinterpret_cast<float*>(smem_raw + (base - smem_u32(smem_raw)));
#pragma unroll
                for (int c0 = 0; c0 < NP; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld16(tmem + ((uint32_t)(quad * 32) << 16) + c0, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 16; ++i) red[(c0 + i) * kTileM + lrow] = __uint_as_float(r[i]);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
        }
        int seg = 0;
        for (long long u = u0; u < u1 && !CLUSTER; ++seg) {
            const int tile = (int)(u / KB), kb_begin = (int)(u - (long long)tile * KB);
            const int kb_end = (int)min((long long)KB, kb_begin + (u1 - u));
            const int b = seg & 1;
            const uint32_t acc_parity = (seg >> 1) & 1;
            const uint32_t tacc = tmem + ((uint32_t)(quad * 32) << 16) + b * NP;
            const bool partial = !(kb_begin == 0 && kb_end == KB);
            int parts = 1, part = 0;
            if (partial) {
                const int g_first = cta_of_unit((long long)tile * KB, U, G);
                parts = cta_of_unit((long long)(tile + 1) * KB - 1, U, G) - g_first + 1;
                part = g - g_first;
            }
            float* const ws_tile = p.ws + (size_t)tile * p.max_parts * part_elems + lrow;

            // ---- part 0: look for the other parts while the MMAs are still running ----
            bool early = false;
            float hi[NP];
            if (partial && part == 0) {
                if (etid == 0) {
                    int mode = 0;                     // 0 = accumulator came first, 1 = other parts are all there
                    for (uint32_t it = 0;; ++it) {
                        if (abort_flag || mbar_test_wait(acc_full(b), acc_parity)) break;
                        if (ld_acquire(p.counters + tile) == parts - 1) { mode = 1; break; }
                        if (it >= kPollLimit) {
                            abort_flag = 1;
                            if (p.status) atomicExch(p.status, 5);
                            break;
                        }
                        __nanosleep(64);
                    }
                    ep_mode = mode;
                }
                epi_bar();
                early = ep_mode == 1;
                epi_bar();                            // ep_mode is rewritten below
                if (early) {
                    __threadfence();
                    // descending j, all loads of a part in flight together
#pragma unroll
                    for (int c = 0; c < NP; ++c) hi[c] = __ldcg(ws_tile + (size_t)(parts - 1) * part_elems + (size_t)c * kTileM);
                    for (int j = parts - 2; j >= 1; --j) {
                        float t[NP];
#pragma unroll
                        for (int c = 0; c < NP; ++c) t[c] = __ldcg(ws_tile + (size_t)j * part_elems + (size_t)c * kTileM);
#pragma unroll
                        for (int c = 0; c < NP; ++c) hi[c] += t[c];
                    }
                }
            }

            // ---- wait for the accumulator; the four warps leave together (they share named barrier 1) ----
            if (lane == 0 && !abort_flag && !mbar_wait(acc_full(b), acc_parity)) {
                abort_flag = 1;
                if (p.status) atomicExch(p.status, 3);
            }
            epi_bar();
            if (etid == 0) ep_mode = abort_flag ? 2 : 0;
            epi_bar();
            if (ep_mode == 2) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (etid == 0) { MLK_TL(7); MLK_TLV(9, (long long)(!partial ? 0 : (early ? 1 : 2)) + 10 * parts + 100 * part); }

            // emits 16 finished columns (tokens c0 .. c0+15) of this thread's accumulator row
            const int row = tile * kTileM + wrow;
            const float bia = (p.bias != nullptr) ? load_scalar16<WT>(p.bias, row) : 0.f;
            auto emit16 = [&](int c0, const float (&o)[16]) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int c = c0 + i;
                    const float val = fmaf(p.alpha, o[i], bia);
                    if (p.c_layout == 0) {
                        if constexpr (WT == kFP16)
                            reinterpret_cast<__half*>(out_stage)[c * kTileM + wrow] = __float2half_rn(val);
                        else
                            reinterpret_cast<__nv_bfloat16*>(out_stage)[c * kTileM + wrow] = __float2bfloat16_rn(val);
                    } else if (c < p.n) {
                        const int NB = p.n >> 4;
                        const size_t idx = ((((size_t)(row >> 5) * NB + (c >> 4)) * 4 + ((row >> 3) & 3)) * 16 + (c & 15)) * 8 + (row & 7);
                        if constexpr (WT == kFP16)
                            reinterpret_cast<__half*>(p.C)[idx] = __float2half_rn(val);
                        else
                            reinterpret_cast<__nv_bfloat16*>(p.C)[idx] = __float2bfloat16_rn(val);
                    }
                }
            };
            auto load_acc16 = [&](int c0, float (&o)[16]) {
                uint32_t r[16];
                tmem_ld16(tacc + c0, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; ++i) o[i] = __uint_as_float(r[i]);
            };
            auto release_acc = [&]() {
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(b)) : "memory");
            };

            bool wrote = true;
            if (!partial) {
#pragma unroll
                for (int c0 = 0; c0 < NP; c0 += 16) {
                    float o[16];
                    load_acc16(c0, o);
                    emit16(c0, o);
                }
                release_acc();
            } else if (early) {
#pragma unroll
                for (int c0 = 0; c0 < NP; c0 += 16) {
                    float o[16];
                    load_acc16(c0, o);
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = hi[c0 + i] + o[i];    // part 0 is the last addend
                    emit16(c0, o);
                }
                release_acc();
                if (etid == 0) p.counters[tile] = 0;   // ready for the next launch
            } else {
                // park this part
                float* const mine = ws_tile + (size_t)part * part_elems;
#pragma unroll
                for (int c0 = 0; c0 < NP; c0 += 16) {
                    float o[16];
                    load_acc16(c0, o);
#pragma unroll
                    for (int i = 0; i < 16; ++i) __stcg(mine + (size_t)(c0 + i) * kTileM, o[i]);
                }
                release_acc();
                __threadfence();
                epi_bar();
                if (etid == 0) last_flag = (atomicAdd(p.counters + tile, 1) == parts - 1) ? 1 : 0;
                epi_bar();
                wrote = last_flag != 0;          // the last arriver adds all parts in descending order
                if (wrote) {
                    __threadfence();
                    // 64 loads in flight per thread (whole parts); the adds keep descending part order
                    constexpr int UN = 64 / NP;
                    float acc[NP];
                    for (int jb = parts - 1; jb >= 0; jb -= UN) {
                        float t[UN][NP];
#pragma unroll
                        for (int jj = 0; jj < UN; ++jj)
#pragma unroll
                            for (int c = 0; c < NP; ++c)
                                t[jj][c] = (jb - jj >= 0) ? __ldcg(ws_tile + (size_t)(jb - jj) * part_elems + (size_t)c * kTileM) : 0.f;
#pragma unroll
                        for (int jj = 0; jj < UN; ++jj)
#pragma unroll
                            for (int c = 0; c < NP; ++c) {
                                if (jb == parts - 1 && jj == 0) acc[c] = t[0][c];
                                else if (jb - jj >= 0) acc[c] += t[jj][c];
                            }
                    }
#pragma unroll
                    for (int c0 = 0; c0 < NP; c0 += 16) {
                        float o[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = acc[c0 + i];
                        emit16(c0, o);
                    }
                    if (etid == 0) p.counters[tile] = 0;   // ready for the next launch
                }
                epi_bar();                               // last_flag may be rewritten by the next segment
            }

            if (etid == 0) { MLK_TL(8); MLK_TLV(10, (long long)wrote); }
            if (p.c_layout == 0) {
                // staged tile [token][128 rows] -> C[token][tile rows]: 256 contiguous bytes per token
                epi_bar();
                if (wrote) {
                    uint8_t* const cbase = reinterpret_cast<uint8_t*>(p.C) + (size_t)tile * kTileM * 2;
                    for (int idx = etid; idx < p.n * 16; idx += 128) {
                        const int c = idx >> 4, ch = idx & 15;
                        const uint4 val = *reinterpret_cast<const uint4*>(out_stage + c * (kTileM * 2) + ch * 16);
                        *reinterpret_cast<uint4*>(cbase + (size_t)c * p.m * 2 + ch * 16) = val;
                    }
                }
                epi_bar();                               // the staging tile is reused by the next segment
            }
            u += kb_end - kb_begin;
        }
        if (etid == 0) MLK_TL(5);
    }
    __syncwarp();

    if constexpr (CLUSTER) {
        // ---- cluster split-K: every CTA of the cluster adds one slice of accumulator rows over all ranks
        // (descending rank, fixed order) through distributed shared memory and writes that slice of C ----
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (warp >= 2) {
            const int etid = tid - 64;
            const int rank = blockIdx.y;
            if constexpr (CLUSTER == 2) {
                // clusters of up to 16 CTAs: one accumulator row per thread and step (the 16-byte form below would hold
                // 64 partial sums per thread and cost this kernel a resident CTA per SM)
                const int r0 = kTileM * rank / SK, rows = kTileM * (rank + 1) / SK - r0;
                constexpr int kMaxSK = CLUSTER == 2 ? 16 : 8;
                uint32_t remote[kMaxSK];
#pragma unroll
                for (int q = 0; q < kMaxSK; ++q)
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[q]) : "r"(base), "r"(q < SK ? q : 0));
                const int total = p.n * rows;
                for (int idx = etid; idx < total; idx += 128) {
                    const int c = idx / rows, rho = r0 + idx - c * rows;
                    const uint32_t off = (uint32_t)(c * kTileM + rho) * 4u;
                    float t[kMaxSK];
#pragma unroll
                    for (int q = 0; q < kMaxSK; ++q) {
                        t[q] = 0.f;
                        if (q < SK) asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(t[q]) : "r"(remote[q] + off) : "memory");
                    }
                    float acc = 0.f;
                    bool first = true;
#pragma unroll
                    for (int q = kMaxSK - 1; q >= 0; --q) {
                        if (q < SK) {
                            acc = first ? t[q] : acc + t[q];
                            first = false;
                        }
                    }
                    const int row = g * kTileM + ((rho & 63) >> 3) * 16 + (rho >> 6) * 8 + (rho & 7);
                    const float bia = (p.bias != nullptr) ? load_scalar16<WT>(p.bias, row) : 0.f;
                    const float val = fmaf(p.alpha, acc, bia);
                    size_t o;
                    if (p.c_layout == 0) {
                        o = (size_t)c * p.m + row;
                    } else {
                        const int NB = p.n >> 4;
                        o = ((((size_t)(row >> 5) * NB + (c >> 4)) * 4 + ((row >> 3) & 3)) * 16 + (c & 15)) * 8 + (row & 7);
                    }
                    if constexpr (WT == kFP16)
                        reinterpret_cast<__half*>(p.C)[o] = __float2half_rn(val);
                    else
                        reinterpret_cast<__nv_bfloat16*>(p.C)[o] = __float2bfloat16_rn(val);
                }
            } else {
                // slices in units of four accumulator rows: one 16-byte distributed-shared-memory load per rank brings four
                // rows of one token, which are four consecutive weight rows (and output elements)
                const int q0 = (kTileM / 4) * rank / SK, quads = (kTileM / 4) * (rank + 1) / SK - q0;
                constexpr int kMaxSK = CLUSTER == 2 ? 16 : 8;
                uint32_t remote[kMaxSK];
#pragma unroll
                for (int q = 0; q < kMaxSK; ++q)
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[q]) : "r"(base), "r"(q < SK ? q : 0));
                const int total = p.n * quads;
                for (int idx = etid; idx < total; idx += 128) {
                    const int c = idx / quads, rho = 4 * (q0 + idx - c * quads);
                    const uint32_t off = (uint32_t)(c * kTileM + rho) * 4u;
                    float4 t[kMaxSK];
#pragma unroll
                    for (int q = 0; q < kMaxSK; ++q) {
                        t[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (q < SK)
                            asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                         : "=f"(t[q].x), "=f"(t[q].y), "=f"(t[q].z), "=f"(t[q].w)
                                         : "r"(remote[q] + off)
                                         : "memory");
                    }
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                    bool first = true;
#pragma unroll
                    for (int q = kMaxSK - 1; q >= 0; --q) {
                        if (q < SK) {
                            acc = first ? t[q] : make_float4(acc.x + t[q].x, acc.y + t[q].y, acc.z + t[q].z, acc.w + t[q].w);
                            first = false;
                        }
                    }
                    const int row = g * kTileM + ((rho & 63) >> 3) * 16 + (rho >> 6) * 8 + (rho & 7);
                    float4 bia = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (p.bias != nullptr)
                        bia = make_float4(load_scalar16<WT>(p.bias, row), load_scalar16<WT>(p.bias, row + 1),
                                          load_scalar16<WT>(p.bias, row + 2), load_scalar16<WT>(p.bias, row + 3));
                    size_t o;
                    if (p.c_layout == 0) {
                        o = (size_t)c * p.m + row;
                    } else {
                        const int NB = p.n >> 4;
                        o = ((((size_t)(row >> 5) * NB + (c >> 4)) * 4 + ((row >> 3) & 3)) * 16 + (c & 15)) * 8 + (row & 7);
                    }
                    // four consecutive 16-bit outputs, 8-byte aligned (row is a multiple of 4, m a multiple of 128)
                    uint2 packed;
                    packed.x = pack2<WT>(fmaf(p.alpha, acc.x, bia.x), fmaf(p.alpha, acc.y, bia.y));
                    packed.y = pack2<WT>(fmaf(p.alpha, acc.z, bia.z), fmaf(p.alpha, acc.w, bia.w));
                    *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.C) + o) = packed;
                }
            }
            if (etid == 0) MLK_TL(5);
        }
        // nobody leaves while its shared memory may still be read
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    }

    // ---- teardown ----
    // If the pipeline stopped early, wait (bounded) until every TMA copy this CTA issued has landed, so that no
    // copy is in flight into shared memory when the CTA exits.
    if (warp == 0 && lane == 0 && abort_flag) {
        for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(full_bar(i % STAGES), (i / STAGES) & 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
    if (tid == 0) MLK_TL(6);
}

// ---- host ------------------------------------------------------------------------------------------------

template <int WT, int NP, int CLUSTER>
const void* kernel_for_stages(int stages) {
    switch (stages) {
        case 2: return reinterpret_cast<const void*>(dense_umma_kernel<WT, NP, 2, CLUSTER>);
        case 3: return reinterpret_cast<const void*>(dense_umma_kernel<WT, NP, 3, CLUSTER>);
        case 4: return reinterpret_cast<const void*>(dense_umma_kernel<WT, NP, 4, CLUSTER>);
        case 5: return reinterpret_cast<const void*>(dense_umma_kernel<WT, NP, 5, CLUSTER>);
        case 6: return reinterpret_cast<const void*>(dense_umma_kernel<WT, NP, 6, CLUSTER>);
        case 8: return reinterpret_cast<const void*>(dense_umma_kernel<WT, NP, 8, CLUSTER>);
    }
    return nullptr;
}

template <int WT, int CLUSTER>
const void* kernel_for(int np, int stages) {
    switch (np) {
        case 16: return kernel_for_stages<WT, 16, CLUSTER>(stages);
        case 32: return kernel_for_stages<WT, 32, CLUSTER>(stages);
        case 64: return kernel_for_stages<WT, 64, CLUSTER>(stages);
    }
    return nullptr;
}

// ring + (stream-K only) the output staging tile + alignment slack; the cluster mode parks its fp32 partial tile
// (np * 512 bytes) in the idle ring, which two stages always cover
size_t smem_bytes(int np, int stages, bool clustered) {
    return (size_t)stages * (kABytes + np * 128) + (clustered ? 0 : (size_t)np * kTileM * 2) + 1024;
}

}  // namespace

// Workspace slots per tile needed when tiles * kblocks work units are split over G CTAs.
int umma_max_parts(int tiles, int kblocks, int G) {
    const long long U = (long long)tiles * kblocks;
    int mx = 1;
    for (int t = 0; t < tiles; ++t) {
        const int gf = (int)((((long long)t * kblocks + 1) * G - 1) / U);
        const int gl = (int)((((long long)(t + 1) * kblocks) * G - 1) / U);
        mx = gl - gf + 1 > mx ? gl - gf + 1 : mx;
    }
    return mx;
}

// ctas_per_sm: resident CTAs per SM the grid is sized for (grid = ctas_per_sm * SM count, capped by the number of
// work units); stages: ring depth (2, 3, 4, 5, 6 or 8; a ring of at most about 110 KB lets two launches share an
// SM); cluster_k: 0 or 1 = the persistent stream-K grid described above, 2..16 = one thread-block cluster of that
// many CTAs per 128-row tile, each CTA taking an equal share of k, partial tiles added through distributed shared
// memory (no workspace; meant for shapes with few tiles and a long k, where stream-K would share every tile among
// many CTAs that all finish at the same moment).
int launch_dense_umma(int wt, const DenseParams& p, int ctas_per_sm, int stages, int cluster_k, const DenseAux* aux,
                      cudaStream_t stream) {
    if (wt != kBF16 && wt != kFP16) return fail(kUnsupported, "dense (tcgen05): 16-bit weights only");
    if (!p.A || !p.X || !p.C) return fail(kInvalidArg, "dense: null pointer");
    if (p.x_layout == 1 && p.n % 16 != 0) return fail(kInvalidArg, "dense: layout B needs n %% 16 == 0");
    if (p.m % kTileM != 0 || p.k % kBlockK != 0) return fail(kInvalidArg, "dense (tcgen05): need m %% 128 == 0 and k %% 64 == 0");
    if (p.n < 1 || p.n > 64) return fail(kUnsupported, "dense (tcgen05): 1..64 tokens per launch (got %d)", p.n);
    if (p.c_layout == 1 && p.n % 16 != 0) return fail(kInvalidArg, "dense: layout C needs n %% 16 == 0");
    if (((uintptr_t)p.A & 15) || ((uintptr_t)p.X & 15) || ((uintptr_t)p.C & 15))
        return fail(kInvalidArg, "dense (tcgen05): A, B and C must be 16-byte aligned");
    if (encode_fn() == nullptr) return fail(kUnsupported, "dense (tcgen05): cuTensorMapEncodeTiled is not available");
    if (ctas_per_sm < 1 || ctas_per_sm > 4) return fail(kInvalidArg, "dense (tcgen05): CTAs per SM must be 1..4 (got %d)", ctas_per_sm);
    const int np = p.n <= 16 ? 16 : (p.n <= 32 ? 32 : 64);
    const int tiles = p.m / kTileM;
    const int kblocks = p.k / kBlockK;
    if (cluster_k < 0 || cluster_k > 16) return fail(kInvalidArg, "dense (tcgen05): cluster split must be 0..16 (got %d)", cluster_k);
    const bool clustered = cluster_k > 1;
    const void* kern = cluster_k > 8 ? (wt == kFP16 ? kernel_for<kFP16, 2>(np, stages) : kernel_for<kBF16, 2>(np, stages))
                       : clustered   ? (wt == kFP16 ? kernel_for<kFP16, 1>(np, stages) : kernel_for<kBF16, 1>(np, stages))
                                     : (wt == kFP16 ? kernel_for<kFP16, 0>(np, stages) : kernel_for<kBF16, 0>(np, stages));
    if (kern == nullptr) return fail(kInvalidArg, "dense (tcgen05): stages must be one of 2, 3, 4, 5, 6, 8 (got %d)", stages);
    int resident = 0;
    const size_t smem = prepare_kernel(kern, 192, smem_bytes(np, stages, clustered), 2 * np < 32 ? 32 : 2 * np, cluster_k > 8, &resident);
    if (smem == 0 || resident < 1) return fail(kCudaError, "dense (tcgen05): a CTA with %d stages does not fit on this device", stages);
    if (ctas_per_sm > resident) ctas_per_sm = resident;
    if (clustered && cluster_k > p.k / kBlockK) return fail(kInvalidArg, "dense (tcgen05): cluster split %d exceeds the %d k blocks", cluster_k, p.k / kBlockK);
    long long G = (long long)sm_count() * ctas_per_sm;
    const long long U = (long long)tiles * kblocks;
    if (G > U) G = U;
    // Without scratch only whole tiles can be handed out: one CTA per tile.
    const bool have_aux = aux && aux->workspace && aux->counters;
    if (!have_aux || clustered) G = tiles;
    const int max_parts = umma_max_parts(tiles, kblocks, (int)G);
    if (have_aux && max_parts > 1) {
        const long long need = (long long)tiles * max_parts * np * kTileM * 4;
        if (aux->workspace_bytes < need)
            return fail(kInvalidArg, "dense (tcgen05): workspace holds %lld bytes, needs %lld", (long long)aux->workspace_bytes, need);
        if (aux->n_counters < tiles) return fail(kInvalidArg, "dense (tcgen05): %d counters, needs %d", aux->n_counters, tiles);
    }
    CUtensorMap ma, mx;
    if (!make_map_a16(&ma, p.A, p.m, p.k, wt)) return fail(kUnsupported, "dense (tcgen05): weight tensor map rejected");
    if (!(p.x_layout == 0 ? make_map_x(&mx, p.X, p.n, p.k, wt, np) : make_map_xb(&mx, p.X, p.n, p.k, wt, np))) return fail(kUnsupported, "dense (tcgen05): activation tensor map rejected");
    UmmaParams up{};
    up.x_layout = p.x_layout;
    up.C = p.C; up.bias = p.bias; up.alpha = p.alpha; up.m = p.m; up.n = p.n; up.k = p.k; up.c_layout = p.c_layout;
    up.kblocks = kblocks;
    up.ws = have_aux ? reinterpret_cast<float*>(aux->workspace) : nullptr;
    up.max_parts = max_parts;
    up.counters = have_aux ? aux->counters : nullptr;
    up.status = aux ? aux->status : nullptr;
    int static_weights = option(kOptStaticWeights);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)G, clustered ? cluster_k : 1, 1);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = launch_attrs(attr, clustered ? cluster_k : 1);
    void* args[4] = {&ma, &mx, &up, &static_weights};
    const cudaError_t e = cudaLaunchKernelExC(&cfg, kern, args);
    if (e != cudaSuccess) return fail(kCudaError, "dense_umma launch: %s", cudaGetErrorString(e));
    return kOk;
}

// Upper bound of the workspace launch_dense_umma can need for this shape on a device with `sms` SMs.
long long umma_workspace_bytes(int m, int n, int k, int sms, int ctas_per_sm) {
    const int np = n <= 16 ? 16 : (n <= 32 ? 32 : 64);
    const int tiles = m / kTileM, kblocks = k / kBlockK;
    long long G = (long long)sms * ctas_per_sm;
    if (G > (long long)tiles * kblocks) G = (long long)tiles * kblocks;
    return (long long)tiles * umma_max_parts(tiles, kblocks, (int)G) * np * kTileM * 4;
}

}  // namespace mlk

#ifdef MLK_UMMA_TIMELINE
extern "C" int mlk_umma_timeline_read(long long* host) {
    return (int)cudaMemcpyFromSymbol(host, mlk::g_timeline, sizeof(long long) * 1024 * 16);
}
#endif
