// Fused-MoE expert GEMMs on the 5th-generation tensor cores (16..128 slots per work item; 16..64 with e4m3 weights).
//
// Same tile and pipeline as dense_umma.cu in cluster mode: 128 weight rows are the UMMA M dimension, the slots of one
// work item (one expert, up to 128 of its routed slots) the N dimension, TMA feeds a shared-memory ring, one thread
// issues tcgen05.mma into tensor memory, the k range is split over the CTAs of a cluster and the partial tiles are
// added through distributed shared memory in a fixed order.  What is specific to the MoE:
//   * the grid is (row tiles, cluster, work items); the work list is the one the alignment kernel writes, items past
//     its length leave at once;
//   * the weight tensor map covers all experts ([E * rows, k]); the item's expert selects the tile rows;
//   * the activation rows of an item must be contiguous for the TMA tile, so a gather pass first copies the routed
//     token rows into compact position order (the routed slots numbered expert by expert, without the padding of
//     sorted_token_ids; the work item carries its first compact position);
//   * MODE 1 (first GEMM): every CTA holds the gate tile and the matching up tile of W1 (two accumulators fed by the
//     same token tile) and writes silu(gate) * up of the fp32 sums as the [position, I] activation;
//   * MODE 2 (second GEMM): reads that activation by position, multiplies by the slot's routing weight and writes the
//     fp32 row of the slot into the combine scratch (the fixed-order combine kernel adds a token's top-k rows).
// Slots beyond the item's count inside the 16/32/64-wide tile belong to other items: they are computed and dropped.
//
// Role in the reference: fused_moe_first/second_group_gemm_kernel (csrc/moe_kernels/group_gemm_first.h:355,
// group_gemm_second.h:356) for the token counts where its CTA-tile kernels are used.
#include <algorithm>

#include "moe.cuh"
#include "moe_umma.cuh"
#include "umma_common.cuh"

namespace mlk {

namespace {

using namespace umma;

template <int WT, int NP, int STAGES, int MODE>
__global__ void __launch_bounds__(192, 2) moe_umma_kernel(const __grid_constant__ CUtensorMap map_a,
                                                          const __grid_constant__ CUtensorMap map_x,
                                                          const MoeUmmaParams p, const int static_weights) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int NA = MODE == 1 ? 2 : 1;               // weight tiles (and accumulators) per CTA
    constexpr int kBBytes = NP * 128;
    constexpr int kStageBytes = NA * kABytes + kBBytes;
    constexpr uint32_t kTmemCols = NA * NP < 32 ? 32 : NA * NP;
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint64_t wpol = l2_evict_first_policy();       // weights are read once: first out of L2
    const int tile = blockIdx.x, rank = blockIdx.y, SK = gridDim.y;

    // the work list comes from the alignment kernel earlier in the stream: nothing can start before it
    pdl_wait();
    pdl_launch_dependents();
    // both loads go out together (the list holds an entry for every z of the grid, live or not)
    const int n_items = p.worklist[0].x;
    const int4 item = p.worklist[1 + blockIdx.z];
    if ((int)blockIdx.z >= n_items) return;             // uniform over the cluster (clusters span y only)
    const int expert = item.x, pos0 = item.y, nslots = item.z, cpos0 = item.w;

    const int KB = p.kblocks;
    const int kb0 = (int)((long long)KB * rank / SK), kb1 = (int)((long long)KB * (rank + 1) / SK);
    const int nunits = kb1 - kb0;
    const int a_tile = expert * p.tiles_per_expert + tile;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
    const uint32_t acc_full = bar0 + 8u * (2 * STAGES);
    auto a_addr = [&](int s, int which) { return base + s * kStageBytes + which * kABytes; };
    auto b_addr = [&](int s) { return base + s * kStageBytes + NA * kABytes; };

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(acc_full, 1);
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

    int issued = 0;
    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        for (int i = 0; i < nunits; ++i) {
            const int s = i % STAGES;
            if (i >= STAGES && !mbar_wait(empty_bar(s), ((i / STAGES) - 1) & 1)) {
                abort_flag = 1;
                if (p.status) atomicExch(p.status, 1);
            }
            if (abort_flag) break;
            mbar_expect_tx(full_bar(s), kStageBytes);
            tma_load_4d_hint(a_addr(s, 0), &map_a, full_bar(s), 0, (kb0 + i) * (kBlockK / 8), a_tile * (kTileM / 16), 0, wpol);
            if constexpr (MODE == 1)
                tma_load_4d_hint(a_addr(s, 1), &map_a, full_bar(s), 0, (kb0 + i) * (kBlockK / 8),
                            (a_tile + p.up_tile_offset) * (kTileM / 16), 0, wpol);
            tma_load_2d(b_addr(s), &map_x, full_bar(s), (kb0 + i) * kBlockK, cpos0);
            ++issued;
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        constexpr uint32_t idesc = instr_desc<WT, NP>();
        for (int i = 0; i < nunits; ++i) {
            const int s = i % STAGES;
            if (abort_flag || !mbar_wait(full_bar(s), (i / STAGES) & 1)) {
                if (!abort_flag && p.status) atomicExch(p.status, 2);
                abort_flag = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kk = 0; kk < kBlockK / 16; ++kk) {
                const uint64_t db = smem_desc(b_addr(s) + kk * 32, 16, 1024, 2);
#pragma unroll
                for (int w = 0; w < NA; ++w) {
                    const uint64_t da = smem_desc(a_addr(s, w) + kk * 256, 128, 1024, 0);
                    umma_f16(tmem + w * NP, da, db, idesc, (i > 0 || kk > 0) ? 1u : 0u);
                }
            }
            umma_commit(empty_bar(s));
        }
        if (!abort_flag) umma_commit(acc_full);
    } else if (warp >= 2) {
        // ---- epilogue warps: accumulators -> fp32 partial tiles [which][slot][accumulator row] in the idle ring ----
        if (lane == 0 && (abort_flag || !mbar_wait(acc_full, 0))) {
            if (!abort_flag && p.status) atomicExch(p.status, 3);
            abort_flag = 1;
        }
        __syncwarp();
    }
    __syncwarp();

    // Epilogue in chunks of at most 64 slots, so that the partial tiles [which][slot][accumulator row] of a chunk fit
    // in the idle ring even for 128-slot work items.
    constexpr int CHUNK = NP > 64 ? 64 : NP;
#pragma unroll 1
    for (int cb = 0; cb < NP; cb += CHUNK) {
        if (warp >= 2 && !abort_flag) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int quad = warp & 3, lrow = quad * 32 + lane;
            float* const red = reinterpret_cast<float*>(base_ptr);
#pragma unroll
            for (int w = 0; w < NA; ++w)
#pragma unroll
                for (int c0 = 0; c0 < CHUNK; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld16(tmem + ((uint32_t)(quad * 32) << 16) + w * NP + cb + c0, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 16; ++i) red[(w * CHUNK + c0 + i) * kTileM + lrow] = __uint_as_float(r[i]);
                }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
        __syncwarp();
        const int left = nslots - cb;
        moe_cluster_epilogue<WT, CHUNK, MODE, false>(p, base, tile, rank, SK, left < 0 ? 0 : (left > CHUNK ? CHUNK : left),
                                                     pos0 + cb, cpos0 + cb, tid);
    }

    // ---- teardown ----
    if (warp == 0 && lane == 0 && abort_flag) {
        for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(full_bar(i % STAGES), (i / STAGES) & 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// ---- e4m3 weights: TMA -> raw ring -> decode into tensor memory -> tcgen05.mma with A from tensor memory ----
// (pipeline of dense_umma_f8.cu; NA weight tiles per stage share the token tile; activations are bf16)
constexpr int kRawBytes = kTileM * kBlockK;      // 8 KB of e4m3 per tile and stage
constexpr int kAColumns = kBlockK / 2;           // 32-bit tensor-memory columns of one decoded tile
// Decoded weight tiles kept in tensor memory (= depth of the token-tile ring): as many as fit beside the accumulators
// in 128 columns, so that four CTAs share an SM's tensor memory; the 64-slot gate/up kernel needs 256 columns anyway.
constexpr int f8_conv_stages(int na, int np) {
    return na == 2 ? (np <= 32 ? 1 : 2) : (np <= 32 ? 3 : 2);
}

template <int NP, int STAGES, int MODE>
__global__ void __launch_bounds__(192, 2) moe_umma_f8_kernel(const __grid_constant__ CUtensorMap map_a,
                                                             const __grid_constant__ CUtensorMap map_x,
                                                             const MoeUmmaParams p, const int static_weights) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int NA = MODE == 1 ? 2 : 1;
    constexpr int S2 = f8_conv_stages(NA, NP);
    constexpr int kBBytes = NP * 128;
    constexpr int kStageBytes = NA * kRawBytes;
    constexpr int kRingBytes = STAGES * kStageBytes > NA * NP * 512 ? STAGES * kStageBytes : NA * NP * 512;
    constexpr uint32_t kTmemCols = (NA * NP + S2 * NA * kAColumns) <= 128 ? 128 : 256;
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 2 * S2 + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint64_t wpol = l2_evict_first_policy();       // weights are read once: first out of L2
    const int tile = blockIdx.x, rank = blockIdx.y, SK = gridDim.y;

    pdl_wait();
    pdl_launch_dependents();
    // both loads go out together (the list holds an entry for every z of the grid, live or not)
    const int n_items = p.worklist[0].x;
    const int4 item = p.worklist[1 + blockIdx.z];
    if ((int)blockIdx.z >= n_items) return;
    const int expert = item.x, pos0 = item.y, nslots = item.z, cpos0 = item.w;

    const int KB = p.kblocks;
    const int kb0 = (int)((long long)KB * rank / SK), kb1 = (int)((long long)KB * (rank + 1) / SK);
    const int nunits = kb1 - kb0;
    const int a_tile = expert * p.tiles_per_expert + tile;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t b_base = base + kRingBytes;
    const uint32_t bar0 = smem_u32(bars);
    auto raw_full = [&](int s) { return bar0 + 8u * s; };
    auto raw_empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto cv_full = [&](int s) { return bar0 + 8u * (2 * STAGES + s); };
    auto cv_empty = [&](int s) { return bar0 + 8u * (2 * STAGES + S2 + s); };
    const uint32_t acc_full = bar0 + 8u * (2 * STAGES + 2 * S2);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(raw_full(s), 1);
            mbar_init(raw_empty(s), 4);
        }
        for (int s = 0; s < S2; ++s) {
            mbar_init(cv_full(s), 5);
            mbar_init(cv_empty(s), 1);
        }
        mbar_init(acc_full, 1);
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

    int raw_issued = 0;
    if (warp == 0 && lane == 0) {
        // ---- TMA producer: raw weight tiles and token tiles are two independent streams, polled without blocking ----
        int ri = 0, bi = 0;
        uint32_t idle = 0;
        while ((bi < nunits || ri < nunits) && !abort_flag) {
            bool progressed = false;
            if (bi < nunits && (bi < S2 || mbar_test_wait(cv_empty(bi % S2), ((bi / S2) - 1) & 1))) {
                const int s2 = bi % S2;
                mbar_expect_tx(cv_full(s2), kBBytes);
                tma_load_2d(b_base + s2 * kBBytes, &map_x, cv_full(s2), (kb0 + bi) * kBlockK, cpos0);
                ++bi;
                progressed = true;
            }
            if (ri < nunits && (ri < STAGES || mbar_test_wait(raw_empty(ri % STAGES), ((ri / STAGES) - 1) & 1))) {
                const int s = ri % STAGES;
                mbar_expect_tx(raw_full(s), kStageBytes);
                tma_load_3d_hint(base + s * kStageBytes, &map_a, raw_full(s), 0, (kb0 + ri) * (kBlockK / 8), a_tile * (kTileM / 16), wpol);
                if constexpr (MODE == 1)
                    tma_load_3d_hint(base + s * kStageBytes + kRawBytes, &map_a, raw_full(s), 0, (kb0 + ri) * (kBlockK / 8),
                                (a_tile + p.up_tile_offset) * (kTileM / 16), wpol);
                ++raw_issued;
                ++ri;
                progressed = true;
            }
            if (progressed) {
                idle = 0;
            } else if (++idle > 4 * kSpinLimit) {
                abort_flag = 1;
                if (p.status) atomicExch(p.status, 1);
            } else {
                __nanosleep(32);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        constexpr uint32_t idesc = instr_desc<kBF16, NP>();
        for (int i = 0; i < nunits; ++i) {
            const int s2 = i % S2;
            if (abort_flag || !mbar_wait(cv_full(s2), (i / S2) & 1)) {
                if (!abort_flag && p.status) atomicExch(p.status, 2);
                abort_flag = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kk = 0; kk < kBlockK / 16; ++kk) {
                const uint64_t db = smem_desc(b_base + s2 * kBBytes + kk * 32, 16, 1024, 2);
#pragma unroll
                for (int w = 0; w < NA; ++w) {
                    const uint32_t ta = tmem + NA * NP + (s2 * NA + w) * kAColumns + kk * 8;
                    umma_f16_ts(tmem + w * NP, ta, db, idesc, (i > 0 || kk > 0) ? 1u : 0u);
                }
            }
            umma_commit(cv_empty(s2));
        }
        if (!abort_flag) umma_commit(acc_full);
    } else if (warp >= 2) {
        // ---- converter warps (thread = tile row = tensor-memory lane), then epilogue ----
        const int quad = warp & 3, lrow = quad * 32 + lane;
        // block scales: a 128-row tile is one scale row, a 64-wide k block half a scale column; the values of the
        // next unit are requested before this unit's waits
        const int scale_ld = KB >> 1;
        const float* srow[NA];
        float sc_next[NA];
        uint32_t c2[NA];
        ScaledRebias sr[NA];
#pragma unroll
        for (int w = 0; w < NA; ++w) {
            srow[w] = p.scale ? p.scale + (size_t)(a_tile + w * p.up_tile_offset) * scale_ld : nullptr;
            sc_next[w] = (p.scale && nunits > 0) ? __ldg(srow[w] + (kb0 >> 1)) : 1.f;
            c2[w] = kRebias2;
            sr[w] = ScaledRebias{};
        }
        for (int i = 0; i < nunits; ++i) {
            const int s = i % STAGES, s2 = i % S2;
            float sc[NA];
#pragma unroll
            for (int w = 0; w < NA; ++w) {
                sc[w] = sc_next[w];
                if (p.scale && i + 1 < nunits) sc_next[w] = __ldg(srow[w] + ((kb0 + i + 1) >> 1));
            }
            bool ok = true;
            if (lane == 0) {
                ok = !abort_flag && mbar_wait(raw_full(s), (i / STAGES) & 1);
                if (ok && i >= S2) ok = mbar_wait(cv_empty(s2), ((i / S2) - 1) & 1);
                if (!ok) {
                    if (!abort_flag && p.status) atomicExch(p.status, 8);
                    abort_flag = 1;
                }
            }
            ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int w = 0; w < NA; ++w) {
                const uint8_t* raw = base_ptr + s * kStageBytes + w * kRawBytes + (lrow >> 4) * 1024 + (lrow & 15) * 8;
                uint32_t v[32];
                // c2: the factor of the decode's one multiply (2^120, or that times a block scale rounded to bf16); 0 = general form
                if (p.scale && (i == 0 || ((kb0 + i) & 1) == 0)) {     // a scale column spans two k blocks
                    sr[w] = scaled_rebias(sc[w], p.full_scales != 0);
                    c2[w] = sr[w].one_multiply ? sr[w].hi2 : 0u;
                }
                if (c2[w] != 0u) {
#pragma unroll
                    for (int o = 0; o < 8; ++o) {
                        const uint2 x = *reinterpret_cast<const uint2*>(raw + o * 128);
                        v[4 * o + 0] = e4m3x2_to_bf16x2_by(x.x, p.sel01, c2[w]);
                        v[4 * o + 1] = e4m3x2_to_bf16x2_by(x.x, p.sel23, c2[w]);
                        v[4 * o + 2] = e4m3x2_to_bf16x2_by(x.y, p.sel01, c2[w]);
                        v[4 * o + 3] = e4m3x2_to_bf16x2_by(x.y, p.sel23, c2[w]);
                    }
                } else {
#pragma unroll
                    for (int o = 0; o < 8; ++o) {
                        const uint2 x = *reinterpret_cast<const uint2*>(raw + o * 128);
                        v[4 * o + 0] = e4m3x2_scaled(x.x, p.sel01, sr[w]);
                        v[4 * o + 1] = e4m3x2_scaled(x.x, p.sel23, sr[w]);
                        v[4 * o + 2] = e4m3x2_scaled(x.y, p.sel01, sr[w]);
                        v[4 * o + 3] = e4m3x2_scaled(x.y, p.sel23, sr[w]);
                    }
                }
                tmem_st32(tmem + ((uint32_t)(quad * 32) << 16) + NA * NP + (s2 * NA + w) * kAColumns, v);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(cv_full(s2)) : "memory");
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(raw_empty(s)) : "memory");
            }
        }
        if (lane == 0 && (abort_flag || !mbar_wait(acc_full, 0))) {
            if (!abort_flag && p.status) atomicExch(p.status, 3);
            abort_flag = 1;
        }
        __syncwarp();
        if (!abort_flag) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float* const red = reinterpret_cast<float*>(base_ptr);
#pragma unroll
            for (int c0 = 0; c0 < NA * NP; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(tmem + ((uint32_t)(quad * 32) << 16) + c0, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; ++i) red[(c0 + i) * kTileM + lrow] = __uint_as_float(r[i]);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
    }
    __syncwarp();

    moe_cluster_epilogue<kBF16, NP, MODE, true>(p, base, tile, rank, SK, nslots, pos0, cpos0, tid);

    if (warp == 0 && lane == 0 && abort_flag) {
        for (int i = max(0, raw_issued - STAGES); i < raw_issued; ++i) mbar_wait(raw_full(i % STAGES), (i / STAGES) & 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// Routed token rows in compact position order: xg[first compact position + c] = x[sorted[first position + c] / topk]
// for every slot c of every work item; one CTA per item.
__global__ void __launch_bounds__(256) moe_gather_positions_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ sorted,
                                                                   const int4* __restrict__ worklist, int topk, int h8,
                                                                   uint4* __restrict__ xg) {
    pdl_wait();
    pdl_launch_dependents();
    if ((int)blockIdx.x >= worklist[0].x) return;
    const int4 item = worklist[1 + blockIdx.x];
    const int total = item.z * h8;
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int c = i / h8, u = i - c * h8;
        const int slot = sorted[item.y + c];
        xg[(size_t)(item.w + c) * h8 + u] = x[(size_t)(slot / topk) * h8 + u];
    }
}

template <int WT, int NP, int MODE>
const void* moe_kernel_for_stages(int stages) {
    switch (stages) {
        case 2: return reinterpret_cast<const void*>(moe_umma_kernel<WT, NP, 2, MODE>);
        case 3: return reinterpret_cast<const void*>(moe_umma_kernel<WT, NP, 3, MODE>);
        case 4: return reinterpret_cast<const void*>(moe_umma_kernel<WT, NP, 4, MODE>);
        case 6: return reinterpret_cast<const void*>(moe_umma_kernel<WT, NP, 6, MODE>);
    }
    return nullptr;
}
template <int NP, int MODE>
const void* moe_f8_kernel_for_stages(int stages) {
    switch (stages) {
        case 2: return reinterpret_cast<const void*>(moe_umma_f8_kernel<NP, 2, MODE>);
        case 3: return reinterpret_cast<const void*>(moe_umma_f8_kernel<NP, 3, MODE>);
        case 4: return reinterpret_cast<const void*>(moe_umma_f8_kernel<NP, 4, MODE>);
        case 6: return reinterpret_cast<const void*>(moe_umma_f8_kernel<NP, 6, MODE>);
    }
    return nullptr;
}
template <int MODE>
const void* moe_f8_kernel_for(int np, int stages) {
    switch (np) {
        case 16: return moe_f8_kernel_for_stages<16, MODE>(stages);
        case 32: return moe_f8_kernel_for_stages<32, MODE>(stages);
        case 64: return moe_f8_kernel_for_stages<64, MODE>(stages);
    }
    return nullptr;
}
template <int WT, int MODE>
const void* moe_kernel_for(int np, int stages) {
    switch (np) {
        case 16: return moe_kernel_for_stages<WT, 16, MODE>(stages);
        case 32: return moe_kernel_for_stages<WT, 32, MODE>(stages);
        case 64: return moe_kernel_for_stages<WT, 64, MODE>(stages);
        case 128: return moe_kernel_for_stages<WT, 128, MODE>(stages);
    }
    return nullptr;
}

}  // namespace

int launch_moe_gather_positions(const void* x, const int32_t* sorted, const int4* worklist, int topk, int H, void* xg,
                                int max_items, cudaStream_t s) {
    if (H % 8 != 0) return fail(kInvalidArg, "moe gather: H must be a multiple of 8");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)max_items);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = launch_attrs(attr, 1);
    cudaError_t e = cudaLaunchKernelEx(&cfg, moe_gather_positions_kernel, reinterpret_cast<const uint4*>(x), sorted, worklist, topk,
                                       H / 8, reinterpret_cast<uint4*>(xg));
    if (e != cudaSuccess) return fail(kCudaError, "moe gather launch: %s", cudaGetErrorString(e));
    return kOk;
}

// One grouped GEMM.  mode 1: W = w1 [E, 2I, k=H], X = gathered tokens [n_slots, H], out = act [n_slots, I] (both in
// compact position order); mode 2: W = w2 [E, H, k=I], X = act [n_slots, I], out = scratch [n_slots, H] fp32 by slot.
int launch_moe_umma(int mode, int wt, const void* W, int E, int rows, int k, const void* X, long long x_rows, void* out,
                    const int4* worklist, const int32_t* sorted, const void* topk_weights, int n_slots, int np, int stages,
                    int cluster_k, int max_items, int fp8_order, const float* scale, int* status, cudaStream_t s) {
    const bool f8 = wt == kE4M3;
    if (wt != kBF16 && wt != kFP16 && !f8) return fail(kUnsupported, "moe (tcgen05): unsupported weight type");
    if (rows % kTileM != 0 || k % kBlockK != 0) return fail(kInvalidArg, "moe (tcgen05): sizes must be multiples of 128 (rows) and 64 (k)");
    if (cluster_k < 1 || cluster_k > 8 || cluster_k > k / kBlockK) return fail(kInvalidArg, "moe (tcgen05): cluster size %d out of range", cluster_k);
    if (encode_fn() == nullptr) return fail(kUnsupported, "moe (tcgen05): cuTensorMapEncodeTiled is not available");
    const void* kern = nullptr;
    if (f8) kern = mode == 1 ? moe_f8_kernel_for<1>(np, stages) : moe_f8_kernel_for<2>(np, stages);
    else if (mode == 1) kern = wt == kFP16 ? moe_kernel_for<kFP16, 1>(np, stages) : moe_kernel_for<kBF16, 1>(np, stages);
    else kern = wt == kFP16 ? moe_kernel_for<kFP16, 2>(np, stages) : moe_kernel_for<kBF16, 2>(np, stages);
    if (kern == nullptr) return fail(kInvalidArg, "moe (tcgen05): token tile %d / stages %d not built", np, stages);
    const int na = mode == 1 ? 2 : 1;
    const size_t want = f8 ? std::max((size_t)stages * na * kRawBytes, (size_t)na * np * 512) + (size_t)f8_conv_stages(na, np) * np * 128 + 1024
                           : std::max((size_t)stages * (na * kABytes + np * 128), (size_t)na * std::min(np, 64) * 512) + 1024;
    if (want > 227 * 1024) return fail(kUnsupported, "moe (tcgen05): %d stages do not fit in shared memory", stages);
    // tensor-memory columns of one CTA (as the kernels compute them): resident CTAs per SM are capped accordingly
    const int tmem_cols = f8 ? ((na * np + f8_conv_stages(na, np) * na * kAColumns) <= 128 ? 128 : 256)
                             : (na * np < 32 ? 32 : na * np);
    const size_t smem = prepare_kernel(kern, 192, want, tmem_cols);
    if (smem == 0) return fail(kCudaError, "moe (tcgen05): a CTA with %d stages does not fit on this device", stages);
    cudaError_t e = cudaSuccess;
    const long long w_rows = (long long)E * (mode == 1 ? 2 * rows : rows);
    CUtensorMap ma, mx;
    if (!(f8 ? make_map_a8(&ma, W, w_rows, k) : make_map_a16(&ma, W, w_rows, k, wt)))
        return fail(kUnsupported, "moe (tcgen05): weight tensor map rejected");
    if (!make_map_x(&mx, X, (int)x_rows, k, f8 ? kBF16 : wt, np)) return fail(kUnsupported, "moe (tcgen05): activation tensor map rejected");
    MoeUmmaParams mp{};
    mp.worklist = worklist; mp.sorted = sorted; mp.topk_weights = topk_weights; mp.out = out;
    mp.rows = rows;
    mp.tiles_per_expert = (mode == 1 ? 2 * rows : rows) / kTileM;
    mp.up_tile_offset = rows / kTileM;
    mp.kblocks = k / kBlockK;
    mp.n_slots = n_slots;
    mp.sel01 = fp8_order ? kSelRep01 : kSelNat01;
    mp.sel23 = fp8_order ? kSelRep23 : kSelNat23;
    mp.scale = (wt == kE4M3) ? scale : nullptr;
    mp.full_scales = option(kOptFullScales);
    mp.status = status;
    int static_weights = option(kOptStaticWeights);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(rows / kTileM), (unsigned)cluster_k, (unsigned)max_items);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = launch_attrs(attr, cluster_k);
    void* args[4] = {&ma, &mx, &mp, &static_weights};
    e = cudaLaunchKernelExC(&cfg, kern, args);
    if (e != cudaSuccess) return fail(kCudaError, "moe_umma launch: %s", cudaGetErrorString(e));
    return kOk;
}

}  // namespace mlk
