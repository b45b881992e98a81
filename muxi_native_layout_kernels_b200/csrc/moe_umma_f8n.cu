// Fused-MoE expert GEMMs with e4m3 weights fed to the tensor cores undecoded (tcgen05.mma.kind::f8f6f4): the grouped
// form of dense_umma_f8n.cu, with the work decomposition of moe_umma.cu.
//
//   * grid (128-row weight tiles, cluster, work items); a work item is one expert and up to 64 of its routed slots;
//   * the activation rows of an item are consecutive rows of "split planes" (f8n_common.cuh: every bf16 activation as
//     two e4m3 terms under a power-of-two scale per row), numbered by compact position (the routed slots expert by
//     expert, no padding).  For the first GEMM a kernel in front gathers the routed token rows and splits them in one
//     pass; for the second GEMM the [position, I] activation written by the first one is split in place;
//   * the mover warps copy the raw weight bytes of a stage from the TMA-landed tile into tensor memory (the A operand,
//     one row per lane): no instruction touches a weight byte otherwise;
//   * MODE 1 (first GEMM): gate tile and matching up tile per CTA, two accumulators fed by the same token tile,
//     silu(gate) * up on the fp32 sums; MODE 2 (second GEMM): x routing weight -> fp32 row per slot for the fixed-order
//     combine.  The inverse row scale is applied when the accumulators are parked for the cluster reduction.
// Block scales are not handled (the decode kernels of moe_umma.cu take those calls).
//
// Role in the reference: fused_moe_first/second_group_gemm_kernel with e4m3 weights
// (csrc/moe_kernels/soft_fp8_group_gemm_first.h:134, soft_fp8_group_gemm_second.h:122).
#include <algorithm>

#include "f8n_common.cuh"
#include "moe.cuh"
#include "moe_umma.cuh"

namespace mlk {

namespace {

using namespace umma;
using namespace f8n;

constexpr int kBK = 64;                          // k elements (weight bytes per row) of one stage
constexpr int kRaw = kTileM * kBK;               // 8 KB of e4m3 per tile and stage
constexpr int kACols = kBK / 4;                  // tensor-memory columns of one raw tile
// weight-tile slots in tensor memory beside the accumulators (64, 128 or 256 columns in all)
constexpr int f8n_slots(int na, int np) { return na == 2 ? (np == 16 ? 3 : (np == 32 ? 2 : 4)) : (np == 16 ? 3 : (np == 32 ? 2 : 4)); }
constexpr uint32_t f8n_tmem_cols(int na, int np) {
    const int need = na * np + f8n_slots(na, np) * na * kACols;
    return need <= 64 ? 64 : (need <= 128 ? 128 : 256);
}

template <int NP, int STAGES, int MODE, int BK>
__global__ void __launch_bounds__(192, 2) moe_umma_f8n_kernel(const __grid_constant__ CUtensorMap map_a,
                                                              const __grid_constant__ CUtensorMap map_x,
                                                              const MoeUmmaParams p, const int static_weights) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int NA = MODE == 1 ? 2 : 1;
    constexpr int S2 = BK == 64 ? f8n_slots(NA, NP) : 2;
    constexpr int kXTile = NP * 128;                   // split planes of one 64-wide k block
    constexpr int kRawB = kTileM * BK;                 // weight bytes of one tile and stage: BK = 64 or 128 k per stage
    constexpr int kACol = BK / 4;                      // their tensor-memory columns
    constexpr int kStageBytes = NA * kRawB + (BK / 64) * kXTile;
    constexpr int kColsNeeded = NA * NP + S2 * NA * kACol;
    constexpr uint32_t kTmemCols = kColsNeeded <= 64 ? 64 : (kColsNeeded <= 128 ? 128 : (kColsNeeded <= 256 ? 256 : 512));
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 2 * S2 + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, rank = blockIdx.y, SK = gridDim.y;
    const uint64_t wpol = l2_evict_first_policy();       // weights are read once: first out of L2

    // the work list and the split planes come from kernels earlier in the stream: nothing can start before them
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
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto a_full = [&](int s) { return bar0 + 8u * (2 * STAGES + s); };
    auto a_empty = [&](int s) { return bar0 + 8u * (2 * STAGES + S2 + s); };
    const uint32_t acc_full = bar0 + 8u * (2 * STAGES + 2 * S2);

    int early = 0;
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
        }
        for (int s = 0; s < S2; ++s) {
            mbar_init(a_full(s), 4);
            mbar_init(a_empty(s), 1);
        }
        mbar_init(acc_full, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the first ring's worth of weights and planes is on its way while tensor memory is being allocated: the
        // barriers are this thread's own, nobody else touches the ring yet
        for (; early < STAGES && early < nunits; ++early) {
            mbar_expect_tx(full(early), kStageBytes);
            tma_load_3d_hint(base + early * kStageBytes, &map_a, full(early), 0, (kb0 + early) * (BK / 8), a_tile * (kTileM / 16), wpol);
            if constexpr (MODE == 1)
                tma_load_3d_hint(base + early * kStageBytes + kRawB, &map_a, full(early), 0, (kb0 + early) * (BK / 8),
                            (a_tile + p.up_tile_offset) * (kTileM / 16), wpol);
#pragma unroll
            for (int h = 0; h < BK / 64; ++h)
                tma_load_2d(base + early * kStageBytes + NA * kRawB + h * kXTile, &map_x, full(early),
                            ((kb0 + early) * (BK / 64) + h) * 128, cpos0);
        }
    }
    // inverse row scale of every accumulator column (lane l: columns l and l + 32), in flight across the prologue
    constexpr int NCH = (NP + 31) / 32;
    float my_inv[NCH];
#pragma unroll
    for (int h = 0; h < NCH; ++h) {
        const int c = lane + 32 * h;
        my_inv[h] = (warp >= 2 && c < NP && c < nslots) ? __ldg(p.inv_scale + cpos0 + c) : 0.f;
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

    int issued = early;
    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        for (int i = early; i < nunits; ++i) {
            const int s = i % STAGES;
            if (i >= STAGES && !mbar_wait(empty(s), ((i / STAGES) - 1) & 1)) {
                abort_flag = 1;
                if (p.status) atomicExch(p.status, 1);
            }
            if (abort_flag) break;
            mbar_expect_tx(full(s), kStageBytes);
            tma_load_3d_hint(base + s * kStageBytes, &map_a, full(s), 0, (kb0 + i) * (BK / 8), a_tile * (kTileM / 16), wpol);
            if constexpr (MODE == 1)
                tma_load_3d_hint(base + s * kStageBytes + kRawB, &map_a, full(s), 0, (kb0 + i) * (BK / 8),
                            (a_tile + p.up_tile_offset) * (kTileM / 16), wpol);
#pragma unroll
            for (int h = 0; h < BK / 64; ++h)
                tma_load_2d(base + s * kStageBytes + NA * kRawB + h * kXTile, &map_x, full(s), ((kb0 + i) * (BK / 64) + h) * 128, cpos0);
            ++issued;
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        constexpr uint32_t idesc = instr_desc_f8<NP>();
        for (int i = 0; i < nunits; ++i) {
            const int s = i % STAGES, s2 = i % S2;
            if (abort_flag || !mbar_wait(a_full(s2), (i / S2) & 1)) {
                if (!abort_flag && p.status) atomicExch(p.status, 2);
                abort_flag = 1;
                break;
            }
            mbar_wait(full(s), (i / STAGES) & 1);       // already complete (the movers waited for it)
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int h = 0; h < BK / 64; ++h) {
                const uint32_t xt = base + s * kStageBytes + NA * kRawB + h * kXTile;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
#pragma unroll
                    for (int term = 0; term < 2; ++term) {
                        // token tile [NP][hi 64 | lo 64], 128-byte swizzle: hi operand at byte 32 j of every row, lo 64 further
                        const uint64_t db = smem_desc(xt + term * 64 + j * 32, 16, 1024, 2);
#pragma unroll
                        for (int w = 0; w < NA; ++w) {
                            const uint32_t ta = tmem + NA * NP + (s2 * NA + w) * kACol + h * 16 + j * 8;
                            umma_f8_ts(tmem + w * NP, ta, db, idesc, (i > 0 || h > 0 || j > 0 || term > 0) ? 1u : 0u);
                        }
                    }
                }
            }
            umma_commit(empty(s));
            umma_commit(a_empty(s2));
        }
        if (!abort_flag) umma_commit(acc_full);
    } else if (warp >= 2) {
        // ---- mover warps (thread = tile row = tensor-memory lane), then epilogue ----
        const int quad = warp & 3, lrow = quad * 32 + lane;
        for (int i = 0; i < nunits; ++i) {
            const int s = i % STAGES, s2 = i % S2;
            bool ok = true;
            if (lane == 0) {
                ok = !abort_flag && mbar_wait(full(s), (i / STAGES) & 1);
                if (ok && i >= S2) ok = mbar_wait(a_empty(s2), ((i / S2) - 1) & 1);
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
                const uint8_t* raw = base_ptr + s * kStageBytes + w * kRawB + (lrow >> 4) * (BK * 16) + (lrow & 15) * 8;
#pragma unroll
                for (int h = 0; h < BK / 64; ++h) {
                    uint32_t v[16];
#pragma unroll
                    for (int o = 0; o < 8; ++o) {
                        const uint2 x = *reinterpret_cast<const uint2*>(raw + (h * 8 + o) * 128);
                        v[2 * o] = x.x;
                        v[2 * o + 1] = x.y;
                    }
                    tmem_st16(tmem + ((uint32_t)(quad * 32) << 16) + NA * NP + (s2 * NA + w) * kACol + h * 16, v);
                }
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a_full(s2)) : "memory");
        }
        if (lane == 0 && (abort_flag || !mbar_wait(acc_full, 0))) {
            if (!abort_flag && p.status) atomicExch(p.status, 3);
            abort_flag = 1;
        }
        __syncwarp();
        if (MODE == 1 && SK == 1) {
            // no cluster: straight from tensor memory to the activation.  This thread holds gate row lrow (first
            // accumulator) and up row lrow (second) of the tile; a warp writes 32 consecutive elements of a slot's row.
            if (!abort_flag) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint16_t* const out = reinterpret_cast<uint16_t*>(p.out) + (size_t)cpos0 * p.rows + (size_t)tile * kTileM + lrow;
#pragma unroll
                for (int c0 = 0; c0 < NP; c0 += 16) {
                    if (c0 < nslots) {
                        uint32_t g[16], u[16];
                        tmem_ld16(tmem + ((uint32_t)(quad * 32) << 16) + c0, g);
                        tmem_ld16(tmem + ((uint32_t)(quad * 32) << 16) + NP + c0, u);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            if (c0 + i < nslots) {
                                const float inv = __shfl_sync(0xFFFFFFFFu, my_inv[(c0 + i) >> 5], (c0 + i) & 31);
                                const float gate = __uint_as_float(g[i]) * inv, up = __uint_as_float(u[i]) * inv;
                                out[(size_t)(c0 + i) * p.rows] = __bfloat16_as_ushort(__float2bfloat16_rn(gate / (1.f + __expf(-gate)) * up));
                            }
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
        } else if (!abort_flag) {
            // accumulators x inverse row scale -> fp32 partial tiles [which][slot][tile row] in the idle ring
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float* const red = reinterpret_cast<float*>(base_ptr);
#pragma unroll
            for (int c0 = 0; c0 < NA * NP; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(tmem + ((uint32_t)(quad * 32) << 16) + c0, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int c = (c0 + i) % NP;
                    const float inv = __shfl_sync(0xFFFFFFFFu, my_inv[c >> 5], c & 31);      // 0 past the item's slots
                    red[(c0 + i) * kTileM + lrow] = __uint_as_float(r[i]) * inv;
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
    }
    __syncwarp();

    if (!(MODE == 1 && SK == 1)) moe_cluster_epilogue<kBF16, NP, MODE, true>(p, base, tile, rank, SK, nslots, pos0, cpos0, tid);

    if (warp == 0 && lane == 0 && abort_flag) {
        for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(full(i % STAGES), (i / STAGES) & 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// Second GEMM with several 128-row weight tiles per CTA.  With a short k (the intermediate size of a fine-grained
// expert: 768 = 12 stages) a CTA that handles one tile spends as long on its start-up and its epilogue as on streaming.
// Here a CTA walks R consecutive row tiles of its work item: barriers, tensor memory and the TMA ring are set up once
// and the ring keeps streaming across tile boundaries; the accumulator is double-buffered (up to 32 slots per item), so
// the MMAs of the next tile run while the mover warps write the previous tile's rows; no cluster, so the epilogue goes
// straight from tensor memory to the fp32 rows of the combine scratch (128 consecutive floats per slot and warp pass).
template <int NP, int STAGES, int BK>
__global__ void __launch_bounds__(192, (NP <= 16 && BK == 64) ? 6 : 2) moe_umma_f8n_rows_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                   const __grid_constant__ CUtensorMap map_x,
                                                                   const MoeUmmaParams p, const int tiles_per_cta) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int AB = NP <= 32 ? 2 : 1;               // accumulator buffers
    constexpr int S2 = NP == 16 ? 2 : (NP == 32 ? 2 : 4);
    constexpr int kXTile = NP * 128;                   // split planes of one 64-wide k block
    constexpr int kRawB = kTileM * BK;                 // weight bytes of one stage: BK = 64 or 128 k per stage
    constexpr int kACol = BK / 4;                      // their tensor-memory columns
    constexpr int kStageBytes = kRawB + (BK / 64) * kXTile;
    constexpr uint32_t kTmemCols = (AB * NP + S2 * kACol) <= 64 ? 64 : ((AB * NP + S2 * kACol) <= 128 ? 128 : 256);
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 2 * S2 + 2 * AB];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;
    __shared__ int slot_w[4][NP];          // per mover warp: slot and factor of every accumulator column
    __shared__ float factor_w[4][NP];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint64_t wpol = l2_evict_first_policy();       // weights are read once: first out of L2

    pdl_wait();
    pdl_launch_dependents();
    // both loads go out together (the list holds an entry for every z of the grid, live or not)
    const int n_items = p.worklist[0].x;
    const int4 item = p.worklist[1 + blockIdx.z];
    if ((int)blockIdx.z >= n_items) return;
    const int expert = item.x, pos0 = item.y, nslots = item.z, cpos0 = item.w;
    const int tiles_total = p.tiles_per_expert;
    const int tile0 = blockIdx.x * tiles_per_cta;
    const int ntiles = min(tiles_per_cta, tiles_total - tile0);
    const int KB = p.kblocks;
    const int total = ntiles * KB;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto a_full = [&](int s) { return bar0 + 8u * (2 * STAGES + s); };
    auto a_empty = [&](int s) { return bar0 + 8u * (2 * STAGES + S2 + s); };
    auto acc_full = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 * S2 + b); };
    auto acc_empty = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 * S2 + AB + b); };

    int early = 0;
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
        }
        for (int s = 0; s < S2; ++s) {
            mbar_init(a_full(s), 4);
            mbar_init(a_empty(s), 1);
        }
        for (int b = 0; b < AB; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 4);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the first ring's worth of weights and planes is on its way while the other warps finish the prologue
        // (tensor-memory allocation, the slots' factors): the barriers are this thread's own, nobody else touches the ring yet
        for (; early < STAGES && early < total; ++early) {
            const int tl = early / KB, kb = early - tl * KB;
            mbar_expect_tx(full(early), kStageBytes);
            tma_load_3d_hint(base + early * kStageBytes, &map_a, full(early), 0, kb * (BK / 8),
                        (expert * tiles_total + tile0 + tl) * (kTileM / 16), wpol);
#pragma unroll
            for (int h = 0; h < BK / 64; ++h)
                tma_load_2d(base + early * kStageBytes + kRawB + h * kXTile, &map_x, full(early), (kb * (BK / 64) + h) * 128, cpos0);
        }
    }
    // slot and factor (inverse row scale x routing weight) of every column of the accumulator: every mover warp loads
    // them for itself (lane l: columns l and l + 32), so that the loads stay in flight across the prologue and the
    // weights' first round trip ...
    constexpr int NCH = (NP + 31) / 32;
    int my_slot[NCH];
    float my_factor[NCH];
#pragma unroll
    for (int h = 0; h < NCH; ++h) {
        my_slot[h] = -1;
        my_factor[h] = 0.f;
        const int c = lane + 32 * h;
        if (warp >= 2 && c < NP && c < nslots) {
            my_slot[h] = p.sorted[pos0 + c];
            my_factor[h] = __ldg(p.inv_scale + cpos0 + c);
        }
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

    int issued = early;
    if (warp == 0 && lane == 0) {
        // ---- TMA producer: units (tile, k block), tile-major ----
        int tl = early / KB, kb = early - tl * KB;
        for (int u = early; u < total; ++u) {
            const int s = u % STAGES;
            if (u >= STAGES && !mbar_wait(empty(s), ((u / STAGES) - 1) & 1)) {
                abort_flag = 1;
                if (p.status) atomicExch(p.status, 1);
            }
            if (abort_flag) break;
            mbar_expect_tx(full(s), kStageBytes);
            tma_load_3d_hint(base + s * kStageBytes, &map_a, full(s), 0, kb * (BK / 8),
                        (expert * tiles_total + tile0 + tl) * (kTileM / 16), wpol);
#pragma unroll
            for (int h = 0; h < BK / 64; ++h)
                tma_load_2d(base + s * kStageBytes + kRawB + h * kXTile, &map_x, full(s), (kb * (BK / 64) + h) * 128, cpos0);
            ++issued;
            if (++kb == KB) { kb = 0; ++tl; }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        constexpr uint32_t idesc = instr_desc_f8<NP>();
        int tl = 0, kb = 0;
        for (int u = 0; u < total; ++u) {
            const int s = u % STAGES, s2 = u % S2, b = tl % AB;
            bool ok = !abort_flag;
            if (ok && kb == 0 && tl >= AB) ok = mbar_wait(acc_empty(b), ((tl / AB) - 1) & 1);   // the epilogue has read it
            if (ok) ok = mbar_wait(a_full(s2), (u / S2) & 1);
            if (!ok) {
                if (!abort_flag && p.status) atomicExch(p.status, 2);
                abort_flag = 1;
                break;
            }
            mbar_wait(full(s), (u / STAGES) & 1);       // already complete (the movers waited for it)
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int h = 0; h < BK / 64; ++h) {
                const uint32_t xt = base + s * kStageBytes + kRawB + h * kXTile;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
#pragma unroll
                    for (int term = 0; term < 2; ++term) {
                        const uint64_t db = smem_desc(xt + term * 64 + j * 32, 16, 1024, 2);
                        umma_f8_ts(tmem + b * NP, tmem + AB * NP + s2 * kACol + h * 16 + j * 8, db, idesc,
                                   (kb > 0 || h > 0 || j > 0 || term > 0) ? 1u : 0u);
                    }
                }
            }
            umma_commit(empty(s));
            umma_commit(a_empty(s2));
            if (++kb == KB) {
                umma_commit(acc_full(b));
                kb = 0;
                ++tl;
            }
        }
    } else if (warp >= 2) {
        // ---- mover warps (thread = tile row = tensor-memory lane); after a tile's last k block, its epilogue ----
        const int quad = warp & 3, lrow = quad * 32 + lane;
        // ... and published in this warp's own copy in shared memory (no barrier across the mover warps needed)
#pragma unroll
        for (int h = 0; h < NCH; ++h) {
            if (my_slot[h] >= 0 && my_slot[h] < p.n_slots) my_factor[h] *= load_scalar16<kBF16>(p.topk_weights, my_slot[h]);
            else my_slot[h] = -1;
            if (lane + 32 * h < NP) {
                slot_w[quad][lane + 32 * h] = my_slot[h];
                factor_w[quad][lane + 32 * h] = my_factor[h];
            }
        }
        __syncwarp();
        int u = 0;
        for (int tl = 0; tl < ntiles && !abort_flag; ++tl) {
            bool ok = true;
            for (int kb = 0; kb < KB; ++kb, ++u) {
                const int s = u % STAGES, s2 = u % S2;
                if (lane == 0) {
                    ok = !abort_flag && mbar_wait(full(s), (u / STAGES) & 1);
                    if (ok && u >= S2) ok = mbar_wait(a_empty(s2), ((u / S2) - 1) & 1);
                    if (!ok) {
                        if (!abort_flag && p.status) atomicExch(p.status, 8);
                        abort_flag = 1;
                    }
                }
                ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint8_t* raw = base_ptr + s * kStageBytes + (lrow >> 4) * (BK * 16) + (lrow & 15) * 8;
#pragma unroll
                for (int h = 0; h < BK / 64; ++h) {
                    uint32_t v[16];
#pragma unroll
                    for (int o = 0; o < 8; ++o) {
                        const uint2 x = *reinterpret_cast<const uint2*>(raw + (h * 8 + o) * 128);
                        v[2 * o] = x.x;
                        v[2 * o + 1] = x.y;
                    }
                    tmem_st16(tmem + ((uint32_t)(quad * 32) << 16) + AB * NP + s2 * kACol + h * 16, v);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a_full(s2)) : "memory");
            }
            if (!ok) break;
            const int b = tl % AB;
            if (lane == 0 && (abort_flag || !mbar_wait(acc_full(b), (tl / AB) & 1))) {
                if (!abort_flag && p.status) atomicExch(p.status, 3);
                abort_flag = 1;
            }
            ok = __shfl_sync(0xFFFFFFFFu, abort_flag ? 0 : 1, 0) != 0;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float* const out = reinterpret_cast<float*>(p.out) + (size_t)(tile0 + tl) * kTileM + lrow;
#pragma unroll
            for (int c0 = 0; c0 < NP; c0 += 16) {
                if (c0 < nslots) {
                    uint32_t r[16];
                    tmem_ld16(tmem + ((uint32_t)(quad * 32) << 16) + b * NP + c0, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int slot = slot_w[quad][c0 + i];
                        if (slot >= 0) out[(size_t)slot * p.rows] = __uint_as_float(r[i]) * factor_w[quad][c0 + i];
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(b)) : "memory");
        }
    }
    __syncwarp();

    if (warp == 0 && lane == 0 && abort_flag) {
        for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(full(i % STAGES), (i / STAGES) & 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// Split planes of the routed token rows in compact position order: row r is token cpos_slot[r] / topk of x; one CTA
// per compact position, positions past the routed count (worklist[0].y) leave at once.
__global__ void __launch_bounds__(512) moe_split_gather_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ cpos_slot,
                                                              const int4* __restrict__ worklist, int topk, int k,
                                                              int repacked, uint8_t* __restrict__ planes,
                                                              float* __restrict__ inv_scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x;
    if (row >= worklist[0].y) return;
    const int token = cpos_slot[row] / topk;
    split_row_cta(x + (size_t)token * (k >> 3), false, k, repacked, planes + (size_t)row * 2 * k, inv_scale + row);
}

// Split planes of the [position, k] activation, in place (a row of k bf16 elements and its planes are both 2 k bytes).
__global__ void __launch_bounds__(512) moe_split_inplace_kernel(uint4* __restrict__ act, const int4* __restrict__ worklist, int k,
                                                               int repacked, float* __restrict__ inv_scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x;
    if (row >= worklist[0].y) return;
    uint4* const r = act + (size_t)row * (k >> 3);
    split_row_cta(r, false, k, repacked, reinterpret_cast<uint8_t*>(r), inv_scale + row);
}

// The two kernels above with one row per warp (rows of at most 2048 elements): eight rows per CTA, no CTA barrier.
__global__ void __launch_bounds__(256) moe_split_gather_warp_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ cpos_slot,
                                                                   const int4* __restrict__ worklist, int topk, int k,
                                                                   int repacked, uint8_t* __restrict__ planes,
                                                                   float* __restrict__ inv_scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= worklist[0].y) return;
    const int token = cpos_slot[row] / topk;
    split_row_warp(x + (size_t)token * (k >> 3), k, repacked, planes + (size_t)row * 2 * k, inv_scale + row);
}

__global__ void __launch_bounds__(256) moe_split_inplace_warp_kernel(uint4* __restrict__ act, const int4* __restrict__ worklist,
                                                                    int k, int repacked, float* __restrict__ inv_scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= worklist[0].y) return;
    uint4* const r = act + (size_t)row * (k >> 3);
    split_row_warp(r, k, repacked, reinterpret_cast<uint8_t*>(r), inv_scale + row);
}

template <int NP, int MODE, int BK>
const void* kernel_for_stages(int stages) {
    switch (stages) {
        case 2: return reinterpret_cast<const void*>(moe_umma_f8n_kernel<NP, 2, MODE, BK>);
        case 3: return reinterpret_cast<const void*>(moe_umma_f8n_kernel<NP, 3, MODE, BK>);
        case 4: return reinterpret_cast<const void*>(moe_umma_f8n_kernel<NP, 4, MODE, BK>);
        case 6: return reinterpret_cast<const void*>(moe_umma_f8n_kernel<NP, 6, MODE, BK>);
    }
    return nullptr;
}
template <int MODE>
const void* kernel_for(int np, int stages, int bk) {
    if (bk == 128) {
        // 128 k per stage: the first GEMM with 64-slot tiles (where the mover / MMA chain per k block weighs most)
        if (MODE == 1 && np == 64 && stages <= 3) return kernel_for_stages<64, 1, 128>(stages);
        return nullptr;
    }
    switch (np) {
        case 16: return kernel_for_stages<16, MODE, 64>(stages);
        case 32: return kernel_for_stages<32, MODE, 64>(stages);
        case 64: return kernel_for_stages<64, MODE, 64>(stages);
    }
    return nullptr;
}

template <int NP, int BK>
const void* rows_kernel_for_stages(int stages) {
    switch (stages) {
        case 2: return reinterpret_cast<const void*>(moe_umma_f8n_rows_kernel<NP, 2, BK>);
        case 3: return reinterpret_cast<const void*>(moe_umma_f8n_rows_kernel<NP, 3, BK>);
        case 4: return reinterpret_cast<const void*>(moe_umma_f8n_rows_kernel<NP, 4, BK>);
        case 6: return reinterpret_cast<const void*>(moe_umma_f8n_rows_kernel<NP, 6, BK>);
    }
    return nullptr;
}
const void* rows_kernel_for(int np, int stages, int bk) {
    if (bk == 128) {
        switch (np) {
            case 16: return rows_kernel_for_stages<16, 128>(stages);
            case 32: return rows_kernel_for_stages<32, 128>(stages);
            case 64: return rows_kernel_for_stages<64, 128>(stages);
        }
        return nullptr;
    }
    switch (np) {
        case 16: return rows_kernel_for_stages<16, 64>(stages);
        case 32: return rows_kernel_for_stages<32, 64>(stages);
        case 64: return rows_kernel_for_stages<64, 64>(stages);
    }
    return nullptr;
}

int launch_split(const void* kern, const void* warp_kern, void** args, int rows, int k, cudaStream_t s) {
    cudaLaunchConfig_t cfg = {};
    const bool by_warp = k <= kSplitWarpMaxK;
    if (by_warp) kern = warp_kern;
    cfg.gridDim = dim3((unsigned)(by_warp ? (rows + 7) / 8 : rows));
    cfg.blockDim = dim3(by_warp ? 256 : split_threads(k));
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = launch_attrs(attr, 1);
    const cudaError_t e = cudaLaunchKernelExC(&cfg, kern, args);
    if (e != cudaSuccess) return fail(kCudaError, "moe activation split launch: %s", cudaGetErrorString(e));
    return kOk;
}

}  // namespace

bool moe_f8n_supported(int H, int I) { return H % 128 == 0 && I % 128 == 0 && H <= kSplitMaxK && I <= kSplitMaxK; }

int launch_moe_split_gather(const void* x, const int32_t* cpos_slot, const int4* worklist, int topk, int H, int repacked,
                            void* planes, float* inv_scale, int n_slots, cudaStream_t s) {
    void* args[8] = {&x, &cpos_slot, &worklist, &topk, &H, &repacked, &planes, &inv_scale};
    return launch_split(reinterpret_cast<const void*>(moe_split_gather_kernel), reinterpret_cast<const void*>(moe_split_gather_warp_kernel),
                        args, n_slots, H, s);
}

int launch_moe_split_inplace(void* act, const int4* worklist, int I, int repacked, float* inv_scale, int n_slots,
                             cudaStream_t s) {
    void* args[5] = {&act, &worklist, &I, &repacked, &inv_scale};
    return launch_split(reinterpret_cast<const void*>(moe_split_inplace_kernel), reinterpret_cast<const void*>(moe_split_inplace_warp_kernel),
                        args, n_slots, I, s);
}

// One grouped GEMM on split planes.  mode 1: W = w1 [E, 2I, k=H], planes of the gathered tokens, out = act [n_slots, I]
// bf16 by compact position; mode 2: W = w2 [E, H, k=I], planes of the activation, out = scratch [n_slots, H] fp32 by slot.
int launch_moe_umma_f8n(int mode, const void* W, int E, int rows, int k, const void* planes, const float* inv_scale,
                        long long plane_rows, void* out, const int4* worklist, const int32_t* sorted,
                        const void* topk_weights, int n_slots, int np, int stages, int cluster_k, int max_items, int* status,
                        cudaStream_t s) {
    if (rows % kTileM != 0 || k % kBK != 0) return fail(kInvalidArg, "moe (tcgen05, native e4m3): sizes must be multiples of 128 (rows) and 64 (k)");
    if (mode == 2 && cluster_k >= 11 && cluster_k <= 18) {
        // second GEMM, no cluster, cluster_k - 10 row tiles per CTA
        const int tiles_per_cta = cluster_k - 10;
        if (encode_fn() == nullptr) return fail(kUnsupported, "moe (tcgen05): cuTensorMapEncodeTiled is not available");
        if (((uintptr_t)planes & 127) != 0) return fail(kInvalidArg, "moe (tcgen05, native e4m3): split planes must be 128-byte aligned");
        // stages >= 40: 128 k per stage (stages - 40 ring stages), half as many steps of the mover / MMA chain per tile
        int bk = kBK;
        if (stages >= 40) {
            stages -= 40;
            if (k % 128 == 0) bk = 128;
        }
        const void* kern = rows_kernel_for(np, stages, bk);
        if (kern == nullptr) return fail(kInvalidArg, "moe (tcgen05, native e4m3): token tile %d / stages %d not built", np, stages);
        const size_t want = (size_t)stages * (kTileM * bk + (bk / 64) * np * 128) + 1024;
        const int s2 = np == 64 ? 4 : 2, ab = np <= 32 ? 2 : 1;
        const int cols = ab * np + s2 * (bk / 4);
        const size_t smem = prepare_kernel(kern, 192, want, cols <= 64 ? 64 : (cols <= 128 ? 128 : 256));
        if (smem == 0) return fail(kCudaError, "moe (tcgen05, native e4m3): a CTA with %d stages does not fit on this device", stages);
        CUtensorMap ma, mx;
        if (!make_map_a8_bk(&ma, W, (long long)E * rows, k, bk)) return fail(kUnsupported, "moe (tcgen05): weight tensor map rejected");
        if (!make_map_planes(&mx, planes, plane_rows, k, np)) return fail(kUnsupported, "moe (tcgen05): activation tensor map rejected");
        MoeUmmaParams mp{};
        mp.worklist = worklist; mp.sorted = sorted; mp.topk_weights = topk_weights; mp.out = out;
        mp.rows = rows;
        mp.tiles_per_expert = rows / kTileM;
        mp.kblocks = k / bk;
        mp.n_slots = n_slots;
        mp.status = status;
        mp.inv_scale = inv_scale;
        int tpc = tiles_per_cta;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)((rows / kTileM + tiles_per_cta - 1) / tiles_per_cta), 1, (unsigned)max_items);
        cfg.blockDim = dim3(192);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[2];
        cfg.attrs = attr;
        cfg.numAttrs = launch_attrs(attr, 1);
        void* args[4] = {&ma, &mx, &mp, &tpc};
        const cudaError_t e = cudaLaunchKernelExC(&cfg, kern, args);
        if (e != cudaSuccess) return fail(kCudaError, "moe_umma_f8n_rows launch: %s", cudaGetErrorString(e));
        return kOk;
    }
    // stages >= 40: 128 k per stage (stages - 40 ring stages) where that form is built (first GEMM, 64-slot tiles, no cluster)
    int bk = kBK;
    if (stages >= 40) {
        stages -= 40;
        if (mode == 1 && np == 64 && stages <= 3 && cluster_k == 1 && k % 128 == 0) bk = 128;
    }
    if (cluster_k < 1 || cluster_k > 8 || cluster_k > k / bk) return fail(kInvalidArg, "moe (tcgen05, native e4m3): cluster size %d out of range", cluster_k);
    if (encode_fn() == nullptr) return fail(kUnsupported, "moe (tcgen05): cuTensorMapEncodeTiled is not available");
    if (((uintptr_t)planes & 127) != 0) return fail(kInvalidArg, "moe (tcgen05, native e4m3): split planes must be 128-byte aligned");
    const void* kern = mode == 1 ? kernel_for<1>(np, stages, bk) : kernel_for<2>(np, stages, bk);
    if (kern == nullptr) return fail(kInvalidArg, "moe (tcgen05, native e4m3): token tile %d / stages %d not built", np, stages);
    const int na = mode == 1 ? 2 : 1;
    const size_t want = std::max((size_t)stages * (na * kTileM * bk + (bk / 64) * np * 128), (size_t)na * np * 512) + 1024;
    if (want > 227 * 1024) return fail(kUnsupported, "moe (tcgen05, native e4m3): %d stages do not fit in shared memory", stages);
    const int cols = bk == 64 ? (int)f8n_tmem_cols(na, np) : na * np + 2 * na * (bk / 4);
    const size_t smem = prepare_kernel(kern, 192, want, cols <= 64 ? 64 : (cols <= 128 ? 128 : (cols <= 256 ? 256 : 512)));
    if (smem == 0) return fail(kCudaError, "moe (tcgen05, native e4m3): a CTA with %d stages does not fit on this device", stages);
    const long long w_rows = (long long)E * (mode == 1 ? 2 * rows : rows);
    CUtensorMap ma, mx;
    if (!make_map_a8_bk(&ma, W, w_rows, k, bk)) return fail(kUnsupported, "moe (tcgen05): weight tensor map rejected");
    if (!make_map_planes(&mx, planes, plane_rows, k, np)) return fail(kUnsupported, "moe (tcgen05): activation tensor map rejected");
    MoeUmmaParams mp{};
    mp.worklist = worklist; mp.sorted = sorted; mp.topk_weights = topk_weights; mp.out = out;
    mp.rows = rows;
    mp.tiles_per_expert = (mode == 1 ? 2 * rows : rows) / kTileM;
    mp.up_tile_offset = rows / kTileM;
    mp.kblocks = k / bk;
    mp.n_slots = n_slots;
    mp.status = status;
    mp.inv_scale = inv_scale;
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
    const cudaError_t e = cudaLaunchKernelExC(&cfg, kern, args);
    if (e != cudaSuccess) return fail(kCudaError, "moe_umma_f8n launch: %s", cudaGetErrorString(e));
    return kOk;
}

}  // namespace mlk
