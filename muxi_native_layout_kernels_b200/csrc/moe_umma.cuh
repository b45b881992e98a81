// Pieces shared by the tcgen05 expert-GEMM kernels of the fused MoE (moe_umma.cu, moe_umma_f8n.cu): the kernel
// parameters and the cluster epilogue.
#pragma once

#include "moe.cuh"
#include "umma_common.cuh"

namespace mlk {

using umma::kTileM;

struct MoeUmmaParams {
    const int4* worklist;       // [0] = {n_items,..}; then {expert, first position, slots, first compact position}
    const int32_t* sorted;      // slot id of every position; >= n_slots marks padding
    const void* topk_weights;   // [n_slots] activation dtype (MODE 2)
    void* out;                  // MODE 1: act [compact positions, rows] 16-bit; MODE 2: scratch [n_slots, rows] fp32
    int rows;                   // output features: I (MODE 1) or H (MODE 2)
    int tiles_per_expert;       // weight row tiles of one expert in the tensor map: 2I/128 (MODE 1) or H/128
    int up_tile_offset;         // MODE 1: I/128
    int kblocks;
    int n_slots;
    uint32_t sel01, sel23;      // e4m3 kernels: byte selectors of the decode (natural or repacked order)
    const float* scale;         // e4m3 kernels: fp32 block scales [experts * tiles_per_expert][kblocks / 2], or null
    int full_scales;            // block scales with two bf16 terms instead of one (see common.cuh, scaled_rebias)
    int* status;
    const float* inv_scale;     // native-e4m3 kernels: [compact positions] factor of every activation row's fp32 sums
};

// Cluster epilogue shared by the two kernels: after a cluster barrier every CTA adds one slice of accumulator rows over
// all ranks (descending rank, fixed order) through distributed shared memory and emits it.  The partial tiles sit at
// `base` in every CTA as fp32 [which][slot][accumulator row].  NATURAL: accumulator row = tile row; otherwise row rho
// holds weight row 16*(rho%64 / 8) + 8*(rho / 64) + rho%8 of the tile (layout of the TMA-loaded 16-bit tile).
template <int WT, int NP, int MODE, bool NATURAL>
__device__ __forceinline__ void moe_cluster_epilogue(const MoeUmmaParams& p, uint32_t base, int tile, int rank, int SK,
                                                     int nslots, int pos0, int cpos0, int tid) {
    const int warp = tid >> 5;
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (warp >= 2) {
        const int etid = tid - 64;
        // slices in units of four accumulator rows: one 16-byte distributed-shared-memory load per rank brings four
        // rows of one slot, which are four consecutive weight rows (and output elements)
        const int q0 = (kTileM / 4) * rank / SK, quads = (kTileM / 4) * (rank + 1) / SK - q0;
        uint32_t remote[8];
#pragma unroll
        for (int q = 0; q < 8; ++q)
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[q]) : "r"(base), "r"(q < SK ? q : 0));
        auto cluster_sum = [&](uint32_t off) {
            float4 t[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
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
            for (int q = 7; q >= 0; --q) {
                if (q < SK) {
                    acc = first ? t[q] : make_float4(acc.x + t[q].x, acc.y + t[q].y, acc.z + t[q].z, acc.w + t[q].w);
                    first = false;
                }
            }
            return acc;
        };
        auto silu_mul = [](float gate, float up) { return gate / (1.f + __expf(-gate)) * up; };
        const int total = nslots * quads;
        for (int idx = etid; idx < total; idx += 128) {
            const int c = idx / quads, rho = 4 * (q0 + idx - c * quads);
            const int row = tile * kTileM + (NATURAL ? rho : ((rho & 63) >> 3) * 16 + (rho >> 6) * 8 + (rho & 7));
            const uint32_t off = (uint32_t)(c * kTileM + rho) * 4u;
            if constexpr (MODE == 1) {
                const float4 gate = cluster_sum(off);
                const float4 up = cluster_sum(off + (uint32_t)NP * kTileM * 4u);
                // four consecutive 16-bit outputs, 8-byte aligned (row is a multiple of 4, p.rows of 128)
                uint2 packed;
                packed.x = pack2<WT>(silu_mul(gate.x, up.x), silu_mul(gate.y, up.y));
                packed.y = pack2<WT>(silu_mul(gate.z, up.z), silu_mul(gate.w, up.w));
                const size_t o = (size_t)(cpos0 + c) * p.rows + row;
                *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.out) + o) = packed;
            } else {
                const int slot = p.sorted[pos0 + c];
                if (slot < p.n_slots) {
                    const float w = load_scalar16<WT>(p.topk_weights, slot);
                    const float4 v = cluster_sum(off);
                    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + (size_t)slot * p.rows + row) =
                        make_float4(w * v.x, w * v.y, w * v.z, w * v.w);
                }
            }
        }
    }
    // nobody leaves while its shared memory may still be read
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

}  // namespace mlk
