// Host-side launch interface of the fused-MoE kernels (router, token alignment, expert compute).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mlk {

int launch_router(const void* gating_output, int score_fun, int T, int E, int n_groups, int topk_groups,
                  int32_t* experts_ids, void* weights, int topk, const void* bias, int dtype, cudaStream_t s,
                  int renormalize = 0);

// Router GEMM (x [T,H] times gate_weight [E,H]^T, rounded to the 16-bit type) fused with the routing above.
int launch_router_gemm(const void* x, const void* gate_weight, int score_fun, int T, int H, int E, int n_groups,
                       int topk_groups, int32_t* experts_ids, void* weights, int topk, const void* bias, int dtype,
                       int renormalize, void* logits_out, cudaStream_t s);

// worklist == nullptr: alignment only (the stand-alone reference op).  Otherwise the kernel also writes
// the expert-compute work list (see MoeWorkHeader) for blocks of `block_slots` slots.
int launch_moe_align(int T, int E, int topk, int mbs, const int32_t* topk_ids, int32_t* sorted_token_ids,
                     int32_t* cumsum, int32_t* padded_num_experts, int32_t* experts_ids_out,
                     const int32_t* experts_map, int experts_map_len, cudaStream_t s, void* worklist = nullptr,
                     int block_slots = 0, int32_t* cpos_slot = nullptr);

// Work list written by the alignment kernel into the spare half of the caller's workspace C:
//   int32 header[4] = {n_items, routed slots on this rank, 0, 0}; then n_items x int4 {expert, first position in sorted_token_ids, slots,
//   first compact position}: compact positions number the routed slots expert by expert without the padding
struct MoeWorkHeader {
    int n_items, pad0, pad1, pad2;
};

struct MoeParams {
    const void* w1;   // [E, 2I, H] layout A per expert (gate rows, then up rows)
    const void* w2;   // [E, H, I]  layout A per expert
    const void* x;    // [T, H]
    int T, E, topk, H, I;
    const int32_t* topk_ids;      // [T, topk]
    const void* topk_weights;     // [T, topk] activation dtype
    int32_t* sorted_token_ids;    // [T*topk + E*(mbs-1)], pre-filled with T*topk
    int32_t* cumsum;              // [E+1]
    int32_t* padded_num_experts;  // [1]
    int32_t* experts_ids;         // [ceil(len/mbs)]
    void* C;                      // workspace, T*topk*2I activation elements
    void* y;                      // [T, H], zero on entry
    const float* w1_scale;        // e4m3: [E, 2I/128, H/128] or null
    const float* w2_scale;        // e4m3: [E, H/128, I/128] or null
    int dtype, fp8_order, mbs;
    const int32_t* experts_map;
    int experts_map_len;
    float* scratch;               // optional [T*topk, H] fp32 for the deterministic combine
    long long scratch_bytes;
    int y_fp32;                   // y is [T, H] fp32: the token sums un-rounded (needs the combine scratch)
    // routing fused in front (mlk_fused_routing_experts_compute): gating != nullptr makes topk_ids / topk_weights outputs
    const void* gating;           // [T, n_global_experts] router logits, activation dtype
    const void* gating_bias;
    int n_global, score_fun, n_groups, topk_groups, renormalize;
    int* status;                  // sticky error word of the bounded waits inside the tcgen05 kernels (0 = ok), or null
    int nt, wm1, sk1, rg, wm2, sk2;   // tuning (0 = choose by shape): token tiles, GEMM1 row warps / split-K, GEMM2 row groups / row warps / split-K;
                                      // wm1 = 100 + s1 and wm2 = 100 + s2 select the tcgen05 kernels (combine scratch given)
                                      // with s1 / s2 ring stages and sk1 / sk2 CTAs per cluster; 200 + s1 / 200 + s2 the
                                      // native-e4m3 tcgen05 kernels (e4m3 weights without block scales); there sk2 = 10 + r
                                      // (11..18) runs the second GEMM without clusters, r 128-row tiles per CTA
};

int launch_fused_experts(const MoeParams& p, cudaStream_t s);

// tcgen05 expert GEMMs (moe_umma.cu): gather of the routed token rows into position order, and one grouped GEMM
// (mode 1: gate/up + SiLU*up into the [position, I] activation; mode 2: routing-weighted fp32 rows per slot).
int launch_moe_gather_positions(const void* x, const int32_t* sorted, const int4* worklist, int topk, int H, void* xg,
                                int max_items, cudaStream_t s);
int launch_moe_umma(int mode, int wt, const void* W, int E, int rows, int k, const void* X, long long x_rows, void* out,
                    const int4* worklist, const int32_t* sorted, const void* topk_weights, int n_slots, int np, int stages,
                    int cluster_k, int max_items, int fp8_order, const float* scale, int* status, cudaStream_t s);
// the same two GEMMs with e4m3 weights undecoded into the 8-bit MMA (moe_umma_f8n.cu): activation rows as split planes
bool moe_f8n_supported(int H, int I);
int launch_moe_split_gather(const void* x, const int32_t* cpos_slot, const int4* worklist, int topk, int H, int repacked,
                            void* planes, float* inv_scale, int n_slots, cudaStream_t s);
int launch_moe_split_inplace(void* act, const int4* worklist, int I, int repacked, float* inv_scale, int n_slots,
                             cudaStream_t s);
int launch_moe_umma_f8n(int mode, const void* W, int E, int rows, int k, const void* planes, const float* inv_scale,
                        long long plane_rows, void* out, const int4* worklist, const int32_t* sorted,
                        const void* topk_weights, int n_slots, int np, int stages, int cluster_k, int max_items, int* status,
                        cudaStream_t s);
// decode batches (at most 8 tokens, 64 routed slots) as one cooperative kernel (moe_decode.cu); tuning values of 300 or
// more in both "row warps" fields select it
bool moe_decode_supported(const MoeParams& m);
int launch_moe_decode(const MoeParams& m, cudaStream_t s);
int launch_fused_experts_static(const MoeParams& p, cudaStream_t s);   // combine scratch in a built-in device array

// Expert-parallel exchange helpers (moe_exchange.cu).
int launch_gather_rows(const void* x, const int32_t* idx, void* out, long long n_rows, int H, long long x_rows,
                       cudaStream_t s);
int launch_unpermute_sum(const void* rows, const int32_t* pos, void* y, long long T, int topk, int H, long long n_rows,
                         int dtype, cudaStream_t s);

// Sum of the ranks' fp32 shares over peer memory, rounded once, finished rows stored into every rank's output
// (ep_reduce.cu).  The three arguments are DEVICE arrays of `world` pointers (every rank's share / output / flag block).
long long ep_reduce_flag_bytes();
long long ep_reduce_recv_bytes(int world, long long T, int H);      // receive buffer of the one-pass form, 0 = share too large for it
int launch_ep_reduce(const void* const* shares_dev, void* const* outs_dev, void* const* flags_dev, void* const* recv_dev,
                     int rank, int world, long long T, int H, int dtype, int* status, cudaStream_t s);

}  // namespace mlk
