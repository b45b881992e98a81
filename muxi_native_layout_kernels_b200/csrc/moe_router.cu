// MoE router: score function + optional selection bias + group-limited top-k, one warp per token.
//
// Semantics follow the reference's torch formulation (muxi_layout_kernels/utils.py:160-216) with the
// tie rule of its device kernel (csrc/moe_kernels/fused_topK.h:255-262, "lower id wins"):
//   score = softmax(logits) or sigmoid(logits), fp32 math, rounded to the logits' 16-bit type
//   sel   = score + bias (rounded) if a bias is given, else score
//   group score = max of sel in the group, or the rounded sum of its two largest sel with a bias
//   keep the topk_groups best groups (ties: lower group id); sel of every other group becomes 0
//   pick topk largest sel (ties: lower expert id); returned weights are the un-biased scores
//   output order: ascending expert id for softmax, selection order for sigmoid (fused_topK.h:294-306, :575-586)
// Unlike the reference launcher (fused_gating.h:22: only 8 groups / 4 kept / top-8), any E <= 256 that the
// group count divides is accepted.
#include <algorithm>

#include "common.cuh"
#include "moe.cuh"
#include "moe_route.cuh"
#include "status.h"

namespace mlk {

namespace {

template <int WT>
__global__ void __launch_bounds__(128) router_kernel(const void* __restrict__ logits, int score_fun, int T, int E,
                                                     int G, int KG, int32_t* __restrict__ ids, void* __restrict__ wts,
                                                     int topk, const void* __restrict__ bias, int renormalize) {
    extern __shared__ float sm[];
    // the logits come from the preceding kernel of the stream; the kernels behind this one may become resident
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= T) return;
    float* ssel = sm + warp * (E + 2 * G);
    float* sg = ssel + E;
    int* gmask = reinterpret_cast<int*>(sg + G);
    float x[kVPT];
#pragma unroll
    for (int i = 0; i < kVPT; ++i) {
        const int e = lane + 32 * i;
        x[i] = (e < E) ? load_scalar16<WT>(logits, (int64_t)row * E + e) : -INFINITY;
    }
    route_token<WT>(x, row, lane, score_fun, E, G, KG, ids, wts, topk, bias, renormalize, ssel, sg, gmask);
}

// Router GEMM fused with the routing: logits[t, e] = sum_h x[t, h] * Wg[e, h] (fp32 sum, rounded once to the 16-bit
// type, exactly what a 16-bit linear layer hands to the router), then route_token.  One CTA of 8 warps handles
// kTokPerCta tokens (the gate weights are read once per CTA, 16-byte loads, lanes along h), the logits meet in shared
// memory, then warp t routes token t.  Meant for decode batches; the gate matrix (E x H) stays in L2.
constexpr int kTokPerCta = 4;

template <int WT>
__global__ void __launch_bounds__(256) router_gemm_kernel(const void* __restrict__ xin, const void* __restrict__ wg,
                                                          int score_fun, int T, int H, int E, int G, int KG,
                                                          int32_t* __restrict__ ids, void* __restrict__ wts, int topk,
                                                          const void* __restrict__ bias, int renormalize,
                                                          void* __restrict__ logits_out) {
    extern __shared__ float sm[];
    float* slog = sm;                                   // [kTokPerCta][E]
    float* scratch = sm + kTokPerCta * E;               // [kTokPerCta][E + 2 * G]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t0 = blockIdx.x * kTokPerCta;
    const int nt = min(kTokPerCta, T - t0);
    pdl_wait();
    pdl_launch_dependents();
    // Every warp owns one eighth of h for all experts and all of the CTA's tokens: its activations stay in registers,
    // and the loads of the gate rows of different experts are independent, so many are in flight at once.  Partial
    // dot products meet in shared memory (one row of E sums per warp and token), then are added in warp order.
    const uint4* x4 = reinterpret_cast<const uint4*>(xin);
    const uint4* w4 = reinterpret_cast<const uint4*>(wg);
    const int h8 = H >> 3;
    float* part = scratch;                               // [8 warps][kTokPerCta][E] (routing scratch is used later)
    constexpr int EB = 16;                               // experts per pass: EB independent gate-row loads per lane
    for (int e0 = 0; e0 < E; e0 += EB) {
        float acc[EB][kTokPerCta];
#pragma unroll
        for (int j = 0; j < EB; ++j)
#pragma unroll
            for (int t = 0; t < kTokPerCta; ++t) acc[j][t] = 0.f;
        for (int u = warp * 32 + lane; u < h8; u += 256) {
            float2 xv[kTokPerCta][4];
#pragma unroll
            for (int t = 0; t < kTokPerCta; ++t) {
                const uint4 v = (t < nt) ? x4[(size_t)(t0 + t) * h8 + u] : make_uint4(0, 0, 0, 0);
                xv[t][0] = unpack2<WT>(v.x); xv[t][1] = unpack2<WT>(v.y); xv[t][2] = unpack2<WT>(v.z); xv[t][3] = unpack2<WT>(v.w);
            }
            uint4 wv[EB];
#pragma unroll
            for (int j = 0; j < EB; ++j) wv[j] = (e0 + j < E) ? w4[(size_t)(e0 + j) * h8 + u] : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int j = 0; j < EB; ++j) {
                {
                    const uint4 w = wv[j];
                    const float2 w0 = unpack2<WT>(w.x), w1 = unpack2<WT>(w.y), w2 = unpack2<WT>(w.z), w3 = unpack2<WT>(w.w);
#pragma unroll
                    for (int t = 0; t < kTokPerCta; ++t) {
                        float a = acc[j][t];
                        a = fmaf(w0.x, xv[t][0].x, a); a = fmaf(w0.y, xv[t][0].y, a); a = fmaf(w1.x, xv[t][1].x, a); a = fmaf(w1.y, xv[t][1].y, a);
                        a = fmaf(w2.x, xv[t][2].x, a); a = fmaf(w2.y, xv[t][2].y, a); a = fmaf(w3.x, xv[t][3].x, a); a = fmaf(w3.y, xv[t][3].y, a);
                        acc[j][t] = a;
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < EB; ++j)
#pragma unroll
            for (int t = 0; t < kTokPerCta; ++t) {
                const float v = warp_sum(acc[j][t]);
                if (lane == 0 && e0 + j < E) part[(warp * kTokPerCta + t) * E + e0 + j] = v;
            }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nt * E; i += blockDim.x) {
        const int t = i / E, e = i - t * E;
        float v = part[t * E + e];
#pragma unroll
        for (int w = 1; w < 8; ++w) v += part[(w * kTokPerCta + t) * E + e];
        v = round16<WT>(v);
        slog[t * E + e] = v;
        if (logits_out != nullptr) {
            if constexpr (WT == kFP16)
                reinterpret_cast<__half*>(logits_out)[(size_t)(t0 + t) * E + e] = __float2half_rn(v);
            else
                reinterpret_cast<__nv_bfloat16*>(logits_out)[(size_t)(t0 + t) * E + e] = __float2bfloat16_rn(v);
        }
    }
    __syncthreads();
    if (warp < nt) {
        float x[kVPT];
#pragma unroll
        for (int i = 0; i < kVPT; ++i) {
            const int e = lane + 32 * i;
            x[i] = (e < E) ? slog[warp * E + e] : -INFINITY;
        }
        float* ssel = scratch + warp * (E + 2 * G);
        float* sg = ssel + E;
        int* gmask = reinterpret_cast<int*>(sg + G);
        route_token<WT>(x, t0 + warp, lane, score_fun, E, G, KG, ids, wts, topk, bias, renormalize, ssel, sg, gmask);
    }
}

}  // namespace

int launch_router_gemm(const void* x, const void* gate_weight, int score_fun, int T, int H, int E, int n_groups,
                       int topk_groups, int32_t* experts_ids, void* weights, int topk, const void* bias, int dtype,
                       int renormalize, void* logits_out, cudaStream_t s) {
    if (!x || !gate_weight || !experts_ids || !weights) return fail(kInvalidArg, "fused_router_gemm_gate: null pointer");
    if (T < 0) return fail(kInvalidArg, "fused_router_gemm_gate: negative batch size");
    if (T == 0) return kOk;
    if (H <= 0 || H % 8 != 0) return fail(kInvalidArg, "fused_router_gemm_gate: hidden size must be a positive multiple of 8 (got %d)", H);
    if (((uintptr_t)x & 15) || ((uintptr_t)gate_weight & 15)) return fail(kInvalidArg, "fused_router_gemm_gate: x and the gate weight must be 16-byte aligned");
    if (score_fun != 0 && score_fun != 1) return fail(kInvalidArg, "fused_router_gemm_gate: score_fun must be 0 (softmax) or 1 (sigmoid)");
    if (E <= 0 || E > 32 * kVPT) return fail(kUnsupported, "fused_router_gemm_gate: 1 <= num_experts <= 256 (got %d)", E);
    if (n_groups <= 0 || E % n_groups != 0) return fail(kInvalidArg, "fused_router_gemm_gate: n_groups=%d must divide num_experts=%d", n_groups, E);
    if (topk_groups <= 0 || topk_groups > n_groups) return fail(kInvalidArg, "fused_router_gemm_gate: topK_groups=%d out of range", topk_groups);
    if (topk <= 0 || topk > 32 || topk > E) return fail(kInvalidArg, "fused_router_gemm_gate: topK=%d out of range (1..min(32,E))", topk);
    if (dtype != 0 && dtype != 1) return fail(kInvalidArg, "fused_router_gemm_gate: activations must be bf16 or fp16");
    const int grid = (T + kTokPerCta - 1) / kTokPerCta;
    // logits [tokens][E] + the larger of the per-warp partial sums [8][tokens][E] and the routing scratch
    const size_t smem = (size_t)kTokPerCta * (E + std::max(8 * E, E + 2 * n_groups)) * sizeof(float);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = launch_attrs(attr, 1);
    cudaError_t e;
    if (dtype == 1)
        e = cudaLaunchKernelEx(&cfg, router_gemm_kernel<kFP16>, x, gate_weight, score_fun, T, H, E, n_groups, topk_groups,
                               experts_ids, weights, topk, bias, renormalize, logits_out);
    else
        e = cudaLaunchKernelEx(&cfg, router_gemm_kernel<kBF16>, x, gate_weight, score_fun, T, H, E, n_groups, topk_groups,
                               experts_ids, weights, topk, bias, renormalize, logits_out);
    if (e != cudaSuccess) return fail(kCudaError, "fused_router_gemm_gate launch: %s", cudaGetErrorString(e));
    return kOk;
}

int launch_router(const void* gating_output, int score_fun, int T, int E, int n_groups, int topk_groups,
                  int32_t* experts_ids, void* weights, int topk, const void* bias, int dtype, cudaStream_t s,
                  int renormalize) {
    if (!gating_output || !experts_ids || !weights) return fail(kInvalidArg, "fused_routing_gate: null pointer");
    if (T < 0) return fail(kInvalidArg, "fused_routing_gate: negative batch size");
    if (T == 0) return kOk;
    if (score_fun != 0 && score_fun != 1) return fail(kInvalidArg, "fused_routing_gate: score_fun must be 0 (softmax) or 1 (sigmoid)");
    if (E <= 0 || E > 32 * kVPT) return fail(kUnsupported, "fused_routing_gate: 1 <= num_experts <= 256 (got %d)", E);
    if (n_groups <= 0 || E % n_groups != 0) return fail(kInvalidArg, "fused_routing_gate: n_groups=%d must divide num_experts=%d", n_groups, E);
    if (topk_groups <= 0 || topk_groups > n_groups) return fail(kInvalidArg, "fused_routing_gate: topK_groups=%d out of range", topk_groups);
    if (topk <= 0 || topk > 32 || topk > E) return fail(kInvalidArg, "fused_routing_gate: topK=%d out of range (1..min(32,E))", topk);
    if (dtype != 0 && dtype != 1) return fail(kInvalidArg, "fused_routing_gate: gating_output must be bf16 or fp16");
    const int warps = 4;
    const int grid = (T + warps - 1) / warps;
    const size_t smem = (size_t)warps * (E + 2 * n_groups) * sizeof(float);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(warps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = launch_attrs(attr, 1);
    const cudaError_t e = dtype == 1 ? cudaLaunchKernelEx(&cfg, router_kernel<kFP16>, gating_output, score_fun, T, E, n_groups, topk_groups,
                                                          experts_ids, weights, topk, bias, renormalize)
                                     : cudaLaunchKernelEx(&cfg, router_kernel<kBF16>, gating_output, score_fun, T, E, n_groups, topk_groups,
                                                          experts_ids, weights, topk, bias, renormalize);
    if (e != cudaSuccess) return fail(kCudaError, "fused_routing_gate launch: %s", cudaGetErrorString(e));
    return kOk;
}

}  // namespace mlk
