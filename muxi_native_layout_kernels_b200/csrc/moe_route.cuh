// Routing of one token by one warp: score function + optional selection bias + group-limited top-k.  Shared by the
// stand-alone router kernels (moe_router.cu) and the single-kernel decode path (moe_decode.cu).
//
// Semantics follow the reference's torch formulation (muxi_layout_kernels/utils.py:160-216) with the tie rule of its
// device kernel (csrc/moe_kernels/fused_topK.h:255-262, "lower id wins"); moe_router.cu states them in full.
#pragma once

#include "common.cuh"

namespace mlk {

constexpr int kVPT = 8;   // experts per lane, strided: e = lane + 32*i

__device__ __forceinline__ void argmax_pair(float& v, int& e) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, v, o);
        const int oe = __shfl_xor_sync(0xFFFFFFFFu, e, o);
        if (ov > v || (ov == v && oe < e)) { v = ov; e = oe; }
    }
}

// Routing of one token by one warp.  x[i] = logit of expert lane + 32*i (already a value of the 16-bit type, -inf
// beyond E); ssel / sg / gmask: this warp's scratch of E + 2*G floats in shared memory.
template <int WT>
__device__ __forceinline__ void route_token(const float (&x)[kVPT], int row, int lane, int score_fun, int E, int G, int KG,
                                            int32_t* __restrict__ ids, void* __restrict__ wts, int topk,
                                            const void* __restrict__ bias, int renormalize, float* ssel, float* sg,
                                            int* gmask) {
    const float NEG = -INFINITY;
    float score[kVPT], sel[kVPT];
    if (score_fun == 0) {
        float mx = x[0];
#pragma unroll
        for (int i = 1; i < kVPT; ++i) mx = fmaxf(mx, x[i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < kVPT; ++i) {
            const int e = lane + 32 * i;
            score[i] = (e < E) ? expf(x[i] - mx) : 0.f;
            sum += score[i];
        }
        sum = warp_sum(sum);
#pragma unroll
        for (int i = 0; i < kVPT; ++i) score[i] = round16<WT>(__fdiv_rn(score[i], sum));
    } else {
#pragma unroll
        for (int i = 0; i < kVPT; ++i) score[i] = round16<WT>(__fdiv_rn(1.f, 1.f + expf(-x[i])));
    }
#pragma unroll
    for (int i = 0; i < kVPT; ++i) {
        const int e = lane + 32 * i;
        if (e < E) {
            sel[i] = (bias != nullptr) ? round16<WT>(score[i] + load_scalar16<WT>(bias, e)) : score[i];
        } else {
            sel[i] = NEG;
        }
    }

    if (G > 1) {
        const int gs = E / G;
#pragma unroll
        for (int i = 0; i < kVPT; ++i) {
            const int e = lane + 32 * i;
            if (e < E) ssel[e] = sel[i];
        }
        __syncwarp();
        for (int gi = lane; gi < G; gi += 32) {
            float m1 = NEG, m2 = NEG;
            for (int j = 0; j < gs; ++j) {
                const float v = ssel[gi * gs + j];
                if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) { m2 = v; }
            }
            sg[gi] = (bias != nullptr && gs > 1) ? round16<WT>(m1 + m2) : m1;
            gmask[gi] = 0;
        }
        __syncwarp();
        for (int r = 0; r < KG; ++r) {
            float bv = NEG;
            int bg = 0x7FFFFFFF;
            for (int gi = lane; gi < G; gi += 32) {
                if (gmask[gi]) continue;
                const float v = sg[gi];
                if (v > bv || bg == 0x7FFFFFFF) { bv = v; bg = gi; }
            }
            argmax_pair(bv, bg);
            __syncwarp();
            if (lane == 0 && bg < G) gmask[bg] = 1;
            __syncwarp();
        }
#pragma unroll
        for (int i = 0; i < kVPT; ++i) {
            const int e = lane + 32 * i;
            if (e < E && !gmask[e / gs]) sel[i] = 0.f;
        }
    }

    int my_id = 0x7FFFFFFF;
    float my_w = 0.f;
    for (int r = 0; r < topk; ++r) {
        float bv = NEG;
        int be = 0x7FFFFFFF;
#pragma unroll
        for (int i = 0; i < kVPT; ++i) {
            const int e = lane + 32 * i;
            if (e < E && (sel[i] > bv || be == 0x7FFFFFFF)) { bv = sel[i]; be = e; }
        }
        argmax_pair(bv, be);
        const int owner = be & 31, oi = be >> 5;
        float sc = 0.f;
#pragma unroll
        for (int i = 0; i < kVPT; ++i) {
            if (i == oi) {
                sc = score[i];
                if (lane == owner) sel[i] = NEG;
            }
        }
        sc = __shfl_sync(0xFFFFFFFFu, sc, owner);
        if (lane == r) { my_id = be; my_w = sc; }
    }
    if (renormalize) {
        // w / sum(w) in the logits' dtype, as torch evaluates `w / w.sum(-1, keepdim=True)` on a 16-bit tensor:
        // fp32 sum rounded to 16 bits, fp32 quotient rounded to 16 bits
        const float s16 = round16<WT>(warp_sum(lane < topk ? my_w : 0.f));
        my_w = round16<WT>(__fdiv_rn(my_w, s16));
    }
    int pos = lane;
    if (score_fun == 0) {
        pos = 0;
        for (int j = 0; j < topk; ++j) {
            const int idj = __shfl_sync(0xFFFFFFFFu, my_id, j);
            pos += (idj < my_id) ? 1 : 0;
        }
    }
    if (lane < topk) {
        ids[(int64_t)row * topk + pos] = my_id;
        if constexpr (WT == kFP16)
            reinterpret_cast<__half*>(wts)[(int64_t)row * topk + pos] = __float2half_rn(my_w);
        else
            reinterpret_cast<__nv_bfloat16*>(wts)[(int64_t)row * topk + pos] = __float2bfloat16_rn(my_w);
    }
}

}  // namespace mlk
