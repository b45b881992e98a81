// Device-side building blocks shared by every kernel of the library (sm_100a only).
//
// Conventions used throughout:
//   * "layout A" is the prepacked weight order [m/16][k/8][16 rows][8 elems]; a 16-row group's
//     whole K extent is one contiguous run (reference: benchmark_and_test/gemm_benchmark.py:41-42).
//   * Warp-level tensor-core tiles are mma.sync m16n8k16 with fp32 accumulators.  Lane l is
//     (g = l >> 2, t = l & 3).  Weights are the 16-row operand, tokens the 8-column operand.
//   * The contraction index inside one 32-element K chunk is permuted identically for both
//     operands (lane t owns k-octet 4c+t), so one 16-byte load per lane feeds two MMAs and
//     neither operand needs a shuffle.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "status.h"

namespace mlk {


// ---------------------------------------------------------------------------------------------
// Global / shared memory access
// ---------------------------------------------------------------------------------------------

// 16-byte streaming load of weight bytes: read-only path, not kept in L1 (each weight byte is
// used exactly once per launch).
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

// The same with an L2 eviction policy created once by the caller (createpolicy): weights are read once, their lines
// are first to leave the L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint4 ldg_stream16_pol(const void* p, uint64_t pol) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p), "l"(pol));
    return r;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint4 lds16(uint32_t addr) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "r"(addr));
    return r;
}

// 16-byte asynchronous global->shared copy.  src_bytes == 0 writes zeros (used for K tails).
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
                 "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Tensor-core tile: D(16x8,f32) += A(16x16) * B(16x8)
// ---------------------------------------------------------------------------------------------
template <int WT>
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    if constexpr (WT == kFP16) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

// ---------------------------------------------------------------------------------------------
// Soft-FP8: two e4m3 bytes -> one packed bf16x2 register, exact.
//
// The reference decodes by placing the 7 exponent/mantissa bits at bits 26..20 of an fp32
// pattern and multiplying by 2^120 (csrc/utils.cuh:232-251).  The same idea in packed 16-bit
// form: put s at bit 15 and eeeemmm at bits 10..4 of each half (a bf16 whose exponent field is
// 0000eeee), then one packed multiply by 2^120 re-biases the exponent (7 -> 127) and normalises
// e4m3 subnormals.  The result is the exact bf16 value of the e4m3 number.
//
// `sel` picks which two bytes of the 32-bit word go to the (low, high) half; that is the only
// place where the byte order produced by fp8_weight_repack differs from natural order.
// ---------------------------------------------------------------------------------------------
constexpr uint32_t kSelNat01 = 0x4140;  // natural order: bytes 0,1
constexpr uint32_t kSelNat23 = 0x4342;  // natural order: bytes 2,3
constexpr uint32_t kSelRep01 = 0x4240;  // "1324" repacked word [b0,b2,b1,b3]: elements 0,1
constexpr uint32_t kSelRep23 = 0x4341;  // repacked: elements 2,3

constexpr uint32_t kRebias2 = 0x7B807B80u;   // 2^120 in both halves

// The same decode with the re-biasing factor supplied by the caller: `c2` holds one bf16 in both halves.  With
// c2 = 2^120 the result is the exact value.
__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2_by(uint32_t w, uint32_t sel, uint32_t c2) {
    uint32_t v = __byte_perm(w, 0u, sel);        // [b_lo, 0, b_hi, 0]
    uint32_t x = (v << 4) + 0x78007800u;         // carries the sign from bit 11 up to bit 15
    x &= 0x87F087F0u;                            // s0000eeeemmm0000 per half
    uint32_t r;
    asm("mul.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(x), "r"(c2));
    return r;
}

__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2(uint32_t w, uint32_t sel) {
    return e4m3x2_to_bf16x2_by(w, sel, kRebias2);   // * 2^120, exact
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// Block-scaled decode.  The scale s of a 128 x 128 block enters the packed arithmetic of the decode in one of two forms:
//   one term   bf16(s) folded into the re-biasing factor: rne_bf16(value * bf16(s)), the same instruction count as
//              the unscaled decode;
//   two terms  s = hi + lo in bf16 (16 significant bits): value * hi is exact inside the fused multiply-add (4 x 8
//              bits), value * lo is a correction below half an ulp of the result, so the sum is rne_bf16(value * s)
//              up to a 2^-17 relative slip of the rounding boundary: the number the reference's torch check
//              dequantises to (muxi_layout_kernels/utils.py:14-25).
// The reference's kernels truncate fp32(value) * s to bf16; all forms are within one bf16 ulp of the exact product.
struct ScaledRebias {
    uint32_t pre2;         // first factor, both halves: 2^120 (exact decode) or 1.0 when 2^120 is folded into hi/lo
    uint32_t hi2, lo2;     // the two terms of the scale, both halves
    bool one_multiply;     // value = raw * hi2 is all there is to do
};

__device__ __forceinline__ ScaledRebias scaled_rebias(float s, bool two_terms) {
    const __nv_bfloat16 h = __float2bfloat16_rn(s);
    const float rest = (two_terms && fabsf(s) <= 3.0e38f) ? s - __bfloat162float(h) : 0.f;
    const __nv_bfloat16 l = __float2bfloat16_rn(rest);
    const uint32_t hb = (uint32_t)__bfloat16_as_ushort(h), lb = (uint32_t)__bfloat16_as_ushort(l);
    const uint32_t he = (hb >> 7) & 0xFFu, le = (lb >> 7) & 0xFFu;
    const bool lzero = (lb & 0x7FFFu) == 0u;
    // multiplying a normal bf16 by 2^120 adds 120 to its exponent field; terms that leave the normal range that way
    // (|s| >= 256, zero, subnormal) are applied after an exact decode instead
    const bool folded = he >= 1u && he < 127u + 8u && (le >= 1u || lzero);
    const uint32_t hx = folded ? hb + (120u << 7) : hb;
    const uint32_t lx = (folded && le >= 1u) ? lb + (120u << 7) : lb;
    ScaledRebias r;
    r.pre2 = folded ? 0x3F803F80u : kRebias2;
    r.hi2 = hx | (hx << 16);
    r.lo2 = lx | (lx << 16);
    r.one_multiply = folded && lzero;
    return r;
}

// general form: (raw * pre) * hi + (raw * pre) * lo, three packed operations
__device__ __forceinline__ uint32_t e4m3x2_scaled(uint32_t w, uint32_t sel, const ScaledRebias& r) {
    const uint32_t e = e4m3x2_to_bf16x2_by(w, sel, r.pre2);
    return fma_bf16x2(e, r.hi2, mul_bf16x2(e, r.lo2));
}

// ---------------------------------------------------------------------------------------------
// 16-bit <-> fp32 helpers
// ---------------------------------------------------------------------------------------------
template <int WT>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if constexpr (WT == kFP16) {
        __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    } else {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
}

template <int WT>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
    if constexpr (WT == kFP16) {
        return __half22float2(*reinterpret_cast<__half2*>(&w));
    } else {
        // bf16 -> fp32 is a 16-bit shift
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
    }
}

template <int WT>
__device__ __forceinline__ float load_scalar16(const void* base, int64_t idx) {
    if constexpr (WT == kFP16) {
        return __half2float(reinterpret_cast<const __half*>(base)[idx]);
    } else {
        return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
    }
}

template <int WT>
__device__ __forceinline__ float round16(float v) {
    if constexpr (WT == kFP16) {
        return __half2float(__float2half_rn(v));
    } else {
        return __bfloat162float(__float2bfloat16_rn(v));
    }
}

// Programmatic dependent launch: lets the next kernel of the stream become resident while this one drains.
// wait() returns once every kernel this launch depends on has completed and its writes are visible; nothing
// produced by an earlier kernel may be read, and nothing may be written, before it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

}  // namespace mlk
