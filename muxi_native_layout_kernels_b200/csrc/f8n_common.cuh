// Pieces shared by the kernels that hand e4m3 weights to the tensor cores undecoded (tcgen05.mma.kind::f8f6f4):
// the split of bf16 activations into two e4m3 terms, the kernel that prepares a batch of activation rows that way,
// and the PTX wrappers of the 8-bit MMA.
//
// Why a split: a bf16 activation x has 8 significant bits, an e4m3 number 4.  After an exact scaling by a power of
// two, x * 2^s = hi + lo with hi = x * 2^s truncated to 4 significant bits and lo the remainder (at most 4 significant
// bits): two e4m3 operands whose products with an e4m3 weight add up to the exact product x * w * 2^s in the fp32
// accumulator.  Two MMAs per 32-wide k step instead of one bf16 MMA per 16-wide step: the tensor-pipe time of the
// bf16 kernels, and no instruction at all spent on the weight bytes.
//   * The scale 2^s is chosen per row (token) from the largest magnitude of the row, so that hi stays below the e4m3
//     maximum (448) for any finite input: scaled row maximum in [128, 256).  Elements more than 2^11 below their row
//     maximum lose low bits against the e4m3 subnormal grid (2^-9): an absolute error of at most 2^-17 of the row
//     maximum per element, three orders of magnitude below the bf16 rounding of a result.  The inverse scale is applied
//     to the fp32 sums in the epilogue of the GEMM.
//   * A row that holds an Inf or a NaN yields NaN operands, hence NaN results for that token.
//   * An e4m3 NaN encoding (0x7F, 0xFF) in the weights is a NaN for the tensor core, as it is for the reference's torch
//     recipe (weight.to(bf16)); the reference's bit-trick kernels and the decode kernels of this library read those
//     two bytes as +-480.
//
// Prepared activations ("split planes"): one row of 2 * K bytes per activation row; every 64-wide k block is 128 bytes,
// the 64 hi bytes followed by the 64 lo bytes, so that one TMA box of 128 bytes x NP rows with the 128-byte swizzle
// delivers both K-major operand tiles of that k block.  With weights that went through fp8_weight_repack the bytes of
// every group of four are stored in the order [0, 2, 1, 3], the order of the weight bytes.
#pragma once

#include "umma_common.cuh"

namespace mlk {
namespace f8n {

__device__ __forceinline__ void umma_f8_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}

// D = f32, A = B = e4m3 (format code 0), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
template <int NP>
constexpr uint32_t instr_desc_f8() {
    return (1u << 4) | ((uint32_t)(NP >> 3) << 17) | ((uint32_t)(umma::kTileM >> 4) << 24);
}

// two fp32 -> two e4m3 bytes (round to nearest, saturating): `lo` in bits 0..7, `hi` in bits 8..15
__device__ __forceinline__ uint32_t cvt_e4m3x2(float hi, float lo) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return (uint32_t)r;
}

// Eight bf16 activations (one 16-byte chunk) times the power of two `f` -> eight hi bytes and eight lo bytes (e4m3), in
// k order or, for repacked weights, in the order [0,2,1,3] of every group of four.
__device__ __forceinline__ void split_chunk(const uint4 raw, float f, int repacked, uint2& hi8, uint2& lo8) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float a = __uint_as_float(w[i] << 16) * f, b = __uint_as_float(w[i] & 0xFFFF0000u) * f;
        const float ah = __uint_as_float(__float_as_uint(a) & 0xFFF00000u), bh = __uint_as_float(__float_as_uint(b) & 0xFFF00000u);
        h[i] = cvt_e4m3x2(bh, ah);
        l[i] = cvt_e4m3x2(b - bh, a - ah);
    }
    // h[0] = elements 0,1; h[1] = 2,3: natural word = h[0] | h[1] << 16; repacked word = bytes [e0, e2, e1, e3]
    const uint32_t sel = repacked ? 0x5140u : 0x5410u;
    hi8.x = __byte_perm(h[0], h[1], sel);
    hi8.y = __byte_perm(h[2], h[3], sel);
    lo8.x = __byte_perm(l[0], l[1], sel);
    lo8.y = __byte_perm(l[2], l[3], sel);
}

// Power-of-two scale of a row from its largest magnitude, given as the bf16 bit pattern of |x| (a NaN pattern, larger
// than every finite one, stands for "the row holds a NaN"): scaled maximum in [128, 256); 1 for an all-zero row.
// A non-finite maximum gives a tiny scale; the Inf / NaN elements themselves become NaN operands.
__device__ __forceinline__ float row_scale_from_bits(uint32_t amax_bf16_bits) {
    const uint32_t e = (amax_bf16_bits >> 7) & 0xFFu;      // biased exponent
    if (e == 0u) return 1.f;                               // zero (a row of bf16 subnormals is left as it is)
    // 2^(7 - (e - 127)) = 2^(134 - e): biased exponent 261 - e, clamped to the normal range
    int be = 261 - (int)e;
    be = be < 1 ? 1 : (be > 254 ? 254 : be);
    return __uint_as_float((uint32_t)be << 23);
}

// Work of one CTA on one activation row: largest magnitude of the row -> its scale -> split planes.
//   xr        the row: k bf16 elements (k % 64 == 0, k <= kSplitMaxK), 16-byte aligned; zero_row: treat it as all zeros
//             (nothing is read)
//   out       2 k bytes of split planes as described at the top of this file; may be the row itself (the row is read
//             completely into registers before anything is written)
//   inv_scale where to store what the fp32 sums of this row have to be multiplied by
// Every thread of the CTA must call it (it synchronises the CTA); blockDim.x * kSplitChunks >= k / 8, blockDim.x <= 512.
constexpr int kSplitChunks = 8;                       // 16-byte chunks a thread keeps in registers
constexpr int kSplitMaxK = 8 * kSplitChunks * 512;    // 32768

__device__ __forceinline__ void split_row_cta(const uint4* xr, bool zero_row, int k, int repacked, uint8_t* out,
                                              float* inv_scale) {
    const int chunks = k >> 3;
    uint4 v[kSplitChunks];
    uint32_t m = 0;          // largest |x| as bf16 bits; a NaN (> 0x7F80) wins every comparison
#pragma unroll
    for (int r = 0; r < kSplitChunks; ++r) {
        const int c = threadIdx.x + r * blockDim.x;
        v[r] = make_uint4(0u, 0u, 0u, 0u);
        if (c < chunks && !zero_row) {
            asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v[r].x), "=r"(v[r].y), "=r"(v[r].z), "=r"(v[r].w) : "l"(xr + c));
            const uint32_t w[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                m = max(m, w[i] & 0x7FFFu);
                m = max(m, (w[i] >> 16) & 0x7FFFu);
            }
        }
    }
    m = __reduce_max_sync(0xFFFFFFFFu, m);
    __shared__ uint32_t wm[16];
    __shared__ float scale_s;
    if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
    __syncthreads();          // also: every load of the row has completed before the first store below
    if (threadIdx.x == 0) {
        for (int i = 1; i < (int)(blockDim.x >> 5); ++i) m = max(m, wm[i]);
        const float sc = row_scale_from_bits(m);
        scale_s = sc;
        *inv_scale = 1.f / sc;       // exact: a power of two
    }
    __syncthreads();
    const float sc = scale_s;
#pragma unroll
    for (int r = 0; r < kSplitChunks; ++r) {
        const int c = threadIdx.x + r * blockDim.x;
        if (c < chunks) {
            uint2 hi8, lo8;
            split_chunk(v[r], sc, repacked, hi8, lo8);
            // chunk c = k elements 8c .. 8c+7: k block c / 8, bytes 8 (c % 8) .. of its hi half; the lo half 64 bytes on
            uint8_t* const dst = out + (c >> 3) * 128 + (c & 7) * 8;
            *reinterpret_cast<uint2*>(dst) = hi8;
            *reinterpret_cast<uint2*>(dst + 64) = lo8;
        }
    }
}

// The same for one row per WARP (k <= 32 * 8 * kSplitChunks = 2048): no CTA barrier, all of the row's loads in flight
// at once, one warp-wide maximum.  Every lane of the warp must call it.
constexpr int kSplitWarpMaxK = 32 * 8 * kSplitChunks;

__device__ __forceinline__ void split_row_warp(const uint4* xr, int k, int repacked, uint8_t* out, float* inv_scale) {
    const int chunks = k >> 3;
    const int lane = threadIdx.x & 31;
    uint4 v[kSplitChunks];
    uint32_t m = 0;
#pragma unroll
    for (int r = 0; r < kSplitChunks; ++r) {
        const int c = lane + r * 32;
        v[r] = make_uint4(0u, 0u, 0u, 0u);
        if (c < chunks)
            asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v[r].x), "=r"(v[r].y), "=r"(v[r].z), "=r"(v[r].w) : "l"(xr + c));
    }
#pragma unroll
    for (int r = 0; r < kSplitChunks; ++r) {
        const uint32_t w[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            m = max(m, w[i] & 0x7FFFu);
            m = max(m, (w[i] >> 16) & 0x7FFFu);
        }
    }
    m = __reduce_max_sync(0xFFFFFFFFu, m);      // also: every lane's loads of the row have completed (in-place use)
    const float sc = row_scale_from_bits(m);
    if (lane == 0) *inv_scale = 1.f / sc;       // exact: a power of two
#pragma unroll
    for (int r = 0; r < kSplitChunks; ++r) {
        const int c = lane + r * 32;
        if (c < chunks) {
            uint2 hi8, lo8;
            split_chunk(v[r], sc, repacked, hi8, lo8);
            uint8_t* const dst = out + (c >> 3) * 128 + (c & 7) * 8;
            *reinterpret_cast<uint2*>(dst) = hi8;
            *reinterpret_cast<uint2*>(dst + 64) = lo8;
        }
    }
}

// CTA size for rows of k elements: a multiple of 32 with kSplitChunks chunks per thread at most
inline int split_threads(int k) {
    const int chunks = k / 8;
    int t = (chunks + kSplitChunks - 1) / kSplitChunks;
    t = (t + 31) / 32 * 32;
    if (t < 64) t = 64;
    return t > 512 ? 512 : t;
}

// Split planes as a TMA operand: 2-D view (2 k bytes per row, rows), box (128 bytes, np rows), 128-byte swizzle: the
// box of k block b of rows r0 .. r0 + np - 1 lands as the K-major SW128 tile [np][hi 64 | lo 64]; rows beyond `rows`
// read as zero.
inline bool make_map_planes(CUtensorMap* map, const void* planes, long long rows, int k, int np) {
    return umma::cached_map(map, 7, planes, rows, k, np, [&](CUtensorMap* m) {
        const cuuint64_t dims[2] = {(cuuint64_t)2 * k, (cuuint64_t)rows};
        const cuuint64_t strides[1] = {(cuuint64_t)2 * k};
        const cuuint32_t box[2] = {128, (cuuint32_t)np};
        const cuuint32_t estr[2] = {1, 1};
        return umma::encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(planes), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    });
}

// e4m3 weight tile map for stages of bk weight bytes per row: global layout A is [row group][k-octet][16 rows][8 bytes];
// the 3-D view (128-byte block, k-octet, row group) with box (128, bk / 8, 8) lands a 128 x bk tile as
// [row group][k-octet][16 rows x 8 bytes].  `rows` may span several matrices stored back to back.
inline bool make_map_a8_bk(CUtensorMap* map, const void* A, long long rows, int k, int bk) {
    return umma::cached_map(map, 5, A, rows, k, bk, [&](CUtensorMap* mp) {
        const cuuint64_t dims[3] = {128, (cuuint64_t)(k / 8), (cuuint64_t)(rows / 16)};
        const cuuint64_t strides[2] = {128, (cuuint64_t)16 * k};
        const cuuint32_t box[3] = {128, (cuuint32_t)(bk / 8), umma::kTileM / 16};
        const cuuint32_t estr[3] = {1, 1, 1};
        return umma::encode_fn()(mp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(A), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    });
}

}  // namespace f8n
}  // namespace mlk
