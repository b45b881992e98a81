// Weight-streaming tensor-core core shared by the dense (GeMV / narrow GEMM) and MoE kernels.
//
// One CTA owns `16*RG*WM` weight rows.  Its warps are arranged WM (rows) x WK (K split); a
// cluster of SK such CTAs splits K once more.  Every warp streams the layout-A bytes of its
// RG row groups straight from global memory into MMA operand registers (16-byte loads, no
// shared-memory staging: that is what the native layout buys), while the small token tile is
// staged through shared memory with cp.async and shared by the WM row warps.
//
// Reference kernels with the same role: GemmMmaJustLayoutAKernel (csrc/gemm_layout_A.cu:20),
// MvMmaLayoutKernel (csrc/layout_gemv_kernel.cuh:19), fused_moe_first/second_group_gemm_kernel
// (csrc/moe_kernels/group_gemm_first.h:355, group_gemm_second.h:356).  Those use 64-lane warps,
// 16x16x16 MMAs and 16-bit atomics for split-K; here split-K partial sums stay fp32 and are
// reduced in a fixed order through (distributed) shared memory, so results are reproducible.
#pragma once

#include <cooperative_groups.h>

#include "common.cuh"

namespace mlk {

namespace cg = cooperative_groups;

constexpr int kMaxWarps = 8;     // 256 threads per CTA at most
constexpr int kTokBlock = 64;    // tokens handled by one CTA pass (NT <= 8 tiles of 8)

template <int NT, int RG>
struct CoreShape {
    // K chunks (32 elements each) kept in flight per warp = chunks per shared-memory stage.
    static constexpr int CH = (NT * RG <= 2) ? 8 : 4;
    static constexpr int NTP = NT * 8;          // padded token count
    static constexpr int PITCH = CH * 64;       // bytes of one token row in a stage
    static constexpr int UNITS = CH * 4;        // 16-byte units per token row per stage
};

// Per-CTA bookkeeping that lives in static shared memory.
struct CoreShared {
    int c0[kMaxWarps];                 // first chunk of K slice wk
    int c1[kMaxWarps];                 // one past the last chunk of K slice wk
    unsigned long long xrow[kTokBlock];  // global byte address of token row r at k = 0
};

struct CoreArgs {
    const uint8_t* a_lane[2];   // this lane's address for chunk 0 of its K slice, per row group
    const float* scale[2];      // fp8 block scale of this warp's first 128-k block, per row group
    int nchunks;                // chunks this warp owns
    int steps;                  // stage steps, uniform over the CTA
    int nt;                     // valid token rows (<= NT*8)
    int wk, WK;                 // this warp's K slice and the number of K slices in the CTA
    int stages;                 // 2 or 3 shared-memory stages
    uint32_t xs_base;           // shared address of stage 0
    uint32_t stage_bytes;       // bytes per stage = WK * xrows * PITCH
    int xrows;                  // token rows allocated per slice in a stage
    long long cstride;          // global bytes between consecutive 32-k chunks of one token row
    long long qstride;          // global bytes between consecutive k-octets inside a chunk
    uint32_t sel01, sel23;      // e4m3 byte selectors
};

template <int WT>
constexpr int chunk_bytes() { return WT == kE4M3 ? 512 : 1024; }   // per row group, per 32-k chunk

// Stage fill: copies, for every K slice w and token row r, the CH*32 activations of step `s`.
template <int NT, int RG>
__device__ __forceinline__ void fill_stage(const CoreArgs& a, const CoreShared& sh, int s,
                                           int slot) {
    using S = CoreShape<NT, RG>;
    const int total = a.WK * S::NTP * S::UNITS;
    const uint32_t dst0 = a.xs_base + slot * a.stage_bytes;
    for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
        const int u = idx & (S::UNITS - 1);
        const int r = (idx / S::UNITS) & (S::NTP - 1);
        const int w = idx / (S::UNITS * S::NTP);
        if (r >= a.nt) continue;
        const int chunk = sh.c0[w] + s * S::CH + (u >> 2);
        const bool valid = chunk < sh.c1[w];
        const unsigned long long src =
            sh.xrow[r] + (valid ? (unsigned long long)(chunk * a.cstride + (u & 3) * a.qstride) : 0ull);
        const uint32_t dst = dst0 + (w * a.xrows + r) * S::PITCH + ((u ^ ((r & 1) << 2)) << 4);
        cp_async16(dst, reinterpret_cast<const void*>(src), valid ? 16 : 0);
    }
}

// Loads one chunk of weights for row group r of this lane.
template <int WT>
struct AFrag {
    uint4 v[WT == kE4M3 ? 1 : 2];
};

template <int WT>
__device__ __forceinline__ void load_afrag(AFrag<WT>& f, const uint8_t* p, bool valid) {
    if (valid) {
        f.v[0] = ldg_stream16(p);
        if constexpr (WT != kE4M3) f.v[1] = ldg_stream16(p + 128);
    } else {
        f.v[0] = make_uint4(0, 0, 0, 0);
        if constexpr (WT != kE4M3) f.v[1] = make_uint4(0, 0, 0, 0);
    }
}

// Issues the first CH chunks of this lane's weight stream (the prefetch ring).
template <int WT, int NT, int RG>
__device__ __forceinline__ void ring_init(AFrag<WT> (&ring)[CoreShape<NT, RG>::CH][RG], const CoreArgs& a) {
    constexpr int CH = CoreShape<NT, RG>::CH;
    constexpr int CB = chunk_bytes<WT>();
#pragma unroll
    for (int cc = 0; cc < CH; ++cc)
#pragma unroll
        for (int r = 0; r < RG; ++r)
            load_afrag<WT>(ring[cc][r], a.a_lane[r] + (long long)cc * CB, cc < a.nchunks);
}

__device__ __forceinline__ uint4 ldg_cached16(const void* p) {
    uint4 r;
    asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

// The main loop.  acc[r][j] is the 16x8 fp32 tile of row group r and token tile j.
//
// Lane (g,t) addressing inside a 32-k chunk c:
//   16-bit weights: rows g and g+8 of k-octet 4c+t  (two 16-byte loads, 128 bytes apart)
//   e4m3 weights:   rows 2g and 2g+1 of k-octet 4c+t (one 16-byte load); the MMA row index
//                   rho maps to weight row 2*rho (rho < 8) or 2*(rho-8)+1, undone when the
//                   accumulators are written out.
//   tokens:         row 8j+g, k-octet 4c+t (one 16-byte load)
// XDIRECT (NT == 1 only): the token fragments come straight from global memory through L1 with their own
// register ring -- no shared-memory stages and no CTA barrier in the loop, every warp streams on its own.
// Otherwise the token tile is staged through shared memory (cp.async, 2-3 stages) and shared by the row warps.
template <int WT, int NT, int RG, bool SCALE, bool XDIRECT>
__device__ __forceinline__ void stream_mma(float (&acc)[RG][NT][4], AFrag<WT> (&ring)[CoreShape<NT, RG>::CH][RG],
                                           const CoreArgs& a, const CoreShared& sh) {
    using S = CoreShape<NT, RG>;
    constexpr int CH = S::CH;
    constexpr int CB = chunk_bytes<WT>();
    static_assert(!XDIRECT || NT == 1, "direct token loads are for a single token tile");
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

#pragma unroll
    for (int r = 0; r < RG; ++r)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[r][j][i] = 0.f;

    float blk[SCALE ? RG : 1][SCALE ? NT : 1][4];
    float sc[RG];
    if constexpr (SCALE) {
#pragma unroll
        for (int r = 0; r < RG; ++r) {
            sc[r] = 0.f;
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) blk[r][j][i] = 0.f;
        }
    }

    uint4 xring[XDIRECT ? CH : 1];
    const uint8_t* xlane = nullptr;
    if constexpr (XDIRECT) {
        const bool has_row = g < a.nt;
        xlane = has_row ? reinterpret_cast<const uint8_t*>(sh.xrow[g]) + (long long)sh.c0[a.wk] * a.cstride + t * a.qstride
                        : nullptr;
#pragma unroll
        for (int cc = 0; cc < CH; ++cc)
            xring[cc] = (has_row && cc < a.nchunks) ? ldg_cached16(xlane + (long long)cc * a.cstride) : make_uint4(0, 0, 0, 0);
    } else {
        // token-tile prologue
        for (int st = 0; st < a.stages - 1; ++st) {
            if (st < a.steps) fill_stage<NT, RG>(a, sh, st, st);
            cp_async_commit();
        }
    }

    const uint32_t lane_x = ((uint32_t)t ^ ((uint32_t)(g & 1) << 2)) << 4;
    const int steps = XDIRECT ? (a.nchunks + CH - 1) / CH : a.steps;

    for (int s = 0; s < steps; ++s) {
        uint32_t xs = 0;
        if constexpr (!XDIRECT) {
            if (a.stages == 3) cp_async_wait<1>(); else cp_async_wait<0>();
            __syncthreads();
            {
                const int sf = s + a.stages - 1;
                if (sf < a.steps) fill_stage<NT, RG>(a, sh, sf, sf % a.stages);
                cp_async_commit();
            }
            xs = a.xs_base + (s % a.stages) * a.stage_bytes + a.wk * a.xrows * S::PITCH + g * S::PITCH;
        }

#pragma unroll
        for (int cc = 0; cc < CH; ++cc) {
            // token fragments of this chunk
            uint4 xb[NT];
            if constexpr (XDIRECT) {
                xb[0] = xring[cc];
                const int cn = (s + 1) * CH + cc;
                xring[cc] = (xlane != nullptr && cn < a.nchunks) ? ldg_cached16(xlane + (long long)cn * a.cstride)
                                                               : make_uint4(0, 0, 0, 0);
            } else {
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    if (8 * j + g < a.nt) {
                        xb[j] = lds16(xs + j * 8 * S::PITCH + (((uint32_t)cc << 6) ^ lane_x));
                    } else {
                        xb[j] = make_uint4(0, 0, 0, 0);
                    }
                }
            }
            if constexpr (SCALE) {
                if ((cc & 3) == 0) {
                    const int c = s * CH + cc;
#pragma unroll
                    for (int r = 0; r < RG; ++r) sc[r] = (c < a.nchunks) ? __ldg(a.scale[r] + (c >> 2)) : 0.f;
                }
            }
#pragma unroll
            for (int r = 0; r < RG; ++r) {
                uint32_t p0, p1, p2, p3, q0, q1, q2, q3;
                if constexpr (WT == kE4M3) {
                    const uint4 w = ring[cc][r].v[0];
                    p0 = e4m3x2_to_bf16x2(w.x, a.sel01);
                    p1 = e4m3x2_to_bf16x2(w.x, a.sel23);
                    p2 = e4m3x2_to_bf16x2(w.y, a.sel01);
                    p3 = e4m3x2_to_bf16x2(w.y, a.sel23);
                    q0 = e4m3x2_to_bf16x2(w.z, a.sel01);
                    q1 = e4m3x2_to_bf16x2(w.z, a.sel23);
                    q2 = e4m3x2_to_bf16x2(w.w, a.sel01);
                    q3 = e4m3x2_to_bf16x2(w.w, a.sel23);
                } else {
                    const uint4 lo = ring[cc][r].v[0], hi = ring[cc][r].v[1];
                    p0 = lo.x; p1 = lo.y; p2 = lo.z; p3 = lo.w;
                    q0 = hi.x; q1 = hi.y; q2 = hi.z; q3 = hi.w;
                }
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    if constexpr (SCALE) {
                        mma16816<WT>(blk[r][j], p0, q0, p1, q1, xb[j].x, xb[j].y);
                        mma16816<WT>(blk[r][j], p2, q2, p3, q3, xb[j].z, xb[j].w);
                    } else {
                        mma16816<WT>(acc[r][j], p0, q0, p1, q1, xb[j].x, xb[j].y);
                        mma16816<WT>(acc[r][j], p2, q2, p3, q3, xb[j].z, xb[j].w);
                    }
                }
                // refill this ring slot with the chunk CH ahead
                const int cn = (s + 1) * CH + cc;
                load_afrag<WT>(ring[cc][r], a.a_lane[r] + (long long)cn * CB, cn < a.nchunks);
            }
            if constexpr (SCALE) {
                if ((cc & 3) == 3) {
#pragma unroll
                    for (int r = 0; r < RG; ++r)
#pragma unroll
                        for (int j = 0; j < NT; ++j)
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                acc[r][j][i] = fmaf(sc[r], blk[r][j][i], acc[r][j][i]);
                                blk[r][j][i] = 0.f;
                            }
                }
            }
        }
    }
    if constexpr (!XDIRECT) cp_async_wait<0>();
    __syncthreads();   // every warp is done with the token stages: shared memory can be reused
}

// Writes this warp's accumulators into the CTA's partial-sum buffer
//   part[wk][token][PR]   (fp32, PR = rows_cta + 4 to keep the writes bank-conflict free)
// `lrow0[r]` is the CTA-local row index of row group r's first row.
template <int WT, int NT, int RG>
__device__ __forceinline__ void store_partials(float* part, const float (&acc)[RG][NT][4],
                                               int wk, int PR, const int (&lrow0)[RG]) {
    constexpr int NTP = NT * 8;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int ra = (WT == kE4M3) ? 2 * g : g;
    const int rb = (WT == kE4M3) ? 2 * g + 1 : g + 8;
#pragma unroll
    for (int r = 0; r < RG; ++r)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            float* p = part + ((size_t)(wk * NTP + 8 * j + 2 * t)) * PR + lrow0[r];
            p[ra] = acc[r][j][0];
            p[PR + ra] = acc[r][j][1];
            p[rb] = acc[r][j][2];
            p[PR + rb] = acc[r][j][3];
        }
}

// Fixed-order reduction of the partial sums over the CTA's WK slices and the cluster's SK CTAs,
// followed by `emit(token, row_octet, v[NV][8])` exactly once per (token, 8-row octet) of the tile.
// NV = 1: every octet of the tile is emitted on its own.  NV = 2: the tile holds two row planes of
// `plane_rows` rows each (gate rows, then up rows) and octet `ro` of both planes is emitted together.
// Must be called by all threads of all CTAs of the cluster.
struct Oct8 {
    float4 a, b;
};
__device__ __forceinline__ void oct_add(Oct8& o, const float* q) {
    const float4 c = *reinterpret_cast<const float4*>(q);
    const float4 d = *reinterpret_cast<const float4*>(q + 4);
    o.a.x += c.x; o.a.y += c.y; o.a.z += c.z; o.a.w += c.w;
    o.b.x += d.x; o.b.y += d.y; o.b.z += d.z; o.b.w += d.w;
}
__device__ __forceinline__ void oct_unpack(const Oct8& o, float (&v)[8]) {
    v[0] = o.a.x; v[1] = o.a.y; v[2] = o.a.z; v[3] = o.a.w;
    v[4] = o.b.x; v[5] = o.b.y; v[6] = o.b.z; v[7] = o.b.w;
}

template <int NV, class Emit>
__device__ __forceinline__ void reduce_and_emit(float* part, int WK, int NTP, int PR, int nt,
                                                int octets, int plane_rows, int SK, Emit&& emit) {
    __syncthreads();
    const int items = nt * octets;
    const size_t wstride = (size_t)NTP * PR;
    if (SK == 1) {
        for (int it = threadIdx.x; it < items; it += blockDim.x) {
            const int tk = it / octets, ro = it - tk * octets;
            float v[NV][8];
#pragma unroll
            for (int pl = 0; pl < NV; ++pl) {
                const float* p = part + (size_t)tk * PR + pl * plane_rows + ro * 8;
                Oct8 o;
                o.a = *reinterpret_cast<const float4*>(p);
                o.b = *reinterpret_cast<const float4*>(p + 4);
                for (int w = 1; w < WK; ++w) oct_add(o, p + w * wstride);
                oct_unpack(o, v[pl]);
            }
            emit(tk, ro, v);
        }
        return;
    }
    // in-CTA pass: fold the WK slices into slice 0
    if (WK > 1) {
        for (int it = threadIdx.x; it < items * NV; it += blockDim.x) {
            const int pl = it / items, i2 = it - pl * items;
            const int tk = i2 / octets, ro = i2 - tk * octets;
            float* p = part + (size_t)tk * PR + pl * plane_rows + ro * 8;
            Oct8 o;
            o.a = *reinterpret_cast<const float4*>(p);
            o.b = *reinterpret_cast<const float4*>(p + 4);
            for (int w = 1; w < WK; ++w) oct_add(o, p + w * wstride);
            *reinterpret_cast<float4*>(p) = o.a;
            *reinterpret_cast<float4*>(p + 4) = o.b;
        }
    }
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int cr = (int)cluster.block_rank();
    for (int it = cr * blockDim.x + threadIdx.x; it < items; it += SK * blockDim.x) {
        const int tk = it / octets, ro = it - tk * octets;
        float v[NV][8];
#pragma unroll
        for (int pl = 0; pl < NV; ++pl) {
            float* p = part + (size_t)tk * PR + pl * plane_rows + ro * 8;
            Oct8 o;
            o.a = make_float4(0.f, 0.f, 0.f, 0.f);
            o.b = o.a;
            for (int rk = 0; rk < SK; ++rk) oct_add(o, cluster.map_shared_rank(p, rk));
            oct_unpack(o, v[pl]);
        }
        emit(tk, ro, v);
    }
    cluster.sync();   // keep every CTA's shared memory alive until all remote reads are done
}

// Splits `total_chunks` 32-k chunks over `parts` slices in units of `gran` chunks.
__host__ __device__ inline void k_partition(int total_chunks, int gran, int parts, int part,
                                            int& c0, int& c1) {
    const long long units = total_chunks / gran;
    c0 = (int)(units * part / parts) * gran;
    c1 = (int)(units * (part + 1) / parts) * gran;
    if (part == parts - 1) c1 = total_chunks;
}

__host__ __device__ inline int max_part_chunks(int total_chunks, int gran, int parts) {
    const int units = total_chunks / gran;
    int mx = ((units + parts - 1) / parts) * gran;
    // the last slice also takes the remainder that is not a multiple of gran
    const int rem = total_chunks - units * gran;
    return mx + rem;
}

}  // namespace mlk
