// Fused-MoE expert compute ("plan C"): alignment -> gather-GEMM1 with fused SiLU*up -> GEMM2 with fused
// routing-weight scale, un-permute and accumulation into y.  Three launches, no host synchronisation.
//
// Replaces fused_experts_compute and its helpers (csrc/moe_kernels/fused_experts_compute.cu:50-296,
// fused_experts_compute.h:50-163; kernels group_gemm_first.h:355, silu_and_mul.h:62, group_gemm_second.h:356
// and their soft-fp8 twins).  Differences by design:
//   * a work item is (expert, up to 64 of its slots), not a fixed 16-slot block, so for T <= 64 every
//     selected expert's weights are streamed exactly once per layer call;
//   * gate and up rows of W1 are paired inside one warp, so SiLU(gate)*up is applied to the fp32 sums and
//     only the [slots, I] activation (not [slots, 2I]) goes through memory -- one launch and two 16-bit
//     roundings fewer than the reference;
//   * split-K partial sums are reduced in fp32 through (distributed) shared memory instead of 16-bit atomics.
//   The only atomics left are the per-token accumulation of the top-k expert outputs into y, as in the
//   reference (group_gemm_second.h:333-346).
#include <algorithm>
#include <mutex>

#include "moe.cuh"
#include "status.h"
#include "stream_core.cuh"

namespace mlk {

namespace {

constexpr int kSmemLimit = 200 * 1024;

struct MoeGemmParams {
    const uint8_t* w;            // expert weights, layout A per expert
    long long w_expert_bytes;
    const float* scale;          // e4m3 block scales or null
    long long scale_expert;      // floats per expert
    const uint8_t* xsrc;         // GEMM1: x [T,H];  GEMM2: act [slots, I]
    int x_row_div;               // GEMM1: topk (token = slot / topk);  GEMM2: 1
    long long x_row_bytes;
    void* out;                   // GEMM1: act [slots, I];  GEMM2: y [T,H]
    const int32_t* sorted;
    const int4* worklist;
    const void* topk_weights;
    int topk;
    int rows;                    // weight rows handled per expert: GEMM1: I (gate rows; up rows are +I); GEMM2: H
    int k;
    int wm, stages, fp8_order;
    float* scratch;              // GEMM2: [slots, H] fp32 weighted outputs (deterministic combine) or null (atomics)
};

// MODE 1: RG == 2, row group 0 = gate rows, row group 1 = the matching up rows.
// MODE 2: plain rows, epilogue scales by the routing weight and accumulates into y.
template <int WT, int NT, int RG, bool SCALE, int MODE>
__global__ void __launch_bounds__(256) moe_gemm_kernel(const MoeGemmParams p) {
    using S = CoreShape<NT, RG>;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ CoreShared sh;
    __shared__ int slot_of[kTokBlock];

    // the work list comes from the alignment kernel earlier in the stream
    pdl_wait();
    pdl_launch_dependents();
    constexpr bool XDIRECT = (NT == 1);
    const int n_items = p.worklist[0].x;
    if ((int)blockIdx.z >= n_items) return;   // uniform over the cluster (clusters span y only)
    const int4 item = p.worklist[1 + blockIdx.z];
    const int expert = item.x, pos0 = item.y, nt = item.z;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int warps = blockDim.x >> 5;
    const int WM = p.wm, WK = warps / WM;
    const int wm = warp % WM, wk = warp / WM;
    const int SK = gridDim.y, cr = blockIdx.y;
    const int total_chunks = p.k >> 5;
    constexpr int gran = SCALE ? 4 : 1;
    const int parts = SK * WK;

    CoreArgs a;
    int c0, c1;
    k_partition(total_chunks, gran, parts, cr * WK + wk, c0, c1);
    a.nchunks = c1 - c0;
    constexpr int esz = (WT == kE4M3) ? 1 : 2;
    const int ldscale = (p.k + 127) >> 7;
    const uint8_t* wbase = p.w + (long long)expert * p.w_expert_bytes;
    const float* sbase = SCALE ? p.scale + (long long)expert * p.scale_expert : nullptr;
    // CTA tile: MODE 1 -> WM gate groups + the WM matching up groups; MODE 2 -> RG*WM groups
    const int tile_groups = (MODE == 1) ? WM : RG * WM;
#pragma unroll
    for (int r = 0; r < RG; ++r) {
        int rgidx;
        if (MODE == 1)
            rgidx = blockIdx.x * WM + wm + r * (p.rows >> 4);
        else
            rgidx = blockIdx.x * tile_groups + wm * RG + r;
        a.a_lane[r] = wbase + (size_t)rgidx * 16 * p.k * esz + (size_t)c0 * chunk_bytes<WT>() + t * (128 * esz) + g * 16;
        a.scale[r] = SCALE ? sbase + (size_t)((rgidx * 16) >> 7) * ldscale + (c0 >> 2) : nullptr;
    }
    AFrag<WT> ring[S::CH][RG];
    ring_init<WT, NT, RG>(ring, a);

    if (tid < WK) k_partition(total_chunks, gran, parts, cr * WK + tid, sh.c0[tid], sh.c1[tid]);
    if (tid < nt) {
        const int slot = p.sorted[pos0 + tid];
        slot_of[tid] = slot;
        sh.xrow[tid] = (unsigned long long)p.xsrc + (unsigned long long)(slot / p.x_row_div) * p.x_row_bytes;
    }
    __syncthreads();

    a.steps = (max_part_chunks(total_chunks, gran, parts) + S::CH - 1) / S::CH;
    a.nt = nt;
    a.wk = wk;
    a.WK = WK;
    a.stages = p.stages;
    a.xs_base = smem_u32(smem);
    a.xrows = nt;
    a.stage_bytes = WK * nt * S::PITCH;
    a.cstride = 64;
    a.qstride = 16;
    a.sel01 = p.fp8_order ? kSelRep01 : kSelNat01;
    a.sel23 = p.fp8_order ? kSelRep23 : kSelNat23;

    float acc[RG][NT][4];
    stream_mma<WT, NT, RG, SCALE, XDIRECT>(acc, ring, a, sh);

    float* part = reinterpret_cast<float*>(smem);
    const int rows_cta = 16 * RG * WM;
    const int PR = rows_cta + 4;
    int lrow0[RG];
#pragma unroll
    for (int r = 0; r < RG; ++r) lrow0[r] = (MODE == 1) ? (r * WM + wm) * 16 : (wm * RG + r) * 16;
    store_partials<WT, NT, RG>(part, acc, wk, PR, lrow0);

    if constexpr (MODE == 1) {
        // act[slot, col] = silu(gate) * up, one rounding
        const int col0 = blockIdx.x * WM * 16;
        reduce_and_emit<2>(part, WK, S::NTP, PR, nt, 2 * WM, 16 * WM, SK, [&](int tk, int ro, float (&v)[2][8]) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float gt = v[0][i];
                o[i] = (gt / (1.f + __expf(-gt))) * v[1][i];
            }
            uint4 w;
            w.x = pack2<WT == kFP16 ? kFP16 : kBF16>(o[0], o[1]);
            w.y = pack2<WT == kFP16 ? kFP16 : kBF16>(o[2], o[3]);
            w.z = pack2<WT == kFP16 ? kFP16 : kBF16>(o[4], o[5]);
            w.w = pack2<WT == kFP16 ? kFP16 : kBF16>(o[6], o[7]);
            uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + ((size_t)slot_of[tk] * p.rows + col0 + ro * 8) * 2;
            *reinterpret_cast<uint4*>(dst) = w;
        });
    } else {
        const int row0 = blockIdx.x * rows_cta;
        const int H = p.rows;
        reduce_and_emit<1>(part, WK, S::NTP, PR, nt, rows_cta >> 3, 0, SK, [&](int tk, int ro, float (&v)[1][8]) {
            const int slot = slot_of[tk];
            const float wgt = load_scalar16<WT == kFP16 ? kFP16 : kBF16>(p.topk_weights, slot);
            if (p.scratch != nullptr) {
                float4* dst = reinterpret_cast<float4*>(p.scratch + (size_t)slot * H + row0 + ro * 8);
                dst[0] = make_float4(wgt * v[0][0], wgt * v[0][1], wgt * v[0][2], wgt * v[0][3]);
                dst[1] = make_float4(wgt * v[0][4], wgt * v[0][5], wgt * v[0][6], wgt * v[0][7]);
                return;
            }
            const size_t off = (size_t)(slot / p.topk) * H + row0 + ro * 8;
            if constexpr (WT == kFP16) {
                __half2* y = reinterpret_cast<__half2*>(reinterpret_cast<__half*>(p.out) + off);
#pragma unroll
                for (int i = 0; i < 4; ++i) atomicAdd(y + i, __floats2half2_rn(wgt * v[0][2 * i], wgt * v[0][2 * i + 1]));
            } else {
                __nv_bfloat162* y = reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(p.out) + off);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    atomicAdd(y + i, __floats2bfloat162_rn(wgt * v[0][2 * i], wgt * v[0][2 * i + 1]));
            }
        });
    }
}

// Un-permute + sum: y[t, :] = round16( sum_j scratch[t*topk + j, :] ) over the slots whose expert lives on this
// rank, in ascending j.  One thread per (token, 8 columns).
template <int WT, bool F32>
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ scratch,
                                                         const int32_t* __restrict__ topk_ids,
                                                         const int32_t* __restrict__ experts_map, int map_len, int E,
                                                         int T, int topk, int H, void* __restrict__ y) {
    // the rows come from the second GEMM, the preceding kernel of the stream
    pdl_wait();
    pdl_launch_dependents();
    const int octs = H >> 3;
    const long long total = (long long)T * octs;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / octs), o = (int)(i - (long long)t * octs);
        float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < topk; ++j) {
            int e = topk_ids[t * topk + j];
            if (experts_map != nullptr) e = (e >= 0 && e < map_len) ? experts_map[e] : -1;
            if (e < 0 || e >= E) continue;
            const float4* src = reinterpret_cast<const float4*>(scratch + ((size_t)t * topk + j) * H + o * 8);
            const float4 u = src[0], w = src[1];
            a[0] += u.x; a[1] += u.y; a[2] += u.z; a[3] += u.w;
            a[4] += w.x; a[5] += w.y; a[6] += w.z; a[7] += w.w;
        }
        if constexpr (F32) {
            // the un-rounded sums (expert-parallel callers add the shares of the ranks before the one rounding)
            float4* const dst = reinterpret_cast<float4*>(y) + 2 * i;
            dst[0] = make_float4(a[0], a[1], a[2], a[3]);
            dst[1] = make_float4(a[4], a[5], a[6], a[7]);
        } else {
            uint4 out;
            out.x = pack2<WT>(a[0], a[1]);
            out.y = pack2<WT>(a[2], a[3]);
            out.z = pack2<WT>(a[4], a[5]);
            out.w = pack2<WT>(a[6], a[7]);
            reinterpret_cast<uint4*>(y)[i] = out;
        }
    }
}

// y[t, :] = sum of the token's rows in the combine scratch, in the activation type or (y_fp32) un-rounded
int launch_combine(const MoeParams& m, int wt, cudaStream_t s) {
    const long long total = (long long)m.T * (m.H / 8);
    const int grid = (int)std::min<long long>((total + 255) / 256, 8LL * sm_count());
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = launch_attrs(attr, 1);
    auto kern = m.y_fp32 ? moe_combine_kernel<kBF16, true> : (wt == kFP16 ? moe_combine_kernel<kFP16, false> : moe_combine_kernel<kBF16, false>);
    const float* scratch = m.scratch;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, scratch, m.topk_ids, m.experts_map, m.experts_map_len, m.E, m.T, m.topk, m.H, m.y);
    if (e != cudaSuccess) return fail(kCudaError, "moe_combine launch: %s", cudaGetErrorString(e));
    return kOk;
}

template <int WT, int NT, int RG, bool SCALE, int MODE>
int launch_moe_inst(const MoeGemmParams& p0, int tiles, int sk, int max_items, cudaStream_t stream) {
    using S = CoreShape<NT, RG>;
    MoeGemmParams p = p0;
    const int warps = 8;
    const int WK = warps / p.wm;
    const int rows_cta = 16 * RG * p.wm;
    const size_t stage = (NT == 1) ? 0 : (size_t)WK * S::NTP * S::PITCH;
    const size_t part = (size_t)WK * S::NTP * (rows_cta + 4) * sizeof(float);
    int stages = 3;
    if (std::max(stage * 3, part) > (size_t)kSmemLimit) stages = 2;
    const size_t smem = std::max(stage * stages, part);
    if (smem > (size_t)kSmemLimit) return fail(kUnsupported, "moe: tile needs %zu bytes of shared memory", smem);
    p.stages = stages;

    auto kern = moe_gemm_kernel<WT, NT, RG, SCALE, MODE>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
        if (e != cudaSuccess) return fail(kCudaError, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        attr_set[dev & 63] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, sk, max_items);
    cfg.blockDim = dim3(warps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = launch_attrs(attr, sk);
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    if (e != cudaSuccess) return fail(kCudaError, "moe gemm launch: %s", cudaGetErrorString(e));
    return kOk;
}

template <int WT, bool SCALE, int MODE>
int launch_moe_nt(const MoeGemmParams& p, int nt_tiles, int rg, int tiles, int sk, int max_items, cudaStream_t s) {
#define MLK_CASE(NT_, RG_) \
    if (nt_tiles == NT_ && rg == RG_) return launch_moe_inst<WT, NT_, RG_, SCALE, MODE>(p, tiles, sk, max_items, s);
    if constexpr (MODE == 1) {
        MLK_CASE(1, 2) MLK_CASE(2, 2) MLK_CASE(4, 2) MLK_CASE(8, 2)
    } else {
        MLK_CASE(1, 1) MLK_CASE(2, 1) MLK_CASE(4, 1) MLK_CASE(8, 1)
        MLK_CASE(1, 2) MLK_CASE(2, 2) MLK_CASE(4, 2) MLK_CASE(8, 2)
    }
#undef MLK_CASE
    return fail(kInvalidArg, "moe: unsupported tile (tokens tiles %d, row groups %d)", nt_tiles, rg);
}

template <int MODE>
int launch_moe_gemm(int wt, bool scale, const MoeGemmParams& p, int nt_tiles, int rg, int tiles, int sk,
                    int max_items, cudaStream_t s) {
    switch (wt) {
        case kBF16: return launch_moe_nt<kBF16, false, MODE>(p, nt_tiles, rg, tiles, sk, max_items, s);
        case kFP16: return launch_moe_nt<kFP16, false, MODE>(p, nt_tiles, rg, tiles, sk, max_items, s);
        case kE4M3:
            return scale ? launch_moe_nt<kE4M3, true, MODE>(p, nt_tiles, rg, tiles, sk, max_items, s)
                         : launch_moe_nt<kE4M3, false, MODE>(p, nt_tiles, rg, tiles, sk, max_items, s);
    }
    return fail(kUnsupported, "moe: unknown weight type %d", wt);
}

int pick_sk(int ctas, int chunks, int wk) {
    int sk = 1;
    while (sk < 8 && ctas * sk < 2 * sm_count() && chunks / (wk * sk * 2) >= 4) sk *= 2;
    return sk;
}

}  // namespace

int launch_fused_experts(const MoeParams& m0, cudaStream_t s) {
    MoeParams m = m0;
    if (!m.w1 || !m.w2 || !m.x || !m.topk_ids || !m.topk_weights || !m.sorted_token_ids || !m.cumsum ||
        !m.padded_num_experts || !m.experts_ids || !m.C || !m.y)
        return fail(kInvalidArg, "fused_experts_compute: null pointer");
    if (m.T < 0 || m.E <= 0 || m.topk <= 0 || m.H <= 0 || m.I <= 0)
        return fail(kInvalidArg, "fused_experts_compute: bad sizes");
    if (m.T == 0) return kOk;
    if (m.dtype < 0 || m.dtype > 2) return fail(kInvalidArg, "fused_experts_compute: Unsupported data type");
    if (m.H % 32 != 0 || m.I % 32 != 0)
        return fail(kInvalidArg, "fused_experts_compute: hidden and intermediate sizes must be multiples of 32 (H=%d I=%d)", m.H, m.I);
    const bool scale = m.dtype == 2 && m.w1_scale && m.w2_scale;
    if (m.dtype == 2 && (!!m.w1_scale != !!m.w2_scale))
        return fail(kInvalidArg, "fused_experts_compute: give both block scales or neither");
    if (scale && (m.H % 128 != 0 || m.I % 128 != 0))
        return fail(kInvalidArg, "fused_experts_compute: 128x128 block scales need H and I to be multiples of 128");
    const int mbs = m.mbs > 0 ? m.mbs : 16;
    const int wt = m.dtype;
    const int esz = (wt == kE4M3) ? 1 : 2;

    // slots per work item: the token tile the GEMM kernels are instantiated for
    // Sized from the expected load (the host cannot see the routing without a sync): twice the mean number of
    // slots per expert, never more than the tokens (an expert gets a token at most once).  Experts that receive
    // more than one block are split into several items and stream their weights once per item.
    const long long slots = (long long)m.T * m.topk;
    const long long mean2 = (2 * slots + m.E - 1) / m.E;
    const long long want = std::min<long long>(m.T, mean2);
    // decode batches as one cooperative kernel (moe_decode.cu): tuning values of 300 or more for both GEMMs; a routing
    // fused in front runs inside that kernel too
    if (m.wm1 >= 300 && m.wm2 >= 300) {
        if (moe_decode_supported(m)) return launch_moe_decode(m, s);
        m.nt = m.wm1 = m.sk1 = m.rg = m.wm2 = m.sk2 = 0;     // too many tokens for it: the library's own choice
    }
    if (m.gating != nullptr) {
        // every other path: the router kernel first
        if (int st = launch_router(m.gating, m.score_fun, m.T, m.n_global, m.n_groups, m.topk_groups,
                                   const_cast<int32_t*>(m.topk_ids), const_cast<void*>(m.topk_weights), m.topk, m.gating_bias,
                                   m.dtype == kFP16 ? 1 : 0, s, m.renormalize))
            return st;
        m.gating = nullptr;
    }
    // No tuning arguments at all (a geometry without a row in the table): what the tuner finds on the tabulated
    // geometries, as rules.
    //   * decode batches (one or two tokens) of fine-grained experts (at most 16 MB of weights each): the single
    //     cooperative kernel;
    //   * otherwise the tcgen05 kernels where they apply: 16-bit weights always; e4m3 without block scales on the
    //     native 8-bit kernels at any load (token tiles of 16 / 32 / 64 slots); e4m3 with block scales from about 16
    //     slots per expert on (below that the warp-level kernels, which decode in the registers of many small CTAs,
    //     measured faster).  One cluster per (work item, 128-row tile): enough CTAs for about four per SM, every CTA
    //     with at least four k blocks; the native second GEMM without clusters, one row tile per CTA, once that alone
    //     gives four CTAs per SM.
    const bool no_tune = m.nt == 0 && m.wm1 == 0 && m.sk1 == 0 && m.rg == 0 && m.wm2 == 0 && m.sk2 == 0;
    if (no_tune && m.T <= 2 && (long long)3 * m.I * m.H * esz <= (16LL << 20) && moe_decode_supported(m))
        return launch_moe_decode(m, s);
    const bool f8n_ok = wt == kE4M3 && !scale && moe_f8n_supported(m.H, m.I);
    if (no_tune && m.scratch != nullptr && m.I % 128 == 0 && m.H % 128 == 0 && slots * m.H * 4 <= m.scratch_bytes &&
        (wt != kE4M3 || f8n_ok || want > 16)) {
        const long long items = std::min<long long>(m.E, slots);
        auto cluster = [&](int tiles, int kblocks) {
            const long long ctas = items * tiles;
            int sk = (int)std::min<long long>(8, (600 + ctas - 1) / ctas);
            while (sk > 1 && kblocks / sk < 4) --sk;
            return sk;
        };
        const int fam = f8n_ok ? 200 : 100;
        m.wm1 = fam + (f8n_ok ? 4 : 3); m.sk1 = cluster(m.I / 128, m.H / 64);
        m.wm2 = fam + 3; m.sk2 = cluster(m.H / 128, m.I / 64);
        if (f8n_ok && items * (m.H / 128) >= 4LL * sm_count()) {
            m.sk2 = 11;
            if (m.I % 128 == 0 && want <= 32) m.wm2 = fam + 42;       // 128 k per stage, two ring stages
        }
        if (f8n_ok) m.nt = want <= 16 ? 2 : (want <= 32 ? 4 : 8);
        if (wt != kE4M3 && want > 64) m.nt = 16;
    }
    int nt_tiles = want <= 8 ? 1 : (want <= 16 ? 2 : (want <= 32 ? 4 : 8));
    if (m.nt == 1 || m.nt == 2 || m.nt == 4 || m.nt == 8) nt_tiles = m.nt;
    // 16 tiles (128 slots per work item) exist for the tcgen05 kernels with 16-bit weights only
    if (m.nt == 16) nt_tiles = (wt != kE4M3 && m.wm1 >= 100 && m.wm1 < 200 && m.wm2 >= 100 && m.wm2 < 200 && m.scratch != nullptr) ? 16 : 8;
    const int block_slots = nt_tiles * 8;
    const int max_items = (int)std::min<long long>(slots, (long long)std::min<long long>(m.E, slots) + slots / block_slots);

    // tcgen05 path (moe_umma.cu): asked for by the tuning arguments, 16-bit or e4m3 weights (block scales ride on the
    // decode), fp32 combine scratch present.
    // Its buffers are indexed by compact position (the routed slots expert by expert, no padding): the [slots, I]
    // activation takes the front of C like the warp-level path's, and the gathered token rows [slots, H] borrow the
    // combine scratch until the second GEMM overwrites it.
    const size_t c_bytes = (size_t)slots * 2 * m.I * 2;
    const size_t wl_bytes = 16 * (size_t)(max_items + 1);
    // native-e4m3 tcgen05 kernels (moe_umma_f8n.cu): tuning values 200 + stages; e4m3 weights without block scales
    // only, otherwise the same arguments run the decode kernels (100 + stages)
    if (m.wm1 >= 200 && m.wm2 >= 200 && !(wt == kE4M3 && !scale && moe_f8n_supported(m.H, m.I))) {
        m.wm1 -= 100;
        m.wm2 -= 100;
        if (m.sk2 > 8) m.sk2 = 1;      // "row tiles per CTA" exists for the native kernels only
    }
    const bool f8n = m.wm1 >= 200 && m.wm2 >= 200 && m.scratch != nullptr && (long long)slots * m.H * 4 <= m.scratch_bytes;
    const bool umma = !f8n && m.wm1 >= 100 && m.wm1 < 200 && m.wm2 >= 100 && m.wm2 < 200 && m.scratch != nullptr && m.I % 128 == 0 &&
                      m.H % 128 == 0 && (long long)slots * m.H * 4 <= m.scratch_bytes;
    if (nt_tiles == 16 && !umma) return fail(kInvalidArg, "fused_experts_compute: 128-slot work items need the tcgen05 kernels (sizes multiples of 128, combine scratch)");

    if (!umma && !f8n && (m.wm1 >= 100 || m.wm2 >= 100)) {
        // tuned for the tcgen05 kernels but this call cannot use them: the warp-level kernels choose for themselves
        m.wm1 = m.sk1 = m.rg = m.wm2 = m.sk2 = 0;
    }

    // work list lives in the half of C that the fused activation does not need
    uint8_t* cbytes = reinterpret_cast<uint8_t*>(m.C);
    const size_t wl_off = ((size_t)slots * m.I * 2 + 15) & ~(size_t)15;
    if (wl_off + wl_bytes > c_bytes)
        return fail(kInvalidArg, "fused_experts_compute: workspace C too small for the work list");
    void* worklist = cbytes + wl_off;

    // native-e4m3 path: the slot of every compact position and the two arrays of inverse row scales follow the work list
    const size_t aux_off = (wl_off + wl_bytes + 15) & ~(size_t)15;
    if (f8n && aux_off + 12 * (size_t)slots > c_bytes)
        return fail(kInvalidArg, "fused_experts_compute: workspace C too small for the native-e4m3 bookkeeping");
    int32_t* const cpos_slot = f8n ? reinterpret_cast<int32_t*>(cbytes + aux_off) : nullptr;
    float* const inv1 = reinterpret_cast<float*>(cbytes + aux_off + 4 * (size_t)slots);
    float* const inv2 = inv1 + slots;

    if (int st = launch_moe_align(m.T, m.E, m.topk, mbs, m.topk_ids, m.sorted_token_ids, m.cumsum,
                                  m.padded_num_experts, m.experts_ids, m.experts_map, m.experts_map_len, s, worklist,
                                  block_slots, cpos_slot))
        return st;

    if (f8n) {
        // split planes of the routed token rows borrow the combine scratch (2 H bytes per row of its 4 H) until the
        // second GEMM overwrites it; the [position, I] activation in the front of C is split in place
        const int np = block_slots < 16 ? 16 : block_slots;
        const int4* wl = reinterpret_cast<const int4*>(worklist);
        if (int st = launch_moe_split_gather(m.x, cpos_slot, wl, m.topk, m.H, m.fp8_order, m.scratch, inv1, (int)slots, s)) return st;
        if (int st = launch_moe_umma_f8n(1, m.w1, m.E, m.I, m.H, m.scratch, inv1, slots, m.C, wl, m.sorted_token_ids, m.topk_weights,
                                         (int)slots, np, m.wm1 - 200, m.sk1 > 0 ? m.sk1 : 1, max_items, m.status, s))
            return st;
        if (int st = launch_moe_split_inplace(m.C, wl, m.I, m.fp8_order, inv2, (int)slots, s)) return st;
        if (int st = launch_moe_umma_f8n(2, m.w2, m.E, m.H, m.I, m.C, inv2, slots, m.scratch, wl, m.sorted_token_ids, m.topk_weights,
                                         (int)slots, np, m.wm2 - 200, m.sk2 > 0 ? m.sk2 : 1, max_items, m.status, s))
            return st;
        return launch_combine(m, wt, s);
    }

    if (umma) {
        const int np = block_slots < 16 ? 16 : block_slots;
        if (int st = launch_moe_gather_positions(m.x, m.sorted_token_ids, reinterpret_cast<const int4*>(worklist), m.topk, m.H,
                                                 m.scratch, max_items, s))
            return st;
        if (int st = launch_moe_umma(1, wt, m.w1, m.E, m.I, m.H, m.scratch, slots, m.C, reinterpret_cast<const int4*>(worklist),
                                     m.sorted_token_ids, m.topk_weights, (int)slots, np, m.wm1 - 100, m.sk1 > 0 ? m.sk1 : 1,
                                     max_items, m.fp8_order, scale ? m.w1_scale : nullptr, m.status, s))
            return st;
        if (int st = launch_moe_umma(2, wt, m.w2, m.E, m.H, m.I, m.C, slots, m.scratch, reinterpret_cast<const int4*>(worklist),
                                     m.sorted_token_ids, m.topk_weights, (int)slots, np, m.wm2 - 100, m.sk2 > 0 ? m.sk2 : 1,
                                     max_items, m.fp8_order, scale ? m.w2_scale : nullptr, m.status, s))
            return st;
        return launch_combine(m, wt, s);
    }

    // ---- GEMM1: act[slot, 0..I) = silu(x W1_gate^T) * (x W1_up^T)
    MoeGemmParams g1{};
    g1.w = reinterpret_cast<const uint8_t*>(m.w1);
    g1.w_expert_bytes = (long long)2 * m.I * m.H * esz;
    g1.scale = scale ? m.w1_scale : nullptr;
    g1.scale_expert = (long long)((2 * m.I + 127) / 128) * ((m.H + 127) / 128);
    g1.xsrc = reinterpret_cast<const uint8_t*>(m.x);
    g1.x_row_div = m.topk;
    g1.x_row_bytes = (long long)m.H * 2;
    g1.out = m.C;
    g1.sorted = m.sorted_token_ids;
    g1.worklist = reinterpret_cast<const int4*>(worklist);
    g1.topk_weights = m.topk_weights;
    g1.topk = m.topk;
    g1.rows = m.I;
    g1.k = m.H;
    g1.fp8_order = m.fp8_order;
    int wm1 = (nt_tiles >= 8) ? 4 : (nt_tiles >= 2 ? 2 : 1);
    if (m.wm1 == 1 || m.wm1 == 2 || m.wm1 == 4 || m.wm1 == 8) wm1 = m.wm1;
    while (wm1 > 1 && (m.I / 16) % wm1 != 0) wm1 >>= 1;
    if ((m.I / 16) % wm1 != 0) return fail(kInvalidArg, "fused_experts_compute: I must be a multiple of 16");
    g1.wm = wm1;
    const int tiles1 = (m.I / 16) / wm1;
    int sk1 = m.sk1 > 0 ? m.sk1 : pick_sk(tiles1 * std::min(m.E, (int)slots), m.H / 32, 8 / wm1);
    if (sk1 != 1 && sk1 != 2 && sk1 != 4 && sk1 != 8) return fail(kInvalidArg, "fused_experts_compute: split-K must be 1, 2, 4 or 8");
    if (int st = launch_moe_gemm<1>(wt, scale, g1, nt_tiles, 2, tiles1, sk1, max_items, s)) return st;

    // ---- GEMM2: y[token] += w[slot] * (act[slot] W2^T)
    MoeGemmParams g2{};
    g2.w = reinterpret_cast<const uint8_t*>(m.w2);
    g2.w_expert_bytes = (long long)m.H * m.I * esz;
    g2.scale = scale ? m.w2_scale : nullptr;
    g2.scale_expert = (long long)((m.H + 127) / 128) * ((m.I + 127) / 128);
    g2.xsrc = reinterpret_cast<const uint8_t*>(m.C);
    g2.x_row_div = 1;
    g2.x_row_bytes = (long long)m.I * 2;
    g2.out = m.y;
    g2.sorted = m.sorted_token_ids;
    g2.worklist = reinterpret_cast<const int4*>(worklist);
    g2.topk_weights = m.topk_weights;
    g2.topk = m.topk;
    g2.rows = m.H;
    g2.k = m.I;
    g2.fp8_order = m.fp8_order;
    int rg2 = (m.rg == 1 || m.rg == 2) ? m.rg : ((nt_tiles >= 2 && m.H % 32 == 0) ? 2 : 1);
    int wm2 = (nt_tiles >= 8) ? 4 : (nt_tiles >= 2 ? 2 : 1);
    if (m.wm2 == 1 || m.wm2 == 2 || m.wm2 == 4 || m.wm2 == 8) wm2 = m.wm2;
    while (wm2 > 1 && (m.H / 16) % (rg2 * wm2) != 0) wm2 >>= 1;
    if ((m.H / 16) % (rg2 * wm2) != 0) rg2 = 1;
    g2.wm = wm2;
    const int tiles2 = (m.H / 16) / (rg2 * wm2);
    int sk2 = m.sk2 > 0 ? m.sk2 : pick_sk(tiles2 * std::min(m.E, (int)slots), m.I / 32, 8 / wm2);
    if (sk2 != 1 && sk2 != 2 && sk2 != 4 && sk2 != 8) return fail(kInvalidArg, "fused_experts_compute: split-K must be 1, 2, 4 or 8");
    const bool det = m.scratch != nullptr;
    if (m.y_fp32 && !det) return fail(kInvalidArg, "fused_experts_compute: fp32 output needs the combine scratch");
    if (det && m.scratch_bytes < (long long)slots * m.H * 4)
        return fail(kInvalidArg, "fused_experts_compute: combine scratch holds %lld bytes, needs %lld", m.scratch_bytes,
                    (long long)slots * m.H * 4);
    if (det && m.H % 8 != 0) return fail(kInvalidArg, "fused_experts_compute: H must be a multiple of 8");
    g2.scratch = det ? m.scratch : nullptr;
    if (int st = launch_moe_gemm<2>(wt, scale, g2, nt_tiles, rg2, tiles2, sk2, max_items, s)) return st;
    if (!det) return kOk;
    return launch_combine(m, wt, s);
}

// ---------------------------------------------------------------------------------------------------------
// Expert compute for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at all: a plugin that runs inside a memory pool it does not
// own, or a serving loop whose memory budget was fixed at start-up and
// whose allocator is off limits on the request path.  For them the fp32 buffer of the fixed-order combine (one row
// of H floats per routed slot) lives in this file-scope device array instead of a caller-provided pointer.
//
//   * Size limit: T * topK * H <= kStaticCombineFloats (2 Mi floats = 8 MiB); larger problems are rejected.
//   * Every GPU that loads the library carries these 8 MiB until the process exits.
//   * In host code the array's name is only a stand-in; the device address is fetched once per device with
//     cudaGetSymbolAddress while that device is current (first call on the device).  Make that first call before
//     any stream capture.
//   * All calls share the array and it keeps the previous call's contents.  Nothing in it has to start at zero:
//     the second GEMM writes every row that the combine kernel later reads (rows of slots whose expert is not on
//     this rank are never read).  Two calls that overlap on the GPU (different streams) race on it.
constexpr long long kStaticCombineFloats = 2LL << 20;
static __device__ __align__(256) float g_static_combine[kStaticCombineFloats];

int launch_fused_experts_static(const MoeParams& p0, cudaStream_t s) {
    const long long need = (long long)p0.T * p0.topk * p0.H;
    if (p0.T < 0 || p0.topk <= 0 || p0.H <= 0) return fail(kInvalidArg, "fused_experts_compute_static: bad sizes");
    if (need > kStaticCombineFloats)
        return fail(kInvalidArg,
                    "fused_experts_compute_static: batch_size * topK * hidden = %lld floats exceeds the built-in scratch of "
                    "%lld floats; use mlk_fused_experts_compute with a caller-provided buffer",
                    need, kStaticCombineFloats);
    static float* dev_addr[64] = {};
    static std::mutex mu;       // host threads may make their first calls at the same time
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(kCudaError, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(kUnsupported, "fused_experts_compute_static: device index %d out of range", dev);
    float* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev_addr[dev] == nullptr) {
            float* ptr = nullptr;
            e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_combine);
            if (e != cudaSuccess || ptr == nullptr)
                return fail(kCudaError, "cudaGetSymbolAddress(static combine scratch): %s", cudaGetErrorString(e));
            dev_addr[dev] = ptr;
        }
        scratch = dev_addr[dev];
    }
    MoeParams p = p0;
    p.scratch = scratch;
    p.scratch_bytes = kStaticCombineFloats * (long long)sizeof(float);
    return launch_fused_experts(p, s);
}

}  // namespace mlk
