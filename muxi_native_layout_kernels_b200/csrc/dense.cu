// GeMV and narrow GEMM on native-layout weights: C[n,m] = alpha * X[n,k] * A[m,k]^T (+ bias).
//
// Replaces the reference launch paths
//   gemv_layoutA_wapper            csrc/gemv_layout_a.cu:17-71   (kernels layout_gemv_kernel.cuh:19,239)
//   gemm_layoutA_wapper            csrc/gemm_layout_A.cu:684-750
//   gemm_layoutA_soft_fp8_wapper   csrc/gemm_layout_A_soft_fp8.cu:749
//   gemm_layoutAB_ContinuousC_wapper  csrc/gemm_layout_ab_continuous_c.cu:982
//   gemm_layoutABC_wapper          csrc/gemm_layout_abc.cu:685
// with two kernel families: a tensor-core streaming kernel (kernelId 1) for 1..256 tokens and a
// CUDA-core FMA + shuffle kernel (kernelId 2) for single-token GeMV.
#include "dense.cuh"

#include <algorithm>

#include "status.h"
#include "stream_core.cuh"

namespace mlk {

namespace {

constexpr int kSmemLimit = 200 * 1024;

struct DenseKernelParams {
    DenseParams p;
    int stages;
    int static_weights;
};

// Output store shared by both families: 8 consecutive weight rows of one token, 16 bytes.
template <int WT>
__device__ __forceinline__ void emit_dense(const DenseParams& p, int token, int row, float (&v)[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] *= p.alpha;
    if (p.bias != nullptr) {
        const uint4 b = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.bias) + (size_t)row * 2);
        const float2 b0 = unpack2<WT>(b.x), b1 = unpack2<WT>(b.y), b2 = unpack2<WT>(b.z), b3 = unpack2<WT>(b.w);
        v[0] += b0.x; v[1] += b0.y; v[2] += b1.x; v[3] += b1.y;
        v[4] += b2.x; v[5] += b2.y; v[6] += b3.x; v[7] += b3.y;
    }
    uint4 o;
    o.x = pack2<WT>(v[0], v[1]);
    o.y = pack2<WT>(v[2], v[3]);
    o.z = pack2<WT>(v[4], v[5]);
    o.w = pack2<WT>(v[6], v[7]);
    size_t unit;
    if (p.c_layout == 0) {
        unit = ((size_t)token * p.m + row) >> 3;
    } else {
        // layout C: C5[mb][nb][q][r][e] = C[16nb + r][32mb + 8q + e]
        const int NB = p.n >> 4;
        unit = (((size_t)(row >> 5) * NB + (token >> 4)) * 4 + ((row >> 3) & 3)) * 16 + (token & 15);
    }
    reinterpret_cast<uint4*>(p.C)[unit] = o;
}

// ---------------------------------------------------------------------------------------------
// Family 1: tensor-core streaming kernel
// ---------------------------------------------------------------------------------------------
template <int WT, int NT, int RG, bool SCALE>
__global__ void __launch_bounds__(256) dense_mma_kernel(const DenseKernelParams kp) {
    using S = CoreShape<NT, RG>;
    constexpr bool XDIRECT = (NT == 1);
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ CoreShared sh;
    const DenseParams& p = kp.p;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int warps = blockDim.x >> 5;
    const int WM = p.wm, WK = warps / WM;
    const int wm = warp % WM, wk = warp / WM;
    const int SK = gridDim.y, cr = blockIdx.y;
    const int rows_cta = 16 * RG * WM;
    const int row0 = blockIdx.x * rows_cta;
    const int tok0 = blockIdx.z * kTokBlock;
    const int nt = min(p.n - tok0, S::NTP);
    const int total_chunks = p.k >> 5;
    constexpr int gran = SCALE ? 4 : 1;
    const int parts = SK * WK;

    // this warp's K slice and weight addresses need nothing but kernel arguments
    CoreArgs a;
    int c0, c1;
    k_partition(total_chunks, gran, parts, cr * WK + wk, c0, c1);
    a.nchunks = c1 - c0;
    constexpr int esz = (WT == kE4M3) ? 1 : 2;
    const int ldscale = (p.k + 127) >> 7;
#pragma unroll
    for (int r = 0; r < RG; ++r) {
        const int rgidx = blockIdx.x * (RG * WM) + wm * RG + r;
        a.a_lane[r] = reinterpret_cast<const uint8_t*>(p.A) + (size_t)rgidx * 16 * p.k * esz +
                      (size_t)c0 * chunk_bytes<WT>() + t * (128 * esz) + g * 16;
        a.scale[r] = SCALE ? p.scale + (size_t)((rgidx * 16) >> 7) * ldscale + (c0 >> 2) : nullptr;
    }
    AFrag<WT> ring[S::CH][RG];
    if (kp.static_weights) {
        // weights are never written by a kernel of this stream: start streaming them before the kernels this
        // launch depends on have finished, and let the next launch do the same
        ring_init<WT, NT, RG>(ring, a);
        pdl_launch_dependents();
        pdl_wait();
    } else {
        pdl_wait();
        pdl_launch_dependents();
        ring_init<WT, NT, RG>(ring, a);
    }

    if (tid < WK) k_partition(total_chunks, gran, parts, cr * WK + tid, sh.c0[tid], sh.c1[tid]);
    if (tid < nt) {
        const int row = tok0 + tid;
        const unsigned long long base = (unsigned long long)p.X;
        sh.xrow[tid] = (p.x_layout == 0)
                           ? base + (unsigned long long)row * p.k * 2
                           : base + (unsigned long long)(row >> 4) * 1024 + (row & 15) * 16;
    }
    __syncthreads();

    a.steps = (max_part_chunks(total_chunks, gran, parts) + S::CH - 1) / S::CH;
    a.nt = nt;
    a.wk = wk;
    a.WK = WK;
    a.stages = kp.stages;
    a.xs_base = smem_u32(smem);
    a.xrows = nt;
    a.stage_bytes = WK * nt * S::PITCH;
    a.cstride = (p.x_layout == 0) ? 64 : (long long)(p.n >> 4) * 1024;
    a.qstride = (p.x_layout == 0) ? 16 : 256;
    a.sel01 = p.fp8_order ? kSelRep01 : kSelNat01;
    a.sel23 = p.fp8_order ? kSelRep23 : kSelNat23;

    float acc[RG][NT][4];
    stream_mma<WT, NT, RG, SCALE, XDIRECT>(acc, ring, a, sh);

    float* part = reinterpret_cast<float*>(smem);
    const int PR = rows_cta + 4;
    int lrow0[RG];
#pragma unroll
    for (int r = 0; r < RG; ++r) lrow0[r] = (wm * RG + r) * 16;
    store_partials<WT, NT, RG>(part, acc, wk, PR, lrow0);

    reduce_and_emit<1>(part, WK, S::NTP, PR, nt, rows_cta >> 3, 0, SK,
                       [&](int tk, int ro, float (&v)[1][8]) { emit_dense<WT>(p, tok0 + tk, row0 + ro * 8, v[0]); });
}

template <int WT, int NT, int RG, bool SCALE>
int launch_mma_inst(const DenseParams& p, cudaStream_t stream) {
    using S = CoreShape<NT, RG>;
    // A token tile that is wide relative to the CTA's K split may not fit in shared memory; drop K-split warps
    // (never below the requested row warps) until it does.  Results do not depend on the K split.
    int threads = p.threads;
    const int rows_cta = 16 * RG * p.wm;
    const int ntmax = std::min(p.n, S::NTP);
    size_t smem = 0;
    int stages = 3;
    for (;;) {
        const int WK = (threads / 32) / p.wm;
        const size_t stage = (NT == 1) ? 0 : (size_t)WK * ntmax * S::PITCH;   // one token tile: no staging
        const size_t part = (size_t)WK * S::NTP * (rows_cta + 4) * sizeof(float);
        stages = (std::max(stage * 3, part) > (size_t)kSmemLimit) ? 2 : 3;
        smem = std::max(stage * stages, part);
        if (smem <= (size_t)kSmemLimit || threads / 64 < p.wm || threads <= 32) break;
        threads /= 2;
    }
    if (smem > (size_t)kSmemLimit)
        return fail(kUnsupported, "dense: tile needs %zu bytes of shared memory (rg=%d wm=%d threads=%d n=%d)",
                    smem, RG, p.wm, p.threads, p.n);

    auto kern = dense_mma_kernel<WT, NT, RG, SCALE>;
    static bool attr_set[64] = {};   // per instantiation, per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
        if (e != cudaSuccess) return fail(kCudaError, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        attr_set[dev & 63] = true;
    }
    DenseKernelParams kp{p, stages, option(kOptStaticWeights)};
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.m / rows_cta, p.sk, (p.n + kTokBlock - 1) / kTokBlock);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = launch_attrs(attr, p.sk);
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, kp);
    if (e != cudaSuccess) return fail(kCudaError, "dense_mma launch: %s", cudaGetErrorString(e));
    return kOk;
}

template <int WT, bool SCALE>
int launch_mma_wt(const DenseParams& p, cudaStream_t stream) {
    const int nt = p.n <= 8 ? 1 : (p.n <= 16 ? 2 : (p.n <= 32 ? 4 : 8));
#define MLK_CASE(NT_, RG_) \
    if (nt == NT_ && p.rg == RG_) return launch_mma_inst<WT, NT_, RG_, SCALE>(p, stream);
    MLK_CASE(1, 1) MLK_CASE(1, 2) MLK_CASE(2, 1) MLK_CASE(2, 2)
    MLK_CASE(4, 1) MLK_CASE(4, 2) MLK_CASE(8, 1) MLK_CASE(8, 2)
#undef MLK_CASE
    return fail(kInvalidArg, "dense: unsupported rg=%d", p.rg);
}

// ---------------------------------------------------------------------------------------------
// Family 2: CUDA-core GeMV (one token).  Lane l owns weight row l%16 of k-octet 2u + l/16; every
// 16-byte weight load is matched by a 16-byte load of x (L1-resident, shared by half a warp) and
// 8 fp32 FMAs.  One xor-16 shuffle folds the two octet halves, shared memory folds the K slices.
// ---------------------------------------------------------------------------------------------
template <int WT, int RG, int NTOK>
__global__ void __launch_bounds__(256) gemv_simt_kernel(const DenseParams p, const int static_weights) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int D = 8;   // 16-byte weight loads in flight per row group
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int WK = blockDim.x >> 5;
    const int SK = gridDim.y, cr = blockIdx.y;
    const int row = lane & 15, half = lane >> 4;
    const int rows_cta = 16 * RG;
    const int total_units = p.k >> 4;   // one unit = 2 k-octets = 512 weight bytes per row group
    int u0, u1;
    k_partition(total_units, 1, SK * WK, cr * WK + warp, u0, u1);
    const int nunits = u1 - u0;

    const uint8_t* ap[RG];
#pragma unroll
    for (int r = 0; r < RG; ++r)
        ap[r] = reinterpret_cast<const uint8_t*>(p.A) + (size_t)(blockIdx.x * RG + r) * 16 * p.k * 2 +
                (size_t)(u0 * 2 + half) * 256 + row * 16;
    const uint8_t* xp = reinterpret_cast<const uint8_t*>(p.X) + (size_t)(u0 * 2 + half) * 16;
    const size_t xstride = (size_t)p.k * 2;   // bytes between token rows

    float acc[RG][NTOK];
#pragma unroll
    for (int r = 0; r < RG; ++r)
#pragma unroll
        for (int q = 0; q < NTOK; ++q) acc[r][q] = 0.f;

    const uint64_t wpol = l2_policy_evict_first();
    uint4 ring[D][RG];
    if (!static_weights) {
        pdl_wait();
        pdl_launch_dependents();
    }
#pragma unroll
    for (int d = 0; d < D; ++d)
#pragma unroll
        for (int r = 0; r < RG; ++r)
            ring[d][r] = (d < nunits) ? ldg_stream16_pol(ap[r] + (size_t)d * 512, wpol) : make_uint4(0, 0, 0, 0);
    if (static_weights) {   // see dense_mma_kernel
        pdl_launch_dependents();
        pdl_wait();
    }

    for (int ub = 0; ub < nunits; ub += D) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const int u = ub + d;
            float2 xf[NTOK][4];
#pragma unroll
            for (int q = 0; q < NTOK; ++q) {
                uint4 xv = make_uint4(0, 0, 0, 0);
                if (u < nunits && q < p.n) xv = __ldg(reinterpret_cast<const uint4*>(xp + q * xstride + (size_t)u * 32));
                xf[q][0] = unpack2<WT>(xv.x); xf[q][1] = unpack2<WT>(xv.y);
                xf[q][2] = unpack2<WT>(xv.z); xf[q][3] = unpack2<WT>(xv.w);
            }
#pragma unroll
            for (int r = 0; r < RG; ++r) {
                const uint4 w = ring[d][r];
                const float2 w0 = unpack2<WT>(w.x), w1 = unpack2<WT>(w.y), w2 = unpack2<WT>(w.z), w3 = unpack2<WT>(w.w);
#pragma unroll
                for (int q = 0; q < NTOK; ++q) {
                    float s = acc[r][q];
                    s = fmaf(w0.x, xf[q][0].x, s); s = fmaf(w0.y, xf[q][0].y, s);
                    s = fmaf(w1.x, xf[q][1].x, s); s = fmaf(w1.y, xf[q][1].y, s);
                    s = fmaf(w2.x, xf[q][2].x, s); s = fmaf(w2.y, xf[q][2].y, s);
                    s = fmaf(w3.x, xf[q][3].x, s); s = fmaf(w3.y, xf[q][3].y, s);
                    acc[r][q] = s;
                }
                const int un = u + D;
                ring[d][r] = (un < nunits) ? ldg_stream16_pol(ap[r] + (size_t)un * 512, wpol) : make_uint4(0, 0, 0, 0);
            }
        }
    }

    float* part = reinterpret_cast<float*>(smem);   // [WK][NTOK][PR]
    const int PR = rows_cta + 4;
#pragma unroll
    for (int r = 0; r < RG; ++r)
#pragma unroll
        for (int q = 0; q < NTOK; ++q) {
            const float s = acc[r][q] + __shfl_xor_sync(0xFFFFFFFFu, acc[r][q], 16);
            if (half == 0) part[(warp * NTOK + q) * PR + r * 16 + row] = s;
        }
    const int row0 = blockIdx.x * rows_cta;
    reduce_and_emit<1>(part, WK, NTOK, PR, p.n, rows_cta >> 3, 0, SK,
                       [&](int tk, int ro, float (&v)[1][8]) { emit_dense<WT>(p, tk, row0 + ro * 8, v[0]); });
}

template <int WT, int RG, int NTOK>
int launch_simt_inst(const DenseParams& p, cudaStream_t stream) {
    const int warps = p.threads / 32;
    const size_t smem = (size_t)warps * NTOK * (16 * RG + 4) * sizeof(float);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.m / (16 * RG), p.sk, 1);
    cfg.blockDim = dim3(p.threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = launch_attrs(attr, p.sk);
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_simt_kernel<WT, RG, NTOK>, p, option(kOptStaticWeights));
    if (e != cudaSuccess) return fail(kCudaError, "gemv_simt launch: %s", cudaGetErrorString(e));
    return kOk;
}

int check_common(const DenseParams& p) {
    if (!p.A || !p.X || !p.C) return fail(kInvalidArg, "dense: null pointer");
    if (p.m <= 0 || p.n <= 0 || p.k <= 0) return fail(kInvalidArg, "dense: m, n, k must be positive");
    if (p.m % 16 != 0) return fail(kInvalidArg, "dense: m %% 16 must be 0 (m=%d)", p.m);
    if (p.k % 32 != 0) return fail(kInvalidArg, "dense: k %% 32 must be 0 (k=%d)", p.k);
    if (p.threads != 64 && p.threads != 128 && p.threads != 256)
        return fail(kInvalidArg, "dense: block size must be one of 64, 128, 256 (got %d)", p.threads);
    if (p.sk != 1 && p.sk != 2 && p.sk != 4 && p.sk != 8)
        return fail(kInvalidArg, "dense: split-K must be one of 1, 2, 4, 8 (got %d)", p.sk);
    if (p.rg != 1 && p.rg != 2) return fail(kInvalidArg, "dense: APerWarp must be 1 or 2 (got %d)", p.rg);
    if ((p.x_layout == 1 || p.c_layout == 1) && p.n % 16 != 0)
        return fail(kInvalidArg, "dense: layout B / layout C need n %% 16 == 0 (n=%d)", p.n);
    if (p.c_layout == 1 && p.m % 32 != 0) return fail(kInvalidArg, "dense: layout C needs m %% 32 == 0");
    return kOk;
}

}  // namespace

int launch_dense_mma(int wt, const DenseParams& p, cudaStream_t stream) {
    if (int s = check_common(p)) return s;
    if (p.wm != 1 && p.wm != 2 && p.wm != 4 && p.wm != 8)
        return fail(kInvalidArg, "dense: row warps per CTA must be one of 1, 2, 4, 8 (got %d)", p.wm);
    if ((p.threads / 32) % p.wm != 0)
        return fail(kInvalidArg, "dense: %d threads cannot hold %d row warps", p.threads, p.wm);
    if (p.m % (16 * p.rg * p.wm) != 0)
        return fail(kInvalidArg, "dense: m=%d is not a multiple of the CTA row tile %d", p.m, 16 * p.rg * p.wm);
    if (p.n > 4 * kTokBlock) return fail(kInvalidArg, "dense: n=%d exceeds the narrow-GEMM limit of 256 tokens", p.n);
    if (p.scale != nullptr && wt != kE4M3) return fail(kInvalidArg, "dense: block scales need e4m3 weights");
    if (p.scale != nullptr && p.k % 128 != 0) return fail(kInvalidArg, "dense: block scales need k %% 128 == 0");
    switch (wt) {
        case kBF16: return launch_mma_wt<kBF16, false>(p, stream);
        case kFP16: return launch_mma_wt<kFP16, false>(p, stream);
        case kE4M3:
            return p.scale ? launch_mma_wt<kE4M3, true>(p, stream) : launch_mma_wt<kE4M3, false>(p, stream);
    }
    return fail(kUnsupported, "dense: unknown weight type %d", wt);
}

int launch_gemv_simt(int wt, const DenseParams& p, int, cudaStream_t stream) {
    if (int s = check_common(p)) return s;
    if (p.n > 4) return fail(kUnsupported, "the CUDA-core kernel handles 1..4 tokens; n=%d", p.n);
    if (p.x_layout != 0 || p.c_layout != 0) return fail(kInvalidArg, "the CUDA-core kernel needs row-major activations and output");
    if (wt == kE4M3) return fail(kUnsupported, "gemv kernel 2 (CUDA-core) has no e4m3 variant; use kernel 1");
    if (p.m % (16 * p.rg) != 0) return fail(kInvalidArg, "gemv: m=%d is not a multiple of %d", p.m, 16 * p.rg);
    const int ntok = p.n <= 1 ? 1 : (p.n <= 2 ? 2 : 4);
#define MLK_CASE(WT_, RG_, NT_) \
    if (wt == WT_ && p.rg == RG_ && ntok == NT_) return launch_simt_inst<WT_, RG_, NT_>(p, stream);
    MLK_CASE(kBF16, 1, 1) MLK_CASE(kBF16, 2, 1) MLK_CASE(kFP16, 1, 1) MLK_CASE(kFP16, 2, 1)
    MLK_CASE(kBF16, 1, 2) MLK_CASE(kBF16, 2, 2) MLK_CASE(kFP16, 1, 2) MLK_CASE(kFP16, 2, 2)
    MLK_CASE(kBF16, 1, 4) MLK_CASE(kBF16, 2, 4) MLK_CASE(kFP16, 1, 4) MLK_CASE(kFP16, 2, 4)
#undef MLK_CASE
    return fail(kUnsupported, "gemv: unknown weight type %d", wt);
}

}  // namespace mlk
