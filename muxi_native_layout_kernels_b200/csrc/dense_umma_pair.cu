// Narrow GEMM for 17..64 tokens on the 5th-generation tensor cores with TWO 128-row weight tiles per CTA:
// C[n,m] = alpha * X[n,k] * A[m,k]^T (+ bias), 16-bit weights, row-major activations.
//
// Same pipeline as the cluster mode of dense_umma.cu (TMA -> shared-memory ring -> tcgen05.mma -> tensor memory, one
// thread-block cluster per unit of output rows, k split over the cluster's CTAs, fp32 partial tiles added through
// distributed shared memory in a fixed order).  The difference is what one CTA owns: 256 weight rows, as two M = 128
// accumulators that are fed by the SAME token tile.  Every CTA fetches the token tile of each k block from L2 (NP x 128
// bytes beside 16 KB of weights per 128 rows: half as much again as the weights at 64 tokens); two tiles per CTA
// halve that traffic without any load that crosses CTAs.  Measured on B200 this does NOT pay on the shapes of the
// packaged tables (4096 x 4096, 14336 x 4096, 4096 x 14336 at 32 and 64 tokens: 1.0-6 us slower than the one-tile
// kernel, whose extra time at 64 tokens turned out to sit in the epilogue, not in the token traffic): half as
// many CTAs cost more than the saved L2 reads.  It is kept as kernelId 8 for the tuner to try on other shapes.
//
// Warp roles (192 threads): warp 0 lane 0 = TMA producer, warp 1 = tensor-memory owner and (lane 0) MMA issuer,
// warps 2..5 = epilogue.  Every wait is bounded: on expiry the kernel records a code in *status, stops, waits
// (bounded) for its own TMA copies, frees its tensor memory and returns.
//
// Role in the reference: the CTA-tile kernel GemmMmaJustLayoutAKernel2 (csrc/gemm_layout_A.cu:296) with its larger
// row tile.
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "common.cuh"
#include "dense.cuh"
#include "status.h"
#include "umma_common.cuh"

namespace mlk {

namespace {

using namespace umma;

constexpr int kPairRows = 2 * kTileM;

struct PairParams {
    void* C;
    const void* bias;
    float alpha;
    int m, n, k;
    int c_layout;
    int kblocks;       // k / 64
    int* status;       // sticky error word (0 = ok), may be null
};

template <int WT, int NP, int STAGES>
__global__ void __launch_bounds__(192, 2) dense_umma_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                 const __grid_constant__ CUtensorMap map_x,
                                                                 const PairParams p, const int static_weights) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int kBBytes = NP * 128;
    constexpr int kStageA = 2 * kABytes;
    constexpr uint32_t kTmemCols = 2 * NP < 32 ? 32 : 2 * NP;     // two accumulators side by side
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = blockIdx.x, rank = blockIdx.y, SK = gridDim.y;
    const int KB = p.kblocks;
    const int kb0 = (int)((long long)KB * rank / SK), kb1 = (int)((long long)KB * (rank + 1) / SK);
    const int nunits = kb1 - kb0;

    // 1024-byte aligned operand ring: all weight stages (two tiles each), then all token stages
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_base = base, b_base = base + STAGES * kStageA;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
    const uint32_t acc_full = bar0 + 8u * (2 * STAGES);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(acc_full, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
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

    int issued = 0;
    if (warp == 0 && lane == 0) {
        // ---- TMA producer: one stage per k block, up to STAGES ahead of the MMAs ----
        auto load_a = [&](int s, int kb) {
            tma_load_4d(a_base + s * kStageA, &map_a, full_bar(s), 0, kb * (kBlockK / 8), (2 * g) * (kTileM / 16), 0);
            tma_load_4d(a_base + s * kStageA + kABytes, &map_a, full_bar(s), 0, kb * (kBlockK / 8),
                        (2 * g + 1) * (kTileM / 16), 0);
        };
        int i = 0;
        if (static_weights) {
            // weights may stream before the preceding kernel has finished; activations never do
            pdl_launch_dependents();
            const int pre = nunits < STAGES ? nunits : STAGES;
            for (; i < pre; ++i) {
                mbar_expect_tx(full_bar(i), kStageA + kBBytes);
                load_a(i, kb0 + i);
            }
            pdl_wait();
            for (int j = 0; j < pre; ++j) tma_load_2d(b_base + j * kBBytes, &map_x, full_bar(j), (kb0 + j) * kBlockK, 0);
            issued = pre;
        } else {
            pdl_wait();
            pdl_launch_dependents();
        }
        for (; i < nunits; ++i) {
            const int s = i % STAGES;
            if (i >= STAGES && !mbar_wait(empty_bar(s), ((i / STAGES) - 1) & 1)) {
                abort_flag = 1;
                if (p.status) atomicExch(p.status, 1);
            }
            if (abort_flag) break;
            mbar_expect_tx(full_bar(s), kStageA + kBBytes);
            load_a(s, kb0 + i);
            tma_load_2d(b_base + s * kBBytes, &map_x, full_bar(s), (kb0 + i) * kBlockK, 0);
            ++issued;
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer: both tiles consume the stage's token tile ----
        constexpr uint32_t idesc = instr_desc<WT, NP>();
        for (int i = 0; i < nunits; ++i) {
            const int s = i % STAGES;
            if (abort_flag || !mbar_wait(full_bar(s), (i / STAGES) & 1)) {
                if (!abort_flag && p.status) atomicExch(p.status, 2);
                abort_flag = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kk = 0; kk < kBlockK / 16; ++kk) {
                // A: no swizzle, [half][row group][k-octet][8 rows x 16 B]: 8-row step 1024 B, k-octet step 128 B
                // B: 128-byte swizzle, 8-token step 1024 B; one MMA consumes 32 bytes of each 128-byte row
                const uint64_t db = smem_desc(b_base + s * kBBytes + kk * 32, 16, 1024, 2);
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    const uint64_t da = smem_desc(a_base + s * kStageA + t * kABytes + kk * 256, 128, 1024, 0);
                    umma_f16(tmem + t * NP, da, db, idesc, (i > 0 || kk > 0) ? 1u : 0u);
                }
            }
            umma_commit(empty_bar(s));     // arrives when the MMAs above have finished reading the stage
        }
        if (!abort_flag) umma_commit(acc_full);
    } else if (warp >= 2) {
        // ---- epilogue warps: park the fp32 partial tiles [tile][token][accumulator row] in the (now idle) ring ----
        const int quad = warp & 3, lrow = quad * 32 + lane;      // accumulator row = tensor-memory lane
        if (lane == 0 && (abort_flag || !mbar_wait(acc_full, 0))) {
            if (!abort_flag && p.status) atomicExch(p.status, 3);
            abort_flag = 1;
        }
        __syncwarp();
        if (!abort_flag) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float* const red = reinterpret_cast<float*>(smem_raw + (base - smem_u32(smem_raw)));
#pragma unroll
            for (int c0 = 0; c0 < 2 * NP; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(tmem + ((uint32_t)(quad * 32) << 16) + c0, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; ++i) red[(c0 + i) * kTileM + lrow] = __uint_as_float(r[i]);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
    }
    __syncwarp();

    // ---- every CTA of the cluster adds one slice of the 256 accumulator rows over all ranks (descending rank, fixed
    // order) through distributed shared memory and writes that slice of C ----
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (warp >= 2) {
        const int etid = tid - 64;
        const int r0 = kPairRows * rank / SK, rows = kPairRows * (rank + 1) / SK - r0;
        uint32_t remote[8];
#pragma unroll
        for (int q = 0; q < 8; ++q)
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[q]) : "r"(base), "r"(q < SK ? q : 0));
        const int total = p.n * rows;
        for (int idx = etid; idx < total; idx += 128) {
            const int c = idx / rows, rr = r0 + idx - c * rows;
            const int t = rr >> 7, rho = rr & (kTileM - 1);
            const uint32_t off = (uint32_t)((t * NP + c) * kTileM + rho) * 4u;
            float v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                v[q] = 0.f;
                if (q < SK) asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v[q]) : "r"(remote[q] + off) : "memory");
            }
            float acc = 0.f;
            bool first = true;
#pragma unroll
            for (int q = 7; q >= 0; --q) {
                if (q < SK) {
                    acc = first ? v[q] : acc + v[q];
                    first = false;
                }
            }
            // accumulator row rho holds weight row 16*(rho%64 / 8) + 8*(rho / 64) + rho%8 of its tile
            const int row = (2 * g + t) * kTileM + ((rho & 63) >> 3) * 16 + (rho >> 6) * 8 + (rho & 7);
            const float bia = (p.bias != nullptr) ? load_scalar16<WT>(p.bias, row) : 0.f;
            const float val = fmaf(p.alpha, acc, bia);
            size_t o;
            if (p.c_layout == 0) {
                o = (size_t)c * p.m + row;
            } else {
                const int NB = p.n >> 4;
                o = ((((size_t)(row >> 5) * NB + (c >> 4)) * 4 + ((row >> 3) & 3)) * 16 + (c & 15)) * 8 + (row & 7);
            }
            if constexpr (WT == kFP16)
                reinterpret_cast<__half*>(p.C)[o] = __float2half_rn(val);
            else
                reinterpret_cast<__nv_bfloat16*>(p.C)[o] = __float2bfloat16_rn(val);
        }
    }
    // nobody leaves while its shared memory may still be read
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");

    // ---- teardown: if the pipeline stopped early, wait (bounded) for the TMA copies still in flight ----
    if (warp == 0 && lane == 0 && abort_flag) {
        for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(full_bar(i % STAGES), (i / STAGES) & 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// ---- host ------------------------------------------------------------------------------------------------

// Weight tile map: global layout A is [row group][k-octet][half][8 rows][8 k]; the 4-D view (64 elements = one 8-row
// core matrix, k-octet, row group, half) with box (64, 8, 8, 2) lands one 128 x 64 tile in shared memory as
// [half][row group][k-octet][128 B], uniform strides for one M = 128 descriptor.
bool make_map_a_pair(CUtensorMap* map, const void* A, int m, int k, int wt) {
    const cuuint64_t dims[4] = {64, (cuuint64_t)(k / 8), (cuuint64_t)(m / 16), 2};
    const cuuint64_t strides[3] = {256, (cuuint64_t)16 * k * 2, 128};
    const cuuint32_t box[4] = {64, kBlockK / 8, kTileM / 16, 2};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return encode_fn()(map, wt == kFP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                       const_cast<void*>(A), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int WT, int NP>
const void* pair_kernel_for_stages(int stages) {
    switch (stages) {
        case 2: return reinterpret_cast<const void*>(dense_umma_pair_kernel<WT, NP, 2>);
        case 3: return reinterpret_cast<const void*>(dense_umma_pair_kernel<WT, NP, 3>);
        case 4: return reinterpret_cast<const void*>(dense_umma_pair_kernel<WT, NP, 4>);
    }
    return nullptr;
}

template <int WT>
const void* pair_kernel_for(int np, int stages) {
    switch (np) {
        case 16: return pair_kernel_for_stages<WT, 16>(stages);
        case 32: return pair_kernel_for_stages<WT, 32>(stages);
        case 64: return pair_kernel_for_stages<WT, 64>(stages);
    }
    return nullptr;
}

}  // namespace

// stages: ring depth (2, 3, 4; a stage is 32 KB of weights + np * 128 bytes of tokens); cluster_k: 1..8 CTAs per
// 256-row unit.
int launch_dense_umma_pair(int wt, const DenseParams& p, int stages, int cluster_k, int* status, cudaStream_t stream) {
    if (wt != kBF16 && wt != kFP16) return fail(kUnsupported, "dense (tcgen05, 256 rows): 16-bit weights only");
    if (!p.A || !p.X || !p.C) return fail(kInvalidArg, "dense: null pointer");
    if (p.x_layout != 0) return fail(kUnsupported, "dense (tcgen05, 256 rows): activations must be row-major");
    if (p.m % kPairRows != 0 || p.k % kBlockK != 0)
        return fail(kInvalidArg, "dense (tcgen05, 256 rows): need m %% 256 == 0 and k %% 64 == 0");
    if (p.n < 1 || p.n > 64) return fail(kUnsupported, "dense (tcgen05): 1..64 tokens per launch (got %d)", p.n);
    if (p.c_layout == 1 && p.n % 16 != 0) return fail(kInvalidArg, "dense: layout C needs n %% 16 == 0");
    if (((uintptr_t)p.A & 15) || ((uintptr_t)p.X & 15)) return fail(kInvalidArg, "dense (tcgen05): A and B must be 16-byte aligned");
    if (encode_fn() == nullptr) return fail(kUnsupported, "dense (tcgen05): cuTensorMapEncodeTiled is not available");
    if (cluster_k < 1 || cluster_k > 8) return fail(kInvalidArg, "dense (tcgen05, 256 rows): cluster split must be 1..8 (got %d)", cluster_k);
    if (cluster_k > p.k / kBlockK) return fail(kInvalidArg, "dense (tcgen05): cluster split %d exceeds the %d k blocks", cluster_k, p.k / kBlockK);
    const int np = p.n <= 16 ? 16 : (p.n <= 32 ? 32 : 64);
    const void* kern = wt == kFP16 ? pair_kernel_for<kFP16>(np, stages) : pair_kernel_for<kBF16>(np, stages);
    if (kern == nullptr) return fail(kInvalidArg, "dense (tcgen05, 256 rows): stages must be 2, 3 or 4 (got %d)", stages);
    // the ring is reused for the fp32 partial tiles [2][np][128]
    const size_t ring = (size_t)stages * (2 * kABytes + np * 128);
    if (ring < (size_t)2 * np * kTileM * 4) return fail(kInvalidArg, "dense (tcgen05, 256 rows): ring too small for the partial tiles");
    const size_t smem = ring + 1024;
    static std::mutex mu;
    static bool attr_set[2][3][3][64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> lock(mu);
        bool& done = attr_set[wt == kFP16 ? 1 : 0][stages - 2][np == 16 ? 0 : np == 32 ? 1 : 2][dev & 63];
        if (!done) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return fail(kCudaError, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            done = true;
        }
    }
    CUtensorMap ma, mx;
    if (!make_map_a_pair(&ma, p.A, p.m, p.k, wt)) return fail(kUnsupported, "dense (tcgen05): weight tensor map rejected");
    if (!make_map_x(&mx, p.X, p.n, p.k, wt, np)) return fail(kUnsupported, "dense (tcgen05): activation tensor map rejected");
    PairParams pp{};
    pp.C = p.C; pp.bias = p.bias; pp.alpha = p.alpha; pp.m = p.m; pp.n = p.n; pp.k = p.k; pp.c_layout = p.c_layout;
    pp.kblocks = p.k / kBlockK;
    pp.status = status;
    int static_weights = option(kOptStaticWeights);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.m / kPairRows), (unsigned)cluster_k, 1);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = launch_attrs(attr, cluster_k);
    void* args[4] = {&ma, &mx, &pp, &static_weights};
    const cudaError_t e = cudaLaunchKernelExC(&cfg, kern, args);
    if (e != cudaSuccess) return fail(kCudaError, "dense_umma_pair launch: %s", cudaGetErrorString(e));
    return kOk;
}

}  // namespace mlk
