// GEMM for many tokens (65 .. thousands) on the prepacked weights: C[n,m] = alpha * X[n,k] * A[m,k]^T (+ bias), the
// prefill-side consumer of the same layout-A tensors the GeMV / narrow-GEMM kernels stream.
//
// Above about 300 tokens the work is a real dense contraction (compute-bound), so the tile is as large as one CTA's
// tensor memory and shared memory allow: 128 weight rows (UMMA M, "swap-AB" as in dense_umma.cu: the weight tile needs
// no shuffle, its layout-A blocks are K-major core matrices) x NT = 128 or 256 tokens (UMMA N), the fp32 accumulator
// [128 x NT] in tensor memory, the whole k range in one CTA (no split: (m / 128) x ceil(n / NT) CTAs).
//   TMA (one thread)   per 64-wide k block: weight tile 16 KB (4-D map of dense_umma.cu) + token tile NT x 128 B
//                      (128-byte swizzle; rows beyond n are zero-filled)
//   MMA (one thread)   4 x tcgen05.mma.kind::f16 M128 x N(NT) x K16 per stage, tcgen05.commit frees the stage
//   4 epilogue warps   tcgen05.ld 16 token columns at a time -> alpha, bias, rounding -> staged in shared memory as
//                      [token][128 rows] -> 16-byte stores of 256 contiguous bytes per token
// Every mbarrier wait is bounded (status word, clean exit) as in the other tcgen05 kernels.
//
// Role in the reference: muxi_hgemm_layoutA (csrc/muxi_hgemm_layoutA.cu:12-217, kernel
// layoutA_hgemm_tn_128x128x128_4m1n8k_256t in muxi_hgemm_layoutA.cuh:792), benchmarked at 1024 tokens
// (benchmark_and_test/gemm_test_soft_fp8.py:159).
#include <algorithm>

#include "dense.cuh"
#include "umma_common.cuh"

namespace mlk {

namespace {

using namespace umma;

struct HgemmParams {
    void* C;
    const void* bias;
    float alpha;
    int m, n, k;
    int kblocks;
    int* status;
};

template <int WT, int NT>
constexpr uint32_t instr_desc_nt() {
    constexpr uint32_t fmt = (WT == kFP16) ? 0u : 1u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
}

template <int WT, int NT, int STAGES>
__global__ void __launch_bounds__(192, 1) hgemm_umma_kernel(const __grid_constant__ CUtensorMap map_a,
                                                            const __grid_constant__ CUtensorMap map_x, const HgemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int kBBytes = NT * 128;
    constexpr int kStageBytes = kABytes + kBBytes;
    constexpr uint32_t kTmemCols = NT;
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, tok0 = blockIdx.y * NT;
    const int KB = p.kblocks;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
    const uint32_t acc_full = bar0 + 8u * (2 * STAGES);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
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

    // activations (and the output buffer) belong to the preceding kernel of the stream until it has finished
    pdl_wait();
    pdl_launch_dependents();

    int issued = 0;
    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        for (int i = 0; i < KB; ++i) {
            const int s = i % STAGES;
            if (i >= STAGES && !mbar_wait(empty(s), ((i / STAGES) - 1) & 1)) {
                abort_flag = 1;
                if (p.status) atomicExch(p.status, 1);
            }
            if (abort_flag) break;
            mbar_expect_tx(full(s), kStageBytes);
            tma_load_4d(base + s * kStageBytes, &map_a, full(s), 0, i * (kBlockK / 8), tile * (kTileM / 16), 0);
            tma_load_2d(base + s * kStageBytes + kABytes, &map_x, full(s), i * kBlockK, tok0);
            ++issued;
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        constexpr uint32_t idesc = instr_desc_nt<WT, NT>();
        for (int i = 0; i < KB; ++i) {
            const int s = i % STAGES;
            if (abort_flag || !mbar_wait(full(s), (i / STAGES) & 1)) {
                if (!abort_flag && p.status) atomicExch(p.status, 2);
                abort_flag = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kk = 0; kk < kBlockK / 16; ++kk) {
                // A: no swizzle, [half][row group][k-octet][8 rows x 16 B]: 8-row step 1024 B, k-octet step 128 B
                const uint64_t da = smem_desc(base + s * kStageBytes + kk * 256, 128, 1024, 0);
                // B: 128-byte swizzle, 8-token step 1024 B; one MMA consumes 32 bytes of each 128-byte row
                const uint64_t db = smem_desc(base + s * kStageBytes + kABytes + kk * 32, 16, 1024, 2);
                umma_f16(tmem, da, db, idesc, (i > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(empty(s));
        }
        if (!abort_flag) umma_commit(acc_full);
    } else if (warp >= 2) {
        // ---- epilogue warps ----
        const int quad = warp & 3, lrow = quad * 32 + lane;          // accumulator row = tensor-memory lane
        // accumulator row rho holds weight row 16*(rho%64 / 8) + 8*(rho / 64) + rho%8 of the tile (see make_map_a16)
        const int wrow = ((lrow & 63) >> 3) * 16 + (lrow >> 6) * 8 + (lrow & 7);
        const int row = tile * kTileM + wrow;
        const float bia = (p.bias != nullptr) ? load_scalar16<WT>(p.bias, row) : 0.f;
        if (lane == 0 && (abort_flag || !mbar_wait(acc_full, 0))) {
            if (!abort_flag && p.status) atomicExch(p.status, 3);
            abort_flag = 1;
        }
        __syncwarp();
        asm volatile("bar.sync 1, 128;" ::: "memory");               // the four warps agree on abort_flag
        if (!abort_flag) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // staged tile [token][128 rows] 16-bit in the (now idle) ring: NT * 256 bytes
            uint16_t* const stage = reinterpret_cast<uint16_t*>(base_ptr);
#pragma unroll 1
            for (int c0 = 0; c0 < NT; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(tmem + ((uint32_t)(quad * 32) << 16) + c0, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float v = fmaf(p.alpha, __uint_as_float(r[i]), bia);
                    uint16_t h;
                    if constexpr (WT == kFP16) h = __half_as_ushort(__float2half_rn(v));
                    else h = __bfloat16_as_ushort(__float2bfloat16_rn(v));
                    stage[(c0 + i) * kTileM + wrow] = h;
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int etid = tid - 64;
            const int valid = min(NT, p.n - tok0);
            uint8_t* const cbase = reinterpret_cast<uint8_t*>(p.C) + ((size_t)tok0 * p.m + (size_t)tile * kTileM) * 2;
            for (int idx = etid; idx < valid * 16; idx += 128) {
                const int c = idx >> 4, ch = idx & 15;
                const uint4 val = *reinterpret_cast<const uint4*>(base_ptr + c * (kTileM * 2) + ch * 16);
                *reinterpret_cast<uint4*>(cbase + (size_t)c * p.m * 2 + ch * 16) = val;
            }
        }
    }
    __syncwarp();

    // ---- teardown ----
    if (warp == 0 && lane == 0 && abort_flag) {
        for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(full(i % STAGES), (i / STAGES) & 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

template <int WT, int NT>
const void* hgemm_kernel_for_stages(int stages) {
    switch (stages) {
        case 2: return reinterpret_cast<const void*>(hgemm_umma_kernel<WT, NT, 2>);
        case 3: return reinterpret_cast<const void*>(hgemm_umma_kernel<WT, NT, 3>);
        case 4: return reinterpret_cast<const void*>(hgemm_umma_kernel<WT, NT, 4>);
        case 6: return reinterpret_cast<const void*>(hgemm_umma_kernel<WT, NT, 6>);
    }
    return nullptr;
}

}  // namespace

// nt: tokens per tile (128 or 256; 0 = by token count); stages: ring depth (2, 3, 4, 6; 0 = as many as fit, 4 at most).
int launch_hgemm_umma(int wt, const DenseParams& p, int nt, int stages, int* status, cudaStream_t stream) {
    if (wt != kBF16 && wt != kFP16) return fail(kUnsupported, "hgemm (tcgen05): 16-bit weights only");
    if (!p.A || !p.X || !p.C) return fail(kInvalidArg, "hgemm: null pointer");
    if (p.x_layout != 0 || p.c_layout != 0) return fail(kUnsupported, "hgemm (tcgen05): row-major B and C");
    if (p.m % kTileM != 0 || p.k % kBlockK != 0) return fail(kInvalidArg, "hgemm (tcgen05): need m %% 128 == 0 and k %% 64 == 0");
    if (p.n < 1) return fail(kInvalidArg, "hgemm: n must be positive");
    if (((uintptr_t)p.A & 15) || ((uintptr_t)p.X & 15) || ((uintptr_t)p.C & 15))
        return fail(kInvalidArg, "hgemm (tcgen05): A, B and C must be 16-byte aligned");
    if (encode_fn() == nullptr) return fail(kUnsupported, "hgemm (tcgen05): cuTensorMapEncodeTiled is not available");
    if (nt == 0) {
        // 256-token tiles halve the weight re-reads; 128-token tiles when they give the SMs more tiles to share
        const long long t256 = (long long)(p.m / kTileM) * ((p.n + 255) / 256);
        nt = (p.n <= 128 || t256 < sm_count()) ? 128 : 256;
    }
    if (nt != 128 && nt != 256) return fail(kInvalidArg, "hgemm (tcgen05): tokens per tile must be 128 or 256 (got %d)", nt);
    if (stages == 0) stages = nt == 256 ? 4 : 4;
    const void* kern = nullptr;
    if (wt == kFP16) kern = nt == 128 ? hgemm_kernel_for_stages<kFP16, 128>(stages) : hgemm_kernel_for_stages<kFP16, 256>(stages);
    else kern = nt == 128 ? hgemm_kernel_for_stages<kBF16, 128>(stages) : hgemm_kernel_for_stages<kBF16, 256>(stages);
    if (kern == nullptr) return fail(kInvalidArg, "hgemm (tcgen05): stages must be one of 2, 3, 4, 6 (got %d)", stages);
    const size_t want = std::max((size_t)stages * (kABytes + nt * 128), (size_t)nt * kTileM * 2) + 1024;
    if (want > 227 * 1024) return fail(kUnsupported, "hgemm (tcgen05): %d stages do not fit in shared memory", stages);
    const size_t smem = prepare_kernel(kern, 192, want, nt);
    if (smem == 0) return fail(kCudaError, "hgemm (tcgen05): a CTA with %d stages does not fit on this device", stages);
    CUtensorMap ma, mx;
    if (!make_map_a16(&ma, p.A, p.m, p.k, wt)) return fail(kUnsupported, "hgemm (tcgen05): weight tensor map rejected");
    if (!make_map_x(&mx, p.X, p.n, p.k, wt, nt)) return fail(kUnsupported, "hgemm (tcgen05): activation tensor map rejected");
    HgemmParams hp{};
    hp.C = p.C; hp.bias = p.bias; hp.alpha = p.alpha; hp.m = p.m; hp.n = p.n; hp.k = p.k;
    hp.kblocks = p.k / kBlockK;
    hp.status = status;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.m / kTileM), (unsigned)((p.n + nt - 1) / nt), 1);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = launch_attrs(attr, 1);
    void* args[3] = {&ma, &mx, &hp};
    const cudaError_t e = cudaLaunchKernelExC(&cfg, kern, args);
    if (e != cudaSuccess) return fail(kCudaError, "hgemm_umma launch: %s", cudaGetErrorString(e));
    return kOk;
}

}  // namespace mlk
