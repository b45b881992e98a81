// Soft-FP8 narrow GEMM with the e4m3 weights fed to the tensor cores as they are:
// C[n,m] = alpha * X[n,k] * value(A[m,k])^T (+ bias), A in e4m3 (layout A), X and C in bf16.
//
// The decode kernels (dense_umma_f8.cu, dense.cu) turn every weight byte into a bf16 with four integer / packed
// instructions, and at HBM speed that instruction stream is as expensive as the memory stream (measured: neither is
// saturated, both sit near 50 %).  tcgen05.mma.kind::f8f6f4 multiplies e4m3 operands directly, with exact products
// and fp32 accumulation, so here no instruction is spent on a weight byte.  The price is paid on the activations, once
// per launch and proportional to the tokens, not to the weights: a kernel in front rewrites the bf16 activations as two
// e4m3 terms per element (f8n_common.cuh: exact hi + lo split under a power-of-two scale per token).
//
// The native weight layout [16 rows][8 bytes] interleaves the rows of a 16-row group at 8-byte granularity, which no
// shared-memory operand layout of the MMA can express (a K-major core matrix wants 16 contiguous bytes per row).
// Tensor memory can: the A operand of tcgen05.mma may live there with one row per lane, so the four "mover" warps
// copy each thread's 64 weight bytes of a stage from the TMA-landed tile into its lane (8 shared-memory loads, one
// tcgen05.st, no arithmetic).
//
// Pipeline per CTA (192 threads), one thread-block cluster per 128-row tile, k split over the cluster's CTAs:
//   TMA (one thread)      per stage: raw e4m3 tile [8 row groups][BK/8 k-octets][16 rows x 8 B] and BK/64 token tiles
//                         [NP tokens][hi 64 B | lo 64 B] from the split planes (128-byte swizzle)
//   4 mover warps         raw tile -> tensor memory (thread = tile row = lane)
//   MMA (one thread)      per 64-wide k block 2 k steps x {hi, lo} tcgen05.mma.kind::f8f6f4, A from tensor memory;
//                         tcgen05.commit releases the stage and the tensor-memory slot
//   epilogue              accumulator x inverse token scale -> fp32 partial tile -> cluster reduction over distributed
//                         shared memory in a fixed order -> C
// Block scales of the weights are not handled here (they would have to multiply the activations of each 128-row tile
// separately): calls with a scale tensor run on the decode kernels.
//
// Role in the reference: GemmMmaJustLayoutASoftFp8Kernel (csrc/gemm_layout_A_soft_fp8.cu) and the soft-FP8 GeMV
// (csrc/layout_gemv_kernel_soft_fp8.cuh), which decode in registers.
#include <algorithm>

#include "dense.cuh"
#include "f8n_common.cuh"

namespace mlk {

namespace {

using namespace umma;
using namespace f8n;

// BK = k elements (= weight bytes per row) of one stage: 64 or 128.  A raw weight tile is 128 * BK bytes and takes
// BK / 4 tensor-memory columns (four bytes per 32-bit column).  Weight tiles kept in tensor memory: what fits beside
// the accumulator in 64 or 128 columns.
constexpr int mover_stages(int np, int bk) {
    return bk == 64 ? (np == 16 ? 3 : (np == 32 ? 2 : 4)) : (np == 16 ? 3 : (np == 32 ? 3 : 2));
}
constexpr uint32_t tmem_cols_for(int np, int bk) { return (np + mover_stages(np, bk) * (bk / 4)) <= 64 ? 64 : 128; }

struct F8NParams {
    void* C;
    const void* bias;
    float alpha;
    int m, n, k;
    int c_layout;
    int kblocks;             // k / BK
    const float* inv_scale;  // [n] what the fp32 sums of token t are multiplied by (written by the kernel in front)
    int* status;
};

template <int NP, int BK, int STAGES>
__global__ void __launch_bounds__(192, 2) dense_umma_f8n_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                const __grid_constant__ CUtensorMap map_x,
                                                                const F8NParams p, const int static_weights) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int S2 = mover_stages(NP, BK);
    constexpr int kRawBytes = kTileM * BK;           // e4m3 weight tile of one stage
    constexpr int kAColumns = BK / 4;                // its tensor-memory columns
    constexpr int kXTile = NP * 128;                 // token tile of one 64-wide k block: [NP][hi 64 | lo 64]
    constexpr int kStageBytes = kRawBytes + (BK / 64) * kXTile;
    constexpr uint32_t kTmemCols = tmem_cols_for(NP, BK);
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 2 * S2 + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint64_t wpol = l2_evict_first_policy();       // weights are read once: first out of L2
    const int tile = blockIdx.x, rank = blockIdx.y, SK = gridDim.y;
    const int KB = p.kblocks;
    const int kb0 = (int)((long long)KB * rank / SK), kb1 = (int)((long long)KB * (rank + 1) / SK);
    const int nunits = kb1 - kb0;

    // 1024-byte aligned ring of stages (raw weight tile, then the token tiles), reused for the fp32 partial tile at the
    // end (NP * 512 bytes <= two stages)
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };                       // TMA landed
    auto empty = [&](int s) { return bar0 + 8u * (STAGES + s); };           // the stage's MMAs are complete
    auto a_full = [&](int s) { return bar0 + 8u * (2 * STAGES + s); };      // weight tile is in tensor-memory slot s
    auto a_empty = [&](int s) { return bar0 + 8u * (2 * STAGES + S2 + s); };
    const uint32_t acc_full = bar0 + 8u * (2 * STAGES + 2 * S2);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);           // tcgen05.commit
        }
        for (int s = 0; s < S2; ++s) {
            mbar_init(a_full(s), 4);          // one arrival per mover warp
            mbar_init(a_empty(s), 1);         // tcgen05.commit
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
        // ---- TMA producer ----
        auto load_a = [&](int i) {
            const int s = i % STAGES;
            tma_load_3d_hint(base + s * kStageBytes, &map_a, full(s), 0, (kb0 + i) * (BK / 8), tile * (kTileM / 16), wpol);
        };
        auto load_x = [&](int i) {
            const int s = i % STAGES;
#pragma unroll
            for (int b = 0; b < BK / 64; ++b)
                tma_load_2d(base + s * kStageBytes + kRawBytes + b * kXTile, &map_x, full(s), ((kb0 + i) * (BK / 64) + b) * 128, 0);
        };
        int i = 0;
        if (static_weights) {
            // weights may stream before the preceding kernel has finished; activations never do
            pdl_launch_dependents();
            const int pre = nunits < STAGES ? nunits : STAGES;
            for (; i < pre; ++i) {
                mbar_expect_tx(full(i), kStageBytes);
                load_a(i);
            }
            pdl_wait();
            for (int j = 0; j < pre; ++j) load_x(j);
            issued = pre;
        } else {
            pdl_wait();
            pdl_launch_dependents();
        }
        for (; i < nunits; ++i) {
            const int s = i % STAGES;
            if (i >= STAGES && !mbar_wait(empty(s), ((i / STAGES) - 1) & 1)) {
                abort_flag = 1;
                if (p.status) atomicExch(p.status, 1);
            }
            if (abort_flag) break;
            mbar_expect_tx(full(s), kStageBytes);
            load_a(i);
            load_x(i);
            ++issued;
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        // every wait below depends on the token tiles, which follow the preceding kernel of the stream: the bounded
        // waits must not start counting before that kernel has finished
        pdl_wait();
        constexpr uint32_t idesc = instr_desc_f8<NP>();
        for (int i = 0; i < nunits; ++i) {
            const int s = i % STAGES, s2 = i % S2;
            // a_full implies full: the movers waited for the stage before they copied from it
            if (abort_flag || !mbar_wait(a_full(s2), (i / S2) & 1)) {
                if (!abort_flag && p.status) atomicExch(p.status, 2);
                abort_flag = 1;
                break;
            }
            // (already complete; observed by this thread as well before it hands the TMA-written tiles to the MMA)
            mbar_wait(full(s), (i / STAGES) & 1);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int b = 0; b < BK / 64; ++b) {
                const uint32_t xt = base + s * kStageBytes + kRawBytes + b * kXTile;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    // A: tensor memory, 8 columns (32 bytes of k) per MMA.  B: 128-byte swizzle, 8-token step 1024 B; the
                    // hi operand is bytes 32 j .. of every row, the lo operand 64 bytes further on
                    const uint32_t ta = tmem + NP + s2 * kAColumns + b * 16 + j * 8;
#pragma unroll
                    for (int term = 0; term < 2; ++term) {
                        const uint64_t db = smem_desc(xt + term * 64 + j * 32, 16, 1024, 2);
                        umma_f8_ts(tmem, ta, db, idesc, (i > 0 || b > 0 || j > 0 || term > 0) ? 1u : 0u);
                    }
                }
            }
            umma_commit(empty(s));
            umma_commit(a_empty(s2));
        }
        if (!abort_flag) umma_commit(acc_full);
    } else if (warp >= 2) {
        // ---- mover warps, then epilogue ----
        const int quad = warp & 3, lrow = quad * 32 + lane;     // tile row = tensor-memory lane
        // Raw weight tiles may arrive (static weights) and be moved while the preceding kernel of the stream still
        // runs; every later wait depends on the token tiles, which follow that kernel: wait for it before the first of
        // them, so that no bounded wait runs out on the predecessor's account.
        bool after_pred = false;
        if (!static_weights) {
            pdl_wait();
            after_pred = true;
        }
        for (int i = 0; i < nunits; ++i) {
            const int s = i % STAGES, s2 = i % S2;
            if (i >= S2 && !after_pred) {
                pdl_wait();
                after_pred = true;
            }
            bool ok = true;
            if (lane == 0) {
                ok = !abort_flag && mbar_wait(full(s), (i / STAGES) & 1);
                if (ok && i >= S2) ok = mbar_wait(a_empty(s2), ((i / S2) - 1) & 1);
                if (!ok) {
                    if (!abort_flag && p.status) atomicExch(p.status, 8);
                    abort_flag = 1;
                }
            }
            ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");   // the slot's previous MMAs are complete
            // tile row lrow = BK / 8 k-octets of 8 bytes, 128 bytes apart in [row group][k-octet][16 rows x 8 bytes]
            const uint8_t* raw = base_ptr + s * kStageBytes + (lrow >> 4) * (BK * 16) + (lrow & 15) * 8;
#pragma unroll
            for (int half = 0; half < BK / 64; ++half) {
                uint32_t v[16];
#pragma unroll
                for (int o = 0; o < 8; ++o) {
                    const uint2 w = *reinterpret_cast<const uint2*>(raw + (half * 8 + o) * 128);
                    v[2 * o] = w.x;
                    v[2 * o + 1] = w.y;
                }
                tmem_st16(tmem + ((uint32_t)(quad * 32) << 16) + NP + s2 * kAColumns + half * 16, v);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a_full(s2)) : "memory");
        }
        // accumulator x inverse token scale -> fp32 partial tile [token][tile row] in this CTA's (now idle) ring
        if (!after_pred) pdl_wait();
        if (lane == 0 && (abort_flag || !mbar_wait(acc_full, 0))) {
            if (!abort_flag && p.status) atomicExch(p.status, 3);
            abort_flag = 1;
        }
        __syncwarp();
        if (!abort_flag) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float* const red = reinterpret_cast<float*>(base_ptr);
#pragma unroll
            for (int c0 = 0; c0 < NP; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(tmem + ((uint32_t)(quad * 32) << 16) + c0, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float inv = (c0 + i < p.n) ? __ldg(p.inv_scale + c0 + i) : 0.f;
                    red[(c0 + i) * kTileM + lrow] = __uint_as_float(r[i]) * inv;
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
    }
    __syncwarp();

    // ---- every CTA of the cluster adds one slice of tile rows over all ranks (descending rank, fixed order) through
    // distributed shared memory and writes that slice of C ----
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (warp >= 2) {
        const int etid = tid - 64;
        // slices in units of four rows: one 16-byte distributed-shared-memory load per rank brings four consecutive
        // weight rows (output elements) of one token
        const int q0 = (kTileM / 4) * rank / SK, quads = (kTileM / 4) * (rank + 1) / SK - q0;
        uint32_t remote[8];
#pragma unroll
        for (int q = 0; q < 8; ++q)
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[q]) : "r"(base), "r"(q < SK ? q : 0));
        const int total = p.n * quads;
        for (int idx = etid; idx < total; idx += 128) {
            const int c = idx / quads, rho = 4 * (q0 + idx - c * quads);
            const uint32_t off = (uint32_t)(c * kTileM + rho) * 4u;
            float4 t[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                t[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (q < SK)
                    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                 : "=f"(t[q].x), "=f"(t[q].y), "=f"(t[q].z), "=f"(t[q].w)
                                 : "r"(remote[q] + off)
                                 : "memory");
            }
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            bool first = true;
#pragma unroll
            for (int q = 7; q >= 0; --q) {
                if (q < SK) {
                    acc = first ? t[q] : make_float4(acc.x + t[q].x, acc.y + t[q].y, acc.z + t[q].z, acc.w + t[q].w);
                    first = false;
                }
            }
            const int row = tile * kTileM + rho;
            float4 bia = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p.bias != nullptr)
                bia = make_float4(load_scalar16<kBF16>(p.bias, row), load_scalar16<kBF16>(p.bias, row + 1),
                                  load_scalar16<kBF16>(p.bias, row + 2), load_scalar16<kBF16>(p.bias, row + 3));
            size_t o;
            if (p.c_layout == 0) {
                o = (size_t)c * p.m + row;
            } else {
                const int NB = p.n >> 4;
                o = ((((size_t)(row >> 5) * NB + (c >> 4)) * 4 + ((row >> 3) & 3)) * 16 + (c & 15)) * 8 + (row & 7);
            }
            uint2 packed;
            packed.x = pack2<kBF16>(fmaf(p.alpha, acc.x, bia.x), fmaf(p.alpha, acc.y, bia.y));
            packed.y = pack2<kBF16>(fmaf(p.alpha, acc.z, bia.z), fmaf(p.alpha, acc.w, bia.w));
            *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.C) + o) = packed;
        }
    }
    // nobody leaves while its shared memory may still be read
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");

    // ---- teardown: if the pipeline stopped early, wait (bounded) for the TMA copies still in flight ----
    if (warp == 0 && lane == 0 && abort_flag) {
        for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(full(i % STAGES), (i / STAGES) & 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// One CTA per token: the row's scale and its split planes (f8n_common.cuh).
__global__ void __launch_bounds__(512) act_split_rows_kernel(const uint4* __restrict__ x, int k, int repacked,
                                                            uint8_t* __restrict__ planes, float* __restrict__ inv_scale) {
    // the GEMM behind this kernel may become resident (and, with static weights, start streaming them) right away
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    split_row_cta(x + (size_t)row * (k >> 3), false, k, repacked, planes + (size_t)row * 2 * k, inv_scale + row);
}

template <int NP, int BK>
const void* f8n_kernel_for_stages(int stages) {
    switch (stages) {
        case 2: return reinterpret_cast<const void*>(dense_umma_f8n_kernel<NP, BK, 2>);
        case 3: return reinterpret_cast<const void*>(dense_umma_f8n_kernel<NP, BK, 3>);
        case 4: return reinterpret_cast<const void*>(dense_umma_f8n_kernel<NP, BK, 4>);
        case 6: return reinterpret_cast<const void*>(dense_umma_f8n_kernel<NP, BK, 6>);
        case 8: return reinterpret_cast<const void*>(dense_umma_f8n_kernel<NP, BK, 8>);
    }
    return nullptr;
}
template <int BK>
const void* f8n_kernel_for(int np, int stages) {
    switch (np) {
        case 16: return f8n_kernel_for_stages<16, BK>(stages);
        case 32: return f8n_kernel_for_stages<32, BK>(stages);
        case 64: return f8n_kernel_for_stages<64, BK>(stages);
    }
    return nullptr;
}

}  // namespace

// Scratch the native-e4m3 GEMM needs for n tokens of k elements: 256 floats of inverse scales, then the split planes.
long long f8n_scratch_bytes(int n, int k) { return 1024 + (long long)n * 2 * k; }
int f8n_max_k() { return kSplitMaxK; }

// bk: k elements per stage (64 or 128); stages: depth of the ring (2, 3, 4, 6, 8); cluster_k: 1..8 CTAs per 128-row
// tile.  scratch: f8n_scratch_bytes(n, k) bytes of device memory (any content, 128-byte aligned), owned by the call
// until it completes.
int launch_dense_umma_f8n(const DenseParams& p, int bk, int stages, int cluster_k, void* scratch, long long scratch_bytes,
                          int* status, cudaStream_t stream) {
    if (!p.A || !p.X || !p.C) return fail(kInvalidArg, "dense: null pointer");
    if (p.scale != nullptr) return fail(kUnsupported, "dense (tcgen05, native e4m3): block scales are handled by the decode kernels (kernelId 1..4)");
    if (bk != 64 && bk != 128) return fail(kInvalidArg, "dense (tcgen05, native e4m3): k per stage must be 64 or 128 (got %d)", bk);
    if (p.x_layout != 0) return fail(kUnsupported, "dense (tcgen05, native e4m3): activations must be row-major");
    if (p.m % kTileM != 0 || p.k % bk != 0) return fail(kInvalidArg, "dense (tcgen05): need m %% 128 == 0 and k %% %d == 0", bk);
    if (p.n < 1 || p.n > 64) return fail(kUnsupported, "dense (tcgen05): 1..64 tokens per launch (got %d)", p.n);
    if (p.k > kSplitMaxK) return fail(kUnsupported, "dense (tcgen05, native e4m3): k <= %d (got %d)", kSplitMaxK, p.k);
    if (p.c_layout == 1 && p.n % 16 != 0) return fail(kInvalidArg, "dense: layout C needs n %% 16 == 0");
    if (((uintptr_t)p.A & 15) || ((uintptr_t)p.X & 15)) return fail(kInvalidArg, "dense (tcgen05): A and B must be 16-byte aligned");
    if (encode_fn() == nullptr) return fail(kUnsupported, "dense (tcgen05): cuTensorMapEncodeTiled is not available");
    if (cluster_k < 1 || cluster_k > 8) return fail(kInvalidArg, "dense (tcgen05, native e4m3): cluster split must be 1..8 (got %d)", cluster_k);
    if (cluster_k > p.k / bk) return fail(kInvalidArg, "dense (tcgen05): cluster split %d exceeds the %d k blocks", cluster_k, p.k / bk);
    if (scratch == nullptr || ((uintptr_t)scratch & 127) || scratch_bytes < f8n_scratch_bytes(p.n, p.k))
        return fail(kInvalidArg, "dense (tcgen05, native e4m3): needs %lld bytes of 128-byte aligned scratch (mlk_aux.workspace)",
                    f8n_scratch_bytes(p.n, p.k));
    const int np = p.n <= 16 ? 16 : (p.n <= 32 ? 32 : 64);
    const void* kern = bk == 64 ? f8n_kernel_for<64>(np, stages) : f8n_kernel_for<128>(np, stages);
    if (kern == nullptr) return fail(kInvalidArg, "dense (tcgen05, native e4m3): stages must be one of 2, 3, 4, 6, 8 (got %d)", stages);
    const size_t want = std::max((size_t)stages * (kTileM * bk + (bk / 64) * np * 128), (size_t)np * 512) + 1024;
    if (want > 227 * 1024) return fail(kUnsupported, "dense (tcgen05, native e4m3): %d stages of %d do not fit in shared memory", stages, bk);
    const size_t smem = prepare_kernel(kern, 192, want, (int)tmem_cols_for(np, bk));
    if (smem == 0) return fail(kCudaError, "dense (tcgen05, native e4m3): a CTA with %d stages does not fit on this device", stages);
    float* const inv_scale = reinterpret_cast<float*>(scratch);
    uint8_t* const planes = reinterpret_cast<uint8_t*>(scratch) + 1024;
    CUtensorMap ma, mx;
    if (!make_map_a8_bk(&ma, p.A, p.m, p.k, bk)) return fail(kUnsupported, "dense (tcgen05): weight tensor map rejected");
    if (!make_map_planes(&mx, planes, p.n, p.k, np)) return fail(kUnsupported, "dense (tcgen05): activation tensor map rejected");

    // scales and split planes of the activations
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)p.n, 1, 1);
        cfg.blockDim = dim3(split_threads(p.k));
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        cfg.attrs = attr;
        cfg.numAttrs = launch_attrs(attr, 1);
        const cudaError_t e = cudaLaunchKernelEx(&cfg, act_split_rows_kernel, reinterpret_cast<const uint4*>(p.X), p.k, p.fp8_order,
                                                 planes, inv_scale);
        if (e != cudaSuccess) return fail(kCudaError, "act_split launch: %s", cudaGetErrorString(e));
    }
    F8NParams fp{};
    fp.C = p.C; fp.bias = p.bias; fp.alpha = p.alpha; fp.m = p.m; fp.n = p.n; fp.k = p.k; fp.c_layout = p.c_layout;
    fp.kblocks = p.k / bk;
    fp.inv_scale = inv_scale;
    fp.status = status;
    int static_weights = option(kOptStaticWeights);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.m / kTileM), (unsigned)cluster_k, 1);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    cfg.attrs = attr;
    cfg.numAttrs = launch_attrs(attr, cluster_k);
    void* args[4] = {&ma, &mx, &fp, &static_weights};
    const cudaError_t e = cudaLaunchKernelExC(&cfg, kern, args);
    if (e != cudaSuccess) return fail(kCudaError, "dense_umma_f8n launch: %s", cudaGetErrorString(e));
    return kOk;
}

}  // namespace mlk
