// Soft-FP8 narrow GEMM on the 5th-generation tensor cores: C[n,m] = alpha * X[n,k] * bf16(A[m,k])^T (+ bias), A in e4m3.
//
// Same "swap-AB" tile as dense_umma.cu (128 weight rows = UMMA M, tokens = N, fp32 accumulator in tensor memory)
// and the same one-cluster-per-tile decomposition (k split over the cluster's CTAs, partial tiles added through
// distributed shared memory).  The difference is the weight path.  The e4m3 bytes cannot be handed to the bf16 MMA,
// and decoding them in the registers of the warps that also wait for the loads is what limits the warp-level kernel
// (every byte in flight costs registers there).  Here the three steps run in different agents, coupled by mbarriers:
//   TMA (one thread)        global e4m3 tile [8 row groups][8 k-octets][16 rows x 8 bytes] -> raw ring (8 KB / stage)
//   4 converter warps       raw ring -> exact bf16 in registers (prmt / shift / and / packed multiply, common.cuh) ->
//                           tensor memory with tcgen05.st: thread = tile row = TMEM lane, 32 columns of bf16 pairs
//                           per 64-wide k block
//   MMA (one thread)        tcgen05.mma with the A operand in tensor memory and the TMA-loaded token tile as B,
//                           tcgen05.commit frees the slot
// so the bytes in flight sit in shared memory, the decode runs on warps that have nothing else to do (the four
// converter warps are the epilogue warps, idle until the accumulator is complete), and the decoded weights never
// touch shared memory: staging them there as well (raw write + raw read + bf16 write + bf16 read per byte) was
// measured to run into the shared-memory bandwidth before HBM.
// Block scales (one fp32 per 128 x 128 weights, so one per tile and k block pair) are applied in the decode.  By
// default the scale is rounded to bf16 and folded into the factor of the decode's one packed multiply, which costs
// nothing: weight = rne_bf16(w * bf16(s)).  With the full-scales option the scale enters as two bf16 terms (a packed
// multiply and a packed fused multiply-add more), which yields rne_bf16(w * s), the value the reference's torch
// check dequantises to; the decode being the bottleneck, that costs throughput (common.cuh, scaled_rebias).  The
// reference's kernels truncate fp32(w) * s to bf16; the warp-level kernel here applies s to the fp32 sums of each
// 128-wide k block.
//
// Role in the reference: GemmMmaJustLayoutASoftFp8Kernel (csrc/gemm_layout_A_soft_fp8.cu), which decodes in registers.
#include <algorithm>

#include "dense.cuh"
#include "umma_common.cuh"

namespace mlk {

namespace {

using namespace umma;

constexpr int kRawBytes = kTileM * kBlockK;      // 8 KB of e4m3 per stage
// decoded weight tiles in tensor memory (and depth of the token-tile ring): as many as fit beside the accumulator in
// 128 columns, so that four CTAs share an SM's tensor memory
constexpr int conv_stages(int np) { return np <= 32 ? 3 : 2; }
constexpr int kAColumns = kBlockK / 2;           // 32-bit columns of one decoded tile: two bf16 per column

struct F8Params {
    void* C;
    const void* bias;
    float alpha;
    int m, n, k;
    int c_layout;
    int kblocks;
    uint32_t sel01, sel23;   // byte selectors of the decode (natural or repacked order)
    const float* scale;      // fp32 block scales [m/128][scale_ld], one per 128 x 128 weights, or null
    int scale_ld;
    int full_scales;         // block scales with two bf16 terms instead of one (see common.cuh, scaled_rebias)
    int* status;
};

template <int NP, int STAGES>
__global__ void __launch_bounds__(192, 2) dense_umma_f8_kernel(const __grid_constant__ CUtensorMap map_a,
                                                               const __grid_constant__ CUtensorMap map_x,
                                                               const F8Params p, const int static_weights) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int kBBytes = NP * 128;
    // tensor memory: accumulator (NP columns), then kConvStages decoded weight tiles; power of two
    constexpr int S2 = conv_stages(NP);
    constexpr uint32_t kTmemCols = (NP + S2 * kAColumns) <= 128 ? 128 : 256;
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 2 * S2 + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint64_t wpol = l2_evict_first_policy();       // weights are read once: first out of L2
    const int tile = blockIdx.x, rank = blockIdx.y, SK = gridDim.y;
    const int KB = p.kblocks;
    const int kb0 = (int)((long long)KB * rank / SK), kb1 = (int)((long long)KB * (rank + 1) / SK);
    const int nunits = kb1 - kb0;

    // 1024-byte aligned: raw ring (reused for the fp32 partial tile at the end, NP * 512 bytes), then the token ring
    constexpr int kRingBytes = STAGES * kRawBytes > NP * 512 ? STAGES * kRawBytes : NP * 512;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t r_base = base, b_base = base + kRingBytes;
    const uint32_t bar0 = smem_u32(bars);
    auto raw_full = [&](int s) { return bar0 + 8u * s; };
    auto raw_empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto cv_full = [&](int s) { return bar0 + 8u * (2 * STAGES + s); };
    auto cv_empty = [&](int s) { return bar0 + 8u * (2 * STAGES + S2 + s); };
    const uint32_t acc_full = bar0 + 8u * (2 * STAGES + 2 * S2);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(raw_full(s), 1);
            mbar_init(raw_empty(s), 4);       // one arrival per converter warp
        }
        for (int s = 0; s < S2; ++s) {
            mbar_init(cv_full(s), 5);         // four converter warps + the producer's expect_tx for the token tile
            mbar_init(cv_empty(s), 1);        // tcgen05.commit
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

    int raw_issued = 0;
    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        auto load_raw = [&](int i) {
            const int s = i % STAGES;
            mbar_expect_tx(raw_full(s), kRawBytes);
            tma_load_3d_hint(r_base + s * kRawBytes, &map_a, raw_full(s), 0, (kb0 + i) * (kBlockK / 8), tile * (kTileM / 16), wpol);
            ++raw_issued;
        };
        int ri = 0;      // next unit whose weights are requested
        if (static_weights) {
            // weights may stream before the preceding kernel has finished; activations never do
            pdl_launch_dependents();
            const int pre = nunits < STAGES ? nunits : STAGES;
            for (; ri < pre; ++ri) load_raw(ri);
            pdl_wait();
        } else {
            pdl_wait();
            pdl_launch_dependents();
        }
        // Two independent streams from this one thread: token tiles (slot free once the MMAs of unit bi - S2 are done)
        // and raw weight tiles (slot free once unit ri - STAGES is converted).  Neither may block the other, so both
        // are polled without blocking; the idle count bounds the wait.
        int bi = 0;
        uint32_t idle = 0;
        while ((bi < nunits || ri < nunits) && !abort_flag) {
            bool progressed = false;
            if (bi < nunits && (bi < S2 || mbar_test_wait(cv_empty(bi % S2), ((bi / S2) - 1) & 1))) {
                const int s2 = bi % S2;
                mbar_expect_tx(cv_full(s2), kBBytes);
                tma_load_2d(b_base + s2 * kBBytes, &map_x, cv_full(s2), (kb0 + bi) * kBlockK, 0);
                ++bi;
                progressed = true;
            }
            if (ri < nunits && (ri < STAGES || mbar_test_wait(raw_empty(ri % STAGES), ((ri / STAGES) - 1) & 1))) {
                load_raw(ri);
                ++ri;
                progressed = true;
            }
            if (progressed) {
                idle = 0;
            } else if (++idle > 4 * kSpinLimit) {
                abort_flag = 1;
                if (p.status) atomicExch(p.status, 1);
            } else {
                __nanosleep(32);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        // the token tiles are requested only after the preceding kernel of the stream has finished: the bounded waits
        // below must not start counting before that
        pdl_wait();
        constexpr uint32_t idesc = instr_desc<kBF16, NP>();
        for (int i = 0; i < nunits; ++i) {
            const int s2 = i % S2;
            if (abort_flag || !mbar_wait(cv_full(s2), (i / S2) & 1)) {
                if (!abort_flag && p.status) atomicExch(p.status, 2);
                abort_flag = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kk = 0; kk < kBlockK / 16; ++kk) {
                // A: tensor memory, 8 columns (16 bf16) per MMA; B: 128-byte swizzle, 32 bytes of each row per MMA
                const uint32_t ta = tmem + NP + s2 * kAColumns + kk * 8;
                const uint64_t db = smem_desc(b_base + s2 * kBBytes + kk * 32, 16, 1024, 2);
                umma_f16_ts(tmem, ta, db, idesc, (i > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(cv_empty(s2));
        }
        if (!abort_flag) umma_commit(acc_full);
    } else if (warp >= 2) {
        // ---- converter warps, then epilogue ----
        const int quad = warp & 3, lrow = quad * 32 + lane;     // tile row = tensor-memory lane
        // block scale of a unit: one 128-row tile is one scale row, a 64-wide k block half a scale column; the value
        // for the next unit is requested before this unit's waits
        const float* const srow = p.scale ? p.scale + (size_t)tile * p.scale_ld : nullptr;
        float sc_next = (srow && nunits > 0) ? __ldg(srow + (kb0 >> 1)) : 1.f;
        uint32_t c2 = kRebias2;
        ScaledRebias sr{};
        // Raw weight tiles may arrive (static weights) and be decoded while the preceding kernel of the stream still
        // runs; every other wait depends on the token tiles, which follow that kernel: wait for it before the first of
        // them, so that no bounded wait runs out on the predecessor's account.
        bool after_pred = false;
        if (!static_weights) {
            pdl_wait();
            after_pred = true;
        }
        for (int i = 0; i < nunits; ++i) {
            const int s = i % STAGES, s2 = i % S2;
            const float sc = sc_next;
            if (srow && i + 1 < nunits) sc_next = __ldg(srow + ((kb0 + i + 1) >> 1));
            if (i >= S2 && !after_pred) {
                pdl_wait();
                after_pred = true;
            }
            bool ok = true;
            if (lane == 0) {
                ok = !abort_flag && mbar_wait(raw_full(s), (i / STAGES) & 1);
                if (ok && i >= S2) ok = mbar_wait(cv_empty(s2), ((i / S2) - 1) & 1);
                if (!ok) {
                    if (!abort_flag && p.status) atomicExch(p.status, 8);
                    abort_flag = 1;
                }
            }
            ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");   // the slot's previous MMAs are complete
            // this thread decodes tile row lrow = its TMEM lane: 8 k-octets of 8 bytes, 128 bytes apart in the raw tile
            // [row group][k-octet][16 rows x 8 bytes]
            const uint8_t* raw = base_ptr + s * kRawBytes + (lrow >> 4) * 1024 + (lrow & 15) * 8;
            uint32_t v[32];
            // c2: the factor of the decode's one multiply (2^120, or that times a block scale rounded to bf16); 0 = general form
            if (srow && (i == 0 || ((kb0 + i) & 1) == 0)) {     // a scale column spans two k blocks
                sr = scaled_rebias(sc, p.full_scales != 0);
                c2 = sr.one_multiply ? sr.hi2 : 0u;
            }
            if (c2 != 0u) {
#pragma unroll
                for (int o = 0; o < 8; ++o) {
                    const uint2 w = *reinterpret_cast<const uint2*>(raw + o * 128);
                    v[4 * o + 0] = e4m3x2_to_bf16x2_by(w.x, p.sel01, c2);
                    v[4 * o + 1] = e4m3x2_to_bf16x2_by(w.x, p.sel23, c2);
                    v[4 * o + 2] = e4m3x2_to_bf16x2_by(w.y, p.sel01, c2);
                    v[4 * o + 3] = e4m3x2_to_bf16x2_by(w.y, p.sel23, c2);
                }
            } else {
#pragma unroll
                for (int o = 0; o < 8; ++o) {
                    const uint2 w = *reinterpret_cast<const uint2*>(raw + o * 128);
                    v[4 * o + 0] = e4m3x2_scaled(w.x, p.sel01, sr);
                    v[4 * o + 1] = e4m3x2_scaled(w.x, p.sel23, sr);
                    v[4 * o + 2] = e4m3x2_scaled(w.y, p.sel01, sr);
                    v[4 * o + 3] = e4m3x2_scaled(w.y, p.sel23, sr);
                }
            }
            tmem_st32(tmem + ((uint32_t)(quad * 32) << 16) + NP + s2 * kAColumns, v);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(cv_full(s2)) : "memory");
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(raw_empty(s)) : "memory");
            }
        }
        // accumulator -> fp32 partial tile [token][accumulator row] in this CTA's (now idle) raw ring
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
                for (int i = 0; i < 16; ++i) red[(c0 + i) * kTileM + lrow] = __uint_as_float(r[i]);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
    }
    __syncwarp();

    // ---- every CTA of the cluster adds one slice of accumulator rows over all ranks (descending rank, fixed order)
    // through distributed shared memory and writes that slice of C ----
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (warp >= 2) {
        const int etid = tid - 64;
        // slices in units of four accumulator rows: one 16-byte distributed-shared-memory load per rank brings four
        // rows of one token, which are four consecutive weight rows (and output elements)
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
            const int row = tile * kTileM + rho;       // accumulator rows are the tile's rows in natural order
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
            // four consecutive bf16 outputs, 8-byte aligned (row is a multiple of 4, m a multiple of 128)
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
        for (int i = max(0, raw_issued - STAGES); i < raw_issued; ++i) mbar_wait(raw_full(i % STAGES), (i / STAGES) & 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

template <int NP>
const void* f8_kernel_for_stages(int stages) {
    switch (stages) {
        case 2: return reinterpret_cast<const void*>(dense_umma_f8_kernel<NP, 2>);
        case 3: return reinterpret_cast<const void*>(dense_umma_f8_kernel<NP, 3>);
        case 4: return reinterpret_cast<const void*>(dense_umma_f8_kernel<NP, 4>);
        case 6: return reinterpret_cast<const void*>(dense_umma_f8_kernel<NP, 6>);
        case 8: return reinterpret_cast<const void*>(dense_umma_f8_kernel<NP, 8>);
    }
    return nullptr;
}

}  // namespace

// stages: depth of the raw e4m3 ring (2, 3, 4, 6, 8; 8 KB each); cluster_k: 1..8 CTAs per 128-row tile.
int launch_dense_umma_f8(const DenseParams& p, int stages, int cluster_k, int* status, cudaStream_t stream) {
    if (!p.A || !p.X || !p.C) return fail(kInvalidArg, "dense: null pointer");
    if (p.x_layout != 0) return fail(kUnsupported, "dense (tcgen05): activations must be row-major");
    if (p.m % kTileM != 0 || p.k % kBlockK != 0) return fail(kInvalidArg, "dense (tcgen05): need m %% 128 == 0 and k %% 64 == 0");
    if (p.n < 1 || p.n > 64) return fail(kUnsupported, "dense (tcgen05): 1..64 tokens per launch (got %d)", p.n);
    if (p.c_layout == 1 && p.n % 16 != 0) return fail(kInvalidArg, "dense: layout C needs n %% 16 == 0");
    if (((uintptr_t)p.A & 15) || ((uintptr_t)p.X & 15)) return fail(kInvalidArg, "dense (tcgen05): A and B must be 16-byte aligned");
    if (encode_fn() == nullptr) return fail(kUnsupported, "dense (tcgen05): cuTensorMapEncodeTiled is not available");
    if (cluster_k < 1 || cluster_k > 8) return fail(kInvalidArg, "dense (tcgen05, e4m3): cluster split must be 1..8 (got %d)", cluster_k);
    if (cluster_k > p.k / kBlockK) return fail(kInvalidArg, "dense (tcgen05): cluster split %d exceeds the %d k blocks", cluster_k, p.k / kBlockK);
    const int np = p.n <= 16 ? 16 : (p.n <= 32 ? 32 : 64);
    const void* kern = np == 16 ? f8_kernel_for_stages<16>(stages) : (np == 32 ? f8_kernel_for_stages<32>(stages) : f8_kernel_for_stages<64>(stages));
    if (kern == nullptr) return fail(kInvalidArg, "dense (tcgen05, e4m3): stages must be one of 2, 3, 4, 6, 8 (got %d)", stages);
    // 128 tensor-memory columns per CTA: never more than four CTAs on an SM
    const size_t smem = prepare_kernel(kern, 192, std::max((size_t)stages * kRawBytes, (size_t)np * 512) + (size_t)conv_stages(np) * np * 128 + 1024, 128);
    if (smem == 0) return fail(kCudaError, "dense (tcgen05, e4m3): a CTA with %d stages does not fit on this device", stages);
    CUtensorMap ma, mx;
    if (!make_map_a8(&ma, p.A, p.m, p.k)) return fail(kUnsupported, "dense (tcgen05): weight tensor map rejected");
    if (!make_map_x(&mx, p.X, p.n, p.k, kBF16, np)) return fail(kUnsupported, "dense (tcgen05): activation tensor map rejected");
    F8Params fp{};
    fp.C = p.C; fp.bias = p.bias; fp.alpha = p.alpha; fp.m = p.m; fp.n = p.n; fp.k = p.k; fp.c_layout = p.c_layout;
    fp.kblocks = p.k / kBlockK;
    fp.sel01 = p.fp8_order ? kSelRep01 : kSelNat01;
    fp.sel23 = p.fp8_order ? kSelRep23 : kSelNat23;
    fp.scale = p.scale;
    fp.scale_ld = (p.k + 127) / 128;
    fp.full_scales = option(kOptFullScales);
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
    if (e != cudaSuccess) return fail(kCudaError, "dense_umma_f8 launch: %s", cudaGetErrorString(e));
    return kOk;
}

}  // namespace mlk
