// Pieces shared by the tcgen05 / tensor-memory kernels: PTX wrappers (mbarrier, TMA, tcgen05), shared-memory and
// instruction descriptors, and the tensor-map helpers of the host side.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "status.h"

namespace mlk {
namespace umma {

constexpr int kTileM = 128;
constexpr int kBlockK = 64;                       // k elements per stage
constexpr int kABytes = kTileM * kBlockK * 2;     // 16 KB
constexpr uint32_t kSpinLimit = 1u << 20;         // try_wait attempts before giving up (about a second at worst)

// ---- PTX wrappers ---------------------------------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; false = gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// The same load with an L2 eviction hint: weights are read exactly once per launch, so their lines are marked
// evict-first and leave the L2 to what is re-read (token tiles, the expert outputs the combine reads back).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                                 uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d_hint(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3,
                                                 uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Same with the A operand in tensor memory (lane = row, one 32-bit column = two consecutive k elements).
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 consecutive columns of this thread's tensor-memory lane (the warp covers its 32-lane quarter).
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
          "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
          "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}

// Shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets in 16-byte units,
// version 1, layout type in bits 61..63 (0 = no swizzle, 2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)layout << 61;
    return d;
}

template <int WT, int NP>
constexpr uint32_t instr_desc() {
    // D = f32 (1 << 4); A, B formats at bits 7 / 10 (0 = f16, 1 = bf16); both K-major; N >> 3 at 17; M >> 4 at 24
    constexpr uint32_t fmt = (WT == kFP16) ? 0u : 1u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(NP >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
}


__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(ptr);
    });
    return fn;
}

// ---- host: tensor-map cache ---------------------------------------------------------------------------------
// Encoding a tensor map costs about a microsecond of host time, and a serving loop launches the same (pointer, shape)
// pairs over and over: the maps of the last launches are kept per host thread, keyed by what determines them.
template <class Build>
inline bool cached_map(CUtensorMap* out, int kind, const void* ptr, long long a, long long b, long long c, Build&& build) {
    struct Entry {
        int kind;
        const void* ptr;
        long long a, b, c;
        bool valid;
        CUtensorMap map;
    };
    constexpr int kEntries = 128;
    thread_local Entry cache[kEntries] = {};
    unsigned long long h = (unsigned long long)(uintptr_t)ptr * 0x9E3779B97F4A7C15ull;
    h ^= (unsigned long long)a * 0xC2B2AE3D27D4EB4Full + (unsigned long long)b * 0x165667B19E3779F9ull +
         (unsigned long long)c * 0x27D4EB2F165667C5ull + (unsigned long long)kind;
    Entry& e = cache[(h >> 32) % kEntries];
    if (e.valid && e.kind == kind && e.ptr == ptr && e.a == a && e.b == b && e.c == c) {
        std::memcpy(out, &e.map, sizeof(CUtensorMap));
        return true;
    }
    if (!build(out)) return false;
    e.kind = kind; e.ptr = ptr; e.a = a; e.b = b; e.c = c; e.valid = true;
    std::memcpy(&e.map, out, sizeof(CUtensorMap));
    return true;
}

// ---- host: per-kernel launch preparation -------------------------------------------------------------------
// Tensor memory has 512 columns per SM and tcgen05.alloc blocks until its request fits.  A CTA that holds its columns
// and waits at a cluster barrier for a peer that is itself blocked in tcgen05.alloc on another SM would never be
// released, so a launch must not let more CTAs of one kernel become resident on an SM than their allocations allow.
// prepare_kernel raises the kernel's dynamic shared-memory limit (only ever upwards, once per kernel, device and size)
// and returns the dynamic shared-memory size to launch with: `smem`, padded where necessary until at most
// 512 / tmem_cols CTAs fit on an SM (the kernels carve their buffers from the front, the padding stays unused).
// 0 = the kernel cannot be launched this way on the current device.  *resident receives the CTAs per SM.
inline size_t prepare_kernel(const void* kern, int threads, size_t smem, int tmem_cols, bool big_clusters = false,
                             int* resident = nullptr) {
    struct Prepared {
        size_t launch_smem;
        int resident;
    };
    static std::mutex mu;
    static std::unordered_map<unsigned long long, Prepared> done;     // (kernel, device, smem, columns) -> result
    static std::unordered_map<unsigned long long, size_t> attr_max;   // (kernel, device) -> limit set so far
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    const unsigned long long kd = (unsigned long long)(uintptr_t)kern * 64ull + (unsigned)(dev & 63);
    const unsigned long long key = kd * 0x9E3779B97F4A7C15ull ^ ((unsigned long long)smem << 12) ^ (unsigned)tmem_cols;
    std::lock_guard<std::mutex> lock(mu);
    auto it = done.find(key);
    if (it != done.end()) {
        if (resident) *resident = it->second.resident;
        return it->second.launch_smem;
    }
    int optin = 0;
    if (cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return 0;
    if (big_clusters) cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);   // up to 16 CTAs
    const int limit = tmem_cols > 0 ? 512 / tmem_cols : 1 << 30;
    Prepared r{0, 0};
    for (size_t s = smem; s <= (size_t)optin; s += 2048) {
        size_t& cur = attr_max[kd];
        if (s > cur) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s) != cudaSuccess) break;
            cur = s;
        }
        int occ = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, threads, s) != cudaSuccess || occ < 1) break;
        if (occ <= limit) {
            r.launch_smem = s;
            r.resident = occ;
            break;
        }
    }
    cudaGetLastError();     // a failed probe must not leak into the caller's next error check
    done[key] = r;
    if (resident) *resident = r.resident;
    return r.launch_smem;
}

inline bool make_map_x(CUtensorMap* map, const void* X, int n, int k, int wt, int np) {
    return cached_map(map, 1, X, n, k, wt * 1024 + np, [&](CUtensorMap* m) {
        const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)n};
        const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
        const cuuint32_t box[2] = {kBlockK, (cuuint32_t)np};
        const cuuint32_t estr[2] = {1, 1};
        return encode_fn()(m, wt == kFP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                           const_cast<void*>(X), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    });
}

// e4m3 weight tile map: global layout A is [row group][k-octet][16 rows][8 bytes]; a 3-D view (128-byte block,
// k-octet, row group) with box (128, 8, 8) lands a 128 x 64 tile as [row group][k-octet][16 rows x 8 bytes].
inline bool make_map_a8(CUtensorMap* map, const void* A, long long m, int k) {
    return cached_map(map, 2, A, m, k, 0, [&](CUtensorMap* mp) {
        const cuuint64_t dims[3] = {128, (cuuint64_t)(k / 8), (cuuint64_t)(m / 16)};
        const cuuint64_t strides[2] = {128, (cuuint64_t)16 * k};
        const cuuint32_t box[3] = {128, kBlockK / 8, kTileM / 16};
        const cuuint32_t estr[3] = {1, 1, 1};
        return encode_fn()(mp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(A), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    });
}

// Token tile map for activations in layout B [k/32][n/16][4 k-octets][16 tokens][8 k]: viewed as (one 8-token x 8-k
// core matrix of 128 bytes, token half, 16-token block, k-octet, 32-k chunk) with box (64, 2, np/16, 4, 2), the tile
// of np tokens x 64 k lands as [k-octet (8)][8-token group (np/8)][128 B]: the UMMA no-swizzle K-major layout with a
// k-octet step of np * 16 bytes and an 8-token step of 128 bytes.  Token blocks beyond n are zero-filled.
inline bool make_map_xb(CUtensorMap* map, const void* X, int n, int k, int wt, int np) {
    return cached_map(map, 3, X, n, k, wt * 1024 + np, [&](CUtensorMap* m) {
        const cuuint64_t dims[5] = {64, 2, (cuuint64_t)(n / 16), 4, (cuuint64_t)(k / 32)};
        const cuuint64_t strides[4] = {128, 1024, 256, (cuuint64_t)(n / 16) * 1024};
        const cuuint32_t box[5] = {64, 2, (cuuint32_t)(np / 16), 4, kBlockK / 32};
        const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        return encode_fn()(m, wt == kFP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5,
                           const_cast<void*>(X), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    });
}

// 16-bit weight tile map.  Global layout A is [row group][k-octet][half][8 rows][8 k]; the 4-D view (64 elements =
// one 8-row core matrix, k-octet, row group, half) with box (64, 8, 8, 2) is traversed k-octet first, so each row
// group's 2 KB run of a k block is fetched as consecutive requests, and lands in shared memory as
// [half][row group][k-octet][128 B]: core matrix (accumulator 8-row group i = 8*half + row group, k-octet o) sits at
// i*1024 + o*128, uniform strides for one M = 128 descriptor.  `rows` may span several matrices stored back to back
// (the experts of a fused-MoE weight tensor).
inline bool make_map_a16(CUtensorMap* map, const void* A, long long rows, int k, int wt) {
    return cached_map(map, 4, A, rows, k, wt, [&](CUtensorMap* m) {
        const cuuint64_t dims[4] = {64, (cuuint64_t)(k / 8), (cuuint64_t)(rows / 16), 2};
        const cuuint64_t strides[3] = {256, (cuuint64_t)16 * k * 2, 128};
        const cuuint32_t box[4] = {64, kBlockK / 8, kTileM / 16, 2};
        const cuuint32_t estr[4] = {1, 1, 1, 1};
        return encode_fn()(m, wt == kFP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                           const_cast<void*>(A), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    });
}

}  // namespace umma
}  // namespace mlk
