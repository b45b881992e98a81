// Layout permutations: pure 8/16-byte chunk moves, HBM-bound.
//
//   layout A  (weights):      A4[g][o][r][e]      = A[16g + r][8o + e]
//       reference recipe: benchmark_and_test/gemm_benchmark.py:41-42 (done with torch view/permute there;
//       a device op here so that 100+ MB weights are prepacked at copy speed)
//   layout B  (activations):  B5[c][nb][q][r][e]  = B[16nb + r][32c + 8q + e]     csrc/layout_b.cu:65-99
//   layout C  (outputs):      C[16nb + r][32mb + 8q + e] = C5[mb][nb][q][r][e]    csrc/re_layout_c.cu:63-95
//   fp8 repack: bytes [b0,b1,b2,b3] of every aligned 32-bit word -> [b0,b2,b1,b3]  csrc/fp8_weight_repack.cu:35-36
//
// Every kernel is grid-stride with one chunk group per thread; the side that cannot be contiguous
// per thread is made contiguous across the lanes of a warp (r is the fastest thread index).
#include <cuda_runtime.h>
#include <stdint.h>

#include "status.h"

namespace mlk {

namespace {

template <typename V>   // V = uint4 (16-bit elements) or uint2 (8-bit elements): one 8-element chunk
__global__ void layout_a_kernel(const V* __restrict__ in, V* __restrict__ out, long long groups, int octets,
                                int inverse) {
    // one thread per (g, octet pair, r): two chunks that are adjacent in the row-major matrix
    const int pairs = (octets + 1) >> 1;
    const long long total = groups * pairs * 16;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i & 15);
        const long long gp = i >> 4;
        const int op = (int)(gp % pairs);
        const long long g = gp / pairs;
        const long long rm = (g * 16 + r) * octets + 2 * op;          // row-major chunk index
        const long long la = (g * octets + 2 * op) * 16 + r;          // layout-A chunk index
        const bool two = 2 * op + 1 < octets;
        if (!inverse) {
            out[la] = in[rm];
            if (two) out[la + 16] = in[rm + 1];
        } else {
            out[rm] = in[la];
            if (two) out[rm + 1] = in[la + 16];
        }
    }
}

__global__ void layout_b_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int n, int kchunks) {
    // one thread per (c, nb, r): 4 chunks = 64 contiguous bytes of one token row
    const int NB = n >> 4;
    const long long total = (long long)kchunks * NB * 16;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i & 15);
        const long long cn = i >> 4;
        const int nb = (int)(cn % NB);
        const long long c = cn / NB;
        const uint4* src = in + ((long long)(nb * 16 + r) * kchunks + c) * 4;
        uint4* dst = out + (c * NB + nb) * 64 + r;
#pragma unroll
        for (int q = 0; q < 4; ++q) dst[q * 16] = src[q];
    }
}

__global__ void relayout_c_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int n, int mblocks) {
    // one thread per (mb, nb, r): reads 4 chunks 256 bytes apart, writes 64 contiguous bytes
    const int NB = n >> 4;
    const long long total = (long long)mblocks * NB * 16;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i & 15);
        const long long mn = i >> 4;
        const int nb = (int)(mn % NB);
        const long long mb = mn / NB;
        const uint4* src = in + (mb * NB + nb) * 64 + r;
        uint4* dst = out + ((long long)(nb * 16 + r) * mblocks + mb) * 4;
#pragma unroll
        for (int q = 0; q < 4; ++q) dst[q] = src[q * 16];
    }
}

__device__ __forceinline__ uint32_t swap12(uint32_t w) { return __byte_perm(w, 0u, 0x3120); }

__global__ void fp8_repack_kernel16(const uint4* __restrict__ in, uint4* __restrict__ out, long long n16) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n16;
         i += (long long)gridDim.x * blockDim.x) {
        uint4 v = in[i];
        v.x = swap12(v.x); v.y = swap12(v.y); v.z = swap12(v.z); v.w = swap12(v.w);
        out[i] = v;
    }
}

__global__ void fp8_repack_kernel4(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, long long n4) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x)
        out[i] = swap12(in[i]);
}

int grid_for(long long total, int block) {
    long long b = (total + block - 1) / block;
    const long long cap = 16LL * sm_count();   // 16 CTAs of 256 threads fill an SM; grid-stride covers the rest
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (int)b;
}

}  // namespace

int launch_layout_a(const void* in, void* out, long long m, long long k, int elem_bytes, int inverse,
                    cudaStream_t stream) {
    if (!in || !out) return fail(kInvalidArg, "layoutA: null pointer");
    if (m <= 0 || k <= 0 || m % 16 != 0 || k % 8 != 0)
        return fail(kInvalidArg, "layoutA: need m %% 16 == 0 and k %% 8 == 0 (m=%lld k=%lld)", m, k);
    if (elem_bytes != 1 && elem_bytes != 2) return fail(kInvalidArg, "layoutA: element size must be 1 or 2 bytes");
    const long long groups = m / 16;
    const int octets = (int)(k / 8);
    const long long total = groups * ((octets + 1) / 2) * 16;
    const int grid = grid_for(total, 256);
    if (elem_bytes == 2)
        layout_a_kernel<uint4><<<grid, 256, 0, stream>>>((const uint4*)in, (uint4*)out, groups, octets, inverse);
    else
        layout_a_kernel<uint2><<<grid, 256, 0, stream>>>((const uint2*)in, (uint2*)out, groups, octets, inverse);
    return check_launch("layoutA");
}

int launch_layout_b(const void* in, void* out, int n, int k, cudaStream_t stream) {
    if (!in || !out) return fail(kInvalidArg, "layoutB: null pointer");
    if (n <= 0 || n % 16 != 0) return fail(kInvalidArg, "n must be a multiple of 16");
    if (k <= 0 || k % 32 != 0) return fail(kInvalidArg, "k must be a multiple of 32");
    const long long total = (long long)(k / 32) * n;
    layout_b_kernel<<<grid_for(total, 256), 256, 0, stream>>>((const uint4*)in, (uint4*)out, n, k / 32);
    return check_launch("layoutB");
}

int launch_relayout_c(const void* in, void* out, int m, int n, cudaStream_t stream) {
    if (!in || !out) return fail(kInvalidArg, "reLayoutC: null pointer");
    if (n <= 0 || n % 16 != 0) return fail(kInvalidArg, "reLayoutC: n must be a multiple of 16");
    if (m <= 0 || m % 32 != 0) return fail(kInvalidArg, "reLayoutC: m must be a multiple of 32");
    const long long total = (long long)(m / 32) * n;
    relayout_c_kernel<<<grid_for(total, 256), 256, 0, stream>>>((const uint4*)in, (uint4*)out, n, m / 32);
    return check_launch("reLayoutC");
}

int launch_fp8_repack(const void* in, void* out, long long nbytes, cudaStream_t stream) {
    if (!in || !out) return fail(kInvalidArg, "fp8_weight_repack: null pointer");
    if (nbytes < 0 || nbytes % 4 != 0)
        return fail(kInvalidArg, "fp8_weight_repack: byte count must be a multiple of 4 (got %lld)", nbytes);
    if (nbytes == 0) return kOk;
    const bool vec = (nbytes % 16 == 0) && ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0);
    if (vec) {
        const long long n16 = nbytes / 16;
        fp8_repack_kernel16<<<grid_for(n16, 256), 256, 0, stream>>>((const uint4*)in, (uint4*)out, n16);
    } else {
        const long long n4 = nbytes / 4;
        fp8_repack_kernel4<<<grid_for(n4, 256), 256, 0, stream>>>((const uint32_t*)in, (uint32_t*)out, n4);
    }
    return check_launch("fp8_weight_repack");
}

}  // namespace mlk
