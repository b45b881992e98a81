// Row movers around the expert-parallel token exchange (no counterpart in the reference, which is single-GPU:
// its only multi-GPU hook is the experts_map argument, csrc/moe_kernels/moe_align_tokens.h:46-49).
//
//   gather_rows:     out[i, :] = x[idx[i], :]                       -- builds the dispatch send buffer
//   unpermute_sum:   y[t, :]   = round16( sum_j float(rows[pos[t*topk + j], :]) ), j ascending, pos < 0 skipped
//                                                                     -- combine: the weighted expert outputs come
//                                                                     back in send order; each token adds its topk
//                                                                     rows in fp32 in a fixed order, one rounding
// Both are 16-byte-per-thread copies, HBM/L2 bound, launched on the caller's stream; rows are 16-bit, H % 8 == 0.
#include "common.cuh"
#include "moe.cuh"
#include "status.h"

namespace mlk {

namespace {

__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ idx,
                                                         uint4* __restrict__ out, long long n_rows, int octs,
                                                         long long x_rows) {
    const long long total = n_rows * octs;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / octs;
        const int o = (int)(i - r * octs);
        const long long src = idx[r];
        out[i] = (src >= 0 && src < x_rows) ? x[src * octs + o] : make_uint4(0, 0, 0, 0);
    }
}

template <int WT, bool ROWS32>
__global__ void __launch_bounds__(256) unpermute_sum_kernel(const void* __restrict__ rows_,
                                                           const int32_t* __restrict__ pos, uint4* __restrict__ y,
                                                           long long T, int topk, int octs, long long n_rows) {
    const long long total = T * octs;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / octs;
        const int o = (int)(i - t * octs);
        float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < topk; ++j) {
            const long long p = pos[t * topk + j];
            if (p < 0 || p >= n_rows) continue;
            if constexpr (ROWS32) {
                const float4* src = reinterpret_cast<const float4*>(rows_) + (p * octs + o) * 2;
                const float4 u = src[0], w = src[1];
                a[0] += u.x; a[1] += u.y; a[2] += u.z; a[3] += u.w;
                a[4] += w.x; a[5] += w.y; a[6] += w.z; a[7] += w.w;
            } else {
                const uint4 v = reinterpret_cast<const uint4*>(rows_)[p * octs + o];
                const float2 v0 = unpack2<WT>(v.x), v1 = unpack2<WT>(v.y), v2 = unpack2<WT>(v.z), v3 = unpack2<WT>(v.w);
                a[0] += v0.x; a[1] += v0.y; a[2] += v1.x; a[3] += v1.y;
                a[4] += v2.x; a[5] += v2.y; a[6] += v3.x; a[7] += v3.y;
            }
        }
        uint4 out;
        out.x = pack2<WT>(a[0], a[1]);
        out.y = pack2<WT>(a[2], a[3]);
        out.z = pack2<WT>(a[4], a[5]);
        out.w = pack2<WT>(a[6], a[7]);
        y[i] = out;
    }
}

int grid_for(long long total) {
    long long b = (total + 255) / 256;
    const long long cap = 8LL * sm_count();
    if (b > cap) b = cap;
    return (int)(b < 1 ? 1 : b);
}

}  // namespace

int launch_gather_rows(const void* x, const int32_t* idx, void* out, long long n_rows, int H, long long x_rows,
                       cudaStream_t s) {
    if (n_rows < 0 || H <= 0 || H % 8 != 0) return fail(kInvalidArg, "moe_gather_rows: need H %% 8 == 0 and n_rows >= 0");
    if (n_rows == 0) return kOk;
    if (!x || !idx || !out) return fail(kInvalidArg, "moe_gather_rows: null pointer");
    const int octs = H / 8;
    gather_rows_kernel<<<grid_for(n_rows * octs), 256, 0, s>>>((const uint4*)x, idx, (uint4*)out, n_rows, octs, x_rows);
    return check_launch("moe_gather_rows");
}

int launch_unpermute_sum(const void* rows, const int32_t* pos, void* y, long long T, int topk, int H, long long n_rows,
                         int dtype, cudaStream_t s) {
    if (T < 0 || topk <= 0 || H <= 0 || H % 8 != 0) return fail(kInvalidArg, "moe_unpermute_sum: bad sizes");
    if (dtype < 0 || dtype > 3) return fail(kInvalidArg, "moe_unpermute_sum: dtype code must be 0..3");
    if (T == 0) return kOk;
    if (!pos || !y || (n_rows > 0 && !rows)) return fail(kInvalidArg, "moe_unpermute_sum: null pointer");
    const int octs = H / 8;
    const int g = grid_for(T * octs);
    switch (dtype) {
        case 0: unpermute_sum_kernel<kBF16, false><<<g, 256, 0, s>>>(rows, pos, (uint4*)y, T, topk, octs, n_rows); break;
        case 1: unpermute_sum_kernel<kFP16, false><<<g, 256, 0, s>>>(rows, pos, (uint4*)y, T, topk, octs, n_rows); break;
        case 2: unpermute_sum_kernel<kBF16, true><<<g, 256, 0, s>>>(rows, pos, (uint4*)y, T, topk, octs, n_rows); break;
        default: unpermute_sum_kernel<kFP16, true><<<g, 256, 0, s>>>(rows, pos, (uint4*)y, T, topk, octs, n_rows); break;
    }
    return check_launch("moe_unpermute_sum");
}

}  // namespace mlk
