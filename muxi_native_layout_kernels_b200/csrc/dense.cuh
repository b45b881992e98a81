// Host-visible description of one dense launch (GeMV and the three narrow-GEMM variants).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mlk {

struct DenseParams {
    const void* A;        // weights, layout A [m/16][k/8][16][8]
    const void* X;        // activations: row-major [n,k] or layout B [k/32][n/16][4][16][8]
    void* C;              // output: row-major [n,m] or layout C [m/32][n/16][4][16][8]
    const void* bias;     // [m] in the activation dtype, or null
    const float* scale;   // e4m3 only: [ceil(m/128)][ceil(k/128)] fp32 block scales, or null
    int m, n, k;
    float alpha;
    int x_layout;         // 0 row-major, 1 layout B
    int c_layout;         // 0 row-major, 1 layout C
    int fp8_order;        // 0 natural byte order, 1 order written by fp8_weight_repack
    // tuning
    int rg;               // row groups per warp (1 or 2)          -- "APerWarp"
    int wm;               // row warps per CTA (1,2,4,8)
    int sk;               // cluster split-K (1,2,4,8)
    int threads;          // CTA size (64,128,256)
};

// Caller-provided scratch for kernels that split K over independent CTAs (all pointers device memory).
struct DenseAux {
    void* workspace;             // fp32 partial tiles, any content
    long long workspace_bytes;
    int* counters;               // zero on entry; every kernel leaves them zero again
    int n_counters;
    int* status;                 // sticky error word, 0 = ok; may be null
};

// wt: kBF16 / kFP16 / kE4M3.  Returns an mlk status code.
int launch_dense_mma(int wt, const DenseParams& p, cudaStream_t stream);
int launch_dense_umma(int wt, const DenseParams& p, int ctas_per_sm, int stages, int cluster_k, const DenseAux* aux,
                      cudaStream_t stream);
long long umma_workspace_bytes(int m, int n, int k, int sms, int ctas_per_sm);
// e4m3 weights through the TMA -> convert -> tcgen05 pipeline (block scales applied in the decode); status may be null
int launch_dense_umma_f8(const DenseParams& p, int stages, int cluster_k, int* status, cudaStream_t stream);
// e4m3 weights handed to tcgen05.mma.kind::f8f6f4 undecoded, activations rewritten as two e4m3 terms by a kernel in
// front (dense_umma_f8n.cu); scratch: f8n_scratch_bytes(n, k) bytes, 128-byte aligned, owned by the call until it completes
long long f8n_scratch_bytes(int n, int k);
int f8n_max_k();   // longest row the activation split handles
int launch_dense_umma_f8n(const DenseParams& p, int bk, int stages, int cluster_k, void* scratch, long long scratch_bytes,
                          int* status, cudaStream_t stream);
// many-token GEMM on the tcgen05 tile kernel (hgemm_umma.cu): nt = tokens per tile (128, 256; 0 = automatic), 16-bit weights
int launch_hgemm_umma(int wt, const DenseParams& p, int nt, int stages, int* status, cudaStream_t stream);
int launch_gemv_simt(int wt, const DenseParams& p, int rows_per_warp_log2, cudaStream_t stream);

}  // namespace mlk
