/*
 * C ABI of the B200 native-layout kernel library (libmlk_b200.so).
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, launches hand-written
 * sm_100a kernels on that stream and returns a status code.  No entry point allocates device
 * memory, synchronises the host or throws.  Each one replaces one operator of the reference
 * extension module `muxi_layout_kernels_ext` (reference file:line given per function);
 * "dim letters" follow the reference: m = weight rows (output features), n = tokens, k = reduction,
 * C[n,m] = alpha * B[n,k] * A[m,k]^T (+ bias[m]).
 *
 * dtype codes: 0 = bf16, 1 = fp16, 2 = e4m3 weights with bf16 activations ("soft FP8").
 */
#ifndef MLK_B200_H_
#define MLK_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* mlk_stream_t; /* == cudaStream_t */

enum {
    MLK_OK = 0,
    MLK_ERR_INVALID_ARG = 1, /* a precondition the reference enforces with TORCH_CHECK is violated */
    MLK_ERR_UNSUPPORTED = 2, /* valid request no kernel of this build implements */
    MLK_ERR_CUDA = 3,        /* a CUDA runtime call failed */
    MLK_ERR_IO = 4           /* dispatch table file could not be opened */
};

enum { MLK_BF16 = 0, MLK_FP16 = 1, MLK_E4M3 = 2 };

/* Dispatch tables, one per packaged CSV file (reference: csrc/arg_selector.cu:80,157,232,303,375,454,531). */
enum {
    MLK_TABLE_GEMM_ABC = 0,           /* layout_gemm_dispatch_arg.csv            */
    MLK_TABLE_GEMM_CONTINUOUS_C = 1,  /* continuous_gemm_dispatch_arg.csv        */
    MLK_TABLE_GEMM_LAYOUT_A = 2,      /* layoutA_gemm_dispatch_arg.csv           */
    MLK_TABLE_GEMM_LAYOUT_A_FP8 = 3,  /* layoutA_Soft_Fp8_gemm_dispatch_arg.csv  */
    MLK_TABLE_GEMV_FP16 = 4,          /* layout_gemv_dispatch_arg.csv            */
    MLK_TABLE_GEMV_BF16 = 5,          /* layout_gemv_bf16_dispatch_arg.csv       */
    MLK_TABLE_GEMV_FP8 = 6            /* layout_gemv_soft_fp8_dispatch_arg.csv   */
};

/* ---- library ------------------------------------------------------------------------------- */

const char* mlk_status_string(int status);
/* Message of the last failing call on the calling thread ("" if none). */
const char* mlk_last_error(void);
/* Build identification: "sm_100a" plus the ABI version. */
const char* mlk_build_info(void);

/* Library-wide options.
 *   MLK_OPT_PDL (default 1): kernels are launched with programmatic stream serialization, so a kernel may become
 *     resident while its predecessor in the stream drains; every kernel waits (griddepcontrol.wait) before it reads
 *     anything an earlier kernel may have written and before it writes anything.
 *   MLK_OPT_STATIC_WEIGHTS (default 0): promise that weight tensors (A, w1, w2, block scales) are not written by any
 *     kernel of the calling stream while these ops are in flight (weights prepacked once, the serving situation).
 *     The dense kernels then start streaming weights before that wait.  Leave it 0 if a kernel that produces
 *     weights (e.g. mlk_layoutA) can immediately precede a GEMM on the same stream.
 *   MLK_OPT_FULL_SCALES (default 0): how the tcgen05 e4m3 kernels apply a 128x128 block scale s in the decode.
 *     0: s is rounded to bf16 and folded into the decode's one packed multiply: weight = rne_bf16(w * bf16(s)), no
 *        extra instruction (unit scales, powers of two and other 8-bit scales are exact);
 *     1: s enters as two bf16 terms (16 significant bits) through a packed multiply and a packed fused multiply-add:
 *        weight = rne_bf16(w * s) up to a 2^-17 slip of the rounding boundary, what the reference's torch recipe
 *        dequantises to (muxi_layout_kernels/utils.py:14-25); the decode is the bottleneck of these kernels, so
 *        this costs throughput (measured: 1.2-1.6x the time).
 *     The reference's kernels truncate fp32(w) * s to bf16; every form stays within one bf16 ulp per weight of the
 *     exact product.  The warp-level kernels (kernelId 1, 3, 4) apply s to the fp32 sums of each 128-wide k block.
 *   MLK_OPT_WAIT_LOG2 (default 0 = built-in, 24): log2 of the number of polls mlk_ep_reduce_shares waits for a peer GPU
 *     before it gives up (4..30).  Smaller values turn a missing peer into an error status sooner. */
enum { MLK_OPT_PDL = 0, MLK_OPT_STATIC_WEIGHTS = 1, MLK_OPT_FULL_SCALES = 2, MLK_OPT_WAIT_LOG2 = 3 };
int mlk_set_option(int option_id, int value);
int mlk_get_option(int option_id);

/* ---- dispatch tables (reference: csrc/arg_selector.cu:14-87, class per table) ------------------ */

/* Reads a CSV table (header line + integer rows).  A file that cannot be opened yields MLK_ERR_IO and
 * leaves the table empty, i.e. every lookup falls back to the shape-based default. */
int mlk_table_load(int table, const char* csv_path);
/* Exact-key lookup; out4 = {kernelId,p1,p2,p3} for GEMM tables, {BLOCK_DIM_X,KernelId,p1,p2} for GeMV
 * tables (n is ignored there).  *hit is 1 when the key was present, 0 when the default was returned. */
int mlk_table_lookup(int table, int m, int n, int k, int out4[4], int* hit);
const char* mlk_table_file_name(int table);

/* ---- prepack ops ---------------------------------------------------------------------------- */

/* W[m,k] row-major -> layout A [m/16][k/8][16][8] (inverse != 0: back).  elem_bytes 2 (bf16/fp16) or 1 (e4m3).
 * The reference builds this layout with torch view/permute (benchmark_and_test/gemm_benchmark.py:41-42). */
int mlk_layoutA(const void* in, void* out, int64_t m, int64_t k, int elem_bytes, int inverse, mlk_stream_t s);
/* B[n,k] row-major 16-bit -> layout B [k/32][n/16][4][16][8].  Reference: layoutB, csrc/layout_b.cu:65-99. */
int mlk_layoutB(const void* B, void* B_out, int n, int k, mlk_stream_t s);
/* Layout C [m/32][n/16][4][16][8] 16-bit -> C[n,m] row-major.  Reference: reLayoutC, csrc/re_layout_c.cu:63-95. */
int mlk_reLayoutC(const void* C_in, void* C_out, int m, int n, mlk_stream_t s);
/* Bytes [b0,b1,b2,b3] of every 32-bit word -> [b0,b2,b1,b3]; its own inverse.
 * Reference: fp8_weight_repack, csrc/fp8_weight_repack.cu:44-67. */
int mlk_fp8_weight_repack(const void* weight, void* out, int64_t nbytes, mlk_stream_t s);

/* Scratch lent to one call (device pointers); every GeMV / GEMM entry point takes one, NULL = none.
 * workspace: fp32 scratch, any content: mlk_gemm_workspace_bytes(m, n, k) bytes cover every kernel of that shape.
 * counters: >= m/128 ints that are zero on entry; every kernel leaves them zero again, so one block per stream can be
 * reused by successive calls.  status: one int, sticky error word of the bounded waits inside the tcgen05 kernels
 * (0 = ok), may be NULL.  A kernel whose wait expired leaves its output unwritten (and, in the persistent stream-K
 * mode, possibly non-zero counters): clear the counters and the word before the block is used again. */
typedef struct mlk_aux {
    void* workspace;
    int64_t workspace_bytes;
    int32_t* counters;
    int32_t n_counters;
    int32_t* status;
} mlk_aux;

/* Workspace size (bytes) that covers every kernelId-2 launch of this shape on the current device; 0 if the shape
 * cannot use that kernel. */
int64_t mlk_gemm_workspace_bytes(int m, int n, int k);
/* Workspace size (bytes, 128-byte aligned) the native-e4m3 kernels (GEMM kernelId 9, GeMV KernelId 4) need for n tokens
 * of k elements: 1 KB of token scales plus 2 k bytes per token for the activations rewritten as two e4m3 terms; 0 if
 * those kernels cannot run (n > 64, k % 64 != 0). */
int64_t mlk_soft_fp8_workspace_bytes(int n, int k);

/* ---- GeMV: y[1,m] = alpha * A x (+ bias) ------------------------------------------------------- */

/* Explicit tuning arguments.  Reference: gemv_layoutA_wapper, csrc/gemv_layout_a.cu:17-71.
 *   kernelId 1: tensor-core streaming kernel, kernelParam1 = row groups per warp (1,2), kernelParam2 = split-K (1,2,4,8)
 *   kernelId 2: CUDA-core FMA + shuffle kernel, same two parameters (bf16/fp16 only)
 *   kernelId 3: e4m3 only, m % 128 == 0, k % 64 == 0: the TMA -> convert -> tcgen05 pipeline of the
 *               soft-FP8 GEMM (see kernelId 2 there); kernelParam1 = raw ring stages (2,3,4,6,8), kernelParam2 =
 *               cluster size (1..8), blockDimX ignored
 *   kernelId 4: e4m3 only, no scale_matrix, m % 128 == 0: the weights go to the 8-bit tensor-core MMA undecoded (see
 *               kernelId 9 of the narrow GEMM); blockDimX = k per stage (64; 128 or 256 = 128, k a multiple of it),
 *               kernelParam1 = ring stages (2,3,4,6,8), kernelParam2 = cluster size (1..8); needs aux->workspace of
 *               mlk_soft_fp8_workspace_bytes(1, k) bytes
 *   scale_matrix: e4m3 only, fp32 [ceil(m/128)][ceil(k/128)], may be NULL (= all ones)
 *   fp8_order: 0 natural bytes, 1 bytes as written by mlk_fp8_weight_repack
 *   beta is accepted and ignored, as in the reference kernels. */
int mlk_gemv_layoutA_wapper(const void* A, const void* x, void* y, int m, int k, int dtype, float alpha, float beta,
                            int blockDimX, int kernelId, int kernelParam1, int kernelParam2,
                            const float* scale_matrix, const void* bias, int fp8_order, const mlk_aux* aux,
                            mlk_stream_t s);
/* Table-driven.  Reference: gemv_layoutA, csrc/gemv_layout_a.cu:73-150. */
int mlk_gemv_layoutA(const void* A, const void* x, void* y, int m, int k, int dtype, float alpha, float beta,
                     const float* scale_matrix, const void* bias, int fp8_order, const mlk_aux* aux, mlk_stream_t s);

/* ---- narrow GEMM: C[n,m] = alpha * B A^T (+ bias), n <= 256 ------------------------------------------- */

/* kernelId 1, 3, 4 (warp-level tensor-core streaming kernel with 256, 128, 64 threads per CTA, any n <= 256):
 *   kernelParam1 = row groups per warp (1,2), kernelParam2 = row warps per CTA (1,2,4,8; the other warps split K),
 *   kernelParam3 = split-K over a thread-block cluster (1,2,4,8).
 * kernelId 2 (tcgen05 / tensor-memory tile kernel, 16-bit weights, row-major B, n <= 64): persistent CTAs that split
 *   the (128-row tile, 64-wide k block) work units evenly; kernelParam1 = CTAs per SM the grid is sized for (1..4),
 *   kernelParam2 = TMA pipeline stages (2,3,4,5,6,8), kernelParam3 = 0 or 1.  Splitting tiles between CTAs needs
 *   the caller-provided scratch below; without it the kernel runs one CTA per tile.
 *   kernelParam3 = 2..16 selects the other decomposition of the same kernel: one thread-block cluster of that many
 *   CTAs per 128-row tile, each CTA streaming an equal share of k, partial tiles added through distributed shared
 *   memory (no scratch needed; kernelParam1 is ignored).
 *   With e4m3 weights (soft_fp8 entry points) kernelId 2 is the TMA -> convert -> tcgen05 pipeline: the e4m3
 *   tile is decoded to bf16 into tensor memory by the four warps that later run the epilogue;
 *   kernelParam2 = stages of the raw e4m3 ring (2,3,4,6,8), kernelParam3 = cluster size (1..8), kernelParam1 ignored.
 *   Block scales are applied in the decode as rne_bf16(w * s), the weight the reference's torch recipe
 *   (muxi_layout_kernels/utils.py:14-25) dequantises to; kernelId 1, 3, 4 apply s to the fp32 sums of each 128-wide
 *   k block instead, and the reference's kernels truncate fp32(w) * s to bf16: all within one bf16 ulp per weight.
 * kernelId 9 (soft_fp8 entry points, no block scales, row-major B, n <= 64): the e4m3 weight bytes are fed to
 *   tcgen05.mma.kind::f8f6f4 as they are (moved from the TMA-landed tile into tensor memory, no arithmetic), and a small
 *   kernel in front rewrites the bf16 activations as two e4m3 terms each (hi + lo, exact under a power-of-two scale per
 *   token chosen from the token's largest magnitude), so every product is exact and is accumulated in fp32.
 *   kernelParam1 = k per stage (64 or 128; 0 / 1 = 64), kernelParam2 = ring stages (2,3,4,6,8), kernelParam3 = cluster
 *   size (1..8).  Needs aux->workspace of mlk_soft_fp8_workspace_bytes(n, k) bytes, 128-byte aligned.  Differences a
 *   caller can see: an e4m3 NaN byte (0x7F, 0xFF) in the weights is a NaN (the decode kernels, like the reference's,
 *   read it as +-480); activations more than 2^11 below the largest magnitude of their token lose low bits (absolute
 *   error <= 2^-17 of that maximum per element); a token that holds an Inf or NaN yields NaN outputs.  The table-driven
 *   entry point uses it by default and falls back to kernelId 2 (same kernelParam2 / 3) when a scale tensor is
 *   passed or the scratch is missing.
 * kernelId 5, 6, 7 (CUDA-core FMA + shuffle kernel with 256, 128, 64 threads; 16-bit weights, row-major B and C,
 *   n <= 4): kernelParam1 = row groups per warp (1,2), kernelParam2 unused, kernelParam3 = cluster split-K. */

/* A layout A, B row-major [n,k], C row-major [n,m].  Reference: gemm_layoutA_wapper, csrc/gemm_layout_A.cu:684-750. */
int mlk_gemm_layoutA_wapper(const void* A, const void* B, void* C, int m, int n, int k, int dtype, float alpha,
                            float beta, int kernelParam1, int kernelParam2, int kernelParam3, int kernelId,
                            const void* bias, const mlk_aux* aux, mlk_stream_t s);
/* Reference: gemm_layoutA, csrc/gemm_layout_A.cu:752-787. */
int mlk_gemm_layoutA(const void* A, const void* B, void* C, int m, int n, int k, int dtype, float alpha, float beta,
                     const void* bias, const mlk_aux* aux, mlk_stream_t s);
/* e4m3 A with fp32 128x128 block scales (NULL = ones), bf16 B and C.
 * Reference: gemm_layoutA_soft_fp8_wapper, csrc/gemm_layout_A_soft_fp8.cu:749. */
int mlk_gemm_layoutA_soft_fp8_wapper(const void* A, const float* A_scale, const void* B, void* C, int m, int n, int k,
                                     float alpha, float beta, int kernelParam1, int kernelParam2, int kernelParam3,
                                     int kernelId, const void* bias, int fp8_order, const mlk_aux* aux, mlk_stream_t s);
/* Reference: gemm_layoutA_soft_fp8, csrc/gemm_layout_A_soft_fp8.cu:825. */
int mlk_gemm_layoutA_soft_fp8(const void* A, const float* A_scale, const void* B, void* C, int m, int n, int k,
                              float alpha, float beta, const void* bias, int fp8_order, const mlk_aux* aux,
                              mlk_stream_t s);
/* Many-token GEMM on the same prepacked weights (any n; the prefill-side consumer of layout A): 16-bit weights with more
 * than 64 tokens run on a tcgen05 tile kernel with 128 x 128 or 128 x 256 (weight rows x tokens) tiles and the whole k
 * range per CTA (kernelId 10 of mlk_gemm_layoutA_wapper: kernelParam1 = tokens per tile, kernelParam2 = ring stages);
 * e4m3 weights (scale_matrix NULL = unit scales) and calls with few tokens run the narrow kernels 64 tokens at a time.
 * Reference: muxi_hgemm_layoutA, csrc/muxi_hgemm_layoutA.cu:12-217 (beta accepted and ignored; the reference adds
 * beta * C of its own freshly allocated C). */
int mlk_muxi_hgemm_layoutA(const void* A, const float* scale_matrix, const void* B, void* C, int m, int n, int k, int dtype,
                           float alpha, float beta, const void* bias, int fp8_order, const mlk_aux* aux, mlk_stream_t s);
/* A layout A, B layout B, C row-major.  Reference: gemm_layoutAB_ContinuousC_wapper,
 * csrc/gemm_layout_ab_continuous_c.cu:982; table-driven form :1051. */
int mlk_gemm_layoutAB_ContinuousC_wapper(const void* A, const void* B, void* C, int m, int n, int k, int dtype,
                                         float alpha, float beta, int kernelParam1, int kernelParam2,
                                         int kernelParam3, int kernelId, const void* bias, const mlk_aux* aux,
                                         mlk_stream_t s);
int mlk_gemm_layoutAB_ContinuousC(const void* A, const void* B, void* C, int m, int n, int k, int dtype, float alpha,
                                  float beta, const void* bias, const mlk_aux* aux, mlk_stream_t s);
/* A layout A, B layout B, C layout C.  Reference: gemm_layoutABC_wapper, csrc/gemm_layout_abc.cu:685;
 * table-driven form :754. */
int mlk_gemm_layoutABC_wapper(const void* A, const void* B, void* C, int m, int n, int k, int dtype, float alpha,
                              float beta, int kernelParam1, int kernelParam2, int kernelParam3, int kernelId,
                              const void* bias, const mlk_aux* aux, mlk_stream_t s);
int mlk_gemm_layoutABC(const void* A, const void* B, void* C, int m, int n, int k, int dtype, float alpha, float beta,
                       const void* bias, const mlk_aux* aux, mlk_stream_t s);

/* ---- fused MoE ("plan C") ------------------------------------------------------------------------ */

/* Router: softmax (score_fun 0) or sigmoid (1) of gating_output[T,E] (bf16/fp16, dtype code 0/1), optional
 * per-expert selection bias, group-limited top-k with "lower id wins" ties; writes experts_ids int32 [T,topK]
 * and the un-biased scores selected_experts_weights [T,topK] (same dtype as the logits).
 * Any E <= 256 divisible by n_groups, any topK_groups <= n_groups, topK <= 32.
 * Reference: fused_routing_gate, csrc/moe_kernels/fused_gating.cu:5-67 (kernels fused_topK.h:24,332). */
int mlk_fused_routing_gate(const void* gating_output, int score_fun, int batch_size, int num_experts, int n_groups,
                           int topK_groups, int32_t* experts_ids, void* selected_experts_weights, int topK,
                           const void* load_balance_bias, int dtype, mlk_stream_t s);

/* Same, with the weights of every token divided by their sum when renormalize != 0 (the step the reference's Python
 * orchestrator does with two torch ops, muxi_layout_kernels/muxi_moe_planC.py:69-70): fp32 sum rounded to the logits'
 * dtype, fp32 quotient rounded to the logits' dtype. */
int mlk_fused_routing_gate_renorm(const void* gating_output, int score_fun, int batch_size, int num_experts,
                                  int n_groups, int topK_groups, int32_t* experts_ids, void* selected_experts_weights,
                                  int topK, const void* load_balance_bias, int dtype, int renormalize, mlk_stream_t s);

/* Router GEMM fused with the routing (no counterpart in the reference, whose fused_moe starts from gating_output):
 * logits[t, e] = sum_h x[t, h] * gate_weight[e, h] in fp32, rounded once to the activation dtype -- what a 16-bit linear
 * layer would hand to the router -- followed by exactly the routing of mlk_fused_routing_gate_renorm.  x [T, H] and
 * gate_weight [E, H] row-major in the activation dtype, 16-byte aligned, H % 8 == 0.  logits_out: optional [T, E] copy
 * of the rounded logits (NULL to skip).  Meant for decode batches: one CTA per four tokens re-reads the gate matrix. */
int mlk_fused_router_gemm_gate(const void* x, const void* gate_weight, int score_fun, int batch_size, int hidden_size,
                               int num_experts, int n_groups, int topK_groups, int32_t* experts_ids,
                               void* selected_experts_weights, int topK, const void* load_balance_bias, int dtype,
                               int renormalize, void* logits_out, mlk_stream_t s);

/* Token alignment: groups the flat slots i = token*topK + j by (mapped) expert, pads every expert's run to a
 * multiple of microBatchSize with the caller's sentinel, and records one expert id per block.
 *   sorted_token_ids  [T*topK + E*(mbs-1)]  every position that holds no slot is set to the sentinel T*topK (the
 *                     reference expects the caller to pre-fill it; doing so is harmless)
 *   cumsum_buffer     [E+1]   on return: [e] = start_e + count_e for e < E, [E] = padded total
 *   padded_num_experts[1]     number of blocks
 *   experts_ids_out   [ceil(len/mbs)] expert of each block
 *   experts_map       [experts_map_len] global -> local expert id or -1, may be NULL; an id outside the map
 *                     is skipped like a -1 entry
 * Reference: batched_routed_activation_indexed_to_expert_block_indexed, csrc/moe_kernels/fused_experts_compute.cu:6-48. */
int mlk_moe_align(int batchSize, int expertCount, int topK, int microBatchSize, const int32_t* topk_ids,
                  int32_t* sorted_token_ids, int32_t* cumsum_buffer, int32_t* padded_num_experts,
                  int32_t* experts_ids_out, const int32_t* experts_map, int experts_map_len, mlk_stream_t s);

/* Expert compute: alignment, gather-GEMM1 with fused SiLU*up, GEMM2 with fused routing-weight scale, then the
 * un-permute and sum over each token's topK experts.  w1 [E,2I,H] (gate rows then up rows) and w2 [E,H,I], each
 * expert in layout A; x [T,H]; topk_ids/topk_weights [T,topK]; C is caller workspace of T*topK*2I elements;
 * y [T,H] must be zero.
 * dtype 0/1: 16-bit weights; dtype 2: e4m3 weights with optional fp32 block scales w1_scale [E,2I/128,H/128],
 * w2_scale [E,H/128,I/128] (NULL = ones).
 * tune: NULL, or six host ints {token tiles per work item (1,2,4,8 = 8..64 slots), row warps of GEMM1 (1,2,4),
 * cluster split-K of GEMM1 (1,2,4,8), row groups per warp of GEMM2 (1,2), row warps of GEMM2 (1,2,4), cluster split-K of
 * GEMM2}; a 0 lets the library choose that value from the shape.  Values of the two "row warps" fields select
 * the kernel family:
 *     1, 2, 4        warp-level mma.sync kernels (any shape, 16-bit atomics or fp32 combine)
 *     100 + stages   tcgen05 kernels, 16-bit weights or e4m3 decoded to bf16 on the way into tensor memory (block
 *                    scales allowed); needs hidden % 128 == 0, inter % 128 == 0 and a combine scratch; token tiles
 *                    per work item may then also be 16 (128 slots, 16-bit weights only)
 *     200 + stages   tcgen05 kernels that multiply the e4m3 weight bytes undecoded (kind::f8f6f4): the routed token
 *                    rows and the activation are rewritten as two e4m3 terms under a per-row power-of-two scale.
 *                    e4m3 weights without block scales only; with scales or 16-bit weights the same row runs as
 *                    100 + stages.  For this family "cluster split-K of GEMM2" = 10 + R (R = 1..8) selects the
 *                    second-GEMM kernel without a cluster in which one CTA walks R consecutive 128-row tiles of
 *                    the same work item.  240 + stages (instead of 200 + stages) streams 128 k per ring stage
 *                    where that form is built: the second GEMM without a cluster (inter % 128 == 0) and the first
 *                    GEMM with 64-slot token tiles, 2 or 3 stages, no cluster (hidden % 128 == 0); elsewhere it
 *                    runs as 200 + stages.
 *     300            decode batches (batch_size <= 8, batch_size * topK <= 64): the whole expert compute as one
 *                    cooperative kernel, see mlk_fused_routing_experts_compute; larger batches run the library's choice
 *   Both fields name the same family; a mixed pair, or a tcgen05 family on a call that cannot use it, runs the
 *   warp-level kernels with the library's own values.  ring stages: 2..8.
 * status: one device int, sticky error word of the bounded waits inside the tcgen05 expert kernels (0 = ok), or NULL.
 * out_fp32 != 0 (needs combine_scratch): y is [T, H] fp32 and receives the un-rounded sums over this rank's experts,
 *   so that an expert-parallel caller can add the ranks' shares before the one rounding.
 * combine_scratch: optional T*topK*H floats.  With it the weighted expert outputs are kept in fp32 and summed per
 * token in a fixed order with one final rounding (bit-reproducible).  With NULL they are accumulated into y with
 * 16-bit atomics, as the reference does (csrc/moe_kernels/group_gemm_second.h:333-346): one rounding per addend
 * and an unspecified order.
 * Reference: fused_experts_compute (both overloads), csrc/moe_kernels/fused_experts_compute.cu:50-188,190-296. */
int mlk_fused_experts_compute(const void* w1, const void* w2, const void* x, int batch_size, int expert_count,
                              int topK, int hidden, int inter, const int32_t* topk_ids, const void* topk_weights,
                              int32_t* sorted_token_ids, int32_t* cumsum_buffer, int32_t* padded_num_experts,
                              int32_t* experts_ids, void* C, void* y, const float* w1_scale, const float* w2_scale,
                              int dtype, int fp8_order, int microBatchSize, const int32_t* experts_map,
                              int experts_map_len, float* combine_scratch, int64_t combine_scratch_bytes,
                              const int32_t* tune, int32_t* status, int out_fp32, mlk_stream_t s);

/* Routing and expert compute in one call: mlk_fused_routing_gate_renorm on gating_output [batch_size, num_experts]
 * (arguments as there; topk_ids and topk_weights are OUTPUTS here) followed by mlk_fused_experts_compute (all other
 * arguments as there).  Same results as the two calls.  For decode batches -- at most 8 tokens and 64 routed slots,
 * num_experts <= 256, both "row warps" fields of tune >= 300 -- the whole layer is one cooperative kernel, one CTA per
 * SM: every CTA routes the tokens for itself, a producer warp streams the CTA's share of both weight matrices through a
 * 192 KB shared-memory ring with bulk copies, sixteen consumer warps multiply the segments as they land, one bounded
 * grid barrier separates the two GEMMs, and the per-token sums are formed in the CTA that owns the output rows (no
 * combine scratch needed on that path).  Every other call runs the router kernel and then the expert compute.
 * (The same tuning values on mlk_fused_experts_compute run the decode kernel without the routing.)
 * Reference: the sequence issued by muxi_layout_kernels/muxi_moe_planC.py:56-149. */
int mlk_fused_routing_experts_compute(const void* gating_output, int num_experts, int score_fun, int n_groups,
                                      int topK_groups, const void* gating_bias, int renormalize, const void* w1,
                                      const void* w2, const void* x, int batch_size, int expert_count, int topK,
                                      int hidden, int inter, int32_t* topk_ids, void* topk_weights,
                                      int32_t* sorted_token_ids, int32_t* cumsum_buffer, int32_t* padded_num_experts,
                                      int32_t* experts_ids, void* C, void* y, const float* w1_scale,
                                      const float* w2_scale, int dtype, int fp8_order, int microBatchSize,
                                      const int32_t* experts_map, int experts_map_len, float* combine_scratch,
                                      int64_t combine_scratch_bytes, const int32_t* tune, int32_t* status, int out_fp32,
                                      mlk_stream_t s);

/* Expert compute for callers that must not allocate device memory (a plugin running under another runtime's memory
 * pool, a serving loop whose allocator is off limits on the request path).  It has no
 * counterpart in the reference.  Same arguments (tune and status included) and results as mlk_fused_experts_compute
 * with a combine scratch, except that the scratch is a device array built into the library: 8 MiB per GPU that loads the library, held
 * until the process exits, which limits batch_size * topK * hidden to 2 Mi (2097152) floats -- larger calls fail
 * with MLK_ERR_INVALID_ARG.  The first call on a device looks the array's address up; make that call before any
 * stream capture.  All calls share the array: calls that overlap on the GPU (different streams) race on it. */
int mlk_fused_experts_compute_static(const void* w1, const void* w2, const void* x, int batch_size, int expert_count,
                                     int topK, int hidden, int inter, const int32_t* topk_ids, const void* topk_weights,
                                     int32_t* sorted_token_ids, int32_t* cumsum_buffer, int32_t* padded_num_experts,
                                     int32_t* experts_ids, void* C, void* y, const float* w1_scale,
                                     const float* w2_scale, int dtype, int fp8_order, int microBatchSize,
                                     const int32_t* experts_map, int experts_map_len, const int32_t* tune,
                                     int32_t* status, int out_fp32, mlk_stream_t s);

/* ---- expert-parallel token exchange (no counterpart in the reference, which is single-GPU) ------------------ */

/* out[i,:] = x[idx[i],:] for n_rows rows of `hidden` 16-bit elements (hidden % 8 == 0); an index outside
 * [0, x_rows) gives a zero row.  Builds the send buffer of the dispatch all-to-all. */
int mlk_moe_gather_rows(const void* x, const int32_t* idx, void* out, int64_t n_rows, int hidden, int64_t x_rows,
                        mlk_stream_t s);
/* y[t,:] = round( sum_j float(rows[pos[t*topK + j],:]) ), j ascending, entries with pos outside [0, n_rows) skipped.
 * Combine step: `rows` are the weighted expert outputs as they come back from the combine all-to-all.
 * dtype: 0 / 1 = rows and y in bf16 / fp16; 2 / 3 = rows in fp32 (un-rounded weighted outputs), y in bf16 / fp16. */
int mlk_moe_unpermute_sum(const void* rows, const int32_t* pos, void* y, int64_t T, int topK, int hidden,
                          int64_t n_rows, int dtype, mlk_stream_t s);

/* Expert-parallel combine over peer memory (NVLink / NVSwitch), one kernel per rank instead of an all-reduce and a
 * cast: rank i adds rows [T i / world, T (i + 1) / world) of every rank's fp32 share [T, hidden] in rank order, rounds
 * once to `dtype` (0 = bf16, 1 = fp16) and stores the finished rows into every rank's output [T, hidden].
 *   shares_dev / outs_dev / flags_dev: DEVICE arrays of `world` pointers -- every rank's share, output and flag block,
 *   all peer-accessible (symmetric memory, IPC or cuMemMap'd allocations).  A flag block is
 *   mlk_ep_reduce_flag_bytes() bytes, zero before the first call and owned by these calls from then on.
 *   recv_dev: NULL, or the same kind of array for every rank's receive buffer of mlk_ep_reduce_recv_bytes(world, T,
 *   hidden) bytes (0 = share too large).  With it, shares of at most min(256 Ki, 1 Mi / world) elements take a one-pass
 *   form without any barrier: every rank stores its share into every peer's receive buffer as (value, epoch) pairs and
 *   adds, in rank order, what it receives as the pairs land; every rank computes the whole output itself.
 * All ranks must issue the same sequence of calls (same T, hidden).  The launch is capturable in a CUDA graph.  Waits on
 * peers are bounded: on expiry *status (may be NULL) receives 0x0E000001 and the output of that call is incomplete.
 * The kernels use plain loads and stores on the peer pointers, no TMA, no multicast. */
int64_t mlk_ep_reduce_flag_bytes(void);
int64_t mlk_ep_reduce_recv_bytes(int world, int64_t T, int hidden);
int mlk_ep_reduce_shares(const void* const* shares_dev, void* const* outs_dev, void* const* flags_dev, void* const* recv_dev,
                         int rank, int world, int64_t T, int hidden, int dtype, int32_t* status, mlk_stream_t s);

#ifdef __cplusplus
}
#endif

#endif /* MLK_B200_H_ */
