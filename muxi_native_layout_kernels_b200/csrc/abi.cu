// extern "C" entry points declared in include/mlk_b200.h: argument checks, table lookup, dispatch.
#include "../../include/mlk_b200.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "dense.cuh"
#include "moe.cuh"
#include "selector.h"
#include "status.h"

namespace mlk {

namespace {
thread_local char g_err[512] = {0};
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
const char* last_error() { return g_err; }
void clear_error() { g_err[0] = 0; }

namespace {
int g_options[kNumOptions] = {1, 0, 0, 0};
}
int option(int which) { return (which >= 0 && which < kNumOptions) ? g_options[which] : 0; }
void set_option(int which, int value) {
    if (which >= 0 && which < kNumOptions) g_options[which] = value;
}

int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    int& c = cached[dev & 63];
    if (c == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        c = v;
    }
    return c;
}

int launch_layout_a(const void*, void*, long long, long long, int, int, cudaStream_t);
int launch_layout_b(const void*, void*, int, int, cudaStream_t);
int launch_relayout_c(const void*, void*, int, int, cudaStream_t);
int launch_fp8_repack(const void*, void*, long long, cudaStream_t);

namespace {

int wt_of(int dtype) {
    switch (dtype) {
        case MLK_BF16: return kBF16;
        case MLK_FP16: return kFP16;
        case MLK_E4M3: return kE4M3;
    }
    return -1;
}

// The reference's GEMM entry points require m % 128 == 0 and k % 128 == 0 (csrc/gemm_layout_A.cu:774-776).
int check_gemm_shape(int m, int n, int k) {
    if (m <= 0 || n <= 0 || k <= 0) return fail(kInvalidArg, "gemm: m, n, k must be positive");
    if (m % 128 != 0) return fail(kInvalidArg, "m must be a multiple of 128 (m=%d)", m);
    if (k % 128 != 0) return fail(kInvalidArg, "k must be a multiple of 128 (k=%d)", k);
    return kOk;
}

int gemm_table(int table, int variant_x, int variant_c, const void* A, const float* scale, const void* B, void* C,
               int m, int n, int k, int dtype, float alpha, const void* bias, int fp8_order, cudaStream_t s,
               const mlk_aux* aux);

// The many-token tile kernel gives every CTA the whole k range, so it wants about as many (128-row, 128-token) tiles as
// there are SMs.  With fewer tiles and at most 256 tokens the narrow kernels (k split over clusters), 64 tokens per
// launch, finish sooner although they stream the weights once per launch.
bool few_tiles_for_hgemm(int m, int n) { return n <= 256 && (long long)(m / 128) * ((n + 127) / 128) * 10 < 7LL * sm_count(); }

int gemm_in_token_chunks(int table, const void* A, const float* scale, const void* B, void* C, int m, int n, int k, int dtype,
                         float alpha, const void* bias, int fp8_order, cudaStream_t s, const mlk_aux* aux) {
    for (int n0 = 0; n0 < n; n0 += 64) {
        const int nn = n - n0 < 64 ? n - n0 : 64;
        const void* Bc = reinterpret_cast<const uint8_t*>(B) + (size_t)n0 * k * 2;
        void* Cc = reinterpret_cast<uint8_t*>(C) + (size_t)n0 * m * 2;
        if (int st = gemm_table(table, 0, 0, A, scale, Bc, Cc, m, nn, k, dtype, alpha, bias, fp8_order, s, aux)) return st;
    }
    return kOk;
}

int gemm_common(int variant_x, int variant_c, const void* A, const float* scale, const void* B, void* C, int m, int n,
                int k, int dtype, float alpha, int p1, int p2, int p3, int kernelId, const void* bias, int fp8_order,
                cudaStream_t s, const mlk_aux* aux = nullptr) {
    clear_error();
    const int wt = wt_of(dtype);
    if (wt < 0) return fail(kInvalidArg, "Unsupported data type code %d", dtype);
    if (int st = check_gemm_shape(m, n, k)) return st;
    DenseParams p{};
    p.A = A; p.X = B; p.C = C; p.bias = bias; p.scale = scale;
    p.m = m; p.n = n; p.k = k; p.alpha = alpha;
    p.x_layout = variant_x; p.c_layout = variant_c; p.fp8_order = fp8_order;
    if (kernelId == 10) {
        // many-token tile kernel (hgemm_umma.cu): kernelParam1 = tokens per tile (128, 256; 0 = automatic), kernelParam2 =
        // ring stages (2, 3, 4, 6; 0 = automatic)
        if (wt == kE4M3) return fail(kUnsupported, "gemm: kernelId 10 takes 16-bit weights");
        if (variant_x != 0 || variant_c != 0) return fail(kUnsupported, "gemm: kernelId 10 needs row-major B and C");
        if (p1 <= 1 && few_tiles_for_hgemm(m, n)) return gemm_in_token_chunks(kTableGemmLayoutA, A, nullptr, B, C, m, n, k, dtype, alpha, bias, 0, s, aux);
        return launch_hgemm_umma(wt, p, p1 == 1 ? 0 : p1, p2 == 1 ? 0 : p2, aux ? aux->status : nullptr, s);
    }
    if (kernelId == 9) {
        // e4m3 weights undecoded into tcgen05.mma.kind::f8f6f4: kernelParam1 = k per stage (64, or 128; 0 / 1 = 64),
        // kernelParam2 = ring stages, kernelParam3 = cluster size
        if (wt != kE4M3) return fail(kUnsupported, "gemm: kernelId 9 takes e4m3 weights");
        if (variant_c != 0 && n % 16 != 0) return fail(kInvalidArg, "gemm: layout C needs n %% 16 == 0");
        return launch_dense_umma_f8n(p, p1 <= 1 ? 64 : p1, p2, p3 < 1 ? 1 : p3, aux ? aux->workspace : nullptr,
                                     aux ? (long long)aux->workspace_bytes : 0, aux ? aux->status : nullptr, s);
    }
    if (kernelId == 2 && wt == kE4M3) {
        // TMA -> convert -> tcgen05 pipeline for e4m3 weights: kernelParam2 = raw ring stages, kernelParam3 = cluster
        // size; block scales ride on the decode (rounded to bf16 first, as the reference's torch check does)
        if (variant_c != 0 && n % 16 != 0) return fail(kInvalidArg, "gemm: layout C needs n %% 16 == 0");
        return launch_dense_umma_f8(p, p2, p3 < 1 ? 1 : p3, aux ? aux->status : nullptr, s);
    }
    if (kernelId == 2) {
        DenseAux da{};
        if (aux) {
            da.workspace = aux->workspace; da.workspace_bytes = aux->workspace_bytes; da.counters = aux->counters;
            da.n_counters = aux->n_counters; da.status = aux->status;
        }
        return launch_dense_umma(wt, p, p1, p2, p3, aux ? &da : nullptr, s);
    }
    if (kernelId >= 5 && kernelId <= 7) {
        // CUDA-core FMA kernel for 1..4 tokens; 5 / 6 / 7 = 256 / 128 / 64 threads; kernelParam1 = row groups per
        // warp, kernelParam3 = cluster split-K
        if (variant_x != 0 || variant_c != 0) return fail(kUnsupported, "gemm: the CUDA-core kernel needs row-major B and C");
        p.rg = p1; p.wm = 1; p.sk = p3; p.threads = kernelId == 5 ? 256 : (kernelId == 6 ? 128 : 64);
        return launch_gemv_simt(wt, p, 0, s);
    }
    if (kernelId != 1 && kernelId != 3 && kernelId != 4)
        return fail(kUnsupported, "gemm: kernelId %d is not built (1, 3, 4 = warp-level streaming kernel with 256, 128, 64 threads; 2 = tcgen05 tile kernel)", kernelId);
    p.rg = p1; p.wm = p2; p.sk = p3; p.threads = kernelId == 1 ? 256 : (kernelId == 3 ? 128 : 64);
    return launch_dense_mma(wt, p, s);
}

int gemm_table(int table, int variant_x, int variant_c, const void* A, const float* scale, const void* B, void* C,
               int m, int n, int k, int dtype, float alpha, const void* bias, int fp8_order, cudaStream_t s,
               const mlk_aux* aux) {
    clear_error();
    if (int st = check_gemm_shape(m, n, k)) return st;
    TuneArgs t = global_table(table).get(m, n, k, nullptr);
    // A table row that this shape cannot run with (e.g. copied from another GPU's table) falls back to the default.
    const int twarps = t.a == 1 ? 8 : (t.a == 3 ? 4 : (t.a == 4 ? 2 : 0));
    const bool ok1 = twarps > 0 && (t.b == 1 || t.b == 2) && (t.c == 1 || t.c == 2 || t.c == 4 || t.c == 8) &&
                     t.c <= twarps && (t.d == 1 || t.d == 2 || t.d == 4 || t.d == 8) && m % (16 * t.b * t.c) == 0;
    const bool ok2 = t.a == 2 && (variant_x == 0 || dtype != MLK_E4M3) && n <= 64 &&
                     (dtype != MLK_E4M3
                          ? (t.b >= 1 && t.b <= 4 && ((t.c >= 2 && t.c <= 6) || t.c == 8) && t.d >= 0 && t.d <= 16)
                          : ((t.c == 2 || t.c == 3 || t.c == 4 || t.c == 6 || t.c == 8) && t.d >= 1 && t.d <= 8));
    const bool have_f8n = dtype == MLK_E4M3 && scale == nullptr && variant_x == 0 && n <= 64 && k <= f8n_max_k() && aux != nullptr &&
                          aux->workspace != nullptr && ((uintptr_t)aux->workspace & 127) == 0 &&
                          aux->workspace_bytes >= f8n_scratch_bytes(n, k);
    const bool ok9 = t.a == 9 && have_f8n && (t.b <= 1 || t.b == 64 || t.b == 128) &&
                     (t.c == 2 || t.c == 3 || t.c == 4 || t.c == 6 || t.c == 8) && t.d >= 1 && t.d <= 8 &&
                     t.d <= k / (t.b == 128 ? 128 : 64);
    const bool ok5 = t.a >= 5 && t.a <= 7 && n <= 4 && variant_x == 0 && variant_c == 0 && dtype != MLK_E4M3 &&
                     (t.b == 1 || t.b == 2) && (t.d == 1 || t.d == 2 || t.d == 4 || t.d == 8) && m % (16 * t.b) == 0;
    const bool ok10 = t.a == 10 && variant_x == 0 && variant_c == 0 && dtype != MLK_E4M3 && (t.b == 0 || t.b == 128 || t.b == 256) &&
                      (t.c == 0 || t.c == 2 || t.c == 3 || t.c == 4 || t.c == 6) &&
                      (t.c == 0 || (size_t)t.c * (16384 + (t.b == 128 ? 128 : 256) * 128) + 1024 <= 227 * 1024);
    if (!ok1 && !ok2 && !ok5 && !ok9 && !ok10) t = default_args(table, m, n, k);
    // the native-e4m3 kernel needs the caller's scratch and has no block scales; otherwise the decode pipeline runs
    // (kernelParam2 = raw ring stages and kernelParam3 = cluster size mean the same there)
    if (t.a == 9 && !have_f8n) t.a = 2;
    // the tcgen05 kernel reads through tensor maps, which want 16-byte aligned bases; e4m3 activations in layout B
    // have no tcgen05 variant
    if ((t.a == 2 || t.a == 9 || t.a == 10) && ((((uintptr_t)A | (uintptr_t)C | (uintptr_t)B) & 15) != 0 || (variant_x != 0 && dtype == MLK_E4M3)))
        t = warp_level_default_args(table, m, n, k);
    return gemm_common(variant_x, variant_c, A, scale, B, C, m, n, k, dtype, alpha, t.b, t.c, t.d, t.a, bias,
                       fp8_order, s, aux);
}

}  // namespace
}  // namespace mlk

using namespace mlk;

extern "C" {

const char* mlk_status_string(int status) {
    switch (status) {
        case MLK_OK: return "ok";
        case MLK_ERR_INVALID_ARG: return "invalid argument";
        case MLK_ERR_UNSUPPORTED: return "unsupported";
        case MLK_ERR_CUDA: return "CUDA error";
        case MLK_ERR_IO: return "I/O error";
    }
    return "unknown status";
}

const char* mlk_last_error(void) { return last_error(); }

const char* mlk_build_info(void) { return "mlk_b200 abi 1, sm_100a"; }

int mlk_set_option(int option_id, int value) {
    clear_error();
    if (option_id < 0 || option_id >= kNumOptions) return fail(kInvalidArg, "unknown option %d", option_id);
    set_option(option_id, value);
    return kOk;
}
int mlk_get_option(int option_id) { return option(option_id); }

int64_t mlk_soft_fp8_workspace_bytes(int n, int k) {
    if (n <= 0 || n > 64 || k <= 0 || k % 64 != 0 || k > f8n_max_k()) return 0;
    return f8n_scratch_bytes(n, k);
}

int64_t mlk_gemm_workspace_bytes(int m, int n, int k) {
    if (m <= 0 || n <= 0 || k <= 0 || m % 128 != 0 || k % 64 != 0 || n > 64) return 0;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return 0;
    long long best = 0;
    for (int c = 1; c <= 4; ++c) {
        const long long b = umma_workspace_bytes(m, n, k, sms, c);
        best = b > best ? b : best;
    }
    return best;
}

int mlk_table_load(int table, const char* csv_path) {
    clear_error();
    if (table < 0 || table >= kNumTables) return fail(kInvalidArg, "table id %d out of range", table);
    if (!csv_path) return fail(kInvalidArg, "null path");
    if (global_table(table).load(csv_path) != 0) return fail(kIoError, "cannot open %s", csv_path);
    return kOk;
}

int mlk_table_lookup(int table, int m, int n, int k, int out4[4], int* hit) {
    clear_error();
    if (table < 0 || table >= kNumTables) return fail(kInvalidArg, "table id %d out of range", table);
    if (!out4) return fail(kInvalidArg, "null output");
    bool h = false;
    const TuneArgs t = global_table(table).get(m, n, k, &h);
    out4[0] = t.a; out4[1] = t.b; out4[2] = t.c; out4[3] = t.d;
    if (hit) *hit = h ? 1 : 0;
    return kOk;
}

const char* mlk_table_file_name(int table) { return table_file_name(table); }

int mlk_layoutA(const void* in, void* out, int64_t m, int64_t k, int elem_bytes, int inverse, mlk_stream_t s) {
    clear_error();
    return launch_layout_a(in, out, m, k, elem_bytes, inverse, (cudaStream_t)s);
}
int mlk_layoutB(const void* B, void* B_out, int n, int k, mlk_stream_t s) {
    clear_error();
    return launch_layout_b(B, B_out, n, k, (cudaStream_t)s);
}
int mlk_reLayoutC(const void* C_in, void* C_out, int m, int n, mlk_stream_t s) {
    clear_error();
    return launch_relayout_c(C_in, C_out, m, n, (cudaStream_t)s);
}
int mlk_fp8_weight_repack(const void* weight, void* out, int64_t nbytes, mlk_stream_t s) {
    clear_error();
    return launch_fp8_repack(weight, out, nbytes, (cudaStream_t)s);
}

int mlk_gemv_layoutA_wapper(const void* A, const void* x, void* y, int m, int k, int dtype, float alpha, float,
                            int blockDimX, int kernelId, int kernelParam1, int kernelParam2,
                            const float* scale_matrix, const void* bias, int fp8_order, const mlk_aux* aux,
                            mlk_stream_t s) {
    clear_error();
    const int wt = wt_of(dtype);
    if (wt < 0) return fail(kInvalidArg, "Unsupported data type code %d", dtype);
    if (m <= 0 || k <= 0) return fail(kInvalidArg, "gemv: m and k must be positive");
    if (m % 16 != 0) return fail(kInvalidArg, "GEMV m %% 16(at least) must be 0");
    if (k % 32 != 0) return fail(kInvalidArg, "GEMV k %% 32(at least) must be 0");
    DenseParams p{};
    p.A = A; p.X = x; p.C = y; p.bias = bias; p.scale = scale_matrix;
    p.m = m; p.n = 1; p.k = k; p.alpha = alpha;
    p.x_layout = 0; p.c_layout = 0; p.fp8_order = fp8_order;
    p.rg = kernelParam1; p.wm = 1; p.sk = kernelParam2; p.threads = blockDimX;
    if (kernelId == 1) return launch_dense_mma(wt, p, (cudaStream_t)s);
    if (kernelId == 2) return launch_gemv_simt(wt, p, 0, (cudaStream_t)s);
    if (kernelId == 3 && wt == kE4M3) {
        // TMA -> convert -> tcgen05 pipeline: kernelParam1 = raw ring stages, kernelParam2 = cluster size
        return launch_dense_umma_f8(p, kernelParam1, kernelParam2, aux ? aux->status : nullptr, (cudaStream_t)s);
    }
    if (kernelId == 4 && wt == kE4M3) {
        // e4m3 weights undecoded into tcgen05.mma.kind::f8f6f4: blockDimX = k per stage (64, or 128 for 128 and 256),
        // kernelParam1 = ring stages, kernelParam2 = cluster size
        return launch_dense_umma_f8n(p, blockDimX == 64 ? 64 : 128, kernelParam1, kernelParam2, aux ? aux->workspace : nullptr,
                                     aux ? (long long)aux->workspace_bytes : 0, aux ? aux->status : nullptr, (cudaStream_t)s);
    }
    return fail(kUnsupported, "gemv: kernelId %d is not built (1 = tensor-core, 2 = CUDA-core, 3 / 4 = tcgen05 for e4m3)", kernelId);
}

int mlk_gemv_layoutA(const void* A, const void* x, void* y, int m, int k, int dtype, float alpha, float beta,
                     const float* scale_matrix, const void* bias, int fp8_order, const mlk_aux* aux, mlk_stream_t s) {
    clear_error();
    if (m <= 0 || k <= 0) return fail(kInvalidArg, "gemv: m and k must be positive");
    if (m % 16 != 0) return fail(kInvalidArg, "GEMV m %% 16(at least) must be 0");
    if (k % 32 != 0) return fail(kInvalidArg, "GEMV k %% 32(at least) must be 0");
    const int table = dtype == MLK_E4M3 ? kTableGemvSoftFp8 : (dtype == MLK_FP16 ? kTableGemvFp16 : kTableGemvBf16);
    TuneArgs t = global_table(table).get(m, 1, k, nullptr);
    // Same safety net as the reference (csrc/gemv_layout_a.cu:132-143): a row that cannot run falls back.
    const bool ok = (t.a == 64 || t.a == 128 || t.a == 256) && (t.b == 1 || (t.b == 2 && dtype != MLK_E4M3)) &&
                    (t.c == 1 || t.c == 2) && (t.d == 1 || t.d == 2 || t.d == 4 || t.d == 8) && m % (16 * t.c) == 0;
    const bool ok3 = dtype == MLK_E4M3 && t.b == 3 && m % 128 == 0 && k % 64 == 0 &&
                     (t.c == 2 || t.c == 3 || t.c == 4 || t.c == 6 || t.c == 8) && t.d >= 1 && t.d <= 8;
    const bool have_scratch = aux != nullptr && aux->workspace != nullptr && ((uintptr_t)aux->workspace & 127) == 0 &&
                              aux->workspace_bytes >= f8n_scratch_bytes(1, k) && scale_matrix == nullptr && k <= f8n_max_k();
    const bool ok4 = dtype == MLK_E4M3 && t.b == 4 && m % 128 == 0 && k % 64 == 0 && have_scratch && ((uintptr_t)A & 15) == 0 &&
                     ((uintptr_t)x & 15) == 0 && (t.c == 2 || t.c == 3 || t.c == 4 || t.c == 6 || t.c == 8) && t.d >= 1 &&
                     t.d <= 8 && t.d <= k / (t.a == 64 ? 64 : 128) && k % (t.a == 64 ? 64 : 128) == 0;
    if (!ok && !ok3 && !ok4) t = default_args(table, m, 1, k);
    if (t.b == 4 && !(dtype == MLK_E4M3 && m % 128 == 0 && k % (t.a == 64 ? 64 : 128) == 0 && have_scratch &&
                      ((uintptr_t)A & 15) == 0 && ((uintptr_t)x & 15) == 0)) {
        // no scratch, block scales or unaligned operands: the warp-level kernel
        int sk = 1;
        while (sk < 8 && (m / 16) * sk < 2 * sm_count() && (k / 32) / (8 * sk * 2) >= 4) sk *= 2;
        t = TuneArgs{256, 1, 1, sk};
    }
    return mlk_gemv_layoutA_wapper(A, x, y, m, k, dtype, alpha, beta, t.a, t.b, t.c, t.d, scale_matrix, bias,
                                   fp8_order, aux, s);
}

int mlk_gemm_layoutA_wapper(const void* A, const void* B, void* C, int m, int n, int k, int dtype, float alpha, float,
                            int p1, int p2, int p3, int kernelId, const void* bias, const mlk_aux* aux, mlk_stream_t s) {
    if (dtype == MLK_E4M3) { clear_error(); return fail(kInvalidArg, "gemm_layoutA: use the soft_fp8 entry point for e4m3 weights"); }
    return gemm_common(0, 0, A, nullptr, B, C, m, n, k, dtype, alpha, p1, p2, p3, kernelId, bias, 0, (cudaStream_t)s, aux);
}
int mlk_gemm_layoutA(const void* A, const void* B, void* C, int m, int n, int k, int dtype, float alpha, float,
                     const void* bias, const mlk_aux* aux, mlk_stream_t s) {
    if (dtype == MLK_E4M3) { clear_error(); return fail(kInvalidArg, "gemm_layoutA: use the soft_fp8 entry point for e4m3 weights"); }
    return gemm_table(kTableGemmLayoutA, 0, 0, A, nullptr, B, C, m, n, k, dtype, alpha, bias, 0, (cudaStream_t)s, aux);
}
int mlk_gemm_layoutA_soft_fp8_wapper(const void* A, const float* A_scale, const void* B, void* C, int m, int n, int k,
                                     float alpha, float, int p1, int p2, int p3, int kernelId, const void* bias,
                                     int fp8_order, const mlk_aux* aux, mlk_stream_t s) {
    return gemm_common(0, 0, A, A_scale, B, C, m, n, k, MLK_E4M3, alpha, p1, p2, p3, kernelId, bias, fp8_order,
                       (cudaStream_t)s, aux);
}
int mlk_gemm_layoutA_soft_fp8(const void* A, const float* A_scale, const void* B, void* C, int m, int n, int k,
                              float alpha, float, const void* bias, int fp8_order, const mlk_aux* aux, mlk_stream_t s) {
    return gemm_table(kTableGemmLayoutASoftFp8, 0, 0, A, A_scale, B, C, m, n, k, MLK_E4M3, alpha, bias, fp8_order,
                      (cudaStream_t)s, aux);
}
int mlk_muxi_hgemm_layoutA(const void* A, const float* scale_matrix, const void* B, void* C, int m, int n, int k, int dtype,
                           float alpha, float, const void* bias, int fp8_order, const mlk_aux* aux, mlk_stream_t s) {
    clear_error();
    const int wt = wt_of(dtype);
    if (wt < 0) return fail(kInvalidArg, "Unsupported data type code %d", dtype);
    if (m <= 0 || n <= 0 || k <= 0) return fail(kInvalidArg, "muxi_hgemm_layoutA: m, n, k must be positive");
    if (m % 128 != 0) return fail(kInvalidArg, "m must be a multiple of 128 (m=%d)", m);
    if (k % 128 != 0) return fail(kInvalidArg, "k must be a multiple of 128 (k=%d)", k);
    if (wt != kE4M3 && scale_matrix != nullptr) return fail(kInvalidArg, "muxi_hgemm_layoutA: scale_matrix needs 1-byte weights");
    if (wt != kE4M3 && n > 64 && !few_tiles_for_hgemm(m, n)) {
        DenseParams p{};
        p.A = A; p.X = B; p.C = C; p.bias = bias; p.m = m; p.n = n; p.k = k; p.alpha = alpha;
        return launch_hgemm_umma(wt, p, 0, 0, aux ? aux->status : nullptr, (cudaStream_t)s);
    }
    // e4m3 weights, and 16-bit calls with few tokens or few tiles: the narrow kernels, 64 tokens per launch
    return gemm_in_token_chunks(wt == kE4M3 ? kTableGemmLayoutASoftFp8 : kTableGemmLayoutA, A, wt == kE4M3 ? scale_matrix : nullptr, B,
                                C, m, n, k, dtype, alpha, bias, wt == kE4M3 ? fp8_order : 0, (cudaStream_t)s, aux);
}

int mlk_gemm_layoutAB_ContinuousC_wapper(const void* A, const void* B, void* C, int m, int n, int k, int dtype,
                                         float alpha, float, int p1, int p2, int p3, int kernelId, const void* bias,
                                         const mlk_aux* aux, mlk_stream_t s) {
    if (dtype == MLK_E4M3) { clear_error(); return fail(kInvalidArg, "gemm_layoutAB_ContinuousC: 16-bit weights only"); }
    return gemm_common(1, 0, A, nullptr, B, C, m, n, k, dtype, alpha, p1, p2, p3, kernelId, bias, 0, (cudaStream_t)s, aux);
}
int mlk_gemm_layoutAB_ContinuousC(const void* A, const void* B, void* C, int m, int n, int k, int dtype, float alpha,
                                  float, const void* bias, const mlk_aux* aux, mlk_stream_t s) {
    if (dtype == MLK_E4M3) { clear_error(); return fail(kInvalidArg, "gemm_layoutAB_ContinuousC: 16-bit weights only"); }
    return gemm_table(kTableGemmContinuousC, 1, 0, A, nullptr, B, C, m, n, k, dtype, alpha, bias, 0, (cudaStream_t)s, aux);
}
int mlk_gemm_layoutABC_wapper(const void* A, const void* B, void* C, int m, int n, int k, int dtype, float alpha,
                              float, int p1, int p2, int p3, int kernelId, const void* bias, const mlk_aux* aux,
                              mlk_stream_t s) {
    if (dtype == MLK_E4M3) { clear_error(); return fail(kInvalidArg, "gemm_layoutABC: 16-bit weights only"); }
    return gemm_common(1, 1, A, nullptr, B, C, m, n, k, dtype, alpha, p1, p2, p3, kernelId, bias, 0, (cudaStream_t)s, aux);
}
int mlk_gemm_layoutABC(const void* A, const void* B, void* C, int m, int n, int k, int dtype, float alpha, float,
                       const void* bias, const mlk_aux* aux, mlk_stream_t s) {
    if (dtype == MLK_E4M3) { clear_error(); return fail(kInvalidArg, "gemm_layoutABC: 16-bit weights only"); }
    return gemm_table(kTableGemmABC, 1, 1, A, nullptr, B, C, m, n, k, dtype, alpha, bias, 0, (cudaStream_t)s, aux);
}

int mlk_fused_routing_gate(const void* gating_output, int score_fun, int batch_size, int num_experts, int n_groups,
                           int topK_groups, int32_t* experts_ids, void* selected_experts_weights, int topK,
                           const void* load_balance_bias, int dtype, mlk_stream_t s) {
    clear_error();
    return launch_router(gating_output, score_fun, batch_size, num_experts, n_groups, topK_groups, experts_ids,
                         selected_experts_weights, topK, load_balance_bias, dtype, (cudaStream_t)s);
}

int mlk_fused_routing_gate_renorm(const void* gating_output, int score_fun, int batch_size, int num_experts,
                                  int n_groups, int topK_groups, int32_t* experts_ids, void* selected_experts_weights,
                                  int topK, const void* load_balance_bias, int dtype, int renormalize, mlk_stream_t s) {
    clear_error();
    return launch_router(gating_output, score_fun, batch_size, num_experts, n_groups, topK_groups, experts_ids,
                         selected_experts_weights, topK, load_balance_bias, dtype, (cudaStream_t)s, renormalize);
}

int mlk_fused_router_gemm_gate(const void* x, const void* gate_weight, int score_fun, int batch_size, int hidden_size,
                               int num_experts, int n_groups, int topK_groups, int32_t* experts_ids,
                               void* selected_experts_weights, int topK, const void* load_balance_bias, int dtype,
                               int renormalize, void* logits_out, mlk_stream_t s) {
    clear_error();
    return launch_router_gemm(x, gate_weight, score_fun, batch_size, hidden_size, num_experts, n_groups, topK_groups,
                              experts_ids, selected_experts_weights, topK, load_balance_bias, dtype, renormalize,
                              logits_out, (cudaStream_t)s);
}

int mlk_moe_align(int batchSize, int expertCount, int topK, int microBatchSize, const int32_t* topk_ids,
                  int32_t* sorted_token_ids, int32_t* cumsum_buffer, int32_t* padded_num_experts,
                  int32_t* experts_ids_out, const int32_t* experts_map, int experts_map_len, mlk_stream_t s) {
    clear_error();
    return launch_moe_align(batchSize, expertCount, topK, microBatchSize, topk_ids, sorted_token_ids, cumsum_buffer,
                            padded_num_experts, experts_ids_out, experts_map, experts_map_len, (cudaStream_t)s);
}

int mlk_moe_gather_rows(const void* x, const int32_t* idx, void* out, int64_t n_rows, int hidden, int64_t x_rows,
                        mlk_stream_t s) {
    clear_error();
    return launch_gather_rows(x, idx, out, n_rows, hidden, x_rows, (cudaStream_t)s);
}

int mlk_moe_unpermute_sum(const void* rows, const int32_t* pos, void* y, int64_t T, int topK, int hidden,
                          int64_t n_rows, int dtype, mlk_stream_t s) {
    clear_error();
    return launch_unpermute_sum(rows, pos, y, T, topK, hidden, n_rows, dtype, (cudaStream_t)s);
}

int64_t mlk_ep_reduce_flag_bytes(void) { return ep_reduce_flag_bytes(); }
int64_t mlk_ep_reduce_recv_bytes(int world, int64_t T, int hidden) { return ep_reduce_recv_bytes(world, T, hidden); }

int mlk_ep_reduce_shares(const void* const* shares_dev, void* const* outs_dev, void* const* flags_dev, void* const* recv_dev,
                         int rank, int world, int64_t T, int hidden, int dtype, int32_t* status, mlk_stream_t s) {
    clear_error();
    return launch_ep_reduce(shares_dev, outs_dev, flags_dev, recv_dev, rank, world, T, hidden, dtype, status, (cudaStream_t)s);
}

namespace {
MoeParams moe_params(const void* w1, const void* w2, const void* x, int batch_size, int expert_count, int topK, int hidden,
                     int inter, const int32_t* topk_ids, const void* topk_weights, int32_t* sorted_token_ids,
                     int32_t* cumsum_buffer, int32_t* padded_num_experts, int32_t* experts_ids, void* C, void* y,
                     const float* w1_scale, const float* w2_scale, int dtype, int fp8_order, int microBatchSize,
                     const int32_t* experts_map, int experts_map_len, const int32_t* tune, int32_t* status, int out_fp32) {
    MoeParams p{};
    p.w1 = w1; p.w2 = w2; p.x = x; p.T = batch_size; p.E = expert_count; p.topk = topK; p.H = hidden; p.I = inter;
    p.topk_ids = topk_ids; p.topk_weights = topk_weights; p.sorted_token_ids = sorted_token_ids;
    p.cumsum = cumsum_buffer; p.padded_num_experts = padded_num_experts; p.experts_ids = experts_ids;
    p.C = C; p.y = y; p.w1_scale = w1_scale; p.w2_scale = w2_scale; p.dtype = dtype; p.fp8_order = fp8_order;
    p.mbs = microBatchSize; p.experts_map = experts_map; p.experts_map_len = experts_map_len;
    p.status = status;
    p.y_fp32 = out_fp32;
    if (tune) { p.nt = tune[0]; p.wm1 = tune[1]; p.sk1 = tune[2]; p.rg = tune[3]; p.wm2 = tune[4]; p.sk2 = tune[5]; }
    return p;
}
}  // namespace

int mlk_fused_experts_compute(const void* w1, const void* w2, const void* x, int batch_size, int expert_count,
                              int topK, int hidden, int inter, const int32_t* topk_ids, const void* topk_weights,
                              int32_t* sorted_token_ids, int32_t* cumsum_buffer, int32_t* padded_num_experts,
                              int32_t* experts_ids, void* C, void* y, const float* w1_scale, const float* w2_scale,
                              int dtype, int fp8_order, int microBatchSize, const int32_t* experts_map,
                              int experts_map_len, float* combine_scratch, int64_t combine_scratch_bytes,
                              const int32_t* tune, int32_t* status, int out_fp32, mlk_stream_t s) {
    clear_error();
    MoeParams p = moe_params(w1, w2, x, batch_size, expert_count, topK, hidden, inter, topk_ids, topk_weights,
                             sorted_token_ids, cumsum_buffer, padded_num_experts, experts_ids, C, y, w1_scale, w2_scale,
                             dtype, fp8_order, microBatchSize, experts_map, experts_map_len, tune, status, out_fp32);
    p.scratch = combine_scratch; p.scratch_bytes = combine_scratch_bytes;
    return launch_fused_experts(p, (cudaStream_t)s);
}

int mlk_fused_routing_experts_compute(const void* gating_output, int num_experts, int score_fun, int n_groups,
                                      int topK_groups, const void* gating_bias, int renormalize, const void* w1,
                                      const void* w2, const void* x, int batch_size, int expert_count, int topK,
                                      int hidden, int inter, int32_t* topk_ids, void* topk_weights,
                                      int32_t* sorted_token_ids, int32_t* cumsum_buffer, int32_t* padded_num_experts,
                                      int32_t* experts_ids, void* C, void* y, const float* w1_scale,
                                      const float* w2_scale, int dtype, int fp8_order, int microBatchSize,
                                      const int32_t* experts_map, int experts_map_len, float* combine_scratch,
                                      int64_t combine_scratch_bytes, const int32_t* tune, int32_t* status, int out_fp32,
                                      mlk_stream_t s) {
    clear_error();
    if (!gating_output) return fail(kInvalidArg, "fused_routing_experts_compute: gating_output is null");
    MoeParams p = moe_params(w1, w2, x, batch_size, expert_count, topK, hidden, inter, topk_ids, topk_weights,
                             sorted_token_ids, cumsum_buffer, padded_num_experts, experts_ids, C, y, w1_scale, w2_scale,
                             dtype, fp8_order, microBatchSize, experts_map, experts_map_len, tune, status, out_fp32);
    p.scratch = combine_scratch; p.scratch_bytes = combine_scratch_bytes;
    p.gating = gating_output; p.gating_bias = gating_bias; p.n_global = num_experts; p.score_fun = score_fun;
    p.n_groups = n_groups; p.topk_groups = topK_groups; p.renormalize = renormalize;
    return launch_fused_experts(p, (cudaStream_t)s);
}

int mlk_fused_experts_compute_static(const void* w1, const void* w2, const void* x, int batch_size, int expert_count,
                                     int topK, int hidden, int inter, const int32_t* topk_ids, const void* topk_weights,
                                     int32_t* sorted_token_ids, int32_t* cumsum_buffer, int32_t* padded_num_experts,
                                     int32_t* experts_ids, void* C, void* y, const float* w1_scale,
                                     const float* w2_scale, int dtype, int fp8_order, int microBatchSize,
                                     const int32_t* experts_map, int experts_map_len, const int32_t* tune,
                                     int32_t* status, int out_fp32, mlk_stream_t s) {
    clear_error();
    const MoeParams p = moe_params(w1, w2, x, batch_size, expert_count, topK, hidden, inter, topk_ids, topk_weights,
                                   sorted_token_ids, cumsum_buffer, padded_num_experts, experts_ids, C, y, w1_scale,
                                   w2_scale, dtype, fp8_order, microBatchSize, experts_map, experts_map_len, tune, status,
                                   out_fp32);
    return launch_fused_experts_static(p, (cudaStream_t)s);
}

}  // extern "C"
