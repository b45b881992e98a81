// Dispatch tables: exact-key lookup (m,n,k) or (m,k) -> four tuning integers, read once from CSV.
//
// The reference has seven copies of the same class (csrc/arg_selector.h:9-125, arg_selector.cu:14-538),
// one per table; here it is one class and seven instances.  Behaviour kept from the reference:
//   * first line of the file is a header and is skipped;
//   * a data line must hold exactly 7 (GEMM) or 6 (GeMV) comma-separated integers, else it is
//     reported on stderr and skipped;
//   * a later duplicate key overwrites an earlier one;
//   * a miss prints one warning, inserts a default for that key (so the warning appears once) and
//     returns the default; a missing file only warns.
// Difference: the default is not the constant (1,1,1,1) / (256,1,1,1) tuned for another GPU but a
// shape-based choice that keeps all SMs of the current device (148 on a B200) busy.
#include "selector.h"

#include "status.h"

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <sstream>
#include <vector>

namespace mlk {

namespace {

const char* const kTableFile[kNumTables] = {
    "layout_gemm_dispatch_arg.csv",            // gemm_layoutABC            (arg_selector.cu:80)
    "continuous_gemm_dispatch_arg.csv",        // gemm_layoutAB_ContinuousC (arg_selector.cu:157)
    "layoutA_gemm_dispatch_arg.csv",           // gemm_layoutA              (arg_selector.cu:303)
    "layoutA_Soft_Fp8_gemm_dispatch_arg.csv",  // gemm_layoutA_soft_fp8     (arg_selector.cu:375)
    "layout_gemv_dispatch_arg.csv",            // gemv_layoutA, fp16        (arg_selector.cu:232)
    "layout_gemv_bf16_dispatch_arg.csv",       // gemv_layoutA, bf16        (arg_selector.cu:531)
    "layout_gemv_soft_fp8_dispatch_arg.csv",   // gemv_layoutA, e4m3        (arg_selector.cu:454)
};

bool is_gemv(int table) { return table >= kTableGemvFp16; }

}  // namespace

const char* table_file_name(int table) {
    return (table >= 0 && table < kNumTables) ? kTableFile[table] : nullptr;
}

// Shape-based default used when a key is not in the table.
//   GEMM tables: {kernelId, APerWarp, rowWarps, splitK}
//   GeMV tables: {BLOCK_DIM_X, KernelId, APerWarp, splitK}
TuneArgs default_args(int table, int m, int n, int k) {
    // Target: at least ~2 CTAs of 8 warps per SM so that enough 16-byte loads are in flight.
    const int target_ctas = 2 * sm_count();
    if (table == kTableGemvSoftFp8 && m % 128 == 0 && k % 128 == 0) {
        // the same kernel for one token (KernelId 4): BLOCK_DIM_X = k per stage, KernelParam1 = ring stages,
        // KernelParam2 = CTAs per cluster; the entry point falls back to KernelId 1 when it cannot run
        const TuneArgs g = default_args(kTableGemmLayoutASoftFp8, m, 1, k);
        return TuneArgs{g.b, 4, g.c, g.d};
    }
    if (is_gemv(table)) {
        int rg = 1;
        int ctas = m / 16;
        int sk = 1;
        while (sk < 8 && ctas * sk < target_ctas && (k / 32) / (8 * sk * 2) >= 4) sk *= 2;
        return TuneArgs{256, 1, rg, sk};
    }
    if (table == kTableGemmLayoutA && m % 128 == 0 && k % 64 == 0 && n > 64) {
        // more tokens than the narrow tcgen05 tile holds: the many-token tile kernel (kernelId 10), tile and ring chosen
        // by the launcher
        return TuneArgs{10, 0, 0, 0};
    }
    if (table == kTableGemmLayoutASoftFp8 && m % 128 == 0 && k % 128 == 0 && n >= 1 && n <= 64) {
        // e4m3 weights straight into the 8-bit tensor-core MMA (kernelId 9; the entry point falls back to the decode
        // pipeline, kernelId 2 with the same kernelParam2 / 3, for calls with block scales or without scratch):
        // kernelParam1 = k per stage, kernelParam2 = ring stages, kernelParam3 = CTAs per cluster, chosen so that all
        // CTAs are resident at once (one wave) and fill most of it
        const int tiles = m / 128;
        const int np = n <= 16 ? 16 : (n <= 32 ? 32 : 64);
        const int bk = (np == 16 && tiles >= 150) ? 64 : 128;
        const int stages = 3;
        const int smem = stages * (128 * bk + (bk / 64) * np * 128) + 2048;
        int resident = (200 * 1024) / smem;
        if (resident > 5) resident = 5;
        if (resident < 1) resident = 1;
        int ck = (sm_count() * resident) / tiles;
        if (ck > 8) ck = 8;
        while (ck > 1 && (k / bk) / ck < 2) --ck;
        if (ck < 1) ck = 1;
        return TuneArgs{9, bk, stages, ck};
    }
    if (m % 128 == 0 && k % 64 == 0 && n >= 2 && n <= 64) {
        // tcgen05 tile kernel, one cluster per 128-row tile: enough CTAs for three to four per SM (they are small, and
        // the start and tail of one overlap the streaming of the others), every CTA with at least four k blocks;
        // kernelParam2 = ring stages, kernelParam3 = CTAs per cluster (the 16-bit kernel wants 2 or more)
        const int tiles = m / 128, kblocks = k / 64;
        int ck = (512 + tiles - 1) / tiles;
        if (ck > 8) ck = 8;
        while (ck > 1 && kblocks / ck < 4) --ck;
        if (table != kTableGemmLayoutASoftFp8 && ck < 2) ck = kblocks >= 2 ? 2 : 0;
        // ring depth: 16-bit 4 (3 for the 64-token tile, whose stages are 24 KB); e4m3 stages are 8 KB, 6 for the
        // 16-token tile, 4 above
        const int stages = table == kTableGemmLayoutASoftFp8 ? (n <= 16 ? 6 : 4) : (n > 32 ? 3 : 4);
        return TuneArgs{2, 1, stages, ck};
    }
    return warp_level_default_args(table, m, n, k);
}

// Launch arguments of the warp-level streaming kernel (kernelId 1) for any shape it accepts.
TuneArgs warp_level_default_args(int table, int m, int n, int k) {
    const int target_ctas = 2 * sm_count();
    (void)table;
    int rg = (n > 8 && m % 32 == 0) ? 2 : 1;
    int wm = 1;
    if (n > 32) wm = 4;
    else if (n > 16) wm = 2;
    else if (n > 8) wm = 2;
    while (wm > 1 && m % (16 * rg * wm) != 0) wm >>= 1;
    if (m % (16 * rg * wm) != 0) rg = 1;
    int ctas = m / (16 * rg * wm);
    int wk = 8 / wm;
    int sk = 1;
    while (sk < 8 && ctas * sk < target_ctas && (k / 32) / (wk * sk * 2) >= 4) sk *= 2;
    return TuneArgs{1, rg, wm, sk};
}

DispatchTable::DispatchTable(int table) : table_(table) {}

int DispatchTable::load(const std::string& path) {
    std::lock_guard<std::mutex> lock(mu_);
    map_.clear();
    loaded_ = true;
    path_ = path;
    std::ifstream file(path);
    if (!file.is_open()) {
        std::fprintf(stderr, "Error opening file: %s\nAll shapes of this table fall back to default args\n",
                     path.c_str());
        return 1;
    }
    const size_t want = is_gemv(table_) ? 6 : 7;
    std::string line;
    std::getline(file, line);   // header
    while (std::getline(file, line)) {
        if (line.empty() || line == "\r") continue;
        std::istringstream ss(line);
        std::string tok;
        std::vector<int> v;
        bool bad = false;
        while (std::getline(ss, tok, ',')) {
            char* end = nullptr;
            long x = std::strtol(tok.c_str(), &end, 10);
            if (end == tok.c_str()) { bad = true; break; }
            v.push_back((int)x);
        }
        if (bad || v.size() != want) {
            std::fprintf(stderr, "Invalid line: %s\n", line.c_str());
            continue;
        }
        if (is_gemv(table_))
            map_[Key{v[0], 0, v[1]}] = TuneArgs{v[2], v[3], v[4], v[5]};
        else
            map_[Key{v[0], v[1], v[2]}] = TuneArgs{v[3], v[4], v[5], v[6]};
    }
    return 0;
}

TuneArgs DispatchTable::get(int m, int n, int k, bool* hit) {
    std::lock_guard<std::mutex> lock(mu_);
    const Key key{m, is_gemv(table_) ? 0 : n, k};
    auto it = map_.find(key);
    if (it != map_.end()) {
        if (hit) *hit = true;
        return it->second;
    }
    if (hit) *hit = false;
    const TuneArgs d = default_args(table_, m, n, k);
    if (is_gemv(table_))
        std::fprintf(stderr, " Warning: No matching arguments found for %s shape: %d, %d. Fallback args %d,%d,%d,%d\n",
                     kTableFile[table_], m, k, d.a, d.b, d.c, d.d);
    else
        std::fprintf(stderr, " Warning: No matching arguments found for %s shape: %d, %d, %d. Fallback args %d,%d,%d,%d\n",
                     kTableFile[table_], m, n, k, d.a, d.b, d.c, d.d);
    map_[key] = d;   // warn once per key
    return d;
}

size_t DispatchTable::size() {
    std::lock_guard<std::mutex> lock(mu_);
    return map_.size();
}

DispatchTable& global_table(int table) {
    static DispatchTable tables[kNumTables] = {DispatchTable(0), DispatchTable(1), DispatchTable(2), DispatchTable(3),
                                               DispatchTable(4), DispatchTable(5), DispatchTable(6)};
    return tables[table];
}

}  // namespace mlk
