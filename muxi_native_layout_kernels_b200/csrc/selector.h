// Dispatch-table class; see selector.cpp.
#pragma once

#include <cstddef>
#include <map>
#include <mutex>
#include <string>
#include <tuple>

namespace mlk {

enum Table : int {
    kTableGemmABC = 0,
    kTableGemmContinuousC = 1,
    kTableGemmLayoutA = 2,
    kTableGemmLayoutASoftFp8 = 3,
    kTableGemvFp16 = 4,
    kTableGemvBf16 = 5,
    kTableGemvSoftFp8 = 6,
    kNumTables = 7,
};

// GEMM tables: a=kernelId b=kernelParam1 c=kernelParam2 d=kernelParam3
// GeMV tables: a=BLOCK_DIM_X b=KernelId c=KernelParam1 d=KernelParam2
struct TuneArgs {
    int a, b, c, d;
};

const char* table_file_name(int table);
TuneArgs default_args(int table, int m, int n, int k);
TuneArgs warp_level_default_args(int table, int m, int n, int k);   // GEMM tables: kernelId 1 arguments

class DispatchTable {
  public:
    explicit DispatchTable(int table);
    int load(const std::string& path);               // 0 ok, 1 file could not be opened
    TuneArgs get(int m, int n, int k, bool* hit);    // n ignored for GeMV tables
    bool loaded() const { return loaded_; }
    size_t size();

  private:
    using Key = std::tuple<int, int, int>;
    int table_;
    bool loaded_ = false;
    std::string path_;
    std::map<Key, TuneArgs> map_;
    std::mutex mu_;
};

DispatchTable& global_table(int table);

}  // namespace mlk
