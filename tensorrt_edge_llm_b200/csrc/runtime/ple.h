// Per-layer-embedding (PLE) store: a large [vocab, row_bytes] table that lives in a file (memory-mapped) while a
// small row cache lives on the GPU.  Each step asks for the rows of its token ids; the planner splits them into
// cache hits and misses, coalesces the misses into contiguous file runs, the IO budget caps how many bytes a step
// may read, and a small thread pool copies the runs into a (pinned) staging buffer the caller uploads.
//
// Counterparts in the reference: cpp/runtime/embedding/{pleTable,pleRowStore,pleCache,pleReadExecutor,pleReadPlan,
// pleIoBudget,pleFileUtils}.cpp.  The device side (cache tensor, scatter of new rows, gather of a step's rows) is
// done by the caller with the framework's embedding-gather and index-copy kernels.
#pragma once

#include <condition_variable>
#include <cstdint>
#include <functional>
#include <list>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace telb {

// File: magic "TELBPLE1", u32 rows, u32 row_bytes, u32 layers, u32 dtype code, then rows * row_bytes bytes.
class PleTable {
  public:
    static void write(const std::string& path, const void* data, uint32_t rows, uint32_t row_bytes, uint32_t layers, uint32_t dtype);
    explicit PleTable(const std::string& path);
    ~PleTable();
    PleTable(const PleTable&) = delete;
    uint32_t rows() const { return rows_; }
    uint32_t row_bytes() const { return row_bytes_; }
    uint32_t layers() const { return layers_; }
    uint32_t dtype() const { return dtype_; }
    const uint8_t* row(uint32_t r) const { return base_ + kHeader + static_cast<size_t>(r) * row_bytes_; }

  private:
    static constexpr size_t kHeader = 24;
    int fd_ = -1;
    uint8_t* base_ = nullptr;
    size_t size_ = 0;
    uint32_t rows_ = 0, row_bytes_ = 0, layers_ = 0, dtype_ = 0;
};

struct PleRun {
    uint32_t first_row = 0, count = 0;     // rows [first_row, first_row + count) of the table ...
    uint32_t staging_row = 0;              // ... land at this row of the staging buffer
};

struct PleReadPlan {
    std::vector<int32_t> slots;            // per requested token: cache slot holding its row (-1 = deferred by the budget)
    std::vector<uint32_t> miss_rows;       // table rows to read, in staging order
    std::vector<int32_t> miss_slots;       // cache slot each staged row is scattered to
    std::vector<PleRun> runs;              // the same misses as contiguous file runs
    uint32_t hits = 0, misses = 0, deferred = 0;
    uint64_t bytes = 0;
};

// Bytes a step may read; unused allowance carries over up to `burst` steps' worth.
class PleIoBudget {
  public:
    PleIoBudget(uint64_t bytes_per_step, int burst_steps = 2) : per_step_(bytes_per_step), cap_(bytes_per_step * burst_steps), avail_(bytes_per_step) {}
    void begin_step() { avail_ = std::min(cap_, avail_ + per_step_); }
    bool take(uint64_t bytes) {
        if (per_step_ == 0) return true;       // 0 = unlimited
        if (bytes > avail_) return false;
        avail_ -= bytes;
        return true;
    }
    uint64_t available() const { return per_step_ == 0 ? ~0ull : avail_; }

  private:
    uint64_t per_step_, cap_, avail_;
};

// Host-side bookkeeping of the device row cache: table row → slot, least-recently-used eviction that never evicts
// a row the current step uses.
class PleCache {
  public:
    explicit PleCache(int slots);
    int slots() const { return static_cast<int>(row_of_.size()); }
    uint64_t hits() const { return hits_; }
    uint64_t misses() const { return misses_; }
    // Builds the plan for `ids` (duplicates share a slot).  Rows beyond the budget are deferred (slot -1).
    PleReadPlan plan(const std::vector<int32_t>& ids, uint32_t row_bytes, PleIoBudget* budget);
    int lookup(uint32_t row) const;

  private:
    std::vector<int64_t> row_of_;                          // slot → table row (-1 = empty)
    std::unordered_map<uint32_t, int> slot_of_;
    std::list<int> lru_;                                   // front = most recent
    std::vector<std::list<int>::iterator> where_;
    std::vector<uint64_t> stamp_;                          // step that last used the slot
    uint64_t step_ = 0, hits_ = 0, misses_ = 0;
};

// Copies the plan's runs from the table into `staging` (row-major, row_bytes per row) on worker threads.
class PleReadExecutor {
  public:
    explicit PleReadExecutor(int threads = 2);
    ~PleReadExecutor();
    void read(const PleTable& table, const PleReadPlan& plan, uint8_t* staging);       // returns when every run is copied

  private:
    void worker();
    std::vector<std::thread> threads_;
    std::mutex mu_;
    std::condition_variable cv_, done_cv_;
    std::vector<std::function<void()>> jobs_;
    int pending_ = 0;
    bool stop_ = false;
};

}  // namespace telb
