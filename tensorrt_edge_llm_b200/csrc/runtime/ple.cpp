#include "ple.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <fstream>
#include <stdexcept>

namespace telb {

static const char kMagic[8] = {'T', 'E', 'L', 'B', 'P', 'L', 'E', '1'};

void PleTable::write(const std::string& path, const void* data, uint32_t rows, uint32_t row_bytes, uint32_t layers, uint32_t dtype) {
    std::ofstream f(path, std::ios::binary | std::ios::trunc);
    if (!f) throw std::runtime_error("cannot create " + path);
    f.write(kMagic, 8);
    const uint32_t hdr[4] = {rows, row_bytes, layers, dtype};
    f.write(reinterpret_cast<const char*>(hdr), sizeof(hdr));
    f.write(static_cast<const char*>(data), static_cast<std::streamsize>(rows) * row_bytes);
    if (!f) throw std::runtime_error("short write to " + path);
}

PleTable::PleTable(const std::string& path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) throw std::runtime_error("cannot open " + path);
    struct stat st {};
    if (::fstat(fd_, &st) != 0 || static_cast<size_t>(st.st_size) < kHeader) {
        ::close(fd_);
        throw std::runtime_error("not a PLE table: " + path);
    }
    size_ = static_cast<size_t>(st.st_size);
    void* p = ::mmap(nullptr, size_, PROT_READ, MAP_SHARED, fd_, 0);
    if (p == MAP_FAILED) {
        ::close(fd_);
        throw std::runtime_error("mmap failed for " + path);
    }
    base_ = static_cast<uint8_t*>(p);
    uint32_t hdr[4];
    std::memcpy(hdr, base_ + 8, sizeof(hdr));
    rows_ = hdr[0];
    row_bytes_ = hdr[1];
    layers_ = hdr[2];
    dtype_ = hdr[3];
    if (std::memcmp(base_, kMagic, 8) != 0 || kHeader + static_cast<size_t>(rows_) * row_bytes_ > size_) {
        ::munmap(base_, size_);
        ::close(fd_);
        throw std::runtime_error("corrupt PLE table: " + path);
    }
    ::madvise(base_, size_, MADV_RANDOM);
}

PleTable::~PleTable() {
    if (base_) ::munmap(base_, size_);
    if (fd_ >= 0) ::close(fd_);
}

PleCache::PleCache(int slots) : row_of_(slots, -1), where_(slots), stamp_(slots, 0) {
    if (slots <= 0) throw std::runtime_error("the PLE cache needs at least one slot");
    for (int s = 0; s < slots; ++s) {
        lru_.push_back(s);
        where_[s] = std::prev(lru_.end());
    }
}

int PleCache::lookup(uint32_t row) const {
    auto it = slot_of_.find(row);
    return it == slot_of_.end() ? -1 : it->second;
}

PleReadPlan PleCache::plan(const std::vector<int32_t>& ids, uint32_t row_bytes, PleIoBudget* budget) {
    ++step_;
    if (budget) budget->begin_step();
    PleReadPlan p;
    p.slots.assign(ids.size(), -1);
    std::unordered_map<uint32_t, int> this_step;           // row → slot decided in this plan (or -1 when deferred)
    auto touch = [&](int s) {
        lru_.erase(where_[s]);
        lru_.push_front(s);
        where_[s] = lru_.begin();
        stamp_[s] = step_;
    };
    for (size_t i = 0; i < ids.size(); ++i) {
        if (ids[i] < 0) throw std::runtime_error("negative token id");
        const uint32_t row = static_cast<uint32_t>(ids[i]);
        auto seen = this_step.find(row);
        if (seen != this_step.end()) {
            p.slots[i] = seen->second;
            continue;
        }
        int s = lookup(row);
        if (s >= 0) {
            ++p.hits;
            ++hits_;
            touch(s);
        } else {
            ++misses_;
            // the least recently used slot that this step does not use
            int victim = -1;
            for (auto it = lru_.rbegin(); it != lru_.rend(); ++it)
                if (stamp_[*it] != step_) {
                    victim = *it;
                    break;
                }
            if (victim < 0 || (budget && !budget->take(row_bytes))) {
                ++p.deferred;                                   // cache too small for one step, or out of IO budget
                this_step[row] = -1;
                continue;
            }
            if (row_of_[victim] >= 0) slot_of_.erase(static_cast<uint32_t>(row_of_[victim]));
            row_of_[victim] = row;
            slot_of_[row] = victim;
            touch(victim);
            s = victim;
            ++p.misses;
            p.miss_rows.push_back(row);
            p.miss_slots.push_back(s);
        }
        this_step[row] = s;
        p.slots[i] = s;
    }
    // coalesce: sort the misses by table row (keeping slot pairing), then merge neighbours into runs
    std::vector<size_t> order(p.miss_rows.size());
    for (size_t i = 0; i < order.size(); ++i) order[i] = i;
    std::sort(order.begin(), order.end(), [&](size_t a, size_t b) { return p.miss_rows[a] < p.miss_rows[b]; });
    std::vector<uint32_t> rows(order.size());
    std::vector<int32_t> slots(order.size());
    for (size_t i = 0; i < order.size(); ++i) {
        rows[i] = p.miss_rows[order[i]];
        slots[i] = p.miss_slots[order[i]];
    }
    p.miss_rows.swap(rows);
    p.miss_slots.swap(slots);
    for (size_t i = 0; i < p.miss_rows.size(); ++i) {
        if (!p.runs.empty() && p.runs.back().first_row + p.runs.back().count == p.miss_rows[i]) ++p.runs.back().count;
        else p.runs.push_back(PleRun{p.miss_rows[i], 1, static_cast<uint32_t>(i)});
    }
    p.bytes = static_cast<uint64_t>(p.miss_rows.size()) * row_bytes;
    return p;
}

PleReadExecutor::PleReadExecutor(int threads) {
    for (int i = 0; i < std::max(threads, 1); ++i) threads_.emplace_back([this] { worker(); });
}

PleReadExecutor::~PleReadExecutor() {
    {
        std::lock_guard<std::mutex> lk(mu_);
        stop_ = true;
    }
    cv_.notify_all();
    for (auto& t : threads_) t.join();
}

void PleReadExecutor::worker() {
    for (;;) {
        std::function<void()> job;
        {
            std::unique_lock<std::mutex> lk(mu_);
            cv_.wait(lk, [&] { return stop_ || !jobs_.empty(); });
            if (stop_ && jobs_.empty()) return;
            job = std::move(jobs_.back());
            jobs_.pop_back();
        }
        job();
        {
            std::lock_guard<std::mutex> lk(mu_);
            --pending_;
        }
        done_cv_.notify_all();
    }
}

void PleReadExecutor::read(const PleTable& table, const PleReadPlan& plan, uint8_t* staging) {
    const size_t rb = table.row_bytes();
    {
        std::lock_guard<std::mutex> lk(mu_);
        for (const PleRun& r : plan.runs) {
            if (r.first_row + r.count > table.rows()) throw std::runtime_error("PLE read beyond the table");
            jobs_.push_back([&table, r, staging, rb] { std::memcpy(staging + r.staging_row * rb, table.row(r.first_row), r.count * rb); });
            ++pending_;
        }
    }
    cv_.notify_all();
    std::unique_lock<std::mutex> lk(mu_);
    done_cv_.wait(lk, [&] { return pending_ == 0; });
}

}  // namespace telb
