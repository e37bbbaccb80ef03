// Host-side truth of the paged KV cache: page allocator with reference counts (shared prefix
// pages), per-seat page table with dirty-row tracking, resident slot pool, and the
// content-addressed prefix index used for context reuse.
//
// Counterparts in the reference: cpp/runtime/state/kvPageTable.{h,cpp} (host-truth table, -1 =
// unused, dirty-row upload), cpp/runtime/kvCacheManager.{h,cpp}, cpp/runtime/state/residentSlotPool.*
// and cpp/runtime/state/contextCache/{blockHash,blockIndex,evictionPlanner}.* .  The device pool
// itself is a torch tensor owned by the Python side; this code never touches device memory.
#pragma once

#include <cstdint>
#include <list>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace telb {

constexpr int32_t kUnusedPage = -1;

class PageAllocator {
  public:
    explicit PageAllocator(int num_pages);
    int num_pages() const { return static_cast<int>(ref_.size()); }
    int free_pages() const { return static_cast<int>(free_.size()); }
    std::vector<int32_t> alloc(int n);            // throws std::bad_alloc-like runtime_error when exhausted
    void retain(const std::vector<int32_t>& pages);
    void release(const std::vector<int32_t>& pages);
    int refcount(int32_t page) const { return ref_.at(page); }

  private:
    std::vector<int32_t> free_;
    std::vector<int32_t> ref_;
};

// [seats, max_pages] table; a row is the logical → physical page map of one resident sequence.
class KVPageTable {
  public:
    KVPageTable(int num_pages, int page_size, int max_seats, int max_pages_per_seq);

    int page_size() const { return page_size_; }
    int max_seats() const { return max_seats_; }
    int max_pages_per_seq() const { return max_pages_; }
    int free_pages() const { return alloc_.free_pages(); }
    int length(int seat) const { return lengths_.at(seat); }
    int capacity_tokens(int seat) const { return static_cast<int>(pages_.at(seat).size()) * page_size_; }
    const std::vector<int32_t>& pages(int seat) const { return pages_.at(seat); }

    void reserve(int seat, int total_tokens);          // grow to hold total_tokens
    bool can_reserve(int seat, int total_tokens) const;
    void adopt_prefix(int seat, const std::vector<int32_t>& pages, int tokens);   // share filled pages
    void commit(int seat, int new_tokens) { lengths_.at(seat) += new_tokens; }
    void rewind(int seat, int length);                 // speculative rejection: drop the tail, keep pages
    void free_seat(int seat);
    // Bounded sliding-window storage: give back every page that lies wholly before `first_live_token`.  The
    // logical positions stay (their table entries become kUnusedPage), so later pages keep their indices.
    // Returns the number of pages released.
    int retire_before(int seat, int first_live_token);
    int live_pages(int seat) const;

    const int32_t* row(int seat) const { return table_.data() + static_cast<size_t>(seat) * max_pages_; }
    const std::vector<int32_t>& table() const { return table_; }
    // Rows changed since the last call (to be re-uploaded to the device copy).
    std::vector<int> take_dirty_rows();
    PageAllocator& allocator() { return alloc_; }

  private:
    PageAllocator alloc_;
    int page_size_, max_seats_, max_pages_;
    std::vector<int32_t> table_;
    std::vector<int> lengths_;
    std::vector<std::vector<int32_t>> pages_;
    std::vector<uint8_t> dirty_;
};

// Seats (rows of the resident state pools).  Each hand-out bumps the seat's epoch so stale
// references from an earlier occupant can be recognised.
class ResidentSlotPool {
  public:
    explicit ResidentSlotPool(int n);
    int acquire();                       // -1 when full
    void release(int slot);
    uint32_t epoch(int slot) const { return epoch_.at(slot); }
    int in_use() const { return in_use_; }
    int capacity() const { return static_cast<int>(epoch_.size()); }

  private:
    std::vector<int> free_;
    std::vector<uint32_t> epoch_;
    std::vector<uint8_t> used_;
    int in_use_ = 0;
};

// Content-addressed index of full KV pages: hash(parent hash, page tokens) → physical page.
// A page is inserted when a sequence has filled it; a later prompt that starts with the same
// tokens adopts the pages instead of recomputing them.  Entries hold one reference on their
// page; least-recently-used entries are evicted when the pool runs short.
class PrefixCache {
  public:
    PrefixCache(PageAllocator& alloc, int page_size, int max_records);
    static uint64_t hash_block(uint64_t parent, const int32_t* tokens, int n);
    // A second, independent hash of the same block (different mixing function and constants).  It is stored with the
    // entry and compared on every hit, so two prompts must collide in 128 bits before they could share a page.
    static uint64_t check_block(uint64_t parent_check, const int32_t* tokens, int n);
    // Seed of a hash chain for everything besides token ids that decides what the KV of a prompt holds: the LoRA
    // adapter a request runs under (name + load generation) and an optional isolation key.  Requests with different
    // seeds never see each other's pages.
    static uint64_t extras_seed(const std::string& adapter, uint64_t adapter_generation, const std::string& isolation_key);

    struct Match {
        std::vector<int32_t> pages;
        int tokens = 0;
    };
    // Longest cached prefix of `tokens` in whole pages (never the whole prompt: at least one token
    // is left to compute so the step produces logits).
    // `seed` starts the hash chain (0 = base model, no isolation; see extras_seed).
    Match lookup(const std::vector<int32_t>& tokens, uint64_t seed = 0);
    // Register the first `filled_tokens` (whole pages only) of a sequence whose pages are `pages`.
    int insert(const std::vector<int32_t>& tokens, int filled_tokens, const std::vector<int32_t>& pages, uint64_t seed = 0);
    // Eviction is planned before it is carried out.  A plan is the shortest run of least-recently-used records whose pages
    // would actually return to the pool (the cache holds their last reference); records whose pages a resident sequence still
    // shares are passed over.  Chains are touched leaves-first, so a prefix's later pages go before the pages every
    // continuation depends on.
    struct EvictionPlan {
        int pages_wanted = 0;
        int reclaimable_pages = 0;
        int pinned_skipped = 0;           // records passed over because their page is shared with a resident sequence
        bool satisfied = false;
        std::vector<uint64_t> victims;    // block hashes, least recently used first
    };
    EvictionPlan plan_eviction(int pages_wanted) const;
    int evict(const EvictionPlan& plan);  // returns pages freed
    int evict(int pages_wanted);          // plan + evict; returns pages freed (0: nothing reclaimable)
    int drop_records(int n);              // forget the n oldest records whatever their pages' state (record-count limit)
    int records() const { return static_cast<int>(map_.size()); }
    uint64_t hits() const { return hits_; }
    uint64_t misses() const { return misses_; }
    uint64_t check_mismatches() const { return mismatches_; }

  private:
    struct Entry {
        int32_t page;
        uint64_t check;
        std::list<uint64_t>::iterator lru;
    };
    void touch_chain(const std::vector<std::list<uint64_t>::iterator>& chain);
    PageAllocator& alloc_;
    int page_size_, max_records_;
    std::unordered_map<uint64_t, Entry> map_;
    std::list<uint64_t> lru_;             // front = most recent
    uint64_t hits_ = 0, misses_ = 0, mismatches_ = 0;
};

}  // namespace telb
