#include "paged_kv.h"

#include <algorithm>

namespace telb {

PageAllocator::PageAllocator(int num_pages) : ref_(num_pages, 0) {
    free_.reserve(num_pages);
    for (int p = num_pages - 1; p >= 0; --p) free_.push_back(p);
}

std::vector<int32_t> PageAllocator::alloc(int n) {
    if (n > static_cast<int>(free_.size()))
        throw std::runtime_error("KV pool exhausted: want " + std::to_string(n) + " pages, " + std::to_string(free_.size()) + " free");
    std::vector<int32_t> out(n);
    for (int i = 0; i < n; ++i) {
        out[i] = free_.back();
        free_.pop_back();
        ref_[out[i]] = 1;
    }
    return out;
}

void PageAllocator::retain(const std::vector<int32_t>& pages) {
    for (int32_t p : pages) {
        if (ref_.at(p) <= 0) throw std::runtime_error("retain of free page " + std::to_string(p));
        ++ref_[p];
    }
}

void PageAllocator::release(const std::vector<int32_t>& pages) {
    for (int32_t p : pages) {
        if (ref_.at(p) <= 0) throw std::runtime_error("double free of page " + std::to_string(p));
        if (--ref_[p] == 0) free_.push_back(p);
    }
}

KVPageTable::KVPageTable(int num_pages, int page_size, int max_seats, int max_pages_per_seq)
    : alloc_(num_pages), page_size_(page_size), max_seats_(max_seats), max_pages_(max_pages_per_seq),
      table_(static_cast<size_t>(max_seats) * max_pages_per_seq, kUnusedPage), lengths_(max_seats, 0), pages_(max_seats),
      dirty_(max_seats, 0) {}

bool KVPageTable::can_reserve(int seat, int total_tokens) const {
    const int need = (total_tokens + page_size_ - 1) / page_size_;
    if (need > max_pages_) return false;
    const int have = static_cast<int>(pages_.at(seat).size());
    return need - have <= alloc_.free_pages();
}

void KVPageTable::reserve(int seat, int total_tokens) {
    const int need = (total_tokens + page_size_ - 1) / page_size_;
    if (need > max_pages_)
        throw std::runtime_error("sequence of " + std::to_string(total_tokens) + " tokens exceeds " + std::to_string(max_pages_) + " pages");
    auto& have = pages_.at(seat);
    if (need > static_cast<int>(have.size())) {
        const auto fresh = alloc_.alloc(need - static_cast<int>(have.size()));
        int32_t* r = table_.data() + static_cast<size_t>(seat) * max_pages_;
        for (int32_t p : fresh) {
            r[have.size()] = p;
            have.push_back(p);
        }
        dirty_[seat] = 1;
    }
}

void KVPageTable::adopt_prefix(int seat, const std::vector<int32_t>& pages, int tokens) {
    if (!pages_.at(seat).empty()) throw std::runtime_error("adopt_prefix on a non-empty seat");
    if (static_cast<int>(pages.size()) > max_pages_) throw std::runtime_error("prefix longer than a page-table row");
    alloc_.retain(pages);
    pages_[seat] = pages;
    std::copy(pages.begin(), pages.end(), table_.begin() + static_cast<size_t>(seat) * max_pages_);
    lengths_[seat] = tokens;
    dirty_[seat] = 1;
}

void KVPageTable::rewind(int seat, int length) {
    if (length > lengths_.at(seat) || length < 0) throw std::runtime_error("rewind beyond the committed length");
    lengths_[seat] = length;
}

int KVPageTable::retire_before(int seat, int first_live_token) {
    auto& have = pages_.at(seat);
    const int upto = std::min(static_cast<int>(have.size()), std::max(first_live_token, 0) / page_size_);
    int32_t* r = table_.data() + static_cast<size_t>(seat) * max_pages_;
    std::vector<int32_t> gone;
    for (int i = 0; i < upto; ++i)
        if (have[i] != kUnusedPage) {
            gone.push_back(have[i]);
            have[i] = kUnusedPage;
            r[i] = kUnusedPage;
        }
    if (!gone.empty()) {
        alloc_.release(gone);
        dirty_[seat] = 1;
    }
    return static_cast<int>(gone.size());
}

int KVPageTable::live_pages(int seat) const {
    int n = 0;
    for (int32_t p : pages_.at(seat)) n += p != kUnusedPage;
    return n;
}

void KVPageTable::free_seat(int seat) {
    std::vector<int32_t> live;
    for (int32_t p : pages_.at(seat))
        if (p != kUnusedPage) live.push_back(p);
    alloc_.release(live);
    pages_[seat].clear();
    std::fill_n(table_.begin() + static_cast<size_t>(seat) * max_pages_, max_pages_, kUnusedPage);
    lengths_[seat] = 0;
    dirty_[seat] = 1;
}

std::vector<int> KVPageTable::take_dirty_rows() {
    std::vector<int> rows;
    for (int s = 0; s < max_seats_; ++s)
        if (dirty_[s]) {
            rows.push_back(s);
            dirty_[s] = 0;
        }
    return rows;
}

ResidentSlotPool::ResidentSlotPool(int n) : epoch_(n, 0), used_(n, 0) {
    for (int s = n - 1; s >= 0; --s) free_.push_back(s);
}

int ResidentSlotPool::acquire() {
    if (free_.empty()) return -1;
    const int s = free_.back();
    free_.pop_back();
    used_[s] = 1;
    ++epoch_[s];
    ++in_use_;
    return s;
}

void ResidentSlotPool::release(int slot) {
    if (!used_.at(slot)) throw std::runtime_error("release of a free slot");
    used_[slot] = 0;
    free_.push_back(slot);
    --in_use_;
}

PrefixCache::PrefixCache(PageAllocator& alloc, int page_size, int max_records)
    : alloc_(alloc), page_size_(page_size), max_records_(max_records) {}

uint64_t PrefixCache::hash_block(uint64_t parent, const int32_t* tokens, int n) {
    uint64_t h = 0xcbf29ce484222325ull ^ (parent * 0x9E3779B97F4A7C15ull);     // FNV-1a over the bytes, seeded by the parent
    const uint8_t* b = reinterpret_cast<const uint8_t*>(tokens);
    for (int i = 0; i < n * 4; ++i) {
        h ^= b[i];
        h *= 0x100000001b3ull;
    }
    return h ? h : 1;
}

uint64_t PrefixCache::check_block(uint64_t parent_check, const int32_t* tokens, int n) {
    // splitmix64-style mixing over whole tokens: shares no structure with the byte-wise FNV-1a of hash_block
    uint64_t h = parent_check ^ 0xD6E8FEB86659FD93ull;
    for (int i = 0; i < n; ++i) {
        uint64_t z = h + 0x9E3779B97F4A7C15ull + static_cast<uint32_t>(tokens[i]);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        h = z ^ (z >> 31);
    }
    return h;
}

uint64_t PrefixCache::extras_seed(const std::string& adapter, uint64_t adapter_generation, const std::string& isolation_key) {
    if (adapter.empty() && isolation_key.empty()) return 0;
    uint64_t h = 0xcbf29ce484222325ull;
    auto mix = [&h](const void* p, size_t n) {
        const uint8_t* b = static_cast<const uint8_t*>(p);
        for (size_t i = 0; i < n; ++i) {
            h ^= b[i];
            h *= 0x100000001b3ull;
        }
    };
    mix(adapter.data(), adapter.size());
    const uint8_t sep = 0xff;
    mix(&sep, 1);
    mix(&adapter_generation, sizeof(adapter_generation));
    mix(&sep, 1);
    mix(isolation_key.data(), isolation_key.size());
    return h ? h : 1;
}

PrefixCache::Match PrefixCache::lookup(const std::vector<int32_t>& tokens, uint64_t seed) {
    Match m;
    const int full = (static_cast<int>(tokens.size()) - 1) / page_size_;   // leave >= 1 token to compute
    uint64_t parent = seed, check = seed;
    std::vector<std::list<uint64_t>::iterator> chain;
    for (int b = 0; b < full; ++b) {
        const int32_t* blk = tokens.data() + static_cast<size_t>(b) * page_size_;
        const uint64_t h = hash_block(parent, blk, page_size_);
        check = check_block(check, blk, page_size_);
        auto it = map_.find(h);
        if (it == map_.end()) break;
        if (it->second.check != check) {       // same 64-bit key, other content: not this prompt's page
            ++mismatches_;
            break;
        }
        chain.push_back(it->second.lru);
        m.pages.push_back(it->second.page);
        m.tokens += page_size_;
        parent = h;
    }
    touch_chain(chain);
    if (m.tokens > 0) ++hits_; else ++misses_;
    return m;
}

// Mark a chain of entries (given root first) as just used, leaves first: the root ends up the most recent of them, so eviction
// from the old end of the list takes a chain's tail pages before the pages every continuation of the prefix depends on.
void PrefixCache::touch_chain(const std::vector<std::list<uint64_t>::iterator>& chain) {
    for (auto it = chain.rbegin(); it != chain.rend(); ++it) lru_.splice(lru_.begin(), lru_, *it);
}

int PrefixCache::insert(const std::vector<int32_t>& tokens, int filled_tokens, const std::vector<int32_t>& pages, uint64_t seed) {
    const int full = std::min<int>(filled_tokens, static_cast<int>(tokens.size())) / page_size_;
    uint64_t parent = seed, check = seed;
    int added = 0;
    std::vector<std::list<uint64_t>::iterator> chain;
    for (int b = 0; b < full && b < static_cast<int>(pages.size()); ++b) {
        const int32_t* blk = tokens.data() + static_cast<size_t>(b) * page_size_;
        const uint64_t h = hash_block(parent, blk, page_size_);
        check = check_block(check, blk, page_size_);
        parent = h;
        auto it = map_.find(h);
        if (it != map_.end()) {
            if (it->second.check != check) {   // the slot belongs to other content: the rest of this chain stays uncached
                ++mismatches_;
                break;
            }
            chain.push_back(it->second.lru);
            continue;
        }
        if (static_cast<int>(map_.size()) >= max_records_) {
            // at the record limit: drop the oldest record that is not part of the chain being registered
            touch_chain(chain);
            chain.clear();
            if (drop_records(1) == 0) break;
        }
        alloc_.retain({pages[b]});
        lru_.push_front(h);
        map_[h] = Entry{pages[b], check, lru_.begin()};
        chain.push_back(lru_.begin());
        ++added;
    }
    touch_chain(chain);
    return added;
}

int PrefixCache::drop_records(int n) {
    int dropped = 0;
    while (dropped < n && !lru_.empty()) {
        const uint64_t h = lru_.back();
        lru_.pop_back();
        auto it = map_.find(h);
        if (it != map_.end()) {
            alloc_.release({it->second.page});
            map_.erase(it);
            ++dropped;
        }
    }
    return dropped;
}

// Read-only simulation: walk the records from least to most recently used; a record's page comes back to the pool only when the
// cache holds the last reference (no resident sequence shares it).  The plan is the shortest such run of victims that covers
// the demand; records whose pages are still shared are passed over, since dropping them frees nothing and loses the entry.
PrefixCache::EvictionPlan PrefixCache::plan_eviction(int pages_wanted) const {
    EvictionPlan plan;
    plan.pages_wanted = pages_wanted;
    for (auto it = lru_.rbegin(); it != lru_.rend() && plan.reclaimable_pages < pages_wanted; ++it) {
        auto e = map_.find(*it);
        if (e == map_.end()) continue;
        if (alloc_.refcount(e->second.page) == 1) {
            plan.victims.push_back(*it);
            ++plan.reclaimable_pages;
        } else {
            ++plan.pinned_skipped;
        }
    }
    plan.satisfied = plan.reclaimable_pages >= pages_wanted;
    return plan;
}

// Carry out a plan (records that vanished or became shared since it was made are passed over).  Returns the pages freed.
int PrefixCache::evict(const EvictionPlan& plan) {
    int freed = 0;
    for (uint64_t h : plan.victims) {
        auto it = map_.find(h);
        if (it == map_.end() || alloc_.refcount(it->second.page) != 1) continue;
        alloc_.release({it->second.page});
        lru_.erase(it->second.lru);
        map_.erase(it);
        ++freed;
    }
    return freed;
}

int PrefixCache::evict(int pages_wanted) { return evict(plan_eviction(pages_wanted)); }

}  // namespace telb
