#include "cache_manager.h"

#include <algorithm>
#include <numeric>

namespace axon {

namespace {
// splitmix64: a small seeded generator for the shuffled hand-out order.
uint64_t splitmix(uint64_t& s) {
    s += 0x9e3779b97f4a7c15ull;
    uint64_t z = s;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
}  // namespace

PageAllocator::PageAllocator(int n_pages, uint64_t shuffle_seed) {
    if (n_pages < 0) throw CacheError("a pool cannot have a negative number of pages");
    refs_.assign(n_pages, 0);
    state_.assign(n_pages, 0);
    free_.resize(n_pages);
    // LIFO: the back is handed out first, so page 0 goes first without a shuffle
    for (int i = 0; i < n_pages; ++i) free_[i] = n_pages - 1 - i;
    if (shuffle_seed) {
        uint64_t s = shuffle_seed;
        for (int i = n_pages - 1; i > 0; --i) std::swap(free_[i], free_[splitmix(s) % (uint64_t)(i + 1)]);
    }
}

int PageAllocator::alloc() {
    if (free_.empty()) return -1;
    const int p = free_.back();
    free_.pop_back();
    refs_[p] = 1;
    state_[p] = 1;
    return p;
}

void PageAllocator::retain(int page) {
    if (page < 0 || page >= n_pages() || state_[page] != 1)
        throw CacheError("retain of page " + std::to_string(page) + ", which is not held");
    ++refs_[page];
}

void PageAllocator::release(int page) {
    if (page < 0 || page >= n_pages()) throw CacheError("release of page " + std::to_string(page) + ", which does not exist");
    if (state_[page] != 1 || refs_[page] <= 0)
        throw CacheError("page " + std::to_string(page) + " was freed twice");
    if (--refs_[page] == 0) {
        state_[page] = 2;
        retired_.push_back(page);
    }
}

void PageAllocator::flush() {
    for (int p : retired_) {
        state_[p] = 0;
        free_.push_back(p);
    }
    retired_.clear();
}

int PageAllocator::refs(int page) const {
    if (page < 0 || page >= n_pages()) throw CacheError("page " + std::to_string(page) + " does not exist");
    return refs_[page];
}

void PageAllocator::check() const {
    std::vector<int> seen(n_pages(), 0);
    for (int p : free_) {
        if (p < 0 || p >= n_pages()) throw CacheError("free list holds page " + std::to_string(p));
        if (state_[p] != 0 || refs_[p] != 0) throw CacheError("page " + std::to_string(p) + " is free and in use");
        ++seen[p];
    }
    for (int p : retired_) {
        if (p < 0 || p >= n_pages()) throw CacheError("retired list holds page " + std::to_string(p));
        if (state_[p] != 2 || refs_[p] != 0) throw CacheError("page " + std::to_string(p) + " is retired and in use");
        ++seen[p];
    }
    for (int p = 0; p < n_pages(); ++p) {
        if (state_[p] == 1) {
            if (refs_[p] <= 0) throw CacheError("page " + std::to_string(p) + " is held without a reference");
            ++seen[p];
        }
        if (seen[p] != 1) throw CacheError("page " + std::to_string(p) + " is accounted " + std::to_string(seen[p]) + " times");
    }
}

// ---------------------------------------------------------------------------

CacheManager::CacheManager(std::vector<GroupConfig> groups, int max_slots, int max_positions,
                           uint64_t shuffle_seed)
    : groups_(std::move(groups)), max_slots_(max_slots), max_positions_(max_positions) {
    if (max_slots_ <= 0) throw CacheError("the cache needs at least one request slot");
    if (max_positions_ <= 0) throw CacheError("the cache needs room for at least one position");
    for (size_t g = 0; g < groups_.size(); ++g) {
        const GroupConfig& c = groups_[g];
        if (c.page_size <= 0) throw CacheError("page size must be positive");
        if (c.window < 0) throw CacheError("a window cannot be negative");
        allocs_.emplace_back(c.n_pages, shuffle_seed ? shuffle_seed + 0x1000 * (g + 1) : 0);
        strides_.push_back((max_positions_ + c.page_size - 1) / c.page_size);
        tables_.emplace_back((size_t)max_slots_ * strides_.back(), (int32_t)c.n_pages);
        versions_.push_back(1);
    }
    slots_.resize(max_slots_);
    for (auto& s : slots_) s.first_page.assign(groups_.size(), 0);
    for (int i = max_slots_ - 1; i >= 0; --i) free_slots_.push_back(i);
}

int CacheManager::open_slot() {
    if (free_slots_.empty()) return -1;
    const int s = free_slots_.back();
    free_slots_.pop_back();
    Slot& sl = slots_[s];
    sl.open = true;
    sl.length = 0;
    sl.reserved = 0;
    std::fill(sl.first_page.begin(), sl.first_page.end(), 0);
    return s;
}

bool CacheManager::is_open(int slot) const { return slot >= 0 && slot < max_slots_ && slots_[slot].open; }

int CacheManager::n_open() const { return max_slots_ - (int)free_slots_.size(); }

int CacheManager::length(int slot) const {
    if (!is_open(slot)) throw CacheError("slot " + std::to_string(slot) + " is not open");
    return slots_[slot].length;
}

int CacheManager::reserved_length(int slot) const {
    if (!is_open(slot)) throw CacheError("slot " + std::to_string(slot) + " is not open");
    return slots_[slot].reserved;
}

int CacheManager::logical_pages(int g, int positions) const {
    const int ps = groups_[g].page_size;
    return (positions + ps - 1) / ps;
}

int CacheManager::first_needed(int g, int next_query_pos) const {
    const GroupConfig& c = groups_[g];
    if (c.window == 0) return 0;
    const int first_key = std::max(0, next_query_pos - c.window + 1);
    return first_key / c.page_size;
}

void CacheManager::close_slot(int slot) {
    if (!is_open(slot)) throw CacheError("slot " + std::to_string(slot) + " was closed twice");
    Slot& sl = slots_[slot];
    for (int g = 0; g < n_groups(); ++g) {
        int32_t* row = tables_[g].data() + (size_t)slot * strides_[g];
        const int hi = logical_pages(g, sl.reserved);
        for (int lp = sl.first_page[g]; lp < hi; ++lp) {
            allocs_[g].release(row[lp]);
            row[lp] = groups_[g].n_pages;
        }
        ++versions_[g];
    }
    sl.open = false;
    sl.length = sl.reserved = 0;
    free_slots_.push_back(slot);
}

int CacheManager::pages_short(int slot, int new_len) const {
    if (!is_open(slot)) throw CacheError("slot " + std::to_string(slot) + " is not open");
    const Slot& sl = slots_[slot];
    int shortfall = 0;
    for (int g = 0; g < n_groups(); ++g) {
        const int need = logical_pages(g, std::max(new_len, sl.reserved)) - logical_pages(g, sl.reserved);
        shortfall += std::max(0, need - allocs_[g].n_free());
    }
    return shortfall;
}

bool CacheManager::reserve(int slot, int new_len) {
    if (!is_open(slot)) throw CacheError("slot " + std::to_string(slot) + " is not open");
    if (new_len > max_positions_)
        throw CacheError("a request of " + std::to_string(new_len) + " positions exceeds the cache's limit of " +
                         std::to_string(max_positions_));
    Slot& sl = slots_[slot];
    if (new_len <= sl.reserved) return true;
    if (pages_short(slot, new_len) > 0) return false;
    for (int g = 0; g < n_groups(); ++g) {
        int32_t* row = tables_[g].data() + (size_t)slot * strides_[g];
        const int lo = logical_pages(g, sl.reserved), hi = logical_pages(g, new_len);
        for (int lp = lo; lp < hi; ++lp) row[lp] = allocs_[g].alloc();
        if (hi > lo) ++versions_[g];
    }
    sl.reserved = new_len;
    return true;
}

void CacheManager::commit(int slot, int new_len) {
    if (!is_open(slot)) throw CacheError("slot " + std::to_string(slot) + " is not open");
    Slot& sl = slots_[slot];
    if (new_len < sl.length) throw CacheError("a request's length cannot shrink");
    if (new_len > sl.reserved) throw CacheError("positions were written without pages reserved for them");
    sl.length = new_len;
    for (int g = 0; g < n_groups(); ++g) {
        const int keep_from = std::min(first_needed(g, new_len), logical_pages(g, sl.reserved));
        if (keep_from <= sl.first_page[g]) continue;
        int32_t* row = tables_[g].data() + (size_t)slot * strides_[g];
        for (int lp = sl.first_page[g]; lp < keep_from; ++lp) {
            allocs_[g].release(row[lp]);
            row[lp] = groups_[g].n_pages;
        }
        sl.first_page[g] = keep_from;
        ++versions_[g];
    }
}

void CacheManager::flush() {
    for (auto& a : allocs_) a.flush();
}

int CacheManager::stage_decode(const int* slots, const int* tokens, const unsigned char* wanted, int n, int vocab,
                               int32_t* out, int* bad) {
    *bad = -1;
    if (n <= 0) return 1;
    stage_seen_.assign((size_t)max_slots_, 0);
    for (int i = 0; i < n; ++i) {
        const int s = slots[i];
        if (s < 0 || s >= max_slots_ || !is_open(s) || stage_seen_[s]) return 1;
        stage_seen_[s] = 1;
        if (tokens[i] < 0 || tokens[i] >= vocab) return 1;
        if (slots_[s].length + 1 > max_positions_) return 1;
    }
    flush();
    for (int i = 0; i < n; ++i) {
        if (!reserve(slots[i], slots_[slots[i]].length + 1)) { *bad = i; return 2; }
    }
    int32_t* tok = out; int32_t* pos = out + n; int32_t* sl = out + 2 * n; int32_t* seg = out + 3 * n;
    int32_t* want = out + 7 * n;
    int n_want = 0;
    for (int i = 0; i < n; ++i) {
        const int start = slots_[slots[i]].length;
        tok[i] = tokens[i]; pos[i] = start; sl[i] = slots[i];
        seg[i] = slots[i]; seg[n + i] = i; seg[2 * n + i] = 1; seg[3 * n + i] = start + 1;
        if (wanted[i]) want[n_want++] = i;
    }
    int32_t* items = want + n_want;
    for (int i = 0; i < n; ++i) { items[2 * i] = i; items[2 * i + 1] = 0; }
    return 0;
}

void CacheManager::commit_decode(const int* slots, int n) {
    for (int i = 0; i < n; ++i) commit(slots[i], slots_[slots[i]].length + 1);
}

int CacheManager::stage_step(const int* slots, const int* tok_off, const int32_t* tokens, const int* want_off,
                             const int* wants, int n_entries, int vocab, int max_step_tokens, int32_t* out,
                             long long out_capacity, StepLayout* lay, int* bad) {
    *bad = -1;
    if (n_entries <= 0) return 1;
    const int S = n_entries;
    if (tok_off[0] != 0 || want_off[0] != 0) return 1;
    const long long T = tok_off[S], W = want_off[S];
    if (T > max_step_tokens) return 1;
    stage_seen_.assign((size_t)max_slots_, 0);
    bool decode_only = true;
    for (int i = 0; i < S; ++i) {
        const int s = slots[i];
        if (s < 0 || s >= max_slots_ || !is_open(s) || stage_seen_[s]) return 1;
        stage_seen_[s] = 1;
        const int k = tok_off[i + 1] - tok_off[i];
        if (k <= 0 || want_off[i + 1] < want_off[i]) return 1;
        if (k != 1) decode_only = false;
        for (int t = tok_off[i]; t < tok_off[i + 1]; ++t)
            if (tokens[t] < 0 || tokens[t] >= vocab) return 1;
        for (int w = want_off[i]; w < want_off[i + 1]; ++w)
            if (wants[w] < 0 || wants[w] >= k) return 1;
        if ((long long)slots_[s].length + k > max_positions_) return 1;
    }
    const long long total = 3 * T + 4 * S + W + (decode_only ? 2 * S : 0);
    if (total > out_capacity) return 1;
    flush();
    for (int i = 0; i < S; ++i) {
        if (!reserve(slots[i], slots_[slots[i]].length + (tok_off[i + 1] - tok_off[i]))) { *bad = i; return 2; }
    }
    int32_t* tok = out; int32_t* pos = out + T; int32_t* sl = out + 2 * T; int32_t* seg = out + 3 * T;
    int32_t* want = seg + 4 * S;
    int n_want = 0;
    for (int i = 0; i < S; ++i) {
        const int at = tok_off[i], k = tok_off[i + 1] - at, start = slots_[slots[i]].length;
        for (int j = 0; j < k; ++j) { tok[at + j] = tokens[at + j]; pos[at + j] = start + j; sl[at + j] = slots[i]; }
        seg[i] = slots[i]; seg[S + i] = at; seg[2 * S + i] = k; seg[3 * S + i] = start + k;
        for (int w = want_off[i]; w < want_off[i + 1]; ++w) want[n_want++] = at + wants[w];
    }
    if (decode_only) {
        int32_t* items = want + n_want;
        for (int i = 0; i < S; ++i) { items[2 * i] = i; items[2 * i + 1] = 0; }
    }
    lay->n_tokens = (int)T; lay->n_entries = S; lay->n_want = n_want; lay->decode_only = decode_only ? 1 : 0;
    lay->total = (int)total;
    return 0;
}

void CacheManager::commit_step(const int32_t* segments, int n_entries) {
    for (int i = 0; i < n_entries; ++i) commit(segments[i], segments[3 * n_entries + i]);
}

int CacheManager::slot_pages(int g, int slot) const {
    if (!is_open(slot)) return 0;
    const Slot& sl = slots_[slot];
    return logical_pages(g, sl.reserved) - sl.first_page.at(g);
}

int CacheManager::pages_for(int tokens) const {
    int n = 0;
    for (int g = 0; g < n_groups(); ++g) n += logical_pages(g, tokens);
    return n;
}

int CacheManager::pages_needed(int g, int slot, int new_len) const {
    if (!is_open(slot)) throw CacheError("slot " + std::to_string(slot) + " is not open");
    const Slot& sl = slots_[slot];
    return logical_pages(g, std::max(new_len, sl.reserved)) - logical_pages(g, sl.reserved);
}

int CacheManager::coverable(int slot, int spare) const {
    if (!is_open(slot)) throw CacheError("slot " + std::to_string(slot) + " is not open");
    const Slot& sl = slots_[slot];
    long long reach = max_positions_;
    for (int g = 0; g < n_groups(); ++g) {
        const long long pages = logical_pages(g, sl.reserved) + std::max(0, allocs_[g].n_free() - spare);
        reach = std::min(reach, pages * groups_[g].page_size);
    }
    return (int)reach;
}

bool CacheManager::could_ever_hold(int tokens) const {
    if (tokens > max_positions_) return false;
    for (int g = 0; g < n_groups(); ++g)
        if (logical_pages(g, tokens) > groups_[g].n_pages) return false;
    return true;
}

void CacheManager::check() const {
    for (int g = 0; g < n_groups(); ++g) {
        allocs_[g].check();
        const int n = groups_[g].n_pages;
        std::vector<int> held(n, 0);
        for (int s = 0; s < max_slots_; ++s) {
            const int32_t* row = tables_[g].data() + (size_t)s * strides_[g];
            const Slot& sl = slots_[s];
            const int lo = sl.open ? sl.first_page[g] : 0;
            const int hi = sl.open ? logical_pages(g, sl.reserved) : 0;
            for (int lp = 0; lp < strides_[g]; ++lp) {
                const bool inside = sl.open && lp >= lo && lp < hi;
                if (inside) {
                    if (row[lp] < 0 || row[lp] >= n)
                        throw CacheError("slot " + std::to_string(s) + " lost the page of logical page " + std::to_string(lp));
                    if (++held[row[lp]] > 1)
                        throw CacheError("page " + std::to_string(row[lp]) + " is held twice");
                    if (allocs_[g].refs(row[lp]) != 1)
                        throw CacheError("page " + std::to_string(row[lp]) + " is in a table but not held");
                } else if (row[lp] != n) {
                    throw CacheError("slot " + std::to_string(s) + " has a page outside what it holds");
                }
            }
        }
        int total = 0;
        for (int p = 0; p < n; ++p) total += held[p];
        if (total != allocs_[g].n_held())
            throw CacheError("group " + std::to_string(g) + ": " + std::to_string(allocs_[g].n_held()) +
                             " pages are held but tables name " + std::to_string(total));
    }
}

}  // namespace axon
