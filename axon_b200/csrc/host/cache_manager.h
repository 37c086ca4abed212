// The cache manager's host side: pages, block tables and request slots.
//
// A *group* is a set of layers with the same needs (bytes per token, keep all
// positions or a window of them).  Each group has its own pool of pages and, for
// every request slot, its own block table: logical page (position / page_size)
// -> physical page.  A page covers `page_size` positions of every layer of its
// group.  Entries that hold no page point at the *sink page* (index n_pages,
// one extra page behind the pool) so that a stray access lands somewhere harmless
// (the reference's sink idea: src/cuda/qwen2/slots.rs:52-55,288-306).
//
// Freeing is two-phase as in the reference's PageMap (src/cuda/qwen2/pages.rs:141-153,
// 308-311): a released page is *retired* and becomes free at the next flush(), which
// the engine calls once the step that may still read it has been queued.
// A slot's table grows only at its end; window groups give up pages from the front
// once every position they cover has left the window.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace axon {

struct CacheError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

class PageAllocator {
public:
    // shuffle_seed != 0 hands pages out in a seeded random order, which shows
    // kernels that wrongly assume neighbouring pages (src/cuda/qwen2/pages.rs:354-366).
    explicit PageAllocator(int n_pages, uint64_t shuffle_seed = 0);

    int alloc();               // a page with one reference, or -1 when none is free
    void retain(int page);     // one more reference
    void release(int page);    // one less; the last one retires the page
    void flush();              // retired pages become free
    int n_pages() const { return (int)refs_.size(); }
    int n_free() const { return (int)free_.size(); }
    int n_retired() const { return (int)retired_.size(); }
    int n_held() const { return n_pages() - n_free() - n_retired(); }
    int refs(int page) const;
    // Every page is free, retired or held, exactly once; throws CacheError otherwise.
    void check() const;

private:
    std::vector<int32_t> free_;     // LIFO
    std::vector<int32_t> retired_;
    std::vector<int32_t> refs_;
    std::vector<uint8_t> state_;    // 0 free, 1 held, 2 retired
};

struct GroupConfig {
    int page_size = 16;
    int n_pages = 0;
    int window = 0;  // 0: keep every position; else only the last `window`
};

class CacheManager {
public:
    CacheManager(std::vector<GroupConfig> groups, int max_slots, int max_positions,
                 uint64_t shuffle_seed = 0);

    int n_groups() const { return (int)groups_.size(); }
    int max_slots() const { return max_slots_; }
    int max_positions() const { return max_positions_; }
    const GroupConfig& group(int g) const { return groups_.at(g); }
    int table_stride(int g) const { return strides_.at(g); }
    int sink_page(int g) const { return groups_.at(g).n_pages; }

    // Slots: one per live request; the slot id also indexes the per-request state slabs.
    int open_slot();            // -1 when every slot is taken
    void close_slot(int slot);  // gives back every page the slot holds
    bool is_open(int slot) const;
    int n_open() const;
    int length(int slot) const;  // positions committed so far

    // Pages the slot would have to take, per group summed, to hold positions 0..new_len-1.
    int pages_short(int slot, int new_len) const;  // how many more than are free (0: fits)
    // Take pages for positions up to new_len (all groups or none).  False: not enough pages.
    bool reserve(int slot, int new_len);
    // The step that wrote positions up to new_len is queued: remember the length and let
    // window groups give up pages no later query can reach.
    void commit(int slot, int new_len);
    // Retired pages become free.
    void flush();

    // A step of one token for each of `n` requests, laid out for the device in one call (what the
    // step function otherwise does entry by entry): checks the slots (open, distinct), the tokens
    // (0 <= t < vocab) and the context limit, flushes, takes the pages, and fills `out`:
    //   tokens[n] positions[n] slots[n] segments[4][n] (slot, q_start, 1, kv_len) wanted rows[n_want]
    //   items[n][2] (segment, 0)
    // wanted[i] != 0 asks for request i's logits.  Returns 0; 1 when the input is irregular (nothing
    // is taken; the caller's own checks find the words for it); 2 when request *bad has no pages.
    int stage_decode(const int* slots, const int* tokens, const unsigned char* wanted, int n, int vocab,
                     int32_t* out, int* bad);
    // The lengths of those requests grow by one.
    void commit_decode(const int* slots, int n);

    // Any step, laid out for the device in one call: entry i brings tokens[tok_off[i] .. tok_off[i+1])
    // for the request in slots[i] and wants the logits at the places wants[want_off[i] .. want_off[i+1])
    // among them.  Checks as stage_decode (and that a step holds at most max_step_tokens tokens and
    // every wanted place lies inside its entry), flushes, takes the pages, and fills `out`:
    //   tokens[T] positions[T] slots[T] segments[4][S] (slot, q_start, q_len, kv_len) wanted rows[W]
    //   and, when every entry brings one token, items[S][2] (segment, 0)
    // with T tokens, S entries and W wanted places in all (`lay`).  `out` must hold
    // 3 T + 6 S + W values.  Returns as stage_decode.
    struct StepLayout { int n_tokens = 0, n_entries = 0, n_want = 0, decode_only = 0, total = 0; };
    int stage_step(const int* slots, const int* tok_off, const int32_t* tokens, const int* want_off, const int* wants,
                   int n_entries, int vocab, int max_step_tokens, int32_t* out, long long out_capacity,
                   StepLayout* lay, int* bad);
    // The lengths of the step's requests grow by what the step brought (`segments` as laid out above).
    void commit_step(const int32_t* segments, int n_entries);

    int free_pages(int g) const { return allocs_.at(g).n_free(); }
    int retired_pages(int g) const { return allocs_.at(g).n_retired(); }
    int held_pages(int g) const { return allocs_.at(g).n_held(); }
    int slot_pages(int g, int slot) const;  // pages the slot holds in group g
    int reserved_length(int slot) const;    // positions its pages cover
    // Pages needed to hold `tokens` positions from empty, summed over groups (window
    // groups count at most what a window spans).
    int pages_for(int tokens) const;
    // Pages of group g the slot would have to take to hold positions 0..new_len-1.
    int pages_needed(int g, int slot, int new_len) const;
    // How many positions the slot could cover with the pages it holds plus the free
    // ones, leaving `spare` pages of every group untouched.
    int coverable(int slot, int spare) const;
    // Whether an otherwise empty pool holds `tokens` positions of one request.
    bool could_ever_hold(int tokens) const;

    // The host copy of group g's block table: [max_slots][table_stride(g)] int32.
    const int32_t* table(int g) const { return tables_.at(g).data(); }
    int32_t* table_mut(int g) { return tables_.at(g).data(); }
    // Raised when a row of a table changes; the engine copies changed tables to the device.
    uint64_t version(int g) const { return versions_.at(g); }

    // No page lost, held twice or freed twice; tables agree with what slots hold.
    void check() const;

private:
    struct Slot {
        bool open = false;
        int length = 0;
        int reserved = 0;  // positions covered by pages
        std::vector<int> first_page;  // per group: first logical page still held
    };
    int logical_pages(int g, int positions) const;
    int first_needed(int g, int next_query_pos) const;

    std::vector<unsigned char> stage_seen_;   // scratch of stage_decode
    std::vector<GroupConfig> groups_;
    int max_slots_, max_positions_;
    std::vector<PageAllocator> allocs_;
    std::vector<int> strides_;
    std::vector<std::vector<int32_t>> tables_;
    std::vector<uint64_t> versions_;
    std::vector<Slot> slots_;
    std::vector<int> free_slots_;
};

}  // namespace axon
