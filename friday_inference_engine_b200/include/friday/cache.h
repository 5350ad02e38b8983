// The cache of a model: a slot for each live sequence, groups of paged keys and values,
// fixed-size states.
//
// It is built from what the model's mixers ask for, entry by entry (parts.h,
// CacheRequest).  Requests for keys and values with the same needs (kv heads, head size,
// window) form a group with storage of its own:
//
//   k_pool, v_pool   [entries, pages, PAGE, kv_heads, head_dim] in the activation dtype
//   a free list of page numbers (a page number means the same rows in every entry)
//   table            host array [slots, width]: page of each logical page of each slot, -1 where none is held
//
// A group without a window keeps every position of a live sequence.  A group with a
// window W gives a page back as soon as every position in it is more than W-1 behind the
// sequence's end: no later query can reach it, so a long sequence holds about
// W/PAGE + 2 pages of such a group.  Every state request gets a tensor [slots, *shape]
// that is zeroed when a slot is taken.  Lengths, not contents, decide what is valid:
// slots and pages are used again without being cleared.
//
// Capacity is given in tokens: `max_tokens` is the most that live sequences hold together,
// each counted in whole pages of 64; `max_seq_tokens` bounds one sequence.  The
// reference keeps two flat buffers [layers][ctx][kv] for its one sequence
// (transformer.h:145-149, transformer.cpp:483-497); pages and slots are this library's.
#pragma once
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "friday/base.h"
#include "friday/ops.h"
#include "friday/parts.h"

namespace friday {

constexpr int PAGE = 64;

// Hands out the integers 0 .. n-1, lowest first among those given back last.
class FreeList {
public:
    FreeList(int n, const std::string& what);
    int take();                      // CacheFull if none is free
    void give(int i);                // CacheError if i is not held (freed twice, or never taken)
    bool holds(int i) const { return i >= 0 && i < n_ && held_[i]; }
    int free_count() const { return (int)free_.size(); }
    int held_count() const { return n_ - (int)free_.size(); }
    int size() const { return n_; }

private:
    int n_;
    std::string what_;
    std::vector<int> free_;
    std::vector<char> held_;
};

class KVGroup {
public:
    KVGroup(const CacheRequest& request, const std::vector<int>& entries, int n_slots, int n_pages, int width,
            DType dtype, bool on_device);
    CacheRequest request;
    std::vector<int> entries;        // cache entry ids, in pool order
    int window, n_pages, width;
    DType dtype;
    FreeList pages;
    std::vector<int> table;          // [slots][width]
    DeviceBuffer k_pool, v_pool;

    int index_of(int entry) const;
    size_t entry_bytes() const { return (size_t)n_pages * PAGE * request.n_kv_heads * request.head_dim * dtype_size(dtype); }
    int first_needed_page(int start_pos) const;                     // logical page of the earliest key a query at start_pos or later sees
    std::vector<int> pages_missing(int slot, int start_pos, int new_len) const;
    void reserve(int slot, int start_pos, int new_len);
    void release_behind(int slot, int length);                      // pages no query at position >= length can reach
    void release_all(int slot);
    std::vector<int> held_pages(int slot) const;
    const int* table_row(int slot) const { return &table[(size_t)slot * width]; }
};

class Cache {
public:
    // requests: cache entry id -> what the mixer that writes it asks for.  on_device false builds the
    // book-keeping alone (no pools, no states): what the tests of slots and pages use where there is no GPU.
    Cache(const std::map<int, CacheRequest>& requests, int64_t max_tokens, int max_seq_tokens, DType dtype, int max_slots,
          bool on_device, cudaStream_t stream = nullptr);

    int alloc_slot();                // lengths start at 0, states at zero
    void free_slot(int slot);        // CacheError if the slot is not held
    // Pages for the tokens that each slot is about to take.  Either all of it succeeds or nothing is held
    // afterwards that was not held before.
    void reserve(const std::vector<int>& slots, const std::vector<int>& q_lens);
    void commit(const std::vector<int>& slots, const std::vector<int>& q_lens);
    // Group g's block table rows of `slots`, appended to `out` ([n][width] ints).
    void table_rows(int g, const std::vector<int>& slots, std::vector<int>& out) const;
    // The view of `entry` for one layer call; tables: per group, this step's block table on the device.
    CacheView view(int entry, bool write, const std::vector<const int*>& step_tables, const int* seq_slots_dev) const;

    int64_t held_tokens() const;
    size_t bytes() const;
    int64_t capacity_tokens() const { return groups.empty() ? 0 : (int64_t)groups[0]->n_pages * PAGE; }

    int max_seq_tokens, max_slots;
    FreeList slots;
    std::vector<int> lens;
    std::vector<std::unique_ptr<KVGroup>> groups;
    std::map<int, int> group_of;                    // entry -> index into groups
    struct State { std::vector<int64_t> shape; DType dtype; size_t slot_bytes; DeviceBuffer memory; };
    std::map<int, State> states;                    // entry -> [slots, *shape]

private:
    bool on_device_;
    cudaStream_t stream_;
};

}  // namespace friday
