// Slots and pages: who holds what (cache.h).  Book-keeping on the host; the pools are device memory.
#include "friday/cache.h"

#include <algorithm>
#include <tuple>

namespace friday {

FreeList::FreeList(int n, const std::string& what) : n_(n), what_(what), held_((size_t)n, 0) {
    free_.reserve((size_t)n);
    for (int i = n - 1; i >= 0; --i) free_.push_back(i);          // take() gives 0 first
}

int FreeList::take() {
    if (free_.empty()) throw CacheFull(format("no free %s (all %d are held)", what_.c_str(), n_));
    const int i = free_.back();
    free_.pop_back();
    held_[i] = 1;
    return i;
}

void FreeList::give(int i) {
    if (!holds(i)) throw CacheError(format("%s %d is not held (freed twice, or never taken)", what_.c_str(), i));
    held_[i] = 0;
    free_.push_back(i);
}

KVGroup::KVGroup(const CacheRequest& req, const std::vector<int>& ents, int n_slots, int pages_, int width_, DType dt,
                 bool on_device)
    : request(req), entries(ents), window(req.window), n_pages(pages_), width(width_), dtype(dt), pages(pages_, "page"),
      table((size_t)n_slots * width_, -1) {
    if (on_device) {
        k_pool = DeviceBuffer(entry_bytes() * entries.size());
        v_pool = DeviceBuffer(entry_bytes() * entries.size());
    }
}

int KVGroup::index_of(int entry) const {
    for (size_t i = 0; i < entries.size(); ++i)
        if (entries[i] == entry) return (int)i;
    return -1;
}

int KVGroup::first_needed_page(int start_pos) const {
    if (window <= 0) return 0;
    return std::max(0, start_pos - window + 1) / PAGE;
}

std::vector<int> KVGroup::pages_missing(int slot, int start_pos, int new_len) const {
    if (new_len > width * PAGE)
        throw CacheError(format("a sequence of %d tokens does not fit the cache's %d tokens per sequence", new_len, width * PAGE));
    std::vector<int> out;
    const int* row = table_row(slot);
    const int lo = first_needed_page(start_pos), hi = (new_len + PAGE - 1) / PAGE;
    for (int lp = lo; lp < hi; ++lp)
        if (row[lp] < 0) out.push_back(lp);
    return out;
}

void KVGroup::reserve(int slot, int start_pos, int new_len) {
    for (int lp : pages_missing(slot, start_pos, new_len)) table[(size_t)slot * width + lp] = pages.take();
}

void KVGroup::release_behind(int slot, int length) {
    if (window <= 0) return;
    int* row = &table[(size_t)slot * width];
    const int end = std::min(width, std::max(0, length - window + 1) / PAGE);
    for (int lp = 0; lp < end; ++lp)
        if (row[lp] >= 0) {
            pages.give(row[lp]);
            row[lp] = -1;
        }
}

void KVGroup::release_all(int slot) {
    int* row = &table[(size_t)slot * width];
    for (int lp = 0; lp < width; ++lp)
        if (row[lp] >= 0) {
            pages.give(row[lp]);
            row[lp] = -1;
        }
}

std::vector<int> KVGroup::held_pages(int slot) const {
    std::vector<int> out;
    const int* row = table_row(slot);
    for (int lp = 0; lp < width; ++lp)
        if (row[lp] >= 0) out.push_back(row[lp]);
    return out;
}

static int pages_for(int64_t tokens) { return (int)std::max<int64_t>(1, (tokens + PAGE - 1) / PAGE); }

Cache::Cache(const std::map<int, CacheRequest>& requests, int64_t max_tokens, int max_seq, DType dtype, int max_slots_,
             bool on_device, cudaStream_t stream)
    : max_seq_tokens(max_seq), max_slots(max_slots_ > 0 ? max_slots_ : std::min(pages_for(max_tokens), 4096)),
      slots(max_slots, "slot"), lens((size_t)max_slots, 0), on_device_(on_device), stream_(stream) {
    const int n_pages = pages_for(max_tokens);
    // A sequence's table has a place for every page of the longest sequence.  Without a window a sequence can never
    // hold more pages than there are, so the table need not be wider than that; with a window it holds few pages
    // at a time but at any logical place.
    const int seq_pages = std::max(1, (max_seq_tokens + PAGE - 1) / PAGE);
    typedef std::tuple<int, int, int> Need;
    std::vector<std::pair<Need, std::vector<int>>> by_need;          // in order of first appearance
    for (const auto& kv : requests) {
        const CacheRequest& r = kv.second;
        if (r.kind == CacheRequest::KV) {
            const Need need(r.n_kv_heads, r.head_dim, r.window);
            auto it = std::find_if(by_need.begin(), by_need.end(), [&](const auto& p) { return p.first == need; });
            if (it == by_need.end()) by_need.emplace_back(need, std::vector<int>{kv.first});
            else it->second.push_back(kv.first);
        } else if (r.kind == CacheRequest::State) {
            State s;
            s.shape = r.state_shape;
            s.dtype = r.state_dtype;
            int64_t n = 1;
            for (int64_t d : r.state_shape) n *= d;
            s.slot_bytes = (size_t)n * dtype_size(r.state_dtype);
            if (on_device) s.memory = DeviceBuffer(s.slot_bytes * max_slots, true);
            states.emplace(kv.first, std::move(s));
        }
    }
    for (auto& p : by_need) {
        const CacheRequest req = requests.at(p.second[0]);
        const int width = req.window > 0 ? seq_pages : std::min(n_pages, seq_pages);
        groups.emplace_back(new KVGroup(req, p.second, max_slots, n_pages, width, dtype, on_device));
        for (int e : p.second) group_of[e] = (int)groups.size() - 1;
    }
}

int Cache::alloc_slot() {
    const int slot = slots.take();
    lens[slot] = 0;
    if (on_device_)
        for (auto& kv : states)
            cuda_check(cudaMemsetAsync((char*)kv.second.memory.get() + (size_t)slot * kv.second.slot_bytes, 0,
                                       kv.second.slot_bytes, stream_), "cudaMemsetAsync");
    return slot;
}

void Cache::free_slot(int slot) {
    slots.give(slot);
    for (auto& g : groups) g->release_all(slot);
    lens[slot] = 0;
}

void Cache::reserve(const std::vector<int>& slot_ids, const std::vector<int>& q_lens) {
    for (auto& g : groups) {
        int need = 0;
        for (size_t i = 0; i < slot_ids.size(); ++i) {
            const int slot = slot_ids[i];
            if (!slots.holds(slot)) throw CacheError(format("slot %d is not held", slot));
            need += (int)g->pages_missing(slot, lens[slot], lens[slot] + q_lens[i]).size();
        }
        if (need > g->pages.free_count())
            throw CacheFull(format("the cache is full: %d more pages of %d tokens are needed, %d are free (capacity %d tokens)",
                                   need, PAGE, g->pages.free_count(), g->n_pages * PAGE));
    }
    for (auto& g : groups)
        for (size_t i = 0; i < slot_ids.size(); ++i) g->reserve(slot_ids[i], lens[slot_ids[i]], lens[slot_ids[i]] + q_lens[i]);
}

void Cache::commit(const std::vector<int>& slot_ids, const std::vector<int>& q_lens) {
    for (size_t i = 0; i < slot_ids.size(); ++i) {
        lens[slot_ids[i]] += q_lens[i];
        for (auto& g : groups) g->release_behind(slot_ids[i], lens[slot_ids[i]]);
    }
}

void Cache::table_rows(int g, const std::vector<int>& slot_ids, std::vector<int>& out) const {
    const KVGroup& grp = *groups[g];
    for (int s : slot_ids) out.insert(out.end(), grp.table_row(s), grp.table_row(s) + grp.width);
}

CacheView Cache::view(int entry, bool write, const std::vector<const int*>& step_tables, const int* seq_slots_dev) const {
    CacheView v;
    v.write = write;
    auto g = group_of.find(entry);
    if (g != group_of.end()) {
        const KVGroup& grp = *groups[g->second];
        const int i = grp.index_of(entry);
        v.kind = CacheRequest::KV;
        v.k_pool = (char*)grp.k_pool.get() + (size_t)i * grp.entry_bytes();
        v.v_pool = (char*)grp.v_pool.get() + (size_t)i * grp.entry_bytes();
        v.pool_pages = grp.n_pages;
        v.block_table = step_tables[g->second];
        v.table_width = grp.width;
        v.page_size = PAGE;
        v.window = grp.window;
        v.n_kv_heads = grp.request.n_kv_heads;
        v.head_dim = grp.request.head_dim;
        v.dtype = grp.dtype;
        return v;
    }
    auto s = states.find(entry);
    if (s != states.end()) {
        v.kind = CacheRequest::State;
        std::vector<int64_t> dims{(int64_t)max_slots};
        dims.insert(dims.end(), s->second.shape.begin(), s->second.shape.end());
        v.state = Tensor::make(s->second.memory.get(), s->second.dtype, dims);
        v.seq_slots = seq_slots_dev;
        return v;
    }
    return v;
}

int64_t Cache::held_tokens() const {
    return groups.empty() ? 0 : (int64_t)groups[0]->pages.held_count() * PAGE;
}

size_t Cache::bytes() const {
    size_t b = 0;
    for (const auto& g : groups) b += 2 * g->entry_bytes() * g->entries.size();
    for (const auto& kv : states) b += kv.second.slot_bytes * max_slots;
    return b;
}

}  // namespace friday
