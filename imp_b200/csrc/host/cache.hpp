// The cache manager: pages of keys and values with a block table per request, one pool per group
// of layers with the same needs, and slots of fixed-size state.
//
// What the reference has (src/memory/): one pool for all attention layers with a LIFO free list that
// hands out page 0 first (kv_cache.cu:74-79, 97-116), a map from sequence id to its page list with
// all-or-nothing allocation (kv_cache_manager.cpp:37-69), `free_sequence` at the end of a request,
// and a pool of fixed-size state indexed by `request id % max_sequences` (ssm_state.h:16-49), which
// can collide.  What differs here:
//   * layers are grouped by what they need of the cache (all keys; a window of them; fixed-size
//     state); each paged group has a pool and block tables of its own, shared by the layers of the
//     group (one page id addresses the same slot in each of them);
//   * a windowed group gives a page back as soon as every later query is past it;
//   * state slots come from a free list, so two live requests never share one;
//   * nothing is evicted behind a request's back: `reserve` either gets all the pages or fails with
//     OutOfPages and leaves everything as it was; what to do then is the scheduler's decision.
// The bookkeeping is host-only and needs no GPU; `allocate_storage` makes the device memory.
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "parts.hpp"

namespace imp {

// Not enough free pages (or state slots) for what was asked.
struct OutOfPages : Error {
    explicit OutOfPages(const std::string& m) : Error(IMP_ERROR_OUT_OF_MEMORY, m) {}
};

// Free list over `n` ids.  LIFO; id 0 comes out first.
class IdPool {
public:
    explicit IdPool(int n);
    int size() const { return n_; }
    int n_free() const { return (int)free_.size(); }
    int alloc();                  // throws OutOfPages
    void release(int id);         // throws on ids outside the pool or freed twice
    bool held(int id) const { return held_[(size_t)id] != 0; }
    const std::vector<int>& free_list() const { return free_; }

private:
    int n_;
    std::vector<int> free_;
    std::vector<uint8_t> held_;
};

// Layers that share page ids: same kv heads, head size and window.  Block tables live in one int32
// matrix [slots, width] (-1 = no page), so that a batch's table is one gather by slot.  Invariant: for
// a live request of committed length n, every entry in [first_live_page(n), n_entries) holds a page
// and every entry outside holds -1.
struct PagedGroup {
    int gid = 0;
    CacheSpec spec;
    std::vector<int> layers;            // run positions that own storage in this group
    int page_size = 0;
    IdPool pool;
    int width = 0;                      // columns of the table
    std::vector<int32_t> table;         // [slots, width]
    std::vector<int> n_entries;         // logical pages per slot (held or given back)
    DeviceBuffer storage;               // [layers, 2, pages, kv_heads, page_size, head_dim]
    PagedGroup(int gid, const CacheSpec& spec, int page_size, int num_pages, int num_slots, int width);
    int32_t* row(int slot) { return table.data() + (size_t)slot * width; }
    const int32_t* row(int slot) const { return table.data() + (size_t)slot * width; }
    void ensure_width(int n_logical, int num_slots);
    int first_live_page(int length) const;
    int pages_needed_n(int n_entries, int cur_len, int new_len) const;
    size_t layer_bytes(int elem) const;   // bytes of one layer's keys and values
};

// Layers with the same fixed-size state; slot ids are shared by all state groups.
struct StateGroup {
    int gid = 0;
    CacheSpec spec;
    std::vector<int> layers;
    std::vector<DeviceBuffer> storage;    // per state tensor: [layers, slots, *shape]
};

struct LayerCacheRef {
    int kind = 0;     // CacheSpec::Kind
    int group = -1;
    int index = 0;    // the layer's index inside its group's storage
};

class CacheManager {
public:
    // layer_specs[j]: what run position j asks for (None for positions without a cache of their own).
    CacheManager(const std::vector<CacheSpec>& layer_specs, int page_size, int num_pages, int num_state_slots,
                 int max_pages_per_seq = 0);

    int page_size() const { return page_size_; }
    int num_pages() const { return num_pages_; }
    std::vector<PagedGroup>& paged() { return paged_; }
    const std::vector<PagedGroup>& paged() const { return paged_; }
    std::vector<StateGroup>& state() { return state_; }
    const std::vector<LayerCacheRef>& layer_ref() const { return layer_ref_; }
    IdPool& slots() { return slots_; }
    const IdPool& slots() const { return slots_; }

    bool has(int64_t rid) const { return live_.count(rid) != 0; }
    int length(int64_t rid) const;
    int slot_of(int64_t rid) const;
    std::vector<int64_t> live_requests() const;

    int add_request(int64_t rid);                    // gives it a state slot; returns the slot
    int pages_needed(int64_t rid, int new_len) const;   // most pages any group lacks for rid to grow to new_len
    int pages_for_new(int new_len) const;            // the same for a request that is not live yet
    int free_pages() const;                          // free pages of the scarcest group
    void reserve(int64_t rid, int new_len);          // all or nothing; throws OutOfPages
    int commit(int64_t rid, int new_len);            // records the length; returns how many pages a window gave back
    void release(int64_t rid);                       // pages of every group and the slot go back
    void release_all();
    std::vector<int> block_table(int group, int64_t rid) const;

    void check_invariants() const;                   // throws Error(IMP_ERROR_INTERNAL) naming the fault
    Json info_json() const;

    // Device storage (zero-filled, as the reference's pool: kv_cache.cu:53).
    void allocate_storage(int dtype);
    size_t storage_bytes(int elem) const;            // of the paged groups
    void zero_state(int slot, cudaStream_t stream);
    // The cache view of run position `position` (block table left empty: it belongs to a batch).
    ImpCacheView layer_view(int position, int dtype) const;

private:
    struct Live {
        int slot, length, reserved;
    };
    const Live& live(int64_t rid) const;
    int page_size_, num_pages_, max_pages_per_seq_;
    std::vector<PagedGroup> paged_;
    std::vector<StateGroup> state_;
    std::vector<LayerCacheRef> layer_ref_;
    IdPool slots_;
    std::unordered_map<int64_t, Live> live_;
    int dtype_ = BF16;
};

}  // namespace imp
