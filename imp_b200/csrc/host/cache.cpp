#include "cache.hpp"

#include <algorithm>
#include <set>

namespace imp {

namespace {
[[noreturn]] void misuse(const std::string& m) { fail(IMP_ERROR_INVALID_ARG, m); }
}

// --------------------------------------------------------------------------------------- pool
IdPool::IdPool(int n) : n_(n), held_((size_t)std::max(n, 0), 0) {
    if (n <= 0) misuse("a pool needs at least one entry");
    free_.reserve((size_t)n);
    for (int i = n - 1; i >= 0; --i) free_.push_back(i);
}

int IdPool::alloc() {
    if (free_.empty()) throw OutOfPages("the pool is empty");
    int id = free_.back();
    free_.pop_back();
    held_[(size_t)id] = 1;
    return id;
}

void IdPool::release(int id) {
    if (id < 0 || id >= n_) misuse("id " + std::to_string(id) + " is outside the pool of " + std::to_string(n_));
    if (!held_[(size_t)id]) misuse("id " + std::to_string(id) + " freed twice");
    held_[(size_t)id] = 0;
    free_.push_back(id);
}

// ------------------------------------------------------------------------------------- groups
PagedGroup::PagedGroup(int g, const CacheSpec& s, int ps, int num_pages, int num_slots, int w)
    : gid(g), spec(s), page_size(ps), pool(num_pages), width(std::max(w, 1)),
      table((size_t)num_slots * (size_t)std::max(w, 1), -1), n_entries((size_t)num_slots, 0) {}

void PagedGroup::ensure_width(int n_logical, int num_slots) {
    if (n_logical <= width) return;
    const int wider = std::max(n_logical, 2 * width);
    std::vector<int32_t> t((size_t)num_slots * wider, -1);
    for (int s = 0; s < num_slots; ++s) std::copy(row(s), row(s) + width, t.begin() + (size_t)s * wider);
    table.swap(t);
    width = wider;
}

int PagedGroup::first_live_page(int length) const {
    if (spec.window <= 0) return 0;
    return std::max(0, length - spec.window + 1) / page_size;
}

int PagedGroup::pages_needed_n(int entries, int cur_len, int new_len) const {
    const int n_logical = (new_len + page_size - 1) / page_size;
    return std::max(0, n_logical - std::max(entries, first_live_page(cur_len)));
}

size_t PagedGroup::layer_bytes(int elem) const {
    return (size_t)2 * pool.size() * spec.num_kv_heads * page_size * spec.head_dim * (size_t)elem;
}

// ------------------------------------------------------------------------------------ manager
CacheManager::CacheManager(const std::vector<CacheSpec>& layer_specs, int page_size, int num_pages, int num_state_slots,
                           int max_pages_per_seq)
    : page_size_(page_size), num_pages_(num_pages), max_pages_per_seq_(max_pages_per_seq > 0 ? max_pages_per_seq : num_pages),
      slots_(std::max(1, num_state_slots)) {
    if (page_size <= 0) misuse("page_size must be positive");
    if (num_pages <= 0) misuse("a page pool needs at least one page");
    std::map<std::string, std::pair<int, int>> by_key;   // key -> (kind, group index)
    paged_.reserve(layer_specs.size());
    for (size_t j = 0; j < layer_specs.size(); ++j) {
        const CacheSpec& s = layer_specs[j];
        LayerCacheRef ref;
        if (s.kind == CacheSpec::None) {
            layer_ref_.push_back(ref);
            continue;
        }
        auto it = by_key.find(s.key());
        if (it == by_key.end()) {
            int g;
            if (s.kind == CacheSpec::Paged) {
                g = (int)paged_.size();
                paged_.emplace_back(g, s, page_size, num_pages, slots_.size(), max_pages_per_seq_);
            } else {
                g = (int)state_.size();
                StateGroup sg;
                sg.gid = g;
                sg.spec = s;
                state_.push_back(std::move(sg));
            }
            it = by_key.emplace(s.key(), std::make_pair((int)s.kind, g)).first;
        }
        ref.kind = s.kind;
        ref.group = it->second.second;
        auto& layers = s.kind == CacheSpec::Paged ? paged_[(size_t)ref.group].layers : state_[(size_t)ref.group].layers;
        ref.index = (int)layers.size();
        layers.push_back((int)j);
        layer_ref_.push_back(ref);
    }
}

const CacheManager::Live& CacheManager::live(int64_t rid) const {
    auto it = live_.find(rid);
    if (it == live_.end()) misuse("unknown request " + std::to_string(rid));
    return it->second;
}
int CacheManager::length(int64_t rid) const { return live(rid).length; }
int CacheManager::slot_of(int64_t rid) const { return live(rid).slot; }

std::vector<int64_t> CacheManager::live_requests() const {
    std::vector<int64_t> out;
    for (const auto& kv : live_) out.push_back(kv.first);
    std::sort(out.begin(), out.end());
    return out;
}

int CacheManager::add_request(int64_t rid) {
    if (live_.count(rid)) misuse("request " + std::to_string(rid) + " is already live");
    int slot;
    try {
        slot = slots_.alloc();
    } catch (const OutOfPages&) {
        throw OutOfPages("no free state slot");
    }
    live_[rid] = Live{slot, 0, 0};
    for (auto& g : paged_) g.n_entries[(size_t)slot] = 0;
    return slot;
}

int CacheManager::pages_needed(int64_t rid, int new_len) const {
    const Live& l = live(rid);
    int need = 0;
    for (const auto& g : paged_) need = std::max(need, g.pages_needed_n(g.n_entries[(size_t)l.slot], l.length, new_len));
    return need;
}

int CacheManager::pages_for_new(int new_len) const {
    int need = 0;
    for (const auto& g : paged_) need = std::max(need, g.pages_needed_n(0, 0, new_len));
    return need;
}

int CacheManager::free_pages() const {
    if (paged_.empty()) return num_pages_;
    int f = paged_[0].pool.n_free();
    for (const auto& g : paged_) f = std::min(f, g.pool.n_free());
    return f;
}

void CacheManager::reserve(int64_t rid, int new_len) {
    auto it = live_.find(rid);
    if (it == live_.end()) misuse("unknown request " + std::to_string(rid));
    Live& l = it->second;
    if (new_len < l.length)
        misuse("request " + std::to_string(rid) + ": cannot reserve " + std::to_string(new_len) + " tokens below its length " +
               std::to_string(l.length));
    for (auto& g : paged_) {
        const int need = g.pages_needed_n(g.n_entries[(size_t)l.slot], l.length, new_len);
        if (need > g.pool.n_free())
            throw OutOfPages("group " + std::to_string(g.gid) + ": request " + std::to_string(rid) + " needs " +
                             std::to_string(need) + " more pages for " + std::to_string(new_len) + " tokens, " +
                             std::to_string(g.pool.n_free()) + " free");
    }
    for (auto& g : paged_) {
        const int n_logical = (new_len + g.page_size - 1) / g.page_size;
        g.ensure_width(n_logical, slots_.size());
        int32_t* row = g.row(l.slot);
        for (int i = std::max(g.n_entries[(size_t)l.slot], g.first_live_page(l.length)); i < n_logical; ++i)
            row[i] = g.pool.alloc();
        if (n_logical > g.n_entries[(size_t)l.slot]) g.n_entries[(size_t)l.slot] = n_logical;
    }
    l.reserved = std::max(l.reserved, new_len);
}

int CacheManager::commit(int64_t rid, int new_len) {
    auto it = live_.find(rid);
    if (it == live_.end()) misuse("unknown request " + std::to_string(rid));
    Live& l = it->second;
    if (new_len > l.reserved)
        misuse("request " + std::to_string(rid) + ": commit of " + std::to_string(new_len) + " tokens beyond the reserved " +
               std::to_string(l.reserved));
    if (new_len < l.length)
        misuse("request " + std::to_string(rid) + ": length cannot shrink from " + std::to_string(l.length) + " to " +
               std::to_string(new_len));
    const int old_len = l.length;
    l.length = new_len;
    int freed = 0;
    for (auto& g : paged_) {
        if (g.spec.window <= 0) continue;
        int32_t* row = g.row(l.slot);
        const int hi = std::min(g.first_live_page(new_len), g.n_entries[(size_t)l.slot]);
        const int lo = g.first_live_page(old_len);
        for (int i = std::min(lo, hi); i < hi; ++i)
            if (row[i] >= 0) {
                g.pool.release(row[i]);
                row[i] = -1;
                ++freed;
            }
    }
    return freed;
}

void CacheManager::release(int64_t rid) {
    auto it = live_.find(rid);
    if (it == live_.end()) misuse("release of unknown request " + std::to_string(rid) + " (released twice?)");
    const Live l = it->second;
    for (auto& g : paged_) {
        int32_t* row = g.row(l.slot);
        const int n = g.n_entries[(size_t)l.slot];
        for (int i = g.first_live_page(l.length); i < n; ++i)
            if (row[i] >= 0) g.pool.release(row[i]);
        std::fill(row, row + n, -1);
        g.n_entries[(size_t)l.slot] = 0;
    }
    slots_.release(l.slot);
    live_.erase(it);
}

void CacheManager::release_all() {
    for (int64_t rid : live_requests()) release(rid);
}

std::vector<int> CacheManager::block_table(int group, int64_t rid) const {
    const Live& l = live(rid);
    const PagedGroup& g = paged_.at((size_t)group);
    return std::vector<int>(g.row(l.slot), g.row(l.slot) + g.n_entries[(size_t)l.slot]);
}

void CacheManager::check_invariants() const {
    auto broken = [](const std::string& m) { fail(IMP_ERROR_INTERNAL, "cache invariant broken: " + m); };
    for (const auto& g : paged_) {
        std::set<int> seen;
        for (const auto& kv : live_) {
            const int32_t* row = g.row(kv.second.slot);
            for (int i = 0; i < g.n_entries[(size_t)kv.second.slot]; ++i) {
                const int p = row[i];
                if (p < 0) continue;
                const std::string where = "group " + std::to_string(g.gid) + ": page " + std::to_string(p);
                if (p >= g.pool.size()) broken(where + " out of range");
                if (!seen.insert(p).second) broken(where + " held twice");
                if (!g.pool.held(p)) broken(where + " in a table but marked free");
            }
        }
        if ((int)seen.size() + g.pool.n_free() != g.pool.size())
            broken("group " + std::to_string(g.gid) + ": " + std::to_string(g.pool.size() - (int)seen.size() - g.pool.n_free()) +
                   " pages lost");
        std::set<int> fl(g.pool.free_list().begin(), g.pool.free_list().end());
        if (fl.size() != g.pool.free_list().size()) broken("group " + std::to_string(g.gid) + ": a page is on the free list twice");
    }
    std::set<int> slots;
    for (const auto& kv : live_)
        if (!slots.insert(kv.second.slot).second) broken("a state slot is held twice");
    if ((int)slots.size() + slots_.n_free() != slots_.size()) broken("a state slot was lost");
}

Json CacheManager::info_json() const {
    Json j = Json::object();
    j["page_size"] = page_size_;
    j["num_pages"] = num_pages_;
    j["free_pages"] = free_pages();
    j["slots"] = slots_.size();
    j["free_slots"] = slots_.n_free();
    Json pg = Json::array();
    for (const auto& g : paged_) {
        Json o = g.spec.to_json();
        o["layers"] = Json::array_of(g.layers);
        o["free"] = g.pool.n_free();
        Json tables = Json::object();
        for (const auto& kv : live_) {
            const int32_t* row = g.row(kv.second.slot);
            tables[std::to_string(kv.first)] =
                Json::array_of(std::vector<int>(row, row + g.n_entries[(size_t)kv.second.slot]));
        }
        o["tables"] = tables;
        pg.push(o);
    }
    j["paged"] = pg;
    Json sg = Json::array();
    for (const auto& g : state_) {
        Json o = g.spec.to_json();
        o["layers"] = Json::array_of(g.layers);
        sg.push(o);
    }
    j["state"] = sg;
    Json refs = Json::array();
    for (const auto& r : layer_ref_) {
        Json o = Json::object();
        o["kind"] = r.kind == CacheSpec::Paged ? "paged" : r.kind == CacheSpec::State ? "state" : "none";
        o["group"] = r.group;
        o["index"] = r.index;
        refs.push(o);
    }
    j["positions"] = refs;
    Json reqs = Json::object();
    for (const auto& kv : live_) {
        Json o = Json::object();
        o["slot"] = kv.second.slot;
        o["length"] = kv.second.length;
        o["reserved"] = kv.second.reserved;
        reqs[std::to_string(kv.first)] = o;
    }
    j["requests"] = reqs;
    return j;
}

// ------------------------------------------------------------------------------------ storage
void CacheManager::allocate_storage(int dtype) {
    dtype_ = dtype;
    for (auto& g : paged_) g.storage = DeviceBuffer(g.layers.size() * g.layer_bytes((int)elem_size(dtype)), true);
    for (auto& g : state_) {
        g.storage.clear();
        for (const auto& t : g.spec.states) {
            int64_t n = 1;
            for (int64_t d : t.shape) n *= d;
            g.storage.emplace_back(g.layers.size() * (size_t)slots_.size() * (size_t)n * elem_size(t.dtype), true);
        }
    }
}

size_t CacheManager::storage_bytes(int elem) const {
    size_t total = 0;
    for (const auto& g : paged_) total += g.layers.size() * g.layer_bytes(elem);
    return total;
}

void CacheManager::zero_state(int slot, cudaStream_t stream) {
    for (auto& g : state_)
        for (size_t ti = 0; ti < g.spec.states.size(); ++ti) {
            if (!g.storage[ti].data()) continue;
            int64_t n = 1;
            for (int64_t d : g.spec.states[ti].shape) n *= d;
            const size_t per_slot = (size_t)n * elem_size(g.spec.states[ti].dtype);
            for (size_t l = 0; l < g.layers.size(); ++l)
                IMP_CUDA(cudaMemsetAsync((char*)g.storage[ti].data() + (l * (size_t)slots_.size() + (size_t)slot) * per_slot, 0,
                                         per_slot, stream));
        }
}

ImpCacheView CacheManager::layer_view(int position, int dtype) const {
    ImpCacheView v{};
    const LayerCacheRef& ref = layer_ref_.at((size_t)position);
    if (ref.kind == CacheSpec::Paged) {
        const PagedGroup& g = paged_[(size_t)ref.group];
        v.kind = 1;
        const size_t lb = g.layer_bytes((int)elem_size(dtype));
        v.k_pages = g.storage.data() ? (char*)g.storage.data() + (size_t)ref.index * lb : nullptr;
        v.v_pages = g.storage.data() ? (char*)v.k_pages + lb / 2 : nullptr;
        v.num_pages = g.pool.size();
        v.kv_heads = g.spec.num_kv_heads;
        v.page_size = g.page_size;
        v.head_dim = g.spec.head_dim;
        v.window = g.spec.window;
    } else if (ref.kind == CacheSpec::State) {
        const StateGroup& g = state_[(size_t)ref.group];
        v.kind = 2;
        v.n_states = (int)g.spec.states.size();
        for (size_t ti = 0; ti < g.spec.states.size(); ++ti) {
            const auto& t = g.spec.states[ti];
            std::vector<int64_t> shape{slots_.size()};
            shape.insert(shape.end(), t.shape.begin(), t.shape.end());
            if (shape.size() > 4) fail(IMP_ERROR_UNSUPPORTED, "a state tensor has at most three dimensions per slot");
            int64_t n = 1;
            for (int64_t d : shape) n *= d;
            void* base = g.storage.size() > ti && g.storage[ti].data()
                             ? (char*)g.storage[ti].data() + (size_t)ref.index * (size_t)n * elem_size(t.dtype)
                             : nullptr;
            v.states[ti] = tensor_nd(base, t.dtype, shape);
        }
    }
    return v;
}

}  // namespace imp
