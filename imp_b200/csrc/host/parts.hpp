// Interfaces of the parts a model is put together from, and the registry of part kinds.
//
// A part is built from (params, tensors, runtime): `params` are its sizes and constants (from the
// plan, never from a model class), `tensors` its weights by local name, the runtime gives the
// precision, the stream, the status word and the workspace.  No part knows which model it is in.
//
//   norm          add_norm(step, h, branch, rows) -> normalised activations; h is the 32-bit
//                 residual stream, `branch` (if any) is added into it first; with `rows` only
//                 those rows are produced and h is left as it is.
//   position      rotary_tables() for encodings the fused kernels know; apply(q, k) otherwise.
//   mixer         cache_spec(params) (class level) -> paged keys/values | fixed-size state | none;
//                 tilings(): how it wants prompt portions cut into tiles, filled by the step
//                 function; forward(step, x, cache) -> branch output [T, hidden].
//   feed_forward  forward(step, x) -> branch output [T, hidden].
//   block         part_slots(params) (class level): the parts it arranges, by slot name;
//                 forward(step, h, pending, cache) -> the branch it leaves pending.
//   embedding     forward(step) -> [T, hidden] float32 stream.
//   head          forward(step, x_rows) -> [R, vocab] float32 logits.
//
// Unsummed branch outputs.  A matrix product of few rows is cut over the contraction and leaves
// partial results that someone has to add (Branch::parts).  A norm that can add them while it reads
// the branch says so through takes_split_sum(); a mixer or feed-forward whose `defer_out` has been
// set by whoever arranges it may then return such a branch.  Both default to false, so a part that
// knows nothing of this never meets one.
#pragma once

#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "core.hpp"
#include "plan.hpp"

namespace imp {

// ------------------------------------------------------------------------------ cache needs
struct StateTensorSpec {
    std::string name;
    std::vector<int64_t> shape;   // per slot
    int dtype = F32;
};

// What a mixer asks of the cache.  Paged: keys and values per token, [kv_heads, head_dim] each;
// window == 0 keeps every token, window == W keeps what a query at position p may still see
// (positions > p - W).  State: named tensors of fixed size per request, zero at a request's start.
struct CacheSpec {
    enum Kind { None = 0, Paged = 1, State = 2 } kind = None;
    int num_kv_heads = 0, head_dim = 0, window = 0;
    std::vector<StateTensorSpec> states;
    std::string key() const;      // equal keys share a cache group
    Json to_json() const;
    static CacheSpec from_json(const Json& j);
    static CacheSpec paged(int kv_heads, int head_dim, int window) {
        CacheSpec s;
        s.kind = Paged;
        s.num_kv_heads = kv_heads;
        s.head_dim = head_dim;
        s.window = window;
        return s;
    }
};

// How a mixer wants the new tokens of each sequence cut: runs of up to `tile` consecutive tokens
// of one sequence, over the sequences whose portion holds min_len <= n < max_len tokens
// (max_len == 0: no upper bound).  The step function fills what the model's mixers declared.
struct TilingSpec {
    int tile = 32, min_len = 0, max_len = 0;
    bool operator==(const TilingSpec& o) const { return tile == o.tile && min_len == o.min_len && max_len == o.max_len; }
};
struct Tiles {
    const int32_t* tok0 = nullptr;   // device: first token of each tile (index into the batch)
    const int32_t* rows = nullptr;   // device: tokens in each tile
    int count = 0;
};

// ---------------------------------------------------------------------------------- one step
struct Step {
    Runtime* rt = nullptr;
    ImpBatchView view{};                       // device arrays and sizes, as parts outside the library see them
    std::vector<int> q_lens, starts, slots;    // host copies, per sequence
    std::vector<int64_t> rids;
    std::vector<const int32_t*> block_tables;  // per paged cache group: [n_seqs, bt_stride]
    int bt_stride = 0;
    std::vector<Tiles> tiles;                  // per tiling the model declared (empty in decode-only steps)
    struct Diagnostics* diag = nullptr;        // stage timers / statistics when a debugging switch is set
    int layer = -1;                            // index of the layer that is running (for stage names)
    int context = 0;                           // the sequences' mean length after this step, rounded to a power of two: what
                                               // launch choices may depend on (a decode graph is kept per batch size and context)
    int T() const { return view.n_tokens; }
    int B() const { return view.n_seqs; }
    int R() const { return view.n_rows; }
    bool decode_only() const { return view.decode_only != 0; }
};

// What a mixer gets of the cache for one run position.
struct LayerCache {
    ImpCacheView view{};
    int group = 0;     // index of the cache group among the groups of its kind
    bool paged() const { return view.kind == 1; }
};

// A named point of the forward pass: with IMP_B200_PROFILE a timer stops here, with
// IMP_B200_DEBUG_FORWARD the tensor's statistics are printed.  Does nothing otherwise.
void stage(Step& st, const char* name, const Tensor& t);
struct Branch;
void stage(Step& st, const char* name, const Branch& b);   // an unsummed branch stops the timer and has no statistics

// A branch output: nothing, a tensor, or the unsummed parts of one ([n_splits, M, N] float32 whose
// sum in split order, rounded to `t`'s type, is the value that belongs into `t`).
struct Branch {
    Tensor t{};
    float* parts = nullptr;
    int n_splits = 0;
    bool empty() const { return t.data == nullptr; }
    bool split() const { return parts != nullptr; }
    static Branch of(const Tensor& t) { Branch b; b.t = t; return b; }
};

// ------------------------------------------------------------------------------------- parts
struct Part {
    virtual ~Part() = default;
    virtual bool graph_safe() const { return true; }   // its launches depend on the batch's sizes only
    virtual const char* category() const = 0;
    // Uniform entry for callers outside the library (imp_part_forward).
    virtual void call(Step& st, ImpCall& c) = 0;
};

struct Norm : Part {
    const char* category() const override { return "norm"; }
    virtual bool takes_split_sum() const { return false; }
    virtual Tensor add_norm(Step& st, Tensor h, const Branch& branch, const int32_t* rows = nullptr, int n_rows = 0) = 0;
    void call(Step& st, ImpCall& c) override;
};

struct Position : Part {
    const char* category() const override { return "position"; }
    struct Rotary { const float* cos; const float* sin; int rot_dim; int max_pos; };
    virtual bool rotary(Rotary* out) const { (void)out; return false; }
    virtual void apply(Step& st, Tensor q, Tensor k);   // q [T, Hq, Dh], k [T, Hkv, Dh] in place
    void call(Step& st, ImpCall& c) override;
};

struct Mixer : Part {
    const char* category() const override { return "mixer"; }
    bool defer_out = false;
    std::vector<int> tiling_ids;                         // index into Step::tiles of each declared tiling
    virtual std::vector<TilingSpec> tilings() const { return {}; }
    virtual Branch forward(Step& st, Tensor x, LayerCache* cache) = 0;
    void call(Step& st, ImpCall& c) override;
};

struct FeedForward : Part {
    const char* category() const override { return "feed_forward"; }
    bool defer_out = false;
    virtual Branch forward(Step& st, Tensor x) = 0;
    void call(Step& st, ImpCall& c) override;
};

struct Block : Part {
    const char* category() const override { return "block"; }
    bool defer_pending = false;                          // set by the model: the pending it returns may be unsummed
    virtual bool takes_split_sum() const { return false; }   // the pending it is given may be unsummed
    virtual Mixer* mixer() const { return nullptr; }     // the part that owns this layer's cache, if any
    virtual std::vector<Part*> parts() const = 0;
    virtual Branch forward(Step& st, Tensor h, const Branch& pending, LayerCache* cache) = 0;
    void call(Step& st, ImpCall& c) override;
};

struct Embedding : Part {
    const char* category() const override { return "embedding"; }
    virtual Tensor forward(Step& st) = 0;
    void call(Step& st, ImpCall& c) override;
};

struct Head : Part {
    const char* category() const override { return "head"; }
    virtual Tensor forward(Step& st, Tensor x) = 0;
    void call(Step& st, ImpCall& c) override;
};

// ---------------------------------------------------------------------------------- registry
// Device tensors of a model: the loader puts checkpoint tensors here; a part that rearranges its
// weights (concatenated q,k,v; interleaved gate and up) allocates the new tensor and releases the old.
class WeightStore {
public:
    Tensor alloc(int dtype, const std::vector<int64_t>& shape);
    void release(const void* data);
    size_t bytes() const { return bytes_; }

private:
    std::map<const void*, DeviceBuffer> buffers_;
    size_t bytes_ = 0;
};

class PartFactory;

struct Slot {
    std::string name, category;
};

struct BuildArgs {
    std::string category, kind;
    Json params;
    std::vector<std::pair<std::string, Tensor>> tensors;   // this part's weights on the device, by local name
    std::vector<std::pair<std::string, Part*>> parts;      // a block's built parts, by slot
    Runtime* rt = nullptr;
    WeightStore* store = nullptr;
    PartFactory* factory = nullptr;
    bool has(const std::string& name) const;
    Tensor tensor(const std::string& name) const;          // throws when absent
    Part* part(const std::string& slot) const;             // nullptr when absent
    void drop(const std::string& name);                    // release a tensor the part does not keep
};

struct PartClass {
    std::function<TensorSpecs(const Json& params)> tensor_specs;      // may be empty: no tensors
    std::function<CacheSpec(const Json& params)> cache_spec;          // mixers
    std::function<std::vector<Slot>(const Json& params)> part_slots;  // blocks
    std::function<Part*(BuildArgs&)> create;
};

extern const char* const PART_CATEGORIES[7];
void register_part_class(const std::string& category, const std::string& kind, PartClass cls, bool replace = false);
void unregister_part_class(const std::string& category, const std::string& kind);
const PartClass& part_class(const std::string& category, const std::string& kind);   // throws, listing known kinds
std::vector<std::string> known_parts(const std::string& category);
void ensure_builtin_parts();   // registers the library's own kinds once

// Builds parts and owns them.  Parts without tensors are shared between equal specs.
class PartFactory {
public:
    PartFactory(Runtime* rt, WeightStore* store) : rt_(rt), store_(store) {}
    Part* build(const std::string& category, const PartSpec& spec,
                std::vector<std::pair<std::string, Tensor>> tensors,
                std::vector<std::pair<std::string, Part*>> parts = {});
    Part* shared(const std::string& category, const Json& spec_json);   // {"kind", "params"}
    Runtime* rt() const { return rt_; }

private:
    Runtime* rt_;
    WeightStore* store_;
    std::vector<std::unique_ptr<Part>> owned_;
    std::map<std::string, Part*> shared_;
};

template <typename T> T* part_cast(Part* p, const char* what) {
    T* t = dynamic_cast<T*>(p);
    if (!t) fail(IMP_ERROR_INVALID_ARG, std::string("a part of category '") + (p ? p->category() : "none") +
                                            "' stands where " + what + " is expected");
    return t;
}

}  // namespace imp
