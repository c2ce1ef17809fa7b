// Choice of the attention kernel for a step, and the per-head-size libraries.
//
// float32: always the plain kernel (fixed reduction order per token).
// bfloat16: the kernels of variants/attention_mma.cu, one library per head size: the split-key decode
// kernel when every sequence brings one token, else the tiled prefill kernel (a decode token beside
// prompt portions is a tile of one row).  For head sizes 64 and 128 and page sizes that tile 128 keys
// the portions of 64 tokens and more go to the tensor-memory kernel of variants/attention_tc.cu in
// tiles of 128 tokens instead, and only the short ones to the 32-token kernel
// (IMP_B200_ATTN_PREFILL=mma keeps everything on the latter).
#include <dirent.h>
#include <dlfcn.h>
#include <sys/stat.h>

#include <cmath>
#include <map>
#include <mutex>

#include "kernels.h"
#include "ops.hpp"

namespace imp {

namespace {

using DecodeFn = int (*)(void*, int64_t, const void*, int64_t, const void*, const void*, const int*, int, const int*, const int*,
                         int, int, int, int, int, int, float, int, int, float*, int*, void*);
using DecodeFusedFn = int (*)(void*, int64_t, const void*, int64_t, void*, void*, const int*, int, const int*, const int*, int,
                              int, int, int, int, int, float, int, int, float*, const float*, const float*, float,
                              const float*, const float*, int, int*, void*);
using PrefillFn = int (*)(void*, int64_t, const void*, int64_t, const void*, const void*, const int*, int, const int*,
                          const int*, const int*, const int*, int, int, int, int, int, int, float, int, int*, void*);
using PrefillTcFn = int (*)(void*, int64_t, const void*, int64_t, int, const void*, const void*, const int*, int, const int*,
                            const int*, const int*, const int*, int, int, int, int, int, int, float, int, int*, void*);

struct MmaVariant {
    void* handle = nullptr;
    const char* (*last_error)() = nullptr;
    int64_t (*scratch_floats)(int, int, int) = nullptr;
    DecodeFn decode = nullptr;
    DecodeFusedFn decode_fused = nullptr;
    PrefillFn prefill = nullptr;
};
struct TcVariant {
    void* handle = nullptr;
    const char* (*last_error)() = nullptr;
    int (*supported)(int64_t, int64_t, int) = nullptr;
    PrefillTcFn prefill = nullptr;
};

std::mutex g_mutex;
std::map<int, MmaVariant> g_mma;
std::map<int, TcVariant> g_tc;
VariantResolver g_resolver = nullptr;

// The folder this library was loaded from: variants built beside it are found without a resolver.
std::string own_folder() {
    Dl_info info;
    if (dladdr((void*)&own_folder, &info) && info.dli_fname) {
        std::string p = info.dli_fname;
        size_t slash = p.find_last_of('/');
        return slash == std::string::npos ? "." : p.substr(0, slash);
    }
    return ".";
}

std::string find_variant(const char* source, int head_dim) {
    if (g_resolver) {
        const char* p = g_resolver(source, head_dim);
        if (p && *p) return p;
    }
    std::string stem = source;
    if (stem.size() > 3 && stem.substr(stem.size() - 3) == ".cu") stem.resize(stem.size() - 3);
    const std::string prefix = "libimp_" + stem + "_imp_attn_dh" + std::to_string(head_dim) + "-";
    const std::string dir = env_string("IMP_B200_BUILD_DIR", own_folder());
    std::string best;
    time_t best_time = 0;
    if (DIR* d = opendir(dir.c_str())) {
        while (dirent* e = readdir(d)) {
            const std::string name = e->d_name;
            if (name.compare(0, prefix.size(), prefix) != 0 || name.size() < 3 || name.substr(name.size() - 3) != ".so") continue;
            struct stat st;
            const std::string full = dir + "/" + name;
            if (stat(full.c_str(), &st) == 0 && (best.empty() || st.st_mtime > best_time)) {
                best = full;
                best_time = st.st_mtime;
            }
        }
        closedir(d);
    }
    if (best.empty())
        fail(IMP_ERROR_UNSUPPORTED, "the attention library for head size " + std::to_string(head_dim) + " (" + source +
                                        ") has not been built in " + dir + "; build it with `python -m imp_b200.csrc.build --all`");
    return best;
}

template <typename F> void bind(void* h, const char* name, F& fn, const std::string& path) {
    fn = (F)dlsym(h, name);
    if (!fn) fail(IMP_ERROR_INTERNAL, path + " lacks the entry point " + name + "; rebuild it");
}

MmaVariant& mma_variant(int head_dim) {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_mma.find(head_dim);
    if (it != g_mma.end()) return it->second;
    if (head_dim % 16 || head_dim < 16 || head_dim > 256)
        fail(IMP_ERROR_UNSUPPORTED, "attention kernels exist for head sizes 16...256 in steps of 16, not " + std::to_string(head_dim));
    const std::string path = find_variant("attention_mma.cu", head_dim);
    MmaVariant v;
    v.handle = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!v.handle) fail(IMP_ERROR_INTERNAL, "cannot load " + path + ": " + dlerror());
    int (*dh)() = nullptr;
    bind(v.handle, "imp_attn_head_dim", dh, path);
    if (dh() != head_dim) fail(IMP_ERROR_INTERNAL, path + " was built for another head size");
    bind(v.handle, "imp_last_error", v.last_error, path);
    bind(v.handle, "imp_attn_decode_scratch_floats", v.scratch_floats, path);
    bind(v.handle, "imp_attn_decode", v.decode, path);
    bind(v.handle, "imp_attn_decode_fused", v.decode_fused, path);
    bind(v.handle, "imp_attn_prefill", v.prefill, path);
    return g_mma[head_dim] = v;
}

TcVariant& tc_variant(int head_dim) {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_tc.find(head_dim);
    if (it != g_tc.end()) return it->second;
    const std::string path = find_variant("attention_tc.cu", head_dim);
    TcVariant v;
    v.handle = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!v.handle) fail(IMP_ERROR_INTERNAL, "cannot load " + path + ": " + dlerror());
    int (*dh)() = nullptr;
    bind(v.handle, "imp_attn_tc_head_dim", dh, path);
    if (dh() != head_dim) fail(IMP_ERROR_INTERNAL, path + " was built for another head size");
    bind(v.handle, "imp_last_error", v.last_error, path);
    bind(v.handle, "imp_attn_prefill_tc_supported", v.supported, path);
    bind(v.handle, "imp_attn_prefill_tc", v.prefill, path);
    return g_tc[head_dim] = v;
}

void check_variant(Runtime& rt, int rc, const char* what, const char* (*last_error)()) {
    ++rt.launches;
    if (rc != 0) fail(rc < 0 ? IMP_ERROR_INVALID_ARG : IMP_ERROR_CUDA, std::string(what) + " failed (" + std::to_string(rc) + "): " + last_error());
}

bool tc_prefill_enabled() {
    static int v = -1;
    if (v < 0) {
        const std::string s = env_string("IMP_B200_ATTN_PREFILL", "tcgen05");
        if (s != "tcgen05" && s != "mma") fail(IMP_ERROR_INVALID_ARG, "IMP_B200_ATTN_PREFILL must be 'tcgen05' or 'mma'");
        v = s == "tcgen05" ? 1 : 0;
    }
    return v == 1;
}
bool decode_fused_enabled() {
    static int v = -1;
    if (v < 0) v = env_flag("IMP_B200_ATTN_FUSED", true) ? 1 : 0;
    return v == 1;
}

void need(bool cond, const char* what) {
    if (!cond) fail(IMP_ERROR_INVALID_ARG, what);
}

constexpr int DECODE_MAX_SPLITS = 32;
constexpr int TILE = 32, WIDE_TILE = 128, WIDE_MIN = 64;

}  // namespace

void set_variant_resolver(VariantResolver fn) {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_resolver = fn;
}

// All sequences in tiles of 32 tokens; those with 64 tokens and more in tiles of 128; the others in tiles of 32; and the
// first and the third again without the sequences that bring a single token (those go to the decode kernel when they
// stand at the head of a mixed batch).
std::vector<TilingSpec> attention_tilings() {
    return {TilingSpec{TILE, 0, 0}, TilingSpec{WIDE_TILE, WIDE_MIN, 0}, TilingSpec{TILE, 0, WIDE_MIN},
            TilingSpec{TILE, 2, 0}, TilingSpec{TILE, 2, WIDE_MIN}};
}

// The bulk-copy kernel (page sizes that are multiples of 16) keeps two CTAs resident per SM: with fewer
// (token, kv head) pairs than such slots the keys are split until the slots are full.  With more, the
// split count with the least modelled time is taken.  The model (fitted to whole decode steps at 36 to 112
// sequences and contexts of 1,024 and 4,096 on a B200; it picks the fastest split count at 15 of those 16
// points and loses 1 % at the other): a CTA alone streams about 1/150 of what its 148 SMs can, so a wave of
// CTAs runs at full speed from about one CTA per SM up, and a last wave of fewer runs as slowly as each of
// its CTAs; a CTA's time is its share of the keys (context / splits, in units of 4,096 keys) plus a fixed
// part for its start, its end and the merge: 0.02 unsplit, 0.04 with two splits, 0.05 with more.  So short
// contexts are never split (the fixed part dominates) and long ones are split wherever that fills the last wave.
// `context`: the sequences' typical length (0: 4,096).
constexpr double B200_SMS = 148.0;   // the part the model's constant was fitted on

int decode_splits(int n_tokens, int n_kv_heads, int group, int page_size, int sm_count, int context) {
    static const int forced = [] { const std::string e = env_string("IMP_B200_DECODE_SPLITS", ""); return e.empty() ? 0 : std::atoi(e.c_str()); }();
    if (forced > 0) return std::min(forced, DECODE_MAX_SPLITS);    // for measurements
    const int sms = sm_count > 0 ? sm_count : std::max(1, imp_device_sm_count());
    const int base = std::max(1, n_tokens * n_kv_heads * ((group + 15) / 16));
    if (page_size % 16) return std::max(1, std::min(DECODE_MAX_SPLITS, sms * 3 / base));
    const int slots = 2 * sms;
    if (base <= slots) {
        // the largest power of two that keeps every CTA resident at once (measured: 16 splits beat 18 at two
        // sequences, 8 beat 9 at four, although the latter fill more slots)
        int s = std::max(1, std::min(DECODE_MAX_SPLITS, slots / base));
        // a split of fewer than 128 keys (two stages of the ring) is all start and end: short contexts get fewer
        if (context > 0) s = std::max(1, std::min(s, context / 128));
        int p = 1;
        while (p * 2 <= s) p *= 2;
        return p;
    }
    const double saturating = sms * (150.0 / B200_SMS);   // scaled with the SMs the device has
    const double keys = (context > 0 ? context : 4096) / 4096.0;
    int best = 1;
    double best_t = 0;
    for (int s = 1; s <= 8; ++s) {
        const int ctas = base * s, full = ctas / slots, tail = ctas % slots;
        double t = full * slots / saturating + (tail ? tail / std::min(saturating, (double)tail) : 0.0);
        t *= (s == 1 ? 0.02 : s == 2 ? 0.04 : 0.05) + keys / s;
        if (s == 1 || t < best_t) {
            best = s;
            best_t = t;
        }
    }
    return best;
}

static void check_cache(const LayerCache& c, const AttentionGeometry& g) {
    need(c.view.kind == 1 && c.view.k_pages && c.view.v_pages && c.view.block_table, "attention needs a paged cache with a block table");
    need(c.view.kv_heads == g.hkv && c.view.head_dim == g.dh, "the cache's geometry is not the attention's");
}

static void decode_attention(Step& st, Tensor out, const Tensor& q, const AttentionGeometry& g, const LayerCache& cache) {
    Runtime& rt = *st.rt;
    MmaVariant& lib = mma_variant(g.dh);
    const ImpCacheView& c = cache.view;
    const int T = (int)rows(q);
    const int n_splits = decode_splits(T, g.hkv, g.hq / g.hkv, c.page_size, rt.sm_count, st.context);
    const int64_t n_floats = lib.scratch_floats(T, g.hq, n_splits);
    float* scratch = n_floats ? (float*)rt.arena->alloc((size_t)n_floats * 4) : nullptr;
    check_variant(rt,
                  lib.decode(out.data, out.stride0, q.data, q.stride0, c.k_pages, c.v_pages, c.block_table, c.bt_stride,
                             st.view.seq_of_token, st.view.positions, T, st.B(), g.hq, g.hkv, c.page_size, c.num_pages, g.scale,
                             g.window, n_splits, scratch, rt.status, rt.stream),
                  "attention decode", lib.last_error);
}

bool decode_attention_fused(Step& st, Tensor out, const Tensor& qkv, const AttentionGeometry& g, const LayerCache& cache,
                            const QkNorm& norm, const Position::Rotary& rot) {
    Runtime& rt = *st.rt;
    const ImpCacheView& c = cache.view;
    if (!decode_fused_enabled() || g.dh % 64 || c.page_size % 16) return false;
    check_cache(cache, g);
    need(qkv.dtype == BF16 && out.dtype == BF16 && cols(qkv) >= (int64_t)(g.hq + 2 * g.hkv) * g.dh && rot.rot_dim == g.dh,
         "fused decode attention: bfloat16 rows of q | k | v and a rotation over the whole head");
    MmaVariant& lib = mma_variant(g.dh);
    const int T = (int)rows(qkv);
    const int n_splits = decode_splits(T, g.hkv, g.hq / g.hkv, c.page_size, rt.sm_count, st.context);
    const int64_t n_floats = lib.scratch_floats(T, g.hq, n_splits);
    float* scratch = n_floats ? (float*)rt.arena->alloc((size_t)n_floats * 4) : nullptr;
    const int rc = lib.decode_fused(out.data, out.stride0, qkv.data, qkv.stride0, c.k_pages, c.v_pages, c.block_table, c.bt_stride,
                                    st.view.seq_of_token, st.view.positions, T, st.B(), g.hq, g.hkv, c.page_size, c.num_pages,
                                    g.scale, g.window, n_splits, scratch, norm.q_w, norm.k_w, norm.eps, rot.cos, rot.sin,
                                    rot.max_pos, rt.status, rt.stream);
    if (rc == -2) return false;
    check_variant(rt, rc, "attention decode (fused)", lib.last_error);
    return true;
}

static void prefill_attention(Step& st, Tensor out, const Tensor& q, const AttentionGeometry& g, const LayerCache& cache,
                              const Tiles& tiles) {
    Runtime& rt = *st.rt;
    MmaVariant& lib = mma_variant(g.dh);
    const ImpCacheView& c = cache.view;
    check_variant(rt,
                  lib.prefill(out.data, out.stride0, q.data, q.stride0, c.k_pages, c.v_pages, c.block_table, c.bt_stride,
                              st.view.seq_of_token, st.view.positions, tiles.tok0, tiles.rows, tiles.count, st.B(), g.hq, g.hkv,
                              c.page_size, c.num_pages, g.scale, g.window, rt.status, rt.stream),
                  "attention prefill", lib.last_error);
}

static bool prefill_tc_supported(const Tensor& q, const Tensor& out, const AttentionGeometry& g, const ImpCacheView& c) {
    if (!tc_prefill_enabled() || (g.dh != 64 && g.dh != 128) || q.dtype != BF16) return false;
    if ((uintptr_t)q.data % 16 || (uintptr_t)out.data % 16 || (uintptr_t)c.k_pages % 16) return false;
    return tc_variant(g.dh).supported(q.stride0, out.stride0, c.page_size) != 0;
}

void paged_attention(Step& st, Tensor out, const Tensor& q, const AttentionGeometry& g, const LayerCache& cache,
                     const std::vector<int>& tiling_ids) {
    Runtime& rt = *st.rt;
    check_cache(cache, g);
    const ImpCacheView& c = cache.view;
    need(rows(out) == rows(q) && out.dtype == q.dtype, "attention: out and q must agree");
    if (rt.is_f32()) {
        ++rt.launches;
        check_launch(imp_paged_attention_generic(out.data, out.stride0, q.data, q.stride0, c.k_pages, c.v_pages, c.block_table,
                                                 c.bt_stride, st.view.seq_of_token, st.view.positions, (int)rows(q), st.B(), g.hq,
                                                 g.hkv, g.dh, c.page_size, c.num_pages, g.scale, g.window, q.dtype, rt.status,
                                                 rt.stream),
                     "paged_attention_generic");
        return;
    }
    need(q.dtype == BF16, "attention: bfloat16 or float32");
    if (st.decode_only()) {
        decode_attention(st, out, q, g, cache);
        return;
    }
    need(tiling_ids.size() == 5, "attention: the step holds no tilings for this mixer");
    // Sequences that decode beside the portions of prompts: as a tile of one row each, a CTA walks all their keys alone
    // (8 decoding sequences at context 4,096 beside a 512-token portion: 19.2 ms a step against 4.0 + 9.1 for the two
    // alone).  The scheduler puts them first, one token each, so they are the batch's first rows: the split-key decode
    // kernel takes those rows, the tiled kernels the rest.  (IMP_B200_ATTN_MIXED_DECODE=0: tiles of one row as before.)
    static const bool split_singles = env_flag("IMP_B200_ATTN_MIXED_DECODE", true);
    int n_single = 0;
    while (n_single < st.B() && st.q_lens[(size_t)n_single] == 1) ++n_single;
    bool singles = split_singles && n_single > 0;
    for (int i = n_single; singles && i < st.B(); ++i)
        if (st.q_lens[(size_t)i] == 1) singles = false;      // single tokens further on: no leading block, the tiled kernels take all
    if (singles) decode_attention(st, first_rows(out, n_single), first_rows(q, n_single), g, cache);
    const Tiles& all = st.tiles.at((size_t)tiling_ids[singles ? 3 : 0]);
    const Tiles& wide = st.tiles.at((size_t)tiling_ids[1]);
    const Tiles& rest = st.tiles.at((size_t)tiling_ids[singles ? 4 : 2]);
    if (wide.count && prefill_tc_supported(q, out, g, c)) {
        TcVariant& lib = tc_variant(g.dh);
        check_variant(rt,
                      lib.prefill(out.data, out.stride0, q.data, q.stride0, (int)rows(q), c.k_pages, c.v_pages, c.block_table,
                                  c.bt_stride, st.view.seq_of_token, st.view.positions, wide.tok0, wide.rows, wide.count, st.B(),
                                  g.hq, g.hkv, c.page_size, c.num_pages, g.scale, g.window, rt.status, rt.stream),
                      "attention prefill (tcgen05)", lib.last_error);
        if (rest.count) prefill_attention(st, out, q, g, cache, rest);
        return;
    }
    if (all.count) prefill_attention(st, out, q, g, cache, all);
}

bool linear_qkv_rope(Step& st, Tensor q_out, const Tensor& x, const Tensor& w, const AttentionGeometry& g, const LayerCache& cache,
                     const QkNorm& norm, const Position::Rotary& rot) {
    Runtime& rt = *st.rt;
    static int lib = -1;
    if (lib < 0) lib = env_string("IMP_B200_GEMM", "tcgen05") == "cublas" ? 1 : 0;
    if (lib || x.dtype != BF16 || w.dtype != BF16) return false;
    const int T = (int)rows(x);
    if (T < 256 || (g.dh != 64 && g.dh != 128) || rot.rot_dim != g.dh) return false;
    check_cache(cache, g);
    const ImpCacheView& c = cache.view;
    need(rows(w) == (int64_t)(g.hq + 2 * g.hkv) * g.dh && cols(w) == cols(x) && q_out.dtype == BF16 && rows(q_out) == T &&
             cols(q_out) == (int64_t)g.hq * g.dh,
         "linear_qkv_rope: shapes do not agree");
    const int rc = imp_gemm_bf16_tc_qkv_rope(x.data, x.stride0, w.data, w.stride0, T, (int)cols(x), g.hq, g.hkv, g.dh, norm.q_w,
                                             norm.k_w, norm.eps, rot.cos, rot.sin, rot.max_pos, st.view.positions,
                                             st.view.seq_of_token, c.block_table, c.bt_stride, st.B(), q_out.data, q_out.stride0,
                                             c.k_pages, c.v_pages, c.page_size, c.num_pages, rt.status, rt.stream);
    if (rc == -2) return false;
    ++rt.launches;
    check_launch(rc, "gemm_bf16_tc_qkv_rope");
    return true;
}

void qk_norm_rope_kv_write(Step& st, Tensor qkv, const AttentionGeometry& g, const Tensor* q_norm_w, const Tensor* k_norm_w,
                           float eps, const Position::Rotary* rot, const LayerCache* cache) {
    Runtime& rt = *st.rt;
    need(cols(qkv) >= (int64_t)(g.hq + 2 * g.hkv) * g.dh, "qk_norm_rope_kv_write: rows must hold q | k | v");
    const int w_dtype = q_norm_w ? q_norm_w->dtype : F32;
    if (q_norm_w) need(k_norm_w && numel(*q_norm_w) == g.dh && numel(*k_norm_w) == g.dh && k_norm_w->dtype == w_dtype, "q/k norm weights must be [head_dim] of one type");
    const ImpCacheView* c = cache ? &cache->view : nullptr;
    if (c) check_cache(*cache, g);
    ++rt.launches;
    check_launch(imp_qk_norm_rope_kv_write(qkv.data, qkv.stride0, (int)rows(qkv), g.hq, g.hkv, g.dh, q_norm_w ? q_norm_w->data : nullptr,
                                           k_norm_w ? k_norm_w->data : nullptr, eps, 0.f, w_dtype, rot ? rot->cos : nullptr,
                                           rot ? rot->sin : nullptr, rot ? rot->rot_dim : 0, rot ? rot->max_pos : 0, st.view.positions,
                                           c ? st.view.seq_of_token : nullptr, c ? c->block_table : nullptr, c ? c->bt_stride : 0,
                                           c ? st.B() : 0, c ? c->k_pages : nullptr, c ? c->v_pages : nullptr, c ? c->page_size : 0,
                                           c ? c->num_pages : 0, qkv.dtype, rt.status, rt.stream),
                 "qk_norm_rope_kv_write");
}

}  // namespace imp
