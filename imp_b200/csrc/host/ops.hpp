// Tensor-level operations of the host: argument checks, the choice of the matrix kernel by shape,
// and the choice of the attention kernel for a step.  Nothing here computes on the host.
#pragma once

#include "parts.hpp"

namespace imp {

// out[M,N] = x[M,K] w[N,K]^T with 32-bit accumulation.
//   float32 x float32 -> the plain FFMA kernel (never a reduced-precision mode).
//   bfloat16 x bfloat16 -> by rows: the weight-streaming kernel (up to 7), the swap-AB tcgen05 kernel
//   (up to 128, and long contractions at any row count), the persistent tcgen05 kernel (up to 255), CTA
//   pairs (more); shapes the TMA descriptors cannot take go to the small-M kernel or the plain kernel
//   (counted in Runtime::fallback_calls); IMP_B200_GEMM=cublas sends products of more than 16 rows to
//   cuBLASLt, what the reference's engine calls for its T>1 products (src/compute/gemm.cu:303-445).
//   bfloat16 x float32 weight (a tensor the checkpoint stores in 32-bit) -> x is widened, FFMA kernel.
// may_defer: the caller hands the result to add_rmsnorm (or calls summed() on it), so a product the
// tcgen05 kernel splits over K may come back with its parts unsummed, the summing kernel saved.
Branch linear(Runtime& rt, Tensor out, const Tensor& x, const Tensor& w, bool may_defer = false);

// out[M,F] = silu(x Wg^T) * (x Wu^T) with Wg and Wu interleaved in runs of 8 rows.
void linear_swiglu(Runtime& rt, Tensor out, const Tensor& x, const Tensor& w_interleaved);
constexpr int SWIGLU_INTERLEAVE = 8;
// Stack gate[F, d] and up[F, d] as runs of 8 gate rows and their 8 up rows (F a multiple of 8).
Tensor interleave_gate_up(Runtime& rt, WeightStore& store, const Tensor& gate, const Tensor& up);
// Stack matrices along the output dimension (widening to float32 if their types differ).
Tensor cat_rows(Runtime& rt, WeightStore& store, const std::vector<Tensor>& parts);
Tensor to_float32(Runtime& rt, WeightStore& store, const Tensor& t);   // a 32-bit copy of a small weight

void swiglu(Runtime& rt, Tensor out, const Tensor& gate_up, int interleave);
void cast(Runtime& rt, Tensor dst, const Tensor& src);

// The tensor a branch stands for (runs the summing kernel if its parts are still apart).
Tensor summed(Runtime& rt, const Branch& b);
inline Tensor summed(Step& st, const Branch& b) { return summed(*st.rt, b); }

// h (+= branch); out = rmsnorm(h) * (weight + offset).  With `rows`, output row r reads stream row
// rows[r] and h is left untouched.  A branch with unsummed parts is added on the way.
void add_rmsnorm(Runtime& rt, Tensor h, const Branch& branch, const Tensor& weight, Tensor out, float eps, float offset,
                 const int32_t* rows, int n_rows);

void embedding(Runtime& rt, Tensor out, const Tensor& table, const int32_t* ids, int n, float scale);

// ------------------------------------------------------------------------------- attention
struct AttentionGeometry {
    int hq, hkv, dh, window;
    float scale;
};
struct QkNorm {
    const float* q_w = nullptr;   // 32-bit copies of the per-head norm weights, or null
    const float* k_w = nullptr;
    float eps = 1e-6f;
};

// The tilings the attention kernels want of a step (see TilingSpec): every portion in 32-token
// tiles; portions of 64 tokens and more in 128-token tiles; the shorter ones in 32-token tiles.
std::vector<TilingSpec> attention_tilings();

// out[t] = softmax(scale q[t] K^T) V over the cached positions token t may see.  float32: the plain
// kernel (fixed reduction order per token).  bfloat16: the split-key decode kernel when every sequence
// brings one token, else the tiled prefill kernels (tensor-memory kernel for long portions where the
// head and page sizes allow it).  `tiling_ids`: where Step::tiles holds the three tilings above.
void paged_attention(Step& st, Tensor out, const Tensor& q, const AttentionGeometry& g, const LayerCache& cache,
                     const std::vector<int>& tiling_ids);

// The decode step from the raw rows of the q,k,v product: per-head norm and rotation of q and of the
// new key happen inside the attention kernel, which writes the new key and value into their pages.
// Returns false, with nothing done, where that kernel does not apply.
bool decode_attention_fused(Step& st, Tensor out, const Tensor& qkv, const AttentionGeometry& g, const LayerCache& cache,
                            const QkNorm& norm, const Position::Rotary& rot);

// q, k, v = x w_qkv^T with the per-head norm, the rotation and the cache write in the product's
// epilogue (256 rows and more, head sizes 64 / 128).  Returns false, having done nothing, otherwise.
bool linear_qkv_rope(Step& st, Tensor q_out, const Tensor& x, const Tensor& w_qkv, const AttentionGeometry& g,
                     const LayerCache& cache, const QkNorm& norm, const Position::Rotary& rot);

// Per-head norm (optional), rotation (optional) and cache write (optional) on the rows of a q,k,v product.
void qk_norm_rope_kv_write(Step& st, Tensor qkv, const AttentionGeometry& g, const Tensor* q_norm_w, const Tensor* k_norm_w,
                           float eps, const Position::Rotary* rot, const LayerCache* cache);

// Key splits of the decode kernel: a function of the batch size alone (a captured graph must not depend
// on the context length).
int decode_splits(int n_tokens, int n_kv_heads, int group, int page_size, int sm_count, int context = 0);

// Where the per-head-size attention libraries are found: a function that returns the path of the
// library built from `source` ("attention_mma.cu" / "attention_tc.cu") for a head size, or NULL.
typedef const char* (*VariantResolver)(const char* source, int head_dim);
void set_variant_resolver(VariantResolver fn);

}  // namespace imp
