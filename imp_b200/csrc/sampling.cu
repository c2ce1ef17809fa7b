// Token selection from 32-bit logits: argmax, repetition/frequency/presence
// penalties, and temperature sampling with min-p, top-k and top-p filters.
//
// Reference counterparts (src/compute/sampling.cu): argmax with the lowest
// index winning ties (:29-84), penalties (:700-736: divide positive / multiply
// negative logits of seen tokens by the repetition penalty, subtract
// frequency*count and presence), min-p as a cut at max + log(min_p) on the raw
// logits (:767-810), and topk_topp_sample_kernel (:253-557): softmax of
// logits/T over the whole vocabulary, the k most probable, the shortest prefix
// of them whose probability reaches top_p, renormalise, one uniform draw.
// Differences: one block per row for any number of rows at once; k is not
// capped at 128 (the kept tokens are found by a radix selection over ordered
// keys into a short list of up to 1024 candidates, where the cuts and the draw
// are made; wider sets take a bitwise search over the keys, 32 passes per filter); ties at a cut are kept; the uniform number is an input
// (the reference re-seeds an LCG with the same seed on every call, :541-543,
// which draws the same number at every step); the draw walks the kept tokens in
// index order.  Every reduction has a fixed order, so a row's result does not
// depend on the other rows.
#include "common.cuh"

constexpr int SAMPLE_BLOCK = 1024;
constexpr int SAMPLE_CAND = 1024;    // tokens the sampler's short list holds (one per thread)

__device__ __forceinline__ unsigned ordered_key(float f) {
    const unsigned b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ int block_sum_int(int v, int* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int t = lane < nwarp ? scratch[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// ------------------------------------------------------------------- argmax
__device__ __forceinline__ void argmax_row(const float* __restrict__ x, int V, float* s_val, int* s_idx,
                                           float& best_v, int& best_i) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = x[i];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) { s_val[warp] = bv; s_idx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < nwarp ? s_val[lane] : -INFINITY;
        bi = lane < nwarp ? s_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { s_val[32] = bv; s_idx[32] = bi; }
    }
    __syncthreads();
    best_v = s_val[32];
    best_i = s_idx[32];
}

__global__ void __launch_bounds__(SAMPLE_BLOCK) argmax_kernel(const float* __restrict__ logits, int64_t ld, int V,
                                                             int* __restrict__ out) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float s_val[33];
    __shared__ int s_idx[33];
    float bv;
    int bi;
    argmax_row(logits + (int64_t)blockIdx.x * ld, V, s_val, s_idx, bv, bi);
    if (threadIdx.x == 0) out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
}

// Two-stage form for large vocabularies: ARGMAX_CHUNKS blocks per row each reduce a contiguous
// slice, a second kernel reduces the per-slice winners (lowest index on ties in both stages).
constexpr int ARGMAX_CHUNKS = 32;

__global__ void __launch_bounds__(256) argmax_partial_kernel(const float* __restrict__ logits, int64_t ld, int V,
                                                             float* __restrict__ pval, int* __restrict__ pidx) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float s_val[33];
    __shared__ int s_idx[33];
    const int r = blockIdx.y, c = blockIdx.x;
    const int per = (V + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
    const int lo = c * per, hi = min(V, lo + per);
    const float* x = logits + (int64_t)r * ld;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = x[i];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (lane == 0) { s_val[warp] = bv; s_idx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < nwarp ? s_val[lane] : -INFINITY;
        bi = lane < nwarp ? s_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { pval[r * ARGMAX_CHUNKS + c] = bv; pidx[r * ARGMAX_CHUNKS + c] = bi; }
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ pval, const int* __restrict__ pidx, int* __restrict__ out) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x, lane = threadIdx.x;
    float bv = lane < ARGMAX_CHUNKS ? pval[r * ARGMAX_CHUNKS + lane] : -INFINITY;
    int bi = lane < ARGMAX_CHUNKS ? pidx[r * ARGMAX_CHUNKS + lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out[r] = (bi == 0x7fffffff) ? 0 : bi;
}

// Words of scratch (4 bytes each) imp_argmax wants for `n_rows` rows; without scratch it runs one block per row.
IMP_API int imp_argmax_scratch_words(int n_rows) { return 2 * ARGMAX_CHUNKS * n_rows; }

IMP_API int imp_argmax(const float* logits, int64_t ld, int n_rows, int V, int* out, void* scratch, void* stream) {
    if (n_rows == 0) return 0;
    IMP_CHECK_ARG(logits && out && V > 0 && ld >= V, "imp_argmax: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    if (scratch && V >= 8192 && n_rows <= 65535) {
        float* pval = (float*)scratch;
        int* pidx = (int*)scratch + (size_t)ARGMAX_CHUNKS * n_rows;
        imp_launch(argmax_partial_kernel, dim3(ARGMAX_CHUNKS, n_rows), dim3(256), 0, s, logits, ld, V, pval, pidx);
        imp_launch(argmax_final_kernel, dim3(n_rows), dim3(32), 0, s, (const float*)pval, (const int*)pidx, out);
    } else {
        argmax_kernel<<<n_rows, SAMPLE_BLOCK, 0, s>>>(logits, ld, V, out);
    }
    IMP_RETURN_LAUNCH();
}

// ---------------------------------------------------------------- penalties
// counts: [n_rows, V] int32 scratch, zeroed here.  history: tokens of all rows back to back,
// row r owning history[hist_start[r] .. hist_start[r+1]).
__global__ void count_history_kernel(int* __restrict__ counts, const int* __restrict__ history,
                                     const int* __restrict__ hist_start, int V) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.y;
    const int b = hist_start[r], e = hist_start[r + 1];
    for (int i = b + blockIdx.x * blockDim.x + threadIdx.x; i < e; i += gridDim.x * blockDim.x) {
        const int tok = history[i];
        if (tok >= 0 && tok < V) atomicAdd(&counts[(int64_t)r * V + tok], 1);
    }
}

__global__ void apply_penalties_kernel(float* __restrict__ logits, int64_t ld, const int* __restrict__ counts,
                                       int V, const float* __restrict__ rep, const float* __restrict__ freq,
                                       const float* __restrict__ pres) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= V) return;
    const int c = counts[(int64_t)r * V + i];
    if (c == 0) return;
    float x = logits[(int64_t)r * ld + i];
    const float rp = rep[r];
    if (rp != 1.f) x = x > 0.f ? x / rp : x * rp;
    x -= freq[r] * (float)c;
    x -= pres[r];
    logits[(int64_t)r * ld + i] = x;
}

IMP_API int imp_apply_penalties(float* logits, int64_t ld, int n_rows, int V, const int* history,
                                const int* hist_start, int max_hist, const float* rep, const float* freq,
                                const float* pres, int* counts_scratch, void* stream) {
    if (n_rows == 0 || max_hist == 0) return 0;
    IMP_CHECK_ARG(logits && history && hist_start && rep && freq && pres && counts_scratch,
                  "imp_apply_penalties: null pointer");
    IMP_CHECK_ARG(n_rows <= 65535, "imp_apply_penalties: too many rows");
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(counts_scratch, 0, (size_t)n_rows * V * sizeof(int), s);
    if (e != cudaSuccess) { imp_set_error("imp_apply_penalties: %s", cudaGetErrorString(e)); return (int)e; }
    const int gx = (max_hist + 255) / 256;
    count_history_kernel<<<dim3(gx, n_rows), 256, 0, s>>>(counts_scratch, history, hist_start, V);
    apply_penalties_kernel<<<dim3((V + 255) / 256, n_rows), 256, 0, s>>>(logits, ld, counts_scratch, V, rep, freq, pres);
    IMP_RETURN_LAUNCH();
}

// ------------------------------------------------------------------- the draw
// One token among those that `keep` accepts, with weights `weight`, from the
// uniform number u: the first kept index, in index order, whose running weight
// exceeds u * total.  Thread t owns the contiguous range [t*chunk, (t+1)*chunk);
// thread 0 turns the per-thread sums into exclusive prefixes in a fixed order.
// Returns -1 when nothing is kept.  All threads of the block must call it.
template <class Keep, class Weight>
__device__ __forceinline__ int draw_in_index_order(int V, float u, Keep keep, Weight weight, float* part,
                                                   float* scratch, int* s_pick) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int chunk = (V + nthr - 1) / nthr;
    const int lo = min(V, tid * chunk), hi = min(V, lo + chunk);
    float mine = 0.f;
    for (int i = lo; i < hi; ++i)
        if (keep(i)) mine += weight(i);
    __syncthreads();
    part[tid] = mine;
    if (tid == 0) *s_pick = -1;
    __syncthreads();
    if (tid == 0) {
        float run = 0.f;
        for (int t = 0; t < nthr; ++t) {
            const float v = part[t];
            part[t] = run;  // exclusive prefix
            run += v;
        }
        scratch[0] = run;
    }
    __syncthreads();
    const float total = scratch[0];
    const float target = u * total;
    const float before = part[tid];
    if (mine > 0.f && before <= target && target < before + mine) {
        float run = before;
        int pick = -1, last = -1;
        for (int i = lo; i < hi; ++i) {
            if (keep(i)) {
                run += weight(i);
                last = i;
                if (run > target) { pick = i; break; }
            }
        }
        *s_pick = pick >= 0 ? pick : last;
    }
    __syncthreads();
    return *s_pick;
}

// ------------------------------------------------------------------- sample
// Per row r: temperature[r] <= 0 or top_k[r] == 1 -> argmax.  Otherwise:
//   keep i with logit_i >= max + log(min_p)           (min_p > 0)
//   x_i = logit_i / T, e_i = exp(x_i - max x) over kept i, Z = sum e_i
//   keep the top_k largest x_i (ties with the k-th kept)  (0 < top_k < V)
//   keep the most probable tokens until their e-mass reaches top_p * Z (ties kept)  (0 < top_p < 1)
//   draw: target = u * mass(kept); the first kept i, in index order, whose running mass exceeds target.
__global__ void __launch_bounds__(SAMPLE_BLOCK) sample_kernel(
    const float* __restrict__ logits, int64_t ld, int V, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
    const float* __restrict__ uniform, int* __restrict__ out) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float s_val[33];
    __shared__ int s_idx[33];
    __shared__ float scratch[33];
    __shared__ int iscratch[33];
    __shared__ float part[SAMPLE_BLOCK];
    __shared__ int s_pick;

    const int r = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (int64_t)r * ld;
    float max_logit;
    int arg;
    argmax_row(x, V, s_val, s_idx, max_logit, arg);
    const float T = temperature[r];
    const int k = top_k[r];
    if (T <= 0.f || k == 1 || arg == 0x7fffffff) {
        if (tid == 0) out[r] = (arg == 0x7fffffff) ? 0 : arg;
        return;
    }
    const float inv_T = 1.f / T;
    const float mp = min_p[r];
    const float floor_logit = mp > 0.f ? max_logit + logf(mp) : -INFINITY;
    const float xmax = max_logit * inv_T;
#define KEPT0(i) (x[i] >= floor_logit)
#define EVAL(i) expf(x[i] * inv_T - xmax)

    float z = 0.f;
    for (int i = tid; i < V; i += SAMPLE_BLOCK)
        if (KEPT0(i)) z += EVAL(i);
    z = block_sum(z, scratch);

    // ---- short list: when the filters leave at most SAMPLE_CAND tokens, find them with a radix selection
    // (four passes over the row instead of 32 per filter), bring them into shared memory in index order and
    // do the nucleus cut and the draw there.  Same kept set and same draw rule as the passes below, which
    // remain for the cases the short list cannot hold (no top-k and a nucleus wider than SAMPLE_CAND tokens).
    {
        const float tp0 = top_p[r];
        const bool k_on = k > 0 && k < V, p_on = tp0 > 0.f && tp0 < 1.f;
        const int want_n = k_on ? k : SAMPLE_CAND;
        if ((k_on || p_on) && want_n <= SAMPLE_CAND) {
            __shared__ int hist[256];
            __shared__ int s_sel[3];                  // chosen bin, tokens still wanted, candidates so far
            __shared__ int c_idx[SAMPLE_CAND], c_tmp[SAMPLE_CAND];
            __shared__ float c_e[SAMPLE_CAND], c_x[SAMPLE_CAND];
            // the want_n-th largest ordered key among the tokens min-p keeps, 8 bits at a time
            unsigned prefix = 0u;
            int remaining = want_n;
            bool all_kept = false;                    // fewer than want_n tokens in all: everything is a candidate
            for (int shift = 24; shift >= 0; shift -= 8) {
                for (int b = tid; b < 256; b += SAMPLE_BLOCK) hist[b] = 0;
                __syncthreads();
                const unsigned hi_mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
                for (int i0 = 0; i0 < V; i0 += SAMPLE_BLOCK) {
                    const int i = i0 + tid;
                    int bin = -1;
                    if (i < V && KEPT0(i)) {
                        const unsigned key = ordered_key(x[i]);
                        if ((key & hi_mask) == prefix) bin = (int)((key >> shift) & 255u);
                    }
                    // lanes of a warp that hit the same bin add up first: one atomic per bin and warp
                    const unsigned peers = __match_any_sync(0xffffffffu, bin);
                    if (bin >= 0 && (int)(__ffs(peers) - 1) == (tid & 31)) atomicAdd(&hist[bin], __popc(peers));
                }
                __syncthreads();
                if (tid == 0) {
                    int acc = 0, b = 255;
                    for (; b >= 0; --b) {
                        if (acc + hist[b] >= remaining) break;
                        acc += hist[b];
                    }
                    s_sel[0] = b;                     // -1: not enough tokens under this prefix
                    s_sel[1] = remaining - acc;
                    // everything above the chosen bin plus the whole bin fits the list: no need to look closer,
                    // the exact cut is made among the candidates
                    if (b >= 0 && (want_n - remaining) + acc + hist[b] <= SAMPLE_CAND) s_sel[0] = b | 0x100;
                }
                __syncthreads();
                if (s_sel[0] < 0) { all_kept = true; break; }
                prefix |= (unsigned)(s_sel[0] & 0xff) << shift;
                remaining = s_sel[1];
                const bool stop = (s_sel[0] & 0x100) != 0;
                __syncthreads();
                if (stop) break;
            }
            const unsigned tau_k = all_kept ? 0u : prefix;   // lower edge of the last bin looked at
            // candidates: min-p kept and key >= tau_k; more than the list holds (ties) -> the general passes
            if (tid == 0) s_sel[2] = 0;
            __syncthreads();
            for (int i = tid; i < V; i += SAMPLE_BLOCK)
                if (KEPT0(i) && ordered_key(x[i]) >= tau_k) {
                    const int slot = atomicAdd(&s_sel[2], 1);
                    if (slot < SAMPLE_CAND) c_tmp[slot] = i;
                }
            __syncthreads();
            const int c = s_sel[2];
            if (c >= 1 && c <= SAMPLE_CAND) {
                // into index order (the order they arrived in varies from run to run; the sums below must not)
                if (tid < c) {
                    const int me = c_tmp[tid];
                    int rank = 0;
                    for (int j = 0; j < c; ++j) rank += c_tmp[j] < me;
                    c_idx[rank] = me;
                }
                __syncthreads();
                if (tid < c) {
                    c_x[tid] = x[c_idx[tid]];
                    c_e[tid] = EVAL(c_idx[tid]);
                }
                __syncthreads();
                bool keep = tid < c;
                if (k_on && tid < c) {                 // the list may hold more than k: keep those with fewer than k above them
                    int greater = 0;
                    const float mine = c_x[tid];
                    for (int j = 0; j < c; ++j) greater += c_x[j] > mine;
                    keep = greater < k;
                }
                bool usable = true;
                if (p_on) {
                    const float want = tp0 * z;
                    if (!k_on) {
                        // without top-k the list must contain the whole nucleus: its mass has to reach the target
                        if (tid == 0) {
                            float m = 0.f;
                            for (int j = 0; j < c; ++j) m += c_e[j];
                            scratch[0] = m;
                        }
                        __syncthreads();
                        usable = scratch[0] >= want || all_kept;
                        __syncthreads();
                    }
                    if (usable && tid < c) {
                        float above = 0.f;            // mass of the strictly more probable candidates
                        const float mine = c_x[tid];
                        for (int j = 0; j < c; ++j)
                            if (c_x[j] > mine) above += c_e[j];
                        keep = keep && above < want;
                    }
                }
                if (usable) {
                    part[tid] = keep ? c_e[tid] : 0.f;
                    if (tid < c) c_tmp[tid] = keep ? 1 : 0;
                    if (tid == 0) s_pick = -1;
                    __syncthreads();
                    if (tid == 0) {
                        float run = 0.f;
                        for (int j = 0; j < c; ++j) {
                            const float v = part[j];
                            part[j] = run;            // exclusive prefix in index order
                            run += v;
                        }
                        scratch[0] = run;
                    }
                    __syncthreads();
                    const float target = uniform[r] * scratch[0];
                    if (keep && c_e[tid] > 0.f && part[tid] <= target && target < part[tid] + c_e[tid]) s_pick = c_idx[tid];
                    __syncthreads();
                    if (tid == 0) {
                        int pick = s_pick;
                        if (pick < 0) {               // rounding left no owner: the last kept candidate, else the most probable
                            for (int j = c - 1; j >= 0 && pick < 0; --j)
                                if (c_tmp[j]) pick = c_idx[j];
                            if (pick < 0) pick = arg;
                        }
                        out[r] = pick;
                    }
                    return;
                }
            }
            __syncthreads();
        }
    }

    unsigned tau = 0u;  // keep keys >= tau
    if (k > 0 && k < V) {
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = tau | (1u << bit);
            int c = 0;
            for (int i = tid; i < V; i += SAMPLE_BLOCK)
                if (KEPT0(i) && ordered_key(x[i]) >= cand) ++c;
            c = block_sum_int(c, iscratch);
            if (c >= k) tau = cand;
        }
    }
    const float tp = top_p[r];
    if (tp > 0.f && tp < 1.f) {
        const float want = tp * z;
        unsigned tau_p = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = tau_p | (1u << bit);
            float mass = 0.f;
            for (int i = tid; i < V; i += SAMPLE_BLOCK)
                if (KEPT0(i) && ordered_key(x[i]) >= cand) mass += EVAL(i);
            mass = block_sum(mass, scratch);
            if (mass >= want) tau_p = cand;
        }
        if (tau_p > tau) tau = tau_p;
    }

    const int pick = draw_in_index_order(V, uniform[r], [&](int i) { return KEPT0(i) && ordered_key(x[i]) >= tau; },
                                         [&](int i) { return EVAL(i); }, part, scratch, &s_pick);
    if (tid == 0) out[r] = pick >= 0 ? pick : arg;  // rounding left no owner: the most probable token
#undef KEPT0
#undef EVAL
}

IMP_API int imp_sample(const float* logits, int64_t ld, int n_rows, int V, const float* temperature,
                       const int* top_k, const float* top_p, const float* min_p, const float* uniform, int* out,
                       void* stream) {
    if (n_rows == 0) return 0;
    IMP_CHECK_ARG(logits && temperature && top_k && top_p && min_p && uniform && out && V > 0 && ld >= V,
                  "imp_sample: bad argument");
    sample_kernel<<<n_rows, SAMPLE_BLOCK, 0, (cudaStream_t)stream>>>(logits, ld, V, temperature, top_k, top_p, min_p,
                                                                    uniform, out);
    IMP_RETURN_LAUNCH();
}

// ------------------------------------------------------------------- DRY
// logits[rows[i]][tokens[i]] -= values[i]: the sparse form of the "don't repeat
// yourself" penalty, whose (token, value) pairs the host finds by matching the
// end of the request's tokens against their earlier occurrences
// (src/compute/sampling.cu:811-915 does the same split between host and device).
__global__ void sparse_subtract_kernel(float* __restrict__ logits, int64_t ld, int V, const int* __restrict__ rows,
                                       const int* __restrict__ tokens, const float* __restrict__ values, int n,
                                       int n_rows) {
    pdl_wait();
    pdl_launch_dependents();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int r = rows[i], t = tokens[i];
    if (r < 0 || r >= n_rows || t < 0 || t >= V) return;
    logits[(int64_t)r * ld + t] -= values[i];  // the host lists a (row, token) pair once
}

IMP_API int imp_sparse_subtract(float* logits, int64_t ld, int n_rows, int V, const int* rows, const int* tokens,
                                const float* values, int n, void* stream) {
    if (n == 0 || n_rows == 0) return 0;
    IMP_CHECK_ARG(logits && rows && tokens && values && n > 0 && V > 0 && ld >= V, "imp_sparse_subtract: bad argument");
    sparse_subtract_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(logits, ld, V, rows, tokens, values, n,
                                                                           n_rows);
    IMP_RETURN_LAUNCH();
}

// ------------------------------------------------------------------- typical-p
// Locally typical filtering on the raw logits (src/compute/sampling.cu:917-1064;
// order after min-p as in src/graph/executor.cu:92-97).  Over the tokens that
// min-p keeps: p = softmax(logits), H = -sum p log2 p, dev_i = |-log2 p_i - H|;
// the tokens of smallest deviation are kept until their mass reaches typical_p
// (ties at the cut kept), every other logit becomes -inf.  The reference finds
// the cut with a 256-bucket histogram of deviations and so keeps up to one bucket
// more; here the cut is exact (a bitwise search over the deviation's bits).
// Rows with typical_p outside (0, 1) are left untouched.
__global__ void __launch_bounds__(SAMPLE_BLOCK) typical_filter_kernel(float* __restrict__ logits, int64_t ld, int V,
                                                                      const float* __restrict__ typical_p,
                                                                      const float* __restrict__ min_p) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float s_val[33];
    __shared__ int s_idx[33];
    __shared__ float scratch[33];
    const int r = blockIdx.x, tid = threadIdx.x;
    const float tp = typical_p[r];
    if (!(tp > 0.f && tp < 1.f)) return;
    float* x = logits + (int64_t)r * ld;
    float max_logit;
    int arg;
    argmax_row(x, V, s_val, s_idx, max_logit, arg);
    if (arg == 0x7fffffff) return;
    const float mp = min_p[r];
    const float floor_logit = mp > 0.f ? max_logit + logf(mp) : -INFINITY;
#define TYP_KEPT(i) (x[i] >= floor_logit && x[i] > -INFINITY)
    float z = 0.f;
    for (int i = tid; i < V; i += SAMPLE_BLOCK)
        if (TYP_KEPT(i)) z += expf(x[i] - max_logit);
    z = block_sum(z, scratch);
    const float lse = max_logit + logf(z);
    const float inv_z = 1.f / z;
    constexpr float LOG2E = 1.4426950408889634f;
    float h = 0.f;
    for (int i = tid; i < V; i += SAMPLE_BLOCK)
        if (TYP_KEPT(i)) h += expf(x[i] - max_logit) * inv_z * ((lse - x[i]) * LOG2E);
    h = block_sum(h, scratch);
#define DEV_KEY(i) __float_as_uint(fabsf((lse - x[i]) * LOG2E - h))
    // The largest T with mass{key < T} < typical_p is the smallest key whose closed set reaches it.
    unsigned cut = 0u;
    for (int bit = 31; bit >= 0; --bit) {
        const unsigned cand = cut | (1u << bit);
        float mass = 0.f;
        for (int i = tid; i < V; i += SAMPLE_BLOCK)
            if (TYP_KEPT(i) && DEV_KEY(i) < cand) mass += expf(x[i] - max_logit) * inv_z;
        mass = block_sum(mass, scratch);
        if (mass < tp) cut = cand;
    }
    for (int i = tid; i < V; i += SAMPLE_BLOCK)
        if (!(TYP_KEPT(i) && DEV_KEY(i) <= cut)) x[i] = -INFINITY;
#undef DEV_KEY
#undef TYP_KEPT
}

IMP_API int imp_typical_filter(float* logits, int64_t ld, int n_rows, int V, const float* typical_p,
                               const float* min_p, void* stream) {
    if (n_rows == 0) return 0;
    IMP_CHECK_ARG(logits && typical_p && min_p && V > 0 && ld >= V, "imp_typical_filter: bad argument");
    typical_filter_kernel<<<n_rows, SAMPLE_BLOCK, 0, (cudaStream_t)stream>>>(logits, ld, V, typical_p, min_p);
    IMP_RETURN_LAUNCH();
}

// ------------------------------------------------------------------- Mirostat v2
// src/compute/sampling.cu:1067-1236: with p = softmax(logits / T), keep the
// tokens whose surprise -log2 p_i is at most mu (all of them if none passes),
// draw one, and report its surprise under the unfiltered distribution; the host
// then moves mu by -eta * (surprise - tau).  Rows with active[r] == 0 are left
// alone.  The draw uses the given uniform number and walks in index order.
__global__ void __launch_bounds__(SAMPLE_BLOCK) mirostat_kernel(
    const float* __restrict__ logits, int64_t ld, int V, const int* __restrict__ active,
    const float* __restrict__ temperature, const float* __restrict__ mu, const float* __restrict__ uniform,
    int* __restrict__ out, float* __restrict__ surprise) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float s_val[33];
    __shared__ int s_idx[33];
    __shared__ float scratch[33];
    __shared__ float part[SAMPLE_BLOCK];
    __shared__ int s_pick;
    const int r = blockIdx.x, tid = threadIdx.x;
    if (!active[r]) return;
    const float* x = logits + (int64_t)r * ld;
    float max_logit;
    int arg;
    argmax_row(x, V, s_val, s_idx, max_logit, arg);
    if (arg == 0x7fffffff) {
        if (tid == 0) { out[r] = 0; surprise[r] = 0.f; }
        return;
    }
    const float T = temperature[r] > 0.f ? temperature[r] : 1.f;
    const float inv_T = 1.f / T;
    float z = 0.f;
    for (int i = tid; i < V; i += SAMPLE_BLOCK) z += expf((x[i] - max_logit) * inv_T);
    z = block_sum(z, scratch);
    float threshold = max_logit + T * (logf(z) - mu[r] * 0.6931471805599453f);
    float zf = 0.f;
    for (int i = tid; i < V; i += SAMPLE_BLOCK)
        if (x[i] >= threshold) zf += expf((x[i] - max_logit) * inv_T);
    zf = block_sum(zf, scratch);
    if (!(zf > 0.f)) threshold = -INFINITY;
    const int pick = draw_in_index_order(V, uniform[r], [&](int i) { return x[i] >= threshold; },
                                         [&](int i) { return expf((x[i] - max_logit) * inv_T); }, part, scratch,
                                         &s_pick);
    if (tid == 0) {
        const int chosen = pick >= 0 ? pick : arg;
        const float p = expf((x[chosen] - max_logit) * inv_T) / z;
        out[r] = chosen;
        surprise[r] = -log2f(fmaxf(p, 1e-30f));
    }
}

IMP_API int imp_sample_mirostat(const float* logits, int64_t ld, int n_rows, int V, const int* active,
                                const float* temperature, const float* mu, const float* uniform, int* out,
                                float* surprise, void* stream) {
    if (n_rows == 0) return 0;
    IMP_CHECK_ARG(logits && active && temperature && mu && uniform && out && surprise && V > 0 && ld >= V,
                  "imp_sample_mirostat: bad argument");
    mirostat_kernel<<<n_rows, SAMPLE_BLOCK, 0, (cudaStream_t)stream>>>(logits, ld, V, active, temperature, mu, uniform,
                                                                      out, surprise);
    IMP_RETURN_LAUNCH();
}
