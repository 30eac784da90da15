// Softmax attention over the paged cache with the options of windowed designs: grouped
// key/value heads, key and value heads of different sizes, a sliding window that may keep a
// sequence's first tokens visible, a bias that grows with the distance of query and key, a
// root-mean-square norm over the whole query (and key) projection, a query temperature that
// grows with the position, a norm per head before or after the rotation, biases, rotary
// positions on a head's first coordinates, a learned sink per head in the softmax's
// denominator, and a gate per head or per value coordinate on the result.  Every option is a
// parameter; a mixer that leaves one out passes 0 / null.
//
//   visible(i, j) = j <= i and (i - j < window or j < keep_first)         (window 0: all j <= i)
//   score(i, j)   = (q_i . k_j) * scale - slope_h * (i - j)
//   w(i, j)       = exp(score(i, j)) / (sum_j' exp(score(i, j')) + exp(sink_h))
//   o_i           = (sum_j w(i, j) v_j) * sigmoid(gate_i,h or gate_i,h,c) * out_scale
//
// Cache: one pool per layer, one row per (token, key/value head): [k (dim) | v (vdim)], so a
// key and its value come with one page look-up and their sizes need not be equal.
//
// wattn_prepare: a CTA per token.  Reads the fused projection's 32-bit result; norms q and k
// over all heads at once (if they have norm weights), multiplies q by its temperature, turns
// the first rot_dims coordinates of every head (rotate-half layout, angles in 32-bit), leaves q
// in 32-bit beside the step and writes the token's cache rows (unless the layer reads the cache
// of another layer).
//
// wattn_tile: a CTA takes up to tq consecutive token rows and ONE key/value head; the query
// heads that share it ride together.  Keys go in blocks of 32 ABSOLUTE positions, first the
// blocks of kept first tokens that lie before the window's, then the window's; a warp owns up
// to WT_PPW (query, head) pairs, a lane one key of the block for the scores and vdim / 32 value
// coordinates for the sums.  Which keys meet in which partial sum depends on absolute positions
// only: a query's result does not depend on the tile, the portion or the batch it falls in.
//
// wattn: a CTA per (token, query head) for sizes the tiled kernel does not take.
// All arithmetic is 32-bit.
#include "common.cuh"

namespace {
constexpr int WA_THREADS = 128;
constexpr int WA_SEG = 256;         // keys scored at a time
constexpr int WA_MAX_V = 4;         // value coordinates a thread owns at most (vdim <= 512)
constexpr int NO_WINDOW = 1 << 30;

__device__ __forceinline__ float wa_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// A learned sink joins a finished softmax: the denominator l (taken against the maximum m)
// becomes l * f + exp(sink - max(m, sink)) and the weighted sums are multiplied by f.
__device__ __forceinline__ void wa_join_sink(float sink, float m, float& l, float& f) {
    const float top = fmaxf(m, sink);
    f = (m == -INFINITY) ? 0.0f : expf(m - top);
    l = l * f + expf(sink - top);
}
// The gate of head h (gate_per 1: one number a head; else one per value coordinate jj).
__device__ __forceinline__ float wa_gate(const float* gate, size_t row, int h, int jj, int gate_per) {
    if (gate == nullptr) return 1.0f;
    return wa_sigmoid(gate[row + (size_t)h * gate_per + (gate_per > 1 ? jj : 0)]);
}

// One projection (q or k) of a token: norm over all n numbers, a factor, rotation per head.
// Element i of head hd goes to dst(hd)[i].
template <typename D, typename F>
__device__ __forceinline__ void wa_project(const float* __restrict__ src, int n_heads, int dim,
                                           int rot_dims, const float* __restrict__ norm_w,
                                           float eps, float factor, float pos,
                                           const float* __restrict__ freq,
                                           const float* __restrict__ freq_lo, float* scratch, F dst) {
    float inv = factor;
    if (norm_w != nullptr) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < n_heads * dim; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
        ss = prb_block_sum(ss, scratch);
        inv = factor / sqrtf(ss / (float)(n_heads * dim) + eps);
    }
    const int half = rot_dims / 2;
    const int units = half + (dim - rot_dims);       // per head: pairs, then coordinates that stay
    for (int u = threadIdx.x; u < n_heads * units; u += blockDim.x) {
        const int hd = u / units, w = u - hd * units;
        const float* s = src + hd * dim;
        const float* nw = norm_w ? norm_w + hd * dim : nullptr;
        D* d = dst(hd);
        if (w < half) {
            float sn, cs;
            prb_sincos_angle(pos, freq[w], &sn, &cs, freq_lo ? freq_lo[w] : 0.0f);
            const float a = s[w] * inv * (nw ? nw[w] : 1.0f);
            const float b = s[w + half] * inv * (nw ? nw[w + half] : 1.0f);
            d[w] = prb_from_float<D>(a * cs - b * sn);
            d[w + half] = prb_from_float<D>(b * cs + a * sn);
        } else {
            const int i = w - half + rot_dims;
            d[i] = prb_from_float<D>(s[i] * inv * (nw ? nw[i] : 1.0f));
        }
    }
}

// The same with a norm per HEAD (norm_mode 2: before the rotation, with a weight of `dim`
// numbers that all heads share; 3: after the rotation, without a weight) and a bias that joins
// the projection first.  A warp takes a head: its sum of squares is a warp's, whatever the
// number of heads.
template <typename D, typename F>
__device__ __forceinline__ void wa_project_heads(const float* __restrict__ src,
                                                 const float* __restrict__ bias, int n_heads,
                                                 int dim, int rot_dims, int norm_mode,
                                                 const float* __restrict__ norm_w, float eps,
                                                 float factor, float pos,
                                                 const float* __restrict__ freq,
                                                 const float* __restrict__ freq_lo, F dst) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int half = rot_dims / 2;
    const int units = half + (dim - rot_dims);
    for (int hd = warp; hd < n_heads; hd += nwarps) {
        const float* s = src + hd * dim;
        const float* bb = bias ? bias + hd * dim : nullptr;
        float inv = 1.0f;
        if (norm_mode == 2) {
            float ss = 0.0f;
            for (int i = lane; i < dim; i += 32) {
                const float v = s[i] + (bb ? bb[i] : 0.0f);
                ss = fmaf(v, v, ss);
            }
            inv = 1.0f / sqrtf(prb_warp_sum(ss) / (float)dim + eps);
        } else if (norm_mode == 3) {
            float ss = 0.0f;
            for (int u = lane; u < units; u += 32) {
                if (u < half) {
                    float sn, cs;
                    prb_sincos_angle(pos, freq[u], &sn, &cs, freq_lo ? freq_lo[u] : 0.0f);
                    const float a = s[u] + (bb ? bb[u] : 0.0f);
                    const float b = s[u + half] + (bb ? bb[u + half] : 0.0f);
                    const float ra = a * cs - b * sn, rb = b * cs + a * sn;
                    ss = fmaf(ra, ra, fmaf(rb, rb, ss));
                } else {
                    const int i = u - half + rot_dims;
                    const float v = s[i] + (bb ? bb[i] : 0.0f);
                    ss = fmaf(v, v, ss);
                }
            }
            inv = 1.0f / sqrtf(prb_warp_sum(ss) / (float)dim + eps);
        }
        const float pre = norm_mode == 2 ? inv : 1.0f;
        const float post = (norm_mode == 3 ? inv : 1.0f) * factor;
        const float* nw = norm_mode == 2 ? norm_w : nullptr;
        D* d = dst(hd);
        for (int u = lane; u < units; u += 32) {
            if (u < half) {
                float sn, cs;
                prb_sincos_angle(pos, freq[u], &sn, &cs, freq_lo ? freq_lo[u] : 0.0f);
                const float a = (s[u] + (bb ? bb[u] : 0.0f)) * pre * (nw ? nw[u] : 1.0f);
                const float b = (s[u + half] + (bb ? bb[u + half] : 0.0f)) * pre * (nw ? nw[u + half] : 1.0f);
                d[u] = prb_from_float<D>((a * cs - b * sn) * post);
                d[u + half] = prb_from_float<D>((b * cs + a * sn) * post);
            } else {
                const int i = u - half + rot_dims;
                d[i] = prb_from_float<D>((s[i] + (bb ? bb[i] : 0.0f)) * pre * (nw ? nw[i] : 1.0f) * post);
            }
        }
    }
}

template <typename C>
__global__ void wattn_prepare_kernel(float* __restrict__ q_out, C* __restrict__ cache,
                                     const float* __restrict__ proj, long ld, int q_col, int k_col,
                                     int v_col, const float* __restrict__ q_norm,
                                     const float* __restrict__ k_norm, const int* __restrict__ slots,
                                     const int* __restrict__ positions,
                                     const float* __restrict__ freq, int n_tokens, int heads,
                                     int kv_heads, int dim, int vdim, int rot_dims, float eps,
                                     float temp_coef, int temp_every, int page_size, int num_pages,
                                     int norm_mode, const float* __restrict__ q_bias,
                                     const float* __restrict__ k_bias,
                                     const float* __restrict__ v_bias,
                                     const float* __restrict__ freq_lo, int* status) {
    __shared__ float scratch[32];
    prb_grid_launch_dependents();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const float* row = proj + (size_t)t * ld;
    const int p = positions[t];
    const float pos = (float)p;
    float temp = 1.0f;
    if (temp_every > 0) temp = 1.0f + temp_coef * logf((float)((p + 1) / temp_every) + 1.0f);
    float* qo = q_out + (size_t)t * heads * dim;
    const bool per_head = norm_mode >= 2 || q_bias != nullptr || k_bias != nullptr;
    if (per_head)
        wa_project_heads<float>(row + q_col, q_bias, heads, dim, rot_dims, norm_mode, q_norm, eps,
                                temp, pos, freq, freq_lo, [&](int hd) { return qo + hd * dim; });
    else
        wa_project<float>(row + q_col, heads, dim, rot_dims, q_norm, eps, temp, pos, freq, freq_lo, scratch,
                          [&](int hd) { return qo + hd * dim; });
    if (slots == nullptr) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int page = slot / page_size, off = slot - page * page_size;
    if (page >= num_pages) {
        if (threadIdx.x == 0) prb_set_status(status, PRB_S_SLOT_RANGE, t, slot, num_pages);
        return;
    }
    const int rowlen = dim + vdim;
    C* base = cache + (((size_t)page * kv_heads) * page_size + off) * rowlen;
    const size_t head_step = (size_t)page_size * rowlen;
    if (per_head)
        wa_project_heads<C>(row + k_col, k_bias, kv_heads, dim, rot_dims, norm_mode, k_norm, eps,
                            1.0f, pos, freq, freq_lo, [&](int hd) { return base + hd * head_step; });
    else
        wa_project<C>(row + k_col, kv_heads, dim, rot_dims, k_norm, eps, 1.0f, pos, freq, freq_lo, scratch,
                      [&](int hd) { return base + hd * head_step; });
    for (int u = threadIdx.x; u < kv_heads * vdim; u += blockDim.x) {
        const int g = u / vdim, j = u - g * vdim;
        base[g * head_step + dim + j] =
            prb_from_float<C>(row[v_col + u] + (v_bias ? v_bias[u] : 0.0f));
    }
}

// ------------------------------------------------------------- a CTA per (token, head)
template <typename C, typename O>
__global__ void __launch_bounds__(WA_THREADS)
wattn_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ q,
             const C* __restrict__ cache, const int* __restrict__ block_table,
             const int* __restrict__ seq_of_token, const int* __restrict__ positions,
             const float* __restrict__ gate, long gate_ld, const float* __restrict__ slopes,
             int n_tokens, int heads, int kv_heads, int dim, int vdim, int page_size,
             int max_pages, int num_pages, int window, int keep_first, float scale,
             float out_scale, const float* __restrict__ sinks, int gate_per, int* status) {
    extern __shared__ float smem[];
    __shared__ float scratch[32];
    float* qs = smem;                        // [dim]
    float* wgt = qs + dim;                   // [WA_SEG]
    float* part = wgt + WA_SEG;              // [WA_THREADS]
    prb_grid_launch_dependents();
    const int t = blockIdx.x, h = blockIdx.y;
    if (t >= n_tokens) return;
    const int b = seq_of_token[t];
    const int pos = positions[t];
    O* o = out + (size_t)t * out_ld + (size_t)h * vdim;
    if (b < 0 || pos < 0 || pos >= max_pages * page_size) {
        if (b >= 0 && threadIdx.x == 0)
            prb_set_status(status, PRB_S_POSITION_RANGE, t, pos, max_pages * page_size);
        for (int j = threadIdx.x; j < vdim; j += blockDim.x) o[j] = prb_from_float<O>(0.0f);
        return;
    }
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int n_first = min(keep_first, lo);         // kept first tokens that lie before the window
    const int n = n_first + pos - lo + 1;
    const int g = h / (heads / kv_heads);
    const int rowlen = dim + vdim;
    const float slope = slopes ? slopes[h] : 0.0f;
    const int* table = block_table + (size_t)b * max_pages;
    const float* qp = q + ((size_t)t * heads + h) * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) qs[i] = qp[i];

    const int vthreads = vdim < WA_THREADS ? vdim : WA_THREADS;
    const int kgroups = WA_THREADS / vthreads;
    const int vj = threadIdx.x % vthreads, kg = threadIdx.x / vthreads;
    const bool vlive = kg < kgroups;
    float acc[WA_MAX_V];
#pragma unroll
    for (int x = 0; x < WA_MAX_V; ++x) acc[x] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    __syncthreads();

    for (int s0 = 0; s0 < n; s0 += WA_SEG) {
        const int ns = min(WA_SEG, n - s0);
        float mx = -INFINITY;
        for (int i = threadIdx.x; i < ns; i += blockDim.x) {
            const int v = s0 + i;
            const int j = v < n_first ? v : lo + (v - n_first);
            const int page = table[j / page_size];
            float s = -INFINITY;
            if (page < 0 || page >= num_pages) {
                prb_set_status(status, PRB_S_PAGE_RANGE, t, j, page);
            } else {
                const C* kp = cache + (((size_t)page * kv_heads + g) * page_size + (j % page_size)) * rowlen;
                float a = 0.0f;
                for (int d = 0; d < dim; ++d) a = fmaf(qs[d], prb_to_float<C>(kp[d]), a);
                s = a * scale - slope * (float)(pos - j);
            }
            wgt[i] = s;
            mx = fmaxf(mx, s);
        }
        mx = prb_block_max(mx, scratch);
        const float nm = fmaxf(m, mx);
        const float f = (nm == -INFINITY) ? 1.0f : expf(m - nm);
        float sum = 0.0f;
        for (int i = threadIdx.x; i < ns; i += blockDim.x) {
            const float e = (wgt[i] == -INFINITY) ? 0.0f : expf(wgt[i] - nm);
            wgt[i] = e;
            sum += e;
        }
        sum = prb_block_sum(sum, scratch);
        __syncthreads();                         // the weights are written
        l = l * f + sum;
        m = nm;
        if (vlive) {
#pragma unroll
            for (int x = 0; x < WA_MAX_V; ++x) acc[x] *= f;
            for (int i = kg; i < ns; i += kgroups) {
                const float e = wgt[i];
                if (e == 0.0f) continue;
                const int v = s0 + i;
                const int j = v < n_first ? v : lo + (v - n_first);
                const int page = table[j / page_size];
                if (page < 0 || page >= num_pages) continue;
                const C* vp = cache + (((size_t)page * kv_heads + g) * page_size + (j % page_size)) * rowlen + dim;
#pragma unroll
                for (int x = 0; x < WA_MAX_V; ++x) {
                    const int jj = vj + x * vthreads;
                    if (jj < vdim) acc[x] = fmaf(e, prb_to_float<C>(vp[jj]), acc[x]);
                }
            }
        }
        __syncthreads();                         // before the next segment overwrites the weights
    }
    float fin = 1.0f;                            // the sink joins the denominator, once
    if (sinks) wa_join_sink(sinks[h], m, l, fin);
#pragma unroll
    for (int x = 0; x < WA_MAX_V; ++x) {
        part[threadIdx.x] = acc[x];
        __syncthreads();
        const int jj = vj + x * vthreads;
        if (kg == 0 && jj < vdim) {
            float tot = 0.0f;
            for (int gg = 0; gg < kgroups; ++gg) tot += part[gg * vthreads + vj];
            const float gt = wa_gate(gate, (size_t)t * gate_ld, h, jj, gate_per) * out_scale;
            o[jj] = prb_from_float<O>(l > 0.0f ? tot * fin / l * gt : 0.0f);
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------- the tiled kernel
constexpr int WT_WARPS = 8;
constexpr int WT_PPW = 4;            // (query, head) pairs a warp owns
constexpr int WT_VC = 4;             // value coordinates a lane owns at most (vdim <= 128)
constexpr int WT_KB = 32;            // keys per block

template <typename C, typename O, int VC>
__global__ void __launch_bounds__(WT_WARPS * 32, 2)
wattn_tile_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ q,
                  const C* __restrict__ cache, const int* __restrict__ block_table,
                  const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                  const float* __restrict__ gate, long gate_ld, const float* __restrict__ slopes,
                  int n_tokens, int heads, int kv_heads, int dim, int vdim, int page_size,
                  int max_pages, int num_pages, int window, int keep_first, int tq, float scale,
                  float out_scale, const float* __restrict__ sinks, int gate_per, int* status) {
    extern __shared__ __align__(16) float smem[];
    __shared__ int pages_s[WT_KB];
    prb_grid_launch_dependents();
    const int hg = heads / kv_heads;
    const int g = blockIdx.y;
    const int rowlen = dim + vdim;
    const int kpitch = dim + 1;                      // odd: lanes read their own key's row
    const int qpitch = (dim + 3) / 4 * 4;
    float* Ks = smem;                                // [WT_KB][kpitch]
    float* Vs = Ks + (WT_KB * kpitch + 3) / 4 * 4;   // [WT_KB][vdim]
    float* Qs = Vs + (WT_KB * vdim + 3) / 4 * 4;     // [WT_WARPS * WT_PPW][qpitch]
    float* Ps = Qs + WT_WARPS * WT_PPW * qpitch;     // [WT_WARPS][WT_KB][WT_PPW]: a block's weights
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r_begin = blockIdx.x * tq;
    const int r_end = min(n_tokens, r_begin + tq);
    const int win = window > 0 ? window : NO_WINDOW;
    int r = r_begin;
    while (r < r_end) {
        const int b = seq_of_token[r];
        if (b < 0) {                                 // a padding row
            for (int j = threadIdx.x; j < hg * vdim; j += blockDim.x)
                out[(size_t)r * out_ld + (size_t)g * hg * vdim + j] = prb_from_float<O>(0.0f);
            ++r;
            continue;
        }
        const int p0 = positions[r];
        int r1 = r;
        while (r1 + 1 < r_end && seq_of_token[r1 + 1] == b && positions[r1 + 1] == p0 + (r1 + 1 - r)) ++r1;
        const int nq = r1 - r + 1;
        const int p_last = p0 + nq - 1;
        if (p0 < 0 || p_last >= max_pages * page_size) {
            if (threadIdx.x == 0) prb_set_status(status, PRB_S_POSITION_RANGE, r, p_last, max_pages * page_size);
            for (int j = threadIdx.x; j < nq * hg * vdim; j += blockDim.x) {
                const int qi = j / (hg * vdim), rest = j - qi * hg * vdim;
                out[(size_t)(r + qi) * out_ld + (size_t)g * hg * vdim + rest] = prb_from_float<O>(0.0f);
            }
            r = r1 + 1;
            continue;
        }
        // the window's blocks begin at win_start; kept first tokens before it have blocks of
        // their own, 0 .. first_end - 1
        const int lo_min = max(0, p0 - win + 1);
        const int win_start = (lo_min / WT_KB) * WT_KB;
        const int first_end = min(keep_first, win_start);
        const int first_blocks = (first_end + WT_KB - 1) / WT_KB;
        const int n_blocks = first_blocks + (p_last - win_start) / WT_KB + 1;
        const int* table = block_table + (size_t)b * max_pages;
        __syncthreads();                             // the pass before is done with shared memory
        const int n_pairs = nq * hg;                 // pair = qi * hg + hh
        for (int e = threadIdx.x; e < n_pairs * dim; e += blockDim.x) {
            const int pair = e / dim, d = e - pair * dim;
            const int qi = pair / hg, hh = pair - qi * hg;
            Qs[pair * qpitch + d] = q[((size_t)(r + qi) * heads + g * hg + hh) * dim + d] * scale;
        }
        float acc[WT_PPW][VC];
        float m[WT_PPW], l[WT_PPW], slope[WT_PPW];
        int pi[WT_PPW];
#pragma unroll
        for (int x = 0; x < WT_PPW; ++x) {
            const int pair = x * WT_WARPS + warp;
            m[x] = -INFINITY;
            l[x] = 0.0f;
            pi[x] = pair < n_pairs ? p0 + pair / hg : -1;
            slope[x] = (slopes && pair < n_pairs) ? slopes[g * hg + pair % hg] : 0.0f;
#pragma unroll
            for (int c = 0; c < VC; ++c) acc[x][c] = 0.0f;
        }
        for (int blk = 0; blk < n_blocks; ++blk) {
            const int j0 = blk < first_blocks ? blk * WT_KB : win_start + (blk - first_blocks) * WT_KB;
            const int j_end = blk < first_blocks ? first_end : p_last + 1;     // keys staged: j < j_end
            __syncthreads();                         // the block before has been consumed
            if (threadIdx.x < WT_KB) {
                const int jj = j0 + (int)threadIdx.x;
                int pg = -1;
                // (only keys some query of the pass may see are fetched: others may lie on pages
                // the window has given back)
                if (jj < j_end && (jj >= lo_min || jj < keep_first)) {
                    pg = table[jj / page_size];
                    if (pg < 0 || pg >= num_pages) {
                        prb_set_status(status, PRB_S_PAGE_RANGE, r, jj, pg);
                        pg = -1;
                    }
                }
                pages_s[threadIdx.x] = pg;
            }
            __syncthreads();
            constexpr int VE = 16 / (int)sizeof(C);
            if (rowlen % VE == 0 && dim % VE == 0) {
                const int nv = rowlen / VE;
#pragma unroll 2
                for (int e = threadIdx.x; e < WT_KB * nv; e += blockDim.x) {
                    const int kk = e / nv, vi = e - kk * nv;
                    const int pg = pages_s[kk];
                    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
                    if (pg >= 0)
                        raw = *reinterpret_cast<const uint4*>(
                            cache + (((size_t)pg * kv_heads + g) * page_size + ((j0 + kk) % page_size)) * rowlen + vi * VE);
                    const C* vals = reinterpret_cast<const C*>(&raw);
                    const int off = vi * VE;
                    float* dst = off < dim ? Ks + kk * kpitch + off : Vs + kk * vdim + off - dim;
#pragma unroll
                    for (int x = 0; x < VE; ++x) dst[x] = prb_to_float<C>(vals[x]);
                }
            } else {
                for (int e = threadIdx.x; e < WT_KB * rowlen; e += blockDim.x) {
                    const int kk = e / rowlen, off = e - kk * rowlen;
                    const int pg = pages_s[kk];
                    const float val = pg < 0 ? 0.0f : prb_to_float<C>(
                        cache[(((size_t)pg * kv_heads + g) * page_size + ((j0 + kk) % page_size)) * rowlen + off]);
                    if (off < dim) Ks[kk * kpitch + off] = val;
                    else Vs[kk * vdim + off - dim] = val;
                }
            }
            __syncthreads();
            const int j = j0 + lane;
            const float* krow = Ks + lane * kpitch;
            bool act[WT_PPW];
            float s[WT_PPW];
            int k_hi = 0;
#pragma unroll
            for (int x = 0; x < WT_PPW; ++x) {
                // the pair sees at least one key of this block
                act[x] = pi[x] >= 0 && j0 <= pi[x] && j0 < j_end &&
                         (j0 + WT_KB - 1 >= pi[x] - win + 1 || j0 < keep_first);
                if (act[x]) k_hi = max(k_hi, min(min(WT_KB, j_end - j0), pi[x] - j0 + 1));
                s[x] = 0.0f;
            }
            if (k_hi == 0) continue;                 // nothing of this block is seen by the warp
            if (dim % 4 == 0) {
                for (int d = 0; d < dim; d += 4) {
                    const float a0 = krow[d], a1 = krow[d + 1], a2 = krow[d + 2], a3 = krow[d + 3];
#pragma unroll
                    for (int x = 0; x < WT_PPW; ++x) {
                        const float4 u = *reinterpret_cast<const float4*>(Qs + (x * WT_WARPS + warp) * qpitch + d);
                        s[x] = fmaf(u.w, a3, fmaf(u.z, a2, fmaf(u.y, a1, fmaf(u.x, a0, s[x]))));
                    }
                }
            } else {
                for (int d = 0; d < dim; ++d) {
                    const float a0 = krow[d];
#pragma unroll
                    for (int x = 0; x < WT_PPW; ++x) s[x] = fmaf(Qs[(x * WT_WARPS + warp) * qpitch + d], a0, s[x]);
                }
            }
            float e[WT_PPW];
#pragma unroll
            for (int x = 0; x < WT_PPW; ++x) {
                e[x] = 0.0f;
                if (!act[x]) continue;
                const bool vis = j < j_end && j <= pi[x] && (pi[x] - j < win || j < keep_first);
                const float tt = vis ? s[x] - slope[x] * (float)(pi[x] - j) : -INFINITY;
                const float nm = fmaxf(m[x], prb_warp_max(tt));
                const float f = expf(m[x] - nm);                   // (exp(-inf) = 0)
                e[x] = vis ? expf(tt - nm) : 0.0f;
                l[x] = l[x] * f + prb_warp_sum(e[x]);
                m[x] = nm;
#pragma unroll
                for (int c = 0; c < VC; ++c) acc[x][c] *= f;
            }
            // a key's weights for the warp's four pairs go through shared memory: one 16-byte
            // load that all lanes share instead of four shuffles a key
            static_assert(WT_PPW == 4, "a key's weights are one float4");
            float* pw = Ps + (size_t)warp * WT_KB * WT_PPW;
            __syncwarp();                            // the block before has been read
            *reinterpret_cast<float4*>(pw + lane * WT_PPW) = make_float4(e[0], e[1], e[2], e[3]);
            __syncwarp();
            for (int kk = 0; kk < k_hi; ++kk) {
                float v[VC];
#pragma unroll
                for (int c = 0; c < VC; ++c) v[c] = (lane + 32 * c < vdim) ? Vs[kk * vdim + lane + 32 * c] : 0.0f;
                const float4 w4 = *reinterpret_cast<const float4*>(pw + kk * WT_PPW);
                const float w[WT_PPW] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                for (int x = 0; x < WT_PPW; ++x) {
#pragma unroll
                    for (int c = 0; c < VC; ++c) acc[x][c] = fmaf(w[x], v[c], acc[x][c]);
                }
            }
        }
#pragma unroll
        for (int x = 0; x < WT_PPW; ++x) {
            const int pair = x * WT_WARPS + warp;
            if (pair >= n_pairs) break;
            const int qi = pair / hg, hh = pair - qi * hg;
            const int h = g * hg + hh;
            float fin = 1.0f, lx = l[x];
            if (sinks) wa_join_sink(sinks[h], m[x], lx, fin);
            O* dst = out + (size_t)(r + qi) * out_ld + (size_t)h * vdim;
#pragma unroll
            for (int c = 0; c < VC; ++c)
                if (lane + 32 * c < vdim) {
                    const float gt = wa_gate(gate, (size_t)(r + qi) * gate_ld, h, lane + 32 * c, gate_per) * out_scale;
                    dst[lane + 32 * c] = prb_from_float<O>(lx > 0.0f ? acc[x][c] * fin / lx * gt : 0.0f);
                }
        }
        r = r1 + 1;
    }
}

// ------------------------------------------------------------ the single-token kernel
// A CTA per (token, key/value head) for steps whose requests bring one token each.  The key
// blocks of the tiled kernel (32 ABSOLUTE positions; the kept first tokens' before the
// window's) are dealt to the CTA's warps round by round: a round stages one block per warp in
// shared memory with all threads loading, then every warp scores its own block for all query
// heads of the key/value head (a lane a key) and adds its values to sums of its own.  The
// warps' states (maximum, sum, weighted values) are joined at the end in warp order.  Where
// the step's tokens leave SMs idle, a (token, key/value head) is a thread-block cluster of
// gridDim.z CTAs that take the rounds in turn; the cluster's first CTA joins all CTAs' warps
// (in CTA, then warp order) through distributed shared memory.
constexpr int WS_MAX_PPW = 8;        // query heads a key/value head at most

__device__ __forceinline__ void ws_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ws_ld_cluster(const float* local, int rank) {
    const uint32_t laddr = (uint32_t)__cvta_generic_to_shared(local);
    uint32_t raddr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(laddr), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(raddr) : "memory");
    return v;
}

// A staged key row holds the cache's own numbers (bfloat16 rows are half the size of 32-bit
// ones: twice the keys a round, or several CTAs an SM); its pitch is an odd number of 4-byte
// words, so that the lanes, a key each, read their rows without bank conflicts.
template <typename C>
__device__ __forceinline__ void ws_k4(const uint32_t* krow, int d, float& a0, float& a1, float& a2, float& a3);
template <>
__device__ __forceinline__ void ws_k4<float>(const uint32_t* krow, int d, float& a0, float& a1, float& a2, float& a3) {
    const float* f = reinterpret_cast<const float*>(krow);
    a0 = f[d]; a1 = f[d + 1]; a2 = f[d + 2]; a3 = f[d + 3];
}
template <>
__device__ __forceinline__ void ws_k4<__nv_bfloat16>(const uint32_t* krow, int d, float& a0, float& a1, float& a2, float& a3) {
    const uint32_t w0 = krow[d >> 1], w1 = krow[(d >> 1) + 1];       // (a bfloat16 is a float's upper half)
    a0 = __uint_as_float(w0 << 16); a1 = __uint_as_float(w0 & 0xffff0000u);
    a2 = __uint_as_float(w1 << 16); a3 = __uint_as_float(w1 & 0xffff0000u);
}
__host__ __device__ inline int ws_kwords(int dim, int csize) { return ((dim * csize + 3) / 4) | 1; }
__host__ __device__ inline int ws_vbytes(int vdim, int csize) { return (vdim * csize + 15) / 16 * 16; }

template <typename C, typename O, int VC, int PPW>
__global__ void __launch_bounds__(WT_WARPS * 32)
wattn_single_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ q,
                    const C* __restrict__ cache, const int* __restrict__ block_table,
                    const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                    const float* __restrict__ gate, long gate_ld, const float* __restrict__ slopes,
                    int n_tokens, int heads, int kv_heads, int dim, int vdim, int page_size,
                    int max_pages, int num_pages, int window, int keep_first, float scale,
                    float out_scale, const float* __restrict__ sinks, int gate_per, int* status) {
    extern __shared__ __align__(16) float smem[];
    __shared__ long long rows_s[WT_WARPS * WT_KB];   // a staged key's row of the cache, or -1
    prb_grid_launch_dependents();
    const int nw = blockDim.x >> 5;                  // warps: key blocks a round
    const int hg = heads / kv_heads;
    const int g = blockIdx.y, r = blockIdx.x;
    const int rowlen = dim + vdim;
    const int qpitch = (dim + 3) / 4 * 4;
    const int keys = nw * WT_KB;
    const int jpitch = 2 + vdim;
    const int pw = ws_kwords(dim, (int)sizeof(C));   // a staged key's pitch in 4-byte words (odd)
    const int vpb = ws_vbytes(vdim, (int)sizeof(C)); // a staged value row's pitch in bytes
    float* Qs = smem;                                // [hg][qpitch]
    float* Js = Qs + hg * qpitch;                    // [nw][hg][2 + vdim]
    uint32_t* Kw = reinterpret_cast<uint32_t*>(Js + (nw * hg * jpitch + 3) / 4 * 4);   // [keys][pw]
    unsigned char* Vb = reinterpret_cast<unsigned char*>(Kw + (keys * pw + 3) / 4 * 4); // [keys][vpb]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    O* orow = out + (size_t)r * out_ld + (size_t)g * hg * vdim;
    const int b = seq_of_token[r];
    const int p = b < 0 ? 0 : positions[r];
    const int splits = gridDim.z, split = blockIdx.z;            // the cluster and this CTA's rank
    if (b < 0 || p < 0 || p >= max_pages * page_size) {          // a padding row, or a bad one
        if (split > 0) return;                                   // (so for the whole cluster)
        if (b >= 0 && threadIdx.x == 0)
            prb_set_status(status, PRB_S_POSITION_RANGE, r, p, max_pages * page_size);
        for (int j = threadIdx.x; j < hg * vdim; j += blockDim.x) orow[j] = prb_from_float<O>(0.0f);
        return;
    }
    const int win = window > 0 ? window : NO_WINDOW;
    const int lo_min = max(0, p - win + 1);
    const int win_start = (lo_min / WT_KB) * WT_KB;
    const int first_end = min(keep_first, win_start);
    const int first_blocks = (first_end + WT_KB - 1) / WT_KB;
    const int n_blocks = first_blocks + (p - win_start) / WT_KB + 1;
    const int* table = block_table + (size_t)b * max_pages;
    for (int e = threadIdx.x; e < hg * dim; e += blockDim.x) {
        const int hh = e / dim, d = e - hh * dim;
        Qs[hh * qpitch + d] = q[((size_t)r * heads + g * hg + hh) * dim + d] * scale;
    }
    float acc[PPW][VC];
    float m[PPW], l[PPW], slope[PPW];
#pragma unroll
    for (int x = 0; x < PPW; ++x) {
        m[x] = -INFINITY;
        l[x] = 0.0f;
        slope[x] = (slopes && x < hg) ? slopes[g * hg + x] : 0.0f;
#pragma unroll
        for (int c = 0; c < VC; ++c) acc[x][c] = 0.0f;
    }
    for (int blk0 = split * nw; blk0 < n_blocks; blk0 += splits * nw) {
        __syncthreads();                             // the round before has been consumed
        for (int kk = threadIdx.x; kk < keys; kk += blockDim.x) {
            const int blk = blk0 + kk / WT_KB;
            long long row = -1;
            if (blk < n_blocks) {
                const int j0 = blk < first_blocks ? blk * WT_KB : win_start + (blk - first_blocks) * WT_KB;
                const int j_end = blk < first_blocks ? first_end : p + 1;
                const int jj = j0 + kk % WT_KB;
                // (only keys the query may see are fetched)
                if (jj < j_end && (jj >= lo_min || jj < keep_first)) {
                    const int pg = table[jj / page_size];
                    if (pg < 0 || pg >= num_pages) prb_set_status(status, PRB_S_PAGE_RANGE, r, jj, pg);
                    else row = ((long long)pg * kv_heads + g) * page_size + jj % page_size;
                }
            }
            rows_s[kk] = row;
        }
        __syncthreads();
        constexpr int VE = 16 / (int)sizeof(C);
        if (rowlen % VE == 0 && dim % VE == 0) {
            const int nv = rowlen / VE;
#pragma unroll 8
            for (int e = threadIdx.x; e < keys * nv; e += blockDim.x) {
                const int kk = e / nv, vi = e - kk * nv;
                const long long row = rows_s[kk];
                uint4 raw = make_uint4(0u, 0u, 0u, 0u);
                if (row >= 0) raw = *reinterpret_cast<const uint4*>(cache + (size_t)row * rowlen + vi * VE);
                const int off = vi * VE;
                if (off < dim) {                     // (the odd pitch: word by word)
                    uint32_t* dst = Kw + kk * pw + off * (int)sizeof(C) / 4;
                    dst[0] = raw.x; dst[1] = raw.y; dst[2] = raw.z; dst[3] = raw.w;
                } else {
                    *reinterpret_cast<uint4*>(Vb + (size_t)kk * vpb + (size_t)(off - dim) * sizeof(C)) = raw;
                }
            }
        } else {
            for (int e = threadIdx.x; e < keys * rowlen; e += blockDim.x) {
                const int kk = e / rowlen, off = e - kk * rowlen;
                const long long row = rows_s[kk];
                const C val = row < 0 ? prb_from_float<C>(0.0f) : cache[(size_t)row * rowlen + off];
                if (off < dim) reinterpret_cast<C*>(Kw + kk * pw)[off] = val;
                else reinterpret_cast<C*>(Vb + (size_t)kk * vpb)[off - dim] = val;
            }
        }
        __syncthreads();
        const int blk = blk0 + warp;
        if (blk >= n_blocks) continue;
        const int j0 = blk < first_blocks ? blk * WT_KB : win_start + (blk - first_blocks) * WT_KB;
        const int j_end = blk < first_blocks ? first_end : p + 1;
        const int k_hi = min(min(WT_KB, j_end - j0), p - j0 + 1);
        if (k_hi <= 0) continue;
        const int j = j0 + lane;
        const uint32_t* krow = Kw + (warp * WT_KB + lane) * pw;
        const unsigned char* vblk = Vb + (size_t)warp * WT_KB * vpb;
        float s[PPW];
#pragma unroll
        for (int x = 0; x < PPW; ++x) s[x] = 0.0f;
        if (dim % 4 == 0) {
            for (int d = 0; d < dim; d += 4) {
                float a0, a1, a2, a3;
                ws_k4<C>(krow, d, a0, a1, a2, a3);
#pragma unroll
                for (int x = 0; x < PPW; ++x) {
                    if (x < hg) {
                        const float4 u = *reinterpret_cast<const float4*>(Qs + x * qpitch + d);
                        s[x] = fmaf(u.w, a3, fmaf(u.z, a2, fmaf(u.y, a1, fmaf(u.x, a0, s[x]))));
                    }
                }
            }
        } else {
            for (int d = 0; d < dim; ++d) {
                const float a0 = prb_to_float<C>(reinterpret_cast<const C*>(krow)[d]);
#pragma unroll
                for (int x = 0; x < PPW; ++x)
                    if (x < hg) s[x] = fmaf(Qs[x * qpitch + d], a0, s[x]);
            }
        }
        const bool vis = j < j_end && j <= p && (p - j < win || j < keep_first);
        float e[PPW];
#pragma unroll
        for (int x = 0; x < PPW; ++x) {
            e[x] = 0.0f;
            if (x >= hg) continue;
            const float tt = vis ? s[x] - slope[x] * (float)(p - j) : -INFINITY;
            const float nm = fmaxf(m[x], prb_warp_max(tt));
            if (nm == -INFINITY) continue;           // (no key of the block is seen)
            const float f = expf(m[x] - nm);         // (exp(-inf) = 0)
            e[x] = vis ? expf(tt - nm) : 0.0f;
            l[x] = l[x] * f + prb_warp_sum(e[x]);
            m[x] = nm;
#pragma unroll
            for (int c = 0; c < VC; ++c) acc[x][c] *= f;
        }
        for (int kk = 0; kk < k_hi; ++kk) {
            float v[VC];
#pragma unroll
            for (int c = 0; c < VC; ++c)
                v[c] = (lane + 32 * c < vdim)
                    ? prb_to_float<C>(reinterpret_cast<const C*>(vblk + (size_t)kk * vpb)[lane + 32 * c]) : 0.0f;
#pragma unroll
            for (int x = 0; x < PPW; ++x) {
                const float w = __shfl_sync(0xffffffffu, e[x], kk);
#pragma unroll
                for (int c = 0; c < VC; ++c) acc[x][c] = fmaf(w, v[c], acc[x][c]);
            }
        }
    }
    // the warps' states, then a thread per (head, value coordinate) joins them in warp order
#pragma unroll
    for (int x = 0; x < PPW; ++x) {
        if (x >= hg) break;
        float* st = Js + ((size_t)warp * hg + x) * jpitch;
        if (lane == 0) {
            st[0] = m[x];
            st[1] = l[x];
        }
#pragma unroll
        for (int c = 0; c < VC; ++c)
            if (lane + 32 * c < vdim) st[2 + lane + 32 * c] = acc[x][c];
    }
    if (splits > 1) ws_cluster_sync();               // every CTA's states are in place
    else __syncthreads();
    if (split == 0) {
        for (int e = threadIdx.x; e < hg * vdim; e += blockDim.x) {
            const int hh = e / vdim, jv = e - hh * vdim;
            float top = -INFINITY;
            for (int ss = 0; ss < splits; ++ss)
                for (int w = 0; w < nw; ++w) {
                    const float* st = Js + ((size_t)w * hg + hh) * jpitch;
                    top = fmaxf(top, splits > 1 ? ws_ld_cluster(st, ss) : st[0]);
                }
            float lsum = 0.0f, a = 0.0f;
            for (int ss = 0; ss < splits; ++ss)
                for (int w = 0; w < nw; ++w) {
                    const float* st = Js + ((size_t)w * hg + hh) * jpitch;
                    const float mw = splits > 1 ? ws_ld_cluster(st, ss) : st[0];
                    const float f = mw == -INFINITY ? 0.0f : expf(mw - top);
                    lsum = fmaf(splits > 1 ? ws_ld_cluster(st + 1, ss) : st[1], f, lsum);
                    a = fmaf(splits > 1 ? ws_ld_cluster(st + 2 + jv, ss) : st[2 + jv], f, a);
                }
            const int h = g * hg + hh;
            if (sinks) {
                float fin = 1.0f;
                wa_join_sink(sinks[h], top, lsum, fin);
                a *= fin;
            }
            const float gt = wa_gate(gate, (size_t)r * gate_ld, h, jv, gate_per) * out_scale;
            orow[e] = prb_from_float<O>(lsum > 0.0f ? a / lsum * gt : 0.0f);
        }
    }
    if (splits > 1) ws_cluster_sync();               // the states have been read: CTAs may leave
}

size_t ws_smem(int hg, int dim, int vdim, int nw, int csize) {
    const int keys = nw * WT_KB;
    return (size_t)(hg * ((dim + 3) / 4 * 4) + (nw * hg * (2 + vdim) + 3) / 4 * 4 +
                    (keys * ws_kwords(dim, csize) + 3) / 4 * 4) * 4 + (size_t)keys * ws_vbytes(vdim, csize);
}

// Warps (key blocks a round) of the single-token kernel for these sizes and a cache of `csize`
// bytes a number; 0: it does not take them.
int ws_warps(int heads, int kv_heads, int dim, int vdim, int csize) {
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0) return 0;
    const int hg = heads / kv_heads;
    if (hg > WS_MAX_PPW || vdim > 32 * WT_VC || dim > 512) return 0;
    for (int nw = WT_WARPS; nw >= 1; nw >>= 1)
        if (ws_smem(hg, dim, vdim, nw, csize) <= 200 * 1024) return nw;
    return 0;
}

size_t wt_smem(int dim, int vdim) {
    return (size_t)((WT_KB * (dim + 1) + 3) / 4 * 4 + (WT_KB * vdim + 3) / 4 * 4 +
                    WT_WARPS * WT_PPW * ((dim + 3) / 4 * 4) + WT_WARPS * WT_KB * WT_PPW) * sizeof(float);
}
}  // namespace

PRB_API int prb_wattn_prepare(float* q_out, void* cache, const float* proj, long ld, int q_col,
                              int k_col, int v_col, const float* q_norm, const float* k_norm,
                              const int* slots, const int* positions, const float* freq,
                              int n_tokens, int heads, int kv_heads, int dim, int vdim, int rot_dims,
                              float eps, float temp_coef, int temp_every, int page_size,
                              int num_pages, int cache_dtype, int norm_mode, const float* q_bias,
                              const float* k_bias, const float* v_bias, const float* freq_lo,
                              int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (norm_mode < 0 || norm_mode > 3) return PRB_E_ARG;
    if (heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || rot_dims < 0 || rot_dims % 2 ||
        rot_dims > dim || page_size <= 0)
        return PRB_E_SIZE;
    if (cache_dtype == PRB_F32)
        wattn_prepare_kernel<float><<<n_tokens, 256, 0, stream>>>(
            q_out, (float*)cache, proj, ld, q_col, k_col, v_col, q_norm, k_norm, slots, positions,
            freq, n_tokens, heads, kv_heads, dim, vdim, rot_dims, eps, temp_coef, temp_every,
            page_size, num_pages, norm_mode, q_bias, k_bias, v_bias, freq_lo, status);
    else if (cache_dtype == PRB_BF16)
        wattn_prepare_kernel<__nv_bfloat16><<<n_tokens, 256, 0, stream>>>(
            q_out, (__nv_bfloat16*)cache, proj, ld, q_col, k_col, v_col, q_norm, k_norm, slots,
            positions, freq, n_tokens, heads, kv_heads, dim, vdim, rot_dims, eps, temp_coef,
            temp_every, page_size, num_pages, norm_mode, q_bias, k_bias, v_bias, freq_lo, status);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_wattn(void* out, long out_ld, const float* q, const void* cache,
                      const int* block_table, const int* seq_of_token, const int* positions,
                      const float* gate, long gate_ld, const float* slopes, int n_tokens, int heads,
                      int kv_heads, int dim, int vdim, int page_size, int max_pages, int num_pages,
                      int window, int keep_first, float scale, float out_scale, int cache_dtype,
                      int out_dtype, const float* sinks, int gate_per, int* status,
                      cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || heads > 65535 || dim <= 0 ||
        vdim <= 0 || vdim > WA_THREADS * WA_MAX_V || page_size <= 0 || max_pages <= 0 ||
        window < 0 || keep_first < 0)
        return PRB_E_SIZE;
    const size_t smem = (size_t)(dim + WA_SEG + WA_THREADS) * sizeof(float);
    if (smem > 48 * 1024) return PRB_E_SIZE;
    dim3 grid(n_tokens, heads);
#define WATTN(CT, OT)                                                                            \
    wattn_kernel<CT, OT><<<grid, WA_THREADS, smem, stream>>>(                                    \
        (OT*)out, out_ld, q, (const CT*)cache, block_table, seq_of_token, positions, gate,       \
        gate_ld, slopes, n_tokens, heads, kv_heads, dim, vdim, page_size, max_pages, num_pages,  \
        window, keep_first, scale, out_scale, sinks, gate_per, status)
    if (cache_dtype == PRB_F32 && out_dtype == PRB_F32) WATTN(float, float);
    else if (cache_dtype == PRB_BF16 && out_dtype == PRB_BF16) WATTN(__nv_bfloat16, __nv_bfloat16);
    else return PRB_E_DTYPE;
#undef WATTN
    PRB_LAUNCH_CHECK();
    return 0;
}

// Rows a CTA of the tiled kernel takes at most for these sizes (0: it does not take them).
PRB_API int prb_wattn_tile_rows(int heads, int kv_heads, int dim, int vdim) {
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0) return 0;
    const int hg = heads / kv_heads;
    if (vdim > 32 * WT_VC || hg > WT_WARPS * WT_PPW || dim > 512) return 0;
    if (wt_smem(dim, vdim) > 160 * 1024) return 0;
    return (WT_WARPS * WT_PPW) / hg;
}

PRB_API int prb_wattn_tile(void* out, long out_ld, const float* q, const void* cache,
                           const int* block_table, const int* seq_of_token, const int* positions,
                           const float* gate, long gate_ld, const float* slopes, int n_tokens,
                           int heads, int kv_heads, int dim, int vdim, int page_size, int max_pages,
                           int num_pages, int window, int keep_first, int tq, float scale,
                           float out_scale, int cache_dtype, int out_dtype, const float* sinks,
                           int gate_per, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int most = prb_wattn_tile_rows(heads, kv_heads, dim, vdim);
    if (most <= 0 || kv_heads > 65535 || page_size <= 0 || max_pages <= 0 || window < 0 ||
        keep_first < 0)
        return PRB_E_SIZE;
    if (tq <= 0 || tq > most) tq = most;
    const size_t smem = wt_smem(dim, vdim);
    dim3 grid((n_tokens + tq - 1) / tq, kv_heads);
#define WATT1(CT, OT, VCN)                                                                       \
    do {                                                                                         \
        if (smem > 40 * 1024)       /* (static shared memory counts toward the 48 KB too) */ \
            cudaFuncSetAttribute(wattn_tile_kernel<CT, OT, VCN>,                                 \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
        wattn_tile_kernel<CT, OT, VCN><<<grid, WT_WARPS * 32, smem, stream>>>(                   \
            (OT*)out, out_ld, q, (const CT*)cache, block_table, seq_of_token, positions, gate,   \
            gate_ld, slopes, n_tokens, heads, kv_heads, dim, vdim, page_size, max_pages,         \
            num_pages, window, keep_first, tq, scale, out_scale, sinks, gate_per, status);       \
    } while (0)
#define WATT(CT, OT)                                                                             \
    do {                                                                                         \
        switch ((vdim + 31) / 32) {         /* value coordinates a lane owns */                  \
            case 1: WATT1(CT, OT, 1); break;                                                     \
            case 2: WATT1(CT, OT, 2); break;                                                     \
            case 3: WATT1(CT, OT, 3); break;                                                     \
            default: WATT1(CT, OT, 4); break;                                                    \
        }                                                                                        \
    } while (0)
    if (cache_dtype == PRB_F32 && out_dtype == PRB_F32) WATT(float, float);
    else if (cache_dtype == PRB_BF16 && out_dtype == PRB_BF16) WATT(__nv_bfloat16, __nv_bfloat16);
    else return PRB_E_DTYPE;
#undef WATT
#undef WATT1
    PRB_LAUNCH_CHECK();
    return 0;
}

// 1 if the single-token kernel takes these sizes.
PRB_API int prb_wattn_single_supports(int heads, int kv_heads, int dim, int vdim) {
    return ws_warps(heads, kv_heads, dim, vdim, 4) > 0 ? 1 : 0;     // (a 32-bit cache is the larger)
}

PRB_API int prb_wattn_single(void* out, long out_ld, const float* q, const void* cache,
                             const int* block_table, const int* seq_of_token, const int* positions,
                             const float* gate, long gate_ld, const float* slopes, int n_tokens,
                             int heads, int kv_heads, int dim, int vdim, int page_size,
                             int max_pages, int num_pages, int window, int keep_first, float scale,
                             float out_scale, int cache_dtype, int out_dtype, const float* sinks,
                             int gate_per, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (cache_dtype != PRB_F32 && cache_dtype != PRB_BF16) return PRB_E_DTYPE;
    const int csize = cache_dtype == PRB_F32 ? 4 : 2;
    const int nw = ws_warps(heads, kv_heads, dim, vdim, csize);
    if (nw <= 0 || kv_heads > 65535 || page_size <= 0 || max_pages <= 0 || window < 0 ||
        keep_first < 0)
        return PRB_E_SIZE;
    const int hg = heads / kv_heads;
    const size_t smem = ws_smem(hg, dim, vdim, nw, csize);
    // CTAs a (token, key/value head): as many as the SMs the step would leave idle allow, while
    // a request's keys (at most the window's and the kept ones) still give every CTA a round
    long long most = (long long)max_pages * page_size;
    if (window > 0 && (long long)window + keep_first + WT_KB < most) most = (long long)window + keep_first + WT_KB;
    const long long rounds = (most + nw * WT_KB - 1) / (nw * WT_KB);
    int splits = 1;
    while (splits < 8 && splits + 1 <= rounds &&
           (long long)n_tokens * kv_heads * (splits + 1) <= prb_sm_count())
        ++splits;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tokens, kv_heads, splits);
    cfg.blockDim = dim3(nw * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = (unsigned)splits;
    cfg.attrs = attr;
    cfg.numAttrs = splits > 1 ? 1 : 0;
#define WS2(CT, OT, VCN, PN)                                                                     \
    do {                                                                                         \
        if (smem > 40 * 1024)       /* (static shared memory counts toward the 48 KB too) */ \
            cudaFuncSetAttribute(wattn_single_kernel<CT, OT, VCN, PN>,                           \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
        cudaLaunchKernelEx(&cfg, wattn_single_kernel<CT, OT, VCN, PN>, (OT*)out, out_ld, q,      \
                           (const CT*)cache, block_table, seq_of_token, positions, gate,         \
                           gate_ld, slopes, n_tokens, heads, kv_heads, dim, vdim, page_size,     \
                           max_pages, num_pages, window, keep_first, scale, out_scale, sinks,    \
                           gate_per, status);                                                    \
    } while (0)
#define WS1(CT, OT, VCN)                                                                         \
    do {                                                                                         \
        if (hg <= 2) WS2(CT, OT, VCN, 2);                                                        \
        else if (hg <= 4) WS2(CT, OT, VCN, 4);                                                   \
        else WS2(CT, OT, VCN, 8);                                                                \
    } while (0)
#define WS(CT, OT)                                                                               \
    do {                                                                                         \
        if (vdim <= 64) WS1(CT, OT, 2);                                                          \
        else WS1(CT, OT, 4);                                                                     \
    } while (0)
    if (cache_dtype == PRB_F32 && out_dtype == PRB_F32) WS(float, float);
    else if (cache_dtype == PRB_BF16 && out_dtype == PRB_BF16) WS(__nv_bfloat16, __nv_bfloat16);
    else return PRB_E_DTYPE;
#undef WS
#undef WS1
#undef WS2
    PRB_LAUNCH_CHECK();
    return 0;
}
