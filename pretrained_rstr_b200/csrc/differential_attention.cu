// Differential attention over the paged cache: every query head runs TWO softmax attentions
// ("maps") over the same values and subtracts them,
//     o = a1 - lambda a2,   o <- o / sqrt(mean(o^2) + eps) * out_scale    (per head, over vdim)
// with grouped key/value heads and an optional block mask: a query at position p sees keys
// floor(p / block) * block .. p (block 0: all keys 0 .. p), counted from the sequence's start.
//
// Cache: one pool per layer, one row per (token, key/value head): [k map 1 | k map 2 | v],
// 2 * dim + vdim numbers, so a key's two maps and its value come with one page look-up.
//
// diff_prepare: a CTA per token.  Reads the fused projection's 32-bit result, turns the first
// rot_dims coordinates of every map of q and k by the token's position (rotate-half layout,
// angles in 32-bit), leaves q in 32-bit beside the step and writes the token's cache rows.
//
// diff_attention: a CTA per (token, query head), 32-bit arithmetic; keys in segments of SEG
// with running maxima and sums per map.  Reduction orders depend on the visible range and the
// sizes only, never on the batch.
#include "common.cuh"

namespace {
constexpr int DA_THREADS = 128;
constexpr int DA_SEG = 256;         // keys scored at a time
constexpr int DA_MAX_V = 4;         // value coordinates a thread owns at most (vdim <= 512)

template <typename C>
__global__ void diff_prepare_kernel(float* __restrict__ q_out, C* __restrict__ cache,
                                    const float* __restrict__ proj, long ld, int q_col, int k_col,
                                    int v_col, const int* __restrict__ slots,
                                    const int* __restrict__ positions, const float* __restrict__ freq,
                                    int n_tokens, int heads, int kv_heads, int dim, int vdim,
                                    int rot_dims, int page_size, int num_pages, int* status) {
    prb_grid_launch_dependents();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const float* row = proj + (size_t)t * ld;
    const float pos = (float)positions[t];
    const int half = rot_dims / 2;
    const int units = half + (dim - rot_dims);       // per map: pairs, then coordinates that stay
    // queries: heads * 2 maps
    float* qo = q_out + (size_t)t * heads * 2 * dim;
    for (int u = threadIdx.x; u < heads * 2 * units; u += blockDim.x) {
        const int m = u / units, w = u - m * units;
        const float* src = row + q_col + m * dim;
        float* dst = qo + m * dim;
        if (w < half) {
            float sn, cs;
            sincosf(pos * freq[w], &sn, &cs);
            const float a = src[w], b = src[w + half];
            dst[w] = a * cs - b * sn;
            dst[w + half] = b * cs + a * sn;
        } else {
            const int i = w - half + rot_dims;
            dst[i] = src[i];
        }
    }
    if (slots == nullptr) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int page = slot / page_size, off = slot - page * page_size;
    if (page >= num_pages) {
        if (threadIdx.x == 0) prb_set_status(status, PRB_S_SLOT_RANGE, t, slot, num_pages);
        return;
    }
    const int rowlen = 2 * dim + vdim;
    for (int u = threadIdx.x; u < kv_heads * 2 * units; u += blockDim.x) {
        const int m = u / units, w = u - m * units;          // m = kv head * 2 + map
        const int g = m >> 1;
        const float* src = row + k_col + m * dim;
        C* dst = cache + (((size_t)page * kv_heads + g) * page_size + off) * rowlen + (m & 1) * dim;
        if (w < half) {
            float sn, cs;
            sincosf(pos * freq[w], &sn, &cs);
            const float a = src[w], b = src[w + half];
            dst[w] = prb_from_float<C>(a * cs - b * sn);
            dst[w + half] = prb_from_float<C>(b * cs + a * sn);
        } else {
            const int i = w - half + rot_dims;
            dst[i] = prb_from_float<C>(src[i]);
        }
    }
    for (int u = threadIdx.x; u < kv_heads * vdim; u += blockDim.x) {
        const int g = u / vdim, j = u - g * vdim;
        cache[(((size_t)page * kv_heads + g) * page_size + off) * rowlen + 2 * dim + j] =
            prb_from_float<C>(row[v_col + u]);
    }
}

template <typename C, typename O>
__global__ void __launch_bounds__(DA_THREADS)
diff_attention_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ q,
                      const C* __restrict__ cache, const int* __restrict__ block_table,
                      const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                      int n_tokens, int heads, int kv_heads, int dim, int vdim, int page_size,
                      int max_pages, int num_pages, int block, float scale, float lambda,
                      float eps, float out_scale, int* status) {
    extern __shared__ float smem[];
    __shared__ float scratch[32];
    float* qs = smem;                        // [2 * dim]
    float* w1 = qs + 2 * dim;                // [DA_SEG] weights of map 1
    float* w2 = w1 + DA_SEG;                 // [DA_SEG]
    float* part = w2 + DA_SEG;               // [DA_THREADS * 2]
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
    const int lo = block > 0 ? (pos / block) * block : 0;
    const int n = pos - lo + 1;
    const int g = h / (heads / kv_heads);
    const int rowlen = 2 * dim + vdim;
    const int* table = block_table + (size_t)b * max_pages;
    const float* qp = q + ((size_t)t * heads + h) * 2 * dim;
    for (int i = threadIdx.x; i < 2 * dim; i += blockDim.x) qs[i] = qp[i];

    // thread (kg, j): value coordinates j, j + vthreads, ... of keys kg, kg + kgroups, ...
    const int vthreads = vdim < DA_THREADS ? vdim : DA_THREADS;
    const int kgroups = DA_THREADS / vthreads;
    const int vj = threadIdx.x % vthreads, kg = threadIdx.x / vthreads;
    const bool vlive = kg < kgroups;
    float acc1[DA_MAX_V], acc2[DA_MAX_V];
#pragma unroll
    for (int x = 0; x < DA_MAX_V; ++x) acc1[x] = acc2[x] = 0.0f;
    float m1 = -INFINITY, m2 = -INFINITY, l1 = 0.0f, l2 = 0.0f;
    __syncthreads();

    for (int s0 = 0; s0 < n; s0 += DA_SEG) {
        const int ns = min(DA_SEG, n - s0);
        float mx1 = -INFINITY, mx2 = -INFINITY;
        for (int i = threadIdx.x; i < ns; i += blockDim.x) {
            const int j = lo + s0 + i;
            const int page = table[j / page_size];
            float s1 = -INFINITY, s2 = -INFINITY;
            if (page < 0 || page >= num_pages) {
                prb_set_status(status, PRB_S_PAGE_RANGE, t, j, page);
            } else {
                const C* kp = cache + (((size_t)page * kv_heads + g) * page_size + (j % page_size)) * rowlen;
                float a1 = 0.0f, a2 = 0.0f;
                for (int d = 0; d < dim; ++d) {
                    a1 = fmaf(qs[d], prb_to_float<C>(kp[d]), a1);
                    a2 = fmaf(qs[dim + d], prb_to_float<C>(kp[dim + d]), a2);
                }
                s1 = a1 * scale;
                s2 = a2 * scale;
            }
            w1[i] = s1;
            w2[i] = s2;
            mx1 = fmaxf(mx1, s1);
            mx2 = fmaxf(mx2, s2);
        }
        mx1 = prb_block_max(mx1, scratch);
        mx2 = prb_block_max(mx2, scratch);
        const float n1 = fmaxf(m1, mx1), n2 = fmaxf(m2, mx2);
        // (a segment whose keys are all missing leaves the running state as it is)
        const float f1 = (n1 == -INFINITY) ? 1.0f : expf(m1 - n1);
        const float f2 = (n2 == -INFINITY) ? 1.0f : expf(m2 - n2);
        float sum1 = 0.0f, sum2 = 0.0f;
        for (int i = threadIdx.x; i < ns; i += blockDim.x) {
            const float e1 = (w1[i] == -INFINITY) ? 0.0f : expf(w1[i] - n1);
            const float e2 = (w2[i] == -INFINITY) ? 0.0f : expf(w2[i] - n2);
            w1[i] = e1;
            w2[i] = e2;
            sum1 += e1;
            sum2 += e2;
        }
        sum1 = prb_block_sum(sum1, scratch);
        sum2 = prb_block_sum(sum2, scratch);
        __syncthreads();                         // the weights are written
        l1 = l1 * f1 + sum1;
        l2 = l2 * f2 + sum2;
        m1 = n1;
        m2 = n2;
        if (vlive) {
#pragma unroll
            for (int x = 0; x < DA_MAX_V; ++x) {
                acc1[x] *= f1;
                acc2[x] *= f2;
            }
            for (int i = kg; i < ns; i += kgroups) {
                const float e1 = w1[i], e2 = w2[i];
                if (e1 == 0.0f && e2 == 0.0f) continue;
                const int j = lo + s0 + i;
                const int page = table[j / page_size];
                if (page < 0 || page >= num_pages) continue;
                const C* vp = cache + (((size_t)page * kv_heads + g) * page_size + (j % page_size)) * rowlen + 2 * dim;
#pragma unroll
                for (int x = 0; x < DA_MAX_V; ++x) {
                    const int jj = vj + x * vthreads;
                    if (jj < vdim) {
                        const float v = prb_to_float<C>(vp[jj]);
                        acc1[x] = fmaf(e1, v, acc1[x]);
                        acc2[x] = fmaf(e2, v, acc2[x]);
                    }
                }
            }
        }
        __syncthreads();                         // before the next segment overwrites the weights
    }

    // join the key groups in group order, combine the maps, unit RMS over the head
    float mine[DA_MAX_V];
    float ss = 0.0f;
#pragma unroll
    for (int x = 0; x < DA_MAX_V; ++x) {
        part[threadIdx.x * 2] = acc1[x];
        part[threadIdx.x * 2 + 1] = acc2[x];
        __syncthreads();
        mine[x] = 0.0f;
        const int jj = vj + x * vthreads;
        if (kg == 0 && jj < vdim) {
            float t1 = 0.0f, t2 = 0.0f;
            for (int gg = 0; gg < kgroups; ++gg) {
                t1 += part[(gg * vthreads + vj) * 2];
                t2 += part[(gg * vthreads + vj) * 2 + 1];
            }
            const float a1 = l1 > 0.0f ? t1 / l1 : 0.0f;
            const float a2 = l2 > 0.0f ? t2 / l2 : 0.0f;
            mine[x] = a1 - lambda * a2;
            ss = fmaf(mine[x], mine[x], ss);
        }
        __syncthreads();
    }
    ss = prb_block_sum(ss, scratch);
    const float inv = out_scale / sqrtf(ss / (float)vdim + eps);
#pragma unroll
    for (int x = 0; x < DA_MAX_V; ++x) {
        const int jj = vj + x * vthreads;
        if (kg == 0 && jj < vdim) o[jj] = prb_from_float<O>(mine[x] * inv);
    }
}
// ---------------------------------------------------------------------- the tiled kernel
// A CTA takes up to `tq` consecutive token rows of the step and ONE key/value head; the
// HG = heads / kv_heads query heads that share it ride together, so a key's row is fetched
// once for tq * HG (query, head) pairs.  Keys go in blocks of 32 ABSOLUTE positions (block m
// holds positions 32 m .. 32 m + 31, whatever the tile or the portion of the prompt), staged
// in shared memory as 32-bit numbers by coalesced loads; a warp owns up to DT_PPW pairs
// (pair x * DT_WARPS + warp: a single token's few pairs go to a warp each), a
// lane one key of the block for the two scores and vdim / 32 value coordinates for the sums.
// Running maxima and sums per map, 32-bit.  Which keys meet in which partial sum depends on
// absolute positions only: a query's result does not depend on the tile it falls in.
constexpr int DT_WARPS = 8;
constexpr int DT_PPW = 4;            // (query, head) pairs a warp owns
constexpr int DT_VC = 4;             // value coordinates a lane owns at most (vdim <= 128)
constexpr int DT_KB = 32;            // keys per block

template <typename C, typename O, int VC>
__global__ void __launch_bounds__(DT_WARPS * 32)
diff_attention_tile_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ q,
                           const C* __restrict__ cache, const int* __restrict__ block_table,
                           const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                           int n_tokens, int heads, int kv_heads, int dim, int vdim, int page_size,
                           int max_pages, int num_pages, int block, int tq, float scale,
                           float lambda, float eps, float out_scale, int* status) {
    extern __shared__ __align__(16) float smem[];
    __shared__ int pages_s[DT_KB];
    prb_grid_launch_dependents();
    const int hg = heads / kv_heads;
    const int g = blockIdx.y;
    const int rowlen = 2 * dim + vdim;
    const int kpitch = 2 * dim + 1;                  // odd: lanes read their own key's row
    float* Ks = smem;                                // [DT_KB][kpitch]
    float* Vs = Ks + DT_KB * kpitch;                 // [DT_KB][vdim]
    float* Qs = Vs + DT_KB * vdim;                   // [DT_WARPS * DT_PPW][2 * dim]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r_begin = blockIdx.x * tq;
    const int r_end = min(n_tokens, r_begin + tq);
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
        const int lo_min = block > 0 ? (p0 / block) * block : 0;
        const int* table = block_table + (size_t)b * max_pages;
        __syncthreads();                             // the pass before is done with shared memory
        // queries of this pass, scaled: pair = qi * hg + hh
        const int n_pairs = nq * hg;
        for (int e = threadIdx.x; e < n_pairs * 2 * dim; e += blockDim.x) {
            const int pair = e / (2 * dim), d = e - pair * 2 * dim;
            const int qi = pair / hg, hh = pair - qi * hg;
            Qs[pair * 2 * dim + d] = q[((size_t)(r + qi) * heads + g * hg + hh) * 2 * dim + d] * scale;
        }
        float acc1[DT_PPW][VC], acc2[DT_PPW][VC];
        float m1[DT_PPW], m2[DT_PPW], l1[DT_PPW], l2[DT_PPW];
#pragma unroll
        for (int x = 0; x < DT_PPW; ++x) {
            m1[x] = m2[x] = -INFINITY;
            l1[x] = l2[x] = 0.0f;
#pragma unroll
            for (int c = 0; c < VC; ++c) acc1[x][c] = acc2[x][c] = 0.0f;
        }
        for (int j0 = (lo_min / DT_KB) * DT_KB; j0 <= p_last; j0 += DT_KB) {
            __syncthreads();                         // the block before has been consumed
            // one page look-up per key, then the rows in 16-byte pieces (or element by element
            // where a row is no whole number of pieces): no load waits for another
            if (threadIdx.x < DT_KB) {
                const int jj = j0 + (int)threadIdx.x;
                int pg = -1;
                if (jj >= lo_min && jj <= p_last) {
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
            if (rowlen % VE == 0 && (2 * dim) % VE == 0) {
                const int nv = rowlen / VE;
#pragma unroll 2
                for (int e = threadIdx.x; e < DT_KB * nv; e += blockDim.x) {
                    const int kk = e / nv, vi = e - kk * nv;
                    const int pg = pages_s[kk];
                    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
                    if (pg >= 0)
                        raw = *reinterpret_cast<const uint4*>(
                            cache + (((size_t)pg * kv_heads + g) * page_size + ((j0 + kk) % page_size)) * rowlen + vi * VE);
                    const C* vals = reinterpret_cast<const C*>(&raw);
                    const int off = vi * VE;
                    float* dst = off < 2 * dim ? Ks + kk * kpitch + off : Vs + kk * vdim + off - 2 * dim;
#pragma unroll
                    for (int x = 0; x < VE; ++x) dst[x] = prb_to_float<C>(vals[x]);
                }
            } else {
                for (int e = threadIdx.x; e < DT_KB * rowlen; e += blockDim.x) {
                    const int kk = e / rowlen, off = e - kk * rowlen;
                    const int pg = pages_s[kk];
                    const float val = pg < 0 ? 0.0f : prb_to_float<C>(
                        cache[(((size_t)pg * kv_heads + g) * page_size + ((j0 + kk) % page_size)) * rowlen + off]);
                    if (off < 2 * dim) Ks[kk * kpitch + off] = val;
                    else Vs[kk * vdim + off - 2 * dim] = val;
                }
            }
            __syncthreads();
            // scores of this lane's key for all pairs of the warp: a key's numbers are loaded
            // once for the pairs, a pair's query in 16-byte pieces
            const int j = j0 + lane;
            const float* krow = Ks + lane * kpitch;
            bool act[DT_PPW];
            int last[DT_PPW], first[DT_PPW];
            float s1[DT_PPW], s2[DT_PPW];
            int k_hi = 0;
#pragma unroll
            for (int x = 0; x < DT_PPW; ++x) {
                const int pair = x * DT_WARPS + warp;
                const int pi = p0 + (pair < n_pairs ? pair / hg : 0);
                first[x] = block > 0 ? (pi / block) * block : 0;
                last[x] = pi;
                act[x] = pair < n_pairs && j0 <= pi && j0 + DT_KB > first[x];
                if (act[x]) k_hi = max(k_hi, min(DT_KB, pi - j0 + 1));
                s1[x] = s2[x] = 0.0f;
            }
            if (k_hi == 0) continue;                     // nothing of this block is seen by the warp
            if (dim % 4 == 0) {
                for (int d = 0; d < dim; d += 4) {
                    const float a0 = krow[d], a1 = krow[d + 1], a2 = krow[d + 2], a3 = krow[d + 3];
                    const float b0 = krow[dim + d], b1 = krow[dim + d + 1], b2 = krow[dim + d + 2],
                                b3 = krow[dim + d + 3];
#pragma unroll
                    for (int x = 0; x < DT_PPW; ++x) {
                        const float* qrow = Qs + (x * DT_WARPS + warp) * 2 * dim;
                        const float4 u = *reinterpret_cast<const float4*>(qrow + d);
                        const float4 w = *reinterpret_cast<const float4*>(qrow + dim + d);
                        s1[x] = fmaf(u.w, a3, fmaf(u.z, a2, fmaf(u.y, a1, fmaf(u.x, a0, s1[x]))));
                        s2[x] = fmaf(w.w, b3, fmaf(w.z, b2, fmaf(w.y, b1, fmaf(w.x, b0, s2[x]))));
                    }
                }
            } else {
                for (int d = 0; d < dim; ++d) {
                    const float a0 = krow[d], b0 = krow[dim + d];
#pragma unroll
                    for (int x = 0; x < DT_PPW; ++x) {
                        const float* qrow = Qs + (x * DT_WARPS + warp) * 2 * dim;
                        s1[x] = fmaf(qrow[d], a0, s1[x]);
                        s2[x] = fmaf(qrow[dim + d], b0, s2[x]);
                    }
                }
            }
            float e1[DT_PPW], e2[DT_PPW];
#pragma unroll
            for (int x = 0; x < DT_PPW; ++x) {
                e1[x] = e2[x] = 0.0f;
                if (!act[x]) continue;
                const bool vis = j >= first[x] && j <= last[x];
                const float t1 = vis ? s1[x] : -INFINITY, t2 = vis ? s2[x] : -INFINITY;
                const float n1 = fmaxf(m1[x], prb_warp_max(t1)), n2 = fmaxf(m2[x], prb_warp_max(t2));
                const float f1 = expf(m1[x] - n1), f2 = expf(m2[x] - n2);    // (exp(-inf) = 0)
                e1[x] = vis ? expf(t1 - n1) : 0.0f;
                e2[x] = vis ? expf(t2 - n2) : 0.0f;
                l1[x] = l1[x] * f1 + prb_warp_sum(e1[x]);
                l2[x] = l2[x] * f2 + prb_warp_sum(e2[x]);
                m1[x] = n1;
                m2[x] = n2;
#pragma unroll
                for (int c = 0; c < VC; ++c) {
                    acc1[x][c] *= f1;
                    acc2[x][c] *= f2;
                }
            }
            // weighted values: a key's value coordinates are loaded once for the pairs (keys a
            // pair does not see have weight zero)
            for (int kk = 0; kk < k_hi; ++kk) {
                float v[VC];
#pragma unroll
                for (int c = 0; c < VC; ++c) v[c] = (lane + 32 * c < vdim) ? Vs[kk * vdim + lane + 32 * c] : 0.0f;
#pragma unroll
                for (int x = 0; x < DT_PPW; ++x) {
                    const float w1 = __shfl_sync(0xffffffffu, e1[x], kk), w2 = __shfl_sync(0xffffffffu, e2[x], kk);
#pragma unroll
                    for (int c = 0; c < VC; ++c) {
                        acc1[x][c] = fmaf(w1, v[c], acc1[x][c]);
                        acc2[x][c] = fmaf(w2, v[c], acc2[x][c]);
                    }
                }
            }
        }
        // combine the maps, unit RMS over the head, write
#pragma unroll
        for (int x = 0; x < DT_PPW; ++x) {
            const int pair = x * DT_WARPS + warp;        // (few pairs spread over the warps)
            if (pair >= n_pairs) break;
            const int qi = pair / hg, hh = pair - qi * hg;
            float o[VC];
            float ss = 0.0f;
#pragma unroll
            for (int c = 0; c < VC; ++c) {
                const float a1 = l1[x] > 0.0f ? acc1[x][c] / l1[x] : 0.0f;
                const float a2 = l2[x] > 0.0f ? acc2[x][c] / l2[x] : 0.0f;
                o[c] = (lane + 32 * c < vdim) ? a1 - lambda * a2 : 0.0f;
                ss = fmaf(o[c], o[c], ss);
            }
            ss = prb_warp_sum(ss);
            const float inv = out_scale / sqrtf(ss / (float)vdim + eps);
            O* dst = out + (size_t)(r + qi) * out_ld + (size_t)(g * hg + hh) * vdim;
#pragma unroll
            for (int c = 0; c < VC; ++c)
                if (lane + 32 * c < vdim) dst[lane + 32 * c] = prb_from_float<O>(o[c] * inv);
        }
        r = r1 + 1;
    }
}
// ------------------------------------------------------------ single tokens (decoding)
// A CTA per (token, key/value head) (several where more than four query heads share the
// head); its few (query head) pairs ride together.  Keys go in
// super-blocks of nw * 32 ABSOLUTE positions, staged at once by all warps; warp w then takes the
// 32 keys w * 32 .. of the super-block for every pair, with a running state of its own, and the
// warps' states are joined in warp order at the end.  The order of every sum depends on
// absolute positions and nw only (nw: from the sizes alone).
template <typename C, typename O, int VC>
__global__ void __launch_bounds__(DT_WARPS * 32)
diff_attention_single_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ q,
                             const C* __restrict__ cache, const int* __restrict__ block_table,
                             const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                             int n_tokens, int heads, int kv_heads, int dim, int vdim, int page_size,
                             int max_pages, int num_pages, int block, float scale, float lambda,
                             float eps, float out_scale, int* status) {
    extern __shared__ __align__(16) float smem[];
    __shared__ int pages_s[DT_WARPS * DT_KB];
    prb_grid_launch_dependents();
    const int nw = blockDim.x >> 5;
    // (more than DT_PPW query heads a key/value head: several CTAs share the head, each with
    // up to DT_PPW of its query heads)
    const int per_kv = heads / kv_heads;
    const int parts = (per_kv + DT_PPW - 1) / DT_PPW;
    const int g = blockIdx.y / parts, part = blockIdx.y - g * parts, t = blockIdx.x;
    const int h0 = g * per_kv + part * DT_PPW;       // first query head of this CTA
    const int hg = min(DT_PPW, per_kv - part * DT_PPW);
    if (t >= n_tokens) return;
    const int rowlen = 2 * dim + vdim;
    const int kpitch = 2 * dim + 1;
    const int span = nw * DT_KB;
    float* Ks = smem;                                // [span][kpitch]
    float* Vs = Ks + span * kpitch;                  // [span][vdim]
    float* Qs = Vs + span * vdim;                    // [hg][2 * dim]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b = seq_of_token[t];
    const int pos = positions[t];
    if (b < 0 || pos < 0 || pos >= max_pages * page_size) {
        if (b >= 0 && threadIdx.x == 0)
            prb_set_status(status, PRB_S_POSITION_RANGE, t, pos, max_pages * page_size);
        for (int j = threadIdx.x; j < hg * vdim; j += blockDim.x)
            out[(size_t)t * out_ld + (size_t)h0 * vdim + j] = prb_from_float<O>(0.0f);
        return;
    }
    const int lo = block > 0 ? (pos / block) * block : 0;
    const int* table = block_table + (size_t)b * max_pages;
    for (int e = threadIdx.x; e < hg * 2 * dim; e += blockDim.x)
        Qs[e] = q[((size_t)t * heads + h0) * 2 * dim + e] * scale;
    float acc1[DT_PPW][VC], acc2[DT_PPW][VC];
    float m1[DT_PPW], m2[DT_PPW], l1[DT_PPW], l2[DT_PPW];
#pragma unroll
    for (int x = 0; x < DT_PPW; ++x) {
        m1[x] = m2[x] = -INFINITY;
        l1[x] = l2[x] = 0.0f;
#pragma unroll
        for (int c = 0; c < VC; ++c) acc1[x][c] = acc2[x][c] = 0.0f;
    }
    for (int j0 = (lo / span) * span; j0 <= pos; j0 += span) {
        __syncthreads();
        for (int kk = threadIdx.x; kk < span; kk += blockDim.x) {
            const int jj = j0 + kk;
            int pg = -1;
            if (jj >= lo && jj <= pos) {
                pg = table[jj / page_size];
                if (pg < 0 || pg >= num_pages) {
                    prb_set_status(status, PRB_S_PAGE_RANGE, t, jj, pg);
                    pg = -1;
                }
            }
            pages_s[kk] = pg;
        }
        __syncthreads();
        constexpr int VE = 16 / (int)sizeof(C);
        if (rowlen % VE == 0 && (2 * dim) % VE == 0) {
            const int nv = rowlen / VE;
#pragma unroll 4
            for (int e = threadIdx.x; e < span * nv; e += blockDim.x) {
                const int kk = e / nv, vi = e - kk * nv;
                const int pg = pages_s[kk];
                uint4 raw = make_uint4(0u, 0u, 0u, 0u);
                if (pg >= 0)
                    raw = *reinterpret_cast<const uint4*>(
                        cache + (((size_t)pg * kv_heads + g) * page_size + ((j0 + kk) % page_size)) * rowlen + vi * VE);
                const C* vals = reinterpret_cast<const C*>(&raw);
                const int off = vi * VE;
                float* dst = off < 2 * dim ? Ks + kk * kpitch + off : Vs + kk * vdim + off - 2 * dim;
#pragma unroll
                for (int x = 0; x < VE; ++x) dst[x] = prb_to_float<C>(vals[x]);
            }
        } else {
            for (int e = threadIdx.x; e < span * rowlen; e += blockDim.x) {
                const int kk = e / rowlen, off = e - kk * rowlen;
                const int pg = pages_s[kk];
                const float val = pg < 0 ? 0.0f : prb_to_float<C>(
                    cache[(((size_t)pg * kv_heads + g) * page_size + ((j0 + kk) % page_size)) * rowlen + off]);
                if (off < 2 * dim) Ks[kk * kpitch + off] = val;
                else Vs[kk * vdim + off - 2 * dim] = val;
            }
        }
        __syncthreads();
        const int jb = j0 + warp * DT_KB;            // this warp's 32 keys
        if (jb > pos || jb + DT_KB <= lo) continue;
        const int j = jb + lane;
        const bool vis = j >= lo && j <= pos;
        const float* krow = Ks + (warp * DT_KB + lane) * kpitch;
        const float* vblk = Vs + (size_t)warp * DT_KB * vdim;
        const int k_hi = min(DT_KB, pos - jb + 1);
        // scores of this lane's key for all pairs: the key's numbers are loaded once, a pair's
        // query in 16-byte pieces
        float s1[DT_PPW], s2[DT_PPW];
#pragma unroll
        for (int x = 0; x < DT_PPW; ++x) s1[x] = s2[x] = 0.0f;
        if (dim % 4 == 0) {
            for (int d = 0; d < dim; d += 4) {
                const float a0 = krow[d], a1 = krow[d + 1], a2 = krow[d + 2], a3 = krow[d + 3];
                const float b0 = krow[dim + d], b1 = krow[dim + d + 1], b2 = krow[dim + d + 2],
                            b3 = krow[dim + d + 3];
#pragma unroll
                for (int x = 0; x < DT_PPW; ++x) {
                    if (x < hg) {
                        const float* qrow = Qs + x * 2 * dim;
                        const float4 u = *reinterpret_cast<const float4*>(qrow + d);
                        const float4 w = *reinterpret_cast<const float4*>(qrow + dim + d);
                        s1[x] = fmaf(u.w, a3, fmaf(u.z, a2, fmaf(u.y, a1, fmaf(u.x, a0, s1[x]))));
                        s2[x] = fmaf(w.w, b3, fmaf(w.z, b2, fmaf(w.y, b1, fmaf(w.x, b0, s2[x]))));
                    }
                }
            }
        } else {
            for (int d = 0; d < dim; ++d) {
                const float a0 = krow[d], b0 = krow[dim + d];
#pragma unroll
                for (int x = 0; x < DT_PPW; ++x) {
                    if (x < hg) {
                        s1[x] = fmaf(Qs[x * 2 * dim + d], a0, s1[x]);
                        s2[x] = fmaf(Qs[x * 2 * dim + dim + d], b0, s2[x]);
                    }
                }
            }
        }
        float e1[DT_PPW], e2[DT_PPW];
#pragma unroll
        for (int x = 0; x < DT_PPW; ++x) {
            e1[x] = e2[x] = 0.0f;
            if (x >= hg) continue;
            const float t1 = vis ? s1[x] : -INFINITY, t2 = vis ? s2[x] : -INFINITY;
            const float n1 = fmaxf(m1[x], prb_warp_max(t1)), n2 = fmaxf(m2[x], prb_warp_max(t2));
            const float f1 = expf(m1[x] - n1), f2 = expf(m2[x] - n2);
            e1[x] = vis ? expf(t1 - n1) : 0.0f;
            e2[x] = vis ? expf(t2 - n2) : 0.0f;
            l1[x] = l1[x] * f1 + prb_warp_sum(e1[x]);
            l2[x] = l2[x] * f2 + prb_warp_sum(e2[x]);
            m1[x] = n1;
            m2[x] = n2;
#pragma unroll
            for (int c = 0; c < VC; ++c) {
                acc1[x][c] *= f1;
                acc2[x][c] *= f2;
            }
        }
        for (int kk = 0; kk < k_hi; ++kk) {
            float v[VC];
#pragma unroll
            for (int c = 0; c < VC; ++c) v[c] = (lane + 32 * c < vdim) ? vblk[kk * vdim + lane + 32 * c] : 0.0f;
#pragma unroll
            for (int x = 0; x < DT_PPW; ++x) {
                if (x < hg) {
                    const float w1 = __shfl_sync(0xffffffffu, e1[x], kk), w2 = __shfl_sync(0xffffffffu, e2[x], kk);
#pragma unroll
                    for (int c = 0; c < VC; ++c) {
                        acc1[x][c] = fmaf(w1, v[c], acc1[x][c]);
                        acc2[x][c] = fmaf(w2, v[c], acc2[x][c]);
                    }
                }
            }
        }
    }
    // join the warps' states in warp order: [warp][pair][m1, l1, m2, l2, acc1[vdim], acc2[vdim]]
    __syncthreads();
    const int rec = 4 + 2 * vdim;
    float* J = smem;
#pragma unroll
    for (int x = 0; x < DT_PPW; ++x) {
        if (x >= hg) break;
        float* mine = J + ((size_t)warp * hg + x) * rec;
        if (lane == 0) {
            mine[0] = m1[x]; mine[1] = l1[x]; mine[2] = m2[x]; mine[3] = l2[x];
        }
#pragma unroll
        for (int c = 0; c < VC; ++c)
            if (lane + 32 * c < vdim) {
                mine[4 + lane + 32 * c] = acc1[x][c];
                mine[4 + vdim + lane + 32 * c] = acc2[x][c];
            }
    }
    __syncthreads();
    for (int x = warp; x < hg; x += nw) {            // a pair a warp
        float M1 = -INFINITY, M2 = -INFINITY;
        for (int w = 0; w < nw; ++w) {
            const float* rcd = J + ((size_t)w * hg + x) * rec;
            M1 = fmaxf(M1, rcd[0]);
            M2 = fmaxf(M2, rcd[2]);
        }
        float L1 = 0.0f, L2 = 0.0f, a1[VC], a2[VC];
#pragma unroll
        for (int c = 0; c < VC; ++c) a1[c] = a2[c] = 0.0f;
        for (int w = 0; w < nw; ++w) {
            const float* rcd = J + ((size_t)w * hg + x) * rec;
            const float f1 = rcd[0] == -INFINITY ? 0.0f : expf(rcd[0] - M1);
            const float f2 = rcd[2] == -INFINITY ? 0.0f : expf(rcd[2] - M2);
            L1 = fmaf(rcd[1], f1, L1);
            L2 = fmaf(rcd[3], f2, L2);
#pragma unroll
            for (int c = 0; c < VC; ++c)
                if (lane + 32 * c < vdim) {
                    a1[c] = fmaf(rcd[4 + lane + 32 * c], f1, a1[c]);
                    a2[c] = fmaf(rcd[4 + vdim + lane + 32 * c], f2, a2[c]);
                }
        }
        float o[VC];
        float ss = 0.0f;
#pragma unroll
        for (int c = 0; c < VC; ++c) {
            const float u1 = L1 > 0.0f ? a1[c] / L1 : 0.0f;
            const float u2 = L2 > 0.0f ? a2[c] / L2 : 0.0f;
            o[c] = (lane + 32 * c < vdim) ? u1 - lambda * u2 : 0.0f;
            ss = fmaf(o[c], o[c], ss);
        }
        ss = prb_warp_sum(ss);
        const float inv = out_scale / sqrtf(ss / (float)vdim + eps);
        O* dst = out + (size_t)t * out_ld + (size_t)(h0 + x) * vdim;
#pragma unroll
        for (int c = 0; c < VC; ++c)
            if (lane + 32 * c < vdim) dst[lane + 32 * c] = prb_from_float<O>(o[c] * inv);
    }
}
}  // namespace

PRB_API int prb_diff_prepare(float* q_out, void* cache, const float* proj, long ld, int q_col,
                             int k_col, int v_col, const int* slots, const int* positions,
                             const float* freq, int n_tokens, int heads, int kv_heads, int dim,
                             int vdim, int rot_dims, int page_size, int num_pages, int cache_dtype,
                             int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || rot_dims < 0 || rot_dims > dim ||
        rot_dims % 2 != 0 || page_size <= 0)
        return PRB_E_SIZE;
    const int work = heads * 2 * dim;
    const int threads = work >= 256 ? 256 : ((work + 31) / 32) * 32;
    if (cache_dtype == PRB_F32)
        diff_prepare_kernel<float><<<n_tokens, threads, 0, stream>>>(
            q_out, (float*)cache, proj, ld, q_col, k_col, v_col, slots, positions, freq, n_tokens,
            heads, kv_heads, dim, vdim, rot_dims, page_size, num_pages, status);
    else if (cache_dtype == PRB_BF16)
        diff_prepare_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            q_out, (__nv_bfloat16*)cache, proj, ld, q_col, k_col, v_col, slots, positions, freq,
            n_tokens, heads, kv_heads, dim, vdim, rot_dims, page_size, num_pages, status);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_diff_attention(void* out, long out_ld, const float* q, const void* cache,
                               const int* block_table, const int* seq_of_token,
                               const int* positions, int n_tokens, int heads, int kv_heads, int dim,
                               int vdim, int page_size, int max_pages, int num_pages, int block,
                               float scale, float lambda, float eps, float out_scale,
                               int cache_dtype, int out_dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || heads > 65535 || kv_heads <= 0 || heads % kv_heads != 0 || dim <= 0 ||
        vdim <= 0 || vdim > DA_THREADS * DA_MAX_V || page_size <= 0 || max_pages <= 0 || block < 0)
        return PRB_E_SIZE;
    const size_t smem = (size_t)(2 * dim + 2 * DA_SEG + 2 * DA_THREADS) * sizeof(float);
    if (smem > 48 * 1024) return PRB_E_SIZE;
    dim3 grid(n_tokens, heads);
#define DIFF(CT, OT)                                                                            \
    diff_attention_kernel<CT, OT><<<grid, DA_THREADS, smem, stream>>>(                          \
        (OT*)out, out_ld, q, (const CT*)cache, block_table, seq_of_token, positions, n_tokens,   \
        heads, kv_heads, dim, vdim, page_size, max_pages, num_pages, block, scale, lambda, eps, \
        out_scale, status)
    if (cache_dtype == PRB_F32 && out_dtype == PRB_F32) DIFF(float, float);
    else if (cache_dtype == PRB_BF16 && out_dtype == PRB_BF16) DIFF(__nv_bfloat16, __nv_bfloat16);
    else return PRB_E_DTYPE;
#undef DIFF
    PRB_LAUNCH_CHECK();
    return 0;
}

// Rows a CTA of the tiled kernel takes (0: sizes it does not take; the kernel above runs then).
PRB_API int prb_diff_attention_tile_rows(int heads, int kv_heads, int dim, int vdim) {
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0) return 0;
    const int hg = heads / kv_heads;
    if (vdim > 32 * DT_VC || hg > DT_WARPS * DT_PPW || dim > 256) return 0;
    const size_t smem = (size_t)(DT_KB * (2 * dim + 1) + DT_KB * vdim + DT_WARPS * DT_PPW * 2 * dim) * sizeof(float);
    if (smem > 160 * 1024) return 0;
    return (DT_WARPS * DT_PPW) / hg;
}

PRB_API int prb_diff_attention_tile(void* out, long out_ld, const float* q, const void* cache,
                                    const int* block_table, const int* seq_of_token,
                                    const int* positions, int n_tokens, int heads, int kv_heads,
                                    int dim, int vdim, int page_size, int max_pages, int num_pages,
                                    int block, int tq, float scale, float lambda, float eps,
                                    float out_scale, int cache_dtype, int out_dtype, int* status,
                                    cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int most = prb_diff_attention_tile_rows(heads, kv_heads, dim, vdim);
    if (most <= 0 || kv_heads > 65535 || page_size <= 0 || max_pages <= 0 || block < 0) return PRB_E_SIZE;
    if (tq <= 0 || tq > most) tq = most;
    const size_t smem = (size_t)(DT_KB * (2 * dim + 1) + DT_KB * vdim + DT_WARPS * DT_PPW * 2 * dim) * sizeof(float);
    dim3 grid((n_tokens + tq - 1) / tq, kv_heads);
#define DIFFT1(CT, OT, VCN)                                                                      \
    do {                                                                                         \
        if (smem > 40 * 1024)                                                                    \
            cudaFuncSetAttribute(diff_attention_tile_kernel<CT, OT, VCN>,                        \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
        diff_attention_tile_kernel<CT, OT, VCN><<<grid, DT_WARPS * 32, smem, stream>>>(          \
            (OT*)out, out_ld, q, (const CT*)cache, block_table, seq_of_token, positions,         \
            n_tokens, heads, kv_heads, dim, vdim, page_size, max_pages, num_pages, block, tq,    \
            scale, lambda, eps, out_scale, status);                                              \
    } while (0)
#define DIFFT(CT, OT)                                                                            \
    do {                                                                                         \
        switch ((vdim + 31) / 32) {         /* value coordinates a lane owns */                  \
            case 1: DIFFT1(CT, OT, 1); break;                                                    \
            case 2: DIFFT1(CT, OT, 2); break;                                                    \
            case 3: DIFFT1(CT, OT, 3); break;                                                    \
            default: DIFFT1(CT, OT, 4); break;                                                   \
        }                                                                                        \
    } while (0)
    if (cache_dtype == PRB_F32 && out_dtype == PRB_F32) DIFFT(float, float);
    else if (cache_dtype == PRB_BF16 && out_dtype == PRB_BF16) DIFFT(__nv_bfloat16, __nv_bfloat16);
    else return PRB_E_DTYPE;
#undef DIFFT
#undef DIFFT1
    PRB_LAUNCH_CHECK();
    return 0;
}

// Warps of the single-token kernel for these sizes (0: it does not take them).
PRB_API int prb_diff_attention_single_warps(int heads, int kv_heads, int dim, int vdim) {
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0) return 0;
    const int hg = heads / kv_heads < DT_PPW ? heads / kv_heads : DT_PPW;
    if (vdim > 32 * DT_VC || dim > 256) return 0;
    const size_t fixed = (size_t)hg * 2 * dim * sizeof(float);
    const size_t per_warp = (size_t)DT_KB * (2 * dim + 1 + vdim) * sizeof(float);
    int nw = (int)((180 * 1024 - fixed) / per_warp);
    if (nw > DT_WARPS) nw = DT_WARPS;
    return nw < 1 ? 0 : nw;
}

PRB_API int prb_diff_attention_single(void* out, long out_ld, const float* q, const void* cache,
                                      const int* block_table, const int* seq_of_token,
                                      const int* positions, int n_tokens, int heads, int kv_heads,
                                      int dim, int vdim, int page_size, int max_pages,
                                      int num_pages, int block, float scale, float lambda,
                                      float eps, float out_scale, int cache_dtype, int out_dtype,
                                      int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int nw = prb_diff_attention_single_warps(heads, kv_heads, dim, vdim);
    if (nw <= 0 || kv_heads > 65535 || page_size <= 0 || max_pages <= 0 || block < 0) return PRB_E_SIZE;
    const int per_kv = heads / kv_heads;
    const int hg = per_kv < DT_PPW ? per_kv : DT_PPW;
    const int parts = (per_kv + DT_PPW - 1) / DT_PPW;
    if ((long)kv_heads * parts > 65535) return PRB_E_SIZE;
    size_t smem = (size_t)(nw * DT_KB * (2 * dim + 1 + vdim) + hg * 2 * dim) * sizeof(float);
    const size_t join = (size_t)nw * hg * (4 + 2 * vdim) * sizeof(float);
    if (join > smem) smem = join;
    dim3 grid(n_tokens, kv_heads * parts);
#define DIFFS1(CT, OT, VCN)                                                                      \
    do {                                                                                         \
        if (smem > 40 * 1024)                                                                    \
            cudaFuncSetAttribute(diff_attention_single_kernel<CT, OT, VCN>,                      \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
        diff_attention_single_kernel<CT, OT, VCN><<<grid, nw * 32, smem, stream>>>(              \
            (OT*)out, out_ld, q, (const CT*)cache, block_table, seq_of_token, positions,         \
            n_tokens, heads, kv_heads, dim, vdim, page_size, max_pages, num_pages, block, scale, \
            lambda, eps, out_scale, status);                                                     \
    } while (0)
#define DIFFS(CT, OT)                                                                            \
    do {                                                                                         \
        switch ((vdim + 31) / 32) {                                                              \
            case 1: DIFFS1(CT, OT, 1); break;                                                    \
            case 2: DIFFS1(CT, OT, 2); break;                                                    \
            case 3: DIFFS1(CT, OT, 3); break;                                                    \
            default: DIFFS1(CT, OT, 4); break;                                                   \
        }                                                                                        \
    } while (0)
    if (cache_dtype == PRB_F32 && out_dtype == PRB_F32) DIFFS(float, float);
    else if (cache_dtype == PRB_BF16 && out_dtype == PRB_BF16) DIFFS(__nv_bfloat16, __nv_bfloat16);
    else return PRB_E_DTYPE;
#undef DIFFS
#undef DIFFS1
    PRB_LAUNCH_CHECK();
    return 0;
}
