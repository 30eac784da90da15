// Time mixing with a decay per channel that depends on the token (the recurrence of RWKV-style
// layers) over a running 32-bit state per request.
//
// With h_t the mixer's input and h_(t-1) the previous token's (zeros at a sequence's start),
// every projection s reads its own blend  x_s = h_t + (h_(t-1) - h_t) * mu_s.  Per head, with
// r, k (dim numbers) and v (vdim numbers) per token and a decay w in (0, 1) per key channel,
//
//     o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t         S_t = diag(w_t) S_(t-1) + k_t v_t^T
//     w_t = exp(-exp(w0 + W2 tanh(lr_t)))               lr_t: a low-rank projection of x_w
//
// then each head's o is brought to unit root-mean-square, multiplied by a weight per channel,
// by silu(gate) and by a constant.
//
// tmix_shift: a CTA per token; writes the blends side by side, [T, n_mix * width], or (without
//   mu) the row beside its difference from the previous one, [h_t | h_(t-1) - h_t]: a blend's
//   projection is linear, W x_s = W h_t + (W diag(mu_s)) (h_(t-1) - h_t), so one product of that
//   pair with [W | W diag(mu_s)] of all projections serves them all.  The
//   previous row of a request's first token of the step is the request's state row (the
//   input of its last token so far), or zeros at position 0.
// tmix_scan: a CTA per (head, request, group of value columns).  A column of S is independent
//   of the others; its `dim` numbers are spread over L neighbouring lanes (up to 16 numbers a
//   lane in registers; the dot with r is closed by shuffles).  Tokens come in chunks of 16 whose
//   r, k, v and decays (computed in 32-bit while loading) are staged in shared memory.  The state is zero at
//   position 0 (a slot's earlier owner is never read) and goes back to the slot at the end; the
//   request's last input row is saved for the next step's shift.
// tmix_finish: a warp per (token, head).
// Everything here is 32-bit arithmetic; the order of every sum depends on the sizes only.
#include "common.cuh"

namespace {
constexpr int TM_CHUNK = 16;         // tokens staged at a time
constexpr int TM_KPL = 16;           // numbers of a column a lane holds at most

__device__ __forceinline__ float tm_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename A>
__global__ void tmix_shift_kernel(A* __restrict__ out, long out_ld, const A* __restrict__ h,
                                  long h_ld, const A* __restrict__ prev_state,
                                  const float* __restrict__ mu, const int* __restrict__ seq_of_token,
                                  const int* __restrict__ positions, const int* __restrict__ q_start,
                                  const int* __restrict__ state_slot, int n_tokens, int width,
                                  int n_mix, int n_slots, int* status) {
    prb_grid_launch_dependents();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int b = seq_of_token[t];
    A* o = out + (size_t)t * out_ld;
    if (b < 0) {
        for (int i = threadIdx.x; i < n_mix * width; i += blockDim.x) o[i] = prb_from_float<A>(0.0f);
        return;
    }
    const A* cur = h + (size_t)t * h_ld;
    const A* prev = nullptr;
    if (positions[t] > 0) {
        if (t > q_start[b]) {
            prev = h + (size_t)(t - 1) * h_ld;
        } else {
            const int slot = state_slot[b];
            if (slot < 0 || slot >= n_slots) {
                if (threadIdx.x == 0) prb_set_status(status, PRB_S_ROW_RANGE, t, slot, n_slots);
            } else {
                prev = prev_state + (size_t)slot * width;
            }
        }
    }
    if (mu == nullptr) {                             // [h_t | h_(t-1) - h_t]
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float c = prb_to_float<A>(cur[i]);
            o[i] = cur[i];
            o[(size_t)width + i] = prb_from_float<A>((prev ? prb_to_float<A>(prev[i]) : 0.0f) - c);
        }
        return;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float c = prb_to_float<A>(cur[i]);
        const float d = (prev ? prb_to_float<A>(prev[i]) : 0.0f) - c;
        for (int s = 0; s < n_mix; ++s)
            o[(size_t)s * width + i] = prb_from_float<A>(fmaf(d, mu[(size_t)s * width + i], c));
    }
}

// The finish inside the scan (out == nullptr: the scan writes raw sums and tmix_finish follows).
template <typename A>
struct TmFinish {
    A* out;
    long out_ld;
    int g_col;
    const float* norm_w;
    float eps, out_scale;
};

template <typename A>
__global__ void __launch_bounds__(1024)
tmix_scan_kernel(float* __restrict__ raw, long raw_ld, const float* __restrict__ proj, long ld,
                 int r_col, int k_col, int v_col, int lr_col, const float* __restrict__ w2,
                 const float* __restrict__ w0, const float* __restrict__ u,
                 float* __restrict__ state, const A* __restrict__ h, long h_ld,
                 A* __restrict__ prev_state, const int* __restrict__ q_start,
                 const int* __restrict__ state_slot, const int* __restrict__ positions,
                 int n_requests, int heads, int dim, int vdim, int rank, int width, int lanes,
                 int cols, int n_slots, int* status, TmFinish<A> fin) {
    extern __shared__ float sm[];
    float* r_s = sm;                                 // [TM_CHUNK][dim]
    float* k_s = r_s + TM_CHUNK * dim;
    float* w_s = k_s + TM_CHUNK * dim;
    float* v_s = w_s + TM_CHUNK * dim;               // [TM_CHUNK][vdim]
    float* th_s = v_s + TM_CHUNK * vdim;             // [TM_CHUNK][rank]
    float* o_s = th_s + TM_CHUNK * rank;             // [TM_CHUNK][vdim], with the finish inside
    prb_grid_launch_dependents();
    const int hd = blockIdx.x, b = blockIdx.y, cg = blockIdx.z;
    if (b >= n_requests) return;
    const int t0 = q_start[b], t1 = q_start[b + 1];
    if (t1 <= t0) return;
    const int slot = state_slot[b];
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) prb_set_status(status, PRB_S_ROW_RANGE, t0, slot, n_slots);
        return;
    }
    const int ln = threadIdx.x % lanes, cl = threadIdx.x / lanes;
    const int c = cg * cols + cl;                    // this thread's value column
    const bool live = cl < cols && c < vdim;
    const int kpl = (dim + lanes - 1) / lanes;
    float S[TM_KPL], uu[TM_KPL];
    float* sp = state + (((size_t)slot * heads + hd) * vdim + (live ? c : 0)) * dim;
    const bool fresh = positions[t0] == 0;
#pragma unroll
    for (int i = 0; i < TM_KPL; ++i) {
        const int kk = ln + i * lanes;
        const bool ok = live && i < kpl && kk < dim;
        S[i] = (ok && !fresh) ? sp[kk] : 0.0f;
        uu[i] = ok ? u[(size_t)hd * dim + kk] : 0.0f;
    }
    for (int c0 = t0; c0 < t1; c0 += TM_CHUNK) {
        const int nt = min(TM_CHUNK, t1 - c0);
        __syncthreads();                             // the chunk before has been consumed
        for (int e = threadIdx.x; e < nt * rank; e += blockDim.x) {
            const int tt = e / rank, j = e - tt * rank;
            th_s[e] = tanhf(proj[(size_t)(c0 + tt) * ld + lr_col + j]);
        }
        for (int e = threadIdx.x; e < nt * dim; e += blockDim.x) {
            const int tt = e / dim, kk = e - tt * dim;
            const float* row = proj + (size_t)(c0 + tt) * ld + (size_t)hd * dim + kk;
            r_s[e] = row[r_col];
            k_s[e] = row[k_col];
        }
        for (int e = threadIdx.x; e < nt * vdim; e += blockDim.x) {
            const int tt = e / vdim, j = e - tt * vdim;
            v_s[e] = proj[(size_t)(c0 + tt) * ld + v_col + (size_t)hd * vdim + j];
        }
        __syncthreads();
        for (int e = threadIdx.x; e < nt * dim; e += blockDim.x) {
            const int tt = e / dim, kk = e - tt * dim;
            const int ch = hd * dim + kk;
            const float* wr = w2 + (size_t)ch * rank;
            float z = w0[ch];
            for (int j = 0; j < rank; ++j) z = fmaf(wr[j], th_s[tt * rank + j], z);
            w_s[e] = expf(-expf(z));
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float vc = live ? v_s[tt * vdim + c] : 0.0f;
            float part = 0.0f;
#pragma unroll
            for (int i = 0; i < TM_KPL; ++i) {
                const int kk = ln + i * lanes;
                if (i < kpl && kk < dim) {
                    const float kv = k_s[tt * dim + kk] * vc;
                    part = fmaf(r_s[tt * dim + kk], fmaf(uu[i], kv, S[i]), part);
                    S[i] = fmaf(w_s[tt * dim + kk], S[i], kv);
                }
            }
            for (int o = lanes >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            if (live && ln == 0) {
                if (fin.out) o_s[tt * vdim + c] = part;
                else raw[(size_t)(c0 + tt) * raw_ld + (size_t)hd * vdim + c] = part;
            }
        }
        if (fin.out) {
            // the CTA holds all of the head's columns: unit RMS, weight, gate and the
            // activation type here, a warp per token (the sums of tmix_finish, in its order)
            __syncthreads();
            const int lane = threadIdx.x & 31;
            for (int tt = threadIdx.x >> 5; tt < nt; tt += blockDim.x >> 5) {
                const float* src = o_s + tt * vdim;
                float ss = 0.0f;
                for (int j = lane; j < vdim; j += 32) ss = fmaf(src[j], src[j], ss);
                ss = prb_warp_sum(ss);
                const float inv = fin.out_scale / sqrtf(ss / (float)vdim + fin.eps);
                const float* gp = proj + (size_t)(c0 + tt) * ld + fin.g_col + (size_t)hd * vdim;
                A* o = fin.out + (size_t)(c0 + tt) * fin.out_ld + (size_t)hd * vdim;
                for (int j = lane; j < vdim; j += 32) {
                    const float gz = gp[j];
                    o[j] = prb_from_float<A>(src[j] * inv * fin.norm_w[(size_t)hd * vdim + j] *
                                             (gz * tm_sigmoid(gz)));
                }
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < TM_KPL; ++i) {
            const int kk = ln + i * lanes;
            if (i < kpl && kk < dim) sp[kk] = S[i];
        }
    }
    if (hd == 0 && cg == 0) {                        // the request's last input row, for the next shift
        const A* last = h + (size_t)(t1 - 1) * h_ld;
        A* dst = prev_state + (size_t)slot * width;
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = last[i];
    }
}


// ------------------------------------------------------------- long portions in segments
// Portions are cut into segments of TS_SEG tokens that run side by side:
//   tmix_decay:        w_t = exp(-exp(w0 + W2 tanh(lr_t))) of every token into a buffer of its own;
//   pass 1 (MODE 1):   every segment but a request's last builds, from zero, what its own tokens
//                      add to the state, and the product of its decays per key channel;
//   pass 2 (carry):    per request the states at the segments' starts, one after the other:
//                      U_0 = the carried state (zero at position 0), U_(s+1) = diag(product of
//                      segment s's decays) U_s + (pass 1 of segment s);
//   pass 3 (MODE 2):   every segment runs the recurrence from its U_s with outputs; a request's
//                      last segment leaves the state in the slot and saves the last input row.
// Segment z of the launch is segment s of request b: requests' segments are numbered in request
// order.  A lane holds KPL neighbouring numbers of its column.
constexpr int TS_SEG = 64;
constexpr int TS_BLOCK = 16;         // tokens staged at a time

struct SegArgs {
    float* raw; long raw_ld;
    const float* proj; long ld;
    int r_col, k_col, v_col, lr_col;
    float* decay; long decay_ld;                     // [T, heads * dim]: the decays of every token
    const float* w2; const float* w0; const float* u;
    float* state;
    const void* h; long h_ld; void* prev_state;
    const int* q_start; const int* state_slot; const int* positions;
    int n_tokens, n_requests, heads, dim, vdim, rank, width, lanes, cols, n_slots;
    float* seg_own; float* seg_start; float* seg_decay;
    int* status;
};

__device__ __forceinline__ bool tm_find_segment(const int* q_start, int n_requests, int z, int& b,
                                                int& s, int& nseg) {
    int base = 0;
    for (b = 0; b < n_requests; ++b) {
        const int n = q_start[b + 1] - q_start[b];
        nseg = n > 0 ? (n + TS_SEG - 1) / TS_SEG : 0;
        if (z < base + nseg) {
            s = z - base;
            return true;
        }
        base += nseg;
    }
    return false;
}

// A CTA per TD_TOKENS tokens: their low-rank rows' tanh in shared memory; a thread per channel
// holds nothing but walks its row of W2 once per token (the row stays in L1 for the CTA's tokens).
constexpr int TD_TOKENS = 8;
__global__ void tmix_decay_kernel(SegArgs a) {
    extern __shared__ float th[];                    // [TD_TOKENS][rank]
    prb_grid_launch_dependents();
    const int t0 = blockIdx.x * TD_TOKENS;
    const int nt = min(TD_TOKENS, a.n_tokens - t0);
    for (int e = threadIdx.x; e < nt * a.rank; e += blockDim.x) {
        const int tt = e / a.rank, j = e - tt * a.rank;
        th[e] = tanhf(a.proj[(size_t)(t0 + tt) * a.ld + a.lr_col + j]);
    }
    __syncthreads();
    for (int ch = threadIdx.x; ch < a.heads * a.dim; ch += blockDim.x) {
        const float* wr = a.w2 + (size_t)ch * a.rank;
        const float z0 = a.w0[ch];
        float z[TD_TOKENS];
#pragma unroll
        for (int tt = 0; tt < TD_TOKENS; ++tt) z[tt] = z0;
        for (int j = 0; j < a.rank; ++j) {
            const float wj = wr[j];
#pragma unroll
            for (int tt = 0; tt < TD_TOKENS; ++tt)
                if (tt < nt) z[tt] = fmaf(wj, th[tt * a.rank + j], z[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < TD_TOKENS; ++tt)
            if (tt < nt) a.decay[(size_t)(t0 + tt) * a.decay_ld + ch] = expf(-expf(z[tt]));
    }
}

constexpr int ts_threads(int kpl) { return kpl >= 8 ? 512 : 1024; }

template <typename A, int KPL, int MODE>
__global__ void __launch_bounds__(ts_threads(KPL)) tmix_seg_kernel(SegArgs a) {
    extern __shared__ __align__(16) float sm[];
    prb_grid_launch_dependents();
    const int hd = blockIdx.x, cg = blockIdx.z;
    int b, s, nseg;
    if (!tm_find_segment(a.q_start, a.n_requests, blockIdx.y, b, s, nseg)) return;
    int t0 = a.q_start[b], t1 = a.q_start[b + 1];
    if (t0 < 0 || t1 > a.n_tokens) return;
    const bool last = s == nseg - 1;
    if (MODE == 1 && last) return;                   // (a last segment's own sum is never needed)
    const int slot = a.state_slot[b];
    if (slot < 0 || slot >= a.n_slots) {
        if (MODE == 2 && threadIdx.x == 0) prb_set_status(a.status, PRB_S_ROW_RANGE, t0, slot, a.n_slots);
        return;
    }
    const int t_end = t1;
    t0 += s * TS_SEG;
    t1 = min(t1, t0 + TS_SEG);
    const int L = a.lanes, dim_pad = L * KPL, dim = a.dim, vdim = a.vdim, cols = a.cols;
    float* r_s = sm;                                 // [TS_BLOCK][dim_pad]
    float* k_s = r_s + TS_BLOCK * dim_pad;
    float* w_s = k_s + TS_BLOCK * dim_pad;
    float* v_s = w_s + TS_BLOCK * dim_pad;           // [TS_BLOCK][cols]
    const int ln = threadIdx.x % L, cl = threadIdx.x / L;
    const int c = cg * cols + cl;
    const bool live = cl < cols && c < vdim;
    const size_t per_head = (size_t)vdim * dim, per_state = (size_t)a.heads * per_head;
    const size_t column = ((size_t)hd * vdim + (live ? c : 0)) * dim;
    float S[KPL], uu[KPL], Pd[KPL];
    {
        const float* from = MODE == 2 ? a.seg_start + (size_t)blockIdx.y * per_state + column : nullptr;
#pragma unroll
        for (int i = 0; i < KPL; ++i) {
            const int kk = ln * KPL + i;
            S[i] = (live && from != nullptr && kk < dim) ? from[kk] : 0.0f;
            uu[i] = (MODE == 2 && kk < dim) ? a.u[(size_t)hd * dim + kk] : 0.0f;
            Pd[i] = 1.0f;
        }
    }
    for (int tb = t0; tb < t1; tb += TS_BLOCK) {
        const int nb = min(TS_BLOCK, t1 - tb);
        __syncthreads();                             // the block before has been consumed
        for (int e = threadIdx.x; e < nb * dim_pad; e += blockDim.x) {
            const int tok = e / dim_pad, kk = e - tok * dim_pad;
            float rr = 0.0f, kx = 0.0f, ww = 0.0f;
            if (kk < dim) {
                const float* row = a.proj + (size_t)(tb + tok) * a.ld + (size_t)hd * dim + kk;
                if (MODE == 2) rr = row[a.r_col];
                kx = row[a.k_col];
                ww = a.decay[(size_t)(tb + tok) * a.decay_ld + (size_t)hd * dim + kk];
            }
            r_s[e] = rr;
            k_s[e] = kx;
            w_s[e] = ww;
        }
        for (int e = threadIdx.x; e < nb * cols; e += blockDim.x) {
            const int tok = e / cols, cc = e - tok * cols;
            const int vc = cg * cols + cc;
            v_s[e] = vc < vdim ? a.proj[(size_t)(tb + tok) * a.ld + a.v_col + (size_t)hd * vdim + vc] : 0.0f;
        }
        __syncthreads();
#pragma unroll 2
        for (int tok = 0; tok < nb; ++tok) {
            const float v = cl < cols ? v_s[tok * cols + cl] : 0.0f;
            const float4* k4 = reinterpret_cast<const float4*>(k_s + tok * dim_pad + ln * KPL);
            const float4* w4 = reinterpret_cast<const float4*>(w_s + tok * dim_pad + ln * KPL);
            const float4* r4 = reinterpret_cast<const float4*>(r_s + tok * dim_pad + ln * KPL);
            float part = 0.0f;
#pragma unroll
            for (int g = 0; g < KPL / 4; ++g) {      // (sums in an order that dim alone fixes)
                const float4 kk = k4[g], ww = w4[g];
                const float kv0 = kk.x * v, kv1 = kk.y * v, kv2 = kk.z * v, kv3 = kk.w * v;
                if (MODE == 2) {
                    const float4 rr = r4[g];
                    part = fmaf(rr.x, fmaf(uu[4 * g + 0], kv0, S[4 * g + 0]), part);
                    part = fmaf(rr.y, fmaf(uu[4 * g + 1], kv1, S[4 * g + 1]), part);
                    part = fmaf(rr.z, fmaf(uu[4 * g + 2], kv2, S[4 * g + 2]), part);
                    part = fmaf(rr.w, fmaf(uu[4 * g + 3], kv3, S[4 * g + 3]), part);
                }
                S[4 * g + 0] = fmaf(ww.x, S[4 * g + 0], kv0);
                S[4 * g + 1] = fmaf(ww.y, S[4 * g + 1], kv1);
                S[4 * g + 2] = fmaf(ww.z, S[4 * g + 2], kv2);
                S[4 * g + 3] = fmaf(ww.w, S[4 * g + 3], kv3);
                if (MODE == 1 && cl == 0) {
                    Pd[4 * g + 0] *= ww.x;
                    Pd[4 * g + 1] *= ww.y;
                    Pd[4 * g + 2] *= ww.z;
                    Pd[4 * g + 3] *= ww.w;
                }
            }
            if (MODE == 2) {
                for (int o = L >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                if (live && ln == 0) a.raw[(size_t)(tb + tok) * a.raw_ld + (size_t)hd * vdim + c] = part;
            }
        }
    }
    float* to = nullptr;
    if (MODE == 1) to = a.seg_own + (size_t)blockIdx.y * per_state + column;
    if (MODE == 2 && last) to = a.state + (size_t)slot * per_state + column;
    if (live && to != nullptr) {
#pragma unroll
        for (int i = 0; i < KPL; ++i) {
            const int kk = ln * KPL + i;
            if (kk < dim) to[kk] = S[i];
        }
    }
    if (MODE == 1 && cl == 0 && cg == 0) {
#pragma unroll
        for (int i = 0; i < KPL; ++i) {
            const int kk = ln * KPL + i;
            if (kk < dim) a.seg_decay[((size_t)blockIdx.y * a.heads + hd) * dim + kk] = Pd[i];
        }
    }
    if (MODE == 2 && last && hd == 0 && cg == 0) {   // the request's last input row, for the next shift
        const A* lastrow = (const A*)a.h + (size_t)(t_end - 1) * a.h_ld;
        A* dst = (A*)a.prev_state + (size_t)slot * a.width;
        for (int i = threadIdx.x; i < a.width; i += blockDim.x) dst[i] = lastrow[i];
    }
}

// Pass 2: a thread per state number of a (head, request), 1,024 numbers a CTA; the request's
// segments in order.
__global__ void tmix_carry_kernel(SegArgs a) {
    prb_grid_launch_dependents();
    const int hd = blockIdx.x, b = blockIdx.y;
    const int t0 = a.q_start[b], t1 = a.q_start[b + 1];
    if (t1 <= t0 || t0 < 0 || t1 > a.n_tokens) return;
    const int slot = a.state_slot[b];
    if (slot < 0 || slot >= a.n_slots) return;
    int base = 0;
    for (int bb = 0; bb < b; ++bb) {
        const int n = a.q_start[bb + 1] - a.q_start[bb];
        base += n > 0 ? (n + TS_SEG - 1) / TS_SEG : 0;
    }
    const int nseg = (t1 - t0 + TS_SEG - 1) / TS_SEG;
    const size_t per_head = (size_t)a.vdim * a.dim, per_state = (size_t)a.heads * per_head;
    const bool carried = a.positions[t0] > 0;
    for (size_t e = (size_t)blockIdx.z * 1024 + threadIdx.x;
         e < min(per_head, ((size_t)blockIdx.z + 1) * 1024); e += blockDim.x) {
        const size_t at = (size_t)hd * per_head + e;
        const int kk = (int)(e % a.dim);
        float S = carried ? a.state[(size_t)slot * per_state + at] : 0.0f;
        for (int s = 0; s < nseg; ++s) {
            a.seg_start[(size_t)(base + s) * per_state + at] = S;
            if (s + 1 < nseg)
                S = fmaf(a.seg_decay[((size_t)(base + s) * a.heads + hd) * a.dim + kk], S,
                         a.seg_own[(size_t)(base + s) * per_state + at]);
        }
    }
}

template <typename O>
__global__ void tmix_finish_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ raw,
                                   long raw_ld, const float* __restrict__ proj, long ld, int g_col,
                                   const float* __restrict__ norm_w,
                                   const int* __restrict__ seq_of_token, int n_tokens, int heads,
                                   int vdim, float eps, float out_scale) {
    prb_grid_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= n_tokens * heads) return;
    const int t = unit / heads, hd = unit - t * heads;
    O* o = out + (size_t)t * out_ld + (size_t)hd * vdim;
    if (seq_of_token[t] < 0) {
        for (int j = lane; j < vdim; j += 32) o[j] = prb_from_float<O>(0.0f);
        return;
    }
    const float* src = raw + (size_t)t * raw_ld + (size_t)hd * vdim;
    float ss = 0.0f;
    for (int j = lane; j < vdim; j += 32) ss = fmaf(src[j], src[j], ss);
    ss = prb_warp_sum(ss);
    const float inv = out_scale / sqrtf(ss / (float)vdim + eps);
    const float* gp = proj + (size_t)t * ld + g_col + (size_t)hd * vdim;
    for (int j = lane; j < vdim; j += 32) {
        const float gz = gp[j];
        o[j] = prb_from_float<O>(src[j] * inv * norm_w[(size_t)hd * vdim + j] * (gz * tm_sigmoid(gz)));
    }
}

int tm_lanes(int dim) {
    int lanes = 1;
    while (lanes < 32 && lanes * TM_KPL < dim) lanes *= 2;
    return lanes * TM_KPL >= dim ? lanes : 0;
}
}  // namespace

// Lanes a column of the state is spread over (0: the head size is beyond the kernel).
PRB_API int prb_tmix_lanes(int dim) { return dim > 0 ? tm_lanes(dim) : 0; }

PRB_API int prb_tmix_shift(void* out, long out_ld, const void* h, long h_ld, const void* prev_state,
                           const float* mu, const int* seq_of_token, const int* positions,
                           const int* q_start, const int* state_slot, int n_tokens, int width,
                           int n_mix, int n_slots, int dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || n_mix <= 0) return PRB_E_SIZE;
    if (dtype == PRB_F32)
        tmix_shift_kernel<float><<<n_tokens, 256, 0, stream>>>(
            (float*)out, out_ld, (const float*)h, h_ld, (const float*)prev_state, mu, seq_of_token,
            positions, q_start, state_slot, n_tokens, width, n_mix, n_slots, status);
    else if (dtype == PRB_BF16)
        tmix_shift_kernel<__nv_bfloat16><<<n_tokens, 256, 0, stream>>>(
            (__nv_bfloat16*)out, out_ld, (const __nv_bfloat16*)h, h_ld,
            (const __nv_bfloat16*)prev_state, mu, seq_of_token, positions, q_start, state_slot,
            n_tokens, width, n_mix, n_slots, status);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}

// 1 if the scan of a step takes the finish inside (a CTA holds all of a head's value columns).
PRB_API int prb_tmix_step_supports(int dim, int vdim) {
    const int lanes = dim > 0 ? tm_lanes(dim) : 0;
    return lanes > 0 && vdim > 0 && vdim * lanes <= 1024 ? 1 : 0;
}

// out != nullptr: the finish inside (unit RMS, weight, gate, constant; raw is not written).
PRB_API int prb_tmix_scan(float* raw, long raw_ld, const float* proj, long ld, int r_col, int k_col,
                          int v_col, int lr_col, const float* w2, const float* w0, const float* u,
                          float* state, const void* h, long h_ld, void* prev_state,
                          const int* q_start, const int* state_slot, const int* positions,
                          int n_requests, int heads, int dim, int vdim, int rank, int width,
                          int n_slots, int dtype, int* status, void* out, long out_ld, int g_col,
                          const float* norm_w, float eps, float out_scale, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    const int lanes = tm_lanes(dim);
    if (lanes == 0 || heads <= 0 || vdim <= 0 || rank <= 0 || n_requests > 65535) return PRB_E_SIZE;
    int cols = 1024 / lanes;
    if (cols > vdim) cols = vdim;
    const int groups = (vdim + cols - 1) / cols;
    if (out != nullptr && groups != 1) return PRB_E_SIZE;
    int threads = (cols * lanes + 31) / 32 * 32;
    const size_t smem = (size_t)TM_CHUNK * (3 * dim + 2 * vdim + rank) * sizeof(float);
    if (smem > 200 * 1024) return PRB_E_SIZE;
    dim3 grid(heads, n_requests, groups);
#define TSCAN(AT)                                                                                \
    do {                                                                                         \
        if (smem > 48 * 1024)                                                                    \
            cudaFuncSetAttribute(tmix_scan_kernel<AT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                     \
        TmFinish<AT> fin{(AT*)out, out_ld, g_col, norm_w, eps, out_scale};                       \
        tmix_scan_kernel<AT><<<grid, threads, smem, stream>>>(                                   \
            raw, raw_ld, proj, ld, r_col, k_col, v_col, lr_col, w2, w0, u, state, (const AT*)h,  \
            h_ld, (AT*)prev_state, q_start, state_slot, positions, n_requests, heads, dim, vdim, \
            rank, width, lanes, cols, n_slots, status, fin);                                     \
    } while (0)
    if (dtype == PRB_F32) TSCAN(float);
    else if (dtype == PRB_BF16) TSCAN(__nv_bfloat16);
    else return PRB_E_DTYPE;
#undef TSCAN
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_tmix_segment() { return TS_SEG; }
PRB_API int prb_tmix_max_segments(int t_cap, int b_cap) { return t_cap / TS_SEG + b_cap; }

// The scan of long portions in segments: four launches.  decay [n_tokens, decay_ld] receives the
// decays; seg_own and seg_start [segments, heads, vdim, dim], seg_decay [segments, heads, dim]
// are workspaces (segments >= prb_tmix_max_segments(n_tokens, n_requests)).
PRB_API int prb_tmix_scan_segments(float* raw, long raw_ld, const float* proj, long ld, int r_col,
                                   int k_col, int v_col, int lr_col, float* decay, long decay_ld,
                                   const float* w2,
                                   const float* w0, const float* u, float* state, const void* h,
                                   long h_ld, void* prev_state, const int* q_start,
                                   const int* state_slot, const int* positions, int n_tokens,
                                   int n_requests, int heads, int dim, int vdim, int rank, int width,
                                   int n_slots, int dtype, float* seg_own, float* seg_start,
                                   float* seg_decay, int segments, int* status,
                                   cudaStream_t stream) {
    if (n_requests <= 0 || n_tokens <= 0) return 0;
    if (heads <= 0 || dim <= 0 || dim > 512 || vdim <= 0 || rank <= 0 || n_requests > 65535)
        return PRB_E_SIZE;
    const int need = prb_tmix_max_segments(n_tokens, n_requests);
    if (segments < need || need > 65535) return PRB_E_SIZE;
    if (dtype != PRB_F32 && dtype != PRB_BF16) return PRB_E_DTYPE;
    // numbers of a column a lane holds: 4 while 32 lanes hold a column (measured at heads of
    // 64: own sums 45 us and outputs 101 us with 4 a lane, 68 and 109 us with 8)
    const int kpl = dim <= 128 ? 4 : dim <= 256 ? 8 : 16;
    int lanes = 1;
    while (lanes * kpl < dim) lanes *= 2;
    int cols = ts_threads(kpl) / lanes;
    if (cols > vdim) cols = vdim;
    const int groups = (vdim + cols - 1) / cols;
    const int threads = (cols * lanes + 31) / 32 * 32;
    const size_t smem = (size_t)TS_BLOCK * (3 * lanes * kpl + cols) * sizeof(float);
    SegArgs a{raw, raw_ld, proj, ld, r_col, k_col, v_col, lr_col, decay, decay_ld, w2, w0, u, state, h, h_ld,
              prev_state, q_start, state_slot, positions, n_tokens, n_requests, heads, dim, vdim,
              rank, width, lanes, cols, n_slots, seg_own, seg_start, seg_decay, status};
    tmix_decay_kernel<<<(n_tokens + TD_TOKENS - 1) / TD_TOKENS, 256,
                        (size_t)TD_TOKENS * rank * sizeof(float), stream>>>(a);
    PRB_LAUNCH_CHECK();
    const dim3 grid(heads, need, groups);
    const size_t per_head = (size_t)vdim * dim;
    const dim3 cgrid(heads, n_requests, (unsigned)((per_head + 1023) / 1024));
#define TSEG2(AT, K)                                                                             \
    do {                                                                                         \
        if (smem > 48 * 1024) {                                                                  \
            cudaFuncSetAttribute(tmix_seg_kernel<AT, K, 1>,                                      \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
            cudaFuncSetAttribute(tmix_seg_kernel<AT, K, 2>,                                      \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
        }                                                                                        \
        tmix_seg_kernel<AT, K, 1><<<grid, threads, smem, stream>>>(a);                           \
        tmix_carry_kernel<<<cgrid, 256, 0, stream>>>(a);                                         \
        tmix_seg_kernel<AT, K, 2><<<grid, threads, smem, stream>>>(a);                           \
    } while (0)
#define TSEG(AT)                                                                                 \
    do {                                                                                         \
        if (kpl == 4) TSEG2(AT, 4);                                                              \
        else if (kpl == 8) TSEG2(AT, 8);                                                         \
        else TSEG2(AT, 16);                                                                      \
    } while (0)
    if (dtype == PRB_F32) TSEG(float);
    else TSEG(__nv_bfloat16);
#undef TSEG
#undef TSEG2
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_tmix_finish(void* out, long out_ld, const float* raw, long raw_ld, const float* proj,
                            long ld, int g_col, const float* norm_w, const int* seq_of_token,
                            int n_tokens, int heads, int vdim, float eps, float out_scale,
                            int out_dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || vdim <= 0) return PRB_E_SIZE;
    const int warps = 8;
    const int blocks = (n_tokens * heads + warps - 1) / warps;
    if (out_dtype == PRB_F32)
        tmix_finish_kernel<float><<<blocks, warps * 32, 0, stream>>>(
            (float*)out, out_ld, raw, raw_ld, proj, ld, g_col, norm_w, seq_of_token, n_tokens, heads,
            vdim, eps, out_scale);
    else if (out_dtype == PRB_BF16)
        tmix_finish_kernel<__nv_bfloat16><<<blocks, warps * 32, 0, stream>>>(
            (__nv_bfloat16*)out, out_ld, raw, raw_ld, proj, ld, g_col, norm_w, seq_of_token, n_tokens,
            heads, vdim, eps, out_scale);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}
