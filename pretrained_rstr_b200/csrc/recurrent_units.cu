// Two recurrent mixers over a 32-bit state per request.  Everything that enters a recurrence
// here is 32-bit: gates, decays and their logarithms, exponentials, the states, unit norms.
//
// (1) A gated linear recurrence per channel (the recurrent block of Griffin-style layers):
//       u_t = conv(x)_t                      a causal convolution per channel, `taps` long
//       r_t = sigmoid(A_b u_t,b + a_b)       per block b of the channels, square matrices
//       i_t = sigmoid(B_b u_t,b + b_b)
//       log a_t = decay_c * r_t              decay_c = -const * softplus(lambda_c), given
//       S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t          (S_(-1) = 0)
//     (a_t travels as a_t - 1 = expm1(log a_t), 1 - a_t^2 is -(a_t - 1)(a_t + 1): both keep their
//     precision when a_t is close to one)
//       out_t = S_t * gelu_tanh(y_t)
//     lru_conv (a CTA per token; the taps before a portion's first token come from the
//     request's saved inputs), lru_gates (a CTA per (8 tokens, block): the two block matrices
//     in 32-bit FMA, a_t - 1 and the recurrence's input), lru_scan (a thread per (request,
//     channel) walks the request's tokens in order from and to the state slot, multiplies by
//     the other branch and brings the saved inputs up to date).
//
// (2) A matrix memory with exponential gates and a running maximum (mLSTM-style):
//       i_t = cap tanh(i'_t / cap), f_t = logsigmoid(cap tanh(f'_t / cap))     (cap 0: none)
//       m_t = max(f_t + m_(t-1), i_t)                                            (m_(-1) = 0)
//       S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T        (n_t likewise, k alone)
//       o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//     then a unit root-mean-square per head, a weight per coordinate and sigmoid(gate).
//     mmem_step: a CTA per (head, request) keeps S in shared memory and walks the request's
//     tokens of the step in order, from and to the state slot.
//
// A request's state is zero at position 0 (a slot's earlier owner is never read), so a
// prompt may be cut anywhere and decoding is the same kernels with one token.  The order of
// every sum depends on the sizes only, never on the cut or the batch.
#include "common.cuh"

namespace {
__device__ __forceinline__ float ru_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float ru_logsigmoid(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

// One step of S <- a S + input, given a - 1.  A decay close to one, rounded to 32 bits, is off
// by up to 3e-8, which is a relative error of 3e-8 / (1 - a) in how fast the state fades: over
// a thousand tokens at a = 0.999 a far token's weight would be off by 3e-5.  a - 1 = expm1(log
// a) keeps its full relative precision, so the decay travels as a - 1 and the step is taken as
// S + (input + (a - 1) S).
__device__ __forceinline__ float lru_decay(float s, float a_minus_1, float input) {
    return s + fmaf(a_minus_1, s, input);
}

// ------------------------------------------------------------------ (1) convolution
// conv_state: [slots, taps - 1, width], the branch's inputs (bias added) at the request's last
// taps - 1 positions, the latest last.
__global__ void lru_conv_kernel(float* __restrict__ u, const float* __restrict__ proj, long ld,
                                int x_col, const float* __restrict__ x_bias,
                                const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                                const float* __restrict__ conv_state,
                                const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                                const int* __restrict__ q_start, const int* __restrict__ state_slot,
                                int n_tokens, int width, int taps, int n_slots, int b_cap) {
    prb_grid_launch_dependents();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int b = seq_of_token[t];
    if (b < 0 || b >= b_cap) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) u[(size_t)t * width + c] = 0.0f;
        return;
    }
    const int p = positions[t];
    const int r0 = q_start[b];
    const int p0 = positions[r0];
    const int slot = state_slot[b];
    const bool has_slot = slot >= 0 && slot < n_slots;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = conv_b ? conv_b[c] : 0.0f;
        const float xb = x_bias ? x_bias[c] : 0.0f;
        for (int j = 0; j < taps; ++j) {
            const int d = taps - 1 - j;
            const int s = p - d;
            if (s < 0) continue;
            float xv = 0.0f;
            if (s >= p0) xv = proj[(size_t)(t - d) * ld + x_col + c] + xb;
            else if (has_slot) xv = conv_state[((size_t)slot * (taps - 1) + (taps - 1 - (p0 - s))) * width + c];
            acc = fmaf(conv_w[(size_t)c * taps + j], xv, acc);
        }
        u[(size_t)t * width + c] = acc;
    }
}

// ------------------------------------------------------------------------ (1) gates
constexpr int LRU_TOK = 8;
// wa_t, wi_t: [blocks, bw (in), bw (out)]; a_out[t, c] = a_t - 1; u[t, c] <- sqrt(1 - a^2) * i * u.
template <typename W>
__global__ void __launch_bounds__(128)
lru_gates_kernel(float* __restrict__ a_out, float* __restrict__ u, const W* __restrict__ wa_t,
                 const W* __restrict__ wi_t, const float* __restrict__ ba,
                 const float* __restrict__ bi, const float* __restrict__ decay, int n_tokens,
                 int width, int bw) {
    extern __shared__ float us[];                    // [LRU_TOK][bw]
    prb_grid_launch_dependents();
    const int t0 = blockIdx.x * LRU_TOK, blk = blockIdx.y;
    const int nt = min(LRU_TOK, n_tokens - t0);
    for (int e = threadIdx.x; e < LRU_TOK * bw; e += blockDim.x) {
        const int k = e / bw, i = e - k * bw;
        us[e] = k < nt ? u[(size_t)(t0 + k) * width + blk * bw + i] : 0.0f;
    }
    __syncthreads();
    const W* wa = wa_t + (size_t)blk * bw * bw;
    const W* wi = wi_t + (size_t)blk * bw * bw;
    for (int o = threadIdx.x; o < bw; o += blockDim.x) {
        float ra[LRU_TOK], ri[LRU_TOK];
#pragma unroll
        for (int k = 0; k < LRU_TOK; ++k) ra[k] = ri[k] = 0.0f;
#pragma unroll 4
        for (int i = 0; i < bw; ++i) {
            const float va = prb_to_float<W>(wa[(size_t)i * bw + o]);
            const float vi = prb_to_float<W>(wi[(size_t)i * bw + o]);
#pragma unroll
            for (int k = 0; k < LRU_TOK; ++k) {
                const float uu = us[k * bw + i];
                ra[k] = fmaf(va, uu, ra[k]);
                ri[k] = fmaf(vi, uu, ri[k]);
            }
        }
        const int c = blk * bw + o;
        const float dc = decay[c], bac = ba[c], bic = bi[c];
#pragma unroll
        for (int k = 0; k < LRU_TOK; ++k) {
            if (k >= nt) break;
            const float r = ru_sigmoid(ra[k] + bac), g = ru_sigmoid(ri[k] + bic);
            const float am1 = expm1f(dc * r);                    // a - 1 (log a = dc r <= 0); see lru_decay
            const float in = sqrtf(fmaxf(-am1 * (am1 + 2.0f), 0.0f)) * g * us[k * bw + o];   // 1 - a^2 = -(a - 1)(a + 1)
            a_out[(size_t)(t0 + k) * width + c] = am1;
            u[(size_t)(t0 + k) * width + c] = in;
        }
    }
}

// ------------------------------------------------------------------------- (1) scan
constexpr int LRU_MAX_TAPS = 16;
template <typename O>
__global__ void __launch_bounds__(128)
lru_scan_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ a_in,
                const float* __restrict__ in, const float* __restrict__ proj, long ld, int y_col,
                int x_col, const float* __restrict__ y_bias, const float* __restrict__ x_bias,
                float* __restrict__ state, float* __restrict__ conv_state,
                const int* __restrict__ q_start, const int* __restrict__ state_slot,
                const int* __restrict__ positions, int n_tokens, int n_slots, int width, int taps,
                float out_scale) {
    prb_grid_launch_dependents();
    const int b = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int r0 = q_start[b], r1 = min(q_start[b + 1], n_tokens);
    if (c >= width || r0 >= r1) return;
    const int slot = state_slot[b];
    const bool has_slot = slot >= 0 && slot < n_slots;
    const int p0 = positions[r0];
    float s = (p0 > 0 && has_slot) ? state[(size_t)slot * width + c] : 0.0f;
    const float yb = y_bias ? y_bias[c] : 0.0f;
#pragma unroll 4
    for (int r = r0; r < r1; ++r) {
        s = lru_decay(s, a_in[(size_t)r * width + c], in[(size_t)r * width + c]);
        const float y = prb_activate(proj[(size_t)r * ld + y_col + c] + yb, PRB_ACT_GELU_TANH);
        out[(size_t)r * out_ld + c] = prb_from_float<O>(s * y * out_scale);
    }
    if (!has_slot) return;
    state[(size_t)slot * width + c] = s;
    // the branch's inputs at the last taps - 1 positions: from the step's rows, or, where the
    // step brought fewer, from what was saved (read before anything is written)
    const int keep = taps - 1;
    const int n = r1 - r0;
    const float xb = x_bias ? x_bias[c] : 0.0f;
    float* cs = conv_state + (size_t)slot * keep * width + c;
    float old[LRU_MAX_TAPS];
#pragma unroll
    for (int k = 0; k < LRU_MAX_TAPS; ++k) old[k] = (k < keep && p0 > 0) ? cs[(size_t)k * width] : 0.0f;
#pragma unroll
    for (int k = 0; k < LRU_MAX_TAPS; ++k) {
        if (k >= keep) break;
        const int back = keep - k;                   // the value `back` positions before the end
        float v;
        if (back <= n) v = proj[(size_t)(r1 - back) * ld + x_col + c] + xb;
        else {
            const int ko = k + n;                    // (k + n < keep here)
            v = 0.0f;
#pragma unroll
            for (int z = 0; z < LRU_MAX_TAPS; ++z) if (z == ko) v = old[z];
        }
        cs[(size_t)k * width] = v;
    }
}

// ------------------------------------------------- (1) steps of few tokens: one launch
// A CTA per (request, block of channels), a thread per channel of the block: the convolution
// of up to LRU_TOK tokens into shared memory, the block matrices for those tokens (weights
// read once per group of tokens), then the recurrence over them in the thread's registers,
// from and to the slot; the saved inputs are brought up to date at the end.  The sums are those
// of the three kernels, in their order.
struct LruStepArgs {
    void* out; long out_ld;
    const float* proj; long ld; int y_col, x_col;
    const float* y_bias; const float* x_bias;
    const float* conv_w; const float* conv_b;
    const void* wa_t; const void* wi_t;
    const float* ba; const float* bi; const float* decay;
    float* state; float* conv_state;
    const int* q_start; const int* state_slot; const int* positions;
    int n_tokens, n_slots, width, bw, taps;
    float out_scale;
};

template <typename W, typename O>
__global__ void lru_step_kernel(LruStepArgs g) {
    extern __shared__ float us[];                    // [LRU_TOK][bw]
    prb_grid_launch_dependents();
    const int b = blockIdx.x, blk = blockIdx.y;
    const int r0 = g.q_start[b], r1 = min(g.q_start[b + 1], g.n_tokens);
    if (r0 >= r1 || r0 < 0) return;
    const int bw = g.bw, taps = g.taps, width = g.width;
    const int slot = g.state_slot[b];
    const bool has_slot = slot >= 0 && slot < g.n_slots;
    const int p0 = g.positions[r0];
    const int o = threadIdx.x;
    const bool live = o < bw;
    const int c = blk * bw + (live ? o : 0);
    const W* wa = reinterpret_cast<const W*>(g.wa_t) + (size_t)blk * bw * bw;
    const W* wi = reinterpret_cast<const W*>(g.wi_t) + (size_t)blk * bw * bw;
    O* out = reinterpret_cast<O*>(g.out);
    const float xb = g.x_bias ? g.x_bias[c] : 0.0f, yb = g.y_bias ? g.y_bias[c] : 0.0f;
    const float cb = g.conv_b ? g.conv_b[c] : 0.0f;
    const float dc = g.decay[c], bac = g.ba[c], bic = g.bi[c];
    const float* cs_old = g.conv_state + (size_t)(has_slot ? slot : 0) * (taps - 1) * width + c;
    float s = (live && p0 > 0 && has_slot) ? g.state[(size_t)slot * width + c] : 0.0f;
    for (int tb = r0; tb < r1; tb += LRU_TOK) {
        const int nt = min(LRU_TOK, r1 - tb);
        __syncthreads();                             // the group before has been consumed
        if (live) {
            for (int k = 0; k < nt; ++k) {
                const int t = tb + k, p = p0 + (t - r0);
                float acc = cb;
                for (int j = 0; j < taps; ++j) {
                    const int d = taps - 1 - j, sp = p - d;
                    if (sp < 0) continue;
                    float xv = 0.0f;
                    if (sp >= p0) xv = g.proj[(size_t)(t - d) * g.ld + g.x_col + c] + xb;
                    else if (has_slot) xv = cs_old[(size_t)(taps - 1 - (p0 - sp)) * width];
                    acc = fmaf(g.conv_w[(size_t)c * taps + j], xv, acc);
                }
                us[k * bw + o] = acc;
            }
            for (int k = nt; k < LRU_TOK; ++k) us[k * bw + o] = 0.0f;
        }
        __syncthreads();
        if (!live) continue;
        float ra[LRU_TOK], ri[LRU_TOK];
#pragma unroll
        for (int k = 0; k < LRU_TOK; ++k) ra[k] = ri[k] = 0.0f;
#pragma unroll 4
        for (int i = 0; i < bw; ++i) {
            const float va = prb_to_float<W>(wa[(size_t)i * bw + o]);
            const float vi = prb_to_float<W>(wi[(size_t)i * bw + o]);
#pragma unroll
            for (int k = 0; k < LRU_TOK; ++k) {
                const float uu = us[k * bw + i];
                ra[k] = fmaf(va, uu, ra[k]);
                ri[k] = fmaf(vi, uu, ri[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < LRU_TOK; ++k) {
            if (k >= nt) break;
            const float r = ru_sigmoid(ra[k] + bac), gi = ru_sigmoid(ri[k] + bic);
            const float am1 = expm1f(dc * r);                    // a - 1; 1 - a^2 = -(a - 1)(a + 1)
            const float in = sqrtf(fmaxf(-am1 * (am1 + 2.0f), 0.0f)) * gi * us[k * bw + o];
            s = lru_decay(s, am1, in);
            const float y = prb_activate(g.proj[(size_t)(tb + k) * g.ld + g.y_col + c] + yb, PRB_ACT_GELU_TANH);
            out[(size_t)(tb + k) * g.out_ld + c] = prb_from_float<O>(s * y * g.out_scale);
        }
    }
    // (the convolution read the saved inputs above; every thread of the CTA is past its last
    // read of its own channel's rows, which no other thread touches)
    if (!live || !has_slot) return;
    g.state[(size_t)slot * width + c] = s;
    const int keep = taps - 1, n = r1 - r0;
    float* cs = g.conv_state + (size_t)slot * keep * width + c;
    float old[LRU_MAX_TAPS];
#pragma unroll
    for (int k = 0; k < LRU_MAX_TAPS; ++k) old[k] = (k < keep && p0 > 0) ? cs[(size_t)k * width] : 0.0f;
#pragma unroll
    for (int k = 0; k < LRU_MAX_TAPS; ++k) {
        if (k >= keep) break;
        const int back = keep - k;
        float v;
        if (back <= n) v = g.proj[(size_t)(r1 - back) * g.ld + g.x_col + c] + xb;
        else {
            const int ko = k + n;
            v = 0.0f;
#pragma unroll
            for (int z = 0; z < LRU_MAX_TAPS; ++z) if (z == ko) v = old[z];
        }
        cs[(size_t)k * width] = v;
    }
}

// ------------------------------------------------- (1) long portions: the scan in segments
// Segment z of the launch is segment s of request b (numbered in request order).  Pass 1: a
// thread per (segment, channel) builds, from zero, what the segment's own tokens leave and the
// product of its decays minus one.  Pass 2: a thread per (segment, channel) first walks the request's
// earlier segments, U <- product U + own from the carried state, then runs its own tokens with
// outputs; a request's last segment leaves the state and the saved inputs in the slot.
constexpr int LRU_SEG = 64;
__device__ __forceinline__ bool lru_find_segment(const int* q_start, int n_requests, int z, int& b,
                                                 int& s, int& nseg, int& base) {
    base = 0;
    for (b = 0; b < n_requests; ++b) {
        const int n = q_start[b + 1] - q_start[b];
        nseg = n > 0 ? (n + LRU_SEG - 1) / LRU_SEG : 0;
        if (z < base + nseg) {
            s = z - base;
            return true;
        }
        base += nseg;
    }
    return false;
}

__global__ void __launch_bounds__(128)
lru_seg_own_kernel(float* __restrict__ seg_own, float* __restrict__ seg_keep,
                   const float* __restrict__ a_in, const float* __restrict__ in,
                   const int* __restrict__ q_start, int n_tokens, int n_requests, int width) {
    prb_grid_launch_dependents();
    int b, s, nseg, base;
    if (!lru_find_segment(q_start, n_requests, blockIdx.x, b, s, nseg, base)) return;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width || s == nseg - 1) return;         // (a last segment's own sum is never needed)
    const int t0 = q_start[b] + s * LRU_SEG, t1 = min(min(q_start[b + 1], n_tokens), t0 + LRU_SEG);
    float own = 0.0f, keep = 0.0f;                   // (keep: the decays' product MINUS ONE)
#pragma unroll 8
    for (int r = t0; r < t1; ++r) {
        const float am1 = a_in[(size_t)r * width + c];
        own = lru_decay(own, am1, in[(size_t)r * width + c]);
        keep = fmaf(keep, am1, keep + am1);          // (1 + keep)(1 + am1) - 1
    }
    seg_own[(size_t)blockIdx.x * width + c] = own;
    seg_keep[(size_t)blockIdx.x * width + c] = keep;
}

template <typename O>
__global__ void __launch_bounds__(128)
lru_seg_scan_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ a_in,
                    const float* __restrict__ in, const float* __restrict__ seg_own,
                    const float* __restrict__ seg_keep, const float* __restrict__ proj, long ld,
                    int y_col, int x_col, const float* __restrict__ y_bias,
                    const float* __restrict__ x_bias, float* __restrict__ state,
                    float* __restrict__ conv_state, const int* __restrict__ q_start,
                    const int* __restrict__ state_slot, const int* __restrict__ positions,
                    int n_tokens, int n_requests, int n_slots, int width, int taps,
                    float out_scale) {
    prb_grid_launch_dependents();
    int b, sg, nseg, base;
    if (!lru_find_segment(q_start, n_requests, blockIdx.x, b, sg, nseg, base)) return;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int r0 = q_start[b], r1 = min(q_start[b + 1], n_tokens);
    const int slot = state_slot[b];
    const bool has_slot = slot >= 0 && slot < n_slots;
    const int p0 = positions[r0];
    float s = (p0 > 0 && has_slot) ? state[(size_t)slot * width + c] : 0.0f;
    for (int z = 0; z < sg; ++z)
        s = lru_decay(s, seg_keep[(size_t)(base + z) * width + c], seg_own[(size_t)(base + z) * width + c]);
    const int t0 = r0 + sg * LRU_SEG, t1 = min(r1, t0 + LRU_SEG);
    const float yb = y_bias ? y_bias[c] : 0.0f;
#pragma unroll 8
    for (int r = t0; r < t1; ++r) {
        s = lru_decay(s, a_in[(size_t)r * width + c], in[(size_t)r * width + c]);
        const float y = prb_activate(proj[(size_t)r * ld + y_col + c] + yb, PRB_ACT_GELU_TANH);
        out[(size_t)r * out_ld + c] = prb_from_float<O>(s * y * out_scale);
    }
    if (!has_slot || sg != nseg - 1) return;
    state[(size_t)slot * width + c] = s;
    const int keep = taps - 1;
    const int n = r1 - r0;
    const float xb = x_bias ? x_bias[c] : 0.0f;
    float* cs = conv_state + (size_t)slot * keep * width + c;
    float old[LRU_MAX_TAPS];
#pragma unroll
    for (int k = 0; k < LRU_MAX_TAPS; ++k) old[k] = (k < keep && p0 > 0) ? cs[(size_t)k * width] : 0.0f;
#pragma unroll
    for (int k = 0; k < LRU_MAX_TAPS; ++k) {
        if (k >= keep) break;
        const int back = keep - k;
        float v;
        if (back <= n) v = proj[(size_t)(r1 - back) * ld + x_col + c] + xb;
        else {
            const int ko = k + n;
            v = 0.0f;
#pragma unroll
            for (int z = 0; z < LRU_MAX_TAPS; ++z) if (z == ko) v = old[z];
        }
        cs[(size_t)k * width] = v;
    }
}

// ------------------------------------------------------------------ (2) matrix memory
constexpr int MM_THREADS = 256;
struct MmemArgs {
    void* out; long out_ld;                       // [T, heads * vdim] in O
    const float* proj; long ld;                   // [T, ld]
    int q_col, k_col, v_col, i_col, f_col, g_col;
    const float* i_bias; const float* f_bias;     // [heads]
    const float* norm_w;                          // [heads * vdim]
    float* state_s;                               // [slots, heads, vdim, dim]
    float* state_n;                               // [slots, heads, dim]
    float* state_m;                               // [slots, heads]
    const int* q_start; const int* state_slot; const int* positions;
    int n_tokens, n_slots, heads, dim, vdim;
    float cap, q_scale, eps, out_scale;
};

template <typename O>
__global__ void __launch_bounds__(MM_THREADS) mmem_step_kernel(MmemArgs a) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float scratch[32];
    prb_grid_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y;
    const int dim = a.dim, vdim = a.vdim;
    const int r0 = a.q_start[b], r1 = min(a.q_start[b + 1], a.n_tokens);
    if (r0 >= r1) return;
    const int slot = a.state_slot[b];
    const bool has_slot = slot >= 0 && slot < a.n_slots;
    const bool carried = has_slot && a.positions[r0] > 0;
    const int vt = vdim < MM_THREADS ? vdim : MM_THREADS;     // columns a pass
    const int dsplit = MM_THREADS / vt;                       // parts of a column's sum
    float* S = sm;                                 // [dim][vdim]
    float* nn = S + (size_t)dim * vdim;            // [dim]
    float* qs = nn + dim;                          // [dim]
    float* ks = qs + dim;                          // [dim]
    float* vs = ks + dim;                          // [vdim]
    float* part = vs + vdim;                       // [dsplit][vdim]
    const int tid = threadIdx.x;
    const int vi = tid % vt, dj = tid / vt;
    const bool live = dj < dsplit;
    const size_t sh = ((size_t)(has_slot ? slot : 0) * a.heads + h);
    for (int e = tid; e < dim * vdim; e += MM_THREADS)          // (memory: [vdim][dim])
        S[(size_t)(e % dim) * vdim + e / dim] = carried ? a.state_s[sh * dim * vdim + e] : 0.0f;
    for (int e = tid; e < dim; e += MM_THREADS) nn[e] = carried ? a.state_n[sh * dim + e] : 0.0f;
    float m = carried ? a.state_m[sh] : 0.0f;
    O* out = reinterpret_cast<O*>(a.out);
    for (int r = r0; r < r1; ++r) {
        const float* row = a.proj + (size_t)r * a.ld;
        __syncthreads();                           // the token before is done with q, k, v
        for (int e = tid; e < dim; e += MM_THREADS) {
            qs[e] = row[a.q_col + h * dim + e] * a.q_scale;
            ks[e] = row[a.k_col + h * dim + e];
        }
        for (int e = tid; e < vdim; e += MM_THREADS) vs[e] = row[a.v_col + h * vdim + e];
        // the gates: every thread computes the same numbers
        float ig = row[a.i_col + h] + (a.i_bias ? a.i_bias[h] : 0.0f);
        float fg = row[a.f_col + h] + (a.f_bias ? a.f_bias[h] : 0.0f);
        if (a.cap > 0.0f) {
            ig = a.cap * tanhf(ig / a.cap);
            fg = a.cap * tanhf(fg / a.cap);
        }
        fg = ru_logsigmoid(fg);
        const float m_new = fmaxf(fg + m, ig);
        const float df = expf(fg + m - m_new), di = expf(ig - m_new);
        m = m_new;
        __syncthreads();
        float nq = 0.0f;
        for (int e = tid; e < dim; e += MM_THREADS) {
            const float v = fmaf(df, nn[e], di * ks[e]);
            nn[e] = v;
            nq = fmaf(v, qs[e], nq);
        }
        nq = prb_block_sum(nq, scratch);
        if (live) {
            for (int v = vi; v < vdim; v += vt) {
                const float dv = di * vs[v];
                float num = 0.0f;
                for (int d = dj; d < dim; d += dsplit) {
                    const float sv = fmaf(df, S[(size_t)d * vdim + v], ks[d] * dv);
                    S[(size_t)d * vdim + v] = sv;
                    num = fmaf(sv, qs[d], num);
                }
                part[dj * vdim + v] = num;
            }
        }
        __syncthreads();
        const float den = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
        float ss = 0.0f;
        for (int v = tid; v < vdim; v += MM_THREADS) {
            float num = part[v];
            for (int z = 1; z < dsplit; ++z) num += part[z * vdim + v];
            num /= den;
            vs[v] = num;                           // (v was consumed above)
            ss = fmaf(num, num, ss);
        }
        ss = prb_block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)vdim + a.eps);
        for (int v = tid; v < vdim; v += MM_THREADS) {
            const float g = ru_sigmoid(row[a.g_col + h * vdim + v]);
            out[(size_t)r * a.out_ld + h * vdim + v] =
                prb_from_float<O>(vs[v] * inv * a.norm_w[h * vdim + v] * g * a.out_scale);
        }
    }
    if (!has_slot) return;
    __syncthreads();
    for (int e = tid; e < dim * vdim; e += MM_THREADS)
        a.state_s[sh * dim * vdim + e] = S[(size_t)(e % dim) * vdim + e / dim];
    for (int e = tid; e < dim; e += MM_THREADS) a.state_n[sh * dim + e] = nn[e];
    if (tid == 0) a.state_m[sh] = m;
}

// ------------------------------------------------- (2) the matrix memory, long portions
// The gates first, for all tokens: the running maximum is a scalar recurrence per (head,
// request), so a CTA per (head, request) computes the capped gates of 128 tokens side by side,
// one thread walks the maximum through them, and all threads turn them into the token's
// factors (keep = exp(f + m_(t-1) - m_t), take = exp(i - m_t), floor = exp(-m_t)).  With the
// factors known, S and n follow a linear recurrence: a column of S (one value coordinate) is
// independent of the others and is spread over R neighbouring lanes (NI numbers a lane, in
// registers; every column's lanes keep a copy of n); the dots with q are closed by shuffles.
// Portions are cut into segments of 64 tokens that run side by side: pass 1 builds, from
// zero, what a segment's own tokens add and the product of its keep factors; pass 2 walks a
// request's segments in order, U_(s+1) = product_s U_s + own_s, from the carried state; pass 3
// runs every segment from its U_s with outputs, and a request's last segment leaves the state
// in the slot.  mmem_finish: a warp per (token, head): unit RMS, weight, sigmoid(gate).
constexpr int MS_BLOCK = 16;        // tokens staged at a time
constexpr int MS_SEG = 64;          // tokens of a segment
constexpr int MG_THREADS = 128;

struct MgateArgs {
    float* gates;                   // [T, heads, 4]: keep, take, floor
    const float* proj; long ld; int i_col, f_col;
    const float* i_bias; const float* f_bias;
    float* state_m;                 // [slots, heads]
    const int* q_start; const int* state_slot; const int* positions;
    int n_tokens, n_slots, heads;
    float cap;
};

__global__ void __launch_bounds__(MG_THREADS) mmem_gates_kernel(MgateArgs a) {
    __shared__ float ig_s[MG_THREADS], fg_s[MG_THREADS], m_s[MG_THREADS + 1];
    prb_grid_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y;
    const int t0 = a.q_start[b], t1 = min(a.q_start[b + 1], a.n_tokens);
    if (t1 <= t0 || t0 < 0) return;
    const int slot = a.state_slot[b];
    const bool has_slot = slot >= 0 && slot < a.n_slots;
    float m = (has_slot && a.positions[t0] > 0) ? a.state_m[(size_t)slot * a.heads + h] : 0.0f;
    const float ib = a.i_bias ? a.i_bias[h] : 0.0f, fb = a.f_bias ? a.f_bias[h] : 0.0f;
    for (int tb = t0; tb < t1; tb += MG_THREADS) {
        const int nb = min(MG_THREADS, t1 - tb);
        __syncthreads();
        if ((int)threadIdx.x < nb) {
            const float* row = a.proj + (size_t)(tb + threadIdx.x) * a.ld;
            float ig = row[a.i_col + h] + ib, fg = row[a.f_col + h] + fb;
            if (a.cap > 0.0f) {
                ig = a.cap * tanhf(ig / a.cap);
                fg = a.cap * tanhf(fg / a.cap);
            }
            ig_s[threadIdx.x] = ig;
            fg_s[threadIdx.x] = ru_logsigmoid(fg);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            m_s[0] = m;
            for (int k = 0; k < nb; ++k) m_s[k + 1] = fmaxf(fg_s[k] + m_s[k], ig_s[k]);
        }
        __syncthreads();
        if ((int)threadIdx.x < nb) {
            const float mp = m_s[threadIdx.x], mn = m_s[threadIdx.x + 1];
            float* g = a.gates + ((size_t)(tb + threadIdx.x) * a.heads + h) * 4;
            g[0] = expf(fg_s[threadIdx.x] + mp - mn);
            g[1] = expf(ig_s[threadIdx.x] - mn);
            g[2] = expf(-mn);
        }
        m = m_s[nb];
    }
    if (has_slot && threadIdx.x == 0) a.state_m[(size_t)slot * a.heads + h] = m;
}

struct MscanArgs {
    float* o_raw;                   // [T, heads * vdim]
    const float* proj; long ld; int q_col, k_col, v_col;
    const float* gates;             // [T, heads, 4]
    float* state_s;                 // [slots, heads, vdim, dim]
    float* state_n;                 // [slots, heads, dim]
    const int* q_start; const int* state_slot; const int* positions;
    int n_tokens, n_slots, heads, dim, vdim, cols, lanes;
    float q_scale;
    int n_requests, seg_len;        // seg_len 0: no segments
    float* seg_own_s; float* seg_start_s;     // [segments, heads, vdim, dim]
    float* seg_own_n; float* seg_start_n;     // [segments, heads, dim]
    float* seg_keep;                          // [segments, heads]
};

__device__ __forceinline__ bool ms_find_segment(const int* q_start, int n_requests, int seg_len,
                                                int z, int& b, int& s, int& nseg) {
    int base = 0;
    for (b = 0; b < n_requests; ++b) {
        const int n = q_start[b + 1] - q_start[b];
        nseg = n > 0 ? (n + seg_len - 1) / seg_len : 0;
        if (z < base + nseg) {
            s = z - base;
            return true;
        }
        base += nseg;
    }
    return false;
}

// MODE 0: a whole portion from and to the slot; 1: a segment's own sums from zero; 2: a
// segment from its start with outputs.
template <int NI, int MODE>
__global__ void mmem_scan_kernel(MscanArgs a) {
    extern __shared__ __align__(16) float smem[];
    prb_grid_launch_dependents();
    const int chunk = blockIdx.x, h = blockIdx.y;
    int b = blockIdx.z, s = 0, nseg = 1;
    if (MODE != 0 && !ms_find_segment(a.q_start, a.n_requests, a.seg_len, blockIdx.z, b, s, nseg)) return;
    int t0 = a.q_start[b], t1 = a.q_start[b + 1];
    if (t1 <= t0 || t0 < 0 || t1 > a.n_tokens) return;
    const bool carried = a.positions[t0] > 0;
    if (MODE != 0) {
        if (MODE == 1 && s == nseg - 1) return;      // (a last segment's own sum is never needed)
        t0 += s * a.seg_len;
        t1 = min(t1, t0 + a.seg_len);
    }
    const int R = a.lanes, dim_pad = R * NI;
    float* qs = smem;                               // [MS_BLOCK][dim_pad]
    float* ks = qs + MS_BLOCK * dim_pad;            // [MS_BLOCK][dim_pad]
    float* vs = ks + MS_BLOCK * dim_pad;            // [MS_BLOCK][cols]
    float* gs = vs + MS_BLOCK * a.cols;             // [MS_BLOCK][4]
    const int r = threadIdx.x % R, c = threadIdx.x / R;
    const int col = chunk * a.cols + c;
    const bool live = c < a.cols && col < a.vdim;
    const int slot = a.state_slot[b];
    if (slot < 0 || slot >= a.n_slots) return;
    const size_t column = ((size_t)h * a.vdim + (live ? col : 0)) * a.dim;
    const size_t per_s = (size_t)a.heads * a.vdim * a.dim, per_n = (size_t)a.heads * a.dim;
    float* srow = a.state_s + (size_t)slot * per_s + column;
    float* nrow = a.state_n + (size_t)slot * per_n + (size_t)h * a.dim;
    float S[NI], N[NI];
    {
        const float* from_s = nullptr;
        const float* from_n = nullptr;
        if (MODE == 0 && carried) { from_s = srow; from_n = nrow; }
        if (MODE == 2) {
            from_s = a.seg_start_s + (size_t)blockIdx.z * per_s + column;
            from_n = a.seg_start_n + (size_t)blockIdx.z * per_n + (size_t)h * a.dim;
        }
#pragma unroll
        for (int ii = 0; ii < NI; ++ii) {
            const int i = r * NI + ii;
            S[ii] = (live && from_s != nullptr && i < a.dim) ? from_s[i] : 0.0f;
            N[ii] = (from_n != nullptr && i < a.dim) ? from_n[i] : 0.0f;
        }
    }
    float kept = 1.0f;                              // the product of the keep factors (pass 1)
    for (int tb = t0; tb < t1; tb += MS_BLOCK) {
        const int nb = min(MS_BLOCK, t1 - tb);
        __syncthreads();                            // the block before has been consumed
        for (int u = threadIdx.x; u < nb * a.dim; u += blockDim.x) {
            const int tok = u / a.dim, i = u - tok * a.dim;
            const float* row = a.proj + (size_t)(tb + tok) * a.ld + h * a.dim + i;
            if (MODE != 1) qs[tok * dim_pad + i] = row[a.q_col] * a.q_scale;
            ks[tok * dim_pad + i] = row[a.k_col];
        }
        for (int u = threadIdx.x; u < nb * (dim_pad - a.dim); u += blockDim.x) {
            const int tok = u / (dim_pad - a.dim), i = a.dim + u % (dim_pad - a.dim);
            qs[tok * dim_pad + i] = 0.0f;
            ks[tok * dim_pad + i] = 0.0f;
        }
        for (int u = threadIdx.x; u < nb * a.cols; u += blockDim.x) {
            const int tok = u / a.cols, cc = u - tok * a.cols;
            const int vc = chunk * a.cols + cc;
            vs[tok * a.cols + cc] = vc < a.vdim
                ? a.proj[(size_t)(tb + tok) * a.ld + a.v_col + h * a.vdim + vc] : 0.0f;
        }
        for (int u = threadIdx.x; u < nb * 4; u += blockDim.x)
            gs[u] = a.gates[((size_t)(tb + u / 4) * a.heads + h) * 4 + (u & 3)];
        __syncthreads();
#pragma unroll 2
        for (int tok = 0; tok < nb; ++tok) {
            const float keep = gs[tok * 4], take = gs[tok * 4 + 1];
            const float tv = take * (c < a.cols ? vs[tok * a.cols + c] : 0.0f);
            const float4* q4 = reinterpret_cast<const float4*>(qs + tok * dim_pad + r * NI);
            const float4* k4 = reinterpret_cast<const float4*>(ks + tok * dim_pad + r * NI);
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, nac[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (MODE == 1) kept *= keep;
#pragma unroll
            for (int g = 0; g < NI / 4; ++g) {      // (sums in an order that dim alone fixes)
                const float4 kk = k4[g];
                S[4 * g + 0] = fmaf(keep, S[4 * g + 0], kk.x * tv);
                S[4 * g + 1] = fmaf(keep, S[4 * g + 1], kk.y * tv);
                S[4 * g + 2] = fmaf(keep, S[4 * g + 2], kk.z * tv);
                S[4 * g + 3] = fmaf(keep, S[4 * g + 3], kk.w * tv);
                N[4 * g + 0] = fmaf(keep, N[4 * g + 0], kk.x * take);
                N[4 * g + 1] = fmaf(keep, N[4 * g + 1], kk.y * take);
                N[4 * g + 2] = fmaf(keep, N[4 * g + 2], kk.z * take);
                N[4 * g + 3] = fmaf(keep, N[4 * g + 3], kk.w * take);
                if (MODE != 1) {
                    const float4 qq = q4[g];
                    acc[0] = fmaf(S[4 * g + 0], qq.x, acc[0]);
                    acc[1] = fmaf(S[4 * g + 1], qq.y, acc[1]);
                    acc[2] = fmaf(S[4 * g + 2], qq.z, acc[2]);
                    acc[3] = fmaf(S[4 * g + 3], qq.w, acc[3]);
                    nac[0] = fmaf(N[4 * g + 0], qq.x, nac[0]);
                    nac[1] = fmaf(N[4 * g + 1], qq.y, nac[1]);
                    nac[2] = fmaf(N[4 * g + 2], qq.z, nac[2]);
                    nac[3] = fmaf(N[4 * g + 3], qq.w, nac[3]);
                }
            }
            if (MODE != 1) {
                float o = (acc[0] + acc[1]) + (acc[2] + acc[3]);
                float nq = (nac[0] + nac[1]) + (nac[2] + nac[3]);
                for (int m = 1; m < R; m <<= 1) {
                    o += __shfl_xor_sync(0xffffffffu, o, m);
                    nq += __shfl_xor_sync(0xffffffffu, nq, m);
                }
                if (live && r == 0)
                    a.o_raw[(size_t)(tb + tok) * a.heads * a.vdim + h * a.vdim + col] =
                        o / (fmaxf(fabsf(nq), gs[tok * 4 + 2]) + 1e-6f);
            }
        }
    }
    float* to_s = nullptr;
    float* to_n = nullptr;
    if (MODE == 0 || (MODE == 2 && s == nseg - 1)) { to_s = srow; to_n = nrow; }
    if (MODE == 1) {
        to_s = a.seg_own_s + (size_t)blockIdx.z * per_s + column;
        to_n = a.seg_own_n + (size_t)blockIdx.z * per_n + (size_t)h * a.dim;
        if (chunk == 0 && threadIdx.x == 0) a.seg_keep[(size_t)blockIdx.z * a.heads + h] = kept;
    }
    if (to_s != nullptr) {
#pragma unroll
        for (int ii = 0; ii < NI; ++ii) {
            const int i = r * NI + ii;
            if (i >= a.dim) continue;
            if (live) to_s[i] = S[ii];
            if (chunk == 0 && c == 0) to_n[i] = N[ii];
        }
    }
}

// Pass 2: a thread per state number of a (head, request), the request's segments in order.
__global__ void mmem_carry_kernel(MscanArgs a) {
    prb_grid_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y;
    const int t0 = a.q_start[b], t1 = a.q_start[b + 1];
    if (t1 <= t0 || t0 < 0 || t1 > a.n_tokens) return;
    const int slot = a.state_slot[b];
    if (slot < 0 || slot >= a.n_slots) return;
    int base = 0;
    for (int bb = 0; bb < b; ++bb) {
        const int n = a.q_start[bb + 1] - a.q_start[bb];
        base += n > 0 ? (n + a.seg_len - 1) / a.seg_len : 0;
    }
    const int nseg = (t1 - t0 + a.seg_len - 1) / a.seg_len;
    const size_t per_s = (size_t)a.heads * a.vdim * a.dim, per_n = (size_t)a.heads * a.dim;
    const size_t head_s = (size_t)a.vdim * a.dim;
    const bool carried = a.positions[t0] > 0;
    for (size_t e = (size_t)blockIdx.z * 1024 + threadIdx.x;
         e < min(head_s, ((size_t)blockIdx.z + 1) * 1024); e += blockDim.x) {
        const size_t at = (size_t)h * head_s + e;
        float S = carried ? a.state_s[(size_t)slot * per_s + at] : 0.0f;
        for (int s = 0; s < nseg; ++s) {
            a.seg_start_s[(size_t)(base + s) * per_s + at] = S;
            if (s + 1 < nseg)
                S = fmaf(a.seg_keep[(size_t)(base + s) * a.heads + h], S,
                         a.seg_own_s[(size_t)(base + s) * per_s + at]);
        }
    }
    if (blockIdx.z == 0) {
        for (int e = threadIdx.x; e < a.dim; e += blockDim.x) {
            const size_t at = (size_t)h * a.dim + e;
            float N = carried ? a.state_n[(size_t)slot * per_n + at] : 0.0f;
            for (int s = 0; s < nseg; ++s) {
                a.seg_start_n[(size_t)(base + s) * per_n + at] = N;
                if (s + 1 < nseg)
                    N = fmaf(a.seg_keep[(size_t)(base + s) * a.heads + h], N,
                             a.seg_own_n[(size_t)(base + s) * per_n + at]);
            }
        }
    }
}

template <typename O>
__global__ void mmem_finish_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ o_raw,
                                   const float* __restrict__ proj, long ld, int g_col,
                                   const float* __restrict__ norm_w, const int* __restrict__ seq,
                                   int n_tokens, int heads, int vdim, float eps, float out_scale) {
    prb_grid_launch_dependents();
    const int lane = threadIdx.x & 31;
    const size_t pair = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= (size_t)n_tokens * heads) return;
    const int t = (int)(pair / heads), h = (int)(pair % heads);
    O* o = out + (size_t)t * out_ld + (size_t)h * vdim;
    if (seq[t] < 0) {
        for (int j = lane; j < vdim; j += 32) o[j] = prb_from_float<O>(0.0f);
        return;
    }
    const float* raw = o_raw + ((size_t)t * heads + h) * vdim;
    float ss = 0.0f;
    for (int j = lane; j < vdim; j += 32) ss = fmaf(raw[j], raw[j], ss);
    const float inv = 1.0f / sqrtf(prb_warp_sum(ss) / (float)vdim + eps);
    const float* g = proj + (size_t)t * ld + g_col + h * vdim;
    for (int j = lane; j < vdim; j += 32)
        o[j] = prb_from_float<O>(raw[j] * inv * norm_w[h * vdim + j] * ru_sigmoid(g[j]) * out_scale);
}

int ms_ni(int dim) { return dim <= 128 ? 4 : 16; }
int ms_lanes(int dim) {
    if (dim <= 0) return 0;
    const int ni = ms_ni(dim);
    int r = 1;
    while (r * ni < dim) r <<= 1;
    return r <= 32 ? r : 0;
}

template <int NI>
void ms_launch(const MscanArgs& a, int mode, dim3 grid, int threads, size_t smem, cudaStream_t stream) {
    if (smem > 40 * 1024) {
        cudaFuncSetAttribute(mmem_scan_kernel<NI, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(mmem_scan_kernel<NI, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(mmem_scan_kernel<NI, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    if (mode == 0) mmem_scan_kernel<NI, 0><<<grid, threads, smem, stream>>>(a);
    else if (mode == 1) mmem_scan_kernel<NI, 1><<<grid, threads, smem, stream>>>(a);
    else mmem_scan_kernel<NI, 2><<<grid, threads, smem, stream>>>(a);
}

size_t mmem_smem(int dim, int vdim) {
    const int vt = vdim < MM_THREADS ? vdim : MM_THREADS;
    return ((size_t)dim * vdim + 3 * (size_t)dim + vdim + (size_t)(MM_THREADS / vt) * vdim) * sizeof(float);
}
}  // namespace

// ------------------------------------------------------------------------- exports
PRB_API int prb_lru_max_taps() { return LRU_MAX_TAPS; }

PRB_API int prb_lru_conv(float* u, const float* proj, long ld, int x_col, const float* x_bias,
                         const float* conv_w, const float* conv_b, const float* conv_state,
                         const int* seq_of_token, const int* positions, const int* q_start,
                         const int* state_slot, int n_tokens, int width, int taps, int n_slots,
                         int b_cap, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || taps < 1 || taps > LRU_MAX_TAPS) return PRB_E_SIZE;
    const int threads = width >= 256 ? 256 : ((width + 31) / 32) * 32;
    lru_conv_kernel<<<n_tokens, threads, 0, stream>>>(u, proj, ld, x_col, x_bias, conv_w, conv_b,
                                                      conv_state, seq_of_token, positions, q_start,
                                                      state_slot, n_tokens, width, taps, n_slots,
                                                      b_cap);
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_lru_gates(float* a_out, float* u, const void* wa_t, const void* wi_t,
                          const float* ba, const float* bi, const float* decay, int n_tokens,
                          int width, int blocks, int w_dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || blocks <= 0 || width % blocks != 0 || blocks > 65535) return PRB_E_SIZE;
    const int bw = width / blocks;
    const size_t smem = (size_t)LRU_TOK * bw * sizeof(float);
    if (smem > 160 * 1024) return PRB_E_SIZE;
    dim3 grid((n_tokens + LRU_TOK - 1) / LRU_TOK, blocks);
    if (w_dtype == PRB_F32) {
        if (smem > 40 * 1024)
            cudaFuncSetAttribute(lru_gates_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        lru_gates_kernel<float><<<grid, 128, smem, stream>>>(
            a_out, u, (const float*)wa_t, (const float*)wi_t, ba, bi, decay, n_tokens, width, bw);
    } else if (w_dtype == PRB_BF16) {
        if (smem > 40 * 1024)
            cudaFuncSetAttribute(lru_gates_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        lru_gates_kernel<__nv_bfloat16><<<grid, 128, smem, stream>>>(
            a_out, u, (const __nv_bfloat16*)wa_t, (const __nv_bfloat16*)wi_t, ba, bi, decay,
            n_tokens, width, bw);
    } else {
        return PRB_E_DTYPE;
    }
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_lru_scan(void* out, long out_ld, const float* a_in, const float* in,
                         const float* proj, long ld, int y_col, int x_col, const float* y_bias,
                         const float* x_bias, float* state, float* conv_state, const int* q_start,
                         const int* state_slot, const int* positions, int n_tokens,
                         int n_requests, int n_slots, int width, int taps, float out_scale,
                         int out_dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || n_requests <= 0) return 0;
    if (width <= 0 || taps < 1 || taps > LRU_MAX_TAPS) return PRB_E_SIZE;
    dim3 grid(n_requests, (width + 127) / 128);
    if (out_dtype == PRB_F32)
        lru_scan_kernel<float><<<grid, 128, 0, stream>>>(
            (float*)out, out_ld, a_in, in, proj, ld, y_col, x_col, y_bias, x_bias, state,
            conv_state, q_start, state_slot, positions, n_tokens, n_slots, width, taps, out_scale);
    else if (out_dtype == PRB_BF16)
        lru_scan_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
            (__nv_bfloat16*)out, out_ld, a_in, in, proj, ld, y_col, x_col, y_bias, x_bias, state,
            conv_state, q_start, state_slot, positions, n_tokens, n_slots, width, taps, out_scale);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}

// The scan in segments side by side (two launches): seg_own and seg_keep are [segments, width]
// for segments >= prb_lru_max_segments(n_tokens, n_requests).
PRB_API int prb_lru_segment() { return LRU_SEG; }
PRB_API int prb_lru_max_segments(int t_cap, int b_cap) { return t_cap / LRU_SEG + b_cap; }
PRB_API int prb_lru_scan_segments(void* out, long out_ld, const float* a_in, const float* in,
                                  float* seg_own, float* seg_keep, int segments,
                                  const float* proj, long ld, int y_col, int x_col,
                                  const float* y_bias, const float* x_bias, float* state,
                                  float* conv_state, const int* q_start, const int* state_slot,
                                  const int* positions, int n_tokens, int n_requests, int n_slots,
                                  int width, int taps, float out_scale, int out_dtype,
                                  cudaStream_t stream) {
    if (n_tokens <= 0 || n_requests <= 0) return 0;
    if (width <= 0 || taps < 1 || taps > LRU_MAX_TAPS) return PRB_E_SIZE;
    const int most = prb_lru_max_segments(n_tokens, n_requests);
    if (segments < most || most > 65535 * 32) return PRB_E_SIZE;
    if (out_dtype != PRB_F32 && out_dtype != PRB_BF16) return PRB_E_DTYPE;
    dim3 grid(most, (width + 127) / 128);
    lru_seg_own_kernel<<<grid, 128, 0, stream>>>(seg_own, seg_keep, a_in, in, q_start, n_tokens,
                                                 n_requests, width);
    PRB_LAUNCH_CHECK();
    if (out_dtype == PRB_F32)
        lru_seg_scan_kernel<float><<<grid, 128, 0, stream>>>(
            (float*)out, out_ld, a_in, in, seg_own, seg_keep, proj, ld, y_col, x_col, y_bias,
            x_bias, state, conv_state, q_start, state_slot, positions, n_tokens, n_requests,
            n_slots, width, taps, out_scale);
    else
        lru_seg_scan_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
            (__nv_bfloat16*)out, out_ld, a_in, in, seg_own, seg_keep, proj, ld, y_col, x_col,
            y_bias, x_bias, state, conv_state, q_start, state_slot, positions, n_tokens,
            n_requests, n_slots, width, taps, out_scale);
    PRB_LAUNCH_CHECK();
    return 0;
}

// 1 if the one-launch form takes blocks of `bw` channels (a thread per channel of a block).
PRB_API int prb_lru_step_supports(int bw) { return bw > 0 && bw <= 1024 ? 1 : 0; }

// Convolution, gates and recurrence of a step of few tokens in one launch (see
// lru_step_kernel); wa_t, wi_t: [blocks, in, out].
PRB_API int prb_lru_step(void* out, long out_ld, const float* proj, long ld, int y_col, int x_col,
                         const float* y_bias, const float* x_bias, const float* conv_w,
                         const float* conv_b, const void* wa_t, const void* wi_t, const float* ba,
                         const float* bi, const float* decay, float* state, float* conv_state,
                         const int* q_start, const int* state_slot, const int* positions,
                         int n_tokens, int n_requests, int n_slots, int width, int blocks,
                         int taps, float out_scale, int w_dtype, int out_dtype,
                         cudaStream_t stream) {
    if (n_tokens <= 0 || n_requests <= 0) return 0;
    if (width <= 0 || blocks <= 0 || width % blocks != 0 || blocks > 65535 || taps < 1 ||
        taps > LRU_MAX_TAPS || !prb_lru_step_supports(width / blocks))
        return PRB_E_SIZE;
    const int bw = width / blocks;
    LruStepArgs g{out, out_ld, proj, ld, y_col, x_col, y_bias, x_bias, conv_w, conv_b, wa_t, wi_t,
                  ba, bi, decay, state, conv_state, q_start, state_slot, positions, n_tokens,
                  n_slots, width, bw, taps, out_scale};
    const size_t smem = (size_t)LRU_TOK * bw * sizeof(float);
    const int threads = (bw + 31) / 32 * 32;
    dim3 grid(n_requests, blocks);
    if (w_dtype == PRB_F32 && out_dtype == PRB_F32)
        lru_step_kernel<float, float><<<grid, threads, smem, stream>>>(g);
    else if (w_dtype == PRB_BF16 && out_dtype == PRB_BF16)
        lru_step_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, threads, smem, stream>>>(g);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}

// 1 if the matrix memory's kernel takes heads of these sizes (the state of a head fits a
// CTA's shared memory).
PRB_API int prb_mmem_supports(int dim, int vdim) {
    return dim > 0 && vdim > 0 && mmem_smem(dim, vdim) <= 200 * 1024 ? 1 : 0;
}

PRB_API int prb_mmem_step(void* out, long out_ld, const float* proj, long ld, int q_col, int k_col,
                          int v_col, int i_col, int f_col, int g_col, const float* i_bias,
                          const float* f_bias, const float* norm_w, float* state_s, float* state_n,
                          float* state_m, const int* q_start, const int* state_slot,
                          const int* positions, int n_tokens, int n_requests, int n_slots,
                          int heads, int dim, int vdim, float cap, float q_scale, float eps,
                          float out_scale, int out_dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || n_requests <= 0) return 0;
    if (heads <= 0 || n_requests > 65535 || !prb_mmem_supports(dim, vdim)) return PRB_E_SIZE;
    MmemArgs a{out, out_ld, proj, ld, q_col, k_col, v_col, i_col, f_col, g_col, i_bias, f_bias,
               norm_w, state_s, state_n, state_m, q_start, state_slot, positions, n_tokens,
               n_slots, heads, dim, vdim, cap, q_scale, eps, out_scale};
    const size_t smem = mmem_smem(dim, vdim);
    dim3 grid(heads, n_requests);
    if (out_dtype == PRB_F32) {
        if (smem > 40 * 1024)
            cudaFuncSetAttribute(mmem_step_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mmem_step_kernel<float><<<grid, MM_THREADS, smem, stream>>>(a);
    } else if (out_dtype == PRB_BF16) {
        if (smem > 40 * 1024)
            cudaFuncSetAttribute(mmem_step_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mmem_step_kernel<__nv_bfloat16><<<grid, MM_THREADS, smem, stream>>>(a);
    } else {
        return PRB_E_DTYPE;
    }
    PRB_LAUNCH_CHECK();
    return 0;
}

// Tokens of a segment, the most segments a step of `t_cap` token rows and `b_cap` requests can
// have (what the workspaces are sized for), and whether the scan takes heads of `dim`.
PRB_API int prb_mmem_segment() { return MS_SEG; }
PRB_API int prb_mmem_max_segments(int t_cap, int b_cap) { return t_cap / MS_SEG + b_cap; }
PRB_API int prb_mmem_scan_supports(int dim) { return ms_lanes(dim) > 0 ? 1 : 0; }

// The matrix memory over long portions: gates, scan (one CTA per (columns, head, request), or,
// with workspaces, in segments side by side), finish.  `gates`: [T, heads, 4]; `o_raw`: [T,
// heads * vdim]; workspaces: seg_s two of [segments, heads, vdim, dim], seg_n two of [segments,
// heads, dim], seg_keep [segments, heads].  The state is [slots, heads, vdim, dim].
PRB_API int prb_mmem_scan(void* out, long out_ld, float* o_raw, float* gates, const float* proj,
                          long ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                          int g_col, const float* i_bias, const float* f_bias,
                          const float* norm_w, float* state_s, float* state_n, float* state_m,
                          const int* q_start, const int* state_slot, const int* positions,
                          const int* seq_of_token, int n_tokens, int n_requests, int n_slots,
                          int heads, int dim, int vdim, float cap, float q_scale, float eps,
                          float out_scale, int cols, float* seg_own_s, float* seg_start_s,
                          float* seg_own_n, float* seg_start_n, float* seg_keep, int segments,
                          int out_dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || n_requests <= 0) return 0;
    const int lanes = ms_lanes(dim);
    if (heads <= 0 || heads > 65535 || n_requests > 65535 || vdim <= 0 || lanes == 0 || cols <= 0)
        return PRB_E_SIZE;
    if (ld % 4 != 0 || ((uintptr_t)proj) % 16 != 0) return PRB_E_ALIGN;
    if (out_dtype != PRB_F32 && out_dtype != PRB_BF16) return PRB_E_DTYPE;
    const bool segmented = seg_own_s && seg_start_s && seg_own_n && seg_start_n && seg_keep && segments > 0;
    if (segmented && (segments > 65535 || segments < prb_mmem_max_segments(n_tokens, n_requests)))
        return PRB_E_SIZE;
    MgateArgs g{gates, proj, ld, i_col, f_col, i_bias, f_bias, state_m, q_start, state_slot,
                positions, n_tokens, n_slots, heads, cap};
    mmem_gates_kernel<<<dim3(heads, n_requests), MG_THREADS, 0, stream>>>(g);
    PRB_LAUNCH_CHECK();
    if (cols > vdim) cols = vdim;
    while (cols * lanes > 1024) cols = (cols + 1) / 2;
    const int threads = (cols * lanes + 31) / 32 * 32;
    const int chunks = (vdim + cols - 1) / cols;
    const int ni = ms_ni(dim);
    MscanArgs a{o_raw, proj, ld, q_col, k_col, v_col, gates, state_s, state_n, q_start, state_slot,
                positions, n_tokens, n_slots, heads, dim, vdim, cols, lanes, q_scale, n_requests,
                segmented ? MS_SEG : 0, seg_own_s, seg_start_s, seg_own_n, seg_start_n, seg_keep};
    const size_t smem = (size_t)MS_BLOCK * (2 * lanes * ni + cols + 4) * sizeof(float);
    if (!segmented) {
        const dim3 grid(chunks, heads, n_requests);
        if (ni == 4) ms_launch<4>(a, 0, grid, threads, smem, stream);
        else ms_launch<16>(a, 0, grid, threads, smem, stream);
        PRB_LAUNCH_CHECK();
    } else {
        const dim3 grid(chunks, heads, prb_mmem_max_segments(n_tokens, n_requests));
        if (ni == 4) ms_launch<4>(a, 1, grid, threads, smem, stream);
        else ms_launch<16>(a, 1, grid, threads, smem, stream);
        PRB_LAUNCH_CHECK();
        mmem_carry_kernel<<<dim3(heads, n_requests, ((size_t)vdim * dim + 1023) / 1024), 256, 0, stream>>>(a);
        PRB_LAUNCH_CHECK();
        if (ni == 4) ms_launch<4>(a, 2, grid, threads, smem, stream);
        else ms_launch<16>(a, 2, grid, threads, smem, stream);
        PRB_LAUNCH_CHECK();
    }
    const int warps = 4;
    const unsigned blocks = (unsigned)(((size_t)n_tokens * heads + warps - 1) / warps);
    if (out_dtype == PRB_F32)
        mmem_finish_kernel<float><<<blocks, warps * 32, 0, stream>>>(
            (float*)out, out_ld, o_raw, proj, ld, g_col, norm_w, seq_of_token, n_tokens, heads,
            vdim, eps, out_scale);
    else
        mmem_finish_kernel<__nv_bfloat16><<<blocks, warps * 32, 0, stream>>>(
            (__nv_bfloat16*)out, out_ld, o_raw, proj, ld, g_col, norm_w, seq_of_token, n_tokens,
            heads, vdim, eps, out_scale);
    PRB_LAUNCH_CHECK();
    return 0;
}
