// Two recurrent mixers over a 32-bit state per request.  Everything that enters a recurrence
// here is 32-bit: gates, decays and their logarithms, exponentials, the states, unit norms.
//
// (1) A gated linear recurrence per channel (the recurrent block of Griffin-style layers):
//       u_t = conv(x)_t                      a causal convolution per channel, `taps` long
//       r_t = sigmoid(A_b u_t,b + a_b)       per block b of the channels, square matrices
//       i_t = sigmoid(B_b u_t,b + b_b)
//       log a_t = decay_c * r_t              decay_c = -const * softplus(lambda_c), given
//       S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t          (S_(-1) = 0)
//       out_t = S_t * gelu_tanh(y_t)
//     lru_conv (a CTA per token; the taps before a portion's first token come from the
//     request's saved inputs), lru_gates (a CTA per (8 tokens, block): the two block matrices
//     in 32-bit FMA, a_t and the recurrence's input), lru_scan (a thread per (request,
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
// wa_t, wi_t: [blocks, bw (in), bw (out)]; a_out[t, c] = a_t; u[t, c] <- sqrt(1 - a^2) * i * u.
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
            const float la = dc * r;                             // log a <= 0
            const float a = expf(la);
            const float in = sqrtf(fmaxf(-expm1f(2.0f * la), 0.0f)) * g * us[k * bw + o];
            a_out[(size_t)(t0 + k) * width + c] = a;
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
        s = fmaf(a_in[(size_t)r * width + c], s, in[(size_t)r * width + c]);
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

// ------------------------------------------------------------------ (2) matrix memory
constexpr int MM_THREADS = 256;
struct MmemArgs {
    void* out; long out_ld;                       // [T, heads * vdim] in O
    const float* proj; long ld;                   // [T, ld]
    int q_col, k_col, v_col, i_col, f_col, g_col;
    const float* i_bias; const float* f_bias;     // [heads]
    const float* norm_w;                          // [heads * vdim]
    float* state_s;                               // [slots, heads, dim, vdim]
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
    for (int e = tid; e < dim * vdim; e += MM_THREADS) S[e] = carried ? a.state_s[sh * dim * vdim + e] : 0.0f;
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
    for (int e = tid; e < dim * vdim; e += MM_THREADS) a.state_s[sh * dim * vdim + e] = S[e];
    for (int e = tid; e < dim; e += MM_THREADS) a.state_n[sh * dim + e] = nn[e];
    if (tid == 0) a.state_m[sh] = m;
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
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(lru_gates_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        lru_gates_kernel<float><<<grid, 128, smem, stream>>>(
            a_out, u, (const float*)wa_t, (const float*)wi_t, ba, bi, decay, n_tokens, width, bw);
    } else if (w_dtype == PRB_BF16) {
        if (smem > 48 * 1024)
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
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(mmem_step_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mmem_step_kernel<float><<<grid, MM_THREADS, smem, stream>>>(a);
    } else if (out_dtype == PRB_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(mmem_step_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mmem_step_kernel<__nv_bfloat16><<<grid, MM_THREADS, smem, stream>>>(a);
    } else {
        return PRB_E_DTYPE;
    }
    PRB_LAUNCH_CHECK();
    return 0;
}
