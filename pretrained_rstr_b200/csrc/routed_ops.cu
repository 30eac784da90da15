// Small kernels of designs that scale their embedding, re-inject it, and route tokens to
// experts by independent scores:
//   * token embedding times a constant, optionally kept a second time (a stream that is
//     joined by its own beginning again later);
//   * a router by scores: z in 32-bit, s = sigmoid(z) (or z itself), the `top` largest, their
//     scores as weights, optionally divided by their sum;
//   * the activation of routed experts whose weight multiplies the expert's INPUT:
//     act(w * u) with u = up(h) (up is linear, so up(w h) = w up(h)), zero for experts a
//     token did not choose.
// All arithmetic is 32-bit.
#include "common.cuh"

namespace {
__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

// ------------------------------------------------------------------ scaled embedding
template <typename W>
__global__ void embed_scaled_kernel(float* __restrict__ out, float* __restrict__ keep,
                                    const int* __restrict__ tokens, const W* __restrict__ table,
                                    int n_tokens, int width, int vocab, float scale, int* status) {
    prb_grid_launch_dependents();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int tok = tokens[t];
    float* o = out + (size_t)t * width;
    float* k = keep ? keep + (size_t)t * width : nullptr;
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) prb_set_status(status, PRB_S_TOKEN_RANGE, t, tok, vocab);
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            o[i] = 0.0f;
            if (k) k[i] = 0.0f;
        }
        return;
    }
    const W* e = table + (size_t)tok * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = prb_to_float<W>(e[i]) * scale;
        o[i] = v;
        if (k) k[i] = v;
    }
}

// ------------------------------------------------------------------ router by scores
// z[e] = x . w[e] (32-bit accumulation; x in X), or, with w == null, x[t, e] holds z already.
// score_fn 0: s = sigmoid(z); 1: s = z; 2: s = softmax(z) over ALL experts.  Chosen scores are
// multiplied by `factor`.  The `top` largest s are chosen, by their z (the same
// order, and large logits whose sigmoids all round to 1 still differ; ties: the lower index).  weights[t, e] = s[e] at chosen experts (divided by the chosen scores' sum when
// `renorm`), zero elsewhere; chosen / chosen_w list them by rank.
template <typename X, typename W>
__global__ void route_scores_kernel(float* __restrict__ weights, int* __restrict__ chosen,
                                    float* __restrict__ chosen_w, const X* __restrict__ x,
                                    long x_ld, const W* __restrict__ w, int n_tokens, int width,
                                    int n_experts, int top, int score_fn, int renorm,
                                    float factor) {
    extern __shared__ float s[];                 // [n_experts]
    prb_grid_launch_dependents();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const X* xr = x + (size_t)t * x_ld;
    if (w == nullptr) {
        for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
            s[e] = prb_to_float<X>(xr[e]);
        }
    } else {
        for (int e = warp; e < n_experts; e += nwarps) {
            const W* we = w + (size_t)e * width;
            float acc = 0.0f;
            for (int i = lane; i < width; i += 32)
                acc = fmaf(prb_to_float<X>(xr[i]), prb_to_float<W>(we[i]), acc);
            acc = prb_warp_sum(acc);
            if (lane == 0) s[e] = acc;
        }
    }
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) weights[(size_t)t * n_experts + e] = 0.0f;
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.0f;
        float z_max = -INFINITY, z_den = 1.0f;
        if (score_fn == 2) {                    // the softmax's maximum and denominator, in index order
            for (int e = 0; e < n_experts; ++e) z_max = fmaxf(z_max, s[e]);
            z_den = 0.0f;
            for (int e = 0; e < n_experts; ++e) z_den += expf(s[e] - z_max);
        }
        for (int k = 0; k < top; ++k) {
            int arg = -1;
            float best = -INFINITY;
            for (int e = 0; e < n_experts; ++e) {
                const float v = s[e];
                if (v == v && (arg < 0 || v > best)) { best = v; arg = e; }
            }
            if (arg < 0) arg = k;               // (a row of NaNs: padding, or a fault upstream)
            const float score = score_fn == 0 ? sigmoidf_(best)
                              : score_fn == 2 ? expf(best - z_max) / z_den : best;
            chosen[(size_t)t * top + k] = arg;
            chosen_w[(size_t)t * top + k] = score;
            sum += score;
            s[arg] = NAN;                       // taken
        }
        for (int k = 0; k < top; ++k) {
            float p = chosen_w[(size_t)t * top + k];
            if (renorm) p /= sum;
            p *= factor;
            chosen_w[(size_t)t * top + k] = p;
            weights[(size_t)t * n_experts + chosen[(size_t)t * top + k]] = p;
        }
    }
}

// --------------------------------------------------------- activation of routed experts
// out[t, i] = act(weights[t, i / group] * in[t, in_col + i]) (or, with on_output, the weight
// times act(in)); act 0: relu(.)^2, 1: relu, 2: gelu
// (tanh form), 3: silu.  Columns of experts a token did not choose come out as act(0) = 0.
__device__ __forceinline__ float routed_act(float v, int act) {
    switch (act) {
        case 0: { const float r = fmaxf(v, 0.0f); return r * r; }
        case 1: return fmaxf(v, 0.0f);
        case 2: return prb_activate(v, PRB_ACT_GELU_TANH);
        default: return v * sigmoidf_(v);
    }
}

template <typename O>
__global__ void routed_act_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ in,
                                  long in_ld, int in_col, int n, int n_rows,
                                  const float* __restrict__ weights, long w_ld, int group, int act,
                                  int on_output) {
    prb_grid_launch_dependents();
    const int n4 = n / 4;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_rows * n4) return;
    const int t = (int)(idx / n4), i = (int)(idx - (size_t)t * n4) * 4;
    const float wgt = weights[(size_t)t * w_ld + i / group];
    O* o = out + (size_t)t * out_ld + i;
    float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (wgt != 0.0f) {                          // (rows of experts not chosen are not read)
        const float4 u = *reinterpret_cast<const float4*>(in + (size_t)t * in_ld + in_col + i);
        const float wi = on_output ? 1.0f : wgt, wo = on_output ? wgt : 1.0f;
        v[0] = wo * routed_act(wi * u.x, act);
        v[1] = wo * routed_act(wi * u.y, act);
        v[2] = wo * routed_act(wi * u.z, act);
        v[3] = wo * routed_act(wi * u.w, act);
    }
    if constexpr (sizeof(O) == 4) {
        *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        uint2 pk;
        pk.x = *reinterpret_cast<const uint32_t*>(&lo);
        pk.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(o) = pk;
    }
}

template <typename O>
__global__ void routed_act1_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ in,
                                   long in_ld, int in_col, int n, int n_rows,
                                   const float* __restrict__ weights, long w_ld, int group, int act,
                                  int on_output) {
    prb_grid_launch_dependents();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_rows * n) return;
    const int t = (int)(idx / n), i = (int)(idx - (size_t)t * n);
    const float wgt = weights[(size_t)t * w_ld + i / group];
    const float u = wgt != 0.0f ? in[(size_t)t * in_ld + in_col + i] : 0.0f;
    const float v = wgt == 0.0f ? 0.0f : (on_output ? wgt * routed_act(u, act) : routed_act(wgt * u, act));
    out[(size_t)t * out_ld + i] = prb_from_float<O>(v);
}
// ------------------------------------------------- router and activation in one launch
// CTAs (token, slice of the row's columns): the scores of the token's router logits (columns of
// the same 32-bit product that holds the experts' first results) and the choice, by every CTA
// of the token for itself, then the activation of the CTA's columns with the chosen experts'
// weights (the others' columns come out zero and are not read).
template <typename O>
__global__ void route_act_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ in,
                                 long in_ld, int in_col, int router_col, int n_rows, int n_experts,
                                 int top, int score_fn, int renorm, int group, int act,
                                 int on_output, float* __restrict__ weights_out) {
    extern __shared__ float sh[];                // [n_experts] scores, then [n_experts] weights
    float* sc = sh;
    float* wt = sh + n_experts;
    prb_grid_launch_dependents();
    const int t = blockIdx.x;
    if (t >= n_rows) return;
    const float* row = in + (size_t)t * in_ld;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        sc[e] = row[router_col + e];             // chosen by the logits: see route_scores
        wt[e] = 0.0f;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.0f;
        for (int k = 0; k < top; ++k) {
            int arg = -1;
            float best = -INFINITY;
            for (int e = 0; e < n_experts; ++e) {
                const float v = sc[e];
                if (v == v && (arg < 0 || v > best)) { best = v; arg = e; }
            }
            if (arg < 0) break;                  // (a row of NaNs: padding, or a fault upstream)
            const float score = score_fn == 0 ? sigmoidf_(best) : best;
            wt[arg] = score;
            sum += score;
            sc[arg] = NAN;                       // taken
        }
        if (renorm)
            for (int e = 0; e < n_experts; ++e) wt[e] /= sum;
    }
    __syncthreads();
    if (weights_out && blockIdx.y == 0)
        for (int e = threadIdx.x; e < n_experts; e += blockDim.x) weights_out[(size_t)t * n_experts + e] = wt[e];
    const int n_all = n_experts * group;
    const int per_cta = (n_all + gridDim.y - 1) / gridDim.y;
    const int c_lo = ((blockIdx.y * per_cta + 3) / 4) * 4;              // slices start at multiples of 4
    const int n = min(n_all, (((blockIdx.y + 1) * per_cta + 3) / 4) * 4);
    O* o = out + (size_t)t * out_ld;
    const bool vec = group % 4 == 0 && in_col % 4 == 0 && in_ld % 4 == 0 && out_ld % 4 == 0 &&
                     ((uintptr_t)in) % 16 == 0 && ((uintptr_t)out) % (4 * sizeof(O)) == 0;
    if (vec) {
        for (int i = c_lo + threadIdx.x * 4; i < n; i += blockDim.x * 4) {
            const float wgt = wt[i / group];
            float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (wgt != 0.0f) {
                const float4 u = *reinterpret_cast<const float4*>(row + in_col + i);
                const float wi = on_output ? 1.0f : wgt, wo = on_output ? wgt : 1.0f;
                v[0] = wo * routed_act(wi * u.x, act);
                v[1] = wo * routed_act(wi * u.y, act);
                v[2] = wo * routed_act(wi * u.z, act);
                v[3] = wo * routed_act(wi * u.w, act);
            }
            if constexpr (sizeof(O) == 4) {
                *reinterpret_cast<float4*>(o + i) = make_float4(v[0], v[1], v[2], v[3]);
            } else {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
                uint2 pk;
                pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(o + i) = pk;
            }
        }
    } else {
        for (int i = c_lo + threadIdx.x; i < n; i += blockDim.x) {
            const float wgt = wt[i / group];
            float v = 0.0f;
            if (wgt != 0.0f) {
                const float u = row[in_col + i];
                v = on_output ? wgt * routed_act(u, act) : routed_act(wgt * u, act);
            }
            o[i] = prb_from_float<O>(v);
        }
    }
}
}  // namespace

PRB_API int prb_embed_scaled(float* out, float* keep, const int* tokens, const void* table,
                             int n_tokens, int width, int vocab, float scale, int table_dtype,
                             int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || vocab <= 0) return PRB_E_SIZE;
    const int threads = width >= 256 ? 256 : ((width + 31) / 32) * 32;
    if (table_dtype == PRB_F32)
        embed_scaled_kernel<float><<<n_tokens, threads, 0, stream>>>(
            out, keep, tokens, (const float*)table, n_tokens, width, vocab, scale, status);
    else if (table_dtype == PRB_BF16)
        embed_scaled_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            out, keep, tokens, (const __nv_bfloat16*)table, n_tokens, width, vocab, scale, status);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_route_scores(float* weights, int* chosen, float* chosen_w, const void* x, long x_ld,
                             const void* w, int n_tokens, int width, int n_experts, int top,
                             int score_fn, int renorm, float factor, int x_dtype, int w_dtype,
                             cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || n_experts <= 0 || top <= 0 || top > n_experts || n_experts > 8192)
        return PRB_E_SIZE;
    if (score_fn < 0 || score_fn > 2) return PRB_E_ARG;
    const size_t smem = (size_t)n_experts * sizeof(float);
#define ROUTE(XT, WT)                                                                          \
    route_scores_kernel<XT, WT><<<n_tokens, 128, smem, stream>>>(                              \
        weights, chosen, chosen_w, (const XT*)x, x_ld, (const WT*)w, n_tokens, width, n_experts, \
        top, score_fn, renorm, factor)
    if (w == nullptr) w_dtype = PRB_F32;
    if (x_dtype == PRB_F32 && w_dtype == PRB_F32) ROUTE(float, float);
    else if (x_dtype == PRB_F32 && w_dtype == PRB_BF16) ROUTE(float, __nv_bfloat16);
    else if (x_dtype == PRB_BF16 && w_dtype == PRB_BF16) ROUTE(__nv_bfloat16, __nv_bfloat16);
    else if (x_dtype == PRB_BF16 && w_dtype == PRB_F32) ROUTE(__nv_bfloat16, float);
    else return PRB_E_DTYPE;
#undef ROUTE
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_routed_act(void* out, long out_ld, const float* in, long in_ld, int in_col, int n,
                           int n_rows, const float* weights, long w_ld, int group, int act,
                           int on_output, int out_dtype, cudaStream_t stream) {
    if (n <= 0 || n_rows <= 0) return 0;
    if (group <= 0 || act < 0 || act > 3) return PRB_E_ARG;
    if (out_dtype != PRB_F32 && out_dtype != PRB_BF16) return PRB_E_DTYPE;
    const size_t total = (size_t)n * n_rows;
    const size_t esz = out_dtype == PRB_F32 ? 4 : 2;
    const bool vec = n % 4 == 0 && in_col % 4 == 0 && in_ld % 4 == 0 && out_ld % 4 == 0 &&
                     group % 4 == 0 && ((uintptr_t)in) % 16 == 0 && ((uintptr_t)out) % (4 * esz) == 0;
    if (vec) {
        const unsigned blocks = (unsigned)((total / 4 + 255) / 256);
        if (out_dtype == PRB_F32)
            routed_act_kernel<float><<<blocks, 256, 0, stream>>>(
                (float*)out, out_ld, in, in_ld, in_col, n, n_rows, weights, w_ld, group, act, on_output);
        else
            routed_act_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
                (__nv_bfloat16*)out, out_ld, in, in_ld, in_col, n, n_rows, weights, w_ld, group, act, on_output);
    } else {
        const unsigned blocks = (unsigned)((total + 255) / 256);
        if (out_dtype == PRB_F32)
            routed_act1_kernel<float><<<blocks, 256, 0, stream>>>(
                (float*)out, out_ld, in, in_ld, in_col, n, n_rows, weights, w_ld, group, act, on_output);
        else
            routed_act1_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
                (__nv_bfloat16*)out, out_ld, in, in_ld, in_col, n, n_rows, weights, w_ld, group, act, on_output);
    }
    PRB_LAUNCH_CHECK();
    return 0;
}

// Router (logits at columns router_col.. of `in`) and the experts' activation (their first
// results at columns in_col..) in one launch; `weights_out` (may be null): [rows, experts].
PRB_API int prb_route_act(void* out, long out_ld, const float* in, long in_ld, int in_col,
                          int router_col, int n_rows, int n_experts, int top, int score_fn,
                          int renorm, int group, int act, int on_output, float* weights_out,
                          int out_dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (n_experts <= 0 || top <= 0 || top > n_experts || n_experts > 4096 || group <= 0)
        return PRB_E_SIZE;
    if (score_fn < 0 || score_fn > 1 || act < 0 || act > 3) return PRB_E_ARG;
    const size_t smem = (size_t)2 * n_experts * sizeof(float);
    // slices of 4,096 columns, fewer while the rows alone fill the GPU
    int slices = (n_experts * group + 4095) / 4096;
    if (slices > 64) slices = 64;
    while (slices > 1 && (long)n_rows * slices > 8L * prb_sm_count()) slices = (slices + 1) / 2;
    const dim3 grid(n_rows, slices);
    if (out_dtype == PRB_F32)
        route_act_kernel<float><<<grid, 256, smem, stream>>>(
            (float*)out, out_ld, in, in_ld, in_col, router_col, n_rows, n_experts, top, score_fn,
            renorm, group, act, on_output, weights_out);
    else if (out_dtype == PRB_BF16)
        route_act_kernel<__nv_bfloat16><<<grid, 256, smem, stream>>>(
            (__nv_bfloat16*)out, out_ld, in, in_ld, in_col, router_col, n_rows, n_experts, top,
            score_fn, renorm, group, act, on_output, weights_out);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}
