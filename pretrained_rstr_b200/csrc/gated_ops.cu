// Memory-bound kernels of designs with gated branches and norms after the sum:
//   * token embedding plus a hashed row for the (previous token, token) pair, the previous
//     token of every request kept in a state row on the device;
//   * root-mean-square norm with one learned number or a weight per coordinate, optionally of
//     alpha * x + sigmoid(gate) * y (a gated branch joined to the stream before the norm), or
//     of the branch alone with the stream added after it (alpha * x + norm(y)),
//     optionally with a copy of the result in the activation type for the next product;
//   * the gated pair of a feed-forward: f(g) * (u + shift) with optional clamps and an
//     optional per-(token, group) scale (a router's weights);
//   * a router: logits in 32-bit, the largest `top`, softmax over those.
// All arithmetic is 32-bit; reduction trees depend on the row's width only.
#include "common.cuh"

namespace {
__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

// ------------------------------------------------------------- embedding with pair rows
// x[t] = table[token] * scale + pairs[row], row = (prev * mul_prev + token * mul_cur) mod buckets,
// or row `buckets` for a sequence's first token.  prev is the token before in the step, or,
// for a request's first token of the step, what prev_state[slot] holds; the CTA of that first
// token then stores the request's last token of the step there.
template <typename W>
__global__ void embed_pair_kernel(float* __restrict__ out, const int* __restrict__ tokens,
                                  const int* __restrict__ positions, const int* __restrict__ seq,
                                  const int* __restrict__ q_start, const int* __restrict__ state_slot,
                                  int* __restrict__ prev_state, const W* __restrict__ table,
                                  const W* __restrict__ pairs, int n_tokens, int width, int vocab,
                                  long long buckets, long long mul_prev, long long mul_cur,
                                  int n_slots, int b_cap, float scale, int* status) {
    prb_grid_launch_dependents();          // (a product that follows may set itself up meanwhile)
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    float* o = out + (size_t)t * width;
    const int b = seq[t];
    const int tok = tokens[t];
    if (b < 0 || b >= b_cap || tok < 0 || tok >= vocab) {
        if (b >= 0 && threadIdx.x == 0) prb_set_status(status, PRB_S_TOKEN_RANGE, t, tok, vocab);
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    const int first = q_start[b], slot = state_slot[b];
    const bool has_slot = slot >= 0 && slot < n_slots;
    int prev = -1;
    if (positions[t] > 0) prev = t > first ? tokens[t - 1] : (has_slot ? prev_state[slot] : -1);
    __syncthreads();                        // every thread has read the state before it changes
    if (t == first && threadIdx.x == 0 && has_slot) {
        const int last = q_start[b + 1] - 1;
        if (last >= t && last < n_tokens) prev_state[slot] = tokens[last];
    }
    long long row = buckets;
    if (prev >= 0)
        row = ((prev % buckets) * mul_prev + (tok % buckets) * mul_cur) % buckets;
    const W* e = table + (size_t)tok * width;
    const W* p = pairs + (size_t)row * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        o[i] = fmaf(prb_to_float<W>(e[i]), scale, prb_to_float<W>(p[i]));
}

// --------------------------------------------------------------- a gate per coordinate
// out[t, i] = in[t, i] * sigmoid(gate[t, i]) for i < n (in, gate: 32-bit rows of pitch in_ld /
// gate_ld; out in the activation type).
template <typename O>
__global__ void gate_mul_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ in,
                                long in_ld, const float* __restrict__ gate, long gate_ld, int n,
                                long total) {
    prb_grid_launch_dependents();
    const long e = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    const long t = e / n;
    const int i = (int)(e - t * n);
    out[t * out_ld + i] = prb_from_float<O>(in[t * in_ld + i] * sigmoidf_(gate[t * gate_ld + i]));
}

// ------------------------------------------------------------------------- RMS norm
struct RmsArgs {
    void* out;              // [n_rows, width] in O, or null
    float* x_out;           // [n_rows, width] float32, or null (may be x itself when rows == null)
    const float* x;         // [n_rows_in, width]
    const float* y;         // [n_rows_in, width] or null: a branch joined before the norm
    const float* gate;      // [n_rows_in, gate_ld] or null: y is multiplied by sigmoid(gate + gate_bias)
    long gate_ld;
    const float* gate_bias; // [width] or null
    const float* gain;      // one number, or null
    const float* weight;    // [width], or null
    const int* rows;        // gather, or null
    int n_rows, n_rows_in, width;
    float alpha, eps;
    int branch_only;        // 1: r = alpha * x + norm(y): the norm is the branch's alone
    int* status;
};

template <typename O>
__global__ void rms_norm_kernel(RmsArgs a) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    prb_grid_launch_dependents();
    const int r = blockIdx.x;
    if (r >= a.n_rows) return;
    const int width = a.width;
    O* out = reinterpret_cast<O*>(a.out);
    const int src = a.rows ? a.rows[r] : r;
    if (src < 0 || src >= a.n_rows_in) {
        if (threadIdx.x == 0) prb_set_status(a.status, PRB_S_ROW_RANGE, r, src, a.n_rows_in);
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            if (out) out[(size_t)r * width + i] = prb_from_float<O>(0.0f);
            if (a.x_out) a.x_out[(size_t)r * width + i] = 0.0f;
        }
        return;
    }
    const float* xr = a.x + (size_t)src * width;
    float s = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = a.branch_only ? 0.0f : a.alpha * xr[i];
        if (a.y) {
            float yy = a.y[(size_t)src * width + i];
            if (a.gate)
                yy *= sigmoidf_(a.gate[(size_t)src * a.gate_ld + i] + (a.gate_bias ? a.gate_bias[i] : 0.0f));
            v += yy;
        }
        row[i] = v;
        s += v * v;
    }
    const float ms = prb_block_sum(s, scratch) / (float)width;
    const float inv = (a.gain ? a.gain[0] : 1.0f) / sqrtf(ms + a.eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float o = row[i] * inv * (a.weight ? a.weight[i] : 1.0f);
        if (a.branch_only) o += a.alpha * xr[i];
        if (a.x_out) a.x_out[(size_t)r * width + i] = o;
        if (out) out[(size_t)r * width + i] = prb_from_float<O>(o);
    }
}

// --------------------------------------------------------------------- gated pair
// out[t, out_col + i] = g' * sigmoid(act_alpha * g') * (u' + up_shift) * scale[t, i / group]
// with g' = min(g, limit) and u' = clamp(u, -limit, limit) when limit > 0.
template <typename O>
__global__ void gated_pair_kernel(O* __restrict__ out, long out_ld, int out_col,
                                  const float* __restrict__ in, long in_ld, int gate_col, int up_col,
                                  int n, int n_rows, float limit, float act_alpha, float up_shift,
                                  const float* __restrict__ scale, long scale_ld, int group) {
    prb_grid_launch_dependents();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_rows * n) return;
    const int t = (int)(idx / n), i = (int)(idx - (size_t)t * n);
    float g = in[(size_t)t * in_ld + gate_col + i];
    float u = in[(size_t)t * in_ld + up_col + i];
    if (limit > 0.0f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
    }
    float v = g * sigmoidf_(act_alpha * g) * (u + up_shift);
    if (scale) v *= scale[(size_t)t * scale_ld + i / group];
    out[(size_t)t * out_ld + out_col + i] = prb_from_float<O>(v);
}

// The same, four neighbouring columns a thread (16-byte loads; n, the columns' offsets, the
// row pitches and the group all multiples of 4).
template <typename O>
__global__ void gated_pair4_kernel(O* __restrict__ out, long out_ld, int out_col,
                                   const float* __restrict__ in, long in_ld, int gate_col, int up_col,
                                   int n, int n_rows, float limit, float act_alpha, float up_shift,
                                   const float* __restrict__ scale, long scale_ld, int group) {
    prb_grid_launch_dependents();
    const int n4 = n / 4;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_rows * n4) return;
    const int t = (int)(idx / n4), i = (int)(idx - (size_t)t * n4) * 4;
    const float4 g4 = *reinterpret_cast<const float4*>(in + (size_t)t * in_ld + gate_col + i);
    const float4 u4 = *reinterpret_cast<const float4*>(in + (size_t)t * in_ld + up_col + i);
    const float sc = scale ? scale[(size_t)t * scale_ld + i / group] : 1.0f;
    float g[4] = {g4.x, g4.y, g4.z, g4.w}, u[4] = {u4.x, u4.y, u4.z, u4.w}, v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (limit > 0.0f) {
            g[k] = fminf(g[k], limit);
            u[k] = fminf(fmaxf(u[k], -limit), limit);
        }
        v[k] = g[k] * sigmoidf_(act_alpha * g[k]) * (u[k] + up_shift) * sc;
    }
    O* o = out + (size_t)t * out_ld + out_col + i;
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

// ------------------------------------------------------------------------- router
// z[e] = x . w[e] + bias[e] in 32-bit; the `top` largest (ties: the lower index); their
// weights are the softmax over those alone.  With w == null, x[t, :n_experts] are logits a
// matrix product has already made (32-bit accumulators).  scale[t, :] holds the weights at the chosen
// experts and zero elsewhere; chosen / chosen_w list them in order of rank.
template <typename W>
__global__ void route_kernel(float* __restrict__ scale, int* __restrict__ chosen,
                             float* __restrict__ chosen_w, const float* __restrict__ x, long x_ld,
                             const W* __restrict__ w, const float* __restrict__ bias, int n_tokens,
                             int width, int n_experts, int top) {
    extern __shared__ float z[];                 // [n_experts]
    prb_grid_launch_dependents();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const float* xr = x + (size_t)t * x_ld;
    if (w == nullptr) {                           // x holds the logits already (bias apart)
        for (int e = threadIdx.x; e < n_experts; e += blockDim.x)
            z[e] = xr[e] + (bias ? bias[e] : 0.0f);
    }
    for (int e = warp; w != nullptr && e < n_experts; e += nwarps) {
        const W* we = w + (size_t)e * width;
        float acc = 0.0f;
        for (int i = lane; i < width; i += 32) acc = fmaf(xr[i], prb_to_float<W>(we[i]), acc);
        acc = prb_warp_sum(acc);
        if (lane == 0) z[e] = acc + (bias ? bias[e] : 0.0f);
    }
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) scale[(size_t)t * n_experts + e] = 0.0f;
    __syncthreads();
    if (threadIdx.x == 0) {
        float best0 = 0.0f, denom = 0.0f;
        for (int k = 0; k < top; ++k) {
            int arg = -1;
            float best = -INFINITY;
            for (int e = 0; e < n_experts; ++e)
                if (arg < 0 || z[e] > best) { best = z[e]; arg = e; }
            if (k == 0) best0 = best;
            const float p = expf(best - best0);
            chosen[(size_t)t * top + k] = arg;
            chosen_w[(size_t)t * top + k] = p;
            denom += p;
            z[arg] = -INFINITY;
        }
        for (int k = 0; k < top; ++k) {
            const float p = chosen_w[(size_t)t * top + k] / denom;
            chosen_w[(size_t)t * top + k] = p;
            scale[(size_t)t * n_experts + chosen[(size_t)t * top + k]] = p;
        }
    }
}
}  // namespace

PRB_API int prb_embed_pair(float* out, const int* tokens, const int* positions, const int* seq,
                           const int* q_start, const int* state_slot, int* prev_state,
                           const void* table, const void* pairs, int n_tokens, int width, int vocab,
                           long buckets, long mul_prev, long mul_cur, int n_slots, int b_cap,
                           int table_dtype, float scale, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || vocab <= 0 || buckets <= 0 || mul_prev < 0 || mul_cur < 0 ||
        buckets > (1L << 31) || mul_prev >= (1L << 31) || mul_cur >= (1L << 31))
        return PRB_E_SIZE;
    const int threads = width >= 256 ? 256 : ((width + 31) / 32) * 32;
    if (table_dtype == PRB_F32)
        embed_pair_kernel<float><<<n_tokens, threads, 0, stream>>>(
            out, tokens, positions, seq, q_start, state_slot, prev_state, (const float*)table,
            (const float*)pairs, n_tokens, width, vocab, buckets, mul_prev, mul_cur, n_slots, b_cap,
            scale, status);
    else if (table_dtype == PRB_BF16)
        embed_pair_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            out, tokens, positions, seq, q_start, state_slot, prev_state,
            (const __nv_bfloat16*)table, (const __nv_bfloat16*)pairs, n_tokens, width, vocab,
            buckets, mul_prev, mul_cur, n_slots, b_cap, scale, status);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_gate_mul(void* out, long out_ld, const float* in, long in_ld, const float* gate,
                         long gate_ld, int n_rows, int n, int out_dtype, cudaStream_t stream) {
    if (n_rows <= 0 || n <= 0) return 0;
    const long total = (long)n_rows * n;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == PRB_F32)
        gate_mul_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, out_ld, in, in_ld, gate,
                                                           gate_ld, n, total);
    else if (out_dtype == PRB_BF16)
        gate_mul_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, out_ld, in,
                                                                   in_ld, gate, gate_ld, n, total);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_rms_norm(void* out, float* x_out, const float* x, const float* y, const float* gate,
                         long gate_ld, const float* gate_bias, const float* gain,
                         const float* weight, const int* rows, int n_rows, int n_rows_in, int width,
                         float alpha, float eps, int branch_only, int out_dtype, int* status,
                         cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (branch_only && y == nullptr) return PRB_E_ARG;
    if (width <= 0 || (size_t)width * 4 > 200 * 1024) return PRB_E_SIZE;
    if (out == nullptr && x_out == nullptr) return PRB_E_ARG;
    if (rows != nullptr && x_out == x) return PRB_E_ARG;        // a gather cannot work in place
    RmsArgs a{out, x_out, x, y, gate, gate_ld, gate_bias, gain, weight, rows, n_rows, n_rows_in,
              width, alpha, eps, branch_only, status};
    const int threads = width >= 256 ? 256 : ((width + 31) / 32) * 32;
    const size_t smem = (size_t)width * sizeof(float);
    if (out_dtype == PRB_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(rms_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem);
        rms_norm_kernel<float><<<n_rows, threads, smem, stream>>>(a);
    } else if (out_dtype == PRB_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(rms_norm_kernel<__nv_bfloat16>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        rms_norm_kernel<__nv_bfloat16><<<n_rows, threads, smem, stream>>>(a);
    } else {
        return PRB_E_DTYPE;
    }
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_gated_pair(void* out, long out_ld, int out_col, const float* in, long in_ld,
                           int gate_col, int up_col, int n, int n_rows, float limit,
                           float act_alpha, float up_shift, const float* scale, long scale_ld,
                           int group, int out_dtype, cudaStream_t stream) {
    if (n <= 0 || n_rows <= 0) return 0;
    if (scale != nullptr && group <= 0) return PRB_E_ARG;
    const size_t total = (size_t)n * n_rows;
    const size_t esz = out_dtype == PRB_F32 ? 4 : 2;
    if (n % 4 == 0 && gate_col % 4 == 0 && up_col % 4 == 0 && out_col % 4 == 0 && in_ld % 4 == 0 &&
        out_ld % 4 == 0 && (scale == nullptr || group % 4 == 0) && ((uintptr_t)in) % 16 == 0 &&
        ((uintptr_t)out) % (4 * esz) == 0 && (out_dtype == PRB_F32 || out_dtype == PRB_BF16)) {
        const unsigned blocks4 = (unsigned)((total / 4 + 255) / 256);
        if (out_dtype == PRB_F32)
            gated_pair4_kernel<float><<<blocks4, 256, 0, stream>>>(
                (float*)out, out_ld, out_col, in, in_ld, gate_col, up_col, n, n_rows, limit,
                act_alpha, up_shift, scale, scale_ld, group);
        else
            gated_pair4_kernel<__nv_bfloat16><<<blocks4, 256, 0, stream>>>(
                (__nv_bfloat16*)out, out_ld, out_col, in, in_ld, gate_col, up_col, n, n_rows, limit,
                act_alpha, up_shift, scale, scale_ld, group);
        PRB_LAUNCH_CHECK();
        return 0;
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == PRB_F32)
        gated_pair_kernel<float><<<blocks, 256, 0, stream>>>(
            (float*)out, out_ld, out_col, in, in_ld, gate_col, up_col, n, n_rows, limit, act_alpha,
            up_shift, scale, scale_ld, group);
    else if (out_dtype == PRB_BF16)
        gated_pair_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
            (__nv_bfloat16*)out, out_ld, out_col, in, in_ld, gate_col, up_col, n, n_rows, limit,
            act_alpha, up_shift, scale, scale_ld, group);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_route(float* scale, int* chosen, float* chosen_w, const float* x, long x_ld, const void* w,
                      const float* bias, int n_tokens, int width, int n_experts, int top,
                      int w_dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || n_experts <= 0 || top <= 0 || top > n_experts || n_experts > 8192)
        return PRB_E_SIZE;
    const size_t smem = (size_t)n_experts * sizeof(float);
    if (w_dtype == PRB_F32)
        route_kernel<float><<<n_tokens, 128, smem, stream>>>(scale, chosen, chosen_w, x, x_ld,
                                                            (const float*)w, bias, n_tokens, width,
                                                            n_experts, top);
    else if (w_dtype == PRB_BF16)
        route_kernel<__nv_bfloat16><<<n_tokens, 128, smem, stream>>>(
            scale, chosen, chosen_w, x, x_ld, (const __nv_bfloat16*)w, bias, n_tokens, width,
            n_experts, top);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}
