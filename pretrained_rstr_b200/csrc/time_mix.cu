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
// tmix_shift: a CTA per token; writes the blends side by side, [T, n_mix * width].  The
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
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float c = prb_to_float<A>(cur[i]);
        const float d = (prev ? prb_to_float<A>(prev[i]) : 0.0f) - c;
        for (int s = 0; s < n_mix; ++s)
            o[(size_t)s * width + i] = prb_from_float<A>(fmaf(d, mu[(size_t)s * width + i], c));
    }
}

template <typename A>
__global__ void __launch_bounds__(1024)
tmix_scan_kernel(float* __restrict__ raw, long raw_ld, const float* __restrict__ proj, long ld,
                 int r_col, int k_col, int v_col, int lr_col, const float* __restrict__ w2,
                 const float* __restrict__ w0, const float* __restrict__ u,
                 float* __restrict__ state, const A* __restrict__ h, long h_ld,
                 A* __restrict__ prev_state, const int* __restrict__ q_start,
                 const int* __restrict__ state_slot, const int* __restrict__ positions,
                 int n_requests, int heads, int dim, int vdim, int rank, int width, int lanes,
                 int cols, int n_slots, int* status) {
    extern __shared__ float sm[];
    float* r_s = sm;                                 // [TM_CHUNK][dim]
    float* k_s = r_s + TM_CHUNK * dim;
    float* w_s = k_s + TM_CHUNK * dim;
    float* v_s = w_s + TM_CHUNK * dim;               // [TM_CHUNK][vdim]
    float* th_s = v_s + TM_CHUNK * vdim;             // [TM_CHUNK][rank]
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
            if (live && ln == 0) raw[(size_t)(c0 + tt) * raw_ld + (size_t)hd * vdim + c] = part;
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

PRB_API int prb_tmix_scan(float* raw, long raw_ld, const float* proj, long ld, int r_col, int k_col,
                          int v_col, int lr_col, const float* w2, const float* w0, const float* u,
                          float* state, const void* h, long h_ld, void* prev_state,
                          const int* q_start, const int* state_slot, const int* positions,
                          int n_requests, int heads, int dim, int vdim, int rank, int width,
                          int n_slots, int dtype, int* status, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    const int lanes = tm_lanes(dim);
    if (lanes == 0 || heads <= 0 || vdim <= 0 || rank <= 0 || n_requests > 65535) return PRB_E_SIZE;
    int cols = 1024 / lanes;
    if (cols > vdim) cols = vdim;
    const int groups = (vdim + cols - 1) / cols;
    int threads = (cols * lanes + 31) / 32 * 32;
    const size_t smem = (size_t)TM_CHUNK * (3 * dim + vdim + rank) * sizeof(float);
    if (smem > 200 * 1024) return PRB_E_SIZE;
    dim3 grid(heads, n_requests, groups);
#define TSCAN(AT)                                                                                \
    do {                                                                                         \
        if (smem > 48 * 1024)                                                                    \
            cudaFuncSetAttribute(tmix_scan_kernel<AT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                     \
        tmix_scan_kernel<AT><<<grid, threads, smem, stream>>>(                                   \
            raw, raw_ld, proj, ld, r_col, k_col, v_col, lr_col, w2, w0, u, state, (const AT*)h,  \
            h_ld, (AT*)prev_state, q_start, state_slot, positions, n_requests, heads, dim, vdim, \
            rank, width, lanes, cols, n_slots, status);                                          \
    } while (0)
    if (dtype == PRB_F32) TSCAN(float);
    else if (dtype == PRB_BF16) TSCAN(__nv_bfloat16);
    else return PRB_E_DTYPE;
#undef TSCAN
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
