// Attention over ONE low-rank latent per token that all heads share.
//
// A token's cache row is [c (rank) | r (rot_dim)]: c is the normed latent from which a head's
// keys and values would be expanded (k_h = Uk_h c, v_h = Uv_h c), r a rotated key part common
// to the heads.  Nothing is expanded here.  With the query folded through Uk,
//     qa_h = [Uk_h^T q_h (rank) | rotated q_h (rot_dim)],
// the score of head h for key j is qa_h . [c_j | r_j], and the head's result is
// Uv_h (sum_j w_j c_j): every head reads the same rows, once, whatever the number of heads.
//
//   prb_latent_prepare   norms the two latents of a token, rotates r, writes the cache row
//   prb_latent_fold      q -> qa: the product with Uk_h per head, the rotation of the rest
//   prb_latent_attention scores, softmax with an optional sink per head, sum_j w_j c_j
//   prb_latent_unfold    Uv_h (.) per head, times sigmoid(gate) per head
//
// Rotation: the first `rot_dims` coordinates of the rotated part in the rotate-half layout,
// coordinate i with i + rot_dims/2 by the angle position * freq[i] (the product in 64-bit,
// with freq_lo[i], the part of the frequency that 32 bits leave out, where given).  Scores, softmax
// weights, norms and all sums are 32-bit; the cache and the weights are float32 or bfloat16.
// Sums run over keys, and over a head's coordinates, in an order that depends on the position
// only, never on the rest of the batch.
#include "common.cuh"

namespace {
constexpr int LA_THREADS = 128;
constexpr int LA_GROUP = 8;          // tokens that share a CTA's pass over a head's matrix
constexpr int LA_MAX_ACC = 8;        // rank <= LA_THREADS * LA_MAX_ACC
constexpr int LA_OUT = 32;           // outputs a CTA of the fold / unfold makes (one per lane)
constexpr int LA_SLICES = LA_THREADS / 32;   // parts of the reduction (one per warp)
constexpr int LU_THREADS = 256;      // the unfold's reduction is the longer one: eight warps
constexpr int LU_SLICES = LU_THREADS / 32;

__device__ __forceinline__ float la_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// Two CTAs per token (blockIdx.y: 0 the query latent, 1 the key/value latent and the cache row;
// side by side, since each is a reduction and a round trip long).  proj: float32 [T, ld];
// columns q_col.. hold the query latent (q_rank), kv_col.. the key/value latent (rank) followed
// by the part to rotate (rot_dim).
template <typename C, typename A>
__global__ void __launch_bounds__(LA_THREADS)
latent_prepare_kernel(A* __restrict__ cq, long cq_ld, C* __restrict__ cache,
                      const float* __restrict__ proj, long ld, int q_col, int kv_col,
                      const float* __restrict__ wq, const float* __restrict__ wkv,
                      const int* __restrict__ slots, const int* __restrict__ positions,
                      const float* __restrict__ freq, int n_tokens, int q_rank, int rank,
                      int rot_dim, int rot_dims, int page_size, int num_pages, float eps,
                      float rot_scale, const float* __restrict__ freq_lo, int* status) {
    __shared__ float scratch[32];
    prb_grid_launch_dependents();          // (a product that follows may set itself up meanwhile)
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const float* p = proj + (size_t)t * ld;
    if (blockIdx.y == 0) {
        if (cq == nullptr) return;
        float s = 0.0f;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) s += p[q_col + i] * p[q_col + i];
        const float inv = 1.0f / sqrtf(prb_block_sum(s, scratch) / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
            cq[(size_t)t * cq_ld + i] = prb_from_float<A>(p[q_col + i] * inv * wq[i]);
        return;
    }
    const int slot = slots ? slots[t] : -1;
    if (slot < 0) return;                                     // padding, or nothing to keep
    const int page = slot / page_size, off = slot - page * page_size;
    if (page >= num_pages) {
        if (threadIdx.x == 0) prb_set_status(status, PRB_S_SLOT_RANGE, t, slot, num_pages);
        return;
    }
    float s = 0.0f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) s += p[kv_col + i] * p[kv_col + i];
    const float inv = 1.0f / sqrtf(prb_block_sum(s, scratch) / (float)rank + eps);
    C* row = cache + ((size_t)page * page_size + off) * (rank + rot_dim);
    for (int i = threadIdx.x; i < rank; i += blockDim.x)
        row[i] = prb_from_float<C>(p[kv_col + i] * inv * wkv[i]);
    const float* r = p + kv_col + rank;
    const int half = rot_dims / 2;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < rot_dim; i += blockDim.x) {
        float v = r[i];
        if (i < half) {
            float sn, cs;
            prb_sincos_angle(pos, freq[i], &sn, &cs, freq_lo ? freq_lo[i] : 0.0f);
            v = (r[i] * cs - r[i + half] * sn) * rot_scale;
        } else if (i < rot_dims) {
            float sn, cs;
            prb_sincos_angle(pos, freq[i - half], &sn, &cs, freq_lo ? freq_lo[i - half] : 0.0f);
            v = (r[i] * cs + r[i - half] * sn) * rot_scale;
        }
        row[rank + i] = prb_from_float<C>(v);
    }
}

// grid (ceil(T / LA_GROUP), heads, ceil(rank / LA_OUT) + 1).  q: float32 [T, ld], head h at
// columns h*(dim+rot_dim); uk: [heads*dim, rank]; qa: [T, heads, rank + rot_dim], float32 or
// (for the tensor-core kernel) bfloat16.  A CTA makes LA_OUT coordinates of the folded query
// for LA_GROUP tokens of one head: lane = coordinate, warp = a quarter of the head's `dim`
// (every fourth d), the quarters summed in warp order through shared memory; the loads of a
// thread's weights do not depend on one another, so they are all in flight at once.  The last
// z-block rotates the rest of the head's query.
template <typename W, typename O>
__global__ void __launch_bounds__(LA_THREADS)
latent_fold_kernel(O* __restrict__ qa, const float* __restrict__ q, long ld,
                   const W* __restrict__ uk, const int* __restrict__ positions,
                   const float* __restrict__ freq, const float* __restrict__ freq_lo, int n_tokens,
                   int heads, int dim, int rot_dim, int rot_dims, int rank) {
    extern __shared__ float qs[];                        // [LA_GROUP][dim]
    __shared__ float part[LA_SLICES][LA_GROUP][LA_OUT];
    const int t0 = blockIdx.x * LA_GROUP, h = blockIdx.y;
    const int hd = dim + rot_dim, D = rank + rot_dim;
    if ((int)blockIdx.z * LA_OUT >= rank) {              // the rotated part
        const int half = rot_dims / 2;
        for (int e = threadIdx.x; e < LA_GROUP * rot_dim; e += blockDim.x) {
            const int j = e / rot_dim, i = e - j * rot_dim;
            const int t = t0 + j;
            if (t >= n_tokens) continue;
            const float* r = q + (size_t)t * ld + h * hd + dim;
            const float pos = (float)positions[t];
            float v = r[i];
            if (i < half) {
                float sn, cs;
                prb_sincos_angle(pos, freq[i], &sn, &cs, freq_lo ? freq_lo[i] : 0.0f);
                v = r[i] * cs - r[i + half] * sn;
            } else if (i < rot_dims) {
                float sn, cs;
                prb_sincos_angle(pos, freq[i - half], &sn, &cs, freq_lo ? freq_lo[i - half] : 0.0f);
                v = r[i] * cs + r[i - half] * sn;
            }
            qa[((size_t)t * heads + h) * D + rank + i] = prb_from_float<O>(v);
        }
        return;
    }
    for (int e = threadIdx.x; e < LA_GROUP * dim; e += blockDim.x) {
        const int j = e / dim, d = e - j * dim;
        qs[e] = (t0 + j < n_tokens) ? q[(size_t)(t0 + j) * ld + h * hd + d] : 0.0f;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
    const int r = blockIdx.z * LA_OUT + lane;
    float acc[LA_GROUP];
#pragma unroll
    for (int j = 0; j < LA_GROUP; ++j) acc[j] = 0.0f;
    if (r < rank) {
        const W* w = uk + (size_t)h * dim * rank + r;
#pragma unroll 8
        for (int d = slice; d < dim; d += LA_SLICES) {
            const float wv = prb_to_float<W>(w[(size_t)d * rank]);
#pragma unroll
            for (int j = 0; j < LA_GROUP; ++j) acc[j] = fmaf(qs[j * dim + d], wv, acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < LA_GROUP; ++j) part[slice][j][lane] = acc[j];
    __syncthreads();
    for (int e = threadIdx.x; e < LA_GROUP * LA_OUT; e += blockDim.x) {
        const int j = e / LA_OUT, l = e - j * LA_OUT;
        const int rr = blockIdx.z * LA_OUT + l;
        if (t0 + j >= n_tokens || rr >= rank) continue;
        float v = part[0][j][l];
#pragma unroll
        for (int sl = 1; sl < LA_SLICES; ++sl) v += part[sl][j][l];
        qa[((size_t)(t0 + j) * heads + h) * D + rr] = prb_from_float<O>(v);
    }
}

// grid (T, heads): token t of request b at position p sees keys lo..p (lo = 0, or
// p - window + 1), in chunks of LA_THREADS keys with a running maximum and sum.
template <typename C>
__global__ void __launch_bounds__(LA_THREADS)
latent_attention_kernel(float* __restrict__ out, const float* __restrict__ qa,
                        const C* __restrict__ cache, const int* __restrict__ block_table,
                        const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                        const float* __restrict__ sinks, int n_tokens, int heads, int rank,
                        int rot_dim, int page_size, int max_pages, int num_pages, float scale,
                        int window, int* status) {
    extern __shared__ float smem[];
    __shared__ float scratch[32];
    __shared__ float wts[LA_THREADS];
    __shared__ long long rows[LA_THREADS];
    const int D = rank + rot_dim;
    float* qs = smem;                                     // [D]
    const int t = blockIdx.x, h = blockIdx.y;
    if (t >= n_tokens) return;
    float* o = out + ((size_t)t * heads + h) * rank;
    const int b = seq_of_token[t];
    const int pos = positions[t];
    if (b < 0 || pos < 0 || pos >= max_pages * page_size) {
        if (b >= 0 && threadIdx.x == 0)
            prb_set_status(status, PRB_S_POSITION_RANGE, t, pos, max_pages * page_size);
        for (int d = threadIdx.x; d < rank; d += blockDim.x) o[d] = 0.0f;
        return;
    }
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int* table = block_table + (size_t)b * max_pages;
    const float* qp = qa + ((size_t)t * heads + h) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = qp[d];
    __syncthreads();
    float acc[LA_MAX_ACC];
#pragma unroll
    for (int k = 0; k < LA_MAX_ACC; ++k) acc[k] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    for (int c0 = lo; c0 <= pos; c0 += LA_THREADS) {
        const int j = c0 + threadIdx.x;
        float s = -INFINITY;
        long long row = -1;
        if (j <= pos) {
            const int page = table[j / page_size];
            if (page < 0 || page >= num_pages) {
                prb_set_status(status, PRB_S_PAGE_RANGE, t, j, page);
            } else {
                row = ((long long)page * page_size + (j % page_size)) * D;
                const C* kp = cache + row;
                float dot = 0.0f;
                for (int d = 0; d < D; ++d) dot = fmaf(qs[d], prb_to_float<C>(kp[d]), dot);
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m, prb_block_max(s, scratch));
        const float w = (s == -INFINITY) ? 0.0f : expf(s - m_new);
        wts[threadIdx.x] = w;
        rows[threadIdx.x] = row;
        const float csum = prb_block_sum(w, scratch);         // (its barriers publish wts, rows)
        __syncthreads();
        const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        l = l * corr + csum;
        const int n = min(LA_THREADS, pos - c0 + 1);
#pragma unroll
        for (int k = 0; k < LA_MAX_ACC; ++k) {
            const int d = threadIdx.x + k * LA_THREADS;
            if (d >= rank) break;
            float a = acc[k] * corr;
            for (int i = 0; i < n; ++i) {
                const float wi = wts[i];
                if (wi != 0.0f) a = fmaf(wi, prb_to_float<C>(cache[rows[i] + d]), a);
            }
            acc[k] = a;
        }
        m = m_new;
        __syncthreads();
    }
    // the sink: one more term of the denominator, with no key and no value
    float top = m, extra = 0.0f;
    if (sinks != nullptr) {
        const float sk = sinks[h];
        top = fmaxf(m, sk);
        extra = expf(sk - top);
    }
    const float shrink = (m == -INFINITY) ? 0.0f : expf(m - top);
    const float denom = l * shrink + extra;
#pragma unroll
    for (int k = 0; k < LA_MAX_ACC; ++k) {
        const int d = threadIdx.x + k * LA_THREADS;
        if (d >= rank) break;
        o[d] = denom > 0.0f ? acc[k] * shrink / denom : 0.0f;
    }
}

// grid (ceil(T / LA_GROUP), heads, ceil(vdim / LA_OUT)).  lat: float32 [T, heads, rank]; uvt:
// [heads, rank, vdim] (the value expansion with the latent axis outermost); out: [T,
// heads*vdim] in O; gate: float32, head h of token t at gate[t*gate_ld + h] (gate_per 1), or
// one number per value coordinate at gate[t*gate_ld + h*vdim + v] (gate_per vdim), or null.  Like
// the fold: lane = value coordinate, warp = every eighth latent coordinate, summed in warp
// order.
template <typename W, typename O>
__global__ void __launch_bounds__(LU_THREADS)
latent_unfold_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ lat,
                     const W* __restrict__ uvt, const float* __restrict__ gate, long gate_ld,
                     int gate_per, int n_tokens, int heads, int rank, int vdim) {
    extern __shared__ float ls[];                        // [LA_GROUP][rank]
    __shared__ float part[LU_SLICES][LA_GROUP][LA_OUT];
    const int t0 = blockIdx.x * LA_GROUP, h = blockIdx.y;
    for (int e = threadIdx.x; e < LA_GROUP * rank; e += blockDim.x) {
        const int j = e / rank, r = e - j * rank;
        ls[e] = (t0 + j < n_tokens) ? lat[((size_t)(t0 + j) * heads + h) * rank + r] : 0.0f;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
    const int v = blockIdx.z * LA_OUT + lane;
    float acc[LA_GROUP];
#pragma unroll
    for (int j = 0; j < LA_GROUP; ++j) acc[j] = 0.0f;
    if (v < vdim) {
        const W* w = uvt + (size_t)h * rank * vdim + v;
#pragma unroll 16
        for (int r = slice; r < rank; r += LU_SLICES) {
            const float wv = prb_to_float<W>(w[(size_t)r * vdim]);
#pragma unroll
            for (int j = 0; j < LA_GROUP; ++j) acc[j] = fmaf(ls[j * rank + r], wv, acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < LA_GROUP; ++j) part[slice][j][lane] = acc[j];
    __syncthreads();
    for (int e = threadIdx.x; e < LA_GROUP * LA_OUT; e += blockDim.x) {
        const int j = e / LA_OUT, l = e - j * LA_OUT;
        const int vv = blockIdx.z * LA_OUT + l, t = t0 + j;
        if (t >= n_tokens || vv >= vdim) continue;
        float sum = part[0][j][l];
#pragma unroll
        for (int sl = 1; sl < LU_SLICES; ++sl) sum += part[sl][j][l];
        const float g = gate ? la_sigmoid(gate[(size_t)t * gate_ld + (size_t)h * gate_per +
                                               (gate_per > 1 ? vv : 0)]) : 1.0f;
        out[(size_t)t * out_ld + h * vdim + vv] = prb_from_float<O>(sum * g);
    }
}
}  // namespace

PRB_API int prb_latent_prepare(void* cq, long cq_ld, void* cache, const float* proj, long ld,
                               int q_col, int kv_col, const float* wq, const float* wkv,
                               const int* slots, const int* positions, const float* freq,
                               int n_tokens, int q_rank, int rank, int rot_dim, int rot_dims,
                               int page_size, int num_pages, float eps, int cache_dtype,
                               int act_dtype, float rot_scale, const float* freq_lo, int* status,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rank <= 0 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || rot_dims % 2 != 0 ||
        page_size <= 0 || (cq != nullptr && q_rank <= 0))
        return PRB_E_SIZE;
#define PRB_LP(C, A)                                                                              \
    latent_prepare_kernel<C, A><<<dim3(n_tokens, 2), LA_THREADS, 0, stream>>>(                    \
        (A*)cq, cq_ld, (C*)cache, proj, ld, q_col, kv_col, wq, wkv, slots, positions, freq,       \
        n_tokens, q_rank, rank, rot_dim, rot_dims, page_size, num_pages, eps, rot_scale, freq_lo,  \
        status)
    if (cache_dtype == PRB_F32 && act_dtype == PRB_F32) PRB_LP(float, float);
    else if (cache_dtype == PRB_BF16 && act_dtype == PRB_BF16) PRB_LP(__nv_bfloat16, __nv_bfloat16);
    else if (cache_dtype == PRB_BF16 && act_dtype == PRB_F32) PRB_LP(__nv_bfloat16, float);
    else if (cache_dtype == PRB_F32 && act_dtype == PRB_BF16) PRB_LP(float, __nv_bfloat16);
    else return PRB_E_DTYPE;
#undef PRB_LP
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_latent_fold(void* qa, const float* q, long ld, const void* uk,
                            const int* positions, const float* freq, const float* freq_lo,
                            int n_tokens, int heads, int dim, int rot_dim, int rot_dims, int rank,
                            int w_dtype, int out_dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || heads > 65535 || dim <= 0 || rank <= 0 || rot_dim < 0 || rot_dims > rot_dim ||
        rot_dims % 2 != 0)
        return PRB_E_SIZE;
    const size_t smem = (size_t)LA_GROUP * dim * sizeof(float);
    if (smem > 48 * 1024) return PRB_E_SIZE;
    dim3 grid((n_tokens + LA_GROUP - 1) / LA_GROUP, heads, (rank + LA_OUT - 1) / LA_OUT + 1);
    if (w_dtype == PRB_F32 && out_dtype == PRB_F32)
        latent_fold_kernel<float, float><<<grid, LA_THREADS, smem, stream>>>(
            (float*)qa, q, ld, (const float*)uk, positions, freq, freq_lo, n_tokens, heads, dim,
            rot_dim, rot_dims, rank);
    else if (w_dtype == PRB_BF16 && out_dtype == PRB_F32)
        latent_fold_kernel<__nv_bfloat16, float><<<grid, LA_THREADS, smem, stream>>>(
            (float*)qa, q, ld, (const __nv_bfloat16*)uk, positions, freq, freq_lo, n_tokens, heads,
            dim, rot_dim, rot_dims, rank);
    else if (w_dtype == PRB_BF16 && out_dtype == PRB_BF16)
        latent_fold_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, LA_THREADS, smem, stream>>>(
            (__nv_bfloat16*)qa, q, ld, (const __nv_bfloat16*)uk, positions, freq, freq_lo, n_tokens,
            heads, dim, rot_dim, rot_dims, rank);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_latent_attention(float* out, const float* qa, const void* cache,
                                 const int* block_table, const int* seq_of_token,
                                 const int* positions, const float* sinks, int n_tokens, int heads,
                                 int rank, int rot_dim, int page_size, int max_pages, int num_pages,
                                 float scale, int window, int cache_dtype, int* status,
                                 cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || heads > 65535 || rank <= 0 || rank > LA_THREADS * LA_MAX_ACC || rot_dim < 0 ||
        page_size <= 0 || max_pages <= 0)
        return PRB_E_SIZE;
    const size_t smem = (size_t)(rank + rot_dim) * sizeof(float);
    dim3 grid(n_tokens, heads);
    if (cache_dtype == PRB_F32)
        latent_attention_kernel<float><<<grid, LA_THREADS, smem, stream>>>(
            out, qa, (const float*)cache, block_table, seq_of_token, positions, sinks, n_tokens,
            heads, rank, rot_dim, page_size, max_pages, num_pages, scale, window, status);
    else if (cache_dtype == PRB_BF16)
        latent_attention_kernel<__nv_bfloat16><<<grid, LA_THREADS, smem, stream>>>(
            out, qa, (const __nv_bfloat16*)cache, block_table, seq_of_token, positions, sinks,
            n_tokens, heads, rank, rot_dim, page_size, max_pages, num_pages, scale, window, status);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_latent_unfold(void* out, long out_ld, const float* lat, const void* uvt,
                              const float* gate, long gate_ld, int gate_per, int n_tokens,
                              int heads, int rank, int vdim, int w_dtype, int out_dtype,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || heads > 65535 || rank <= 0 || vdim <= 0) return PRB_E_SIZE;
    const size_t smem = (size_t)LA_GROUP * rank * sizeof(float);
    if (smem > 48 * 1024) return PRB_E_SIZE;
    dim3 grid((n_tokens + LA_GROUP - 1) / LA_GROUP, heads, (vdim + LA_OUT - 1) / LA_OUT);
#define PRB_LU(W, O)                                                                      \
    latent_unfold_kernel<W, O><<<grid, LU_THREADS, smem, stream>>>(                       \
        (O*)out, out_ld, lat, (const W*)uvt, gate, gate_ld, gate_per, n_tokens, heads, rank, vdim)
    if (w_dtype == PRB_F32 && out_dtype == PRB_F32) PRB_LU(float, float);
    else if (w_dtype == PRB_BF16 && out_dtype == PRB_BF16) PRB_LU(__nv_bfloat16, __nv_bfloat16);
    else if (w_dtype == PRB_BF16 && out_dtype == PRB_F32) PRB_LU(__nv_bfloat16, float);
    else if (w_dtype == PRB_F32 && out_dtype == PRB_BF16) PRB_LU(float, __nv_bfloat16);
    else return PRB_E_DTYPE;
#undef PRB_LU
    PRB_LAUNCH_CHECK();
    return 0;
}
