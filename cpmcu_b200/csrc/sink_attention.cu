// Softmax attention over the paged cache with capped scores, a sliding window and a sink, and the kernel that
// prepares its queries and keys.
//
//   s(i, j) = q_i . k_j * scale;   s <- cap * tanh(s / cap)   (cap > 0)
//   j is seen by i when 0 <= i - j < window   (window > 0; else every j <= i)
//   p_j = exp(s_j) / (sink + sum_j' exp(s_j'))     sink = 1: one more key of score 0 that has no value; 0: plain softmax
//
// Query and key heads have d channels, value heads dv.  Everything between the projections and the weighted sum of
// values is fp32: biases, angles, the rotation, the unit root mean square of q and k, scores, cap, weights.
#include "common.cuh"

constexpr int kPrepMaxPerLane = 8;      // heads of up to 256 channels
constexpr int kPrepWarps = 4;

// proj: fp32 rows of ``stride`` floats, [heads*d | kv_heads*d | kv_heads*dv] (has_kv) or [heads*d].  One warp per
// (token, head of q, k or v): adds the bias, turns the pairs (c, c + rot_dim/2) of the first rot_dim channels by
// position * inv_freq[c], divides the head by its root mean square (unit_rms), and writes q to q_out [tokens, heads, d],
// k into the key page and v (bias only) into the transposed value page of the token's position.
template <typename T>
__global__ void qk_prepare_store_kernel(const float* __restrict__ proj, int64_t stride, const float* __restrict__ q_bias,
                                        const float* __restrict__ k_bias, const float* __restrict__ v_bias,
                                        T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                        const int* __restrict__ positions, const int* __restrict__ token_seq,
                                        const int* __restrict__ slots, const int* __restrict__ page_table, int max_pages,
                                        const float* __restrict__ inv_freq, int rot_dim, int unit_rms, float eps,
                                        int n_tokens, int n_heads, int n_kv, int d, int dv, int has_kv) {
    extern __shared__ float prep_smem[];       // [warps][d]
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int units = n_heads + (has_kv ? 2 * n_kv : 0);
    const int64_t w = (int64_t)blockIdx.x * kPrepWarps + warp;
    if (w >= (int64_t)n_tokens * units) return;
    const int t = (int)(w / units), unit = (int)(w % units);
    const int pos = positions[t];
    const float* row = proj + (int64_t)t * stride;
    int page = 0;
    if (unit >= n_heads) {
        const int slot = slots[token_seq[t]];
        page = CPM_PAGE(page_table + (int64_t)slot * max_pages, pos / kPageTokens, max_pages);
    }
    if (unit >= n_heads + n_kv) {                                  // a value head: bias, transposed store
        const int kvh = unit - n_heads - n_kv;
        const float* src = row + (int64_t)(n_heads + n_kv) * d + (int64_t)kvh * dv;
        const int64_t base = value_offset(page, kvh, 0, pos % kPageTokens, n_kv, dv);
        for (int c = lane; c < dv; c += 32) {
            const float x = src[c] + (v_bias ? v_bias[kvh * dv + c] : 0.f);
            v_cache[base + (int64_t)c * kPageTokens] = from_f32<T>(x);
        }
        return;
    }
    const bool is_q = unit < n_heads;
    const float* bias = is_q ? q_bias : k_bias;
    const int head = is_q ? unit : unit - n_heads;
    const float* src = row + (int64_t)unit * d;                    // q heads, then k heads, all d wide
    float* xs = prep_smem + warp * d;
    for (int c = lane; c < d; c += 32) xs[c] = src[c] + (bias ? bias[head * d + c] : 0.f);
    __syncwarp();
    const int half = rot_dim >> 1;
    float val[kPrepMaxPerLane];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kPrepMaxPerLane; ++i) {
        const int c = lane + 32 * i;
        float x = 0.f;
        if (c < d) {
            x = xs[c];
            if (inv_freq != nullptr && c < rot_dim) {
                const int f = c < half ? c : c - half;
                float sn, cs;
                sincosf((float)pos * inv_freq[f], &sn, &cs);
                x = c < half ? x * cs - xs[c + half] * sn : x * cs + xs[c - half] * sn;
            }
        }
        val[i] = x;
        ss = fmaf(x, x, ss);
    }
    const float f = unit_rms ? 1.0f / sqrtf(warp_sum(ss) / (float)d + eps) : 1.f;
    T* dst = is_q ? q_out + ((int64_t)t * n_heads + head) * d
                  : k_cache + page_row_offset(page, head, pos % kPageTokens, n_kv, d);
#pragma unroll
    for (int i = 0; i < kPrepMaxPerLane; ++i) {
        const int c = lane + 32 * i;
        if (c < d) dst[c] = from_f32<T>(val[i] * f);
    }
}

CPM_API int cpm_qk_prepare_store(const float* proj, int64_t stride, const float* q_bias, const float* k_bias,
                                 const float* v_bias, void* q_out, void* k_cache, void* v_cache, const int* positions,
                                 const int* token_seq, const int* slots, const int* page_table, int max_pages,
                                 const float* inv_freq, int rot_dim, int unit_rms, float eps, int n_tokens, int n_heads,
                                 int n_kv, int d, int dv, int has_kv, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (d < 1 || d > 32 * kPrepMaxPerLane || dv < 1 || n_heads < 1 || n_kv < 1 || rot_dim < 0 || rot_dim > d || (rot_dim & 1))
        return CPM_BAD_ARGUMENT;
    if (has_kv && (!k_cache || !v_cache)) return CPM_BAD_ARGUMENT;
    const int units = n_heads + (has_kv ? 2 * n_kv : 0);
    const int64_t blocks = ((int64_t)n_tokens * units + kPrepWarps - 1) / kPrepWarps;
    const size_t smem = (size_t)kPrepWarps * d * sizeof(float);
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchRope, qk_prepare_store_kernel<bf16>, dim3((unsigned)blocks), dim3(kPrepWarps * 32), smem, stream, proj,
                   stride, q_bias, k_bias, v_bias, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, positions, token_seq, slots,
                   page_table, max_pages, inv_freq, rot_dim, unit_rms, eps, n_tokens, n_heads, n_kv, d, dv, has_kv);
    else
        cpm_launch(kLaunchRope, qk_prepare_store_kernel<float>, dim3((unsigned)blocks), dim3(kPrepWarps * 32), smem, stream, proj,
                   stride, q_bias, k_bias, v_bias, (float*)q_out, (float*)k_cache, (float*)v_cache, positions, token_seq, slots,
                   page_table, max_pages, inv_freq, rot_dim, unit_rms, eps, n_tokens, n_heads, n_kv, d, dv, has_kv);
    return launch_status();
}

// ---------------------------------------------------------------------------
// The kernel of every size and of the 32-bit path: one warp per (query token, head), fp32 arithmetic throughout.  A
// lane owns a key in the scores and value channels in the weighted sum.  The sink enters as the start of the running
// maximum and sum (maximum 0, sum 1) instead of (-inf, 0).
// ---------------------------------------------------------------------------
constexpr int kSinkMaxPerLane = 8;      // value heads of up to 256 channels

template <typename T>
__global__ void sink_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_cache,
                                              const T* __restrict__ v_cache, T* __restrict__ out,
                                              const int* __restrict__ positions, const int* __restrict__ token_seq,
                                              const int* __restrict__ slots, const int* __restrict__ page_table,
                                              int max_pages, int window, int n_heads, int n_kv, int d, int dv, float scale,
                                              float cap, int sink) {
    extern __shared__ float sink_q_smem[];   // [warps][d]
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int h = blockIdx.y * (blockDim.x >> 5) + warp;
    if (h >= n_heads) return;
    const int kvh = h / (n_heads / n_kv);
    const int p = positions[t];
    const int* pages = page_table + (int64_t)slots[token_seq[t]] * max_pages;
    float* qs = sink_q_smem + warp * d;
    const T* qrow = q + ((int64_t)t * n_heads + h) * d;
    for (int c = lane; c < d; c += 32) qs[c] = to_f32(qrow[c]);
    __syncwarp();
    float m = sink ? 0.f : -INFINITY, l = sink ? 1.f : 0.f;
    float acc[kSinkMaxPerLane];
#pragma unroll
    for (int i = 0; i < kSinkMaxPerLane; ++i) acc[i] = 0.f;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
    for (int j0 = lo; j0 <= p; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j <= p;
        float s = -INFINITY;
        if (valid) {
            const int page = CPM_PAGE(pages, j / kPageTokens, max_pages);
            const T* krow = k_cache + page_row_offset(page, kvh, j % kPageTokens, n_kv, d);
            float dot = 0.f;
            for (int c = 0; c < d; ++c) dot = fmaf(qs[c], to_f32(krow[c]), dot);
            s = dot * scale;
            if (cap > 0.f) s = cap * tanhf(s * inv_cap);
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float pr = valid ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(pr);
#pragma unroll
        for (int i = 0; i < kSinkMaxPerLane; ++i) acc[i] *= corr;
        m = m_new;
        const int n_here = min(32, p + 1 - j0);
        for (int jj = 0; jj < n_here; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, pr, jj);
            const int key = j0 + jj;
            const int page = CPM_PAGE(pages, key / kPageTokens, max_pages);
            const T* vcol = v_cache + value_offset(page, kvh, 0, key % kPageTokens, n_kv, dv);
#pragma unroll
            for (int i = 0; i < kSinkMaxPerLane; ++i) {
                const int c = lane + 32 * i;
                if (c < dv) acc[i] = fmaf(pj, to_f32(vcol[(int64_t)c * kPageTokens]), acc[i]);
            }
        }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* orow = out + ((int64_t)t * n_heads + h) * dv;
#pragma unroll
    for (int i = 0; i < kSinkMaxPerLane; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) orow[c] = from_f32<T>(acc[i] * inv);
    }
}

CPM_API int cpm_sink_attention_generic(const void* q, const void* k_cache, const void* v_cache, void* out, const int* positions,
                                       const int* token_seq, const int* slots, const int* page_table, int max_pages,
                                       int window, int n_tokens, int n_heads, int n_kv, int d, int dv, float scale, float cap,
                                       int sink, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (d <= 0 || dv <= 0 || dv > 32 * kSinkMaxPerLane || n_kv <= 0 || n_heads % n_kv != 0 || window < 0) return CPM_BAD_ARGUMENT;
    const int warps = 4;
    dim3 grid(n_tokens, (n_heads + warps - 1) / warps);
    const size_t smem = (size_t)warps * d * sizeof(float);
    if (smem > 48 * 1024) return CPM_BAD_ARGUMENT;
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchAttention, sink_attention_generic_kernel<bf16>, grid, dim3(warps * 32), smem, stream, (const bf16*)q,
                   (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, positions, token_seq, slots, page_table, max_pages, window,
                   n_heads, n_kv, d, dv, scale, cap, sink);
    else
        cpm_launch(kLaunchAttention, sink_attention_generic_kernel<float>, grid, dim3(warps * 32), smem, stream, (const float*)q,
                   (const float*)k_cache, (const float*)v_cache, (float*)out, positions, token_seq, slots, page_table, max_pages,
                   window, n_heads, n_kv, d, dv, scale, cap, sink);
    return launch_status();
}

CPM_BOUNDS_TU(sink_attention)
