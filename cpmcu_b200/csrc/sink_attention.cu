// Softmax attention over the paged cache with capped scores, a sliding window and a sink, and the kernel that
// prepares its queries and keys.
//
//   s(i, j) = q_i . k_j * scale;   s <- cap * tanh(s / cap)   (cap > 0)
//   j is seen by i when j <= i and (i - j < window or j < keep_first)   (window > 0; else every j <= i)
//   p_j = exp(s_j) / (exp(b_h) + sum_j' exp(s_j'))   sink: one more key without a value, whose score b_h is a number per
//         head (``sinks``; null: 0) that is neither scaled nor capped; no sink: the plain softmax
//   o_h <- o_h * sigmoid(gate[t][h])                 (``gate``: fp32 rows of ``gate_stride`` floats, one per head; null: none)
//
// Query and key heads have d channels, value heads dv.  Everything between the projections and the weighted sum of
// values is fp32: biases, angles, the rotation, the unit root mean square of q and k, scores, cap, weights.
#include "common.cuh"
#include "mma_bf16.cuh"

constexpr int kPrepMaxPerLane = 8;      // heads of up to 256 channels
constexpr int kPrepWarps = 4;

// proj: fp32 rows of ``stride`` floats, [heads*d | kv_heads*d | kv_heads*dv] (has_kv) or [heads*d].  One warp per
// (token, head of q, k or v): adds the bias, turns the pairs (c, c + rot_dim/2) (``adjacent``: the pairs (2c, 2c + 1)) of
// the first rot_dim channels by position * inv_freq[c], divides the head by its root mean square (unit_rms), and writes q to q_out [tokens, heads, d],
// k into the key page and v (bias only) into the transposed value page of the token's position.
template <typename T>
__global__ void qk_prepare_store_kernel(const float* __restrict__ proj, int64_t stride, const float* __restrict__ q_bias,
                                        const float* __restrict__ k_bias, const float* __restrict__ v_bias,
                                        T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                        const int* __restrict__ positions, const int* __restrict__ token_seq,
                                        const int* __restrict__ slots, const int* __restrict__ page_table, int max_pages,
                                        const float* __restrict__ inv_freq, int rot_dim, int adjacent, int unit_rms,
                                        float eps, int n_tokens, int n_heads, int n_kv, int d, int dv, int has_kv) {
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
                const int f = adjacent ? c >> 1 : (c < half ? c : c - half);
                const bool first = adjacent ? !(c & 1) : c < half;
                const int other = adjacent ? c ^ 1 : (first ? c + half : c - half);
                float sn, cs;
                sincosf((float)pos * inv_freq[f], &sn, &cs);
                x = first ? x * cs - xs[other] * sn : x * cs + xs[other] * sn;
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
                                 const float* inv_freq, int rot_dim, int adjacent, int unit_rms, float eps, int n_tokens,
                                 int n_heads, int n_kv, int d, int dv, int has_kv, int dtype, cudaStream_t stream) {
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
                   page_table, max_pages, inv_freq, rot_dim, adjacent, unit_rms, eps, n_tokens, n_heads, n_kv, d, dv, has_kv);
    else
        cpm_launch(kLaunchRope, qk_prepare_store_kernel<float>, dim3((unsigned)blocks), dim3(kPrepWarps * 32), smem, stream, proj,
                   stride, q_bias, k_bias, v_bias, (float*)q_out, (float*)k_cache, (float*)v_cache, positions, token_seq, slots,
                   page_table, max_pages, inv_freq, rot_dim, adjacent, unit_rms, eps, n_tokens, n_heads, n_kv, d, dv, has_kv);
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
                                              int max_pages, int window, int keep_first, int n_heads, int n_kv, int d, int dv,
                                              float scale, float cap, int sink, const float* __restrict__ sinks,
                                              const float* __restrict__ gate, int64_t gate_stride) {
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
    float m = sink ? (sinks ? sinks[h] : 0.f) : -INFINITY, l = sink ? 1.f : 0.f;
    float acc[kSinkMaxPerLane];
#pragma unroll
    for (int i = 0; i < kSinkMaxPerLane; ++i) acc[i] = 0.f;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
    // two stretches of keys: the kept first tokens that lie before the window, then the window
    const int kept_end = min(keep_first, lo);
    for (int part = 0; part < 2; ++part) {
        const int begin = part == 0 ? 0 : lo, end = part == 0 ? kept_end : p + 1;
        for (int j0 = begin; j0 < end; j0 += 32) {
            const int j = j0 + lane;
            const bool valid = j < end;
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
            const int n_here = min(32, end - j0);
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
    }
    float inv = l > 0.f ? 1.f / l : 0.f;
    if (gate != nullptr) inv *= 1.0f / (1.0f + expf(-gate[(int64_t)t * gate_stride + h]));
    T* orow = out + ((int64_t)t * n_heads + h) * dv;
#pragma unroll
    for (int i = 0; i < kSinkMaxPerLane; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) orow[c] = from_f32<T>(acc[i] * inv);
    }
}

CPM_API int cpm_sink_attention_generic(const void* q, const void* k_cache, const void* v_cache, void* out, const int* positions,
                                       const int* token_seq, const int* slots, const int* page_table, int max_pages,
                                       int window, int keep_first, int n_tokens, int n_heads, int n_kv, int d, int dv,
                                       float scale, float cap, int sink, const float* sinks, const float* gate,
                                       int64_t gate_stride, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (d <= 0 || dv <= 0 || dv > 32 * kSinkMaxPerLane || n_kv <= 0 || n_heads % n_kv != 0 || window < 0 || keep_first < 0)
        return CPM_BAD_ARGUMENT;
    const int warps = 4;
    dim3 grid(n_tokens, (n_heads + warps - 1) / warps);
    const size_t smem = (size_t)warps * d * sizeof(float);
    if (smem > 48 * 1024) return CPM_BAD_ARGUMENT;
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchAttention, sink_attention_generic_kernel<bf16>, grid, dim3(warps * 32), smem, stream, (const bf16*)q,
                   (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, positions, token_seq, slots, page_table, max_pages, window,
                   keep_first, n_heads, n_kv, d, dv, scale, cap, sink, sinks, gate, gate_stride);
    else
        cpm_launch(kLaunchAttention, sink_attention_generic_kernel<float>, grid, dim3(warps * 32), smem, stream, (const float*)q,
                   (const float*)k_cache, (const float*)v_cache, (float*)out, positions, token_seq, slots, page_table, max_pages,
                   window, keep_first, n_heads, n_kv, d, dv, scale, cap, sink, sinks, gate, gate_stride);
    return launch_status();
}

// ---------------------------------------------------------------------------
// bf16 on the tensor cores.  A warp owns 16 rows (query tokens of one head in a prompt; the query heads that share a
// key-value head for a single token) and walks over the keys its rows can see, 32 at a time, straight from the pages
// (16-byte loads along the head size for the scores and along the token axis of the transposed value pages for the
// weighted sum; the thread-to-key assignment is the one of attention_bf16.cu).  Scores, cap, running maximum and sum
// are fp32.  The weights enter the second product as two bf16 numbers each (the rounded weight and what the rounding
// left over), so that they carry 16 bits of mantissa into the fp32 accumulators instead of 8.  The sink joins when a
// row is finished: one more term exp(0 - max) in the sum.
// ---------------------------------------------------------------------------
template <int DV>
struct SinkTile {
    float o[DV / 8][4];
    float m[2];      // running maximum, log2 domain
    float l[2];      // this thread's share of the running sum
    __device__ __forceinline__ void init() {
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.f;
    }
};

// tanh from one exponential: 1 - 2 / (e^(2x) + 1); exact limits at both ends (e = 0 and e = inf)
__device__ __forceinline__ float tanh_by_exp(float x) { return 1.f - __fdividef(2.f, __expf(2.f * x) + 1.f); }

__device__ __forceinline__ void split_bf16(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = pack_bf16(a - __low2float(h), b - __high2float(h));
}

// 32 keys key0 .. key0 + 31 of one page; row r sees a key when lo[r] <= key <= hi[r], or key < keep_first and
// key <= hi[r].  The fragment loads:
// ``kload(t, w)`` gives the 8 channels 32 w + 8 j ... of key 8 (n / 2) + 2 t + (n & 1) of the 32, ``vload(nt)`` the
// 8 tokens 8 j ... of value channel 8 nt + n  (j = lane % 4, n = lane / 4).
template <int D, int DV, typename KLoad, typename VLoad>
__device__ __forceinline__ void sink_attend_keys(SinkTile<DV>& st, const uint4 (&q)[2][D / 32], KLoad kload, VLoad vload,
                                                 int key0, const int (&lo)[2], const int (&hi)[2], int keep_first,
                                                 float scale, float cap, int lane) {
    constexpr float kLog2e = 1.4426950408889634f;
    const int j = lane & 3;
    float s[4][4];
#pragma unroll
    for (int t = 0; t < 4; ++t) s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f;
#pragma unroll
    for (int w = 0; w < D / 32; ++w) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const uint4 kv = kload(t, w);
            mma_16816(s[t], q[0][w].x, q[1][w].x, q[0][w].y, q[1][w].y, kv.x, kv.y);
            mma_16816(s[t], q[0][w].z, q[1][w].z, q[0][w].w, q[1][w].w, kv.z, kv.w);
        }
    }
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f, cap_log2 = cap * kLog2e, scale_log2 = scale * kLog2e;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1, key = key0 + 8 * j + 2 * t + (e & 1);
            float x = cap > 0.f ? cap_log2 * tanh_by_exp(s[t][e] * scale * inv_cap) : s[t][e] * scale_log2;
            x = ((key >= lo[r] || key < keep_first) && key <= hi[r]) ? x : -INFINITY;
            s[t][e] = x;
            mx[r] = fmaxf(mx[r], x);
        }
    float use[2], corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float mn = fmaxf(st.m[r], mx[r]);
        use[r] = mn == -INFINITY ? 0.f : mn;
        corr[r] = exp2f(st.m[r] - use[r]);
        st.m[r] = mn;
    }
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float pr = exp2f(s[t][e] - use[e >> 1]);
            s[t][e] = pr;
            sum[e >> 1] += pr;
        }
    st.l[0] = st.l[0] * corr[0] + sum[0];
    st.l[1] = st.l[1] * corr[1] + sum[1];
#pragma unroll
    for (int nt = 0; nt < DV / 8; ++nt) {
        st.o[nt][0] *= corr[0];
        st.o[nt][1] *= corr[0];
        st.o[nt][2] *= corr[1];
        st.o[nt][3] *= corr[1];
    }
    uint32_t ah[4], al[4], ch[4], cl[4];
    split_bf16(s[0][0], s[0][1], ah[0], al[0]);
    split_bf16(s[0][2], s[0][3], ah[1], al[1]);
    split_bf16(s[1][0], s[1][1], ah[2], al[2]);
    split_bf16(s[1][2], s[1][3], ah[3], al[3]);
    split_bf16(s[2][0], s[2][1], ch[0], cl[0]);
    split_bf16(s[2][2], s[2][3], ch[1], cl[1]);
    split_bf16(s[3][0], s[3][1], ch[2], cl[2]);
    split_bf16(s[3][2], s[3][3], ch[3], cl[3]);
    // four output tiles at a time: their loads, then their products, so that products into one accumulator lie apart
#pragma unroll
    for (int nt0 = 0; nt0 < DV / 8; nt0 += 4) {
        uint4 vv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) vv[i] = vload(nt0 + i);
#pragma unroll
        for (int i = 0; i < 4; ++i) mma_16816(st.o[nt0 + i], ah[0], ah[1], ah[2], ah[3], vv[i].x, vv[i].y);
#pragma unroll
        for (int i = 0; i < 4; ++i) mma_16816(st.o[nt0 + i], ch[0], ch[1], ch[2], ch[3], vv[i].z, vv[i].w);
#pragma unroll
        for (int i = 0; i < 4; ++i) mma_16816(st.o[nt0 + i], al[0], al[1], al[2], al[3], vv[i].x, vv[i].y);
#pragma unroll
        for (int i = 0; i < 4; ++i) mma_16816(st.o[nt0 + i], cl[0], cl[1], cl[2], cl[3], vv[i].z, vv[i].w);
    }
}

// The sink joins a finished row: with M = max(m, b) (b the sink's score in log2 units) the sum becomes
// l 2^(m - M) + 2^(b - M) and the accumulator is scaled by 2^(m - M); returns that scale over the new sum.
__device__ __forceinline__ float sink_join(float m, float l, int sink, float b) {
    if (!sink) return l > 0.f ? 1.f / l : 0.f;
    const float M = fmaxf(m, b);
    const float f = m == -INFINITY ? 0.f : exp2f(m - M);
    return f / (l * f + exp2f(b - M));
}

// Finishes a tile: the quad's shares of the sums join, the sink adds its term (score sink_log2[r] for tile row g + 8r), the
// row is multiplied by row_gate[r], and rows go out as bf16.  out_row(r) gives the output row (dv channels) of tile row
// g + 8r, or null.
template <int DV, typename RowFn>
__device__ __forceinline__ void sink_finish(SinkTile<DV>& st, int sink, const float (&sink_log2)[2], const float (&row_gate)[2],
                                            int lane, RowFn out_row) {
    const int j = lane & 3;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float l = st.l[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        bf16* orow = out_row(r);
        if (orow == nullptr) continue;
        const float inv = sink_join(st.m[r], l, sink, sink_log2[r]) * row_gate[r];
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt)
            *reinterpret_cast<uint32_t*>(orow + 8 * nt + 2 * j) = pack_bf16(st.o[nt][2 * r] * inv, st.o[nt][2 * r + 1] * inv);
    }
}

// Prompt tokens: a block of 4 warps takes 64 consecutive query tokens of one sequence and one head, 16 a warp (the
// tile lists of the plain prefill kernel).  The block walks the pages from the first key its first token sees to its
// last token; a key page and a value page come into shared memory once (cp.async, two pages in flight) and are read
// by the 4 warps, each of which passes over the halves of a page that none of its own rows sees.  The 16-byte chunks
// of odd rows lie shifted by four chunks where rows are a multiple of 128 bytes apart (fragment reads without bank
// conflicts).
constexpr int kSinkTileWarps = 4;
constexpr int kSinkTileRows = kSinkTileWarps * 16;

template <int D, int DV>
struct SinkStage {
    static constexpr int kKeyChunks = D / 8;                              // 16-byte chunks of a key row
    static constexpr bool kSwizzleKeys = kKeyChunks % 8 == 0;
    static constexpr int kKeyBytes = kPageTokens * D * 2;
    static constexpr int kBytes = kKeyBytes + DV * kPageTokens * 2;       // a key page and a value page
};

template <int D, int DV>
__global__ void __launch_bounds__(kSinkTileWarps * 32)
sink_attention_tiles_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                            bf16* __restrict__ out, const int* __restrict__ tile_seq, const int* __restrict__ tile_row,
                            const int* __restrict__ cu_q, const int* __restrict__ kv_len, const int* __restrict__ slots,
                            const int* __restrict__ page_table, int max_pages, int window, int keep_first, int n_heads, int n_kv,
                            float scale, float cap, int sink, const float* __restrict__ sinks, const float* __restrict__ gate,
                            int64_t gate_stride) {
    using S = SinkStage<D, DV>;
    extern __shared__ __align__(128) unsigned char sink_smem[];
    const uint32_t stages = (uint32_t)__cvta_generic_to_shared(sink_smem);
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = lane & 3, g = lane >> 2;
    const int tile = gridDim.y - 1 - blockIdx.y;                 // later tiles of a sequence see more keys: they go first
    const int seq = tile_seq[tile], h = blockIdx.x;
    const int kvh = h / (n_heads / n_kv);
    const int q_begin = cu_q[seq], q_len = cu_q[seq + 1] - q_begin;
    const int tile_row0 = tile_row[tile];
    const int row0 = tile_row0 + 16 * warp;                      // first of this warp's 16 tokens
    const int history = kv_len[seq] - q_len;                     // keys cached before this step's tokens
    const int* pages = page_table + (int64_t)slots[seq] * max_pages;
    // the block's keys, and this warp's (empty when the warp has no rows)
    const int first_page = (window > 0 ? max(0, history + tile_row0 - window + 1) : 0) / kPageTokens;
    const int last_page = (history + min(tile_row0 + kSinkTileRows, q_len) - 1) / kPageTokens;
    const int my_first = window > 0 ? max(0, history + row0 - window + 1) : 0;
    const int my_last = row0 < q_len ? history + min(row0 + 16, q_len) - 1 : -1;
    // the pages of the kept first tokens that lie before the block's first page come first in the walk: step n of the
    // walk is page n while n < kept_pages, then page first_page + n - kept_pages
    const int kept_pages = min((keep_first + kPageTokens - 1) / kPageTokens, first_page);
    const int n_steps = kept_pages + last_page - first_page + 1;
    auto page_of = [&](int n) { return n < kept_pages ? n : first_page + n - kept_pages; };

    auto issue = [&](int n) {
        if (n < n_steps) {
            const int p = page_of(n);
            const int page = CPM_PAGE(pages, p, max_pages);
            const bf16* kpage = k_cache + page_row_offset(page, kvh, 0, n_kv, D);
            const bf16* vpage = v_cache + value_offset(page, kvh, 0, 0, n_kv, DV);
            const uint32_t stage = stages + (n & 1) * S::kBytes;
#pragma unroll 4
            for (int c = threadIdx.x; c < kPageTokens * S::kKeyChunks; c += kSinkTileWarps * 32) {
                const int row = c / S::kKeyChunks, col = c % S::kKeyChunks;
                const int pcol = S::kSwizzleKeys ? (col ^ ((row & 1) << 2)) : col;
                cp_async16(stage + (row * S::kKeyChunks + pcol) * 16, kpage + c * 8);
            }
#pragma unroll 4
            for (int c = threadIdx.x; c < DV * 8; c += kSinkTileWarps * 32) {
                const int row = c >> 3, col = c & 7;                       // a value row holds 64 tokens = 8 chunks
                cp_async16(stage + S::kKeyBytes + (row * 8 + (col ^ ((row & 1) << 2))) * 16, vpage + c * 8);
            }
        }
        cp_async_commit();
    };
    issue(0);
    issue(1);

    uint4 qf[2][D / 32];
    int lo[2], hi[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row0 + g + 8 * r;
        const bool valid = row < q_len;
        hi[r] = valid ? history + row : -1;
        lo[r] = (valid && window > 0) ? max(0, hi[r] - window + 1) : 0;
        const bf16* qrow = q + ((int64_t)(q_begin + (valid ? row : 0)) * n_heads + h) * D + 8 * j;
#pragma unroll
        for (int w = 0; w < D / 32; ++w) qf[r][w] = __ldg(reinterpret_cast<const uint4*>(qrow + 32 * w));
    }
    SinkTile<DV> st;
    st.init();
    for (int n = 0; n < n_steps; ++n) {
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t stage = stages + (n & 1) * S::kBytes;
        const int p = page_of(n);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int key0 = p * kPageTokens + 32 * u;
            if ((key0 + 31 < my_first && key0 >= keep_first) || key0 > my_last) continue;      // the same for the whole warp
            const int krow = 32 * u + 8 * (g >> 1) + (g & 1);
            sink_attend_keys<D, DV>(
                st, qf,
                [&](int t, int w) {
                    const int row = krow + 2 * t;
                    const int swz = S::kSwizzleKeys ? ((row & 1) << 2) : 0;
                    return lds16(stage + (row * S::kKeyChunks + ((4 * w + j) ^ swz)) * 16);
                },
                [&](int nt) {
                    const int row = 8 * nt + g;
                    return lds16(stage + S::kKeyBytes + (row * 8 + ((4 * u + j) ^ ((row & 1) << 2))) * 16);
                },
                key0, lo, hi, keep_first, scale, cap, lane);
        }
        __syncthreads();
        issue(n + 2);
    }
    cp_async_wait<0>();
    if (row0 >= q_len) return;
    constexpr float kLog2e = 1.4426950408889634f;
    const float b = sinks != nullptr ? sinks[h] * kLog2e : 0.f;
    const float sink_log2[2] = {b, b};
    float row_gate[2] = {1.f, 1.f};
    if (gate != nullptr) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = min(row0 + g + 8 * r, q_len - 1);
            row_gate[r] = 1.0f / (1.0f + __expf(-gate[(int64_t)(q_begin + row) * gate_stride + h]));
        }
    }
    sink_finish<DV>(st, sink, sink_log2, row_gate, lane, [&](int r) -> bf16* {
        const int row = row0 + g + 8 * r;
        return row < q_len ? out + ((int64_t)(q_begin + row) * n_heads + h) * DV : nullptr;
    });
}

// Single tokens (a decode step; also any step without tile lists): a block takes one token, one key-value head and up
// to 16 of the query heads that share it as the rows of a tile; its warps split the token's keys among them, 32 at a
// time, and join their maxima, sums and outputs through shared memory.
constexpr int kSinkTokenWarps = 4;

template <int D, int DV>
__global__ void __launch_bounds__(kSinkTokenWarps * 32)
sink_attention_token_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                            bf16* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ token_seq,
                            const int* __restrict__ slots, const int* __restrict__ page_table, int max_pages, int window,
                            int keep_first, int n_heads, int n_kv, float scale, float cap, int sink,
                            const float* __restrict__ sinks, const float* __restrict__ gate, int64_t gate_stride,
                            float* __restrict__ shares) {
    __shared__ float part_o[kSinkTokenWarps - 1][16][DV + 1];
    __shared__ float part_ml[kSinkTokenWarps - 1][16][2];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = lane & 3, g = lane >> 2;
    const int t = blockIdx.x;
    const int group = n_heads / n_kv, chunks = (group + 15) / 16;
    const int kvh = blockIdx.y / chunks, h0 = kvh * group + (blockIdx.y % chunks) * 16;
    const int rows = min(16, (kvh + 1) * group - h0);
    const int p = positions[t];
    const int* pages = page_table + (int64_t)slots[token_seq[t]] * max_pages;
    uint4 qf[2][D / 32];
    int lo[2], hi[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r;
        const bool valid = row < rows;
        hi[r] = valid ? p : -1;
        lo[r] = (valid && window > 0) ? max(0, p - window + 1) : 0;
        const bf16* qrow = q + ((int64_t)t * n_heads + h0 + (valid ? row : 0)) * D + 8 * j;
#pragma unroll
        for (int w = 0; w < D / 32; ++w) qf[r][w] = __ldg(reinterpret_cast<const uint4*>(qrow + 32 * w));
    }
    SinkTile<DV> st;
    st.init();
    const int first = (window > 0 ? max(0, p - window + 1) : 0) & ~31;
    // the steps of 32 keys that hold kept first tokens before the window come first: step b of the walk begins at key 32 b
    // while b < kept_steps, then at key first + 32 (b - kept_steps)
    const int kept_steps = min((keep_first + 31) / 32, first / 32);
    // the token's steps of 32 keys go to gridDim.z blocks (shares != null when more than one), a block's to its warps
    const int n_blocks = kept_steps + (p - first) / 32 + 1;
    const int per_block = (n_blocks + gridDim.z - 1) / gridDim.z;
    const int blk_begin = blockIdx.z * per_block, blk_end = min(n_blocks, blk_begin + per_block);
    const int share = (max(0, blk_end - blk_begin) + kSinkTokenWarps - 1) / kSinkTokenWarps;
    const int b_end = min(blk_end, blk_begin + (warp + 1) * share);
    for (int b = blk_begin + warp * share; b < b_end; ++b) {
        const int key0 = b < kept_steps ? 32 * b : first + 32 * (b - kept_steps);
        const int page = CPM_PAGE(pages, key0 / kPageTokens, max_pages), off = key0 % kPageTokens;
        const bf16* kp = k_cache + page_row_offset(page, kvh, off + 8 * (g >> 1) + (g & 1), n_kv, D) + 8 * j;
        const bf16* vp = v_cache + value_offset(page, kvh, g, off + 8 * j, n_kv, DV);
        sink_attend_keys<D, DV>(st, qf, [&](int t, int w) { return ldg16(kp + 2 * t * D + 32 * w); },
                                [&](int nt) { return ldg16(vp + nt * 8 * kPageTokens); }, key0, lo, hi, keep_first, scale, cap,
                                lane);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
    }
    if (warp > 0) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = g + 8 * r;
            if (j == 0) {
                part_ml[warp - 1][row][0] = st.m[r];
                part_ml[warp - 1][row][1] = st.l[r];
            }
#pragma unroll
            for (int nt = 0; nt < DV / 8; ++nt) {
                part_o[warp - 1][row][8 * nt + 2 * j] = st.o[nt][2 * r];
                part_o[warp - 1][row][8 * nt + 2 * j + 1] = st.o[nt][2 * r + 1];
            }
        }
    }
    __syncthreads();
    if (warp > 0) return;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r;
        float m = st.m[r];
#pragma unroll
        for (int w = 0; w < kSinkTokenWarps - 1; ++w) m = fmaxf(m, part_ml[w][row][0]);
        const float use = m == -INFINITY ? 0.f : m;
        const float mine = exp2f(st.m[r] - use);
        float l = st.l[r] * mine;
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt) {
            st.o[nt][2 * r] *= mine;
            st.o[nt][2 * r + 1] *= mine;
        }
#pragma unroll
        for (int w = 0; w < kSinkTokenWarps - 1; ++w) {
            const float f = exp2f(part_ml[w][row][0] - use);
            l += part_ml[w][row][1] * f;
#pragma unroll
            for (int nt = 0; nt < DV / 8; ++nt) {
                st.o[nt][2 * r] = fmaf(part_o[w][row][8 * nt + 2 * j], f, st.o[nt][2 * r]);
                st.o[nt][2 * r + 1] = fmaf(part_o[w][row][8 * nt + 2 * j + 1], f, st.o[nt][2 * r + 1]);
            }
        }
        if (row >= rows) continue;
        if (shares != nullptr) {            // this block's share as it is: the accumulator, the maximum it refers to, the sum
            float* dst = shares + (((int64_t)blockIdx.z * gridDim.x + t) * n_heads + h0 + row) * (DV + 2);
#pragma unroll
            for (int nt = 0; nt < DV / 8; ++nt)
                *reinterpret_cast<float2*>(dst + 8 * nt + 2 * j) = make_float2(st.o[nt][2 * r], st.o[nt][2 * r + 1]);
            if (j == 0) *reinterpret_cast<float2*>(dst + DV) = make_float2(m, l);
            continue;
        }
        float inv = sink_join(m, l, sink, sinks != nullptr ? sinks[h0 + row] * 1.4426950408889634f : 0.f);
        if (gate != nullptr) inv *= 1.0f / (1.0f + __expf(-gate[(int64_t)t * gate_stride + h0 + row]));
        bf16* orow = out + ((int64_t)t * n_heads + h0 + row) * DV + 2 * j;
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt)
            *reinterpret_cast<uint32_t*>(orow + 8 * nt) = pack_bf16(st.o[nt][2 * r] * inv, st.o[nt][2 * r + 1] * inv);
    }
}

// out[t, h, :] = sum_s o_s 2^(m_s - M) / (sink 2^(b_h - M) + sum_s l_s 2^(m_s - M)), M = max_s m_s, over the shares s of a
// token's keys (rows of dv + 2 floats: o, m, l), times the head's gate.  One warp per token and head.
__global__ void sink_combine_shares_kernel(const float* __restrict__ shares, bf16* __restrict__ out, int n_rows, int dv,
                                           int n_splits, int sink, const float* __restrict__ sinks,
                                           const float* __restrict__ gate, int64_t gate_stride, int n_heads) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    const int64_t stride = (int64_t)n_rows * (dv + 2);
    const float* mine = shares + (int64_t)row * (dv + 2);
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, mine[s * stride + dv]);
    const float use = m == -INFINITY ? 0.f : m;
    float l = 0.f, o[8];                       // channels lane, lane + 32, ... (dv <= 256)
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float* src = mine + s * stride;
        const float f = exp2f(src[dv] - use);
        l = fmaf(src[dv + 1], f, l);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (lane + 32 * i < dv) o[i] = fmaf(src[lane + 32 * i], f, o[i]);
    }
    const int h = row % n_heads;
    float inv = sink_join(use, l, sink, sinks != nullptr ? sinks[h] * 1.4426950408889634f : 0.f);
    if (m == -INFINITY) inv = 0.f;
    if (gate != nullptr) inv *= 1.0f / (1.0f + __expf(-gate[(int64_t)(row / n_heads) * gate_stride + h]));
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (lane + 32 * i < dv) out[(int64_t)row * dv + lane + 32 * i] = __float2bfloat16(o[i] * inv);
}

template <int D, int DV>
static int launch_sink_bf16(const void* q, const void* k_cache, const void* v_cache, void* out, const int* tile_seq,
                            const int* tile_row, int n_tiles, const int* cu_q, const int* kv_len, const int* positions,
                            const int* token_seq, const int* slots, const int* page_table, int max_pages, int window,
                            int keep_first, int n_tokens, int n_heads, int n_kv, float scale, float cap, int sink,
                            const float* sinks, const float* gate, int64_t gate_stride, float* shares, int n_splits,
                            cudaStream_t stream) {
    if (n_tiles > 0) {
        auto kern = sink_attention_tiles_kernel<D, DV>;
        constexpr int smem = 2 * SinkStage<D, DV>::kBytes;
        static bool configured[kMaxDevices] = {};            // per kernel and per device
        if (int st = ensure_dynamic_smem(kern, smem, configured)) return st;
        cpm_launch(kLaunchAttention, kern, dim3(n_heads, n_tiles), dim3(kSinkTileWarps * 32), smem,
                   stream, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, tile_seq, tile_row, cu_q,
                   kv_len, slots, page_table, max_pages, window, keep_first, n_heads, n_kv, scale, cap, sink, sinks, gate,
                   gate_stride);
    } else {
        const int group = n_heads / n_kv;
        cpm_launch(kLaunchAttention, sink_attention_token_kernel<D, DV>,
                   dim3(n_tokens, n_kv * ((group + 15) / 16), n_splits), dim3(kSinkTokenWarps * 32), 0, stream, (const bf16*)q,
                   (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, positions, token_seq, slots, page_table, max_pages,
                   window, keep_first, n_heads, n_kv, scale, cap, sink, sinks, gate, gate_stride,
                   n_splits > 1 ? shares : (float*)nullptr);
        if (n_splits > 1) {
            const int n_rows = n_tokens * n_heads;
            cpm_launch(kLaunchAttention, sink_combine_shares_kernel, dim3((n_rows + 3) / 4), dim3(128), 0, stream,
                       (const float*)shares, (bf16*)out, n_rows, DV, n_splits, sink, sinks, gate, gate_stride, n_heads);
        }
    }
    return launch_status();
}

// Whether the tensor-core kernels are built for these head sizes.
CPM_API int cpm_sink_attention_bf16_sizes(int d, int dv) {
    return (d == 32 || d == 64 || d == 96 || d == 128) && (dv == 32 || dv == 64 || dv == 96 || dv == 128);
}

// bf16 q [tokens, heads, d] -> out [tokens, heads * dv].  With n_tiles > 0 the tokens are prompt tokens packed by
// sequence (cu_q, kv_len, tile lists of 64 rows); else every token is taken alone by its position and sequence, its keys
// shared out over n_splits blocks (n_splits > 1: shares holds n_splits * tokens * heads * (dv + 2) floats).
CPM_API int cpm_sink_attention_bf16(const void* q, const void* k_cache, const void* v_cache, void* out, const int* tile_seq,
                                    const int* tile_row, int n_tiles, const int* cu_q, const int* kv_len,
                                    const int* positions, const int* token_seq, const int* slots, const int* page_table,
                                    int max_pages, int window, int keep_first, int n_tokens, int n_heads, int n_kv, int d, int dv,
                                    float scale, float cap, int sink, const float* sinks, const float* gate,
                                    int64_t gate_stride, float* shares, int n_splits, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (!cpm_sink_attention_bf16_sizes(d, dv) || n_kv <= 0 || n_heads % n_kv != 0 || window < 0 || keep_first < 0 || n_tiles > 65535 ||
        n_splits < 1 || n_splits > 65535 || (n_splits > 1 && !shares))
        return CPM_BAD_ARGUMENT;
    if (n_tiles > 0 ? (!tile_seq || !tile_row || !cu_q || !kv_len) : (!positions || !token_seq)) return CPM_BAD_ARGUMENT;
#define CPM_SINK_CASE(DD, VV)                                                                                              \
    if (d == DD && dv == VV)                                                                                               \
        return launch_sink_bf16<DD, VV>(q, k_cache, v_cache, out, tile_seq, tile_row, n_tiles, cu_q, kv_len, positions,    \
                                        token_seq, slots, page_table, max_pages, window, keep_first, n_tokens, n_heads,    \
                                        n_kv, scale, cap, sink, sinks, gate, gate_stride, shares, n_splits, stream);
#define CPM_SINK_ROW(DD) CPM_SINK_CASE(DD, 32) CPM_SINK_CASE(DD, 64) CPM_SINK_CASE(DD, 96) CPM_SINK_CASE(DD, 128)
    CPM_SINK_ROW(32) CPM_SINK_ROW(64) CPM_SINK_ROW(96) CPM_SINK_ROW(128)
#undef CPM_SINK_ROW
#undef CPM_SINK_CASE
    return CPM_BAD_ARGUMENT;
}

// In place: x[t][h][:] *= sigmoid(gate[t][h]) (an output gate per head); gate: fp32 rows of ``gate_stride`` floats.
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, const float* __restrict__ gate, int64_t gate_stride, int64_t n, int n_heads,
                                 int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t th = i / dv;
    const float z = gate[(th / n_heads) * gate_stride + th % n_heads];
    x[i] = from_f32<T>(to_f32(x[i]) / (1.0f + expf(-z)));
}

// The same for bf16 heads of a multiple of 8 channels: a thread takes 8 channels of one head (16-byte accesses).
__global__ void head_gate_bf16x8_kernel(bf16* __restrict__ x, const float* __restrict__ gate, int64_t gate_stride, int64_t n_vec,
                                        int n_heads, int vec_per_head) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_vec) return;
    const int64_t th = i / vec_per_head;
    const float f = 1.0f / (1.0f + expf(-gate[(th / n_heads) * gate_stride + th % n_heads]));
    uint4 v = *reinterpret_cast<const uint4*>(x + i * 8);
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 a = __bfloat1622float2(p[j]);
        p[j] = __floats2bfloat162_rn(a.x * f, a.y * f);
    }
    *reinterpret_cast<uint4*>(x + i * 8) = v;
}

CPM_API int cpm_head_gate(void* x, const float* gate, int64_t gate_stride, int n_tokens, int n_heads, int dv, int dtype,
                          cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (n_heads < 1 || dv < 1 || !gate) return CPM_BAD_ARGUMENT;
    const int64_t n = (int64_t)n_tokens * n_heads * dv;
    if (dtype == CPM_BF16 && dv % 8 == 0 && ((uintptr_t)x & 15) == 0) {
        cpm_launch(kLaunchOther, head_gate_bf16x8_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, stream, (bf16*)x, gate,
                   gate_stride, n / 8, n_heads, dv / 8);
        return launch_status();
    }
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchOther, head_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (bf16*)x, gate, gate_stride, n, n_heads, dv);
    else
        cpm_launch(kLaunchOther, head_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, gate, gate_stride, n, n_heads,
                   dv);
    return launch_status();
}

CPM_BOUNDS_TU(sink_attention)
