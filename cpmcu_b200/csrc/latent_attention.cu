// Attention over a cached latent: every token leaves one vector c of ``rank`` values in the cache, and the keys
// and values of all heads are linear maps of it, k_h = Uk_h c and v_h = Uv_h c.  With the key map moved to the query
// side and the value map behind the weighted sum,
//
//   score_h(i, j) = scale * (Uk_h^T q_h(i)) . c_j          o_h(i) = Uv_h (sum_j p_h(i, j) c_j)
//
// the attention runs on the cached latents themselves: one shared "key = value" row per token for all heads.
// A query at position p sees the keys j with 0 <= p - j < window (window 0: every j <= p).
//
//   latent_norm_store   RMS-norms the two parts of the fused down projection [tokens, q_rank + rank (+ rot_dim)] (fp32):
//                       the query latent goes on as an activation, the key-value latent into the cache pages, followed
//                       there by the rotated key part that all heads share (when the design has one)
//   rotate_heads        turns a range of channels of every head by the token's position
//   head_project        out[t, h, :] = in[t, h, :] @ w[h]   (w [heads][k][n]; fp32 accumulation), the per-head
//                       maps Uk^T (queries into the latent space) and Uv (weighted latents into values)
//   latent_attention    softmax attention of [tokens, heads, rank] fp32 queries over the latent pages (rank up to 1,024); scores,
//                       softmax and the weighted sum are fp32; a block is one token and up to 16 heads, which share
//                       every tile of 32 latent rows through shared memory
//
// A latent page is [token_in_page][rank] (the key page layout with one key-value head).
#include "common.cuh"

// ---------------------------------------------------------------------------
// proj rows (fp32, ``stride`` floats) begin [q_rank | rank | rot_dim]: the first two parts are RMS-normed; the third (rot_dim
// may be 0) is one key part shared by all heads that is turned by the token's position, pairs (c, c + rot_dim/2) or with
// ``adjacent`` (2c, 2c + 1), angle position * inv_freq[c], and not normed.  The cache row of the token is [rank | rot_dim].
template <typename T>
__global__ void latent_norm_store_kernel(const float* __restrict__ proj, int64_t stride, const float* __restrict__ wq,
                                         const float* __restrict__ wkv, T* __restrict__ cq, T* __restrict__ cache,
                                         const int* __restrict__ positions, const int* __restrict__ token_seq,
                                         const int* __restrict__ slots, const int* __restrict__ page_table, int max_pages,
                                         int q_rank, int rank, int rot_dim, const float* __restrict__ inv_freq, int adjacent,
                                         float eps) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const float* row = proj + (int64_t)t * stride;
    float s = 0.f;
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) s = fmaf(row[c], row[c], s);
    float r = 1.0f / sqrtf(block_sum(s, scratch) / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) cq[(int64_t)t * q_rank + c] = from_f32<T>(row[c] * r * wq[c]);
    row += q_rank;
    s = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) s = fmaf(row[c], row[c], s);
    r = 1.0f / sqrtf(block_sum(s, scratch) / (float)rank + eps);
    if (cache == nullptr) return;
    const int p = positions[t];
    const int* pages = page_table + (int64_t)slots[token_seq[t]] * max_pages;
    const int page = CPM_PAGE(pages, p / kPageTokens, max_pages);
    T* dst = cache + page_row_offset(page, 0, p % kPageTokens, 1, rank + rot_dim);
    for (int c = threadIdx.x; c < rank; c += blockDim.x) dst[c] = from_f32<T>(row[c] * r * wkv[c]);
    row += rank;
    dst += rank;
    const int half = rot_dim >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const int a = adjacent ? 2 * i : i, b = adjacent ? 2 * i + 1 : i + half;
        float sn = 0.f, cs = 1.f;
        if (inv_freq != nullptr) sincosf((float)p * inv_freq[i], &sn, &cs);
        const float u = row[a], v = row[b];
        dst[a] = from_f32<T>(u * cs - v * sn);
        dst[b] = from_f32<T>(v * cs + u * sn);
    }
}

CPM_API int cpm_latent_norm_store(const float* proj, int64_t stride, const float* wq, const float* wkv, void* cq, void* cache,
                                  const int* positions, const int* token_seq, const int* slots, const int* page_table,
                                  int max_pages, int n_tokens, int q_rank, int rank, int rot_dim, const float* inv_freq,
                                  int adjacent, float eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (q_rank <= 0 || rank <= 0 || rot_dim < 0 || (rot_dim & 1) || stride < q_rank + rank + rot_dim) return CPM_BAD_ARGUMENT;
    const int threads = (q_rank + rank) >= 1024 ? 256 : 128;
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchRope, latent_norm_store_kernel<bf16>, n_tokens, threads, 0, stream, proj, stride, wq, wkv, (bf16*)cq,
                   (bf16*)cache, positions, token_seq, slots, page_table, max_pages, q_rank, rank, rot_dim, inv_freq, adjacent, eps);
    else
        cpm_launch(kLaunchRope, latent_norm_store_kernel<float>, n_tokens, threads, 0, stream, proj, stride, wq, wkv, (float*)cq,
                   (float*)cache, positions, token_seq, slots, page_table, max_pages, q_rank, rank, rot_dim, inv_freq, adjacent,
                   eps);
    return launch_status();
}

// out[t][h][:] = in[t][h][:] (fp32 in, storage type out; heads of ``dh`` channels) with the channels [first, first + rot_dim)
// of every head turned by the token's position: pairs (c, c + rot_dim/2) or with ``adjacent`` (2c, 2c + 1) counted from
// ``first``, angle position * inv_freq[c].  One thread per pair or per channel outside the turned part.
template <typename T>
__global__ void rotate_heads_kernel(const float* __restrict__ in, T* __restrict__ out, const int* __restrict__ positions,
                                    const float* __restrict__ inv_freq, int64_t n_units, int n_heads, int dh, int first,
                                    int rot_dim, int adjacent) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_units) return;
    const int per_head = dh - rot_dim / 2;                  // plain channels and pairs of a head
    const int64_t th = i / per_head;
    const int u = (int)(i % per_head);
    const int64_t base = th * dh;
    const int plain = dh - rot_dim;
    if (u < plain) {
        const int c = u < first ? u : u + rot_dim;
        out[base + c] = from_f32<T>(in[base + c]);
        return;
    }
    const int k = u - plain, half = rot_dim >> 1;
    const int a = first + (adjacent ? 2 * k : k), b = first + (adjacent ? 2 * k + 1 : k + half);
    float sn, cs;
    sincosf((float)positions[th / n_heads] * inv_freq[k], &sn, &cs);
    const float x = in[base + a], y = in[base + b];
    out[base + a] = from_f32<T>(x * cs - y * sn);
    out[base + b] = from_f32<T>(y * cs + x * sn);
}

CPM_API int cpm_rotate_heads(const float* in, void* out, const int* positions, const float* inv_freq, int n_tokens, int n_heads,
                             int dh, int first, int rot_dim, int adjacent, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (n_heads < 1 || dh < 1 || first < 0 || rot_dim < 0 || (rot_dim & 1) || first + rot_dim > dh || (rot_dim && !inv_freq))
        return CPM_BAD_ARGUMENT;
    const int64_t n = (int64_t)n_tokens * n_heads * (dh - rot_dim / 2);
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchRope, rotate_heads_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, in, (bf16*)out, positions, inv_freq, n,
                   n_heads, dh, first, rot_dim, adjacent);
    else
        cpm_launch(kLaunchRope, rotate_heads_kernel<float>, dim3(blocks), dim3(256), 0, stream, in, (float*)out, positions, inv_freq,
                   n, n_heads, dh, first, rot_dim, adjacent);
    return launch_status();
}

// ---------------------------------------------------------------------------
constexpr int kProjectTokens = 8;      // tokens of one head that share a pass over the head's matrix
constexpr int kProjectCols = 32;       // output columns of a block
constexpr int kProjectParts = 8;       // parts of the sum over k, one per warp
constexpr int kProjectFlight = 16;     // rows of the matrix a thread asks for before it uses the first

// A block is 8 tokens x one head x 32 output columns; its eight warps split the sum over k (a warp reads 32
// consecutive columns of every eighth row of the head's matrix, sixteen rows in flight) and add up through shared memory.
template <typename In, typename Wt, typename Out>
__global__ void __launch_bounds__(kProjectCols * kProjectParts)
head_project_kernel(const In* __restrict__ in, const Wt* __restrict__ w, Out* __restrict__ out,
                    int n_tokens, int n_heads, int K, int N) {
    extern __shared__ float hp_smem[];      // [kProjectTokens][K] inputs, then [parts][tokens][cols] partial sums
    float* part = hp_smem + kProjectTokens * K;
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y;
    const int t0 = blockIdx.x * kProjectTokens;
    const int nt = min(kProjectTokens, n_tokens - t0);
    for (int i = threadIdx.x; i < kProjectTokens * K; i += blockDim.x) {
        const int tt = i / K, k = i % K;
        hp_smem[i] = tt < nt ? to_f32(in[((int64_t)(t0 + tt) * n_heads + h) * K + k]) : 0.f;
    }
    __syncthreads();
    const int col = threadIdx.x % kProjectCols, kp = threadIdx.x / kProjectCols;
    const int n = blockIdx.z * kProjectCols + col;
    const Wt* wh = w + (int64_t)h * K * N + (n < N ? n : 0);
    float acc[kProjectTokens];
#pragma unroll
    for (int tt = 0; tt < kProjectTokens; ++tt) acc[tt] = 0.f;
    int k = kp;
    for (; k + (kProjectFlight - 1) * kProjectParts < K; k += kProjectFlight * kProjectParts) {
        float wv[kProjectFlight];
#pragma unroll
        for (int u = 0; u < kProjectFlight; ++u) wv[u] = to_f32(wh[(int64_t)(k + u * kProjectParts) * N]);
#pragma unroll
        for (int u = 0; u < kProjectFlight; ++u)
#pragma unroll
            for (int tt = 0; tt < kProjectTokens; ++tt) acc[tt] = fmaf(hp_smem[tt * K + k + u * kProjectParts], wv[u], acc[tt]);
    }
    for (; k < K; k += kProjectParts) {
        const float wv = to_f32(wh[(int64_t)k * N]);
#pragma unroll
        for (int tt = 0; tt < kProjectTokens; ++tt) acc[tt] = fmaf(hp_smem[tt * K + k], wv, acc[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < kProjectTokens; ++tt) part[(kp * kProjectTokens + tt) * kProjectCols + col] = acc[tt];
    __syncthreads();
    const int tt = threadIdx.x / kProjectCols;            // 8 tokens x 32 columns = the block's 256 threads
    if (tt < nt && n < N) {
        float sum = 0.f;
#pragma unroll
        for (int p = 0; p < kProjectParts; ++p) sum += part[(p * kProjectTokens + tt) * kProjectCols + col];
        out[((int64_t)(t0 + tt) * n_heads + h) * N + n] = from_f32<Out>(sum);
    }
}

template <typename In, typename Wt, typename Out>
static int launch_head_project(const void* in, const void* w, void* out, int n_tokens, int n_heads, int K, int N,
                               cudaStream_t stream) {
    const size_t smem = (size_t)kProjectTokens * (K + kProjectParts * kProjectCols) * sizeof(float);
    auto kern = head_project_kernel<In, Wt, Out>;
    if (smem > 227 * 1024) return CPM_BAD_ARGUMENT;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid((n_tokens + kProjectTokens - 1) / kProjectTokens, n_heads, (N + kProjectCols - 1) / kProjectCols);
    const int threads = kProjectCols * kProjectParts;
    cpm_launch(kLaunchProduct, kern, grid, threads, smem, stream, (const In*)in, (const Wt*)w, (Out*)out, n_tokens, n_heads, K, N);
    return launch_status();
}

// in_f32 / out_f32: whether the activations on that side are fp32 (else the storage type ``dtype``); the matrix
// always has the storage type.
CPM_API int cpm_head_project(const void* in, const void* w, void* out, int n_tokens, int n_heads, int K, int N, int in_f32,
                             int out_f32, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (n_heads <= 0 || n_heads > 65535 || K <= 0 || N <= 0 || (N + kProjectCols - 1) / kProjectCols > 65535) return CPM_BAD_ARGUMENT;
    if (dtype == CPM_F32) return launch_head_project<float, float, float>(in, w, out, n_tokens, n_heads, K, N, stream);
    if (in_f32 && out_f32) return launch_head_project<float, bf16, float>(in, w, out, n_tokens, n_heads, K, N, stream);
    if (in_f32) return launch_head_project<float, bf16, bf16>(in, w, out, n_tokens, n_heads, K, N, stream);
    if (out_f32) return launch_head_project<bf16, bf16, float>(in, w, out, n_tokens, n_heads, K, N, stream);
    return launch_head_project<bf16, bf16, bf16>(in, w, out, n_tokens, n_heads, K, N, stream);
}

// ---------------------------------------------------------------------------
constexpr int kLatentTile = 32;        // latent rows per shared-memory tile (one per lane in the scores)
constexpr int kLatentMaxWarps = 16;    // heads per block

// RL = ceil(rank / 32): what a lane keeps of a head's weighted sum.
template <typename T, int RL>
__global__ void latent_attention_kernel(const float* __restrict__ q /* [tokens, heads, rank] */, const T* __restrict__ cache,
                                        float* __restrict__ out /* [tokens, heads, rank] */, const int* __restrict__ positions,
                                        const int* __restrict__ token_seq, const int* __restrict__ slots,
                                        const int* __restrict__ page_table, int max_pages, int window, int n_heads, int rank,
                                        float scale) {
    extern __shared__ float la_smem[];
    const int n_warps = blockDim.x >> 5;
    const int pitch = rank + 1;                       // odd pitch: lane j reads row j without bank conflicts
    float* qs = la_smem;                              // [warps][rank]
    float* tile = la_smem + n_warps * rank;           // [kLatentTile][pitch]
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int h = blockIdx.y * n_warps + warp;
    const bool live = h < n_heads;
    const int p = positions[t];
    const int* pages = page_table + (int64_t)slots[token_seq[t]] * max_pages;
    if (live) {
        const float* qrow = q + ((int64_t)t * n_heads + h) * rank;
        for (int c = lane; c < rank; c += 32) qs[warp * rank + c] = qrow[c] * scale;
    }
    float m = -INFINITY, l = 0.f;
    float acc[RL];
#pragma unroll
    for (int i = 0; i < RL; ++i) acc[i] = 0.f;

    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    for (int j0 = lo; j0 <= p; j0 += kLatentTile) {
        const int n_here = min(kLatentTile, p + 1 - j0);
        __syncthreads();                              // the tile of the previous iteration is no longer read
        for (int r = warp; r < n_here; r += n_warps) {
            const int j = j0 + r;
            const int page = CPM_PAGE(pages, j / kPageTokens, max_pages);
            const T* src = cache + page_row_offset(page, 0, j % kPageTokens, 1, rank);
            for (int c = lane; c < rank; c += 32) tile[r * pitch + c] = to_f32(src[c]);
        }
        __syncthreads();
        if (!live) continue;
        float s = -INFINITY;
        if (lane < n_here) {
            const float* row = tile + lane * pitch;
            const float* qh = qs + warp * rank;
            float dot = 0.f;
            for (int c = 0; c < rank; ++c) dot = fmaf(qh[c], row[c], dot);
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float pr = lane < n_here ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(pr);
#pragma unroll
        for (int i = 0; i < RL; ++i) acc[i] *= corr;
        m = m_new;
        for (int jj = 0; jj < n_here; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, pr, jj);
            const float* row = tile + jj * pitch;
#pragma unroll
            for (int i = 0; i < RL; ++i) {
                const int c = lane + 32 * i;
                if (c < rank) acc[i] = fmaf(pj, row[c], acc[i]);
            }
        }
    }
    if (!live) return;
    const float inv = l > 0.f ? 1.f / l : 0.f;
    float* orow = out + ((int64_t)t * n_heads + h) * rank;
#pragma unroll
    for (int i = 0; i < RL; ++i) {
        const int c = lane + 32 * i;
        if (c < rank) orow[c] = acc[i] * inv;
    }
}

template <typename T, int RL>
static int launch_latent_attention(const float* q, const void* cache, float* out, const int* positions, const int* token_seq,
                                   const int* slots, const int* page_table, int max_pages, int window, int n_tokens,
                                   int n_heads, int rank, float scale, cudaStream_t stream) {
    const int warps = n_heads < kLatentMaxWarps ? n_heads : kLatentMaxWarps;
    const size_t smem = ((size_t)warps * rank + (size_t)kLatentTile * (rank + 1)) * sizeof(float);
    auto kern = latent_attention_kernel<T, RL>;
    if (smem > 227 * 1024) return CPM_BAD_ARGUMENT;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid(n_tokens, (n_heads + warps - 1) / warps);
    cpm_launch(kLaunchOther, kern, grid, warps * 32, smem, stream, q, (const T*)cache, out, positions, token_seq, slots, page_table,
               max_pages, window, n_heads, rank, scale);
    return launch_status();
}

CPM_API int cpm_latent_attention(const float* q, const void* cache, float* out, const int* positions, const int* token_seq,
                                 const int* slots, const int* page_table, int max_pages, int window, int n_tokens, int n_heads,
                                 int rank, float scale, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (n_heads <= 0 || rank <= 0 || rank > 1024 || window < 0) return CPM_BAD_ARGUMENT;
#define CPM_LATENT(RL)                                                                                                        \
    return dtype == CPM_BF16                                                                                                  \
        ? launch_latent_attention<bf16, RL>(q, cache, out, positions, token_seq, slots, page_table, max_pages, window,       \
                                            n_tokens, n_heads, rank, scale, stream)                                           \
        : launch_latent_attention<float, RL>(q, cache, out, positions, token_seq, slots, page_table, max_pages, window,      \
                                             n_tokens, n_heads, rank, scale, stream)
    if (rank <= 64) { CPM_LATENT(2); }
    if (rank <= 128) { CPM_LATENT(4); }
    if (rank <= 256) { CPM_LATENT(8); }
    if (rank <= 512) { CPM_LATENT(16); }
    CPM_LATENT(32);
#undef CPM_LATENT
}

// ---------------------------------------------------------------------------
// The same attention on the tensor cores, for bf16 latents (mma.sync m16n8k16, fp32 accumulation).  A block is one
// token, up to 16 heads (the 16 rows of the tile) and one share of the token's keys; its four warps split the work
// of every tile of 32 latent rows twice: for the scores each warp takes 8 of the 32 keys over the whole rank, for the
// weighted sum each warp takes every fourth group of 8 latent columns over all 32 keys, the latent tile being read
// as the "key" operand straight from its rows and as the "value" operand through ldmatrix.trans.  Scores go through
// shared memory in fp32; the softmax statistics are kept by every warp alike.  With more than one share a block
// leaves (max, sum, unnormalised output) in scratch and a second kernel merges the shares.
constexpr int kMmaKeys = 32;
constexpr int kMmaRows = 16;

__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_exp2(float x) {      // 2^x, about two units in the last place; 0 for x = -inf
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

constexpr int kPageSlots = 256;       // page numbers of a block's keys kept in shared memory (beyond: read from the table);
                                      // 1 KiB, so that three blocks of the rank-512 kernel fit one SM's shared memory

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool real) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
    const int bytes = real ? 16 : 0;                                     // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// NT: column groups of 8 a warp may own in the weighted sum (rank <= 32 * NT); the same number bounds the 16-wide steps
// of the rank a warp owns in the scores (rank / 64, rounded up, <= NT / 2).  Per tile of 32 latent rows: the four warps
// split the rank for the scores (each keeps its part of the 16 query rows in registers for the whole kernel and leaves a
// partial 16 x 32 score tile in shared memory), every warp adds the four partials and keeps the softmax statistics, and
// the warps split the latent columns for the weighted sum.  Tiles arrive by cp.async one tile ahead, in two buffers.
// scratch per (token, head group, share): 16 * (rank + 2) floats.
template <int NT>
__global__ void __launch_bounds__(128)
latent_attention_mma_kernel(const float* __restrict__ q, const bf16* __restrict__ cache, void* __restrict__ out_any, int out_bf16,
                            float* __restrict__ scratch, const int* __restrict__ positions, const int* __restrict__ token_seq,
                            const int* __restrict__ slots, const int* __restrict__ page_table, int max_pages, int window,
                            int n_heads, int rank, float scale, int n_splits) {
    constexpr int KS = NT / 2;                                           // 16-wide steps of the rank per warp, at most
    extern __shared__ __align__(16) unsigned char lm_smem[];
    __shared__ int page_s[kPageSlots];
    const int pitch = rank + 8;                                          // bf16 elements per latent row in shared memory
    bf16* Ks = reinterpret_cast<bf16*>(lm_smem);                         // [2][32][pitch]
    float* Ss = reinterpret_cast<float*>(Ks + 2 * kMmaKeys * pitch);     // [4 warps][16 values][32 lanes]
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
    const int t = blockIdx.x, h0 = blockIdx.y * kMmaRows, split = blockIdx.z;
    const int p = positions[t];
    const int* pages = page_table + (int64_t)slots[token_seq[t]] * max_pages;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const int tiles_total = (p + 1 - lo + kMmaKeys - 1) / kMmaKeys;
    const int per = (tiles_total + n_splits - 1) / n_splits;
    const int tile0 = split * per, tile1 = min(tiles_total, tile0 + per);
    const int k_steps = rank / 16;

    // this warp's part of the queries, as A fragments: 16-wide steps warp, warp + 4, ... of the rank
    uint32_t qa[KS][4];
#pragma unroll
    for (int i = 0; i < KS; ++i) {
        const int ks = warp + 4 * i;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int h = h0 + g + 8 * (e & 1);
            const int c = ks * 16 + 2 * tg + 8 * (e >> 1);
            float2 v = make_float2(0.f, 0.f);
            if (ks < k_steps && h < n_heads) v = *reinterpret_cast<const float2*>(q + ((int64_t)t * n_heads + h) * rank + c);
            qa[i][e] = pack_bf16(v.x, v.y);
        }
    }
    const int first_page = (lo + tile0 * kMmaKeys) / kPageTokens;
    const int last_key = min(p, lo + tile1 * kMmaKeys - 1);
    const int n_block_pages = tile1 > tile0 ? last_key / kPageTokens - first_page + 1 : 0;
    const bool pages_in_smem = n_block_pages <= kPageSlots;
    if (pages_in_smem)
        for (int i = threadIdx.x; i < n_block_pages; i += blockDim.x) page_s[i] = CPM_PAGE(pages, first_page + i, max_pages);
    __syncthreads();

    const int vec_per_row = rank / 8;                                    // 16-byte pieces of a latent row
    // a warp brings every fourth row of a tile (the row's address worked out once), its lanes the row's 16-byte pieces
    auto fetch = [&](int tile, int buf) {
        const int j0 = lo + tile * kMmaKeys;
        bf16* dst = Ks + buf * kMmaKeys * pitch;
#pragma unroll
        for (int rr = 0; rr < kMmaKeys / 4; ++rr) {
            const int r = warp + 4 * rr;
            const int j = j0 + r;
            const bool real = j <= p;
            const bf16* src = cache;
            if (real) {
                const int lp = j / kPageTokens;
                const int page = pages_in_smem ? page_s[lp - first_page] : CPM_PAGE(pages, lp, max_pages);
                src = cache + page_row_offset(page, 0, j % kPageTokens, 1, rank);
            }
            for (int v = lane; v < vec_per_row; v += 32) cp_async_16(dst + r * pitch + 8 * v, real ? src + 8 * v : src, real);
        }
        cp_async_commit();
    };

    // softmax statistics in the base-2 domain: scores are multiplied by scale * log2(e) and weights are exp2
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};             // rows g and g + 8
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    const float scale2 = scale * 1.4426950408889634f;
    // this lane's row addresses of the ldmatrix loads, relative to a tile: four 8 x 8 pieces at once.
    // scores (keys as the n side): pieces (keys 0-7, k 0-7), (keys 0-7, k 8-15), (keys 8-15, k 0-7), (keys 8-15, k 8-15)
    const int s_off = ((lane >> 4) * 8 + (lane & 7)) * pitch + 8 * ((lane >> 3) & 1);
    // weighted sum (keys as the k side, transposed on the way): pieces keys 0-7, 8-15, 16-23, 24-31 of 8 columns
    const int v_off = lane * pitch + 8 * warp;
    float* mine = Ss + warp * 16 * 32;                                   // [16 values][32 lanes] of this warp's partial scores

    if (tile0 < tile1) fetch(tile0, 0);
    for (int tile = tile0; tile < tile1; ++tile) {
        const int buf = (tile - tile0) & 1;
        const int j0 = lo + tile * kMmaKeys;
        if (tile + 1 < tile1) {
            fetch(tile + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();                                                 // the tile is there for every warp
        const bf16* Kt = Ks + buf * kMmaKeys * pitch;
        // partial scores of all 32 keys over this warp's part of the rank: c[n] is the 16 x 8 piece of keys 8n .. 8n + 7
        float c[4][4];
#pragma unroll
        for (int n = 0; n < 4; ++n) c[n][0] = c[n][1] = c[n][2] = c[n][3] = 0.f;
        {
            const uint32_t s_base = (uint32_t)__cvta_generic_to_shared(Kt + s_off);
#pragma unroll
            for (int i = 0; i < KS; ++i) {
                const int ks = warp + 4 * i;
                if (ks < k_steps) {
#pragma unroll
                    for (int np = 0; np < 2; ++np) {
                        uint32_t b[4];
                        const uint32_t addr = s_base + (uint32_t)((16 * np * pitch + ks * 16) * sizeof(bf16));
                        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(addr));
                        mma_bf16_16816(c[2 * np], qa[i], b[0], b[1]);
                        mma_bf16_16816(c[2 * np + 1], qa[i], b[2], b[3]);
                    }
                }
            }
        }
        // the four warps' partial scores are added lane by lane: every warp ends up with the whole 16 x 32 tile in the
        // layout of its own accumulators, which is also the layout of the A fragments of the weighted sum
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) mine[(4 * n + e) * 32 + lane] = c[n][e];
        __syncthreads();
        // (in the same order in every warp, so that all warps hold the very same sums and statistics)
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float* cell = Ss + (4 * n + e) * 32 + lane;
                c[n][e] = (cell[0] + cell[16 * 32]) + (cell[2 * 16 * 32] + cell[3 * 16 * 32]);
            }
        // c[n][0], c[n][1]: row g, keys 8n + 2tg, + 1;  c[n][2], c[n][3]: row g + 8
        const bool ragged = j0 + kMmaKeys - 1 > p;                       // the block's last tile may reach past the query
        if (ragged) {
#pragma unroll
            for (int n = 0; n < 4; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (j0 + 8 * n + 2 * tg + (e & 1) > p) c[n][e] = -INFINITY;
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = -INFINITY;
#pragma unroll
            for (int n = 0; n < 4; ++n) mx = fmaxf(mx, fmaxf(c[n][2 * r], c[n][2 * r + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m[r], mx * scale2);                // finite: a tile holds at least one visible key
            corr[r] = fast_exp2(m[r] - m_new);                           // 0 at the first tile (m = -inf)
            float sum = 0.f;
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                c[n][2 * r] = fast_exp2(fmaf(c[n][2 * r], scale2, -m_new));
                c[n][2 * r + 1] = fast_exp2(fmaf(c[n][2 * r + 1], scale2, -m_new));
                sum += c[n][2 * r] + c[n][2 * r + 1];
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            l[r] = l[r] * corr[r] + sum;
            m[r] = m_new;
        }
        if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                acc[i][0] *= corr[0]; acc[i][1] *= corr[0];
                acc[i][2] *= corr[1]; acc[i][3] *= corr[1];
            }
        }
        uint32_t pa[2][4];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            pa[half][0] = pack_bf16(c[2 * half][0], c[2 * half][1]);          // row g,     keys 16 half + 2tg, + 1
            pa[half][1] = pack_bf16(c[2 * half][2], c[2 * half][3]);          // row g + 8
            pa[half][2] = pack_bf16(c[2 * half + 1][0], c[2 * half + 1][1]);  // row g,     keys 16 half + 8 + 2tg, + 1
            pa[half][3] = pack_bf16(c[2 * half + 1][2], c[2 * half + 1][3]);  // row g + 8
        }
        {
            const uint32_t v_base = (uint32_t)__cvta_generic_to_shared(Kt + v_off);
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                if (8 * (warp + 4 * i) < rank) {
                    uint32_t b[4];
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(v_base + (uint32_t)(32 * i * sizeof(bf16))));
                    mma_bf16_16816(acc[i], pa[0], b[0], b[1]);
                    mma_bf16_16816(acc[i], pa[1], b[2], b[3]);
                }
            }
        }
        __syncthreads();                                                 // this buffer and the scores may be overwritten
    }
    // rows g and g + 8 are heads h0 + g and h0 + g + 8; a thread holds columns col0 + 2tg, + 1 of its column groups
    if (n_splits == 1) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int h = h0 + g + 8 * r;
            if (h >= n_heads) continue;
            const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
            const int64_t o = ((int64_t)t * n_heads + h) * rank;
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                const int c = 8 * (warp + 4 * i) + 2 * tg;
                if (c >= rank) continue;
                if (out_bf16) *reinterpret_cast<uint32_t*>(static_cast<bf16*>(out_any) + o + c) = pack_bf16(acc[i][2 * r] * inv, acc[i][2 * r + 1] * inv);
                else *reinterpret_cast<float2*>(static_cast<float*>(out_any) + o + c) = make_float2(acc[i][2 * r] * inv, acc[i][2 * r + 1] * inv);
            }
        }
        return;
    }
    float* part = scratch + (((int64_t)t * gridDim.y + blockIdx.y) * n_splits + split) * kMmaRows * (rank + 2);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float* prow = part + (g + 8 * r) * (rank + 2);
        if (warp == 0 && tg == 0) { prow[rank] = m[r]; prow[rank + 1] = l[r]; }
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const int c = 8 * (warp + 4 * i) + 2 * tg;
            if (c < rank) { prow[c] = acc[i][2 * r]; prow[c + 1] = acc[i][2 * r + 1]; }
        }
    }
}

// One block per (token, head group, row of the tile): the shares' weights are worked out once, then the threads add up
// the shares' columns.
__global__ void latent_attention_merge_kernel(const float* __restrict__ scratch, void* __restrict__ out_any, int out_bf16, int n_heads,
                                              int rank, int n_splits) {
    __shared__ float weight[64];
    __shared__ float inv_l;
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, hg = blockIdx.y, r = blockIdx.z;
    const int h = hg * kMmaRows + r;
    if (h >= n_heads) return;
    const float* base = scratch + (((int64_t)t * gridDim.y + hg) * n_splits * kMmaRows + r) * (rank + 2);
    const int64_t share = (int64_t)kMmaRows * (rank + 2);
    if (threadIdx.x < 32) {
        float mx = -INFINITY;
        for (int s = threadIdx.x; s < n_splits; s += 32) mx = fmaxf(mx, base[s * share + rank]);
        mx = warp_max(mx);
        float l = 0.f;
        for (int s = threadIdx.x; s < n_splits; s += 32) {
            const float ms = base[s * share + rank];
            const float w = ms == -INFINITY ? 0.f : exp2f(ms - mx);      // the shares' maxima are base-2 logarithms
            weight[s] = w;
            l = fmaf(base[s * share + rank + 1], w, l);
        }
        l = warp_sum(l);
        if (threadIdx.x == 0) inv_l = l > 0.f ? 1.f / l : 0.f;
    }
    __syncthreads();
    const int64_t o = ((int64_t)t * n_heads + h) * rank;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        float acc = 0.f;
        for (int s0 = 0; s0 < n_splits; s0 += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = s0 + u < n_splits ? base[(s0 + u) * share + c] : 0.f;
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (s0 + u < n_splits) acc = fmaf(v[u], weight[s0 + u], acc);
        }
        const float res = acc * inv_l;
        if (out_bf16) static_cast<bf16*>(out_any)[o + c] = __float2bfloat16_rn(res);
        else static_cast<float*>(out_any)[o + c] = res;
    }
}

CPM_API int64_t cpm_latent_attention_scratch_floats(int n_tokens, int n_heads, int rank, int n_splits) {
    if (n_splits <= 1) return 0;
    return (int64_t)n_tokens * ((n_heads + kMmaRows - 1) / kMmaRows) * n_splits * kMmaRows * (rank + 2);
}

template <int NT>
static int launch_latent_mma(const float* q, const void* cache, void* out, int out_bf16, float* scratch, const int* positions,
                             const int* token_seq, const int* slots, const int* page_table, int max_pages, int window,
                             int n_tokens, int n_heads, int rank, float scale, int n_splits, cudaStream_t stream) {
    static bool smem_done[kMaxDevices];
    const size_t smem = (size_t)2 * kMmaKeys * (rank + 8) * sizeof(bf16) + (size_t)4 * 16 * 32 * sizeof(float);
    auto kern = latent_attention_mma_kernel<NT>;
    if (smem > 48 * 1024) {
        int dev = 0;
        cudaGetDevice(&dev);
        const bool first = dev >= 0 && dev < kMaxDevices && !smem_done[dev];
        if (int e = ensure_dynamic_smem(kern, (int)smem, smem_done)) return e;
        // all of the SM's unified memory as shared memory: three blocks of the rank-512 kernel then fit one SM
        if (first) cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    }
    const int groups = (n_heads + kMmaRows - 1) / kMmaRows;
    dim3 grid(n_tokens, groups, n_splits);
    cpm_launch(kLaunchAttention, kern, grid, 128, smem, stream, q, (const bf16*)cache, out, out_bf16, scratch, positions, token_seq, slots,
               page_table, max_pages, window, n_heads, rank, scale, n_splits);
    if (n_splits > 1)
        cpm_launch(kLaunchCombine, latent_attention_merge_kernel, dim3(n_tokens, groups, kMmaRows), 128, 0, stream, (const float*)scratch, out,
                   out_bf16, n_heads, rank, n_splits);
    return launch_status();
}

// bf16 latents, rank a multiple of 16 up to 512; ``out`` fp32, or bf16 with ``out_bf16``; ``scratch``: cpm_latent_attention_scratch_floats floats when n_splits > 1.
CPM_API int cpm_latent_attention_mma(const float* q, const void* cache, void* out, int out_bf16, float* scratch, const int* positions,
                                     const int* token_seq, const int* slots, const int* page_table, int max_pages, int window,
                                     int n_tokens, int n_heads, int rank, float scale, int n_splits, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (n_heads <= 0 || rank <= 0 || rank > 512 || rank % 16 || window < 0 || n_splits < 1 || n_splits > 64) return CPM_BAD_ARGUMENT;
    if (n_splits > 1 && scratch == nullptr) return CPM_BAD_ARGUMENT;
    if ((n_heads + kMmaRows - 1) / kMmaRows > 65535) return CPM_BAD_ARGUMENT;
    if (rank <= 128) return launch_latent_mma<4>(q, cache, out, out_bf16, scratch, positions, token_seq, slots, page_table, max_pages, window,
                                                  n_tokens, n_heads, rank, scale, n_splits, stream);
    if (rank <= 256) return launch_latent_mma<8>(q, cache, out, out_bf16, scratch, positions, token_seq, slots, page_table, max_pages, window,
                                                  n_tokens, n_heads, rank, scale, n_splits, stream);
    return launch_latent_mma<16>(q, cache, out, out_bf16, scratch, positions, token_seq, slots, page_table, max_pages, window, n_tokens,
                                 n_heads, rank, scale, n_splits, stream);
}

CPM_BOUNDS_TU(latent_attention)
