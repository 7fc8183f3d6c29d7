// Linear recurrences with a matrix state per head (gated linear attention, gated delta rule).
//
// Per head the state S is [d, dv] (key channels x value channels), fp32, carried from token to token for each
// sequence and kept in a per-sequence tensor [slots, heads, d, dv] (zeros at position 0).  One step:
//
//   S <- diag(a_t) S                a_t: one number per key channel, or one per head
//   u  = v_t                        (plain form)
//   u  = beta_t (v_t - S^T k_t)     (delta rule: what is stored under k_t is moved toward v_t)
//   S <- S + k_t u^T
//   o_t = S^T q_t * q_scale         (the read-out sees the current token's write)
//
// Every value column of S is independent of the others, so a column belongs to kLanes threads that split the
// key channels among them (registers), and a block holds kCols columns of one head and sequence and walks the
// sequence's tokens of the step, whose operands arrive eight tokens at a time in one of two shared-memory buffers
// (asynchronous copies, the next eight on their way while these are worked).  Query and key head of value head h: h / (heads / qk_heads).
//
// Around it: the short causal convolution over time with SiLU, the unit-length scaling of q and k, the gates of
// the delta rule, the decay of the gated linear attention, and the per-head RMS norm of the read-out times the
// output gate.  All of it fp32; only the last kernel's output has the storage type.
#include "common.cuh"

__device__ __forceinline__ float sigmoid_acc(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float silu_acc(float v) { return v / (1.0f + expf(-v)); }
// log(1 + e^v) without overflow
__device__ __forceinline__ float softplus_acc(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

constexpr int kRecThreads = 256;
constexpr int kRecTile = 8;    // tokens whose operands are staged in shared memory at a time

__device__ __forceinline__ void cp_async_f32(float* smem_dst, const float* gmem_src) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(dst), "l"(gmem_src) : "memory");
}

template <int W>
__device__ __forceinline__ float lanes_sum(float v) {      // over the W consecutive threads of a column
#pragma unroll
    for (int o = 1; o < W; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// kLanes threads share a column (8 for key sizes up to 32, 16 above: shorter chains of dependent products per token)
// and hold PER key channels each; a thread works kCpt adjacent columns at once (the key, query and decay operands are
// loaded once for all of them, and their chains of dependent instructions interleave); a block of 256 threads holds
// 256 / kLanes * kCpt columns.  Staged rows are kLanes * PER floats wide and zero (decay: one) beyond d, so the walk
// needs no bounds.
template <int kLanes, int PER, int kCpt, bool DELTA, bool VECTOR_DECAY>
__global__ void __launch_bounds__(kRecThreads)
linear_recurrence_kernel(const float* __restrict__ q, const float* __restrict__ k, int64_t qk_stride,      // [tokens, qk_heads, d]
                         const float* __restrict__ v, int64_t v_stride,                                    // [tokens, heads, dv]
                         const float* __restrict__ decay, int64_t decay_stride,                            // [tokens, heads(, d)]
                         const float* __restrict__ beta, int64_t beta_stride,                              // [tokens, heads]
                         float* __restrict__ state, const int* __restrict__ positions, const int* __restrict__ cu_q,
                         const int* __restrict__ slots, float* __restrict__ out,                           // [tokens, heads, dv]
                         int heads, int qk_heads, int d, int dv, float q_scale) {
    extern __shared__ float rec_smem[];
    constexpr int kCols = kRecThreads / kLanes * kCpt;           // columns of the block
    constexpr int kWide = kLanes * PER;                          // floats of a staged row of key channels
    constexpr int kAcc = PER >= 8 ? 4 : 2;
    constexpr int kAWidth = VECTOR_DECAY ? kWide : 1;
    constexpr int kStage = kRecTile * (2 * kWide + kAWidth + kCols + 1);
    pdl_launch_dependents();
    // the staged rows' tails beyond d are never copied to: zero (decay: one) for good
    for (int i = threadIdx.x; i < 2 * kStage; i += blockDim.x) {
        const int at = i % kStage;
        rec_smem[i] = (VECTOR_DECAY && at >= 2 * kRecTile * kWide && at < 3 * kRecTile * kWide) ? 1.f : 0.f;
    }
    pdl_wait();
    const int lane = threadIdx.x % kLanes;
    const int lcol = (threadIdx.x / kLanes) * kCpt;              // first of the thread's columns inside the block
    const int col0 = blockIdx.x * kCols;
    const int h = blockIdx.y, seq = blockIdx.z;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    if (t1 <= t0) return;
    const int g = h / (heads / qk_heads);
    float* st = state + (((int64_t)slots[seq] * heads + h) * d) * dv;
    const bool fresh = positions[t0] == 0;
    float S[kCpt][PER];
#pragma unroll
    for (int j = 0; j < kCpt; ++j)
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int c = lane + kLanes * i, col = col0 + lcol + j;
            S[j][i] = (c < d && col < dv && !fresh) ? st[(int64_t)c * dv + col] : 0.f;
        }
    __syncthreads();
    // the operands of up to kRecTile tokens from ``tb`` on are asked for (asynchronous copies into buffer ``buf``)
    auto stage_in = [&](int tb, int buf) {
        float* qs = rec_smem + buf * kStage;
        float* ks = qs + kRecTile * kWide;
        float* as = ks + kRecTile * kWide;
        float* vs = as + kRecTile * kAWidth;
        float* bs = vs + kRecTile * kCols;
        const int nt = min(kRecTile, t1 - tb);
        for (int i = threadIdx.x; i < nt * d; i += blockDim.x) {
            const int tok = i / d, c = i % d;
            cp_async_f32(qs + tok * kWide + c, q + (int64_t)(tb + tok) * qk_stride + (int64_t)g * d + c);
            cp_async_f32(ks + tok * kWide + c, k + (int64_t)(tb + tok) * qk_stride + (int64_t)g * d + c);
            if (VECTOR_DECAY) cp_async_f32(as + tok * kWide + c, decay + (int64_t)(tb + tok) * decay_stride + (int64_t)h * d + c);
        }
        for (int i = threadIdx.x; i < nt * kCols; i += blockDim.x) {
            const int tok = i / kCols, c = min(col0 + i % kCols, dv - 1);
            cp_async_f32(vs + i, v + (int64_t)(tb + tok) * v_stride + (int64_t)h * dv + c);
        }
        if (threadIdx.x < nt) {
            if (!VECTOR_DECAY) cp_async_f32(as + threadIdx.x, decay + (int64_t)(tb + threadIdx.x) * decay_stride + h);
            if (DELTA) cp_async_f32(bs + threadIdx.x, beta + (int64_t)(tb + threadIdx.x) * beta_stride + h);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage_in(t0, 0);
    int buf = 0;
    // The read-out of a token is summed over the column's threads one token late, in the same shuffle rounds as the
    // next token's S^T k: only that sum lies on the chain from one token's state to the next, and a warp that waits for
    // one round of shuffles waits for both.
    float pend[kCpt];
#pragma unroll
    for (int j = 0; j < kCpt; ++j) pend[j] = 0.f;
    int64_t pend_row = -1;
    for (int tb = t0; tb < t1; tb += kRecTile, buf ^= 1) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                         // this tile has arrived; the other buffer is free again
        if (tb + kRecTile < t1) stage_in(tb + kRecTile, buf ^ 1);
        const float* qs = rec_smem + buf * kStage + lane;
        const float* ks = qs + kRecTile * kWide;
        const float* as = ks + kRecTile * kWide;
        const float* vs = rec_smem + buf * kStage + kRecTile * (2 * kWide + kAWidth) + lcol;
        const float* bs = rec_smem + buf * kStage + kRecTile * (2 * kWide + kAWidth + kCols);
        const int nt = min(kRecTile, t1 - tb);
        auto step = [&](int tok) {
            float ck[PER], cq[PER], u[kCpt];
            const float a1 = VECTOR_DECAY ? 1.f : as[tok - lane];
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                ck[i] = ks[tok * kWide + kLanes * i];
                cq[i] = qs[tok * kWide + kLanes * i];
                const float a = VECTOR_DECAY ? as[tok * kWide + kLanes * i] : a1;
#pragma unroll
                for (int j = 0; j < kCpt; ++j) S[j][i] *= a;
            }
#pragma unroll
            for (int j = 0; j < kCpt; ++j) u[j] = vs[tok * kCols + j];
            float dot[kCpt][kAcc] = {};                         // partial sums: short chains of dependent products
            if (DELTA) {
#pragma unroll
                for (int i = 0; i < PER; ++i)
#pragma unroll
                    for (int j = 0; j < kCpt; ++j) dot[j][i % kAcc] = fmaf(S[j][i], ck[i], dot[j][i % kAcc]);
#pragma unroll
                for (int j = 0; j < kCpt; ++j)
#pragma unroll
                    for (int w = kAcc / 2; w > 0; w >>= 1)
#pragma unroll
                        for (int i = 0; i < w; ++i) dot[j][i] += dot[j][i + w];
            }
#pragma unroll
            for (int o = 1; o < kLanes; o <<= 1)
#pragma unroll
                for (int j = 0; j < kCpt; ++j) {
                    if (DELTA) dot[j][0] += __shfl_xor_sync(0xffffffffu, dot[j][0], o);
                    pend[j] += __shfl_xor_sync(0xffffffffu, pend[j], o);
                }
            if (pend_row >= 0 && lane == 0) {
#pragma unroll
                for (int j = 0; j < kCpt; ++j)
                    if (col0 + lcol + j < dv) out[(pend_row * heads + h) * dv + col0 + lcol + j] = pend[j] * q_scale;
            }
            if (DELTA) {
                const float b = bs[tok];
#pragma unroll
                for (int j = 0; j < kCpt; ++j) u[j] = b * (u[j] - dot[j][0]);
            }
            float op[kCpt][kAcc] = {};
#pragma unroll
            for (int i = 0; i < PER; ++i)
#pragma unroll
                for (int j = 0; j < kCpt; ++j) {
                    S[j][i] = fmaf(ck[i], u[j], S[j][i]);
                    op[j][i % kAcc] = fmaf(S[j][i], cq[i], op[j][i % kAcc]);
                }
#pragma unroll
            for (int j = 0; j < kCpt; ++j) {
#pragma unroll
                for (int w = kAcc / 2; w > 0; w >>= 1)
#pragma unroll
                    for (int i = 0; i < w; ++i) op[j][i] += op[j][i + w];
                pend[j] = op[j][0];
            }
            pend_row = tb + tok;
        };
        if (nt == kRecTile) {                                    // a full tile: unrolled, so that later tokens' operands are loaded early
#pragma unroll
            for (int tok = 0; tok < kRecTile; ++tok) step(tok);
        } else {
            for (int tok = 0; tok < nt; ++tok) step(tok);
        }
    }
#pragma unroll
    for (int j = 0; j < kCpt; ++j) {                             // the last token's read-out
        const float o = lanes_sum<kLanes>(pend[j]);
        if (lane == 0 && col0 + lcol + j < dv) out[(pend_row * heads + h) * dv + col0 + lcol + j] = o * q_scale;
    }
#pragma unroll
    for (int j = 0; j < kCpt; ++j)
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int c = lane + kLanes * i, col = col0 + lcol + j;
            if (c < d && col < dv) st[(int64_t)c * dv + col] = S[j][i];
        }
}

template <int LANES, int PER, int CPT>
static void launch_recurrence(bool delta, bool vector_decay, cudaStream_t stream, const float* q, const float* k,
                              int64_t qk_stride, const float* v, int64_t v_stride, const float* decay, int64_t decay_stride,
                              const float* beta, int64_t beta_stride, float* state, const int* positions, const int* cu_q,
                              const int* slots, float* out, int n_seqs, int heads, int qk_heads, int d, int dv, float q_scale) {
    constexpr int cols = kRecThreads / LANES * CPT;
    const dim3 grid((dv + cols - 1) / cols, heads, n_seqs), block(kRecThreads);
    const size_t smem = 2 * (size_t)kRecTile * (2 * LANES * PER + (vector_decay ? LANES * PER : 1) + cols + 1) * sizeof(float);
#define CPM_REC(D, V) do {                                                                                                          \
        static bool configured[kMaxDevices] = {};                                                                                   \
        if (smem > 48 * 1024 &&                                                                                                     \
            ensure_dynamic_smem(linear_recurrence_kernel<LANES, PER, CPT, D, V>, 100 * 1024, configured) != CPM_OK) return;         \
        cpm_launch(kLaunchAttention, linear_recurrence_kernel<LANES, PER, CPT, D, V>, grid, block, smem, stream, q, k, qk_stride,   \
                   v, v_stride, decay, decay_stride, beta, beta_stride, state, positions, cu_q, slots, out, heads, qk_heads, d, dv, \
                   q_scale);                                                                                                        \
    } while (0)
    if (delta && vector_decay) CPM_REC(true, true);
    else if (delta) CPM_REC(true, false);
    else if (vector_decay) CPM_REC(false, true);
    else CPM_REC(false, false);
#undef CPM_REC
}

static int g_recurrence_columns = 1;
// Columns a thread works at once: 1 (default) or 2 (measured slower on a prompt: 857 against 749 us for 16 heads of 128 x 128).
CPM_API int cpm_set_recurrence_columns(int n) {
    g_recurrence_columns = n;
    return CPM_OK;
}

// q, k: fp32 rows of ``qk_stride`` floats holding [qk_heads, d]; v: rows of ``v_stride`` floats holding [heads, dv];
// decay: rows of ``decay_stride`` floats holding [heads, d] (vector_decay) or [heads]; beta: rows holding [heads], or
// null for the plain form.  state [slots, heads, d, dv] fp32.  out [tokens, heads, dv] fp32.
CPM_API int cpm_linear_recurrence(const float* q, const float* k, int64_t qk_stride, const float* v, int64_t v_stride,
                                  const float* decay, int64_t decay_stride, int vector_decay, const float* beta,
                                  int64_t beta_stride, float* state, const int* positions, const int* cu_q, const int* slots,
                                  float* out, int n_seqs, int heads, int qk_heads, int d, int dv, float q_scale,
                                  cudaStream_t stream) {
    if (n_seqs <= 0) return CPM_OK;
    if (heads < 1 || qk_heads < 1 || heads % qk_heads || d < 1 || dv < 1 || d > 256) return CPM_BAD_ARGUMENT;
    const bool delta = beta != nullptr;
#define CPM_REC_PER(L, P, C) launch_recurrence<L, P, C>(delta, vector_decay != 0, stream, q, k, qk_stride, v, v_stride, decay,        \
                                                        decay_stride, beta, beta_stride, state, positions, cu_q, slots, out, n_seqs, \
                                                        heads, qk_heads, d, dv, q_scale)
    // two columns a thread where that still leaves blocks enough (a decode batch, or value heads of 64 and more)
    const bool two = g_recurrence_columns == 2 && dv >= 32;
    if (d <= 32) { if (two) CPM_REC_PER(8, 4, 2); else CPM_REC_PER(8, 4, 1); }
    else if (d <= 64) { if (two) CPM_REC_PER(16, 4, 2); else CPM_REC_PER(16, 4, 1); }      // 451 us against 505 with 8 threads of 8 channels
    else if (d <= 128) { if (two) CPM_REC_PER(16, 8, 2); else CPM_REC_PER(16, 8, 1); }
    else { if (two) CPM_REC_PER(16, 16, 2); else CPM_REC_PER(16, 16, 1); }
#undef CPM_REC_PER
    return launch_status();
}

// ---------------------------------------------------------------------------
// Short causal convolution over time, SiLU, unit length, and the delta rule's gates.
//
// proj rows (fp32, ``stride`` floats) begin with [q: qk_heads*d | k: qk_heads*d | v: heads*dv]; these C channels each
// pass y_t = sum_j taps[c][K-1-j] x_(t-j) (zeros before the sequence's start) and SiLU.  The K-1 inputs before a
// step's first token come from conv_state [slots, K-1, C] (oldest first).  q and k heads are then scaled to unit
// length, x / sqrt(sum x^2 + unit_eps).  One warp per (token, head of q, k or v).  For value head h the first lane
// also forms beta = sigmoid(b_raw) and the decay exp(-exp(A_log[h]) * softplus(a_raw + dt_bias[h])) from the
// columns ``b_col + h`` and ``a_col + h`` of the row (no decay when ``decay`` is null: a caller that forms its own).
// ---------------------------------------------------------------------------
constexpr int kConvMaxPerLane = 8;      // head sizes up to 256
constexpr int kConvMaxTaps = 8;

__global__ void conv_prepare_kernel(const float* __restrict__ proj, int64_t stride, const float* __restrict__ taps,
                                    const float* __restrict__ conv_state, const int* __restrict__ positions,
                                    const int* __restrict__ token_seq, const int* __restrict__ cu_q,
                                    const int* __restrict__ slots, float* __restrict__ qo, float* __restrict__ ko,
                                    float* __restrict__ vo, float* __restrict__ beta, float* __restrict__ decay,
                                    const float* __restrict__ a_log, const float* __restrict__ dt_bias, int b_col, int a_col,
                                    int heads, int qk_heads, int d, int dv, int K, float unit_eps, int n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int units = 2 * qk_heads + heads;
    const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (int64_t)n_tokens * units) return;
    const int t = (int)(w / units), unit = (int)(w % units);
    const int C = 2 * qk_heads * d + heads * dv;
    int width, c0;
    float* dst;
    if (unit < qk_heads) { width = d; c0 = unit * d; dst = qo + ((int64_t)t * qk_heads + unit) * d; }
    else if (unit < 2 * qk_heads) { width = d; c0 = unit * d; dst = ko + ((int64_t)t * qk_heads + unit - qk_heads) * d; }
    else { width = dv; c0 = 2 * qk_heads * d + (unit - 2 * qk_heads) * dv; dst = vo + ((int64_t)t * heads + unit - 2 * qk_heads) * dv; }
    const int seq = token_seq[t];
    const int local = t - cu_q[seq], pos = positions[t];
    const float* cs = conv_state + (int64_t)slots[seq] * (K - 1) * C;
    float val[kConvMaxPerLane];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kConvMaxPerLane; ++i) {
        const int e = lane + 32 * i;
        float acc = 0.f;
        if (e < width) {
            const int c = c0 + e;
            for (int j = 0; j < K; ++j) {              // tap j reaches j tokens back
                if (pos - j < 0) break;
                const float x = local - j >= 0 ? proj[(int64_t)(t - j) * stride + c] : cs[(int64_t)(K - 1 + local - j) * C + c];
                acc = fmaf(taps[(int64_t)c * K + K - 1 - j], x, acc);
            }
            acc = silu_acc(acc);
        }
        val[i] = acc;
        ss = fmaf(acc, acc, ss);
    }
    float f = 1.f;
    if (unit < 2 * qk_heads) f = 1.0f / sqrtf(warp_sum(ss) + unit_eps);
#pragma unroll
    for (int i = 0; i < kConvMaxPerLane; ++i) {
        const int e = lane + 32 * i;
        if (e < width) dst[e] = val[i] * f;
    }
    if (unit >= 2 * qk_heads && lane == 0) {
        const int h = unit - 2 * qk_heads;
        const float* row = proj + (int64_t)t * stride;
        beta[(int64_t)t * heads + h] = sigmoid_acc(row[b_col + h]);
        if (decay != nullptr) decay[(int64_t)t * heads + h] = expf(-expf(a_log[h]) * softplus_acc(row[a_col + h] + dt_bias[h]));
    }
}

// The convolution's state after the step: for every sequence the last K-1 inputs, taken from the step's rows and,
// where the step brought fewer, from the old state.  A thread owns a channel and reads all it needs before it
// writes.  Runs after conv_prepare_kernel, which only reads the state.
__global__ void conv_state_update_kernel(const float* __restrict__ proj, int64_t stride, float* __restrict__ conv_state,
                                         const int* __restrict__ positions, const int* __restrict__ cu_q,
                                         const int* __restrict__ slots, int C, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int seq = blockIdx.y;
    if (c >= C) return;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    const int n = t1 - t0;
    if (n <= 0) return;
    const bool fresh = positions[t0] == 0;
    float* cs = conv_state + (int64_t)slots[seq] * (K - 1) * C + c;
    float keep[kConvMaxTaps];
#pragma unroll
    for (int i = 0; i < kConvMaxTaps; ++i) {
        if (i < K - 1) {
            const int back = K - 1 - i;                // entry i is the input ``back`` tokens before the next token
            if (back <= n) keep[i] = proj[(int64_t)(t1 - back) * stride + c];
            else keep[i] = fresh ? 0.f : cs[(int64_t)(i + n) * C];
        }
    }
#pragma unroll
    for (int i = 0; i < kConvMaxTaps; ++i)
        if (i < K - 1) cs[(int64_t)i * C] = keep[i];
}

CPM_API int cpm_conv_prepare(const float* proj, int64_t stride, const float* taps, float* conv_state, const int* positions,
                             const int* token_seq, const int* cu_q, const int* slots, float* qo, float* ko, float* vo,
                             float* beta, float* decay, const float* a_log, const float* dt_bias, int b_col, int a_col,
                             int n_tokens, int n_seqs, int heads, int qk_heads, int d, int dv, int K, float unit_eps,
                             cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (K < 1 || K > kConvMaxTaps || d > 32 * kConvMaxPerLane || dv > 32 * kConvMaxPerLane || heads < 1 || qk_heads < 1)
        return CPM_BAD_ARGUMENT;
    const int units = 2 * qk_heads + heads;
    const int warps = 8;
    const int64_t blocks = ((int64_t)n_tokens * units + warps - 1) / warps;
    cpm_launch(kLaunchRope, conv_prepare_kernel, dim3((unsigned)blocks), dim3(warps * 32), 0, stream, proj, stride, taps,
               (const float*)conv_state, positions, token_seq, cu_q, slots, qo, ko, vo, beta, decay, a_log, dt_bias, b_col, a_col,
               heads, qk_heads, d, dv, K, unit_eps, n_tokens);
    if (K > 1) {
        const int C = 2 * qk_heads * d + heads * dv;
        cpm_launch(kLaunchOther, conv_state_update_kernel, dim3((C + 127) / 128, n_seqs), dim3(128), 0, stream, proj, stride,
                   conv_state, positions, cu_q, slots, C, K);
    }
    return launch_status();
}

// A decay per head and key channel, in place on fp32 rows [heads * d]:
//   z <- exp(-exp(a_log[h]) * softplus(z + dt_bias[h * d + c]))
__global__ void channel_decay_kernel(float* __restrict__ z, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                     int64_t n, int width, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int c = (int)(i % width);
    z[i] = expf(-expf(a_log[c / d]) * softplus_acc(z[i] + dt_bias[c]));
}

CPM_API int cpm_channel_decay(float* z, const float* a_log, const float* dt_bias, int n_tokens, int heads, int d,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (heads < 1 || d < 1) return CPM_BAD_ARGUMENT;
    const int64_t n = (int64_t)n_tokens * heads * d;
    cpm_launch(kLaunchOther, channel_decay_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, z, a_log, dt_bias, n,
               heads * d, d);
    return launch_status();
}

// Decay of the gated linear attention, in place: z <- sigmoid(z + bias)^(1/tau) = exp(-softplus(-(z + bias)) / tau).
__global__ void sigmoid_power_kernel(float* __restrict__ z, const float* __restrict__ bias, float inv_tau, int64_t n, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = z[i] + bias[i % width];
    z[i] = expf(-softplus_acc(-v) * inv_tau);
}

CPM_API int cpm_sigmoid_power(float* z, const float* bias, float tau, int n_tokens, int width, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (width < 1 || !(tau > 0.f)) return CPM_BAD_ARGUMENT;
    const int64_t n = (int64_t)n_tokens * width;
    cpm_launch(kLaunchOther, sigmoid_power_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, z, bias, 1.0f / tau, n, width);
    return launch_status();
}

// out[t][h][:] = o[t][h][:] / sqrt(mean(o^2) + eps) * weight[:] * act(gate[t][h][:]), act = SiLU or (gate_act 1) the
// sigmoid, one warp per (token, head);
// o fp32 [tokens, heads, dv], gate fp32 rows of ``gate_stride`` floats holding [heads, dv], out in the storage type.
template <typename T>
__global__ void gated_head_norm_kernel(const float* __restrict__ o, const float* __restrict__ gate, int64_t gate_stride,
                                       const float* __restrict__ weight, T* __restrict__ out, int heads, int dv, float eps,
                                       int64_t n_units, int gate_act) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= n_units) return;
    const int64_t t = w / heads;
    const int h = (int)(w % heads);
    const float* row = o + w * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(row[c], row[c], ss);
    const float f = rsqrtf(warp_sum(ss) / (float)dv + eps);
    const float* gr = gate + t * gate_stride + (int64_t)h * dv;
    for (int c = lane; c < dv; c += 32)
        out[w * dv + c] = from_f32<T>(row[c] * f * weight[c] * (gate_act == 1 ? sigmoid_acc(gr[c]) : silu_acc(gr[c])));
}

CPM_API int cpm_gated_head_norm(const float* o, const float* gate, int64_t gate_stride, const float* weight, void* out,
                                int n_tokens, int heads, int dv, float eps, int gate_act, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (heads < 1 || dv < 1 || gate_act < 0 || gate_act > 1) return CPM_BAD_ARGUMENT;
    const int64_t units = (int64_t)n_tokens * heads;
    const int warps = 8;
    const dim3 grid((unsigned)((units + warps - 1) / warps));
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchNorm, gated_head_norm_kernel<bf16>, grid, dim3(warps * 32), 0, stream, o, gate, gate_stride, weight, (bf16*)out,
                   heads, dv, eps, units, gate_act);
    else
        cpm_launch(kLaunchNorm, gated_head_norm_kernel<float>, grid, dim3(warps * 32), 0, stream, o, gate, gate_stride, weight,
                   (float*)out, heads, dv, eps, units, gate_act);
    return launch_status();
}

// The same over groups of ``group`` heads normed together (group = heads: all of a token's heads as one vector), with a
// weight per channel of the group [group * dv] and the gate's activation chosen (0: SiLU, 1: sigmoid); one block per
// (token, group).
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ o, const float* __restrict__ gate, int64_t gate_stride,
                                        const float* __restrict__ weight, T* __restrict__ out, int heads, int dv, int group,
                                        int gate_act, float eps) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int width = group * dv, groups = heads / group;
    const int64_t t = blockIdx.x / groups;
    const int g = blockIdx.x % groups;
    const float* row = o + (t * heads + (int64_t)g * group) * dv;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
    const float f = rsqrtf(block_sum(ss, scratch) / (float)width + eps);
    const float* gr = gate + t * gate_stride + (int64_t)g * width;
    T* dst = out + (t * heads + (int64_t)g * group) * dv;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float a = gate_act == 1 ? sigmoid_acc(gr[c]) : silu_acc(gr[c]);
        dst[c] = from_f32<T>(row[c] * f * weight[c] * a);
    }
}

CPM_API int cpm_gated_group_norm(const float* o, const float* gate, int64_t gate_stride, const float* weight, void* out,
                                 int n_tokens, int heads, int dv, int group, int gate_act, float eps, int dtype,
                                 cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (heads < 1 || dv < 1 || group < 1 || heads % group || gate_act < 0 || gate_act > 1) return CPM_BAD_ARGUMENT;
    const int width = group * dv;
    const dim3 grid((unsigned)((int64_t)n_tokens * (heads / group))), block(width >= 2048 ? 256 : 128);
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchNorm, gated_group_norm_kernel<bf16>, grid, block, 0, stream, o, gate, gate_stride, weight, (bf16*)out, heads,
                   dv, group, gate_act, eps);
    else
        cpm_launch(kLaunchNorm, gated_group_norm_kernel<float>, grid, block, 0, stream, o, gate, gate_stride, weight, (float*)out,
                   heads, dv, group, gate_act, eps);
    return launch_status();
}

// In place on the first ``cols`` floats of every row (``stride`` floats apart): x <- x * sigmoid(x).
__global__ void silu_columns_kernel(float* __restrict__ x, int64_t stride, int cols, int64_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float* p = x + (i / cols) * stride + i % cols;
    *p = silu_acc(*p);
}

CPM_API int cpm_silu_columns(float* x, int64_t stride, int n_tokens, int cols, cudaStream_t stream) {
    if (n_tokens <= 0 || cols <= 0) return CPM_OK;
    if (stride < cols) return CPM_BAD_ARGUMENT;
    const int64_t n = (int64_t)n_tokens * cols;
    cpm_launch(kLaunchOther, silu_columns_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, stride, cols, n);
    return launch_status();
}

// out = (rms(a) * wa + rms(b) * wb) / 2 over the model width: the join of two mixers that ran side by side.
template <typename T>
__global__ void dual_rmsnorm_mean_kernel(const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ wa,
                                         const float* __restrict__ wb, T* __restrict__ out, int W, float eps) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    float sa = 0.f, sb = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float x = to_f32(a[t * W + c]), y = to_f32(b[t * W + c]);
        sa = fmaf(x, x, sa);
        sb = fmaf(y, y, sb);
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float fa = rsqrtf(sa / (float)W + eps), fb = rsqrtf(sb / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x)
        out[t * W + c] = from_f32<T>(0.5f * (to_f32(a[t * W + c]) * fa * wa[c] + to_f32(b[t * W + c]) * fb * wb[c]));
}

CPM_API int cpm_dual_rmsnorm_mean(const void* a, const void* b, const float* wa, const float* wb, void* out, int n_tokens, int W,
                                  float eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (W < 1) return CPM_BAD_ARGUMENT;
    const dim3 block(W >= 1024 ? 256 : 128);
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchNorm, dual_rmsnorm_mean_kernel<bf16>, dim3(n_tokens), block, 0, stream, (const bf16*)a, (const bf16*)b, wa, wb,
                   (bf16*)out, W, eps);
    else
        cpm_launch(kLaunchNorm, dual_rmsnorm_mean_kernel<float>, dim3(n_tokens), block, 0, stream, (const float*)a, (const float*)b, wa,
                   wb, (float*)out, W, eps);
    return launch_status();
}
