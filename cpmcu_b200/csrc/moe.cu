// Routed experts: choice of experts per token, and the experts' products over the tokens that chose them.
//
// Routing (fp32): scores s = softmax(z) over all experts; choice scores c = s + correction; experts form
// ``n_groups`` equal groups of neighbours, a group's score is its largest choice score, and only experts of the
// ``keep`` best groups can be chosen (the others count as minus infinity); the ``top`` largest choice scores are
// chosen, and their weights are the plain scores s, not renormalised.  Ties go to the lower index.
// A second rule (``top_first`` 1): the choice scores are the logits plus a bias, the ``top`` largest are chosen, and
// their weights are the softmax over the chosen logits only.  A third (``top_first`` 2): the scores are the sigmoids of
// the logits, the ``top`` largest are chosen, and their weights are those scores, not renormalised.
//
// Products: the (token, choice) pairs are grouped by expert (counts, offsets, a list of pairs in expert order),
// and tiles of 32 pairs of one expert times 64 output features run as blocks of one launch, whose grid is an upper
// bound on the tile count (blocks beyond the last tile leave at once), so nothing is read back on the host:
//   gated (mode 1):  H[r] = silu(x[token(r)] Wg_e^T) * (x[token(r)] Wu_e^T)     r: place in expert order
//   up (mode 2):     H[r] = relu(s[pair(r)] * (x[token(r)] Wu_e^T))^2           s: a number per pair (null: 1), which is
//                    the expert of the input times s, since the product is linear in its input
//   down (mode 0):   Y[pair(r)] = H[r] Wd_e^T
// and a last kernel adds up a token's pairs with their weights and the shared expert's output times its gate.
// Accumulation is fp32: on the CUDA cores for 32-bit storage (and where K is no multiple of 8), on the tensor cores for bf16.
#include "common.cuh"

constexpr int kRouteMaxPerLane = 16;      // experts <= 512

__device__ __forceinline__ ArgMax warp_argmax(ArgMax a) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
        a = better(a, b);
    }
    return a;
}

// One warp per token.  logits rows of ``ld`` floats: the first E are the router's, column ``gate_col`` (if >= 0) is the
// shared expert's raw gate.
__global__ void moe_route_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ correction,
                                 int* __restrict__ chosen, float* __restrict__ weights, float* __restrict__ shared_gate,
                                 int gate_col, int n_tokens, int E, int top, int n_groups, int keep,
                                 const float* __restrict__ bias, int top_first) {
    extern __shared__ float route_smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= n_tokens) return;
    float* s = route_smem + (size_t)warp * (2 * E + n_groups);      // scores
    float* c = s + E;                                                 // choice scores
    float* gs = c + E;                                                // group scores
    const float* z = logits + (int64_t)t * ld;
    if (top_first == 2) {
        // scores: sigmoid of the logits; the ``top`` largest are chosen and their scores are the weights as they are
        for (int e = lane; e < E; e += 32) c[e] = 1.0f / (1.0f + expf(-(z[e] + (bias ? bias[e] : 0.f))));
        __syncwarp();
        for (int r = 0; r < top; ++r) {
            ArgMax a{-INFINITY, 0x7fffffff};
            for (int e = lane; e < E; e += 32) {
                const float v = c[e];
                if (!isnan(v)) a = better(a, ArgMax{v, e});
            }
            a = warp_argmax(a);
            const int e = a.i < E ? a.i : 0;
            if (lane == 0) {
                chosen[(int64_t)t * top + r] = e;
                weights[(int64_t)t * top + r] = a.v;
                c[e] = NAN;                               // taken
            }
            __syncwarp();
        }
        if (gate_col >= 0 && lane == 0) shared_gate[t] = 1.0f / (1.0f + expf(-z[gate_col]));
        return;
    }
    if (top_first) {
        // choice scores: logits + bias; weights: softmax over the chosen scores (the largest is the first chosen)
        for (int e = lane; e < E; e += 32) c[e] = z[e] + (bias ? bias[e] : 0.f);
        __syncwarp();
        float first = 0.f, sum = 0.f;
        for (int r = 0; r < top; ++r) {
            ArgMax a{-INFINITY, 0x7fffffff};
            for (int e = lane; e < E; e += 32) {
                const float v = c[e];
                if (!isnan(v)) a = better(a, ArgMax{v, e});
            }
            a = warp_argmax(a);
            const int e = a.i < E ? a.i : 0;
            if (r == 0) first = a.v;
            const float ex = expf(a.v - first);
            sum += ex;
            if (lane == 0) {
                chosen[(int64_t)t * top + r] = e;
                weights[(int64_t)t * top + r] = ex;
                c[e] = NAN;                               // taken
            }
            __syncwarp();
        }
        if (lane == 0)
            for (int r = 0; r < top; ++r) weights[(int64_t)t * top + r] /= sum;
        if (gate_col >= 0 && lane == 0) shared_gate[t] = 1.0f / (1.0f + expf(-z[gate_col]));
        return;
    }
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float ex = expf(z[e] - m);
        s[e] = ex;
        sum += ex;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) {
        const float v = s[e] * inv;
        s[e] = v;
        c[e] = v + correction[e];
    }
    __syncwarp();
    const int per = E / n_groups;
    if (n_groups > 1 && keep < n_groups) {
        for (int g = lane; g < n_groups; g += 32) {
            float best = -INFINITY;
            for (int i = 0; i < per; ++i) best = fmaxf(best, c[g * per + i]);
            gs[g] = best;
        }
        __syncwarp();
        // the groups that are not kept: all but the ``keep`` best; a kept group is marked by a score of +inf
        for (int r = 0; r < keep; ++r) {
            ArgMax a{-INFINITY, 0x7fffffff};
            for (int g = lane; g < n_groups; g += 32) {
                const float v = gs[g];
                if (v != INFINITY) a = better(a, ArgMax{v, g});
            }
            a = warp_argmax(a);
            if (lane == 0 && a.i < n_groups) gs[a.i] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != INFINITY) c[e] = -INFINITY;
        __syncwarp();
    }
    for (int r = 0; r < top; ++r) {
        ArgMax a{-INFINITY, 0x7fffffff};
        for (int e = lane; e < E; e += 32) {
            const float v = c[e];
            if (!isnan(v)) a = better(a, ArgMax{v, e});
        }
        a = warp_argmax(a);
        const int e = a.i < E ? a.i : 0;
        if (lane == 0) {
            chosen[(int64_t)t * top + r] = e;
            weights[(int64_t)t * top + r] = s[e];
            c[e] = NAN;                                   // taken
        }
        __syncwarp();
    }
    if (gate_col >= 0 && lane == 0) shared_gate[t] = 1.0f / (1.0f + expf(-z[gate_col]));
}

// One block: pairs per expert, offsets, and the pairs listed in expert order.
__global__ void moe_group_kernel(const int* __restrict__ chosen, int n_pairs, int E, int* __restrict__ offsets /* [E+1] */,
                                 int* __restrict__ order /* [pairs] */) {
    extern __shared__ int group_smem[];      // counts [E], cursor [E]
    int* counts = group_smem;
    int* cursor = counts + E;
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&counts[chosen[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = at;
            cursor[e] = at;
            at += counts[e];
        }
        offsets[E] = at;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) order[atomicAdd(&cursor[chosen[i]], 1)] = i;
}

constexpr int kTileM = 32, kTileN = 64, kTileK = 32;

// C[row_out(r)][n] = sum_k A[row_in(r)][k] * B_e[n][k] for the places r of expert e, tile by tile.
// GATED: A rows are tokens (pair / top), two weight stacks (gate, up) and the result is silu(gate) * up, written at
// row r.  Otherwise A rows are the places r themselves and the result goes to row pair(r).
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_tile_kernel(const T* __restrict__ A, const T* __restrict__ B0, const T* __restrict__ B1, T* __restrict__ C,
                const int* __restrict__ offsets, const int* __restrict__ order, int E, int top, int N, int K,
                const float* __restrict__ in_scale) {
    constexpr bool GATED = MODE == 1, BY_TOKEN = MODE != 0;
    __shared__ float As[kTileM][kTileK + 1], Bs0[kTileN][kTileK + 1], Bs1[GATED ? kTileN : 1][kTileK + 1];
    __shared__ int s_tile[3];
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        int tile = blockIdx.x, e = 0, found = -1, first = 0;
        for (; e < E; ++e) {
            const int n = offsets[e + 1] - offsets[e];
            const int tiles = (n + kTileM - 1) / kTileM;
            if (tile < tiles) { found = e; first = offsets[e] + tile * kTileM; break; }
            tile -= tiles;
        }
        s_tile[0] = found;
        s_tile[1] = first;
        s_tile[2] = found >= 0 ? min(kTileM, offsets[found + 1] - first) : 0;
    }
    __syncthreads();
    const int e = s_tile[0], r0 = s_tile[1], rows = s_tile[2];
    if (e < 0) return;
    const int n0 = blockIdx.y * kTileN;
    const T* W0 = B0 + (int64_t)e * N * K;
    const T* W1 = GATED ? B1 + (int64_t)e * N * K : nullptr;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // 4 columns, 2 rows a thread
    float acc0[2][4] = {}, acc1[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += kTileK) {
        for (int i = threadIdx.x; i < kTileM * kTileK; i += 256) {
            const int r = i / kTileK, kk = i % kTileK;
            float v = 0.f;
            if (r < rows && k0 + kk < K) {
                const int64_t src = BY_TOKEN ? (int64_t)(order[r0 + r] / top) : (int64_t)(r0 + r);
                v = to_f32(A[src * K + k0 + kk]);
            }
            As[r][kk] = v;
        }
        for (int i = threadIdx.x; i < kTileN * kTileK; i += 256) {
            const int n = i / kTileK, kk = i % kTileK;
            const bool ok = n0 + n < N && k0 + kk < K;
            Bs0[n][kk] = ok ? to_f32(W0[(int64_t)(n0 + n) * K + k0 + kk]) : 0.f;
            if (GATED) Bs1[n][kk] = ok ? to_f32(W1[(int64_t)(n0 + n) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < kTileK; ++kk) {
            const float a0 = As[ty * 2][kk], a1 = As[ty * 2 + 1][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = Bs0[tx * 4 + j][kk];
                acc0[0][j] = fmaf(a0, b, acc0[0][j]);
                acc0[1][j] = fmaf(a1, b, acc0[1][j]);
                if (GATED) {
                    const float b1 = Bs1[tx * 4 + j][kk];
                    acc1[0][j] = fmaf(a0, b1, acc1[0][j]);
                    acc1[1][j] = fmaf(a1, b1, acc1[1][j]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = ty * 2 + i;
        if (r >= rows) continue;
        const int64_t dst = BY_TOKEN ? (int64_t)(r0 + r) : (int64_t)order[r0 + r];
        const float sc = (MODE == 2 && in_scale != nullptr) ? in_scale[order[r0 + r]] : 1.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc0[i][j];
            if (GATED) v = v / (1.0f + expf(-v)) * acc1[i][j];
            if (MODE == 2) { v = fmaxf(v * sc, 0.f); v *= v; }
            C[dst * N + n] = from_f32<T>(v);
        }
    }
}


// The same products for bf16 on the tensor cores (mma.sync m16n8k16, fp32 accumulation): tiles of 128 places of one
// expert times 64 output features, eight warps of 32 x 32 each, K in steps of 32 through two shared-memory stages
// filled by asynchronous 16-byte copies (rows padded to 40 elements, so that ldmatrix reads 8 rows from 8 different
// bank groups); fragments come by ldmatrix.x4.  K must be a multiple of 8 (16-byte copies).
constexpr int kMmaM = 128, kMmaN = 64, kMmaK = 32, kMmaPad = 40;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const bf16* smem_row) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// 16 bytes from global to shared memory, or 16 zero bytes when ``valid`` is false (the source is then not read)
__device__ __forceinline__ void cp_async_16(bf16* smem_dst, const bf16* gmem_src, bool valid) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(256)
moe_tile_mma_kernel(const bf16* __restrict__ A, const bf16* __restrict__ B0, const bf16* __restrict__ B1, bf16* __restrict__ C,
                    const int* __restrict__ offsets, const int* __restrict__ order, int E, int top, int N, int K,
                    const float* __restrict__ in_scale) {
    constexpr bool GATED = MODE == 1, BY_TOKEN = MODE != 0;
    __shared__ __align__(16) bf16 As[2][kMmaM][kMmaPad], Bs0[2][kMmaN][kMmaPad], Bs1[GATED ? 2 : 1][GATED ? kMmaN : 1][kMmaPad];
    __shared__ int s_tile[3];
    __shared__ int s_rows[kMmaM];
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        int tile = blockIdx.x, e = 0, found = -1, first = 0;
        for (; e < E; ++e) {
            const int n = offsets[e + 1] - offsets[e];
            const int tiles = (n + kMmaM - 1) / kMmaM;
            if (tile < tiles) { found = e; first = offsets[e] + tile * kMmaM; break; }
            tile -= tiles;
        }
        s_tile[0] = found;
        s_tile[1] = first;
        s_tile[2] = found >= 0 ? min(kMmaM, offsets[found + 1] - first) : 0;
    }
    __syncthreads();
    const int e = s_tile[0], r0 = s_tile[1], rows = s_tile[2];
    if (e < 0) return;
    if (threadIdx.x < kMmaM) s_rows[threadIdx.x] = threadIdx.x < rows ? order[r0 + threadIdx.x] : -1;      // the pair at this place
    __syncthreads();
    const int n0 = blockIdx.y * kMmaN;
    const bf16* W0 = B0 + (int64_t)e * N * K;
    const bf16* W1 = GATED ? B1 + (int64_t)e * N * K : B0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, j = lane & 3;
    const int wm = warp >> 1, wn = warp & 1;                   // the warp's 32 rows and 32 columns of the tile
    // a thread's source rows: two pieces of the A tile (rows p >> 2 for p = tid, tid + 256), one of each B tile
    const bf16* a_src[2];
    bool a_ok[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = (threadIdx.x + 256 * i) >> 2;
        const int pair = s_rows[r];
        a_ok[i] = pair >= 0;
        a_src[i] = A + (int64_t)(a_ok[i] ? (BY_TOKEN ? pair / top : r0 + r) : 0) * K;
    }
    const int b_row = threadIdx.x >> 2, piece = 8 * (threadIdx.x & 3);
    const bool b_ok = n0 + b_row < N;
    const bf16* b_src0 = W0 + (int64_t)(b_ok ? n0 + b_row : 0) * K;
    const bf16* b_src1 = W1 + (int64_t)(b_ok ? n0 + b_row : 0) * K;
    auto issue = [&](int k0, int st) {
        const bool k_ok = k0 + piece < K;
#pragma unroll
        for (int i = 0; i < 2; ++i)
            cp_async_16(&As[st][(threadIdx.x + 256 * i) >> 2][piece], a_src[i] + (k_ok ? k0 + piece : 0), a_ok[i] && k_ok);
        cp_async_16(&Bs0[st][b_row][piece], b_src0 + (k_ok ? k0 + piece : 0), b_ok && k_ok);
        if (GATED) cp_async_16(&Bs1[st][b_row][piece], b_src1 + (k_ok ? k0 + piece : 0), b_ok && k_ok);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float acc0[2][4][4] = {}, acc1[GATED ? 2 : 1][4][4] = {};
    issue(0, 0);
    int st = 0;
    for (int k0 = 0; k0 < K; k0 += kMmaK, st ^= 1) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                       // this stage has arrived; the other one is free again
        if (k0 + kMmaK < K) issue(k0 + kMmaK, st ^ 1);
#pragma unroll
        for (int ks = 0; ks < kMmaK; ks += 16) {
            uint32_t a[2][4], b[2][4], u[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) ldmatrix_x4(a[mt], &As[st][wm * 32 + mt * 16 + (lane & 15)][ks + 8 * (lane >> 4)]);
#pragma unroll
            for (int np = 0; np < 2; ++np) {                   // two column tiles of 8 per ldmatrix
                const int row = wn * 32 + np * 16 + 8 * (lane >> 4) + (lane & 7), col = ks + 8 * ((lane >> 3) & 1);
                ldmatrix_x4(b[np], &Bs0[st][row][col]);
                if (GATED) ldmatrix_x4(u[np], &Bs1[st][row][col]);
            }
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    mma_bf16_16816(acc0[mt][nt], a[mt], b[nt >> 1][2 * (nt & 1)], b[nt >> 1][2 * (nt & 1) + 1]);
                    if (GATED) mma_bf16_16816(acc1[mt][nt], a[mt], u[nt >> 1][2 * (nt & 1)], u[nt >> 1][2 * (nt & 1) + 1]);
                }
        }
    }
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm * 32 + mt * 16 + g + 8 * half;
            if (r >= rows) continue;
            const int64_t dst = BY_TOKEN ? (int64_t)(r0 + r) : (int64_t)s_rows[r];
            const float sc = (MODE == 2 && in_scale != nullptr) ? in_scale[s_rows[r]] : 1.f;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int n = n0 + wn * 32 + nt * 8 + 2 * j + q;
                    if (n >= N) continue;
                    float v = acc0[mt][nt][2 * half + q];
                    if (GATED) v = v / (1.0f + expf(-v)) * acc1[mt][nt][2 * half + q];
                    if (MODE == 2) { v = fmaxf(v * sc, 0.f); v *= v; }
                    C[dst * N + n] = __float2bfloat16_rn(v);
                }
        }
}

// Few pairs (a decode step): every pair is a matrix-vector product that streams its expert's weights once.  A block
// takes one pair and 32 output features (64 weight rows when gated), a warp four of them at a time: the lanes split K
// in 16-byte pieces and the sums meet by shuffles.  No grouping by expert is needed: H and Y are indexed by pair.
constexpr int kGemvFeatures = 32;

template <int MODE>
__global__ void __launch_bounds__(256)
moe_pair_gemv_kernel(const bf16* __restrict__ A, const bf16* __restrict__ B0, const bf16* __restrict__ B1, bf16* __restrict__ C,
                     const int* __restrict__ chosen, int top, int N, int K, const float* __restrict__ in_scale) {
    constexpr bool GATED = MODE == 1, BY_TOKEN = MODE != 0;
    extern __shared__ float gemv_x[];                          // the pair's input row, fp32
    pdl_launch_dependents();
    const int pair = blockIdx.x, n0 = blockIdx.y * kGemvFeatures;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_wait();
    const int e = chosen[pair];
    const bf16* x = A + (int64_t)(BY_TOKEN ? pair / top : pair) * K;
    const float sc = (MODE == 2 && in_scale != nullptr) ? in_scale[pair] : 1.f;
    for (int i = threadIdx.x; i < K; i += blockDim.x) gemv_x[i] = __bfloat162float(x[i]);
    __syncthreads();
    const bf16* W0 = B0 + (int64_t)e * N * K;
    const bf16* W1 = GATED ? B1 + (int64_t)e * N * K : B0;
    for (int f = warp; f < kGemvFeatures; f += 8) {
        const int n = n0 + f;
        if (n >= N) break;
        const bf16* w0 = W0 + (int64_t)n * K;
        const bf16* w1 = W1 + (int64_t)n * K;
        float s0 = 0.f, s1 = 0.f;
        for (int kk = lane * 8; kk < K; kk += 256) {
            const uint4 r0 = *reinterpret_cast<const uint4*>(w0 + kk);
            const __nv_bfloat162* p0 = reinterpret_cast<const __nv_bfloat162*>(&r0);
            uint4 r1 = make_uint4(0, 0, 0, 0);
            if (GATED) r1 = *reinterpret_cast<const uint4*>(w1 + kk);
            const __nv_bfloat162* p1 = reinterpret_cast<const __nv_bfloat162*>(&r1);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 a = __bfloat1622float2(p0[i]);
                s0 = fmaf(a.x, gemv_x[kk + 2 * i], s0);
                s0 = fmaf(a.y, gemv_x[kk + 2 * i + 1], s0);
                if (GATED) {
                    const float2 b = __bfloat1622float2(p1[i]);
                    s1 = fmaf(b.x, gemv_x[kk + 2 * i], s1);
                    s1 = fmaf(b.y, gemv_x[kk + 2 * i + 1], s1);
                }
            }
        }
        s0 = warp_sum(s0);
        if (GATED) s1 = warp_sum(s1);
        if (MODE == 2) { s0 = fmaxf(s0 * sc, 0.f); s0 *= s0; }
        if (lane == 0) C[(int64_t)pair * N + n] = __float2bfloat16_rn(GATED ? s0 / (1.0f + expf(-s0)) * s1 : s0);
    }
}

// The same two products for few pairs, by pair: gated: C = H [pairs, N] by pair from x [tokens, K]; else C = Y [pairs, N]
// from H [pairs, K] by pair.  bf16, K a multiple of 8.
// mode 1: gated; 2: one stack, relu(in_scale[pair] * product)^2, from x by pair; 0: the down product.
CPM_API int cpm_moe_pair_product(const void* A, const void* B0, const void* B1, void* C, const int* chosen, int n_pairs, int top,
                                 int N, int K, int mode, const float* in_scale, cudaStream_t stream) {
    if (n_pairs <= 0) return CPM_OK;
    if (top < 1 || N < 1 || K < 8 || K % 8 || ((uintptr_t)A & 15) || ((uintptr_t)B0 & 15) || ((uintptr_t)B1 & 15) ||
        (size_t)K * sizeof(float) > 48 * 1024)
        return CPM_BAD_ARGUMENT;
    const dim3 grid(n_pairs, (N + kGemvFeatures - 1) / kGemvFeatures);
    if (grid.y > 65535) return CPM_BAD_ARGUMENT;
    if (mode < 0 || mode > 2) return CPM_BAD_ARGUMENT;
#define CPM_GEMV(M) cpm_launch(kLaunchProduct, moe_pair_gemv_kernel<M>, grid, dim3(256), (size_t)K * sizeof(float), stream,      \
                               (const bf16*)A, (const bf16*)B0, (const bf16*)B1, (bf16*)C, chosen, top, N, K, in_scale)
    if (mode == 1) CPM_GEMV(1); else if (mode == 2) CPM_GEMV(2); else CPM_GEMV(0);
#undef CPM_GEMV
    return launch_status();
}

// out[t] = sum_k weights[t][k] * Y[t * top + k] + gate[t] * shared[t]   (weights null: all 1)
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ Y, const float* __restrict__ weights, const T* __restrict__ shared,
                                   const float* __restrict__ gate, T* __restrict__ out, int top, int W) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float v = 0.f;
        for (int k = 0; k < top; ++k) v = fmaf(weights ? weights[t * top + k] : 1.f, to_f32(Y[(t * top + k) * W + c]), v);
        if (shared) v = fmaf(gate ? gate[t] : 1.f, to_f32(shared[t * W + c]), v);
        out[t * W + c] = from_f32<T>(v);
    }
}

static int g_moe_tensor_cores = 1;
// 0: the bf16 products stay on the CUDA cores too (for comparisons and tests)
CPM_API int cpm_set_moe_tensor_cores(int on) {
    g_moe_tensor_cores = on;
    return CPM_OK;
}

CPM_API int cpm_moe_route(const float* logits, int ld, const float* correction, int* chosen, float* weights, float* shared_gate,
                          int gate_col, int n_tokens, int E, int top, int n_groups, int keep, const float* bias, int top_first,
                          cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (top_first < 0 || top_first > 2 || (!top_first && !correction)) return CPM_BAD_ARGUMENT;
    if (E < 1 || E > 32 * kRouteMaxPerLane || top < 1 || top > E || n_groups < 1 || E % n_groups || keep < 1 || keep > n_groups ||
        top > keep * (E / n_groups))
        return CPM_BAD_ARGUMENT;
    const int warps = 4;
    const size_t smem = (size_t)warps * (2 * E + n_groups) * sizeof(float);
    cpm_launch(kLaunchOther, moe_route_kernel, dim3((n_tokens + warps - 1) / warps), dim3(warps * 32), smem, stream, logits, ld,
               correction, chosen, weights, shared_gate, gate_col, n_tokens, E, top, n_groups, keep, bias, top_first);
    return launch_status();
}

CPM_API int cpm_moe_group(const int* chosen, int n_pairs, int E, int* offsets, int* order, cudaStream_t stream) {
    if (n_pairs <= 0) return CPM_OK;
    if (E < 1 || E > 4096) return CPM_BAD_ARGUMENT;
    cpm_launch(kLaunchOther, moe_group_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), stream, chosen, n_pairs, E, offsets,
               order);
    return launch_status();
}

// mode 1: A = x [tokens, K], B0 = gate stack [E, N, K], B1 = up stack, C = H [pairs, N] in expert order.
// mode 2: A = x, B0 = up stack, C = H = relu(in_scale[pair] * product)^2 in expert order (in_scale null: 1).
// mode 0: A = H [pairs, K] in expert order, B0 = down stack [E, N, K], C = Y [pairs, N] by pair.
CPM_API int cpm_moe_expert_product(const void* A, const void* B0, const void* B1, void* C, const int* offsets, const int* order,
                                   int n_pairs, int E, int top, int N, int K, int mode, const float* in_scale, int dtype,
                                   cudaStream_t stream) {
    if (n_pairs <= 0) return CPM_OK;
    if (E < 1 || top < 1 || N < 1 || K < 1 || mode < 0 || mode > 2) return CPM_BAD_ARGUMENT;
    if (dtype == CPM_BF16 && K % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)B0 & 15) == 0 && ((uintptr_t)B1 & 15) == 0 &&
        g_moe_tensor_cores) {
        const dim3 mgrid((n_pairs + kMmaM - 1) / kMmaM + E, (N + kMmaN - 1) / kMmaN);
        if (mgrid.y > 65535) return CPM_BAD_ARGUMENT;
#define CPM_MMA(M) cpm_launch(kLaunchProduct, moe_tile_mma_kernel<M>, mgrid, dim3(256), 0, stream, (const bf16*)A, (const bf16*)B0, \
                              (const bf16*)B1, (bf16*)C, offsets, order, E, top, N, K, in_scale)
        if (mode == 1) CPM_MMA(1); else if (mode == 2) CPM_MMA(2); else CPM_MMA(0);
#undef CPM_MMA
        return launch_status();
    }
    const dim3 grid((n_pairs + kTileM - 1) / kTileM + E, (N + kTileN - 1) / kTileN);
    if (grid.y > 65535) return CPM_BAD_ARGUMENT;
#define CPM_MOE(TT, G) cpm_launch(kLaunchProduct, moe_tile_kernel<TT, G>, grid, dim3(256), 0, stream, (const TT*)A, (const TT*)B0, \
                                  (const TT*)B1, (TT*)C, offsets, order, E, top, N, K, in_scale)
    if (dtype == CPM_BF16) { if (mode == 1) CPM_MOE(bf16, 1); else if (mode == 2) CPM_MOE(bf16, 2); else CPM_MOE(bf16, 0); }
    else { if (mode == 1) CPM_MOE(float, 1); else if (mode == 2) CPM_MOE(float, 2); else CPM_MOE(float, 0); }
#undef CPM_MOE
    return launch_status();
}

CPM_API int cpm_moe_combine(const void* Y, const float* weights, const void* shared, const float* gate, void* out, int n_tokens,
                            int top, int W, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    const dim3 block(W >= 1024 ? 256 : 128);
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchNorm, moe_combine_kernel<bf16>, dim3(n_tokens), block, 0, stream, (const bf16*)Y, weights, (const bf16*)shared,
                   gate, (bf16*)out, top, W);
    else
        cpm_launch(kLaunchNorm, moe_combine_kernel<float>, dim3(n_tokens), block, 0, stream, (const float*)Y, weights,
                   (const float*)shared, gate, (float*)out, top, W);
    return launch_status();
}
