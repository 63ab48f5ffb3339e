// Routed feed-forward (mixture of experts) over a step's tokens.
//
//   route:    per token the `top` largest router logits (ties: the lower index), weights = softmax over those alone;
//             `router` also makes the logits itself (fp32 weights, fp32 sums), a warp a token;
//   group:    the (token, choice) pairs ordered by expert: per-expert counts and offsets, the pair behind every
//             slot, the slot of every pair, and the list of (expert, first slot) row tiles the products walk;
//   gate_up:  act[slot] = f(W_gu[e] x[token]) for the slots of expert e, the rows of gate and up interleaved so that a
//             thread holds a (gate, up) pair: g = min(gate, limit), u = clamp(up, -limit, limit),
//             f = g sigmoid(alpha g) (u + 1);
//   down:     y[slot] = W_down[e] act[slot]  (fp32);
//   combine:  out[token] = sum over its choices, in order, of weight * y[slot]  (stored, or added to what is there).
// Both products come in two forms: tiles of 32 slots x 64 outputs through shared memory (any sizes, any step), and,
// for steps of few tokens, a streaming form in which a block keeps its (at most 16) rows in shared memory and every
// warp streams whole weight rows past them in 16-byte pieces, so an expert's weights are read once at the rate of
// the memory and only the rows that exist are multiplied (fp32 multiply-adds; for bfloat16 with K a multiple of 64 the
// same on mma.sync, weights through per-warp cp.async stages).
//
// Nothing is read back by the host: the products' grids are sized for the most row tiles the step can have and blocks
// beyond the tile list leave at once, so a decode step can be captured into a CUDA graph.  Every output row is a sum
// over k in ascending order and independent of its neighbours in the tile, so a token's result depends neither on
// the other tokens of the step nor on where the grouping put it.
#include "common.cuh"

EMBER_DEFINE_LAST_ERROR

namespace ember {

constexpr int MOE_MAX_EXPERTS = 256;
constexpr int MOE_BM = 32, MOE_BN = 64, MOE_BK = 16;

// How the chosen experts are found and weighed.  sigmoid 0: by the logits, weights = softmax over the chosen logits
// alone.  sigmoid 1: scores s = sigmoid(logit); the choice is by s + correction[e] (correction may be null), the
// weights are the chosen experts' s times scale, divided by their sum first if renormalize.
// sigmoid 2: scores s = softmax(logits) over all experts, otherwise as sigmoid 1.  groups > 0 (at most 32): the experts
// form `groups` equal groups of neighbours, a group's score is its largest s + correction, and only experts of the
// `keep` best groups (ties: the lower index) can be chosen.
struct RouteRule {
    int sigmoid; const float* correction; float scale; int renormalize; int groups; int keep;
};

// One warp a token.  A lane holds experts lane, lane + 32, ... in z.
__device__ __forceinline__ void choose_experts(float (&z)[MOE_MAX_EXPERTS / 32], int E, int top, int* __restrict__ sel,
                                               float* __restrict__ wgt, int t, int lane, const RouteRule& rule);

__global__ void moe_route_kernel(const float* __restrict__ logits, int E, int top, int* __restrict__ sel,
                                 float* __restrict__ wgt, int T, RouteRule rule) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (t >= T) return;
    float z[MOE_MAX_EXPERTS / 32];
#pragma unroll
    for (int i = 0; i < MOE_MAX_EXPERTS / 32; i++) {
        const int e = lane + 32 * i;
        z[i] = e < E ? logits[(size_t)t * E + e] : -INFINITY;
    }
    choose_experts(z, E, top, sel, wgt, t, lane, rule);
}

// The router's product and the choice in one: logits[e] = sum_k x[t, k] w[e, k] with fp32 weights and sums.  A block
// a token: its warps share the experts (four elements a lane and load), the first warp then chooses.
template <typename T>
__global__ void __launch_bounds__(512) moe_router_kernel(const T* __restrict__ x, const float* __restrict__ w, int K, int E, int top,
                                                         int* __restrict__ sel, float* __restrict__ wgt, float* __restrict__ logits,
                                                         RouteRule rule) {
    __shared__ float zs[MOE_MAX_EXPERTS];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const T* row = x + (size_t)t * K;
    const bool vec = (K & 3) == 0;
    for (int e = warp; e < E; e += nw) {
        const float* we = w + (size_t)e * K;
        float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
        if (vec) {
            for (int k = 4 * lane; k < K; k += 128) {
                const float4 wv = *reinterpret_cast<const float4*>(we + k);
                s0 = fmaf(to_float(row[k]), wv.x, s0); s1 = fmaf(to_float(row[k + 1]), wv.y, s1);
                s2 = fmaf(to_float(row[k + 2]), wv.z, s2); s3 = fmaf(to_float(row[k + 3]), wv.w, s3);
            }
        } else {
            for (int k = lane; k < K; k += 32) s0 = fmaf(to_float(row[k]), we[k], s0);
        }
        const float s = warp_sum((s0 + s1) + (s2 + s3));
        if (lane == 0) {
            zs[e] = s;
            if (logits) logits[(size_t)t * E + e] = s;
        }
    }
    __syncthreads();
    if (warp != 0) return;
    float z[MOE_MAX_EXPERTS / 32];
#pragma unroll
    for (int i = 0; i < MOE_MAX_EXPERTS / 32; i++) {
        const int e = lane + 32 * i;
        z[i] = e < E ? zs[e] : -INFINITY;
    }
    choose_experts(z, E, top, sel, wgt, t, lane, rule);
}

__device__ __forceinline__ void choose_experts(float (&z)[MOE_MAX_EXPERTS / 32], int E, int top, int* __restrict__ sel,
                                               float* __restrict__ wgt, int t, int lane, const RouteRule& rule) {
    const int ns = (E + 31) >> 5;                           // slots of a lane that hold an expert: the loops below stop there
    float score[MOE_MAX_EXPERTS / 32];                      // sigmoid rule: s of the lane's experts; z becomes what is compared
    if (rule.sigmoid) {
        float zmax = -INFINITY, zsum = 0.0f;
        if (rule.sigmoid == 2) {                            // softmax over all experts
#pragma unroll
            for (int i = 0; i < MOE_MAX_EXPERTS / 32; i++) {
                if (i >= ns) break;
                if (lane + 32 * i < E) zmax = fmaxf(zmax, z[i]);
            }
            zmax = warp_max(zmax);
#pragma unroll
            for (int i = 0; i < MOE_MAX_EXPERTS / 32; i++) {
                if (i >= ns) break;
                if (lane + 32 * i < E) zsum += expf(z[i] - zmax);
            }
            zsum = warp_sum(zsum);
        }
#pragma unroll
        for (int i = 0; i < MOE_MAX_EXPERTS / 32; i++) {
            if (i >= ns) break;
            const int e = lane + 32 * i;
            if (rule.sigmoid == 2) score[i] = e < E ? expf(z[i] - zmax) / zsum : 0.0f;
            else score[i] = e < E ? 1.0f / (1.0f + expf(-z[i])) : 0.0f;
            if (e < E) z[i] = score[i] + (rule.correction ? rule.correction[e] : 0.0f);
        }
        if (rule.groups > 0) {                              // lane g keeps group g's best; then the best groups, one by one
            const int per = E / rule.groups;
            int grp[MOE_MAX_EXPERTS / 32];                  // the group of each of the lane's experts (one division each)
#pragma unroll
            for (int i = 0; i < MOE_MAX_EXPERTS / 32; i++) {
                if (i >= ns) break;
                grp[i] = lane + 32 * i < E ? (lane + 32 * i) / per : -1;
            }
            float gbest = -INFINITY;
            for (int g = 0; g < rule.groups; g++) {
                float b = -INFINITY;
#pragma unroll
                for (int i = 0; i < MOE_MAX_EXPERTS / 32; i++) {
                    if (i >= ns) break;
                    if (grp[i] == g) b = fmaxf(b, z[i]);
                }
                b = warp_max(b);
                if (lane == g) gbest = b;
            }
            unsigned kept = 0u;
            for (int k = 0; k < rule.keep; k++) {
                float b = (lane < rule.groups && !((kept >> lane) & 1u)) ? gbest : -INFINITY;
                int at = (lane < rule.groups && !((kept >> lane) & 1u)) ? lane : 0x7fffffff;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ob = __shfl_xor_sync(0xffffffffu, b, o);
                    const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                    if (oa != 0x7fffffff && (at == 0x7fffffff || ob > b || (ob == b && oa < at))) { b = ob; at = oa; }
                }
                if (at != 0x7fffffff) kept |= 1u << at;
            }
#pragma unroll
            for (int i = 0; i < MOE_MAX_EXPERTS / 32; i++) {
                if (i >= ns) break;
                if (grp[i] >= 0 && !((kept >> grp[i]) & 1u)) z[i] = -INFINITY;
            }
        }
    }
    float first = 0.0f, sum = 0.0f, mine = 0.0f;            // lane k keeps the k-th choice's weight (top <= 32)
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int at = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < MOE_MAX_EXPERTS / 32; i++) {
            if (i >= ns) break;
            const int e = lane + 32 * i;
            if (e < E && z[i] != -INFINITY && (z[i] > best || (z[i] == best && e < at))) { best = z[i]; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
        }
        if (at == 0x7fffffff) { at = 0; best = first; }     // (no finite logit left: only with NaNs in the row)
        if (k == 0) first = best;
        float w;
        if (rule.sigmoid) {                                 // the chosen expert's own score, from the lane that holds it
            float sc = 0.0f;
#pragma unroll
            for (int i = 0; i < MOE_MAX_EXPERTS / 32; i++) {
                if (i >= ns) break;
                if (i == (at >> 5)) sc = score[i];
            }
            w = __shfl_sync(0xffffffffu, sc, at & 31);
        } else {
            w = expf(best - first);
        }
        sum += w;
        if (lane == k) mine = w;
        if (lane == 0) sel[(size_t)t * top + k] = at;
        if (lane == (at & 31)) {
#pragma unroll
            for (int i = 0; i < MOE_MAX_EXPERTS / 32; i++) {
                if (i >= ns) break;
                if (i == (at >> 5)) z[i] = -INFINITY;
            }
        }
    }
    if (lane < top) {
        if (rule.sigmoid) wgt[(size_t)t * top + lane] = (rule.renormalize ? mine / sum : mine) * rule.scale;
        else wgt[(size_t)t * top + lane] = mine / sum;
    }
}

// One block.  counts / offsets by expert, slots by atomic cursors, then the row tiles.
// meta: [0] number of row tiles; offsets[E + 1]; tile_expert[max_tiles]; tile_row0[max_tiles].
__global__ void __launch_bounds__(1024) moe_group_kernel(const int* __restrict__ sel, int n_pairs, int E, int* __restrict__ offsets,
                                                         int* __restrict__ pair_of_slot, int* __restrict__ slot_of_pair,
                                                         int* __restrict__ n_tiles, int* __restrict__ tile_expert,
                                                         int* __restrict__ tile_row0, int max_tiles, int tile_rows, int tiled) {
    __shared__ int count[MOE_MAX_EXPERTS], start[MOE_MAX_EXPERTS + 1], cursor[MOE_MAX_EXPERTS], tstart[MOE_MAX_EXPERTS + 1];
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&count[sel[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tt = 0;
        for (int e = 0; e < E; e++) {
            start[e] = at; tstart[e] = tt;
            at += count[e];
            if (e < tiled) tt += (count[e] + tile_rows - 1) / tile_rows;     // experts from `tiled` on have no weights: slots, no tiles
        }
        start[E] = at; tstart[E] = tt;
        *n_tiles = tt < max_tiles ? tt : max_tiles;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) {
        offsets[e] = start[e];
        if (e < E) cursor[e] = start[e];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int slot = atomicAdd(&cursor[sel[i]], 1);
        pair_of_slot[slot] = i;
        slot_of_pair[i] = slot;
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int n = tstart[e + 1] - tstart[e];
        for (int j = 0; j < n; j++)
            if (tstart[e] + j < max_tiles) {
                tile_expert[tstart[e] + j] = e;
                tile_row0[tstart[e] + j] = start[e] + j * tile_rows;
            }
    }
}

struct MoeGemmArgs {
    const void* x; int ld_x;             // rows of the A operand: tokens (gathered through the pairs) or slots
    const void* w; long long w_expert;   // [E][N][K]
    void* out; int ld_o;
    const int* offsets; const int* pair_of_slot; const int* n_tiles; const int* tile_expert; const int* tile_row0;
    int top;                             // > 0: row of x = pair / top (a token); 0: row of x = slot
    int N, K;
    float limit, alpha, up_offset;      // (limit may be +inf: no clamps)
    int act;                            // ungated product: 0 stores the sums, 1 stores relu(sum)^2
};

__device__ __forceinline__ float plain_act(float v, int act) { return act == 1 ? (v > 0.0f ? v * v : 0.0f) : v; }

// GATED: N counts interleaved (gate, up) rows, the output has N / 2 columns.
template <typename TX, typename TW, typename TO, bool GATED>
__global__ void __launch_bounds__(256) moe_gemm_kernel(MoeGemmArgs p) {
    __shared__ float As[MOE_BK][MOE_BM + 1];
    __shared__ float Bs[MOE_BK][MOE_BN + 1];
    __shared__ int src[MOE_BM];
    pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.x >= *p.n_tiles) return;
    const int e = p.tile_expert[blockIdx.x], row0 = p.tile_row0[blockIdx.x], n0 = blockIdx.y * MOE_BN;
    const int rows = min(MOE_BM, p.offsets[e + 1] - row0);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    if (threadIdx.x < MOE_BM) {
        int r = -1;
        if ((int)threadIdx.x < rows) r = p.top > 0 ? p.pair_of_slot[row0 + threadIdx.x] / p.top : row0 + threadIdx.x;
        src[threadIdx.x] = r;
    }
    __syncthreads();
    const TW* w = (const TW*)p.w + (size_t)e * p.w_expert;
    const TX* x = (const TX*)p.x;
    float acc[2][4] = {};
    for (int k0 = 0; k0 < p.K; k0 += MOE_BK) {
        for (int idx = threadIdx.x; idx < MOE_BM * MOE_BK; idx += 256) {
            const int r = idx / MOE_BK, k = idx - r * MOE_BK;
            As[k][r] = (src[r] >= 0 && k0 + k < p.K) ? to_float(x[(size_t)src[r] * p.ld_x + k0 + k]) : 0.0f;
        }
        for (int idx = threadIdx.x; idx < MOE_BN * MOE_BK; idx += 256) {
            const int r = idx / MOE_BK, k = idx - r * MOE_BK;
            const int n = n0 + r;
            Bs[k][r] = (n < p.N && k0 + k < p.K) ? to_float(w[(size_t)n * p.K + k0 + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < MOE_BK; k++) {
            float a[2], b[4];
#pragma unroll
            for (int i = 0; i < 2; i++) a[i] = As[k][ty * 2 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 2; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = ty * 2 + i;
        if (r >= rows) continue;
        TO* o = (TO*)p.out + (size_t)(row0 + r) * p.ld_o;
        if (GATED) {
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int n = n0 + tx * 4 + j;
                if (n >= p.N) continue;
                const float g = fminf(acc[i][j], p.limit);
                const float u = fminf(fmaxf(acc[i][j + 1], -p.limit), p.limit);
                o[n >> 1] = from_float<TO>(g / (1.0f + expf(-p.alpha * g)) * (u + p.up_offset));
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int n = n0 + tx * 4 + j;
                if (n < p.N) o[n] = from_float<TO>(plain_act(acc[i][j], p.act));
            }
        }
    }
}

// ------------------------------------------------------------------------- the streaming form (few rows a tile)
constexpr int MS_ROWS = 16, MS_WARPS = 8, MS_PAIRS = 32;      // rows a tile, warps a block, column pairs a block

template <typename T>
struct Piece;                                                 // 16 bytes of a row as floats
template <>
struct Piece<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    }
};
template <>
struct Piece<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
        f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
        f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
        f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
        f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
    }
};

template <typename T, typename TO, bool GATED, int R>
__device__ __forceinline__ void moe_stream_rows(const MoeGemmArgs& p, const uint4* xs, const T* w, int row0, int rows, int pair0) {
    constexpr int PN = Piece<T>::N;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int k16 = p.K / PN;                                  // 16-byte pieces a row
    const int n_pairs = (p.N + 1) / 2;
    for (int pr = pair0 + warp; pr < min(pair0 + MS_PAIRS, n_pairs); pr += MS_WARPS) {
        const int n0 = 2 * pr;
        const bool two = n0 + 1 < p.N;
        const uint4* w0 = reinterpret_cast<const uint4*>(w + (size_t)n0 * p.K);
        const uint4* w1 = reinterpret_cast<const uint4*>(w + (size_t)(two ? n0 + 1 : n0) * p.K);
        float a0[R], a1[R];
#pragma unroll
        for (int r = 0; r < R; r++) { a0[r] = 0.0f; a1[r] = 0.0f; }
#pragma unroll 2
        for (int k = lane; k < k16; k += 32) {
            float f0[PN], f1[PN];
            Piece<T>::unpack(__ldg(w0 + k), f0);
            Piece<T>::unpack(__ldg(w1 + k), f1);
#pragma unroll
            for (int r = 0; r < R; r++) {
                float xf[PN];
                Piece<T>::unpack(xs[(size_t)r * k16 + k], xf);
#pragma unroll
                for (int i = 0; i < PN; i++) { a0[r] = fmaf(f0[i], xf[i], a0[r]); a1[r] = fmaf(f1[i], xf[i], a1[r]); }
            }
        }
#pragma unroll
        for (int r = 0; r < R; r++) { a0[r] = warp_sum(a0[r]); a1[r] = warp_sum(a1[r]); }
        // lane r writes row r
        float v0 = 0.0f, v1 = 0.0f;
#pragma unroll
        for (int r = 0; r < R; r++)
            if (lane == r) { v0 = a0[r]; v1 = a1[r]; }
        if (lane < rows) {
            TO* o = (TO*)p.out + (size_t)(row0 + lane) * p.ld_o;
            if (GATED) {
                const float g = fminf(v0, p.limit), u = fminf(fmaxf(v1, -p.limit), p.limit);
                o[pr] = from_float<TO>(g / (1.0f + expf(-p.alpha * g)) * (u + p.up_offset));
            } else {
                o[n0] = from_float<TO>(plain_act(v0, p.act));
                if (two) o[n0 + 1] = from_float<TO>(plain_act(v1, p.act));
            }
        }
    }
}

template <typename T, typename TO, bool GATED>
__global__ void __launch_bounds__(MS_WARPS * 32) moe_stream_kernel(MoeGemmArgs p) {
    extern __shared__ uint4 xs[];                              // [MS_ROWS][K] of T
    pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.x >= *p.n_tiles) return;
    const int e = p.tile_expert[blockIdx.x], row0 = p.tile_row0[blockIdx.x];
    const int rows = min(MS_ROWS, p.offsets[e + 1] - row0);
    const int k16 = p.K / Piece<T>::N;
    for (int idx = threadIdx.x; idx < rows * k16; idx += blockDim.x) {
        const int r = idx / k16, k = idx - r * k16;
        const int src = p.top > 0 ? p.pair_of_slot[row0 + r] / p.top : row0 + r;
        xs[idx] = reinterpret_cast<const uint4*>((const T*)p.x + (size_t)src * p.ld_x)[k];
    }
    __syncthreads();
    const T* w = (const T*)p.w + (size_t)e * p.w_expert;
    const int pair0 = blockIdx.y * MS_PAIRS;
    if (rows <= 2) moe_stream_rows<T, TO, GATED, 2>(p, xs, w, row0, rows, pair0);
    else if (rows <= 4) moe_stream_rows<T, TO, GATED, 4>(p, xs, w, row0, rows, pair0);
    else if (rows <= 8) moe_stream_rows<T, TO, GATED, 8>(p, xs, w, row0, rows, pair0);
    else moe_stream_rows<T, TO, GATED, 16>(p, xs, w, row0, rows, pair0);
}

// ------------------------------------------------------------- the streaming form on the tensor cores (bfloat16)
// The same tiles of at most 16 slots.  A warp owns 16 weight rows and streams them 64 elements at a time through a
// two-stage buffer of its own (cp.async, 128 contiguous bytes a row); the tile's rows of x wait in shared memory, 512
// elements of K at a time.  mma.sync m16n8k16 with the weights as the row operand: D[weight row, slot], fp32 sums.  The
// kernel does almost no arithmetic; what counts is that every warp always has a piece of its weight rows in flight.
constexpr int MT_WARPS = 4, MT_KS = 64, MT_KC = 512, MT_WLD = MT_KS + 8, MT_XLD = MT_KC + 8;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename TO, bool GATED>
__global__ void __launch_bounds__(MT_WARPS * 32) moe_stream_tc_kernel(MoeGemmArgs p) {
    __shared__ __align__(16) __nv_bfloat16 xs[MS_ROWS * MT_XLD];                    // the tile's rows, one chunk of K
    __shared__ __align__(16) __nv_bfloat16 ws[MT_WARPS * 2 * 16 * MT_WLD];          // per warp: two stages of 16 x 64
    pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.x >= *p.n_tiles) return;
    const int e = p.tile_expert[blockIdx.x], row0 = p.tile_row0[blockIdx.x];
    const int rows = min(MS_ROWS, p.offsets[e + 1] - row0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n0 = (blockIdx.y * MT_WARPS + warp) * 16;                              // the warp's first weight row
    const __nv_bfloat16* w = (const __nv_bfloat16*)p.w + (size_t)e * p.w_expert;
    const __nv_bfloat16* x = (const __nv_bfloat16*)p.x;
    __nv_bfloat16* wb = ws + warp * 2 * 16 * MT_WLD;
    const int steps = p.K / MT_KS;
    auto issue = [&](int s) {
        __nv_bfloat16* dst = wb + (s & 1) * 16 * MT_WLD;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int piece = lane + 32 * i, r = piece >> 3, c = (piece & 7) * 8;
            __nv_bfloat16* d = dst + r * MT_WLD + c;
            if (n0 + r < p.N) {
                const uint32_t sa = (uint32_t)__cvta_generic_to_shared(d);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(w + (size_t)(n0 + r) * p.K + (size_t)s * MT_KS + c) : "memory");
            } else {
                *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float acc[2][4] = {};
    issue(0);
    for (int s = 0; s < steps; s++) {
        if (s % (MT_KC / MT_KS) == 0) {
            __syncthreads();                                    // the chunk before is consumed
            const int k0 = s * MT_KS, kn = min(MT_KC, p.K - k0) / 8;
            for (int idx = threadIdx.x; idx < MS_ROWS * kn; idx += blockDim.x) {
                const int r = idx / kn, c = idx - r * kn;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (r < rows) {
                    const int src = p.top > 0 ? p.pair_of_slot[row0 + r] / p.top : row0 + r;
                    v = reinterpret_cast<const uint4*>(x + (size_t)src * p.ld_x + k0)[c];
                }
                *reinterpret_cast<uint4*>(xs + r * MT_XLD + c * 8) = v;
            }
            __syncthreads();
        }
        if (s + 1 < steps) {
            issue(s + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncwarp();
        const __nv_bfloat16* wa = wb + (s & 1) * 16 * MT_WLD + (lane & 15) * MT_WLD + (lane >> 4) * 8;
        const __nv_bfloat16* xb = xs + ((lane >> 4) * 8 + (lane & 7)) * MT_XLD + (s % (MT_KC / MT_KS)) * MT_KS + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int kk = 0; kk < MT_KS; kk += 16) {
            uint32_t af[4], bf[4];
            ldsm_x4(af, wa + kk);
            ldsm_x4(bf, xb + kk);
            mma_16816(acc[0], af, bf[0], bf[1]);                // slots 0..7
            mma_16816(acc[1], af, bf[2], bf[3]);                // slots 8..15
        }
        __syncwarp();
    }
    // acc[j][0..1]: weight row g, slots 8 j + 2 t, + 1;  acc[j][2..3]: weight row g + 8
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int half = 0; half < 2; half++)
#pragma unroll
            for (int c = 0; c < 2; c++) {
                const float v = acc[j][2 * half + c];
                const int n = n0 + g + 8 * half, slot = 8 * j + 2 * t + c;
                if (GATED) {
                    const float up = __shfl_xor_sync(0xffffffffu, v, 4);     // the odd row beside this even one
                    if ((g & 1) == 0 && n < p.N && slot < rows) {
                        const float gt = fminf(v, p.limit), u = fminf(fmaxf(up, -p.limit), p.limit);
                        ((TO*)p.out)[(size_t)(row0 + slot) * p.ld_o + (n >> 1)] = from_float<TO>(gt / (1.0f + expf(-p.alpha * gt)) * (u + p.up_offset));
                    }
                } else if (n < p.N && slot < rows) {
                    ((TO*)p.out)[(size_t)(row0 + slot) * p.ld_o + n] = from_float<TO>(plain_act(v, p.act));
                }
            }
}

// xs[slot] = x[token of the slot's pair]: the rows of each expert side by side, for products that want plain matrices.
__global__ void moe_gather_kernel(const uint4* __restrict__ x, const int* __restrict__ pair_of_slot, int top, uint4* __restrict__ xs,
                                  int row16) {
    pdl_launch_dependents();
    pdl_wait();
    const int slot = blockIdx.x;
    const uint4* src = x + (size_t)(pair_of_slot[slot] / top) * row16;
    uint4* dst = xs + (size_t)slot * row16;
    for (int i = threadIdx.x; i < row16; i += blockDim.x) dst[i] = src[i];
}

// act[slot, j] = g sigmoid(alpha g) (u + 1), g = min(gu[slot, 2j], limit), u = clamp(gu[slot, 2j + 1], -limit, limit).
template <typename TO>
__global__ void moe_activation_kernel(const float2* __restrict__ gu, TO* __restrict__ act, size_t n, float limit, float alpha,
                                      float up_offset, const float2* __restrict__ bias, int ff) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float2 v = gu[i];
    if (bias) { const float2 b = bias[i % ff]; v.x += b.x; v.y += b.y; }       // (gate, up) biases, interleaved like the rows
    const float g = fminf(v.x, limit), u = fminf(fmaxf(v.y, -limit), limit);
    act[i] = from_float<TO>(g / (1.0f + expf(-alpha * g)) * (u + up_offset));
}

// act[i] = relu(x[i])^2: the activation of an ungated expert whose product left fp32 sums.
template <typename TO>
__global__ void moe_square_relu_kernel(const float* __restrict__ x, TO* __restrict__ act, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = x[i];
    act[i] = from_float<TO>(v > 0.0f ? v * v : 0.0f);
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ wgt, const int* __restrict__ slot_of_pair,
                                   int top, float* __restrict__ out, int accumulate, int hidden, const int* __restrict__ sel,
                                   int experts, const float* __restrict__ same_f, const __nv_bfloat16* __restrict__ same_h) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float s = 0.0f;
        for (int k = 0; k < top; k++) {
            // a choice from `experts` on is an identity expert: its output is the token's input row itself
            const bool same = sel && sel[(size_t)t * top + k] >= experts;
            const float v = same ? (same_f ? same_f[(size_t)t * hidden + i] : to_float(same_h[(size_t)t * hidden + i]))
                                 : y[(size_t)slot_of_pair[(size_t)t * top + k] * hidden + i];
            s = fmaf(wgt[(size_t)t * top + k], v, s);
        }
        out[(size_t)t * hidden + i] = accumulate ? out[(size_t)t * hidden + i] + s : s;
    }
}

}  // namespace ember

using namespace ember;

EMBER_API int ember_moe_tile_rows() { return MOE_BM; }

EMBER_API int ember_moe_route(const float* logits, int T, int E, int top, int* sel, float* wgt, int sigmoid, const float* correction,
                              float scale, int renormalize, int groups, int keep, void* stream) {
    if (T <= 0) return 0;
    if (E <= 0 || E > MOE_MAX_EXPERTS || top <= 0 || top > E || top > 32)
        return fail("moe_route: top %d of %d experts (at most 32 of %d)", top, E, MOE_MAX_EXPERTS);
    launch_kernel(moe_route_kernel, (unsigned)((T + 7) / 8), 256, 0, (cudaStream_t)stream, logits, E, top, sel, wgt, T,
                  RouteRule{sigmoid, correction, scale, renormalize, groups, keep});
    return check_launch("moe_route");
}

EMBER_API int ember_moe_router(const void* x, int x_dtype, const float* w, int T, int K, int E, int top, int* sel, float* wgt,
                               float* logits, int sigmoid, const float* correction, float scale, int renormalize, int groups, int keep,
                               void* stream) {
    if (T <= 0) return 0;
    const RouteRule rule{sigmoid, correction, scale, renormalize, groups, keep};
    if (groups < 0 || groups > 32 || (groups > 0 && (!sigmoid || E % groups || keep < 1 || keep > groups || top > keep * (E / groups))))
        return fail("moe_router: %d groups of which %d are kept, for top %d of %d experts", groups, keep, top, E);
    if (E <= 0 || E > MOE_MAX_EXPERTS || top <= 0 || top > E || top > 32 || K <= 0)
        return fail("moe_router: top %d of %d experts (at most 32 of %d), rows of %d", top, E, MOE_MAX_EXPERTS, K);
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned threads = 32 * (E < 16 ? E : 16);          // a warp an expert, up to sixteen (eight experts: one round, as before)
    if (x_dtype == EMBER_F32) launch_kernel(moe_router_kernel<float>, T, threads, 0, st, (const float*)x, w, K, E, top, sel, wgt, logits, rule);
    else if (x_dtype == EMBER_BF16)
        launch_kernel(moe_router_kernel<__nv_bfloat16>, T, threads, 0, st, (const __nv_bfloat16*)x, w, K, E, top, sel, wgt, logits, rule);
    else return fail("moe_router: unsupported dtype %d", x_dtype);
    return check_launch("moe_router");
}

EMBER_API int ember_moe_group(const int* sel, int n_pairs, int E, int* offsets, int* pair_of_slot, int* slot_of_pair, int* n_tiles,
                              int* tile_expert, int* tile_row0, int max_tiles, int tile_rows, int tiled, void* stream) {
    if (n_pairs <= 0) return 0;
    if (tile_rows != MOE_BM && tile_rows != MS_ROWS) return fail("moe_group: tiles of %d rows (%d or %d)", tile_rows, MOE_BM, MS_ROWS);
    if (E <= 0 || E > MOE_MAX_EXPERTS || max_tiles < n_pairs / tile_rows + E) return fail("moe_group: %d experts, room for %d tiles", E, max_tiles);
    launch_kernel(moe_group_kernel, 1, 1024, 0, (cudaStream_t)stream, sel, n_pairs, E, offsets, pair_of_slot, slot_of_pair, n_tiles,
                  tile_expert, tile_row0, max_tiles, tile_rows, (tiled <= 0 || tiled > E) ? E : tiled);
    return check_launch("moe_group");
}

EMBER_API int ember_moe_gemm(const void* x, int x_dtype, int ld_x, const void* w, int w_dtype, long long w_expert, void* out,
                             int out_dtype, int ld_o, const int* offsets, const int* pair_of_slot, const int* n_tiles,
                             const int* tile_expert, const int* tile_row0, int max_tiles, int top, int N, int K, int gated,
                             float limit, float alpha, float up_offset, int act, void* stream) {
    if (max_tiles <= 0) return 0;
    if (N <= 0 || K <= 0 || (gated && (N & 1))) return fail("moe_gemm: N=%d K=%d", N, K);
    MoeGemmArgs p{x, ld_x, w, w_expert, out, ld_o, offsets, pair_of_slot, n_tiles, tile_expert, tile_row0, top, N, K, limit, alpha, up_offset, act};
    dim3 grid(max_tiles, (N + MOE_BN - 1) / MOE_BN);
    cudaStream_t st = (cudaStream_t)stream;
    const int key = x_dtype * 100 + w_dtype * 10 + out_dtype;       // F32 = 0, BF16 = 1
    if (gated) {
        if (key == 0) launch_kernel(moe_gemm_kernel<float, float, float, true>, grid, 256, 0, st, p);
        else if (key == 111) launch_kernel(moe_gemm_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, true>, grid, 256, 0, st, p);
        else return fail("moe_gemm: unsupported dtypes %d", key);
    } else {
        if (key == 0) launch_kernel(moe_gemm_kernel<float, float, float, false>, grid, 256, 0, st, p);
        else if (key == 110) launch_kernel(moe_gemm_kernel<__nv_bfloat16, __nv_bfloat16, float, false>, grid, 256, 0, st, p);
        else if (key == 111) launch_kernel(moe_gemm_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, false>, grid, 256, 0, st, p);
        else return fail("moe_gemm: unsupported dtypes %d", key);
    }
    return check_launch("moe_gemm");
}

// The streaming form of ember_moe_gemm, for tile lists made with tiles of 16 rows.  Rows of x and of the weights must
// be multiples of 16 bytes, and 16 rows of x must fit in shared memory.
EMBER_API int ember_moe_stream_rows() { return MS_ROWS; }

EMBER_API int ember_moe_stream(const void* x, int x_dtype, int ld_x, const void* w, int w_dtype, long long w_expert, void* out,
                               int out_dtype, int ld_o, const int* offsets, const int* pair_of_slot, const int* n_tiles,
                               const int* tile_expert, const int* tile_row0, int max_tiles, int top, int N, int K, int gated,
                               float limit, float alpha, float up_offset, int act, void* stream) {
    if (max_tiles <= 0) return 0;
    if (N <= 0 || K <= 0 || (gated && (N & 1))) return fail("moe_stream: N=%d K=%d", N, K);
    const int elem = x_dtype == EMBER_F32 ? 4 : 2;
    if (((size_t)K * elem) % 16 || ((size_t)ld_x * elem) % 16) return fail("moe_stream: rows of %d elements are no multiple of 16 bytes", K);
    const size_t smem = (size_t)MS_ROWS * K * elem;
    if (smem > 200 * 1024) return fail("moe_stream: %d rows of %d do not fit in shared memory", MS_ROWS, K);
    MoeGemmArgs p{x, ld_x, w, w_expert, out, ld_o, offsets, pair_of_slot, n_tiles, tile_expert, tile_row0, top, N, K, limit, alpha, up_offset, act};
    cudaStream_t st = (cudaStream_t)stream;
    const int key = x_dtype * 100 + w_dtype * 10 + out_dtype;       // F32 = 0, BF16 = 1
    static int tc_on = -1;
    if (tc_on < 0) { const char* ev = getenv("EMBER_MOE_STREAM_TC"); tc_on = (ev && ev[0] == '0') ? 0 : 1; }
    if (tc_on && x_dtype == EMBER_BF16 && w_dtype == EMBER_BF16 && K % MT_KS == 0) {     // the tensor-core form
        dim3 tgrid(max_tiles, (N + MT_WARPS * 16 - 1) / (MT_WARPS * 16));
        if (gated && out_dtype == EMBER_BF16) launch_kernel(moe_stream_tc_kernel<__nv_bfloat16, true>, tgrid, MT_WARPS * 32, 0, st, p);
        else if (!gated && out_dtype == EMBER_F32) launch_kernel(moe_stream_tc_kernel<float, false>, tgrid, MT_WARPS * 32, 0, st, p);
        else if (!gated && out_dtype == EMBER_BF16) launch_kernel(moe_stream_tc_kernel<__nv_bfloat16, false>, tgrid, MT_WARPS * 32, 0, st, p);
        else return fail("moe_stream: unsupported dtypes %d", key);
        return check_launch("moe_stream_tc");
    }
    dim3 grid(max_tiles, ((N + 1) / 2 + MS_PAIRS - 1) / MS_PAIRS);
    auto run = [&](auto kernel) -> int {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return fail("moe_stream: shared memory %zu: %s", smem, cudaGetErrorString(e));
        }
        launch_kernel(kernel, grid, MS_WARPS * 32, smem, st, p);
        return check_launch("moe_stream");
    };
    if (gated) {
        if (key == 0) return run(moe_stream_kernel<float, float, true>);
        if (key == 111) return run(moe_stream_kernel<__nv_bfloat16, __nv_bfloat16, true>);
    } else {
        if (key == 0) return run(moe_stream_kernel<float, float, false>);
        if (key == 110) return run(moe_stream_kernel<__nv_bfloat16, float, false>);
        if (key == 111) return run(moe_stream_kernel<__nv_bfloat16, __nv_bfloat16, false>);
    }
    return fail("moe_stream: unsupported dtypes %d", key);
}

EMBER_API int ember_moe_gather(const void* x, const int* pair_of_slot, int n_pairs, int top, void* xs, int row_bytes, void* stream) {
    if (n_pairs <= 0) return 0;
    if (row_bytes <= 0 || row_bytes % 16) return fail("moe_gather: rows of %d bytes (a multiple of 16)", row_bytes);
    launch_kernel(moe_gather_kernel, n_pairs, 128, 0, (cudaStream_t)stream, (const uint4*)x, pair_of_slot, top, (uint4*)xs, row_bytes / 16);
    return check_launch("moe_gather");
}

EMBER_API int ember_moe_activation(const float* gu, void* act, int out_dtype, long long n, float limit, float alpha, float up_offset,
                                   const float* bias, int ff, void* stream) {
    if (n <= 0) return 0;
    if (bias && ff <= 0) return fail("moe_activation: biases for rows of %d", ff);
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dtype == EMBER_F32)
        launch_kernel(moe_activation_kernel<float>, blocks, 256, 0, st, (const float2*)gu, (float*)act, (size_t)n, limit, alpha, up_offset, (const float2*)bias, ff);
    else if (out_dtype == EMBER_BF16)
        launch_kernel(moe_activation_kernel<__nv_bfloat16>, blocks, 256, 0, st, (const float2*)gu, (__nv_bfloat16*)act, (size_t)n, limit, alpha, up_offset,
                      (const float2*)bias, ff);
    else return fail("moe_activation: unsupported dtype %d", out_dtype);
    return check_launch("moe_activation");
}

EMBER_API int ember_moe_square_relu(const float* x, void* act, int out_dtype, long long n, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dtype == EMBER_F32) launch_kernel(moe_square_relu_kernel<float>, blocks, 256, 0, st, x, (float*)act, (size_t)n);
    else if (out_dtype == EMBER_BF16) launch_kernel(moe_square_relu_kernel<__nv_bfloat16>, blocks, 256, 0, st, x, (__nv_bfloat16*)act, (size_t)n);
    else return fail("moe_square_relu: unsupported dtype %d", out_dtype);
    return check_launch("moe_square_relu");
}

EMBER_API int ember_moe_combine(const float* y, const float* wgt, const int* slot_of_pair, int T, int top, float* out, int accumulate,
                                int hidden, const int* sel, int experts, const void* same, int same_dtype, void* stream) {
    if (T <= 0) return 0;
    if (sel && (!same || (same_dtype != EMBER_F32 && same_dtype != EMBER_BF16))) return fail("moe_combine: identity experts need the tokens' input rows");
    launch_kernel(moe_combine_kernel, T, 256, 0, (cudaStream_t)stream, y, wgt, slot_of_pair, top, out, accumulate, hidden, sel, experts,
                  (const float*)(sel && same_dtype == EMBER_F32 ? same : nullptr),
                  (const __nv_bfloat16*)(sel && same_dtype == EMBER_BF16 ? same : nullptr));
    return check_launch("moe_combine");
}
