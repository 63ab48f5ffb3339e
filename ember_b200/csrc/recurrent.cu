// Recurrent mixers over a ragged batch: a short causal convolution whose last inputs are carried per request, a blend
// of every token's input with the previous token's (carried likewise), and
// five matrix-state recurrences (delta rule with a decay per key channel, matrix memory with exponential gating,
// selective state space with a scalar decay per head, gated linear attention with a decay per key channel, time mixing
// that reads the state before it is updated and reaches the current token through a bonus).  Everything that enters a recurrence is fp32: decays and
// their logarithms, softplus and exponentials, gates, unit norms, the state itself.
//
// A step's tokens are S runs (query_start [S + 1]); run s belongs to state slot slots[s].  A recurrence kernel runs
// one block per (run, head, tile of value columns): the block holds its [keys x columns] tile of the state in shared
// memory, walks the run's tokens in order and writes the tile back, so a prompt portion and a single decoded token
// are the same code and the state after a step does not depend on how the tokens were cut into steps.
#include "common.cuh"

EMBER_DEFINE_LAST_ERROR

namespace ember {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float logsigmoidf_(float x) { return fminf(x, 0.0f) - log1pf(expf(-fabsf(x))); }

// ------------------------------------------------------------------------------- short causal convolution + silu
// out[t, c] = silu(bias[c] + sum_j taps[c, j] * in(t - (n - 1 - j), c)) (or, silu = 0, the sum itself); inputs before the run come from the
// request's carried inputs carry[slot][j][c] (j = 0 the oldest of n - 1), zeros for a new request.
constexpr int CONV_MAX_TAPS = 8;  // taps the kernel keeps in registers; longer filters read them from memory

__global__ void conv_silu_kernel(const float* __restrict__ x, int ldx, int c0, const float* __restrict__ taps,
                                 const float* __restrict__ bias, int n, const float* __restrict__ carry, long long carry_stride,
                                 const int* __restrict__ seq_of, const int* __restrict__ query_start,
                                 const int* __restrict__ slots, float* __restrict__ out, int C, int silu, int T, int tt) {
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.y * tt,          // a block walks tt tokens: its taps and bias are read once for all of them
               c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float w[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; j++) w[j] = j < n ? taps[(size_t)c * n + j] : 0.0f;
    const float b = bias ? bias[c] : 0.0f;
    for (int t = t0; t < min(t0 + tt, T); t++) {
        const int s = seq_of[t], first = query_start[s];
        const float* cs = carry + (size_t)slots[s] * carry_stride;
        float acc = b;
        if (n <= CONV_MAX_TAPS) {
#pragma unroll
            for (int j = 0; j < CONV_MAX_TAPS; j++) {
                if (j >= n) break;
                const int src = t - (n - 1 - j);
                const float v = src >= first ? x[(size_t)src * ldx + c0 + c] : cs[(size_t)(n - 1 + src - first) * C + c];
                acc = fmaf(w[j], v, acc);
            }
        } else {
            for (int j = 0; j < n; j++) {
                const int src = t - (n - 1 - j);
                const float v = src >= first ? x[(size_t)src * ldx + c0 + c] : cs[(size_t)(n - 1 + src - first) * C + c];
                acc = fmaf(taps[(size_t)c * n + j], v, acc);
            }
        }
        out[(size_t)t * C + c] = silu ? acc / (1.0f + expf(-acc)) : acc;
    }
}

// After the convolution: the request's last n - 1 inputs (from the run, or shifted down from what was carried).
__global__ void conv_carry_kernel(const float* __restrict__ x, int ldx, int c0, int n, float* __restrict__ carry,
                                  long long carry_stride, const int* __restrict__ query_start, const int* __restrict__ slots, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int first = query_start[s], end = query_start[s + 1];
    float* cs = carry + (size_t)slots[s] * carry_stride;
    for (int j = 0; j < n - 1; j++) {                       // ascending: entry j reads entries above j only
        const int src = end - (n - 1) + j;
        cs[(size_t)j * C + c] = src >= first ? x[(size_t)src * ldx + c0 + c] : cs[(size_t)(n - 1 + src - first) * C + c];
    }
}

// ------------------------------------------------------------------------------- blends with the previous token
// out[m][t, c] = x[t, c] + (x'[t, c] - x[t, c]) * mu[m, c] for m < n_mix, x' the row of the token before t in its
// request: the row above inside a run, the request's carried row (zeros for a new request) at the start of a run.
template <typename TI, typename TO>
__global__ void token_shift_kernel(const TI* __restrict__ x, int C, const float* __restrict__ mu, int n_mix,
                                   const float* __restrict__ carry, long long carry_stride, const int* __restrict__ seq_of,
                                   const int* __restrict__ query_start, const int* __restrict__ slots, TO* __restrict__ out,
                                   size_t mix_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int s = seq_of[t];
    const float cur = to_float(x[(size_t)t * C + c]);
    const float before = t > query_start[s] ? to_float(x[(size_t)(t - 1) * C + c]) : carry[(size_t)slots[s] * carry_stride + c];
    const float d = before - cur;
    for (int m = 0; m < n_mix; m++) out[m * mix_stride + (size_t)t * C + c] = from_float<TO>(fmaf(d, mu[(size_t)m * C + c], cur));
}

// The same for rows that are a multiple of 16 bytes on 16-byte boundaries: a thread owns 16 bytes of a token's row
// (eight bfloat16 or four floats) and writes them to every blend.
template <typename T> struct Pack16;
template <> struct Pack16<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float* v) { const float4 a = *reinterpret_cast<const float4*>(p); v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w; }
    __device__ static void store(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Pack16<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void load(const __nv_bfloat16* p, float* v) {
        const uint4 a = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
        for (int j = 0; j < 4; j++) { const float2 f = __bfloat1622float2(h[j]); v[2 * j] = f.x, v[2 * j + 1] = f.y; }
    }
    __device__ static void store(__nv_bfloat16* p, const float* v) {
        uint4 a;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&a);
#pragma unroll
        for (int j = 0; j < 4; j++) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        *reinterpret_cast<uint4*>(p) = a;
    }
};

template <typename T>
__global__ void token_shift_vec_kernel(const T* __restrict__ x, int C, const float* __restrict__ mu, int n_mix,
                                       const float* __restrict__ carry, long long carry_stride, const int* __restrict__ seq_of,
                                       const int* __restrict__ query_start, const int* __restrict__ slots, T* __restrict__ out,
                                       size_t mix_stride) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int N = Pack16<T>::N;
    const int t = blockIdx.y, c = (blockIdx.x * blockDim.x + threadIdx.x) * N;
    if (c >= C) return;
    const int s = seq_of[t];
    float cur[N], d[N], r[N];
    Pack16<T>::load(x + (size_t)t * C + c, cur);
    if (t > query_start[s]) {
        Pack16<T>::load(x + (size_t)(t - 1) * C + c, d);
    } else {
        const float* row = carry + (size_t)slots[s] * carry_stride + c;
#pragma unroll
        for (int j = 0; j < N; j += 4) Pack16<float>::load(row + j, d + j);
    }
#pragma unroll
    for (int j = 0; j < N; j++) d[j] -= cur[j];
    for (int m = 0; m < n_mix; m++) {
        float w[N];
#pragma unroll
        for (int j = 0; j < N; j += 4) Pack16<float>::load(mu + (size_t)m * C + c + j, w + j);
#pragma unroll
        for (int j = 0; j < N; j++) r[j] = fmaf(d[j], w[j], cur[j]);
        Pack16<T>::store(out + m * mix_stride + (size_t)t * C + c, r);
    }
}

// After the blends: every run's last row becomes its request's carried row.
template <typename TI>
__global__ void token_carry_kernel(const TI* __restrict__ x, int C, float* __restrict__ carry, long long carry_stride,
                                   const int* __restrict__ query_start, const int* __restrict__ slots) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int first = query_start[s], end = query_start[s + 1];
    if (end > first) carry[(size_t)slots[s] * carry_stride + c] = to_float(x[(size_t)(end - 1) * C + c]);
}

// ------------------------------------------------------------------------------------------- state tiles
// Shared memory of a recurrence block: the state tile [D][VT] (VT = blockDim.x columns), then vectors.
// (`extra`, where given, is one more column, number V, kept apart from the matrix: D contiguous floats)
__device__ __forceinline__ void load_tile(float* tile, const float* __restrict__ S, int D, int V, int j, bool live,
                                          const float* __restrict__ extra = nullptr) {
    const int VT = blockDim.x;
    for (int i = 0; i < D; i++)
        tile[i * VT + threadIdx.x] = !live ? 0.0f : (j < V ? S[(size_t)i * V + j] : extra[i]);
}
__device__ __forceinline__ void store_tile(const float* tile, float* __restrict__ S, int D, int V, int j, bool live,
                                           float* __restrict__ extra = nullptr) {
    const int VT = blockDim.x;
    if (live)
        for (int i = 0; i < D; i++) {
            if (j < V) S[(size_t)i * V + j] = tile[i * VT + threadIdx.x];
            else extra[i] = tile[i * VT + threadIdx.x];
        }
}

// ---------------------------------------------------------------------- delta rule, one decay per key channel
// Per head (value head h reads query/key head h / (H / G)):
//   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
// with q, k unit vectors (q also times D^-1/2), beta = sigmoid(.), g = exp(-exp(A_log) softplus(a + dt_bias)).
struct DeltaArgs {
    const float* conv; int ld_conv;        // [T, G D | G D | H V] after convolution and silu
    const float* beta; int ld_beta;        // [T, H] logits
    const float* a; int ld_a;              // [T, H D] decay logits (before the bias); a_head: [T, H], one decay per head
    const float* dt_bias;                  // [H D] (a_head: [H])
    const float* A_log;                    // [H]
    float* state; long long state_stride;  // [slot][H][D][V]
    float* out;                            // [T, H V]
    const int* query_start; const int* slots;
    int H, G, D, V;
    float key_eps;
    int a_head;
};

__global__ void delta_scan_kernel(DeltaArgs p) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, VT = blockDim.x, j = blockIdx.z * VT + threadIdx.x;
    const int D = p.D, V = p.V, kv = h / (p.H / p.G);
    const bool live = j < V;
    float* tile = smem;                       // [D][VT]
    float* vec = smem + (size_t)D * VT;       // 2 x (k[D], q[D], g[D])
    float* red = vec + 6 * D;                 // 2 x 2 x 32 partial sums
    float* S = p.state + (size_t)p.slots[s] * p.state_stride + (size_t)h * D * V;
    load_tile(tile, S, D, V, j, live);
    const float rate = expf(p.A_log[h]), qscale = 1.0f / sqrtf((float)D);
    const int first = p.query_start[s], end = p.query_start[s + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = VT >> 5;
    const int off_k = p.G * D, off_v = 2 * p.G * D;
    for (int t = first; t < end; t++) {
        const int b = (t - first) & 1;
        float* kb = vec + b * 3 * D, *qb = kb + D, *gb = qb + D;
        const float* row = p.conv + (size_t)t * p.ld_conv;
        float sk = 0.0f, sq = 0.0f;
        for (int i = threadIdx.x; i < D; i += VT) {
            const float kr = row[off_k + kv * D + i], qr = row[kv * D + i];
            kb[i] = kr; qb[i] = qr;
            sk = fmaf(kr, kr, sk); sq = fmaf(qr, qr, sq);
            const int ai = p.a_head ? h : h * D + i;
            gb[i] = expf(-rate * softplusf_(p.a[(size_t)t * p.ld_a + ai] + p.dt_bias[ai]));
        }
        sk = warp_sum(sk); sq = warp_sum(sq);
        if (lane == 0) { red[b * 64 + warp] = sk; red[b * 64 + 32 + warp] = sq; }
        __syncthreads();
        sk = 0.0f; sq = 0.0f;
        for (int w = 0; w < nwarps; w++) { sk += red[b * 64 + w]; sq += red[b * 64 + 32 + w]; }
        const float kn = 1.0f / sqrtf(sk + p.key_eps), qn = qscale / sqrtf(sq + p.key_eps);
        if (live) {
            const float beta = sigmoidf_(p.beta[(size_t)t * p.ld_beta + h]);
            const float v = row[off_v + h * V + j];
            float acc = 0.0f;
            for (int i = 0; i < D; i++) {
                const float x = tile[i * VT + threadIdx.x] * gb[i];
                tile[i * VT + threadIdx.x] = x;
                acc = fmaf(x, kb[i] * kn, acc);
            }
            const float u = beta * (v - acc);
            float o = 0.0f;
            for (int i = 0; i < D; i++) {
                const float x = fmaf(kb[i] * kn, u, tile[i * VT + threadIdx.x]);
                tile[i * VT + threadIdx.x] = x;
                o = fmaf(x, qb[i], o);
            }
            p.out[(size_t)t * p.H * V + h * V + j] = o * qn;
        }
    }
    store_tile(tile, S, D, V, j, live);
}

// ------------------------------------------------------- gated linear attention, one decay per key channel
//   S <- diag(alpha) S + k v^T;  o = S^T q,  alpha = sigmoid(z + bias)^(1 / tau), q scaled by D^-1/2.
// The general form (the state tile in shared memory), for more than 256 key channels.
struct GlaArgs {
    const float* proj; int ld; int off_q, off_k, off_v;   // [T, ...]: q, k (H D each), v (H V)
    const float* z; int ld_z;                             // [T, H D] decay logits (before the bias)
    const float* z_bias;                                  // [H D] or null
    float decay_power;                                    // 1 / tau
    float* state; long long state_stride;                 // [slot][H][D][V]
    float* out;                                           // [T, H V]
    const int* query_start; const int* slots;
    int H, D, V;
};

__global__ void gla_scan_kernel(GlaArgs p) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, VT = blockDim.x, j = blockIdx.z * VT + threadIdx.x;
    const int D = p.D, V = p.V;
    const bool live = j < V;
    float* tile = smem;                       // [D][VT]
    float* vec = smem + (size_t)D * VT;       // 2 x (k[D], q[D], alpha[D])
    float* S = p.state + (size_t)p.slots[s] * p.state_stride + (size_t)h * D * V;
    load_tile(tile, S, D, V, j, live);
    const float qscale = 1.0f / sqrtf((float)D);
    const int first = p.query_start[s], end = p.query_start[s + 1];
    for (int t = first; t < end; t++) {
        const int b = (t - first) & 1;
        float* kb = vec + b * 3 * D, *qb = kb + D, *gb = qb + D;
        const float* row = p.proj + (size_t)t * p.ld;
        for (int i = threadIdx.x; i < D; i += VT) {
            kb[i] = row[p.off_k + h * D + i];
            qb[i] = row[p.off_q + h * D + i] * qscale;
            gb[i] = expf(logsigmoidf_(p.z[(size_t)t * p.ld_z + h * D + i] + (p.z_bias ? p.z_bias[h * D + i] : 0.0f)) * p.decay_power);
        }
        __syncthreads();
        if (live) {
            const float v = row[p.off_v + h * V + j];
            float o = 0.0f;
            for (int i = 0; i < D; i++) {
                const float x = fmaf(kb[i], v, tile[i * VT + threadIdx.x] * gb[i]);
                tile[i * VT + threadIdx.x] = x;
                o = fmaf(x, qb[i], o);
            }
            p.out[(size_t)t * p.H * V + h * V + j] = o;
        }
    }
    store_tile(tile, S, D, V, j, live);
}

//

// ------------------------------------------------------------------ time mixing, one decay per key channel
//   o = (S + diag(u) k v^T)^T r;  S <- diag(w) S + k v^T,  w = exp(-exp(z + w0)), u a bonus per head and key channel.
// The general form (the state tile in shared memory), for more than 256 key channels.
struct WkvArgs {
    const float* proj; int ld; int off_r, off_k, off_v;   // [T, ...]: r, k (H D each), v (H V)
    const float* z; int ld_z;                             // [T, H D] decay logits (before w0)
    const float* w0; const float* bonus;                  // [H D] each
    float* state; long long state_stride;                 // [slot][H][D][V]
    float* out;                                           // [T, H V]
    const int* query_start; const int* slots;
    int H, D, V;
};

__global__ void wkv_scan_kernel(WkvArgs p) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, VT = blockDim.x, j = blockIdx.z * VT + threadIdx.x;
    const int D = p.D, V = p.V;
    const bool live = j < V;
    float* tile = smem;                       // [D][VT]
    float* vec = smem + (size_t)D * VT;       // 2 x (k[D], r[D], w[D], u k[D])
    float* S = p.state + (size_t)p.slots[s] * p.state_stride + (size_t)h * D * V;
    load_tile(tile, S, D, V, j, live);
    const int first = p.query_start[s], end = p.query_start[s + 1];
    for (int t = first; t < end; t++) {
        const int b = (t - first) & 1;
        float* kb = vec + b * 4 * D, *rb = kb + D, *wb = rb + D, *ub = wb + D;
        const float* row = p.proj + (size_t)t * p.ld;
        for (int i = threadIdx.x; i < D; i += VT) {
            const float k = row[p.off_k + h * D + i];
            kb[i] = k;
            rb[i] = row[p.off_r + h * D + i];
            wb[i] = expf(-expf(p.z[(size_t)t * p.ld_z + h * D + i] + p.w0[h * D + i]));
            ub[i] = p.bonus[h * D + i] * k;
        }
        __syncthreads();
        if (live) {
            const float v = row[p.off_v + h * V + j];
            float o = 0.0f;
            for (int i = 0; i < D; i++) {
                const float x = tile[i * VT + threadIdx.x];
                o = fmaf(fmaf(ub[i], v, x), rb[i], o);
                tile[i * VT + threadIdx.x] = fmaf(kb[i], v, wb[i] * x);
            }
            p.out[(size_t)t * p.H * V + h * V + j] = o;
        }
    }
    store_tile(tile, S, D, V, j, live);
}

// ------------------------------------------------------------- matrix memory with exponential input gate
// Per head, with log gates i~ = cap tanh((i + b_i) / cap), f~ = logsigmoid(cap tanh((f + b_f) / cap)) and a running
// maximum m (0 for a new request):
//   m' = max(f~ + m, i~);  S <- e^(f~ + m - m') S + e^(i~ - m') k v^T;  n likewise with k;
//   o = S^T q / (max(|n . q|, e^(-m')) + 1e-6),  q scaled by D^-1/2.
// n is the matrix's column number V (its "value" is 1), so n . q is that column's read-out.  Two kernels: the first
// runs the scalar recurrence of m, one warp per (run, head), 32 tokens at a time as a prefix scan over the pairs
// (f~, i~) under (a2, b2) o (a1, b1) = (a1 + a2, max(b1 + a2, b2)), and leaves (keep, put, e^-m') per token; the
// second applies them to the columns and leaves S^T q and n . q; the division is the normalising kernel's.
struct MemoryArgs {
    const float* proj; int ld;             // [T, ...]: q, k (H D each), v (H V), input and forget logits (H each)
    int off_q, off_k, off_v, off_i, off_f;
    const float* bias_i; const float* bias_f;   // [H]
    float cap;
    float* state; long long state_stride;  // [slot]: S [H][D][V], then n [H][D], then m [H]
    float* gates;                          // [T, H, 4]: keep, put, e^-m', n . q
    float* out;                            // [T, H V]: S^T q
    const int* query_start; const int* slots;
    int H, D, V;
};

__global__ void memory_gates_kernel(MemoryArgs p) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, H = p.H, lane = threadIdx.x;
    float* mst = p.state + (size_t)p.slots[s] * p.state_stride + (size_t)H * p.D * p.V + (size_t)H * p.D + h;
    const int first = p.query_start[s], end = p.query_start[s + 1];
    float m_in = *mst;
    const float bi = p.bias_i[h], bf = p.bias_f[h];
    for (int t0 = first; t0 < end; t0 += 32) {
        const int t = t0 + lane;
        const bool valid = t < end;
        float fg = 0.0f, ig = -INFINITY;                       // a token beyond the run leaves m as it is
        if (valid) {
            const float* row = p.proj + (size_t)t * p.ld;
            ig = p.cap * tanhf((row[p.off_i + h] + bi) / p.cap);
            fg = logsigmoidf_(p.cap * tanhf((row[p.off_f + h] + bf) / p.cap));
        }
        float a = fg, b = ig;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const float pa = __shfl_up_sync(0xffffffffu, a, off), pb = __shfl_up_sync(0xffffffffu, b, off);
            if (lane >= off) { b = fmaxf(pb + a, b); a = pa + a; }
        }
        const float m = fmaxf(a + m_in, b);
        float m_prev = __shfl_up_sync(0xffffffffu, m, 1);
        if (lane == 0) m_prev = m_in;
        if (valid) {
            float* g = p.gates + ((size_t)t * H + h) * 4;
            g[0] = expf(fg + m_prev - m); g[1] = expf(ig - m); g[2] = expf(-m);
        }
        m_in = __shfl_sync(0xffffffffu, m, 31);
    }
    if (lane == 0 && first < end) *mst = m_in;
}

__global__ void memory_scan_kernel(MemoryArgs p) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, VT = blockDim.x, j = blockIdx.z * VT + threadIdx.x;
    const int D = p.D, V = p.V, H = p.H;
    const bool live = j <= V;                 // column V is n
    float* tile = smem;                       // [D][VT]
    float* vec = smem + (size_t)D * VT;       // 2 x (k[D], q[D])
    float* base = p.state + (size_t)p.slots[s] * p.state_stride;
    float* S = base + (size_t)h * D * V;
    float* nst = base + (size_t)H * D * V + (size_t)h * D;
    load_tile(tile, S, D, V, j, live, nst);
    const int first = p.query_start[s], end = p.query_start[s + 1];
    const float qscale = 1.0f / sqrtf((float)D);
    for (int t = first; t < end; t++) {
        const int b = (t - first) & 1;
        float* kb = vec + b * 2 * D, *qb = kb + D;
        const float* row = p.proj + (size_t)t * p.ld;
        for (int i = threadIdx.x; i < D; i += VT) {
            kb[i] = row[p.off_k + h * D + i];
            qb[i] = row[p.off_q + h * D + i] * qscale;
        }
        float* g = p.gates + ((size_t)t * H + h) * 4;
        const float keep = g[0], put = g[1];
        __syncthreads();
        if (live) {
            const float pv = put * (j < V ? row[p.off_v + h * V + j] : 1.0f);
            float o = 0.0f;
            for (int i = 0; i < D; i++) {
                const float x = fmaf(kb[i], pv, keep * tile[i * VT + threadIdx.x]);
                tile[i * VT + threadIdx.x] = x;
                o = fmaf(x, qb[i], o);
            }
            if (j < V) p.out[(size_t)t * H * V + h * V + j] = o;
            else g[3] = o;
        }
    }
    store_tile(tile, S, D, V, j, live, nst);
}

// ------------------------------------------------------------------- selective state space, scalar decay per head
// Per head (head h reads B, C of group h / (H / G)), dt = softplus(dt_raw + dt_bias):
//   S <- e^(-e^(A_log) dt) S + dt B x^T  (S is N x V);  y = S^T C + D_skip x.
struct SsmArgs {
    const float* conv; int ld_conv;        // [T, H V | G N | G N] after convolution and silu: x, B, C
    const float* dt; int ld_dt;            // [T, H] raw step sizes
    const float* dt_bias; const float* A_log; const float* skip;   // [H]
    float* state; long long state_stride;  // [slot][H][N][V]
    float* out;                            // [T, H V]
    const int* query_start; const int* slots;
    int H, G, N, V;
};

__global__ void ssm_scan_kernel(SsmArgs p) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, VT = blockDim.x, j = blockIdx.z * VT + threadIdx.x;
    const int N = p.N, V = p.V, H = p.H, g = h / (H / p.G);
    const bool live = j < V;
    float* tile = smem;                       // [N][VT]
    float* vec = smem + (size_t)N * VT;       // 2 x (B[N], C[N])
    float* S = p.state + (size_t)p.slots[s] * p.state_stride + (size_t)h * N * V;
    load_tile(tile, S, N, V, j, live);
    const float rate = expf(p.A_log[h]), bias = p.dt_bias[h], skip = p.skip[h];
    const int first = p.query_start[s], end = p.query_start[s + 1];
    const int off_b = H * V + g * N, off_c = H * V + p.G * N + g * N;
    for (int t = first; t < end; t++) {
        const int b = (t - first) & 1;
        float* Bb = vec + b * 2 * N, *Cb = Bb + N;
        const float* row = p.conv + (size_t)t * p.ld_conv;
        for (int i = threadIdx.x; i < N; i += VT) { Bb[i] = row[off_b + i]; Cb[i] = row[off_c + i]; }
        const float dt = softplusf_(p.dt[(size_t)t * p.ld_dt + h] + bias);
        const float keep = expf(-rate * dt);
        __syncthreads();
        if (live) {
            const float x = row[h * V + j], dx = dt * x;
            float y = 0.0f;
            for (int i = 0; i < N; i++) {
                const float v = fmaf(Bb[i], dx, keep * tile[i * VT + threadIdx.x]);
                tile[i * VT + threadIdx.x] = v;
                y = fmaf(v, Cb[i], y);
            }
            p.out[(size_t)t * H * V + h * V + j] = fmaf(skip, x, y);
        }
    }
    store_tile(tile, S, N, V, j, live);
}

// ------------------------------------------------------------------ the same recurrences, state in registers
// For up to 256 state rows a block takes 32 value columns: lane = row group r (RG = 8 or 16 of them) + RG x column,
// and a thread keeps rows r RS .. r RS + RS - 1 of its column in registers.  A dot product over the rows
// is RS multiply-adds and log2(RG) shuffles; the per-token vectors live in shared memory, one padding word per row
// group so that the eight groups read eight banks.  The state goes through a shared tile when it is loaded and
// stored, so that global memory sees whole 128-byte rows.  A prompt portion of one request keeps 8 times the threads
// of the kernels above busy; those stay for more than 256 rows.
constexpr int RCOLS = 32;

// RG row groups (8 or 16 lanes of a warp share a column), RS rows a thread, 32 RG threads a block.  The state goes
// through a shared tile: every thread first fetches RS values of whole 128-byte rows (all loads in flight together).
template <int RS, int RG>
__device__ __forceinline__ void regs_load(float (&st)[RS], float* tile, const float* __restrict__ S, int D, int V, int col0,
                                          const float* __restrict__ extra = nullptr) {
    const int c = threadIdx.x & 31, w = threadIdx.x >> 5;
    float tmp[RS];
#pragma unroll
    for (int k = 0; k < RS; k++) {
        const int i = w + RG * k;                      // (RG warps a block: rows w, w + RG, ...)
        tmp[k] = (i < D && col0 + c < V) ? S[(size_t)i * V + col0 + c]
                                         : ((extra && i < D && col0 + c == V) ? extra[i] : 0.0f);
    }
#pragma unroll
    for (int k = 0; k < RS; k++) tile[(w + RG * k) * 33 + c] = tmp[k];
    __syncthreads();
    const int lane = threadIdx.x & 31, r = lane % RG, cc = w * (32 / RG) + lane / RG;
#pragma unroll
    for (int ii = 0; ii < RS; ii++) st[ii] = tile[(r * RS + ii) * 33 + cc];
}
template <int RS, int RG>
__device__ __forceinline__ void regs_store(const float (&st)[RS], float* tile, float* __restrict__ S, int D, int V, int col0,
                                           float* __restrict__ extra = nullptr) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, r = lane % RG, cc = w * (32 / RG) + lane / RG;
    __syncthreads();
#pragma unroll
    for (int ii = 0; ii < RS; ii++) tile[(r * RS + ii) * 33 + cc] = st[ii];
    __syncthreads();
    const int c = lane;
#pragma unroll
    for (int k = 0; k < RS; k++) {
        const int i = w + RG * k;
        if (i < D) {
            if (col0 + c < V) S[(size_t)i * V + col0 + c] = tile[i * 33 + c];
            else if (extra && col0 + c == V) extra[i] = tile[i * 33 + c];
        }
    }
}
template <int RG>
__device__ __forceinline__ float rows_sum(float v) {
#pragma unroll
    for (int off = 1; off < RG; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// One kernel for the five recurrences (MODE 0 delta rule, 1 matrix memory, 2 state space, 3 gated linear attention:
// S <- diag(alpha) S + k v^T, o = S^T q with alpha = sigmoid(z + bias)^(1 / tau) per key channel and q times D^-1/2; 4 time
// mixing: o = S^T r + (r . (u k)) v read before S <- diag(w) S + k v^T, w = exp(-exp(z + w0)); the bonus's dot product
// r . (u k) is a warp sum made with the token's vectors).  A run is walked in chunks
// of CT tokens: while a chunk is computed from shared memory (no block-wide barrier between its tokens), the next
// chunk's inputs are already on their way into registers; each warp then prepares its tokens of that chunk (unit
// norms, decays, gates: a token's vector is spread over the warp's lanes, so its sums are warp sums) and stores
// them into the other buffer.  Per token a thread does RS multiply-adds per dot product and one round of three
// shuffles: the delta rule's two dot products S^T k and S^T q are both taken of the decayed state (o = q . S_decayed
// + (k . q) u), so they share the round and the rank-one update is off the critical path.
struct ScanArgs {
    float* state; long long state_stride; float* out; const int* query_start; const int* slots;
    int H, G, D, V;                        // D: rows of the state (key channels, or state size)
    const float* x; int ld_x;              // delta, state space: [T, ...] after convolution and silu; matrix memory: the projection
    const float* b; int ld_b;              // delta: write-strength logits [T, H]; state space: raw step sizes [T, H]
    const float* a; int ld_a;              // delta: decay logits [T, H D]
    const float* dt_bias; const float* A_log; const float* skip;
    float key_eps;
    int off_q, off_k, off_v;               // matrix memory: columns of x
    float* gates;                          // matrix memory: [T, H, 4]
    float decay_power;                     // gated linear attention: 1 / tau
    const float* bonus;                    // time mixing: u [H D] (its w0 is dt_bias)
    int a_head;                            // delta: one decay logit (and bias) per head instead of per head and key channel
};

template <int N>
struct TokenRegs {                                  // one token's vectors, scalars and column value, in registers
    float4 v0[N], v1[N], v2[N], sc;
    float val;
};

template <int MODE, int RS, int CT, int RG>
__global__ void __launch_bounds__(32 * RG, CT == 1 ? 3 : 1) scan_chunks_kernel(ScanArgs p) {
    constexpr int RTHREADS = 32 * RG, NW = RG;      // warps a block: 32 columns, 32 / RG of them a warp
    extern __shared__ __align__(16) float smem[];
    pdl_launch_dependents();
    pdl_wait();
    constexpr int NV = (MODE == 0 || MODE == 3 || MODE == 4) ? 3 : 2;
    constexpr int VS = RG * (RS + 4);               // a vector in shared memory: row group r starts at r (RS + 4)
    constexpr int TOK = NV * VS + 4 + RCOLS;        // vectors, four scalars, the block's 32 column values
    constexpr int TPW = (CT + NW - 1) / NW, EPL = RG * RS / 32;   // (CT: 16 or 8 tokens a chunk for prompt portions, 1 for decode steps)
    const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * RCOLS;
    const int D = p.D, V = p.V, H = p.H, grp = h / (H / p.G);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, r = lane % RG;
    const int cw = warp * (32 / RG) + lane / RG, j = col0 + cw, base = r * (RS + 4);
    const int n_cols = MODE == 1 ? V + 1 : V;       // (matrix memory: column V is n)
    const bool live = j < n_cols;
    float* tile = smem;                             // [RG RS][33], used when the state is loaded and stored
    float* chunks = smem + RG * RS * 33;            // 2 x CT x TOK
    float* sbase = p.state + (size_t)p.slots[s] * p.state_stride;
    float* S = sbase + (size_t)h * D * V;
    float* extra = MODE == 1 ? sbase + (size_t)H * D * V + (size_t)h * D : nullptr;
    float st[RS];
    for (int i = threadIdx.x; i < 2 * CT * TOK; i += RTHREADS) chunks[i] = 0.0f;
    const int first = p.query_start[s], end = p.query_start[s + 1];
    const float rate = (MODE == 1 || MODE == 3 || MODE == 4) ? 0.0f : expf(p.A_log[h]);
    const float qscale = 1.0f / sqrtf((float)D);
    // where this head's vectors start in a row of x
    constexpr bool PROJ = MODE == 1 || MODE == 3 || MODE == 4;        // q (or r), k, v at given columns of one projection
    const int off0 = MODE == 0 ? p.G * D + grp * D : (PROJ ? p.off_k + h * D : H * V + grp * D);               // k | k | B
    const int off1 = MODE == 0 ? grp * D : (PROJ ? p.off_q + h * D : H * V + p.G * D + grp * D);               // q | q | C
    const int off_col = MODE == 0 ? 2 * p.G * D + h * V : (PROJ ? p.off_v + h * V : h * V);                    // v | v | x

    float f0[TPW][EPL], f1[TPW][EPL], f2[TPW][EPL], fc[TPW], fs[TPW];
    auto prefetch = [&](int t0) {
#pragma unroll
        for (int w = 0; w < TPW; w++) {
            const int t = t0 + warp + NW * w;
            if (warp + NW * w >= CT || t >= end) continue;
            const float* row = p.x + (size_t)t * p.ld_x;
#pragma unroll
            for (int m = 0; m < EPL; m++) {
                const int i = lane + 32 * m;
                if (i < D) {
                    f0[w][m] = row[off0 + i];
                    f1[w][m] = row[off1 + i];
                    if (MODE == 0 || MODE == 3 || MODE == 4) f2[w][m] = p.a[(size_t)t * p.ld_a + ((MODE == 0 && p.a_head) ? h : h * D + i)];
                }
            }
            const int c = col0 + lane;
            fc[w] = c < V ? row[off_col + c] : 1.0f;
            if (MODE == 0 || MODE == 2) fs[w] = p.b[(size_t)t * p.ld_b + h];
        }
    };
    auto prepare = [&](int t0, float* buf) {
#pragma unroll
        for (int w = 0; w < TPW; w++) {
            const int tt = warp + NW * w, t = t0 + tt;
            if (tt >= CT || t >= end) continue;
            float* tok = buf + tt * TOK;
            float s0 = 0.0f, s1 = 0.0f, s01 = 0.0f;
#pragma unroll
            for (int m = 0; m < EPL; m++) {
                const int i = lane + 32 * m;
                if (i < D) {
                    const int vi = i + (i / RS) * 4;
                    tok[vi] = f0[w][m];
                    tok[VS + vi] = (MODE == 1 || MODE == 3) ? f1[w][m] * qscale : f1[w][m];
                    if (MODE == 3)      // alpha = sigmoid(z)^(1 / tau) = exp(logsigmoid(z) / tau)
                        tok[2 * VS + vi] = expf(logsigmoidf_(f2[w][m] + (p.dt_bias ? p.dt_bias[h * D + i] : 0.0f)) * p.decay_power);
                    if (MODE == 4) {
                        tok[2 * VS + vi] = expf(-expf(f2[w][m] + p.dt_bias[h * D + i]));
                        s0 = fmaf(f1[w][m] * p.bonus[h * D + i], f0[w][m], s0);          // r . (u k)
                    }
                    if (MODE == 0) {
                        tok[2 * VS + vi] = expf(-rate * softplusf_(f2[w][m] + p.dt_bias[p.a_head ? h : h * D + i]));
                        s0 = fmaf(f0[w][m], f0[w][m], s0); s1 = fmaf(f1[w][m], f1[w][m], s1); s01 = fmaf(f0[w][m], f1[w][m], s01);
                    }
                }
            }
            tok[NV * VS + 4 + lane] = fc[w];
            if (MODE == 0) {
                s0 = warp_sum(s0); s1 = warp_sum(s1); s01 = warp_sum(s01);
                if (lane == 0) {
                    tok[NV * VS + 0] = 1.0f / sqrtf(s0 + p.key_eps);            // 1 / |k|
                    tok[NV * VS + 1] = qscale / sqrtf(s1 + p.key_eps);          // D^-1/2 / |q|
                    tok[NV * VS + 2] = s01;                                     // k . q, before the norms
                    tok[NV * VS + 3] = sigmoidf_(fs[w]);
                }
            } else if (MODE == 4) {
                s0 = warp_sum(s0);
                if (lane == 0) tok[NV * VS + 0] = s0;
            } else if (MODE == 1) {
                if (lane == 0) {
                    const float* g = p.gates + ((size_t)t * H + h) * 4;
                    tok[NV * VS + 0] = g[0]; tok[NV * VS + 1] = g[1];
                }
            } else if (MODE == 2 && lane == 0) {
                const float dt = softplusf_(fs[w] + p.dt_bias[h]);
                tok[NV * VS + 0] = expf(-rate * dt); tok[NV * VS + 1] = dt;
            }
        }
    };

    const float skip = MODE == 2 ? p.skip[h] : 0.0f;
    prefetch(first);                                // (before the state: both trips to global memory overlap)
    regs_load<RS, RG>(st, tile, S, D, V, col0, extra);
    prepare(first, chunks);
    __syncthreads();
    int cur = 0;
    for (int t0 = first; t0 < end; t0 += CT, cur ^= 1) {
        const bool more = t0 + CT < end;
        if (more) prefetch(t0 + CT);
        const int n = min(CT, end - t0);
        const float* buf = chunks + cur * CT * TOK;
        // a token's operands are fetched into registers while the token before it is computed (two register sets,
        // the loop unrolled by two), so that no multiply-add waits for shared memory
        auto fetch = [&](int tt, TokenRegs<RS / 4>& x) {
            const float* tok = buf + tt * TOK;
            x.sc = *reinterpret_cast<const float4*>(tok + NV * VS);
            x.val = tok[NV * VS + 4 + cw];
#pragma unroll
            for (int i4 = 0; i4 < RS / 4; i4++) {
                x.v0[i4] = reinterpret_cast<const float4*>(tok + base)[i4];
                x.v1[i4] = reinterpret_cast<const float4*>(tok + VS + base)[i4];
                if (MODE == 0 || MODE == 3 || MODE == 4) x.v2[i4] = reinterpret_cast<const float4*>(tok + 2 * VS + base)[i4];
            }
        };
        auto step = [&](int tt, const TokenRegs<RS / 4>& x) {
            float o;
            if (MODE == 0) {
                float ak[4] = {0.0f, 0.0f, 0.0f, 0.0f}, aq[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int i4 = 0; i4 < RS / 4; i4++) {
                    const float4 k = x.v0[i4], q = x.v1[i4], g = x.v2[i4];
                    st[4 * i4 + 0] *= g.x; st[4 * i4 + 1] *= g.y; st[4 * i4 + 2] *= g.z; st[4 * i4 + 3] *= g.w;
                    ak[0] = fmaf(st[4 * i4 + 0], k.x, ak[0]); ak[1] = fmaf(st[4 * i4 + 1], k.y, ak[1]);
                    ak[2] = fmaf(st[4 * i4 + 2], k.z, ak[2]); ak[3] = fmaf(st[4 * i4 + 3], k.w, ak[3]);
                    aq[0] = fmaf(st[4 * i4 + 0], q.x, aq[0]); aq[1] = fmaf(st[4 * i4 + 1], q.y, aq[1]);
                    aq[2] = fmaf(st[4 * i4 + 2], q.z, aq[2]); aq[3] = fmaf(st[4 * i4 + 3], q.w, aq[3]);
                }
                float sk = (ak[0] + ak[1]) + (ak[2] + ak[3]), sq = (aq[0] + aq[1]) + (aq[2] + aq[3]);
#pragma unroll
                for (int off = 1; off < RG; off <<= 1) {
                    sk += __shfl_xor_sync(0xffffffffu, sk, off);
                    sq += __shfl_xor_sync(0xffffffffu, sq, off);
                }
                const float uk = x.sc.w * (x.val - sk * x.sc.x) * x.sc.x;      // beta (v - S^T k) / |k|
                o = x.sc.y * fmaf(uk, x.sc.z, sq);
#pragma unroll
                for (int i4 = 0; i4 < RS / 4; i4++) {
                    const float4 k = x.v0[i4];
                    st[4 * i4 + 0] = fmaf(k.x, uk, st[4 * i4 + 0]); st[4 * i4 + 1] = fmaf(k.y, uk, st[4 * i4 + 1]);
                    st[4 * i4 + 2] = fmaf(k.z, uk, st[4 * i4 + 2]); st[4 * i4 + 3] = fmaf(k.w, uk, st[4 * i4 + 3]);
                }
            } else if (MODE == 4) {
                float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int i4 = 0; i4 < RS / 4; i4++) {
                    const float4 k = x.v0[i4], q = x.v1[i4], g = x.v2[i4];
                    acc[0] = fmaf(st[4 * i4 + 0], q.x, acc[0]); acc[1] = fmaf(st[4 * i4 + 1], q.y, acc[1]);
                    acc[2] = fmaf(st[4 * i4 + 2], q.z, acc[2]); acc[3] = fmaf(st[4 * i4 + 3], q.w, acc[3]);
                    st[4 * i4 + 0] = fmaf(k.x, x.val, g.x * st[4 * i4 + 0]); st[4 * i4 + 1] = fmaf(k.y, x.val, g.y * st[4 * i4 + 1]);
                    st[4 * i4 + 2] = fmaf(k.z, x.val, g.z * st[4 * i4 + 2]); st[4 * i4 + 3] = fmaf(k.w, x.val, g.w * st[4 * i4 + 3]);
                }
                o = fmaf(x.sc.x, x.val, rows_sum<RG>((acc[0] + acc[1]) + (acc[2] + acc[3])));
            } else if (MODE == 3) {
                float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int i4 = 0; i4 < RS / 4; i4++) {
                    const float4 k = x.v0[i4], q = x.v1[i4], g = x.v2[i4];
                    st[4 * i4 + 0] = fmaf(k.x, x.val, g.x * st[4 * i4 + 0]); st[4 * i4 + 1] = fmaf(k.y, x.val, g.y * st[4 * i4 + 1]);
                    st[4 * i4 + 2] = fmaf(k.z, x.val, g.z * st[4 * i4 + 2]); st[4 * i4 + 3] = fmaf(k.w, x.val, g.w * st[4 * i4 + 3]);
                    acc[0] = fmaf(st[4 * i4 + 0], q.x, acc[0]); acc[1] = fmaf(st[4 * i4 + 1], q.y, acc[1]);
                    acc[2] = fmaf(st[4 * i4 + 2], q.z, acc[2]); acc[3] = fmaf(st[4 * i4 + 3], q.w, acc[3]);
                }
                o = rows_sum<RG>((acc[0] + acc[1]) + (acc[2] + acc[3]));
            } else {
                const float keep = x.sc.x, pv = x.sc.y * x.val;                 // put v | dt x
                float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int i4 = 0; i4 < RS / 4; i4++) {
                    const float4 k = x.v0[i4], q = x.v1[i4];
                    st[4 * i4 + 0] = fmaf(k.x, pv, keep * st[4 * i4 + 0]); st[4 * i4 + 1] = fmaf(k.y, pv, keep * st[4 * i4 + 1]);
                    st[4 * i4 + 2] = fmaf(k.z, pv, keep * st[4 * i4 + 2]); st[4 * i4 + 3] = fmaf(k.w, pv, keep * st[4 * i4 + 3]);
                    acc[0] = fmaf(st[4 * i4 + 0], q.x, acc[0]); acc[1] = fmaf(st[4 * i4 + 1], q.y, acc[1]);
                    acc[2] = fmaf(st[4 * i4 + 2], q.z, acc[2]); acc[3] = fmaf(st[4 * i4 + 3], q.w, acc[3]);
                }
                o = rows_sum<RG>((acc[0] + acc[1]) + (acc[2] + acc[3]));
                if (MODE == 2) o = fmaf(skip, x.val, o);
            }
            if (live && r == 0) {
                const int t = t0 + tt;
                if (j < V) __stcs(p.out + (size_t)t * H * V + h * V + j, o);
                else p.gates[((size_t)t * H + h) * 4 + 3] = o;
            }
        };
        TokenRegs<RS / 4> A, B;
        fetch(0, A);
        int tt = 0;
        for (; tt + 1 < n; tt += 2) {
            fetch(tt + 1, B);
            step(tt, A);
            if (tt + 2 < n) fetch(tt + 2, A);
            step(tt + 1, B);
        }
        if (tt < n) step(tt, A);
        if (more) prepare(t0 + CT, chunks + (cur ^ 1) * CT * TOK);
        __syncthreads();
    }
    regs_store<RS, RG>(st, tile, S, D, V, col0, extra);
}

inline int rows_per_thread(int D) { return D <= 32 ? 4 : (D <= 64 ? 8 : (D <= 128 ? 16 : (D <= 256 ? 32 : 0))); }
inline bool regs_kernels_on() {
    static int on = -1;
    if (on < 0) { const char* e = getenv("EMBER_SCAN_IN_REGISTERS"); on = (e && e[0] == '0') ? 0 : 1; }
    return on != 0;
}

template <int MODE, int RS, int CT, int RG>
inline int launch_scan_ct(const ScanArgs& p, int S, int n_cols, cudaStream_t st) {
    constexpr int NV = (MODE == 0 || MODE == 3 || MODE == 4) ? 3 : 2;
    const size_t smem = ((size_t)RG * RS * 33 + 2 * CT * (NV * RG * (RS + 4) + 4 + RCOLS)) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(scan_chunks_kernel<MODE, RS, CT, RG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail("scan: %s", cudaGetErrorString(e));
    }
    launch_kernel(scan_chunks_kernel<MODE, RS, CT, RG>, dim3(S, p.H, (n_cols + RCOLS - 1) / RCOLS), 32 * RG, smem, st, p);
    return 0;
}
// `single`: every run of the step is one token (a decode step): chunks of one token, small blocks, several per SM
// (the step is bound by the state's bytes).  Eight lanes a column in both cases: sixteen (half the rows a thread, one
// more shuffle) were measured equal for prompt portions (6.49 against 6.34 ms for the eight scans of a 2,048-token
// step at heads of 128), so the kernel keeps the parameter and the launcher one choice.
template <int MODE>
inline int launch_scan(const ScanArgs& p, int S, int n_cols, bool single, cudaStream_t st) {
    switch (rows_per_thread(p.D)) {
        case 4: return single ? launch_scan_ct<MODE, 4, 1, 8>(p, S, n_cols, st) : launch_scan_ct<MODE, 4, 16, 8>(p, S, n_cols, st);
        case 8: return single ? launch_scan_ct<MODE, 8, 1, 8>(p, S, n_cols, st) : launch_scan_ct<MODE, 8, 16, 8>(p, S, n_cols, st);
        case 16: return single ? launch_scan_ct<MODE, 16, 1, 8>(p, S, n_cols, st) : launch_scan_ct<MODE, 16, 16, 8>(p, S, n_cols, st);
        default: return single ? launch_scan_ct<MODE, 32, 1, 8>(p, S, n_cols, st) : launch_scan_ct<MODE, 32, 8, 8>(p, S, n_cols, st);
    }
}

// Columns per block: whole warps, at most 128, fewer while the state tile would not fit in shared memory.
inline int pick_columns(int D, int V, int extra_floats, size_t* smem) {
    int warps = (V + 31) / 32;
    if (warps > 4) warps = 4;
    while (warps > 1 && ((size_t)D * warps * 32 + extra_floats) * sizeof(float) > 96 * 1024) warps--;
    *smem = ((size_t)D * warps * 32 + extra_floats) * sizeof(float);
    return warps * 32;
}

template <typename K>
inline int allow_smem(K kernel, size_t smem, const char* what) {
    if (smem > 200 * 1024) return fail("%s: a state tile of %zu bytes does not fit in shared memory", what, smem);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail("%s: %s", what, cudaGetErrorString(e));
    }
    return 0;
}

}  // namespace ember

using namespace ember;

EMBER_API int ember_conv_silu(const float* x, int ldx, int c0, const float* taps, const float* bias, int n, float* carry,
                              long long carry_stride, const int* seq_of, const int* query_start, const int* slots, float* out,
                              int T, int S, int C, int silu, void* stream) {
    if (T <= 0 || S <= 0) return 0;
    if (C <= 0 || n < 1 || n > 64 || ldx < c0 + C) return fail("conv_silu: %d channels from column %d in rows of %d, %d taps", C, c0, ldx, n);
    if (T > 65535 || S > 65535) return fail("conv_silu: %d tokens in %d runs are too many for one launch", T, S);
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned bx = (unsigned)((C + 127) / 128);
    const int tt = T >= 1024 ? 8 : 1;          // prompt portions: eight tokens a block; small steps keep a block a token
    launch_kernel(conv_silu_kernel, dim3(bx, (T + tt - 1) / tt), 128, 0, st, x, ldx, c0, taps, bias, n, (const float*)carry,
                  carry_stride, seq_of, query_start, slots, out, C, silu, T, tt);
    if (n > 1)
        launch_kernel(conv_carry_kernel, dim3(bx, S), 128, 0, st, x, ldx, c0, n, carry, carry_stride, query_start, slots, C);
    return check_launch("conv_silu");
}

EMBER_API int ember_delta_scan(const float* conv, int ld_conv, const float* beta, int ld_beta, const float* a, int ld_a,
                               const float* dt_bias, const float* A_log, float* state, long long state_stride, float* out,
                               const int* query_start, const int* slots, int T, int S, int H, int G, int D, int V, float key_eps,
                               int a_head, void* stream) {
    if (S <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || V <= 0) return fail("delta_scan: %d/%d heads of %d x %d", H, G, D, V);
    if (S > 65535 || H > 65535) return fail("delta_scan: too many runs or heads for one launch");
    size_t smem;
    const int VT = pick_columns(D, V, 6 * D + 128, &smem);
    if (allow_smem(delta_scan_kernel, smem, "delta_scan")) return 1;
    DeltaArgs p{conv, ld_conv, beta, ld_beta, a, ld_a, dt_bias, A_log, state, state_stride, out, query_start, slots, H, G, D, V, key_eps, a_head};
    if (rows_per_thread(D) && regs_kernels_on()) {
        ScanArgs q{};
        q.state = state; q.state_stride = state_stride; q.out = out; q.query_start = query_start; q.slots = slots;
        q.H = H; q.G = G; q.D = D; q.V = V; q.x = conv; q.ld_x = ld_conv; q.b = beta; q.ld_b = ld_beta; q.a = a; q.ld_a = ld_a;
        q.dt_bias = dt_bias; q.A_log = A_log; q.key_eps = key_eps; q.a_head = a_head;
        if (launch_scan<0>(q, S, V, T == S, (cudaStream_t)stream)) return 1;
        return check_launch("delta_scan");
    }
    launch_kernel(delta_scan_kernel, dim3(S, H, (V + VT - 1) / VT), VT, smem, (cudaStream_t)stream, p);
    return check_launch("delta_scan");
}

EMBER_API int ember_memory_scan(const float* proj, int ld, int off_q, int off_k, int off_v, int off_i, int off_f,
                                const float* bias_i, const float* bias_f, float cap, float* state, long long state_stride,
                                float* gates, float* out, const int* query_start, const int* slots, int T, int S, int H, int D, int V,
                                void* stream) {
    if (S <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0 || !(cap > 0.0f)) return fail("memory_scan: %d heads of %d x %d, cap %g", H, D, V, cap);
    if (S > 65535 || H > 65535) return fail("memory_scan: too many runs or heads for one launch");
    cudaStream_t st = (cudaStream_t)stream;
    MemoryArgs p{proj, ld, off_q, off_k, off_v, off_i, off_f, bias_i, bias_f, cap, state, state_stride, gates, out, query_start, slots, H, D, V};
    launch_kernel(memory_gates_kernel, dim3(S, H), 32, 0, st, p);
    if (rows_per_thread(D) && regs_kernels_on()) {
        ScanArgs q{};
        q.state = state; q.state_stride = state_stride; q.out = out; q.query_start = query_start; q.slots = slots;
        q.H = H; q.G = H; q.D = D; q.V = V; q.x = proj; q.ld_x = ld; q.off_q = off_q; q.off_k = off_k; q.off_v = off_v; q.gates = gates;
        if (launch_scan<1>(q, S, V + 1, T == S, st)) return 1;
        return check_launch("memory_scan");
    }
    size_t smem;
    const int VT = pick_columns(D, V + 1, 4 * D, &smem);
    if (allow_smem(memory_scan_kernel, smem, "memory_scan")) return 1;
    launch_kernel(memory_scan_kernel, dim3(S, H, (V + 1 + VT - 1) / VT), VT, smem, st, p);
    return check_launch("memory_scan");
}

EMBER_API int ember_ssm_scan(const float* conv, int ld_conv, const float* dt, int ld_dt, const float* dt_bias, const float* A_log,
                             const float* skip, float* state, long long state_stride, float* out, const int* query_start,
                             const int* slots, int T, int S, int H, int G, int N, int V, void* stream) {
    if (S <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || N <= 0 || V <= 0) return fail("ssm_scan: %d heads in %d groups, state %d x %d", H, G, N, V);
    if (S > 65535 || H > 65535) return fail("ssm_scan: too many runs or heads for one launch");
    size_t smem;
    const int VT = pick_columns(N, V, 4 * N, &smem);
    if (allow_smem(ssm_scan_kernel, smem, "ssm_scan")) return 1;
    SsmArgs p{conv, ld_conv, dt, ld_dt, dt_bias, A_log, skip, state, state_stride, out, query_start, slots, H, G, N, V};
    if (rows_per_thread(N) && regs_kernels_on()) {
        ScanArgs q{};
        q.state = state; q.state_stride = state_stride; q.out = out; q.query_start = query_start; q.slots = slots;
        q.H = H; q.G = G; q.D = N; q.V = V; q.x = conv; q.ld_x = ld_conv; q.b = dt; q.ld_b = ld_dt; q.dt_bias = dt_bias;
        q.A_log = A_log; q.skip = skip;
        if (launch_scan<2>(q, S, V, T == S, (cudaStream_t)stream)) return 1;
        return check_launch("ssm_scan");
    }
    launch_kernel(ssm_scan_kernel, dim3(S, H, (V + VT - 1) / VT), VT, smem, (cudaStream_t)stream, p);
    return check_launch("ssm_scan");
}

EMBER_API int ember_gla_scan(const float* proj, int ld, int off_q, int off_k, int off_v, const float* z, int ld_z, const float* z_bias,
                             float decay_power, float* state, long long state_stride, float* out, const int* query_start,
                             const int* slots, int T, int S, int H, int D, int V, void* stream) {
    if (S <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0 || !(decay_power > 0.0f)) return fail("gla_scan: %d heads of %d x %d, decay power %g", H, D, V, decay_power);
    if (S > 65535 || H > 65535) return fail("gla_scan: too many runs or heads for one launch");
    cudaStream_t st = (cudaStream_t)stream;
    if (rows_per_thread(D) && regs_kernels_on()) {
        ScanArgs q{};
        q.state = state; q.state_stride = state_stride; q.out = out; q.query_start = query_start; q.slots = slots;
        q.H = H; q.G = H; q.D = D; q.V = V; q.x = proj; q.ld_x = ld; q.off_q = off_q; q.off_k = off_k; q.off_v = off_v;
        q.a = z; q.ld_a = ld_z; q.dt_bias = z_bias; q.decay_power = decay_power;
        if (launch_scan<3>(q, S, V, T == S, st)) return 1;
        return check_launch("gla_scan");
    }
    size_t smem;
    const int VT = pick_columns(D, V, 6 * D, &smem);
    if (allow_smem(gla_scan_kernel, smem, "gla_scan")) return 1;
    GlaArgs p{proj, ld, off_q, off_k, off_v, z, ld_z, z_bias, decay_power, state, state_stride, out, query_start, slots, H, D, V};
    launch_kernel(gla_scan_kernel, dim3(S, H, (V + VT - 1) / VT), VT, smem, st, p);
    return check_launch("gla_scan");
}

EMBER_API int ember_token_shift(const void* x, int x_dtype, const float* mu, int n_mix, float* carry, long long carry_stride,
                                const int* seq_of, const int* query_start, const int* slots, void* out, int out_dtype,
                                long long mix_stride, int T, int S, int C, void* stream) {
    if (T <= 0 || S <= 0) return 0;
    if (C <= 0 || n_mix <= 0 || mix_stride < (long long)T * C) return fail("token_shift: %d blends of rows of %d, %lld apart", n_mix, C, mix_stride);
    if (T > 65535 || S > 65535) return fail("token_shift: %d tokens in %d runs are too many for one launch", T, S);
    if (x_dtype != out_dtype || (x_dtype != EMBER_F32 && x_dtype != EMBER_BF16)) return fail("token_shift: dtypes %d -> %d", x_dtype, out_dtype);
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned bx = (unsigned)((C + 127) / 128);
    const int pack = x_dtype == EMBER_F32 ? 4 : 8;
    const bool vec = C % pack == 0 && carry_stride % 4 == 0 && mix_stride % pack == 0 &&
                     ((((uintptr_t)x | (uintptr_t)out | (uintptr_t)mu | (uintptr_t)carry) & 15) == 0);
    const unsigned vx = (unsigned)((C / pack + 127) / 128);
    if (vec && x_dtype == EMBER_F32) {
        launch_kernel(token_shift_vec_kernel<float>, dim3(vx, T), 128, 0, st, (const float*)x, C, mu, n_mix, (const float*)carry,
                      carry_stride, seq_of, query_start, slots, (float*)out, (size_t)mix_stride);
        launch_kernel(token_carry_kernel<float>, dim3(bx, S), 128, 0, st, (const float*)x, C, carry, carry_stride, query_start, slots);
    } else if (vec) {
        launch_kernel(token_shift_vec_kernel<__nv_bfloat16>, dim3(vx, T), 128, 0, st, (const __nv_bfloat16*)x, C, mu, n_mix,
                      (const float*)carry, carry_stride, seq_of, query_start, slots, (__nv_bfloat16*)out, (size_t)mix_stride);
        launch_kernel(token_carry_kernel<__nv_bfloat16>, dim3(bx, S), 128, 0, st, (const __nv_bfloat16*)x, C, carry, carry_stride,
                      query_start, slots);
    } else if (x_dtype == EMBER_F32) {
        launch_kernel(token_shift_kernel<float, float>, dim3(bx, T), 128, 0, st, (const float*)x, C, mu, n_mix, (const float*)carry,
                      carry_stride, seq_of, query_start, slots, (float*)out, (size_t)mix_stride);
        launch_kernel(token_carry_kernel<float>, dim3(bx, S), 128, 0, st, (const float*)x, C, carry, carry_stride, query_start, slots);
    } else {
        launch_kernel(token_shift_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(bx, T), 128, 0, st, (const __nv_bfloat16*)x, C, mu, n_mix,
                      (const float*)carry, carry_stride, seq_of, query_start, slots, (__nv_bfloat16*)out, (size_t)mix_stride);
        launch_kernel(token_carry_kernel<__nv_bfloat16>, dim3(bx, S), 128, 0, st, (const __nv_bfloat16*)x, C, carry, carry_stride,
                      query_start, slots);
    }
    return check_launch("token_shift");
}

EMBER_API int ember_wkv_scan(const float* proj, int ld, long long off_r, long long off_k, long long off_v, const float* z, int ld_z,
                             const float* w0, const float* bonus, float* state, long long state_stride, float* out,
                             const int* query_start, const int* slots, int T, int S, int H, int D, int V, void* stream) {
    if (S <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0 || !w0 || !bonus) return fail("wkv_scan: %d heads of %d x %d", H, D, V);
    if (S > 65535 || H > 65535) return fail("wkv_scan: too many runs or heads for one launch");
    if (off_r > 0x7fffffffLL || off_k > 0x7fffffffLL || off_v > 0x7fffffffLL) return fail("wkv_scan: column offsets beyond 2^31");
    cudaStream_t st = (cudaStream_t)stream;
    if (rows_per_thread(D) && regs_kernels_on()) {
        ScanArgs q{};
        q.state = state; q.state_stride = state_stride; q.out = out; q.query_start = query_start; q.slots = slots;
        q.H = H; q.G = H; q.D = D; q.V = V; q.x = proj; q.ld_x = ld; q.off_q = (int)off_r; q.off_k = (int)off_k; q.off_v = (int)off_v;
        q.a = z; q.ld_a = ld_z; q.dt_bias = w0; q.bonus = bonus;
        if (launch_scan<4>(q, S, V, T == S, st)) return 1;
        return check_launch("wkv_scan");
    }
    size_t smem;
    const int VT = pick_columns(D, V, 8 * D, &smem);
    if (allow_smem(wkv_scan_kernel, smem, "wkv_scan")) return 1;
    WkvArgs p{proj, ld, (int)off_r, (int)off_k, (int)off_v, z, ld_z, w0, bonus, state, state_stride, out, query_start, slots, H, D, V};
    launch_kernel(wkv_scan_kernel, dim3(S, H, (V + VT - 1) / VT), VT, smem, st, p);
    return check_launch("wkv_scan");
}
