// Softmax attention with a sink over a paged cache, and what two mixers need around it:
//
//   * whole_norm_store:  q/k/v of a token with biases, one RMS norm over the whole query projection and one over the
//     whole key projection (all heads at once), queries out, keys [.., D] and values [.., DV] into their pages;
//   * latent_prepare:    a token's low-rank query latent (RMS norm) out, and its key/value latent (RMS norm) with the
//     rotated shared key part behind it into the token's single cache row [c | k_rot];
//   * rotate_pairs:      rotation of neighbouring pairs (2i, 2i + 1) of a slice of every head, fp32 in, cache type out;
//   * head_gemm:         out[t, h, :] = W[h] x[t, h, :] for every head (a product per head, weights [H, N, K]), with an
//     optional sigmoid gate on the result: folds a head's key up-projection into its query and takes a head's value
//     up-projection of the attended latent; fp32 multiply-adds in general, mma.sync tiles for bfloat16 weights;
//   * sink_attention:    o = sum_j w_j v_j with w = softmax over the visible keys and one more term exp(sink[h]) in the
//     denominator that has no key and no value; visible: j <= i and (no window, or i - j < window, or j < keep_first).
//     Keys have D elements, values DV; with no value pool a value is the first DV elements of the key row (the
//     latent serves as both).  Any number of query heads per key head.
//
// Scores, weights, norms, angles and sums are fp32.  Work unit of the attention: a tile of consecutive query tokens of
// one run x a chunk of the query heads of one key head x one split of the key range; splits have a fixed length
// anchored at key 0 and are merged in ascending order, so a token's result does not depend on the rest of the step.
#include "common.cuh"

EMBER_DEFINE_LAST_ERROR

namespace ember {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// ------------------------------------------------------------------------------------ q/k/v of a windowed layer
struct WholeNormArgs {
    const float* qkv; int ld;          // [T, q | k | v] fp32 (no bias yet)
    const float* bias;                 // [q | k | v] or null
    const float* q_w; const float* k_w;   // weights over the whole projection, or null (no norm)
    float eps;
    int H, G, D, DV;
    const int* positions; const int* seq_of; const int* block_table;
    int max_blocks, page, num_pages;
    void* q_out; void* k_pool; void* v_pool;
    int write_kv;
    int* err;
};

template <typename T>
__global__ void __launch_bounds__(256) whole_norm_store_kernel(WholeNormArgs p) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int QN = p.H * p.D, KN = p.G * p.D, VN = p.G * p.DV;
    const float* row = p.qkv + (size_t)t * p.ld;
    const float* b = p.bias;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < QN; i += blockDim.x) {
        const float v = row[i] + (b ? b[i] : 0.0f);
        ss = fmaf(v, v, ss);
    }
    const float rq = p.q_w ? 1.0f / sqrtf(block_sum(ss, scratch) / (float)QN + p.eps) : 1.0f;
    T* qo = (T*)p.q_out + (size_t)t * QN;
    for (int i = threadIdx.x; i < QN; i += blockDim.x) {
        const float v = row[i] + (b ? b[i] : 0.0f);
        qo[i] = from_float<T>(p.q_w ? v * rq * p.q_w[i] : v);
    }
    if (!p.write_kv) return;
    ss = 0.0f;
    for (int i = threadIdx.x; i < KN; i += blockDim.x) {
        const float v = row[QN + i] + (b ? b[QN + i] : 0.0f);
        ss = fmaf(v, v, ss);
    }
    const float rk = p.k_w ? 1.0f / sqrtf(block_sum(ss, scratch) / (float)KN + p.eps) : 1.0f;
    const int pos = p.positions[t], seq = p.seq_of[t];
    const int blk = p.block_table[(size_t)seq * p.max_blocks + pos / p.page];
    if (blk < 0 || blk >= p.num_pages) {
        if (threadIdx.x == 0 && p.err) atomicOr(p.err, EMBER_ERR_PAGE_RANGE);
        return;
    }
    const int in_page = pos % p.page;
    T* kp = (T*)p.k_pool;
    T* vp = (T*)p.v_pool;
    for (int i = threadIdx.x; i < KN; i += blockDim.x) {
        const int g = i / p.D, d = i - g * p.D;
        const float v = row[QN + i] + (b ? b[QN + i] : 0.0f);
        kp[(((size_t)blk * p.G + g) * p.page + in_page) * p.D + d] = from_float<T>(p.k_w ? v * rk * p.k_w[i] : v);
    }
    for (int i = threadIdx.x; i < VN; i += blockDim.x) {
        const int g = i / p.DV, d = i - g * p.DV;
        const float v = row[QN + KN + i] + (b ? b[QN + KN + i] : 0.0f);
        vp[(((size_t)blk * p.G + g) * p.page + in_page) * p.DV + d] = from_float<T>(v);
    }
}

// --------------------------------------------------------------- q/k/v of a token: norm, rotation, temperature
// The general form of whole_norm_store.  norm_mode 0: none; 1: one RMS norm over the whole query projection and one
// over the whole key projection (weights of that size); 2: an RMS norm per head (weights of D, shared by the heads).
// Then the first `rotary` elements of every query and key head turn (element i with i + rotary / 2) by the angle
// position * inv_freq[i], and the query is multiplied by 1 + qt_coef * ln(floor((position + 1) / qt_every) + 1)
// (qt_every 0: not).  Queries out, keys and values into the token's page.
struct HeadPrepareArgs {
    const float* qkv; int ld;          // [T, q | k | v] fp32
    const float* bias;                 // [q | k | v] or null
    int norm_mode; const float* q_w; const float* k_w; float eps;
    const float* inv_freq; int rotary;
    float qt_coef; int qt_every;
    int H, G, D, DV;
    const int* positions; const int* seq_of; const int* block_table;
    int max_blocks, page, num_pages;
    void* q_out; void* k_pool; void* v_pool;
    int write_kv;
    int* err;
};

template <typename T>
__global__ void __launch_bounds__(256) head_prepare_store_kernel(HeadPrepareArgs p) {
    extern __shared__ float factor[];          // per-head norm factors: H for the queries, then G for the keys
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int D = p.D, QN = p.H * D, KN = p.G * D, VN = p.G * p.DV;
    const float* row = p.qkv + (size_t)t * p.ld;
    const float* b = p.bias;
    const bool kv = p.write_kv != 0;
    auto val = [&](int i) { return row[i] + (b ? b[i] : 0.0f); };
    float rq = 1.0f, rk = 1.0f;
    if (p.norm_mode == 1) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < QN; i += blockDim.x) { const float v = val(i); ss = fmaf(v, v, ss); }
        rq = 1.0f / sqrtf(block_sum(ss, scratch) / (float)QN + p.eps);
        if (kv) {
            ss = 0.0f;
            for (int i = threadIdx.x; i < KN; i += blockDim.x) { const float v = val(QN + i); ss = fmaf(v, v, ss); }
            rk = 1.0f / sqrtf(block_sum(ss, scratch) / (float)KN + p.eps);
        }
    } else if (p.norm_mode == 2) {
        const int heads = p.H + (kv ? p.G : 0);
        for (int h = warp; h < heads; h += nw) {
            float ss = 0.0f;
            for (int d = lane; d < D; d += 32) { const float v = val(h * D + d); ss = fmaf(v, v, ss); }
            ss = warp_sum(ss);
            if (lane == 0) factor[h] = 1.0f / sqrtf(ss / (float)D + p.eps);
        }
        __syncthreads();
    }
    const int pos = p.positions[t];
    const int half = p.rotary / 2;
    // element i of [q | k] (i < QN: a query element), normed and weighed
    auto normed = [&](int i) {
        const bool isq = i < QN;
        const int j = isq ? i : i - QN;
        float v = val(i);
        if (p.norm_mode == 1) v *= (isq ? rq : rk) * (isq ? p.q_w[j] : p.k_w[j]);
        else if (p.norm_mode == 2) v *= factor[i / D] * (isq ? p.q_w[j % D] : p.k_w[j % D]);
        return v;
    };
    // element i of [q | k] after the rotation, handed to write(index, value); a rotated pair (i, i + half) is made by the
    // thread that holds its first element, from one sine and one cosine
    auto emit = [&](int i, float mul, auto&& write) {
        const int d = i % D;
        if (d >= half && d < p.rotary) return;
        const float v = normed(i);
        if (d < half) {
            const float other = normed(i + half);
            float sn, cs;
            sincosf((float)pos * p.inv_freq[d], &sn, &cs);
            write(i, (v * cs - other * sn) * mul);
            write(i + half, (other * cs + v * sn) * mul);
        } else {
            write(i, v * mul);
        }
    };
    float temp = 1.0f;
    if (p.qt_every > 0) temp = 1.0f + p.qt_coef * logf((float)((pos + 1) / p.qt_every) + 1.0f);
    T* qo = (T*)p.q_out + (size_t)t * QN;
    for (int i = threadIdx.x; i < QN; i += blockDim.x) emit(i, temp, [&](int j, float v) { qo[j] = from_float<T>(v); });
    if (!kv) return;
    const int seq = p.seq_of[t];
    const int blk = p.block_table[(size_t)seq * p.max_blocks + pos / p.page];
    if (blk < 0 || blk >= p.num_pages) {
        if (threadIdx.x == 0 && p.err) atomicOr(p.err, EMBER_ERR_PAGE_RANGE);
        return;
    }
    const int in_page = pos % p.page;
    T* kp = (T*)p.k_pool;
    T* vp = (T*)p.v_pool;
    for (int i = threadIdx.x; i < KN; i += blockDim.x)
        emit(QN + i, 1.0f, [&](int j, float v) {
            const int g = (j - QN) / D, d = (j - QN) - g * D;
            kp[(((size_t)blk * p.G + g) * p.page + in_page) * D + d] = from_float<T>(v);
        });
    for (int i = threadIdx.x; i < VN; i += blockDim.x) {
        const int g = i / p.DV, d = i - g * p.DV;
        vp[(((size_t)blk * p.G + g) * p.page + in_page) * p.DV + d] = from_float<T>(val(QN + KN + i));
    }
}

// x[t, h, :] *= sigmoid(gate[t, h]) for an attention result x [T, H, DV]: the gate per head as a pass of its own, behind
// attention kernels that do not take it.
template <typename T>
__global__ void head_gate_apply_kernel(T* __restrict__ x, const float* __restrict__ gate, int ld_gate, int H, int DV, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t th = i / DV;
    x[i] = from_float<T>(to_float(x[i]) * sigmoidf_(gate[(th / H) * (size_t)ld_gate + th % H]));
}

// ------------------------------------------------------------------------------------- latents of a token
struct LatentArgs {
    const float* a; int ld;            // [T, ...] fp32: the fused down-projections
    int q_col, q_rank;                 // query latent (q_rank 0: none)
    int c_col, kv_rank, rot_dim;       // key/value latent and, behind it, the shared key part to rotate
    const float* q_w; const float* c_w;
    float eps;
    const float* inv_freq; int rotary; // rotary <= rot_dim elements are rotated, in neighbouring pairs or (half_layout) i with i + rotary / 2
    int half_layout; float magnitude;  // cosines and sines are multiplied by magnitude
    const int* positions; const int* seq_of; const int* block_table;
    int max_blocks, page, num_pages;
    void* cq_out;                      // [T, q_rank]
    void* pool;                        // [pages, 1, page, kv_rank + rot_dim]
    int write_kv;
    int* err;
};

template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(LatentArgs p) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const float* row = p.a + (size_t)t * p.ld;
    if (p.q_rank > 0) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x) ss = fmaf(row[p.q_col + i], row[p.q_col + i], ss);
        const float r = 1.0f / sqrtf(block_sum(ss, scratch) / (float)p.q_rank + p.eps);
        T* o = (T*)p.cq_out + (size_t)t * p.q_rank;
        for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x) o[i] = from_float<T>(row[p.q_col + i] * r * p.q_w[i]);
    }
    if (!p.write_kv) return;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < p.kv_rank; i += blockDim.x) ss = fmaf(row[p.c_col + i], row[p.c_col + i], ss);
    const float r = 1.0f / sqrtf(block_sum(ss, scratch) / (float)p.kv_rank + p.eps);
    const int pos = p.positions[t], seq = p.seq_of[t];
    const int blk = p.block_table[(size_t)seq * p.max_blocks + pos / p.page];
    if (blk < 0 || blk >= p.num_pages) {
        if (threadIdx.x == 0 && p.err) atomicOr(p.err, EMBER_ERR_PAGE_RANGE);
        return;
    }
    const int W = p.kv_rank + p.rot_dim;
    T* dst = (T*)p.pool + ((size_t)blk * p.page + pos % p.page) * W;
    for (int i = threadIdx.x; i < p.kv_rank; i += blockDim.x) dst[i] = from_float<T>(row[p.c_col + i] * r * p.c_w[i]);
    const float* kr = row + p.c_col + p.kv_rank;
    // pair i of the rotation: elements (2i, 2i + 1), or (i, i + rotary / 2) in the half layout
    for (int i = threadIdx.x; i < p.rotary / 2; i += blockDim.x) {
        const int a = p.half_layout ? i : 2 * i, c = p.half_layout ? i + p.rotary / 2 : 2 * i + 1;
        float sn, cs;
        sincosf((float)pos * p.inv_freq[i], &sn, &cs);
        sn *= p.magnitude; cs *= p.magnitude;
        const float u = kr[a], v = kr[c];
        dst[p.kv_rank + a] = from_float<T>(u * cs - v * sn);
        dst[p.kv_rank + c] = from_float<T>(v * cs + u * sn);
    }
    for (int i = p.rotary + threadIdx.x; i < p.rot_dim; i += blockDim.x) dst[p.kv_rank + i] = from_float<T>(kr[i]);
}

// out[t, h, out_col + i] = rotated in[t, h, in_col + i], i < width; below `rotary`, pairs (2i, 2i + 1) or, in the half
// layout, (i, i + rotary / 2) turn by float(position) * inv_freq[i], cosine and sine times `magnitude`.
template <typename T>
__global__ void rotate_pairs_kernel(const float* __restrict__ in, int ld_in, int in_head, int in_col, T* __restrict__ out,
                                    int ld_out, int out_head, int out_col, int H, int width, int rotary,
                                    const float* __restrict__ inv_freq, const int* __restrict__ positions, int half_layout,
                                    float magnitude) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pairs = rotary / 2, units = pairs + (width - rotary);       // a unit: one pair, or one element that passes
    const float pos = (float)positions[t];
    for (int idx = threadIdx.x; idx < H * units; idx += blockDim.x) {
        const int h = idx / units, i = idx - h * units;
        const float* src = in + (size_t)t * ld_in + (size_t)h * in_head + in_col;
        T* dst = out + (size_t)t * ld_out + (size_t)h * out_head + out_col;
        if (i < pairs) {
            const int a = half_layout ? i : 2 * i, c = half_layout ? i + pairs : 2 * i + 1;
            float sn, cs;
            sincosf(pos * inv_freq[i], &sn, &cs);
            sn *= magnitude; cs *= magnitude;
            const float u = src[a], v = src[c];
            dst[a] = from_float<T>(u * cs - v * sn);
            dst[c] = from_float<T>(v * cs + u * sn);
        } else {
            const int e = rotary + (i - pairs);
            dst[e] = from_float<T>(src[e]);
        }
    }
}

// ----------------------------------------------------------------------------------- a product per head
// out[t, h, n] = sum_k x[t, h, k] w[h, n, k], optionally times sigmoid(gate[t, h, n]).  Tiles of 32 tokens x 64
// outputs, K in steps of 16; k ascends for every output, so a row's result does not depend on the rest of the step.
constexpr int HG_BM = 32, HG_BN = 64, HG_BK = 16;

struct HeadGemmArgs {
    const float* x; int ld_x, x_head, x_col;
    const void* w;                       // [H, N, K]
    void* out; int ld_o, o_head, o_col;
    const float* gate; int ld_g, g_col;  // gate[t, g_col + h N + n] or null
    int T, H, N, K;
};

template <typename TW, typename TO>
__global__ void __launch_bounds__(256) head_gemm_kernel(HeadGemmArgs p) {
    __shared__ float As[HG_BK][HG_BM + 1];
    __shared__ float Bs[HG_BK][HG_BN + 1];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.z, m0 = blockIdx.x * HG_BM, n0 = blockIdx.y * HG_BN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // 16 x 16: outputs (ty * 2 + i, tx * 4 + j)
    const TW* w = (const TW*)p.w + (size_t)h * p.N * p.K;
    float acc[2][4] = {};
    for (int k0 = 0; k0 < p.K; k0 += HG_BK) {
        for (int idx = threadIdx.x; idx < HG_BM * HG_BK; idx += 256) {
            const int r = idx / HG_BK, k = idx - r * HG_BK;
            const int t = m0 + r;
            As[k][r] = (t < p.T && k0 + k < p.K) ? p.x[(size_t)t * p.ld_x + (size_t)h * p.x_head + p.x_col + k0 + k] : 0.0f;
        }
        for (int idx = threadIdx.x; idx < HG_BN * HG_BK; idx += 256) {
            const int r = idx / HG_BK, k = idx - r * HG_BK;
            const int n = n0 + r;
            Bs[k][r] = (n < p.N && k0 + k < p.K) ? to_float(w[(size_t)n * p.K + k0 + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < HG_BK; k++) {
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
        const int t = m0 + ty * 2 + i;
        if (t >= p.T) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= p.N) continue;
            float v = acc[i][j];
            if (p.gate) v *= sigmoidf_(p.gate[(size_t)t * p.ld_g + p.g_col + (size_t)h * p.N + n]);
            ((TO*)p.out)[(size_t)t * p.ld_o + (size_t)h * p.o_head + p.o_col + n] = from_float<TO>(v);
        }
    }
}

inline bool head_gemm_on_tensor_cores() {
    static int on = -1;
    if (on < 0) { const char* e = getenv("EMBER_HEAD_GEMM_TC"); on = (e && e[0] == '0') ? 0 : 1; }
    return on != 0;
}

// ----------------------------------------------------------------------------------------------- attention
constexpr int SA_WARPS = 8;
constexpr int SA_ROWS_PER_WARP = 4;
constexpr int SA_MAX_ROWS = SA_WARPS * SA_ROWS_PER_WARP;   // (query, head) rows of a tile
constexpr int SA_KT = 32;                                    // keys per shared-memory tile

struct SinkAttnParams {
    const void* q;        // [T, H, D]
    const void* k_pool;   // [pages][G][page][D]
    const void* v_pool;   // [pages][G][page][DV], or null: a value is the first DV elements of the key row
    void* out;            // [T, H, DV]
    float* part_o;        // [T, H, n_splits, DV]   (n_splits > 1)
    float* part_ml;       // [T, H, n_splits, 2]
    const int* tiles;     // [n_tiles, 4] = (run, first token row, queries, position of the first query)
    const int* block_table;
    const float* sink;    // [H] or null
    int max_blocks, page, num_pages;
    int H, G, D, DV;
    int head_chunk;       // query heads of one key head a block takes (tile_q * head_chunk <= SA_MAX_ROWS)
    int window, keep_first;
    float scale;
    int n_splits, split_keys;
    int* err;
    int chunk;            // > 0: position i sees j only if i / chunk == j / chunk (chunks counted from position 0 of the sequence)
    float softcap;        // > 0: score <- softcap * tanh(score / softcap), after the scale
    const float* head_gate; int ld_gate;   // [T, ld_gate] logits, one per head: the head's output is multiplied by its sigmoid; or null
};

// First key a tile starting at position pos0 can see, and whether key `key` is visible from position qpos.
__device__ __forceinline__ int first_visible(const SinkAttnParams& p, int pos0) {
    int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    if (p.chunk > 0) lo = max(lo, pos0 - pos0 % p.chunk);
    return lo;
}
__device__ __forceinline__ bool key_visible(const SinkAttnParams& p, int key, int qpos) {
    return key <= qpos && (p.window <= 0 || qpos - key < p.window || key < p.keep_first) &&
           (p.chunk <= 0 || key >= qpos - qpos % p.chunk);
}
__device__ __forceinline__ float capped_score(const SinkAttnParams& p, float dot) {
    const float s = dot * p.scale;
    return p.softcap > 0.0f ? p.softcap * tanhf(s / p.softcap) : s;
}

template <typename T, typename TO, int NC>
__global__ void __launch_bounds__(SA_WARPS * 32)
sink_attention_kernel(SinkAttnParams p) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int D = p.D, DV = p.DV, DP = D + 1;
    const bool alias = p.v_pool == nullptr;
    float* Ks = smem;                                   // [KT][D + 1]
    float* Vs = alias ? Ks : Ks + SA_KT * DP;           // [KT][DV] (or the key rows themselves)
    const int vs_ld = alias ? DP : DV;
    float* Qs = alias ? Ks + SA_KT * DP : Vs + SA_KT * DV;   // [rows][D]

    const int group = p.H / p.G;
    const int chunks = (group + p.head_chunk - 1) / p.head_chunk;
    const int tile = blockIdx.x, kvh = blockIdx.y / chunks, hc = blockIdx.y - kvh * chunks, split = blockIdx.z;
    const int head0 = kvh * group + hc * p.head_chunk;
    const int nh = min(p.head_chunk, group - hc * p.head_chunk);
    const int seq = p.tiles[tile * 4 + 0], row0 = p.tiles[tile * 4 + 1], nq = p.tiles[tile * 4 + 2],
              pos0 = p.tiles[tile * 4 + 3];
    const int rows = nq * nh;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* q = (const T*)p.q;
    const T* kp = (const T*)p.k_pool;
    const T* vp = (const T*)p.v_pool;

    for (int idx = threadIdx.x; idx < rows * D; idx += blockDim.x) {
        const int r = idx / D, d = idx - r * D;
        const int qi = r / nh, g = r - qi * nh;
        Qs[r * D + d] = to_float(q[((size_t)(row0 + qi) * p.H + head0 + g) * D + d]);
    }

    // visible keys of the tile: [0, kept) and [lo, hi); with a split, their part inside the split
    int lo = first_visible(p, pos0);
    int hi = pos0 + nq;
    int kept = p.window > 0 ? min(p.keep_first, lo) : 0;
    int s_lo = 0, s_hi = hi;
    if (p.n_splits > 1) {
        s_lo = split * p.split_keys;
        s_hi = min(hi, (split + 1) * p.split_keys);
    }

    float m[SA_ROWS_PER_WARP], l[SA_ROWS_PER_WARP], acc[SA_ROWS_PER_WARP][NC];
#pragma unroll
    for (int i = 0; i < SA_ROWS_PER_WARP; i++) {
        m[i] = -INFINITY;
        l[i] = 0.0f;
#pragma unroll
        for (int c = 0; c < NC; c++) acc[i][c] = 0.0f;
    }

    const int* bt = p.block_table + (size_t)seq * p.max_blocks;
    const bool vec4 = (D & 3) == 0;                       // (query rows are read four elements at a time then)
    for (int part = 0; part < 2; part++) {
        const int a = max(part == 0 ? 0 : lo, s_lo), b = min(part == 0 ? kept : hi, s_hi);
        if (a >= b) continue;
        for (int k0 = a - (a % SA_KT); k0 < b; k0 += SA_KT) {
            __syncthreads();  // the previous tile is consumed (and the queries are written before the first use)
            // a warp fetches whole key rows: one block-table look-up per row, neighbouring lanes read neighbouring elements
            for (int j = warp; j < SA_KT; j += SA_WARPS) {
                const int key = k0 + j;
                const T* ksrc = nullptr;
                const T* vsrc = nullptr;
                if (key >= a && key < b) {
                    const int blk = bt[key / p.page];
                    if (blk >= 0 && blk < p.num_pages) {
                        const size_t row = ((size_t)blk * p.G + kvh) * p.page + (key % p.page);
                        ksrc = kp + row * D;
                        if (!alias) vsrc = vp + row * DV;
                    } else if (lane == 0 && p.err) {
                        atomicOr(p.err, EMBER_ERR_PAGE_RANGE);
                    }
                }
                float* kd = Ks + j * DP;
                for (int d = lane; d < D; d += 32) kd[d] = ksrc ? to_float(ksrc[d]) : 0.0f;
                if (!alias) {
                    float* vd = Vs + j * DV;
                    for (int d = lane; d < DV; d += 32) vd[d] = vsrc ? to_float(vsrc[d]) : 0.0f;
                }
            }
            __syncthreads();

            // the warp's rows together: a key element read from shared memory serves all of them
            float sc[SA_ROWS_PER_WARP];
            const int key = k0 + lane;
            const float* kr = Ks + lane * DP;
#pragma unroll
            for (int i = 0; i < SA_ROWS_PER_WARP; i++) sc[i] = 0.0f;
            if (vec4) {
                for (int d = 0; d < D; d += 4) {
                    const float k0v = kr[d], k1v = kr[d + 1], k2v = kr[d + 2], k3v = kr[d + 3];
#pragma unroll
                    for (int i = 0; i < SA_ROWS_PER_WARP; i++) {
                        const int r = warp + i * SA_WARPS;
                        if (r < rows) {   // uniform per warp
                            const float4 qv = *reinterpret_cast<const float4*>(Qs + r * D + d);
                            sc[i] = fmaf(qv.x, k0v, sc[i]); sc[i] = fmaf(qv.y, k1v, sc[i]);
                            sc[i] = fmaf(qv.z, k2v, sc[i]); sc[i] = fmaf(qv.w, k3v, sc[i]);
                        }
                    }
                }
            } else {
                for (int d = 0; d < D; d++) {
                    const float kv = kr[d];
#pragma unroll
                    for (int i = 0; i < SA_ROWS_PER_WARP; i++) {
                        const int r = warp + i * SA_WARPS;
                        if (r < rows) sc[i] = fmaf(Qs[r * D + d], kv, sc[i]);
                    }
                }
            }
            float pj[SA_ROWS_PER_WARP];
            bool any = false;
#pragma unroll
            for (int i = 0; i < SA_ROWS_PER_WARP; i++) {
                const int r = warp + i * SA_WARPS;
                pj[i] = 0.0f;
                if (r >= rows) continue;  // uniform per warp
                const int qpos = pos0 + r / nh;
                const bool visible = key >= a && key < b && key_visible(p, key, qpos);
                const float sv = visible ? capped_score(p, sc[i]) : -INFINITY;
                const float m_new = fmaxf(m[i], warp_max(sv));
                if (m_new == -INFINITY) continue;  // nothing visible so far (uniform per warp)
                const float corr = expf(m[i] - m_new);
                pj[i] = visible ? expf(sv - m_new) : 0.0f;
                l[i] = l[i] * corr + warp_sum(pj[i]);
                m[i] = m_new;
                any = true;
#pragma unroll
                for (int c = 0; c < NC; c++) acc[i][c] *= corr;
            }
            if (any) {
                for (int jj = 0; jj < SA_KT; jj++) {
                    float w[SA_ROWS_PER_WARP];
#pragma unroll
                    for (int i = 0; i < SA_ROWS_PER_WARP; i++) w[i] = __shfl_sync(0xffffffffu, pj[i], jj);
                    const float* vr = Vs + jj * vs_ld;
#pragma unroll
                    for (int c = 0; c < NC; c++) {
                        const int d = lane + 32 * c;
                        if (d < DV) {
                            const float vv = vr[d];
#pragma unroll
                            for (int i = 0; i < SA_ROWS_PER_WARP; i++) acc[i][c] = fmaf(w[i], vv, acc[i][c]);
                        }
                    }
                }
            }
        }
    }

#pragma unroll
    for (int i = 0; i < SA_ROWS_PER_WARP; i++) {
        const int r = warp + i * SA_WARPS;
        if (r >= rows) continue;
        const int qi = r / nh, g = r - qi * nh;
        const int head = head0 + g;
        const size_t th = (size_t)(row0 + qi) * p.H + head;
        if (p.n_splits <= 1) {
            // the sink joins the denominator once: it has no key and no value
            float mm = m[i], ll = l[i], corr = 1.0f;
            if (p.sink) {
                const float sk = p.sink[head];
                mm = fmaxf(m[i], sk);
                corr = expf(m[i] - mm);
                ll = l[i] * corr + expf(sk - mm);
            }
            float inv = ll > 0.0f ? corr / ll : 0.0f;
            if (p.head_gate) inv *= sigmoidf_(p.head_gate[(size_t)(row0 + qi) * p.ld_gate + head]);
            TO* o = (TO*)p.out + th * DV;
#pragma unroll
            for (int c = 0; c < NC; c++) {
                const int d = lane + 32 * c;
                if (d < DV) o[d] = from_float<TO>(acc[i][c] * inv);
            }
        } else {
            float* po = p.part_o + (th * p.n_splits + split) * DV;
#pragma unroll
            for (int c = 0; c < NC; c++) {
                const int d = lane + 32 * c;
                if (d < DV) po[d] = acc[i][c];
            }
            if (lane == 0) {
                float* ml = p.part_ml + (th * p.n_splits + split) * 2;
                ml[0] = m[i];
                ml[1] = l[i];
            }
        }
    }
}

// Merges the splits of one (token, head) in ascending order; the sink joins here.
template <typename TO>
__global__ void sink_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const float* __restrict__ sink, TO* __restrict__ out, int n_splits, int DV, int H,
                                    const float* __restrict__ head_gate, int ld_gate) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t th = blockIdx.x;
    const float* ml = part_ml + th * n_splits * 2;
    float M = sink ? sink[th % H] : -INFINITY;
    for (int s = 0; s < n_splits; s++) M = fmaxf(M, ml[2 * s]);
    float L = sink ? expf(sink[th % H] - M) : 0.0f;
    for (int s = 0; s < n_splits; s++) {
        const float ms = ml[2 * s];
        if (ms != -INFINITY) L += ml[2 * s + 1] * expf(ms - M);
    }
    float inv = L > 0.0f ? 1.0f / L : 0.0f;
    if (head_gate) inv *= sigmoidf_(head_gate[(th / H) * (size_t)ld_gate + th % H]);
    for (int d = threadIdx.x; d < DV; d += blockDim.x) {
        float o = 0.0f;
        for (int s = 0; s < n_splits; s++) {
            const float ms = ml[2 * s];
            if (ms != -INFINITY) o = fmaf(part_o[(th * n_splits + s) * DV + d], expf(ms - M), o);
        }
        out[th * DV + d] = from_float<TO>(o * inv);
    }
}

template <typename T, typename TO>
int launch_sink_attention(const SinkAttnParams& p, int n_tiles, int T_tokens, cudaStream_t st) {
    const int D = p.D, DV = p.DV;
    const bool alias = p.v_pool == nullptr;
    const size_t smem = ((size_t)SA_KT * (D + 1) + (alias ? 0 : (size_t)SA_KT * DV) + (size_t)SA_MAX_ROWS * D) * sizeof(float);
    if (smem > 220 * 1024) return fail("sink_attention: heads of %d / %d need %zu bytes of shared memory", D, DV, smem);
    const int group = p.H / p.G, chunks = (group + p.head_chunk - 1) / p.head_chunk;
    dim3 grid(n_tiles, p.G * chunks, p.n_splits);
    const int nc = (DV + 31) / 32;
    auto run = [&](auto kernel) -> int {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return fail("sink_attention: shared memory %zu: %s", smem, cudaGetErrorString(e));
        }
        launch_kernel(kernel, grid, SA_WARPS * 32, smem, st, p);
        return check_launch("sink_attention");
    };
    int rc;
    if (nc <= 1) rc = run(sink_attention_kernel<T, TO, 1>);
    else if (nc <= 2) rc = run(sink_attention_kernel<T, TO, 2>);
    else if (nc <= 4) rc = run(sink_attention_kernel<T, TO, 4>);
    else if (nc <= 8) rc = run(sink_attention_kernel<T, TO, 8>);
    else rc = run(sink_attention_kernel<T, TO, 16>);
    if (rc) return rc;
    if (p.n_splits > 1) {
        launch_kernel(sink_combine_kernel<TO>, (unsigned)((size_t)T_tokens * p.H), DV >= 128 ? 128 : 64, 0, st,
                      (const float*)p.part_o, (const float*)p.part_ml, p.sink, (TO*)p.out, p.n_splits, DV, p.H, p.head_gate, p.ld_gate);
        return check_launch("sink_combine");
    }
    return 0;
}


// ------------------------------------------------- attention over shared key rows on the tensor cores (bfloat16)
// Keys and values from their pools, or (no value pool) one cached row that serves every query head as key and, with
// its first DV elements, as value.  A block takes 64 (query, head) rows and walks the visible keys 32 at a time: scores
// S = Q K^T and O += P V on mma.sync m16n8k16 (bf16 operands, fp32 accumulators), the softmax with its running maximum,
// denominators and the sink in fp32 registers.  Eight warps: warp (wr, wc) owns rows 16 wr .. 16 wr + 15 and the
// half wc of the value columns; both warps of a row slab compute the slab's scores (the same numbers), so no
// exchange is needed.  P enters the second product rounded to bfloat16, as V is.  Key tiles arrive by cp.async into
// two buffers, one tile ahead; with key splits a block leaves partial sums for the merge kernel, like the general form.
constexpr int LT_ROWS = 64, LT_KT = 32, LT_PAD = 8;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// The per-head product on the tensor cores: tiles of 64 tokens x 64 outputs, K in steps of 32, four warps of 16 rows; x is
// rounded to bfloat16 as it enters shared memory (the weights are bfloat16), sums are fp32.
constexpr int HT_BM = 64, HT_BN = 64, HT_BK = 32, HT_LD = HT_BK + 8;

template <typename TO>
__global__ void __launch_bounds__(128) head_gemm_tc_kernel(HeadGemmArgs p) {
    __shared__ __align__(16) __nv_bfloat16 As[HT_BM * HT_LD];
    __shared__ __align__(16) __nv_bfloat16 Bs[HT_BN * HT_LD];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.z, m0 = blockIdx.x * HT_BM, n0 = blockIdx.y * HT_BN;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const __nv_bfloat16* w = (const __nv_bfloat16*)p.w + (size_t)h * p.N * p.K;
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++) { acc[i][0] = 0.0f; acc[i][1] = 0.0f; acc[i][2] = 0.0f; acc[i][3] = 0.0f; }
    for (int k0 = 0; k0 < p.K; k0 += HT_BK) {
        for (int idx = threadIdx.x; idx < HT_BM * (HT_BK / 4); idx += 128) {
            const int r = idx / (HT_BK / 4), c = (idx - r * (HT_BK / 4)) * 4;
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (m0 + r < p.T && k0 + c < p.K)
                v = *reinterpret_cast<const float4*>(p.x + (size_t)(m0 + r) * p.ld_x + (size_t)h * p.x_head + p.x_col + k0 + c);
            uint2 packed;
            packed.x = pack_bf16(v.x, v.y);
            packed.y = pack_bf16(v.z, v.w);
            *reinterpret_cast<uint2*>(As + r * HT_LD + c) = packed;
        }
        for (int idx = threadIdx.x; idx < HT_BN * (HT_BK / 8); idx += 128) {
            const int r = idx / (HT_BK / 8), c = (idx - r * (HT_BK / 8)) * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (n0 + r < p.N && k0 + c < p.K) v = *reinterpret_cast<const uint4*>(w + (size_t)(n0 + r) * p.K + k0 + c);
            *reinterpret_cast<uint4*>(Bs + r * HT_LD + c) = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HT_BK; kk += 16) {
            uint32_t af[4];
            ldmatrix_x4(af, As + (warp * 16 + (lane & 15)) * HT_LD + kk + (lane >> 4) * 8);
#pragma unroll
            for (int nt = 0; nt < 8; nt += 2) {
                uint32_t bf[4];
                ldmatrix_x4(bf, Bs + ((nt + (lane >> 4)) * 8 + (lane & 7)) * HT_LD + kk + ((lane >> 3) & 1) * 8);
                mma_bf16(acc[nt], af, bf[0], bf[1]);
                mma_bf16(acc[nt + 1], af, bf[2], bf[3]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int nt = 0; nt < 8; nt++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int row = m0 + warp * 16 + g + (e >> 1) * 8, n = n0 + nt * 8 + 2 * t + (e & 1);
            if (row >= p.T || n >= p.N) continue;
            float v = acc[nt][e];
            if (p.gate) v *= sigmoidf_(p.gate[(size_t)row * p.ld_g + p.g_col + (size_t)h * p.N + n]);
            ((TO*)p.out)[(size_t)row * p.ld_o + (size_t)h * p.o_head + p.o_col + n] = from_float<TO>(v);
        }
}

// NTO: value-column tiles of 8 a warp owns (DV / 2 <= 8 NTO).
template <typename TO, int NTO>
__global__ void __launch_bounds__(256, 1) shared_row_attention_tc_kernel(SinkAttnParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    pdl_launch_dependents();
    pdl_wait();
    const int D = p.D, DV = p.DV, DP = D + LT_PAD;
    const int VP = DV + LT_PAD;
    const bool alias = p.v_pool == nullptr;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [64][DP]
    __nv_bfloat16* Kb = Qs + LT_ROWS * DP;                                      // 2 x [32][DP]
    __nv_bfloat16* Vb = alias ? Kb : Kb + 2 * LT_KT * DP;                       // 2 x [32][VP], or the key rows themselves
    const int v_ld = alias ? DP : VP;
    const __nv_bfloat16* vp = (const __nv_bfloat16*)p.v_pool;
    const int v8 = DV / 8;
    const int group = p.H / p.G;
    const int chunks = (group + p.head_chunk - 1) / p.head_chunk;
    const int tile = blockIdx.x, kvh = blockIdx.y / chunks, hc = blockIdx.y - kvh * chunks;
    const int head0 = kvh * group + hc * p.head_chunk;
    const int nh = min(p.head_chunk, group - hc * p.head_chunk);
    const int seq = p.tiles[tile * 4 + 0], row0 = p.tiles[tile * 4 + 1], nq = p.tiles[tile * 4 + 2], pos0 = p.tiles[tile * 4 + 3];
    const int rows = nq * nh;
    // Warps: four row slabs of 16 rows, two warps a slab with half of the value columns each.  A tile of at most 16 rows
    // (a decoded token's heads) would leave three slabs idle and two warps with all the work, and a warp's chain of
    // dependent instructions per key tile is what bounds the block: there all eight warps take the one slab and an eighth
    // of the value columns each (every warp computes the slab's scores, as the two of a slab do anyway).  A value
    // column's sums are the same instructions in the same order either way.
    const bool narrow = rows <= 16 && DV % 128 == 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wr = narrow ? 0 : warp & 3, wc = narrow ? warp : warp >> 2;
    const int g = lane >> 2, t = lane & 3;
    const __nv_bfloat16* q = (const __nv_bfloat16*)p.q;
    const __nv_bfloat16* kp = (const __nv_bfloat16*)p.k_pool;
    const int d8 = D / 8;

    for (int idx = threadIdx.x; idx < LT_ROWS * d8; idx += blockDim.x) {
        const int r = idx / d8, c = idx - r * d8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < rows) {
            const int qi = r / nh, gq = r - qi * nh;
            v = reinterpret_cast<const uint4*>(q + ((size_t)(row0 + qi) * p.H + head0 + gq) * D)[c];
        }
        *reinterpret_cast<uint4*>(Qs + r * DP + c * 8) = v;
    }

    const int lo = first_visible(p, pos0);
    const int hi = pos0 + nq;
    const int kept = p.window > 0 ? min(p.keep_first, lo) : 0;
    const int rA = wr * 16 + g, rB = rA + 8;                   // the thread's two rows
    const int qposA = pos0 + rA / nh, qposB = pos0 + rB / nh;
    const bool liveA = rA < rows, liveB = rB < rows;
    const int half = narrow ? DV / 8 : DV / 2, col0 = wc * half;      // the warp's value columns

    float mA = -INFINITY, mB = -INFINITY, lA = 0.0f, lB = 0.0f;
    float o[NTO][4];
#pragma unroll
    for (int i = 0; i < NTO; i++) { o[i][0] = 0.0f; o[i][1] = 0.0f; o[i][2] = 0.0f; o[i][3] = 0.0f; }

    const int* bt = p.block_table + (size_t)seq * p.max_blocks;
    // the key tiles of the two visible ranges ([0, kept) and [lo, hi), inside this block's split), one after the other;
    // tile i + 1 is on its way into the other buffer (cp.async) while tile i is computed
    int s_lo = 0, s_hi = hi;
    if (p.n_splits > 1) { s_lo = blockIdx.z * p.split_keys; s_hi = min(hi, (int)(blockIdx.z + 1) * p.split_keys); }
    const int a0 = max(0, s_lo), b0 = min(kept, s_hi), a1 = max(lo, s_lo), b1 = min(hi, s_hi);
    const int f0 = a0 - (a0 % LT_KT), f1 = a1 - (a1 % LT_KT);
    const int n0 = a0 < b0 ? (b0 - f0 + LT_KT - 1) / LT_KT : 0, n1 = a1 < b1 ? (b1 - f1 + LT_KT - 1) / LT_KT : 0;
    const int n_key_tiles = n0 + n1;
    auto issue = [&](int i) {
        const int k0 = i < n0 ? f0 + i * LT_KT : f1 + (i - n0) * LT_KT;
        const int a = i < n0 ? a0 : a1, b = i < n0 ? b0 : b1;
        __nv_bfloat16* Ks = Kb + (i & 1) * LT_KT * DP;
        __nv_bfloat16* Vs = alias ? Ks : Vb + (i & 1) * LT_KT * VP;
        long long rowi[LT_KT / 8];
#pragma unroll
        for (int u = 0; u < LT_KT / 8; u++) {                  // the warp's rows: all look-ups first
            const int key = k0 + warp + 8 * u;
            rowi[u] = -1;
            if (key >= a && key < b) {
                const int blk = bt[key / p.page];
                if (blk >= 0 && blk < p.num_pages) rowi[u] = ((long long)blk * p.G + kvh) * p.page + (key % p.page);
                else if (lane == 0 && p.err) atomicOr(p.err, EMBER_ERR_PAGE_RANGE);
            }
        }
#pragma unroll
        for (int u = 0; u < LT_KT / 8; u++) {
            const int j = warp + 8 * u;
            for (int c = lane; c < d8; c += 32) {
                __nv_bfloat16* dst = Ks + j * DP + c * 8;
                if (rowi[u] >= 0) {
                    const uint32_t sa = (uint32_t)__cvta_generic_to_shared(dst);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(kp + rowi[u] * D + c * 8) : "memory");
                } else {
                    *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            if (!alias)
                for (int c = lane; c < v8; c += 32) {
                    __nv_bfloat16* dst = Vs + j * VP + c * 8;
                    if (rowi[u] >= 0) {
                        const uint32_t sa = (uint32_t)__cvta_generic_to_shared(dst);
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(vp + rowi[u] * DV + c * 8) : "memory");
                    } else {
                        *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (n_key_tiles > 0) issue(0);
    {
        for (int it = 0; it < n_key_tiles; it++) {
            if (it + 1 < n_key_tiles) {
                issue(it + 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncthreads();                                    // tile `it` has landed (and, the first time, the queries)
            const int k0 = it < n0 ? f0 + it * LT_KT : f1 + (it - n0) * LT_KT;
            const int a = it < n0 ? a0 : a1, b = it < n0 ? b0 : b1;
            const __nv_bfloat16* Ks = Kb + (it & 1) * LT_KT * DP;
            const __nv_bfloat16* Vs = alias ? Ks : Vb + (it & 1) * LT_KT * VP;

            // S = Q K^T for the slab's 16 rows and the tile's 32 keys
            float sc[4][4];
#pragma unroll
            for (int i = 0; i < 4; i++) { sc[i][0] = 0.0f; sc[i][1] = 0.0f; sc[i][2] = 0.0f; sc[i][3] = 0.0f; }
            const __nv_bfloat16* qa = Qs + (wr * 16 + (lane & 15)) * DP + (lane >> 4) * 8;
            const __nv_bfloat16* kb = Ks + ((lane >> 4) * 8 + (lane & 7)) * DP + ((lane >> 3) & 1) * 8;
            for (int kk = 0; kk < D; kk += 16) {
                uint32_t af[4], b01[4], b23[4];
                ldmatrix_x4(af, qa + kk);
                ldmatrix_x4(b01, kb + kk);                      // keys 0..15: (b0, b1) of key tiles 0 and 1
                ldmatrix_x4(b23, kb + 16 * DP + kk);            // keys 16..31
                mma_bf16(sc[0], af, b01[0], b01[1]);
                mma_bf16(sc[1], af, b01[2], b01[3]);
                mma_bf16(sc[2], af, b23[0], b23[1]);
                mma_bf16(sc[3], af, b23[2], b23[3]);
            }
            // mask, running maximum, weights
            float tmA = -INFINITY, tmB = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 4; nt++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int key = k0 + nt * 8 + 2 * t + e;
                    const bool in = key >= a && key < b;
                    const bool vA = liveA && in && key_visible(p, key, qposA);
                    const bool vB = liveB && in && key_visible(p, key, qposB);
                    sc[nt][e] = vA ? capped_score(p, sc[nt][e]) : -INFINITY;
                    sc[nt][2 + e] = vB ? capped_score(p, sc[nt][2 + e]) : -INFINITY;
                    tmA = fmaxf(tmA, sc[nt][e]);
                    tmB = fmaxf(tmB, sc[nt][2 + e]);
                }
            tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 1)); tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 2));
            tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 1)); tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 2));
            const float nA = fmaxf(mA, tmA), nB = fmaxf(mB, tmB);
            const float cA = nA == -INFINITY ? 1.0f : expf(mA - nA), cB = nB == -INFINITY ? 1.0f : expf(mB - nB);
            float sA = 0.0f, sB = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 4; nt++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const float pa = nA == -INFINITY ? 0.0f : expf(sc[nt][e] - nA);
                    const float pb = nB == -INFINITY ? 0.0f : expf(sc[nt][2 + e] - nB);
                    sc[nt][e] = pa; sc[nt][2 + e] = pb;
                    sA += pa; sB += pb;
                }
            sA += __shfl_xor_sync(0xffffffffu, sA, 1); sA += __shfl_xor_sync(0xffffffffu, sA, 2);
            sB += __shfl_xor_sync(0xffffffffu, sB, 1); sB += __shfl_xor_sync(0xffffffffu, sB, 2);
            lA = lA * cA + sA; lB = lB * cB + sB;
            mA = nA; mB = nB;
#pragma unroll
            for (int i = 0; i < NTO; i++) { o[i][0] *= cA; o[i][1] *= cA; o[i][2] *= cB; o[i][3] *= cB; }
            // O += P V: the value of key j is the first DV elements of its row
#pragma unroll
            for (int ks = 0; ks < 2; ks++) {
                uint32_t pf[4];
                pf[0] = pack_bf16(sc[2 * ks][0], sc[2 * ks][1]);
                pf[1] = pack_bf16(sc[2 * ks][2], sc[2 * ks][3]);
                pf[2] = pack_bf16(sc[2 * ks + 1][0], sc[2 * ks + 1][1]);
                pf[3] = pack_bf16(sc[2 * ks + 1][2], sc[2 * ks + 1][3]);
                const __nv_bfloat16* vb = Vs + (ks * 16 + (lane & 15)) * v_ld + col0 + (lane >> 4) * 8;
#pragma unroll
                for (int i = 0; i < NTO; i += 2) {
                    if (i * 8 < half) {                          // uniform
                        uint32_t vf[4];
                        ldmatrix_x4_trans(vf, vb + i * 8);       // value columns i * 8 .. + 15, keys ks * 16 .. + 15
                        mma_bf16(o[i], pf, vf[0], vf[1]);
                        if ((i + 1) * 8 < half) mma_bf16(o[i + 1], pf, vf[2], vf[3]);
                    }
                }
            }
            __syncthreads();                                    // the buffer is free for the tile after next
        }
    }

    if (p.n_splits > 1) {
        // a split leaves its sums, maximum and denominator; the merge kernel adds the sink
#pragma unroll
        for (int i = 0; i < NTO; i++) {
            const int c = i * 8 + 2 * t;
            if (c >= half) continue;
            if (liveA) {
                float* dst = p.part_o + ((((size_t)(row0 + rA / nh) * p.H + head0 + rA % nh) * p.n_splits) + blockIdx.z) * DV + col0 + c;
                dst[0] = o[i][0]; dst[1] = o[i][1];
            }
            if (liveB) {
                float* dst = p.part_o + ((((size_t)(row0 + rB / nh) * p.H + head0 + rB % nh) * p.n_splits) + blockIdx.z) * DV + col0 + c;
                dst[0] = o[i][2]; dst[1] = o[i][3];
            }
        }
        if (wc == 0 && t == 0) {
            if (liveA) {
                float* ml = p.part_ml + ((((size_t)(row0 + rA / nh) * p.H + head0 + rA % nh) * p.n_splits) + blockIdx.z) * 2;
                ml[0] = mA; ml[1] = lA;
            }
            if (liveB) {
                float* ml = p.part_ml + ((((size_t)(row0 + rB / nh) * p.H + head0 + rB % nh) * p.n_splits) + blockIdx.z) * 2;
                ml[0] = mB; ml[1] = lB;
            }
        }
        return;
    }

    // the sink joins the denominator once; write the two rows' columns
    float invA = 0.0f, invB = 0.0f;
    {
        const int hA = head0 + (liveA ? rA % nh : 0), hB = head0 + (liveB ? rB % nh : 0);
        float mm = mA, ll = lA, corr = 1.0f;
        if (p.sink) { const float sk = p.sink[hA]; mm = fmaxf(mA, sk); corr = mA == -INFINITY ? 0.0f : expf(mA - mm); ll = lA * corr + expf(sk - mm); }
        invA = ll > 0.0f ? corr / ll : 0.0f;
        mm = mB; ll = lB; corr = 1.0f;
        if (p.sink) { const float sk = p.sink[hB]; mm = fmaxf(mB, sk); corr = mB == -INFINITY ? 0.0f : expf(mB - mm); ll = lB * corr + expf(sk - mm); }
        invB = ll > 0.0f ? corr / ll : 0.0f;
        if (p.head_gate) {
            if (liveA) invA *= sigmoidf_(p.head_gate[(size_t)(row0 + rA / nh) * p.ld_gate + hA]);
            if (liveB) invB *= sigmoidf_(p.head_gate[(size_t)(row0 + rB / nh) * p.ld_gate + hB]);
        }
    }
#pragma unroll
    for (int i = 0; i < NTO; i++) {
        const int c = i * 8 + 2 * t;
        if (c >= half) continue;
        if (liveA) {
            TO* dst = (TO*)p.out + ((size_t)(row0 + rA / nh) * p.H + head0 + rA % nh) * DV + col0 + c;
            dst[0] = from_float<TO>(o[i][0] * invA); dst[1] = from_float<TO>(o[i][1] * invA);
        }
        if (liveB) {
            TO* dst = (TO*)p.out + ((size_t)(row0 + rB / nh) * p.H + head0 + rB % nh) * DV + col0 + c;
            dst[0] = from_float<TO>(o[i][2] * invB); dst[1] = from_float<TO>(o[i][3] * invB);
        }
    }
}

template <typename TO>
int launch_shared_row_tc(const SinkAttnParams& p, int n_tiles, int T_tokens, cudaStream_t st) {
    const size_t smem = ((size_t)(LT_ROWS + 2 * LT_KT) * (p.D + LT_PAD) + (p.v_pool ? (size_t)2 * LT_KT * (p.DV + LT_PAD) : 0)) * sizeof(__nv_bfloat16);
    if (smem > 220 * 1024) return fail("sink_attention: rows of %d need %zu bytes of shared memory", p.D, smem);
    const int group = p.H / p.G, chunks = (group + p.head_chunk - 1) / p.head_chunk;
    dim3 grid(n_tiles, p.G * chunks, p.n_splits);
    const int nto = (p.DV / 2 + 7) / 8;
    auto run = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail("sink_attention: shared memory %zu: %s", smem, cudaGetErrorString(e));
        launch_kernel(kernel, grid, 256, smem, st, p);
        return check_launch("shared_row_attention_tc");
    };
    int rc;
    if (nto <= 4) rc = run(shared_row_attention_tc_kernel<TO, 4>);
    else if (nto <= 8) rc = run(shared_row_attention_tc_kernel<TO, 8>);
    else if (nto <= 16) rc = run(shared_row_attention_tc_kernel<TO, 16>);
    else rc = run(shared_row_attention_tc_kernel<TO, 32>);
    if (rc) return rc;
    if (p.n_splits > 1) {
        launch_kernel(sink_combine_kernel<TO>, (unsigned)((size_t)T_tokens * p.H), p.DV >= 128 ? 128 : 64, 0, st,
                      (const float*)p.part_o, (const float*)p.part_ml, p.sink, (TO*)p.out, p.n_splits, p.DV, p.H, p.head_gate, p.ld_gate);
        return check_launch("sink_combine");
    }
    return 0;
}

}  // namespace ember

using namespace ember;

EMBER_API int ember_whole_norm_store(const float* qkv, int ld, const float* bias, const float* q_w, const float* k_w, float eps,
                                     int T, int H, int G, int D, int DV, const int* positions, const int* seq_of,
                                     const int* block_table, int max_blocks, int page, int num_pages, void* q_out,
                                     void* k_pool, void* v_pool, int dtype, int write_kv, int* err, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || D <= 0 || DV <= 0 || ld < H * D + G * D + G * DV)
        return fail("whole_norm_store: %d/%d heads of %d/%d in rows of %d", H, G, D, DV, ld);
    if (page <= 0 || max_blocks <= 0 || num_pages <= 0) return fail("whole_norm_store: bad cache geometry");
    WholeNormArgs p{qkv, ld, bias, q_w, k_w, eps, H, G, D, DV, positions, seq_of, block_table, max_blocks, page, num_pages,
                    q_out, k_pool, v_pool, write_kv, err};
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == EMBER_F32) launch_kernel(whole_norm_store_kernel<float>, T, 256, 0, st, p);
    else if (dtype == EMBER_BF16) launch_kernel(whole_norm_store_kernel<__nv_bfloat16>, T, 256, 0, st, p);
    else return fail("whole_norm_store: unsupported dtype %d", dtype);
    return check_launch("whole_norm_store");
}

EMBER_API int ember_head_prepare_store(const float* qkv, int ld, const float* bias, int norm_mode, const float* q_w, const float* k_w,
                                       float eps, const float* inv_freq, int rotary, float qt_coef, int qt_every, int T_tokens, int H,
                                       int G, int D, int DV, const int* positions, const int* seq_of, const int* block_table,
                                       int max_blocks, int page, int num_pages, void* q_out, void* k_pool, void* v_pool, int dtype,
                                       int write_kv, int* err, void* stream) {
    if (T_tokens <= 0) return 0;
    if (H <= 0 || G <= 0 || D <= 0 || DV <= 0 || ld < H * D + G * (D + DV)) return fail("head_prepare_store: %d/%d heads of %d / %d in rows of %d", H, G, D, DV, ld);
    if (norm_mode < 0 || norm_mode > 2 || (norm_mode && (!q_w || !k_w))) return fail("head_prepare_store: norm mode %d", norm_mode);
    if (rotary < 0 || rotary > D || (rotary & 1) || (rotary && !inv_freq)) return fail("head_prepare_store: %d rotated elements of %d", rotary, D);
    if (qt_every < 0 || page <= 0 || max_blocks <= 0 || num_pages <= 0) return fail("head_prepare_store: bad geometry");
    HeadPrepareArgs p{qkv, ld, bias, norm_mode, q_w, k_w, eps, inv_freq, rotary, qt_coef, qt_every, H, G, D, DV, positions, seq_of,
                      block_table, max_blocks, page, num_pages, q_out, k_pool, v_pool, write_kv, err};
    const size_t smem = (size_t)(H + G) * sizeof(float);
    if (smem > 40 * 1024) return fail("head_prepare_store: %d heads are too many", H + G);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == EMBER_F32) launch_kernel(head_prepare_store_kernel<float>, T_tokens, 256, smem, st, p);
    else if (dtype == EMBER_BF16) launch_kernel(head_prepare_store_kernel<__nv_bfloat16>, T_tokens, 256, smem, st, p);
    else return fail("head_prepare_store: unsupported dtype %d", dtype);
    return check_launch("head_prepare_store");
}

EMBER_API int ember_head_gate_apply(void* x, int dtype, const float* gate, int ld_gate, int T_tokens, int H, int DV, void* stream) {
    if (T_tokens <= 0) return 0;
    if (H <= 0 || DV <= 0 || ld_gate < H) return fail("head_gate_apply: %d heads of %d, gate rows of %d", H, DV, ld_gate);
    const size_t n = (size_t)T_tokens * H * DV;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == EMBER_F32) launch_kernel(head_gate_apply_kernel<float>, (unsigned)((n + 255) / 256), 256, 0, st, (float*)x, gate, ld_gate, H, DV, n);
    else if (dtype == EMBER_BF16)
        launch_kernel(head_gate_apply_kernel<__nv_bfloat16>, (unsigned)((n + 255) / 256), 256, 0, st, (__nv_bfloat16*)x, gate, ld_gate, H, DV, n);
    else return fail("head_gate_apply: unsupported dtype %d", dtype);
    return check_launch("head_gate_apply");
}

EMBER_API int ember_latent_prepare(const float* a, int ld, int q_col, int q_rank, int c_col, int kv_rank, int rot_dim,
                                   const float* q_w, const float* c_w, float eps, const float* inv_freq, int rotary, int T,
                                   const int* positions, const int* seq_of, const int* block_table, int max_blocks, int page,
                                   int num_pages, void* cq_out, void* pool, int dtype, int write_kv, int half_layout, float magnitude,
                                   int* err, void* stream) {
    if (T <= 0) return 0;
    if (q_rank < 0 || kv_rank <= 0 || rot_dim < 0 || rotary < 0 || rotary > rot_dim || (rotary & 1))
        return fail("latent_prepare: ranks %d / %d, rotated part %d of %d", q_rank, kv_rank, rotary, rot_dim);
    if (write_kv && (page <= 0 || max_blocks <= 0 || num_pages <= 0)) return fail("latent_prepare: bad cache geometry");
    if (rotary > 0 && !inv_freq) return fail("latent_prepare: a rotation needs its frequencies");
    LatentArgs p{a, ld, q_col, q_rank, c_col, kv_rank, rot_dim, q_w, c_w, eps, inv_freq, rotary, half_layout, magnitude, positions, seq_of, block_table,
                 max_blocks, page, num_pages, cq_out, pool, write_kv, err};
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == EMBER_F32) launch_kernel(latent_prepare_kernel<float>, T, 256, 0, st, p);
    else if (dtype == EMBER_BF16) launch_kernel(latent_prepare_kernel<__nv_bfloat16>, T, 256, 0, st, p);
    else return fail("latent_prepare: unsupported dtype %d", dtype);
    return check_launch("latent_prepare");
}

EMBER_API int ember_rotate_pairs(const float* in, int ld_in, int in_head, int in_col, void* out, int ld_out, int out_head,
                                 int out_col, int dtype, int T, int H, int width, int rotary, const float* inv_freq,
                                 const int* positions, int half_layout, float magnitude, void* stream) {
    if (T <= 0 || width <= 0) return 0;
    if (rotary < 0 || rotary > width || (rotary & 1) || (rotary > 0 && !inv_freq)) return fail("rotate_pairs: %d of %d rotated", rotary, width);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == EMBER_F32)
        launch_kernel(rotate_pairs_kernel<float>, T, 128, 0, st, in, ld_in, in_head, in_col, (float*)out, ld_out, out_head, out_col, H,
                      width, rotary, inv_freq, positions, half_layout, magnitude);
    else if (dtype == EMBER_BF16)
        launch_kernel(rotate_pairs_kernel<__nv_bfloat16>, T, 128, 0, st, in, ld_in, in_head, in_col, (__nv_bfloat16*)out, ld_out,
                      out_head, out_col, H, width, rotary, inv_freq, positions, half_layout, magnitude);
    else return fail("rotate_pairs: unsupported dtype %d", dtype);
    return check_launch("rotate_pairs");
}

EMBER_API int ember_head_gemm(const float* x, int ld_x, int x_head, int x_col, const void* w, int w_dtype, void* out, int out_dtype,
                              int ld_o, int o_head, int o_col, const float* gate, int ld_g, int g_col, int T, int H, int N, int K,
                              void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || N <= 0 || K <= 0 || H > 65535) return fail("head_gemm: %d heads of %d x %d", H, N, K);
    HeadGemmArgs p{x, ld_x, x_head, x_col, w, out, ld_o, o_head, o_col, gate, ld_g, g_col, T, H, N, K};
    cudaStream_t st = (cudaStream_t)stream;
    // bfloat16 weights with rows of whole 16-byte pieces (and x rows of whole float4s): the tensor-core form
    if (w_dtype == EMBER_BF16 && K % 8 == 0 && ld_x % 4 == 0 && x_head % 4 == 0 && x_col % 4 == 0 && head_gemm_on_tensor_cores()) {
        dim3 tgrid((T + HT_BM - 1) / HT_BM, (N + HT_BN - 1) / HT_BN, H);
        if (out_dtype == EMBER_BF16) launch_kernel(head_gemm_tc_kernel<__nv_bfloat16>, tgrid, 128, 0, st, p);
        else launch_kernel(head_gemm_tc_kernel<float>, tgrid, 128, 0, st, p);
        return check_launch("head_gemm_tc");
    }
    dim3 grid((T + HG_BM - 1) / HG_BM, (N + HG_BN - 1) / HG_BN, H);
    if (w_dtype == EMBER_F32 && out_dtype == EMBER_F32) launch_kernel(head_gemm_kernel<float, float>, grid, 256, 0, st, p);
    else if (w_dtype == EMBER_BF16 && out_dtype == EMBER_BF16) launch_kernel(head_gemm_kernel<__nv_bfloat16, __nv_bfloat16>, grid, 256, 0, st, p);
    else if (w_dtype == EMBER_BF16 && out_dtype == EMBER_F32) launch_kernel(head_gemm_kernel<__nv_bfloat16, float>, grid, 256, 0, st, p);
    else return fail("head_gemm: unsupported dtypes %d -> %d", w_dtype, out_dtype);
    return check_launch("head_gemm");
}

// Query heads of one key head that a block takes, and the query tokens of a tile that go with it.
EMBER_API int ember_sink_attention_head_chunk(int group) { return group <= 0 ? 0 : (group < SA_MAX_ROWS ? group : SA_MAX_ROWS); }

EMBER_API int ember_sink_attention(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype, int out_f32,
                                   int T_tokens, int H, int G, int D, int DV, const int* tiles, int n_tiles, int tile_q,
                                   const int* block_table, int max_blocks, int page, int num_pages, int window,
                                   int keep_first, const float* sink, float scale, int n_splits, int split_keys,
                                   float* part_o, float* part_ml, int* err, int key_chunk, float softcap, const float* head_gate, int ld_gate, void* stream) {
    if (n_tiles <= 0 || T_tokens <= 0) return 0;
    if (D <= 0 || DV <= 0 || DV > 512 || (!v_pool && DV > D)) return fail("sink_attention: heads of %d / %d are not taken", D, DV);
    if (H <= 0 || G <= 0 || H % G) return fail("sink_attention: %d heads do not divide into %d groups", H, G);
    const int chunk = ember_sink_attention_head_chunk(H / G);
    if (tile_q <= 0 || tile_q * chunk > SA_MAX_ROWS) return fail("sink_attention: tiles of %d queries x %d heads exceed %d rows", tile_q, chunk, SA_MAX_ROWS);
    if (n_splits < 1 || (n_splits > 1 && (split_keys <= 0 || !part_o || !part_ml)))
        return fail("sink_attention: bad split configuration (%d splits of %d keys)", n_splits, split_keys);
    if (n_splits > 65535 || (long long)G * ((H / G + chunk - 1) / chunk) > 65535) return fail("sink_attention: grid too large");
    if (page <= 0 || max_blocks <= 0 || num_pages <= 0) return fail("sink_attention: bad cache geometry");
    if (window < 0 || keep_first < 0) return fail("sink_attention: window %d, kept first tokens %d", window, keep_first);
    SinkAttnParams p;
    p.q = q; p.k_pool = k_pool; p.v_pool = v_pool; p.out = out; p.part_o = part_o; p.part_ml = part_ml;
    p.tiles = tiles; p.block_table = block_table; p.sink = sink; p.max_blocks = max_blocks; p.page = page; p.num_pages = num_pages;
    p.H = H; p.G = G; p.D = D; p.DV = DV; p.head_chunk = chunk; p.window = window; p.keep_first = keep_first; p.scale = scale;
    p.n_splits = n_splits; p.split_keys = split_keys; p.err = err;
    if (key_chunk < 0 || softcap < 0.0f || (head_gate && ld_gate < H)) return fail("sink_attention: chunk %d, score cap %g, gate rows of %d", key_chunk, softcap, ld_gate);
    p.chunk = key_chunk; p.softcap = softcap; p.head_gate = head_gate; p.ld_gate = ld_gate;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == EMBER_F32) return launch_sink_attention<float, float>(p, n_tiles, T_tokens, st);
    if (dtype == EMBER_BF16)
        return out_f32 ? launch_sink_attention<__nv_bfloat16, float>(p, n_tiles, T_tokens, st)
                       : launch_sink_attention<__nv_bfloat16, __nv_bfloat16>(p, n_tiles, T_tokens, st);
    return fail("sink_attention: unsupported dtype %d", dtype);
}

// The tensor-core form for bfloat16 caches, with a value pool or without (a value is then the first DV elements of
// the key row): D and DV multiples of 16, DV <= 512, tiles of 64 / heads-per-block query tokens; key splits as in
// ember_sink_attention.
EMBER_API int ember_shared_row_attention_tc_head_chunk(int group) { return group <= 0 ? 0 : (group < LT_ROWS ? group : LT_ROWS); }

EMBER_API int ember_shared_row_attention_tc(const void* q, const void* k_pool, const void* v_pool, void* out, int out_f32, int T_tokens, int H, int G, int D,
                                            int DV, const int* tiles, int n_tiles, int tile_q, const int* block_table, int max_blocks,
                                            int page, int num_pages, int window, int keep_first, const float* sink, float scale,
                                            int n_splits, int split_keys, float* part_o, float* part_ml, int* err, int key_chunk, float softcap, const float* head_gate, int ld_gate, void* stream) {
    if (n_tiles <= 0 || T_tokens <= 0) return 0;
    if (D <= 0 || DV <= 0 || (D & 15) || (DV & 15) || (!v_pool && DV > D) || DV > 512) return fail("shared_row_attention_tc: rows of %d / %d are not taken", D, DV);
    if (H <= 0 || G <= 0 || H % G) return fail("shared_row_attention_tc: %d heads do not divide into %d groups", H, G);
    const int chunk = ember_shared_row_attention_tc_head_chunk(H / G);
    if (tile_q <= 0 || tile_q * chunk > LT_ROWS) return fail("shared_row_attention_tc: tiles of %d queries x %d heads exceed %d rows", tile_q, chunk, LT_ROWS);
    if ((long long)G * ((H / G + chunk - 1) / chunk) > 65535 || n_splits > 65535) return fail("shared_row_attention_tc: grid too large");
    if (n_splits < 1 || (n_splits > 1 && (split_keys <= 0 || !part_o || !part_ml)))
        return fail("shared_row_attention_tc: bad split configuration (%d splits of %d keys)", n_splits, split_keys);
    if (page <= 0 || max_blocks <= 0 || num_pages <= 0 || window < 0 || keep_first < 0) return fail("shared_row_attention_tc: bad cache geometry");
    SinkAttnParams p;
    p.q = q; p.k_pool = k_pool; p.v_pool = v_pool; p.out = out; p.part_o = part_o; p.part_ml = part_ml;
    p.tiles = tiles; p.block_table = block_table; p.sink = sink; p.max_blocks = max_blocks; p.page = page; p.num_pages = num_pages;
    p.H = H; p.G = G; p.D = D; p.DV = DV; p.head_chunk = chunk; p.window = window; p.keep_first = keep_first; p.scale = scale;
    p.n_splits = n_splits; p.split_keys = split_keys; p.err = err;
    if (key_chunk < 0 || softcap < 0.0f || (head_gate && ld_gate < H)) return fail("sink_attention: chunk %d, score cap %g, gate rows of %d", key_chunk, softcap, ld_gate);
    p.chunk = key_chunk; p.softcap = softcap; p.head_gate = head_gate; p.ld_gate = ld_gate;
    cudaStream_t st = (cudaStream_t)stream;
    return out_f32 ? launch_shared_row_tc<float>(p, n_tiles, T_tokens, st) : launch_shared_row_tc<__nv_bfloat16>(p, n_tiles, T_tokens, st);
}
