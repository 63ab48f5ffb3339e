// Norms and gates around a sublayer, all statistics in fp32:
//   layer_norm        out[r] = (x - mean) / sqrt(var + eps) * w + b      (var = mean of squared deviations)
//   gated_norm_add    residual[r] += norm(y[r] * sigmoid(gate_logits[r])) for a layer norm or an RMS norm; the new
//                     residual row can also be left rounded to bfloat16 (for a sublayer that reads the stream itself)
//   scaled_add_norm   residual[r] = norm(alpha * residual[r] + y[r] + bias): the norm *after* the sum (a post-norm layer), in place,
//                     with the same optional bfloat16 copy of the new rows
//   pair_norm_sum     out[r] (+)= wa * a[r] / rms(a[r]) + wb * b[r] / rms(b[r]): two branches, each RMS-normed over the row
//   add_row_bias      y[r] += bias
//   round_rows        out = bfloat16(x)
//   group_norm_gate   a token's row cut into groups, each divided by its own root mean square, times a weight,
//                     with a gate before (silu) or after (sigmoid or silu) the norm
//   scaled_sum        out (+)= a x + b y
//   dynamic_tanh      out = tanh(alpha x) * w + b, element by element (a norm without statistics)
//   stream_read       u = sum_s in[s] x_s over the copies of the residual stream (optionally through dynamic_tanh)
//   stream_write      x_t <- sum_s mix[s, t] x_s + multiplier * out[t] * scale * y, all copies at once from the old ones
//   stream_spread     every copy = one row;   stream_sum   one row = the sum of the copies
//   logit_finish      logits <- cap tanh(scale logits / cap)
// Rows are read from the fp32 residual stream or from fp32 results of a product; a row is reduced by one block
// (or one warp for the short rows of a head) in an order fixed by the thread layout.
#include "common.cuh"

EMBER_DEFINE_LAST_ERROR

namespace ember {

constexpr int ROW_THREADS = 256;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// ------------------------------------------------------------------------------------------ layer norm
template <typename TO>
__global__ void __launch_bounds__(ROW_THREADS)
layer_norm_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                  const float* __restrict__ b, float eps, TO* __restrict__ out, int H) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* in = x + (size_t)(rows ? rows[r] : r) * H;
    TO* o = out + (size_t)r * H;
    float s = 0.0f;
    for (int i = threadIdx.x; i < H; i += ROW_THREADS) s += in[i];
    const float mean = block_sum(s, scratch) / (float)H;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += ROW_THREADS) {
        const float d = in[i] - mean;
        ss = fmaf(d, d, ss);
    }
    const float rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += ROW_THREADS)
        o[i] = from_float<TO>((in[i] - mean) * rstd * w[i] + (b ? b[i] : 0.0f));
}

// ------------------------------------------------------------------------------- gate, norm, add to the stream
// v = y * sigmoid(gate + gate_bias) (gate nullable); centred (layer norm) or not (RMS norm); residual += v_hat * w + b.
template <bool CENTRED>
__global__ void __launch_bounds__(ROW_THREADS)
gated_norm_add_kernel(const float* __restrict__ y, const float* __restrict__ gate, const float* __restrict__ gate_bias,
                      const float* __restrict__ w, const float* __restrict__ b, float eps, float* __restrict__ residual,
                      __nv_bfloat16* __restrict__ rounded, int H) {
    extern __shared__ float row[];          // H floats: the gated row
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float s = 0.0f;
    for (int i = threadIdx.x; i < H; i += ROW_THREADS) {
        float v = y[base + i];
        if (gate) v *= sigmoidf_(gate[base + i] + (gate_bias ? gate_bias[i] : 0.0f));
        row[i] = v;
        s += v;
    }
    float mean = 0.0f;
    if (CENTRED) mean = block_sum(s, scratch) / (float)H;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += ROW_THREADS) {
        const float d = row[i] - mean;
        ss = fmaf(d, d, ss);
    }
    const float rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += ROW_THREADS) {
        const float r = residual[base + i] + ((row[i] - mean) * rstd * w[i] + (b ? b[i] : 0.0f));
        residual[base + i] = r;
        if (rounded) rounded[base + i] = __float2bfloat16_rn(r);      // what the next sublayer's products read
    }
}

// ------------------------------------------------------------------------------- norm after the residual sum
// residual[r] = norm(alpha * residual[r] + y[r] + y_bias) * w + b: the stream is scaled, the sublayer's result (and
// the bias its last product left out, if any) added, and the sum normed in place.
template <bool CENTRED>
__global__ void __launch_bounds__(ROW_THREADS)
scaled_add_norm_kernel(const float* __restrict__ y, const float* __restrict__ y_bias, float alpha, const float* __restrict__ w,
                       const float* __restrict__ b, float eps, float* __restrict__ residual, __nv_bfloat16* __restrict__ rounded,
                       int H) {
    extern __shared__ float row[];          // H floats: the sum
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float s = 0.0f;
    for (int i = threadIdx.x; i < H; i += ROW_THREADS) {
        const float v = fmaf(alpha, residual[base + i], y[base + i] + (y_bias ? y_bias[i] : 0.0f));
        row[i] = v;
        s += v;
    }
    float mean = 0.0f;
    if (CENTRED) mean = block_sum(s, scratch) / (float)H;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += ROW_THREADS) {
        const float d = row[i] - mean;
        ss = fmaf(d, d, ss);
    }
    const float rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += ROW_THREADS) {
        const float r = (row[i] - mean) * rstd * w[i] + (b ? b[i] : 0.0f);
        residual[base + i] = r;
        if (rounded) rounded[base + i] = __float2bfloat16_rn(r);
    }
}

// out[r] (+)= wa * a[r] / rms(a[r]) + wb * b[r] / rms(b[r]); each root mean square over the whole row, eps inside the root.
__global__ void __launch_bounds__(ROW_THREADS)
pair_norm_sum_kernel(const float* __restrict__ a, const float* __restrict__ wa, const float* __restrict__ b,
                     const float* __restrict__ wb, float eps, float* __restrict__ out, int accumulate, int H) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float sa = 0.0f, sb = 0.0f;
    for (int i = threadIdx.x; i < H; i += ROW_THREADS) {
        const float x = a[base + i], z = b[base + i];
        sa = fmaf(x, x, sa);
        sb = fmaf(z, z, sb);
    }
    const float ra = 1.0f / sqrtf(block_sum(sa, scratch) / (float)H + eps);
    const float rb = 1.0f / sqrtf(block_sum(sb, scratch) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += ROW_THREADS) {
        const float v = fmaf(a[base + i] * ra, wa[i], b[base + i] * rb * wb[i]);
        out[base + i] = accumulate ? out[base + i] + v : v;
    }
}

__global__ void add_row_bias_kernel(float* __restrict__ y, const float* __restrict__ bias, size_t n, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] += bias[i % H];
}

// ---------------------------------------------------------------------------------- per-group RMS norm with gate
// TPG threads per (token, group): a warp for the short rows of a head, a whole block of 256 for wide groups (a
// state-space layer normalises all its channels as one group or a few).  gate_mode 0: none; 1: out *= sigmoid(gate)
// after the norm; 2: v *= silu(gate) before; 3: out *= silu(gate) after.
template <typename TO, int TPG>
__global__ void __launch_bounds__(256)
group_norm_gate_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ gate, int ldg,
                       const float* __restrict__ w, int w_stride, float eps, int gate_mode,
                       const float* __restrict__ den4, TO* __restrict__ out, int T, int groups, int V) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int row = TPG == 32 ? (blockIdx.x * blockDim.x + threadIdx.x) >> 5 : blockIdx.x;
    const int lane = TPG == 32 ? (threadIdx.x & 31) : threadIdx.x;
    if (row >= T * groups) return;
    const int t = row / groups, g = row - t * groups;
    const float* in = x + (size_t)t * ldx + (size_t)g * V;
    const float* gl = gate ? gate + (size_t)t * ldg + (size_t)g * V : nullptr;
    // den4 (nullable): per (token, group) four floats whose last two are (floor, dot): the group is first divided by
    // max(|dot|, floor) + 1e-6 (the denominator of a matrix memory's read-out)
    const float inv = den4 ? 1.0f / (fmaxf(fabsf(den4[(size_t)row * 4 + 3]), den4[(size_t)row * 4 + 2]) + 1e-6f) : 1.0f;
    float ss = 0.0f;
    for (int j = lane; j < V; j += TPG) {
        float v = in[j] * inv;
        if (gate_mode == 2) { const float z = gl[j]; v *= z * sigmoidf_(z); }
        ss = fmaf(v, v, ss);
    }
    ss = TPG == 32 ? warp_sum(ss) : block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)V + eps);
    TO* o = out + ((size_t)t * groups + g) * V;
    const float* wg = w + (size_t)g * w_stride;
    for (int j = lane; j < V; j += TPG) {
        float v = in[j] * inv;
        if (gate_mode == 2) { const float z = gl[j]; v *= z * sigmoidf_(z); }
        v = v * r * wg[j];
        if (gate_mode == 1) v *= sigmoidf_(gl[j]);
        else if (gate_mode == 3) { const float z = gl[j]; v *= z * sigmoidf_(z); }
        o[j] = from_float<TO>(v);
    }
}

__global__ void round_rows_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16_rn(x[i]);
}

__global__ void scaled_sum_kernel(const float* __restrict__ x, float a, const float* __restrict__ y, float b,
                                  float* __restrict__ out, int accumulate, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = a * x[i] + (y ? b * y[i] : 0.0f);
    out[i] = accumulate ? out[i] + v : v;
}


// ------------------------------------------------------------------------------------------ dynamic tanh
// out[r, i] = (tanh(alpha x[rows[r] or r, i]) * w[i] + b[i]); alpha is a stored scalar (read from the device).
template <typename TO>
__global__ void dynamic_tanh_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ alpha,
                                    const float* __restrict__ w, const float* __restrict__ b, TO* __restrict__ out, int H, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const size_t r = idx / H;
    const int i = (int)(idx - r * H);
    const float v = x[(size_t)(rows ? rows[r] : r) * H + i];
    out[idx] = from_float<TO>(fmaf(tanhf(alpha[0] * v), w[i], b ? b[i] : 0.0f));
}

// ------------------------------------------------------------------- several copies of the residual stream
// X is [T, S, H] fp32.  A sublayer reads u = sum_s in[s] x_s (in null: all ones); with alpha the sum goes through
// tanh(alpha u) * w + b on its way out.
constexpr int MAX_STREAMS = 16;

template <typename TO>
__global__ void stream_read_kernel(const float* __restrict__ X, int S, const float* __restrict__ in_w, const float* __restrict__ alpha,
                                   const float* __restrict__ w, const float* __restrict__ b, TO* __restrict__ out, int H, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const size_t t = idx / H;
    const int i = (int)(idx - t * H);
    const float* src = X + t * S * H + i;
    float u = 0.0f;
    for (int s = 0; s < S; s++) u = fmaf(in_w ? in_w[s] : 1.0f, src[(size_t)s * H], u);
    if (alpha) u = fmaf(tanhf(alpha[0] * u), w[i], b ? b[i] : 0.0f);
    out[idx] = from_float<TO>(u);
}

// x_r <- sum_s mix[s, r] x_s + multiplier * out_w[r] * scale[i] * y  for every copy r, from the old copies (mix null: the
// identity; out_w null: ones; scale null: ones).  A thread owns one (token, column) of all copies.
__global__ void stream_write_kernel(float* __restrict__ X, int S, const float* __restrict__ mix, const float* __restrict__ out_w,
                                    const float* __restrict__ scale, float multiplier, const float* __restrict__ y, int H, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const size_t t = idx / H;
    const int i = (int)(idx - t * H);
    float* col = X + t * S * H + i;
    const float add = multiplier * (scale ? scale[i] : 1.0f) * y[idx];
    float old[MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; s++)
        if (s < S) old[s] = col[(size_t)s * H];
#pragma unroll
    for (int r = 0; r < MAX_STREAMS; r++) {
        if (r >= S) break;
        float v;
        if (mix) {
            v = 0.0f;
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; s++)
                if (s < S) v = fmaf(mix[s * S + r], old[s], v);
        } else {
            v = old[r];
        }
        col[(size_t)r * H] = fmaf(out_w ? out_w[r] : 1.0f, add, v);
    }
}

// The same two kernels for up to four copies and rows that are a multiple of four floats on 16-byte boundaries: a thread
// owns four neighbouring columns of a token in all copies (16-byte loads and stores, the copies' loop unrolled, the mix
// matrix in registers).  Every element is summed in the order of the kernels above, so the results are the same bits.
__device__ __forceinline__ void store4(float* out, size_t i4, float4 v) { reinterpret_cast<float4*>(out)[i4] = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* out, size_t i4, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&lo);
    u.y = *reinterpret_cast<unsigned*>(&hi);
    reinterpret_cast<uint2*>(out)[i4] = u;
}

template <int S, typename TO>
__global__ void stream_read_vec_kernel(const float4* __restrict__ X, const float* __restrict__ in_w, const float* __restrict__ alpha,
                                       const float4* __restrict__ w, const float4* __restrict__ b, TO* __restrict__ out, int H4, size_t n4) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n4) return;
    const size_t t = idx / H4;
    const int i = (int)(idx - t * H4);
    const float4* src = X + t * S * H4 + i;
    float4 u = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int s = 0; s < S; s++) {
        const float4 v = src[(size_t)s * H4];
        const float a = in_w ? in_w[s] : 1.0f;
        u.x = fmaf(a, v.x, u.x), u.y = fmaf(a, v.y, u.y), u.z = fmaf(a, v.z, u.z), u.w = fmaf(a, v.w, u.w);
    }
    if (alpha) {
        const float a = alpha[0];
        const float4 ww = w[i], bb = b ? b[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        u.x = fmaf(tanhf(a * u.x), ww.x, bb.x), u.y = fmaf(tanhf(a * u.y), ww.y, bb.y);
        u.z = fmaf(tanhf(a * u.z), ww.z, bb.z), u.w = fmaf(tanhf(a * u.w), ww.w, bb.w);
    }
    store4(out, idx, u);
}

template <int S>
__global__ void stream_write_vec_kernel(float4* __restrict__ X, const float* __restrict__ mix, const float* __restrict__ out_w,
                                        const float4* __restrict__ scale, float multiplier, const float4* __restrict__ y, int H4, size_t n4) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n4) return;
    const size_t t = idx / H4;
    const int i = (int)(idx - t * H4);
    float4* col = X + t * S * H4 + i;
    const float4 sc = scale ? scale[i] : make_float4(1.0f, 1.0f, 1.0f, 1.0f), yy = y[idx];
    const float4 add = make_float4(multiplier * sc.x * yy.x, multiplier * sc.y * yy.y, multiplier * sc.z * yy.z, multiplier * sc.w * yy.w);
    float4 old[S];
#pragma unroll
    for (int s = 0; s < S; s++) old[s] = col[(size_t)s * H4];
#pragma unroll
    for (int r = 0; r < S; r++) {
        float4 v;
        if (mix) {
            v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int s = 0; s < S; s++) {
                const float m = mix[s * S + r];
                v.x = fmaf(m, old[s].x, v.x), v.y = fmaf(m, old[s].y, v.y), v.z = fmaf(m, old[s].z, v.z), v.w = fmaf(m, old[s].w, v.w);
            }
        } else {
            v = old[r];
        }
        const float o = out_w ? out_w[r] : 1.0f;
        col[(size_t)r * H4] = make_float4(fmaf(o, add.x, v.x), fmaf(o, add.y, v.y), fmaf(o, add.z, v.z), fmaf(o, add.w, v.w));
    }
}

static bool aligned16(const void* a, const void* b = nullptr, const void* c = nullptr, const void* d = nullptr, const void* e = nullptr) {
    return (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d | (uintptr_t)e) & 15) == 0;
}

__global__ void stream_spread_kernel(const float* __restrict__ x, float* __restrict__ X, int S, int H, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const size_t t = idx / H;
    const int i = (int)(idx - t * H);
    const float v = x[idx];
    for (int s = 0; s < S; s++) X[(t * S + s) * H + i] = v;
}

__global__ void stream_sum_kernel(const float* __restrict__ X, const int* __restrict__ rows, int S, float* __restrict__ out, int H,
                                  size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const size_t r = idx / H;
    const int i = (int)(idx - r * H);
    const float* src = X + (size_t)(rows ? rows[r] : r) * S * H + i;
    float v = 0.0f;
    for (int s = 0; s < S; s++) v += src[(size_t)s * H];
    out[idx] = v;
}

// logits <- cap * tanh(scale * logits / cap)  (cap 0: scale * logits); four elements a thread where the buffer allows
__device__ __forceinline__ float capped(float v, float scale, float cap) {
    v *= scale;
    return cap > 0.0f ? cap * tanhf(v / cap) : v;
}

__global__ void logit_finish_kernel(float* __restrict__ logits, float scale, float cap, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    logits[idx] = capped(logits[idx], scale, cap);
}

__global__ void __launch_bounds__(256)
logit_finish_vec_kernel(float4* __restrict__ logits, float scale, float cap, size_t n4) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n4) return;
    float4 v = logits[idx];
    v.x = capped(v.x, scale, cap);
    v.y = capped(v.y, scale, cap);
    v.z = capped(v.z, scale, cap);
    v.w = capped(v.w, scale, cap);
    logits[idx] = v;
}

}  // namespace ember

using namespace ember;

EMBER_API int ember_layer_norm(const float* x, const int* rows, const float* w, const float* b, float eps, void* out,
                               int out_dtype, int n_rows, int H, void* stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0) return fail("layer_norm: bad width %d", H);
    cudaStream_t st = (cudaStream_t)stream;
    if (out_dtype == EMBER_F32)
        launch_kernel(layer_norm_kernel<float>, n_rows, ROW_THREADS, 0, st, x, rows, w, b, eps, (float*)out, H);
    else if (out_dtype == EMBER_BF16)
        launch_kernel(layer_norm_kernel<__nv_bfloat16>, n_rows, ROW_THREADS, 0, st, x, rows, w, b, eps, (__nv_bfloat16*)out, H);
    else
        return fail("layer_norm: unsupported output dtype %d", out_dtype);
    return check_launch("layer_norm");
}

EMBER_API int ember_gated_norm_add(const float* y, const float* gate, const float* gate_bias, const float* w, const float* b, float eps, int centred,
                                   float* residual, void* rounded, int n_rows, int H, void* stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || (size_t)H * 4 > 200 * 1024) return fail("gated_norm_add: width %d is not taken", H);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(gated_norm_add_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(gated_norm_add_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    if (centred) launch_kernel(gated_norm_add_kernel<true>, n_rows, ROW_THREADS, smem, st, y, gate, gate_bias, w, b, eps, residual, (__nv_bfloat16*)rounded, H);
    else launch_kernel(gated_norm_add_kernel<false>, n_rows, ROW_THREADS, smem, st, y, gate, gate_bias, w, b, eps, residual, (__nv_bfloat16*)rounded, H);
    return check_launch("gated_norm_add");
}

EMBER_API int ember_scaled_add_norm(const float* y, const float* y_bias, float alpha, const float* w, const float* b, float eps,
                                    int centred, float* residual, void* rounded, int n_rows, int H, void* stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || (size_t)H * 4 > 200 * 1024) return fail("scaled_add_norm: width %d is not taken", H);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(scaled_add_norm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(scaled_add_norm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    if (centred) launch_kernel(scaled_add_norm_kernel<true>, n_rows, ROW_THREADS, smem, st, y, y_bias, alpha, w, b, eps, residual, (__nv_bfloat16*)rounded, H);
    else launch_kernel(scaled_add_norm_kernel<false>, n_rows, ROW_THREADS, smem, st, y, y_bias, alpha, w, b, eps, residual, (__nv_bfloat16*)rounded, H);
    return check_launch("scaled_add_norm");
}

EMBER_API int ember_pair_norm_sum(const float* a, const float* wa, const float* b, const float* wb, float eps, float* out,
                                  int accumulate, int n_rows, int H, void* stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0) return fail("pair_norm_sum: bad width %d", H);
    launch_kernel(pair_norm_sum_kernel, n_rows, ROW_THREADS, 0, (cudaStream_t)stream, a, wa, b, wb, eps, out, accumulate, H);
    return check_launch("pair_norm_sum");
}

EMBER_API int ember_add_row_bias(float* y, const float* bias, int n_rows, int H, void* stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0) return fail("add_row_bias: bad width %d", H);
    const size_t n = (size_t)n_rows * H;
    launch_kernel(add_row_bias_kernel, (unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream, y, bias, n, H);
    return check_launch("add_row_bias");
}

EMBER_API int ember_group_norm_gate(const float* x, int ldx, const float* gate, int ldg, const float* w, int w_stride,
                                    float eps, int gate_mode, const float* den4, void* out, int out_dtype, int T, int groups, int V,
                                    void* stream) {
    if (T <= 0) return 0;
    if (groups <= 0 || V <= 0 || ldx < groups * V) return fail("group_norm_gate: %d groups of %d in rows of %d", groups, V, ldx);
    if (gate_mode < 0 || gate_mode > 3 || (gate_mode && (!gate || ldg < groups * V))) return fail("group_norm_gate: bad gate");
    cudaStream_t st = (cudaStream_t)stream;
    const long long rows = (long long)T * groups;
    const bool wide = V > 512;
    const unsigned blocks = wide ? (unsigned)rows : (unsigned)((rows + 7) / 8);
#define EMBER_GNG(TO, TPG) launch_kernel(group_norm_gate_kernel<TO, TPG>, blocks, 256, 0, st, x, ldx, gate, ldg, w, w_stride, eps, \
                                         gate_mode, den4, (TO*)out, T, groups, V)
    if (out_dtype == EMBER_F32) { if (wide) EMBER_GNG(float, 256); else EMBER_GNG(float, 32); }
    else if (out_dtype == EMBER_BF16) { if (wide) EMBER_GNG(__nv_bfloat16, 256); else EMBER_GNG(__nv_bfloat16, 32); }
    else return fail("group_norm_gate: unsupported output dtype %d", out_dtype);
#undef EMBER_GNG
    return check_launch("group_norm_gate");
}

EMBER_API int ember_scaled_sum(const float* x, float a, const float* y, float b, float* out, int accumulate, long long n, void* stream) {
    if (n <= 0) return 0;
    launch_kernel(scaled_sum_kernel, (unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream, x, a, y, b, out, accumulate, (size_t)n);
    return check_launch("scaled_sum");
}

EMBER_API int ember_round_rows(const float* x, void* out, long long n, void* stream) {
    if (n <= 0) return 0;
    launch_kernel(round_rows_kernel, (unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream, x, (__nv_bfloat16*)out, (size_t)n);
    return check_launch("round_rows");
}

EMBER_API int ember_dynamic_tanh(const float* x, const int* rows, const float* alpha, const float* w, const float* b, void* out,
                                 int out_dtype, int n_rows, int H, void* stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || !alpha || !w) return fail("dynamic_tanh: rows of %d need alpha and a weight", H);
    const size_t n = (size_t)n_rows * H;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dtype == EMBER_F32) launch_kernel(dynamic_tanh_kernel<float>, blocks, 256, 0, st, x, rows, alpha, w, b, (float*)out, H, n);
    else if (out_dtype == EMBER_BF16)
        launch_kernel(dynamic_tanh_kernel<__nv_bfloat16>, blocks, 256, 0, st, x, rows, alpha, w, b, (__nv_bfloat16*)out, H, n);
    else return fail("dynamic_tanh: unsupported output dtype %d", out_dtype);
    return check_launch("dynamic_tanh");
}

EMBER_API int ember_stream_read(const float* X, int S, const float* in_w, const float* alpha, const float* w, const float* b, void* out,
                                int out_dtype, int T, int H, void* stream) {
    if (T <= 0) return 0;
    if (S <= 0 || S > MAX_STREAMS || H <= 0 || (alpha && !w)) return fail("stream_read: %d copies (at most %d) of rows of %d", S, MAX_STREAMS, H);
    const size_t n = (size_t)T * H;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dtype != EMBER_F32 && out_dtype != EMBER_BF16) return fail("stream_read: unsupported output dtype %d", out_dtype);
    if (S <= 4 && H % 4 == 0 && aligned16(X, w, b, out)) {
        const size_t n4 = n / 4;
        const unsigned vb = (unsigned)((n4 + 255) / 256);
        const float4 *X4 = (const float4*)X, *w4 = (const float4*)w, *b4 = (const float4*)b;
#define EMBER_STREAM_READ(S_)                                                                                                      \
        if (out_dtype == EMBER_F32) launch_kernel(stream_read_vec_kernel<S_, float>, vb, 256, 0, st, X4, in_w, alpha, w4, b4,     \
                                                  (float*)out, H / 4, n4);                                                         \
        else launch_kernel(stream_read_vec_kernel<S_, __nv_bfloat16>, vb, 256, 0, st, X4, in_w, alpha, w4, b4, (__nv_bfloat16*)out, H / 4, n4)
        switch (S) {
            case 1: EMBER_STREAM_READ(1); break;
            case 2: EMBER_STREAM_READ(2); break;
            case 3: EMBER_STREAM_READ(3); break;
            default: EMBER_STREAM_READ(4); break;
        }
#undef EMBER_STREAM_READ
        return check_launch("stream_read");
    }
    if (out_dtype == EMBER_F32) launch_kernel(stream_read_kernel<float>, blocks, 256, 0, st, X, S, in_w, alpha, w, b, (float*)out, H, n);
    else if (out_dtype == EMBER_BF16)
        launch_kernel(stream_read_kernel<__nv_bfloat16>, blocks, 256, 0, st, X, S, in_w, alpha, w, b, (__nv_bfloat16*)out, H, n);
    else return fail("stream_read: unsupported output dtype %d", out_dtype);
    return check_launch("stream_read");
}

EMBER_API int ember_stream_write(float* X, int S, const float* mix, const float* out_w, const float* scale, float multiplier,
                                 const float* y, int T, int H, void* stream) {
    if (T <= 0) return 0;
    if (S <= 0 || S > MAX_STREAMS || H <= 0) return fail("stream_write: %d copies (at most %d) of rows of %d", S, MAX_STREAMS, H);
    const size_t n = (size_t)T * H;
    if (S <= 4 && H % 4 == 0 && aligned16(X, scale, y)) {
        const size_t n4 = n / 4;
        const unsigned vb = (unsigned)((n4 + 255) / 256);
        cudaStream_t st = (cudaStream_t)stream;
        float4* X4 = (float4*)X;
        const float4 *s4 = (const float4*)scale, *y4 = (const float4*)y;
        switch (S) {
            case 1: launch_kernel(stream_write_vec_kernel<1>, vb, 256, 0, st, X4, mix, out_w, s4, multiplier, y4, H / 4, n4); break;
            case 2: launch_kernel(stream_write_vec_kernel<2>, vb, 256, 0, st, X4, mix, out_w, s4, multiplier, y4, H / 4, n4); break;
            case 3: launch_kernel(stream_write_vec_kernel<3>, vb, 256, 0, st, X4, mix, out_w, s4, multiplier, y4, H / 4, n4); break;
            default: launch_kernel(stream_write_vec_kernel<4>, vb, 256, 0, st, X4, mix, out_w, s4, multiplier, y4, H / 4, n4); break;
        }
        return check_launch("stream_write");
    }
    launch_kernel(stream_write_kernel, (unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream, X, S, mix, out_w, scale, multiplier, y, H, n);
    return check_launch("stream_write");
}

EMBER_API int ember_stream_spread(const float* x, float* X, int S, int T, int H, void* stream) {
    if (T <= 0) return 0;
    if (S <= 0 || H <= 0) return fail("stream_spread: %d copies of rows of %d", S, H);
    const size_t n = (size_t)T * H;
    launch_kernel(stream_spread_kernel, (unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream, x, X, S, H, n);
    return check_launch("stream_spread");
}

EMBER_API int ember_stream_sum(const float* X, const int* rows, int S, float* out, int n_rows, int H, void* stream) {
    if (n_rows <= 0) return 0;
    if (S <= 0 || H <= 0) return fail("stream_sum: %d copies of rows of %d", S, H);
    const size_t n = (size_t)n_rows * H;
    launch_kernel(stream_sum_kernel, (unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream, X, rows, S, out, H, n);
    return check_launch("stream_sum");
}

EMBER_API int ember_logit_finish(float* logits, float scale, float cap, long long n, void* stream) {
    if (n <= 0) return 0;
    if (n % 4 == 0 && ((uintptr_t)logits & 15) == 0) {
        const size_t n4 = (size_t)n / 4;
        launch_kernel(logit_finish_vec_kernel, (unsigned)((n4 + 255) / 256), 256, 0, (cudaStream_t)stream, (float4*)logits, scale, cap, n4);
    } else {
        launch_kernel(logit_finish_kernel, (unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream, logits, scale, cap, (size_t)n);
    }
    return check_launch("logit_finish");
}
