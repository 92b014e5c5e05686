// Kernels of the parts that carry a fixed-size state from token to token, and
// the small row-wise kernels around them:
//
// * short_conv: y_t = x_t + sum_j w[:, j] x_(t - taps + 1 + j) per channel, with the
//   inputs before a step's first token taken from the request's history;
// * delta_rule: the recurrence S <- diag(w) S - (a u)(u^T S) + k v^T, o = S^T r with one
//   state matrix per head, decays, rates and unit keys made in 32-bit from the
//   stacked product's output and the decay's logits; decay_logits makes those logits
//   for steps of few tokens;
// * gated_group_norm: x / rms(x per group) * weight * sigmoid(gate);
// * scale, cast_rows (with an activation on the way), add_row_vector, activation (in place,
//   or on the sums of a split product).
//
// Everything that enters the recurrence, and the state itself, is 32-bit in the
// bfloat16 engine too.
#define CHIBI_UNIT sequence_ops
#define CHIBI_UNIT_ID 8
#include "common.cuh"

namespace chibi {

// ---------------------------------------------------------------- short convolution
// grid (channel blocks, chunks of a sequence's tokens, sequences).  A thread owns one
// channel of one chunk of consecutive tokens of one sequence.  Only the
// first chunk of a sequence reads the history (a chunk is at least taps - 1 tokens
// long), and the same thread writes the new history after its last read, so nobody
// reads a history that another thread has replaced.
template <typename TX>
__global__ void __launch_bounds__(128)
short_conv_kernel(const TX* __restrict__ x, long long x_stride, const float* __restrict__ w, TX* history,
                  TX* __restrict__ out, long long out_stride, const int* __restrict__ q_start,
                  const int* __restrict__ slots, int channels, int taps, int chunk,
                  const float* __restrict__ bias, int act, int add_input)
{
    pdl_enter();
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    const int seq = blockIdx.z;
    const int row0 = q_start[seq];
    const int q_len = q_start[seq + 1] - row0;
    const int first = blockIdx.y * chunk;
    if (ch >= channels || first >= q_len)
        return;
    const int keep = taps - 1;
    const int last = min(first + chunk, q_len);
    TX* hist = history + (size_t)slots[seq] * (keep > 0 ? keep : 1) * channels;
    const float* wc = w + (size_t)ch * taps;
    for (int i = first; i < last; ++i) {
        float y = add_input ? to_f32(x[(size_t)(row0 + i) * x_stride + ch]) : 0.f;
        if (bias)
            y += bias[ch];
        for (int j = 0; j < taps; ++j) {
            const int m = i - keep + j;                    // token of the sequence's step, or before it
            const float v = m >= 0 ? to_f32(x[(size_t)(row0 + m) * x_stride + ch])
                                   : to_f32(hist[(size_t)(keep + m) * channels + ch]);
            y = fmaf(wc[j], v, y);
        }
        out[(size_t)(row0 + i) * out_stride + ch] = from_f32<TX>(act >= 0 ? activate(y, act) : y);
    }
    if (first == 0) {
        // new history = the last `keep` entries of [old history ; this step's inputs], oldest first;
        // entry m is read from further along than it is written to, so ascending order is safe
        for (int m = 0; m < keep; ++m) {
            const int at = q_len + m;                      // index into the joined sequence
            hist[(size_t)m * channels + ch] = at < keep ? hist[(size_t)at * channels + ch]
                                                        : x[(size_t)(row0 + at - keep) * x_stride + ch];
        }
    }
}

// The same with 16 bytes of channels per thread (eight bfloat16 or four 32-bit values) and the
// weights transposed ([taps, channels], so that a thread's weights of one tap lie side by side):
// the scalar kernel moved 0.5 TB/s, a fifteenth of what the memory can.
template <typename T> struct Pack;
template <> struct Pack<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4])
    {
        const float4 q = *reinterpret_cast<const float4*>(p);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4])
    {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Pack<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8])
    {
        const uint4 q = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __low2float(h[i]);
            v[2 * i + 1] = __high2float(h[i]);
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8])
    {
        uint4 q;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = q;
    }
};

template <typename TX>
__global__ void __launch_bounds__(128)
short_conv_wide_kernel(const TX* __restrict__ x, long long x_stride, const float* __restrict__ wt, TX* history,
                       TX* __restrict__ out, long long out_stride, const int* __restrict__ q_start,
                       const int* __restrict__ slots, int channels, int taps, int chunk,
                       const float* __restrict__ bias, int act, int add_input)
{
    pdl_enter();
    constexpr int N = Pack<TX>::N;
    const int ch = (blockIdx.x * blockDim.x + threadIdx.x) * N;
    const int seq = blockIdx.z;
    const int row0 = q_start[seq];
    const int q_len = q_start[seq + 1] - row0;
    const int first = blockIdx.y * chunk;
    if (ch >= channels || first >= q_len)
        return;
    const int keep = taps - 1;
    const int last = min(first + chunk, q_len);
    TX* hist = history + (size_t)slots[seq] * (keep > 0 ? keep : 1) * channels;
    for (int i = first; i < last; ++i) {
        float y[N];
        if (add_input) {
            Pack<TX>::load(x + (size_t)(row0 + i) * x_stride + ch, y);
        } else {
#pragma unroll
            for (int e = 0; e < N; ++e)
                y[e] = 0.f;
        }
        if (bias) {
#pragma unroll
            for (int e = 0; e < N; ++e)
                y[e] += bias[ch + e];
        }
        for (int j = 0; j < taps; ++j) {
            const int m = i - keep + j;
            float v[N], w[N];
            Pack<TX>::load(m >= 0 ? x + (size_t)(row0 + m) * x_stride + ch : hist + (size_t)(keep + m) * channels + ch, v);
#pragma unroll
            for (int e = 0; e < N; e += 4)
                Pack<float>::load(wt + (size_t)j * channels + ch + e, *reinterpret_cast<float(*)[4]>(&w[e]));
#pragma unroll
            for (int e = 0; e < N; ++e)
                y[e] = fmaf(w[e], v[e], y[e]);
        }
        if (act >= 0) {
#pragma unroll
            for (int e = 0; e < N; ++e)
                y[e] = activate(y[e], act);
        }
        Pack<TX>::store(out + (size_t)(row0 + i) * out_stride + ch, y);
    }
    if (first == 0) {
        for (int m = 0; m < keep; ++m) {
            const int at = q_len + m;
            float v[N];
            Pack<TX>::load(at < keep ? hist + (size_t)at * channels + ch : x + (size_t)(row0 + at - keep) * x_stride + ch, v);
            Pack<TX>::store(hist + (size_t)m * channels + ch, v);
        }
    }
}

// ---------------------------------------------------------------- delta rule
constexpr int DELTA_LANES = 8;        // threads that share a value column (its key rows in equal parts)
constexpr int DELTA_WARPS = 4;        // warps that run the recurrence
constexpr int DELTA_PRODUCERS = 8;    // warps that make the next chunk's vectors meanwhile
constexpr int DELTA_THREADS = (DELTA_WARPS + DELTA_PRODUCERS) * 32;
constexpr int DELTA_CHUNK = 16;       // most tokens whose vectors are in shared memory at a time

struct DeltaParams {
    const void* proj;                 // [T, stride]: r | k | v | gate | removal | low, heads * d each but low
    long long stride;
    const float* decay_logits;        // [T, heads * d] = tanh(low) W2^T, made before this kernel (a matrix product
                                      // for many tokens, decay_logits_kernel for few)
    const float* decay_bias;          // [heads * d]
    const float* removal_bias;        // [heads * d]
    float* state;                     // [slots, heads, d (value), d (key)]
    float* o;                         // [T, heads * d]
    const int* q_start;
    const int* slots;
    int heads, d, rank, chunk;
    int late_trigger;                 // several chunks: the kernel after this one is let in only at the end
    float decay_scale, key_eps;
};

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }

// grid (column blocks, heads, sequences), four warps.  A thread owns R key rows (rows
// part * R .. part * R + R - 1; rows beyond d are zeros) of CPT neighbouring value columns; the
// eight threads of a column group sit side by side in a warp, a warp holds four groups, a CTA
// 16 * CPT columns.  Several columns to a thread, because every thread reads the same five
// vectors of a token from shared memory: with one column each, those reads (20 KB a token and
// CTA) bound the kernel.  The sequence's tokens are taken in chunks, and the warps have two
// roles.  Eight producer warps turn a chunk's projections into the five vectors of each token
// (decay, rate * unit key, unit key, key, receptance) in one of two buffers in shared memory,
// several tokens to a warp with their loads in flight together; meanwhile the four warps of the
// recurrence walk over the chunk before, each thread on its part of the state, which stays in
// registers from the sequence's first token of the step to its last.  One block barrier a chunk.
// (Alone, the vectors of 2,048 tokens of 16 heads take 0.77 ms and the recurrence 0.60 ms; one
// after the other they took 1.35 ms.)
//
// A sequence of many tokens keeps its CTAs busy for milliseconds.  The kernel that follows must not
// be let in at the start, as the short kernels do it: its CTAs would sit on the SMs waiting and
// take issue slots from the recurrence (a prompt of 2,048 tokens took 38 ms instead of 6).  With
// several chunks the kernel therefore triggers its dependents after the last token.
template <int R, int CPT, typename TX>
__global__ void __launch_bounds__(DELTA_THREADS) delta_rule_kernel(const DeltaParams p)
{
#ifdef CHIBI_TIMELINE
    pdl_enter();
#else
    if (!p.late_trigger)
        pdl_trigger();
    pdl_wait();
#endif
    extern __shared__ __align__(16) float smem[];
    constexpr int DP = R * DELTA_LANES;                     // padded head size
    constexpr int COLS = 16 * CPT;                          // value columns of this CTA
    constexpr int TPW = DELTA_CHUNK / DELTA_PRODUCERS;      // tokens a producer warp prepares per chunk
    const int d = p.d, W = p.heads * d;
    const int head = blockIdx.y, seq = blockIdx.z;
    const int row0 = p.q_start[seq];
    const int q_len = p.q_start[seq + 1] - row0;
    if (q_len <= 0)
        return;
    const bool producer = threadIdx.x >= DELTA_WARPS * 32;
    const int warp = producer ? (threadIdx.x >> 5) - DELTA_WARPS : threadIdx.x >> 5;     // the index within the role
    const int lane = threadIdx.x & 31;
    const int part = lane & (DELTA_LANES - 1);
    const int cta_col0 = blockIdx.x * COLS;
    const int my_col0 = cta_col0 + (warp * 4 + (lane >> 3)) * CPT;       // this thread's first column
    // shared: per token of the chunk [decay | rate * u | u | k | r] (DP each), then v (COLS)
    const int per_token = 5 * DP + COLS;
    const TX* proj = static_cast<const TX*>(p.proj);

    float S[CPT][R];
    float* st = p.state + ((size_t)p.slots[seq] * p.heads + head) * d * d;
    if (!producer) {
#pragma unroll
        for (int j = 0; j < CPT; ++j)
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const int row = part * R + i, col = my_col0 + j;
                S[j][i] = (col < d && row < d) ? st[(size_t)col * d + row] : 0.f;
            }
    }
    float* const buffers = smem;
    const int buffer_floats = p.chunk * per_token;

    // turn c = -1: the producers fill buffer 0 with chunk 0; turn c >= 0: they fill the other buffer
    // with chunk c + 1 while the recurrence walks over chunk c
    const int chunks = (q_len + p.chunk - 1) / p.chunk;
    for (int c = -1; c < chunks; ++c) {
        if (producer) {
        const int base = (c + 1) * p.chunk;
        const int n = min(p.chunk, q_len - base);           // <= 0 after the last chunk
        float* const smem = buffers + ((c + 1) & 1) * buffer_floats;
        if (n > 0) {
        // ---- the chunk's vectors: producer warp w takes tokens w, w + 4, ...
        float inv[TPW];
#pragma unroll
        for (int u = 0; u < TPW; ++u)
            inv[u] = 0.f;
        for (int c = lane; c < d; c += 32) {
            float k[TPW];
#pragma unroll
            for (int u = 0; u < TPW; ++u) {
                const int tt = warp + DELTA_PRODUCERS * u;
                k[u] = tt < n ? to_f32(proj[(size_t)(row0 + base + tt) * p.stride + W + head * d + c]) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < TPW; ++u)
                inv[u] = fmaf(k[u], k[u], inv[u]);
        }
#pragma unroll
        for (int u = 0; u < TPW; ++u)
            inv[u] = 1.f / sqrtf(warp_sum(inv[u]) + p.key_eps);
        for (int c = lane; c < DP; c += 32) {
            const int f = head * d + c;
            float z[TPW], kk[TPW], rr[TPW], aa[TPW];
#pragma unroll
            for (int u = 0; u < TPW; ++u) {
                const int tt = warp + DELTA_PRODUCERS * u;
                z[u] = kk[u] = rr[u] = aa[u] = 0.f;
                if (tt < n && c < d) {
                    const TX* row = proj + (size_t)(row0 + base + tt) * p.stride;
                    kk[u] = to_f32(row[W + f]);
                    rr[u] = to_f32(row[f]);
                    aa[u] = to_f32(row[4 * (size_t)W + f]);
                    z[u] = p.decay_logits[(size_t)(row0 + base + tt) * W + f];
                }
            }
            const float wb = c < d ? p.decay_bias[f] : 0.f, ab = c < d ? p.removal_bias[f] : 0.f;
#pragma unroll
            for (int u = 0; u < TPW; ++u) {
                const int tt = warp + DELTA_PRODUCERS * u;
                if (tt < n) {
                    float* v5 = smem + (size_t)tt * per_token;
                    const float unit = kk[u] * inv[u];
                    v5[c] = c < d ? expf(-p.decay_scale * sigmoidf_(z[u] + wb)) : 0.f;
                    v5[DP + c] = c < d ? sigmoidf_(aa[u] + ab) * unit : 0.f;
                    v5[2 * DP + c] = unit;
                    v5[3 * DP + c] = kk[u];
                    v5[4 * DP + c] = rr[u];
                }
            }
        }
#pragma unroll
        for (int u = 0; u < TPW; ++u) {
            const int tt = warp + DELTA_PRODUCERS * u;
            if (tt < n)
                for (int c = lane; c < COLS; c += 32)
                    smem[(size_t)tt * per_token + 5 * DP + c] = cta_col0 + c < d
                        ? to_f32(proj[(size_t)(row0 + base + tt) * p.stride + 2 * (size_t)W + head * d + cta_col0 + c]) : 0.f;
        }
        }
        } else if (c >= 0) {
        const int base = c * p.chunk;
        const int n = min(p.chunk, q_len - base);
        const float* const smem = buffers + (c & 1) * buffer_floats;
        // ---- the recurrence over the chunk.  A token's turn is a chain: u . S over the thread's
        // rows, three shuffles, the update, S . r, three shuffles.  The state of the next token
        // needs the first half only, so the sum over the lanes of S . r is put off by one token:
        // its shuffles are issued beside those of the next token's u . S and wait with them.
        float acc_prev[CPT];
        int o_prev = -1;                                    // the token whose S . r is still to be added up
#pragma unroll
        for (int j = 0; j < CPT; ++j)
            acc_prev[j] = 0.f;
        for (int tt = 0; tt <= n; ++tt) {
            const bool live = tt < n;
            const int at = live ? tt : n - 1;
            const float* v5 = smem + (size_t)at * per_token + part * R;
            const float* vv = smem + (size_t)at * per_token + 5 * DP + (my_col0 - cta_col0);
            float dot[CPT], dot2[CPT], acc[CPT], acc2[CPT], v[CPT];
#pragma unroll
            for (int j = 0; j < CPT; ++j) {
                dot[j] = dot2[j] = acc[j] = acc2[j] = 0.f;
                v[j] = vv[j];
            }
            if (live) {
#pragma unroll
                for (int i = 0; i < R; i += 4) {
                    const float4 u = *reinterpret_cast<const float4*>(v5 + 2 * DP + i);
#pragma unroll
                    for (int j = 0; j < CPT; ++j) {
                        dot[j] = fmaf(u.x, S[j][i], fmaf(u.y, S[j][i + 1], dot[j]));
                        dot2[j] = fmaf(u.z, S[j][i + 2], fmaf(u.w, S[j][i + 3], dot2[j]));
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < CPT; ++j)
                dot[j] += dot2[j];
#pragma unroll
            for (int step = 1; step < DELTA_LANES; step <<= 1) {
#pragma unroll
                for (int j = 0; j < CPT; ++j) {
                    const float a = __shfl_xor_sync(0xffffffffu, dot[j], step);
                    const float b = __shfl_xor_sync(0xffffffffu, acc_prev[j], step);
                    dot[j] += a;
                    acc_prev[j] += b;
                }
            }
            if (o_prev >= 0 && part == 0) {
                float* dst = p.o + (size_t)(row0 + base + o_prev) * W + head * d + my_col0;
#pragma unroll
                for (int j = 0; j < CPT; ++j)
                    if (my_col0 + j < d)
                        dst[j] = acc_prev[j];
            }
            if (!live)
                break;
#pragma unroll
            for (int i = 0; i < R; i += 4) {
                const float4 w = *reinterpret_cast<const float4*>(v5 + i);
                const float4 au = *reinterpret_cast<const float4*>(v5 + DP + i);
                const float4 k = *reinterpret_cast<const float4*>(v5 + 3 * DP + i);
                const float4 r = *reinterpret_cast<const float4*>(v5 + 4 * DP + i);
#pragma unroll
                for (int j = 0; j < CPT; ++j) {
                    S[j][i] = fmaf(k.x, v[j], fmaf(w.x, S[j][i], -au.x * dot[j]));
                    S[j][i + 1] = fmaf(k.y, v[j], fmaf(w.y, S[j][i + 1], -au.y * dot[j]));
                    S[j][i + 2] = fmaf(k.z, v[j], fmaf(w.z, S[j][i + 2], -au.z * dot[j]));
                    S[j][i + 3] = fmaf(k.w, v[j], fmaf(w.w, S[j][i + 3], -au.w * dot[j]));
                    acc[j] = fmaf(S[j][i], r.x, fmaf(S[j][i + 1], r.y, acc[j]));
                    acc2[j] = fmaf(S[j][i + 2], r.z, fmaf(S[j][i + 3], r.w, acc2[j]));
                }
            }
#pragma unroll
            for (int j = 0; j < CPT; ++j)
                acc_prev[j] = acc[j] + acc2[j];
            o_prev = tt;
        }
        }
        __syncthreads();                                    // the next chunk's vectors are there, this chunk's buffer is free
    }
#ifndef CHIBI_TIMELINE
    if (p.late_trigger)
        pdl_trigger();
#endif
    if (!producer) {
#pragma unroll
        for (int j = 0; j < CPT; ++j)
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const int row = part * R + i, col = my_col0 + j;
                if (col < d && row < d)
                    st[(size_t)col * d + row] = S[j][i];
            }
    }
}

// ---------------------------------------------------------------- the decay's logits for few tokens
// out[t, f] = sum_j tanh(low[t, j]) * w2t[j, f]: grid (blocks of 128 channels, tokens).  For steps of
// few tokens (one launch; the channels of a warp lie side by side in w2t); many tokens take a
// matrix product on the tensor cores instead.
template <typename TX>
__global__ void __launch_bounds__(128)
decay_logits_kernel(const TX* __restrict__ low, long long low_stride, const float* __restrict__ w2t,
                    float* __restrict__ out, int W, int rank)
{
    pdl_enter();
    extern __shared__ float low_s[];
    const int t = blockIdx.y, f = blockIdx.x * 128 + threadIdx.x;
    for (int j = threadIdx.x; j < rank; j += 128)
        low_s[j] = tanhf(to_f32(low[(size_t)t * low_stride + j]));
    __syncthreads();
    if (f >= W)
        return;
    float z = 0.f;
    for (int j0 = 0; j0 < rank; j0 += 8) {
        float w[8];
#pragma unroll
        for (int q = 0; q < 8; ++q)
            w[q] = j0 + q < rank ? w2t[(size_t)(j0 + q) * W + f] : 0.f;
#pragma unroll
        for (int q = 0; q < 8; ++q)
            z = fmaf(w[q], j0 + q < rank ? low_s[j0 + q] : 0.f, z);
    }
    out[(size_t)t * W + f] = z;
}

// ---------------------------------------------------------------- gated group norm
// One warp per (row, group): out = x / sqrt(mean(x^2 over the group) + eps) * weight * sigmoid(gate).
template <typename TG, typename TO>
__global__ void gated_group_norm_kernel(const float* __restrict__ x, const TG* __restrict__ gate,
                                        long long gate_stride, const float* __restrict__ weight,
                                        TO* __restrict__ out, long long rows, int groups, int n, float eps)
{
    pdl_enter();
    const long long job = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (job >= rows * groups)
        return;
    const long long row = job / groups;
    const int g = (int)(job - row * groups);
    const float* src = x + ((size_t)row * groups + g) * n;
    float s = 0.f;
    for (int j = lane; j < n; j += 32)
        s = fmaf(src[j], src[j], s);
    s = warp_sum(s);
    const float inv = 1.f / sqrtf(s / (float)n + eps);
    const TG* gr = gate + (size_t)row * gate_stride + (size_t)g * n;
    TO* dst = out + ((size_t)row * groups + g) * n;
    for (int j = lane; j < n; j += 32)
        dst[j] = from_f32<TO>(src[j] * inv * weight[g * n + j] * sigmoidf_(to_f32(gr[j])));
}

// Groups of 32, 64 or 128 features: LANES = n / 4 threads side by side own a group, four features
// each (16-byte loads of x and the weight), so a warp takes 32 / LANES groups at once.
template <typename T> struct Four;
template <> struct Four<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) { Pack<float>::load(p, v); }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) { Pack<float>::store(p, v); }
};
template <> struct Four<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4])
    {
        const uint2 q = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
        v[0] = __low2float(h[0]); v[1] = __high2float(h[0]); v[2] = __low2float(h[1]); v[3] = __high2float(h[1]);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4])
    {
        uint2 q;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
        h[0] = __floats2bfloat162_rn(v[0], v[1]);
        h[1] = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(p) = q;
    }
};

template <int LANES, typename TG, typename TO>
__global__ void __launch_bounds__(256)
gated_group_norm_four_kernel(const float* __restrict__ x, const TG* __restrict__ gate, long long gate_stride,
                             const float* __restrict__ weight, TO* __restrict__ out, long long rows, int groups,
                             float eps)
{
    pdl_enter();
    constexpr int n = 4 * LANES;
    const long long job = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / LANES;
    const int sub = threadIdx.x % LANES;
    const bool live = job < rows * groups;            // whole sub-groups are live or not; shuffles need all lanes
    const long long row = live ? job / groups : 0;
    const int g = live ? (int)(job - row * groups) : 0;
    float v[4], gt[4], w[4];
    Four<float>::load(x + ((size_t)row * groups + g) * n + 4 * sub, v);
    Four<TG>::load(gate + (size_t)row * gate_stride + (size_t)g * n + 4 * sub, gt);
    Four<float>::load(weight + (size_t)g * n + 4 * sub, w);
    float s = fmaf(v[0], v[0], fmaf(v[1], v[1], fmaf(v[2], v[2], v[3] * v[3])));
#pragma unroll
    for (int step = 1; step < LANES; step <<= 1)
        s += __shfl_xor_sync(0xffffffffu, s, step);
    const float inv = 1.f / sqrtf(s / (float)n + eps);
#pragma unroll
    for (int e = 0; e < 4; ++e)
        v[e] = v[e] * inv * w[e] * sigmoidf_(gt[e]);
    if (live)
        Four<TO>::store(out + ((size_t)row * groups + g) * n + 4 * sub, v);
}

// ---------------------------------------------------------------- row-wise helpers
__global__ void scale_kernel(float* __restrict__ x, float factor, long long total)
{
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x)
        x[i] *= factor;
}

template <typename TX, typename TO>
__global__ void cast_rows_kernel(const TX* __restrict__ x, long long x_stride, TO* __restrict__ out,
                                 long long out_stride, long long rows, int n, int act)
{
    pdl_enter();
    const long long total = rows * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / n;
        const int c = (int)(i - r * n);
        const float v = to_f32(x[(size_t)r * x_stride + c]);
        out[(size_t)r * out_stride + c] = from_f32<TO>(act >= 0 ? activate(v, act) : v);
    }
}

__global__ void add_row_vector_kernel(float* __restrict__ acc, long long stride, const float* __restrict__ vec,
                                      long long rows, int n)
{
    pdl_enter();
    const long long total = rows * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / n;
        const int c = (int)(i - r * n);
        acc[(size_t)r * stride + c] += vec[c];
    }
}

template <typename TX>
__global__ void activation_kernel(TX* __restrict__ x, long long total, int kind)
{
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x)
        x[i] = from_f32<TX>(activate(to_f32(x[i]), kind));
}

// bfloat16, eight values a thread; the result is rounded to bfloat16 at once, so the exact gelu may
// take the cheaper formula (activate_rounded)
__global__ void activation_bf16x8_kernel(__nv_bfloat16* __restrict__ x, long long groups, int kind)
{
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < groups;
         i += (long long)gridDim.x * blockDim.x) {
        float v[8];
        Pack<__nv_bfloat16>::load(x + 8 * i, v);
#pragma unroll
        for (int e = 0; e < 8; ++e)
            v[e] = activate_rounded(v[e], kind);
        Pack<__nv_bfloat16>::store(x + 8 * i, v);
    }
}

// out = act(sum over the splits of a split product's partial sums [splits][total])
template <typename TO>
__global__ void reduce_activation_kernel(const float* __restrict__ partial, int splits, long long total,
                                         TO* __restrict__ out, int kind)
{
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        float s = partial[i];
        for (int sp = 1; sp < splits; ++sp)
            s += partial[(size_t)sp * total + i];
        out[i] = from_f32<TO>(activate(s, kind));
    }
}

static int blocks_for(long long total, int block)
{
    long long b = (total + block - 1) / block;
    const long long cap = 148LL * 16;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

} // namespace chibi

using namespace chibi;

// `w`: [channels, taps]; `wt` (may be null): the same transposed, [taps, channels], for the kernel
// that takes 16 bytes of channels per thread (taken when the sizes and addresses allow it).
// `bias` (may be null) is added to every sum, `act` (an activation's code, -1: none) applied to it; with
// `add_input` the sum starts from the token's own input (y_t = x_t + ...), else from zero.
CHIBI_API int chibi_causal_conv(const void* x, int x_type, long long x_stride, const float* w, const float* wt,
                                void* history, void* out, long long out_stride, const int* q_start, const int* slots,
                                int seqs, int max_q_len, int channels, int taps, const float* bias, int act,
                                int add_input, cudaStream_t stream)
{
    if (seqs <= 0 || max_q_len <= 0)
        return CHIBI_OK;
    if (channels <= 0 || taps < 1)
        return CHIBI_ERR_ARGUMENT;
    // tokens per thread: at least the history's length (see the kernel); few, so that a prompt gives
    // every SM enough threads to hide the loads (16 tokens a thread moved 1.5 TB/s at 4,096 channels)
    const int chunk = taps - 1 > 4 ? taps - 1 : 4;
    const long long chunks = ((long long)max_q_len + chunk - 1) / chunk;
    if (chunks > 65535 || seqs > 65535)
        return CHIBI_ERR_UNSUPPORTED;
    const int per = x_type == CHIBI_BF16 ? 8 : 4;          // channels in 16 bytes
    const bool wide = wt != nullptr && channels % per == 0 && x_stride % per == 0 && out_stride % per == 0
        && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(history)
             | reinterpret_cast<uintptr_t>(wt)) & 15) == 0;
    if (wide) {
        const int threads = channels / per;
        const dim3 grid((unsigned)((threads + 127) / 128), (unsigned)chunks, (unsigned)seqs);
        CHIBI_DISPATCH_TYPE(x_type, TX, {
            launch(short_conv_wide_kernel<TX>, grid, dim3(128), 0, stream, (const TX*)x, x_stride, wt, (TX*)history,
                   (TX*)out, out_stride, q_start, slots, channels, taps, chunk, bias, act, add_input);
        });
        return launch_status();
    }
    const dim3 grid((unsigned)((channels + 127) / 128), (unsigned)chunks, (unsigned)seqs);
    CHIBI_DISPATCH_TYPE(x_type, TX, {
        launch(short_conv_kernel<TX>, grid, dim3(128), 0, stream, (const TX*)x, x_stride, w, (TX*)history, (TX*)out,
               out_stride, q_start, slots, channels, taps, chunk, bias, act, add_input);
    });
    return launch_status();
}

CHIBI_API int chibi_short_conv(const void* x, int x_type, long long x_stride, const float* w, const float* wt,
                               void* history, void* out, long long out_stride, const int* q_start, const int* slots,
                               int seqs, int max_q_len, int channels, int taps, cudaStream_t stream)
{
    return chibi_causal_conv(x, x_type, x_stride, w, wt, history, out, out_stride, q_start, slots, seqs, max_q_len,
                             channels, taps, nullptr, -1, 1, stream);
}

template <int R, int CPT, typename TX>
static int launch_delta(const DeltaParams& p, int seqs, int max_q_len, cudaStream_t stream)
{
    constexpr int DP = R * DELTA_LANES;
    constexpr int COLS = 16 * CPT;
    const int per_token = 5 * DP + COLS;
    // two buffers of `chunk` tokens each, within 96 KB a CTA (two CTAs to an SM)
    int chunk = (int)((96 * 1024) / (2 * per_token * sizeof(float)));
    if (chunk < 1)
        return CHIBI_ERR_UNSUPPORTED;
    chunk = chunk > DELTA_CHUNK ? DELTA_CHUNK : chunk;
    chunk = chunk > max_q_len ? max_q_len : chunk;
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(delta_rule_kernel<R, CPT, TX>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (e != cudaSuccess)
            return (int)e;
        configured = true;
    }
    DeltaParams q = p;
    q.chunk = chunk;
    q.late_trigger = max_q_len > chunk ? 1 : 0;
    const dim3 grid((unsigned)((p.d + COLS - 1) / COLS), (unsigned)p.heads, (unsigned)seqs);
    launch(delta_rule_kernel<R, CPT, TX>, grid, dim3(DELTA_THREADS), (size_t)2 * chunk * per_token * sizeof(float), stream,
           q);
    return launch_status();
}

CHIBI_API int chibi_delta_rule(const void* proj, int x_type, long long stride,
                               const float* decay_logits, const float* decay_bias, const float* removal_bias,
                               float* state, float* o, const int* q_start, const int* slots, int seqs,
                               int max_q_len, int heads, int d, int rank, float decay_scale, float key_eps,
                               cudaStream_t stream)
{
    if (seqs <= 0 || max_q_len <= 0)
        return CHIBI_OK;
    if (heads <= 0 || d <= 0 || rank <= 0 || !decay_logits)
        return CHIBI_ERR_ARGUMENT;
    if (d > 256 || heads > 65535 || seqs > 65535)
        return CHIBI_ERR_UNSUPPORTED;
    DeltaParams p = { proj, stride, decay_logits, decay_bias, removal_bias, state, o, q_start, slots,
                      heads, d, rank, 0, 0, decay_scale, key_eps };
    const int rows = (d + DELTA_LANES - 1) / DELTA_LANES;
    // Columns per thread: one.  More of them (the five vectors of a token are then read once for
    // several columns) were measured and lose: a warp then issues 350 instructions a token, one
    // every 5.6 cycles with nothing beside it on its scheduler, and a token's turn is what bounds
    // a prompt (2,048 tokens of 16 heads: 1.72 ms with four columns a thread).
    CHIBI_DISPATCH_TYPE(x_type, TX, {
        if (rows <= 4)
            return launch_delta<4, 1, TX>(p, seqs, max_q_len, stream);
        if (rows <= 8)
            return launch_delta<8, 1, TX>(p, seqs, max_q_len, stream);
        if (rows <= 12)
            return launch_delta<12, 1, TX>(p, seqs, max_q_len, stream);
        if (rows <= 16)
            return launch_delta<16, 1, TX>(p, seqs, max_q_len, stream);
        if (rows <= 24)
            return launch_delta<24, 1, TX>(p, seqs, max_q_len, stream);
        return launch_delta<32, 1, TX>(p, seqs, max_q_len, stream);
    });
    return CHIBI_OK;
}

CHIBI_API int chibi_decay_logits(const void* low, int x_type, long long low_stride, const float* w2t, float* out,
                                 long long tokens, int W, int rank, cudaStream_t stream)
{
    if (tokens <= 0)
        return CHIBI_OK;
    if (W <= 0 || rank <= 0)
        return CHIBI_ERR_ARGUMENT;
    if (tokens > 65535)
        return CHIBI_ERR_UNSUPPORTED;
    const dim3 grid((unsigned)((W + 127) / 128), (unsigned)tokens);
    CHIBI_DISPATCH_TYPE(x_type, TX, {
        launch(decay_logits_kernel<TX>, grid, dim3(128), (size_t)rank * sizeof(float), stream, (const TX*)low, low_stride,
               w2t, out, W, rank);
    });
    return launch_status();
}

CHIBI_API int chibi_gated_group_norm(const float* x, const void* gate, int gate_type, long long gate_stride,
                                     const float* weight, void* out, int out_type, long long rows, int groups,
                                     int n, float eps, cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    if (groups <= 0 || n <= 0)
        return CHIBI_ERR_ARGUMENT;
    const long long jobs = rows * groups;
    const long long blocks = (jobs + 3) / 4;
    if (blocks > 2147483647LL)
        return CHIBI_ERR_UNSUPPORTED;
    const int per_gate = gate_type == CHIBI_BF16 ? 8 : 16, per_out = out_type == CHIBI_BF16 ? 8 : 16;
    if ((n == 32 || n == 64 || n == 128) && gate_stride % 4 == 0
        && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(weight) & 15) == 0
        && (reinterpret_cast<uintptr_t>(gate) % per_gate) == 0 && (reinterpret_cast<uintptr_t>(out) % per_out) == 0) {
        const long long threads = jobs * (n / 4);
        const dim3 grid((unsigned)((threads + 255) / 256));
        CHIBI_DISPATCH_TYPE(gate_type, TG, CHIBI_DISPATCH_TYPE(out_type, TO, {
            if (n == 32)
                launch(gated_group_norm_four_kernel<8, TG, TO>, grid, dim3(256), 0, stream, x, (const TG*)gate,
                       gate_stride, weight, (TO*)out, rows, groups, eps);
            else if (n == 64)
                launch(gated_group_norm_four_kernel<16, TG, TO>, grid, dim3(256), 0, stream, x, (const TG*)gate,
                       gate_stride, weight, (TO*)out, rows, groups, eps);
            else
                launch(gated_group_norm_four_kernel<32, TG, TO>, grid, dim3(256), 0, stream, x, (const TG*)gate,
                       gate_stride, weight, (TO*)out, rows, groups, eps);
        }));
        return launch_status();
    }
    CHIBI_DISPATCH_TYPE(gate_type, TG, CHIBI_DISPATCH_TYPE(out_type, TO, {
        launch(gated_group_norm_kernel<TG, TO>, dim3((unsigned)blocks), dim3(128), 0, stream, x, (const TG*)gate,
               gate_stride, weight, (TO*)out, rows, groups, n, eps);
    }));
    return launch_status();
}

CHIBI_API int chibi_scale(float* x, float factor, long long total, cudaStream_t stream)
{
    if (total <= 0)
        return CHIBI_OK;
    launch(scale_kernel, dim3(blocks_for(total, 256)), dim3(256), 0, stream, x, factor, total);
    return launch_status();
}

// `act`: -1 none, else the activation by that code is applied on the way.
CHIBI_API int chibi_cast_rows(const void* x, int x_type, long long x_stride, void* out, int out_type,
                              long long out_stride, long long rows, int n, int act, cudaStream_t stream)
{
    if (rows <= 0 || n <= 0)
        return CHIBI_OK;
    if (act < -1 || act > 4)
        return CHIBI_ERR_ARGUMENT;
    CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(out_type, TO, {
        launch(cast_rows_kernel<TX, TO>, dim3(blocks_for(rows * n, 256)), dim3(256), 0, stream, (const TX*)x, x_stride,
               (TO*)out, out_stride, rows, n, act);
    }));
    return launch_status();
}

CHIBI_API int chibi_add_row_vector(float* acc, long long stride, const float* vec, long long rows, int n,
                                   cudaStream_t stream)
{
    if (rows <= 0 || n <= 0)
        return CHIBI_OK;
    launch(add_row_vector_kernel, dim3(blocks_for(rows * n, 256)), dim3(256), 0, stream, acc, stride, vec, rows, n);
    return launch_status();
}

CHIBI_API int chibi_activation(void* x, int x_type, long long total, int kind, cudaStream_t stream)
{
    if (total <= 0)
        return CHIBI_OK;
    if (kind < 0 || kind > 4)
        return CHIBI_ERR_ARGUMENT;
    if (x_type == CHIBI_BF16 && total % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        launch(activation_bf16x8_kernel, dim3(blocks_for(total / 8, 256)), dim3(256), 0, stream, (__nv_bfloat16*)x,
               total / 8, kind);
        return launch_status();
    }
    CHIBI_DISPATCH_TYPE(x_type, TX, {
        launch(activation_kernel<TX>, dim3(blocks_for(total, 256)), dim3(256), 0, stream, (TX*)x, total, kind);
    });
    return launch_status();
}

CHIBI_API int chibi_reduce_activation(const float* partial, int splits, long long total, void* out, int out_type,
                                      int kind, cudaStream_t stream)
{
    if (total <= 0)
        return CHIBI_OK;
    if (kind < 0 || kind > 4 || splits < 1)
        return CHIBI_ERR_ARGUMENT;
    CHIBI_DISPATCH_TYPE(out_type, TO, {
        launch(reduce_activation_kernel<TO>, dim3(blocks_for(total, 256)), dim3(256), 0, stream, partial, splits, total,
               (TO*)out, kind);
    });
    return launch_status();
}
