// Kernels of the parts that a hybrid decoder (attention beside a state-space branch, looped layers,
// routed experts with always-on and identity experts) adds to the others:
//
// * bigram_embed: residual += table[(previous token * a + token * b) mod buckets], the previous token of a
//   step's first token taken from the request's state;
// * stream_enter: x += x0 + step vector (what precedes a pass of a group of layers that runs several times);
// * heads_prepare_append: per head of a q | k | v row: bias, RMS norm with a weight, rotation of the first
//   features, then q to an array and k, v to their pages; the value heads may be fewer than the key heads;
// * differential_combine: o = a1 - lambda a2 per head, divided by its root mean square, times a constant and
//   the head's sigmoid gate;
// * state_space_scan: S <- exp(-exp(A) dt) S + dt B x^T, y = S^T C + D x per head over a step's tokens, from the
//   request's state to the state it leaves; gated_group_rms: y silu(z) normalised in equal parts;
// * clamped_swish_gate: min(g, L) sigmoid(s min(g, L)) (clamp(u, -L, L) + 1);
// * router_choose: softmax over all router outputs, choice by score + correction among the best groups,
//   weights without the correction; identity_rows: the rows of the experts that return their input;
// * scaled_add_norm: residual += vec * delta and the next norm's output; add_weighted: acc += a A + b B.
//
// Statistics, gates, decays, step sizes and the state are 32-bit whatever the activations' type.
#define CHIBI_UNIT hybrid_ops
#define CHIBI_UNIT_ID 12
#include "common.cuh"

namespace chibi {

static inline unsigned blocks_of(long long work, int threads)
{
    long long b = (work + threads - 1) / threads;
    return (unsigned)(b < 1 ? 1 : (b > 1048576 ? 1048576 : b));
}

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---------------------------------------------------------------- bigram embedding
// One block per token.  The block of a sequence's first token of the step is the only reader of the
// request's kept token and, after reading it, its only writer (it stores the step's last token).
template <typename TW>
__global__ void __launch_bounds__(128)
bigram_embed_kernel(float* __restrict__ residual, const TW* __restrict__ table, const int* __restrict__ tokens,
                    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                    const int* __restrict__ q_start, const int* __restrict__ slots, int* kept, int n, int buckets,
                    long long mul_prev, long long mul_cur)
{
    pdl_enter();
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    const int first = q_start[seq];
    __shared__ int row_s;
    if (threadIdx.x == 0) {
        int prev = 0;
        if (t == first) {
            prev = kept[slots[seq]];
            kept[slots[seq]] = tokens[q_start[seq + 1] - 1];
        } else {
            prev = tokens[t - 1];
        }
        long long row = buckets;                       // a sequence's first token: the table's last row
        if (positions[t] > 0) {
            row = ((long long)prev * mul_prev + (long long)tokens[t] * mul_cur) % buckets;
            if (row < 0)
                row += buckets;
        }
        row_s = (int)row;
    }
    __syncthreads();
    const TW* src = table + (size_t)row_s * n;
    float* dst = residual + (size_t)t * n;
    for (int c = threadIdx.x; c < n; c += blockDim.x)
        dst[c] += to_f32(src[c]);
}

__global__ void stream_enter_kernel(float* __restrict__ x, const float* __restrict__ x0,
                                    const float* __restrict__ vec, long long total, int n)
{
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x)
        x[i] += (x0 ? x0[i] : 0.f) + (vec ? vec[i % n] : 0.f);
}

__global__ void add_weighted_kernel(float* __restrict__ acc, const float* __restrict__ a, float wa,
                                    const float* __restrict__ b, float wb, long long total)
{
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x)
        acc[i] += wa * a[i] + (b ? wb * b[i] : 0.f);
}

// ---------------------------------------------------------------- heads: bias, norm, rotation, append
// One warp per (token, job); the jobs of a token are its nq query heads, nk key heads and nv value heads.
// Shared memory: d floats per warp.
template <typename TX, typename TC>
__global__ void __launch_bounds__(128)
heads_prepare_append_kernel(const TX* __restrict__ proj, long long stride, const float* __restrict__ bias,
                            const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                            const float* __restrict__ inv_freq, int rot, const int* __restrict__ positions,
                            const int* __restrict__ seq_of_token, const int* __restrict__ seq_rows,
                            const int* __restrict__ table, long long table_stride, TX* __restrict__ q_out,
                            TC* __restrict__ k_cache, TC* __restrict__ v_cache, long long tokens, int nq, int nk,
                            int nv, int d, int dv, int page_size, int num_pages, int* __restrict__ error)
{
    pdl_enter();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int jobs = nq + (k_cache ? nk + nv : 0);
    const long long job = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (job >= tokens * jobs)
        return;
    const long long t = job / jobs;
    const int j = (int)(job - t * jobs);
    const int pos = positions[t];
    const TX* row = proj + (size_t)t * stride;
    long long slot_row = -1;                                     // (page, position in page) of this token
    if (j >= nq) {
        const int seq = seq_of_token[t];
        const int page = table[(size_t)(seq_rows ? seq_rows[seq] : seq) * table_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (error && lane == 0)
                atomicExch(error, 3);
            return;
        }
        slot_row = (long long)page;
    }
    if (j >= nq + nk) {                                          // a value head: bias and copy
        const int h = j - nq - nk;
        const int col0 = nq * d + nk * d + h * dv;
        TC* dst = v_cache + (((size_t)slot_row * nv + h) * page_size + pos % page_size) * dv;
        for (int c = lane; c < dv; c += 32)
            dst[c] = from_f32<TC>(to_f32(row[col0 + c]) + (bias ? bias[col0 + c] : 0.f));
        return;
    }
    const bool is_q = j < nq;
    const int col0 = is_q ? j * d : nq * d + (j - nq) * d;
    float* xs = smem + (size_t)warp * d;
    float ssq = 0.f;
    for (int c = lane; c < d; c += 32) {
        const float v = to_f32(row[col0 + c]) + (bias ? bias[col0 + c] : 0.f);
        xs[c] = v;
        ssq = fmaf(v, v, ssq);
    }
    const float* w = is_q ? q_norm : k_norm;
    if (w) {
        ssq = warp_sum(ssq);
        const float inv = 1.f / sqrtf(ssq / (float)d + eps);
        for (int c = lane; c < d; c += 32)
            xs[c] = xs[c] * inv * w[c];
    }
    __syncwarp();
    const int half = rot >> 1;
    for (int c = lane; c < half; c += 32) {
        float sn, cs;
        sincosf((float)pos * inv_freq[c], &sn, &cs);
        const float u = xs[c], v = xs[c + half];
        xs[c] = u * cs - v * sn;
        xs[c + half] = v * cs + u * sn;
    }
    __syncwarp();
    if (is_q) {
        TX* dst = q_out + ((size_t)t * nq + j) * d;
        for (int c = lane; c < d; c += 32)
            dst[c] = from_f32<TX>(xs[c]);
    } else {
        TC* dst = k_cache + (((size_t)slot_row * nk + (j - nq)) * page_size + pos % page_size) * d;
        for (int c = lane; c < d; c += 32)
            dst[c] = from_f32<TC>(xs[c]);
    }
}

// ---------------------------------------------------------------- differential attention: combine
// One warp per (token, head).  att [T, 2 heads, dv] float32 in the order the attention kernel wants: the
// heads of a key/value group side by side, first their first maps, then their second ones (group = heads
// per key/value head); gate: logits [T, *], column = head.
template <typename TX>
__global__ void __launch_bounds__(128)
differential_combine_kernel(const float* __restrict__ att, const TX* __restrict__ gate, long long gate_stride,
                            float lambda, float eps, float out_scale, TX* __restrict__ out, long long tokens,
                            int heads, int dv, int group)
{
    pdl_enter();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long job = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (job >= tokens * heads)
        return;
    const long long t = job / heads;
    const int h = (int)(job - t * heads);
    const float* a1 = att + ((size_t)t * 2 * heads + (size_t)(h / group) * 2 * group + h % group) * dv;
    const float* a2 = a1 + (size_t)group * dv;
    float ssq = 0.f;
    for (int c = lane; c < dv; c += 32) {
        const float o = a1[c] - lambda * a2[c];
        ssq = fmaf(o, o, ssq);
    }
    ssq = warp_sum(ssq);
    float f = out_scale / sqrtf(ssq / (float)dv + eps);
    if (gate)
        f *= sigmoid_f(to_f32(gate[(size_t)t * gate_stride + h]));
    TX* dst = out + ((size_t)t * heads + h) * dv;
    for (int c = lane; c < dv; c += 32)
        dst[c] = from_f32<TX>((a1[c] - lambda * a2[c]) * f);
}

// ---------------------------------------------------------------- state-space scan
// grid (blocks of COLS value columns, heads, sequences); a warp owns two neighbouring value columns, lane l
// of it with R of each column's state rows in registers from the sequence's first token of the step to its
// last (a token's B and C rows, which all columns share, are fetched from shared memory once for the two).
// The state is kept value column first: [slots, heads, e, N], so that a column's rows are one contiguous run.
// Tokens come in chunks of SSM_CHUNK through two buffers in shared memory (B and C of the head's group, rows
// padded with zeros to 32 R; the block's x columns; the step sizes and decays): the next chunk's loads are
// issued before the present chunk's arithmetic and stored after it, one block barrier a chunk.  In a full
// chunk the 32 sums over the lanes (16 tokens x 2 columns) are folded together after the chunk's last token:
// at every step of the butterfly a lane passes on the half of its sums that its partner keeps, 31 exchanges
// instead of 160, and lane l ends with the sum of token l / 2, column l % 2.  A token's turn is then 2 R
// multiply-adds a lane and column and nothing that waits for another lane; the warps of a block hide the
// shared-memory loads of one another.
constexpr int SSM_CHUNK = 16;
constexpr int SSM_CW = 2;                               // columns of a warp

// The state row that lane l holds as its i-th: runs of four rows to a lane where a lane has four or more
// (one 16-byte load of B and of C serves four multiply-adds), else row 32 i + l.
template <int R> __device__ __forceinline__ int ssm_row(int i, int l)
{
    return R >= 4 ? (i >> 2) * 128 + l * 4 + (i & 3) : i * 32 + l;
}

// COLS: value columns of a block: 16, or 8 where 16 would leave SMs without a block.
template <typename TX, int R, int COLS>
__global__ void __launch_bounds__(32 * COLS / SSM_CW)
state_space_scan_kernel(const TX* __restrict__ xbc, long long xbc_stride, const TX* __restrict__ dt_raw,
                        long long dt_stride, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                        const float* __restrict__ skip, float* state, float* __restrict__ y,
                        const int* __restrict__ q_start, const int* __restrict__ slots, int heads, int groups, int e,
                        int N)
{
    pdl_enter();
    constexpr int THREADS = 32 * COLS / SSM_CW;
    constexpr int RN = 32 * R;                          // padded rows of a token's B and C
    constexpr int PER = SSM_CHUNK * RN / THREADS;       // values of B (and of C) that a thread fetches a chunk
    constexpr int BUF = 2 * SSM_CHUNK * RN + SSM_CHUNK * COLS + 2 * SSM_CHUNK;
    static_assert(SSM_CHUNK * RN % THREADS == 0 && SSM_CHUNK * COLS <= THREADS && BUF % 4 == 0 && SSM_CHUNK == 16
                  && SSM_CW == 2, "a chunk's values divide evenly among the threads");
    extern __shared__ __align__(16) float smem[];
    const int h = blockIdx.y, seq = blockIdx.z;
    const int g = h / (heads / groups);
    const int inner = heads * e;
    const int col_local = (threadIdx.x >> 5) * SSM_CW, l = threadIdx.x & 31;
    const int col = blockIdx.x * COLS + col_local;      // the warp's first column
    const int row0 = q_start[seq];
    const int q_len = q_start[seq + 1] - row0;
    if (q_len <= 0)
        return;
    float* S = state + (((size_t)slots[seq] * heads + h) * e) * N;
    float s[SSM_CW][R];
#pragma unroll
    for (int w = 0; w < SSM_CW; ++w) {
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int r = ssm_row<R>(i, l);
            s[w][i] = (col + w < e && r < N) ? S[(size_t)(col + w) * N + r] : 0.f;
        }
    }
    const float A = -expf(a_log[h]), bias = dt_bias[h], D = skip[h];

    TX fb[PER], fc[PER], fx, fdt;                       // a chunk on its way from memory to shared memory
    auto fetch = [&](int c0) {
        const int n_tok = min(SSM_CHUNK, q_len - c0);
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int i = threadIdx.x + k * THREADS;
            const int tt = i / RN, r = i - tt * RN;
            fb[k] = fc[k] = from_f32<TX>(0.f);
            if (tt < n_tok && r < N) {
                const TX* src = xbc + (size_t)(row0 + c0 + tt) * xbc_stride + inner + g * N + r;
                fb[k] = src[0];
                fc[k] = src[(size_t)groups * N];
            }
        }
        fx = fdt = from_f32<TX>(0.f);
        if (threadIdx.x < SSM_CHUNK * COLS) {
            const int tt = threadIdx.x / COLS, cc = blockIdx.x * COLS + (threadIdx.x - tt * COLS);
            if (tt < n_tok && cc < e)
                fx = xbc[(size_t)(row0 + c0 + tt) * xbc_stride + h * e + cc];
        }
        if (threadIdx.x < n_tok)
            fdt = dt_raw[(size_t)(row0 + c0 + threadIdx.x) * dt_stride + h];
    };
    auto stash = [&](float* buf) {
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int i = threadIdx.x + k * THREADS;
            buf[i] = to_f32(fb[k]);
            buf[SSM_CHUNK * RN + i] = to_f32(fc[k]);
        }
        if (threadIdx.x < SSM_CHUNK * COLS)
            buf[2 * SSM_CHUNK * RN + threadIdx.x] = to_f32(fx);
        if (threadIdx.x < SSM_CHUNK) {
            const float dt = softplus_f(to_f32(fdt) + bias);
            buf[2 * SSM_CHUNK * RN + SSM_CHUNK * COLS + threadIdx.x] = dt;
            buf[2 * SSM_CHUNK * RN + SSM_CHUNK * COLS + SSM_CHUNK + threadIdx.x] = expf(A * dt);
        }
    };
    // one token's turn on this lane's rows of both columns: the state's update and the rows' part of S^T C
    auto turn = [&](const float* Bt, const float* Ct, float a, float bx0, float bx1, float& sum0, float& sum1) {
        sum0 = sum1 = 0.f;
        if constexpr (R >= 4) {
#pragma unroll
            for (int i = 0; i < R; i += 4) {
                const int r = ssm_row<R>(i, l);
                const float4 b4 = *reinterpret_cast<const float4*>(Bt + r);
                const float4 c4 = *reinterpret_cast<const float4*>(Ct + r);
                const float bv[4] = { b4.x, b4.y, b4.z, b4.w }, cv[4] = { c4.x, c4.y, c4.z, c4.w };
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    s[0][i + j] = fmaf(a, s[0][i + j], bx0 * bv[j]);
                    s[1][i + j] = fmaf(a, s[1][i + j], bx1 * bv[j]);
                    sum0 = fmaf(s[0][i + j], cv[j], sum0);
                    sum1 = fmaf(s[1][i + j], cv[j], sum1);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const int r = ssm_row<R>(i, l);
                const float bv = Bt[r], cv = Ct[r];
                s[0][i] = fmaf(a, s[0][i], bx0 * bv);
                s[1][i] = fmaf(a, s[1][i], bx1 * bv);
                sum0 = fmaf(s[0][i], cv, sum0);
                sum1 = fmaf(s[1][i], cv, sum1);
            }
        }
    };
    fetch(0);
    stash(smem);
    __syncthreads();
    int which = 0;
    for (int c0 = 0; c0 < q_len; c0 += SSM_CHUNK, which ^= 1) {
        const int n_tok = min(SSM_CHUNK, q_len - c0);
        const bool more = c0 + SSM_CHUNK < q_len;
        if (more)
            fetch(c0 + SSM_CHUNK);
        const float* buf = smem + which * BUF;
        const float* Bs = buf;
        const float* Cs = buf + SSM_CHUNK * RN;
        const float* xs = Cs + SSM_CHUNK * RN;
        const float* dts = xs + SSM_CHUNK * COLS;
        const float* decay = dts + SSM_CHUNK;
        if (n_tok == SSM_CHUNK) {
            float acc[SSM_CHUNK * SSM_CW];              // [token][column of the warp]
#pragma unroll
            for (int tt = 0; tt < SSM_CHUNK; ++tt)
                turn(Bs + tt * RN, Cs + tt * RN, decay[tt], dts[tt] * xs[tt * COLS + col_local],
                     dts[tt] * xs[tt * COLS + col_local + 1], acc[2 * tt], acc[2 * tt + 1]);
            // fold: after the steps 16, 8, 4, 2, 1 lane l holds the sum over all lanes of value l
#pragma unroll
            for (int half = SSM_CHUNK * SSM_CW / 2, o = 16; half >= 1; half >>= 1, o >>= 1) {
                const bool upper = (l & o) != 0;
#pragma unroll
                for (int k = 0; k < half; ++k) {
                    const float send = upper ? acc[k] : acc[k + half];
                    const float keep = upper ? acc[k + half] : acc[k];
                    acc[k] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                }
            }
            const int tt = l >> 1, w = l & 1;
            if (col + w < e)
                y[(size_t)(row0 + c0 + tt) * inner + h * e + col + w] = fmaf(D, xs[tt * COLS + col_local + w], acc[0]);
        } else {
            for (int tt = 0; tt < n_tok; ++tt) {
                const float xv0 = xs[tt * COLS + col_local], xv1 = xs[tt * COLS + col_local + 1];
                float a0, a1;
                turn(Bs + tt * RN, Cs + tt * RN, decay[tt], dts[tt] * xv0, dts[tt] * xv1, a0, a1);
                a0 = warp_sum(a0);
                a1 = warp_sum(a1);
                if (l < SSM_CW && col + l < e)
                    y[(size_t)(row0 + c0 + tt) * inner + h * e + col + l] = l ? fmaf(D, xv1, a1) : fmaf(D, xv0, a0);
            }
        }
        if (more)
            stash(smem + (which ^ 1) * BUF);
        __syncthreads();
    }
#pragma unroll
    for (int w = 0; w < SSM_CW; ++w) {
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int r = ssm_row<R>(i, l);
            if (col + w < e && r < N)
                S[(size_t)(col + w) * N + r] = s[w][i];
        }
    }
}

// grid (tokens, parts), out = v / rms(v over the part) * weight with v = y * silu(z).  A part of up to
// 256 * GGR_KEEP values stays in the threads' registers between the sum of squares and the output; a longer
// one is made a second time.
constexpr int GGR_KEEP = 8;

template <typename TX>
__global__ void __launch_bounds__(256)
gated_group_rms_kernel(const float* __restrict__ y, const TX* __restrict__ z, long long z_stride,
                       const float* __restrict__ weight, float eps, TX* __restrict__ out, int width, int part)
{
    pdl_enter();
    __shared__ float scratch[33];
    const size_t t = blockIdx.x;
    const int c0 = blockIdx.y * part;
    const bool kept = part <= 256 * GGR_KEEP;
    float v[GGR_KEEP];
    float ssq = 0.f;
    if (kept) {
#pragma unroll
        for (int k = 0; k < GGR_KEEP; ++k) {
            const int c = threadIdx.x + k * 256;
            v[k] = c < part ? y[t * width + c0 + c] * silu_f(to_f32(z[t * z_stride + c0 + c])) : 0.f;
            ssq = fmaf(v[k], v[k], ssq);
        }
    } else {
        for (int c = threadIdx.x; c < part; c += blockDim.x) {
            const float u = y[t * width + c0 + c] * silu_f(to_f32(z[t * z_stride + c0 + c]));
            ssq = fmaf(u, u, ssq);
        }
    }
    ssq = block_sum(ssq, scratch);
    const float inv = 1.f / sqrtf(ssq / (float)part + eps);
    if (kept) {
#pragma unroll
        for (int k = 0; k < GGR_KEEP; ++k) {
            const int c = threadIdx.x + k * 256;
            if (c < part)
                out[t * width + c0 + c] = from_f32<TX>(v[k] * inv * weight[c0 + c]);
        }
        return;
    }
    for (int c = threadIdx.x; c < part; c += blockDim.x) {
        const float u = y[t * width + c0 + c] * silu_f(to_f32(z[t * z_stride + c0 + c]));
        out[t * width + c0 + c] = from_f32<TX>(u * inv * weight[c0 + c]);
    }
}

// ---------------------------------------------------------------- dense feed-forward's gate
__device__ __forceinline__ float clamped_swish(float g, float u, float limit, float slope)
{
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * sigmoid_f(slope * g) * (u + 1.f);
}

template <typename TX>
__global__ void clamped_swish_gate_kernel(const TX* __restrict__ gate_up, long long stride, TX* __restrict__ out,
                                          long long rows, int n, float limit, float slope)
{
    pdl_enter();
    const long long total = rows * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / n;
        const int c = (int)(i - r * n);
        out[i] = from_f32<TX>(clamped_swish(to_f32(gate_up[r * stride + c]), to_f32(gate_up[r * stride + n + c]), limit,
                                            slope));
    }
}

// bfloat16, eight columns (16 bytes) a thread; n and the row stride are multiples of 8 and the arrays start on
// 16-byte boundaries
__global__ void clamped_swish_gate_wide_kernel(const __nv_bfloat16* __restrict__ gate_up, long long stride,
                                               __nv_bfloat16* __restrict__ out, long long rows, int n, float limit,
                                               float slope)
{
    pdl_enter();
    const int per_row = n / 8;
    const long long total = rows * per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / per_row;
        const int c = (int)(i - r * per_row) * 8;
        const uint4 graw = *reinterpret_cast<const uint4*>(gate_up + r * stride + c);
        const uint4 uraw = *reinterpret_cast<const uint4*>(gate_up + r * stride + n + c);
        const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&graw);
        const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uraw);
        uint4 oraw;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&oraw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(gh[j]), u = __bfloat1622float2(uh[j]);
            oh[j] = __floats2bfloat162_rn(clamped_swish(g.x, u.x, limit, slope), clamped_swish(g.y, u.y, limit, slope));
        }
        *reinterpret_cast<uint4*>(out + r * n + c) = oraw;
    }
}

// ---------------------------------------------------------------- router
// One warp per token.  Shared memory per warp: n scores, n choice scores.  chosen[t, s] is the s-th best
// router output (ties to the lower number), share[t, s] its softmax score times `scale`.
__global__ void __launch_bounds__(128)
router_choose_kernel(const float* __restrict__ logits, long long stride, const float* __restrict__ correction,
                     int* __restrict__ chosen, float* __restrict__ share, long long tokens, int n, int top,
                     int group_count, int group_keep, float scale, int last_choice)
{
    pdl_enter();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long t = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= tokens)
        return;
    float* score = smem + (size_t)warp * 2 * n;
    float* choice = score + n;
    const float* z = logits + (size_t)t * stride;
    float m = -INFINITY;
    for (int i = lane; i < n; i += 32)
        m = fmaxf(m, z[i]);
    m = warp_max(m);
    float sum = 0.f;
    for (int i = lane; i < n; i += 32) {
        const float p = expf(z[i] - m);
        score[i] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int i = lane; i < n; i += 32) {
        score[i] *= inv;
        choice[i] = score[i] + (correction ? correction[i] : 0.f);
    }
    __syncwarp();
    if (group_count > 1 && group_keep < group_count) {
        // a group's score is its best choice score; groups outside the best `group_keep` are closed.  The
        // groups' scores are few: every lane walks them all in the same order.
        const int per = n / group_count;
        unsigned long long keep_lo = 0, keep_hi = 0;            // up to 128 groups
        for (int k = 0; k < group_keep; ++k) {
            float best = -INFINITY;
            int best_g = -1;
            for (int g = 0; g < group_count; ++g) {
                if ((g < 64 ? keep_lo >> g : keep_hi >> (g - 64)) & 1ull)
                    continue;
                float gm = -INFINITY;
                for (int i = 0; i < per; ++i)
                    gm = fmaxf(gm, choice[g * per + i]);
                if (best_g < 0 || gm > best) {
                    best = gm;
                    best_g = g;
                }
            }
            if (best_g < 64)
                keep_lo |= 1ull << best_g;
            else
                keep_hi |= 1ull << (best_g - 64);
        }
        __syncwarp();
        for (int i = lane; i < n; i += 32) {
            const int g = i / per;
            if (!((g < 64 ? keep_lo >> g : keep_hi >> (g - 64)) & 1ull))
                choice[i] = -INFINITY;
        }
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_i = 0x7fffffff;
        for (int i = lane; i < n; i += 32) {
            const float c = choice[i];
            if (c > best || (best_i == 0x7fffffff && c == best)) {
                best = c;
                best_i = i;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ob > best || (ob == best && oi < best_i)) {
                best = ob;
                best_i = oi;
            }
        }
        if (best_i == 0x7fffffff)
            best_i = 0;
        if (lane == 0) {
            chosen[t * top + k] = best_i < last_choice ? best_i : last_choice;
            share[t * top + k] = score[best_i] * scale;
        }
        __syncwarp();
        if (lane == (best_i & 31))
            choice[best_i] = -INFINITY;
        __syncwarp();
        // a choice that was already taken has -inf and loses to any open one; with fewer open outputs
        // than `top` the rest would repeat output 0 with its score, which the host refuses at start-up
    }
}

// y[r] = x[token of row r] for the rows of bucket `bucket` of a route (the experts that return their input)
template <typename TX>
__global__ void identity_rows_kernel(const TX* __restrict__ x, long long x_stride, const int* __restrict__ offsets,
                                     const int* __restrict__ token_of_row, float* __restrict__ y, int n, int bucket)
{
    pdl_enter();
    const int r0 = offsets[bucket], r1 = offsets[bucket + 1];
    const long long total = (long long)(r1 - r0) * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = r0 + (int)(i / n);
        const int c = (int)(i % n);
        y[(size_t)r * n + c] = to_f32(x[(size_t)token_of_row[r] * x_stride + c]);
    }
}

// ---------------------------------------------------------------- residual += vec * delta, then a norm
// One block per token; shared memory: the row (n floats) and 33 sums.
template <typename TW, typename TO>
__global__ void __launch_bounds__(256)
scaled_add_norm_kernel(float* __restrict__ residual, const float* __restrict__ delta, const float* __restrict__ vec,
                       const TW* __restrict__ norm_w, float eps, float offset, TO* __restrict__ out, int n)
{
    pdl_enter();
    extern __shared__ float smem[];
    float* row = smem;
    float* scratch = smem + n;
    const size_t t = blockIdx.x;
    float ssq = 0.f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        const float v = fmaf(vec ? vec[c] : 1.f, delta[t * n + c], residual[t * n + c]);
        residual[t * n + c] = v;
        row[c] = v;
        ssq = fmaf(v, v, ssq);
    }
    if (!out)
        return;
    ssq = block_sum(ssq, scratch);
    const float inv = 1.f / sqrtf(ssq / (float)n + eps);
    for (int c = threadIdx.x; c < n; c += blockDim.x)
        out[t * n + c] = from_f32<TO>(row[c] * inv * (to_f32(norm_w[c]) + offset));
}

} // namespace chibi

using namespace chibi;

CHIBI_API int chibi_bigram_embed(float* residual, const void* table, int table_type, const int* tokens,
                                 const int* positions, const int* seq_of_token, const int* q_start, const int* slots,
                                 int* kept, long long num_tokens, int n, int buckets, long long mul_prev,
                                 long long mul_cur, cudaStream_t stream)
{
    if (num_tokens <= 0)
        return CHIBI_OK;
    if (!residual || !table || !tokens || !kept || n <= 0 || buckets <= 0 || num_tokens > 2147483647LL)
        return CHIBI_ERR_ARGUMENT;
    CHIBI_DISPATCH_TYPE(table_type, TW, {
        launch(bigram_embed_kernel<TW>, dim3((unsigned)num_tokens), dim3(128), 0, stream, residual, (const TW*)table,
               tokens, positions, seq_of_token, q_start, slots, kept, n, buckets, mul_prev, mul_cur);
    });
    return launch_status();
}

CHIBI_API int chibi_stream_enter(float* x, const float* x0, const float* vec, long long rows, int n,
                                 cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    if (!x || n <= 0)
        return CHIBI_ERR_ARGUMENT;
    launch(stream_enter_kernel, dim3(blocks_of(rows * n, 256)), dim3(256), 0, stream, x, x0, vec, rows * n, n);
    return launch_status();
}

CHIBI_API int chibi_add_weighted(float* acc, const float* a, float wa, const float* b, float wb, long long count,
                                 cudaStream_t stream)
{
    if (count <= 0)
        return CHIBI_OK;
    if (!acc || !a)
        return CHIBI_ERR_ARGUMENT;
    launch(add_weighted_kernel, dim3(blocks_of(count, 256)), dim3(256), 0, stream, acc, a, wa, b, wb, count);
    return launch_status();
}

CHIBI_API int chibi_heads_prepare_append(const void* proj, int x_type, long long stride, const float* bias,
                                         const float* q_norm, const float* k_norm, float eps, const float* inv_freq,
                                         int rot, const int* positions, const int* seq_of_token, const int* seq_rows,
                                         const int* table, long long table_stride, void* q_out, void* k_cache,
                                         void* v_cache, int cache_type, long long tokens, int nq, int nk, int nv, int d,
                                         int dv, int page_size, int num_pages, int* error, cudaStream_t stream)
{
    if (tokens <= 0)
        return CHIBI_OK;
    if (!proj || !q_out || nq <= 0 || d <= 0 || rot < 0 || rot > d || rot % 2 != 0 || (rot > 0 && !inv_freq)
        || (k_cache && (!v_cache || !table || nk <= 0 || nv <= 0 || dv <= 0 || page_size <= 0)))
        return CHIBI_ERR_ARGUMENT;
    if (d > 4096)
        return CHIBI_ERR_UNSUPPORTED;
    const int warps = 4;
    const long long jobs = tokens * (nq + (k_cache ? nk + nv : 0));
    const long long blocks = (jobs + warps - 1) / warps;
    if (blocks > 2147483647LL)
        return CHIBI_ERR_UNSUPPORTED;
    const size_t smem = (size_t)warps * d * sizeof(float);
    CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(cache_type, TC, {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(heads_prepare_append_kernel<TX, TC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem);
        launch(heads_prepare_append_kernel<TX, TC>, dim3((unsigned)blocks), dim3(warps * 32), smem, stream,
               (const TX*)proj, stride, bias, q_norm, k_norm, eps, inv_freq, rot, positions, seq_of_token, seq_rows,
               table, table_stride, (TX*)q_out, (TC*)k_cache, (TC*)v_cache, tokens, nq, nk, nv, d, dv, page_size,
               num_pages, error);
    }));
    return launch_status();
}

CHIBI_API int chibi_differential_combine(const float* att, const void* gate, int x_type, long long gate_stride,
                                         float lambda, float eps, float out_scale, void* out, long long tokens,
                                         int heads, int dv, int group, cudaStream_t stream)
{
    if (tokens <= 0)
        return CHIBI_OK;
    if (!att || !out || heads <= 0 || dv <= 0 || group <= 0 || heads % group != 0)
        return CHIBI_ERR_ARGUMENT;
    const long long blocks = (tokens * heads + 3) / 4;
    if (blocks > 2147483647LL)
        return CHIBI_ERR_UNSUPPORTED;
    CHIBI_DISPATCH_TYPE(x_type, TX, {
        launch(differential_combine_kernel<TX>, dim3((unsigned)blocks), dim3(128), 0, stream, att, (const TX*)gate,
               gate_stride, lambda, eps, out_scale, (TX*)out, tokens, heads, dv, group);
    });
    return launch_status();
}

template <typename TX, int R, int COLS>
static void launch_scan(int seqs, cudaStream_t stream, const void* xbc, long long xbc_stride,
                        const void* dt_raw, long long dt_stride, const float* dt_bias, const float* a_log,
                        const float* skip, float* state, float* y, const int* q_start, const int* slots, int heads,
                        int groups, int e, int N)
{
    const dim3 grid((unsigned)((e + COLS - 1) / COLS), (unsigned)heads, (unsigned)seqs);
    const size_t smem = (size_t)2 * (2 * SSM_CHUNK * R * 32 + SSM_CHUNK * COLS + 2 * SSM_CHUNK) * sizeof(float);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(state_space_scan_kernel<TX, R, COLS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    launch(state_space_scan_kernel<TX, R, COLS>, grid, dim3(32 * COLS / SSM_CW), smem, stream, (const TX*)xbc,
           xbc_stride, (const TX*)dt_raw, dt_stride, dt_bias, a_log, skip, state, y, q_start, slots, heads, groups, e, N);
}

CHIBI_API int chibi_state_space_scan(const void* xbc, int x_type, long long xbc_stride, const void* dt_raw,
                                     long long dt_stride, const float* dt_bias, const float* a_log, const float* skip,
                                     float* state, float* y, const int* q_start, const int* slots, int seqs, int heads,
                                     int groups, int e, int N, cudaStream_t stream)
{
    if (seqs <= 0)
        return CHIBI_OK;
    if (!xbc || !dt_raw || !dt_bias || !a_log || !skip || !state || !y || heads <= 0 || groups <= 0
        || heads % groups != 0 || e <= 0 || N <= 0)
        return CHIBI_ERR_ARGUMENT;
    if (N > 16 * 32 || heads > 65535 || seqs > 65535)      // (two buffers of a chunk's B and C must fit shared memory)
        return CHIBI_ERR_UNSUPPORTED;
    // blocks of 16 columns, or of 8 where those would leave SMs without a block
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const bool narrow = (long long)((e + 15) / 16) * heads * seqs < sms && e > 8;
    const int rows = (N + 31) / 32;
#define CHIBI_SCAN(RR)                                                                                       \
    CHIBI_DISPATCH_TYPE(x_type, TX, {                                                                        \
        if (narrow)                                                                                          \
            launch_scan<TX, RR, 8>(seqs, stream, xbc, xbc_stride, dt_raw, dt_stride, dt_bias, a_log, skip,  \
                                   state, y, q_start, slots, heads, groups, e, N);                          \
        else                                                                                                 \
            launch_scan<TX, RR, 16>(seqs, stream, xbc, xbc_stride, dt_raw, dt_stride, dt_bias, a_log, skip, \
                                    state, y, q_start, slots, heads, groups, e, N);                         \
    })
    if (rows <= 1) CHIBI_SCAN(1);
    else if (rows <= 2) CHIBI_SCAN(2);
    else if (rows <= 4) CHIBI_SCAN(4);
    else if (rows <= 8) CHIBI_SCAN(8);
    else {
        // larger states: blocks of 8 columns only (256 threads leave a thread the registers for its rows)
        CHIBI_DISPATCH_TYPE(x_type, TX, {
            launch_scan<TX, 16, 8>(seqs, stream, xbc, xbc_stride, dt_raw, dt_stride, dt_bias, a_log, skip, state, y,
                                   q_start, slots, heads, groups, e, N);
        });
    }
#undef CHIBI_SCAN
    return launch_status();
}

CHIBI_API int chibi_gated_group_rms(const float* y, const void* z, int x_type, long long z_stride,
                                    const float* weight, float eps, void* out, long long tokens, int width, int parts,
                                    cudaStream_t stream)
{
    if (tokens <= 0)
        return CHIBI_OK;
    if (!y || !z || !weight || !out || width <= 0 || parts <= 0 || width % parts != 0)
        return CHIBI_ERR_ARGUMENT;
    if (tokens > 2147483647LL || parts > 65535)
        return CHIBI_ERR_UNSUPPORTED;
    CHIBI_DISPATCH_TYPE(x_type, TX, {
        launch(gated_group_rms_kernel<TX>, dim3((unsigned)tokens, (unsigned)parts), dim3(256), 0, stream, y,
               (const TX*)z, z_stride, weight, eps, (TX*)out, width, width / parts);
    });
    return launch_status();
}

CHIBI_API int chibi_clamped_swish_gate(const void* gate_up, int x_type, long long stride, void* out, long long rows,
                                       int n, float limit, float slope, cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    if (!gate_up || !out || n <= 0 || !(limit > 0.f))
        return CHIBI_ERR_ARGUMENT;
    if (x_type == CHIBI_BF16 && n % 8 == 0 && stride % 8 == 0
        && ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        launch(clamped_swish_gate_wide_kernel, dim3(blocks_of(rows * (n / 8), 256)), dim3(256), 0, stream,
               (const __nv_bfloat16*)gate_up, stride, (__nv_bfloat16*)out, rows, n, limit, slope);
        return launch_status();
    }
    CHIBI_DISPATCH_TYPE(x_type, TX, {
        launch(clamped_swish_gate_kernel<TX>, dim3(blocks_of(rows * n, 256)), dim3(256), 0, stream,
               (const TX*)gate_up, stride, (TX*)out, rows, n, limit, slope);
    });
    return launch_status();
}

CHIBI_API int chibi_router_choose(const float* logits, long long stride, const float* correction, int* chosen,
                                  float* share, long long tokens, int n, int top, int group_count, int group_keep,
                                  float scale, int last_choice, cudaStream_t stream)
{
    if (tokens <= 0)
        return CHIBI_OK;
    if (!logits || !chosen || !share || n <= 0 || top <= 0 || top > n || group_count < 1 || group_keep < 1
        || group_keep > group_count || n % group_count != 0)
        return CHIBI_ERR_ARGUMENT;
    if (n > 2048 || group_count > 128)
        return CHIBI_ERR_UNSUPPORTED;
    const int warps = 4;
    const long long blocks = (tokens + warps - 1) / warps;
    if (blocks > 2147483647LL)
        return CHIBI_ERR_UNSUPPORTED;
    const size_t smem = (size_t)warps * 2 * n * sizeof(float);
    launch(router_choose_kernel, dim3((unsigned)blocks), dim3(warps * 32), smem, stream, logits, stride, correction,
           chosen, share, tokens, n, top, group_count, group_keep, scale, last_choice);
    return launch_status();
}

// `route` as chibi_route_by_table lays it out for `buckets` experts and `max_tiles` tiles
CHIBI_API int chibi_identity_rows(const void* x, int x_type, long long x_stride, const int* route, float* y,
                                  long long pairs, int buckets, int bucket, int max_tiles, int n, cudaStream_t stream)
{
    if (pairs <= 0)
        return CHIBI_OK;
    if (!x || !route || !y || n <= 0 || bucket < 0 || bucket >= buckets)
        return CHIBI_ERR_ARGUMENT;
    const int* offsets = route;
    const int* token_of_row = route + buckets + 1 + 2 * pairs + 2 * (long long)max_tiles;
    CHIBI_DISPATCH_TYPE(x_type, TX, {
        // (how many rows the bucket holds is known on the device only: a grid that fills the SMs, whatever it is)
        const unsigned blocks = blocks_of(pairs * n, 256);
        launch(identity_rows_kernel<TX>, dim3(blocks < 1184u ? blocks : 1184u), dim3(256), 0, stream, (const TX*)x,
               x_stride, offsets, token_of_row, y, n, bucket);
    });
    return launch_status();
}

CHIBI_API int chibi_scaled_add_norm(float* residual, const float* delta, const float* vec, const void* norm_w,
                                    int w_type, float eps, float offset, void* out, int out_type, long long rows,
                                    int n, cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    if (!residual || !delta || n <= 0 || (out && !norm_w) || rows > 2147483647LL)
        return CHIBI_ERR_ARGUMENT;
    const size_t smem = ((size_t)n + 33) * sizeof(float);
    if (smem > 200 * 1024)
        return CHIBI_ERR_UNSUPPORTED;
    CHIBI_DISPATCH_TYPE(w_type, TW, CHIBI_DISPATCH_TYPE(out_type, TO, {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(scaled_add_norm_kernel<TW, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem);
        launch(scaled_add_norm_kernel<TW, TO>, dim3((unsigned)rows), dim3(256), smem, stream, residual, delta, vec,
               (const TW*)norm_w, eps, offset, (TO*)out, n);
    }));
    return launch_status();
}
