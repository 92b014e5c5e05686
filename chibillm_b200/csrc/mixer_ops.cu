// Kernels of the parts that a layer with norms on its sublayers' outputs, a token shift,
// attention over cached latents, plain attention with biases / a norm over the whole
// projection / an output gate, a gated linear recurrence and experts chosen by a router are
// made of:
//
// * norm_rows: layer norm (mean taken off, variance = mean of the squared deviations, weight and
//   bias) or RMS norm of 32-bit rows; the result replaces, or is added to, a 32-bit residual, and
//   may be written in another type as well.
// * token_shift: h[t] = x[t] + (x[t - 1] - x[t]) * w; the token before a step's first comes from
//   the request's state, which then takes the step's last x.
// * latent_prepare: from a row c_q | c | k_rot: RMS norm of c_q -> array; RMS norm of c and the
//   rotation of k_rot -> one cache row k_rot | c.
// * qkv_bias_norm_append: from a row q | k | v | ...: biases, RMS norm over the WHOLE q and the
//   whole k (all heads at once, weights of that size), split-half rotation of every head's first
//   features if asked; q -> array, k and v -> cache pages.
// * sigmoid_gate: x *= sigmoid(g).
// * recurrence_gates / gated_recurrence: q' = silu(q), f = l + (1 - l) sigmoid(f + b), v, all
//   32-bit; then per head S <- diag(f) S + (1 - f) v^T, o = S^T q' over each sequence's tokens,
//   from and to the request's state.
// * router_top: the `top` largest of a row of router logits (ties to the lower index) and the
//   softmax over them.
//
// Sums, norms, angles, gates and states are 32-bit whatever the activations' type is.
#define CHIBI_UNIT mixer_ops
#define CHIBI_UNIT_ID 11
#include "common.cuh"

namespace chibi {

// ---------------------------------------------------------------- norm of rows
// One block per row.  A thread touches the same columns in every pass.
template <typename TW, typename TO>
__global__ void __launch_bounds__(256)
norm_rows_kernel(const float* __restrict__ y, const TW* __restrict__ w, const TW* __restrict__ b, float eps,
                 float offset, int centered, float* residual, TO* __restrict__ out, int n)
{
    pdl_enter();
    extern __shared__ float row[];
    __shared__ float red[33];
    const long long t = blockIdx.x;
    const float* yr = y + t * n;
    float s = 0.f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        const float v = yr[c];
        row[c] = v;
        s += v;
    }
    float mean = 0.f;
    if (centered)
        mean = block_sum(s, red) / (float)n;
    float ss = 0.f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        const float dv = row[c] - mean;
        ss = fmaf(dv, dv, ss);
    }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)n + eps);
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        float v = (row[c] - mean) * inv * (to_f32(w[c]) + offset);
        if (b)
            v += to_f32(b[c]);
        if (residual) {
            v += residual[t * n + c];
            residual[t * n + c] = v;
        }
        if (out)
            out[t * n + c] = from_f32<TO>(v);
    }
}

// ---------------------------------------------------------------- token shift
// One block per token.  Only the block of a sequence's first token of the step touches the state:
// every thread reads its columns of it and then replaces them by the step's last token's.
template <typename TO>
__global__ void __launch_bounds__(256)
token_shift_kernel(const float* __restrict__ x, const float* __restrict__ mix, float* __restrict__ state,
                   const int* __restrict__ q_start, const int* __restrict__ seq_of_token,
                   const int* __restrict__ state_slots, TO* __restrict__ out, int n)
{
    pdl_enter();
    const long long t = blockIdx.x;
    const int seq = seq_of_token[t];
    const int first = q_start[seq];
    const float* xr = x + t * n;
    TO* o = out + t * n;
    if (t > first) {
        const float* before = xr - n;
        for (int c = threadIdx.x; c < n; c += blockDim.x) {
            const float v = xr[c];
            o[c] = from_f32<TO>(fmaf(before[c] - v, mix[c], v));
        }
        return;
    }
    const long long last = q_start[seq + 1] - 1;
    float* st = state + (long long)state_slots[seq] * n;
    const float* xl = x + last * n;
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        const float v = xr[c];
        const float before = st[c];
        o[c] = from_f32<TO>(fmaf(before - v, mix[c], v));
        st[c] = xl[c];
    }
}

// ---------------------------------------------------------------- latents
// One block per token.  Row: q_rank | kv_rank | rot columns (the last two only with a cache).
template <typename TX, typename TC>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const TX* __restrict__ proj, long long stride, TX* __restrict__ cq, TC* __restrict__ k_cache,
                      const float* __restrict__ q_norm, const float* __restrict__ kv_norm, float eps,
                      const float* __restrict__ inv_freq, int q_rank, int kv_rank, int rot,
                      const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                      const int* __restrict__ seq_rows, const int* __restrict__ block_table, int table_stride,
                      int page_size, int num_pages, int* __restrict__ error)
{
    pdl_enter();
    __shared__ float red[33];
    const long long t = blockIdx.x;
    const TX* row = proj + t * stride;
    float ss = 0.f;
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) {
        const float v = to_f32(row[c]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    float inv = 1.f / sqrtf(ss / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x)
        cq[t * q_rank + c] = from_f32<TX>(to_f32(row[c]) * inv * q_norm[c]);
    if (!k_cache)
        return;
    const int pos = positions[t];
    const int seq = seq_of_token[t];
    const int table_row = seq_rows ? seq_rows[seq] : seq;
    const int page = block_table[(size_t)table_row * table_stride + pos / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && error)
            atomicExch(error, 2);
        return;
    }
    TC* dst = k_cache + ((long long)page * page_size + pos % page_size) * (rot + kv_rank);
    const TX* latent = row + q_rank;
    ss = 0.f;
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) {
        const float v = to_f32(latent[c]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    inv = 1.f / sqrtf(ss / (float)kv_rank + eps);
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x)
        dst[rot + c] = from_f32<TC>(to_f32(latent[c]) * inv * kv_norm[c]);
    const TX* shared = latent + kv_rank;
    const int half = rot >> 1;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[j], &sn, &cs);
        const float u = to_f32(shared[j]), v = to_f32(shared[j + half]);
        dst[j] = from_f32<TC>(u * cs - v * sn);
        dst[j + half] = from_f32<TC>(v * cs + u * sn);
    }
}

// ---------------------------------------------------------------- q | k | v: biases, whole norm, append
// One block per token; shared memory holds q | k with their biases in 32-bit.
template <typename TX, typename TC>
__global__ void __launch_bounds__(512)
qkv_bias_norm_append_kernel(const TX* __restrict__ proj, long long stride, TX* __restrict__ q_out,
                            TC* __restrict__ k_cache, TC* __restrict__ v_cache, const float* __restrict__ bias,
                            const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                            const float* __restrict__ inv_freq, int rot, const int* __restrict__ positions,
                            const int* __restrict__ seq_of_token, const int* __restrict__ seq_rows,
                            const int* __restrict__ block_table, int table_stride, int nq, int nkv, int d, int dv,
                            int page_size, int num_pages, int append, int* __restrict__ error)
{
    pdl_enter();
    extern __shared__ float buf[];
    __shared__ float red[33];
    const long long t = blockIdx.x;
    const TX* row = proj + t * stride;
    const int qw = nq * d, kw = append ? nkv * d : 0, vw = append ? nkv * dv : 0;
    float sq = 0.f, sk = 0.f;
    for (int c = threadIdx.x; c < qw + kw; c += blockDim.x) {
        const float v = to_f32(row[c]) + (bias ? bias[c] : 0.f);
        buf[c] = v;
        if (c < qw)
            sq = fmaf(v, v, sq);
        else
            sk = fmaf(v, v, sk);
    }
    if (q_norm) {
        sq = block_sum(sq, red);
        const float inv = 1.f / sqrtf(sq / (float)qw + eps);
        for (int c = threadIdx.x; c < qw; c += blockDim.x)
            buf[c] *= inv * q_norm[c];
    }
    if (k_norm && append) {
        sk = block_sum(sk, red);
        const float inv = 1.f / sqrtf(sk / (float)kw + eps);
        for (int c = qw + threadIdx.x; c < qw + kw; c += blockDim.x)
            buf[c] *= inv * k_norm[c - qw];
    }
    __syncthreads();
    const int pos = positions[t];
    if (rot > 0) {
        // k follows q in the buffer and both have heads of d features: head h starts at h * d
        const int half = rot >> 1;
        const int heads = nq + (append ? nkv : 0);
        for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
            const int h = i / half, j = i - h * half;
            float sn, cs;
            sincosf((float)pos * inv_freq[j], &sn, &cs);
            float* p = buf + (size_t)h * d;
            const float u = p[j], v = p[j + half];
            p[j] = u * cs - v * sn;
            p[j + half] = v * cs + u * sn;
        }
        __syncthreads();
    }
    for (int c = threadIdx.x; c < qw; c += blockDim.x)
        q_out[t * qw + c] = from_f32<TX>(buf[c]);
    if (!append)
        return;
    const int seq = seq_of_token[t];
    const int table_row = seq_rows ? seq_rows[seq] : seq;
    const int page = block_table[(size_t)table_row * table_stride + pos / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && error)
            atomicExch(error, 2);
        return;
    }
    const int slot = pos % page_size;
    for (int c = threadIdx.x; c < kw; c += blockDim.x) {
        const int h = c / d, j = c - h * d;
        k_cache[(((long long)page * nkv + h) * page_size + slot) * d + j] = from_f32<TC>(buf[qw + c]);
    }
    for (int c = threadIdx.x; c < vw; c += blockDim.x) {
        const int h = c / dv, j = c - h * dv;
        const float v = to_f32(row[qw + kw + c]) + (bias ? bias[qw + kw + c] : 0.f);
        v_cache[(((long long)page * nkv + h) * page_size + slot) * dv + j] = from_f32<TC>(v);
    }
}

// Four neighbouring columns of a row at once (V = 4) where the rows allow it, else one; grid (column
// blocks, rows): no division per element.
template <typename T, int V>
__device__ __forceinline__ void load_columns(float (&dst)[V], const T* src)
{
    if constexpr (V == 4 && sizeof(T) == 4) {
        const float4 x = *reinterpret_cast<const float4*>(src);
        dst[0] = x.x, dst[1] = x.y, dst[2] = x.z, dst[3] = x.w;
    } else if constexpr (V == 4) {
        const uint2 x = *reinterpret_cast<const uint2*>(src);
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&x.x);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
        dst[0] = __low2float(lo), dst[1] = __high2float(lo), dst[2] = __low2float(hi), dst[3] = __high2float(hi);
    } else {
        dst[0] = to_f32(src[0]);
    }
}

template <typename T, int V>
__device__ __forceinline__ void store_columns(T* dst, const float (&src)[V])
{
    if constexpr (V == 4 && sizeof(T) == 4) {
        *reinterpret_cast<float4*>(dst) = make_float4(src[0], src[1], src[2], src[3]);
    } else if constexpr (V == 4) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(src[0], src[1]), hi = __floats2bfloat162_rn(src[2], src[3]);
        uint2 x;
        x.x = *reinterpret_cast<const uint32_t*>(&lo), x.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst) = x;
    } else {
        dst[0] = from_f32<T>(src[0]);
    }
}

template <typename TX, int V>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(TX* __restrict__ x, const TX* __restrict__ gate, long long gate_stride, long long rows, int n)
{
    pdl_enter();
    const int c = (blockIdx.x * 256 + threadIdx.x) * V;
    if (c >= n)
        return;
    for (long long t = blockIdx.y; t < rows; t += gridDim.y) {
        float a[V], g[V];
        load_columns<TX, V>(a, x + t * n + c);
        load_columns<TX, V>(g, gate + t * gate_stride + c);
#pragma unroll
        for (int i = 0; i < V; ++i)
            a[i] = a[i] / (1.f + expf(-g[i]));
        store_columns<TX, V>(x + t * n + c, a);
    }
}

// ---------------------------------------------------------------- gated linear recurrence
// out [T, 2 kw + vw] 32-bit: silu(q) | l + (1 - l) sigmoid(f + b) | v, from a row q | f | v.
template <typename TX, int V>
__global__ void __launch_bounds__(256)
recurrence_gates_kernel(const TX* __restrict__ proj, long long stride, const float* __restrict__ bias,
                        const float* __restrict__ floor_, float* __restrict__ out, long long rows, int kw, int vw)
{
    pdl_enter();
    const int w = 2 * kw + vw;
    const int c = (blockIdx.x * 256 + threadIdx.x) * V;        // with V = 4, kw and vw are multiples of 4
    if (c >= w)
        return;
    float l[V], b[V];
    if (c >= kw && c < 2 * kw) {
#pragma unroll
        for (int i = 0; i < V; ++i)
            l[i] = floor_[c - kw + i], b[i] = bias[c - kw + i];
    }
    for (long long t = blockIdx.y; t < rows; t += gridDim.y) {
        float v[V];
        load_columns<TX, V>(v, proj + t * stride + c);
        if (c < kw) {
#pragma unroll
            for (int i = 0; i < V; ++i)
                v[i] = v[i] / (1.f + expf(-v[i]));
        } else if (c < 2 * kw) {
#pragma unroll
            for (int i = 0; i < V; ++i)
                v[i] = l[i] + (1.f - l[i]) / (1.f + expf(-(v[i] + b[i])));
        }
        store_columns<float, V>(out + t * w + c, v);
    }
}

// grid (blocks of COLS value columns, heads, sequences); one warp per value column, lane l with rows
// l R .. l R + R - 1 of the head's key rows of that column in registers, from the sequence's first token
// of the step to its last.  The tokens' q', f and v come through two buffers of shared memory in chunks
// of GR_CHUNK tokens, the next chunk on its way (cp.async) while this one runs.  A token's row in a
// buffer: q' of 32 R rows | f of 32 R rows | v of the block's columns; rows past d hold q' = 0 and
// f = 1, which leave state and sums as they are, so the loop over a whole chunk's tokens has no condition
// in it.  The tokens of a chunk that is not full go one by one.
constexpr int GR_CHUNK = 16;

__device__ __forceinline__ void gr_copy16(float* dst, const float* src)
{
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(src) : "memory");
}

__device__ __forceinline__ void gr_copy4(float* dst, const float* src)
{
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(a), "l"(src) : "memory");
}

template <int R>
__device__ __forceinline__ void gr_load_rows(float (&dst)[R], const float* src)
{
    if constexpr (R % 4 == 0) {
#pragma unroll
        for (int i = 0; i < R; i += 4) {
            const float4 x = *reinterpret_cast<const float4*>(src + i);
            dst[i] = x.x, dst[i + 1] = x.y, dst[i + 2] = x.z, dst[i + 3] = x.w;
        }
    } else if constexpr (R == 2) {
        const float2 x = *reinterpret_cast<const float2*>(src);
        dst[0] = x.x, dst[1] = x.y;
    } else {
#pragma unroll
        for (int i = 0; i < R; ++i)
            dst[i] = src[i];
    }
}

// Sums over the 32 lanes of N values per lane; lanes 2 k and 2 k + 1 end with value k's sum in a[0]
// (N = 16).  Every exchange halves the values a lane still carries: N + 2 exchanges instead of 5 N.
template <int N, int OFF>
__device__ __forceinline__ void gr_fold(float (&a)[GR_CHUNK], bool upper)
{
#pragma unroll
    for (int j = 0; j < N / 2; ++j) {
        const float send = upper ? a[j] : a[j + N / 2];
        const float keep = upper ? a[j + N / 2] : a[j];
        a[j] = keep + __shfl_xor_sync(0xffffffffu, send, OFF);
    }
}

template <int R, int COLS>
__global__ void __launch_bounds__(COLS * 32)
gated_recurrence_kernel(const float* __restrict__ qfv, float* __restrict__ state, float* __restrict__ out,
                        const int* __restrict__ q_start, const int* __restrict__ state_slots, int heads, int d, int e)
{
    static_assert(GR_CHUNK == 16, "the fold below is written for 16 tokens");
    pdl_enter();
    extern __shared__ __align__(16) float sm[];
    const int head = blockIdx.y, seq = blockIdx.z;
    const int t0 = q_start[seq], t1 = q_start[seq + 1];
    if (t1 <= t0)
        return;
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int col = blockIdx.x * COLS + warp;
    const int kw = heads * d, vw = heads * e;
    const int width = 2 * kw + vw;
    constexpr int THREADS = COLS * 32, PITCH = COLS + 1;
    constexpr int ROWS = 32 * R;                            // d rounded up to the warp's rows
    constexpr int PER_TOKEN = 2 * ROWS + COLS;
    float S[R];
    float* st = state + (((long long)state_slots[seq] * heads + head) * d) * e;
    // The block's piece of the state, d rows of COLS columns, comes and goes through shared memory:
    // sixteen neighbouring threads take a row's 64 bytes, where a lane's own rows lie a whole row apart.
    float* tile = sm + 2 * GR_CHUNK * PER_TOKEN;
    for (int i = tid; i < d * COLS; i += THREADS) {
        const int r = i / COLS, c = i % COLS;
        const int cc = blockIdx.x * COLS + c;
        tile[r * PITCH + c] = cc < e ? st[(long long)r * e + cc] : 0.f;
    }
    // rows past d, in both buffers, once: no copy ever writes there
    for (int i = tid; i < 2 * GR_CHUNK * (ROWS - d); i += THREADS) {
        const int tok = i / (ROWS - d), r = d + i % (ROWS - d);
        sm[tok * PER_TOKEN + r] = 0.f;
        sm[tok * PER_TOKEN + ROWS + r] = 1.f;
    }
    // 16 bytes a copy where every piece of a row starts on such a boundary, else 4
    const bool wide = d % 4 == 0 && e % 4 == 0 && (reinterpret_cast<uintptr_t>(qfv) & 15) == 0;
    auto fetch = [&](int first, float* buf) {
        const int count = min(GR_CHUNK, t1 - first);
        if (wide) {
            const int dq = d / 4, units = 2 * dq + COLS / 4;
            for (int i = tid; i < count * units; i += THREADS) {
                const int tok = i / units, u = i - tok * units;
                const float* src = qfv + (long long)(first + tok) * width;
                float* dst = buf + tok * PER_TOKEN;
                if (u < dq) {
                    src += head * d + 4 * u;
                    dst += 4 * u;
                } else if (u < 2 * dq) {
                    src += kw + head * d + 4 * (u - dq);
                    dst += ROWS + 4 * (u - dq);
                } else {
                    const int c = blockIdx.x * COLS + 4 * (u - 2 * dq);
                    src += 2 * kw + head * e + (c < e ? c : e - 4);
                    dst += 2 * ROWS + 4 * (u - 2 * dq);
                }
                gr_copy16(dst, src);
            }
        } else {
            const int units = 2 * d + COLS;
            for (int i = tid; i < count * units; i += THREADS) {
                const int tok = i / units, w = i - tok * units;
                const float* src = qfv + (long long)(first + tok) * width;
                float* dst = buf + tok * PER_TOKEN;
                if (w < d) {
                    src += head * d + w;
                    dst += w;
                } else if (w < 2 * d) {
                    src += kw + head * d + (w - d);
                    dst += ROWS + (w - d);
                } else {
                    const int c = blockIdx.x * COLS + (w - 2 * d);
                    src += 2 * kw + head * e + (c < e ? c : e - 1);
                    dst += 2 * ROWS + (w - 2 * d);
                }
                gr_copy4(dst, src);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(t0, sm);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int r = lane * R + i;
        S[i] = r < d ? tile[r * PITCH + warp] : 0.f;
    }
    const bool writes = (lane & 1) == 0 && col < e;
    int which = 0;
    for (int first = t0; first < t1; first += GR_CHUNK, which ^= 1) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();            // this chunk has arrived, and everyone has left the other buffer
        if (first + GR_CHUNK < t1)
            fetch(first + GR_CHUNK, sm + (which ^ 1) * GR_CHUNK * PER_TOKEN);
        const float* buf = sm + which * GR_CHUNK * PER_TOKEN;
        const int count = min(GR_CHUNK, t1 - first);
        if (count < GR_CHUNK) {
            // the sequence's last tokens (a decode step's only one): one by one, each summed at once
            for (int tok = 0; tok < count; ++tok) {
                float q[R], f[R];
                gr_load_rows<R>(q, buf + tok * PER_TOKEN + lane * R);
                gr_load_rows<R>(f, buf + tok * PER_TOKEN + ROWS + lane * R);
                const float v = buf[tok * PER_TOKEN + 2 * ROWS + warp];
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    S[i] = fmaf(f[i], S[i], (1.f - f[i]) * v);
                    acc = fmaf(S[i], q[i], acc);
                }
#pragma unroll
                for (int o = 16; o; o >>= 1)
                    acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (lane == 0 && col < e)
                    out[(long long)(first + tok) * vw + head * e + col] = acc;
            }
            break;
        }
        // The state's chain is one multiply-add per element and token.  A token's sum over the key rows
        // stays spread over the lanes until the chunk is through; the exchanges follow for all of them.
        float accs[GR_CHUNK];
#pragma unroll
        for (int tok = 0; tok < GR_CHUNK; ++tok) {
            float q[R], f[R];
            gr_load_rows<R>(q, buf + tok * PER_TOKEN + lane * R);
            gr_load_rows<R>(f, buf + tok * PER_TOKEN + ROWS + lane * R);
            const float v = buf[tok * PER_TOKEN + 2 * ROWS + warp];
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < R; ++i) {
                S[i] = fmaf(f[i], S[i], (1.f - f[i]) * v);
                acc = fmaf(S[i], q[i], acc);
            }
            accs[tok] = acc;
        }
        gr_fold<16, 16>(accs, lane & 16);
        gr_fold<8, 8>(accs, lane & 8);
        gr_fold<4, 4>(accs, lane & 4);
        gr_fold<2, 2>(accs, lane & 2);
        const float total = accs[0] + __shfl_xor_sync(0xffffffffu, accs[0], 1);
        const int tok = lane >> 1;
        if (writes)
            out[(long long)(first + tok) * vw + head * e + col] = total;
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int r = lane * R + i;
        if (r < d)
            tile[r * PITCH + warp] = S[i];       // everyone took its rows from here before the first chunk
    }
    __syncthreads();
    for (int i = tid; i < d * COLS; i += THREADS) {
        const int r = i / COLS, c = i % COLS;
        const int cc = blockIdx.x * COLS + c;
        if (cc < e)
            st[(long long)r * e + cc] = tile[r * PITCH + c];
    }
}

// ---------------------------------------------------------------- router
// One warp per token; shared memory: the warp's copy of its row.
constexpr int ROUTER_WARPS = 4;

__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_top_kernel(const float* __restrict__ logits, long long stride, int* __restrict__ chosen,
                  float* __restrict__ share, long long tokens, int experts, int top)
{
    pdl_enter();
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long t = (long long)blockIdx.x * ROUTER_WARPS + warp;
    if (t >= tokens)
        return;
    float* vals = sm + (size_t)warp * (experts + top);
    float* picked = vals + experts;
    for (int e = lane; e < experts; e += 32)
        vals[e] = logits[t * stride + e];
    __syncwarp();
    for (int s = 0; s < top; ++s) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float v = vals[e];
            if (v > best) {                                // a lane meets its experts in rising order
                best = v;
                at = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ov > best || (ov == best && oa < at)) {
                best = ov;
                at = oa;
            }
        }
        if (at == 0x7fffffff)
            at = s;                                        // a row without a finite number left
        if (lane == 0) {
            chosen[t * top + s] = at;
            picked[s] = best;
            vals[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0) {
        const float m = picked[0];
        float sum = 0.f;
        for (int s = 0; s < top; ++s)
            sum += expf(picked[s] - m);
        for (int s = 0; s < top; ++s)
            share[t * top + s] = expf(picked[s] - m) / sum;
    }
}


} // namespace chibi

using namespace chibi;

CHIBI_API int chibi_norm_rows(const float* y, const void* w, const void* b, int w_type, float eps, float offset,
                              int centered, float* residual, void* out, int out_type, long long rows, int n,
                              cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    if (!y || !w || n <= 0 || (!residual && !out))
        return CHIBI_ERR_ARGUMENT;
    const size_t smem = (size_t)n * sizeof(float);
    if (smem > 200 * 1024 || rows > 2147483647LL)
        return CHIBI_ERR_UNSUPPORTED;
    CHIBI_DISPATCH_TYPE(w_type, TW, CHIBI_DISPATCH_TYPE(out_type, TO, {
        auto kernel = norm_rows_kernel<TW, TO>;
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch(kernel, dim3((unsigned)rows), dim3(256), smem, stream, y, (const TW*)w, (const TW*)b, eps, offset,
               centered, residual, (TO*)out, n);
    }));
    return launch_status();
}

CHIBI_API int chibi_token_shift(const float* x, const float* mix, float* state, const int* q_start,
                                const int* seq_of_token, const int* state_slots, void* out, int out_type,
                                long long rows, int n, cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    if (!x || !mix || !state || !q_start || !seq_of_token || !state_slots || !out || n <= 0 || rows > 2147483647LL)
        return CHIBI_ERR_ARGUMENT;
    CHIBI_DISPATCH_TYPE(out_type, TO, {
        launch(token_shift_kernel<TO>, dim3((unsigned)rows), dim3(256), 0, stream, x, mix, state, q_start, seq_of_token,
               state_slots, (TO*)out, n);
    });
    return launch_status();
}

CHIBI_API int chibi_latent_prepare(const void* proj, int x_type, long long stride, void* cq, void* k_cache,
                                   int cache_type, const float* q_norm, const float* kv_norm, float eps,
                                   const float* inv_freq, int q_rank, int kv_rank, int rot, const int* positions,
                                   const int* seq_of_token, const int* seq_rows, const int* block_table,
                                   int table_stride, int page_size, int num_pages, long long rows, int* error,
                                   cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    if (!proj || !cq || !q_norm || q_rank <= 0 || rows > 2147483647LL)
        return CHIBI_ERR_ARGUMENT;
    if (k_cache && (!kv_norm || !inv_freq || !positions || !seq_of_token || !block_table || kv_rank <= 0 || rot <= 0
                    || rot % 2 || page_size <= 0))
        return CHIBI_ERR_ARGUMENT;
    CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(cache_type, TC, {
        launch(latent_prepare_kernel<TX, TC>, dim3((unsigned)rows), dim3(256), 0, stream, (const TX*)proj, stride,
               (TX*)cq, (TC*)k_cache, q_norm, kv_norm, eps, inv_freq, q_rank, kv_rank, rot, positions, seq_of_token,
               seq_rows, block_table, table_stride, page_size, num_pages, error);
    }));
    return launch_status();
}

CHIBI_API int chibi_qkv_bias_norm_append(const void* proj, int x_type, long long stride, void* q_out, void* k_cache,
                                         void* v_cache, int cache_type, const float* bias, const float* q_norm,
                                         const float* k_norm, float eps, const float* inv_freq, int rot,
                                         const int* positions, const int* seq_of_token, const int* seq_rows,
                                         const int* block_table, int table_stride, int nq, int nkv, int d, int dv,
                                         int page_size, int num_pages, long long rows, int* error, cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    const int append = k_cache != nullptr;
    if (!proj || !q_out || !positions || nq <= 0 || nkv <= 0 || d <= 0 || dv <= 0 || rot < 0 || rot % 2 || rot > d
        || (rot > 0 && !inv_freq) || rows > 2147483647LL)
        return CHIBI_ERR_ARGUMENT;
    if (append && (!v_cache || !seq_of_token || !block_table || page_size <= 0))
        return CHIBI_ERR_ARGUMENT;
    const size_t smem = (size_t)(nq + (append ? nkv : 0)) * d * sizeof(float);
    if (smem > 200 * 1024)
        return CHIBI_ERR_UNSUPPORTED;
    CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(cache_type, TC, {
        auto kernel = qkv_bias_norm_append_kernel<TX, TC>;
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch(kernel, dim3((unsigned)rows), dim3(512), smem, stream, (const TX*)proj, stride, (TX*)q_out,
               (TC*)k_cache, (TC*)v_cache, bias, q_norm, k_norm, eps, inv_freq, rot, positions, seq_of_token, seq_rows,
               block_table, table_stride, nq, nkv, d, dv, page_size, num_pages, append, error);
    }));
    return launch_status();
}

CHIBI_API int chibi_sigmoid_gate(void* x, const void* gate, int x_type, long long gate_stride, long long rows, int n,
                                 cudaStream_t stream)
{
    if (rows <= 0 || n <= 0)
        return CHIBI_OK;
    if (!x || !gate)
        return CHIBI_ERR_ARGUMENT;
    const size_t unit = x_type == CHIBI_F32 ? 16 : 8;       // bytes of four columns
    const bool wide = n % 4 == 0 && gate_stride % 4 == 0 && reinterpret_cast<uintptr_t>(x) % unit == 0
                      && reinterpret_cast<uintptr_t>(gate) % unit == 0;
    const unsigned row_blocks = (unsigned)(rows < 16384 ? rows : 16384);
    CHIBI_DISPATCH_TYPE(x_type, TX, {
        if (wide)
            launch(sigmoid_gate_kernel<TX, 4>, dim3((unsigned)((n / 4 + 255) / 256), row_blocks), dim3(256), 0, stream,
                   (TX*)x, (const TX*)gate, gate_stride, rows, n);
        else
            launch(sigmoid_gate_kernel<TX, 1>, dim3((unsigned)((n + 255) / 256), row_blocks), dim3(256), 0, stream,
                   (TX*)x, (const TX*)gate, gate_stride, rows, n);
    });
    return launch_status();
}

CHIBI_API int chibi_recurrence_gates(const void* proj, int x_type, long long stride, const float* bias,
                                     const float* floor_, float* out, long long rows, int kw, int vw,
                                     cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    if (!proj || !bias || !floor_ || !out || kw <= 0 || vw <= 0)
        return CHIBI_ERR_ARGUMENT;
    const int w = 2 * kw + vw;
    const size_t unit = x_type == CHIBI_F32 ? 16 : 8;
    const bool wide = kw % 4 == 0 && vw % 4 == 0 && stride % 4 == 0 && reinterpret_cast<uintptr_t>(proj) % unit == 0
                      && reinterpret_cast<uintptr_t>(out) % 16 == 0;
    const unsigned row_blocks = (unsigned)(rows < 16384 ? rows : 16384);
    CHIBI_DISPATCH_TYPE(x_type, TX, {
        if (wide)
            launch(recurrence_gates_kernel<TX, 4>, dim3((unsigned)((w / 4 + 255) / 256), row_blocks), dim3(256), 0,
                   stream, (const TX*)proj, stride, bias, floor_, out, rows, kw, vw);
        else
            launch(recurrence_gates_kernel<TX, 1>, dim3((unsigned)((w + 255) / 256), row_blocks), dim3(256), 0, stream,
                   (const TX*)proj, stride, bias, floor_, out, rows, kw, vw);
    });
    return launch_status();
}

CHIBI_API int chibi_gated_recurrence(const float* qfv, float* state, float* out, const int* q_start,
                                     const int* state_slots, int seqs, int heads, int d, int e, cudaStream_t stream)
{
    if (seqs <= 0)
        return CHIBI_OK;
    if (!qfv || !state || !out || !q_start || !state_slots || heads <= 0 || d <= 0 || e <= 0)
        return CHIBI_ERR_ARGUMENT;
    if (d > 32 * 8 || heads > 65535 || seqs > 65535)
        return CHIBI_ERR_UNSUPPORTED;
    // 16 columns a block; 8 where that would leave SMs without a block (each column's arithmetic is the same
    // either way)
    const bool narrow = 2LL * ((e + 15) / 16) * heads * seqs <= 148;
    const int cols = narrow ? 8 : 16;
    const dim3 grid((unsigned)((e + cols - 1) / cols), (unsigned)heads, (unsigned)seqs);
#define CHIBI_GR_LAUNCH_COLS(R, COLS)                                                                            \
    do {                                                                                                         \
        auto kernel = gated_recurrence_kernel<R, COLS>;                                                          \
        const size_t smem = ((size_t)2 * GR_CHUNK * (64 * R + COLS) + (size_t)d * (COLS + 1)) * sizeof(float);   \
        if (smem > 48 * 1024)                                                                                    \
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                \
        launch(kernel, grid, dim3(COLS * 32), smem, stream, qfv, state, out, q_start, state_slots, heads, d, e); \
    } while (0)
#define CHIBI_GR_LAUNCH(R)                                                                                       \
    do {                                                                                                         \
        if (narrow)                                                                                              \
            CHIBI_GR_LAUNCH_COLS(R, 8);                                                                          \
        else                                                                                                     \
            CHIBI_GR_LAUNCH_COLS(R, 16);                                                                         \
    } while (0)
    if (d <= 32)
        CHIBI_GR_LAUNCH(1);
    else if (d <= 64)
        CHIBI_GR_LAUNCH(2);
    else if (d <= 128)
        CHIBI_GR_LAUNCH(4);
    else
        CHIBI_GR_LAUNCH(8);
#undef CHIBI_GR_LAUNCH
#undef CHIBI_GR_LAUNCH_COLS
    return launch_status();
}

CHIBI_API int chibi_router_top(const float* logits, long long stride, int* chosen, float* share, long long tokens,
                               int experts, int top, cudaStream_t stream)
{
    if (tokens <= 0)
        return CHIBI_OK;
    if (!logits || !chosen || !share || experts <= 0 || top <= 0 || top > experts)
        return CHIBI_ERR_ARGUMENT;
    const size_t smem = (size_t)ROUTER_WARPS * (experts + top) * sizeof(float);
    if (smem > 48 * 1024)
        return CHIBI_ERR_UNSUPPORTED;
    const long long blocks = (tokens + ROUTER_WARPS - 1) / ROUTER_WARPS;
    if (blocks > 2147483647LL)
        return CHIBI_ERR_UNSUPPORTED;
    launch(router_top_kernel, dim3((unsigned)blocks), dim3(ROUTER_WARPS * 32), smem, stream, logits, stride, chosen,
           share, tokens, experts, top);
    return launch_status();
}
