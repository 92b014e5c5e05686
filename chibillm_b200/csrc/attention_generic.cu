// Causal grouped-query attention over the paged cache, any head size up to
// 1,024, any group size, optional window; element types are template parameters.
//
// This is the attention of the true 32-bit path and the fall-back of the
// bfloat16 path for head sizes the tensor-core kernels do not cover.  One warp
// owns one (token, query head).  Keys are visited in position order in chunks
// of 32: lane l scores key base+l (dot product over d in 32-bit, scaled after
// the sum), the chunk joins the running softmax (m, l, acc rescaled by
// exp(m_old - m_new)), then every lane accumulates its features of the values.
// The order of operations of a row depends only on its own position, never on
// the batch around it.
//
// Query token i of sequence s sits at position ctx_len[s] - q_len[s] + i and
// sees keys max(0, pos - window + 1) .. pos (window 0 = all); with chunk > 0 only those of its own
// block of `chunk` positions, counted from the sequence's start.  Keys have d features, values dv
// (the two caches are [pages, kv heads, page, d] and [.., dv]; the output rows have nq * dv).
//
// Options of the score: a soft cap c (0 = off) replaces s by c * tanh(s / c); a bias by
// distance (r1, r2 per query head, null = off) then takes r1 * ln(1 + r2 * (pos - key)) off.
// A sink (one number per query head, null = off) joins the softmax's denominator as exp(sink): the
// running maximum starts at the sink and the running sum at one, with nothing accumulated for it.
// With r2 null the bias is linear in the distance: r1 * (pos - key).  `kv_share` consecutive key heads
// share one value head (the value cache then has nkv / kv_share heads); the output may be 32-bit
// whatever the queries' type.
#define CHIBI_UNIT attention_generic
#define CHIBI_UNIT_ID 4
#include "common.cuh"

namespace chibi {

constexpr int MAX_D = 1024;      // head sizes up to 256 keep 8 sums per lane, larger ones 32

template <typename TQ, typename TC, typename TO, int SLOTS>
__global__ void __launch_bounds__(128)
attention_generic_kernel(const TQ* __restrict__ q, const TC* __restrict__ k_cache,
                         const TC* __restrict__ v_cache, TO* __restrict__ out,
                         const int* __restrict__ block_table, int table_stride,
                         const int* __restrict__ q_start, const int* __restrict__ ctx_len,
                         const int* __restrict__ seq_of_token, const int* __restrict__ seq_rows,
                         const int* __restrict__ positions,
                         long long tokens, int nq, int nkv, int d, int dv, int page_size, int num_pages,
                         float scale, int window, int chunk, float softcap, const float* __restrict__ bias_r1,
                         const float* __restrict__ bias_r2, const float* __restrict__ sink,
                         int kv_share, int* __restrict__ error)
{
    pdl_enter();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long job = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (job >= tokens * nq)
        return;
    const long long t = job / nq;
    const int head = (int)(job - t * nq);
    const int kv_head = head / (nq / nkv);
    const int seq = seq_of_token[t];
    const int pos = positions[t];
    float* qs = smem + (size_t)warp * d;
    const TQ* qrow = q + ((size_t)t * nq + head) * d;
    for (int j = lane; j < d; j += 32)
        qs[j] = to_f32(qrow[j]);
    __syncwarp();

    const int first = first_visible_key(pos, window, chunk);
    const float r1 = bias_r1 ? bias_r1[head] : 0.f, r2 = bias_r2 ? bias_r2[head] : 0.f;
    const int nv = nkv / kv_share, v_head = kv_head / kv_share;
    const int* table = block_table + (size_t)(seq_rows ? seq_rows[seq] : seq) * table_stride;
    float acc[SLOTS];
#pragma unroll
    for (int i = 0; i < SLOTS; ++i)
        acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    if (sink) {
        m = sink[head];
        l = 1.f;
    }

    for (int base = first; base <= pos; base += 32) {
        const int u = base + lane;
        float s = -INFINITY;
        long long row_off = -1, v_off = -1;
        if (u <= pos) {
            const int page = table[u / page_size];
            if (page < 0 || page >= num_pages) {
                if (error)
                    atomicExch(error, 3);
            } else {
                row_off = ((long long)page * nkv + kv_head) * page_size + (u % page_size);
                v_off = ((long long)page * nv + v_head) * page_size + (u % page_size);
                const TC* krow = k_cache + row_off * d;
                float dot = 0.f;
                for (int j = 0; j < d; ++j)
                    dot = fmaf(qs[j], to_f32(krow[j]), dot);
                s = dot * scale;
                if (softcap > 0.f)
                    s = softcap * tanhf(s / softcap);
                if (bias_r1)
                    s -= bias_r2 ? r1 * log1pf(r2 * (float)(pos - u)) : r1 * (float)(pos - u);
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        // m_new is finite: the chunk holds at least the key at `base`, unless its page is bad.
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < SLOTS; ++i)
            acc[i] *= corr;
        m = m_new;
        const int n = (pos - base + 1 < 32) ? pos - base + 1 : 32;
        for (int kk = 0; kk < n; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            const long long off = __shfl_sync(0xffffffffu, v_off, kk);
            if (off < 0)
                continue;
            const TC* vrow = v_cache + off * dv;
#pragma unroll
            for (int i = 0; i < SLOTS; ++i) {
                const int j = lane + 32 * i;
                if (j < dv)
                    acc[i] = fmaf(pk, to_f32(vrow[j]), acc[i]);
            }
        }
    }
    TO* orow = out + ((size_t)t * nq + head) * dv;
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < SLOTS; ++i) {
        const int j = lane + 32 * i;
        if (j < dv)
            orow[j] = from_f32<TO>(acc[i] * inv);
    }
}

} // namespace chibi

using namespace chibi;

CHIBI_API int chibi_attention_generic(const void* q, int q_type, const void* k_cache,
                                      const void* v_cache, int cache_type, void* out,
                                      const int* block_table, int table_stride,
                                      const int* q_start, const int* ctx_len,
                                      const int* seq_of_token, const int* seq_rows,
                                      const int* positions,
                                      long long tokens, int nq, int nkv, int d, int dv, int page_size,
                                      int num_pages, float scale, int window, int chunk, float softcap,
                                      const float* bias_r1, const float* bias_r2, const float* sink,
                                      int* error, cudaStream_t stream);

CHIBI_API int chibi_attention_generic_shared(const void* q, int q_type, const void* k_cache,
                                             const void* v_cache, int cache_type, void* out, int out_type,
                                             const int* block_table, int table_stride,
                                             const int* q_start, const int* ctx_len,
                                             const int* seq_of_token, const int* seq_rows,
                                             const int* positions,
                                             long long tokens, int nq, int nkv, int d, int dv, int page_size,
                                             int num_pages, float scale, int window, int chunk, float softcap,
                                             const float* bias_r1, const float* bias_r2, const float* sink,
                                             int kv_share, int* error, cudaStream_t stream)
{
    if (tokens <= 0)
        return CHIBI_OK;
    if (d <= 0 || d > MAX_D || dv <= 0 || dv > MAX_D || nkv <= 0 || nq % nkv != 0 || window < 0 || chunk < 0 || softcap < 0.f || (bias_r2 != nullptr && bias_r1 == nullptr) || kv_share < 1 || nkv % kv_share != 0
        || (out_type != q_type && out_type != CHIBI_F32))
        return CHIBI_ERR_UNSUPPORTED;
    const int warps = 4;
    const long long jobs = tokens * nq;
    const long long blocks = (jobs + warps - 1) / warps;
    if (blocks > 2147483647LL)
        return CHIBI_ERR_UNSUPPORTED;
    const size_t smem = (size_t)warps * d * sizeof(float);
#define CHIBI_ATTENTION_GENERIC(TO, SLOTS)                                                                    \
    launch(attention_generic_kernel<TQ, TC, TO, SLOTS>, dim3((unsigned)blocks), dim3(warps * 32), smem, stream,  \
           (const TQ*)q, (const TC*)k_cache, (const TC*)v_cache, (TO*)out, block_table, table_stride, q_start,   \
           ctx_len, seq_of_token, seq_rows, positions, tokens, nq, nkv, d, dv, page_size, num_pages, scale,      \
           window, chunk, softcap, bias_r1, bias_r2, sink, kv_share, error)
    CHIBI_DISPATCH_TYPE(q_type, TQ, CHIBI_DISPATCH_TYPE(cache_type, TC, {
        if (out_type == q_type) {
            if (dv <= 256)
                CHIBI_ATTENTION_GENERIC(TQ, 8);
            else
                CHIBI_ATTENTION_GENERIC(TQ, MAX_D / 32);
        } else {
            if (dv <= 256)
                CHIBI_ATTENTION_GENERIC(float, 8);
            else
                CHIBI_ATTENTION_GENERIC(float, MAX_D / 32);
        }
    }));
#undef CHIBI_ATTENTION_GENERIC
    return launch_status();
}

CHIBI_API int chibi_attention_generic(const void* q, int q_type, const void* k_cache,
                                      const void* v_cache, int cache_type, void* out,
                                      const int* block_table, int table_stride,
                                      const int* q_start, const int* ctx_len,
                                      const int* seq_of_token, const int* seq_rows,
                                      const int* positions,
                                      long long tokens, int nq, int nkv, int d, int dv, int page_size,
                                      int num_pages, float scale, int window, int chunk, float softcap,
                                      const float* bias_r1, const float* bias_r2, const float* sink,
                                      int* error, cudaStream_t stream)
{
    if ((bias_r1 != nullptr) != (bias_r2 != nullptr))
        return CHIBI_ERR_UNSUPPORTED;
    return chibi_attention_generic_shared(q, q_type, k_cache, v_cache, cache_type, out, q_type, block_table,
                                          table_stride, q_start, ctx_len, seq_of_token, seq_rows, positions, tokens,
                                          nq, nkv, d, dv, page_size, num_pages, scale, window, chunk, softcap, bias_r1,
                                          bias_r2, sink, 1, error, stream);
}
