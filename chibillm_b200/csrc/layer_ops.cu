// Kernels of the parts that a layer with two parallel branches, a feed-forward of
// experts chosen by a table, and a per-layer token input are made of:
//
// * heads_rotate_append: per head of a q | k | v row: split-half rotation of the first
//   `rot` features from a frequency table (cosines and sines times an amplitude), then,
//   if asked, the head is divided by its root mean square (a norm AFTER the rotation,
//   without a weight); queries go to an array, keys and values to the pages of the
//   cache.  Keys have d features, values dv.
// * gated_activation: act(gate + b_gate) * (up + b_up) from a gate | up row.
// * route_by_table / expert_rows_gemm / combine_experts: a feed-forward of experts chosen
//   per token id from a table.  The (token, choice) pairs are sorted by expert on the
//   device, the products run as tiles of rows that belong to one expert each (the tile
//   map is made by the sorting kernel, so nothing is read on the host), and the chosen
//   experts' outputs are added in the order of the choices.  (The products of sizes that
//   are multiples of 64 run on tcgen05 from the same map: experts_tcgen05.cu.)
// * layer_end: residual += m * delta, then the per-layer token input
//   (y = P (act(G x) * e[token]); x += m * y / rms(y) * w), then, if asked, the next
//   norm's output.  The products with G and P are done here for few tokens, or taken
//   from `y_in` when the caller ran them as matrix products.
// * softcap, zero.
//
// Sums, norms, angles and the residual are 32-bit whatever the activations' type is.
#define CHIBI_UNIT layer_ops
#define CHIBI_UNIT_ID 9
#include "common.cuh"

namespace chibi {

// ---------------------------------------------------------------- heads: rotate, norm, append
// grid (tokens, ceil(jobs / warps)), one warp per head job: nq query heads, then (append)
// nkv key heads and nkv value heads.  Columns of a row: nq * d | nkv * d | nkv * dv.
template <typename TX, typename TC>
__global__ void heads_rotate_append_kernel(
    const TX* __restrict__ qkv, long long qkv_stride, TX* __restrict__ q_out, TC* __restrict__ k_cache,
    TC* __restrict__ v_cache, const float* __restrict__ inv_freq, float amplitude,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ seq_rows,
    const int* __restrict__ block_table, int table_stride, int nq, int nkv, int d, int dv, int rot,
    int page_size, int num_pages, float eps, int unit_norm, int append, int* __restrict__ error)
{
    pdl_enter();
    extern __shared__ float smem[];
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps = blockDim.x >> 5;
    const int half = rot >> 1;
    float* cs = smem;                                   // [half] cosines, [half] sines
    float* buf = smem + 2 * half + (size_t)warp * d;
    const int pos = positions[t];
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const float a = (float)pos * inv_freq[j];
        float sn, c;
        sincosf(a, &sn, &c);
        cs[j] = c * amplitude;
        cs[half + j] = sn * amplitude;
    }
    __syncthreads();
    const int jobs = append ? nq + 2 * nkv : nq;
    const int job = blockIdx.y * warps + warp;
    if (job >= jobs)
        return;
    const bool is_q = job < nq;
    const bool is_k = !is_q && job < nq + nkv;
    const int head = is_q ? job : (is_k ? job - nq : job - nq - nkv);
    const TX* row = qkv + (size_t)t * qkv_stride;
    const TX* src = is_q ? row + (size_t)head * d
                         : (is_k ? row + (size_t)(nq + head) * d : row + (size_t)(nq + nkv) * d + (size_t)head * dv);
    long long cache_row = -1;
    if (!is_q) {
        const int seq = seq_of_token[t];
        const int table_row = seq_rows ? seq_rows[seq] : seq;
        const int page = block_table[(size_t)table_row * table_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (lane == 0 && error)
                atomicExch(error, 2);
            return;
        }
        cache_row = ((long long)page * nkv + head) * page_size + (pos % page_size);
    }
    if (!is_q && !is_k) {
        TC* dst = v_cache + cache_row * dv;
        for (int j = lane; j < dv; j += 32)
            dst[j] = from_f32<TC>(to_f32(src[j]));
        return;
    }
    for (int j = lane; j < d; j += 32)
        buf[j] = to_f32(src[j]);
    __syncwarp();
    // a lane owns the pairs (j, j + half), j = lane, lane + 32, ...: it reads and writes only those
    for (int j = lane; j < half; j += 32) {
        const float c = cs[j], sn = cs[half + j];
        const float x0 = buf[j], x1 = buf[j + half];
        buf[j] = x0 * c - x1 * sn;
        buf[j + half] = x1 * c + x0 * sn;
    }
    __syncwarp();
    float inv = 1.f;
    if (unit_norm) {
        float s = 0.f;
        for (int j = lane; j < d; j += 32)
            s = fmaf(buf[j], buf[j], s);
        s = warp_sum(s);
        inv = rsqrtf(s / (float)d + eps);
    }
    if (is_q) {
        TX* dst = q_out + ((size_t)t * nq + head) * d;
        for (int j = lane; j < d; j += 32)
            dst[j] = from_f32<TX>(buf[j] * inv);
    } else {
        TC* dst = k_cache + cache_row * d;
        for (int j = lane; j < d; j += 32)
            dst[j] = from_f32<TC>(buf[j] * inv);
    }
}

// ---------------------------------------------------------------- gated activation with biases
template <typename TX, typename TW>
__global__ void gated_activation_kernel(const TX* __restrict__ gate_up, long long stride, const TW* __restrict__ bias,
                                        TX* __restrict__ out, long long rows, int n, int kind, int interleaved)
{
    pdl_enter();
    const long long total = rows * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / n;
        const int c = (int)(i - r * n);
        // columns: all gates then all ups, or (interleaved) blocks of 16 gates followed by their 16 ups
        const int gc = interleaved ? (c / 16) * 32 + c % 16 : c;
        const int uc = interleaved ? gc + 16 : n + c;
        float g = to_f32(gate_up[r * stride + gc]);
        float u = to_f32(gate_up[r * stride + uc]);
        if (bias) {
            g += to_f32(bias[c]);
            u += to_f32(bias[n + c]);
        }
        out[i] = from_f32<TX>(activate(g, kind) * u);
    }
}

// The same for bfloat16 rows whose sizes and addresses allow 16-byte accesses: a thread takes 8
// neighbouring columns (a run of 8 never crosses a block of 16 interleaved columns).
template <typename TW>
__global__ void gated_activation_vec8_kernel(const __nv_bfloat16* __restrict__ gate_up, long long stride,
                                             const TW* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                                             long long rows, int n, int kind, int interleaved)
{
    pdl_enter();
    const int groups = n / 8;
    const long long total = rows * groups;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / groups;
        const int c = (int)(i - r * groups) * 8;
        const int gc = interleaved ? (c / 16) * 32 + c % 16 : c;
        const int uc = interleaved ? gc + 16 : n + c;
        const uint4 graw = *reinterpret_cast<const uint4*>(gate_up + r * stride + gc);
        const uint4 uraw = *reinterpret_cast<const uint4*>(gate_up + r * stride + uc);
        const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&graw);
        const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uraw);
        uint4 oraw;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&oraw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 g = __bfloat1622float2(gh[j]), u = __bfloat1622float2(uh[j]);
            if (bias) {
                g.x += to_f32(bias[c + 2 * j]);
                g.y += to_f32(bias[c + 2 * j + 1]);
                u.x += to_f32(bias[n + c + 2 * j]);
                u.y += to_f32(bias[n + c + 2 * j + 1]);
            }
            oh[j] = __floats2bfloat162_rn(activate(g.x, kind) * u.x, activate(g.y, kind) * u.y);
        }
        *reinterpret_cast<uint4*>(out + r * n + c) = oraw;
    }
}

// ---------------------------------------------------------------- experts chosen by a table
// One block.  pairs = tokens * top; pair p = token p / top, choice p % top.  Writes
// offsets[experts + 1], pair_of_row[pairs] (rows sorted by expert), row_of_pair[pairs],
// the tile map: tile_expert[max_tiles] (-1: unused), tile_row0[max_tiles], every tile
// holding up to tile_rows rows of one expert (max_tiles = ceil(pairs / tile_rows) + experts),
// and token_of_row[pairs] (which row of the tokens' array every sorted row reads).  Without `tokens` the
// table has a row per token of the step (a router's choices) instead of one per token id.
__global__ void __launch_bounds__(1024)
route_by_table_kernel(const int* __restrict__ tokens, const int* __restrict__ table, int vocab, int top, int experts,
                      int num_tokens, int tile_rows, int max_tiles, int with_weights, int* __restrict__ offsets,
                      int* __restrict__ pair_of_row, int* __restrict__ row_of_pair, int* __restrict__ tile_expert,
                      int* __restrict__ tile_row0, int* __restrict__ token_of_row, int* __restrict__ error)
{
    pdl_enter();
    extern __shared__ int counts[];                    // [experts] counts, then [experts] cursors
    int* cursor = counts + experts;
    const int pairs = num_tokens * top;
    for (int e = threadIdx.x; e < experts; e += blockDim.x)
        counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int tok = tokens ? tokens[p / top] : p / top;
        int e = (tok >= 0 && tok < vocab) ? table[(size_t)tok * top + p % top] : -1;
        if (e < 0 || e >= experts) {
            if (error)
                atomicExch(error, 5);
            e = 0;
        }
        atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tile = 0;
        for (int e = 0; e < experts; ++e) {
            offsets[e] = at;
            cursor[e] = at;
            const int end = at + counts[e];
            // (buckets from `with_weights` on get no tiles: their rows are filled by someone else)
            for (int r = at; e < with_weights && r < end && tile < max_tiles; r += tile_rows, ++tile) {
                tile_expert[tile] = e;
                tile_row0[tile] = r;
            }
            at = end;
        }
        offsets[experts] = at;
        for (; tile < max_tiles; ++tile) {
            tile_expert[tile] = -1;
            tile_row0[tile] = 0;
        }
    }
    __syncthreads();
    // Where a row lands within its expert's range depends on the order in which the threads arrive;
    // every row is computed by itself and found again through row_of_pair, so no value depends on it.
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int tok = tokens ? tokens[p / top] : p / top;
        int e = (tok >= 0 && tok < vocab) ? table[(size_t)tok * top + p % top] : 0;
        if (e < 0 || e >= experts)
            e = 0;
        const int r = atomicAdd(&cursor[e], 1);
        pair_of_row[r] = p;
        row_of_pair[p] = r;
        token_of_row[r] = p / top;
    }
}

// Tiles of EG_M rows of one expert times 64 columns; 256 threads, a thread owns 4 x 4 sums.
// out[r, n] = sum_k a[row(r), k] * w[expert][n, k]; GATED: w[expert] holds 2 N rows (gate rows,
// then up rows) and out[r, n] = act(gate sum) * (up sum); not GATED with kind >= 0: out = act(sum).
// row(r) = a_index[r] / a_div when
// a_index is given (the rows of the tokens' array that the sorted pairs point at), else r.
// The K range is walked in order, so a row's sums do not depend on what shares its tile.
constexpr int EG_M = 64, EG_N = 64, EG_K = 16;

template <typename TA, typename TW, typename TO, bool GATED>
__global__ void __launch_bounds__(256)
expert_rows_gemm_kernel(const TA* __restrict__ a, long long a_stride, const int* __restrict__ a_index, int a_div,
                        const TW* __restrict__ w, long long w_expert_stride, TO* __restrict__ out,
                        long long out_stride, const int* __restrict__ offsets, const int* __restrict__ tile_expert,
                        const int* __restrict__ tile_row0, int N, int K, int kind, int interleaved)
{
    pdl_enter();
    const int expert = tile_expert[blockIdx.y];
    if (expert < 0)
        return;
    const int row0 = tile_row0[blockIdx.y];
    const int row_end = min(row0 + EG_M, offsets[expert + 1]);
    const int n0 = blockIdx.x * EG_N;
    __shared__ float As[EG_K][EG_M + 4];
    __shared__ float Bs[GATED ? 2 : 1][EG_K][EG_N + 4];
    const TW* we = w + (size_t)expert * w_expert_stride;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int lr = tid >> 2, lk = (tid & 3) * 4;          // the 4 values of a tile that this thread loads
    const int ar = row0 + lr;
    long long a_row = -1;
    if (ar < row_end)
        a_row = a_index ? a_index[ar] / a_div : ar;
    const int bn = n0 + lr;
    // rows of the gate and of the up matrix for column bn: gate rows then up rows, or (interleaved) blocks
    // of 16 gate rows followed by their 16 up rows
    const size_t gate_row = (GATED && interleaved) ? (size_t)(bn / 16) * 32 + bn % 16 : (size_t)bn;
    const size_t up_row = (GATED && interleaved) ? gate_row + 16 : (size_t)N + bn;
    float acc[GATED ? 2 : 1][4][4];
#pragma unroll
    for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                acc[g][i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += EG_K) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int k = k0 + lk + u;
            As[lk + u][lr] = (a_row >= 0 && k < K) ? to_f32(a[a_row * a_stride + k]) : 0.f;
            Bs[0][lk + u][lr] = (bn < N && k < K) ? to_f32(we[gate_row * K + k]) : 0.f;
            if (GATED)
                Bs[GATED ? 1 : 0][lk + u][lr] = (bn < N && k < K) ? to_f32(we[up_row * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < EG_K; ++k) {
            float av[4], bv[GATED ? 2 : 1][4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                av[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    bv[g][j] = Bs[g][k][tx * 4 + j];
#pragma unroll
            for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        acc[g][i][j] = fmaf(av[i], bv[g][j], acc[g][i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row0 + ty * 4 + i;
        if (r >= row_end)
            continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N)
                continue;
            float v = acc[0][i][j];
            if (GATED)
                v = activate(v, kind) * acc[GATED ? 1 : 0][i][j];
            else if (kind >= 0)
                v = activate(v, kind);
            out[(size_t)r * out_stride + n] = from_f32<TO>(v);
        }
    }
}

// The same product on the tensor cores (bfloat16, 32-bit sums): tiles of 128 rows of one expert
// times 128 columns, K in blocks of 32 through four stages of cp.async, eight warps of 64 x 32
// sums each (mma.sync m16n8k16), two CTAs to an SM (82 KB of shared memory and at most 128 registers
// each; with K blocks of 64 and three stages only one CTA fitted, and its eight warps hid too little:
// 44 % of the tensor pipe cycles, 12 % of the warp slots; 218 -> 242 TFLOP/s at 4,096 rows of 8 experts
// of 2,048 x 3,072).  For a decode step's few rows a kernel with a warp to a column that streams the
// weight rows with plain loads was measured too and was slower (135 to 145 us against 112 to 125 for 7
// experts of that size): every block first walks tile map -> offsets -> row index -> row, four dependent
// trips, for 64 KB of weights; it is not kept.  Rows that a tile does not have are filled with zeros and not
// stored, so a decode step's tiles of one or two rows stream their expert's weights once.
// MODE 1 (gated): the expert's matrix holds blocks of 16 gate rows followed by their 16 up rows, so a
// warp's 32 columns are 16 gate sums and the 16 up sums that belong to them, in the same lanes.
// MODE 2: out = act(sum) in bfloat16 (an expert without a gate); MODE 0: the sums in 32-bit.
constexpr int TG_M = 128, TG_N = 128, TG_K = 32, TG_PAD = 40, TG_STAGES = 4;

__device__ __forceinline__ void tg_cp_async16(void* dst, const void* src, bool valid)
{
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tg_ldmatrix_x4(uint32_t (&r)[4], const void* p)
{
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
}
__device__ __forceinline__ void tg_mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                 "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int MODE>
__global__ void __launch_bounds__(256, 2)
expert_rows_mma_kernel(const __nv_bfloat16* __restrict__ a, long long a_stride, const int* __restrict__ a_index,
                       int a_div, const __nv_bfloat16* __restrict__ w, long long w_expert_stride, void* __restrict__ out,
                       long long out_stride, const int* __restrict__ offsets, const int* __restrict__ tile_expert,
                       const int* __restrict__ tile_row0, int N, int K, int kind)
{
    pdl_enter();
    const int expert = tile_expert[blockIdx.y];
    if (expert < 0)
        return;
    const int row0 = tile_row0[blockIdx.y];
    const int row_end = min(row0 + TG_M, offsets[expert + 1]);
    const int n0 = blockIdx.x * TG_N;
    extern __shared__ __align__(16) unsigned char tg_raw[];
    __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(tg_raw);             // [stage][TG_M][TG_PAD]
    __nv_bfloat16* Bs = As + TG_STAGES * TG_M * TG_PAD;                       // [stage][TG_N][TG_PAD]
    const __nv_bfloat16* we = w + (size_t)expert * w_expert_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int warp_m = warp >> 2, warp_n = warp & 3;

    // what this thread brings in per K block: two 16-byte pieces of the rows' tile, two of the weights'
    const __nv_bfloat16* a_src[2];
    const __nv_bfloat16* b_src[2];
    bool a_ok[2], b_ok[2];
    int dst_off[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c = tid + i * 256;
        const int r = c >> 2, part = c & 3;
        dst_off[i] = r * TG_PAD + part * 8;
        const int ar = row0 + r;
        a_ok[i] = ar < row_end;
        const long long src_row = a_ok[i] ? (a_index ? a_index[ar] / a_div : ar) : 0;
        a_src[i] = a + src_row * a_stride + part * 8;
        b_ok[i] = n0 + r < N;
        b_src[i] = we + (size_t)(b_ok[i] ? n0 + r : 0) * K + part * 8;
    }
    auto issue = [&](int kt, int stage) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            tg_cp_async16(As + (size_t)stage * TG_M * TG_PAD + dst_off[i], a_src[i] + (size_t)kt * TG_K, a_ok[i]);
            tg_cp_async16(Bs + (size_t)stage * TG_N * TG_PAD + dst_off[i], b_src[i] + (size_t)kt * TG_K, b_ok[i]);
        }
    };
    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                acc[i][j][e] = 0.f;
    const int KT = K / TG_K;
    // blocks of 16 rows of this warp's 64 that hold a row at all: a decode step's tile of a few rows
    // costs its one block, not eight
    const int m_tiles = max(0, min(4, (row_end - row0 - warp_m * 64 + 15) / 16));
#pragma unroll
    for (int s = 0; s < TG_STAGES - 1; ++s) {
        if (s < KT)
            issue(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kt = 0; kt < KT; ++kt) {
        asm volatile("cp.async.wait_group %0;" ::"n"(TG_STAGES - 2) : "memory");
        __syncthreads();                       // block kt has landed for everybody, and block kt - 1 has been used by everybody
        const int next = kt + TG_STAGES - 1;
        if (next < KT)
            issue(next, next % TG_STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const __nv_bfloat16* At = As + (size_t)(kt % TG_STAGES) * TG_M * TG_PAD;
        const __nv_bfloat16* Bt = Bs + (size_t)(kt % TG_STAGES) * TG_N * TG_PAD;
        if (m_tiles == 0)
            continue;
#pragma unroll
        for (int ks = 0; ks < TG_K / 16; ++ks) {
            uint32_t af[4][4], bf[2][4];
#pragma unroll
            for (int mi = 0; mi < 4; ++mi)
                if (mi < m_tiles)
                    tg_ldmatrix_x4(af[mi], At + (warp_m * 64 + mi * 16 + (lane & 15)) * TG_PAD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int np = 0; np < 2; ++np)
                tg_ldmatrix_x4(bf[np], Bt + (warp_n * 32 + np * 16 + (lane >> 4) * 8 + (lane & 7)) * TG_PAD + ks * 16
                                           + ((lane >> 3) & 1) * 8);
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) {
                if (mi >= m_tiles)
                    continue;
#pragma unroll
                for (int np = 0; np < 2; ++np) {
                    tg_mma_bf16(acc[mi][2 * np], af[mi], bf[np][0], bf[np][1]);
                    tg_mma_bf16(acc[mi][2 * np + 1], af[mi], bf[np][2], bf[np][3]);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int mi = 0; mi < 4; ++mi) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = row0 + warp_m * 64 + mi * 16 + (lane >> 2) + half * 8;
            if (r >= row_end)
                continue;
            if (MODE == 2) {
                __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(out) + (size_t)r * out_stride;
#pragma unroll
                for (int ni = 0; ni < 4; ++ni)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int col = n0 + warp_n * 32 + ni * 8 + (lane & 3) * 2 + e;
                        if (col < N)
                            orow[col] = __float2bfloat16_rn(activate(acc[mi][ni][half * 2 + e], kind));
                    }
            } else if (MODE == 1) {
                __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(out) + (size_t)r * out_stride;
                const int base = (n0 + warp_n * 32) / 2;
#pragma unroll
                for (int ni = 0; ni < 2; ++ni)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int col = base + ni * 8 + (lane & 3) * 2 + e;
                        if (col < N / 2)
                            orow[col] = __float2bfloat16_rn(activate(acc[mi][ni][half * 2 + e], kind)
                                                            * acc[mi][ni + 2][half * 2 + e]);
                    }
            } else {
                float* orow = static_cast<float*>(out) + (size_t)r * out_stride;
#pragma unroll
                for (int ni = 0; ni < 4; ++ni)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int col = n0 + warp_n * 32 + ni * 8 + (lane & 3) * 2 + e;
                        if (col < N)
                            orow[col] = acc[mi][ni][half * 2 + e];
                    }
            }
        }
    }
}

// acc[t, c] += weight * sum over the token's choices (in their order) of y[row_of_pair[t * top + s], c],
// each times pair_weight[t * top + s] where that is given
__global__ void combine_experts_kernel(const float* __restrict__ y, const int* __restrict__ row_of_pair,
                                       float* __restrict__ acc, long long acc_stride, long long tokens, int n, int top,
                                       float weight, const float* __restrict__ pair_weight)
{
    pdl_enter();
    const long long total = tokens * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / n;
        const int c = (int)(i - t * n);
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            const float v = y[(size_t)row_of_pair[t * top + k] * n + c];
            s = pair_weight ? fmaf(pair_weight[t * top + k], v, s) : s + v;
        }
        acc[t * acc_stride + c] += weight * s;
    }
}

// ---------------------------------------------------------------- the end of a layer
// One block per token.  Shared memory: x [n], y [n], g [side], 32 sums.
template <typename TW, typename TO>
__global__ void __launch_bounds__(256)
layer_end_kernel(float* __restrict__ residual, const float* __restrict__ delta, float mult,
                 const int* __restrict__ tokens, const TW* __restrict__ side_table, long long table_stride,
                 int table_offset, int vocab, const TW* __restrict__ side_gate, const TW* __restrict__ side_proj,
                 const TW* __restrict__ side_norm, const float* __restrict__ y_in, int side, int kind, float eps,
                 const TW* __restrict__ norm_w, float norm_offset, TO* __restrict__ norm_out,
                 TO* __restrict__ copy_out, int n, int* __restrict__ error)
{
    pdl_enter();
    extern __shared__ float sm[];
    float* xs = sm;
    float* ys = sm + n;
    float* gs = sm + 2 * (size_t)n;
    __shared__ float red[32];
    const long long t = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
    float* xr = residual + t * n;
    for (int c = tid; c < n; c += blockDim.x)
        xs[c] = delta ? fmaf(mult, delta[t * n + c], xr[c]) : xr[c];
    __syncthreads();
    if (side > 0 || y_in) {
        if (!y_in) {
            int tok = tokens[t];
            if (tok < 0 || tok >= vocab) {
                if (tid == 0 && error)
                    atomicExch(error, 5);
                tok = 0;
            }
            const TW* e = side_table + (size_t)tok * table_stride + table_offset;
            for (int j = warp; j < side; j += warps) {
                const TW* wr = side_gate + (size_t)j * n;
                float s = 0.f;
                for (int c = lane; c < n; c += 32)
                    s = fmaf(to_f32(wr[c]), xs[c], s);
                s = warp_sum(s);
                if (lane == 0)
                    gs[j] = activate(s, kind) * to_f32(e[j]);
            }
            __syncthreads();
        }
        float ssq = 0.f;
        for (int c = tid; c < n; c += blockDim.x) {
            float y;
            if (y_in) {
                y = y_in[t * n + c];
            } else {
                const TW* wr = side_proj + (size_t)c * side;
                y = 0.f;
                for (int j = 0; j < side; ++j)
                    y = fmaf(to_f32(wr[j]), gs[j], y);
            }
            ys[c] = y;
            ssq = fmaf(y, y, ssq);
        }
        ssq = warp_sum(ssq);
        if (lane == 0)
            red[warp] = ssq;
        __syncthreads();
        float total = 0.f;
        for (int i = 0; i < warps; ++i)
            total += red[i];
        const float inv = rsqrtf(total / (float)n + eps);
        __syncthreads();
        for (int c = tid; c < n; c += blockDim.x)
            xs[c] = fmaf(mult, ys[c] * inv * to_f32(side_norm[c]), xs[c]);
    }
    float ssq = 0.f;
    for (int c = tid; c < n; c += blockDim.x) {
        const float v = xs[c];
        xr[c] = v;
        if (copy_out)
            copy_out[t * n + c] = from_f32<TO>(v);      // the new residual in the activations' type
        ssq = fmaf(v, v, ssq);
    }
    if (!norm_out)
        return;
    ssq = warp_sum(ssq);
    if (lane == 0)
        red[warp] = ssq;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < warps; ++i)
        total += red[i];
    const float inv = rsqrtf(total / (float)n + eps);
    for (int c = tid; c < n; c += blockDim.x)
        norm_out[t * n + c] = from_f32<TO>(xs[c] * inv * (to_f32(norm_w[c]) + norm_offset));
}

// g[t, j] = act(gate[t, j]) * table[token[t], offset + j]
template <typename TX, typename TW>
__global__ void side_gate_kernel(TX* __restrict__ gate, long long stride, const int* __restrict__ tokens,
                                 const TW* __restrict__ table, long long table_stride, int table_offset, int vocab,
                                 long long rows, int side, int kind, int* __restrict__ error)
{
    pdl_enter();
    const long long total = rows * side;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / side;
        const int j = (int)(i - t * side);
        int tok = tokens[t];
        if (tok < 0 || tok >= vocab) {
            if (error)
                atomicExch(error, 5);
            tok = 0;
        }
        const float e = to_f32(table[(size_t)tok * table_stride + table_offset + j]);
        gate[t * stride + j] = from_f32<TX>(activate(to_f32(gate[t * stride + j]), kind) * e);
    }
}

__global__ void softcap_kernel(float* __restrict__ x, float cap, long long total)
{
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

__global__ void zero_kernel(float* __restrict__ x, long long total)
{
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x)
        x[i] = 0.f;
}

static inline unsigned blocks_for(long long total, int threads)
{
    long long b = (total + threads - 1) / threads;
    if (b < 1)
        b = 1;
    return (unsigned)(b > 148LL * 16 ? 148LL * 16 : b);
}

} // namespace chibi

using namespace chibi;

CHIBI_API int chibi_heads_rotate_append(const void* qkv, int x_type, long long qkv_stride, void* q_out, void* k_cache,
                                        void* v_cache, int cache_type, const float* inv_freq, float amplitude,
                                        const int* positions, const int* seq_of_token, const int* seq_rows,
                                        const int* block_table, int table_stride, long long tokens, int nq, int nkv,
                                        int d, int dv, int rot, int page_size, int num_pages, float eps, int unit_norm,
                                        int append, int* error, cudaStream_t stream)
{
    if (tokens <= 0)
        return CHIBI_OK;
    if (!qkv || !q_out || !positions || nq <= 0 || d <= 0 || rot < 0 || rot > d || (rot & 1) || (rot > 0 && !inv_freq))
        return CHIBI_ERR_ARGUMENT;
    if (append && (!k_cache || !v_cache || !block_table || !seq_of_token || nkv <= 0 || dv <= 0 || page_size <= 0))
        return CHIBI_ERR_ARGUMENT;
    if (tokens > 2147483647LL)
        return CHIBI_ERR_UNSUPPORTED;
    const int warps = 4;
    const int jobs = append ? nq + 2 * nkv : nq;
    const size_t smem = ((size_t)rot + (size_t)warps * d) * sizeof(float);
    if (smem > 48 * 1024)
        return CHIBI_ERR_UNSUPPORTED;
    const dim3 grid((unsigned)tokens, (unsigned)((jobs + warps - 1) / warps));
    CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(cache_type, TC, {
        launch(heads_rotate_append_kernel<TX, TC>, grid, dim3(warps * 32), smem, stream, (const TX*)qkv, qkv_stride,
               (TX*)q_out, (TC*)k_cache, (TC*)v_cache, inv_freq, amplitude, positions, seq_of_token, seq_rows,
               block_table, table_stride, nq, nkv, d, dv, rot, page_size, num_pages, eps, unit_norm, append, error);
    }));
    return launch_status();
}

CHIBI_API int chibi_gated_activation(const void* gate_up, int x_type, long long stride, const void* bias, int w_type,
                                     void* out, long long rows, int n, int kind, int interleaved, cudaStream_t stream)
{
    if (rows <= 0 || n <= 0)
        return CHIBI_OK;
    if (!gate_up || !out || kind < 0 || kind > 4 || (interleaved && (n % 16 != 0 || bias)))
        return CHIBI_ERR_ARGUMENT;
    if (x_type == CHIBI_BF16 && n % 8 == 0 && stride % 8 == 0 && (reinterpret_cast<uintptr_t>(gate_up) & 15) == 0
        && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        CHIBI_DISPATCH_TYPE(w_type, TW, {
            launch(gated_activation_vec8_kernel<TW>, dim3(blocks_for(rows * (n / 8), 256)), dim3(256), 0, stream,
                   (const __nv_bfloat16*)gate_up, stride, (const TW*)bias, (__nv_bfloat16*)out, rows, n, kind,
                   interleaved);
        });
        return launch_status();
    }
    CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(w_type, TW, {
        launch(gated_activation_kernel<TX, TW>, dim3(blocks_for(rows * n, 256)), dim3(256), 0, stream,
               (const TX*)gate_up, stride, (const TW*)bias, (TX*)out, rows, n, kind, interleaved);
    }));
    return launch_status();
}

// route: int32 scratch of (experts + 1) + 3 pairs + 2 max_tiles values (max_tiles = ceil(pairs / chibi_expert_tile_rows()) + experts), laid out as
// offsets[experts + 1] | pair_of_row[pairs] | row_of_pair[pairs] | tile_expert[max_tiles] | tile_row0[max_tiles] |
// token_of_row[pairs]
CHIBI_API int chibi_expert_tile_rows() { return EG_M; }
CHIBI_API int chibi_expert_tile_rows_tensor_cores() { return TG_M; }

CHIBI_API int chibi_route_by_table_open(const int* tokens, const int* table, int vocab, int top, int experts,
                                        long long num_tokens, int tile_rows, int with_weights, int* route, int* error,
                                        cudaStream_t stream);

CHIBI_API int chibi_route_by_table(const int* tokens, const int* table, int vocab, int top, int experts,
                                   long long num_tokens, int tile_rows, int* route, int* error, cudaStream_t stream)
{
    return chibi_route_by_table_open(tokens, table, vocab, top, experts, num_tokens, tile_rows, experts, route, error,
                                     stream);
}

// The same with buckets that have no matrices: the (token, choice) pairs of experts `with_weights` .. `experts` - 1
// are sorted and counted like the others but get no tiles, so the products pass over them.
CHIBI_API int chibi_route_by_table_open(const int* tokens, const int* table, int vocab, int top, int experts,
                                        long long num_tokens, int tile_rows, int with_weights, int* route, int* error,
                                        cudaStream_t stream)
{
    if (num_tokens <= 0)
        return CHIBI_OK;
    if (!table || !route || top <= 0 || experts <= 0 || vocab <= 0 || (tile_rows != EG_M && tile_rows != TG_M))
        return CHIBI_ERR_ARGUMENT;
    const long long pairs = num_tokens * top;
    if (pairs > (1LL << 24) || experts > 4096)
        return CHIBI_ERR_UNSUPPORTED;
    const int max_tiles = (int)((pairs + tile_rows - 1) / tile_rows) + experts;
    int* offsets = route;
    int* pair_of_row = offsets + experts + 1;
    int* row_of_pair = pair_of_row + pairs;
    int* tile_expert = row_of_pair + pairs;
    int* tile_row0 = tile_expert + max_tiles;
    launch(route_by_table_kernel, dim3(1), dim3(1024), (size_t)2 * experts * sizeof(int), stream, tokens, table, vocab,
           top, experts, (int)num_tokens, tile_rows, max_tiles, with_weights, offsets, pair_of_row, row_of_pair,
           tile_expert, tile_row0,
           tile_row0 + max_tiles, error);
    return launch_status();
}

// One product of the routed rows.  gated 1: w [experts, 2 N, K], out = act(gate) * up in a's type;
// gated 2: w [experts, N, K], out = act(sum) in a's type (the plain kernel only); gated 0: w [experts, N, K],
// out 32-bit.  gather != 0: row r of the product reads a[pair_of_row[r] / top].
// tile_rows is what the route was made with: 64 runs the plain kernel (any types and sizes; with
// interleaved != 0 a gated matrix holds blocks of 16 gate rows and their 16 up rows), 128 the
// tensor-core kernel (bfloat16, K a multiple of 32, gated matrices interleaved, N a multiple of 16).
CHIBI_API int chibi_expert_rows_gemm(const void* a, int a_type, long long a_stride, int gather, int top, const void* w,
                                     int w_type, void* out, long long out_stride, const int* route, long long pairs,
                                     int experts, int N, int K, int gated, int kind, int tile_rows, int interleaved,
                                     cudaStream_t stream)
{
    if (pairs <= 0)
        return CHIBI_OK;
    if (!a || !w || !out || !route || N <= 0 || K <= 0 || experts <= 0 || top <= 0
        || (tile_rows != EG_M && tile_rows != TG_M))
        return CHIBI_ERR_ARGUMENT;
    const int max_tiles = (int)((pairs + tile_rows - 1) / tile_rows) + experts;
    if (max_tiles > 65535)
        return CHIBI_ERR_UNSUPPORTED;
    const int* offsets = route;
    const int* pair_of_row = offsets + experts + 1;
    const int* tile_expert = pair_of_row + 2 * pairs;
    const int* tile_row0 = tile_expert + max_tiles;
    const long long w_stride = (long long)(gated == 1 ? 2 : 1) * N * K;
    if (tile_rows == TG_M) {
        if (a_type != CHIBI_BF16 || w_type != CHIBI_BF16 || K % TG_K != 0 || a_stride % 8 != 0
            || (reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)
            || (gated == 1 && (!interleaved || N % 16 != 0)))
            return CHIBI_ERR_UNSUPPORTED;
        const int rows_of_w = gated == 1 ? 2 * N : N;
        const dim3 tgrid((unsigned)((rows_of_w + TG_N - 1) / TG_N), (unsigned)max_tiles);
        const size_t smem = (size_t)TG_STAGES * (TG_M + TG_N) * TG_PAD * sizeof(__nv_bfloat16);
        auto kernel = gated == 1 ? expert_rows_mma_kernel<1> : gated == 2 ? expert_rows_mma_kernel<2>
                                                                          : expert_rows_mma_kernel<0>;
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch(kernel, tgrid, dim3(256), smem, stream, (const __nv_bfloat16*)a, a_stride,
               gather ? pair_of_row : (const int*)nullptr, top, (const __nv_bfloat16*)w, w_stride, out, out_stride,
               offsets, tile_expert, tile_row0, rows_of_w, K, kind);
        return launch_status();
    }
    const dim3 grid((unsigned)((N + EG_N - 1) / EG_N), (unsigned)max_tiles);
    CHIBI_DISPATCH_TYPE(a_type, TA, CHIBI_DISPATCH_TYPE(w_type, TW, {
        if (gated == 1)
            launch(expert_rows_gemm_kernel<TA, TW, TA, true>, grid, dim3(256), 0, stream, (const TA*)a, a_stride,
                   gather ? pair_of_row : (const int*)nullptr, top, (const TW*)w, w_stride, (TA*)out, out_stride,
                   offsets, tile_expert, tile_row0, N, K, kind, interleaved);
        else if (gated == 2)
            launch(expert_rows_gemm_kernel<TA, TW, TA, false>, grid, dim3(256), 0, stream, (const TA*)a, a_stride,
                   gather ? pair_of_row : (const int*)nullptr, top, (const TW*)w, w_stride, (TA*)out, out_stride,
                   offsets, tile_expert, tile_row0, N, K, kind, 0);
        else
            launch(expert_rows_gemm_kernel<TA, TW, float, false>, grid, dim3(256), 0, stream, (const TA*)a, a_stride,
                   gather ? pair_of_row : (const int*)nullptr, top, (const TW*)w, w_stride, (float*)out, out_stride,
                   offsets, tile_expert, tile_row0, N, K, -1, 0);
    }));
    return launch_status();
}

CHIBI_API int chibi_combine_experts(const float* y, const int* route, float* acc, long long acc_stride,
                                    long long tokens, int n, int top, int experts, float weight,
                                    const float* pair_weight, cudaStream_t stream)
{
    if (tokens <= 0)
        return CHIBI_OK;
    if (!y || !route || !acc || n <= 0 || top <= 0)
        return CHIBI_ERR_ARGUMENT;
    const int* row_of_pair = route + experts + 1 + tokens * top;
    launch(combine_experts_kernel, dim3(blocks_for(tokens * n, 256)), dim3(256), 0, stream, y, row_of_pair, acc,
           acc_stride, tokens, n, top, weight, pair_weight);
    return launch_status();
}

CHIBI_API int chibi_layer_end(float* residual, const float* delta, float mult, const int* tokens,
                              const void* side_table, long long table_stride, int table_offset, int vocab,
                              const void* side_gate, const void* side_proj, const void* side_norm, const float* y_in,
                              int side, int kind, float eps, const void* norm_w, float norm_offset, void* norm_out,
                              void* copy_out, int out_type, int w_type, long long rows, int n, int* error,
                              cudaStream_t stream)
{
    if (rows <= 0)
        return CHIBI_OK;
    if (!residual || n <= 0 || side < 0 || (norm_out && !norm_w))
        return CHIBI_ERR_ARGUMENT;
    if ((side > 0 || y_in) && !side_norm)
        return CHIBI_ERR_ARGUMENT;
    if (side > 0 && !y_in && (!tokens || !side_table || !side_gate || !side_proj))
        return CHIBI_ERR_ARGUMENT;
    const size_t smem = (2 * (size_t)n + (size_t)side) * sizeof(float);
    if (smem > 200 * 1024 || rows > 2147483647LL)
        return CHIBI_ERR_UNSUPPORTED;
    CHIBI_DISPATCH_TYPE(w_type, TW, CHIBI_DISPATCH_TYPE(out_type, TO, {
        auto kernel = layer_end_kernel<TW, TO>;
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch(kernel, dim3((unsigned)rows), dim3(256), smem, stream, residual, delta, mult, tokens,
               (const TW*)side_table, table_stride, table_offset, vocab, (const TW*)side_gate, (const TW*)side_proj,
               (const TW*)side_norm, y_in, side, kind, eps, (const TW*)norm_w, norm_offset, (TO*)norm_out,
               (TO*)copy_out, n, error);
    }));
    return launch_status();
}

CHIBI_API int chibi_side_gate(void* gate, int x_type, long long stride, const int* tokens, const void* table,
                              int w_type, long long table_stride, int table_offset, int vocab, long long rows, int side,
                              int kind, int* error, cudaStream_t stream)
{
    if (rows <= 0 || side <= 0)
        return CHIBI_OK;
    if (!gate || !tokens || !table)
        return CHIBI_ERR_ARGUMENT;
    CHIBI_DISPATCH_TYPE(x_type, TX, CHIBI_DISPATCH_TYPE(w_type, TW, {
        launch(side_gate_kernel<TX, TW>, dim3(blocks_for(rows * side, 256)), dim3(256), 0, stream, (TX*)gate, stride,
               tokens, (const TW*)table, table_stride, table_offset, vocab, rows, side, kind, error);
    }));
    return launch_status();
}

CHIBI_API int chibi_softcap(float* x, float cap, long long total, cudaStream_t stream)
{
    if (total <= 0)
        return CHIBI_OK;
    if (!x || !(cap > 0.f))
        return CHIBI_ERR_ARGUMENT;
    launch(softcap_kernel, dim3(blocks_for(total, 256)), dim3(256), 0, stream, x, cap, total);
    return launch_status();
}

CHIBI_API int chibi_zero(float* x, long long total, cudaStream_t stream)
{
    if (total <= 0)
        return CHIBI_OK;
    if (!x)
        return CHIBI_ERR_ARGUMENT;
    launch(zero_kernel, dim3(blocks_for(total, 256)), dim3(256), 0, stream, x, total);
    return launch_status();
}
