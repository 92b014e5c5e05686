// The products of a feed-forward of experts on the 5th-generation tensor cores.
//
// The rows (one per (token, choice) pair) lie sorted by expert in one bfloat16 array
// [pairs, K]; all experts' matrices are one array [experts * rows_w, K].  A tile map made on
// the device by route_by_table (layer_ops.cu) names, for every tile of 128 rows, its expert
// and its first row; a tile never holds rows of two experts that it writes.  A CTA takes
// one tile of 128 rows x 128 weight rows: TMA brings the K blocks of 64 of both operands
// (128-byte swizzle) through a ring of stages, one elected thread issues tcgen05.mma
// (128 x 128 x 16) into a TMEM accumulator of 128 columns, four warps read it back with
// tcgen05.ld.  Rows past the expert's last row are computed (they are the next expert's
// rows, or zeros past the array's end) and not written.
//
// MODE 1 (gated): an expert's matrix holds blocks of 16 gate rows followed by their 16 up rows,
// so 32 accumulator columns are 16 gate sums and their 16 up sums; out[r, f] = act(gate) * up
// in bfloat16.  MODE 2: out[r, n] = act(sum) in bfloat16 (an expert without a gate).
// MODE 0: out is 32-bit [pairs, rows_w].
//
// Warp roles (192 threads): warp 0 loads, warp 1 owns TMEM and issues, warps 2..5 are the
// epilogue (warp w reads TMEM lanes 32 * (w % 4) ..).  Every wait has a limit; a wait that
// runs out records a code in the error word and the CTA goes on to free its TMEM.
#define CHIBI_UNIT experts_tcgen05
#define CHIBI_UNIT_ID 10
#include "common.cuh"
#include "sm100.cuh"
#include "tensor_map.cuh"

namespace chibi {

using namespace sm100;

constexpr int XT_M = 128, XT_N = 128, XT_K = 64, XT_UMMA_K = 16, XT_STAGES = 3, XT_THREADS = 192;
constexpr int XT_A_BYTES = XT_M * XT_K * 2, XT_B_BYTES = XT_N * XT_K * 2, XT_STAGE_BYTES = XT_A_BYTES + XT_B_BYTES;
constexpr size_t XT_SMEM = XT_STAGES * XT_STAGE_BYTES + (2 * XT_STAGES + 1) * 8 + 16 + 1024;

struct ExpertTileParams {
    const int* offsets;        // [experts + 1]: first sorted row of every expert
    const int* tile_expert;    // [tiles]: -1 = unused
    const int* tile_row0;      // [tiles]
    int rows_w;                // rows of one expert's matrix (2 F when gated)
    int k_blocks;              // K / 64
    void* out;
    long long out_stride;
    int kind;                  // activation of the gate
    int* error;
};

template <int MODE>
__global__ void __launch_bounds__(XT_THREADS)
expert_rows_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const ExpertTileParams p)
{
    pdl_enter();                                   // the tile map is the kernel before's work
    const int expert = p.tile_expert[blockIdx.y];
    if (expert < 0)
        return;                                    // the whole CTA, before any barrier or TMEM
    const int row0 = p.tile_row0[blockIdx.y];
    const int row_end = min(row0 + XT_M, p.offsets[expert + 1]);
    const int n0 = blockIdx.x * XT_N;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + XT_STAGES * XT_STAGE_BYTES);
    uint64_t* empty_bar = full_bar + XT_STAGES;
    uint64_t* tmem_full_bar = empty_bar + XT_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < XT_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(tmem_full_bar, 1);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, XT_N);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (elect_one()) {
            tma_prefetch_descriptor(&map_a);
            tma_prefetch_descriptor(&map_b);
            for (int i = 0; i < p.k_blocks; ++i) {
                const int s = i % XT_STAGES;
                const uint32_t round = i / XT_STAGES;
                if (i >= XT_STAGES && !mbar_wait(&empty_bar[s], (round - 1) & 1, p.error, 31))
                    break;
                uint8_t* a_dst = smem + s * XT_STAGE_BYTES;
                mbar_arrive_expect_tx(&full_bar[s], XT_STAGE_BYTES);
                tma_load_2d(a_dst, &map_a, &full_bar[s], i * XT_K, row0);
                tma_load_2d(a_dst + XT_A_BYTES, &map_b, &full_bar[s], i * XT_K, expert * p.rows_w + n0);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc = make_idesc_bf16_f32(XT_M, XT_N);
            for (int i = 0; i < p.k_blocks; ++i) {
                const int s = i % XT_STAGES;
                const uint32_t round = i / XT_STAGES;
                if (!mbar_wait(&full_bar[s], round & 1, p.error, 32))
                    break;
                tcgen05_fence_after();
                const uint32_t a_addr = smem_addr(smem + s * XT_STAGE_BYTES);
                const uint32_t b_addr = a_addr + XT_A_BYTES;
#pragma unroll
                for (int k = 0; k < XT_K / XT_UMMA_K; ++k) {
                    const uint64_t a_desc = make_kmajor_sw128_desc(a_addr + k * XT_UMMA_K * 2);
                    const uint64_t b_desc = make_kmajor_sw128_desc(b_addr + k * XT_UMMA_K * 2);
                    tcgen05_mma_bf16(tmem_base, a_desc, b_desc, idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                tcgen05_commit(&empty_bar[s]);     // the stage is free once these MMAs have read it
            }
            tcgen05_commit(tmem_full_bar);
        }
    } else {
        const int quarter = warp & 3;
        const int r = row0 + quarter * 32 + lane;
        const bool ok = mbar_wait(tmem_full_bar, 0, p.error, 33);
        tcgen05_fence_after();
        const bool write = ok && r < row_end;
#pragma unroll 1
        for (int c0 = 0; c0 < XT_N; c0 += 32) {
            uint32_t v[32];
            // every lane of the warp takes part in the load, whether its row is written or not
            tmem_load_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c0, v);
            tmem_load_wait();
            if (!write)
                continue;
            if (MODE == 2) {
                if (n0 + c0 >= p.rows_w)
                    continue;
                __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + (size_t)r * p.out_stride + n0 + c0;
                __nv_bfloat162 h[16];
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    h[j] = __floats2bfloat162_rn(activate(__uint_as_float(v[2 * j]), p.kind),
                                                 activate(__uint_as_float(v[2 * j + 1]), p.kind));
                if (n0 + c0 + 32 <= p.rows_w && p.out_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        reinterpret_cast<uint4*>(dst)[j] = reinterpret_cast<uint4*>(h)[j];
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (n0 + c0 + 2 * j < p.rows_w)
                            dst[2 * j] = h[j].x;
                        if (n0 + c0 + 2 * j + 1 < p.rows_w)
                            dst[2 * j + 1] = h[j].y;
                    }
                }
            } else if (MODE == 1) {
                const int col = (n0 + c0) / 2;          // 32 accumulator columns = 16 features
                if (col >= p.rows_w / 2)
                    continue;
                __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + (size_t)r * p.out_stride + col;
                __nv_bfloat162 h[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    h[j] = __floats2bfloat162_rn(
                        activate(__uint_as_float(v[2 * j]), p.kind) * __uint_as_float(v[16 + 2 * j]),
                        activate(__uint_as_float(v[2 * j + 1]), p.kind) * __uint_as_float(v[16 + 2 * j + 1]));
                if (p.out_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) {
                    reinterpret_cast<uint4*>(dst)[0] = reinterpret_cast<uint4*>(h)[0];
                    reinterpret_cast<uint4*>(dst)[1] = reinterpret_cast<uint4*>(h)[1];
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        dst[2 * j] = h[j].x;
                        dst[2 * j + 1] = h[j].y;
                    }
                }
            } else {
                float* dst = static_cast<float*>(p.out) + (size_t)r * p.out_stride + n0 + c0;
                if (n0 + c0 + 32 <= p.rows_w && p.out_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        reinterpret_cast<float4*>(dst)[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                                        __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (n0 + c0 + j < p.rows_w)
                            dst[j] = __uint_as_float(v[j]);
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, XT_N);
    }
}

} // namespace chibi

using namespace chibi;

// One product of the routed rows on tcgen05.  a: [pairs, K] bfloat16, contiguous, sorted by expert;
// w: [experts, rows_w, K] bfloat16, contiguous (gated: rows_w = 2 F, interleaved in blocks of 16);
// route: as route_by_table lays it out for tiles of 128 rows.  out: gated == 1: bfloat16 [pairs, F]
// with out_stride; gated == 2: bfloat16 [pairs, rows_w], act(sum); else float [pairs, rows_w].  CHIBI_ERR_UNSUPPORTED for sizes it does not take.
CHIBI_API int chibi_expert_rows_tc(const void* a, const void* w, void* out, long long out_stride, const int* route,
                                   long long pairs, int experts, int rows_w, int K, int gated, int kind, int* error,
                                   cudaStream_t stream)
{
    if (pairs <= 0)
        return CHIBI_OK;
    if (!a || !w || !out || !route || experts <= 0 || rows_w <= 0 || K <= 0)
        return CHIBI_ERR_ARGUMENT;
    if (K % XT_K != 0 || (gated == 1 && rows_w % 32 != 0) || (reinterpret_cast<uintptr_t>(a) & 15)
        || (reinterpret_cast<uintptr_t>(w) & 15) || pairs > 2147483647LL - XT_M
        || (long long)experts * rows_w > 2147483647LL - XT_N)
        return CHIBI_ERR_UNSUPPORTED;
    const int max_tiles = (int)((pairs + XT_M - 1) / XT_M) + experts;
    if (max_tiles > 65535)
        return CHIBI_ERR_UNSUPPORTED;
    CUtensorMap map_a, map_b;
    if (!tensor_map_2d(a, pairs, K, K, XT_M, &map_a) || !tensor_map_2d(w, (long long)experts * rows_w, K, K, XT_N, &map_b))
        return CHIBI_ERR_UNSUPPORTED;
    ExpertTileParams p {};
    p.offsets = route;
    p.tile_expert = route + experts + 1 + 2 * pairs;
    p.tile_row0 = p.tile_expert + max_tiles;
    p.rows_w = rows_w;
    p.k_blocks = K / XT_K;
    p.out = out;
    p.out_stride = out_stride;
    p.kind = kind;
    p.error = error;
    const dim3 grid((unsigned)((rows_w + XT_N - 1) / XT_N), (unsigned)max_tiles);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(expert_rows_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)XT_SMEM);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(expert_rows_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)XT_SMEM);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(expert_rows_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)XT_SMEM);
        if (e != cudaSuccess)
            return (int)e;
        configured = true;
    }
    if (gated == 1)
        launch(expert_rows_tc_kernel<1>, grid, dim3(XT_THREADS), XT_SMEM, stream, map_a, map_b, p);
    else if (gated == 2)
        launch(expert_rows_tc_kernel<2>, grid, dim3(XT_THREADS), XT_SMEM, stream, map_a, map_b, p);
    else
        launch(expert_rows_tc_kernel<0>, grid, dim3(XT_THREADS), XT_SMEM, stream, map_a, map_b, p);
    return launch_status();
}
