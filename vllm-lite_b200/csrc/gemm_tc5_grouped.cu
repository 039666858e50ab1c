// The grouped form of the tcgen05 matrix product (csrc/gemm_tc5.cu), for routed feed-forwards with many rows:
//     C[m, :] = A[m, :] * W[g(m)]^T,   rows sorted by group in tiles of 128 (moe.cu: vl_moe_align),
// W [G, N, K] stacked, so that ONE tensor map covers every group's matrix and a tile of W is the box at
// row g * N + n0.  tile_group[y] names the group of the tile of rows y, negative for a tile beyond the
// sorted rows: producer, issuing thread and epilogue all pass over such a tile, so their counts of
// stages and accumulators stay in step.  A box that reaches beyond its group's N rows brings rows of
// the next group; their columns are never stored.
// The epilogue can do what a routed feed-forward needs around its first product: multiply the float32
// sums of row m by row_scale[row_index[m]] (the expert weight on the input: W (s a) = s (W a)), and
// apply the gated activation to blocks of 8 gate and 8 up columns (act 0..2: C is [M, N / 2]) or, act 16, the
// square of max(v, 0) to every column of a plain W.
// Roles, stages, tensor memory and the bounded waits are those of csrc/gemm_tc5.cu.
#include "tc5.cuh"

namespace {
constexpr int BM = 128;
constexpr int BK = 64;                       // one 128-byte swizzle row of bfloat16
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;

}  // namespace
using namespace tc5;

// the gated activations of csrc/activation.cu: 0 silu(g) u, 1 max(g, 0) u, 2 capped swish
__device__ __forceinline__ float gated(float g, float u, int act, float alpha, float limit, float shift) {
    if (act == 1) return fmaxf(g, 0.f) * u;
    if (act == 2) {
        if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
        return g / (1.0f + __expf(-alpha * g)) * (u + shift);
    }
    return g / (1.0f + __expf(-g)) * u;
}

// Tile number -> corner of the tile.  Blocks that run at the same time should share tiles of W
// (and of A) in L2: consecutive numbers walk down a band of up to 16 tiles of M before they move on
// to the next tile of N.
template <int BN>
__device__ __forceinline__ void tile_corner(int tile, int tiles_m, int tiles_n, int& m0, int& n0) {
    constexpr int BAND = 16;
    const int band = tile / (BAND * tiles_n), in_band = tile - band * BAND * tiles_n;
    const int band_rows = min(BAND, tiles_m - band * BAND);
    m0 = (band * BAND + in_band % band_rows) * BM;
    n0 = (in_band / band_rows) * BN;
}

// Persistent: a block takes the tiles blockIdx.x, blockIdx.x + gridDim.x, ...  The ring of stages
// runs on across tiles, and TMEM holds two accumulators, so the epilogue of one tile overlaps the
// products of the next.
template <int BN, int STAGES, typename TO>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_tc5_grouped_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                TO* __restrict__ C, int M, int N, int K, int ldc, unsigned* err, int tiles_m, int tiles_n,
                const int* __restrict__ tile_group, int group_rows, const int* __restrict__ row_index,
                const float* __restrict__ row_scale, int act, float alpha, float limit, float shift) {
    constexpr unsigned A_BYTES = BM * BK * 2, W_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;
    extern __shared__ unsigned char tc5_smem_raw[];
    // tiles of the 128-byte swizzle must start on 1024-byte boundaries
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)tc5_smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full_bar[2], acc_empty_bar[2];
    __shared__ unsigned tmem_base_slot;
    __shared__ int failed;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + BK - 1) / BK;
    const int total_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full_bar[i], 1); mbar_init(&acc_empty_bar[i], 128); }
        mbar_fence_init();
        failed = 0;
    }
    // Tensor memory is taken only after the kernels before this one have completed: a block started as a
    // programmatic dependent then holds nothing of the SM that an earlier kernel may still be waiting for.
    pdl_launch_dependents();
    pdl_wait();                                              // A is written by the kernel before
    if (warp == 1) tc5_alloc(&tmem_base_slot, 2 * BN);       // two accumulators; 2 * BN is a power of two >= 32
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const unsigned tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {                                     // ---- TMA producer ----
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                int m0, n0;
                tile_corner<BN>(tile, tiles_m, tiles_n, m0, n0);
                const int grp = tile_group[m0 / BM];
                if (grp < 0) continue;                       // a tile beyond the sorted rows
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait_bounded(&empty_bar[s], (unsigned)((it / STAGES - 1) & 1))) {
                        atomicOr(&failed, 1);
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&full_bar[s], STAGE_BYTES);
                    unsigned char* st = smem + (size_t)s * STAGE_BYTES;
                    tma_load_2d(st, &map_a, kb * BK, m0, &full_bar[s]);
                    tma_load_2d(st + A_BYTES, &map_w, kb * BK, grp * group_rows + n0, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                     // ---- MMA issuer ----
            constexpr unsigned idesc = make_idesc(BM, BN);
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                int m0, n0;
                tile_corner<BN>(tile, tiles_m, tiles_n, m0, n0);
                if (tile_group[m0 / BM] < 0) continue;
                const int acc = local & 1;
                if (local >= 2 && !mbar_wait_bounded(&acc_empty_bar[acc], (unsigned)((local / 2 - 1) & 1))) {
                    atomicOr(&failed, 2);
                    break;
                }
                tc5_fence_after();
                const unsigned tmem_c = tmem_base + (unsigned)(acc * BN);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait_bounded(&full_bar[s], (unsigned)((it / STAGES) & 1))) {
                        atomicOr(&failed, 4);
                        ok = false;
                        break;
                    }
                    tc5_fence_after();
                    const unsigned char* st = smem + (size_t)s * STAGE_BYTES;
                    const unsigned long long adesc = make_smem_desc(st), bdesc = make_smem_desc(st + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // 16 columns of K further on: 32 bytes inside the swizzled row, i.e. +2 in the address field
                        tc5_mma(tmem_c, adesc + (unsigned long long)(k * 2), bdesc + (unsigned long long)(k * 2), idesc,
                                (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    tc5_commit(&empty_bar[s]);               // the stage is free once these MMAs have read it
                }
                if (ok) tc5_commit(&acc_full_bar[acc]);      // this accumulator is complete
                ++local;
            }
        }
    } else {                                                 // ---- epilogue: warps 2..5 ----
        const int quarter = warp & 3;                        // the TMEM lanes this warp may read
        int local = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            int m0, n0;
            tile_corner<BN>(tile, tiles_m, tiles_n, m0, n0);
            if (tile_group[m0 / BM] < 0) continue;
            const int acc = local & 1;
            if (!mbar_wait_bounded(&acc_full_bar[acc], (unsigned)((local / 2) & 1))) {
                atomicOr(&failed, 8);
                break;
            }
            tc5_fence_after();
            const int row = m0 + quarter * 32 + lane;
            float scale = 1.0f;
            if (row_scale && row < M) {
                const int p = row_index ? row_index[row] : row;
                scale = p >= 0 ? row_scale[p] : 0.f;
            }
            for (int c0 = 0; c0 < BN; c0 += 32) {
                unsigned v[32];
                tc5_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * BN + c0), v);
                if (row >= M) continue;
                if (row_scale) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * scale);
                }
                if (act < 0 || act >= 16) {
                    if (act == 16) {                         // a function of one argument: the square of max(v, 0)
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float f = fmaxf(__uint_as_float(v[i]), 0.f);
                            v[i] = __float_as_uint(f * f);
                        }
                    }
                    store_chunk32<TO>(v, C + (size_t)row * ldc, n0 + c0, N, 0);
                } else {
                    // two blocks of 8 gate and 8 up columns become 16 columns of C at col / 2
                    TO* dst = C + (size_t)row * ldc + (n0 + c0) / 2;
#pragma unroll
                    for (int blk = 0; blk < 2; ++blk) {
                        if (n0 + c0 + 16 * blk + 16 <= N) {
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                dst[8 * blk + i] = from_f32<TO>(gated(__uint_as_float(v[16 * blk + i]),
                                                                      __uint_as_float(v[16 * blk + 8 + i]), act, alpha, limit, shift));
                        }
                    }
                }
            }
            tc5_fence_before();
            mbar_arrive(&acc_empty_bar[acc]);                // 128 arrivals hand the accumulator back
            ++local;
        }
    }
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    if (warp == 1) tc5_dealloc(tmem_base, 2 * BN);
    if (threadIdx.x == 0 && failed && err)
        atomicOr(err, VL_DEV_WAIT_EXPIRED | VL_DEV_IN_GEMM_TC5 | ((unsigned)failed << VL_DEV_ROLE_SHIFT));
}

// ---- host side -------------------------------------------------------------------------------
template <int BN, int STAGES>
static int launch_grouped(const void* A, const void* W, bf16* C, int M, int N, int K, int G, int ldc, unsigned* err,
                          const int* tile_group, const int* row_index, const float* row_scale, int act, float alpha,
                          float limit, float shift, cudaStream_t s) {
    CUtensorMap map_a, map_w;
    int rc = tc5_make_map(&map_a, A, M, K, K, BM);
    if (rc) return rc;
    rc = tc5_make_map(&map_w, W, G * N, K, K, BN);
    if (rc) return rc;
    const size_t smem = (size_t)STAGES * (BM + BN) * BK * 2 + 1024;
    auto kern = gemm_tc5_grouped_kernel<BN, STAGES, bf16>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int tiles_m = M / BM, tiles_n = (N + BN - 1) / BN;
    static int num_sms = 0;
    if (!num_sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0) num_sms = 148;
    }
    const int total = tiles_m * tiles_n;
    dim3 grid(total < num_sms ? total : num_sms);
    return vl_launch(kern, grid, dim3(NUM_THREADS), smem, s, map_a, map_w, C, M, N, K, ldc, err, tiles_m, tiles_n,
                     tile_group, N, row_index, row_scale, act, alpha, limit, shift);
}

// A [M, K] (M = the sorted rows, a multiple of 128), W [G, N, K], C [M, N] or, with act >= 0, [M, N / 2]; bfloat16.
// tile_group [M / 128]; row_scale (optional) is indexed by row_index[m] (row_index null: by m).
extern "C" int vl_gemm_bf16_tc5_grouped(const void* A, const void* W, void* C, int M, int N, int K, int G,
                                        const int* tile_group, const int* row_index, const float* row_scale,
                                        int act, float alpha, float limit, float shift, unsigned* err, void* stream) {
    if (M <= 0 || N <= 0) return VL_OK;
    if (K <= 0 || K % 8 || G <= 0 || M % BM || !tile_group) return VL_ERR_UNSUPPORTED;
    const bool gated = act >= 0 && act < 16;                 // 16: a function of one argument on a plain W
    if (act < -1 || (act > 2 && act != 16) || (gated && N % 16)) return VL_ERR_ARGUMENT;
    if ((long long)G * N >= (1ll << 31)) return VL_ERR_UNSUPPORTED;
    if (((uintptr_t)A | (uintptr_t)W) & 15) return VL_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int ldc = gated ? N / 2 : N;
    if (N > 128) return launch_grouped<256, 4>(A, W, (bf16*)C, M, N, K, G, ldc, err, tile_group, row_index, row_scale, act, alpha,
                                               limit, shift, s);
    return launch_grouped<128, 6>(A, W, (bf16*)C, M, N, K, G, ldc, err, tile_group, row_index, row_scale, act, alpha, limit,
                                  shift, s);
}
