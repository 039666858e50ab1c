// Many small matrix products in one launch:  C_b[M, N] = A_b[M, K] * W_b[N, K]^T.
//
// Two uses.  (1) One product per head on column slices of wide activations (the latent attention's
// query absorption and value expansion): batch b reads A + b * a_bs with row stride lda, W + b * w_bs,
// and writes C + b * c_bs with row stride ldc.  (2) One product per expert on rows that were sorted by
// expert (routed feed-forwards): `tile_group[y]` names the weight matrix (W + g * w_gs) of the tile of
// BM rows number y, or is negative for a tile beyond the sorted rows, which does nothing.
//
// Plain FFMA with float32 accumulation in both dtypes: every output element is the sum over
// k = 0..K-1 in that order, whatever else is in the launch, so a row's result does not depend on its
// place or on its neighbours.  In float32 this is the true 32-bit product; in bfloat16 it is the
// fallback for the sizes that the tensor-core version does not take.
// Tiles of BM x 64 x 16 (BM = 64 or 16), 256 threads; any M, N, K.
#include "common.cuh"

// VLLM_LITE_B200_BATCHED_SIMT=1 keeps bfloat16 products on the FFMA kernel (tests compare the two).
static inline bool vl_batched_simt_only() {
    const char* v = getenv("VLLM_LITE_B200_BATCHED_SIMT");
    return v && v[0] == '1';
}

#define GB_BN 64
#define GB_BK 16

template <typename T, typename TW, typename TC, int BM>
__global__ void __launch_bounds__(256)
gemm_batched_nt_kernel(const T* __restrict__ A, const TW* __restrict__ W, TC* __restrict__ C, int M, int N, int K,
                       int lda, int ldw, int ldc, long long a_bs, long long w_bs, long long c_bs,
                       const int* __restrict__ tile_group, long long w_gs) {
    constexpr int TM = BM / 16;
    __shared__ float As[GB_BK][BM + 4];
    __shared__ float Ws[GB_BK][GB_BN + 4];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * GB_BN;
    const T* Ab = A + (size_t)blockIdx.z * a_bs;
    const TW* Wb = W + (size_t)blockIdx.z * w_bs;
    TC* Cb = C + (size_t)blockIdx.z * c_bs;
    if (tile_group) {
        const int g = tile_group[blockIdx.y];
        if (g < 0) return;
        Wb += (size_t)g * w_gs;
    }
    float acc[TM][4];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GB_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            const int n = n0 + r;
            Ws[kk][r] = (n < N && k < K) ? to_f32(Wb[(size_t)n * ldw + k]) : 0.f;
            if (r < BM) {
                const int m = m0 + r;
                As[kk][r] = (m < M && k < K) ? to_f32(Ab[(size_t)m * lda + k]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GB_BK; ++kk) {
            float a[TM], b[4];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) Cb[(size_t)m * ldc + n] = from_f32<TC>(acc[i][j]);
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// The same products on the tensor cores (bfloat16, mma.sync m16n8k16, float32 accumulation): tiles of
// BM x 64 x 32 (BM = 64: four warps of 16 rows; BM = 16: four warps of 16 columns), operands brought by
// 16-byte cp.async through a ring of four stages of 64 columns of K into padded rows, fragments by ldmatrix.  Taken when
// every row of A and W starts on a 16-byte boundary (K, the strides and the batch offsets multiples of 8).
// Three things a routed feed-forward folds into its first product:
//   row_index  row m of A is row row_index[m] / index_div of the matrix A points to (negative: a row of
//              zeros), so the sorted copy of the tokens is never written;
//   row_scale  the float32 sums of row m are multiplied by row_scale[row_index[m]] before anything else
//              (W (s a) = s (W a): the expert weight on the input, applied to the exact sums);
//   act        W holds blocks of 8 gate rows and their 8 up rows (as the dense products' fused SwiGLU);
//              the tile applies the gated activation (activation.cu's formulas) and writes N / 2 columns.
//              act >= GM_ACT_UNARY: W is a plain matrix and the tile applies a function of one argument to its
//              N columns (GM_ACT_UNARY + 0: the square of max(v, 0)).
// Every output element is summed over K in steps of 16 in order, whatever its place in the tile.
// ---------------------------------------------------------------------------------------------------
#define GM_BN 64
#define GM_BK 64
#define GM_LDS 72
#define GM_NST 4
#define GM_ACT_NONE (-1)
#define GM_ACT_UNARY 16
__device__ __forceinline__ float gm_unary(float v, int act) {
    if (act == GM_ACT_UNARY) { v = fmaxf(v, 0.f); return v * v; }
    return v;
}

__device__ __forceinline__ void gm_cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void gm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void gm_ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void gm_mma16816(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float gm_gated(float g, float u, int act, float alpha, float limit, float shift) {
    if (act == 1) return fmaxf(g, 0.f) * u;
    if (act == 2) {
        if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
        return g / (1.0f + expf(-alpha * g)) * (u + shift);
    }
    return g / (1.0f + expf(-g)) * u;
}

template <int BM, typename TC>
__global__ void __launch_bounds__(128)
gemm_batched_bf16_mma_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W, TC* __restrict__ C, int M, int N, int K,
                             int lda, int ldw, int ldc, long long a_bs, long long w_bs, long long c_bs,
                             const int* __restrict__ tile_group, long long w_gs,
                             const int* __restrict__ row_index, int index_div, const float* __restrict__ row_scale,
                             int act, float alpha, float limit, float shift, int nst) {
    constexpr int WARPS_M = BM / 16, WARPS_N = 4 / WARPS_M, WN = GM_BN / WARPS_N, NT = WN / 8;
    // the ring is larger than the 48 KB a kernel may declare: dynamic shared memory
    extern __shared__ __align__(16) unsigned char gm_smem[];
    bf16 (*As)[BM][GM_LDS] = reinterpret_cast<bf16 (*)[BM][GM_LDS]>(gm_smem);
    bf16 (*Ws)[GM_BN][GM_LDS] = reinterpret_cast<bf16 (*)[GM_BN][GM_LDS]>(gm_smem + (size_t)nst * BM * GM_LDS * sizeof(bf16));
    __shared__ int s_src[BM];                                    // source row of every row of the tile (-1: zeros)
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp % WARPS_M, wn = warp / WARPS_M;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * GM_BN;
    const bf16* Ab = A + (size_t)blockIdx.z * a_bs;
    const bf16* Wb = W + (size_t)blockIdx.z * w_bs;
    TC* Cb = C + (size_t)blockIdx.z * c_bs;
    if (tile_group) {
        const int g = tile_group[blockIdx.y];
        if (g < 0) return;
        Wb += (size_t)g * w_gs;
    }
    if (tid < BM) {
        const int m = m0 + tid;
        int src = m < M ? m : -1;
        if (row_index && src >= 0) {
            const int p = row_index[m];
            src = p < 0 ? -1 : p / index_div;
        }
        s_src[tid] = src;
    }
    __syncthreads();
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const int KT = (K + GM_BK - 1) / GM_BK;
    auto load_stage = [&](int st, int kt) {
        const int k0 = kt * GM_BK;
        constexpr int CH = GM_BK / 8;                           // 16-byte pieces of a row of the stage
        for (int idx = tid; idx < BM * CH; idx += 128) {
            const int r = idx / CH, c = idx % CH, k = k0 + c * 8;
            const int src = s_src[r];
            const bool ok = src >= 0 && k < K;
            gm_cp_async16(&As[st][r][c * 8], ok ? Ab + (size_t)src * lda + k : Ab, ok);
        }
        for (int idx = tid; idx < GM_BN * CH; idx += 128) {
            const int r = idx / CH, c = idx % CH, k = k0 + c * 8;
            const bool ok = n0 + r < N && k < K;
            gm_cp_async16(&Ws[st][r][c * 8], ok ? Wb + (size_t)(n0 + r) * ldw + k : Wb, ok);
        }
    };
    // nst stages (2 to GM_NST: a short K needs no long ring, and a short ring lets more blocks share an SM)
    for (int s = 0; s < nst - 1; ++s) {
        if (s < KT) load_stage(s, s);
        gm_commit();
    }
    for (int kt = 0; kt < KT; ++kt) {
        if (nst == 2) gm_wait<0>(); else if (nst == 3) gm_wait<1>(); else gm_wait<2>();
        __syncthreads();
        const int nk = kt + nst - 1;
        if (nk < KT) load_stage(nk % nst, nk);
        gm_commit();
        const int st = kt % nst;
#pragma unroll
        for (int kk = 0; kk < GM_BK / 16; ++kk) {
            unsigned a[4];
            gm_ldmatrix_x4(a, &As[st][wm * 16 + (lane & 15)][kk * 16 + (lane >> 4) * 8]);
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                unsigned b[4];
                gm_ldmatrix_x4(b, &Ws[st][wn * WN + np * 16 + (lane & 7) + ((lane >> 4) << 3)][kk * 16 + ((lane >> 3) & 1) * 8]);
                gm_mma16816(acc[2 * np], a, b[0], b[1]);
                gm_mma16816(acc[2 * np + 1], a, b[2], b[3]);
            }
        }
    }
    gm_wait<0>();
    const int g = lane >> 2, t2 = (lane & 3) * 2;
    const bool pair_ok = ((ldc | c_bs) & 1) == 0 && (((uintptr_t)C) & 3) == 0;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = wm * 16 + g + half * 8;
        const int m = m0 + r;
        if (m >= M) continue;
        float scale = 1.0f;
        if (row_scale) {
            const int p = row_index ? row_index[m] : m;
            scale = p >= 0 ? row_scale[p] : 0.f;
        }
        TC* crow = Cb + (size_t)m * ldc;
        if (act == GM_ACT_NONE || act >= GM_ACT_UNARY) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int n = n0 + wn * WN + nt * 8 + t2;
                const float v0 = gm_unary(acc[nt][2 * half] * scale, act), v1 = gm_unary(acc[nt][2 * half + 1] * scale, act);
                if (sizeof(TC) == 2 && pair_ok && n + 1 < N) {          // two bfloat16 in one 4-byte store
                    __nv_bfloat162 pr = __floats2bfloat162_rn(v0, v1);
                    *reinterpret_cast<unsigned*>(crow + n) = *reinterpret_cast<unsigned*>(&pr);
                } else {
                    if (n < N) crow[n] = from_f32<TC>(v0);
                    if (n + 1 < N) crow[n + 1] = from_f32<TC>(v1);
                }
            }
        } else {
            // n-tiles come in pairs: 8 gate columns, then their 8 up columns; the pair writes 8 columns
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                const int n = (n0 + wn * WN) / 2 + np * 8 + t2;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float gate = acc[2 * np][2 * half + e] * scale, up = acc[2 * np + 1][2 * half + e] * scale;
                    if (n + e < N / 2) crow[n + e] = from_f32<TC>(gm_gated(gate, up, act, alpha, limit, shift));
                }
            }
        }
    }
}

template <int BM, typename TC, typename... Args>
static int launch_mma_kernel(dim3 grid, cudaStream_t s, int K, Args... args) {
    const int KT = (K + GM_BK - 1) / GM_BK;
    const int nst = KT < 2 ? 2 : (KT > GM_NST ? GM_NST : KT);
    const size_t most = (size_t)GM_NST * (BM + GM_BN) * GM_LDS * sizeof(bf16);
    const size_t smem = (size_t)nst * (BM + GM_BN) * GM_LDS * sizeof(bf16);
    auto kern = gemm_batched_bf16_mma_kernel<BM, TC>;
    static bool ready = false;                               // per instantiation
    if (!ready) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
        if (e != cudaSuccess) return (int)e;
        ready = true;
    }
    return vl_launch(kern, grid, dim3(128), smem, s, args..., nst);
}

static bool gm_aligned(const void* A, const void* W, int K, int lda, int ldw, long long a_bs, long long w_bs, long long w_gs) {
    return !(K % 8 || lda % 8 || ldw % 8 || a_bs % 8 || w_bs % 8 || w_gs % 8 || (((uintptr_t)A | (uintptr_t)W) & 15));
}

static int launch_batched_mma(const bf16* A, const bf16* W, bf16* C, int M, int N, int K, int lda, int ldw, int ldc,
                              long long a_bs, long long w_bs, long long c_bs, int batch, const int* tile_group,
                              long long w_gs, int bm, const int* row_index, int index_div, const float* row_scale,
                              int act, float alpha, float limit, float shift, cudaStream_t s) {
    dim3 grid((N + GM_BN - 1) / GM_BN, (M + bm - 1) / bm, batch);
    if (grid.y > 65535 || grid.z > 65535) return VL_ERR_UNSUPPORTED;
    if (bm == 64)
        return launch_mma_kernel<64, bf16>(grid, s, K, A, W, C, M, N, K, lda, ldw, ldc, a_bs, w_bs, c_bs, tile_group, w_gs,
                                           row_index, index_div, row_scale, act, alpha, limit, shift);
    return launch_mma_kernel<16, bf16>(grid, s, K, A, W, C, M, N, K, lda, ldw, ldc, a_bs, w_bs, c_bs, tile_group, w_gs,
                                       row_index, index_div, row_scale, act, alpha, limit, shift);
}

template <typename T>
static int launch_batched(const T* A, const T* W, T* C, int M, int N, int K, int lda, int ldw, int ldc,
                          long long a_bs, long long w_bs, long long c_bs, int batch, const int* tile_group,
                          long long w_gs, int bm, cudaStream_t s) {
    dim3 grid((N + GB_BN - 1) / GB_BN, (M + bm - 1) / bm, batch);
    if (grid.y > 65535 || grid.z > 65535) return VL_ERR_UNSUPPORTED;
    if (bm == 64)
        return vl_launch(gemm_batched_nt_kernel<T, T, T, 64>, grid, dim3(256), 0, s, A, W, C, M, N, K, lda, ldw, ldc,
                         a_bs, w_bs, c_bs, tile_group, w_gs);
    return vl_launch(gemm_batched_nt_kernel<T, T, T, 16>, grid, dim3(256), 0, s, A, W, C, M, N, K, lda, ldw, ldc,
                     a_bs, w_bs, c_bs, tile_group, w_gs);
}

// bm: rows per tile, 64 or 16.  With tile_group, M is the padded number of sorted rows (a multiple of bm).
extern "C" int vl_gemm_batched_nt(const void* A, const void* W, void* C, int dtype, int M, int N, int K,
                                  int lda, int ldw, int ldc, long long a_bs, long long w_bs, long long c_bs,
                                  int batch, const int* tile_group, long long w_gs, int bm, void* stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return VL_OK;
    if (K <= 0 || lda < K || ldw < K || ldc < N || (bm != 64 && bm != 16)) return VL_ERR_ARGUMENT;
    if (tile_group && M % bm) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return launch_batched<float>((const float*)A, (const float*)W, (float*)C, M, N, K, lda, ldw, ldc,
                                     a_bs, w_bs, c_bs, batch, tile_group, w_gs, bm, s);
    if (dtype == VL_BF16) {
        if (gm_aligned(A, W, K, lda, ldw, a_bs, w_bs, w_gs) && !vl_batched_simt_only())
            return launch_batched_mma((const bf16*)A, (const bf16*)W, (bf16*)C, M, N, K, lda, ldw, ldc, a_bs, w_bs, c_bs,
                                      batch, tile_group, w_gs, bm, nullptr, 1, nullptr, GM_ACT_NONE, 0.f, 0.f, 0.f, s);
        return launch_batched<bf16>((const bf16*)A, (const bf16*)W, (bf16*)C, M, N, K, lda, ldw, ldc,
                                    a_bs, w_bs, c_bs, batch, tile_group, w_gs, bm, s);
    }
    return VL_ERR_UNSUPPORTED;
}

// z[M, N] = a[M, K] * w[N, K]^T with a in the activation dtype, w and z float32 (a router's logits: few
// columns, float32 whatever the model's dtype).  Same kernel, same fixed order over K.
extern "C" int vl_gemm_rows_f32w(const void* A, int a_dtype, const void* W, int w_dtype, float* C, int M, int N, int K,
                                 int slices, void* stream) {
    if (M <= 0 || N <= 0) return VL_OK;
    if (K <= 0 || slices <= 0 || K % slices) return VL_ERR_ARGUMENT;
    // slices: K is cut into that many equal parts, each a "batch" of the launch that reads its columns of A
    // and W and writes its own [M, N] sums to C + slice * M * N (the reader adds them in order)
    const int Kc = K / slices;
    const long long cs = (long long)M * N;
    const int bm = 16;                                    // few columns: short tiles give the launch its blocks
    dim3 grid((N + GB_BN - 1) / GB_BN, (M + bm - 1) / bm, slices);
    if (grid.y > 65535) return VL_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (a_dtype == VL_BF16 && w_dtype == VL_BF16 && gm_aligned(A, W, Kc, K, K, Kc, Kc, 0) && !vl_batched_simt_only()) {
        // both operands bfloat16: their products are exact in float32, the tensor cores add them in float32
        return launch_mma_kernel<16, float>(grid, s, Kc, (const bf16*)A, (const bf16*)W, C, M, N, Kc, K, K, N, (long long)Kc,
                                            (long long)Kc, cs, (const int*)nullptr, 0ll, (const int*)nullptr, 1,
                                            (const float*)nullptr, GM_ACT_NONE, 0.f, 0.f, 0.f);
    }
#define ROWS_CASE(TA, TWV)                                                                                          \
    return vl_launch(gemm_batched_nt_kernel<TA, TWV, float, 16>, grid, dim3(256), 0, s, (const TA*)A, (const TWV*)W, C, M, N, \
                     Kc, K, K, N, (long long)Kc, (long long)Kc, cs, (const int*)nullptr, 0ll)
    if (a_dtype == VL_F32 && w_dtype == VL_F32) ROWS_CASE(float, float);
    if (a_dtype == VL_BF16 && w_dtype == VL_F32) ROWS_CASE(bf16, float);
    if (a_dtype == VL_BF16 && w_dtype == VL_BF16) ROWS_CASE(bf16, bf16);
#undef ROWS_CASE
    return VL_ERR_UNSUPPORTED;
}

// 1 when `vl_gemm_grouped_fused` takes these sizes (bfloat16 only): rows of A and W on 16-byte boundaries.
extern "C" int vl_gemm_grouped_fused_ok(int K, int N, int act) {
    return K % 8 == 0 && (act == GM_ACT_NONE || act >= GM_ACT_UNARY || N % 16 == 0) && !vl_batched_simt_only();
}

// The grouped product of a routed feed-forward with its neighbours folded in (bfloat16, tensor cores):
// row m of the tile list reads row row_index[m] / index_div of A [rows, K] (negative: zeros), the sums are
// multiplied by row_scale[row_index[m]] (row_scale null: not), and with act >= 0 the gated activation turns the
// [cap, N] sums (W: blocks of 8 gate rows and their 8 up rows) into C [cap, N / 2].  M = cap, a multiple of bm.
extern "C" int vl_gemm_grouped_fused(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldc,
                                     const int* tile_group, long long w_gs, int bm, const int* row_index, int index_div,
                                     const float* row_scale, int act, float alpha, float limit, float shift, void* stream) {
    if (M <= 0 || N <= 0) return VL_OK;
    if (K <= 0 || lda < K || (bm != 64 && bm != 16) || M % bm || !tile_group || index_div <= 0) return VL_ERR_ARGUMENT;
    const bool gated = act >= 0 && act < GM_ACT_UNARY;
    if (act < GM_ACT_NONE || (act > 2 && act != GM_ACT_UNARY) || ldc < (gated ? N / 2 : N)) return VL_ERR_ARGUMENT;
    if (!vl_gemm_grouped_fused_ok(K, N, act) || !gm_aligned(A, W, K, lda, K, 0, 0, w_gs)) return VL_ERR_UNSUPPORTED;
    return launch_batched_mma((const bf16*)A, (const bf16*)W, (bf16*)C, M, N, K, lda, K, ldc, 0, 0, 0, 1, tile_group, w_gs, bm,
                              row_index, index_div, row_scale, act, alpha, limit, shift, (cudaStream_t)stream);
}
