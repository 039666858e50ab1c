// Routed feed-forwards (mixtures of experts): routing, sorting rows by expert, and putting the
// experts' results back together.  The products themselves are the grouped form of
// gemm_batched.cu, the experts' activation is in activation.cu.
//
//   vl_moe_route    from the logits z = W_r h (+ bias) (float32, a product of csrc/gemm_batched.cu): score =
//                   sigmoid(z) or softmax(z); the `top` largest pick the experts of a token (ties: the
//                   lower index), weights = the scores as they are or divided by their sum (+ renorm_eps).
//                   `choice_bias` (a number per expert): the choice, also that of the groups, is made on
//                   score + choice_bias instead of the logits; the weights stay the scores without it.
//                   `group_top`: a group counts by the sum of its `group_top` largest choice values (1: its largest).
//                   -> expert ids [T, top], weights float32 [T, top]
//   vl_moe_align    sorts the T * top (token, choice) pairs by expert into tiles of `bm` rows, every
//                   expert's rows padded up to whole tiles: sorted_rows[r] = pair or -1,
//                   tile_group[y] = expert of tile y or -1, place[pair] = r.  One block; where a pair
//                   lands among its expert's rows is not fixed from run to run, and nothing depends
//                   on it: a row's arithmetic does not depend on its place.
//   vl_moe_gather   rows[r] = weight(pair) * h[token(pair)] (or h itself), zeros for padding rows
//   vl_moe_combine  out[t] = sum over the token's choices, in the order of the choices, of
//                   (weight *) result[place[pair]] (+ add[t]: a row that every token gets, added last)
//
// Padded tokens of a graph step are ordinary rows here: they cost a row of work and nobody reads
// their result.
#include "common.cuh"

#define MOE_SCORE_SIGMOID 0
#define MOE_SCORE_SOFTMAX 1
#define MOE_MAX_EXPERTS 1024

// one warp per token; z [ntok, E]: the router's logits (csrc/gemm_batched.cu: vl_gemm_rows_f32w)
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ z, int slices, int ntok, int E, int top,
                 int score_fn, int renorm, int groups, int keep, const float* __restrict__ bias,
                 const float* __restrict__ choice_bias, int group_top, float renorm_eps,
                 int* __restrict__ ids, float* __restrict__ weights) {
    extern __shared__ float s_scores[];                  // [4][E], then [4][groups], then [4][E] logits kept for the weights
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= ntok) return;
    float* sc = s_scores + (size_t)warp * E;
    for (int e = lane; e < E; e += 32) {                 // the logits came as sums over slices of K: added in their order
        float v = 0.f;
        for (int sl = 0; sl < slices; ++sl) v += z[((size_t)sl * ntok + t) * E + e];
        sc[e] = bias ? v + bias[e] : v;
    }
    __syncwarp();
    // The choice is made on the logits: both score functions grow with z, and a sigmoid that has
    // rounded to 1 for several experts would hide which of them is the largest.
    float zmax = -INFINITY, zsum = 0.f;
    if (score_fn == MOE_SCORE_SOFTMAX) {
        for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, sc[e]);
        zmax = warp_max(zmax);
        for (int e = lane; e < E; e += 32) zsum += expf(sc[e] - zmax);
        zsum = warp_sum(zsum);
    }
    float* zl = sc;                                      // where a chosen expert's logit is read for its weight
    if (choice_bias) {
        // the choice runs on score + choice_bias (which is not monotone in the logit across experts); the logits are kept
        zl = s_scores + (size_t)4 * E + (size_t)4 * groups + (size_t)warp * E;
        for (int e = lane; e < E; e += 32) {
            const float v = sc[e];
            zl[e] = v;
            sc[e] = (score_fn == MOE_SCORE_SOFTMAX ? expf(v - zmax) / zsum : 1.0f / (1.0f + expf(-v))) + choice_bias[e];
        }
        __syncwarp();
    }
    if (groups > 1) {
        // A group counts by its largest logit; experts outside the `keep` best groups (ties: the lower group) cannot
        // be chosen.  The scores above were taken over all experts.
        float* gm = s_scores + (size_t)4 * E + (size_t)warp * groups;
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float m = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) m = fmaxf(m, sc[e]);
            if (group_top > 1) {
                // the sum of the group's largest values, taken one by one (ties: the lower index first)
                float sum = 0.f, last = INFINITY;
                int last_e = -1;
                for (int j = 0; j < group_top && j < per; ++j) {
                    float best = -INFINITY;
                    int arg = -1;
                    for (int e = g * per; e < (g + 1) * per; ++e) {
                        const float v = sc[e];
                        const bool after = v < last || (v == last && e > last_e);
                        if (after && v > best) { best = v; arg = e; }
                    }
                    if (arg < 0) break;
                    sum += best; last = best; last_e = arg;
                }
                m = sum;
            }
            gm[g] = m;
        }
        __syncwarp();
        for (int g = lane; g < groups; g += 32) {
            int ahead = 0;                               // groups that come before g in the order (larger, or equal and lower)
            for (int o = 0; o < groups; ++o) ahead += (gm[o] > gm[g] || (gm[o] == gm[g] && o < g)) ? 1 : 0;
            if (ahead >= keep)
                for (int e = g * per; e < (g + 1) * per; ++e) sc[e] = -INFINITY;
        }
        __syncwarp();
    }
    float total = 0.f;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = sc[e];
            if (v > best) { best = v; arg = e; }         // ascending e within a lane: the lower index wins a tie
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        const float zb = zl[arg];
        const float score = score_fn == MOE_SCORE_SOFTMAX ? expf(zb - zmax) / zsum : 1.0f / (1.0f + expf(-zb));
        if (lane == 0) {
            ids[(size_t)t * top + j] = arg;
            weights[(size_t)t * top + j] = score;
            sc[arg] = -INFINITY;
        }
        total += score;
        __syncwarp();
    }
    if (renorm && lane == 0)
        for (int j = 0; j < top; ++j) weights[(size_t)t * top + j] /= (total + renorm_eps);
}

__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ ids, int npairs, int E, int bm, int cap, int max_tiles,
                 int* __restrict__ sorted_rows, int* __restrict__ tile_group, int* __restrict__ place) {
    __shared__ int s_count[MOE_MAX_EXPERTS];
    __shared__ int s_start[MOE_MAX_EXPERTS];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += 1024) s_count[e] = 0;
    __syncthreads();
    for (int p = tid; p < npairs; p += 1024) {
        const int e = ids[p];
        if (e >= 0 && e < E) atomicAdd(&s_count[e], 1);
    }
    for (int r = tid; r < cap; r += 1024) sorted_rows[r] = -1;
    for (int y = tid; y < max_tiles; y += 1024) tile_group[y] = -1;
    __syncthreads();
    if (tid == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            s_start[e] = at;
            const int tiles = (s_count[e] + bm - 1) / bm;
            for (int y = 0; y < tiles; ++y) tile_group[at / bm + y] = e;
            at += tiles * bm;
            s_count[e] = 0;                              // now the cursor of the expert's rows
        }
    }
    __syncthreads();
    for (int p = tid; p < npairs; p += 1024) {
        const int e = ids[p];
        if (e < 0 || e >= E) { place[p] = -1; continue; }
        const int r = s_start[e] + atomicAdd(&s_count[e], 1);
        sorted_rows[r] = p;
        place[p] = r;
    }
}

template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ h, const int* __restrict__ sorted_rows,
                                  const float* __restrict__ weights, int top, int K, int scale_input,
                                  T* __restrict__ rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int p = sorted_rows[r];
    T* dst = rows + (size_t)r * K;
    if (p < 0) {
        for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = from_f32<T>(0.f);
        return;
    }
    const T* src = h + (size_t)(p / top) * K;
    const float w = scale_input ? weights[p] : 1.0f;
    if (K % 8 == 0) {                                    // rows start on 16-byte boundaries: eight values an access
        for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
            float v[8];
            load8(src + k, v);
            if (scale_input) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] *= w;
            }
            store8(dst + k, v);
        }
        return;
    }
    for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = scale_input ? from_f32<T>(w * to_f32(src[k])) : src[k];
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ result, const int* __restrict__ place,
                                   const float* __restrict__ weights, int top, int N, int scale_output,
                                   T* __restrict__ out, const T* __restrict__ add) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (N % 8 == 0) {                                    // eight columns a thread, 16-byte accesses
        for (int n = (blockIdx.y * blockDim.x + threadIdx.x) * 8; n < N; n += gridDim.y * blockDim.x * 8) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < top; ++j) {
                const int r = place[(size_t)t * top + j];
                if (r < 0) continue;
                float v[8];
                load8(result + (size_t)r * N + n, v);
                const float w = scale_output ? weights[(size_t)t * top + j] : 1.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += scale_output ? w * v[i] : v[i];
            }
            if (add) {                                       // one more row for every token (an expert that all tokens share)
                float v[8];
                load8(add + (size_t)t * N + n, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += v[i];
            }
            store8(out + (size_t)t * N + n, acc);
        }
        return;
    }
    for (int n = blockIdx.y * blockDim.x + threadIdx.x; n < N; n += gridDim.y * blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < top; ++j) {
            const int r = place[(size_t)t * top + j];
            if (r < 0) continue;
            const float v = to_f32(result[(size_t)r * N + n]);
            acc += scale_output ? weights[(size_t)t * top + j] * v : v;
        }
        if (add) acc += to_f32(add[(size_t)t * N + n]);
        out[(size_t)t * N + n] = from_f32<T>(acc);
    }
}

extern "C" int vl_moe_route(const float* z, int slices, int T, int E, int top, int score_fn, int renorm, int groups, int keep,
                            const float* bias, const float* choice_bias, int group_top, float renorm_eps, int* ids,
                            float* weights, void* stream) {
    if (T <= 0) return VL_OK;
    if (group_top < 1 || renorm_eps < 0.f) return VL_ERR_ARGUMENT;
    if (E <= 0 || E > MOE_MAX_EXPERTS || top <= 0 || top > E || slices <= 0) return VL_ERR_ARGUMENT;
    if (score_fn != MOE_SCORE_SIGMOID && score_fn != MOE_SCORE_SOFTMAX) return VL_ERR_ARGUMENT;
    if (groups < 1 || E % groups || keep < 1 || keep > groups || keep * (E / groups) < top) return VL_ERR_ARGUMENT;
    return vl_launch(moe_route_kernel, dim3((T + 3) / 4), dim3(128), (size_t)4 * (E + groups + (choice_bias ? E : 0)) * sizeof(float),
                     (cudaStream_t)stream, z, slices, T, E, top, score_fn, renorm, groups, keep, bias, choice_bias, group_top,
                     renorm_eps, ids, weights);
}

// cap = rows of the sorted buffer (a multiple of bm, at least npairs rounded up per expert: npairs + E * (bm - 1)
// rounded up to bm is always enough); max_tiles = cap / bm.
extern "C" int vl_moe_align(const int* ids, int npairs, int E, int bm, int cap, int* sorted_rows, int* tile_group,
                            int* place, void* stream) {
    if (npairs <= 0) return VL_OK;
    if (E <= 0 || E > MOE_MAX_EXPERTS || bm <= 0 || cap % bm || cap < npairs) return VL_ERR_ARGUMENT;
    if ((long long)cap < (long long)npairs + (long long)min(E, npairs) * (bm - 1)) return VL_ERR_ARGUMENT;
    return vl_launch(moe_align_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, ids, npairs, E, bm, cap, cap / bm,
                     sorted_rows, tile_group, place);
}

extern "C" int vl_moe_gather(const void* h, int dtype, const int* sorted_rows, const float* weights, int cap, int top,
                             int K, int scale_input, void* rows, void* stream) {
    if (cap <= 0) return VL_OK;
    if (top <= 0 || K <= 0) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(moe_gather_kernel<float>, dim3(cap), dim3(128), 0, s, (const float*)h, sorted_rows, weights, top, K,
                         scale_input, (float*)rows);
    if (dtype == VL_BF16)
        return vl_launch(moe_gather_kernel<bf16>, dim3(cap), dim3(128), 0, s, (const bf16*)h, sorted_rows, weights, top, K,
                         scale_input, (bf16*)rows);
    return VL_ERR_UNSUPPORTED;
}

extern "C" int vl_moe_combine(const void* result, int dtype, const int* place, const float* weights, int T, int top,
                              int N, int scale_output, void* out, const void* add, void* stream) {
    if (T <= 0) return VL_OK;
    if (top <= 0 || N <= 0) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(moe_combine_kernel<float>, dim3(T, (N + 511) / 512), dim3(128), 0, s, (const float*)result, place, weights, top, N,
                         scale_output, (float*)out, (const float*)add);
    if (dtype == VL_BF16)
        return vl_launch(moe_combine_kernel<bf16>, dim3(T, (N + 511) / 512), dim3(128), 0, s, (const bf16*)result, place, weights, top, N,
                         scale_output, (bf16*)out, (const bf16*)add);
    return VL_ERR_UNSUPPORTED;
}
