// Latent attention: the step between the down-projections and the attention over the latent cache.
//
// A token's row of the stacked down-projection holds [a_q (q_rank values) | a_kv (kv_rank values)].
// Both halves are RMS-normed with a weight of their own (float32 arithmetic):
//     c_q = a_q  / sqrt(mean(a_q^2)  + eps) * w_q      -> cq_out [T, q_rank]   (input of the query up-projection)
//     c   = a_kv / sqrt(mean(a_kv^2) + eps) * w_kv     -> cache row `slots[t]` (the only thing kept per token)
// The cache row is `row_width` wide (kv_rank rounded up to what the attention kernels take); the tail is
// written as zeros, so that keys of any rank are plain rows of a one-head cache [pages, 1, page_size, row_width].
// A row may carry a third part behind a_kv: `rot_dim` values that are NOT normed, one rotated key part shared by all
// heads.  Its first `rot` features are turned by the token's position (pairs (i, i + rot/2), angle = (float)pos *
// inv_freq[i], float32) and the part is written into the cache row behind the latent, [c | rotated part | zeros].
// vl_rope_heads turns the matching part of every query head in place.
// One block of 128 threads per token; the order of every sum depends on the sizes alone.
// A negative slot (a padded token of a graph step) writes no cache row; a slot outside the pool sets
// VL_DEV_BAD_SLOT and is skipped.
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(128)
latent_norm_write_kernel(const T* __restrict__ proj, int ld, int q_rank, int kv_rank,
                         const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                         T* __restrict__ cq_out, const int* __restrict__ slots, T* __restrict__ cache,
                         int row_width, long long num_slots, int rot_dim, int rot, const float* __restrict__ inv_freq,
                         const int* __restrict__ positions, unsigned* err) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const float pos = (rot > 0) ? (float)positions[t] : 0.f;
    pdl_wait();
    const T* row = proj + (size_t)t * ld;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += 128) { const float v = to_f32(row[i]); sq += v * v; }
    for (int i = threadIdx.x; i < kv_rank; i += 128) { const float v = to_f32(row[q_rank + i]); sk += v * v; }
    sq = block_sum<128>(sq, scratch);
    sk = block_sum<128>(sk, scratch);
    const float iq = 1.0f / sqrtf(sq / (float)q_rank + eps);
    const float ik = 1.0f / sqrtf(sk / (float)kv_rank + eps);
    T* cq = cq_out + (size_t)t * q_rank;
    for (int i = threadIdx.x; i < q_rank; i += 128) cq[i] = from_f32<T>(to_f32(row[i]) * iq * wq[i]);
    if (!slots) return;
    const long long slot = slots[t];
    if (slot < 0) return;
    if (slot >= num_slots) {
        if (threadIdx.x == 0) atomicOr(err, VL_DEV_BAD_SLOT);
        return;
    }
    T* dst = cache + (size_t)slot * row_width;
    const int half = rot / 2;
    for (int i = threadIdx.x; i < row_width; i += 128) {
        float v = 0.f;
        if (i < kv_rank) {
            v = to_f32(row[q_rank + i]) * ik * wkv[i];
        } else if (i < kv_rank + rot_dim) {
            const int e = i - kv_rank;
            const T* tail = row + q_rank + kv_rank;
            v = to_f32(tail[e]);
            if (e < rot) {
                const int f = e < half ? e : e - half;
                float sn, cs;
                sincosf(pos * inv_freq[f], &sn, &cs);
                v = e < half ? v * cs - to_f32(tail[e + half]) * sn : v * cs + to_f32(tail[e - half]) * sn;
            }
        }
        dst[i] = from_f32<T>(v);
    }
}

// x [T, ld]: for every head h < heads the features col0 + h * stride + [0, rot) are turned in place by the token's
// position (rotate-half pairs, float32 angles, sine and cosine).  A block per token, a thread per (head, pair).
template <typename T>
__global__ void __launch_bounds__(128)
rope_heads_kernel(T* __restrict__ x, int ld, int col0, int stride, int heads, int rot, const float* __restrict__ inv_freq,
                  const int* __restrict__ positions) {
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const float pos = (float)positions[t];
    pdl_wait();
    const int half = rot / 2;
    T* row = x + (size_t)t * ld + col0;
    for (int idx = threadIdx.x; idx < heads * half; idx += 128) {
        const int h = idx / half, i = idx - h * half;
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        T* p = row + (size_t)h * stride;
        const float u = to_f32(p[i]), v = to_f32(p[i + half]);
        p[i] = from_f32<T>(u * cs - v * sn);
        p[i + half] = from_f32<T>(v * cs + u * sn);
    }
}

extern "C" int vl_rope_heads(void* x, int dtype, int T, int ld, int col0, int stride, int heads, int rot, const float* inv_freq,
                             const int* positions, void* stream) {
    if (T <= 0 || rot <= 0) return VL_OK;
    if ((rot & 1) || heads <= 0 || stride < rot || col0 < 0 || col0 + (heads - 1) * stride + rot > ld || !inv_freq || !positions)
        return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(rope_heads_kernel<float>, dim3(T), dim3(128), 0, s, (float*)x, ld, col0, stride, heads, rot, inv_freq, positions);
    if (dtype == VL_BF16)
        return vl_launch(rope_heads_kernel<bf16>, dim3(T), dim3(128), 0, s, (bf16*)x, ld, col0, stride, heads, rot, inv_freq, positions);
    return VL_ERR_UNSUPPORTED;
}

extern "C" int vl_latent_norm_write(const void* proj, int dtype, int ld, int T, int q_rank, int kv_rank,
                                    const float* wq, const float* wkv, float eps, void* cq_out,
                                    const int* slots, void* cache, int row_width, long long num_slots,
                                    int rot_dim, int rot, const float* inv_freq, const int* positions,
                                    unsigned* err, void* stream) {
    if (T <= 0) return VL_OK;
    if (q_rank <= 0 || kv_rank <= 0 || rot_dim < 0 || ld < q_rank + kv_rank + rot_dim || row_width < kv_rank + rot_dim)
        return VL_ERR_ARGUMENT;
    if (rot < 0 || (rot & 1) || rot > rot_dim || (rot > 0 && (!inv_freq || !positions))) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(latent_norm_write_kernel<float>, dim3(T), dim3(128), 0, s, (const float*)proj, ld, q_rank, kv_rank,
                         wq, wkv, eps, (float*)cq_out, slots, (float*)cache, row_width, num_slots, rot_dim, rot, inv_freq, positions, err);
    if (dtype == VL_BF16)
        return vl_launch(latent_norm_write_kernel<bf16>, dim3(T), dim3(128), 0, s, (const bf16*)proj, ld, q_rank, kv_rank,
                         wq, wkv, eps, (bf16*)cq_out, slots, (bf16*)cache, row_width, num_slots, rot_dim, rot, inv_freq, positions, err);
    return VL_ERR_UNSUPPORTED;
}
