// Embedding gather and RMS norm with the residual sum folded in.
//
// The residual stream `x` is float32 in every mode.  A block hands the next
// norm a pending `delta` (the previous mixer's or feed-forward's output, in the
// activation dtype); the norm kernel adds it into `x` in float32, then norms:
//     x <- x + delta;   h = x / sqrt(mean(x^2) + eps) * w
// (formula: crates/model/src/components/norm/rms_norm.rs:26-49 of the reference).
// One block of 256 threads per row; the order of the additions of the mean is a
// function of the row length alone.
#include "common.cuh"

template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                             float* __restrict__ x, int H, int V, float scale, unsigned* err) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* row = x + (size_t)t * H;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) atomicOr(err, VL_DEV_BAD_TOKEN);
        for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = 0.f;
        return;
    }
    const TW* src = table + (size_t)id * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = to_f32(src[i]) * scale;   // float32; times 1 is exact
}

// rows == nullptr: row r of the output is row r of x (and x is updated in place
// when delta is given).  rows != nullptr: output row r is made from x[rows[r]]
// (+ delta[rows[r]]) and x is left untouched.
template <typename TA>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TA* __restrict__ delta,
                                   const int* __restrict__ rows, const float* __restrict__ w,
                                   TA* __restrict__ out, int H, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* xr = x + (size_t)src * H;
    const TA* dr = delta ? delta + (size_t)src * H : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += 256) {
        float v = xr[i];
        if (dr) {
            v += to_f32(dr[i]);
            if (!rows) xr[i] = v;
        }
        ss += v * v;
    }
    ss = block_sum<256>(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TA* o = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += 256) {
        float v = xr[i];
        if (dr && rows) v += to_f32(dr[i]);
        o[i] = from_f32<TA>(v * inv * w[i]);
    }
}

// The same function with a row kept in registers: 16-byte loads, one pass over memory.
// Thread i holds the float4 pieces i, i + 256, ... of the row (H a multiple of 4, at most
// 256 * 4 * VPT values).  The sum of squares is taken piece by piece in that fixed order.
template <typename TA, int VPT>
__global__ void __launch_bounds__(256)
add_rmsnorm_vec_kernel(float* __restrict__ x, const TA* __restrict__ delta, const int* __restrict__ rows,
                       const float* __restrict__ w, TA* __restrict__ out, int H, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* xr = x + (size_t)src * H;
    const TA* dr = delta ? delta + (size_t)src * H : nullptr;
    const int H4 = H >> 2;
    float4 v[VPT];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < H4) {
            v[i] = Quad<float>::load(xr + 4 * c);
            if (dr) {
                const float4 d = Quad<TA>::load(dr + 4 * c);
                v[i].x += d.x; v[i].y += d.y; v[i].z += d.z; v[i].w += d.w;
                if (!rows) Quad<float>::store(xr + 4 * c, v[i]);
            }
            ss += v[i].x * v[i].x; ss += v[i].y * v[i].y; ss += v[i].z * v[i].z; ss += v[i].w * v[i].w;
        }
    }
    ss = block_sum<256>(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TA* o = out + (size_t)r * H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < H4) {
            const float4 g = Quad<float>::load(w + 4 * c);
            Quad<TA>::store(o + 4 * c, make_float4(v[i].x * inv * g.x, v[i].y * inv * g.y, v[i].z * inv * g.z, v[i].w * inv * g.w));
        }
    }
}

template <typename TA>
static bool launch_rmsnorm_vec(float* x, const TA* delta, const int* rows, const float* w, TA* out, int R, int H,
                               float eps, cudaStream_t s) {
    if (H % 4) return false;
    const int pieces = (H / 4 + 255) / 256;
    if (pieces <= 1) vl_launch(add_rmsnorm_vec_kernel<TA, 1>, dim3(R), dim3(256), 0, s, x, delta, rows, w, out, H, eps);
    else if (pieces <= 2) vl_launch(add_rmsnorm_vec_kernel<TA, 2>, dim3(R), dim3(256), 0, s, x, delta, rows, w, out, H, eps);
    else if (pieces <= 4) vl_launch(add_rmsnorm_vec_kernel<TA, 4>, dim3(R), dim3(256), 0, s, x, delta, rows, w, out, H, eps);
    else if (pieces <= 8) vl_launch(add_rmsnorm_vec_kernel<TA, 8>, dim3(R), dim3(256), 0, s, x, delta, rows, w, out, H, eps);
    else return false;
    return true;
}

// y[r, c] += bias[c] for a linear layer with a bias vector: the product's result is widened, the float32
// bias added and the sum rounded once.
template <typename TA>
__global__ void add_bias_kernel(TA* __restrict__ y, const float* __restrict__ bias, size_t n, int cols) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = from_f32<TA>(to_f32(y[i]) + bias[i % (size_t)cols]);
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f32<TO>(to_f32(in[i]));
}

// Layer norm with a weight and no bias, h = (y - mean y) / sqrt(var y + eps) * w with the variance as the mean of the
// squared deviations (two passes over the row, float32), in the two places a block that norms its sub-layers'
// OUTPUTS needs it:
//   layernorm_add_kernel   x[r] += LN(y[r]) * w  (y: a sub-layer's output in the activation dtype; x: the float32
//                          stream) and, when asked, cast[r] = x[r] in the activation dtype: the next sub-layer's input
//   layernorm_rows_kernel  out[r] = LN(x[rows[r]]) * w  (the model's last norm on the rows whose logits are wanted)
// One block of 256 threads per row; the order of the sums depends on the row length alone.
template <typename TA>
__global__ void __launch_bounds__(256)
layernorm_add_kernel(const TA* __restrict__ y, const float* __restrict__ w, float eps, float* __restrict__ x,
                     TA* __restrict__ cast, int H) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const TA* yr = y + (size_t)r * H;
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += 256) s += to_f32(yr[i]);
    const float mean = block_sum<256>(s, scratch) / (float)H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += 256) { const float d = to_f32(yr[i]) - mean; ss += d * d; }
    const float inv = 1.0f / sqrtf(block_sum<256>(ss, scratch) / (float)H + eps);
    float* xr = x + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += 256) {
        const float v = xr[i] + (to_f32(yr[i]) - mean) * inv * w[i];
        xr[i] = v;
        if (cast) cast[(size_t)r * H + i] = from_f32<TA>(v);
    }
}

// The same with the row of y kept in registers (H a multiple of 4, at most 256 * 4 * VPT values): one read of y,
// one read and one write of x, one write of the cast, 16-byte accesses.  Thread i holds the pieces i, i + 256, ...
template <typename TA, int VPT>
__global__ void __launch_bounds__(256)
layernorm_add_vec_kernel(const TA* __restrict__ y, const float* __restrict__ w, float eps, float* __restrict__ x,
                         TA* __restrict__ cast, int H) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, H4 = H >> 2;
    const TA* yr = y + (size_t)r * H;
    float4 v[VPT];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < H4) {
            v[i] = Quad<TA>::load(yr + 4 * c);
            s += v[i].x; s += v[i].y; s += v[i].z; s += v[i].w;
        }
    }
    const float mean = block_sum<256>(s, scratch) / (float)H;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < H4) {
            v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
            ss += v[i].x * v[i].x; ss += v[i].y * v[i].y; ss += v[i].z * v[i].z; ss += v[i].w * v[i].w;
        }
    }
    const float inv = 1.0f / sqrtf(block_sum<256>(ss, scratch) / (float)H + eps);
    float* xr = x + (size_t)r * H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < H4) {
            const float4 g = Quad<float>::load(w + 4 * c);
            float4 o = Quad<float>::load(xr + 4 * c);
            o.x += v[i].x * inv * g.x; o.y += v[i].y * inv * g.y; o.z += v[i].z * inv * g.z; o.w += v[i].w * inv * g.w;
            Quad<float>::store(xr + 4 * c, o);
            if (cast) Quad<TA>::store(cast + (size_t)r * H + 4 * c, o);
        }
    }
}

template <typename TA>
static bool launch_layernorm_add_vec(const TA* y, const float* w, float eps, float* x, TA* cast, int R, int H, cudaStream_t s) {
    if (H % 4) return false;
    const int pieces = (H / 4 + 255) / 256;
    if (pieces <= 1) vl_launch(layernorm_add_vec_kernel<TA, 1>, dim3(R), dim3(256), 0, s, y, w, eps, x, cast, H);
    else if (pieces <= 2) vl_launch(layernorm_add_vec_kernel<TA, 2>, dim3(R), dim3(256), 0, s, y, w, eps, x, cast, H);
    else if (pieces <= 4) vl_launch(layernorm_add_vec_kernel<TA, 4>, dim3(R), dim3(256), 0, s, y, w, eps, x, cast, H);
    else if (pieces <= 8) vl_launch(layernorm_add_vec_kernel<TA, 8>, dim3(R), dim3(256), 0, s, y, w, eps, x, cast, H);
    else return false;
    return true;
}

template <typename TA>
__global__ void __launch_bounds__(256)
layernorm_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                      float eps, TA* __restrict__ out, int H) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += 256) s += xr[i];
    const float mean = block_sum<256>(s, scratch) / (float)H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += 256) { const float d = xr[i] - mean; ss += d * d; }
    const float inv = 1.0f / sqrtf(block_sum<256>(ss, scratch) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += 256) out[(size_t)r * H + i] = from_f32<TA>((xr[i] - mean) * inv * w[i]);
}

extern "C" int vl_layernorm_add(const void* y, int act_dtype, const float* w, float eps, float* x, void* cast,
                                int R, int H, void* stream) {
    if (R <= 0) return VL_OK;
    if (H <= 0) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == VL_F32) {
        if (launch_layernorm_add_vec<float>((const float*)y, w, eps, x, (float*)cast, R, H, s)) return vl_launch_status();
        return vl_launch(layernorm_add_kernel<float>, dim3(R), dim3(256), 0, s, (const float*)y, w, eps, x, (float*)cast, H);
    }
    if (act_dtype == VL_BF16) {
        if (launch_layernorm_add_vec<bf16>((const bf16*)y, w, eps, x, (bf16*)cast, R, H, s)) return vl_launch_status();
        return vl_launch(layernorm_add_kernel<bf16>, dim3(R), dim3(256), 0, s, (const bf16*)y, w, eps, x, (bf16*)cast, H);
    }
    return VL_ERR_UNSUPPORTED;
}

extern "C" int vl_layernorm_rows(const float* x, const int* rows, const float* w, float eps, void* out, int act_dtype,
                                 int R, int H, void* stream) {
    if (R <= 0) return VL_OK;
    if (H <= 0) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == VL_F32)
        return vl_launch(layernorm_rows_kernel<float>, dim3(R), dim3(256), 0, s, x, rows, w, eps, (float*)out, H);
    if (act_dtype == VL_BF16)
        return vl_launch(layernorm_rows_kernel<bf16>, dim3(R), dim3(256), 0, s, x, rows, w, eps, (bf16*)out, H);
    return VL_ERR_UNSUPPORTED;
}

// RMS norm of a sub-layer's OUTPUT added into the stream with a factor: x[r] += mult * (y[r] / sqrt(mean(y[r]^2) + eps) * w)
// (y in the activation dtype, x the float32 stream, everything between in float32) and, when asked, cast[r] = x[r] in
// the activation dtype: the next sub-layer's input.  `bias` (or null): a vector added to every row of y first, in float32
// (the bias of the product that made y, left to this kernel).  The row of y is kept in registers where it fits (H a multiple of
// 4, at most 256 * 4 * VPT values), else read twice.  The order of the sums depends on the row length alone.
template <typename TA>
__global__ void __launch_bounds__(256)
rmsnorm_add_kernel(const TA* __restrict__ y, const float* __restrict__ bias, const float* __restrict__ w, float eps, float mult,
                   float* __restrict__ x, TA* __restrict__ cast, int H, const TA* __restrict__ y2, float s1, float s2) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const TA* yr = y + (size_t)r * H;
    const TA* y2r = y2 ? y2 + (size_t)r * H : nullptr;          // the normed row is s1 * y + s2 * y2 (two sub-layers side by side)
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += 256) {
        const float d = (y2r ? s1 * to_f32(yr[i]) + s2 * to_f32(y2r[i]) : to_f32(yr[i])) + (bias ? bias[i] : 0.f);
        ss += d * d;
    }
    const float inv = 1.0f / sqrtf(block_sum<256>(ss, scratch) / (float)H + eps);
    float* xr = x + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += 256) {
        const float d = (y2r ? s1 * to_f32(yr[i]) + s2 * to_f32(y2r[i]) : to_f32(yr[i])) + (bias ? bias[i] : 0.f);
        const float v = xr[i] + mult * (d * inv * w[i]);
        xr[i] = v;
        if (cast) cast[(size_t)r * H + i] = from_f32<TA>(v);
    }
}

template <typename TA, int VPT>
__global__ void __launch_bounds__(256)
rmsnorm_add_vec_kernel(const TA* __restrict__ y, const float* __restrict__ bias, const float* __restrict__ w, float eps, float mult,
                       float* __restrict__ x, TA* __restrict__ cast, int H, const TA* __restrict__ y2, float s1, float s2) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, H4 = H >> 2;
    const TA* yr = y + (size_t)r * H;
    const TA* y2r = y2 ? y2 + (size_t)r * H : nullptr;          // the normed row is s1 * y + s2 * y2
    float4 v[VPT];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < H4) {
            v[i] = Quad<TA>::load(yr + 4 * c);
            if (y2r) {
                const float4 u = Quad<TA>::load(y2r + 4 * c);
                v[i].x = s1 * v[i].x + s2 * u.x; v[i].y = s1 * v[i].y + s2 * u.y;
                v[i].z = s1 * v[i].z + s2 * u.z; v[i].w = s1 * v[i].w + s2 * u.w;
            }
            if (bias) {
                const float4 b = Quad<float>::load(bias + 4 * c);
                v[i].x += b.x; v[i].y += b.y; v[i].z += b.z; v[i].w += b.w;
            }
            ss += v[i].x * v[i].x; ss += v[i].y * v[i].y; ss += v[i].z * v[i].z; ss += v[i].w * v[i].w;
        }
    }
    const float inv = 1.0f / sqrtf(block_sum<256>(ss, scratch) / (float)H + eps);
    float* xr = x + (size_t)r * H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < H4) {
            const float4 g = Quad<float>::load(w + 4 * c);
            float4 o = Quad<float>::load(xr + 4 * c);
            o.x += mult * (v[i].x * inv * g.x); o.y += mult * (v[i].y * inv * g.y);
            o.z += mult * (v[i].z * inv * g.z); o.w += mult * (v[i].w * inv * g.w);
            Quad<float>::store(xr + 4 * c, o);
            if (cast) Quad<TA>::store(cast + (size_t)r * H + 4 * c, o);
        }
    }
}

template <typename TA>
static int launch_rmsnorm_add(const TA* y, const float* bias, const float* w, float eps, float mult, float* x, TA* cast, int R, int H,
                              const TA* y2, float s1, float s2, cudaStream_t s) {
    const int pieces = (H / 4 + 255) / 256;
    if (H % 4 == 0 && pieces <= 1) return vl_launch(rmsnorm_add_vec_kernel<TA, 1>, dim3(R), dim3(256), 0, s, y, bias, w, eps, mult, x, cast, H, y2, s1, s2);
    if (H % 4 == 0 && pieces <= 2) return vl_launch(rmsnorm_add_vec_kernel<TA, 2>, dim3(R), dim3(256), 0, s, y, bias, w, eps, mult, x, cast, H, y2, s1, s2);
    if (H % 4 == 0 && pieces <= 4) return vl_launch(rmsnorm_add_vec_kernel<TA, 4>, dim3(R), dim3(256), 0, s, y, bias, w, eps, mult, x, cast, H, y2, s1, s2);
    if (H % 4 == 0 && pieces <= 8) return vl_launch(rmsnorm_add_vec_kernel<TA, 8>, dim3(R), dim3(256), 0, s, y, bias, w, eps, mult, x, cast, H, y2, s1, s2);
    return vl_launch(rmsnorm_add_kernel<TA>, dim3(R), dim3(256), 0, s, y, bias, w, eps, mult, x, cast, H, y2, s1, s2);
}

extern "C" int vl_rmsnorm_add(const void* y, int act_dtype, const float* bias, const float* w, float eps, float mult, float* x, void* cast,
                              int R, int H, const void* y2, float s1, float s2, void* stream) {
    if (R <= 0) return VL_OK;
    if (H <= 0) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == VL_F32) return launch_rmsnorm_add<float>((const float*)y, bias, w, eps, mult, x, (float*)cast, R, H, (const float*)y2, s1, s2, s);
    if (act_dtype == VL_BF16) return launch_rmsnorm_add<bf16>((const bf16*)y, bias, w, eps, mult, x, (bf16*)cast, R, H, (const bf16*)y2, s1, s2, s);
    return VL_ERR_UNSUPPORTED;
}

extern "C" int vl_embed(const int* ids, const void* table, int table_dtype, float* x,
                        int T, int H, int V, float scale, unsigned* err, void* stream) {
    if (T <= 0) return VL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (table_dtype == VL_F32)
        vl_launch(embed_kernel<float>, dim3(T), dim3(256), 0, s, ids, (const float*)table, x, H, V, scale, err);
    else if (table_dtype == VL_BF16)
        vl_launch(embed_kernel<bf16>, dim3(T), dim3(256), 0, s, ids, (const bf16*)table, x, H, V, scale, err);
    else
        return VL_ERR_UNSUPPORTED;
    return vl_launch_status();
}

extern "C" int vl_add_rmsnorm(float* x, const void* delta, const int* rows, const float* w, void* out,
                              int act_dtype, int R, int H, float eps, void* stream) {
    if (R <= 0) return VL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == VL_F32) {
        if (!launch_rmsnorm_vec<float>(x, (const float*)delta, rows, w, (float*)out, R, H, eps, s))
            add_rmsnorm_kernel<float><<<R, 256, 0, s>>>(x, (const float*)delta, rows, w, (float*)out, H, eps);
    } else if (act_dtype == VL_BF16) {
        if (!launch_rmsnorm_vec<bf16>(x, (const bf16*)delta, rows, w, (bf16*)out, R, H, eps, s))
            add_rmsnorm_kernel<bf16><<<R, 256, 0, s>>>(x, (const bf16*)delta, rows, w, (bf16*)out, H, eps);
    } else {
        return VL_ERR_UNSUPPORTED;
    }
    return vl_launch_status();
}

extern "C" int vl_add_bias(void* y, int act_dtype, const float* bias, long long rows, int cols, void* stream) {
    if (rows <= 0 || cols <= 0) return VL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t n = (size_t)rows * (size_t)cols;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (act_dtype == VL_F32)
        add_bias_kernel<float><<<blocks, 256, 0, s>>>((float*)y, bias, n, cols);
    else if (act_dtype == VL_BF16)
        add_bias_kernel<bf16><<<blocks, 256, 0, s>>>((bf16*)y, bias, n, cols);
    else
        return VL_ERR_UNSUPPORTED;
    return vl_launch_status();
}

extern "C" int vl_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n, void* stream) {
    if (n <= 0) return VL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (in_dtype == VL_F32 && out_dtype == VL_BF16)
        cast_kernel<float, bf16><<<blocks, 256, 0, s>>>((const float*)in, (bf16*)out, (size_t)n);
    else if (in_dtype == VL_BF16 && out_dtype == VL_F32)
        cast_kernel<bf16, float><<<blocks, 256, 0, s>>>((const bf16*)in, (float*)out, (size_t)n);
    else
        return VL_ERR_UNSUPPORTED;
    return vl_launch_status();
}
