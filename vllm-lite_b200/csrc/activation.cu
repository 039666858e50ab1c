// SwiGLU activation on the fused gate|up projection:
//     out[t, i] = silu(gate_i) * up_i,   silu(z) = z / (1 + exp(-z))
// (crates/model/src/components/mlp/swiglu.rs:18-31 of the reference).
// Two layouts of the [T, 2I] input: group = 0, the gate columns then the up columns
// (gate_i = gu[t, i], up_i = gu[t, I + i]); group = g > 0, blocks of g gate columns followed by
// their g up columns (gate_i = gu[t, 2g*(i/g) + i%g], up_i = that + g), which is what lets a
// matrix-product kernel apply the activation to the tile it holds.
// The arithmetic is float32; input and output are in the activation dtype.
#include "common.cuh"

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total, int group) {
    pdl_launch_dependents();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const size_t gi = group > 0 ? (size_t)2 * group * (i / group) + i % group : (size_t)i;
    const float g = to_f32(gu[t * 2 * (size_t)I + gi]);
    const float u = to_f32(gu[t * 2 * (size_t)I + gi + (group > 0 ? group : I)]);
    out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

extern "C" int vl_silu_mul(const void* gu, void* out, int dtype, int T, int I, int group, void* stream) {
    if (T <= 0 || I <= 0) return VL_OK;
    if (group < 0 || (group > 0 && I % group)) return VL_ERR_ARGUMENT;
    const size_t total = (size_t)T * I;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)gu, (float*)out, I, total, group);
    else if (dtype == VL_BF16)
        return vl_launch(silu_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)gu, (bf16*)out, I, total, group);
    else
        return VL_ERR_UNSUPPORTED;
    return vl_launch_status();
}

// Gated activations of other feed-forwards, on the same [T, 2I] layouts:  out = f(gate, up)
//   VL_ACT_SILU          silu(g) * u
//   VL_ACT_RELU          max(g, 0) * u
//   VL_ACT_CAPPED_SWISH  g' = min(g, limit), u' = clamp(u, -limit, limit):  g' * sigmoid(alpha * g') * (u' + shift)
// alpha, limit and shift are the caller's constants (a limit <= 0 means no limit).  `bias` (float32 [2I], optional)
// is added to the gate and up columns first: the bias vectors of the two projections, which then need no pass of their own.
#define VL_ACT_SILU 0
#define VL_ACT_RELU 1
#define VL_ACT_CAPPED_SWISH 2

template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total, int group, int act,
                                 float alpha, float limit, float shift, const float* __restrict__ bias) {
    pdl_launch_dependents();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const size_t gi = group > 0 ? (size_t)2 * group * (i / group) + i % group : (size_t)i;
    float g = to_f32(gu[t * 2 * (size_t)I + gi]);
    float u = to_f32(gu[t * 2 * (size_t)I + gi + (group > 0 ? group : I)]);
    if (bias) {                                      // the projections' bias vectors, in the columns' own layout
        g += bias[gi];
        u += bias[gi + (group > 0 ? group : I)];
    }
    float r;
    if (act == VL_ACT_RELU) {
        r = fmaxf(g, 0.f) * u;
    } else if (act == VL_ACT_CAPPED_SWISH) {
        if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
        r = g / (1.0f + expf(-alpha * g)) * (u + shift);
    } else {
        r = g / (1.0f + expf(-g)) * u;
    }
    out[idx] = from_f32<T>(r);
}

// The plain-halves layout (group 0) with I a multiple of 8: eight outputs a thread, 16-byte accesses.
template <typename T>
__global__ void gated_act_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total8, int act,
                                     float alpha, float limit, float shift, const float* __restrict__ bias) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total8) return;
    const int per_row = I / 8;
    const size_t t = idx / per_row;
    const int i = (int)(idx - t * per_row) * 8;
    float g[8], u[8], r[8];
    load8(gu + t * 2 * (size_t)I + i, g);
    load8(gu + t * 2 * (size_t)I + I + i, u);
    if (bias) {
#pragma unroll
        for (int e = 0; e < 8; ++e) { g[e] += bias[i + e]; u[e] += bias[I + i + e]; }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        float gg = g[e], uu = u[e];
        if (act == VL_ACT_RELU) {
            r[e] = fmaxf(gg, 0.f) * uu;
        } else if (act == VL_ACT_CAPPED_SWISH) {
            if (limit > 0.f) { gg = fminf(gg, limit); uu = fminf(fmaxf(uu, -limit), limit); }
            r[e] = gg / (1.0f + expf(-alpha * gg)) * (uu + shift);
        } else {
            r[e] = gg / (1.0f + expf(-gg)) * uu;
        }
    }
    store8(out + t * (size_t)I + i, r);
}

extern "C" int vl_gated_act(const void* gu, void* out, int dtype, int T, int I, int group, int act, float alpha,
                            float limit, float shift, const float* bias, void* stream) {
    if (T <= 0 || I <= 0) return VL_OK;
    if (group < 0 || (group > 0 && I % group) || act < 0 || act > 2) return VL_ERR_ARGUMENT;
    const size_t total = (size_t)T * I;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (group == 0 && I % 8 == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0) {
        const size_t total8 = total / 8;
        const unsigned b8 = (unsigned)((total8 + 255) / 256);
        if (dtype == VL_F32)
            return vl_launch(gated_act_vec_kernel<float>, dim3(b8), dim3(256), 0, s, (const float*)gu, (float*)out, I, total8, act,
                             alpha, limit, shift, bias);
        if (dtype == VL_BF16)
            return vl_launch(gated_act_vec_kernel<bf16>, dim3(b8), dim3(256), 0, s, (const bf16*)gu, (bf16*)out, I, total8, act,
                             alpha, limit, shift, bias);
    }
    if (dtype == VL_F32)
        return vl_launch(gated_act_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)gu, (float*)out, I, total, group,
                         act, alpha, limit, shift, bias);
    if (dtype == VL_BF16)
        return vl_launch(gated_act_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)gu, (bf16*)out, I, total, group,
                         act, alpha, limit, shift, bias);
    return VL_ERR_UNSUPPORTED;
}

// A function of one argument, element by element in float32: act 16 = the square of max(v, 0), 17 = tanh(v) (the codes
// continue those of the gated activations, which take two).
__device__ __forceinline__ float unary_value(float v, int act) {
    if (act == 16) { v = fmaxf(v, 0.f); return v * v; }
    return act == 17 ? tanhf(v) : v;
}
// VEC = 4: a thread takes four neighbouring values (one 16- or 8-byte access each way), when the buffers allow it.
template <typename T, int VEC>
__global__ void unary_act_kernel(const T* __restrict__ in, T* __restrict__ out, size_t n, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = ((size_t)blockIdx.x * 256 + threadIdx.x) * VEC;
    if (i >= n) return;
    if (VEC == 4) {
        const float4 v = Quad<T>::load(in + i);
        Quad<T>::store(out + i, make_float4(unary_value(v.x, act), unary_value(v.y, act), unary_value(v.z, act), unary_value(v.w, act)));
    } else {
        out[i] = from_f32<T>(unary_value(to_f32(in[i]), act));
    }
}

extern "C" int vl_unary_act(const void* in, void* out, int dtype, long long n, int act, void* stream) {
    if (n <= 0) return VL_OK;
    if (act != 16 && act != 17) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = n % 4 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0;
    const unsigned blocks = (unsigned)((n / (vec ? 4 : 1) + 255) / 256);
    if (dtype == VL_F32) {
        if (vec) return vl_launch(unary_act_kernel<float, 4>, dim3(blocks), dim3(256), 0, s, (const float*)in, (float*)out, (size_t)n, act);
        return vl_launch(unary_act_kernel<float, 1>, dim3(blocks), dim3(256), 0, s, (const float*)in, (float*)out, (size_t)n, act);
    }
    if (dtype == VL_BF16) {
        if (vec) return vl_launch(unary_act_kernel<bf16, 4>, dim3(blocks), dim3(256), 0, s, (const bf16*)in, (bf16*)out, (size_t)n, act);
        return vl_launch(unary_act_kernel<bf16, 1>, dim3(blocks), dim3(256), 0, s, (const bf16*)in, (bf16*)out, (size_t)n, act);
    }
    return VL_ERR_UNSUPPORTED;
}

// Logits of a scaled, capped output head, in place on float32:  z <- cap * tanh(z * scale / cap)
// (cap <= 0: only the scale).
__global__ void scale_softcap_kernel(float* __restrict__ z, size_t n, float scale, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = z[i] * scale;
    z[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
}

extern "C" int vl_scale_softcap(float* z, long long n, float scale, float cap, void* stream) {
    if (n <= 0) return VL_OK;
    const unsigned blocks = (unsigned)(((size_t)n + 255) / 256);
    return vl_launch(scale_softcap_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, z, (size_t)n, scale, cap);
}

// out = sa * a + sb * b: what two mixers that run side by side on one input leave (float32 arithmetic).
template <typename T, int VEC>
__global__ void scaled_sum_kernel(const T* __restrict__ a, float sa, const T* __restrict__ b, float sb, T* __restrict__ out, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (i >= n) return;
    if (VEC == 4) {
        const float4 x = Quad<T>::load(a + i), y = Quad<T>::load(b + i);
        Quad<T>::store(out + i, make_float4(sa * x.x + sb * y.x, sa * x.y + sb * y.y, sa * x.z + sb * y.z, sa * x.w + sb * y.w));
    } else {
        out[i] = from_f32<T>(sa * to_f32(a[i]) + sb * to_f32(b[i]));
    }
}

extern "C" int vl_scaled_sum(const void* a, float sa, const void* b, float sb, void* out, int dtype, long long n, void* stream) {
    if (n <= 0) return VL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = n % 4 == 0 && (((uintptr_t)a | (uintptr_t)b | (uintptr_t)out) & 15) == 0;
    const unsigned blocks = (unsigned)((n / (vec ? 4 : 1) + 255) / 256);
    if (dtype == VL_F32) {
        if (vec) return vl_launch(scaled_sum_kernel<float, 4>, dim3(blocks), dim3(256), 0, s, (const float*)a, sa, (const float*)b, sb, (float*)out, (size_t)n);
        return vl_launch(scaled_sum_kernel<float, 1>, dim3(blocks), dim3(256), 0, s, (const float*)a, sa, (const float*)b, sb, (float*)out, (size_t)n);
    }
    if (dtype == VL_BF16) {
        if (vec) return vl_launch(scaled_sum_kernel<bf16, 4>, dim3(blocks), dim3(256), 0, s, (const bf16*)a, sa, (const bf16*)b, sb, (bf16*)out, (size_t)n);
        return vl_launch(scaled_sum_kernel<bf16, 1>, dim3(blocks), dim3(256), 0, s, (const bf16*)a, sa, (const bf16*)b, sb, (bf16*)out, (size_t)n);
    }
    return VL_ERR_UNSUPPORTED;
}

// x[t, i] <- x[t, i] * sigmoid(g[t, gcol + i]) for i < n, element by element in float32 (an output gate on the
// concatenated heads of an attention; x rows ldx wide, g rows ldg wide).
__device__ __forceinline__ float gate_of(float g) { return 1.0f / (1.0f + expf(-g)); }
template <typename T, int VEC>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, int ldx, const T* __restrict__ g, int ldg, int gcol, int n, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = ((size_t)blockIdx.x * 256 + threadIdx.x) * VEC;
    if (idx >= total) return;
    const size_t t = idx / n;
    const int i = (int)(idx - t * n);
    T* p = x + t * ldx + i;
    const T* q = g + t * ldg + gcol + i;
    if (VEC == 4) {
        const float4 v = Quad<T>::load(p), w = Quad<T>::load(q);
        Quad<T>::store(p, make_float4(v.x * gate_of(w.x), v.y * gate_of(w.y), v.z * gate_of(w.z), v.w * gate_of(w.w)));
    } else {
        *p = from_f32<T>(to_f32(*p) * gate_of(to_f32(*q)));
    }
}

extern "C" int vl_sigmoid_gate(void* x, int ldx, const void* g, int ldg, int gcol, int dtype, int T, int n, void* stream) {
    if (T <= 0 || n <= 0) return VL_OK;
    if (ldx < n || gcol < 0 || ldg < gcol + n) return VL_ERR_ARGUMENT;
    const size_t total = (size_t)T * n;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = n % 4 == 0 && ldx % 4 == 0 && ldg % 4 == 0 && gcol % 4 == 0 && (((uintptr_t)x | (uintptr_t)g) & 15) == 0;
    const unsigned blocks = (unsigned)((total / (vec ? 4 : 1) + 255) / 256);
    if (dtype == VL_F32) {
        if (vec) return vl_launch(sigmoid_gate_kernel<float, 4>, dim3(blocks), dim3(256), 0, s, (float*)x, ldx, (const float*)g, ldg, gcol, n, total);
        return vl_launch(sigmoid_gate_kernel<float, 1>, dim3(blocks), dim3(256), 0, s, (float*)x, ldx, (const float*)g, ldg, gcol, n, total);
    }
    if (dtype == VL_BF16) {
        if (vec) return vl_launch(sigmoid_gate_kernel<bf16, 4>, dim3(blocks), dim3(256), 0, s, (bf16*)x, ldx, (const bf16*)g, ldg, gcol, n, total);
        return vl_launch(sigmoid_gate_kernel<bf16, 1>, dim3(blocks), dim3(256), 0, s, (bf16*)x, ldx, (const bf16*)g, ldg, gcol, n, total);
    }
    return VL_ERR_UNSUPPORTED;
}
