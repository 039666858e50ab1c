// Per-head norm of q and k, rotary position encoding, and the write of the new
// keys and values into the paged cache, in one pass over the fused q|k|v rows.
//
//   q_head, k_head <- head / sqrt(mean(head^2) + eps) * w        (optional)
//   angle = (float)pos * inv_freq[i];  pairs (x[i], x[i + rot/2]) of the first
//   `rot` features:  x1' = x1 cos - x2 sin,  x2' = x2 cos + x1 sin   (optional)
// (crates/model/src/components/attention/rope_gqa.rs:214-248 and
//  crates/model/src/components/positional/rope.rs:507-558 of the reference).
// q is rewritten in place; k and v go to the cache slot of their token:
//   page = slot / page_size, offset = slot % page_size,
//   cache[page][kv_head][offset][:]  with cache = [pages, nkv, page_size, hd].
// A token whose slot is negative writes no cache (a call that reads another
// call's cache).  Norm, angles, sine and cosine are float32 in every mode.
//
// head_dim up to 512, any even value.
#include "rope_head.cuh"

#define ROPE_MAX_HD 512

// A block serves one token and `heads_per_block` of its heads: its 4 warps share the token's
// sine/cosine table and walk those heads (many tokens: all heads, so the table is computed once per
// token; few tokens: 4 heads, so that a decode step still fills the SMs).  A warp keeps a head in
// registers: a lane holds pairs of neighbouring features (4-byte accesses for bfloat16, 8-byte for
// float32) of the first rotated half together with their partners in the second half, and pairs of
// the features behind the rotated part.  A warp works on two heads at a time, so that the loads of
// one overlap the arithmetic of the other.
#define ROPE_THREADS 128
// The kernel is compiled for head sizes up to MAXHD = 128 and up to ROPE_MAX_HD: per lane at most
// MAXHD / 128 pairs of the first half and MAXHD / 64 pairs behind the rotated part.

template <typename T, int MAXHD>
__global__ void __launch_bounds__(ROPE_THREADS)
qk_norm_rope_write_kernel(
    T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ slots,
    const float* __restrict__ qw, const float* __restrict__ kw, float eps,
    const float* __restrict__ inv_freq, int rot,
    T* __restrict__ kcache, T* __restrict__ vcache,
    int nq, int nkv, int hd, int page_size, long long num_slots, int row_stride, unsigned* err,
    int heads_per_block) {
    __shared__ float s_cos[MAXHD / 2], s_sin[MAXHD / 2];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head_lo = blockIdx.y * heads_per_block;
    const int head_hi = min(nq + 2 * nkv, head_lo + heads_per_block);
    const int half = rot / 2;
    if (inv_freq) {                                  // positions are part of the step's description: no wait needed
        const float pos = (float)positions[t];
        for (int i = threadIdx.x; i < half; i += ROPE_THREADS) sincosf(pos * inv_freq[i], &s_sin[i], &s_cos[i]);
    }
    pdl_wait();                                      // qkv comes from the kernel before
    __syncthreads();
    const int slot = slots ? slots[t] : -1;
    bool slot_ok = slot >= 0;
    if (slot_ok && (long long)slot >= num_slots) {
        if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(err, VL_DEV_BAD_SLOT);
        slot_ok = false;
    }
    const int page = slot_ok ? slot / page_size : 0, off = slot_ok ? slot - page * page_size : 0;
    // where head `head` of this token is read and written, which norm weight it takes, whether it is rotated
    auto setup = [&](HeadRegs<T, MAXHD>& r, int head) {
        r.live = head < head_hi;
        r.src = qkv; r.out = qkv; r.w = nullptr; r.rot = 0;
        if (!r.live) return;
        r.src = qkv + (size_t)t * row_stride + (size_t)head * hd;
        const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
        if (is_q) {
            r.out = qkv + (size_t)t * row_stride + (size_t)head * hd;
        } else {
            if (!slot_ok) { r.live = false; return; }             // nothing to write for this token
            const int kvh = is_k ? head - nq : head - nq - nkv;
            r.out = (is_k ? kcache : vcache) + (((size_t)page * nkv + kvh) * page_size + off) * hd;
        }
        if (is_q || is_k) {
            r.w = is_q ? qw : kw;
            r.rot = inv_freq ? rot : 0;
        }
    };
    constexpr int WARPS = ROPE_THREADS / 32;
    for (int head = head_lo + warp; head < head_hi; head += 2 * WARPS) {
        HeadRegs<T, MAXHD> r0, r1;
        setup(r0, head);
        setup(r1, head + WARPS);
        r0.load(lane, hd);
        r1.load(lane, hd);
        r0.finish(lane, hd, eps, s_cos, s_sin);
        r1.finish(lane, hd, eps, s_cos, s_sin);
    }
}

// ---- many tokens, the whole head rotated (or none of it), head size 32 .. 512 a power of two ----
// The same function with 16-byte accesses: hd / 16 lanes share a head, a lane holds 8 neighbouring
// features of the first half and their 8 partners in the second half, so a warp works on 512 / hd
// heads at once and on two such groups in flight.  (The kernel above reads 4 bytes per lane and
// load, which leaves a prompt portion's traffic far below what the memory can deliver.)
template <typename T> struct Eight;
template <> struct Eight<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
};
template <> struct Eight<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[8]) {
        const uint4 q = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[8]) {
        uint4 q;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = q;
    }
};

template <typename T>
__global__ void __launch_bounds__(ROPE_THREADS)
qk_norm_rope_write_wide_kernel(
    T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ slots,
    const float* __restrict__ qw, const float* __restrict__ kw, float eps,
    const float* __restrict__ inv_freq, T* __restrict__ kcache, T* __restrict__ vcache,
    int nq, int nkv, int hd, int page_size, long long num_slots, int row_stride, unsigned* err) {
    __shared__ float s_cos[ROPE_MAX_HD / 2], s_sin[ROPE_MAX_HD / 2];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = hd / 2;
    const int lph = hd / 16, hpw = 32 / lph;                      // lanes per head, heads per warp
    const int nheads = nq + 2 * nkv;
    if (inv_freq) {                                  // positions are part of the step's description: no wait needed
        const float pos = (float)positions[t];
        for (int i = threadIdx.x; i < half; i += ROPE_THREADS) sincosf(pos * inv_freq[i], &s_sin[i], &s_cos[i]);
    }
    pdl_wait();                                      // qkv comes from the kernel before
    __syncthreads();
    const int slot = slots ? slots[t] : -1;
    bool slot_ok = slot >= 0;
    if (slot_ok && (long long)slot >= num_slots) {
        if (threadIdx.x == 0) atomicOr(err, VL_DEV_BAD_SLOT);
        slot_ok = false;
    }
    const int page = slot_ok ? slot / page_size : 0, off = slot_ok ? slot - page * page_size : 0;
    const int sub = lane / lph, i0 = 8 * (lane % lph);             // which head of the warp's group, first feature
    constexpr int WARPS = ROPE_THREADS / 32;
    const int per_pass = WARPS * hpw;
    for (int base = 0; base < nheads; base += 2 * per_pass) {
        float a[2][8], b[2][8];
        T* out[2];
        const float* w[2];
        bool live[2], rotate[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int head = base + u * per_pass + warp * hpw + sub;
            live[u] = head < nheads;
            out[u] = nullptr; w[u] = nullptr; rotate[u] = false;
            if (live[u]) {
                T* src = qkv + (size_t)t * row_stride + (size_t)head * hd;
                const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
                if (is_q) out[u] = src;
                else if (slot_ok) out[u] = (is_k ? kcache : vcache) + (((size_t)page * nkv + (is_k ? head - nq : head - nq - nkv)) * page_size + off) * hd;
                else live[u] = false;                              // nothing to write for this token
                if (live[u]) {
                    Eight<T>::load(src + i0, a[u]);
                    Eight<T>::load(src + i0 + half, b[u]);
                    if (is_q || is_k) { w[u] = is_q ? qw : kw; rotate[u] = inv_freq != nullptr; }
                }
            }
            if (!live[u]) {
#pragma unroll
                for (int j = 0; j < 8; ++j) { a[u][j] = 0.f; b[u][j] = 0.f; }
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            // (every lane takes part in the shuffles; lanes of a head agree on w)
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += a[u][j] * a[u][j] + b[u][j] * b[u][j];
            for (int o = 1; o < lph; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (!live[u]) continue;
            if (w[u]) {
                const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
#pragma unroll
                for (int j = 0; j < 8; ++j) { a[u][j] *= inv * w[u][i0 + j]; b[u][j] *= inv * w[u][i0 + half + j]; }
            }
            if (rotate[u]) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float c = s_cos[i0 + j], sn = s_sin[i0 + j], x1 = a[u][j], x2 = b[u][j];
                    a[u][j] = x1 * c - x2 * sn;
                    b[u][j] = x2 * c + x1 * sn;
                }
            }
            Eight<T>::store(out[u] + i0, a[u]);
            Eight<T>::store(out[u] + i0 + half, b[u]);
        }
    }
}

extern "C" int vl_qk_norm_rope_write(
    void* qkv, int dtype, const int* positions, const int* slots,
    const float* qw, const float* kw, float eps, const float* inv_freq, int rot,
    void* kcache, void* vcache, int T, int nq, int nkv, int hd, int page_size,
    long long num_slots, int row_stride, unsigned* err, void* stream) {
    if (T <= 0) return VL_OK;
    if (hd <= 0 || hd > ROPE_MAX_HD || rot < 0 || rot > hd || (rot & 1)) return VL_ERR_UNSUPPORTED;
    if (page_size <= 0 || row_stride < (nq + 2 * nkv) * hd) return VL_ERR_ARGUMENT;
    if (hd & 1) return VL_ERR_UNSUPPORTED;
    const int nheads = nq + 2 * nkv;
    cudaStream_t s = (cudaStream_t)stream;
    const bool pow2 = (hd & (hd - 1)) == 0 && hd >= 32;
    const bool aligned = row_stride % 8 == 0 && (((uintptr_t)qkv | (uintptr_t)kcache | (uintptr_t)vcache) & 31) == 0;
    // (bfloat16 only: in float32 one kernel serves every step, so that a token's result does not depend,
    // not even in its last bit, on how many tokens share the step)
    if (T >= 256 && pow2 && aligned && (rot == hd || !inv_freq) && dtype == VL_BF16)
        return vl_launch(qk_norm_rope_write_wide_kernel<bf16>, dim3(T), dim3(ROPE_THREADS), 0, s, (bf16*)qkv, positions,
                         slots, qw, kw, eps, inv_freq, (bf16*)kcache, (bf16*)vcache, nq, nkv, hd, page_size,
                         num_slots, row_stride, err);
    const int heads_per_block = T >= 256 ? nheads : ROPE_THREADS / 32;
    dim3 grid(T, (nheads + heads_per_block - 1) / heads_per_block);
#define ROPE_LAUNCH(TYPE, MAXHD)                                                                           \
    return vl_launch(qk_norm_rope_write_kernel<TYPE, MAXHD>, grid, dim3(ROPE_THREADS), 0, s,               \
        (TYPE*)qkv, positions, slots, qw, kw, eps, inv_freq, rot, (TYPE*)kcache, (TYPE*)vcache,            \
        nq, nkv, hd, page_size, num_slots, row_stride, err, heads_per_block)
    if (dtype == VL_F32) {
        if (hd <= 128) ROPE_LAUNCH(float, 128);
        ROPE_LAUNCH(float, ROPE_MAX_HD);
    }
    if (dtype == VL_BF16) {
        if (hd <= 128) ROPE_LAUNCH(bf16, 128);
        ROPE_LAUNCH(bf16, ROPE_MAX_HD);
    }
#undef ROPE_LAUNCH
    return VL_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------------------
// The same step for a mixer that norms q and k over the WHOLE projection and whose values are its keys:
//   in [T, ld] float32 = q (nq * hd) | k (nkv * hd), e.g. as a short convolution left them;
//   v <- k as it came;   q <- q / sqrt(mean over all nq * hd values of q^2 + eps) * qw, k likewise with kw
//   (qw, kw of nq * hd and nkv * hd entries), then the rotation of the first `rot` features of every head
//   (pairs (i, i + rot/2)), q to q_out [T, nq * hdp], k and v to the token's cache slot (heads of hdp features).
// hdp >= hd is the head size the attention kernels see; features hd .. hdp - 1 are written as zeros.
// One block per token; sums of squares, angles, sine and cosine in float32.  A token at a negative position
// (a padded row of a replayed step) gets zeros for q and writes no cache.
// With CONV the block makes its row itself, in shared memory, from the product `proj` [T, pld] (q | k columns first):
//   row[c] = sum_j w[c, j] (proj[t - (taps-1) + j, c] + in_bias[c]),   rows before the portion's first token from the
//   request's state [(taps-1), C] (zeros in a fresh slot), in the order of sums of vl_short_conv (the same bits).
// `own_state` (every request of the step brings one token): the block also shifts the token's row into the state;
// else the caller runs vl_short_conv's state pass after this launch.
// ---------------------------------------------------------------------------------------------------------
struct ConvSource {
    const void* proj; int pld;                           // the product, its row length
    const float* w; const float* in_bias; int taps;      // [C, taps], [C] or null
    float* state; long long state_stride;                // a row per state slot
    const int* cu; const int* state_slots; const int* req_index;
    int own_state;
};
// NT threads a block, chosen by the row's length alone (rows_threads), so that the order of the sums of squares is a
// matter of the model's sizes, not of the step.
static inline int rows_threads(long long C) { return C > 2048 ? 512 : (C > 512 ? 256 : 128); }
#define ROWS_UNROLL 4
template <typename T, typename TP, bool CONV, int NT>
__global__ void __launch_bounds__(NT)
rows_norm_rope_write_kernel(const float* __restrict__ in, int ld, ConvSource cs, const int* __restrict__ positions,
                            const int* __restrict__ slots, const float* __restrict__ qw, const float* __restrict__ kw,
                            float eps, const float* __restrict__ inv_freq, int rot, T* __restrict__ q_out,
                            T* __restrict__ kcache, T* __restrict__ vcache, int nq, int nkv, int hd, int hdp, int page_size,
                            long long num_slots, unsigned* err) {
    __shared__ float s_cos[ROPE_MAX_HD / 2], s_sin[ROPE_MAX_HD / 2];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int p = positions[t];
    const int half = inv_freq ? rot / 2 : 0;
    const int Cq = nq * hd, Ck = nkv * hd;
    if (inv_freq) {
        const float pos = (float)p;
        for (int i = threadIdx.x; i < half; i += NT) sincosf(pos * inv_freq[i], &s_sin[i], &s_cos[i]);
    }
    pdl_wait();
    T* qo = q_out + (size_t)t * nq * hdp;
    if (p < 0) {
        for (int e = threadIdx.x; e < nq * hdp; e += NT) qo[e] = from_f32<T>(0.f);
        return;
    }
    const float* row = in + (size_t)t * ld;
    if constexpr (CONV) {
        extern __shared__ float s_row[];
        const TP* proj = (const TP*)cs.proj;
        const int b = cs.req_index[t], s0 = cs.cu[b], i = t - s0, C = Cq + Ck, back = cs.taps - 1;
        float* st = cs.state + (long long)cs.state_slots[b] * cs.state_stride;
        // ROWS_UNROLL channels a thread at a time, their loads in flight together; a channel's sum runs over the taps in order
        for (int c0 = threadIdx.x; c0 < C; c0 += NT * ROWS_UNROLL) {
            float acc[ROWS_UNROLL], ib[ROWS_UNROLL];
#pragma unroll
            for (int u = 0; u < ROWS_UNROLL; ++u) {
                const int c = c0 + u * NT;
                acc[u] = 0.f;
                ib[u] = (cs.in_bias && c < C) ? cs.in_bias[c] : 0.f;
            }
            for (int j = 0; j < cs.taps; ++j) {
                const int at = i - back + j;
#pragma unroll
                for (int u = 0; u < ROWS_UNROLL; ++u) {
                    const int c = c0 + u * NT;
                    if (c < C) {
                        const float v = at >= 0 ? to_f32(proj[(size_t)(s0 + at) * cs.pld + c]) + ib[u] : st[(size_t)(at + back) * C + c];
                        acc[u] += cs.w[(size_t)c * cs.taps + j] * v;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < ROWS_UNROLL; ++u)
                if (c0 + u * NT < C) s_row[c0 + u * NT] = acc[u];
            if (cs.own_state && back > 0) {                  // one token: rows 1.. move up, the token's row comes last
                for (int j = 0; j + 1 < back; ++j) {
                    float up[ROWS_UNROLL];
#pragma unroll
                    for (int u = 0; u < ROWS_UNROLL; ++u)
                        if (c0 + u * NT < C) up[u] = st[(size_t)(j + 1) * C + c0 + u * NT];
#pragma unroll
                    for (int u = 0; u < ROWS_UNROLL; ++u)
                        if (c0 + u * NT < C) st[(size_t)j * C + c0 + u * NT] = up[u];
                }
#pragma unroll
                for (int u = 0; u < ROWS_UNROLL; ++u)
                    if (c0 + u * NT < C)
                        st[(size_t)(back - 1) * C + c0 + u * NT] = to_f32(proj[(size_t)t * cs.pld + c0 + u * NT]) + ib[u];
            }
        }
        __syncthreads();
        row = s_row;
    }
    float ssq = 0.f, ssk = 0.f;
    for (int e = threadIdx.x; e < Cq; e += NT) { const float v = row[e]; ssq += v * v; }
    for (int e = threadIdx.x; e < Ck; e += NT) { const float v = row[Cq + e]; ssk += v * v; }
    ssq = block_sum<NT>(ssq, scratch);
    ssk = block_sum<NT>(ssk, scratch);          // (block_sum's own barriers order the table above, too)
    const float invq = 1.0f / sqrtf(ssq / (float)Cq + eps), invk = 1.0f / sqrtf(ssk / (float)Ck + eps);
    for (int o = threadIdx.x; o < nq * hdp; o += NT) {
        const int h = o / hdp, d = o - h * hdp, e = h * hd + d;
        float v = 0.f;
        if (d < hd) {
            v = row[e] * invq * qw[e];
            if (d < 2 * half) {
                const bool first = d < half;
                const int pe = first ? e + half : e - half, i = first ? d : d - half;
                const float other = row[pe] * invq * qw[pe];
                v = first ? v * s_cos[i] - other * s_sin[i] : v * s_cos[i] + other * s_sin[i];
            }
        }
        qo[o] = from_f32<T>(v);
    }
    if (!slots) return;
    const int slot = slots[t];
    if (slot < 0) return;
    if (slot >= num_slots) {
        if (threadIdx.x == 0) atomicOr(err, VL_DEV_BAD_SLOT);
        return;
    }
    const int page = slot / page_size, off = slot - page * page_size;
    const float* krow = row + Cq;
    for (int o = threadIdx.x; o < nkv * hdp; o += NT) {
        const int kvh = o / hdp, d = o - kvh * hdp, e = kvh * hd + d;
        float v = 0.f, raw = 0.f;
        if (d < hd) {
            raw = krow[e];
            v = raw * invk * kw[e];
            if (d < 2 * half) {
                const bool first = d < half;
                const int pe = first ? e + half : e - half, i = first ? d : d - half;
                const float other = krow[pe] * invk * kw[pe];
                v = first ? v * s_cos[i] - other * s_sin[i] : v * s_cos[i] + other * s_sin[i];
            }
        }
        const size_t at = (((size_t)page * nkv + kvh) * page_size + off) * hdp + d;
        kcache[at] = from_f32<T>(v);
        vcache[at] = from_f32<T>(raw);
    }
}

extern "C" int vl_rows_norm_rope_write(const float* in, int ld, const int* positions, const int* slots, const float* qw,
                                       const float* kw, float eps, const float* inv_freq, int rot, void* q_out, int dtype,
                                       void* kcache, void* vcache, int T, int nq, int nkv, int hd, int hdp, int page_size,
                                       long long num_slots, unsigned* err, void* stream) {
    if (T <= 0) return VL_OK;
    if (hd <= 0 || hdp < hd || nq <= 0 || nkv <= 0 || rot < 0 || rot > hd || (rot & 1) || rot > ROPE_MAX_HD) return VL_ERR_UNSUPPORTED;
    if (page_size <= 0 || ld < (nq + nkv) * hd || !qw || !kw) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const ConvSource none = {};
    const int nt = rows_threads((long long)(nq + nkv) * hd);
#define ROWS_LAUNCH(TT, NTH)                                                                                            \
    return vl_launch(rows_norm_rope_write_kernel<TT, float, false, NTH>, dim3(T), dim3(NTH), 0, s, in, ld, none, positions, slots, \
                     qw, kw, eps, inv_freq, rot, (TT*)q_out, (TT*)kcache, (TT*)vcache, nq, nkv, hd, hdp, page_size, num_slots, err)
    if (dtype == VL_F32) {
        if (nt == 512) ROWS_LAUNCH(float, 512);
        if (nt == 256) ROWS_LAUNCH(float, 256);
        ROWS_LAUNCH(float, 128);
    }
    if (dtype == VL_BF16) {
        if (nt == 512) ROWS_LAUNCH(bf16, 512);
        if (nt == 256) ROWS_LAUNCH(bf16, 256);
        ROWS_LAUNCH(bf16, 128);
    }
#undef ROWS_LAUNCH
    return VL_ERR_UNSUPPORTED;
}

// Most floats of a row that the fused form keeps in shared memory.
#define CONV_ROW_MAX (200 * 1024 / 4)
extern "C" int vl_conv_rows_max() { return CONV_ROW_MAX; }

template <typename T, typename TP, int NT>
static int launch_conv_rows(int T_, size_t smem, cudaStream_t s, const ConvSource& cs, const int* positions, const int* slots,
                            const float* qw, const float* kw, float eps, const float* inv_freq, int rot, void* q_out, void* kcache,
                            void* vcache, int nq, int nkv, int hd, int hdp, int page_size, long long num_slots, unsigned* err) {
    auto kernel = rows_norm_rope_write_kernel<T, TP, true, NT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return vl_launch(kernel, dim3(T_), dim3(NT), smem, s, (const float*)nullptr, 0, cs, positions, slots, qw, kw, eps,
                     inv_freq, rot, (T*)q_out, (T*)kcache, (T*)vcache, nq, nkv, hd, hdp, page_size, num_slots, err);
}

// The convolution of vl_short_conv and vl_rows_norm_rope_write in one launch (see the kernel's comment); the activation
// dtype of proj and of the outputs is `dtype`.  `own_state` != 0 only when every request brings exactly one token.
extern "C" int vl_conv_rows_norm_rope_write(const void* proj, int pld, const float* w, const float* in_bias, int taps, float* state,
                                            long long state_stride, const int* cu, const int* state_slots, const int* req_index,
                                            int own_state, const int* positions, const int* slots, const float* qw, const float* kw,
                                            float eps, const float* inv_freq, int rot, void* q_out, int dtype, void* kcache,
                                            void* vcache, int T, int nq, int nkv, int hd, int hdp, int page_size, long long num_slots,
                                            unsigned* err, void* stream) {
    if (T <= 0) return VL_OK;
    if (hd <= 0 || hdp < hd || nq <= 0 || nkv <= 0 || rot < 0 || rot > hd || (rot & 1) || rot > ROPE_MAX_HD) return VL_ERR_UNSUPPORTED;
    const long long C = (long long)(nq + nkv) * hd;
    if (C > CONV_ROW_MAX) return VL_ERR_UNSUPPORTED;
    if (page_size <= 0 || pld < C || taps <= 0 || !w || !qw || !kw || !proj || !state || !cu || !state_slots || !req_index ||
        state_stride < (long long)(taps - 1) * C) return VL_ERR_ARGUMENT;
    const ConvSource cs = {proj, pld, w, in_bias, taps, state, state_stride, cu, state_slots, req_index, own_state};
    const size_t smem = (size_t)C * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    const int nt = rows_threads(C);
#define CONV_ROWS_LAUNCH(TT, NTH)                                                                                       \
    return launch_conv_rows<TT, TT, NTH>(T, smem, s, cs, positions, slots, qw, kw, eps, inv_freq, rot, q_out, kcache, vcache, \
                                         nq, nkv, hd, hdp, page_size, num_slots, err)
    if (dtype == VL_F32) {
        if (nt == 512) CONV_ROWS_LAUNCH(float, 512);
        if (nt == 256) CONV_ROWS_LAUNCH(float, 256);
        CONV_ROWS_LAUNCH(float, 128);
    }
    if (dtype == VL_BF16) {
        if (nt == 512) CONV_ROWS_LAUNCH(bf16, 512);
        if (nt == 256) CONV_ROWS_LAUNCH(bf16, 256);
        CONV_ROWS_LAUNCH(bf16, 128);
    }
#undef CONV_ROWS_LAUNCH
    return VL_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------------------
// Head work of an attention without rotation: every head of q and k divided by its root mean square
// (a weight per feature, or none), the query then multiplied by a factor that grows with its position,
//     q <- q (1 + temp_coef ln(floor((pos + 1) / temp_every) + 1))          (temp_every <= 0: no factor),
// every value head divided by its own root mean square when `v_norm` (no weight), k and v written to the token's
// cache slot.  Heads lie in rows as [q (nq) | k (nkv) | v (nkv)], each `hd` features wide; the means run over
// the first `qk_dim` / `v_dim` features (what lies behind them in a padded head is zero and stays zero).
// A warp per (token, head), the head in registers; sums and factors in float32.  hd up to ROPE_MAX_HD.
// VEC = 4: a lane holds groups of four neighbouring features (8- or 16-byte accesses), when heads and rows start on such
// boundaries; the sum of squares then runs over the same values in another order of lanes, which changes no kernel of a
// model: the launcher's choice depends on sizes and addresses alone.
// ---------------------------------------------------------------------------------------------------------
#define HEADNORM_PER_LANE (ROPE_MAX_HD / 32)
template <typename T, int VEC>
__global__ void __launch_bounds__(ROPE_THREADS)
head_norm_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ slots,
                       const float* __restrict__ qw, const float* __restrict__ kw, float eps, int qk_dim, int v_norm,
                       int v_dim, float v_eps, float temp_coef, int temp_every, T* __restrict__ kcache, T* __restrict__ vcache,
                       int nq, int nkv, int hd, int page_size, long long num_slots, int row_stride, unsigned* err) {
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * (ROPE_THREADS / 32) + warp;
    if (head >= nq + 2 * nkv) return;
    const int pos = positions[t];
    const int slot = slots ? slots[t] : -1;
    pdl_wait();
    const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
    T* src = qkv + (size_t)t * row_stride + (size_t)head * hd;
    T* dst = src;
    if (!is_q) {
        if (slot < 0) return;
        if ((long long)slot >= num_slots) {
            if (lane == 0 && head == nq) atomicOr(err, VL_DEV_BAD_SLOT);
            return;
        }
        const int page = slot / page_size, off = slot - page * page_size;
        const int kvh = is_k ? head - nq : head - nq - nkv;
        dst = (is_k ? kcache : vcache) + (((size_t)page * nkv + kvh) * page_size + off) * hd;
    }
    float v[HEADNORM_PER_LANE];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < HEADNORM_PER_LANE; k += VEC) {
        const int i = VEC * lane + 32 * k;                            // VEC = 1: lane + 32 k
        if (VEC == 4) {
            const float4 q = i < hd ? Quad<T>::load(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            v[k] = q.x; v[k + 1] = q.y; v[k + 2] = q.z; v[k + 3] = q.w;
            ss += q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
        } else {
            v[k] = i < hd ? to_f32(src[i]) : 0.f;
            ss += v[k] * v[k];
        }
    }
    float f = 1.f;
    const bool normed = is_q || is_k ? qk_dim > 0 : v_norm != 0;
    if (normed) {                                                     // (warp-uniform)
        ss = warp_sum(ss);
        f = 1.0f / sqrtf(ss / (float)(is_q || is_k ? qk_dim : v_dim) + (is_q || is_k ? eps : v_eps));
    }
    if (is_q && temp_every > 0 && pos >= 0) f *= 1.0f + temp_coef * logf((float)((pos + 1) / temp_every + 1));
    const float* w = is_q ? qw : (is_k ? kw : nullptr);
#pragma unroll
    for (int k = 0; k < HEADNORM_PER_LANE; k += VEC) {
        const int i = VEC * lane + 32 * k;
        if (i >= hd) continue;
        if (VEC == 4) {
            float4 q = make_float4(v[k] * f, v[k + 1] * f, v[k + 2] * f, v[k + 3] * f);
            if (w) { q.x *= w[i]; q.y *= w[i + 1]; q.z *= w[i + 2]; q.w *= w[i + 3]; }
            Quad<T>::store(dst + i, q);
        } else {
            dst[i] = from_f32<T>(w ? v[k] * f * w[i] : v[k] * f);
        }
    }
}

extern "C" int vl_head_norm_write(void* qkv, int dtype, const int* positions, const int* slots, const float* qw, const float* kw,
                                  float eps, int qk_dim, int v_norm, int v_dim, float v_eps, float temp_coef, int temp_every, void* kcache,
                                  void* vcache, int T, int nq, int nkv, int hd, int page_size, long long num_slots,
                                  int row_stride, unsigned* err, void* stream) {
    if (T <= 0) return VL_OK;
    if (nq <= 0 || nkv <= 0 || hd <= 0 || hd > ROPE_MAX_HD) return VL_ERR_UNSUPPORTED;
    if (qk_dim < 0 || qk_dim > hd || v_dim <= 0 || v_dim > hd || row_stride < (nq + 2 * nkv) * hd || page_size <= 0)
        return VL_ERR_ARGUMENT;
    const int nheads = nq + 2 * nkv, per = ROPE_THREADS / 32;
    dim3 grid(T, (nheads + per - 1) / per);
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = hd % 4 == 0 && row_stride % 4 == 0 && (((uintptr_t)qkv | (uintptr_t)kcache | (uintptr_t)vcache) & 15) == 0;
#define HNW_LAUNCH(TYPE, VEC)                                                                                                    \
    return vl_launch(head_norm_write_kernel<TYPE, VEC>, grid, dim3(ROPE_THREADS), 0, s, (TYPE*)qkv, positions, slots, qw, kw, eps, \
                     qk_dim, v_norm, v_dim, v_eps, temp_coef, temp_every, (TYPE*)kcache, (TYPE*)vcache, nq, nkv, hd, page_size,   \
                     num_slots, row_stride, err)
    if (dtype == VL_F32) { if (vec) HNW_LAUNCH(float, 4); HNW_LAUNCH(float, 1); }
    if (dtype == VL_BF16) { if (vec) HNW_LAUNCH(bf16, 4); HNW_LAUNCH(bf16, 1); }
#undef HNW_LAUNCH
    return VL_ERR_UNSUPPORTED;
}
