// Mixers that carry a state of fixed size from token to token: a short causal convolution and three
// linear recurrences, each over the tokens that a step brings for every request, from the state the
// steps before left in the request's slot.  A decoded token is a portion of one token: the same kernels.
//
// A step's tokens lie flat, request b owns rows cu[b] .. cu[b+1]-1 and the state row slots[b]; a request
// without tokens (padding of a replayed step) is skipped.  Everything that enters a recurrence is float32:
// decays and their logarithms, softplus and exponentials, step sizes, gates, unit norms and the state.
//
//   vl_short_conv   out[t, c] = act(bias[c] + sum_j w[c, j] in[t - (taps-1) + j, c]), zeros before a request's
//                   first token; the last taps-1 inputs of every channel are part of the state (`longest`: a bound
//                   on the tokens a request brings, which says how many blocks share a request).  `in_bias`: a
//                   number per channel added to every input row as it is read (the bias of the product that made
//                   the rows, left to this kernel); the state keeps the rows with it
//   vl_token_shift  h[t] = x[t] + (x[t-1] - x[t]) mu, the row before a portion's first token being part of the state
//   vl_ssd_scan     S <- exp(-exp(A_log) dt) S + dt B x^T,  y = S^T C + D x          (S: N x P per head, dt =
//                   softplus(raw + bias); heads share B and C in groups)
//   vl_mlstm_scan   m' = max(f + m, i);  S <- e^(f+m-m') S + e^(i-m') k v^T;  n likewise with k alone;
//                   o = S^T q / (max(|n.q|, e^(-m')) + den_eps);  i = cap tanh(a/cap), f = logsigmoid(cap tanh(b/cap))
//   vl_delta_scan   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q   (g one decay per key
//                   channel, q and k unit vectors per head, q scaled)
//   vl_gate_norm    RMS norm over equal parts of a row with a weight and a gate (silu or sigmoid), the gate
//                   before or after the norm
//
// Layout of the scans: a block owns (head, request, tile of value columns); a column of the state is held in
// registers by L lanes of a warp (row r of the state by lane r mod L, four rows a lane where 32 lanes can hold
// the column), so a token costs each lane a few multiply-adds and one or two butterfly sums over the L lanes,
// and the sixteen warps of a block take turns on an SM while each waits for its sums.  The per-token vectors of a chunk of tokens
// are staged in shared memory by the whole block, one chunk ahead of the walk.  The order of every sum depends
// on the sizes alone, never on how the tokens were cut into steps or on what else the launch holds.
#include "common.cuh"

#define RC_MAX_THREADS 512

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
template <int L>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int o = L >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// How a scan block is shaped for a state of N rows and P columns per head: a column is held by L lanes of a warp with
// `rows` rows each (4 rows while 32 lanes can hold the column, so that many warps share the walk of a token; 8 or 16
// for longer columns), and a block is 128, 256 or 512 threads: the fewest that hold all P columns, else 512.
struct ScanShape { int rows, L, threads, CT, Z; };
static inline bool scan_shape(int N, int P, ScanShape* sh) {
    if (N <= 0 || P <= 0 || N > 512) return false;
    sh->rows = N <= 128 ? 4 : (N <= 256 ? 8 : 16);
    int L = 1;
    while (L * sh->rows < N) L <<= 1;
    sh->L = L;
    sh->threads = (128 / L >= P) ? 128 : ((256 / L >= P) ? 256 : RC_MAX_THREADS);
    sh->CT = sh->threads / L;
    sh->Z = (P + sh->CT - 1) / sh->CT;
    return true;
}
// KERNEL<TP, rows, L> for the shape `sh`
#define SCAN_LAUNCH(KERNEL, TP, sh, grid, smem, s, ...)                                                              \
    do {                                                                                                             \
        const dim3 block_(sh.threads);                                                                               \
        if (sh.rows == 16) return vl_launch(KERNEL<TP, 16, 32>, grid, block_, smem, s, __VA_ARGS__);                 \
        if (sh.rows == 8) return vl_launch(KERNEL<TP, 8, 32>, grid, block_, smem, s, __VA_ARGS__);                   \
        switch (sh.L) {                                                                                              \
            case 32: return vl_launch(KERNEL<TP, 4, 32>, grid, block_, smem, s, __VA_ARGS__);                        \
            case 16: return vl_launch(KERNEL<TP, 4, 16>, grid, block_, smem, s, __VA_ARGS__);                        \
            case 8: return vl_launch(KERNEL<TP, 4, 8>, grid, block_, smem, s, __VA_ARGS__);                          \
            case 4: return vl_launch(KERNEL<TP, 4, 4>, grid, block_, smem, s, __VA_ARGS__);                          \
            case 2: return vl_launch(KERNEL<TP, 4, 2>, grid, block_, smem, s, __VA_ARGS__);                          \
            default: return vl_launch(KERNEL<TP, 4, 1>, grid, block_, smem, s, __VA_ARGS__);                         \
        }                                                                                                            \
    } while (0)

// ------------------------------------------------------------------------------------------ convolution
// A block owns 32 channels and CONV_TOKENS tokens of one request.  mode 0: outputs and the new state by the same block
// (every request brings at most CONV_TOKENS tokens: one block per request and channel tile, so nobody else reads
// the state it rewrites); mode 1: outputs only; mode 2: the new state only (a launch of its own after mode 1, when
// requests are cut among several blocks: the blocks that read the old state must have finished).
#define CONV_TOKENS 64
template <typename TP>
__global__ void __launch_bounds__(256)
short_conv_kernel(const TP* __restrict__ in, int ld, int col0, int C, const float* __restrict__ w,
                  const float* __restrict__ bias, const float* __restrict__ in_bias, int taps, float* __restrict__ state,
                  long long state_stride, const int* __restrict__ cu, const int* __restrict__ slots, float* __restrict__ out,
                  int act, int mode) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const int s0 = cu[b], n = cu[b + 1] - s0;
    const int first = blockIdx.z * CONV_TOKENS;
    if (n <= 0 || first >= n) return;
    const int last = mode == 0 ? n : min(n, first + CONV_TOKENS);
    const int c = blockIdx.x * 32 + threadIdx.x;
    const bool live = c < C;
    float* st = state + (long long)slots[b] * state_stride;          // [(taps-1), C]
    const int back = taps - 1;
    const float ib = (live && in_bias) ? in_bias[c] : 0.f;
    if (live && mode != 2) {
        for (int t = first + threadIdx.y; t < last; t += blockDim.y) {
            float acc = bias ? bias[c] : 0.f;
            for (int j = 0; j < taps; ++j) {
                const int at = t - back + j;
                const float v = at >= 0 ? to_f32(in[(size_t)(s0 + at) * ld + col0 + c]) + ib : st[(size_t)(at + back) * C + c];
                acc += w[(size_t)c * taps + j] * v;
            }
            out[(size_t)(s0 + t) * C + c] = act ? silu_f(acc) : acc;
        }
    }
    if (mode == 1) return;
    __syncthreads();
    if (live && threadIdx.y == 0) {
        for (int j = 0; j < back; ++j) {                              // reads run ahead of the writes
            const int at = n - back + j;
            st[(size_t)j * C + c] = at >= 0 ? to_f32(in[(size_t)(s0 + at) * ld + col0 + c]) + ib : st[(size_t)(at + back) * C + c];
        }
    }
}

extern "C" int vl_short_conv(const void* in, int dtype, int ld, int col0, int C, const float* w, const float* bias,
                             const float* in_bias, int taps, float* state, long long state_stride, const int* cu, const int* slots,
                             int B, int longest, float* out, int act, void* stream) {
    if (B <= 0 || C <= 0) return VL_OK;
    if (taps <= 0 || col0 < 0 || col0 + C > ld || longest <= 0) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int cuts = (longest + CONV_TOKENS - 1) / CONV_TOKENS;
    // without `out` only the new state is made (the caller computed the rows itself, from the old state)
    for (int pass = out ? 0 : 1; pass < (cuts > 1 || !out ? 2 : 1); ++pass) {
        const int mode = (cuts > 1 || !out) ? pass + 1 : 0;
        dim3 grid((C + 31) / 32, B, mode == 1 ? cuts : 1), block(32, 8);
        int rc;
        if (dtype == VL_F32)
            rc = vl_launch(short_conv_kernel<float>, grid, block, 0, s, (const float*)in, ld, col0, C, w, bias, in_bias, taps, state,
                           state_stride, cu, slots, out, act, mode);
        else if (dtype == VL_BF16)
            rc = vl_launch(short_conv_kernel<bf16>, grid, block, 0, s, (const bf16*)in, ld, col0, C, w, bias, in_bias, taps, state,
                           state_stride, cu, slots, out, act, mode);
        else
            return VL_ERR_UNSUPPORTED;
        if (rc) return rc;
    }
    return VL_OK;
}

// ------------------------------------------------------------------------------------------ token shift
// h[t] = x[t] + (x[t - 1] - x[t]) * mu, element by element in float32, with x[t - 1] the row of the request's token
// before (the state's row for the first token of a portion; a fresh slot holds zeros).  The block of a portion's
// first token also leaves the portion's LAST row of x in the state: a thread reads the old value of its elements
// before it writes the new one, and no other block touches that state, so one launch serves portions of any length.
// A row at a negative position (a padded row of a replayed step) passes unchanged and touches no state.
template <typename TO>
__global__ void __launch_bounds__(256)
token_shift_kernel(const float* __restrict__ x, const float* __restrict__ mu, float* state,
                   long long state_stride, const int* __restrict__ cu, const int* __restrict__ slots,
                   const int* __restrict__ req_index, const int* __restrict__ positions, TO* __restrict__ out, int W) {
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int b = req_index[t], pos = positions[t];
    const bool live = pos >= 0;
    const int first = live ? cu[b] : 0, last = live ? cu[b + 1] - 1 : 0;
    pdl_wait();
    const float* xr = x + (size_t)t * W;
    TO* o = out + (size_t)t * W;
    if (!live) {
        for (int i = threadIdx.x; i < W; i += 256) o[i] = from_f32<TO>(xr[i]);
        return;
    }
    const bool head = t == first;                                     // the row before lies in the state
    float* st = state + (long long)slots[b] * state_stride;
    const float* keep = x + (size_t)last * W;
    if ((W & 3) == 0 && ((((size_t)st) | ((size_t)mu)) & 15) == 0) {  // 16-byte accesses where the state's row allows them
        for (int i = 4 * threadIdx.x; i < W; i += 1024) {
            const float4 v = Quad<float>::load(xr + i), m = Quad<float>::load(mu + i);
            float4 p;
            if (head) {                                               // the old state first, then the new one
                p = __ldcg(reinterpret_cast<const float4*>(st + i));
                const float4 k = Quad<float>::load(keep + i);
                __threadfence_block();
                Quad<float>::store(st + i, k);
            } else {
                p = Quad<float>::load(xr - W + i);
            }
            float4 r;
            r.x = v.x + (p.x - v.x) * m.x; r.y = v.y + (p.y - v.y) * m.y;
            r.z = v.z + (p.z - v.z) * m.z; r.w = v.w + (p.w - v.w) * m.w;
            Quad<TO>::store(o + i, r);
        }
        return;
    }
    for (int i = threadIdx.x; i < W; i += 256) {
        const float v = xr[i], p = head ? st[i] : xr[i - W];
        if (head) st[i] = keep[i];
        o[i] = from_f32<TO>(v + (p - v) * mu[i]);
    }
}

extern "C" int vl_token_shift(const float* x, const float* mu, float* state, long long state_stride, const int* cu,
                              const int* slots, const int* req_index, const int* positions, void* out, int dtype, int T, int W,
                              void* stream) {
    if (T <= 0) return VL_OK;
    if (W <= 0 || state_stride < W) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(token_shift_kernel<float>, dim3(T), dim3(256), 0, s, x, mu, state, state_stride, cu, slots, req_index,
                         positions, (float*)out, W);
    if (dtype == VL_BF16)
        return vl_launch(token_shift_kernel<bf16>, dim3(T), dim3(256), 0, s, x, mu, state, state_stride, cu, slots, req_index,
                         positions, (bf16*)out, W);
    return VL_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------------ the scans' frame
// A scan block stages the per-token vectors of a chunk of tokens in shared memory, [chunk][VEC] floats.  The values of
// the NEXT chunk are loaded into registers before the tokens of this chunk are walked and stored to the other buffer
// afterwards, so the loads' latency hides behind the walk (RC_PREFETCH values per thread, which bounds the chunk).
// A request's state lies in the order the block's threads hold it: [head][column tile][row i of a lane][thread], so
// that loading and storing it are contiguous; the layout is the kernels' own business (vl_scan_state_floats).
#define RC_PREFETCH 8

template <typename Raw>
__device__ __forceinline__ void scan_prefetch(float (&pf)[RC_PREFETCH], int first_row, int m, int VEC, Raw raw) {
#pragma unroll
    for (int j = 0; j < RC_PREFETCH; ++j) {
        const int idx = threadIdx.x + j * blockDim.x;
        if (idx < m * VEC) {
            const int k = idx / VEC;
            pf[j] = raw(first_row + k, idx - k * VEC);
        }
    }
}
__device__ __forceinline__ void scan_commit(const float (&pf)[RC_PREFETCH], float* buf, int m, int VEC) {
#pragma unroll
    for (int j = 0; j < RC_PREFETCH; ++j) {
        const int idx = threadIdx.x + j * blockDim.x;
        if (idx < m * VEC) buf[idx] = pf[j];
    }
}
static inline int scan_chunk(int VEC, int threads) {
    int m = RC_PREFETCH * threads / VEC;
    return m < 1 ? 0 : (m > 16 ? 16 : m);
}
template <int ROWS>
__device__ __forceinline__ float* scan_state(float* state, long long stride, int slot, int h) {
    return state + (long long)slot * stride + ((size_t)h * gridDim.z + blockIdx.z) * ROWS * blockDim.x + threadIdx.x;
}
extern "C" long long vl_scan_state_floats(int H, int N, int P) {
    ScanShape sh;
    if (H <= 0 || !scan_shape(N, P, &sh)) return -1;
    return (long long)H * sh.Z * sh.rows * sh.threads;
}

// ------------------------------------------------------------------------------------------ state space
// xbc float32 [T, C]: x (H*P) | B (G*N) | C (G*N), the convolution's output.  raw dt: column dt_col + h of `proj`.
// y float32 [T, H*P].  Staged per token: B [N] | C [N] | x [CT] | dt | decay.
template <typename TP, int ROWS, int L>
__global__ void __launch_bounds__(RC_MAX_THREADS)
ssd_scan_kernel(const float* __restrict__ xbc, int C, const TP* __restrict__ proj, int ld, int dt_col,
                const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dw,
                float* __restrict__ state, long long state_stride, const int* __restrict__ cu,
                const int* __restrict__ slots, float* __restrict__ y, int H, int G, int N, int P, int chunk) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y;
    const int s0 = cu[b], n = cu[b + 1] - s0;
    if (n <= 0) return;
    const int NT = blockDim.x, CT = NT / L, tid = threadIdx.x;
    const int col = tid / L, l = tid % L;
    const int p0 = blockIdx.z * CT, p = p0 + col;
    const bool live = p < P;
    const int g = h / (H / G), inner = H * P;
    const int VEC = 2 * N + CT + 2;
    float* S = scan_state<ROWS>(state, state_stride, slots[b], h);
    float s[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) s[i] = S[(size_t)i * NT];
    const float rate = expf(A_log[h]), skip = Dw[h], bias = dt_bias[h];
    auto raw = [&](int row, int e) -> float {
        const float* src = xbc + (size_t)(s0 + row) * C;
        if (e < 2 * N) return src[inner + (e < N ? (size_t)g * N + e : (size_t)(G + g) * N + (e - N))];
        if (e < 2 * N + CT) return p0 + (e - 2 * N) < P ? src[(size_t)h * P + p0 + (e - 2 * N)] : 0.f;
        return e == 2 * N + CT ? to_f32(proj[(size_t)(s0 + row) * ld + dt_col + h]) : 0.f;
    };
    auto finish = [&](float* buf, int m) {                            // dt = softplus(raw + bias), decay = exp(-rate dt)
        if (tid < m) {
            float* v = buf + (size_t)tid * VEC + 2 * N + CT;
            const float dt = softplus_f(v[0] + bias);
            v[0] = dt;
            v[1] = expf(-rate * dt);
        }
    };
    float pf[RC_PREFETCH];
    int m = min(chunk, n);
    scan_prefetch(pf, 0, m, VEC, raw);
    scan_commit(pf, sm, m, VEC);
    __syncthreads();
    finish(sm, m);
    __syncthreads();
    int cur = 0;
    for (int t0 = 0; t0 < n; t0 += chunk) {
        const int mn = min(chunk, n - t0 - m);                        // tokens of the next chunk
        if (mn > 0) scan_prefetch(pf, t0 + m, mn, VEC, raw);
        const float* buf = sm + (size_t)cur * chunk * VEC;
        for (int k = 0; k < m; ++k) {
            const float* v = buf + (size_t)k * VEC;
            const float xv = v[2 * N + col], dx = v[2 * N + CT] * xv, a = v[2 * N + CT + 1];
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < ROWS; ++i) {
                const int r = l + L * i;
                if (r < N) {
                    s[i] = a * s[i] + v[r] * dx;
                    acc += s[i] * v[N + r];
                }
            }
            acc = group_sum<L>(acc);
            if (live && l == 0) y[(size_t)(s0 + t0 + k) * inner + (size_t)h * P + p] = acc + skip * xv;
        }
        if (mn > 0) {
            float* nxt = sm + (size_t)(cur ^ 1) * chunk * VEC;
            scan_commit(pf, nxt, mn, VEC);
            __syncthreads();
            finish(nxt, mn);
        }
        __syncthreads();
        cur ^= 1;
        m = mn;
    }
#pragma unroll
    for (int i = 0; i < ROWS; ++i) S[(size_t)i * NT] = s[i];
}

extern "C" int vl_ssd_scan(const float* xbc, int C, const void* proj, int dtype, int ld, int dt_col, const float* dt_bias,
                           const float* A_log, const float* Dw, float* state, long long state_stride, const int* cu,
                           const int* slots, int B, float* y, int H, int G, int N, int P, void* stream) {
    if (B <= 0) return VL_OK;
    if (H <= 0 || G <= 0 || H % G || N <= 0 || P <= 0 || C != H * P + 2 * G * N) return VL_ERR_ARGUMENT;
    ScanShape sh;
    if (!scan_shape(N, P, &sh)) return VL_ERR_UNSUPPORTED;
    const int CT = sh.CT, VEC = 2 * N + CT + 2, chunk = scan_chunk(VEC, sh.threads);
    if (!chunk) return VL_ERR_UNSUPPORTED;
    dim3 grid(H, B, sh.Z);
    const size_t smem = sizeof(float) * (size_t)2 * chunk * VEC;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        SCAN_LAUNCH(ssd_scan_kernel, float, sh, grid, smem, s, xbc, C, (const float*)proj, ld, dt_col,
                    dt_bias, A_log, Dw, state, state_stride, cu, slots, y, H, G, N, P, chunk);
    if (dtype == VL_BF16)
        SCAN_LAUNCH(ssd_scan_kernel, bf16, sh, grid, smem, s, xbc, C, (const bf16*)proj, ld, dt_col,
                    dt_bias, A_log, Dw, state, state_stride, cu, slots, y, H, G, N, P, chunk);
    return VL_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------------ matrix memory
// proj [T, ld]: q at q_col (H*D), k at k_col (H*D), v at v_col (H*P), raw gates at i_col, f_col (H each).
// state per slot: S in the scans' layout, then n [H][Z][D], then m [H][Z], Z = the number of column tiles of a head
// (vl_mlstm_state_floats): blocks of one head run at different times, so each keeps its own n and m.  o float32 [T, H*P].
// Staged per token: q [D] (scaled) | k [D] | v [CT] | keep | put | floor  (the raw gates arrive in the first two of these).
template <typename TP, int ROWS, int L>
__global__ void __launch_bounds__(RC_MAX_THREADS)
mlstm_scan_kernel(const TP* __restrict__ proj, int ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                  const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale, float den_eps,
                  float* __restrict__ state, long long state_stride, const int* __restrict__ cu,
                  const int* __restrict__ slots, float* __restrict__ o, int H, int D, int P, int chunk) {
    extern __shared__ float sm[];
    __shared__ float sM;
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y;
    const int s0 = cu[b], n = cu[b + 1] - s0;
    if (n <= 0) return;
    const int NT = blockDim.x, CT = NT / L, tid = threadIdx.x;
    const int col = tid / L, l = tid % L;
    const int p0 = blockIdx.z * CT, p = p0 + col;
    const bool live = p < P;
    const int VEC = 2 * D + CT + 3;
    const int Z = gridDim.z, z = blockIdx.z;
    float* S = scan_state<ROWS>(state, state_stride, slots[b], h);
    float* base = state + (long long)slots[b] * state_stride + (size_t)H * Z * ROWS * NT;
    float* nv = base + ((size_t)h * Z + z) * D;
    float* mv = base + (size_t)H * Z * D + (size_t)h * Z + z;
    float s[ROWS], nr[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
        const int r = l + L * i;
        s[i] = S[(size_t)i * NT];
        nr[i] = r < D ? nv[r] : 0.f;
    }
    if (tid == 0) sM = mv[0];
    const float ib = i_bias[h], fb = f_bias[h];
    auto raw = [&](int row, int e) -> float {
        const TP* src = proj + (size_t)(s0 + row) * ld;
        if (e < D) return to_f32(src[q_col + (size_t)h * D + e]) * q_scale;
        if (e < 2 * D) return to_f32(src[k_col + (size_t)h * D + (e - D)]);
        if (e < 2 * D + CT) return p0 + (e - 2 * D) < P ? to_f32(src[v_col + (size_t)h * P + p0 + (e - 2 * D)]) : 0.f;
        if (e == 2 * D + CT) return to_f32(src[i_col + h]);
        return e == 2 * D + CT + 1 ? to_f32(src[f_col + h]) : 0.f;
    };
    auto finish = [&](float* buf, int m) {       // the gates (every token by itself), the running maximum (a chain), the exponentials
        if (tid < m) {
            float* v = buf + (size_t)tid * VEC + 2 * D + CT;
            const float fa = cap * tanhf((v[1] + fb) / cap);
            v[0] = cap * tanhf((v[0] + ib) / cap);
            v[1] = fminf(fa, 0.f) - log1pf(expf(-fabsf(fa)));                        // log sigmoid
        }
        __syncthreads();
        if (tid == 0) {
            float mx = sM;
            for (int k = 0; k < m; ++k) {
                float* v = buf + (size_t)k * VEC + 2 * D + CT;
                const float ig = v[0], fg = v[1];
                const float nm = fmaxf(fg + mx, ig);
                v[0] = fg + mx - nm;
                v[1] = ig - nm;
                v[2] = -nm;
                mx = nm;
            }
            sM = mx;
        }
        __syncthreads();
        if (tid < 3 * m) {
            float* v = buf + (size_t)(tid / 3) * VEC + 2 * D + CT + tid % 3;
            v[0] = expf(v[0]);
        }
    };
    float pf[RC_PREFETCH];
    int m = min(chunk, n);
    scan_prefetch(pf, 0, m, VEC, raw);
    scan_commit(pf, sm, m, VEC);
    __syncthreads();
    finish(sm, m);
    __syncthreads();
    int cur = 0;
    for (int t0 = 0; t0 < n; t0 += chunk) {
        const int mn = min(chunk, n - t0 - m);
        if (mn > 0) scan_prefetch(pf, t0 + m, mn, VEC, raw);
        const float* buf = sm + (size_t)cur * chunk * VEC;
        for (int k = 0; k < m; ++k) {
            const float* v = buf + (size_t)k * VEC;
            const float keep = v[2 * D + CT], put = v[2 * D + CT + 1], pv = put * v[2 * D + col];
            float acc = 0.f, den = 0.f;
#pragma unroll
            for (int i = 0; i < ROWS; ++i) {
                const int r = l + L * i;
                if (r < D) {
                    const float kv = v[D + r], qv = v[r];
                    s[i] = keep * s[i] + kv * pv;
                    nr[i] = keep * nr[i] + put * kv;
                    acc += s[i] * qv;
                    den += nr[i] * qv;
                }
            }
            acc = group_sum<L>(acc);
            den = group_sum<L>(den);
            if (live && l == 0)
                o[(size_t)(s0 + t0 + k) * H * P + (size_t)h * P + p] = acc / (fmaxf(fabsf(den), v[2 * D + CT + 2]) + den_eps);
        }
        if (mn > 0) {
            float* nxt = sm + (size_t)(cur ^ 1) * chunk * VEC;
            scan_commit(pf, nxt, mn, VEC);
            __syncthreads();
            finish(nxt, mn);
        }
        __syncthreads();
        cur ^= 1;
        m = mn;
    }
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
        const int r = l + L * i;
        S[(size_t)i * NT] = s[i];
        if (col == 0 && r < D) nv[r] = nr[i];
    }
    if (tid == 0) mv[0] = sM;
}

extern "C" long long vl_mlstm_state_floats(int H, int D, int P) {
    ScanShape sh;
    if (H <= 0 || !scan_shape(D, P, &sh)) return -1;
    return (long long)H * sh.Z * sh.rows * sh.threads + (long long)H * sh.Z * D + (long long)H * sh.Z;
}

extern "C" int vl_mlstm_scan(const void* proj, int dtype, int ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                             const float* i_bias, const float* f_bias, float cap, float q_scale, float den_eps, float* state,
                             long long state_stride, const int* cu, const int* slots, int B, float* o, int H, int D, int P,
                             void* stream) {
    if (B <= 0) return VL_OK;
    if (H <= 0 || D <= 0 || P <= 0 || !(cap > 0.f)) return VL_ERR_ARGUMENT;
    ScanShape sh;
    if (!scan_shape(D, P, &sh)) return VL_ERR_UNSUPPORTED;
    const int CT = sh.CT, VEC = 2 * D + CT + 3, chunk = scan_chunk(VEC, sh.threads);
    if (!chunk) return VL_ERR_UNSUPPORTED;
    dim3 grid(H, B, sh.Z);
    const size_t smem = sizeof(float) * (size_t)2 * chunk * VEC;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        SCAN_LAUNCH(mlstm_scan_kernel, float, sh, grid, smem, s, (const float*)proj, ld, q_col, k_col, v_col,
                    i_col, f_col, i_bias, f_bias, cap, q_scale, den_eps, state, state_stride, cu, slots, o, H, D, P, chunk);
    if (dtype == VL_BF16)
        SCAN_LAUNCH(mlstm_scan_kernel, bf16, sh, grid, smem, s, (const bf16*)proj, ld, q_col, k_col, v_col,
                    i_col, f_col, i_bias, f_bias, cap, q_scale, den_eps, state, state_stride, cu, slots, o, H, D, P, chunk);
    return VL_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------------ delta rule
// qkv float32 [T, C]: q (G*D) | k (G*D) | v (H*P), the convolutions' output.  raw decay: columns dcol .. of `decay` (rows dld wide),
// raw beta: column beta_col + h of `proj`.  o float32 [T, H*P].
// Staged per token: q [D] | k [D] | decay [D] | v [CT] | beta; a warp per token then makes q and k unit vectors (q scaled),
// the decays exp(-rate softplus(raw + bias)) and beta a sigmoid.
template <typename TP, int ROWS, int L>
__global__ void __launch_bounds__(RC_MAX_THREADS)
delta_scan_kernel(const float* __restrict__ qkv, int C, const TP* __restrict__ decay, int dld, int dcol,
                  const float* __restrict__ dt_bias,
                  const float* __restrict__ A_log, const TP* __restrict__ proj, int ld, int beta_col, float q_scale,
                  float unit_eps, float* __restrict__ state, long long state_stride, const int* __restrict__ cu,
                  const int* __restrict__ slots, float* __restrict__ o, int H, int G, int D, int P, int chunk) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y;
    const int s0 = cu[b], n = cu[b + 1] - s0;
    if (n <= 0) return;
    const int NT = blockDim.x, CT = NT / L, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int col = tid / L, l = tid % L;
    const int p0 = blockIdx.z * CT, p = p0 + col;
    const bool live = p < P;
    const int g = h / (H / G);
    const int VEC = 3 * D + CT + 1;
    float* S = scan_state<ROWS>(state, state_stride, slots[b], h);
    float s[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) s[i] = S[(size_t)i * NT];
    const float rate = expf(A_log[h]);
    auto raw = [&](int row, int e) -> float {
        const size_t t = (size_t)(s0 + row);
        if (e < 2 * D) return qkv[t * C + (e < D ? (size_t)g * D + e : (size_t)(G + g) * D + (e - D))];
        if (e < 3 * D) return to_f32(decay[t * dld + dcol + (size_t)h * D + (e - 2 * D)]);
        if (e < 3 * D + CT) return p0 + (e - 3 * D) < P ? qkv[t * C + (size_t)2 * G * D + (size_t)h * P + p0 + (e - 3 * D)] : 0.f;
        return to_f32(proj[t * ld + beta_col + h]);
    };
    auto finish = [&](float* buf, int m) {
        for (int k = warp; k < m; k += NT / 32) {
            float* v = buf + (size_t)k * VEC;
            float qq = 0.f, kk = 0.f;
            for (int r = lane; r < D; r += 32) { qq += v[r] * v[r]; kk += v[D + r] * v[D + r]; }
            qq = warp_sum(qq);
            kk = warp_sum(kk);
            const float qn = q_scale / sqrtf(qq + unit_eps), kn = 1.f / sqrtf(kk + unit_eps);
            for (int r = lane; r < D; r += 32) {
                v[r] *= qn;
                v[D + r] *= kn;
                v[2 * D + r] = expf(-rate * softplus_f(v[2 * D + r] + dt_bias[(size_t)h * D + r]));
            }
            if (lane == 0) v[3 * D + CT] = sigmoid_f(v[3 * D + CT]);
        }
    };
    float pf[RC_PREFETCH];
    int m = min(chunk, n);
    scan_prefetch(pf, 0, m, VEC, raw);
    scan_commit(pf, sm, m, VEC);
    __syncthreads();
    finish(sm, m);
    __syncthreads();
    int cur = 0;
    for (int t0 = 0; t0 < n; t0 += chunk) {
        const int mn = min(chunk, n - t0 - m);
        if (mn > 0) scan_prefetch(pf, t0 + m, mn, VEC, raw);
        const float* buf = sm + (size_t)cur * chunk * VEC;
        for (int k = 0; k < m; ++k) {
            const float* v = buf + (size_t)k * VEC;
            float back = 0.f;
#pragma unroll
            for (int i = 0; i < ROWS; ++i) {
                const int r = l + L * i;
                if (r < D) {
                    s[i] *= v[2 * D + r];
                    back += s[i] * v[D + r];
                }
            }
            back = group_sum<L>(back);
            const float u = v[3 * D + CT] * (v[3 * D + col] - back);
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < ROWS; ++i) {
                const int r = l + L * i;
                if (r < D) {
                    s[i] += v[D + r] * u;
                    acc += s[i] * v[r];
                }
            }
            acc = group_sum<L>(acc);
            if (live && l == 0) o[(size_t)(s0 + t0 + k) * H * P + (size_t)h * P + p] = acc;
        }
        if (mn > 0) {
            float* nxt = sm + (size_t)(cur ^ 1) * chunk * VEC;
            scan_commit(pf, nxt, mn, VEC);
            __syncthreads();
            finish(nxt, mn);
        }
        __syncthreads();
        cur ^= 1;
        m = mn;
    }
#pragma unroll
    for (int i = 0; i < ROWS; ++i) S[(size_t)i * NT] = s[i];
}

extern "C" int vl_delta_scan(const float* qkv, int C, const void* decay, int dld, int dcol, const float* dt_bias, const float* A_log,
                             const void* proj, int dtype, int ld, int beta_col, float q_scale, float unit_eps, float* state,
                             long long state_stride, const int* cu, const int* slots, int B, float* o, int H, int G, int D,
                             int P, void* stream) {
    if (B <= 0) return VL_OK;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || P <= 0 || C != 2 * G * D + H * P) return VL_ERR_ARGUMENT;
    ScanShape sh;
    if (!scan_shape(D, P, &sh)) return VL_ERR_UNSUPPORTED;
    const int CT = sh.CT, VEC = 3 * D + CT + 1, chunk = scan_chunk(VEC, sh.threads);
    if (!chunk) return VL_ERR_UNSUPPORTED;
    dim3 grid(H, B, sh.Z);
    const size_t smem = sizeof(float) * (size_t)2 * chunk * VEC;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        SCAN_LAUNCH(delta_scan_kernel, float, sh, grid, smem, s, qkv, C, (const float*)decay, dld, dcol, dt_bias, A_log,
                    (const float*)proj, ld, beta_col, q_scale, unit_eps, state, state_stride, cu, slots, o, H, G, D, P, chunk);
    if (dtype == VL_BF16)
        SCAN_LAUNCH(delta_scan_kernel, bf16, sh, grid, smem, s, qkv, C, (const bf16*)decay, dld, dcol, dt_bias, A_log,
                    (const bf16*)proj, ld, beta_col, q_scale, unit_eps, state, state_stride, cu, slots, o, H, G, D, P, chunk);
    return VL_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------------ gate and norm
// y float32 [T, W] in parts of `part` columns; a warp per (token, part).  gate (TP, column gate_col of rows `ld` wide):
// kind 1 silu, 2 sigmoid, 0 none.  gate_first: out = rms(y * gate) * w, else out = rms(y) * w * gate.
// w float32 [wlen], indexed by column modulo wlen (wlen = W: one weight per column; wlen = part: shared by the parts).
#define RC_GATE_SILU 1
#define RC_GATE_SIGMOID 2
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
}
__device__ __forceinline__ void load4(const bf16* p, float (&v)[4]) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
    v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<unsigned*>(&a), *reinterpret_cast<unsigned*>(&b));
}

// VEC = 4: a lane takes four neighbouring columns at a time (16-byte reads of y, 8- or 16-byte accesses of gate and out);
// the launcher picks it when every row and part starts on such a boundary.
template <typename TP, int VEC>
__global__ void __launch_bounds__(128)
gate_norm_kernel(const float* __restrict__ y, const TP* __restrict__ gate, int ld, int gate_col, int gate_kind, int gate_first,
                 const float* __restrict__ w, int wlen, float eps, TP* __restrict__ out, int W, int part, size_t groups) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t gi = (size_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (gi >= groups) return;
    const int lane = threadIdx.x & 31;
    const int per_row = W / part;
    const size_t t = gi / per_row;
    const int c0 = (int)(gi - t * per_row) * part;
    const float* row = y + t * W + c0;
    const TP* grow = gate ? gate + t * ld + gate_col + c0 : nullptr;
    float ss = 0.f;
    for (int c = lane * VEC; c < part; c += 32 * VEC) {
        float v[VEC], g[VEC];
        if (VEC == 4) load4(row + c, reinterpret_cast<float (&)[4]>(v)); else v[0] = row[c];
        if (gate_first && grow) {
            if (VEC == 4) load4(grow + c, reinterpret_cast<float (&)[4]>(g)); else g[0] = to_f32(grow[c]);
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] *= gate_kind == RC_GATE_SILU ? silu_f(g[e]) : sigmoid_f(g[e]);
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) ss += v[e] * v[e];
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / part + eps);
    for (int c = lane * VEC; c < part; c += 32 * VEC) {
        float v[VEC], g[VEC];
        if (VEC == 4) load4(row + c, reinterpret_cast<float (&)[4]>(v)); else v[0] = row[c];
#pragma unroll
        for (int e = 0; e < VEC; ++e) g[e] = 1.f;
        if (grow) {
            if (VEC == 4) load4(grow + c, reinterpret_cast<float (&)[4]>(g)); else g[0] = to_f32(grow[c]);
#pragma unroll
            for (int e = 0; e < VEC; ++e) g[e] = gate_kind == RC_GATE_SILU ? silu_f(g[e]) : sigmoid_f(g[e]);
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const float wv = w[(c0 + c + e) % wlen];
            v[e] = gate_first ? v[e] * g[e] * inv * wv : v[e] * inv * wv * g[e];
        }
        if (VEC == 4) store4(out + t * W + c0 + c, reinterpret_cast<const float (&)[4]>(v));
        else out[t * W + c0 + c] = from_f32<TP>(v[0]);
    }
}

extern "C" int vl_gate_norm(const float* y, const void* gate, int dtype, int ld, int gate_col, int gate_kind, int gate_first,
                            const float* w, int wlen, float eps, void* out, int T, int W, int part, void* stream) {
    if (T <= 0 || W <= 0) return VL_OK;
    if (part <= 0 || W % part || wlen <= 0 || (gate && (gate_kind < 1 || gate_kind > 2))) return VL_ERR_ARGUMENT;
    const size_t groups = (size_t)T * (W / part);
    const unsigned blocks = (unsigned)((groups + 3) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = part % 4 == 0 && W % 4 == 0 && ld % 4 == 0 && gate_col % 4 == 0 &&
                     (((uintptr_t)y | (uintptr_t)gate | (uintptr_t)out) & 15) == 0;
    if (dtype == VL_F32) {
        if (vec) return vl_launch(gate_norm_kernel<float, 4>, dim3(blocks), dim3(128), 0, s, y, (const float*)gate, ld, gate_col,
                                  gate_kind, gate_first, w, wlen, eps, (float*)out, W, part, groups);
        return vl_launch(gate_norm_kernel<float, 1>, dim3(blocks), dim3(128), 0, s, y, (const float*)gate, ld, gate_col, gate_kind,
                         gate_first, w, wlen, eps, (float*)out, W, part, groups);
    }
    if (dtype == VL_BF16) {
        if (vec) return vl_launch(gate_norm_kernel<bf16, 4>, dim3(blocks), dim3(128), 0, s, y, (const bf16*)gate, ld, gate_col,
                                  gate_kind, gate_first, w, wlen, eps, (bf16*)out, W, part, groups);
        return vl_launch(gate_norm_kernel<bf16, 1>, dim3(blocks), dim3(128), 0, s, y, (const bf16*)gate, ld, gate_col, gate_kind,
                         gate_first, w, wlen, eps, (bf16*)out, W, part, groups);
    }
    return VL_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------------ several token shifts at once
// out[s][t] = h[t] + (h[t - 1] - h[t]) * mu[s], s < S: S mixes of a row with the row of the token before, each with its own
// mu [W] (float32 arithmetic; h and out in the activation dtype, out [S, T, W]).  The row before a portion's first token
// is the state's row (float32; zeros in a fresh slot), which the blocks of that token replace by the portion's last row,
// as in vl_token_shift (a thread reads its elements of the old state before it writes the new ones, and no other thread
// touches those elements).  A row at a negative position passes unchanged into every mix and touches no state.
// A thread takes VEC neighbouring elements (4 where every row starts on a 16-byte boundary), a block 256 * VEC of a token.
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
token_shift_multi_kernel(const T* __restrict__ h, const float* __restrict__ mu, int S, float* state, long long state_stride,
                         const int* __restrict__ cu, const int* __restrict__ slots, const int* __restrict__ req_index,
                         const int* __restrict__ positions, T* __restrict__ out, int ntok, int W) {
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int b = req_index[t], pos = positions[t];
    const bool live = pos >= 0;
    const int first = live ? cu[b] : 0, last = live ? cu[b + 1] - 1 : 0;
    const int i = (blockIdx.y * 256 + threadIdx.x) * VEC;
    pdl_wait();
    if (i >= W) return;
    const T* xr = h + (size_t)t * W;
    const bool head = live && t == first;
    float v[VEC], p[VEC];
    if (VEC == 4) {
        const float4 a = Quad<T>::load(xr + i);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    } else {
        v[0] = to_f32(xr[i]);
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) p[e] = v[e];
    if (head) {
        float* st = state + (long long)slots[b] * state_stride + i;
        const T* keep = h + (size_t)last * W + i;
        if (VEC == 4) {
            const float4 o = *reinterpret_cast<const float4*>(st), k = Quad<T>::load(keep);
            p[0] = o.x; p[1] = o.y; p[2] = o.z; p[3] = o.w;
            *reinterpret_cast<float4*>(st) = k;
        } else {
            p[0] = st[0];
            st[0] = to_f32(keep[0]);
        }
    } else if (live) {
        if (VEC == 4) {
            const float4 a = Quad<T>::load(xr - W + i);
            p[0] = a.x; p[1] = a.y; p[2] = a.z; p[3] = a.w;
        } else {
            p[0] = to_f32(xr[i - W]);
        }
    }
    for (int s = 0; s < S; ++s) {
        T* o = out + ((size_t)s * ntok + t) * W + i;
        if (VEC == 4) {
            const float4 m = *reinterpret_cast<const float4*>(mu + (size_t)s * W + i);
            Quad<T>::store(o, make_float4(v[0] + (p[0] - v[0]) * m.x, v[1] + (p[1] - v[1]) * m.y, v[2] + (p[2] - v[2]) * m.z,
                                          v[3] + (p[3] - v[3]) * m.w));
        } else {
            o[0] = from_f32<T>(v[0] + (p[0] - v[0]) * mu[(size_t)s * W + i]);
        }
    }
}

extern "C" int vl_token_shift_multi(const void* h, const float* mu, int S, float* state, long long state_stride, const int* cu,
                                    const int* slots, const int* req_index, const int* positions, void* out, int dtype, int T,
                                    int W, void* stream) {
    if (T <= 0) return VL_OK;
    if (W <= 0 || S <= 0 || state_stride < W) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = W % 4 == 0 && state_stride % 4 == 0 &&
                     (((uintptr_t)h | (uintptr_t)mu | (uintptr_t)state | (uintptr_t)out) & 15) == 0;
    const int per = 256 * (vec ? 4 : 1);
    const dim3 grid(T, (W + per - 1) / per);
#define TSM_LAUNCH(TYPE, VEC)                                                                                                \
    return vl_launch(token_shift_multi_kernel<TYPE, VEC>, grid, dim3(256), 0, s, (const TYPE*)h, mu, S, state, state_stride, \
                     cu, slots, req_index, positions, (TYPE*)out, T, W)
    if (dtype == VL_F32) { if (vec) TSM_LAUNCH(float, 4); TSM_LAUNCH(float, 1); }
    if (dtype == VL_BF16) { if (vec) TSM_LAUNCH(bf16, 4); TSM_LAUNCH(bf16, 1); }
#undef TSM_LAUNCH
    return VL_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------------ memory with a decay per key channel
// Per head, S [D x P] from the request's state:   o_t = (S + diag(u) k_t v_t^T)^T r_t;   S <- diag(w_t) S + k_t v_t^T
// with w_t = exp(-exp(z_t + w0)) per key channel and u [H*D] a bonus for the current token alone.
//
// vl_decay_from_raw turns the raw decays z [T, ld] (columns zc .. zc + H*D) into w in place, one thread an element: the two
// exponentials are taken once per token, outside the walk.
// vl_decay_scan walks the tokens.  r, k, w float32 rows with H*D columns from `rc`, `kc`, `wc` on; v with H*P columns;
// o float32 [T, H*P].  A block of DS_THREADS threads owns (head, request, tile of DS_THREADS / L value columns); a column of
// the state lies in the registers of L lanes, lane l holding the ROWS neighbouring rows from ROWS * l on, so that a lane
// fetches its share of r, k and w of a token with one 16-byte read each (ROWS = 4; 8 and 16 rows: two and four reads).  The
// vectors of a chunk of tokens are staged in shared memory one chunk ahead, as in the other scans; the walk is unrolled so
// that the butterfly sums of neighbouring tokens overlap (only `S <- w S + k v` chains from token to token).  Blocks are
// small (128 threads) so that one request's heads and column tiles spread over every SM.  The state's layout is the
// kernel's own: [head][column tile][row i of a lane][thread] (vl_decay_state_floats).
#define DS_THREADS 128
#define DS_PREFETCH 16
#define DS_PIECES 4          // most 16-byte pieces of a token that one thread copies: 3 D / 4 + a few, over 128 threads (D <= 160)
struct DecayShape { int rows, L, CT, Z; };
static inline bool decay_shape(int D, int P, DecayShape* sh) {
    if (D <= 0 || P <= 0 || D > 512) return false;
    sh->rows = D <= 128 ? 4 : (D <= 256 ? 8 : 16);
    int L = 1;
    while (L * sh->rows < D) L <<= 1;
    sh->L = L;
    sh->CT = DS_THREADS / L;
    sh->Z = (P + sh->CT - 1) / sh->CT;
    return true;
}
extern "C" long long vl_decay_state_floats(int H, int D, int P) {
    DecayShape sh;
    if (H <= 0 || !decay_shape(D, P, &sh)) return -1;
    return (long long)H * sh.Z * sh.rows * DS_THREADS;
}

template <typename TP, int VEC>
__global__ void decay_from_raw_kernel(TP* __restrict__ z, int ld, int zc, const float* __restrict__ w0, int HD, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = ((size_t)blockIdx.x * 256 + threadIdx.x) * VEC;
    if (idx >= total) return;
    const size_t t = idx / HD;
    const int c = (int)(idx - t * HD);
    TP* p = z + t * ld + zc + c;
    if (VEC == 4) {                                            // four neighbouring channels: 16-byte accesses of float32 rows
        const float4 v = Quad<TP>::load(p), b = *reinterpret_cast<const float4*>(w0 + c);
        Quad<TP>::store(p, make_float4(expf(-expf(v.x + b.x)), expf(-expf(v.y + b.y)), expf(-expf(v.z + b.z)), expf(-expf(v.w + b.w))));
    } else {
        *p = from_f32<TP>(expf(-expf(to_f32(*p) + w0[c])));
    }
}

extern "C" int vl_decay_from_raw(void* z, int dtype, int T, int ld, int zc, const float* w0, int HD, void* stream) {
    if (T <= 0) return VL_OK;
    if (HD <= 0 || zc < 0 || zc + HD > ld) return VL_ERR_ARGUMENT;
    const size_t total = (size_t)T * HD;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = HD % 4 == 0 && ld % 4 == 0 && zc % 4 == 0 && (((uintptr_t)z | (uintptr_t)w0) & 15) == 0;
    const unsigned blocks = (unsigned)((total / (vec ? 4 : 1) + 255) / 256);
    if (dtype == VL_F32) {
        if (vec) return vl_launch(decay_from_raw_kernel<float, 4>, dim3(blocks), dim3(256), 0, s, (float*)z, ld, zc, w0, HD, total);
        return vl_launch(decay_from_raw_kernel<float, 1>, dim3(blocks), dim3(256), 0, s, (float*)z, ld, zc, w0, HD, total);
    }
    if (dtype == VL_BF16) {
        if (vec) return vl_launch(decay_from_raw_kernel<bf16, 4>, dim3(blocks), dim3(256), 0, s, (bf16*)z, ld, zc, w0, HD, total);
        return vl_launch(decay_from_raw_kernel<bf16, 1>, dim3(blocks), dim3(256), 0, s, (bf16*)z, ld, zc, w0, HD, total);
    }
    return VL_ERR_UNSUPPORTED;
}

// FAST (float32 rows whose heads start on 16-byte boundaries): the staging is 16-byte cp.async copies, a token's pieces
// spread over the block's threads with no division in sight; else every element through a register (any dtype, any size).
__device__ __forceinline__ void ds_cp_async16(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void ds_cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <typename TP, int ROWS, int L, bool FAST>
__global__ void __launch_bounds__(DS_THREADS)
decay_scan_kernel(const TP* __restrict__ rp, int ldr, int rc, const TP* __restrict__ kp, int ldk, int kc, const TP* __restrict__ vp,
                  int ldv, int vc, const TP* __restrict__ wp, int ldw, int wc, const float* __restrict__ u,
                  float* __restrict__ state, long long state_stride, const int* __restrict__ cu,
                  const int* __restrict__ slots, float* __restrict__ o, int H, int D, int P, int chunk, int DP) {
    extern __shared__ __align__(16) float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y;
    const int s0 = cu[b], n = cu[b + 1] - s0;
    if (n <= 0) return;
    constexpr int NT = DS_THREADS, CT = NT / L;
    const int tid = threadIdx.x;
    const int col = tid / L, l = tid % L;
    const int p0 = blockIdx.z * CT, p = p0 + col;
    const bool live = p < P;
    const int VEC = 3 * DP + CT;                         // DP: D rounded up to whole lanes (L * ROWS), so that a lane's reads stay inside
    float* S = state + (long long)slots[b] * state_stride + ((size_t)h * gridDim.z + blockIdx.z) * ROWS * NT + tid;
    float s[ROWS], ub[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
        s[i] = S[(size_t)i * NT];
        const int r = ROWS * l + i;
        ub[i] = r < D ? u[(size_t)h * D + r] : 0.f;
    }
    auto raw = [&](int row, int e) -> float {
        const size_t t = (size_t)(s0 + row);
        const int part = e / DP, r = e - part * DP;
        if (part == 0) return r < D ? to_f32(rp[t * ldr + rc + (size_t)h * D + r]) : 0.f;
        if (part == 1) return r < D ? to_f32(kp[t * ldk + kc + (size_t)h * D + r]) : 0.f;
        if (part == 2) return r < D ? to_f32(wp[t * ldw + wc + (size_t)h * D + r]) : 0.f;
        return p0 + (e - 3 * DP) < P ? to_f32(vp[t * ldv + vc + (size_t)h * P + p0 + (e - 3 * DP)]) : 0.f;
    };
    float pf[DS_PREFETCH];
    auto prefetch = [&](int first_row, int m) {
#pragma unroll
        for (int j = 0; j < DS_PREFETCH; ++j) {
            const int idx = tid + j * NT;
            if (idx < m * VEC) {
                const int k = idx / VEC;
                pf[j] = raw(first_row + k, idx - k * VEC);
            }
        }
    };
    auto commit = [&](float* buf, int m) {
#pragma unroll
        for (int j = 0; j < DS_PREFETCH; ++j) {
            const int idx = tid + j * NT;
            if (idx < m * VEC) buf[idx] = pf[j];
        }
    };
    // (FAST) 16-byte pieces of a token: D/4 of r, of k and of w, then the tile's columns of v that exist
    const int q4 = D >> 2, vq = (min(P - p0, CT) + 3) >> 2;
    // which pieces this thread copies for every token (up to DS_PIECES of them): where they start in the request's first
    // row, how far the next row lies, where they land in a staged token; worked out once, so a token costs an add and a copy
    const float* psrc[DS_PIECES];
    int pld[DS_PIECES], pdst[DS_PIECES];
    if constexpr (FAST) {
#pragma unroll
        for (int j = 0; j < DS_PIECES; ++j) {
            const int e = tid + j * NT;
            psrc[j] = nullptr; pld[j] = 0; pdst[j] = 0;
            if (e < q4) {
                psrc[j] = reinterpret_cast<const float*>(rp) + (size_t)s0 * ldr + rc + (size_t)h * D + 4 * e; pld[j] = ldr; pdst[j] = 4 * e;
            } else if (e < 2 * q4) {
                psrc[j] = reinterpret_cast<const float*>(kp) + (size_t)s0 * ldk + kc + (size_t)h * D + 4 * (e - q4); pld[j] = ldk; pdst[j] = DP + 4 * (e - q4);
            } else if (e < 3 * q4) {
                psrc[j] = reinterpret_cast<const float*>(wp) + (size_t)s0 * ldw + wc + (size_t)h * D + 4 * (e - 2 * q4); pld[j] = ldw; pdst[j] = 2 * DP + 4 * (e - 2 * q4);
            } else if (e < 3 * q4 + vq) {
                psrc[j] = reinterpret_cast<const float*>(vp) + (size_t)s0 * ldv + vc + (size_t)h * P + p0 + 4 * (e - 3 * q4); pld[j] = ldv; pdst[j] = 3 * DP + 4 * (e - 3 * q4);
            }
        }
    }
    auto stage = [&](float* buf, int first_row, int m_) {
        if constexpr (FAST) {
#pragma unroll
            for (int j = 0; j < DS_PIECES; ++j) {
                if (psrc[j]) {
                    const float* src = psrc[j] + (size_t)first_row * pld[j];
                    float* dst = buf + pdst[j];
                    for (int k = 0; k < m_; ++k, src += pld[j], dst += VEC) ds_cp_async16(dst, src);
                }
            }
        }
    };
    int m = min(chunk, n);
    if constexpr (FAST) {
        for (int i = tid; i < 2 * chunk * VEC; i += NT) sm[i] = 0.f;      // what no copy touches (rows beyond D, columns beyond P) stays zero
        __syncthreads();
        stage(sm, 0, m);
        ds_cp_async_wait_all();
    } else {
        prefetch(0, m);
        commit(sm, m);
    }
    __syncthreads();
    int cur = 0;
    for (int t0 = 0; t0 < n; t0 += chunk) {
        const int mn = min(chunk, n - t0 - m);
        if (mn > 0) {
            if constexpr (FAST) stage(sm + (size_t)(cur ^ 1) * chunk * VEC, t0 + m, mn);
            else prefetch(t0 + m, mn);
        }
        const float* buf = sm + (size_t)cur * chunk * VEC;
#pragma unroll 4
        for (int k = 0; k < m; ++k) {
            const float* v = buf + (size_t)k * VEC;
            const float vj = v[3 * DP + col];
            float rr[ROWS], kk[ROWS], ww[ROWS];
#pragma unroll
            for (int i = 0; i < ROWS; i += 4) {
                const float4 a = *reinterpret_cast<const float4*>(v + ROWS * l + i);
                const float4 c = *reinterpret_cast<const float4*>(v + DP + ROWS * l + i);
                const float4 d = *reinterpret_cast<const float4*>(v + 2 * DP + ROWS * l + i);
                rr[i] = a.x; rr[i + 1] = a.y; rr[i + 2] = a.z; rr[i + 3] = a.w;
                kk[i] = c.x; kk[i + 1] = c.y; kk[i + 2] = c.z; kk[i + 3] = c.w;
                ww[i] = d.x; ww[i + 1] = d.y; ww[i + 2] = d.z; ww[i + 3] = d.w;
            }
            float acc0 = 0.f, acc1 = 0.f;                       // two chains of additions, joined before the lanes' sums
#pragma unroll
            for (int i = 0; i < ROWS; i += 2) {                 // rows beyond D hold zeros in r, k and w: they add nothing
                const float kv0 = kk[i] * vj, kv1 = kk[i + 1] * vj;
                acc0 += rr[i] * (s[i] + ub[i] * kv0);
                acc1 += rr[i + 1] * (s[i + 1] + ub[i + 1] * kv1);
                s[i] = ww[i] * s[i] + kv0;
                s[i + 1] = ww[i + 1] * s[i + 1] + kv1;
            }
            const float acc = group_sum<L>(acc0 + acc1);
            if (live && l == 0) o[(size_t)(s0 + t0 + k) * H * P + (size_t)h * P + p] = acc;
        }
        if (mn > 0) {
            if constexpr (FAST) ds_cp_async_wait_all();
            else commit(sm + (size_t)(cur ^ 1) * chunk * VEC, mn);
        }
        __syncthreads();
        cur ^= 1;
        m = mn;
    }
#pragma unroll
    for (int i = 0; i < ROWS; ++i) S[(size_t)i * NT] = s[i];
}

extern "C" int vl_decay_scan(const void* rp, int ldr, int rc, const void* kp, int ldk, int kc, const void* vp, int ldv, int vc,
                             const void* wp, int ldw, int wc, int dtype, const float* u, float* state,
                             long long state_stride, const int* cu, const int* slots, int B, float* o, int H, int D, int P,
                             void* stream) {
    if (B <= 0) return VL_OK;
    if (H <= 0 || D <= 0 || P <= 0 || rc < 0 || kc < 0 || vc < 0 || wc < 0 || rc + H * D > ldr || kc + H * D > ldk ||
        vc + H * P > ldv || wc + H * D > ldw)
        return VL_ERR_ARGUMENT;
    DecayShape sh;
    if (!decay_shape(D, P, &sh)) return VL_ERR_UNSUPPORTED;
    const int DP = sh.L * sh.rows, VEC = 3 * DP + sh.CT;
    // float32 rows whose heads and column tiles start on 16-byte boundaries are staged by 16-byte asynchronous copies
    const bool fast = dtype == VL_F32 && D % 4 == 0 && P % 4 == 0 && ldr % 4 == 0 && ldk % 4 == 0 && ldv % 4 == 0 && ldw % 4 == 0 &&
                      rc % 4 == 0 && kc % 4 == 0 && vc % 4 == 0 && wc % 4 == 0 && sh.CT % 4 == 0 &&
                      3 * (D / 4) + sh.CT / 4 <= DS_PIECES * DS_THREADS &&
                      (((uintptr_t)rp | (uintptr_t)kp | (uintptr_t)vp | (uintptr_t)wp) & 15) == 0;
    int chunk = fast ? 16 : DS_PREFETCH * DS_THREADS / VEC;
    chunk = chunk > 16 ? 16 : chunk;
    const int fits = (int)(48 * 1024 / (sizeof(float) * 2 * VEC));      // two buffers within the shared memory every launch may have
    chunk = chunk > fits ? fits : chunk;
    if (chunk < 1) return VL_ERR_UNSUPPORTED;
    dim3 grid(H, B, sh.Z);
    const size_t smem = sizeof(float) * (size_t)2 * chunk * VEC;
    cudaStream_t s = (cudaStream_t)stream;
#define DS_LAUNCH1(TP, RR, LL, FF)                                                                                              \
    return vl_launch(decay_scan_kernel<TP, RR, LL, FF>, grid, dim3(DS_THREADS), smem, s, (const TP*)rp, ldr, rc, (const TP*)kp, \
                     ldk, kc, (const TP*)vp, ldv, vc, (const TP*)wp, ldw, wc, u, state, state_stride, cu, slots, o, H, D, P, chunk, DP)
#define DS_LAUNCH(TP, RR, LL)            \
    do {                                 \
        if (fast) DS_LAUNCH1(TP, RR, LL, true); \
        DS_LAUNCH1(TP, RR, LL, false);   \
    } while (0)
#define DS_PICK(TP)                                                                  \
    do {                                                                             \
        if (sh.rows == 16) DS_LAUNCH(TP, 16, 32);                                    \
        if (sh.rows == 8) DS_LAUNCH(TP, 8, 32);                                      \
        switch (sh.L) {                                                              \
            case 32: DS_LAUNCH(TP, 4, 32);                                           \
            case 16: DS_LAUNCH(TP, 4, 16);                                           \
            case 8: DS_LAUNCH(TP, 4, 8);                                             \
            case 4: DS_LAUNCH(TP, 4, 4);                                             \
            case 2: DS_LAUNCH(TP, 4, 2);                                             \
            default: DS_LAUNCH(TP, 4, 1);                                            \
        }                                                                            \
    } while (0)
    if (dtype == VL_F32) DS_PICK(float);
    if (dtype == VL_BF16) DS_PICK(bf16);
#undef DS_PICK
#undef DS_LAUNCH
#undef DS_LAUNCH1
    return VL_ERR_UNSUPPORTED;
}
