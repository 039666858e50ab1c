// Two options on attention scores that every tensor-core attention kernel shares (csrc/flash_attn.cu, csrc/flash_tc5.cu):
// a bound, s <- cap tanh(s / cap), and a bias that grows with the logarithm of the distance, s <- s - a ln(1 + b d).
#pragma once

__device__ __forceinline__ float ss_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// A score y (already scaled, in units of log2) bounded by cap_l2 and less the bias of a key `dist` positions back, still in
// units of log2: cap tanh(y / cap), tanh(z) = 1 - 2 / (1 + e^(2z)); a ln(1 + b d) log2 e = a log2(1 + b d).
__device__ __forceinline__ float shape_score(float y, float cap_l2, float two_over_cap, float da, float db, int dist) {
    if (cap_l2 > 0.f) {
        float r;
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + ss_exp2(y * two_over_cap)));
        y = cap_l2 - 2.f * cap_l2 * r;
    }
    if (da != 0.f) {
        float l;
        asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(l) : "f"(fmaf(db, (float)dist, 1.f)));
        y -= da * l;
    }
    return y;
}
// 2 log2(e) / cap_l2: what a score in units of log2 is multiplied by to give the exponent of 2 that is e^(2 s / cap)
__device__ __forceinline__ float two_over_cap(float cap_l2) { return cap_l2 > 0.f ? 2.f * 1.4426950408889634f / cap_l2 : 0.f; }
