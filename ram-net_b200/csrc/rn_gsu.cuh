// Scalar math of the gated sparse update, shared by the decode and prefill kernels.
//
//   alpha    = (1 - w) / ((1 - w) + e^gamma * w)          (forgetting factor of the slot's mass)
//   mass'    = alpha * mass + w
//   gain     = w / (mass' + eps)
//   slot'    = slot + gain * (x - slot)
//
// (packages/ramnet-ops/src/ramnet_ops/impl/torch_impl.py:56-66 of the reference.)  For
// gamma >= 0 numerator and denominator are scaled by e^-gamma so the exponential never
// overflows; the value of alpha is unchanged.
#pragma once

#include "rn_common.cuh"

struct RnGate {
    float gain;
    float mass;   // updated mass
    float alpha;
};

__device__ __forceinline__ float rn_alpha(float w, float gamma) {
    const float e = expf(-fabsf(gamma));
    const float cw = 1.f - w;
    return gamma >= 0.f ? (cw * e) / (w + e * cw) : cw / (cw + e * w);
}

__device__ __forceinline__ RnGate rn_gate(float w, float gamma, float mass, float eps) {
    RnGate g;
    g.alpha = rn_alpha(w, gamma);
    g.mass = fmaf(g.alpha, mass, w);
    g.gain = w / (g.mass + eps);
    return g;
}
