// The gated unit of the feed-forwards, shared by the row-wise kernel and the experts' kernels:
//   g = min(gate, gate_max);  u = clamp(up, -up_limit, up_limit);  act(g) * (u + up_shift)
// act 0: silu, 1: gelu in its tanh form 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), 2: z sigmoid(alpha z).
// Infinite limits and a shift of 0 give the plain unit act(gate) * up.  float32 throughout.
#pragma once
#include <math.h>

struct GluShape { int kind; float alpha, gate_max, up_limit, up_shift; };

__device__ __forceinline__ float glu_act(float z, const GluShape& p) {
    if (p.kind == 0) return z / (1.f + expf(-z));
    if (p.kind == 2) return z / (1.f + expf(-p.alpha * z));
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float glu_unit(float g, float u, const GluShape& p) {
    g = fminf(g, p.gate_max);
    u = fminf(fmaxf(u, -p.up_limit), p.up_limit);
    return glu_act(g, p) * (u + p.up_shift);
}
