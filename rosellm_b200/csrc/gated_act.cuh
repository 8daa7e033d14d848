// Gated activations of feed-forward layers with two input projections, gate g and up u:
// the unit's value is f(g, u).  Arithmetic in float32.
#pragma once
#include "common.cuh"

#define RL_GATE_RELU 0           // max(g, 0) * u
#define RL_GATE_SILU 1           // g * sigmoid(g) * u
#define RL_GATE_GELU_TANH 2      // gelu_tanh(g) * u
#define RL_GATE_CLAMPED_SWISH 3  // g' = min(g, limit), u' = clamp(u, -limit, limit): g' * sigmoid(alpha g') * (u' + 1)

namespace rl {

__device__ __forceinline__ float gelu_tanh_f32(float z) {
  const float c = 0.7978845608028654f;  // sqrt(2/pi)
  return 0.5f * z * (1.0f + tanhf(c * (z + 0.044715f * z * z * z)));
}

__device__ __forceinline__ float gated_value(float g, float u, int kind, float alpha, float limit) {
  switch (kind) {
    case RL_GATE_RELU: return fmaxf(g, 0.f) * u;
    case RL_GATE_SILU: return g / (1.0f + expf(-g)) * u;
    case RL_GATE_GELU_TANH: return gelu_tanh_f32(g) * u;
    default: {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
    }
  }
}

}  // namespace rl
