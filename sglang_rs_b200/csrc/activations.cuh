// The activation of a gated feed-forward, act(gate) * up, as a number that the part chooses: the
// epilogues of the two tcgen05 products and the stand-alone kernel all call srb_gated().  Another
// activation is one more case here and one more name in parts/mlp.py; no kernel changes.
//
//   SRB_ACT_SILU       g / (1 + exp(-g))                     (crates/sglang-kernel/src/cpu.rs:119-123)
//   SRB_ACT_GELU_TANH  g/2 * (1 + tanh(sqrt(2/pi) * (g + 0.044715 g^3)))
//
// EXACT selects the full-precision exponential and division (the 32-bit path and epilogues whose
// result stays 32-bit); without it the hardware's approximations are used, which is exact enough for
// a result that is rounded to bfloat16.
#pragma once

#define SRB_ACT_SILU 0
#define SRB_ACT_GELU_TANH 1
#define SRB_ACT_COUNT 2

template <bool EXACT>
__device__ __forceinline__ float srb_gated(int activation, float g, float u) {
  if (activation == SRB_ACT_GELU_TANH) {
    const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    // tanh(x) = 1 - 2 / (exp(2x) + 1): finite for every x
    const float t = EXACT ? 1.0f - 2.0f / (expf(2.0f * inner) + 1.0f) : 1.0f - __fdividef(2.0f, __expf(2.0f * inner) + 1.0f);
    return 0.5f * g * (1.0f + t) * u;
  }
  return (EXACT ? g / (1.0f + expf(-g)) : __fdividef(g, 1.0f + __expf(-g))) * u;
}
