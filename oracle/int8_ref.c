/*
 * Plain-C restatement of the per-row symmetric int8 path (test infrastructure only;
 * never linked into the product library).
 *
 * The reference has no int8 code; the contract is this project's baseline
 * configuration: scale = rowwise absmax / 127 (fp32, IEEE division),
 * code = clamp(round_half_even(x / scale), -127, 127), zero rows -> scale 0, codes 0.
 * Compile WITHOUT -ffast-math so that `/` is the IEEE division and nearbyintf() under
 * the default rounding mode is round-half-to-even.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static float bf16_to_f32(uint16_t b) {
  uint32_t u = ((uint32_t)b) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* x: R*C bf16 bit patterns, row-major. */
void oracle_quant_rowwise_bf16(const uint16_t* x, int8_t* codes, float* scales, int64_t R,
                               int64_t C) {
  for (int64_t r = 0; r < R; ++r) {
    const uint16_t* xr = x + r * C;
    float am = 0.0f;
    for (int64_t c = 0; c < C; ++c) {
      float a = fabsf(bf16_to_f32(xr[c]));
      if (a > am) am = a;
    }
    float s = am / 127.0f;
    scales[r] = s;
    for (int64_t c = 0; c < C; ++c) {
      float q = 0.0f;
      if (s > 0.0f) {
        q = nearbyintf(bf16_to_f32(xr[c]) / s);
        if (q > 127.0f) q = 127.0f;
        if (q < -127.0f) q = -127.0f;
      }
      codes[r * C + c] = (int8_t)q;
    }
  }
}

/* y: R*C bf16 bit patterns = round_bf16(float(code) * scale). */
void oracle_dequant_rowwise_bf16(const int8_t* codes, const float* scales, uint16_t* y, int64_t R,
                                 int64_t C) {
  for (int64_t r = 0; r < R; ++r)
    for (int64_t c = 0; c < C; ++c)
      y[r * C + c] = f32_to_bf16((float)codes[r * C + c] * scales[r]);
}
