// Shared device/host helpers for the trinix_b200 kernels (sm_100a only).
//
// Everything here is header-only: 16-byte vector pack/unpack for the three
// activation dtypes, warp/CTA reductions, streaming load/store wrappers and
// the status codes returned through the C ABI.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/trinix_b200.h"

namespace trx {

// ----------------------------------------------------------------------------
// dtype traits: VEC = elements in one 16-byte vector.
// ----------------------------------------------------------------------------
template <typename T>
struct Pack;

template <>
struct Pack<float> {
  static constexpr int VEC = 4;
  static constexpr int DTYPE = TRX_F32;
  __device__ __forceinline__ static void unpack(const uint4& r, float (&f)[4]) {
    f[0] = __uint_as_float(r.x);
    f[1] = __uint_as_float(r.y);
    f[2] = __uint_as_float(r.z);
    f[3] = __uint_as_float(r.w);
  }
  __device__ __forceinline__ static uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                      __float_as_uint(f[3]));
  }
  __device__ __forceinline__ static void unpack2(const uint4& r, float2 (&f)[2]) {
    f[0] = make_float2(__uint_as_float(r.x), __uint_as_float(r.y));
    f[1] = make_float2(__uint_as_float(r.z), __uint_as_float(r.w));
  }
  __device__ __forceinline__ static void unpack2_fma(const uint4& r, float2 (&f)[2]) { unpack2(r, f); }
  // Running max of |x| over a vector; `acc` is an opaque per-thread accumulator.
  using AbsAcc = float;
  __device__ __forceinline__ static AbsAcc absacc_init() { return 0.0f; }
  __device__ __forceinline__ static void absacc(const uint4& r, AbsAcc& a) {
    a = fmaxf(a, fmaxf(fmaxf(fabsf(__uint_as_float(r.x)), fabsf(__uint_as_float(r.y))),
                       fmaxf(fabsf(__uint_as_float(r.z)), fabsf(__uint_as_float(r.w)))));
  }
  __device__ __forceinline__ static float absacc_final(const AbsAcc& a) { return a; }
  // Round an fp32 value to the storage type and back (identity for fp32).
  __device__ __forceinline__ static float round(float v) { return v; }
  __device__ __forceinline__ static float load1(const float* p) { return *p; }
  __device__ __forceinline__ static void store1(float* p, float v) { *p = v; }
};

template <>
struct Pack<__nv_bfloat16> {
  static constexpr int VEC = 8;
  static constexpr int DTYPE = TRX_BF16;
  __device__ __forceinline__ static void unpack(const uint4& r, float (&f)[8]) {
    f[0] = __uint_as_float(r.x << 16);
    f[1] = __uint_as_float(r.x & 0xffff0000u);
    f[2] = __uint_as_float(r.y << 16);
    f[3] = __uint_as_float(r.y & 0xffff0000u);
    f[4] = __uint_as_float(r.z << 16);
    f[5] = __uint_as_float(r.z & 0xffff0000u);
    f[6] = __uint_as_float(r.w << 16);
    f[7] = __uint_as_float(r.w & 0xffff0000u);
  }
  __device__ __forceinline__ static float2 cvt2(uint32_t u) {
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
  }
  __device__ __forceinline__ static void unpack2(const uint4& r, float2 (&f)[4]) {
    f[0] = cvt2(r.x); f[1] = cvt2(r.y); f[2] = cvt2(r.z); f[3] = cvt2(r.w);
  }
  // The same conversion as one mixed-precision add per element (x + -0.0 in fp32: exact, keeps
  // the sign of zero). It runs on the FMA pipe, where the shift / mask pair of cvt2 takes two
  // slots of the half-rate integer pipe.
  __device__ __forceinline__ static float2 cvt2_fma(uint32_t u) {
    float lo, hi;
    asm("{.reg .b16 l, h; mov.b32 {l, h}, %2; add.rn.f32.bf16 %0, l, 0f80000000; "
        "add.rn.f32.bf16 %1, h, 0f80000000;}"
        : "=f"(lo), "=f"(hi)
        : "r"(u));
    return make_float2(lo, hi);
  }
  __device__ __forceinline__ static void unpack2_fma(const uint4& r, float2 (&f)[4]) {
    f[0] = cvt2_fma(r.x); f[1] = cvt2_fma(r.y); f[2] = cvt2_fma(r.z); f[3] = cvt2_fma(r.w);
  }
  using AbsAcc = __nv_bfloat162;
  __device__ __forceinline__ static AbsAcc absacc_init() { return __float2bfloat162_rn(0.0f); }
  // max(|a|, |b|) per lane in one instruction (the sign of the result is a don't-care xor)
  __device__ __forceinline__ static uint32_t absmax2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  __device__ __forceinline__ static void absacc(const uint4& r, AbsAcc& a) {
    const uint32_t m = absmax2(absmax2(r.x, r.y), absmax2(r.z, r.w));
    const uint32_t n = absmax2(*reinterpret_cast<const uint32_t*>(&a), m);
    a = *reinterpret_cast<const __nv_bfloat162*>(&n);
  }
  __device__ __forceinline__ static float absacc_final(const AbsAcc& a) {
    return fmaxf(fabsf(__bfloat162float(a.x)), fabsf(__bfloat162float(a.y)));
  }
  __device__ __forceinline__ static uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ __forceinline__ static uint4 pack(const float (&f)[8]) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
  }
  __device__ __forceinline__ static float round(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
  }
  __device__ __forceinline__ static float load1(const __nv_bfloat16* p) {
    return __bfloat162float(*p);
  }
  __device__ __forceinline__ static void store1(__nv_bfloat16* p, float v) {
    *p = __float2bfloat16_rn(v);
  }
};

template <>
struct Pack<__half> {
  static constexpr int VEC = 8;
  static constexpr int DTYPE = TRX_F16;
  __device__ __forceinline__ static void unpack2(uint32_t u, float& lo, float& hi) {
    __half2 h = *reinterpret_cast<__half2*>(&u);
    float2 f = __half22float2(h);
    lo = f.x;
    hi = f.y;
  }
  __device__ __forceinline__ static void unpack(const uint4& r, float (&f)[8]) {
    unpack2(r.x, f[0], f[1]);
    unpack2(r.y, f[2], f[3]);
    unpack2(r.z, f[4], f[5]);
    unpack2(r.w, f[6], f[7]);
  }
  __device__ __forceinline__ static float2 cvt2(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
  __device__ __forceinline__ static void unpack2(const uint4& r, float2 (&f)[4]) {
    f[0] = cvt2(r.x); f[1] = cvt2(r.y); f[2] = cvt2(r.z); f[3] = cvt2(r.w);
  }
  __device__ __forceinline__ static float2 cvt2_fma(uint32_t u) {
    float lo, hi;
    asm("{.reg .b16 l, h; mov.b32 {l, h}, %2; add.rn.f32.f16 %0, l, 0f80000000; "
        "add.rn.f32.f16 %1, h, 0f80000000;}"
        : "=f"(lo), "=f"(hi)
        : "r"(u));
    return make_float2(lo, hi);
  }
  __device__ __forceinline__ static void unpack2_fma(const uint4& r, float2 (&f)[4]) {
    f[0] = cvt2_fma(r.x); f[1] = cvt2_fma(r.y); f[2] = cvt2_fma(r.z); f[3] = cvt2_fma(r.w);
  }
  using AbsAcc = __half2;
  __device__ __forceinline__ static AbsAcc absacc_init() { return __float2half2_rn(0.0f); }
  __device__ __forceinline__ static uint32_t absmax2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.xorsign.abs.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  __device__ __forceinline__ static void absacc(const uint4& r, AbsAcc& a) {
    const uint32_t m = absmax2(absmax2(r.x, r.y), absmax2(r.z, r.w));
    const uint32_t n = absmax2(*reinterpret_cast<const uint32_t*>(&a), m);
    a = *reinterpret_cast<const __half2*>(&n);
  }
  __device__ __forceinline__ static float absacc_final(const AbsAcc& a) {
    return fmaxf(fabsf(__low2float(a)), fabsf(__high2float(a)));
  }
  __device__ __forceinline__ static uint32_t pack2(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ __forceinline__ static uint4 pack(const float (&f)[8]) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
  }
  __device__ __forceinline__ static float round(float v) { return __half2float(__float2half_rn(v)); }
  __device__ __forceinline__ static float load1(const __half* p) { return __half2float(*p); }
  __device__ __forceinline__ static void store1(__half* p, float v) { *p = __float2half_rn(v); }
};

// ----------------------------------------------------------------------------
// Streaming global memory access. Activations are touched exactly once, so
// they bypass L1 allocation; small replicated operands (weights, tables) use
// the read-only path and stay cached.
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
// Ask the copy engine to bring `bytes` (a multiple of 16, from a 16-byte aligned address) into
// L2. One instruction, no completion to wait for.
__device__ __forceinline__ void l2_prefetch_bulk(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
__device__ __forceinline__ void st_stream16(void* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_stream8(void* p, const uint2& v) {
  asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void st_stream4(void* p, uint32_t v) {
  asm volatile("st.global.cs.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_cached16(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

// Load VEC consecutive parameter values (weight / bias) of runtime dtype as fp32.
template <int VEC>
__device__ __forceinline__ void load_param_vec(const void* base, int dtype, int64_t col,
                                               float (&out)[VEC]) {
  if (dtype == TRX_F32) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + col);
#pragma unroll
    for (int i = 0; i < VEC / 4; ++i) {
      float4 v = __ldg(p + i);
      out[4 * i + 0] = v.x;
      out[4 * i + 1] = v.y;
      out[4 * i + 2] = v.z;
      out[4 * i + 3] = v.w;
    }
  } else {
    const uint16_t* b16 = reinterpret_cast<const uint16_t*>(base) + col;
    uint32_t u[VEC / 2];
    if constexpr (VEC == 8) {
      uint4 v = __ldg(reinterpret_cast<const uint4*>(b16));
      u[0] = v.x; u[1] = v.y; u[2] = v.z; u[3] = v.w;
    } else {
      uint2 v = __ldg(reinterpret_cast<const uint2*>(b16));
      u[0] = v.x; u[1] = v.y;
    }
#pragma unroll
    for (int i = 0; i < VEC / 2; ++i) {
      if (dtype == TRX_BF16) {
        out[2 * i] = __uint_as_float(u[i] << 16);
        out[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
      } else {
        Pack<__half>::unpack2(u[i], out[2 * i], out[2 * i + 1]);
      }
    }
  }
}

// One parameter value as fp32. Plain loads on purpose: the half / bfloat16 overloads of
// __ldg are non-volatile inline asm, which the compiler is free to hoist above a null-pointer
// check of an optional weight or bias.
__device__ __forceinline__ float load_param1(const void* base, int dtype, int64_t col) {
  if (dtype == TRX_F32) return reinterpret_cast<const float*>(base)[col];
  const uint16_t bits = reinterpret_cast<const uint16_t*>(base)[col];
  if (dtype == TRX_BF16) return __uint_as_float(static_cast<uint32_t>(bits) << 16);
  return __half2float(__ushort_as_half(bits));
}

// ----------------------------------------------------------------------------
// Reductions
// ----------------------------------------------------------------------------
template <bool IS_MAX>
__device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = IS_MAX ? fmaxf(v, t) : v + t;
  }
  return v;
}

// Reduce across the TPR threads that share one row. TPR == 32: within the warp only.
// TPR > 32 (== blockDim.x, one row per CTA): one shared-memory hop; `red` has two banks that
// alternate so that no trailing barrier is needed. IS_MAX reduces NON-NEGATIVE values, whose
// fp32 bit patterns order like unsigned integers, with a single redux.sync per warp.
template <int TPR, bool IS_MAX>
__device__ __forceinline__ float row_reduce(float v, float (*red)[32], int& sel) {
  if constexpr (IS_MAX) {
    v = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(v)));
  } else {
    v = warp_reduce<false>(v);
  }
  if constexpr (TPR > 32) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    if (lane == 0) red[sel][warp] = v;
    __syncthreads();
    constexpr int NW = TPR / 32;
    if constexpr (NW <= 8) {
      // every thread reads all partials (broadcast loads) and combines them in registers
      float part[NW];
      if constexpr (NW % 4 == 0) {
#pragma unroll
        for (int i = 0; i < NW / 4; ++i) {
          const float4 q = reinterpret_cast<const float4*>(red[sel])[i];
          part[4 * i] = q.x; part[4 * i + 1] = q.y; part[4 * i + 2] = q.z; part[4 * i + 3] = q.w;
        }
      } else {
        const float2 q = reinterpret_cast<const float2*>(red[sel])[0];
        part[0] = q.x; part[1] = q.y;
      }
      v = part[0];
#pragma unroll
      for (int i = 1; i < NW; ++i) v = IS_MAX ? fmaxf(v, part[i]) : v + part[i];
    } else {
      v = (lane < NW) ? red[sel][lane] : 0.0f;
      if constexpr (IS_MAX) {
        v = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(v)));
      } else {
        v = warp_reduce<false>(v);
      }
    }
    sel ^= 1;
  }
  return v;
}

// The int8 code of one value: round-half-to-even of the true quotient,
// clamped to [-127, 127]. A zero row (scale == 0) encodes to all zeros.
__device__ __forceinline__ int quant_code(float x, float scale) {
  float q = (scale > 0.0f) ? rintf(__fdiv_rn(x, scale)) : 0.0f;
  q = fminf(fmaxf(q, -127.0f), 127.0f);
  return static_cast<int>(q);
}


// ----------------------------------------------------------------------------
// Packed fp32x2 arithmetic (sm_100a): one issue slot for two lanes of work.
// ----------------------------------------------------------------------------
__device__ __forceinline__ float2 fma2(const float2& a, const float2& b, const float2& c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(d)
      : "l"(*reinterpret_cast<const uint64_t*>(&a)), "l"(*reinterpret_cast<const uint64_t*>(&b)),
        "l"(*reinterpret_cast<const uint64_t*>(&c)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 mul2(const float2& a, const float2& b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(*reinterpret_cast<const uint64_t*>(&a)), "l"(*reinterpret_cast<const uint64_t*>(&b)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 add2(const float2& a, const float2& b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(*reinterpret_cast<const uint64_t*>(&a)), "l"(*reinterpret_cast<const uint64_t*>(&b)));
  return *reinterpret_cast<float2*>(&d);
}

// Per-row constants of the int8 encoder.
struct QuantRow {
  float scale;   // absmax / 127 (IEEE division)
  float rcp_lo;  // below 1/scale by 2^-24 .. 2^-20 relative
  float rcp_hi;  // above 1/scale by 2^-24 .. 2^-20 relative
  int mode;      // 0: zero row, 1: bracketed / FMA-refined quotient, 2: plain IEEE division
};
__device__ __forceinline__ QuantRow make_quant_row(float absmax) {
  QuantRow q;
  q.scale = __fdiv_rn(absmax, 127.0f);
  // hardware reciprocal: within 2^-23 relative of 1/scale (the bound used below is 2^-22)
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(q.scale));
  q.rcp_lo = __fmul_rn(r, 1.0f - 0x1p-21f);
  q.rcp_hi = __fmul_rn(r, 1.0f + 0x1p-21f);
  // The refined quotient below equals the IEEE quotient whenever no intermediate
  // can underflow or overflow; keep it to scales comfortably inside the normal range.
  q.mode = !(q.scale > 0.0f) ? 0 : ((q.scale > 1e-18f && q.scale < 1e18f) ? 1 : 2);
  return q;
}

// Fast int8 encoder for mode-1 rows: two codes from two FMAs each, no quotient at all.
// t_lo = RN(x*rcp_lo + 1.5*2^23) and t_hi = RN(x*rcp_hi + 1.5*2^23) are each a single rounding
// of an exact product to the integer grid (half to even). With rho = 1/scale, r within 2^-22 of
// rho and one more rounding (2^-24) in each bracket, rcp_lo <= rho*(1 - 3*2^-24) and rcp_hi >=
// rho*(1 + 3*2^-24), while the IEEE quotient Q = RN(x/scale) is within 2^-24 of x*rho: Q lies
// strictly between x*rcp_lo and x*rcp_hi. Rounding to the integer grid is monotonic, so
// t_lo == t_hi implies RN(Q + 1.5*2^23) is that same value, i.e. the low byte of t_lo is
// rint(Q). When the two differ (Q within ~|Q|*2^-20 of a half-integer, a few values in 10^5)
// `differ` becomes non-zero and the caller re-encodes with quant_pair<1>.
__device__ __forceinline__ void quant_pair_bracketed(const float2& x, const QuantRow& qr,
                                                     uint32_t& b0, uint32_t& b1, uint32_t& differ) {
  const float2 magic = make_float2(12582912.0f, 12582912.0f);
  const float2 lo = fma2(x, make_float2(qr.rcp_lo, qr.rcp_lo), magic);
  const float2 hi = fma2(x, make_float2(qr.rcp_hi, qr.rcp_hi), magic);
  b0 = __float_as_uint(lo.x);
  b1 = __float_as_uint(lo.y);
  differ |= (b0 ^ __float_as_uint(hi.x)) | (b1 ^ __float_as_uint(hi.y));
}

// Two int8 codes at once. The quotient x/scale is formed as q = x*rcp followed by FMA
// residual corrections q += (x - q*scale) * rcp with rcp = RN(1/scale). The first correction
// brings q within a fraction of an ulp of the quotient; the second one (Markstein's final
// step, valid because rcp is correctly rounded and q is then faithful) makes it the correctly
// rounded IEEE quotient. Adding 1.5*2^23 then rounds the quotient half-to-even to an integer
// whose two's-complement low byte is the low mantissa byte. |x| <= absmax keeps the integer
// in [-127, 127], so no clamp is needed.
// MODE: 0 zero row, 1 refined quotient, 2 plain IEEE division (extreme scales).
#ifndef TRX_QUANT_REFINE
#define TRX_QUANT_REFINE 2
#endif
template <int MODE, bool NARROW>
__device__ __forceinline__ void quant_pair(const float2& x, const QuantRow& qr, uint32_t& b0,
                                           uint32_t& b1) {
  float2 q;
  if constexpr (MODE == 1) {
    const float rcp = __frcp_rn(qr.scale);  // this path is rare: not worth a register per row
    const float2 r = make_float2(rcp, rcp);
    const float2 ns = make_float2(-qr.scale, -qr.scale);
    q = mul2(x, r);
    float2 e = fma2(q, ns, x);
    q = fma2(e, r, q);
    if constexpr (TRX_QUANT_REFINE >= 2 || !NARROW) {
      e = fma2(q, ns, x);
      q = fma2(e, r, q);
    }
  } else if constexpr (MODE == 2) {
    q.x = fminf(fmaxf(__fdiv_rn(x.x, qr.scale), -127.0f), 127.0f);
    q.y = fminf(fmaxf(__fdiv_rn(x.y, qr.scale), -127.0f), 127.0f);
  } else {
    q = make_float2(0.0f, 0.0f);
  }
  const float2 y = add2(q, make_float2(12582912.0f, 12582912.0f));
  b0 = __float_as_uint(y.x);
  b1 = __float_as_uint(y.y);
}
// Low bytes of four words -> one word.
__device__ __forceinline__ uint32_t pack_low_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  const uint32_t lo = __byte_perm(a, b, 0x0040);
  const uint32_t hi = __byte_perm(c, d, 0x0040);
  return __byte_perm(lo, hi, 0x5410);
}

// SM count of the current device, cached per device ordinal.
inline int sm_count_of_current_device() {
  static std::atomic<int> cached[64];  // racing first calls store the same value
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int n = cached[dev].load(std::memory_order_acquire);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev].store(n, std::memory_order_release);
  }
  return n;
}

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

}  // namespace trx
