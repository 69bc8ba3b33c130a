// Row kernels: RMSNorm, LayerNorm, per-row int8 quantise, fused RMSNorm -> int8, the residual
// forms RMSNorm(x + r), RMSNorm(x + r) -> int8 and LayerNorm(x + r), and act(RMSNorm(x)).
//
// One skeleton serves the eight ops. A row is read from HBM exactly once with
// 128-bit streaming loads and then lives in registers (VPT 16-byte vectors per
// thread, TPR threads per row); statistics are reduced with warp shuffles
// (plus one shared-memory hop when a row spans more than one warp), and the
// result is produced from the registers — the row is never re-read.
//   TPR == 32 : one warp per row, 8 rows per 256-thread CTA, no barriers at all (short rows).
//   TPR  > 32 : one CTA of TPR threads per row, few vectors per thread.
// The grid is several resident waves of CTAs, each striding over a few rows (see
// launch_cfg_full). Rows of exactly TPR * VPT vectors run a specialisation without guards.
// Rows that do not fit the vector path (columns not a multiple of the vector width,
// unaligned pointers, more than 16384 vectors) take a scalar multi-pass kernel, so nothing
// is ever truncated.
#include <atomic>
#include <type_traits>

#include "common.cuh"

namespace trx {

// (threads per row, vectors per thread) for rows of up to 256 vectors. Few vectors per thread
// keep register pressure low enough for many CTAs per SM; the row then spans several warps
// and pays one barrier per reduction. Rows of up to 512 vectors (4096 bf16 columns, the
// benchmark width) choose per op, see launch_row.
#ifndef TRX_ROW256_TPR
#define TRX_ROW256_TPR 64
#define TRX_ROW256_VPT 4
#endif

// How many rows ahead of the one it is loading a CTA asks the copy engine to pull into L2
// (one bulk-prefetch instruction per row, fire and forget). 0 = off.
#ifndef TRX_ROW_L2_PREFETCH
#define TRX_ROW_L2_PREFETCH 1
#endif

// Sum of squares of a 16-bit row straight from the packed words with the mixed-precision FMA
// (fp32 accumulator, 16-bit multiplicands: the product of two 16-bit values is exact in fp32, so
// the result equals the fp32 FMA on unpacked values bit for bit) instead of unpack + packed FMA.
#ifndef TRX_ROW_MIXED_SS
#define TRX_ROW_MIXED_SS 1
#endif

// Unpack 16-bit pairs to fp32 on the FMA pipe (one mixed-precision add per element) instead of
// the integer pipe (shift + mask) in the int8 ops. Measured on the fused RMSNorm -> int8 kernel
// at 32768 x 4096, 10 CTAs per SM: -1.8 % in the encode pass, +1.8 % in the normalise pass; at
// 16 CTAs per SM, where the ALU pipe is the busiest (59 % against 49 % FMA), the normalise pass
// gains another 1.2 % (69.2 -> 68.4 us), so both passes use it.
#ifndef TRX_QUANT_FMA_UNPACK
#define TRX_QUANT_FMA_UNPACK 1
#endif

// Resident threads per SM asked for the int8 encoders in the 64-thread x 8-vector configuration
// (caps the registers per thread at 64). These kernels are bound by the supply of eligible warps,
// not by a pipe or by DRAM: measured on the fused RMSNorm -> int8 kernel at 32768 x 4096, 640
// threads (96 registers) 76.6 us, 768: 72.1, 896: 70.9, 960 / 1024: 69.4, 1088: 74.5, 1280: 81.3.
#ifndef TRX_ROW64_THREADS_PER_SM
#define TRX_ROW64_THREADS_PER_SM 1024
#endif

enum RowOp {
  OP_RMSNORM = 0,
  OP_LAYERNORM = 1,
  OP_QUANT = 2,
  OP_RMSNORM_QUANT = 3,
  OP_RES_RMSNORM = 4,        // RMSNorm(x + residual)
  OP_RES_RMSNORM_QUANT = 5,  // RMSNorm(x + residual) -> int8
  OP_RMSNORM_ACT = 6,        // act(RMSNorm(x)), act in {mish, quickgelu, squared_relu}
  OP_RES_LAYERNORM = 7       // LayerNorm(x + residual)
};
__host__ __device__ constexpr bool op_is_ln(int op) { return op == OP_LAYERNORM || op == OP_RES_LAYERNORM; }
__host__ __device__ constexpr bool op_is_rms(int op) {
  return op == OP_RMSNORM || op == OP_RMSNORM_QUANT || op == OP_RES_RMSNORM ||
         op == OP_RES_RMSNORM_QUANT || op == OP_RMSNORM_ACT;
}
__host__ __device__ constexpr bool op_has_quant(int op) {
  return op == OP_QUANT || op == OP_RMSNORM_QUANT || op == OP_RES_RMSNORM_QUANT;
}
__host__ __device__ constexpr bool op_has_res(int op) {
  return op == OP_RES_RMSNORM || op == OP_RES_RMSNORM_QUANT || op == OP_RES_LAYERNORM;
}
// Minimum resident CTAs per SM asked of the compiler (caps registers per thread): a thread
// budget per SM that was measured per family, divided by the CTA size.
__host__ __device__ constexpr int row_min_blocks(int op, int tpr, int vpt) {
  if (tpr <= 32) return 3;                      // 256-thread CTAs, 8 rows each
  if (tpr > 256) return 1;
  if (op_has_res(op)) return 768 / tpr;         // two streams + fp32 copies: more registers
  if (tpr == 64 && vpt == 8)  // 8 vectors per thread in flight
    return (op_has_quant(op) ? TRX_ROW64_THREADS_PER_SM : 640) / tpr;

  return 1024 / tpr;
}

struct RowParamsBase {
  const void* x;
  const void* w;
  const void* b;
  void* y;
  int8_t* codes;
  float* scales;
  float* mean;
  float* rstd;
  int64_t R;
  int64_t C;
  int64_t x_stride;      // elements
  int64_t y_stride;      // elements
  int64_t codes_stride;  // bytes == elements
  float eps;
  int w_dtype;
};
// What the residual variants take on top, as a second kernel argument: a parameter block above
// 128 bytes is no longer read field by field, which cost the plain kernels 5-9 %.
struct ResParams {
  const void* res;     // residual added to x before RMSNorm (fp32 sum)
  void* sum_out;       // optional: round_T(x + res)
  int64_t res_stride;  // elements
  int64_t sum_stride;  // elements
};
struct NoRes {};
struct ActParams {
  int act;  // TRX_ACT_*
};
struct RowParams : RowParamsBase {
  ResParams rp;
  ActParams ap;
};
template <int OP>
using ResArg = std::conditional_t<op_has_res(OP), ResParams,
                                  std::conditional_t<OP == OP_RMSNORM_ACT, ActParams, NoRes>>;
template <int OP>
static ResArg<OP> res_arg(const RowParams& p) {
  if constexpr (op_has_res(OP)) return p.rp;
  else if constexpr (OP == OP_RMSNORM_ACT) return p.ap;
  else return NoRes{};
}

// Activations of the fused RMSNorm + activation op, on the fp32 value of the normalised element
// (trinix/layers/fused/rmsnorm_activation.py:79-84). mish(n) = n * tanh(softplus(n)) with
// tanh(ln(1 + u)) = (u^2 + 2u) / (u^2 + 2u + 2), u = e^n: one exponential and one division;
// beyond n = 20 (torch's softplus threshold) softplus(n) = n and tanh(n) = 1 in fp32.
// FAST (16-bit outputs): hardware exp2 on a pre-scaled argument and the approximate division,
// both some 2^-21 relative, far below the storage rounding step; fp32 outputs take expf and the
// IEEE division.
template <bool FAST>
__device__ __forceinline__ float row_exp(float x) {
  if constexpr (FAST) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x * 1.4426950408889634f));
    return r;
  } else {
    return expf(x);
  }
}
template <bool FAST>
__device__ __forceinline__ float row_div(float a, float b) {
  if constexpr (FAST) return __fdividef(a, b);
  else return __fdiv_rn(a, b);
}
template <bool FAST>
__device__ __forceinline__ float row_act(float n, int act) {
  if (act == TRX_ACT_MISH) {
    // e^20 squared is already 2.4e17: q / (q + 2) == 1 in fp32 from there on, so clamping the
    // exponent reproduces softplus's n > 20 shortcut without a branch (and keeps q finite)
    const float u = row_exp<FAST>(fminf(n, 20.0f));
    const float q = u * (u + 2.0f);
    return n * row_div<FAST>(q, q + 2.0f);
  }
  if (act == TRX_ACT_QUICKGELU) return n * row_div<FAST>(1.0f, 1.0f + row_exp<FAST>(-1.702f * n));
  const float r = fmaxf(n, 0.0f);  // squared ReLU
  return r * r;
}

// Packed product of two 16-bit pairs with one rounding per lane.
template <typename T>
__device__ __forceinline__ uint32_t mul_packed16(uint32_t a, uint32_t b);
template <>
__device__ __forceinline__ uint32_t mul_packed16<__nv_bfloat16>(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r =
      __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
template <>
__device__ __forceinline__ uint32_t mul_packed16<__half>(uint32_t a, uint32_t b) {
  const __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
template <>
__device__ __forceinline__ uint32_t mul_packed16<float>(uint32_t a, uint32_t) {
  return a;  // never used: fp32 rows take the scalar-lane path
}

// 1/sqrt(mean + eps) from a row sum: a multiply by 1/C (formed once per thread) and the
// hardware reciprocal square root (2 ulp). The IEEE divide / sqrt / divide sequence costs ~40
// instructions per thread and row and buys nothing: the fp32 summation order already differs
// from any host implementation at that level.
__device__ __forceinline__ float rsqrt_approx(float v) {
  float r;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}

// acc_lo += lo(u)^2, acc_hi += hi(u)^2 for a word of two 16-bit values, in fp32.
template <typename T>
__device__ __forceinline__ void sq_acc_word(uint32_t u, float& acc_lo, float& acc_hi) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    asm("{.reg .b16 l, h; mov.b32 {l, h}, %2; fma.rn.f32.bf16 %0, l, l, %0; "
        "fma.rn.f32.bf16 %1, h, h, %1;}"
        : "+f"(acc_lo), "+f"(acc_hi)
        : "r"(u));
  } else {
    asm("{.reg .b16 l, h; mov.b32 {l, h}, %2; fma.rn.f32.f16 %0, l, l, %0; "
        "fma.rn.f32.f16 %1, h, h, %1;}"
        : "+f"(acc_lo), "+f"(acc_hi)
        : "r"(u));
  }
}

// FULL: every row has exactly TPR * VPT vectors and the row count is a multiple of the rows per
// CTA, so no vector of any thread is padding. The guards disappear, and with them some thirty
// branches per warp and row that kept the four vectors of a thread from being scheduled together.
template <int OP, typename T, int TPR, int VPT, bool FULL>
__global__ void __launch_bounds__((TPR > 32 ? TPR : 256), row_min_blocks(OP, TPR, VPT))
    row_kernel(const RowParamsBase p, const ResArg<OP> rp) {
  using P = Pack<T>;
  constexpr int VEC = P::VEC;
  constexpr int BLOCK = TPR > 32 ? TPR : 256;
  constexpr int ROWS_PER_CTA = BLOCK / TPR;
  constexpr bool HAS_NORM = op_is_rms(OP) || op_is_ln(OP);
  constexpr bool HAS_QUANT = op_has_quant(OP);
  constexpr bool HAS_RES = op_has_res(OP);
  constexpr bool NORM_TO_REGS = (OP == OP_RMSNORM_QUANT || OP == OP_RES_RMSNORM_QUANT);

  __shared__ __align__(16) float red[2][32];
  int sel = 0;

  const int t = threadIdx.x % TPR;
  const int row_in_cta = threadIdx.x / TPR;
  const int nvec = static_cast<int>(p.C / VEC);
  const float inv_C = __fdiv_rn(1.0f, static_cast<float>(p.C));

  const int64_t row_step = static_cast<int64_t>(gridDim.x) * ROWS_PER_CTA;
  // The residual forms keep the fp32 sum x + r of a 16-bit row on chip between the statistics
  // and the normalise pass (it exists nowhere else). The other ops unpack the packed row a
  // second time instead: 32 fewer live registers measured better than 8 fewer instructions.
  constexpr bool KEEP_F32 = (VEC == 8) && (VPT <= 4) && HAS_RES;

  for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * ROWS_PER_CTA; row0 < p.R;
       row0 += row_step) {
    const int64_t row = row0 + row_in_cta;
    const bool row_ok = FULL || row < p.R;
    auto live = [&](int i) -> bool { return FULL || (row_ok && i * TPR + t < nvec); };

    // ---- 1. the one and only HBM read of the row ------------------------------------
    uint4 raw[VPT];
    {
      const T* xrow = reinterpret_cast<const T*>(p.x) + (FULL || row_ok ? row : 0) * p.x_stride;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = i * TPR + t;
        raw[i] = live(i) ? ld_stream16(xrow + static_cast<int64_t>(v) * VEC)
                                      : make_uint4(0u, 0u, 0u, 0u);
      }
    }
    // Measured per op: it pays where a row costs two HBM streams (residual forms, +10-16 %) or
    // two passes over the registers (LayerNorm, +4 %), and costs 5-8 % on the others.
        if constexpr (TRX_ROW_L2_PREFETCH > 0 && (HAS_RES || op_is_ln(OP))) {
      // While this row is in flight, have the row this CTA takes next pulled from HBM into L2, so
      // that its loads find it there: the only rows a CTA waits for at HBM latency are its first.
      const int64_t prow = row + TRX_ROW_L2_PREFETCH * row_step;
      if (t == 0 && prow < p.R) {
        const uint32_t row_bytes = static_cast<uint32_t>(nvec) * 16u;
        l2_prefetch_bulk(reinterpret_cast<const T*>(p.x) + prow * p.x_stride, row_bytes);
        if constexpr (HAS_RES)
          l2_prefetch_bulk(reinterpret_cast<const T*>(rp.res) + prow * rp.res_stride, row_bytes);
      }
    }
    float2 xf[KEEP_F32 ? VPT : 1][VEC / 2];
    (void)xf;

    float mean = 0.0f, rstd = 1.0f;
    // Residual forms: f2 (vector i of x, unpacked) += the residual's vector; the sum is formed and
    // normalised in fp32, as the reference's PyTorch paths do (layers/fused/residual_rmsnorm.py:
    // 66-73, residual_layernorm.py:66-73), and optionally written out rounded. The host
    // guarantees a configuration that keeps the fp32 sum on chip.
    auto add_residual = [&](int i, float2 (&f2)[VEC / 2]) {
      if constexpr (HAS_RES) {
        const T* rrow = reinterpret_cast<const T*>(rp.res) + (FULL || row_ok ? row : 0) * rp.res_stride;
        T* srow = reinterpret_cast<T*>(rp.sum_out) + (FULL || row_ok ? row : 0) * rp.sum_stride;
        const int v = i * TPR + t;
        if (live(i)) {
          const int64_t col = static_cast<int64_t>(v) * VEC;
          float2 r2[VEC / 2];
          P::unpack2(ld_stream16(rrow + col), r2);
#pragma unroll
          for (int j = 0; j < VEC / 2; ++j) f2[j] = add2(f2[j], r2[j]);
          if constexpr (VEC == 4) {
            raw[i] = make_uint4(__float_as_uint(f2[0].x), __float_as_uint(f2[0].y),
                                __float_as_uint(f2[1].x), __float_as_uint(f2[1].y));
            if (rp.sum_out) st_stream16(srow + col, raw[i]);
          } else {
            if (rp.sum_out)
              st_stream16(srow + col, make_uint4(P::pack2(f2[0].x, f2[0].y), P::pack2(f2[1].x, f2[1].y),
                                                 P::pack2(f2[2].x, f2[2].y), P::pack2(f2[3].x, f2[3].y)));
          }
        }
      }
    };
    // ---- 2. statistics -------------------------------------------------------------
    if constexpr (op_is_rms(OP)) {
      float2 ss2 = make_float2(0.0f, 0.0f), ss2b = make_float2(0.0f, 0.0f);  // two chains
      if constexpr (TRX_ROW_MIXED_SS && VEC == 8 && !HAS_RES) {
        // same four accumulation chains, same order, as the unpacked form below
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          sq_acc_word<T>(raw[i].x, ss2.x, ss2.y);
          sq_acc_word<T>(raw[i].y, ss2b.x, ss2b.y);
          sq_acc_word<T>(raw[i].z, ss2.x, ss2.y);
          sq_acc_word<T>(raw[i].w, ss2b.x, ss2b.y);
        }
      } else {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          float2 f2[VEC / 2];
          P::unpack2(raw[i], f2);
          add_residual(i, f2);
#pragma unroll
          for (int j = 0; j < VEC / 2; ++j) {
            if (j & 1) ss2b = fma2(f2[j], f2[j], ss2b);
            else ss2 = fma2(f2[j], f2[j], ss2);
            if constexpr (KEEP_F32) xf[i][j] = f2[j];
          }
        }
      }
      ss2 = add2(ss2, ss2b);
      if constexpr (VEC == 8 && !KEEP_F32) {
        // keep the compiler from carrying the fp32 copies across the reduction after all (it
        // would, by common-subexpression elimination): the packed row is all that stays live
#pragma unroll
        for (int i = 0; i < VPT; ++i)
          asm volatile("" : "+r"(raw[i].x), "+r"(raw[i].y), "+r"(raw[i].z), "+r"(raw[i].w));
      }
      float ss = row_reduce<TPR, false>(ss2.x + ss2.y, red, sel);
      rstd = rsqrt_approx(fmaf(ss, inv_C, p.eps));
    } else if constexpr (op_is_ln(OP)) {
      float2 s2 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        float2 f2[VEC / 2];
        P::unpack2(raw[i], f2);
        add_residual(i, f2);
#pragma unroll
        for (int j = 0; j < VEC / 2; ++j) {
          s2 = add2(s2, f2[j]);
          if constexpr (KEEP_F32) xf[i][j] = f2[j];
        }
      }
      const float s = row_reduce<TPR, false>(s2.x + s2.y, red, sel);
      mean = s * inv_C;
      const float2 nmean2 = make_float2(-mean, -mean);
      float2 cs2 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = i * TPR + t;
        if (FULL || v < nvec) {  // padding vectors must not contribute (0 - mean)^2
          float2 f2[VEC / 2];
          if constexpr (KEEP_F32) {
#pragma unroll
            for (int j = 0; j < VEC / 2; ++j) f2[j] = xf[i][j];
          } else {
            P::unpack2(raw[i], f2);
          }
#pragma unroll
          for (int j = 0; j < VEC / 2; ++j) {
            const float2 d = add2(f2[j], nmean2);
            cs2 = fma2(d, d, cs2);
          }
        }
      }
      float cs = cs2.x + cs2.y;
      cs = row_reduce<TPR, false>(cs, red, sel);
      rstd = rsqrt_approx(fmaf(cs, inv_C, p.eps));
    }
    if constexpr (HAS_NORM) {
      if (row_ok && t == 0) {
        if (p.rstd) p.rstd[row] = rstd;
        if (op_is_ln(OP) && p.mean) p.mean[row] = mean;
      }
    }

    // ---- 3. normalise (registers -> registers, or registers -> HBM) ----------------
    // All dtype / null-pointer decisions are taken once per row, outside the vector loops.
    if constexpr (HAS_NORM) {
      T* yrow = NORM_TO_REGS
                    ? nullptr
                    : reinterpret_cast<T*>(p.y) + (FULL || row_ok ? row : 0) * p.y_stride;
      auto emit = [&](int i, int64_t col, const uint4& packed) {
        if constexpr (NORM_TO_REGS) {
          raw[i] = packed;
        } else {
          st_stream16(yrow + col, packed);
        }
      };
      if constexpr (op_is_ln(OP)) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = i * TPR + t;
          if (live(i)) {
            float f[VEC];
            if constexpr (KEEP_F32) {
#pragma unroll
              for (int j = 0; j < VEC / 2; ++j) {
                f[2 * j] = xf[i][j].x;
                f[2 * j + 1] = xf[i][j].y;
              }
            } else {
              P::unpack(raw[i], f);
            }
            const int64_t col = static_cast<int64_t>(v) * VEC;
            float wv[VEC], bv[VEC];
            if (p.w) load_param_vec<VEC>(p.w, p.w_dtype, col, wv);
            if (p.b) load_param_vec<VEC>(p.b, p.w_dtype, col, bv);
#pragma unroll
            for (int j = 0; j < VEC; ++j) {
              float o = (f[j] - mean) * rstd;
              if constexpr (OP == OP_RES_LAYERNORM) {
                // the reference's fused module casts the normalised value to the input dtype
                // before the affine part and runs that in the parameters' dtype
                // (residual_layernorm.py:73); plain LayerNorm (F.layer_norm) rounds once
                o = P::round(o);
                if (p.w) {
                  o *= wv[j];
                  if (p.w_dtype == P::DTYPE) o = P::round(o);
                }
                if (p.b) o += bv[j];
              } else {
                if (p.w) o *= wv[j];
                if (p.b) o += bv[j];
              }
              f[j] = o;
            }
            emit(i, col, P::pack(f));
          }
        }
      } else {
        // round(x * rstd) to the activation dtype, then times w, then round again: the order
        // of the reference's PyTorch backend.
        bool done = false;
        if constexpr (VEC == 8) {
          if (p.w_dtype == P::DTYPE) {
            // Same 16-bit dtype on both sides: x*rstd as a packed fp32x2 multiply, one packed
            // convert, and the second product as one packed 16-bit multiply (single rounding:
            // the exact product of two 16-bit values fits in fp32).
            done = true;
            const float2 r2 = make_float2(rstd, rstd);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
              const int v = i * TPR + t;
              if (live(i)) {
                const int64_t col = static_cast<int64_t>(v) * VEC;
                const uint4 wraw = ld_cached16(reinterpret_cast<const T*>(p.w) + col);
                const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wraw);
                float2 f2[4];
                if constexpr (KEEP_F32) {
#pragma unroll
                  for (int j = 0; j < 4; ++j) f2[j] = xf[i][j];
                } else {
                  // the int8 forms run with the ALU pipe as their busiest: unpack on the FMA pipe
                  if constexpr (NORM_TO_REGS && TRX_QUANT_FMA_UNPACK != 0) P::unpack2_fma(raw[i], f2);
                  else P::unpack2(raw[i], f2);
                }
                uint32_t yu[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 n = mul2(f2[j], r2);
                  yu[j] = mul_packed16<T>(wu[j], P::pack2(n.x, n.y));
                  if constexpr (OP == OP_RMSNORM_ACT) {
                    // the activation sees the product rounded to the storage dtype
                    const float2 a = P::cvt2(yu[j]);
                    yu[j] = P::pack2(row_act<true>(a.x, rp.act), row_act<true>(a.y, rp.act));
                  }
                }
                emit(i, col, make_uint4(yu[0], yu[1], yu[2], yu[3]));
              }
            }
          }
        }
        if (!done) {
#pragma unroll
          for (int i = 0; i < VPT; ++i) {
            const int v = i * TPR + t;
            if (live(i)) {
              float f[VEC];
              if constexpr (KEEP_F32) {
                // residual forms of a 16-bit row: the fp32 sum x + r lives only in xf
#pragma unroll
                for (int j = 0; j < VEC / 2; ++j) {
                  f[2 * j] = xf[i][j].x;
                  f[2 * j + 1] = xf[i][j].y;
                }
              } else {
                P::unpack(raw[i], f);
              }
              const int64_t col = static_cast<int64_t>(v) * VEC;
              float wv[VEC];
              load_param_vec<VEC>(p.w, p.w_dtype, col, wv);
#pragma unroll
              for (int j = 0; j < VEC; ++j) {
                f[j] = __fmul_rn(wv[j], P::round(__fmul_rn(f[j], rstd)));
                // weight of another dtype: the reference's product is promoted to fp32 and the
                // activation sees it unrounded
                if constexpr (OP == OP_RMSNORM_ACT) f[j] = row_act<(VEC == 8)>(f[j], rp.act);
              }
              emit(i, col, P::pack(f));
            }
          }
        }
      }
    }

    // ---- 4. quantise the (possibly normalised) row held in registers ----------------
    if constexpr (HAS_QUANT) {
      typename P::AbsAcc acc = P::absacc_init();
#pragma unroll
      for (int i = 0; i < VPT; ++i) P::absacc(raw[i], acc);  // padding vectors are zero
      const float am = row_reduce<TPR, true>(P::absacc_final(acc), red, sel);
      const QuantRow qr = make_quant_row(am);
      if (row_ok && t == 0) p.scales[row] = qr.scale;
      int8_t* crow = p.codes + (FULL || row_ok ? row : 0) * p.codes_stride;
      auto encode_row = [&](auto mode_tag) {
        constexpr int MODE = decltype(mode_tag)::value;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int v = i * TPR + t;
          float2 f2[VEC / 2];
          if constexpr (TRX_QUANT_FMA_UNPACK != 0) P::unpack2_fma(raw[i], f2);
          else P::unpack2(raw[i], f2);
          if (live(i)) {
            uint32_t yb[VEC];
            bool exact_path = (MODE != 1);
            if constexpr (MODE == 1) {
              uint32_t differ = 0u;
#pragma unroll
              for (int j = 0; j < VEC / 2; ++j)
                quant_pair_bracketed(f2[j], qr, yb[2 * j], yb[2 * j + 1], differ);
              // a quotient too close to a rounding boundary: about one vector in 10^4. Voted so
              // that the branch is uniform and stays a branch.
              exact_path = __any_sync(__activemask(), differ != 0u);
            }
            if (exact_path) {
#pragma unroll
              for (int j = 0; j < VEC / 2; ++j)
                quant_pair<MODE, (VEC == 8)>(f2[j], qr, yb[2 * j], yb[2 * j + 1]);
            }
            int8_t* dst = crow + static_cast<int64_t>(v) * VEC;
            if constexpr (VEC == 8) {
              st_stream8(dst, make_uint2(pack_low_bytes(yb[0], yb[1], yb[2], yb[3]),
                                         pack_low_bytes(yb[4], yb[5], yb[6], yb[7])));
            } else {
              st_stream4(dst, pack_low_bytes(yb[0], yb[1], yb[2], yb[3]));
            }
          }
        }
      };
      // the mode is uniform over the row: one branch per row, not one per value
      if (qr.mode == 1) encode_row(std::integral_constant<int, 1>{});
      else if (qr.mode == 2) encode_row(std::integral_constant<int, 2>{});
      else encode_row(std::integral_constant<int, 0>{});
    }
  }
}

// Scalar multi-pass fallback: one CTA per row, any C, any alignment. The row is
// re-read from global memory (L2-resident after the first pass).
template <int OP, typename T>
__global__ void __launch_bounds__(256) row_kernel_generic(const RowParamsBase p, const ResArg<OP> rp) {
  using P = Pack<T>;
  __shared__ __align__(16) float red[2][32];
  int sel = 0;
  constexpr bool HAS_QUANT = op_has_quant(OP);
  const float inv_C = __fdiv_rn(1.0f, static_cast<float>(p.C));
  for (int64_t row = blockIdx.x; row < p.R; row += gridDim.x) {
    const T* xrow = reinterpret_cast<const T*>(p.x) + row * p.x_stride;
    float mean = 0.0f, rstd = 1.0f;
    const T* rrow = nullptr;
    T* srow = nullptr;
    if constexpr (op_has_res(OP)) {
      rrow = reinterpret_cast<const T*>(rp.res) + row * rp.res_stride;
      if (rp.sum_out) srow = reinterpret_cast<T*>(rp.sum_out) + row * rp.sum_stride;
    }
    auto xval = [&](int64_t c) -> float {  // x, or the fp32 sum x + residual
      const float f = P::load1(xrow + c);
      return rrow ? f + P::load1(rrow + c) : f;
    };
    if constexpr (op_is_rms(OP)) {
      float ss = 0.0f;
      for (int64_t c = threadIdx.x; c < p.C; c += 256) {
        const float f = xval(c);
        ss = fmaf(f, f, ss);
        if (srow) P::store1(srow + c, f);
      }
      ss = row_reduce<256, false>(ss, red, sel);
      rstd = rsqrt_approx(fmaf(ss, inv_C, p.eps));
    } else if constexpr (op_is_ln(OP)) {
      float s = 0.0f;
      for (int64_t c = threadIdx.x; c < p.C; c += 256) {
        const float f = xval(c);
        s += f;
        if (srow) P::store1(srow + c, f);
      }
      s = row_reduce<256, false>(s, red, sel);
      mean = s * inv_C;
      float cs = 0.0f;
      for (int64_t c = threadIdx.x; c < p.C; c += 256) {
        const float d = xval(c) - mean;
        cs = fmaf(d, d, cs);
      }
      cs = row_reduce<256, false>(cs, red, sel);
      rstd = rsqrt_approx(fmaf(cs, inv_C, p.eps));
    }
    if (OP != OP_QUANT && threadIdx.x == 0) {
      if (p.rstd) p.rstd[row] = rstd;
      if (op_is_ln(OP) && p.mean) p.mean[row] = mean;
    }
    auto normed = [&](int64_t c) -> float {
      const float f = xval(c);
      if constexpr (OP == OP_LAYERNORM) {
        float o = (f - mean) * rstd;
        if (p.w) o *= load_param1(p.w, p.w_dtype, c);
        if (p.b) o += load_param1(p.b, p.w_dtype, c);
        return P::round(o);
      } else if constexpr (OP == OP_RES_LAYERNORM) {
        float o = P::round((f - mean) * rstd);  // rounding order of residual_layernorm.py:73
        if (p.w) {
          o *= load_param1(p.w, p.w_dtype, c);
          if (p.w_dtype == P::DTYPE) o = P::round(o);
        }
        if (p.b) o += load_param1(p.b, p.w_dtype, c);
        return P::round(o);
      } else if constexpr (OP == OP_QUANT) {
        return f;
      } else if constexpr (OP == OP_RMSNORM_ACT) {
        // same-dtype weight: the product is rounded before the activation; any other weight
        // dtype promotes it to fp32 (trinix/layers/fused/rmsnorm_activation.py:77)
        float n = __fmul_rn(load_param1(p.w, p.w_dtype, c), P::round(__fmul_rn(f, rstd)));
        if (p.w_dtype == P::DTYPE) n = P::round(n);
        return P::round(row_act<(P::VEC == 8)>(n, rp.act));
      } else {
        return P::round(
            __fmul_rn(load_param1(p.w, p.w_dtype, c), P::round(__fmul_rn(f, rstd))));
      }
    };
    if constexpr (!HAS_QUANT) {
      T* yrow = reinterpret_cast<T*>(p.y) + row * p.y_stride;
      for (int64_t c = threadIdx.x; c < p.C; c += 256) P::store1(yrow + c, normed(c));
    } else {
      float am = 0.0f;
      for (int64_t c = threadIdx.x; c < p.C; c += 256) am = fmaxf(am, fabsf(normed(c)));
      am = row_reduce<256, true>(am, red, sel);
      const float scale = __fdiv_rn(am, 127.0f);
      if (threadIdx.x == 0) p.scales[row] = scale;
      int8_t* crow = p.codes + row * p.codes_stride;
      for (int64_t c = threadIdx.x; c < p.C; c += 256)
        crow[c] = static_cast<int8_t>(quant_code(normed(c), scale));
    }
  }
}

// ----------------------------------------------------------------------------
// Host-side dispatch
// ----------------------------------------------------------------------------
template <int OP, typename T, int TPR, int VPT, bool FULL>
static int launch_cfg_full(const RowParams& p, cudaStream_t stream) {
  constexpr int BLOCK = TPR > 32 ? TPR : 256;
  constexpr int ROWS_PER_CTA = BLOCK / TPR;
  // The occupancy answer is cached per device ordinal. Host threads that race on the first
  // call each compute the same value and store it atomically.
  static std::atomic<int> blocks_per_sm_of[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return TRX_ERR_CUDA;
  const bool cacheable = dev >= 0 && dev < 64;
  int blocks_per_sm = cacheable ? blocks_per_sm_of[dev].load(std::memory_order_acquire) : 0;
  if (blocks_per_sm == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, row_kernel<OP, T, TPR, VPT, FULL>, BLOCK,
                                                      0) != cudaSuccess ||
        n <= 0)
      n = 1;
    blocks_per_sm = n;
    if (cacheable) blocks_per_sm_of[dev].store(n, std::memory_order_release);
  }
  const int64_t need = (p.R + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
  const int64_t cap = static_cast<int64_t>(sm_count_of_current_device()) * blocks_per_sm;
  // Grid = several resident waves, each CTA striding over a few rows. Exactly one wave of
  // persistent CTAs measured 5-12 % slower on every op (the hardware scheduler evens out SMs
  // that run behind); the two ops without an int8 encoder or a second pass do best with one
  // CTA per row.
#ifndef TRX_ROW_GRID_MULT
#define TRX_ROW_GRID_MULT ((OP == OP_RMSNORM || OP == OP_RES_RMSNORM) ? 64 : 8)
#endif
  const int64_t want = cap * TRX_ROW_GRID_MULT;
  const unsigned grid = static_cast<unsigned>(need < want ? need : want);
  row_kernel<OP, T, TPR, VPT, FULL><<<grid, BLOCK, 0, stream>>>(static_cast<const RowParamsBase&>(p), res_arg<OP>(p));
  return cudaGetLastError() == cudaSuccess ? TRX_OK : TRX_ERR_CUDA;
}

template <int OP, typename T, int TPR, int VPT>
static int launch_cfg(const RowParams& p, cudaStream_t stream) {
  constexpr int ROWS_PER_CTA = (TPR > 32 ? TPR : 256) / TPR;
  if constexpr (VPT <= 4 || (TPR == 64 && VPT == 8)) {  // built where that exact width matters
    if (p.C / Pack<T>::VEC == TPR * VPT && p.R % ROWS_PER_CTA == 0)
      return launch_cfg_full<OP, T, TPR, VPT, true>(p, stream);
  }
  return launch_cfg_full<OP, T, TPR, VPT, false>(p, stream);
}

template <int OP, typename T>
static int launch_row(const RowParams& p, cudaStream_t stream) {
  constexpr int VEC = Pack<T>::VEC;
  if (p.R == 0) return TRX_OK;
  constexpr bool HAS_QUANT = op_has_quant(OP);
  constexpr bool WRITES_Y = (OP == OP_RMSNORM || OP == OP_LAYERNORM || OP == OP_RES_RMSNORM ||
                             OP == OP_RMSNORM_ACT || OP == OP_RES_LAYERNORM);
  bool vec_ok = (p.C % VEC == 0) && aligned_to(p.x, 16) && (p.x_stride % VEC == 0);
  if (WRITES_Y) vec_ok = vec_ok && aligned_to(p.y, 16) && (p.y_stride % VEC == 0);
  if (HAS_QUANT) vec_ok = vec_ok && aligned_to(p.codes, VEC) && (p.codes_stride % VEC == 0);
  if (p.w) vec_ok = vec_ok && aligned_to(p.w, 16);
  if (p.b) vec_ok = vec_ok && aligned_to(p.b, 16);
  const int64_t nvec = p.C / VEC;
  if constexpr (op_has_res(OP)) {
    vec_ok = vec_ok && aligned_to(p.rp.res, 16) && (p.rp.res_stride % VEC == 0);
    if (p.rp.sum_out) vec_ok = vec_ok && aligned_to(p.rp.sum_out, 16) && (p.rp.sum_stride % VEC == 0);
    // the fp32 sum has to stay on chip: fp32 rows hold it in place, 16-bit rows only in the
    // configurations that keep fp32 copies (at most 4 vectors per thread)
    if (VEC == 8 && nvec > 4096) vec_ok = false;
  }
  if (vec_ok && nvec <= 16384) {
    if (nvec <= 32) return launch_cfg<OP, T, 32, 1>(p, stream);
    if (nvec <= 64) return launch_cfg<OP, T, 32, 2>(p, stream);
    if (nvec <= 128) return launch_cfg<OP, T, 32, 4>(p, stream);
    if (nvec <= 256) return launch_cfg<OP, T, TRX_ROW256_TPR, TRX_ROW256_VPT>(p, stream);
    if (nvec <= 512) {
      // Measured on 32768 x 4096 bf16, per family: two input streams per row (residual forms)
      // 256 threads x 2 vectors (93-95 % of the copy rate against 86 % for 128 x 4); the int8
      // encoders 64 x 8 at 10 CTAs per SM (+2-5 % over 128 x 4); LayerNorm 128 x 4. RMSNorm
      // follows RMSNorm -> int8 (which costs it 1 %): the two must sum the squares in the same
      // order to stay equal bit for bit.
      if constexpr (op_has_res(OP)) return launch_cfg<OP, T, 256, 2>(p, stream);
      else if constexpr (op_has_quant(OP) || OP == OP_RMSNORM) return launch_cfg<OP, T, 64, 8>(p, stream);
      else return launch_cfg<OP, T, 128, 4>(p, stream);
    }
    if (nvec <= 1024) return launch_cfg<OP, T, 256, 4>(p, stream);
    if (nvec <= 2048) return launch_cfg<OP, T, 512, 4>(p, stream);
    if (nvec <= 4096) return launch_cfg<OP, T, 1024, 4>(p, stream);
    if (nvec <= 8192) return launch_cfg<OP, T, 1024, 8>(p, stream);
    return launch_cfg<OP, T, 1024, 16>(p, stream);
  }
  const int64_t cap = static_cast<int64_t>(sm_count_of_current_device()) * 8;
  const unsigned grid = static_cast<unsigned>(p.R < cap ? p.R : cap);
  row_kernel_generic<OP, T><<<grid, 256, 0, stream>>>(static_cast<const RowParamsBase&>(p), res_arg<OP>(p));
  return cudaGetLastError() == cudaSuccess ? TRX_OK : TRX_ERR_CUDA;
}

template <int OP>
static int launch_row_dtype(const RowParams& p, int x_dtype, cudaStream_t stream) {
  switch (x_dtype) {
    case TRX_F32: return launch_row<OP, float>(p, stream);
    case TRX_F16: return launch_row<OP, __half>(p, stream);
    case TRX_BF16: return launch_row<OP, __nv_bfloat16>(p, stream);
    default: return TRX_ERR_DTYPE;
  }
}

static bool dtype_ok(int d) { return d == TRX_F32 || d == TRX_F16 || d == TRX_BF16; }

}  // namespace trx

using namespace trx;

extern "C" int trx_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd_or_null, int64_t R,
                               int64_t C, int64_t x_row_stride, int64_t y_row_stride, float eps,
                               int x_dtype, int w_dtype, void* stream) {
  if (!dtype_ok(x_dtype) || !dtype_ok(w_dtype)) return TRX_ERR_DTYPE;
  if (R < 0 || C <= 0) return TRX_ERR_SHAPE;
  if (R == 0) return TRX_OK;
  if (!x || !w || !y) return TRX_ERR_NULL_POINTER;
  if (x_row_stride < C || y_row_stride < C) return TRX_ERR_STRIDE;
  RowParams p{};
  p.x = x; p.w = w; p.y = y; p.rstd = rstd_or_null;
  p.R = R; p.C = C; p.x_stride = x_row_stride; p.y_stride = y_row_stride;
  p.eps = eps; p.w_dtype = w_dtype;
  return launch_row_dtype<OP_RMSNORM>(p, x_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int trx_rmsnorm_act_fwd(const void* x, const void* w, void* y, int64_t R, int64_t C,
                                   int64_t x_row_stride, int64_t y_row_stride, float eps, int act,
                                   int x_dtype, int w_dtype, void* stream) {
  if (!dtype_ok(x_dtype) || !dtype_ok(w_dtype)) return TRX_ERR_DTYPE;
  if (act != TRX_ACT_MISH && act != TRX_ACT_QUICKGELU && act != TRX_ACT_SQUARED_RELU)
    return TRX_ERR_UNSUPPORTED;
  if (R < 0 || C <= 0) return TRX_ERR_SHAPE;
  if (R == 0) return TRX_OK;
  if (!x || !w || !y) return TRX_ERR_NULL_POINTER;
  if (x_row_stride < C || y_row_stride < C) return TRX_ERR_STRIDE;
  RowParams p{};
  p.x = x; p.w = w; p.y = y;
  p.R = R; p.C = C; p.x_stride = x_row_stride; p.y_stride = y_row_stride;
  p.eps = eps; p.w_dtype = w_dtype;
  p.ap.act = act;
  return launch_row_dtype<OP_RMSNORM_ACT>(p, x_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int trx_layernorm_fwd(const void* x, const void* w_or_null, const void* b_or_null,
                                 void* y, float* mean_or_null, float* rstd_or_null, int64_t R,
                                 int64_t C, int64_t x_row_stride, int64_t y_row_stride, float eps,
                                 int x_dtype, int wb_dtype, void* stream) {
  if (!dtype_ok(x_dtype) || !dtype_ok(wb_dtype)) return TRX_ERR_DTYPE;
  if (R < 0 || C <= 0) return TRX_ERR_SHAPE;
  if (R == 0) return TRX_OK;
  if (!x || !y) return TRX_ERR_NULL_POINTER;
  if (x_row_stride < C || y_row_stride < C) return TRX_ERR_STRIDE;
  RowParams p{};
  p.x = x; p.w = w_or_null; p.b = b_or_null; p.y = y; p.mean = mean_or_null;
  p.rstd = rstd_or_null;
  p.R = R; p.C = C; p.x_stride = x_row_stride; p.y_stride = y_row_stride;
  p.eps = eps; p.w_dtype = wb_dtype;
  return launch_row_dtype<OP_LAYERNORM>(p, x_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int trx_quant_rowwise_i8(const void* x, int8_t* codes, float* scales, int64_t R,
                                    int64_t C, int64_t x_row_stride, int64_t codes_row_stride,
                                    int x_dtype, void* stream) {
  if (!dtype_ok(x_dtype)) return TRX_ERR_DTYPE;
  if (R < 0 || C <= 0) return TRX_ERR_SHAPE;
  if (R == 0) return TRX_OK;
  if (!x || !codes || !scales) return TRX_ERR_NULL_POINTER;
  if (x_row_stride < C || codes_row_stride < C) return TRX_ERR_STRIDE;
  RowParams p{};
  p.x = x; p.codes = codes; p.scales = scales;
  p.R = R; p.C = C; p.x_stride = x_row_stride; p.codes_stride = codes_row_stride;
  return launch_row_dtype<OP_QUANT>(p, x_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int trx_rmsnorm_quant_i8(const void* x, const void* w, int8_t* codes, float* scales,
                                    int64_t R, int64_t C, int64_t x_row_stride,
                                    int64_t codes_row_stride, float eps, int x_dtype, int w_dtype,
                                    void* stream) {
  if (!dtype_ok(x_dtype) || !dtype_ok(w_dtype)) return TRX_ERR_DTYPE;
  if (R < 0 || C <= 0) return TRX_ERR_SHAPE;
  if (R == 0) return TRX_OK;
  if (!x || !w || !codes || !scales) return TRX_ERR_NULL_POINTER;
  if (x_row_stride < C || codes_row_stride < C) return TRX_ERR_STRIDE;
  RowParams p{};
  p.x = x; p.w = w; p.codes = codes; p.scales = scales;
  p.R = R; p.C = C; p.x_stride = x_row_stride; p.codes_stride = codes_row_stride;
  p.eps = eps; p.w_dtype = w_dtype;
  return launch_row_dtype<OP_RMSNORM_QUANT>(p, x_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int trx_residual_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y,
                                        void* sum_out_or_null, float* rstd_or_null, int64_t R,
                                        int64_t C, int64_t x_row_stride, int64_t res_row_stride,
                                        int64_t y_row_stride, int64_t sum_row_stride, float eps,
                                        int x_dtype, int w_dtype, void* stream) {
  if (!dtype_ok(x_dtype) || !dtype_ok(w_dtype)) return TRX_ERR_DTYPE;
  if (R < 0 || C <= 0) return TRX_ERR_SHAPE;
  if (R == 0) return TRX_OK;
  if (!x || !residual || !w || !y) return TRX_ERR_NULL_POINTER;
  if (x_row_stride < C || res_row_stride < C || y_row_stride < C ||
      (sum_out_or_null && sum_row_stride < C))
    return TRX_ERR_STRIDE;
  RowParams p{};
  p.x = x; p.rp.res = residual; p.rp.sum_out = sum_out_or_null; p.w = w; p.y = y; p.rstd = rstd_or_null;
  p.R = R; p.C = C; p.x_stride = x_row_stride; p.rp.res_stride = res_row_stride;
  p.y_stride = y_row_stride; p.rp.sum_stride = sum_row_stride;
  p.eps = eps; p.w_dtype = w_dtype;
  return launch_row_dtype<OP_RES_RMSNORM>(p, x_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int trx_residual_layernorm_fwd(const void* x, const void* residual,
                                          const void* w_or_null, const void* b_or_null, void* y,
                                          void* sum_out_or_null, float* mean_or_null,
                                          float* rstd_or_null, int64_t R, int64_t C,
                                          int64_t x_row_stride, int64_t res_row_stride,
                                          int64_t y_row_stride, int64_t sum_row_stride, float eps,
                                          int x_dtype, int w_dtype, void* stream) {
  if (!dtype_ok(x_dtype) || !dtype_ok(w_dtype)) return TRX_ERR_DTYPE;
  if (R < 0 || C <= 0) return TRX_ERR_SHAPE;
  if (R == 0) return TRX_OK;
  if (!x || !residual || !y) return TRX_ERR_NULL_POINTER;
  if (x_row_stride < C || res_row_stride < C || y_row_stride < C ||
      (sum_out_or_null && sum_row_stride < C))
    return TRX_ERR_STRIDE;
  RowParams p{};
  p.x = x; p.rp.res = residual; p.rp.sum_out = sum_out_or_null; p.w = w_or_null; p.b = b_or_null;
  p.y = y; p.mean = mean_or_null; p.rstd = rstd_or_null;
  p.R = R; p.C = C; p.x_stride = x_row_stride; p.rp.res_stride = res_row_stride;
  p.y_stride = y_row_stride; p.rp.sum_stride = sum_row_stride;
  p.eps = eps; p.w_dtype = w_dtype;
  return launch_row_dtype<OP_RES_LAYERNORM>(p, x_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int trx_residual_rmsnorm_quant_i8(const void* x, const void* residual, const void* w,
                                             int8_t* codes, float* scales, void* sum_out_or_null,
                                             int64_t R, int64_t C, int64_t x_row_stride,
                                             int64_t res_row_stride, int64_t codes_row_stride,
                                             int64_t sum_row_stride, float eps, int x_dtype,
                                             int w_dtype, void* stream) {
  if (!dtype_ok(x_dtype) || !dtype_ok(w_dtype)) return TRX_ERR_DTYPE;
  if (R < 0 || C <= 0) return TRX_ERR_SHAPE;
  if (R == 0) return TRX_OK;
  if (!x || !residual || !w || !codes || !scales) return TRX_ERR_NULL_POINTER;
  if (x_row_stride < C || res_row_stride < C || codes_row_stride < C ||
      (sum_out_or_null && sum_row_stride < C))
    return TRX_ERR_STRIDE;
  RowParams p{};
  p.x = x; p.rp.res = residual; p.rp.sum_out = sum_out_or_null; p.w = w; p.codes = codes;
  p.scales = scales;
  p.R = R; p.C = C; p.x_stride = x_row_stride; p.rp.res_stride = res_row_stride;
  p.codes_stride = codes_row_stride; p.rp.sum_stride = sum_row_stride;
  p.eps = eps; p.w_dtype = w_dtype;
  return launch_row_dtype<OP_RES_RMSNORM_QUANT>(p, x_dtype, static_cast<cudaStream_t>(stream));
}
