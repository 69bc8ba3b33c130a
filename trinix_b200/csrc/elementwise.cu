// Streaming elementwise kernels: gated linear units, rotary embedding (q and k
// in one launch) and per-row int8 dequantisation.
//
// All three are pure HBM streams. Each thread moves 16-byte vectors with
// streaming loads/stores; GLU keeps four rows (eight loads) in flight per thread, RoPE the
// two halves of four head vectors, the dequantiser one light row block per thread on a
// very large grid. Grids are 2-D (column-vector block, row block) so no thread ever
// divides to find its row. Shapes or pointers that do not fit the vector path take a
// scalar kernel.
#include "common.cuh"

namespace trx {

// ----------------------------------------------------------------------------
// GLU
// ----------------------------------------------------------------------------
// exp(x). 16-bit outputs take the hardware exp2 on a pre-scaled argument (relative error about
// 2^-22 + |x| * 2^-24, two orders below a bf16 / fp16 rounding step); fp32 outputs keep expf.
template <bool FAST>
__device__ __forceinline__ float glu_exp(float x) {
  if constexpr (FAST) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x * 1.4426950408889634f));
    return r;
  } else {
    return expf(x);
  }
}

template <int ACT, bool FAST>
__device__ __forceinline__ float glu_act(float g) {
  if constexpr (ACT == TRX_GLU_SWIGLU) {
    // silu(g) = g * 1/(1 + exp(-g)). The reciprocal is the hardware approximation (about
    // 1 ulp), far below the storage dtype's rounding step. exp overflow (g -> -inf) gives
    // g * 0 = -0.
    return g * __fdividef(1.0f, 1.0f + glu_exp<FAST>(-g));
  } else if constexpr (ACT == TRX_GLU_GEGLU_TANH) {
    const float kBeta = 0.7978845608028654f;  // sqrt(2/pi)
    const float kKappa = 0.044715f;
    const float inner = kBeta * (g + kKappa * g * g * g);
    // 0.5 * (1 + tanh(u)) == sigmoid(2u): one exponential and one reciprocal instead of a
    // tanhf call, exact at both ends (exp overflow gives g * 0, underflow gives g), and without
    // the cancellation of 1 + tanh(u) for negative g.
    return g * __fdividef(1.0f, 1.0f + glu_exp<FAST>(-2.0f * inner));
  } else {
    return fmaxf(g, 0.0f);
  }
}

constexpr int GLU_ROWS_PER_THREAD = 4;
constexpr int GLU_THREADS = 128;

// y = round(up * round(act(gate))): the activation is rounded to the storage dtype
// before the product, as the reference's PyTorch backend does (x1 * F.silu(x2)).
template <int ACT, typename T>
__global__ void __launch_bounds__(GLU_THREADS)
    glu_kernel(const T* __restrict__ up, const T* __restrict__ gate, T* __restrict__ y, int64_t R,
               int nvec, int64_t up_stride, int64_t gate_stride, int64_t y_stride) {
  using P = Pack<T>;
  constexpr int VEC = P::VEC;
  const int v = blockIdx.x * GLU_THREADS + threadIdx.x;
  if (v >= nvec) return;
  const int64_t col = static_cast<int64_t>(v) * VEC;
  for (int64_t r0 = static_cast<int64_t>(blockIdx.y) * GLU_ROWS_PER_THREAD; r0 < R;
       r0 += static_cast<int64_t>(gridDim.y) * GLU_ROWS_PER_THREAD) {
    uint4 u[GLU_ROWS_PER_THREAD], g[GLU_ROWS_PER_THREAD];
#pragma unroll
    for (int i = 0; i < GLU_ROWS_PER_THREAD; ++i) {
      const int64_t r = r0 + i;
      if (r < R) {
        u[i] = ld_stream16(up + r * up_stride + col);
        g[i] = ld_stream16(gate + r * gate_stride + col);
      }
    }
#pragma unroll
    for (int i = 0; i < GLU_ROWS_PER_THREAD; ++i) {
      const int64_t r = r0 + i;
      if (r < R) {
        float uf[VEC], gf[VEC];
        P::unpack(u[i], uf);
        P::unpack(g[i], gf);
#pragma unroll
        for (int j = 0; j < VEC; ++j) uf[j] = __fmul_rn(uf[j], P::round(glu_act<ACT, (VEC == 8)>(gf[j])));
        st_stream16(y + r * y_stride + col, P::pack(uf));
      }
    }
  }
}

template <int ACT, typename T>
__global__ void __launch_bounds__(256)
    glu_kernel_scalar(const T* __restrict__ up, const T* __restrict__ gate, T* __restrict__ y,
                      int64_t R, int64_t H, int64_t up_stride, int64_t gate_stride,
                      int64_t y_stride) {
  using P = Pack<T>;
  for (int64_t r = blockIdx.x; r < R; r += gridDim.x)
    for (int64_t c = threadIdx.x; c < H; c += 256) {
      const float a = P::round(glu_act<ACT, (P::VEC == 8)>(P::load1(gate + r * gate_stride + c)));
      P::store1(y + r * y_stride + c, __fmul_rn(P::load1(up + r * up_stride + c), a));
    }
}

template <int ACT, typename T>
static int launch_glu(const void* up, const void* gate, void* y, int64_t R, int64_t H,
                      int64_t us, int64_t gs, int64_t ys, cudaStream_t stream) {
  constexpr int VEC = Pack<T>::VEC;
  const bool vec_ok = (H % VEC == 0) && aligned_to(up, 16) && aligned_to(gate, 16) &&
                      aligned_to(y, 16) && us % VEC == 0 && gs % VEC == 0 && ys % VEC == 0 &&
                      H / VEC < (1ll << 31);
  if (vec_ok) {
    const int nvec = static_cast<int>(H / VEC);
    const int64_t row_blocks = (R + GLU_ROWS_PER_THREAD - 1) / GLU_ROWS_PER_THREAD;
    dim3 grid((nvec + GLU_THREADS - 1) / GLU_THREADS,
              static_cast<unsigned>(row_blocks < 65535 ? row_blocks : 65535));
    glu_kernel<ACT, T><<<grid, GLU_THREADS, 0, stream>>>(
        static_cast<const T*>(up), static_cast<const T*>(gate), static_cast<T*>(y), R, nvec, us,
        gs, ys);
  } else {
    const int64_t cap = static_cast<int64_t>(sm_count_of_current_device()) * 8;
    const unsigned grid = static_cast<unsigned>(R < cap ? R : cap);
    glu_kernel_scalar<ACT, T><<<grid, 256, 0, stream>>>(
        static_cast<const T*>(up), static_cast<const T*>(gate), static_cast<T*>(y), R, H, us, gs,
        ys);
  }
  return cudaGetLastError() == cudaSuccess ? TRX_OK : TRX_ERR_CUDA;
}

template <typename T>
static int launch_glu_act(int act, const void* up, const void* gate, void* y, int64_t R, int64_t H,
                          int64_t us, int64_t gs, int64_t ys, cudaStream_t stream) {
  switch (act) {
    case TRX_GLU_SWIGLU: return launch_glu<TRX_GLU_SWIGLU, T>(up, gate, y, R, H, us, gs, ys, stream);
    case TRX_GLU_GEGLU_TANH:
      return launch_glu<TRX_GLU_GEGLU_TANH, T>(up, gate, y, R, H, us, gs, ys, stream);
    case TRX_GLU_REGLU: return launch_glu<TRX_GLU_REGLU, T>(up, gate, y, R, H, us, gs, ys, stream);
    default: return TRX_ERR_UNSUPPORTED;
  }
}

// ----------------------------------------------------------------------------
// RoPE
// ----------------------------------------------------------------------------
struct RopeParams {
  const void* q;
  const void* k;
  void* qo;
  void* ko;
  const void* cos_t;
  const void* sin_t;
  int64_t S;
  int Hq, Hk, D;
  int64_t qs[3], ks[3], qos[3], kos[3];  // (batch, seq, head) strides in elements
  int64_t table_stride;                  // elements
  int inverse;
};

// TABLE_F32: tables are fp32 and all arithmetic is fp32 with one final rounding
// (x * cos promotes to fp32 in the reference's PyTorch path). Otherwise tables have
// the activation dtype and every product and the sum are rounded to it, again
// matching that path op for op. Multiplies and adds are kept separate (no FMA
// contraction) so both modes reproduce its results exactly.
//
// Work split: a thread owns one (token, 8-column slice of the half dim) and walks over all
// heads of q and then k, four heads per step, so the slice's cos/sin values are loaded once
// and eight independent 16-byte loads are in flight per thread. Neighbouring threads cover
// neighbouring slices of the same token, i.e. whole 128-byte lines of each head vector.
constexpr int ROPE_HEADS_PER_STEP = 4;

template <typename T, bool TABLE_F32>
__global__ void __launch_bounds__(128) rope_kernel(const RopeParams p, int vec_per_head,
                                                   int64_t tokens, int heads_per_cta) {
  using P = Pack<T>;
  constexpr int VEC = P::VEC;
  const int half = p.D / 2;
  const int tok_per_cta = blockDim.x / vec_per_head;
  const int64_t token = static_cast<int64_t>(blockIdx.x) * tok_per_cta + threadIdx.x / vec_per_head;
  if (token >= tokens) return;
  const int j = (threadIdx.x % vec_per_head) * VEC;
  const int64_t b = token / p.S;
  const int64_t s = token - b * p.S;

  float c[VEC], sn[VEC];
  if constexpr (TABLE_F32) {
    load_param_vec<VEC>(p.cos_t, TRX_F32, s * p.table_stride + j, c);
    load_param_vec<VEC>(p.sin_t, TRX_F32, s * p.table_stride + j, sn);
  } else {
    load_param_vec<VEC>(p.cos_t, P::DTYPE, s * p.table_stride + j, c);
    load_param_vec<VEC>(p.sin_t, P::DTYPE, s * p.table_stride + j, sn);
  }
  if (p.inverse) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) sn[e] = -sn[e];
  }

  // blockIdx.y selects a chunk of the q + k heads: a thread reuses its table slice over one
  // chunk only, which multiplies the CTAs (a token-only grid was under one resident wave)
  const int H_all = p.Hq + p.Hk;
  const int h_begin = blockIdx.y * heads_per_cta;
  const int H = min(H_all, h_begin + heads_per_cta);
  for (int h0 = h_begin; h0 < H; h0 += ROPE_HEADS_PER_STEP) {
    uint4 r1[ROPE_HEADS_PER_STEP], r2[ROPE_HEADS_PER_STEP];
    T* dst[ROPE_HEADS_PER_STEP];
#pragma unroll
    for (int u = 0; u < ROPE_HEADS_PER_STEP; ++u) {
      const int h_all = h0 + u;
      if (h_all < H) {
        const bool is_q = h_all < p.Hq;
        const int h = is_q ? h_all : h_all - p.Hq;
        const int64_t* st = is_q ? p.qs : p.ks;
        const int64_t* ost = is_q ? p.qos : p.kos;
        const T* src = reinterpret_cast<const T*>(is_q ? p.q : p.k) + b * st[0] + s * st[1] +
                       static_cast<int64_t>(h) * st[2];
        dst[u] = reinterpret_cast<T*>(is_q ? p.qo : p.ko) + b * ost[0] + s * ost[1] +
                 static_cast<int64_t>(h) * ost[2];
        r1[u] = ld_stream16(src + j);
        r2[u] = ld_stream16(src + half + j);
      }
    }
#pragma unroll
    for (int u = 0; u < ROPE_HEADS_PER_STEP; ++u) {
      if (h0 + u < H) {
        float x1[VEC], x2[VEC], o1[VEC], o2[VEC];
        P::unpack(r1[u], x1);
        P::unpack(r2[u], x2);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          if constexpr (TABLE_F32) {
            o1[e] = __fadd_rn(__fmul_rn(x1[e], c[e]), __fmul_rn(-x2[e], sn[e]));
            o2[e] = __fadd_rn(__fmul_rn(x2[e], c[e]), __fmul_rn(x1[e], sn[e]));
          } else {
            o1[e] = __fadd_rn(P::round(__fmul_rn(x1[e], c[e])), P::round(__fmul_rn(-x2[e], sn[e])));
            o2[e] = __fadd_rn(P::round(__fmul_rn(x2[e], c[e])), P::round(__fmul_rn(x1[e], sn[e])));
          }
        }
        st_stream16(dst[u] + j, P::pack(o1));
        st_stream16(dst[u] + half + j, P::pack(o2));
      }
    }
  }
}

template <typename T, bool TABLE_F32>
__global__ void __launch_bounds__(256) rope_kernel_scalar(const RopeParams p) {
  using P = Pack<T>;
  const int half = p.D / 2;
  const int items = (p.Hq + p.Hk) * half;
  const int64_t token = blockIdx.x;
  const int64_t b = token / p.S;
  const int64_t s = token - b * p.S;
  for (int it = threadIdx.x; it < items; it += blockDim.x) {
    const int h_all = it / half;
    const int j = it - h_all * half;
    const bool is_q = h_all < p.Hq;
    const int h = is_q ? h_all : h_all - p.Hq;
    const int64_t* st = is_q ? p.qs : p.ks;
    const int64_t* ost = is_q ? p.qos : p.kos;
    const T* src = reinterpret_cast<const T*>(is_q ? p.q : p.k) + b * st[0] + s * st[1] +
                   static_cast<int64_t>(h) * st[2];
    T* dst = reinterpret_cast<T*>(is_q ? p.qo : p.ko) + b * ost[0] + s * ost[1] +
             static_cast<int64_t>(h) * ost[2];
    const float x1 = P::load1(src + j), x2 = P::load1(src + half + j);
    const int tdt = TABLE_F32 ? TRX_F32 : P::DTYPE;
    const float c = load_param1(p.cos_t, tdt, s * p.table_stride + j);
    float sv = load_param1(p.sin_t, tdt, s * p.table_stride + j);
    if (p.inverse) sv = -sv;
    float o1, o2;
    if constexpr (TABLE_F32) {
      o1 = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(-x2, sv));
      o2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, sv));
    } else {
      o1 = __fadd_rn(P::round(__fmul_rn(x1, c)), P::round(__fmul_rn(-x2, sv)));
      o2 = __fadd_rn(P::round(__fmul_rn(x2, c)), P::round(__fmul_rn(x1, sv)));
    }
    P::store1(dst + j, o1);
    P::store1(dst + half + j, o2);
  }
}

template <typename T, bool TABLE_F32>
static int launch_rope(const RopeParams& p, int64_t B, cudaStream_t stream) {
  constexpr int VEC = Pack<T>::VEC;
  const int half = p.D / 2;
  bool vec_ok = (half % VEC == 0) && aligned_to(p.q, 16) && aligned_to(p.k, 16) &&
                aligned_to(p.qo, 16) && aligned_to(p.ko, 16) && aligned_to(p.cos_t, 16) &&
                aligned_to(p.sin_t, 16) && (p.table_stride % (TABLE_F32 ? 4 : VEC) == 0);
  for (int i = 0; i < 3; ++i)
    vec_ok = vec_ok && p.qs[i] % VEC == 0 && p.ks[i] % VEC == 0 && p.qos[i] % VEC == 0 &&
             p.kos[i] % VEC == 0;
  const int64_t tokens = B * p.S;
  if (tokens == 0) return TRX_OK;
  if (tokens >= (1ll << 31)) return TRX_ERR_SHAPE;
  const int vec_per_head = vec_ok ? half / VEC : 0;
  if (vec_ok && vec_per_head <= 128) {
    const int tok_per_cta = 128 / vec_per_head;
    const int threads = tok_per_cta * vec_per_head;
    const int64_t blocks = (tokens + tok_per_cta - 1) / tok_per_cta;
#ifndef TRX_ROPE_HEADS_PER_CTA
#define TRX_ROPE_HEADS_PER_CTA 8
#endif
    const int heads_per_cta = TRX_ROPE_HEADS_PER_CTA;
    const int head_chunks = (p.Hq + p.Hk + heads_per_cta - 1) / heads_per_cta;
    const dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(head_chunks));
    rope_kernel<T, TABLE_F32><<<grid, threads, 0, stream>>>(p, vec_per_head, tokens, heads_per_cta);
  } else {
    rope_kernel_scalar<T, TABLE_F32><<<static_cast<unsigned>(tokens), 256, 0, stream>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? TRX_OK : TRX_ERR_CUDA;
}

// ----------------------------------------------------------------------------
// Dequantise
// ----------------------------------------------------------------------------
#ifndef TRX_DQ_ROWS
#define TRX_DQ_ROWS 1
#endif
constexpr int DQ_ROWS_PER_THREAD = TRX_DQ_ROWS;
constexpr int DQ_THREADS = 128;

// int8 -> fp32 without a convert instruction: place (code ^ 0x80) in the low mantissa byte
// of 2^23 and subtract 2^23 + 128 (exact).
__device__ __forceinline__ float code_at(uint32_t word_xor80, int byte) {
  const uint32_t bits = __byte_perm(word_xor80, 0x4B000000u, 0x7650 + byte);  // {b, 0, 0, 0x4B}
  return __uint_as_float(bits) - 8388736.0f;
}

// 16 codes per thread per row: one 16-byte load, (16 * sizeof(T)) bytes of stores.
template <typename T>
__global__ void __launch_bounds__(DQ_THREADS)
    dequant_kernel(const int8_t* __restrict__ codes, const float* __restrict__ scales,
                   T* __restrict__ y, int64_t R, int nvec16, int64_t cs, int64_t ys) {
  using P = Pack<T>;
  constexpr int VEC = P::VEC;
  const int v = blockIdx.x * DQ_THREADS + threadIdx.x;
  if (v >= nvec16) return;
  const int64_t col = static_cast<int64_t>(v) * 16;
  for (int64_t r0 = static_cast<int64_t>(blockIdx.y) * DQ_ROWS_PER_THREAD; r0 < R;
       r0 += static_cast<int64_t>(gridDim.y) * DQ_ROWS_PER_THREAD) {
    uint4 c[DQ_ROWS_PER_THREAD];
    float sc[DQ_ROWS_PER_THREAD];
#pragma unroll
    for (int i = 0; i < DQ_ROWS_PER_THREAD; ++i) {
      const int64_t r = r0 + i;
      if (r < R) {
        c[i] = ld_stream16(codes + r * cs + col);
        sc[i] = __ldg(scales + r);
      }
    }
#pragma unroll
    for (int i = 0; i < DQ_ROWS_PER_THREAD; ++i) {
      const int64_t r = r0 + i;
      if (r < R) {
        const uint32_t w[4] = {c[i].x ^ 0x80808080u, c[i].y ^ 0x80808080u, c[i].z ^ 0x80808080u,
                               c[i].w ^ 0x80808080u};
        float f[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) f[j] = __fmul_rn(code_at(w[j >> 2], j & 3), sc[i]);
        T* dst = y + r * ys + col;
#pragma unroll
        for (int k = 0; k < 16 / VEC; ++k) {
          float part[VEC];
#pragma unroll
          for (int j = 0; j < VEC; ++j) part[j] = f[k * VEC + j];
          st_stream16(dst + k * VEC, P::pack(part));
        }
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
    dequant_kernel_scalar(const int8_t* __restrict__ codes, const float* __restrict__ scales,
                          T* __restrict__ y, int64_t R, int64_t C, int64_t cs, int64_t ys) {
  using P = Pack<T>;
  for (int64_t r = blockIdx.x; r < R; r += gridDim.x) {
    const float s = scales[r];
    for (int64_t c = threadIdx.x; c < C; c += 256)
      P::store1(y + r * ys + c, __fmul_rn(static_cast<float>(codes[r * cs + c]), s));
  }
}

template <typename T>
static int launch_dequant(const int8_t* codes, const float* scales, void* y, int64_t R, int64_t C,
                          int64_t cs, int64_t ys, cudaStream_t stream) {
  const bool vec_ok = (C % 16 == 0) && aligned_to(codes, 16) && aligned_to(y, 16) &&
                      cs % 16 == 0 && ys % Pack<T>::VEC == 0 && C / 16 < (1ll << 31);
  if (vec_ok) {
    const int nvec16 = static_cast<int>(C / 16);
    const int64_t row_blocks = (R + DQ_ROWS_PER_THREAD - 1) / DQ_ROWS_PER_THREAD;
    // One row block per CTA up to a grid of some 64 resident waves, beyond which CTAs stride.
    // Measured on [8192, 4096] -> bf16: 17.0 us like this against 22.0 us with 8 rows per thread
    // and a grid of one resident wave: many light CTAs let the hardware scheduler balance the
    // SMs and hide the tail of so short a launch.
#ifndef TRX_DQ_GRID_MULT
#define TRX_DQ_GRID_MULT 64
#endif
    const int64_t col_blocks = (nvec16 + DQ_THREADS - 1) / DQ_THREADS;
    int64_t y_blocks = (static_cast<int64_t>(sm_count_of_current_device()) * 8 * TRX_DQ_GRID_MULT +
                        col_blocks - 1) / col_blocks;
    if (y_blocks > row_blocks) y_blocks = row_blocks;
    if (y_blocks > 65535) y_blocks = 65535;
    if (y_blocks < 1) y_blocks = 1;
    dim3 grid(static_cast<unsigned>(col_blocks), static_cast<unsigned>(y_blocks));
    dequant_kernel<T><<<grid, DQ_THREADS, 0, stream>>>(codes, scales, static_cast<T*>(y), R,
                                                       nvec16, cs, ys);
  } else {
    const int64_t cap = static_cast<int64_t>(sm_count_of_current_device()) * 8;
    const unsigned grid = static_cast<unsigned>(R < cap ? R : cap);
    dequant_kernel_scalar<T><<<grid, 256, 0, stream>>>(codes, scales, static_cast<T*>(y), R, C, cs,
                                                       ys);
  }
  return cudaGetLastError() == cudaSuccess ? TRX_OK : TRX_ERR_CUDA;
}

}  // namespace trx

using namespace trx;

extern "C" int trx_glu_fwd(const void* up, const void* gate, void* y, int64_t R, int64_t H,
                           int64_t up_row_stride, int64_t gate_row_stride, int64_t y_row_stride,
                           int act, int dtype, void* stream) {
  if (act != TRX_GLU_SWIGLU && act != TRX_GLU_GEGLU_TANH && act != TRX_GLU_REGLU)
    return TRX_ERR_UNSUPPORTED;
  if (dtype != TRX_F32 && dtype != TRX_F16 && dtype != TRX_BF16) return TRX_ERR_DTYPE;
  if (R < 0 || H <= 0) return TRX_ERR_SHAPE;
  if (R == 0) return TRX_OK;
  if (!up || !gate || !y) return TRX_ERR_NULL_POINTER;
  if (up_row_stride < H || gate_row_stride < H || y_row_stride < H) return TRX_ERR_STRIDE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case TRX_F32:
      return launch_glu_act<float>(act, up, gate, y, R, H, up_row_stride, gate_row_stride,
                                   y_row_stride, s);
    case TRX_F16:
      return launch_glu_act<__half>(act, up, gate, y, R, H, up_row_stride, gate_row_stride,
                                    y_row_stride, s);
    default:
      return launch_glu_act<__nv_bfloat16>(act, up, gate, y, R, H, up_row_stride, gate_row_stride,
                                           y_row_stride, s);
  }
}

extern "C" int trx_rope_fwd(const void* q, const void* k, const void* cos_table,
                            const void* sin_table, void* q_out, void* k_out, int64_t B, int64_t S,
                            int64_t Hq, int64_t Hk, int64_t D, const int64_t q_strides[3],
                            const int64_t k_strides[3], const int64_t qo_strides[3],
                            const int64_t ko_strides[3], int64_t table_row_stride, int table_dtype,
                            int x_dtype, int inverse, void* stream) {
  if (x_dtype != TRX_F32 && x_dtype != TRX_F16 && x_dtype != TRX_BF16) return TRX_ERR_DTYPE;
  if (table_dtype != TRX_F32 && table_dtype != x_dtype) return TRX_ERR_DTYPE;
  if (B < 0 || S < 0 || Hq < 0 || Hk < 0 || D <= 0 || (D % 2) != 0) return TRX_ERR_SHAPE;
  if (Hq + Hk == 0 || B == 0 || S == 0) return TRX_OK;
  if (Hq > 65535 || Hk > 65535 || D > (1 << 20)) return TRX_ERR_SHAPE;
  if (!cos_table || !sin_table) return TRX_ERR_NULL_POINTER;
  if ((Hq > 0 && (!q || !q_out || !q_strides || !qo_strides)) ||
      (Hk > 0 && (!k || !k_out || !k_strides || !ko_strides)))
    return TRX_ERR_NULL_POINTER;
  if (table_row_stride < D / 2) return TRX_ERR_STRIDE;
  RopeParams p{};
  p.q = q; p.k = k; p.qo = q_out; p.ko = k_out; p.cos_t = cos_table; p.sin_t = sin_table;
  p.S = S; p.Hq = static_cast<int>(Hq); p.Hk = static_cast<int>(Hk); p.D = static_cast<int>(D);
  for (int i = 0; i < 3; ++i) {
    p.qs[i] = Hq > 0 ? q_strides[i] : 0;
    p.qos[i] = Hq > 0 ? qo_strides[i] : 0;
    p.ks[i] = Hk > 0 ? k_strides[i] : 0;
    p.kos[i] = Hk > 0 ? ko_strides[i] : 0;
    if (p.qs[i] < 0 || p.ks[i] < 0 || p.qos[i] < 0 || p.kos[i] < 0) return TRX_ERR_STRIDE;
  }
  p.table_stride = table_row_stride;
  p.inverse = inverse;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool tf32 = (table_dtype == TRX_F32);
  switch (x_dtype) {
    case TRX_F32: return launch_rope<float, true>(p, B, s);
    case TRX_F16:
      return tf32 ? launch_rope<__half, true>(p, B, s) : launch_rope<__half, false>(p, B, s);
    default:
      return tf32 ? launch_rope<__nv_bfloat16, true>(p, B, s)
                  : launch_rope<__nv_bfloat16, false>(p, B, s);
  }
}

extern "C" int trx_dequant_rowwise_i8(const int8_t* codes, const float* scales, void* y, int64_t R,
                                      int64_t C, int64_t codes_row_stride, int64_t y_row_stride,
                                      int y_dtype, void* stream) {
  if (y_dtype != TRX_F32 && y_dtype != TRX_F16 && y_dtype != TRX_BF16) return TRX_ERR_DTYPE;
  if (R < 0 || C <= 0) return TRX_ERR_SHAPE;
  if (R == 0) return TRX_OK;
  if (!codes || !scales || !y) return TRX_ERR_NULL_POINTER;
  if (codes_row_stride < C || y_row_stride < C) return TRX_ERR_STRIDE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (y_dtype) {
    case TRX_F32:
      return launch_dequant<float>(codes, scales, y, R, C, codes_row_stride, y_row_stride, s);
    case TRX_F16:
      return launch_dequant<__half>(codes, scales, y, R, C, codes_row_stride, y_row_stride, s);
    default:
      return launch_dequant<__nv_bfloat16>(codes, scales, y, R, C, codes_row_stride, y_row_stride,
                                           s);
  }
}
