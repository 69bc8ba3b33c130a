// Backward of the row and gate ops: RMSNorm, LayerNorm (dx, dW, db) and the three GLUs.
//
// Norms. A CTA of 128 to 512 threads walks rows blockIdx.x, blockIdx.x + gridDim.x, ...; a row of x and
// of dy is read from HBM once with 128-bit streaming loads and stays in registers. The row's
// statistics are recomputed from x (nothing has to be saved by the forward), dx is written, and
// every thread keeps fp32 running sums of dy * n (and dy) for the columns it owns. At the end
// each CTA writes its sums as one row of a (P, C) fp32 block in the caller's workspace and a
// second kernel adds the P rows in a fixed order: dW and db are deterministic for a given shape
// and device. (The reference accumulates dW across programs under spin locks,
// kernels/rmsnorm_kernel.py:65-150, so its summation order changes from run to run.)
// Rows that do not fit the vector path (odd widths, unaligned pointers, more than 1024 vectors)
// take scalar multi-pass kernels: dx plus per-row (mean, rstd) into the workspace, then column
// sums over row slices into the same (P, C) block.
//
// GLUs: y = up * act(gate), so dup = dy * act(gate), dgate = dy * up * act'(gate); fp32 math, one
// rounding per output, separate row strides for every tensor so that the two gradients can be
// written straight into the halves of a concatenated (R, 2H) gradient.
#include "common.cuh"

// RMSNorm: vectors per thread for rows of 257..512 vectors (512 / this many threads per row)
#ifndef TRX_BWD512_VPT
#define TRX_BWD512_VPT 2
#endif
// rows ahead of the current one that a CTA asks the copy engine to pull into L2 (0 = off)
#ifndef TRX_BWD_L2_PREFETCH
#define TRX_BWD_L2_PREFETCH 1
#endif
// minimum resident CTAs (of up to 256 threads) per SM asked of the compiler (caps registers per thread);
// without it the compiler spends registers freely and the occupancy drops (measured: LayerNorm
// 336 us at 121 registers, 208 us at 80)
#ifndef TRX_BWD_MINB_LN
#define TRX_BWD_MINB_LN 3
#endif
#ifndef TRX_BWD_MINB_RMS
#define TRX_BWD_MINB_RMS 3
#endif
// grid of the norm backward kernel in resident waves
#ifndef TRX_BWD_WAVES
#define TRX_BWD_WAVES 1
#endif

namespace trx {

struct NormBwdParams {
  const void* dy;
  const void* x;
  const void* w;     // may be null (LayerNorm without affine part)
  const void* res;   // may be null; otherwise the row is x + res (fp32 sum), dx serves both
  void* dx;
  float* dw_part;    // (P, C) fp32 or null
  float* db_part;    // (P, C) fp32 or null
  float* stats;      // (R, 2) fp32: mean, rstd (scalar path only)
  int64_t R, C;
  int64_t dy_stride, x_stride, dx_stride, res_stride;  // elements
  float eps;
  int w_dtype;
  int act;           // -1: plain norm; TRX_ACT_*: the upstream gradient is dy * act'(w * n)
};

// Sum of a float2 over the NT threads of a CTA; two alternating banks, one barrier.
template <int NT = 256>
__device__ __forceinline__ float2 block_sum2(float2 v, float2 (*red)[NT / 32], int& sel) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    v.x += __shfl_xor_sync(0xffffffffu, v.x, o);
    v.y += __shfl_xor_sync(0xffffffffu, v.y, o);
  }
  if ((threadIdx.x & 31) == 0) red[sel][threadIdx.x >> 5] = v;
  __syncthreads();
  float2 r = red[sel][0];
#pragma unroll
  for (int i = 1; i < NT / 32; ++i) {
    r.x += red[sel][i].x;
    r.y += red[sel][i].y;
  }
  sel ^= 1;
  return r;
}

// Sum of one float over the NT threads of a CTA, through the x lanes of the same banks.
template <int NT = 256>
__device__ __forceinline__ float block_sum1(float v, float2 (*red)[NT / 32], int& sel) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[sel][threadIdx.x >> 5].x = v;
  __syncthreads();
  float r = red[sel][0].x;
#pragma unroll
  for (int i = 1; i < NT / 32; ++i) r += red[sel][i].x;
  sel ^= 1;
  return r;
}

// act'(z) for the activations of act(RMSNorm(x)): mish z tanh(softplus z), quickgelu
// z sigmoid(1.702 z), squared ReLU max(z, 0)^2. With q = e^z (e^z + 2): tanh(softplus z) =
// q / (q + 2) and 1 - tanh = 2 / (q + 2), so 1 - tanh^2 carries no cancellation; z is clamped at
// 20 for the exponential (the derivative is 1 to fp32 precision beyond that).
// FAST (16-bit tensors): hardware exponential and reciprocal.
template <bool FAST>
__device__ __forceinline__ float act_grad(int act, float z) {
  auto ex = [](float v) { return FAST ? __expf(v) : expf(v); };
  auto rcp = [](float v) { return FAST ? __fdividef(1.0f, v) : __fdiv_rn(1.0f, v); };
  if (act == TRX_ACT_MISH) {
    const float e = ex(fminf(z, 20.0f));
    const float q = e * (e + 2.0f);
    const float r = rcp(q + 2.0f);
    const float th = q * r;
    const float sg = e * rcp(1.0f + e);
    return fmaf(z * sg, 2.0f * r * (1.0f + th), th);
  }
  if (act == TRX_ACT_QUICKGELU) {
    const float a = 1.702f * z;
    const float e = ex(-fabsf(a));
    const float sp = rcp(1.0f + e), sm = e * sp;
    const float s = a >= 0.0f ? sp : sm, t = a >= 0.0f ? sm : sp;
    return s * fmaf(a, t, 1.0f);
  }
  return 2.0f * fmaxf(z, 0.0f);
}

template <bool LN, typename T, int VPT, int NT>
__global__ void __launch_bounds__(NT, NT <= 256 ? (LN ? TRX_BWD_MINB_LN : TRX_BWD_MINB_RMS) : 1) norm_bwd_kernel(const NormBwdParams p) {
  using P = Pack<T>;
  constexpr int VEC = P::VEC;
  __shared__ float2 red[2][NT / 32];
  int sel = 0;
  const int t = threadIdx.x;
  const int nvec = static_cast<int>(p.C / VEC);
  const float inv_C = __fdiv_rn(1.0f, static_cast<float>(p.C));

  constexpr int H2 = VEC / 2;
  float2 dwacc[VPT][H2];
  float2 dbacc[LN ? VPT : 1][H2];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < H2; ++j) {
      dwacc[i][j] = make_float2(0.0f, 0.0f);
      if constexpr (LN) dbacc[i][j] = make_float2(0.0f, 0.0f);
    }

  for (int64_t row = blockIdx.x; row < p.R; row += gridDim.x) {
    const T* xrow = reinterpret_cast<const T*>(p.x) + row * p.x_stride;
    const T* grow = reinterpret_cast<const T*>(p.dy) + row * p.dy_stride;
    uint4 xr[VPT], gr[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = i * NT + t;
      const bool live = v < nvec;
      xr[i] = live ? ld_stream16(xrow + static_cast<int64_t>(v) * VEC) : make_uint4(0u, 0u, 0u, 0u);
      gr[i] = live ? ld_stream16(grow + static_cast<int64_t>(v) * VEC) : make_uint4(0u, 0u, 0u, 0u);
    }
    if constexpr (TRX_BWD_L2_PREFETCH > 0) {
      // the rows this CTA takes next come from HBM into L2 while this one is worked on
      const int64_t prow = row + static_cast<int64_t>(TRX_BWD_L2_PREFETCH) * gridDim.x;
      if (t == 0 && prow < p.R) {
        const uint32_t row_bytes = static_cast<uint32_t>(nvec) * 16u;
        l2_prefetch_bulk(reinterpret_cast<const T*>(p.x) + prow * p.x_stride, row_bytes);
        l2_prefetch_bulk(reinterpret_cast<const T*>(p.dy) + prow * p.dy_stride, row_bytes);
        if (p.res) l2_prefetch_bulk(reinterpret_cast<const T*>(p.res) + prow * p.res_stride, row_bytes);
      }
    }
    // fp32 pairs: the arithmetic below is packed (two lanes per instruction)
    float2 xf[VPT][H2], gf[VPT][H2];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      P::unpack2(xr[i], xf[i]);
      P::unpack2(gr[i], gf[i]);
    }
    if (p.res) {  // residual forms: the normalised row is the fp32 sum x + r, as in the forward
      const T* rrow = reinterpret_cast<const T*>(p.res) + row * p.res_stride;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = i * NT + t;
        if (v < nvec) {
          float2 rf[H2];
          P::unpack2(ld_stream16(rrow + static_cast<int64_t>(v) * VEC), rf);
#pragma unroll
          for (int j = 0; j < H2; ++j) xf[i][j] = add2(xf[i][j], rf[j]);
        }
      }
    }
    // ---- statistics, recomputed from x --------------------------------------------
    float mean = 0.0f, rstd;
    if constexpr (LN) {
      float2 s2 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int j = 0; j < H2; ++j) s2 = add2(s2, xf[i][j]);
      mean = block_sum1<NT>(s2.x + s2.y, red, sel) * inv_C;
      const float2 nmean2 = make_float2(-mean, -mean);
      float2 cs2 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        if (i * NT + t < nvec) {  // padding vectors must not contribute (0 - mean)^2
#pragma unroll
          for (int j = 0; j < H2; ++j) {
            xf[i][j] = add2(xf[i][j], nmean2);  // centred from here on
            cs2 = fma2(xf[i][j], xf[i][j], cs2);
          }
        }
      }
      rstd = rsqrtf(fmaf(block_sum1<NT>(cs2.x + cs2.y, red, sel), inv_C, p.eps));
    } else {
      float2 ss2 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int j = 0; j < H2; ++j) ss2 = fma2(xf[i][j], xf[i][j], ss2);
      rstd = rsqrtf(fmaf(block_sum1<NT>(ss2.x + ss2.y, red, sel), inv_C, p.eps));
    }
    // ---- n = (x - mean) * rstd, g = dy * w, running column sums, row sums ----------
    const float2 rstd2 = make_float2(rstd, rstd);
    float2 c1 = make_float2(0.0f, 0.0f), c2 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = i * NT + t;
      if (v < nvec) {
        float wv[VEC];
        if (p.w) load_param_vec<VEC>(p.w, p.w_dtype, static_cast<int64_t>(v) * VEC, wv);
#pragma unroll
        for (int j = 0; j < H2; ++j) {
          const float2 n = mul2(xf[i][j], rstd2);
          float2 dyv = gf[i][j];
          if constexpr (!LN) {
            if (p.act >= 0) {  // act(RMSNorm): chain through the activation at z = w * n
              dyv.x *= act_grad<sizeof(T) == 2>(p.act, n.x * wv[2 * j]);
              dyv.y *= act_grad<sizeof(T) == 2>(p.act, n.y * wv[2 * j + 1]);
            }
          }
          dwacc[i][j] = fma2(dyv, n, dwacc[i][j]);
          if constexpr (LN) dbacc[i][j] = add2(dbacc[i][j], dyv);
          const float2 g = p.w ? mul2(dyv, make_float2(wv[2 * j], wv[2 * j + 1])) : dyv;
          xf[i][j] = n;
          gf[i][j] = g;
          c1 = fma2(g, n, c1);
          if constexpr (LN) c2 = add2(c2, g);
        }
      }
    }
    float m1, m2 = 0.0f;
    if constexpr (LN) {
      const float2 c = block_sum2<NT>(make_float2(c1.x + c1.y, c2.x + c2.y), red, sel);
      m1 = c.x * inv_C;
      m2 = c.y * inv_C;
    } else {
      m1 = block_sum1<NT>(c1.x + c1.y, red, sel) * inv_C;
    }
    // ---- dx = rstd * (g - mean(g) - n * mean(g * n)) ------------------------------
    const float2 nm1 = make_float2(-m1, -m1), nm2 = make_float2(-m2, -m2);
    T* dxrow = reinterpret_cast<T*>(p.dx) + row * p.dx_stride;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = i * NT + t;
      if (v < nvec) {
        float o[VEC];
#pragma unroll
        for (int j = 0; j < H2; ++j) {
          float2 d = fma2(xf[i][j], nm1, gf[i][j]);
          if constexpr (LN) d = add2(d, nm2);
          d = mul2(d, rstd2);
          o[2 * j] = d.x;
          o[2 * j + 1] = d.y;
        }
        st_stream16(dxrow + static_cast<int64_t>(v) * VEC, P::pack(o));
      }
    }
  }
  // ---- this CTA's column sums -> row blockIdx.x of the (P, C) blocks ----------------
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = i * NT + t;
    if (v < nvec) {
      const int64_t off = static_cast<int64_t>(blockIdx.x) * p.C + static_cast<int64_t>(v) * VEC;
#pragma unroll
      for (int q = 0; q < VEC / 4; ++q) {
        if (p.dw_part)
          *reinterpret_cast<float4*>(p.dw_part + off + 4 * q) =
              make_float4(dwacc[i][2 * q].x, dwacc[i][2 * q].y, dwacc[i][2 * q + 1].x, dwacc[i][2 * q + 1].y);
        if constexpr (LN) {
          if (p.db_part)
            *reinterpret_cast<float4*>(p.db_part + off + 4 * q) =
                make_float4(dbacc[i][2 * q].x, dbacc[i][2 * q].y, dbacc[i][2 * q + 1].x, dbacc[i][2 * q + 1].y);
        }
      }
    }
  }
}

// Scalar path, step 1: dx for any C and alignment, (mean, rstd) of every row into p.stats.
template <bool LN, typename T>
__global__ void __launch_bounds__(256) norm_bwd_generic_dx(const NormBwdParams p) {
  using P = Pack<T>;
  __shared__ float2 red[2][8];
  int sel = 0;
  const float inv_C = __fdiv_rn(1.0f, static_cast<float>(p.C));
  for (int64_t row = blockIdx.x; row < p.R; row += gridDim.x) {
    const T* xrow = reinterpret_cast<const T*>(p.x) + row * p.x_stride;
    const T* grow = reinterpret_cast<const T*>(p.dy) + row * p.dy_stride;
    T* dxrow = reinterpret_cast<T*>(p.dx) + row * p.dx_stride;
    const T* rrow = p.res ? reinterpret_cast<const T*>(p.res) + row * p.res_stride : nullptr;
    auto xval = [&](int64_t c) -> float {  // x, or the fp32 sum x + residual
      const float f = P::load1(xrow + c);
      return rrow ? f + P::load1(rrow + c) : f;
    };
    float mean = 0.0f;
    if constexpr (LN) {
      float s = 0.0f;
      for (int64_t c = threadIdx.x; c < p.C; c += 256) s += xval(c);
      mean = block_sum2(make_float2(s, 0.0f), red, sel).x * inv_C;
    }
    float cs = 0.0f;
    for (int64_t c = threadIdx.x; c < p.C; c += 256) {
      const float d = xval(c) - mean;
      cs = fmaf(d, d, cs);
    }
    const float rstd = rsqrtf(fmaf(block_sum2(make_float2(cs, 0.0f), red, sel).x, inv_C, p.eps));
    float c1 = 0.0f, c2 = 0.0f;
    for (int64_t c = threadIdx.x; c < p.C; c += 256) {
      const float n = (xval(c) - mean) * rstd;
      float g = P::load1(grow + c);
      if (p.w) {
        const float wc = load_param1(p.w, p.w_dtype, c);
        if (p.act >= 0) g *= act_grad<sizeof(T) == 2>(p.act, n * wc);
        g *= wc;
      }
      c1 = fmaf(g, n, c1);
      c2 += g;
    }
    const float2 cc = block_sum2(make_float2(c1, c2), red, sel);
    c1 = cc.x * inv_C;
    c2 = LN ? cc.y * inv_C : 0.0f;
    for (int64_t c = threadIdx.x; c < p.C; c += 256) {
      const float n = (xval(c) - mean) * rstd;
      float g = P::load1(grow + c);
      if (p.w) {
        const float wc = load_param1(p.w, p.w_dtype, c);
        if (p.act >= 0) g *= act_grad<sizeof(T) == 2>(p.act, n * wc);
        g *= wc;
      }
      P::store1(dxrow + c, rstd * (g - c2 - n * c1));
    }
    if (threadIdx.x == 0 && p.stats) {
      p.stats[2 * row] = mean;
      p.stats[2 * row + 1] = rstd;
    }
  }
}

// Scalar path, step 2: one thread per column, one row slice per blockIdx.y.
template <typename T>
__global__ void __launch_bounds__(256) norm_bwd_generic_partials(const NormBwdParams p) {
  using P = Pack<T>;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (c >= p.C) return;
  float dw = 0.0f, db = 0.0f;
  for (int64_t row = blockIdx.y; row < p.R; row += gridDim.y) {
    const float dyv = P::load1(reinterpret_cast<const T*>(p.dy) + row * p.dy_stride + c);
    float xv = P::load1(reinterpret_cast<const T*>(p.x) + row * p.x_stride + c);
    if (p.res) xv += P::load1(reinterpret_cast<const T*>(p.res) + row * p.res_stride + c);
    const float n = (xv - p.stats[2 * row]) * p.stats[2 * row + 1];
    float dz = dyv;
    if (p.act >= 0) dz *= act_grad<sizeof(T) == 2>(p.act, n * load_param1(p.w, p.w_dtype, c));
    dw = fmaf(dz, n, dw);
    db += dyv;
  }
  const int64_t off = static_cast<int64_t>(blockIdx.y) * p.C + c;
  if (p.dw_part) p.dw_part[off] = dw;
  if (p.db_part) p.db_part[off] = db;
}

// out[c] = sum over the P rows of part (fixed order), stored in the parameter dtype. 32 columns x
// 32 row slices per CTA: a warp reads 128 contiguous bytes, a thread adds every 32nd row, the 32
// slice sums of a column are added in slice order. blockIdx.y selects dW (0) or db (1).
struct ReduceParams {
  const float* part[2];
  void* out[2];
};
__global__ void __launch_bounds__(1024) reduce_partials_kernel(const ReduceParams rp, int P_rows,
                                                               int64_t C, int dtype) {
  __shared__ float sm[32][33];
  const float* part = rp.part[blockIdx.y];
  void* out = rp.out[blockIdx.y];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * 32 + tx;
  float a0 = 0.0f, a1 = 0.0f;
  if (c < C) {
    int pr = ty;
    for (; pr + 32 < P_rows; pr += 64) {  // two loads in flight per thread
      a0 += part[static_cast<int64_t>(pr) * C + c];
      a1 += part[static_cast<int64_t>(pr + 32) * C + c];
    }
    if (pr < P_rows) a0 += part[static_cast<int64_t>(pr) * C + c];
  }
  sm[ty][tx] = a0 + a1;
  __syncthreads();
  if (ty == 0 && c < C) {
    float s = sm[0][tx];
#pragma unroll
    for (int i = 1; i < 32; ++i) s += sm[i][tx];
    if (dtype == TRX_F32) reinterpret_cast<float*>(out)[c] = s;
    else if (dtype == TRX_BF16) reinterpret_cast<__nv_bfloat16*>(out)[c] = __float2bfloat16_rn(s);
    else reinterpret_cast<__half*>(out)[c] = __float2half_rn(s);
  }
}

// Rows of partial sums for a (R, C) problem: bounded so that the two (P, C) blocks stay small.
static int64_t norm_bwd_partial_rows(int64_t R, int64_t C) {
  int64_t cap = (static_cast<int64_t>(1) << 22) / (C > 0 ? C : 1);
  if (cap < 8) cap = 8;
  if (cap > 1024) cap = 1024;
  return R < cap ? R : cap;
}

// TRX_BWD_WAVES resident waves of CTAs (each walks R / grid rows); P_rows comes back as the grid size, i.e.
// the number of rows of partial sums that were written.
template <bool LN, typename T, int VPT, int NT>
static void launch_norm_bwd_vec(const NormBwdParams& p, int64_t& P_rows, cudaStream_t stream) {
  static std::atomic<int> blocks_per_sm_of[64];  // racing first calls store the same value
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = -1;
  const bool cacheable = dev >= 0 && dev < 64;
  int blocks_per_sm = cacheable ? blocks_per_sm_of[dev].load(std::memory_order_acquire) : 0;
  if (blocks_per_sm == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, norm_bwd_kernel<LN, T, VPT, NT>, NT, 0) !=
            cudaSuccess || n <= 0)
      n = 1;
    blocks_per_sm = n;
    if (cacheable) blocks_per_sm_of[dev].store(n, std::memory_order_release);
  }
  const int64_t resident = static_cast<int64_t>(sm_count_of_current_device()) * blocks_per_sm * TRX_BWD_WAVES;
  if (P_rows > resident) P_rows = resident;
  norm_bwd_kernel<LN, T, VPT, NT><<<static_cast<unsigned>(P_rows), NT, 0, stream>>>(p);
}

template <bool LN, typename T>
static int launch_norm_bwd(NormBwdParams p, void* dw, void* db, float* ws, cudaStream_t stream) {
  constexpr int VEC = Pack<T>::VEC;
  int64_t P_rows = norm_bwd_partial_rows(p.R, p.C);
  float* part0 = ws;
  float* part1 = ws + norm_bwd_partial_rows(p.R, p.C) * p.C;
  p.stats = part1 + norm_bwd_partial_rows(p.R, p.C) * p.C;
  p.dw_part = dw ? part0 : nullptr;
  p.db_part = db ? part1 : nullptr;
  if (p.R > 0) {
    bool vec_ok = (p.C % VEC == 0) && aligned_to(p.x, 16) && aligned_to(p.dy, 16) &&
                  aligned_to(p.dx, 16) && (p.x_stride % VEC == 0) && (p.dy_stride % VEC == 0) &&
                  (p.dx_stride % VEC == 0) && aligned_to(ws, 16);
    if (p.w) vec_ok = vec_ok && aligned_to(p.w, 16);
    if (p.res) vec_ok = vec_ok && aligned_to(p.res, 16) && (p.res_stride % VEC == 0);
    const int64_t nvec = p.C / VEC;
    if (vec_ok && nvec <= 1024) {
      // few vectors per thread: the running column sums cost 8 (16 for LayerNorm) registers each
      if (nvec <= 256) launch_norm_bwd_vec<LN, T, 1, 256>(p, P_rows, stream);
      else if (nvec <= 512) {
        // measured on 32768 x 4096 bf16: RMSNorm 256 threads x 2 vectors (146 us; 159 us at
        // 128 x 4), LayerNorm 128 x 4 (170 us; 188 us at 256 x 2): LayerNorm has three CTA-wide
        // reductions per row, which four warps finish sooner than eight; 512 threads x 1 vector
        // is slower for both (213 / 278 us)
        if constexpr (LN) launch_norm_bwd_vec<LN, T, 4, 128>(p, P_rows, stream);
        else launch_norm_bwd_vec<LN, T, TRX_BWD512_VPT, 512 / TRX_BWD512_VPT>(p, P_rows, stream);
      }
      else launch_norm_bwd_vec<LN, T, 2, 512>(p, P_rows, stream);
    } else {
      const int64_t cap = static_cast<int64_t>(sm_count_of_current_device()) * 8;
      norm_bwd_generic_dx<LN, T><<<static_cast<unsigned>(p.R < cap ? p.R : cap), 256, 0, stream>>>(p);
      if (dw || db) {
        const dim3 grid(static_cast<unsigned>((p.C + 255) / 256), static_cast<unsigned>(P_rows));
        norm_bwd_generic_partials<T><<<grid, 256, 0, stream>>>(p);
      }
    }
  } else {
    P_rows = 0;
  }
  if (dw || db) {
    ReduceParams rp{};
    int n = 0;
    if (dw) { rp.part[n] = p.dw_part; rp.out[n] = dw; ++n; }
    if (db) { rp.part[n] = p.db_part; rp.out[n] = db; ++n; }
    const dim3 cgrid(static_cast<unsigned>((p.C + 31) / 32), static_cast<unsigned>(n));
    reduce_partials_kernel<<<cgrid, 1024, 0, stream>>>(rp, static_cast<int>(P_rows), p.C, p.w_dtype);
  }
  return cudaGetLastError() == cudaSuccess ? TRX_OK : TRX_ERR_CUDA;
}

static bool bwd_dtype_ok(int d) { return d == TRX_F32 || d == TRX_F16 || d == TRX_BF16; }

static size_t norm_bwd_workspace(int64_t R, int64_t C) {
  if (R < 0 || C <= 0) return 0;
  const int64_t floats = 2 * norm_bwd_partial_rows(R, C) * C + 2 * R;
  return static_cast<size_t>(floats) * sizeof(float) + 16;
}

template <bool LN>
static int norm_bwd_entry(const void* dy, const void* x, const void* w, void* dx, void* dw, void* db,
                          int64_t R, int64_t C, int64_t dy_stride, int64_t x_stride,
                          int64_t dx_stride, float eps, int x_dtype, int w_dtype, void* workspace,
                          size_t workspace_bytes, void* stream, const void* res = nullptr,
                          int64_t res_stride = 0, int act = -1) {
  if (!bwd_dtype_ok(x_dtype) || !bwd_dtype_ok(w_dtype)) return TRX_ERR_DTYPE;
  if (R < 0 || C <= 0) return TRX_ERR_SHAPE;
  if (R > 0 && (!dy || !x || !dx)) return TRX_ERR_NULL_POINTER;
  if (!LN && !w) return TRX_ERR_NULL_POINTER;
  if (R > 0 && (dy_stride < C || x_stride < C || dx_stride < C)) return TRX_ERR_STRIDE;
  if (R > 0 && res && res_stride < C) return TRX_ERR_STRIDE;
  if (R == 0 && !dw && !db) return TRX_OK;
  if (!workspace || workspace_bytes < norm_bwd_workspace(R, C)) return TRX_ERR_WORKSPACE;
  if (!aligned_to(workspace, 4)) return TRX_ERR_ALIGNMENT;
  NormBwdParams p{};
  p.dy = dy; p.x = x; p.w = w; p.dx = dx; p.res = res; p.res_stride = res_stride;
  p.R = R; p.C = C; p.dy_stride = dy_stride; p.x_stride = x_stride; p.dx_stride = dx_stride;
  p.eps = eps; p.w_dtype = w_dtype; p.act = act;
  float* ws = static_cast<float*>(workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (x_dtype) {
    case TRX_F32: return launch_norm_bwd<LN, float>(p, dw, db, ws, s);
    case TRX_F16: return launch_norm_bwd<LN, __half>(p, dw, db, ws, s);
    default: return launch_norm_bwd<LN, __nv_bfloat16>(p, dw, db, ws, s);
  }
}

// ----------------------------------------------------------------------------
// GLU backward
// ----------------------------------------------------------------------------
// act(g) and act'(g) in fp32. SwiGLU: silu; GeGLU: tanh form with the reference's constants
// (kernels/geglu_kernel.py:37-38), written through sigmoid(2u) = (1 + tanh u) / 2; ReGLU:
// max(g, 0). The sigmoids are built from e = exp(-|z|) in (0, 1], so nothing overflows for
// large |z| and 1 - sigmoid is formed without cancellation. FAST (16-bit tensors): hardware
// exponential and reciprocal, whose error is far below the storage rounding step.
template <bool FAST>
__device__ __forceinline__ void sigmoid_pair(float z, float& s, float& one_minus_s) {
  const float e = FAST ? __expf(-fabsf(z)) : expf(-fabsf(z));
  const float sp = FAST ? __fdividef(1.0f, 1.0f + e) : __fdiv_rn(1.0f, 1.0f + e);
  const float sm = e * sp;
  s = z >= 0.0f ? sp : sm;
  one_minus_s = z >= 0.0f ? sm : sp;
}

template <int ACT, bool FAST>
__device__ __forceinline__ void act_and_grad(float g, float& a, float& da) {
  if constexpr (ACT == TRX_GLU_SWIGLU) {
    float s, t;
    sigmoid_pair<FAST>(g, s, t);
    a = g * s;
    da = s * fmaf(g, t, 1.0f);
  } else if constexpr (ACT == TRX_GLU_GEGLU_TANH) {
    const float k = 0.7978845608028654f, c = 0.044715f;
    const float g2 = g * g;
    const float u = k * g * fmaf(c, g2, 1.0f);
    float h, t;  // h = (1 + tanh u) / 2, t = 1 - h; (1 - tanh^2 u) / 2 = 2 h t
    sigmoid_pair<FAST>(2.0f * u, h, t);
    const float du = k * fmaf(3.0f * c, g2, 1.0f);
    a = g * h;
    da = fmaf(g * du, 2.0f * h * t, h);
  } else {
    a = fmaxf(g, 0.0f);
    da = g > 0.0f ? 1.0f : 0.0f;
  }
}

struct GluBwdParams {
  const void* dy;
  const void* up;
  const void* gate;
  void* dup;
  void* dgate;
  int64_t R, H;
  int64_t dy_stride, up_stride, gate_stride, dup_stride, dgate_stride;  // elements
};

template <int ACT, typename T, bool VECTOR>
__global__ void __launch_bounds__(128) glu_bwd_kernel(const GluBwdParams p) {
  using P = Pack<T>;
  constexpr int VEC = VECTOR ? P::VEC : 1;
  constexpr bool FAST = sizeof(T) == 2;
  const int64_t v = static_cast<int64_t>(blockIdx.x) * 128 + threadIdx.x;
  const int64_t col = v * VEC;
  if (col >= p.H) return;
  for (int64_t row = blockIdx.y; row < p.R; row += gridDim.y) {
    const T* dy = reinterpret_cast<const T*>(p.dy) + row * p.dy_stride + col;
    const T* up = reinterpret_cast<const T*>(p.up) + row * p.up_stride + col;
    const T* gate = reinterpret_cast<const T*>(p.gate) + row * p.gate_stride + col;
    T* dup = reinterpret_cast<T*>(p.dup) + row * p.dup_stride + col;
    T* dgate = reinterpret_cast<T*>(p.dgate) + row * p.dgate_stride + col;
    if constexpr (VECTOR) {
      float d[P::VEC], u[P::VEC], g[P::VEC], ou[P::VEC], og[P::VEC];
      P::unpack(ld_stream16(dy), d);
      P::unpack(ld_stream16(up), u);
      P::unpack(ld_stream16(gate), g);
#pragma unroll
      for (int j = 0; j < P::VEC; ++j) {
        float a, da;
        act_and_grad<ACT, FAST>(g[j], a, da);
        ou[j] = d[j] * a;
        og[j] = d[j] * u[j] * da;
      }
      st_stream16(dup, P::pack(ou));
      st_stream16(dgate, P::pack(og));
    } else {
      float a, da;
      const float d = P::load1(dy);
      act_and_grad<ACT, FAST>(P::load1(gate), a, da);
      P::store1(dup, d * a);
      P::store1(dgate, d * P::load1(up) * da);
    }
  }
}

template <int ACT, typename T>
static int launch_glu_bwd(const GluBwdParams& p, cudaStream_t stream) {
  constexpr int VEC = Pack<T>::VEC;
  const bool vec_ok = (p.H % VEC == 0) && aligned_to(p.dy, 16) && aligned_to(p.up, 16) &&
                      aligned_to(p.gate, 16) && aligned_to(p.dup, 16) && aligned_to(p.dgate, 16) &&
                      (p.dy_stride % VEC == 0) && (p.up_stride % VEC == 0) &&
                      (p.gate_stride % VEC == 0) && (p.dup_stride % VEC == 0) &&
                      (p.dgate_stride % VEC == 0);
  const int64_t units = vec_ok ? p.H / VEC : p.H;
  const int64_t gx = (units + 127) / 128;
  // enough CTAs for several resident waves; a CTA walks rows blockIdx.y, + gridDim.y, ...
  int64_t gy = (static_cast<int64_t>(sm_count_of_current_device()) * 64 + gx - 1) / gx;
  if (gy > p.R) gy = p.R;
  if (gy > 65535) gy = 65535;
  if (gx > 0x7fffffff) return TRX_ERR_SHAPE;
  const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
  if (vec_ok) glu_bwd_kernel<ACT, T, true><<<grid, 128, 0, stream>>>(p);
  else glu_bwd_kernel<ACT, T, false><<<grid, 128, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? TRX_OK : TRX_ERR_CUDA;
}

template <typename T>
static int launch_glu_bwd_act(const GluBwdParams& p, int act, cudaStream_t stream) {
  switch (act) {
    case TRX_GLU_SWIGLU: return launch_glu_bwd<TRX_GLU_SWIGLU, T>(p, stream);
    case TRX_GLU_GEGLU_TANH: return launch_glu_bwd<TRX_GLU_GEGLU_TANH, T>(p, stream);
    case TRX_GLU_REGLU: return launch_glu_bwd<TRX_GLU_REGLU, T>(p, stream);
    default: return TRX_ERR_UNSUPPORTED;
  }
}

}  // namespace trx

using namespace trx;

extern "C" size_t trx_norm_bwd_workspace_bytes(int64_t R, int64_t C) { return norm_bwd_workspace(R, C); }

extern "C" int trx_rmsnorm_bwd(const void* dy, const void* x, const void* w, void* dx,
                               void* dw_or_null, int64_t R, int64_t C, int64_t dy_row_stride,
                               int64_t x_row_stride, int64_t dx_row_stride, float eps, int x_dtype,
                               int w_dtype, void* workspace, size_t workspace_bytes, void* stream) {
  return norm_bwd_entry<false>(dy, x, w, dx, dw_or_null, nullptr, R, C, dy_row_stride, x_row_stride,
                               dx_row_stride, eps, x_dtype, w_dtype, workspace, workspace_bytes,
                               stream);
}

extern "C" int trx_layernorm_bwd(const void* dy, const void* x, const void* w_or_null, void* dx,
                                 void* dw_or_null, void* db_or_null, int64_t R, int64_t C,
                                 int64_t dy_row_stride, int64_t x_row_stride, int64_t dx_row_stride,
                                 float eps, int x_dtype, int wb_dtype, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  return norm_bwd_entry<true>(dy, x, w_or_null, dx, dw_or_null, db_or_null, R, C, dy_row_stride,
                              x_row_stride, dx_row_stride, eps, x_dtype, wb_dtype, workspace,
                              workspace_bytes, stream);
}

extern "C" int trx_residual_rmsnorm_bwd(const void* dy, const void* x, const void* residual,
                                        const void* w, void* dx, void* dw_or_null, int64_t R,
                                        int64_t C, int64_t dy_row_stride, int64_t x_row_stride,
                                        int64_t res_row_stride, int64_t dx_row_stride, float eps,
                                        int x_dtype, int w_dtype, void* workspace,
                                        size_t workspace_bytes, void* stream) {
  if (R > 0 && !residual) return TRX_ERR_NULL_POINTER;
  return norm_bwd_entry<false>(dy, x, w, dx, dw_or_null, nullptr, R, C, dy_row_stride, x_row_stride,
                               dx_row_stride, eps, x_dtype, w_dtype, workspace, workspace_bytes,
                               stream, residual, res_row_stride);
}

extern "C" int trx_residual_layernorm_bwd(const void* dy, const void* x, const void* residual,
                                          const void* w_or_null, void* dx, void* dw_or_null,
                                          void* db_or_null, int64_t R, int64_t C,
                                          int64_t dy_row_stride, int64_t x_row_stride,
                                          int64_t res_row_stride, int64_t dx_row_stride, float eps,
                                          int x_dtype, int wb_dtype, void* workspace,
                                          size_t workspace_bytes, void* stream) {
  if (R > 0 && !residual) return TRX_ERR_NULL_POINTER;
  return norm_bwd_entry<true>(dy, x, w_or_null, dx, dw_or_null, db_or_null, R, C, dy_row_stride,
                              x_row_stride, dx_row_stride, eps, x_dtype, wb_dtype, workspace,
                              workspace_bytes, stream, residual, res_row_stride);
}

extern "C" int trx_rmsnorm_act_bwd(const void* dy, const void* x, const void* w, void* dx,
                                   void* dw_or_null, int64_t R, int64_t C, int64_t dy_row_stride,
                                   int64_t x_row_stride, int64_t dx_row_stride, float eps, int act,
                                   int x_dtype, int w_dtype, void* workspace,
                                   size_t workspace_bytes, void* stream) {
  if (act != TRX_ACT_MISH && act != TRX_ACT_QUICKGELU && act != TRX_ACT_SQUARED_RELU)
    return TRX_ERR_UNSUPPORTED;
  return norm_bwd_entry<false>(dy, x, w, dx, dw_or_null, nullptr, R, C, dy_row_stride, x_row_stride,
                               dx_row_stride, eps, x_dtype, w_dtype, workspace, workspace_bytes,
                               stream, nullptr, 0, act);
}

extern "C" int trx_glu_bwd(const void* dy, const void* up, const void* gate, void* dup, void* dgate,
                           int64_t R, int64_t H, int64_t dy_row_stride, int64_t up_row_stride,
                           int64_t gate_row_stride, int64_t dup_row_stride,
                           int64_t dgate_row_stride, int act, int dtype, void* stream) {
  if (!bwd_dtype_ok(dtype)) return TRX_ERR_DTYPE;
  if (act != TRX_GLU_SWIGLU && act != TRX_GLU_GEGLU_TANH && act != TRX_GLU_REGLU)
    return TRX_ERR_UNSUPPORTED;
  if (R < 0 || H <= 0) return TRX_ERR_SHAPE;
  if (R == 0) return TRX_OK;
  if (!dy || !up || !gate || !dup || !dgate) return TRX_ERR_NULL_POINTER;
  if (dy_row_stride < H || up_row_stride < H || gate_row_stride < H || dup_row_stride < H ||
      dgate_row_stride < H)
    return TRX_ERR_STRIDE;
  GluBwdParams p{dy, up, gate, dup, dgate, R, H, dy_row_stride, up_row_stride, gate_row_stride,
                 dup_row_stride, dgate_row_stride};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case TRX_F32: return launch_glu_bwd_act<float>(p, act, s);
    case TRX_F16: return launch_glu_bwd_act<__half>(p, act, s);
    default: return launch_glu_bwd_act<__nv_bfloat16>(p, act, s);
  }
}
