// Attention forward for sm_100a: softmax(scale * Q K^T + bias) V with online softmax.
//
// One CTA owns two 128-row Q tiles that ping-pong on the tensor pipe: the same 128 query rows of
// two query heads that share a kv head (GQA / MQA: both tiles then see exactly the same keys), or
// 256 consecutive rows of one head otherwise. Roles (576 threads):
//   warps 0-7   softmax of Q tile 0: warp w owns the 16 rows (= TMEM lanes) 32*(w%4)+16*(w/4)..,
//               read in the 16x256b fragment shape: a quad of threads shares a row, a thread
//               holds 2 rows x 32 columns, row maxima cost two shuffles
//   warps 8-15  softmax of Q tile 1, same split
//   warp  16    TMA producer: Q once, then K and V tiles through a 4-stage shared-memory ring
//               (cp.async.bulk.tensor, 128-byte swizzle, no multicast)
//   warp  17    MMA issuer: tcgen05.mma kind::f16, S = Q K^T (both operands from shared memory)
//               and O += P V (P read from TMEM, V from shared memory, MN-major); one thread,
//               flat scalar code, specialised for the rounds in which both Q tiles are active
// TMEM (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each; P (16-bit) overwrites the
// first 64 columns of its S. The softmax groups read S with tcgen05.ld, exponentiate with
// exp2 (scale*log2e folded into one FMA, ALiBi as one more), write P back with tcgen05.st,
// rescale O in TMEM only when the running row max grew by more than 2^8 (lazy rescale) and
// run the epilogue (O / l -> global). KV tiles outside the causal / window range of a Q tile
// are never visited; masks are applied only on boundary tiles. Query head h reads kv head
// h / (Hq / Hk), so GQA / MQA need no tiled copies. With ALiBi under a causal mask the KV tiles
// of a row block are visited from the diagonal backwards: the bias grows with the key index, so
// in that order the first tile holds the row maximum and O is never rescaled again.
//
// Every wait on an mbarrier is bounded: after a fixed number of polls the kernel records a
// code in the status word of the caller's workspace, raises a CTA-wide abort flag, drains its
// own copies and MMAs (bounded again), frees its TMEM and returns.
#include <cuda.h>

#include <atomic>
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace trx {

constexpr int ATT_BM = 128;       // rows per Q tile
constexpr int ATT_BN = 128;       // keys per KV tile
constexpr int ATT_NQ = 2;         // Q tiles per CTA
constexpr int ATT_STAGES = 4;     // KV ring depth (K and V tiles alternate)
constexpr int ATT_SM_WARPS = 16;    // softmax warps: two warpgroups per Q tile, half a row per thread
constexpr int ATT_THREADS = (ATT_SM_WARPS + 2) * 32;
constexpr uint32_t ATT_WAIT_LIMIT = 1u << 26;  // hard cap on polls per wait
constexpr uint64_t ATT_WAIT_NS = 400ull * 1000 * 1000;  // wall-time budget of one wait
constexpr float ATT_LAZY_RESCALE = 8.0f;       // log2 units

enum AttnStatus : unsigned {
  ATT_ST_PRODUCER = 1u,
  ATT_ST_MMA = 2u,
  ATT_ST_SOFTMAX = 4u,
  ATT_ST_DRAIN = 8u,
};

struct AttnParams {
  CUtensorMap tm_q;
  CUtensorMap tm_k;
  CUtensorMap tm_v;
  void* out;
  float* lse;
  const float* slopes;
  unsigned int* status;
  int B, Sq, Sk, Hq;
  int k_hdiv, v_hdiv;  // query heads per kv head (Hq when the tensor's heads are collapsed)
  int k_bmul, v_bmul;  // 1, or 0 when the batch dim is broadcast
  long long o_stride_b, o_stride_s, o_stride_h;
  long long lse_stride_b, lse_stride_h;
  float scale_log2;    // softmax scale * log2(e)
  int causal;
  int win_left, win_right;  // < 0: no window
  int is_bf16;
  int reverse_m;       // schedule the heaviest (last) row blocks first
  int reverse_kv;      // visit a row block's KV tiles from the last to the first
  int pair_heads;      // the two Q tiles of a CTA: same 128 rows of two query heads that share a
                       // kv head (1), or two consecutive 128-row blocks of one head (0)
  // dense additive mask (B, Hq, Sq, Sk) with unit key stride; batch / head strides may be 0
  const void* bias;
  long long bias_sb, bias_sh, bias_sq;  // elements
  int bias_kind;       // 0 none, 1 fp32, 2 the activation dtype
  // dropout on the normalised probabilities: an element is dropped when its random byte is
  // below drop_thr (0 = no dropout); kept ones are scaled by drop_scale = 256 / (256 - drop_thr)
  unsigned drop_thr;
  float drop_scale;
  unsigned seed_lo, seed_hi, drop_offset;
};

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", 2011): a counter
// based generator, so that any element's random byte can be recomputed anywhere, on the host
// too. The dropout stream is keyed by the caller's 64-bit seed; the counter is
// (key index / 16, query row, batch * heads + head, offset) and the 16 bytes of the result
// belong to the 16 consecutive keys of that block, least significant byte first.
__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
    c = make_uint4(hi1 ^ c.y ^ k0, lo1, hi0 ^ c.w ^ k1, lo0);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c;
}

// ------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: gives up after ATT_WAIT_NS of wall time. Returns false if the CTA is aborting
// (this wait ran out or another one did); the first to give up records `code` in the status word.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned int* status, unsigned code) {
#pragma unroll 1
  for (int fast = 0; fast < 64; ++fast)
    if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_ns();
#pragma unroll 1
  for (uint32_t i = 0; i < ATT_WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u) {
      if (*abort_flag) return false;
      if (global_ns() - t0 > ATT_WAIT_NS) break;
    }
  }
  *abort_flag = 1;
  atomicOr(status, code);
  return false;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tm, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
// D[tmem] = A[smem] * B[smem]  (first) / D[tmem] += A[smem] * B[smem]  (acc)
__device__ __forceinline__ void mma_ss_first(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                             uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc)
      : "memory");
}
__device__ __forceinline__ void mma_ss_acc(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; `acc` = 0 overwrites D
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  if constexpr (BF16) return Pack<__nv_bfloat16>::pack2(lo, hi);
  else return Pack<__half>::pack2(lo, hi);
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 2^x on the special-function unit; 2^-inf = +0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base lane + t).
template <int OFF, int N>
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[N]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[OFF + 0]), "=r"(r[OFF + 1]), "=r"(r[OFF + 2]), "=r"(r[OFF + 3]), "=r"(r[OFF + 4]),
        "=r"(r[OFF + 5]), "=r"(r[OFF + 6]), "=r"(r[OFF + 7]), "=r"(r[OFF + 8]), "=r"(r[OFF + 9]),
        "=r"(r[OFF + 10]), "=r"(r[OFF + 11]), "=r"(r[OFF + 12]), "=r"(r[OFF + 13]),
        "=r"(r[OFF + 14]), "=r"(r[OFF + 15]), "=r"(r[OFF + 16]), "=r"(r[OFF + 17]),
        "=r"(r[OFF + 18]), "=r"(r[OFF + 19]), "=r"(r[OFF + 20]), "=r"(r[OFF + 21]),
        "=r"(r[OFF + 22]), "=r"(r[OFF + 23]), "=r"(r[OFF + 24]), "=r"(r[OFF + 25]),
        "=r"(r[OFF + 26]), "=r"(r[OFF + 27]), "=r"(r[OFF + 28]), "=r"(r[OFF + 29]),
        "=r"(r[OFF + 30]), "=r"(r[OFF + 31])
      : "r"(taddr)
      : "memory");
}
template <int OFF, int N>
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[N]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[OFF + 0]), "r"(r[OFF + 1]), "r"(r[OFF + 2]), "r"(r[OFF + 3]),
        "r"(r[OFF + 4]), "r"(r[OFF + 5]), "r"(r[OFF + 6]), "r"(r[OFF + 7]), "r"(r[OFF + 8]),
        "r"(r[OFF + 9]), "r"(r[OFF + 10]), "r"(r[OFF + 11]), "r"(r[OFF + 12]), "r"(r[OFF + 13]),
        "r"(r[OFF + 14]), "r"(r[OFF + 15]), "r"(r[OFF + 16]), "r"(r[OFF + 17]), "r"(r[OFF + 18]),
        "r"(r[OFF + 19]), "r"(r[OFF + 20]), "r"(r[OFF + 21]), "r"(r[OFF + 22]), "r"(r[OFF + 23]),
        "r"(r[OFF + 24]), "r"(r[OFF + 25]), "r"(r[OFF + 26]), "r"(r[OFF + 27]), "r"(r[OFF + 28]),
        "r"(r[OFF + 29]), "r"(r[OFF + 30]), "r"(r[OFF + 31])
      : "memory");
}
// 16 lanes x 256 bits per repetition (8 fp32 columns). Thread t of the warp holds, for column
// group g (8 columns each): r[4g+0..1] = lane (t/4), columns 8g + 2(t%4) + {0,1};
// r[4g+2..3] = lane (t/4) + 8, same columns. Four threads (a quad) share a lane.
__device__ __forceinline__ void tmem_ld_16x256b_x16(uint32_t taddr, uint32_t (&r)[64]) {
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st_16x256b_x16(uint32_t taddr, const uint32_t (&r)[64]) {
  asm volatile("tcgen05.st.sync.aligned.16x256b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63, %64};"
               :
               : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(r[32]), "r"(r[33]), "r"(r[34]), "r"(r[35]), "r"(r[36]), "r"(r[37]), "r"(r[38]), "r"(r[39]), "r"(r[40]), "r"(r[41]), "r"(r[42]), "r"(r[43]), "r"(r[44]), "r"(r[45]), "r"(r[46]), "r"(r[47]), "r"(r[48]), "r"(r[49]), "r"(r[50]), "r"(r[51]), "r"(r[52]), "r"(r[53]), "r"(r[54]), "r"(r[55]), "r"(r[56]), "r"(r[57]), "r"(r[58]), "r"(r[59]), "r"(r[60]), "r"(r[61]), "r"(r[62]), "r"(r[63])
               : "memory");
}
__device__ __forceinline__ void tmem_st_16x256b_x8(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile("tcgen05.st.sync.aligned.16x256b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
               :
               : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
               : "memory");
}
// 16 lanes x 128 bits per repetition (4 columns): r[2g+0] = lane (t/4), column 4g + (t%4);
// r[2g+1] = lane (t/4) + 8, same column.
template <int N>
__device__ __forceinline__ void tmem_st_16x128b_x16(uint32_t taddr, const uint32_t (&r)[N]) {
  asm volatile("tcgen05.st.sync.aligned.16x128b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
               :
               : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
               : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, sm_100 version field = 1.
//   K-major operand : rows of 64 16-bit elements (128 B); 8-row groups 1024 B apart (SBO).
//   MN-major operand: 64 contiguous MN elements per 128-B row of K; 8 K-rows per 1024-B group
//                     (SBO); the next 64 MN elements start LBO bytes further.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes,
                                              uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version
  d |= 2ull << 61;  // SWIZZLE_128B
  return d;
}
// Instruction descriptor for kind::f16 with fp32 accumulation.
__host__ __device__ constexpr uint32_t make_idesc(int is_bf16, int m, int n, int a_mn_major,
                                                  int b_mn_major) {
  return (1u << 4) |                                   // D format fp32
         (static_cast<uint32_t>(is_bf16 ? 1 : 0) << 7) |   // A format
         (static_cast<uint32_t>(is_bf16 ? 1 : 0) << 10) |  // B format
         (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

template <int D>
struct AttnSmem {
  static constexpr int CHUNKS = D / 64;              // 64-element (128-byte) column chunks
  static constexpr int CHUNK_BYTES = ATT_BN * 128;   // 128 rows x 128 B = 16 KB
  static constexpr int TILE_BYTES = CHUNKS * CHUNK_BYTES;
  static constexpr int Q_OFF = 0;
  static constexpr int KV_OFF = ATT_NQ * TILE_BYTES;
  static constexpr int BAR_OFF = KV_OFF + ATT_STAGES * TILE_BYTES;
  static constexpr int NUM_BARS = 2 + 2 * ATT_STAGES + 6 + 1 + 2;
  static constexpr int XCH_OFF = BAR_OFF + NUM_BARS * 8 + 64;      // row max / sum exchange
  static constexpr int XCH_BYTES = ATT_NQ * 2 * ATT_BM * 4;
  static constexpr int TOTAL = XCH_OFF + XCH_BYTES;
  static constexpr int DYN_BYTES = TOTAL + 1024;  // slack for 1024-byte alignment
};

struct TileRange {
  int jlo, jhi;  // KV tiles [jlo, jhi)
};

__device__ __forceinline__ TileRange tile_range(const AttnParams& p, int row0) {
  TileRange r{0, 0};
  if (row0 >= p.Sq) return r;
  const int row1 = min(p.Sq, row0 + ATT_BM) - 1;
  int hi = p.Sk - 1;
  if (p.causal) hi = min(hi, row1);
  if (p.win_right >= 0) hi = min(hi, row1 + p.win_right);
  int lo = 0;
  if (p.win_left >= 0) lo = max(0, row0 - p.win_left);
  if (hi < lo) return r;
  r.jlo = lo / ATT_BN;
  r.jhi = hi / ATT_BN + 1;
  return r;
}

// BIAS: the instantiation with the rarely used features — a dense additive mask and / or dropout,
// each behind a run-time flag; the other instantiation carries none of it.
template <int D, bool BF16, bool BIAS>
__global__ void __launch_bounds__(ATT_THREADS, 1)
    attn_fwd_kernel(const __grid_constant__ AttnParams p) {
  using L = AttnSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + L::BAR_OFF;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  // barrier indices
  constexpr int B_QFULL = 0;                        // [2]
  constexpr int B_KVFULL = 2;                       // [STAGES]
  constexpr int B_KVEMPTY = 2 + ATT_STAGES;         // [STAGES]
  constexpr int B_SFULL = 2 + 2 * ATT_STAGES;       // [2]
  constexpr int B_PFULL = B_SFULL + 2;              // [2]
  constexpr int B_ODONE = B_PFULL + 2;              // [2]
  constexpr int B_DRAIN = B_ODONE + 2;              // [1]
  constexpr int B_XCH = B_DRAIN + 1;                // [2] row-statistics exchange per Q tile
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + L::BAR_OFF + L::NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  int* fills_issued = reinterpret_cast<int*>(tmem_holder + 2);  // [STAGES]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int mblk = p.reverse_m ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int b = blockIdx.z;
  // Q tile t of this CTA: rows m0 + t * t_rows .. + 127 of query head h + t * t_head. Paired heads
  // see the same keys, so both tiles are active in every round; paired row blocks differ by one
  // KV tile at either end of their ranges, where one tile then works alone.
  const int t_rows = p.pair_heads ? 0 : ATT_BM;
  const int t_head = p.pair_heads ? 1 : 0;
  const int h = p.pair_heads ? 2 * blockIdx.y : blockIdx.y;
  const int m0 = mblk * (p.pair_heads ? ATT_BM : ATT_NQ * ATT_BM);

  TileRange rng[ATT_NQ];
#pragma unroll
  for (int t = 0; t < ATT_NQ; ++t) rng[t] = tile_range(p, m0 + t * t_rows);
  int JLO = 1 << 30, JHI = 0;
#pragma unroll
  for (int t = 0; t < ATT_NQ; ++t)
    if (rng[t].jhi > rng[t].jlo) {
      JLO = min(JLO, rng[t].jlo);
      JHI = max(JHI, rng[t].jhi);
    }
  if (JHI <= JLO) { JLO = 0; JHI = 0; }

  // A launch that follows a recorded failure does no work: the host must read and clear
  // the status word first.
  __shared__ int skip_launch;

  // visiting order of the KV tiles: ascending, or descending from the last one
  const int kv_step = p.reverse_kv ? -1 : 1;
  const int kv_first = p.reverse_kv ? JHI - 1 : JLO;
  // One K or V tile into ring stage fill % STAGES (K and V tiles alternate: even fills are K).
  auto issue_fill = [&](int fill) {
    const int s = fill % ATT_STAGES;
    const int j = kv_first + (fill >> 1) * kv_step;
    const bool is_k = (fill & 1) == 0;
    mbar_expect_tx(bar(B_KVFULL + s), L::TILE_BYTES);
    fills_issued[s] = fill / ATT_STAGES + 1;
    const CUtensorMap* tm = is_k ? &p.tm_k : &p.tm_v;
    const int hh = h / (is_k ? p.k_hdiv : p.v_hdiv);
    const int bb = b * (is_k ? p.k_bmul : p.v_bmul);
#pragma unroll
    for (int c = 0; c < L::CHUNKS; ++c)
      tma_load_4d(sbase + L::KV_OFF + s * L::TILE_BYTES + c * L::CHUNK_BYTES, tm,
                  bar(B_KVFULL + s), c * 64, j * ATT_BN, hh, bb);
  };
  // The producer warp's first lane sets up the barriers and starts the Q and first K/V copies
  // before the CTA-wide sync, so that they run under the TMEM allocation and the sync itself.
  if (warp == ATT_SM_WARPS && lane == 0) {
    skip_launch = (*reinterpret_cast<volatile unsigned int*>(p.status) != 0u) ? 1 : 0;
  }
  if (warp == ATT_SM_WARPS && lane == 0 && !skip_launch) {
    mbar_init(bar(B_QFULL + 0), 1);
    mbar_init(bar(B_QFULL + 1), 1);
    for (int s = 0; s < ATT_STAGES; ++s) {
      mbar_init(bar(B_KVFULL + s), 1);
      mbar_init(bar(B_KVEMPTY + s), 1);
      fills_issued[s] = 0;
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar(B_SFULL + t), 1);
      mbar_init(bar(B_PFULL + t), ATT_SM_WARPS / ATT_NQ);  // one arrival per softmax warp
      mbar_init(bar(B_ODONE + t), 1);
      mbar_init(bar(B_XCH + t), ATT_SM_WARPS / ATT_NQ);
    }
    mbar_init(bar(B_DRAIN), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (JHI > JLO) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&p.tm_q) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&p.tm_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&p.tm_v) : "memory");
#pragma unroll
      for (int t = 0; t < ATT_NQ; ++t) {
        if (rng[t].jhi > rng[t].jlo) {
          mbar_expect_tx(bar(B_QFULL + t), L::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < L::CHUNKS; ++c)
            tma_load_4d(sbase + L::Q_OFF + t * L::TILE_BYTES + c * L::CHUNK_BYTES, &p.tm_q,
                        bar(B_QFULL + t), c * 64, m0 + t * t_rows, h + t * t_head, b);
        }
      }
      // the ring is empty: its first round of fills waits for nobody
      const int first_round = min(ATT_STAGES, 2 * (JHI - JLO));
      for (int fill = 0; fill < first_round; ++fill) issue_fill(fill);
    }
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_holder)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  if (skip_launch) {  // nothing was started: give the TMEM columns back and leave
    if (warp == 0)
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"(512u)
                   : "memory");
    return;
  }

  if (warp == ATT_SM_WARPS) {
    // =========================== TMA producer =========================================
    if (lane == 0 && JHI > JLO) {
      // Q and the first round of the ring were issued before the CTA-wide sync
      const int total = 2 * (JHI - JLO);
      bool ok = true;
      for (int fill = ATT_STAGES; fill < total && ok; ++fill) {
        const uint32_t par = ((fill / ATT_STAGES) & 1) ^ 1;
        ok = mbar_wait(bar(B_KVEMPTY + fill % ATT_STAGES), par, abort_flag, p.status,
                       ATT_ST_PRODUCER);
        if (ok) issue_fill(fill);
      }
    }
  } else if (warp == ATT_SM_WARPS + 1) {
    // =========================== MMA issuer ===========================================
    if (lane == 0 && JHI > JLO) {
      const uint32_t idesc_qk = make_idesc(BF16 ? 1 : 0, ATT_BM, ATT_BN, 0, 0);
      const uint32_t idesc_pv = make_idesc(BF16 ? 1 : 0, ATT_BM, D, 0, 1);
      static_assert((ATT_STAGES & (ATT_STAGES - 1)) == 0, "ring depth must be a power of two");
      // This thread sits between the softmax warps and the tensor pipe: every cycle it spends
      // between two groups of MMAs is a cycle the pipe idles once its short queue has drained
      // (the same 32 MMAs per KV tile issued from a loop with per-tile state in arrays, lambdas
      // and modulo arithmetic ran at 1.40 PFLOP/s with nothing to wait for; from straight-line
      // code on scalars at 1.83). So: scalars only, one flat loop, both K/V waits up front.
      const int jlo0 = rng[0].jlo, jhi0 = rng[0].jhi, jlo1 = rng[1].jlo, jhi1 = rng[1].jhi;
      // Descriptors differ only in their 14-bit start-address field (address >> 4), which is
      // the low part of the low word: build the constant part once and add offsets with one
      // 32-bit add per operand.
      const uint64_t desc_k_major = make_desc(0, 16, 1024);               // K-major, SBO 1 KB
      const uint64_t desc_mn_major = make_desc(0, L::CHUNK_BYTES, 1024);  // MN-major V
      const uint32_t dk_hi = static_cast<uint32_t>(desc_k_major >> 32);
      const uint32_t dv_hi = static_cast<uint32_t>(desc_mn_major >> 32);
      constexpr uint32_t T16 = L::TILE_BYTES >> 4;
      const uint32_t q_lo = static_cast<uint32_t>(desc_k_major) + ((sbase + L::Q_OFF) >> 4);
      const uint32_t k_lo = static_cast<uint32_t>(desc_k_major) + ((sbase + L::KV_OFF) >> 4);
      const uint32_t v_lo = static_cast<uint32_t>(desc_mn_major) + ((sbase + L::KV_OFF) >> 4);
      auto desc_of = [](uint32_t lo, uint32_t hi) {
        return (static_cast<uint64_t>(hi) << 32) | lo;
      };
      auto wait = [&](int b, uint32_t parity) {
        return mbar_wait(bar(b), parity, abort_flag, p.status, ATT_ST_MMA);
      };
      bool ok = true;
      uint32_t ppar0 = 0, ppar1 = 0;  // parity of the next P hand-over per Q tile
      // a Q tile is waited for right before its first Q K^T (the second tile lands some 700
      // cycles after the first); the flags only exist in the general rounds
      bool q0_ready = false, q1_ready = false;

      // O_t += P_t V (P from TMEM, V MN-major from ring stage `vst`); `acc` = 0 clears O first
      auto pv = [&](int t, uint32_t vst, uint32_t acc) {
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + 2 * ATT_BN + t * ATT_BN;
        const uint32_t a_tmem = tmem_base + t * ATT_BN;
#pragma unroll
        for (int kk = 0; kk < ATT_BN / 16; ++kk)
          mma_ts(d_tmem, a_tmem + kk * 8, desc_of(vst + kk * (2048 >> 4), dv_hi), idesc_pv,
                 kk == 0 ? acc : 1u);
      };
      // S_t = Q_t K^T (both operands K-major in shared memory), then announce S_t
      auto qk = [&](int t, uint32_t kst) {
        tc_fence_after();
        const uint32_t qst = q_lo + t * T16;
        const uint32_t d_tmem = tmem_base + t * ATT_BN;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk / 4) * L::CHUNK_BYTES + (kk % 4) * 32) >> 4;
          if (kk == 0)
            mma_ss_first(d_tmem, desc_of(qst + off, dk_hi), desc_of(kst + off, dk_hi), idesc_qk);
          else
            mma_ss_acc(d_tmem, desc_of(qst + off, dk_hi), desc_of(kst + off, dk_hi), idesc_qk);
        }
        tc_commit(bar(B_SFULL + t));
      };

      // The O accumulator is announced once, after the last P V of a Q tile: before that the
      // softmax warps learn of a finished P V from the next S (its commit covers everything
      // issued earlier), so the rescale of O needs no barrier of its own.
      // Round j issues P V of KV tile j and Q K^T of tile j + 1 for each Q tile that has them;
      // the first round (j = JLO - 1) is the prologue, S(JLO) alone. Ring fills: K(j) is fill
      // 2 (j - JLO), V(j) the one after.
      // Round r (-1 .. n - 1) issues P V of the r-th visited KV tile and Q K^T of the next one;
      // the visiting order is ascending or descending (reverse_kv). `STEADY` rounds (both Q
      // tiles have this KV tile and the next, neither is at its first): every test below is a
      // compile-time constant and what is left is waits, MMAs, commits.
      const int n_rounds = JHI - JLO;
      auto run = [&](auto rev_tag) {
      constexpr bool rev = decltype(rev_tag)::value;
      const int first0 = rev ? jhi0 - 1 : jlo0, last0 = rev ? jlo0 : jhi0 - 1;
      const int first1 = rev ? jhi1 - 1 : jlo1, last1 = rev ? jlo1 : jhi1 - 1;
      auto round = [&](int r, auto steady_tag) {
        constexpr bool STEADY = decltype(steady_tag)::value;
        const int f = 2 * r;  // ring fills: K of visit r is fill 2r, V the one after
        const bool has_pv = STEADY || r >= 0, has_qk = STEADY || r + 1 < n_rounds;
        const int jp = rev ? JHI - 1 - r : JLO + r;  // KV tile of the P V
        const int jq = rev ? jp - 1 : jp + 1;        // KV tile of the next Q K^T
        const uint32_t fv = static_cast<uint32_t>(f + 1), fk = static_cast<uint32_t>(f + 2);
        const uint32_t sv = fv & (ATT_STAGES - 1), sk = fk & (ATT_STAGES - 1);
        if (has_pv) ok = wait(B_KVFULL + sv, (fv / ATT_STAGES) & 1);
        if (ok && has_qk) ok = wait(B_KVFULL + sk, (fk / ATT_STAGES) & 1);
        const uint32_t vst = v_lo + sv * T16, kst = k_lo + sk * T16;
        if (ok && (STEADY || (has_pv && jp >= jlo0 && jp < jhi0))) {
          ok = wait(B_PFULL + 0, ppar0);
          ppar0 ^= 1u;
          if (ok) {
            pv(0, vst, (STEADY || jp != first0) ? 1u : 0u);
            if (!STEADY && jp == last0) tc_commit(bar(B_ODONE + 0));
          }
        }
        if (ok && (STEADY || (has_qk && jq >= jlo0 && jq < jhi0))) {
          if (!STEADY && !q0_ready) {
            ok = wait(B_QFULL + 0, 0);
            q0_ready = true;
          }
          if (ok) qk(0, kst);
        }
        if (ok && (STEADY || (has_pv && jp >= jlo1 && jp < jhi1))) {
          ok = wait(B_PFULL + 1, ppar1);
          ppar1 ^= 1u;
          if (ok) {
            pv(1, vst, (STEADY || jp != first1) ? 1u : 0u);
            if (!STEADY && jp == last1) tc_commit(bar(B_ODONE + 1));
          }
        }
        if (ok && (STEADY || (has_qk && jq >= jlo1 && jq < jhi1))) {
          if (!STEADY && !q1_ready) {
            ok = wait(B_QFULL + 1, 0);
            q1_ready = true;
          }
          if (ok) qk(1, kst);
        }
        if (ok) {
          if (has_pv) tc_commit(bar(B_KVEMPTY + sv));
          if (has_qk) tc_commit(bar(B_KVEMPTY + sk));
        }
      };
      // steady rounds: the P V tile lies in (max(jlo), min(jhi) - 1) and is not a Q tile's first
      // or last, the next tile is inside both ranges
      const int lo_s = max(jlo0, jlo1) + 1, hi_s = min(jhi0, jhi1) - 2;  // jp in [lo_s, hi_s]
      const int rs = rev ? JHI - 1 - hi_s : lo_s - JLO;                  // first steady round
      const int re = rev ? JHI - 1 - lo_s + 1 : hi_s - JLO + 1;          // one past the last
      int r = -1;
#pragma unroll 1
      for (; r < n_rounds && r < rs && ok; ++r) round(r, std::false_type{});
#pragma unroll 1
      for (; r < re && ok; ++r) round(r, std::true_type{});
#pragma unroll 1
      for (; r < n_rounds && ok; ++r) round(r, std::false_type{});
      };
      if (p.reverse_kv) run(std::true_type{});
      else run(std::false_type{});
      if (!ok) {
        // drain whatever was issued before giving up
        tc_commit(bar(B_DRAIN));
        const uint64_t t0 = global_ns();
        while (!mbar_try_wait(bar(B_DRAIN), 0) && global_ns() - t0 < ATT_WAIT_NS) {
        }
      }
    }
  } else {
    // =========================== softmax groups =======================================
    // 8 warps per Q tile. Warp w of the tile owns 16 rows: TMEM lanes 32*(w%4) + 16*(w/4) .. +15,
    // read with the 16x256b shape, so that each row is spread over the four threads of a quad
    // (32 of the 128 score columns each) and each thread works on two rows (lane t/4 and
    // t/4 + 8). Row maxima need two quad shuffles and no traffic between warps; the partial row
    // sums are only combined in the epilogue. The epilogue itself re-partitions the tile (one
    // row per thread, half of the head dim) to write 128 contiguous bytes per thread, and gets
    // the row sums through shared memory once per CTA.
    constexpr int WPT = ATT_SM_WARPS / ATT_NQ;              // softmax warps per Q tile
    const int t = warp / WPT;                               // Q tile of this warp
    const int wq = warp & 3;                                // TMEM lane quarter of this warp
    const int sub = (warp >> 2) & 1;                        // which 16 lanes of the quarter
    const int q4 = lane & 3;                                // position in the quad
    const int rl = wq * 32 + sub * 16 + (lane >> 2);        // first row (second is rl + 8)
    const int row0 = m0 + t * t_rows;                       // first row of the Q tile
    const int hq = h + t * t_head;                          // query head of the Q tile
    const int row1 = min(p.Sq, row0 + ATT_BM) - 1;
    const uint32_t lane16 = static_cast<uint32_t>(wq * 32 + sub * 16) << 16;
    const uint32_t s_addr = tmem_base + lane16 + t * ATT_BN;
    const uint32_t o_addr16 = tmem_base + lane16 + 2 * ATT_BN + t * ATT_BN;
    const int n_it = rng[t].jhi - rng[t].jlo;
    float* xch = reinterpret_cast<float*>(smem + L::XCH_OFF) + t * 2 * ATT_BM;  // [2][128]

    int row_g[2], hi_i[2], lo_i[2];  // global row and its visible key range lo <= col <= hi
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      row_g[hr] = row0 + rl + 8 * hr;
      hi_i[hr] = p.Sk - 1;
      lo_i[hr] = 0;
      if (p.causal) hi_i[hr] = min(hi_i[hr], row_g[hr]);
      if (p.win_right >= 0) hi_i[hr] = min(hi_i[hr], row_g[hr] + p.win_right);
      if (p.win_left >= 0) lo_i[hr] = max(0, row_g[hr] - p.win_left);
    }
    int hi_min = p.Sk - 1, lo_max = 0;  // tile-level bounds (first / last row of the tile)
    if (p.causal) hi_min = min(hi_min, row0);
    if (p.win_right >= 0) hi_min = min(hi_min, row0 + p.win_right);
    if (p.win_left >= 0) lo_max = max(0, row1 - p.win_left);

    const float sl2 = p.scale_log2;
    const float slope2 = p.slopes ? p.slopes[hq] * 1.4426950408889634f : 0.0f;
    const bool has_alibi = p.slopes != nullptr;
    const bool has_bias = BIAS && p.bias_kind != 0;
    const bool has_drop = BIAS && p.drop_thr != 0u;
    // rows of the dense mask that this thread's two score rows read (valid rows only)
    const uint8_t* brow[2] = {nullptr, nullptr};
    if (has_bias) {
      const int esz = p.bias_kind == 1 ? 4 : 2;
#pragma unroll
      for (int hr = 0; hr < 2; ++hr)
        if (row0 + rl + 8 * hr < p.Sq)
          brow[hr] = reinterpret_cast<const uint8_t*>(p.bias) +
                     esz * (b * p.bias_sb + hq * p.bias_sh +
                            static_cast<long long>(row0 + rl + 8 * hr) * p.bias_sq);
    }

    const int j_first = p.reverse_kv ? rng[t].jhi - 1 : rng[t].jlo;  // first KV tile visited
    float m_run[2] = {-INFINITY, -INFINITY};  // reference max (log2 domain) per row
    float l_run[2] = {0.0f, 0.0f};            // this thread's share of the row sums
    bool ok = true;

    for (int itn = 0; itn < n_it && ok; ++itn) {
      const int j = j_first + itn * kv_step;
      const int c0 = j * ATT_BN;  // first key of the tile
      ok = __all_sync(0xffffffffu,
                      mbar_wait(bar(B_SFULL + t), itn & 1, abort_flag, p.status, ATT_ST_SOFTMAX));
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[64];  // sr[4g + 2hr + e] = S(row hr, column 8g + 2*q4 + e)
      tmem_ld_16x256b_x16(s_addr, sr);
      tmem_wait_ld();

      const bool need_mask = (c0 + ATT_BN - 1 > hi_min) || (c0 < lo_max);
      // ALiBi on a tile that lies entirely on one side of the diagonal is linear in the
      // column: -slope*|i-j| = sgn*slope*(j-i). It then folds into the raw score as
      // t = s + (sgn*slope2/sl2)*c, and the per-tile, per-row constant `off` below.
      int alibi_sgn = 0;
      if (has_alibi) {
        // under a causal mask (or a window that ends at the query) every VISIBLE key is at or
        // before its query, on the diagonal tile too; hidden keys are masked anyway
        if (p.causal || p.win_right == 0 || c0 + ATT_BN - 1 <= row0) alibi_sgn = 1;
        else if (c0 >= row1) alibi_sgn = -1;          // every key at or after every query
      }
      // general path: a tile that straddles the diagonal under ALiBi, or a non-positive scale
      const bool general = (has_alibi && alibi_sgn == 0) || !(sl2 > 0.0f) || has_bias || has_drop;
      float m_tile[2] = {-INFINITY, -INFINITY};
      float off[2] = {0.0f, 0.0f};  // fast path: x = t * sl2 + off
      if (general) {
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
          const float fi = static_cast<float>(row_g[hr] - c0 - 2 * q4);
#pragma unroll
          for (int g = 0; g < 16; ++g) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int i = 4 * g + 2 * hr + e;
              float x = __uint_as_float(sr[i]) * sl2;
              if (has_alibi) x = fmaf(-slope2, fabsf(fi - static_cast<float>(8 * g + e)), x);
              if (has_bias) {
                const int col = c0 + 8 * g + 2 * q4 + e;
                if (brow[hr] != nullptr && col < p.Sk) {
                  float bv;
                  if (p.bias_kind == 1) bv = reinterpret_cast<const float*>(brow[hr])[col];
                  else if (BF16) bv = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(brow[hr])[col]);
                  else bv = __half2float(reinterpret_cast<const __half*>(brow[hr])[col]);
                  x = fmaf(bv, 1.4426950408889634f, x);  // -inf stays -inf
                }
              }
              if (need_mask) {
                const int col = c0 + 8 * g + 2 * q4 + e;
                if (col < lo_i[hr] || col > hi_i[hr]) x = -INFINITY;
              }
              sr[i] = __float_as_uint(x);
              m_tile[hr] = fmaxf(m_tile[hr], x);
            }
          }
        }
      } else {
        if (need_mask) {
          // boundary tile: hide keys outside [lo, hi] in the raw domain (sl2 > 0 keeps -inf
          // at -inf), then continue on the fast path
          // a tile is cut by the upper bound (diagonal), by the lower one (left edge of a
          // window), seldom by both: one comparison per score where one is enough
          const bool cut_hi = c0 + ATT_BN - 1 > hi_min, cut_lo = c0 < lo_max;
#pragma unroll
          for (int hr = 0; hr < 2; ++hr) {
            const int lo_c = lo_i[hr] - c0 - 2 * q4, hi_c = hi_i[hr] - c0 - 2 * q4;
            if (cut_hi && !cut_lo) {
#pragma unroll
              for (int g = 0; g < 16; ++g) {
#pragma unroll
                for (int e = 0; e < 2; ++e)
                  if (8 * g + e > hi_c) sr[4 * g + 2 * hr + e] = 0xff800000u;
              }
            } else if (cut_lo && !cut_hi) {
#pragma unroll
              for (int g = 0; g < 16; ++g) {
#pragma unroll
                for (int e = 0; e < 2; ++e)
                  if (8 * g + e < lo_c) sr[4 * g + 2 * hr + e] = 0xff800000u;
              }
            } else {
#pragma unroll
              for (int g = 0; g < 16; ++g) {
#pragma unroll
                for (int e = 0; e < 2; ++e)
                  if (8 * g + e < lo_c || 8 * g + e > hi_c) sr[4 * g + 2 * hr + e] = 0xff800000u;
              }
            }
          }
        }
        if (alibi_sgn != 0) {
          const float sk = static_cast<float>(alibi_sgn) * slope2;
          const float kc = __fdividef(sk, sl2);
#pragma unroll
          for (int hr = 0; hr < 2; ++hr)
            off[hr] = sk * static_cast<float>(c0 + 2 * q4 - row_g[hr]);
          // + kc * (8g + e), as packed adds of a running (column, column + 1) pair
          float2 cp = make_float2(0.0f, kc);
          const float2 step = make_float2(8.0f * kc, 8.0f * kc);
#pragma unroll
          for (int g = 0; g < 16; ++g) {
#pragma unroll
            for (int hr = 0; hr < 2; ++hr) {
              const float2 v = add2(make_float2(__uint_as_float(sr[4 * g + 2 * hr]),
                                                __uint_as_float(sr[4 * g + 2 * hr + 1])), cp);
              sr[4 * g + 2 * hr] = __float_as_uint(v.x);
              sr[4 * g + 2 * hr + 1] = __float_as_uint(v.y);
            }
            cp = add2(cp, step);
          }
        }
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
          float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
          for (int g = 0; g < 16; g += 2) {
            mx0 = max3(mx0, __uint_as_float(sr[4 * g + 2 * hr]), __uint_as_float(sr[4 * g + 2 * hr + 1]));
            mx1 = max3(mx1, __uint_as_float(sr[4 * g + 4 + 2 * hr]),
                       __uint_as_float(sr[4 * g + 5 + 2 * hr]));
          }
          const float mraw = fmaxf(mx0, mx1);
          m_tile[hr] = (mraw == -INFINITY) ? -INFINITY : fmaf(mraw, sl2, off[hr]);
        }
      }
      // the four threads of a quad hold the four column slices of the same two rows
#pragma unroll
      for (int hr = 0; hr < 2; ++hr) {
        m_tile[hr] = fmaxf(m_tile[hr], __shfl_xor_sync(0xffffffffu, m_tile[hr], 1));
        m_tile[hr] = fmaxf(m_tile[hr], __shfl_xor_sync(0xffffffffu, m_tile[hr], 2));
      }

      // lazy rescale: keep the old reference max unless the new one is much larger
      float factor[2] = {1.0f, 1.0f};
      bool rescale = false;
      float m_ref[2];
#pragma unroll
      for (int hr = 0; hr < 2; ++hr) {
        if (m_tile[hr] > m_run[hr] + ATT_LAZY_RESCALE ||
            (m_run[hr] == -INFINITY && m_tile[hr] > -INFINITY)) {
          factor[hr] = fast_exp2(m_run[hr] - m_tile[hr]);  // 0 when m_run == -inf
          rescale = rescale || (itn > 0);
          m_run[hr] = m_tile[hr];
          l_run[hr] *= factor[hr];
        }
        m_ref[hr] = (m_run[hr] == -INFINITY) ? 0.0f : m_run[hr];
      }

      // P = exp2(x - m_ref), packed to 16-bit pairs IN PLACE: sr[2g + hr] = P(row hr, column
      // 4g + q4). Slot 2g + hr never lies ahead of the scores still to be read (4g + 2hr ..).
      float2 lsum[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
      if (general) {
        uint4 rnd[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
#pragma unroll
        for (int g = 0; g < 16; ++g) {
#pragma unroll
          for (int hr = 0; hr < 2; ++hr) {
            float p0 = fast_exp2(__uint_as_float(sr[4 * g + 2 * hr]) - m_ref[hr]);
            float p1 = fast_exp2(__uint_as_float(sr[4 * g + 2 * hr + 1]) - m_ref[hr]);
            lsum[hr].x += p0;  // the normaliser sums the undropped probabilities
            lsum[hr].y += p1;
            if (has_drop) {
              // one generator call per 16 keys: group g (8 keys) and g + 1 share it
              if ((g & 1) == 0)
                rnd[hr] = philox4x32_10(
                    make_uint4(static_cast<uint32_t>((c0 + 8 * g) >> 4),
                               static_cast<uint32_t>(row_g[hr]),
                               static_cast<uint32_t>(b * p.Hq + hq), p.drop_offset),
                    p.seed_lo, p.seed_hi);
              // keys 8g + 2*q4 + {0, 1} of the tile = bytes 8(g&1) + 2*q4 + {0, 1} of the block
              const int lc = 8 * (g & 1) + 2 * q4;
              const uint32_t* rw = reinterpret_cast<const uint32_t*>(&rnd[hr]);
              const uint32_t word = (lc < 4) ? rw[0] : (lc < 8) ? rw[1] : (lc < 12) ? rw[2] : rw[3];
              const uint32_t two = word >> (8 * (lc & 3));  // lc is even: both bytes in one word
              if ((two & 0xffu) < p.drop_thr) p0 = 0.0f;
              if (((two >> 8) & 0xffu) < p.drop_thr) p1 = 0.0f;
            }
            sr[2 * g + hr] = pack16<BF16>(p0, p1);
          }
        }
      } else {
        const float2 sc2 = make_float2(sl2, sl2);
        const float2 nm2[2] = {make_float2(off[0] - m_ref[0], off[0] - m_ref[0]),
                               make_float2(off[1] - m_ref[1], off[1] - m_ref[1])};
#pragma unroll
        for (int g = 0; g < 16; ++g) {
#pragma unroll
          for (int hr = 0; hr < 2; ++hr) {
            const float2 x = fma2(make_float2(__uint_as_float(sr[4 * g + 2 * hr]),
                                              __uint_as_float(sr[4 * g + 2 * hr + 1])),
                                  sc2, nm2[hr]);
            const float2 pe = make_float2(fast_exp2(x.x), fast_exp2(x.y));
            lsum[hr] = add2(lsum[hr], pe);
            sr[2 * g + hr] = pack16<BF16>(pe.x, pe.y);
          }
        }
      }
      l_run[0] += lsum[0].x + lsum[0].y;
      l_run[1] += lsum[1].x + lsum[1].y;
      tmem_st_16x128b_x16(s_addr, sr);

      // O rescale (rare after the first tiles): needs the previous P V of this tile done, which
      // the S of this iteration implies (its commit was issued after that P V)
      if (__any_sync(0xffffffffu, rescale)) {
        {
          uint32_t orr[D / 2];  // same fragment layout as the scores
          if constexpr (D == 128) tmem_ld_16x256b_x16(o_addr16, orr);
          else tmem_ld_16x256b_x8(o_addr16, orr);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < D / 2; ++i)
            orr[i] = __float_as_uint(__uint_as_float(orr[i]) * factor[(i >> 1) & 1]);
          if constexpr (D == 128) tmem_st_16x256b_x16(o_addr16, orr);
          else tmem_st_16x256b_x8(o_addr16, orr);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_PFULL + t));
    }

    // ---- epilogue: O / l -> global --------------------------------------------------
    // Row statistics go through shared memory once: xch[0][row] = row sum, xch[1][row] = max.
    if (ok) {
#pragma unroll
      for (int hr = 0; hr < 2; ++hr) {
        float l = l_run[hr];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (q4 == 0) {
          xch[rl + 8 * hr] = l;
          xch[ATT_BM + rl + 8 * hr] = m_run[hr];
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_XCH + t));
      ok = __all_sync(0xffffffffu,
                      mbar_wait(bar(B_XCH + t), 0, abort_flag, p.status, ATT_ST_SOFTMAX));
    }
    if (ok && n_it > 0) {
      ok = __all_sync(0xffffffffu,
                      mbar_wait(bar(B_ODONE + t), 0, abort_flag, p.status, ATT_ST_SOFTMAX));
      tc_fence_after();
    }
    if (ok) {
      // one row per thread (TMEM lane 32*wq + lane), columns [OC*sub, OC*sub + OC) of the head
      constexpr int OC = D / 2;
      const int r = wq * 32 + lane;
      const int row = row0 + r;
      const float l_row = xch[r];
      const float m_row = xch[ATT_BM + r];
      float inv = (n_it > 0 && l_row > 0.0f) ? __fdividef(1.0f, l_row) : 0.0f;
      if (BIAS && p.drop_thr != 0u) inv *= p.drop_scale;  // kept probabilities count 1 / (1 - p)
      const uint32_t o_addr = tmem_base + (static_cast<uint32_t>(wq * 32) << 16) + 2 * ATT_BN +
                              t * ATT_BN + sub * OC;
      uint8_t* orow = reinterpret_cast<uint8_t*>(p.out) +
                      2ll * (b * p.o_stride_b + static_cast<long long>(row) * p.o_stride_s +
                             hq * p.o_stride_h + sub * OC);
#pragma unroll
      for (int cc = 0; cc < OC; cc += 32) {
        uint32_t orr[32];
        if (n_it > 0) {
          tmem_ld32<0>(o_addr + cc, orr);  // warp-collective: executed by every lane
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) orr[e] = 0u;
        }
        if (row < p.Sq) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 v;
            uint32_t* vv = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float a0 = __uint_as_float(orr[e + 2 * q]) * inv;
              const float a1 = __uint_as_float(orr[e + 2 * q + 1]) * inv;
              vv[q] = pack16<BF16>(a0, a1);
            }
            *reinterpret_cast<uint4*>(orow + 2 * (cc + e)) = v;
          }
        }
      }
      if (p.lse && sub == 0 && row < p.Sq) {
        const float lse = (n_it > 0 && l_row > 0.0f)
                              ? (m_row + log2f(l_row)) * 0.6931471805599453f
                              : -INFINITY;
        p.lse[b * p.lse_stride_b + hq * p.lse_stride_h + row] = lse;
      }
    }
  }

  // ------------------------------- teardown -------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // make sure no bulk copy of this CTA is still in flight before shared memory is released
    for (int s = 0; s < ATT_STAGES; ++s) {
      const int n = fills_issued[s];
      if (n > 0) {
        bool done = false;
        const uint64_t t0 = global_ns();
        while (!(done = mbar_try_wait(bar(B_KVFULL + s), (n - 1) & 1)) &&
               global_ns() - t0 < ATT_WAIT_NS) {
        }
        if (!done) atomicOr(p.status, ATT_ST_DRAIN);
      }
    }
    for (int t = 0; t < ATT_NQ; ++t)
      if (rng[t].jhi > rng[t].jlo) {
        bool done = false;
        const uint64_t t0 = global_ns();
        while (!(done = mbar_try_wait(bar(B_QFULL + t), 0)) && global_ns() - t0 < ATT_WAIT_NS) {
        }
        if (!done) atomicOr(p.status, ATT_ST_DRAIN);
      }
  }
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(512u)
                 : "memory");
  }
}

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;  // host threads that race on the first call all see the result
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// (D, S, H, B) view of a (B, S, H, D) tensor with element strides (b, s, h); box = 64 x 128.
// Dims with stride 0 (broadcast) are collapsed to size 1 by the caller.
static int make_map(CUtensorMap* tm, const void* base, int is_bf16, int64_t D, int64_t S,
                    int64_t H, int64_t B, int64_t sb, int64_t ss, int64_t sh) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return TRX_ERR_CUDA;
  if (!aligned_to(base, 16)) return TRX_ERR_ALIGNMENT;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S),
                        static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(B)};
  // size-1 dims may carry any stride; give them a legal one
  if (S == 1) ss = D;
  if (H == 1) sh = ss * S;
  if (B == 1) sb = (sh * H > ss * S) ? sh * H : ss * S;
  if (ss < D || sh <= 0 || sb <= 0) return TRX_ERR_STRIDE;
  if ((ss * 2) % 16 || (sh * 2) % 16 || (sb * 2) % 16) return TRX_ERR_ALIGNMENT;
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(ss * 2), static_cast<cuuint64_t>(sh * 2),
                           static_cast<cuuint64_t>(sb * 2)};
  for (int i = 0; i < 3; ++i)
    if (strides[i] >= (1ull << 40)) return TRX_ERR_STRIDE;
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(ATT_BM), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(tm, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                   4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? TRX_OK : TRX_ERR_CUDA;
}

template <int D, bool BF16, bool BIAS>
static int launch_attn_bias(const AttnParams& p, cudaStream_t stream) {
  // The attribute is set once per device; host threads that race on the first call each set
  // the same value (the call is idempotent) and publish the flag atomically.
  static std::atomic<bool> configured[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return TRX_ERR_CUDA;
  const bool cacheable = dev >= 0 && dev < 64;
  if (!cacheable || !configured[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<D, BF16, BIAS>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             AttnSmem<D>::DYN_BYTES) != cudaSuccess)
      return TRX_ERR_CUDA;
    if (cacheable) configured[dev].store(true, std::memory_order_release);
  }
  const int rows_per_cta = p.pair_heads ? ATT_BM : ATT_NQ * ATT_BM;
  const int mblocks = (p.Sq + rows_per_cta - 1) / rows_per_cta;
  dim3 grid(mblocks, p.pair_heads ? p.Hq / 2 : p.Hq, p.B);
  attn_fwd_kernel<D, BF16, BIAS><<<grid, ATT_THREADS, AttnSmem<D>::DYN_BYTES, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? TRX_OK : TRX_ERR_CUDA;
}

template <int D, bool BF16>
static int launch_attn(const AttnParams& p, cudaStream_t stream) {
  return (p.bias_kind != 0 || p.drop_thr != 0u) ? launch_attn_bias<D, BF16, true>(p, stream)
                                                : launch_attn_bias<D, BF16, false>(p, stream);
}

}  // namespace trx

using namespace trx;

extern "C" size_t trx_attn_workspace_bytes(void) { return 256; }

// Validation and parameter block shared by the attention entry points; nothing is enqueued.
// `bias` may be null (no dense mask). Returns TRX_OK with *nothing_to_do set for empty problems.
static int attn_fwd_prepare(AttnParams& p, bool* nothing_to_do, const void* q, const void* k,
                            const void* v, void* out, float* lse_or_null,
                            const float* slopes_or_null, const void* bias, int bias_dtype,
                            const int64_t* bias_strides, int64_t B, int64_t Sq, int64_t Sk,
                            int64_t Hq, int64_t Hk, int64_t D, const int64_t q_strides[3],
                            const int64_t k_strides[3], const int64_t v_strides[3],
                            const int64_t o_strides[3], float scale, int causal,
                            int64_t window_left, int64_t window_right, int dtype,
                            void* workspace, size_t workspace_bytes, float dropout_p = 0.0f,
                            uint64_t seed = 0, uint32_t offset = 0) {
  *nothing_to_do = false;
  if (!(dropout_p >= 0.0f) || !(dropout_p < 1.0f)) return TRX_ERR_SHAPE;
  if (dtype != TRX_BF16 && dtype != TRX_F16) return TRX_ERR_DTYPE;
  if (bias) {
    if (bias_dtype != TRX_F32 && bias_dtype != dtype) return TRX_ERR_DTYPE;
    if (!bias_strides) return TRX_ERR_NULL_POINTER;
    if (bias_strides[0] < 0 || bias_strides[1] < 0 || bias_strides[2] < Sk)
      return TRX_ERR_STRIDE;
  }
  if (B < 0 || Sq < 0 || Sk < 0 || Hq <= 0 || Hk <= 0 || D <= 0) return TRX_ERR_SHAPE;
  if (Hq % Hk != 0) return TRX_ERR_SHAPE;
  if (D != 64 && D != 128) return TRX_ERR_UNSUPPORTED;
  if ((window_left < 0) != (window_right < 0)) return TRX_ERR_SHAPE;
  if (B == 0 || Sq == 0) {
    *nothing_to_do = true;
    return TRX_OK;
  }
  if (!q || !out || !q_strides || !k_strides || !v_strides || !o_strides)
    return TRX_ERR_NULL_POINTER;
  if (Sk > 0 && (!k || !v)) return TRX_ERR_NULL_POINTER;
  if (!workspace) return TRX_ERR_WORKSPACE;
  if (workspace_bytes < trx_attn_workspace_bytes() || !aligned_to(workspace, 16))
    return TRX_ERR_WORKSPACE;
  if (Sq >= (1ll << 30) || Sk >= (1ll << 30) || Hq > 65535 || B > 65535)
    return TRX_ERR_SHAPE;
  if (!aligned_to(out, 16) || o_strides[0] % 8 || o_strides[1] % 8 || o_strides[2] % 8)
    return TRX_ERR_ALIGNMENT;
  for (int i = 0; i < 3; ++i)
    if (q_strides[i] < 0 || k_strides[i] < 0 || v_strides[i] < 0 || o_strides[i] < 0)
      return TRX_ERR_STRIDE;

  p = AttnParams{};
  const int is_bf16 = dtype == TRX_BF16;
  int rc = make_map(&p.tm_q, q, is_bf16, D, Sq, Hq, B, q_strides[0], q_strides[1], q_strides[2]);
  if (rc != TRX_OK) return rc;
  // Broadcast (stride-0) head or batch dims of k / v collapse to extent 1.
  const int64_t Sk_map = Sk > 0 ? Sk : 1;
  const void* kk = Sk > 0 ? k : q;
  const void* vv = Sk > 0 ? v : q;
  const bool k_hb = (Hk > 1 && k_strides[2] == 0), v_hb = (Hk > 1 && v_strides[2] == 0);
  const bool k_bb = (B > 1 && k_strides[0] == 0), v_bb = (B > 1 && v_strides[0] == 0);
  rc = make_map(&p.tm_k, kk, is_bf16, D, Sk_map, k_hb ? 1 : Hk, k_bb ? 1 : B, k_strides[0],
                k_strides[1], k_strides[2]);
  if (rc != TRX_OK) return rc;
  rc = make_map(&p.tm_v, vv, is_bf16, D, Sk_map, v_hb ? 1 : Hk, v_bb ? 1 : B, v_strides[0],
                v_strides[1], v_strides[2]);
  if (rc != TRX_OK) return rc;
  p.out = out;
  p.lse = lse_or_null;
  p.slopes = slopes_or_null;
  p.status = reinterpret_cast<unsigned int*>(workspace);
  p.B = static_cast<int>(B);
  p.Sq = static_cast<int>(Sq);
  p.Sk = static_cast<int>(Sk);
  p.Hq = static_cast<int>(Hq);
  const int group = static_cast<int>(Hq / Hk);
  p.k_hdiv = k_hb ? static_cast<int>(Hq) : group;
  p.v_hdiv = v_hb ? static_cast<int>(Hq) : group;
  p.k_bmul = k_bb ? 0 : 1;
  p.v_bmul = v_bb ? 0 : 1;
  p.o_stride_b = o_strides[0];
  p.o_stride_s = o_strides[1];
  p.o_stride_h = o_strides[2];
  p.lse_stride_b = Hq * Sq;
  p.lse_stride_h = Sq;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal ? 1 : 0;
  p.win_left = window_left < 0 ? -1 : static_cast<int>(window_left > (1ll << 29) ? (1ll << 29) : window_left);
  p.win_right = window_right < 0 ? -1 : static_cast<int>(window_right > (1ll << 29) ? (1ll << 29) : window_right);
  p.is_bf16 = is_bf16;
  p.reverse_m = causal ? 1 : 0;
  // ALiBi under a causal mask (or a window that ends at the query): the bias grows with the key
  // index, so walking the keys forwards raises the row maximum by slope * 128 on every tile and
  // with it comes a rescale of the whole O accumulator; walking them backwards the first tile
  // holds the maximum and later ones never beat it by more than the lazy-rescale margin.
  p.reverse_kv = (slopes_or_null != nullptr && (causal || window_right == 0)) ? 1 : 0;
  // two query heads per CTA when each pair (2i, 2i + 1) reads one kv head in K and in V
  p.pair_heads = (Hq % 2 == 0 && p.k_hdiv % 2 == 0 && p.v_hdiv % 2 == 0) ? 1 : 0;
  if (bias && Sk > 0) {
    p.bias = bias;
    p.bias_sb = bias_strides[0];
    p.bias_sh = bias_strides[1];
    p.bias_sq = bias_strides[2];
    p.bias_kind = bias_dtype == TRX_F32 ? 1 : 2;
  }
  if (dropout_p > 0.0f) {
    // the drop probability is realised in steps of 1/256 (one random byte per element)
    unsigned thr = static_cast<unsigned>(dropout_p * 256.0f + 0.5f);
    thr = thr < 1u ? 1u : (thr > 255u ? 255u : thr);
    p.drop_thr = thr;
    p.drop_scale = 256.0f / static_cast<float>(256u - thr);
    p.seed_lo = static_cast<unsigned>(seed & 0xffffffffull);
    p.seed_hi = static_cast<unsigned>(seed >> 32);
    p.drop_offset = offset;
  }
  return TRX_OK;
}

static int attn_fwd_launch(const AttnParams& p, int64_t D, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D == 128) return p.is_bf16 ? launch_attn<128, true>(p, s) : launch_attn<128, false>(p, s);
  return p.is_bf16 ? launch_attn<64, true>(p, s) : launch_attn<64, false>(p, s);
}

static int attn_fwd_impl(const void* q, const void* k, const void* v, void* out,
                         float* lse_or_null, const float* slopes_or_null, const void* bias,
                         int bias_dtype, const int64_t* bias_strides, int64_t B, int64_t Sq,
                         int64_t Sk, int64_t Hq, int64_t Hk, int64_t D,
                         const int64_t q_strides[3], const int64_t k_strides[3],
                         const int64_t v_strides[3], const int64_t o_strides[3], float scale,
                         int causal, int64_t window_left, int64_t window_right, int dtype,
                         void* workspace, size_t workspace_bytes, void* stream,
                         float dropout_p = 0.0f, uint64_t seed = 0, uint32_t offset = 0) {
  AttnParams p;
  bool nothing_to_do = false;
  const int rc = attn_fwd_prepare(p, &nothing_to_do, q, k, v, out, lse_or_null, slopes_or_null,
                                  bias, bias_dtype, bias_strides, B, Sq, Sk, Hq, Hk, D, q_strides,
                                  k_strides, v_strides, o_strides, scale, causal, window_left,
                                  window_right, dtype, workspace, workspace_bytes, dropout_p, seed,
                                  offset);
  if (rc != TRX_OK || nothing_to_do) return rc;
  return attn_fwd_launch(p, D, stream);
}

// Status word of a workspace, without a synchronisation. `host_word` is host memory the caller
// keeps alive (pinned memory makes the copy asynchronous). If the word copied there by an
// earlier call is already non-zero, a kernel gave up on a bounded wait: TRX_ERR_DEVICE_STATUS,
// nothing is enqueued. Otherwise a 4-byte copy of the device word into *host_word is enqueued
// on `stream`, behind the launches already there.
extern "C" int trx_attn_status(const void* workspace, unsigned int* host_word, void* stream) {
  if (!workspace || !host_word) return TRX_ERR_NULL_POINTER;
  if (*reinterpret_cast<volatile unsigned int*>(host_word) != 0u) return TRX_ERR_DEVICE_STATUS;
  if (cudaMemcpyAsync(host_word, workspace, sizeof(unsigned int), cudaMemcpyDeviceToHost,
                      static_cast<cudaStream_t>(stream)) != cudaSuccess)
    return TRX_ERR_CUDA;
  return TRX_OK;
}

extern "C" int trx_attn_fwd(const void* q, const void* k, const void* v, void* out,
                            float* lse_or_null, const float* slopes_or_null, int64_t B, int64_t Sq,
                            int64_t Sk, int64_t Hq, int64_t Hk, int64_t D,
                            const int64_t q_strides[3], const int64_t k_strides[3],
                            const int64_t v_strides[3], const int64_t o_strides[3], float scale,
                            int causal, int64_t window_left, int64_t window_right, int dtype,
                            void* workspace, size_t workspace_bytes, void* stream) {
  return attn_fwd_impl(q, k, v, out, lse_or_null, slopes_or_null, nullptr, 0, nullptr, B, Sq, Sk,
                       Hq, Hk, D, q_strides, k_strides, v_strides, o_strides, scale, causal,
                       window_left, window_right, dtype, workspace, workspace_bytes, stream);
}

extern "C" int trx_attn_fwd_mask(const void* q, const void* k, const void* v, void* out,
                                 float* lse_or_null, const float* slopes_or_null,
                                 const void* mask, int mask_dtype, const int64_t mask_strides[3],
                                 int64_t B, int64_t Sq, int64_t Sk, int64_t Hq, int64_t Hk,
                                 int64_t D, const int64_t q_strides[3],
                                 const int64_t k_strides[3], const int64_t v_strides[3],
                                 const int64_t o_strides[3], float scale, int causal,
                                 int64_t window_left, int64_t window_right, int dtype,
                                 void* workspace, size_t workspace_bytes, void* stream) {
  if (!mask) return TRX_ERR_NULL_POINTER;
  return attn_fwd_impl(q, k, v, out, lse_or_null, slopes_or_null, mask, mask_dtype, mask_strides,
                       B, Sq, Sk, Hq, Hk, D, q_strides, k_strides, v_strides, o_strides, scale,
                       causal, window_left, window_right, dtype, workspace, workspace_bytes, stream);
}

extern "C" int trx_attn_fwd_dropout(const void* q, const void* k, const void* v, void* out,
                                    float* lse_or_null, const float* slopes_or_null,
                                    const void* mask_or_null, int mask_dtype,
                                    const int64_t mask_strides[3], int64_t B, int64_t Sq,
                                    int64_t Sk, int64_t Hq, int64_t Hk, int64_t D,
                                    const int64_t q_strides[3], const int64_t k_strides[3],
                                    const int64_t v_strides[3], const int64_t o_strides[3],
                                    float scale, int causal, int64_t window_left,
                                    int64_t window_right, int dtype, float dropout_p,
                                    uint64_t seed, uint32_t offset, void* workspace,
                                    size_t workspace_bytes, void* stream) {
  return attn_fwd_impl(q, k, v, out, lse_or_null, slopes_or_null, mask_or_null, mask_dtype,
                       mask_strides, B, Sq, Sk, Hq, Hk, D, q_strides, k_strides, v_strides,
                       o_strides, scale, causal, window_left, window_right, dtype, workspace,
                       workspace_bytes, stream, dropout_p, seed, offset);
}

// ------------------------------------------------------------------------------------------
// Attention without a caller-supplied workspace
// ------------------------------------------------------------------------------------------
// Some hosts can hand this library pointers but cannot produce device memory of their own at
// call time: an inference-engine plugin whose memory plan was frozen when the engine was
// built and whose execute hook must not allocate, or a process in which a memory broker owns
// the whole device and hands out nothing on demand. For them the attention kernel's scratch
// (its 256-byte status / scheduler block) lives in the library image instead: one static
// array per loaded copy of the library, i.e. 256 bytes on every GPU that loads it, held until
// the process exits.
constexpr size_t ATT_STATIC_SCRATCH_BYTES = 256;
static __device__ __align__(256) unsigned char g_attn_static_scratch[ATT_STATIC_SCRATCH_BYTES];

// In host code `g_attn_static_scratch` is only a handle for the runtime, not an address a
// kernel could use; the device address is looked up once per device, with that device
// current, and cached here.
static std::mutex g_scratch_mutex;
static void* g_scratch_addr[64] = {nullptr};

static int static_scratch_for_current_device(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TRX_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_attn_static_scratch) != cudaSuccess || ptr == nullptr)
      return TRX_ERR_CUDA;
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return TRX_OK;
}

extern "C" int trx_attn_fwd_static_scratch(
    const void* q, const void* k, const void* v, void* out, float* lse_or_null,
    const float* slopes_or_null, int64_t B, int64_t Sq, int64_t Sk, int64_t Hq, int64_t Hk,
    int64_t D, const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
    const int64_t o_strides[3], float scale, int causal, int64_t window_left, int64_t window_right,
    int dtype, unsigned int* status_out_or_null, void* stream) {
  // The kernel's scratch need does not grow with the problem; should a later revision of the
  // kernel ever ask for more than the static array holds, refuse instead of overrunning it.
  if (trx_attn_workspace_bytes() > ATT_STATIC_SCRATCH_BYTES) return TRX_ERR_WORKSPACE;
  void* scratch = nullptr;
  const int rc = static_scratch_for_current_device(&scratch);
  if (rc != TRX_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Every argument is checked before anything is enqueued: an argument error leaves the stream
  // untouched.
  AttnParams p;
  bool nothing_to_do = false;
  const int checked = attn_fwd_prepare(
      p, &nothing_to_do, q, k, v, out, lse_or_null, slopes_or_null, nullptr, 0, nullptr, B, Sq, Sk,
      Hq, Hk, D, q_strides, k_strides, v_strides, o_strides, scale, causal, window_left,
      window_right, dtype, scratch, ATT_STATIC_SCRATCH_BYTES);
  if (checked != TRX_OK || nothing_to_do) return checked;
  // The array keeps whatever the previous call left in it. The status word must start at
  // zero (a non-zero word makes the kernel skip its work), so clear the block in stream order.
  if (cudaMemsetAsync(scratch, 0, ATT_STATIC_SCRATCH_BYTES, s) != cudaSuccess) return TRX_ERR_CUDA;
  const int launched = attn_fwd_launch(p, D, stream);
  if (launched != TRX_OK) return launched;
  // The one error that can follow the launch: the runtime refusing the 4-byte status copy. The
  // attention output is then valid all the same; only *status_out_or_null was not written.
  if (status_out_or_null != nullptr &&
      cudaMemcpyAsync(status_out_or_null, scratch, sizeof(unsigned int), cudaMemcpyDefault, s) !=
          cudaSuccess)
    return TRX_ERR_CUDA;
  return TRX_OK;
}
