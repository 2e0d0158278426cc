// gemm_tc.cu -- the prompt-chunk GEMM on the 5th-generation tensor cores (tcgen05 + tensor memory):
// Y[T x rows] = X[T x cols] . W^T for the quantised kinds, the role of ie_gemm_q4kr / ie_gemm_q6kr
// (kernels/ie_kernels.c:1315-1465, :2015-2158; dispatch src/hip.c:965-1003).
//
// The quant scales change every 32 columns, so an integer MMA needs a scaling step on the CUDA cores per 32 x row x
// token (the wall the reference's own GEMM hit, and the bound of the mma.sync kernel in gemm_mma.cu). Here nothing is
// scaled inside the main loop: both operands are turned into f16 ONCE and the tensor cores accumulate in fp32 over the
// whole K in tensor memory:
//   activations  a pre-pass expands each token's Q8 row to x = d_a * q (f32) and splits it into two f16 terms
//                x = x_hi + x_lo (22 significant bits), stored in the order the MMA wants (cost ~ T x K, once per chunk);
//   weights      sixteen producer warps dequantise the CTA's 256 rows of the current 32-column block (d (q - 8); d sc q -
//                dmin mn; d sc (q - 32)) to f32 and split them the same way, w = w_hi + w_lo, straight into shared
//                memory in the canonical K-major core-matrix layout (cost ~ rows x K, once per 256 tokens);
//   MMA          one thread issues, per 16 columns, w_hi x_hi + w_hi x_lo + w_lo x_hi (the dropped w_lo x_lo term is
//                below 2^-22 of a product) as tcgen05.mma kind::f16, M = 128, N = up to 256 tokens, two 128-row tiles per
//                CTA, accumulators in tensor memory (2 x 256 columns);
//   epilogue     the producer warps read the accumulators back (tcgen05.ld, one row and 128 tokens per thread), add bias / residual
//                and store token rows (32 consecutive rows per warp store: coalesced).
// A three-stage ring (64 KB per stage: 32 KB of weights, 32 KB of activations brought by one bulk copy) is handed over
// through mbarriers; tcgen05.commit frees a stage when the MMAs that read it have completed. Matrices with few rows
// (3584 x 18944: 14 CTAs) are split along K over grid.z, every split writing its partial sums to scratch, which a second
// kernel adds in split order (deterministic). Every mbarrier wait is bounded by wall time and reports through the device
// error word; tensor memory is freed on every path.
//
// Half precision has a narrow exponent range, so both sides are scaled by exact powers of two before they are split (a value
// below 2^-14 would lose its low term to the subnormal grid): the weights by 2^S_w, S_w chosen once per matrix from a bound on
// its largest weight (ie_b200_mat_tc_exp), each token by 2^S_n chosen from its largest Q8 scale; the epilogue multiplies row n
// of the result by 2^-(S_w + S_n).
//
// Result: equal to the one-token GEMV (which is bit-exact with the CPU) to fp32 rounding: not bit for bit, as the
// reference's GEMM against its GEMV.
#include <cuda_fp16.h>
#include <math.h>
#include <string.h>

#include "common.cuh"

namespace ieb {

constexpr int TC_ROWS = 256, TC_TOK = 256, TC_KS = 32, TC_STAGES = 3, TC_PROD_WARPS = 16, TC_THREADS = (TC_PROD_WARPS + 2) * 32;
constexpr int TC_A_TILE = 128 * TC_KS * 2;       // one 128-row tile, one f16 term, one stage: 8 KB
constexpr int TC_A_STAGE = 4 * TC_A_TILE;        // two tiles x (hi, lo)
constexpr int TC_B_TERM = TC_TOK * TC_KS * 2;    // 16 KB
constexpr int TC_B_STAGE = 2 * TC_B_TERM;        // (hi, lo): what the pre-pass writes per (token tile, block), one bulk copy
constexpr int TC_SMEM = TC_STAGES * (TC_A_STAGE + TC_B_STAGE) + 256;
constexpr uint64_t TC_WAIT_NS = 2000000000ull;

struct TcArgs {
  const uint8_t *w;
  size_t rowb;
  uint32_t rows, nb, T;
  uint32_t blocks_per_split;
  const uint8_t *bp;  // expanded activations: [token tile][block][hi | lo][4 chunks][32 groups][8 tokens][8 halves]
  float *y;
  const float *bias, *res;
  size_t ys, rs;
  float *partial;     // grid.z > 1: [split][T][rows]
  uint32_t *err;
  float w_scale;      // 2^S_w applied to every weight before the split
  const float *tok_inv;  // per token: 2^-(S_w + S_n)
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t tc_now() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)); }
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Wait for the phase of the given parity; false after the time limit or once another thread of the CTA has given up.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort) {
  const uint32_t a = smem_u32(bar);
  uint64_t t0 = 0;
  for (uint32_t i = 0;; i++) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(a), "r"(parity)
        : "memory");
    if (ok) return true;
    if (*abort) return false;
    if ((i & 63u) == 63u) {
      const uint64_t now = tc_now();
      if (t0 == 0) t0 = now;
      else if (now - t0 > TC_WAIT_NS) {
        *abort = 1u;
        return false;
      }
    }
  }
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes),
               "r"(smem_u32(bar))
               : "memory");
}
// Shared-memory matrix descriptor, K-major, no swizzle: 8 x 16-byte core matrices; lbo = bytes between the two core matrices
// along K of one MMA, sbo = bytes between 8-row groups; bits 46-47 = 1 (descriptor version of this architecture).
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, "
      "%22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
        "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// x = hi + lo as two f16 (22 significant bits), for two values at a time.
__device__ __forceinline__ void tc_split2(float x, float y, uint32_t &hi, uint32_t &lo) {
  const __half2 h = __floats2half2_rn(x, y);
  const float2 hf = __half22float2(h);
  const __half2 l = __floats2half2_rn(x - hf.x, y - hf.y);
  hi = *reinterpret_cast<const uint32_t *>(&h), lo = *reinterpret_cast<const uint32_t *>(&l);
}

// One warp per token: S_n from the largest Q8 scale of the row, so that the largest |d q| 2^S_n lies in [2048, 4096];
// tok_scale[n] = 2^S_n, tok_inv[n] = 2^-(S_n) * w_inv.
__global__ void __launch_bounds__(256) tc_tokscale_kernel(const uint8_t *xq, size_t xs, uint32_t T, uint32_t nb, float w_inv, float *tok_scale, float *tok_inv) {
  pdl_prologue();
  const uint32_t n = blockIdx.x * 8u + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
  if (n >= T) return;
  const float *d = reinterpret_cast<const float *>(xq + xs * n + 32u * (size_t)nb);
  float m = 0.0f;
  for (uint32_t b = lane; b < nb; b += 32u) m = fmaxf(m, fabsf(d[b]));
  m = warp_max(m) * 127.0f;
  int e = 0;
  if (m > 0.0f && m < 3.0e38f) {
    int ex;
    frexpf(m, &ex);  // m = f * 2^ex, f in [0.5, 1)
    e = 12 - ex;     // m * 2^e in [2048, 4096)
    e = e > 100 ? 100 : (e < -100 ? -100 : e);
  }
  if (lane == 0) tok_scale[n] = ldexpf(1.0f, e), tok_inv[n] = ldexpf(w_inv, -e);
}

// ---- activations: Q8 rows -> f16 hi / lo in MMA order -----------------------------------------------------------------
// grid (nb, token tiles), 256 threads: thread = token of the tile; writes its 32 values of the block as 4 + 4 16-byte
// pieces (consecutive tokens write consecutive pieces). Tokens past T are zero.
__global__ void __launch_bounds__(256) tc_expand_kernel(const uint8_t *xq, size_t xs, uint32_t T, uint32_t nb, const float *tok_scale, uint8_t *bp) {
  pdl_prologue();
  const uint32_t b = blockIdx.x, nt = blockIdx.y, nl = threadIdx.x, n = nt * TC_TOK + nl;
  uint4 hi[4], lo[4];
#pragma unroll
  for (int c = 0; c < 4; c++) hi[c] = lo[c] = make_uint4(0u, 0u, 0u, 0u);
  if (n < T) {
    const uint8_t *row = xq + xs * n;
    const uint4 q0 = *reinterpret_cast<const uint4 *>(row + 32u * b), q1 = *reinterpret_cast<const uint4 *>(row + 32u * b + 16u);
    const float d = __fmul_rn(*reinterpret_cast<const float *>(row + 32u * (size_t)nb + 4u * b), tok_scale[n]);  // exact: a power of two
    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (int c = 0; c < 4; c++) {  // chunk c: values 8c .. 8c + 7 = words 2c, 2c + 1
      uint32_t h[4], l[4];
#pragma unroll
      for (int p = 0; p < 4; p++) {
        const uint32_t wd = qw[2 * c + (p >> 1)];
        const int s0 = (int)(int8_t)(wd >> (16 * (p & 1))), s1 = (int)(int8_t)(wd >> (16 * (p & 1) + 8));
        tc_split2(__fmul_rn(d, (float)s0), __fmul_rn(d, (float)s1), h[p], l[p]);
      }
      hi[c] = make_uint4(h[0], h[1], h[2], h[3]), lo[c] = make_uint4(l[0], l[1], l[2], l[3]);
    }
  }
  uint8_t *base = bp + ((size_t)nt * nb + b) * TC_B_STAGE + (nl >> 3) * 128u + (nl & 7u) * 16u;
#pragma unroll
  for (int c = 0; c < 4; c++) {
    *reinterpret_cast<uint4 *>(base + c * 4096u) = hi[c];
    *reinterpret_cast<uint4 *>(base + TC_B_TERM + c * 4096u) = lo[c];
  }
}

// ---- weights: one 32-weight block of one row -> 32 floats in column order --------------------------------------------
template <int KIND>
struct TcBlk;
template <>
struct TcBlk<IE_B200_MAT_Q4> {
  uint4 w;
  uint16_t d;
  __device__ __forceinline__ void load(const uint8_t *rp, uint32_t b, uint32_t nb) {
    w = __ldg(reinterpret_cast<const uint4 *>(rp + 16u * (size_t)b));
    d = __ldg(reinterpret_cast<const uint16_t *>(rp + 16u * (size_t)nb + 2u * b));
  }
  // columns 16 hf .. 16 hf + 15 of the block: the low (hf = 0) or high nibbles of the four words
  __device__ __forceinline__ void values16(float (&f)[16], uint32_t, uint32_t hf) const {
    const float df = h2f(d);
    const uint32_t ww[4] = {w.x >> (4u * hf), w.y >> (4u * hf), w.z >> (4u * hf), w.w >> (4u * hf)};
#pragma unroll
    for (int j = 0; j < 16; j++) f[j] = __fmul_rn(df, (float)((int)((ww[j >> 2] >> (8 * (j & 3))) & 15u) - 8));
  }
};
template <>
struct TcBlk<IE_B200_MAT_Q8> {
  uint4 w0, w1;
  uint16_t d;
  __device__ __forceinline__ void load(const uint8_t *rp, uint32_t b, uint32_t nb) {
    w0 = __ldg(reinterpret_cast<const uint4 *>(rp + 32u * (size_t)b));
    w1 = __ldg(reinterpret_cast<const uint4 *>(rp + 32u * (size_t)b + 16u));
    d = __ldg(reinterpret_cast<const uint16_t *>(rp + 32u * (size_t)nb + 2u * b));
  }
  // columns 16 hf .. 16 hf + 15: the signed bytes of the first (hf = 0) or second four words
  __device__ __forceinline__ void values16(float (&f)[16], uint32_t, uint32_t hf) const {
    const float df = h2f(d);
    const uint4 v = hf ? w1 : w0;
    const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 16; j++) f[j] = __fmul_rn(df, (float)(int8_t)(ww[j >> 2] >> (8 * (j & 3))));
  }
};
template <>
struct TcBlk<IE_B200_MAT_Q4K> {
  uint4 w, h;
  __device__ __forceinline__ void load(const uint8_t *rp, uint32_t b, uint32_t nb) {
    w = __ldg(reinterpret_cast<const uint4 *>(rp + 16u * (size_t)b));
    h = __ldg(reinterpret_cast<const uint4 *>(rp + 16u * (size_t)nb + 16u * (b >> 3)));
  }
  __device__ __forceinline__ void values16(float (&f)[16], uint32_t b, uint32_t hf) const {
    const uint32_t fld = q4k_field(h, (int)(b & 7u));
    const float s = __fmul_rn(h2f((uint16_t)(h.x & 0xFFFFu)), (float)(fld & 63u));
    const float mm = __fmul_rn(h2f((uint16_t)(h.x >> 16)), (float)(fld >> 6));
    const uint32_t ww[4] = {w.x >> (4u * hf), w.y >> (4u * hf), w.z >> (4u * hf), w.w >> (4u * hf)};
#pragma unroll
    for (int j = 0; j < 16; j++) f[j] = __fmaf_rn(s, (float)((ww[j >> 2] >> (8 * (j & 3))) & 15u), -mm);
  }
};
template <>
struct TcBlk<IE_B200_MAT_Q6K> {
  uint4 w;
  uint2 hw;
  uint16_t sc, d;
  __device__ __forceinline__ void load(const uint8_t *rp, uint32_t b, uint32_t nb) {
    w = __ldg(reinterpret_cast<const uint4 *>(rp + 16u * (size_t)b));
    hw = __ldg(reinterpret_cast<const uint2 *>(rp + 16u * (size_t)nb + 8u * b));
    sc = __ldg(reinterpret_cast<const uint16_t *>(rp + 24u * (size_t)nb + 2u * b));
    d = __ldg(reinterpret_cast<const uint16_t *>(rp + 26u * (size_t)nb + 2u * (b >> 3)));
  }
  __device__ __forceinline__ void values16(float (&f)[16], uint32_t, uint32_t hf) const {
    const float s = __fmul_rn(h2f(d), (float)(int8_t)(hf ? sc >> 8 : sc & 255u));
    const uint32_t ww[4] = {w.x >> (4u * hf), w.y >> (4u * hf), w.z >> (4u * hf), w.w >> (4u * hf)}, hh = hf ? hw.y : hw.x;
#pragma unroll
    for (int j = 0; j < 16; j++) {
      // weight 16 hf + 4 k + i: nibble hf of byte i of word k; its two high bits at bits 8 i + 2 k of the half's high-bit word
      const int k = j >> 2, i = j & 3;
      const uint32_t lo4 = (ww[k] >> (8 * i)) & 15u, hi2 = (hh >> (8 * i + 2 * k)) & 3u;
      f[j] = __fmul_rn(s, (float)((int)(lo4 | (hi2 << 4)) - 32));
    }
  }
};

template <int KIND>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const TcArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_tc[];
  uint8_t *sA = smem_tc;                                   // [stage][tile][term] 8 KB each
  uint8_t *sB = smem_tc + TC_STAGES * TC_A_STAGE;          // [stage][term] 16 KB each
  uint64_t *bars = reinterpret_cast<uint64_t *>(sB + TC_STAGES * TC_B_STAGE);
  uint64_t *full_a = bars, *full_b = bars + TC_STAGES, *empty = bars + 2 * TC_STAGES, *done = bars + 3 * TC_STAGES;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * TC_STAGES + 1);
  __shared__ uint32_t s_abort;
  __shared__ float s_inv[TC_TOK];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t m0 = blockIdx.x * TC_ROWS, nt = blockIdx.y, split = blockIdx.z;
  const uint32_t kb0 = split * a.blocks_per_split, kb1 = min(a.nb, kb0 + a.blocks_per_split), n_it = kb1 - kb0;
  const uint32_t n_tok = min((uint32_t)TC_TOK, a.T - nt * TC_TOK), n_eff = (n_tok + 15u) & ~15u;  // MMA N: a multiple of 16
  const uint32_t n_tiles = a.rows - m0 > 128u ? 2u : 1u;

  if (tid == 0) {
    s_abort = 0u;
    for (int s = 0; s < TC_STAGES; s++) mbar_init(&full_a[s], (uint32_t)TC_PROD_WARPS), mbar_init(&full_b[s], 1u), mbar_init(&empty[s], 1u);
    mbar_init(done, 1u);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == TC_PROD_WARPS) {  // tensor memory: all 512 columns (two accumulators of up to 256 columns), by one warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();  // the expanded activations (and the residual) are complete
  for (uint32_t j = tid; j < TC_TOK; j += TC_THREADS) s_inv[j] = nt * TC_TOK + j < a.T ? a.tok_inv[nt * TC_TOK + j] : 0.0f;
  __syncthreads();

  if (warp < TC_PROD_WARPS) {
    // ---------------- producers: warp w dequantises half h = w & 1 (16 columns) of the block for 32 rows of tile w >> 3 ----------------
    // (16 warps of one half block per thread: four warps per scheduler hide the conversion latency behind each other; with
    // four warps of two whole blocks per thread the tensor pipe waited for the producers)
    const uint32_t t = (uint32_t)warp >> 3, hf = (uint32_t)warp & 1u, rl = (((uint32_t)warp >> 1) & 3u) * 32u + lane;  // tile, column half, row in the tile
    const bool ok = m0 + t * 128u + rl < a.rows;
    const uint8_t *rp = a.w + (size_t)(m0 + t * 128u + rl) * a.rowb;
    TcBlk<KIND> cur, nxt, nx2;  // the blocks of this stage and of the two after it: their bytes are on the way while this one is converted
    if (ok) {
      if (n_it > 0u) cur.load(rp, kb0, a.nb);
      if (n_it > 1u) nxt.load(rp, kb0 + 1u, a.nb);
    }
    for (uint32_t it = 0; it < n_it; it++) {
      const uint32_t s = it % TC_STAGES, round = it / TC_STAGES, b = kb0 + it;
      if (it + 2u < n_it && ok) nx2.load(rp, b + 2u, a.nb);
      if (round > 0 && !mbar_wait(&empty[s], (round - 1u) & 1u, &s_abort)) break;
      float f[16];
      if (ok) {
        cur.values16(f, b, hf);
#pragma unroll
        for (int j = 0; j < 16; j++) f[j] = __fmul_rn(f[j], a.w_scale);  // exact: a power of two
      } else {
#pragma unroll
        for (int j = 0; j < 16; j++) f[j] = 0.0f;
      }
      uint8_t *dst = sA + s * TC_A_STAGE + t * 2 * TC_A_TILE + (rl >> 3) * 128u + (rl & 7u) * 16u + hf * 2u * 2048u;
#pragma unroll
      for (int c = 0; c < 2; c++) {  // 8-column chunks 2 hf + c of the block
        uint32_t h[4], l[4];
#pragma unroll
        for (int p = 0; p < 4; p++) tc_split2(f[8 * c + 2 * p], f[8 * c + 2 * p + 1], h[p], l[p]);
        *reinterpret_cast<uint4 *>(dst + c * 2048u) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4 *>(dst + TC_A_TILE + c * 2048u) = make_uint4(l[0], l[1], l[2], l[3]);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor cores read shared memory through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_a[s]);
      cur = nxt, nxt = nx2;
    }
    // ---------------- epilogue: accumulators -> token rows ----------------
    const bool finished = mbar_wait(done, 0u, &s_abort);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (finished && !s_abort) {
      // warp w reads lanes 32 (w & 3) .. + 31 of tensor memory (a warp reaches the quarter w mod 4 only): tile (w >> 2) & 1,
      // token columns [128 (w >> 3), + 128)
      const uint32_t q = (uint32_t)warp & 3u, te = ((uint32_t)warp >> 2) & 1u, ch = (uint32_t)warp >> 3;
      const uint32_t row = m0 + te * 128u + q * 32u + lane;
      const float bias = (a.bias && row < a.rows && !a.partial) ? a.bias[row] : 0.0f;
      if (te < n_tiles) {
        for (uint32_t c0 = ch * 128u; c0 < min(n_eff, ch * 128u + 128u); c0 += 32u) {
          uint32_t v[32];
          tc_ld32(tmem + ((q * 32u) << 16) + te * TC_TOK + c0, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (row < a.rows) {
#pragma unroll
            for (int j = 0; j < 32; j++) {
              const uint32_t n = nt * TC_TOK + c0 + j;
              if (n < a.T) {
                float o = __fmul_rn(__uint_as_float(v[j]), s_inv[c0 + j]);
                if (a.partial) {
                  a.partial[((size_t)split * a.T + n) * a.rows + row] = o;
                } else {
                  if (a.bias) o = __fadd_rn(o, bias);
                  if (a.res) o = __fadd_rn(*reinterpret_cast<const float *>(reinterpret_cast<const char *>(a.res) + a.rs * n + 4u * (size_t)row), o);
                  *reinterpret_cast<float *>(reinterpret_cast<char *>(a.y) + a.ys * n + 4u * (size_t)row) = o;
                }
              }
            }
          }
        }
      }
    }
  } else if (warp == TC_PROD_WARPS) {
    // ---------------- MMA issue: one thread ----------------
    if (lane == 0) {
      // instruction descriptor: D f32, A and B f16, both K-major, N = n_eff, M = 128
      const uint32_t idesc = (1u << 4) | ((n_eff >> 3) << 17) | ((128u >> 4) << 24);
      bool ok = true;
      for (uint32_t it = 0; it < n_it && ok; it++) {
        const uint32_t s = it % TC_STAGES, par = (it / TC_STAGES) & 1u;
        ok = mbar_wait(&full_a[s], par, &s_abort) && mbar_wait(&full_b[s], par, &s_abort);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_base = smem_u32(sA + s * TC_A_STAGE), b_base = smem_u32(sB + s * TC_B_STAGE);
        for (uint32_t t = 0; t < n_tiles; t++) {
#pragma unroll
          for (uint32_t j = 0; j < TC_KS / 16; j++) {  // 16 columns per MMA: two 8-column core matrices
            const uint64_t a_hi = tc_desc(a_base + t * 2 * TC_A_TILE + j * 4096u, 2048u, 128u), a_lo = tc_desc(a_base + t * 2 * TC_A_TILE + TC_A_TILE + j * 4096u, 2048u, 128u);
            const uint64_t b_hi = tc_desc(b_base + j * 8192u, 4096u, 128u), b_lo = tc_desc(b_base + TC_B_TERM + j * 8192u, 4096u, 128u);
            const uint32_t d = tmem + t * TC_TOK;
            tc_mma(d, a_hi, b_hi, idesc, (it | j) ? 1u : 0u);
            tc_mma(d, a_hi, b_lo, idesc, 1u);
            tc_mma(d, a_lo, b_hi, idesc, 1u);
          }
        }
        tc_commit(&empty[s]);  // arrives when the MMAs issued so far have completed: the stage may be refilled
      }
      tc_commit(done);
    }
  } else {
    // ---------------- activations: one bulk copy per stage ----------------
    if (lane == 0) {
      uint32_t issued = 0;
      for (uint32_t it = 0; it < n_it; it++) {
        const uint32_t s = it % TC_STAGES, round = it / TC_STAGES;
        if (round > 0 && !mbar_wait(&empty[s], (round - 1u) & 1u, &s_abort)) break;
        mbar_expect_tx(&full_b[s], TC_B_STAGE);
        bulk_g2s(sB + s * TC_B_STAGE, a.bp + ((size_t)nt * a.nb + kb0 + it) * TC_B_STAGE, TC_B_STAGE, &full_b[s]);
        issued = it + 1u;
      }
      if (s_abort) {  // gave up: do not leave while copies are still on their way into this CTA's shared memory
        for (uint32_t it = issued > TC_STAGES ? issued - TC_STAGES : 0u; it < issued; it++) {
          const uint64_t t0 = tc_now();
          uint32_t ok = 0;
          while (!ok && tc_now() - t0 < 10000000ull)
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok) : "r"(smem_u32(&full_b[it % TC_STAGES])), "r"((it / TC_STAGES) & 1u) : "memory");
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && s_abort && a.err) atomicExch(a.err, 5u);
  __syncwarp();
  if (warp == TC_PROD_WARPS) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

// y[n][row] = sum over the splits (in order) of partial[split][n][row] (+ bias) (+ res).
__global__ void __launch_bounds__(256) tc_reduce_kernel(const float *partial, uint32_t splits, uint32_t T, uint32_t rows, float *y, const float *bias,
                                                        const float *res, size_t ys, size_t rs) {
  pdl_prologue();
  const uint32_t n = blockIdx.y;
  for (uint32_t r = blockIdx.x * 256u + threadIdx.x; r < rows; r += gridDim.x * 256u) {
    float o = 0.0f;
    for (uint32_t s = 0; s < splits; s++) o = __fadd_rn(o, partial[((size_t)s * T + n) * rows + r]);
    if (bias) o = __fadd_rn(o, bias[r]);
    if (res) o = __fadd_rn(*reinterpret_cast<const float *>(reinterpret_cast<const char *>(res) + rs * n + 4u * (size_t)r), o);
    *reinterpret_cast<float *>(reinterpret_cast<char *>(y) + ys * n + 4u * (size_t)r) = o;
  }
}

static uint32_t tc_splits(uint32_t rows, uint32_t nb, uint32_t T) {
  const uint32_t ctas = ((rows + TC_ROWS - 1) / TC_ROWS) * ((T + TC_TOK - 1) / TC_TOK);
  const uint32_t sms = (uint32_t)sm_count();
  if (ctas * 2u > sms) return 1u;
  uint32_t s = sms / ctas;
  if (s > nb / 8u) s = nb / 8u;  // at least 8 blocks (256 columns) per split
  if (s > 16u) s = 16u;
  return s < 1u ? 1u : s;
}

}  // namespace ieb

using namespace ieb;

extern "C" size_t ie_b200_gemm_tc_scratch_bytes(uint32_t rows, uint32_t cols, uint32_t T) {
  const uint32_t nb = cols / 32u, nt = (T + TC_TOK - 1) / TC_TOK, splits = tc_splits(rows, nb, T);
  const size_t bp = (size_t)nt * nb * TC_B_STAGE, part = splits > 1u ? (size_t)splits * T * rows * sizeof(float) : 0u;
  const size_t scales = ((size_t)2 * nt * TC_TOK * sizeof(float) + 255u) & ~(size_t)255u;
  return bp + part + scales + 512u;
}

namespace ieb {
// Largest possible |weight| of a matrix from its scale fields: Q4_0 8 |d|; Q4_K 63 (15 |d| + |dmin|); Q6_K 128 * 32 |d|.
template <int KIND>
__global__ void __launch_bounds__(256) tc_wbound_kernel(const uint8_t *w, size_t rowb, uint32_t rows, uint32_t nb, uint32_t *out_bits) {
  float m = 0.0f;
  const uint32_t per = (KIND == IE_B200_MAT_Q4 || KIND == IE_B200_MAT_Q8) ? nb : nb / 8u;
  for (size_t i = (size_t)blockIdx.x * 256u + threadIdx.x; i < (size_t)rows * per; i += (size_t)gridDim.x * 256u) {
    const uint8_t *rp = w + (i / per) * rowb;
    const uint32_t b = (uint32_t)(i % per);
    float v;
    if (KIND == IE_B200_MAT_Q4) {
      v = 8.0f * fabsf(h2f(*reinterpret_cast<const uint16_t *>(rp + 16u * (size_t)nb + 2u * b)));
    } else if (KIND == IE_B200_MAT_Q8) {
      v = 128.0f * fabsf(h2f(*reinterpret_cast<const uint16_t *>(rp + 32u * (size_t)nb + 2u * b)));
    } else if (KIND == IE_B200_MAT_Q4K) {
      const uint32_t dd = *reinterpret_cast<const uint32_t *>(rp + 16u * (size_t)nb + 16u * b);
      v = 63.0f * (15.0f * fabsf(h2f((uint16_t)(dd & 0xFFFFu))) + fabsf(h2f((uint16_t)(dd >> 16))));
    } else {
      v = 4096.0f * fabsf(h2f(*reinterpret_cast<const uint16_t *>(rp + 26u * (size_t)nb + 2u * b)));
    }
    if (v < 3.0e38f) m = fmaxf(m, v);
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) atomicMax(out_bits, __float_as_uint(m));  // non-negative floats order as their bits
}
}  // namespace ieb

extern "C" int ie_b200_mat_tc_exp(int kind, const void *d_w, uint32_t rows, uint32_t cols, int *h_exp, void *stream) {
  if (!d_w || !h_exp) return fail(IE_B200_E_ARG, "ie_b200_mat_tc_exp: NULL pointer");
  if (kind != IE_B200_MAT_Q4 && kind != IE_B200_MAT_Q8 && kind != IE_B200_MAT_Q4K && kind != IE_B200_MAT_Q6K)
    return fail(IE_B200_E_ARG, "ie_b200_mat_tc_exp: matrix kind %d", kind);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t *d_bits = nullptr, bits = 0;
  IEB_CUDA(cudaMalloc(&d_bits, 4));
  IEB_CUDA(cudaMemsetAsync(d_bits, 0, 4, st));
  const uint8_t *w = static_cast<const uint8_t *>(d_w);
  const size_t rowb = row_bytes_of(kind, cols);
  const uint32_t nb = cols / 32u, grid = 592;
  if (kind == IE_B200_MAT_Q4) tc_wbound_kernel<IE_B200_MAT_Q4><<<grid, 256, 0, st>>>(w, rowb, rows, nb, d_bits);
  else if (kind == IE_B200_MAT_Q8) tc_wbound_kernel<IE_B200_MAT_Q8><<<grid, 256, 0, st>>>(w, rowb, rows, nb, d_bits);
  else if (kind == IE_B200_MAT_Q4K) tc_wbound_kernel<IE_B200_MAT_Q4K><<<grid, 256, 0, st>>>(w, rowb, rows, nb, d_bits);
  else tc_wbound_kernel<IE_B200_MAT_Q6K><<<grid, 256, 0, st>>>(w, rowb, rows, nb, d_bits);
  count_launch();
  cudaError_t e = cudaMemcpyAsync(&bits, d_bits, 4, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  cudaFree(d_bits);
  if (e != cudaSuccess) return cuda_fail(e, "ie_b200_mat_tc_exp");
  float m;
  memcpy(&m, &bits, 4);
  int ex = 0, s = 0;
  if (m > 0.0f) {
    frexpf(m, &ex);  // m < 2^ex
    s = 13 - ex;     // bound * 2^s < 8192
    s = s > 100 ? 100 : (s < -100 ? -100 : s);
  }
  *h_exp = s;
  return IE_B200_OK;
}

extern "C" int ie_b200_gemm_tc(int kind, const void *d_w, uint32_t rows, uint32_t cols, int w_exp, const void *d_xq, float *d_y, const float *d_bias,
                               const float *d_res, uint32_t T, size_t x_stride, size_t y_stride, size_t res_stride, void *d_scratch, size_t scratch_bytes,
                               uint32_t *d_err, void *stream) {
  if (!d_w || !d_xq || !d_y || !d_scratch) return fail(IE_B200_E_ARG, "ie_b200_gemm_tc: NULL pointer");
  if (kind != IE_B200_MAT_Q4 && kind != IE_B200_MAT_Q8 && kind != IE_B200_MAT_Q4K && kind != IE_B200_MAT_Q6K)
    return fail(IE_B200_E_ARG, "ie_b200_gemm_tc: matrix kind %d (Q4_0, Q8_0, Q4_K, Q6_K)", kind);
  if (cols == 0 || cols % ((kind == IE_B200_MAT_Q4 || kind == IE_B200_MAT_Q8) ? 32u : 256u)) return fail(IE_B200_E_SIZE, "ie_b200_gemm_tc: %u columns", cols);
  if (rows == 0 || T == 0) return IE_B200_OK;
  if (!aligned16(d_w) || !aligned16(d_xq) || (x_stride & 15u) || (y_stride & 3u) || (res_stride & 3u) || ((uintptr_t)d_scratch & 255u))
    return fail(IE_B200_E_ARG, "ie_b200_gemm_tc: the matrix and the Q8 rows must be 16-byte aligned, strides multiples of 4, the scratch 256-byte aligned");
  if (scratch_bytes < ie_b200_gemm_tc_scratch_bytes(rows, cols, T)) return fail(IE_B200_E_SIZE, "ie_b200_gemm_tc: scratch of %zu bytes, %zu needed", scratch_bytes, ie_b200_gemm_tc_scratch_bytes(rows, cols, T));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint32_t nb = cols / 32u, nt = (T + TC_TOK - 1) / TC_TOK, splits = tc_splits(rows, nb, T);
  if (w_exp < -100 || w_exp > 100) return fail(IE_B200_E_ARG, "ie_b200_gemm_tc: weight exponent %d", w_exp);
  uint8_t *bp = static_cast<uint8_t *>(d_scratch);
  const size_t bp_bytes = ((size_t)nt * nb * TC_B_STAGE + 255u) & ~(size_t)255u, sc_bytes = ((size_t)2 * nt * TC_TOK * sizeof(float) + 255u) & ~(size_t)255u;
  float *tok_scale = reinterpret_cast<float *>(bp + bp_bytes), *tok_inv = tok_scale + (size_t)nt * TC_TOK;
  float *partial = splits > 1u ? reinterpret_cast<float *>(bp + bp_bytes + sc_bytes) : nullptr;
  IEB_LAUNCH_PDL("tc_tokscale_kernel", tc_tokscale_kernel, dim3((T + 7u) / 8u), dim3(256), 0, st, static_cast<const uint8_t *>(d_xq), x_stride, T, nb,
                 ldexpf(1.0f, -w_exp), tok_scale, tok_inv);
  IEB_LAUNCH_PDL("tc_expand_kernel", tc_expand_kernel, dim3(nb, nt), dim3(256), 0, st, static_cast<const uint8_t *>(d_xq), x_stride, T, nb,
                 static_cast<const float *>(tok_scale), bp);
  TcArgs a = {};
  a.w = static_cast<const uint8_t *>(d_w), a.rowb = row_bytes_of(kind, cols), a.rows = rows, a.nb = nb, a.T = T;
  a.blocks_per_split = (nb + splits - 1u) / splits;
  if (kind != IE_B200_MAT_Q4 && kind != IE_B200_MAT_Q8) a.blocks_per_split = (a.blocks_per_split + 7u) & ~7u;
  a.bp = bp, a.y = d_y, a.bias = d_bias, a.res = d_res, a.ys = y_stride, a.rs = res_stride, a.partial = partial, a.err = d_err;
  a.w_scale = ldexpf(1.0f, w_exp), a.tok_inv = tok_inv;
  const uint32_t used_splits = (nb + a.blocks_per_split - 1u) / a.blocks_per_split;
  const dim3 grid((rows + TC_ROWS - 1) / TC_ROWS, nt, partial ? used_splits : 1u);
  void (*k)(TcArgs) = kind == IE_B200_MAT_Q4 ? gemm_tc_kernel<IE_B200_MAT_Q4> : kind == IE_B200_MAT_Q8 ? gemm_tc_kernel<IE_B200_MAT_Q8>
                      : kind == IE_B200_MAT_Q4K ? gemm_tc_kernel<IE_B200_MAT_Q4K> : gemm_tc_kernel<IE_B200_MAT_Q6K>;
  if (int r = ensure_dynamic_smem(reinterpret_cast<const void *>(k), TC_SMEM)) return r;
  IEB_LAUNCH_PDL("gemm_tc_kernel", k, grid, dim3(TC_THREADS), TC_SMEM, st, a);
  if (partial)
    IEB_LAUNCH_PDL("tc_reduce_kernel", tc_reduce_kernel, dim3((rows + 255u) / 256u, T), dim3(256), 0, st, static_cast<const float *>(partial), used_splits, T, rows, d_y,
                   d_bias, d_res, y_stride, res_stride);
  return IE_B200_OK;
}
