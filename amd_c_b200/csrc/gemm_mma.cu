// gemm_mma.cu -- the prompt-chunk GEMM: Y[T x rows] = Q8(X)[T x cols] . W^T for the quantised kinds, T >= 17.
//
// One int8 tensor-core instruction (mma.sync m16n8k32, s8 x s8 -> s32) covers exactly one 32-weight quant block
// for 16 weight rows x 8 tokens, so its result IS the exact int32 block dot of the reference; the per-block
// scales are applied in fp32 right in the registers that hold it (acc = fma(sw * da, (float)dot, acc), or the
// Q4_K / Q6_K nestings of the GEMV), block after block in order. That fp32 work, not the tensor pipe, bounds
// the kernel (3-4 ALU operations per 32 MACs), which is why the dots stay in registers (mma.sync) instead of
// travelling through tensor memory. Results equal the one-token GEMV's to fp32 rounding (the order of the
// per-block sums differs: all blocks in sequence here, lane-strided + tree there), as in the reference
// (kernels/ie_kernels.c:1315-1465: "not bitwise vs GEMV").
//
// The streaming row layout needs no staging: the lane that owns columns 4t..4t+3 and 16+4t..19+4t of a row in
// the A fragment needs exactly nibble word t of the block (low nibbles = the first, high nibbles = the second),
// one 4-byte load; the B fragment is two 4-byte loads from a token's Q8 row. CTA = 8 warps as 2 (rows) x 4
// (tokens), warp tile 32 rows x 32 tokens, CTA tile 64 rows x 128 tokens.
#include "common.cuh"

namespace ieb {

constexpr int GM_MT = 2, GM_NT = 4;  // 16-row and 8-token tiles per warp
constexpr int GM_ROWS = 2 * 16 * GM_MT, GM_TOKS = 4 * 8 * GM_NT;

struct GemmArgs {
  const uint8_t *w;
  size_t rowb;
  uint32_t rows, nb, T;
  const uint8_t *xq;
  float *y;
  const float *bias, *res;
  size_t xs, ys, rs;
};

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

template <int KIND>
__global__ void __launch_bounds__(256, 2) gemm_mma_kernel(const GemmArgs a) {
  pdl_prologue();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const uint32_t row0 = blockIdx.x * GM_ROWS + (warp & 1) * 16 * GM_MT, tok0 = blockIdx.y * GM_TOKS + (warp >> 1) * 8 * GM_NT;
  if (row0 >= a.rows || tok0 >= a.T) return;
  const uint32_t nb = a.nb;
  // rows of the A fragments (g and g + 8 of each 16-row tile) and tokens of the B fragments (g) and of the C
  // fragments (2t, 2t + 1), clamped into range: out-of-range rows / tokens compute a copy that is never stored
  const uint8_t *rp[GM_MT][2];
#pragma unroll
  for (int i = 0; i < GM_MT; i++)
#pragma unroll
    for (int h = 0; h < 2; h++) rp[i][h] = a.w + (size_t)min(row0 + 16u * i + 8u * h + g, a.rows - 1u) * a.rowb;
  uint32_t ob[GM_NT], oc[GM_NT][2];
#pragma unroll
  for (int j = 0; j < GM_NT; j++) {
    ob[j] = (uint32_t)(min(tok0 + 8u * j + g, a.T - 1u) * a.xs);
    oc[j][0] = (uint32_t)(min(tok0 + 8u * j + 2u * t, a.T - 1u) * a.xs), oc[j][1] = (uint32_t)(min(tok0 + 8u * j + 2u * t + 1u, a.T - 1u) * a.xs);
  }
  float acc[GM_MT][GM_NT][4];
#pragma unroll
  for (int i = 0; i < GM_MT; i++)
#pragma unroll
    for (int j = 0; j < GM_NT; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) acc[i][j][e] = 0.0f;

  for (uint32_t b = 0; b < nb; b++) {
    // ---- the tokens' side of block b
    uint32_t bq[GM_NT][2];
    float da[GM_NT][2], das[GM_NT][2];
#pragma unroll
    for (int j = 0; j < GM_NT; j++) {
      const uint8_t *q = a.xq + ob[j] + 32u * b + 4u * t;
      bq[j][0] = *reinterpret_cast<const uint32_t *>(q), bq[j][1] = *reinterpret_cast<const uint32_t *>(q + 16);
#pragma unroll
      for (int e = 0; e < 2; e++) {
        da[j][e] = *reinterpret_cast<const float *>(a.xq + oc[j][e] + 32u * (size_t)nb + 4u * b);
        das[j][e] = 0.0f;
        if (KIND == IE_B200_MAT_Q4K) das[j][e] = __fmul_rn(da[j][e], (float)*reinterpret_cast<const int *>(a.xq + oc[j][e] + 36u * (size_t)nb + 4u * b));
      }
    }
    // ---- the rows' side, one 16-row tile at a time, and the products
#pragma unroll
    for (int i = 0; i < GM_MT; i++) {
      uint32_t wl[2], wh[2];  // the A fragment: columns 4t.. (low nibbles) and 16 + 4t.. (high nibbles) of rows g, g + 8
      float s0[2], s1[2];     // per row: Q4_0 d; Q4_K d * sc and dmin * mn; Q6_K d * sc0 and d * sc1
#pragma unroll
      for (int h = 0; h < 2; h++) {
        const uint8_t *r = rp[i][h];
        const uint32_t wv = *reinterpret_cast<const uint32_t *>(r + 16u * (size_t)b + 4u * t);
        if (KIND == IE_B200_MAT_Q4) {
          wl[h] = __vsub4(wv & 0x0F0F0F0Fu, 0x08080808u), wh[h] = __vsub4((wv >> 4) & 0x0F0F0F0Fu, 0x08080808u);
          s0[h] = h2f(*reinterpret_cast<const uint16_t *>(r + 16u * (size_t)nb + 2u * b)), s1[h] = 0.0f;
        } else if (KIND == IE_B200_MAT_Q4K) {
          wl[h] = wv & 0x0F0F0F0Fu, wh[h] = (wv >> 4) & 0x0F0F0F0Fu;
          const uint4 hd = *reinterpret_cast<const uint4 *>(r + 16u * (size_t)nb + 16u * (b >> 3));
          const uint32_t f = q4k_field(hd, (int)(b & 7u));
          s0[h] = __fmul_rn(h2f((uint16_t)(hd.x & 0xFFFFu)), (float)(f & 63u));
          s1[h] = __fmul_rn(h2f((uint16_t)(hd.x >> 16)), (float)(f >> 6));
        } else {
          const uint2 hw = *reinterpret_cast<const uint2 *>(r + 16u * (size_t)nb + 8u * b);
          wl[h] = (uint32_t)q6_sw(wv & 0x0F0F0F0Fu, hw.x, t), wh[h] = (uint32_t)q6_sw((wv >> 4) & 0x0F0F0F0Fu, hw.y, t);
          const uint16_t sc = *reinterpret_cast<const uint16_t *>(r + 24u * (size_t)nb + 2u * b);
          const float df = h2f(*reinterpret_cast<const uint16_t *>(r + 26u * (size_t)nb + 2u * (b >> 3)));
          s0[h] = __fmul_rn(df, (float)(int8_t)(sc & 255u)), s1[h] = __fmul_rn(df, (float)(int8_t)(sc >> 8));
        }
      }
#pragma unroll
      for (int j = 0; j < GM_NT; j++) {
        int c[4];
        if (KIND == IE_B200_MAT_Q6K) {  // the two 16-weight halves have scales of their own: two products with the other half zeroed
          int c2[4];
          mma_s8(c, wl[0], wl[1], 0u, 0u, bq[j][0], bq[j][1]);
          mma_s8(c2, 0u, 0u, wh[0], wh[1], bq[j][0], bq[j][1]);
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const int h = e >> 1, tk = e & 1;
            acc[i][j][e] = __fmaf_rn(__fmaf_rn(s1[h], (float)c2[e], __fmul_rn(s0[h], (float)c[e])), da[j][tk], acc[i][j][e]);
          }
        } else {
          mma_s8(c, wl[0], wl[1], wh[0], wh[1], bq[j][0], bq[j][1]);
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const int h = e >> 1, tk = e & 1;  // C fragment: e = 0, 1: row g, tokens 2t, 2t + 1; e = 2, 3: row g + 8
            if (KIND == IE_B200_MAT_Q4) acc[i][j][e] = __fmaf_rn(__fmul_rn(s0[h], da[j][tk]), (float)c[e], acc[i][j][e]);
            else acc[i][j][e] = __fmaf_rn(-s1[h], das[j][tk], __fmaf_rn(__fmul_rn(s0[h], (float)c[e]), da[j][tk], acc[i][j][e]));
          }
        }
      }
    }
  }
  // ---- y = acc (+ bias[row]); y = res + y
#pragma unroll
  for (int i = 0; i < GM_MT; i++)
#pragma unroll
    for (int j = 0; j < GM_NT; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const uint32_t row = row0 + 16u * i + 8u * (e >> 1) + g, tok = tok0 + 8u * j + 2u * t + (e & 1);
        if (row < a.rows && tok < a.T) {
          float o = acc[i][j][e];
          if (a.bias) o = __fadd_rn(o, a.bias[row]);
          if (a.res) o = __fadd_rn(reinterpret_cast<const float *>(reinterpret_cast<const char *>(a.res) + a.rs * tok)[row], o);
          reinterpret_cast<float *>(reinterpret_cast<char *>(a.y) + a.ys * tok)[row] = o;
        }
      }
}


// ---------------------------------------------------------------------------------------------------------------
// The staged form (the default): the same arithmetic, operands brought into shared memory by 16 / 8 / 4-byte
// asynchronous copies, three stages of four quant blocks each in flight, so the warps read fragments at
// shared-memory latency instead of waiting on L2. Rows are padded to strides (80 B of nibbles, 144 B of int8
// activations, 40 B of Q6_K high-bit words) that spread the eight rows / tokens of a fragment over all 32 banks.
// Needs nb % 4 == 0 and 16-byte aligned token rows; other shapes take the direct kernel above.
constexpr int GS_KB = 4, GS_STAGES = 3, GS_WS = 80, GS_XS = 144, GS_HS = 40;

template <int KIND, int TOKS>
struct GsLay {
  static constexpr int W = 0;                                   // [64 rows][80 B]: 4 blocks of 16 B nibbles
  static constexpr int SC = W + GM_ROWS * GS_WS;                // Q4_0: [64][4 f16]; Q4_K: [64][16 B header]; Q6_K: [64][4 u16]
  static constexpr int SC_BYTES = KIND == IE_B200_MAT_Q4K ? GM_ROWS * 16 : GM_ROWS * 8;
  static constexpr int HI = SC + SC_BYTES;                      // Q6_K: [64][40 B]: 4 blocks of 8 B high-bit words
  static constexpr int HI_BYTES = KIND == IE_B200_MAT_Q6K ? GM_ROWS * GS_HS : 0;
  static constexpr int X = HI + HI_BYTES;                       // [TOKS tokens][144 B]: 4 blocks of 32 int8
  static constexpr int DA = X + TOKS * GS_XS;                   // [4 blocks][TOKS tokens] f32
  static constexpr int AS = DA + GS_KB * TOKS * 4;              // [4 blocks][TOKS tokens] i32
  static constexpr int SS = AS + GS_KB * TOKS * 4;               // Q4_K: [64 rows][4 blocks] (d sc, dmin mn) f32 pairs, 40-byte rows, worked out once per stage
  static constexpr int SS_BYTES = KIND == IE_B200_MAT_Q4K ? GM_ROWS * 40 : 0;
  static constexpr int STAGE = SS + SS_BYTES;
};

__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(void *dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void *dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// NT: 8-token tiles per warp; the CTA covers 64 rows x (32 NT) tokens. NT = 4 by default, NT = 2 when the grid would
// otherwise leave most SMs idle (few rows).
template <int KIND, int NT>
__global__ void __launch_bounds__(256, 2) gemm_staged_kernel(const GemmArgs a) {
  constexpr int TOKS = 4 * 8 * NT;
  using L = GsLay<KIND, TOKS>;
  extern __shared__ uint4 gs_smem[];
  uint8_t *sm = reinterpret_cast<uint8_t *>(gs_smem);
  pdl_prologue();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int wm = warp & 1, wn = warp >> 1;  // warp tile: rows wm * 32 .., tokens wn * 8 NT .. of the CTA tile
  const uint32_t row0 = blockIdx.x * GM_ROWS, tok0 = blockIdx.y * TOKS, nb = a.nb;
  const uint32_t n_steps = nb / GS_KB;

  // what this thread copies per stage (rows / tokens past the end repeat the last one; their results are not stored)
  const uint8_t *w_src = a.w + (size_t)min(row0 + (tid >> 2), a.rows - 1u) * a.rowb;  // row tid / 4, 16-byte piece tid % 4
  constexpr int XI = TOKS * 8 / 256, SI = GS_KB * TOKS / 256;  // 16-byte activation pieces and 4-byte scales per thread and stage
  const uint8_t *x_src[XI];
#pragma unroll
  for (int i = 0; i < XI; i++) x_src[i] = a.xq + (size_t)min(tok0 + ((tid + 256 * i) >> 3), a.T - 1u) * a.xs;
  const uint8_t *s_src = a.xq + (size_t)min(tok0 + (tid % TOKS), a.T - 1u) * a.xs;  // scales of token tid % TOKS, blocks tid / TOKS + (256 / TOKS) i
  auto issue = [&](uint32_t step) {
    if (step < n_steps) {
      uint8_t *st = sm + (step % GS_STAGES) * L::STAGE;
      const uint32_t b0 = step * GS_KB;
      cp_async16(st + L::W + (tid >> 2) * GS_WS + (tid & 3) * 16, w_src + 16u * (size_t)(b0 + (tid & 3)));
#pragma unroll
      for (int i = 0; i < XI; i++) {
        const int item = tid + 256 * i;
        cp_async16(st + L::X + (item >> 3) * GS_XS + (item & 7) * 16, x_src[i] + 32u * (size_t)b0 + 16u * (item & 7));
      }
#pragma unroll
      for (int i = 0; i < SI; i++) {
        const int kb = tid / TOKS + (256 / TOKS) * i, tk = tid % TOKS;
        cp_async4(st + L::DA + (kb * TOKS + tk) * 4, s_src + 32u * (size_t)nb + 4u * (b0 + kb));
        if (KIND == IE_B200_MAT_Q4K) cp_async4(st + L::AS + (kb * TOKS + tk) * 4, s_src + 36u * (size_t)nb + 4u * (b0 + kb));
      }
      if (KIND == IE_B200_MAT_Q4) {
        if (tid < GM_ROWS) cp_async8(st + L::SC + tid * 8, a.w + (size_t)min(row0 + tid, a.rows - 1u) * a.rowb + 16u * (size_t)nb + 2u * b0);
      } else if (KIND == IE_B200_MAT_Q4K) {
        if (tid < GM_ROWS) cp_async16(st + L::SC + tid * 16, a.w + (size_t)min(row0 + tid, a.rows - 1u) * a.rowb + 16u * (size_t)nb + 16u * (b0 >> 3));
      } else {
        cp_async8(st + L::HI + (tid >> 2) * GS_HS + (tid & 3) * 8, w_src + 16u * (size_t)nb + 8u * (size_t)(b0 + (tid & 3)));
        if (tid < GM_ROWS) cp_async8(st + L::SC + tid * 8, a.w + (size_t)min(row0 + tid, a.rows - 1u) * a.rowb + 24u * (size_t)nb + 2u * b0);
      }
    }
    cp_async_commit();
  };

  float acc[GM_MT][NT][4];
#pragma unroll
  for (int i = 0; i < GM_MT; i++)
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) acc[i][j][e] = 0.0f;
  // Q6_K: the f16 super-block scale of this lane's four rows (it changes every 8 blocks = 2 steps), read from global
  const uint8_t *drow[GM_MT][2];
  float dq6[GM_MT][2];
  if (KIND == IE_B200_MAT_Q6K) {
#pragma unroll
    for (int i = 0; i < GM_MT; i++)
#pragma unroll
      for (int h = 0; h < 2; h++)
        drow[i][h] = a.w + (size_t)min(row0 + wm * 32 + 16 * i + 8 * h + g, a.rows - 1u) * a.rowb + 26u * (size_t)nb;
  }

#pragma unroll
  for (int s = 0; s < GS_STAGES - 1; s++) issue(s);
  for (uint32_t step = 0; step < n_steps; step++) {
    cp_async_wait<GS_STAGES - 2>();
    __syncthreads();  // step's stage is complete for everybody, and everybody is done with the stage refilled next
    issue(step + GS_STAGES - 1);
    uint8_t *st = sm + (step % GS_STAGES) * L::STAGE;
    if (KIND == IE_B200_MAT_Q4K) {  // the 256 (row, block) scale pairs of the stage, one per thread, instead of 4 per lane and block
      const int row = tid >> 2, kb = tid & 3;
      const uint4 hd = *reinterpret_cast<const uint4 *>(st + L::SC + row * 16);
      const uint32_t f = q4k_field(hd, (int)((step * GS_KB + kb) & 7u));
      *reinterpret_cast<float2 *>(st + L::SS + row * 40 + kb * 8) =
          make_float2(__fmul_rn(h2f((uint16_t)(hd.x & 0xFFFFu)), (float)(f & 63u)), __fmul_rn(h2f((uint16_t)(hd.x >> 16)), (float)(f >> 6)));
      __syncthreads();
    }
    if (KIND == IE_B200_MAT_Q6K && (step & 1u) == 0u) {
#pragma unroll
      for (int i = 0; i < GM_MT; i++)
#pragma unroll
        for (int h = 0; h < 2; h++) dq6[i][h] = h2f(*reinterpret_cast<const uint16_t *>(drow[i][h] + 2u * (step >> 1)));
    }
#pragma unroll
    for (int kb = 0; kb < GS_KB; kb++) {
      uint32_t wl[GM_MT][2], wh[GM_MT][2];
      float s0[GM_MT][2], s1[GM_MT][2];
#pragma unroll
      for (int i = 0; i < GM_MT; i++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const int rl = wm * 32 + 16 * i + 8 * h + g;
          const uint32_t wv = *reinterpret_cast<const uint32_t *>(st + L::W + rl * GS_WS + kb * 16 + 4 * t);
          if (KIND == IE_B200_MAT_Q4) {
            wl[i][h] = __vsub4(wv & 0x0F0F0F0Fu, 0x08080808u), wh[i][h] = __vsub4((wv >> 4) & 0x0F0F0F0Fu, 0x08080808u);
            s0[i][h] = h2f(*reinterpret_cast<const uint16_t *>(st + L::SC + rl * 8 + 2 * kb)), s1[i][h] = 0.0f;
          } else if (KIND == IE_B200_MAT_Q4K) {
            wl[i][h] = wv & 0x0F0F0F0Fu, wh[i][h] = (wv >> 4) & 0x0F0F0F0Fu;
            const float2 ss = *reinterpret_cast<const float2 *>(st + L::SS + rl * 40 + kb * 8);
            s0[i][h] = ss.x, s1[i][h] = ss.y;
          } else {
            const uint2 hw = *reinterpret_cast<const uint2 *>(st + L::HI + rl * GS_HS + kb * 8);
            wl[i][h] = (uint32_t)q6_sw(wv & 0x0F0F0F0Fu, hw.x, t), wh[i][h] = (uint32_t)q6_sw((wv >> 4) & 0x0F0F0F0Fu, hw.y, t);
            const uint16_t sc = *reinterpret_cast<const uint16_t *>(st + L::SC + rl * 8 + 2 * kb);
            s0[i][h] = __fmul_rn(dq6[i][h], (float)(int8_t)(sc & 255u)), s1[i][h] = __fmul_rn(dq6[i][h], (float)(int8_t)(sc >> 8));
          }
        }
      // B fragments of two token tiles per ldmatrix: an 8 x 8 matrix of 16-bit words = 8 tokens x 16 bytes, and lane (g, t)
      // receives bytes 4t .. 4t + 3 of token g: matrices (tile j, bytes 0..15), (tile j, 16..31), (tile j + 1, 0..15), (.., 16..31)
      uint32_t bf[NT][2];
#pragma unroll
      for (int j = 0; j < NT; j += 2) {
        uint32_t r4[4];
        const uint8_t *q = st + L::X + (wn * 8 * NT + 8 * (j + (lane >> 4)) + (lane & 7)) * GS_XS + kb * 32 + ((lane >> 3) & 1) * 16;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r4[0]), "=r"(r4[1]), "=r"(r4[2]), "=r"(r4[3]) : "r"((uint32_t)__cvta_generic_to_shared(q)));
        bf[j][0] = r4[0], bf[j][1] = r4[1], bf[j + 1][0] = r4[2], bf[j + 1][1] = r4[3];
      }
#pragma unroll
      for (int j = 0; j < NT; j++) {
        const int tl = wn * 8 * NT + 8 * j;
        const uint32_t b0 = bf[j][0], b1 = bf[j][1];
        const float2 da2 = *reinterpret_cast<const float2 *>(st + L::DA + (kb * TOKS + tl + 2 * t) * 4);
        const float da[2] = {da2.x, da2.y};
        float das[2] = {0.0f, 0.0f};
        if (KIND == IE_B200_MAT_Q4K) {
          const int2 as2 = *reinterpret_cast<const int2 *>(st + L::AS + (kb * TOKS + tl + 2 * t) * 4);
          das[0] = __fmul_rn(da[0], (float)as2.x), das[1] = __fmul_rn(da[1], (float)as2.y);
        }
#pragma unroll
        for (int i = 0; i < GM_MT; i++) {
          int c[4];
          if (KIND == IE_B200_MAT_Q6K) {
            int c2[4];
            mma_s8(c, wl[i][0], wl[i][1], 0u, 0u, b0, b1);
            mma_s8(c2, 0u, 0u, wh[i][0], wh[i][1], b0, b1);
#pragma unroll
            for (int e = 0; e < 4; e++) {
              const int h = e >> 1, tk = e & 1;
              acc[i][j][e] = __fmaf_rn(__fmaf_rn(s1[i][h], (float)c2[e], __fmul_rn(s0[i][h], (float)c[e])), da[tk], acc[i][j][e]);
            }
          } else {
            mma_s8(c, wl[i][0], wl[i][1], wh[i][0], wh[i][1], b0, b1);
#pragma unroll
            for (int e = 0; e < 4; e++) {
              const int h = e >> 1, tk = e & 1;
              if (KIND == IE_B200_MAT_Q4) acc[i][j][e] = __fmaf_rn(__fmul_rn(s0[i][h], da[tk]), (float)c[e], acc[i][j][e]);
              else acc[i][j][e] = __fmaf_rn(-s1[i][h], das[tk], __fmaf_rn(__fmul_rn(s0[i][h], (float)c[e]), da[tk], acc[i][j][e]));
            }
          }
        }
      }
    }
  }
  cp_async_wait<0>();
  // ---- y = acc (+ bias[row]); y = res + y
#pragma unroll
  for (int i = 0; i < GM_MT; i++)
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const uint32_t row = row0 + wm * 32 + 16u * i + 8u * (e >> 1) + g, tok = tok0 + wn * 8 * NT + 8u * j + 2u * t + (e & 1);
        if (row < a.rows && tok < a.T) {
          float o = acc[i][j][e];
          if (a.bias) o = __fadd_rn(o, a.bias[row]);
          if (a.res) o = __fadd_rn(reinterpret_cast<const float *>(reinterpret_cast<const char *>(a.res) + a.rs * tok)[row], o);
          reinterpret_cast<float *>(reinterpret_cast<char *>(a.y) + a.ys * tok)[row] = o;
        }
      }
}

template <int KIND, int NT>
static int launch_staged_nt(const GemmArgs &a, cudaStream_t st) {
  constexpr int TOKS = 4 * 8 * NT;
  const size_t smem = (size_t)GS_STAGES * GsLay<KIND, TOKS>::STAGE;
  auto k = gemm_staged_kernel<KIND, NT>;
  if (int r = ensure_dynamic_smem(reinterpret_cast<const void *>(k), smem)) return r;
  const dim3 grid((a.rows + GM_ROWS - 1) / GM_ROWS, (a.T + TOKS - 1) / TOKS);
  IEB_LAUNCH_PDL("gemm_staged_kernel", k, grid, dim3(256), smem, st, a);
  return IE_B200_OK;
}
template <int KIND>
static int launch_staged(const GemmArgs &a, cudaStream_t st) {
  // 64 x 128 tiles unless they would fill less than two thirds of the resident CTA slots (2 per SM): then 64 x 64
  const uint64_t big = (uint64_t)((a.rows + GM_ROWS - 1) / GM_ROWS) * ((a.T + 127) / 128);
  if (a.T > 64 && big * 3 < (uint64_t)sm_count() * 2 * 2) return launch_staged_nt<KIND, 2>(a, st);
  return launch_staged_nt<KIND, 4>(a, st);
}

}  // namespace ieb

using namespace ieb;

extern "C" int ie_b200_gemm(int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_xq, float *d_y, const float *d_bias,
                            const float *d_res, uint32_t T, size_t x_stride, size_t y_stride, size_t res_stride, void *stream) {
  if (!d_w || !d_xq || !d_y) return fail(IE_B200_E_ARG, "ie_b200_gemm: NULL pointer");
  if (kind != IE_B200_MAT_Q4 && kind != IE_B200_MAT_Q4K && kind != IE_B200_MAT_Q6K) return fail(IE_B200_E_ARG, "ie_b200_gemm: matrix kind %d (Q4_0, Q4_K, Q6_K)", kind);
  if (cols == 0 || cols % (kind == IE_B200_MAT_Q4 ? 32u : 256u)) return fail(IE_B200_E_SIZE, "ie_b200_gemm: %u columns", cols);
  if (rows == 0 || T == 0) return IE_B200_OK;
  if (!aligned16(d_w) || ((uintptr_t)d_xq & 3u) || (x_stride & 3u) || (y_stride & 3u) || (res_stride & 3u))
    return fail(IE_B200_E_ARG, "ie_b200_gemm: the matrix must be 16-byte aligned, activations and strides 4-byte aligned");
  if ((uint64_t)T * x_stride > 0xFFFFFFFFull) return fail(IE_B200_E_SIZE, "ie_b200_gemm: %u tokens of %zu bytes exceed 4 GB of activations", T, x_stride);
  GemmArgs a;
  a.w = static_cast<const uint8_t *>(d_w), a.rowb = row_bytes_of(kind, cols), a.rows = rows, a.nb = cols / 32u, a.T = T;
  a.xq = static_cast<const uint8_t *>(d_xq), a.y = d_y, a.bias = d_bias, a.res = d_res;
  a.xs = x_stride, a.ys = y_stride, a.rs = res_stride;
  const dim3 grid((rows + GM_ROWS - 1) / GM_ROWS, (T + GM_TOKS - 1) / GM_TOKS);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // rows of whole stages (4 blocks) and 16-byte aligned token rows go through the shared-memory staged kernel,
  // every other shape through the kernel that reads its fragments straight from global memory
  if (a.nb % GS_KB == 0 && aligned16(d_xq) && x_stride % 16u == 0) {
    switch (kind) {
      case IE_B200_MAT_Q4: return launch_staged<IE_B200_MAT_Q4>(a, st);
      case IE_B200_MAT_Q4K: return launch_staged<IE_B200_MAT_Q4K>(a, st);
      default: return launch_staged<IE_B200_MAT_Q6K>(a, st);
    }
  }
  switch (kind) {
    case IE_B200_MAT_Q4: IEB_LAUNCH_PDL("gemm_mma_kernel", gemm_mma_kernel<IE_B200_MAT_Q4>, grid, dim3(256), 0, st, a); break;
    case IE_B200_MAT_Q4K: IEB_LAUNCH_PDL("gemm_mma_kernel", gemm_mma_kernel<IE_B200_MAT_Q4K>, grid, dim3(256), 0, st, a); break;
    default: IEB_LAUNCH_PDL("gemm_mma_kernel", gemm_mma_kernel<IE_B200_MAT_Q6K>, grid, dim3(256), 0, st, a); break;
  }
  return IE_B200_OK;
}
