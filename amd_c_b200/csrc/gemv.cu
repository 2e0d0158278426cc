// gemv.cu -- quantised-weight x Q8-activation GEMV (Q4_0, Q4_K, Q6_K) and the
// f32 GEMV for batch-1 decode on sm_100a. HBM-bound: no tensor cores.
//
// Work split (the reference's, so results match its CPU backend bit for bit):
// one warp per row; lane l accumulates blocks l, l+32, l+64, ... in that
// order starting from 0.0f, then the warp reduces by shuffle-down 16, 8, 4,
// 2, 1 and lane 0 applies the epilogue.
//
// Memory: a persistent grid (a few CTAs per SM) stages the token's Q8
// activations once per CTA in shared memory as two 16-byte planes per block
// (conflict-free 16-byte reads) and then streams row panels: each lane has
// R x U 16-byte weight loads in flight (R rows per warp pass, U lane steps per
// chunk) before any arithmetic depends on them.
#include "common.cuh"
#include "gemv_blocks.cuh"

namespace ieb {

constexpr int GEMV_THREADS = 256, GEMV_WARPS = GEMV_THREADS / 32;

// Stage one token's Q8 buffer into shared memory: plane A0 = words 0..3 of
// every block, plane A1 = words 4..7, then the scales and the block sums.
__device__ __forceinline__ void stage_q8(const uint8_t *xq, uint32_t nb, uint4 *A0, uint4 *A1, float *da, int *as) {
  const uint4 *src = reinterpret_cast<const uint4 *>(xq);
  for (uint32_t i = threadIdx.x; i < 2u * nb; i += blockDim.x) {
    const uint4 v = src[i];
    if (i & 1u) A1[i >> 1] = v;
    else A0[i >> 1] = v;
  }
  const float *d = reinterpret_cast<const float *>(xq + 32u * (size_t)nb);
  const int *s = reinterpret_cast<const int *>(xq + 36u * (size_t)nb);
  for (uint32_t i = threadIdx.x; i < nb; i += blockDim.x) da[i] = d[i], as[i] = s[i];
}

template <int KIND, int R, int U>
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_q_kernel(const uint8_t *__restrict__ w, size_t rowb, uint32_t rows, uint32_t nb, const uint8_t *__restrict__ x, float *y,
              const float *__restrict__ bias, const float *res, size_t xs, size_t ys, size_t rs) {
  extern __shared__ uint4 smem[];
  uint4 *A0 = smem, *A1 = smem + nb;
  float *da = reinterpret_cast<float *>(smem + 2u * nb);
  int *as = reinterpret_cast<int *>(da + nb);
  const uint32_t t = blockIdx.y;
  stage_q8(x + t * xs, nb, A0, A1, da, as);
  __syncthreads();
  y = reinterpret_cast<float *>(reinterpret_cast<char *>(y) + t * ys);
  if (res) res = reinterpret_cast<const float *>(reinterpret_cast<const char *>(res) + t * rs);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t stride = gridDim.x * GEMV_WARPS * R;
  for (uint32_t r0 = (blockIdx.x * GEMV_WARPS + warp) * R; r0 < rows; r0 += stride) {
    float acc[R];
#pragma unroll
    for (int i = 0; i < R; i++) acc[i] = 0.0f;
    for (uint32_t c = 0; c < nb; c += 32u * U) {
      Blk<KIND, false> blk[R][U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const uint32_t b = c + 32u * u + lane;
#pragma unroll
        for (int i = 0; i < R; i++)
          if (b < nb && r0 + i < rows) blk[i][u].load(w + (size_t)(r0 + i) * rowb, b, nb);
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        const uint32_t b = c + 32u * u + lane;
        if (b < nb) {
          const uint4 a0 = A0[b], a1 = A1[b];
          const float d = da[b];
          const int s = as[b];
#pragma unroll
          for (int i = 0; i < R; i++)
            if (r0 + i < rows) acc[i] = blk[i][u].accum(acc[i], a0, a1, d, s, b);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < R; i++) {
      const float v = warp_tree(acc[i]);
      const uint32_t r = r0 + i;
      if (lane == 0 && r < rows) {
        float o = v;
        if (bias) o = __fadd_rn(o, bias[r]);
        if (res) o = __fadd_rn(res[r], o);
        y[r] = o;
      }
    }
  }
}

// Several tokens per pass over the weights (2..16 tokens: speculative verification, short prompt tails; the role of
// ie_gemv_q4kq8_tr / _ts2 in the reference, kernels/ie_kernels.c:483-628): a CTA stages the Q8 buffers of TT tokens
// and every loaded weight block is applied to each of them, every token in exactly the one-token order (lane l:
// blocks l, l + 32, ... from 0.0f, then the tree), so each row of the result is bit for bit the one-token GEMV's.
template <int KIND, int U, int TT>
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_mt_kernel(const uint8_t *__restrict__ w, size_t rowb, uint32_t rows, uint32_t nb, const uint8_t *__restrict__ x, float *y,
               const float *__restrict__ bias, const float *res, uint32_t T, size_t xs, size_t ys, size_t rs) {
  extern __shared__ uint4 smem[];
  const uint32_t t0 = blockIdx.y * TT, nt = min((uint32_t)TT, T - t0);
  // per token: A0 plane, A1 plane (nb uint4 each), scales and sums (nb words each)
  const size_t per_tok = (size_t)nb * 40u / 16u;  // in uint4
  for (uint32_t t = 0; t < nt; t++) {
    uint4 *A0 = smem + t * per_tok, *A1 = A0 + nb;
    stage_q8(x + (size_t)(t0 + t) * xs, nb, A0, A1, reinterpret_cast<float *>(A1 + nb), reinterpret_cast<int *>(reinterpret_cast<float *>(A1 + nb) + nb));
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (uint32_t r = blockIdx.x * GEMV_WARPS + warp; r < rows; r += gridDim.x * GEMV_WARPS) {
    float acc[TT];
#pragma unroll
    for (int t = 0; t < TT; t++) acc[t] = 0.0f;
    for (uint32_t c = 0; c < nb; c += 32u * U) {
      Blk<KIND, false> blk[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const uint32_t b = c + 32u * u + lane;
        if (b < nb) blk[u].load(w + (size_t)r * rowb, b, nb);
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        const uint32_t b = c + 32u * u + lane;
        if (b < nb) {
#pragma unroll
          for (int t = 0; t < TT; t++) {
            if ((uint32_t)t < nt) {
              const uint4 *A0 = smem + t * per_tok, *A1 = A0 + nb;
              const float *da = reinterpret_cast<const float *>(A1 + nb);
              const int *as = reinterpret_cast<const int *>(da + nb);
              acc[t] = blk[u].accum(acc[t], A0[b], A1[b], da[b], as[b], b);
            }
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < TT; t++) {
      const float v = warp_tree(acc[t]);
      if (lane == 0 && (uint32_t)t < nt) {
        float o = v;
        if (bias) o = __fadd_rn(o, bias[r]);
        if (res) o = __fadd_rn(reinterpret_cast<const float *>(reinterpret_cast<const char *>(res) + (size_t)(t0 + t) * rs)[r], o);
        reinterpret_cast<float *>(reinterpret_cast<char *>(y) + (size_t)(t0 + t) * ys)[r] = o;
      }
    }
  }
}

// f32 matrix: lane l sums elements l, l+32, ... in order (product rounded,
// then added), then the tree. x staged in shared memory; 8 loads in flight per lane.
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_f32_kernel(const float *__restrict__ w, uint32_t rows, uint32_t cols, const float *__restrict__ x, float *y,
                const float *__restrict__ bias, const float *res, size_t xs, size_t ys, size_t rs) {
  extern __shared__ uint4 smem[];
  float *xsm = reinterpret_cast<float *>(smem);
  const uint32_t t = blockIdx.y;
  const float *xt = reinterpret_cast<const float *>(reinterpret_cast<const char *>(x) + t * xs);
  for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) xsm[i] = xt[i];
  __syncthreads();
  y = reinterpret_cast<float *>(reinterpret_cast<char *>(y) + t * ys);
  if (res) res = reinterpret_cast<const float *>(reinterpret_cast<const char *>(res) + t * rs);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int U = 8;
  for (uint32_t r = blockIdx.x * GEMV_WARPS + warp; r < rows; r += gridDim.x * GEMV_WARPS) {
    const float *row = w + (size_t)r * cols;
    float acc = 0.0f;
    for (uint32_t c = 0; c < cols; c += 32u * U) {
      float v[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const uint32_t i = c + 32u * u + lane;
        v[u] = i < cols ? ld_stream_f32(row + i) : 0.0f;
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        const uint32_t i = c + 32u * u + lane;
        if (i < cols) acc = __fadd_rn(acc, __fmul_rn(v[u], xsm[i]));
      }
    }
    const float s = warp_tree(acc);
    if (lane == 0) {
      float o = s;
      if (bias) o = __fadd_rn(o, bias[r]);
      if (res) o = __fadd_rn(res[r], o);
      y[r] = o;
    }
  }
}

// Test hook: one thread per (row, block).
template <int KIND>
__global__ void block_dots_kernel(const uint8_t *__restrict__ w, size_t rowb, uint32_t rows, uint32_t nb, const uint8_t *__restrict__ xq,
                                  int32_t *dots) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * nb) return;
  const uint32_t r = (uint32_t)(i / nb), b = (uint32_t)(i % nb);
  const uint8_t *rp = w + (size_t)r * rowb;
  const uint4 *a = reinterpret_cast<const uint4 *>(xq) + 2u * b;
  const uint4 a0 = a[0], a1 = a[1];
  if (KIND == IE_B200_MAT_Q8) {  // eight signed dot4 (core/ie_core.h:220-233)
    const int *q8 = reinterpret_cast<const int *>(rp + 32u * (size_t)b);
    const int av[8] = {(int)a0.x, (int)a0.y, (int)a0.z, (int)a0.w, (int)a1.x, (int)a1.y, (int)a1.z, (int)a1.w};
    int dot = 0;
#pragma unroll
    for (int k = 0; k < 8; k++) dot = __dp4a(q8[k], av[k], dot);
    dots[i] = dot;
    return;
  }
  const uint4 q = *reinterpret_cast<const uint4 *>(rp + 16u * (size_t)b);
  if (KIND == IE_B200_MAT_Q6K) {
    const uint2 hw = *reinterpret_cast<const uint2 *>(rp + 16u * (size_t)nb + 8u * b);
    int d0, d1;
    q6_dots(q, hw, a0, a1, d0, d1);
    dots[2 * i] = d0, dots[2 * i + 1] = d1;
  } else if (KIND == IE_B200_MAT_Q4K) {
    dots[i] = q4_dot(q, a0, a1);
  } else {
    const int asum = reinterpret_cast<const int *>(xq + 36u * (size_t)nb)[b];
    dots[i] = q4_dot(q, a0, a1) - 8 * asum;
  }
}

// Grid: enough CTAs to fill the machine a few times over, never more than the rows need.
static unsigned gemv_grid(uint32_t rows, int rows_per_cta, int ctas_per_sm) {
  const unsigned need = (rows + rows_per_cta - 1) / rows_per_cta;
  const unsigned cap = (unsigned)(sm_count() * ctas_per_sm);
  return need < cap ? (need ? need : 1u) : cap;
}

template <int KIND, int U, int TT>
static int launch_mt(const void *w, uint32_t rows, uint32_t cols, const void *x, float *y, const float *bias, const float *res, uint32_t T,
                     size_t xs, size_t ys, size_t rs, cudaStream_t st) {
  const uint32_t nb = cols / 32u;
  const size_t smem = (size_t)nb * 40u * TT;
  auto k = gemv_mt_kernel<KIND, U, TT>;
  if (int r = ensure_dynamic_smem(reinterpret_cast<const void *>(k), smem)) return r;
  const dim3 grid(gemv_grid(rows, GEMV_WARPS, smem > 100u * 1024u ? 1 : 2), (T + TT - 1) / TT);
  k<<<grid, GEMV_THREADS, smem, st>>>(static_cast<const uint8_t *>(w), row_bytes_of(KIND, cols), rows, nb, static_cast<const uint8_t *>(x), y,
                                      bias, res, T, xs, ys, rs);
  IEB_LAUNCHED("gemv_mt_kernel");
  return IE_B200_OK;
}

template <int KIND, int R, int U>
static int launch_q(const void *w, uint32_t rows, uint32_t cols, const void *x, float *y, const float *bias, const float *res, uint32_t T,
                    size_t xs, size_t ys, size_t rs, cudaStream_t st) {
  const uint32_t nb = cols / 32u;
  // several tokens: one pass over the weights for up to 8 (4 when the rows are long) tokens, if their Q8 buffers fit
  if (T >= 2 && nb % 2u == 0 && (size_t)nb * 40u * 8u <= 200u * 1024u) return launch_mt<KIND, U, 8>(w, rows, cols, x, y, bias, res, T, xs, ys, rs, st);
  if (T >= 2 && nb % 2u == 0 && (size_t)nb * 40u * 4u <= 200u * 1024u) return launch_mt<KIND, U, 4>(w, rows, cols, x, y, bias, res, T, xs, ys, rs, st);
  const size_t smem = (size_t)nb * 40u;
  auto k = gemv_q_kernel<KIND, R, U>;
  if (int r = ensure_dynamic_smem(reinterpret_cast<const void *>(k), smem)) return r;
  const dim3 grid(gemv_grid(rows, GEMV_WARPS * R, 8), T);
  k<<<grid, GEMV_THREADS, smem, st>>>(static_cast<const uint8_t *>(w), row_bytes_of(KIND, cols), rows, nb, static_cast<const uint8_t *>(x), y,
                                      bias, res, xs, ys, rs);
  IEB_LAUNCHED("gemv_q_kernel");
  return IE_B200_OK;
}

}  // namespace ieb

using namespace ieb;

extern "C" int ie_b200_gemv(int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_x, float *d_y, const float *d_bias,
                            const float *d_res, uint32_t T, size_t x_stride, size_t y_stride, size_t res_stride, void *stream) {
  if (!d_w || !d_x || !d_y) return fail(IE_B200_E_ARG, "ie_b200_gemv: NULL pointer");
  if (!aligned16(d_w) || !aligned16(d_x)) return fail(IE_B200_E_ARG, "ie_b200_gemv: weights and activations must be 16-byte aligned");
  if (rows == 0 || T == 0) return IE_B200_OK;
  if (T > 65535u) return fail(IE_B200_E_SIZE, "ie_b200_gemv: T %u > 65535", T);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint32_t nb = cols / 32u;
  if (kind == IE_B200_MAT_F32) {
    if (cols == 0 || (size_t)cols * 4u > 200u * 1024u) return fail(IE_B200_E_SIZE, "ie_b200_gemv: f32 cols %u unsupported", cols);
    const size_t smem = (size_t)cols * 4u;
    if (int r = ensure_dynamic_smem(reinterpret_cast<const void *>(gemv_f32_kernel), smem)) return r;
    const dim3 grid(gemv_grid(rows, GEMV_WARPS, 8), T);
    gemv_f32_kernel<<<grid, GEMV_THREADS, smem, st>>>(static_cast<const float *>(d_w), rows, cols, static_cast<const float *>(d_x), d_y, d_bias,
                                                     d_res, x_stride, y_stride, res_stride);
    IEB_LAUNCHED("gemv_f32_kernel");
    return IE_B200_OK;
  }
  if (cols == 0 || cols % 32u) return fail(IE_B200_E_SIZE, "ie_b200_gemv: cols %u is not a multiple of 32", cols);
  if (nb > 4096u) return fail(IE_B200_E_SIZE, "ie_b200_gemv: %u blocks per row > 4096", nb);
  if (T > 1 && (x_stride & 15u) != 0) return fail(IE_B200_E_ARG, "ie_b200_gemv: x_stride must be a multiple of 16");
  switch (kind) {
    case IE_B200_MAT_Q4: return launch_q<IE_B200_MAT_Q4, 2, 4>(d_w, rows, cols, d_x, d_y, d_bias, d_res, T, x_stride, y_stride, res_stride, st);
    case IE_B200_MAT_Q8: return launch_q<IE_B200_MAT_Q8, 2, 2>(d_w, rows, cols, d_x, d_y, d_bias, d_res, T, x_stride, y_stride, res_stride, st);
    case IE_B200_MAT_Q4K:
      if (nb % 8u) return fail(IE_B200_E_SIZE, "ie_b200_gemv: Q4_K needs cols %% 256 == 0");
      return launch_q<IE_B200_MAT_Q4K, 2, 4>(d_w, rows, cols, d_x, d_y, d_bias, d_res, T, x_stride, y_stride, res_stride, st);
    case IE_B200_MAT_Q6K:
      if (nb % 8u) return fail(IE_B200_E_SIZE, "ie_b200_gemv: Q6_K needs cols %% 256 == 0");
      return launch_q<IE_B200_MAT_Q6K, 2, 2>(d_w, rows, cols, d_x, d_y, d_bias, d_res, T, x_stride, y_stride, res_stride, st);
    default: return fail(IE_B200_E_ARG, "ie_b200_gemv: unknown matrix kind %d", kind);
  }
}

extern "C" int ie_b200_block_dots(int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_xq, int32_t *d_dots, void *stream) {
  if (!d_w || !d_xq || !d_dots) return fail(IE_B200_E_ARG, "ie_b200_block_dots: NULL pointer");
  if (cols == 0 || cols % 32u) return fail(IE_B200_E_SIZE, "ie_b200_block_dots: cols %u is not a multiple of 32", cols);
  const uint32_t nb = cols / 32u;
  const size_t n = (size_t)rows * nb;
  if (n == 0) return IE_B200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((n + 255) / 256);
  const uint8_t *w = static_cast<const uint8_t *>(d_w), *x = static_cast<const uint8_t *>(d_xq);
  switch (kind) {
    case IE_B200_MAT_Q4: block_dots_kernel<IE_B200_MAT_Q4><<<grid, 256, 0, st>>>(w, row_bytes_of(kind, cols), rows, nb, x, d_dots); break;
    case IE_B200_MAT_Q8: block_dots_kernel<IE_B200_MAT_Q8><<<grid, 256, 0, st>>>(w, row_bytes_of(kind, cols), rows, nb, x, d_dots); break;
    case IE_B200_MAT_Q4K: block_dots_kernel<IE_B200_MAT_Q4K><<<grid, 256, 0, st>>>(w, row_bytes_of(kind, cols), rows, nb, x, d_dots); break;
    case IE_B200_MAT_Q6K: block_dots_kernel<IE_B200_MAT_Q6K><<<grid, 256, 0, st>>>(w, row_bytes_of(kind, cols), rows, nb, x, d_dots); break;
    default: return fail(IE_B200_E_ARG, "ie_b200_block_dots: unknown matrix kind %d", kind);
  }
  IEB_LAUNCHED("block_dots_kernel");
  return IE_B200_OK;
}
