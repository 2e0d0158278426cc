// glue.cu -- the small per-token kernels around the GEMVs: Q8 quantiser,
// embedding row, RMSNorm (+Q8), SwiGLU (+Q8), RoPE + KV store, argmax.
// All are latency-bound at decode; they exist so that a whole step runs on
// the device. T tokens are handled by blockIdx.y (or .x where noted) with
// byte strides between token rows.
#include <float.h>

#include <mutex>

#include "common.cuh"
#include "norm_quant.cuh"

namespace ieb {

template <typename T>
__device__ __forceinline__ T *row_ptr(T *p, size_t stride, uint32_t t) {
  return reinterpret_cast<T *>(reinterpret_cast<char *>(const_cast<typename std::remove_const<T>::type *>(p)) + stride * t);
}

// ---- Q8 quantiser: one warp per block of 32 ----
__global__ void __launch_bounds__(256) quant_q8_kernel(const float *x, uint8_t *q, uint32_t nb, size_t xs, size_t qs) {
  pdl_prologue();
  const uint32_t t = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const uint32_t b = blockIdx.x * 8u + (threadIdx.x >> 5);
  if (b >= nb) return;
  const float *xt = row_ptr(x, xs, t);
  quant_block_warp(xt[32u * b + lane], row_ptr(q, qs, t), nb, b, lane);
}

// ---- embedding row ----
__global__ void __launch_bounds__(256) embed_q4_kernel(const uint8_t *w, size_t rowb, uint32_t nb, const uint32_t *tok, float *out, size_t os) {
  pdl_prologue();
  const uint32_t t = blockIdx.y;
  const uint8_t *rp = w + (size_t)tok[t] * rowb;
  float *o = row_ptr(out, os, t);
  for (uint32_t e = blockIdx.x * blockDim.x + threadIdx.x; e < nb * 32u; e += gridDim.x * blockDim.x) {
    const uint32_t b = e >> 5, j = e & 31u;
    const uint32_t word = reinterpret_cast<const uint32_t *>(rp + 16u * (size_t)b)[(j & 15u) >> 2];
    const uint32_t nib = (word >> (8u * (j & 3u) + 4u * (j >> 4))) & 15u;
    const float d = h2f(reinterpret_cast<const uint16_t *>(rp + 16u * (size_t)nb)[b]);
    o[e] = __fmul_rn(d, (float)((int)nib - 8));
  }
}
// Q8_0 row: d * (float)(int8) weight (mat_row, src/cpu.c:257-265)
__global__ void __launch_bounds__(256) embed_q8_kernel(const uint8_t *w, size_t rowb, uint32_t nb, const uint32_t *tok, float *out, size_t os) {
  pdl_prologue();
  const uint32_t t = blockIdx.y;
  const uint8_t *rp = w + (size_t)tok[t] * rowb;
  float *o = row_ptr(out, os, t);
  for (uint32_t e = blockIdx.x * blockDim.x + threadIdx.x; e < nb * 32u; e += gridDim.x * blockDim.x) {
    const float d = h2f(reinterpret_cast<const uint16_t *>(rp + 32u * (size_t)nb)[e >> 5]);
    o[e] = __fmul_rn(d, (float)reinterpret_cast<const int8_t *>(rp)[e]);
  }
}
__global__ void __launch_bounds__(256) embed_f32_kernel(const float *w, uint32_t cols, const uint32_t *tok, float *out, size_t os) {
  pdl_prologue();
  const uint32_t t = blockIdx.y;
  const float *rp = w + (size_t)tok[t] * cols;
  float *o = row_ptr(out, os, t);
  for (uint32_t e = blockIdx.x * blockDim.x + threadIdx.x; e < cols; e += gridDim.x * blockDim.x) o[e] = rp[e];
}

// ---- RMSNorm (+Q8): one CTA of 1024 threads per token ----
__global__ void __launch_bounds__(1024) rmsnorm_kernel(const float *x, const float *__restrict__ w, float *y, uint32_t n, float eps, uint8_t *q,
                                                      size_t xs, size_t ys, size_t qs) {
  pdl_prologue();
  __shared__ float red[32];
  const uint32_t t = blockIdx.x;
  const float *xt = row_ptr(x, xs, t);
  float *yt = row_ptr(y, ys, t);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float ss = 0.0f;
  for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(xt[i], xt[i], ss);
  ss = warp_sum_all(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = lane < nw ? red[lane] : 0.0f;
  tot = warp_sum_all(tot);
  const float s = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(tot, (float)n), eps)));
  // each warp takes whole blocks of 32 so that the Q8 copy is a warp matter
  uint8_t *qt = q ? row_ptr(q, qs, t) : nullptr;
  for (uint32_t b = warp; b < n / 32u; b += nw) {
    const uint32_t i = 32u * b + lane;
    const float v = __fmul_rn(__fmul_rn(xt[i], s), w[i]);
    yt[i] = v;
    if (qt) quant_block_warp(v, qt, n / 32u, b, lane);
  }
  for (uint32_t i = (n / 32u) * 32u + threadIdx.x; i < n; i += blockDim.x) yt[i] = __fmul_rn(__fmul_rn(xt[i], s), w[i]);
}

// The same for vectors of whole 32-blocks up to 16384 elements, 16-byte aligned: each thread keeps its float4s in
// registers (one pass over x), the norm weights are fetched ahead of the dependency wait, and the Q8 copy needs no
// shared memory (norm_quant.cuh).
template <int ITERS>
__global__ void __launch_bounds__(1024) rmsnorm_vec_kernel(const float *x, const float *__restrict__ w, float *y, uint32_t n, float eps, uint8_t *q,
                                                          size_t xs, size_t ys, size_t qs) {
  __shared__ float red[32];
  const uint32_t t = blockIdx.x;
  float4 x4[ITERS], w4[ITERS];
  pdl_launch_dependents();
#pragma unroll
  for (int it = 0; it < ITERS; it++) {
    const uint32_t i = 4u * (threadIdx.x + 1024u * it);
    w4[it] = x4[it] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < n) w4[it] = *reinterpret_cast<const float4 *>(w + i);
  }
  pdl_wait();
  const float *xt = row_ptr(x, xs, t);
#pragma unroll
  for (int it = 0; it < ITERS; it++) {
    const uint32_t i = 4u * (threadIdx.x + 1024u * it);
    if (i < n) x4[it] = *reinterpret_cast<const float4 *>(xt + i);
  }
  norm_quant_vec<ITERS, 1024>(x4, w4, n, eps, row_ptr(y, ys, t), q ? row_ptr(q, qs, t) : nullptr, red);
}

// ---- SwiGLU (+Q8): one warp per 32 elements ----
__global__ void __launch_bounds__(256) swiglu_kernel(float *a, const float *b, uint32_t n, uint8_t *q, size_t as, size_t qs) {
  pdl_prologue();
  const uint32_t t = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const uint32_t blk = blockIdx.x * 8u + (threadIdx.x >> 5);
  if (blk >= (n + 31u) / 32u) return;
  float *at = row_ptr(a, as, t);
  const float *bt = row_ptr(b, as, t);
  const uint32_t i = 32u * blk + lane;
  float v = 0.0f;
  if (i < n) {
    const float g = at[i];
    v = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), bt[i]);
    at[i] = v;
  }
  if (q && 32u * blk + 32u <= n) quant_block_warp(v, row_ptr(q, qs, t), n / 32u, blk, lane);
}

// The same for interleaved input gu[2i] = gate_i, gu[2i + 1] = up_i (the layout whose GEMV rows come in gate / up
// pairs): h[i] = silu(gate_i) * up_i into a buffer of its own.
__global__ void __launch_bounds__(256) swiglu_il_kernel(const float *gu, float *h, uint32_t n, uint8_t *q, size_t gs, size_t hs, size_t qs) {
  pdl_prologue();
  const uint32_t t = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const uint32_t blk = blockIdx.x * 8u + (threadIdx.x >> 5);
  if (blk >= (n + 31u) / 32u) return;
  const uint32_t i = 32u * blk + lane;
  float v = 0.0f;
  if (i < n) {
    const float2 p = *reinterpret_cast<const float2 *>(row_ptr(gu, gs, t) + 2u * i);
    v = __fmul_rn(__fdiv_rn(p.x, __fadd_rn(1.0f, expf(-p.x))), p.y);
    row_ptr(h, hs, t)[i] = v;
  }
  if (q && 32u * blk + 32u <= n) quant_block_warp(v, row_ptr(q, qs, t), n / 32u, blk, lane);
}

// ---- RoPE of q and k in place, then K/V of the position into the cache ----
// Cache layout: [kv head][row][hd], row = position % kv_len.
template <typename KV>
__global__ void __launch_bounds__(256)
rope_kv_kernel(float *q, float *k, const float *v, KV *kc, KV *vc, const float *__restrict__ cs, const float *__restrict__ sn,
               const uint32_t *pos0, uint32_t nq, uint32_t nkv, uint32_t hd, int neox, uint32_t kv_len, size_t stride) {
  pdl_prologue();
  const uint32_t t = blockIdx.y, pos = *pos0 + t, h2 = hd / 2u;
  const uint32_t npair = (nq + nkv) * h2, total = npair + nkv * hd;
  float *qt = row_ptr(q, stride, t), *kt = row_ptr(k, stride, t);
  const float *vt = row_ptr(v, stride, t);
  const size_t row = pos % kv_len;
  for (uint32_t e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
    if (e < npair) {
      const uint32_t h = e / h2, i = e % h2;
      const bool isk = h >= nq;
      float *vec = isk ? kt + (size_t)(h - nq) * hd : qt + (size_t)h * hd;
      const uint32_t i0 = neox ? i : 2u * i, i1 = neox ? i + h2 : 2u * i + 1u;
      const float a = vec[i0], b = vec[i1], c = cs[(size_t)pos * h2 + i], s = sn[(size_t)pos * h2 + i];
      const float r0 = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)), r1 = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
      vec[i0] = r0, vec[i1] = r1;
      if (isk) {
        KV *dst = kc + ((size_t)(h - nq) * kv_len + row) * hd;
        dst[i0] = (KV)r0, dst[i1] = (KV)r1;
      }
    } else {
      const uint32_t j = e - npair, h = j / hd, i = j % hd;
      vc[((size_t)h * kv_len + row) * hd + i] = (KV)vt[j];
    }
  }
}

// ---- argmax: NG partial CTAs per row, then a merge CTA ----
constexpr int ARGMAX_NG = 64;
struct ArgPart {
  float mx;
  uint32_t idx;
  float sum;  // sum of exp(x - mx) over the part
  uint32_t pad;
};
__global__ void __launch_bounds__(256) argmax_part_kernel(const float *x, uint32_t n, ArgPart *part, size_t xs) {
  pdl_prologue();
  __shared__ float smx[8], ssum[8];
  __shared__ uint32_t sidx[8];
  const uint32_t t = blockIdx.y;
  const float *xt = row_ptr(x, xs, t);
  const uint32_t per = (n + ARGMAX_NG - 1) / ARGMAX_NG, lo = blockIdx.x * per, hi = min(n, lo + per);
  float mx = -INFINITY;
  uint32_t idx = 0xFFFFFFFFu;
  for (uint32_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = xt[i];
    if (v > mx) mx = v, idx = i;  // i rises per thread: keeps the first maximum
  }
  for (int o = 16; o; o >>= 1) {
    const float om = __shfl_xor_sync(0xFFFFFFFFu, mx, o);
    const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
    if (om > mx || (om == mx && oi < idx)) mx = om, idx = oi;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) smx[warp] = mx, sidx[warp] = idx;
  __syncthreads();
  float bm = smx[0];
  uint32_t bi = sidx[0];
  for (int k = 1; k < 8; k++)
    if (smx[k] > bm || (smx[k] == bm && sidx[k] < bi)) bm = smx[k], bi = sidx[k];
  float s = 0.0f;
  for (uint32_t i = lo + threadIdx.x; i < hi; i += blockDim.x) s += expf(xt[i] - bm);
  s = warp_sum_all(s);
  if (lane == 0) ssum[warp] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.0f;
    for (int k = 0; k < 8; k++) tot += ssum[k];
    ArgPart p = {bm, bi, tot, 0u};
    part[(size_t)t * ARGMAX_NG + blockIdx.x] = p;
  }
}
__global__ void __launch_bounds__(32) argmax_merge_kernel(const ArgPart *part, uint32_t *out, size_t os) {
  pdl_prologue();
  const uint32_t t = blockIdx.x;
  const int lane = threadIdx.x;
  float mx = -INFINITY, sum = 0.0f;
  uint32_t idx = 0xFFFFFFFFu;
  for (int k = lane; k < ARGMAX_NG; k += 32) {
    const ArgPart p = part[(size_t)t * ARGMAX_NG + k];
    if (p.idx == 0xFFFFFFFFu) continue;
    if (p.mx > mx || (p.mx == mx && p.idx < idx)) {
      sum = sum * expf(mx - p.mx) + p.sum;
      mx = p.mx, idx = p.idx;
    } else {
      sum += p.sum * expf(p.mx - mx);
    }
  }
  for (int o = 16; o; o >>= 1) {
    const float om = __shfl_xor_sync(0xFFFFFFFFu, mx, o), osum = __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
    if (oi == 0xFFFFFFFFu) continue;
    if (idx == 0xFFFFFFFFu || om > mx || (om == mx && oi < idx)) {
      sum = (idx == 0xFFFFFFFFu ? 0.0f : sum * expf(mx - om)) + osum;
      mx = om, idx = oi;
    } else {
      sum += osum * expf(om - mx);
    }
  }
  if (lane == 0) {
    uint32_t *o = row_ptr(out, os, t);
    o[0] = idx == 0xFFFFFFFFu ? 0u : idx;
    o[1] = __float_as_uint(sum > 0.0f ? 1.0f / sum : 0.0f);
  }
}

// ---- top K of a row: K <= 64 largest values, descending, equal values by rising index ----
// Two launches: every CTA of the first keeps a slice of 2048 values in registers (8 per thread) and takes its K best one at
// a time (the thread's own best, a shuffle tree over the warp, eight warp winners through shared memory; the owner of the
// winner strikes it out); the second does the same over the slices' K candidates of a row.
constexpr int TK_THREADS = 256, TK_SLICE = 2048, TK_MAXK = 64, TK_MERGE_PER = 24;
constexpr uint32_t TK_NONE = 0xFFFFFFFFu;
__device__ __forceinline__ bool tk_better(float v, uint32_t i, float bv, uint32_t bi) {
  return i != TK_NONE && (bi == TK_NONE || v > bv || (v == bv && i < bi));
}
template <int PER>
__device__ __forceinline__ void tk_select(float (&v)[PER], uint32_t (&id)[PER], uint32_t K, float *out_v, uint32_t *out_i) {
  __shared__ float wv[TK_THREADS / 32];
  __shared__ uint32_t wi[TK_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (uint32_t k = 0; k < K; k++) {
    float bv = 0.0f;
    uint32_t bi = TK_NONE;
#pragma unroll
    for (int j = 0; j < PER; j++)
      if (tk_better(v[j], id[j], bv, bi)) bv = v[j], bi = id[j];
    for (int o = 16; o; o >>= 1) {
      const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
      const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
      if (tk_better(ov, oi, bv, bi)) bv = ov, bi = oi;
    }
    if (lane == 0) wv[warp] = bv, wi[warp] = bi;
    __syncthreads();
    bv = wv[0], bi = wi[0];
#pragma unroll
    for (int w = 1; w < TK_THREADS / 32; w++)
      if (tk_better(wv[w], wi[w], bv, bi)) bv = wv[w], bi = wi[w];
    __syncthreads();
    if (threadIdx.x == 0) out_v[k] = bi == TK_NONE ? -INFINITY : bv, out_i[k] = bi;
#pragma unroll
    for (int j = 0; j < PER; j++)
      if (id[j] == bi) id[j] = TK_NONE;  // indices are unique within a row: only the owner strikes
  }
}
__global__ void __launch_bounds__(TK_THREADS) topk_part_kernel(const float *x, uint32_t nv, size_t xs, uint32_t K, uint32_t ng, float *cv, uint32_t *ci) {
  pdl_prologue();
  const uint32_t g = blockIdx.x, t = blockIdx.y;
  const float *row = row_ptr(x, xs, t);
  float v[TK_SLICE / TK_THREADS];
  uint32_t id[TK_SLICE / TK_THREADS];
#pragma unroll
  for (int j = 0; j < TK_SLICE / TK_THREADS; j++) {
    const uint32_t i = g * TK_SLICE + j * TK_THREADS + threadIdx.x;
    v[j] = i < nv ? row[i] : 0.0f, id[j] = i < nv ? i : TK_NONE;
  }
  tk_select(v, id, K, cv + ((size_t)t * ng + g) * K, ci + ((size_t)t * ng + g) * K);
}
__global__ void __launch_bounds__(TK_THREADS) topk_merge_kernel(const float *cv, const uint32_t *ci, uint32_t nc, uint32_t K, float *ov, uint32_t *oi) {
  pdl_prologue();
  const uint32_t t = blockIdx.x;
  float v[TK_MERGE_PER];
  uint32_t id[TK_MERGE_PER];
#pragma unroll
  for (int j = 0; j < TK_MERGE_PER; j++) {
    const uint32_t p = j * TK_THREADS + threadIdx.x;
    v[j] = p < nc ? cv[(size_t)t * nc + p] : 0.0f, id[j] = p < nc ? ci[(size_t)t * nc + p] : TK_NONE;
  }
  tk_select(v, id, K, ov + (size_t)t * K, oi + (size_t)t * K);
}

}  // namespace ieb

using namespace ieb;

extern "C" size_t ie_b200_topk_scratch_bytes(uint32_t nv, uint32_t K, uint32_t T) {
  const size_t ng = (nv + TK_SLICE - 1) / TK_SLICE;
  return (size_t)T * ng * K * 8u + 256u;
}

extern "C" int ie_b200_topk(const float *d_x, uint32_t nv, uint32_t K, uint32_t T, size_t x_stride, float *d_val, uint32_t *d_idx, void *d_scratch,
                            void *stream) {
  if (!d_x || !d_val || !d_idx || !d_scratch) return fail(IE_B200_E_ARG, "ie_b200_topk: NULL pointer");
  const uint32_t ng = (nv + TK_SLICE - 1) / TK_SLICE;
  if (K == 0 || K > (uint32_t)TK_MAXK || K > nv || (uint64_t)ng * K > (uint64_t)TK_MERGE_PER * TK_THREADS)
    return fail(IE_B200_E_SIZE, "ie_b200_topk: K = %u of %u values (1 .. %d, at most %d candidates per row)", K, nv, TK_MAXK, TK_MERGE_PER * TK_THREADS);
  if (T == 0) return IE_B200_OK;
  if (T > 65535u) return fail(IE_B200_E_SIZE, "ie_b200_topk: T %u > 65535", T);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float *cv = static_cast<float *>(d_scratch);
  uint32_t *ci = reinterpret_cast<uint32_t *>(cv + (size_t)T * ng * K);
  IEB_LAUNCH_PDL("topk_part_kernel", topk_part_kernel, dim3(ng, T), dim3(TK_THREADS), 0, st, d_x, nv, x_stride, K, ng, cv, ci);
  IEB_LAUNCH_PDL("topk_merge_kernel", topk_merge_kernel, dim3(T), dim3(TK_THREADS), 0, st, static_cast<const float *>(cv), static_cast<const uint32_t *>(ci),
                 ng * K, K, d_val, d_idx);
  return IE_B200_OK;
}

extern "C" int ie_b200_quant_q8(const float *d_x, void *d_q, uint32_t nb, uint32_t T, size_t x_stride, size_t q_stride, void *stream) {
  if (!d_x || !d_q) return fail(IE_B200_E_ARG, "ie_b200_quant_q8: NULL pointer");
  if (((uintptr_t)d_q & 3u) || (q_stride & 3u)) return fail(IE_B200_E_ARG, "ie_b200_quant_q8: output must be 4-byte aligned");
  if (nb == 0 || T == 0) return IE_B200_OK;
  if (T > 65535u) return fail(IE_B200_E_SIZE, "ie_b200_quant_q8: T %u > 65535", T);
  IEB_LAUNCH_PDL("quant_q8_kernel", quant_q8_kernel, dim3((nb + 7u) / 8u, T), dim3(256), 0, static_cast<cudaStream_t>(stream), d_x,
                 static_cast<uint8_t *>(d_q), nb, x_stride, q_stride);
  return IE_B200_OK;
}

extern "C" int ie_b200_embed(int kind, const void *d_w, uint32_t cols, const uint32_t *d_tok, float *d_out, uint32_t T, size_t out_stride,
                             void *stream) {
  if (!d_w || !d_tok || !d_out) return fail(IE_B200_E_ARG, "ie_b200_embed: NULL pointer");
  if (T == 0 || cols == 0) return IE_B200_OK;
  if (T > 65535u) return fail(IE_B200_E_SIZE, "ie_b200_embed: T %u > 65535", T);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid((cols + 255u) / 256u, T);
  if (kind == IE_B200_MAT_Q4) {
    if (cols % 32u) return fail(IE_B200_E_SIZE, "ie_b200_embed: cols %u is not a multiple of 32", cols);
    IEB_LAUNCH_PDL("embed_q4_kernel", embed_q4_kernel, grid, dim3(256), 0, st, static_cast<const uint8_t *>(d_w), row_bytes_of(kind, cols),
                   cols / 32u, d_tok, d_out, out_stride);
  } else if (kind == IE_B200_MAT_Q8) {
    if (cols % 32u) return fail(IE_B200_E_SIZE, "ie_b200_embed: cols %u is not a multiple of 32", cols);
    IEB_LAUNCH_PDL("embed_q8_kernel", embed_q8_kernel, grid, dim3(256), 0, st, static_cast<const uint8_t *>(d_w), row_bytes_of(kind, cols),
                   cols / 32u, d_tok, d_out, out_stride);
  } else if (kind == IE_B200_MAT_F32) {
    IEB_LAUNCH_PDL("embed_f32_kernel", embed_f32_kernel, grid, dim3(256), 0, st, static_cast<const float *>(d_w), cols, d_tok, d_out, out_stride);
  } else {
    return fail(IE_B200_E_ARG, "ie_b200_embed: kind %d has no embedding kernel", kind);
  }
  return IE_B200_OK;
}

extern "C" int ie_b200_rmsnorm(const float *d_x, const float *d_w, float *d_y, uint32_t n, float eps, void *d_q, uint32_t T, size_t x_stride,
                               size_t y_stride, size_t q_stride, void *stream) {
  if (!d_x || !d_w || !d_y) return fail(IE_B200_E_ARG, "ie_b200_rmsnorm: NULL pointer");
  if (d_q && n % 32u) return fail(IE_B200_E_SIZE, "ie_b200_rmsnorm: the Q8 copy needs n %% 32 == 0 (n = %u)", n);
  if (n == 0 || T == 0) return IE_B200_OK;
  if (n % 32u == 0 && n <= 16384u && aligned16(d_x) && aligned16(d_w) && aligned16(d_y) && (!d_q || aligned16(d_q)) &&
      (T == 1 || (x_stride % 16u == 0 && y_stride % 16u == 0 && q_stride % 16u == 0))) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t *q = static_cast<uint8_t *>(d_q);
    const uint32_t iters = (n + 4095u) / 4096u;
    if (iters == 1) IEB_LAUNCH_PDL("rmsnorm_vec_kernel", rmsnorm_vec_kernel<1>, dim3(T), dim3(1024), 0, st, d_x, d_w, d_y, n, eps, q, x_stride, y_stride, q_stride);
    else if (iters == 2) IEB_LAUNCH_PDL("rmsnorm_vec_kernel", rmsnorm_vec_kernel<2>, dim3(T), dim3(1024), 0, st, d_x, d_w, d_y, n, eps, q, x_stride, y_stride, q_stride);
    else IEB_LAUNCH_PDL("rmsnorm_vec_kernel", rmsnorm_vec_kernel<4>, dim3(T), dim3(1024), 0, st, d_x, d_w, d_y, n, eps, q, x_stride, y_stride, q_stride);
    return IE_B200_OK;
  }
  IEB_LAUNCH_PDL("rmsnorm_kernel", rmsnorm_kernel, dim3(T), dim3(1024), 0, static_cast<cudaStream_t>(stream), d_x, d_w, d_y, n, eps,
                 static_cast<uint8_t *>(d_q), x_stride, y_stride, q_stride);
  return IE_B200_OK;
}

extern "C" int ie_b200_swiglu(float *d_a, const float *d_b, uint32_t n, void *d_q, uint32_t T, size_t a_stride, size_t q_stride, void *stream) {
  if (!d_a || !d_b) return fail(IE_B200_E_ARG, "ie_b200_swiglu: NULL pointer");
  if (d_q && n % 32u) return fail(IE_B200_E_SIZE, "ie_b200_swiglu: the Q8 copy needs n %% 32 == 0 (n = %u)", n);
  if (n == 0 || T == 0) return IE_B200_OK;
  if (T > 65535u) return fail(IE_B200_E_SIZE, "ie_b200_swiglu: T %u > 65535", T);
  const uint32_t nblk = (n + 31u) / 32u;
  IEB_LAUNCH_PDL("swiglu_kernel", swiglu_kernel, dim3((nblk + 7u) / 8u, T), dim3(256), 0, static_cast<cudaStream_t>(stream), d_a, d_b, n,
                 static_cast<uint8_t *>(d_q), a_stride, q_stride);
  return IE_B200_OK;
}

extern "C" int ie_b200_swiglu_il(const float *d_gu, float *d_h, uint32_t n, void *d_q, uint32_t T, size_t gu_stride, size_t h_stride,
                                 size_t q_stride, void *stream) {
  if (!d_gu || !d_h) return fail(IE_B200_E_ARG, "ie_b200_swiglu_il: NULL pointer");
  if (d_q && n % 32u) return fail(IE_B200_E_SIZE, "ie_b200_swiglu_il: the Q8 copy needs n %% 32 == 0 (n = %u)", n);
  if (((uintptr_t)d_gu & 7u) || (gu_stride & 7u)) return fail(IE_B200_E_ARG, "ie_b200_swiglu_il: the gate / up pairs must be 8-byte aligned");
  if (n == 0 || T == 0) return IE_B200_OK;
  if (T > 65535u) return fail(IE_B200_E_SIZE, "ie_b200_swiglu_il: T %u > 65535", T);
  const uint32_t nblk = (n + 31u) / 32u;
  IEB_LAUNCH_PDL("swiglu_il_kernel", swiglu_il_kernel, dim3((nblk + 7u) / 8u, T), dim3(256), 0, static_cast<cudaStream_t>(stream), d_gu, d_h, n,
                 static_cast<uint8_t *>(d_q), gu_stride, h_stride, q_stride);
  return IE_B200_OK;
}

extern "C" int ie_b200_rope_kv(float *d_q, float *d_k, const float *d_v, void *d_kc, void *d_vc, const float *d_cos, const float *d_sin,
                               const uint32_t *d_pos, uint32_t nq, uint32_t nkv, uint32_t hd, int neox, int kv_f32, uint32_t kv_len, uint32_t T,
                               size_t qkv_stride, void *stream) {
  if (!d_q || !d_k || !d_v || !d_kc || !d_vc || !d_cos || !d_sin || !d_pos) return fail(IE_B200_E_ARG, "ie_b200_rope_kv: NULL pointer");
  if (hd == 0 || hd % 2u || kv_len == 0) return fail(IE_B200_E_SIZE, "ie_b200_rope_kv: head dim %u, cache rows %u", hd, kv_len);
  if (T == 0) return IE_B200_OK;
  if (T > 65535u) return fail(IE_B200_E_SIZE, "ie_b200_rope_kv: T %u > 65535", T);
  const uint32_t total = (nq + nkv) * (hd / 2u) + nkv * hd;
  const dim3 grid((total + 255u) / 256u, T);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (kv_f32)
    IEB_LAUNCH_PDL("rope_kv_kernel", rope_kv_kernel<float>, grid, dim3(256), 0, st, d_q, d_k, d_v, static_cast<float *>(d_kc),
                   static_cast<float *>(d_vc), d_cos, d_sin, d_pos, nq, nkv, hd, neox, kv_len, qkv_stride);
  else
    IEB_LAUNCH_PDL("rope_kv_kernel", rope_kv_kernel<__half>, grid, dim3(256), 0, st, d_q, d_k, d_v, static_cast<__half *>(d_kc),
                   static_cast<__half *>(d_vc), d_cos, d_sin, d_pos, nq, nkv, hd, neox, kv_len, qkv_stride);
  return IE_B200_OK;
}

extern "C" size_t ie_b200_argmax_part_bytes(uint32_t T) { return (size_t)T * ARGMAX_NG * sizeof(ArgPart); }

extern "C" int ie_b200_argmax(const float *d_x, uint32_t n, uint32_t *d_out, uint32_t T, size_t x_stride, size_t out_stride, void *d_part,
                              void *stream) {
  if (!d_x || !d_out || !d_part) return fail(IE_B200_E_ARG, "ie_b200_argmax: NULL pointer");
  if (n == 0) return fail(IE_B200_E_SIZE, "ie_b200_argmax: empty row");
  if (T == 0) return IE_B200_OK;
  if (T > 65535u) return fail(IE_B200_E_SIZE, "ie_b200_argmax: T %u > 65535", T);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  IEB_LAUNCH_PDL("argmax_part_kernel", argmax_part_kernel, dim3(ARGMAX_NG, T), dim3(256), 0, st, d_x, n, static_cast<ArgPart *>(d_part), x_stride);
  IEB_LAUNCH_PDL("argmax_merge_kernel", argmax_merge_kernel, dim3(T), dim3(32), 0, st, static_cast<const ArgPart *>(d_part), d_out, out_stride);
  return IE_B200_OK;
}

// ---- argmax for callers that must not allocate --------------------------------------------------------------
// Some hosts of this library have handed out all of their device memory before the first token: a server that
// sizes its arena and KV cache to fill the GPU at start-up, or code running inside a region where the CUDA
// allocator may not be entered (a latency-critical sampling callback, a memory-audited deployment). They cannot
// cudaMalloc the partials that ie_b200_argmax needs. This variant keeps them in a fixed array in the library's
// own device image instead: 64 rows x 64 partials x 16 bytes = 64 KB, held by every GPU that loads the library
// until the process exits.
namespace ieb {
constexpr uint32_t ARGMAX_STATIC_ROWS = 64;
static __device__ __align__(256) ArgPart g_argmax_scratch[ARGMAX_STATIC_ROWS * ARGMAX_NG];

// The device address of g_argmax_scratch on the current device. In host code the array's name is only a
// stand-in for the symbol, not an address a kernel can use, so the address is asked for once per device (with
// that device current) and remembered.
static int argmax_scratch_ptr(ArgPart **out) {
  constexpr int MAX_DEV = 64;
  static ArgPart *cached[MAX_DEV] = {};
  static std::mutex mu;
  int dev = 0;
  IEB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEV) return fail(IE_B200_E_ARG, "ie_b200_argmax_static: device %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    void *p = nullptr;
    IEB_CUDA(cudaGetSymbolAddress(&p, g_argmax_scratch));
    cached[dev] = static_cast<ArgPart *>(p);
  }
  *out = cached[dev];
  return IE_B200_OK;
}
}  // namespace ieb

extern "C" uint32_t ie_b200_argmax_static_max_rows(void) { return ARGMAX_STATIC_ROWS; }

extern "C" int ie_b200_argmax_static(const float *d_x, uint32_t n, uint32_t *d_out, uint32_t T, size_t x_stride, size_t out_stride, void *stream) {
  if (!d_x || !d_out) return fail(IE_B200_E_ARG, "ie_b200_argmax_static: NULL pointer");
  if (n == 0) return fail(IE_B200_E_SIZE, "ie_b200_argmax_static: empty row");
  if (T > ARGMAX_STATIC_ROWS)
    return fail(IE_B200_E_SIZE, "ie_b200_argmax_static: %u rows exceed the %u the built-in scratch holds (use ie_b200_argmax with your own scratch)", T,
                ARGMAX_STATIC_ROWS);
  if (T == 0) return IE_B200_OK;
  ArgPart *part = nullptr;
  if (int r = argmax_scratch_ptr(&part)) return r;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  IEB_LAUNCH_PDL("argmax_part_kernel", argmax_part_kernel, dim3(ARGMAX_NG, T), dim3(256), 0, st, d_x, n, part, x_stride);
  IEB_LAUNCH_PDL("argmax_merge_kernel", argmax_merge_kernel, dim3(T), dim3(32), 0, st, static_cast<const ArgPart *>(part), d_out, out_stride);
  return IE_B200_OK;
}
