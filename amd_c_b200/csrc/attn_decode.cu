// attn_decode.cu -- split-KV decode attention with the K/V of a KV head read
// once for all of its G query heads (grouped-query attention).
//
// Grid: (split s, KV head g, token t). The positions 0 .. np-1 of token t
// (np = first position + t + 1) are cut into S equal spans, a multiple of the
// tile (64 positions). A CTA streams its span tile by tile: K and V tiles
// (contiguous in the head-major cache [kv head][row][hd]) arrive in shared
// memory through double-buffered 16-byte async copies; 8 lanes share one
// position for q.k (q in registers, 3 shuffles per head), one warp per head
// keeps the running max / sum (online softmax), and every lane owns hd/32
// output dims for p.v. Each CTA writes (max, sum, out[hd]) per head to the
// partials buffer; the last CTA of a (token, KV head) to arrive merges the S
// partials in split order, divides, and writes the f32 output and its Q8 copy.
// Bound by HBM at long context: 2 * np * hd * sizeof(KV) bytes per KV head.
#include <cuda_pipeline_primitives.h>

#include "common.cuh"

namespace ieb {

constexpr int ATT_THREADS = 256, ATT_WARPS = 8, ATT_TILE = 64;

template <typename KV>
__device__ __forceinline__ void load_slice(const KV *p, float *out, int n);
template <>
__device__ __forceinline__ void load_slice<float>(const float *p, float *out, int n) {
  for (int j = 0; j < n; j += 4) {
    const float4 v = *reinterpret_cast<const float4 *>(p + j);
    out[j] = v.x, out[j + 1] = v.y, out[j + 2] = v.z, out[j + 3] = v.w;
  }
}
template <>
__device__ __forceinline__ void load_slice<__half>(const __half *p, float *out, int n) {
  for (int j = 0; j < n; j += 4) {
    const uint2 v = *reinterpret_cast<const uint2 *>(p + j);
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&v.x)), b = __half22float2(*reinterpret_cast<const __half2 *>(&v.y));
    out[j] = a.x, out[j + 1] = a.y, out[j + 2] = b.x, out[j + 3] = b.y;
  }
}

struct AttnArgs {
  const float *q;
  const void *kc, *vc;
  float *out;
  uint8_t *oq;
  const uint32_t *pos;
  uint32_t n_head, n_kv, kv_len, S;
  size_t q_stride, out_stride, oq_stride;
  float *part;
  uint32_t *count;
  float scale;
  // fused RoPE + KV store (one token): q is the un-rotated q of the qkv buffer, k_new / v_new the un-rotated k
  // and the v of this position, cs / sn the RoPE table rows of all positions
  const float *k_new, *v_new, *cs, *sn;
  int neox;
};

constexpr uint32_t ATT_MIN_SPAN = 256;  // positions a split covers at least: short contexts stay in one CTA per KV head (no merge)

// a * c - b * s and a * s + b * c with every product rounded, as the RoPE kernel and the CPU do
__device__ __forceinline__ float rope_lo(float a, float b, float c, float s) { return __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)); }
__device__ __forceinline__ float rope_hi(float a, float b, float c, float s) { return __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c)); }

template <typename KV, int HD, int G, bool FUSED>
__global__ void __launch_bounds__(ATT_THREADS) attn_decode_kernel(const AttnArgs a) {
  constexpr int DPL = HD / 8;   // dims per lane in the q.k phase (8 lanes per position)
  constexpr int DPV = HD / 32;  // dims per lane in the p.v phase
  constexpr int TILE = ATT_TILE;
  constexpr int TILE_ELEMS = TILE * HD;
  extern __shared__ uint4 smem_raw[];
  KV *kbuf = reinterpret_cast<KV *>(smem_raw);           // [2][TILE][HD]
  KV *vbuf = kbuf + 2 * TILE_ELEMS;                      // [2][TILE][HD]
  float *P = reinterpret_cast<float *>(vbuf + 2 * TILE_ELEMS);  // [G][TILE] scores, then probabilities
  float *alpha = P + G * TILE;                           // [G]
  __shared__ float run_m[8], run_l[8];
  __shared__ uint32_t is_last;

  pdl_prologue();
  const uint32_t s = blockIdx.x, g = blockIdx.y, t = blockIdx.z, S = a.S;
  const uint32_t np = *a.pos + t + 1u;
  uint32_t span = max((np + S - 1u) / S, ATT_MIN_SPAN);
  span = (span + TILE - 1u) / TILE * TILE;
  const uint32_t A = (np + span - 1u) / span;  // splits that hold positions; the others have nothing to do
  if (s >= A) return;
  const uint32_t p_lo = s * span, p_hi = min(np, p_lo + span);
  const bool owns_new = FUSED && s == A - 1u;  // this CTA's span ends with the step's own position
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float *qt = reinterpret_cast<const float *>(reinterpret_cast<const char *>(a.q) + a.q_stride * t) + (size_t)g * G * HD;
  const KV *kh = static_cast<const KV *>(a.kc) + (size_t)g * a.kv_len * HD, *vh = static_cast<const KV *>(a.vc) + (size_t)g * a.kv_len * HD;

  float o[G][DPV];
#pragma unroll
  for (int h = 0; h < G; h++)
#pragma unroll
    for (int d = 0; d < DPV; d++) o[h][d] = 0.0f;
  if (threadIdx.x < 8) run_m[threadIdx.x] = -INFINITY, run_l[threadIdx.x] = 0.0f;

  if (p_lo < p_hi) {
    // q slices of this lane for the q.k phase
    const int sub = lane & 7, grp = lane >> 3;
    float qr[G][DPL];
#pragma unroll
    for (int h = 0; h < G; h++)
#pragma unroll
      for (int j = 0; j < DPL; j++) qr[h][j] = qt[h * HD + sub * DPL + j];
    if (FUSED) {  // rotate q in registers with the table row of this position
      const float *cs = a.cs + (size_t)(np - 1u) * (HD / 2), *sn = a.sn + (size_t)(np - 1u) * (HD / 2);
      if (!a.neox) {  // pairs (2i, 2i+1): both in this lane
#pragma unroll
        for (int j = 0; j < DPL; j += 2) {
          const int i = (sub * DPL + j) / 2;
          const float c = cs[i], sv = sn[i];
#pragma unroll
          for (int h = 0; h < G; h++) {
            const float x0 = qr[h][j], x1 = qr[h][j + 1];
            qr[h][j] = rope_lo(x0, x1, c, sv), qr[h][j + 1] = rope_hi(x0, x1, c, sv);
          }
        }
      } else {  // pairs (i, i + hd/2): the partner dim sits in the lane 4 further in the 8-lane group
#pragma unroll
        for (int j = 0; j < DPL; j++) {
          const int dim = sub * DPL + j, i = dim < HD / 2 ? dim : dim - HD / 2;
          const float c = cs[i], sv = sn[i];
#pragma unroll
          for (int h = 0; h < G; h++) {
            const float mine = qr[h][j], other = __shfl_xor_sync(0xFFFFFFFFu, mine, 4);
            qr[h][j] = dim < HD / 2 ? rope_lo(mine, other, c, sv) : rope_hi(other, mine, c, sv);
          }
        }
      }
    }
    // the step's own K and V row: rotated, written to the cache, and (below) dropped into the last tile
    KV newk0 = KV(0.f), newk1 = KV(0.f), newv = KV(0.f);
    int nk0 = 0, nk1 = 0;
    if (owns_new) {
      const uint32_t row = (np - 1u) % a.kv_len;
      if (threadIdx.x < HD / 2) {
        const int i = threadIdx.x;
        nk0 = a.neox ? i : 2 * i, nk1 = a.neox ? i + HD / 2 : 2 * i + 1;
        const float x0 = a.k_new[g * HD + nk0], x1 = a.k_new[g * HD + nk1];
        const float c = a.cs[(size_t)(np - 1u) * (HD / 2) + i], sv = a.sn[(size_t)(np - 1u) * (HD / 2) + i];
        newk0 = KV(rope_lo(x0, x1, c, sv)), newk1 = KV(rope_hi(x0, x1, c, sv));
        KV *dst = const_cast<KV *>(kh) + (size_t)row * HD;
        dst[nk0] = newk0, dst[nk1] = newk1;
      } else if (threadIdx.x >= 128 && threadIdx.x < 128 + HD) {
        const int i = threadIdx.x - 128;
        newv = KV(a.v_new[g * HD + i]);
        const_cast<KV *>(vh)[(size_t)row * HD + i] = newv;
      }
    }

    constexpr int CHUNKS = TILE_ELEMS * (int)sizeof(KV) / 16;  // 16-byte pieces per tile
    constexpr int PER_ROW = HD * (int)sizeof(KV) / 16;
    auto issue = [&](uint32_t tile_lo, int buf) {
      const char *ks = reinterpret_cast<const char *>(kh + (size_t)tile_lo * HD), *vs = reinterpret_cast<const char *>(vh + (size_t)tile_lo * HD);
      char *kd = reinterpret_cast<char *>(kbuf + buf * TILE_ELEMS), *vd = reinterpret_cast<char *>(vbuf + buf * TILE_ELEMS);
      const uint32_t rows_ok = p_hi - tile_lo - (owns_new ? 1u : 0u);  // rows past the span (and the step's own row, placed below) are zero-filled
      for (int c = threadIdx.x; c < CHUNKS; c += ATT_THREADS) {
        const bool ok = (uint32_t)(c / PER_ROW) < rows_ok;
        const size_t off = ok ? (size_t)c * 16u : 0u;
        __pipeline_memcpy_async(kd + (size_t)c * 16u, ks + off, 16, ok ? 0 : 16);
        __pipeline_memcpy_async(vd + (size_t)c * 16u, vs + off, 16, ok ? 0 : 16);
      }
      __pipeline_commit();
    };

    const uint32_t n_tiles = (p_hi - p_lo + TILE - 1u) / TILE;
    issue(p_lo, 0);
    for (uint32_t it = 0; it < n_tiles; it++) {
      const int buf = it & 1;
      const uint32_t tile_lo = p_lo + it * TILE;
      if (it + 1 < n_tiles) issue(tile_lo + TILE, buf ^ 1);
      else __pipeline_commit();
      __pipeline_wait_prior(1);
      __syncthreads();
      if (owns_new && it + 1 == n_tiles) {  // the step's own row goes into the tile from registers
        const uint32_t pr = np - 1u - tile_lo;
        if (threadIdx.x < HD / 2) {
          KV *dk = kbuf + buf * TILE_ELEMS + pr * HD;
          dk[nk0] = newk0, dk[nk1] = newk1;
        } else if (threadIdx.x >= 128 && threadIdx.x < 128 + HD) {
          vbuf[buf * TILE_ELEMS + pr * HD + (threadIdx.x - 128)] = newv;
        }
        __syncthreads();
      }
      // ---- scores: 8 lanes per position, each warp 8 positions of the tile
      const KV *kt = kbuf + buf * TILE_ELEMS;
#pragma unroll
      for (int r = 0; r < 2; r++) {
        const int pi = warp * 8 + r * 4 + grp;
        float kr[DPL];
        load_slice<KV>(kt + pi * HD + sub * DPL, kr, DPL);
#pragma unroll
        for (int h = 0; h < G; h++) {
          float d = 0.0f;
#pragma unroll
          for (int j = 0; j < DPL; j++) d = fmaf(qr[h][j], kr[j], d);
          d += __shfl_xor_sync(0xFFFFFFFFu, d, 1);
          d += __shfl_xor_sync(0xFFFFFFFFu, d, 2);
          d += __shfl_xor_sync(0xFFFFFFFFu, d, 4);
          if (sub == 0) P[h * TILE + pi] = tile_lo + pi < p_hi ? d * a.scale : -INFINITY;
        }
      }
      __syncthreads();
      // ---- running max / sum: warp h owns head h
      if (warp < G) {
        const float s0 = P[warp * TILE + lane], s1 = P[warp * TILE + 32 + lane];
        const float m_old = run_m[warp], m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
        const float e0 = expf(s0 - m_new), e1 = expf(s1 - m_new);
        P[warp * TILE + lane] = e0, P[warp * TILE + 32 + lane] = e1;
        const float sum = warp_sum_all(e0 + e1), al = expf(m_old - m_new);
        if (lane == 0) run_l[warp] = run_l[warp] * al + sum, run_m[warp] = m_new, alpha[warp] = al;
      }
      __syncthreads();
      // ---- p.v: warp w takes positions w, w+8, ... of the tile
      const KV *vt = vbuf + buf * TILE_ELEMS;
#pragma unroll
      for (int h = 0; h < G; h++) {
        const float al = alpha[h];
#pragma unroll
        for (int d = 0; d < DPV; d++) o[h][d] *= al;
      }
      for (int pi = warp; pi < TILE; pi += ATT_WARPS) {
        float vr[DPV];
        if (DPV >= 4) {
          load_slice<KV>(vt + pi * HD + lane * DPV, vr, DPV);
        } else {
#pragma unroll
          for (int d = 0; d < DPV; d++) vr[d] = (float)vt[pi * HD + lane * DPV + d];
        }
#pragma unroll
        for (int h = 0; h < G; h++) {
          const float p = P[h * TILE + pi];
#pragma unroll
          for (int d = 0; d < DPV; d++) o[h][d] = fmaf(p, vr[d], o[h][d]);
        }
      }
      __syncthreads();
    }
    __pipeline_wait_prior(0);
  }
  __syncthreads();

  // ---- reduce the 8 warps' partial outputs (shared memory, reusing the tile buffers)
  float *red = reinterpret_cast<float *>(smem_raw);  // [ATT_WARPS][G][HD]
#pragma unroll
  for (int h = 0; h < G; h++)
#pragma unroll
    for (int d = 0; d < DPV; d++) red[(warp * G + h) * HD + lane * DPV + d] = o[h][d];
  __syncthreads();
  // ---- final values of this KV head's G heads in shared memory: directly when one split held everything,
  // else through the partials buffer, merged by the last split to arrive
  const size_t rec = HD + 2;
  float *fin = red + ATT_WARPS * G * HD;  // [G][HD]
  if (A == 1u) {
    for (int e = threadIdx.x; e < G * HD; e += ATT_THREADS) {
      float acc = 0.0f;
#pragma unroll
      for (int w = 0; w < ATT_WARPS; w++) acc += red[w * G * HD + e];
      fin[e] = acc * (1.0f / run_l[e / HD]);
    }
  } else {
    for (int e = threadIdx.x; e < G * HD; e += ATT_THREADS) {
      const int h = e / HD;
      float acc = 0.0f;
#pragma unroll
      for (int w = 0; w < ATT_WARPS; w++) acc += red[w * G * HD + e];
      float *pr = a.part + (((size_t)t * a.n_head + (size_t)g * G + h) * S + s) * rec;
      pr[2 + (e % HD)] = acc;
      if (e % HD == 0) pr[0] = run_m[h], pr[1] = run_l[h];
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t prev = atomicAdd(&a.count[t * a.n_kv + g], 1u);
      is_last = prev == A - 1u;
      if (is_last) a.count[t * a.n_kv + g] = 0u;  // left zero for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int e = threadIdx.x; e < G * HD; e += ATT_THREADS) {  // merge the A partials in split order
      const float *pr = a.part + ((size_t)t * a.n_head + (size_t)g * G + e / HD) * S * rec;
      float M = -INFINITY;
      for (uint32_t k = 0; k < A; k++) M = fmaxf(M, __ldcg(pr + k * rec));
      float L = 0.0f, acc = 0.0f;
      for (uint32_t k = 0; k < A; k++) {
        const float wk = expf(__ldcg(pr + k * rec) - M);
        L = fmaf(wk, __ldcg(pr + k * rec + 1), L);
        acc = fmaf(wk, __ldcg(pr + k * rec + 2 + (e % HD)), acc);
      }
      fin[e] = acc * (1.0f / L);
    }
  }
  __syncthreads();
  // ---- write out, one warp per block of 32 values (which is also a Q8 block of the output vector)
  float *ot = reinterpret_cast<float *>(reinterpret_cast<char *>(a.out) + a.out_stride * t) + (size_t)g * G * HD;
  uint8_t *oqt = a.oq ? a.oq + a.oq_stride * t : nullptr;
  const uint32_t nbq = a.n_head * HD / 32u;
  for (int b = warp; b < G * HD / 32; b += ATT_WARPS) {
    const float v = fin[32 * b + lane];
    ot[32 * b + lane] = v;
    if (oqt) quant_block_warp(v, oqt, nbq, g * (G * HD / 32u) + b, lane);
  }
}

template <typename KV, int HD, int G, bool FUSED>
static int launch_attn(const AttnArgs &a, uint32_t T, cudaStream_t st) {
  const size_t tile = (size_t)4 * ATT_TILE * HD * sizeof(KV) + (size_t)(G * ATT_TILE + 8) * sizeof(float);
  const size_t red = (size_t)(ATT_WARPS + 1) * G * HD * sizeof(float);
  const size_t smem = tile > red ? tile : red;
  auto k = attn_decode_kernel<KV, HD, G, FUSED>;
  if (int r = ensure_dynamic_smem(reinterpret_cast<const void *>(k), smem)) return r;
  IEB_LAUNCH_PDL("attn_decode_kernel", k, dim3(a.S, a.n_kv, T), dim3(ATT_THREADS), smem, st, a);
  return IE_B200_OK;
}

template <typename KV, int HD, bool FUSED>
static int dispatch_g(const AttnArgs &a, uint32_t G, uint32_t T, cudaStream_t st) {
  switch (G) {
    case 1: return launch_attn<KV, HD, 1, FUSED>(a, T, st);
    case 2: return launch_attn<KV, HD, 2, FUSED>(a, T, st);
    case 4: return launch_attn<KV, HD, 4, FUSED>(a, T, st);
    case 5: return launch_attn<KV, HD, 5, FUSED>(a, T, st);
    case 7: return launch_attn<KV, HD, 7, FUSED>(a, T, st);
    case 8: return launch_attn<KV, HD, 8, FUSED>(a, T, st);
    default: return fail(IE_B200_E_SIZE, "ie_b200_attn_decode: %u query heads per KV head unsupported (1, 2, 4, 5, 7, 8)", G);
  }
}

// Splits (grid.x): enough CTAs for about two per SM when every split is busy, spans of at least ATT_MIN_SPAN positions.
static uint32_t attn_splits(uint32_t n_kv, uint32_t n_ctx, uint32_t T) {
  const uint32_t by_len = (n_ctx + ATT_MIN_SPAN - 1u) / ATT_MIN_SPAN;
  uint32_t by_sm = (2u * (uint32_t)sm_count() + n_kv * T - 1u) / (n_kv * T);
  if (by_sm < 1u) by_sm = 1u;
  uint32_t S = by_len < by_sm ? by_len : by_sm;
  return S ? S : 1u;
}

template <bool FUSED>
static int dispatch_attn(const AttnArgs &a, uint32_t hd, int kv_f32, uint32_t T, cudaStream_t st) {
  const uint32_t G = a.n_head / a.n_kv;
  if (kv_f32) {
    switch (hd) {
      case 32: return dispatch_g<float, 32, FUSED>(a, G, T, st);
      case 64: return dispatch_g<float, 64, FUSED>(a, G, T, st);
      case 128: return dispatch_g<float, 128, FUSED>(a, G, T, st);
    }
  } else {
    switch (hd) {
      case 32: return dispatch_g<__half, 32, FUSED>(a, G, T, st);
      case 64: return dispatch_g<__half, 64, FUSED>(a, G, T, st);
      case 128: return dispatch_g<__half, 128, FUSED>(a, G, T, st);
    }
  }
  return fail(IE_B200_E_SIZE, "ie_b200_attn_decode: head dim %u unsupported (32, 64, 128)", hd);
}

}  // namespace ieb

using namespace ieb;

extern "C" size_t ie_b200_attn_part_bytes(uint32_t n_head, uint32_t hd, uint32_t n_ctx, uint32_t T) {
  // an upper bound over every KV-head count: splits never exceed ceil(n_ctx / 256)
  const size_t S = (n_ctx + ATT_MIN_SPAN - 1u) / ATT_MIN_SPAN;
  return (size_t)T * n_head * (S ? S : 1u) * (hd + 2u) * sizeof(float);
}
extern "C" size_t ie_b200_attn_count_words(uint32_t n_head, uint32_t T) { return (size_t)n_head * T; }

extern "C" int ie_b200_attn_decode(const float *d_q, const void *d_kc, const void *d_vc, float *d_out, void *d_oq, const uint32_t *d_pos,
                                   uint32_t n_head, uint32_t n_kv, uint32_t hd, int kv_f32, uint32_t kv_len, uint32_t n_ctx, uint32_t T,
                                   size_t q_stride, size_t out_stride, size_t oq_stride, void *d_part, uint32_t *d_count, void *stream) {
  if (!d_q || !d_kc || !d_vc || !d_out || !d_pos || !d_part || !d_count) return fail(IE_B200_E_ARG, "ie_b200_attn_decode: NULL pointer");
  if (n_kv == 0 || n_head % n_kv) return fail(IE_B200_E_SIZE, "ie_b200_attn_decode: %u heads over %u KV heads", n_head, n_kv);
  if (kv_len < n_ctx) return fail(IE_B200_E_SIZE, "ie_b200_attn_decode: cache rows %u < context %u (ring caches unsupported)", kv_len, n_ctx);
  if (!aligned16(d_kc) || !aligned16(d_vc) || !aligned16(d_q) || (q_stride & 15u))
    return fail(IE_B200_E_ARG, "ie_b200_attn_decode: q and the caches must be 16-byte aligned");
  if (T == 0) return IE_B200_OK;
  if (T > 65535u) return fail(IE_B200_E_SIZE, "ie_b200_attn_decode: T %u > 65535", T);
  AttnArgs a;
  a.q = d_q, a.kc = d_kc, a.vc = d_vc, a.out = d_out, a.oq = static_cast<uint8_t *>(d_oq), a.pos = d_pos;
  a.n_head = n_head, a.n_kv = n_kv, a.kv_len = kv_len, a.S = attn_splits(n_kv, n_ctx, T);
  a.q_stride = q_stride, a.out_stride = out_stride, a.oq_stride = oq_stride;
  a.part = static_cast<float *>(d_part), a.count = d_count;
  a.scale = 1.0f / sqrtf((float)hd);
  a.k_new = a.v_new = a.cs = a.sn = nullptr, a.neox = 0;
  return dispatch_attn<false>(a, hd, kv_f32, T, static_cast<cudaStream_t>(stream));
}

extern "C" int ie_b200_attn_decode_fused(const float *d_q, const float *d_k, const float *d_v, void *d_kc, void *d_vc, const float *d_cos,
                                         const float *d_sin, float *d_out, void *d_oq, const uint32_t *d_pos, uint32_t n_head, uint32_t n_kv,
                                         uint32_t hd, int neox, int kv_f32, uint32_t kv_len, uint32_t n_ctx, void *d_part, uint32_t *d_count,
                                         void *stream) {
  if (!d_q || !d_k || !d_v || !d_kc || !d_vc || !d_cos || !d_sin || !d_out || !d_pos || !d_part || !d_count)
    return fail(IE_B200_E_ARG, "ie_b200_attn_decode_fused: NULL pointer");
  if (n_kv == 0 || n_head % n_kv) return fail(IE_B200_E_SIZE, "ie_b200_attn_decode_fused: %u heads over %u KV heads", n_head, n_kv);
  if (kv_len < n_ctx) return fail(IE_B200_E_SIZE, "ie_b200_attn_decode_fused: cache rows %u < context %u (ring caches unsupported)", kv_len, n_ctx);
  if (!aligned16(d_kc) || !aligned16(d_vc) || !aligned16(d_q)) return fail(IE_B200_E_ARG, "ie_b200_attn_decode_fused: q and the caches must be 16-byte aligned");
  AttnArgs a;
  a.q = d_q, a.kc = d_kc, a.vc = d_vc, a.out = d_out, a.oq = static_cast<uint8_t *>(d_oq), a.pos = d_pos;
  a.n_head = n_head, a.n_kv = n_kv, a.kv_len = kv_len, a.S = attn_splits(n_kv, n_ctx, 1);
  a.q_stride = a.out_stride = a.oq_stride = 0;
  a.part = static_cast<float *>(d_part), a.count = d_count;
  a.scale = 1.0f / sqrtf((float)hd);
  a.k_new = d_k, a.v_new = d_v, a.cs = d_cos, a.sn = d_sin, a.neox = neox;
  return dispatch_attn<true>(a, hd, kv_f32, 1, static_cast<cudaStream_t>(stream));
}
