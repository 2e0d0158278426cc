// attn_decode.cu -- attention over the KV cache, the K / V of a KV head read once for all of its G query heads
// (grouped-query attention). Three kernels share the geometry:
//   attn_decode_kernel       one token per CTA set, CUDA cores (float or half cache, any supported head size)
//   attn_decode_mma_kernel   the same on tensor cores for the half cache (hd 64 / 128): the decode default
//   attn_prefill_mma_kernel  prompt chunks: 16 / G tokens of a KV head share one pass over the cache
//
// Decode grid: (split s, KV head g, token t). The positions 0 .. np-1 of token t (np = first position + t + 1) are
// cut into up to S spans, multiples of the tile (64 positions), at least ATT_MIN_SPAN long. A CTA streams its span
// tile by tile: K and V tiles (contiguous in the head-major cache [kv head][row][hd]) arrive in shared memory
// through 16-byte async copies, two or three tiles ahead; every warp owns some positions of each tile and keeps its
// own running max / sum / output (online softmax), merged across the warps at the end. With one split the CTA
// writes the result itself; otherwise it writes (max, sum, out[hd]) per head to the partials buffer and the last
// CTA of a (token, KV head) to arrive merges the partials in split order, divides, and writes the f32 output and
// its Q8 copy. The one-token form can also rotate q, rotate and store the step's own K / V row (FUSED).
// Bound by HBM at long context: 2 * np * hd * sizeof(KV) bytes per KV head; by latency at short.
#include <cuda_pipeline_primitives.h>

#include <cstdlib>

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
  // Set when the kernel before this one in the stream lets its dependents go only after its own dependency wait:
  // when this kernel starts, everything older than that kernel is complete, so the position scalar and the cache
  // rows of earlier steps may be read ahead of this kernel's own wait.
  int early_kv;
};

constexpr uint32_t ATT_MIN_SPAN = 256;  // about the positions of a split; up to twice as many stay in one CTA per KV head (no merge)

// The span of one split for np positions over at most S splits: as many splits as spans of ATT_MIN_SPAN positions fit
// (at least one), and the positions dealt evenly over them (in whole tiles), so that no split is left with a sliver
// while another holds a full span (300 positions: 192 + 108 rather than 256 + 44).
__device__ __forceinline__ uint32_t att_span(uint32_t np, uint32_t S) {
  uint32_t want = np <= 2u * ATT_MIN_SPAN ? 1u : (np + ATT_MIN_SPAN - 1u) / ATT_MIN_SPAN;  // one CTA up to 512 positions: a merge costs more than four tiles
  want = want < 1u ? 1u : (want > S ? S : want);
  const uint32_t span = (np + want - 1u) / want;
  return (span + ATT_TILE - 1u) / ATT_TILE * ATT_TILE;
}

// a * c - b * s and a * s + b * c with every product rounded, as the RoPE kernel and the CPU do
__device__ __forceinline__ float rope_lo(float a, float b, float c, float s) { return __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)); }
__device__ __forceinline__ float rope_hi(float a, float b, float c, float s) { return __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c)); }

// The last split to arrive merges the A partial records (max, sum, out[hd]) of every head of its KV head, in split
// order. The weights exp(max_k - max) and the denominators are worked out once in shared memory (a warp per head); the outputs are
// then summed with many independent loads in flight per thread (a plain loop over the splits is one L2 round trip
// per split and per pass: 16 us at 17 splits).
// part: the records of this token's first head of the KV head, [G][S][hd + 2]; scr: (2 A + 2) G floats of shared memory.
// A split's record of one head in global memory: out[hd], then (max, sum) and two floats of padding, so that records start
// on 16-byte boundaries and the merge reads them four floats per load.
template <int HD>
struct AttRec {
  static constexpr int FLOATS = HD + 4;
};

template <int G, int HD, int THREADS>
__device__ __forceinline__ void merge_partials(const float *part, uint32_t S, uint32_t A, float *fin, float *scr) {
  constexpr size_t rec = AttRec<HD>::FLOATS;
  float *mk = scr, *lk = scr + G * A, *mh = lk + G * A, *lh = mh + G;
  for (uint32_t i = threadIdx.x; i < G * A; i += THREADS) {
    const float2 ml2 = __ldcg(reinterpret_cast<const float2 *>(part + ((size_t)(i / A) * S + i % A) * rec + HD));
    mk[i] = ml2.x, lk[i] = ml2.y;
  }
  __syncthreads();
  // one warp per head: its lanes share the splits (maximum, weights exp(max_k - max), denominator), no block-wide steps
  for (int h = threadIdx.x >> 5; h < G; h += THREADS / 32) {
    const int lane = threadIdx.x & 31;
    float M = -INFINITY;
    for (uint32_t k = lane; k < A; k += 32u) M = fmaxf(M, mk[h * A + k]);
    M = warp_max(M);
    float L = 0.0f;
    for (uint32_t k = lane; k < A; k += 32u) {
      const float w = expf(mk[h * A + k] - M);
      mk[h * A + k] = w;  // now the weight of split k
      L = fmaf(w, lk[h * A + k], L);
    }
    L = warp_sum_all(L);
    if (lane == 0) mh[h] = M, lh[h] = L;
  }
  __syncthreads();
  // a thread owns groups of four consecutive output elements; four splits at a time: (groups x 4) independent 16-byte
  // loads per round trip. The sum over the splits runs in split order for every element, as one element at a time would.
  constexpr int QUADS = G * HD / 4, QPT = (QUADS + THREADS - 1) / THREADS;
  float4 acc[QPT];
#pragma unroll
  for (int i = 0; i < QPT; i++) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (uint32_t k0 = 0; k0 < A; k0 += 4u) {
    float4 v[QPT][4];
#pragma unroll
    for (int i = 0; i < QPT; i++) {
      const int q = threadIdx.x + THREADS * i, e = 4 * q;
      const float *pr = part + (size_t)(e / HD) * S * rec + (e % HD);
#pragma unroll
      for (int j = 0; j < 4; j++)
        v[i][j] = (q < QUADS && k0 + j < A) ? __ldcg(reinterpret_cast<const float4 *>(pr + (size_t)(k0 + j) * rec)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < QPT; i++) {
      const int q = threadIdx.x + THREADS * i, e = 4 * q;
      if (q < QUADS) {
        const float *w = mk + (e / HD) * A;
#pragma unroll
        for (int j = 0; j < 4; j++)
          if (k0 + j < A) {
            acc[i].x = fmaf(w[k0 + j], v[i][j].x, acc[i].x), acc[i].y = fmaf(w[k0 + j], v[i][j].y, acc[i].y);
            acc[i].z = fmaf(w[k0 + j], v[i][j].z, acc[i].z), acc[i].w = fmaf(w[k0 + j], v[i][j].w, acc[i].w);
          }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < QPT; i++) {
    const int q = threadIdx.x + THREADS * i, e = 4 * q;
    if (q < QUADS) {
      const float inv = 1.0f / lh[e / HD];
      fin[e] = acc[i].x * inv, fin[e + 1] = acc[i].y * inv, fin[e + 2] = acc[i].z * inv, fin[e + 3] = acc[i].w * inv;
    }
  }
}

template <typename KV, int HD>
struct AttGeom {
  static constexpr int TILE_BYTES = 2 * ATT_TILE * HD * (int)sizeof(KV);  // one K tile + one V tile
  static constexpr int NB_FIT = 200 * 1024 / TILE_BYTES;
  static constexpr int NB = NB_FIT > 4 ? 4 : (NB_FIT < 2 ? 2 : NB_FIT);  // tile buffers: NB - 1 tiles in flight ahead of the one in use
};

// HS: the G query heads of the KV head are dealt to HS groups of eight warps (G / HS heads each) that share the K / V
// tiles: twice the warps halve the arithmetic per warp, which is what a short context waits for.
template <typename KV, int HD, int G, bool FUSED, int HS>
__global__ void __launch_bounds__(ATT_THREADS * HS) attn_decode_kernel(const AttnArgs a) {
  constexpr int GH = G / HS, THREADS = ATT_THREADS * HS;
  static_assert(G % HS == 0, "heads split evenly over the warp groups");
  constexpr int DPL = HD / 8;   // dims per lane in the q.k phase (8 lanes per position)
  constexpr int DPV = HD / 32;  // dims per lane in the p.v phase
  constexpr int TILE = ATT_TILE, TILE_ELEMS = TILE * HD, NB = AttGeom<KV, HD>::NB;
  constexpr int PPW = TILE / ATT_WARPS;  // positions of a tile per warp
  static_assert(PPW % 4 == 0, "a warp scores four positions at a time");
  extern __shared__ uint4 smem_raw[];
  KV *kbuf = reinterpret_cast<KV *>(smem_raw);                          // [NB][TILE][HD]
  KV *vbuf = kbuf + NB * TILE_ELEMS;                                     // [NB][TILE][HD]
  float *Pw = reinterpret_cast<float *>(vbuf + NB * TILE_ELEMS);         // [warp][PPW][GH] probabilities of the warp's positions
  __shared__ uint32_t is_last;

  pdl_launch_dependents();
  const bool early = FUSED && a.early_kv;
  if (!early) pdl_wait();
  const uint32_t s = blockIdx.x, g = blockIdx.y, t = blockIdx.z, S = a.S;
  const uint32_t np = *a.pos + t + 1u;
  const uint32_t span = att_span(np, S);
  const uint32_t A = (np + span - 1u) / span;  // splits that hold positions; the others have nothing to do
  if (s >= A) return;
  const uint32_t p_lo = s * span, p_hi = min(np, p_lo + span);
  const bool owns_new = FUSED && s == A - 1u;  // this CTA's span ends with the step's own position
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wq = warp % ATT_WARPS, hg = warp / ATT_WARPS;  // which positions of a tile, which heads
  const int sub = lane & 7, grp = lane >> 3;
  const float *qt = reinterpret_cast<const float *>(reinterpret_cast<const char *>(a.q) + a.q_stride * t) + (size_t)g * G * HD;
  const KV *kh = static_cast<const KV *>(a.kc) + (size_t)g * a.kv_len * HD, *vh = static_cast<const KV *>(a.vc) + (size_t)g * a.kv_len * HD;
  const uint32_t n_tiles = (p_hi - p_lo + TILE - 1u) / TILE;

  // Tile `it` of the span into buffer it % NB: only rows that exist in the cache are copied (the step's own row
  // arrives from registers, rows past the span are never read).
  constexpr int PER_ROW = HD * (int)sizeof(KV) / 16;  // 16-byte pieces per row
  auto issue = [&](uint32_t it) {
    if (it < n_tiles) {
      const uint32_t tile_lo = p_lo + it * TILE;
      const uint32_t rows = min((uint32_t)TILE, p_hi - tile_lo - ((owns_new && it + 1u == n_tiles) ? 1u : 0u));
      const char *ks = reinterpret_cast<const char *>(kh + (size_t)tile_lo * HD), *vs = reinterpret_cast<const char *>(vh + (size_t)tile_lo * HD);
      char *kd = reinterpret_cast<char *>(kbuf + (it % NB) * TILE_ELEMS), *vd = reinterpret_cast<char *>(vbuf + (it % NB) * TILE_ELEMS);
      for (uint32_t c = threadIdx.x; c < rows * PER_ROW; c += THREADS) {
        __pipeline_memcpy_async(kd + (size_t)c * 16u, ks + (size_t)c * 16u, 16);
        __pipeline_memcpy_async(vd + (size_t)c * 16u, vs + (size_t)c * 16u, 16);
      }
    }
    __pipeline_commit();
  };
#pragma unroll
  for (int i = 0; i < NB - 1; i++) issue(i);
  // RoPE table values of this lane's q dims (pairs (2i, 2i+1): DPL / 2 of them; pairs (i, i + hd/2): DPL) and of the
  // k pair this thread rotates: constants, fetched ahead of the dependency wait when the position is known by then
  float tc[DPL], ts[DPL], kc_ = 0.f, ks_ = 0.f;
  auto load_tables = [&]() {
    if (!FUSED) return;
    const float *cs = a.cs + (size_t)(np - 1u) * (HD / 2), *sn = a.sn + (size_t)(np - 1u) * (HD / 2);
    const int nt = a.neox ? DPL : DPL / 2, i0 = a.neox ? (sub * DPL) % (HD / 2) : sub * (DPL / 2);
#pragma unroll
    for (int j = 0; j < DPL; j += 2) {
      if (j < nt) {
        const float2 c2 = *reinterpret_cast<const float2 *>(cs + i0 + j), s2 = *reinterpret_cast<const float2 *>(sn + i0 + j);
        tc[j] = c2.x, tc[j + 1] = c2.y, ts[j] = s2.x, ts[j + 1] = s2.y;
      }
    }
    if (owns_new && threadIdx.x < HD / 2) kc_ = cs[threadIdx.x], ks_ = sn[threadIdx.x];
  };
  if (early) load_tables();
  if (early) pdl_wait();

  // ---- q of this lane for the q.k phase (rotated here when fused), the step's own K / V row
  float qr[GH][DPL];
#pragma unroll
  for (int h = 0; h < GH; h++)
#pragma unroll
    for (int j = 0; j < DPL; j += 4) {
      const float4 v = *reinterpret_cast<const float4 *>(qt + (hg * GH + h) * HD + sub * DPL + j);
      qr[h][j] = v.x, qr[h][j + 1] = v.y, qr[h][j + 2] = v.z, qr[h][j + 3] = v.w;
    }
  KV newk0 = KV(0.f), newk1 = KV(0.f), newv = KV(0.f);
  int nk0 = 0, nk1 = 0;
  if (FUSED) {
    float x0 = 0.f, x1 = 0.f, vn = 0.f;
    if (owns_new) {  // the loads of the new row go out together with the q loads above
      if (threadIdx.x < HD / 2) {
        const int i = threadIdx.x;
        nk0 = a.neox ? i : 2 * i, nk1 = a.neox ? i + HD / 2 : 2 * i + 1;
        x0 = a.k_new[g * HD + nk0], x1 = a.k_new[g * HD + nk1];
      } else if (threadIdx.x >= 128 && threadIdx.x < 128 + HD) {
        vn = a.v_new[g * HD + (threadIdx.x - 128)];
      }
    }
    if (!early) load_tables();
    if (!a.neox) {  // pairs (2i, 2i+1): both in this lane
#pragma unroll
      for (int j = 0; j < DPL; j += 2)
#pragma unroll
        for (int h = 0; h < GH; h++) {
          const float y0 = qr[h][j], y1 = qr[h][j + 1];
          qr[h][j] = rope_lo(y0, y1, tc[j / 2], ts[j / 2]), qr[h][j + 1] = rope_hi(y0, y1, tc[j / 2], ts[j / 2]);
        }
    } else {  // pairs (i, i + hd/2): the partner dim sits in the lane 4 further in the 8-lane group
#pragma unroll
      for (int j = 0; j < DPL; j++)
#pragma unroll
        for (int h = 0; h < GH; h++) {
          const float mine = qr[h][j], other = __shfl_xor_sync(0xFFFFFFFFu, mine, 4);
          qr[h][j] = sub < 4 ? rope_lo(mine, other, tc[j], ts[j]) : rope_hi(other, mine, tc[j], ts[j]);
        }
    }
    if (owns_new) {  // rotate k, store the row in the cache; it joins the last tile from registers below
      const uint32_t row = (np - 1u) % a.kv_len;
      if (threadIdx.x < HD / 2) {
        newk0 = KV(rope_lo(x0, x1, kc_, ks_)), newk1 = KV(rope_hi(x0, x1, kc_, ks_));
        KV *dst = const_cast<KV *>(kh) + (size_t)row * HD;
        dst[nk0] = newk0, dst[nk1] = newk1;
      } else if (threadIdx.x >= 128 && threadIdx.x < 128 + HD) {
        newv = KV(vn);
        const_cast<KV *>(vh)[(size_t)row * HD + (threadIdx.x - 128)] = newv;
      }
    }
  }

  // ---- the span, tile by tile. Every warp keeps its own running max / sum / output over the positions it owns
  // (PPW per tile), so the only block-wide synchronisation is the hand-over of tile buffers.
  float o[GH][DPV], run_m[GH], run_l[GH];
#pragma unroll
  for (int h = 0; h < GH; h++) {
    run_m[h] = -INFINITY, run_l[h] = 0.0f;
#pragma unroll
    for (int d = 0; d < DPV; d++) o[h][d] = 0.0f;
  }
  float *pw = Pw + warp * PPW * GH;
  for (uint32_t it = 0; it < n_tiles; it++) {
    const int buf = it % NB;
    const uint32_t tile_lo = p_lo + it * TILE;
    if (owns_new && it + 1u == n_tiles) {  // nobody else writes this row of the buffer
      const uint32_t pr = np - 1u - tile_lo;
      if (threadIdx.x < HD / 2) {
        KV *dk = kbuf + buf * TILE_ELEMS + pr * HD;
        dk[nk0] = newk0, dk[nk1] = newk1;
      } else if (threadIdx.x >= 128 && threadIdx.x < 128 + HD) {
        vbuf[buf * TILE_ELEMS + pr * HD + (threadIdx.x - 128)] = newv;
      }
    }
    __pipeline_wait_prior(NB - 2);
    __syncthreads();          // tile `it` is complete; everybody is done with tile it - 1, whose buffer is refilled now
    issue(it + NB - 1u);
    const uint32_t valid = p_hi - tile_lo;  // positions of this tile that exist (>= 1)
    if ((uint32_t)(wq * PPW) < valid) {
      const KV *kt = kbuf + buf * TILE_ELEMS, *vt = vbuf + buf * TILE_ELEMS;
      // scores: 8 lanes per position, 4 positions per round
      float sc[PPW / 4][GH];
#pragma unroll
      for (int r = 0; r < PPW / 4; r++) {
        const int pi = wq * PPW + r * 4 + grp;
        float kr[DPL];
        load_slice<KV>(kt + pi * HD + sub * DPL, kr, DPL);
#pragma unroll
        for (int h = 0; h < GH; h++) {
          float d = 0.0f;
#pragma unroll
          for (int j = 0; j < DPL; j++) d = fmaf(qr[h][j], kr[j], d);
          d += __shfl_xor_sync(0xFFFFFFFFu, d, 1);
          d += __shfl_xor_sync(0xFFFFFFFFu, d, 2);
          d += __shfl_xor_sync(0xFFFFFFFFu, d, 4);
          sc[r][h] = (uint32_t)pi < valid ? d * a.scale : -INFINITY;
        }
      }
      // the warp's running softmax; position warp * PPW exists, so the new maximum is finite
#pragma unroll
      for (int h = 0; h < GH; h++) {
        float mx = sc[0][h];
#pragma unroll
        for (int r = 1; r < PPW / 4; r++) mx = fmaxf(mx, sc[r][h]);
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 16));
        const float m_new = fmaxf(run_m[h], mx), al = expf(run_m[h] - m_new);
        float sum = 0.0f;
#pragma unroll
        for (int r = 0; r < PPW / 4; r++) {
          const float pv = expf(sc[r][h] - m_new);
          sum += pv;
          if (sub == 0) pw[(r * 4 + grp) * GH + h] = pv;
        }
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 8);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 16);
        run_l[h] = run_l[h] * al + sum, run_m[h] = m_new;
#pragma unroll
        for (int d = 0; d < DPV; d++) o[h][d] *= al;
      }
      __syncwarp();
      // p.v over the warp's positions: every lane owns DPV output dims
#pragma unroll
      for (int j = 0; j < PPW; j++) {
        if ((uint32_t)(wq * PPW + j) < valid) {  // uniform over the warp
          float vr[DPV];
          if (DPV >= 4) {
            load_slice<KV>(vt + (wq * PPW + j) * HD + lane * DPV, vr, DPV);
          } else {
#pragma unroll
            for (int d = 0; d < DPV; d++) vr[d] = (float)vt[(wq * PPW + j) * HD + lane * DPV + d];
          }
#pragma unroll
          for (int h = 0; h < GH; h++) {
            const float pv = pw[j * GH + h];
#pragma unroll
            for (int d = 0; d < DPV; d++) o[h][d] = fmaf(pv, vr[d], o[h][d]);
          }
        }
      }
      __syncwarp();
    }
  }
  __pipeline_wait_prior(0);
  __syncthreads();

  // ---- merge the warps' (max, sum, output) in shared memory, reusing the tile buffers
  float *red = reinterpret_cast<float *>(smem_raw);   // [ATT_WARPS][G][HD]
  float *ml = red + ATT_WARPS * G * HD;               // [ATT_WARPS][G][2]
  float *fin = ml + ATT_WARPS * G * 2;                // [G][HD]
#pragma unroll
  for (int h = 0; h < GH; h++) {
    const int hh = hg * GH + h;  // the head's index within the KV head
#pragma unroll
    for (int d = 0; d < DPV; d++) red[(wq * G + hh) * HD + lane * DPV + d] = o[h][d];
    if (lane == 0) ml[(wq * G + hh) * 2] = run_m[h], ml[(wq * G + hh) * 2 + 1] = run_l[h];
  }
  __syncthreads();
  // final values of this KV head's G heads: directly when one split held everything, else through the partials
  // buffer, merged by the last split to arrive
  const size_t rec = HD + 2;
  constexpr size_t grec = AttRec<HD>::FLOATS;  // the record in global memory
  for (int e = threadIdx.x; e < G * HD; e += THREADS) {
    const int h = e / HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; w++) M = fmaxf(M, ml[(w * G + h) * 2]);
    float L = 0.0f, acc = 0.0f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; w++) {
      const float wk = expf(ml[(w * G + h) * 2] - M);  // a warp without positions has max -inf: weight 0
      L = fmaf(wk, ml[(w * G + h) * 2 + 1], L);
      acc = fmaf(wk, red[(w * G + h) * HD + (e % HD)], acc);
    }
    if (A == 1u) {
      fin[e] = acc * (1.0f / L);
    } else {
      float *pr = a.part + (((size_t)t * a.n_head + (size_t)g * G + h) * S + s) * grec;
      pr[e % HD] = acc;
      if (e % HD == 0) pr[HD] = M, pr[HD + 1] = L;
    }
  }
  if (A > 1u) {
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
    merge_partials<G, HD, THREADS>(a.part + ((size_t)t * a.n_head + (size_t)g * G) * S * grec, S, A, fin, fin + G * HD);
  }
  __syncthreads();
  // ---- write out, one warp per block of 32 values (which is also a Q8 block of the output vector)
  float *ot = reinterpret_cast<float *>(reinterpret_cast<char *>(a.out) + a.out_stride * t) + (size_t)g * G * HD;
  uint8_t *oqt = a.oq ? a.oq + a.oq_stride * t : nullptr;
  const uint32_t nbq = a.n_head * HD / 32u;
  for (int b = warp; b < G * HD / 32; b += ATT_WARPS * HS) {
    const float v = fin[32 * b + lane];
    ot[32 * b + lane] = v;
    if (oqt) quant_block_warp(v, oqt, nbq, g * (G * HD / 32u) + b, lane);
  }
}

template <typename KV, int HD, int G, bool FUSED>
static int launch_attn(const AttnArgs &a, uint32_t T, cudaStream_t st) {
  constexpr int HS = (G % 2 == 0) ? 2 : 1;
  const size_t tile = (size_t)AttGeom<KV, HD>::NB * AttGeom<KV, HD>::TILE_BYTES + (size_t)ATT_WARPS * (ATT_TILE / ATT_WARPS) * G * sizeof(float);
  const size_t red = (size_t)((ATT_WARPS + 1) * G * HD + ATT_WARPS * G * 2 + (2 * a.S + 2) * G) * sizeof(float);
  const size_t smem = tile > red ? tile : red;
  auto k = attn_decode_kernel<KV, HD, G, FUSED, HS>;
  if (int r = ensure_dynamic_smem(reinterpret_cast<const void *>(k), smem)) return r;
  IEB_LAUNCH_PDL("attn_decode_kernel", k, dim3(a.S, a.n_kv, T), dim3(ATT_THREADS * HS), smem, st, a);
  return IE_B200_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// The half-precision-cache form on tensor cores (mma.sync m16n8k16, f16 x f16 -> f32): the scalar kernel above is
// bound by instruction issue (about 8000 warp instructions per 64-position tile, 830 GB/s at 4096 positions); here
// a tile is 4 warps x (32 MMAs + 16 ldmatrix), so the kernel waits on HBM only. The cache's f16 K / V rows are the
// exact operands; the fp32 sides are split into two f16 terms so that nothing is rounded away: q = q_hi + q_lo
// for S = q . k (two MMAs per step), p = p_hi + p_lo for O = p . v. Layout of the decode kernel: the cache rows take
// the 16-row side of the MMA, the group's (at most 8) heads the 8-column side, S[16 positions x heads] = K . Q^T and
// O^T[16 dims x heads] += V^T . P^T, the C fragment of S turned into the B fragment of P^T by two 8 x 8 register
// transposes (movmatrix) per term. (The chunk kernel further down keeps queries on the row side: it has 16 rows of
// them.) Each warp owns 16 of the tile's 64 positions and keeps its own running max / sum / output; rows are
// padded to hd + 8 halves so that the 8 rows of an ldmatrix hit 8 different bank groups.
constexpr int AM_WARPS = 4, AM_THREADS = 128, AM_PAD = 8;
// NB tile buffers (NB - 1 tiles in flight ahead of the one in use): 4 with one CTA per SM while the splits leave SMs
// free anyway (short contexts: three of the first four tiles arrive during the kernel before this one), 3 with two
// CTAs per SM once there are more splits than SMs (long contexts).

__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void *p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
// An 8 x 8 block of 16-bit values held as one MMA fragment register per lane (row lane / 4, columns 2 (lane % 4), + 1), transposed.
__device__ __forceinline__ uint32_t movm_t(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], const void *p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// x = hi + lo with hi = f16(x), lo = f16(x - hi): two halves carry 22 bits of the float
__device__ __forceinline__ void split2(float x, float y, uint32_t &hi, uint32_t &lo) {
  const __half2 h = __floats2half2_rn(x, y);
  const float2 hf = __half22float2(h);
  const __half2 l = __floats2half2_rn(x - hf.x, y - hf.y);
  hi = *reinterpret_cast<const uint32_t *>(&h), lo = *reinterpret_cast<const uint32_t *>(&l);
}

// Shared memory of the cluster form behind the tile buffers / merge scratch: the records (max, sum, out[hd]) of the CL CTAs of a
// split, written into the leader's memory by every CTA of the cluster.
__host__ __device__ constexpr size_t am_main_bytes(int HD, int G, int NB, uint32_t S) {
  const size_t tile = (size_t)NB * 2 * ATT_TILE * (HD + AM_PAD) * sizeof(__half);
  const size_t red = (size_t)((AM_WARPS + 1) * G * HD + AM_WARPS * G * 2 + (2 * S + 2) * G) * sizeof(float);
  return ((tile > red ? tile : red) + 15u) & ~(size_t)15u;
}

// CL: CTAs per split. 1: a CTA streams its whole split. 4: a thread-block cluster shares the split, a CTA takes every
// CL-th part of its tiles, and the parts meet in the leader's shared memory (distributed shared memory, one cluster
// barrier): for short contexts, where one CTA per KV head leaves the fetch of the cache rows to a single SM.
template <int HD, int G, bool FUSED, int NB, int CL>
__global__ void __launch_bounds__(AM_THREADS, NB == 3 ? 2 : 1) attn_decode_mma_kernel(const AttnArgs a) {
  constexpr int TILE = ATT_TILE, ROW = HD + AM_PAD, TILE_ELEMS = TILE * ROW, KS = HD / 16;
  static_assert(G <= 8, "the heads of a KV head fill the 8 columns of the MMA");
  extern __shared__ uint4 smem_raw[];
  __half *kbuf = reinterpret_cast<__half *>(smem_raw);  // [NB][TILE][ROW]
  __half *vbuf = kbuf + NB * TILE_ELEMS;                // [NB][TILE][ROW]
  __shared__ uint32_t is_last;

  pdl_launch_dependents();
  const bool early = FUSED && a.early_kv;
  if (!early) pdl_wait();
  const uint32_t s = blockIdx.x / CL, cr = blockIdx.x % CL, g = blockIdx.y, t = blockIdx.z, S = a.S;
  const uint32_t np = *a.pos + t + 1u;
  const uint32_t span = att_span(np, S);
  const uint32_t A = (np + span - 1u) / span;
  if (s >= A) return;  // (the whole cluster of such a split returns here)
  if (CL > 1) cluster_arrive();
  uint32_t p_lo = s * span, p_hi = min(np, p_lo + span);
  if (CL > 1) {  // this CTA's tiles of the split: ceil(tiles / CL) consecutive ones; the last CTAs may hold none
    const uint32_t tiles = (p_hi - p_lo + TILE - 1u) / TILE, per = (tiles + CL - 1u) / CL;
    const uint32_t lo2 = min(p_hi, p_lo + cr * per * TILE);
    p_hi = min(p_hi, lo2 + per * TILE), p_lo = lo2;
  }
  const bool owns_new = FUSED && s == A - 1u && p_lo < np && np <= p_hi;  // the CTA whose positions end with this step's own
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, hq = lane >> 2, tq = lane & 3;  // hq: the fragment row (a position, a dim) and the head whose q this lane holds; tq: the column pair (heads 2tq, + 1)
  const float *qt = reinterpret_cast<const float *>(reinterpret_cast<const char *>(a.q) + a.q_stride * t) + (size_t)g * G * HD;
  const __half *kh = static_cast<const __half *>(a.kc) + (size_t)g * a.kv_len * HD, *vh = static_cast<const __half *>(a.vc) + (size_t)g * a.kv_len * HD;
  const uint32_t n_tiles = (p_hi - p_lo + TILE - 1u) / TILE;

  // tile `it` into buffer it % NB: cache rows by 16-byte async copies, rows past the span zero-filled (a zero
  // probability times an uninitialised value must stay zero), the step's own row left to the registers below
  constexpr int PER_ROW = HD * 2 / 16, RPP = AM_THREADS / PER_ROW;  // 16-byte pieces per row; rows covered by one pass of the CTA
  const uint32_t my_piece = (threadIdx.x % PER_ROW) * 16u, my_row = threadIdx.x / PER_ROW;
  auto issue = [&](uint32_t it) {
    if (it < n_tiles) {
      const uint32_t tile_lo = p_lo + it * TILE;
      const uint32_t have = p_hi - tile_lo;
      const bool with_new = owns_new && it + 1u == n_tiles;
      const uint32_t rows = min((uint32_t)TILE, have - (with_new ? 1u : 0u));
      const char *ks = reinterpret_cast<const char *>(kh + (size_t)tile_lo * HD) + my_piece, *vs = reinterpret_cast<const char *>(vh + (size_t)tile_lo * HD) + my_piece;
      char *kd = reinterpret_cast<char *>(kbuf + (it % NB) * TILE_ELEMS) + my_piece, *vd = reinterpret_cast<char *>(vbuf + (it % NB) * TILE_ELEMS) + my_piece;
#pragma unroll
      for (int j = 0; j < TILE / RPP; j++) {
        const uint32_t r = my_row + RPP * j;
        if (with_new && r == have - 1u) continue;  // the new row comes from registers
        const bool ok = r < rows;
        const size_t src = ok ? (size_t)r * HD * 2u : 0u;
        __pipeline_memcpy_async(kd + (size_t)r * ROW * 2u, ks + src, 16, ok ? 0 : 16);
        __pipeline_memcpy_async(vd + (size_t)r * ROW * 2u, vs + src, 16, ok ? 0 : 16);
      }
    }
    __pipeline_commit();
  };
#pragma unroll
  for (int i = 0; i < NB - 1; i++) issue(i);

  // RoPE table values for this lane's q dims: it holds, for every 16-dim step ks, dims 16 ks + {2tq, 2tq+1, 2tq+8, 2tq+9}.
  // Pairs (2i, 2i+1) sit side by side; pairs (i, i + hd/2) are steps ks and ks + KS/2 of the same lane.
  float tc[KS][2], ts[KS][2], kc_ = 0.f, ks_ = 0.f;
  auto load_tables = [&]() {
    if (!FUSED) return;
    const float *cs = a.cs + (size_t)(np - 1u) * (HD / 2), *sn = a.sn + (size_t)(np - 1u) * (HD / 2);
    if (!a.neox) {  // (the other pairing reads its entries where it rotates)
#pragma unroll
      for (int k = 0; k < KS; k++)
#pragma unroll
        for (int e = 0; e < 2; e++) tc[k][e] = cs[8 * k + tq + 4 * e], ts[k][e] = sn[8 * k + tq + 4 * e];  // pair (16k + 2tq + 8e) / 2
    }
    if (owns_new && threadIdx.x < HD / 2) kc_ = cs[threadIdx.x], ks_ = sn[threadIdx.x];
  };
  if (early) load_tables();
  if (early) pdl_wait();

  // ---- q of head hq in fragment order (dims 16k + 2tq, + 1, + 8, + 9), rotated when fused, split into two f16 terms
  float qf[KS][4];
#pragma unroll
  for (int k = 0; k < KS; k++) {
    float2 lo2 = make_float2(0.f, 0.f), hi2 = lo2;
    if (hq < G) {
      lo2 = *reinterpret_cast<const float2 *>(qt + hq * HD + 16 * k + 2 * tq);
      hi2 = *reinterpret_cast<const float2 *>(qt + hq * HD + 16 * k + 2 * tq + 8);
    }
    qf[k][0] = lo2.x, qf[k][1] = lo2.y, qf[k][2] = hi2.x, qf[k][3] = hi2.y;
  }
  __half newk0 = __half(0.f), newk1 = __half(0.f), newv = __half(0.f);
  int nk0 = 0, nk1 = 0;
  if (FUSED) {
    float x0 = 0.f, x1 = 0.f, vn = 0.f;
    if (owns_new) {
      if (threadIdx.x < HD / 2) {
        const int i = threadIdx.x;
        nk0 = a.neox ? i : 2 * i, nk1 = a.neox ? i + HD / 2 : 2 * i + 1;
        x0 = a.k_new[g * HD + nk0], x1 = a.k_new[g * HD + nk1];
      }
      if (threadIdx.x < HD) vn = a.v_new[g * HD + threadIdx.x];
    }
    if (!early) load_tables();
    if (!a.neox) {
#pragma unroll
      for (int k = 0; k < KS; k++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
          const float y0 = qf[k][2 * e], y1 = qf[k][2 * e + 1];
          qf[k][2 * e] = rope_lo(y0, y1, tc[k][e], ts[k][e]), qf[k][2 * e + 1] = rope_hi(y0, y1, tc[k][e], ts[k][e]);
        }
    } else {
      const float *cs = a.cs + (size_t)(np - 1u) * (HD / 2), *sn = a.sn + (size_t)(np - 1u) * (HD / 2);
#pragma unroll
      for (int k = 0; k < KS / 2; k++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const int i = 16 * k + 2 * tq + (e & 1) + 8 * (e >> 1);  // dim i pairs with dim i + hd/2 (step k + KS/2, same slot)
          const float c = cs[i], sv = sn[i], y0 = qf[k][e], y1 = qf[k + KS / 2][e];
          qf[k][e] = rope_lo(y0, y1, c, sv), qf[k + KS / 2][e] = rope_hi(y0, y1, c, sv);
        }
    }
    if (owns_new) {
      const uint32_t row = (np - 1u) % a.kv_len;
      if (threadIdx.x < HD / 2) {
        newk0 = __half(rope_lo(x0, x1, kc_, ks_)), newk1 = __half(rope_hi(x0, x1, kc_, ks_));
        __half *dst = const_cast<__half *>(kh) + (size_t)row * HD;
        dst[nk0] = newk0, dst[nk1] = newk1;
      }
      if (threadIdx.x < HD) {
        newv = __half(vn);
        const_cast<__half *>(vh)[(size_t)row * HD + threadIdx.x] = newv;
      }
    }
  }
  uint32_t qh[KS][2], ql[KS][2];  // B fragment registers b0, b1 of Q^T[16 dims x heads]: column hq
#pragma unroll
  for (int k = 0; k < KS; k++) {
    split2(qf[k][0], qf[k][1], qh[k][0], ql[k][0]);
    split2(qf[k][2], qf[k][3], qh[k][1], ql[k][1]);
  }

  // Both products run with the cache rows on the 16-row side of the MMA and the (at most 8) heads on its 8-column side, so
  // that no half of a tile multiplies zero rows: S[16 positions x heads] = K . Q^T, then O^T[16 dims x heads] += V^T . P^T.
  // A lane holds, in every C fragment, heads 2tq and 2tq + 1: their running max and sum live in its registers.
  float o[HD / 16][4], run_m[2] = {-INFINITY, -INFINITY}, run_l[2] = {0.0f, 0.0f};  // o[u][j], o[u][2 + j]: head 2tq + j, dims 16u + hq, + 8
#pragma unroll
  for (int u = 0; u < HD / 16; u++)
#pragma unroll
    for (int e = 0; e < 4; e++) o[u][e] = 0.0f;
  const int lm = lane >> 3, lr = lane & 7;  // ldmatrix: this lane supplies row lr of matrix lm
  for (uint32_t it = 0; it < n_tiles; it++) {
    const int buf = it % NB;
    const uint32_t tile_lo = p_lo + it * TILE;
    if (owns_new && it + 1u == n_tiles) {  // nobody else writes this row of the buffer
      const uint32_t pr = np - 1u - tile_lo;
      if (threadIdx.x < HD / 2) {
        __half *dk = kbuf + buf * TILE_ELEMS + pr * ROW;
        dk[nk0] = newk0, dk[nk1] = newk1;
      }
      if (threadIdx.x < HD) vbuf[buf * TILE_ELEMS + pr * ROW + threadIdx.x] = newv;
    }
    __pipeline_wait_prior(NB - 2);
    __syncthreads();
    issue(it + NB - 1u);
    const uint32_t valid = p_hi - tile_lo;
    const int p0 = warp * 16;  // this warp's positions of the tile
    if ((uint32_t)p0 < valid) {
      const __half *kt = kbuf + buf * TILE_ELEMS, *vt = vbuf + buf * TILE_ELEMS;
      // ---- S[16 positions x heads]: sc[j] = position p0 + hq, sc[2 + j] = position p0 + hq + 8, of head 2tq + j
      float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int k = 0; k < KS; k++) {
        uint32_t ka[4];  // matrices: (positions lo, dims lo), (positions hi, dims lo), (positions lo, dims hi), (positions hi, dims hi)
        ldsm4(ka, kt + (p0 + (lm & 1) * 8 + lr) * ROW + 16 * k + (lm >> 1) * 8);
        mma_f16(sc, ka[0], ka[1], ka[2], ka[3], qh[k][0], qh[k][1]);
        mma_f16(sc, ka[0], ka[1], ka[2], ka[3], ql[k][0], ql[k][1]);
      }
      const bool ok0 = (uint32_t)(p0 + hq) < valid, ok1 = (uint32_t)(p0 + hq + 8) < valid;
      sc[0] = ok0 ? sc[0] * a.scale : -INFINITY, sc[1] = ok0 ? sc[1] * a.scale : -INFINITY;
      sc[2] = ok1 ? sc[2] * a.scale : -INFINITY, sc[3] = ok1 ? sc[3] * a.scale : -INFINITY;
      float al[2], pv[4];
#pragma unroll
      for (int j = 0; j < 2; j++) {  // a head's 16 positions sit in the 8 lanes of one tq
        float mx = fmaxf(sc[j], sc[2 + j]);
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 4));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 16));
        const float m_new = fmaxf(run_m[j], mx);  // position p0 exists: m_new is finite
        al[j] = expf(run_m[j] - m_new);
        pv[j] = expf(sc[j] - m_new), pv[2 + j] = expf(sc[2 + j] - m_new);
        float sum = pv[j] + pv[2 + j];
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 8);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 16);
        run_l[j] = run_l[j] * al[j] + sum, run_m[j] = m_new;
      }
      // P as two f16 terms, each 8 x 8 block [positions x heads] transposed into the B fragment [positions (k) x heads (n)]
      uint32_t ph[2], pl[2];
      split2(pv[0], pv[1], ph[0], pl[0]);
      split2(pv[2], pv[3], ph[1], pl[1]);
#pragma unroll
      for (int e = 0; e < 2; e++) ph[e] = movm_t(ph[e]), pl[e] = movm_t(pl[e]);
      // ---- O^T[hd x heads] = al * O^T + V^T . P^T, 16 dims per ldmatrix
#pragma unroll
      for (int u = 0; u < HD / 16; u++) {
        uint32_t va[4];  // transposed on load: (dims lo, positions lo), (dims hi, positions lo), (dims lo, positions hi), (dims hi, positions hi)
        ldsm4t(va, vt + (p0 + (lm >> 1) * 8 + lr) * ROW + 16 * u + (lm & 1) * 8);
        o[u][0] *= al[0], o[u][1] *= al[1], o[u][2] *= al[0], o[u][3] *= al[1];
        mma_f16(o[u], va[0], va[1], va[2], va[3], ph[0], ph[1]);
        mma_f16(o[u], va[0], va[1], va[2], va[3], pl[0], pl[1]);
      }
    }
  }
  __pipeline_wait_prior(0);
  __syncthreads();

  // ---- merge the warps' (max, sum, output) in shared memory, reusing the tile buffers
  float *red = reinterpret_cast<float *>(smem_raw);  // [AM_WARPS][G][HD]
  float *ml = red + AM_WARPS * G * HD;                // [AM_WARPS][G][2]
  float *fin = ml + AM_WARPS * G * 2;                 // [G][HD]
#pragma unroll
  for (int j = 0; j < 2; j++) {
    const int h = 2 * tq + j;
    if (h < G) {
#pragma unroll
      for (int u = 0; u < HD / 16; u++) red[(warp * G + h) * HD + 16 * u + hq] = o[u][j], red[(warp * G + h) * HD + 16 * u + hq + 8] = o[u][2 + j];
      if (hq == 0) ml[(warp * G + h) * 2] = run_m[j], ml[(warp * G + h) * 2 + 1] = run_l[j];
    }
  }
  __syncthreads();
  const size_t rec = HD + 2;
  constexpr size_t grec = AttRec<HD>::FLOATS;  // the record in global memory
  float *recv = reinterpret_cast<float *>(reinterpret_cast<char *>(smem_raw) + am_main_bytes(HD, G, NB, S));  // [CL][G][HD + 2], used in the leader
  if (CL > 1) {
    // every CTA's record into the leader's memory, then one cluster barrier; a CTA without positions sends (max -inf, sum 0)
    cluster_wait();  // (the leader runs: its memory may be written)
    const uint32_t base = cluster_map_shared(recv + (size_t)cr * G * rec, 0u);
    for (int e = threadIdx.x; e < G * HD; e += AM_THREADS) {
      const int h = e / HD;
      float M = -INFINITY, L = 0.0f, acc = 0.0f;
      if (p_lo < p_hi) {
#pragma unroll
        for (int w = 0; w < AM_WARPS; w++) M = fmaxf(M, ml[(w * G + h) * 2]);
#pragma unroll
        for (int w = 0; w < AM_WARPS; w++) {
          const float wk = expf(ml[(w * G + h) * 2] - M);
          L = fmaf(wk, ml[(w * G + h) * 2 + 1], L);
          acc = fmaf(wk, red[(w * G + h) * HD + (e % HD)], acc);
        }
      }
      cluster_st_f32(base + (uint32_t)((h * rec + 2 + (e % HD)) * sizeof(float)), acc);
      if (e % HD == 0) cluster_st_f32(base + (uint32_t)(h * rec * sizeof(float)), M), cluster_st_f32(base + (uint32_t)((h * rec + 1) * sizeof(float)), L);
    }
    cluster_sync_all();
    if (cr != 0u) return;
  }
  for (int e = threadIdx.x; e < G * HD; e += AM_THREADS) {
    const int h = e / HD;
    float M = -INFINITY;
    float L = 0.0f, acc = 0.0f;
    if (CL > 1) {  // the leader: the cluster's records in rank order (rank 0 always holds positions: M is finite)
#pragma unroll
      for (int c = 0; c < CL; c++) M = fmaxf(M, recv[(c * G + h) * rec]);
#pragma unroll
      for (int c = 0; c < CL; c++) {
        const float wk = expf(recv[(c * G + h) * rec] - M);
        L = fmaf(wk, recv[(c * G + h) * rec + 1], L);
        acc = fmaf(wk, recv[(c * G + h) * rec + 2 + (e % HD)], acc);
      }
    } else {
#pragma unroll
      for (int w = 0; w < AM_WARPS; w++) M = fmaxf(M, ml[(w * G + h) * 2]);
#pragma unroll
      for (int w = 0; w < AM_WARPS; w++) {
        const float wk = expf(ml[(w * G + h) * 2] - M);  // a warp without positions has max -inf: weight 0
        L = fmaf(wk, ml[(w * G + h) * 2 + 1], L);
        acc = fmaf(wk, red[(w * G + h) * HD + (e % HD)], acc);
      }
    }
    if (A == 1u) {
      fin[e] = acc * (1.0f / L);
    } else {
      float *pr = a.part + (((size_t)t * a.n_head + (size_t)g * G + h) * S + s) * grec;
      pr[e % HD] = acc;
      if (e % HD == 0) pr[HD] = M, pr[HD + 1] = L;
    }
  }
  if (A > 1u) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t prev = atomicAdd(&a.count[t * a.n_kv + g], 1u);
      is_last = prev == A - 1u;
      if (is_last) a.count[t * a.n_kv + g] = 0u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    merge_partials<G, HD, AM_THREADS>(a.part + ((size_t)t * a.n_head + (size_t)g * G) * S * grec, S, A, fin, fin + G * HD);
  }
  __syncthreads();
  float *ot = reinterpret_cast<float *>(reinterpret_cast<char *>(a.out) + a.out_stride * t) + (size_t)g * G * HD;
  uint8_t *oqt = a.oq ? a.oq + a.oq_stride * t : nullptr;
  const uint32_t nbq = a.n_head * HD / 32u;
  for (int b = warp; b < G * HD / 32; b += AM_WARPS) {
    const float v = fin[32 * b + lane];
    ot[32 * b + lane] = v;
    if (oqt) quant_block_warp(v, oqt, nbq, g * (G * HD / 32u) + b, lane);
  }
}

// IE_B200_ATTN=single: one CTA per split at every length (the form without clusters).
static bool attn_cluster_on() {
  static const bool on = [] {
    const char *v = getenv("IE_B200_ATTN");
    return !(v && v[0] == 's' && v[1] == 'i');
  }();
  return on;
}

template <int HD, int G, bool FUSED, int NB, int CL>
static int launch_attn_mma_nb(const AttnArgs &a, uint32_t T, cudaStream_t st) {
  const size_t smem = am_main_bytes(HD, G, NB, a.S) + (CL > 1 ? (size_t)CL * G * (HD + 2) * sizeof(float) : 0);
  auto k = attn_decode_mma_kernel<HD, G, FUSED, NB, CL>;
  if (int r = ensure_dynamic_smem(reinterpret_cast<const void *>(k), smem)) return r;
  if (CL > 1) {
    cudaError_t e_ = launch_pdl_cluster(k, dim3(a.S * CL, a.n_kv, T), dim3(AM_THREADS), smem, st, CL, a);
    count_launch();
    if (e_ != cudaSuccess) return cuda_fail(e_, "attn_decode_mma_kernel (cluster)");
    return IE_B200_OK;
  }
  IEB_LAUNCH_PDL("attn_decode_mma_kernel", k, dim3(a.S, a.n_kv, T), dim3(AM_THREADS), smem, st, a);
  return IE_B200_OK;
}
constexpr int AM_CLUSTER = 4;
template <int HD, int G, bool FUSED>
static int launch_attn_mma(const AttnArgs &a, uint32_t T, cudaStream_t st) {
  const uint64_t ctas = (uint64_t)a.S * a.n_kv * T;
  if (ctas > (uint64_t)sm_count()) return launch_attn_mma_nb<HD, G, FUSED, 3, 1>(a, T, st);
  // few splits (short contexts): four CTAs per split while every CTA still has an SM of its own
  if (ctas * AM_CLUSTER <= (uint64_t)sm_count() && attn_cluster_on()) return launch_attn_mma_nb<HD, G, FUSED, 4, AM_CLUSTER>(a, T, st);
  return launch_attn_mma_nb<HD, G, FUSED, 4, 1>(a, T, st);
}

// ---------------------------------------------------------------------------------------------------------------
// Prompt chunks (T tokens at positions pos0 .. pos0 + T - 1, their K / V rows already in the cache): the same
// tensor-core scheme with all 16 MMA rows in use: a CTA takes QT = 16 / G consecutive tokens of one KV head (rows =
// token-major (token, head) pairs) and streams the cache once for all of them, masking every row at its own token's
// position (causal). No split over positions: a chunk has T / QT x n_kv CTAs already.
struct PrefillArgs {
  const float *q;
  const void *kc, *vc;
  float *out;
  uint8_t *oq;
  const uint32_t *pos;  // position of token 0
  uint32_t n_head, n_kv, kv_len, T;
  size_t q_stride, out_stride, oq_stride;
  float scale;
};

template <int HD, int G>
__global__ void __launch_bounds__(AM_THREADS, 2) attn_prefill_mma_kernel(const PrefillArgs a) {
  constexpr int TILE = ATT_TILE, ROW = HD + AM_PAD, TILE_ELEMS = TILE * ROW, KS = HD / 16, NB = 3;
  constexpr int QT = 16 / G, ROWS = QT * G;  // tokens per CTA, MMA rows in use
  static_assert(G >= 1 && G <= 16, "at least one token's heads fill the 16 MMA rows");
  extern __shared__ uint4 smem_raw[];
  __half *kbuf = reinterpret_cast<__half *>(smem_raw);
  __half *vbuf = kbuf + NB * TILE_ELEMS;

  pdl_prologue();
  const uint32_t t0 = blockIdx.x * QT, g = blockIdx.y;
  const uint32_t nt = min((uint32_t)QT, a.T - t0);            // tokens of this CTA
  const uint32_t pos0 = *a.pos + t0, p_hi = pos0 + nt;         // token i sees positions 0 .. pos0 + i
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, hq = lane >> 2, tq = lane & 3;
  const __half *kh = static_cast<const __half *>(a.kc) + (size_t)g * a.kv_len * HD, *vh = static_cast<const __half *>(a.vc) + (size_t)g * a.kv_len * HD;
  const uint32_t n_tiles = (p_hi + TILE - 1u) / TILE;

  constexpr int PER_ROW = HD * 2 / 16, RPP = AM_THREADS / PER_ROW;
  const uint32_t my_piece = (threadIdx.x % PER_ROW) * 16u, my_row = threadIdx.x / PER_ROW;
  auto issue = [&](uint32_t it) {
    if (it < n_tiles) {
      const uint32_t tile_lo = it * TILE, rows = min((uint32_t)TILE, p_hi - tile_lo);
      const char *ks = reinterpret_cast<const char *>(kh + (size_t)tile_lo * HD) + my_piece, *vs = reinterpret_cast<const char *>(vh + (size_t)tile_lo * HD) + my_piece;
      char *kd = reinterpret_cast<char *>(kbuf + (it % NB) * TILE_ELEMS) + my_piece, *vd = reinterpret_cast<char *>(vbuf + (it % NB) * TILE_ELEMS) + my_piece;
#pragma unroll
      for (int j = 0; j < TILE / RPP; j++) {
        const uint32_t r = my_row + RPP * j;
        const bool ok = r < rows;
        const size_t src = ok ? (size_t)r * HD * 2u : 0u;
        __pipeline_memcpy_async(kd + (size_t)r * ROW * 2u, ks + src, 16, ok ? 0 : 16);
        __pipeline_memcpy_async(vd + (size_t)r * ROW * 2u, vs + src, 16, ok ? 0 : 16);
      }
    }
    __pipeline_commit();
  };
#pragma unroll
  for (int i = 0; i < NB - 1; i++) issue(i);

  // ---- q (already rotated) of this lane's two rows hq and hq + 8, split into two f16 terms; lim = positions the row sees
  uint32_t qh[KS][4], ql[KS][4], lim[2];
#pragma unroll
  for (int h = 0; h < 2; h++) {
    const int r = hq + 8 * h, tk = r / G, hd_ = r % G;
    const bool real = r < ROWS && (uint32_t)tk < nt;
    lim[h] = real ? pos0 + tk + 1u : 0u;
    const float *qp = reinterpret_cast<const float *>(reinterpret_cast<const char *>(a.q) + a.q_stride * (t0 + (real ? tk : 0))) + ((size_t)g * G + hd_) * HD;
#pragma unroll
    for (int k = 0; k < KS; k++) {
      float2 lo2 = make_float2(0.f, 0.f), hi2 = lo2;
      if (real) lo2 = *reinterpret_cast<const float2 *>(qp + 16 * k + 2 * tq), hi2 = *reinterpret_cast<const float2 *>(qp + 16 * k + 2 * tq + 8);
      split2(lo2.x, lo2.y, qh[k][h], ql[k][h]);          // a0 (row hq) / a1 (row hq + 8): columns 2tq, 2tq + 1
      split2(hi2.x, hi2.y, qh[k][2 + h], ql[k][2 + h]);  // a2 / a3: columns 2tq + 8, 2tq + 9
    }
  }
  float o[HD / 8][4], run_m[2] = {-INFINITY, -INFINITY}, run_l[2] = {0.0f, 0.0f};
#pragma unroll
  for (int n = 0; n < HD / 8; n++)
#pragma unroll
    for (int e = 0; e < 4; e++) o[n][e] = 0.0f;
  const int lm = lane >> 3, lr = lane & 7;
  for (uint32_t it = 0; it < n_tiles; it++) {
    const int buf = it % NB;
    const uint32_t tile_lo = it * TILE;
    __pipeline_wait_prior(NB - 2);
    __syncthreads();
    issue(it + NB - 1u);
    const uint32_t p0 = tile_lo + warp * 16u;  // this warp's 16 positions
    if (p0 < p_hi) {
      const __half *kt = kbuf + buf * TILE_ELEMS, *vt = vbuf + buf * TILE_ELEMS;
      float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int k = 0; k < KS; k++) {
        uint32_t kb[4];
        ldsm4(kb, kt + (warp * 16 + (lm >> 1) * 8 + lr) * ROW + 16 * k + (lm & 1) * 8);
        mma_f16(sa, qh[k][0], qh[k][1], qh[k][2], qh[k][3], kb[0], kb[1]);
        mma_f16(sa, ql[k][0], ql[k][1], ql[k][2], ql[k][3], kb[0], kb[1]);
        mma_f16(sb, qh[k][0], qh[k][1], qh[k][2], qh[k][3], kb[2], kb[3]);
        mma_f16(sb, ql[k][0], ql[k][1], ql[k][2], ql[k][3], kb[2], kb[3]);
      }
      uint32_t ph[4], pl[4];  // A fragment of P: a0 / a1 = rows hq / hq + 8 at positions 2tq, +1; a2 / a3 at 8 + 2tq, +1
      float al[2];
#pragma unroll
      for (int h = 0; h < 2; h++) {
        float sc[4];
        sc[0] = p0 + 2 * tq < lim[h] ? sa[2 * h] * a.scale : -INFINITY;
        sc[1] = p0 + 2 * tq + 1 < lim[h] ? sa[2 * h + 1] * a.scale : -INFINITY;
        sc[2] = p0 + 8 + 2 * tq < lim[h] ? sb[2 * h] * a.scale : -INFINITY;
        sc[3] = p0 + 8 + 2 * tq + 1 < lim[h] ? sb[2 * h + 1] * a.scale : -INFINITY;
        float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
        const float m_new = fmaxf(run_m[h], mx), mref = m_new == -INFINITY ? 0.0f : m_new;  // a row may see none of these positions
        al[h] = expf(run_m[h] - mref);
        float pv[4], sum = 0.0f;
#pragma unroll
        for (int e = 0; e < 4; e++) pv[e] = expf(sc[e] - mref), sum += pv[e];
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
        run_l[h] = run_l[h] * al[h] + sum, run_m[h] = m_new;
        split2(pv[0], pv[1], ph[h], pl[h]);
        split2(pv[2], pv[3], ph[2 + h], pl[2 + h]);
      }
#pragma unroll
      for (int u = 0; u < HD / 16; u++) {
        uint32_t vb[4];
        ldsm4t(vb, vt + (warp * 16 + (lm & 1) * 8 + lr) * ROW + 16 * u + (lm >> 1) * 8);
#pragma unroll
        for (int e = 0; e < 4; e++) o[2 * u][e] *= al[e >> 1], o[2 * u + 1][e] *= al[e >> 1];
        mma_f16(o[2 * u], ph[0], ph[1], ph[2], ph[3], vb[0], vb[1]);
        mma_f16(o[2 * u], pl[0], pl[1], pl[2], pl[3], vb[0], vb[1]);
        mma_f16(o[2 * u + 1], ph[0], ph[1], ph[2], ph[3], vb[2], vb[3]);
        mma_f16(o[2 * u + 1], pl[0], pl[1], pl[2], pl[3], vb[2], vb[3]);
      }
    }
  }
  __pipeline_wait_prior(0);
  __syncthreads();
  // ---- merge the warps' (max, sum, output) per row in shared memory, reusing the tile buffers
  float *red = reinterpret_cast<float *>(smem_raw);  // [AM_WARPS][16][HD]
  float *ml = red + AM_WARPS * 16 * HD;               // [AM_WARPS][16][2]
  float *fin = ml + AM_WARPS * 16 * 2;                // [16][HD]
#pragma unroll
  for (int h = 0; h < 2; h++) {
    const int r = hq + 8 * h;
#pragma unroll
    for (int n = 0; n < HD / 8; n++) *reinterpret_cast<float2 *>(red + (warp * 16 + r) * HD + 8 * n + 2 * tq) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
    if (tq == 0) ml[(warp * 16 + r) * 2] = run_m[h], ml[(warp * 16 + r) * 2 + 1] = run_l[h];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < ROWS * HD; e += AM_THREADS) {
    const int r = e / HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < AM_WARPS; w++) M = fmaxf(M, ml[(w * 16 + r) * 2]);
    float L = 0.0f, acc = 0.0f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < AM_WARPS; w++) {
        const float wk = expf(ml[(w * 16 + r) * 2] - M);
        L = fmaf(wk, ml[(w * 16 + r) * 2 + 1], L);
        acc = fmaf(wk, red[(w * 16 + r) * HD + (e % HD)], acc);
      }
    }
    fin[e] = L > 0.0f ? acc * (1.0f / L) : 0.0f;
  }
  __syncthreads();
  // ---- write out: one warp per 32 values of a (token, head) row, which is also a Q8 block of that token's output
  const uint32_t nbq = a.n_head * HD / 32u;
  for (int b = warp; b < ROWS * HD / 32; b += AM_WARPS) {
    const int r = (32 * b) / HD, tk = r / G, hd_ = r % G;
    if ((uint32_t)tk >= nt) continue;
    const float v = fin[32 * b + lane];
    const uint32_t col = ((uint32_t)g * G + hd_) * HD + (32 * b) % HD;
    reinterpret_cast<float *>(reinterpret_cast<char *>(a.out) + a.out_stride * (t0 + tk))[col + lane] = v;
    if (a.oq) quant_block_warp(v, a.oq + a.oq_stride * (t0 + tk), nbq, col / 32u, lane);
  }
}

template <int HD, int G>
static int launch_prefill(const PrefillArgs &a, cudaStream_t st) {
  constexpr int QT = 16 / G;
  const size_t tile = (size_t)3 * 2 * ATT_TILE * (HD + AM_PAD) * sizeof(__half);
  const size_t red = (size_t)((AM_WARPS + 1) * 16 * HD + AM_WARPS * 16 * 2) * sizeof(float);
  const size_t smem = tile > red ? tile : red;
  auto k = attn_prefill_mma_kernel<HD, G>;
  if (int r = ensure_dynamic_smem(reinterpret_cast<const void *>(k), smem)) return r;
  IEB_LAUNCH_PDL("attn_prefill_mma_kernel", k, dim3((a.T + QT - 1) / QT, a.n_kv), dim3(AM_THREADS), smem, st, a);
  return IE_B200_OK;
}
template <int HD>
static int dispatch_prefill(const PrefillArgs &a, uint32_t G, cudaStream_t st) {
  switch (G) {
    case 1: return launch_prefill<HD, 1>(a, st);
    case 2: return launch_prefill<HD, 2>(a, st);
    case 3: return launch_prefill<HD, 3>(a, st);
    case 4: return launch_prefill<HD, 4>(a, st);
    case 5: return launch_prefill<HD, 5>(a, st);
    case 6: return launch_prefill<HD, 6>(a, st);
    case 7: return launch_prefill<HD, 7>(a, st);
    case 8: return launch_prefill<HD, 8>(a, st);
    default: return fail(IE_B200_E_SIZE, "ie_b200_attn_prefill: %u query heads per KV head unsupported (1 .. 8)", G);
  }
}

// IE_B200_ATTN=scalar keeps the CUDA-core kernel for the half cache as well.
static bool attn_use_mma() {
  static const bool on = [] {
    const char *v = getenv("IE_B200_ATTN");
    return !(v && v[0] == 's' && v[1] == 'c');
  }();
  return on;
}

template <int HD, bool FUSED>
static int dispatch_g_mma(const AttnArgs &a, uint32_t G, uint32_t T, cudaStream_t st) {
  switch (G) {
    case 1: return launch_attn_mma<HD, 1, FUSED>(a, T, st);
    case 2: return launch_attn_mma<HD, 2, FUSED>(a, T, st);
    case 3: return launch_attn_mma<HD, 3, FUSED>(a, T, st);
    case 4: return launch_attn_mma<HD, 4, FUSED>(a, T, st);
    case 5: return launch_attn_mma<HD, 5, FUSED>(a, T, st);
    case 6: return launch_attn_mma<HD, 6, FUSED>(a, T, st);
    case 7: return launch_attn_mma<HD, 7, FUSED>(a, T, st);
    case 8: return launch_attn_mma<HD, 8, FUSED>(a, T, st);
    default: return fail(IE_B200_E_SIZE, "ie_b200_attn_decode: %u query heads per KV head unsupported (1 .. 8)", G);
  }
}

template <typename KV, int HD, bool FUSED>
static int dispatch_g(const AttnArgs &a, uint32_t G, uint32_t T, cudaStream_t st) {
  switch (G) {
    case 1: return launch_attn<KV, HD, 1, FUSED>(a, T, st);
    case 2: return launch_attn<KV, HD, 2, FUSED>(a, T, st);
    case 3: return launch_attn<KV, HD, 3, FUSED>(a, T, st);
    case 4: return launch_attn<KV, HD, 4, FUSED>(a, T, st);
    case 5: return launch_attn<KV, HD, 5, FUSED>(a, T, st);
    case 6: return launch_attn<KV, HD, 6, FUSED>(a, T, st);
    case 7: return launch_attn<KV, HD, 7, FUSED>(a, T, st);
    case 8: return launch_attn<KV, HD, 8, FUSED>(a, T, st);
    default: return fail(IE_B200_E_SIZE, "ie_b200_attn_decode: %u query heads per KV head unsupported (1 .. 8)", G);
  }
}

// Splits (grid.x): as many as fit the SMs in one wave (ctas_per_sm resident CTAs each; a partial second wave would
// double the time), spans of at least ATT_MIN_SPAN positions.
static uint32_t attn_splits(uint32_t n_kv, uint32_t n_ctx, uint32_t T, uint32_t ctas_per_sm) {
  const uint32_t by_len = (n_ctx + ATT_MIN_SPAN - 1u) / ATT_MIN_SPAN;
  uint32_t by_sm = ctas_per_sm * (uint32_t)sm_count() / (n_kv * T);
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
    if (attn_use_mma() && hd == 64) return dispatch_g_mma<64, FUSED>(a, G, T, st);
    if (attn_use_mma() && hd == 128) return dispatch_g_mma<128, FUSED>(a, G, T, st);
    switch (hd) {
      case 32: return dispatch_g<__half, 32, FUSED>(a, G, T, st);
      case 64: return dispatch_g<__half, 64, FUSED>(a, G, T, st);
      case 128: return dispatch_g<__half, 128, FUSED>(a, G, T, st);
    }
  }
  return fail(IE_B200_E_SIZE, "ie_b200_attn_decode: head dim %u unsupported (32, 64, 128)", hd);
}

// Resident CTAs per SM of the kernel that will run (shared memory decides): the tensor-core kernel keeps 3 tile
// buffers of 34 KB (hd 128), two CTAs per SM; the CUDA-core kernel fills an SM's shared memory with one.
static uint32_t attn_ctas_per_sm(uint32_t hd, int kv_f32) { return (!kv_f32 && attn_use_mma() && (hd == 64 || hd == 128)) ? 2u : 1u; }

}  // namespace ieb

using namespace ieb;

extern "C" size_t ie_b200_attn_part_bytes(uint32_t n_head, uint32_t hd, uint32_t n_ctx, uint32_t T) {
  // an upper bound over every KV-head count: splits never exceed ceil(n_ctx / 256)
  const size_t S = (n_ctx + ATT_MIN_SPAN - 1u) / ATT_MIN_SPAN;
  return (size_t)T * n_head * (S ? S : 1u) * (hd + 4u) * sizeof(float);
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
  a.n_head = n_head, a.n_kv = n_kv, a.kv_len = kv_len, a.S = attn_splits(n_kv, n_ctx, T, attn_ctas_per_sm(hd, kv_f32));
  a.q_stride = q_stride, a.out_stride = out_stride, a.oq_stride = oq_stride;
  a.part = static_cast<float *>(d_part), a.count = d_count;
  a.scale = 1.0f / sqrtf((float)hd);
  a.k_new = a.v_new = a.cs = a.sn = nullptr, a.neox = 0, a.early_kv = 0;
  return dispatch_attn<false>(a, hd, kv_f32, T, static_cast<cudaStream_t>(stream));
}

namespace ieb {
// early: the kernel launched right before this one releases its dependents only after its own dependency wait
// (gemv_direct's late_trigger), so the position and older cache rows may be read ahead of this kernel's wait.
int attn_decode_fused(const float *d_q, const float *d_k, const float *d_v, void *d_kc, void *d_vc, const float *d_cos, const float *d_sin, float *d_out,
                      void *d_oq, const uint32_t *d_pos, uint32_t n_head, uint32_t n_kv, uint32_t hd, int neox, int kv_f32, uint32_t kv_len, uint32_t n_ctx,
                      void *d_part, uint32_t *d_count, cudaStream_t st, bool early) {
  if (!d_q || !d_k || !d_v || !d_kc || !d_vc || !d_cos || !d_sin || !d_out || !d_pos || !d_part || !d_count)
    return fail(IE_B200_E_ARG, "ie_b200_attn_decode_fused: NULL pointer");
  if (n_kv == 0 || n_head % n_kv) return fail(IE_B200_E_SIZE, "ie_b200_attn_decode_fused: %u heads over %u KV heads", n_head, n_kv);
  if (kv_len < n_ctx) return fail(IE_B200_E_SIZE, "ie_b200_attn_decode_fused: cache rows %u < context %u (ring caches unsupported)", kv_len, n_ctx);
  if (!aligned16(d_kc) || !aligned16(d_vc) || !aligned16(d_q)) return fail(IE_B200_E_ARG, "ie_b200_attn_decode_fused: q and the caches must be 16-byte aligned");
  AttnArgs a;
  a.q = d_q, a.kc = d_kc, a.vc = d_vc, a.out = d_out, a.oq = static_cast<uint8_t *>(d_oq), a.pos = d_pos;
  a.n_head = n_head, a.n_kv = n_kv, a.kv_len = kv_len, a.S = attn_splits(n_kv, n_ctx, 1, attn_ctas_per_sm(hd, kv_f32));
  a.q_stride = a.out_stride = a.oq_stride = 0;
  a.part = static_cast<float *>(d_part), a.count = d_count;
  a.scale = 1.0f / sqrtf((float)hd);
  a.k_new = d_k, a.v_new = d_v, a.cs = d_cos, a.sn = d_sin, a.neox = neox;
  a.early_kv = early ? 1 : 0;
  return dispatch_attn<true>(a, hd, kv_f32, 1, st);
}
}  // namespace ieb

extern "C" int ie_b200_attn_decode_fused(const float *d_q, const float *d_k, const float *d_v, void *d_kc, void *d_vc, const float *d_cos,
                                         const float *d_sin, float *d_out, void *d_oq, const uint32_t *d_pos, uint32_t n_head, uint32_t n_kv,
                                         uint32_t hd, int neox, int kv_f32, uint32_t kv_len, uint32_t n_ctx, void *d_part, uint32_t *d_count,
                                         void *stream) {
  return attn_decode_fused(d_q, d_k, d_v, d_kc, d_vc, d_cos, d_sin, d_out, d_oq, d_pos, n_head, n_kv, hd, neox, kv_f32, kv_len, n_ctx, d_part, d_count,
                           static_cast<cudaStream_t>(stream), false);
}

extern "C" int ie_b200_attn_prefill(const float *d_q, const void *d_kc, const void *d_vc, float *d_out, void *d_oq, const uint32_t *d_pos,
                                    uint32_t n_head, uint32_t n_kv, uint32_t hd, uint32_t kv_len, uint32_t T, size_t q_stride, size_t out_stride,
                                    size_t oq_stride, void *stream) {
  if (!d_q || !d_kc || !d_vc || !d_out || !d_pos) return fail(IE_B200_E_ARG, "ie_b200_attn_prefill: NULL pointer");
  if (n_kv == 0 || n_head % n_kv) return fail(IE_B200_E_SIZE, "ie_b200_attn_prefill: %u heads over %u KV heads", n_head, n_kv);
  if (hd != 64 && hd != 128) return fail(IE_B200_E_SIZE, "ie_b200_attn_prefill: head dim %u (64, 128; half-precision cache)", hd);
  if (!aligned16(d_kc) || !aligned16(d_vc) || ((uintptr_t)d_q & 7u) || (q_stride & 7u)) return fail(IE_B200_E_ARG, "ie_b200_attn_prefill: alignment");
  if (T == 0) return IE_B200_OK;
  PrefillArgs a;
  a.q = d_q, a.kc = d_kc, a.vc = d_vc, a.out = d_out, a.oq = static_cast<uint8_t *>(d_oq), a.pos = d_pos;
  a.n_head = n_head, a.n_kv = n_kv, a.kv_len = kv_len, a.T = T;
  a.q_stride = q_stride, a.out_stride = out_stride, a.oq_stride = oq_stride;
  a.scale = 1.0f / sqrtf((float)hd);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return hd == 64 ? dispatch_prefill<64>(a, n_head / n_kv, st) : dispatch_prefill<128>(a, n_head / n_kv, st);
}
