// step_kernel.cu -- whole decode steps as ONE persistent cooperative kernel: the role of the reference's
// megakernel (kernels/ie_mk.c:43-95 with the grid barrier of kernels/ie_kernels.c:417-463 and the recorder of
// src/hip.c:445-566), designed for B200: one CTA of 16 warps per SM walks a list of phases; dependent phases are
// separated by a grid barrier (one atomic arrival per CTA, bounded wait), and everything a phase needs that does
// not depend on the barrier -- the weights -- is requested from HBM before the CTA arrives, so the weight stream
// does not stop at a phase boundary:
//
//   GEMV     every warp owns rows (4 at a time, 16 16-byte loads per lane in flight); the activations are staged
//            per CTA by a prologue: a Q8 buffer, or RMSNorm + Q8 of the residual stream, or SwiGLU + Q8 of the
//            gate / up pairs, computed redundantly by every CTA (a few KB from L2) instead of a phase of its own.
//            Arithmetic and order as the decode GEMV: bit-exact with the reference CPU GEMV.
//   ATTN     the (KV head, split) items of a layer go to groups of four warps (two per CTA) running the tensor-core
//            tile loop of the decode attention (f16 cache, q / p as two f16 terms, RoPE and the KV store folded in);
//            with up to 37 splits per KV head a short context is one 64-position tile per group. The other warps
//            pull the next matrices into L2 meanwhile.
//   MERGE    one warp per head: the splits' (max, sum, out) records -> output and its Q8 copy.
//   ARGMAX / FINISH   slices of the logits, then CTA 0 merges, logs the token and advances token and position, so
//            the kernel loops over K tokens without the host.
//   tensor parallel: a K-split GEMV stores its finished rows into every rank's low-latency slots (peer_ll.cuh);
//            REDUCE (one warp per 32 rows) polls the slots, adds the ranks' partials in rank order onto the residual
//            stream; XARGMAX exchanges the ranks' local winners.
//
// Every wait (grid barrier, peer slots) is bounded by wall time; a wait that runs out sets the device error word
// and the abort flag, every CTA leaves at its next barrier, the host reports IE_B200_E_DEVICE.
#include <cuda_fp16.h>
#include <math.h>

#include "act_stage.cuh"
#include "common.cuh"
#include "gemv_blocks.cuh"
#include "step_kernel.cuh"

namespace ieb {

// 8 warps per CTA, one CTA per SM: 255 registers per thread, so that neither the GEMV loop with 24 loads per lane in flight
// nor the attention tile loop (64 accumulator registers) spills. (16 warps at 128 registers spilled about 1 KB per thread;
// with the kernel's shared memory leaving an L1 of a few tens of KB, that traffic went to L2 and tripled the step time.)
constexpr int SK_WARPS = 8, SK_THREADS = SK_WARPS * 32;
constexpr int SK_GROUPS = 2, SK_GW = 4, SK_GT = SK_GW * 32;  // attention: two groups of four warps per CTA
constexpr int SK_TILE = 64, SK_PAD = 8, SK_NB = 3;            // 64-position tiles, rows padded by 8 halves, 3 tile buffers per group

struct SkArgPart {
  float mx;
  uint32_t idx;
  float sum;
  uint32_t pad;
};

__device__ __forceinline__ uint32_t ld_cg_u32(const uint32_t *p) { return __ldcg(p); }
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void group_sync(int id) { asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(SK_GT) : "memory"); }
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *src, bool ok) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst), n = ok ? 16u : 0u;  // n = 0: sixteen zero bytes
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ---- the grid barrier ----------------------------------------------------------------------------------------
// Arrivals are counted in bar[0] (zero at launch, never reset inside the kernel: the n-th barrier waits for
// n * gridDim.x). One thread per CTA arrives (after a fence that publishes the CTA's writes) and polls with
// acquire loads; the others wait at the CTA barrier. False: the wait ran out or another CTA gave up.
struct SkBar {
  uint32_t *count, *abort, *err;
  uint32_t target;
  uint64_t wait_ns;
  unsigned long long *trace;  // CTA 0 only: time from the last release to this arrival and from arrival to release, per phase kind
  uint64_t t_rel;
};
__device__ __forceinline__ bool grid_sync(SkBar &b, uint32_t *s_ok, int kind) {
  __syncthreads();
  b.target += gridDim.x;
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(b.count, 1u);
    uint32_t ok = 1u;
    const uint64_t t0 = ar_now();
    while ((int32_t)(ld_acquire_u32(b.count) - b.target) < 0) {
      if (*(volatile uint32_t *)b.abort) {
        ok = 0u;
        break;
      }
      if (ar_now() - t0 > b.wait_ns) {
        atomicExch(b.err, 4u);
        *(volatile uint32_t *)b.abort = 1u;
        ok = 0u;
        break;
      }
    }
    *s_ok = ok;
    if (b.trace) {
      const uint64_t t1 = ar_now();
      b.trace[3 * kind] += t0 - b.t_rel, b.trace[3 * kind + 1] += t1 - t0, b.trace[3 * kind + 2] += 1ull;
      b.t_rel = t1;
    }
  }
  __syncthreads();
  return *s_ok != 0u;
}

// Part `part` of `nparts` of the lines of [p, p + bytes) into L2, by the `nthr` threads numbered `t`.
__device__ __forceinline__ void prefetch_part(const uint8_t *p, uint64_t bytes, uint32_t part, uint32_t nparts, uint32_t t, uint32_t nthr) {
  const uint64_t lines = (bytes + 127u) >> 7;
  const uint64_t per = (lines + nparts - 1u) / nparts, lo = per * part;
  const uint64_t hi = lo + per < lines ? lo + per : lines;
  for (uint64_t i = lo + t; i < hi; i += nthr) prefetch_l2(p + (i << 7));
}

// ---- GEMV ------------------------------------------------------------------------------------------------------
// Rows are dealt in groups of R to all warps of the grid (warp w of CTA c is number w * gridDim.x + c, so a matrix
// with fewer groups than warps still uses every SM): whole rounds first, then the rest spread evenly.
struct SkRows {
  uint32_t W, gw, full, base, rp;
};
template <int R>
__device__ __forceinline__ SkRows sk_rows(uint32_t rows, int warp, bool pairs) {
  static_assert(R % 2 == 0, "row pairs stay in one group");
  SkRows s;
  s.W = gridDim.x * SK_WARPS, s.gw = (uint32_t)warp * gridDim.x + blockIdx.x;
  s.full = rows / (R * s.W), s.base = s.full * s.W * R;
  s.rp = (rows - s.base + s.W - 1u) / s.W;
  if (pairs) s.rp = (s.rp + 1u) & ~1u;  // (gate, up) pairs are not split between warps
  return s;
}

template <int KIND, int R, int U>
__device__ __forceinline__ void sk_group(const StepPhase &ph, const StepArgs &a, uint32_t r0, uint32_t nr, const uint4 *A0, const uint4 *A1,
                                         const float *da, const int *as, int lane, uint32_t ep) {
  const uint32_t nb = ph.nb;
  const size_t rowb = ph.rowb;
  // the residual / bias of row r0 + lane early: their latency hides behind the weights
  float rv = 0.0f, bv = 0.0f;
  if ((uint32_t)lane < nr) {
    if (ph.res) rv = __ldcg(ph.res + r0 + lane);
    if (ph.bias) bv = __ldg(ph.bias + r0 + lane);
  }
  float acc[R];
#pragma unroll
  for (int i = 0; i < R; i++) acc[i] = 0.0f;
  for (uint32_t c = 0; c < nb; c += 32u * U) {
    Blk<KIND, false> blk[R][U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const uint32_t b = c + 32u * u + lane;
      if (b < nb) {
#pragma unroll
        for (int i = 0; i < R; i++)
          if ((uint32_t)i < nr) blk[i][u].load(ph.w + (size_t)(r0 + i) * rowb, b, nb);
      }
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
          if ((uint32_t)i < nr) acc[i] = blk[i][u].accum(acc[i], a0, a1, d, s, b);
      }
    }
  }
  float v[R];
#pragma unroll
  for (int i = 0; i < R; i++) v[i] = __shfl_sync(0xFFFFFFFFu, warp_tree(acc[i]), 0);
  if (ph.swi) {
    // rows r0 + 2j, r0 + 2j + 1 are gate and up of output (r0 >> 1) + j (r0 and nr are even): the SwiGLU kernel's arithmetic
#pragma unroll
    for (int j = 0; j < R / 2; j++) {
      if (lane == j && (uint32_t)(2 * j + 1) < nr) {
        const float g = v[2 * j];
        ph.y[(r0 >> 1) + j] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), v[2 * j + 1]);
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < R; i++) {
    if (lane == i && (uint32_t)i < nr) {
      float o = v[i];
      if (ph.bias) o = __fadd_rn(o, bv);
      if (ph.res) o = __fadd_rn(rv, o);
      ph.y[r0 + i] = o;
    }
  }
  if (ph.push) {  // tensor parallel: the rows to every rank's slots (the own rank's too: the reduction polls them all alike)
    if ((uint32_t)lane < a.push.world) {
      unsigned long long *dst = a.push.ll[lane] + ((size_t)(ep & 1u) * a.push.world + a.push.rank) * a.push.max_n + r0;
#pragma unroll
      for (int i = 0; i < R; i++)
        if ((uint32_t)i < nr) ll_store(dst + i, ep, __float_as_uint(v[i]));
    }
  }
}

// The rows [r0, r0 + nr) of a matrix into L2 (whole rows, at most 16 KB each), by one warp.
__device__ __forceinline__ void sk_prefetch_rows(const uint8_t *w, size_t rowb, uint32_t r0, uint32_t nr, int lane) {
  const uint32_t lines = (uint32_t)((rowb + 127u) >> 7);
  for (uint32_t i = 0; i < nr; i++) {
    const uint8_t *rp = w + (size_t)(r0 + i) * rowb;
    for (uint32_t l = lane; l < lines && l < 128u; l += 32u) prefetch_l2(rp + ((size_t)l << 7));
  }
}

// One copy of the group code per instantiation (whole rounds and the evenly spread rest share it): two inlined copies cost
// some 30 registers more. Before a group is worked on, the rows of the warp's next group are asked into L2, so that only the
// first group of a phase pays the full trip to HBM.
template <int KIND, int R, int U>
__device__ __forceinline__ void sk_gemv(const StepPhase &ph, const StepArgs &a, const uint4 *A0, const uint4 *A1, const float *da, const int *as, int warp,
                                        int lane, uint32_t ep) {
  const SkRows s = sk_rows<R>(ph.rows, warp, ph.swi != 0u);
  const uint32_t rows = ph.rows;
  auto group_of = [&](uint32_t k, uint32_t &r0, uint32_t &nr) {
    r0 = (k * s.W + s.gw) * R, nr = R;
    if (k == s.full) {
      r0 = s.base + s.gw * s.rp;
      nr = (s.rp && r0 < rows) ? min(s.rp, rows - r0) : 0u;
    }
  };
  for (uint32_t k = 0; k <= s.full; k++) {
    uint32_t r0, nr;
    group_of(k, r0, nr);
    if ((a.knobs & 1u) && k < s.full) {
      uint32_t rn, nn;
      group_of(k + 1u, rn, nn);
      sk_prefetch_rows(ph.w, ph.rowb, rn, nn, lane);
    }
    if (nr) sk_group<KIND, R, U>(ph, a, r0, nr, A0, A1, da, as, lane, ep);
  }
}

// Rows per group of the instantiation that takes a matrix (must agree with the dispatch in the kernel).
__device__ __forceinline__ int sk_rows_per_group(int mkind, uint32_t nb) {
  (void)nb;
  return mkind == IE_B200_MAT_Q4 ? 4 : 2;
}

// The rows of this warp's first group of a GEMV phase into L2 (called before the barrier in front of the phase).
__device__ __forceinline__ void sk_gemv_prefetch(const StepPhase &ph, int warp, int lane) {
  const int R = sk_rows_per_group(ph.mkind, ph.nb);
  const uint32_t W = gridDim.x * SK_WARPS, gw = (uint32_t)warp * gridDim.x + blockIdx.x;
  const uint32_t full = ph.rows / (R * W);
  uint32_t r0, nr;
  if (full) {
    r0 = gw * R, nr = R;
  } else {
    uint32_t rp = (ph.rows + W - 1u) / W;
    if (ph.swi) rp = (rp + 1u) & ~1u;
    r0 = gw * rp, nr = rp;
  }
  if (r0 < ph.rows) sk_prefetch_rows(ph.w, ph.rowb, r0, min(nr, ph.rows - r0), lane);
}

// Q8 of an f32 vector into the activation planes: thread t owns half-blocks t, t + SK_THREADS, ... (16 values each).
__device__ __forceinline__ void sk_stage_quant(const float *x, uint32_t nb, uint4 *A0, uint4 *A1, float *da, int *as) {
  const uint32_t HB = 2u * nb;
  for (uint32_t k0 = 0; k0 < HB; k0 += SK_THREADS) {  // uniform trip count: the shuffles need every lane
    const uint32_t hb = k0 + threadIdx.x, b = hb >> 1, h = hb & 1u;
    const bool valid = hb < HB;
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; j += 4) {
      float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
      if (valid) p = __ldcg(reinterpret_cast<const float4 *>(x + 16u * (size_t)hb + j));
      v[j] = p.x, v[j + 1] = p.y, v[j + 2] = p.z, v[j + 3] = p.w;
    }
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; j++) amax = fmaxf(amax, fabsf(v[j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    const float d = __fdiv_rn(amax, 127.0f), rinv = __frcp_rn(d);
    uint32_t pk[4] = {0u, 0u, 0u, 0u};
    int s = 0;
#pragma unroll
    for (int j = 0; j < 16; j++) {
      int q = 0;
      if (d != 0.0f) q = q8_round(v[j], d, rinv);
      s += q;
      pk[j >> 2] |= (uint32_t)(q & 255) << (8 * (j & 3));
    }
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
    if (valid) {
      (h ? A1 : A0)[b] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      if (h == 0u) da[b] = d, as[b] = s;
    }
  }
}

// SwiGLU + Q8 of interleaved (gate_i, up_i) pairs into the activation planes: thread t owns half-blocks t, t + 512,
// ... (16 outputs each), the arithmetic of the SwiGLU kernel and of the CPU: h = (g / (1 + exp(-g))) * u.
__device__ __forceinline__ void sk_stage_swiglu(const float *gu, uint32_t nb, uint4 *A0, uint4 *A1, float *da, int *as) {
  const uint32_t HB = 2u * nb;
  for (uint32_t k0 = 0; k0 < HB; k0 += SK_THREADS) {  // uniform trip count: the shuffles need every lane
    const uint32_t hb = k0 + threadIdx.x, b = hb >> 1, h = hb & 1u;
    const bool valid = hb < HB;
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; j += 2) {
      float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
      if (valid) p = __ldcg(reinterpret_cast<const float4 *>(gu + 32u * (size_t)hb + 2 * j));
      v[j] = __fmul_rn(__fdiv_rn(p.x, __fadd_rn(1.0f, expf(-p.x))), p.y);
      v[j + 1] = __fmul_rn(__fdiv_rn(p.z, __fadd_rn(1.0f, expf(-p.z))), p.w);
    }
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; j++) amax = fmaxf(amax, fabsf(v[j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    const float d = __fdiv_rn(amax, 127.0f), rinv = __frcp_rn(d);
    uint32_t pk[4] = {0u, 0u, 0u, 0u};
    int s = 0;
#pragma unroll
    for (int j = 0; j < 16; j++) {
      int q = 0;
      if (d != 0.0f) q = q8_round(v[j], d, rinv);
      s += q;
      pk[j >> 2] |= (uint32_t)(q & 255) << (8 * (j & 3));
    }
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
    if (valid) {
      (h ? A1 : A0)[b] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      if (h == 0u) da[b] = d, as[b] = s;
    }
  }
}

// ---- attention: one (KV head g, split s) item by a group of four warps ------------------------------------------
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void *p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], const void *p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void split2(float x, float y, uint32_t &hi, uint32_t &lo) {
  const __half2 h = __floats2half2_rn(x, y);
  const float2 hf = __half22float2(h);
  const __half2 l = __floats2half2_rn(x - hf.x, y - hf.y);
  hi = *reinterpret_cast<const uint32_t *>(&h), lo = *reinterpret_cast<const uint32_t *>(&l);
}
__device__ __forceinline__ float rope_lo(float a, float b, float c, float s) { return __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)); }
__device__ __forceinline__ float rope_hi(float a, float b, float c, float s) { return __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c)); }

// Splits of np positions over at most smax: one 64-position tile per split while the groups last.
__device__ __forceinline__ void sk_splits(uint32_t np, uint32_t smax, uint32_t &span, uint32_t &A) {
  const uint32_t tiles = (np + SK_TILE - 1u) / SK_TILE;
  const uint32_t want = tiles < smax ? tiles : smax;
  span = ((np + want - 1u) / want + SK_TILE - 1u) / SK_TILE * SK_TILE;
  A = (np + span - 1u) / span;
}

// Shared memory of a group: SK_NB K tiles, SK_NB V tiles ([64][HD + 8] halves each), then the q fragments
// ([HD / 16][32 lanes] x {hi a0, hi a2, lo a0, lo a2}).
template <int HD>
struct SkAttnSmem {
  static constexpr int ROW = HD + SK_PAD, TILE_ELEMS = SK_TILE * ROW;
  static constexpr int TILES_BYTES = 2 * SK_NB * TILE_ELEMS * 2;
  static constexpr int Q_BYTES = (HD / 16) * 32 * 16;
  static constexpr int BYTES = TILES_BYTES + Q_BYTES;
};

template <int HD>
__device__ __forceinline__ void sk_attn_item(const StepArgs &a, const StepPhase &ph, uint32_t g, uint32_t s, uint32_t A, uint32_t span, uint32_t np,
                                             uint8_t *gsm, int gtid, int bar_id) {
  using SM = SkAttnSmem<HD>;
  constexpr int ROW = SM::ROW, TILE_ELEMS = SM::TILE_ELEMS, KS = HD / 16;
  __half *kbuf = reinterpret_cast<__half *>(gsm);
  __half *vbuf = kbuf + SK_NB * TILE_ELEMS;
  uint4 *qsm = reinterpret_cast<uint4 *>(gsm + SM::TILES_BYTES);
  const uint32_t G = a.n_head / a.n_kv;
  const int lane = gtid & 31, warp = gtid >> 5, hq = lane >> 2, tq = lane & 3;
  const float scale = 1.0f / sqrtf((float)HD);
  const float *qt = ph.q + (size_t)g * G * HD;
  const float *k_new = ph.q + (size_t)a.n_head * HD + (size_t)g * HD, *v_new = ph.q + (size_t)(a.n_head + a.n_kv) * HD + (size_t)g * HD;
  const __half *kh = static_cast<const __half *>(ph.kc) + (size_t)g * a.kv_len * HD, *vh = static_cast<const __half *>(ph.vc) + (size_t)g * a.kv_len * HD;
  const uint32_t p_lo = s * span, p_hi = min(np, p_lo + span);
  const bool owns_new = s == A - 1u;  // this item's span ends with the step's own position
  const uint32_t n_tiles = (p_hi - p_lo + SK_TILE - 1u) / SK_TILE;

  // tile `it` into buffer it % SK_NB: cache rows by 16-byte async copies, rows past the span zero-filled, the
  // step's own row left to the registers below
  constexpr int PER_ROW = HD * 2 / 16, RPP = SK_GT / PER_ROW;
  const uint32_t my_piece = (gtid % PER_ROW) * 16u, my_row = gtid / PER_ROW;
  auto issue = [&](uint32_t it) {
    if (it < n_tiles) {
      const uint32_t tile_lo = p_lo + it * SK_TILE;
      const uint32_t have = p_hi - tile_lo;
      const bool with_new = owns_new && it + 1u == n_tiles;
      const uint32_t rows = min((uint32_t)SK_TILE, have - (with_new ? 1u : 0u));
      const char *ks = reinterpret_cast<const char *>(kh + (size_t)tile_lo * HD) + my_piece, *vs = reinterpret_cast<const char *>(vh + (size_t)tile_lo * HD) + my_piece;
      char *kd = reinterpret_cast<char *>(kbuf + (it % SK_NB) * TILE_ELEMS) + my_piece, *vd = reinterpret_cast<char *>(vbuf + (it % SK_NB) * TILE_ELEMS) + my_piece;
#pragma unroll
      for (int j = 0; j < SK_TILE / RPP; j++) {
        const uint32_t r = my_row + RPP * j;
        if (with_new && r == have - 1u) continue;
        const bool ok = r < rows;
        const size_t src = ok ? (size_t)r * HD * 2u : 0u;
        cp_async16(kd + (size_t)r * ROW * 2u, ks + src, ok);
        cp_async16(vd + (size_t)r * ROW * 2u, vs + src, ok);
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int i = 0; i < SK_NB - 1; i++) issue(i);

  // ---- q of head hq in A-fragment order (this warp's share of the 16-dim steps), rotated, as two f16 terms, into
  // shared memory; pairs (2i, 2i+1) sit side by side, pairs (i, i + hd/2) are steps k and k + KS/2 of one lane
  const float *cs = a.cs + (size_t)(np - 1u) * (HD / 2), *sn = a.sn + (size_t)(np - 1u) * (HD / 2);
  for (int k = warp; k < KS / 2; k += SK_GW) {
    float qa[4], qb[4];  // steps k and k + KS/2: dims 16 k + {2tq, 2tq+1, 2tq+8, 2tq+9}
    const int k2 = k + KS / 2;
#pragma unroll
    for (int e = 0; e < 4; e++) qa[e] = qb[e] = 0.0f;
    if ((uint32_t)hq < G) {
      const float2 a0 = __ldcg(reinterpret_cast<const float2 *>(qt + hq * HD + 16 * k + 2 * tq)), a1 = __ldcg(reinterpret_cast<const float2 *>(qt + hq * HD + 16 * k + 2 * tq + 8));
      const float2 b0 = __ldcg(reinterpret_cast<const float2 *>(qt + hq * HD + 16 * k2 + 2 * tq)), b1 = __ldcg(reinterpret_cast<const float2 *>(qt + hq * HD + 16 * k2 + 2 * tq + 8));
      qa[0] = a0.x, qa[1] = a0.y, qa[2] = a1.x, qa[3] = a1.y;
      qb[0] = b0.x, qb[1] = b0.y, qb[2] = b1.x, qb[3] = b1.y;
    }
    if (!a.neox) {
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int ia = 8 * k + tq + 4 * e, ib = 8 * k2 + tq + 4 * e;  // pair index (16 k + 2 tq + 8 e) / 2
        const float ca = __ldg(cs + ia), sa_ = __ldg(sn + ia), cb = __ldg(cs + ib), sb_ = __ldg(sn + ib);
        const float y0 = qa[2 * e], y1 = qa[2 * e + 1], z0 = qb[2 * e], z1 = qb[2 * e + 1];
        qa[2 * e] = rope_lo(y0, y1, ca, sa_), qa[2 * e + 1] = rope_hi(y0, y1, ca, sa_);
        qb[2 * e] = rope_lo(z0, z1, cb, sb_), qb[2 * e + 1] = rope_hi(z0, z1, cb, sb_);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int i = 16 * k + 2 * tq + (e & 1) + 8 * (e >> 1);  // dim i pairs with dim i + hd/2
        const float c = __ldg(cs + i), sv = __ldg(sn + i), y0 = qa[e], y1 = qb[e];
        qa[e] = rope_lo(y0, y1, c, sv), qb[e] = rope_hi(y0, y1, c, sv);
      }
    }
    uint4 fa, fb;
    split2(qa[0], qa[1], fa.x, fa.z);
    split2(qa[2], qa[3], fa.y, fa.w);
    split2(qb[0], qb[1], fb.x, fb.z);
    split2(qb[2], qb[3], fb.y, fb.w);
    qsm[k * 32 + lane] = fa, qsm[k2 * 32 + lane] = fb;  // {hi a0, hi a2, lo a0, lo a2}
  }
  // ---- the step's own K / V row: rotate k, store both in the cache; they join the last tile from registers
  __half newk0 = __half(0.f), newk1 = __half(0.f), newv = __half(0.f);
  int nk0 = 0, nk1 = 0;
  if (owns_new) {
    const uint32_t row = (np - 1u) % a.kv_len;
    if (gtid < HD / 2) {
      nk0 = a.neox ? gtid : 2 * gtid, nk1 = a.neox ? gtid + HD / 2 : 2 * gtid + 1;
      const float x0 = __ldcg(k_new + nk0), x1 = __ldcg(k_new + nk1), c = __ldg(cs + gtid), sv = __ldg(sn + gtid);
      newk0 = __half(rope_lo(x0, x1, c, sv)), newk1 = __half(rope_hi(x0, x1, c, sv));
      __half *dst = const_cast<__half *>(kh) + (size_t)row * HD;
      dst[nk0] = newk0, dst[nk1] = newk1;
    }
    if (gtid < HD) {
      newv = __half(__ldcg(v_new + gtid));
      const_cast<__half *>(vh)[(size_t)row * HD + gtid] = newv;
    }
  }

  float o[HD / 8][4], run_m = -INFINITY, run_l = 0.0f;  // O^T C fragments: o[n][0..1] = head hq, dims 8n + 2tq, + 1
#pragma unroll
  for (int n = 0; n < HD / 8; n++)
#pragma unroll
    for (int e = 0; e < 4; e++) o[n][e] = 0.0f;
  const int lm = lane >> 3, lr = lane & 7;
  for (uint32_t it = 0; it < n_tiles; it++) {
    const int buf = it % SK_NB;
    const uint32_t tile_lo = p_lo + it * SK_TILE;
    if (owns_new && it + 1u == n_tiles) {  // nobody else writes this row of the buffer
      const uint32_t pr = np - 1u - tile_lo;
      if (gtid < HD / 2) {
        __half *dk = kbuf + buf * TILE_ELEMS + pr * ROW;
        dk[nk0] = newk0, dk[nk1] = newk1;
      }
      if (gtid < HD) vbuf[buf * TILE_ELEMS + pr * ROW + gtid] = newv;
    }
    cp_async_wait<SK_NB - 2>();
    group_sync(bar_id);  // tile `it` (and, the first time, the q fragments) complete; tile it - 1 may be refilled
    issue(it + SK_NB - 1u);
    const uint32_t valid = p_hi - tile_lo;
    const int p0 = warp * 16;
    if ((uint32_t)p0 < valid) {
      const __half *kt = kbuf + buf * TILE_ELEMS, *vt = vbuf + buf * TILE_ELEMS;
      float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int k = 0; k < KS; k++) {
        uint32_t kb[4];
        ldsm4(kb, kt + (p0 + (lm >> 1) * 8 + lr) * ROW + 16 * k + (lm & 1) * 8);
        const uint4 qf = qsm[k * 32 + lane];
        mma_f16(sa, qf.x, 0u, qf.y, 0u, kb[0], kb[1]);
        mma_f16(sa, qf.z, 0u, qf.w, 0u, kb[0], kb[1]);
        mma_f16(sb, qf.x, 0u, qf.y, 0u, kb[2], kb[3]);
        mma_f16(sb, qf.z, 0u, qf.w, 0u, kb[2], kb[3]);
      }
      float sc[4];
      sc[0] = (uint32_t)(p0 + 2 * tq) < valid ? sa[0] * scale : -INFINITY;
      sc[1] = (uint32_t)(p0 + 2 * tq + 1) < valid ? sa[1] * scale : -INFINITY;
      sc[2] = (uint32_t)(p0 + 8 + 2 * tq) < valid ? sb[0] * scale : -INFINITY;
      sc[3] = (uint32_t)(p0 + 8 + 2 * tq + 1) < valid ? sb[1] * scale : -INFINITY;
      float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
      const float m_new = fmaxf(run_m, mx), al = expf(run_m - m_new);  // position p0 exists: m_new is finite
      float pv[4], sum = 0.0f;
#pragma unroll
      for (int e = 0; e < 4; e++) pv[e] = expf(sc[e] - m_new), sum += pv[e];
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
      run_l = run_l * al + sum, run_m = m_new;
      uint32_t phh[2], pll[2];
      split2(pv[0], pv[1], phh[0], pll[0]);
      split2(pv[2], pv[3], phh[1], pll[1]);
#pragma unroll
      for (int u = 0; u < HD / 16; u++) {
        uint32_t vb[4];
        ldsm4t(vb, vt + (p0 + (lm & 1) * 8 + lr) * ROW + 16 * u + (lm >> 1) * 8);
#pragma unroll
        for (int e = 0; e < 4; e++) o[2 * u][e] *= al, o[2 * u + 1][e] *= al;
        mma_f16(o[2 * u], phh[0], 0u, phh[1], 0u, vb[0], vb[1]);
        mma_f16(o[2 * u], pll[0], 0u, pll[1], 0u, vb[0], vb[1]);
        mma_f16(o[2 * u + 1], phh[0], 0u, phh[1], 0u, vb[2], vb[3]);
        mma_f16(o[2 * u + 1], pll[0], 0u, pll[1], 0u, vb[2], vb[3]);
      }
    }
  }
  cp_async_wait<0>();
  group_sync(bar_id);

  // ---- merge the four warps' (max, sum, output) in shared memory (reusing the tile buffers), write the record
  float *red = reinterpret_cast<float *>(gsm);  // [4][8][HD]
  float *ml = red + SK_GW * 8 * HD;              // [4][8][2]
  if ((uint32_t)hq < G) {
#pragma unroll
    for (int n = 0; n < HD / 8; n++) *reinterpret_cast<float2 *>(red + (warp * 8 + hq) * HD + 8 * n + 2 * tq) = make_float2(o[n][0], o[n][1]);
    if (tq == 0) ml[(warp * 8 + hq) * 2] = run_m, ml[(warp * 8 + hq) * 2 + 1] = run_l;
  }
  group_sync(bar_id);
  const size_t rec = HD + 2;
  for (uint32_t e = gtid; e < G * HD; e += SK_GT) {
    const uint32_t h = e / HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < SK_GW; w++) M = fmaxf(M, ml[(w * 8 + h) * 2]);
    float L = 0.0f, acc = 0.0f;
#pragma unroll
    for (int w = 0; w < SK_GW; w++) {
      const float wk = expf(ml[(w * 8 + h) * 2] - M);  // a warp without positions has max -inf: weight 0
      L = fmaf(wk, ml[(w * 8 + h) * 2 + 1], L);
      acc = fmaf(wk, red[(w * 8 + h) * HD + (e % HD)], acc);
    }
    float *pr = a.part + (((size_t)g * G + h) * a.smax + s) * rec;
    pr[2 + (e % HD)] = acc;
    if (e % HD == 0) pr[0] = M, pr[1] = L;
  }
  group_sync(bar_id);  // the buffers are free for the group's next item
}

// One warp per head: the A records of the head -> out[hd] = sum_k w_k o_k / sum_k w_k l_k, w_k = exp(m_k - max m),
// and the Q8 copy (a head's dims are whole Q8 blocks of the output vector). Lane l holds dims l, l + 32, ...
template <int HD>
__device__ __forceinline__ void sk_merge_head(const StepArgs &a, const StepPhase &ph, uint32_t head, uint32_t A, int lane) {
  constexpr int DPL = HD / 32;
  const size_t rec = HD + 2;
  const float *pr = a.part + (size_t)head * a.smax * rec;
  // every load of the first eight splits goes out before anything is used: one trip to L2 for a short context
  float mk[2] = {-INFINITY, -INFINITY}, lk[2] = {0.0f, 0.0f};
#pragma unroll
  for (int j = 0; j < 2; j++) {
    const uint32_t k = lane + 32u * j;
    if (k < A) mk[j] = __ldcg(pr + k * rec), lk[j] = __ldcg(pr + k * rec + 1);
  }
  float v0[8][DPL];
#pragma unroll
  for (int j = 0; j < 8; j++)
#pragma unroll
    for (int d = 0; d < DPL; d++) v0[j][d] = (uint32_t)j < A ? __ldcg(pr + (size_t)j * rec + 2 + lane + 32 * d) : 0.0f;
  const float M = warp_max(fmaxf(mk[0], mk[1]));
  const float w0 = expf(mk[0] - M), w1 = expf(mk[1] - M);  // lane k holds the weight of split k (and k + 32)
  const float L = warp_sum_all(fmaf(w0, lk[0], w1 * lk[1]));
  float acc[DPL];
#pragma unroll
  for (int d = 0; d < DPL; d++) acc[d] = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const float wk = __shfl_sync(0xFFFFFFFFu, w0, j);
#pragma unroll
    for (int d = 0; d < DPL; d++) acc[d] = fmaf(wk, v0[j][d], acc[d]);  // a missing split: weight exp(-inf) = 0, value 0
  }
  for (uint32_t k0 = 8u; k0 < A; k0 += 4u) {
    float v[4][DPL];
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
      for (int d = 0; d < DPL; d++) v[j][d] = k0 + j < A ? __ldcg(pr + (size_t)(k0 + j) * rec + 2 + lane + 32 * d) : 0.0f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const uint32_t k = k0 + j;
      const float wk = __shfl_sync(0xFFFFFFFFu, k < 32u ? w0 : w1, k & 31u);
#pragma unroll
      for (int d = 0; d < DPL; d++) acc[d] = fmaf(wk, v[j][d], acc[d]);
    }
  }
  const float inv = 1.0f / L;
  const uint32_t nbq = a.n_head * HD / 32u;
#pragma unroll
  for (int d = 0; d < DPL; d++) {
    const float v = acc[d] * inv;
    ph.att[(size_t)head * HD + 32 * d + lane] = v;
    if (ph.attq) quant_block_warp(v, ph.attq, nbq, head * DPL + d, lane);
  }
}

// ---- the kernel --------------------------------------------------------------------------------------------------
// KSET: the matrix kinds of the model's GEMVs the instantiation carries code for: 0 Q4_0, 1 Q4_K + Q6_K, 2 all three.
template <int HD, int KSET>
__global__ void __launch_bounds__(SK_THREADS, 1) step_kernel(const __grid_constant__ StepArgs a) {
  extern __shared__ uint4 smem_sk[];
  __shared__ float red[SK_WARPS];
  __shared__ uint32_t s_ok;
  __shared__ float s_mx[SK_WARPS], s_sum[SK_WARPS];
  __shared__ uint32_t s_idx[SK_WARPS];
  __shared__ StepPhase s_ph[2];  // the phase being executed and the next one (fetched while this one runs)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    const uint32_t aborted = *(volatile uint32_t *)(a.bar + 1);
    if (aborted) atomicCAS(a.err, 0u, 4u);  // the abort flag is up (an earlier launch gave up, or the host raised it): report, do nothing
    s_ok = (!aborted && *(volatile uint32_t *)a.err == 0u) ? 1u : 0u;
  }
  __syncthreads();
  if (!s_ok) return;
  SkBar bar = {a.bar, a.bar + 1, a.err, 0u, a.wait_ns, blockIdx.x == 0 ? a.trace : nullptr, ar_now()};
  uint32_t ep = 0u;  // tensor parallel: the epoch of the last exchange
  if (a.push.world > 1u) ep = __ldcg(a.push.epoch);

  constexpr uint32_t PH_WORDS = sizeof(StepPhase) / 8u;
  if (threadIdx.x < PH_WORDS) reinterpret_cast<uint64_t *>(&s_ph[0])[threadIdx.x] = reinterpret_cast<const uint64_t *>(a.prog)[threadIdx.x];
  uint32_t cur = 0u;
  for (uint32_t step = 0; step < a.n_steps; step++) {
    for (uint32_t p = 0; p < a.n_phases; p++, cur ^= 1u) {
      __syncthreads();  // the record of phase p is in s_ph[cur]; nobody still reads the previous phase's staged activations
      // the next phase's record travels from global memory while this phase runs
      const uint32_t pn = p + 1u < a.n_phases ? p + 1u : 0u;
      uint64_t nxt_word = 0ull;
      if (threadIdx.x < PH_WORDS) nxt_word = reinterpret_cast<const uint64_t *>(a.prog + pn)[threadIdx.x];
      const StepPhase &ph = s_ph[cur];
      const int32_t ph_kind = ph.kind, ph_nobar = ph.nobar;
      // the head of a matrix that a later phase streams, into L2 while this phase runs (the attention phase leaves that to its idle groups)
      if ((a.knobs & 2u) && ph.pf && ph_kind != PH_ATTN) prefetch_part(ph.pf, ph.pf_bytes, blockIdx.x, gridDim.x, threadIdx.x, SK_THREADS);
      switch (ph_kind) {
        case PH_EMBED: {
          if (blockIdx.x == 0) {
            const uint32_t tok = ld_cg_u32(a.scalars);
            if (a.emb_kind == IE_B200_MAT_Q4) {
              const uint32_t nb = a.dim / 32u;
              const uint8_t *rp = a.emb + (size_t)tok * row_bytes_of(IE_B200_MAT_Q4, a.dim);
              for (uint32_t e = threadIdx.x; e < a.dim; e += SK_THREADS) {
                const uint32_t b = e >> 5, j = e & 31u;
                const uint32_t word = reinterpret_cast<const uint32_t *>(rp + 16u * (size_t)b)[(j & 15u) >> 2];
                const uint32_t nib = (word >> (8u * (j & 3u) + 4u * (j >> 4))) & 15u;
                const float d = h2f(reinterpret_cast<const uint16_t *>(rp + 16u * (size_t)nb)[b]);
                a.x[e] = __fmul_rn(d, (float)((int)nib - 8));
              }
            } else {
              const float *rp = reinterpret_cast<const float *>(a.emb) + (size_t)tok * a.dim;
              for (uint32_t e = threadIdx.x; e < a.dim; e += SK_THREADS) a.x[e] = rp[e];
            }
          }
          break;
        }
        case PH_GEMV: {
          const uint32_t nb = ph.nb;
          const bool tr = bar.trace != nullptr && threadIdx.x == 0;
          const uint64_t tg0 = tr ? ar_now() : 0ull;
          uint4 *A0 = smem_sk, *A1 = smem_sk + nb;
          float *da = reinterpret_cast<float *>(smem_sk + 2u * nb);
          int *as = reinterpret_cast<int *>(da + nb);
          if (ph.pro == PRO_Q8) {
            ActSrc src = {};
            src.xq = static_cast<const uint8_t *>(ph.src);
            stage_activations<false, SK_WARPS>(src, nb, A0, A1, da, as, red, false, [] { __syncthreads(); });
          } else if (ph.pro == PRO_NORM) {
            ActSrc src = {};
            src.xf = static_cast<const float *>(ph.src), src.norm_w = ph.norm_w, src.eps = a.eps;
            stage_activations<true, SK_WARPS>(src, nb, A0, A1, da, as, red, false, [] { __syncthreads(); });
          } else if (ph.pro == PRO_SWIGLU) {
            sk_stage_swiglu(static_cast<const float *>(ph.src), nb, A0, A1, da, as);
            __syncthreads();
          } else if (ph.pro == PRO_QUANT) {
            sk_stage_quant(static_cast<const float *>(ph.src), nb, A0, A1, da, as);
            __syncthreads();
          }
          if (ph.push) ep++;
          const uint64_t tg1 = tr ? ar_now() : 0ull;
          // rows per group x lane steps per chunk = 16-byte loads a lane keeps in flight: 16 for Q4_0 (4 rows x 4 steps), 8 for
          // the K kinds (8 registers per block). One instantiation per kind: rows longer than 128 blocks loop over chunks (their
          // later chunks are in L2 by then: whole rows are asked for ahead).
          if (KSET != 1 && ph.mkind == IE_B200_MAT_Q4) sk_gemv<IE_B200_MAT_Q4, 4, 4>(ph, a, A0, A1, da, as, warp, lane, ep);
          else if (KSET != 0 && ph.mkind == IE_B200_MAT_Q4K) sk_gemv<IE_B200_MAT_Q4K, 2, 4>(ph, a, A0, A1, da, as, warp, lane, ep);
          else if (KSET != 0 && ph.mkind == IE_B200_MAT_Q6K) sk_gemv<IE_B200_MAT_Q6K, 2, 4>(ph, a, A0, A1, da, as, warp, lane, ep);
          if (tr) {  // slots 8 + prologue kind: {prologue ns, rows loop ns of warp 0, phases}
            const uint64_t tg2 = ar_now();
            unsigned long long *t = bar.trace + 3 * (8 + (ph.pro == PRO_QUANT ? PRO_SWIGLU : ph.pro));
            t[0] += tg1 - tg0, t[1] += tg2 - tg1, t[2] += 1ull;
          }
          break;
        }
        case PH_ATTN: {
          const uint32_t np = ld_cg_u32(a.scalars + a.Tm + 1u) + 1u;
          uint32_t span, A;
          sk_splits(np, a.smax, span, A);
          {
            const int grp = warp / SK_GW;
            uint8_t *gsm = reinterpret_cast<uint8_t *>(smem_sk) + (size_t)grp * SkAttnSmem<HD>::BYTES;
            const uint32_t n_items = a.n_kv * A, n_slots = gridDim.x * SK_GROUPS;
            const uint32_t first = (uint32_t)grp * gridDim.x + blockIdx.x;
            // a group without an item pulls its share of the next matrix into L2 instead (most groups, at a short context)
            if ((a.knobs & 2u) && first >= n_items && ph.pf)
              prefetch_part(ph.pf, ph.pf_bytes, blockIdx.x * SK_GROUPS + grp, gridDim.x * SK_GROUPS, threadIdx.x - grp * SK_GT, SK_GT);
            for (uint32_t item = first; item < n_items; item += n_slots)
              sk_attn_item<HD>(a, ph, item % a.n_kv, item / a.n_kv, A, span, np, gsm, threadIdx.x - grp * SK_GT, 1 + grp);
          }
          break;
        }
        case PH_MERGE: {
          const uint32_t np = ld_cg_u32(a.scalars + a.Tm + 1u) + 1u;
          uint32_t span, A;
          sk_splits(np, a.smax, span, A);
          const uint32_t W = gridDim.x * SK_WARPS;
          for (uint32_t head = (uint32_t)warp * gridDim.x + blockIdx.x; head < a.n_head; head += W) sk_merge_head<HD>(a, ph, head, A, lane);
          break;
        }
        case PH_ARGMAX: {
          const uint32_t n = a.n_logits, per = (n + gridDim.x - 1u) / gridDim.x, lo = blockIdx.x * per, hi = min(n, lo + per);
          float mx = -INFINITY;
          uint32_t idx = 0xFFFFFFFFu;
          for (uint32_t i = lo + threadIdx.x; i < hi; i += SK_THREADS) {
            const float v = __ldcg(a.logits + i);
            if (v > mx) mx = v, idx = i;  // i rises per thread: keeps the first maximum
          }
          for (int o = 16; o; o >>= 1) {
            const float om = __shfl_xor_sync(0xFFFFFFFFu, mx, o);
            const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, idx, o);
            if (om > mx || (om == mx && oi < idx)) mx = om, idx = oi;
          }
          if (lane == 0) s_mx[warp] = mx, s_idx[warp] = idx;
          __syncthreads();
          float bm = s_mx[0];
          uint32_t bi = s_idx[0];
          for (int k = 1; k < SK_WARPS; k++)
            if (s_mx[k] > bm || (s_mx[k] == bm && s_idx[k] < bi)) bm = s_mx[k], bi = s_idx[k];
          float sum = 0.0f;
          for (uint32_t i = lo + threadIdx.x; i < hi; i += SK_THREADS) sum += expf(__ldcg(a.logits + i) - bm);
          sum = warp_sum_all(sum);
          if (lane == 0) s_sum[warp] = sum;
          __syncthreads();
          if (threadIdx.x == 0) {
            float tot = 0.0f;
            for (int k = 0; k < SK_WARPS; k++) tot += s_sum[k];
            SkArgPart rec = {bm, bi, tot, 0u};
            static_cast<SkArgPart *>(a.amax_part)[blockIdx.x] = rec;
          }
          break;
        }
        case PH_FINISH:
        case PH_XARGMAX: {
          if (ph_kind == PH_XARGMAX) ep++;
          if (blockIdx.x == 0 && warp == 0) {
            const SkArgPart *part = static_cast<const SkArgPart *>(a.amax_part);
            float mx = -INFINITY, sum = 0.0f;
            uint32_t idx = 0xFFFFFFFFu;
            for (uint32_t k = lane; k < gridDim.x; k += 32u) {
              SkArgPart q;
              const uint4 raw = __ldcg(reinterpret_cast<const uint4 *>(part + k));
              q.mx = __uint_as_float(raw.x), q.idx = raw.y, q.sum = __uint_as_float(raw.z);
              if (q.idx == 0xFFFFFFFFu) continue;
              if (q.mx > mx || (q.mx == mx && q.idx < idx)) {
                sum = sum * expf(mx - q.mx) + q.sum;
                mx = q.mx, idx = q.idx;
              } else {
                sum += q.sum * expf(q.mx - mx);
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
            uint32_t win = idx == 0xFFFFFFFFu ? 0u : idx;
            float prob = sum > 0.0f ? 1.0f / sum : 0.0f;
            if (ph_kind == PH_XARGMAX) {
              // every rank's (logit, global index, probability within its slice) to every rank; the largest logit wins,
              // ties go to the smaller index; the denominators add up relative to the winner
              const uint32_t par = ep & 1u, world = a.push.world, rank = a.push.rank;
              if ((uint32_t)lane < world && (uint32_t)lane != rank) {
                unsigned long long *dst = a.push.ll[lane] + ((size_t)par * world + rank) * a.push.max_n;
                ll_store(dst, ep, __float_as_uint(mx));
                ll_store(dst + 1, ep, win + a.vocab_off);
                ll_store(dst + 2, ep, __float_as_uint(prob));
                ll_store(dst + 3, ep, 0u);
              }
              float v = -INFINITY, pr = 0.0f;
              uint32_t gi = 0xFFFFFFFFu;
              bool gave_up = false;
              if ((uint32_t)lane == rank) {
                v = mx, gi = win + a.vocab_off, pr = prob;
              } else if ((uint32_t)lane < world) {
                uint32_t wv[4];
                const unsigned long long *src = a.push.ll[rank] + ((size_t)par * world + lane) * a.push.max_n;
                const uint64_t t0 = ar_now();
                for (;;) {
                  unsigned long long w4[4];
#pragma unroll
                  for (int c = 0; c < 4; c++) w4[c] = ll_load(src + c);
                  bool all = true;
#pragma unroll
                  for (int c = 0; c < 4; c++) all = all && (uint32_t)(w4[c] >> 32) == ep, wv[c] = (uint32_t)w4[c];
                  if (all) break;
                  if (*(volatile uint32_t *)(a.bar + 1) || ar_now() - t0 > a.wait_ns) {
                    gave_up = true;
                    break;
                  }
                }
                if (!gave_up) v = __uint_as_float(wv[0]), gi = wv[1], pr = __uint_as_float(wv[2]);
              }
              if (gave_up) {
                atomicExch(a.err, 3u);
                *(volatile uint32_t *)(a.bar + 1) = 1u;
              }
              float bv = v;
              uint32_t bi = gi;
              for (int o = 16; o; o >>= 1) {
                const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
                const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
              }
              float den = pr > 0.0f ? expf(v - bv) / pr : 0.0f;
              den = warp_sum_all(den);
              win = bi, prob = den > 0.0f ? 1.0f / den : 0.0f;
            }
            if (lane == 0) {
              a.result[0] = win, a.result[1] = __float_as_uint(prob);
              const uint32_t c = ld_cg_u32(a.hist + a.hist_cap);
              a.hist[c % a.hist_cap] = win;
              a.hist[a.hist_cap] = c + 1u;
              a.scalars[0] = win;
              a.scalars[a.Tm] = ld_cg_u32(a.scalars + a.Tm) + 1u;
            }
            for (uint32_t t = lane; t < a.Tm; t += 32u) a.scalars[a.Tm + 1u + t] = ld_cg_u32(a.scalars + a.Tm + 1u + t) + 1u;
          }
          break;
        }
        case PH_REDUCE: {
          // rows of 32 per warp: poll every rank's slot of the row (the own rank's included), add in rank order onto x
          const uint32_t par = ep & 1u, world = a.push.world, W = gridDim.x * SK_WARPS;
          const unsigned long long *my = a.push.ll[a.push.rank] + (size_t)par * world * a.push.max_n;
          bool gave_up = false;
          for (uint32_t r0 = ((uint32_t)warp * gridDim.x + blockIdx.x) * 32u; r0 < ph.rows; r0 += W * 32u) {
            const uint32_t r = r0 + lane;
            if (r >= ph.rows) continue;
            float acc = __ldcg(ph.res + r);
            unsigned long long v[AR_MAX_RANKS];
            const uint64_t t0 = ar_now();
            for (;;) {
              bool all = true;
#pragma unroll
              for (int j = 0; j < AR_MAX_RANKS; j++)
                if ((uint32_t)j < world) v[j] = ll_load(my + (size_t)j * a.push.max_n + r);
#pragma unroll
              for (int j = 0; j < AR_MAX_RANKS; j++)
                if ((uint32_t)j < world) all = all && (uint32_t)(v[j] >> 32) == ep;
              if (all) break;
              if (gave_up || *(volatile uint32_t *)(a.bar + 1) || ar_now() - t0 > a.wait_ns) {
                gave_up = true;
                break;
              }
            }
#pragma unroll
            for (int j = 0; j < AR_MAX_RANKS; j++)
              if ((uint32_t)j < world) acc = __fadd_rn(acc, __uint_as_float((uint32_t)v[j]));
            ph.y[r] = acc;
          }
          if (gave_up) {
            atomicExch(a.err, 3u);
            *(volatile uint32_t *)(a.bar + 1) = 1u;
          }
          break;
        }
        default: break;
      }
      if (threadIdx.x < PH_WORDS) reinterpret_cast<uint64_t *>(&s_ph[cur ^ 1u])[threadIdx.x] = nxt_word;
      if (!ph_nobar) {
        // ask for what the next phase streams first, then arrive: the weights are on their way while the CTAs gather
        __syncthreads();
        if ((p + 1u < a.n_phases || step + 1u < a.n_steps) && s_ph[cur ^ 1u].kind == PH_GEMV) sk_gemv_prefetch(s_ph[cur ^ 1u], warp, lane);
        if (!grid_sync(bar, &s_ok, ph_kind)) return;
      }
    }
  }
  if (a.push.world > 1u && blockIdx.x == 0 && threadIdx.x == 0) *a.push.epoch = ep;
}

static size_t sk_smem_bytes(uint32_t hd) {
  const size_t attn = (size_t)SK_GROUPS * (hd == 64 ? SkAttnSmem<64>::BYTES : SkAttnSmem<128>::BYTES);
  const size_t gemv = 1024u * 40u;
  return attn > gemv ? attn : gemv;
}

bool step_kernel_supports(uint32_t hd, uint32_t n_head, uint32_t n_kv, int kv_f32) {
  return !kv_f32 && (hd == 64 || hd == 128) && n_kv && n_head % n_kv == 0 && n_head / n_kv <= 8;
}

uint32_t step_kernel_smax(uint32_t n_kv) {
  const uint32_t slots = (uint32_t)sm_count() * SK_GROUPS;
  const uint32_t s = slots / (n_kv ? n_kv : 1u);
  return s < 1u ? 1u : (s > 64u ? 64u : s);
}

size_t step_kernel_amax_bytes() { return (size_t)sm_count() * sizeof(SkArgPart); }

int step_kernel_launch(const StepArgs &a, uint32_t hd, int kset, cudaStream_t st) {
  const void *k = nullptr;
  if (hd == 64) k = kset == 0 ? reinterpret_cast<const void *>(step_kernel<64, 0>) : kset == 1 ? reinterpret_cast<const void *>(step_kernel<64, 1>) : reinterpret_cast<const void *>(step_kernel<64, 2>);
  else k = kset == 0 ? reinterpret_cast<const void *>(step_kernel<128, 0>) : kset == 1 ? reinterpret_cast<const void *>(step_kernel<128, 1>) : reinterpret_cast<const void *>(step_kernel<128, 2>);
  const size_t smem = sk_smem_bytes(hd);
  if (int r = ensure_dynamic_smem(k, smem)) return r;
  static thread_local int coop_dev = -1, coop = 0;
  int dev = 0;
  IEB_CUDA(cudaGetDevice(&dev));
  if (dev != coop_dev) {
    IEB_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    coop_dev = dev;
  }
  if (!coop) return fail(IE_B200_E_CUDA, "the device does not support cooperative launches (the step kernel's CTAs wait for one another)");
  IEB_CUDA(cudaMemsetAsync(a.bar, 0, 4, st));  // the arrival counter; the abort flag (bar[1]) stays as it is
  StepArgs args = a;
  void *params[] = {&args};
  const cudaError_t e = cudaLaunchCooperativeKernel(k, dim3((unsigned)sm_count()), dim3(SK_THREADS), params, smem, st);
  count_launch();
  if (e != cudaSuccess) return cuda_fail(e, "step_kernel");
  return IE_B200_OK;
}

}  // namespace ieb

using namespace ieb;

// The attention phases of the persistent kernel as a call of their own: what the kernel runs per layer (RoPE, KV
// store, split attention by groups of four warps, merge by one warp per head), on caller-provided buffers.
extern "C" size_t ie_b200_attn_persistent_scratch_bytes(uint32_t n_head, uint32_t n_kv, uint32_t hd) {
  return 2 * sizeof(StepPhase) + 32 + (size_t)n_head * step_kernel_smax(n_kv) * (hd + 2u) * sizeof(float);
}

extern "C" int ie_b200_attn_persistent(const float *d_qkv, void *d_kc, void *d_vc, const float *d_cos, const float *d_sin, float *d_out, void *d_oq,
                                       const uint32_t *d_pos, uint32_t n_head, uint32_t n_kv, uint32_t hd, int neox, uint32_t kv_len, void *d_scratch,
                                       uint32_t *d_err, void *stream) {
  if (!d_qkv || !d_kc || !d_vc || !d_cos || !d_sin || !d_out || !d_pos || !d_scratch || !d_err) return fail(IE_B200_E_ARG, "ie_b200_attn_persistent: NULL pointer");
  if (!step_kernel_supports(hd, n_head, n_kv, 0)) return fail(IE_B200_E_SIZE, "ie_b200_attn_persistent: heads of 64 or 128, at most 8 query heads per KV head");
  if (!aligned16(d_kc) || !aligned16(d_vc) || !aligned16(d_qkv) || !aligned16(d_scratch)) return fail(IE_B200_E_ARG, "ie_b200_attn_persistent: 16-byte alignment");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  StepPhase ph[2] = {};
  ph[0].kind = PH_ATTN, ph[0].q = d_qkv, ph[0].kc = d_kc, ph[0].vc = d_vc;
  ph[1].kind = PH_MERGE, ph[1].att = d_out, ph[1].attq = static_cast<uint8_t *>(d_oq);
  char *sc = static_cast<char *>(d_scratch);
  IEB_CUDA(cudaMemcpyAsync(sc, ph, sizeof ph, cudaMemcpyHostToDevice, st));
  IEB_CUDA(cudaMemsetAsync(sc + sizeof ph, 0, 32, st));
  StepArgs a = {};
  a.prog = reinterpret_cast<const StepPhase *>(sc), a.n_phases = 2, a.n_steps = 1;
  a.scalars = const_cast<uint32_t *>(d_pos) - 1, a.Tm = 0;  // the kernel reads the position at scalars[Tm + 1]
  a.bar = reinterpret_cast<uint32_t *>(sc + sizeof ph), a.err = d_err;
  a.n_head = n_head, a.n_kv = n_kv, a.kv_len = kv_len, a.neox = neox ? 1u : 0u, a.cs = d_cos, a.sn = d_sin;
  a.part = reinterpret_cast<float *>(sc + sizeof ph + 32), a.smax = step_kernel_smax(n_kv);
  a.wait_ns = AR_WAIT_NS;
  return step_kernel_launch(a, hd, 0, st);
}
