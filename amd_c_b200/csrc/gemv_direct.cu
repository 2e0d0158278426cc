// gemv_direct.cu -- the decode (one token) GEMV that streams weights straight
// from HBM into registers, launched with programmatic dependent launch.
//
// Every warp of a persistent grid (exactly the resident CTAs: three of eight
// warps per SM at 80 registers) takes row pairs round-robin (pair g, g + W, ...
// for W warps in the grid); lane l takes blocks l, l+32, ... of its rows, so
// each lane keeps up to 8 16-byte loads in flight (16 in the one-row-per-warp
// variant for long rows). The first loads of a warp are issued BEFORE the
// kernel waits for its predecessor (the weights do not depend on it): the
// launch latency, the DRAM latency and the predecessor's tail overlap with
// weight traffic that is already on its way. Only then are the activations
// staged (optionally computed: fused RMSNorm + Q8, see act_stage.cuh) and
// consumed. Optional tails: RMSNorm + Q8 of the finished vector by the last CTA
// to arrive; tensor parallel: every finished row pair also stored into the
// other ranks' slots (peer_ll.cuh).
//
// Arithmetic and order are the reference's (one warp per row, blocks
// l, l+32, ... in order, shuffle-down tree): bit-exact with its CPU GEMV.
#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "act_stage.cuh"
#include "common.cuh"
#include "gemv_blocks.cuh"
#include "peer_ll.cuh"

namespace ieb {

constexpr int GD_WARPS = 8, GD_THREADS = GD_WARPS * 32;

struct GdArgs {
  const uint8_t *w;
  size_t rowb;
  uint32_t rows, nb;
  ActSrc act;
  float *y;
  const float *bias, *res;
  // norm tail (optional): once every CTA has written its rows, the last CTA to finish computes
  // tail.xn_out = rmsnorm(y) * tail.norm_w and its Q8 copy tail.xq_out for the next GEMV
  ActSrc tail;        // tail.norm_w == NULL: no tail
  uint32_t late;      // let dependents start only after this kernel's own dependency wait (LaunchHints::late_trigger)
  uint32_t *work;     // two words, zero between launches; word 1 counts the CTAs that have finished (norm tail only)
  ArPush push;        // TP kernels only: every finished row also goes to the other ranks' slots
  float *swi_h;       // SwiGLU kernels only (LaunchHints::swi_h): outputs, their Q8 copy, arrival counters per 32 outputs
  uint8_t *swi_q;
  uint32_t *swi_count;
};

// R rows of one warp, U lane steps (blocks l, l+32, ... of each row) per chunk: R x U 16-byte loads per lane
// are issued before any of them is consumed.
template <int KIND, int R, int U>
__device__ __forceinline__ void gd_load(Blk<KIND, false> (&blk)[R][U], const uint8_t *w, size_t rowb, uint32_t r, uint32_t r_hi, uint32_t c,
                                        uint32_t nb, int lane) {
#pragma unroll
  for (int u = 0; u < U; u++) {
    const uint32_t b = c + 32u * u + lane;
    if (b < nb) {
#pragma unroll
      for (int i = 0; i < R; i++)
        if (r + i < r_hi) blk[i][u].load(w + (size_t)(r + i) * rowb, b, nb);
    }
  }
}

// MODE: 0 plain; 1 tensor-parallel partial (rows also stored to the peers); 2 SwiGLU (R = 2: a warp's row pair is (gate_i,
// up_i), it writes silu(gate) * up and the warp that completes 32 outputs writes their Q8 block).
template <int KIND, bool NORM, int R, int U, int MINB, int MODE>
__global__ void __launch_bounds__(GD_THREADS, MINB) gemv_direct_kernel(const GdArgs a) {
  constexpr bool TP = MODE == 1, SWI = MODE == 2;
  static_assert(!SWI || R == 2, "a gate / up pair per warp");
  extern __shared__ uint4 smem_gd[];
  const uint32_t nb = a.nb;
  uint4 *A0 = smem_gd, *A1 = smem_gd + nb;
  float *da = reinterpret_cast<float *>(smem_gd + 2u * nb);
  int *as = reinterpret_cast<int *>(da + nb);
  __shared__ float red[GD_WARPS];
  __shared__ uint32_t last;

  tl_mark(TL_GEMV, 0);
  if (!a.late) pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // Row groups of R are dealt round-robin over all warps of the grid, so at any moment the grid reads one
  // contiguous window. (Handing groups out through a device counter was tried: one atomic per group on one
  // address serialises in L2 and halved the bandwidth on large matrices.)
  const uint32_t W = gridDim.x * GD_WARPS, groups = (a.rows + R - 1u) / R, r_hi = a.rows;
  uint32_t grp = blockIdx.x * GD_WARPS + warp;

  Blk<KIND, false> first[R][U];
  if (grp < groups) gd_load<KIND, R, U>(first, a.w, a.rowb, grp * R, r_hi, 0u, nb, lane);

  // the norm weights (a constant vector) into L2 while waiting: the norm after the wait then pays one L2 round trip
  if (NORM) {
    for (uint32_t i = 32u * threadIdx.x; i < 32u * nb; i += 32u * GD_THREADS) prefetch_l2(a.act.norm_w + i);
  } else if (a.tail.norm_w && blockIdx.x == 0) {
    for (uint32_t i = 32u * threadIdx.x; i < a.rows; i += 32u * GD_THREADS) prefetch_l2(a.tail.norm_w + i);
  }
  tl_mark(TL_GEMV, 2);
  pdl_wait();
  if (a.late) pdl_launch_dependents();
  tl_mark(TL_GEMV, 1);
  uint32_t ep = 0u;  // TP: the epoch of this exchange (the previous one is complete: its kernel is)
  if (TP) ep = *(volatile uint32_t *)a.push.epoch + 1u;
  stage_activations<NORM, GD_WARPS>(a.act, nb, A0, A1, da, as, red, blockIdx.x == 0, [] { __syncthreads(); });
  tl_mark(TL_GEMV, 3);

  auto chunk = [&](const Blk<KIND, false>(&blk)[R][U], float(&acc)[R], uint32_t rr, uint32_t c) {
#pragma unroll
    for (int u = 0; u < U; u++) {
      const uint32_t b = c + 32u * u + lane;
      if (b < nb) {
        const uint4 a0 = A0[b], a1 = A1[b];
        const float d = da[b];
        const int s = as[b];
#pragma unroll
        for (int i = 0; i < R; i++)
          if (rr + i < r_hi) acc[i] = blk[i][u].accum(acc[i], a0, a1, d, s, b);
      }
    }
  };
  auto finish = [&](float(&acc)[R], uint32_t rr) {
    float v[R];
#pragma unroll
    for (int i = 0; i < R; i++) v[i] = warp_tree(acc[i]);
    if (SWI) {
      // rows rr, rr + 1 = gate and up of output rr / 2: the same arithmetic as the SwiGLU kernel, then one arrival per
      // output on the counter of its block of 32; whoever brings it to 32 quantises the block (and clears the counter)
      const uint32_t i = rr >> 1, blk = i >> 5;
      uint32_t prev = 0u;
      if (lane == 0) {
        const float g = v[0], h = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), v[R - 1]);
        a.swi_h[i] = h;
        __threadfence();
        prev = atomicAdd(a.swi_count + blk, 1u);
      }
      prev = __shfl_sync(0xFFFFFFFFu, prev, 0);
      if (prev == 31u) {
        __threadfence();
        const float hv = __ldcg(a.swi_h + 32u * blk + lane);
        quant_block_warp(hv, a.swi_q, a.rows / 64u, blk, lane);
        if (lane == 0) a.swi_count[blk] = 0u;
      }
      return;
    }
#pragma unroll
    for (int i = 0; i < R; i++) {
      if (lane == 0 && rr + i < r_hi) {
        float o = v[i];
        if (a.bias) o = __fadd_rn(o, a.bias[rr + i]);
        if (a.res) o = __fadd_rn(a.res[rr + i], o);
        a.y[rr + i] = o;
      }
    }
    if (TP) {
      // The rows go to every other rank right away (lane j stores to rank j), so the transfer overlaps the rest of the
      // GEMV; a warp's two adjacent rows travel as one 16-byte store (each half carries its own epoch). Collecting a
      // whole CTA's rows first (one 128-byte store per rank and round) was tried: the barrier it needs per round cost
      // the GEMV far more than the fewer packets saved.
#pragma unroll
      for (int i = 0; i < R; i++) v[i] = __shfl_sync(0xFFFFFFFFu, v[i], 0);
      if ((uint32_t)lane < a.push.world && (uint32_t)lane != a.push.rank) {
        unsigned long long *dst = a.push.ll[lane] + ((size_t)(ep & 1u) * a.push.world + a.push.rank) * a.push.max_n + rr;
        if (R == 2 && rr + 1 < r_hi) {
          ll_store2(dst, ep, __float_as_uint(v[0]), __float_as_uint(v[R - 1]));
        } else {
#pragma unroll
          for (int i = 0; i < R; i++)
            if (rr + i < r_hi) ll_store(dst + i, ep, __float_as_uint(v[i]));
        }
      }
    }
  };
  // one row group; PRE: its first chunk is already in `first`
  auto group = [&](uint32_t g, auto pre_tag) {
    constexpr bool PRE = decltype(pre_tag)::value;
    const uint32_t r = g * R;
    float acc[R];
#pragma unroll
    for (int i = 0; i < R; i++) acc[i] = 0.0f;
    if (PRE) chunk(first, acc, r, 0u);
    for (uint32_t c = PRE ? 32u * U : 0u; c < nb; c += 32u * U) {
      Blk<KIND, false> blk[R][U];
      gd_load<KIND, R, U>(blk, a.w, a.rowb, r, r_hi, c, nb, lane);
      chunk(blk, acc, r, c);
    }
    finish(acc, r);
  };
  if (grp < groups) {
    group(grp, std::true_type{});
    grp += W;
  }
  for (; grp < groups; grp += W) group(grp, std::false_type{});
  tl_mark(TL_GEMV, 4);
  if (a.work && a.tail.norm_w) {  // the norm tail: count arrivals, the last CTA normalises the finished vector
    __threadfence();  // this thread's rows are visible before the arrival is counted
    __syncthreads();
    if (threadIdx.x == 0) {
      last = atomicAdd(a.work + 1, 1u) == gridDim.x - 1u;
      if (last) a.work[0] = 0u, a.work[1] = 0u;
    }
    __syncthreads();
    if (last) {
      __threadfence();
      stage_activations<true, GD_WARPS>(a.tail, a.rows / 32u, nullptr, nullptr, nullptr, nullptr, red, true, [] { __syncthreads(); });
      if (threadIdx.x == 0) tl_mark_any(TL_GEMV, 5);
    }
  }
  tl_mark(TL_GEMV, 15);
  if (threadIdx.x == 0) tl_mark_any(TL_GEMV, 14);  // every CTA's exit (timeline builds)
}

template <int KIND, bool NORM, int R, int U, int MINB, int MODE>
static int launch_direct(const GdArgs &a, cudaStream_t st) {
  const size_t smem = (size_t)a.nb * 40u;
  auto k = gemv_direct_kernel<KIND, NORM, R, U, MINB, MODE>;
  if (int r = ensure_dynamic_smem(reinterpret_cast<const void *>(k), smem)) return r;
  // One group per warp up to a persistent grid of exactly the resident CTAs (MINB per SM), whose warps loop:
  // measured on B200, 3 per SM gives 6.45 TB/s on a 295 MB matrix, 8 per SM 5.98, 4 per SM (1.33 waves) 5.17.
  // (Shrinking the grid so that every warp gets the same number of groups -- 7168 groups over 2392 warps instead of
  // 3552, where 64 warps take a third one -- was tried: 6 % slower on 14336 x 4096, 3 % on the whole step; the
  // rounds are latency-bound and the extra warps help more than the ragged last round costs.)
  // (Four CTAs per SM at 64 registers, with 132 bytes of spills: 7 % faster on 14336 x 4096 alone, slower on the small
  // matrices and 1.5 % slower on the whole step.)
  const unsigned need = (a.rows + R * GD_WARPS - 1) / (R * GD_WARPS);
  unsigned grid = (unsigned)(sm_count() * MINB);
  if (grid > need) grid = need ? need : 1u;
  // (L2 bulk prefetches were tried three ways and all lost: the warp's own further rows ahead of the dependency wait,
  // 4 % slower per step; the weights of the first, second or third GEMV after this one, asked for by every CTA before
  // its own work, 5-7 % slower; the same from a side stream forked inside the step graph, which also broke the
  // programmatic-launch chain. Weights that come through L2 a little early do not stream faster than from HBM here.)
  IEB_LAUNCH_PDL("gemv_direct_kernel", k, dim3(grid), dim3(GD_THREADS), smem, st, a);
  return IE_B200_OK;
}

// Long rows with few of them (the FFN down projection: 4096 x 14336) are a chain of dependent chunks per warp at
// two rows per warp; one row per warp with the whole row's loads in flight at once (up to 16 lane steps, 2 CTAs
// per SM for the registers that takes) shortens the chain to one round trip per row.
template <int KIND, bool NORM, int MODE>
static int pick_direct(const GdArgs &a, cudaStream_t st) {
  constexpr int U2 = KIND == IE_B200_MAT_Q4 ? 4 : 2;
  static const int long_mode = [] {  // IE_B200_GEMV_LONG: 0 never, 1 (default) 16 lane steps at 2 CTAs/SM, 2: 8 lane steps at 3 CTAs/SM
    const char *v = getenv("IE_B200_GEMV_LONG");
    return v ? atoi(v) : 1;
  }();
  const bool few_long = MODE != 2 && long_mode && a.nb >= 256u && (uint64_t)a.rows * 2u <= (uint64_t)sm_count() * 3u * GD_WARPS * 4u;
  if (few_long && long_mode == 2) return launch_direct<KIND, NORM, 1, 2 * U2, 3, MODE == 2 ? 0 : MODE>(a, st);
  if (few_long) return launch_direct<KIND, NORM, 1, 4 * U2, 2, MODE == 2 ? 0 : MODE>(a, st);  // Q4_0: 16 lane steps = rows of up to 512 blocks in one chunk
  return launch_direct<KIND, NORM, 2, U2, 3, MODE>(a, st);
}

template <bool NORM, int MODE>
int dispatch_direct(int kind, const GdArgs &a, cudaStream_t st) {
  switch (kind) {
    case IE_B200_MAT_Q4: return pick_direct<IE_B200_MAT_Q4, NORM, MODE>(a, st);
    case IE_B200_MAT_Q4K: return pick_direct<IE_B200_MAT_Q4K, NORM, MODE>(a, st);
    case IE_B200_MAT_Q6K: return pick_direct<IE_B200_MAT_Q6K, NORM, MODE>(a, st);
    default: return fail(IE_B200_E_ARG, "gemv_direct: matrix kind %d has no streaming kernel", kind);
  }
}

// Entry used by gemv_stream.cu's dispatcher.
int gemv_direct(int kind, const void *d_w, uint32_t rows, uint32_t cols, const ActSrc &act, bool norm, float *d_y, const float *d_bias,
                const float *d_res, const ActSrc *tail, uint32_t *work, cudaStream_t st, const ArPush *push) {
  GdArgs a = {};
  const LaunchHints hints = take_hints();
  a.late = hints.late_trigger ? 1u : 0u;
  a.w = static_cast<const uint8_t *>(d_w), a.rowb = row_bytes_of(kind, cols), a.rows = rows, a.nb = cols / 32u;
  a.act = act, a.y = d_y, a.bias = d_bias, a.res = d_res;
  a.work = work;
  if (tail) a.tail = *tail, a.tail.xf = d_y;
  if (push) {
    if (norm || tail || d_bias || d_res) return fail(IE_B200_E_ARG, "gemv_direct: a tensor-parallel partial takes no norm, bias or residual");
    a.push = *push;
    return dispatch_direct<false, 1>(kind, a, st);
  }
  if (hints.swi_h) {
    if (norm || tail || d_bias || d_res || !hints.swi_q || !hints.swi_count || rows % 64u)
      return fail(IE_B200_E_ARG, "gemv_direct: the SwiGLU form takes interleaved gate / up rows (a multiple of 64), no norm, bias or residual");
    a.swi_h = hints.swi_h, a.swi_q = hints.swi_q, a.swi_count = hints.swi_count;
    return dispatch_direct<false, 2>(kind, a, st);
  }
  return norm ? dispatch_direct<true, 0>(kind, a, st) : dispatch_direct<false, 0>(kind, a, st);
}

}  // namespace ieb
