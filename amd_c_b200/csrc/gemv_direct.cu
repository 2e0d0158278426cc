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
  uint32_t late;      // let dependents start only after this kernel's own dependency wait: a dependent that starts then knows that
                      // everything older than this kernel has completed
  uint32_t *work;     // two words, zero between launches; word 1 counts the CTAs that have finished (norm tail only)
  ArPush push;        // TP kernels only: every finished row also goes to the other ranks' slots
  uint32_t swi;       // rows are interleaved (gate_i, up_i) pairs (two rows per warp): y[i] = silu(gate_i) * up_i instead of the rows
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

// TP: a tensor-parallel partial whose finished rows are also stored to the peers.
template <int KIND, bool NORM, int R, int U, int MINB, bool TP>
__global__ void __launch_bounds__(GD_THREADS, MINB) gemv_direct_kernel(const GdArgs a) {
  extern __shared__ uint4 smem_gd[];
  const uint32_t nb = a.nb;
  uint4 *A0 = smem_gd, *A1 = smem_gd + nb;
  float *da = reinterpret_cast<float *>(smem_gd + 2u * nb);
  int *as = reinterpret_cast<int *>(da + nb);
  __shared__ float red[GD_WARPS];
  __shared__ uint32_t last;

  if (!a.late) pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // Row groups of R are dealt round-robin over all warps of the grid, so at any moment the grid reads one
  // contiguous window.
  const uint32_t W = gridDim.x * GD_WARPS, groups = (a.rows + R - 1u) / R, r_hi = a.rows;
  uint32_t grp = blockIdx.x * GD_WARPS + warp;

  Blk<KIND, false> first[R][U];
  if (grp < groups) gd_load<KIND, R, U>(first, a.w, a.rowb, grp * R, r_hi, 0u, nb, lane);

  // the norm weights (a constant vector) into L2 while waiting: the norm after the wait then pays one L2 round trip
  if (NORM) {
    if (a.act.norm_w)
      for (uint32_t i = 32u * threadIdx.x; i < 32u * nb; i += 32u * GD_THREADS) prefetch_l2(a.act.norm_w + i);
  } else if (a.tail.norm_w && blockIdx.x == 0) {
    for (uint32_t i = 32u * threadIdx.x; i < a.rows; i += 32u * GD_THREADS) prefetch_l2(a.tail.norm_w + i);
  }
  pdl_wait();
  if (a.late) pdl_launch_dependents();
  uint32_t ep = 0u;  // TP: the epoch of this exchange (the previous one is complete: its kernel is)
  if (TP) ep = *(volatile uint32_t *)a.push.epoch + 1u;
  stage_activations<NORM, GD_WARPS>(a.act, nb, A0, A1, da, as, red, blockIdx.x == 0, [] { __syncthreads(); });

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
    if (R == 2 && a.swi) {  // the SwiGLU kernel's arithmetic on the pair this warp owns
      if (lane == 0 && rr + 1 < r_hi) {
        const float g = v[0];
        a.y[rr >> 1] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), v[R - 1]);
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
      // GEMV; a warp's two adjacent rows travel as one 16-byte store (each half carries its own epoch).
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
    }
  }
}

template <int KIND, bool NORM, int R, int U, int MINB, bool TP>
static int launch_direct(const GdArgs &a, cudaStream_t st) {
  const size_t smem = (size_t)a.nb * 40u;
  auto k = gemv_direct_kernel<KIND, NORM, R, U, MINB, TP>;
  if (int r = ensure_dynamic_smem(reinterpret_cast<const void *>(k), smem)) return r;
  // One group per warp up to a persistent grid of exactly the resident CTAs (MINB per SM), whose warps loop.
  const unsigned need = (a.rows + R * GD_WARPS - 1) / (R * GD_WARPS);
  unsigned grid = (unsigned)(sm_count() * MINB);
  if (grid > need) grid = need ? need : 1u;
  IEB_LAUNCH_PDL("gemv_direct_kernel", k, dim3(grid), dim3(GD_THREADS), smem, st, a);
  return IE_B200_OK;
}

// Long rows with few of them (the FFN down projection: 4096 x 14336) are a chain of dependent chunks per warp at
// two rows per warp; one row per warp with the whole row's loads in flight at once (up to 16 lane steps, 2 CTAs
// per SM for the registers that takes) shortens the chain to one round trip per row.
template <int KIND, bool NORM, bool TP>
static int pick_direct(const GdArgs &a, cudaStream_t st) {
  constexpr int U2 = KIND == IE_B200_MAT_Q4 ? 4 : 2;
  const bool few_long = !a.swi && a.nb >= 256u && (uint64_t)a.rows * 2u <= (uint64_t)sm_count() * 3u * GD_WARPS * 4u;
  if (few_long) return launch_direct<KIND, NORM, 1, 4 * U2, 2, TP>(a, st);  // Q4_0: 16 lane steps = rows of up to 512 blocks in one chunk
  return launch_direct<KIND, NORM, 2, U2, 3, TP>(a, st);
}

template <bool NORM, bool TP>
int dispatch_direct(int kind, const GdArgs &a, cudaStream_t st) {
  switch (kind) {
    case IE_B200_MAT_Q4: return pick_direct<IE_B200_MAT_Q4, NORM, TP>(a, st);
    case IE_B200_MAT_Q8: return pick_direct<IE_B200_MAT_Q8, NORM, TP>(a, st);
    case IE_B200_MAT_Q4K: return pick_direct<IE_B200_MAT_Q4K, NORM, TP>(a, st);
    case IE_B200_MAT_Q6K: return pick_direct<IE_B200_MAT_Q6K, NORM, TP>(a, st);
    default: return fail(IE_B200_E_ARG, "gemv_direct: matrix kind %d has no streaming kernel", kind);
  }
}

int gemv_direct(int kind, const void *d_w, uint32_t rows, uint32_t cols, const ActSrc &act, bool norm, float *d_y, const float *d_bias,
                const float *d_res, const ActSrc *tail, uint32_t *work, cudaStream_t st, const ArPush *push, bool late_trigger, bool swiglu_pairs) {
  GdArgs a = {};
  a.late = late_trigger ? 1u : 0u;
  if (swiglu_pairs) {
    if (tail || push || d_bias || d_res || rows % 2u) return fail(IE_B200_E_ARG, "gemv_direct: the SwiGLU form takes interleaved gate / up rows, no bias, residual or tail");
    a.swi = 1u;
  }
  a.w = static_cast<const uint8_t *>(d_w), a.rowb = row_bytes_of(kind, cols), a.rows = rows, a.nb = cols / 32u;
  a.act = act, a.y = d_y, a.bias = d_bias, a.res = d_res;
  a.work = work;
  if (tail) a.tail = *tail, a.tail.xf = d_y;
  if (push) {
    if ((norm && act.norm_w) || tail || d_bias || d_res) return fail(IE_B200_E_ARG, "gemv_direct: a tensor-parallel partial takes no norm, bias or residual");
    a.push = *push;
    return norm ? dispatch_direct<true, true>(kind, a, st) : dispatch_direct<false, true>(kind, a, st);
  }
  return norm ? dispatch_direct<true, false>(kind, a, st) : dispatch_direct<false, false>(kind, a, st);
}

bool gemv_direct_ok(int kind, uint32_t cols) {
  return kind != IE_B200_MAT_F32 && cols % 32u == 0 && cols / 32u <= 1024u;
}

}  // namespace ieb

using namespace ieb;

static int check_common(const char *who, int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_y) {
  if (!d_w || !d_y) return fail(IE_B200_E_ARG, "%s: NULL pointer", who);
  if (!aligned16(d_w)) return fail(IE_B200_E_ARG, "%s: weights must be 16-byte aligned", who);
  if (cols == 0 || cols % 32u) return fail(IE_B200_E_SIZE, "%s: cols %u is not a multiple of 32", who, cols);
  if ((kind == IE_B200_MAT_Q4K || kind == IE_B200_MAT_Q6K) && cols % 256u) return fail(IE_B200_E_SIZE, "%s: K kinds need cols %% 256 == 0", who);
  if (cols / 32u > 1024u) return fail(IE_B200_E_SIZE, "%s: %u blocks per row > 1024", who, cols / 32u);
  (void)rows;
  return IE_B200_OK;
}

extern "C" int ie_b200_gemv_stream(int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_xq, float *d_y, const float *d_bias,
                                   const float *d_res, void *stream) {
  if (int e = check_common("ie_b200_gemv_stream", kind, d_w, rows, cols, d_y)) return e;
  if (!d_xq || !aligned16(d_xq)) return fail(IE_B200_E_ARG, "ie_b200_gemv_stream: activations must be a 16-byte aligned Q8 buffer");
  if (rows == 0) return IE_B200_OK;
  ActSrc act = {};
  act.xq = static_cast<const uint8_t *>(d_xq);
  return gemv_direct(kind, d_w, rows, cols, act, false, d_y, d_bias, d_res, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int ie_b200_norm_gemv_stream(int kind, const void *d_w, uint32_t rows, uint32_t cols, const float *d_x, const float *d_norm_w,
                                        float eps, float *d_xn_out, void *d_xq_out, float *d_y, const float *d_bias, const float *d_res,
                                        void *stream) {
  if (int e = check_common("ie_b200_norm_gemv_stream", kind, d_w, rows, cols, d_y)) return e;
  if (!d_x || !d_norm_w) return fail(IE_B200_E_ARG, "ie_b200_norm_gemv_stream: NULL pointer");
  if (rows == 0) return IE_B200_OK;
  ActSrc act = {};
  act.xf = d_x, act.norm_w = d_norm_w, act.eps = eps, act.xn_out = d_xn_out, act.xq_out = static_cast<uint8_t *>(d_xq_out);
  return gemv_direct(kind, d_w, rows, cols, act, true, d_y, d_bias, d_res, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int ie_b200_gemv_swiglu(int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_xq, float *d_h, void *stream) {
  if (int e = check_common("ie_b200_gemv_swiglu", kind, d_w, rows, cols, d_h)) return e;
  if (!d_xq || !aligned16(d_xq)) return fail(IE_B200_E_ARG, "ie_b200_gemv_swiglu: activations must be a 16-byte aligned Q8 buffer");
  if (rows == 0) return IE_B200_OK;
  ActSrc act = {};
  act.xq = static_cast<const uint8_t *>(d_xq);
  return gemv_direct(kind, d_w, rows, cols, act, false, d_h, nullptr, nullptr, nullptr, nullptr, static_cast<cudaStream_t>(stream), nullptr, false, true);
}

extern "C" int ie_b200_quant_gemv_stream(int kind, const void *d_w, uint32_t rows, uint32_t cols, const float *d_x, void *d_xq_out, float *d_y,
                                         const float *d_bias, const float *d_res, void *stream) {
  if (int e = check_common("ie_b200_quant_gemv_stream", kind, d_w, rows, cols, d_y)) return e;
  if (!d_x || !aligned16(d_x)) return fail(IE_B200_E_ARG, "ie_b200_quant_gemv_stream: the vector must be 16-byte aligned");
  if (rows == 0) return IE_B200_OK;
  ActSrc act = {};
  act.xf = d_x, act.norm_w = nullptr, act.eps = 0.0f, act.xq_out = static_cast<uint8_t *>(d_xq_out);
  return gemv_direct(kind, d_w, rows, cols, act, true, d_y, d_bias, d_res, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int ie_b200_gemv_norm_tail(int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_xq, float *d_y, const float *d_bias,
                                      const float *d_res, const float *d_norm_w, float eps, float *d_xn_out, void *d_xq_out, uint32_t *d_counter,
                                      void *stream) {
  if (int e = check_common("ie_b200_gemv_norm_tail", kind, d_w, rows, cols, d_y)) return e;
  if (!d_xq || !aligned16(d_xq) || !d_norm_w || !d_counter) return fail(IE_B200_E_ARG, "ie_b200_gemv_norm_tail: NULL or misaligned pointer");
  if (rows == 0 || rows % 32u) return fail(IE_B200_E_SIZE, "ie_b200_gemv_norm_tail: the norm of the result needs rows %% 32 == 0 (rows = %u)", rows);
  if ((d_xn_out && !aligned16(d_xn_out)) || (d_xq_out && !aligned16(d_xq_out)) || !aligned16(d_y))
    return fail(IE_B200_E_ARG, "ie_b200_gemv_norm_tail: outputs must be 16-byte aligned");
  ActSrc act = {}, tail = {};
  act.xq = static_cast<const uint8_t *>(d_xq);
  tail.norm_w = d_norm_w, tail.eps = eps, tail.xn_out = d_xn_out, tail.xq_out = static_cast<uint8_t *>(d_xq_out);
  return gemv_direct(kind, d_w, rows, cols, act, false, d_y, d_bias, d_res, &tail, d_counter, static_cast<cudaStream_t>(stream));
}
