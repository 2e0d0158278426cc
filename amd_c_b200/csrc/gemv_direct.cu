// gemv_direct.cu -- the decode (one token) GEMV that streams weights straight
// from HBM into registers, launched with programmatic dependent launch.
//
// Every warp of a persistent grid (two CTAs of eight warps per SM) takes row
// pairs round-robin (pair g, g + W, ... for W warps in the grid); lane l takes
// blocks l, l+32, ... of its rows, so each lane keeps up to 8 16-byte loads
// in flight. The first loads of a warp are issued BEFORE the kernel
// waits for its predecessor (the weights do not depend on it): the launch
// latency, the DRAM latency and the predecessor's tail overlap with weight
// traffic that is already on its way. Only then are the activations staged
// (optionally computed: fused RMSNorm + Q8, see act_stage.cuh) and consumed.
// Registers are capped at 80 per thread (three CTAs per SM): a kernel's own
// two CTAs plus one early CTA of its successor are resident together.
//
// Arithmetic and order are the reference's (one warp per row, blocks
// l, l+32, ... in order, shuffle-down tree): bit-exact with its CPU GEMV.
#include "act_stage.cuh"
#include "common.cuh"
#include "gemv_blocks.cuh"

namespace ieb {

constexpr int GD_WARPS = 8, GD_THREADS = GD_WARPS * 32, GD_CTAS_PER_SM = 2;

struct GdArgs {
  const uint8_t *w;
  size_t rowb;
  uint32_t rows, nb;
  ActSrc act;
  float *y;
  const float *bias, *res;
  // norm tail (optional): once every CTA has written its rows, the last CTA to finish computes
  // tail.xn_out = rmsnorm(y) * tail.norm_w and its Q8 copy tail.xq_out for the next GEMV
  ActSrc tail;
  uint32_t *counter;  // zero between launches
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

template <int KIND, bool NORM, int R, int U>
__global__ void __launch_bounds__(GD_THREADS, 3) gemv_direct_kernel(const GdArgs a) {
  extern __shared__ uint4 smem_gd[];
  const uint32_t nb = a.nb;
  uint4 *A0 = smem_gd, *A1 = smem_gd + nb;
  float *da = reinterpret_cast<float *>(smem_gd + 2u * nb);
  int *as = reinterpret_cast<int *>(da + nb);
  __shared__ float red[GD_WARPS];
  __shared__ uint32_t last;

  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // row groups of R are dealt round-robin over all warps of the grid: at any moment the grid reads one contiguous window
  const uint32_t stride = gridDim.x * GD_WARPS * R, r_hi = a.rows;
  uint32_t r = (blockIdx.x * GD_WARPS + warp) * R;

  // the first chunk of this warp's first rows: in flight while we wait for the previous kernel
  Blk<KIND, false> first[R][U];
  if (r < r_hi) gd_load<KIND, R, U>(first, a.w, a.rowb, r, r_hi, 0u, nb, lane);

  pdl_wait();
  stage_activations<NORM, GD_WARPS>(a.act, nb, A0, A1, da, as, red, blockIdx.x == 0, [] { __syncthreads(); });

  // one row group: chunk by chunk, R x U loads in flight, then the tree and the epilogue
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
#pragma unroll
    for (int i = 0; i < R; i++) {
      const float v = warp_tree(acc[i]);
      if (lane == 0 && rr + i < r_hi) {
        float o = v;
        if (a.bias) o = __fadd_rn(o, a.bias[rr + i]);
        if (a.res) o = __fadd_rn(a.res[rr + i], o);
        a.y[rr + i] = o;
      }
    }
  };
  if (r < r_hi) {  // the first group: its first chunk is already in registers
    float acc[R];
#pragma unroll
    for (int i = 0; i < R; i++) acc[i] = 0.0f;
    chunk(first, acc, r, 0u);
    for (uint32_t c = 32u * U; c < nb; c += 32u * U) {
      Blk<KIND, false> blk[R][U];
      gd_load<KIND, R, U>(blk, a.w, a.rowb, r, r_hi, c, nb, lane);
      chunk(blk, acc, r, c);
    }
    finish(acc, r);
    r += stride;
  }
  for (; r < r_hi; r += stride) {
    float acc[R];
#pragma unroll
    for (int i = 0; i < R; i++) acc[i] = 0.0f;
    for (uint32_t c = 0; c < nb; c += 32u * U) {
      Blk<KIND, false> blk[R][U];
      gd_load<KIND, R, U>(blk, a.w, a.rowb, r, r_hi, c, nb, lane);
      chunk(blk, acc, r, c);
    }
    finish(acc, r);
  }
  if (a.counter) {  // the norm tail (uniform over the grid: every CTA takes this branch)
    __threadfence();  // this thread's rows are visible before the arrival is counted
    __syncthreads();
    if (threadIdx.x == 0) {
      last = atomicAdd(a.counter, 1u) == gridDim.x - 1u;
      if (last) *a.counter = 0u;
    }
    __syncthreads();
    if (last) {
      __threadfence();
      stage_activations<true, GD_WARPS>(a.tail, a.rows / 32u, nullptr, nullptr, nullptr, nullptr, red, true, [] { __syncthreads(); });
    }
  }
}

template <int KIND, bool NORM, int R, int U>
static int launch_direct(const GdArgs &a, cudaStream_t st) {
  const size_t smem = (size_t)a.nb * 40u;
  auto k = gemv_direct_kernel<KIND, NORM, R, U>;
  if (int r = ensure_dynamic_smem(reinterpret_cast<const void *>(k), smem)) return r;
  // NORM (the activations are computed in every CTA's prologue): a persistent grid, two CTAs per SM, three for a
  // large matrix. Otherwise R rows per warp and as many CTAs as one pass takes, capped at 8 per SM (three are
  // resident; beyond the cap a CTA loops, which amortises its activation staging over more rows).
  const unsigned need = (a.rows + R * GD_WARPS - 1) / (R * GD_WARPS);
  unsigned grid;
  if (NORM) {
    const bool big = a.rowb * a.rows > (24u << 20);
    grid = (unsigned)(sm_count() * (big ? 3 : GD_CTAS_PER_SM));
  } else {
    grid = (unsigned)(sm_count() * 8);
  }
  if (grid > need) grid = need ? need : 1u;
  IEB_LAUNCH_PDL("gemv_direct_kernel", k, dim3(grid), dim3(GD_THREADS), smem, st, a);
  return IE_B200_OK;
}

// Long rows with few of them (the FFN down projection: 4096 x 14336) leave SMs short of warps at two rows per
// warp; one row per warp with twice the lane steps in flight doubles the CTAs at the same bytes in flight.
template <int KIND, bool NORM>
static int pick_direct(const GdArgs &a, cudaStream_t st) {
  constexpr int U2 = KIND == IE_B200_MAT_Q4 ? 4 : 2;
  const bool few_long = (a.rows + 15u) / 16u < (uint32_t)(sm_count() * 3) && a.nb >= 256u;
  if (few_long) return launch_direct<KIND, NORM, 1, 2 * U2>(a, st);
  return launch_direct<KIND, NORM, 2, U2>(a, st);
}

template <bool NORM>
int dispatch_direct(int kind, const GdArgs &a, cudaStream_t st) {
  switch (kind) {
    case IE_B200_MAT_Q4: return pick_direct<IE_B200_MAT_Q4, NORM>(a, st);
    case IE_B200_MAT_Q4K: return pick_direct<IE_B200_MAT_Q4K, NORM>(a, st);
    case IE_B200_MAT_Q6K: return pick_direct<IE_B200_MAT_Q6K, NORM>(a, st);
    default: return fail(IE_B200_E_ARG, "gemv_direct: matrix kind %d has no streaming kernel", kind);
  }
}

// Entry used by gemv_stream.cu's dispatcher.
int gemv_direct(int kind, const void *d_w, uint32_t rows, uint32_t cols, const ActSrc &act, bool norm, float *d_y, const float *d_bias,
                const float *d_res, const ActSrc *tail, uint32_t *counter, cudaStream_t st) {
  GdArgs a = {};
  a.w = static_cast<const uint8_t *>(d_w), a.rowb = row_bytes_of(kind, cols), a.rows = rows, a.nb = cols / 32u;
  a.act = act, a.y = d_y, a.bias = d_bias, a.res = d_res;
  if (tail) a.tail = *tail, a.tail.xf = d_y, a.counter = counter;
  return norm ? dispatch_direct<true>(kind, a, st) : dispatch_direct<false>(kind, a, st);
}

}  // namespace ieb
