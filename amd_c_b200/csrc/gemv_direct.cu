// gemv_direct.cu -- the decode (one token) GEMV that streams weights straight
// from HBM into registers, launched with programmatic dependent launch.
//
// Every warp of a persistent grid (two CTAs of eight warps per SM) takes row
// pairs round-robin (pair g, g + W, ... for W warps in the grid); lane l takes
// blocks l, l+32, ... of both rows, so each lane keeps up to 2 x 4 16-byte
// loads in flight. The first loads of a warp are issued BEFORE the kernel
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
// lane steps (blocks per row) loaded before any is consumed: 4 for Q4_0 (5 registers a block), 2 for the K kinds
template <int KIND>
struct GdU {
  static constexpr int value = KIND == IE_B200_MAT_Q4 ? 4 : 2;
};

struct GdArgs {
  const uint8_t *w;
  size_t rowb;
  uint32_t rows, nb;
  ActSrc act;
  float *y;
  const float *bias, *res;
};

template <int KIND>
__device__ __forceinline__ void gd_load(Blk<KIND, false> (&blk)[2][GdU<KIND>::value], const uint8_t *w, size_t rowb, uint32_t r, uint32_t r_hi, uint32_t c, uint32_t nb,
                                        int lane) {
#pragma unroll
  for (int u = 0; u < GdU<KIND>::value; u++) {
    const uint32_t b = c + 32u * u + lane;
    if (b < nb) {
      blk[0][u].load(w + (size_t)r * rowb, b, nb);
      if (r + 1u < r_hi) blk[1][u].load(w + (size_t)(r + 1u) * rowb, b, nb);
    }
  }
}

template <int KIND, bool NORM>
__global__ void __launch_bounds__(GD_THREADS, 3) gemv_direct_kernel(const GdArgs a) {
  constexpr int GD_U = GdU<KIND>::value;
  extern __shared__ uint4 smem_gd[];
  const uint32_t nb = a.nb;
  uint4 *A0 = smem_gd, *A1 = smem_gd + nb;
  float *da = reinterpret_cast<float *>(smem_gd + 2u * nb);
  int *as = reinterpret_cast<int *>(da + nb);
  __shared__ float red[GD_WARPS];

  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // row pairs are dealt round-robin over all warps of the grid: at any moment the grid reads one contiguous window
  const uint32_t stride = gridDim.x * GD_WARPS * 2u, r_hi = a.rows;
  uint32_t r = (blockIdx.x * GD_WARPS + warp) * 2u;

  // the first chunk of this warp's first row pair: in flight while we wait for the previous kernel
  Blk<KIND, false> blk[2][GD_U];
  if (r < r_hi) gd_load<KIND>(blk, a.w, a.rowb, r, r_hi, 0u, nb, lane);

  pdl_wait();
  stage_activations<NORM, GD_WARPS>(a.act, nb, A0, A1, da, as, red, blockIdx.x == 0, [] { __syncthreads(); });

  bool loaded = true;
  for (; r < r_hi; r += stride) {
    const bool two = r + 1u < r_hi;
    float acc0 = 0.0f, acc1 = 0.0f;
    for (uint32_t c = 0; c < nb; c += 32u * GD_U) {
      if (!loaded) gd_load<KIND>(blk, a.w, a.rowb, r, r_hi, c, nb, lane);
      loaded = false;
#pragma unroll
      for (int u = 0; u < GD_U; u++) {
        const uint32_t b = c + 32u * u + lane;
        if (b < nb) {
          const uint4 a0 = A0[b], a1 = A1[b];
          const float d = da[b];
          const int s = as[b];
          acc0 = blk[0][u].accum(acc0, a0, a1, d, s, b);
          if (two) acc1 = blk[1][u].accum(acc1, a0, a1, d, s, b);
        }
      }
    }
    const float v0 = warp_tree(acc0), v1 = warp_tree(acc1);
    if (lane == 0) {
      float o = v0;
      if (a.bias) o = __fadd_rn(o, a.bias[r]);
      if (a.res) o = __fadd_rn(a.res[r], o);
      a.y[r] = o;
      if (two) {
        o = v1;
        if (a.bias) o = __fadd_rn(o, a.bias[r + 1u]);
        if (a.res) o = __fadd_rn(a.res[r + 1u], o);
        a.y[r + 1u] = o;
      }
    }
  }
}

template <int KIND, bool NORM>
static int launch_direct(const GdArgs &a, cudaStream_t st) {
  const size_t smem = (size_t)a.nb * 40u;
  auto k = gemv_direct_kernel<KIND, NORM>;
  if (int r = ensure_dynamic_smem(reinterpret_cast<const void *>(k), smem)) return r;
  // two CTAs per SM leave room for the next kernel's early CTA; a large matrix (more than 24 MB) is worth all
  // three slots, its own streaming rate matters more than the overlap with its successor
  const bool big = a.rowb * a.rows > (24u << 20);
  unsigned grid = (unsigned)(sm_count() * (big ? 3 : GD_CTAS_PER_SM));
  const unsigned need = (a.rows + 2 * GD_WARPS - 1) / (2 * GD_WARPS);  // at least one row pair per warp
  if (grid > need) grid = need ? need : 1u;
  IEB_LAUNCH_PDL("gemv_direct_kernel", k, dim3(grid), dim3(GD_THREADS), smem, st, a);
  return IE_B200_OK;
}

template <bool NORM>
int dispatch_direct(int kind, const GdArgs &a, cudaStream_t st) {
  switch (kind) {
    case IE_B200_MAT_Q4: return launch_direct<IE_B200_MAT_Q4, NORM>(a, st);
    case IE_B200_MAT_Q4K: return launch_direct<IE_B200_MAT_Q4K, NORM>(a, st);
    case IE_B200_MAT_Q6K: return launch_direct<IE_B200_MAT_Q6K, NORM>(a, st);
    default: return fail(IE_B200_E_ARG, "gemv_direct: matrix kind %d has no streaming kernel", kind);
  }
}

// Entry used by gemv_stream.cu's dispatcher.
int gemv_direct(int kind, const void *d_w, uint32_t rows, uint32_t cols, const ActSrc &act, bool norm, float *d_y, const float *d_bias,
                const float *d_res, cudaStream_t st) {
  GdArgs a = {};
  a.w = static_cast<const uint8_t *>(d_w), a.rowb = row_bytes_of(kind, cols), a.rows = rows, a.nb = cols / 32u;
  a.act = act, a.y = d_y, a.bias = d_bias, a.res = d_res;
  return norm ? dispatch_direct<true>(kind, a, st) : dispatch_direct<false>(kind, a, st);
}

}  // namespace ieb
