// gemv_stream.cu -- the decode (one token) GEMV: weight row panels stream
// from HBM into a shared-memory ring through bulk asynchronous copies
// (cp.async.bulk + mbarrier, the 1-D form of TMA), and the kernel is
// launched with programmatic dependent launch so that its ring fills while
// the previous kernel of the step is still running.
//
// One CTA per SM owns a contiguous range of rows. A producer thread keeps
// STAGES copies in flight (each RPS consecutive rows = one contiguous span of
// the row-panel layout); RPS / 2 consumer warps take two rows each from a
// stage, sharing the activation reads.
// The weights do not depend on the previous kernel, so the producer starts
// copying at once; the consumers first wait for the previous grid
// (griddepcontrol.wait), stage the activations, then consume. The shared
// memory of a CTA stays under half an SM so that the CTAs of two consecutive
// kernels are resident together: HBM traffic continues across kernel
// boundaries.
//
// Arithmetic and order are those of gemv.cu (one warp per row, lane l takes
// blocks l, l+32, ... in order, shuffle-down tree): bit-exact with the
// reference CPU GEMV. With NORM the activations are produced in the prologue
// from the f32 residual stream: rmsnorm + the per-32 Q8 quantiser, computed
// redundantly by every CTA (16 KB read from L2), which removes a kernel and
// its launch gap from the dependency chain.
//
// Every wait on an mbarrier is bounded by wall time (2 s): a thread that gives
// up sets the error word and the CTA drains; a kernel that finds the error word
// already set does nothing, so one failure does not stall the rest of a step.
//
// Ring discipline: a parity wait only tells "the current or the previous phase
// is complete", so a waiter must never be two phases ahead of its stage. Every
// consumer warp therefore waits on every stage in iteration order, also for
// the stages whose rows belong to another warp group.
#include <cstdlib>

#include "common.cuh"
#include "act_stage.cuh"
#include "gemv_blocks.cuh"
#include "peer_ll.cuh"

namespace ieb {

constexpr int GS_CONSUMER_WARPS = 8;
constexpr int GS_THREADS = (GS_CONSUMER_WARPS + 1) * 32;
constexpr int GS_MAX_STAGES = 8;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;  // 2 s: far beyond any healthy wait (a step is about a millisecond)
constexpr size_t GS_CTA_SMEM = 110u * 1024u;  // per CTA, so that the CTAs of two consecutive kernels fit one SM

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Wait for the phase with the given parity, for at most WAIT_LIMIT_NS of wall time; false if it ran out.
// (A poll may itself sleep for a hardware-chosen time, so the bound is on the clock, not on a poll count.)
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
  const uint32_t a = smem_u32(bar);
  uint64_t t0 = 0;
  for (uint32_t i = 0;; i++) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(a), "r"(parity)
        : "memory");
    if (ok) return true;
    const uint64_t now = global_ns();
    if (i == 0) t0 = now;
    else if (now - t0 > WAIT_LIMIT_NS) return false;
  }
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src),
               "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(GS_CONSUMER_WARPS * 32) : "memory"); }

struct GsArgs {
  const uint8_t *w;
  size_t rowb;
  uint32_t rows, nb;
  const uint8_t *xq;     // Q8 activations (NORM = false)
  const float *xf;       // f32 input of the fused norm (NORM = true)
  const float *norm_w;
  float eps;
  float *xn_out;         // optional: the normalised vector, written by CTA 0
  uint8_t *xq_out;       // optional: its Q8 copy, written by CTA 0
  float *y;
  const float *bias, *res;
  uint32_t *err;          // device error word: 1 = a bounded wait ran out, 2 = a bounds self-check failed
  uint32_t rps, stages, stage_bytes;
  size_t w_bytes;         // extent of the matrix, for the producer's bounds self-check
};

// Shared layout: ring | A0 | A1 | da | as | (NORM: f32 scratch nb*32) | barriers
template <int KIND, bool NORM>
__global__ void __launch_bounds__(GS_THREADS, 2) gemv_stream_kernel(const GsArgs a) {
  extern __shared__ __align__(128) uint8_t smem_gs[];
  const uint32_t nb = a.nb;
  uint8_t *ring = smem_gs;
  uint4 *A0 = reinterpret_cast<uint4 *>(ring + (size_t)a.stages * a.stage_bytes);
  uint4 *A1 = A0 + nb;
  float *da = reinterpret_cast<float *>(A1 + nb);
  int *as = reinterpret_cast<int *>(da + nb);
  uint64_t *full = reinterpret_cast<uint64_t *>(as + nb);  // 40 nb bytes of activations keep 8-byte alignment
  uint64_t *empty = full + GS_MAX_STAGES;
  __shared__ float red[GS_CONSUMER_WARPS];
  __shared__ uint32_t failed, skip;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t G = gridDim.x, c = blockIdx.x;
  const uint32_t r_lo = (uint32_t)((uint64_t)a.rows * c / G), r_hi = (uint32_t)((uint64_t)a.rows * (c + 1) / G);
  const uint32_t n_it = (r_hi - r_lo + a.rps - 1u) / a.rps;
  const uint32_t wps = a.rps / 2u;                    // consumer warps per stage: each takes two rows
  const uint32_t groups = GS_CONSUMER_WARPS / wps;    // warp groups that alternate over the stages

  if (threadIdx.x == 0) {
    skip = a.err ? *(volatile uint32_t *)a.err : 0u;  // an earlier kernel already failed: do nothing
    failed = 0;
    for (uint32_t s = 0; s < a.stages; s++) mbar_init(&full[s], 1), mbar_init(&empty[s], wps);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();  // the next kernel may begin its own prefetch

  if (warp == GS_CONSUMER_WARPS) {
    // ---------------- producer: one thread keeps the ring full ----------------
    if (lane == 0 && !skip) {
      for (uint32_t it = 0; it < n_it; it++) {
        const uint32_t s = it % a.stages;
        if (it >= a.stages && !mbar_wait(&empty[s], ((it / a.stages) - 1u) & 1u)) {
          failed = 1;
          if (a.err) atomicExch(a.err, 1u);
          break;
        }
        if (*(volatile uint32_t *)&failed) break;
        const uint32_t row0 = r_lo + it * a.rps;
        const uint32_t nrow = min(a.rps, r_hi - row0);
        const uint32_t bytes = nrow * (uint32_t)a.rowb;
        // self-check: the copy stays inside the matrix and inside its ring slot, and is 16-byte granular
        if ((size_t)row0 * a.rowb + bytes > a.w_bytes || bytes > a.stage_bytes || (bytes & 15u) || nrow == 0u ||
            ((uintptr_t)(a.w + (size_t)row0 * a.rowb) & 15u)) {
          failed = 1;
          if (a.err) atomicExch(a.err, 2u);
          break;
        }
        mbar_expect_tx(&full[s], bytes);
        bulk_g2s(ring + (size_t)s * a.stage_bytes, a.w + (size_t)row0 * a.rowb, bytes, &full[s]);
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  pdl_wait();  // the previous kernel's results (activations, residual) are complete and visible
  if (skip) return;
  ActSrc src;
  src.xq = a.xq, src.xf = a.xf, src.norm_w = a.norm_w, src.eps = a.eps, src.xn_out = a.xn_out, src.xq_out = a.xq_out;
  stage_activations<NORM, GS_CONSUMER_WARPS>(src, nb, A0, A1, da, as, red, c == 0, [] { consumer_sync(); });
  consumer_sync();

  const uint32_t grp = warp / wps, wrow = (warp % wps) * 2u;
  for (uint32_t it = 0; it < n_it; it++) {
    const uint32_t s = it % a.stages;
    if (*(volatile uint32_t *)&failed) break;
    if (!mbar_wait(&full[s], (it / a.stages) & 1u)) {  // every warp follows every stage (see the header)
      failed = 1;
      if (a.err) atomicExch(a.err, 1u);
      break;
    }
    if (it % groups != grp) continue;
    const uint32_t r = r_lo + it * a.rps + wrow;
    if (r < r_hi) {
      const bool two = r + 1u < r_hi;
      const uint8_t *rp0 = ring + (size_t)s * a.stage_bytes + (size_t)wrow * a.rowb, *rp1 = rp0 + a.rowb;
      float acc0 = 0.0f, acc1 = 0.0f;
      for (uint32_t b = lane; b < nb; b += 32u) {
        Blk<KIND, true> b0, b1;
        b0.load(rp0, b, nb);
        if (two) b1.load(rp1, b, nb);
        const uint4 a0 = A0[b], a1 = A1[b];
        const float d = da[b];
        const int sm = as[b];
        acc0 = b0.accum(acc0, a0, a1, d, sm, b);
        if (two) acc1 = b1.accum(acc1, a0, a1, d, sm, b);
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
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
  }
}

template <int KIND, bool NORM>
static int launch_stream(GsArgs &a, cudaStream_t st) {
  // rows per stage: 16 (two per consumer warp) if three such stages fit beside the activations, else 8, 4, 2
  // (for very long rows two stages of two rows must fit)
  const size_t fixed = (size_t)a.nb * 40u + 2u * GS_MAX_STAGES * 8u;
  if (fixed + 2u * 2u * a.rowb > GS_CTA_SMEM) return fail(IE_B200_E_SIZE, "gemv_stream: rows of %zu bytes do not fit the ring", a.rowb);
  const size_t budget = GS_CTA_SMEM - fixed;
  uint32_t rps = 2u * GS_CONSUMER_WARPS;
  while (rps > 2u && 3u * rps * a.rowb > budget) rps >>= 1;
  const size_t stage = (size_t)rps * a.rowb;
  uint32_t stages = (uint32_t)(budget / stage);
  if (stages > (uint32_t)GS_MAX_STAGES) stages = GS_MAX_STAGES;
  a.rps = rps, a.stages = stages, a.stage_bytes = (uint32_t)stage;
  const size_t smem = stage * stages + fixed;
  auto k = gemv_stream_kernel<KIND, NORM>;
  if (int r = ensure_dynamic_smem(reinterpret_cast<const void *>(k), GS_CTA_SMEM)) return r;
  unsigned grid = (unsigned)sm_count();
  if (grid > a.rows) grid = a.rows;
  IEB_LAUNCH_PDL("gemv_stream_kernel", k, dim3(grid), dim3(GS_THREADS), smem, st, a);
  return IE_B200_OK;
}

template <bool NORM>
static int dispatch_stream(int kind, GsArgs &a, cudaStream_t st) {
  switch (kind) {
    case IE_B200_MAT_Q4: return launch_stream<IE_B200_MAT_Q4, NORM>(a, st);
    case IE_B200_MAT_Q4K: return launch_stream<IE_B200_MAT_Q4K, NORM>(a, st);
    case IE_B200_MAT_Q6K: return launch_stream<IE_B200_MAT_Q6K, NORM>(a, st);
    default: return fail(IE_B200_E_ARG, "gemv_stream: matrix kind %d has no streaming kernel", kind);
  }
}


// Which decode GEMV runs: "direct" (registers, default) or "ring" (bulk copies into shared memory); IE_B200_GEMV selects.
bool gemv_uses_ring() {
  static const bool ring = [] {
    const char *v = getenv("IE_B200_GEMV");
    return v && v[0] == 'r';
  }();
  return ring;
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
                                   const float *d_res, uint32_t *d_err, uint32_t *d_work, void *stream) {
  if (int e = check_common("ie_b200_gemv_stream", kind, d_w, rows, cols, d_y)) return e;
  if (!d_xq || !aligned16(d_xq)) return fail(IE_B200_E_ARG, "ie_b200_gemv_stream: activations must be a 16-byte aligned Q8 buffer");
  if (rows == 0) return IE_B200_OK;
  if (!gemv_uses_ring()) {
    ActSrc act = {};
    act.xq = static_cast<const uint8_t *>(d_xq);
    return gemv_direct(kind, d_w, rows, cols, act, false, d_y, d_bias, d_res, nullptr, d_work, static_cast<cudaStream_t>(stream));
  }
  GsArgs a = {};
  a.w = static_cast<const uint8_t *>(d_w), a.rowb = row_bytes_of(kind, cols), a.rows = rows, a.nb = cols / 32u;
  a.w_bytes = a.rowb * rows;
  a.xq = static_cast<const uint8_t *>(d_xq), a.y = d_y, a.bias = d_bias, a.res = d_res, a.err = d_err;
  return dispatch_stream<false>(kind, a, static_cast<cudaStream_t>(stream));
}

extern "C" int ie_b200_norm_gemv_stream(int kind, const void *d_w, uint32_t rows, uint32_t cols, const float *d_x, const float *d_norm_w,
                                        float eps, float *d_xn_out, void *d_xq_out, float *d_y, const float *d_bias, const float *d_res,
                                        uint32_t *d_err, uint32_t *d_work, void *stream) {
  if (int e = check_common("ie_b200_norm_gemv_stream", kind, d_w, rows, cols, d_y)) return e;
  if (!d_x || !d_norm_w) return fail(IE_B200_E_ARG, "ie_b200_norm_gemv_stream: NULL pointer");
  if (rows == 0) return IE_B200_OK;
  if (!gemv_uses_ring()) {
    ActSrc act = {};
    act.xf = d_x, act.norm_w = d_norm_w, act.eps = eps, act.xn_out = d_xn_out, act.xq_out = static_cast<uint8_t *>(d_xq_out);
    return gemv_direct(kind, d_w, rows, cols, act, true, d_y, d_bias, d_res, nullptr, d_work, static_cast<cudaStream_t>(stream));
  }
  GsArgs a = {};
  a.w = static_cast<const uint8_t *>(d_w), a.rowb = row_bytes_of(kind, cols), a.rows = rows, a.nb = cols / 32u;
  a.w_bytes = a.rowb * rows;
  a.xf = d_x, a.norm_w = d_norm_w, a.eps = eps, a.xn_out = d_xn_out, a.xq_out = static_cast<uint8_t *>(d_xq_out);
  a.y = d_y, a.bias = d_bias, a.res = d_res, a.err = d_err;
  return dispatch_stream<true>(kind, a, static_cast<cudaStream_t>(stream));
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
