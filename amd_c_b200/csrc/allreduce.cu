// allreduce.cu -- the latency-bound all-reduce of a tensor-parallel decode
// step: the sum over ranks of a dim-float partial (16-20 KB) after every
// K-split GEMV, fused with the residual add. One process per GPU; every rank
// maps the other ranks' receive buffers with CUDA IPC and the kernel moves the
// data itself with plain peer stores over NVLink (nothing replicated by the switch, no TMA):
//
//   push   each CTA writes its slice of this rank's partial into slot [rank]
//          of EVERY rank's receive buffer (its own included), then publishes
//          the call's epoch in that rank's flag word for (this rank, this CTA)
//          after a system-scope fence;
//   wait   the same CTA waits until the flags of all ranks for its slice show
//          the epoch (bounded by wall time: a missing rank sets the error
//          word instead of hanging the GPU);
//   sum    out = res + slot[0] + slot[1] + ... in rank order, read from this
//          GPU's own memory: every rank computes the same bits.
//
// Receive buffers are double-buffered by epoch parity: a rank can only be one
// call ahead of the slowest rank, because finishing call k needs everybody's
// flag k. The epoch lives on the device and is advanced by the last CTA of a
// call, so the kernel can sit in a replayed CUDA graph.
//
// The decode step uses two leaner kernels built on the same state (one CTA each, no fences): every 32-bit
// payload word travels as one 64-bit store {epoch, word}, so the receiver polls the data words themselves
// and a value is complete as soon as its epoch matches ("low-latency" slots, double-buffered by parity):
//   ar_norm_kernel    x = x + sum over ranks of part, then RMSNorm and the Q8 copy of x for the next GEMVs;
//   ar_argmax_kernel  the (value, global index) pairs of the ranks' local argmax, best one to every rank.
#include <cstring>

#include "common.cuh"
#include "ie_b200_tp.h"
#include "norm_quant.cuh"
#include "peer_ll.cuh"

namespace ieb {

constexpr int AR_THREADS = 256, AR_MAX_CTAS = 296;  // (all CTAs of a call are resident at once: 256 threads, few registers)

struct ArDev {
  float *slots[AR_MAX_RANKS];     // rank j's receive buffer: [2][world][max_n] floats
  uint32_t *flags[AR_MAX_RANKS];  // rank j's flags: [world][AR_MAX_CTAS]
  unsigned long long *ll[AR_MAX_RANKS];  // rank j's low-latency slots: [2][world][max_n] words of {epoch << 32 | payload}
  uint32_t *epoch;                // local: number of completed calls
  uint32_t *done;                 // local: CTAs that finished the current call
  uint32_t rank, world, max_n;
};

__global__ void __launch_bounds__(AR_THREADS) allreduce_add_kernel(const ArDev s, const float *part, const float *res, float *out, uint32_t n,
                                                                   uint32_t *err) {
  pdl_prologue();
  __shared__ uint32_t ok;
  // an earlier kernel of this step already gave up on a peer: push, advance the epoch, but do not wait again
  const bool dead = err && *(volatile uint32_t *)err != 0u;
  const uint32_t k = *(volatile uint32_t *)s.epoch + 1u, par = k & 1u;
  const uint32_t per = (n / 4u + gridDim.x - 1u) / gridDim.x * 4u;  // floats per CTA, a multiple of 4
  const uint32_t lo = blockIdx.x * per, hi = min(n, lo + per);
  // ---- push my slice to every rank
  for (uint32_t i = lo + 4u * threadIdx.x; i < hi; i += 4u * AR_THREADS) {
    const float4 v = *reinterpret_cast<const float4 *>(part + i);
    for (uint32_t j = 0; j < s.world; j++)
      *reinterpret_cast<float4 *>(s.slots[j] + ((size_t)par * s.world + s.rank) * s.max_n + i) = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < s.world) {
    volatile uint32_t *f = s.flags[threadIdx.x] + s.rank * AR_MAX_CTAS + blockIdx.x;
    *f = k;
  }
  if (threadIdx.x == 0) ok = 1u;
  __syncthreads();
  // ---- wait for every rank's slice (thread j watches rank j)
  if (threadIdx.x < s.world) {
    volatile uint32_t *f = s.flags[s.rank] + threadIdx.x * AR_MAX_CTAS + blockIdx.x;
    const uint64_t t0 = ar_now();
    while ((int32_t)(*f - k) < 0) {
      if (dead || ar_now() - t0 > AR_WAIT_NS) {
        ok = 0u;
        if (err) atomicExch(err, 3u);
        break;
      }
    }
  }
  __syncthreads();
  __threadfence_system();
  // ---- sum in rank order from my own memory
  if (ok) {
    const float *mine = s.slots[s.rank] + (size_t)par * s.world * s.max_n;
    // four float4 per thread and round, every rank's loads of a round in flight before the first sum (a prompt chunk's
    // exchange is megabytes: one dependent load per iteration left it bound by the latency of a load)
    constexpr uint32_t UN = 4u, STEP = 4u * AR_THREADS;
    for (uint32_t i0 = lo + 4u * threadIdx.x; i0 < hi; i0 += UN * STEP) {
      float4 acc[UN];
#pragma unroll
      for (uint32_t u = 0; u < UN; u++) {
        const uint32_t i = i0 + u * STEP;
        acc[u] = (i < hi && res) ? *reinterpret_cast<const float4 *>(res + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      for (uint32_t j = 0; j < s.world; j++) {
        float4 v[UN];
#pragma unroll
        for (uint32_t u = 0; u < UN; u++) {
          const uint32_t i = i0 + u * STEP;
          v[u] = i < hi ? __ldcv(reinterpret_cast<const float4 *>(mine + (size_t)j * s.max_n + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (uint32_t u = 0; u < UN; u++)
          acc[u].x = __fadd_rn(acc[u].x, v[u].x), acc[u].y = __fadd_rn(acc[u].y, v[u].y), acc[u].z = __fadd_rn(acc[u].z, v[u].z),
          acc[u].w = __fadd_rn(acc[u].w, v[u].w);
      }
#pragma unroll
      for (uint32_t u = 0; u < UN; u++) {
        const uint32_t i = i0 + u * STEP;
        if (i < hi) *reinterpret_cast<float4 *>(out + i) = acc[u];
      }
    }
  }
  // ---- the last CTA of the call advances the epoch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(s.done, 1u) == gridDim.x - 1u) {
      *s.done = 0u;
      *(volatile uint32_t *)s.epoch = k;
    }
  }
}


constexpr int ARN_MAX_THREADS = 1024;
constexpr int ARN_CL = 8, ARN_CL_THREADS = 128;  // the cluster form: 8 CTAs of 128 threads

// x (= res, may alias out) + the ranks' partials in rank order, then y = x * rsqrt(mean x^2 + eps) * w
// and the Q8 copy of y (the same arithmetic as the RMSNorm kernel and the norm tail of the GEMV).
// Thread t owns elements 4 (t + all threads * it) .. + 3; eight neighbouring threads hold one Q8 block.
// PEERS: how many ranks' words a thread polls together (4: worlds of up to four ranks; 8: larger worlds, all seven peers'
// loads in flight at once: one trip to L2 per poll instead of two).
// CL = 1: one CTA. CL = ARN_CL: one thread-block cluster of CL CTAs, each polling, summing, normalising and quantising
// its own columns; only the sum of squares crosses CTAs (distributed shared memory, one cluster barrier). What a rank
// receives grows with the world (world - 1 rows of 8-byte words: 229 KB at 8 ranks of a 4096-float row), and one SM's
// path to L2 carries that in microseconds; eight SMs take an eighth each.
template <int ITERS, int ARN_THREADS, int PEERS, int CL>
__global__ void __launch_bounds__(ARN_THREADS) ar_norm_kernel(const ArDev s, const float *part, const float *res, float *out, const float *norm_w, float eps,
                                                              float *xn, uint8_t *xq, uint32_t n, uint32_t *err, int pushed, int early) {
  __shared__ float red[32 + ARN_CL];
  const int tid = CL > 1 ? (int)(blockIdx.x * ARN_THREADS + threadIdx.x) : (int)threadIdx.x;  // the thread's place in the vector
  constexpr int ALL = ARN_THREADS * CL;
  float4 acc[ITERS], mine[ITERS], w4[ITERS];
  if (CL > 1) cluster_arrive();
  pdl_launch_dependents();
  // ahead of the dependency wait: the norm weights (constant) and, when the kernel before this one releases its
  // dependents late (`early`), everything older than that kernel: the epoch and the residual stream
#pragma unroll
  for (int it = 0; it < ITERS; it++) {
    const uint32_t i = 4u * (tid + ALL * it);
    acc[it] = w4[it] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < n && norm_w) w4[it] = *reinterpret_cast<const float4 *>(norm_w + i);
    if (i < n && early) acc[it] = *reinterpret_cast<const float4 *>(res + i);
  }
  uint32_t k = 0u;
  if (early) k = *(volatile uint32_t *)s.epoch + 1u;
  pdl_wait();
  if (!early) k = *(volatile uint32_t *)s.epoch + 1u;
  const uint32_t par = k & 1u;
#pragma unroll
  for (int it = 0; it < ITERS; it++) {
    const uint32_t i = 4u * (tid + ALL * it);
    mine[it] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < n) {
      mine[it] = *reinterpret_cast<const float4 *>(part + i);
      const uint32_t pw[4] = {__float_as_uint(mine[it].x), __float_as_uint(mine[it].y), __float_as_uint(mine[it].z), __float_as_uint(mine[it].w)};
      for (uint32_t j = 0; j < s.world && !pushed; j++) {  // pushed: the producing GEMV has already delivered its rows
        if (j == s.rank) continue;
        ll_store4(s.ll[j] + ((size_t)par * s.world + s.rank) * s.max_n + i, k, pw);
      }
      if (!early) acc[it] = *reinterpret_cast<const float4 *>(res + i);
    }
  }
  // ---- the sum, in rank order; peers' words are polled in place, up to four peers' loads in flight together.
  // If an earlier kernel of this step already gave up on a peer, one look at the slots is all this one takes.
  // (the error word is looked at only once a poll has come back empty: nothing on the path of a step that runs well)
  bool gave_up = false, looked = false;
  const uint64_t t0 = ar_now();
  const unsigned long long *my = s.ll[s.rank] + (size_t)par * s.world * s.max_n;
#pragma unroll
  for (int it = 0; it < ITERS; it++) {
    const uint32_t i = 4u * (tid + ALL * it);
    if (i >= n) continue;
    for (uint32_t j0 = 0; j0 < s.world; j0 += PEERS) {
      unsigned long long v[PEERS][4];
      for (;;) {
        bool all = true;
#pragma unroll
        for (int q = 0; q < PEERS; q++) {
          const uint32_t j = j0 + q;
          if (j < s.world && j != s.rank) ll_load4(my + (size_t)j * s.max_n + i, v[q]);
        }
#pragma unroll
        for (int q = 0; q < PEERS; q++) {
          const uint32_t j = j0 + q;
          if (j < s.world && j != s.rank) {
#pragma unroll
            for (int c = 0; c < 4; c++) all = all && (uint32_t)(v[q][c] >> 32) == k;
          }
        }
        if (all) break;
        if (!looked) looked = true, gave_up = err && *(volatile uint32_t *)err != 0u;
        if (gave_up || ar_now() - t0 > AR_WAIT_NS) {
          gave_up = true;
          break;
        }
      }
#pragma unroll
      for (int q = 0; q < PEERS; q++) {
        const uint32_t j = j0 + q;
        if (j >= s.world) continue;
        float4 pv = mine[it];
        if (j != s.rank)
          pv = make_float4(__uint_as_float((uint32_t)v[q][0]), __uint_as_float((uint32_t)v[q][1]), __uint_as_float((uint32_t)v[q][2]),
                           __uint_as_float((uint32_t)v[q][3]));
        acc[it].x = __fadd_rn(acc[it].x, pv.x), acc[it].y = __fadd_rn(acc[it].y, pv.y);
        acc[it].z = __fadd_rn(acc[it].z, pv.z), acc[it].w = __fadd_rn(acc[it].w, pv.w);
      }
    }
  }
  if (gave_up && err) atomicExch(err, 3u);
#pragma unroll
  for (int it = 0; it < ITERS; it++) {
    const uint32_t i = 4u * (tid + ALL * it);
    if (i < n) *reinterpret_cast<float4 *>(out + i) = acc[it];
  }
  if (CL > 1) cluster_wait();  // every CTA of the cluster runs (and has read the epoch) from here on
  if (norm_w) norm_quant_vec<ITERS, ARN_THREADS, CL>(acc, w4, n, eps, xn, xq, red);  // (norm_w is the same in every CTA: all reach its cluster barrier)
  if (tid == 0) *(volatile uint32_t *)s.epoch = k;  // read by later kernels only, and those start after every CTA of this one
}

// One warp: every rank's (logit, global index) of its local argmax to every rank; the largest logit wins, ties
// go to the smaller index (what one argmax over the whole vocabulary gives). result[0] = the winning index.
__global__ void __launch_bounds__(32) ar_argmax_kernel(const ArDev s, const float *logits, uint32_t *result, uint32_t vocab_offset, uint32_t *err) {
  pdl_prologue();
  const uint32_t k = *(volatile uint32_t *)s.epoch + 1u, par = k & 1u;
  const uint32_t lane = threadIdx.x;
  const uint32_t li = result[0], lp = result[1];  // local index and its probability within this rank's slice
  const float lv = logits[li];
  if (lane < s.world && lane != s.rank) {
    unsigned long long *dst = s.ll[lane] + ((size_t)par * s.world + s.rank) * s.max_n;
    ll_store(dst, k, __float_as_uint(lv));
    ll_store(dst + 1, k, li + vocab_offset);
    ll_store(dst + 2, k, lp);
    ll_store(dst + 3, k, 0u);
  }
  float v = -INFINITY, pr = 0.0f;
  uint32_t idx = 0xFFFFFFFFu;
  bool gave_up = err && *(volatile uint32_t *)err != 0u;
  if (lane == s.rank) {
    v = lv, idx = li + vocab_offset, pr = __uint_as_float(lp);
  } else if (lane < s.world) {
    uint32_t wv[4];
    if (ll_wait4(s.ll[s.rank] + ((size_t)par * s.world + lane) * s.max_n, k, wv, &gave_up, ar_now()))
      v = __uint_as_float(wv[0]), idx = wv[1], pr = __uint_as_float(wv[2]);
  }
  if (gave_up && err) atomicExch(err, 3u);
  float bv = v;
  uint32_t bi = idx;
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
    const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
  }
  // softmax denominator over all slices, relative to the winning logit: a slice's own is 1 / its probability
  float den = pr > 0.0f ? expf(v - bv) / pr : 0.0f;
  den = warp_sum_all(den);
  if (lane == 0) {
    result[0] = bi;
    result[1] = __float_as_uint(den > 0.0f ? 1.0f / den : 0.0f);
    *(volatile uint32_t *)s.epoch = k;
  }
}

}  // namespace ieb

using namespace ieb;

struct ie_b200_allreduce {
  ArDev d = {};
  char *base = nullptr;  // one allocation (one IPC handle): slots, flags, low-latency slots
  size_t off_flags = 0, off_ll = 0;
  uint32_t *epoch = nullptr;
  void *opened[AR_MAX_RANKS] = {};
  int n_opened = 0;
  bool connected = false;
};

static inline size_t up256(size_t n) { return (n + 255u) & ~(size_t)255u; }

namespace ieb {
// What a kernel outside this file needs to exchange rows through the state's low-latency slots (step_kernel.cu).
void ar_push_info(const ie_b200_allreduce *a, ArPush *out) {
  *out = ArPush();
  if (!a) return;
  for (uint32_t j = 0; j < a->d.world; j++) out->ll[j] = a->d.ll[j];
  out->epoch = a->d.epoch, out->rank = a->d.rank, out->world = a->d.world, out->max_n = a->d.max_n;
}
bool ar_connected(const ie_b200_allreduce *a) { return a && a->connected; }
}  // namespace ieb

extern "C" int ie_b200_ar_create(uint32_t rank, uint32_t world, uint32_t max_floats, ie_b200_allreduce **out) {
  if (!out || world < 1 || world > (uint32_t)AR_MAX_RANKS || rank >= world || max_floats == 0 || max_floats % 4u)
    return fail(IE_B200_E_ARG, "ie_b200_ar_create: rank %u of %u, %u floats (1..8 ranks, a multiple of 4 floats)", rank, world, max_floats);
  ie_b200_allreduce *a = new ie_b200_allreduce();
  const size_t sb = up256((size_t)2 * world * max_floats * 4u), fb = up256((size_t)world * AR_MAX_CTAS * 4u);
  const size_t lb = up256((size_t)2 * world * max_floats * 8u);
  a->off_flags = sb, a->off_ll = sb + fb;
  cudaError_t e = cudaMalloc(&a->base, sb + fb + lb);
  if (e == cudaSuccess) e = cudaMalloc(&a->epoch, 8);
  if (e == cudaSuccess) e = cudaMemset(a->base, 0, sb + fb + lb);
  if (e == cudaSuccess) e = cudaMemset(a->epoch, 0, 8);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(a->base), cudaFree(a->epoch);
    delete a;
    return cuda_fail(e, "ie_b200_ar_create");
  }
  a->d.rank = rank, a->d.world = world, a->d.max_n = max_floats;
  a->d.epoch = a->epoch, a->d.done = a->epoch + 1;
  a->d.slots[rank] = reinterpret_cast<float *>(a->base), a->d.flags[rank] = reinterpret_cast<uint32_t *>(a->base + a->off_flags);
  a->d.ll[rank] = reinterpret_cast<unsigned long long *>(a->base + a->off_ll);
  a->connected = world == 1;
  *out = a;
  return IE_B200_OK;
}

extern "C" int ie_b200_ar_handles(ie_b200_allreduce *a, void *h_out128) {
  if (!a || !h_out128) return fail(IE_B200_E_ARG, "ie_b200_ar_handles: NULL argument");
  cudaIpcMemHandle_t h;
  IEB_CUDA(cudaIpcGetMemHandle(&h, a->base));
  static_assert(sizeof(h) == 64, "an IPC handle is 64 bytes");
  memset(h_out128, 0, 128);
  memcpy(h_out128, &h, sizeof h);
  return IE_B200_OK;
}

extern "C" int ie_b200_ar_connect(ie_b200_allreduce *a, const void *h_all) {
  if (!a || !h_all) return fail(IE_B200_E_ARG, "ie_b200_ar_connect: NULL argument");
  if (a->connected) return IE_B200_OK;
  const char *blobs = static_cast<const char *>(h_all);
  for (uint32_t j = 0; j < a->d.world; j++) {
    if (j == a->d.rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, blobs + (size_t)128 * j, sizeof h);
    void *pb = nullptr;
    IEB_CUDA(cudaIpcOpenMemHandle(&pb, h, cudaIpcMemLazyEnablePeerAccess));
    a->opened[a->n_opened++] = pb;
    char *b = static_cast<char *>(pb);
    a->d.slots[j] = reinterpret_cast<float *>(b), a->d.flags[j] = reinterpret_cast<uint32_t *>(b + a->off_flags);
    a->d.ll[j] = reinterpret_cast<unsigned long long *>(b + a->off_ll);
  }
  a->connected = true;
  return IE_B200_OK;
}

extern "C" int ie_b200_ar_connect_local(ie_b200_allreduce *a, ie_b200_allreduce *const *all) {
  if (!a || !all) return fail(IE_B200_E_ARG, "ie_b200_ar_connect_local: NULL argument");
  for (uint32_t j = 0; j < a->d.world; j++) {
    if (j == a->d.rank) continue;
    const ie_b200_allreduce *p = all[j];
    if (!p || p->d.world != a->d.world || p->d.rank != j || p->d.max_n != a->d.max_n)
      return fail(IE_B200_E_ARG, "ie_b200_ar_connect_local: state %u does not belong to this world", j);
    a->d.slots[j] = reinterpret_cast<float *>(p->base), a->d.flags[j] = reinterpret_cast<uint32_t *>(p->base + p->off_flags);
    a->d.ll[j] = reinterpret_cast<unsigned long long *>(p->base + p->off_ll);
  }
  a->connected = true;
  return IE_B200_OK;
}

extern "C" int ie_b200_ar_allreduce_add(ie_b200_allreduce *a, const float *d_part, const float *d_res, float *d_out, uint32_t n, uint32_t *d_err,
                                        void *stream) {
  if (!a || !d_part || !d_out) return fail(IE_B200_E_ARG, "ie_b200_ar_allreduce_add: NULL argument");
  if (!a->connected) return fail(IE_B200_E_STATE, "ie_b200_ar_allreduce_add: peers not connected");
  if (n == 0 || n % 4u || n > a->d.max_n) return fail(IE_B200_E_SIZE, "ie_b200_ar_allreduce_add: %u floats (a multiple of 4, at most %u)", n, a->d.max_n);
  if (!aligned16(d_part) || !aligned16(d_out) || (d_res && !aligned16(d_res))) return fail(IE_B200_E_ARG, "ie_b200_ar_allreduce_add: 16-byte alignment");
  unsigned grid = (n / 4u + AR_THREADS - 1) / AR_THREADS;  // one float4 per thread
  if (grid > (unsigned)AR_MAX_CTAS) grid = AR_MAX_CTAS;
  IEB_LAUNCH_PDL("allreduce_add_kernel", allreduce_add_kernel, dim3(grid), dim3(AR_THREADS), 0, static_cast<cudaStream_t>(stream), a->d, d_part, d_res,
                 d_out, n, d_err);
  return IE_B200_OK;
}

// Which form of the reduction kernel a row takes: the cluster once a rank receives more than one SM fetches quickly
// (worlds of four ranks and more, rows of a real model). Measured on the 8B-class model, one CTA against the cluster:
// 2 ranks 4.1 / 4.5 us per stop (the cluster's barrier costs more than its CTAs save), 4 ranks 0.970 / 0.942 ms per
// step of 65 stops, 8 ranks 7.8 / 5.7 us per stop. IE_B200_AR_NORM=single / cluster: one form for every world (for comparison).
static bool ar_norm_cluster_on(uint32_t world, uint32_t n) {
  static const int mode = [] {
    const char *v = getenv("IE_B200_AR_NORM");
    return !v ? 0 : !strcmp(v, "single") ? 1 : !strcmp(v, "cluster") ? 2 : 0;
  }();
  if (mode == 1 || n < 1024u) return false;
  return mode == 2 || world > 2u;
}

// d_res: what the ranks' partials are added to (NULL: d_x itself, in place); d_x receives the sum.
static int ar_norm_launch(ie_b200_allreduce *a, const float *d_part, const float *d_res, float *d_x, const float *d_norm_w, float eps, float *d_xn,
                          void *d_xq, uint32_t n, uint32_t *d_err, void *stream, int pushed, int early = 0) {
  if (!a || !d_part || !d_x || !d_norm_w) return fail(IE_B200_E_ARG, "ie_b200_ar_allreduce_norm: NULL argument");
  if (!d_res) d_res = d_x;
  if (!a->connected) return fail(IE_B200_E_STATE, "ie_b200_ar_allreduce_norm: peers not connected");
  if (n == 0 || n % 32u || n > a->d.max_n || n > 4u * 4u * ARN_MAX_THREADS)
    return fail(IE_B200_E_SIZE, "ie_b200_ar_allreduce_norm: %u floats (a multiple of 32, at most %u)", n, a->d.max_n < 16384u ? a->d.max_n : 16384u);
  if (!aligned16(d_part) || !aligned16(d_x) || !aligned16(d_res) || !aligned16(d_norm_w) || (d_xn && !aligned16(d_xn)) || (d_xq && !aligned16(d_xq)))
    return fail(IE_B200_E_ARG, "ie_b200_ar_allreduce_norm: 16-byte alignment");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t *xq = static_cast<uint8_t *>(d_xq);
#define IEB_ARN(IT, TH, PE)                                                                                                                  \
  IEB_LAUNCH_PDL("ar_norm_kernel", (ar_norm_kernel<IT, TH, PE, 1>), dim3(1), dim3(TH), 0, st, a->d, d_part, d_res, d_x, d_norm_w, eps, d_xn, xq, n, d_err, \
                 pushed, early)
#define IEB_ARN_CL(IT, PE)                                                                                                                    \
  do {                                                                                                                                       \
    cudaError_t e_ = launch_pdl_cluster(ar_norm_kernel<IT, ARN_CL_THREADS, PE, ARN_CL>, dim3(ARN_CL), dim3(ARN_CL_THREADS), 0, st, ARN_CL, a->d, d_part, \
                                        d_res, d_x, d_norm_w, eps, d_xn, xq, n, d_err, pushed, early);                                       \
    count_launch();                                                                                                                          \
    if (e_ != cudaSuccess) return cuda_fail(e_, "ar_norm_kernel (cluster)");                                                                 \
  } while (0)
  if (ar_norm_cluster_on(a->d.world, n)) {
    const uint32_t iters = (n + 4u * ARN_CL * ARN_CL_THREADS - 1u) / (4u * ARN_CL * ARN_CL_THREADS);
    if (a->d.world > 4u) {
      if (iters <= 1) IEB_ARN_CL(1, 8);
      else if (iters <= 2) IEB_ARN_CL(2, 8);
      else IEB_ARN_CL(4, 8);
    } else {
      if (iters <= 1) IEB_ARN_CL(1, 4);
      else if (iters <= 2) IEB_ARN_CL(2, 4);
      else IEB_ARN_CL(4, 4);
    }
  } else if (a->d.world > 4u) {  // 512 threads, all peers polled together
    const uint32_t iters = (n + 4u * 512u - 1u) / (4u * 512u);
    if (iters <= 1) IEB_ARN(1, 512, 8);
    else if (iters <= 2) IEB_ARN(2, 512, 8);
    else if (iters <= 4) IEB_ARN(4, 512, 8);
    else IEB_ARN(8, 512, 8);
  } else {
    const uint32_t iters = (n + 4u * 1024u - 1u) / (4u * 1024u);
    if (iters <= 1) IEB_ARN(1, 1024, 4);
    else if (iters <= 2) IEB_ARN(2, 1024, 4);
    else IEB_ARN(4, 1024, 4);
  }
#undef IEB_ARN
#undef IEB_ARN_CL
  return IE_B200_OK;
}

extern "C" int ie_b200_ar_allreduce_norm(ie_b200_allreduce *a, const float *d_part, float *d_x, const float *d_norm_w, float eps, float *d_xn, void *d_xq,
                                         uint32_t n, uint32_t *d_err, void *stream) {
  return ar_norm_launch(a, d_part, nullptr, d_x, d_norm_w, eps, d_xn, d_xq, n, d_err, stream, 0);
}

namespace ieb {
// The K-split GEMV that pushes its rows, with the activations either a Q8 buffer (act.xq) or an f32 vector quantised in the
// prologue (act.xf, plain = true).
int gemv_push_act(ie_b200_allreduce *a, int kind, const void *d_w, uint32_t rows, uint32_t cols, const ActSrc &act, bool plain, float *d_part, cudaStream_t st) {
  if (!a || !d_w || !d_part || !(plain ? (const void *)act.xf : (const void *)act.xq)) return fail(IE_B200_E_ARG, "ie_b200_gemv_push: NULL argument");
  if (!a->connected) return fail(IE_B200_E_STATE, "ie_b200_gemv_push: peers not connected");
  if (kind != IE_B200_MAT_Q4 && kind != IE_B200_MAT_Q8 && kind != IE_B200_MAT_Q4K && kind != IE_B200_MAT_Q6K)
    return fail(IE_B200_E_ARG, "ie_b200_gemv_push: matrix kind %d", kind);
  if (rows == 0 || rows % 32u || rows > a->d.max_n) return fail(IE_B200_E_SIZE, "ie_b200_gemv_push: %u rows (a multiple of 32, at most %u)", rows, a->d.max_n);
  if (cols == 0 || cols % ((kind == IE_B200_MAT_Q4 || kind == IE_B200_MAT_Q8) ? 32u : 256u) || cols / 32u > 1024u)
    return fail(IE_B200_E_SIZE, "ie_b200_gemv_push: %u columns", cols);
  if (!aligned16(d_w) || !aligned16(plain ? (const void *)act.xf : (const void *)act.xq)) return fail(IE_B200_E_ARG, "ie_b200_gemv_push: 16-byte alignment");
  ArPush push;
  ar_push_info(a, &push);
  // the GEMV releases its dependents only after its own dependency wait: when the reduction kernel starts, everything
  // before the GEMV is complete, and it may fetch the epoch and the residual stream while the GEMV still runs
  return gemv_direct(kind, d_w, rows, cols, act, plain, d_part, nullptr, nullptr, nullptr, nullptr, st, &push, true);
}
}  // namespace ieb

extern "C" int ie_b200_gemv_push(ie_b200_allreduce *a, int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_xq, float *d_part, void *stream) {
  ActSrc act0 = {};
  act0.xq = static_cast<const uint8_t *>(d_xq);
  return gemv_push_act(a, kind, d_w, rows, cols, act0, false, d_part, static_cast<cudaStream_t>(stream));
}

namespace ieb {
// The reduction behind a GEMV that pushed its rows (pushed) or behind anything else (the kernel pushes d_part itself);
// d_res NULL: onto d_x in place.
int ar_norm_reduce(ie_b200_allreduce *a, const float *d_part, const float *d_res, float *d_x, const float *d_norm_w, float eps, float *d_xn, void *d_xq,
                   uint32_t n, uint32_t *d_err, cudaStream_t st, bool pushed) {
  return ar_norm_launch(a, d_part, d_res, d_x, d_norm_w, eps, d_xn, d_xq, n, d_err, st, pushed ? 1 : 0, pushed ? 1 : 0);
}
}  // namespace ieb

extern "C" int ie_b200_ar_reduce_norm(ie_b200_allreduce *a, const float *d_part, float *d_x, const float *d_norm_w, float eps, float *d_xn, void *d_xq,
                                      uint32_t n, uint32_t *d_err, void *stream) {
  return ar_norm_launch(a, d_part, nullptr, d_x, d_norm_w, eps, d_xn, d_xq, n, d_err, stream, 1, 0);
}

extern "C" int ie_b200_gemv_allreduce_norm(ie_b200_allreduce *a, int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_xq, float *d_part,
                                           float *d_x, const float *d_norm_w, float eps, float *d_xn, void *d_xq_out, uint32_t *d_err, void *stream) {
  if (!d_x || !d_norm_w) return fail(IE_B200_E_ARG, "ie_b200_gemv_allreduce_norm: NULL argument");
  if (int r = ie_b200_gemv_push(a, kind, d_w, rows, cols, d_xq, d_part, stream)) return r;
  return ar_norm_launch(a, d_part, nullptr, d_x, d_norm_w, eps, d_xn, d_xq_out, rows, d_err, stream, 1, 1);
}

extern "C" int ie_b200_ar_argmax(ie_b200_allreduce *a, const float *d_logits, uint32_t *d_result, uint32_t vocab_offset, uint32_t *d_err, void *stream) {
  if (!a || !d_logits || !d_result) return fail(IE_B200_E_ARG, "ie_b200_ar_argmax: NULL argument");
  if (!a->connected) return fail(IE_B200_E_STATE, "ie_b200_ar_argmax: peers not connected");
  IEB_LAUNCH_PDL("ar_argmax_kernel", ar_argmax_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), a->d, d_logits, d_result, vocab_offset,
                 d_err);
  return IE_B200_OK;
}

extern "C" void ie_b200_ar_destroy(ie_b200_allreduce *a) {
  if (!a) return;
  cudaDeviceSynchronize();
  for (int i = 0; i < a->n_opened; i++) cudaIpcCloseMemHandle(a->opened[i]);
  cudaFree(a->base), cudaFree(a->epoch);
  delete a;
}
