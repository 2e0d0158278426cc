// allreduce.cu -- the latency-bound all-reduce of a tensor-parallel decode
// step: the sum over ranks of a dim-float partial (16-20 KB) after every
// K-split GEMV, fused with the residual add. One process per GPU; every rank
// maps the other ranks' receive buffers with CUDA IPC and the kernel moves the
// data itself with plain peer stores over NVLink (no multicast, no TMA):
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
#include <cstring>

#include "common.cuh"
#include "ie_b200_tp.h"

namespace ieb {

constexpr int AR_MAX_RANKS = 8, AR_THREADS = 256, AR_MAX_CTAS = 32;
constexpr uint64_t AR_WAIT_NS = 2000000000ull;  // 2 s

struct ArDev {
  float *slots[AR_MAX_RANKS];     // rank j's receive buffer: [2][world][max_n] floats
  uint32_t *flags[AR_MAX_RANKS];  // rank j's flags: [world][AR_MAX_CTAS]
  uint32_t *epoch;                // local: number of completed calls
  uint32_t *done;                 // local: CTAs that finished the current call
  uint32_t rank, world, max_n;
};

__device__ __forceinline__ uint64_t ar_now() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__global__ void __launch_bounds__(AR_THREADS) allreduce_add_kernel(const ArDev s, const float *part, const float *res, float *out, uint32_t n,
                                                                   uint32_t *err) {
  pdl_prologue();
  __shared__ uint32_t ok;
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
      if (ar_now() - t0 > AR_WAIT_NS) {
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
    for (uint32_t i = lo + 4u * threadIdx.x; i < hi; i += 4u * AR_THREADS) {
      float4 acc = res ? *reinterpret_cast<const float4 *>(res + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      for (uint32_t j = 0; j < s.world; j++) {
        const float4 v = __ldcv(reinterpret_cast<const float4 *>(mine + (size_t)j * s.max_n + i));
        acc.x = __fadd_rn(acc.x, v.x), acc.y = __fadd_rn(acc.y, v.y), acc.z = __fadd_rn(acc.z, v.z), acc.w = __fadd_rn(acc.w, v.w);
      }
      *reinterpret_cast<float4 *>(out + i) = acc;
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

}  // namespace ieb

using namespace ieb;

struct ie_b200_allreduce {
  ArDev d = {};
  float *slots = nullptr;
  uint32_t *flags = nullptr, *epoch = nullptr;
  void *opened[2 * AR_MAX_RANKS] = {};
  int n_opened = 0;
  bool connected = false;
};

extern "C" int ie_b200_ar_create(uint32_t rank, uint32_t world, uint32_t max_floats, ie_b200_allreduce **out) {
  if (!out || world < 1 || world > (uint32_t)AR_MAX_RANKS || rank >= world || max_floats == 0 || max_floats % 4u)
    return fail(IE_B200_E_ARG, "ie_b200_ar_create: rank %u of %u, %u floats (1..8 ranks, a multiple of 4 floats)", rank, world, max_floats);
  ie_b200_allreduce *a = new ie_b200_allreduce();
  const size_t sb = (size_t)2 * world * max_floats * 4u, fb = (size_t)world * AR_MAX_CTAS * 4u;
  cudaError_t e = cudaMalloc(&a->slots, sb);
  if (e == cudaSuccess) e = cudaMalloc(&a->flags, fb);
  if (e == cudaSuccess) e = cudaMalloc(&a->epoch, 8);
  if (e == cudaSuccess) e = cudaMemset(a->slots, 0, sb);
  if (e == cudaSuccess) e = cudaMemset(a->flags, 0, fb);
  if (e == cudaSuccess) e = cudaMemset(a->epoch, 0, 8);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(a->slots), cudaFree(a->flags), cudaFree(a->epoch);
    delete a;
    return cuda_fail(e, "ie_b200_ar_create");
  }
  a->d.rank = rank, a->d.world = world, a->d.max_n = max_floats;
  a->d.epoch = a->epoch, a->d.done = a->epoch + 1;
  a->d.slots[rank] = a->slots, a->d.flags[rank] = a->flags;
  a->connected = world == 1;
  *out = a;
  return IE_B200_OK;
}

extern "C" int ie_b200_ar_handles(ie_b200_allreduce *a, void *h_out128) {
  if (!a || !h_out128) return fail(IE_B200_E_ARG, "ie_b200_ar_handles: NULL argument");
  cudaIpcMemHandle_t h[2];
  IEB_CUDA(cudaIpcGetMemHandle(&h[0], a->slots));
  IEB_CUDA(cudaIpcGetMemHandle(&h[1], a->flags));
  static_assert(sizeof(h) == 128, "two IPC handles are 128 bytes");
  memcpy(h_out128, h, sizeof h);
  return IE_B200_OK;
}

extern "C" int ie_b200_ar_connect(ie_b200_allreduce *a, const void *h_all) {
  if (!a || !h_all) return fail(IE_B200_E_ARG, "ie_b200_ar_connect: NULL argument");
  const cudaIpcMemHandle_t *h = static_cast<const cudaIpcMemHandle_t *>(h_all);
  for (uint32_t j = 0; j < a->d.world; j++) {
    if (j == a->d.rank) continue;
    void *ps = nullptr, *pf = nullptr;
    IEB_CUDA(cudaIpcOpenMemHandle(&ps, h[2 * j], cudaIpcMemLazyEnablePeerAccess));
    a->opened[a->n_opened++] = ps;
    IEB_CUDA(cudaIpcOpenMemHandle(&pf, h[2 * j + 1], cudaIpcMemLazyEnablePeerAccess));
    a->opened[a->n_opened++] = pf;
    a->d.slots[j] = static_cast<float *>(ps), a->d.flags[j] = static_cast<uint32_t *>(pf);
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

extern "C" void ie_b200_ar_destroy(ie_b200_allreduce *a) {
  if (!a) return;
  cudaDeviceSynchronize();
  for (int i = 0; i < a->n_opened; i++) cudaIpcCloseMemHandle(a->opened[i]);
  cudaFree(a->slots), cudaFree(a->flags), cudaFree(a->epoch);
  delete a;
}
