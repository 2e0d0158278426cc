// common.cuh -- shared helpers of the sm_100a kernels: error plumbing, the
// streaming-layout geometry, cache-hinted loads and the integer block dots.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "ie_b200.h"

namespace ieb {

// ---- host-side error plumbing (abi.cu) ----
int fail(int code, const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);
void count_launch(unsigned n = 1);
int sm_count();
// Programmatic dependent launch is on unless the environment says IE_B200_PDL=0 (then every launch is a
// plain stream-ordered launch and the griddepcontrol instructions in the kernels do nothing).
bool pdl_enabled();
// Raise (never lower) a kernel's opt-in dynamic shared memory limit on the current device. Monotone, so that
// launches already captured into a CUDA graph with a larger size stay valid when a smaller launch follows.
int ensure_dynamic_smem(const void *func, size_t bytes);
// Hints from the engine to the next launch made on this thread (read and cleared by take_hints()):
//   late_trigger        the kernel lets its dependents start only after its own dependency wait, so a dependent
//                       that starts knows that everything before this kernel has completed;
//   after_late_trigger  the kernel before this one was launched with late_trigger.
//   swi_h               the GEMV's rows are interleaved (gate_i, up_i) pairs: write silu(gate) * up to swi_h[i] instead of
//                       the two rows, count arrivals per 32 outputs in swi_count (zero between launches), and let the
//                       warp that completes a block write its Q8 copy into swi_q.
struct LaunchHints {
  bool late_trigger = false, after_late_trigger = false;
  float *swi_h = nullptr;
  uint8_t *swi_q = nullptr;
  uint32_t *swi_count = nullptr;
};
void set_hints(const LaunchHints &h);
bool gemv_uses_ring();  // IE_B200_GEMV=ring selects the bulk-copy ring kernel instead of the direct one (gemv_stream.cu)
LaunchHints take_hints();

#define IEB_CUDA(call)                                   \
  do {                                                   \
    cudaError_t e_ = (call);                             \
    if (e_ != cudaSuccess) return ieb::cuda_fail(e_, #call); \
  } while (0)

// After a kernel launch: count it and surface a launch error.
#define IEB_LAUNCHED(what)                                \
  do {                                                    \
    ieb::count_launch();                                  \
    cudaError_t e_ = cudaPeekAtLastError();               \
    if (e_ != cudaSuccess) return ieb::cuda_fail(e_, what); \
  } while (0)

static inline bool aligned16(const void *p) { return ((uintptr_t)p & 15u) == 0; }

#ifdef __CUDACC__
// Launch with programmatic dependent launch: the kernel may start while its predecessor in the stream
// is still running. Only for kernels that call pdl_wait() before touching anything a predecessor wrote.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at, cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#define IEB_LAUNCH_PDL(what, kernel, grid, block, smem, st, ...)                                  \
  do {                                                                                            \
    cudaError_t e_ = ieb::launch_pdl(kernel, grid, block, smem, st, __VA_ARGS__);                 \
    ieb::count_launch();                                                                          \
    if (e_ != cudaSuccess) return ieb::cuda_fail(e_, what);                                       \
  } while (0)
#endif

// ---- streaming layout geometry (see ie_b200.h) ----
__host__ __device__ inline size_t round16(size_t n) { return (n + 15u) & ~(size_t)15u; }
__host__ __device__ inline size_t row_bytes_of(int kind, uint32_t cols) {
  const size_t nb = cols / 32u;
  switch (kind) {
    case IE_B200_MAT_Q4: return round16(nb * 18u);
    case IE_B200_MAT_Q4K: return nb * 16u + (nb / 8u) * 16u;
    case IE_B200_MAT_Q6K: return round16(nb * 26u + (nb / 8u) * 2u);
    default: return (size_t)cols * 4u;
  }
}

// ---- device helpers ----
#ifdef __CUDACC__

// ---- device timeline (only in builds with -DIEB_TIMELINE; otherwise tl_mark() is nothing) ----
// The first and the last CTA of a kernel record (global timer, kernel id, phase) into a per-source-file
// buffer; ie_b200_timeline_read() (abi.cu) gathers the buffers. Phase 0 = entry, 1 = past the dependency
// wait, 15 = exit; kernels add their own in between.
enum { TL_GEMV = 1, TL_ATTN, TL_SWIGLU, TL_ROPE, TL_RMSNORM, TL_EMBED, TL_ARGMAX, TL_ARGMAX_MERGE, TL_QUANT, TL_ALLREDUCE, TL_ADVANCE, TL_GEMV_SIMPLE };
#ifdef IEB_TIMELINE
struct TlRec {
  unsigned long long t;
  uint32_t tag, cta;
};
// A record goes to the slot its own time stamp names (32 ns per slot, a window of 8 ms): one plain store, no
// atomic whose round trip would stretch the phase being measured. Two marks in the same 32 ns lose one.
constexpr uint32_t TL_CAP = 1u << 18;
static __device__ TlRec tl_buf[TL_CAP];
__device__ __forceinline__ void tl_put(uint32_t kernel, uint32_t phase, uint32_t who) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  tl_buf[(uint32_t)(t >> 5) & (TL_CAP - 1u)] = TlRec{t, kernel << 8 | phase, who};
}
__device__ __forceinline__ void tl_mark(uint32_t kernel, uint32_t phase) {
  const bool first = (blockIdx.x | blockIdx.y | blockIdx.z) == 0u;
  const bool last = blockIdx.x == gridDim.x - 1u && blockIdx.y == gridDim.y - 1u && blockIdx.z == gridDim.z - 1u;
  if ((threadIdx.x | threadIdx.y) == 0u && (first || last)) tl_put(kernel, phase, first ? 0u : 1u);
}
// one record from the calling thread, whatever its CTA
__device__ __forceinline__ void tl_mark_any(uint32_t kernel, uint32_t phase) { tl_put(kernel, phase, 2u); }
#else
__device__ __forceinline__ void tl_mark(uint32_t, uint32_t) {}
__device__ __forceinline__ void tl_mark_any(uint32_t, uint32_t) {}
#endif

#ifdef IEB_TIMELINE
// host side: every source file registers a reader of its own buffer
void tl_register(uint32_t (*reader)(void *out, uint32_t cap));
static uint32_t tl_read_tu(void *out, uint32_t cap) {
  static TlRec *host = nullptr;
  if (!host) host = static_cast<TlRec *>(malloc(sizeof(TlRec) * TL_CAP));
  if (!host || cudaMemcpyFromSymbol(host, tl_buf, sizeof(TlRec) * TL_CAP) != cudaSuccess) return 0;
  uint32_t n = 0;
  for (uint32_t i = 0; i < TL_CAP && n < cap; i++)
    if (host[i].t) static_cast<TlRec *>(out)[n++] = host[i];
  void *dev = nullptr;
  if (cudaGetSymbolAddress(&dev, tl_buf) == cudaSuccess) cudaMemset(dev, 0, sizeof(TlRec) * TL_CAP);
  return n;
}
namespace {
struct TlRegistrar {
  TlRegistrar() { tl_register(&tl_read_tu); }
} tl_registrar;
}  // namespace
#endif

// Programmatic dependent launch: let the next kernel of the stream start (its own pdl_wait keeps it from
// reading our results early), and wait until the previous kernel has completed and its writes are visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Every kernel launched through launch_pdl starts with this.
__device__ __forceinline__ void pdl_prologue(uint32_t tl_kernel = 0) {
  tl_mark(tl_kernel, 0);
  pdl_launch_dependents();
  pdl_wait();
  tl_mark(tl_kernel, 1);
}

// Ask for the 128-byte line at p to be brought into L2 (no register, no wait).
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// 16-byte streaming load of weights that are read once: read-only path, not
// kept in L1.
__device__ __forceinline__ uint4 ld_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ld_stream8(const void *p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint16_t ld_stream2(const void *p) {
  uint16_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_stream_f32(const void *p) {
  float v;
  asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// Sum over the 32 nibbles q (0..15) of q * a. Word k of the weight block
// holds weights 4k..4k+3 in its low nibbles and 16+4k..16+4k+3 in its high
// nibbles; a0 are activation words 0..3, a1 words 4..7. Nibble bytes are
// below 128, so the signed byte product equals the unsigned-by-signed one.
__device__ __forceinline__ int q4_dot(const uint4 &w, const uint4 &a0, const uint4 &a1) {
  int acc = 0;
  acc = __dp4a((int)(w.x & 0x0F0F0F0Fu), (int)a0.x, acc);
  acc = __dp4a((int)((w.x >> 4) & 0x0F0F0F0Fu), (int)a1.x, acc);
  acc = __dp4a((int)(w.y & 0x0F0F0F0Fu), (int)a0.y, acc);
  acc = __dp4a((int)((w.y >> 4) & 0x0F0F0F0Fu), (int)a1.y, acc);
  acc = __dp4a((int)(w.z & 0x0F0F0F0Fu), (int)a0.z, acc);
  acc = __dp4a((int)((w.z >> 4) & 0x0F0F0F0Fu), (int)a1.z, acc);
  acc = __dp4a((int)(w.w & 0x0F0F0F0Fu), (int)a0.w, acc);
  acc = __dp4a((int)((w.w >> 4) & 0x0F0F0F0Fu), (int)a1.w, acc);
  return acc;
}

// One byte-quad of Q6_K values minus 32 as signed bytes: v = nibbles | two
// high bits << 4, then ((v | 0x80808080) - 0x20202020) ^ 0x80808080.
__device__ __forceinline__ int q6_sw(uint32_t nib4, uint32_t hword, int k) {
  const uint32_t v = nib4 | (((hword >> (2 * k)) & 0x03030303u) << 4);
  return (int)(((v | 0x80808080u) - 0x20202020u) ^ 0x80808080u);
}
// The two half dots of a Q6_K sub-block: weights 0..15 against a0, 16..31 against a1.
__device__ __forceinline__ void q6_dots(const uint4 &w, const uint2 &hw, const uint4 &a0, const uint4 &a1, int &d0, int &d1) {
  int s0 = 0, s1 = 0;
  s0 = __dp4a(q6_sw(w.x & 0x0F0F0F0Fu, hw.x, 0), (int)a0.x, s0);
  s0 = __dp4a(q6_sw(w.y & 0x0F0F0F0Fu, hw.x, 1), (int)a0.y, s0);
  s0 = __dp4a(q6_sw(w.z & 0x0F0F0F0Fu, hw.x, 2), (int)a0.z, s0);
  s0 = __dp4a(q6_sw(w.w & 0x0F0F0F0Fu, hw.x, 3), (int)a0.w, s0);
  s1 = __dp4a(q6_sw((w.x >> 4) & 0x0F0F0F0Fu, hw.y, 0), (int)a1.x, s1);
  s1 = __dp4a(q6_sw((w.y >> 4) & 0x0F0F0F0Fu, hw.y, 1), (int)a1.y, s1);
  s1 = __dp4a(q6_sw((w.z >> 4) & 0x0F0F0F0Fu, hw.y, 2), (int)a1.z, s1);
  s1 = __dp4a(q6_sw((w.w >> 4) & 0x0F0F0F0Fu, hw.y, 3), (int)a1.w, s1);
  d0 = s0, d1 = s1;
}

// The 12-bit (sc | mn << 6) field j of a Q4_K super-block header (words y, z, w).
__device__ __forceinline__ uint32_t q4k_field(const uint4 &h, int j) {
  const int o = 12 * j, i = o >> 5, sh = o & 31;
  const uint32_t lo = i == 0 ? h.y : i == 1 ? h.z : h.w;
  const uint32_t hi = i == 0 ? h.z : h.w;
  return __funnelshift_r(lo, hi, sh) & 0xFFFu;
}

// The wave tree of the reference: shuffle down by 16, 8, 4, 2, 1; lane 0 holds the sum.
__device__ __forceinline__ float warp_tree(float v) {
  v = __fadd_rn(v, __shfl_down_sync(0xFFFFFFFFu, v, 16));
  v = __fadd_rn(v, __shfl_down_sync(0xFFFFFFFFu, v, 8));
  v = __fadd_rn(v, __shfl_down_sync(0xFFFFFFFFu, v, 4));
  v = __fadd_rn(v, __shfl_down_sync(0xFFFFFFFFu, v, 2));
  v = __fadd_rn(v, __shfl_down_sync(0xFFFFFFFFu, v, 1));
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum_all(float v) {
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

// q = round-half-away(v / d) exactly as the CPU quantiser's IEEE division gives it, without paying for a division
// per element: t = v * (1/d) is within 7e-5 of the rounded quotient (|t| <= 127), so away from a rounding
// boundary (k + 0.5) by more than 2.5e-4 both round to the same integer; only the rare element near a boundary,
// or a block with a denormal-range scale, takes the exact division. rinv = __frcp_rn(d), once per block.
__device__ __forceinline__ int q8_round(float v, float d, float rinv) {
  const float t = __fmul_rn(v, rinv);
  const float f = fabsf(t) - truncf(fabsf(t));
  if (!(d > 1e-30f) || fabsf(f - 0.5f) < 2.5e-4f) return (int)roundf(__fdiv_rn(v, d));
  return (int)roundf(t);
}

// Q8 of one block of 32 floats held one per lane: writes q, d, asum of block
// b into a Q8 buffer of nb blocks. d = amax / 127 and q = round-half-away(x /
// d) with IEEE division, as the CPU quantiser.
__device__ __forceinline__ void quant_block_warp(float x, uint8_t *q, uint32_t nb, uint32_t b, int lane) {
  const float amax = warp_max(fabsf(x));
  const float d = __fdiv_rn(amax, 127.0f);
  int v = 0;
  if (d != 0.0f) v = q8_round(x, d, __frcp_rn(d));
  int s = v;
  for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
  ((int8_t *)q)[32u * b + lane] = (int8_t)v;
  if (lane == 0) {
    ((float *)(q + 32u * (size_t)nb))[b] = d;
    ((uint32_t *)(q + 36u * (size_t)nb))[b] = (uint32_t)s;
  }
}
#endif  // __CUDACC__

}  // namespace ieb
