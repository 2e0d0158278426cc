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
// The same for a kernel of thread-block clusters of cluster_x CTAs along x (grid.x a multiple of it).
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, unsigned cluster_x, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = cluster_x, at[0].val.clusterDim.y = 1, at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at, cfg.numAttrs = pdl_enabled() ? 2 : 1;
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
    case IE_B200_MAT_Q8: return round16(nb * 34u);
    case IE_B200_MAT_Q4K: return nb * 16u + (nb / 8u) * 16u;
    case IE_B200_MAT_Q6K: return round16(nb * 26u + (nb / 8u) * 2u);
    default: return (size_t)cols * 4u;
  }
}

// ---- device helpers ----
#ifdef __CUDACC__

// Programmatic dependent launch: let the next kernel of the stream start (its own pdl_wait keeps it from
// reading our results early), and wait until the previous kernel has completed and its writes are visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Every kernel launched through launch_pdl starts with this.
__device__ __forceinline__ void pdl_prologue() {
  pdl_launch_dependents();
  pdl_wait();
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

// dot4 of four unsigned bytes with four signed bytes, added to c (dp4a.u32.s32).
__device__ __forceinline__ int dp4a_us(uint32_t a_u8, int b_s8, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8), "r"(b_s8), "r"(c));
  return d;
}

// Sum over the 32 nibbles q (0..15) of q * a. Word k of the weight block
// holds weights 4k..4k+3 in its low nibbles and 16+4k..16+4k+3 in its high
// nibbles; a0 are activation words 0..3, a1 words 4..7. Nibble bytes are
// below 128, so the signed byte product equals the unsigned-by-signed one.
__device__ __forceinline__ int q4_dot(const uint4 &w, const uint4 &a0, const uint4 &a1) {
  // low nibbles against words 0..3, high nibbles against words 4..7. The high nibbles stay where they are: a byte
  // 0xN0 is 16 N, so their dot comes out as 16 times the wanted one and one exact shift at the end undoes it (one
  // AND per word instead of shift + AND). Integer arithmetic: the same int32 as the nibble-by-nibble sum.
  int lo = 0, hi = 0;
  lo = dp4a_us(w.x & 0x0F0F0F0Fu, (int)a0.x, lo), hi = dp4a_us(w.x & 0xF0F0F0F0u, (int)a1.x, hi);
  lo = dp4a_us(w.y & 0x0F0F0F0Fu, (int)a0.y, lo), hi = dp4a_us(w.y & 0xF0F0F0F0u, (int)a1.y, hi);
  lo = dp4a_us(w.z & 0x0F0F0F0Fu, (int)a0.z, lo), hi = dp4a_us(w.z & 0xF0F0F0F0u, (int)a1.z, hi);
  lo = dp4a_us(w.w & 0x0F0F0F0Fu, (int)a0.w, lo), hi = dp4a_us(w.w & 0xF0F0F0F0u, (int)a1.w, hi);
  return lo + (hi >> 4);
}

// One byte-quad of Q6_K values minus 32 as signed bytes: v = nibbles | two
// high bits << 4, then ((v | 0x80808080) - 0x20202020) ^ 0x80808080.
__device__ __forceinline__ int q6_sw(uint32_t nib4, uint32_t hword, int k) {
  const uint32_t v = nib4 | (((hword >> (2 * k)) & 0x03030303u) << 4);
  return (int)(((v | 0x80808080u) - 0x20202020u) ^ 0x80808080u);
}
// One byte-quad of Q6_K values as they are stored (0..63, without the - 32): nibbles | two high bits << 4. hi_half: the
// nibbles are the high ones of nib_src.
__device__ __forceinline__ uint32_t q6_uw(uint32_t nib_src, bool hi_half, uint32_t hword, int k) {
  const uint32_t hs = k < 2 ? hword << (4 - 2 * k) : hword >> (2 * k - 4);  // the two bits of every byte moved to bits 4, 5
  return ((hi_half ? nib_src >> 4 : nib_src) & 0x0F0F0F0Fu) | (hs & 0x30303030u);
}
// The two half dots of a Q6_K sub-block: weights 0..15 against a0, 16..31 against a1. sum (q - 32) a is taken as
// sum q a - 32 sum a: the stored bytes go into the dot as they are (unsigned by signed), and the sums of the sixteen
// activations of each half (four dot4 with ones; the same for every row that shares the activation block) replace the
// three operations per word that would turn every byte into q - 32. Integer arithmetic: the same int32 either way.
__device__ __forceinline__ void q6_dots(const uint4 &w, const uint2 &hw, const uint4 &a0, const uint4 &a1, int &d0, int &d1) {
  int s0 = 0, s1 = 0, h0 = 0, h1 = 0;
  s0 = dp4a_us(q6_uw(w.x, false, hw.x, 0), (int)a0.x, s0), h0 = __dp4a(0x01010101, (int)a0.x, h0);
  s0 = dp4a_us(q6_uw(w.y, false, hw.x, 1), (int)a0.y, s0), h0 = __dp4a(0x01010101, (int)a0.y, h0);
  s0 = dp4a_us(q6_uw(w.z, false, hw.x, 2), (int)a0.z, s0), h0 = __dp4a(0x01010101, (int)a0.z, h0);
  s0 = dp4a_us(q6_uw(w.w, false, hw.x, 3), (int)a0.w, s0), h0 = __dp4a(0x01010101, (int)a0.w, h0);
  s1 = dp4a_us(q6_uw(w.x, true, hw.y, 0), (int)a1.x, s1), h1 = __dp4a(0x01010101, (int)a1.x, h1);
  s1 = dp4a_us(q6_uw(w.y, true, hw.y, 1), (int)a1.y, s1), h1 = __dp4a(0x01010101, (int)a1.y, h1);
  s1 = dp4a_us(q6_uw(w.z, true, hw.y, 2), (int)a1.z, s1), h1 = __dp4a(0x01010101, (int)a1.z, h1);
  s1 = dp4a_us(q6_uw(w.w, true, hw.y, 3), (int)a1.w, s1), h1 = __dp4a(0x01010101, (int)a1.w, h1);
  d0 = s0 - 32 * h0, d1 = s1 - 32 * h1;
}

// The 12-bit (sc | mn << 6) field j of a Q4_K super-block header (words y, z, w).
__device__ __forceinline__ uint32_t q4k_field(const uint4 &h, int j) {
  // fields 0..2 start in word y, 3..5 in z, 6..7 in w (12 j >> 5); a field that crosses a word boundary (2 and 5) takes
  // its upper bits from the next word through the funnel shift
  const uint32_t lo = j < 3 ? h.y : j < 6 ? h.z : h.w;
  const uint32_t hi = j < 3 ? h.z : h.w;
  return __funnelshift_r(lo, hi, (12 * j) & 31) & 0xFFFu;
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
// ---- thread-block clusters: a word into the shared memory of another CTA of the cluster, and the cluster's barrier
__device__ __forceinline__ uint32_t cluster_map_shared(const void *p, uint32_t cta_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(p)), "r"(cta_rank));
  return remote;
}
__device__ __forceinline__ void cluster_st_f32(uint32_t addr, float v) { asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
// The two halves of the barrier: a CTA's shared memory may be written by its peers only once it runs, so a kernel
// arrives when it starts and waits just before its first store into a peer (by then nobody waits in practice).
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
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
