// peer_ll.cuh -- "low-latency" slots for small cross-GPU exchanges over peer memory: every 32-bit payload word
// travels as one 64-bit store {epoch << 32 | word} into the receiver's memory, and the receiver polls the words
// themselves: a value is complete as soon as its epoch matches, so there is no separate flag and no fence.
// Slots are [2][world][max_n] words per rank, double-buffered by the parity of the call's epoch (a rank can be
// at most one call ahead of the slowest: finishing call k needs every rank's data of call k).
#pragma once

#include "act_stage.cuh"
#include "common.cuh"

namespace ieb {

constexpr int AR_MAX_RANKS = 8;
constexpr uint64_t AR_WAIT_NS = 2000000000ull;  // 2 s: a peer that has not delivered by then is reported, not waited for

__device__ __forceinline__ uint64_t ar_now() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void ll_store(unsigned long long *p, uint32_t epoch, uint32_t payload) {
  const unsigned long long v = (unsigned long long)epoch << 32 | payload;
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// Two adjacent words in one 16-byte store (p 16-byte aligned); each half is complete on its own epoch.
__device__ __forceinline__ void ll_store2(unsigned long long *p, uint32_t epoch, uint32_t w0, uint32_t w1) {
  const unsigned long long v0 = (unsigned long long)epoch << 32 | w0, v1 = (unsigned long long)epoch << 32 | w1;
  asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(v0), "l"(v1) : "memory");
}
// Four adjacent words in one 32-byte store / load (p 32-byte aligned): a warp then moves 1 KB contiguous, which the
// links carry as a few full-size packets instead of 128 eight-byte ones.
__device__ __forceinline__ void ll_store4(unsigned long long *p, uint32_t epoch, const uint32_t (&w)[4]) {
  const unsigned long long e = (unsigned long long)epoch << 32;
  asm volatile("st.relaxed.sys.global.v4.u64 [%0], {%1, %2, %3, %4};" ::"l"(p), "l"(e | w[0]), "l"(e | w[1]), "l"(e | w[2]), "l"(e | w[3]) : "memory");
}
__device__ __forceinline__ void ll_load4(const unsigned long long *p, unsigned long long (&v)[4]) {
  asm volatile("ld.relaxed.sys.global.v4.u64 {%0, %1, %2, %3}, [%4];" : "=l"(v[0]), "=l"(v[1]), "=l"(v[2]), "=l"(v[3]) : "l"(p) : "memory");
}
__device__ __forceinline__ unsigned long long ll_load(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// Four consecutive words of epoch k; false (after the time limit, or at once when *gave_up is set) if they did not all arrive.
__device__ __forceinline__ bool ll_wait4(const unsigned long long *p, uint32_t k, uint32_t (&out)[4], bool *gave_up, uint64_t t0) {
  for (;;) {
    unsigned long long v[4];
#pragma unroll
    for (int c = 0; c < 4; c++) v[c] = ll_load(p + c);
    bool all = true;
#pragma unroll
    for (int c = 0; c < 4; c++) all = all && (uint32_t)(v[c] >> 32) == k;
#pragma unroll
    for (int c = 0; c < 4; c++) out[c] = (uint32_t)v[c];
    if (all) return true;
    if (*gave_up || ar_now() - t0 > AR_WAIT_NS) {
      *gave_up = true;
      return false;
    }
  }
}

// What a GEMV needs to deliver its rows to the other ranks as it produces them (gemv_direct.cu); the reduction
// kernel that follows (allreduce.cu) then only has to wait for the peers' rows.
struct ArPush {
  unsigned long long *ll[AR_MAX_RANKS];  // rank j's slots
  uint32_t *epoch;                       // local: completed calls (this exchange is call *epoch + 1)
  uint32_t rank, world, max_n;
};

// The direct decode GEMV (gemv_direct.cu). tail: RMSNorm + Q8 of the finished vector by the last CTA; push (no
// tail / bias / res): a tensor-parallel partial whose rows are also stored into the other ranks' slots;
// late_trigger: the kernel lets its dependents start only after its own dependency wait; swiglu_pairs: the rows are
// interleaved (gate_i, up_i) pairs and d_y receives silu(gate_i) * up_i (rows / 2 values).
int gemv_direct(int kind, const void *d_w, uint32_t rows, uint32_t cols, const ActSrc &act, bool norm, float *d_y, const float *d_bias,
                const float *d_res, const ActSrc *tail, uint32_t *work, cudaStream_t st, const ArPush *push = nullptr, bool late_trigger = false,
                bool swiglu_pairs = false);
// Whether the direct decode GEMV takes this matrix (a quantised kind, at most 1024 blocks per row).
bool gemv_direct_ok(int kind, uint32_t cols);

}  // namespace ieb
