// gemv_blocks.cuh -- one quantised 32-weight block of a row panel: how to load
// it (from global memory with streaming loads, or from the shared-memory ring)
// and how to add its contribution to a lane's accumulator in the reference's
// arithmetic order. Shared by gemv.cu and gemv_stream.cu.
#pragma once

#include "common.cuh"

namespace ieb {

template <bool SMEM>
__device__ __forceinline__ uint4 blk_ld16(const void *p) {
  if (SMEM) return *reinterpret_cast<const uint4 *>(p);
  return ld_stream16(p);
}
template <bool SMEM>
__device__ __forceinline__ uint2 blk_ld8(const void *p) {
  if (SMEM) return *reinterpret_cast<const uint2 *>(p);
  return ld_stream8(p);
}
template <bool SMEM>
__device__ __forceinline__ uint16_t blk_ld2(const void *p) {
  if (SMEM) return *reinterpret_cast<const uint16_t *>(p);
  return ld_stream2(p);
}

template <int KIND, bool SMEM>
struct Blk;

// Q4_0: 16 B nibbles at 16 b, f16 scale at 16 nb + 2 b.
template <bool SMEM>
struct Blk<IE_B200_MAT_Q4, SMEM> {
  uint4 w;
  uint16_t d;
  __device__ __forceinline__ void load(const uint8_t *rp, uint32_t b, uint32_t nb) {
    w = blk_ld16<SMEM>(rp + 16u * (size_t)b);
    d = blk_ld2<SMEM>(rp + 16u * (size_t)nb + 2u * b);
  }
  // acc = acc + (dw * da) * (float)dot, each operation rounded on its own.
  __device__ __forceinline__ float accum(float acc, const uint4 &a0, const uint4 &a1, float da, int asum, uint32_t) const {
    const int dot = q4_dot(w, a0, a1) - 8 * asum;
    return __fadd_rn(acc, __fmul_rn(__fmul_rn(h2f(d), da), (float)dot));
  }
};

// Q8_0: 32 signed bytes at 32 b (weights 4k .. 4k + 3 in word k, as the activations), f16 scale at 32 nb + 2 b.
template <bool SMEM>
struct Blk<IE_B200_MAT_Q8, SMEM> {
  uint4 w0, w1;
  uint16_t d;
  __device__ __forceinline__ void load(const uint8_t *rp, uint32_t b, uint32_t nb) {
    w0 = blk_ld16<SMEM>(rp + 32u * (size_t)b);
    w1 = blk_ld16<SMEM>(rp + 32u * (size_t)b + 16u);
    d = blk_ld2<SMEM>(rp + 32u * (size_t)nb + 2u * b);
  }
  // acc = acc + (dw * da) * (float)dot, dot = eight signed dot4 in word order.
  __device__ __forceinline__ float accum(float acc, const uint4 &a0, const uint4 &a1, float da, int, uint32_t) const {
    int dot = __dp4a((int)w0.x, (int)a0.x, 0);
    dot = __dp4a((int)w0.y, (int)a0.y, dot), dot = __dp4a((int)w0.z, (int)a0.z, dot), dot = __dp4a((int)w0.w, (int)a0.w, dot);
    dot = __dp4a((int)w1.x, (int)a1.x, dot), dot = __dp4a((int)w1.y, (int)a1.y, dot), dot = __dp4a((int)w1.z, (int)a1.z, dot);
    dot = __dp4a((int)w1.w, (int)a1.w, dot);
    return __fadd_rn(acc, __fmul_rn(__fmul_rn(h2f(d), da), (float)dot));
  }
};

// Q4_K: nibbles as Q4_0; per super-block a 16 B header at 16 nb + 16 (b / 8).
template <bool SMEM>
struct Blk<IE_B200_MAT_Q4K, SMEM> {
  uint4 w, h;
  __device__ __forceinline__ void load(const uint8_t *rp, uint32_t b, uint32_t nb) {
    w = blk_ld16<SMEM>(rp + 16u * (size_t)b);
    h = blk_ld16<SMEM>(rp + 16u * (size_t)nb + 16u * (b >> 3));
  }
  // acc = fma(-(dmin mn), da * (float)asum, fma((d sc) * (float)dq, da, acc)).
  __device__ __forceinline__ float accum(float acc, const uint4 &a0, const uint4 &a1, float da, int asum, uint32_t b) const {
    const int dq = q4_dot(w, a0, a1);
    const uint32_t f = q4k_field(h, (int)(b & 7u));
    const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&h.x));  // (d, dmin): both halves of the word in one unpack
    const float s = __fmul_rn(dd.x, (float)(f & 63u));
    const float mm = __fmul_rn(dd.y, (float)(f >> 6));
    return __fmaf_rn(-mm, __fmul_rn(da, (float)asum), __fmaf_rn(__fmul_rn(s, (float)dq), da, acc));
  }
};

// Q6_K: nibbles at 16 b, high-bit words at 16 nb + 8 b, (sc0 | sc1 << 8) at
// 24 nb + 2 b, f16 d at 26 nb + 2 (b / 8).
template <bool SMEM>
struct Blk<IE_B200_MAT_Q6K, SMEM> {
  uint4 w;
  uint2 hw;
  uint16_t sc, d;
  __device__ __forceinline__ void load(const uint8_t *rp, uint32_t b, uint32_t nb) {
    w = blk_ld16<SMEM>(rp + 16u * (size_t)b);
    hw = blk_ld8<SMEM>(rp + 16u * (size_t)nb + 8u * b);
    sc = blk_ld2<SMEM>(rp + 24u * (size_t)nb + 2u * b);
    d = blk_ld2<SMEM>(rp + 26u * (size_t)nb + 2u * (b >> 3));
  }
  // acc = fma(fma(d sc1, (float)d1, (d sc0) * (float)d0), da, acc).
  __device__ __forceinline__ float accum(float acc, const uint4 &a0, const uint4 &a1, float da, int, uint32_t) const {
    int d0, d1;
    q6_dots(w, hw, a0, a1, d0, d1);
    const float df = h2f(d);
    const float s0 = __fmul_rn(df, (float)(int8_t)(sc & 255u)), s1 = __fmul_rn(df, (float)(int8_t)(sc >> 8));
    return __fmaf_rn(__fmaf_rn(s1, (float)d1, __fmul_rn(s0, (float)d0)), da, acc);
  }
};

}  // namespace ieb
