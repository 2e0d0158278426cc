// act_stage.cuh -- the prologue shared by the decode GEMV kernels: bring one token's activations into shared
// memory as two 16-byte planes per 32-block (A0 = int8 0..15, A1 = int8 16..31) plus the block scales and sums.
// Either from a Q8 buffer in global memory, or (NORM) computed on the spot from the f32 residual stream:
// y = x * rsqrt(mean x^2 + eps) * w, then the per-32 quantiser d = amax / 127, q = round(y / d), as the
// stand-alone RMSNorm kernel does. Every CTA repeats the work; CTA `writer` also stores y and its Q8 copy.
#pragma once

#include "common.cuh"

namespace ieb {

struct ActSrc {
  const uint8_t *xq;    // Q8 buffer (NORM = false)
  const float *xf;      // f32 vector (NORM = true)
  const float *norm_w;  // NULL with NORM: no norm, the Q8 quantiser of xf alone (y = x)
  float eps;
  float *xn_out;        // optional outputs of the fused norm
  uint8_t *xq_out;
};

// Called by the first WARPS warps of a CTA (threadIdx.x < 32 * WARPS); `sync` synchronises exactly those threads.
template <bool NORM, int WARPS, typename Sync>
__device__ __forceinline__ void stage_activations(const ActSrc &a, uint32_t nb, uint4 *A0, uint4 *A1, float *da, int *as, float *red, bool writer,
                                                  Sync sync) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr uint32_t NT = WARPS * 32;
  if (!NORM) {
    const uint4 *src = reinterpret_cast<const uint4 *>(a.xq);
    for (uint32_t i = tid; i < 2u * nb; i += NT) {
      const uint4 v = __ldcg(src + i);  // from L2: inside a persistent kernel another SM has just written it
      if (i & 1u) A1[i >> 1] = v;
      else A0[i >> 1] = v;
    }
    const float *d = reinterpret_cast<const float *>(a.xq + 32u * (size_t)nb);
    const int *s = reinterpret_cast<const int *>(a.xq + 36u * (size_t)nb);
    for (uint32_t i = tid; i < nb; i += NT) da[i] = __ldcg(d + i), as[i] = __ldcg(s + i);
  } else {
    // Thread t owns half-blocks t, t + NT, ...: 16 consecutive elements each, so the quantiser needs no
    // warp-wide reductions (one exchange with the neighbour lane that holds the other half) and one thread
    // writes a whole 16-byte plane entry. The first half-block (all of them when n <= 16 * NT) stays in
    // registers between the sum of squares and the quantiser: one round trip to L2 instead of two.
    const uint32_t n = nb * 32u, HB = 2u * nb;
    float x0[16], w0[16];
    {
      const bool own = (uint32_t)tid < HB;
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        float4 x4 = make_float4(0.f, 0.f, 0.f, 0.f), w4 = x4;
        if (own) {
          x4 = __ldcg(reinterpret_cast<const float4 *>(a.xf + 16u * tid + j));  // L2: other CTAs may just have written it
          if (a.norm_w) w4 = *reinterpret_cast<const float4 *>(a.norm_w + 16u * tid + j);
        }
        x0[j] = x4.x, x0[j + 1] = x4.y, x0[j + 2] = x4.z, x0[j + 3] = x4.w;
        w0[j] = w4.x, w0[j + 1] = w4.y, w0[j + 2] = w4.z, w0[j + 3] = w4.w;
      }
    }
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; j++) ss = fmaf(x0[j], x0[j], ss);
    for (uint32_t hb = tid + NT; hb < HB; hb += NT) {
      float4 x4[4];
#pragma unroll
      for (int j = 0; j < 4; j++) x4[j] = __ldcg(reinterpret_cast<const float4 *>(a.xf + 16u * hb) + j);
#pragma unroll
      for (int j = 0; j < 4; j++) ss = fmaf(x4[j].x, x4[j].x, ss), ss = fmaf(x4[j].y, x4[j].y, ss), ss = fmaf(x4[j].z, x4[j].z, ss), ss = fmaf(x4[j].w, x4[j].w, ss);
    }
    ss = warp_sum_all(ss);
    if (lane == 0) red[warp] = ss;
    sync();
    float tot = lane < WARPS ? red[lane] : 0.0f;
    tot = warp_sum_all(tot);
    const float sc = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(tot, (float)n), a.eps)));
    const bool plain = a.norm_w == nullptr;
    for (uint32_t k0 = 0; k0 < HB; k0 += NT) {  // uniform trip count: the shuffles below need every lane
      const uint32_t hb = k0 + tid, b = hb >> 1, h = hb & 1u, base = 16u * hb;
      const bool valid = hb < HB;
      float v[16];
      if (k0 != 0u) {
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
          float4 x4 = make_float4(0.f, 0.f, 0.f, 0.f), w4 = x4;
          if (valid) {
            x4 = __ldcg(reinterpret_cast<const float4 *>(a.xf + base + j));
            if (!plain) w4 = *reinterpret_cast<const float4 *>(a.norm_w + base + j);
          }
          x0[j] = x4.x, x0[j + 1] = x4.y, x0[j + 2] = x4.z, x0[j + 3] = x4.w;
          w0[j] = w4.x, w0[j + 1] = w4.y, w0[j + 2] = w4.z, w0[j + 3] = w4.w;
        }
      }
      float amax = 0.0f;
#pragma unroll
      for (int j = 0; j < 16; j++) {
        v[j] = plain ? x0[j] : __fmul_rn(__fmul_rn(x0[j], sc), w0[j]);
        amax = fmaxf(amax, fabsf(v[j]));
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));  // the other half of the block
      const float d = __fdiv_rn(amax, 127.0f), rinv = __frcp_rn(d);
      uint32_t pk[4] = {0u, 0u, 0u, 0u};
      int s = 0;
#pragma unroll
      for (int j = 0; j < 16; j++) {
        int q = 0;
        if (d != 0.0f) q = q8_round(v[j], d, rinv);
        s += q;
        pk[j >> 2] |= (uint32_t)(q & 255) << (8 * (j & 3));
      }
      s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
      if (valid) {
        const uint4 packed = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        if (A0) {  // A0 == nullptr: only the global copies are wanted (the norm tail of a producing GEMV)
          (h ? A1 : A0)[b] = packed;
          if (h == 0u) da[b] = d, as[b] = s;
        }
        if (writer) {
          if (a.xn_out) {
#pragma unroll
            for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4 *>(a.xn_out + base + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          }
          if (a.xq_out) {
            *reinterpret_cast<uint4 *>(a.xq_out + base) = packed;
            if (h == 0u) {
              reinterpret_cast<float *>(a.xq_out + 32u * (size_t)nb)[b] = d;
              reinterpret_cast<int *>(a.xq_out + 36u * (size_t)nb)[b] = s;
            }
          }
        }
      }
    }
  }
  sync();
}

}  // namespace ieb
