// norm_quant.cuh -- RMSNorm + per-32 Q8 of one vector held in registers by one CTA: thread t owns elements
// 4 (t + THREADS it) .. + 3 for it < ITERS, so eight neighbouring threads hold one Q8 block and the quantiser
// needs three shuffles, no shared memory. y = x * rsqrt(mean x^2 + eps) * w with every product rounded, then
// d = amax / 127, q = round-half-away(y / d), as the CPU reference does. Used by the stand-alone RMSNorm of one
// token and by the tensor-parallel reduction kernel. CL > 1: the vector is spread over the CL CTAs of ONE thread-block
// cluster (the whole grid; thread t of CTA c owns elements 4 (c THREADS + t + CL THREADS it) ..), and the CTAs' sums of
// squares meet in every CTA's shared memory (a store into each peer CTA, one cluster barrier), added in CTA order.
#pragma once

#include "common.cuh"

namespace ieb {

// red: THREADS / 32 floats of shared memory (+ CL more behind them when CL > 1). Elements at or past n must be zero in x
// (they count as zeros). With CL > 1 every thread of every CTA of the cluster must make the call.
template <int ITERS, int THREADS, int CL = 1>
__device__ __forceinline__ void norm_quant_vec(const float4 (&x)[ITERS], const float4 (&w4)[ITERS], uint32_t n, float eps, float *xn, uint8_t *xq,
                                               float *red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tid = CL > 1 ? (int)(blockIdx.x * THREADS + threadIdx.x) : (int)threadIdx.x;  // the thread's place in the vector
  constexpr int ALL = THREADS * CL;
  float ss = 0.0f;
#pragma unroll
  for (int it = 0; it < ITERS; it++) ss = fmaf(x[it].x, x[it].x, ss), ss = fmaf(x[it].y, x[it].y, ss), ss = fmaf(x[it].z, x[it].z, ss), ss = fmaf(x[it].w, x[it].w, ss);
  ss = warp_sum_all(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = warp_sum_all(lane < THREADS / 32 ? red[lane] : 0.0f);
  if (CL > 1) {
    float *all = red + THREADS / 32;  // [CL]: the CTAs' sums, the same in every CTA
    if (threadIdx.x < CL) cluster_st_f32(cluster_map_shared(all + blockIdx.x, threadIdx.x), tot);
    cluster_sync_all();
    tot = 0.0f;
#pragma unroll
    for (int c = 0; c < CL; c++) tot = __fadd_rn(tot, all[c]);
  }
  const float sc = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(tot, (float)n), eps)));
  const uint32_t nb = n / 32u;
#pragma unroll
  for (int it = 0; it < ITERS; it++) {
    const uint32_t i = 4u * (tid + ALL * it);
    const float v[4] = {__fmul_rn(__fmul_rn(x[it].x, sc), w4[it].x), __fmul_rn(__fmul_rn(x[it].y, sc), w4[it].y),
                        __fmul_rn(__fmul_rn(x[it].z, sc), w4[it].z), __fmul_rn(__fmul_rn(x[it].w, sc), w4[it].w)};
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 4));
    const float d = __fdiv_rn(amax, 127.0f), rinv = __frcp_rn(d);
    uint32_t pk = 0u;
    int sum = 0;
#pragma unroll
    for (int c = 0; c < 4; c++) {
      int q = 0;
      if (d != 0.0f) q = q8_round(v[c], d, rinv);
      sum += q;
      pk |= (uint32_t)(q & 255) << (8 * c);
    }
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
    if (i < n) {
      if (xn) *reinterpret_cast<float4 *>(xn + i) = make_float4(v[0], v[1], v[2], v[3]);
      if (xq) {
        *reinterpret_cast<uint32_t *>(xq + i) = pk;
        if ((tid & 7) == 0) {
          reinterpret_cast<float *>(xq + 32u * (size_t)nb)[i / 32u] = d;
          reinterpret_cast<int *>(xq + 36u * (size_t)nb)[i / 32u] = sum;
        }
      }
    }
  }
}

}  // namespace ieb
