// repack.cu -- load-time re-layout of quantised weights into the streaming
// "row panel" layout (see ie_b200.h): from raw GGUF tensor bytes, or from the
// word/scale arrays that the reference's model loader hands to its matrix
// sink. One thread per 32-weight block; runs once per matrix.
#include "common.cuh"

namespace ieb {

__device__ __forceinline__ uint32_t pack4(uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) { return b0 | (b1 << 8) | (b2 << 16) | (b3 << 24); }

// The 6-bit scale and min of sub-block j from the 12 packed bytes of a GGUF
// Q4_K super-block (ggml's get_scale_min_k4 rule).
__device__ __forceinline__ void gguf_q4k_sc_mn(int j, const uint8_t *p, uint32_t &sc, uint32_t &mn) {
  if (j < 4) {
    sc = p[j] & 63u, mn = p[j + 4] & 63u;
  } else {
    sc = (p[j + 4] & 15u) | ((uint32_t)(p[j - 4] >> 6) << 4);
    mn = (uint32_t)(p[j + 4] >> 4) | ((uint32_t)(p[j] >> 6) << 4);
  }
}

// Eight (sc, mn) pairs -> three words of 12-bit fields (sc | mn << 6), field j at bit 12 j.
__device__ __forceinline__ void pack_q4k_fields(const uint32_t *sc, const uint32_t *mn, uint32_t *w3) {
  unsigned long long lo = 0;  // fields 0..4 (60 bits) + low 4 bits of field 5
  uint32_t f[8];
  for (int j = 0; j < 8; j++) f[j] = (sc[j] & 63u) | ((mn[j] & 63u) << 6);
  for (int j = 0; j < 5; j++) lo |= (unsigned long long)f[j] << (12 * j);
  lo |= (unsigned long long)(f[5] & 15u) << 60;
  w3[0] = (uint32_t)lo, w3[1] = (uint32_t)(lo >> 32);
  w3[2] = (f[5] >> 4) | (f[6] << 8) | (f[7] << 20);
}

// ---- from GGUF bytes ----
__global__ void repack_gguf_q4_0(const uint8_t *__restrict__ src, uint32_t rows, uint32_t nb, uint8_t *dst, size_t rowb) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * nb) return;
  const uint32_t r = (uint32_t)(i / nb), b = (uint32_t)(i % nb);
  const uint16_t *s = reinterpret_cast<const uint16_t *>(src + i * 18u);  // 18 i is even
  uint8_t *rp = dst + (size_t)r * rowb;
  uint32_t w[4];
  for (int k = 0; k < 4; k++) w[k] = (uint32_t)s[1 + 2 * k] | ((uint32_t)s[2 + 2 * k] << 16);
  *reinterpret_cast<uint4 *>(rp + 16u * (size_t)b) = make_uint4(w[0], w[1], w[2], w[3]);
  reinterpret_cast<uint16_t *>(rp + 16u * (size_t)nb)[b] = s[0];
}

// Q8_0: 34-byte blocks {f16 d, 32 int8}; the weight bytes keep their order (word k = weights 4k .. 4k + 3).
__global__ void repack_gguf_q8_0(const uint8_t *__restrict__ src, uint32_t rows, uint32_t nb, uint8_t *dst, size_t rowb) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * nb) return;
  const uint32_t r = (uint32_t)(i / nb), b = (uint32_t)(i % nb);
  const uint16_t *s = reinterpret_cast<const uint16_t *>(src + i * 34u);  // 34 i is even
  uint8_t *rp = dst + (size_t)r * rowb;
  uint32_t w[8];
  for (int k = 0; k < 8; k++) w[k] = (uint32_t)s[1 + 2 * k] | ((uint32_t)s[2 + 2 * k] << 16);
  *reinterpret_cast<uint4 *>(rp + 32u * (size_t)b) = make_uint4(w[0], w[1], w[2], w[3]);
  *reinterpret_cast<uint4 *>(rp + 32u * (size_t)b + 16u) = make_uint4(w[4], w[5], w[6], w[7]);
  reinterpret_cast<uint16_t *>(rp + 32u * (size_t)nb)[b] = s[0];
}

__global__ void repack_gguf_q4_k(const uint8_t *__restrict__ src, uint32_t rows, uint32_t nb, uint8_t *dst, size_t rowb) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * nb) return;
  const uint32_t r = (uint32_t)(i / nb), b = (uint32_t)(i % nb), k = b & 7u;
  const uint8_t *blk = src + ((size_t)r * (nb / 8u) + b / 8u) * 144u;
  const uint8_t *qb = blk + 16u + 32u * (k / 2u);
  uint8_t *rp = dst + (size_t)r * rowb;
  uint32_t by[16];
  for (int j = 0; j < 16; j++) {
    const uint32_t lo = (k & 1u) ? (uint32_t)(qb[j] >> 4) : (uint32_t)(qb[j] & 15u);
    const uint32_t hi = (k & 1u) ? (uint32_t)(qb[j + 16] >> 4) : (uint32_t)(qb[j + 16] & 15u);
    by[j] = lo | (hi << 4);
  }
  *reinterpret_cast<uint4 *>(rp + 16u * (size_t)b) =
      make_uint4(pack4(by[0], by[1], by[2], by[3]), pack4(by[4], by[5], by[6], by[7]), pack4(by[8], by[9], by[10], by[11]),
                 pack4(by[12], by[13], by[14], by[15]));
  if (k == 0u) {
    uint32_t sc[8], mn[8], w3[3];
    for (int j = 0; j < 8; j++) gguf_q4k_sc_mn(j, blk + 4, sc[j], mn[j]);
    pack_q4k_fields(sc, mn, w3);
    const uint32_t ddm = (uint32_t)blk[0] | ((uint32_t)blk[1] << 8) | ((uint32_t)blk[2] << 16) | ((uint32_t)blk[3] << 24);
    *reinterpret_cast<uint4 *>(rp + 16u * (size_t)nb + 16u * (b >> 3)) = make_uint4(ddm, w3[0], w3[1], w3[2]);
  }
}

__global__ void repack_gguf_q6_k(const uint8_t *__restrict__ src, uint32_t rows, uint32_t nb, uint8_t *dst, size_t rowb) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * nb) return;
  const uint32_t r = (uint32_t)(i / nb), b = (uint32_t)(i % nb), sub = b & 7u, n = sub / 4u, m = sub % 4u;
  const uint8_t *blk = src + ((size_t)r * (nb / 8u) + b / 8u) * 210u;
  uint8_t *rp = dst + (size_t)r * rowb;
  uint32_t q[32];
  for (int l = 0; l < 32; l++) {
    const uint32_t ql = blk[64u * n + 32u * (m & 1u) + l], qh = blk[128u + 32u * n + l];
    q[l] = (m < 2u ? (ql & 15u) : (ql >> 4)) | (((qh >> (2u * m)) & 3u) << 4);
  }
  uint32_t w[4], hw[2] = {0u, 0u};
  for (int k = 0; k < 4; k++) {
    w[k] = 0;
    for (int e = 0; e < 4; e++) w[k] |= ((q[4 * k + e] & 15u) | ((q[4 * k + e + 16] & 15u) << 4)) << (8 * e);
  }
  for (int h = 0; h < 2; h++)
    for (int e = 0; e < 16; e++) hw[h] |= ((q[16 * h + e] >> 4) & 3u) << (8 * (e % 4) + 2 * (e / 4));
  *reinterpret_cast<uint4 *>(rp + 16u * (size_t)b) = make_uint4(w[0], w[1], w[2], w[3]);
  *reinterpret_cast<uint2 *>(rp + 16u * (size_t)nb + 8u * b) = make_uint2(hw[0], hw[1]);
  reinterpret_cast<uint16_t *>(rp + 24u * (size_t)nb)[b] = (uint16_t)(blk[192u + 2u * sub] | (blk[192u + 2u * sub + 1u] << 8));
  if (sub == 0u) reinterpret_cast<uint16_t *>(rp + 26u * (size_t)nb)[b >> 3] = (uint16_t)(blk[208] | (blk[209] << 8));
}

// ---- from the reference's repacked arrays (qw words, qs u16 entries) ----
template <int KIND>
__global__ void repack_ref_kernel(const uint32_t *__restrict__ qw, const uint16_t *__restrict__ qs, uint32_t rows, uint32_t nb, uint8_t *dst,
                                  size_t rowb) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * nb) return;
  const uint32_t r = (uint32_t)(i / nb), b = (uint32_t)(i % nb);
  uint8_t *rp = dst + (size_t)r * rowb;
  if (KIND == IE_B200_MAT_Q8) {  // eight words per block (core/ie_core.h:201-205), scales one per block
    *reinterpret_cast<uint4 *>(rp + 32u * (size_t)b) = *reinterpret_cast<const uint4 *>(qw + i * 8u);
    *reinterpret_cast<uint4 *>(rp + 32u * (size_t)b + 16u) = *reinterpret_cast<const uint4 *>(qw + i * 8u + 4u);
    reinterpret_cast<uint16_t *>(rp + 32u * (size_t)nb)[b] = qs[i];
    return;
  }
  *reinterpret_cast<uint4 *>(rp + 16u * (size_t)b) = *reinterpret_cast<const uint4 *>(qw + i * 4u);
  if (KIND == IE_B200_MAT_Q4) {
    reinterpret_cast<uint16_t *>(rp + 16u * (size_t)nb)[b] = qs[i];
  } else if (KIND == IE_B200_MAT_Q4K) {
    if ((b & 7u) == 0u) {
      uint32_t sc[8], mn[8], w3[3];
      for (int j = 0; j < 8; j++) sc[j] = qs[i + j] & 63u, mn[j] = (qs[i + j] >> 8) & 63u;
      pack_q4k_fields(sc, mn, w3);
      const size_t dd = (size_t)rows * nb + ((size_t)r * (nb / 8u) + b / 8u) * 2u;
      *reinterpret_cast<uint4 *>(rp + 16u * (size_t)nb + 16u * (b >> 3)) = make_uint4((uint32_t)qs[dd] | ((uint32_t)qs[dd + 1] << 16), w3[0], w3[1], w3[2]);
    }
  } else {  // Q6_K
    const uint32_t *hw = qw + (size_t)rows * nb * 4u + i * 2u;
    *reinterpret_cast<uint2 *>(rp + 16u * (size_t)nb + 8u * b) = make_uint2(hw[0], hw[1]);
    reinterpret_cast<uint16_t *>(rp + 24u * (size_t)nb)[b] = qs[i];
    if ((b & 7u) == 0u) reinterpret_cast<uint16_t *>(rp + 26u * (size_t)nb)[b >> 3] = qs[(size_t)rows * nb + (size_t)r * (nb / 8u) + b / 8u];
  }
}

static int check_shape(const char *who, int kind, uint32_t rows, uint32_t cols) {
  if (cols == 0 || cols % 32u) return fail(IE_B200_E_SIZE, "%s: cols %u is not a multiple of 32", who, cols);
  if ((kind == IE_B200_MAT_Q4K || kind == IE_B200_MAT_Q6K) && cols % 256u) return fail(IE_B200_E_SIZE, "%s: K kinds need cols %% 256 == 0", who);
  if ((uint64_t)rows * (cols / 32u) >= (1ull << 31)) return fail(IE_B200_E_SIZE, "%s: %u x %u has too many blocks", who, rows, cols);
  return IE_B200_OK;
}

}  // namespace ieb

using namespace ieb;

extern "C" size_t ie_b200_row_bytes(int kind, uint32_t cols) { return row_bytes_of(kind, cols); }
extern "C" size_t ie_b200_mat_bytes(int kind, uint32_t rows, uint32_t cols) { return row_bytes_of(kind, cols) * rows; }

extern "C" int ie_b200_repack_gguf(int ggml_type, const void *d_src, uint32_t rows, uint32_t cols, void *d_dst, void *stream) {
  if (!d_src || !d_dst) return fail(IE_B200_E_ARG, "ie_b200_repack_gguf: NULL pointer");
  if (!aligned16(d_dst) || ((uintptr_t)d_src & 1u)) return fail(IE_B200_E_ARG, "ie_b200_repack_gguf: misaligned pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows == 0) return IE_B200_OK;
  if (ggml_type == IE_B200_GGML_F32) {
    IEB_CUDA(cudaMemcpyAsync(d_dst, d_src, (size_t)rows * cols * 4u, cudaMemcpyDeviceToDevice, st));
    return IE_B200_OK;
  }
  const int kind = ggml_type == IE_B200_GGML_Q4_0 ? IE_B200_MAT_Q4 : ggml_type == IE_B200_GGML_Q8_0 ? IE_B200_MAT_Q8
                   : ggml_type == IE_B200_GGML_Q4_K ? IE_B200_MAT_Q4K : ggml_type == IE_B200_GGML_Q6_K ? IE_B200_MAT_Q6K : -1;
  if (kind < 0) return fail(IE_B200_E_ARG, "ie_b200_repack_gguf: GGML type %d unsupported", ggml_type);
  if (int e = check_shape("ie_b200_repack_gguf", kind, rows, cols)) return e;
  const uint32_t nb = cols / 32u;
  const size_t n = (size_t)rows * nb, rowb = row_bytes_of(kind, cols);
  const unsigned grid = (unsigned)((n + 127) / 128);
  const uint8_t *s = static_cast<const uint8_t *>(d_src);
  uint8_t *d = static_cast<uint8_t *>(d_dst);
  if (kind == IE_B200_MAT_Q4) repack_gguf_q4_0<<<grid, 128, 0, st>>>(s, rows, nb, d, rowb);
  else if (kind == IE_B200_MAT_Q8) repack_gguf_q8_0<<<grid, 128, 0, st>>>(s, rows, nb, d, rowb);
  else if (kind == IE_B200_MAT_Q4K) repack_gguf_q4_k<<<grid, 128, 0, st>>>(s, rows, nb, d, rowb);
  else repack_gguf_q6_k<<<grid, 128, 0, st>>>(s, rows, nb, d, rowb);
  IEB_LAUNCHED("repack_gguf");
  return IE_B200_OK;
}

extern "C" int ie_b200_repack_ref(int kind, const void *d_qw, const void *d_qs, uint32_t rows, uint32_t cols, void *d_dst, void *stream) {
  if (!d_qw || !d_dst) return fail(IE_B200_E_ARG, "ie_b200_repack_ref: NULL pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows == 0) return IE_B200_OK;
  if (kind == IE_B200_MAT_F32) {
    IEB_CUDA(cudaMemcpyAsync(d_dst, d_qw, (size_t)rows * cols * 4u, cudaMemcpyDeviceToDevice, st));
    return IE_B200_OK;
  }
  if (!d_qs) return fail(IE_B200_E_ARG, "ie_b200_repack_ref: NULL scale array");
  if (!aligned16(d_dst) || !aligned16(d_qw)) return fail(IE_B200_E_ARG, "ie_b200_repack_ref: misaligned pointer");
  if (int e = check_shape("ie_b200_repack_ref", kind, rows, cols)) return e;
  const uint32_t nb = cols / 32u;
  const size_t n = (size_t)rows * nb, rowb = row_bytes_of(kind, cols);
  const unsigned grid = (unsigned)((n + 127) / 128);
  const uint32_t *qw = static_cast<const uint32_t *>(d_qw);
  const uint16_t *qs = static_cast<const uint16_t *>(d_qs);
  uint8_t *d = static_cast<uint8_t *>(d_dst);
  if (kind == IE_B200_MAT_Q4) repack_ref_kernel<IE_B200_MAT_Q4><<<grid, 128, 0, st>>>(qw, qs, rows, nb, d, rowb);
  else if (kind == IE_B200_MAT_Q8) repack_ref_kernel<IE_B200_MAT_Q8><<<grid, 128, 0, st>>>(qw, qs, rows, nb, d, rowb);
  else if (kind == IE_B200_MAT_Q4K) repack_ref_kernel<IE_B200_MAT_Q4K><<<grid, 128, 0, st>>>(qw, qs, rows, nb, d, rowb);
  else if (kind == IE_B200_MAT_Q6K) repack_ref_kernel<IE_B200_MAT_Q6K><<<grid, 128, 0, st>>>(qw, qs, rows, nb, d, rowb);
  else return fail(IE_B200_E_ARG, "ie_b200_repack_ref: unknown matrix kind %d", kind);
  IEB_LAUNCHED("repack_ref");
  return IE_B200_OK;
}

// ---- a part of a matrix in the streaming layout (tensor-parallel shards): row ranges one after the other, one column range ----
namespace {
struct PartAreas {
  uint32_t n;             // areas per row
  uint32_t src[4], dst[4], len[4];  // byte offsets within the source / destination row, bytes (all multiples of 2)
};

// One CTA per destination row.
__global__ void mat_part_kernel(const uint8_t *src, size_t src_rowb, uint8_t *dst, size_t dst_rowb, uint32_t src_row0, uint32_t dst_row0, PartAreas a) {
  const uint8_t *s = src + (size_t)(src_row0 + blockIdx.x) * src_rowb;
  uint8_t *d = dst + (size_t)(dst_row0 + blockIdx.x) * dst_rowb;
  for (uint32_t k = 0; k < a.n; k++) {
    const uint16_t *sp = reinterpret_cast<const uint16_t *>(s + a.src[k]);
    uint16_t *dp = reinterpret_cast<uint16_t *>(d + a.dst[k]);
    for (uint32_t i = threadIdx.x; i < a.len[k] / 2u; i += blockDim.x) dp[i] = sp[i];
  }
  // the padding of a row (rows are rounded up to 16 bytes) stays defined
  const uint32_t end = a.dst[a.n - 1] + a.len[a.n - 1];
  for (uint32_t i = end + threadIdx.x; i < dst_rowb; i += blockDim.x) d[i] = 0;
}
}  // namespace

extern "C" int ie_b200_mat_part(int kind, const void *d_src, uint32_t rows, uint32_t cols, uint32_t n_ranges, const uint32_t *row0, const uint32_t *n_rows,
                                uint32_t col0, uint32_t n_cols, void *d_dst, void *stream) {
  if (!d_src || !d_dst || !row0 || !n_rows || n_ranges == 0) return fail(IE_B200_E_ARG, "ie_b200_mat_part: NULL argument");
  if (kind != IE_B200_MAT_F32 && kind != IE_B200_MAT_Q4 && kind != IE_B200_MAT_Q8 && kind != IE_B200_MAT_Q4K && kind != IE_B200_MAT_Q6K)
    return fail(IE_B200_E_ARG, "ie_b200_mat_part: matrix kind %d", kind);
  const uint32_t unit = kind == IE_B200_MAT_F32 ? 1u : (kind == IE_B200_MAT_Q4 || kind == IE_B200_MAT_Q8) ? 32u : 256u;
  if (n_cols == 0 || col0 % unit || n_cols % unit || (uint64_t)col0 + n_cols > cols)
    return fail(IE_B200_E_SIZE, "ie_b200_mat_part: columns [%u, %u) of %u (whole blocks of %u)", col0, col0 + n_cols, cols, unit);
  if (kind != IE_B200_MAT_F32)
    if (int e = check_shape("ie_b200_mat_part", kind, rows, cols)) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint32_t nb = cols / 32u, b0 = col0 / 32u, nbl = n_cols / 32u;
  PartAreas a = {};
  switch (kind) {
    case IE_B200_MAT_F32: a.n = 1, a.src[0] = col0 * 4u, a.dst[0] = 0, a.len[0] = n_cols * 4u; break;
    case IE_B200_MAT_Q4:
      a.n = 2;
      a.src[0] = b0 * 16u, a.dst[0] = 0, a.len[0] = nbl * 16u;
      a.src[1] = nb * 16u + b0 * 2u, a.dst[1] = nbl * 16u, a.len[1] = nbl * 2u;
      break;
    case IE_B200_MAT_Q8:
      a.n = 2;
      a.src[0] = b0 * 32u, a.dst[0] = 0, a.len[0] = nbl * 32u;
      a.src[1] = nb * 32u + b0 * 2u, a.dst[1] = nbl * 32u, a.len[1] = nbl * 2u;
      break;
    case IE_B200_MAT_Q4K:
      a.n = 2;
      a.src[0] = b0 * 16u, a.dst[0] = 0, a.len[0] = nbl * 16u;
      a.src[1] = nb * 16u + (b0 / 8u) * 16u, a.dst[1] = nbl * 16u, a.len[1] = (nbl / 8u) * 16u;
      break;
    default:  // Q6_K
      a.n = 4;
      a.src[0] = b0 * 16u, a.dst[0] = 0, a.len[0] = nbl * 16u;
      a.src[1] = nb * 16u + b0 * 8u, a.dst[1] = nbl * 16u, a.len[1] = nbl * 8u;
      a.src[2] = nb * 24u + b0 * 2u, a.dst[2] = nbl * 24u, a.len[2] = nbl * 2u;
      a.src[3] = nb * 26u + (b0 / 8u) * 2u, a.dst[3] = nbl * 26u, a.len[3] = (nbl / 8u) * 2u;
      break;
  }
  const size_t src_rowb = row_bytes_of(kind, cols), dst_rowb = row_bytes_of(kind, n_cols);
  uint32_t out_row = 0;
  for (uint32_t k = 0; k < n_ranges; k++) {
    if ((uint64_t)row0[k] + n_rows[k] > rows) return fail(IE_B200_E_SIZE, "ie_b200_mat_part: rows [%u, %u) of %u", row0[k], row0[k] + n_rows[k], rows);
    if (n_rows[k] == 0) continue;
    mat_part_kernel<<<n_rows[k], 128, 0, st>>>(static_cast<const uint8_t *>(d_src), src_rowb, static_cast<uint8_t *>(d_dst), dst_rowb, row0[k], out_row, a);
    IEB_LAUNCHED("mat_part_kernel");
    out_row += n_rows[k];
  }
  return IE_B200_OK;
}
