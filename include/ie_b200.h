/* ie_b200.h -- the C ABI of libie_b200.so: hand-written sm_100a CUDA kernels
 * for the decode hot path of amd-infer, and a small engine that runs a
 * decode-step op list with them.
 *
 * Conventions
 *  - Plain C types only. Pointers named d_* are device pointers, h_* host
 *    pointers. `stream` is a cudaStream_t passed as void* (NULL: the legacy
 *    default stream).
 *  - Every function returns 0 on success or a negative IE_B200_E_* code;
 *    ie_b200_last_error() gives the message of the calling thread's last
 *    failure. Nothing here prints or exits: the C backend above this ABI
 *    (src/cuda.c) turns an error into the reference's die-with-message
 *    convention (src/common.c:6-14 of the reference).
 *  - There is no CPU fallback: without a CUDA device every launch fails with
 *    IE_B200_E_CUDA.
 *
 * Each entry point cites the reference interface it stands in for
 * (path:line inside the amd-infer tree).
 */
#ifndef IE_B200_H
#define IE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  IE_B200_OK = 0,
  IE_B200_E_ARG = -1,   /* a NULL or misaligned pointer, an unknown kind */
  IE_B200_E_SIZE = -2,  /* a size outside what the kernels support */
  IE_B200_E_CUDA = -3,  /* a CUDA runtime error (message in last_error) */
  IE_B200_E_STATE = -4, /* engine call out of order */
  IE_B200_E_DEVICE = -5 /* a kernel set the device error word (a bounded wait ran out) */
};

/* Matrix kinds: the reference's MAT_* numbering (src/model.h:15). */
enum { IE_B200_MAT_Q4 = 0, IE_B200_MAT_F32 = 1, IE_B200_MAT_Q8 = 2, IE_B200_MAT_Q4K = 3, IE_B200_MAT_Q6K = 4 };

/* GGML tensor types accepted by the GGUF repack (src/common.h:11-13). */
enum { IE_B200_GGML_F32 = 0, IE_B200_GGML_Q4_0 = 2, IE_B200_GGML_Q8_0 = 8, IE_B200_GGML_Q4_K = 12, IE_B200_GGML_Q6_K = 14 };

const char *ie_b200_last_error(void);
/* Number of CUDA devices visible (0 without a driver or a GPU). */
int ie_b200_device_count(void);
/* How many kernels this library has launched in this process (all threads). */
uint64_t ie_b200_launch_count(void);

/* ---------------------------------------------------------------- layout
 * The streaming layout of a quantised matrix ("row panels"): each row is one
 * contiguous, 16-byte aligned run of bytes holding, for its nb = cols/32
 * blocks, first all 16-byte nibble blocks, then the per-block scales, then
 * (K kinds) the per-super-block constants; rows follow each other at
 * ie_b200_row_bytes(). A warp that owns a row therefore streams one
 * contiguous span with 16-byte loads, and a group of rows is one bulk copy.
 *   Q4_0: nb x 16 B nibbles (the GGUF nibble bytes), nb x f16 d          = 18 B/block
 *   Q8_0: nb x 32 B signed bytes (the GGUF weight bytes), nb x f16 d     = 34 B/block
 *   Q4_K: nb x 16 B nibbles (Q4_0 order per sub-block), nb/8 x 16 B
 *         {f16 d, f16 dmin, 8 x 12 bit (sc | mn << 6)}                     = 18 B/block
 *   Q6_K: nb x 16 B low nibbles, nb x 8 B high-bit words, nb x 2 B
 *         (sc0 | sc1 << 8), nb/8 x f16 d                                   = 26.25 B/block
 * Replaces the word/scale arrays of the reference's `mat`
 * (src/model.h:15-43, index maps core/ie_core.h:72-77, :261-263, :323-327).
 * Block ownership (lane l <- blocks l, l+32, ...) and block contents are
 * unchanged; only addresses differ. F32 matrices stay rows x cols floats. */
size_t ie_b200_row_bytes(int kind, uint32_t cols);
size_t ie_b200_mat_bytes(int kind, uint32_t rows, uint32_t cols);

/* GGUF tensor bytes (already on the device) -> streaming layout. Stands in
 * for repack_q4 / repack_q8 / repack_q4k / repack_q6k (src/model.c:205, :221, :246, :271).
 * ggml_type: IE_B200_GGML_*; F32 is a plain copy. */
int ie_b200_repack_gguf(int ggml_type, const void *d_src, uint32_t rows, uint32_t cols, void *d_dst, void *stream);
/* The reference's repacked arrays qw / qs (on the device, as ie_mat_sink
 * receives them from model_load, src/model.c:649-658) -> streaming layout. */
int ie_b200_repack_ref(int kind, const void *d_qw, const void *d_qs, uint32_t rows, uint32_t cols, void *d_dst, void *stream);
/* A part of a matrix that is already in the streaming layout, again in the streaming layout: n_ranges row ranges
 * [row0[k], row0[k] + n_rows[k]) one after the other, columns [col0, col0 + n_cols) (whole blocks: 32 columns for
 * MAT_Q4 / MAT_Q8, 256 for the K kinds, any for MAT_F32). row0 / n_rows are host arrays. What a tensor-parallel shard holds of a
 * matrix; the reference, which runs on one device, has no counterpart. */
int ie_b200_mat_part(int kind, const void *d_src, uint32_t rows, uint32_t cols, uint32_t n_ranges, const uint32_t *row0, const uint32_t *n_rows,
                     uint32_t col0, uint32_t n_cols, void *d_dst, void *stream);

/* ------------------------------------------------------------- kernels */

/* Q8 activation quantiser for T token rows: per 32 floats d = amax/127,
 * q = round(x/d), asum = sum q; output buffer [int8 x 32nb][f32 d x nb]
 * [u32 asum x nb]. Bit-exact with cpu_quant_q8 (src/cpu.c:36-53); argument
 * list after ie_quant_q8 {x,q,nb,xs,qs} (src/hip.c:924). Strides in bytes. */
int ie_b200_quant_q8(const float *d_x, void *d_q, uint32_t nb, uint32_t T, size_t x_stride, size_t q_stride, void *stream);

/* y[T][rows] = W x (+bias) (+res): W in the streaming layout, x a Q8 buffer
 * per token (f32 for MAT_F32). One warp per (row, token); lane l accumulates
 * blocks l, l+32, ... in order and the warp reduces by shuffle-down 16, 8, 4,
 * 2, 1, so the result equals cpu_gemv_q4 / _q4k / _q6k / _q8 / cpu_gemv_f32 bit for
 * bit (src/cpu.c:64-174, :238-249); epilogue y = acc (+bias[r]), y = res[r] + y
 * (src/cpu.c:515-520). Argument list after ie_gemv_q4q8
 * {qw,qs,xq,y,rows,nb,bias,res,...} (src/hip.c:930) and its multi-token
 * forms {...,T,xs,ys,rs} (src/hip.c:1000). res may alias y. */
int ie_b200_gemv(int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_x, float *d_y, const float *d_bias,
                 const float *d_res, uint32_t T, size_t x_stride, size_t y_stride, size_t res_stride, void *stream);

/* The prompt-chunk GEMM on the int8 mma.sync path (kept beside ie_b200_gemm_tc, which replaced it as the default:
 * it needs no scratch and takes any alignment): y[T][rows] = W Q8(x) (+bias) (+res) for T >= 17 tokens with the weights read once
 * per 128 tokens; the role of ie_gemm_q4kr / ie_gemm_q6kr (kernels/ie_kernels.c:1315-1465, :2015-2158;
 * dispatch src/hip.c:965-1003), for MAT_Q4 as well. Every 32-weight block dot is one int8 tensor-core product
 * (exact int32, as the reference's MMA trick), scaled in fp32 block after block; the result equals
 * ie_b200_gemv's to fp32 rounding (the order of the block sums differs), not bit for bit -- as in the
 * reference. Same operands as ie_b200_gemv (Q8 buffers per token; strides in bytes, multiples of 4). */
int ie_b200_gemm(int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_xq, float *d_y, const float *d_bias,
                 const float *d_res, uint32_t T, size_t x_stride, size_t y_stride, size_t res_stride, void *stream);

/* The same GEMM on the tcgen05 tensor cores with the accumulators in tensor memory: the prompt-chunk default. Nothing is
 * scaled inside the main loop: a pre-pass expands the Q8 rows to f16 pairs x = x_hi + x_lo once per call, producer warps
 * dequantise each 256-row x 32-column weight block to f16 pairs w = w_hi + w_lo in shared memory, and one thread issues
 * w_hi x_hi + w_hi x_lo + w_lo x_hi as tcgen05.mma kind::f16 (M 128, N up to 256 tokens, fp32 accumulation over the whole K);
 * matrices with few rows are split along K, the partial sums added in split order by a second kernel. Equal to ie_b200_gemv
 * to fp32 rounding. d_scratch: ie_b200_gemm_tc_scratch_bytes() bytes, 256-byte aligned (the expanded activations and the
 * K-split partials); d_err (may be NULL): set to 5 if a bounded wait inside the kernel ran out. x_stride a multiple of 16.
 * w_exp: the power of two the weights are scaled by before they are split into half-precision terms, as ie_b200_mat_tc_exp
 * gives it for the matrix (once, at load time: it reads the matrix's scale fields and synchronises the stream): the largest
 * possible weight times 2^w_exp stays below 8192, and small weights keep their low term out of the subnormal range. */
int ie_b200_mat_tc_exp(int kind, const void *d_w, uint32_t rows, uint32_t cols, int *h_exp, void *stream);
size_t ie_b200_gemm_tc_scratch_bytes(uint32_t rows, uint32_t cols, uint32_t T);
int ie_b200_gemm_tc(int kind, const void *d_w, uint32_t rows, uint32_t cols, int w_exp, const void *d_xq, float *d_y, const float *d_bias,
                    const float *d_res, uint32_t T, size_t x_stride, size_t y_stride, size_t res_stride, void *d_scratch, size_t scratch_bytes,
                    uint32_t *d_err, void *stream);

/* The one-token GEMV of a decode step, same result as ie_b200_gemv with T = 1: every warp of a persistent grid
 * streams its rows straight from HBM into registers with 16-byte loads (up to 16 per lane in flight), and the
 * launch uses programmatic dependent launch: the first loads are issued before the kernel waits for its
 * predecessor in the stream (the weights do not depend on it; the activations are read only after the previous
 * kernel has completed). Replaces ie_gemv_q4q8 / _q4kq8 / _q6kq8 at decode (kernels/ie_kernels.c:310, :401, :675). */
int ie_b200_gemv_stream(int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_xq, float *d_y, const float *d_bias,
                        const float *d_res, void *stream);
/* The same with RMSNorm + the Q8 quantiser of the f32 vector d_x (cols floats) folded into the prologue: the role
 * of the reference's fused norm tail (gemv_norm_tail, kernels/ie_kernels.c:274-285; src/model.c:1265-1293) moved
 * to the consumer side. d_xn_out / d_xq_out (may be NULL): the normalised vector and its Q8 copy, written once. */
int ie_b200_norm_gemv_stream(int kind, const void *d_w, uint32_t rows, uint32_t cols, const float *d_x, const float *d_norm_w, float eps,
                             float *d_xn_out, void *d_xq_out, float *d_y, const float *d_bias, const float *d_res, void *stream);

/* SwiGLU moved into the GEMVs around it (one launch less per layer; the tensor-parallel step uses it): ie_b200_gemv_swiglu is
 * the gate / up GEMV over a matrix whose rows alternate gate_i, up_i -- the warp that owns a pair writes d_h[i] = silu(gate_i) *
 * up_i (rows / 2 floats, the arithmetic of ie_b200_swiglu_il) instead of the two rows; ie_b200_quant_gemv_stream is the GEMV
 * that follows, with the Q8 quantiser of the f32 vector d_x (cols floats) in its prologue (d_xq_out, may be NULL: the Q8 copy,
 * written once). Together they give the bits of GEMV, ie_b200_swiglu_il, GEMV (src/cpu.c:579-582 between two cpu_gemv_q4). */
int ie_b200_gemv_swiglu(int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_xq, float *d_h, void *stream);
int ie_b200_quant_gemv_stream(int kind, const void *d_w, uint32_t rows, uint32_t cols, const float *d_x, void *d_xq_out, float *d_y, const float *d_bias,
                              const float *d_res, void *stream);

/* The one-token GEMV with the reference's fused norm tail (gemv_norm_tail, kernels/ie_kernels.c:274-285;
 * IE_NORM_FUSE, src/model.c:1265-1293): after y = W x (+bias) (+res) is complete, the last CTA to finish writes
 * d_xn_out = rmsnorm(y) * d_norm_w and its Q8 copy d_xq_out (either may be NULL). rows % 32 == 0. d_counter: two
 * u32 in device memory, zero before the first launch and left zero by every launch (they count the CTAs that
 * have finished); launches that share them must not overlap on the GPU. */
int ie_b200_gemv_norm_tail(int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_xq, float *d_y, const float *d_bias,
                           const float *d_res, const float *d_norm_w, float eps, float *d_xn_out, void *d_xq_out, uint32_t *d_counter,
                           void *stream);

/* Test hook: the int32 dot of every (row, block) of a Q4_0 / Q8_0 / Q4_K matrix
 * (Q4_K: the unsigned-nibble dot) and, for Q6_K, the two half dots
 * (dots[2 (r nb + b) + h]); what core/ie_core.h:161, :220, :281, :385 define. */
int ie_b200_block_dots(int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_xq, int32_t *d_dots, void *stream);

/* Row `tok` of the token embedding as floats (MAT_Q4, MAT_Q8 or MAT_F32):
 * mat_row (src/cpu.c:252-274), ie_embed_q4 / _f32 (kernels/ie_kernels.c:171-191).
 * d_tok: T token ids on the device. */
int ie_b200_embed(int kind, const void *d_w, uint32_t cols, const uint32_t *d_tok, float *d_out, uint32_t T, size_t out_stride,
                  void *stream);

/* y = x * rsqrt(mean x^2 + eps) * w, optionally with the Q8 copy of y
 * (d_q != NULL): rmsnorm (src/cpu.c:276-281) + cpu_quant_q8; ie_rmsnorm
 * {x,w,y,n,eps,q,xs,ys,qs} (src/hip.c:917). The sum of squares is a tree sum
 * (differs from the CPU's sequential sum by rounding only). */
int ie_b200_rmsnorm(const float *d_x, const float *d_w, float *d_y, uint32_t n, float eps, void *d_q, uint32_t T, size_t x_stride,
                    size_t y_stride, size_t q_stride, void *stream);

/* a = silu(a) * b, optionally with the Q8 copy (src/cpu.c:579-582, ie_swiglu
 * kernels/ie_kernels.c:2458). */
int ie_b200_swiglu(float *d_a, const float *d_b, uint32_t n, void *d_q, uint32_t T, size_t a_stride, size_t q_stride, void *stream);

/* SwiGLU for the interleaved layout gu[2i] = gate_i, gu[2i + 1] = up_i (what a GEMV over a matrix whose rows alternate
 * gate_i, up_i produces): h[i] = silu(gate_i) * up_i, same arithmetic and Q8 copy as ie_b200_swiglu. The decode engine
 * and the prompt chunks both use it after a GEMV over the interleaved matrix. */
int ie_b200_swiglu_il(const float *d_gu, float *d_h, uint32_t n, void *d_q, uint32_t T, size_t gu_stride, size_t h_stride, size_t q_stride,
                      void *stream);

/* RoPE of q (nq heads) and k (nkv heads) in place with the table rows of
 * each token's position, then store k and v of that position into the KV
 * cache (half or float elements): OP_ROPE_KV (src/cpu.c:537-546), ie_rope_kv
 * {q,k,v,kc,vc,cs,sn,nq,nkv,hd,neox} (src/hip.c:1284). d_pos: first position
 * (device scalar); token t is at *d_pos + t. Cache row = position % kv_len. */
int ie_b200_rope_kv(float *d_q, float *d_k, const float *d_v, void *d_kc, void *d_vc, const float *d_cos, const float *d_sin,
                    const uint32_t *d_pos, uint32_t nq, uint32_t nkv, uint32_t hd, int neox, int kv_f32, uint32_t kv_len, uint32_t T,
                    size_t qkv_stride, void *stream);

/* Split-KV decode attention for T tokens (token t attends to positions
 * 0 .. *d_pos + t): K/V of a KV head are streamed once for all its query
 * heads; splits of the position range write (max, sum, out[hd]) partials to
 * d_part and the last split to finish merges them. Optional Q8 copy of the
 * output. The role of ie_attn_kv {q,kc,vc,part,out,pos,hd,nh,nkv,smax,...}
 * (src/hip.c:1492-1493, kernels/ie_kernels.c:2721) and, for parity, of
 * attention() (src/cpu.c:301-329). d_part: ie_b200_attn_part_bytes() of
 * scratch; d_count: ie_b200_attn_count_words() zeroed u32 counters (left zero). */
size_t ie_b200_attn_part_bytes(uint32_t n_head, uint32_t hd, uint32_t n_ctx, uint32_t T);
size_t ie_b200_attn_count_words(uint32_t n_head, uint32_t T);
int ie_b200_attn_decode(const float *d_q, const void *d_kc, const void *d_vc, float *d_out, void *d_oq, const uint32_t *d_pos,
                        uint32_t n_head, uint32_t n_kv, uint32_t hd, int kv_f32, uint32_t kv_len, uint32_t n_ctx, uint32_t T,
                        size_t q_stride, size_t out_stride, size_t oq_stride, void *d_part, uint32_t *d_count, void *stream);

/* One decode token: OP_ROPE_KV and OP_ATTN in one kernel. d_q / d_k / d_v are the un-rotated q, k and the v of the
 * position *d_pos (the parts of the qkv buffer); q is rotated in registers (it is not written back), k is rotated
 * and stored with v into the caches and taken into the attention from registers. Same results as ie_b200_rope_kv
 * followed by ie_b200_attn_decode (src/cpu.c:537-546 + :301-329; ie_rope_kv + ie_attn_kv, src/hip.c:1284, :1492). */
int ie_b200_attn_decode_fused(const float *d_q, const float *d_k, const float *d_v, void *d_kc, void *d_vc, const float *d_cos,
                              const float *d_sin, float *d_out, void *d_oq, const uint32_t *d_pos, uint32_t n_head, uint32_t n_kv, uint32_t hd,
                              int neox, int kv_f32, uint32_t kv_len, uint32_t n_ctx, void *d_part, uint32_t *d_count, void *stream);

/* The same step (OP_ROPE_KV + OP_ATTN of one token on the half-precision cache) as the persistent step kernel runs it
 * per layer (include/ie_b200_engine.h, ie_b200_engine_set_step_mode): a cooperative launch of one CTA per SM whose groups
 * of four warps each take a (KV head, split) item -- one 64-position tile per item while there are more groups than tiles --
 * followed, behind a grid barrier, by the merge of the splits' records (one warp per head) into d_out and its Q8 copy d_oq.
 * The role of ie_attn_kv inside the reference's megakernel (kernels/ie_mk.c:43-95, kernels/ie_kernels.c:2721-2868). d_qkv: the
 * un-rotated q | k | v of position *d_pos (n_head + 2 n_kv heads of hd floats); hd 64 or 128, at most 8 query heads per KV head.
 * d_scratch: ie_b200_attn_persistent_scratch_bytes() bytes, 16-byte aligned, any contents; d_err: the device error word
 * (set if a bounded wait of the kernel ran out). */
size_t ie_b200_attn_persistent_scratch_bytes(uint32_t n_head, uint32_t n_kv, uint32_t hd);
int ie_b200_attn_persistent(const float *d_qkv, void *d_kc, void *d_vc, const float *d_cos, const float *d_sin, float *d_out, void *d_oq,
                            const uint32_t *d_pos, uint32_t n_head, uint32_t n_kv, uint32_t hd, int neox, uint32_t kv_len, void *d_scratch,
                            uint32_t *d_err, void *stream);

/* Causal attention of a prompt chunk: T tokens at positions *d_pos .. *d_pos + T - 1 whose (rotated) K / V rows are
 * already in the half-precision cache (ie_b200_rope_kv); token t sees positions 0 .. *d_pos + t. The role of
 * ie_attn_pfg / ie_attn_fa (kernels/ie_kernels.c:3471-3693; dispatch src/hip.c:1432-1463): 16 / G consecutive tokens
 * of one KV head share one pass over the cache on the tensor cores (f16 MMA, fp32 softmax and accumulation, q and p
 * carried as two f16 terms). hd 64 or 128; d_q rows of n_head * hd floats (already rotated), output rows and their
 * Q8 copies (d_oq may be NULL) as ie_b200_attn_decode; strides in bytes. No scratch. */
int ie_b200_attn_prefill(const float *d_q, const void *d_kc, const void *d_vc, float *d_out, void *d_oq, const uint32_t *d_pos,
                         uint32_t n_head, uint32_t n_kv, uint32_t hd, uint32_t kv_len, uint32_t T, size_t q_stride, size_t out_stride,
                         size_t oq_stride, void *stream);

/* First index of the maximum of each of T rows, and the softmax probability
 * of that maximum: OP_ARGMAX (src/cpu.c:608-614), ie_argmax
 * {x,n,out,part,count,ng} (src/hip.c:1537). out: {u32 index, f32 prob} per row.
 * d_part: ie_b200_argmax_part_bytes(T) of scratch. */
size_t ie_b200_argmax_part_bytes(uint32_t T);
int ie_b200_argmax(const float *d_x, uint32_t n, uint32_t *d_out, uint32_t T, size_t x_stride, size_t out_stride, void *d_part,
                   void *stream);

/* The K largest values of each of T rows and their indices, per row value descending, equal values smaller index first:
 * backend.topk (src/backend.h:33-37; ie_topk_part / ie_topk_merge, kernels/ie_kernels.c:4018-4035, launcher src/hip.c:1762-1782).
 * K <= 64 and at most 6144 candidates per row (K times the 2048-value slices of a row); otherwise IE_B200_E_SIZE, and the
 * caller selects on the host as the reference does when its backend returns 0. d_val / d_idx: T * K entries;
 * d_scratch: ie_b200_topk_scratch_bytes() bytes. */
size_t ie_b200_topk_scratch_bytes(uint32_t nv, uint32_t K, uint32_t T);
int ie_b200_topk(const float *d_x, uint32_t nv, uint32_t K, uint32_t T, size_t x_stride, float *d_val, uint32_t *d_idx, void *d_scratch, void *stream);

/* ie_b200_argmax for callers that cannot allocate device memory. It has no counterpart in the reference; it
 * exists for hosts that have already committed all device memory (arena and KV cache sized to fill the GPU at
 * start-up) or that call from a place where the CUDA allocator must not be entered. Same result as
 * ie_b200_argmax, but the partial results live in a 64 KB array inside the library's device image (held by every
 * GPU that loads the library, until exit) instead of caller-provided scratch.
 *  - At most ie_b200_argmax_static_max_rows() (64) rows per call; more is refused with IE_B200_E_SIZE.
 *  - Nothing is allocated or freed, by this call or by anything it uses.
 *  - The first call on a device looks up the array's device address (once per device); make that first call
 *    before starting any stream capture.
 *  - All calls on a device share the array and it keeps the last call's partials; every call overwrites the
 *    entries it reads, so nothing needs clearing, but two calls that overlap on the GPU (different streams
 *    without an ordering between them) race on it. Issue them on one stream or order them with events. */
uint32_t ie_b200_argmax_static_max_rows(void);
int ie_b200_argmax_static(const float *d_x, uint32_t n, uint32_t *d_out, uint32_t T, size_t x_stride, size_t out_stride, void *stream);

#ifdef __cplusplus
}
#endif
#endif
