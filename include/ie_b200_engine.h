/* ie_b200_engine.h -- the decode engine of libie_b200.so: it owns the
 * weights, the activation arena and the KV cache of ONE GPU and runs a static
 * op list (the reference's "graph", src/model.h:177-331) for one token per
 * step or T tokens per run. It is what a backend behind the reference's
 * `struct backend` vtable (src/backend.h:7-49) drives: src/cuda.c of this
 * repository translates the reference's model / graph into these calls, and
 * the Python host (amd_c_b200/backend.py) builds the same op list itself.
 *
 * A one-token step is captured once into a CUDA graph and replayed; token id
 * and position travel through device scalars, so the graph is static.
 * All functions return 0 or a negative IE_B200_E_* code (see ie_b200.h);
 * handles are non-negative ints.
 */
#ifndef IE_B200_ENGINE_H
#define IE_B200_ENGINE_H

#include "ie_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ie_b200_engine ie_b200_engine;

#define IE_B200_NONE UINT64_MAX

/* Op kinds: the subset of the reference's op enum (src/model.h:177-231) that
 * llama / qwen2 graphs emit, plus two ops for tensor-parallel shards. */
enum {
  IE_B200_OP_EMBED = 0,   /* a = row tok of matrix `mat`                                   (OP_EMBED) */
  IE_B200_OP_RMSNORM = 1, /* b = rmsnorm(a) * vec, Q8 copy in qo; if res is set, first
                             a = a + res (the all-reduced partial of a sharded GEMV)      (OP_RMSNORM) */
  IE_B200_OP_QUANT = 2,   /* b = Q8(a)                                                     (OP_QUANT) */
  IE_B200_OP_GEMV = 3,    /* b = mat a (+ vec bias) (+ res); a is Q8 (f32 for MAT_F32)    (OP_GEMV_*) */
  IE_B200_OP_ROPE_KV = 4, /* rotate a (q, nh heads) and b (k); store b and c (v) in the
                             KV cache of `layer`                                          (OP_ROPE_KV) */
  IE_B200_OP_ATTN = 5,    /* b = attention(q = a, cache of `layer`), Q8 copy in qo       (OP_ATTN) */
  IE_B200_OP_SWIGLU = 6,  /* a = silu(a) * b, Q8 copy in qo                               (OP_SWIGLU);
                           * nh = 1: a holds interleaved (gate_i, up_i) pairs, b receives silu(gate_i) * up_i: the form
                           * for a gate / up matrix loaded with alternating rows (one 8-byte load per output) */
  IE_B200_OP_ARGMAX = 7,  /* b = {argmax(a), prob}                                        (OP_ARGMAX) */
  IE_B200_OP_ALLREDUCE = 8, /* c = (res if given, else c) + sum over the ranks of a (n floats per token): served by the
                               engine once a collective is attached (ie_b200_engine_set_collective); without one the
                               caller does it and an enqueue range only stops here (ie_b200_engine_enqueue) */
  IE_B200_OP_ADD = 9      /* c = a + b, n floats                                          (OP_ADD) */
};

typedef struct {
  int32_t kind;
  int32_t mat;   /* matrix handle or -1 */
  int32_t vec;   /* vector handle (bias / norm weight) or -1 */
  int32_t layer; /* KV-cache layer index (ROPE_KV, ATTN) */
  uint32_t n;    /* elements of a (the reference's op.n) */
  uint32_t nh;   /* ROPE_KV: query heads */
  /* arena byte offsets of token 0, IE_B200_NONE if absent; *_stride: bytes from one token row to the next */
  uint64_t a, b, c, qo, res;
  uint32_t a_stride, b_stride, c_stride, qo_stride, res_stride;
} ie_b200_op;

typedef struct {
  uint32_t n_head, n_kv, hd; /* heads held by this engine (a tensor-parallel rank holds a slice) */
  uint32_t n_ctx;            /* KV-cache positions */
  uint32_t n_kv_layers;      /* layers with a KV cache */
  uint32_t T_max;            /* most tokens of one run (graph.T of the reference) */
  uint32_t vocab;            /* logits per row */
  float eps;                 /* RMSNorm epsilon */
  int32_t neox;              /* RoPE pairs (i, i + hd/2) instead of (2i, 2i+1) */
  int32_t kv_f32;            /* 1: float KV cache (parity runs), 0: half */
  uint64_t arena_bytes;      /* activation arena (plan_arena's graph.arena, src/plan.c:24) */
  uint64_t logits_off, argmax_off; /* arena offsets of the logits and of the {index, prob} pair */
  uint32_t logits_stride, argmax_stride;
} ie_b200_engine_desc;

/* gpu_open (src/hip.c:568): allocate arena, KV cache and scratch on the current CUDA device. */
int ie_b200_engine_create(const ie_b200_engine_desc *desc, ie_b200_engine **out);
/* backend.close (src/backend.h:12). */
void ie_b200_engine_destroy(ie_b200_engine *e);

/* Upload one matrix and re-lay it out for streaming; returns its handle.
 *  _gguf: raw GGUF tensor bytes on the host (what model_load reads, src/model.c:401).
 *  _ref:  the reference loader's repacked arrays, as its matrix sink receives them
 *         (ie_mat_sink, src/model.h:160-163; the upload of src/hip.c:278-303). h_qs NULL for MAT_F32
 *         (h_qw then points at the floats).
 *  _device: adopt a matrix already in the streaming layout in device memory (not freed by the engine). */
int ie_b200_engine_add_mat_gguf(ie_b200_engine *e, int ggml_type, uint32_t rows, uint32_t cols, const void *h_bytes);
int ie_b200_engine_add_mat_ref(ie_b200_engine *e, int kind, uint32_t rows, uint32_t cols, const void *h_qw, const void *h_qs);
int ie_b200_engine_add_mat_device(ie_b200_engine *e, int kind, uint32_t rows, uint32_t cols, const void *d_data);
/* A tensor-parallel shard's part of a matrix given as _ref gives the whole one: the row ranges [row0[k], row0[k] + n_rows[k])
 * one after the other (q / k / v heads or the gate / up slices of a merged matrix: src/model.h:55-58) and the columns
 * [col0, col0 + n_cols) (whole blocks: 32 columns for MAT_Q4, 256 for the K kinds). No reference counterpart. */
int ie_b200_engine_add_mat_ref_part(ie_b200_engine *e, int kind, uint32_t rows, uint32_t cols, const void *h_qw, const void *h_qs, uint32_t n_ranges,
                                    const uint32_t *row0, const uint32_t *n_rows, uint32_t col0, uint32_t n_cols);
/* A float vector (norm weight, bias); returns its handle. */
int ie_b200_engine_add_vec(ie_b200_engine *e, const float *h_f, uint32_t n);
/* RoPE tables [n_ctx][hd / 2] (graph.rope_cos / rope_sin, src/model.c:1655-1664). */
int ie_b200_engine_set_rope(ie_b200_engine *e, const float *h_cos, const float *h_sin);
/* The op list; i_head = first op of the output head (graph.i_head): a run with last_only executes the
 * ops before it for all T tokens and the head for the last token only (src/hip.c:1560-1563). */
int ie_b200_engine_set_ops(ie_b200_engine *e, const ie_b200_op *ops, uint32_t n_ops, uint32_t i_head);
/* Tensor parallel (no reference counterpart: the reference drives one device): attach the connected
 * all-reduce state of include/ie_b200_tp.h. The engine then serves its ALLREDUCE ops itself (fused with the
 * RMSNORM that follows where it can) and, after ARGMAX, exchanges the ranks' local winners, so step / decode /
 * run return the argmax over the whole vocabulary on every rank; vocab_offset = first vocabulary row of this
 * shard's output head. Every rank must make the same calls in the same order. The state is not owned. */
struct ie_b200_allreduce;
int ie_b200_engine_set_collective(ie_b200_engine *e, struct ie_b200_allreduce *ar, uint32_t vocab_offset);

/* backend.step (src/backend.h:10): one token at position pos; h_logits (vocab floats) may be NULL;
 * *next = the argmax token; *ms (may be NULL) = device time of the step. Host buffers in and out. */
int ie_b200_engine_step(ie_b200_engine *e, uint32_t tok, uint32_t pos, float *h_logits, uint32_t *next, double *ms);
/* A bounded wait that ran out leaves the device error word set, and every later step / decode / run reports
 * IE_B200_E_DEVICE (the all-reduce kernels then stop waiting: they look once and go on). Once the caller has dealt
 * with the failure (the ranks of a tensor-parallel run are back in step: same number of calls made on each), this
 * clears the word. */
int ie_b200_engine_clear_error(ie_b200_engine *e);
/* How a one-token step (step, decode) runs. 1 (default): as a CUDA graph of one kernel per op, chained by programmatic
 * dependent launch. 2: as ONE persistent cooperative kernel that walks the whole op list with grid barriers between dependent
 * ops and loops over the K tokens of a decode call by itself -- the role of the reference's megakernel (kernels/ie_mk.c:43-95,
 * grid barrier kernels/ie_kernels.c:417-463, recorder src/hip.c:445-566); IE_B200_E_STATE where the op list or the shapes have
 * no program (it needs the half-precision cache, heads of 64 or 128 and the llama / qwen2 op patterns). 0: the kernel where
 * it can run, else the graph. On B200 the graph is the faster of the two (a kernel boundary under programmatic dependent launch
 * costs less than a software barrier over 148 CTAs), which is why it is the default; the environment variable
 * IE_B200_STEP=graph|kernel|auto sets the default of new engines.
 * ie_b200_engine_step_is_kernel: 1 if steps of the current op list run as the persistent kernel. */
int ie_b200_engine_set_step_mode(ie_b200_engine *e, int mode);
int ie_b200_engine_step_is_kernel(ie_b200_engine *e);
/* Where the persistent kernel's time goes: with enable != 0, CTA 0 of the kernel sums, per kind of phase (the PH_* numbering
 * of the kernel: 0 embed, 1 GEMV, 2 attention, 3 merge, 4 argmax, 5 finish, 6 reduce, 7 argmax exchange), the time it spent
 * between leaving one grid barrier and arriving at the next (its own work in the phase) and the time between arriving and
 * leaving (waiting for the slowest CTA). h_ms36 (may be NULL) receives the sums since the last call as 12 x {ms, ms, count}:
 * entries 0..7 per phase kind {work, barrier wait, barriers}; entries 8..11 the GEMV phases by the way their activations are
 * staged (8 a Q8 buffer, 9 RMSNorm + Q8, 10 SwiGLU + Q8, 11 kept from the phase before) {staging, rows loop of warp 0, phases}.
 * Every call clears the sums; enable = 0 switches the record off. The role of the reference's
 * per-op profile of its megakernel (src/hip.c:1840-1900, IE_PROFILE). */
int ie_b200_engine_phase_times(ie_b200_engine *e, int enable, double *h_ms36);
/* Failure injection from the host (for tests of the recovery path; nothing on the GPU faults): raises the abort
 * flag that a CTA of the persistent kernel raises when one of its bounded waits runs out. The next step / decode
 * then ends at once with the device error word set and returns IE_B200_E_DEVICE; ie_b200_engine_clear_error
 * lowers the flag again. */
int ie_b200_engine_inject_abort(ie_b200_engine *e);
/* K greedy tokens without a host round trip per token: the step graph is replayed K times and a one-CTA
 * kernel feeds each argmax back as the next token on the device (what the decode loop of src/main.c:192-225
 * does on the host). h_out: the K generated tokens; *ms: device time of the K steps. K <= 4096 per call. */
int ie_b200_engine_decode(ie_b200_engine *e, uint32_t tok, uint32_t pos, uint32_t K, uint32_t *h_out, double *ms);
/* backend.run (src/backend.h:20), section 0: T tokens at positions pos .. pos + T - 1; out: T argmax
 * tokens (only out[T-1] is meaningful when last_only), prob: T floats or NULL. */
int ie_b200_engine_run(ie_b200_engine *e, const uint32_t *toks, uint32_t T, uint32_t pos, int last_only, uint32_t *out, float *prob);
/* step, decode and run in two halves each: _begin enqueues the work and the copies of its results into the engine's own
 * pinned memory and returns without waiting; _end waits and hands the results out (step = step_begin + step_end, and so
 * on). For a host thread that drives the shards of one model on several GPUs (ie_b200_tp_group in ie_b200_tp.h): it
 * begins every shard before it ends any, since each shard's kernels wait for the others' rows. No reference counterpart. */
int ie_b200_engine_step_begin(ie_b200_engine *e, uint32_t tok, uint32_t pos, int timed);
int ie_b200_engine_step_end(ie_b200_engine *e, float *h_logits, uint32_t *next, double *ms);
int ie_b200_engine_decode_begin(ie_b200_engine *e, uint32_t tok, uint32_t pos, uint32_t K);
int ie_b200_engine_decode_end(ie_b200_engine *e, uint32_t *h_out, double *ms);
int ie_b200_engine_run_begin(ie_b200_engine *e, const uint32_t *toks, uint32_t T, uint32_t pos, int last_only);
int ie_b200_engine_run_end(ie_b200_engine *e, uint32_t *out, float *prob);
/* backend.read_rows / copy_rows (src/backend.h:27-31) on arena offsets: n rows of `stride` bytes. */
int ie_b200_engine_read_rows(ie_b200_engine *e, uint64_t off, uint32_t stride, uint32_t r0, uint32_t n, void *h_dst);
int ie_b200_engine_copy_rows(ie_b200_engine *e, uint64_t dst_off, uint32_t dst_stride, uint32_t d0, uint64_t src_off, uint32_t src_stride,
                             uint32_t r0, uint32_t n, uint32_t row_bytes, int zero);

/* backend.topk (src/backend.h:33-37) on arena offsets: the K largest of the first nv floats of n rows from row r0, to the
 * host; returns 1 if done, 0 if K is too large for the kernel (the caller then selects on the host), negative on an error.
 * backend.snap's row copy (src/backend.h:42-48) uses read_rows and write_rows: llama / qwen2 keep no state outside the KV
 * cache, so a snapshot is row 0 of the hbuf buffer, if any. */
int ie_b200_engine_topk(ie_b200_engine *e, uint64_t off, uint32_t stride, uint32_t r0, uint32_t n, uint32_t nv, uint32_t K, float *h_val, uint32_t *h_idx);
int ie_b200_engine_write_rows(ie_b200_engine *e, uint64_t off, uint32_t stride, uint32_t r0, uint32_t n, const void *h_src);

/* For callers that interleave their own work (collectives of a tensor-parallel run) with the ops:
 * write token ids and the first position to the device scalars on `stream`, then enqueue ops
 * [first, last) for T tokens on `stream`. OP_ALLREDUCE ops inside the range are skipped. */
int ie_b200_engine_set_input(ie_b200_engine *e, const uint32_t *toks, uint32_t T, uint32_t pos, void *stream);
int ie_b200_engine_enqueue(ie_b200_engine *e, uint32_t first, uint32_t last, uint32_t T, void *stream);
/* As enqueue, restricted to the ops whose kind bit (1 << IE_B200_OP_*) is set in kind_mask: lets a
 * benchmark time one kernel family on the shapes of the real op list. */
int ie_b200_engine_enqueue_kinds(ie_b200_engine *e, uint32_t first, uint32_t last, uint32_t kind_mask, uint32_t T, void *stream);
/* Device address of the arena (to hand buffers to a collective) and of the {tokens[T_max], pos} scalars. */
void *ie_b200_engine_arena(ie_b200_engine *e);
void *ie_b200_engine_input_scalars(ie_b200_engine *e);
/* Bytes of weights this engine streams per decode step (the GEMVs of the op list): the reference's
 * graph.weight_bytes_per_token (src/model.c:1617-1635), 18 B per Q4_0/Q4_K block, 26.25 B per Q6_K block. */
uint64_t ie_b200_engine_weight_bytes_per_token(ie_b200_engine *e);
/* Kernels launched per one-token step (the nodes of the captured graph). */
uint32_t ie_b200_engine_launches_per_step(ie_b200_engine *e);

#ifdef __cplusplus
}
#endif
#endif
