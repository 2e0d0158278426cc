/* ie_b200_tp.h -- the cross-GPU piece of a tensor-parallel decode step: a one-shot all-reduce (+ residual add)
 * over peer memory for the dim-float partial sums that follow every K-split GEMV (attn_output, ffn_down).
 * The reference has no counterpart: it runs on one device (src/hip.c:574 sets device 0 and nothing else);
 * this is the exchange step that sharding its GEMVs by rows / columns needs (one per half layer).
 *
 * One process per GPU. Each rank creates its state, the 128-byte handle blobs are exchanged by the host
 * (any transport: the Python host uses torch.distributed all_gather), and connect() maps the peers' buffers
 * with CUDA IPC. The kernel then pushes with plain peer stores over NVLink and sums in rank order from local
 * memory, so every rank gets the same bits; its waits are bounded (2 s) and report through a device error word.
 */
#ifndef IE_B200_TP_H
#define IE_B200_TP_H

#include "ie_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ie_b200_allreduce ie_b200_allreduce;

/* Receive buffers for vectors of up to max_floats (a multiple of 4) on the current device; world <= 8. */
int ie_b200_ar_create(uint32_t rank, uint32_t world, uint32_t max_floats, ie_b200_allreduce **out);
/* This rank's 128-byte IPC handle blob (one allocation: receive buffers, flags; the rest is zero). */
int ie_b200_ar_handles(ie_b200_allreduce *a, void *h_out128);
/* h_all: the world blobs in rank order (world * 128 bytes). Not needed when world == 1. */
int ie_b200_ar_connect(ie_b200_allreduce *a, const void *h_all);
/* The same for states that live in THIS process on GPUs that can address each other (or on one GPU): all[j] is
 * rank j's state. For hosts that drive several GPUs from one process, and for exercising the bounded waits: a
 * call made on one rank only finds no partner, gives up after the time limit, sets the error word and returns. */
int ie_b200_ar_connect_local(ie_b200_allreduce *a, ie_b200_allreduce *const *all);
/* out = (res ? res : 0) + sum over ranks of part, n floats (a multiple of 4). Every rank must make the same
 * sequence of calls. d_err (may be NULL): set to 3 if a peer did not arrive within the time limit. out may
 * alias res. */
int ie_b200_ar_allreduce_add(ie_b200_allreduce *a, const float *d_part, const float *d_res, float *d_out, uint32_t n, uint32_t *d_err,
                             void *stream);
/* The decode step's form, one kernel of one CTA: x = x + sum over ranks of part (rank order), then
 * xn = x * rsqrt(mean x^2 + eps) * norm_w and its Q8 copy xq (layout of ie_b200_quant_q8) for the GEMVs that
 * follow: the all-reduce, the residual add and the RMSNorm of src/model.c's layer loop in one launch. n is a
 * multiple of 32, at most min(max_floats, 16384). d_xn / d_xq may be NULL. Values travel as 64-bit
 * {epoch, word} stores that the receiver polls in place, so there is no flag round and no fence. */
int ie_b200_ar_allreduce_norm(ie_b200_allreduce *a, const float *d_part, float *d_x, const float *d_norm_w, float eps, float *d_xn, void *d_xq,
                              uint32_t n, uint32_t *d_err, void *stream);
/* The same stop together with the K-split GEMV that produces the partial (the decode step's default): part = W xq
 * (kind / layout / xq as ie_b200_gemv_stream; no bias), and every finished row is stored to the other ranks at
 * once, so the transfer overlaps the rest of the GEMV; the one-CTA kernel launched behind it then only waits for
 * the peers' rows, adds the partials in rank order onto d_x and writes RMSNorm(d_x) and its Q8 copy. rows = n of
 * the exchange (a multiple of 32, at most max_floats). */
int ie_b200_gemv_allreduce_norm(ie_b200_allreduce *a, int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_xq, float *d_part,
                                float *d_x, const float *d_norm_w, float eps, float *d_xn, void *d_xq_out, uint32_t *d_err, void *stream);
/* The two halves of ie_b200_gemv_allreduce_norm as calls of their own, for a host that drives several ranks from one
 * thread (it must launch every rank's GEMV before any rank's reduction, or the first reduction waits for rows nobody has
 * sent yet) and for tests that run the ranks of a world one after the other on one GPU: ie_b200_gemv_push is the K-split
 * GEMV that writes its partial to d_part and stores every finished row into the other ranks' slots; ie_b200_ar_reduce_norm
 * waits for the peers' rows of that exchange (already pushed), adds the partials in rank order onto d_x and normalises. */
int ie_b200_gemv_push(ie_b200_allreduce *a, int kind, const void *d_w, uint32_t rows, uint32_t cols, const void *d_xq, float *d_part, void *stream);
int ie_b200_ar_reduce_norm(ie_b200_allreduce *a, const float *d_part, float *d_x, const float *d_norm_w, float eps, float *d_xn, void *d_xq, uint32_t n,
                           uint32_t *d_err, void *stream);
/* The output head split by vocabulary rows: d_result = {local argmax index, its probability within the local
 * slice (f32 bits)} as ie_b200_argmax leaves them, d_logits the local logits. On return d_result = {global
 * index of the largest logit over all ranks (ties: the smaller index), its probability over the whole
 * vocabulary}, the same on every rank. */
int ie_b200_ar_argmax(ie_b200_allreduce *a, const float *d_logits, uint32_t *d_result, uint32_t vocab_offset, uint32_t *d_err, void *stream);
void ie_b200_ar_destroy(ie_b200_allreduce *a);

/* ---- one host thread, several GPUs ----
 * The form a single-process host program needs (the reference's ie-run is one; src/cuda.c uses this under IE_TP=N): the
 * group owns the all-reduce states of `world` distinct GPUs of this process (devices: world device ordinals, NULL for
 * 0 .. world-1; peer access is enabled both ways and the states are connected in place, no IPC). The caller makes the
 * rank's device current with _use, builds that rank's shard engine (ie_b200_engine.h) and attaches it; step / run /
 * decode then have backend.step / run semantics (src/backend.h:10, :20) for the whole sharded model: every rank's work is
 * enqueued before any rank is waited for, h_logits receives the ranks' vocabulary slices side by side, and the ranks'
 * tokens are checked to be identical. max_floats: the largest exchange (dim floats, times the chunk length T if prompt
 * chunks should take one exchange per stop). _destroy detaches the engines; they stay the caller's to destroy. */
struct ie_b200_engine;
typedef struct ie_b200_tp_group ie_b200_tp_group;
int ie_b200_tp_group_create(uint32_t world, const int *devices, uint32_t max_floats, ie_b200_tp_group **out);
int ie_b200_tp_group_use(ie_b200_tp_group *g, uint32_t rank);
int ie_b200_tp_group_attach(ie_b200_tp_group *g, uint32_t rank, struct ie_b200_engine *e, uint32_t vocab_offset, uint32_t vocab_local);
int ie_b200_tp_group_step(ie_b200_tp_group *g, uint32_t tok, uint32_t pos, float *h_logits, uint32_t *next, double *ms);
int ie_b200_tp_group_run(ie_b200_tp_group *g, const uint32_t *toks, uint32_t T, uint32_t pos, int last_only, uint32_t *out, float *prob);
int ie_b200_tp_group_decode(ie_b200_tp_group *g, uint32_t tok, uint32_t pos, uint32_t K, uint32_t *h_out, double *ms);
void ie_b200_tp_group_destroy(ie_b200_tp_group *g);

#ifdef __cplusplus
}
#endif
#endif
