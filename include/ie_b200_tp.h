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
/* This rank's 128-byte IPC handle blob (receive buffer, flags). */
int ie_b200_ar_handles(ie_b200_allreduce *a, void *h_out128);
/* h_all: the world blobs in rank order (world * 128 bytes). Not needed when world == 1. */
int ie_b200_ar_connect(ie_b200_allreduce *a, const void *h_all);
/* out = (res ? res : 0) + sum over ranks of part, n floats (a multiple of 4). Every rank must make the same
 * sequence of calls. d_err (may be NULL): set to 3 if a peer did not arrive within the time limit. out may
 * alias res. */
int ie_b200_ar_allreduce_add(ie_b200_allreduce *a, const float *d_part, const float *d_res, float *d_out, uint32_t n, uint32_t *d_err,
                             void *stream);
void ie_b200_ar_destroy(ie_b200_allreduce *a);

#ifdef __cplusplus
}
#endif
#endif
