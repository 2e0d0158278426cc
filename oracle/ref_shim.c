/* ref_shim.c -- TEST INFRASTRUCTURE. Thin ctypes-friendly wrappers around
 * the reference's own CPU implementation (src/cpu.c, src/model.c, src/plan.c,
 * src/gguf.c, src/common.c), compiled where those sources lie into
 * oracle/_ref/libie_ref.so by oracle/build.py. Nothing here computes: every
 * entry point forwards to a reference function, so that the restatement in
 * ie_oracle.c and the CUDA kernels can be compared with the reference itself.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "backend.h"
#include "common.h"
#include "gguf.h"
#include "model.h"

/* cpu_quant_q8 (src/cpu.c:36). */
void ref_quant_q8(const float *x, uint8_t *q, uint32_t nb) { cpu_quant_q8(x, q, nb); }

/* A matrix from GGUF bytes as model_load makes it (src/model.c:481
 * model_mat_from_gguf). Returns a handle; ref_mat_kind etc. read it. */
void *ref_mat_new(uint32_t ttype, const uint8_t *src, uint32_t rows, uint32_t cols) {
  mat *w = calloc(1, sizeof *w);
  model_mat_from_gguf(w, ttype, src, rows, cols);
  return w;
}
int ref_mat_kind(const void *h) { return ((const mat *)h)->kind; }
uint32_t ref_mat_nb(const void *h) { return ((const mat *)h)->nb; }
const uint32_t *ref_mat_qw(const void *h) { return ((const mat *)h)->qw; }
const uint16_t *ref_mat_qs(const void *h) { return ((const mat *)h)->qs; }
const float *ref_mat_f(const void *h) { return ((const mat *)h)->f; }
uint64_t ref_mat_qw_words(const void *h) {
  const mat *w = h;
  return mat_qw_words(w->kind, w->rows, w->cols);
}
uint64_t ref_mat_qs_n(const void *h) {
  const mat *w = h;
  return mat_qs_n(w->kind, w->rows, w->cols);
}
void ref_mat_free(void *h) {
  mat *w = h;
  free(w->qw), free(w->qs), free(w->f), free(w);
}

/* y = W xq by the reference's CPU GEMV of the matrix's kind (src/cpu.c:64,
 * :93, :123). Quantised kinds only. Returns 0, or -1 for another kind. */
int ref_gemv(const void *h, const uint8_t *xq, float *y) {
  const mat *w = h;
  switch (w->kind) {
    case MAT_Q4: cpu_gemv_q4(w, xq, y); return 0;
    case MAT_Q4K: cpu_gemv_q4k(w, xq, y); return 0;
    case MAT_Q6K: cpu_gemv_q6k(w, xq, y); return 0;
    case MAT_Q8: cpu_gemv_q8(w, xq, y); return 0;
    default: return -1;
  }
}

/* A loaded model with the CPU backend (src/main.c:100-140 without the CLI). */
typedef struct {
  gguf_file g;
  model m;
  graph gr;
  backend *b;
} ref_engine;

void *ref_open(const char *path, uint32_t n_ctx) {
  ref_engine *e = calloc(1, sizeof *e);
  gguf_open(&e->g, path);
  model_load(&e->m, &e->g);
  graph_build(&e->gr, &e->m, n_ctx, 1, 0);
  plan_arena(&e->gr, 0);
  e->b = cpu_open(&e->m, &e->gr);
  return e;
}

uint32_t ref_vocab(const void *h) { return ((const ref_engine *)h)->m.vocab; }
uint32_t ref_dim(const void *h) { return ((const ref_engine *)h)->m.dim; }
uint32_t ref_n_layer(const void *h) { return ((const ref_engine *)h)->m.n_layer; }
uint64_t ref_weight_bytes_per_token(const void *h) { return ((const ref_engine *)h)->gr.weight_bytes_per_token; }

/* backend.step of the CPU backend (src/cpu.c:483). */
uint32_t ref_step(void *h, uint32_t tok, uint32_t pos, float *logits, double *ms) {
  ref_engine *e = h;
  return e->b->step(e->b, tok, pos, logits, ms);
}

/* The residual stream x after each layer for (tok, pos): the step is run
 * with the op list cut after each layer's last op (the KV writes of a
 * position are the same in every run), and the result buffer of that op is
 * read from the arena. out: [n_layer][dim]. The cache must already hold
 * positions 0 .. pos-1. */
void ref_layer_outputs(void *h, uint32_t tok, uint32_t pos, float *out) {
  ref_engine *e = h;
  graph *g = &e->gr;
  const uint32_t full = g->n_ops;
  /* the CPU backend keeps its arena first in its private struct after the
   * vtable; read results through a step's logits instead: not possible for
   * inner buffers, so find the arena by running with a marker op list. */
  for (uint32_t l = 0; l < e->m.n_layer; l++) {
    uint32_t last = 0;
    for (uint32_t i = 0; i < full; i++)
      if (g->ops[i].layer == (int)l && g->ops[i].res >= 0) last = i; /* the down GEMV: the layer's last residual add */
    /* run ops 0 .. last, then an argmax-free tail: keep logits/argmax valid ids */
    g->n_ops = last + 1;
    /* cpu_step reads the argmax buffer at the end: harmless */
    e->b->step(e->b, tok, pos, NULL, NULL);
    g->n_ops = full;
    /* cpu_backend layout (src/cpu.c:19-24): {backend base; const model *m; const graph *g; uint8_t *arena; ...} */
    struct peek {
      backend base;
      const model *m;
      const graph *g;
      uint8_t *arena;
    };
    const uint8_t *arena = ((struct peek *)e->b)->arena;
    memcpy(out + (size_t)l * e->m.dim, arena + g->bufs[g->ops[last].b].off + g->ops[last].boff, (size_t)e->m.dim * 4);
  }
}

void ref_close(void *h) {
  ref_engine *e = h;
  e->b->close(e->b);
  graph_free(&e->gr);
  model_free(&e->m);
  gguf_close(&e->g);
  free(e);
}
