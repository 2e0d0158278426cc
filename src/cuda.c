/* cuda.c -- the GPU backend of amd-infer for NVIDIA B200 (sm_100a), a drop-in
 * for the reference's src/hip.c: it exports the same two constructors
 * (gpu_open, gpu_stream_init: src/backend.h:55-58) and fills the same
 * `struct backend` vtable (src/backend.h:7-49), so model.c, plan.c, gen.c,
 * main.c and serve.c are compiled unchanged and `ie-run --backend gpu` works.
 *
 * All device work is behind the C ABI of libie_b200.so (include/ie_b200.h,
 * include/ie_b200_engine.h): this file only translates the reference's model
 * (matrices in its repacked word/scale arrays) and graph (op list, arena
 * offsets: src/model.h:177-331) into engine calls. Errors follow the
 * reference's convention: a message and exit(1) through ie_die.
 *
 * Built for llama / qwen2 graphs: EMBED, RMSNORM, QUANT, GEMV (Q4_0, Q4_K,
 * Q6_K, f32; bias, residual, fused norm tail), ROPE_KV, ATTN, SWIGLU, ARGMAX.
 * Other architectures' ops (qwen35, flint, MTP, DFlash) are refused by name.
 *
 * Compile inside the reference tree's include path, e.g.
 *   gcc -std=c11 -O2 -I$REF/src -Iinclude $REF/src/{common,gguf,model,plan,cpu,gen,main}.c src/cuda.c -lie_b200
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "backend.h"
#include "common.h"
#include "model.h"

#include "ie_b200_engine.h"

typedef struct {
  backend base;
  const model *m;
  const graph *g;
  ie_b200_engine *e;
  uint32_t *out_tmp;
  void *snap_row[2]; /* prompt-cache snapshots: row 0 of the hbuf buffer (llama / qwen2 keep nothing else outside the KV cache) */
  int snap_buf[2];
} cuda_backend;

#define CHECK(call)                                                          \
  do {                                                                       \
    int rc_ = (call);                                                        \
    if (rc_ < 0) ie_die("cuda backend: %s (status %d)", ie_b200_last_error(), rc_); \
  } while (0)

/* The reference streams each matrix to the device during the load through
 * ie_mat_sink (src/hip.c:304-309). This backend uploads in gpu_open from the
 * loader's host arrays instead (the reference's IE_STREAM=0 mode), so there
 * is nothing to start here; the hook stays unset. */
void gpu_stream_init(void) {}

/* ---- handle tables: one device copy per distinct host array ---- */
typedef struct {
  const void *key;
  int handle;
} slot;
typedef struct {
  slot *s;
  int n, cap;
} table;

static int table_find(const table *t, const void *key) {
  for (int i = 0; i < t->n; i++)
    if (t->s[i].key == key) return t->s[i].handle;
  return -1;
}
static void table_put(table *t, const void *key, int handle) {
  if (t->n == t->cap) {
    t->cap = t->cap ? 2 * t->cap : 64;
    t->s = realloc(t->s, (size_t)t->cap * sizeof(slot));
    if (!t->s) ie_die("out of memory");
  }
  t->s[t->n].key = key, t->s[t->n].handle = handle, t->n++;
}

static int mat_handle(cuda_backend *B, table *t, const mat *w) {
  const void *key = w->kind == MAT_F32 ? (const void *)w->f : (const void *)w->qw; /* a tied output shares the embedding's arrays */
  if (!key) ie_die("cuda backend: matrix without host arrays (unset IE_STREAM or set IE_STREAM=0)");
  int h = table_find(t, key);
  if (h >= 0) return h;
  if (w->n_exp > 1) ie_die("cuda backend: expert matrices are not built");
  switch (w->kind) {
    case MAT_Q4: h = ie_b200_engine_add_mat_ref(B->e, IE_B200_MAT_Q4, w->rows, w->cols, w->qw, w->qs); break;
    case MAT_Q4K: h = ie_b200_engine_add_mat_ref(B->e, IE_B200_MAT_Q4K, w->rows, w->cols, w->qw, w->qs); break;
    case MAT_Q6K: h = ie_b200_engine_add_mat_ref(B->e, IE_B200_MAT_Q6K, w->rows, w->cols, w->qw, w->qs); break;
    case MAT_F32: h = ie_b200_engine_add_mat_ref(B->e, IE_B200_MAT_F32, w->rows, w->cols, w->f, NULL); break;
    default: ie_die("cuda backend: matrix kind %d (Q8_0, Q5_K, IQ4_XS) is not built", w->kind);
  }
  CHECK(h);
  table_put(t, key, h);
  return h;
}

static int vec_handle(cuda_backend *B, table *t, const vec *v) {
  if (!v || !v->n) return -1;
  int h = table_find(t, v->f);
  if (h >= 0) return h;
  h = ie_b200_engine_add_vec(B->e, v->f, v->n);
  CHECK(h);
  table_put(t, v->f, h);
  return h;
}

static uint64_t off_of(const graph *g, int id, uint32_t extra) { return id < 0 ? IE_B200_NONE : (uint64_t)g->bufs[id].off + extra; }
static uint32_t stride_of(const graph *g, int id) { return id < 0 ? 0u : g->bufs[id].stride; }

/* ---- the vtable ---- */

static uint32_t cuda_step(backend *bk, uint32_t tok, uint32_t pos, float *logits, double *ms) {
  cuda_backend *B = (cuda_backend *)bk;
  if (tok >= B->m->vocab) ie_die("token %u >= vocab %u", tok, B->m->vocab);
  if (pos >= B->g->n_ctx) ie_die("position %u >= context %u", pos, B->g->n_ctx);
  uint32_t next = 0;
  CHECK(ie_b200_engine_step(B->e, tok, pos, logits, &next, ms));
  return next;
}

static void cuda_run(backend *bk, int sec, const uint32_t *toks, uint32_t T, uint32_t pos, int last_only, uint32_t *out, float *prob) {
  cuda_backend *B = (cuda_backend *)bk;
  if (sec != 0) ie_die("cuda backend: run section %d (MTP / DFlash) is not built", sec);
  if (T == 0 || T > B->g->T) ie_die("run of %u tokens (1 .. %u)", T, B->g->T);
  if ((uint64_t)pos + T > B->g->n_ctx) ie_die("positions %u .. %u exceed the context %u", pos, pos + T - 1, B->g->n_ctx);
  /* a prompt chunk computes the output head for its last token only, unless all logits are wanted (perplexity) */
  CHECK(ie_b200_engine_run(B->e, toks, T, pos, last_only && !bk->all_logits, out ? out : B->out_tmp, prob));
}

static void cuda_accept(backend *bk, uint32_t k) { (void)bk, (void)k; /* no recurrent state in llama / qwen2 */ }

static void cuda_read_rows(backend *bk, int id, uint32_t r0, uint32_t n, float *dst) {
  cuda_backend *B = (cuda_backend *)bk;
  if (id < 0 || (uint32_t)id >= B->g->n_bufs) ie_die("read_rows: buffer %d", id);
  const buf *b = &B->g->bufs[id];
  CHECK(ie_b200_engine_read_rows(B->e, b->off, b->stride, r0, n, dst));
}

static void cuda_copy_rows(backend *bk, int dst, uint32_t d0, int src, uint32_t r0, uint32_t n) {
  cuda_backend *B = (cuda_backend *)bk;
  const graph *g = B->g;
  if (dst < 0 || (uint32_t)dst >= g->n_bufs || (src >= 0 && (uint32_t)src >= g->n_bufs)) ie_die("copy_rows: buffer %d <- %d", dst, src);
  const buf *d = &g->bufs[dst], *s = src >= 0 ? &g->bufs[src] : d;
  const uint32_t bytes = d->stride < s->stride ? d->stride : s->stride;
  CHECK(ie_b200_engine_copy_rows(B->e, d->off, d->stride, d0, s->off, s->stride, r0, n, bytes, src < 0));
}

/* backend.topk (src/backend.h:33-37): 1 if done on the GPU, 0 if K is too large (gen.c then selects on the host). */
static int cuda_topk(backend *bk, int id, uint32_t r0, uint32_t n, uint32_t nv, uint32_t K, float *val, uint32_t *idx) {
  cuda_backend *B = (cuda_backend *)bk;
  if (id < 0 || (uint32_t)id >= B->g->n_bufs) ie_die("topk: buffer %d", id);
  const buf *b = &B->g->bufs[id];
  const int r = ie_b200_engine_topk(B->e, b->off, b->stride, r0, n, nv, K, val, idx);
  CHECK(r);
  return r;
}

/* backend.snap (src/backend.h:42-48). llama / qwen2 have no linear-attention state and no conv ring: what is not kept per
 * position is nothing, so a snapshot is row 0 of buffer hbuf (if any), held on the host; the KV caches are not copied. */
static void cuda_snap(backend *bk, int save, int k, int hbuf) {
  cuda_backend *B = (cuda_backend *)bk;
  if (k < 0 || k > 1) ie_die("snap: snapshot %d", k);
  if (save) {
    B->snap_buf[k] = hbuf;
    if (hbuf < 0) return;
    if ((uint32_t)hbuf >= B->g->n_bufs) ie_die("snap: buffer %d", hbuf);
    const buf *b = &B->g->bufs[hbuf];
    B->snap_row[k] = realloc(B->snap_row[k], b->stride ? b->stride : 4);
    if (!B->snap_row[k]) ie_die("out of memory");
    CHECK(ie_b200_engine_read_rows(B->e, b->off, b->stride, 0, 1, B->snap_row[k]));
  } else {
    const int id = B->snap_buf[k];
    if (id < 0 || !B->snap_row[k]) return;
    const buf *b = &B->g->bufs[id];
    CHECK(ie_b200_engine_write_rows(B->e, b->off, b->stride, 0, 1, B->snap_row[k]));
  }
}

static void cuda_close(backend *bk) {
  cuda_backend *B = (cuda_backend *)bk;
  ie_b200_engine_destroy(B->e);
  free(B->out_tmp), free(B->snap_row[0]), free(B->snap_row[1]);
  free(B);
}

/* One reference op -> one engine op (a GEMV with the fused norm tail -> two). */
static void translate(cuda_backend *B, table *mats, table *vecs, const op *o, ie_b200_op *out, uint32_t *n_out) {
  const graph *g = B->g;
  const model *m = B->m;
  ie_b200_op e;
  memset(&e, 0, sizeof e);
  e.mat = e.vec = e.layer = -1;
  e.a = off_of(g, o->a, o->aoff), e.b = off_of(g, o->b, o->boff), e.c = off_of(g, o->c, o->coff);
  e.a_stride = stride_of(g, o->a), e.b_stride = stride_of(g, o->b), e.c_stride = stride_of(g, o->c);
  e.qo = off_of(g, o->qo, 0), e.qo_stride = stride_of(g, o->qo);
  e.res = off_of(g, o->res, 0), e.res_stride = stride_of(g, o->res);
  e.n = o->n, e.nh = o->nh;
  switch (o->kind) {
    case OP_EMBED: e.kind = IE_B200_OP_EMBED, e.mat = mat_handle(B, mats, &m->tok); break;
    case OP_RMSNORM: e.kind = IE_B200_OP_RMSNORM, e.vec = vec_handle(B, vecs, o->v); break;
    case OP_QUANT: e.kind = IE_B200_OP_QUANT; break;
    case OP_GEMV_Q4:
    case OP_GEMV_Q4K:
    case OP_GEMV_Q6K:
    case OP_GEMV_F32:
      e.kind = IE_B200_OP_GEMV, e.mat = mat_handle(B, mats, o->w), e.vec = vec_handle(B, vecs, o->v);
      break;
    case OP_ROPE_KV:
    case OP_ATTN:
      if (o->layer < 0 || m->l[o->layer].rec) ie_die("cuda backend: attention op outside an attention layer");
      if (o->kind == OP_ATTN && (o->win || o->sk || o->gt >= 0)) ie_die("cuda backend: sliding window, sinks and gated attention are not built");
      e.kind = o->kind == OP_ROPE_KV ? IE_B200_OP_ROPE_KV : IE_B200_OP_ATTN;
      e.layer = (int32_t)m->l[o->layer].kvi;
      if (o->kind == OP_ATTN) e.c = IE_B200_NONE; /* the scores buffer is the CPU's; the engine has its own partials */
      break;
    case OP_SWIGLU: e.kind = IE_B200_OP_SWIGLU, e.nh = 0; break; /* planar [gate; up], as graph_build lays it out (src/model.c:882-887) */
    case OP_ARGMAX: e.kind = IE_B200_OP_ARGMAX; break;
    case OP_ADD: e.kind = IE_B200_OP_ADD; break;
    default: ie_die("cuda backend: op kind %d is not built (llama / qwen2 graphs only)", o->kind);
  }
  out[(*n_out)++] = e;
  if (o->nv) { /* the fused RMSNorm of a GEMV result (IE_NORM_FUSE=1, src/model.c:1265-1293) as an op of its own */
    ie_b200_op t;
    memset(&t, 0, sizeof t);
    t.kind = IE_B200_OP_RMSNORM, t.mat = -1, t.layer = -1, t.vec = vec_handle(B, vecs, o->nv), t.n = o->w->rows;
    t.a = e.b, t.a_stride = e.b_stride;
    t.b = off_of(g, o->nout, 0), t.b_stride = stride_of(g, o->nout);
    t.qo = off_of(g, o->nq, 0), t.qo_stride = stride_of(g, o->nq);
    t.c = t.res = IE_B200_NONE;
    out[(*n_out)++] = t;
  }
}

backend *gpu_open(const model *m, const graph *g, const char *hsaco) {
  (void)hsaco; /* the kernels are linked in; the AMD code-object path has no meaning here */
  if (ie_b200_device_count() < 1) ie_die("cuda backend: no CUDA device (libie_b200 has no CPU fallback)");
  if (m->arch != ARCH_LLAMA && m->arch != ARCH_QWEN2) ie_die("cuda backend: only llama and qwen2 graphs are built");
  if (m->n_rot != m->hd) ie_die("cuda backend: partial RoPE is not built");
  for (uint32_t i = 0; i < m->n_kvl; i++)
    if (g->kv_len[i] != g->n_ctx) ie_die("cuda backend: ring (sliding window) KV caches are not built");
  cuda_backend *B = calloc(1, sizeof *B);
  if (!B) ie_die("out of memory");
  B->m = m, B->g = g;
  const char *kv = getenv("IE_KV_F32");
  ie_b200_engine_desc d;
  memset(&d, 0, sizeof d);
  d.n_head = m->n_head, d.n_kv = m->n_kv, d.hd = m->hd, d.n_ctx = g->n_ctx, d.n_kv_layers = m->n_kvl, d.T_max = g->T, d.vocab = m->vocab;
  d.eps = m->eps, d.neox = m->rope == ROPE_NEOX, d.kv_f32 = kv && kv[0] == '1';
  d.arena_bytes = g->arena;
  d.logits_off = g->bufs[g->logits].off, d.logits_stride = g->bufs[g->logits].stride;
  d.argmax_off = g->bufs[g->argmax].off, d.argmax_stride = g->bufs[g->argmax].stride;
  CHECK(ie_b200_engine_create(&d, &B->e));
  CHECK(ie_b200_engine_set_rope(B->e, g->rope_cos, g->rope_sin));
  table mats = {0}, vecs = {0};
  ie_b200_op *ops = calloc((size_t)g->n_main * 2 + 1, sizeof *ops);
  uint32_t n = 0, i_head = 0;
  for (uint32_t i = 0; i < g->n_main; i++) {
    if (i == g->i_head) i_head = n;
    translate(B, &mats, &vecs, &g->ops[i], ops, &n);
  }
  CHECK(ie_b200_engine_set_ops(B->e, ops, n, i_head));
  free(ops), free(mats.s), free(vecs.s);
  B->out_tmp = calloc(g->T ? g->T : 1, sizeof(uint32_t));
  B->base.step = cuda_step, B->base.close = cuda_close, B->base.run = cuda_run, B->base.accept = cuda_accept;
  B->base.read_rows = cuda_read_rows, B->base.copy_rows = cuda_copy_rows;
  B->base.topk = cuda_topk, B->base.snap = cuda_snap;
  B->snap_buf[0] = B->snap_buf[1] = -1;
  B->base.verify_max = 0;
  fprintf(stderr, "cuda: %u ops, %u matrices, arena %.2f MB, KV %s, weights %.2f MB/token, %u launches/step\n", n, (unsigned)mats.n,
          g->arena / 1e6, d.kv_f32 ? "f32" : "f16", ie_b200_engine_weight_bytes_per_token(B->e) / 1e6, ie_b200_engine_launches_per_step(B->e));
  return &B->base;
}
