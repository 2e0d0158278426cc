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
 * Built for llama / qwen2 graphs: EMBED, RMSNORM, QUANT, GEMV (Q4_0, Q8_0, Q4_K,
 * Q6_K, f32; bias, residual, fused norm tail), ROPE_KV, ATTN, SWIGLU, ARGMAX.
 * Other architectures' ops (qwen35, flint, MTP, DFlash) are refused by name.
 *
 * IE_TP=N (2, 4 or 8; default 1) shards the model over N GPUs of this process: q / k / v, gate / up and the output
 * head by rows (heads, FFN slice, vocabulary slice), attn_output and ffn_down by columns with one exchange over NVLink
 * peer memory behind each (include/ie_b200_tp.h: ie_b200_tp_group). The reference drives one device (src/hip.c:574) and
 * has no counterpart; its graph, arena offsets and host program are used unchanged -- a shard's vectors simply fill the
 * front of the buffers the reference planned for the whole model.
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
#include "ie_b200_tp.h"

#define MAX_TP 8

typedef struct {
  backend base;
  const model *m;
  const graph *g;
  uint32_t tp;                 /* GPUs the model is sharded over (IE_TP; 1: one GPU, no collective) */
  ie_b200_engine *e[MAX_TP];   /* e[r]: rank r's shard (e[0]: the whole model when tp == 1) */
  ie_b200_tp_group *grp;       /* tp > 1 */
  uint32_t qd_l, kvd_l, ffn_l, vocab_l; /* a shard's q rows, k / v rows, FFN rows and vocabulary rows */
  uint64_t part_off;           /* tp > 1: the partial result of a column-split GEMV (T rows of dim floats), behind the reference's arena */
  uint32_t *out_tmp;
  void *snap_row[2]; /* prompt-cache snapshots: row 0 of the hbuf buffer of every shard (llama / qwen2 keep nothing else outside the KV cache) */
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

/* ---- handle tables: one device copy per distinct host array (and part of it) ---- */
typedef struct {
  const void *key;
  int role, handle;
} slot;
typedef struct {
  slot *s;
  int n, cap;
} table;

static int table_find(const table *t, const void *key, int role) {
  for (int i = 0; i < t->n; i++)
    if (t->s[i].key == key && t->s[i].role == role) return t->s[i].handle;
  return -1;
}
static void table_put(table *t, const void *key, int role, int handle) {
  if (t->n == t->cap) {
    t->cap = t->cap ? 2 * t->cap : 64;
    t->s = realloc(t->s, (size_t)t->cap * sizeof(slot));
    if (!t->s) ie_die("out of memory");
  }
  t->s[t->n].key = key, t->s[t->n].role = role, t->s[t->n].handle = handle, t->n++;
}

/* What a shard holds of a matrix (tp > 1). */
enum { WHOLE, P_QKV, P_Q, P_K, P_V, P_WO, P_GU, P_GATE, P_UP, P_DOWN, P_HEAD };

static int role_of(const model *m, const mat *w) {
  if (w == &m->out) return P_HEAD;
  for (uint32_t i = 0; i < m->n_layer; i++) {
    const layer *L = &m->l[i];
    if (w == &L->wqkv) return P_QKV;
    if (w == &L->wq) return P_Q;
    if (w == &L->wk) return P_K;
    if (w == &L->wv) return P_V;
    if (w == &L->wo) return P_WO;
    if (w == &L->wgu) return P_GU;
    if (w == &L->wgate) return P_GATE;
    if (w == &L->wup) return P_UP;
    if (w == &L->wdown) return P_DOWN;
  }
  return WHOLE;
}

/* The rows (up to three ranges, one after the other) and columns of `w` that rank `rank` holds in `role`. */
typedef struct {
  uint32_t n, row0[3], rows[3], col0, cols;
} part;

static part part_of(const cuda_backend *B, const mat *w, int role, uint32_t rank) {
  const model *m = B->m;
  const uint32_t qd = m->n_head * m->hd, kvd = m->n_kv * m->hd;
  part p;
  memset(&p, 0, sizeof p);
  p.n = 1, p.row0[0] = 0, p.rows[0] = w->rows, p.col0 = 0, p.cols = w->cols;
  switch (role) {
    case P_QKV:
      p.n = 3;
      p.row0[0] = rank * B->qd_l, p.rows[0] = B->qd_l;
      p.row0[1] = qd + rank * B->kvd_l, p.rows[1] = B->kvd_l;
      p.row0[2] = qd + kvd + rank * B->kvd_l, p.rows[2] = B->kvd_l;
      break;
    case P_Q: p.row0[0] = rank * B->qd_l, p.rows[0] = B->qd_l; break;
    case P_K:
    case P_V: p.row0[0] = rank * B->kvd_l, p.rows[0] = B->kvd_l; break;
    case P_WO: p.col0 = rank * B->qd_l, p.cols = B->qd_l; break;
    case P_GU:
      p.n = 2;
      p.row0[0] = rank * B->ffn_l, p.rows[0] = B->ffn_l;
      p.row0[1] = m->ffn + rank * B->ffn_l, p.rows[1] = B->ffn_l;
      break;
    case P_GATE:
    case P_UP: p.row0[0] = rank * B->ffn_l, p.rows[0] = B->ffn_l; break;
    case P_DOWN: p.col0 = rank * B->ffn_l, p.cols = B->ffn_l; break;
    case P_HEAD: p.row0[0] = rank * B->vocab_l, p.rows[0] = B->vocab_l; break;
    default: break;
  }
  return p;
}

static int mat_kind(const mat *w) {
  switch (w->kind) {
    case MAT_Q4: return IE_B200_MAT_Q4;
    case MAT_Q8: return IE_B200_MAT_Q8;
    case MAT_Q4K: return IE_B200_MAT_Q4K;
    case MAT_Q6K: return IE_B200_MAT_Q6K;
    case MAT_F32: return IE_B200_MAT_F32;
    default: ie_die("cuda backend: matrix kind %d (Q5_K, IQ4_XS) is not built", w->kind);
  }
  return -1;
}

static int mat_handle(cuda_backend *B, uint32_t rank, table *t, const mat *w, int role) {
  const void *key = w->kind == MAT_F32 ? (const void *)w->f : (const void *)w->qw; /* a tied output shares the embedding's arrays */
  if (!key) ie_die("cuda backend: matrix without host arrays (unset IE_STREAM or set IE_STREAM=0)");
  int h = table_find(t, key, role);
  if (h >= 0) return h;
  if (w->n_exp > 1) ie_die("cuda backend: expert matrices are not built");
  const int kind = mat_kind(w);
  const void *qs = w->kind == MAT_F32 ? NULL : (const void *)w->qs;
  if (role == WHOLE) {
    h = ie_b200_engine_add_mat_ref(B->e[rank], kind, w->rows, w->cols, key, qs);
  } else {
    const part p = part_of(B, w, role, rank);
    h = ie_b200_engine_add_mat_ref_part(B->e[rank], kind, w->rows, w->cols, key, qs, p.n, p.row0, p.rows, p.col0, p.cols);
  }
  CHECK(h);
  table_put(t, key, role, h);
  return h;
}

/* A norm weight or bias; role != WHOLE: the rows of the bias that go with the matrix part of that role. */
static int vec_handle(cuda_backend *B, uint32_t rank, table *t, const vec *v, const mat *w, int role) {
  if (!v || !v->n) return -1;
  int h = table_find(t, v->f, role);
  if (h >= 0) return h;
  if (role == WHOLE) {
    h = ie_b200_engine_add_vec(B->e[rank], v->f, v->n);
  } else {
    const part p = part_of(B, w, role, rank);
    uint32_t n = 0;
    for (uint32_t k = 0; k < p.n; k++) n += p.rows[k];
    float *tmp = malloc((size_t)n * sizeof(float));
    if (!tmp) ie_die("out of memory");
    n = 0;
    for (uint32_t k = 0; k < p.n; k++) {
      if ((uint64_t)p.row0[k] + p.rows[k] > v->n) ie_die("cuda backend: a bias of %u values for rows up to %u", v->n, p.row0[k] + p.rows[k]);
      memcpy(tmp + n, v->f + p.row0[k], (size_t)p.rows[k] * sizeof(float));
      n += p.rows[k];
    }
    h = ie_b200_engine_add_vec(B->e[rank], tmp, n);
    free(tmp);
  }
  CHECK(h);
  table_put(t, v->f, role, h);
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
  if (B->tp > 1) CHECK(ie_b200_tp_group_step(B->grp, tok, pos, logits, &next, ms));
  else CHECK(ie_b200_engine_step(B->e[0], tok, pos, logits, &next, ms));
  return next;
}

static void cuda_run(backend *bk, int sec, const uint32_t *toks, uint32_t T, uint32_t pos, int last_only, uint32_t *out, float *prob) {
  cuda_backend *B = (cuda_backend *)bk;
  if (sec != 0) ie_die("cuda backend: run section %d (MTP / DFlash) is not built", sec);
  if (T == 0 || T > B->g->T) ie_die("run of %u tokens (1 .. %u)", T, B->g->T);
  if ((uint64_t)pos + T > B->g->n_ctx) ie_die("positions %u .. %u exceed the context %u", pos, pos + T - 1, B->g->n_ctx);
  /* a prompt chunk computes the output head for its last token only, unless all logits are wanted (perplexity) */
  const int last = last_only && !bk->all_logits;
  if (B->tp > 1) CHECK(ie_b200_tp_group_run(B->grp, toks, T, pos, last, out ? out : B->out_tmp, prob));
  else CHECK(ie_b200_engine_run(B->e[0], toks, T, pos, last, out ? out : B->out_tmp, prob));
}

static void cuda_accept(backend *bk, uint32_t k) { (void)bk, (void)k; /* no recurrent state in llama / qwen2 */ }

/* Sharded: the logits rows are gathered from the ranks' vocabulary slices; every other buffer is read from rank 0
 * (the residual stream and its norms are the same on every rank; q / k / v, attention and FFN buffers hold rank 0's
 * slice in front). */
static void cuda_read_rows(backend *bk, int id, uint32_t r0, uint32_t n, float *dst) {
  cuda_backend *B = (cuda_backend *)bk;
  if (id < 0 || (uint32_t)id >= B->g->n_bufs) ie_die("read_rows: buffer %d", id);
  const buf *b = &B->g->bufs[id];
  if (B->tp > 1 && id == B->g->logits) {
    char *row = malloc(b->stride ? b->stride : 4);
    if (!row) ie_die("out of memory");
    for (uint32_t t = 0; t < n; t++)
      for (uint32_t r = 0; r < B->tp; r++) {
        CHECK(ie_b200_engine_read_rows(B->e[r], b->off, b->stride, r0 + t, 1, row));
        memcpy((char *)dst + (size_t)t * b->stride + (size_t)r * B->vocab_l * 4u, row, (size_t)B->vocab_l * 4u);
      }
    free(row);
    return;
  }
  CHECK(ie_b200_engine_read_rows(B->e[0], b->off, b->stride, r0, n, dst));
}

static void cuda_copy_rows(backend *bk, int dst, uint32_t d0, int src, uint32_t r0, uint32_t n) {
  cuda_backend *B = (cuda_backend *)bk;
  const graph *g = B->g;
  if (dst < 0 || (uint32_t)dst >= g->n_bufs || (src >= 0 && (uint32_t)src >= g->n_bufs)) ie_die("copy_rows: buffer %d <- %d", dst, src);
  const buf *d = &g->bufs[dst], *s = src >= 0 ? &g->bufs[src] : d;
  const uint32_t bytes = d->stride < s->stride ? d->stride : s->stride;
  for (uint32_t r = 0; r < B->tp; r++)
    CHECK(ie_b200_engine_copy_rows(B->e[r], d->off, d->stride, d0, s->off, s->stride, r0, n, bytes, src < 0));
}

/* backend.topk (src/backend.h:33-37): 1 if done on the GPU, 0 if K is too large (gen.c then selects on the host).
 * Sharded: every rank selects the K best of its vocabulary slice, the host keeps the K best of those N x K (larger
 * value first, then the smaller index: the order of one selection over the whole row). */
static int cuda_topk(backend *bk, int id, uint32_t r0, uint32_t n, uint32_t nv, uint32_t K, float *val, uint32_t *idx) {
  cuda_backend *B = (cuda_backend *)bk;
  if (id < 0 || (uint32_t)id >= B->g->n_bufs) ie_die("topk: buffer %d", id);
  const buf *b = &B->g->bufs[id];
  if (B->tp == 1) {
    const int r = ie_b200_engine_topk(B->e[0], b->off, b->stride, r0, n, nv, K, val, idx);
    CHECK(r);
    return r;
  }
  if (id != B->g->logits || nv != B->m->vocab || K > B->vocab_l || n == 0) return 0;
  const size_t per = (size_t)n * K;
  float *cv = malloc(per * B->tp * sizeof(float));
  uint32_t *ci = malloc(per * B->tp * sizeof(uint32_t));
  if (!cv || !ci) ie_die("out of memory");
  int done = 1;
  for (uint32_t r = 0; r < B->tp && done; r++) {
    done = ie_b200_engine_topk(B->e[r], b->off, b->stride, r0, n, B->vocab_l, K, cv + per * r, ci + per * r);
    CHECK(done);
  }
  for (uint32_t t = 0; t < n && done; t++) {
    uint32_t at[MAX_TP] = {0}; /* every rank's list is sorted: merge their heads */
    for (uint32_t k = 0; k < K; k++) {
      int best = -1;
      float bv = 0;
      uint32_t bi = 0;
      for (uint32_t r = 0; r < B->tp; r++) {
        if (at[r] >= K) continue;
        const float v = cv[per * r + (size_t)t * K + at[r]];
        const uint32_t i = ci[per * r + (size_t)t * K + at[r]] + r * B->vocab_l;
        if (best < 0 || v > bv || (v == bv && i < bi)) best = (int)r, bv = v, bi = i;
      }
      val[(size_t)t * K + k] = bv, idx[(size_t)t * K + k] = bi;
      at[best]++;
    }
  }
  free(cv), free(ci);
  return done;
}

/* backend.snap (src/backend.h:42-48). llama / qwen2 have no linear-attention state and no conv ring: what is not kept per
 * position is nothing, so a snapshot is row 0 of buffer hbuf (if any) of every shard, held on the host; the KV caches are
 * not copied. */
static void cuda_snap(backend *bk, int save, int k, int hbuf) {
  cuda_backend *B = (cuda_backend *)bk;
  if (k < 0 || k > 1) ie_die("snap: snapshot %d", k);
  if (save) {
    B->snap_buf[k] = hbuf;
    if (hbuf < 0) return;
    if ((uint32_t)hbuf >= B->g->n_bufs) ie_die("snap: buffer %d", hbuf);
    const buf *b = &B->g->bufs[hbuf];
    const size_t row = b->stride ? b->stride : 4;
    B->snap_row[k] = realloc(B->snap_row[k], row * B->tp);
    if (!B->snap_row[k]) ie_die("out of memory");
    for (uint32_t r = 0; r < B->tp; r++) CHECK(ie_b200_engine_read_rows(B->e[r], b->off, b->stride, 0, 1, (char *)B->snap_row[k] + row * r));
  } else {
    const int id = B->snap_buf[k];
    if (id < 0 || !B->snap_row[k]) return;
    const buf *b = &B->g->bufs[id];
    const size_t row = b->stride ? b->stride : 4;
    for (uint32_t r = 0; r < B->tp; r++) CHECK(ie_b200_engine_write_rows(B->e[r], b->off, b->stride, 0, 1, (char *)B->snap_row[k] + row * r));
  }
}

static void cuda_close(backend *bk) {
  cuda_backend *B = (cuda_backend *)bk;
  if (B->grp) ie_b200_tp_group_destroy(B->grp); /* detaches the engines */
  for (uint32_t r = 0; r < B->tp; r++) ie_b200_engine_destroy(B->e[r]);
  free(B->out_tmp), free(B->snap_row[0]), free(B->snap_row[1]);
  free(B);
}

/* Buffers whose shard is shorter than the reference planned: remembered while the op list is walked. */
typedef struct {
  int att_buf; /* the attention output of the current layer (qd_l floats on a shard) */
  int swi_buf; /* the SwiGLU output (ffn_l floats on a shard) */
} track;

/* One reference op -> engine ops of rank `rank` (a GEMV with the fused norm tail -> two; a column-split GEMV of a
 * shard -> the GEMV of the partial, the exchange that adds the ranks' partials to the residual, then the tail). */
static void translate(cuda_backend *B, uint32_t rank, table *mats, table *vecs, const op *o, ie_b200_op *out, uint32_t *n_out, track *tk) {
  const graph *g = B->g;
  const model *m = B->m;
  const int tp = B->tp > 1;
  ie_b200_op e;
  memset(&e, 0, sizeof e);
  e.mat = e.vec = e.layer = -1;
  e.a = off_of(g, o->a, o->aoff), e.b = off_of(g, o->b, o->boff), e.c = off_of(g, o->c, o->coff);
  e.a_stride = stride_of(g, o->a), e.b_stride = stride_of(g, o->b), e.c_stride = stride_of(g, o->c);
  e.qo = off_of(g, o->qo, 0), e.qo_stride = stride_of(g, o->qo);
  e.res = off_of(g, o->res, 0), e.res_stride = stride_of(g, o->res);
  e.n = o->n, e.nh = o->nh;
  int split_cols = 0;
  switch (o->kind) {
    case OP_EMBED: e.kind = IE_B200_OP_EMBED, e.mat = mat_handle(B, rank, mats, &m->tok, WHOLE); break;
    case OP_RMSNORM: e.kind = IE_B200_OP_RMSNORM, e.vec = vec_handle(B, rank, vecs, o->v, NULL, WHOLE); break;
    case OP_QUANT:
      e.kind = IE_B200_OP_QUANT;
      if (tp && o->a == tk->att_buf) e.n = B->qd_l;
      if (tp && o->a == tk->swi_buf) e.n = B->ffn_l;
      break;
    case OP_GEMV_Q4:
    case OP_GEMV_Q8:
    case OP_GEMV_Q4K:
    case OP_GEMV_Q6K:
    case OP_GEMV_F32: {
      const int role = tp ? role_of(m, o->w) : WHOLE;
      e.kind = IE_B200_OP_GEMV, e.mat = mat_handle(B, rank, mats, o->w, role);
      switch (role) {
        case WHOLE: e.vec = vec_handle(B, rank, vecs, o->v, NULL, WHOLE); break;
        case P_WO:
        case P_DOWN:
          if (o->v && o->v->n) ie_die("cuda backend: IE_TP with a bias on a column-split matrix is not built");
          split_cols = 1;
          e.n = role == P_WO ? B->qd_l : B->ffn_l;
          e.b = B->part_off, e.b_stride = o->w->rows * 4u; /* the partial; the exchange below adds the residual */
          e.res = IE_B200_NONE, e.res_stride = 0;
          break;
        default: /* split by rows: the bias rows go with them, the result lands in front of the shared buffer */
          if (o->res >= 0) ie_die("cuda backend: IE_TP with a residual on a row-split matrix is not built");
          e.vec = vec_handle(B, rank, vecs, o->v, o->w, role);
          if (role == P_K) e.b = off_of(g, o->b, B->qd_l * 4u);
          if (role == P_V) e.b = off_of(g, o->b, (B->qd_l + B->kvd_l) * 4u);
          if (role == P_UP) e.b = off_of(g, o->b, B->ffn_l * 4u);
          break;
      }
      break;
    }
    case OP_ROPE_KV:
    case OP_ATTN:
      if (o->layer < 0 || m->l[o->layer].rec) ie_die("cuda backend: attention op outside an attention layer");
      if (o->kind == OP_ATTN && (o->win || o->sk || o->gt >= 0)) ie_die("cuda backend: sliding window, sinks and gated attention are not built");
      e.kind = o->kind == OP_ROPE_KV ? IE_B200_OP_ROPE_KV : IE_B200_OP_ATTN;
      e.layer = (int32_t)m->l[o->layer].kvi;
      if (o->kind == OP_ATTN) e.c = IE_B200_NONE; /* the scores buffer is the CPU's; the engine has its own partials */
      if (tp) {
        e.n = B->qd_l;
        if (o->kind == OP_ROPE_KV) {
          e.nh = m->n_head / B->tp;
          e.b = off_of(g, o->b, B->qd_l * 4u), e.c = off_of(g, o->c, (B->qd_l + B->kvd_l) * 4u);
        } else {
          tk->att_buf = o->b;
        }
      }
      break;
    case OP_SWIGLU:
      e.kind = IE_B200_OP_SWIGLU, e.nh = 0; /* planar [gate; up], as graph_build lays it out (src/model.c:882-887) */
      if (tp) e.n = B->ffn_l, e.b = off_of(g, o->b, B->ffn_l * 4u), tk->swi_buf = o->a;
      break;
    case OP_ARGMAX:
      e.kind = IE_B200_OP_ARGMAX;
      if (tp) e.n = B->vocab_l;
      break;
    case OP_ADD:
      if (tp) ie_die("cuda backend: IE_TP with an ADD op is not built");
      e.kind = IE_B200_OP_ADD;
      break;
    default: ie_die("cuda backend: op kind %d is not built (llama / qwen2 graphs only)", o->kind);
  }
  out[(*n_out)++] = e;
  if (split_cols) { /* result = residual + the sum over the ranks of the partials */
    ie_b200_op x;
    memset(&x, 0, sizeof x);
    x.kind = IE_B200_OP_ALLREDUCE, x.mat = x.vec = x.layer = -1, x.n = o->w->rows;
    x.a = e.b, x.a_stride = e.b_stride;
    x.b = x.qo = IE_B200_NONE;
    x.c = off_of(g, o->b, o->boff), x.c_stride = stride_of(g, o->b);
    x.res = off_of(g, o->res, 0), x.res_stride = stride_of(g, o->res);
    out[(*n_out)++] = x;
  }
  if (o->nv) { /* the fused RMSNorm of a GEMV result (IE_NORM_FUSE=1, src/model.c:1265-1293) as an op of its own */
    ie_b200_op t;
    memset(&t, 0, sizeof t);
    t.kind = IE_B200_OP_RMSNORM, t.mat = -1, t.layer = -1, t.vec = vec_handle(B, rank, vecs, o->nv, NULL, WHOLE), t.n = o->w->rows;
    t.a = off_of(g, o->b, o->boff), t.a_stride = stride_of(g, o->b);
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
  B->m = m, B->g = g, B->tp = 1;
  const char *tpv = getenv("IE_TP");
  if (tpv && tpv[0]) {
    const long n = strtol(tpv, NULL, 10);
    if (n != 1 && n != 2 && n != 4 && n != 8) ie_die("cuda backend: IE_TP=%s (1, 2, 4 or 8 GPUs)", tpv);
    if ((int)n > ie_b200_device_count()) ie_die("cuda backend: IE_TP=%ld with %d CUDA devices", n, ie_b200_device_count());
    B->tp = (uint32_t)n;
  }
  const uint32_t N = B->tp;
  if (m->n_head % N || m->n_kv % N || m->ffn % (32u * N) || m->vocab % N)
    ie_die("cuda backend: IE_TP=%u does not divide %u heads / %u KV heads, FFN %u (in whole blocks of 32) or vocabulary %u", N, m->n_head, m->n_kv,
           m->ffn, m->vocab);
  B->qd_l = m->n_head / N * m->hd, B->kvd_l = m->n_kv / N * m->hd, B->ffn_l = m->ffn / N, B->vocab_l = m->vocab / N;
  const char *kv = getenv("IE_KV_F32");
  ie_b200_engine_desc d;
  memset(&d, 0, sizeof d);
  d.n_head = m->n_head / N, d.n_kv = m->n_kv / N, d.hd = m->hd, d.n_ctx = g->n_ctx, d.n_kv_layers = m->n_kvl, d.T_max = g->T, d.vocab = m->vocab;
  d.eps = m->eps, d.neox = m->rope == ROPE_NEOX, d.kv_f32 = kv && kv[0] == '1';
  d.arena_bytes = g->arena;
  if (N > 1) { /* the partial sums of the column-split GEMVs live behind the reference's arena */
    B->part_off = ((uint64_t)g->arena + 255u) & ~(uint64_t)255u;
    d.arena_bytes = B->part_off + (uint64_t)(g->T ? g->T : 1) * m->dim * 4u;
    CHECK(ie_b200_tp_group_create(N, NULL, m->dim * (g->T ? g->T : 1), &B->grp));
  }
  d.logits_off = g->bufs[g->logits].off, d.logits_stride = g->bufs[g->logits].stride;
  d.argmax_off = g->bufs[g->argmax].off, d.argmax_stride = g->bufs[g->argmax].stride;
  uint32_t n = 0, n_mats = 0;
  for (uint32_t r = 0; r < N; r++) {
    if (B->grp) CHECK(ie_b200_tp_group_use(B->grp, r)); /* the engine is created on the current device */
    CHECK(ie_b200_engine_create(&d, &B->e[r]));
    CHECK(ie_b200_engine_set_rope(B->e[r], g->rope_cos, g->rope_sin));
    table mats = {0}, vecs = {0};
    track tk = {-1, -1};
    ie_b200_op *ops = calloc((size_t)g->n_main * 3 + 1, sizeof *ops);
    if (!ops) ie_die("out of memory");
    uint32_t i_head = 0;
    n = 0;
    for (uint32_t i = 0; i < g->n_main; i++) {
      if (i == g->i_head) i_head = n;
      translate(B, r, &mats, &vecs, &g->ops[i], ops, &n, &tk);
    }
    CHECK(ie_b200_engine_set_ops(B->e[r], ops, n, i_head));
    if (B->grp) CHECK(ie_b200_tp_group_attach(B->grp, r, B->e[r], r * B->vocab_l, B->vocab_l));
    n_mats = (uint32_t)mats.n;
    free(ops), free(mats.s), free(vecs.s);
  }
  if (B->grp) CHECK(ie_b200_tp_group_use(B->grp, 0));
  B->out_tmp = calloc(g->T ? g->T : 1, sizeof(uint32_t));
  B->base.step = cuda_step, B->base.close = cuda_close, B->base.run = cuda_run, B->base.accept = cuda_accept;
  B->base.read_rows = cuda_read_rows, B->base.copy_rows = cuda_copy_rows;
  B->base.topk = cuda_topk, B->base.snap = cuda_snap;
  B->snap_buf[0] = B->snap_buf[1] = -1;
  B->base.verify_max = 0;
  fprintf(stderr, "cuda: %u GPU%s, %u ops, %u matrices, arena %.2f MB, KV %s, weights %.2f MB/token per GPU, %u launches/step\n", N, N > 1 ? "s" : "", n,
          n_mats, d.arena_bytes / 1e6, d.kv_f32 ? "f32" : "f16", ie_b200_engine_weight_bytes_per_token(B->e[0]) / 1e6,
          ie_b200_engine_launches_per_step(B->e[0]));
  return &B->base;
}
