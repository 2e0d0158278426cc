// The shards of one tensor-parallel model driven from ONE host thread: a group owns the peer-memory all-reduce states
// of `world` GPUs of this process (peer access enabled both ways, states connected in place: no IPC), the caller builds
// one engine per rank on the rank's device and attaches it, and step / run / decode enqueue every rank's work before
// they wait for any rank. That is the form a single-process host program needs (the reference's ie-run is one: its
// backend vtable has one step call per token, src/backend.h:7-49); a host with one process per GPU uses the states
// directly (ie_b200_tp.h) and needs no group.
//
// Every rank's kernels wait for the other ranks' rows with bounded waits, and the ranks' launches leave this thread a
// few hundred microseconds apart: far inside the bound. No two kernels that wait for one another ever share a GPU.
#include <vector>

#include "common.cuh"
#include "ie_b200_engine.h"
#include "ie_b200_tp.h"

using namespace ieb;

struct ie_b200_tp_group {
  uint32_t world = 0;
  int dev[8] = {};
  ie_b200_allreduce *ar[8] = {};
  ie_b200_engine *eng[8] = {};
  uint32_t vocab_l[8] = {};   // logits per rank (the head is split by vocabulary rows)
  std::vector<uint32_t> tmp;  // a rank's tokens, to compare with rank 0's
  bool ready = false;
};

extern "C" int ie_b200_tp_group_create(uint32_t world, const int *devices, uint32_t max_floats, ie_b200_tp_group **out) {
  if (!out || world < 1 || world > 8) return fail(IE_B200_E_ARG, "ie_b200_tp_group_create: %u ranks (1 .. 8)", world);
  int n_dev = 0;
  IEB_CUDA(cudaGetDeviceCount(&n_dev));
  ie_b200_tp_group *g = new ie_b200_tp_group();
  g->world = world;
  for (uint32_t r = 0; r < world; r++) {
    g->dev[r] = devices ? devices[r] : (int)r;
    if (g->dev[r] < 0 || g->dev[r] >= n_dev) {
      delete g;
      return fail(IE_B200_E_ARG, "ie_b200_tp_group_create: device %d of %d", devices ? devices[r] : (int)r, n_dev);
    }
    for (uint32_t q = 0; q < r; q++)
      if (g->dev[q] == g->dev[r]) {
        const int twice = g->dev[r];
        delete g;
        return fail(IE_B200_E_ARG, "ie_b200_tp_group_create: device %d twice (kernels that wait for one another must not share a GPU)", twice);
      }
  }
  int rc = IE_B200_OK;
  for (uint32_t r = 0; r < world && rc == IE_B200_OK; r++) {
    cudaError_t e = cudaSetDevice(g->dev[r]);
    for (uint32_t q = 0; q < world && e == cudaSuccess; q++) {
      if (q == r) continue;
      int can = 0;
      e = cudaDeviceCanAccessPeer(&can, g->dev[r], g->dev[q]);
      if (e == cudaSuccess && !can) rc = fail(IE_B200_E_STATE, "ie_b200_tp_group_create: device %d cannot address device %d", g->dev[r], g->dev[q]);
      if (e != cudaSuccess || rc) break;
      e = cudaDeviceEnablePeerAccess(g->dev[q], 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) e = cudaSuccess, (void)cudaGetLastError();
    }
    if (e != cudaSuccess && rc == IE_B200_OK) rc = cuda_fail(e, "ie_b200_tp_group_create (peer access)");
    if (rc == IE_B200_OK) rc = ie_b200_ar_create(r, world, max_floats, &g->ar[r]);
  }
  for (uint32_t r = 0; r < world && rc == IE_B200_OK; r++) {
    cudaSetDevice(g->dev[r]);
    rc = ie_b200_ar_connect_local(g->ar[r], g->ar);
  }
  cudaSetDevice(g->dev[0]);
  if (rc != IE_B200_OK) {
    for (uint32_t r = 0; r < world; r++)
      if (g->ar[r]) cudaSetDevice(g->dev[r]), ie_b200_ar_destroy(g->ar[r]);
    delete g;
    return rc;
  }
  *out = g;
  return IE_B200_OK;
}

extern "C" int ie_b200_tp_group_use(ie_b200_tp_group *g, uint32_t rank) {
  if (!g || rank >= g->world) return fail(IE_B200_E_ARG, "ie_b200_tp_group_use: rank %u", rank);
  IEB_CUDA(cudaSetDevice(g->dev[rank]));
  return IE_B200_OK;
}

extern "C" int ie_b200_tp_group_attach(ie_b200_tp_group *g, uint32_t rank, ie_b200_engine *e, uint32_t vocab_offset, uint32_t vocab_local) {
  if (!g || !e || rank >= g->world) return fail(IE_B200_E_ARG, "ie_b200_tp_group_attach: rank %u", rank);
  IEB_CUDA(cudaSetDevice(g->dev[rank]));
  if (int r = ie_b200_engine_set_collective(e, g->ar[rank], vocab_offset)) return r;
  g->eng[rank] = e, g->vocab_l[rank] = vocab_local, g->ready = false;
  return IE_B200_OK;
}

static int complete(ie_b200_tp_group *g, const char *who) {
  if (!g) return fail(IE_B200_E_ARG, "%s: NULL group", who);
  if (g->ready) return IE_B200_OK;
  for (uint32_t r = 0; r < g->world; r++)
    if (!g->eng[r]) return fail(IE_B200_E_STATE, "%s: rank %u has no engine attached", who, r);
  // every rank's step graph (or persistent kernel's program) is made now: a first step that captured rank 1's graph while
  // rank 0's kernels already wait for rank 1 would spend part of their time limit on it
  for (uint32_t r = 0; r < g->world; r++)
    if (ie_b200_engine_launches_per_step(g->eng[r]) == 0) return fail(IE_B200_E_STATE, "%s: rank %u has no step to run (no op list, or its graph could not be made)", who, r);
  g->ready = true;
  return IE_B200_OK;
}

extern "C" int ie_b200_tp_group_step(ie_b200_tp_group *g, uint32_t tok, uint32_t pos, float *h_logits, uint32_t *next, double *ms) {
  if (int r = complete(g, "ie_b200_tp_group_step")) return r;
  if (!next) return fail(IE_B200_E_ARG, "ie_b200_tp_group_step: NULL argument");
  int rc = IE_B200_OK;
  uint32_t off = 0, begun = 0;
  for (uint32_t r = 0; r < g->world && rc == IE_B200_OK; r++) {
    rc = ie_b200_engine_step_begin(g->eng[r], tok, pos, r == 0 && ms);
    if (rc == IE_B200_OK) begun++;
  }
  uint32_t first = 0;
  for (uint32_t r = 0; r < begun; r++) {  // every rank that was begun is waited for, also after an error; rank r's slice of
    uint32_t t = 0;                       // the logits lands at its vocabulary offset
    const int e = ie_b200_engine_step_end(g->eng[r], h_logits ? h_logits + off : nullptr, &t, r == 0 ? ms : nullptr);
    off += g->vocab_l[r];
    if (e != IE_B200_OK && rc == IE_B200_OK) rc = e;
    if (r == 0) first = t;
    else if (rc == IE_B200_OK && t != first) rc = fail(IE_B200_E_DEVICE, "ie_b200_tp_group_step: rank %u chose token %u, rank 0 token %u", r, t, first);
  }
  cudaSetDevice(g->dev[0]);
  if (rc == IE_B200_OK) *next = first;
  return rc;
}

extern "C" int ie_b200_tp_group_run(ie_b200_tp_group *g, const uint32_t *toks, uint32_t T, uint32_t pos, int last_only, uint32_t *out, float *prob) {
  if (int r = complete(g, "ie_b200_tp_group_run")) return r;
  if (!toks || !out) return fail(IE_B200_E_ARG, "ie_b200_tp_group_run: NULL argument");
  int rc = IE_B200_OK;
  uint32_t begun = 0;
  for (uint32_t r = 0; r < g->world && rc == IE_B200_OK; r++) {
    rc = ie_b200_engine_run_begin(g->eng[r], toks, T, pos, last_only);
    if (rc == IE_B200_OK) begun++;
  }
  g->tmp.resize(T ? T : 1);
  for (uint32_t r = 0; r < begun; r++) {
    const int e = ie_b200_engine_run_end(g->eng[r], r == 0 ? out : g->tmp.data(), r == 0 ? prob : nullptr);
    if (e != IE_B200_OK && rc == IE_B200_OK) rc = e;
    // with last_only the rows before the last hold no result; the last token's must agree
    if (r && rc == IE_B200_OK && g->tmp[T - 1] != out[T - 1])
      rc = fail(IE_B200_E_DEVICE, "ie_b200_tp_group_run: rank %u chose token %u, rank 0 token %u", r, g->tmp[T - 1], out[T - 1]);
  }
  cudaSetDevice(g->dev[0]);
  return rc;
}

extern "C" int ie_b200_tp_group_decode(ie_b200_tp_group *g, uint32_t tok, uint32_t pos, uint32_t K, uint32_t *h_out, double *ms) {
  if (int r = complete(g, "ie_b200_tp_group_decode")) return r;
  if (!h_out) return fail(IE_B200_E_ARG, "ie_b200_tp_group_decode: NULL argument");
  if (K == 0) return IE_B200_OK;
  int rc = IE_B200_OK;
  uint32_t begun = 0;
  g->tmp.resize((size_t)K * g->world);
  for (uint32_t r = 0; r < g->world && rc == IE_B200_OK; r++) {
    rc = ie_b200_engine_decode_begin(g->eng[r], tok, pos, K);
    if (rc == IE_B200_OK) begun++;
  }
  for (uint32_t r = 0; r < begun; r++) {
    const int e = ie_b200_engine_decode_end(g->eng[r], r == 0 ? h_out : g->tmp.data() + (size_t)K * r, r == 0 ? ms : nullptr);
    if (e != IE_B200_OK && rc == IE_B200_OK) rc = e;
  }
  for (uint32_t r = 1; r < begun && rc == IE_B200_OK; r++)
    for (uint32_t k = 0; k < K; k++)
      if (g->tmp[(size_t)K * r + k] != h_out[k]) {
        rc = fail(IE_B200_E_DEVICE, "ie_b200_tp_group_decode: rank %u chose token %u at step %u, rank 0 token %u", r, g->tmp[(size_t)K * r + k], k, h_out[k]);
        break;
      }
  cudaSetDevice(g->dev[0]);
  return rc;
}

extern "C" void ie_b200_tp_group_destroy(ie_b200_tp_group *g) {
  if (!g) return;
  for (uint32_t r = 0; r < g->world; r++) {
    cudaSetDevice(g->dev[r]);
    cudaDeviceSynchronize();
    if (g->eng[r]) ie_b200_engine_set_collective(g->eng[r], nullptr, 0);
    if (g->ar[r]) ie_b200_ar_destroy(g->ar[r]);
  }
  cudaSetDevice(g->dev[0]);
  delete g;
}
