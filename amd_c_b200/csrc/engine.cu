// engine.cu -- the decode engine: owns weights, arena, KV cache and scratch of
// one GPU; runs a static op list with the kernels of this library. A
// one-token step is one CUDA-graph launch bracketed by an 8-byte upload
// (token, position) and an 8-byte download (argmax, probability).
#include <climits>
#include <cstdlib>
#include <cstring>
#include <cstdio>
#include <vector>

#include "common.cuh"
#include "ie_b200_engine.h"
#include "ie_b200_tp.h"
#include "peer_ll.cuh"
#include "step_kernel.cuh"

namespace ieb {

struct EMat {
  int kind;
  uint32_t rows, cols;
  void *d;
  bool owned;
  int tc_exp = INT32_MIN;  // power-of-two scale of the weights for the tcgen05 GEMM (worked out at first use)
};
struct EVec {
  float *d;
  uint32_t n;
};

__global__ void add_kernel(const float *a, const float *b, float *c, uint32_t n, size_t as, size_t bs, size_t cs) {
  const uint32_t t = blockIdx.y;
  const float *at = reinterpret_cast<const float *>(reinterpret_cast<const char *>(a) + as * t);
  const float *bt = reinterpret_cast<const float *>(reinterpret_cast<const char *>(b) + bs * t);
  float *ct = reinterpret_cast<float *>(reinterpret_cast<char *>(c) + cs * t);
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) ct[i] = __fadd_rn(at[i], bt[i]);
}

// After a one-token step: feed the argmax back as the next token, advance the positions, and log the
// token in a history ring (hist[cap] counts the steps since the last reset).
__global__ void advance_kernel(uint32_t *scalars, uint32_t Tm, const uint32_t *argmax, uint32_t *hist, uint32_t cap) {
  const uint32_t idx = argmax[0];
  if (threadIdx.x == 0) {
    const uint32_t c = hist[cap];
    hist[c % cap] = idx;
    hist[cap] = c + 1u;
    scalars[0] = idx;
    scalars[Tm] += 1u;
  }
  for (uint32_t t = threadIdx.x; t < Tm; t += blockDim.x) scalars[Tm + 1u + t] += 1u;
}

}  // namespace ieb

using namespace ieb;

constexpr uint32_t HIST_CAP = 4096;

struct ie_b200_engine {
  ie_b200_engine_desc d;
  int device = 0;
  cudaStream_t stream = nullptr;
  uint8_t *arena = nullptr;
  void *kc = nullptr, *vc = nullptr;  // [layer][kv head][n_ctx][hd]
  size_t kv_layer_bytes = 0;
  float *rope_cos = nullptr, *rope_sin = nullptr;
  uint32_t *scalars = nullptr;  // tokens[T_max], then the first position
  uint32_t *h_scalars = nullptr, *h_result = nullptr;  // pinned
  void *attn_part = nullptr;
  uint32_t *attn_count = nullptr;
  void *argmax_part = nullptr;
  uint32_t *hist = nullptr;  // HIST_CAP tokens + the step counter
  uint32_t *err = nullptr;   // device error word: set by a kernel whose bounded wait ran out; err[2..3]: the GEMVs' work and arrival counters
  bool no_attn_fuse = false; // IE_B200_ATTN_FUSE=0: RoPE + KV store as a kernel of its own
  bool no_prefill_attn = false;  // IE_B200_PREFILL_ATTN=0: a chunk's attention through the decode kernel, one CTA set per token
  bool no_gemm = false;      // IE_B200_GEMM=0: prompt chunks through the multi-token GEMV (bit-exact with the one-token path)
  bool gemm_mma = false;     // IE_B200_GEMM=mma: the int8 mma.sync GEMM instead of the tcgen05 one
  uint32_t ctx_bound = 0;    // positions the captured step graph's attention grid is sized for (0: the whole context)
  bool timed = false;        // the step begun last records its device time
  uint32_t run_T = 0;        // tokens of the chunk (or steps of the decode run) begun last
  int swi_epi = -1;          // IE_B200_SWIGLU=gemv: SwiGLU in the gate / up GEMV's epilogue and the Q8 quantiser in the down GEMV's
                             // prologue (one launch less per layer). Off unless asked for: every CTA of the down GEMV then quantises
                             // the whole vector itself, which costs more than the launch it saves (measured at 1 and 2 GPUs)
  void *topk_scratch = nullptr;  // candidates and results of ie_b200_engine_topk
  size_t topk_bytes = 0;
  void *gemm_scratch = nullptr;  // expanded activations and K-split partials of the tcgen05 GEMM
  size_t gemm_scratch_bytes = 0;
  int norm_mode = 2;         // IE_B200_NORM: 2 (default) a kernel of its own, 0 "tail": in the producing GEMV's last CTA, 1 "prologue": in the consuming GEMVs
  uint32_t T_att = 1;
  ie_b200_allreduce *ar = nullptr;  // tensor parallel: serves the ALLREDUCE ops and the argmax exchange (not owned)
  uint32_t vocab_off = 0;           // first vocabulary row of this shard's output head
  std::vector<EMat> mats;
  std::vector<EVec> vecs;
  std::vector<ie_b200_op> ops;
  uint32_t i_head = 0;
  uint32_t logits_n = 0;  // floats the output head writes per token (a vocabulary-split shard holds fewer than d.vocab)
  cudaGraphExec_t step_graph = nullptr;
  uint32_t step_launches = 0;
  // the persistent step kernel (step_kernel.cu): the op list translated into phases, and its scratch
  int step_mode = 1;          // 1: the step graph (default: measured faster on B200, see ie_b200_engine_set_step_mode); 2: the persistent kernel, or
                              // an error where it cannot run; 0: the kernel where the op list and shapes allow it, else the graph
  int kernel_state = 0;       // 0: not examined yet, 1: program built, -1: this op list / shape has no program
  StepPhase *d_prog = nullptr;
  StepArgs sk = {};
  int sk_kset = 0;            // matrix kinds of the program's GEMVs (0 Q4_0, 1 Q4_K / Q6_K, 2 mixed)
  float *sk_part = nullptr;
  void *sk_amax = nullptr;
  uint32_t *sk_bar = nullptr;  // {arrival counter, abort flag}
  unsigned long long *sk_trace = nullptr;  // per phase kind {work ns, barrier ns, barriers} of CTA 0 (ie_b200_engine_phase_times)
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
};

static inline void *at(ie_b200_engine *e, uint64_t off, uint32_t stride, uint32_t t0) {
  return off == IE_B200_NONE ? nullptr : e->arena + off + (size_t)stride * t0;
}

// Host to device on the engine's stream, then wait: a plain cudaMemcpy from pageable memory may return while its last piece
// is still on the way, and the engine's stream (non-blocking) does not order itself behind the default stream.
static cudaError_t h2d(ie_b200_engine *e, void *dst, const void *src, size_t n) {
  cudaError_t r = cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, e->stream);
  return r == cudaSuccess ? cudaStreamSynchronize(e->stream) : r;
}

namespace ieb {
int gemv_push_act(ie_b200_allreduce *a, int kind, const void *d_w, uint32_t rows, uint32_t cols, const ActSrc &act, bool plain, float *d_part, cudaStream_t st);
int ar_norm_reduce(ie_b200_allreduce *a, const float *d_part, const float *d_res, float *d_x, const float *d_norm_w, float eps, float *d_xn, void *d_xq,
                   uint32_t n, uint32_t *d_err, cudaStream_t st, bool pushed);
void ar_push_info(const ie_b200_allreduce *a, ArPush *out);  // allreduce.cu
bool ar_connected(const ie_b200_allreduce *a);
int attn_decode_fused(const float *d_q, const float *d_k, const float *d_v, void *d_kc, void *d_vc, const float *d_cos, const float *d_sin, float *d_out,
                      void *d_oq, const uint32_t *d_pos, uint32_t n_head, uint32_t n_kv, uint32_t hd, int neox, int kv_f32, uint32_t kv_len, uint32_t n_ctx,
                      void *d_part, uint32_t *d_count, cudaStream_t st, bool early);  // attn_decode.cu
}

// Can the one-token decode GEMV take this matrix?
static bool stream_ok(const EMat &m) { return gemv_direct_ok(m.kind, m.cols); }

// One op for tokens [t0, t0 + T) of a run.
static int launch_op(ie_b200_engine *e, const ie_b200_op &o, uint32_t t0, uint32_t T, cudaStream_t st) {
  const ie_b200_engine_desc &d = e->d;
  void *a = at(e, o.a, o.a_stride, t0), *b = at(e, o.b, o.b_stride, t0), *c = at(e, o.c, o.c_stride, t0);
  void *qo = at(e, o.qo, o.qo_stride, t0), *res = at(e, o.res, o.res_stride, t0);
  const uint32_t *tok = e->scalars + t0, *pos = e->scalars + d.T_max;
  switch (o.kind) {
    case IE_B200_OP_EMBED: {
      if (o.mat < 0 || (size_t)o.mat >= e->mats.size()) return fail(IE_B200_E_ARG, "EMBED: bad matrix handle %d", o.mat);
      const EMat &m = e->mats[o.mat];
      return ie_b200_embed(m.kind, m.d, m.cols, tok, static_cast<float *>(a), T, o.a_stride, st);
    }
    case IE_B200_OP_RMSNORM: {
      if (o.vec < 0 || (size_t)o.vec >= e->vecs.size()) return fail(IE_B200_E_ARG, "RMSNORM: bad vector handle %d", o.vec);
      if (res) {  // a = a + res first (the reduced partial of a sharded GEMV)
        add_kernel<<<dim3((o.n + 255u) / 256u, T), 256, 0, st>>>(static_cast<float *>(a), static_cast<float *>(res), static_cast<float *>(a), o.n,
                                                                o.a_stride, o.res_stride, o.a_stride);
        IEB_LAUNCHED("add_kernel");
      }
      return ie_b200_rmsnorm(static_cast<float *>(a), e->vecs[o.vec].d, static_cast<float *>(b), o.n, d.eps, qo, T, o.a_stride, o.b_stride,
                             o.qo_stride, st);
    }
    case IE_B200_OP_QUANT: return ie_b200_quant_q8(static_cast<float *>(a), b, o.n / 32u, T, o.a_stride, o.b_stride, st);
    case IE_B200_OP_GEMV: {
      if (o.mat < 0 || (size_t)o.mat >= e->mats.size()) return fail(IE_B200_E_ARG, "GEMV: bad matrix handle %d", o.mat);
      const EMat &m = e->mats[o.mat];
      const float *bias = o.vec >= 0 ? e->vecs[o.vec].d : nullptr;
      if (T == 1 && stream_ok(m))
        return ie_b200_gemv_stream(m.kind, m.d, m.rows, m.cols, a, static_cast<float *>(b), bias, static_cast<float *>(res), st);
      // a prompt chunk (the reference's threshold, src/hip.c:965): the tensor-core GEMM reads the weights once per 128 tokens
      const bool tc_ok = !e->gemm_mma && o.a_stride % 16u == 0;
      // (Q8_0 has no mma.sync form: where the tcgen05 kernel cannot run it takes the multi-token GEMV below, 8 tokens per pass)
      if (T >= 17 && m.kind != IE_B200_MAT_F32 && !e->no_gemm && (tc_ok || m.kind != IE_B200_MAT_Q8)) {
        if (tc_ok) {  // tcgen05 / tensor memory
          EMat &mm = e->mats[o.mat];
          // (normally done by prepare_chunks before anything of the run is enqueued; here for callers that enqueue ranges themselves)
          if (mm.tc_exp == INT32_MIN)
            if (int r = ie_b200_mat_tc_exp(mm.kind, mm.d, mm.rows, mm.cols, &mm.tc_exp, st)) return r;
          const size_t need = ie_b200_gemm_tc_scratch_bytes(mm.rows, mm.cols, e->d.T_max);
          if (need > e->gemm_scratch_bytes) {
            IEB_CUDA(cudaStreamSynchronize(st));
            cudaFree(e->gemm_scratch), e->gemm_scratch = nullptr, e->gemm_scratch_bytes = 0;
            IEB_CUDA(cudaMalloc(&e->gemm_scratch, need));
            e->gemm_scratch_bytes = need;
          }
          return ie_b200_gemm_tc(mm.kind, mm.d, mm.rows, mm.cols, mm.tc_exp, a, static_cast<float *>(b), bias, static_cast<float *>(res), T, o.a_stride,
                                 o.b_stride, o.res_stride, e->gemm_scratch, e->gemm_scratch_bytes, e->err, st);
        }
        return ie_b200_gemm(m.kind, m.d, m.rows, m.cols, a, static_cast<float *>(b), bias, static_cast<float *>(res), T, o.a_stride, o.b_stride,
                            o.res_stride, st);
      }
      return ie_b200_gemv(m.kind, m.d, m.rows, m.cols, a, static_cast<float *>(b), bias, static_cast<float *>(res), T, o.a_stride, o.b_stride,
                          o.res_stride, st);
    }
    case IE_B200_OP_ROPE_KV: {
      char *kcl = static_cast<char *>(e->kc) + e->kv_layer_bytes * o.layer, *vcl = static_cast<char *>(e->vc) + e->kv_layer_bytes * o.layer;
      // positions of tokens t0.. : the kernel adds its token index to *pos, so offset the q/k/v rows only
      // and pass a position scalar that already includes t0 (scalars[T_max + 1 + t0] holds pos + t0)
      return ie_b200_rope_kv(static_cast<float *>(a), static_cast<float *>(b), static_cast<float *>(c), kcl, vcl, e->rope_cos, e->rope_sin,
                             pos + 1 + t0, o.nh, d.n_kv, d.hd, d.neox, d.kv_f32, d.n_ctx, T, o.a_stride, st);
    }
    case IE_B200_OP_ATTN: {
      char *kcl = static_cast<char *>(e->kc) + e->kv_layer_bytes * o.layer, *vcl = static_cast<char *>(e->vc) + e->kv_layer_bytes * o.layer;
      // a prompt chunk on a half-precision cache: tokens share passes over the cache on the tensor cores
      if (T > 1 && !d.kv_f32 && (d.hd == 64 || d.hd == 128) && !e->no_prefill_attn)
        return ie_b200_attn_prefill(static_cast<float *>(at(e, o.a, o.a_stride, t0)), kcl, vcl, static_cast<float *>(at(e, o.b, o.b_stride, t0)),
                                    at(e, o.qo, o.qo_stride, t0), pos + 1 + t0, d.n_head, d.n_kv, d.hd, d.n_ctx, T, o.a_stride, o.b_stride,
                                    o.qo_stride, st);
      for (uint32_t s = 0; s < T; s += e->T_att) {  // bounded scratch: at most T_att tokens per launch
        const uint32_t n = T - s < e->T_att ? T - s : e->T_att;
        int r = ie_b200_attn_decode(static_cast<float *>(at(e, o.a, o.a_stride, t0 + s)), kcl, vcl, static_cast<float *>(at(e, o.b, o.b_stride, t0 + s)),
                                    at(e, o.qo, o.qo_stride, t0 + s), pos + 1 + t0 + s, d.n_head, d.n_kv, d.hd, d.kv_f32, d.n_ctx, d.n_ctx, n,
                                    o.a_stride, o.b_stride, o.qo_stride, e->attn_part, e->attn_count, st);
        if (r) return r;
      }
      return IE_B200_OK;
    }
    case IE_B200_OP_SWIGLU:
      if (o.nh == 1u) return ie_b200_swiglu_il(static_cast<float *>(a), static_cast<float *>(b), o.n, qo, T, o.a_stride, o.b_stride, o.qo_stride, st);
      return ie_b200_swiglu(static_cast<float *>(a), static_cast<float *>(b), o.n, qo, T, o.a_stride, o.qo_stride, st);
    case IE_B200_OP_ARGMAX: {
      if (int r = ie_b200_argmax(static_cast<float *>(a), o.n, static_cast<uint32_t *>(b), T, o.a_stride, o.b_stride, e->argmax_part, st)) return r;
      if (!e->ar) return IE_B200_OK;
      for (uint32_t t = 0; t < T; t++)  // sharded head: the ranks' local winners, best one to everybody
        if (int r = ie_b200_ar_argmax(e->ar, static_cast<float *>(at(e, o.a, o.a_stride, t0 + t)), static_cast<uint32_t *>(at(e, o.b, o.b_stride, t0 + t)),
                                      e->vocab_off, e->err, st))
          return r;
      return IE_B200_OK;
    }
    case IE_B200_OP_ALLREDUCE: {  // c = (res, or c itself) + the sum over the ranks of a
      if (!e->ar) return IE_B200_OK;  // no collective attached: the caller serves these stops between enqueue calls
      const bool own_res = o.res != IE_B200_NONE;
      // a prompt chunk whose token rows lie back to back: one exchange over T x n floats (the state's buffers permitting)
      if (T > 1 && o.a_stride == o.n * 4u && o.c_stride == o.n * 4u && (!own_res || o.res_stride == o.n * 4u)) {
        ArPush info;
        ar_push_info(e->ar, &info);
        if ((uint64_t)o.n * T <= info.max_n) {
          float *x = static_cast<float *>(at(e, o.c, o.c_stride, t0));
          const float *rs = own_res ? static_cast<const float *>(at(e, o.res, o.res_stride, t0)) : x;
          return ie_b200_ar_allreduce_add(e->ar, static_cast<float *>(at(e, o.a, o.a_stride, t0)), rs, x, o.n * T, e->err, st);
        }
      }
      for (uint32_t t = 0; t < T; t++) {
        float *x = static_cast<float *>(at(e, o.c, o.c_stride, t0 + t));
        const float *rs = own_res ? static_cast<const float *>(at(e, o.res, o.res_stride, t0 + t)) : x;
        if (int r = ie_b200_ar_allreduce_add(e->ar, static_cast<float *>(at(e, o.a, o.a_stride, t0 + t)), rs, x, o.n, e->err, st)) return r;
      }
      return IE_B200_OK;
    }
    case IE_B200_OP_ADD:
      add_kernel<<<dim3((o.n + 255u) / 256u, T), 256, 0, st>>>(static_cast<float *>(a), static_cast<float *>(b), static_cast<float *>(c), o.n,
                                                              o.a_stride, o.b_stride, o.c_stride);
      IEB_LAUNCHED("add_kernel");
      return IE_B200_OK;
    default: return fail(IE_B200_E_ARG, "unknown op kind %d", o.kind);
  }
}

// Ops [first, last) for T tokens. For one token, an RMSNORM whose Q8 copy feeds the GEMVs right after it is
// folded into those GEMVs' prologues (every CTA recomputes the norm; CTA 0 of the first GEMV still writes the
// norm's f32 and Q8 outputs for any later reader), which takes a kernel out of the dependency chain.
static int enqueue_range(ie_b200_engine *e, uint32_t first, uint32_t last, uint32_t T, uint32_t kind_mask, cudaStream_t st) {
  // RoPE + KV store folded into the attention kernel of the same layer (one token)?
  auto rope_fuses = [&](uint32_t i) {
    if (T != 1 || i + 1 >= last || e->no_attn_fuse) return false;
    const ie_b200_op &o = e->ops[i], &nx = e->ops[i + 1];
    return o.kind == IE_B200_OP_ROPE_KV && nx.kind == IE_B200_OP_ATTN && nx.layer == o.layer && nx.a == o.a &&
           (kind_mask & (1u << IE_B200_OP_ROPE_KV)) && (kind_mask & (1u << IE_B200_OP_ATTN));
  };
  // The fused attention kernel reads the position and older cache rows ahead of its dependency wait when the
  // kernel launched right before it is a decode GEMV told to release its dependents only after its own wait.
  bool prev_late = false;
  const bool swi_epi = T == 1 && e->swi_epi == 1 && (kind_mask & (1u << IE_B200_OP_SWIGLU)) && (kind_mask & (1u << IE_B200_OP_GEMV));
  uint64_t h_q8 = IE_B200_NONE, h_f32 = IE_B200_NONE;  // the Q8 buffer a skipped SWIGLU op would have written, and the f32 vector that stands for it
  for (uint32_t i = first; i < last; i++) {
    const ie_b200_op &o = e->ops[i];
    if (!(kind_mask & (1u << o.kind))) continue;
    const bool was_late = prev_late;
    prev_late = false;
    // gate / up GEMV over interleaved rows: SwiGLU in its epilogue (a warp owns a pair), the op after it is skipped
    if (swi_epi && o.kind == IE_B200_OP_GEMV && i + 2 < last && o.mat >= 0 && stream_ok(e->mats[o.mat]) && o.vec < 0 && o.res == IE_B200_NONE) {
      const ie_b200_op &sw = e->ops[i + 1], &dn = e->ops[i + 2];
      const EMat &m = e->mats[o.mat];
      if (sw.kind == IE_B200_OP_SWIGLU && sw.nh == 1u && sw.a == o.b && sw.qo != IE_B200_NONE && sw.b != IE_B200_NONE && m.rows == 2u * sw.n && sw.n % 32u == 0 &&
          dn.kind == IE_B200_OP_GEMV && dn.a == sw.qo && dn.mat >= 0 && stream_ok(e->mats[dn.mat]) && e->mats[dn.mat].cols == sw.n) {
        ActSrc act = {};
        act.xq = static_cast<const uint8_t *>(at(e, o.a, 0, 0));
        if (int r = gemv_direct(m.kind, m.d, m.rows, m.cols, act, false, static_cast<float *>(at(e, sw.b, 0, 0)), nullptr, nullptr, nullptr, nullptr, st, nullptr,
                                false, true))
          return r;
        h_q8 = sw.qo, h_f32 = sw.b;
        i++;
        continue;
      }
    }
    // the GEMV that reads the skipped op's Q8 buffer: it quantises the f32 vector in its own prologue (CTA 0 also writes the Q8 buffer)
    if (T == 1 && h_q8 != IE_B200_NONE && o.kind == IE_B200_OP_GEMV && o.a == h_q8) {
      const EMat &m = e->mats[o.mat];
      ActSrc act = {};
      act.xf = static_cast<const float *>(at(e, h_f32, 0, 0)), act.xq_out = static_cast<uint8_t *>(at(e, h_q8, 0, 0));
      h_q8 = IE_B200_NONE;
      if (e->ar && i + 2 < last && o.vec < 0 && o.res == IE_B200_NONE && (kind_mask & (1u << IE_B200_OP_ALLREDUCE)) && (kind_mask & (1u << IE_B200_OP_RMSNORM))) {
        const ie_b200_op &ar = e->ops[i + 1], &nx = e->ops[i + 2];
        if (ar.kind == IE_B200_OP_ALLREDUCE && ar.a == o.b && ar.n == m.rows && nx.kind == IE_B200_OP_RMSNORM && nx.a == ar.c && nx.res == IE_B200_NONE &&
            nx.vec >= 0 && nx.n == m.rows && m.rows % 32u == 0) {
          if (int r = gemv_push_act(e->ar, m.kind, m.d, m.rows, m.cols, act, true, static_cast<float *>(at(e, o.b, 0, 0)), st)) return r;
          if (int r = ar_norm_reduce(e->ar, static_cast<float *>(at(e, o.b, 0, 0)), static_cast<const float *>(at(e, ar.res, 0, 0)),
                                     static_cast<float *>(at(e, ar.c, 0, 0)), e->vecs[nx.vec].d, e->d.eps, static_cast<float *>(at(e, nx.b, 0, 0)),
                                     at(e, nx.qo, 0, 0), m.rows, e->err, st, true))
            return r;
          i += 2;
          continue;
        }
      }
      if (int r = gemv_direct(m.kind, m.d, m.rows, m.cols, act, true, static_cast<float *>(at(e, o.b, 0, 0)), o.vec >= 0 ? e->vecs[o.vec].d : nullptr,
                              static_cast<float *>(at(e, o.res, 0, 0)), nullptr, nullptr, st))
        return r;
      continue;
    }
    if (T == 1 && o.kind == IE_B200_OP_GEMV && o.mat >= 0 && (size_t)o.mat < e->mats.size() && stream_ok(e->mats[o.mat]) && rope_fuses(i + 1)) {
      const EMat &m = e->mats[o.mat];
      ActSrc act = {};
      act.xq = static_cast<const uint8_t *>(at(e, o.a, 0, 0));
      if (int r = gemv_direct(m.kind, m.d, m.rows, m.cols, act, false, static_cast<float *>(at(e, o.b, 0, 0)), o.vec >= 0 ? e->vecs[o.vec].d : nullptr,
                              static_cast<float *>(at(e, o.res, 0, 0)), nullptr, nullptr, st, nullptr, true))
        return r;
      prev_late = true;
      continue;
    }
    if (rope_fuses(i)) {
      const ie_b200_op &nx = e->ops[i + 1];
      char *kcl = static_cast<char *>(e->kc) + e->kv_layer_bytes * o.layer, *vcl = static_cast<char *>(e->vc) + e->kv_layer_bytes * o.layer;
      int r = attn_decode_fused(static_cast<float *>(at(e, o.a, 0, 0)), static_cast<float *>(at(e, o.b, 0, 0)), static_cast<float *>(at(e, o.c, 0, 0)), kcl,
                                vcl, e->rope_cos, e->rope_sin, static_cast<float *>(at(e, nx.b, 0, 0)), at(e, nx.qo, 0, 0), e->scalars + e->d.T_max + 1,
                                e->d.n_head, e->d.n_kv, e->d.hd, e->d.neox, e->d.kv_f32, e->d.n_ctx, e->ctx_bound ? e->ctx_bound : e->d.n_ctx, e->attn_part, e->attn_count, st,
                                was_late);
      if (r) return r;
      i++;
      continue;
    }
    // tensor parallel: a K-split GEMV that stores every finished row to the other ranks as well, then the one-CTA kernel
    // that waits for the peers' rows, reduces onto the residual stream and normalises
    if (T == 1 && e->ar && o.kind == IE_B200_OP_GEMV && i + 2 < last && o.mat >= 0 && stream_ok(e->mats[o.mat]) &&
        o.vec < 0 && o.res == IE_B200_NONE && (kind_mask & (1u << IE_B200_OP_ALLREDUCE)) && (kind_mask & (1u << IE_B200_OP_RMSNORM))) {
      const ie_b200_op &ar = e->ops[i + 1], &nx = e->ops[i + 2];
      const EMat &m = e->mats[o.mat];
      if (ar.kind == IE_B200_OP_ALLREDUCE && ar.a == o.b && ar.n == m.rows && nx.kind == IE_B200_OP_RMSNORM && nx.a == ar.c && nx.res == IE_B200_NONE &&
          nx.vec >= 0 && nx.n == m.rows && m.rows % 32u == 0) {
        ActSrc act = {};
        act.xq = static_cast<const uint8_t *>(at(e, o.a, 0, 0));
        if (int r = gemv_push_act(e->ar, m.kind, m.d, m.rows, m.cols, act, false, static_cast<float *>(at(e, o.b, 0, 0)), st)) return r;
        if (int r = ar_norm_reduce(e->ar, static_cast<float *>(at(e, o.b, 0, 0)), static_cast<const float *>(at(e, ar.res, 0, 0)),
                                   static_cast<float *>(at(e, ar.c, 0, 0)), e->vecs[nx.vec].d, e->d.eps, static_cast<float *>(at(e, nx.b, 0, 0)),
                                   at(e, nx.qo, 0, 0), m.rows, e->err, st, true))
          return r;
        i += 2;
        continue;
      }
    }
    // tensor parallel: all-reduce + residual add + the RMSNorm that follows, one kernel
    if (T == 1 && e->ar && o.kind == IE_B200_OP_ALLREDUCE && i + 1 < last && (kind_mask & (1u << IE_B200_OP_RMSNORM))) {
      const ie_b200_op &nx = e->ops[i + 1];
      if (nx.kind == IE_B200_OP_RMSNORM && nx.a == o.c && nx.res == IE_B200_NONE && nx.vec >= 0 && nx.n == o.n && o.n % 32u == 0 && o.n <= 16384u) {
        int r = ar_norm_reduce(e->ar, static_cast<float *>(at(e, o.a, 0, 0)), static_cast<const float *>(at(e, o.res, 0, 0)),
                               static_cast<float *>(at(e, o.c, 0, 0)), e->vecs[nx.vec].d, e->d.eps, static_cast<float *>(at(e, nx.b, 0, 0)),
                               at(e, nx.qo, 0, 0), o.n, e->err, st, false);
        if (r) return r;
        i++;
        continue;
      }
    }
    // norm tail: a one-token GEMV whose result is normalised by the very next op
    if (T == 1 && e->norm_mode == 0 && o.kind == IE_B200_OP_GEMV && i + 1 < last && o.mat >= 0 && stream_ok(e->mats[o.mat]) &&
        (kind_mask & (1u << IE_B200_OP_RMSNORM))) {
      const ie_b200_op &nx = e->ops[i + 1];
      const EMat &m = e->mats[o.mat];
      if (nx.kind == IE_B200_OP_RMSNORM && nx.a == o.b && nx.res == IE_B200_NONE && nx.vec >= 0 && nx.n == m.rows && m.rows % 32u == 0) {
        int r = ie_b200_gemv_norm_tail(m.kind, m.d, m.rows, m.cols, at(e, o.a, 0, 0), static_cast<float *>(at(e, o.b, 0, 0)),
                                       o.vec >= 0 ? e->vecs[o.vec].d : nullptr, static_cast<float *>(at(e, o.res, 0, 0)), e->vecs[nx.vec].d, e->d.eps,
                                       static_cast<float *>(at(e, nx.b, 0, 0)), at(e, nx.qo, 0, 0), e->err + 2, st);
        if (r) return r;
        i++;
        continue;
      }
    }
    if (T == 1 && e->norm_mode == 1 && o.kind == IE_B200_OP_RMSNORM && o.qo != IE_B200_NONE && o.res == IE_B200_NONE && o.vec >= 0 && o.n % 32u == 0) {
      uint32_t j = i + 1;
      while (j < last && e->ops[j].kind == IE_B200_OP_GEMV && e->ops[j].a == o.qo && e->ops[j].mat >= 0 && stream_ok(e->mats[e->ops[j].mat]) &&
             e->mats[e->ops[j].mat].cols == o.n && e->ops[j].b != o.a && (kind_mask & (1u << IE_B200_OP_GEMV)))
        j++;
      if (j > i + 1) {
        for (uint32_t k = i + 1; k < j; k++) {
          const ie_b200_op &g = e->ops[k];
          const EMat &m = e->mats[g.mat];
          const bool firstg = k == i + 1;
          int r = ie_b200_norm_gemv_stream(m.kind, m.d, m.rows, m.cols, static_cast<float *>(at(e, o.a, 0, 0)), e->vecs[o.vec].d, e->d.eps,
                                           firstg ? static_cast<float *>(at(e, o.b, 0, 0)) : nullptr, firstg ? at(e, o.qo, 0, 0) : nullptr,
                                           static_cast<float *>(at(e, g.b, 0, 0)), g.vec >= 0 ? e->vecs[g.vec].d : nullptr,
                                           static_cast<float *>(at(e, g.res, 0, 0)), st);
          if (r) return r;
        }
        i = j - 1;
        continue;
      }
    }
    if (int r = launch_op(e, o, 0, T, st)) return r;
  }
  return IE_B200_OK;
}

// scalars layout: [0, T_max) token ids; [T_max] first position; [T_max + 1 + t] = first position + t.
static int upload_input(ie_b200_engine *e, const uint32_t *toks, uint32_t T, uint32_t pos, cudaStream_t st) {
  const uint32_t Tm = e->d.T_max;
  if (T == 0 || T > Tm) return fail(IE_B200_E_SIZE, "run of %u tokens (1 .. %u)", T, Tm);
  if ((uint64_t)pos + T > e->d.n_ctx) return fail(IE_B200_E_SIZE, "positions %u .. %u exceed the context %u", pos, pos + T - 1, e->d.n_ctx);
  for (uint32_t t = 0; t < T; t++) {
    if (toks[t] >= e->d.vocab) return fail(IE_B200_E_SIZE, "token %u >= vocab %u", toks[t], e->d.vocab);
    e->h_scalars[t] = toks[t];
  }
  e->h_scalars[Tm] = pos;
  for (uint32_t t = 0; t < Tm; t++) e->h_scalars[Tm + 1 + t] = pos + t;
  IEB_CUDA(cudaMemcpyAsync(e->scalars, e->h_scalars, (size_t)(2 * Tm + 1) * 4, cudaMemcpyHostToDevice, st));
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_create(const ie_b200_engine_desc *desc, ie_b200_engine **out) {
  if (!desc || !out) return fail(IE_B200_E_ARG, "ie_b200_engine_create: NULL argument");
  if (ie_b200_device_count() < 1) return fail(IE_B200_E_CUDA, "no CUDA device: the engine has no CPU fallback");
  const ie_b200_engine_desc &d = *desc;
  if (!d.n_head || !d.n_kv || d.n_head % d.n_kv || !d.hd || !d.n_ctx || !d.T_max || !d.vocab || !d.arena_bytes)
    return fail(IE_B200_E_SIZE, "ie_b200_engine_create: empty or inconsistent description");
  ie_b200_engine *e = new ie_b200_engine();
  e->d = d;
  int rc = IE_B200_OK;
  auto chk = [&](cudaError_t err, const char *what) {
    if (err != cudaSuccess && rc == IE_B200_OK) rc = cuda_fail(err, what);
  };
  chk(cudaGetDevice(&e->device), "cudaGetDevice");
  chk(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking), "cudaStreamCreate");
  chk(cudaMalloc(&e->arena, d.arena_bytes + 256), "cudaMalloc(arena)");
  if (rc == IE_B200_OK) chk(cudaMemset(e->arena, 0, d.arena_bytes + 256), "cudaMemset(arena)");
  e->kv_layer_bytes = (size_t)d.n_kv * d.n_ctx * d.hd * (d.kv_f32 ? 4u : 2u);
  const size_t kvb = e->kv_layer_bytes * (d.n_kv_layers ? d.n_kv_layers : 1u);
  chk(cudaMalloc(&e->kc, kvb), "cudaMalloc(K cache)");
  chk(cudaMalloc(&e->vc, kvb), "cudaMalloc(V cache)");
  if (rc == IE_B200_OK) chk(cudaMemset(e->kc, 0, kvb), "cudaMemset"), chk(cudaMemset(e->vc, 0, kvb), "cudaMemset");
  const size_t rope_n = (size_t)d.n_ctx * (d.hd / 2u) * 4u;
  chk(cudaMalloc(&e->rope_cos, rope_n), "cudaMalloc(rope)");
  chk(cudaMalloc(&e->rope_sin, rope_n), "cudaMalloc(rope)");
  chk(cudaMalloc(&e->scalars, (size_t)(2 * d.T_max + 1) * 4), "cudaMalloc(scalars)");
  chk(cudaMallocHost(&e->h_scalars, (size_t)(2 * d.T_max + 1) * 4), "cudaMallocHost");
  chk(cudaMallocHost(&e->h_result, (size_t)d.T_max * 8 + 8), "cudaMallocHost");
  e->T_att = d.T_max < 16u ? d.T_max : 16u;
  chk(cudaMalloc(&e->attn_part, ie_b200_attn_part_bytes(d.n_head, d.hd, d.n_ctx, e->T_att)), "cudaMalloc(attention partials)");
  const size_t cw = ie_b200_attn_count_words(d.n_head, e->T_att) * 4u;
  chk(cudaMalloc(&e->attn_count, cw), "cudaMalloc(attention counters)");
  if (rc == IE_B200_OK) chk(cudaMemset(e->attn_count, 0, cw), "cudaMemset");
  chk(cudaMalloc(&e->argmax_part, ie_b200_argmax_part_bytes(d.T_max)), "cudaMalloc(argmax partials)");
  chk(cudaMalloc(&e->err, 16), "cudaMalloc(error word)");
  if (rc == IE_B200_OK) chk(cudaMemset(e->err, 0, 16), "cudaMemset");
  if (const char *af = getenv("IE_B200_ATTN_FUSE")) e->no_attn_fuse = af[0] == '0';
  if (const char *gm = getenv("IE_B200_GEMM")) e->no_gemm = gm[0] == '0', e->gemm_mma = gm[0] == 'm';
  if (const char *pa = getenv("IE_B200_PREFILL_ATTN")) e->no_prefill_attn = pa[0] == '0';
  if (const char *sw = getenv("IE_B200_SWIGLU")) e->swi_epi = sw[0] == 'g' ? 1 : sw[0] == 'k' ? 0 : -1;
  if (const char *nm = getenv("IE_B200_NORM")) e->norm_mode = nm[0] == 'p' ? 1 : nm[0] == 't' ? 0 : 2;
  if (const char *sm = getenv("IE_B200_STEP")) e->step_mode = sm[0] == 'g' ? 1 : sm[0] == 'k' ? 2 : sm[0] == 'a' ? 0 : 1;
  chk(cudaMalloc(&e->sk_bar, 8), "cudaMalloc(barrier words)");
  if (rc == IE_B200_OK) chk(cudaMemset(e->sk_bar, 0, 8), "cudaMemset");
  chk(cudaMalloc(&e->hist, (size_t)(HIST_CAP + 1) * 4), "cudaMalloc(history)");
  if (rc == IE_B200_OK) chk(cudaMemset(e->hist, 0, (size_t)(HIST_CAP + 1) * 4), "cudaMemset");
  chk(cudaEventCreate(&e->ev0), "cudaEventCreate");
  chk(cudaEventCreate(&e->ev1), "cudaEventCreate");
  if (rc != IE_B200_OK) {
    ie_b200_engine_destroy(e);
    return rc;
  }
  *out = e;
  return IE_B200_OK;
}

// A release that fails must not leave its error behind for the next launch check to find (cudaPeekAtLastError): note it in
// the library's error text, on stderr, and clear it.
static void released(cudaError_t r, const char *what) {
  if (r == cudaSuccess) return;
  fprintf(stderr, "libie_b200: %s while releasing an engine: %s\n", what, cudaGetErrorString(r));
  cuda_fail(r, what);
  (void)cudaGetLastError();
}
#define IEB_RELEASE(call) released((call), #call)

extern "C" void ie_b200_engine_destroy(ie_b200_engine *e) {
  if (!e) return;
  IEB_RELEASE(cudaSetDevice(e->device));
  if (e->stream) IEB_RELEASE(cudaStreamSynchronize(e->stream));
  if (e->step_graph) IEB_RELEASE(cudaGraphExecDestroy(e->step_graph));
  for (auto &m : e->mats)
    if (m.owned) IEB_RELEASE(cudaFree(m.d));
  for (auto &v : e->vecs) IEB_RELEASE(cudaFree(v.d));
  IEB_RELEASE(cudaFree(e->arena)), IEB_RELEASE(cudaFree(e->kc)), IEB_RELEASE(cudaFree(e->vc)), IEB_RELEASE(cudaFree(e->rope_cos));
  IEB_RELEASE(cudaFree(e->rope_sin)), IEB_RELEASE(cudaFree(e->scalars));
  IEB_RELEASE(cudaFree(e->attn_part)), IEB_RELEASE(cudaFree(e->attn_count)), IEB_RELEASE(cudaFree(e->argmax_part)), IEB_RELEASE(cudaFree(e->hist));
  IEB_RELEASE(cudaFree(e->err));
  IEB_RELEASE(cudaFree(e->gemm_scratch)), IEB_RELEASE(cudaFree(e->topk_scratch));
  IEB_RELEASE(cudaFree(e->d_prog)), IEB_RELEASE(cudaFree(e->sk_part)), IEB_RELEASE(cudaFree(e->sk_amax)), IEB_RELEASE(cudaFree(e->sk_bar));
  IEB_RELEASE(cudaFree(e->sk_trace));
  if (e->h_scalars) IEB_RELEASE(cudaFreeHost(e->h_scalars));
  if (e->h_result) IEB_RELEASE(cudaFreeHost(e->h_result));
  if (e->ev0) IEB_RELEASE(cudaEventDestroy(e->ev0));
  if (e->ev1) IEB_RELEASE(cudaEventDestroy(e->ev1));
  if (e->stream) IEB_RELEASE(cudaStreamDestroy(e->stream));
  delete e;
}

static int kind_of_ggml(int t) {
  return t == IE_B200_GGML_F32 ? IE_B200_MAT_F32 : t == IE_B200_GGML_Q4_0 ? IE_B200_MAT_Q4 : t == IE_B200_GGML_Q8_0 ? IE_B200_MAT_Q8
         : t == IE_B200_GGML_Q4_K ? IE_B200_MAT_Q4K : t == IE_B200_GGML_Q6_K ? IE_B200_MAT_Q6K : -1;
}
static size_t gguf_bytes(int t, uint32_t rows, uint32_t cols) {
  const size_t n = (size_t)rows * cols;
  return t == IE_B200_GGML_F32 ? n * 4u : t == IE_B200_GGML_Q4_0 ? n / 32u * 18u : t == IE_B200_GGML_Q8_0 ? n / 32u * 34u
         : t == IE_B200_GGML_Q4_K ? n / 256u * 144u : n / 256u * 210u;
}

// Invalidate the captured step graph: the op list or a handle table changed.
static void drop_graph(ie_b200_engine *e) {
  if (e->step_graph) cudaGraphExecDestroy(e->step_graph), e->step_graph = nullptr;
  e->kernel_state = 0;
}

extern "C" int ie_b200_engine_add_mat_gguf(ie_b200_engine *e, int ggml_type, uint32_t rows, uint32_t cols, const void *h_bytes) {
  if (!e || !h_bytes) return fail(IE_B200_E_ARG, "ie_b200_engine_add_mat_gguf: NULL argument");
  IEB_CUDA(cudaSetDevice(e->device));
  const int kind = kind_of_ggml(ggml_type);
  if (kind < 0) return fail(IE_B200_E_ARG, "ie_b200_engine_add_mat_gguf: GGML type %d unsupported", ggml_type);
  const size_t src_n = gguf_bytes(ggml_type, rows, cols), dst_n = ie_b200_mat_bytes(kind, rows, cols);
  void *tmp = nullptr, *dst = nullptr;
  IEB_CUDA(cudaMalloc(&dst, dst_n ? dst_n : 16));
  if (kind == IE_B200_MAT_F32) {
    IEB_CUDA(h2d(e, dst, h_bytes, src_n));
  } else {
    IEB_CUDA(cudaMalloc(&tmp, src_n ? src_n : 16));
    IEB_CUDA(cudaMemcpyAsync(tmp, h_bytes, src_n, cudaMemcpyHostToDevice, e->stream));
    int r = ie_b200_repack_gguf(ggml_type, tmp, rows, cols, dst, e->stream);
    cudaStreamSynchronize(e->stream);
    cudaFree(tmp);
    if (r) {
      cudaFree(dst);
      return r;
    }
  }
  e->mats.push_back(EMat{kind, rows, cols, dst, true});
  return (int)e->mats.size() - 1;
}

extern "C" int ie_b200_engine_add_mat_ref(ie_b200_engine *e, int kind, uint32_t rows, uint32_t cols, const void *h_qw, const void *h_qs) {
  if (!e || !h_qw) return fail(IE_B200_E_ARG, "ie_b200_engine_add_mat_ref: NULL argument");
  IEB_CUDA(cudaSetDevice(e->device));
  const size_t nb = cols / 32u, n = (size_t)rows * nb;
  size_t qw_n, qs_n;
  switch (kind) {
    case IE_B200_MAT_F32: qw_n = (size_t)rows * cols * 4u, qs_n = 0; break;
    case IE_B200_MAT_Q4: qw_n = n * 16u, qs_n = n * 2u; break;
    case IE_B200_MAT_Q8: qw_n = n * 32u, qs_n = n * 2u; break;
    case IE_B200_MAT_Q4K: qw_n = n * 16u, qs_n = (n + (size_t)rows * (nb / 8u) * 2u) * 2u; break;
    case IE_B200_MAT_Q6K: qw_n = n * 24u, qs_n = (n + (size_t)rows * (nb / 8u)) * 2u; break;
    default: return fail(IE_B200_E_ARG, "ie_b200_engine_add_mat_ref: kind %d unsupported", kind);
  }
  if (kind != IE_B200_MAT_F32 && !h_qs) return fail(IE_B200_E_ARG, "ie_b200_engine_add_mat_ref: NULL scale array");
  void *dqw = nullptr, *dqs = nullptr, *dst = nullptr;
  const size_t dst_n = ie_b200_mat_bytes(kind, rows, cols);
  IEB_CUDA(cudaMalloc(&dst, dst_n ? dst_n : 16));
  if (kind == IE_B200_MAT_F32) {
    IEB_CUDA(h2d(e, dst, h_qw, qw_n));
  } else {
    IEB_CUDA(cudaMalloc(&dqw, qw_n ? qw_n : 16));
    IEB_CUDA(cudaMalloc(&dqs, qs_n ? qs_n : 16));
    IEB_CUDA(cudaMemcpyAsync(dqw, h_qw, qw_n, cudaMemcpyHostToDevice, e->stream));
    IEB_CUDA(cudaMemcpyAsync(dqs, h_qs, qs_n, cudaMemcpyHostToDevice, e->stream));
    int r = ie_b200_repack_ref(kind, dqw, dqs, rows, cols, dst, e->stream);
    cudaStreamSynchronize(e->stream);
    cudaFree(dqw), cudaFree(dqs);
    if (r) {
      cudaFree(dst);
      return r;
    }
  }
  e->mats.push_back(EMat{kind, rows, cols, dst, true});
  return (int)e->mats.size() - 1;
}

extern "C" int ie_b200_engine_add_mat_ref_part(ie_b200_engine *e, int kind, uint32_t rows, uint32_t cols, const void *h_qw, const void *h_qs,
                                               uint32_t n_ranges, const uint32_t *row0, const uint32_t *n_rows, uint32_t col0, uint32_t n_cols) {
  if (!e || !row0 || !n_rows || n_ranges == 0) return fail(IE_B200_E_ARG, "ie_b200_engine_add_mat_ref_part: NULL argument");
  IEB_CUDA(cudaSetDevice(e->device));
  const int whole = ie_b200_engine_add_mat_ref(e, kind, rows, cols, h_qw, h_qs);
  if (whole < 0) return whole;
  uint32_t part_rows = 0;
  for (uint32_t k = 0; k < n_ranges; k++) part_rows += n_rows[k];
  void *dst = nullptr;
  const size_t dst_n = ie_b200_mat_bytes(kind, part_rows, n_cols);
  cudaError_t ce = cudaMalloc(&dst, dst_n ? dst_n : 16);
  int r = ce == cudaSuccess ? ie_b200_mat_part(kind, e->mats[whole].d, rows, cols, n_ranges, row0, n_rows, col0, n_cols, dst, e->stream)
                            : cuda_fail(ce, "cudaMalloc(matrix part)");
  cudaStreamSynchronize(e->stream);
  cudaFree(e->mats[whole].d);  // the whole matrix was only the source of the part
  if (r) {
    cudaFree(dst);
    e->mats.pop_back();
    return r;
  }
  e->mats[whole] = EMat{kind, part_rows, n_cols, dst, true};
  return whole;
}

extern "C" int ie_b200_engine_add_mat_device(ie_b200_engine *e, int kind, uint32_t rows, uint32_t cols, const void *d_data) {
  if (!e || !d_data) return fail(IE_B200_E_ARG, "ie_b200_engine_add_mat_device: NULL argument");
  if (!aligned16(d_data)) return fail(IE_B200_E_ARG, "ie_b200_engine_add_mat_device: the matrix must be 16-byte aligned");
  e->mats.push_back(EMat{kind, rows, cols, const_cast<void *>(d_data), false});
  return (int)e->mats.size() - 1;
}

extern "C" int ie_b200_engine_add_vec(ie_b200_engine *e, const float *h_f, uint32_t n) {
  if (!e || !h_f) return fail(IE_B200_E_ARG, "ie_b200_engine_add_vec: NULL argument");
  IEB_CUDA(cudaSetDevice(e->device));
  float *dptr = nullptr;
  IEB_CUDA(cudaMalloc(&dptr, (size_t)(n ? n : 1) * 4));
  IEB_CUDA(h2d(e, dptr, h_f, (size_t)n * 4));
  e->vecs.push_back({dptr, n});
  return (int)e->vecs.size() - 1;
}

extern "C" int ie_b200_engine_set_rope(ie_b200_engine *e, const float *h_cos, const float *h_sin) {
  if (!e || !h_cos || !h_sin) return fail(IE_B200_E_ARG, "ie_b200_engine_set_rope: NULL argument");
  const size_t n = (size_t)e->d.n_ctx * (e->d.hd / 2u) * 4u;
  IEB_CUDA(h2d(e, e->rope_cos, h_cos, n));
  IEB_CUDA(h2d(e, e->rope_sin, h_sin, n));
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_set_ops(ie_b200_engine *e, const ie_b200_op *ops, uint32_t n_ops, uint32_t i_head) {
  if (!e || !ops) return fail(IE_B200_E_ARG, "ie_b200_engine_set_ops: NULL argument");
  if (i_head > n_ops) return fail(IE_B200_E_ARG, "ie_b200_engine_set_ops: head index %u > %u ops", i_head, n_ops);
  const uint64_t cap = e->d.arena_bytes;
  for (uint32_t i = 0; i < n_ops; i++) {
    const ie_b200_op &o = ops[i];
    const uint64_t offs[5] = {o.a, o.b, o.c, o.qo, o.res};
    for (uint64_t off : offs)
      if (off != IE_B200_NONE && off >= cap) return fail(IE_B200_E_ARG, "op %u: offset %llu outside the arena (%llu bytes)", i, (unsigned long long)off, (unsigned long long)cap);
    if ((o.kind == IE_B200_OP_ROPE_KV || o.kind == IE_B200_OP_ATTN) && (o.layer < 0 || (uint32_t)o.layer >= e->d.n_kv_layers))
      return fail(IE_B200_E_ARG, "op %u: KV layer %d of %u", i, o.layer, e->d.n_kv_layers);
    if (o.mat >= (int)e->mats.size() || o.vec >= (int)e->vecs.size()) return fail(IE_B200_E_ARG, "op %u: unknown handle", i);
  }
  e->ops.assign(ops, ops + n_ops);
  e->i_head = i_head;
  e->logits_n = e->d.vocab;
  for (uint32_t i = 0; i < n_ops; i++)
    if (ops[i].kind == IE_B200_OP_GEMV && ops[i].b == e->d.logits_off && ops[i].mat >= 0) e->logits_n = e->mats[ops[i].mat].rows;
  drop_graph(e);
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_set_collective(ie_b200_engine *e, ie_b200_allreduce *ar, uint32_t vocab_offset) {
  if (!e) return fail(IE_B200_E_ARG, "ie_b200_engine_set_collective: NULL engine");
  e->ar = ar, e->vocab_off = vocab_offset;
  drop_graph(e);
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_set_input(ie_b200_engine *e, const uint32_t *toks, uint32_t T, uint32_t pos, void *stream) {
  if (!e || !toks) return fail(IE_B200_E_ARG, "ie_b200_engine_set_input: NULL argument");
  return upload_input(e, toks, T, pos, static_cast<cudaStream_t>(stream));
}

extern "C" int ie_b200_engine_enqueue(ie_b200_engine *e, uint32_t first, uint32_t last, uint32_t T, void *stream) {
  if (!e) return fail(IE_B200_E_ARG, "ie_b200_engine_enqueue: NULL engine");
  if (first > last || last > e->ops.size()) return fail(IE_B200_E_ARG, "ie_b200_engine_enqueue: ops [%u, %u) of %zu", first, last, e->ops.size());
  if (T == 0 || T > e->d.T_max) return fail(IE_B200_E_SIZE, "ie_b200_engine_enqueue: %u tokens (1 .. %u)", T, e->d.T_max);
  return enqueue_range(e, first, last, T, ~0u, static_cast<cudaStream_t>(stream));
}


// ---- the persistent step kernel: op list -> phases -----------------------------------------------------------
// Recognised: EMBED; RMSNORM(+Q8) feeding GEMVs (folded into their prologue); GEMV (+bias, +residual) of the
// quantised kinds; ROPE_KV + ATTN of one layer on the half cache; interleaved SWIGLU(+Q8) feeding a GEMV (folded into
// its prologue); ARGMAX; with a collective attached: GEMV -> ALLREDUCE -> RMSNORM. Anything else: no program
// (returns 0) and the step graph runs instead.
static int build_program(ie_b200_engine *e) {
  const ie_b200_engine_desc &d = e->d;
  e->kernel_state = -1;
  if (!step_kernel_supports(d.hd, d.n_head, d.n_kv, d.kv_f32) || e->ops.empty() || e->ops[0].kind != IE_B200_OP_EMBED) return 0;
  const bool tp = e->ar != nullptr;
  if (tp && !ar_connected(e->ar)) return 0;
  std::vector<StepPhase> ph;
  auto A = [&](uint64_t off) -> uint8_t * { return off == IE_B200_NONE ? nullptr : e->arena + off; };
  const ie_b200_op &emb = e->ops[0];
  if (emb.mat < 0 || (e->mats[emb.mat].kind != IE_B200_MAT_Q4 && e->mats[emb.mat].kind != IE_B200_MAT_F32) || e->mats[emb.mat].cols != emb.n) return 0;
  {
    StepPhase p = {};
    p.kind = PH_EMBED;
    ph.push_back(p);
  }
  const ie_b200_op *norm = nullptr, *swi = nullptr;
  bool swi_in_gemv = false;
  uint64_t attq_off = IE_B200_NONE;
  const void *last_act = nullptr;  // what the previous GEMV phase staged (a following GEMV over the same activations keeps them)
  bool have_argmax = false;
  const uint32_t n = (uint32_t)e->ops.size();
  for (uint32_t i = 1; i < n; i++) {
    const ie_b200_op &o = e->ops[i];
    switch (o.kind) {
      case IE_B200_OP_RMSNORM:
        if (o.res != IE_B200_NONE || o.qo == IE_B200_NONE || o.vec < 0 || o.n % 32u || o.n / 32u > 1024u) return 0;
        norm = &o, last_act = nullptr;
        break;
      case IE_B200_OP_SWIGLU:
        if (o.nh != 1u || o.qo == IE_B200_NONE || o.n % 32u || o.n / 32u > 1024u) return 0;
        swi = &o, last_act = nullptr, swi_in_gemv = false;
        // the GEMV right before it produced the (gate, up) pairs: it writes silu(gate) * up itself (a warp owns whole pairs)
        if (!ph.empty() && ph.back().kind == PH_GEMV && ph.back().y == reinterpret_cast<float *>(A(o.a)) && !ph.back().bias && !ph.back().res &&
            !ph.back().push && ph.back().rows == 2u * o.n && o.b != IE_B200_NONE)
          ph.back().swi = 1u, ph.back().y = reinterpret_cast<float *>(A(o.b)), swi_in_gemv = true;
        break;
      case IE_B200_OP_GEMV: {
        if (o.mat < 0) return 0;
        const EMat &m = e->mats[o.mat];
        if (!gemv_direct_ok(m.kind, m.cols) || m.kind == IE_B200_MAT_Q8) return 0;  // (no Q8_0 instantiation in the persistent kernel)
        StepPhase p = {};
        p.kind = PH_GEMV, p.mkind = m.kind, p.w = static_cast<const uint8_t *>(m.d), p.rowb = row_bytes_of(m.kind, m.cols), p.rows = m.rows, p.nb = m.cols / 32u;
        p.y = reinterpret_cast<float *>(A(o.b)), p.bias = o.vec >= 0 ? e->vecs[o.vec].d : nullptr, p.res = reinterpret_cast<const float *>(A(o.res));
        const void *act = nullptr;
        if (norm && o.a == norm->qo && m.cols == norm->n) {
          p.pro = PRO_NORM, p.src = A(norm->a), p.norm_w = e->vecs[norm->vec].d, act = norm;
        } else if (swi && o.a == swi->qo && m.cols == swi->n) {
          p.pro = swi_in_gemv ? PRO_QUANT : PRO_SWIGLU, p.src = A(swi_in_gemv ? swi->b : swi->a), act = swi;
        } else if (attq_off != IE_B200_NONE && o.a == attq_off) {
          p.pro = PRO_Q8, p.src = A(o.a), act = A(o.a);
        } else {
          return 0;
        }
        if (act == last_act && !ph.empty() && ph.back().kind == PH_GEMV && !ph.back().push) p.pro = PRO_KEEP, ph.back().nobar = 1;
        last_act = act;
        if (tp && i + 1 < n && e->ops[i + 1].kind == IE_B200_OP_ALLREDUCE) {
          const ie_b200_op &ar = e->ops[i + 1];
          if (ar.a != o.b || ar.n != m.rows || o.vec >= 0 || o.res != IE_B200_NONE) return 0;
          p.push = 1, p.nobar = 1;
          ph.push_back(p);
          StepPhase r = {};
          r.kind = PH_REDUCE, r.rows = ar.n, r.res = reinterpret_cast<const float *>(A(ar.res != IE_B200_NONE ? ar.res : ar.c)), r.y = reinterpret_cast<float *>(A(ar.c));
          ph.push_back(r);
          last_act = nullptr;
          i++;
          break;
        }
        ph.push_back(p);
        break;
      }
      case IE_B200_OP_ROPE_KV: {
        if (i + 1 >= n) return 0;
        const ie_b200_op &at_ = e->ops[i + 1];
        if (at_.kind != IE_B200_OP_ATTN || at_.layer != o.layer || at_.a != o.a || at_.qo == IE_B200_NONE || o.nh != d.n_head) return 0;
        if (o.b != o.a + (uint64_t)d.n_head * d.hd * 4u || o.c != o.a + (uint64_t)(d.n_head + d.n_kv) * d.hd * 4u) return 0;
        StepPhase p = {};
        p.kind = PH_ATTN, p.q = reinterpret_cast<const float *>(A(o.a));
        p.kc = static_cast<char *>(e->kc) + e->kv_layer_bytes * o.layer, p.vc = static_cast<char *>(e->vc) + e->kv_layer_bytes * o.layer;
        ph.push_back(p);
        StepPhase q = {};
        q.kind = PH_MERGE, q.att = reinterpret_cast<float *>(A(at_.b)), q.attq = A(at_.qo);
        ph.push_back(q);
        attq_off = at_.qo, last_act = nullptr;
        i++;
        break;
      }
      case IE_B200_OP_ARGMAX: {
        if (o.a != d.logits_off || o.b != d.argmax_off) return 0;
        StepPhase p = {};
        p.kind = PH_ARGMAX;
        ph.push_back(p);
        StepPhase f = {};
        f.kind = tp ? PH_XARGMAX : PH_FINISH;
        ph.push_back(f);
        have_argmax = true;
        e->sk.logits = reinterpret_cast<const float *>(A(o.a)), e->sk.n_logits = o.n;
        break;
      }
      default: return 0;
    }
  }
  if (!have_argmax || ph.back().kind == PH_ARGMAX) return 0;
  // Which phase pulls the head of which later matrix into L2: the weights form one stream in program order (cyclic: after
  // the output head comes layer 0 of the next token); every phase claims the next unclaimed matrix (its first 24 MB) while
  // less than 40 MB are claimed and not yet consumed, so the fetch from HBM runs ahead of the GEMVs through attention,
  // merge and barriers, and never ahead by more than the L2 can hold. Two laps: the second one is the steady state.
  {
    std::vector<size_t> g;
    for (size_t k = 0; k < ph.size(); k++)
      if (ph[k].kind == PH_GEMV) g.push_back(k);
    const uint64_t WINDOW = 40ull << 20, CAP = 24ull << 20;
    std::vector<uint64_t> claimed(ph.size(), 0);
    uint64_t ahead = 0;
    size_t next = 0, outstanding = 0;
    for (int lap = 0; lap < 2 && g.size() > 1; lap++)
      for (size_t k = 0; k < ph.size(); k++) {
        if (ph[k].kind == PH_GEMV) {
          if (claimed[k]) ahead -= claimed[k] < ahead ? claimed[k] : ahead, claimed[k] = 0, outstanding--;
          else if (g[next] == k) next = (next + 1) % g.size();  // nobody fetched it ahead: its own loads do
        }
        ph[k].pf = nullptr, ph[k].pf_bytes = 0;
        if (ahead < WINDOW && outstanding + 1 < g.size() && g[next] != k && !claimed[g[next]]) {
          const size_t j = g[next];
          const uint64_t bytes = ph[j].rowb * ph[j].rows, take = bytes < CAP ? bytes : CAP;
          ph[k].pf = ph[j].w, ph[k].pf_bytes = take;
          claimed[j] = take, ahead += take, outstanding++;
          next = (next + 1) % g.size();
        }
      }
  }
  bool has_q4 = false, has_k = false;
  for (const StepPhase &q : ph)
    if (q.kind == PH_GEMV) (q.mkind == IE_B200_MAT_Q4 ? has_q4 : has_k) = true;
  e->sk_kset = has_q4 && has_k ? 2 : has_k ? 1 : 0;
  StepArgs &a = e->sk;
  a.smax = step_kernel_smax(d.n_kv);
  cudaFree(e->d_prog), cudaFree(e->sk_part), cudaFree(e->sk_amax);
  e->d_prog = nullptr, e->sk_part = nullptr, e->sk_amax = nullptr;
  IEB_CUDA(cudaMalloc(&e->d_prog, ph.size() * sizeof(StepPhase)));
  IEB_CUDA(h2d(e, e->d_prog, ph.data(), ph.size() * sizeof(StepPhase)));
  IEB_CUDA(cudaMalloc(&e->sk_part, (size_t)d.n_head * a.smax * (d.hd + 2u) * sizeof(float)));
  IEB_CUDA(cudaMalloc(&e->sk_amax, step_kernel_amax_bytes()));
  a.prog = e->d_prog, a.n_phases = (uint32_t)ph.size(), a.n_steps = 1;
  a.scalars = e->scalars, a.Tm = d.T_max, a.hist = e->hist, a.hist_cap = HIST_CAP, a.bar = e->sk_bar, a.err = e->err, a.eps = d.eps;
  a.n_head = d.n_head, a.n_kv = d.n_kv, a.kv_len = d.n_ctx, a.neox = d.neox ? 1u : 0u, a.cs = e->rope_cos, a.sn = e->rope_sin;
  a.part = e->sk_part, a.amax_part = e->sk_amax, a.result = reinterpret_cast<uint32_t *>(e->arena + d.argmax_off);
  a.emb = static_cast<const uint8_t *>(e->mats[emb.mat].d), a.emb_kind = e->mats[emb.mat].kind, a.dim = emb.n, a.x = reinterpret_cast<float *>(A(emb.a));
  ar_push_info(e->ar, &a.push);
  a.vocab_off = e->vocab_off, a.wait_ns = AR_WAIT_NS, a.trace = e->sk_trace;
  a.knobs = 3u;
  e->kernel_state = 1;
  return 1;
}

// Does a one-token step run as the persistent kernel? Builds the program on first use.
static int use_step_kernel(ie_b200_engine *e, bool *yes) {
  *yes = false;
  if (e->step_mode == 1) return IE_B200_OK;
  if (e->kernel_state == 0) {
    const int r = build_program(e);
    if (r < 0) return r;
  }
  if (e->kernel_state != 1 && e->step_mode == 2)
    return fail(IE_B200_E_STATE, "the persistent step kernel was requested, but this op list / shape has no program (half cache, heads of 64 or 128, llama / qwen2 ops)");
  *yes = e->kernel_state == 1;
  return IE_B200_OK;
}

// Capture ops [0, n_ops) for one token into an executable graph.
static int capture_step(ie_b200_engine *e) {
  cudaGraph_t g = nullptr;
  const uint64_t before = ie_b200_launch_count();
  IEB_CUDA(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
  int r = IE_B200_OK;
  r = enqueue_range(e, 0, (uint32_t)e->ops.size(), 1, ~0u, e->stream);
  if (r == IE_B200_OK) {
    advance_kernel<<<1, 256, 0, e->stream>>>(e->scalars, e->d.T_max, reinterpret_cast<const uint32_t *>(e->arena + e->d.argmax_off), e->hist, HIST_CAP);
    count_launch();
  }
  cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
  if (r != IE_B200_OK) {
    if (g) cudaGraphDestroy(g);
    return r;
  }
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaStreamEndCapture");
  e->step_launches = (uint32_t)(ie_b200_launch_count() - before);
  ce = cudaGraphInstantiate(&e->step_graph, g, 0);
  cudaGraphDestroy(g);
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaGraphInstantiate");
  return IE_B200_OK;
}

// The step graph's attention grid is sized for a bound on the positions, not for the whole context: a chat at position 200
// of an 8192-position context would otherwise launch the splits of 8192 positions every step (and miss the short-context
// form of the kernel). The bound doubles from 512; the graph is captured again when the positions outgrow it, or fall to a
// quarter of it. (Correctness does not hang on it: a split simply grows past the bound.)
static int step_graph_for(ie_b200_engine *e, uint32_t positions) {
  uint32_t want = 512u;
  while (want < positions && want < e->d.n_ctx) want *= 2u;
  if (want > e->d.n_ctx) want = e->d.n_ctx;
  if (e->step_graph && (want > e->ctx_bound || want * 4u <= e->ctx_bound)) cudaGraphExecDestroy(e->step_graph), e->step_graph = nullptr;
  if (e->step_graph) return IE_B200_OK;
  if (want > e->ctx_bound || want * 4u <= e->ctx_bound || e->ctx_bound == 0) e->ctx_bound = want;
  return capture_step(e);
}

// A step, a decode run and a prompt chunk each come as two halves: everything up to and including the copies of the results
// (asynchronous, on the engine's stream) and the wait for them. A host that drives the shards of one model on several GPUs
// from one thread enqueues every shard's first half before it waits for any of them.
extern "C" int ie_b200_engine_step_begin(ie_b200_engine *e, uint32_t tok, uint32_t pos, int timed) {
  if (!e) return fail(IE_B200_E_ARG, "ie_b200_engine_step: NULL argument");
  if (e->ops.empty()) return fail(IE_B200_E_STATE, "ie_b200_engine_step: no op list");
  IEB_CUDA(cudaSetDevice(e->device));
  bool kernel = false;
  if (int r = use_step_kernel(e, &kernel)) return r;
  if (!kernel)
    if (int r = step_graph_for(e, pos + 1u)) return r;
  cudaStream_t st = e->stream;
  e->timed = timed != 0;
  if (timed) IEB_CUDA(cudaEventRecord(e->ev0, st));
  if (int r = upload_input(e, &tok, 1, pos, st)) return r;
  if (kernel) {
    e->sk.n_steps = 1;
    if (int r = step_kernel_launch(e->sk, e->d.hd, e->sk_kset, st)) return r;
  } else {
    IEB_CUDA(cudaGraphLaunch(e->step_graph, st));
    count_launch(e->step_launches);
  }
  IEB_CUDA(cudaMemcpyAsync(e->h_result, e->arena + e->d.argmax_off, 8, cudaMemcpyDeviceToHost, st));
  IEB_CUDA(cudaMemcpyAsync(e->h_result + 2, e->err, 4, cudaMemcpyDeviceToHost, st));
  if (timed) IEB_CUDA(cudaEventRecord(e->ev1, st));
  return IE_B200_OK;
}

// (The first half copies into the engine's own pinned memory only: a copy into the caller's pageable memory would make the
// host wait for the step, and with it for ranks whose work this thread has not enqueued yet.)
extern "C" int ie_b200_engine_step_end(ie_b200_engine *e, float *h_logits, uint32_t *next, double *ms) {
  if (!e || !next) return fail(IE_B200_E_ARG, "ie_b200_engine_step: NULL argument");
  IEB_CUDA(cudaSetDevice(e->device));
  IEB_CUDA(cudaStreamSynchronize(e->stream));
  if (h_logits) IEB_CUDA(cudaMemcpy(h_logits, e->arena + e->d.logits_off, (size_t)e->logits_n * 4, cudaMemcpyDeviceToHost));
  if (ms && e->timed) {
    float f = 0;
    IEB_CUDA(cudaEventElapsedTime(&f, e->ev0, e->ev1));
    *ms = f;
  }
  if (e->h_result[2]) return fail(IE_B200_E_DEVICE, "a kernel gave up a bounded wait (device error word %u)", e->h_result[2]);
  *next = e->h_result[0];
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_step(ie_b200_engine *e, uint32_t tok, uint32_t pos, float *h_logits, uint32_t *next, double *ms) {
  if (!e || !next) return fail(IE_B200_E_ARG, "ie_b200_engine_step: NULL argument");
  if (int r = ie_b200_engine_step_begin(e, tok, pos, ms != nullptr)) return r;
  return ie_b200_engine_step_end(e, h_logits, next, ms);
}

extern "C" int ie_b200_engine_decode_begin(ie_b200_engine *e, uint32_t tok, uint32_t pos, uint32_t K) {
  if (!e) return fail(IE_B200_E_ARG, "ie_b200_engine_decode: NULL argument");
  if (e->ops.empty()) return fail(IE_B200_E_STATE, "ie_b200_engine_decode: no op list");
  if (K == 0 || K > HIST_CAP) return fail(IE_B200_E_SIZE, "ie_b200_engine_decode: %u steps (1 .. %u per call)", K, HIST_CAP);
  if ((uint64_t)pos + K > e->d.n_ctx) return fail(IE_B200_E_SIZE, "ie_b200_engine_decode: positions %u .. %u exceed the context %u", pos, pos + K - 1, e->d.n_ctx);
  IEB_CUDA(cudaSetDevice(e->device));
  bool kernel = false;
  if (int r = use_step_kernel(e, &kernel)) return r;
  if (!kernel)
    if (int r = step_graph_for(e, pos + K)) return r;
  cudaStream_t st = e->stream;
  if (int r = upload_input(e, &tok, 1, pos, st)) return r;
  IEB_CUDA(cudaMemsetAsync(e->hist + HIST_CAP, 0, 4, st));
  IEB_CUDA(cudaEventRecord(e->ev0, st));
  if (kernel) {  // one launch: the kernel loops over the K tokens itself
    e->sk.n_steps = K;
    if (int r = step_kernel_launch(e->sk, e->d.hd, e->sk_kset, st)) return r;
  } else {
    for (uint32_t k = 0; k < K; k++) IEB_CUDA(cudaGraphLaunch(e->step_graph, st));
    count_launch(e->step_launches * K);
  }
  IEB_CUDA(cudaEventRecord(e->ev1, st));
  IEB_CUDA(cudaMemcpyAsync(e->h_result + 2, e->err, 4, cudaMemcpyDeviceToHost, st));
  e->run_T = K;
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_decode_end(ie_b200_engine *e, uint32_t *h_out, double *ms) {
  if (!e || !h_out) return fail(IE_B200_E_ARG, "ie_b200_engine_decode: NULL argument");
  IEB_CUDA(cudaSetDevice(e->device));
  IEB_CUDA(cudaStreamSynchronize(e->stream));
  IEB_CUDA(cudaMemcpy(h_out, e->hist, (size_t)e->run_T * 4, cudaMemcpyDeviceToHost));
  if (e->h_result[2]) return fail(IE_B200_E_DEVICE, "a kernel gave up a bounded wait (device error word %u)", e->h_result[2]);
  if (ms) {
    float f = 0;
    IEB_CUDA(cudaEventElapsedTime(&f, e->ev0, e->ev1));
    *ms = f;
  }
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_decode(ie_b200_engine *e, uint32_t tok, uint32_t pos, uint32_t K, uint32_t *h_out, double *ms) {
  if (!e || !h_out) return fail(IE_B200_E_ARG, "ie_b200_engine_decode: NULL argument");
  if (K == 0) return e->ops.empty() ? fail(IE_B200_E_STATE, "ie_b200_engine_decode: no op list") : IE_B200_OK;
  if (int r = ie_b200_engine_decode_begin(e, tok, pos, K)) return r;
  return ie_b200_engine_decode_end(e, h_out, ms);
}

extern "C" int ie_b200_engine_enqueue_kinds(ie_b200_engine *e, uint32_t first, uint32_t last, uint32_t kind_mask, uint32_t T, void *stream) {
  if (!e) return fail(IE_B200_E_ARG, "ie_b200_engine_enqueue_kinds: NULL engine");
  if (first > last || last > e->ops.size()) return fail(IE_B200_E_ARG, "ie_b200_engine_enqueue_kinds: ops [%u, %u) of %zu", first, last, e->ops.size());
  if (T == 0 || T > e->d.T_max) return fail(IE_B200_E_SIZE, "ie_b200_engine_enqueue_kinds: %u tokens (1 .. %u)", T, e->d.T_max);
  return enqueue_range(e, first, last, T, kind_mask, static_cast<cudaStream_t>(stream));
}

// What a prompt chunk's tensor-core GEMMs need once per matrix (the scale exponent, which is read back from the device) and
// once per engine (the scratch), made ready BEFORE anything of the run is enqueued: both wait for the stream, and a wait in
// the middle of a run would wait for exchange kernels whose partners on other GPUs this thread has not enqueued yet.
static int prepare_chunks(ie_b200_engine *e, uint32_t T) {
  if (T < 17 || e->no_gemm || e->gemm_mma) return IE_B200_OK;
  size_t need = 0;
  for (const ie_b200_op &o : e->ops) {
    if (o.kind != IE_B200_OP_GEMV || o.mat < 0 || (size_t)o.mat >= e->mats.size() || o.a_stride % 16u) continue;
    EMat &m = e->mats[o.mat];
    if (m.kind == IE_B200_MAT_F32) continue;
    if (m.tc_exp == INT32_MIN)
      if (int r = ie_b200_mat_tc_exp(m.kind, m.d, m.rows, m.cols, &m.tc_exp, e->stream)) return r;
    const size_t n = ie_b200_gemm_tc_scratch_bytes(m.rows, m.cols, e->d.T_max);
    need = n > need ? n : need;
  }
  if (need > e->gemm_scratch_bytes) {
    IEB_CUDA(cudaStreamSynchronize(e->stream));
    cudaFree(e->gemm_scratch), e->gemm_scratch = nullptr, e->gemm_scratch_bytes = 0;
    IEB_CUDA(cudaMalloc(&e->gemm_scratch, need));
    e->gemm_scratch_bytes = need;
  }
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_run_begin(ie_b200_engine *e, const uint32_t *toks, uint32_t T, uint32_t pos, int last_only) {
  if (!e || !toks) return fail(IE_B200_E_ARG, "ie_b200_engine_run: NULL argument");
  if (e->ops.empty()) return fail(IE_B200_E_STATE, "ie_b200_engine_run: no op list");
  IEB_CUDA(cudaSetDevice(e->device));
  if (int r = prepare_chunks(e, T)) return r;
  cudaStream_t st = e->stream;
  if (int r = upload_input(e, toks, T, pos, st)) return r;
  const uint32_t n_ops = (uint32_t)e->ops.size(), ih = last_only ? e->i_head : n_ops;
  for (uint32_t i = 0; i < ih; i++)
    if (int r = launch_op(e, e->ops[i], 0, T, st)) return r;
  for (uint32_t i = ih; i < n_ops; i++)  // the output head for the last token only
    if (int r = launch_op(e, e->ops[i], T - 1, 1, st)) return r;
  IEB_CUDA(cudaMemcpy2DAsync(e->h_result, 8, e->arena + e->d.argmax_off, e->d.argmax_stride ? e->d.argmax_stride : 8, 8, T, cudaMemcpyDeviceToHost, st));
  IEB_CUDA(cudaMemcpyAsync(e->h_result + 2 * e->d.T_max, e->err, 4, cudaMemcpyDeviceToHost, st));
  e->run_T = T;
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_run_end(ie_b200_engine *e, uint32_t *out, float *prob) {
  if (!e || !out) return fail(IE_B200_E_ARG, "ie_b200_engine_run: NULL argument");
  IEB_CUDA(cudaSetDevice(e->device));
  IEB_CUDA(cudaStreamSynchronize(e->stream));
  if (e->h_result[2 * e->d.T_max]) return fail(IE_B200_E_DEVICE, "a kernel gave up a bounded wait (device error word %u)", e->h_result[2 * e->d.T_max]);
  for (uint32_t t = 0; t < e->run_T; t++) {
    out[t] = e->h_result[2 * t];
    if (prob) std::memcpy(&prob[t], &e->h_result[2 * t + 1], 4);
  }
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_run(ie_b200_engine *e, const uint32_t *toks, uint32_t T, uint32_t pos, int last_only, uint32_t *out, float *prob) {
  if (!e || !toks || !out) return fail(IE_B200_E_ARG, "ie_b200_engine_run: NULL argument");
  if (int r = ie_b200_engine_run_begin(e, toks, T, pos, last_only)) return r;
  return ie_b200_engine_run_end(e, out, prob);
}

extern "C" int ie_b200_engine_read_rows(ie_b200_engine *e, uint64_t off, uint32_t stride, uint32_t r0, uint32_t n, void *h_dst) {
  if (!e || !h_dst) return fail(IE_B200_E_ARG, "ie_b200_engine_read_rows: NULL argument");
  const uint64_t lo = off + (uint64_t)stride * r0, len = (uint64_t)stride * n;
  if (lo + len > e->d.arena_bytes) return fail(IE_B200_E_ARG, "ie_b200_engine_read_rows: rows outside the arena");
  IEB_CUDA(cudaMemcpyAsync(h_dst, e->arena + lo, len, cudaMemcpyDeviceToHost, e->stream));
  IEB_CUDA(cudaStreamSynchronize(e->stream));
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_write_rows(ie_b200_engine *e, uint64_t off, uint32_t stride, uint32_t r0, uint32_t n, const void *h_src) {
  if (!e || !h_src) return fail(IE_B200_E_ARG, "ie_b200_engine_write_rows: NULL argument");
  const uint64_t lo = off + (uint64_t)stride * r0, len = (uint64_t)stride * n;
  if (lo + len > e->d.arena_bytes) return fail(IE_B200_E_ARG, "ie_b200_engine_write_rows: rows outside the arena");
  IEB_CUDA(cudaMemcpyAsync(e->arena + lo, h_src, len, cudaMemcpyHostToDevice, e->stream));
  IEB_CUDA(cudaStreamSynchronize(e->stream));
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_topk(ie_b200_engine *e, uint64_t off, uint32_t stride, uint32_t r0, uint32_t n, uint32_t nv, uint32_t K, float *h_val,
                                   uint32_t *h_idx) {
  if (!e || !h_val || !h_idx) return fail(IE_B200_E_ARG, "ie_b200_engine_topk: NULL argument");
  if (n == 0) return 1;
  if (K == 0 || K > 64u || K > nv || (uint64_t)((nv + 2047u) / 2048u) * K > 6144u) return 0;  // the caller selects on the host
  if (off + (uint64_t)stride * (r0 + n - 1) + (uint64_t)nv * 4u > e->d.arena_bytes) return fail(IE_B200_E_ARG, "ie_b200_engine_topk: rows outside the arena");
  IEB_CUDA(cudaSetDevice(e->device));
  const size_t need = ie_b200_topk_scratch_bytes(nv, K, n) + (size_t)n * K * 8u;
  if (need > e->topk_bytes) {
    IEB_CUDA(cudaStreamSynchronize(e->stream));
    cudaFree(e->topk_scratch), e->topk_scratch = nullptr, e->topk_bytes = 0;
    IEB_CUDA(cudaMalloc(&e->topk_scratch, need));
    e->topk_bytes = need;
  }
  float *d_val = static_cast<float *>(e->topk_scratch);
  uint32_t *d_idx = reinterpret_cast<uint32_t *>(d_val + (size_t)n * K);
  void *scratch = d_idx + (size_t)n * K;
  if (int r = ie_b200_topk(reinterpret_cast<const float *>(e->arena + off + (uint64_t)stride * r0), nv, K, n, stride, d_val, d_idx, scratch, e->stream)) return r;
  IEB_CUDA(cudaMemcpyAsync(h_val, d_val, (size_t)n * K * 4u, cudaMemcpyDeviceToHost, e->stream));
  IEB_CUDA(cudaMemcpyAsync(h_idx, d_idx, (size_t)n * K * 4u, cudaMemcpyDeviceToHost, e->stream));
  IEB_CUDA(cudaStreamSynchronize(e->stream));
  return 1;
}

extern "C" int ie_b200_engine_copy_rows(ie_b200_engine *e, uint64_t dst_off, uint32_t dst_stride, uint32_t d0, uint64_t src_off, uint32_t src_stride,
                                        uint32_t r0, uint32_t n, uint32_t row_bytes, int zero) {
  if (!e) return fail(IE_B200_E_ARG, "ie_b200_engine_copy_rows: NULL engine");
  if (n == 0) return IE_B200_OK;
  uint8_t *dst = e->arena + dst_off + (uint64_t)dst_stride * d0;
  if (dst_off + (uint64_t)dst_stride * (d0 + n - 1) + row_bytes > e->d.arena_bytes) return fail(IE_B200_E_ARG, "ie_b200_engine_copy_rows: outside the arena");
  if (zero) {
    IEB_CUDA(cudaMemset2DAsync(dst, dst_stride, 0, row_bytes, n, e->stream));
  } else {
    if (src_off + (uint64_t)src_stride * (r0 + n - 1) + row_bytes > e->d.arena_bytes) return fail(IE_B200_E_ARG, "ie_b200_engine_copy_rows: outside the arena");
    IEB_CUDA(cudaMemcpy2DAsync(dst, dst_stride, e->arena + src_off + (uint64_t)src_stride * r0, src_stride, row_bytes, n, cudaMemcpyDeviceToDevice, e->stream));
  }
  IEB_CUDA(cudaStreamSynchronize(e->stream));
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_clear_error(ie_b200_engine *e) {
  if (!e) return fail(IE_B200_E_ARG, "ie_b200_engine_clear_error: NULL engine");
  IEB_CUDA(cudaSetDevice(e->device));
  IEB_CUDA(cudaMemsetAsync(e->err, 0, 4, e->stream));
  IEB_CUDA(cudaMemsetAsync(e->sk_bar, 0, 8, e->stream));
  IEB_CUDA(cudaStreamSynchronize(e->stream));
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_set_step_mode(ie_b200_engine *e, int mode) {
  if (!e || mode < 0 || mode > 2) return fail(IE_B200_E_ARG, "ie_b200_engine_set_step_mode: mode %d (0 auto, 1 graph, 2 kernel)", mode);
  e->step_mode = mode;
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_step_is_kernel(ie_b200_engine *e) {
  if (!e || e->ops.empty()) return 0;
  bool kernel = false;
  if (cudaSetDevice(e->device) != cudaSuccess || use_step_kernel(e, &kernel) != IE_B200_OK) return 0;
  return kernel ? 1 : 0;
}

extern "C" int ie_b200_engine_phase_times(ie_b200_engine *e, int enable, double *h_ms36) {
  if (!e) return fail(IE_B200_E_ARG, "ie_b200_engine_phase_times: NULL engine");
  IEB_CUDA(cudaSetDevice(e->device));
  IEB_CUDA(cudaStreamSynchronize(e->stream));
  if (h_ms36) {
    unsigned long long raw[36] = {};
    if (e->sk_trace) IEB_CUDA(cudaMemcpy(raw, e->sk_trace, sizeof raw, cudaMemcpyDeviceToHost));
    for (int i = 0; i < 36; i++) h_ms36[i] = i % 3 == 2 ? (double)raw[i] : (double)raw[i] * 1e-6;
  }
  if (enable && !e->sk_trace) IEB_CUDA(cudaMalloc(&e->sk_trace, 36 * sizeof(unsigned long long)));
  if (e->sk_trace) IEB_CUDA(cudaMemset(e->sk_trace, 0, 36 * sizeof(unsigned long long)));
  if (!enable && e->sk_trace) cudaFree(e->sk_trace), e->sk_trace = nullptr;
  e->sk.trace = e->sk_trace;
  return IE_B200_OK;
}

extern "C" int ie_b200_engine_inject_abort(ie_b200_engine *e) {
  if (!e) return fail(IE_B200_E_ARG, "ie_b200_engine_inject_abort: NULL engine");
  IEB_CUDA(cudaSetDevice(e->device));
  const uint32_t one = 1u;
  IEB_CUDA(cudaMemcpyAsync(e->sk_bar + 1, &one, 4, cudaMemcpyHostToDevice, e->stream));
  IEB_CUDA(cudaStreamSynchronize(e->stream));
  return IE_B200_OK;
}

extern "C" void *ie_b200_engine_arena(ie_b200_engine *e) { return e ? e->arena : nullptr; }
extern "C" void *ie_b200_engine_input_scalars(ie_b200_engine *e) { return e ? e->scalars : nullptr; }

extern "C" uint64_t ie_b200_engine_weight_bytes_per_token(ie_b200_engine *e) {
  if (!e) return 0;
  uint64_t wb = 0;
  for (const auto &o : e->ops) {
    if (o.kind != IE_B200_OP_GEMV || o.mat < 0) continue;
    const EMat &m = e->mats[o.mat];
    const uint64_t nblk = (uint64_t)m.rows * (m.cols / 32u);
    wb += m.kind == IE_B200_MAT_F32 ? (uint64_t)m.rows * m.cols * 4u : m.kind == IE_B200_MAT_Q6K ? nblk * 210u / 8u : m.kind == IE_B200_MAT_Q8 ? nblk * 34u : nblk * 18u;
  }
  return wb;
}

extern "C" uint32_t ie_b200_engine_launches_per_step(ie_b200_engine *e) {
  if (!e || e->ops.empty()) return 0;
  bool kernel = false;
  if (cudaSetDevice(e->device) != cudaSuccess || use_step_kernel(e, &kernel) != IE_B200_OK) return 0;
  if (kernel) return 1;
  if (!e->step_graph) step_graph_for(e, e->ctx_bound ? e->ctx_bound : 1u);
  return e->step_launches;
}
