// step_kernel.cuh -- the program a persistent decode-step kernel executes (step_kernel.cu) and its launcher.
// The engine translates its op list into phases once; the kernel walks the phases for every token with a grid
// barrier between dependent phases, so a whole decode step (or K of them) is one launch.
#pragma once

#include "common.cuh"
#include "peer_ll.cuh"

namespace ieb {

enum {
  PH_EMBED = 0,   // x = embedding row of the step's token (CTA 0)
  PH_GEMV = 1,    // y = W act (+bias) (+res); act staged by the prologue `pro`
  PH_ATTN = 2,    // RoPE, KV store and the split attention of one layer: partial records per (head, split)
  PH_MERGE = 3,   // partial records -> attention output and its Q8 copy (one warp per head)
  PH_ARGMAX = 4,  // every CTA's (max, first index, sum of exp) over its slice of the logits
  PH_FINISH = 5,  // CTA 0 merges the slices, writes {token, probability}, logs the token and advances token / position
  PH_REDUCE = 6,  // tensor parallel: x += sum over the ranks of the partial rows a PH_GEMV pushed (rank order)
  PH_XARGMAX = 7  // tensor parallel: the ranks' local winners to every rank, best one kept (in PH_FINISH's place)
};
enum {
  PRO_Q8 = 0,      // src: a Q8 buffer
  PRO_NORM = 1,    // src: f32 vector; act = Q8(rmsnorm(src) * norm_w)
  PRO_SWIGLU = 2,  // src: interleaved (gate_i, up_i) f32 pairs; act = Q8(silu(gate) * up)
  PRO_KEEP = 3,    // the activations the previous phase staged are still in shared memory
  PRO_QUANT = 4    // src: f32 vector; act = Q8(src)
};

struct StepPhase {
  int32_t kind, mkind, pro, nobar;  // nobar: the next phase does not depend on this one (no grid barrier after it)
  const uint8_t *w;
  uint64_t rowb;
  uint32_t rows, nb;
  const void *src;
  const float *norm_w;
  float *y;
  const float *bias, *res;
  void *kc, *vc;              // PH_ATTN: the layer's caches [kv head][position][hd] half
  const float *q;             // PH_ATTN: the un-rotated q | k | v of the step
  float *att;                 // PH_MERGE: attention output, and its Q8 copy
  uint8_t *attq;
  const uint8_t *pf;          // weights that idle warps of this phase pull into L2 (the matrices of the next phases)
  uint64_t pf_bytes;
  uint32_t push;              // PH_GEMV under tensor parallelism: finished rows also go to the peers' slots
  uint32_t swi;               // PH_GEMV over interleaved (gate_i, up_i) rows: y[i] = silu(gate_i) * up_i instead of the two rows
};

struct StepArgs {
  const StepPhase *prog;      // device memory
  uint32_t n_phases, n_steps;
  uint32_t *scalars;          // [0, Tm) token ids, [Tm] first position, [Tm + 1 + t] position of token t
  uint32_t Tm;
  uint32_t *hist, hist_cap;   // generated-token ring and its counter (hist[hist_cap])
  uint32_t *bar;              // [0] arrivals of the grid barrier (zero at launch), [1] abort flag
  uint32_t *err;              // device error word
  float eps;
  uint32_t n_head, n_kv, kv_len, neox;
  const float *cs, *sn;       // RoPE tables [position][hd / 2]
  float *part;                // attention partial records [head][smax][hd + 2]
  uint32_t smax;              // most splits per KV head
  void *amax_part;            // PH_ARGMAX records, one per CTA
  const float *logits;
  uint32_t n_logits;
  uint32_t *result;           // {argmax index, f32 bits of its softmax probability}
  const uint8_t *emb;         // embedding matrix (streaming layout or f32 rows)
  int32_t emb_kind;
  uint32_t dim;
  float *x;                   // residual stream
  ArPush push;                // tensor parallel (world > 1): the peers' low-latency slots
  uint32_t vocab_off;
  uint64_t wait_ns;           // limit of every wait inside the kernel
  uint32_t knobs;             // bit 0: a warp asks its next row group into L2 before it works on the current one; bit 1: phases pull the head of
                              // a later phase's matrix (StepPhase::pf) into L2
  unsigned long long *trace;  // NULL, or 8 x {work ns, barrier ns, barriers} summed by CTA 0 per kind of the phase a barrier closes
};

// Head sizes and cache type the kernel is built for.
bool step_kernel_supports(uint32_t hd, uint32_t n_head, uint32_t n_kv, int kv_f32);
// Most splits per KV head the kernel will use on the current device (sizes StepArgs::part).
uint32_t step_kernel_smax(uint32_t n_kv);
// Bytes of one PH_ARGMAX record times the CTAs of the kernel.
size_t step_kernel_amax_bytes();
// One cooperative launch of n_steps steps (the launcher clears the arrival counter on the stream). kset: the matrix kinds of
// the program's GEMVs: 0 Q4_0 only, 1 Q4_K / Q6_K only, 2 any.
int step_kernel_launch(const StepArgs &a, uint32_t hd, int kset, cudaStream_t st);

}  // namespace ieb
