// Argument block of the whole-step decode kernel (mega.cu), shared with the decode stack that launches it.
#pragma once

#include "gemv_common.cuh"

#define MG_MAX_SPLITS 18

struct MegaLayer {
  const void *qkv, *o, *gate, *up, *down, *ln1, *ln2;
  void *k_cache, *v_cache;
};

struct MegaArgs {
  const MegaLayer* layers;  // device array [L]
  const void *embed, *final_norm, *lm_head, *cos_t, *sin_t;
  long long* state;         // {step, tokens in cache, cache position, position id, token}
  int32_t* seq_len32;
  long long* out_tokens;
  int out_capacity;
  void *h, *qkv_out, *t, *logits;
  float* attn_part;         // [Hq][MG_MAX_SPLITS][128 + 2]
  float* argmax_val;        // [grid]
  int* argmax_idx;          // [grid]
  unsigned long long* bar;  // [0] grid-barrier arrival counter (monotonic), [1] completed megakernel steps
  int L, H, I, Hq, Hkv, V, max_seq, embed_vocab;
  int x_elems;              // capacity of the staged activation vector (elements)
  float eps, scale_log2;
  unsigned long long* trace;
  unsigned long long* op_trace;  // optional [2 * op_trace_cap]: {tag, %globaltimer} stamps of CTA 0 at phase boundaries
  int op_trace_cap;
};

size_t mui_mega_smem_bytes(int x_elems, int Hq);
int mui_mega_x_elems(int H, int I, int Hq, int Hkv);
mui_status_t mui_launch_mega_step(cudaStream_t stream, mui_dtype_t dtype, const MegaArgs& args, int G_ratio, int grid,
                                  int pdl);
