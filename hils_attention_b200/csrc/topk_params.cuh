// Arguments of the chunk-selection kernels (topk.cu, topk_tc.cu).
#pragma once
#include <stdint.h>

namespace hils {

struct TopkParams {
  const void* q; const void* lmks; const void* lse_swa; const float* bias; const float* gumbel;
  const int32_t* drop_mask; int32_t* indices; void* scores; float* lse_total; float* rank_keys;
  int B, L, N, h_kv, G, D, topk, block_size, window_size, is_causal, q_offset, per_qhead, lse_dtype;
  int RW;
  float scale;
  float* dots;   // decode, bf16: raw q.k' of every candidate, written by the streaming kernel (or null)
  // decode kernels only: the inter-chunk softmax of the step fused behind the selection.  weights (B, L, h_kv*G, K+1(+1))
  // in the element type, or null: softmax over [scores + bias of the selected chunks, lse_swa(, 0 when softmax1)]
  void* weights; int softmax1;
  const int32_t* q_offsets;   // decode kernels only: position of query row 0 of each batch entry (null: q_offset for all)
};

}  // namespace hils
