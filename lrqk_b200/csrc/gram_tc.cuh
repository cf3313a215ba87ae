// Interface of the tensor-core Gram pass (gram_tc.cu) towards the prompt factorisation.
#pragma once

#include "common.cuh"

namespace lrqk {

struct GramTcArgs {
  const void *Q, *K;           // bf16 [B,Hq,S,128], [B,Hkv,S,128]
  const float *A_Q0, *A_K0;    // fp32 [B,Hq,S,r]; rounded to bf16 on the way into the tensor core
  float *part;                 // [2][B*Hq][splits][Wp*Wp] partial Gram blocks, Wp = pad16(r + 128)
  int32_t *status;             // device word, set to LRQK_ETIMEOUT if a bounded wait ran out
  int64_t seq_len;
  int32_t bsz, q_heads, kv_heads, head_dim, r, splits, rows_per_split;
};

// Prompt rows per pipeline stage; rows_per_split must be a multiple of it.
int gram_tc_tile_rows();
// LRQK_OK, or LRQK_EUNSUPPORTED when the shape or the alignment of the operands rules the path out.
int launch_gram_tc(const GramTcArgs &a, cudaStream_t stream);

}  // namespace lrqk
