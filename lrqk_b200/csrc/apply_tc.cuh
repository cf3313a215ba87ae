// Interface of the tensor-core apply pass (apply_tc.cu) towards the prompt factorisation.
#pragma once

#include "common.cuh"

namespace lrqk {

struct ApplyTcArgs {
  const void *K;        // bf16 [B,Hkv,S,128]
  void *A_K;            // bf16 [B,Hq,a_capacity,r]: rows [0,S) are written
  const float *ws;      // factorisation workspace; the per-sweep results start at sweep_base (floats)
  int32_t *status;      // device word, set to LRQK_ETIMEOUT if a bounded wait ran out
  int64_t seq_len, a_capacity, sweep_base;
  int32_t sweep_stride, sweeps, bsz, q_heads, kv_heads, head_dim, r;
  float tol;
};

// LRQK_OK, or LRQK_EUNSUPPORTED when the shape or the alignment of the operands rules the path out.
int launch_apply_tc(const ApplyTcArgs &a, cudaStream_t stream);

}  // namespace lrqk
