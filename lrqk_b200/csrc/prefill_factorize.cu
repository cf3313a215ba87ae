// Prompt factorisation (placeholder while the kernels are brought up: entry points reject).
#include "common.cuh"

extern "C" size_t lrqk_prefill_factorize_workspace_bytes(const lrqk_layer *L, int64_t seq_len) {
  (void)L; (void)seq_len;
  return 0;
}

extern "C" int lrqk_prefill_factorize(const lrqk_layer *L, const void *Q, const void *K, float *A_Q, float *A_K_init,
                                      int64_t seq_len, int32_t sweeps, float tol, void *a_q_last, int32_t *sweeps_out,
                                      void *workspace, lrqk_stream_t stream) {
  (void)L; (void)Q; (void)K; (void)A_Q; (void)A_K_init; (void)seq_len; (void)sweeps; (void)tol; (void)a_q_last;
  (void)sweeps_out; (void)workspace; (void)stream;
  return LRQK_EUNSUPPORTED;
}
