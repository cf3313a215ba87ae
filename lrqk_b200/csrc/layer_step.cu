// One decode step of a layer as a single host call: the kernels of the step are enqueued
// back to back on the caller's stream, with no host synchronisation in between (the miss
// count, the early-exit decision and the slot-table update all stay on the device).
#include "common.cuh"
#include "update_head.cuh"

extern "C" int lrqk_layer_step(const lrqk_layer *L, const lrqk_step_args *a, lrqk_stream_t stream) {
  using namespace lrqk;
  if (!L || !a) return LRQK_EINVAL;
  if (!a->q || !a->k_new || !a->v_new || !a->q_hat || !a->wanted || !a->mask || !a->miss_count || !a->miss_list ||
      !a->counters || !a->project_workspace)
    return LRQK_EINVAL;
  if ((a->attn_out || a->peers) && !a->attn_workspace) return LRQK_EINVAL;
  // The ring write is done by the projection kernel (its solver CTAs store the step's key/value, the
  // streaming CTAs take that row from k_new); a ring-write kernel only runs on the steps that flush
  // the ring to the host store.  The miss-list length is cleared by the projection's second kernel,
  // the hit/miss difference runs as the tail of the scoring kernel, the miss fetch inside the attention kernel.
  if (a->lite_slot < 0 || a->lite_slot >= L->m) return LRQK_ECAPACITY;
  if (a->flush_rows != 0 && a->flush_rows != L->m) return LRQK_EINVAL;
  // Where the scoring stage is one kernel, that kernel also applies the projection's update (early-exit
  // decision, rank-1 step on B_Q / B_K, q_hat, the new A_K row): four launches per step instead of five.
  UpdateArgs deferred;
  const bool fold = score_topk_can_fold_update(L, a->candidates, a->score_workspace, a->score_workspace_bytes);
  int rc = project_update_enqueue(L, a->q, a->k_new, a->max_iter, a->tol, a->position, a->q_hat, a->counters + 2,
                                  a->project_workspace, a->counters, as_stream(stream), a->v_new, a->lite_slot,
                                  fold ? &deferred : nullptr);
  if (rc != LRQK_OK) return rc;
  if (a->flush_rows) {
    rc = lite_flush_enqueue(L, a->host_row, as_stream(stream));
    if (rc != LRQK_OK) return rc;
  }
  FusedDiff diff;
  diff.mask = a->mask; diff.miss_count = a->miss_count; diff.list = a->miss_list;
  diff.list_len = a->counters; diff.status = a->counters + 1;
  rc = score_topk_enqueue(L, a->q_hat, a->candidates, a->wanted, nullptr, 0, nullptr, as_stream(stream), &diff,
                          a->score_workspace, a->score_workspace_bytes, fold ? &deferred : nullptr);
  if (rc != LRQK_OK) return rc;
  if (!a->peers && !a->attn_out)  // no attention asked for: only refill the missed slots
    return lrqk_miss_gather(L, a->miss_list, a->counters, stream);
  // the attention kernel fetches the missed rows itself
  rc = lrqk_fetch_attend(L, a->mask, a->q, a->attn_out, a->scale, a->attn_workspace, a->peers, a->push_seq, stream);
  if (rc != LRQK_OK) return rc;
  if (a->peers && a->wait_status)  // ... and the wait for every rank's rows of this push, in the same call
    rc = lrqk_allgather_wait(a->peers, a->push_seq, a->gathered_out, a->wait_status, stream);
  return rc;
}

// How many kernels lrqk_layer_step enqueues for these arguments (for launch accounting).
extern "C" int lrqk_layer_step_launches(const lrqk_layer *L, const lrqk_step_args *a) {
  using namespace lrqk;
  if (!L || !a) return LRQK_EINVAL;
  const bool fold = score_topk_can_fold_update(L, a->candidates, a->score_workspace, a->score_workspace_bytes);
  int n = 1 /* projection */ + (fold ? 0 : 1) /* update */ + 1 /* scoring + difference */ + (fold ? 0 : 1) /* key pass */ +
          1 /* miss fetch, with the attention when the step ends in one */;
  if (a->flush_rows) n += 1;
  if (a->peers && a->wait_status) n += 1;
  return n;
}
