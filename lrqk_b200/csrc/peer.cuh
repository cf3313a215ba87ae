// Layout of the exchange buffer shared by the attention epilogue and the wait kernel.
#pragma once

#include "common.cuh"

namespace lrqk {

// Bytes of the data part: two halves of [world][heads_per_rank][d] elements, each half rounded
// up to 256 bytes so that the flags behind them stay aligned.
inline size_t peer_data_bytes(int world, int heads_per_rank, int head_dim, int dtype) {
  const size_t half = ((size_t)world * heads_per_rank * head_dim * elt_size(dtype) + 255) / 256 * 256;
  return 2 * half;
}

int check_peer_group(const lrqk_peer_group *g);

// What the attention epilogue needs to push its rows (passed by value to the kernel).
struct PushTargets {
  char *data[LRQK_MAX_PEERS];      // start of half (seq & 1), slot `rank`, on every peer
  int32_t *flag[LRQK_MAX_PEERS];   // arrival word [seq & 1][rank] on every peer
  int32_t *local_counter;
  int32_t world, heads, seq;
};

}  // namespace lrqk
