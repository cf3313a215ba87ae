// Exchange buffers for the attention outputs of head-sharded ranks: allocation, CUDA IPC
// mapping, and the bounded wait for a push to arrive.  The push itself is the epilogue of the
// attention kernel (flash_decode.cu).
#include <string.h>

#include "common.cuh"
#include "peer.cuh"

namespace lrqk {
namespace {

uint32_t g_peer_wait_polls = 1u << 22;  // polls (with a short sleep each) before a wait gives up

struct WaitParams {
  const int32_t *flags;   // this rank's arrival words
  const uint4 *data;      // this rank's data half for `seq`
  uint4 *out;
  int32_t *status;
  int32_t world, seq, vecs;  // vecs: 16-byte pieces of one half
  uint32_t polls;
};

__global__ void __launch_bounds__(256) allgather_wait_kernel(WaitParams p) {
  __shared__ int ok;
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < p.world) {
    const int32_t *f = p.flags + (p.seq & 1) * p.world + threadIdx.x;
    bool arrived = false;
    for (uint32_t i = 0; i < p.polls; ++i) {
      int32_t v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if (v >= p.seq) { arrived = true; break; }
      __nanosleep(64);
    }
    if (!arrived) {
      ok = 0;
      atomicExch(p.status, (int32_t)LRQK_ETIMEOUT);
    }
  }
  __syncthreads();
  if (!p.out) return;
  if (!ok) {
    // the rows did not arrive: hand out NaNs (all-ones bit patterns in either dtype) rather than leave the
    // previous step's rows in place, so that a caller that does not look at the status word cannot miss it
    for (int i = threadIdx.x; i < p.vecs; i += blockDim.x) p.out[i] = make_uint4(~0u, ~0u, ~0u, ~0u);
    return;
  }
  for (int i = threadIdx.x; i < p.vecs; i += blockDim.x) p.out[i] = p.data[i];
}

}  // namespace

int check_peer_group(const lrqk_peer_group *g) {
  if (!g) return LRQK_EINVAL;
  if (g->world < 1 || g->world > LRQK_MAX_PEERS || g->rank < 0 || g->rank >= g->world) return LRQK_EINVAL;
  if (g->heads_per_rank <= 0 || !g->local_counter) return LRQK_EINVAL;
  if (g->dtype != LRQK_F32 && g->dtype != LRQK_BF16) return LRQK_EUNSUPPORTED;
  if (g->head_dim != 64 && g->head_dim != 128) return LRQK_EUNSUPPORTED;
  for (int i = 0; i < g->world; ++i)
    if (!g->base[i]) return LRQK_EINVAL;
  return LRQK_OK;
}

}  // namespace lrqk

extern "C" size_t lrqk_peer_buffer_bytes(int32_t world, int32_t heads_per_rank, int32_t head_dim, int32_t dtype) {
  if (world < 1 || heads_per_rank < 1 || head_dim < 1) return 0;
  return lrqk::peer_data_bytes(world, heads_per_rank, head_dim, dtype) + 2 * (size_t)world * sizeof(int32_t);
}

extern "C" int lrqk_peer_buffer_create(size_t bytes, void **dev_ptr, unsigned char handle[64]) {
  using namespace lrqk;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C ABI carries IPC handles as 64 bytes");
  if (!dev_ptr || !handle || bytes == 0) return LRQK_EINVAL;
  const int rc = check_device();
  if (rc != LRQK_OK) return rc;
  void *ptr = nullptr;
  LRQK_CUDA_TRY(cudaMalloc(&ptr, bytes));
  cudaError_t e = cudaMemset(ptr, 0, bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) {
    note_cuda_error(e);
    cudaFree(ptr);
    return LRQK_ELAUNCH;
  }
  memcpy(handle, &h, 64);
  *dev_ptr = ptr;
  return LRQK_OK;
}

extern "C" int lrqk_peer_buffer_open(const unsigned char handle[64], void **dev_ptr) {
  using namespace lrqk;
  if (!handle || !dev_ptr) return LRQK_EINVAL;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  LRQK_CUDA_TRY(cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return LRQK_OK;
}

extern "C" int lrqk_peer_buffer_close(void *dev_ptr) {
  if (!dev_ptr) return LRQK_OK;
  LRQK_CUDA_TRY(cudaIpcCloseMemHandle(dev_ptr));
  return LRQK_OK;
}

extern "C" int lrqk_peer_buffer_destroy(void *dev_ptr) {
  if (!dev_ptr) return LRQK_OK;
  LRQK_CUDA_TRY(cudaFree(dev_ptr));
  return LRQK_OK;
}

extern "C" int lrqk_peer_set_wait_polls(uint32_t polls) {
  if (polls == 0) return LRQK_EINVAL;
  lrqk::g_peer_wait_polls = polls;
  return LRQK_OK;
}

extern "C" int lrqk_allgather_wait(const lrqk_peer_group *g, int32_t seq, void *gathered_out, int32_t *status,
                                   lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  rc = check_peer_group(g);
  if (rc != LRQK_OK) return rc;
  if (seq < 1 || !status) return LRQK_EINVAL;
  const size_t half = peer_data_bytes(g->world, g->heads_per_rank, g->head_dim, g->dtype) / 2;
  WaitParams p;
  char *mine = reinterpret_cast<char *>(g->base[g->rank]);
  p.flags = reinterpret_cast<const int32_t *>(mine + 2 * half);
  p.data = reinterpret_cast<const uint4 *>(mine + (size_t)(seq & 1) * half);
  p.out = reinterpret_cast<uint4 *>(gathered_out);
  p.status = status;
  p.world = g->world;
  p.seq = seq;
  p.vecs = (int32_t)(half / 16);
  p.polls = g_peer_wait_polls;
  LRQK_CUDA_TRY(launch_dependent(allgather_wait_kernel, dim3(1), dim3(256), 0, as_stream(stream), 0, p));
  return LRQK_OK;
}
