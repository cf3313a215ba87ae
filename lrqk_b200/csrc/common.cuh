// Shared device/host helpers of liblrqk_sm100.so (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "lrqk_sm100.h"

namespace lrqk {

constexpr int kNumSMs = 148;  // B200: two dies of 74 SMs

// ---- host side -------------------------------------------------------------------------
void note_cuda_error(cudaError_t e);
void note_error_text(const char *text);  // free-form detail, returned by lrqk_last_cuda_error()

#define LRQK_CUDA_TRY(expr)                      \
  do {                                           \
    cudaError_t _e = (expr);                     \
    if (_e != cudaSuccess) {                     \
      ::lrqk::note_cuda_error(_e);               \
      return LRQK_ELAUNCH;                       \
    }                                            \
  } while (0)

#define LRQK_LAUNCH_CHECK() LRQK_CUDA_TRY(cudaGetLastError())

int check_device();              // LRQK_OK or LRQK_ENODEVICE
int check_layer(const lrqk_layer *L);

inline cudaStream_t as_stream(lrqk_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }
inline size_t elt_size(int dtype) { return dtype == LRQK_BF16 ? 2 : 4; }
inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- device side -----------------------------------------------------------------------
// Order-preserving map float -> uint32 (larger float <=> larger key); -0 folds onto +0.
__device__ __forceinline__ uint32_t order_key(float f) {
  if (f == 0.0f) f = 0.0f;
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <typename T> struct Elt;
template <> struct Elt<float> {
  static constexpr int kPerVec = 4;  // elements per 16-byte vector
  __device__ static __forceinline__ void unpack(const uint4 &v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  __device__ static __forceinline__ float to_float(float x) { return x; }
  __device__ static __forceinline__ float from_float(float x) { return x; }
};
template <> struct Elt<__nv_bfloat16> {
  static constexpr int kPerVec = 8;
  __device__ static __forceinline__ void unpack(const uint4 &v, float (&f)[8]) {
    // bf16 -> fp32 is a 16-bit shift
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xFFFF0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xFFFF0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xFFFF0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xFFFF0000u);
  }
  __device__ static __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ static __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};

// Streaming 16-byte load that bypasses L1 allocation.  (The L2 evict-first qualifier exists
// only for 32-byte loads on sm_100; the scoring kernel uses those where a row allows.)
__device__ __forceinline__ uint4 ld_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld16(const void *p) { return *reinterpret_cast<const uint4 *>(p); }
__device__ __forceinline__ void st16(void *p, const uint4 &v) { *reinterpret_cast<uint4 *>(p) = v; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

// ---- bulk asynchronous copies completing on an mbarrier -----------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

constexpr uint32_t kMbarWaitLimit = 1u << 22;  // polls of an mbarrier before a wait gives up

__device__ __forceinline__ void mbarrier_init(uint64_t *bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals));
}
__device__ __forceinline__ void mbarrier_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// Wait for the phase with the given parity; false if the poll limit ran out (the caller records it
// and carries on with whatever the buffer holds, so that no CTA is left waiting).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity) {
  const uint32_t a = smem_addr(bar);
  for (uint32_t i = 0; i < kMbarWaitLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(a), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}

// One thread: expect `bytes` on the barrier and start the copy global -> shared (both 16-byte aligned,
// bytes a multiple of 16).
__device__ __forceinline__ void bulk_load(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_addr(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}

// ---- one-time function attributes, per device ---------------------------------------------------
// cudaFuncSetAttribute applies to the device that is current when it is called, so what has been set
// is remembered per device (a process may drive several GPUs, one after another or from several threads).
constexpr int kMaxDevices = 64;
struct SmemOptIn {
  size_t set[kMaxDevices] = {};
  template <typename K>
  cudaError_t ensure(K kernel, size_t bytes) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (bytes <= set[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) set[dev] = bytes;
    return e;
  }
};

// ---- programmatic dependent launch -------------------------------------------------------------
// The kernels of a decode step depend on one another in stream order.  Each is launched with the
// programmatic-stream-serialization attribute, calls pdl_launch_dependents() first thing and
// pdl_wait() before it touches global memory: the next kernel's CTAs are then placed, and run
// their set-up (shared-memory clears, barrier initialisation), while the previous kernel is still
// finishing, and block in pdl_wait() until that kernel has completed and its writes are visible.
// Launched without the attribute both calls do nothing, so the same kernels serve the
// stage-by-stage entry points.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// cudaLaunchKernelEx with the programmatic attribute and, if cluster_x > 1, a cluster dimension.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    int cluster_x, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[n].val.programmaticStreamSerializationAllowed = 1;
  ++n;
  if (cluster_x > 0) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = (unsigned)cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// lrqk_score_topk with one extra duty for the fused step: *clear_word = 0 (the miss-list length the
// next kernel appends to), which saves a memset node between two dependent kernels.
// With `diff`, the kernel also runs the hit/miss difference of every head against L->table right
// after its selection (what lrqk_slot_diff does as a kernel of its own); *diff->list_len must be
// zero before the kernel starts.
struct UpdateArgs;  // update_head.cuh
struct FusedDiff {
  uint8_t *mask;
  int32_t *miss_count;
  lrqk_miss *list;
  int32_t *list_len, *status;
};
// `workspace` (optional, lrqk_score_topk_workspace_bytes): room for the keys of the two-kernel plan.
// `update` (optional): the deferred update of project_update_enqueue -- the kernel derives q_hat from the
// projection's workspace itself and one CTA per head applies the update while the hit/miss difference runs.
// score_topk_can_fold_update() says whether that is possible for the plan these arguments get.
int score_topk_enqueue(const lrqk_layer *L, const void *q_hat, int64_t candidates, int32_t *wanted, float *scores_out,
                       int64_t scores_stride, int32_t *clear_word, cudaStream_t stream, const FusedDiff *diff = nullptr,
                       void *workspace = nullptr, size_t workspace_bytes = 0, const UpdateArgs *update = nullptr);
bool score_topk_can_fold_update(const lrqk_layer *L, int64_t candidates, void *workspace, size_t workspace_bytes);
int plan_score_topk(const lrqk_layer *L, int64_t candidates, int n_heads, int *csize_out, int *seg_len_out);

// lrqk_decode_project_update with extra duties for the fused step: *clear_word = 0 at the end, and --
// when v_new is given -- the ring write of the step's key/value into lite slot `lite_slot` (position
// append_row), so that no separate ring-write kernel is needed unless the ring is flushed.
// With `deferred`, only the projection kernel is launched: the arguments of the update (early-exit decision,
// rank-1 step on B_Q / B_K, q_hat, the new A_K row) are handed back for the scoring kernel to apply.
int project_update_enqueue(const lrqk_layer *L, const void *q, const void *k_new, int32_t max_iter, float tol,
                           int64_t append_row, void *q_hat, int32_t *iters_out, void *workspace, int32_t *clear_word,
                           cudaStream_t stream, const void *v_new, int32_t lite_slot, UpdateArgs *deferred = nullptr,
                           bool update_only = false);
// The flush half of lrqk_lite_append alone: the ring of every KV head to host rows [host_row, host_row + m).
int lite_flush_enqueue(const lrqk_layer *L, int64_t host_row, cudaStream_t stream);

// Dispatch on the element type of a layer.
#define LRQK_DISPATCH_DTYPE(dtype, T, ...)                       \
  do {                                                           \
    if ((dtype) == LRQK_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else if ((dtype) == LRQK_F32) { using T = float; __VA_ARGS__; }     \
    else return LRQK_EUNSUPPORTED;                               \
  } while (0)

}  // namespace lrqk
