// Library-level entry points: version, error text, device check, page-locked host memory.
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>

#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace lrqk {

static thread_local char g_last_cuda_error[256] = "";
static std::mutex g_host_mutex;
static std::unordered_map<void *, std::pair<void *, size_t>> g_host_maps;  // registered mappings: address -> (mmap base, length)

void note_cuda_error(cudaError_t e) {
  const char *name = cudaGetErrorName(e);
  const char *text = cudaGetErrorString(e);
  snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: %s", name ? name : "?", text ? text : "?");
  cudaGetLastError();  // clear the sticky-free error so later launches are judged on their own
}

void note_error_text(const char *text) { snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s", text); }

int check_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return LRQK_ENODEVICE; }
  static int cached_dev = -2, cached_ok = 0;
  if (dev != cached_dev) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
      cudaGetLastError();
      return LRQK_ENODEVICE;
    }
    cached_ok = (major == 10);
    cached_dev = dev;
  }
  return cached_ok ? LRQK_OK : LRQK_ENODEVICE;
}

int check_layer(const lrqk_layer *L) {
  if (!L) return LRQK_EINVAL;
  if (L->dtype != LRQK_F32 && L->dtype != LRQK_BF16) return LRQK_EUNSUPPORTED;
  if (L->bsz <= 0 || L->q_heads <= 0 || L->kv_heads <= 0 || L->head_dim <= 0) return LRQK_EINVAL;
  if (L->q_heads % L->kv_heads != 0) return LRQK_EINVAL;
  if (L->r <= 0 || L->k <= 0 || L->m <= 0) return LRQK_EINVAL;
  if (L->a_capacity <= 0 || L->host_capacity < 0) return LRQK_EINVAL;
  if (L->head_dim != 64 && L->head_dim != 128) return LRQK_EUNSUPPORTED;
  if (L->r != 8 && L->r != 16 && L->r != 32 && L->r != 64) return LRQK_EUNSUPPORTED;
  if ((int64_t)L->bsz * L->q_heads * (int64_t)L->k >= (1ll << 31)) return LRQK_EUNSUPPORTED;
  if (L->a_capacity >= (1ll << 31)) return LRQK_EUNSUPPORTED;
  for (int i = 0; i < 4; ++i)
    if (!(L->weights[i] >= 0.0f) || L->weights[i] > 3.0e38f) return LRQK_EINVAL;  // negative, NaN or infinite
  return LRQK_OK;
}

}  // namespace lrqk

extern "C" {

const char *lrqk_version(void) { return "lrqk_sm100 0.2.0 (sm_100a)"; }

const char *lrqk_strerror(int code) {
  switch (code) {
    case LRQK_OK: return "ok";
    case LRQK_EINVAL: return "invalid argument";
    case LRQK_ECAPACITY: return "index or length exceeds the given capacity";
    case LRQK_EUNSUPPORTED: return "shape or dtype not supported by the sm_100a kernels";
    case LRQK_ELAUNCH: return "CUDA runtime error (see lrqk_last_cuda_error)";
    case LRQK_ETIMEOUT: return "bounded device-side wait ran out";
    case LRQK_ENODEVICE: return "no sm_100 CUDA device is current (there is no CPU fallback)";
    case LRQK_ENOMEM: return "host allocation failed";
    default: return "unknown lrqk error code";
  }
}

const char *lrqk_last_cuda_error(void) { return lrqk::g_last_cuda_error; }

int lrqk_device_supported(void) { return lrqk::check_device() == LRQK_OK ? 1 : 0; }

// Page-locked host memory.  cudaHostAlloc spends ~0.4 ms per MiB faulting in and pinning 4 KiB pages
// (0.22 s for the 540 MB store of one layer at a 128K context).  Anonymous memory that asks for
// transparent huge pages, is touched by a few threads and is then registered with the driver is
// ready three times sooner, comes zero-filled from the kernel, and behaves the same afterwards
// (portable, mapped into the device address space).  cudaHostAlloc remains the fallback.
int lrqk_host_alloc(void **host_ptr, size_t bytes) {
  if (!host_ptr || bytes == 0) return LRQK_EINVAL;
  *host_ptr = nullptr;
  const size_t huge = (size_t)2 << 20;
  const size_t span = bytes + huge;
  void *base = mmap(nullptr, span, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
  if (base != MAP_FAILED) {
    char *aligned = reinterpret_cast<char *>((reinterpret_cast<uintptr_t>(base) + huge - 1) & ~(uintptr_t)(huge - 1));
    madvise(aligned, bytes, MADV_HUGEPAGE);  // best effort
    const int n_thr = bytes >= ((size_t)64 << 20) ? 4 : 1;
    std::vector<std::thread> workers;
    for (int t = 0; t < n_thr; ++t) {
      workers.emplace_back([=]() {
        const size_t lo = bytes / n_thr * t, hi = t == n_thr - 1 ? bytes : bytes / n_thr * (t + 1);
        for (size_t i = lo & ~(size_t)4095; i < hi; i += 4096) reinterpret_cast<volatile char *>(aligned)[i] = 0;
      });
    }
    for (auto &w : workers) w.join();
    const cudaError_t e = cudaHostRegister(aligned, bytes, cudaHostRegisterMapped | cudaHostRegisterPortable);
    if (e == cudaSuccess) {
      std::lock_guard<std::mutex> lock(lrqk::g_host_mutex);
      lrqk::g_host_maps[aligned] = {base, span};
      *host_ptr = aligned;
      return LRQK_OK;
    }
    cudaGetLastError();
    munmap(base, span);
  }
  cudaError_t e = cudaHostAlloc(host_ptr, bytes, cudaHostAllocMapped | cudaHostAllocPortable);
  if (e != cudaSuccess) {
    lrqk::note_cuda_error(e);
    return e == cudaErrorMemoryAllocation ? LRQK_ENOMEM : LRQK_ELAUNCH;
  }
  memset(*host_ptr, 0, bytes);  // same contract as the mapped path: zero-filled
  return LRQK_OK;
}

int lrqk_host_free(void *host_ptr) {
  if (!host_ptr) return LRQK_OK;
  std::pair<void *, size_t> m{nullptr, 0};
  {
    std::lock_guard<std::mutex> lock(lrqk::g_host_mutex);
    auto it = lrqk::g_host_maps.find(host_ptr);
    if (it != lrqk::g_host_maps.end()) {
      m = it->second;
      lrqk::g_host_maps.erase(it);
    }
  }
  if (m.first) {
    LRQK_CUDA_TRY(cudaHostUnregister(host_ptr));
    munmap(m.first, m.second);
    return LRQK_OK;
  }
  LRQK_CUDA_TRY(cudaFreeHost(host_ptr));
  return LRQK_OK;
}

int lrqk_host_device_ptr(void *host_ptr, void **device_ptr) {
  if (!host_ptr || !device_ptr) return LRQK_EINVAL;
  LRQK_CUDA_TRY(cudaHostGetDevicePointer(device_ptr, host_ptr, 0));
  return LRQK_OK;
}

}  // extern "C"
