// host_call.h — helpers of the synchronous host-pointer entry points (copy in, run, copy out).
#pragma once

#include <utility>
#include <vector>

#include "ops.h"

namespace mb {

// Device buffers of one host-pointer call; everything is released when the call returns.
struct Temps {
  std::vector<std::pair<void*, size_t>> bufs;
  ~Temps() {
    for (auto& b : bufs) dev_free(b.first, b.second);
  }
  int alloc(void** p, size_t bytes, const char* tag) {
    MB_TRY(dev_alloc(p, bytes ? bytes : 4, tag));
    bufs.emplace_back(*p, bytes ? bytes : 4);
    return MIMIR_B200_OK;
  }
  int upload(const float** dev, const float* host, size_t n, const char* tag) {
    void* p;
    MB_TRY(alloc(&p, n * sizeof(float), tag));
    MB_CUDA(cudaMemcpy(p, host, n * sizeof(float), cudaMemcpyHostToDevice));
    *dev = static_cast<const float*>(p);
    return MIMIR_B200_OK;
  }
  int out(float** dev, size_t n, const char* tag) {
    void* p;
    MB_TRY(alloc(&p, n * sizeof(float), tag));
    *dev = static_cast<float*>(p);
    return MIMIR_B200_OK;
  }
};

inline int finish_download(float* host, const float* dev, size_t n) {
  MB_TRY(check_device_error_word(nullptr));
  MB_CUDA(cudaMemcpy(host, dev, n * sizeof(float), cudaMemcpyDeviceToHost));
  return MIMIR_B200_OK;
}

#define MB_REQUIRE_INIT() \
  if (!ctx().initialised) return fail(MIMIR_B200_E_NOT_INIT, "mimir_b200_init has not been called")


}  // namespace mb
