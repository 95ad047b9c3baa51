// Stand-in for the part of the third-party "moderngpu" library that the
// reference's CUDA build touches.  TEST INFRASTRUCTURE ONLY.
//
// The reference pins moderngpu at commit 2b3985541c8e88a133769598c406c33ddde9d0a5
// (cmake/moderngpu.cmake:24-25 of the reference) and downloads it at configure
// time; it is not part of the reference tree and not available offline.  The
// reference uses exactly two things of it (optimized_transducer/csrc/cuda.cu:56,
// optimized_transducer/csrc/moderngpu-allocator.h:18-39): the context base
// class with virtual alloc/free hooks, and load_balance_search, which has no
// arithmetic in it (it turns row splits into row ids).  This header and
// kernel_load_balance.hxx restate those two interfaces from their published
// behaviour so that the reference's own CUDA sources (cuda.cu, kernels.cu)
// compile unmodified; nothing here is taken from moderngpu's source.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

namespace mgpu {

enum memory_space_t { memory_space_device = 0, memory_space_host = 1 };

// A CUDA stream plus allocation hooks; the reference derives its
// torch-allocator-backed context from this.
class standard_context_t {
 public:
  standard_context_t(bool /*print_prop*/, cudaStream_t stream) : stream_(stream) {}
  virtual ~standard_context_t() {}
  virtual void *alloc(size_t size, memory_space_t space) {
    void *p = nullptr;
    if (space == memory_space_device) cudaMalloc(&p, size); else cudaMallocHost(&p, size);
    return p;
  }
  virtual void free(void *p, memory_space_t space) {
    if (space == memory_space_device) cudaFree(p); else cudaFreeHost(p);
  }
  cudaStream_t stream() const { return stream_; }

 private:
  cudaStream_t stream_;
};

typedef standard_context_t context_t;

}  // namespace mgpu
