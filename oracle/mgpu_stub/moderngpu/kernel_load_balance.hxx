// Stand-in for moderngpu's load_balance_search (see context.hxx in this
// directory for why it exists).  TEST INFRASTRUCTURE ONLY.
//
// Published behaviour: given `num_segments` ascending segment starts
// (segments[0] == 0) and `count` work items, write for every item i the index
// of the segment that contains it: the largest s with segments[s] <= i.  The
// reference calls it with the row splits of the batch to get the row ids
// (optimized_transducer/csrc/cuda.cu:40-59).  One thread per item, binary search.
#pragma once

#include "moderngpu/context.hxx"

namespace mgpu {

template <typename segments_it, typename output_it>
__global__ void load_balance_search_kernel(int count, segments_it segments, int num_segments,
                                           output_it out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  int lo = 0, hi = num_segments;  // segments[lo] <= i < segments[hi] (hi == num_segments: the end)
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (segments[mid] <= i) lo = mid; else hi = mid;
  }
  out[i] = lo;
}

template <typename segments_it, typename output_it>
void load_balance_search(int count, segments_it segments, int num_segments, output_it out,
                         context_t &context) {
  if (count <= 0) return;
  const int threads = 256;
  load_balance_search_kernel<<<(count + threads - 1) / threads, threads, 0, context.stream()>>>(
      count, segments, num_segments, out);
}

}  // namespace mgpu
