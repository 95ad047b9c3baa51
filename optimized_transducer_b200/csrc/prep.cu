// Stage 0 (input check + row/cell splits) and the reduction of the scores to
// the loss.
//
// Stage 0 replaces, without a host round trip, the data-dependent checks of
// ot::ComputeTransducerLoss (optimized_transducer/csrc/transducer-loss.cc:49-66)
// and the row_splits construction of ot::ComputeTransducerLossCuda
// (optimized_transducer/csrc/cuda.cu:411-414).  The reference's row_ids array
// (cuda.cu:40-59, moderngpu load_balance_search) has no counterpart: later
// stages find the owning utterance with a binary search over the splits, or
// walk their rows in order.
#include "ot_common.cuh"

namespace otb {

namespace {

constexpr int kPrepThreads = 512;

__device__ __forceinline__ void raise(int32_t *status, int code, int index) {
  if (atomicCAS(status + kStatusCode, 0, code) == 0) status[kStatusIndex] = index;
}

// Block-wide exclusive prefix sum of one value per thread; `total` gets the sum.
__device__ __forceinline__ long long block_exclusive_scan(long long mine, long long *smem,
                                                          long long *total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  long long incl = mine;
#pragma unroll
  for (int o = 1; o < kWarp; o <<= 1) {
    const long long v = __shfl_up_sync(kFull, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == kWarp - 1) smem[warp] = incl;
  __syncthreads();
  long long base = 0, tot = 0;
  for (int w = 0; w < kPrepThreads / kWarp; ++w) {
    if (w < warp) base += smem[w];
    tot += smem[w];
  }
  __syncthreads();
  *total = tot;
  return base + incl - mine;
}

// One CTA.  Thread i owns the contiguous utterance range [i*per, (i+1)*per).
__global__ void __launch_bounds__(kPrepThreads)
prepare_kernel(const int32_t *__restrict__ targets, const int32_t *__restrict__ Tl,
               const int32_t *__restrict__ Ul, int N, int64_t rows, int V,
               int max_u, int modified, int64_t max_cells,
               int32_t *__restrict__ status, int64_t *__restrict__ split,
               int64_t *__restrict__ cell_split) {
  __shared__ long long scan_buf[kPrepThreads / kWarp];
  __shared__ int warp_maxu[kPrepThreads / kWarp];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < kStatusWords) status[tid] = 0;
  __syncthreads();

  const int per = (N + kPrepThreads - 1) / kPrepThreads;
  const int b0 = min(tid * per, N), b1 = min(b0 + per, N);
  long long my_rows = 0, my_cells = 0;
  int my_maxu = -1;
  for (int b = b0; b < b1; ++b) {
    const int t = Tl[b], u = Ul[b];
    if (t <= 0) raise(status, OT_B200_INPUT_BAD_LOGIT_LENGTH, b);
    if (u < 0 || u > max_u) raise(status, OT_B200_INPUT_BAD_TARGET_LENGTH, b);
    if (modified && u > t - 1) raise(status, OT_B200_INPUT_ONE_SYM_INFEASIBLE, b);
    const int tc = max(t, 0), uc = min(max(u, 0), max_u);
    my_rows += (long long)tc * (uc + 1);
    my_cells += cell_block(tc, uc, modified != 0);
    my_maxu = max(my_maxu, u);
  }
  long long total_rows, total_cells;
  long long run_rows = block_exclusive_scan(my_rows, scan_buf, &total_rows);
  long long run_cells = block_exclusive_scan(my_cells, scan_buf, &total_cells);
  int wmax = my_maxu;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) wmax = max(wmax, __shfl_xor_sync(kFull, wmax, o));
  if (lane == 0) warp_maxu[warp] = wmax;
  __syncthreads();
  for (int b = b0; b < b1; ++b) {
    split[b] = run_rows;
    cell_split[b] = run_cells;
    const int tc = max(Tl[b], 0), uc = min(max(Ul[b], 0), max_u);
    run_rows += (long long)tc * (uc + 1);
    run_cells += cell_block(tc, uc, modified != 0);
  }
  if (tid == 0) {
    int maxu_all = -1;
    for (int w = 0; w < kPrepThreads / kWarp; ++w) maxu_all = max(maxu_all, warp_maxu[w]);
    split[N] = total_rows;
    cell_split[N] = total_cells;
    if (total_rows != rows) raise(status, OT_B200_INPUT_ROWS_MISMATCH, 0);
    if (maxu_all != max_u) raise(status, OT_B200_INPUT_MAX_U_MISMATCH, 0);
    // Cannot happen for consistent inputs (the host sizes the workspace from
    // rows, N and max_u); guards the per-cell arrays against inconsistent ones.
    if (total_cells > max_cells) raise(status, OT_B200_INPUT_ROWS_MISMATCH, 0);
  }
  // targets.max() < V over the whole (N, max_u) array, as the reference
  // checks it; in addition the entries that are used must not be negative.
  const long long cells = (long long)N * max_u;
  for (long long i = tid; i < cells; i += kPrepThreads) {
    const int v = targets[i];
    const int b = (int)(i / max_u), u = (int)(i % max_u);
    if (v >= V || (u < Ul[b] && v < 0)) raise(status, OT_B200_INPUT_TARGET_RANGE, b);
  }
}

// One warp: *loss_out = loss_scale * -(sum_b scores[b])   (the reduction of the
// reference's Python layer, transducer_loss.py:145-152).  Lane-strided partial
// sums in double and a fixed shuffle tree: the result does not depend on timing.
template <typename T>
__global__ void __launch_bounds__(kWarp)
loss_kernel(const T *__restrict__ scores, const int32_t *__restrict__ status, int N,
            T *__restrict__ loss_out, double loss_scale) {
  if (status[kStatusCode] != 0) return;
  double acc = 0;
  for (int b = threadIdx.x; b < N; b += kWarp) acc += (double)scores[b];
  acc = warp_sum(acc);
  if (threadIdx.x == 0) *loss_out = (T)(-acc * loss_scale);
}

}  // namespace

cudaError_t launch_prepare(const Problem &p, cudaStream_t s) {
  prepare_kernel<<<1, kPrepThreads, 0, s>>>(
      p.targets, p.T, p.U, p.N, p.rows, p.V, p.max_u,
      (p.flags & OT_B200_ONE_SYM_PER_FRAME) ? 1 : 0, p.lay.max_cells,
      reinterpret_cast<int32_t *>(p.ws + p.lay.status),
      reinterpret_cast<int64_t *>(p.ws + p.lay.split),
      reinterpret_cast<int64_t *>(p.ws + p.lay.cell_split));
  return cudaGetLastError();
}

cudaError_t launch_loss(const Problem &p, const void *scores, void *loss_out,
                        double loss_scale, cudaStream_t s) {
  const int32_t *status = reinterpret_cast<const int32_t *>(p.ws + p.lay.status);
  if (p.flags & OT_B200_FP64)
    loss_kernel<double><<<1, kWarp, 0, s>>>(static_cast<const double *>(scores), status, p.N,
                                            static_cast<double *>(loss_out), loss_scale);
  else
    loss_kernel<float><<<1, kWarp, 0, s>>>(static_cast<const float *>(scores), status, p.N,
                                           static_cast<float *>(loss_out), loss_scale);
  return cudaGetLastError();
}

}  // namespace otb
