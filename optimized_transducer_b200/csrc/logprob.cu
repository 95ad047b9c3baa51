// Stage 1: row-wise logsumexp of the packed logits fused with the gather of the
// blank and next-symbol log-probabilities.
//
// Replaces `logits.logsumexp(1)` (optimized_transducer/csrc/cuda.cu:427) and
// ComputeLogProbs (optimized_transducer/csrc/kernels.cu:30-60), and, for
// log-softmax input, ComputeLogProbsForLogSoftmax (kernels.cu:62-88).
//
// One warp owns a row at a time.  The row is read once with 16-byte coalesced
// loads (all loads of a chunk are issued before the first use), reduced with an
// online (max, sum) pair per lane and merged across the warp with shuffles;
// the two gathered entries are re-read from the lines just fetched.  HBM
// traffic: V*sizeof(T) bytes read and 3*sizeof(T) bytes written per row.
#include "ot_common.cuh"

namespace otb {

namespace {

constexpr int kThreads = 256;

template <typename T, int VEC> struct VecOf;
template <> struct VecOf<float, 4> { using type = float4; };
template <> struct VecOf<float, 1> { using type = float; };
template <> struct VecOf<double, 2> { using type = double2; };
template <> struct VecOf<double, 1> { using type = double; };

// T: element type.  VEC: elements per load (16 bytes, or 1 element when the
// row stride or the base pointer is not 16-byte aligned).  CH: loads per lane
// per chunk, i.e. a chunk covers 32*VEC*CH elements of the row.
template <typename T, int VEC, int CH, bool MODIFIED>
__global__ void __launch_bounds__(kThreads)
logprob_kernel(const T *__restrict__ logits, const int32_t *__restrict__ targets,
               const int32_t *__restrict__ Tl, const int32_t *__restrict__ Ul,
               const int64_t *__restrict__ split,
               const int32_t *__restrict__ status, int N, int64_t rows, int V,
               int max_u, int blank, T *__restrict__ den, T *__restrict__ lp) {
  if (status[kStatusCode] != 0) return;
  using VT = typename VecOf<T, VEC>::type;
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const int nvec = V / VEC;
  const T ninf = neg_inf<T>();

  for (int64_t row = warp0; row < rows; row += nwarps) {
    const T *p = logits + row * (int64_t)V;
    const int b = find_utt(split, N, row);
    const int U = __ldg(Ul + b), U1 = U + 1;
    const int idx = (int)(row - __ldg(split + b));
    const int t = idx / U1, u = idx - t * U1;
    if (MODIFIED) {
      // Cells outside the band u <= t <= u + (T-1-U) are never used
      // (optimized_transducer/csrc/cpu.cc:295): skip their rows entirely.
      const int diff = __ldg(Tl + b) - 1 - U;
      if (u > t || t - u > diff) continue;
    }
    T m = ninf, s = 0;
    for (int base = 0; base < nvec; base += kWarp * CH) {
      T x[CH][VEC];
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int vi = base + j * kWarp + lane;
        if (vi < nvec) {
          const VT v = *reinterpret_cast<const VT *>(p + (int64_t)vi * VEC);
          const T *e = reinterpret_cast<const T *>(&v);
#pragma unroll
          for (int k = 0; k < VEC; ++k) x[j][k] = e[k];
        } else {
#pragma unroll
          for (int k = 0; k < VEC; ++k) x[j][k] = ninf;
        }
      }
      T cm = ninf;
#pragma unroll
      for (int j = 0; j < CH; ++j)
#pragma unroll
        for (int k = 0; k < VEC; ++k) cm = r_max(cm, x[j][k]);
      if (cm > m) { s *= r_exp(m - cm); m = cm; }  // m == -inf: s is 0, stays 0
      if (m > ninf) {
#pragma unroll
        for (int j = 0; j < CH; ++j)
#pragma unroll
          for (int k = 0; k < VEC; ++k) s += r_exp(x[j][k] - m);
      }
    }
    const T M = warp_max(m);
    // Follows ATen's logsumexp: an infinite maximum is replaced by 0 before
    // the subtraction, which makes the result that same infinity.
    T d;
    if (M - M == (T)0) {
      const T part = (m > ninf) ? s * r_exp(m - M) : (T)0;
      d = r_log(warp_sum(part)) + M;
    } else {
      d = M;
    }
    // Gather: lane 0 fetches the blank entry, lane 1 the symbol entry.
    T g = 0;
    if (lane == 0) g = p[blank] - d;
    if (lane == 1 && u < U) g = p[__ldg(targets + (int64_t)b * max_u + u)] - d;
    const T g1 = __shfl_sync(kFull, g, 1);
    if (lane == 0) {
      den[row] = d;
      T *q = lp + 2 * row;
      q[0] = g;
      q[1] = g1;
    }
  }
}

// Log-softmax input: nothing to reduce, only the gather (thread per row).
template <typename T>
__global__ void __launch_bounds__(kThreads)
gather_kernel(const T *__restrict__ logp, const int32_t *__restrict__ targets,
              const int32_t *__restrict__ Ul, const int64_t *__restrict__ split,
              const int32_t *__restrict__ status, int N, int64_t rows, int V,
              int max_u, int blank, T *__restrict__ lp) {
  if (status[kStatusCode] != 0) return;
  const int64_t row = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (row >= rows) return;
  const int b = find_utt(split, N, row);
  const int U = __ldg(Ul + b), U1 = U + 1;
  const int u = (int)((row - __ldg(split + b)) % U1);
  const T *p = logp + row * (int64_t)V;
  lp[2 * row] = p[blank];
  lp[2 * row + 1] = (u < U) ? p[__ldg(targets + (int64_t)b * max_u + u)] : (T)0;
}

template <typename T, int VEC, int CH>
cudaError_t launch_lse(const Problem &p, cudaStream_t s) {
  const int32_t *status = reinterpret_cast<const int32_t *>(p.ws + p.lay.status);
  const int64_t *split = reinterpret_cast<const int64_t *>(p.ws + p.lay.split);
  T *den = reinterpret_cast<T *>(p.ws + p.lay.den);
  T *lp = reinterpret_cast<T *>(p.ws + p.lay.lp);
  const T *x = static_cast<const T *>(p.logits);
  // Persistent grid: a multiple of the SM count, never more warps than rows.
  const int64_t want = (p.rows + (kThreads / kWarp) - 1) / (kThreads / kWarp);
  const int64_t cap = (int64_t)sm_count() * 8;
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  if (p.flags & OT_B200_ONE_SYM_PER_FRAME)
    logprob_kernel<T, VEC, CH, true><<<grid, kThreads, 0, s>>>(
        x, p.targets, p.T, p.U, split, status, p.N, p.rows, p.V, p.max_u, p.blank, den, lp);
  else
    logprob_kernel<T, VEC, CH, false><<<grid, kThreads, 0, s>>>(
        x, p.targets, p.T, p.U, split, status, p.N, p.rows, p.V, p.max_u, p.blank, den, lp);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_logprob_t(const Problem &p, cudaStream_t s) {
  if (p.flags & OT_B200_FROM_LOG_SOFTMAX) {
    const unsigned grid = (unsigned)((p.rows + kThreads - 1) / kThreads);
    gather_kernel<T><<<grid, kThreads, 0, s>>>(
        static_cast<const T *>(p.logits), p.targets, p.U,
        reinterpret_cast<const int64_t *>(p.ws + p.lay.split),
        reinterpret_cast<const int32_t *>(p.ws + p.lay.status), p.N, p.rows, p.V,
        p.max_u, p.blank, reinterpret_cast<T *>(p.ws + p.lay.lp));
    return cudaGetLastError();
  }
  constexpr int VEC = Vec16<T>::n;
  const bool vec_ok = (p.V % VEC == 0) &&
                      (reinterpret_cast<uintptr_t>(p.logits) % 16 == 0);
  if (vec_ok) {
    const int per_lane = (p.V / VEC + kWarp - 1) / kWarp;  // 16-byte loads per lane
    if (per_lane <= 1) return launch_lse<T, VEC, 1>(p, s);
    if (per_lane <= 2) return launch_lse<T, VEC, 2>(p, s);
    if (per_lane <= 4) return launch_lse<T, VEC, 4>(p, s);
    return launch_lse<T, VEC, 8>(p, s);
  }
  const int per_lane = (p.V + kWarp - 1) / kWarp;
  if (per_lane <= 4) return launch_lse<T, 1, 4>(p, s);
  return launch_lse<T, 1, 16>(p, s);
}

}  // namespace

cudaError_t launch_logprob(const Problem &p, cudaStream_t s) {
  return (p.flags & OT_B200_FP64) ? launch_logprob_t<double>(p, s)
                                  : launch_logprob_t<float>(p, s);
}

}  // namespace otb
