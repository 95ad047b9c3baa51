// Stage 2: the alpha (forward) and beta (backward) recursions over each
// utterance's T x (U+1) lattice.
//
// Replaces ComputeAlpha / ComputeAlphaOneSymPerFrame
// (optimized_transducer/csrc/kernels.cu:200-313) and ComputeBeta /
// ComputeBetaOneSymPerFrame (kernels.cu:415-519); the recursions themselves are
// those of optimized_transducer/csrc/cpu.cc:162-451.
//
// One CTA per (utterance, direction): 2N CTAs, alpha and beta of an utterance
// run concurrently.  Thread u owns lattice column u and keeps the wavefront in
// registers: its own previous value is the t-neighbour, the u-neighbour comes
// from the adjacent lane by a warp shuffle and across warps through two
// shared-memory words per warp and one named barrier per step.  The log-probs
// a step needs do not depend on the recursion, so they are loaded kPrefetch
// steps ahead into a register ring.  Alpha and beta are written to global
// memory as a side effect (the gradient stage needs them), never read back.
//
//   standard transducer : anti-diagonal wavefront, T+U-1 steps
//   one symbol per frame: both predecessors lie in the previous frame, so the
//                         sweep is frame-synchronous, T-1 steps
//
// Lattices wider than 1024 columns use the generic kernel at the end of the
// file (several columns per thread, wavefront kept in global memory).
#include "ot_common.cuh"

namespace otb {

namespace {

constexpr int kPrefetch = 8;
constexpr int kMaxWarps = 32;

// Barrier over the first `nthreads` threads of the CTA (the warps that own a
// lattice column); warps beyond them have already returned.
__device__ __forceinline__ void bar_active(int nthreads) {
  asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}

// Hands `own` of column u to column u+1 (DOWN == false) or to column u-1
// (DOWN == true) and returns what this thread receives.
template <typename T, bool DOWN>
__device__ __forceinline__ T neighbour(T own, T (*xchg)[kMaxWarps], int step,
                                       int lane, int warp, int nwarps) {
  T got = DOWN ? __shfl_down_sync(kFull, own, 1) : __shfl_up_sync(kFull, own, 1);
  if (nwarps > 1) {
    const int edge_out = DOWN ? 0 : kWarp - 1;
    const int edge_in = DOWN ? kWarp - 1 : 0;
    if (lane == edge_out) xchg[step & 1][warp] = own;
    bar_active(nwarps * kWarp);
    const int src = DOWN ? warp + 1 : warp - 1;
    if (lane == edge_in && src >= 0 && src < nwarps) got = xchg[step & 1][src];
  }
  return got;
}

template <typename T, bool FAST, bool MODIFIED>
__global__ void __launch_bounds__(1024)
lattice_kernel(const T *__restrict__ lp, const int32_t *__restrict__ Tl,
               const int32_t *__restrict__ Ul, const int64_t *__restrict__ split,
               const int32_t *__restrict__ status, T *__restrict__ alpha,
               T *__restrict__ beta, T *__restrict__ scores,
               T *__restrict__ scores_beta) {
  __shared__ T xchg[2][kMaxWarps];
  if (status[kStatusCode] != 0) return;
  const int b = blockIdx.x >> 1;
  const bool backward = blockIdx.x & 1;
  const int Tn = Tl[b], U = Ul[b], U1 = U + 1;
  const int u = threadIdx.x, lane = u & 31, warp = u >> 5;
  const int nwarps = (U1 + kWarp - 1) / kWarp;
  if (warp >= nwarps) return;
  const int64_t off = split[b];
  const T *lpb = lp + 2 * off;
  const bool col = u < U1;  // this thread owns a lattice column
  const int diff = Tn - 1 - U;

  if (!backward) {
    // ------------------------------ alpha ------------------------------
    T *al = alpha + off;
    T own = 0;
    if (u == 0) al[0] = 0;
    int xs = 0;  // exchange counter: selects the shared-memory buffer
    T left = neighbour<T, false>(own, xchg, xs++, lane, warp, nwarps);
    const int first = 1;
    const int last = MODIFIED ? Tn - 1 : Tn - 1 + U;
    // Step s computes cell (t, u) with t = s (modified) or t = s - u (standard).
    auto fetch = [&](int s, T &vb, T &vs) {
      vb = 0; vs = 0;
      const int t = MODIFIED ? s : s - u;
      const int tmin = MODIFIED ? 1 : 0;
      if (!col || t < tmin || t >= Tn) return;
      if (MODIFIED) {
        if (u > t || t - u > diff) return;
        if (t > u) vb = lpb[2 * ((int64_t)(t - 1) * U1 + u)];
        if (u >= 1) vs = lpb[2 * ((int64_t)(t - 1) * U1 + u - 1) + 1];
      } else {
        if (t >= 1) vb = lpb[2 * ((int64_t)(t - 1) * U1 + u)];
        if (u >= 1) vs = lpb[2 * ((int64_t)t * U1 + u - 1) + 1];
      }
    };
    T pb[kPrefetch], ps[kPrefetch];
#pragma unroll
    for (int k = 0; k < kPrefetch; ++k) fetch(first + k, pb[k], ps[k]);
    for (int s0 = first; s0 <= last; s0 += kPrefetch) {
#pragma unroll
      for (int k = 0; k < kPrefetch; ++k) {
        const int s = s0 + k;
        if (s > last) break;
        const T lb = pb[k], ls = ps[k];
        fetch(s + kPrefetch, pb[k], ps[k]);
        const int t = MODIFIED ? s : s - u;
        bool active = col && t >= 0 && t < Tn;
        if (MODIFIED) active = active && u <= t && t - u <= diff;
        if (active) {
          T nv;
          if (u == 0) nv = own + lb;
          else if (MODIFIED ? (t == u) : (t == 0)) nv = left + ls;
          else nv = log_add<T, FAST>(own + lb, left + ls);
          al[(int64_t)t * U1 + u] = nv;
          own = nv;
        }
        left = neighbour<T, false>(own, xchg, xs++, lane, warp, nwarps);
      }
    }
    if (u == U) scores[b] = own + lpb[2 * ((int64_t)(Tn - 1) * U1 + U)];
  } else {
    // ------------------------------- beta ------------------------------
    T *be = beta + off;
    T own = 0;
    if (u == U) {
      own = lpb[2 * ((int64_t)(Tn - 1) * U1 + U)];
      be[(int64_t)(Tn - 1) * U1 + U] = own;
    }
    int xs = 0;
    T right = neighbour<T, true>(own, xchg, xs++, lane, warp, nwarps);
    const int first = MODIFIED ? Tn - 2 : Tn - 2 + U;  // counts down to 0
    auto fetch = [&](int s, T &vb, T &vs) {
      vb = 0; vs = 0;
      const int t = MODIFIED ? s : s - u;
      if (!col || s < 0 || t < 0 || t >= Tn) return;
      if (MODIFIED && (u > t || t - u > diff)) return;
      const T *q = lpb + 2 * ((int64_t)t * U1 + u);
      if constexpr (sizeof(T) == 4) {
        const float2 v = *reinterpret_cast<const float2 *>(q);
        vb = v.x; vs = v.y;
      } else {
        const double2 v = *reinterpret_cast<const double2 *>(q);
        vb = v.x; vs = v.y;
      }
    };
    T pb[kPrefetch], ps[kPrefetch];
#pragma unroll
    for (int k = 0; k < kPrefetch; ++k) fetch(first - k, pb[k], ps[k]);
    for (int s0 = first; s0 >= 0; s0 -= kPrefetch) {
#pragma unroll
      for (int k = 0; k < kPrefetch; ++k) {
        const int s = s0 - k;
        if (s < 0) break;
        const T lb = pb[k], ls = ps[k];
        fetch(s - kPrefetch, pb[k], ps[k]);
        const int t = MODIFIED ? s : s - u;
        bool active = col && t >= 0 && t < Tn;
        if (MODIFIED) active = active && u <= t && t - u <= diff;
        if (active) {
          T nv;
          if (u == U) nv = own + lb;
          else if (MODIFIED ? (t - u == diff) : (t == Tn - 1)) nv = right + ls;
          else nv = log_add<T, FAST>(own + lb, right + ls);
          be[(int64_t)t * U1 + u] = nv;
          own = nv;
        }
        right = neighbour<T, true>(own, xchg, xs++, lane, warp, nwarps);
      }
    }
    if (u == 0) scores_beta[b] = own;
  }
}

// Generic fallback for lattices with more than 1024 columns: thread i owns the
// columns i, i+blockDim, ...; the wavefront lives in the alpha/beta arrays in
// global memory and one CTA barrier separates consecutive steps.
template <typename T, bool MODIFIED>
__global__ void __launch_bounds__(1024)
lattice_generic_kernel(const T *__restrict__ lp, const int32_t *__restrict__ Tl,
                       const int32_t *__restrict__ Ul,
                       const int64_t *__restrict__ split,
                       const int32_t *__restrict__ status, T *alpha, T *beta,
                       T *__restrict__ scores, T *__restrict__ scores_beta) {
  if (status[kStatusCode] != 0) return;
  const int b = blockIdx.x >> 1;
  const bool backward = blockIdx.x & 1;
  const int Tn = Tl[b], U = Ul[b], U1 = U + 1;
  const int64_t off = split[b];
  const T *lpb = lp + 2 * off;
  const int diff = Tn - 1 - U;
  auto LPB = [&](int t, int u) { return lpb[2 * ((int64_t)t * U1 + u)]; };
  auto LPS = [&](int t, int u) { return lpb[2 * ((int64_t)t * U1 + u) + 1]; };
  if (!backward) {
    T *al = alpha + off;
    if (threadIdx.x == 0) al[0] = 0;
    __syncthreads();
    const int last = MODIFIED ? Tn - 1 : Tn - 1 + U;
    for (int s = 1; s <= last; ++s) {
      for (int u = threadIdx.x; u < U1; u += blockDim.x) {
        const int t = MODIFIED ? s : s - u;
        if (t < 0 || t >= Tn) continue;
        if (MODIFIED) {
          if (u > t || t - u > diff) continue;
          T nv;
          if (u == 0) nv = al[(int64_t)(t - 1) * U1] + LPB(t - 1, 0);
          else if (t == u) nv = al[(int64_t)(t - 1) * U1 + u - 1] + LPS(t - 1, u - 1);
          else nv = log_add<T, false>(al[(int64_t)(t - 1) * U1 + u] + LPB(t - 1, u),
                                      al[(int64_t)(t - 1) * U1 + u - 1] + LPS(t - 1, u - 1));
          al[(int64_t)t * U1 + u] = nv;
        } else {
          T nv;
          if (u == 0) nv = al[(int64_t)(t - 1) * U1] + LPB(t - 1, 0);
          else if (t == 0) nv = al[u - 1] + LPS(0, u - 1);
          else nv = log_add<T, false>(al[(int64_t)(t - 1) * U1 + u] + LPB(t - 1, u),
                                      al[(int64_t)t * U1 + u - 1] + LPS(t, u - 1));
          al[(int64_t)t * U1 + u] = nv;
        }
      }
      __syncthreads();
    }
    if (threadIdx.x == 0) scores[b] = al[(int64_t)(Tn - 1) * U1 + U] + LPB(Tn - 1, U);
  } else {
    T *be = beta + off;
    if (threadIdx.x == 0) be[(int64_t)(Tn - 1) * U1 + U] = LPB(Tn - 1, U);
    __syncthreads();
    const int first = MODIFIED ? Tn - 2 : Tn - 2 + U;
    for (int s = first; s >= 0; --s) {
      for (int u = threadIdx.x; u < U1; u += blockDim.x) {
        const int t = MODIFIED ? s : s - u;
        if (t < 0 || t >= Tn) continue;
        T nv;
        if (MODIFIED) {
          if (u > t || t - u > diff) continue;
          if (u == U) nv = be[(int64_t)(t + 1) * U1 + U] + LPB(t, U);
          else if (t - u == diff) nv = be[(int64_t)(t + 1) * U1 + u + 1] + LPS(t, u);
          else nv = log_add<T, false>(be[(int64_t)(t + 1) * U1 + u] + LPB(t, u),
                                      be[(int64_t)(t + 1) * U1 + u + 1] + LPS(t, u));
        } else {
          if (u == U) nv = be[(int64_t)(t + 1) * U1 + U] + LPB(t, U);
          else if (t == Tn - 1) nv = be[(int64_t)t * U1 + u + 1] + LPS(t, u);
          else nv = log_add<T, false>(be[(int64_t)(t + 1) * U1 + u] + LPB(t, u),
                                      be[(int64_t)t * U1 + u + 1] + LPS(t, u));
        }
        be[(int64_t)t * U1 + u] = nv;
      }
      __syncthreads();
    }
    if (threadIdx.x == 0) scores_beta[b] = be[0];
  }
}

template <typename T>
cudaError_t launch_lattice_t(const Problem &p, void *scores, cudaStream_t s) {
  const int32_t *status = reinterpret_cast<const int32_t *>(p.ws + p.lay.status);
  const int64_t *split = reinterpret_cast<const int64_t *>(p.ws + p.lay.split);
  const T *lp = reinterpret_cast<const T *>(p.ws + p.lay.lp);
  T *alpha = reinterpret_cast<T *>(p.ws + p.lay.alpha);
  T *beta = reinterpret_cast<T *>(p.ws + p.lay.beta);
  T *sb = reinterpret_cast<T *>(p.ws + p.lay.scores_beta);
  T *sa = static_cast<T *>(scores);
  const bool modified = p.flags & OT_B200_ONE_SYM_PER_FRAME;
  const bool fast = p.flags & OT_B200_FAST_MATH;
  const unsigned grid = 2u * (unsigned)p.N;
  const int cols = p.max_u + 1;
  if (cols > 1024) {
    if (modified) lattice_generic_kernel<T, true><<<grid, 1024, 0, s>>>(lp, p.T, p.U, split, status, alpha, beta, sa, sb);
    else lattice_generic_kernel<T, false><<<grid, 1024, 0, s>>>(lp, p.T, p.U, split, status, alpha, beta, sa, sb);
    return cudaGetLastError();
  }
  const unsigned block = (unsigned)((cols + kWarp - 1) / kWarp * kWarp);
#define OTB_LAT(F, M) lattice_kernel<T, F, M><<<grid, block, 0, s>>>(lp, p.T, p.U, split, status, alpha, beta, sa, sb)
  if (fast) { if (modified) OTB_LAT(true, true); else OTB_LAT(true, false); }
  else      { if (modified) OTB_LAT(false, true); else OTB_LAT(false, false); }
#undef OTB_LAT
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_lattice(const Problem &p, void *scores, cudaStream_t s) {
  return (p.flags & OT_B200_FP64) ? launch_lattice_t<double>(p, scores, s)
                                  : launch_lattice_t<float>(p, scores, s);
}

}  // namespace otb
