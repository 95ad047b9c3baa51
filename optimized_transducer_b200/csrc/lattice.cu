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
// shared-memory words per warp and one named barrier per step.
//
//   standard transducer : anti-diagonal wavefront, T+U-1 steps
//   one symbol per frame: both predecessors lie in the previous frame, so the
//                         sweep is frame-synchronous, T-1 steps
//
// The per-cell arrays (lp in, alpha/beta out) are stored in wavefront order
// (see cell_pos in ot_common.cuh): at every step the threads of a warp read and
// write consecutive addresses, and the address of a thread advances by U+1
// entries per step.  The log-probs do not depend on the recursion, so they are
// loaded kPrefetch steps ahead into a register ring.  Alpha and beta are
// written as a side effect (the gradient stage needs them), never read back.
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
// (DOWN == true) and returns what this thread receives.  `xs` counts the
// exchanges and selects one of two shared-memory buffers, so a warp that runs
// ahead cannot overwrite a word a slower warp has not read yet.
template <typename T, bool DOWN>
__device__ __forceinline__ T neighbour(T own, T (*xchg)[kMaxWarps], int xs,
                                       int lane, int warp, int nwarps) {
  T got = DOWN ? __shfl_down_sync(kFull, own, 1) : __shfl_up_sync(kFull, own, 1);
  if (nwarps > 1) {
    const int edge_out = DOWN ? 0 : kWarp - 1;
    const int edge_in = DOWN ? kWarp - 1 : 0;
    if (lane == edge_out) xchg[xs & 1][warp] = own;
    bar_active(nwarps * kWarp);
    const int src = DOWN ? warp + 1 : warp - 1;
    if (lane == edge_in && src >= 0 && src < nwarps) got = xchg[xs & 1][src];
  }
  return got;
}

template <typename T> struct Pair;
template <> struct Pair<float> { using type = float2; };
template <> struct Pair<double> { using type = double2; };

template <typename T, bool FAST, bool MODIFIED>
__global__ void __launch_bounds__(1024)
lattice_kernel(const T *__restrict__ lp, const int32_t *__restrict__ Tl,
               const int32_t *__restrict__ Ul, const int64_t *__restrict__ cell_split,
               const int32_t *__restrict__ status, T *__restrict__ alpha,
               T *__restrict__ beta, T *__restrict__ scores,
               T *__restrict__ scores_beta) {
  __shared__ T xchg[2][kMaxWarps];
  if (status[kStatusCode] != 0) return;
  using P = typename Pair<T>::type;
  const int b = blockIdx.x >> 1;
  const bool backward = blockIdx.x & 1;
  const int Tn = Tl[b], U = Ul[b], U1 = U + 1;
  const int u = threadIdx.x, lane = u & 31, warp = u >> 5;
  const int nwarps = (U1 + kWarp - 1) / kWarp;
  if (warp >= nwarps) return;
  const int64_t off = cell_split[b];
  const P *lp2 = reinterpret_cast<const P *>(lp) + off;
  const bool col = u < U1;  // this thread owns a lattice column
  const int diff = Tn - 1 - U;
  // Steps (first..last) during which this thread computes a cell, and the
  // lattice row t of its first step.  Standard: step s is diagonal s, t = s - u.
  // Modified: step s is frame s, the band is u <= t <= u + diff.
  int s_lo, s_hi;
  if (MODIFIED) { s_lo = u; s_hi = u + diff; }
  else { s_lo = u; s_hi = u + Tn - 1; }
  if (!col) { s_lo = 1 << 30; s_hi = -1; }
  int xs = 0;

  if (!backward) {
    // ------------------------------ alpha ------------------------------
    // cell (step s, column u) lives at entry s*U1 + u in both layouts.
    T *al = alpha + off;
    T own = 0;
    if (u == 0) al[0] = 0;
    T left = neighbour<T, false>(own, xchg, xs++, lane, warp, nwarps);
    const int last = MODIFIED ? Tn - 1 : Tn - 1 + U;
    // What step s needs sits in the previous wavefront row: the blank log-prob
    // of this column, (s-1)*U1 + u, and the symbol log-prob of column u-1.
    // Standard: blank(t-1,u), sym(t,u-1).  Modified: blank(t-1,u), sym(t-1,u-1).
    auto fetch = [&](int s, T &vb, T &vs) {
      vb = 0; vs = 0;
      if (s <= s_lo || s > s_hi) {          // not active, or the first cell of the column
        if (s != s_lo || u == 0) return;    // ... which still needs the symbol term
      }
      const T *q = reinterpret_cast<const T *>(lp2 + ((int64_t)(s - 1) * U1 + u));
      if (s > s_lo) vb = q[0];
      if (u >= 1) vs = q[-1];
    };
    T pb[kPrefetch], ps[kPrefetch];
#pragma unroll
    for (int k = 0; k < kPrefetch; ++k) fetch(1 + k, pb[k], ps[k]);
    T *st = al + (int64_t)U1 + u;  // entry of step 1
    for (int s0 = 1; s0 <= last; s0 += kPrefetch) {
#pragma unroll
      for (int k = 0; k < kPrefetch; ++k) {
        const int s = s0 + k;
        if (s > last) break;
        const T lb = pb[k], ls = ps[k];
        fetch(s + kPrefetch, pb[k], ps[k]);
        if (s >= s_lo && s <= s_hi && s > 0) {
          T nv;
          if (u == 0) nv = own + lb;                 // only the blank predecessor
          else if (s == s_lo) nv = left + ls;        // only the symbol predecessor
          else nv = log_add<T, FAST>(own + lb, left + ls);
          *st = nv;
          own = nv;
        }
        st += U1;
        left = neighbour<T, false>(own, xchg, xs++, lane, warp, nwarps);
      }
    }
    if (u == U) {
      const int64_t fin = cell_pos<MODIFIED>(Tn - 1, U, U1);
      scores[b] = own + reinterpret_cast<const T *>(lp2 + fin)[0];
    }
  } else {
    // ------------------------------- beta ------------------------------
    // Runs the steps backwards; step s needs (blank, symbol) of its own cell.
    T *be = beta + off;
    T own = 0;
    const int top = MODIFIED ? Tn - 1 : Tn - 1 + U;  // step of the final cell (T-1, U)
    if (u == U) {
      own = reinterpret_cast<const T *>(lp2 + ((int64_t)top * U1 + U))[0];
      be[(int64_t)top * U1 + U] = own;
    }
    T right = neighbour<T, true>(own, xchg, xs++, lane, warp, nwarps);
    // The final cell is done; column U therefore stops one step earlier.
    const int hi = (u == U) ? s_hi - 1 : s_hi;
    auto fetch = [&](int s, T &vb, T &vs) {
      vb = 0; vs = 0;
      if (s < s_lo || s > hi) return;
      const P v = lp2[(int64_t)s * U1 + u];
      vb = v.x; vs = v.y;
    };
    const int first = top - 1;
    T pb[kPrefetch], ps[kPrefetch];
#pragma unroll
    for (int k = 0; k < kPrefetch; ++k) fetch(first - k, pb[k], ps[k]);
    T *st = be + ((int64_t)first * U1 + u);
    for (int s0 = first; s0 >= 0; s0 -= kPrefetch) {
#pragma unroll
      for (int k = 0; k < kPrefetch; ++k) {
        const int s = s0 - k;
        if (s < 0) break;
        const T lb = pb[k], ls = ps[k];
        fetch(s - kPrefetch, pb[k], ps[k]);
        if (s >= s_lo && s <= hi) {
          T nv;
          if (u == U) nv = own + lb;               // only the blank successor
          else if (s == s_hi) nv = right + ls;     // last row / band edge: only the symbol successor
          else nv = log_add<T, FAST>(own + lb, right + ls);
          *st = nv;
          own = nv;
        }
        st -= U1;
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
                       const int64_t *__restrict__ cell_split,
                       const int32_t *__restrict__ status, T *alpha, T *beta,
                       T *__restrict__ scores, T *__restrict__ scores_beta) {
  if (status[kStatusCode] != 0) return;
  const int b = blockIdx.x >> 1;
  const bool backward = blockIdx.x & 1;
  const int Tn = Tl[b], U = Ul[b], U1 = U + 1;
  const int64_t off = cell_split[b];
  const T *lpb = lp + 2 * off;
  const int diff = Tn - 1 - U;
  auto C = [&](int t, int u) { return cell_pos<MODIFIED>(t, u, U1); };
  auto LPB = [&](int t, int u) { return lpb[2 * C(t, u)]; };
  auto LPS = [&](int t, int u) { return lpb[2 * C(t, u) + 1]; };
  if (!backward) {
    T *al = alpha + off;
    if (threadIdx.x == 0) al[0] = 0;
    __syncthreads();
    const int last = MODIFIED ? Tn - 1 : Tn - 1 + U;
    for (int s = 1; s <= last; ++s) {
      for (int u = threadIdx.x; u < U1; u += blockDim.x) {
        const int t = MODIFIED ? s : s - u;
        if (t < 0 || t >= Tn) continue;
        T nv;
        if (MODIFIED) {
          if (u > t || t - u > diff) continue;
          if (u == 0) nv = al[C(t - 1, 0)] + LPB(t - 1, 0);
          else if (t == u) nv = al[C(t - 1, u - 1)] + LPS(t - 1, u - 1);
          else nv = log_add<T, false>(al[C(t - 1, u)] + LPB(t - 1, u),
                                      al[C(t - 1, u - 1)] + LPS(t - 1, u - 1));
        } else {
          if (u == 0) nv = al[C(t - 1, 0)] + LPB(t - 1, 0);
          else if (t == 0) nv = al[C(0, u - 1)] + LPS(0, u - 1);
          else nv = log_add<T, false>(al[C(t - 1, u)] + LPB(t - 1, u),
                                      al[C(t, u - 1)] + LPS(t, u - 1));
        }
        al[C(t, u)] = nv;
      }
      __syncthreads();
    }
    if (threadIdx.x == 0) scores[b] = al[C(Tn - 1, U)] + LPB(Tn - 1, U);
  } else {
    T *be = beta + off;
    if (threadIdx.x == 0) be[C(Tn - 1, U)] = LPB(Tn - 1, U);
    __syncthreads();
    const int first = MODIFIED ? Tn - 2 : Tn - 2 + U;
    for (int s = first; s >= 0; --s) {
      for (int u = threadIdx.x; u < U1; u += blockDim.x) {
        const int t = MODIFIED ? s : s - u;
        if (t < 0 || t >= Tn) continue;
        T nv;
        if (MODIFIED) {
          if (u > t || t - u > diff) continue;
          if (u == U) nv = be[C(t + 1, U)] + LPB(t, U);
          else if (t - u == diff) nv = be[C(t + 1, u + 1)] + LPS(t, u);
          else nv = log_add<T, false>(be[C(t + 1, u)] + LPB(t, u),
                                      be[C(t + 1, u + 1)] + LPS(t, u));
        } else {
          if (u == U) nv = be[C(t + 1, U)] + LPB(t, U);
          else if (t == Tn - 1) nv = be[C(t, u + 1)] + LPS(t, u);
          else nv = log_add<T, false>(be[C(t + 1, u)] + LPB(t, u),
                                      be[C(t, u + 1)] + LPS(t, u));
        }
        be[C(t, u)] = nv;
      }
      __syncthreads();
    }
    if (threadIdx.x == 0) scores_beta[b] = be[0];
  }
}

template <typename T>
cudaError_t launch_lattice_t(const Problem &p, void *scores, cudaStream_t s) {
  const int32_t *status = reinterpret_cast<const int32_t *>(p.ws + p.lay.status);
  const int64_t *csplit = reinterpret_cast<const int64_t *>(p.ws + p.lay.cell_split);
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
    if (modified) lattice_generic_kernel<T, true><<<grid, 1024, 0, s>>>(lp, p.T, p.U, csplit, status, alpha, beta, sa, sb);
    else lattice_generic_kernel<T, false><<<grid, 1024, 0, s>>>(lp, p.T, p.U, csplit, status, alpha, beta, sa, sb);
    return cudaGetLastError();
  }
  const unsigned block = (unsigned)((cols + kWarp - 1) / kWarp * kWarp);
#define OTB_LAT(F, M) lattice_kernel<T, F, M><<<grid, block, 0, s>>>(lp, p.T, p.U, csplit, status, alpha, beta, sa, sb)
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
