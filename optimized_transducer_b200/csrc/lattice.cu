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
// from the adjacent lane by a warp shuffle.  Across warps there are two
// kernels: lattice_skew_kernel (the default) delays each warp by one block of
// 16 steps against its neighbour, so the boundary values travel through a
// shared-memory ring and the CTA meets at one barrier per block;
// lattice_kernel keeps all warps in lockstep with one barrier per step (used
// when the skewed kernel's stages do not fit into shared memory).
//
//   standard transducer : anti-diagonal wavefront, T+U-1 steps
//   one symbol per frame: both predecessors lie in the previous frame, so the
//                         sweep is frame-synchronous, T-1 steps
//
// The kernel is latency-bound (a chain of T+U dependent log-add-exps), so
// nothing on the chain may wait for global memory.  The per-cell arrays are
// stored in wavefront order (cell_pos in ot_common.cuh): the log-probs the
// steps consume are one contiguous stream, which TMA bulk copies
// (cp.async.bulk + mbarrier, kStages chunks in flight) bring into shared memory
// ahead of the recursion; a step reads its two log-probs from shared memory,
// one step early.  Alpha and beta are written to global memory as a side effect
// (coalesced, never read back here).
//
// Lattices wider than 1024 columns use the generic kernel at the end of the
// file (several columns per thread, wavefront kept in global memory).
//
// Arithmetic of the skewed kernel (struct Num below).  The reference adds in the
// log domain: every step is max, subtract, exp, log1p, and every partial sum is
// rounded at ulp(|alpha|); that is the default here too, and it reproduces the
// reference's alpha/beta almost rounding by rounding.  OT_B200_LINEAR_DOMAIN
// (float) carries each value as m * 2^e instead (float m, int e): a step is two
// multiplies, an exponent alignment (integer subtract, clamp, shift) and one
// fused multiply-add; the exp of the two log-probs a step consumes is taken one
// step early and the log only when a value is stored.  Its rounding error is
// relative to m (2^-24), so alpha and beta land within one float rounding of the
// float64 recursion, about ten times closer than the log-domain float recursion
// (the reference's included).  It is the SLOWER of the two: the recursion is one
// warp per 32 columns issuing in order at about five cycles per instruction
// (measured: issue slots 17-21 % busy, stalls split between fixed-latency
// dependencies and the scoreboard), so the step time follows the instruction
// count, 63 per step against 35 (88 us against 56 us on four benchmark
// utterances), not the length of the dependency chain.
#include <stdlib.h>
#include <string.h>

#include "ot_common.cuh"

namespace otb {

namespace {

constexpr int kMaxWarps = 32;
constexpr int kStages = 3;
constexpr int kChunkBytes = 16384;         // target size of one staged chunk

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

// The value a column carries through the recursion.  ARITH 0: log domain with
// the reference's exact log-add; 1: log domain, ex2/lg2 approximations; 2
// (float only): scaled linear domain, value = m * 2^e.
constexpr int kArithLog = 0, kArithLogFast = 1, kArithLinear = 2;

template <typename T, int ARITH>
struct Num {
  T v;
  static __device__ __forceinline__ Num zero() { return {neg_inf<T>()}; }
  static __device__ __forceinline__ Num from_log(T x) { return {x}; }
  __device__ __forceinline__ T log() const { return v; }
  __device__ __forceinline__ Num up() const { return {__shfl_up_sync(kFull, v, 1)}; }
  __device__ __forceinline__ Num down() const { return {__shfl_down_sync(kFull, v, 1)}; }
  // a * pa + b * pb
  static __device__ __forceinline__ Num mad2(Num a, Num pa, Num b, Num pb) {
    return {log_add<T, ARITH == kArithLogFast>(a.v + pa.v, b.v + pb.v)};
  }
  static __device__ __forceinline__ Num pick(bool c, Num a, Num b) { return {c ? a.v : b.v}; }
  __device__ __forceinline__ void renorm() {}
};

template <>
struct Num<float, kArithLinear> {
  float m;  // >= 0 (or NaN: a poisoned log-prob stays visible)
  int e;
  // Exponent of a zero: far below every real exponent, so that a zero never wins
  // the alignment in mad2, and small enough that 17 of them add up inside int.
  static constexpr int kZeroExp = -(1 << 21);
  static constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: float <-> int without cvt
  static __device__ __forceinline__ Num zero() { return {0.0f, kZeroExp}; }
  // exp(x) as m * 2^e with m in [2^-0.5, 2^0.5]; -inf (no lattice cell) gives (0, kZeroExp)
  static __device__ __forceinline__ Num from_log(float x) {
    const float v = fmaxf(x * kLog2e, (float)kZeroExp);
    const float r = v + kMagic;   // the integer nearest to v sits in the low mantissa bits
    const float fl = r - kMagic;
    Num n;
    n.e = __float_as_int(r) - __float_as_int(kMagic);
    // x*log2(e) - fl with the product unrounded; log2(e) in two pieces
    float f = fmaf(x, 1.4426950216293335f, -fl);
    f = fmaf(x, 1.9259629911e-8f, f);
    n.m = ex2_approx(f);
    return n;
  }
  __device__ __forceinline__ float log() const {
    float l2;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(l2) : "f"(m));
    const float ef = __int_as_float(e + __float_as_int(kMagic)) - kMagic;  // (float)e, |e| < 2^22; any finite value for a zero
    // (l2 + e) * ln 2, ln 2 in two pieces, the large term through the fma unrounded
    return fmaf(ef, 0.693147182464599609375f, fmaf(ef, -1.904654323148236e-9f, l2 * 0.6931471805599453f));
  }
  __device__ __forceinline__ Num up() const {
    return {__shfl_up_sync(kFull, m, 1), __shfl_up_sync(kFull, e, 1)};
  }
  __device__ __forceinline__ Num down() const {
    return {__shfl_down_sync(kFull, m, 1), __shfl_down_sync(kFull, e, 1)};
  }
  static __device__ __forceinline__ Num mad2(Num a, Num pa, Num b, Num pb) {
    const float ma = a.m * pa.m, mb = b.m * pb.m;
    const int ea = a.e + pa.e, eb = b.e + pb.e;
    const int d = ea - eb;
    const int nd = max(min(d, -d), -127);                  // -|d|; 2^-127 is written as 0
    const float sc = __int_as_float((nd + 127) << 23);     // 2^nd
    const bool a_big = d >= 0;
    const float big = a_big ? ma : mb, small = a_big ? mb : ma;
    return {fmaf(small, sc, big), max(ea, eb)};
  }
  static __device__ __forceinline__ Num pick(bool c, Num a, Num b) {
    return {c ? a.m : b.m, c ? a.e : b.e};
  }
  // m back into [1, 2).  Between two calls m grows by at most 2*sqrt(2) per step
  // and shrinks by at most sqrt(2): call at least every 16 steps.
  __device__ __forceinline__ void renorm() {
    const int bits = __float_as_int(m);
    const bool finite = bits > 0 && bits < 0x7f800000;
    e = finite ? e + ((bits >> 23) - 127) : (m == 0.0f ? kZeroExp : e);
    m = finite ? __int_as_float((bits & 0x007fffff) | 0x3f800000) : m;
  }
};

// `rows_per_chunk` (even) wavefront rows are staged per bulk copy; the dynamic
// shared memory holds kStages chunks of rows_per_chunk * (max_u+1) pairs.
template <typename T, bool FAST, bool MODIFIED>
__global__ void __launch_bounds__(1024)
lattice_kernel(const T *__restrict__ lp, const int32_t *__restrict__ Tl,
               const int32_t *__restrict__ Ul, const int64_t *__restrict__ cell_split,
               int32_t *__restrict__ status, T *__restrict__ alpha,
               T *__restrict__ beta, T *__restrict__ scores,
               T *__restrict__ scores_beta, int rows_per_chunk, int stage_pairs, int group) {
  using P = typename Pair<T>::type;
  extern __shared__ __align__(128) unsigned char stage_mem[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ T xchg[2][kMaxWarps];
  pdl_wait();
  pdl_trigger();
  if (status[kStatusCode] != 0) return;
  const int b = blockIdx.x >> 1;
  {
    int lo, hi;
    group_range(status, group, (int)(gridDim.x >> 1), lo, hi);
    if (b < lo || b >= hi) return;  // an utterance of the other group
  }
  const bool backward = blockIdx.x & 1;
  const int Tn = Tl[b], U = Ul[b], U1 = U + 1;
  const int u = threadIdx.x, lane = u & 31, warp = u >> 5;
  const int nwarps = (U1 + kWarp - 1) / kWarp;
  if (warp >= nwarps) return;
  const int nact = nwarps * kWarp;
  const int64_t off = cell_split[b];
  const P *lp2 = reinterpret_cast<const P *>(lp) + off;
  // two pairs of slack in front: column 0 reads (and discards) the pair before its row
  P *stage = reinterpret_cast<P *>(stage_mem) + 2;
  const bool col = u < U1;  // this thread owns a lattice column
  const int diff = Tn - 1 - U;
  // Steps (s_lo..s_hi) during which this thread computes a cell.  Standard:
  // step s is diagonal s, t = s - u.  Modified: step s is frame s, and the band
  // is u <= t <= u + diff.  In both layouts cell (step s, column u) is entry
  // s*U1 + u of the utterance's block.
  int s_lo, s_hi;
  if (MODIFIED) { s_lo = u; s_hi = u + diff; }
  else { s_lo = u; s_hi = u + Tn - 1; }
  if (!col) { s_lo = 1 << 30; s_hi = -1; }
  const int top = MODIFIED ? Tn - 1 : Tn - 1 + U;  // step of the final cell (T-1, U)

  // Wavefront rows 0 .. top-1 are streamed: alpha's step s reads row s-1
  // (ascending), beta's step s reads row s (descending).
  const int nrows = top;
  const int R = rows_per_chunk;
  const int nchunks = (nrows + R - 1) / R;
  if (u == 0) {
    for (int i = 0; i < kStages; ++i) mbar_init(&full_bar[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (nwarps > 1) bar_active(nact); else __syncwarp();
  // Chunk j in processing order covers memory rows [row0, row0 + n).
  auto chunk_rows = [&](int j, int &row0, int &n) {
    const int m = backward ? nchunks - 1 - j : j;
    row0 = m * R;
    n = min(R, nrows - row0);
  };
  auto issue = [&](int j) {  // thread 0 only
    int row0, n;
    chunk_rows(j, row0, n);
    // whole pairs, rounded up to 16 bytes (the block is padded to an even count)
    const uint32_t bytes = (uint32_t)((((int64_t)n * U1 * sizeof(P)) + 15) & ~int64_t(15));
    uint64_t *bar = &full_bar[j % kStages];
    mbar_expect_tx(bar, bytes);
    tma_load_1d(stage + (int64_t)(j % kStages) * stage_pairs, lp2 + (int64_t)row0 * U1, bytes, bar);
  };
  if (u == 0) for (int j = 0; j < kStages && j < nchunks; ++j) issue(j);
  auto wait_chunk = [&](int j) {
    uint64_t *bar = &full_bar[j % kStages];
    const uint32_t parity = (uint32_t)((j / kStages) & 1);
    // Bounded: a copy that never lands is reported through the status word and
    // the recursion goes on with whatever the stage holds (no thread leaves the
    // barriers of the steps early, so nothing can hang).
    for (int spin = 0; spin < (1 << 22); ++spin)
      if (mbar_try_wait(bar, parity)) return;
    atomicCAS(status + kStatusCopyTimeout, 0, 1 + b);
  };
  int xs = 0;
  const T ninf = neg_inf<T>();
  const int uc = col ? u : U;  // column used for addressing (keeps idle lanes in bounds)
  // A step is branch-free: both predecessors always enter the log-add, and a
  // predecessor that does not exist contributes -inf (a column that has not
  // started holds -inf, a log-prob outside the column's step range is read as
  // -inf), for which log_add returns the other operand exactly.

  if (!backward) {
    // ------------------------------ alpha ------------------------------
    T *al = alpha + off;
    T own = (u == 0) ? (T)0 : ninf;
    if (u == 0) al[0] = 0;
    T left = neighbour<T, false>(own, xchg, xs++, lane, warp, nwarps);
    T *st = al + (int64_t)U1 + uc;  // entry of step 1
    const unsigned span = (unsigned)(s_hi - s_lo);
    for (int j = 0; j < nchunks; ++j) {
      int row0, n;
      chunk_rows(j, row0, n);
      wait_chunk(j);
      const P *rowp = stage + (int64_t)(j % kStages) * stage_pairs + uc;
      // Step s = row + 1 needs, from wavefront row `row`: the blank log-prob of
      // this column (blank(t-1,u)) if s_lo < s <= s_hi, and the symbol log-prob
      // of column u-1 (standard sym(t,u-1); modified sym(t-1,u-1)) if u >= 1
      // and s_lo <= s <= s_hi.
      auto fetch = [&](int s, const P *q, T &vb, T &vs) {
        const T x = q[0].x, y = q[-1].y;
        const unsigned rel = (unsigned)(s - s_lo);
        vb = (rel - 1u < span) ? x : ninf;
        vs = (rel <= span && u >= 1) ? y : ninf;
      };
      T nb, ns;
      fetch(row0 + 1, rowp, nb, ns);
#pragma unroll 2
      for (int i = 0; i < n; ++i) {
        const int s = row0 + 1 + i;
        const T lb = nb, ls = ns;
        rowp += U1;
        if (i + 1 < n) fetch(s + 1, rowp, nb, ns);
        const T nv = log_add<T, FAST>(own + lb, left + ls);
        const bool act = (unsigned)(s - s_lo) <= span;
        if (act) *st = nv;
        own = act ? nv : own;  // a column changes only during its own steps
        st += U1;
        left = neighbour<T, false>(own, xchg, xs++, lane, warp, nwarps);
      }
      // Every thread is past its last read of this stage (it took part in the
      // exchange of the chunk's last step): refill it.
      if (nwarps == 1) __syncwarp();
      if (u == 0 && j + kStages < nchunks) issue(j + kStages);
    }
    if (u == U) {
      const int64_t fin = cell_pos<MODIFIED>(Tn - 1, U, U1);
      scores[b] = own + lp2[fin].x;
    }
  } else {
    // ------------------------------- beta ------------------------------
    // Runs the steps backwards; step s needs (blank, symbol) of its own cell.
    T *be = beta + off;
    T own = ninf;
    if (u == U) {
      own = lp2[(int64_t)top * U1 + U].x;
      be[(int64_t)top * U1 + U] = own;
    }
    T right = neighbour<T, true>(own, xchg, xs++, lane, warp, nwarps);
    // The final cell is done; column U therefore stops one step earlier.
    const int hi = (u == U) ? s_hi - 1 : s_hi;
    const unsigned span = (hi >= s_lo) ? (unsigned)(hi - s_lo) : 0u;
    const bool any = hi >= s_lo;
    T *st = be + ((int64_t)(top - 1) * U1 + uc);  // entry of the first step
    for (int j = 0; j < nchunks; ++j) {
      int row0, n;
      chunk_rows(j, row0, n);
      wait_chunk(j);
      const P *rowp = stage + (int64_t)(j % kStages) * stage_pairs + (int64_t)(n - 1) * U1 + uc;
      // (blank(t,u), sym(t,u)) of the step's own cell; column U has no symbol.
      auto fetch = [&](int s, const P *q, T &vb, T &vs) {
        const P v = q[0];
        const bool in = any && (unsigned)(s - s_lo) <= span;
        vb = in ? v.x : ninf;
        vs = (in && u < U) ? v.y : ninf;
      };
      T nb, ns;
      fetch(row0 + n - 1, rowp, nb, ns);
#pragma unroll 2
      for (int i = n - 1; i >= 0; --i) {
        const int s = row0 + i;
        const T lb = nb, ls = ns;
        rowp -= U1;
        if (i > 0) fetch(s - 1, rowp, nb, ns);
        const T nv = log_add<T, FAST>(own + lb, right + ls);
        const bool act = any && (unsigned)(s - s_lo) <= span;
        if (act) *st = nv;
        own = act ? nv : own;   // column U keeps the final cell until its steps begin
        st -= U1;
        right = neighbour<T, true>(own, xchg, xs++, lane, warp, nwarps);
      }
      if (nwarps == 1) __syncwarp();
      if (u == 0 && j + kStages < nchunks) issue(j + kStages);
    }
    if (u == 0) scores_beta[b] = own;
  }
}

// ---------------------------------------------------------------------------
// Skewed variant: one CTA barrier per K steps instead of one per step.
//
// The recursion is cut into blocks of K consecutive steps (K = the rows of one
// staged chunk).  In phase p, warp w works on block p - delay(w), where the
// delay grows by one per warp in the direction the boundary values flow (alpha:
// delay = w; beta: delay = nwarps-1-w).  The value a warp needs from its
// neighbour at step s was therefore produced one phase earlier: it is read
// from a small shared-memory ring (indexed by step) with a plain load, one step
// ahead, and nothing is exchanged inside a phase.  Cost: nwarps-1 extra phases
// while the pipeline of warps fills; gain: the barrier and the shared-memory
// round trip leave the per-step dependency chain, which is then only
// shuffle -> add -> log-add.
//
// Chunk c of the log-probs (rows [cK, cK+K) of the wavefront-ordered array) is
// used in phases c .. c+nwarps-1 and is requested two phases before its first
// use, so the stage ring needs nwarps + 3 stages.
constexpr int kSkewRing = 64;   // ring entries per warp boundary; >= 4*K
constexpr int kSkewMaxK = 16;
constexpr int kSkewMaxStages = kMaxWarps + 3;

template <typename T, int ARITH, bool MODIFIED>
__global__ void __launch_bounds__(1024)
lattice_skew_kernel(const T *__restrict__ lp, const int32_t *__restrict__ Tl,
                    const int32_t *__restrict__ Ul, const int64_t *__restrict__ cell_split,
                    int32_t *__restrict__ status, T *__restrict__ alpha,
                    T *__restrict__ beta, T *__restrict__ scores,
                    T *__restrict__ scores_beta, int K, int stage_pairs, int nstages, int group) {
  using P = typename Pair<T>::type;
  using N = Num<T, ARITH>;
  extern __shared__ __align__(128) unsigned char stage_mem[];
  __shared__ __align__(8) uint64_t full_bar[kSkewMaxStages];
  __shared__ N edge[kMaxWarps][kSkewRing];  // edge[w][s & 63]: boundary column of warp w after step s
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x >> 1;
  const bool backward = blockIdx.x & 1;
  // four independent loads, one round trip
  const int bad = status[kStatusCode];
  const int Tn = Tl[b], U = Ul[b], U1 = U + 1;
  const int64_t off = cell_split[b];
  if (bad != 0) return;
  {
    int lo, hi;
    group_range(status, group, (int)(gridDim.x >> 1), lo, hi);
    if (b < lo || b >= hi) return;  // an utterance of the other group
  }
  if (threadIdx.x == 0) trace_begin(status, trace_slot(kStageLattice, group));
  const int u = threadIdx.x, lane = u & 31, warp = u >> 5;
  const int nwarps = (U1 + kWarp - 1) / kWarp;
  // The warp behind the last column warp (the launcher adds one when the block has
  // room) does nothing but request the log-prob chunks: two dozen instructions per
  // block of steps that the first column warp, which heads the dependency chain,
  // no longer issues.  Without it thread 0 requests them.
  const bool has_loader = (int)blockDim.x > nwarps * kWarp;
  if (warp > nwarps || (warp == nwarps && !has_loader)) return;
  const bool loader = warp == nwarps;
  const bool requests = has_loader ? (loader && lane == 0) : (u == 0);
  const int nact = (nwarps + (has_loader ? 1 : 0)) * kWarp;
  const bool solo = nact == kWarp;  // one warp in all: a warp barrier will do
  const P *lp2 = reinterpret_cast<const P *>(lp) + off;
  P *stage = reinterpret_cast<P *>(stage_mem) + 2;  // slack: column 0 reads the pair before its row
  const bool col = u < U1;
  const int diff = Tn - 1 - U;
  int s_lo, s_hi;
  if (MODIFIED) { s_lo = u; s_hi = u + diff; }
  else { s_lo = u; s_hi = u + Tn - 1; }
  if (!col) { s_lo = 1 << 30; s_hi = -1; }
  const int top = MODIFIED ? Tn - 1 : Tn - 1 + U;
  const T ninf = neg_inf<T>();
  const int uc = col ? u : U;
  constexpr int kMask = kSkewRing - 1;

  const int nrows = top;  // wavefront rows 0 .. top-1 are streamed
  const int nchunks = (nrows + K - 1) / K;
  const int nphases = nchunks > 0 ? nchunks + nwarps - 1 : 0;
  const int delay = backward ? nwarps - 1 - warp : warp;
  if (requests) {
    for (int i = 0; i < nstages; ++i) mbar_init(&full_bar[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  // Chunk j (processing order) covers memory rows [row0, row0 + n).
  auto chunk_rows = [&](int j, int &row0, int &n) {
    const int m = backward ? nchunks - 1 - j : j;
    row0 = m * K;
    n = min(K, nrows - row0);
  };
  // Chunk j lives in ring stage j % nstages and completes phase (j / nstages) & 1 of
  // that stage's barrier.  Both are carried along instead of computed: a division by
  // the run-time ring size costs some 25 dependent instructions, at the head of every
  // block of steps, on a warp that has nothing else to issue.
  auto issue = [&](int j, int slot) {  // thread 0 only; slot = j % nstages
    int row0, n;
    chunk_rows(j, row0, n);
    const uint32_t bytes = (uint32_t)((((int64_t)n * U1 * sizeof(P)) + 15) & ~int64_t(15));
    uint64_t *bar = &full_bar[slot];
    mbar_expect_tx(bar, bytes);
    tma_load_1d(stage + (int64_t)slot * stage_pairs, lp2 + (int64_t)row0 * U1, bytes, bar);
  };
  auto wait_chunk = [&](int slot, uint32_t parity) {
    uint64_t *bar = &full_bar[slot];
    for (int spin = 0; spin < (1 << 22); ++spin)
      if (mbar_try_wait(bar, parity)) return;
    atomicCAS(status + kStatusCopyTimeout, 0, 1 + b);  // bounded: report and carry on
  };
  int issue_slot = 2;           // of chunk p + 2 (nstages >= 4)
  int slot = 0;                 // of the chunk this warp works on next
  uint32_t slot_parity = 0;
  // The completion of the NEXT chunk is looked at once, without waiting, at the head
  // of a block of steps; the answer is needed a block later, so the barrier's latency
  // (about 90 cycles, which used to open every block) runs beside the steps.  A chunk
  // that has not landed by then is waited for at the head of its own block as before.
  bool landed = false;
  auto advance = [&](bool more) {
    if (++slot == nstages) { slot = 0; slot_parity ^= 1u; }
    landed = more && mbar_try_wait(&full_bar[slot], slot_parity);
  };

  if (loader) {
    if (lane == 0) for (int j = 0; j < 2 && j < nchunks; ++j) issue(j, j);
    bar_active(nact);
    for (int p = 0; p < nphases; ++p) {
      if (lane == 0 && p + 2 < nchunks) issue(p + 2, issue_slot);
      if (++issue_slot == nstages) issue_slot = 0;
      bar_active(nact);
    }
    return;
  }
  if (!backward) {
    // ------------------------------ alpha ------------------------------
    const bool produce = (lane == kWarp - 1) && (warp + 1 < nwarps);
    const bool consume = (lane == 0) && (warp > 0);
    N *out_edge = edge[warp];
    const N *in_edge = edge[consume ? warp - 1 : 0];  // lanes that do not consume read (and drop) a valid word
    // The value of step s sits in ring entry (s-1) & 63.
    // "after step 0": columns 31, 63, ... have not started
    if (lane == 0) out_edge[kMask] = N::zero();
    T *al = alpha + off;
    N own = (u == 0) ? N::from_log((T)0) : N::zero();
    if (u == 0) al[0] = 0;
    if (requests) for (int j = 0; j < 2 && j < nchunks; ++j) issue(j, j);  // by the thread that initialised the barriers
    // blank log-prob of the final cell, for the score (fetched long before it is needed)
    const T fin_blank = (u == U) ? lp2[cell_pos<MODIFIED>(Tn - 1, U, U1)].x : (T)0;
    if (!solo) bar_active(nact); else __syncwarp();
    const bool first_col = (u == 0);  // has no symbol predecessor
    for (int p = 0; p < nphases; ++p) {
      if (requests && p + 2 < nchunks) issue(p + 2, issue_slot);
      if (++issue_slot == nstages) issue_slot = 0;
      const int q = p - delay;
      if (q >= 0 && q < nchunks) {
        int row0, n;
        chunk_rows(q, row0, n);
        if (!landed) wait_chunk(slot, slot_parity);
        const P *rowp = stage + (int64_t)slot * stage_pairs + uc;
        advance(q + 1 < nchunks);
        T *st = al + (int64_t)(row0 + 1) * U1 + uc;  // entry of the block's first step
        // No range checks anywhere in a step.  Log-probs: entries that are no
        // lattice cell hold -inf (stage 0 fills, stage 1 overwrites the real
        // cells), and a column that has not started holds -inf itself.  Stores:
        // every (step, column) pair has an entry in the utterance's block, and
        // what lands in the entries that are no cell is never read.
        N lb = N::from_log(rowp[0].x);
        N ls = N::from_log(first_col ? ninf : rowp[-1].y);
        N e_cur = in_edge[(row0 - 1) & kMask];  // column u-1 after step row0
        // One step; `e_in` / `e_out` are the ring entries of this step.
        auto step = [&](const bool more, const N *e_in, N *e_out) {
          // loads (and the conversion of the log-probs) for the next step first
          rowp += U1;
          T x_next = ninf, y_next = ninf;
          N e_next = N::zero();
          if (more) {
            x_next = rowp[0].x;
            y_next = rowp[-1].y;
            e_next = *e_in;
          }
          y_next = first_col ? ninf : y_next;
          const N lb_next = N::from_log(x_next), ls_next = N::from_log(y_next);
          // the chain
          const N up = own.up();
          const N left = N::pick(consume, e_cur, up);
          // What a column holds after its last cell is never consumed (its
          // neighbour's cells end one step later).
          own = N::mad2(own, lb, left, ls);
          if (col) *st = own.log();
          st += U1;
          if (produce) *e_out = own;
          lb = lb_next; ls = ls_next;
          e_cur = e_next;
        };
        if (n == kSkewMaxK && K == kSkewMaxK) {
          // row0 is a multiple of 16: the block's ring entries do not wrap, and
          // with the loop unrolled they are constant offsets from one base.
          const N *e_in = in_edge + (row0 & kMask);
          N *e_out = out_edge + (row0 & kMask);
#pragma unroll
          for (int i = 0; i < kSkewMaxK; ++i) step(i + 1 < kSkewMaxK, e_in + i, e_out + i);
        } else {
          for (int i = 0; i < n; ++i)
            step(i + 1 < n, in_edge + ((row0 + i) & kMask), out_edge + ((row0 + i) & kMask));
        }
        own.renorm();  // K <= 16 steps since the last one
      }
      if (!solo) bar_active(nact); else __syncwarp();
    }
    if (u == U) scores[b] = own.log() + fin_blank;  // column U's last step is the last step
    if (u == 0) trace_end(status, trace_slot(kStageLattice, group));
  } else {
    // ------------------------------- beta ------------------------------
    const bool produce = (lane == 0) && (warp > 0);
    const bool consume = (lane == kWarp - 1) && (warp + 1 < nwarps);
    N *out_edge = edge[warp];
    const N *in_edge = edge[consume ? warp + 1 : 0];
    T *be = beta + off;
    const T fin = lp2[(int64_t)top * U1 + U].x;  // beta(T-1,U)
    N own = N::zero();
    if (u == U) {
      own = N::from_log(fin);
      be[(int64_t)top * U1 + U] = fin;
    }
    // "after step top": the boundary column of this warp before any step
    if (lane == 0) out_edge[top & kMask] = own;  // column U: the final cell; every other column: nothing yet
    if (requests) for (int j = 0; j < 2 && j < nchunks; ++j) issue(j, j);
    if (!solo) bar_active(nact); else __syncwarp();
    // Column U starts with the final cell and computes from the first step on,
    // unless it has no other cell (standard: T == 1; one symbol per frame:
    // U == T-1): then it must keep the final cell for column U-1 to read.
    const int hi = (u == U) ? s_hi - 1 : s_hi;
    const bool keep = (u == U) && hi < s_lo;
    const bool wr = col && !keep;
    for (int p = 0; p < nphases; ++p) {
      if (requests && p + 2 < nchunks) issue(p + 2, issue_slot);
      if (++issue_slot == nstages) issue_slot = 0;
      const int q = p - delay;
      if (q >= 0 && q < nchunks) {
        int row0, n;
        chunk_rows(q, row0, n);
        if (!landed) wait_chunk(slot, slot_parity);
        const P *rowp = stage + (int64_t)slot * stage_pairs + (int64_t)(n - 1) * U1 + uc;
        advance(q + 1 < nchunks);
        T *st = be + (int64_t)(row0 + n - 1) * U1 + uc;  // entry of the block's first step
        N lb, ls;
        {
          const P v = rowp[0];  // (-inf, -inf) where (step, column) is no lattice cell
          lb = N::from_log(v.x); ls = N::from_log(v.y);
        }
        N e_cur = in_edge[(row0 + n) & kMask];  // column u+1 after step row0+n
        // One step (no range checks, as in the alpha sweep); the value of step
        // s sits in ring entry s & 63.
        auto step = [&](const bool more, const N *e_in, N *e_out) {
          rowp -= U1;
          P v_next;
          v_next.x = ninf; v_next.y = ninf;
          N e_next = N::zero();
          if (more) {
            v_next = rowp[0];
            e_next = *e_in;
          }
          const N lb_next = N::from_log(v_next.x), ls_next = N::from_log(v_next.y);
          const N dn = own.down();
          const N right = N::pick(consume, e_cur, dn);
          const N nv = N::mad2(own, lb, right, ls);
          own = N::pick(keep, own, nv);
          if (wr) *st = nv.log();
          st -= U1;
          if (produce) *e_out = own;
          lb = lb_next; ls = ls_next;
          e_cur = e_next;
        };
        if (n == kSkewMaxK && K == kSkewMaxK) {
          const N *e_in = in_edge + (row0 & kMask);
          N *e_out = out_edge + (row0 & kMask);
#pragma unroll
          for (int i = kSkewMaxK - 1; i >= 0; --i) step(i > 0, e_in + i, e_out + i);
        } else {
          for (int i = n - 1; i >= 0; --i)
            step(i > 0, in_edge + ((row0 + i) & kMask), out_edge + ((row0 + i) & kMask));
        }
        own.renorm();
      }
      if (!solo) bar_active(nact); else __syncwarp();
    }
    if (u == 0) scores_beta[b] = own.log();  // column 0's last step is the last step
    if (u == 0) trace_end(status, trace_slot(kStageLattice, group));
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
                       T *__restrict__ scores, T *__restrict__ scores_beta, int group) {
  pdl_wait();
  pdl_trigger();
  if (status[kStatusCode] != 0) return;
  const int b = blockIdx.x >> 1;
  {
    int lo, hi;
    group_range(status, group, (int)(gridDim.x >> 1), lo, hi);
    if (b < lo || b >= hi) return;  // an utterance of the other group
  }
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

// The skewed kernel needs (warps + 3) stages of K rows; it is used when that
// fits into kSkewSmemBudget with K >= 2.  OT_B200_LATTICE=lockstep forces the
// per-step-barrier kernel (for comparison).
constexpr size_t kSkewSmemBudget = 160 * 1024;

bool lockstep_forced() {
  static std::atomic<int> cached{-1};
  int c = cached.load(std::memory_order_relaxed);
  if (c < 0) {
    const char *e = getenv("OT_B200_LATTICE");
    c = (e && strcmp(e, "lockstep") == 0) ? 1 : 0;
    cached.store(c, std::memory_order_relaxed);
  }
  return c == 1;
}

// Returns cudaErrorNotSupported when the lattice is too wide for the skewed kernel.
// OT_B200_LATTICE_LOADER=0: the log-prob chunks are requested by the first column
// warp, as before the loader warp was added (to measure one against the other).
bool loader_warp_wanted() {
  const char *e = getenv("OT_B200_LATTICE_LOADER");
  return !(e && strcmp(e, "0") == 0);
}

template <typename T, int ARITH, bool MODIFIED>
cudaError_t launch_skewed(const Problem &p, void *scores, cudaStream_t s) {
  using P = typename Pair<T>::type;
  auto kernel = lattice_skew_kernel<T, ARITH, MODIFIED>;
  const int cols = p.max_u + 1;
  const int nwarps = (cols + kWarp - 1) / kWarp;
  const int nstages = nwarps + 3;
  int K = kSkewMaxK;
  size_t smem = 0;
  int stage_pairs = 0;
  for (; K >= 2; K -= 2) {
    stage_pairs = ((K * cols + 1) & ~1) + 2;
    smem = ((size_t)nstages * stage_pairs + 2) * sizeof(P);
    if (smem <= kSkewSmemBudget) break;
  }
  if (K < 2 || lockstep_forced()) return cudaErrorNotSupported;
  static SmemGrant grant;  // per device: dynamic shared memory opted in so far
  {
    const cudaError_t e = grant.ensure(kernel, smem);
    if (e != cudaSuccess) return e;
  }
  const int loader_warps = (nwarps < kMaxWarps && loader_warp_wanted()) ? 1 : 0;  // see the kernel
  const cudaError_t le = launch_pdl(kernel, 2u * (unsigned)p.N, (unsigned)((nwarps + loader_warps) * kWarp), smem, s,
      reinterpret_cast<const T *>(p.ws + p.lay.lp), p.T, p.U,
      reinterpret_cast<const int64_t *>(p.ws + p.lay.cell_split),
      reinterpret_cast<int32_t *>(p.ws + p.lay.status),
      reinterpret_cast<T *>(p.ws + p.lay.alpha), reinterpret_cast<T *>(p.ws + p.lay.beta),
      static_cast<T *>(scores), reinterpret_cast<T *>(p.ws + p.lay.scores_beta), K, stage_pairs,
      nstages, p.group);
  return le != cudaSuccess ? le : cudaGetLastError();
}

template <typename T, bool FAST, bool MODIFIED>
cudaError_t launch_staged(const Problem &p, void *scores, cudaStream_t s) {
  using P = typename Pair<T>::type;
  {
    // float: the scaled linear arithmetic when the caller asks for it
    constexpr bool kCanLinear = sizeof(T) == 4;
    cudaError_t e;
    if constexpr (kCanLinear) {
      e = (p.flags & OT_B200_LINEAR_DOMAIN)
              ? launch_skewed<T, kArithLinear, MODIFIED>(p, scores, s)
              : launch_skewed<T, FAST ? kArithLogFast : kArithLog, MODIFIED>(p, scores, s);
    } else {
      e = launch_skewed<T, FAST ? kArithLogFast : kArithLog, MODIFIED>(p, scores, s);
    }
    if (e != cudaErrorNotSupported) return e;
  }
  auto kernel = lattice_kernel<T, FAST, MODIFIED>;
  const int cols = p.max_u + 1;
  // rows per chunk: even, at least 2, about kChunkBytes per chunk
  int R = (int)(kChunkBytes / ((int64_t)cols * sizeof(P)));
  R = (R < 2) ? 2 : (R > 256 ? 256 : (R & ~1));
  const int stage_pairs = ((R * cols + 1) & ~1) + 2;  // + slack for the 16-byte round-up
  const size_t smem = ((size_t)kStages * stage_pairs + 2) * sizeof(P);
  // always opt in: static shared memory counts against the 48 KB default as well
  static SmemGrant grant;
  {
    const cudaError_t e = grant.ensure(kernel, smem);
    if (e != cudaSuccess) return e;
  }
  const unsigned block = (unsigned)((cols + kWarp - 1) / kWarp * kWarp);
  const cudaError_t le = launch_pdl(kernel, 2u * (unsigned)p.N, block, smem, s,
      reinterpret_cast<const T *>(p.ws + p.lay.lp), p.T, p.U,
      reinterpret_cast<const int64_t *>(p.ws + p.lay.cell_split),
      reinterpret_cast<int32_t *>(p.ws + p.lay.status),
      reinterpret_cast<T *>(p.ws + p.lay.alpha), reinterpret_cast<T *>(p.ws + p.lay.beta),
      static_cast<T *>(scores), reinterpret_cast<T *>(p.ws + p.lay.scores_beta), R, stage_pairs, p.group);
  return le != cudaSuccess ? le : cudaGetLastError();
}

template <typename T>
cudaError_t launch_lattice_t(const Problem &p, void *scores, cudaStream_t s) {
  const bool modified = p.flags & OT_B200_ONE_SYM_PER_FRAME;
  const bool fast = p.flags & OT_B200_FAST_MATH;
  if (p.max_u + 1 > 1024) {
    const int32_t *status = reinterpret_cast<const int32_t *>(p.ws + p.lay.status);
    const int64_t *csplit = reinterpret_cast<const int64_t *>(p.ws + p.lay.cell_split);
    const T *lp = reinterpret_cast<const T *>(p.ws + p.lay.lp);
    T *alpha = reinterpret_cast<T *>(p.ws + p.lay.alpha);
    T *beta = reinterpret_cast<T *>(p.ws + p.lay.beta);
    T *sb = reinterpret_cast<T *>(p.ws + p.lay.scores_beta);
    T *sa = static_cast<T *>(scores);
    const unsigned grid = 2u * (unsigned)p.N;
    if (modified) lattice_generic_kernel<T, true><<<grid, 1024, 0, s>>>(lp, p.T, p.U, csplit, status, alpha, beta, sa, sb, p.group);
    else lattice_generic_kernel<T, false><<<grid, 1024, 0, s>>>(lp, p.T, p.U, csplit, status, alpha, beta, sa, sb, p.group);
    return cudaGetLastError();
  }
  if (fast) return modified ? launch_staged<T, true, true>(p, scores, s) : launch_staged<T, true, false>(p, scores, s);
  return modified ? launch_staged<T, false, true>(p, scores, s) : launch_staged<T, false, false>(p, scores, s);
}

}  // namespace

cudaError_t launch_lattice(const Problem &p, void *scores, cudaStream_t s) {
  return (p.flags & OT_B200_FP64) ? launch_lattice_t<double>(p, scores, s)
                                  : launch_lattice_t<float>(p, scores, s);
}

}  // namespace otb
