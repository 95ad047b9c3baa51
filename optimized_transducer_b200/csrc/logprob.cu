// Stage 1: row-wise logsumexp of the packed logits fused with the gather of the
// blank and next-symbol log-probabilities.
//
// Replaces `logits.logsumexp(1)` (optimized_transducer/csrc/cuda.cu:427) and
// ComputeLogProbs (optimized_transducer/csrc/kernels.cu:30-60), and, for
// log-softmax input, ComputeLogProbsForLogSoftmax (kernels.cu:62-88).
//
// The kernel is HBM-bound only if it is lean: at the roofline an SM has about
// 150 issue slots per 2000-byte row.  So
//  * a row is owned by a GROUP of LPR lanes (32, 16 or 8), i.e. a warp works on
//    32/LPR rows at once: the per-row bookkeeping (position in the lattice,
//    reductions, gather, stores) is paid once per warp instruction for all of
//    them, and the shuffle reductions are log2(LPR) deep;
//  * the reduction costs one FFMA, one ex2 and one add per element
//    (exp(x - m) = 2^(x*log2e - m*log2e));
//  * a group takes runs of kRun consecutive rows and walks (b, t, u)
//    incrementally inside a run, so the owning utterance is searched once per
//    run, not once per row.
// One short-lived block per 128 or 256 rows (a lane group takes one run), or one
// resident wave with OT_B200_GRID=wave.  Runs are dealt in order, so the grid
// sweeps the buffer front to back and the rows read last are contiguous at the
// end, where stage 3 starts.  A row is read once with 16-byte coalesced loads,
// all issued before the first use; the two gathered entries are requested with
// them and fall into the lines just fetched.  HBM traffic per row:
// V*sizeof(X) bytes read, 3*sizeof(T) bytes written.  Float rows of 260..512
// columns take the bulk-copy staged variant further down.
#include <stdlib.h>

#include <stdlib.h>
#include <string.h>

#include "ot_common.cuh"

namespace otb {

namespace {

constexpr int kThreads = 256;
constexpr int kRun = 8;  // rows a group takes at a time

// sum_k exp(x_k - m) accumulated into s, for one lane's part of a chunk.
template <int N>
__device__ __forceinline__ float add_exps(const float (&x)[N], float m, float s) {
  const float mneg = -m * kLog2e;
#pragma unroll
  for (int k = 0; k < N; ++k) s += ex2_approx(fmaf(x[k], kLog2e, mneg));
  return s;
}
template <int N>
__device__ __forceinline__ double add_exps(const double (&x)[N], double m, double s) {
#pragma unroll
  for (int k = 0; k < N; ++k) s += exp(x[k] - m);
  return s;
}

template <typename T, int LPR>
__device__ __forceinline__ T group_max(T v, unsigned mask) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v = r_max(v, __shfl_xor_sync(mask, v, o));
  return v;
}
template <typename T, int LPR>
__device__ __forceinline__ T group_sum(T v, unsigned mask) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(mask, v, o);
  return v;
}

// X: storage type of the logits, T = Real<X>: type of the arithmetic and of the
// outputs.  VEC: elements per load (one vector of Vec16<X>, or 1 element when
// the row stride or the base pointer is not aligned to it).  LPR: lanes per row.
// CH: loads per lane per chunk, i.e. a chunk covers LPR*VEC*CH elements.
template <typename X, int VEC, int CH, int LPR, bool MODIFIED, int MINB = 4>
__global__ void __launch_bounds__(kThreads, MINB)
logprob_kernel(const X *__restrict__ logits, const int32_t *__restrict__ targets,
               const int32_t *__restrict__ Tl, const int32_t *__restrict__ Ul,
               const int64_t *__restrict__ split, const int64_t *__restrict__ cell_split,
               const int32_t *__restrict__ status, int N, int64_t row_begin, int64_t rows, int V,
               int max_u, int blank, typename Real<X>::type *__restrict__ den,
               typename Real<X>::type *__restrict__ lp, int trace_group) {
  // This launch covers the packed rows [row_begin, rows); `trace_group` only names
  // the timeline slot.
  pdl_wait();
  pdl_trigger();
  if (status[kStatusCode] != 0) return;
  if (threadIdx.x == 0) trace_begin(status, trace_slot(kStageLogprob, trace_group));
  using T = typename Real<X>::type;
  using VT = typename VecOf<X, VEC>::type;
  constexpr int kGroups = kWarp / LPR;  // rows a warp works on at once
  const int lane = threadIdx.x & 31;
  const int gl = lane % LPR;            // lane within the group
  const unsigned gmask = (LPR == 32) ? kFull : (((1u << LPR) - 1u) << (lane - gl));
  const int64_t group = ((((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5) * kGroups) + lane / LPR;
  const int64_t ngroups = (((int64_t)gridDim.x * kThreads) >> 5) * kGroups;
  const int nvec = V / VEC;
  const T ninf = neg_inf<T>();
  const int64_t nruns = (rows - row_begin + kRun - 1) / kRun;

  for (int64_t run = group; run < nruns; run += ngroups) {
    const int64_t r0 = row_begin + run * kRun;
    const int64_t r1 = (r0 + kRun < rows) ? r0 + kRun : rows;
    // Position of the run's first row; afterwards (b, t, u) advance with the rows.
    int b = find_utt(split, N, r0);
    int Tn = __ldg(Tl + b), U = __ldg(Ul + b), U1 = U + 1;
    int64_t next_split = __ldg(split + b + 1);
    int64_t coff = __ldg(cell_split + b);
    int t, u;
    {
      const int idx = (int)(r0 - __ldg(split + b));
      t = idx / U1; u = idx - t * U1;
    }
    for (int64_t row = r0; row < r1; ++row) {
      const X *p = logits + row * (int64_t)V;
      bool skip = false;
      if (MODIFIED) {
        // Cells outside the band u <= t <= u + (T-1-U) are never used
        // (optimized_transducer/csrc/cpu.cc:295): their rows are not read.
        skip = (u > t) || (t - u > Tn - 1 - U);
      }
      if (!skip) {
        T m = ninf, s = 0;
        // The gather (lane 0 of the group: blank entry, lane 1: symbol entry) is
        // requested together with the row, not after the reduction: the symbol's
        // index first, the two entries right behind the row's own loads (they
        // fall into lines those loads are fetching anyway).
        const int tsym = (gl == 1 && u < U) ? __ldg(targets + (int64_t)b * max_u + u) : -1;
        T graw = ninf;
        for (int base = 0; base < nvec; base += LPR * CH) {
          T x[CH * VEC];
#pragma unroll
          for (int j = 0; j < CH; ++j) {
            const int vi = base + j * LPR + gl;
            if (vi < nvec) {
              const VT v = *reinterpret_cast<const VT *>(p + (int64_t)vi * VEC);
              const X *e = reinterpret_cast<const X *>(&v);
#pragma unroll
              for (int k = 0; k < VEC; ++k) x[j * VEC + k] = to_real(e[k]);
            } else {
#pragma unroll
              for (int k = 0; k < VEC; ++k) x[j * VEC + k] = ninf;
            }
          }
          if (base == 0) {
            if (gl == 0) graw = to_real(p[blank]);
            if (tsym >= 0) graw = to_real(p[tsym]);
          }
          T cm = x[0];
#pragma unroll
          for (int k = 1; k < CH * VEC; ++k) cm = r_max(cm, x[k]);
          cm = group_max<T, LPR>(cm, gmask);  // the running maximum is uniform across the group
          if (cm > m) { s *= s_exp(m - cm); m = cm; }  // first chunk: s is 0
          // An infinite maximum needs no sum (see below); skipping it avoids inf - inf.
          if (m - m == (T)0) s = add_exps(x, m, s);
        }
        // ATen's logsumexp replaces an infinite maximum by 0 before subtracting,
        // which makes the result that same infinity.
        const T d = (m - m == (T)0) ? r_log(group_sum<T, LPR>(s, gmask)) + m : m;
        // Lane 0 holds the blank entry, lane 1 the symbol entry; the last column
        // has no next symbol: -inf, "no such transition".
        const T g = (gl == 0 || tsym >= 0) ? graw - d : ninf;
        const T g1 = __shfl_sync(gmask, g, (lane - gl) + 1);
        if (gl == 0) {
          den[row] = d;
          T *q = lp + 2 * (coff + cell_pos<MODIFIED>(t, u, U1));
          if constexpr (sizeof(T) == 4) *reinterpret_cast<float2 *>(q) = make_float2(g, g1);
          else *reinterpret_cast<double2 *>(q) = make_double2(g, g1);
        }
      }
      // advance to the next row
      if (++u == U1) { u = 0; ++t; }
      if (row + 1 == next_split && row + 1 < rows) {
        ++b;
        Tn = __ldg(Tl + b); U = __ldg(Ul + b); U1 = U + 1;
        next_split = __ldg(split + b + 1);
        coff = __ldg(cell_split + b);
        t = 0; u = 0;
      }
    }
  }
  if (threadIdx.x == 0) trace_end(status, trace_slot(kStageLogprob, trace_group));
}

// ---------------------------------------------------------------------------
// Maximum of two packed pairs of 16-bit values (exact; NaN handling of fmaxf).
template <typename X> __device__ __forceinline__ uint32_t pmax16(uint32_t a, uint32_t b);
template <> __device__ __forceinline__ uint32_t pmax16<__nv_bfloat16>(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&a),
                                   *reinterpret_cast<const __nv_bfloat162 *>(&b));
  return *reinterpret_cast<const uint32_t *>(&r);
}
template <> __device__ __forceinline__ uint32_t pmax16<__half>(uint32_t a, uint32_t b) {
  const __half2 r = __hmax2(*reinterpret_cast<const __half2 *>(&a), *reinterpret_cast<const __half2 *>(&b));
  return *reinterpret_cast<const uint32_t *>(&r);
}
template <> __device__ __forceinline__ uint32_t pmax16<float>(uint32_t a, uint32_t) { return a; }  // unused
template <typename X> __device__ __forceinline__ uint32_t packed_neg_inf() { return 0u; }
template <> __device__ __forceinline__ uint32_t packed_neg_inf<__nv_bfloat16>() { return 0xff80ff80u; }
template <> __device__ __forceinline__ uint32_t packed_neg_inf<__half>() { return 0xfc00fc00u; }

// The same stage with the rows staged through shared memory by bulk copies, for
// the common shape: float rows of 64 < V/4 <= 128 vectors (V = 260..512,
// V % 4 == 0), standard transducer.  A block walks over `tiles_per_block`
// consecutive tiles of 16 rows (16 of them, fewer in a launch of at most three
// waves: see the launcher); thread 0 keeps kTmaStages tiles (16 * V * 4 bytes each,
// one contiguous piece of the packed buffer) in flight with cp.async.bulk +
// mbarrier, the 16 lane groups of the block each reduce one row of the tile out
// of shared memory.  What this buys: the bytes in flight no longer depend on
// the registers a warp can hold (two blocks x 3 stages x 32 KB per SM instead
// of 32 warps x 4 KB, and none while a warp computes), so the loads and the
// exp-sum overlap fully.
constexpr int kTmaRows = 16;     // rows per tile = lane groups per block
constexpr int kTmaStagesMax = 3;
constexpr int kTmaTiles = 16;    // tiles per block in a launch of many waves

// kTmaStages: tiles in flight per block (three); kBlocks: resident blocks per SM the
// registers are capped for (two; see the launcher for what else was measured).
// kFull: the first kFull of a lane's eight vectors exist in every row the launcher
// sends here (4 for V/4 > 64, 7 for V/4 > 112), so only the others are range-checked.
template <typename X, int kTmaStages, int kBlocks, int kFull>
__global__ void __launch_bounds__(kThreads, kBlocks)
logprob_tma_kernel(const X *__restrict__ logits, const int32_t *__restrict__ targets,
                   const int32_t *__restrict__ Tl, const int32_t *__restrict__ Ul,
                   const int64_t *__restrict__ split, const int64_t *__restrict__ cell_split,
                   int32_t *__restrict__ status, int N, int64_t row_begin, int64_t rows, int V,
                   int max_u, int blank, float *__restrict__ den, float *__restrict__ lp,
                   int tiles_per_block, int trace_group) {
  // This launch covers the packed rows [row_begin, rows); row_begin is a multiple
  // of the tile height, so every tile starts on a 16-byte boundary.
  extern __shared__ __align__(128) unsigned char tile_mem[];
  __shared__ __align__(8) uint64_t full_bar[kTmaStages];
  // The first tiles are requested BEFORE this grid waits for stage 0: they only
  // read the logits, which whoever ran before stage 0 has finished writing
  // (stage 0 releases this grid after its own wait), and which are valid memory
  // whatever the lengths turn out to be.  Stage 0's few microseconds then run
  // under the first loads.
  pdl_trigger();
  constexpr int LPR = 16, CH = 8;
  const int lane = threadIdx.x & 31, gl = lane & (LPR - 1);
  const int g = threadIdx.x / LPR;  // lane group = row within the tile
  const unsigned gmask = ((1u << LPR) - 1u) << (lane - gl);
  using VT = typename VecOf<X, 4>::type;  // 4 elements: 16 bytes of float, 8 bytes of a 16-bit type
  const int nvec = V >> 2;
  const float ninf = neg_inf<float>();
  const uint32_t row_bytes = (uint32_t)V * (uint32_t)sizeof(X);
  const uint32_t tile_bytes = kTmaRows * row_bytes;
  const int64_t ntiles_all = (rows - row_begin + kTmaRows - 1) / kTmaRows;
  const int64_t tile0 = (int64_t)blockIdx.x * tiles_per_block;
  const int ntiles = (int)((ntiles_all - tile0 < tiles_per_block) ? (ntiles_all - tile0) : tiles_per_block);
  if (ntiles <= 0) return;  // cannot happen with the launcher's grid

  auto issue = [&](int k) {  // thread 0 only
    const int64_t r0 = row_begin + (tile0 + k) * kTmaRows;
    const int64_t nr = (rows - r0 < kTmaRows) ? (rows - r0) : kTmaRows;
    uint64_t *bar = &full_bar[k % kTmaStages];
    // a multiple of 16: V % 4 == 0, and for 16-bit rows the launcher requires an
    // even row count, so every tile and the tail are whole pairs of rows
    const uint32_t bytes = (uint32_t)nr * row_bytes;
    mbar_expect_tx(bar, bytes);
    tma_load_1d(tile_mem + (size_t)(k % kTmaStages) * tile_bytes, logits + r0 * (int64_t)V, bytes, bar);
  };
  if (threadIdx.x == 0) {
    for (int i = 0; i < kTmaStages; ++i) mbar_init(&full_bar[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    for (int k = 0; k < kTmaStages && k < ntiles; ++k) issue(k);
  }
  __syncthreads();
  pdl_wait();  // from here on: status, splits and the -inf fill of stage 0 are visible
  if (status[kStatusCode] != 0) {
    // bad input: nothing is computed, but the copies in flight must land before
    // the block gives its shared memory back (bounded wait, like every other)
    if (threadIdx.x == 0)
      for (int k = 0; k < kTmaStages && k < ntiles; ++k)
        for (int spin = 0; spin < (1 << 22); ++spin)
          if (mbar_try_wait(&full_bar[k], 0)) break;
    __syncthreads();
    return;
  }
  if (threadIdx.x == 0) trace_begin(status, trace_slot(kStageLogprob, trace_group));

  // Position of this group's first row; it then advances by 16 rows per tile.
  int64_t row = row_begin + tile0 * kTmaRows + g;
  int b = 0, Tn = 1, U = 0, U1 = 1, t = 0, u = 0;
  int64_t next_split = 0, coff = 0;
  auto locate = [&]() {
    b = find_utt(split, N, row);
    Tn = __ldg(Tl + b); U = __ldg(Ul + b); U1 = U + 1;
    next_split = __ldg(split + b + 1);
    coff = __ldg(cell_split + b);
    const int idx = (int)(row - __ldg(split + b));
    t = idx / U1; u = idx - t * U1;
  };
  if (row < rows) locate();
  (void)Tn;

  for (int k = 0; k < ntiles; ++k) {
    uint64_t *bar = &full_bar[k % kTmaStages];
    const uint32_t parity = (uint32_t)((k / kTmaStages) & 1);
    // index of the symbol entry, fetched while the tile is still on its way
    const int tsym = (gl == 0 && row < rows && u < U) ? __ldg(targets + (int64_t)b * max_u + u) : -1;
    bool arrived = false;
    for (int spin = 0; spin < (1 << 22); ++spin)  // bounded: report and carry on
      if (mbar_try_wait(bar, parity)) { arrived = true; break; }
    if (!arrived) atomicCAS(status + kStatusCopyTimeout, 0, 1);
    if (row < rows) {
      const X *p = reinterpret_cast<const X *>(tile_mem + (size_t)(k % kTmaStages) * tile_bytes) + (size_t)g * V;
      float x[CH * 4];
      // 16-bit rows: the maximum is taken on the packed pairs (half the instructions)
      [[maybe_unused]] uint32_t pm = packed_neg_inf<X>();
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int vi = j * LPR + gl;
        if (j < kFull || vi < nvec) {
          const VT v = *reinterpret_cast<const VT *>(p + vi * 4);
          if constexpr (sizeof(X) == 2) {  // two words of two elements each
            const uint32_t *w = reinterpret_cast<const uint32_t *>(&v);
            pm = pmax16<X>(pm, pmax16<X>(w[0], w[1]));
            const float2 a = Pair16<X>::widen(w[0]), b = Pair16<X>::widen(w[1]);
            x[j * 4 + 0] = a.x; x[j * 4 + 1] = a.y; x[j * 4 + 2] = b.x; x[j * 4 + 3] = b.y;
          } else {
            const X *e = reinterpret_cast<const X *>(&v);
            x[j * 4 + 0] = to_real(e[0]); x[j * 4 + 1] = to_real(e[1]);
            x[j * 4 + 2] = to_real(e[2]); x[j * 4 + 3] = to_real(e[3]);
          }
        } else {
          x[j * 4 + 0] = ninf; x[j * 4 + 1] = ninf; x[j * 4 + 2] = ninf; x[j * 4 + 3] = ninf;
        }
      }
      float m;
      if constexpr (sizeof(X) == 2) {
        const float2 mm = Pair16<X>::widen(pm);
        m = fmaxf(mm.x, mm.y);
      } else {
        m = x[0];
#pragma unroll
        for (int i = 1; i < CH * 4; ++i) m = fmaxf(m, x[i]);
      }
      m = group_max<float, LPR>(m, gmask);
      float s = 0;
      if (m - m == 0.0f) s = add_exps(x, m, s);  // an infinite maximum needs no sum
      const float d = (m - m == 0.0f) ? logf(group_sum<float, LPR>(s, gmask)) + m : m;
      if (gl == 0) {
        const float gb = to_real(p[blank]) - d;
        const float gs = (tsym >= 0) ? to_real(p[tsym]) - d : ninf;
        den[row] = d;
        *reinterpret_cast<float2 *>(lp + 2 * (coff + cell_pos<false>(t, u, U1))) = make_float2(gb, gs);
      }
    }
    __syncthreads();  // every group is done with this stage
    if (threadIdx.x == 0 && k + kTmaStages < ntiles) issue(k + kTmaStages);
    // advance by one tile
    row += kTmaRows;
    if (row < rows) {
      if (row >= next_split) {
        locate();
      } else {
        u += kTmaRows;
        while (u >= U1) { u -= U1; ++t; }
      }
    }
  }
  if (threadIdx.x == 0) trace_end(status, trace_slot(kStageLogprob, trace_group));
}

// Log-softmax input: nothing to reduce, only the gather (thread per row).
template <typename X, bool MODIFIED>
__global__ void __launch_bounds__(kThreads)
gather_kernel(const X *__restrict__ logp, const int32_t *__restrict__ targets,
              const int32_t *__restrict__ Ul, const int64_t *__restrict__ split,
              const int64_t *__restrict__ cell_split,
              const int32_t *__restrict__ status, int N, int64_t rows, int V,
              int max_u, int blank, typename Real<X>::type *__restrict__ lp) {
  pdl_wait();
  pdl_trigger();
  if (status[kStatusCode] != 0) return;
  using T = typename Real<X>::type;
  const int64_t row = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (row >= rows) return;
  const int b = find_utt(split, N, row);
  const int U = __ldg(Ul + b), U1 = U + 1;
  const int idx = (int)(row - __ldg(split + b));
  const int t = idx / U1, u = idx - t * U1;
  const X *p = logp + row * (int64_t)V;
  T *q = lp + 2 * (__ldg(cell_split + b) + cell_pos<MODIFIED>(t, u, U1));
  q[0] = to_real(p[blank]);
  q[1] = (u < U) ? to_real(p[__ldg(targets + (int64_t)b * max_u + u)]) : neg_inf<T>();
}

template <typename X, int VEC, int CH, int LPR, bool MODIFIED>
cudaError_t launch_lse_m(const Problem &p, cudaStream_t s) {
  using T = typename Real<X>::type;
  // Four resident blocks per SM (64 registers): capping the registers for five
  // or six blocks spills the row buffer and is slower (forward 0.341 / 0.414 ms
  // against 0.314 ms on 686 128 rows of 500).
  auto kernel = logprob_kernel<X, VEC, CH, LPR, MODIFIED, 4>;
  static std::atomic<int> per_sm_cache{0};  // occupancy of this instantiation (same on every B200)
  int per_sm = per_sm_cache.load(std::memory_order_relaxed);
  if (per_sm == 0) {
    per_sm = blocks_per_sm(kernel, kThreads);
    per_sm_cache.store(per_sm, std::memory_order_relaxed);
  }
  constexpr int groups_per_block = (kThreads / kWarp) * (kWarp / LPR);
  const int64_t row_end = p.row_end > 0 ? p.row_end : p.rows;
  const int64_t nruns = (row_end - p.row_begin + kRun - 1) / kRun;  // a lane group takes one run at a time
  int64_t want = (nruns + groups_per_block - 1) / groups_per_block;
  if (wave_grids()) {
    const int64_t cap = (int64_t)resident_sms(p.flags) * per_sm;
    if (want > cap) want = cap;
  }
  const unsigned grid = (unsigned)(want < 1 ? 1 : (want < 0x7fffffff ? want : 0x7fffffff));
  const cudaError_t e = launch_pdl(kernel, grid, (unsigned)kThreads, 0, s,
      static_cast<const X *>(p.logits), p.targets, p.T, p.U,
      reinterpret_cast<const int64_t *>(p.ws + p.lay.split),
      reinterpret_cast<const int64_t *>(p.ws + p.lay.cell_split),
      reinterpret_cast<const int32_t *>(p.ws + p.lay.status), p.N, p.row_begin, row_end, p.V,
      p.max_u, p.blank, reinterpret_cast<T *>(p.ws + p.lay.den),
      reinterpret_cast<T *>(p.ws + p.lay.lp), p.group);
  return e != cudaSuccess ? e : cudaGetLastError();
}

template <typename X, int VEC, int CH, int LPR>
cudaError_t launch_lse(const Problem &p, cudaStream_t s) {
  return (p.flags & OT_B200_ONE_SYM_PER_FRAME) ? launch_lse_m<X, VEC, CH, LPR, true>(p, s)
                                               : launch_lse_m<X, VEC, CH, LPR, false>(p, s);
}

// OT_B200_LOGPROB=plain keeps the register-staged kernel for every shape.
bool plain_loads_forced() {  // read on every call, so that a test can compare the two kernels
  const char *e = getenv("OT_B200_LOGPROB");
  return e && strcmp(e, "plain") == 0;
}

template <typename X>
cudaError_t launch_logprob_t(const Problem &p, cudaStream_t s) {
  using T = typename Real<X>::type;
  if (p.flags & OT_B200_FROM_LOG_SOFTMAX) {
    const unsigned grid = (unsigned)((p.rows + kThreads - 1) / kThreads);
    const X *x = static_cast<const X *>(p.logits);
    const int64_t *split = reinterpret_cast<const int64_t *>(p.ws + p.lay.split);
    const int64_t *csplit = reinterpret_cast<const int64_t *>(p.ws + p.lay.cell_split);
    const int32_t *status = reinterpret_cast<const int32_t *>(p.ws + p.lay.status);
    T *lp = reinterpret_cast<T *>(p.ws + p.lay.lp);
    if (p.flags & OT_B200_ONE_SYM_PER_FRAME)
      gather_kernel<X, true><<<grid, kThreads, 0, s>>>(x, p.targets, p.U, split, csplit, status,
                                                       p.N, p.rows, p.V, p.max_u, p.blank, lp);
    else
      gather_kernel<X, false><<<grid, kThreads, 0, s>>>(x, p.targets, p.U, split, csplit, status,
                                                        p.N, p.rows, p.V, p.max_u, p.blank, lp);
    return cudaGetLastError();
  }
  constexpr int VEC = Vec16<X>::n;
  const bool vec_ok = (p.V % VEC == 0) &&
                      (reinterpret_cast<uintptr_t>(p.logits) % (VEC * sizeof(X)) == 0);
  if constexpr (sizeof(X) <= 4) {
    const int nv = p.V / 4;
    // 16-bit rows: a tile is a multiple of 16 bytes only for whole pairs of rows,
    // so the row count must be even (the last tile then ends on a pair as well)
    const int64_t row_end = p.row_end > 0 ? p.row_end : p.rows;
    const bool tiles_ok = p.row_begin % kTmaRows == 0 &&
                          (sizeof(X) == 4 || (row_end % 2 == 0 && reinterpret_cast<uintptr_t>(p.logits) % 16 == 0));
    if (vec_ok && tiles_ok && nv > 64 && nv <= 128 && !(p.flags & OT_B200_ONE_SYM_PER_FRAME) && !plain_loads_forced()) {
      // Two stages for the launches of a two-group call (so that a recursion CTA fits
      // beside the two resident blocks) were measured and are NOT used: stage 1 of
      // half the batch went from 118 to 126 us and the step from 0.669 to 0.684 ms.
      // Two resident blocks per SM, three tiles in flight per block, for float and for
      // 16-bit rows.  A 16-bit tile is half the bytes for the same instructions (about
      // 180 warp instructions per row either way), so that stage is bound by
      // instruction issue (71 % of the issue slots busy over the whole benchmark
      // batch, 4.3 TB/s), not by bytes in flight: measured per half of the 16-bit
      // benchmark batch, six tiles in flight per block 86 -> 104 us, three resident
      // blocks per SM (registers capped at 80) 86 -> 89 us.
      constexpr int kBlocksHere = 2;
      const bool wide = nv > 112;  // V/4 in (112, 128]: seven of a lane's eight vectors always exist
      auto tma_kernel = wide ? logprob_tma_kernel<X, kTmaStagesMax, kBlocksHere, 7>
                             : logprob_tma_kernel<X, kTmaStagesMax, kBlocksHere, 4>;
      constexpr int kStagesHere = kTmaStagesMax;
      const size_t smem = (size_t)kStagesHere * kTmaRows * p.V * sizeof(X);
      static SmemGrant grant_wide, grant_narrow;
      {
        const cudaError_t e = (wide ? grant_wide : grant_narrow)
                                  .ensure(tma_kernel, (size_t)kStagesHere * kTmaRows * 512 * sizeof(X));
        if (e != cudaSuccess) return e;
      }
      const int64_t ntiles = (row_end - p.row_begin + kTmaRows - 1) / kTmaRows;
      // Tiles per block.  Two blocks are resident per SM; a launch of a few waves of
      // 16-tile blocks ends with a mostly empty last wave (85 000 rows: 334 blocks on
      // 296 slots, 46 us against 36 us with every slot filled once), so such a launch
      // is cut into as few full waves as blocks of at most 24 tiles allow: equal
      // blocks, at least one tile more than the pipeline holds.
      // In a grouped call the recursion of the PREVIOUS group starts while this launch
      // fills the SMs: a recursion CTA (up to ~100 KB of shared memory) fits beside one
      // resident block but not beside two, and the blocks of a one-wave launch all live
      // as long as the launch (measured: recursions starting 22-29 us late), so such a
      // launch leaves one slot free on as many SMs as the batch has recursion CTAs.
      int tiles_per_block = kTmaTiles;
      {
        int64_t slots = kBlocksHere * (int64_t)sm_count();
        if (p.group >= 0) slots -= (2 * (int64_t)p.N < 64 ? 2 * (int64_t)p.N : 64);
        if (ntiles <= 3 * slots * kTmaTiles) {
          const int64_t waves = (ntiles + slots * 24 - 1) / (slots * 24);
          const int64_t even = (ntiles + slots * waves - 1) / (slots * waves);
          tiles_per_block = (int)(even < kStagesHere + 1 ? kStagesHere + 1 : even);
        }
      }
      const unsigned grid = (unsigned)((ntiles + tiles_per_block - 1) / tiles_per_block);
      const cudaError_t e = launch_pdl(tma_kernel,
          grid, (unsigned)kThreads, smem, s,
          static_cast<const X *>(p.logits), p.targets, p.T, p.U,
          reinterpret_cast<const int64_t *>(p.ws + p.lay.split),
          reinterpret_cast<const int64_t *>(p.ws + p.lay.cell_split),
          reinterpret_cast<int32_t *>(p.ws + p.lay.status), p.N, p.row_begin, row_end, p.V, p.max_u,
          p.blank, reinterpret_cast<float *>(p.ws + p.lay.den), reinterpret_cast<float *>(p.ws + p.lay.lp),
          tiles_per_block, p.group);
      return e != cudaSuccess ? e : cudaGetLastError();
    }
  }
  if (vec_ok) {
    const int nvec = p.V / VEC;  // vector loads per row
    // Up to 8 loads per lane: pick the narrowest group that covers the row in
    // one chunk; rows longer than 32*8 loads loop over chunks.
    if (nvec <= 8 * 4) return launch_lse<X, VEC, 4, 8>(p, s);
    if (nvec <= 8 * 8) return launch_lse<X, VEC, 8, 8>(p, s);
    if (nvec <= 16 * 8) return launch_lse<X, VEC, 8, 16>(p, s);
    return launch_lse<X, VEC, 8, 32>(p, s);
  }
  const int per_lane = (p.V + kWarp - 1) / kWarp;
  if (per_lane <= 4) return launch_lse<X, 1, 4, 32>(p, s);
  return launch_lse<X, 1, 16, 32>(p, s);
}

}  // namespace

cudaError_t launch_logprob(const Problem &p, cudaStream_t s) {
  if (p.flags & OT_B200_FP64) return launch_logprob_t<double>(p, s);
  if (p.flags & OT_B200_BF16) return launch_logprob_t<__nv_bfloat16>(p, s);
  if (p.flags & OT_B200_FP16) return launch_logprob_t<__half>(p, s);
  return launch_logprob_t<float>(p, s);
}

}  // namespace otb
