// Stage 0 (input check + row/cell splits) and stage 2c (per-row gradient
// coefficients + the reduced loss) of the transducer-loss path.
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

// Block 0: the input check and the splits; thread i owns the contiguous
// utterance range [i*per, (i+1)*per).  The other blocks only fill (see below).
__global__ void __launch_bounds__(kPrepThreads)
prepare_kernel(const int32_t *__restrict__ targets, const int32_t *__restrict__ Tl,
               const int32_t *__restrict__ Ul, int N, int64_t rows, int V,
               int max_u, int modified, int64_t max_cells,
               int32_t *__restrict__ status, int64_t *__restrict__ split,
               int64_t *__restrict__ cell_split, uint4 *__restrict__ lp_fill,
               int64_t lp_fill_count, uint4 fill_pattern, int trace, GroupCuts cuts) {
  __shared__ long long scan_buf[kPrepThreads / kWarp];
  __shared__ int warp_maxu[kPrepThreads / kWarp];
  __shared__ int group_count[kMaxGroups + 1];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait();     // the previous call's kernels may still be reading this workspace
  pdl_trigger();
  if (blockIdx.x > 0) {
    // Blocks 1.. set every (blank, symbol) log-prob pair to -inf, 16 bytes at a
    // time.  Stage 1 then overwrites the pairs of real lattice cells; what is
    // left at -inf are the entries of the wavefront-ordered blocks that are no
    // cell, which is exactly the value the recursions need to read there ("no
    // such predecessor").
    const int64_t stride = (int64_t)(gridDim.x - 1) * kPrepThreads;
    for (int64_t i = (int64_t)(blockIdx.x - 1) * kPrepThreads + tid; i < lp_fill_count; i += stride)
      lp_fill[i] = fill_pattern;
    return;
  }
  if (tid < kStatusBlockWords) {
    // trace slots: "first start" begins at the maximum, "last end" at 0
    const bool min_slot = tid >= kTraceWord && tid < kTraceWord + 4 * kTraceSlots && ((tid - kTraceWord) & 3) < 2;
    status[tid] = min_slot ? -1 : (tid == kStatusTraceOn ? trace : 0);
  }
  if (tid <= kMaxGroups) group_count[tid] = 0;
  __syncthreads();
  if (tid == 0) trace_begin(status, kStagePrepare);

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
  int ends_early[kMaxGroups + 1] = {0, 0, 0, 0, 0};  // [g]: my utterances that end at or before cut g
  for (int b = b0; b < b1; ++b) {
    split[b] = run_rows;
    cell_split[b] = run_cells;
    const int tc = max(Tl[b], 0), uc = min(max(Ul[b], 0), max_u);
    run_rows += (long long)tc * (uc + 1);
    run_cells += cell_block(tc, uc, modified != 0);
#pragma unroll
    for (int g = 1; g < kMaxGroups; ++g) ends_early[g] += (g < cuts.n && run_rows <= cuts.row[g]) ? 1 : 0;
  }
  // Utterance ends grow with b, so the count IS the first utterance of group g.
#pragma unroll
  for (int g = 1; g < kMaxGroups; ++g)
    if (ends_early[g]) atomicAdd(&group_count[g], ends_early[g]);
  __syncthreads();
  if (tid <= kMaxGroups && cuts.n > 0)
    status[kStatusGroupSplit + tid] = (tid == 0) ? 0 : (tid < cuts.n ? group_count[tid] : N);
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
  constexpr int kBatch = 8;  // independent loads in flight per thread
  for (long long i0 = tid; i0 < cells; i0 += (long long)kPrepThreads * kBatch) {
    int v[kBatch];
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      const long long i = i0 + (long long)k * kPrepThreads;
      v[k] = (i < cells) ? __ldg(targets + i) : 0;
    }
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      const long long i = i0 + (long long)k * kPrepThreads;
      if (i < cells) {
        const int b = (int)(i / max_u), u = (int)(i % max_u);
        if (v[k] >= V || (v[k] < 0 && u < Ul[b])) raise(status, OT_B200_INPUT_TARGET_RANGE, b);
      }
    }
  }
  if (tid == 0) trace_end(status, kStagePrepare);  // block 0 only: the fill blocks are not waited for
}

// Thread per workspace cell, in the order alpha and beta are stored, so their
// reads are coalesced; the 32-byte (16-byte) record of the cell's row is the
// only scattered access.  Produces what the streaming gradient kernels read.
// Branch order and the order of the floating-point additions follow
// ComputeGradient / ...OneSymPerFrame / ...ForLogSoftmax[OneSymPerFrame]
// (optimized_transducer/csrc/cpu.cc:500-526, 582-604, 655-672, 722-745).
// A non-finite log-likelihood zeroes the utterance's rows
// (optimized_transducer/csrc/kernels.cu:556-563).
//
// Warp 0 of block 0 also closes the forward half: it settles the verdict of the
// call, reduces the scores to the loss
//   *loss_out = loss_scale * -(sum_b scores[b])      (transducer_loss.py:145-152)
// and delivers the optional reports into mapped host memory (the host polls the
// sequence word, or looks at the record of the last failed call: no copy or
// event has to sit in the stream).  The verdict is the input check of stage 0,
// then a bulk-copy wait that ran out in stage 1 or 2, then (only when a report
// is asked for) the reference's consistency check of the two total scores,
// torch::allclose(alpha-total, beta-total) (cpu.cc:795-797: rtol 1e-5, atol
// 1e-8; equal infinities and NaNs pass here, they give zero gradient rows).
// A verdict other than 0 is stored into the status word, so the gradient pass
// writes nothing; the loss becomes NaN, and so do the scores if no recursion
// ran.
template <typename T>
__device__ __forceinline__ T quiet_nan();
template <> __device__ __forceinline__ float quiet_nan<float>() { return __int_as_float(0x7fc00000); }
template <> __device__ __forceinline__ double quiet_nan<double>() { return __longlong_as_double(0x7ff8000000000000LL); }

// Warp 0 of block 0, step 1: the verdict over the utterances [lo, hi) of this
// launch.  Returns it (warp-uniform) and stores it into the status word if it is
// new there.
template <typename T>
__device__ __forceinline__ int settle(int32_t *status, int lo, int hi,
                                      const int64_t *__restrict__ cell_split,
                                      const T *__restrict__ beta, const T *__restrict__ scores,
                                      bool check_totals) {
  const int lane = threadIdx.x;
  int code = status[kStatusCode], index = status[kStatusIndex];
  const int was = code;
  if (code == 0 && status[kStatusCopyTimeout] != 0) {
    code = OT_B200_COPY_TIMEOUT;
    index = status[kStatusCopyTimeout] - 1;
  }
  if (code == 0 && check_totals) {
    int first_bad = 0x7fffffff;
    for (int b = lo + lane; b < hi; b += kWarp) {
      const T a = scores[b];
      const T l = beta[cell_split[b]];  // beta(0,0): the first entry of the utterance's block
      const bool fa = (a - a == (T)0), fl = (l - l == (T)0);
      const bool differ = (fa && fl) ? (fabs((double)a - (double)l) > 1e-8 + 1e-5 * fabs((double)l))
                                     : (fa != fl);
      if (differ && b < first_bad) first_bad = b;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) first_bad = min(first_bad, __shfl_xor_sync(kFull, first_bad, o));
    if (first_bad != 0x7fffffff) { code = OT_B200_TOTALS_DIFFER; index = first_bad; }
  }
  if (lane == 0 && code != was) {
    status[kStatusIndex] = index;
    status[kStatusCode] = code;
  }
  return code;
}

// Step 2, once per call: the loss, NaN scores where no recursion ran, the reports.
template <typename T>
__device__ __forceinline__ void deliver(const int32_t *status, int code, int N, T *__restrict__ scores,
                                        T *__restrict__ loss_out, double loss_scale,
                                        volatile int32_t *report, volatile int32_t *sticky,
                                        int32_t report_seq) {
  const int lane = threadIdx.x;
  double acc = 0;
  if (code == 0) {
    for (int b = lane; b < N; b += kWarp) acc += (double)scores[b];
    acc = warp_sum(acc);
  } else if (code <= OT_B200_INPUT_ONE_SYM_INFEASIBLE) {  // an input error: no recursion ran
    for (int b = lane; b < N; b += kWarp) scores[b] = quiet_nan<T>();
  }
  if (lane == 0) {
    if (loss_out != nullptr) *loss_out = code != 0 ? quiet_nan<T>() : (T)(-acc * loss_scale);
    if (sticky != nullptr && code != 0) {
      sticky[1] = status[kStatusIndex];
      sticky[2] = report_seq;
      __threadfence_system();
      sticky[0] = code;
    }
    if (report != nullptr) {
      report[0] = code;
      report[1] = status[kStatusIndex];
      __threadfence_system();
      report[2] = report_seq;
    }
  }
}

// The closing step alone, for calls that ran as two groups: one warp.
template <typename T>
__global__ void __launch_bounds__(kWarp)
close_kernel(int32_t *status, int N, T *scores, T *__restrict__ loss_out, double loss_scale,
             int32_t *report, int32_t *sticky, int32_t report_seq) {
  pdl_wait();
  pdl_trigger();
  int code = status[kStatusCode];
  if (code == 0 && status[kStatusCopyTimeout] != 0) {
    code = OT_B200_COPY_TIMEOUT;
    if (threadIdx.x == 0) {
      status[kStatusIndex] = status[kStatusCopyTimeout] - 1;
      status[kStatusCode] = code;
    }
    __syncwarp();
  }
  deliver<T>(status, code, N, scores, loss_out, loss_scale, report, sticky, report_seq);
}

template <typename T, bool MODE_B, bool MODIFIED>
__global__ void __launch_bounds__(256)
coef_kernel(const int32_t *__restrict__ targets, const int32_t *__restrict__ Tl,
            const int32_t *__restrict__ Ul, const int64_t *__restrict__ split,
            const int64_t *__restrict__ cell_split,
            int32_t *status, int N, int max_u, int blank,
            const T *__restrict__ den, const T *__restrict__ lp,
            const T *__restrict__ alpha, const T *__restrict__ beta,
            void *__restrict__ coef_out, T *scores,
            T *__restrict__ loss_out, double loss_scale,
            int32_t *report, int32_t *sticky, int32_t report_seq, int group) {
  pdl_wait();
  pdl_trigger();
  const bool bad_input = status[kStatusCode] != 0;
  int lo, hi;
  group_range(status, group, N, lo, hi);
  if (blockIdx.x == 0 && threadIdx.x < kWarp) {
    const int code = settle<T>(status, lo, hi, cell_split, beta, scores, report != nullptr || sticky != nullptr);
    // a call that runs as two groups closes in close_kernel, after both
    if (group < 0) deliver<T>(status, code, N, scores, loss_out, loss_scale, report, sticky, report_seq);
  }
  if (bad_input) return;
  if (threadIdx.x == 0) trace_begin(status, trace_slot(kStageCoef, group));
  const int64_t cell = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  // The chain of dependent loads decides this kernel's time (thousands of small
  // blocks, each a few L2 round trips long), so it is kept at three: (1) the
  // per-utterance tables of the whole batch into shared memory, one coalesced
  // pass; (2) every per-cell value the record can need, all requested at once;
  // (3) the store.  Batches of more than kMetaMax utterances read the tables
  // from global memory instead.
  constexpr int kMetaMax = 512;
  __shared__ int64_t s_csplit[kMetaMax + 1];
  __shared__ int64_t s_split[kMetaMax];
  __shared__ int32_t s_T[kMetaMax], s_U[kMetaMax];
  const bool meta = N <= kMetaMax;
  if (meta) {
    for (int i = threadIdx.x; i <= N; i += blockDim.x) {
      s_csplit[i] = __ldg(cell_split + i);
      if (i < N) { s_split[i] = __ldg(split + i); s_T[i] = __ldg(Tl + i); s_U[i] = __ldg(Ul + i); }
    }
    __syncthreads();
  }
  const int64_t *cs = meta ? s_csplit : cell_split;
  if (cell < cs[lo] || cell >= cs[hi]) return;  // not a cell of this launch's utterances
  const int b = meta ? find_utt_plain(s_csplit, N, cell) : find_utt(cell_split, N, cell);
  const int64_t coff = cs[b];
  const int Tn = meta ? s_T[b] : __ldg(Tl + b), U = meta ? s_U[b] : __ldg(Ul + b), U1 = U + 1;
  const int64_t p = cell - coff;
  int t, u;
  if (MODIFIED) {
    t = (int)(p / U1); u = (int)(p - (int64_t)t * U1);
    if (t >= Tn) return;  // rounding pad of the block
  } else {
    const int d = (int)(p / U1);
    u = (int)(p - (int64_t)d * U1);
    t = d - u;
    if (t < 0 || t >= Tn) return;  // no lattice cell is stored here
  }
  const int64_t row = (meta ? s_split[b] : __ldg(split + b)) + (int64_t)t * U1 + u;
  const int diff = Tn - 1 - U;
  const bool off_band = MODIFIED && (u > t || t - u > diff);
  const bool last = (t == Tn - 1 && u == U);
  const bool blank_ok = MODIFIED ? (t - u < diff) : (t < Tn - 1);
  // successors: blank -> (t+1,u), symbol -> (t,u+1) or (t+1,u+1) if modified;
  // in both storage orders they sit U1 and U1+1 entries further.  Which of them
  // exist depends on (t, u) alone, so all loads go out together.
  const bool live = !off_band;
  const T L = beta[coff];  // beta(0,0) is the first entry in both layouts
  const T a_here = live ? alpha[cell] : (T)0;
  const T b_here_v = live ? beta[cell] : (T)0;
  const T den_v = (live && !MODE_B) ? den[row] : (T)0;
  const int target_u = (live && u < U) ? __ldg(targets + (int64_t)b * max_u + u) : -1;
  const T b_sym_next = (live && u < U) ? beta[cell + U1 + 1] : neg_inf<T>();
  const T b_blank_next = (live && !last && blank_ok) ? beta[cell + U1] : neg_inf<T>();
  T lp_b = 0, lp_s = 0;
  if (MODE_B && live) { lp_b = lp[2 * cell]; lp_s = lp[2 * cell + 1]; }

  const bool zero = off_band || !(L - L == (T)0);  // off the band, or an infinite / NaN likelihood

  T c = 0, b_here = 0, sub_blank = neg_inf<T>(), sub_sym = neg_inf<T>();
  int32_t tgt = kTgtNone;
  bool blank_term = false, sym_term = false;
  if (!zero) {
    const T loss = -L;
    c = a_here + loss;
    if (!MODE_B) c = c - den_v;
    b_here = b_here_v;
    if (last) {
      sub_blank = 0; blank_term = true;
    } else if (blank_ok) {
      sub_blank = b_blank_next; blank_term = true;
    } else if (u < U && target_u == blank) {
      sub_blank = b_sym_next; blank_term = true;
    }
    if (u < U && target_u != blank) {
      sub_sym = b_sym_next; tgt = target_u; sym_term = true;
    }
  }
  if (MODE_B) {
    CoefB<T> r;
    r.val_blank = blank_term ? -r_exp((lp_b + c) + sub_blank) : (T)0;
    r.val_sym = sym_term ? -r_exp((lp_s + c) + sub_sym) : (T)0;
    r.tgt = zero ? kTgtZeroRow : tgt;
    r.utt = b;
    reinterpret_cast<CoefB<T> *>(coef_out)[row] = r;
  } else {
    CoefA<T> r;
    r.c = c; r.beta = b_here; r.sub_blank = sub_blank; r.sub_sym = sub_sym;
    r.tgt = zero ? kTgtZeroRow : tgt;
    r.utt = b;
    reinterpret_cast<CoefA<T> *>(coef_out)[row] = r;
  }
  if (threadIdx.x == 0) trace_end(status, trace_slot(kStageCoef, group));  // one thread per block: cheap, close enough
}

template <typename T>
cudaError_t launch_coef_t(const Problem &p, void *scores, void *loss_out,
                          double loss_scale, cudaStream_t s) {
  const bool mode_b = p.flags & OT_B200_FROM_LOG_SOFTMAX;
  const bool modified = p.flags & OT_B200_ONE_SYM_PER_FRAME;
  int32_t *status = reinterpret_cast<int32_t *>(p.ws + p.lay.status);
  const int64_t *split = reinterpret_cast<const int64_t *>(p.ws + p.lay.split);
  const int64_t *csplit = reinterpret_cast<const int64_t *>(p.ws + p.lay.cell_split);
  const T *den = reinterpret_cast<const T *>(p.ws + p.lay.den);
  const T *lp = reinterpret_cast<const T *>(p.ws + p.lay.lp);
  const T *alpha = reinterpret_cast<const T *>(p.ws + p.lay.alpha);
  const T *beta = reinterpret_cast<const T *>(p.ws + p.lay.beta);
  void *coef = p.ws + p.lay.coef;
  const unsigned grid = (unsigned)((p.lay.max_cells + 255) / 256);
  cudaError_t e = cudaSuccess;
  // A group launch sits on the high-priority stream behind the group's recursion:
  // an ordinary launch there (see launch_maybe_pdl).
#define OTB_COEF(MB, MOD)                                                        \
  e = launch_maybe_pdl(p.group < 0, coef_kernel<T, MB, MOD>, grid, 256u, 0, s, p.targets, p.T, p.U, split,   \
      csplit, status, p.N, p.max_u, p.blank, den, lp, alpha, beta, coef,         \
      static_cast<T *>(scores), static_cast<T *>(loss_out), loss_scale,          \
      p.report, p.sticky, p.report_seq, p.group)
  if (mode_b) { if (modified) OTB_COEF(true, true); else OTB_COEF(true, false); }
  else        { if (modified) OTB_COEF(false, true); else OTB_COEF(false, false); }
#undef OTB_COEF
  return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace

cudaError_t launch_prepare(const Problem &p, cudaStream_t s) {
  // lp holds max_cells pairs; in 16-byte units that is max_cells/2 (float) or
  // max_cells (double) stores of the -inf bit pattern.
  const bool fp64 = p.flags & OT_B200_FP64;
  const int64_t units = fp64 ? p.lay.max_cells : (p.lay.max_cells + 1) / 2;
  uint4 pattern;
  if (fp64) { pattern.x = 0u; pattern.y = 0xfff00000u; pattern.z = 0u; pattern.w = 0xfff00000u; }
  else { pattern.x = pattern.y = pattern.z = pattern.w = 0xff800000u; }
  int64_t fill_blocks = (units + kPrepThreads * 8 - 1) / (kPrepThreads * 8);
  const int64_t cap = 2 * (int64_t)sm_count();
  if (fill_blocks > cap) fill_blocks = cap;
  // Launched like the later stages: when the previous kernel in the stream is
  // this library's gradient pass (training loops), the blocks are resident when
  // it drains; behind any other kernel the attribute changes nothing.
  const cudaError_t e = launch_pdl(prepare_kernel, (unsigned)(1 + fill_blocks), (unsigned)kPrepThreads, 0, s,
      p.targets, p.T, p.U, p.N, p.rows, p.V, p.max_u,
      (p.flags & OT_B200_ONE_SYM_PER_FRAME) ? 1 : 0, p.lay.max_cells,
      reinterpret_cast<int32_t *>(p.ws + p.lay.status),
      reinterpret_cast<int64_t *>(p.ws + p.lay.split),
      reinterpret_cast<int64_t *>(p.ws + p.lay.cell_split),
      reinterpret_cast<uint4 *>(p.ws + p.lay.lp), units, pattern,
      (p.flags & OT_B200_TRACE) ? 1 : 0, p.cuts);
  return e != cudaSuccess ? e : cudaGetLastError();
}

cudaError_t launch_coef(const Problem &p, void *scores, void *loss_out,
                        double loss_scale, cudaStream_t s) {
  return (p.flags & OT_B200_FP64) ? launch_coef_t<double>(p, scores, loss_out, loss_scale, s)
                                  : launch_coef_t<float>(p, scores, loss_out, loss_scale, s);
}

cudaError_t launch_close(const Problem &p, void *scores, void *loss_out, double loss_scale,
                         cudaStream_t s) {
  int32_t *status = reinterpret_cast<int32_t *>(p.ws + p.lay.status);
  cudaError_t e;
  if (p.flags & OT_B200_FP64)
    e = launch_pdl(close_kernel<double>, 1u, (unsigned)kWarp, 0, s, status, p.N, static_cast<double *>(scores),
                   static_cast<double *>(loss_out), loss_scale, p.report, p.sticky, p.report_seq);
  else
    e = launch_pdl(close_kernel<float>, 1u, (unsigned)kWarp, 0, s, status, p.N, static_cast<float *>(scores),
                   static_cast<float *>(loss_out), loss_scale, p.report, p.sticky, p.report_seq);
  return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace otb
