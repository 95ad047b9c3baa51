// Stage 3: the gradient w.r.t. the packed logits, one streaming pass.
//
// Mode A (raw logits; may write in place over the logits) replaces
// ComputeGradient / ComputeGradientOneSymPerFrame
// (optimized_transducer/csrc/kernels.cu:522-651): per row, with the
// coefficients (c, beta, sub_blank, sub_sym, tgt) of stage 2c,
//     grad[v] = scale * ( exp((x[v]+c)+beta) - [v==blank] exp((x[v]+c)+sub_blank)
//                                            - [v==tgt]   exp((x[v]+c)+sub_sym) )
// The additions are made in the reference's order (cpu.cc:509-522) so that the
// rounding of x[v]+c, which dominates the error for long utterances, is the
// same as the reference's.
//
// Mode B (log-softmax input) replaces ComputeGradientForLogSoftmax /
// ...OneSymPerFrame (kernels.cu:653-779): rows are zero except for the blank
// and symbol entries, so the kernel only writes.
//
// `scale` folds the two elementwise passes of the reference's Python layer
// (division by N for reduction="mean", multiplication by the upstream
// gradient; transducer_loss.py:150,162) into this pass.
//
// Mode A: one warp per row, one short-lived block per 8 rows (OT_B200_GRID=wave:
// one resident wave that strides); rows are visited from the END of the buffer
// towards its start: the rows stage 1 read last are the ones still resident in
// L2.  Mode B is written as one front of 2 KB chunks.  HBM traffic per row:
// V*sizeof(X) read + V*sizeof(X) written (mode A), V*sizeof(X) written (mode B),
// plus one 32-byte (16-byte) coefficient record.

#include <stdlib.h>
#include <string.h>

#include "ot_common.cuh"

namespace otb {

namespace {

constexpr int kThreads = 256;

template <typename T>
__device__ __forceinline__ CoefA<T> load_coef(const CoefA<T> *p) {
  // Every lane reads the same record: the loads are broadcasts.
  CoefA<T> r;
  if constexpr (sizeof(T) == 4) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p));
    r.c = a.x; r.beta = a.y; r.sub_blank = a.z; r.sub_sym = a.w;
    const int2 i = __ldg(reinterpret_cast<const int2 *>(p) + 2);
    r.tgt = i.x; r.utt = i.y;
  } else {
    const double2 a = __ldg(reinterpret_cast<const double2 *>(p));
    const double2 b = __ldg(reinterpret_cast<const double2 *>(p) + 1);
    r.c = a.x; r.beta = a.y; r.sub_blank = b.x; r.sub_sym = b.y;
    const int2 i = __ldg(reinterpret_cast<const int2 *>(p) + 4);
    r.tgt = i.x; r.utt = i.y;
  }
  return r;
}

// X: storage type of logits and gradient, T = Real<X>: type of the arithmetic.
// PER_UTT: d_scale holds one factor per utterance instead of one scalar.
template <typename X, int VEC, int CH, bool PER_UTT, int MINB = 5>
__global__ void __launch_bounds__(kThreads, MINB)
gradient_kernel(const X *x, X *g, const CoefA<typename Real<X>::type> *__restrict__ coef,
                const int32_t *__restrict__ status, int64_t rows, int V,
                int blank, const typename Real<X>::type *__restrict__ d_scale,
                typename Real<X>::type scale_host, bool eager,
                const int64_t *__restrict__ split, int N, int group) {
  pdl_wait();
  pdl_trigger();
  if (status[kStatusCode] != 0) return;
  // The rows of this launch: all of them, or those of one group of utterances.
  int64_t row_lo = 0;
  if (group >= 0) {
    int lo, hi;
    group_range(status, group, N, lo, hi);
    row_lo = __ldg(split + lo);
    rows = __ldg(split + hi);
  }
  if (threadIdx.x == 0) trace_begin(status, trace_slot(kStageGradient, group));
  using T = typename Real<X>::type;
  using VT = typename VecOf<X, VEC>::type;
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const int nvec = V / VEC;
  const T scale_all = (!PER_UTT && d_scale) ? scale_host * __ldg(d_scale) : scale_host;
  const int bvec = blank / VEC, bk = blank % VEC;

  for (int64_t row = rows - 1 - warp0; row >= row_lo; row -= nwarps) {
    const CoefA<T> rec = load_coef(coef + row);
    const T scale = PER_UTT ? scale_host * __ldg(d_scale + rec.utt) : scale_all;
    const X *px = x + row * (int64_t)V;
    X *pg = g + row * (int64_t)V;
    VT v[CH];
    // The first chunk of the row is requested before the record is looked at, so
    // the two round trips overlap.  (`eager` is off for the band-limited
    // recursion, whose many zero rows would then be read for nothing.)
    if (eager) {
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int vi = j * kWarp + lane;
        if (vi < nvec) v[j] = *reinterpret_cast<const VT *>(px + (int64_t)vi * VEC);
      }
    }
    if (rec.tgt == kTgtZeroRow) {
      VT z;
      X *ze = reinterpret_cast<X *>(&z);
#pragma unroll
      for (int k = 0; k < VEC; ++k) ze[k] = from_real<X>((T)0);
      for (int vi = lane; vi < nvec; vi += kWarp)
        *reinterpret_cast<VT *>(pg + (int64_t)vi * VEC) = z;
      continue;
    }
    const int tvec = rec.tgt >= 0 ? rec.tgt / VEC : -1;
    const int tk = rec.tgt >= 0 ? rec.tgt % VEC : 0;
    [[maybe_unused]] const float k2 = (float)((rec.c + rec.beta) * (T)kLog2e);  // 16-bit rows, see below
    for (int base = 0; base < nvec; base += kWarp * CH) {
      if (!(eager && base == 0)) {
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          const int vi = base + j * kWarp + lane;
          if (vi < nvec) v[j] = *reinterpret_cast<const VT *>(px + (int64_t)vi * VEC);
        }
      }
      // The 16-bit pass is bound by instruction issue, not by bytes (half the bytes
      // per element, the same arithmetic), so the two columns with a second term
      // are kept out of the common code: their logits are taken out of the
      // registers of the lanes that hold them (warp-uniform branches, one shuffle
      // each), every element then takes the one-term formula, and the two lanes
      // store their corrected element after their vector.  Same operations on
      // those elements as in the general code, so the same bits.
      X fix_b = from_real<X>((T)0), fix_t = from_real<X>((T)0);
      bool own_b = false, own_t = false;
      if constexpr (sizeof(X) == 2) {
        const auto take = [&](int vec, int k) {  // logit k of vector `vec` of this chunk
          const int jj = (vec - base) >> 5;
          VT cand = v[0];
#pragma unroll
          for (int j = 1; j < CH; ++j)
            if (j == jj) cand = v[j];
          const X *ce = reinterpret_cast<const X *>(&cand);
          X xs = ce[0];
#pragma unroll
          for (int q = 1; q < VEC; ++q)
            if (q == k) xs = ce[q];
          return __shfl_sync(kFull, to_real(xs), (vec - base) & 31);
        };
        if (bvec >= base && bvec < base + kWarp * CH && bvec < nvec) {
          const T gv = take(bvec, bk) + rec.c;
          fix_b = from_real<X>((s_exp(gv + rec.beta) - s_exp(gv + rec.sub_blank)) * scale);
          own_b = ((bvec - base) & 31) == lane;
        }
        if (tvec >= base && tvec < base + kWarp * CH && !(tvec == bvec && tk == bk)) {
          const T gv = take(tvec, tk) + rec.c;
          fix_t = from_real<X>((s_exp(gv + rec.beta) - s_exp(gv + rec.sub_sym)) * scale);
          own_t = ((tvec - base) & 31) == lane;
        }
      }
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int vi = base + j * kWarp + lane;
        if (vi < nvec) {
          X *e = reinterpret_cast<X *>(&v[j]);
          if constexpr (sizeof(X) == 2 && VEC == 4) {
            // One FFMA, one ex2, one multiply per element and one conversion per
            // pair: the row's constants are folded, 2^(x*log2e + (c+beta)*log2e).
            // (Folding c + beta rounds once at the magnitude of the log-likelihood,
            // as x + c does in the float pass; far below half an ulp of a 16-bit result.)
            uint32_t *w = reinterpret_cast<uint32_t *>(&v[j]);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const float2 a = Pair16<X>::widen(w[h]);
              w[h] = Pair16<X>::round(ex2_approx(fmaf(a.x, kLog2e, k2)) * scale,
                                      ex2_approx(fmaf(a.y, kLog2e, k2)) * scale);
            }
          } else if constexpr (sizeof(X) == 2) {
#pragma unroll
            for (int k = 0; k < VEC; ++k)
              e[k] = from_real<X>(s_exp((to_real(e[k]) + rec.c) + rec.beta) * scale);
          } else {
            const int bsel = (vi == bvec) ? bk : -1;
            const int tsel = (vi == tvec) ? tk : -1;
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
              const T gv = to_real(e[k]) + rec.c;
              T val = s_exp(gv + rec.beta);
              if (k == bsel) val -= s_exp(gv + rec.sub_blank);
              else if (k == tsel) val -= s_exp(gv + rec.sub_sym);
              e[k] = from_real<X>(val * scale);
            }
          }
          *reinterpret_cast<VT *>(pg + (int64_t)vi * VEC) = v[j];
        }
      }
      if constexpr (sizeof(X) == 2) {
        // after the vector stores of the same thread, so these land on top
        if (own_b) pg[blank] = fix_b;
        if (own_t) pg[rec.tgt] = fix_t;
      }
    }
  }
  if (threadIdx.x == 0) trace_end(status, trace_slot(kStageGradient, group));
}

// The same pass for 16-bit rows of at most 512 columns (V % 4 == 0, 8-byte
// aligned rows), software-pipelined.  A 16-bit row is half as many bytes per warp
// as a float row, so with one row per warp in flight the pass waits on memory
// latency (measured: 5.1 TB/s, long-scoreboard stalls, DRAM half idle).  Here a
// warp requests its NEXT row (record and vectors) before it works on the current
// one, which doubles the bytes it keeps in flight; one resident wave of blocks
// strides over the buffer from its end, so the next row is known.  Arithmetic:
// one FFMA, one ex2 and one multiply per element with the row's constants folded
// (2^(x*log2e + (c+beta)*log2e + log2 scale)), one conversion per pair; the two
// columns that carry a second term get a per-row factor (see `finish`).
template <typename X, bool PER_UTT>
__global__ void __launch_bounds__(kThreads, 5)
gradient16_kernel(const X *x, X *g, const CoefA<float> *__restrict__ coef,
                  const int32_t *__restrict__ status, int64_t rows, int V, int blank,
                  const float *__restrict__ d_scale, float scale_host,
                  const int64_t *__restrict__ split, int N, int group) {
  pdl_wait();
  pdl_trigger();
  if (status[kStatusCode] != 0) return;
  int64_t row_lo = 0;
  if (group >= 0) {
    int lo, hi;
    group_range(status, group, N, lo, hi);
    row_lo = __ldg(split + lo);
    rows = __ldg(split + hi);
  }
  if (threadIdx.x == 0) trace_begin(status, trace_slot(kStageGradient, group));
  constexpr int CH = 4;  // vectors of 4 elements per lane: 512 columns
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const int nvec = V >> 2;
  const float scale_all = (!PER_UTT && d_scale) ? scale_host * __ldg(d_scale) : scale_host;
  const int b_lane = (blank >> 2) & 31, b_j = blank >> 7, b_k = blank & 3;

  const auto fetch = [&](int64_t row, CoefA<float> &rec, uint2 (&v)[CH]) {
    rec = load_coef(coef + row);
    const uint2 *px = reinterpret_cast<const uint2 *>(x + row * (int64_t)V);
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      const int vi = j * kWarp + lane;
      if (vi < nvec) v[j] = px[vi];
    }
  };
  // One row.  FOLD: the scale is positive and finite, so it moves into the exponent
  // (scale * 2^y = 2^(y + log2 scale)) and the multiply per element disappears.
  // The two columns that carry a second term: with y = scale * exp(x + c + beta)
  // already computed for every element,
  //     scale * (exp(x+c+beta) - exp(x+c+sub)) = y * (1 - exp(sub - beta)),
  // so the row needs two factors (warp-uniform, one ex2 each) and the lane that
  // owns such a column multiplies its element before it is rounded; where that
  // element sits (vector, word, half) is warp-uniform, so the patch is a uniform
  // branch taken once per row, not a select per element.
  const auto finish = [&](int64_t row, const CoefA<float> &rec, uint2 (&v)[CH]) {
    uint2 *pg = reinterpret_cast<uint2 *>(g + row * (int64_t)V);
    if (rec.tgt == kTgtZeroRow) {
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int vi = j * kWarp + lane;
        if (vi < nvec) pg[vi] = make_uint2(0u, 0u);  // +0 in both 16-bit formats
      }
      return;
    }
    const float scale = PER_UTT ? scale_host * __ldg(d_scale + rec.utt) : scale_all;
    const bool fold = scale > 0.f && scale < 3.0e38f;
    const float mul = fold ? 1.f : scale;
    const float k2 = (rec.c + rec.beta) * kLog2e + (fold ? __log2f(scale) : 0.f);
    const bool reachable = rec.beta > neg_inf<float>();  // else every term of the row is 0
    const float f_b = reachable ? 1.f - ex2_approx((rec.sub_blank - rec.beta) * kLog2e) : 1.f;
    const float f_t = reachable ? 1.f - ex2_approx((rec.sub_sym - rec.beta) * kLog2e) : 1.f;
    const int t_j = rec.tgt >= 0 ? rec.tgt >> 7 : -1, t_lane = (rec.tgt >> 2) & 31, t_k = rec.tgt & 3;
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      const int vi = j * kWarp + lane;
      if (vi < nvec) {
        const float2 a = Pair16<X>::widen(v[j].x), b = Pair16<X>::widen(v[j].y);
        float y0 = ex2_approx(fmaf(a.x, kLog2e, k2)), y1 = ex2_approx(fmaf(a.y, kLog2e, k2));
        float y2 = ex2_approx(fmaf(b.x, kLog2e, k2)), y3 = ex2_approx(fmaf(b.y, kLog2e, k2));
        if (!fold) { y0 *= mul; y1 *= mul; y2 *= mul; y3 *= mul; }  // uniform: rare
        if (j == b_j) {  // uniform: the vector that holds the blank column
          const float f = lane == b_lane ? f_b : 1.f;
          y0 *= b_k == 0 ? f : 1.f; y1 *= b_k == 1 ? f : 1.f; y2 *= b_k == 2 ? f : 1.f; y3 *= b_k == 3 ? f : 1.f;
        }
        if (j == t_j) {  // uniform: the vector that holds the target column
          const float f = lane == t_lane ? f_t : 1.f;
          y0 *= t_k == 0 ? f : 1.f; y1 *= t_k == 1 ? f : 1.f; y2 *= t_k == 2 ? f : 1.f; y3 *= t_k == 3 ? f : 1.f;
        }
        pg[vi] = make_uint2(Pair16<X>::round(y0, y1), Pair16<X>::round(y2, y3));
      }
    }
  };

  // Two register sets alternate between "being fetched" and "being finished".
  CoefA<float> rec_a, rec_b;
  uint2 va[CH], vb[CH];
  int64_t row = rows - 1 - warp0;
  if (row >= row_lo) fetch(row, rec_a, va);
  while (row >= row_lo) {
    const int64_t next = row - nwarps;
    if (next >= row_lo) fetch(next, rec_b, vb);
    finish(row, rec_a, va);
    if (next < row_lo) break;
    const int64_t after = next - nwarps;
    if (after >= row_lo) fetch(after, rec_a, va);
    finish(next, rec_b, vb);
    row = after;
  }
  if (threadIdx.x == 0) trace_end(status, trace_slot(kStageGradient, group));
}

template <typename X, int VEC, bool PER_UTT>
__global__ void __launch_bounds__(kThreads)
gradient_logsoftmax_kernel(X *__restrict__ g, const CoefB<typename Real<X>::type> *__restrict__ coef,
                           const int32_t *__restrict__ status, int64_t rows,
                           int V, int blank, const typename Real<X>::type *__restrict__ d_scale,
                           typename Real<X>::type scale_host) {
  pdl_wait();
  pdl_trigger();
  if (status[kStatusCode] != 0) return;
  using T = typename Real<X>::type;
  using VT = typename VecOf<X, VEC>::type;
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const int nvec = V / VEC;
  const T scale_all = (!PER_UTT && d_scale) ? scale_host * __ldg(d_scale) : scale_host;
  const int bvec = blank / VEC, bk = blank % VEC;
  // The output is written as ONE front that moves through memory: a warp takes
  // chunks of kChunk consecutive vectors of the flattened (rows x nvec) array,
  // consecutive warps take consecutive chunks.  (A warp per row would, for long
  // rows, keep thousands of fronts open that are a row pitch apart, which costs
  // DRAM page locality: 5.5 instead of 7 TB/s at V = 5000.)
  constexpr int kPer = 4, kChunk = kWarp * kPer;
  const int64_t total = rows * (int64_t)nvec;
  const int64_t nchunks = (total + kChunk - 1) / kChunk;
  for (int64_t chunk = warp0; chunk < nchunks; chunk += nwarps) {
    const int64_t first = chunk * kChunk;
    const int64_t row0 = first / nvec;
    const int col0 = (int)(first - row0 * nvec);
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int64_t g_index = first + j * kWarp + lane;
      if (g_index >= total) break;
      int64_t row = row0;
      int vi = col0 + j * kWarp + lane;
      while (vi >= nvec) { vi -= nvec; ++row; }
      const CoefB<T> rec = coef[row];  // 16 bytes shared by a whole row: L1 hits
      const bool zero = rec.tgt == kTgtZeroRow;
      const int tvec = (!zero && rec.tgt >= 0) ? rec.tgt / VEC : -1;
      VT z;
      X *ze = reinterpret_cast<X *>(&z);
#pragma unroll
      for (int k = 0; k < VEC; ++k) ze[k] = from_real<X>((T)0);
      if ((vi == bvec && !zero) || vi == tvec) {  // at most two vectors of a row are not all zero
        const T scale = PER_UTT ? scale_host * __ldg(d_scale + rec.utt) : scale_all;
        const int tk = rec.tgt >= 0 ? rec.tgt % VEC : 0;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          T val = 0;
          if (!zero && vi == bvec && k == bk) val = rec.val_blank * scale;
          else if (vi == tvec && k == tk) val = rec.val_sym * scale;
          ze[k] = from_real<X>(val);
        }
      }
      *reinterpret_cast<VT *>(g + g_index * VEC) = z;
    }
  }
  if (threadIdx.x == 0) trace_end(status, kStageGradient);
}

// Blocks for `units` warp-sized units of work (8 per block): all of them, or,
// with OT_B200_GRID=wave, at most one resident wave (the kernels loop).
template <typename K>
unsigned stream_grid(K kernel, std::atomic<int> *per_sm_cache, int64_t units, uint32_t flags, bool one_wave = false) {
  int64_t want = (units + (kThreads / kWarp) - 1) / (kThreads / kWarp);
  if (want < 1) want = 1;
  if (one_wave || wave_grids()) {
    int per_sm = per_sm_cache->load(std::memory_order_relaxed);
    if (per_sm == 0) {
      per_sm = blocks_per_sm(kernel, kThreads);
      per_sm_cache->store(per_sm, std::memory_order_relaxed);
    }
    const int64_t cap = (int64_t)resident_sms(flags) * per_sm;
    if (want > cap) want = cap;
  }
  return (unsigned)(want < 0x7fffffff ? want : 0x7fffffff);
}

template <typename X, int VEC, int CH, bool PER_UTT>
cudaError_t launch_grad_a2(const Problem &p, void *grad, const void *d_scale,
                           double scale_host, cudaStream_t s) {
  using T = typename Real<X>::type;
  static std::atomic<int> per_sm{0};
  // Six resident blocks per SM (40 registers) for the vectorised passes: with
  // short-lived blocks the bytes in flight are (resident warps) x (one row), and
  // the step from 5 to 6 blocks took the float pass from 436 to 408 us on
  // 686 128 rows of 500; 7 or 8 blocks need spills and are slower (488 us).  The
  // 16-bit pass waits on memory latency most of the time once the two special
  // columns are out of its common code, and gains too (292 -> 277 us).
  constexpr int kMinBlocks = ((sizeof(X) == 4 || sizeof(X) == 2) && VEC == 4) ? 6 : (sizeof(X) == 8 ? 3 : 5);
  auto kernel = gradient_kernel<X, VEC, CH, PER_UTT, kMinBlocks>;
  // 16-bit rows are half as many bytes per warp; there one resident wave that
  // strides over the buffer measured faster (277 against 289 us on bf16 cfg2).
  // A group launch is sized for the rows between the group's cuts, which the group
  // cannot exceed by much (its first utterance may begin before the cut): the
  // kernel strides, so a few blocks take a second row.
  const int64_t span = p.group >= 0 ? p.cuts.row[p.group + 1] - p.cuts.row[p.group] : p.rows;
  const cudaError_t e = launch_pdl(kernel,
      stream_grid(kernel, &per_sm, span > 0 ? span : 1, p.flags, sizeof(X) == 2), (unsigned)kThreads, 0, s,
      static_cast<const X *>(p.logits), static_cast<X *>(grad),
      reinterpret_cast<const CoefA<T> *>(p.ws + p.lay.coef),
      reinterpret_cast<const int32_t *>(p.ws + p.lay.status), p.rows, p.V,
      p.blank, static_cast<const T *>(d_scale), (T)scale_host,
      (p.flags & OT_B200_ONE_SYM_PER_FRAME) == 0,
      reinterpret_cast<const int64_t *>(p.ws + p.lay.split), p.N, p.group);
  return e != cudaSuccess ? e : cudaGetLastError();
}

// OT_B200_GRAD16=plain keeps the general kernel for 16-bit rows (for comparison).
bool grad16_plain_forced() {
  const char *e = getenv("OT_B200_GRAD16");
  return e && strcmp(e, "plain") == 0;
}

template <typename X, bool PER_UTT>
cudaError_t launch_grad16(const Problem &p, void *grad, const void *d_scale, double scale_host,
                          cudaStream_t s) {
  static std::atomic<int> per_sm{0};
  auto kernel = gradient16_kernel<X, PER_UTT>;
  unsigned grid = stream_grid(kernel, &per_sm, p.rows, p.flags, true);
  if (p.group >= 0 && p.group + 1 < p.cuts.n) {
    // In a grouped call the next group's recursion and coefficient kernels must
    // find room UNDER this resident wave (measured with five blocks per SM: the
    // coefficient kernel of group b started 42 us late, when the first blocks of
    // this kernel retired): leave one block slot per SM free.  The last group's
    // pass has nothing to make room for and keeps the full wave (four blocks per
    // SM cost 139 us per half of the benchmark batch against 123 us).
    const int blocks = per_sm.load(std::memory_order_relaxed);
    if (blocks > 1) {
      const unsigned smaller = (unsigned)(sm_count() * (blocks - 1));
      if (grid > smaller) grid = smaller;
    }
  }
  const cudaError_t e = launch_pdl(kernel, grid,
      (unsigned)kThreads, 0, s, static_cast<const X *>(p.logits), static_cast<X *>(grad),
      reinterpret_cast<const CoefA<float> *>(p.ws + p.lay.coef),
      reinterpret_cast<const int32_t *>(p.ws + p.lay.status), p.rows, p.V, p.blank,
      static_cast<const float *>(d_scale), (float)scale_host,
      reinterpret_cast<const int64_t *>(p.ws + p.lay.split), p.N, p.group);
  return e != cudaSuccess ? e : cudaGetLastError();
}

template <typename X, int VEC, int CH>
cudaError_t launch_grad_a(const Problem &p, void *grad, const void *d_scale,
                          double scale_host, cudaStream_t s) {
  if constexpr (sizeof(X) == 2 && VEC == 4) {
    if (p.V <= 512 && !grad16_plain_forced())
      return (p.flags & OT_B200_SCALE_PER_UTTERANCE) ? launch_grad16<X, true>(p, grad, d_scale, scale_host, s)
                                                     : launch_grad16<X, false>(p, grad, d_scale, scale_host, s);
  }
  return (p.flags & OT_B200_SCALE_PER_UTTERANCE)
             ? launch_grad_a2<X, VEC, CH, true>(p, grad, d_scale, scale_host, s)
             : launch_grad_a2<X, VEC, CH, false>(p, grad, d_scale, scale_host, s);
}

template <typename X, int VEC, bool PER_UTT>
cudaError_t launch_grad_b(const Problem &p, void *grad, const void *d_scale,
                          double scale_host, cudaStream_t s) {
  using T = typename Real<X>::type;
  static std::atomic<int> per_sm{0};
  auto kernel = gradient_logsoftmax_kernel<X, VEC, PER_UTT>;
  const int64_t chunks = (p.rows * (int64_t)(p.V / VEC) + 127) / 128;  // 128 vectors per warp, see the kernel
  kernel<<<stream_grid(kernel, &per_sm, chunks, p.flags), kThreads, 0, s>>>(
      static_cast<X *>(grad), reinterpret_cast<const CoefB<T> *>(p.ws + p.lay.coef),
      reinterpret_cast<const int32_t *>(p.ws + p.lay.status), p.rows, p.V, p.blank,
      static_cast<const T *>(d_scale), (T)scale_host);
  return cudaGetLastError();
}

template <typename X>
cudaError_t launch_gradient_t(const Problem &p, void *grad, const void *d_scale,
                              double scale_host, cudaStream_t s) {
  constexpr int VEC = Vec16<X>::n;
  constexpr uintptr_t kAlign = VEC * sizeof(X);
  const bool aligned = (p.V % VEC == 0) &&
                       (reinterpret_cast<uintptr_t>(grad) % kAlign == 0);
  if (p.flags & OT_B200_FROM_LOG_SOFTMAX) {
    const bool per_utt = p.flags & OT_B200_SCALE_PER_UTTERANCE;
    if (aligned)
      return per_utt ? launch_grad_b<X, VEC, true>(p, grad, d_scale, scale_host, s)
                     : launch_grad_b<X, VEC, false>(p, grad, d_scale, scale_host, s);
    return per_utt ? launch_grad_b<X, 1, true>(p, grad, d_scale, scale_host, s)
                   : launch_grad_b<X, 1, false>(p, grad, d_scale, scale_host, s);
  }
  const bool vec_ok = aligned && (reinterpret_cast<uintptr_t>(p.logits) % kAlign == 0);
  if (vec_ok) {
    const int per_lane = (p.V / VEC + kWarp - 1) / kWarp;
    if (per_lane <= 1) return launch_grad_a<X, VEC, 1>(p, grad, d_scale, scale_host, s);
    if (per_lane <= 2) return launch_grad_a<X, VEC, 2>(p, grad, d_scale, scale_host, s);
    return launch_grad_a<X, VEC, 4>(p, grad, d_scale, scale_host, s);
  }
  const int per_lane = (p.V + kWarp - 1) / kWarp;
  if (per_lane <= 4) return launch_grad_a<X, 1, 4>(p, grad, d_scale, scale_host, s);
  return launch_grad_a<X, 1, 8>(p, grad, d_scale, scale_host, s);
}

// g *= *d_scale, unless the factor is exactly 1: then every block returns after
// one load and the buffer is not touched.  The counterpart of the reference's
// `ctx.grad.mul_(loss_grad)` (transducer_loss.py:162) for a gradient that was
// computed eagerly: the usual upstream gradient of a loss is 1.
template <typename X>
__global__ void __launch_bounds__(kThreads)
scale_gradient_kernel(X *__restrict__ g, int64_t count, const typename Real<X>::type *__restrict__ d_scale) {
  using T = typename Real<X>::type;
  const T scale = __ldg(d_scale);
  if (scale == (T)1) return;
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  const int64_t first = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  constexpr int VEC = 16 / (int)sizeof(X);
  if (reinterpret_cast<uintptr_t>(g) % 16 == 0) {
    const int64_t nvec = count / VEC;
    uint4 *gv = reinterpret_cast<uint4 *>(g);
    for (int64_t i = first; i < nvec; i += stride) {
      uint4 v = gv[i];
      X *e = reinterpret_cast<X *>(&v);
#pragma unroll
      for (int k = 0; k < VEC; ++k) e[k] = from_real<X>(to_real(e[k]) * scale);
      gv[i] = v;
    }
    for (int64_t i = nvec * VEC + first; i < count; i += stride) g[i] = from_real<X>(to_real(g[i]) * scale);
  } else {
    for (int64_t i = first; i < count; i += stride) g[i] = from_real<X>(to_real(g[i]) * scale);
  }
}

template <typename X>
cudaError_t launch_scale_t(void *g, int64_t count, const void *d_scale, cudaStream_t s) {
  // one resident wave: with the factor 1 the launch must cost next to nothing
  const int64_t want = (count / (16 / (int64_t)sizeof(X)) + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)sm_count() * 8;
  const unsigned grid = (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
  scale_gradient_kernel<X><<<grid, kThreads, 0, s>>>(static_cast<X *>(g), count,
      static_cast<const typename Real<X>::type *>(d_scale));
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_scale(void *g, int64_t count, const void *d_scale, uint32_t flags, cudaStream_t s) {
  if (flags & OT_B200_FP64) return launch_scale_t<double>(g, count, d_scale, s);
  if (flags & OT_B200_BF16) return launch_scale_t<__nv_bfloat16>(g, count, d_scale, s);
  if (flags & OT_B200_FP16) return launch_scale_t<__half>(g, count, d_scale, s);
  return launch_scale_t<float>(g, count, d_scale, s);
}

cudaError_t launch_gradient(const Problem &p, void *grad, const void *d_scale,
                            double scale_host, cudaStream_t s) {
  if (p.flags & OT_B200_FP64) return launch_gradient_t<double>(p, grad, d_scale, scale_host, s);
  if (p.flags & OT_B200_BF16) return launch_gradient_t<__nv_bfloat16>(p, grad, d_scale, scale_host, s);
  if (p.flags & OT_B200_FP16) return launch_gradient_t<__half>(p, grad, d_scale, scale_host, s);
  return launch_gradient_t<float>(p, grad, d_scale, scale_host, s);
}

}  // namespace otb
