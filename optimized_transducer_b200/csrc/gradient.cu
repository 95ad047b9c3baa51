// Stage 3: the gradient w.r.t. the packed logits, one streaming pass.
//
// Mode A (raw logits; may write in place over the logits) replaces
// ComputeGradient / ComputeGradientOneSymPerFrame
// (optimized_transducer/csrc/kernels.cu:522-651): per row, with
//     c = (alpha(t,u) - L) - den(t,u),  L = beta(0,0)
//     grad[v] = scale * ( exp((x[v]+c)+beta(t,u)) - [v==blank] exp((x[v]+c)+sub_blank)
//                                                 - [v==tgt]   exp((x[v]+c)+sub_sym) )
// The additions are made in the reference's order (cpu.cc:509-522) so that the
// rounding of x[v]+c, which dominates the error for long utterances, is the
// same as the reference's.  sub_blank / sub_sym are the beta of the successor
// cells, chosen with the reference's branch priority (cpu.cc:514-522,
// 593-603): the final cell subtracts exp(g) (sub_blank = 0); a blank successor
// exists iff t < T-1 (standard) or t-u < T-1-U (modified); the symbol successor
// is (t,u+1) or, modified, (t+1,u+1); a target equal to the blank is taken by
// the blank column.  Rows outside the band of the modified recursion, and all
// rows of an utterance whose log-likelihood is not finite
// (kernels.cu:556-563), are zero.
//
// Mode B (log-softmax input) replaces ComputeGradientForLogSoftmax /
// ...OneSymPerFrame (kernels.cu:653-779): rows are zero except for the blank
// and symbol entries, -exp((lp + alpha - L) + beta_successor), so the kernel
// only writes.
//
// `scale` folds the two elementwise passes of the reference's Python layer
// (division by N for reduction="mean", multiplication by the upstream
// gradient; transducer_loss.py:150,162) into this pass.
//
// The per-row scalars (alpha, three betas, den, target) are loaded by the
// streaming kernel itself: they sit in L2 (the arrays are ~1 % of the logits)
// and a separate pass that materialised them per row cost 19 us plus a 32-byte
// record per row in both directions.
//
// A row is owned by a group of LPR lanes (see logprob.cu); a group takes runs of
// kRun rows and walks (b, t, u) incrementally.  Runs are dealt from the END of
// the buffer towards its start: the rows stage 1 read last are the ones still
// resident in L2.  HBM traffic per row: V*sizeof(T) read + V*sizeof(T) written
// (mode A), V*sizeof(T) written (mode B).
#include "ot_common.cuh"

namespace otb {

namespace {

constexpr int kThreads = 256;
constexpr int kRun = 8;

// Where a group stands in the batch while it walks a run of rows.
struct Cursor {
  int b, Tn, U, U1, t, u;
  int64_t next_split, coff;
};

__device__ __forceinline__ void cursor_seek(Cursor &c, int64_t row, const int64_t *__restrict__ split,
                                            const int64_t *__restrict__ cell_split,
                                            const int32_t *__restrict__ Tl,
                                            const int32_t *__restrict__ Ul, int N) {
  c.b = find_utt(split, N, row);
  c.Tn = __ldg(Tl + c.b); c.U = __ldg(Ul + c.b); c.U1 = c.U + 1;
  c.next_split = __ldg(split + c.b + 1);
  c.coff = __ldg(cell_split + c.b);
  const int idx = (int)(row - __ldg(split + c.b));
  c.t = idx / c.U1; c.u = idx - c.t * c.U1;
}
// Moves from `row` to row + 1; returns true when a new utterance starts.
__device__ __forceinline__ bool cursor_next(Cursor &c, int64_t row, int64_t rows,
                                            const int64_t *__restrict__ split,
                                            const int64_t *__restrict__ cell_split,
                                            const int32_t *__restrict__ Tl,
                                            const int32_t *__restrict__ Ul) {
  if (++c.u == c.U1) { c.u = 0; ++c.t; }
  if (row + 1 == c.next_split && row + 1 < rows) {
    ++c.b;
    c.Tn = __ldg(Tl + c.b); c.U = __ldg(Ul + c.b); c.U1 = c.U + 1;
    c.next_split = __ldg(split + c.b + 1);
    c.coff = __ldg(cell_split + c.b);
    c.t = 0; c.u = 0;
    return true;
  }
  return false;
}

// What one row's gradient needs besides the row itself.
template <typename T>
struct RowTerms {
  bool zero;        // the whole row is zero
  T c, beta;        // mode A: see the file comment; mode B: c = alpha - L
  T sub_blank, sub_sym;  // beta of the successors, -inf = nothing to subtract
  bool blank_term, sym_term;
  int tgt;          // symbol column or -1
};

template <typename T, bool MODE_B, bool MODIFIED>
__device__ __forceinline__ RowTerms<T> row_terms(const Cursor &c, int64_t row, T L,
                                                 const int32_t *__restrict__ targets, int max_u,
                                                 int blank, const T *__restrict__ den,
                                                 const T *__restrict__ alpha,
                                                 const T *__restrict__ beta) {
  RowTerms<T> r;
  const int diff = c.Tn - 1 - c.U;
  r.zero = !(L - L == (T)0);  // inf or nan
  if (MODIFIED && (c.u > c.t || c.t - c.u > diff)) r.zero = true;
  r.c = 0; r.beta = 0; r.sub_blank = neg_inf<T>(); r.sub_sym = neg_inf<T>();
  r.blank_term = false; r.sym_term = false; r.tgt = -1;
  if (r.zero) return r;
  const int64_t cell = c.coff + cell_pos<MODIFIED>(c.t, c.u, c.U1);
  r.c = alpha[cell] + (-L);
  if (!MODE_B) r.c = r.c - den[row];
  r.beta = beta[cell];
  const bool last = (c.t == c.Tn - 1 && c.u == c.U);
  const bool blank_ok = MODIFIED ? (c.t - c.u < diff) : (c.t < c.Tn - 1);
  const int target_u = (c.u < c.U) ? __ldg(targets + (int64_t)c.b * max_u + c.u) : -1;
  // successors: blank -> (t+1,u), symbol -> (t,u+1) or (t+1,u+1) if modified;
  // in both storage orders they sit U1 and U1+1 entries further.
  const T b_sym_next = (c.u < c.U) ? beta[cell + c.U1 + 1] : neg_inf<T>();
  if (last) {
    r.sub_blank = 0; r.blank_term = true;
  } else if (blank_ok) {
    r.sub_blank = beta[cell + c.U1]; r.blank_term = true;
  } else if (c.u < c.U && target_u == blank) {
    r.sub_blank = b_sym_next; r.blank_term = true;
  }
  if (c.u < c.U && target_u != blank) {
    r.sub_sym = b_sym_next; r.tgt = target_u; r.sym_term = true;
  }
  return r;
}

template <typename T, int VEC, int CH, int LPR, bool MODIFIED>
__global__ void __launch_bounds__(kThreads, sizeof(T) == 4 ? 5 : 2)
gradient_kernel(const T *x, T *g, const int32_t *__restrict__ targets,
                const int32_t *__restrict__ Tl, const int32_t *__restrict__ Ul,
                const int64_t *__restrict__ split, const int64_t *__restrict__ cell_split,
                const T *__restrict__ den, const T *__restrict__ alpha,
                const T *__restrict__ beta, const int32_t *__restrict__ status, int N,
                int64_t rows, int V, int max_u, int blank, const T *__restrict__ d_scale,
                T scale_host) {
  if (status[kStatusCode] != 0) return;
  using VT = typename VecOf<T, VEC>::type;
  constexpr int kGroups = kWarp / LPR;
  const int lane = threadIdx.x & 31;
  const int gl = lane % LPR;
  const int64_t group = ((((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5) * kGroups) + lane / LPR;
  const int64_t ngroups = (((int64_t)gridDim.x * kThreads) >> 5) * kGroups;
  const int nvec = V / VEC;
  const T scale = d_scale ? scale_host * __ldg(d_scale) : scale_host;
  const int bvec = blank / VEC, bk = blank % VEC;
  const int64_t nruns = (rows + kRun - 1) / kRun;

  for (int64_t run = nruns - 1 - group; run >= 0; run -= ngroups) {
    const int64_t r0 = run * kRun;
    const int64_t r1 = (r0 + kRun < rows) ? r0 + kRun : rows;
    Cursor cur;
    cursor_seek(cur, r0, split, cell_split, Tl, Ul, N);
    T L = beta[cur.coff];  // beta(0,0) is the first entry in both storage orders
    for (int64_t row = r0; row < r1; ++row) {
      const T *px = x + row * (int64_t)V;
      T *pg = g + row * (int64_t)V;
      // The row's first chunk is requested before its scalars: nothing in the
      // loads depends on them, and the scalars' own latency hides behind them.
      const bool offband = MODIFIED && (cur.u > cur.t || cur.t - cur.u > cur.Tn - 1 - cur.U);
      VT v[CH];
      if (!offband) {
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          const int vi = j * LPR + gl;
          if (vi < nvec) v[j] = *reinterpret_cast<const VT *>(px + (int64_t)vi * VEC);
        }
      }
      const RowTerms<T> rt = row_terms<T, false, MODIFIED>(cur, row, L, targets, max_u, blank, den, alpha, beta);
      if (rt.zero) {
        VT z;
        T *ze = reinterpret_cast<T *>(&z);
#pragma unroll
        for (int k = 0; k < VEC; ++k) ze[k] = 0;
        for (int vi = gl; vi < nvec; vi += LPR)
          *reinterpret_cast<VT *>(pg + (int64_t)vi * VEC) = z;
      } else {
        const int tvec = rt.tgt >= 0 ? rt.tgt / VEC : -1;
        const int tk = rt.tgt >= 0 ? rt.tgt % VEC : 0;
        for (int base = 0; base < nvec; base += LPR * CH) {
          if (base > 0) {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int vi = base + j * LPR + gl;
              if (vi < nvec) v[j] = *reinterpret_cast<const VT *>(px + (int64_t)vi * VEC);
            }
          }
#pragma unroll
          for (int j = 0; j < CH; ++j) {
            const int vi = base + j * LPR + gl;
            if (vi < nvec) {
              T *e = reinterpret_cast<T *>(&v[j]);
              const int bsel = (vi == bvec && rt.blank_term) ? bk : -1;
              const int tsel = (vi == tvec) ? tk : -1;
#pragma unroll
              for (int k = 0; k < VEC; ++k) {
                const T gv = e[k] + rt.c;
                T val = s_exp(gv + rt.beta);
                if (k == bsel) val -= s_exp(gv + rt.sub_blank);
                else if (k == tsel) val -= s_exp(gv + rt.sub_sym);
                e[k] = val * scale;
              }
              *reinterpret_cast<VT *>(pg + (int64_t)vi * VEC) = v[j];
            }
          }
        }
      }
      if (cursor_next(cur, row, rows, split, cell_split, Tl, Ul)) L = beta[cur.coff];
    }
  }
}

template <typename T, int VEC, int LPR, bool MODIFIED>
__global__ void __launch_bounds__(kThreads)
gradient_logsoftmax_kernel(T *__restrict__ g, const int32_t *__restrict__ targets,
                           const int32_t *__restrict__ Tl, const int32_t *__restrict__ Ul,
                           const int64_t *__restrict__ split,
                           const int64_t *__restrict__ cell_split, const T *__restrict__ lp,
                           const T *__restrict__ alpha, const T *__restrict__ beta,
                           const int32_t *__restrict__ status, int N, int64_t rows, int V,
                           int max_u, int blank, const T *__restrict__ d_scale, T scale_host) {
  if (status[kStatusCode] != 0) return;
  using VT = typename VecOf<T, VEC>::type;
  constexpr int kGroups = kWarp / LPR;
  const int lane = threadIdx.x & 31;
  const int gl = lane % LPR;
  const int64_t group = ((((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5) * kGroups) + lane / LPR;
  const int64_t ngroups = (((int64_t)gridDim.x * kThreads) >> 5) * kGroups;
  const int nvec = V / VEC;
  const T scale = d_scale ? scale_host * __ldg(d_scale) : scale_host;
  const int bvec = blank / VEC, bk = blank % VEC;
  const int64_t nruns = (rows + kRun - 1) / kRun;
  for (int64_t run = group; run < nruns; run += ngroups) {
    const int64_t r0 = run * kRun;
    const int64_t r1 = (r0 + kRun < rows) ? r0 + kRun : rows;
    Cursor cur;
    cursor_seek(cur, r0, split, cell_split, Tl, Ul, N);
    T L = beta[cur.coff];
    for (int64_t row = r0; row < r1; ++row) {
      const RowTerms<T> rt = row_terms<T, true, MODIFIED>(cur, row, L, targets, max_u, blank, nullptr, alpha, beta);
      T val_blank = 0, val_sym = 0;
      if (!rt.zero) {
        const int64_t cell = cur.coff + cell_pos<MODIFIED>(cur.t, cur.u, cur.U1);
        // -exp((lp + (alpha - L)) + beta_successor), cpu.cc:661-668
        if (rt.blank_term) val_blank = -r_exp((lp[2 * cell] + rt.c) + rt.sub_blank) * scale;
        if (rt.sym_term) val_sym = -r_exp((lp[2 * cell + 1] + rt.c) + rt.sub_sym) * scale;
      }
      const int tvec = rt.tgt >= 0 ? rt.tgt / VEC : -1;
      const int tk = rt.tgt >= 0 ? rt.tgt % VEC : 0;
      T *pg = g + row * (int64_t)V;
      for (int vi = gl; vi < nvec; vi += LPR) {
        VT z;
        T *ze = reinterpret_cast<T *>(&z);
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          T val = 0;
          if (vi == bvec && k == bk) val = val_blank;
          else if (vi == tvec && k == tk) val = val_sym;
          ze[k] = val;
        }
        *reinterpret_cast<VT *>(pg + (int64_t)vi * VEC) = z;
      }
      if (cursor_next(cur, row, rows, split, cell_split, Tl, Ul)) L = beta[cur.coff];
    }
  }
}

// Exactly one resident wave of `kernel` (never more groups than rows): a larger
// grid-stride grid would run a partial second wave at the end.
template <typename K>
unsigned stream_grid(K kernel, int *per_sm, int64_t rows, int rows_per_block) {
  if (*per_sm == 0) *per_sm = blocks_per_sm(kernel, kThreads);
  const int64_t want = (rows + rows_per_block - 1) / rows_per_block;
  const int64_t cap = (int64_t)sm_count() * *per_sm;
  return (unsigned)(want < cap ? (want > 0 ? want : 1) : cap);
}

template <typename T> struct Arrays {
  const int32_t *status;
  const int64_t *split, *cell_split;
  const T *den, *lp, *alpha, *beta;
  explicit Arrays(const Problem &p)
      : status(reinterpret_cast<const int32_t *>(p.ws + p.lay.status)),
        split(reinterpret_cast<const int64_t *>(p.ws + p.lay.split)),
        cell_split(reinterpret_cast<const int64_t *>(p.ws + p.lay.cell_split)),
        den(reinterpret_cast<const T *>(p.ws + p.lay.den)),
        lp(reinterpret_cast<const T *>(p.ws + p.lay.lp)),
        alpha(reinterpret_cast<const T *>(p.ws + p.lay.alpha)),
        beta(reinterpret_cast<const T *>(p.ws + p.lay.beta)) {}
};

template <typename T, int VEC, int CH, int LPR, bool MODIFIED>
cudaError_t launch_grad_a(const Problem &p, void *grad, const void *d_scale,
                          double scale_host, cudaStream_t s) {
  static int per_sm = 0;
  auto kernel = gradient_kernel<T, VEC, CH, LPR, MODIFIED>;
  const Arrays<T> a(p);
  constexpr int rows_per_block = (kThreads / kWarp) * (kWarp / LPR);
  kernel<<<stream_grid(kernel, &per_sm, p.rows, rows_per_block), kThreads, 0, s>>>(
      static_cast<const T *>(p.logits), static_cast<T *>(grad), p.targets, p.T, p.U, a.split,
      a.cell_split, a.den, a.alpha, a.beta, a.status, p.N, p.rows, p.V, p.max_u, p.blank,
      static_cast<const T *>(d_scale), (T)scale_host);
  return cudaGetLastError();
}

template <typename T, int VEC, int CH, int LPR>
cudaError_t launch_grad_a_m(const Problem &p, void *grad, const void *d_scale,
                            double scale_host, cudaStream_t s) {
  return (p.flags & OT_B200_ONE_SYM_PER_FRAME)
             ? launch_grad_a<T, VEC, CH, LPR, true>(p, grad, d_scale, scale_host, s)
             : launch_grad_a<T, VEC, CH, LPR, false>(p, grad, d_scale, scale_host, s);
}

template <typename T, int VEC, bool MODIFIED>
cudaError_t launch_grad_b(const Problem &p, void *grad, const void *d_scale,
                          double scale_host, cudaStream_t s) {
  static int per_sm = 0;
  auto kernel = gradient_logsoftmax_kernel<T, VEC, 32, MODIFIED>;
  const Arrays<T> a(p);
  kernel<<<stream_grid(kernel, &per_sm, p.rows, kThreads / kWarp), kThreads, 0, s>>>(
      static_cast<T *>(grad), p.targets, p.T, p.U, a.split, a.cell_split, a.lp, a.alpha, a.beta,
      a.status, p.N, p.rows, p.V, p.max_u, p.blank, static_cast<const T *>(d_scale), (T)scale_host);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_gradient_t(const Problem &p, void *grad, const void *d_scale,
                              double scale_host, cudaStream_t s) {
  constexpr int VEC = Vec16<T>::n;
  const bool modified = p.flags & OT_B200_ONE_SYM_PER_FRAME;
  const bool aligned = (p.V % VEC == 0) &&
                       (reinterpret_cast<uintptr_t>(grad) % 16 == 0);
  if (p.flags & OT_B200_FROM_LOG_SOFTMAX) {
    if (aligned)
      return modified ? launch_grad_b<T, VEC, true>(p, grad, d_scale, scale_host, s)
                      : launch_grad_b<T, VEC, false>(p, grad, d_scale, scale_host, s);
    return modified ? launch_grad_b<T, 1, true>(p, grad, d_scale, scale_host, s)
                    : launch_grad_b<T, 1, false>(p, grad, d_scale, scale_host, s);
  }
  const bool vec_ok = aligned && (reinterpret_cast<uintptr_t>(p.logits) % 16 == 0);
  if (vec_ok) {
    const int nvec = p.V / VEC;
    if (nvec <= 8 * 4) return launch_grad_a_m<T, VEC, 4, 8>(p, grad, d_scale, scale_host, s);
    if (nvec <= 16 * 4) return launch_grad_a_m<T, VEC, 4, 16>(p, grad, d_scale, scale_host, s);
    return launch_grad_a_m<T, VEC, 4, 32>(p, grad, d_scale, scale_host, s);
  }
  const int per_lane = (p.V + kWarp - 1) / kWarp;
  if (per_lane <= 4) return launch_grad_a_m<T, 1, 4, 32>(p, grad, d_scale, scale_host, s);
  return launch_grad_a_m<T, 1, 8, 32>(p, grad, d_scale, scale_host, s);
}

}  // namespace

cudaError_t launch_gradient(const Problem &p, void *grad, const void *d_scale,
                            double scale_host, cudaStream_t s) {
  return (p.flags & OT_B200_FP64)
             ? launch_gradient_t<double>(p, grad, d_scale, scale_host, s)
             : launch_gradient_t<float>(p, grad, d_scale, scale_host, s);
}

}  // namespace otb
