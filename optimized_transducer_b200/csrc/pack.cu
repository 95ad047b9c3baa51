// Callers' side of the packed layout: building the packed (rows, D) tensors the
// loss expects from padded batch tensors, and taking gradients back.
//
// The reference leaves this to the user as a Python list comprehension plus
// torch.cat (README.md:165-177 of the reference):
//     x_b = encoder_out[b, :T_b].unsqueeze(1) + decoder_out[b, :U_b+1].unsqueeze(0)
//     x   = cat([x_b.reshape(-1, D) for b in range(N)])
// and its tests convert a padded (N, maxT, maxU+1, V) tensor by slicing
// (python/tests/test_compute_transducer_loss.py:36-56).  Here each of these is
// one streaming kernel over the packed rows:
//   pack_add      out[row(b,t,u)]  = enc[b,t] + dec[b,u]            (joiner input)
//   pack_copy     out[row(b,t,u)]  = padded[b,t,u]                  (padded -> packed)
//   unpack_copy   padded[b,t,u]    = in[row(b,t,u)], 0 elsewhere    (packed -> padded)
//   sum_over_u    genc[b,t] = sum_u g[row(b,t,u)],  0 for t >= T_b  (backward of pack_add)
//   sum_over_t    gdec[b,u] = sum_t g[row(b,t,u)],  0 for u >  U_b
//                 (both from one read of g where the batch is large enough:
//                 pack_sum_slab_kernel)
// The copies give one warp a packed row (16-byte loads when D % 4 == 0 and the
// bases are aligned); a warp takes runs of 8 rows and walks (b, t, u)
// incrementally.  pack_add writes by frames and the sums read rows a fixed stride
// apart (see the kernels).  All of them are HBM-bound: rows * D * sizeof(T) bytes
// written or read once.
#include "ot_common.cuh"

namespace otb {
namespace {

constexpr int kThreads = 256;
constexpr int kRun = 8;

// What a kernel of this file does when the lengths are inconsistent (status != 0):
// it must not follow them, but it does not leave its output uninitialised either.
// Every element it was to produce becomes NaN, so a caller that has not looked at
// the status cannot mistake the result for data.  `count` elements, all blocks of
// the grid take part.
template <typename T>
__device__ __forceinline__ void poison(T *out, int64_t count) {
  const int64_t nthreads = (int64_t)gridDim.x * gridDim.y * blockDim.x;
  const int64_t first = ((int64_t)blockIdx.y * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x;
  const T nan = from_real<T>((typename Real<T>::type)__int_as_float(0x7fc00000));
  for (int64_t i = first; i < count; i += nthreads) out[i] = nan;
}

// One CTA: split[b] = sum_{b' < b} T_b' * (U_b' + 1); flags inconsistent lengths
// (status word: 1 + the first offending utterance found, or -1 when only the sum
// differs from `rows`).  `sticky`: NULL, or the device view of the mapped host
// record of the last failed call (see api.cu), written on failure.
__global__ void __launch_bounds__(1024)
pack_prepare_kernel(const int32_t *__restrict__ Tl, const int32_t *__restrict__ Ul, int N,
                    int64_t rows, int max_t, int max_u1, int64_t *__restrict__ split,
                    int32_t *__restrict__ status, volatile int32_t *sticky, int32_t seq) {
  __shared__ long long part[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) status[0] = 0;
  __syncthreads();
  const int per = (N + blockDim.x - 1) / blockDim.x;
  const int b0 = min(tid * per, N), b1 = min(b0 + per, N);
  long long mine = 0;
  for (int b = b0; b < b1; ++b) {
    const int t = Tl[b], u = Ul[b];
    if (t <= 0 || t > max_t || u < 0 || u + 1 > max_u1) atomicExch(status, 1 + b);
    mine += (long long)max(t, 0) * (long long)(max(u, 0) + 1);
  }
  long long incl = mine;
#pragma unroll
  for (int o = 1; o < kWarp; o <<= 1) {
    const long long v = __shfl_up_sync(kFull, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == kWarp - 1) part[warp] = incl;
  __syncthreads();
  long long base = 0, total = 0;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
    if (w < warp) base += part[w];
    total += part[w];
  }
  long long run = base + incl - mine;
  for (int b = b0; b < b1; ++b) {
    split[b] = run;
    run += (long long)max(Tl[b], 0) * (long long)(max(Ul[b], 0) + 1);
  }
  __syncthreads();  // every thread's verdict on its utterances is in
  if (tid == 0) {
    split[N] = total;
    if (status[0] == 0 && total != rows) status[0] = -1;
    if (sticky != nullptr && status[0] != 0) {
      sticky[1] = status[0] > 0 ? status[0] - 1 : 0;
      sticky[2] = seq;
      __threadfence_system();
      sticky[0] = OT_B200_INPUT_PACK_LENGTHS;
    }
  }
}

enum Mode { kAdd = 0, kCopy = 1, kUnpack = 2 };

// kAdd:    out (rows, D) = a[b,t,:] + bsrc[b,u,:]     a: (N,max_t,D), bsrc: (N,max_u1,D)
// kCopy:   out (rows, D) = a[b,t,u,:]                 a: (N,max_t,max_u1,D)
// kUnpack: out[b,t,u,:]  = a[row,:]                   a: (rows, D), out: (N,max_t,max_u1,D)
template <typename T, int VEC, int MODE>
__global__ void __launch_bounds__(kThreads)
pack_rows_kernel(const T *__restrict__ a, const T *__restrict__ bsrc, T *__restrict__ out,
                 const int32_t *__restrict__ Tl, const int32_t *__restrict__ Ul,
                 const int64_t *__restrict__ split, const int32_t *__restrict__ status, int N,
                 int64_t rows, int D, int max_t, int max_u1) {
  if (status[0] != 0) {
    if (MODE != kUnpack) poison(out, rows * (int64_t)D);  // the padded output was zeroed and stays so
    return;
  }
  using VT = typename VecOf<T, VEC>::type;
  using R = typename Real<T>::type;
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  const int nvec = D / VEC;
  const int64_t nruns = (rows + kRun - 1) / kRun;
  for (int64_t run = warp; run < nruns; run += nwarps) {
    const int64_t r0 = run * kRun;
    const int64_t r1 = (r0 + kRun < rows) ? r0 + kRun : rows;
    int b = find_utt(split, N, r0);
    int U1 = __ldg(Ul + b) + 1;
    int64_t next_split = __ldg(split + b + 1);
    int t, u;
    {
      const int idx = (int)(r0 - __ldg(split + b));
      t = idx / U1; u = idx - t * U1;
    }
    // Frame whose encoder vector the registers hold (rows of a run mostly share
    // their frame: only u advances), when a row fits into one chunk.
    constexpr int kCh = 4;
    const bool one_chunk = nvec <= kWarp * kCh;
    int64_t held = -1;
    VT x[kCh];
    for (int64_t row = r0; row < r1; ++row) {
      const int64_t padded = (((int64_t)b * max_t + t) * max_u1 + u) * D;
      if (MODE == kAdd) {
        const int64_t frame = (int64_t)b * max_t + t;
        const T *pa = a + frame * D;
        const T *pb = bsrc + ((int64_t)b * max_u1 + u) * D;
        T *po = out + row * (int64_t)D;
        // kCh vectors per lane at a time, all loads issued before the first
        // add.  Both operands are small and L2-resident, but at one encoder and
        // one decoder load per stored vector the L2 would have to deliver twice
        // the bytes the pass writes; keeping the encoder vector halves that.
        for (int base = 0; base < nvec; base += kWarp * kCh) {
          VT y[kCh];
          const bool reload = !(one_chunk && held == frame);
#pragma unroll
          for (int j = 0; j < kCh; ++j) {
            const int vi = base + j * kWarp + lane;
            if (vi < nvec) {
              if (reload) x[j] = *reinterpret_cast<const VT *>(pa + (int64_t)vi * VEC);
              y[j] = *reinterpret_cast<const VT *>(pb + (int64_t)vi * VEC);
            }
          }
          held = frame;
#pragma unroll
          for (int j = 0; j < kCh; ++j) {
            const int vi = base + j * kWarp + lane;
            if (vi < nvec) {
              VT z;
              const T *xe = reinterpret_cast<const T *>(&x[j]);
              const T *ye = reinterpret_cast<const T *>(&y[j]);
              T *ze = reinterpret_cast<T *>(&z);
#pragma unroll
              for (int k = 0; k < VEC; ++k) ze[k] = from_real<T>((R)(to_real(xe[k]) + to_real(ye[k])));
              *reinterpret_cast<VT *>(po + (int64_t)vi * VEC) = z;
            }
          }
        }
      } else {
        const T *ps = (MODE == kCopy) ? a + padded : a + row * (int64_t)D;
        T *po = (MODE == kCopy) ? out + row * (int64_t)D : out + padded;
        for (int vi = lane; vi < nvec; vi += kWarp)
          *reinterpret_cast<VT *>(po + (int64_t)vi * VEC) =
              *reinterpret_cast<const VT *>(ps + (int64_t)vi * VEC);
      }
      if (++u == U1) { u = 0; ++t; }
      if (row + 1 == next_split && row + 1 < rows) {
        ++b;
        U1 = __ldg(Ul + b) + 1;
        next_split = __ldg(split + b + 1);
        t = 0; u = 0;
      }
    }
  }
}

constexpr int kAddCh = 4;       // decoder vectors a thread keeps in registers
constexpr int kAddFrames = 16;  // frames one block writes

// The joiner input by frames.  The packed rows of one frame (b, t) are one
// contiguous piece of (U_b+1)*D elements, and that piece is the utterance's
// decoder block dec[b, 0..U_b, :] (contiguous too) plus enc[b, t, :] repeated.  A
// block takes 256*kAddCh consecutive vectors of the decoder block into registers
// once and writes them out for kAddFrames frames; per stored vector it loads one
// vector of the frame's 2 KB encoder row, which the first warp brings into L1.
// The L2 then delivers a small fraction of the bytes the pass writes, where the
// row-by-row kernel asks it for one decoder vector per stored vector.
// Grid: x = chunk of the decoder block + chunks_max * group of frames, y =
// utterance; blocks past their utterance's own extent leave at once.
template <typename T, int VEC>
__global__ void __launch_bounds__(kThreads)
pack_add_frames_kernel(const T *__restrict__ enc, const T *__restrict__ dec, T *__restrict__ out,
                       const int32_t *__restrict__ Tl, const int32_t *__restrict__ Ul,
                       const int64_t *__restrict__ split, const int32_t *__restrict__ status,
                       int N, int64_t rows, int D, int max_t, int max_u1, int chunks_max) {
  if (status[0] != 0) {
    poison(out, rows * (int64_t)D);
    return;
  }
  using VT = typename VecOf<T, VEC>::type;
  using R = typename Real<T>::type;
  const int nvec = D / VEC;
  const int chunk = (int)(blockIdx.x % (unsigned)chunks_max);
  const int t0 = (int)(blockIdx.x / (unsigned)chunks_max) * kAddFrames;
  const int64_t i0 = (int64_t)chunk * (kThreads * kAddCh) + threadIdx.x;
  for (int b = blockIdx.y; b < N; b += gridDim.y) {
    const int Tn = __ldg(Tl + b), U1 = __ldg(Ul + b) + 1;
    const int64_t nvb = (int64_t)U1 * nvec;  // vectors in one frame's piece
    if ((int64_t)chunk * (kThreads * kAddCh) >= nvb || t0 >= Tn) continue;
    const int t1 = min(Tn, t0 + kAddFrames);
    const VT *decv = reinterpret_cast<const VT *>(dec + (int64_t)b * max_u1 * D);
    VT y[kAddCh];
    int dv[kAddCh];
    bool ok[kAddCh];
#pragma unroll
    for (int k = 0; k < kAddCh; ++k) {
      const int64_t i = i0 + (int64_t)k * kThreads;
      ok[k] = i < nvb;
      dv[k] = ok[k] ? (int)(i % nvec) : 0;
      if (ok[k]) y[k] = decv[i];
    }
    const VT *encv = reinterpret_cast<const VT *>(enc + ((int64_t)b * max_t + t0) * D);
    VT *outv = reinterpret_cast<VT *>(out + (__ldg(split + b) + (int64_t)t0 * U1) * D) + i0;
#pragma unroll 2
    for (int t = t0; t < t1; ++t, encv += nvec, outv += nvb) {
      VT x[kAddCh];
#pragma unroll
      for (int k = 0; k < kAddCh; ++k)
        if (ok[k]) x[k] = encv[dv[k]];
#pragma unroll
      for (int k = 0; k < kAddCh; ++k) {
        if (ok[k]) {
          VT z;
          const T *xe = reinterpret_cast<const T *>(&x[k]);
          const T *ye = reinterpret_cast<const T *>(&y[k]);
          T *ze = reinterpret_cast<T *>(&z);
#pragma unroll
          for (int e = 0; e < VEC; ++e) ze[e] = from_real<T>((R)(to_real(xe[e]) + to_real(ye[e])));
          outv[(int64_t)k * kThreads] = z;
        }
      }
    }
  }
}

// acc[e] += element e of the vector v, in the arithmetic type R.
template <typename T, int VEC>
struct Acc {
  typename Real<T>::type v[VEC];
};
template <typename T, int VEC, typename VT>
__device__ __forceinline__ void acc_add(Acc<T, VEC> &acc, const VT &v) {
  const T *ve = reinterpret_cast<const T *>(&v);
#pragma unroll
  for (int e = 0; e < VEC; ++e) acc.v[e] += to_real(ve[e]);
}

// OVER_U: CTA (t, b): out[b,t,:] = sum_u g[row(b,t,u),:]   (zero for t >= T_b)
// else  : CTA (u, b): out[b,u,:] = sum_t g[row(b,t,u),:]   (zero for u >  U_b)
// Either way the CTA adds up n rows of D elements that lie `stride` apart.  With
// nvec = D/VEC vectors per row, R = 256/nvec rows are read side by side (thread =
// (row lane, vector)), eight rows deep per thread with all loads issued before the
// first add; the R partial sums meet in shared memory in a fixed order, so the
// result does not depend on timing.  Rows longer than 256 vectors: R = 1 and the
// threads walk the row.  The sums are kept in the arithmetic type (float for
// 16-bit storage) and rounded once, on the store.
template <typename T, int VEC, bool OVER_U>
__global__ void __launch_bounds__(kThreads)
pack_sum_kernel(const T *__restrict__ g, T *__restrict__ out, const int32_t *__restrict__ Tl,
                const int32_t *__restrict__ Ul, const int64_t *__restrict__ split,
                const int32_t *__restrict__ status, int D, int extent) {
  using VT = typename VecOf<T, VEC>::type;
  using A = Acc<T, VEC>;
  using Rt = typename Real<T>::type;
  const int tid = threadIdx.x;
  const int b = blockIdx.y, i = blockIdx.x;  // i: frame t (OVER_U) or column u
  if (status[0] != 0) {  // this block's own D outputs
    T *o = out + ((int64_t)b * extent + i) * D;
    const T nan = from_real<T>((Rt)__int_as_float(0x7fc00000));
    for (int d = tid; d < D; d += kThreads) o[d] = nan;
    return;
  }
  __shared__ A part[kThreads];
  constexpr int kDeep = 8;
  const int Tn = Tl[b], U1 = Ul[b] + 1;
  VT *po = reinterpret_cast<VT *>(out + ((int64_t)b * extent + i) * D);
  const bool live = OVER_U ? (i < Tn) : (i < U1);
  const int n = live ? (OVER_U ? U1 : Tn) : 0;
  const int nvec = D / VEC;
  // distance between consecutive rows of the sum, in vectors
  const int64_t stride = OVER_U ? (int64_t)nvec : (int64_t)U1 * nvec;
  const VT *base = reinterpret_cast<const VT *>(
      g + (split[b] + (OVER_U ? (int64_t)i * U1 : (int64_t)i)) * D);
  A zero;
#pragma unroll
  for (int e = 0; e < VEC; ++e) zero.v[e] = (Rt)0;
  const auto store = [&](VT *dst, const A &a) {
    VT z;
    T *ze = reinterpret_cast<T *>(&z);
#pragma unroll
    for (int e = 0; e < VEC; ++e) ze[e] = from_real<T>(a.v[e]);
    *dst = z;
  };
  const int R = nvec <= kThreads ? kThreads / nvec : 1;
  const int rl = nvec <= kThreads ? tid / nvec : 0;
  const int64_t step = (int64_t)R * stride;
  for (int dv = nvec <= kThreads ? tid - rl * nvec : tid; dv < nvec; dv += kThreads) {
    A acc = zero;
    if (rl < R) {
      const VT *p = base + (int64_t)rl * stride + dv;
      int r = rl;
      for (; r + (kDeep - 1) * R < n; r += kDeep * R, p += kDeep * step) {
        VT v[kDeep];
#pragma unroll
        for (int j = 0; j < kDeep; ++j) v[j] = p[j * step];
#pragma unroll
        for (int j = 0; j < kDeep; ++j) acc_add<T, VEC>(acc, v[j]);
      }
      for (; r < n; r += R, p += step) acc_add<T, VEC>(acc, *p);
    }
    if (R == 1) {
      if (rl < R) store(po + dv, acc);  // nvec in (128, 256]: the threads past the row idle
    } else {
      if (rl < R) part[tid] = acc;
      __syncthreads();
      if (tid < nvec) {
        A s = part[tid];
        for (int q = 1; q < R; ++q) {
          const A &o = part[q * nvec + tid];
#pragma unroll
          for (int e = 0; e < VEC; ++e) s.v[e] += o.v[e];
        }
        store(po + tid, s);
      }
    }
    if (nvec <= kThreads) break;  // one vector per thread in this arrangement
  }
}

// Both sums of the backward pass from ONE read of the gradient.  A CTA takes one
// utterance and one piece of LANES vectors (128 bytes) of every packed row of it, all
// frames: thread = (row lane rl, vector dv), RL = THREADS / LANES packed rows side by
// side.  Consecutive rows of a frame are consecutive u, so thread (rl, dv) meets
// u = rl, rl + RL, ... (at most KU of them: U + 1 <= RL * KU) in every frame:
//   sum over t: one accumulator per u of the thread, in registers, stored at the end;
//               nobody else has that (u, vector);
//   sum over u: the thread's KU values of a frame, then the row lanes of its warp by
//               shuffles, then one entry per warp and frame in shared memory; the
//               warps meet once per round of FR frames (two buffers, one barrier per
//               round), in a fixed order.
// All loads of a round (FR * KU vectors per thread) are issued before the first add.
// Results do not depend on timing.  The outputs' padding (t >= T_b, u > U_b) is zeroed
// by the CTA for its piece.
// The CTAs of an utterance all take as long as the utterance has rows, and a CTA alone
// streams only a few tens of GB/s, so the order matters at the end of the launch:
// blockIdx.y is the utterance's RANK by rows, largest first (found by the CTA itself
// from the lengths, for batches of up to THREADS utterances).
constexpr int kSlabMaxU1 = 128;

template <typename T, int VEC, int LANES, int THREADS, int KU, int FR, int BLOCKS>
__global__ void __launch_bounds__(THREADS, BLOCKS)
pack_sum_slab_kernel(const T *__restrict__ g, T *__restrict__ genc, T *__restrict__ gdec,
                     const int32_t *__restrict__ Tl, const int32_t *__restrict__ Ul,
                     const int64_t *__restrict__ split, const int32_t *__restrict__ status, int N,
                     int D, int max_t, int max_u1) {
  using VT = typename VecOf<T, VEC>::type;
  using A = Acc<T, VEC>;
  using Rt = typename Real<T>::type;
  constexpr int RL = THREADS / LANES;
  constexpr int kWarps = THREADS / kWarp;
  static_assert(LANES <= kWarp && FR * LANES <= THREADS && RL * KU >= kSlabMaxU1, "layout");
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rl = tid / LANES, dv = tid % LANES;
  int b = blockIdx.y;
  if (status[0] == 0 && N <= THREADS) {
    __shared__ int ranked;
    if (tid < N) {
      const int64_t mine = (int64_t)Tl[tid] * (Ul[tid] + 1);
      int before = 0;
      for (int j = 0; j < N; ++j) {
        const int64_t other = (int64_t)Tl[j] * (Ul[j] + 1);
        before += (other > mine || (other == mine && j < tid)) ? 1 : 0;
      }
      if (before == (int)blockIdx.y) ranked = tid;
    }
    __syncthreads();
    b = ranked;
  }
  const int nvec = D / VEC;
  const int vi = blockIdx.x * LANES + dv;  // this thread's vector of a row
  const bool col = vi < nvec;
  VT *oe = reinterpret_cast<VT *>(genc + (int64_t)b * max_t * D);
  VT *od = reinterpret_cast<VT *>(gdec + (int64_t)b * max_u1 * D);
  const auto pack = [](const A &a) {
    VT z;
    T *ze = reinterpret_cast<T *>(&z);
#pragma unroll
    for (int e = 0; e < VEC; ++e) ze[e] = from_real<T>(a.v[e]);
    return z;
  };
  A zero;
#pragma unroll
  for (int e = 0; e < VEC; ++e) zero.v[e] = (Rt)0;
  if (status[0] != 0) {  // this CTA's piece of both outputs
    A n;
#pragma unroll
    for (int e = 0; e < VEC; ++e) n.v[e] = (Rt)__int_as_float(0x7fc00000);
    const VT nan = pack(n);
    if (col) {
      for (int t = rl; t < max_t; t += RL) oe[(int64_t)t * nvec + vi] = nan;
      for (int u = rl; u < max_u1; u += RL) od[(int64_t)u * nvec + vi] = nan;
    }
    return;
  }
  __shared__ A red[2][kWarps][FR][LANES];
  const int Tn = Tl[b], U1 = Ul[b] + 1;
  const VT *base = reinterpret_cast<const VT *>(g) + (split[b] + rl) * nvec + vi;
  const VT vzero = pack(zero);
  A dec[KU];
#pragma unroll
  for (int k = 0; k < KU; ++k) dec[k] = zero;
  int round = 0;
  for (int f0 = 0; f0 < Tn; f0 += FR, ++round) {  // Tn is the CTA's: so are the barriers
    VT v[FR][KU];
#pragma unroll
    for (int j = 0; j < FR; ++j)
#pragma unroll
      for (int k = 0; k < KU; ++k)
        v[j][k] = (col && f0 + j < Tn && rl + k * RL < U1)
                      ? __ldcs(base + ((int64_t)(f0 + j) * U1 + k * RL) * nvec) : vzero;
    A(*mine)[FR][LANES] = red[round & 1];
#pragma unroll
    for (int j = 0; j < FR; ++j) {
      A e = zero;
#pragma unroll
      for (int k = 0; k < KU; ++k) {
        acc_add<T, VEC>(e, v[j][k]);
        acc_add<T, VEC>(dec[k], v[j][k]);
      }
      // the row lanes of this warp that hold the same vector: lanes dv, dv + LANES, ...
#pragma unroll
      for (int o = LANES; o < kWarp; o <<= 1)
#pragma unroll
        for (int x = 0; x < VEC; ++x) e.v[x] += __shfl_xor_sync(kFull, e.v[x], o);
      if (lane < LANES) mine[warp][j][lane] = e;
    }
    __syncthreads();
    // A buffer is rewritten two rounds later, i.e. after the next barrier, which every
    // reader of this round has passed by then.
    if (tid < FR * LANES) {
      const int j = tid / LANES, d = tid % LANES;
      const int vo = blockIdx.x * LANES + d;
      if (f0 + j < Tn && vo < nvec) {
        A sum = mine[0][j][d];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) {
          const A &o = mine[w][j][d];
#pragma unroll
          for (int x = 0; x < VEC; ++x) sum.v[x] += o.v[x];
        }
        oe[(int64_t)(f0 + j) * nvec + vo] = pack(sum);
      }
    }
  }
  if (col) {
#pragma unroll
    for (int k = 0; k < KU; ++k) {
      const int u = rl + k * RL;
      if (u < U1) od[(int64_t)u * nvec + vi] = pack(dec[k]);
    }
    for (int t = Tn + rl; t < max_t; t += RL) oe[(int64_t)t * nvec + vi] = vzero;
    for (int u = U1 + rl; u < max_u1; u += RL) od[(int64_t)u * nvec + vi] = vzero;
  }
}

// OT_B200_PACK_SUM=two: the backward pass as two kernels that each read the gradient
// (pack_sum_kernel) even where the one-read kernel applies; read at every call.
bool two_pass_sums_forced() {
  const char *v = getenv("OT_B200_PACK_SUM");
  return v != nullptr && strcmp(v, "two") == 0;
}

int fail(int code, const char *msg) {
  set_last_error(msg);
  return code;
}

// OT_B200_PACK=rows: the joiner input row by row (pack_rows_kernel) instead of by
// frames; read at every call, so a process can measure both.
bool add_by_rows_forced() {
  const char *v = getenv("OT_B200_PACK");
  return v != nullptr && strcmp(v, "rows") == 0;
}

// One warp per run of kRun rows: as many short-lived blocks as that takes, or, with
// OT_B200_GRID=wave, at most one resident wave (the kernel loops).
template <typename K>
unsigned rows_grid(K kernel, int64_t rows) {
  int64_t want = (rows + (kThreads / kWarp) * kRun - 1) / ((kThreads / kWarp) * kRun);
  if (want < 1) want = 1;
  if (wave_grids()) {
    const int64_t cap = (int64_t)sm_count() * blocks_per_sm(kernel, kThreads);
    if (want > cap) want = cap;
  }
  return (unsigned)(want < 0x7fffffff ? want : 0x7fffffff);
}

template <typename T, int MODE>
int launch_rows(const void *a, const void *b, void *out, const int32_t *Tl, const int32_t *Ul,
                int N, int64_t rows, int D, int max_t, int max_u1, void *ws, uint32_t flags,
                cudaStream_t s) {
  int64_t *split = static_cast<int64_t *>(ws);
  int32_t *status = reinterpret_cast<int32_t *>(split + N + 1);
  int32_t *sticky = nullptr;
  int32_t seq = 0;
  {
    const int rc = begin_reported_call(flags, &sticky, &seq);
    if (rc) return rc;
  }
  pack_prepare_kernel<<<1, 1024, 0, s>>>(Tl, Ul, N, rows, max_t, max_u1, split, status, sticky, seq);
  constexpr int VEC = Vec16<T>::n;
  const bool vec = (D % VEC == 0) && (reinterpret_cast<uintptr_t>(a) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(out) % 16 == 0) &&
                   (b == nullptr || reinterpret_cast<uintptr_t>(b) % 16 == 0);
  const int nvec = vec ? D / VEC : D;
  const int chunks_max =
      (int)(((int64_t)max_u1 * nvec + kThreads * kAddCh - 1) / (kThreads * kAddCh));
  const int groups_max = (max_t + kAddFrames - 1) / kAddFrames;
  if (MODE == kAdd && !add_by_rows_forced() && (int64_t)chunks_max * groups_max < 0x7fffffff) {
    // by frames (see pack_add_frames_kernel); OT_B200_PACK=rows keeps the row-by-row kernel
    const dim3 grid((unsigned)((int64_t)chunks_max * groups_max), (unsigned)(N < 65535 ? N : 65535));
    if (vec)
      pack_add_frames_kernel<T, VEC><<<grid, kThreads, 0, s>>>(
          static_cast<const T *>(a), static_cast<const T *>(b), static_cast<T *>(out), Tl, Ul, split,
          status, N, rows, D, max_t, max_u1, chunks_max);
    else
      pack_add_frames_kernel<T, 1><<<grid, kThreads, 0, s>>>(
          static_cast<const T *>(a), static_cast<const T *>(b), static_cast<T *>(out), Tl, Ul, split,
          status, N, rows, D, max_t, max_u1, chunks_max);
  } else if (vec)
    pack_rows_kernel<T, VEC, MODE><<<rows_grid(pack_rows_kernel<T, VEC, MODE>, rows), kThreads, 0, s>>>(
        static_cast<const T *>(a), static_cast<const T *>(b), static_cast<T *>(out), Tl, Ul, split,
        status, N, rows, D, max_t, max_u1);
  else
    pack_rows_kernel<T, 1, MODE><<<rows_grid(pack_rows_kernel<T, 1, MODE>, rows), kThreads, 0, s>>>(
        static_cast<const T *>(a), static_cast<const T *>(b), static_cast<T *>(out), Tl, Ul, split,
        status, N, rows, D, max_t, max_u1);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(OT_B200_ERR_CUDA, cudaGetErrorString(e));
  return OT_B200_OK;
}

int check(const void *a, const void *out, const int32_t *Tl, const int32_t *Ul, int32_t N,
          int64_t rows, int32_t D, int32_t max_t, int32_t max_u1, const void *ws, uint32_t flags) {
  if (N <= 0 || rows <= 0 || D <= 0 || max_t <= 0 || max_u1 <= 0)
    return fail(OT_B200_ERR_ARGUMENT, "pack: N, rows, D, max_t and max_u1 must be positive");
  const uint32_t types = flags & (OT_B200_FP64 | OT_B200_BF16 | OT_B200_FP16);
  if ((flags & ~(OT_B200_FP64 | OT_B200_BF16 | OT_B200_FP16 | OT_B200_REPORT_ERRORS)) || (types & (types - 1)))
    return fail(OT_B200_ERR_ARGUMENT, "pack: flags may hold one of OT_B200_FP64/BF16/FP16 and OT_B200_REPORT_ERRORS");
  if (!a || !out || !Tl || !Ul) return fail(OT_B200_ERR_ARGUMENT, "pack: a required device pointer is NULL");
  if (!ws || reinterpret_cast<uintptr_t>(ws) % 8 != 0)
    return fail(OT_B200_ERR_WORKSPACE, "pack: workspace missing or not 8-byte aligned");
  return OT_B200_OK;
}

}  // namespace
}  // namespace otb

using namespace otb;

// return FN<element type selected by the flags, MODE>(args...)
#define OTB_PACK_BY_TYPE(flags, FN, MODE, ...)                                  \
  do {                                                                          \
    if ((flags) & OT_B200_FP64) return FN<double, MODE>(__VA_ARGS__);           \
    if ((flags) & OT_B200_BF16) return FN<__nv_bfloat16, MODE>(__VA_ARGS__);    \
    if ((flags) & OT_B200_FP16) return FN<__half, MODE>(__VA_ARGS__);           \
    return FN<float, MODE>(__VA_ARGS__);                                        \
  } while (0)

extern "C" {

int ot_b200_pack_workspace_bytes(int32_t N, uint64_t *bytes_out) {
  if (N <= 0 || !bytes_out) return fail(OT_B200_ERR_ARGUMENT, "pack: N must be positive and bytes_out non-NULL");
  *bytes_out = (uint64_t)(N + 1) * sizeof(int64_t) + 64;  // row splits + one status word
  return OT_B200_OK;
}

int ot_b200_pack_joiner_input(const void *d_encoder_out, const void *d_decoder_out,
                              const int32_t *d_logit_lengths, const int32_t *d_target_lengths,
                              int32_t N, int64_t rows, int32_t D, int32_t max_t, int32_t max_u1,
                              uint32_t flags, void *d_workspace, void *d_out, void *stream) {
  int rc = check(d_encoder_out, d_out, d_logit_lengths, d_target_lengths, N, rows, D, max_t, max_u1, d_workspace, flags);
  if (rc) return rc;
  if (!d_decoder_out) return fail(OT_B200_ERR_ARGUMENT, "pack: decoder_out is NULL");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  OTB_PACK_BY_TYPE(flags, launch_rows, kAdd, d_encoder_out, d_decoder_out, d_out, d_logit_lengths,
                   d_target_lengths, N, rows, D, max_t, max_u1, d_workspace, flags, s);
}

int ot_b200_pack_joiner_input_backward(const void *d_grad_out, const int32_t *d_logit_lengths,
                                       const int32_t *d_target_lengths, int32_t N, int64_t rows,
                                       int32_t D, int32_t max_t, int32_t max_u1, uint32_t flags,
                                       void *d_workspace, void *d_grad_encoder, void *d_grad_decoder,
                                       void *stream) {
  int rc = check(d_grad_out, d_grad_encoder, d_logit_lengths, d_target_lengths, N, rows, D, max_t, max_u1, d_workspace, flags);
  if (rc) return rc;
  if (!d_grad_decoder) return fail(OT_B200_ERR_ARGUMENT, "pack: grad_decoder is NULL");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int64_t *split = static_cast<int64_t *>(d_workspace);
  int32_t *status = reinterpret_cast<int32_t *>(split + N + 1);
  int32_t *sticky = nullptr;
  int32_t seq = 0;
  rc = begin_reported_call(flags, &sticky, &seq);
  if (rc) return rc;
  pack_prepare_kernel<<<1, 1024, 0, s>>>(d_logit_lengths, d_target_lengths, N, rows, max_t, max_u1, split, status, sticky, seq);
  const dim3 ge((unsigned)max_t, (unsigned)N), gd((unsigned)max_u1, (unsigned)N);
  const auto aligned = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool al = aligned(d_grad_out) && aligned(d_grad_encoder) && aligned(d_grad_decoder);
  // The one-read kernel needs whole vectors, U + 1 <= 128 and enough CTAs (utterances
  // x row pieces) to fill the device twice: a CTA alone streams only a few tens of
  // GB/s, so a handful of long utterances is better served by the two kernels below,
  // whose grids follow the frames and the columns.
  const int sum_vec = (flags & OT_B200_FP64) ? 2 : 4;
  const int sum_lanes = (flags & (OT_B200_BF16 | OT_B200_FP16)) ? 16 : 8;  // 128 bytes of a row
  if (al && D % sum_vec == 0 && max_u1 <= kSlabMaxU1 && !two_pass_sums_forced()) {
    const int pieces = (D / sum_vec + sum_lanes - 1) / sum_lanes;
    if ((int64_t)N * pieces >= 2 * (int64_t)sm_count() && N <= 65535) {
      const dim3 gs((unsigned)pieces, (unsigned)N);
      // 256 threads: 32 rows side by side (512 threads, 64 rows and half the accumulators
      // per thread, measured 0.43 against 0.32 ms on the benchmark's lengths with D = 512)
#define OTB_PACK_SLAB(T, VEC, LANES, FR)                                                            \
  pack_sum_slab_kernel<T, VEC, LANES, kThreads, kSlabMaxU1 * LANES / kThreads, FR, 2>               \
      <<<gs, kThreads, 0, s>>>(static_cast<const T *>(d_grad_out), static_cast<T *>(d_grad_encoder), \
                               static_cast<T *>(d_grad_decoder), d_logit_lengths, d_target_lengths, \
                               split, status, N, D, max_t, max_u1)
      if (flags & OT_B200_FP64) OTB_PACK_SLAB(double, 2, 8, 4);
      else if (flags & OT_B200_BF16) OTB_PACK_SLAB(__nv_bfloat16, 4, 16, 2);
      else if (flags & OT_B200_FP16) OTB_PACK_SLAB(__half, 4, 16, 2);
      else OTB_PACK_SLAB(float, 4, 8, 4);
#undef OTB_PACK_SLAB
      const cudaError_t es = cudaGetLastError();
      if (es != cudaSuccess) return fail(OT_B200_ERR_CUDA, cudaGetErrorString(es));
      return OT_B200_OK;
    }
  }
#define OTB_PACK_SUM(T, VEC)                                                                        \
  do {                                                                                              \
    pack_sum_kernel<T, VEC, true><<<ge, kThreads, 0, s>>>(                                          \
        static_cast<const T *>(d_grad_out), static_cast<T *>(d_grad_encoder), d_logit_lengths,      \
        d_target_lengths, split, status, D, max_t);                                                 \
    pack_sum_kernel<T, VEC, false><<<gd, kThreads, 0, s>>>(                                         \
        static_cast<const T *>(d_grad_out), static_cast<T *>(d_grad_decoder), d_logit_lengths,      \
        d_target_lengths, split, status, D, max_u1);                                                \
  } while (0)
  if (flags & OT_B200_FP64) {
    if (al && D % 2 == 0) OTB_PACK_SUM(double, 2); else OTB_PACK_SUM(double, 1);
  } else if (flags & OT_B200_BF16) {
    if (al && D % 4 == 0) OTB_PACK_SUM(__nv_bfloat16, 4); else OTB_PACK_SUM(__nv_bfloat16, 1);
  } else if (flags & OT_B200_FP16) {
    if (al && D % 4 == 0) OTB_PACK_SUM(__half, 4); else OTB_PACK_SUM(__half, 1);
  } else {
    if (al && D % 4 == 0) OTB_PACK_SUM(float, 4); else OTB_PACK_SUM(float, 1);
  }
#undef OTB_PACK_SUM
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(OT_B200_ERR_CUDA, cudaGetErrorString(e));
  return OT_B200_OK;
}

int ot_b200_pack_padded(const void *d_padded, const int32_t *d_logit_lengths,
                        const int32_t *d_target_lengths, int32_t N, int64_t rows, int32_t D,
                        int32_t max_t, int32_t max_u1, uint32_t flags, void *d_workspace,
                        void *d_packed, void *stream) {
  int rc = check(d_padded, d_packed, d_logit_lengths, d_target_lengths, N, rows, D, max_t, max_u1, d_workspace, flags);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  OTB_PACK_BY_TYPE(flags, launch_rows, kCopy, d_padded, nullptr, d_packed, d_logit_lengths,
                   d_target_lengths, N, rows, D, max_t, max_u1, d_workspace, flags, s);
}

int ot_b200_unpack_to_padded(const void *d_packed, const int32_t *d_logit_lengths,
                             const int32_t *d_target_lengths, int32_t N, int64_t rows, int32_t D,
                             int32_t max_t, int32_t max_u1, uint32_t flags, void *d_workspace,
                             void *d_padded, void *stream) {
  int rc = check(d_packed, d_padded, d_logit_lengths, d_target_lengths, N, rows, D, max_t, max_u1, d_workspace, flags);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t es = (flags & OT_B200_FP64) ? 8 : ((flags & (OT_B200_BF16 | OT_B200_FP16)) ? 2 : 4);
  // everything outside the lattices is zero
  cudaError_t e = cudaMemsetAsync(d_padded, 0, (size_t)N * max_t * max_u1 * D * es, s);
  if (e != cudaSuccess) return fail(OT_B200_ERR_CUDA, cudaGetErrorString(e));
  OTB_PACK_BY_TYPE(flags, launch_rows, kUnpack, d_packed, nullptr, d_padded, d_logit_lengths,
                   d_target_lengths, N, rows, D, max_t, max_u1, d_workspace, flags, s);
}

}  // extern "C"
