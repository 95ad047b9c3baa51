// Shared declarations of the sm_100a transducer-loss kernels.
//
// Notation used in every file of this directory:
//   N        utterances in the batch
//   T_b, U_b frames and target symbols of utterance b; the lattice has
//            T_b x (U_b+1) cells, U1 = U_b + 1
//   row      index into the packed (rows, V) logits; row(b,t,u) = split[b] + t*U1 + u
//   cell     index into the per-cell workspace arrays (lp, alpha, beta);
//            cell(b,t,u) = cell_split[b] + cell_pos(t,u), see below
//   lp       per cell (blank log-prob, next-symbol log-prob)
//   den      per row logsumexp of the logits
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/ot_b200.h"

namespace otb {

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;

// Workspace status words (int32 each).
constexpr int kStatusCode = 0;   // ot_b200_input_error, 0 = inputs are valid
constexpr int kStatusIndex = 1;  // utterance the code refers to
constexpr int kStatusCopyTimeout = 2;  // 1 + utterance (or 1) whose bounded wait for a bulk copy ran out
constexpr int kStatusWords = 16;
// Diagnostic timeline (OT_B200_TRACE): word kStatusTraceOn holds the switch;
// from int32 word kTraceWord on, one (first block started, last block ended)
// pair of %globaltimer values (uint64, ns) per stage.  The status segment of
// the workspace has kStatusBlockWords words.
constexpr int kStatusTraceOn = 3;
constexpr int kTraceWord = 16;
// Words kStatusGroupSplit .. kStatusGroupSplit + kMaxGroups: when a call runs as
// groups of utterances (the pipelined schedules of api.cu), word g holds the first
// utterance of group g (word 0: 0; the words from the number of groups on: N);
// stage 0 derives them from the rows at which the host cut the batch.
constexpr int kMaxGroups = 4;
constexpr int kStatusGroupSplit = 4;
constexpr int kStatusBlockWords = 128;
enum Stage { kStagePrepare = 0, kStageLogprob = 1, kStageLattice = 2, kStageCoef = 3, kStageGradient = 4, kStages_ = 5 };
// Timeline slot of a stage: the launches of group g > 0 of a grouped call use slots
// g*kStages_ .. (g+1)*kStages_-1, everything else 0 .. kStages_-1.
__host__ __device__ __forceinline__ int trace_slot(int stage, int group) {
  return group > 0 ? stage + group * kStages_ : stage;
}
constexpr int kTraceSlots = kMaxGroups * kStages_;
static_assert(kTraceWord + 4 * kTraceSlots <= kStatusBlockWords, "the trace slots must fit into the status block");

// Packed rows at which the host cuts a batch into n groups: row[0] = 0 < row[1] <
// ... < row[n] = rows.  An utterance belongs to the group in whose range
// (row[g], row[g+1]] it ENDS.  n == 0: the call is not grouped.
struct GroupCuts {
  int n = 0;
  int64_t row[kMaxGroups + 1] = {0, 0, 0, 0, 0};
};

// Marker values of the `tgt` field of a gradient-coefficient record.
constexpr int32_t kTgtNone = -1;     // no symbol column to patch in this row
constexpr int32_t kTgtZeroRow = -2;  // the whole gradient row is zero

// Layout of the per-cell arrays of one utterance.
//
// Standard transducer: the recursion advances along anti-diagonals d = t + u,
// so cells are stored diagonal-major ("skewed"): cell_pos(t,u) = (t+u)*U1 + u.
// At step d the threads u = 0..U touch consecutive addresses, i.e. every load
// and store of the wavefront is coalesced.  The block has (T+U)*U1 entries; the
// entries that correspond to no lattice cell are never read or written.
//
// One symbol per frame: both predecessors lie in frame t-1, the recursion is
// frame-synchronous and the natural row-major order t*U1 + u is the coalesced
// one.
template <bool MODIFIED>
__host__ __device__ __forceinline__ int64_t cell_pos(int t, int u, int U1) {
  return MODIFIED ? (int64_t)t * U1 + u : (int64_t)(t + u) * U1 + u;
}
// Entries of one utterance's block, rounded up to an even count so that every
// block starts 16-byte aligned in the (blank, symbol) array.
__host__ __device__ __forceinline__ int64_t cell_block(int T, int U, bool modified) {
  const int64_t n = modified ? (int64_t)T * (U + 1) : (int64_t)(T + U) * (U + 1);
  return (n + 1) & ~int64_t(1);
}

// Per-row coefficients of the gradient w.r.t. raw logits (mode A), produced
// once per row after alpha and beta are known, so that the streaming gradient
// kernel needs a single broadcast load per row:
//   grad[v] = exp((x[v] + c) + beta) - [v == blank] exp((x[v] + c) + sub_blank)
//                                    - [v == tgt]   exp((x[v] + c) + sub_sym)
// sub_* = -inf means "nothing to subtract".
template <typename T>
struct alignas(32) CoefA {
  T c;          // alpha(t,u) - L - den(t,u), evaluated as (alpha + (-L)) - den
  T beta;       // beta(t,u)
  T sub_blank;  // beta of the blank successor (0 for the final cell)
  T sub_sym;    // beta of the symbol successor
  int32_t tgt;  // symbol column, or kTgtNone / kTgtZeroRow
  int32_t utt;  // utterance the row belongs to (for a per-utterance scale)
};

// Mode B (input already log-softmax): the gradient row is zero except for at
// most two entries, whose final values are stored directly.
template <typename T>
struct alignas(16) CoefB {
  T val_blank;  // gradient at the blank column (0 if none)
  T val_sym;    // gradient at the symbol column
  int32_t tgt;  // symbol column, or kTgtNone / kTgtZeroRow
  int32_t utt;  // utterance the row belongs to
};

struct Layout {
  uint64_t total, status, split, cell_split, den, lp, alpha, beta, coef, scores_beta;
  int64_t max_cells;  // capacity of the per-cell arrays
};

// Computes the workspace layout (all segments 256-byte aligned).
Layout make_layout(int32_t N, int64_t rows, int32_t max_u, uint32_t flags);

struct Problem {
  const void *logits;
  const int32_t *targets;
  const int32_t *T;
  const int32_t *U;
  int32_t N;
  int64_t rows;
  int32_t V;
  int32_t max_u;
  int32_t blank;
  uint32_t flags;
  char *ws;
  Layout lay;
  // A launch covers the whole batch (group < 0) or one of the groups of utterances
  // that `cuts` defines.  Stage 1 is cut at rows ([row_begin, row_end), host-known);
  // the later stages read the utterance boundaries stage 0 stored in the status
  // words from kStatusGroupSplit on.
  int group = -1;
  GroupCuts cuts;
  int64_t row_begin = 0;
  int64_t row_end = 0;  // 0: `rows`
  // Error reports (device views of mapped host words, or NULL), written by the
  // last kernel of the forward half:
  int32_t *report = nullptr;   // {code, utterance, sequence}: the verdict of THIS call, always stored
  int32_t *sticky = nullptr;   // {code, utterance, sequence}: stored only when the verdict is an error
  int32_t report_seq = 0;      // sequence number of this call
};

// Number of SMs of the current device (cached per device).
int sm_count();
// Grid policy of the streaming kernels.  Default: one short-lived block per
// 8 rows (or 8 runs), as many blocks as the buffer needs.  OT_B200_GRID=wave:
// exactly one resident wave of blocks that stride over the buffer.  On B200 the
// same row-per-warp in-place pass moves 6.8 TB/s with the first and 5.85 TB/s
// with the second (a read-only pass 7.5 against 7.2).
bool wave_grids();
// SMs the one-wave grids of the streaming kernels are sized for: all of them,
// or one fewer with OT_B200_SHARE_SMS, so that a kernel that is resident beside
// this path (a collective waiting for its peers) does not keep some of the
// wave's blocks from starting with the others.
inline int resident_sms(uint32_t flags) {
  const int n = sm_count();
  return ((flags & OT_B200_SHARE_SMS) && n > 1) ? n - 1 : n;
}

// Stores the message ot_b200_last_error() returns for the calling thread.
void set_last_error(const char *msg);

// For entry points that honour OT_B200_REPORT_ERRORS (see include/ot_b200.h).
// Without the flag: *sticky = NULL, returns OT_B200_OK.  With it: if an earlier
// call on this device left an error record, takes it and returns
// OT_B200_ERR_INPUT (nothing must be launched then); otherwise *sticky is the
// device view of the record a failing kernel fills in and *seq the number of
// this call.
int begin_reported_call(uint32_t flags, int32_t **sticky, int32_t *seq);

// Blocks of `kernel` that fit on one SM at `threads` threads per block.
template <typename K>
int blocks_per_sm(K kernel, int threads) {
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, 0) != cudaSuccess || n < 1) n = 1;
  return n;
}

// Ordinal of the current device, clamped to the size of the per-device caches.
constexpr int kMaxDevices = 64;
inline int current_device_slot() {
  int dev = 0;
  cudaGetDevice(&dev);
  return (dev < 0 || dev >= kMaxDevices) ? 0 : dev;
}

// Per-device cache of "dynamic shared memory opted in so far" for one kernel.
// Host threads may race here; the worst case is a redundant cudaFuncSetAttribute.
struct SmemGrant {
  std::atomic<size_t> granted[kMaxDevices];
  SmemGrant() { for (auto &g : granted) g.store(0, std::memory_order_relaxed); }
  template <typename K>
  cudaError_t ensure(K kernel, size_t bytes) {
    const int dev = current_device_slot();
    if (bytes <= granted[dev].load(std::memory_order_acquire)) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) granted[dev].store(bytes, std::memory_order_release);
    return e;
  }
};

// Programmatic dependent launch: the kernel may be scheduled while its
// predecessor in the stream is still running (its CTAs then block in pdl_wait()
// until the predecessor's memory is visible), which takes the launch latency
// and the ramp-up of a full-occupancy grid out of the gap between two stages.
// `programmatic` = false is the ordinary launch: the kernel starts when its
// predecessor in the stream has completed.  It is what a kernel with many blocks
// needs behind a kernel with few on a high-priority stream: launched
// programmatically its blocks would become resident at once, wait inside
// pdl_wait() and keep the SM slots from the streaming kernel of another stream
// that should be running there.
template <typename... Exp, typename... Act>
cudaError_t launch_maybe_pdl(bool programmatic, void (*kernel)(Exp...), unsigned grid, unsigned block,
                             size_t smem, cudaStream_t s, Act &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = programmatic ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Exp>(args)...);
}
template <typename... Exp, typename... Act>
cudaError_t launch_pdl(void (*kernel)(Exp...), unsigned grid, unsigned block, size_t smem,
                       cudaStream_t s, Act &&...args) {
  return launch_maybe_pdl(true, kernel, grid, block, smem, s, static_cast<Act &&>(args)...);
}
#ifdef __CUDACC__
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Called by one thread per block; a no-op unless the trace is switched on.
__device__ __forceinline__ void trace_begin(const int32_t *status, int stage) {
  if (status[kStatusTraceOn])
    atomicMin(reinterpret_cast<unsigned long long *>(const_cast<int32_t *>(status) + kTraceWord) + 2 * stage, global_ns());
}
__device__ __forceinline__ void trace_end(const int32_t *status, int stage) {
  if (status[kStatusTraceOn])
    atomicMax(reinterpret_cast<unsigned long long *>(const_cast<int32_t *>(status) + kTraceWord) + 2 * stage + 1, global_ns());
}
// mbarrier + one-dimensional bulk copy (TMA) helpers.
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// One-dimensional TMA copy global -> this CTA's shared memory, completion
// signalled on `bar`.  dst, src and bytes are multiples of 16.
__device__ __forceinline__ void tma_load_1d(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Utterances [lo, hi) a launch works on (see Problem::group).
__device__ __forceinline__ void group_range(const int32_t *status, int group, int N, int &lo, int &hi) {
  lo = 0;
  hi = N;
  if (group >= 0) {
    lo = status[kStatusGroupSplit + group];
    hi = status[kStatusGroupSplit + group + 1];
  }
}

// First statement of every kernel that reads what an earlier kernel wrote
// (a no-op when the kernel was launched the ordinary way) ...
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// ... and the permission for the next kernel in the stream to be scheduled.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// Host launchers, one per stage; each returns the cudaError_t of its launch.
cudaError_t launch_prepare(const Problem &p, cudaStream_t s);
cudaError_t launch_logprob(const Problem &p, cudaStream_t s);
cudaError_t launch_lattice(const Problem &p, void *scores, cudaStream_t s);
cudaError_t launch_coef(const Problem &p, void *scores, void *loss_out,
                        double loss_scale, cudaStream_t s);
cudaError_t launch_gradient(const Problem &p, void *grad, const void *d_scale,
                            double scale_host, cudaStream_t s);
// Stage 1 computed from the joiner's operands (x: (rows, D), w: (V, D), bfloat16)
// instead of from logits; fills den and lp like launch_logprob.
cudaError_t launch_linear_logprob(const Problem &p, const void *x, const void *w, const float *bias,
                                  int D, cudaStream_t s);
// In-place multiplication of a gradient by a device scalar (skipped when it is 1).
cudaError_t launch_scale(void *g, int64_t count, const void *d_scale, uint32_t flags, cudaStream_t s);
// After both groups of a two-group call: the loss and the error reports.
cudaError_t launch_close(const Problem &p, void *scores, void *loss_out, double loss_scale,
                         cudaStream_t s);

// ---------------------------------------------------------------------------
// Device helpers
// ---------------------------------------------------------------------------

// Storage type X of the logits / gradient -> type the arithmetic runs in.
// 16-bit logits (OT_B200_BF16 / OT_B200_FP16) are converted on load and rounded
// to nearest on store; everything between (logsumexp, log-probs, alpha, beta,
// scores, loss) is float32.
template <typename X> struct Real { using type = X; };
template <> struct Real<__nv_bfloat16> { using type = float; };
template <> struct Real<__half> { using type = float; };

// Widest vector a streaming kernel loads: 16 bytes for float and double; 8 bytes
// (4 elements) for the 16-bit types, whose rows are only 8-byte aligned at the
// usual vocabulary sizes (V = 500: 1000-byte rows).
template <typename X> struct Vec16;
template <> struct Vec16<float> { using type = float4; static constexpr int n = 4; };
template <> struct Vec16<double> { using type = double2; static constexpr int n = 2; };
template <> struct Vec16<__nv_bfloat16> { using type = uint2; static constexpr int n = 4; };
template <> struct Vec16<__half> { using type = uint2; static constexpr int n = 4; };

template <typename X, int VEC> struct VecOf;
template <> struct VecOf<float, 4> { using type = float4; };
template <> struct VecOf<float, 1> { using type = float; };
template <> struct VecOf<double, 2> { using type = double2; };
template <> struct VecOf<double, 1> { using type = double; };
template <> struct VecOf<__nv_bfloat16, 4> { using type = uint2; };
template <> struct VecOf<__nv_bfloat16, 1> { using type = __nv_bfloat16; };
template <> struct VecOf<__half, 4> { using type = uint2; };
template <> struct VecOf<__half, 1> { using type = __half; };

#ifdef __CUDACC__
__device__ __forceinline__ float to_real(float v) { return v; }
__device__ __forceinline__ double to_real(double v) { return v; }
__device__ __forceinline__ float to_real(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_real(__half v) { return __half2float(v); }
template <typename X> __device__ __forceinline__ X from_real(typename Real<X>::type v);
template <> __device__ __forceinline__ float from_real<float>(float v) { return v; }
template <> __device__ __forceinline__ double from_real<double>(double v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_real<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_real<__half>(float v) { return __float2half_rn(v); }
#endif

#ifdef __CUDACC__
// Two 16-bit elements in one 32-bit word <-> two floats: one or two ALU
// instructions to widen (bfloat16 is the upper half of a float), ONE conversion
// instruction to round both back (cvt.rn.bf16x2.f32 / cvt.rn.f16x2.f32).
template <typename X> struct Pair16;
template <> struct Pair16<__nv_bfloat16> {
  static __device__ __forceinline__ float2 widen(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  }
  static __device__ __forceinline__ uint32_t round(float lo, float hi) {
    const __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&r);
  }
};
template <> struct Pair16<__half> {
  static __device__ __forceinline__ float2 widen(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2 *>(&w));
  }
  static __device__ __forceinline__ uint32_t round(float lo, float hi) {
    const __half2 r = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&r);
  }
};
#endif

template <typename T> __device__ __forceinline__ T neg_inf();
template <> __device__ __forceinline__ float neg_inf<float>() { return -__int_as_float(0x7f800000); }
template <> __device__ __forceinline__ double neg_inf<double>() { return -__longlong_as_double(0x7ff0000000000000LL); }

__device__ __forceinline__ float r_exp(float x) { return expf(x); }
__device__ __forceinline__ double r_exp(double x) { return exp(x); }
__device__ __forceinline__ float r_log(float x) { return logf(x); }
__device__ __forceinline__ double r_log(double x) { return log(x); }
__device__ __forceinline__ float r_log1p(float x) { return log1pf(x); }
__device__ __forceinline__ double r_log1p(double x) { return log1p(x); }
__device__ __forceinline__ float r_max(float a, float b) { return fmaxf(a, b); }
__device__ __forceinline__ double r_max(double a, double b) { return fmax(a, b); }

constexpr float kLog2e = 1.4426950408889634f;

// 2^x by the hardware approximation (relative error about 2^-22).
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// exp(x) for the streaming kernels: one multiply and one ex2.  For the
// arguments that matter there (|x| < 30, results <= 1) the error is below
// 2e-6 relative, far inside the 1e-5 absolute gradient tolerance.  Double
// precision keeps the library routine.
__device__ __forceinline__ float s_exp(float x) { return ex2_approx(x * kLog2e); }
__device__ __forceinline__ double s_exp(double x) { return exp(x); }

template <typename T> __device__ __forceinline__ T min_log_diff();
// log(machine epsilon): below this the smaller operand of a log-add is dropped
// (optimized_transducer/csrc/cpu.cc:15-16,30).
template <> __device__ __forceinline__ float min_log_diff<float>() { return -15.9423847198486328125f; }
template <> __device__ __forceinline__ double min_log_diff<double>() { return -36.04365338911715; }

// log(exp(a) + exp(b)) with the reference's cut-off (cpu.cc:18-35): a NaN or
// too negative difference returns the larger operand.
template <typename T, bool FAST>
__device__ __forceinline__ T log_add(T a, T b) {
  // Written without branches: the correction is always evaluated, so a warp
  // never diverges inside the recursion.
  if constexpr (FAST && sizeof(T) == 4) {
    // ex2/lg2 approximations: absolute error of the correction < 3e-7.  The
    // difference is clamped instead of compared with the cut-off: below the
    // cut-off the correction is < 1.2e-7 anyway, and the clamp also turns the
    // NaN of (-inf) - (-inf) into "no correction" (fmaxf drops a NaN operand).
    float hi;  // max that propagates a NaN operand: a poisoned log-prob must stay visible
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(hi) : "f"(a), "f"(b));
    const float lo = fminf(a, b);
    const float d = fmaxf(lo - hi, -64.0f);
    float l2;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(l2) : "f"(1.0f + ex2_approx(d * kLog2e)));
    return fmaf(l2, 0.6931471805599453f, hi);
  } else {
    const T hi = (a < b) ? b : a;
    const T d = (a < b) ? (a - b) : (b - a);
    const T corr = r_log1p(r_exp(d));
    return (d >= min_log_diff<T>()) ? hi + corr : hi;
  }
}

template <typename T>
__device__ __forceinline__ T warp_max(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = r_max(v, __shfl_xor_sync(kFull, v, o));
  return v;
}
template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
  return v;
}

// Utterance that owns `row`: the b with split[b] <= row < split[b+1].
__device__ __forceinline__ int find_utt(const int64_t *__restrict__ split, int N,
                                        int64_t row) {
  int lo = 0, hi = N;  // invariant: split[lo] <= row < split[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(split + mid) <= row) lo = mid; else hi = mid;
  }
  return lo;
}

// The same search with ordinary loads, for a table in shared memory.
__device__ __forceinline__ int find_utt_plain(const int64_t *split, int N, int64_t row) {
  int lo = 0, hi = N;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (split[mid] <= row) lo = mid; else hi = mid;
  }
  return lo;
}

}  // namespace otb
