// ot_b200_scores_noalloc: per-utterance log-likelihoods from log-softmax input,
// for callers that cannot hand the library a workspace.
//
// Who needs this: code that runs under a fixed device-memory budget.  An
// inference server that gives the whole GPU to its own arena at start-up, or a
// plug-in whose "execute" hook is forbidden to allocate, has no way to create
// the workspace the other entry points ask for: cudaMalloc either fails (no
// memory is left outside the arena) or is not allowed at that point.  This
// entry point therefore allocates nothing, neither on the device nor through
// any library: its only scratch, the alpha lattice, lives in a fixed array
// that is part of the library image.
//
// Price and limits:
//  * The array is reserved on EVERY GPU that loads the library, until the
//    process exits: kMaxCells floats + a header = 16 MiB.
//  * A batch may have at most kMaxCells lattice cells (sum_b T_b*(U_b+1));
//    larger batches are rejected with OT_B200_ERR_ARGUMENT.
//  * float32, standard transducer, log-softmax input, scores only (no
//    gradient).  It is a variant of the alpha recursion of lattice.cu that
//    keeps the wavefront in (this) global memory and gathers the two
//    log-probabilities of a cell straight from the input.
//  * All calls share the one array and it keeps whatever the previous call left
//    in it.  Every alpha cell is written before it is read, so stale values are
//    harmless; the header words (error flag) are cleared at the start of every
//    call.  Two calls whose kernels overlap on the GPU (different streams)
//    race on the array: serialise them.
//  * The first call on a device looks up the array's device address
//    (cudaGetSymbolAddress) and caches it.  Make that first call outside any
//    stream capture.
#include <stdio.h>

#include "ot_common.cuh"

namespace otb {
namespace {

constexpr int64_t kMaxCells = 4ll << 20;  // 4 Mi cells
constexpr int kHeaderFloats = 64;         // [0] error flag (int), rest unused

// The scratch.  In host code this name is only a handle for
// cudaGetSymbolAddress, never a pointer a kernel may be given.
static __device__ __align__(256) float g_alpha_scratch[kHeaderFloats + kMaxCells];

// One CTA per utterance; thread i owns the columns i, i+blockDim, ...
// Recursion of ComputeAlpha (optimized_transducer/csrc/cpu.cc:187-240).
__global__ void __launch_bounds__(1024)
scores_noalloc_kernel(const float *__restrict__ logp, const int32_t *__restrict__ targets,
                      const int32_t *__restrict__ Tl, const int32_t *__restrict__ Ul,
                      int N, int64_t rows, int V, int max_u, int blank,
                      float *scratch, float *__restrict__ scores) {
  int *flag = reinterpret_cast<int *>(scratch);
  float *cells = scratch + kHeaderFloats;
  const int b = blockIdx.x;
  // First row of this utterance (N is small; every CTA sums the lengths before
  // it).  An invalid length ANYWHERE before this utterance makes its offset
  // meaningless, so it is rejected as well: no pointer is formed from lengths
  // that have not been checked, and the sum runs over clamped values, so it can
  // neither go negative nor overflow.
  int64_t off = 0;
  bool bad = false;
  for (int i = 0; i < b; ++i) {
    const int ti = Tl[i], ui = Ul[i];
    bad |= (ti <= 0 || ui < 0 || ui > max_u);
    off += (int64_t)max(ti, 0) * (min(max(ui, 0), max_u) + 1);
  }
  const int Tn = Tl[b], U = Ul[b], U1 = U + 1;
  bad |= (Tn <= 0 || U < 0 || U > max_u);
  if (bad || off + (int64_t)Tn * U1 > rows || off + (int64_t)Tn * U1 > kMaxCells) {
    if (threadIdx.x == 0) { atomicExch(flag, 1 + b); scores[b] = __int_as_float(0x7fc00000); }
    return;
  }
  float *al = cells + off;
  const float *x = logp + off * (int64_t)V;
  const int32_t *tg = targets + (int64_t)b * max_u;
  auto blank_lp = [&](int t, int u) { return x[((int64_t)t * U1 + u) * V + blank]; };
  // a target outside [0, V) is not dereferenced: it poisons the score instead
  auto sym_lp = [&](int t, int u) {
    const int v = tg[u];
    return ((unsigned)v < (unsigned)V) ? x[((int64_t)t * U1 + u) * V + v] : __int_as_float(0x7fc00000);
  };
  if (threadIdx.x == 0) al[0] = 0.f;
  __syncthreads();
  for (int d = 1; d <= Tn - 1 + U; ++d) {
    for (int u = threadIdx.x; u < U1; u += blockDim.x) {
      const int t = d - u;
      if (t < 0 || t >= Tn) continue;
      float nv;
      if (u == 0) nv = al[(int64_t)(t - 1) * U1] + blank_lp(t - 1, 0);
      else if (t == 0) nv = al[u - 1] + sym_lp(0, u - 1);
      else nv = log_add<float, false>(al[(int64_t)(t - 1) * U1 + u] + blank_lp(t - 1, u),
                                      al[(int64_t)t * U1 + u - 1] + sym_lp(t, u - 1));
      al[(int64_t)t * U1 + u] = nv;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) scores[b] = al[(int64_t)(Tn - 1) * U1 + U] + blank_lp(Tn - 1, U);
}

// Device address of the scratch on the current device, looked up once per device.
cudaError_t scratch_address(float **out) {
  static std::atomic<float *> cached[kMaxDevices];  // zero-initialised; a race only repeats the lookup
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  float *p = cached[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_alpha_scratch);
    if (e != cudaSuccess) return e;
    cached[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return cudaSuccess;
}

}  // namespace
}  // namespace otb

extern "C" {

int ot_b200_scores_noalloc(const float *d_log_probs, const int32_t *d_targets,
                           const int32_t *d_logit_lengths, const int32_t *d_target_lengths,
                           int32_t N, int64_t rows, int32_t V, int32_t max_u, int32_t blank,
                           float *d_scores, void *stream) {
  using namespace otb;
  auto fail = [](int code, const char *msg) {
    set_last_error(msg);  // readable through ot_b200_last_error()
    return code;
  };
  if (N <= 0 || rows <= 0 || V <= 0 || max_u < 0 || blank < 0 || blank >= V)
    return fail(OT_B200_ERR_ARGUMENT, "ot_b200_scores_noalloc: bad N, rows, V, max_u or blank");
  if (!d_log_probs || !d_logit_lengths || !d_target_lengths || !d_scores || (max_u > 0 && !d_targets))
    return fail(OT_B200_ERR_ARGUMENT, "ot_b200_scores_noalloc: a required device pointer is NULL");
  if (rows > kMaxCells) {
    char msg[256];
    snprintf(msg, sizeof(msg),
             "ot_b200_scores_noalloc: %lld lattice cells exceed the built-in scratch of %lld cells; "
             "use ot_b200_forward with a caller-provided workspace",
             (long long)rows, (long long)kMaxCells);
    return fail(OT_B200_ERR_ARGUMENT, msg);
  }
  float *scratch = nullptr;
  cudaError_t e = scratch_address(&scratch);
  if (e != cudaSuccess) return fail(OT_B200_ERR_CUDA, cudaGetErrorString(e));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the header must start at zero; the cells need no clearing
  e = cudaMemsetAsync(scratch, 0, kHeaderFloats * sizeof(float), s);
  if (e != cudaSuccess) return fail(OT_B200_ERR_CUDA, cudaGetErrorString(e));
  int threads = ((max_u + 1 + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  scores_noalloc_kernel<<<(unsigned)N, threads, 0, s>>>(d_log_probs, d_targets, d_logit_lengths,
                                                        d_target_lengths, N, rows, V, max_u, blank,
                                                        scratch, d_scores);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(OT_B200_ERR_CUDA, cudaGetErrorString(e));
  return OT_B200_OK;
}

}  // extern "C"
