// C ABI of libot_b200.so (declared in include/ot_b200.h): argument checks,
// workspace layout and the launch sequence of the stages.
//
// Host-side counterpart of ot::ComputeTransducerLoss
// (optimized_transducer/csrc/transducer-loss.cc:21-96) and
// ot::ComputeTransducerLossCuda (optimized_transducer/csrc/cuda.cu:402-457).
// Where the reference blocks on seven device-to-host reads per call
// (transducer-loss.cc:49,53,62; cuda.cu:166,169,242,245) this sequence has
// none, unless the caller asks for the input-check status.
#include <stdarg.h>
#include <stdio.h>

#include <chrono>
#include <string.h>

#include "ot_common.cuh"

namespace otb {

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int fail_cuda(cudaError_t e, const char *what) {
  return fail(OT_B200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

uint64_t align256(uint64_t x) { return (x + 255u) & ~uint64_t(255); }

const char *input_error_text(int code) {
  switch (code) {
    case OT_B200_INPUT_BAD_LOGIT_LENGTH: return "a logit length is not positive";
    case OT_B200_INPUT_BAD_TARGET_LENGTH: return "a target length is negative or exceeds targets.size(1)";
    case OT_B200_INPUT_ROWS_MISMATCH: return "logits.size(0) differs from sum(logit_lengths * (target_lengths + 1))";
    case OT_B200_INPUT_TARGET_RANGE: return "Expect targets.max() < logits.size(1) and used targets >= 0";
    case OT_B200_INPUT_MAX_U_MISMATCH: return "targets.size(1) should be equal to target_lengths.max()";
    case OT_B200_INPUT_ONE_SYM_INFEASIBLE: return "one_sym_per_frame needs target_length <= logit_length - 1";
    default: return "unknown input error";
  }
}

// Mapped pinned words for the optional input-check report, one set per host
// thread and device, created on first use and kept for the thread's lifetime.
// Stage 0 writes {code, utterance, sequence number} into them; the host polls
// the sequence number.  Nothing but kernels is ever enqueued on the stream.
struct StatusSlot {
  volatile int32_t *host = nullptr;
  int32_t *dev = nullptr;
  int32_t seq = 0;
};
thread_local StatusSlot g_slots[64];

int get_slot(StatusSlot **out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) return fail(OT_B200_ERR_ARGUMENT, "device ordinal %d not supported", dev);
  StatusSlot &s = g_slots[dev];
  if (!s.host) {
    void *h = nullptr;
    e = cudaHostAlloc(&h, kStatusWords * sizeof(int32_t), cudaHostAllocMapped);
    if (e != cudaSuccess) return fail_cuda(e, "cudaHostAlloc(status)");
    memset(h, 0, kStatusWords * sizeof(int32_t));
    void *d = nullptr;
    e = cudaHostGetDevicePointer(&d, h, 0);
    if (e != cudaSuccess) return fail_cuda(e, "cudaHostGetDevicePointer(status)");
    s.host = static_cast<volatile int32_t *>(h);
    s.dev = static_cast<int32_t *>(d);
  }
  *out = &s;
  return OT_B200_OK;
}

constexpr uint32_t kKnownFlags = OT_B200_FROM_LOG_SOFTMAX | OT_B200_ONE_SYM_PER_FRAME |
                                 OT_B200_FP64 | OT_B200_CHECK_INPUTS | OT_B200_FAST_MATH |
                                 OT_B200_SCALE_PER_UTTERANCE | OT_B200_SHARE_SMS |
                                 OT_B200_BF16 | OT_B200_FP16 | OT_B200_TRACE;

int check_sizes(int32_t N, int64_t rows, int32_t max_u, uint32_t flags) {
  if (N <= 0) return fail(OT_B200_ERR_ARGUMENT, "N must be positive, got %d", N);
  if (rows <= 0) return fail(OT_B200_ERR_ARGUMENT, "rows must be positive, got %lld", (long long)rows);
  if (max_u < 0) return fail(OT_B200_ERR_ARGUMENT, "max_u must not be negative, got %d", max_u);
  if (flags & ~kKnownFlags) return fail(OT_B200_ERR_ARGUMENT, "unknown bits in flags: 0x%x", flags);
  const uint32_t types = flags & (OT_B200_FP64 | OT_B200_BF16 | OT_B200_FP16);
  if (types & (types - 1))
    return fail(OT_B200_ERR_ARGUMENT, "at most one of OT_B200_FP64, OT_B200_BF16, OT_B200_FP16 (flags 0x%x)", flags);
  return OT_B200_OK;
}

int check_common(int32_t N, int64_t rows, int32_t V, int32_t max_u, int32_t blank,
                 uint32_t flags, const void *ws, uint64_t ws_bytes, Layout *lay) {
  int rc = check_sizes(N, rows, max_u, flags);
  if (rc) return rc;
  if (V <= 0) return fail(OT_B200_ERR_ARGUMENT, "V must be positive, got %d", V);
  if (blank < 0 || blank >= V)
    return fail(OT_B200_ERR_ARGUMENT, "blank vs logits.size(1) is %d vs %d. Expect 0 <= blank < logits.size(1)", blank, V);
  *lay = make_layout(N, rows, max_u, flags);
  if (!ws) return fail(OT_B200_ERR_WORKSPACE, "workspace is NULL");
  if (reinterpret_cast<uintptr_t>(ws) % 256 != 0)
    return fail(OT_B200_ERR_WORKSPACE, "workspace must be 256-byte aligned");
  if (ws_bytes < lay->total)
    return fail(OT_B200_ERR_WORKSPACE, "workspace has %llu bytes, %llu needed",
                (unsigned long long)ws_bytes, (unsigned long long)lay->total);
  return OT_B200_OK;
}

}  // namespace

void set_last_error(const char *msg) { snprintf(g_err, sizeof(g_err), "%s", msg); }

bool wave_grids() {
  static int cached = -1;
  if (cached < 0) {
    const char *e = getenv("OT_B200_GRID");
    cached = (e && strcmp(e, "wave") == 0) ? 1 : 0;
  }
  return cached == 1;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

Layout make_layout(int32_t N, int64_t rows, int32_t max_u, uint32_t flags) {
  const uint64_t es = (flags & OT_B200_FP64) ? 8 : 4;
  const bool mode_b = flags & OT_B200_FROM_LOG_SOFTMAX;
  const bool modified = flags & OT_B200_ONE_SYM_PER_FRAME;
  const uint64_t coef_rec = mode_b ? ((flags & OT_B200_FP64) ? sizeof(CoefB<double>) : sizeof(CoefB<float>))
                                   : ((flags & OT_B200_FP64) ? sizeof(CoefA<double>) : sizeof(CoefA<float>));
  // Cells: the host knows rows, N and max_u but not the individual lengths.
  // Standard (diagonal-major) blocks hold (T+U)*(U+1) entries, i.e. the rows of
  // the utterance plus U*(U+1) <= max_u*(max_u+1); every block is rounded up by
  // at most one entry.
  Layout l;
  l.max_cells = rows + (int64_t)N +
                (modified ? 0 : (int64_t)N * (int64_t)max_u * ((int64_t)max_u + 1));
  const uint64_t cells = (uint64_t)l.max_cells;
  uint64_t off = 0;
  l.status = off;       off = align256(off + kStatusBlockWords * sizeof(int32_t));
  l.split = off;        off = align256(off + (uint64_t)(N + 1) * sizeof(int64_t));
  l.cell_split = off;   off = align256(off + (uint64_t)(N + 1) * sizeof(int64_t));
  l.den = off;          off = align256(off + (mode_b ? 0 : (uint64_t)rows * es));
  l.lp = off;           off = align256(off + (cells + 1) * 2 * es);  // + 1: filled 16 bytes at a time
  l.alpha = off;        off = align256(off + cells * es);
  l.beta = off;         off = align256(off + cells * es);
  l.coef = off;         off = align256(off + (uint64_t)rows * coef_rec);
  l.scores_beta = off;  off = align256(off + (uint64_t)N * es);
  l.total = off;
  return l;
}

}  // namespace otb

using namespace otb;

extern "C" {

int ot_b200_abi_version(void) { return OT_B200_ABI_VERSION; }

const char *ot_b200_last_error(void) { return g_err; }

int ot_b200_workspace_layout_query(int32_t N, int64_t rows, int32_t max_u, uint32_t flags,
                                   ot_b200_workspace_layout *out) {
  if (!out) return fail(OT_B200_ERR_ARGUMENT, "out is NULL");
  int rc = check_sizes(N, rows, max_u, flags);
  if (rc) return rc;
  const Layout l = make_layout(N, rows, max_u, flags);
  out->total_bytes = l.total;
  out->status_off = l.status;
  out->split_off = l.split;
  out->cell_split_off = l.cell_split;
  out->den_off = l.den;
  out->lp_off = l.lp;
  out->alpha_off = l.alpha;
  out->beta_off = l.beta;
  out->coef_off = l.coef;
  out->scores_beta_off = l.scores_beta;
  out->max_cells = (uint64_t)l.max_cells;
  return OT_B200_OK;
}

int ot_b200_workspace_bytes(int32_t N, int64_t rows, int32_t max_u, uint32_t flags,
                            uint64_t *bytes_out) {
  if (!bytes_out) return fail(OT_B200_ERR_ARGUMENT, "bytes_out is NULL");
  int rc = check_sizes(N, rows, max_u, flags);
  if (rc) return rc;
  *bytes_out = make_layout(N, rows, max_u, flags).total;
  return OT_B200_OK;
}

int ot_b200_forward(const void *d_logits, const int32_t *d_targets,
                    const int32_t *d_logit_lengths, const int32_t *d_target_lengths,
                    int32_t N, int64_t rows, int32_t V, int32_t max_u, int32_t blank,
                    uint32_t flags, void *d_workspace, uint64_t workspace_bytes,
                    void *d_scores, void *d_loss, double loss_scale, void *stream) {
  Problem p;
  int rc = check_common(N, rows, V, max_u, blank, flags, d_workspace, workspace_bytes, &p.lay);
  if (rc) return rc;
  if (!d_logits || !d_logit_lengths || !d_target_lengths || !d_scores)
    return fail(OT_B200_ERR_ARGUMENT, "a required device pointer is NULL");
  if (max_u > 0 && !d_targets) return fail(OT_B200_ERR_ARGUMENT, "targets pointer is NULL");
  const uint64_t es = (flags & OT_B200_FP64) ? 8 : ((flags & (OT_B200_BF16 | OT_B200_FP16)) ? 2 : 4);
  if (reinterpret_cast<uintptr_t>(d_logits) % es != 0)
    return fail(OT_B200_ERR_ARGUMENT, "logits pointer is not aligned to its element size");
  p.logits = d_logits; p.targets = d_targets; p.T = d_logit_lengths; p.U = d_target_lengths;
  p.N = N; p.rows = rows; p.V = V; p.max_u = max_u; p.blank = blank; p.flags = flags;
  p.ws = static_cast<char *>(d_workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  StatusSlot *slot = nullptr;
  if (flags & OT_B200_CHECK_INPUTS) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaError_t e = cudaStreamIsCapturing(s, &cap);
    if (e != cudaSuccess) return fail_cuda(e, "cudaStreamIsCapturing");
    if (cap != cudaStreamCaptureStatusNone)
      return fail(OT_B200_ERR_ARGUMENT, "OT_B200_CHECK_INPUTS cannot be used while the stream is being captured");
    rc = get_slot(&slot);
    if (rc) return rc;
  }

  if (slot) {
    p.host_status = slot->dev;
    p.host_seq = ++slot->seq;
  }
  cudaError_t e = launch_prepare(p, s);
  if (e != cudaSuccess) return fail_cuda(e, "launch prepare");
  e = launch_logprob(p, s);
  if (e != cudaSuccess) return fail_cuda(e, "launch logprob");
  e = launch_lattice(p, d_scores, s);
  if (e != cudaSuccess) return fail_cuda(e, "launch lattice");
  e = launch_coef(p, d_scores, d_loss, loss_scale, s);
  if (e != cudaSuccess) return fail_cuda(e, "launch coef");
  if (slot) {
    // Everything has been enqueued; now wait until stage 0 of THIS call has
    // reported (it runs as soon as the stream reaches it).  Bounded: 60 s.
    const int32_t want = slot->seq;
    const auto t0 = std::chrono::steady_clock::now();
    long spins = 0;
    while (slot->host[2] != want) {
      if ((++spins & 1023) == 0) {
        if (cudaStreamQuery(s) == cudaSuccess && slot->host[2] != want)
          return fail(OT_B200_ERR_CUDA, "the input check did not report although the stream is idle");
        if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(60))
          return fail(OT_B200_ERR_CUDA, "timed out waiting for the input check");
      }
    }
    if (slot->host[kStatusCode] != 0)
      return fail(OT_B200_ERR_INPUT, "input check failed (code %d, utterance %d): %s",
                  slot->host[kStatusCode], slot->host[kStatusIndex],
                  input_error_text(slot->host[kStatusCode]));
  }
  return OT_B200_OK;
}

int ot_b200_backward(const void *d_logits, void *d_grad, int32_t N, int64_t rows,
                     int32_t V, int32_t max_u, int32_t blank, uint32_t flags,
                     const void *d_workspace, uint64_t workspace_bytes,
                     const void *d_scale, double scale_host, void *stream) {
  Problem p;
  int rc = check_common(N, rows, V, max_u, blank, flags, d_workspace, workspace_bytes, &p.lay);
  if (rc) return rc;
  if (!d_grad) return fail(OT_B200_ERR_ARGUMENT, "grad pointer is NULL");
  const bool mode_b = flags & OT_B200_FROM_LOG_SOFTMAX;
  if (!mode_b && !d_logits) return fail(OT_B200_ERR_ARGUMENT, "logits pointer is NULL");
  if (mode_b && d_grad == d_logits)
    return fail(OT_B200_ERR_ARGUMENT, "with OT_B200_FROM_LOG_SOFTMAX the gradient needs its own buffer");
  if ((flags & OT_B200_SCALE_PER_UTTERANCE) && !d_scale)
    return fail(OT_B200_ERR_ARGUMENT, "OT_B200_SCALE_PER_UTTERANCE needs d_scale (N factors)");
  p.logits = d_logits; p.targets = nullptr; p.T = nullptr; p.U = nullptr;
  p.N = N; p.rows = rows; p.V = V; p.max_u = max_u; p.blank = blank; p.flags = flags;
  p.ws = static_cast<char *>(const_cast<void *>(d_workspace));
  cudaError_t e = launch_gradient(p, d_grad, d_scale, scale_host, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail_cuda(e, "launch gradient");
  return OT_B200_OK;
}

int ot_b200_compute_transducer_loss(const void *d_logits, void *d_grad,
                                    const int32_t *d_targets,
                                    const int32_t *d_logit_lengths,
                                    const int32_t *d_target_lengths, int32_t N,
                                    int64_t rows, int32_t V, int32_t max_u, int32_t blank,
                                    uint32_t flags, void *d_workspace,
                                    uint64_t workspace_bytes, void *d_scores, void *stream) {
  int rc = ot_b200_forward(d_logits, d_targets, d_logit_lengths, d_target_lengths, N, rows,
                           V, max_u, blank, flags, d_workspace, workspace_bytes, d_scores,
                           nullptr, 1.0, stream);
  if (rc || !d_grad) return rc;
  return ot_b200_backward(d_logits, d_grad, N, rows, V, max_u, blank, flags, d_workspace,
                          workspace_bytes, nullptr, 1.0, stream);
}

int ot_b200_read_input_status(const void *d_workspace, uint64_t workspace_bytes,
                              int32_t *code_out, int32_t *index_out, void *stream) {
  if (!d_workspace || !code_out) return fail(OT_B200_ERR_ARGUMENT, "NULL argument");
  if (workspace_bytes < kStatusWords * sizeof(int32_t))
    return fail(OT_B200_ERR_WORKSPACE, "workspace too small");
  int32_t host[2] = {0, 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the status words are the first segment of every workspace
  cudaError_t e = cudaMemcpyAsync(host, d_workspace, sizeof(host), cudaMemcpyDeviceToHost, s);
  if (e != cudaSuccess) return fail_cuda(e, "copy status");
  e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail_cuda(e, "synchronize");
  *code_out = host[0];
  if (index_out) *index_out = host[1];
  if (host[0] != 0)
    fail(OT_B200_ERR_INPUT, "input check failed (code %d, utterance %d): %s", host[0], host[1],
         input_error_text(host[0]));
  return OT_B200_OK;
}

}  // extern "C"
