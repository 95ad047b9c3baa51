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

#include <string.h>

#include <atomic>
#include <chrono>
#include <mutex>

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
    case OT_B200_TOTALS_DIFFER: return "total scores computed from forward/backward passes are not equal";
    case OT_B200_COPY_TIMEOUT: return "a bulk copy into shared memory did not complete in time";
    case OT_B200_INPUT_PACK_LENGTHS: return "packing: the lengths do not fit rows, max_t or max_u1 (the output was filled with NaN)";
    default: return "unknown input error";
  }
}

// Mapped pinned host words for the error reports, one block per device, created
// by the first call on the device that asks for a report and kept until the
// process exits (a few KB; freeing it at exit would race with the teardown of
// the CUDA context).  Layout, in int32 words:
//   [4*i .. 4*i+2], i < kReportSlots   {code, utterance, sequence} of the blocking
//                                      call whose sequence number is i mod kReportSlots
//   [4*kReportSlots .. +2]             the record of the last FAILED call that ran
//                                      with OT_B200_REPORT_ERRORS (code 0: none)
// The last kernel of the forward half stores them; nothing but kernels is ever
// enqueued on the stream.
constexpr int kReportSlots = 64;  // blocking calls in flight at once, per device
constexpr int kReportWords = 4 * kReportSlots + 4;
struct ReportBlock {
  std::atomic<int32_t *> host{nullptr};
  int32_t *dev = nullptr;
  std::atomic<uint32_t> seq{0};
};
ReportBlock g_reports[kMaxDevices];
std::mutex g_reports_mutex;

int get_reports(ReportBlock **out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return fail(OT_B200_ERR_ARGUMENT, "device ordinal %d not supported", dev);
  ReportBlock &r = g_reports[dev];
  if (r.host.load(std::memory_order_acquire) == nullptr) {
    std::lock_guard<std::mutex> lock(g_reports_mutex);
    if (r.host.load(std::memory_order_relaxed) == nullptr) {
      void *h = nullptr;
      e = cudaHostAlloc(&h, kReportWords * sizeof(int32_t), cudaHostAllocMapped);
      if (e != cudaSuccess) return fail_cuda(e, "cudaHostAlloc(error reports)");
      memset(h, 0, kReportWords * sizeof(int32_t));
      void *d = nullptr;
      e = cudaHostGetDevicePointer(&d, h, 0);
      if (e != cudaSuccess) return fail_cuda(e, "cudaHostGetDevicePointer(error reports)");
      r.dev = static_cast<int32_t *>(d);
      r.host.store(static_cast<int32_t *>(h), std::memory_order_release);
    }
  }
  *out = &r;
  return OT_B200_OK;
}

int fail_verdict(int code, int index) {
  return fail(OT_B200_ERR_INPUT, "input check failed (code %d, utterance %d): %s", code, index,
              input_error_text(code));
}

// Takes (and clears) the record of a failed OT_B200_REPORT_ERRORS call, if any.
int take_sticky(ReportBlock *r, int32_t *index, int32_t *seq) {
  volatile int32_t *s = r->host.load(std::memory_order_acquire) + 4 * kReportSlots;
  const int32_t code = s[0];
  if (code == 0) return 0;
  *index = s[1];
  *seq = s[2];
  s[0] = 0;
  return code;
}

int fail_earlier(int code, int index, int seq) {
  return fail(OT_B200_ERR_INPUT,
              "an earlier call on this device (number %d) failed (code %d, utterance %d): %s; "
              "its results are NaN and it wrote no gradient",
              seq, code, index, input_error_text(code));
}

// Resources of the grouped schedules (see run_two_groups, run_chained_groups): per
// device a few side streams and events, created by the first call that uses a
// grouped schedule and kept until the process exits.  `lock` serialises the enqueue
// sequences of concurrent host threads on one device (a sequence records and waits
// on the shared events; it takes a few tens of microseconds and never waits for the
// GPU).
struct Pipeline {
  std::mutex lock;
  bool ready = false;
  cudaStream_t side = nullptr;     // the second group's streaming kernels
  cudaStream_t urgent = nullptr;   // both groups' recursions: highest priority, so that their few
                                   // blocks are placed ahead of the streaming kernels' thousands
  cudaEvent_t ev[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  // chained groups: per group a highest-priority stream for recursion + coefficients
  // and an ordinary one for the gradient pass, and three events
  cudaStream_t chain[kMaxGroups] = {nullptr, nullptr, nullptr, nullptr};
  cudaStream_t grad[kMaxGroups] = {nullptr, nullptr, nullptr, nullptr};
  cudaEvent_t staged[kMaxGroups], coefd[kMaxGroups], done[kMaxGroups];
};
Pipeline g_pipelines[kMaxDevices];

cudaError_t pipeline_init(Pipeline &pl) {
  if (pl.ready) return cudaSuccess;
  int least = 0, greatest = 0;
  cudaError_t e = cudaDeviceGetStreamPriorityRange(&least, &greatest);
  if (e != cudaSuccess) return e;
  e = cudaStreamCreateWithPriority(&pl.side, cudaStreamNonBlocking, least);
  if (e != cudaSuccess) return e;
  e = cudaStreamCreateWithPriority(&pl.urgent, cudaStreamNonBlocking, greatest);
  if (e != cudaSuccess) return e;
  for (auto &ev : pl.ev) {
    e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (e != cudaSuccess) return e;
  }
  for (int g = 0; g < kMaxGroups; ++g) {
    e = cudaStreamCreateWithPriority(&pl.chain[g], cudaStreamNonBlocking, greatest);
    if (e != cudaSuccess) return e;
    e = cudaStreamCreateWithPriority(&pl.grad[g], cudaStreamNonBlocking, least);
    if (e != cudaSuccess) return e;
    for (cudaEvent_t *ev : {&pl.staged[g], &pl.coefd[g], &pl.done[g]}) {
      e = cudaEventCreateWithFlags(ev, cudaEventDisableTiming);
      if (e != cudaSuccess) return e;
    }
  }
  pl.ready = true;
  return cudaSuccess;
}

// OT_B200_PIPELINE=0 keeps every call on the caller's stream, one stage after
// the other (read at every call, so a process can compare the two schedules).
bool two_groups_allowed() {
  const char *e = getenv("OT_B200_PIPELINE");
  return !(e && strcmp(e, "0") == 0);
}
// OT_B200_PIPELINE=always: the chained groups for every batch they can serve,
// whatever its size (tests compare the schedules on small batches with it).
bool chained_groups_forced() {
  const char *e = getenv("OT_B200_PIPELINE");
  return e && strcmp(e, "always") == 0;
}

// OT_B200_PIPELINE=chain: the chained groups also for batches of the two-group size
// (to measure one schedule against the other on the same batch).
bool chain_preferred() {
  const char *e = getenv("OT_B200_PIPELINE");
  return e && strcmp(e, "chain") == 0;
}

// Batches below this many lattice cells (rows * V) run as one group: the
// streaming kernels of half the batch must outlast a recursion for the overlap to
// pay.  Measured, float: 343 M cells 0.725 -> 0.669 ms, 171 M cells 0.39 ms either
// way; bfloat16 (whose stage 1 is bound by exp throughput, not bytes): 343 M cells
// 0.526 -> 0.512 ms.
constexpr uint64_t kTwoGroupsMinCells = 192ull << 20;
// Below that, a batch of at least this many cells runs as up to four chained
// groups (run_chained_groups).  Measured on shards of the benchmark batch, step
// time on one stream -> chained: 16 utterances (171 M cells) 0.389 -> 0.372 ms,
// 8 utterances (86 M cells) 0.230 -> 0.223 ms, 3-5 utterances (43 M cells)
// 0.147 -> 0.148..0.153 ms: there the step is the longest utterance's own chain
// (stage 1, recursion, gradient) plus 6-10 us per cross-stream edge, and the
// schedule costs 60 us more host time per call.
constexpr uint64_t kChainedGroupsMinCells = 64ull << 20;

constexpr uint32_t kKnownFlags = OT_B200_FROM_LOG_SOFTMAX | OT_B200_ONE_SYM_PER_FRAME |
                                 OT_B200_FP64 | OT_B200_CHECK_INPUTS | OT_B200_FAST_MATH |
                                 OT_B200_SCALE_PER_UTTERANCE | OT_B200_SHARE_SMS |
                                 OT_B200_BF16 | OT_B200_FP16 | OT_B200_TRACE |
                                 OT_B200_REPORT_ERRORS | OT_B200_LINEAR_DOMAIN;

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

int begin_reported_call(uint32_t flags, int32_t **sticky, int32_t *seq) {
  *sticky = nullptr;
  *seq = 0;
  if (!(flags & OT_B200_REPORT_ERRORS)) return OT_B200_OK;
  ReportBlock *rep = nullptr;
  const int rc = get_reports(&rep);
  if (rc) return rc;
  int32_t index = 0, failed = 0;
  const int code = take_sticky(rep, &index, &failed);
  if (code) return fail_earlier(code, index, failed);
  *sticky = rep->dev + 4 * kReportSlots;
  *seq = (int32_t)((rep->seq.fetch_add(1, std::memory_order_relaxed) + 1) & 0x7fffffffu);
  return OT_B200_OK;
}

bool wave_grids() {
  static std::atomic<int> cached{-1};
  int c = cached.load(std::memory_order_relaxed);
  if (c < 0) {
    const char *e = getenv("OT_B200_GRID");
    c = (e && strcmp(e, "wave") == 0) ? 1 : 0;
    cached.store(c, std::memory_order_relaxed);
  }
  return c == 1;
}

int sm_count() {
  static std::atomic<int> cached[kMaxDevices];  // zero-initialised
  const int dev = current_device_slot();
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    n = n > 0 ? n : 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
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

namespace {

// Error reports for a forward half: takes a pending record of an earlier call
// (OT_B200_REPORT_ERRORS: returns OT_B200_ERR_INPUT, nothing must be launched),
// numbers this call and points the problem at its report words.  *slot: the
// host words a blocking call (OT_B200_CHECK_INPUTS) polls, else NULL.
int attach_reports(Problem *p, uint32_t flags, cudaStream_t s, volatile int32_t **slot) {
  *slot = nullptr;
  const bool blocking = flags & OT_B200_CHECK_INPUTS;
  const bool deferred = flags & OT_B200_REPORT_ERRORS;
  if (!blocking && !deferred) return OT_B200_OK;
  if (blocking) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaError_t e = cudaStreamIsCapturing(s, &cap);
    if (e != cudaSuccess) return fail_cuda(e, "cudaStreamIsCapturing");
    if (cap != cudaStreamCaptureStatusNone)
      return fail(OT_B200_ERR_ARGUMENT, "OT_B200_CHECK_INPUTS cannot be used while the stream is being captured");
  }
  ReportBlock *rep = nullptr;
  int rc = get_reports(&rep);
  if (rc) return rc;
  if (deferred) {
    int32_t index = 0, seq = 0;
    const int code = take_sticky(rep, &index, &seq);
    if (code) return fail_earlier(code, index, seq);
    p->sticky = rep->dev + 4 * kReportSlots;
  }
  const uint32_t seq = rep->seq.fetch_add(1, std::memory_order_relaxed) + 1;
  p->report_seq = (int32_t)(seq & 0x7fffffffu);
  if (blocking) {
    const int i = (int)(seq % kReportSlots);
    *slot = rep->host.load(std::memory_order_acquire) + 4 * i;
    p->report = rep->dev + 4 * i;
  }
  return OT_B200_OK;
}

// The whole call as two groups of utterances on three streams, so that the
// recursion of one group (a latency chain that keeps a few dozen SMs busy and
// the memory system idle) runs under the streaming kernels of the other:
//
//   caller's stream   K0  K1(a) ..........  K3(a) .............        close
//   side                  K1(b) ..........          K3(b) .............
//   urgent                      K2(a) K2c(a)  K2(b) K2c(b)
//
// Group a = the utterances that end at or before row r1 (half the batch), group
// b = the rest; stage 1 is cut at r1 itself.  Only events order the streams; the
// host never waits.  What the order relies on, as measured on B200: kernels of
// equal priority are dispatched in arrival order (a later kernel gets SM slots
// once the earlier one has handed out all its blocks), so K1(b) fills the tail
// of K1(a) and K3(b) that of K3(a) without slowing them; the recursions and the
// coefficient kernels sit on a highest-priority stream, so their few blocks are
// placed at once, under whichever streaming kernel is running.  Results are
// bitwise those of the one-stream schedule.
int run_two_groups(Problem p, void *d_grad, void *d_scores, void *d_loss, double loss_scale,
                   double grad_scale, cudaStream_t s) {
  const int dev = current_device_slot();
  Pipeline &pl = g_pipelines[dev];
  std::lock_guard<std::mutex> guard(pl.lock);
  cudaError_t e = pipeline_init(pl);
  if (e != cudaSuccess) return fail_cuda(e, "create the streams of the two-group schedule");
  const int64_t r1 = (p.rows / 2) & ~int64_t(15);  // a multiple of the stage-1 tile height
  p.cuts.n = 2;
  p.cuts.row[0] = 0; p.cuts.row[1] = r1; p.cuts.row[2] = p.rows;
  Problem a = p, b = p;
  a.group = 0; a.row_begin = 0; a.row_end = r1;
  b.group = 1; b.row_begin = r1; b.row_end = p.rows;
#define OTB_TRY(call, what)                          \
  do {                                               \
    e = (call);                                      \
    if (e != cudaSuccess) return fail_cuda(e, what); \
  } while (0)
  OTB_TRY(launch_prepare(p, s), "launch prepare");
  OTB_TRY(cudaEventRecord(pl.ev[0], s), "record");
  OTB_TRY(launch_logprob(a, s), "launch logprob");
  OTB_TRY(cudaEventRecord(pl.ev[1], s), "record");
  OTB_TRY(cudaStreamWaitEvent(pl.side, pl.ev[0], 0), "wait");      // stage 1 of group b needs stage 0 only
  OTB_TRY(launch_logprob(b, pl.side), "launch logprob");
  OTB_TRY(cudaEventRecord(pl.ev[2], pl.side), "record");
  OTB_TRY(cudaStreamWaitEvent(pl.urgent, pl.ev[1], 0), "wait");
  OTB_TRY(launch_lattice(a, d_scores, pl.urgent), "launch lattice");
  OTB_TRY(launch_coef(a, d_scores, nullptr, 1.0, pl.urgent), "launch coef");
  OTB_TRY(cudaEventRecord(pl.ev[3], pl.urgent), "record");
  OTB_TRY(cudaStreamWaitEvent(s, pl.ev[3], 0), "wait");
  OTB_TRY(launch_gradient(a, d_grad, nullptr, grad_scale, s), "launch gradient");
  // The utterance that straddles r1 belongs to group b and has rows on either
  // side of the cut: its recursion needs both halves of stage 1 (the urgent
  // stream has already waited for the first).
  OTB_TRY(cudaStreamWaitEvent(pl.urgent, pl.ev[2], 0), "wait");
  OTB_TRY(launch_lattice(b, d_scores, pl.urgent), "launch lattice");
  OTB_TRY(launch_coef(b, d_scores, nullptr, 1.0, pl.urgent), "launch coef");
  OTB_TRY(cudaEventRecord(pl.ev[4], pl.urgent), "record");
  OTB_TRY(cudaStreamWaitEvent(pl.side, pl.ev[4], 0), "wait");
  OTB_TRY(launch_gradient(b, d_grad, nullptr, grad_scale, pl.side), "launch gradient");
  OTB_TRY(cudaEventRecord(pl.ev[5], pl.side), "record");
  OTB_TRY(cudaStreamWaitEvent(s, pl.ev[5], 0), "wait");
  OTB_TRY(launch_close(p, d_scores, d_loss, loss_scale, s), "launch close");
#undef OTB_TRY
  return OT_B200_OK;
}

// The schedule for batches whose streaming kernels are SHORTER than a recursion
// (a few utterances per GPU): the batch is cut into up to four groups of
// consecutive utterances, stage 1 runs group after group on the caller's stream,
// and every group continues on streams of its own as soon as its rows are staged:
//
//   s        : K0, K1(0), K1(1), ..., K1(G-1)                      ... wait all, close
//   chain[g] :        (K1(g) done) K2(g), coef(g)                   highest priority
//   grad[g]  :                       (coef(g) done) K3(g)
//
// so the recursions of all groups run side by side (two CTAs per utterance), the
// first one starts when a G-th of stage 1 is done, and a group's gradient pass
// runs under the recursions of the groups that are still busy.  Measured on four
// utterances of the benchmark batch (what each of 8 GPUs holds): one stream is
// prepare 7 + K1 36 + K2 51 + coef 4 + K3 53 us, one after the other.
// Callers that know the lengths on the host cut at utterance boundaries, shortest
// utterances first (their gradient pass then runs while stage 1 of the later groups
// still streams); otherwise the cuts are the G-quantiles of the rows.
int run_chained_groups(Problem p, void *d_grad, void *d_scores, void *d_loss, double loss_scale,
                       double grad_scale, cudaStream_t s) {
  const int dev = current_device_slot();
  Pipeline &pl = g_pipelines[dev];
  std::lock_guard<std::mutex> guard(pl.lock);
  cudaError_t e = pipeline_init(pl);
  if (e != cudaSuccess) return fail_cuda(e, "create the streams of the grouped schedule");
  const int G = p.cuts.n;
#define OTB_TRY(call, what)                          \
  do {                                               \
    e = (call);                                      \
    if (e != cudaSuccess) return fail_cuda(e, what); \
  } while (0)
  OTB_TRY(launch_prepare(p, s), "launch prepare");
  // stage 1 of group g: the rows from its cut (rounded up to the tile height, so
  // that every launch starts on a tile) to the next group's; the rows of a group's
  // first utterance that lie before the cut belong to the previous launch
  // (a group's kernels are enqueued right behind its stage 1, not after the stage 1
  // of every group: a host that is not ahead of the device would otherwise hold
  // back the first recursion by the launches of all the others)
  int64_t begin = 0;
  for (int g = 0; g < G; ++g) {
    int64_t end = (g + 1 == G) ? p.rows : ((p.cuts.row[g + 1] + 15) & ~int64_t(15));
    if (end > p.rows) end = p.rows;
    Problem q = p;
    q.group = g;
    if (end > begin) {
      q.row_begin = begin; q.row_end = end;
      OTB_TRY(launch_logprob(q, s), "launch logprob");
      begin = end;
    }
    OTB_TRY(cudaEventRecord(pl.staged[g], s), "record");
    q.row_begin = 0; q.row_end = 0;
    OTB_TRY(cudaStreamWaitEvent(pl.chain[g], pl.staged[g], 0), "wait");
    OTB_TRY(launch_lattice(q, d_scores, pl.chain[g]), "launch lattice");
    OTB_TRY(launch_coef(q, d_scores, nullptr, 1.0, pl.chain[g]), "launch coef");
    OTB_TRY(cudaEventRecord(pl.coefd[g], pl.chain[g]), "record");
    OTB_TRY(cudaStreamWaitEvent(pl.grad[g], pl.coefd[g], 0), "wait");
    OTB_TRY(launch_gradient(q, d_grad, nullptr, grad_scale, pl.grad[g]), "launch gradient");
    OTB_TRY(cudaEventRecord(pl.done[g], pl.grad[g]), "record");
  }
  for (int g = 0; g < G; ++g) OTB_TRY(cudaStreamWaitEvent(s, pl.done[g], 0), "wait");
  OTB_TRY(launch_close(p, d_scores, d_loss, loss_scale, s), "launch close");
#undef OTB_TRY
  return OT_B200_OK;
}

// Waits (bounded) for the verdict of a call made with OT_B200_CHECK_INPUTS.
int wait_for_verdict(volatile int32_t *slot, int32_t want, cudaStream_t s) {
  const auto t0 = std::chrono::steady_clock::now();
  long spins = 0;
  while (slot[2] != want) {
    if ((++spins & 1023) == 0) {
      if (cudaStreamQuery(s) == cudaSuccess && slot[2] != want)
        return fail(OT_B200_ERR_CUDA, "the forward half did not report although the stream is idle");
      if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(60))
        return fail(OT_B200_ERR_CUDA, "timed out waiting for the report of the forward half");
    }
  }
  if (slot[kStatusCode] != 0) return fail_verdict(slot[kStatusCode], slot[kStatusIndex]);
  return OT_B200_OK;
}

}  // namespace

}  // namespace otb

namespace otb {
// fused_linear.cu
cudaError_t launch_linear_gradient(const Problem &p, const void *x, const void *w, const float *bias,
                                   int D, void *grad, const float *d_scale, float scale_host,
                                   cudaStream_t s);
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

  volatile int32_t *slot = nullptr;
  rc = attach_reports(&p, flags, s, &slot);
  if (rc) return rc;

  cudaError_t e = launch_prepare(p, s);
  if (e != cudaSuccess) return fail_cuda(e, "launch prepare");
  e = launch_logprob(p, s);
  if (e != cudaSuccess) return fail_cuda(e, "launch logprob");
  e = launch_lattice(p, d_scores, s);
  if (e != cudaSuccess) return fail_cuda(e, "launch lattice");
  e = launch_coef(p, d_scores, d_loss, loss_scale, s);
  if (e != cudaSuccess) return fail_cuda(e, "launch coef");
  // Everything has been enqueued; with OT_B200_CHECK_INPUTS wait until the last
  // forward kernel of THIS call has delivered the verdict (bounded: the stream
  // going idle without a report, or 60 s).
  if (slot) return wait_for_verdict(slot, p.report_seq, s);
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
  if (flags & OT_B200_REPORT_ERRORS) {
    ReportBlock *rep = nullptr;
    rc = get_reports(&rep);
    if (rc) return rc;
    int32_t index = 0, seq = 0;
    const int code = take_sticky(rep, &index, &seq);
    if (code) return fail_earlier(code, index, seq);
  }
  p.logits = d_logits; p.targets = nullptr; p.T = nullptr; p.U = nullptr;
  p.N = N; p.rows = rows; p.V = V; p.max_u = max_u; p.blank = blank; p.flags = flags;
  p.ws = static_cast<char *>(const_cast<void *>(d_workspace));
  cudaError_t e = launch_gradient(p, d_grad, d_scale, scale_host, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail_cuda(e, "launch gradient");
  return OT_B200_OK;
}

int ot_b200_loss_and_gradient_groups(const void *d_logits, void *d_grad, const int32_t *d_targets,
                                     const int32_t *d_logit_lengths, const int32_t *d_target_lengths,
                                     int32_t N, int64_t rows, int32_t V, int32_t max_u, int32_t blank,
                                     uint32_t flags, void *d_workspace, uint64_t workspace_bytes,
                                     void *d_scores, void *d_loss, double loss_scale, double grad_scale,
                                     const int64_t *group_rows, int32_t n_groups, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool mode_b = flags & OT_B200_FROM_LOG_SOFTMAX;
  const uint64_t es = (flags & OT_B200_FP64) ? 8 : ((flags & (OT_B200_BF16 | OT_B200_FP16)) ? 2 : 4);
  GroupCuts cuts;
  if (group_rows != nullptr || n_groups != 0) {
    if (!group_rows || n_groups < 1 || n_groups > kMaxGroups)
      return fail(OT_B200_ERR_ARGUMENT, "group_rows needs 1 to %d groups, got %d", kMaxGroups, n_groups);
    bool ok = group_rows[0] == 0 && group_rows[n_groups] == rows;
    for (int g = 0; g < n_groups; ++g) ok = ok && group_rows[g] < group_rows[g + 1];
    if (!ok)
      return fail(OT_B200_ERR_ARGUMENT, "group_rows must rise strictly from 0 to rows (%lld)", (long long)rows);
    cuts.n = n_groups;
    for (int g = 0; g <= n_groups; ++g) cuts.row[g] = group_rows[g];
  }
  const bool splittable = d_grad != nullptr && !mode_b && N >= 2 && rows >= 64 && V > 0 && two_groups_allowed();
  const uint64_t cells = (uint64_t)(rows > 0 ? rows : 0) * (uint64_t)(V > 0 ? V : 0);
  bool two = splittable && cells >= kTwoGroupsMinCells && !chain_preferred();
  bool chained = splittable && !two && cuts.n != 1 &&
                 (cells >= kChainedGroupsMinCells || chained_groups_forced() || chain_preferred());
  if (two || chained) {  // not while the stream is being captured: the schedules span several streams
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) two = chained = false;
  }
  if (!two && !chained) {
    int rc = ot_b200_forward(d_logits, d_targets, d_logit_lengths, d_target_lengths, N, rows, V,
                             max_u, blank, flags, d_workspace, workspace_bytes, d_scores, d_loss,
                             loss_scale, stream);
    if (rc || !d_grad) return rc;
    return ot_b200_backward(d_logits, d_grad, N, rows, V, max_u, blank,
                            flags & ~(OT_B200_CHECK_INPUTS | OT_B200_REPORT_ERRORS), d_workspace,
                            workspace_bytes, nullptr, grad_scale, stream);
  }
  Problem p;
  int rc = check_common(N, rows, V, max_u, blank, flags, d_workspace, workspace_bytes, &p.lay);
  if (rc) return rc;
  if (!d_logits || !d_logit_lengths || !d_target_lengths || !d_scores)
    return fail(OT_B200_ERR_ARGUMENT, "a required device pointer is NULL");
  if (max_u > 0 && !d_targets) return fail(OT_B200_ERR_ARGUMENT, "targets pointer is NULL");
  if (reinterpret_cast<uintptr_t>(d_logits) % es != 0)
    return fail(OT_B200_ERR_ARGUMENT, "logits pointer is not aligned to its element size");
  p.logits = d_logits; p.targets = d_targets; p.T = d_logit_lengths; p.U = d_target_lengths;
  p.N = N; p.rows = rows; p.V = V; p.max_u = max_u; p.blank = blank; p.flags = flags;
  p.ws = static_cast<char *>(d_workspace);
  volatile int32_t *slot = nullptr;
  rc = attach_reports(&p, flags, s, &slot);
  if (rc) return rc;
  if (two) {
    rc = run_two_groups(p, d_grad, d_scores, d_loss, loss_scale, grad_scale, s);
  } else {
    if (cuts.n == 0) {  // the G-quantiles of the rows, on tile boundaries
      const int G = N < kMaxGroups ? N : kMaxGroups;
      cuts.n = G;
      for (int g = 0; g <= G; ++g) cuts.row[g] = (g == G) ? rows : ((rows * g / G) & ~int64_t(15));
    }
    p.cuts = cuts;
    rc = run_chained_groups(p, d_grad, d_scores, d_loss, loss_scale, grad_scale, s);
  }
  if (rc) return rc;
  if (slot) return wait_for_verdict(slot, p.report_seq, s);
  return OT_B200_OK;
}

int ot_b200_loss_and_gradient(const void *d_logits, void *d_grad, const int32_t *d_targets,
                              const int32_t *d_logit_lengths, const int32_t *d_target_lengths,
                              int32_t N, int64_t rows, int32_t V, int32_t max_u, int32_t blank,
                              uint32_t flags, void *d_workspace, uint64_t workspace_bytes,
                              void *d_scores, void *d_loss, double loss_scale, double grad_scale,
                              void *stream) {
  return ot_b200_loss_and_gradient_groups(d_logits, d_grad, d_targets, d_logit_lengths, d_target_lengths,
                                          N, rows, V, max_u, blank, flags, d_workspace, workspace_bytes,
                                          d_scores, d_loss, loss_scale, grad_scale, nullptr, 0, stream);
}

int ot_b200_forward_linear(const void *d_x, const void *d_w, const float *d_bias,
                           const int32_t *d_targets, const int32_t *d_logit_lengths,
                           const int32_t *d_target_lengths, int32_t N, int64_t rows, int32_t D,
                           int32_t V, int32_t max_u, int32_t blank, uint32_t flags,
                           void *d_workspace, uint64_t workspace_bytes, void *d_scores, void *d_loss,
                           double loss_scale, void *stream) {
  if (flags & (OT_B200_FROM_LOG_SOFTMAX | OT_B200_ONE_SYM_PER_FRAME | OT_B200_FP64 | OT_B200_BF16 | OT_B200_FP16))
    return fail(OT_B200_ERR_ARGUMENT, "ot_b200_forward_linear: standard transducer, bfloat16 operands, float results; "
                                      "flags may hold OT_B200_CHECK_INPUTS, OT_B200_REPORT_ERRORS, OT_B200_FAST_MATH, OT_B200_TRACE");
  Problem p;
  int rc = check_common(N, rows, V, max_u, blank, flags, d_workspace, workspace_bytes, &p.lay);
  if (rc) return rc;
  if (!d_x || !d_w || !d_logit_lengths || !d_target_lengths || !d_scores)
    return fail(OT_B200_ERR_ARGUMENT, "a required device pointer is NULL");
  if (max_u > 0 && !d_targets) return fail(OT_B200_ERR_ARGUMENT, "targets pointer is NULL");
  if (D <= 0 || D % 8 != 0)
    return fail(OT_B200_ERR_ARGUMENT, "ot_b200_forward_linear: D must be a positive multiple of 8 (rows of 16-byte units), got %d", D);
  if (reinterpret_cast<uintptr_t>(d_x) % 16 != 0 || reinterpret_cast<uintptr_t>(d_w) % 16 != 0)
    return fail(OT_B200_ERR_ARGUMENT, "ot_b200_forward_linear: x and w must be 16-byte aligned");
  p.logits = nullptr; p.targets = d_targets; p.T = d_logit_lengths; p.U = d_target_lengths;
  p.N = N; p.rows = rows; p.V = V; p.max_u = max_u; p.blank = blank; p.flags = flags;
  p.ws = static_cast<char *>(d_workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  volatile int32_t *slot = nullptr;
  rc = attach_reports(&p, flags, s, &slot);
  if (rc) return rc;
  cudaError_t e = launch_prepare(p, s);
  if (e != cudaSuccess) return fail_cuda(e, "launch prepare");
  e = launch_linear_logprob(p, d_x, d_w, d_bias, D, s);
  if (e == cudaErrorNotSupported)
    return fail(OT_B200_ERR_CUDA, "ot_b200_forward_linear: the driver's tensor-map encoder is not available or refused the operands");
  if (e != cudaSuccess) return fail_cuda(e, "launch linear+logprob");
  e = launch_lattice(p, d_scores, s);
  if (e != cudaSuccess) return fail_cuda(e, "launch lattice");
  e = launch_coef(p, d_scores, d_loss, loss_scale, s);
  if (e != cudaSuccess) return fail_cuda(e, "launch coef");
  if (slot) return wait_for_verdict(slot, p.report_seq, s);
  return OT_B200_OK;
}

int ot_b200_backward_linear(const void *d_x, const void *d_w, const float *d_bias, int32_t N,
                            int64_t rows, int32_t D, int32_t V, int32_t max_u, int32_t blank,
                            uint32_t flags, const void *d_workspace, uint64_t workspace_bytes,
                            void *d_grad_logits, const float *d_scale, double scale_host, void *stream) {
  if (flags & (OT_B200_FROM_LOG_SOFTMAX | OT_B200_ONE_SYM_PER_FRAME | OT_B200_FP64 | OT_B200_BF16 | OT_B200_FP16 |
               OT_B200_SCALE_PER_UTTERANCE | OT_B200_CHECK_INPUTS))
    return fail(OT_B200_ERR_ARGUMENT, "ot_b200_backward_linear: standard transducer, bfloat16 operands; flags may "
                                      "hold OT_B200_REPORT_ERRORS, OT_B200_FAST_MATH, OT_B200_TRACE");
  Problem p;
  int rc = check_common(N, rows, V, max_u, blank, flags, d_workspace, workspace_bytes, &p.lay);
  if (rc) return rc;
  if (!d_x || !d_w || !d_grad_logits) return fail(OT_B200_ERR_ARGUMENT, "a required device pointer is NULL");
  if (D <= 0 || D % 8 != 0)
    return fail(OT_B200_ERR_ARGUMENT, "ot_b200_backward_linear: D must be a positive multiple of 8, got %d", D);
  if (V % 4 != 0)
    return fail(OT_B200_ERR_ARGUMENT, "ot_b200_backward_linear: V must be a multiple of 4 (8-byte groups of the bfloat16 gradient), got %d", V);
  if (reinterpret_cast<uintptr_t>(d_x) % 16 != 0 || reinterpret_cast<uintptr_t>(d_w) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(d_grad_logits) % 8 != 0)
    return fail(OT_B200_ERR_ARGUMENT, "ot_b200_backward_linear: x and w must be 16-byte, the gradient 8-byte aligned");
  p.logits = nullptr; p.targets = nullptr; p.T = nullptr; p.U = nullptr;
  p.N = N; p.rows = rows; p.V = V; p.max_u = max_u; p.blank = blank; p.flags = flags;
  p.ws = static_cast<char *>(const_cast<void *>(d_workspace));
  {  // a pending record of a failed call (the forward half of this very loss, perhaps) is raised here
    int32_t *sticky = nullptr;
    int32_t seq = 0;
    rc = begin_reported_call(flags, &sticky, &seq);
    if (rc) return rc;
  }
  const cudaError_t e = launch_linear_gradient(p, d_x, d_w, d_bias, D, d_grad_logits, d_scale, (float)scale_host,
                                               static_cast<cudaStream_t>(stream));
  if (e == cudaErrorNotSupported)
    return fail(OT_B200_ERR_CUDA, "ot_b200_backward_linear: the driver's tensor-map encoder is not available or refused the operands");
  if (e != cudaSuccess) return fail_cuda(e, "launch linear gradient");
  return OT_B200_OK;
}

int ot_b200_scale_gradient(void *d_grad, int64_t count, const void *d_scale, uint32_t flags,
                           void *stream) {
  if (!d_grad || !d_scale || count <= 0)
    return fail(OT_B200_ERR_ARGUMENT, "ot_b200_scale_gradient: NULL pointer or count <= 0");
  const uint32_t types = flags & (OT_B200_FP64 | OT_B200_BF16 | OT_B200_FP16);
  if ((flags & ~(OT_B200_FP64 | OT_B200_BF16 | OT_B200_FP16 | OT_B200_REPORT_ERRORS)) || (types & (types - 1)))
    return fail(OT_B200_ERR_ARGUMENT, "ot_b200_scale_gradient: flags may hold one of OT_B200_FP64/BF16/FP16 and OT_B200_REPORT_ERRORS");
  {  // a pending record of a failed call (the forward half of this very loss, perhaps) is raised here
    int32_t *sticky = nullptr;
    int32_t seq = 0;
    const int rc = begin_reported_call(flags, &sticky, &seq);
    if (rc) return rc;
  }
  const cudaError_t e = launch_scale(d_grad, count, d_scale, flags, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail_cuda(e, "launch scale");
  return OT_B200_OK;
}

int ot_b200_compute_transducer_loss(const void *d_logits, void *d_grad,
                                    const int32_t *d_targets,
                                    const int32_t *d_logit_lengths,
                                    const int32_t *d_target_lengths, int32_t N,
                                    int64_t rows, int32_t V, int32_t max_u, int32_t blank,
                                    uint32_t flags, void *d_workspace,
                                    uint64_t workspace_bytes, void *d_scores, void *stream) {
  return ot_b200_loss_and_gradient(d_logits, d_grad, d_targets, d_logit_lengths, d_target_lengths,
                                   N, rows, V, max_u, blank, flags, d_workspace, workspace_bytes,
                                   d_scores, nullptr, 1.0, 1.0, stream);
}

int ot_b200_poll_errors(int32_t *code_out, int32_t *index_out, int32_t *seq_out, void *stream,
                        int32_t wait) {
  if (wait) {
    const cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail_cuda(e, "synchronize");
  }
  ReportBlock *rep = nullptr;
  const int rc = get_reports(&rep);
  if (rc) return rc;
  int32_t index = 0, seq = 0;
  const int code = take_sticky(rep, &index, &seq);
  if (code_out) *code_out = code;
  if (index_out) *index_out = index;
  if (seq_out) *seq_out = seq;
  if (code) fail_earlier(code, index, seq);  // leaves the message for ot_b200_last_error()
  return OT_B200_OK;
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
  if (host[0] != 0) fail_verdict(host[0], host[1]);
  return OT_B200_OK;
}

}  // extern "C"
