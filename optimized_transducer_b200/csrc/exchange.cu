// Exchange of one scalar per rank between the GPUs of a node over peer memory:
// the sum of the per-shard losses of a batch that is sharded by utterance.
//
// The reference is single-GPU and has no counterpart.  The usual way, an NCCL
// all-reduce of the 0-dim loss, puts a fat kernel beside the streaming kernels
// of this path: those fill every SM with exactly one wave of blocks, so the
// collective either waits until they end or keeps part of the next wave from
// starting.  Here nothing waits on the critical path:
//
//   publish  (1 warp)  rank r stores {value, seq} into entry [slot][r] of EVERY
//                      rank's table, with plain stores through peer-mapped
//                      pointers (NVLink / NVSwitch); value first, then a
//                      system-scope release store of seq.  It never waits.
//   gather   (1 warp)  lane p polls entry [slot][p] of the OWN table until its
//                      seq is the expected one, then the values are summed in
//                      rank order (the same order, hence the same bits, on every
//                      rank).  The poll is bounded by a time limit; on expiry
//                      the error word is set, the result is NaN and the kernel
//                      returns.  32 threads and a handful of registers: it fits
//                      beside a full wave of the gradient kernel.
//
// A table is ring x world entries of 16 bytes, zero-initialised by the caller
// before any rank publishes (seq 0 = nothing); step k uses slot k % ring and
// seq k + 1, so a gather can tell an entry that was overwritten by a rank more
// than `ring` steps ahead (error 2) from one that has not arrived (error 1).
#include <mutex>

#include "ot_common.cuh"

namespace otb {

namespace {

// Resources of ot_b200_exchange_allreduce: per device one highest-priority stream
// (the two one-warp kernels must be placed beside whatever streaming kernel fills
// the SMs) and two events, created on first use and kept until the process exits.
struct ExchangeLane {
  std::mutex lock;
  bool ready = false;
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, done = nullptr;
  bool pending = false;  // `done` has been recorded at least once
};
ExchangeLane g_lanes[kMaxDevices];

cudaError_t lane_init(ExchangeLane &l) {
  if (l.ready) return cudaSuccess;
  int least = 0, greatest = 0;
  cudaError_t e = cudaDeviceGetStreamPriorityRange(&least, &greatest);
  if (e != cudaSuccess) return e;
  e = cudaStreamCreateWithPriority(&l.stream, cudaStreamNonBlocking, greatest);
  if (e != cudaSuccess) return e;
  e = cudaEventCreateWithFlags(&l.fork, cudaEventDisableTiming);
  if (e != cudaSuccess) return e;
  e = cudaEventCreateWithFlags(&l.done, cudaEventDisableTiming);
  if (e != cudaSuccess) return e;
  l.ready = true;
  return cudaSuccess;
}

struct alignas(16) ExEntry {
  double value;
  unsigned long long seq;
};

template <typename T>
__global__ void __launch_bounds__(32)
exchange_publish_kernel(const T *__restrict__ value, ExEntry *const *__restrict__ tables,
                        int world, int rank, int slot, unsigned long long seq) {
  const int p = threadIdx.x;
  if (p >= world) return;
  ExEntry *e = tables[p] + (size_t)slot * world + rank;
  *reinterpret_cast<volatile double *>(&e->value) = (double)*value;
  __threadfence_system();
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(&e->seq), "l"(seq) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(32)
exchange_gather_kernel(const ExEntry *mine, int world, int slot, unsigned long long seq,
                       T *__restrict__ out, double scale, int32_t *__restrict__ error,
                       unsigned long long max_wait_ns) {
  const int p = threadIdx.x;
  double v = 0;
  int bad = 0;
  if (p < world) {
    const ExEntry *e = mine + (size_t)slot * world + p;
    const unsigned long long t0 = global_ns();
    unsigned long long s = 0;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(s) : "l"(&e->seq) : "memory");
      if (s >= seq) break;
      if (global_ns() - t0 > max_wait_ns) { bad = 1; break; }  // the wait is bounded
      __nanosleep(200);
    }
    if (!bad && s != seq) bad = 2;
    if (!bad) v = *reinterpret_cast<const volatile double *>(&e->value);
  }
  const unsigned failed = __ballot_sync(kFull, bad != 0);
  const int who = failed ? __ffs(failed) - 1 : 0;
  const int why = __shfl_sync(kFull, bad, who);
  double total = 0;
  for (int q = 0; q < world; ++q) total += __shfl_sync(kFull, v, q);
  if (p == 0) {
    if (failed) {
      // error word: 1 + rank that did not arrive in time, or 101 + rank whose
      // entry had already been overwritten by a later step
      atomicCAS(error, 0, (why == 2 ? 101 : 1) + who);
      *out = (T)__longlong_as_double(0x7ff8000000000000LL);
    } else {
      *out = (T)(total * scale);
    }
  }
}

}  // namespace

}  // namespace otb

using namespace otb;

extern "C" {

int ot_b200_exchange_bytes(int32_t world, int32_t ring, uint64_t *bytes_out) {
  if (world < 1 || world > 32 || ring < 1 || !bytes_out) {
    set_last_error("ot_b200_exchange_bytes: need 1 <= world <= 32, ring >= 1 and a result pointer");
    return OT_B200_ERR_ARGUMENT;
  }
  *bytes_out = (uint64_t)world * (uint64_t)ring * sizeof(ExEntry);
  return OT_B200_OK;
}

int ot_b200_exchange_publish(const void *d_value, uint32_t flags, void *const *d_tables,
                             int32_t world, int32_t rank, int32_t ring, uint64_t step,
                             void *stream) {
  if (!d_value || !d_tables || world < 1 || world > 32 || rank < 0 || rank >= world || ring < 1) {
    set_last_error("ot_b200_exchange_publish: bad argument");
    return OT_B200_ERR_ARGUMENT;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  ExEntry *const *tables = reinterpret_cast<ExEntry *const *>(d_tables);
  const int slot = (int)(step % (uint64_t)ring);
  if (flags & OT_B200_FP64)
    exchange_publish_kernel<double><<<1, 32, 0, s>>>(static_cast<const double *>(d_value), tables, world, rank, slot, step + 1);
  else
    exchange_publish_kernel<float><<<1, 32, 0, s>>>(static_cast<const float *>(d_value), tables, world, rank, slot, step + 1);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return OT_B200_ERR_CUDA;
  }
  return OT_B200_OK;
}

int ot_b200_exchange_allreduce(const void *d_value, void *d_out, uint32_t flags, void *const *d_tables,
                               const void *d_table, int32_t world, int32_t rank, int32_t ring,
                               uint64_t step, double scale, int32_t *d_error, uint64_t max_wait_ns,
                               void *stream) {
  if (!d_value || !d_out || !d_tables || !d_table || !d_error || world < 1 || world > 32 || rank < 0 ||
      rank >= world || ring < 1) {
    set_last_error("ot_b200_exchange_allreduce: bad argument");
    return OT_B200_ERR_ARGUMENT;
  }
  ExchangeLane &l = g_lanes[current_device_slot()];
  std::lock_guard<std::mutex> guard(l.lock);
  cudaError_t e = lane_init(l);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (e == cudaSuccess) e = cudaEventRecord(l.fork, s);             // the value is ready in `stream` order
  if (e == cudaSuccess) e = cudaStreamWaitEvent(l.stream, l.fork, 0);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return OT_B200_ERR_CUDA;
  }
  int rc = ot_b200_exchange_publish(d_value, flags, d_tables, world, rank, ring, step, l.stream);
  if (rc) return rc;
  rc = ot_b200_exchange_gather(d_table, world, ring, step, d_out, flags, scale, d_error, max_wait_ns, l.stream);
  if (rc) return rc;
  e = cudaEventRecord(l.done, l.stream);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return OT_B200_ERR_CUDA;
  }
  l.pending = true;
  return OT_B200_OK;
}

int ot_b200_exchange_wait(void *stream) {
  ExchangeLane &l = g_lanes[current_device_slot()];
  std::lock_guard<std::mutex> guard(l.lock);
  if (!l.pending) return OT_B200_OK;
  const cudaError_t e = cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), l.done, 0);
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return OT_B200_ERR_CUDA;
  }
  return OT_B200_OK;
}

int ot_b200_exchange_gather(const void *d_table, int32_t world, int32_t ring, uint64_t step,
                            void *d_out, uint32_t flags, double scale, int32_t *d_error,
                            uint64_t max_wait_ns, void *stream) {
  if (!d_table || !d_out || !d_error || world < 1 || world > 32 || ring < 1) {
    set_last_error("ot_b200_exchange_gather: bad argument");
    return OT_B200_ERR_ARGUMENT;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const ExEntry *mine = static_cast<const ExEntry *>(d_table);
  const int slot = (int)(step % (uint64_t)ring);
  if (flags & OT_B200_FP64)
    exchange_gather_kernel<double><<<1, 32, 0, s>>>(mine, world, slot, step + 1, static_cast<double *>(d_out), scale, d_error, max_wait_ns);
  else
    exchange_gather_kernel<float><<<1, 32, 0, s>>>(mine, world, slot, step + 1, static_cast<float *>(d_out), scale, d_error, max_wait_ns);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    return OT_B200_ERR_CUDA;
  }
  return OT_B200_OK;
}

}  // extern "C"
