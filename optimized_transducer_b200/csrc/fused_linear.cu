// Stage 1 without logits: the joiner's output projection fused with the row-wise
// logsumexp and the gather of the blank / next-symbol log-probabilities.
//
//   logits[r, v] = sum_d x[r, d] * w[v, d] (+ bias[v])        x: (rows, D)  w: (V, D)  bfloat16
//   den[r]       = log sum_v exp(logits[r, v])
//   lp[cell(r)]  = (logits[r, blank] - den[r], logits[r, target(r)] - den[r])
//
// The reference materialises the (rows, V) logits and reads them back
// (`logits.logsumexp(1)`, optimized_transducer/csrc/cuda.cu:427, and
// ComputeLogProbs, optimized_transducer/csrc/kernels.cu:30-60); its README
// (README.md:3-5) names the memory of that tensor as the problem the packed
// layout reduces.  Here the tensor never exists: a 128-row tile of the product
// lives in tensor memory, the epilogue keeps a running (max, sum) per row and
// the two gathered entries, and only den and lp (12 bytes per row) are written.
//
// This is the one contraction on the path, so it runs on the 5th-generation
// tensor cores: tcgen05.mma (kind::f16, bfloat16 operands, float accumulators in
// TMEM) issued by one thread, operands staged in shared memory by TMA tensor
// copies (cp.async.bulk.tensor.2d, 128-byte swizzle, no multicast), accumulators
// read back with tcgen05.ld.  One CTA per SM, persistent over row tiles:
//
//   warp 0      TMA producer: per (row tile, column tile, K block) one A box
//               (128 rows x 64) and one B box (256 columns x 64) into a 4-stage ring
//   warp 1      MMA issuer: 4 MMAs (M=128, N=256, K=16) per K block into one of two
//               256-column TMEM accumulators; tcgen05.commit releases the stage /
//               publishes the accumulator
//   warps 2-9   epilogue: two warps per TMEM lane quarter, thread = row; each takes
//               every other 32-column chunk of the finished accumulator (bias from
//               shared memory, running max and sum, the blank / target entries picked
//               by a select tree) while the MMA warp fills the other accumulator;
//               the two halves of a row meet in shared memory at the end of its tile
//
// Every wait on an mbarrier is bounded; on expiry the CTA raises its abort flag,
// records status word kStatusCopyTimeout, all roles leave their loops, the
// producer waits (bounded) for its copies in flight, TMEM is freed and the CTA
// returns.
#include <cuda.h>  // CUtensorMap and its enums only; the encoder is looked up at run time

#include "ot_common.cuh"

namespace otb {

namespace {

constexpr int kTileM = 128;     // rows per tile = TMEM lanes
constexpr int kTileN = 256;     // columns per MMA = half of TMEM
constexpr int kBlockK = 64;     // bfloat16 elements per K block = one 128-byte swizzle row
constexpr int kMmaK = 16;       // K of one tcgen05.mma for 16-bit operands
constexpr int kRing = 4;        // shared-memory stages of the forward kernel
constexpr int kRingGrad = 3;    // ... of the gradient kernel, whose epilogue needs a staging buffer too
constexpr int kOutPitch = 18;   // words per row of a warp's 32 x 16-word output staging tile (8-byte aligned rows)
constexpr int kEpilogueWarps = 8;
constexpr int kFusedThreads = 64 + 32 * kEpilogueWarps;
constexpr int kGradEpilogueWarps = 16;  // the gradient kernel: four warps per TMEM lane quarter
constexpr int kGradThreads = 64 + 32 * kGradEpilogueWarps;
constexpr uint32_t kOutBytes = kGradEpilogueWarps * 32 * kOutPitch * 4;
constexpr int kMaxBiasColumns = 7680;  // bias staged in shared memory behind the ring: vocabularies up to this size
constexpr uint32_t kBytesA = kTileM * kBlockK * 2;   // 16 KB
constexpr uint32_t kBytesB = kTileN * kBlockK * 2;   // 32 KB
constexpr uint32_t kStageBytes = kBytesA + kBytesB;  // 48 KB
constexpr uint32_t kTmemColumns = 512;
constexpr int kSpinLimit = 1 << 22;

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Bounded wait; false when it ran out, or when another role of the CTA has given up.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, const volatile int *abort) {
  for (int spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 255) == 255 && *abort) return false;
  }
  return false;
}

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int c0, int c1, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are 128
// bytes (64 bfloat16) in the 128-byte swizzle TMA writes: 8-row groups 1024 bytes
// apart (stride byte offset), leading byte offset unused (1), descriptor version 1
// (sm_100), layout type 2 (SWIZZLE_128B).  Addresses in units of 16 bytes.
__device__ __forceinline__ uint64_t smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);   // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                        // leading byte offset, bits [16,30)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                        // version, bits [46,48)
  d |= (uint64_t)2 << 61;                        // layout type, bits [61,64)
  return d;
}

// Instruction descriptor: float accumulator (bits [4,6) = 1), bfloat16 A and B
// (bits [7,10) = [10,13) = 1), both K-major (bits 15, 16 = 0), N >> 3 at bit 17,
// M >> 4 at bit 24.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                ((uint32_t)(kTileN >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);

__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(kInstrDesc), "r"(accumulate)
      : "memory");
}

// The mbarrier receives one arrival when every MMA issued so far has completed.
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// The same load without the wait, and the wait as a statement that "produces" the
// registers, so that nothing that reads them can be scheduled above it.
__device__ __forceinline__ void tmem_load_32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_load_32_wait(uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
        "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
        "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
        "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
      :
      : "memory");
}

struct FusedShared {
  uint64_t full[kRing];        // TMA -> MMA: the stage's two boxes have landed
  uint64_t empty[kRing];       // MMA -> TMA: the stage's MMAs have completed
  uint64_t acc_full[2];        // MMA -> epilogue: the accumulator is complete
  uint64_t acc_empty[2];       // epilogue -> MMA: the accumulator has been read (one arrival per epilogue thread)
  uint32_t tmem_base;
  volatile int abort;
  float4 half[kTileM];         // (max, sum, blank entry, target entry) of the rows' second halves
};

// Element idx (0..31, may differ per lane) of a register array: a tree of selects.
__device__ __forceinline__ float pick32(const float (&x)[32], int idx) {
  float a[16], b[8], c[4], d[2];
#pragma unroll
  for (int i = 0; i < 16; ++i) a[i] = (idx & 16) ? x[i + 16] : x[i];
#pragma unroll
  for (int i = 0; i < 8; ++i) b[i] = (idx & 8) ? a[i + 8] : a[i];
#pragma unroll
  for (int i = 0; i < 4; ++i) c[i] = (idx & 4) ? b[i + 4] : b[i];
#pragma unroll
  for (int i = 0; i < 2; ++i) d[i] = (idx & 2) ? c[i + 2] : c[i];
  return (idx & 1) ? d[1] : d[0];
}

// What the gradient variant needs besides the operands (see linear_gradient_kernel).
struct GradArgs {
  const CoefA<float> *coef;   // per-row coefficient records of the forward half
  __nv_bfloat16 *grad;        // (rows, V) out
  const float *d_scale;       // device scalar or NULL
  float scale_host;
};

// Body of both kernels.  kGrad == false: stage 1 (den, lp).  kGrad == true: the
// gradient with respect to the logits, from the RECOMPUTED logits tile.
template <bool kGrad>
__device__ __forceinline__ void
linear_body(const CUtensorMap &map_x, const CUtensorMap &map_w,
            const float *__restrict__ bias, const int32_t *__restrict__ targets,
            const int32_t *__restrict__ Tl, const int32_t *__restrict__ Ul,
            const int64_t *__restrict__ split, const int64_t *__restrict__ cell_split,
            int32_t *__restrict__ status, int N, int64_t rows, int D, int V, int max_u,
            int blank, float *__restrict__ den, float *__restrict__ lp, const GradArgs ga) {
  constexpr int R = kGrad ? kRingGrad : kRing;  // stages of the operand ring
  constexpr int kEW = kGrad ? kGradEpilogueWarps : kEpilogueWarps;  // epilogue warps
  constexpr int kThreadsHere = 64 + 32 * kEW;
  extern __shared__ __align__(1024) unsigned char ring_mem[];
  __shared__ FusedShared sh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char *ring = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(ring_mem) + 1023) & ~uintptr_t(1023));  // swizzle atoms are 1024-byte aligned
  // behind the ring: the bias of every column, padded with zeros to whole column tiles
  float *bias_s = reinterpret_cast<float *>(ring + (size_t)R * kStageBytes);
  const int padded_v = ((V + kTileN - 1) / kTileN) * kTileN;
  for (int i = threadIdx.x; i < padded_v; i += kThreadsHere)
    bias_s[i] = (bias != nullptr && i < V) ? __ldg(bias + i) : 0.f;
  // gradient kernel: behind the bias, per epilogue warp a 32 x 16-word tile through
  // which a chunk of the gradient is turned from "thread = row" into row-contiguous stores
  [[maybe_unused]] uint32_t *out_s = reinterpret_cast<uint32_t *>(bias_s + padded_v);

  pdl_wait();     // stage 0 (splits, status, the -inf fill of lp) is complete
  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int i = 0; i < R; ++i) { mbar_init(&sh.full[i], 1); mbar_init(&sh.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sh.acc_full[i], 1); mbar_init(&sh.acc_empty[i], 32 * kEW); }
    sh.abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {  // one warp allocates all of tensor memory (one CTA per SM) and frees it at the end
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&sh.tmem_base)), "r"(kTmemColumns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = sh.tmem_base;
  const bool run = status[kStatusCode] == 0;  // bad inputs: nothing is computed
  if (run && threadIdx.x == 0) trace_begin(status, kGrad ? kStageGradient : kStageLogprob);

  const int64_t row_tiles = (rows + kTileM - 1) / kTileM;
  const int col_tiles = (V + kTileN - 1) / kTileN;
  const int k_blocks = (D + kBlockK - 1) / kBlockK;

  if (run && warp == 0 && lane == 0) {
    // ------------------------------ TMA producer ------------------------------
    uint32_t it = 0;  // stages handed out so far
    for (int64_t tile = blockIdx.x; tile < row_tiles && !sh.abort; tile += gridDim.x) {
      for (int ct = 0; ct < col_tiles && !sh.abort; ++ct) {
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % R;
          if (it >= R && !mbar_wait(&sh.empty[s], ((it / R) - 1) & 1, &sh.abort)) { sh.abort = 1; break; }
          unsigned char *a = ring + (size_t)s * kStageBytes;
          mbar_expect_tx(&sh.full[s], kStageBytes);
          // rows / columns past the ends of x and w are filled with zeros by the copy
          tma_load_2d(a, &map_x, kb * kBlockK, (int)(tile * kTileM), &sh.full[s]);
          tma_load_2d(a + kBytesA, &map_w, kb * kBlockK, ct * kTileN, &sh.full[s]);
        }
      }
    }
    if (sh.abort) {  // let the copies in flight land before the CTA gives its shared memory back
      __shared__ int never;  // the drain must not stop because of the abort flag itself
      never = 0;
      const volatile int *nullptr_abort = &never;
      for (uint32_t j = (it > R ? it - R : 0); j < it; ++j) mbar_wait(&sh.full[j % R], (j / R) & 1, nullptr_abort);
      atomicCAS(status + kStatusCopyTimeout, 0, 1);
    }
  } else if (run && warp == 1 && lane == 0) {
    // ------------------------------- MMA issuer -------------------------------
    uint32_t it = 0, acc_it = 0;  // stages consumed, accumulators filled
    for (int64_t tile = blockIdx.x; tile < row_tiles && !sh.abort; tile += gridDim.x) {
      for (int ct = 0; ct < col_tiles && !sh.abort; ++ct, ++acc_it) {
        const int buf = acc_it & 1;
        if (acc_it >= 2 && !mbar_wait(&sh.acc_empty[buf], ((acc_it >> 1) - 1) & 1, &sh.abort)) { sh.abort = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d = tmem + (uint32_t)(buf * kTileN);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % R;
          if (!mbar_wait(&sh.full[s], (it / R) & 1, &sh.abort)) { sh.abort = 1; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a = smem_u32(ring + (size_t)s * kStageBytes);
          const uint64_t da = smem_desc(a), db = smem_desc(a + kBytesA);
#pragma unroll
          for (int k = 0; k < kBlockK / kMmaK; ++k)  // 32 bytes further along K inside the swizzle row
            mma_bf16(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), (kb | k) != 0);
          mma_commit(&sh.empty[s]);  // the stage may be refilled once these MMAs are done
        }
        if (sh.abort) break;
        mma_commit(&sh.acc_full[buf]);
      }
    }
    if (sh.abort) atomicCAS(status + kStatusCopyTimeout, 0, 1);
  } else if (run && warp >= 2) {
   if constexpr (kGrad) {
    // --------------------------- epilogue, gradient ---------------------------
    // Thread = row, as below.  Per row the record of the coefficient kernel gives
    //   k2 = (c + beta) * log2(e) + log2(scale),   y[v] = 2^(logit[v] * log2(e) + k2)
    // (the formula of gradient16_kernel, gradient.cu), the two columns that carry a
    // second term are multiplied by 1 - exp(sub - beta), and the row's part of the
    // chunk is rounded to bfloat16 and stored; the four warps of a TMEM lane quarter
    // take every fourth chunk each and never meet.
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;
    const int r_in_tile = quarter * 32 + lane;
    const float scale_all = ga.d_scale ? ga.scale_host * __ldg(ga.d_scale) : ga.scale_host;
    const bool fold = scale_all > 0.f && scale_all < 3.0e38f;
    const float mul = fold ? 1.f : scale_all;
    const float k_scale = fold ? __log2f(scale_all) : 0.f;
    uint32_t acc_it = 0;
    for (int64_t tile = blockIdx.x; tile < row_tiles && !sh.abort; tile += gridDim.x) {
      const int64_t row = tile * kTileM + r_in_tile;
      const bool live = row < rows;
      bool zero_row = true;
      float k2 = 0.f, f_b = 1.f, f_t = 1.f;
      int tgt = -1;
      if (live) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(ga.coef + row));
        const int2 ids = __ldg(reinterpret_cast<const int2 *>(ga.coef + row) + 2);
        zero_row = ids.x == kTgtZeroRow;
        k2 = (a.x + a.y) * kLog2e + k_scale;
        const bool reachable = a.y > neg_inf<float>();  // else every term of the row is 0
        f_b = reachable ? 1.f - ex2_approx((a.z - a.y) * kLog2e) : 1.f;
        f_t = reachable ? 1.f - ex2_approx((a.w - a.y) * kLog2e) : 1.f;
        tgt = ids.x >= 0 ? ids.x : -1;
      }
      uint32_t *mine = out_s + (warp - 2) * 32 * kOutPitch;
      for (int ct = 0; ct < col_tiles && !sh.abort; ++ct, ++acc_it) {
        const int buf = acc_it & 1;
        if (!mbar_wait(&sh.acc_full[buf], (acc_it >> 1) & 1, &sh.abort)) { sh.abort = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kTileN);
        // The warp's chunks of this accumulator (c = part, part + kParts, ...); the
        // accumulator goes back to the MMA warp as soon as the warp's last load has
        // landed, before that chunk is worked on and stored.
        constexpr int kParts = kEW / 4;
        uint32_t cur[32];
        bool arrived = false;
#pragma unroll
        for (int k = 0; k < kTileN / 32 / kParts; ++k) {
          const int c = part + kParts * k;
          const int col0 = ct * kTileN + c * 32;
          if (col0 < V) {  // warp-uniform
            tmem_load_32_issue(taddr + (uint32_t)(c * 32), cur);
            tmem_load_32_wait(cur);
            if (!(k + 1 < kTileN / 32 / kParts && col0 + 32 * kParts < V)) {
              asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
              mbar_arrive(&sh.acc_empty[buf]);
              arrived = true;
            }
            if (live) {  // the collective loads are executed by every lane; the rest is per row
              float x[32];
              const float4 *bs = reinterpret_cast<const float4 *>(bias_s + col0);  // broadcast loads
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float4 bv = bs[i];
                x[4 * i + 0] = __uint_as_float(cur[4 * i + 0]) + bv.x; x[4 * i + 1] = __uint_as_float(cur[4 * i + 1]) + bv.y;
                x[4 * i + 2] = __uint_as_float(cur[4 * i + 2]) + bv.z; x[4 * i + 3] = __uint_as_float(cur[4 * i + 3]) + bv.w;
              }
#pragma unroll
              for (int i = 0; i < 32; ++i) x[i] = zero_row ? 0.f : ex2_approx(fmaf(x[i], kLog2e, k2));
              if (!fold) {  // uniform, rare: a scale that cannot move into the exponent
#pragma unroll
                for (int i = 0; i < 32; ++i) x[i] *= mul;
              }
              if ((unsigned)(blank - col0) < 32u) {  // warp-uniform
                const int bi = blank - col0;
#pragma unroll
                for (int i = 0; i < 32; ++i) x[i] = (i == bi) ? x[i] * f_b : x[i];
              }
              if ((unsigned)(tgt - col0) < 32u) {  // per row: one chunk in sixteen
                const int ti = tgt - col0;
#pragma unroll
                for (int i = 0; i < 32; ++i) x[i] = (i == ti) ? x[i] * f_t : x[i];
              }
              // round to bfloat16 pairs and leave the row's 16 words in the warp's staging tile
#pragma unroll
              for (int j = 0; j < 8; ++j)
                *reinterpret_cast<uint2 *>(mine + lane * kOutPitch + 2 * j) =
                    make_uint2(Pair16<__nv_bfloat16>::round(x[4 * j], x[4 * j + 1]),
                               Pair16<__nv_bfloat16>::round(x[4 * j + 2], x[4 * j + 3]));
            }
            __syncwarp();
            // Row-contiguous stores: a store instruction covers the 64 bytes of this chunk
            // in four rows (eight lanes of 8 bytes each), i.e. 8-12 sectors, where a
            // thread-per-row store touches 32 (measured with 8-byte stores per row: 0.30
            // of the tensor peak).  V % 4 == 0 (the launcher checks): a group of four
            // columns is inside the row or outside, and every row starts on 8 bytes.
            {
              const int pair = lane & 7;
              const bool col_ok = col0 + 4 * pair < V;
#pragma unroll
              for (int r4 = 0; r4 < 8; ++r4) {
                const int rw = 4 * r4 + (lane >> 3);
                const int64_t orow = tile * kTileM + quarter * 32 + rw;
                if (col_ok && orow < rows)
                  reinterpret_cast<uint2 *>(ga.grad + orow * (int64_t)V + col0)[pair] =
                      *reinterpret_cast<const uint2 *>(mine + rw * kOutPitch + 2 * pair);
              }
            }
            __syncwarp();  // the tile is rewritten by the next chunk
          }
        }
        if (!arrived) {  // this warp has no chunk in this column tile
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          mbar_arrive(&sh.acc_empty[buf]);
        }
      }
    }
    if (sh.abort && lane == 0) atomicCAS(status + kStatusCopyTimeout, 0, 1);
   } else {
    // -------------------------------- epilogue --------------------------------
    // TMEM lanes 32*(warp % 4) .. +31 are the ones a warp may read; the two warps of
    // a quarter take the even / the odd 32-column chunks.
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;  // 0: even chunks, writes the row; 1: odd chunks
    const int r_in_tile = quarter * 32 + lane;
    const float ninf = neg_inf<float>();
    uint32_t acc_it = 0;
    for (int64_t tile = blockIdx.x; tile < row_tiles && !sh.abort; tile += gridDim.x) {
      const int64_t row = tile * kTileM + r_in_tile;
      const bool live = row < rows;
      int tsym = -1;
      int64_t cell = 0;
      if (live) {
        const int b = find_utt(split, N, row);
        const int U = __ldg(Ul + b), U1 = U + 1;
        const int idx = (int)(row - __ldg(split + b));
        const int t = idx / U1, u = idx - t * U1;
        if (u < U) tsym = __ldg(targets + (int64_t)b * max_u + u);
        cell = __ldg(cell_split + b) + cell_pos<false>(t, u, U1);
      }
      float m = ninf, ssum = 0.f, g_blank = ninf, g_sym = ninf;
      for (int ct = 0; ct < col_tiles && !sh.abort; ++ct, ++acc_it) {
        const int buf = acc_it & 1;
        if (!mbar_wait(&sh.acc_full[buf], (acc_it >> 1) & 1, &sh.abort)) { sh.abort = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kTileN);
#pragma unroll 1
        for (int c = part; c < kTileN / 32; c += 2) {
          const int col0 = ct * kTileN + c * 32;
          if (col0 >= V) break;  // only padding columns from here on (warp-uniform)
          float x[32];
          tmem_load_32(taddr + (uint32_t)(c * 32), x);
          const float4 *bs = reinterpret_cast<const float4 *>(bias_s + col0);  // broadcast loads
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 bv = bs[i];
            x[4 * i + 0] += bv.x; x[4 * i + 1] += bv.y; x[4 * i + 2] += bv.z; x[4 * i + 3] += bv.w;
          }
          if (col0 + 32 > V) {  // the chunk that straddles V: its padding columns drop out
#pragma unroll
            for (int i = 0; i < 32; ++i) x[i] = (col0 + i < V) ? x[i] : ninf;
          }
          // the two gathered entries, when this chunk holds them
          if ((unsigned)(blank - col0) < 32u) g_blank = pick32(x, blank - col0);
          if (__any_sync(kFull, (unsigned)(tsym - col0) < 32u)) {
            const float v = pick32(x, (tsym - col0) & 31);
            if ((unsigned)(tsym - col0) < 32u) g_sym = v;
          }
          // running maximum and sum, four independent chains each
          float c0 = fmaxf(x[0], x[1]), c1 = fmaxf(x[2], x[3]), c2 = fmaxf(x[4], x[5]), c3 = fmaxf(x[6], x[7]);
#pragma unroll
          for (int i = 8; i < 32; i += 4) {
            c0 = fmaxf(c0, x[i]); c1 = fmaxf(c1, x[i + 1]); c2 = fmaxf(c2, x[i + 2]); c3 = fmaxf(c3, x[i + 3]);
          }
          const float cm = fmaxf(fmaxf(c0, c1), fmaxf(c2, c3));
          if (cm > m) { ssum *= ex2_approx((m - cm) * kLog2e); m = cm; }  // first chunk: ssum is 0
          if (m - m == 0.f) {  // an infinite maximum needs no sum
            const float mneg = -m * kLog2e;
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              s0 += ex2_approx(fmaf(x[i], kLog2e, mneg));
              s1 += ex2_approx(fmaf(x[i + 1], kLog2e, mneg));
              s2 += ex2_approx(fmaf(x[i + 2], kLog2e, mneg));
              s3 += ex2_approx(fmaf(x[i + 3], kLog2e, mneg));
            }
            ssum += (s0 + s1) + (s2 + s3);
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(&sh.acc_empty[buf]);  // one arrival per epilogue thread: the accumulator has been read
      }
      // The two halves of a row meet: part 1 leaves its (max, sum, entries), part 0 merges and writes.
      if (part == 1) sh.half[r_in_tile] = make_float4(m, ssum, g_blank, g_sym);
      asm volatile("bar.sync 2, %0;" ::"r"(32 * kEpilogueWarps) : "memory");
      if (part == 0 && live && !sh.abort) {
        const float4 o = sh.half[r_in_tile];
        const float mm = fmaxf(m, o.x);
        float tot = 0.f;
        if (mm - mm == 0.f)
          tot = ssum * ex2_approx((m - mm) * kLog2e) + o.y * ex2_approx((o.x - mm) * kLog2e);
        const float d = (mm - mm == 0.f) ? logf(tot) + mm : mm;
        const float gb = fmaxf(g_blank, o.z), gs = fmaxf(g_sym, o.w);  // the half that did not see it holds -inf
        den[row] = d;
        *reinterpret_cast<float2 *>(lp + 2 * cell) = make_float2(gb - d, tsym >= 0 ? gs - d : ninf);
      }
      asm volatile("bar.sync 2, %0;" ::"r"(32 * kEpilogueWarps) : "memory");  // half[] may be overwritten again
    }
    if (sh.abort && lane == 0) atomicCAS(status + kStatusCopyTimeout, 0, 1);
   }
  }
  // Everybody meets here, whatever happened; then tensor memory goes back.
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (run && threadIdx.x == 0) trace_end(status, kGrad ? kStageGradient : kStageLogprob);
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemColumns) : "memory");
  if (kGrad && !run) {
    // the forward half refused its inputs: the gradient is all zeros (the loss is NaN
    // and the failure is reported by the forward call's verdict)
    uint32_t *g = reinterpret_cast<uint32_t *>(ga.grad);
    const int64_t words = rows * (int64_t)V / 2;
    for (int64_t i = (int64_t)blockIdx.x * kThreadsHere + threadIdx.x; i < words; i += (int64_t)gridDim.x * kThreadsHere)
      g[i] = 0u;
  }
}

__global__ void __launch_bounds__(kFusedThreads, 1)
linear_logprob_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                      const float *__restrict__ bias, const int32_t *__restrict__ targets,
                      const int32_t *__restrict__ Tl, const int32_t *__restrict__ Ul,
                      const int64_t *__restrict__ split, const int64_t *__restrict__ cell_split,
                      int32_t *__restrict__ status, int N, int64_t rows, int D, int V, int max_u,
                      int blank, float *__restrict__ den, float *__restrict__ lp) {
  linear_body<false>(map_x, map_w, bias, targets, Tl, Ul, split, cell_split, status, N, rows, D, V, max_u,
                     blank, den, lp, GradArgs{nullptr, nullptr, nullptr, 1.f});
}

// The gradient of -sum(scores) with respect to the logits, times `scale`, in
// bfloat16, from the joiner's operands: the 128-row logits tile is recomputed on
// the tensor cores exactly as in linear_logprob_kernel (same copies, same MMAs,
// same accumulators) and the epilogue applies the formula of the streaming
// gradient pass (exp(logit + c + beta) minus the special terms on at most two
// columns, optimized_transducer/csrc/kernels.cu:522-779 of the reference) with the
// per-row records the coefficient kernel left in the workspace.  The logits are
// never stored, in the forward half or here; what is stored is the gradient tile.
__global__ void __launch_bounds__(kGradThreads, 1)
linear_gradient_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                       const float *__restrict__ bias, int32_t *__restrict__ status, int64_t rows, int D,
                       int V, int blank, const CoefA<float> *__restrict__ coef,
                       __nv_bfloat16 *__restrict__ grad, const float *__restrict__ d_scale, float scale_host) {
  linear_body<true>(map_x, map_w, bias, nullptr, nullptr, nullptr, nullptr, nullptr, status, 0, rows, D, V, 0,
                    blank, nullptr, nullptr, GradArgs{coef, grad, d_scale, scale_host});
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime (the library
// does not link libcuda).
EncodeTiledFn encoder() {
  static std::atomic<EncodeTiledFn> cached{nullptr};
  EncodeTiledFn fn = cached.load(std::memory_order_acquire);
  if (fn == nullptr) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
    cached.store(fn, std::memory_order_release);
  }
  return fn;
}

// (outer, inner) bfloat16 matrix, row-major; boxes of box_outer x 64 elements, 128-byte swizzle.
bool make_map(CUtensorMap *map, const void *base, uint64_t outer, uint64_t inner, uint32_t box_outer) {
  EncodeTiledFn fn = encoder();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {inner * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBlockK, box_outer};
  const cuuint32_t elem[2] = {1, 1};
  const auto encode = [&]() {
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = encode();
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // The encoder is a driver call and wants the device's context current on this
    // thread.  A thread that has only been handed cached memory so far (an autograd
    // worker whose first job is a small batch) has made no runtime call that binds
    // it: bind it the way the runtime does for its own calls, and ask again.
    (void)cudaFree(nullptr);
    r = encode();
  }
  return r == CUDA_SUCCESS;
}

}  // namespace

// Stage 1 from the joiner's operands.  D must be a multiple of 8 (16-byte rows),
// x and w 16-byte aligned.  Returns cudaErrorNotSupported when the tensor maps
// cannot be made.
cudaError_t launch_linear_logprob(const Problem &p, const void *x, const void *w, const float *bias,
                                  int D, cudaStream_t s) {
  CUtensorMap map_x, map_w;
  if (!make_map(&map_x, x, (uint64_t)p.rows, (uint64_t)D, kTileM) ||
      !make_map(&map_w, w, (uint64_t)p.V, (uint64_t)D, kTileN))
    return cudaErrorNotSupported;
  if (p.V > kMaxBiasColumns) return cudaErrorNotSupported;
  const int padded = ((p.V + kTileN - 1) / kTileN) * kTileN;
  // the ring, room to align it to 1024 bytes, and the bias of every (padded) column
  const size_t smem = (size_t)kRing * kStageBytes + 1024 + (size_t)padded * sizeof(float);
  static SmemGrant grant;
  cudaError_t e = grant.ensure(linear_logprob_kernel, smem);
  if (e != cudaSuccess) return e;
  const int64_t row_tiles = (p.rows + kTileM - 1) / kTileM;
  const int sms = sm_count();
  const unsigned grid = (unsigned)(row_tiles < sms ? row_tiles : sms);
  e = launch_pdl(linear_logprob_kernel, grid, (unsigned)kFusedThreads, smem, s, map_x, map_w, bias,
                 p.targets, p.T, p.U, reinterpret_cast<const int64_t *>(p.ws + p.lay.split),
                 reinterpret_cast<const int64_t *>(p.ws + p.lay.cell_split),
                 reinterpret_cast<int32_t *>(p.ws + p.lay.status), p.N, p.rows, D, p.V, p.max_u, p.blank,
                 reinterpret_cast<float *>(p.ws + p.lay.den), reinterpret_cast<float *>(p.ws + p.lay.lp));
  return e != cudaSuccess ? e : cudaGetLastError();
}

// The gradient with respect to the logits from the joiner's operands (see
// linear_gradient_kernel).  V must be a multiple of 4 and grad 8-byte aligned.
cudaError_t launch_linear_gradient(const Problem &p, const void *x, const void *w, const float *bias,
                                   int D, void *grad, const float *d_scale, float scale_host,
                                   cudaStream_t s) {
  CUtensorMap map_x, map_w;
  if (!make_map(&map_x, x, (uint64_t)p.rows, (uint64_t)D, kTileM) ||
      !make_map(&map_w, w, (uint64_t)p.V, (uint64_t)D, kTileN))
    return cudaErrorNotSupported;
  if (p.V > kMaxBiasColumns || p.V % 4 != 0) return cudaErrorNotSupported;
  const int padded = ((p.V + kTileN - 1) / kTileN) * kTileN;
  const size_t smem = (size_t)kRingGrad * kStageBytes + 1024 + (size_t)padded * sizeof(float) + kOutBytes;
  static SmemGrant grant;
  cudaError_t e = grant.ensure(linear_gradient_kernel, smem);
  if (e != cudaSuccess) return e;
  const int64_t row_tiles = (p.rows + kTileM - 1) / kTileM;
  const int sms = sm_count();
  const unsigned grid = (unsigned)(row_tiles < sms ? row_tiles : sms);
  e = launch_pdl(linear_gradient_kernel, grid, (unsigned)kGradThreads, smem, s, map_x, map_w, bias,
                 reinterpret_cast<int32_t *>(p.ws + p.lay.status), p.rows, D, p.V, p.blank,
                 reinterpret_cast<const CoefA<float> *>(p.ws + p.lay.coef),
                 static_cast<__nv_bfloat16 *>(grad), d_scale, scale_host);
  return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace otb
