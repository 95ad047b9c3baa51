/* CPU oracle for the transducer-loss hot path, in plain C.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the checker that the CUDA path is
 * compared with (tests, the smoke check, and the CPU-baseline leg of the
 * benchmark).  Nothing in the product package may call it.
 *
 * It restates the algorithm of the reference's CPU implementation,
 * optimized_transducer/csrc/cpu.cc, in float (the reference's precision) and in
 * double (the reference rejects anything but float32,
 * optimized_transducer/csrc/transducer-loss.cc:33, so the double version is the
 * only 64-bit oracle there is).  The float version is pinned against outputs of
 * the reference's own CPU build and against brute-force path enumeration.
 *
 * Build:  make -C oracle        (gcc -O2 -fopenmp -shared -fPIC)
 * Threads: the row-wise logsumexp, the per-utterance recursions and the
 * gradient rows are OpenMP loops; omp_set_num_threads via ot_oracle_set_threads.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define REAL float
#define FN(x) x##_f32
#define R_EXP expf
#define R_LOG logf
#define R_LOG1P log1pf
#define R_MIN_LOG_DIFF (-15.9423847198486328125f) /* logf(FLT_EPSILON) */
#include "transducer_oracle.inc"
#undef REAL
#undef FN
#undef R_EXP
#undef R_LOG
#undef R_LOG1P
#undef R_MIN_LOG_DIFF

#define REAL double
#define FN(x) x##_f64
#define R_EXP exp
#define R_LOG log
#define R_LOG1P log1p
#define R_MIN_LOG_DIFF (-36.04365338911715) /* log(DBL_EPSILON) */
#include "transducer_oracle.inc"
#undef REAL
#undef FN
#undef R_EXP
#undef R_LOG
#undef R_LOG1P
#undef R_MIN_LOG_DIFF

/* Sets the OpenMP thread count; returns the count in effect (1 without OpenMP). */
int ot_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}
