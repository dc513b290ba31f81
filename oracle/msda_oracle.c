/*
 * TEST INFRASTRUCTURE - not part of the product.
 *
 * CPU oracle for multi-scale deformable attention (forward and backward), a
 * plain-C restatement of the reference operator's arithmetic.  It exists so that
 * the CUDA kernels can be checked on machines where the reference library is not
 * installed.  Only tests, the smoke check and the benchmark's CPU-baseline leg
 * may load it; the product never does.
 *
 * Parity status: PINNED.  tests/test_oracle_golden.py checks this file against
 * fixtures produced by running the reference library itself (its eager backend
 * with torch autograd, and its grid_sample reference) - see
 * tests/golden/make_golden.py - and against the reference's own known-answer
 * boundary table (tests/deformops/test_msda_eager.py:54-80 in the reference).
 *
 * Build: make -C oracle   (gcc -O2 -fopenmp, no fast-math, no FMA contraction)
 */
#include <math.h>
#include <stdint.h>

#define MSDA_ORACLE_MAX_POINTS 256 /* L*K bound for the on-stack softmax scratch */

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)

#define REAL float
#define FN(name) CAT(name, _f32)
#define FLOOR floorf
#define EXP expf
#include "msda_oracle_body.inc"
#undef REAL
#undef FN
#undef FLOOR
#undef EXP

#define REAL double
#define FN(name) CAT(name, _f64)
#define FLOOR floor
#define EXP exp
#include "msda_oracle_body.inc"
#undef REAL
#undef FN
#undef FLOOR
#undef EXP

int msda_oracle_max_points(void) { return MSDA_ORACLE_MAX_POINTS; }
