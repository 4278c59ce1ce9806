/* Shared by the backward restatements (test infrastructure only; no counterpart in the reference).
 * With magnitude mode on, every backward function of the oracle adds |term| wherever it normally adds
 * term, so its outputs become the sum of absolute contributions per gradient element: the scale the
 * tests multiply their relative tolerance with.  The terms themselves are computed exactly as in
 * normal mode.  The switch is process-wide: not for concurrent callers. */
#ifndef HINGE_ORACLE_TERMS_H
#define HINGE_ORACLE_TERMS_H
#include <math.h>
extern int ho_magnitude_mode;
static inline float ho_term(float t) { return ho_magnitude_mode ? fabsf(t) : t; }
#endif
