/*
 * CPU oracle for the oxmera matmul path.  TEST INFRASTRUCTURE ONLY.
 *
 * Nothing in the shipped library links, loads or calls this file.  It exists
 * so that tests, the smoke check and the bench's CPU-baseline leg have a
 * ground truth to compare the CUDA path against.
 *
 * What it restates: oxmera's CPU reference backend, whose matmul body is
 * `todo!()` in the reference tree (crates/oxmera-cpu/src/lib.rs:71-76).  The
 * behaviour is therefore taken from the contract and the spec that pin it:
 *   - crates/oxmera-ops/src/lib.rs:53-59   [m,k] x [k,n] -> [m,n], rank 2,
 *                                          typed errors, no coercion
 *   - crates/oxmera-ops/src/lib.rs:9-19    same dtype, fresh contiguous output
 *   - exercises/a4-reference-matmul/README.md:7-19  "three nested loops",
 *                                          operands read through their views
 *   - crates/oxmera-core/src/layout.rs:6-34 element strides, signed, offset in
 *                                          elements
 *   - crates/oxmera-core/src/shape.rs:49-55 NumPy broadcasting (batch dims)
 *
 * Parity pin: the hand-computed products and laws of
 * exercises/a4-reference-matmul/tests/spec.rs:31-130 and
 * crates/oxmera-cpu/tests/harness.rs:13-24 (restated as data in
 * tests/golden/).  Accumulator width, summation order, 16-bit floats and
 * batched matmul are NOT pinned by the reference; for those this file is the
 * definition and parity is "unpinned" beyond the stated tolerances.
 */
#ifndef OXM_ORACLE_H
#define OXM_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORC_MAX_DIMS 8

/* dtype tags: identical numbering to include/oxmera_b200.h */
enum {
  ORC_F32 = 0, ORC_F64 = 1, ORC_I32 = 2, ORC_I64 = 3, ORC_U8 = 4, ORC_BOOL = 5,
  ORC_BF16 = 6, ORC_F16 = 7,
  ORC_F8E4M3 = 8, /* finite-only 1-4-3 ("fn"), max 448 */
  ORC_F8E5M2 = 9  /* IEEE-like 1-5-2 */
};

/* status codes: identical numbering to include/oxmera_b200.h */
enum {
  ORC_OK = 0,
  ORC_SHAPE_MISMATCH = 1,
  ORC_BROADCAST_INCOMPATIBLE = 2,
  ORC_DTYPE_MISMATCH = 3,
  ORC_UNSUPPORTED_DTYPE = 4,
  ORC_DEVICE_MISMATCH = 5,
  ORC_INDEX_OUT_OF_BOUNDS = 6,
  ORC_RANK_MISMATCH = 7,
  ORC_BACKEND_UNAVAILABLE = 8,
  ORC_NOT_IMPLEMENTED = 9,
  ORC_DIVIDE_BY_ZERO = 13 /* integer div met a zero divisor (crates/oxmera-ops/src/lib.rs:47-49) */
};

/* A tensor view over host memory: oxmera's Layout plus a storage pointer
 * (crates/oxmera-core/src/layout.rs:26-34). */
typedef struct {
  int32_t dtype;
  int32_t ndim;
  int64_t shape[ORC_MAX_DIMS];
  int64_t strides[ORC_MAX_DIMS]; /* elements, signed */
  int64_t offset;                /* elements */
  void *base;
} orc_view;

/* accumulation modes */
enum {
  ORC_ACC_NATIVE = 0, /* f32 running sum, k ascending: the naive reference */
  ORC_ACC_F64 = 1     /* f64 running sum: the parity oracle for f32 */
};

/* Rank-2 matmul, exactly the MatmulOps::matmul contract.  `out` must have
 * shape [m,n]; its dtype may be f32, f64, bf16 or f16 (the running sum is
 * rounded to nearest-even on store). */
int orc_matmul(const orc_view *a, const orc_view *b, const orc_view *out,
               int acc_mode, int nthreads);

/* Rank >= 2 with NumPy-broadcast leading dims (the batched extension). */
int orc_batched_matmul(const orc_view *a, const orc_view *b,
                       const orc_view *out, int acc_mode, int nthreads);

/* The fused form (no counterpart in the reference, whose nn / autograd crates
 * are empty): per output element, in the accumulator's precision,
 *   r = sum_k a b;  r += bias[n];  r = act(r);  r += out[m,n]
 * each step optional.  `bias` is NULL or a rank-1 view of N elements;
 * act: 0 none, 1 relu, 2 gelu = 0.5 x (1 + erf(x / sqrt 2)). */
int orc_matmul_fused(const orc_view *a, const orc_view *b, const orc_view *out, const orc_view *bias, int act,
                     int accumulate, int acc_mode, int nthreads);

/* The block-scaled fp8 product (OCP Microscaling Formats v1.0, MXFP8): fp8
 * operands, one E8M0 scale (a U8: 2^(e - 127), 255 = NaN) per 32 contraction
 * elements of every row of A ([.., M, K/32]) and column of B ([.., K/32, N]);
 * every output element is summed in double.  No counterpart in the reference. */
int orc_matmul_mx(const orc_view *a, const orc_view *a_scale, const orc_view *b, const orc_view *b_scale,
                  const orc_view *out);

/* Validation only: the status orc_matmul / orc_batched_matmul would return. */
int orc_check_matmul(const orc_view *a, const orc_view *b, const orc_view *out,
                     int batched);

/* The other op families of oxmera's Backend (crates/oxmera-ops/src/lib.rs:27-50,
 * 61-69), restated as plain loops: every element computed in double (i64 for
 * integer dtypes) and rounded once on store.  `out` is row-major contiguous.
 * unary op: 0 neg, 1 exp, 2 ln, 3 abs.  binary op: 0 add, 1 sub, 2 mul, 3 div,
 * operands broadcast by NumPy rules.  reduce op: 0 sum, 1 max over `axes`
 * (naxes = 0: all axes), ascending index order; max propagates NaN.  dtypes:
 * f32, f64, i32, i64, bf16, f16 with the same refusals as the device library.
 * Integer div truncates toward zero (the most negative value over -1 wraps to
 * itself); a zero divisor anywhere returns ORC_DIVIDE_BY_ZERO, with 0 stored
 * for those elements ("Integer division by zero is a typed error",
 * crates/oxmera-ops/src/lib.rs:47-49). */
int orc_unary(int op, const orc_view *a, const orc_view *out);
int orc_binary(int op, const orc_view *a, const orc_view *b, const orc_view *out);
int orc_reduce(int op, const orc_view *a, const int32_t *axes, int naxes, const orc_view *out);

/* NumPy broadcast of two shapes; returns ORC_OK or
 * ORC_BROADCAST_INCOMPATIBLE.  out_dims must hold ORC_MAX_DIMS entries. */
int orc_broadcast_shapes(const int64_t *lhs, int lhs_ndim, const int64_t *rhs,
                         int rhs_ndim, int64_t *out_dims, int *out_ndim);

/* Round-to-nearest-even conversions shared by every test input. */
uint16_t orc_f32_to_bf16(float x);
float orc_bf16_to_f32(uint16_t h);
uint16_t orc_f32_to_f16(float x);
float orc_f16_to_f32(uint16_t h);
/* fp8: nearest even, saturating to the largest finite value (NaN stays NaN). */
uint8_t orc_f32_to_fp8(float x, int32_t dtype);
float orc_fp8_to_f32(uint8_t b, int32_t dtype);

/* Counter-based synthetic data: element i of stream (seed, stream) depends
 * only on (seed, stream, i), so any slice can be generated anywhere.
 * dist: 0 = U(-1,1), 1 = N(0,1) * scale.  dtype: f32, f64, bf16, f16 or fp8;
 * any other tag returns ORC_UNSUPPORTED_DTYPE and writes nothing. */
int orc_fill(void *dst, int32_t dtype, int64_t n, uint64_t seed,
             uint64_t stream, int dist, double scale, int nthreads);

#ifdef __cplusplus
}
#endif
#endif
