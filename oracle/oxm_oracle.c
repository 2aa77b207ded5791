/*
 * CPU oracle for the oxmera matmul path.  TEST INFRASTRUCTURE ONLY: see the
 * header for what it restates and how it is pinned.  Plain C, no vector
 * intrinsics, no fast-math: the loop order i-j-k and the "multiply, then add"
 * of every term are part of the definition.
 */
#include "oxm_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ */
/* 16-bit float conversions (round to nearest, ties to even)           */
/* ------------------------------------------------------------------ */

static inline uint32_t f32_bits(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  return u;
}
static inline float bits_f32(uint32_t u) {
  float x;
  memcpy(&x, &u, 4);
  return x;
}

uint16_t orc_f32_to_bf16(float x) {
  uint32_t u = f32_bits(x);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

float orc_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

uint16_t orc_f32_to_f16(float x) {
  uint32_t u = f32_bits(x);
  uint32_t sign = (u >> 16) & 0x8000u;
  uint32_t absu = u & 0x7fffffffu;
  if (absu > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);      /* NaN */
  if (absu >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);     /* >= 65536: inf */
  if (absu < 0x33000001u) return (uint16_t)sign;                  /* rounds to zero */
  int32_t exp = (int32_t)(absu >> 23) - 127;
  uint32_t man = (absu & 0x7fffffu) | 0x800000u;                  /* 24-bit significand */
  int shift = (exp < -14) ? (13 + (-14 - exp)) : 13;             /* bits to drop */
  uint32_t kept = man >> shift;
  uint32_t rem = man & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (kept & 1u))) kept++;
  uint32_t h;
  if (exp < -14) {
    h = kept; /* subnormal; a carry into bit 10 lands on the smallest normal */
  } else {
    h = ((uint32_t)(exp + 15) << 10) + (kept - 0x400u); /* carry bumps the exponent */
  }
  if (h >= 0x7c00u) h = 0x7c00u;
  return (uint16_t)(sign | h);
}

float orc_f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return bits_f32(sign);
    float v = (float)man * (1.0f / 16777216.0f); /* man * 2^-24, exact */
    return sign ? -v : v;
  }
  if (exp == 31) return bits_f32(sign | 0x7f800000u | (man << 13));
  return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* fp8 e4m3 (bias 7, no infinities, 0x7f = NaN, max 0x7e = 448) and e5m2
 * (bias 15, IEEE-like, max finite 0x7b = 57344). */
float orc_fp8_to_f32(uint8_t b, int32_t dtype) {
  const int mbits = dtype == ORC_F8E4M3 ? 3 : 2, bias = dtype == ORC_F8E4M3 ? 7 : 15;
  const int sign = b >> 7, exp = (b & 0x7f) >> mbits, man = b & ((1 << mbits) - 1);
  float v;
  if (dtype == ORC_F8E4M3 && (b & 0x7f) == 0x7f) return bits_f32(0x7fc00000u);
  if (dtype == ORC_F8E5M2 && exp == 31) v = man ? bits_f32(0x7fc00000u) : bits_f32(0x7f800000u);
  else if (exp == 0) v = ldexpf((float)man, 1 - bias - mbits);
  else v = ldexpf((float)((1 << mbits) | man), exp - bias - mbits);
  return sign ? -v : v;
}

uint8_t orc_f32_to_fp8(float x, int32_t dtype) {
  const int mbits = dtype == ORC_F8E4M3 ? 3 : 2, bias = dtype == ORC_F8E4M3 ? 7 : 15;
  const uint8_t max_code = dtype == ORC_F8E4M3 ? 0x7e : 0x7b;
  const uint32_t u = f32_bits(x);
  const uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
  const uint32_t absu = u & 0x7fffffffu;
  if (absu > 0x7f800000u) return (uint8_t)(sign | 0x7f);  /* NaN */
  if (absu == 0) return sign;
  int32_t exp = (int32_t)(absu >> 23) - 127;
  uint32_t man = (absu & 0x7fffffu) | 0x800000u;
  if ((absu >> 23) == 0) return sign;                     /* f32 subnormals are far below fp8's range */
  if (exp > 20) return (uint8_t)(sign | max_code);        /* inf and anything huge saturate */
  const int emin = 1 - bias;
  int shift = 23 - mbits + (exp < emin ? emin - exp : 0);
  if (shift > 25) return sign;                            /* below half of the smallest subnormal */
  uint32_t kept = man >> shift;
  const uint32_t rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (kept & 1u))) kept++;
  uint32_t code;
  if (exp < emin) code = kept;                            /* a carry lands on the smallest normal */
  else code = ((uint32_t)(exp + bias) << mbits) + (kept - (1u << mbits));
  if (code > max_code) code = max_code;
  return (uint8_t)(sign | code);
}

/* ------------------------------------------------------------------ */
/* shapes                                                               */
/* ------------------------------------------------------------------ */

/* crates/oxmera-core/src/shape.rs:49-55: align trailing dims; each pair must
 * be equal or contain a 1. */
int orc_broadcast_shapes(const int64_t *lhs, int lhs_ndim, const int64_t *rhs,
                         int rhs_ndim, int64_t *out_dims, int *out_ndim) {
  int n = lhs_ndim > rhs_ndim ? lhs_ndim : rhs_ndim;
  if (n > ORC_MAX_DIMS) return ORC_NOT_IMPLEMENTED;
  for (int i = 0; i < n; ++i) {
    int li = lhs_ndim - 1 - i, ri = rhs_ndim - 1 - i;
    int64_t l = li >= 0 ? lhs[li] : 1;
    int64_t r = ri >= 0 ? rhs[ri] : 1;
    int64_t o;
    if (l == r) o = l;
    else if (l == 1) o = r;
    else if (r == 1) o = l;
    else return ORC_BROADCAST_INCOMPATIBLE;
    out_dims[n - 1 - i] = o;
  }
  *out_ndim = n;
  return ORC_OK;
}

static int is_matmul_dtype(int32_t d) {
  return d == ORC_F32 || d == ORC_BF16 || d == ORC_F16 || d == ORC_F8E4M3 || d == ORC_F8E5M2;
}
static int is_out_dtype(int32_t d) { return is_matmul_dtype(d) || d == ORC_F64; }

int orc_check_matmul(const orc_view *a, const orc_view *b, const orc_view *out, int batched) {
  if (a->ndim > ORC_MAX_DIMS || b->ndim > ORC_MAX_DIMS) return ORC_NOT_IMPLEMENTED;
  if (!batched) {
    /* rank-1 operands must refuse (a4 spec.rs:78-83). */
    if (a->ndim != 2 || b->ndim != 2) return ORC_SHAPE_MISMATCH;
  } else {
    if (a->ndim < 2 || b->ndim < 2) return ORC_SHAPE_MISMATCH;
  }
  if (a->dtype != b->dtype) return ORC_DTYPE_MISMATCH;
  if (!is_matmul_dtype(a->dtype)) return ORC_UNSUPPORTED_DTYPE;
  int64_t m = a->shape[a->ndim - 2], k = a->shape[a->ndim - 1];
  int64_t kb = b->shape[b->ndim - 2], n = b->shape[b->ndim - 1];
  if (k != kb) return ORC_SHAPE_MISMATCH; /* a4 spec.rs:68-76 */
  int64_t bdims[ORC_MAX_DIMS];
  int bnd = 0;
  int st = orc_broadcast_shapes(a->shape, a->ndim - 2, b->shape, b->ndim - 2, bdims, &bnd);
  if (st != ORC_OK) return st;
  if (out) {
    if (!is_out_dtype(out->dtype)) return ORC_UNSUPPORTED_DTYPE;
    if (out->ndim != bnd + 2) return ORC_SHAPE_MISMATCH;
    for (int i = 0; i < bnd; ++i)
      if (out->shape[i] != bdims[i]) return ORC_SHAPE_MISMATCH;
    if (out->shape[bnd] != m || out->shape[bnd + 1] != n) return ORC_SHAPE_MISMATCH;
  }
  return ORC_OK;
}

/* ------------------------------------------------------------------ */
/* the triple loop                                                      */
/* ------------------------------------------------------------------ */

static inline float load_as_f32(const void *base, int32_t dtype, int64_t idx) {
  switch (dtype) {
    case ORC_F32: return ((const float *)base)[idx];
    case ORC_BF16: return orc_bf16_to_f32(((const uint16_t *)base)[idx]);
    case ORC_F16: return orc_f16_to_f32(((const uint16_t *)base)[idx]);
    default: return orc_fp8_to_f32(((const uint8_t *)base)[idx], dtype);
  }
}

static inline void store_from_f64(void *base, int32_t dtype, int64_t idx, double v) {
  switch (dtype) {
    case ORC_F64: ((double *)base)[idx] = v; break;
    case ORC_F32: ((float *)base)[idx] = (float)v; break;
    case ORC_BF16: ((uint16_t *)base)[idx] = orc_f32_to_bf16((float)v); break;
    case ORC_F16: ((uint16_t *)base)[idx] = orc_f32_to_f16((float)v); break;
    default: ((uint8_t *)base)[idx] = orc_f32_to_fp8((float)v, dtype); break;
  }
}

static inline double load_as_f64(const void *base, int32_t dtype, int64_t idx) {
  if (dtype == ORC_F64) return ((const double *)base)[idx];
  return (double)load_as_f32(base, dtype, idx);
}

typedef struct {
  const orc_view *bias; /* NULL for none */
  int act, accumulate;
} orc_epi;

static inline double activate_f64(double r, int act) {
  if (act == 1) return r > 0.0 ? r : 0.0;
  if (act == 2) return 0.5 * r * (1.0 + erf(r * 0.70710678118654752440));
  return r;
}
static inline float activate_f32(float r, int act) {
  if (act == 1) return r > 0.0f ? r : 0.0f;
  if (act == 2) return 0.5f * r * (1.0f + erff(r * 0.70710678118654752440f));
  return r;
}

typedef struct {
  const orc_view *a, *b, *out;
  orc_epi epi;
  int acc_mode;
  int64_t m, n, k, nbatch;
  int bnd;                       /* number of batch dims of the output */
  int64_t bdims[ORC_MAX_DIMS];
  int64_t a_bs[ORC_MAX_DIMS], b_bs[ORC_MAX_DIMS], o_bs[ORC_MAX_DIMS]; /* 0 where broadcast */
  int64_t next_row;              /* work counter over nbatch*m rows */
  pthread_mutex_t mu;
} mm_job;

/* One output row: i fixed, loop j then k.  The A row is staged as f32 first
 * (a pure copy through the view's strides; the arithmetic order is unchanged). */
#define ROW_KERNEL(NAME, BT, BLOAD, ACC_T, ACT)                                         \
  static void NAME(const float *arow, const BT *bptr, int64_t b_ks, int64_t b_ns,       \
                   int64_t n, int64_t k, void *obase, int32_t odt, int64_t o_off,       \
                   int64_t o_ns, const orc_epi *E) {                                    \
    for (int64_t j = 0; j < n; ++j) {                                                   \
      ACC_T acc = 0;                                                                    \
      const BT *bp = bptr + j * b_ns;                                                   \
      for (int64_t kk = 0; kk < k; ++kk) {                                              \
        ACC_T prod = (ACC_T)arow[kk] * (ACC_T)BLOAD(bp[kk * b_ks]);                     \
        acc = acc + prod;                                                               \
      }                                                                                 \
      if (E->bias)                                                                      \
        acc = acc + (ACC_T)load_as_f64(E->bias->base, E->bias->dtype,                   \
                                       E->bias->offset + j * E->bias->strides[0]);      \
      acc = ACT(acc, E->act);                                                           \
      if (E->accumulate) acc = acc + (ACC_T)load_as_f64(obase, odt, o_off + j * o_ns);  \
      store_from_f64(obase, odt, o_off + j * o_ns, (double)acc);                        \
    }                                                                                   \
  }

#define ID_F32(x) (x)
ROW_KERNEL(row_f32_native, float, ID_F32, float, activate_f32)
ROW_KERNEL(row_f32_f64, float, ID_F32, double, activate_f64)
ROW_KERNEL(row_bf16_native, uint16_t, orc_bf16_to_f32, float, activate_f32)
ROW_KERNEL(row_bf16_f64, uint16_t, orc_bf16_to_f32, double, activate_f64)
ROW_KERNEL(row_f16_native, uint16_t, orc_f16_to_f32, float, activate_f32)
ROW_KERNEL(row_f16_f64, uint16_t, orc_f16_to_f32, double, activate_f64)
#define E4M3(x) orc_fp8_to_f32((x), ORC_F8E4M3)
#define E5M2(x) orc_fp8_to_f32((x), ORC_F8E5M2)
ROW_KERNEL(row_e4m3_native, uint8_t, E4M3, float, activate_f32)
ROW_KERNEL(row_e4m3_f64, uint8_t, E4M3, double, activate_f64)
ROW_KERNEL(row_e5m2_native, uint8_t, E5M2, float, activate_f32)
ROW_KERNEL(row_e5m2_f64, uint8_t, E5M2, double, activate_f64)

static void *mm_worker(void *arg) {
  mm_job *J = (mm_job *)arg;
  const orc_view *a = J->a, *b = J->b, *o = J->out;
  const int an = a->ndim, bn = b->ndim, on = o->ndim;
  const int64_t a_ms = a->strides[an - 2], a_ks = a->strides[an - 1];
  const int64_t b_ks = b->strides[bn - 2], b_ns = b->strides[bn - 1];
  const int64_t o_ms = o->strides[on - 2], o_ns = o->strides[on - 1];
  float *arow = (float *)malloc(sizeof(float) * (size_t)(J->k > 0 ? J->k : 1));
  const int64_t total = J->nbatch * J->m;
  const int64_t chunk = 4;
  for (;;) {
    pthread_mutex_lock(&J->mu);
    int64_t r0 = J->next_row;
    J->next_row += chunk;
    pthread_mutex_unlock(&J->mu);
    if (r0 >= total) break;
    int64_t r1 = r0 + chunk < total ? r0 + chunk : total;
    for (int64_t r = r0; r < r1; ++r) {
      int64_t bi = r / J->m, i = r % J->m;
      int64_t a_off = a->offset, b_off = b->offset, o_off = o->offset;
      int64_t rem = bi;
      for (int d = J->bnd - 1; d >= 0; --d) {
        int64_t idx = rem % J->bdims[d];
        rem /= J->bdims[d];
        a_off += idx * J->a_bs[d];
        b_off += idx * J->b_bs[d];
        o_off += idx * J->o_bs[d];
      }
      a_off += i * a_ms;
      o_off += i * o_ms;
      for (int64_t kk = 0; kk < J->k; ++kk) arow[kk] = load_as_f32(a->base, a->dtype, a_off + kk * a_ks);
      const int f64 = J->acc_mode == ORC_ACC_F64;
      if (b->dtype == ORC_F32) {
        const float *bp = (const float *)b->base + b_off;
        (f64 ? row_f32_f64 : row_f32_native)(arow, bp, b_ks, b_ns, J->n, J->k, o->base, o->dtype, o_off, o_ns, &J->epi);
      } else if (b->dtype == ORC_BF16) {
        const uint16_t *bp = (const uint16_t *)b->base + b_off;
        (f64 ? row_bf16_f64 : row_bf16_native)(arow, bp, b_ks, b_ns, J->n, J->k, o->base, o->dtype, o_off, o_ns, &J->epi);
      } else if (b->dtype == ORC_F16) {
        const uint16_t *bp = (const uint16_t *)b->base + b_off;
        (f64 ? row_f16_f64 : row_f16_native)(arow, bp, b_ks, b_ns, J->n, J->k, o->base, o->dtype, o_off, o_ns, &J->epi);
      } else if (b->dtype == ORC_F8E4M3) {
        const uint8_t *bp = (const uint8_t *)b->base + b_off;
        (f64 ? row_e4m3_f64 : row_e4m3_native)(arow, bp, b_ks, b_ns, J->n, J->k, o->base, o->dtype, o_off, o_ns, &J->epi);
      } else {
        const uint8_t *bp = (const uint8_t *)b->base + b_off;
        (f64 ? row_e5m2_f64 : row_e5m2_native)(arow, bp, b_ks, b_ns, J->n, J->k, o->base, o->dtype, o_off, o_ns, &J->epi);
      }
    }
  }
  free(arow);
  return NULL;
}

static int run_matmul(const orc_view *a, const orc_view *b, const orc_view *out,
                      int acc_mode, int nthreads, int batched, const orc_epi *epi) {
  int st = orc_check_matmul(a, b, out, batched);
  if (st != ORC_OK) return st;
  mm_job J;
  memset(&J, 0, sizeof(J));
  if (epi) {
    if (epi->bias) {
      if (epi->bias->ndim != 1 || epi->bias->shape[0] != b->shape[b->ndim - 1]) return ORC_SHAPE_MISMATCH;
      if (epi->bias->dtype != a->dtype) return ORC_DTYPE_MISMATCH;
    }
    J.epi = *epi;
  }
  J.a = a; J.b = b; J.out = out; J.acc_mode = acc_mode;
  J.m = a->shape[a->ndim - 2];
  J.k = a->shape[a->ndim - 1];
  J.n = b->shape[b->ndim - 1];
  J.bnd = out->ndim - 2;
  J.nbatch = 1;
  for (int d = 0; d < J.bnd; ++d) {
    J.bdims[d] = out->shape[d];
    J.nbatch *= out->shape[d];
    int ad = d - (J.bnd - (a->ndim - 2));
    int bd = d - (J.bnd - (b->ndim - 2));
    J.a_bs[d] = (ad >= 0 && a->shape[ad] != 1) ? a->strides[ad] : 0;
    J.b_bs[d] = (bd >= 0 && b->shape[bd] != 1) ? b->strides[bd] : 0;
    J.o_bs[d] = out->strides[d];
  }
  if (J.nbatch * J.m * J.n == 0) return ORC_OK;
  pthread_mutex_init(&J.mu, NULL);
  if (nthreads < 1) nthreads = 1;
  if (nthreads > 256) nthreads = 256;
  if ((int64_t)nthreads > J.nbatch * J.m) nthreads = (int)(J.nbatch * J.m);
  if (nthreads == 1) {
    mm_worker(&J);
  } else {
    pthread_t th[256];
    for (int t = 0; t < nthreads; ++t) pthread_create(&th[t], NULL, mm_worker, &J);
    for (int t = 0; t < nthreads; ++t) pthread_join(th[t], NULL);
  }
  pthread_mutex_destroy(&J.mu);
  return ORC_OK;
}

/* The block-scaled fp8 product (OCP Microscaling Formats specification v1.0,
 * MXFP8: 32 elements share one E8M0 scale 2^(e - 127), e = 255 is NaN).  The
 * reference has no quantised product (its DType stops at U8 / Bool,
 * crates/oxmera-core/src/dtype.rs:9-22), so this restates the published
 * definition: per output element, in double,
 *   sum over blocks kb of  sa[i, kb] * sb[kb, j] * (sum over the block's 32 k of a[i, k] * b[k, j]).
 * Scales are U8 views shaped like their operand with the contraction dim / 32;
 * batch dims broadcast as in orc_batched_matmul.  out is F32 or F64. */
static double e8m0(uint8_t e) { return e == 255 ? (double)bits_f32(0x7fc00000u) : ldexp(1.0, (int)e - 127); }

int orc_matmul_mx(const orc_view *a, const orc_view *a_scale, const orc_view *b, const orc_view *b_scale, const orc_view *out) {
  int st = orc_check_matmul(a, b, out, 1);
  if (st != ORC_OK) return st;
  if (a->dtype != ORC_F8E4M3 && a->dtype != ORC_F8E5M2) return ORC_UNSUPPORTED_DTYPE;
  if (out->dtype != ORC_F32 && out->dtype != ORC_F64) return ORC_UNSUPPORTED_DTYPE;
  const int an = a->ndim, bn = b->ndim, on = out->ndim;
  const int64_t m = a->shape[an - 2], k = a->shape[an - 1], n = b->shape[bn - 1];
  if (k % 32) return ORC_SHAPE_MISMATCH;
  if (a_scale->dtype != 4 || b_scale->dtype != 4) return ORC_DTYPE_MISMATCH; /* U8 */
  if (a_scale->ndim != an || b_scale->ndim != bn) return ORC_SHAPE_MISMATCH;
  for (int i = 0; i < an; ++i)
    if (a_scale->shape[i] != (i == an - 1 ? k / 32 : a->shape[i])) return ORC_SHAPE_MISMATCH;
  for (int i = 0; i < bn; ++i)
    if (b_scale->shape[i] != (i == bn - 2 ? k / 32 : b->shape[i])) return ORC_SHAPE_MISMATCH;
  const int bnd = on - 2;
  int64_t nbatch = 1;
  for (int d = 0; d < bnd; ++d) nbatch *= out->shape[d];
  for (int64_t bi = 0; bi < nbatch; ++bi) {
    int64_t a_off = a->offset, b_off = b->offset, o_off = out->offset, sa_off = a_scale->offset, sb_off = b_scale->offset;
    int64_t rem = bi;
    for (int d = bnd - 1; d >= 0; --d) {
      const int64_t idx = rem % out->shape[d];
      rem /= out->shape[d];
      const int ad = d - (bnd - (an - 2)), bd = d - (bnd - (bn - 2));
      if (ad >= 0 && a->shape[ad] != 1) { a_off += idx * a->strides[ad]; sa_off += idx * a_scale->strides[ad]; }
      if (bd >= 0 && b->shape[bd] != 1) { b_off += idx * b->strides[bd]; sb_off += idx * b_scale->strides[bd]; }
      o_off += idx * out->strides[d];
    }
    for (int64_t i = 0; i < m; ++i)
      for (int64_t j = 0; j < n; ++j) {
        double acc = 0.0;
        for (int64_t kb = 0; kb < k / 32; ++kb) {
          double blk = 0.0;
          for (int64_t kk = kb * 32; kk < kb * 32 + 32; ++kk)
            blk += (double)orc_fp8_to_f32(((const uint8_t *)a->base)[a_off + i * a->strides[an - 2] + kk * a->strides[an - 1]], a->dtype) *
                   (double)orc_fp8_to_f32(((const uint8_t *)b->base)[b_off + kk * b->strides[bn - 2] + j * b->strides[bn - 1]], b->dtype);
          const double sa = e8m0(((const uint8_t *)a_scale->base)[sa_off + i * a_scale->strides[an - 2] + kb * a_scale->strides[an - 1]]);
          const double sb = e8m0(((const uint8_t *)b_scale->base)[sb_off + kb * b_scale->strides[bn - 2] + j * b_scale->strides[bn - 1]]);
          acc += sa * sb * blk;
        }
        store_from_f64(out->base, out->dtype, o_off + i * out->strides[on - 2] + j * out->strides[on - 1], acc);
      }
  }
  return ORC_OK;
}

int orc_matmul(const orc_view *a, const orc_view *b, const orc_view *out, int acc_mode, int nthreads) {
  return run_matmul(a, b, out, acc_mode, nthreads, 0, NULL);
}

int orc_batched_matmul(const orc_view *a, const orc_view *b, const orc_view *out, int acc_mode, int nthreads) {
  return run_matmul(a, b, out, acc_mode, nthreads, 1, NULL);
}

int orc_matmul_fused(const orc_view *a, const orc_view *b, const orc_view *out, const orc_view *bias, int act,
                     int accumulate, int acc_mode, int nthreads) {
  orc_epi e;
  e.bias = bias;
  e.act = act;
  e.accumulate = accumulate;
  return run_matmul(a, b, out, acc_mode, nthreads, 1, &e);
}

/* ------------------------------------------------------------------ */
/* elementwise and reductions                                           */
/* ------------------------------------------------------------------ */

static int is_int_dtype(int32_t d) { return d == ORC_I32 || d == ORC_I64; }
static int is_float_dtype(int32_t d) { return d == ORC_F32 || d == ORC_F64 || d == ORC_BF16 || d == ORC_F16; }

static double get_f(const orc_view *v, int64_t idx) { return load_as_f64(v->base, v->dtype, idx); }
static int64_t get_i(const orc_view *v, int64_t idx) {
  return v->dtype == ORC_I32 ? (int64_t)((const int32_t *)v->base)[idx] : ((const int64_t *)v->base)[idx];
}
static void put_f(const orc_view *v, int64_t idx, double x) { store_from_f64(v->base, v->dtype, idx, x); }
static void put_i(const orc_view *v, int64_t idx, int64_t x) {
  if (v->dtype == ORC_I32) ((int32_t *)v->base)[idx] = (int32_t)x;
  else ((int64_t *)v->base)[idx] = x;
}

/* storage offset of the i-th element (row-major over `shape`) of an operand
 * right-aligned against that shape, extent-1 dims broadcasting */
static int64_t bcast_offset(const orc_view *v, const int64_t *shape, int ndim, int64_t i) {
  int64_t off = v->offset;
  for (int d = ndim - 1; d >= 0; --d) {
    int64_t idx = i % shape[d];
    i /= shape[d];
    int vd = d - (ndim - v->ndim);
    if (vd >= 0 && v->shape[vd] != 1) off += idx * v->strides[vd];
  }
  return off;
}

int orc_unary(int op, const orc_view *a, const orc_view *out) {
  if (!(is_float_dtype(a->dtype) || is_int_dtype(a->dtype))) return ORC_UNSUPPORTED_DTYPE;
  if ((op == 1 || op == 2) && !is_float_dtype(a->dtype)) return ORC_UNSUPPORTED_DTYPE;
  if (out->dtype != a->dtype) return ORC_DTYPE_MISMATCH;
  int64_t n = 1;
  for (int d = 0; d < a->ndim; ++d) n *= a->shape[d];
  for (int64_t i = 0; i < n; ++i) {
    int64_t off = bcast_offset(a, a->shape, a->ndim, i);
    if (is_int_dtype(a->dtype)) {
      int64_t x = get_i(a, off);
      put_i(out, out->offset + i, op == 0 ? -x : (x < 0 ? -x : x));
    } else {
      double x = get_f(a, off);
      put_f(out, out->offset + i, op == 0 ? -x : op == 1 ? exp(x) : op == 2 ? log(x) : fabs(x));
    }
  }
  return ORC_OK;
}

int orc_binary(int op, const orc_view *a, const orc_view *b, const orc_view *out) {
  if (a->dtype != b->dtype) return ORC_DTYPE_MISMATCH;
  if (!(is_float_dtype(a->dtype) || is_int_dtype(a->dtype))) return ORC_UNSUPPORTED_DTYPE;
  int64_t shape[ORC_MAX_DIMS];
  int nd = 0;
  int st = orc_broadcast_shapes(a->shape, a->ndim, b->shape, b->ndim, shape, &nd);
  if (st != ORC_OK) return st;
  if (out->ndim != nd) return ORC_SHAPE_MISMATCH;
  int64_t n = 1;
  for (int d = 0; d < nd; ++d) {
    if (out->shape[d] != shape[d]) return ORC_SHAPE_MISMATCH;
    n *= shape[d];
  }
  int zero_divisor = 0;
  for (int64_t i = 0; i < n; ++i) {
    int64_t ao = bcast_offset(a, shape, nd, i), bo = bcast_offset(b, shape, nd, i);
    if (is_int_dtype(a->dtype)) {
      int64_t x = get_i(a, ao), y = get_i(b, bo), r;
      if (op == 3) {
        /* crates/oxmera-ops/src/lib.rs:47-49: "Integer division by zero is a typed error".
         * Truncating division; the most negative value over -1 wraps to itself. */
        if (y == 0) { zero_divisor = 1; r = 0; }
        else if (y == -1) r = (int64_t)(0ull - (uint64_t)x);
        else r = x / y;
      } else {
        r = op == 0 ? x + y : op == 1 ? x - y : x * y;
      }
      put_i(out, out->offset + i, r);
    } else {
      double x = get_f(a, ao), y = get_f(b, bo);
      put_f(out, out->offset + i, op == 0 ? x + y : op == 1 ? x - y : op == 2 ? x * y : x / y);
    }
  }
  return zero_divisor ? ORC_DIVIDE_BY_ZERO : ORC_OK;
}

int orc_reduce(int op, const orc_view *a, const int32_t *axes, int naxes, const orc_view *out) {
  if (!(is_float_dtype(a->dtype) || is_int_dtype(a->dtype))) return ORC_UNSUPPORTED_DTYPE;
  int reduced[ORC_MAX_DIMS] = {0};
  if (naxes == 0) for (int d = 0; d < a->ndim; ++d) reduced[d] = 1;
  for (int i = 0; i < naxes; ++i) {
    if (axes[i] < 0 || axes[i] >= a->ndim || reduced[axes[i]]) return ORC_INDEX_OUT_OF_BOUNDS;
    reduced[axes[i]] = 1;
  }
  int64_t kshape[ORC_MAX_DIMS], kstr[ORC_MAX_DIMS], rshape[ORC_MAX_DIMS], rstr[ORC_MAX_DIMS];
  int nk = 0, nr = 0;
  int64_t n_out = 1, n_red = 1;
  for (int d = 0; d < a->ndim; ++d) {
    if (reduced[d]) { rshape[nr] = a->shape[d]; rstr[nr] = a->strides[d]; nr++; n_red *= a->shape[d]; }
    else { kshape[nk] = a->shape[d]; kstr[nk] = a->strides[d]; nk++; n_out *= a->shape[d]; }
  }
  if (out->ndim != nk) return ORC_SHAPE_MISMATCH;
  for (int d = 0; d < nk; ++d) if (out->shape[d] != kshape[d]) return ORC_SHAPE_MISMATCH;
  if (n_out > 0 && n_red == 0 && op == 1) return ORC_NOT_IMPLEMENTED; /* no identity to invent */
  for (int64_t o = 0; o < n_out; ++o) {
    int64_t base = a->offset, t = o;
    for (int d = nk - 1; d >= 0; --d) { base += (t % kshape[d]) * kstr[d]; t /= kshape[d]; }
    double facc = 0.0;
    int64_t iacc = 0;
    for (int64_t r = 0; r < n_red; ++r) {
      int64_t off = base, u = r;
      for (int d = nr - 1; d >= 0; --d) { off += (u % rshape[d]) * rstr[d]; u /= rshape[d]; }
      if (is_int_dtype(a->dtype)) {
        int64_t x = get_i(a, off);
        iacc = (r == 0) ? x : (op == 0 ? iacc + x : (x > iacc ? x : iacc));
      } else {
        double x = get_f(a, off);
        /* max propagates NaN (a NaN anywhere in the slice makes the result NaN) */
        facc = (r == 0) ? x : (op == 0 ? facc + x : (facc != facc ? facc : (x != x ? x : (x > facc ? x : facc))));
      }
    }
    if (is_int_dtype(a->dtype)) put_i(out, out->offset + o, iacc);
    else put_f(out, out->offset + o, facc);
  }
  return ORC_OK;
}

/* ------------------------------------------------------------------ */
/* synthetic data                                                       */
/* ------------------------------------------------------------------ */

static inline uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

typedef struct {
  void *dst;
  int32_t dtype;
  int64_t lo, hi;
  uint64_t key;
  int dist;
  double scale;
} fill_job;

static void *fill_worker(void *arg) {
  fill_job *F = (fill_job *)arg;
  const double two_pi = 6.283185307179586476925286766559;
  for (int64_t i = F->lo; i < F->hi; ++i) {
    uint64_t h1 = splitmix64(F->key + 2ull * (uint64_t)i);
    double v;
    if (F->dist == 0) {
      v = 2.0 * ((double)(h1 >> 11) * (1.0 / 9007199254740992.0)) - 1.0;
    } else {
      uint64_t h2 = splitmix64(F->key + 2ull * (uint64_t)i + 1ull);
      double u1 = ((double)(h1 >> 11) + 1.0) * (1.0 / 9007199254740992.0);
      double u2 = (double)(h2 >> 11) * (1.0 / 9007199254740992.0);
      v = sqrt(-2.0 * log(u1)) * cos(two_pi * u2) * F->scale;
    }
    float f = (float)v;
    if (F->dtype == ORC_F64) { ((double *)F->dst)[i] = v; continue; }
    if (F->dtype == ORC_F32) ((float *)F->dst)[i] = f;
    else if (F->dtype == ORC_BF16) ((uint16_t *)F->dst)[i] = orc_f32_to_bf16(f);
    else if (F->dtype == ORC_F16) ((uint16_t *)F->dst)[i] = orc_f32_to_f16(f);
    else ((uint8_t *)F->dst)[i] = orc_f32_to_fp8(f, F->dtype);
  }
  return NULL;
}

int orc_fill(void *dst, int32_t dtype, int64_t n, uint64_t seed, uint64_t stream,
             int dist, double scale, int nthreads) {
  if (!(dtype == ORC_F32 || dtype == ORC_F64 || dtype == ORC_BF16 || dtype == ORC_F16 || dtype == ORC_F8E4M3 ||
        dtype == ORC_F8E5M2))
    return ORC_UNSUPPORTED_DTYPE; /* writing one byte per element into a wider buffer would leave it uninitialised */
  uint64_t key = splitmix64(splitmix64(seed) ^ splitmix64(stream * 0xD1342543DE82EF95ull + 0x632BE59BD9B4E019ull));
  if (nthreads < 1) nthreads = 1;
  if (nthreads > 256) nthreads = 256;
  if (n < 65536) nthreads = 1;
  fill_job jobs[256];
  pthread_t th[256];
  int64_t per = (n + nthreads - 1) / nthreads;
  for (int t = 0; t < nthreads; ++t) {
    jobs[t].dst = dst; jobs[t].dtype = dtype; jobs[t].key = key;
    jobs[t].dist = dist; jobs[t].scale = scale;
    jobs[t].lo = t * per < n ? t * per : n;
    jobs[t].hi = (t + 1) * per < n ? (t + 1) * per : n;
  }
  if (nthreads == 1) { fill_worker(&jobs[0]); return ORC_OK; }
  for (int t = 0; t < nthreads; ++t) pthread_create(&th[t], NULL, fill_worker, &jobs[t]);
  for (int t = 0; t < nthreads; ++t) pthread_join(th[t], NULL);
  return ORC_OK;
}
