// C ABI of the oxmera B200 backend (declared in include/oxmera_b200.h):
// argument validation with oxmera's typed errors, view normalisation, kernel
// selection and launch.  No CPU compute path exists here: an operation either
// runs on the GPU or returns an error.
#include "../../include/oxmera_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "elementwise.cuh"
#include "gemm_instances.cuh"
#include "kernels_simt.cuh"

namespace {

using namespace oxm;

thread_local std::string g_last_error;

int fail(int status, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return status;
}

#define CUDA_TRY(expr)                                                                   \
  do {                                                                                   \
    cudaError_t e__ = (expr);                                                            \
    if (e__ != cudaSuccess)                                                              \
      return fail(OXM_CUDA_ERROR, "%s failed: %s", #expr, cudaGetErrorString(e__));      \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

constexpr size_t kSkFlagWords = 256 * 8;  // up to 256 SMs, 8 epilogue warps each

struct Workspace {
  void *ptr = nullptr;
  size_t bytes = 0;
};

}  // namespace

struct oxm_ctx {
  int device = 0;
  int num_sms = 0;
  cudaStream_t stream = nullptr;
  uint32_t *status_dev = nullptr;   // device status word written by kernels
  uint32_t *status_host = nullptr;  // pinned mirror
  uint32_t *sk_flags = nullptr;     // stream-K publication counters, one per (run, CTA of the pair, epilogue warp)
  uint32_t sk_epoch = 0;            // launch counter the flags are compared against
  EncodeTiledFn encode = nullptr;
  std::mutex mu;
  std::mutex host_mu;  // serialises calls that use the host staging buffers
  Workspace pack_ws[5];  // packed A, packed B, split-K partial sums, scale atoms of A and of B (block-scaled products)
  Workspace host_stage[3];
  cudaStream_t copy_in = nullptr, copy_out = nullptr;  // host entry point: copies overlapped with compute
  cudaEvent_t pipe_events[2 * 16 + 1] = {};
  // options
  int64_t opt_kernel = 0, opt_tile_n = 0, opt_cta_pair = -1, opt_wait_limit_ms = 2000, opt_group_m = 0, opt_tma_store = 1, opt_split_k = -1, opt_host_chunks = 0, opt_stream_k = -1, opt_simt_tile = 0;
  int64_t launches[4] = {0, 0, 0, 0};
  char last_kernel[96] = "none";
};

struct oxm_event {
  cudaEvent_t ev = nullptr;
  int device = 0;
};

namespace {

int dtype_size(int dt) {
  switch (dt) {
    case OXM_F32: case OXM_I32: return 4;
    case OXM_F64: case OXM_I64: return 8;
    case OXM_U8: case OXM_BOOL: return 1;
    case OXM_BF16: case OXM_F16: return 2;
    case OXM_F8E4M3: case OXM_F8E5M2: return 1;
    default: return 0;
  }
}

const char *dtype_name(int dt) {
  static const char *names[] = {"F32", "F64", "I32", "I64", "U8", "Bool", "BF16", "F16", "F8E4M3", "F8E5M2"};
  return (dt >= 0 && dt < 10) ? names[dt] : "?";
}

std::string shape_str(const oxm_view *v) {
  std::string s = "[";
  for (int i = 0; i < v->ndim; ++i) {
    if (i) s += ", ";
    s += std::to_string(v->shape[i]);
  }
  return s + "]";
}

bool is_fp8(int dt) { return dt == OXM_F8E4M3 || dt == OXM_F8E5M2; }
bool is_matmul_dtype(int dt) { return dt == OXM_F32 || dt == OXM_BF16 || dt == OXM_F16 || is_fp8(dt); }

// The checks of MatmulOps::matmul, in the order the reference's errors imply:
// rank, device, dtype, inner dimension, batch broadcast, output shape.
int validate(const oxm_ctx *ctx, const oxm_view *a, const oxm_view *b, const oxm_view *out, bool batched,
             bool host_views) {
  const char *op = batched ? "batched_matmul" : "matmul";
  if (!ctx || !a || !b || !out) return fail(OXM_INVALID_ARGUMENT, "%s: null argument", op);
  for (const oxm_view *v : {a, b, out}) {
    if (v->ndim < 0 || v->ndim > OXM_MAX_DIMS) return fail(OXM_NOT_IMPLEMENTED, "%s is not implemented for rank %d", op, v->ndim);
    for (int i = 0; i < v->ndim; ++i)
      if (v->shape[i] < 0) return fail(OXM_INVALID_ARGUMENT, "%s: negative extent in %s", op, shape_str(v).c_str());
  }
  if (!batched) {
    if (a->ndim != 2 || b->ndim != 2)
      return fail(OXM_SHAPE_MISMATCH, "shape mismatch: expected rank-2 operands, got %s and %s in %s",
                  shape_str(a).c_str(), shape_str(b).c_str(), op);
  } else if (a->ndim < 2 || b->ndim < 2) {
    return fail(OXM_SHAPE_MISMATCH, "shape mismatch: expected operands of rank >= 2, got %s and %s in %s",
                shape_str(a).c_str(), shape_str(b).c_str(), op);
  }
  if (!host_views) {
    if (a->device != b->device)
      return fail(OXM_DEVICE_MISMATCH, "device mismatch: Cuda{index: %d} vs Cuda{index: %d} in %s", a->device, b->device, op);
    if (a->device != ctx->device || out->device != ctx->device)
      return fail(OXM_DEVICE_MISMATCH, "device mismatch: operands on Cuda{index: %d}, output on Cuda{index: %d}, backend serves Cuda{index: %d} in %s",
                  a->device, out->device, ctx->device, op);
  }
  if (a->dtype != b->dtype)
    return fail(OXM_DTYPE_MISMATCH, "dtype mismatch: expected %s, got %s in %s", dtype_name(a->dtype), dtype_name(b->dtype), op);
  if (!is_matmul_dtype(a->dtype))
    return fail(OXM_UNSUPPORTED_DTYPE, "dtype %s is not supported by %s", dtype_name(a->dtype), op);
  // fp8 products may be kept in a wider type; everything else keeps the operands' dtype
  const bool widened = is_fp8(a->dtype) && (out->dtype == OXM_BF16 || out->dtype == OXM_F16 || out->dtype == OXM_F32);
  if (out->dtype != a->dtype && !widened)
    return fail(OXM_DTYPE_MISMATCH, "dtype mismatch: expected %s, got %s in %s (output)", dtype_name(a->dtype), dtype_name(out->dtype), op);
  const int64_t m = a->shape[a->ndim - 2], k = a->shape[a->ndim - 1];
  const int64_t kb = b->shape[b->ndim - 2], n = b->shape[b->ndim - 1];
  if (k != kb)
    return fail(OXM_SHAPE_MISMATCH, "shape mismatch: expected [%lld, %lld], got %s in %s (inner dimensions of %s x %s)",
                (long long)k, (long long)n, shape_str(b).c_str(), op, shape_str(a).c_str(), shape_str(b).c_str());
  const int abn = a->ndim - 2, bbn = b->ndim - 2;
  const int nbd = std::max(abn, bbn);
  int64_t bd[OXM_MAX_DIMS];
  for (int i = 0; i < nbd; ++i) {
    const int ai = abn - 1 - i, bi = bbn - 1 - i;
    const int64_t l = ai >= 0 ? a->shape[ai] : 1, r = bi >= 0 ? b->shape[bi] : 1;
    if (l != r && l != 1 && r != 1)
      return fail(OXM_BROADCAST_INCOMPATIBLE, "cannot broadcast %s with %s", shape_str(a).c_str(), shape_str(b).c_str());
    bd[nbd - 1 - i] = (l == 1) ? r : l;
  }
  bool out_ok = out->ndim == nbd + 2;
  for (int i = 0; out_ok && i < nbd; ++i) out_ok = out->shape[i] == bd[i];
  if (out_ok) out_ok = out->shape[nbd] == m && out->shape[nbd + 1] == n;
  if (!out_ok) {
    std::string exp = "[";
    for (int i = 0; i < nbd; ++i) exp += std::to_string(bd[i]) + ", ";
    exp += std::to_string(m) + ", " + std::to_string(n) + "]";
    return fail(OXM_SHAPE_MISMATCH, "shape mismatch: expected %s, got %s in %s (output)", exp.c_str(), shape_str(out).c_str(), op);
  }
  return OXM_OK;
}

// A matmul problem with coalesced batch dims.  B is held as rows = N, so both
// operands are "rows x K" matrices.
struct Problem {
  int dtype, elt;          // operands
  int out_dtype, oelt;     // output (differs from the operands' only for fp8 products)
  int64_t M, N, K;
  int nbd;
  int64_t bdims[OXM_MAX_DIMS];
  const void *a, *b;
  void *o;
  int64_t a_off, b_off, o_off;
  int64_t a_rs, a_ks, b_rs, b_ks, o_rs, o_cs;
  int64_t a_bs[OXM_MAX_DIMS], b_bs[OXM_MAX_DIMS], o_bs[OXM_MAX_DIMS];
  int64_t nbatch;
  Epilogue epi;
};

// `merge` = false keeps every batch dim of extent > 1 as it is (the block-scaled product walks
// its scale views by the same dims).
Problem normalise(const oxm_view *a, const oxm_view *b, const oxm_view *out, bool merge = true) {
  Problem P{};
  P.dtype = a->dtype;
  P.elt = dtype_size(a->dtype);
  P.out_dtype = out->dtype;
  P.oelt = dtype_size(out->dtype);
  P.M = a->shape[a->ndim - 2];
  P.K = a->shape[a->ndim - 1];
  P.N = b->shape[b->ndim - 1];
  P.a = a->base; P.b = b->base; P.o = out->base;
  P.a_off = a->offset; P.b_off = b->offset; P.o_off = out->offset;
  P.a_rs = a->strides[a->ndim - 2]; P.a_ks = a->strides[a->ndim - 1];
  P.b_ks = b->strides[b->ndim - 2]; P.b_rs = b->strides[b->ndim - 1];
  P.o_rs = out->strides[out->ndim - 2]; P.o_cs = out->strides[out->ndim - 1];
  const int nbd = out->ndim - 2;
  // Gather batch dims (dropping extent-1 dims), broadcast strides as 0.
  int n = 0;
  int64_t dims[OXM_MAX_DIMS], as[OXM_MAX_DIMS], bs[OXM_MAX_DIMS], os[OXM_MAX_DIMS];
  for (int d = 0; d < nbd; ++d) {
    if (out->shape[d] == 1) continue;
    const int ad = d - (nbd - (a->ndim - 2)), bd = d - (nbd - (b->ndim - 2));
    dims[n] = out->shape[d];
    as[n] = (ad >= 0 && a->shape[ad] != 1) ? a->strides[ad] : 0;
    bs[n] = (bd >= 0 && b->shape[bd] != 1) ? b->strides[bd] : 0;
    os[n] = out->strides[d];
    ++n;
  }
  // Merge neighbours that every tensor walks with one stride.
  int w = 0;
  for (int d = 0; d < n; ++d) {
    if (merge && w > 0 && as[w - 1] == as[d] * dims[d] && bs[w - 1] == bs[d] * dims[d] && os[w - 1] == os[d] * dims[d]) {
      dims[w - 1] *= dims[d];
      as[w - 1] = as[d]; bs[w - 1] = bs[d]; os[w - 1] = os[d];
    } else {
      dims[w] = dims[d]; as[w] = as[d]; bs[w] = bs[d]; os[w] = os[d];
      ++w;
    }
  }
  // A single batch dim over a shared B folds into M: one tall GEMM.
  if (merge && w == 1 && bs[0] == 0 && as[0] == P.M * P.a_rs && os[0] == P.M * P.o_rs && P.M > 0) {
    P.M *= dims[0];
    w = 0;
  }
  P.nbd = w;
  P.nbatch = 1;
  for (int d = 0; d < w; ++d) {
    P.bdims[d] = dims[d]; P.a_bs[d] = as[d]; P.b_bs[d] = bs[d]; P.o_bs[d] = os[d];
    P.nbatch *= dims[d];
  }
  return P;
}

// ---------------------------------------------------------------------------
// SIMT path
// ---------------------------------------------------------------------------
int launch_simt(oxm_ctx *ctx, const Problem &P) {
  if (P.nbd > kSimtMaxBatchDims) return fail(OXM_NOT_IMPLEMENTED, "matmul is not implemented for %d batch dims", P.nbd);
  if (P.M > INT32_MAX || P.N > INT32_MAX || P.K > INT32_MAX) return fail(OXM_NOT_IMPLEMENTED, "matmul is not implemented for extents above 2^31");
  SimtParams p{};
  p.a = P.a; p.b = P.b; p.out = P.o;
  p.dtype = P.dtype; p.out_dtype = P.out_dtype;
  p.M = (int32_t)P.M; p.N = (int32_t)P.N; p.K = (int32_t)P.K;
  // 64-wide tiles wherever they can occupy half of the SMs, alone or with the contraction of
  // each tile split over a cluster of up to 8 CTAs; 32-wide tiles for outputs smaller than that.
  const int64_t tiles64 = ((P.M + 63) / 64) * ((P.N + 63) / 64) * P.nbatch;
  int ts = tiles64 * 8 >= ctx->num_sms / 2 ? 64 : 32;
  if (ctx->opt_simt_tile == 32 || ctx->opt_simt_tile == 64) ts = (int)ctx->opt_simt_tile;
  p.tiles_m = (int32_t)((P.M + ts - 1) / ts); p.tiles_n = (int32_t)((P.N + ts - 1) / ts);
  p.a_off = P.a_off; p.b_off = P.b_off; p.o_off = P.o_off;
  p.a_rs = P.a_rs; p.a_cs = P.a_ks; p.b_rs = P.b_ks; p.b_cs = P.b_rs; p.o_rs = P.o_rs; p.o_cs = P.o_cs;
  p.nbd = P.nbd;
  for (int d = 0; d < P.nbd; ++d) {
    p.bdims[d] = (int32_t)P.bdims[d]; p.a_bs[d] = P.a_bs[d]; p.b_bs[d] = P.b_bs[d]; p.o_bs[d] = P.o_bs[d];
  }
  p.epi = P.epi;
  const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n * P.nbatch;
  // Too few tiles for the SMs and a contraction worth cutting: a cluster of 2, 4 or 8 CTAs per
  // tile - as many as still fit the GPU in one wave (two CTAs per SM) with at least one staged
  // block of k each (2048 / ts elements).  Measured on a 256 x 512 x 384 f32 product: 64-wide
  // tiles in clusters of 8 take 14.4 us, clusters of 4 18.5, 32-wide tiles 16.4 at best.
  int ksplit = 1;
  if (ctx->opt_split_k != 0)
    while (ksplit < 8 && tiles * ksplit * 2 <= 2 * (int64_t)ctx->num_sms && P.K / (ksplit * 2) >= 2048 / ts) ksplit *= 2;
  if (ctx->opt_split_k == 2 || ctx->opt_split_k == 4 || ctx->opt_split_k == 8)  // forced: a cluster of that many CTAs per tile
    ksplit = (int)std::min<int64_t>(ctx->opt_split_k, std::max<int64_t>(1, P.K / 16));
  p.ksplit = ksplit;
  p.kchunk = (int32_t)(((P.K + ksplit - 1) / ksplit + 15) / 16 * 16);
  const int64_t blocks = tiles * ksplit;
  if (blocks > INT32_MAX) return fail(OXM_NOT_IMPLEMENTED, "matmul is not implemented for %lld output tiles", (long long)blocks);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)blocks, 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  if (ksplit > 1) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)ksplit; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
  }
  if (ts == 64) CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_simt_kernel<64>, p));
  else CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_simt_kernel<32>, p));
  ctx->launches[0]++; ctx->launches[2]++;
  snprintf(ctx->last_kernel, sizeof(ctx->last_kernel), "gemm_simt_ffma_%dx%d%s", ts, ts, ksplit > 1 ? "_ksplit" : "");
  return OXM_OK;
}

// ---------------------------------------------------------------------------
// tensor-core path
// ---------------------------------------------------------------------------

// One operand as the TMA engine will see it.
struct Staged {
  const void *ptr;     // address of element (0,0) of batch 0
  bool mn_major;
  int64_t rows, K;     // K in staged elements
  int64_t ld_bytes;    // stride of the non-contiguous matrix dim
  int64_t nb;          // collapsed batch count
  int64_t bs_bytes;    // batch stride
  int32_t bmul[kMaxBatchDims];
};

int grow(oxm_ctx *ctx, Workspace &w, size_t bytes) {
  if (w.bytes >= bytes) return OXM_OK;
  if (w.ptr) CUDA_TRY(cudaFreeAsync(w.ptr, ctx->stream));
  w.ptr = nullptr; w.bytes = 0;
  size_t want = std::max(bytes, (size_t)1 << 20);
  CUDA_TRY(cudaMallocAsync(&w.ptr, want, ctx->stream));
  w.bytes = want;
  return OXM_OK;
}

// Can the TMA engine address this operand in place?  Fills `s` when it can.
bool stage_direct(const Problem &P, bool is_b, Staged &s) {
  if (P.elt != 2 && P.elt != 1) return false;  // f32 is always packed (TF32 split)
  const void *base = is_b ? P.b : P.a;
  const int64_t off = is_b ? P.b_off : P.a_off;
  const int64_t rows = is_b ? P.N : P.M, K = P.K;
  const int64_t rs = is_b ? P.b_rs : P.a_rs, ks = is_b ? P.b_ks : P.a_ks;
  const int64_t *bs = is_b ? P.b_bs : P.a_bs;
  const uintptr_t addr = reinterpret_cast<uintptr_t>(base) + off * P.elt;
  if (addr % 16) return false;
  auto ld_ok = [&](int64_t ld, int64_t extent) { return extent == 1 || (ld > 0 && (ld * P.elt) % 16 == 0 && ld * P.elt < (1ll << 40)); };
  bool k_major = (ks == 1 || K == 1) && ld_ok(rs, rows);
  bool mn_major = !k_major && (rs == 1 || rows == 1) && ld_ok(ks, K);
  if (!k_major && !mn_major) return false;
  if (rows >= (1ll << 31) || K >= (1ll << 31)) return false;
  s.ptr = reinterpret_cast<const void *>(addr);
  s.mn_major = mn_major;
  s.rows = rows; s.K = K;
  const int64_t inner = k_major ? K : rows;
  const int64_t outer = k_major ? rows : K;
  int64_t ld = k_major ? rs : ks;
  if (outer == 1) ld = (inner * P.elt + 15) / 16 * 16 / P.elt;  // any legal value: never stepped
  s.ld_bytes = ld * P.elt;
  // Own (non-broadcast) batch dims must fold into one strided dim.
  s.nb = 1; s.bs_bytes = 0;
  int64_t inner_stride = 0;
  bool have = false;
  for (int d = P.nbd - 1; d >= 0; --d) {
    if (bs[d] == 0) { s.bmul[d] = 0; continue; }
    if (!have) { inner_stride = bs[d]; have = true; }
    else if (bs[d] != inner_stride * s.nb) return false;
    if (s.nb > INT32_MAX) return false;
    s.bmul[d] = (int32_t)s.nb;
    s.nb *= P.bdims[d];
  }
  if (have) {
    if (inner_stride <= 0 || (inner_stride * P.elt) % 16 || inner_stride * P.elt >= (1ll << 40)) return false;
    s.bs_bytes = inner_stride * P.elt;
  } else {
    s.bs_bytes = std::max<int64_t>(16, (s.ld_bytes * outer + 15) / 16 * 16);
  }
  if (s.nb >= (1ll << 31)) return false;
  return true;
}

// Pack an operand into K-major rows in workspace `slot`.  f32 becomes the
// three-term TF32 layout (see pack_kernel).
int stage_packed(oxm_ctx *ctx, const Problem &P, bool is_b, int slot, Staged &s) {
  const int64_t rows = is_b ? P.N : P.M;
  const int64_t rs = is_b ? P.b_rs : P.a_rs, ks = is_b ? P.b_ks : P.a_ks;
  const int64_t *bs = is_b ? P.b_bs : P.a_bs;
  const bool split = P.elt == 4;
  const int64_t Kp = split ? (P.K + 31) / 32 * 32 : (P.K + 15) / 16 * 16;  // rows stay 16-byte multiples
  const int64_t row_elems = split ? 3 * Kp : Kp;
  PackParams pp{};
  pp.src = is_b ? P.b : P.a;
  pp.elt = P.elt;
  pp.mode = split ? (is_b ? 2 : 1) : 0;
  pp.rows = (int32_t)rows; pp.K = (int32_t)P.K; pp.Kp = (int32_t)Kp;
  pp.dst_row_elems = row_elems;
  pp.src_off = is_b ? P.b_off : P.a_off;
  pp.src_rs = rs; pp.src_ks = ks;
  // Only the operand's own batch dims are materialised; broadcast dims stay virtual.
  int64_t nb = 1;
  pp.nbd = 0;
  for (int d = 0; d < P.nbd; ++d) s.bmul[d] = 0;
  for (int d = P.nbd - 1; d >= 0; --d) {
    if (bs[d] == 0) continue;
    s.bmul[d] = (int32_t)nb;
    nb *= P.bdims[d];
  }
  for (int d = 0; d < P.nbd; ++d) {
    if (bs[d] == 0) continue;
    pp.bdims[pp.nbd] = (int32_t)P.bdims[d];
    pp.src_bs[pp.nbd] = bs[d];
    pp.nbd++;
  }
  if (rows >= (1ll << 31) || Kp >= (1ll << 30) || nb >= (1ll << 31)) return fail(OXM_NOT_IMPLEMENTED, "matmul is not implemented for extents above 2^31");
  const size_t bytes = (size_t)nb * rows * row_elems * P.elt;
  int st = grow(ctx, ctx->pack_ws[slot], bytes);
  if (st) return st;
  pp.dst = ctx->pack_ws[slot].ptr;
  pp.tiles_r = (int32_t)((rows + 31) / 32);
  pp.tiles_k = (int32_t)((Kp + 31) / 32);
  const int64_t blocks = (int64_t)pp.tiles_r * pp.tiles_k * nb;
  if (blocks > INT32_MAX) return fail(OXM_NOT_IMPLEMENTED, "matmul is not implemented for %lld pack tiles", (long long)blocks);
  pack_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(pp);
  CUDA_TRY(cudaGetLastError());
  ctx->launches[0]++; ctx->launches[3]++;
  s.ptr = pp.dst;
  s.mn_major = false;
  s.rows = rows; s.K = row_elems;
  s.ld_bytes = row_elems * P.elt;
  s.nb = nb;
  s.bs_bytes = rows * row_elems * P.elt;
  return OXM_OK;
}

int make_map(oxm_ctx *ctx, CUtensorMap *tm, const Staged &s, int dtype, int elt, int box_rows_kmajor, int box_k) {
  const CUtensorMapDataType dt = dtype == OXM_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == OXM_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : dtype == OXM_F16  ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const cuuint32_t inner_box = (cuuint32_t)(kStageKBytes / elt);
  cuuint64_t dims[3];
  cuuint32_t box[3];
  if (s.mn_major) {
    dims[0] = (cuuint64_t)s.rows; dims[1] = (cuuint64_t)s.K;
    box[0] = inner_box; box[1] = (cuuint32_t)box_k;
  } else {
    dims[0] = (cuuint64_t)s.K; dims[1] = (cuuint64_t)s.rows;
    box[0] = inner_box; box[1] = (cuuint32_t)box_rows_kmajor;
  }
  dims[2] = (cuuint64_t)s.nb;
  box[2] = 1;
  cuuint64_t strides[2] = {(cuuint64_t)s.ld_bytes, (cuuint64_t)s.bs_bytes};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = ctx->encode(tm, dt, 3, const_cast<void *>(s.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(OXM_CUDA_ERROR, "cuTensorMapEncodeTiled failed (%d): dims [%llu,%llu,%llu] strides [%llu,%llu] box [%u,%u,1] ptr %p",
                (int)r, (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
                (unsigned long long)strides[0], (unsigned long long)strides[1], box[0], box[1], s.ptr);
  return OXM_OK;
}

// Fill the kernel's batch-dim arrays.  The tiles enumerate batch entries with the last listed dim
// fastest; listed last is the dim along which the fewest operand bytes change from one entry to
// the next (a broadcast operand changes none), so tiles in flight at the same time share the
// larger operand in L2.  `o_bstride` = the output's element stride per dim (the caller's), and the
// store map's batch coordinate counts entries in the output's own (row-major) order.
void fill_batch_dims(GemmParams &p, const Problem &P, const Staged &sa, const Staged &sb, const int64_t *o_bstride) {
  int order[kMaxBatchDims];
  for (int d = 0; d < P.nbd; ++d) order[d] = d;
  const double a_entry = (double)sa.rows * (double)sa.K, b_entry = (double)sb.rows * (double)sb.K;
  auto changing = [&](int d) { return (sa.bmul[d] ? a_entry : 0.0) + (sb.bmul[d] ? b_entry : 0.0); };
  std::stable_sort(order, order + P.nbd, [&](int x, int y) { return changing(x) > changing(y); });
  int64_t row_major[kMaxBatchDims];
  int64_t run = 1;
  for (int d = P.nbd - 1; d >= 0; --d) { row_major[d] = run; run *= P.bdims[d]; }
  for (int i = 0; i < P.nbd; ++i) {
    const int d = order[i];
    p.bdims[i] = (int32_t)P.bdims[d];
    p.a_bmul[i] = sa.bmul[d];
    p.b_bmul[i] = sb.bmul[d];
    p.o_bmul[i] = (int32_t)row_major[d];
    p.o_bstride[i] = o_bstride[d];
  }
}

// Launch one instance of the tensor-core GEMM (defined in the gemm_*.cu units).
int launch_gemm(oxm_ctx *ctx, int kind, bool a_mn, bool b_mn, int bn, int pair, const CUtensorMap &tmA, const CUtensorMap &tmB,
                const CUtensorMap &tmC, const GemmParams &p, int grid, const CUtensorMap *sf = nullptr) {
  // whole tiles with a 16-bit result: the wide tile's register-packed epilogue
  const bool packed = bn == 512 && kind != 1 && p.sk_tiles == 0 && (p.out_dtype == OXM_BF16 || p.out_dtype == OXM_F16);
  const GemmLaunch l{bn, pair, packed, b_mn, grid, ctx->stream, sf};
  const GemmLaunchFn fn = kind == 1 ? launch_gemm_tf32
                          : kind == 3 ? launch_gemm_mx
                          : kind == 2 ? (a_mn ? (b_mn ? launch_gemm_f8_mn : launch_gemm_f8_mk) : (b_mn ? launch_gemm_f8_kn : launch_gemm_f8_kk))
                                      : (a_mn ? (b_mn ? launch_gemm_f16_mn : launch_gemm_f16_mk) : (b_mn ? launch_gemm_f16_kn : launch_gemm_f16_kk));
  cudaError_t e = fn(l, tmA, tmB, tmC, p, ctx->last_kernel, sizeof(ctx->last_kernel));
  if (e != cudaSuccess) {
    cudaGetLastError();  // a refused launch also parks its error for the next caller of cudaGetLastError: take it away
    return fail(OXM_CUDA_ERROR, "launch of %s failed: %s", ctx->last_kernel, cudaGetErrorString(e));
  }
  return OXM_OK;
}

// Store tensor map over the output: {N, M, batch} in boxes of 128 bytes x 32
// rows.  Returns false when the output cannot be described (the kernel then
// stores through plain strided writes).
bool make_out_map(oxm_ctx *ctx, CUtensorMap *tm, void *ptr, int dtype, int elt, int64_t M, int64_t N, int64_t nb,
                  int64_t rs_elems, int64_t bs_elems) {
  if (reinterpret_cast<uintptr_t>(ptr) % 16) return false;
  // The engine clips a store box at the tensor's edge, but it writes whole 16-byte units: a row
  // of, say, one f32 element had the three elements after it overwritten.  Rows that do not end
  // on a 16-byte boundary therefore take the strided-store epilogue.
  if ((N * elt) % 16) return false;
  if (M > 1 && (rs_elems <= 0 || (rs_elems * elt) % 16)) return false;
  if (nb > 1 && (bs_elems <= 0 || (bs_elems * elt) % 16)) return false;
  if (nb >= (1ll << 31)) return false;
  const int64_t rs_bytes = M > 1 ? rs_elems * elt : (N * elt + 15) / 16 * 16;
  const int64_t bs_bytes = nb > 1 ? bs_elems * elt : std::max<int64_t>(16, (rs_bytes * M + 15) / 16 * 16);
  if (rs_bytes >= (1ll << 40) || bs_bytes >= (1ll << 40)) return false;
  const CUtensorMapDataType dt = dtype == OXM_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                : dtype == OXM_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                    : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)nb};
  cuuint64_t strides[2] = {(cuuint64_t)rs_bytes, (cuuint64_t)bs_bytes};
  cuuint32_t box[3] = {(cuuint32_t)(kStageKBytes / elt), 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return ctx->encode(tm, dt, 3, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tile shape, CTA pairing and split-K factor for one product.
struct TileChoice {
  int bn, pair, splits;  // bn: the tile's width, any multiple of 32 up to its kernel's capacity
  int64_t sk_tiles;  // > 0: that many of the last tiles are shared out by contraction block (stream-K)
};

// The kernel instance (its widest tile) that runs tiles of `bn` columns.
int tile_class(int bn) { return bn > 256 ? 512 : bn > 128 ? 256 : bn > 64 ? 128 : 64; }
// Columns per tcgen05.mma: tiles wider than 256 are two MMAs side by side.
int tile_subn(int bn) { return bn > 256 ? bn / 2 : bn; }

// Stream-K applies when the tile count does not divide by the number of CTAs
// (or pairs): the remainder, plus one whole wave when the remainder is less
// than half a wave, is cut into equal runs, so that no tile is split more than
// three ways.  Returns the number of tiles shared out that way, or 0.
int64_t stream_k_tiles(int64_t tiles, int64_t slots, int32_t num_kb) {
  const int64_t full = tiles / slots, r = tiles % slots;
  if (r == 0 || num_kb < 16) return 0;
  if (r * 2 >= slots) return r;
  if (full == 0) return 0;  // fewer than half a wave of tiles: a split contraction serves better
  return slots + r;
}

// The longest accumulation chain the f32 path allows, in pipeline stages (K = 1024).
constexpr int kMaxChainKb = 3 * 1024 / 32;

// Pick the configuration with the smallest modelled time.  The model takes the
// larger of two bounds and adds the price of the reduction pass when the
// contraction is split:
//   - waves of tiles over the SMs (or SM pairs), each tile costing its
//     contraction blocks at the shape's measured rate, or its epilogue when the
//     contraction is too short to hide it;
//   - the unique bytes over HBM bandwidth (reads and writes at their own rates).
// One CTA cannot finish a contraction block faster than ~0.3 us whatever the
// tile's width (measured on a single L2-resident tile, K = 8192: 128 x 64 takes
// 41 us, 128 x 256 43 us; spreading the block's four tcgen05.mma over
// independent accumulators changed nothing, so it is the issuing thread's
// ~120 clocks per tcgen05 instruction, not a dependency).  At 256 columns that
// equals the tensor pipe's own time; narrower tiles leave the pipe idle.  So
// products too skinny to fill the SMs with 256-wide tiles get a split
// contraction rather than narrow tiles: [1..128, 8192] x [8192, 8192] takes
// 45.7 us unsplit at every tile width and 31 us split four ways.
TileChoice choose_tiles(const oxm_ctx *ctx, const Problem &P, bool tf32, int32_t num_kb, int min_b_rows, bool b_mn,
                        bool a_mn = false) {
  struct Cand { int cls, pair; double us_per_kb, us_epilogue; };
  // Microseconds per pipeline stage of one full-width tile at the ~1.45 GHz the
  // power cap sustains, and per epilogue.  With two accumulators the epilogue
  // hides behind the next tile's main loop unless the contraction is short; the
  // 512-wide class has one accumulator, whose first half is handed back after
  // one round of tensor-memory loads (the rest drains under the next tile's
  // first MMAs), so it pays a short epilogue always.
  static const Cand cands[] = {{512, 1, 0.706 / 1.03, 0.7}, {256, 1, 0.353, 3.0}, {256, 0, 0.353 / 0.93, 2.0},
                               {128, 0, 0.177 / 0.75, 1.5}, {128, 1, 0.177 / 0.59, 2.0}, {64, 0, 0.088 / 0.5, 1.0}};
  constexpr double kHbmRead = 6.0e6;    // bytes per microsecond from HBM
  constexpr double kHbmWrite = 4.3e6;   // ... and to it (measured on products that only write)
  const int32_t min_splits = tf32 ? std::max(1, (num_kb + kMaxChainKb - 1) / kMaxChainKb) : 1;
  static const int mult[] = {1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64};
  TileChoice best{256, 0, min_splits, 0};
  double best_t = 1e300;
  double a_nb = 1, b_nb = 1;  // batches each operand owns (broadcast dims repeat one copy)
  for (int d = 0; d < P.nbd; ++d) {
    if (P.a_bs[d] != 0) a_nb *= (double)P.bdims[d];
    if (P.b_bs[d] != 0) b_nb *= (double)P.bdims[d];
  }
  const double hbm_us = (double)P.nbatch * ((double)P.M * P.N * P.oelt) / kHbmWrite +
                        ((double)P.M * P.K * a_nb + (double)P.N * P.K * b_nb) * P.elt * (tf32 ? 3.0 : 1.0) / kHbmRead;
  const int forced_class = ctx->opt_tile_n ? tile_class((int)ctx->opt_tile_n) : 0;
  // A forced pairing that no candidate of the forced width has is dropped on the second pass.
  for (int pass = 0; pass < 2 && best_t == 1e300; ++pass)
  for (const Cand &c : cands) {
    // an N-major fp8 B tile is staged in boxes of 128 columns: each CTA must own at least one
    if ((c.pair ? c.cls / 2 : c.cls) < min_b_rows) continue;
    if (forced_class && c.cls != forced_class && ctx->opt_tile_n >= min_b_rows) continue;
    if (pass == 0 && ctx->opt_cta_pair >= 0 && c.pair != ctx->opt_cta_pair) continue;
    const int tm = kTileM * (c.pair ? 2 : 1);
    const int64_t slots = c.pair ? ctx->num_sms / 2 : ctx->num_sms;
    // Widths of this class: the full width, and narrower ones in steps of 32 columns down to
    // just above the next class (a tile count that fits the SMs better can beat a wider tile).
    const int w_lo = c.cls == 64 ? 64 : c.cls / 2 + 32;
    for (int bn = c.cls; bn >= w_lo; bn -= 32) {
      if (ctx->opt_tile_n && ctx->opt_tile_n >= min_b_rows) {
        if (bn != ctx->opt_tile_n) continue;
      } else {
        if (c.pair && P.M <= kTileM) continue;          // nothing for the second CTA to do
        if (bn > std::max(64, min_b_rows) && P.N <= bn / 2) continue;  // at least half of the tile is outside the matrix
        // narrower widths only where whole tiles of them cover the columns with less waste
        if (bn != c.cls && c.cls < 512) continue;
        // An MN-major B arrives in whole boxes of 128 bytes of columns: a narrower tile loads the
        // same boxes as the full one and only saves tensor time, which measured as no gain at all.
        if (bn != c.cls && b_mn) continue;
      }
      // An MN-major B is fetched in boxes that start at multiples of a CTA's share of the columns:
      // the TMA engine wants those starts on 16-byte boundaries.
      const int subc = tile_subn(bn) / (c.pair ? 2 : 1);
      if (b_mn && (subc * P.elt) % 16) continue;
      if ((c.pair ? subc * 2 : subc) % 16) continue;      // the MMA's N extent
      const int64_t tiles = ((P.M + tm - 1) / tm) * ((P.N + bn - 1) / bn) * P.nbatch;
      const double width = (double)bn / (double)c.cls;
      // A narrower tile moves the same A bytes for fewer flops: charge half of the lost width back.
      // With both operands MN-major (a weight gradient) the 256-wide pair tile measured 15 % slower
      // per block than with K-major ones (0.51 against 0.44 us), the 512-wide one the same.
      const double major = (a_mn && b_mn && c.cls <= 256) ? 1.15 : 1.0;
      const double kb_us = std::max(c.us_per_kb * major * (width + 0.04 * (1.0 - width)), 0.30);
      for (int m : mult) {
        const int32_t splits = min_splits * m;
        if (m > 1 && (ctx->opt_split_k == 0 || num_kb / splits < 16)) break;
        if (ctx->opt_split_k > 0 && splits != std::max<int64_t>(min_splits, ctx->opt_split_k)) continue;
        const double slab_bytes = (double)P.nbatch * P.M * P.N * 4.0;
        if (splits > 1 && slab_bytes * splits > 2e9) break;
        const int64_t waves = (tiles * splits + slots - 1) / slots;
        const int32_t kb = (num_kb + splits - 1) / splits;
        // one accumulator: the epilogue is exposed, and longer when the main loop is too
        // short for the previous tile's stores to drain meanwhile
        const double tile_us = c.cls > 256 ? kb * kb_us + c.us_epilogue * (kb < 16 ? 4.0 : 1.0)
                                           : std::max(kb * kb_us + 0.3, c.us_epilogue);
        double wave_us = (double)waves * tile_us;
        // Stream-K: every CTA gets the same number of blocks, at the price of one more epilogue and
        // the hand-over of a partial tile (~12 us), and of CTAs that walk K out of step, so that
        // tiles sharing an operand panel stop sharing its L2 lines.  Measured: it pays when whole
        // waves of ordinary tiles run beside the shared-out ones (4096^3: 127 -> 116 us; the weight
        // gradient of the linear layer: 427 -> 412 us) and loses badly when every tile is shared
        // out (1024 x 8192 x 8192: 97 -> 125 us).  Automatic only in the first situation.
        int64_t sk = 0;
        if (splits == 1 && ctx->opt_stream_k != 0 && ctx->opt_split_k != 0) {
          sk = stream_k_tiles(tiles, slots, kb);
          // (the one-accumulator tile shares work out with its two-phase epilogue, which keeps the
          // accumulator for about 7 us per tile; whole tiles get the register-packed one)
          const double sk_tile_us = c.cls > 256 ? kb * kb_us + 7.0 : tile_us;
          const double even_us = (double)tiles / (double)slots * sk_tile_us + 12.0;
          const bool whole_waves_beside = tiles - sk >= slots;
          if (sk > 0 && (ctx->opt_stream_k == 1 || (whole_waves_beside && even_us < wave_us))) wave_us = std::min(wave_us, even_us);
          else sk = 0;
        }
        double t = std::max(wave_us, hbm_us) + 0.01 * wave_us;  // the second term orders memory-bound ties
        if (splits > 1) t += 4.0 + slab_bytes * (splits + 1) / 4.0e6;  // launch + traffic of the reduction
        if (splits == min_splits ? t <= best_t : t < best_t) {  // ties go to the narrower, later candidate
          best_t = t; best = TileChoice{bn, c.pair, splits, sk};
        }
      }
    }
  }
  return best;
}

// Where the FFMA kernel and the tensor-core path cross on this GPU (the f32 path has two pack
// launches in front of its GEMM).
bool wants_tensor_cores(const Problem &P) {
  const double flops = 2.0 * (double)P.M * (double)P.N * (double)P.K * (double)P.nbatch;
  return P.K > 0 && flops >= (P.elt == 4 ? 2.0e8 : 8.0e6);
}

int launch_tcgen05(oxm_ctx *ctx, const Problem &P) {
  if (P.nbd > kMaxBatchDims) return fail(OXM_NOT_IMPLEMENTED, "matmul is not implemented for %d batch dims", P.nbd);
  if (P.M >= (1ll << 31) || P.N >= (1ll << 31) || P.K >= (1ll << 29) || P.nbatch >= (1ll << 31))
    return fail(OXM_NOT_IMPLEMENTED, "matmul is not implemented for extents above 2^31");
  const bool tf32 = P.elt == 4;
  const int kind = tf32 ? 1 : (P.elt == 1 ? 2 : 0);
  Staged sa{}, sb{};
  if (!stage_direct(P, false, sa)) {
    int st = stage_packed(ctx, P, false, 0, sa);
    if (st) return st;
  }
  if (!stage_direct(P, true, sb)) {
    int st = stage_packed(ctx, P, true, 1, sb);
    if (st) return st;
  }
  const int64_t Kst = tf32 ? sa.K : P.K;  // staged contraction length
  const int bk = kStageKBytes / P.elt;

  const int32_t num_kb_all = (int32_t)((Kst + bk - 1) / bk);
  const TileChoice choice = choose_tiles(ctx, P, tf32, num_kb_all, (kind == 2 && sb.mn_major) ? 128 : 0, sb.mn_major, sa.mn_major);
  const int bn = choice.bn, pair = choice.pair;
  const int cls = tile_class(bn), subn = tile_subn(bn);
  const int subc = pair ? subn / 2 : subn;  // B rows (columns of the product) one CTA stages per MMA
  const int tm = kTileM * (pair ? 2 : 1);

  GemmParams p{};
  p.M = (int32_t)P.M; p.N = (int32_t)P.N; p.K = (int32_t)Kst;
  p.bn = bn; p.subn = subn;
  p.tiles_m = (int32_t)((P.M + tm - 1) / tm);
  p.tiles_n = (int32_t)((P.N + bn - 1) / bn);
  p.num_kb = (int32_t)((Kst + bk - 1) / bk);
  p.nbatch = (int32_t)P.nbatch;
  p.num_tiles = (int64_t)p.tiles_m * p.tiles_n * P.nbatch;
  p.nbd = P.nbd;
  bool vec = P.o_cs == 1 && !is_fp8(P.out_dtype) && (reinterpret_cast<uintptr_t>(P.o) + P.o_off * P.oelt) % 16 == 0 &&
             (P.o_rs * P.oelt) % 16 == 0;
  int64_t obs[kMaxBatchDims] = {0};  // the output's (or the partial-sum workspace's) stride per batch dim
  for (int d = 0; d < P.nbd; ++d) {
    obs[d] = P.o_bs[d];
    if ((P.o_bs[d] * P.oelt) % 16) vec = false;
  }
  p.out = static_cast<uint8_t *>(P.o) + P.o_off * P.oelt;
  p.out_rs = P.o_rs; p.out_cs = P.o_cs;
  p.out_dtype = P.out_dtype;
  p.out_vec = vec ? 1 : 0;
  // format codes of the instruction descriptor: f16 0 / bf16 1 / tf32 2; in the f8f6f4 kind e4m3 0 / e5m2 1
  const uint32_t fmt = tf32 ? 2u : (P.dtype == OXM_BF16 || P.dtype == OXM_F8E5M2) ? 1u : 0u;
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((sa.mn_major ? 1u : 0u) << 15) | ((sb.mn_major ? 1u : 0u) << 16) |
            ((uint32_t)(subn >> 3) << 17) | ((uint32_t)(tm >> 4) << 24);
  p.status = ctx->status_dev;
  p.wait_limit_ns = (uint64_t)ctx->opt_wait_limit_ms * 1000000ull;
  p.splits = 1;
  p.kb_per_split = p.num_kb;
  p.tiles_per_split = p.num_tiles;
  p.split_ostride = 0;
  p.group_m = ctx->opt_group_m > 0 ? (int32_t)ctx->opt_group_m : (pair && bn <= 256 ? 8 : 16);
  p.epi = P.epi;
  // The tensor core adds each MMA's products into the fp32 accumulator with
  // truncation, an error of about 2^-24 per instruction that grows with the
  // length of the chain.  For f32 results that would pass 1e-5 beyond
  // K = 1024, so longer contractions are cut into chains of that length whose
  // partial sums are added afterwards in round-to-nearest fp32.
  ReduceParams rp{};
  if (choice.splits > 1) {
    p.splits = choice.splits;
    p.kb_per_split = (p.num_kb + p.splits - 1) / p.splits;
    p.splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;
    const int64_t slab = P.nbatch * P.M * P.N;
    int st2 = grow(ctx, ctx->pack_ws[2], (size_t)slab * p.splits * sizeof(float));
    if (st2) return st2;
    rp.ws = static_cast<const float *>(ctx->pack_ws[2].ptr);
    rp.out = P.o;
    rp.out_dtype = P.out_dtype;
    rp.epi = P.epi;  // the reduction, not the GEMM, finishes split products
    p.epi = Epilogue{};
    rp.splits = p.splits; rp.M = p.M; rp.N = p.N;
    rp.split_stride = slab; rp.total = slab;
    rp.o_off = P.o_off; rp.o_rs = P.o_rs; rp.o_cs = P.o_cs;
    rp.nbd = P.nbd;
    int64_t dense = P.M * P.N;
    for (int d = P.nbd - 1; d >= 0; --d) {
      rp.bdims[d] = (int32_t)P.bdims[d];
      rp.o_bs[d] = P.o_bs[d];
      obs[d] = dense;
      dense *= P.bdims[d];
    }
    p.out = ctx->pack_ws[2].ptr;
    p.out_rs = P.N; p.out_cs = 1;
    p.out_dtype = OXM_F32;  // partial sums stay fp32 whatever the operand type
    p.out_vec = (P.N % 4 == 0) ? 1 : 0;
    p.split_ostride = slab;
    p.num_tiles *= p.splits;
  }

  fill_batch_dims(p, P, sa, sb, obs);

  p.dp_tiles = p.num_tiles;
  p.sk_tiles = 0;
  if (p.splits == 1 && choice.sk_tiles > 0) {
    const int64_t slots = pair ? ctx->num_sms / 2 : ctx->num_sms;
    const size_t ws_bytes = (size_t)slots * (pair ? 2 : 1) * kTileM * cls * sizeof(float);  // the kernel spaces runs by its widest tile
    if ((size_t)slots * (pair ? 2 : 1) * 8 <= kSkFlagWords) {
      int st2 = grow(ctx, ctx->pack_ws[2], ws_bytes);
      if (st2) return st2;
      p.sk_tiles = choice.sk_tiles;
      p.dp_tiles = p.num_tiles - p.sk_tiles;
      p.sk_ws = static_cast<float *>(ctx->pack_ws[2].ptr);
      p.sk_flags = ctx->sk_flags;
      if (++ctx->sk_epoch == 0) ctx->sk_epoch = 1;
      p.sk_epoch = ctx->sk_epoch;
    }
  }

  CUtensorMap tmA, tmB, tmC;
  memset(&tmC, 0, sizeof(tmC));
  // Rows the box would fetch beyond the matrix are zero-filled at a cost per
  // row, so a K-major A of fewer than 128 rows gets a box of just its rows; the
  // tile's other rows keep whatever shared memory held and feed accumulator
  // rows that are never stored.
  const int a_box_rows = (!pair && !sa.mn_major && P.M < kTileM) ? (int)((P.M + 7) / 8 * 8) : kTileM;
  // Bytes one CTA's loads deliver per stage: its A rows, and per MMA its share of B, which an
  // MN-major B brings in whole boxes of `boxw` columns.
  const int boxw = kStageKBytes / P.elt;
  const int b_cols = sb.mn_major ? (subc + boxw - 1) / boxw * boxw : subc;
  p.stage_tx = (uint32_t)(kStageKBytes * (a_box_rows + (bn > 256 ? 2 : 1) * b_cols));
  int st = make_map(ctx, &tmA, sa, P.dtype, P.elt, a_box_rows, bk);
  if (st) return st;
  st = make_map(ctx, &tmB, sb, P.dtype, P.elt, subc, bk);
  if (st) return st;
  // The epilogue writes through a bulk tensor store when the output is a
  // row-contiguous, 16-byte-aligned window whose batch dims fold into one stride.
  if (p.splits > 1) {
    // fp32 partial sums from 16-bit operands take the strided-store epilogue
    p.out_tma = tf32 && make_out_map(ctx, &tmC, p.out, OXM_F32, 4, P.M, P.N, P.nbatch * p.splits, P.N, P.M * P.N) ? 1 : 0;
  } else if ((P.o_cs == 1 || P.N == 1) && (tf32 ? P.out_dtype == OXM_F32 : (P.out_dtype == OXM_BF16 || P.out_dtype == OXM_F16))) {
    // the staged epilogue writes 4-byte chunks for the f32 path and 2-byte chunks otherwise
    bool fold = true;
    for (int d = 0; d + 1 < P.nbd; ++d) fold = fold && P.o_bs[d] == P.o_bs[d + 1] * P.bdims[d + 1];
    p.out_tma = fold && make_out_map(ctx, &tmC, p.out, P.out_dtype, P.oelt, P.M, P.N, P.nbatch, P.o_rs,
                                     P.nbd ? P.o_bs[P.nbd - 1] : 0) ? 1 : 0;
  }
  if (ctx->opt_tma_store == 0) p.out_tma = 0;

  int grid;
  if (p.sk_tiles > 0) grid = pair ? 2 * (ctx->num_sms / 2) : ctx->num_sms;  // every run needs its CTA
  else if (pair) grid = 2 * (int)std::min<int64_t>(p.num_tiles, ctx->num_sms / 2);
  else grid = (int)std::min<int64_t>(p.num_tiles, ctx->num_sms);

  st = launch_gemm(ctx, kind, sa.mn_major, sb.mn_major, cls, pair, tmA, tmB, tmC, p, grid);
  if (st) return st;
  if (bn != cls) {  // the instance's name carries its capacity; say what width it ran at
    const size_t len = strlen(ctx->last_kernel);
    snprintf(ctx->last_kernel + len, sizeof(ctx->last_kernel) - len, "_w%d", bn);
  }
  ctx->launches[0]++; ctx->launches[1]++;
  if (p.splits > 1) {
    const int64_t blocks = std::min<int64_t>((rp.total + 255) / 256, (int64_t)ctx->num_sms * 16);
    splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(rp);
    CUDA_TRY(cudaGetLastError());
    ctx->launches[0]++; ctx->launches[3]++;
  }
  return OXM_OK;
}

// ---------------------------------------------------------------------------
// block-scaled fp8 product (MX): C = (A * 2^(sa - 127)) . (B * 2^(sb - 127)),
// one E8M0 scale per 32 contraction elements of every row of A and column of B
// ---------------------------------------------------------------------------

// Regroup one operand's scale view into atoms in workspace `slot` and describe them to the TMA
// engine as {128 words, row groups, stages, batch}; a load takes one atom (A) or three
// neighbouring row groups' atoms (B: all that a tile's columns can touch).
int stage_scale_atoms(oxm_ctx *ctx, const Problem &P, bool is_b, const oxm_view *sv, const int64_t *sv_bs, int slot,
                      CUtensorMap *tm) {
  const int64_t rows = is_b ? P.N : P.M, kblocks = P.K / 32;
  SfParams sp{};
  sp.src = static_cast<const uint8_t *>(sv->base);
  sp.src_off = sv->offset;
  sp.src_rs = sv->strides[sv->ndim - (is_b ? 1 : 2)];
  sp.src_ks = sv->strides[sv->ndim - (is_b ? 2 : 1)];
  sp.rows = (int32_t)rows; sp.kblocks = (int32_t)kblocks;
  sp.row_groups = (int32_t)((rows + 127) / 128);
  sp.stages = (int32_t)((kblocks + 3) / 4);
  const int64_t *obs = is_b ? P.b_bs : P.a_bs;
  int64_t nb = 1;
  sp.nbd = 0;
  for (int d = 0; d < P.nbd; ++d) {
    if (obs[d] == 0) continue;  // the operand repeats over this dim, and so do its scales
    sp.bdims[sp.nbd] = (int32_t)P.bdims[d];
    sp.src_bs[sp.nbd] = sv_bs[d];
    sp.nbd++;
    nb *= P.bdims[d];
  }
  const int64_t atoms = nb * sp.row_groups * sp.stages;
  if (nb * sp.row_groups >= (1ll << 31) || atoms >= (1ll << 40)) return fail(OXM_NOT_IMPLEMENTED, "matmul_mx is not implemented for %lld scale atoms", (long long)atoms);
  sp.total_words = atoms * 128;
  int st = grow(ctx, ctx->pack_ws[slot], (size_t)atoms * kSfAtomBytes);
  if (st) return st;
  sp.dst = static_cast<uint32_t *>(ctx->pack_ws[slot].ptr);
  const int64_t blocks = std::min<int64_t>((sp.total_words + 255) / 256, (int64_t)ctx->num_sms * 32);
  mx_scale_atoms_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(sp);
  CUDA_TRY(cudaGetLastError());
  ctx->launches[0]++; ctx->launches[3]++;
  cuuint64_t dims[4] = {128, (cuuint64_t)sp.row_groups, (cuuint64_t)sp.stages, (cuuint64_t)nb};
  cuuint64_t strides[3] = {(cuuint64_t)kSfAtomBytes, (cuuint64_t)kSfAtomBytes * (cuuint64_t)sp.row_groups,
                           (cuuint64_t)kSfAtomBytes * (cuuint64_t)sp.row_groups * (cuuint64_t)sp.stages};
  cuuint32_t box[4] = {128, is_b ? (cuuint32_t)kSfMaxBAtoms : 1u, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = ctx->encode(tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, sp.dst, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(OXM_CUDA_ERROR, "cuTensorMapEncodeTiled failed (%d) for the scale atoms", (int)r);
  return OXM_OK;
}

int launch_mx(oxm_ctx *ctx, const Problem &P, const oxm_view *a_scale, const int64_t *sa_bs, const oxm_view *b_scale,
              const int64_t *sb_bs) {
  if (P.nbd > kMaxBatchDims) return fail(OXM_NOT_IMPLEMENTED, "matmul_mx is not implemented for %d batch dims", P.nbd);
  if (P.M >= (1ll << 31) || P.N >= (1ll << 31) || P.K >= (1ll << 29) || P.nbatch >= (1ll << 31))
    return fail(OXM_NOT_IMPLEMENTED, "matmul_mx is not implemented for extents above 2^31");
  // operands: K-major for the tensor core, in place where the TMA engine can address them
  Staged sa{}, sb{};
  if (!stage_direct(P, false, sa) || sa.mn_major) {
    int st = stage_packed(ctx, P, false, 0, sa);
    if (st) return st;
  }
  if (!stage_direct(P, true, sb) || sb.mn_major) {
    int st = stage_packed(ctx, P, true, 1, sb);
    if (st) return st;
  }
  CUtensorMap sf[2];
  int st = stage_scale_atoms(ctx, P, false, a_scale, sa_bs, 3, &sf[0]);
  if (st) return st;
  st = stage_scale_atoms(ctx, P, true, b_scale, sb_bs, 4, &sf[1]);
  if (st) return st;

  // Tile widths of this kind: the MMA takes B's scales from the tensor-memory column its address
  // names, one column per 32 columns of B, and that address must be even: a tile that starts 32
  // or 96 columns into a 128-column scale atom, or a second sub-tile that starts an odd number of
  // 32-column groups after the first (width 320), is refused by the hardware with "misaligned
  // address" (seen on widths 160, 224 and 320; 128, 192, 256 and 384 run).  A tile's columns may
  // touch at most three atoms.  So: 128 or 192 columns for the two-accumulator tile, 256 or 384
  // for the one-accumulator tile (two MMAs side by side, which read every A stage twice).
  // Whichever leaves the fewest idle pair-waves wins.
  const int tm = 2 * kTileM;
  const int64_t tiles_m = (P.M + tm - 1) / tm, slots = std::max(1, ctx->num_sms / 2);
  // Per column of tile width the four shapes measured (8192^3, TFLOP/s): 384: 2175, 256: 1705,
  // 192: 1655, 128: 1288 - the wider the tile, the fewer scale copies and MMA instructions per flop.
  auto cost = [&](int w) {
    const int64_t tiles = tiles_m * ((P.N + w - 1) / w) * P.nbatch;
    const double per_col = w == 384 ? 1.0 : w == 256 ? 1.28 : w == 192 ? 1.31 : 1.69;
    return (double)((tiles + slots - 1) / slots) * (w * per_col + 24);  // a tile's time grows with its width, plus its drain
  };
  int bn = 384;
  for (int w : {256, 192, 128})
    if (cost(w) < cost(bn) * 0.97) bn = w;
  if (ctx->opt_tile_n == 128 || ctx->opt_tile_n == 192 || ctx->opt_tile_n == 256 || ctx->opt_tile_n == 384) bn = (int)ctx->opt_tile_n;
  const int cls = bn > 192 ? 512 : 256;
  const int nsub = cls == 512 ? 2 : 1;
  const int subn = bn / nsub, subc = subn / 2;
  const int bk = kStageKBytes;  // one byte per element

  GemmParams p{};
  p.M = (int32_t)P.M; p.N = (int32_t)P.N; p.K = (int32_t)P.K;
  p.bn = bn; p.subn = subn;
  p.tiles_m = (int32_t)tiles_m;
  p.tiles_n = (int32_t)((P.N + bn - 1) / bn);
  p.num_kb = (int32_t)((P.K + bk - 1) / bk);
  p.nbatch = (int32_t)P.nbatch;
  p.num_tiles = (int64_t)p.tiles_m * p.tiles_n * P.nbatch;
  p.nbd = P.nbd;
  bool vec = P.o_cs == 1 && !is_fp8(P.out_dtype) && (reinterpret_cast<uintptr_t>(P.o) + P.o_off * P.oelt) % 16 == 0 &&
             (P.o_rs * P.oelt) % 16 == 0;
  for (int d = 0; d < P.nbd; ++d)
    if ((P.o_bs[d] * P.oelt) % 16) vec = false;
  fill_batch_dims(p, P, sa, sb, P.o_bs);
  p.out = static_cast<uint8_t *>(P.o) + P.o_off * P.oelt;
  p.out_rs = P.o_rs; p.out_cs = P.o_cs;
  p.out_dtype = P.out_dtype;
  p.out_vec = vec ? 1 : 0;
  // block-scaled instruction descriptor: operand formats e4m3 0 / e5m2 1, E8M0 scales, N and M
  // of one MMA; the kernel adds each contraction block's scale ids
  const uint32_t fmt = P.dtype == OXM_F8E5M2 ? 1u : 0u;
  p.idesc = (fmt << 7) | (fmt << 10) | ((uint32_t)(subn >> 3) << 17) | (1u << 23) | ((uint32_t)(tm >> 4) << 24);
  p.status = ctx->status_dev;
  p.wait_limit_ns = (uint64_t)ctx->opt_wait_limit_ms * 1000000ull;
  p.splits = 1;
  p.kb_per_split = p.num_kb;
  p.tiles_per_split = p.num_tiles;
  p.dp_tiles = p.num_tiles;
  p.group_m = ctx->opt_group_m > 0 ? (int32_t)ctx->opt_group_m : (cls == 512 ? 16 : 8);
  p.epi = P.epi;
  // per CTA and stage: its A rows, its share of B, the atom of its rows' scales and three atoms of B's
  p.stage_tx = (uint32_t)(kStageKBytes * (kTileM + nsub * subc) + kSfAtomBytes * (1 + kSfMaxBAtoms));

  CUtensorMap tmA, tmB, tmC;
  memset(&tmC, 0, sizeof(tmC));
  st = make_map(ctx, &tmA, sa, P.dtype, 1, kTileM, bk);
  if (st) return st;
  st = make_map(ctx, &tmB, sb, P.dtype, 1, subc, bk);
  if (st) return st;
  if ((P.o_cs == 1 || P.N == 1) && (P.out_dtype == OXM_BF16 || P.out_dtype == OXM_F16)) {
    bool fold = true;
    for (int d = 0; d + 1 < P.nbd; ++d) fold = fold && P.o_bs[d] == P.o_bs[d + 1] * P.bdims[d + 1];
    p.out_tma = fold && make_out_map(ctx, &tmC, p.out, P.out_dtype, P.oelt, P.M, P.N, P.nbatch, P.o_rs,
                                     P.nbd ? P.o_bs[P.nbd - 1] : 0) ? 1 : 0;
  }
  if (ctx->opt_tma_store == 0) p.out_tma = 0;
  const int grid = 2 * (int)std::min<int64_t>(p.num_tiles, slots);
  st = launch_gemm(ctx, 3, false, false, cls, 1, tmA, tmB, tmC, p, grid, sf);
  if (st) return st;
  const size_t len = strlen(ctx->last_kernel);
  snprintf(ctx->last_kernel + len, sizeof(ctx->last_kernel) - len, "_w%d", bn);
  ctx->launches[0]++; ctx->launches[1]++;
  return OXM_OK;
}

// The scale view of one operand: u8 (E8M0), the operand's shape with the contraction dim divided
// by 32.  Fills the view's stride for every batch dim of the normalised problem.
int check_scale_view(const oxm_ctx *ctx, const char *which, const oxm_view *operand, const oxm_view *sv, bool is_b,
                     const oxm_view *out, const Problem &P, int64_t *sv_bs) {
  if (sv->dtype != OXM_U8)
    return fail(OXM_DTYPE_MISMATCH, "dtype mismatch: expected U8, got %s in matmul_mx (%s: E8M0 scales are bytes)", dtype_name(sv->dtype), which);
  if (sv->device != ctx->device)
    return fail(OXM_DEVICE_MISMATCH, "device mismatch: Cuda{index: %d} vs Cuda{index: %d} in matmul_mx (%s)", ctx->device, sv->device, which);
  bool ok = sv->ndim == operand->ndim;
  const int kd = operand->ndim - (is_b ? 2 : 1);  // the contraction dim
  std::string exp = "[";
  for (int i = 0; i < operand->ndim; ++i) {
    const int64_t e = i == kd ? operand->shape[i] / 32 : operand->shape[i];
    if (ok && sv->shape[i] != e) ok = false;
    exp += (i ? ", " : "") + std::to_string(e);
  }
  exp += "]";
  if (!ok) return fail(OXM_SHAPE_MISMATCH, "shape mismatch: expected %s, got %s in matmul_mx (%s)", exp.c_str(), shape_str(sv).c_str(), which);
  int64_t numel = 1;
  for (int i = 0; i < sv->ndim; ++i) numel *= sv->shape[i];
  if (numel > 0 && !sv->base) return fail(OXM_INVALID_ARGUMENT, "matmul_mx: %s with null storage", which);
  // strides over the problem's batch dims, in normalise()'s order (extent-1 dims dropped)
  const int nbd = out->ndim - 2;
  const int64_t *obs = is_b ? P.b_bs : P.a_bs;
  int n = 0;
  for (int d = 0; d < nbd; ++d) {
    if (out->shape[d] == 1) continue;
    const int od = d - (nbd - (operand->ndim - 2));
    sv_bs[n] = (od >= 0 && sv->shape[od] != 1) ? sv->strides[od] : 0;
    if ((obs[n] == 0) != (sv_bs[n] == 0))
      return fail(OXM_INVALID_ARGUMENT, "matmul_mx: %s must repeat over batch dim %d exactly where its operand does", which, d);
    ++n;
  }
  return OXM_OK;
}

int run_matmul_mx(oxm_ctx *ctx, const oxm_view *a, const oxm_view *a_scale, const oxm_view *b, const oxm_view *b_scale,
                  const oxm_view *out) {
  if (!a_scale || !b_scale) return fail(OXM_INVALID_ARGUMENT, "matmul_mx: null argument");
  int st = validate(ctx, a, b, out, true, false);
  if (st) return st;
  if (!is_fp8(a->dtype)) return fail(OXM_UNSUPPORTED_DTYPE, "dtype %s is not supported by matmul_mx (F8E4M3 or F8E5M2 operands)", dtype_name(a->dtype));
  const int64_t K = a->shape[a->ndim - 1];
  if (K % 32)
    return fail(OXM_SHAPE_MISMATCH, "shape mismatch: expected a contraction length that is a multiple of 32, got %lld in matmul_mx", (long long)K);
  for (const oxm_view *v : {a, b, out}) {
    int64_t numel = 1;
    for (int i = 0; i < v->ndim; ++i) numel *= v->shape[i];
    if (numel > 0 && v->base == nullptr) return fail(OXM_INVALID_ARGUMENT, "matmul_mx: view with null storage");
  }
  Problem P = normalise(a, b, out, false);
  int64_t sa_bs[OXM_MAX_DIMS] = {0}, sb_bs[OXM_MAX_DIMS] = {0};
  st = check_scale_view(ctx, "a_scale", a, a_scale, false, out, P, sa_bs);
  if (st) return st;
  st = check_scale_view(ctx, "b_scale", b, b_scale, true, out, P, sb_bs);
  if (st) return st;
  if (P.M == 0 || P.N == 0 || P.nbatch == 0) return OXM_OK;
  std::lock_guard<std::mutex> lock(ctx->mu);
  CUDA_TRY(cudaSetDevice(ctx->device));
  if (K == 0) return launch_simt(ctx, P);  // an empty contraction: zeros, written by the FFMA kernel's store path
  return launch_mx(ctx, P, a_scale, sa_bs, b_scale, sb_bs);
}

int run_matmul(oxm_ctx *ctx, const oxm_view *a, const oxm_view *b, const oxm_view *out, bool batched,
               const oxm_epilogue *ep = nullptr) {
  int st = validate(ctx, a, b, out, batched, false);
  if (st) return st;
  Epilogue epi{};
  if (ep) {
    const char *op = "matmul_fused";
    if (ep->activation < OXM_ACT_NONE || ep->activation > OXM_ACT_GELU)
      return fail(OXM_INVALID_ARGUMENT, "%s: unknown activation %d", op, ep->activation);
    if (ep->bias) {
      const oxm_view *bv = ep->bias;
      const int64_t n = b->shape[b->ndim - 1];
      if (bv->ndim != 1 || bv->shape[0] != n)
        return fail(OXM_SHAPE_MISMATCH, "shape mismatch: expected [%lld], got %s in %s (bias)", (long long)n, shape_str(bv).c_str(), op);
      if (bv->dtype != a->dtype)
        return fail(OXM_DTYPE_MISMATCH, "dtype mismatch: expected %s, got %s in %s (bias)", dtype_name(a->dtype), dtype_name(bv->dtype), op);
      if (bv->device != ctx->device)
        return fail(OXM_DEVICE_MISMATCH, "device mismatch: Cuda{index: %d} vs Cuda{index: %d} in %s (bias)", a->device, bv->device, op);
      if (n > 0 && !bv->base) return fail(OXM_INVALID_ARGUMENT, "%s: bias view with null storage", op);
      epi.bias = static_cast<const uint8_t *>(bv->base) + bv->offset * dtype_size(bv->dtype);
      epi.bias_stride = bv->strides[0];
      epi.bias_dtype = bv->dtype;
    }
    epi.activation = ep->activation;
    epi.accumulate = ep->accumulate ? 1 : 0;
    epi.any = (epi.bias || epi.activation || epi.accumulate) ? 1 : 0;
  }
  for (const oxm_view *v : {a, b, out}) {
    int64_t numel = 1;
    for (int i = 0; i < v->ndim; ++i) numel *= v->shape[i];
    if (numel > 0 && v->base == nullptr) return fail(OXM_INVALID_ARGUMENT, "matmul: view with null storage");
  }
  Problem P = normalise(a, b, out);
  P.epi = epi;
  if (P.M == 0 || P.N == 0 || P.nbatch == 0) return OXM_OK;  // nothing to write
  std::lock_guard<std::mutex> lock(ctx->mu);
  CUDA_TRY(cudaSetDevice(ctx->device));
  // Small products and empty contractions go to the FFMA kernel; the rest to
  // the tensor cores.  Both are GPU kernels; there is no host path.
  bool use_tc;
  if (ctx->opt_kernel == 1) use_tc = false;
  else if (ctx->opt_kernel == 2) use_tc = P.K > 0;
  else use_tc = wants_tensor_cores(P);
  return use_tc ? launch_tcgen05(ctx, P) : launch_simt(ctx, P);
}

}  // namespace

// The decisions run_matmul would take for these views with default options, without touching a GPU.
extern "C" int oxm_plan_matmul(const oxm_view *a, const oxm_view *b, const oxm_view *out, int num_sms, int32_t plan[8]) {
  if (!a || !b || !out || !plan || num_sms < 2) return fail(OXM_INVALID_ARGUMENT, "plan_matmul: null argument or fewer than 2 SMs");
  oxm_ctx fake;
  fake.device = a->device;
  fake.num_sms = num_sms;
  int st = validate(&fake, a, b, out, true, false);
  if (st) return st;
  const Problem P = normalise(a, b, out);
  for (int i = 0; i < 8; ++i) plan[i] = 0;
  if (P.M == 0 || P.N == 0 || P.nbatch == 0) return OXM_OK;  // nothing to launch
  if (!wants_tensor_cores(P)) { plan[0] = 1; return OXM_OK; }
  const bool tf32 = P.elt == 4;
  Staged sa{}, sb{};
  const bool a_direct = stage_direct(P, false, sa), b_direct = stage_direct(P, true, sb);
  const int64_t Kst = tf32 ? 3 * ((P.K + 31) / 32 * 32) : P.K;
  const int bk = kStageKBytes / P.elt;
  const TileChoice c = choose_tiles(&fake, P, tf32, (int32_t)((Kst + bk - 1) / bk), (P.elt == 1 && b_direct && sb.mn_major) ? 128 : 0,
                                    b_direct && sb.mn_major, a_direct && sa.mn_major);
  plan[0] = 2; plan[1] = c.bn; plan[2] = c.pair; plan[3] = c.splits;
  plan[4] = a_direct ? 0 : 1; plan[5] = b_direct ? 0 : 1;
  plan[6] = (int32_t)c.sk_tiles;
  return OXM_OK;
}

namespace {

int check_status(oxm_ctx *ctx) {
  CUDA_TRY(cudaMemcpyAsync(ctx->status_host, ctx->status_dev, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
  CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  const uint32_t s = *ctx->status_host;
  if (s != 0) {
    CUDA_TRY(cudaMemsetAsync(ctx->status_dev, 0, sizeof(uint32_t), ctx->stream));
    if (s == OXM_TIMEOUT)
      return fail(OXM_TIMEOUT, "a bounded device-side wait expired in %s; the result of that launch is undefined", ctx->last_kernel);
    if (s == OXM_DIVIDE_BY_ZERO)
      return fail(OXM_DIVIDE_BY_ZERO, "integer division by zero in div (the elements with a zero divisor were written as 0)");
    return fail(OXM_CUDA_ERROR, "device-side status %u in %s", s, ctx->last_kernel);
  }
  return OXM_OK;
}

// Element range [lo, hi] a view touches, relative to its base.
void view_extent(const oxm_view *v, int64_t *lo, int64_t *hi, int64_t *numel) {
  int64_t l = v->offset, h = v->offset, n = 1;
  for (int i = 0; i < v->ndim; ++i) {
    n *= v->shape[i];
    if (v->shape[i] > 0) {
      const int64_t span = (v->shape[i] - 1) * v->strides[i];
      if (span > 0) h += span; else l += span;
    }
  }
  *lo = l; *hi = h; *numel = n;
}

}  // namespace

// ===========================================================================
// exported functions
// ===========================================================================
extern "C" {

const char *oxm_last_error(void) { return g_last_error.c_str(); }

const char *oxm_status_name(int status) {
  static const char *names[] = {"Ok", "ShapeMismatch", "BroadcastIncompatible", "DTypeMismatch", "UnsupportedDType",
                                "DeviceMismatch", "IndexOutOfBounds", "RankMismatch", "BackendUnavailable",
                                "NotImplemented", "CudaError", "Timeout", "InvalidArgument", "DivisionByZero"};
  return (status >= 0 && status <= 13) ? names[status] : "Unknown";
}

const char *oxm_backend_name(void) { return "b200-tcgen05"; }

int oxm_device_count(int *count) {
  if (!count) return fail(OXM_INVALID_ARGUMENT, "oxm_device_count: null argument");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  *count = n;
  return OXM_OK;
}

int oxm_ctx_create(int device_index, oxm_ctx **out) {
  if (!out) return fail(OXM_INVALID_ARGUMENT, "oxm_ctx_create: null argument");
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  if (device_index < 0 || device_index >= n)
    return fail(OXM_BACKEND_UNAVAILABLE, "no backend available for device Cuda { index: %d } (%d CUDA devices visible)", device_index, n);
  cudaDeviceProp prop;
  CUDA_TRY(cudaGetDeviceProperties(&prop, device_index));
  if (prop.major != 10)
    return fail(OXM_BACKEND_UNAVAILABLE, "no backend available for device Cuda { index: %d }: %s is sm_%d%d, this backend is built for sm_100a",
                device_index, prop.name, prop.major, prop.minor);
  CUDA_TRY(cudaSetDevice(device_index));
  oxm_ctx *ctx = new oxm_ctx();
  ctx->device = device_index;
  ctx->num_sms = prop.multiProcessorCount;
  cudaError_t e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaMalloc(&ctx->status_dev, sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemset(ctx->status_dev, 0, sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMalloc(&ctx->sk_flags, kSkFlagWords * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemset(ctx->sk_flags, 0, kSkFlagWords * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaHostAlloc(&ctx->status_host, sizeof(uint32_t), cudaHostAllocDefault);
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (e == cudaSuccess) e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || !fn) {
    int st = fail(OXM_CUDA_ERROR, "context set-up failed: %s", e != cudaSuccess ? cudaGetErrorString(e) : "cuTensorMapEncodeTiled not found");
    oxm_ctx_destroy(ctx);
    return st;
  }
  ctx->encode = reinterpret_cast<EncodeTiledFn>(fn);
  if (const char *env = getenv("OXM_WAIT_LIMIT_MS")) {
    const long v = atol(env);
    if (v >= 1 && v <= 600000) ctx->opt_wait_limit_ms = v;
  }
  // Keep freed blocks in the pool: allocation in the steady state costs no driver call.
  cudaMemPool_t pool;
  if (cudaDeviceGetDefaultMemPool(&pool, device_index) == cudaSuccess) {
    uint64_t thresh = UINT64_MAX;
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &thresh);
  }
  *out = ctx;
  return OXM_OK;
}

int oxm_ctx_destroy(oxm_ctx *ctx) {
  if (!ctx) return OXM_OK;
  cudaSetDevice(ctx->device);
  if (ctx->stream) cudaStreamSynchronize(ctx->stream);
  for (auto &w : ctx->pack_ws) if (w.ptr) cudaFree(w.ptr);
  for (auto &w : ctx->host_stage) if (w.ptr) cudaFree(w.ptr);
  for (auto &e : ctx->pipe_events) if (e) cudaEventDestroy(e);
  if (ctx->copy_in) cudaStreamDestroy(ctx->copy_in);
  if (ctx->copy_out) cudaStreamDestroy(ctx->copy_out);
  if (ctx->status_dev) cudaFree(ctx->status_dev);
  if (ctx->sk_flags) cudaFree(ctx->sk_flags);
  if (ctx->status_host) cudaFreeHost(ctx->status_host);
  if (ctx->stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
  return OXM_OK;
}

int oxm_ctx_device(const oxm_ctx *ctx, int *device_index) {
  if (!ctx || !device_index) return fail(OXM_INVALID_ARGUMENT, "oxm_ctx_device: null argument");
  *device_index = ctx->device;
  return OXM_OK;
}

int oxm_alloc(oxm_ctx *ctx, size_t bytes, void **out) {
  if (!ctx || !out) return fail(OXM_INVALID_ARGUMENT, "oxm_alloc: null argument");
  *out = nullptr;
  CUDA_TRY(cudaSetDevice(ctx->device));
  if (bytes == 0) bytes = 16;
  CUDA_TRY(cudaMallocAsync(out, bytes, ctx->stream));
  return OXM_OK;
}

int oxm_free(oxm_ctx *ctx, void *ptr) {
  if (!ctx) return fail(OXM_INVALID_ARGUMENT, "oxm_free: null context");
  if (!ptr) return OXM_OK;
  CUDA_TRY(cudaSetDevice(ctx->device));
  CUDA_TRY(cudaFreeAsync(ptr, ctx->stream));
  return OXM_OK;
}

int oxm_h2d(oxm_ctx *ctx, void *dst_device, const void *src_host, size_t bytes) {
  if (!ctx || (bytes && (!dst_device || !src_host))) return fail(OXM_INVALID_ARGUMENT, "oxm_h2d: null argument");
  CUDA_TRY(cudaSetDevice(ctx->device));
  if (bytes) CUDA_TRY(cudaMemcpyAsync(dst_device, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return OXM_OK;
}

int oxm_d2h(oxm_ctx *ctx, void *dst_host, const void *src_device, size_t bytes) {
  if (!ctx || (bytes && (!dst_host || !src_device))) return fail(OXM_INVALID_ARGUMENT, "oxm_d2h: null argument");
  CUDA_TRY(cudaSetDevice(ctx->device));
  if (bytes) CUDA_TRY(cudaMemcpyAsync(dst_host, src_device, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  std::lock_guard<std::mutex> lock(ctx->mu);
  return check_status(ctx);
}

int oxm_memset(oxm_ctx *ctx, void *dst_device, int byte, size_t bytes) {
  if (!ctx || (bytes && !dst_device)) return fail(OXM_INVALID_ARGUMENT, "oxm_memset: null argument");
  CUDA_TRY(cudaSetDevice(ctx->device));
  if (bytes) CUDA_TRY(cudaMemsetAsync(dst_device, byte, bytes, ctx->stream));
  return OXM_OK;
}

int oxm_copy_peer(oxm_ctx *dst_ctx, void *dst_device, oxm_ctx *src_ctx, const void *src_device, size_t bytes) {
  if (!dst_ctx || !src_ctx || (bytes && (!dst_device || !src_device))) return fail(OXM_INVALID_ARGUMENT, "oxm_copy_peer: null argument");
  if (bytes == 0) return OXM_OK;
  // The copy waits for what the source context has queued so far (its uploads), and runs on the
  // destination's stream, so the destination's later kernels see the bytes.
  cudaEvent_t ready = nullptr;
  CUDA_TRY(cudaSetDevice(src_ctx->device));
  CUDA_TRY(cudaEventCreateWithFlags(&ready, cudaEventDisableTiming));
  cudaError_t e = cudaEventRecord(ready, src_ctx->stream);
  if (e == cudaSuccess) e = cudaSetDevice(dst_ctx->device);
  if (e == cudaSuccess && dst_ctx->device != src_ctx->device) {
    // direct copies over NVLink where the pair allows it; without it the runtime stages the copy
    int can = 0;
    if (cudaDeviceCanAccessPeer(&can, dst_ctx->device, src_ctx->device) == cudaSuccess && can) {
      const cudaError_t pe = cudaDeviceEnablePeerAccess(src_ctx->device, 0);
      if (pe != cudaSuccess) cudaGetLastError();  // already enabled, or refused: the copy works either way
    }
  }
  if (e == cudaSuccess) e = cudaStreamWaitEvent(dst_ctx->stream, ready, 0);
  if (e == cudaSuccess)
    e = cudaMemcpyPeerAsync(dst_device, dst_ctx->device, src_device, src_ctx->device, bytes, dst_ctx->stream);
  cudaEventDestroy(ready);  // released once the work that uses it has completed
  if (e != cudaSuccess) return fail(OXM_CUDA_ERROR, "oxm_copy_peer failed: %s", cudaGetErrorString(e));
  return OXM_OK;
}

int oxm_sync(oxm_ctx *ctx) {
  if (!ctx) return fail(OXM_INVALID_ARGUMENT, "oxm_sync: null context");
  CUDA_TRY(cudaSetDevice(ctx->device));
  std::lock_guard<std::mutex> lock(ctx->mu);
  return check_status(ctx);
}

int oxm_host_alloc(size_t bytes, void **out) {
  if (!out) return fail(OXM_INVALID_ARGUMENT, "oxm_host_alloc: null argument");
  *out = nullptr;
  CUDA_TRY(cudaHostAlloc(out, bytes ? bytes : 16, cudaHostAllocDefault));
  return OXM_OK;
}

int oxm_host_free(void *ptr) {
  if (ptr) CUDA_TRY(cudaFreeHost(ptr));
  return OXM_OK;
}

int oxm_matmul(oxm_ctx *ctx, const oxm_view *a, const oxm_view *b, const oxm_view *out) {
  return run_matmul(ctx, a, b, out, false);
}

int oxm_batched_matmul(oxm_ctx *ctx, const oxm_view *a, const oxm_view *b, const oxm_view *out) {
  return run_matmul(ctx, a, b, out, true);
}

int oxm_matmul_mx(oxm_ctx *ctx, const oxm_view *a, const oxm_view *a_scale, const oxm_view *b, const oxm_view *b_scale,
                  const oxm_view *out) {
  return run_matmul_mx(ctx, a, a_scale, b, b_scale, out);
}

int oxm_matmul_fused(oxm_ctx *ctx, const oxm_view *a, const oxm_view *b, const oxm_view *out, const oxm_epilogue *ep) {
  return run_matmul(ctx, a, b, out, true, ep);
}

int oxm_batched_matmul_host(oxm_ctx *ctx, const oxm_view *a, const oxm_view *b, const oxm_view *out) {
  int st = validate(ctx, a, b, out, true, true);
  if (st) return st;
  CUDA_TRY(cudaSetDevice(ctx->device));
  std::lock_guard<std::mutex> host_lock(ctx->host_mu);
  const oxm_view *hv[3] = {a, b, out};
  oxm_view dv[3];
  int64_t lo[3], hi[3], numel[3];
  const int elt = dtype_size(a->dtype);
  if (out->dtype != a->dtype) return fail(OXM_NOT_IMPLEMENTED, "matmul is not implemented for a widened fp8 output through the host entry point");
  {
    std::lock_guard<std::mutex> lock(ctx->mu);
    for (int i = 0; i < 3; ++i) {
      view_extent(hv[i], &lo[i], &hi[i], &numel[i]);
      dv[i] = *hv[i];
      dv[i].device = ctx->device;
      if (numel[i] == 0) { dv[i].base = nullptr; continue; }
      if (!hv[i]->base) return fail(OXM_INVALID_ARGUMENT, "matmul: view with null storage");
      if (i == 2 && hi[i] - lo[i] + 1 != numel[i])
        return fail(OXM_INVALID_ARGUMENT, "matmul: a host output must be dense (the reference output is fresh and contiguous)");
      const size_t bytes = (size_t)(hi[i] - lo[i] + 1) * elt;
      st = grow(ctx, ctx->host_stage[i], bytes);
      if (st) return st;
      dv[i].base = ctx->host_stage[i].ptr;
      dv[i].offset = hv[i]->offset - lo[i];
    }
  }
  if (numel[2] == 0) return OXM_OK;

  // Large products are cut along the output's leading dim (batch entries, or
  // rows of a rank-2 product) so that the copy-in of slice i+1, the multiply of
  // slice i and the copy-out of slice i-1 run at the same time on three streams.
  int chunks = 1;
  const int64_t lead = out->shape[0];
  bool row_major = true;
  {
    int64_t expect = 1;
    for (int d = out->ndim - 1; d >= 0; --d) {
      if (out->shape[d] != 1 && out->strides[d] != expect) row_major = false;
      expect *= out->shape[d];
    }
  }
  const int64_t unit = out->ndim == 2 ? 512 : 1;  // rows per slice are kept a multiple of the tile height
  if (row_major && ((size_t)numel[2] * elt >= ((size_t)16 << 20) || ctx->opt_host_chunks > 1) && lead >= 2 * unit &&
      ctx->opt_host_chunks != 1)
    chunks = (int)std::min<int64_t>(ctx->opt_host_chunks > 1 ? ctx->opt_host_chunks : 8, lead / unit);
  if (chunks <= 1) {
    for (int i = 0; i < 2; ++i)
      if (numel[i] > 0)
        CUDA_TRY(cudaMemcpyAsync(dv[i].base, static_cast<const uint8_t *>(hv[i]->base) + lo[i] * elt,
                                 (size_t)(hi[i] - lo[i] + 1) * elt, cudaMemcpyHostToDevice, ctx->stream));
    st = run_matmul(ctx, &dv[0], &dv[1], &dv[2], true);
    if (st) return st;
    CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t *>(out->base) + lo[2] * elt, dv[2].base, (size_t)numel[2] * elt,
                             cudaMemcpyDeviceToHost, ctx->stream));
    std::lock_guard<std::mutex> lock(ctx->mu);
    return check_status(ctx);
  }

  if (!ctx->copy_in) {
    CUDA_TRY(cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking));
    CUDA_TRY(cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking));
    for (auto &e : ctx->pipe_events) CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  }
  cudaEvent_t ev_alloc = ctx->pipe_events[0];
  // Which dim of each operand follows the output's leading dim, and whether its
  // slices are disjoint byte ranges of the host buffer (else it is copied whole).
  int xd[2];
  bool sliced[2];
  for (int i = 0; i < 2; ++i) {
    const oxm_view *v = hv[i];
    xd[i] = out->ndim == 2 ? (i == 0 ? 0 : -1) : (v->ndim == out->ndim && v->shape[0] != 1 ? 0 : -1);
    sliced[i] = xd[i] >= 0 && v->strides[xd[i]] > 0 &&
                (double)v->strides[xd[i]] * (double)v->shape[xd[i]] >= 0.9 * (double)(hi[i] - lo[i] + 1);
  }
  // From here on a failing call must not return past the streams: copies already queued would
  // keep writing the caller's buffers, and the staging buffers could be freed under them.  The
  // first error is kept, no further work is queued, and the common tail below drains all three
  // streams before the error is returned.
  cudaError_t cuda_err = cudaSuccess;
  const char *cuda_what = "";
  auto ok = [&](cudaError_t e, const char *what) {
    if (e != cudaSuccess && cuda_err == cudaSuccess) { cuda_err = e; cuda_what = what; }
    return e == cudaSuccess;
  };
  ok(cudaEventRecord(ev_alloc, ctx->stream), "cudaEventRecord");  // staging buffers exist from here on
  ok(cudaStreamWaitEvent(ctx->copy_in, ev_alloc, 0), "cudaStreamWaitEvent");
  ok(cudaStreamWaitEvent(ctx->copy_out, ev_alloc, 0), "cudaStreamWaitEvent");
  for (int i = 0; i < 2 && cuda_err == cudaSuccess; ++i)
    if (!sliced[i] && numel[i] > 0)
      ok(cudaMemcpyAsync(dv[i].base, static_cast<const uint8_t *>(hv[i]->base) + lo[i] * elt,
                         (size_t)(hi[i] - lo[i] + 1) * elt, cudaMemcpyHostToDevice, ctx->copy_in),
         "copy of an operand to the device");
  const int64_t per = ((lead + chunks - 1) / chunks + unit - 1) / unit * unit;
  int c = 0;
  for (int64_t i0 = 0; i0 < lead && st == OXM_OK && cuda_err == cudaSuccess; i0 += per, ++c) {
    const int64_t len = std::min(per, lead - i0);
    oxm_view cv[3] = {dv[0], dv[1], dv[2]};
    for (int i = 0; i < 2; ++i) {
      if (xd[i] < 0) continue;
      cv[i].shape[xd[i]] = len;
      cv[i].offset += i0 * hv[i]->strides[xd[i]];
      if (sliced[i]) {
        oxm_view hs = *hv[i];
        hs.shape[xd[i]] = len;
        hs.offset += i0 * hv[i]->strides[xd[i]];
        int64_t clo, chi, cn;
        view_extent(&hs, &clo, &chi, &cn);
        if (cn > 0)
          ok(cudaMemcpyAsync(static_cast<uint8_t *>(dv[i].base) + (clo - lo[i]) * elt,
                             static_cast<const uint8_t *>(hv[i]->base) + clo * elt, (size_t)(chi - clo + 1) * elt,
                             cudaMemcpyHostToDevice, ctx->copy_in), "copy of an operand slice to the device");
      }
    }
    if (cuda_err != cudaSuccess) break;
    cv[2].shape[0] = len;
    cv[2].offset += i0 * out->strides[0];
    cudaEvent_t ev_in = ctx->pipe_events[1 + 2 * c], ev_done = ctx->pipe_events[2 + 2 * c];
    if (!ok(cudaEventRecord(ev_in, ctx->copy_in), "cudaEventRecord") ||
        !ok(cudaStreamWaitEvent(ctx->stream, ev_in, 0), "cudaStreamWaitEvent")) break;
    st = run_matmul(ctx, &cv[0], &cv[1], &cv[2], true);
    if (st) break;
    if (!ok(cudaEventRecord(ev_done, ctx->stream), "cudaEventRecord") ||
        !ok(cudaStreamWaitEvent(ctx->copy_out, ev_done, 0), "cudaStreamWaitEvent")) break;
    const int64_t o0 = (out->offset + i0 * out->strides[0]) * elt;
    const int64_t d0 = (dv[2].offset + i0 * out->strides[0]) * elt;
    ok(cudaMemcpyAsync(static_cast<uint8_t *>(out->base) + o0, static_cast<uint8_t *>(dv[2].base) + d0,
                       (size_t)(len * out->strides[0]) * elt, cudaMemcpyDeviceToHost, ctx->copy_out),
       "copy of a result slice to the host");
  }
  const std::string first_detail = g_last_error;  // check_status below may overwrite the message of `st`
  cudaError_t e1 = cudaStreamSynchronize(ctx->copy_in), e2 = cudaStreamSynchronize(ctx->copy_out);
  int st2;
  {
    std::lock_guard<std::mutex> lock(ctx->mu);
    st2 = check_status(ctx);  // drains the compute stream
  }
  if (st) { g_last_error = first_detail; return st; }
  if (cuda_err != cudaSuccess) return fail(OXM_CUDA_ERROR, "host matmul: %s failed: %s", cuda_what, cudaGetErrorString(cuda_err));
  if (e1 != cudaSuccess || e2 != cudaSuccess)
    return fail(OXM_CUDA_ERROR, "host matmul copy failed: %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
  return st2;
}

namespace {
unsigned ew_plan_tiles(const oxm_ctx *ctx, EwParams &p, bool binary, int esz);
void ew_collapse(EwParams &p);
bool ew_linear(const int64_t *shape, const int64_t *strides, int ndim);
}  // namespace

int oxm_contiguous(oxm_ctx *ctx, const oxm_view *src, const oxm_view *dst) {
  if (!ctx || !src || !dst) return fail(OXM_INVALID_ARGUMENT, "contiguous: null argument");
  if (src->ndim < 0 || src->ndim > OXM_MAX_DIMS) return fail(OXM_NOT_IMPLEMENTED, "contiguous is not implemented for rank %d", src->ndim);
  if (src->dtype != dst->dtype)
    return fail(OXM_DTYPE_MISMATCH, "dtype mismatch: expected %s, got %s in contiguous", dtype_name(src->dtype), dtype_name(dst->dtype));
  if (dtype_size(src->dtype) == 0) return fail(OXM_UNSUPPORTED_DTYPE, "dtype %d is not supported by contiguous", src->dtype);
  if (src->device != ctx->device || dst->device != ctx->device)
    return fail(OXM_DEVICE_MISMATCH, "device mismatch: Cuda{index: %d} vs Cuda{index: %d} in contiguous", src->device, dst->device);
  bool same = src->ndim == dst->ndim;
  for (int i = 0; same && i < src->ndim; ++i) same = src->shape[i] == dst->shape[i];
  if (!same) return fail(OXM_SHAPE_MISMATCH, "shape mismatch: expected %s, got %s in contiguous", shape_str(src).c_str(), shape_str(dst).c_str());
  CopyParams p{};
  p.n = 1;
  int64_t expect = 1;
  bool empty = false;
  for (int i = 0; i < src->ndim; ++i) empty = empty || src->shape[i] == 0;
  for (int i = src->ndim - 1; i >= 0; --i) {
    if (!empty && dst->shape[i] != 1 && dst->strides[i] != expect)
      return fail(OXM_INVALID_ARGUMENT, "contiguous: the destination view must be row-major contiguous");
    expect *= dst->shape[i];
    p.n *= src->shape[i];
    p.shape[i] = src->shape[i];
    p.strides[i] = src->strides[i];
  }
  if (p.n == 0) return OXM_OK;
  if (!src->base || !dst->base) return fail(OXM_INVALID_ARGUMENT, "contiguous: view with null storage");
  p.src = src->base; p.dst = dst->base;
  p.elt = dtype_size(src->dtype); p.ndim = src->ndim;
  p.src_off = src->offset; p.dst_off = dst->offset;
  std::lock_guard<std::mutex> lock(ctx->mu);
  CUDA_TRY(cudaSetDevice(ctx->device));
  // a transposed source goes through 32x32 shared-memory tiles so that both sides move whole sectors
  EwParams e{};
  e.ndim = src->ndim; e.n = p.n;
  for (int d = 0; d < src->ndim; ++d) { e.shape[d] = src->shape[d]; e.a_strides[d] = e.b_strides[d] = src->shape[d] != 1 ? src->strides[d] : 0; }
  ew_collapse(e);
  e.contiguous = ew_linear(e.shape, e.a_strides, e.ndim) ? 1 : 0;
  e.a = e.b = src->base; e.a_off = e.b_off = src->offset;
  e.out = static_cast<uint8_t *>(dst->base) + dst->offset * p.elt;
  if (const unsigned tb = ew_plan_tiles(ctx, e, false, p.elt)) {
    switch (p.elt) {
      case 1: ew_tile_kernel<uint8_t, 2, true, false><<<tb, 256, 0, ctx->stream>>>(e); break;
      case 2:
        if (e.quads) ew_reg2_kernel<uint16_t, 2, true, false><<<tb, 256, 0, ctx->stream>>>(e);
        else if (e.pairs) ew_tile2_kernel<uint16_t, 2, true, false><<<tb, 256, 0, ctx->stream>>>(e);
        else ew_tile_kernel<uint16_t, 2, true, false><<<tb, 256, 0, ctx->stream>>>(e);
        break;
      case 4: ew_tile_kernel<uint32_t, 2, true, false><<<tb, 256, 0, ctx->stream>>>(e); break;
      default: ew_tile_kernel<uint64_t, 2, true, false><<<tb, 256, 0, ctx->stream>>>(e); break;
    }
  } else {
    const int64_t blocks = std::min<int64_t>((p.n + 255) / 256, (int64_t)ctx->num_sms * 16);
    copy_strided_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(p);
  }
  CUDA_TRY(cudaGetLastError());
  ctx->launches[0]++; ctx->launches[3]++;
  return OXM_OK;
}

int oxm_fill(oxm_ctx *ctx, void *dst_device, int dtype, int64_t n, uint64_t seed, uint64_t stream, int dist, double scale) {
  if (!ctx || (n > 0 && !dst_device)) return fail(OXM_INVALID_ARGUMENT, "oxm_fill: null argument");
  if (!is_matmul_dtype(dtype)) return fail(OXM_UNSUPPORTED_DTYPE, "dtype %s is not supported by fill", dtype_name(dtype));
  if (dist < 0 || dist > 1 || n < 0) return fail(OXM_INVALID_ARGUMENT, "oxm_fill: bad distribution or count");
  if (n == 0) return OXM_OK;
  const uint64_t key = splitmix64(splitmix64(seed) ^ splitmix64(stream * 0xD1342543DE82EF95ull + 0x632BE59BD9B4E019ull));
  std::lock_guard<std::mutex> lock(ctx->mu);
  CUDA_TRY(cudaSetDevice(ctx->device));
  const int64_t blocks = std::min<int64_t>((n + 255) / 256, (int64_t)ctx->num_sms * 32);
  fill_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(dst_device, dtype, n, key, dist, (float)scale);
  CUDA_TRY(cudaGetLastError());
  return OXM_OK;
}

int oxm_selftest_bounded_wait(oxm_ctx *ctx, int64_t limit_ms) {
  if (!ctx) return fail(OXM_INVALID_ARGUMENT, "oxm_selftest_bounded_wait: null context");
  if (limit_ms < 1 || limit_ms > 1000) return fail(OXM_INVALID_ARGUMENT, "oxm_selftest_bounded_wait: limit must be 1..1000 ms");
  CUDA_TRY(cudaSetDevice(ctx->device));
  uint32_t *flag = nullptr;
  CUDA_TRY(cudaMallocAsync(&flag, sizeof(uint32_t), ctx->stream));
  CUDA_TRY(cudaMemsetAsync(flag, 0xff, sizeof(uint32_t), ctx->stream));
  int st;
  uint32_t gave_up = 0;
  {
    std::lock_guard<std::mutex> lock(ctx->mu);
    snprintf(ctx->last_kernel, sizeof(ctx->last_kernel), "bounded_wait_selftest");
    bounded_wait_selftest_kernel<<<1, 32, 0, ctx->stream>>>(ctx->status_dev, (uint64_t)limit_ms * 1000000ull, flag);
    CUDA_TRY(cudaGetLastError());
    CUDA_TRY(cudaMemcpyAsync(ctx->status_host, flag, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    gave_up = *ctx->status_host;
    st = check_status(ctx);  // reports and clears the status word
  }
  CUDA_TRY(cudaFreeAsync(flag, ctx->stream));
  if (st == OXM_TIMEOUT && gave_up != 1) return fail(OXM_CUDA_ERROR, "bounded wait self-test: status set but the waiter did not give up");
  return st;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// UnaryOps / BinaryOps / ReduceOps
// ---------------------------------------------------------------------------
namespace {

bool is_ew_dtype(int dt) { return dt == OXM_F32 || dt == OXM_F64 || dt == OXM_I32 || dt == OXM_I64 || dt == OXM_BF16 || dt == OXM_F16; }
bool is_float_dtype(int dt) { return dt == OXM_F32 || dt == OXM_F64 || dt == OXM_BF16 || dt == OXM_F16; }

// The output of every operation is fresh and contiguous (ops/lib.rs:16-17).
int check_fresh_output(const oxm_view *out, const int64_t *shape, int ndim, int dtype, const char *op) {
  bool ok = out->ndim == ndim;
  for (int i = 0; ok && i < ndim; ++i) ok = out->shape[i] == shape[i];
  if (!ok) {
    oxm_view exp{};
    exp.ndim = ndim;
    for (int i = 0; i < ndim; ++i) exp.shape[i] = shape[i];
    return fail(OXM_SHAPE_MISMATCH, "shape mismatch: expected %s, got %s in %s (output)", shape_str(&exp).c_str(), shape_str(out).c_str(), op);
  }
  if (out->dtype != dtype)
    return fail(OXM_DTYPE_MISMATCH, "dtype mismatch: expected %s, got %s in %s (output)", dtype_name(dtype), dtype_name(out->dtype), op);
  int64_t expect = 1;
  for (int i = 0; i < ndim; ++i)
    if (out->shape[i] == 0) return OXM_OK;  // an empty tensor is contiguous whatever its strides say
  for (int i = ndim - 1; i >= 0; --i) {
    if (out->shape[i] != 1 && out->strides[i] != expect) return fail(OXM_INVALID_ARGUMENT, "%s: the output view must be row-major contiguous", op);
    expect *= out->shape[i];
  }
  return OXM_OK;
}

template <template <typename> class Launcher, typename... Args>
int dispatch_dtype(int dtype, Args &&...args) {
  switch (dtype) {
    case OXM_F32: return Launcher<float>::run(args...);
    case OXM_F64: return Launcher<double>::run(args...);
    case OXM_I32: return Launcher<int32_t>::run(args...);
    case OXM_I64: return Launcher<int64_t>::run(args...);
    case OXM_BF16: return Launcher<__nv_bfloat16>::run(args...);
    default: return Launcher<__half>::run(args...);
  }
}

template <typename T> struct UnaryLauncher {
  static int run(oxm_ctx *ctx, const EwParams &p, unsigned blocks) {
    if constexpr (sizeof(T) == 2) {
      if (p.tile_r >= 0 && p.quads) {
        ew_reg2_kernel<T, 0, true, false><<<blocks, 256, 0, ctx->stream>>>(p);
        return OXM_OK;
      }
      if (p.tile_r >= 0 && p.pairs) {
        ew_tile2_kernel<T, 0, true, false><<<blocks, 256, 0, ctx->stream>>>(p);
        return OXM_OK;
      }
    }
    if (p.tile_r >= 0) ew_tile_kernel<T, 0, true, false><<<blocks, 256, 0, ctx->stream>>>(p);
    else if (p.rows) ew_rows_kernel<T, false><<<blocks, 256, 0, ctx->stream>>>(p);
    else unary_kernel<T><<<blocks, 256, 0, ctx->stream>>>(p);
    return OXM_OK;
  }
};
template <typename T> struct BinaryLauncher {
  static int run(oxm_ctx *ctx, const EwParams &p, unsigned blocks) {
    if constexpr (sizeof(T) == 2) {
      if (p.tile_r >= 0 && p.quads) {
        if (p.a_turn && p.b_turn) ew_reg2_kernel<T, 1, true, true><<<blocks, 256, 0, ctx->stream>>>(p);
        else if (p.a_turn) ew_reg2_kernel<T, 1, true, false><<<blocks, 256, 0, ctx->stream>>>(p);
        else ew_reg2_kernel<T, 1, false, true><<<blocks, 256, 0, ctx->stream>>>(p);
        return OXM_OK;
      }
    }
    // (the pair-access tile kernel measured no faster than this one for two operands)
    if (p.tile_r >= 0) {
      if (p.a_turn && p.b_turn) ew_tile_kernel<T, 1, true, true><<<blocks, 256, 0, ctx->stream>>>(p);
      else if (p.a_turn) ew_tile_kernel<T, 1, true, false><<<blocks, 256, 0, ctx->stream>>>(p);
      else ew_tile_kernel<T, 1, false, true><<<blocks, 256, 0, ctx->stream>>>(p);
    }
    else if (p.rows) ew_rows_kernel<T, true><<<blocks, 256, 0, ctx->stream>>>(p);
    else binary_kernel<T><<<blocks, 256, 0, ctx->stream>>>(p);
    return OXM_OK;
  }
};

// A transposed operand steps through the innermost dim with a stride other
// than 0 or 1 and has its unit stride on another dim of at least 32 elements.
// Returns that dim, or -1.
int ew_turned_dim(const EwParams &p, const int64_t *st) {
  const int nd = p.ndim - 1;
  if (nd < 1 || st[nd] == 0 || st[nd] == 1) return -1;
  for (int d = 0; d < nd; ++d)
    if (st[d] == 1 && p.shape[d] >= 32) return d;
  return -1;
}

// Tiles apply when some operand is transposed and all transposed operands agree on the dim.
unsigned ew_plan_tiles(const oxm_ctx *ctx, EwParams &p, bool binary, int esz) {
  p.tile_r = -1; p.a_turn = 0; p.b_turn = 0;
  if (p.contiguous || p.ndim < 2 || p.shape[p.ndim - 1] < 8) return 0;
  const int ra = ew_turned_dim(p, p.a_strides), rb = binary ? ew_turned_dim(p, p.b_strides) : -1;
  if (ra < 0 && rb < 0) return 0;
  if (ra >= 0 && rb >= 0 && ra != rb) return 0;
  p.tile_r = ra >= 0 ? ra : rb;
  p.a_turn = ra >= 0; p.b_turn = rb >= 0;
  const int64_t R = p.shape[p.tile_r], C = p.shape[p.ndim - 1];
  const int64_t T = esz >= 8 ? 32 : 64;  // EwTile<T>
  const int64_t tiles = ((R + T - 1) / T) * ((C + T - 1) / T) * (p.n / (R * C));
  if (tiles >= (1ll << 31)) { p.tile_r = -1; return 0; }  // the kernel counts tiles in 32 bits
  // Pairs: 2-byte elements, even tile extents, every row of every operand starting on a 4-byte boundary.
  p.pairs = 0; p.quads = 0;
  if (esz == 2 && R % 2 == 0 && C % 2 == 0 && reinterpret_cast<uintptr_t>(p.out) % 4 == 0) {
    const int nd = p.ndim - 1;
    auto pair_ok = [&](const void *base, int64_t off, const int64_t *st, bool turned) {
      if ((reinterpret_cast<uintptr_t>(base) + off * 2) % 4) return false;
      const int unit = turned ? p.tile_r : nd;
      if (st[unit] != 1) return false;
      for (int d = 0; d <= nd; ++d)
        if (d != unit && st[d] % 2) return false;
      return true;
    };
    p.pairs = (pair_ok(p.a, p.a_off, p.a_strides, p.a_turn) && (!binary || pair_ok(p.b, p.b_off, p.b_strides, p.b_turn))) ? 1 : 0;
    // Quads (the turn in registers): on top of that, the straight operands and the output move 8 bytes
    // along C: C a multiple of 4, their rows 8-byte aligned.
    auto quad_ok = [&](const void *base, int64_t off, const int64_t *st, bool turned) {
      if (turned) return true;  // read in pairs along R: the pair conditions are all it needs
      if ((reinterpret_cast<uintptr_t>(base) + off * 2) % 8) return false;
      for (int d = 0; d < nd; ++d)
        if (st[d] % 4) return false;
      return true;
    };
    p.quads = (p.pairs && C % 4 == 0 && reinterpret_cast<uintptr_t>(p.out) % 8 == 0 && quad_ok(p.a, p.a_off, p.a_strides, p.a_turn) &&
               (!binary || quad_ok(p.b, p.b_off, p.b_strides, p.b_turn))) ? 1 : 0;
  }
  return (unsigned)std::min<int64_t>(tiles, (int64_t)ctx->num_sms * 16);
}

// Decide between the flat kernels, the row kernel and the tile kernel, and whether rows can move 16 bytes at a time.
unsigned ew_plan(const oxm_ctx *ctx, EwParams &p, int esz, bool binary) {
  p.rows = 0; p.rows_vec = 0;
  if (const unsigned tb = ew_plan_tiles(ctx, p, binary, esz)) return tb;
  if (!p.contiguous && p.ndim >= 1 && p.shape[p.ndim - 1] >= 128) {
    const int nd = p.ndim - 1, V = 16 / esz;
    p.rows = 1;
    auto ok = [&](const void *base, int64_t off, const int64_t *st) {
      if (st[nd] != 0 && st[nd] != 1) return false;
      if (st[nd] == 0) return true;  // a per-row scalar needs no alignment
      if ((reinterpret_cast<uintptr_t>(base) + off * esz) % 16) return false;
      for (int d = 0; d < nd; ++d) if (st[d] % V) return false;
      return true;
    };
    p.rows_vec = (p.shape[nd] % V == 0 && reinterpret_cast<uintptr_t>(p.out) % 16 == 0 && ok(p.a, p.a_off, p.a_strides) &&
                  (!binary || ok(p.b, p.b_off, p.b_strides))) ? 1 : 0;
    return (unsigned)std::min<int64_t>(p.n / p.shape[nd], (int64_t)ctx->num_sms * 32);
  }
  return (unsigned)std::min<int64_t>((p.n + 255) / 256, (int64_t)ctx->num_sms * 16);
}
// CTAs of 256 threads of `kernel` that one SM holds at once (asked of the runtime once per kernel).
template <typename K> int resident_ctas(K kernel, std::atomic<int> &cache) {
  int nb = cache.load(std::memory_order_relaxed);
  if (nb > 0) return nb;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kernel, 256, 0) != cudaSuccess || nb < 1) nb = 1;
  cache.store(nb, std::memory_order_relaxed);
  return nb;
}

template <typename T> struct ReduceLauncher {
  // The operation is a template argument of the kernels: chosen per element at run time, both
  // combinations were computed for every element and 2-byte sums ran out of issue slots before
  // they ran out of memory bandwidth.
  // The slices are planned here, from what the chosen kernel really keeps resident: all CTAs of
  // the pass must run at once (a few CTAs over and they run alone in a second pass as long as the
  // first), so the slice count is rounded down.
  template <int OP, typename K>
  static int plan_and_launch(K kernel, std::atomic<int> &cache, oxm_ctx *ctx, ReduceOpParams &p, unsigned blocks_x, int64_t max_splits) {
    const int64_t target = (int64_t)ctx->num_sms * resident_ctas(kernel, cache);
    if (p.warp_rows) {
      // whole rows per warp: as many warps as fit at once, each with the same number of rows
      const int64_t rows_per_warp = (p.n_out + target * 8 - 1) / (target * 8);
      blocks_x = (unsigned)((p.n_out + rows_per_warp * 8 - 1) / (rows_per_warp * 8));
    }
    p.splits = (int32_t)std::max<int64_t>(1, std::min<int64_t>({target / blocks_x, max_splits, (int64_t)1024}));
    p.chunk = (p.n_red + p.splits - 1) / p.splits;
    p.splits = (int32_t)((p.n_red + p.chunk - 1) / p.chunk);
    if (p.splits > 1) {
      const int st = grow(ctx, ctx->pack_ws[2], (size_t)p.splits * p.n_out * 8);
      if (st) return st;
      p.partial = ctx->pack_ws[2].ptr;
    }
    kernel<<<dim3(blocks_x, (unsigned)p.splits, 1), 256, 0, ctx->stream>>>(p);
    if (p.splits > 1) {
      if (p.n_out < 2048 && p.splits >= 32) {
        reduce_finish_wide_kernel<T, OP><<<(unsigned)p.n_out, 256, 0, ctx->stream>>>(p);
      } else {
        const unsigned fb = (unsigned)std::min<int64_t>((p.n_out + 255) / 256, (int64_t)ctx->num_sms * 8);
        reduce_finish_kernel<T, OP><<<fb, 256, 0, ctx->stream>>>(p);
      }
    }
    return OXM_OK;
  }
  template <int OP> static int launch(oxm_ctx *ctx, ReduceOpParams &p, bool row_mode, unsigned blocks_x, int64_t max_splits) {
    static std::atomic<int> occ[4];
    if (row_mode && p.warp_rows) return plan_and_launch<OP>(reduce_roww_kernel<T, OP>, occ[0], ctx, p, blocks_x, max_splits);
    if (row_mode) return plan_and_launch<OP>(reduce_row_kernel<T, OP>, occ[1], ctx, p, blocks_x, max_splits);
    if (p.col_vec) return plan_and_launch<OP>(reduce_colv_kernel<T, OP>, occ[2], ctx, p, blocks_x, max_splits);
    return plan_and_launch<OP>(reduce_col_kernel<T, OP>, occ[3], ctx, p, blocks_x, max_splits);
  }
  static int run(oxm_ctx *ctx, ReduceOpParams &p, bool row_mode, unsigned blocks_x, int64_t max_splits) {
    return p.op == 0 ? launch<0>(ctx, p, row_mode, blocks_x, max_splits) : launch<1>(ctx, p, row_mode, blocks_x, max_splits);
  }
};

// Drop extent-1 dims and merge neighbours that are walked with one stride.
int collapse_dims(int n, int64_t *shape, int64_t *strides) {
  int w = 0;
  for (int d = 0; d < n; ++d) {
    if (shape[d] == 1) continue;
    if (w > 0 && strides[w - 1] == strides[d] * shape[d]) {
      shape[w - 1] *= shape[d];
      strides[w - 1] = strides[d];
    } else {
      shape[w] = shape[d];
      strides[w] = strides[d];
      ++w;
    }
  }
  return w;
}

// Fill the elementwise parameter block for output shape `shape`; operand dims
// are right-aligned against it, extent-1 dims broadcast with stride 0.
void ew_operand(const oxm_view *v, int ndim, int64_t *strides, int64_t *off) {
  *off = v->offset;
  for (int d = 0; d < ndim; ++d) {
    const int vd = d - (ndim - v->ndim);
    strides[d] = (vd >= 0 && v->shape[vd] != 1) ? v->strides[vd] : 0;
  }
}

// Drop extent-1 dims and merge neighbours both operands walk with one stride.
void ew_collapse(EwParams &p) {
  int w = 0;
  for (int d = 0; d < p.ndim; ++d) {
    if (p.shape[d] == 1) continue;
    if (w > 0 && p.a_strides[w - 1] == p.a_strides[d] * p.shape[d] && p.b_strides[w - 1] == p.b_strides[d] * p.shape[d]) {
      p.shape[w - 1] *= p.shape[d];
      p.a_strides[w - 1] = p.a_strides[d];
      p.b_strides[w - 1] = p.b_strides[d];
    } else {
      p.shape[w] = p.shape[d];
      p.a_strides[w] = p.a_strides[d];
      p.b_strides[w] = p.b_strides[d];
      ++w;
    }
  }
  p.ndim = w;
}

bool ew_linear(const int64_t *shape, const int64_t *strides, int ndim) {
  int64_t expect = 1;
  for (int d = ndim - 1; d >= 0; --d) {
    if (shape[d] != 1 && strides[d] != expect) return false;
    expect *= shape[d];
  }
  return true;
}

}  // namespace

extern "C" int oxm_unary(oxm_ctx *ctx, int op, const oxm_view *a, const oxm_view *out) {
  static const char *names[] = {"neg", "exp", "ln", "abs"};
  if (!ctx || !a || !out) return fail(OXM_INVALID_ARGUMENT, "unary: null argument");
  if (op < OXM_NEG || op > OXM_ABS) return fail(OXM_INVALID_ARGUMENT, "unary: unknown operation %d", op);
  const char *name = names[op];
  if (a->ndim < 0 || a->ndim > OXM_MAX_DIMS) return fail(OXM_NOT_IMPLEMENTED, "%s is not implemented for rank %d", name, a->ndim);
  if (!is_ew_dtype(a->dtype) || ((op == OXM_EXP || op == OXM_LN) && !is_float_dtype(a->dtype)))
    return fail(OXM_UNSUPPORTED_DTYPE, "dtype %s is not supported by %s", dtype_name(a->dtype), name);
  if (a->device != ctx->device || out->device != ctx->device)
    return fail(OXM_DEVICE_MISMATCH, "device mismatch: Cuda{index: %d} vs Cuda{index: %d} in %s", a->device, out->device, name);
  int st = check_fresh_output(out, a->shape, a->ndim, a->dtype, name);
  if (st) return st;
  EwParams p{};
  p.op = op; p.ndim = a->ndim; p.n = 1;
  for (int d = 0; d < a->ndim; ++d) { p.shape[d] = a->shape[d]; p.n *= a->shape[d]; }
  if (p.n == 0) return OXM_OK;
  if (!a->base || !out->base) return fail(OXM_INVALID_ARGUMENT, "%s: view with null storage", name);
  ew_operand(a, a->ndim, p.a_strides, &p.a_off);
  for (int d = 0; d < p.ndim; ++d) p.b_strides[d] = p.a_strides[d];
  ew_collapse(p);
  p.contiguous = ew_linear(p.shape, p.a_strides, p.ndim) ? 1 : 0;
  p.a = a->base; p.b = a->base;
  p.out = static_cast<uint8_t *>(out->base) + out->offset * dtype_size(out->dtype);
  const int esz = dtype_size(a->dtype);
  p.vec = (p.contiguous && (reinterpret_cast<uintptr_t>(p.a) + p.a_off * esz) % 16 == 0 && reinterpret_cast<uintptr_t>(p.out) % 16 == 0) ? 1 : 0;
  std::lock_guard<std::mutex> lock(ctx->mu);
  CUDA_TRY(cudaSetDevice(ctx->device));
  const unsigned blocks = ew_plan(ctx, p, esz, false);
  dispatch_dtype<UnaryLauncher>(a->dtype, ctx, p, blocks);
  CUDA_TRY(cudaGetLastError());
  ctx->launches[0]++;
  snprintf(ctx->last_kernel, sizeof(ctx->last_kernel), "unary_%s", name);
  return OXM_OK;
}

extern "C" int oxm_binary(oxm_ctx *ctx, int op, const oxm_view *a, const oxm_view *b, const oxm_view *out) {
  static const char *names[] = {"add", "sub", "mul", "div"};
  if (!ctx || !a || !b || !out) return fail(OXM_INVALID_ARGUMENT, "binary: null argument");
  if (op < OXM_ADD || op > OXM_DIV) return fail(OXM_INVALID_ARGUMENT, "binary: unknown operation %d", op);
  const char *name = names[op];
  for (const oxm_view *v : {a, b})
    if (v->ndim < 0 || v->ndim > OXM_MAX_DIMS) return fail(OXM_NOT_IMPLEMENTED, "%s is not implemented for rank %d", name, v->ndim);
  if (a->device != b->device)
    return fail(OXM_DEVICE_MISMATCH, "device mismatch: Cuda{index: %d} vs Cuda{index: %d} in %s", a->device, b->device, name);
  if (a->device != ctx->device || out->device != ctx->device)
    return fail(OXM_DEVICE_MISMATCH, "device mismatch: Cuda{index: %d} vs Cuda{index: %d} in %s", a->device, out->device, name);
  if (a->dtype != b->dtype)
    return fail(OXM_DTYPE_MISMATCH, "dtype mismatch: expected %s, got %s in %s", dtype_name(a->dtype), dtype_name(b->dtype), name);
  if (!is_ew_dtype(a->dtype))
    return fail(OXM_UNSUPPORTED_DTYPE, "dtype %s is not supported by %s", dtype_name(a->dtype), name);
  // NumPy broadcasting (shape.rs:49-55)
  int nd = std::max(a->ndim, b->ndim);
  int64_t shape[OXM_MAX_DIMS];
  for (int i = 0; i < nd; ++i) {
    const int ai = a->ndim - 1 - i, bi = b->ndim - 1 - i;
    const int64_t l = ai >= 0 ? a->shape[ai] : 1, r = bi >= 0 ? b->shape[bi] : 1;
    if (l != r && l != 1 && r != 1)
      return fail(OXM_BROADCAST_INCOMPATIBLE, "cannot broadcast %s with %s", shape_str(a).c_str(), shape_str(b).c_str());
    shape[nd - 1 - i] = l == 1 ? r : l;
  }
  int st = check_fresh_output(out, shape, nd, a->dtype, name);
  if (st) return st;
  EwParams p{};
  p.op = op; p.ndim = nd; p.n = 1;
  for (int d = 0; d < nd; ++d) { p.shape[d] = shape[d]; p.n *= shape[d]; }
  if (p.n == 0) return OXM_OK;
  if (!a->base || !b->base || !out->base) return fail(OXM_INVALID_ARGUMENT, "%s: view with null storage", name);
  ew_operand(a, nd, p.a_strides, &p.a_off);
  ew_operand(b, nd, p.b_strides, &p.b_off);
  ew_collapse(p);
  nd = p.ndim;
  p.contiguous = (ew_linear(p.shape, p.a_strides, nd) && ew_linear(p.shape, p.b_strides, nd)) ? 1 : 0;
  p.a = a->base; p.b = b->base;
  p.out = static_cast<uint8_t *>(out->base) + out->offset * dtype_size(out->dtype);
  const int esz = dtype_size(a->dtype);
  p.vec = (p.contiguous && (reinterpret_cast<uintptr_t>(p.a) + p.a_off * esz) % 16 == 0 &&
           (reinterpret_cast<uintptr_t>(p.b) + p.b_off * esz) % 16 == 0 && reinterpret_cast<uintptr_t>(p.out) % 16 == 0) ? 1 : 0;
  std::lock_guard<std::mutex> lock(ctx->mu);
  CUDA_TRY(cudaSetDevice(ctx->device));
  if (op == OXM_DIV && !is_float_dtype(a->dtype)) {
    // Integer division reports a zero divisor as a typed error, so it is the one compute call
    // that waits for its kernel: the status word is read back before returning.
    const unsigned blocks = (unsigned)std::min<int64_t>((p.n + 255) / 256, (int64_t)ctx->num_sms * 16);
    if (a->dtype == OXM_I32) int_div_kernel<int32_t><<<blocks, 256, 0, ctx->stream>>>(p, ctx->status_dev);
    else int_div_kernel<int64_t><<<blocks, 256, 0, ctx->stream>>>(p, ctx->status_dev);
    CUDA_TRY(cudaGetLastError());
    ctx->launches[0]++;
    snprintf(ctx->last_kernel, sizeof(ctx->last_kernel), "binary_%s", name);
    return check_status(ctx);
  }
  const unsigned blocks = ew_plan(ctx, p, esz, true);
  dispatch_dtype<BinaryLauncher>(a->dtype, ctx, p, blocks);
  CUDA_TRY(cudaGetLastError());
  ctx->launches[0]++;
  snprintf(ctx->last_kernel, sizeof(ctx->last_kernel), "binary_%s", name);
  return OXM_OK;
}

extern "C" int oxm_reduce(oxm_ctx *ctx, int op, const oxm_view *a, const int32_t *axes, int naxes, const oxm_view *out) {
  static const char *names[] = {"sum", "max"};
  if (!ctx || !a || !out || (naxes > 0 && !axes)) return fail(OXM_INVALID_ARGUMENT, "reduce: null argument");
  if (op < OXM_SUM || op > OXM_MAX) return fail(OXM_INVALID_ARGUMENT, "reduce: unknown operation %d", op);
  const char *name = names[op];
  if (a->ndim < 0 || a->ndim > OXM_MAX_DIMS) return fail(OXM_NOT_IMPLEMENTED, "%s is not implemented for rank %d", name, a->ndim);
  if (!is_ew_dtype(a->dtype)) return fail(OXM_UNSUPPORTED_DTYPE, "dtype %s is not supported by %s", dtype_name(a->dtype), name);
  if (a->device != ctx->device || out->device != ctx->device)
    return fail(OXM_DEVICE_MISMATCH, "device mismatch: Cuda{index: %d} vs Cuda{index: %d} in %s", a->device, out->device, name);
  bool reduced[OXM_MAX_DIMS] = {};
  if (naxes == 0) {
    for (int d = 0; d < a->ndim; ++d) reduced[d] = true;  // empty axes means all axes
  } else {
    for (int i = 0; i < naxes; ++i) {
      if (axes[i] < 0 || axes[i] >= a->ndim || reduced[axes[i]])
        return fail(OXM_INDEX_OUT_OF_BOUNDS, "index [%d] out of bounds for shape %s (axes of %s)", axes[i], shape_str(a).c_str(), name);
      reduced[axes[i]] = true;
    }
  }
  ReduceOpParams p{};
  p.op = op; p.n_out = 1; p.n_red = 1; p.a_off = a->offset; p.splits = 1;
  int64_t oshape[OXM_MAX_DIMS];
  int nk_full = 0;
  for (int d = 0; d < a->ndim; ++d) {
    if (reduced[d]) {
      p.red_shape[p.nred] = a->shape[d]; p.red_strides[p.nred] = a->strides[d]; p.nred++;
      p.n_red *= a->shape[d];
    } else {
      oshape[nk_full++] = a->shape[d];
      p.kept_shape[p.nkept] = a->shape[d]; p.kept_strides[p.nkept] = a->strides[d]; p.nkept++;
      p.n_out *= a->shape[d];
    }
  }
  int st = check_fresh_output(out, oshape, nk_full, a->dtype, name);
  if (st) return st;
  if (p.n_out == 0) return OXM_OK;
  if (p.n_red == 0 && op == OXM_MAX)
    return fail(OXM_NOT_IMPLEMENTED, "max is not implemented for an empty reduction extent of %s (there is no identity to invent)", shape_str(a).c_str());
  if (!out->base || (p.n_red > 0 && !a->base)) return fail(OXM_INVALID_ARGUMENT, "%s: view with null storage", name);
  p.a = a->base;
  p.out = static_cast<uint8_t *>(out->base) + out->offset * dtype_size(out->dtype);
  std::lock_guard<std::mutex> lock(ctx->mu);
  CUDA_TRY(cudaSetDevice(ctx->device));
  if (p.n_red == 0) {  // an empty sum is zero
    CUDA_TRY(cudaMemsetAsync(p.out, 0, (size_t)p.n_out * dtype_size(a->dtype), ctx->stream));
    return OXM_OK;
  }
  p.nkept = collapse_dims(p.nkept, p.kept_shape, p.kept_strides);
  p.nred = collapse_dims(p.nred, p.red_shape, p.red_strides);
  // Threads follow whichever group owns the smallest stride, so that a warp's loads are adjacent.
  auto min_stride = [](int n, const int64_t *st) {
    int64_t m = INT64_MAX;
    for (int d = 0; d < n; ++d) m = std::min<int64_t>(m, st[d] < 0 ? -st[d] : st[d]);
    return m;
  };
  const bool row_mode = p.nkept == 0 || min_stride(p.nred, p.red_strides) < min_stride(p.nkept, p.kept_strides);
  unsigned blocks_x;
  int64_t max_splits;
  p.warp_rows = 0;
  if (row_mode && p.nred == 1 && p.red_strides[0] == 1 && p.n_red * dtype_size(a->dtype) <= (48 << 10) &&
      p.n_out >= (int64_t)ctx->num_sms * 64) {
    // many short contiguous rows (under 48 KiB: longer ones keep a CTA busy on their own): a warp per
    // row, eight rows per CTA, no slices
    p.warp_rows = 1;
    blocks_x = (unsigned)std::min<int64_t>((p.n_out + 7) / 8, (int64_t)ctx->num_sms * 16);
    max_splits = 1;
  } else if (row_mode) {
    blocks_x = (unsigned)std::min<int64_t>(p.n_out, 65535 * 16);
    max_splits = (p.n_red + 8191) / 8192;    // at least 8 Ki elements per slice
  } else {
    // one contiguous run of kept elements, everything 16-byte aligned: 16 bytes of outputs per thread
    const int esz = dtype_size(a->dtype), V = 16 / esz;
    bool vec = p.nkept == 1 && p.kept_strides[0] == 1 && p.n_out % V == 0 &&
               (reinterpret_cast<uintptr_t>(p.a) + p.a_off * esz) % 16 == 0 && reinterpret_cast<uintptr_t>(p.out) % 16 == 0;
    for (int d = 0; vec && d < p.nred; ++d) vec = p.red_strides[d] % V == 0;
    p.col_vec = vec ? 1 : 0;
    const int64_t threads = vec ? p.n_out / V : p.n_out;
    blocks_x = (unsigned)std::min<int64_t>((threads + 255) / 256, (int64_t)ctx->num_sms * 16);
    max_splits = (p.n_red + 63) / 64;        // at least 64 serial steps per thread
  }
  st = dispatch_dtype<ReduceLauncher>(a->dtype, ctx, p, row_mode, blocks_x, max_splits);  // plans the slices, launches
  if (st) return st;
  CUDA_TRY(cudaGetLastError());
  ctx->launches[0] += p.splits > 1 ? 2 : 1;
  snprintf(ctx->last_kernel, sizeof(ctx->last_kernel), "reduce_%s_%s_x%d", name, !row_mode ? "col" : p.warp_rows ? "roww" : "row", p.splits);
  return OXM_OK;
}

extern "C" {

int oxm_event_create(oxm_ctx *ctx, oxm_event **out) {
  if (!ctx || !out) return fail(OXM_INVALID_ARGUMENT, "oxm_event_create: null argument");
  CUDA_TRY(cudaSetDevice(ctx->device));
  oxm_event *e = new oxm_event();
  e->device = ctx->device;
  cudaError_t r = cudaEventCreate(&e->ev);
  if (r != cudaSuccess) {
    delete e;
    return fail(OXM_CUDA_ERROR, "cudaEventCreate failed: %s", cudaGetErrorString(r));
  }
  *out = e;
  return OXM_OK;
}

int oxm_event_destroy(oxm_event *ev) {
  if (!ev) return OXM_OK;
  cudaSetDevice(ev->device);
  cudaEventDestroy(ev->ev);
  delete ev;
  return OXM_OK;
}

int oxm_event_record(oxm_ctx *ctx, oxm_event *ev) {
  if (!ctx || !ev) return fail(OXM_INVALID_ARGUMENT, "oxm_event_record: null argument");
  CUDA_TRY(cudaSetDevice(ctx->device));
  CUDA_TRY(cudaEventRecord(ev->ev, ctx->stream));
  return OXM_OK;
}

int oxm_event_elapsed_ms(oxm_event *start, oxm_event *stop, float *ms) {
  if (!start || !stop || !ms) return fail(OXM_INVALID_ARGUMENT, "oxm_event_elapsed_ms: null argument");
  CUDA_TRY(cudaSetDevice(stop->device));
  CUDA_TRY(cudaEventSynchronize(stop->ev));
  CUDA_TRY(cudaEventElapsedTime(ms, start->ev, stop->ev));
  return OXM_OK;
}

int oxm_stream_handle(oxm_ctx *ctx, void **cuda_stream) {
  if (!ctx || !cuda_stream) return fail(OXM_INVALID_ARGUMENT, "oxm_stream_handle: null argument");
  *cuda_stream = ctx->stream;
  return OXM_OK;
}

int oxm_set_option(oxm_ctx *ctx, const char *key, int64_t value) {
  if (!ctx || !key) return fail(OXM_INVALID_ARGUMENT, "oxm_set_option: null argument");
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (!strcmp(key, "kernel") && value >= 0 && value <= 2) ctx->opt_kernel = value;
  else if (!strcmp(key, "tile_n") && (value == 0 || (value >= 64 && value <= 512 && value % 32 == 0))) ctx->opt_tile_n = value;
  else if (!strcmp(key, "cta_pair") && value >= -1 && value <= 1) ctx->opt_cta_pair = value;
  else if (!strcmp(key, "wait_limit_ms") && value >= 1 && value <= 600000) ctx->opt_wait_limit_ms = value;
  else if (!strcmp(key, "group_m") && value >= 0 && value <= 1024) ctx->opt_group_m = value;
  else if (!strcmp(key, "stream_k") && value >= -1 && value <= 1) ctx->opt_stream_k = value;
  else if (!strcmp(key, "tma_store") && (value == 0 || value == 1)) ctx->opt_tma_store = value;
  else if (!strcmp(key, "split_k") && value >= -1 && value <= 64) ctx->opt_split_k = value;
  else if (!strcmp(key, "host_chunks") && value >= 0 && value <= 16) ctx->opt_host_chunks = value;
  else if (!strcmp(key, "simt_tile") && (value == 0 || value == 32 || value == 64)) ctx->opt_simt_tile = value;
  else return fail(OXM_INVALID_ARGUMENT, "oxm_set_option: unknown option or value: %s = %lld", key, (long long)value);
  return OXM_OK;
}

int oxm_get_option(oxm_ctx *ctx, const char *key, int64_t *value) {
  if (!ctx || !key || !value) return fail(OXM_INVALID_ARGUMENT, "oxm_get_option: null argument");
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (!strcmp(key, "kernel")) *value = ctx->opt_kernel;
  else if (!strcmp(key, "tile_n")) *value = ctx->opt_tile_n;
  else if (!strcmp(key, "cta_pair")) *value = ctx->opt_cta_pair;
  else if (!strcmp(key, "wait_limit_ms")) *value = ctx->opt_wait_limit_ms;
  else if (!strcmp(key, "group_m")) *value = ctx->opt_group_m;
  else if (!strcmp(key, "stream_k")) *value = ctx->opt_stream_k;
  else if (!strcmp(key, "tma_store")) *value = ctx->opt_tma_store;
  else if (!strcmp(key, "split_k")) *value = ctx->opt_split_k;
  else if (!strcmp(key, "host_chunks")) *value = ctx->opt_host_chunks;
  else if (!strcmp(key, "simt_tile")) *value = ctx->opt_simt_tile;
  else return fail(OXM_INVALID_ARGUMENT, "oxm_get_option: unknown option: %s", key);
  return OXM_OK;
}

int oxm_launch_counts(oxm_ctx *ctx, int64_t counts[4]) {
  if (!ctx || !counts) return fail(OXM_INVALID_ARGUMENT, "oxm_launch_counts: null argument");
  std::lock_guard<std::mutex> lock(ctx->mu);
  for (int i = 0; i < 4; ++i) counts[i] = ctx->launches[i];
  return OXM_OK;
}

const char *oxm_last_kernel(oxm_ctx *ctx) { return ctx ? ctx->last_kernel : "none"; }

int oxm_memory_stats(oxm_ctx *ctx, int64_t stats[4]) {
  if (!ctx || !stats) return fail(OXM_INVALID_ARGUMENT, "oxm_memory_stats: null argument");
  CUDA_TRY(cudaSetDevice(ctx->device));
  cudaMemPool_t pool;
  CUDA_TRY(cudaDeviceGetDefaultMemPool(&pool, ctx->device));
  uint64_t reserved = 0, used = 0;
  CUDA_TRY(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemCurrent, &reserved));
  CUDA_TRY(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemCurrent, &used));
  size_t free_b = 0, total_b = 0;
  CUDA_TRY(cudaMemGetInfo(&free_b, &total_b));
  stats[0] = (int64_t)reserved; stats[1] = (int64_t)used; stats[2] = (int64_t)free_b; stats[3] = (int64_t)total_b;
  return OXM_OK;
}

}  // extern "C"

// ===========================================================================
// Allocation-free f32 matmul
//
// Some hosts of this library must not allocate device memory once they are
// running: a server or training loop that handed all of HBM to its own arena
// at start-up, or a latency-critical loop that cannot afford the device-wide
// synchronisation and the failure modes of an allocator call in mid-flight.
// For them the packed TF32 operands and split-K partial sums of the f32
// tensor-core path live in a fixed array that is part of the loaded module.
// ===========================================================================
namespace {

constexpr size_t kNoAllocScratchBytes = OXM_NOALLOC_SCRATCH_BYTES;

// Every GPU that loads this library holds these 32 MiB until the process ends.
// In host code this name is only a handle for cudaGetSymbolAddress, never an
// address a kernel may be given.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

std::mutex g_noalloc_mu;
void *g_noalloc_ptr[64] = {};  // device address of the array, per CUDA device

// Resolve the array's device address once per device, with that device current.
int noalloc_scratch(int device, unsigned char **out) {
  if (device < 0 || device >= 64) return fail(OXM_INVALID_ARGUMENT, "matmul_f32_noalloc: device index %d out of range", device);
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (!g_noalloc_ptr[device]) {
    CUDA_TRY(cudaSetDevice(device));
    void *ptr = nullptr;
    CUDA_TRY(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    if (!ptr) return fail(OXM_CUDA_ERROR, "matmul_f32_noalloc: cudaGetSymbolAddress returned a null address");
    g_noalloc_ptr[device] = ptr;
  }
  *out = static_cast<unsigned char *>(g_noalloc_ptr[device]);
  return OXM_OK;
}

size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

// The pack step of the f32 path, writing to a caller-chosen address.
int pack_f32_into(oxm_ctx *ctx, const Problem &P, bool is_b, void *dst, int64_t Kp, Staged &s) {
  const int64_t rows = is_b ? P.N : P.M;
  PackParams pp{};
  pp.src = is_b ? P.b : P.a;
  pp.dst = dst;
  pp.elt = 4;
  pp.mode = is_b ? 2 : 1;
  pp.rows = (int32_t)rows; pp.K = (int32_t)P.K; pp.Kp = (int32_t)Kp;
  pp.dst_row_elems = 3 * Kp;
  pp.src_off = is_b ? P.b_off : P.a_off;
  pp.src_rs = is_b ? P.b_rs : P.a_rs;
  pp.src_ks = is_b ? P.b_ks : P.a_ks;
  pp.nbd = 0;
  pp.tiles_r = (int32_t)((rows + 31) / 32);
  pp.tiles_k = (int32_t)(Kp / 32);
  const int64_t blocks = (int64_t)pp.tiles_r * pp.tiles_k;
  pack_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(pp);
  CUDA_TRY(cudaGetLastError());
  ctx->launches[0]++; ctx->launches[3]++;
  s = Staged{};
  s.ptr = dst;
  s.mn_major = false;
  s.rows = rows; s.K = 3 * Kp;
  s.ld_bytes = 3 * Kp * 4;
  s.nb = 1;
  s.bs_bytes = rows * 3 * Kp * 4;
  return OXM_OK;
}

}  // namespace

extern "C" int oxm_matmul_f32_noalloc(oxm_ctx *ctx, const oxm_view *a, const oxm_view *b, const oxm_view *out) {
  int st = validate(ctx, a, b, out, false, false);
  if (st) return st;
  if (a->dtype != OXM_F32)
    return fail(OXM_UNSUPPORTED_DTYPE, "dtype %s is not supported by matmul_f32_noalloc (f32 only)", dtype_name(a->dtype));
  for (const oxm_view *v : {a, b, out}) {
    if (v->shape[0] * v->shape[1] > 0 && v->base == nullptr) return fail(OXM_INVALID_ARGUMENT, "matmul_f32_noalloc: view with null storage");
  }
  const Problem P = normalise(a, b, out);
  if (P.M == 0 || P.N == 0) return OXM_OK;
  if (P.M >= (1ll << 31) || P.N >= (1ll << 31) || P.K >= (1ll << 29))
    return fail(OXM_NOT_IMPLEMENTED, "matmul_f32_noalloc is not implemented for extents above 2^31");

  // Scratch plan: [packed A | packed B | split-K partial sums], each 256-byte aligned.
  const int64_t Kp = (P.K + 31) / 32 * 32;
  const int32_t num_kb = (int32_t)(3 * Kp / 32);
  int32_t splits = 1, kb_per_split = num_kb;
  if (num_kb > kMaxChainKb) {
    splits = (num_kb + kMaxChainKb - 1) / kMaxChainKb;
    kb_per_split = (num_kb + splits - 1) / splits;
    splits = (num_kb + kb_per_split - 1) / kb_per_split;
  }
  const size_t a_bytes = align256((size_t)P.M * 3 * Kp * 4);
  const size_t b_bytes = align256((size_t)P.N * 3 * Kp * 4);
  const size_t part_bytes = splits > 1 ? align256((size_t)splits * P.M * P.N * 4) : 0;
  const size_t need = a_bytes + b_bytes + part_bytes;
  if (need > kNoAllocScratchBytes)
    return fail(OXM_NOT_IMPLEMENTED,
                "matmul_f32_noalloc is not implemented for [%lld, %lld] x [%lld, %lld]: it needs %zu bytes of scratch "
                "(packed operands%s) and the static scratch holds %zu; use oxm_matmul",
                (long long)P.M, (long long)P.K, (long long)P.K, (long long)P.N, need,
                splits > 1 ? " and split-K partial sums" : "", kNoAllocScratchBytes);

  std::lock_guard<std::mutex> lock(ctx->mu);
  CUDA_TRY(cudaSetDevice(ctx->device));
  if (P.K == 0) return launch_simt(ctx, P);  // an empty contraction: zeros, no scratch involved
  unsigned char *scratch = nullptr;
  st = noalloc_scratch(ctx->device, &scratch);
  if (st) return st;

  // The pack kernel rewrites every scratch element the GEMM will read, zero
  // padding included, and the GEMM writes every partial sum the reduction
  // reads: nothing left over from an earlier call is ever consumed, so no
  // clearing pass is needed.
  Staged sa{}, sb{};
  st = pack_f32_into(ctx, P, false, scratch, Kp, sa);
  if (st) return st;
  st = pack_f32_into(ctx, P, true, scratch + a_bytes, Kp, sb);
  if (st) return st;

  const int bn = P.N > 128 ? 256 : (P.N > 64 ? 128 : 64);
  const int pair = (bn == 256 && P.M > kTileM) ? 1 : 0;
  const int tm = kTileM * (pair ? 2 : 1);
  GemmParams p{};
  p.M = (int32_t)P.M; p.N = (int32_t)P.N; p.K = (int32_t)(3 * Kp);
  p.bn = bn; p.subn = bn;
  p.tiles_m = (int32_t)((P.M + tm - 1) / tm);
  p.tiles_n = (int32_t)((P.N + bn - 1) / bn);
  p.num_kb = num_kb;
  p.nbatch = 1;
  p.num_tiles = (int64_t)p.tiles_m * p.tiles_n;
  p.nbd = 0;
  p.out_dtype = OXM_F32;
  p.idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(tm >> 4) << 24);
  p.status = ctx->status_dev;
  p.wait_limit_ns = (uint64_t)ctx->opt_wait_limit_ms * 1000000ull;
  p.splits = splits;
  p.kb_per_split = kb_per_split;
  p.tiles_per_split = p.num_tiles;
  p.group_m = pair ? 8 : 16;
  ReduceParams rp{};
  if (splits > 1) {
    float *partials = reinterpret_cast<float *>(scratch + a_bytes + b_bytes);
    p.out = partials;
    p.out_rs = P.N; p.out_cs = 1;
    p.out_vec = (P.N % 4 == 0) ? 1 : 0;
    p.split_ostride = P.M * P.N;
    p.num_tiles *= splits;
    rp.ws = partials;
    rp.out = P.o;
    rp.out_dtype = OXM_F32;
    rp.splits = splits; rp.M = p.M; rp.N = p.N;
    rp.split_stride = P.M * P.N; rp.total = P.M * P.N;
    rp.o_off = P.o_off; rp.o_rs = P.o_rs; rp.o_cs = P.o_cs;
    rp.nbd = 0;
  } else {
    p.out = static_cast<uint8_t *>(P.o) + P.o_off * 4;
    p.out_rs = P.o_rs; p.out_cs = P.o_cs;
    p.out_vec = (P.o_cs == 1 && (reinterpret_cast<uintptr_t>(p.out) % 16) == 0 && (P.o_rs * 4) % 16 == 0) ? 1 : 0;
    p.split_ostride = 0;
  }
  CUtensorMap tmA, tmB, tmC;
  memset(&tmC, 0, sizeof(tmC));
  p.out_tma = 0;  // plain strided stores: the output may be any view
  p.dp_tiles = p.num_tiles;  // whole tiles only: stream-K would need a workspace
  p.sk_tiles = 0;
  p.stage_tx = (uint32_t)(kStageKBytes * (kTileM + (pair ? bn / 2 : bn)));  // per CTA
  st = make_map(ctx, &tmA, sa, OXM_F32, 4, kTileM, 32);
  if (st) return st;
  st = make_map(ctx, &tmB, sb, OXM_F32, 4, pair ? bn / 2 : bn, 32);
  if (st) return st;
  const int grid = pair ? 2 * (int)std::min<int64_t>(p.num_tiles, ctx->num_sms / 2)
                        : (int)std::min<int64_t>(p.num_tiles, ctx->num_sms);
  st = launch_gemm(ctx, 1, false, false, bn, pair, tmA, tmB, tmC, p, grid);
  if (st) return st;
  ctx->launches[0]++; ctx->launches[1]++;
  if (splits > 1) {
    const int64_t blocks = std::min<int64_t>((rp.total + 255) / 256, (int64_t)ctx->num_sms * 16);
    splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(rp);
    CUDA_TRY(cudaGetLastError());
    ctx->launches[0]++; ctx->launches[3]++;
  }
  return OXM_OK;
}
