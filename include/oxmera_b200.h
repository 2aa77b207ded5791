/*
 * oxmera_b200 — C ABI of the B200 (sm_100a) matmul backend for oxmera.
 *
 * This is the boundary a Rust `oxmera-b200` backend crate binds with
 * `extern "C"` (build.rs drives nvcc).  Every entry point names the item of
 * the oxmera reference it stands behind.  Plain pointers and sizes only; no
 * exceptions, aborts or C++ types cross this boundary.  All functions return
 * an oxm_status; OXM_OK is 0.
 *
 * Threading: every function may be called concurrently from any host thread
 * (oxmera's `Backend: Send + Sync`, crates/oxmera-runtime/src/lib.rs:29).
 * Work submitted through one context runs in submission order on that
 * context's stream.  Compute calls are asynchronous; device-side failures
 * surface from oxm_sync / oxm_d2h.
 */
#ifndef OXMERA_B200_H
#define OXMERA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OXM_MAX_DIMS 8

/* Element types.  0..5 are oxmera's DType in declaration order
 * (crates/oxmera-core/src/dtype.rs:9-22); BF16/F16 are the two variants the
 * backend adds to that non_exhaustive enum. */
typedef enum {
  OXM_F32 = 0, OXM_F64 = 1, OXM_I32 = 2, OXM_I64 = 3, OXM_U8 = 4, OXM_BOOL = 5,
  OXM_BF16 = 6, OXM_F16 = 7,
  OXM_F8E4M3 = 8, /* 1-4-3, finite only, max 448 (the "fn" encoding) */
  OXM_F8E5M2 = 9  /* 1-5-2, IEEE-like */
} oxm_dtype;

/* Status codes.  1..9 map one-to-one onto the variants of oxmera's Error
 * (crates/oxmera-core/src/error.rs:12-102) in declaration order; the rest are
 * backend conditions the Rust side folds into NotImplemented / a backend
 * error string obtained from oxm_last_error. */
typedef enum {
  OXM_OK = 0,
  OXM_SHAPE_MISMATCH = 1,
  OXM_BROADCAST_INCOMPATIBLE = 2,
  OXM_DTYPE_MISMATCH = 3,
  OXM_UNSUPPORTED_DTYPE = 4,
  OXM_DEVICE_MISMATCH = 5,
  OXM_INDEX_OUT_OF_BOUNDS = 6,
  OXM_RANK_MISMATCH = 7,
  OXM_BACKEND_UNAVAILABLE = 8,
  OXM_NOT_IMPLEMENTED = 9,
  OXM_CUDA_ERROR = 10,      /* a CUDA runtime / driver call failed */
  OXM_TIMEOUT = 11,         /* a bounded device-side wait expired */
  OXM_INVALID_ARGUMENT = 12, /* null pointer, bad handle, bad option */
  OXM_DIVIDE_BY_ZERO = 13    /* integer division met a zero divisor (BinaryOps::div,
                              * crates/oxmera-ops/src/lib.rs:47-49: "Integer division by zero
                              * is a typed error"); oxmera's Error is non_exhaustive and has
                              * no variant for it yet, so the Rust side adds one */
} oxm_status;

/* A tensor as the backend sees it: oxmera's Layout {shape, strides, offset}
 * (crates/oxmera-core/src/layout.rs:26-34; strides are signed ELEMENT strides,
 * offset is in elements) plus the device pointer and device index of the
 * Storage behind it (crates/oxmera-tensor/src/storage.rs:12-17). */
typedef struct {
  int32_t dtype;                 /* oxm_dtype */
  int32_t ndim;                  /* 0..OXM_MAX_DIMS */
  int64_t shape[OXM_MAX_DIMS];
  int64_t strides[OXM_MAX_DIMS];
  int64_t offset;
  void *base;                    /* device pointer to element 0 of the storage */
  int32_t device;                /* CUDA device index (Device::Cuda{index}) */
  int32_t reserved;
} oxm_view;

typedef struct oxm_ctx oxm_ctx;
typedef struct oxm_event oxm_event;

/* ---- backend identity and lifetime ------------------------------------
 * One context per Device::Cuda{index}; stands behind `Backend::device()` and
 * `Backend::name()` (crates/oxmera-runtime/src/lib.rs:29-34).  Creation fails
 * with OXM_BACKEND_UNAVAILABLE when no sm_100 device with that index exists
 * (crates/oxmera-runtime/src/lib.rs:36-44: "never a panic"). */
int oxm_device_count(int *count);
int oxm_ctx_create(int device_index, oxm_ctx **out);
int oxm_ctx_destroy(oxm_ctx *ctx);
int oxm_ctx_device(const oxm_ctx *ctx, int *device_index);
const char *oxm_backend_name(void); /* "b200-tcgen05" */

/* Human-readable detail of the last non-OK status returned to this thread. */
const char *oxm_last_error(void);
/* Stable name of a status code ("ShapeMismatch", ...). */
const char *oxm_status_name(int status);

/* ---- storage ------------------------------------------------------------
 * Stand behind the device variant of StorageData
 * (crates/oxmera-tensor/src/storage.rs:24-32) and the host<->device
 * constructors a device tensor needs in place of from_vec_f32 / get_f32
 * (crates/oxmera-tensor/src/tensor.rs:33,96).  Allocation is stream-ordered
 * and pooled.  Copies are ordered on the context's stream; oxm_d2h returns
 * after the bytes have landed and reports any pending device-side failure. */
int oxm_alloc(oxm_ctx *ctx, size_t bytes, void **out);
int oxm_free(oxm_ctx *ctx, void *ptr);
int oxm_h2d(oxm_ctx *ctx, void *dst_device, const void *src_host, size_t bytes);
int oxm_d2h(oxm_ctx *ctx, void *dst_host, const void *src_device, size_t bytes);
int oxm_memset(oxm_ctx *ctx, void *dst_device, int byte, size_t bytes);
/* Copy between two GPUs of one box: `bytes` from `src_device` (memory of
 * src_ctx's device) into `dst_device` (memory of dst_ctx's device), ordered on
 * dst_ctx's stream after everything submitted to src_ctx so far.  This is how a
 * replicated operand reaches the other GPUs without crossing PCIe again
 * (placement before launch: kernels only ever read their own GPU's memory).
 * No counterpart in the reference, whose Storage lives on one Device
 * (crates/oxmera-tensor/src/storage.rs:12-17) and has no device-to-device copy. */
int oxm_copy_peer(oxm_ctx *dst_ctx, void *dst_device, oxm_ctx *src_ctx, const void *src_device, size_t bytes);
int oxm_sync(oxm_ctx *ctx);
/* Page-locked host staging memory (faster, truly asynchronous copies). */
int oxm_host_alloc(size_t bytes, void **out);
int oxm_host_free(void *ptr);

/* ---- the operator surface ----------------------------------------------
 * oxm_matmul stands behind `MatmulOps::matmul`
 * (crates/oxmera-ops/src/lib.rs:53-59) as implemented by
 * `CpuBackend::matmul` (crates/oxmera-cpu/src/lib.rs:71-76):
 * [m,k] x [k,n] -> [m,n], rank 2 exactly, operands read through their views.
 * Inner-dimension or rank violations are OXM_SHAPE_MISMATCH, differing dtypes
 * OXM_DTYPE_MISMATCH, non-float dtypes OXM_UNSUPPORTED_DTYPE, differing
 * devices OXM_DEVICE_MISMATCH.  `out` is caller-allocated (the host wrapper
 * makes it fresh and contiguous, crates/oxmera-ops/src/lib.rs:16-17) and is
 * written through its own strides, so a shard may write into a window of a
 * parent tensor.  `out` must not alias the operands.
 *
 * oxm_batched_matmul is the batched extension of the same trait: rank >= 2,
 * leading dims broadcast by NumPy rules
 * (crates/oxmera-core/src/shape.rs:49-55), trailing two dims as above.
 *
 * dtypes: f32 (fp32 result; 3xTF32 tensor-core path or an FFMA tile kernel;
 * infinities and NaNs in the operands propagate as in IEEE arithmetic on
 * either),
 * bf16 and f16 (fp32 accumulate, result rounded to the operand dtype), and
 * fp8 e4m3 / e5m2 (fp32 accumulate; `out` may be the operands' fp8 type —
 * rounded to nearest even, saturating to the largest finite value — or bf16,
 * f16 or f32, the one place an output may be wider than its operands). */
int oxm_matmul(oxm_ctx *ctx, const oxm_view *a, const oxm_view *b, const oxm_view *out);
int oxm_batched_matmul(oxm_ctx *ctx, const oxm_view *a, const oxm_view *b, const oxm_view *out);

/* The product with the step a caller runs next fused into the GEMM's epilogue
 * (fp32, before the single rounding to the output dtype):
 *     r = sum_k a[m,k] b[k,n];  r += bias[n];  r = act(r);  r += out[m,n]
 * each step optional.  `bias` is a rank-1 view of N elements of the operand
 * dtype (a linear layer's forward, with `activation`); `accumulate` adds what
 * `out` already holds (dW += dY^T.X across micro-batches).  Shapes broadcast as
 * in oxm_batched_matmul.  oxmera reserves the crates these steps belong to
 * (crates/oxmera-nn/src/lib.rs, crates/oxmera-autograd/src/lib.rs) and has no
 * signature for them yet; this entry point is the backend half they will call. */
enum { OXM_ACT_NONE = 0, OXM_ACT_RELU = 1, OXM_ACT_GELU = 2 /* 0.5 x (1 + erf(x / sqrt 2)) */ };
typedef struct {
  const oxm_view *bias; /* NULL for none */
  int32_t activation;   /* OXM_ACT_* */
  int32_t accumulate;   /* non-zero: out += result */
} oxm_epilogue;
int oxm_matmul_fused(oxm_ctx *ctx, const oxm_view *a, const oxm_view *b, const oxm_view *out, const oxm_epilogue *ep);

/* Block-scaled fp8 product (the OCP Microscaling format MXFP8):
 *   out[i, j] = sum over blocks kb of
 *               2^(a_scale[i, kb] - 127) * 2^(b_scale[kb, j] - 127) *
 *               sum over the block's 32 k of a[i, k] * b[k, j],
 * accumulated in fp32.  `a` and `b` are F8E4M3 or F8E5M2 views (the same
 * type), shaped and broadcast as for oxm_batched_matmul, with a contraction
 * length that is a multiple of 32; `a_scale` and `b_scale` are U8 views of
 * E8M0 exponents with their operand's shape except that the contraction dim
 * is divided by 32 ([.., M, K/32] and [.., K/32, N]); a scale byte of 255 is
 * NaN.  `out` is BF16, F16, F32 or the operands' type.  Operands the tensor
 * core cannot read in place (contraction dim not contiguous, odd pitches) are
 * packed first; the scales are always regrouped on the device into the
 * 512-byte atoms the tensor core reads, a pass over K/32 bytes per operand
 * row.  oxmera's DType stops at the 8-bit integer types
 * (crates/oxmera-core/src/dtype.rs:9-23) and no crate of it has a quantised
 * product: this entry point has no counterpart in the reference and stands
 * beside oxm_matmul_fused as the backend half such an op would call. */
int oxm_matmul_mx(oxm_ctx *ctx, const oxm_view *a, const oxm_view *a_scale, const oxm_view *b, const oxm_view *b_scale,
                  const oxm_view *out);

/* ---- the other op families of Backend --------------------------------------
 * Stand behind UnaryOps, BinaryOps and ReduceOps (crates/oxmera-ops/src/lib.rs:
 * 27-50,61-69) for Device::Cuda.  Inputs are any views; `out` is a fresh
 * row-major contiguous tensor of the result's shape and the operands' dtype
 * (crates/oxmera-ops/src/lib.rs:16-17).  dtypes: f32, f64, bf16, f16 for
 * everything; i32, i64 for neg, abs, add, sub, mul, div, sum, max.  exp / ln
 * on integers and any op on u8 / bool are OXM_UNSUPPORTED_DTYPE.  Integer div
 * truncates toward zero (the most negative value / -1 wraps to itself); a zero
 * divisor anywhere makes the call return OXM_DIVIDE_BY_ZERO, as the trait
 * asks (crates/oxmera-ops/src/lib.rs:47-49) — for that the integer form waits
 * for its kernel before returning, unlike every other compute call.  max
 * propagates NaN.
 * Binary operands broadcast by NumPy rules (crates/oxmera-core/src/shape.rs:
 * 49-55) and must share dtype and device.  oxm_reduce removes `axes` from the
 * shape; naxes = 0 means all axes (a scalar result); a sum over an empty
 * extent is 0, a max over one is refused ("there is no identity to invent"). */
enum { OXM_NEG = 0, OXM_EXP = 1, OXM_LN = 2, OXM_ABS = 3 };
enum { OXM_ADD = 0, OXM_SUB = 1, OXM_MUL = 2, OXM_DIV = 3 };
enum { OXM_SUM = 0, OXM_MAX = 1 };
int oxm_unary(oxm_ctx *ctx, int op, const oxm_view *a, const oxm_view *out);
int oxm_binary(oxm_ctx *ctx, int op, const oxm_view *a, const oxm_view *b, const oxm_view *out);
int oxm_reduce(oxm_ctx *ctx, int op, const oxm_view *a, const int32_t *axes, int naxes, const oxm_view *out);

/* Same operation on HOST views: `base` pointers are host memory.  The
 * operands are staged to the device, multiplied, and the result copied back
 * into `out`'s (contiguous) host buffer before returning.  Large products are
 * cut along the output's leading dim so that copy-in, multiply and copy-out
 * of successive slices overlap (page-locked host buffers are needed for the
 * overlap; pageable ones still give the right result).  This is what
 * `Tensor::matmul` costs when the tensors start and end in host memory
 * (crates/oxmera-runtime/src/lib.rs:68-69,99-102). */
int oxm_batched_matmul_host(oxm_ctx *ctx, const oxm_view *a, const oxm_view *b, const oxm_view *out);

/* f32 rank-2 matmul that allocates nothing.  It has no counterpart in the
 * oxmera reference; it exists for hosts that cannot allocate device memory
 * while they run: one that gave all of HBM to its own arena at start-up, or a
 * latency-critical loop where an allocator call (a possible device-wide
 * synchronisation, a possible out-of-memory failure) is not acceptable.
 *
 * Same contract and typed errors as oxm_matmul for f32 operands, always on the
 * tensor-core 3xTF32 path.  The scratch that path needs (both operands packed
 * as TF32 hi/lo terms, plus split-K partial sums when K > 1024) lives in a
 * fixed array of OXM_NOALLOC_SCRATCH_BYTES inside the library's device image;
 * every GPU that loads the library holds that array until the process exits.
 * The call makes no cudaMalloc / cudaFree / pool call.
 *
 * Limit: 256-byte-rounded  M*3*Kp*4 + N*3*Kp*4 (+ S*M*N*4 when K > 1024),
 * with Kp = K rounded up to 32 and S = ceil(3*Kp / 3072), must not exceed
 * OXM_NOALLOC_SCRATCH_BYTES; larger products are refused with
 * OXM_NOT_IMPLEMENTED and a message that states both sizes.
 *
 * The first call on each device looks the array's address up (and may make
 * the driver load the module); make that call during start-up, before any
 * stream capture begins.  All calls share the one array: two calls whose
 * kernels can overlap on the GPU (different contexts on the same device)
 * race on it; calls through one context are ordered by its stream.  Nothing
 * in the array needs clearing between calls: each call rewrites every element
 * it later reads. */
#define OXM_NOALLOC_SCRATCH_BYTES (32u << 20)
int oxm_matmul_f32_noalloc(oxm_ctx *ctx, const oxm_view *a, const oxm_view *b, const oxm_view *out);

/* Stands behind the device half of `Tensor::contiguous`
 * (crates/oxmera-tensor/src/tensor.rs:86-90): gathers `src` (any strides, any
 * dtype) in logical order into `dst`, a row-major contiguous view of the same
 * shape and dtype in different storage. */
int oxm_contiguous(oxm_ctx *ctx, const oxm_view *src, const oxm_view *dst);

/* ---- instrumentation ------------------------------------------------------
 * Not part of the reference surface: timing on the context's stream and
 * kernel selection for tests and benchmarks. */
int oxm_event_create(oxm_ctx *ctx, oxm_event **out);
int oxm_event_destroy(oxm_event *ev);
int oxm_event_record(oxm_ctx *ctx, oxm_event *ev);
int oxm_event_elapsed_ms(oxm_event *start, oxm_event *stop, float *ms); /* syncs on stop */
int oxm_stream_handle(oxm_ctx *ctx, void **cuda_stream);

/* Seeded synthetic data written straight into device memory (f32, bf16 or
 * f16): dist 0 = U(-1,1), dist 1 = N(0,1) * scale.  Element i depends only on
 * (seed, stream, i). */
int oxm_fill(oxm_ctx *ctx, void *dst_device, int dtype, int64_t n, uint64_t seed, uint64_t stream, int dist, double scale);

/* Failure-path self-test: launches a kernel whose only thread waits, with the
 * bound `limit_ms` (1..1000), on a barrier nothing arrives on.  Returns
 * OXM_TIMEOUT when the wait gave up and the status word reached the host, as
 * a stuck pipeline would report; the context stays usable.  Nothing faults. */
int oxm_selftest_bounded_wait(oxm_ctx *ctx, int64_t limit_ms);

/* Options (key, value):
 *   "kernel"      0 auto, 1 force the SIMT FFMA kernel, 2 force the tcgen05
 *                 kernel (packing operands it cannot address directly)
 *   "tile_n"      0 auto, else the tile's width: a multiple of 32 from 64 to 512
 *                 (288 and wider: CTA pairs only).  oxm_matmul_mx takes 128, 192,
 *                 256 or 384 from it and ignores other values
 *   "cta_pair"    -1 auto, 0 one CTA per tile, 1 CTA pairs (cta_group::2)
 *   "host_chunks" slices of the host entry point's copy/compute pipeline:
 *                 0 auto (up to 8 for outputs of 16 MiB or more), 1 off, 2..16
 *   "split_k"     -1 auto, 0 never split beyond what f32 accuracy needs, else
 *                 the number of contraction chains (the FFMA kernel takes 2, 4
 *                 or 8 from it: CTAs of a cluster per tile)
 *   "tma_store"   1 (default) write results with bulk tensor stores when the
 *                 output allows it, 0 always use plain strided stores
 *   "group_m"     0 auto, else the number of tile rows walked together
 *   "stream_k"    -1 auto, 0 whole tiles only, 1 share the last tiles out by
 *                 contraction block whenever the tile count does not divide
 *                 by the SM count ("split_k" 0 also turns this off: one
 *                 accumulation chain per output element).  Auto uses it only
 *                 where whole waves of ordinary tiles run beside the
 *                 shared-out ones and the model sees more than 12 us saved
 *   "simt_tile"   0 auto, 32 or 64: the FFMA kernel's tile edge
 *   "wait_limit_ms"  bound of every device-side wait (default 2000, or the
 *                 environment variable OXM_WAIT_LIMIT_MS at context creation)
 * Unknown keys or values are OXM_INVALID_ARGUMENT. */
int oxm_set_option(oxm_ctx *ctx, const char *key, int64_t value);
int oxm_get_option(oxm_ctx *ctx, const char *key, int64_t *value);

/* Counters since context creation: kernels launched by this library.  index 0
 * total, 1 tensor-core GEMM, 2 FFMA GEMM, 3 auxiliary kernels of a product
 * (operand pack, split-K reduction, strided copy). */
int oxm_launch_counts(oxm_ctx *ctx, int64_t counts[4]);
/* Name of the compute kernel the last matmul on this context selected. */
const char *oxm_last_kernel(oxm_ctx *ctx);
/* Device memory as this process sees it, in bytes: stats[0] reserved and
 * stats[1] in use in the device's stream-ordered pool (what oxm_alloc and the
 * library's workspaces draw from), stats[2] free and stats[3] total on the
 * device (cudaMemGetInfo).  No counterpart in the reference; tests use it to
 * show that a call allocated nothing. */
int oxm_memory_stats(oxm_ctx *ctx, int64_t stats[4]);

/* The decisions oxm_batched_matmul would take for these views on a GPU of
 * `num_sms` SMs with default options; runs on the host alone (no context, no
 * GPU; storage pointers are only inspected for alignment).  No counterpart in
 * the reference: it exists so that the planner can be tested where there is
 * no GPU.  plan[0] kernel (0 nothing to launch, 1 FFMA, 2 tcgen05), plan[1]
 * tile width, plan[2] CTA pairs, plan[3] contraction chains (split-K factor),
 * plan[4] / plan[5] whether A / B is packed first (1) or read in place (0),
 * plan[6] how many of the last tiles are shared out by contraction block
 * (stream-K; 0 = whole tiles only), plan[7] reserved (0).
 * Validation errors are those of oxm_batched_matmul. */
int oxm_plan_matmul(const oxm_view *a, const oxm_view *b, const oxm_view *out, int num_sms, int32_t plan[8]);

#ifdef __cplusplus
}
#endif
#endif
