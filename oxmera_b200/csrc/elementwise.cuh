// The HBM-bound half of oxmera's Backend trait on the device: UnaryOps
// (neg, exp, ln, abs), BinaryOps (add, sub, mul, div with NumPy broadcasting)
// and ReduceOps (sum, max over axes).  Inputs are read through their views
// (signed element strides, broadcast dims as stride 0); outputs are fresh and
// contiguous, so consecutive threads write consecutive elements.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

namespace oxm {

constexpr int kEwMaxDims = 8;

// dtype tags of the C ABI: 0 f32, 1 f64, 2 i32, 3 i64, 6 bf16, 7 f16.
// 16-bit floats compute in f32, f32 in f32, f64 in f64, integers in i64.
template <typename T> struct EwTraits;
template <> struct EwTraits<float> { using C = float; };
template <> struct EwTraits<double> { using C = double; };
template <> struct EwTraits<int32_t> { using C = int64_t; };
template <> struct EwTraits<int64_t> { using C = int64_t; };
template <> struct EwTraits<__nv_bfloat16> { using C = float; };
template <> struct EwTraits<__half> { using C = float; };
// raw element widths, for copies that do no arithmetic
template <> struct EwTraits<uint8_t> { using C = uint8_t; };
template <> struct EwTraits<uint16_t> { using C = uint16_t; };
template <> struct EwTraits<uint32_t> { using C = uint32_t; };
template <> struct EwTraits<uint64_t> { using C = uint64_t; };

template <typename T> __device__ __forceinline__ typename EwTraits<T>::C ew_load(const T *p, int64_t i) {
  return static_cast<typename EwTraits<T>::C>(p[i]);
}
template <> __device__ __forceinline__ float ew_load<__nv_bfloat16>(const __nv_bfloat16 *p, int64_t i) { return __bfloat162float(p[i]); }
template <> __device__ __forceinline__ float ew_load<__half>(const __half *p, int64_t i) { return __half2float(p[i]); }

template <typename T> __device__ __forceinline__ void ew_store(T *p, int64_t i, typename EwTraits<T>::C v) { p[i] = static_cast<T>(v); }
template <> __device__ __forceinline__ void ew_store<__nv_bfloat16>(__nv_bfloat16 *p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void ew_store<__half>(__half *p, int64_t i, float v) { p[i] = __float2half_rn(v); }

struct EwParams {
  const void *a, *b;  // b unused by unary ops
  void *out;
  int32_t op, ndim;
  int64_t n;          // output elements
  int64_t shape[kEwMaxDims];
  int64_t a_strides[kEwMaxDims], b_strides[kEwMaxDims];  // 0 where broadcast
  int64_t a_off, b_off;
  int32_t contiguous;  // both inputs are row-major over the output shape: offsets are linear
  int32_t vec;         // ... and every pointer is 16-byte aligned: 16 bytes per thread per step
  int32_t rows;        // 1: one CTA per row of the innermost dim (no per-element index arithmetic)
  int32_t rows_vec;    // ... with inner strides 0 or 1 and 16-byte-aligned rows
  int32_t tile_r;      // >= 0: 32x32 tiles over (this dim, innermost dim); an operand whose unit stride is on this dim turns through shared memory
  int32_t a_turn, b_turn;
  int32_t pairs;       // 2-byte elements, everything 4-byte aligned: the tile kernel moves two elements per access
  int32_t quads;       // ... and rows of the straight operands and of the output 8-byte aligned, C a multiple of 4:
                       // the turn happens in registers (ew_reg2_kernel)
};

__device__ __forceinline__ void ew_offsets(const EwParams &p, int64_t i, int64_t &ao, int64_t &bo) {
  if (p.contiguous) {
    ao = p.a_off + i;
    bo = p.b_off + i;
    return;
  }
  ao = p.a_off;
  bo = p.b_off;
  for (int d = p.ndim - 1; d >= 0; --d) {
    const int64_t idx = i % p.shape[d];
    i /= p.shape[d];
    ao += idx * p.a_strides[d];
    bo += idx * p.b_strides[d];
  }
}

template <typename C> __device__ __forceinline__ C unary_apply(int op, C x);
template <> __device__ __forceinline__ float unary_apply<float>(int op, float x) {
  return op == 0 ? -x : op == 1 ? expf(x) : op == 2 ? logf(x) : fabsf(x);
}
template <> __device__ __forceinline__ double unary_apply<double>(int op, double x) {
  return op == 0 ? -x : op == 1 ? exp(x) : op == 2 ? log(x) : fabs(x);
}
template <> __device__ __forceinline__ int64_t unary_apply<int64_t>(int op, int64_t x) {
  return op == 0 ? -x : (x < 0 ? -x : x);  // exp / ln are refused for integers on the host
}

template <typename C> __device__ __forceinline__ C binary_apply(int op, C x, C y) {
  return op == 0 ? x + y : op == 1 ? x - y : op == 2 ? x * y : x / y;  // integer div has its own kernel
}
// 16 bytes of T, moved with one vector load / store.
template <typename T> struct alignas(16) EwVec { T v[16 / sizeof(T)]; };

template <typename T>
__global__ void __launch_bounds__(256) unary_kernel(const EwParams p) {
  using C = typename EwTraits<T>::C;
  const T *a = static_cast<const T *>(p.a);
  T *out = static_cast<T *>(p.out);
  int64_t first = 0;
  if (p.vec) {
    constexpr int V = 16 / sizeof(T);
    const int64_t nv = p.n / V;
    const EwVec<T> *av = reinterpret_cast<const EwVec<T> *>(a + p.a_off);
    EwVec<T> *ov = reinterpret_cast<EwVec<T> *>(out);
    for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < nv; i += static_cast<int64_t>(gridDim.x) * 256) {
      const EwVec<T> x = av[i];
      EwVec<T> r;
#pragma unroll
      for (int e = 0; e < V; ++e) ew_store<T>(r.v, e, unary_apply<C>(p.op, ew_load<T>(x.v, e)));
      ov[i] = r;
    }
    first = nv * V;  // the ragged tail falls through to the scalar loop
  }
  for (int64_t i = first + blockIdx.x * 256ll + threadIdx.x; i < p.n; i += static_cast<int64_t>(gridDim.x) * 256) {
    int64_t ao, bo;
    ew_offsets(p, i, ao, bo);
    ew_store<T>(out, i, unary_apply<C>(p.op, ew_load<T>(a, ao)));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) binary_kernel(const EwParams p) {
  using C = typename EwTraits<T>::C;
  const T *a = static_cast<const T *>(p.a), *b = static_cast<const T *>(p.b);
  T *out = static_cast<T *>(p.out);
  int64_t first = 0;
  if (p.vec) {
    constexpr int V = 16 / sizeof(T);
    const int64_t nv = p.n / V;
    const EwVec<T> *av = reinterpret_cast<const EwVec<T> *>(a + p.a_off), *bv = reinterpret_cast<const EwVec<T> *>(b + p.b_off);
    EwVec<T> *ov = reinterpret_cast<EwVec<T> *>(out);
    for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < nv; i += static_cast<int64_t>(gridDim.x) * 256) {
      const EwVec<T> x = av[i], y = bv[i];
      EwVec<T> r;
#pragma unroll
      for (int e = 0; e < V; ++e) ew_store<T>(r.v, e, binary_apply<C>(p.op, ew_load<T>(x.v, e), ew_load<T>(y.v, e)));
      ov[i] = r;
    }
    first = nv * V;
  }
  for (int64_t i = first + blockIdx.x * 256ll + threadIdx.x; i < p.n; i += static_cast<int64_t>(gridDim.x) * 256) {
    int64_t ao, bo;
    ew_offsets(p, i, ao, bo);
    ew_store<T>(out, i, binary_apply<C>(p.op, ew_load<T>(a, ao), ew_load<T>(b, bo)));
  }
}

// Integer division (BinaryOps::div on i32 / i64): truncates toward zero; the
// most negative value divided by -1 wraps to itself, as two's-complement
// negation does.  A zero divisor is a typed error for the caller: the thread
// that meets one stores 0 for that element and records kStatusDivideByZero in
// the context's status word, which the host reads before the call returns.
constexpr uint32_t kStatusDivideByZero = 13;  // OXM_DIVIDE_BY_ZERO

template <typename T>
__global__ void __launch_bounds__(256) int_div_kernel(const EwParams p, uint32_t *status) {
  const T *a = static_cast<const T *>(p.a), *b = static_cast<const T *>(p.b);
  T *out = static_cast<T *>(p.out);
  bool zero_seen = false;
  for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < p.n; i += static_cast<int64_t>(gridDim.x) * 256) {
    int64_t ao, bo;
    ew_offsets(p, i, ao, bo);
    const int64_t x = static_cast<int64_t>(a[ao]), y = static_cast<int64_t>(b[bo]);
    int64_t r = 0;
    if (y == 0) zero_seen = true;
    else if (y == -1) r = static_cast<int64_t>(0ull - static_cast<uint64_t>(x));
    else r = x / y;
    out[i] = static_cast<T>(r);
  }
  if (zero_seen) atomicCAS(status, 0u, kStatusDivideByZero);
}

// Strided or broadcast operands with a long innermost dim: one CTA per row.
// The row's base offsets are unravelled once; along the row each operand
// advances by its inner stride (0 for a broadcast operand), so a bias row, a
// per-row scalar or a narrowed window all stream at full width.  Bound to eight
// CTAs per SM: at the 64 registers the compiler took unasked, four CTAs per SM
// held too few loads in flight (a [16400] f32 row added to [16000, 16400]: 0.76
// of the HBM copy rate at four, 0.89 at eight; the spills are in the row setup).
template <typename T, bool BINARY>
__global__ void __launch_bounds__(256, 8) ew_rows_kernel(const EwParams p) {
  using C = typename EwTraits<T>::C;
  constexpr int V = 16 / sizeof(T);
  const T *a = static_cast<const T *>(p.a), *b = static_cast<const T *>(p.b);
  T *out = static_cast<T *>(p.out);
  const int nd = p.ndim - 1;
  const int64_t L = p.shape[nd], rows = p.n / L;
  const int64_t ais = p.a_strides[nd], bis = BINARY ? p.b_strides[nd] : 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    int64_t ao = p.a_off, bo = p.b_off, t = row;
    for (int d = nd - 1; d >= 0; --d) {
      const int64_t idx = t % p.shape[d];
      t /= p.shape[d];
      ao += idx * p.a_strides[d];
      bo += idx * p.b_strides[d];
    }
    T *orow = out + row * L;
    if (p.rows_vec) {
      const C a0 = ais == 0 ? ew_load<T>(a, ao) : C(0), b0 = (BINARY && bis == 0) ? ew_load<T>(b, bo) : C(0);
      for (int64_t x = threadIdx.x; x < L / V; x += 256) {
        EwVec<T> xa, xb, r;
        if (ais) xa = reinterpret_cast<const EwVec<T> *>(a + ao)[x];
        if (BINARY && bis) xb = reinterpret_cast<const EwVec<T> *>(b + bo)[x];
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const C va = ais ? ew_load<T>(xa.v, e) : a0;
          if (BINARY) ew_store<T>(r.v, e, binary_apply<C>(p.op, va, bis ? ew_load<T>(xb.v, e) : b0));
          else ew_store<T>(r.v, e, unary_apply<C>(p.op, va));
        }
        reinterpret_cast<EwVec<T> *>(orow)[x] = r;
      }
    } else {
      for (int64_t x = threadIdx.x; x < L; x += 256) {
        const C va = ew_load<T>(a, ao + x * ais);
        if (BINARY) ew_store<T>(orow, x, binary_apply<C>(p.op, va, ew_load<T>(b, bo + x * bis)));
        else ew_store<T>(orow, x, unary_apply<C>(p.op, va));
      }
    }
  }
}

// A transposed operand: its unit stride lies on dim R, not on the innermost
// dim C that the output is contiguous in.  Walking it along C touches one
// element per 32-byte sector.  Here each CTA takes TILE x TILE tiles of (R, C):
// a turned operand is read along R (coalesced) into padded shared memory and
// read back along C; other operands are read in place.  Every thread has
// TILE*TILE/256 independent loads in flight per phase.  Tiles are walked along
// diagonals so that CTAs running together differ in both coordinates and a
// power-of-two pitch does not pile their traffic onto a few DRAM channels.
// MODE 0 unary op, 1 binary op, 2 plain copy (T is then an unsigned integer of
// the element's width).  A_TURN / B_TURN: which operands are turned (B_TURN
// only with MODE 1).
template <typename T> struct EwTile { static constexpr int value = sizeof(T) >= 8 ? 32 : 64; };

template <typename T, int MODE, bool A_TURN, bool B_TURN>
__global__ void __launch_bounds__(256, (sizeof(T) >= 8 || MODE == 1) ? 4 : 6) ew_tile_kernel(const EwParams p) {
  using C = typename EwTraits<T>::C;
  constexpr int TILE = EwTile<T>::value, STEP = 256 / TILE, ITERS = TILE / STEP;
  __shared__ T sa[A_TURN ? TILE : 1][TILE + 1], sb[B_TURN ? TILE : 1][TILE + 1];
  const T *a = static_cast<const T *>(p.a), *b = static_cast<const T *>(p.b);
  T *out = static_cast<T *>(p.out);
  const int nd = p.ndim - 1, rd = p.tile_r;
  const int64_t R = p.shape[rd], Cn = p.shape[nd];
  // tile counts fit 32 bits (the host checks): 64-bit divisions would cost more than the tile's own work
  const uint32_t tiles_c = static_cast<uint32_t>((Cn + TILE - 1) / TILE), tiles_r = static_cast<uint32_t>((R + TILE - 1) / TILE);
  const uint32_t per_batch = tiles_c * tiles_r;
  const uint32_t ntiles = per_batch * static_cast<uint32_t>(p.n / (R * Cn));
  const int64_t asr = p.a_strides[rd], asc = p.a_strides[nd], bsr = p.b_strides[rd], bsc = p.b_strides[nd];
  const int tx = threadIdx.x % TILE, ty = threadIdx.x / TILE;
  for (uint32_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const uint32_t batch = tile / per_batch, in_batch = tile - batch * per_batch;
    const uint32_t y = in_batch / tiles_c, x = in_batch - y * tiles_c;
    const int64_t r0 = static_cast<int64_t>((y + x) % tiles_r) * TILE, c0 = static_cast<int64_t>(x) * TILE;  // consecutive tiles step along a diagonal
    int64_t t = batch, ao = p.a_off, bo = p.b_off, oo = 0, os = Cn, osr = 0;
    for (int d = nd - 1; d >= 0; --d) {
      if (d == rd) {
        osr = os;
      } else {
        const int64_t idx = t % p.shape[d];
        t /= p.shape[d];
        ao += idx * p.a_strides[d];
        bo += idx * p.b_strides[d];
        oo += idx * os;
      }
      os *= p.shape[d];
    }
    // every global load of the tile is issued before the first store: a turned
    // operand along R into shared memory, any other in the output's own mapping.
    // Addresses advance by one constant per step; tiles inside the matrix skip the edge tests.
    const bool inside = r0 + TILE <= R && c0 + TILE <= Cn;
    const int64_t c = c0 + tx;
    const T *pa_t = a + ao + (r0 + tx) * asr + (c0 + ty) * asc;  // turned mapping: thread x walks R
    const T *pa_d = a + ao + (r0 + ty) * asr + c * asc;          // direct mapping: thread x walks C
    const T *pb_t = b + bo + (r0 + tx) * bsr + (c0 + ty) * bsc;
    const T *pb_d = b + bo + (r0 + ty) * bsr + c * bsc;
    T da[ITERS], db[MODE == 1 ? ITERS : 1];
    {
      T va[ITERS], vb[MODE == 1 ? ITERS : 1];
      if (inside) {
#pragma unroll
        for (int i = 0; i < ITERS; ++i) {
          if constexpr (A_TURN) va[i] = pa_t[i * STEP * asc];
          else da[i] = pa_d[i * STEP * asr];
          if constexpr (MODE == 1) {
            if constexpr (B_TURN) vb[i] = pb_t[i * STEP * bsc];
            else db[i] = pb_d[i * STEP * bsr];
          }
        }
      } else {
        const bool r_in = r0 + tx < R, c_in = c < Cn;
#pragma unroll
        for (int i = 0; i < ITERS; ++i) {
          const bool in_t = r_in && c0 + ty + STEP * i < Cn, in_d = c_in && r0 + ty + STEP * i < R;
          if constexpr (A_TURN) { if (in_t) va[i] = pa_t[i * STEP * asc]; }
          else if (in_d) da[i] = pa_d[i * STEP * asr];
          if constexpr (MODE == 1) {
            if constexpr (B_TURN) { if (in_t) vb[i] = pb_t[i * STEP * bsc]; }
            else if (in_d) db[i] = pb_d[i * STEP * bsr];
          }
        }
      }
#pragma unroll
      for (int i = 0; i < ITERS; ++i) {
        const int cl = ty + STEP * i;
        if constexpr (A_TURN) sa[tx][cl] = va[i];
        if constexpr (B_TURN) sb[tx][cl] = vb[i];
      }
    }
    __syncthreads();
    T *po = out + oo + (r0 + ty) * osr + c;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int rl = ty + STEP * i;
      if (inside || (r0 + rl < R && c < Cn)) {
        const T ra = A_TURN ? sa[rl][tx] : da[i];
        if constexpr (MODE == 2) {
          po[i * STEP * osr] = ra;
        } else if constexpr (MODE == 1) {
          const T rb = B_TURN ? sb[rl][tx] : db[i];
          ew_store<T>(po, i * STEP * osr, binary_apply<C>(p.op, ew_load<T>(&ra, 0), ew_load<T>(&rb, 0)));
        } else {
          ew_store<T>(po, i * STEP * osr, unary_apply<C>(p.op, ew_load<T>(&ra, 0)));
        }
      }
    }
    __syncthreads();
  }
}

// The tile kernel for 2-byte elements when every address involved is 4-byte
// aligned and both tile extents are even: each thread moves two neighbouring
// elements per global access (a turned operand's pair lies along R, everything
// else's along C), which halves the global instructions of the scalar version.
// Used for copies and unary operators (3.1 -> 3.8 TB/s on a bf16 transposed
// copy); with two operands it measured no faster than the scalar kernel.
// Shared memory rows are 66 elements: the pair stores of the turning step
// conflict two ways, the pair loads of the read-back not at all.
template <typename T, int MODE, bool A_TURN, bool B_TURN>
__global__ void __launch_bounds__(256, MODE == 1 ? 4 : 6) ew_tile2_kernel(const EwParams p) {
  static_assert(sizeof(T) == 2, "pairs of 2-byte elements");
  using C = typename EwTraits<T>::C;
  constexpr int TILE = 64, PITCH = 66, ITERS = 8;
  __shared__ __align__(4) T sa[A_TURN ? TILE : 1][PITCH];
  __shared__ __align__(4) T sb[B_TURN ? TILE : 1][PITCH];
  const T *a = static_cast<const T *>(p.a), *b = static_cast<const T *>(p.b);
  T *out = static_cast<T *>(p.out);
  const int nd = p.ndim - 1, rd = p.tile_r;
  const int64_t R = p.shape[rd], Cn = p.shape[nd];
  const uint32_t tiles_c = static_cast<uint32_t>((Cn + TILE - 1) / TILE), tiles_r = static_cast<uint32_t>((R + TILE - 1) / TILE);
  const uint32_t per_batch = tiles_c * tiles_r;
  const uint32_t ntiles = per_batch * static_cast<uint32_t>(p.n / (R * Cn));
  const int64_t asr = p.a_strides[rd], asc = p.a_strides[nd], bsr = p.b_strides[rd], bsc = p.b_strides[nd];
  const int tx = (threadIdx.x & 31) * 2, ty = threadIdx.x >> 5;  // this thread's pair starts at tx; 8 rows (or columns) per step
  for (uint32_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const uint32_t batch = tile / per_batch, in_batch = tile - batch * per_batch;
    const uint32_t y = in_batch / tiles_c, x = in_batch - y * tiles_c;
    const int64_t r0 = static_cast<int64_t>((y + x) % tiles_r) * TILE, c0 = static_cast<int64_t>(x) * TILE;
    int64_t t = batch, ao = p.a_off, bo = p.b_off, oo = 0, os = Cn, osr = 0;
    for (int d = nd - 1; d >= 0; --d) {
      if (d == rd) {
        osr = os;
      } else {
        const int64_t idx = t % p.shape[d];
        t /= p.shape[d];
        ao += idx * p.a_strides[d];
        bo += idx * p.b_strides[d];
        oo += idx * os;
      }
      os *= p.shape[d];
    }
    // turned operand: the pair (r0 + tx, r0 + tx + 1) of column c0 + ty + 8 i, unit stride along R;
    // any other operand and the output: the pair (c0 + tx, c0 + tx + 1) of row r0 + ty + 8 i.
    const bool rp_in = r0 + tx < R, cp_in = c0 + tx < Cn;  // extents are even: a pair is inside or outside as a whole
    const T *pa_t = a + ao + (r0 + tx) + (c0 + ty) * asc;
    const T *pb_t = b + bo + (r0 + tx) + (c0 + ty) * bsc;
    const T *pa_d = a + ao + (r0 + ty) * asr + (c0 + tx);
    const T *pb_d = b + bo + (r0 + ty) * bsr + (c0 + tx);
    uint32_t da[ITERS], db[MODE == 1 ? ITERS : 1];
    {
      uint32_t va[ITERS], vb[MODE == 1 ? ITERS : 1];
#pragma unroll
      for (int i = 0; i < ITERS; ++i) {
        const bool in_t = rp_in && c0 + ty + 8 * i < Cn, in_d = cp_in && r0 + ty + 8 * i < R;
        if constexpr (A_TURN) { if (in_t) va[i] = *reinterpret_cast<const uint32_t *>(pa_t + i * 8 * asc); }
        else if (in_d) da[i] = *reinterpret_cast<const uint32_t *>(pa_d + i * 8 * asr);
        if constexpr (MODE == 1) {
          if constexpr (B_TURN) { if (in_t) vb[i] = *reinterpret_cast<const uint32_t *>(pb_t + i * 8 * bsc); }
          else if (in_d) db[i] = *reinterpret_cast<const uint32_t *>(pb_d + i * 8 * bsr);
        }
      }
#pragma unroll
      for (int i = 0; i < ITERS; ++i) {
        const int cl = ty + 8 * i;
        if constexpr (A_TURN) {
          reinterpret_cast<uint16_t *>(&sa[tx][cl])[0] = static_cast<uint16_t>(va[i] & 0xffffu);
          reinterpret_cast<uint16_t *>(&sa[tx + 1][cl])[0] = static_cast<uint16_t>(va[i] >> 16);
        }
        if constexpr (B_TURN) {
          reinterpret_cast<uint16_t *>(&sb[tx][cl])[0] = static_cast<uint16_t>(vb[i] & 0xffffu);
          reinterpret_cast<uint16_t *>(&sb[tx + 1][cl])[0] = static_cast<uint16_t>(vb[i] >> 16);
        }
      }
    }
    __syncthreads();
    T *po = out + oo + (r0 + ty) * osr + (c0 + tx);
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int rl = ty + 8 * i;
      if (cp_in && r0 + rl < R) {
        uint32_t wa, wb = 0;
        if constexpr (A_TURN) wa = *reinterpret_cast<const uint32_t *>(&sa[rl][tx]);
        else wa = da[i];
        if constexpr (MODE == 1) {
          if constexpr (B_TURN) wb = *reinterpret_cast<const uint32_t *>(&sb[rl][tx]);
          else wb = db[i];
        }
        uint32_t w;
        if constexpr (MODE == 2) {
          w = wa;
        } else {
          alignas(4) T ea[2];
          alignas(4) T eb[2];
          alignas(4) T eo[2];
          *reinterpret_cast<uint32_t *>(ea) = wa;
          *reinterpret_cast<uint32_t *>(eb) = wb;
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            if constexpr (MODE == 1) ew_store<T>(eo, e, binary_apply<C>(p.op, ew_load<T>(ea, e), ew_load<T>(eb, e)));
            else ew_store<T>(eo, e, unary_apply<C>(p.op, ew_load<T>(ea, e)));
          }
          w = *reinterpret_cast<const uint32_t *>(eo);
        }
        *reinterpret_cast<uint32_t *>(po + i * 8 * osr) = w;
      }
    }
    __syncthreads();
  }
}

// 2-byte elements with a transposed operand, turned in registers instead of
// shared memory.  A thread owns a block of 2 rows (R) x 4 columns (C): it reads
// a turned operand as four 4-byte pairs along R (one per column), a straight
// operand as two 8-byte runs along C (one per row), computes, and writes two
// 8-byte runs of the output.  A warp is 8 threads along R by 4 along C, so every
// access of a warp touches whole 32-byte sectors (8 x 4 bytes along R for the
// turned operand, 4 x 8 bytes along C for the rest), and the eight warps of a
// CTA cover whole 128-byte lines of every operand within one 64 x 64 tile.  No
// shared memory, no barrier, 12 to 16 independent loads in flight per thread.
// Needs: R even, C a multiple of 4, turned operands 4-byte aligned with even
// other strides, straight operands and the output 8-byte aligned with other
// strides that are multiples of 4.
template <typename T, int MODE, bool A_TURN, bool B_TURN>
__global__ void __launch_bounds__(256) ew_reg2_kernel(const EwParams p) {
  static_assert(sizeof(T) == 2, "2-byte elements");
  using C = typename EwTraits<T>::C;
  constexpr int TILE = 64;
  const T *a = static_cast<const T *>(p.a), *b = static_cast<const T *>(p.b);
  T *out = static_cast<T *>(p.out);
  const int nd = p.ndim - 1, rd = p.tile_r;
  const int64_t R = p.shape[rd], Cn = p.shape[nd];
  const uint32_t tiles_c = static_cast<uint32_t>((Cn + TILE - 1) / TILE), tiles_r = static_cast<uint32_t>((R + TILE - 1) / TILE);
  const uint32_t per_batch = tiles_c * tiles_r;
  const uint32_t ntiles = per_batch * static_cast<uint32_t>(p.n / (R * Cn));
  const int64_t asr = p.a_strides[rd], asc = p.a_strides[nd], bsr = p.b_strides[rd], bsc = p.b_strides[nd];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tr = (warp & 3) * 16 + (lane & 7) * 2;   // this thread's first row within the tile
  const int tc = (warp >> 2) * 16 + (lane >> 3) * 4;  // ... and first column; a second block sits 32 columns on
  for (uint32_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const uint32_t batch = tile / per_batch, in_batch = tile - batch * per_batch;
    const uint32_t y = in_batch / tiles_c, x = in_batch - y * tiles_c;
    const int64_t r0 = static_cast<int64_t>((y + x) % tiles_r) * TILE, c0 = static_cast<int64_t>(x) * TILE;
    int64_t t = batch, ao = p.a_off, bo = p.b_off, oo = 0, os = Cn, osr = 0;
    for (int d = nd - 1; d >= 0; --d) {
      if (d == rd) {
        osr = os;
      } else {
        const int64_t idx = t % p.shape[d];
        t /= p.shape[d];
        ao += idx * p.a_strides[d];
        bo += idx * p.b_strides[d];
        oo += idx * os;
      }
      os *= p.shape[d];
    }
    const int64_t r = r0 + tr;
    const bool r_in = r < R;  // R is even: both rows or neither
    uint32_t ta[2][4], tb[2][4];  // turned operands: [block][column] = the pair (r, r + 1) of that column
    uint2 sa[2][2], sb[2][2];     // straight operands: [block][row] = columns c .. c + 3 of that row
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int64_t c = c0 + tc + 32 * k;
      const bool in = r_in && c < Cn;  // C is a multiple of 4: all four columns or none
      if (!in) continue;
      if constexpr (A_TURN) {
#pragma unroll
        for (int j = 0; j < 4; ++j) ta[k][j] = *reinterpret_cast<const uint32_t *>(a + ao + r + (c + j) * asc);
      } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) sa[k][i] = *reinterpret_cast<const uint2 *>(a + ao + (r + i) * asr + c);
      }
      if constexpr (MODE == 1) {
        if constexpr (B_TURN) {
#pragma unroll
          for (int j = 0; j < 4; ++j) tb[k][j] = *reinterpret_cast<const uint32_t *>(b + bo + r + (c + j) * bsc);
        } else {
#pragma unroll
          for (int i = 0; i < 2; ++i) sb[k][i] = *reinterpret_cast<const uint2 *>(b + bo + (r + i) * bsr + c);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int64_t c = c0 + tc + 32 * k;
      if (!(r_in && c < Cn)) continue;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        // row i of the block as four 16-bit patterns, from either form
        uint16_t ea[4], eb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if constexpr (A_TURN) ea[j] = static_cast<uint16_t>(ta[k][j] >> (16 * i));
          else ea[j] = static_cast<uint16_t>((j < 2 ? sa[k][i].x : sa[k][i].y) >> (16 * (j & 1)));
          if constexpr (MODE == 1) {
            if constexpr (B_TURN) eb[j] = static_cast<uint16_t>(tb[k][j] >> (16 * i));
            else eb[j] = static_cast<uint16_t>((j < 2 ? sb[k][i].x : sb[k][i].y) >> (16 * (j & 1)));
          }
        }
        uint16_t eo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if constexpr (MODE == 2) {
            eo[j] = ea[j];
          } else {
            T va, vb, vo;
            memcpy(&va, &ea[j], 2);
            if constexpr (MODE == 1) {
              memcpy(&vb, &eb[j], 2);
              ew_store<T>(&vo, 0, binary_apply<C>(p.op, ew_load<T>(&va, 0), ew_load<T>(&vb, 0)));
            } else {
              ew_store<T>(&vo, 0, unary_apply<C>(p.op, ew_load<T>(&va, 0)));
            }
            memcpy(&eo[j], &vo, 2);
          }
        }
        uint2 w;
        w.x = static_cast<uint32_t>(eo[0]) | (static_cast<uint32_t>(eo[1]) << 16);
        w.y = static_cast<uint32_t>(eo[2]) | (static_cast<uint32_t>(eo[3]) << 16);
        *reinterpret_cast<uint2 *>(out + oo + (r + i) * osr + c) = w;
      }
    }
  }
}

// Reduction.  The host splits the input's dims into kept dims (the output's
// index space, row-major) and reduced dims, drops extent-1 dims and merges
// neighbours that share one stride.  op 0 sum, 1 max.
//
// Two thread mappings, chosen by which group holds the smallest stride:
//   ROW  one CTA per output; its 256 threads walk the reduced extent, so a
//        reduced innermost dim is read coalesced (16-byte loads when it is
//        contiguous), then fold through shuffles and shared memory;
//   COL  one thread per output, consecutive threads on consecutive kept-dim
//        elements, each walking the reduced extent serially.
// Either way the reduced extent can be cut into `splits` slices (gridDim.y) so
// that few-output reductions still fill the GPU; slices write partial results
// in the compute type to a workspace and reduce_finish_kernel combines them.
struct ReduceOpParams {
  const void *a;
  void *out;       // final output (splits == 1) ...
  void *partial;   // ... or [splits][n_out] partial results in the compute type
  int32_t op, nkept, nred, splits;
  int32_t col_vec;              // COL mapping with 16 bytes of neighbouring outputs per thread
  int32_t warp_rows;            // ROW mapping with one warp per output (many short contiguous rows)
  int64_t n_out, n_red, chunk;  // chunk: reduced elements per slice
  int64_t kept_shape[kEwMaxDims], kept_strides[kEwMaxDims];
  int64_t red_shape[kEwMaxDims], red_strides[kEwMaxDims];
  int64_t a_off;
};

// max propagates NaN: once either side is NaN the result stays NaN, whatever the order of combination.
template <typename C> __device__ __forceinline__ C reduce_max(C x, C y) { return x != x ? x : (y != y ? y : (y > x ? y : x)); }
// f32 (the compute type of bf16 and f16 too): the NaN-propagating maximum is one instruction
template <> __device__ __forceinline__ float reduce_max<float>(float x, float y) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(x), "f"(y));
  return r;
}
template <typename C> __device__ __forceinline__ C reduce_combine(int op, C x, C y) { return op == 0 ? x + y : reduce_max<C>(x, y); }

template <typename C> __device__ __forceinline__ C reduce_identity(int op);
template <> __device__ __forceinline__ float reduce_identity<float>(int op) { return op == 0 ? 0.0f : -INFINITY; }
template <> __device__ __forceinline__ double reduce_identity<double>(int op) { return op == 0 ? 0.0 : -static_cast<double>(INFINITY); }
template <> __device__ __forceinline__ int64_t reduce_identity<int64_t>(int op) { return op == 0 ? 0 : INT64_MIN; }

__device__ __forceinline__ int64_t unravel(int64_t i, int nd, const int64_t *shape, const int64_t *strides) {
  int64_t off = 0;
  for (int d = nd - 1; d >= 0; --d) {
    off += (i % shape[d]) * strides[d];
    i /= shape[d];
  }
  return off;
}

template <typename C> __device__ __forceinline__ C shfl_down(C v, int d) { return __shfl_down_sync(0xffffffffu, v, d); }

template <typename T, int OP>
__global__ void __launch_bounds__(256) reduce_row_kernel(const ReduceOpParams p) {
  using C = typename EwTraits<T>::C;
  constexpr int V = 16 / sizeof(T);
  __shared__ C part[8];
  const T *a = static_cast<const T *>(p.a);
  const int64_t r0 = blockIdx.y * p.chunk, r1 = min(r0 + p.chunk, p.n_red);
  for (int64_t o = blockIdx.x; o < p.n_out; o += gridDim.x) {
    const int64_t base = p.a_off + unravel(o, p.nkept, p.kept_shape, p.kept_strides);
    C acc = reduce_identity<C>(OP);
    if (p.nred == 1 && p.red_strides[0] == 1) {
      // a contiguous run: scalar head up to a 16-byte boundary, vector body, scalar tail
      const T *run = a + base;
      const int64_t mis = (reinterpret_cast<uintptr_t>(run + r0) / sizeof(T)) % V;
      const int64_t head = min((V - mis) % V, r1 - r0);
      const int64_t nv = (r1 - r0 - head) / V;
      if (static_cast<int64_t>(threadIdx.x) < head) acc = reduce_combine<C>(OP, acc, ew_load<T>(run, r0 + threadIdx.x));
      const EwVec<T> *vec = reinterpret_cast<const EwVec<T> *>(run + r0 + head);
      // four running results per thread: one chain of dependent additions per 16 bytes (eight of
      // them for 2-byte elements) held bf16 sums at half the rate of f32 ones
      C lane_acc[4] = {acc, reduce_identity<C>(OP), reduce_identity<C>(OP), reduce_identity<C>(OP)};
#pragma unroll 4
      for (int64_t i = threadIdx.x; i < nv; i += 256) {
        const EwVec<T> x = vec[i];
#pragma unroll
        for (int e = 0; e < V; ++e) lane_acc[e & 3] = reduce_combine<C>(OP, lane_acc[e & 3], ew_load<T>(x.v, e));
      }
      acc = reduce_combine<C>(OP, reduce_combine<C>(OP, lane_acc[0], lane_acc[1]), reduce_combine<C>(OP, lane_acc[2], lane_acc[3]));
      for (int64_t r = r0 + head + nv * V + threadIdx.x; r < r1; r += 256) acc = reduce_combine<C>(OP, acc, ew_load<T>(run, r));
    } else if (p.nred == 1) {
      for (int64_t r = r0 + threadIdx.x; r < r1; r += 256) acc = reduce_combine<C>(OP, acc, ew_load<T>(a, base + r * p.red_strides[0]));
    } else {
      for (int64_t r = r0 + threadIdx.x; r < r1; r += 256)
        acc = reduce_combine<C>(OP, acc, ew_load<T>(a, base + unravel(r, p.nred, p.red_shape, p.red_strides)));
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc = reduce_combine<C>(OP, acc, shfl_down<C>(acc, d));
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      C total = part[0];
      for (int w = 1; w < 8; ++w) total = reduce_combine<C>(OP, total, part[w]);
      if (p.splits == 1) ew_store<T>(static_cast<T *>(p.out), o, total);
      else static_cast<C *>(p.partial)[blockIdx.y * p.n_out + o] = total;
    }
    __syncthreads();
  }
}

// ROW mapping for many short contiguous rows: one WARP per output.  A row of a few
// tens of kilobytes is eight loads per thread of a 256-thread CTA, and the two
// block barriers and the serial tail of the CTA-per-row kernel then cost as much
// as the row itself (bf16 [16000, 16400] summed over rows: 0.59 of the HBM copy
// rate where f32, with rows twice as long in bytes, reached 0.98).  Here a warp
// walks its row in 512-byte steps and finishes with shuffles alone.
template <typename T, int OP>
__global__ void __launch_bounds__(256, 6) reduce_roww_kernel(const ReduceOpParams p) {
  using C = typename EwTraits<T>::C;
  constexpr int V = 16 / sizeof(T);
  const T *a = static_cast<const T *>(p.a);
  const int lane = threadIdx.x & 31;
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * 8;
  for (int64_t o = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); o < p.n_out; o += nwarps) {
    const T *run = a + p.a_off + unravel(o, p.nkept, p.kept_shape, p.kept_strides);
    const int64_t mis = (reinterpret_cast<uintptr_t>(run) / sizeof(T)) % V;
    const int64_t head = min((V - mis) % V, p.n_red);
    const int64_t nv = (p.n_red - head) / V;
    C acc = reduce_identity<C>(OP);
    if (lane < head) acc = reduce_combine<C>(OP, acc, ew_load<T>(run, lane));
    const EwVec<T> *vec = reinterpret_cast<const EwVec<T> *>(run + head);
    C lane_acc[4] = {acc, reduce_identity<C>(OP), reduce_identity<C>(OP), reduce_identity<C>(OP)};  // see reduce_row_kernel
    // eight loads in flight per thread and six CTAs per SM: a warp alone on its row is bound by
    // the latency of its loads, and 8 x 48 warps hold more of them than 4 x 64
#pragma unroll 8
    for (int64_t i = lane; i < nv; i += 32) {
      const EwVec<T> x = vec[i];
#pragma unroll
      for (int e = 0; e < V; ++e) lane_acc[e & 3] = reduce_combine<C>(OP, lane_acc[e & 3], ew_load<T>(x.v, e));
    }
    acc = reduce_combine<C>(OP, reduce_combine<C>(OP, lane_acc[0], lane_acc[1]), reduce_combine<C>(OP, lane_acc[2], lane_acc[3]));
    for (int64_t r = head + nv * V + lane; r < p.n_red; r += 32) acc = reduce_combine<C>(OP, acc, ew_load<T>(run, r));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc = reduce_combine<C>(OP, acc, shfl_down<C>(acc, d));
    if (lane == 0) ew_store<T>(static_cast<T *>(p.out), o, acc);
  }
}

template <typename T, int OP>
__global__ void __launch_bounds__(256) reduce_col_kernel(const ReduceOpParams p) {
  using C = typename EwTraits<T>::C;
  const T *a = static_cast<const T *>(p.a);
  const int64_t r0 = blockIdx.y * p.chunk, r1 = min(r0 + p.chunk, p.n_red);
  for (int64_t o = blockIdx.x * 256ll + threadIdx.x; o < p.n_out; o += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t base = p.a_off + unravel(o, p.nkept, p.kept_shape, p.kept_strides);
    C acc = reduce_identity<C>(OP);
    if (p.nred == 1) {
      const int64_t rs = p.red_strides[0];
      for (int64_t r = r0; r < r1; ++r) acc = reduce_combine<C>(OP, acc, ew_load<T>(a, base + r * rs));
    } else {
      for (int64_t r = r0; r < r1; ++r) acc = reduce_combine<C>(OP, acc, ew_load<T>(a, base + unravel(r, p.nred, p.red_shape, p.red_strides)));
    }
    if (p.splits == 1) ew_store<T>(static_cast<T *>(p.out), o, acc);
    else static_cast<C *>(p.partial)[blockIdx.y * p.n_out + o] = acc;
  }
}

// COL mapping, 16 bytes wide: the kept elements are one contiguous run, so a
// thread owns 16 / sizeof(T) neighbouring outputs and every load is a full
// vector (the host checks alignment and that every reduced stride keeps it).
template <typename T, int OP>
__global__ void __launch_bounds__(256) reduce_colv_kernel(const ReduceOpParams p) {
  using C = typename EwTraits<T>::C;
  constexpr int V = 16 / sizeof(T);
  const T *a = static_cast<const T *>(p.a);
  const int64_t r0 = blockIdx.y * p.chunk, r1 = min(r0 + p.chunk, p.n_red);
  const int64_t nvec = p.n_out / V;
  for (int64_t ov = blockIdx.x * 256ll + threadIdx.x; ov < nvec; ov += static_cast<int64_t>(gridDim.x) * 256) {
    const T *col = a + p.a_off + ov * V;
    C acc[V];
#pragma unroll
    for (int e = 0; e < V; ++e) acc[e] = reduce_identity<C>(OP);
    if (p.nred == 1) {
      const int64_t rs = p.red_strides[0];
#pragma unroll 4
      for (int64_t r = r0; r < r1; ++r) {
        const EwVec<T> x = *reinterpret_cast<const EwVec<T> *>(col + r * rs);
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = reduce_combine<C>(OP, acc[e], ew_load<T>(x.v, e));
      }
    } else {
      for (int64_t r = r0; r < r1; ++r) {
        const EwVec<T> x = *reinterpret_cast<const EwVec<T> *>(col + unravel(r, p.nred, p.red_shape, p.red_strides));
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] = reduce_combine<C>(OP, acc[e], ew_load<T>(x.v, e));
      }
    }
    if (p.splits == 1) {
      EwVec<T> o;
#pragma unroll
      for (int e = 0; e < V; ++e) ew_store<T>(o.v, e, acc[e]);
      reinterpret_cast<EwVec<T> *>(p.out)[ov] = o;
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) static_cast<C *>(p.partial)[blockIdx.y * p.n_out + ov * V + e] = acc[e];
    }
  }
}

template <typename T, int OP>
__global__ void __launch_bounds__(256) reduce_finish_kernel(const ReduceOpParams p) {
  using C = typename EwTraits<T>::C;
  const C *partial = static_cast<const C *>(p.partial);
  for (int64_t o = blockIdx.x * 256ll + threadIdx.x; o < p.n_out; o += static_cast<int64_t>(gridDim.x) * 256) {
    C acc = partial[o];
#pragma unroll 8  // the loads of a step are independent: eight of them in flight, not one
    for (int s = 1; s < p.splits; ++s) acc = reduce_combine<C>(OP, acc, partial[s * p.n_out + o]);
    ew_store<T>(static_cast<T *>(p.out), o, acc);
  }
}

// Few outputs, many slices (a sum over everything: one output, 1024 slices): a
// CTA per output, its threads across the slices, so that the last step costs a
// couple of loads per thread instead of a thousand one after another.
template <typename T, int OP>
__global__ void __launch_bounds__(256) reduce_finish_wide_kernel(const ReduceOpParams p) {
  using C = typename EwTraits<T>::C;
  __shared__ C part[8];
  const C *partial = static_cast<const C *>(p.partial);
  for (int64_t o = blockIdx.x; o < p.n_out; o += gridDim.x) {
    C acc = reduce_identity<C>(OP);
    for (int s = threadIdx.x; s < p.splits; s += 256) acc = reduce_combine<C>(OP, acc, partial[s * p.n_out + o]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc = reduce_combine<C>(OP, acc, shfl_down<C>(acc, d));
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      C total = part[0];
      for (int w = 1; w < 8; ++w) total = reduce_combine<C>(OP, total, part[w]);
      ew_store<T>(static_cast<T *>(p.out), o, total);
    }
    __syncthreads();
  }
}

}  // namespace oxm
