// SIMT kernels of the backend: the FFMA tile GEMM that reads any strided view
// directly, and the pack kernel that lays an arbitrary view out as K-major
// rows for the tensor-core path (splitting f32 into TF32 hi/lo parts on the way).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

#include "elem.cuh"
#include "gemm_tcgen05.cuh"

namespace oxm {

constexpr int kSimtMaxBatchDims = 6;

// Self-test of the bounded wait: one thread waits on a barrier that nothing
// will ever arrive on.  The wait must give up after `limit_ns`, record
// OXM_TIMEOUT in the status word and let the kernel return normally.
__global__ void bounded_wait_selftest_kernel(uint32_t *status, uint64_t limit_ns, uint32_t *gave_up) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    ptx::fence_barrier_init();
    WaitCtx wc{&abort_flag, status, limit_ns};
    const bool ok = bounded_wait(ptx::smem_u32(&bar), 0, wc);
    *gave_up = ok ? 0u : 1u;
  }
}


// ---------------------------------------------------------------------------
// FFMA tile GEMM.  A square output tile per 256-thread CTA, the contraction
// walked in ascending k in blocks of 16.  Reads A, B and writes
// C through signed element strides, so transposed / narrowed / flipped views
// and broadcast batch dims need no preparation.
//
// The loads of the next two blocks are in flight while a block is multiplied
// (they wait in registers until the shared-memory tiles are free again), so a
// CTA pays the latency of global memory once, not once per block.
//
// Products with too few tiles to fill the GPU split the contraction over the
// `ksplit` CTAs of a thread-block cluster (the CTAs of one cluster are
// consecutive blocks of the grid).  Each adds up its own range of k; the
// partial tiles meet in the first CTA's registers through distributed shared
// memory, always in rank order, so the result does not depend on timing.
// With ksplit = 1 every output element is one fp32 chain in ascending k.
// ---------------------------------------------------------------------------
struct SimtParams {
  const void *a, *b;
  void *out;
  int32_t dtype, out_dtype;
  int32_t M, N, K;
  int32_t tiles_m, tiles_n;
  int32_t ksplit, kchunk;            // CTAs per tile along k (the cluster size); k elements per CTA, a multiple of 16
  int64_t a_off, b_off, o_off;       // elements
  int64_t a_rs, a_cs, b_rs, b_cs, o_rs, o_cs;
  int32_t nbd;
  int32_t bdims[kSimtMaxBatchDims];
  int64_t a_bs[kSimtMaxBatchDims], b_bs[kSimtMaxBatchDims], o_bs[kSimtMaxBatchDims];
  Epilogue epi;
};

// TS x TS output tile per 256-thread CTA (TS = 64: 4 x 4 per thread; TS = 32:
// 2 x 2 per thread, for products with too few 64-wide tiles to fill the GPU).
//
// The contraction is staged in blocks of BK = 2048 / TS elements (64 for the
// small tile): one block is 8 elements of each operand per thread, fetched into
// registers while the previous block is being multiplied, so a CTA that owns
// 128 elements of k (the usual share when a cluster splits the contraction)
// synchronises four times in all.  Per thread, the addresses of its 8 elements
// differ by a constant, so the loop adds one stride per block and no index is
// rebuilt.  Every output element accumulates its products in ascending k, and a
// cluster's partial tiles are added in rank order: the result does not depend
// on the tile size or on who does the adding.
template <int TS>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const SimtParams p) {
  constexpr int BK = 2048 / TS, TT = TS / 16, PER_THREAD = 8;
  static_assert(TS * BK == 256 * PER_THREAD, "eight elements of each operand per thread and block");
  // Row pitch: a multiple of the vector load's width that is not a multiple of 32 banks (a
  // k-fastest operand is written one column at a time: 2 floats of padding keep that to two-way
  // conflicts for the small tile, 4 floats to four-way for the large one).
  constexpr int PITCH = TS + (TT == 4 ? 4 : 2);
  __shared__ __align__(16) float As[BK][PITCH];
  __shared__ __align__(16) float Bs[BK][PITCH];
  __shared__ __align__(16) float red[TS][PITCH];  // a CTA's partial tile, read by the other CTAs of its cluster

  const int32_t krank = p.ksplit > 1 ? static_cast<int32_t>(blockIdx.x % p.ksplit) : 0;
  const int64_t tile = p.ksplit > 1 ? blockIdx.x / p.ksplit : blockIdx.x;
  const int32_t tpb = p.tiles_m * p.tiles_n;
  int32_t batch = static_cast<int32_t>(tile / tpb);
  const int32_t t = static_cast<int32_t>(tile % tpb);
  const int32_t m0 = (t / p.tiles_n) * TS;
  const int32_t n0 = (t % p.tiles_n) * TS;
  int64_t a_off = p.a_off, b_off = p.b_off, o_off = p.o_off;
  for (int d = p.nbd - 1; d >= 0; --d) {
    const int32_t idx = batch % p.bdims[d];
    batch /= p.bdims[d];
    a_off += idx * p.a_bs[d];
    b_off += idx * p.b_bs[d];
    o_off += idx * p.o_bs[d];
  }
  const int32_t k_begin = krank * p.kchunk;
  const int32_t k_end = min(p.K, k_begin + p.kchunk);

  const int tx = threadIdx.x & 15;  // column group
  const int ty = threadIdx.x >> 4;  // row group
  float acc[TT][TT];
#pragma unroll
  for (int i = 0; i < TT; ++i)
#pragma unroll
    for (int j = 0; j < TT; ++j) acc[i][j] = 0.f;

  // Element r of this thread in a block of A (TS rows x BK of k) is e = tid + 256 r; the faster
  // index of e follows the operand's unit stride, so a warp reads consecutive addresses.
  //   k fastest:   row = e / BK = row0 + (256 / BK) r,  k = e % BK = kk0          (the same k for every r)
  //   row fastest: row = e % TS = row0,                 k = e / TS = kk0 + (256 / TS) r
  const bool a_kfast = p.a_cs == 1, b_kfast = p.b_rs == 1;
  const int a_row0 = a_kfast ? threadIdx.x / BK : threadIdx.x % TS, a_kk0 = a_kfast ? threadIdx.x % BK : threadIdx.x / TS;
  const int b_col0 = b_kfast ? threadIdx.x / BK : threadIdx.x % TS, b_kk0 = b_kfast ? threadIdx.x % BK : threadIdx.x / TS;
  const int a_drow = a_kfast ? 256 / BK : 0, a_dk = a_kfast ? 0 : 256 / TS;
  const int b_dcol = b_kfast ? 256 / BK : 0, b_dk = b_kfast ? 0 : 256 / TS;
  const int64_t a_step = static_cast<int64_t>(a_drow) * p.a_rs + static_cast<int64_t>(a_dk) * p.a_cs;  // from element r to r + 1
  const int64_t b_step = static_cast<int64_t>(b_dcol) * p.b_cs + static_cast<int64_t>(b_dk) * p.b_rs;
  int64_t a_idx = a_off + static_cast<int64_t>(m0 + a_row0) * p.a_rs + static_cast<int64_t>(k_begin + a_kk0) * p.a_cs;
  int64_t b_idx = b_off + static_cast<int64_t>(n0 + b_col0) * p.b_cs + static_cast<int64_t>(k_begin + b_kk0) * p.b_rs;
  const int64_t a_blk = static_cast<int64_t>(BK) * p.a_cs, b_blk = static_cast<int64_t>(BK) * p.b_rs;  // from block to block
  const bool f32 = p.dtype == 0;

  float ra[PER_THREAD], rb[PER_THREAD];
  auto fetch = [&](int32_t k0) {
#pragma unroll
    for (int r = 0; r < PER_THREAD; ++r) {
      const bool a_ok = m0 + a_row0 + r * a_drow < p.M && k0 + a_kk0 + r * a_dk < k_end;
      const bool b_ok = n0 + b_col0 + r * b_dcol < p.N && k0 + b_kk0 + r * b_dk < k_end;
      if (f32) {
        ra[r] = a_ok ? __ldg(static_cast<const float *>(p.a) + a_idx + r * a_step) : 0.f;
        rb[r] = b_ok ? __ldg(static_cast<const float *>(p.b) + b_idx + r * b_step) : 0.f;
      } else {
        ra[r] = a_ok ? load_elem(p.a, p.dtype, a_idx + r * a_step) : 0.f;
        rb[r] = b_ok ? load_elem(p.b, p.dtype, b_idx + r * b_step) : 0.f;
      }
    }
    a_idx += a_blk;
    b_idx += b_blk;
  };
  if (k_begin < k_end) fetch(k_begin);
  for (int32_t k0 = k_begin; k0 < k_end; k0 += BK) {
#pragma unroll
    for (int r = 0; r < PER_THREAD; ++r) {
      As[a_kk0 + r * a_dk][a_row0 + r * a_drow] = ra[r];
      Bs[b_kk0 + r * b_dk][b_col0 + r * b_dcol] = rb[r];
    }
    __syncthreads();
    if (k0 + BK < k_end) fetch(k0 + BK);  // in flight while this block is multiplied
    // all BK steps, whatever is left of k: the fetch wrote zeros beyond k_end, and a loop of known
    // length lets the compiler run the shared-memory loads well ahead of the FMAs that use them
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      // one vector load per operand: with scalar loads the 2 x 2 tile issues a load per FMA
      float av[TT], bv[TT];
      if constexpr (TT == 4) {
        const float4 a4 = *reinterpret_cast<const float4 *>(&As[kk][ty * TT]);
        const float4 b4 = *reinterpret_cast<const float4 *>(&Bs[kk][tx * TT]);
        av[0] = a4.x; av[1] = a4.y; av[2] = a4.z; av[3] = a4.w;
        bv[0] = b4.x; bv[1] = b4.y; bv[2] = b4.z; bv[3] = b4.w;
      } else {
        const float2 a2 = *reinterpret_cast<const float2 *>(&As[kk][ty * TT]);
        const float2 b2 = *reinterpret_cast<const float2 *>(&Bs[kk][tx * TT]);
        av[0] = a2.x; av[1] = a2.y;
        bv[0] = b2.x; bv[1] = b2.y;
      }
#pragma unroll
      for (int i = 0; i < TT; ++i)
#pragma unroll
        for (int j = 0; j < TT; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }

  if (p.ksplit > 1) {
    // Every CTA of the cluster leaves its partial tile in its own shared memory; CTA r then adds
    // up and stores the rows r, r + ksplit, ... of the tile, taking the partial sums in rank
    // order (its own included) so that the result is the one a single adder would produce.
#pragma unroll
    for (int i = 0; i < TT; ++i)
#pragma unroll
      for (int j = 0; j < TT; ++j) red[ty * TT + i][tx * TT + j] = acc[i][j];
    ptx::cluster_arrive();
    ptx::cluster_wait();
    for (int e = threadIdx.x; e < TS * TS; e += 256) {
      const int row = e / TS, col = e % TS;
      if (row % p.ksplit != krank) continue;
      const int32_t gm = m0 + row, gn = n0 + col;
      if (gm >= p.M || gn >= p.N) continue;
      // all the remote loads first, then the additions: a load followed by the addition that needs
      // it would hold the next load back for a full trip through distributed shared memory
      const uint32_t local = ptx::smem_u32(&red[row][col]);
      float v[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        v[r] = 0.f;
        if (r < p.ksplit)
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v[r]) : "r"(ptx::mapa_shared(local, static_cast<uint32_t>(r))) : "memory");
      }
      float sum = v[0];
#pragma unroll
      for (int r = 1; r < 8; ++r)
        if (r < p.ksplit) sum += v[r];
      const int64_t idx = o_off + gm * p.o_rs + gn * p.o_cs;
      if (p.epi.any) sum = apply_epilogue(p.epi, sum, gn, p.out, p.out_dtype, idx);
      store_elem(p.out, p.out_dtype, idx, sum);
    }
    ptx::cluster_arrive();
    ptx::cluster_wait();  // nobody leaves while its shared memory may still be read
    return;
  }

#pragma unroll
  for (int i = 0; i < TT; ++i) {
    const int32_t gm = m0 + ty * TT + i;
    if (gm >= p.M) continue;
#pragma unroll
    for (int j = 0; j < TT; ++j) {
      const int32_t gn = n0 + tx * TT + j;
      if (gn < p.N) {
        const int64_t idx = o_off + gm * p.o_rs + gn * p.o_cs;
        float r = acc[i][j];
        if (p.epi.any) r = apply_epilogue(p.epi, r, gn, p.out, p.out_dtype, idx);
        store_elem(p.out, p.out_dtype, idx, r);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Pack: copy a [batch..., rows, K] view into contiguous K-major rows
//   dst[b][r][kp],  kp in [0, Kp), zero padded past K.
// mode 0: 16-bit or 32-bit copy.
// mode 1: f32 -> three TF32 terms per 32-wide K block, laid out so that one
//         ordinary TF32 GEMM over the tripled K computes the 3xTF32 product:
//           A side: [hi | hi | lo]      B side: [hi | lo | hi]
//         hi = tf32(x) (round to nearest), lo = tf32(x - hi).  An infinity
//         or NaN is written as [x | 0 | 0] on both sides.
// A 32x32 tile goes through shared memory so that both the read and the write
// are coalesced whichever of (row, k) is the source's unit stride.
// ---------------------------------------------------------------------------
struct PackParams {
  const void *src;
  void *dst;
  int32_t elt;        // bytes per element: 1, 2 or 4
  int32_t mode;       // 0 copy, 1 tf32 split (A side), 2 tf32 split (B side)
  int32_t rows, K, Kp;   // Kp: padded K of the SOURCE blocks (multiple of 32 in split mode)
  int64_t dst_row_elems; // elements per destination row (Kp, or 3*Kp in split mode)
  int64_t src_off, src_rs, src_ks;
  int32_t nbd;
  int32_t bdims[kSimtMaxBatchDims];
  int64_t src_bs[kSimtMaxBatchDims];
  int32_t tiles_r, tiles_k;
};

// ---------------------------------------------------------------------------
// Scale atoms of the block-scaled product.  The E8M0 scales of one operand
// (a view: row r, contraction block kb, any strides, broadcast batch dims left
// out) are regrouped into the 512-byte atoms the tensor core's scale copy
// takes: atom (batch, r / 128, kb / 4) holds, at byte (r % 32) * 16 +
// (r % 128) / 32 * 4 + kb % 4, the scale of row r and block kb.  Atoms are
// ordered [batch][stage][row group] (the atoms of neighbouring row groups at
// one stage lie side by side: one load fetches all a tile needs); positions
// beyond the operand hold 0x7F
// (2^0), which only ever multiplies the zeros the loads fill in there.
// ---------------------------------------------------------------------------
struct SfParams {
  const uint8_t *src;
  uint32_t *dst;
  int64_t src_off, src_rs, src_ks;
  int32_t rows, kblocks;   // extents of the view
  int32_t row_groups, stages;  // ceil(rows / 128), ceil(kblocks / 4)
  int32_t nbd;
  int32_t bdims[kSimtMaxBatchDims];
  int64_t src_bs[kSimtMaxBatchDims];
  int64_t total_words;
};

__global__ void __launch_bounds__(256) mx_scale_atoms_kernel(const SfParams p) {
  for (int64_t w = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; w < p.total_words;
       w += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int32_t within = static_cast<int32_t>(w & 127);
    int64_t atom = w >> 7;
    const int32_t rg = static_cast<int32_t>(atom % p.row_groups);
    atom /= p.row_groups;
    const int32_t stage = static_cast<int32_t>(atom % p.stages);
    int64_t batch = atom / p.stages;
    const int32_t r = rg * 128 + (within & 3) * 32 + (within >> 2);
    int64_t off = p.src_off;
    for (int d = p.nbd - 1; d >= 0; --d) {
      off += (batch % p.bdims[d]) * p.src_bs[d];
      batch /= p.bdims[d];
    }
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int32_t kb = stage * 4 + i;
      const uint32_t byte = (r < p.rows && kb < p.kblocks) ? p.src[off + static_cast<int64_t>(r) * p.src_rs + static_cast<int64_t>(kb) * p.src_ks] : 0x7Fu;
      word |= byte << (8 * i);
    }
    p.dst[w] = word;
  }
}

__device__ __forceinline__ float tf32_round(float x) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}

__global__ void __launch_bounds__(256) pack_kernel(const PackParams p) {
  __shared__ uint32_t tile[32][33];
  const int64_t blk = blockIdx.x;
  const int32_t tpb = p.tiles_r * p.tiles_k;
  int32_t batch = static_cast<int32_t>(blk / tpb);
  const int32_t t = static_cast<int32_t>(blk % tpb);
  const int32_t r0 = (t / p.tiles_k) * 32;
  const int32_t k0 = (t % p.tiles_k) * 32;
  const int64_t dst_batch = static_cast<int64_t>(batch) * p.rows * p.dst_row_elems;
  int64_t src_off = p.src_off;
  for (int d = p.nbd - 1; d >= 0; --d) {
    const int32_t idx = batch % p.bdims[d];
    batch /= p.bdims[d];
    src_off += idx * p.src_bs[d];
  }
  const int x = threadIdx.x & 31, y = threadIdx.x >> 5;  // 32 x 8
  const bool k_fast = (p.src_ks == 1) || (p.src_rs != 1);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rr = k_fast ? (y + i * 8) : x;
    const int kk = k_fast ? x : (y + i * 8);
    const int32_t gr = r0 + rr, gk = k0 + kk;
    uint32_t v = 0;
    if (gr < p.rows && gk < p.K) {
      const int64_t idx = src_off + gr * p.src_rs + gk * p.src_ks;
      v = p.elt == 4   ? static_cast<const uint32_t *>(p.src)[idx]
          : p.elt == 2 ? static_cast<uint32_t>(static_cast<const uint16_t *>(p.src)[idx])
                       : static_cast<uint32_t>(static_cast<const uint8_t *>(p.src)[idx]);
    }
    tile[rr][kk] = v;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rr = y + i * 8, kk = x;
    const int32_t gr = r0 + rr, gk = k0 + kk;
    if (gr >= p.rows || gk >= p.Kp) continue;
    const uint32_t v = tile[rr][kk];
    if (p.mode == 0) {
      const int64_t o = dst_batch + static_cast<int64_t>(gr) * p.dst_row_elems + gk;
      if (p.elt == 4) static_cast<uint32_t *>(p.dst)[o] = v;
      else if (p.elt == 2) static_cast<uint16_t *>(p.dst)[o] = static_cast<uint16_t>(v);
      else static_cast<uint8_t *>(p.dst)[o] = static_cast<uint8_t>(v);
    } else {
      const float xv = __uint_as_float(v);
      float hi = tf32_round(xv);
      float lo = tf32_round(xv - hi);
      if (!isfinite(hi)) {  // inf / NaN, or a finite value that rounds past the largest tf32
        hi = xv;
        lo = 0.f;
      }
      float second = (p.mode == 1) ? hi : lo, third = (p.mode == 1) ? lo : hi;
      // An infinity or NaN must meet its partner exactly once, as in IEEE
      // arithmetic: it goes into the first block alone, where it multiplies the
      // partner's leading term (inf * 2 = inf, inf * 0 = NaN), and the blocks
      // that would pair it with a correction term (inf * 0 = NaN, or an
      // infinity of the other sign) hold zero.
      if (!isfinite(xv)) second = third = 0.f;
      // k0 is a multiple of 32, so this tile is exactly one 32-wide K block.
      const int64_t o = dst_batch + static_cast<int64_t>(gr) * p.dst_row_elems + 3ll * k0 + kk;
      float *d = static_cast<float *>(p.dst);
      d[o] = hi;
      d[o + 32] = second;
      d[o + 64] = third;
    }
  }
}

// ---------------------------------------------------------------------------
// Split-K reduction: out[b][m][n] = sum over s of ws[s][b][m][n] (f32, added in
// ascending s with round-to-nearest), rounded to the output dtype and written
// through the output's strides.
// ---------------------------------------------------------------------------
struct ReduceParams {
  const float *ws;
  void *out;
  int32_t out_dtype;  // 0 f32, 6 bf16, 7 f16
  int32_t splits, M, N;
  int64_t split_stride;  // elements between partial-sum slabs
  int64_t total;         // nbatch * M * N
  int64_t o_off, o_rs, o_cs;
  int32_t nbd;
  int32_t bdims[kSimtMaxBatchDims];
  int64_t o_bs[kSimtMaxBatchDims];
  Epilogue epi;
};

__global__ void __launch_bounds__(256) splitk_reduce_kernel(const ReduceParams p) {
  const int64_t mn = static_cast<int64_t>(p.M) * p.N;
  // Four neighbours of one output row per thread when rows and slabs allow 16-byte loads.
  const bool vec = (p.N % 4 == 0) && (p.split_stride % 4 == 0) && (reinterpret_cast<uintptr_t>(p.ws) % 16 == 0);
  const int64_t step = vec ? 4 : 1;
  const int64_t units = p.total / step;
  const int esz = p.out_dtype == 0 ? 4 : (p.out_dtype >= 8 ? 1 : 2);
  for (int64_t u = blockIdx.x * 256ll + threadIdx.x; u < units; u += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t i = u * step;
    float acc[4];
    if (vec) {
      float4 t = *reinterpret_cast<const float4 *>(p.ws + i);
      acc[0] = t.x; acc[1] = t.y; acc[2] = t.z; acc[3] = t.w;
      for (int s = 1; s < p.splits; ++s) {
        t = *reinterpret_cast<const float4 *>(p.ws + i + s * p.split_stride);
        acc[0] += t.x; acc[1] += t.y; acc[2] += t.z; acc[3] += t.w;
      }
    } else {
      acc[0] = p.ws[i];
      for (int s = 1; s < p.splits; ++s) acc[0] += p.ws[i + s * p.split_stride];
    }
    int64_t batch = i / mn;
    const int64_t r = i - batch * mn;
    const int32_t col = static_cast<int32_t>(r % p.N);
    int64_t off = p.o_off + (r / p.N) * p.o_rs + col * p.o_cs;
    for (int d = p.nbd - 1; d >= 0; --d) {
      off += (batch % p.bdims[d]) * p.o_bs[d];
      batch /= p.bdims[d];
    }
    if (p.epi.any) {
      for (int e = 0; e < step; ++e) acc[e] = apply_epilogue(p.epi, acc[e], col + e, p.out, p.out_dtype, off + e * p.o_cs);
    }
    uint8_t *dst = static_cast<uint8_t *>(p.out) + off * esz;
    if (vec && p.o_cs == 1 && p.out_dtype == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0) {
      *reinterpret_cast<float4 *>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    } else if (vec && p.o_cs == 1 && (p.out_dtype == 6 || p.out_dtype == 7) && reinterpret_cast<uintptr_t>(dst) % 8 == 0) {
      uint2 w;
      if (p.out_dtype == 6) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[0], acc[1]), hi = __floats2bfloat162_rn(acc[2], acc[3]);
        w.x = *reinterpret_cast<const uint32_t *>(&lo); w.y = *reinterpret_cast<const uint32_t *>(&hi);
      } else {
        const __half2 lo = __floats2half2_rn(acc[0], acc[1]), hi = __floats2half2_rn(acc[2], acc[3]);
        w.x = *reinterpret_cast<const uint32_t *>(&lo); w.y = *reinterpret_cast<const uint32_t *>(&hi);
      }
      *reinterpret_cast<uint2 *>(dst) = w;
    } else {
      for (int e = 0; e < step; ++e) store_elem(p.out, p.out_dtype, off + e * p.o_cs, acc[e]);
    }
  }
}

// ---------------------------------------------------------------------------
// Strided gather into contiguous storage: the device side of Tensor::contiguous.
// ---------------------------------------------------------------------------
struct CopyParams {
  const void *src;
  void *dst;
  int32_t elt, ndim;
  int64_t shape[8], strides[8];
  int64_t src_off, dst_off, n;
};

__global__ void __launch_bounds__(256) copy_strided_kernel(const CopyParams p) {
  for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < p.n; i += static_cast<int64_t>(gridDim.x) * 256) {
    int64_t rem = i, off = p.src_off;
    for (int d = p.ndim - 1; d >= 0; --d) {
      off += (rem % p.shape[d]) * p.strides[d];
      rem /= p.shape[d];
    }
    switch (p.elt) {
      case 1: static_cast<uint8_t *>(p.dst)[p.dst_off + i] = static_cast<const uint8_t *>(p.src)[off]; break;
      case 2: static_cast<uint16_t *>(p.dst)[p.dst_off + i] = static_cast<const uint16_t *>(p.src)[off]; break;
      case 4: static_cast<uint32_t *>(p.dst)[p.dst_off + i] = static_cast<const uint32_t *>(p.src)[off]; break;
      default: static_cast<uint64_t *>(p.dst)[p.dst_off + i] = static_cast<const uint64_t *>(p.src)[off]; break;
    }
  }
}

// ---------------------------------------------------------------------------
// Seeded synthetic data written straight into device memory (benchmarks).
// Counter based: element i depends only on (key, i).  dist 0: U(-1,1);
// dist 1: N(0,1) * scale by Box-Muller.
// ---------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

__global__ void __launch_bounds__(256) fill_kernel(void *dst, int dtype, int64_t n, uint64_t key, int dist, float scale) {
  for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * 256) {
    const uint64_t h1 = splitmix64(key + 2ull * static_cast<uint64_t>(i));
    float v;
    if (dist == 0) {
      v = 2.0f * (static_cast<float>(h1 >> 40) * (1.0f / 16777216.0f)) - 1.0f;
    } else {
      const uint64_t h2 = splitmix64(key + 2ull * static_cast<uint64_t>(i) + 1ull);
      const float u1 = (static_cast<float>(h1 >> 40) + 1.0f) * (1.0f / 16777216.0f);
      const float u2 = static_cast<float>(h2 >> 40) * (1.0f / 16777216.0f);
      v = sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2) * scale;
    }
    store_elem(dst, dtype, i, v);
  }
}

}  // namespace oxm
