// The tensor-core GEMM of the oxmera B200 backend: C[b] = A[b] * B[b] with
// fp32 accumulation in tensor memory.
//
// Shape of the kernel
//   - persistent: one CTA (or one CTA pair) per SM walks a static tile list;
//   - warp specialised: warp 0 issues TMA loads, warp 1 owns tensor memory
//     and issues tcgen05.mma, warps 2..5 drain accumulators to global memory;
//   - operands are staged by TMA into 128-byte-swizzled shared-memory tiles,
//     STAGES deep, handed over with mbarriers;
//   - two accumulators live in tensor memory so the epilogue of tile i
//     overlaps the main loop of tile i+1;
//   - either operand may be K-major (contraction dim contiguous) or MN-major
//     (row/column dim contiguous): the transposed views of a linear layer's
//     backward need no copy;
//   - PAIR = 1 runs cta_group::2: two CTAs of a cluster share one 256-row tile,
//     each staging its own A rows and its own half of B (no multicast);
//   - KIND = 3 is the block-scaled fp8 product (MX: one E8M0 scale per 32
//     contraction elements of every operand row): the scales travel beside the
//     operands, 512 bytes per 128 rows and stage, and the MMA warp copies them
//     into spare tensor-memory columns ahead of each stage's MMAs.
//
// Every wait is bounded.  When a bound expires the waiter records
// OXM_TIMEOUT in the status word, raises the CTA's abort flag, and every role
// falls through to the common teardown, which frees tensor memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "elem.cuh"
#include "ptx.cuh"

namespace oxm {

constexpr int kMaxBatchDims = 6;
constexpr int kTileM = 128;        // accumulator rows per CTA (= TMEM lanes)
constexpr int kStageKBytes = 128;  // contraction bytes per pipeline stage (one swizzle row)
constexpr int kMmaKBytes = 32;     // contraction bytes per tcgen05.mma
// Threads per CTA: a TMA warp, an MMA warp, and four epilogue warps per group.
// Tiles of 256 columns and more get two groups, each draining half of the
// columns: the per-warp chain tensor memory -> registers -> staging -> bulk
// store is latency bound, so a second group halves the time per tile, which
// shows wherever the epilogue is exposed (one accumulator, or short contractions).
// With two groups the CTA is three warpgroups - {TMA, MMA, two idle warps} and
// the two epilogue groups - so that the first can hand most of its registers
// to the other two (setmaxnreg): an epilogue warp then holds a whole 256-column
// share of an accumulator in registers at once.
__host__ __device__ constexpr int gemm_epi_groups(int bn) { return bn >= 256 ? 2 : 1; }
__host__ __device__ constexpr int gemm_threads(int bn) { return gemm_epi_groups(bn) == 2 ? 384 : 192; }
constexpr int kProducerRegs = 56, kEpilogueRegs = 224;  // 128 x 56 + 256 x 224 = 64512 of the SM's 65536
constexpr uint32_t kStatusTimeout = 11;  // OXM_TIMEOUT

struct GemmParams {
  int32_t M, N, K;           // K counts elements of the staged operands
  int32_t bn;                // tile width in columns: a multiple of 32, at most the kernel's BN
  int32_t subn;              // columns per tcgen05.mma (bn, or bn / 2 for tiles wider than 256)
  int32_t tiles_m, tiles_n;  // tiles_m counts (kTileM * ctas-per-tile)-row blocks
  int32_t num_kb;            // contraction blocks per tile
  int32_t nbatch;
  int64_t num_tiles;
  int32_t nbd;               // output batch dims
  int32_t bdims[kMaxBatchDims];
  // The batch dims in the order the tiles walk them (last one fastest): the host puts last the dim
  // along which the fewest operand bytes change, so that tiles in flight share the larger operand.
  int32_t a_bmul[kMaxBatchDims];  // batch index -> operand batch coordinate
  int32_t b_bmul[kMaxBatchDims];
  int32_t o_bmul[kMaxBatchDims];  // batch index -> batch coordinate of the store tensor map
  int64_t o_bstride[kMaxBatchDims];  // elements
  void *out;
  int64_t out_rs, out_cs;  // elements
  int32_t out_dtype;       // 0 f32, 6 bf16, 7 f16, 8 / 9 fp8
  int32_t out_vec;         // rows may be written with 16-byte stores
  int32_t out_tma;         // the output is described by the store tensor map
  uint32_t idesc;
  uint32_t stage_tx;       // bytes one CTA's loads of one stage deliver (the boxes follow the tile's width; a short A gets a short box)
  uint32_t *status;
  uint64_t wait_limit_ns;
  // Split-K: the contraction is cut into `splits` chains of `kb_per_split`
  // blocks, each written to its own slab of a partial-sum workspace.
  int32_t splits, kb_per_split;
  int64_t tiles_per_split;
  int64_t split_ostride;  // elements
  // Stream-K: the last `sk_tiles` tiles are cut into
  // equal runs of contraction blocks, one run per CTA (or CTA pair), so that a
  // tile count that does not divide by the SM count still keeps every SM busy
  // to the end.  A run that starts inside a tile leaves its partial sums in
  // `sk_ws`; the run holding the tile's first block adds them and writes the
  // tile.  It evens out the block counts but staggers the CTAs along K, so
  // tiles that share an operand panel no longer read it at the same time and
  // L2 hits turn into HBM reads: the host uses it only where whole waves of
  // ordinary tiles run beside the shared-out ones.
  int64_t dp_tiles;       // tiles [0, dp_tiles) go round-robin as whole tiles; == num_tiles without stream-K
  int64_t sk_tiles;       // tiles [dp_tiles, dp_tiles + sk_tiles) are shared out by contraction block
  float *sk_ws;           // [run][cta of the pair][128][BN] partial sums
  uint32_t *sk_flags;     // [run][cta of the pair][8 epilogue warps]: the launch counter of the last publication
  uint32_t sk_epoch;      // this launch's counter value (never 0)
  int32_t group_m;        // tile rows walked together (L2 reuse)
  Epilogue epi;           // applied here unless the contraction is split (then by the reduction)
};

// Scales of the block-scaled kind, per stage: one 512-byte atom for this CTA's
// 128 rows of A, then the atoms (128 columns each, aligned to 128 in the
// matrix) that cover the tile's columns of B: at most three.  Tiles are 128,
// 192, 256 or 384 columns wide, so a tile (and the second sub-tile of a wide
// one) starts 0 or 64 columns into an atom and the MMA's scale address is that
// of the atom's first or third column (an odd column offset is refused by the
// hardware as a misaligned address).
constexpr int kSfAtomBytes = 512;
constexpr int kSfMaxBAtoms = 3;
constexpr int kSfStageBytes = kSfAtomBytes * (1 + kSfMaxBAtoms);
constexpr int kSfTmemCols = 16;  // 4 columns for A's scales + 12 for B's: one set
constexpr int kSfSets = 2;       // sets of scale columns at the top of tensor memory (480..511), taken in turn by stage
// B rows one CTA of the pair stages per sub-tile in the block-scaled instances: 96.  The
// two-accumulator tile is at most 192 columns wide (its accumulators sit at columns 0 and 256 of
// tensor memory), the one-accumulator tile at most 384 (two sub-tiles of 192); both leave columns
// 480..511 to the scales.
__host__ __device__ constexpr int mx_subc_cap(int) { return 96; }

// Tensor maps of the scale arrays: present only in the block-scaled instances.
template <int MX> struct SfMaps {};
template <> struct SfMaps<1> { CUtensorMap a, b; };

template <int BN, int STAGES, int PAIR, int MX = 0>
struct GemmSmem {
  // B rows staged by one CTA
  static constexpr int kBNC = MX ? mx_subc_cap(BN) * (BN > 256 ? 2 : 1) : PAIR ? BN / 2 : BN;
  static constexpr int kABytes = kTileM * kStageKBytes;
  static constexpr int kBBytes = kBNC * kStageKBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // one 32-row x 128-byte staging tile per epilogue warp for the TMA-store epilogue
  static constexpr int kStagingOffset = STAGES * kStageBytes;
  static constexpr int kStagingTile = 32 * kStageKBytes;
  static constexpr int kStagingBytes = 4 * gemm_epi_groups(BN) * kStagingTile;
  static constexpr int kSfOffset = kStagingOffset + kStagingBytes;
  static constexpr int kSfStage = MX ? kSfStageBytes : 0;
  static constexpr int kBarOffset = kSfOffset + STAGES * kSfStage;
  // full[STAGES] empty[STAGES] tmem_full[2] tmem_empty[2] teardown, then two u32 slots
  static constexpr int kNumBars = 2 * STAGES + 5;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16;
  static constexpr int kDynamic = kTotal + 1024;  // room to align the base to 1 KiB
};

// Shared-memory matrix descriptor for a 128-byte-swizzled tile.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(sbo_bytes >> 4) << 32;
  d |= 1ull << 46;  // descriptor version of this architecture
  d |= 2ull << 61;  // 128-byte swizzle
  return d;
}

// Descriptor of one scale atom for the shared -> tensor memory copy: 32 rows of
// 16 bytes, dense, no swizzle (groups of 8 rows 128 bytes apart).
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(16u >> 4) << 16;
  d |= static_cast<uint64_t>(128u >> 4) << 32;
  d |= 1ull << 46;
  return d;
}

struct WaitCtx {
  volatile int *abort_flag;  // shared memory, per CTA
  uint32_t *status;          // global status word
  uint64_t limit_ns;
};

// Wait for `parity` of `bar` with a time bound.  Returns false when the CTA is
// aborting (either this wait expired or another one did).  The clock is only
// consulted after a few hundred failed polls: reading %globaltimer costs a
// sizeable fraction of a microsecond, which a wait that data in flight is
// about to satisfy must not pay.
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, const WaitCtx &w) {
  for (int i = 0; i < 512; ++i)
    if (ptx::mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (ptx::mbar_try_wait(bar, parity)) return true;
    if (*w.abort_flag) return false;
    if (ptx::globaltimer_ns() - t0 > w.limit_ns) {
      *w.abort_flag = 1;
      atomicCAS(w.status, 0u, kStatusTimeout);
      return false;
    }
  }
}

struct TileCoord {
  int32_t m_blk, n_blk;
  int32_t a_batch, b_batch;
  int32_t kb0, nkb;  // contraction blocks [kb0, kb0 + nkb) of this tile
  int32_t o_batch;   // batch coordinate of the store tensor map
  int64_t o_off;
};

__device__ __forceinline__ TileCoord decode_tile(const GemmParams &p, int64_t tile) {
  TileCoord c;
  const int32_t split = static_cast<int32_t>(tile / p.tiles_per_split);
  tile -= split * p.tiles_per_split;
  c.kb0 = split * p.kb_per_split;
  c.nkb = min(p.kb_per_split, p.num_kb - c.kb0);
  const int32_t tpb = p.tiles_m * p.tiles_n;
  int32_t batch = static_cast<int32_t>(tile / tpb);
  const int32_t t = static_cast<int32_t>(tile - static_cast<int64_t>(batch) * tpb);
  c.o_batch = split * p.nbatch;
  // Walk GROUP_M tile rows at a time so that concurrently resident CTAs share
  // A and B panels in L2.
  const int32_t GROUP_M = p.group_m;
  const int32_t gt = GROUP_M * p.tiles_n;
  const int32_t g = t / gt;
  const int32_t first = g * GROUP_M;
  const int32_t gsz = min(GROUP_M, p.tiles_m - first);
  const int32_t r = t - g * gt;
  c.m_blk = first + r % gsz;
  c.n_blk = r / gsz;
  c.a_batch = 0;
  c.b_batch = 0;
  c.o_off = static_cast<int64_t>(split) * p.split_ostride;
  for (int d = p.nbd - 1; d >= 0; --d) {
    const int32_t idx = batch % p.bdims[d];
    batch /= p.bdims[d];
    c.a_batch += idx * p.a_bmul[d];
    c.b_batch += idx * p.b_bmul[d];
    c.o_batch += idx * p.o_bmul[d];
    c.o_off += static_cast<int64_t>(idx) * p.o_bstride[d];
  }
  return c;
}

// The sequence of work items of one CTA (or CTA pair): first its run of the
// stream-K region, then whole tiles round-robin.  Every role of the CTA walks
// the same sequence.
struct WorkItem {
  int64_t tile;
  int32_t kb0, nkb;  // blocks [kb0, kb0 + nkb) of the tile's own contraction range (-1: take the tile's)
  int32_t kind;      // 0 whole tile, 1 owner (holds the first block, adds the others' partial sums), 2 contributor
};

// Run `r` of `runs` over `units` contraction blocks: equal shares, the first `units % runs` one longer.
__device__ __forceinline__ void sk_run(int64_t units, int64_t runs, int64_t r, int64_t &begin, int64_t &end) {
  const int64_t base = units / runs, rem = units % runs;
  begin = r * base + min(r, rem);
  end = begin + base + (r < rem ? 1 : 0);
}

struct WorkIter {
  int64_t u, e;    // stream-K blocks still to do
  int64_t dp;      // next whole tile
  int64_t stride;  // CTAs (or pairs) in the grid
  // Pair `who` takes run (stride - 1 - who): a run's partial sums are then always needed by a
  // higher-numbered run, i.e. by a lower-numbered CTA, which was launched no later.
  __device__ __forceinline__ void init(const GemmParams &p, int64_t who, int64_t stride_) {
    stride = stride_;
    dp = who;
    u = e = 0;
    if (p.sk_tiles > 0) sk_run(p.sk_tiles * p.num_kb, stride, stride - 1 - who, u, e);
  }
  __device__ __forceinline__ bool next(const GemmParams &p, WorkItem &w) {
    if (u < e) {
      const int64_t t = u / p.num_kb;
      w.tile = p.dp_tiles + t;
      w.kb0 = static_cast<int32_t>(u - t * p.num_kb);
      w.nkb = static_cast<int32_t>(min(static_cast<int64_t>(p.num_kb - w.kb0), e - u));
      w.kind = w.nkb == p.num_kb ? 0 : (w.kb0 == 0 ? 1 : 2);
      u += w.nkb;
      return true;
    }
    if (dp < p.dp_tiles) {
      w.tile = dp;
      w.kb0 = -1; w.nkb = -1; w.kind = 0;
      dp += stride;
      return true;
    }
    return false;
  }
};

__device__ __forceinline__ TileCoord decode_item(const GemmParams &p, const WorkItem &w) {
  TileCoord c = decode_tile(p, w.tile);
  if (w.kb0 >= 0) { c.kb0 = w.kb0; c.nkb = w.nkb; }
  return c;
}

// PACKED (the one-accumulator tile with a 16-bit result, whole tiles only): the epilogue packs its
// share of the accumulator into registers and hands the accumulator back before it stores anything.
// The two epilogues live in separate instances: compiled into one, each costs the other registers.
template <int BN, int STAGES, int A_MN, int B_MN, int KIND, int PAIR, int PACKED = 0>
__global__ void __launch_bounds__(gemm_threads(BN), 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const GemmParams p,
                    const __grid_constant__ SfMaps<KIND == 3> sfm) {
  constexpr bool MX = KIND == 3;
  static_assert(!(KIND == 1 && (A_MN || B_MN)), "the tf32 path stages K-major operands only");
  static_assert(!MX || ((BN == 512 || BN == 256) && PAIR && !A_MN && !B_MN), "the block-scaled kind: pair tiles, K-major operands");
  static_assert(BN % 64 == 0 && BN >= 64 && BN <= 512, "tile width");
  static_assert(BN <= 256 || PAIR, "tiles wider than one MMA need the CTA pair");
  static_assert(!PACKED || (BN > 256 && KIND != 1), "the packed drain is the wide tile's, for 16-bit results");
  using L = GemmSmem<BN, STAGES, PAIR, MX>;
  constexpr int ELT = KIND == 1 ? 4 : KIND >= 2 ? 1 : 2;  // operand bytes per element
  constexpr int BK = kStageKBytes / ELT;   // contraction elements per stage
  constexpr int BOXW = kStageKBytes / ELT; // elements along MN in one MN-major box
  constexpr int MMAS = kStageKBytes / kMmaKBytes;
  constexpr int MMA_K = kMmaKBytes / ELT;  // contraction elements per tcgen05.mma
  constexpr int TM = kTileM * (PAIR ? 2 : 1);
  // BN is the widest tile this instance can hold; the tile's actual width p.bn
  // may be any multiple of 32 up to it (the shared-memory slots and the tensor
  // memory columns keep BN's spacing, the TMA boxes and the MMAs follow p.bn).
  // A tile wider than 256 columns is two MMAs of p.subn columns side by side in
  // tensor memory.  Two accumulators (epilogue overlapped with the next main
  // loop) while they fit the 512 columns, one otherwise.
  constexpr bool WIDE = BN > 256;
  constexpr int NSUB = WIDE ? 2 : 1;
  constexpr int SUBC_CAP = MX ? mx_subc_cap(BN) : (BN / NSUB) / (PAIR ? 2 : 1);  // B rows one CTA can stage per sub-tile
  // block-scaled kind: the two sets of scale columns, 480..511, above every accumulator (two of
  // at most 192 columns at 0 and 256, or one of at most 384)
  constexpr uint32_t SF_COL0 = 512 - kSfSets * kSfTmemCols;
  constexpr uint32_t SF_SET = kSfTmemCols;
  constexpr int ACC = WIDE ? 1 : 2;
  constexpr int EPI_GROUPS = gemm_epi_groups(BN);
  constexpr int CH = BN >= 128 ? 4 : 2;   // 32-column chunks an epilogue warp drains per wait
  constexpr int NPH = WIDE ? 2 : 1;       // drain phases per tile
  static_assert(NPH * EPI_GROUPS * CH * 32 == BN, "the epilogue warps cover the widest tile exactly");
  // The one-accumulator tile starts the next tile's MMAs on the first sub-tile
  // alone, for PRO contraction blocks, as soon as the columns below 256 have
  // been read out; the second sub-tile follows once the rest is out.  Each
  // column still sees its products in ascending k, so no bit changes.
  constexpr int PRO = WIDE ? STAGES - 1 : 0;
  constexpr uint32_t TMEM_COLS = (ACC * BN <= 128) ? 128 : (ACC * BN <= 256) ? 256 : 512;
  constexpr uint32_t EPI_WARP0 = EPI_GROUPS == 2 ? 4 : 2;  // first epilogue warp

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - raw_addr);

  const uint32_t bars = base + L::kBarOffset;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  // two accumulators: one "drained" barrier each; one accumulator: [0] columns below 256, [1] the rest
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  const uint32_t teardown_bar = bars + 8u * (2 * STAGES + 4);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(base_ptr + L::kBarOffset + L::kNumBars * 8);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t cta_rank = PAIR ? ptx::cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  const int32_t bn = p.bn;
  const int32_t subn = p.subn;
  const int32_t subc = PAIR ? (subn >> 1) : subn;  // B rows this CTA stages per sub-tile

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), (PAIR ? 8 : 4) * EPI_GROUPS);
    }
    ptx::mbar_init(teardown_bar, 1);
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB);
    if (p.out_tma) ptx::prefetch_tensormap(&tmC);
    if constexpr (MX) {
      ptx::prefetch_tensormap(&sfm.a);
      ptx::prefetch_tensormap(&sfm.b);
    }
  }
  if (warp == 1) {
    ptx::tmem_alloc<PAIR>(ptx::smem_u32(tmem_slot), TMEM_COLS);
  }
  ptx::tc_fence_before();
  if constexpr (PAIR) {
    __syncthreads();
    ptx::cluster_arrive();
    ptx::cluster_wait();
  } else {
    __syncthreads();
  }
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wc{abort_flag, p.status, p.wait_limit_ns};
  const int64_t tile_stride = PAIR ? (gridDim.x >> 1) : gridDim.x;
  const int64_t tile_first = PAIR ? (blockIdx.x >> 1) : blockIdx.x;

  if (warp < EPI_WARP0) {
  // Registers move from the warpgroup of the two single-thread roles to the epilogue warpgroups.
  if constexpr (EPI_GROUPS == 2) ptx::setmaxnreg_dec<kProducerRegs>();
  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      bool ok = true;
      WorkIter it;
      WorkItem wi;
      it.init(p, tile_first, tile_stride);
      const int32_t b_boxes = (subc + BOXW - 1) / BOXW;  // MN-major B: boxes of BOXW columns per sub-tile
      while (ok && it.next(p, wi)) {
        const TileCoord tc = decode_item(p, wi);
        const int32_t m0 = tc.m_blk * TM + static_cast<int32_t>(cta_rank) * kTileM;
        const int32_t n0 = tc.n_blk * bn + static_cast<int32_t>(cta_rank) * subc;  // + sub * subn per sub-tile
        for (int32_t kb = 0; kb < tc.nkb; ++kb) {
          if (!bounded_wait(empty_bar(s), ph ^ 1u, wc)) { ok = false; break; }
          const uint32_t sa = base + s * L::kStageBytes;
          const uint32_t sb = sa + L::kABytes;
          const int32_t k0 = (tc.kb0 + kb) * BK;
          if constexpr (PAIR) {
            // The leader's barrier collects the bytes of both CTAs' loads.
            const uint32_t fb = ptx::mapa_shared(full_bar(s), 0);
            // (block-scaled kind: stage_tx counts the scale atoms too, which warp 2 loads)
            if (leader) ptx::mbar_arrive_expect_tx(full_bar(s), 2u * p.stage_tx);
            if constexpr (A_MN) {
#pragma unroll
              for (int j = 0; j < kTileM / BOXW; ++j)
                ptx::tma_load_3d_pair(sa + j * (BK * kStageKBytes), &tmA, fb, m0 + j * BOXW, k0, tc.a_batch);
            } else {
              ptx::tma_load_3d_pair(sa, &tmA, fb, k0, m0, tc.a_batch);
            }
#pragma unroll
            for (int sub = 0; sub < NSUB; ++sub) {
              const uint32_t sbs = sb + sub * (SUBC_CAP * kStageKBytes);
              const int32_t ns = n0 + sub * subn;
              if constexpr (B_MN) {
                for (int j = 0; j < b_boxes; ++j)
                  ptx::tma_load_3d_pair(sbs + j * (BK * kStageKBytes), &tmB, fb, ns + j * BOXW, k0, tc.b_batch);
              } else {
                ptx::tma_load_3d_pair(sbs, &tmB, fb, k0, ns, tc.b_batch);
              }
            }
          } else {
            const uint32_t fb = full_bar(s);
            ptx::mbar_arrive_expect_tx(fb, p.stage_tx);
            if constexpr (A_MN) {
#pragma unroll
              for (int j = 0; j < kTileM / BOXW; ++j)
                ptx::tma_load_3d(sa + j * (BK * kStageKBytes), &tmA, fb, m0 + j * BOXW, k0, tc.a_batch);
            } else {
              ptx::tma_load_3d(sa, &tmA, fb, k0, m0, tc.a_batch);
            }
            if constexpr (B_MN) {
              for (int j = 0; j < b_boxes; ++j)
                ptx::tma_load_3d(sb + j * (BK * kStageKBytes), &tmB, fb, n0 + j * BOXW, k0, tc.b_batch);
            } else {
              ptx::tma_load_3d(sb, &tmB, fb, k0, n0, tc.b_batch);
            }
          }
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
      if (*abort_flag) {
        // Give loads already in flight time to land before shared memory goes away.
        const uint64_t t0 = ptx::globaltimer_ns();
        while (ptx::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && leader) {
      // K-major tile: rows of 128 B, 8-row swizzle atoms 1 KiB apart.
      // MN-major tile: boxes of BK rows x 128 B; LBO = one box, 8-row groups 1 KiB apart.
      constexpr uint32_t A_LBO = A_MN ? BK * kStageKBytes : 16;
      constexpr uint32_t B_LBO = B_MN ? BK * kStageKBytes : 16;
      constexpr uint32_t A_ADV = (A_MN ? MMA_K * kStageKBytes : kMmaKBytes) >> 4;
      constexpr uint32_t B_ADV = (B_MN ? MMA_K * kStageKBytes : kMmaKBytes) >> 4;
      constexpr uint32_t B_SUB = (SUBC_CAP * kStageKBytes) >> 4;  // descriptor distance between the sub-tiles' slots
      uint32_t s = 0, ph = 0, as = 0, aph = 0;
      bool ok = true;
      WorkIter it;
      WorkItem wi;
      it.init(p, tile_first, tile_stride);
      // Block-scaled kind: stage `st`'s scales go from shared memory to one of the two sets of
      // scale columns of tensor memory (taken in turn, so that a copy never waits for the MMAs of
      // the stage before it, which read the other set), in order with the MMAs issued around
      // them.  Returns the set's first column: A's scales there, B's from four columns on.
      int32_t sfb_atoms = 0;    // atoms of B's scales the current tile's columns touch
      uint32_t sfb_first = 0;   // the tile's first column within the first atom, in 32-column groups
      auto stage_scales = [&](uint32_t st) -> uint32_t {
        const uint32_t set = tmem_base + SF_COL0 + (st & 1u) * SF_SET;
        const uint32_t sf = base + L::kSfOffset + st * L::kSfStage;
        ptx::tmem_cp_32x128b_x4<PAIR>(set, make_sf_desc(sf));
        for (int32_t g = 0; g < sfb_atoms; ++g)
          ptx::tmem_cp_32x128b_x4<PAIR>(set + 4u + 4u * g, make_sf_desc(sf + kSfAtomBytes * (1 + g)));
        return set;
      };
      // The four MMAs of one contraction block for sub-tile `sub`, from stage `st`.
      auto issue = [&](uint32_t st, int sub, uint32_t d_tmem, int32_t kb) {
        const uint32_t sa = base + st * L::kStageBytes;
        const uint32_t sb = sa + L::kABytes;
        const uint64_t adesc = make_smem_desc(sa, A_LBO, 1024);
        const uint64_t bdesc = make_smem_desc(sb, B_LBO, 1024) + static_cast<uint64_t>(sub * B_SUB);
        if constexpr (MX) {
          const uint32_t set = stage_scales(st);
#pragma unroll
          for (int j = 0; j < MMAS; ++j)  // contraction block j of the stage: scale byte j of either operand
            ptx::umma_mx<PAIR>(d_tmem + sub * subn, adesc + static_cast<uint64_t>(j * A_ADV), bdesc + static_cast<uint64_t>(j * B_ADV),
                               p.idesc | (static_cast<uint32_t>(j) << 4) | (static_cast<uint32_t>(j) << 29), set,
                               set + 4u + sfb_first + static_cast<uint32_t>(sub * (subn >> 5)), (kb | j) != 0 ? 1u : 0u);
        } else {
#pragma unroll
          for (int j = 0; j < MMAS; ++j)
            ptx::umma<PAIR, KIND>(d_tmem + sub * subn, adesc + static_cast<uint64_t>(j * A_ADV),
                                  bdesc + static_cast<uint64_t>(j * B_ADV), p.idesc, (kb | j) != 0 ? 1u : 0u);
        }
      };
      auto release_stage = [&](uint32_t st) {
        if constexpr (PAIR) ptx::umma_commit_pair(empty_bar(st), 3);
        else ptx::umma_commit(empty_bar(st));
      };
      while (ok && it.next(p, wi)) {
        int32_t nkb = wi.nkb;
        if (nkb < 0) {
          const int32_t split = static_cast<int32_t>(wi.tile / p.tiles_per_split);
          nkb = min(p.kb_per_split, p.num_kb - split * p.kb_per_split);
        }
        if constexpr (MX) {
          const int32_t tile_n0 = decode_item(p, wi).n_blk * bn;
          sfb_atoms = ((tile_n0 & 127) + bn + 127) >> 7;
          sfb_first = static_cast<uint32_t>((tile_n0 & 127) >> 5);
        }
        if (!bounded_wait(tempty_bar(WIDE ? 0 : as), aph ^ 1u, wc)) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BN;
        int32_t kb = 0;
        if constexpr (WIDE) {
          // The first sub-tile's columns are free: run it ahead for up to PRO blocks
          // while the epilogue warps finish reading the second sub-tile's.
          const int32_t pro = min(PRO, nkb);
          uint32_t s2 = s, ph2 = ph;
          for (int32_t k2 = 0; k2 < pro; ++k2) {
            if (!bounded_wait(full_bar(s2), ph2, wc)) { ok = false; break; }
            ptx::tc_fence_after();
            issue(s2, 0, d_tmem, k2);
            if (++s2 == STAGES) { s2 = 0; ph2 ^= 1u; }
          }
          if (!ok) break;
          if (!bounded_wait(tempty_bar(1), aph ^ 1u, wc)) break;
          ptx::tc_fence_after();
          for (int32_t k2 = 0; k2 < pro; ++k2) {
            issue(s, 1, d_tmem, k2);
            release_stage(s);
            if (++s == STAGES) { s = 0; ph ^= 1u; }
          }
          kb = pro;
        }
        for (; kb < nkb; ++kb) {
          if (!bounded_wait(full_bar(s), ph, wc)) { ok = false; break; }
          ptx::tc_fence_after();
          if constexpr (WIDE) {
            // sub-tiles side by side, k step by k step: both reuse the A slice while it is hot
            const uint32_t sa = base + s * L::kStageBytes;
            const uint32_t sb = sa + L::kABytes;
            const uint64_t adesc = make_smem_desc(sa, A_LBO, 1024);
            const uint64_t bdesc = make_smem_desc(sb, B_LBO, 1024);
            if constexpr (MX) {
              const uint32_t set = stage_scales(s);
#pragma unroll
              for (int j = 0; j < MMAS; ++j) {
#pragma unroll
                for (int sub = 0; sub < NSUB; ++sub)
                  ptx::umma_mx<PAIR>(d_tmem + sub * subn, adesc + static_cast<uint64_t>(j * A_ADV),
                                     bdesc + static_cast<uint64_t>(j * B_ADV + sub * B_SUB),
                                     p.idesc | (static_cast<uint32_t>(j) << 4) | (static_cast<uint32_t>(j) << 29), set,
                                     set + 4u + sfb_first + static_cast<uint32_t>(sub * (subn >> 5)), (kb | j) != 0 ? 1u : 0u);
              }
            } else {
#pragma unroll
            for (int j = 0; j < MMAS; ++j) {
#pragma unroll
              for (int sub = 0; sub < NSUB; ++sub)
                ptx::umma<PAIR, KIND>(d_tmem + sub * subn, adesc + static_cast<uint64_t>(j * A_ADV),
                                      bdesc + static_cast<uint64_t>(j * B_ADV + sub * B_SUB), p.idesc, (kb | j) != 0 ? 1u : 0u);
            }
            }
          } else {
            issue(s, 0, d_tmem, kb);
          }
          release_stage(s);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        if constexpr (PAIR) ptx::umma_commit_pair(tfull_bar(as), 3);
        else ptx::umma_commit(tfull_bar(as));
        if (++as == ACC) { as = 0; aph ^= 1u; }
      }
      if (*abort_flag) {
        // Let tensor-core work already issued retire before tensor memory is freed.
        if constexpr (PAIR) ptx::umma_commit_pair(teardown_bar, 1);
        else ptx::umma_commit(teardown_bar);
        const uint64_t t0 = ptx::globaltimer_ns();
        while (!ptx::mbar_try_wait(teardown_bar, 0) && ptx::globaltimer_ns() - t0 < 10000000ull) {
        }
      }
    }
    __syncwarp();
  } else if (MX && warp == 2) {
    // ---------------- scale producer (block-scaled kind) ----------------
    // The third warp of the producer warpgroup loads every stage's scale atoms: the atom of this
    // CTA's 128 rows of A, and the three atoms from the one the tile's first column lies in on
    // for B (each CTA of the pair multiplies its rows by ALL the tile's columns, so both load
    // them; atoms beyond the matrix read as zeros).  It walks the same tiles and stages as the
    // TMA warp and waits on the same "stage empty" barriers; its bytes are counted on the same
    // "stage full" barrier.  (With these loads on the TMA warp, seven copies per stage from one
    // thread, the stages arrived too slowly for the tensor pipe.)
    if constexpr (MX) {
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      bool ok = true;
      WorkIter it;
      WorkItem wi;
      it.init(p, tile_first, tile_stride);
      while (ok && it.next(p, wi)) {
        const TileCoord tc = decode_item(p, wi);
        const int32_t rg_a = (tc.m_blk * TM + static_cast<int32_t>(cta_rank) * kTileM) >> 7;
        const int32_t rg_b = (tc.n_blk * bn) >> 7;
        for (int32_t kb = 0; kb < tc.nkb; ++kb) {
          if (!bounded_wait(empty_bar(s), ph ^ 1u, wc)) { ok = false; break; }
          const uint32_t fb = ptx::mapa_shared(full_bar(s), 0);
          const uint32_t sf = base + L::kSfOffset + s * L::kSfStage;
          ptx::tma_load_4d_pair(sf, &sfm.a, fb, 0, rg_a, tc.kb0 + kb, tc.a_batch);
          ptx::tma_load_4d_pair(sf + kSfAtomBytes, &sfm.b, fb, 0, rg_b, tc.kb0 + kb, tc.b_batch);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
      if (*abort_flag) {
        const uint64_t t0 = ptx::globaltimer_ns();
        while (ptx::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
    __syncwarp();
    }
  }
  } else {
    // ---------------- epilogue: TMEM -> registers -> global ----------------
    if constexpr (EPI_GROUPS == 2) ptx::setmaxnreg_inc<kEpilogueRegs>();
    const uint32_t ew = warp - EPI_WARP0;
    const uint32_t q = warp & 3u;  // the TMEM lane quarter this warp may read
    const uint32_t grp = ew >> 2;  // which share of the columns this warp drains
    const uint32_t stage_smem = base + L::kStagingOffset + ew * L::kStagingTile;
    const int esz = p.out_dtype == 0 ? 4 : (p.out_dtype >= 8 ? 1 : 2);
    const int32_t nchunks = bn >> 5;  // 32-column chunks of a tile
    uint32_t as = 0, aph = 0;
    WorkIter it;
    WorkItem wi;
    it.init(p, tile_first, tile_stride);
    const int64_t my_run = tile_stride - 1 - tile_first;  // this CTA's (pair's) stream-K run
    constexpr int CPT = PAIR ? 2 : 1;
    constexpr int WARP_COLS = NPH * CH * 32;  // columns one warp drains from the widest tile
    while (it.next(p, wi)) {
      const TileCoord tc = decode_item(p, wi);
      // tcgen05.ld is warp-collective: leave the loop as a whole warp or not at all.
      const bool ready = bounded_wait(tfull_bar(as), aph, wc);
      if (!__all_sync(0xffffffffu, ready)) break;
      ptx::tc_fence_after();
      // Stream-K: where this warp's part of a run's partial sums lives, and how many later runs
      // hold the rest of an owned tile.
      const int64_t sk_warp_elems = static_cast<int64_t>(kTileM) * BN;
      float *sk_mine = p.sk_ws + (my_run * CPT + cta_rank) * sk_warp_elems;
      int sk_others = 0;
      if (wi.kind == 1) {
        int32_t left = p.num_kb - wi.nkb;
        bool arrived = true;
        for (int64_t r = my_run + 1; left > 0 && r < tile_stride; ++r, ++sk_others) {
          int64_t rb, re;
          sk_run(p.sk_tiles * p.num_kb, tile_stride, r, rb, re);
          left -= static_cast<int32_t>(min(re - rb, static_cast<int64_t>(left)));
          // wait (bounded) until run r's warp of the same rows and columns has published its sums
          const uint32_t *flag = p.sk_flags + (r * CPT + cta_rank) * 8 + ew;
          if (arrived && ptx::ld_acquire_gpu(flag) != p.sk_epoch) {
            const uint64_t t0 = ptx::globaltimer_ns();
            while (ptx::ld_acquire_gpu(flag) != p.sk_epoch) {
              if (*wc.abort_flag) { arrived = false; break; }
              if (ptx::globaltimer_ns() - t0 > wc.limit_ns) {
                *wc.abort_flag = 1;
                atomicCAS(wc.status, 0u, kStatusTimeout);
                arrived = false;
                break;
              }
              __nanosleep(200);
            }
          }
        }
        if (!__all_sync(0xffffffffu, arrived)) break;
      }
      const int32_t row = tc.m_blk * TM + static_cast<int32_t>(cta_rank) * kTileM + static_cast<int32_t>(q * 32u + lane);
      const bool row_ok = row < p.M;
      uint8_t *rowp = static_cast<uint8_t *>(p.out) + (tc.o_off + static_cast<int64_t>(row) * p.out_rs) * esz;
      // One 32-column chunk of this thread's row: convert and store through the output's strides.
      auto store_chunk = [&](const uint32_t (&v)[32], int32_t col0) {
        if (!row_ok || col0 >= p.N) return;
        if (p.out_vec && col0 + 32 <= p.N) {
          if (p.out_dtype == 0) {
            uint4 *dst = reinterpret_cast<uint4 *>(rowp + static_cast<int64_t>(col0) * 4);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          } else {
            uint32_t h[16];
            if (p.out_dtype == 6) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                h[i] = *reinterpret_cast<uint32_t *>(&t);
              }
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                __half2 t = __floats2half2_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                h[i] = *reinterpret_cast<uint32_t *>(&t);
              }
            }
            uint4 *dst = reinterpret_cast<uint4 *>(rowp + static_cast<int64_t>(col0) * 2);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[i] = make_uint4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (col0 + i < p.N) {
              const float f = __uint_as_float(v[i]);
              const int64_t e = static_cast<int64_t>(col0 + i) * p.out_cs;
              if constexpr (KIND >= 2) {
                store_elem(rowp, p.out_dtype, e, f);  // fp8 operands: the output may be fp8 or wider
              } else {
                if (p.out_dtype == 0) reinterpret_cast<float *>(rowp)[e] = f;
                else if (p.out_dtype == 6) reinterpret_cast<__nv_bfloat16 *>(rowp)[e] = __float2bfloat16_rn(f);
                else reinterpret_cast<__half *>(rowp)[e] = __float2half_rn(f);
              }
            }
          }
        }
      };
      const uint32_t t_row = tmem_base + as * BN + ((q * 32u) << 16);
      const int32_t tile_col0 = tc.n_blk * bn;
      const int32_t row0 = row - static_cast<int32_t>(lane);  // first of this warp's 32 rows
      // One 128-byte-wide chunk of the warp's 32 rows: staged in shared memory in
      // the 128-byte swizzle (16-byte piece j of row r lands at piece j ^ (r & 7)),
      // then written by one bulk tensor store, which clips at the tensor's edge.
      auto emit = [&](const uint4 (&piece)[8], int32_t col) {
        if (row0 >= p.M || col >= p.N) return;  // warp-uniform
        if (lane == 0) ptx::bulk_wait_read_all();  // the previous store has released the staging tile
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t addr = stage_smem + lane * kStageKBytes + ((static_cast<uint32_t>(j) ^ (lane & 7u)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(piece[j].x), "r"(piece[j].y),
                       "r"(piece[j].z), "r"(piece[j].w) : "memory");
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          ptx::tma_store_3d(&tmC, stage_smem, col, row0, tc.o_batch);
          ptx::bulk_commit_group();
        }
      };
      // The one-accumulator tile with a 16-bit result: this warp's whole share of the accumulator
      // (up to 256 columns) is rounded and packed into 128 registers, the accumulator is handed
      // back, and only then does anything get stored - the next tile's main loop never waits for a
      // store (one staged bulk store takes microseconds; four of them per warp used to sit between
      // two tiles).
      if constexpr (PACKED) {
        {
          uint32_t pk[NPH][CH][16];
          constexpr int RC = 2;  // four at once would not fit beside the packed half
#pragma unroll
          for (int dp = 0; dp < NPH; ++dp) {
            const int32_t ch0 = dp * (CH * EPI_GROUPS) + static_cast<int32_t>(grp) * CH;
            // RC chunks (32 columns each) per round of tensor-memory loads: 32 RC registers of raw
            // sums beside the up to 128 packed ones
#pragma unroll
            for (int r = 0; r < CH / RC; ++r) {
              uint32_t v[RC][32];
#pragma unroll
              for (int i = 0; i < RC; ++i)
                if (ch0 + RC * r + i < nchunks) ptx::tmem_ld_32x32(t_row + static_cast<uint32_t>((ch0 + RC * r + i) * 32), v[i]);
              ptx::tmem_ld_wait();
              if (p.epi.any) {
                const int32_t colb = tile_col0 + (ch0 + RC * r) * 32;
#pragma unroll
                for (int i = 0; i < RC; ++i) {
                  if (ch0 + RC * r + i >= nchunks) continue;
#pragma unroll
                  for (int e = 0; e < 32; ++e) {
                    const int32_t col = colb + i * 32 + e;
                    if (row_ok && col < p.N) {
                      const int64_t idx = tc.o_off + static_cast<int64_t>(row) * p.out_rs + static_cast<int64_t>(col) * p.out_cs;
                      v[i][e] = __float_as_uint(apply_epilogue(p.epi, __uint_as_float(v[i][e]), col, p.out, p.out_dtype, idx));
                    }
                  }
                }
              }
#pragma unroll
              for (int i = 0; i < RC; ++i) {
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                  const float lo = __uint_as_float(v[i][2 * e]), hi = __uint_as_float(v[i][2 * e + 1]);
                  if (p.out_dtype == 6) {
                    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
                    pk[dp][RC * r + i][e] = *reinterpret_cast<uint32_t *>(&t);
                  } else {
                    __half2 t = __floats2half2_rn(lo, hi);
                    pk[dp][RC * r + i][e] = *reinterpret_cast<uint32_t *>(&t);
                  }
                }
              }
            }
            // This half of the accumulator (phase 0: the columns below 256, which hold the first
            // sub-tile) is in registers: hand it back.  The MMA warp starts the next tile on the
            // first sub-tile while the second half is still being read out here.
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if constexpr (PAIR) ptx::mbar_arrive_cluster(ptx::mapa_shared(tempty_bar(dp), 0));
              else ptx::mbar_arrive(tempty_bar(dp));
            }
          }
          // One packed 32-column chunk of this thread's row through plain stores (no partner chunk to
          // fill a store box with, or an output the bulk store cannot describe).
          auto store_packed = [&](const uint32_t (&h)[16], int32_t col0) {
            if (!row_ok || col0 >= p.N) return;
            if (p.out_vec && col0 + 32 <= p.N) {
              uint4 *dst = reinterpret_cast<uint4 *>(rowp + static_cast<int64_t>(col0) * 2);
#pragma unroll
              for (int i = 0; i < 4; ++i) dst[i] = make_uint4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N)
                  reinterpret_cast<uint16_t *>(rowp)[static_cast<int64_t>(col0 + i) * p.out_cs] =
                      static_cast<uint16_t>(h[i >> 1] >> (16 * (i & 1)));
            }
          };
#pragma unroll
          for (int dp = 0; dp < NPH; ++dp) {
            const int32_t ch0 = dp * (CH * EPI_GROUPS) + static_cast<int32_t>(grp) * CH;
#pragma unroll
            for (int i = 0; i < CH / 2; ++i) {
              const int32_t c = ch0 + 2 * i, col = tile_col0 + c * 32;
              if (c >= nchunks) continue;
              if (p.out_tma && c + 1 < nchunks) {
                uint4 piece[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const uint32_t *src = j < 4 ? &pk[dp][2 * i][4 * j] : &pk[dp][2 * i + 1][4 * (j - 4)];
                  piece[j] = make_uint4(src[0], src[1], src[2], src[3]);
                }
                emit(piece, col);
              } else {
                store_packed(pk[dp][2 * i], col);
                if (c + 1 < nchunks) store_packed(pk[dp][2 * i + 1], col + 32);
              }
            }
          }
        }
      } else {
#pragma unroll 1
      for (int dp = 0; dp < NPH; ++dp) {
        // this warp's chunks of the phase: [ch0, ch0 + CH), those below nchunks exist
        const int32_t ch0 = dp * (CH * EPI_GROUPS) + static_cast<int32_t>(grp) * CH;
        uint32_t v[CH][32];
#pragma unroll
        for (int i = 0; i < CH; ++i)
          if (ch0 + i < nchunks) ptx::tmem_ld_32x32(t_row + static_cast<uint32_t>((ch0 + i) * 32), v[i]);
        ptx::tmem_ld_wait();
        if (WIDE || dp == NPH - 1) {
          // These columns now live in registers: hand them back before converting and storing.
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            const uint32_t bar = tempty_bar(WIDE ? dp : static_cast<int>(as));
            if constexpr (PAIR) ptx::mbar_arrive_cluster(ptx::mapa_shared(bar, 0));
            else ptx::mbar_arrive(bar);
          }
        }
        if (wi.kind == 2) {
          // contributor: this run started inside the tile; leave the raw sums for the tile's owner.
          // The hand-over area is private to the two warps involved (same rows, same columns,
          // same registers), so it is laid out by register: every store is 512 contiguous bytes.
          uint4 *dst = reinterpret_cast<uint4 *>(sk_mine + static_cast<int64_t>(ew) * (32 * WARP_COLS)) + lane;
#pragma unroll
          for (int i = 0; i < CH; ++i) {
            if (ch0 + i >= nchunks) continue;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              dst[((dp * CH + i) * 8 + j) * 32] = make_uint4(v[i][4 * j], v[i][4 * j + 1], v[i][4 * j + 2], v[i][4 * j + 3]);
          }
          continue;
        }
        if (wi.kind == 1) {
          // owner: add the later runs' sums of these columns, in run order
          for (int o = 0; o < sk_others; ++o) {
            const float4 *src = reinterpret_cast<const float4 *>(p.sk_ws + ((my_run + 1 + o) * CPT + cta_rank) * sk_warp_elems +
                                                                 static_cast<int64_t>(ew) * (32 * WARP_COLS)) + lane;
#pragma unroll
            for (int i = 0; i < CH; ++i) {
              if (ch0 + i >= nchunks) continue;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 t = __ldcg(src + ((dp * CH + i) * 8 + j) * 32);
                v[i][4 * j] = __float_as_uint(__uint_as_float(v[i][4 * j]) + t.x);
                v[i][4 * j + 1] = __float_as_uint(__uint_as_float(v[i][4 * j + 1]) + t.y);
                v[i][4 * j + 2] = __float_as_uint(__uint_as_float(v[i][4 * j + 2]) + t.z);
                v[i][4 * j + 3] = __float_as_uint(__uint_as_float(v[i][4 * j + 3]) + t.w);
              }
            }
          }
        }
        const int32_t colb = tile_col0 + ch0 * 32;
        if (p.epi.any) {
          // bias, activation and accumulation on the fp32 sums, before rounding
#pragma unroll
          for (int i = 0; i < CH; ++i) {
            if (ch0 + i >= nchunks) continue;
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int32_t col = colb + i * 32 + e;
              if (row_ok && col < p.N) {
                const int64_t idx = tc.o_off + static_cast<int64_t>(row) * p.out_rs + static_cast<int64_t>(col) * p.out_cs;
                v[i][e] = __float_as_uint(apply_epilogue(p.epi, __uint_as_float(v[i][e]), col, p.out, p.out_dtype, idx));
              }
            }
          }
        }
        if (p.out_tma) {
          if constexpr (KIND == 1) {
#pragma unroll
            for (int i = 0; i < CH; ++i) {
              if (ch0 + i >= nchunks) continue;
              uint4 piece[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) piece[j] = make_uint4(v[i][4 * j], v[i][4 * j + 1], v[i][4 * j + 2], v[i][4 * j + 3]);
              emit(piece, colb + i * 32);
            }
          } else {
#pragma unroll
            for (int i = 0; i < CH / 2; ++i) {
              if (ch0 + 2 * i >= nchunks) continue;
              if (ch0 + 2 * i + 1 >= nchunks) {
                // the tile's last chunk has no partner to fill a 128-byte box with
                store_chunk(v[2 * i], colb + i * 64);
                continue;
              }
              uint4 piece[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const uint32_t *src = j < 4 ? &v[2 * i][8 * j] : &v[2 * i + 1][8 * (j - 4)];
                uint32_t h[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float lo = __uint_as_float(src[2 * e]), hi = __uint_as_float(src[2 * e + 1]);
                  if (p.out_dtype == 6) {
                    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
                    h[e] = *reinterpret_cast<uint32_t *>(&t);
                  } else {
                    __half2 t = __floats2half2_rn(lo, hi);
                    h[e] = *reinterpret_cast<uint32_t *>(&t);
                  }
                }
                piece[j] = make_uint4(h[0], h[1], h[2], h[3]);
              }
              emit(piece, colb + i * 64);
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < CH; ++i)
            if (ch0 + i < nchunks) store_chunk(v[i], colb + i * 32);
        }
      }
      }  // two-phase drain
      if (wi.kind == 2) {
        // publish: the sums above are visible to whoever reads this launch's counter here
        __threadfence();
        __syncwarp();
        if (lane == 0) ptx::st_release_gpu(p.sk_flags + (my_run * CPT + cta_rank) * 8 + ew, p.sk_epoch);
      }
      if (++as == ACC) { as = 0; aph ^= 1u; }
    }
    if (lane == 0) ptx::bulk_wait_read_all();  // staging tiles are still being read until here
    __syncwarp();
  }

  // ---------------- teardown ----------------
  ptx::tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) {
    // Neither CTA may leave while its peer can still touch its shared or tensor memory.
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<PAIR>(tmem_base, TMEM_COLS);
  }
}

}  // namespace oxm
