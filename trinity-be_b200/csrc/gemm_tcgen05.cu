// BF16 GEMM with fused epilogue on the 5th-generation tensor cores.
//
//   out[M,N] = act(A[M,K] @ B[K,N] + bias)            FP32 accumulation in TMEM
//   out[M,N] = (A@B) * silu(A@B2)                     gated form, two accumulators per tile
//
// One persistent CTA per SM, 192 threads, warp-specialised:
//   warp 0    TMA producer: A tile [128 x 64] (K-major) and B tile [64 x BN] (N-major, i.e. the
//             row-major [K,N] weight as it lies in memory) into a multi-stage 128B-swizzled ring
//   warp 1    MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN, K=16) four times
//             per stage and commits the stage's "empty" barrier; accumulators are double
//             buffered in TMEM (2 x BN columns) so the epilogue of tile i overlaps tile i+1
//   warps 2-5 epilogue: tcgen05.ld 32 columns at a time, bias / activation in FP32, one
//             rounding to the output type, 128B-swizzled staging and a TMA store per warp
//   warps 6-9 only in the row-parallel form with the cross-GPU sum (352 threads): reducers that
//             add the ranks' partial tiles over NVLink peer memory while the MMAs go on
//   warp 10   (same form) tells the other GPUs' reducers which partial tiles are complete
//
//
// Large problems run on CTA pairs (a cluster of two CTAs, tcgen05 cta_group::2): a pair owns a
// 256 x 256 output tile, each CTA loads its own 128 rows of A and its own 128 of the 256 B
// columns (in the gated form 64 up-weight and the matching 64 gate-weight columns), the
// even CTA issues M=256 MMAs that read both CTAs' shared memory and write each CTA's 128
// accumulator rows into its own TMEM, and both CTAs run their own epilogue.  A stage is 32 KB
// per CTA instead of 48, so every SM reads and writes a third less shared memory per FLOP.
//
// Few output rows against a large weight (at most 64 rows, fewer tiles of 256 accumulator columns
// than half the SMs; plain or gated) run in the split form: a cluster of 2, 4 or 8 CTAs shares
// one tile, each CTA streams its own part of K (32 or 64 rows of A per K block), and the partial sums
// meet in the first CTA's shared memory (one bulk copy per CTA), where they are added in a fixed
// order before the epilogue.
//
// Algorithmic traffic per launch: (M*K + K*N [+K*N]) * 2 + bias + M*N*out_bytes.
#include <cstdlib>
#include <mutex>
#include <vector>

#include "host_common.h"
#include "sm100_ptx.cuh"

namespace trinity_sm100 {
namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 192;        // TMA producer, MMA issuer, four epilogue warps
constexpr int kGemmFusedThreads = 352;   // ... plus four warps that do the cross-GPU reduction and one that signals
constexpr int kGroupM = 16;           // tile rasterisation: 16 row blocks share B columns in L2
constexpr int kStageBytesA = kBM * kBK * 2;
constexpr int kSplitRowsMax = 64;        // the split form serves up to this many output rows
constexpr int kSplitPitch = 256 + 4;     // floats between rows of a partial sum in shared memory (16-byte
                                         // accesses by eight consecutive rows then fall into distinct banks)
constexpr int kStoreBufBytes = 32 * 128;  // 32 rows x 128 B per epilogue warp
constexpr int kStagingBytes = 4 * 2 * kStoreBufBytes;

// Peer-mapped output buffers and flag pads for the fused all-reduce epilogue.
constexpr int kPairStages = 6;        // 32 KB stages of a CTA pair
constexpr int kGemmMaxWorld = 8;
// The first words of a flag pad belong to the plain all-reduce kernel (allreduce.cu); the fused
// epilogue's flags start behind them so that one pad can serve both kernels in turn.
constexpr int kGemmFlagOffset = 64;
struct GemmPeers {
  uint4* buffers[kGemmMaxWorld];   // the [M,N] BF16 output on every rank (buffers[rank] is local)
  uint32_t* flags[kGemmMaxWorld];  // flag pads: ready[tile][source rank], done[rank], counter
  int world, rank;
  uint32_t epoch;
  uint32_t* epoch_counter;         // persistent artifacts: the call number lives on the device (peer table)
                                   // and the kernel advances it; then `epoch` above is ignored
  long long ld_vectors;            // output row pitch in 16-byte vectors
};

// Milestones of CTA 0 of the most recent fused launch on this device, in nanoseconds of the
// global timer: kernel start, last MMA committed, last partial tile flagged, last owned rows
// reduced, kernel end.  Read by trinity_sm100_gemm_allreduce_stamps (a diagnostic).
__device__ unsigned long long g_fused_stamps[8];
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

struct GemmParams {
  const __nv_bfloat16* bias;
  long long ld_bias;
  int bias_mode;
  int activation;
  int m, n, k;
  int tiles_m, tiles_n, num_tiles, num_kb;
  int flag_tiles;          // 128-row tiles the cross-GPU flags are numbered over (tiles_m rounded up to even)
  // batched form: num_tiles = batch * tiles_per_batch, batch z = tile / tiles_per_batch
  int tiles_per_batch;
  int b_shared;            // one right operand for every batch entry (its map has no batch axis)
  // A tensor map lists its axes by increasing pitch.  When the batch entries are interleaved
  // (batch stride below the row pitch, e.g. [rows, heads, k] with the heads as the batch), the
  // batch axis comes before the row axis and the two coordinates swap places.
  int a_batch_inside, out_batch_inside;
  long long stride_bias;   // elements between the side operands of consecutive batch entries
  int split_rows;          // split form: accumulator rows a CTA hands to its cluster's first CTA (16, 32 or 64)
  int split_a_rows;        // split form: rows of A loaded per K block (32 or 64)
  void* out;               // split form: the output, which its epilogue stores without a tensor map
  long long ldo;           // ... and its row pitch in elements
};

// In a CTA pair each CTA stages only half of the tile's B columns.
template <int kBN, bool kPair = false>
__host__ __device__ constexpr int stage_bytes() {
  return kStageBytesA + kBK * (kPair ? kBN / 2 : kBN) * 2;
}
template <int kBN, int kStages, bool kPair = false>
__host__ __device__ constexpr int gemm_smem_bytes() {
  return 1024 + kStages * stage_bytes<kBN, kPair>() + kStagingBytes + 256;
}

// Rasterisation: groups of `group_rows` tile rows are walked column by column so that the
// tiles in flight share B columns in L2.
__device__ __forceinline__ void tile_coords(int tiles_m, int tiles_n, int group_rows, int tile, int& m_blk,
                                            int& n_blk) {
  const int group_size = group_rows * tiles_n;
  const int group = tile / group_size;
  const int first_m = group * group_rows;
  const int rows_in_group = min(group_rows, tiles_m - first_m);
  const int local = tile - group * group_size;
  m_blk = first_m + local % rows_in_group;
  n_blk = local / rows_in_group;
}

// Where unit `unit` of the persistent loop lies: a 128-row tile, or in pair mode a pair of
// vertically adjacent 128-row tiles of which CTA `rank` takes the `rank`-th.  `flag_tile` numbers
// the 128-row tiles for the cross-GPU flags (the same on every GPU).
template <bool kPair>
__device__ __forceinline__ void locate_tile(const GemmParams& p, int unit, uint32_t rank, int& m_blk, int& n_blk,
                                            int& flag_tile) {
  if (kPair) {
    tile_coords((p.tiles_m + 1) / 2, p.tiles_n, kGroupM / 2, unit, m_blk, n_blk);
    m_blk = m_blk * 2 + int(rank);
    flag_tile = unit * 2 + int(rank);
  } else {
    tile_coords(p.tiles_m, p.tiles_n, kGroupM, unit, m_blk, n_blk);
    flag_tile = unit;
  }
}

// 1 / (1 + exp(-x)) with the exponential and the reciprocal both from the special-function
// unit (two instructions instead of an IEEE division's dozen: the epilogue warps share their
// schedulers with the threads that feed the tensor pipe).  Relative error about 2^-22, far below
// the BF16 rounding of the result; exp(-x) = inf gives 0, exp(-x) = 0 gives 1.
__device__ __forceinline__ float fast_sigmoid(float x) {
  return __fdividef(1.0f, 1.0f + __expf(-x));
}

__device__ __forceinline__ float apply_activation(float x, int activation) {
  if (activation == TRINITY_SM100_ACT_RELU) return x < 0.0f ? 0.0f : x;
  if (activation == TRINITY_SM100_ACT_SILU) return x * fast_sigmoid(x);
  return x;
}

// Fused all-reduce duty of the reducer warps (128 threads, `tid` in [0,128), named barrier
// `barrier_id`).  Every rank owns the same 128/world rows of *every* tile: it waits until all
// ranks have stored their partial of the tile, adds the partials of its rows in rank order in
// FP32, rounds once and pushes the result into every rank's buffer.  Small equal duties per tile
// keep NVLink busy all the time; a duty costs about one NVLink round trip, which is why it
// runs on warps of its own and not on the epilogue warps the tensor pipe waits for.
// Returns false if a wait gave up (uniform over the 128 threads).
template <int kBN>
__device__ __forceinline__ bool reduce_owned_tile(const GemmParams& p, const GemmPeers& peers, int tile,
                                                  int m0, int n0, int tid, int barrier_id) {
  uint32_t good = 1;
  if (tid < peers.world)
    good = wait_flag(peers.flags[peers.rank] + static_cast<long long>(tile) * peers.world + tid, peers.epoch,
                     0x801) ? 1u : 0u;
  uint32_t all_good;
  asm volatile(
      "{\n"
      ".reg .pred a, b;\n"
      "setp.ne.u32 a, %1, 0;\n"
      "bar.red.and.pred b, %2, 128, a;\n"
      "selp.u32 %0, 1, 0, b;\n"
      "}\n"
      : "=r"(all_good)
      : "r"(good), "r"(barrier_id)
      : "memory");
  if (!all_good) return false;
  // Four vectors per thread and step, all loads issued before the first add: with NVLink round
  // trips of a few microseconds the duty is latency-bound, so memory-level parallelism decides
  // how long an owned tile takes.  The sum is always taken in rank order.
  constexpr int kVecPerRow = kBN / 8;
  constexpr int kBatch = 4;
  const int slice_rows = kBM / peers.world;
  m0 += peers.rank * slice_rows;
#pragma unroll 1
  for (int base = 0; base < slice_rows * kVecPerRow; base += 128 * kBatch) {
    uint32_t v[kBatch];   // vector index in every rank's buffer (the launcher keeps it below 2^32)
    bool live[kBatch];
    uint4 part[kBatch][kGemmMaxWorld];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int idx = base + u * 128 + tid;
      const int row = m0 + idx / kVecPerRow;
      const int col = n0 + (idx % kVecPerRow) * 8;
      live[u] = idx < slice_rows * kVecPerRow && row < p.m && col < p.n;
      v[u] = static_cast<uint32_t>(static_cast<long long>(row) * peers.ld_vectors + (col >> 3));
    }
    // (register arrays are indexed statically on purpose: a dynamically indexed destination would
    // consume each load at once and serialise the round trips)
#pragma unroll
    for (int r = 0; r < kGemmMaxWorld; ++r) {
      if (r < peers.world) {
#pragma unroll
        for (int u = 0; u < kBatch; ++u)
          if (live[u]) part[u][r] = peer_load(peers.buffers[r] + v[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      if (!live[u]) continue;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int r = 0; r < kGemmMaxWorld; ++r) {
        if (r < peers.world) {
          const uint32_t w[4] = {part[u][r].x, part[u][r].y, part[u][r].z, part[u][r].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[2 * e] += bf16_lo(w[e]);
            acc[2 * e + 1] += bf16_hi(w[e]);
          }
        }
      }
      const uint4 o = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                 pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
#pragma unroll
      for (int r = 0; r < kGemmMaxWorld; ++r)
        if (r < peers.world) peer_store(peers.buffers[r] + v[u], o);
    }
  }
  return true;
}

// (the split form leaves the epilogue loop of the other forms unreachable in its instantiations)
#pragma nv_diag_suppress 128
template <int kBN, int kStages, bool kGated, bool kOutF32, bool kFused = false, bool kBatched = false,
          bool kPair = false, bool kSplit = false>
__global__ void __launch_bounds__(kFused ? kGemmFusedThreads : kGemmThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                         const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_b2,
                         const __grid_constant__ CUtensorMap map_out, const GemmParams p,
                         const GemmPeers launch_peers) {
  // With a device-side call counter every thread reads it before anything of this launch can
  // have advanced it (the last thread block to retire does that).
  GemmPeers peers = launch_peers;
  if (kFused && peers.epoch_counter) peers.epoch = *reinterpret_cast<volatile uint32_t*>(peers.epoch_counter) + 1u;
  constexpr int kOutN = kGated ? kBN / 2 : kBN;      // output columns per tile
  constexpr int kStage = stage_bytes<kBN, kPair>();
  constexpr int kChunksB = (kPair ? kBN / 2 : kBN) / 64;   // 64-column TMA boxes this CTA loads per stage
  constexpr uint32_t kTmemCols = 2 * kBN;            // double-buffered accumulator
  constexpr uint32_t kIdesc = umma_idesc_bf16(kPair ? 2 * kBM : kBM, kBN, 0, 1);
  static_assert(kTmemCols == 128 || kTmemCols == 256 || kTmemCols == 512,
                "TMEM allocation must be a power of two");
  static_assert(!(kBatched && (kFused || kGated)), "the batched form is the plain GEMM + epilogue");
  static_assert(!(kPair && kBatched) && (!kPair || kBN == 256), "pairs work on 256 x 256 tiles of one matrix");
  // Split form (at most 32 output rows, a weight stream): the CTAs of a cluster share one
  // 256-column tile and each walks its own part of K; see the epilogue.
  static_assert(!kSplit || (kBN == 256 && !kFused && !kBatched && !kPair),
                "the split form works on 256 accumulator columns of one matrix (plain or gated)");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t staging_base = smem_base + kStages * kStage;
  uint8_t* staging = smem + kStages * kStage;
  const uint32_t bar_base = staging_base + kStagingBytes;
  // barrier layout (8 bytes each): full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  volatile uint32_t* tmem_holder =
      reinterpret_cast<volatile uint32_t*>(staging + kStagingBytes + 8 * (2 * kStages + 4));
  // fused form: counts epilogue warps whose stores of a tile have landed (four per tile); a
  // counter and not an mbarrier because the epilogue may run several tiles ahead of its reader
  const uint32_t stored_count = bar_base + 8u * (2 * kStages + 4) + 8u;
  // split form: partial_bar (first CTA) counts the bytes of the other CTAs' partial sums; go_bar
  // (other CTAs) is the first CTA's word that its stage ring is free to receive them
  const uint32_t partial_bar = stored_count + 8u;
  const uint32_t go_bar = stored_count + 16u;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Pair mode: CTA 0 of the cluster issues the MMAs; its `full` barriers count the bytes of both
  // CTAs' loads and its `tmem_empty` barriers the epilogue warps of both CTAs.
  const uint32_t rank = kPair ? cluster_rank() : 0u;
  const uint32_t split_rank = kSplit ? cluster_rank() : 0u;
  const uint32_t split_size = kSplit ? cluster_size() : 1u;
  const int first_unit = kPair ? int(blockIdx.x >> 1) : kSplit ? int(blockIdx.x / split_size) : int(blockIdx.x);
  const int unit_stride = kPair ? int(gridDim.x >> 1) : kSplit ? int(gridDim.x / split_size) : int(gridDim.x);
  const int num_units = kPair ? ((p.tiles_m + 1) / 2) * p.tiles_n : p.num_tiles;
  // K blocks this CTA walks (the launcher gives every CTA of a cluster at least one, and a
  // cluster exactly one tile)
  const int kb_begin = kSplit ? int(static_cast<long long>(split_rank) * p.num_kb / split_size) : 0;
  const int kb_end = kSplit ? int(static_cast<long long>(split_rank + 1) * p.num_kb / split_size) : p.num_kb;
  const uint32_t partial_bytes = kSplit ? uint32_t(p.split_rows) * kSplitPitch * 4u : 0u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), kPair ? 8 : 4);
    }
    asm volatile("st.shared::cta.u32 [%0], %1;" ::"r"(stored_count), "r"(0u) : "memory");
    if (kSplit) {
      mbar_init(partial_bar, 1);
      mbar_init(go_bar, 1);
      if (split_rank == 0) mbar_arrive_expect_tx(partial_bar, (split_size - 1u) * partial_bytes);
    }
    if (kFused && blockIdx.x == 0) g_fused_stamps[0] = global_ns();
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if (kGated) tma_prefetch_desc(&map_b2);
    tma_prefetch_desc(&map_out);
  }
  if (warp == 2) {
    if (kPair) {
      tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (kPair || kSplit) cluster_sync_all();   // the other CTAs' barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  if (!kFused) {
    // Set-up is done and has touched no operand: the next kernel of the stream may be scheduled,
    // and this one goes on once the previous kernel's results are visible.  (The form with the
    // cross-GPU sum is always launched the ordinary way.)
    grid_dependents_may_launch();
    grid_dependency_wait();
  }

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = first_unit; tile < num_units && ok; tile += unit_stride) {
        int m_blk, n_blk, flag_tile;
        const int z = kBatched ? tile / p.tiles_per_batch : 0;   // batch entry (tensor maps are 3-D)
        locate_tile<kPair>(p, kBatched ? tile - z * p.tiles_per_batch : tile, rank, m_blk, n_blk, flag_tile);
        const int m0 = m_blk * kBM;
        const int n0 = n_blk * kOutN;
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t phase = (it / kStages) & 1u;
          if (!mbar_wait(empty_bar(s), phase ^ 1u, 0x101)) { ok = false; break; }
          const uint32_t a_dst = smem_base + s * kStage;
          const uint32_t b_dst = a_dst + kStageBytesA;
          if (kPair) {
            // the issuing CTA expects the bytes of both CTAs on its barrier
            if (rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * kStage);
            const uint32_t bar = map_to_peer(full_bar(s), 0);
            tma_load_2d_pair(a_dst, &map_a, bar, kb * kBK, m0);
            // plain: this CTA's half of the 256 columns.  gated: this CTA's 64 of the tile's 128
            // output columns from the up weight, then the same 64 from the gate weight, so the
            // accumulator columns read [up 0-63 | gate 0-63 | up 64-127 | gate 64-127] and both
            // CTAs stream both weights.
#pragma unroll
            for (int j = 0; j < kChunksB; ++j) {
              if (kGated)
                tma_load_2d_pair(b_dst + j * 8192, j ? &map_b2 : &map_b, bar, n0 + int(rank) * 64, kb * kBK);
              else
                tma_load_2d_pair(b_dst + j * 8192, &map_b, bar, n0 + int(rank) * (kBN / 2) + j * 64, kb * kBK);
            }
            continue;
          }
          // (split form: the A box holds 32 or 64 rows; the MMA reads all 128 rows of the stage, and
          // what the other rows hold only reaches accumulator rows that are never stored)
          mbar_arrive_expect_tx(full_bar(s), kSplit ? kStage - kStageBytesA + p.split_a_rows * kBK * 2 : kStage);
          if (kBatched) {
            tma_load_3d(a_dst, &map_a, full_bar(s), kb * kBK, p.a_batch_inside ? z : m0,
                        p.a_batch_inside ? m0 : z);
#pragma unroll
            for (int j = 0; j < kChunksB; ++j)
              tma_load_3d(b_dst + j * 8192, &map_b, full_bar(s), n0 + j * 64, kb * kBK, p.b_shared ? 0 : z);
            continue;
          }
          tma_load_2d(a_dst, &map_a, full_bar(s), kb * kBK, m0);
#pragma unroll
          for (int j = 0; j < kChunksB; ++j) {
            if (kGated && j >= kChunksB / 2)
              tma_load_2d(b_dst + j * 8192, &map_b2, full_bar(s), n0 + (j - kChunksB / 2) * 64,
                          kb * kBK);
            else
              tma_load_2d(b_dst + j * 8192, &map_b, full_bar(s), n0 + j * 64, kb * kBK);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && rank == 0) {
      uint32_t it = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      for (int tile = first_unit; tile < num_units && ok; tile += unit_stride, ++local_tile) {
        const uint32_t acc = local_tile & 1u;
        const uint32_t acc_phase = (local_tile >> 1) & 1u;
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, 0x201)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t phase = (it / kStages) & 1u;
          if (!mbar_wait(full_bar(s), phase, 0x202)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + s * kStage;
          const uint32_t b_addr = a_addr + kStageBytesA;
#pragma unroll
          for (int k4 = 0; k4 < kBK / 16; ++k4) {
            // A: K-major, rows 128 B apart, 8-row groups 1024 B apart; 16 K elements = 32 B.
            const uint64_t a_desc = umma_smem_desc(a_addr + k4 * 32, 16, 1024);
            // B: N-major, 64-column chunks 8192 B apart, 8-row K groups 1024 B apart.
            const uint64_t b_desc = umma_smem_desc(b_addr + k4 * 2048, 8192, 1024);
            if (kPair)
              umma_bf16_ss_pair(d_tmem, a_desc, b_desc, kIdesc, (kb | k4) != 0 ? 1u : 0u);
            else
              umma_bf16_ss(d_tmem, a_desc, b_desc, kIdesc, (kb != kb_begin || k4 != 0) ? 1u : 0u);
          }
          if (kPair) umma_commit_pair(empty_bar(s)); else umma_commit(empty_bar(s));
        }
        if (ok) {
          if (kPair) umma_commit_pair(tmem_full_bar(acc)); else umma_commit(tmem_full_bar(acc));
        }
        if (kFused && blockIdx.x == 0) g_fused_stamps[1] = global_ns();
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    uint8_t* my_staging = staging + quad * 2 * kStoreBufBytes;
    const uint32_t my_staging_u32 = staging_base + quad * 2 * kStoreBufBytes;
    constexpr int kSubPerStore = kOutF32 ? 1 : 2;       // 32-column sub-chunks per 128 B row
    constexpr int kColsPerStore = 32 * kSubPerStore;
    uint32_t local_tile = 0;
    uint32_t store_buf = 0;
    bool ok = true;
    const int etid = threadIdx.x - 64;      // 0..127 within the epilogue group
    for (int unit = first_unit; unit < num_units && ok; unit += unit_stride, ++local_tile) {
      int m_blk, n_blk, tile;
      const int z = kBatched ? unit / p.tiles_per_batch : 0;
      locate_tile<kPair>(p, kBatched ? unit - z * p.tiles_per_batch : unit, rank, m_blk, n_blk, tile);
      const __nv_bfloat16* bias_base = p.bias + (kBatched ? z * p.stride_bias : 0);
      const int m0 = m_blk * kBM;
      const int n0 = n_blk * kOutN;
      const uint32_t acc = local_tile & 1u;
      const uint32_t acc_phase = (local_tile >> 1) & 1u;
      if (kFused || kSplit) {
        // a give-up must be uniform over the group because these paths use group barriers
        uint32_t good = mbar_wait(tmem_full_bar(acc), acc_phase, 0x301) ? 1u : 0u, all_good;
        asm volatile(
            "{\n"
            ".reg .pred a, b;\n"
            "setp.ne.u32 a, %1, 0;\n"
            "bar.red.and.pred b, 1, 128, a;\n"
            "selp.u32 %0, 1, 0, b;\n"
            "}\n"
            : "=r"(all_good)
            : "r"(good)
            : "memory");
        if (!all_good) { ok = false; break; }
      } else if (!mbar_wait(tmem_full_bar(acc), acc_phase, 0x301)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + quad * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kBN;
      float row_bias = 0.0f;
      if (p.bias_mode == TRINITY_SM100_BIAS_ROW_VECTOR && row < p.m)
        row_bias = __bfloat162float(bias_base[row]);
      if (kSplit) {
        // Split form.  The output has at most 64 rows, in the TMEM lanes of the first one or two
        // quadrants, which only those quadrants' warps can read.  Every CTA of the cluster holds
        // the sum over its own part of K; those warps lay it out in the CTA's idle stage ring as
        // [row][column] FP32.
        // The other CTAs send theirs into the first CTA's ring with one bulk copy per warp, once the
        // first CTA says its ring is idle too (its own MMAs have completed).  There all four
        // epilogue warps add the parts in a fixed order (own, then by CTA rank), so the result
        // does not depend on timing, apply the epilogue and store eight columns per thread.
        const int rows = p.split_rows;
        float* mine = reinterpret_cast<float*>(smem) +
                      (split_rank == 0 ? (split_size - 1u) * (partial_bytes / 4u) : 0u);
        const bool stages = quad * 32 < rows;   // this warp's TMEM lanes hold output rows
        if (split_rank == 0 && quad == 0 && lane == 0)
          for (uint32_t r = 1; r < split_size; ++r) mbar_arrive_cluster(map_to_peer(go_bar, r));
        if (stages) {
#pragma unroll 1
          for (int c0 = 0; c0 < kBN; c0 += 32) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(t_row + c0, v);
            tmem_ld_wait();
            if (quad * 32 + lane < rows) {
              float4* dst = reinterpret_cast<float4*>(mine + (quad * 32 + lane) * kSplitPitch + c0);
#pragma unroll
              for (int q = 0; q < 8; ++q)
                dst[q] = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                     __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
            }
          }
        }
        if (split_rank != 0) {
          if (stages) {
            // each warp sends the rows it laid out (a contiguous slab of the part)
            fence_async_smem();
            __syncwarp();
            if (!mbar_wait_cluster(go_bar, 0, 0x302)) { ok = false; break; }
            if (lane == 0) {
              const uint32_t slab_rows = uint32_t(min(32, rows - quad * 32));
              const uint32_t slab = uint32_t(quad) * 32u * kSplitPitch * 4u;
              asm volatile(
                  "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                  ::"r"(map_to_peer(smem_base + (split_rank - 1u) * partial_bytes + slab, 0)), "r"(smem_base + slab),
                    "r"(slab_rows * kSplitPitch * 4u), "r"(map_to_peer(partial_bar, 0))
                  : "memory");
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tmem_empty_bar(acc));
          continue;
        }
        {
          // the parts have landed and the first CTA's own part is laid out: a vote, so that a
          // wait that gave up takes the whole group out together
          uint32_t good = mbar_wait_cluster(partial_bar, 0, 0x303) ? 1u : 0u, all_good;
          asm volatile(
              "{\n"
              ".reg .pred a, b;\n"
              "setp.ne.u32 a, %1, 0;\n"
              "bar.red.and.pred b, 1, 128, a;\n"
              "selp.u32 %0, 1, 0, b;\n"
              "}\n"
              : "=r"(all_good)
              : "r"(good)
              : "memory");
          if (!all_good) { ok = false; break; }
        }
        const float* parts = reinterpret_cast<const float*>(smem);
        const uint32_t part_words = partial_bytes / 4u;
        const int out_row = etid % rows;
        // sum over the parts of eight accumulator columns from `first_col` on, own part first
        auto summed = [&](int first_col, float (&x)[8]) {
          const float4* own = reinterpret_cast<const float4*>(parts + (split_size - 1u) * part_words +
                                                              out_row * kSplitPitch + first_col);
          const float4 lo = own[0], hi = own[1];
          x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w;
          x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
          for (uint32_t r = 1; r < split_size; ++r) {
            const float4* theirs = reinterpret_cast<const float4*>(parts + (r - 1u) * part_words +
                                                                   out_row * kSplitPitch + first_col);
            const float4 tl = theirs[0], th = theirs[1];
            x[0] += tl.x; x[1] += tl.y; x[2] += tl.z; x[3] += tl.w;
            x[4] += th.x; x[5] += th.y; x[6] += th.z; x[7] += th.w;
          }
        };
        for (int cb = etid / rows; cb < kOutN / 8; cb += 128 / rows) {
          const int col = cb * 8, gcol = n0 + col;
          if (gcol >= p.n) break;
          float x[8];
          summed(col, x);
          if (kGated) {
            float gate[8];
            summed(kOutN + col, gate);
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] *= gate[j] * fast_sigmoid(gate[j]);
          }
          if (out_row >= p.m) continue;
          const bool whole = gcol + 8 <= p.n;
          if (p.bias_mode == TRINITY_SM100_BIAS_ROW_VECTOR) {
            const float b = __bfloat162float(bias_base[out_row]);
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] += b;
          } else if (p.bias_mode != TRINITY_SM100_BIAS_NONE) {
            const __nv_bfloat16* src = p.bias_mode == TRINITY_SM100_BIAS_COL_VECTOR
                                           ? bias_base + gcol
                                           : bias_base + static_cast<long long>(out_row) * p.ld_bias + gcol;
            if (whole) {
              const uint4 b = __ldg(reinterpret_cast<const uint4*>(src));
              const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                x[e * 2] += bf16_lo(w[e]);
                x[e * 2 + 1] += bf16_hi(w[e]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (gcol + j < p.n) x[j] += __bfloat162float(src[j]);
            }
          }
          if (!kGated && p.activation != TRINITY_SM100_ACT_NONE) {
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = apply_activation(x[j], p.activation);
          }
          if (kOutF32) {
            float* dst = static_cast<float*>(p.out) + static_cast<long long>(out_row) * p.ldo + gcol;
            if (whole) {
              reinterpret_cast<float4*>(dst)[0] = make_float4(x[0], x[1], x[2], x[3]);
              reinterpret_cast<float4*>(dst)[1] = make_float4(x[4], x[5], x[6], x[7]);
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (gcol + j < p.n) dst[j] = x[j];
            }
          } else {
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(out_row) * p.ldo + gcol;
            if (whole) {
              *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]),
                                                          pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (gcol + j < p.n) dst[j] = __float2bfloat16(x[j]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tmem_empty_bar(acc));
        continue;
      }

      for (int c0 = 0; c0 < kOutN; c0 += kColsPerStore) {
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        uint8_t* buf = my_staging + store_buf * kStoreBufBytes;
#pragma unroll
        for (int sub = 0; sub < kSubPerStore; ++sub) {
          const int col = c0 + sub * 32;
          // accumulator columns of this sub-chunk's values and (gated form) of its gates
          const int acc_col = (kPair && kGated) ? (col / 64) * 128 + col % 64 : col;
          const int gate_col = (kPair && kGated) ? acc_col + 64 : kOutN + col;
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_row + acc_col, v);
          float x[32];
          if (kGated) {
            uint32_t g[32];
            tmem_ld_32x32b_x32(t_row + gate_col, g);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float gate = __uint_as_float(g[j]);
              x[j] = __uint_as_float(v[j]) * (gate * fast_sigmoid(gate));
            }
          } else {
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] = __uint_as_float(v[j]);
          }
          const int gcol = n0 + col;
          if (p.bias_mode == TRINITY_SM100_BIAS_COL_VECTOR) {
            if (gcol + 32 <= p.n) {
              const uint4* src = reinterpret_cast<const uint4*>(bias_base + gcol);
#pragma unroll
              for (int v4 = 0; v4 < 4; ++v4) {
                const uint4 b = __ldg(src + v4);
                const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  x[v4 * 8 + e * 2] += bf16_lo(w[e]);
                  x[v4 * 8 + e * 2 + 1] += bf16_hi(w[e]);
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (gcol + j < p.n) x[j] += __bfloat162float(bias_base[gcol + j]);
            }
          } else if (p.bias_mode == TRINITY_SM100_BIAS_ROW_VECTOR) {
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] += row_bias;
          } else if (p.bias_mode == TRINITY_SM100_BIAS_MATRIX) {
            if (row < p.m) {
              const __nv_bfloat16* brow = bias_base + static_cast<long long>(row) * p.ld_bias + gcol;
              if (gcol + 32 <= p.n) {
                const uint4* src = reinterpret_cast<const uint4*>(brow);
#pragma unroll
                for (int v4 = 0; v4 < 4; ++v4) {
                  const uint4 b = __ldg(src + v4);
                  const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    x[v4 * 8 + e * 2] += bf16_lo(w[e]);
                    x[v4 * 8 + e * 2 + 1] += bf16_hi(w[e]);
                  }
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (gcol + j < p.n) x[j] += __bfloat162float(brow[j]);
              }
            }
          }
          if (!kGated && p.activation != TRINITY_SM100_ACT_NONE) {
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] = apply_activation(x[j], p.activation);
          }
          // Staging row `lane` is 128 B = eight 16 B units; unit u lives at u ^ (lane & 7).
          uint8_t* srow = buf + lane * 128;
          if (kOutF32) {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              uint4 o;
              o.x = __float_as_uint(x[u * 4 + 0]);
              o.y = __float_as_uint(x[u * 4 + 1]);
              o.z = __float_as_uint(x[u * 4 + 2]);
              o.w = __float_as_uint(x[u * 4 + 3]);
              *reinterpret_cast<uint4*>(srow + ((u ^ (lane & 7)) << 4)) = o;
            }
          } else {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 o;
              o.x = pack_bf16x2(x[u * 8 + 0], x[u * 8 + 1]);
              o.y = pack_bf16x2(x[u * 8 + 2], x[u * 8 + 3]);
              o.z = pack_bf16x2(x[u * 8 + 4], x[u * 8 + 5]);
              o.w = pack_bf16x2(x[u * 8 + 6], x[u * 8 + 7]);
              const int unit = sub * 4 + u;
              *reinterpret_cast<uint4*>(srow + ((unit ^ (lane & 7)) << 4)) = o;
            }
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (m0 + quad * 32 < p.m && n0 + c0 < p.n) {
            if (kBatched)
              tma_store_3d(&map_out, my_staging_u32 + store_buf * kStoreBufBytes, n0 + c0,
                           p.out_batch_inside ? z : m0 + quad * 32, p.out_batch_inside ? m0 + quad * 32 : z);
            else
              tma_store_2d(&map_out, my_staging_u32 + store_buf * kStoreBufBytes, n0 + c0,
                           m0 + quad * 32);
          }
          tma_store_commit();
        }
        store_buf ^= 1u;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (kPair) mbar_arrive_cluster(map_to_peer(tmem_empty_bar(acc), 0));
        else mbar_arrive(tmem_empty_bar(acc));
      }
      if (kFused) {
        if (lane == 0) {
          // Once this warp's part of the partial tile has landed in memory the warp is free for
          // the next tile; telling the other GPUs (a system-scope release, which waits for
          // writes in flight) is left to the signalling warp.
          tma_store_wait_all();
          asm volatile("red.release.cta.shared::cta.add.u32 [%0], 1;" ::"r"(stored_count) : "memory");
        }
        if (blockIdx.x == 0 && etid == 0) g_fused_stamps[2] = global_ns();
      }
    }
    if (lane == 0) tma_store_wait_all();
  }
  if (kFused && warp == 10) {
    // ------------------------------------------------------------ signalling warp (fused all-reduce)
    // Lane r tells rank r's reducer warps (this rank's own included) that this rank's partial of a
    // tile is complete in memory, as soon as the epilogue warps' stores of the tile have landed.
    // A warp of its own: the system-scope release of the flag store waits for the storing
    // thread's earlier writes, and a reducer thread has 28 pushes across NVLink in flight per tile,
    // which put a second round trip into every tile's chain while the reducers sent the flags.
    // The give-up case is caught by the reducers' flag wait: nobody will have flagged the tile.
    if (lane < peers.world) {
      uint32_t local_tile = 0;
      bool landed = true;
      for (int unit = first_unit; unit < num_units && landed; unit += unit_stride, ++local_tile) {
        int m_blk, n_blk, tile;
        locate_tile<kPair>(p, unit, rank, m_blk, n_blk, tile);
        const uint32_t target = 4u * (local_tile + 1u);
        const long long start = clock64();
        landed = false;
        for (;;) {
          uint32_t seen;
          asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(seen) : "r"(stored_count) : "memory");
          if (static_cast<int32_t>(seen - target) >= 0) { landed = true; break; }
          if (clock64() - start > wait_budget()) { report_timeout(0x803); break; }
          __nanosleep(100);
        }
        if (landed)
          flag_store(peers.flags[lane] + static_cast<long long>(tile) * peers.world + peers.rank, peers.epoch);
      }
    }
  } else if (kFused && warp >= 6) {
    // ------------------------------------------------------------ reducer warps (fused all-reduce)
    // They follow the CTA's own tile sequence: the same CTA index on every rank works on the same
    // tile at about the same time, so the partials of a tile arrive together.
    const int rtid = threadIdx.x - kGemmThreads;
    bool ok = true;
    uint32_t local_tile = 0;
    for (int unit = first_unit; unit < num_units && ok; unit += unit_stride, ++local_tile) {
      int m_blk, n_blk, tile;
      locate_tile<kPair>(p, unit, rank, m_blk, n_blk, tile);
      ok = reduce_owned_tile<kBN>(p, peers, tile, m_blk * kBM, n_blk * kBN, rtid, 2);
    }
    if (blockIdx.x == 0 && rtid == 0) g_fused_stamps[3] = global_ns();
    {
      // Retire: once every CTA of this rank has pushed its tiles, tell the peers; the last CTA
      // stays until every peer has said the same, so the output is complete when the kernel ends.
      __threadfence_system();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (rtid == 0) {
        uint32_t* mine = peers.flags[peers.rank] + static_cast<long long>(p.flag_tiles) * peers.world;
        const unsigned prev = atomicAdd(mine + kGemmMaxWorld, 1u);
        if (prev == gridDim.x - 1) {
          mine[kGemmMaxWorld] = 0;
          if (peers.epoch_counter) *reinterpret_cast<volatile uint32_t*>(peers.epoch_counter) = peers.epoch;
          __threadfence_system();
          for (int r = 0; r < peers.world; ++r)
            flag_store(peers.flags[r] + static_cast<long long>(p.flag_tiles) * peers.world + peers.rank, peers.epoch);
          for (int r = 0; r < peers.world; ++r)
            if (!wait_flag(mine + r, peers.epoch, 0x802)) break;
        }
        if (blockIdx.x == 0) g_fused_stamps[4] = global_ns();
      }
    }
  }

  // Common exit: every role leaves its loop (normally or after a wait gave up) and meets here.
  // In pair mode neither CTA leaves while the other may still arrive on its barriers or its MMAs
  // read this CTA's shared memory; in the split form none leaves while its partial sums are
  // still being copied out of its shared memory (the first CTA comes here after it has them).
  tc_fence_before();
  __syncthreads();
  if (kPair || kSplit) cluster_sync_all();
  if (warp == 2) {
    if (g_device_status != 0) {
      // A wait gave up somewhere: give copies still in flight time to land before the
      // shared memory and TMEM of this CTA are released.
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    if (kPair) tmem_dealloc_pair(tmem_base, kTmemCols); else tmem_dealloc(tmem_base, kTmemCols);
  }
}

#pragma nv_diag_default 128

// Shared-memory opt-in of one instantiation, once per device.
template <int kBN, int kStages, bool kGated, bool kOutF32, bool kFused = false, bool kBatched = false,
          bool kPair = false, bool kSplit = false>
int opt_in_gemm() {
  static unsigned long long configured = 0;
  return opt_in_shared_memory(
      reinterpret_cast<const void*>(
          &gemm_bf16_tcgen05_kernel<kBN, kStages, kGated, kOutF32, kFused, kBatched, kPair, kSplit>),
      gemm_smem_bytes<kBN, kStages, kPair>(), &configured, "gemm");
}

// How many two-CTA clusters of a pair-mode instantiation the current device keeps resident at
// once (one CTA per SM; a GPC with an odd number of SMs leaves one unpaired).  Cached per device.
template <int kBN, int kStages, bool kGated, bool kOutF32, bool kFused>
int resident_pairs(int* pairs) {
  static std::mutex mutex;
  static int cached[64] = {};
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= 64)
    return fail(TRINITY_SM100_E_CUDA, "gemm: cudaGetDevice: %s", cudaGetErrorString(e));
  std::lock_guard<std::mutex> lock(mutex);
  if (!cached[device]) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * 148);
    config.blockDim = dim3(kFused ? kGemmFusedThreads : kGemmThreads);
    config.dynamicSmemBytes = gemm_smem_bytes<kBN, kStages, true>();
    cudaLaunchAttribute cluster;
    cluster.id = cudaLaunchAttributeClusterDimension;
    cluster.val.clusterDim.x = 2;
    cluster.val.clusterDim.y = 1;
    cluster.val.clusterDim.z = 1;
    config.attrs = &cluster;
    config.numAttrs = 1;
    int count = 0;
    e = cudaOccupancyMaxActiveClusters(
        &count, gemm_bf16_tcgen05_kernel<kBN, kStages, kGated, kOutF32, kFused, false, true>, &config);
    if (e != cudaSuccess || count < 1)
      return fail(TRINITY_SM100_E_CUDA, "gemm: cluster occupancy query: %s (%d clusters)", cudaGetErrorString(e),
                  count);
    cached[device] = count;
  }
  *pairs = cached[device];
  return 0;
}

template <int kBN, int kStages, bool kGated, bool kOutF32, bool kFused = false, bool kBatched = false,
          bool kPair = false, bool kSplit = false>
int launch_gemm(const trinity_sm100_gemm& g, int sm_count, cudaStream_t stream, const GemmPeers* fused = nullptr,
                const trinity_sm100_gemm_batch* batch = nullptr, int split = 1) {
  constexpr int kOutN = kGated ? kBN / 2 : kBN;
  constexpr int kSmem = gemm_smem_bytes<kBN, kStages, kPair>();
  static_assert(kSmem <= 232448, "exceeds the 227 KB shared-memory limit");
  auto kernel = gemm_bf16_tcgen05_kernel<kBN, kStages, kGated, kOutF32, kFused, kBatched, kPair, kSplit>;
  if (int rc = opt_in_gemm<kBN, kStages, kGated, kOutF32, kFused, kBatched, kPair, kSplit>()) return rc;
  CUtensorMap map_a, map_b, map_b2, map_out;
  int rc;
  const int out_bytes = kOutF32 ? 4 : 2;
  const long long entries = kBatched ? batch->batch : 1;
  if (kBatched) {
    // a third, outermost axis over the batch entries; a shared right operand keeps extent 1
    const bool shared_b = batch->stride_b == 0;
    if (batch->stride_a < g.lda) {
      if ((rc = make_tensor_map_3d(&map_a, g.a, 2, g.k, entries, g.m, batch->stride_a * 2, g.lda * 2, kBK, 1, kBM, 128)))
        return rc;
    } else if ((rc = make_tensor_map_3d(&map_a, g.a, 2, g.k, g.m, entries, g.lda * 2, batch->stride_a * 2, kBK, kBM, 1, 128))) {
      return rc;
    }
    if ((rc = make_tensor_map_3d(&map_b, g.b, 2, g.n, g.k, shared_b ? 1 : entries, g.ldb * 2,
                                 shared_b ? g.ldb * 2 * g.k : batch->stride_b * 2, 64, kBK, 1, 128)))
      return rc;
    map_b2 = map_b;
    if (batch->stride_out < g.ldo) {
      if ((rc = make_tensor_map_3d(&map_out, g.out, out_bytes, g.n, entries, g.m, batch->stride_out * out_bytes,
                                   g.ldo * out_bytes, 128 / out_bytes, 1, 32, 128)))
        return rc;
    } else if ((rc = make_tensor_map_3d(&map_out, g.out, out_bytes, g.n, g.m, entries, g.ldo * out_bytes,
                                        batch->stride_out * out_bytes, 128 / out_bytes, 32, 1, 128))) {
      return rc;
    }
  } else {
    if ((rc = make_tensor_map_2d(&map_a, g.a, 2, g.k, g.m, g.lda * 2, kBK, kSplit ? (g.m <= 32 ? 32 : 64) : kBM, true)))
      return rc;
    if ((rc = make_tensor_map_2d(&map_b, g.b, 2, g.n, g.k, g.ldb * 2, 64, kBK, true))) return rc;
    if ((rc = make_tensor_map_2d(&map_b2, kGated ? g.b2 : g.b, 2, g.n, g.k, g.ldb * 2, 64, kBK,
                                 true)))
      return rc;
    if ((rc = make_tensor_map_2d(&map_out, g.out, out_bytes, g.n, g.m, g.ldo * out_bytes,
                                 128 / out_bytes, 32, true)))
      return rc;
  }
  GemmParams p;
  p.bias = static_cast<const __nv_bfloat16*>(g.bias);
  p.ld_bias = g.ld_bias;
  p.bias_mode = g.bias_mode;
  p.activation = g.activation;
  p.m = int(g.m);
  p.n = int(g.n);
  p.k = int(g.k);
  p.tiles_m = int((g.m + kBM - 1) / kBM);
  p.tiles_n = int((g.n + kOutN - 1) / kOutN);
  p.tiles_per_batch = p.tiles_m * p.tiles_n;
  p.num_tiles = int(p.tiles_per_batch * entries);
  p.b_shared = kBatched && batch->stride_b == 0 ? 1 : 0;
  p.a_batch_inside = kBatched && batch->stride_a < g.lda ? 1 : 0;
  p.out_batch_inside = kBatched && batch->stride_out < g.ldo ? 1 : 0;
  p.stride_bias = kBatched ? batch->stride_bias : 0;
  p.num_kb = int((g.k + kBK - 1) / kBK);
  p.flag_tiles = (p.tiles_m + 1) / 2 * 2 * p.tiles_n;
  p.split_rows = g.m <= 16 ? 16 : g.m <= 32 ? 32 : 64;
  p.split_a_rows = g.m <= 32 ? 32 : 64;
  p.out = g.out;
  p.ldo = g.ldo;
  GemmPeers peers = {};
  if (fused) peers = *fused;
  if constexpr (kSplit) {
    // one cluster of `split` CTAs per column tile, each CTA a part of K
    if (p.tiles_m != 1 || g.m > kSplitRowsMax || split < 2 || split > 8 || p.num_kb < split ||
        static_cast<size_t>(split) * p.split_rows * kSplitPitch * 4 > static_cast<size_t>(kStages) * stage_bytes<kBN>())
      return fail(TRINITY_SM100_E_INVALID, "gemm (split form): %d rows, %d K blocks, %d parts", int(g.m), p.num_kb, split);
    KernelLaunch launch(dim3(p.num_tiles * split), dim3(kGemmThreads), kSmem, stream, unsigned(split));
    cudaError_t e = cudaLaunchKernelEx(&launch.config, kernel, map_a, map_b, map_b2, map_out, p, peers);
    if (e != cudaSuccess) return fail(TRINITY_SM100_E_CUDA, "gemm_bf16_tcgen05 (split) launch: %s", cudaGetErrorString(e));
    count_launch();
    return check_launch("gemm_bf16_tcgen05");
  }
  if constexpr (kPair) {
    // a persistent grid of as many CTA pairs as are resident together
    int pairs = 0;
    if ((rc = resident_pairs<kBN, kStages, kGated, kOutF32, kFused>(&pairs))) return rc;
    const int units = (p.tiles_m + 1) / 2 * p.tiles_n;
    if (units < pairs) pairs = units;
    KernelLaunch launch(dim3(2 * pairs), dim3(kFused ? kGemmFusedThreads : kGemmThreads), kSmem, stream, 2);
    if (kFused) launch.config.numAttrs = 1;   // the cluster only: no early start beside a cross-GPU exchange
    cudaError_t e = cudaLaunchKernelEx(&launch.config, kernel, map_a, map_b, map_b2, map_out, p, peers);
    if (e != cudaSuccess) return fail(TRINITY_SM100_E_CUDA, "gemm_bf16_tcgen05 (pairs) launch: %s", cudaGetErrorString(e));
    count_launch();
    return check_launch("gemm_bf16_tcgen05");
  }
  const int grid = p.num_tiles < sm_count ? p.num_tiles : sm_count;
  KernelLaunch launch(dim3(grid), dim3(kFused ? kGemmFusedThreads : kGemmThreads), kSmem, stream);
  if (kFused) launch.config.numAttrs = 0;
  cudaError_t e = cudaLaunchKernelEx(&launch.config, kernel, map_a, map_b, map_b2, map_out, p, peers);
  if (e != cudaSuccess) return fail(TRINITY_SM100_E_CUDA, "gemm_bf16_tcgen05 launch: %s", cudaGetErrorString(e));
  count_launch();
  return check_launch("gemm_bf16_tcgen05");
}

}  // namespace

int gemm_prepare_device() {
  // every instantiation an entry point can select
  int rc = 0;
#define TRINITY_OPT_IN(...) if (!rc) rc = opt_in_gemm<__VA_ARGS__>();
  TRINITY_OPT_IN(256, 4, true, true) TRINITY_OPT_IN(256, 4, true, false)
  TRINITY_OPT_IN(256, 4, false, true) TRINITY_OPT_IN(256, 4, false, false)
  TRINITY_OPT_IN(128, 6, false, true) TRINITY_OPT_IN(128, 6, false, false)
  TRINITY_OPT_IN(64, 8, false, true) TRINITY_OPT_IN(64, 8, false, false)
  TRINITY_OPT_IN(256, 4, false, true, false, true) TRINITY_OPT_IN(256, 4, false, false, false, true)
  TRINITY_OPT_IN(128, 6, false, true, false, true) TRINITY_OPT_IN(128, 6, false, false, false, true)
  TRINITY_OPT_IN(64, 8, false, true, false, true) TRINITY_OPT_IN(64, 8, false, false, false, true)
  TRINITY_OPT_IN(256, 4, false, false, true)
  TRINITY_OPT_IN(256, kPairStages, true, true, false, false, true) TRINITY_OPT_IN(256, kPairStages, true, false, false, false, true)
  TRINITY_OPT_IN(256, kPairStages, false, true, false, false, true) TRINITY_OPT_IN(256, kPairStages, false, false, false, false, true)
  TRINITY_OPT_IN(256, kPairStages, false, false, true, false, true)
  TRINITY_OPT_IN(256, 4, false, true, false, false, false, true) TRINITY_OPT_IN(256, 4, false, false, false, false, false, true)
  TRINITY_OPT_IN(256, 4, true, true, false, false, false, true) TRINITY_OPT_IN(256, 4, true, false, false, false, false, true)
#undef TRINITY_OPT_IN
  return rc;
}
}  // namespace trinity_sm100

using namespace trinity_sm100;

namespace {
// Argument checks shared by the single and the batched entry point.
int check_gemm_arguments(const trinity_sm100_gemm& g) {
  const bool gated = g.activation == TRINITY_SM100_ACT_SILU_GATE;
  if (!g.a || !g.b || !g.out) return fail(TRINITY_SM100_E_INVALID, "gemm: null operand");
  if (g.m <= 0 || g.n <= 0 || g.k <= 0 || g.m > INT32_MAX || g.n > INT32_MAX || g.k > INT32_MAX)
    return fail(TRINITY_SM100_E_INVALID, "gemm: extents must be in [1, 2^31)");
  if (gated && !g.b2) return fail(TRINITY_SM100_E_INVALID, "gemm: gated form needs b2");
  if (g.activation < TRINITY_SM100_ACT_NONE || g.activation > TRINITY_SM100_ACT_SILU_GATE)
    return fail(TRINITY_SM100_E_INVALID, "gemm: unknown activation %d", g.activation);
  if (g.bias_mode < TRINITY_SM100_BIAS_NONE || g.bias_mode > TRINITY_SM100_BIAS_MATRIX)
    return fail(TRINITY_SM100_E_INVALID, "gemm: unknown bias mode %d", g.bias_mode);
  if (g.bias_mode != TRINITY_SM100_BIAS_NONE && !g.bias)
    return fail(TRINITY_SM100_E_INVALID, "gemm: bias mode %d without a bias pointer", g.bias_mode);
  if (gated && g.bias_mode != TRINITY_SM100_BIAS_NONE)
    return fail(TRINITY_SM100_E_UNSUPPORTED, "gemm: the gated form takes no bias");
  if (g.out_dtype != TRINITY_SM100_BF16 && g.out_dtype != TRINITY_SM100_FP32)
    return fail(TRINITY_SM100_E_INVALID, "gemm: unknown output dtype %d", g.out_dtype);
  if (g.lda < g.k || g.ldb < g.n || g.ldo < g.n)
    return fail(TRINITY_SM100_E_INVALID, "gemm: leading dimension smaller than the row");
  const int out_bytes = g.out_dtype == TRINITY_SM100_FP32 ? 4 : 2;
  if (g.lda % 8 || g.ldb % 8 || (g.ldo * out_bytes) % 16)
    return fail(TRINITY_SM100_E_INVALID,
                "gemm: row pitches must be multiples of 16 bytes (lda %lld, ldb %lld, ldo %lld)",
                (long long)g.lda, (long long)g.ldb, (long long)g.ldo);
  if (!aligned16(g.a) || !aligned16(g.b) || !aligned16(g.out) || (gated && !aligned16(g.b2)))
    return fail(TRINITY_SM100_E_INVALID, "gemm: operand pointers must be 16-byte aligned");
  if (g.bias_mode == TRINITY_SM100_BIAS_COL_VECTOR && !aligned16(g.bias))
    return fail(TRINITY_SM100_E_INVALID, "gemm: bias vector must be 16-byte aligned");
  if (g.bias_mode == TRINITY_SM100_BIAS_MATRIX &&
      (!aligned16(g.bias) || g.ld_bias % 8 || g.ld_bias < g.n))
    return fail(TRINITY_SM100_E_INVALID, "gemm: bias matrix needs 16-byte aligned rows");
  return 0;
}
}  // namespace

namespace {
// Set by the workspace entry point around its call of the host-epoch entry point (same thread).
thread_local uint32_t* g_epoch_counter_for_next_launch = nullptr;
// TRINITY_SM100_GEMM_PAIRS=0 keeps every GEMM on single CTAs; =1 (default) lets large plain and
// all-reduce-fused problems run on CTA pairs; =2 also the gated form, which measures slower on
// pairs than on single CTAs (B200, 16384 x 8192 x 28672) and therefore stays on single CTAs by
// default.  Read at every call; a tuning override, not part of the ABI.
int pairs_mode() {
  const char* v = getenv("TRINITY_SM100_GEMM_PAIRS");
  return v && v[0] >= '0' && v[0] <= '2' ? v[0] - '0' : 1;
}
bool pairs_allowed() { return pairs_mode() != 0; }
}  // namespace

// CTA pairs of the plain pair-mode GEMM that the current device keeps resident at once.
extern "C" int trinity_sm100_gemm_pair_capacity(int32_t* pairs) {
  if (!pairs) return fail(TRINITY_SM100_E_INVALID, "gemm_pair_capacity: null pointer");
  if (int rc = require_sm100(nullptr)) return rc;
  if (int rc = opt_in_gemm<256, kPairStages, false, false, false, false, true>()) return rc;
  int count = 0;
  if (int rc = resident_pairs<256, kPairStages, false, false, false>(&count)) return rc;
  *pairs = count;
  return 0;
}

extern "C" int trinity_sm100_gemm_bf16(const trinity_sm100_gemm* args, void* stream_handle) {
  if (!args) return fail(TRINITY_SM100_E_INVALID, "gemm: null argument block");
  const trinity_sm100_gemm& g = *args;
  if (int rc = check_gemm_arguments(g)) return rc;
  const bool gated = g.activation == TRINITY_SM100_ACT_SILU_GATE;
  int sm_count = 0;
  if (int rc = require_sm100(&sm_count)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  const bool f32 = g.out_dtype == TRINITY_SM100_FP32;
  const long long row_tiles = (g.m + kBM - 1) / kBM;
  // CTA pairs once there are at least as many 256-row x 256-column (gated: x 128) pair tiles as
  // SM pairs; an odd last row tile costs its pair half a tile of zero work.
  const long long pair_units = (row_tiles + 1) / 2 * ((g.n + (gated ? 127 : 255)) / (gated ? 128 : 256));
  const bool pairs = pairs_allowed() && row_tiles >= 2 && pair_units >= sm_count / 2;
  // One row tile (decode-time GEMMs: a few output rows against a large weight) makes the kernel
  // a weight stream.  An MMA with both operands in shared memory takes 128 cycles or more
  // whatever its width (measured: 128 at 256 columns, 165 at 64), so only tiles of 256
  // accumulator columns, 8 KB of weights per MMA, let an SM take in weights faster than its
  // share of the memory bandwidth.  With fewer such tiles than half the SMs and at most 64 rows,
  // the CTAs of a cluster share a tile and each walks a part of K (up to 8 parts for 16 rows, 4
  // for 32, 2 for 64, while every part keeps at least four K blocks: the parts' partial sums
  // must fit the stage ring).
  const long long wide_tiles = row_tiles * ((g.n + (gated ? 127 : 255)) / (gated ? 128 : 256));
  int split = 1;
  if (row_tiles == 1 && g.m <= kSplitRowsMax) {
    const long long k_blocks = (g.k + kBK - 1) / kBK;
    while (split < (g.m <= 16 ? 8 : g.m <= 32 ? 4 : 2) && wide_tiles * split * 2 <= sm_count && k_blocks >= split * 2 * 4) split *= 2;
  }
  if (gated) {
    if (split > 1)
      return f32 ? launch_gemm<256, 4, true, true, false, false, false, true>(g, sm_count, stream, nullptr, nullptr, split)
                 : launch_gemm<256, 4, true, false, false, false, false, true>(g, sm_count, stream, nullptr, nullptr, split);
    if (pairs && pairs_mode() == 2)
      return f32 ? launch_gemm<256, kPairStages, true, true, false, false, true>(g, sm_count, stream)
                 : launch_gemm<256, kPairStages, true, false, false, false, true>(g, sm_count, stream);
    return f32 ? launch_gemm<256, 4, true, true>(g, sm_count, stream)
               : launch_gemm<256, 4, true, false>(g, sm_count, stream);
  }
  if (pairs)
    return f32 ? launch_gemm<256, kPairStages, false, true, false, false, true>(g, sm_count, stream)
               : launch_gemm<256, kPairStages, false, false, false, false, true>(g, sm_count, stream);
  if (row_tiles == 1) {
    if (split > 1)
      return f32 ? launch_gemm<256, 4, false, true, false, false, false, true>(g, sm_count, stream, nullptr, nullptr, split)
                 : launch_gemm<256, 4, false, false, false, false, false, true>(g, sm_count, stream, nullptr, nullptr, split);
    if (wide_tiles * 2 > sm_count)
      return f32 ? launch_gemm<256, 4, false, true>(g, sm_count, stream)
                 : launch_gemm<256, 4, false, false>(g, sm_count, stream);
  }
  // Wide tiles once there are enough of them to fill the machine.  Otherwise the tile width
  // that finishes in the fewest column-steps: a persistent CTA works through
  // ceil(tiles / SMs) tiles of that width.
  if (wide_tiles >= sm_count) {
    return f32 ? launch_gemm<256, 4, false, true>(g, sm_count, stream)
               : launch_gemm<256, 4, false, false>(g, sm_count, stream);
  }
  const long long steps128 = (row_tiles * ((g.n + 127) / 128) + sm_count - 1) / sm_count * 128;
  const long long steps64 = (row_tiles * ((g.n + 63) / 64) + sm_count - 1) / sm_count * 64;
  if (steps64 < steps128) {
    return f32 ? launch_gemm<64, 8, false, true>(g, sm_count, stream)
               : launch_gemm<64, 8, false, false>(g, sm_count, stream);
  }
  return f32 ? launch_gemm<128, 6, false, true>(g, sm_count, stream)
             : launch_gemm<128, 6, false, false>(g, sm_count, stream);
}

extern "C" int trinity_sm100_gemm_batched_bf16(const trinity_sm100_gemm* args,
                                               const trinity_sm100_gemm_batch* batch, void* stream_handle) {
  if (!args || !batch) return fail(TRINITY_SM100_E_INVALID, "gemm_batched: null argument block");
  const trinity_sm100_gemm& g = *args;
  const trinity_sm100_gemm_batch& b = *batch;
  if (int rc = check_gemm_arguments(g)) return rc;
  if (g.activation == TRINITY_SM100_ACT_SILU_GATE)
    return fail(TRINITY_SM100_E_UNSUPPORTED, "gemm_batched: the gated form is not batched");
  if (b.batch <= 0 || b.batch > 65535) return fail(TRINITY_SM100_E_INVALID, "gemm_batched: batch must be in [1, 65535]");
  const int out_bytes = g.out_dtype == TRINITY_SM100_FP32 ? 4 : 2;
  if (b.stride_a <= 0 || b.stride_a % 8 || b.stride_b < 0 || b.stride_b % 8 || b.stride_out <= 0 ||
      (b.stride_out * out_bytes) % 16)
    return fail(TRINITY_SM100_E_INVALID,
                "gemm_batched: strides must be positive multiples of 16 bytes (stride_b may be 0 for a shared operand)");
  if (g.bias_mode != TRINITY_SM100_BIAS_NONE && (b.stride_bias < 0 || b.stride_bias % 8))
    return fail(TRINITY_SM100_E_INVALID, "gemm_batched: stride_bias must be a non-negative multiple of 8 elements");
  const long long row_tiles = (g.m + kBM - 1) / kBM;
  if (row_tiles * ((g.n + 63) / 64) * b.batch > INT32_MAX)
    return fail(TRINITY_SM100_E_UNSUPPORTED, "gemm_batched: too many tiles");
  int sm_count = 0;
  if (int rc = require_sm100(&sm_count)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  const bool f32 = g.out_dtype == TRINITY_SM100_FP32;
  // tile width as for the single GEMM, counting the tiles of all batch entries
  if (row_tiles * ((g.n + 255) / 256) * b.batch >= sm_count)
    return f32 ? launch_gemm<256, 4, false, true, false, true>(g, sm_count, stream, nullptr, &b)
               : launch_gemm<256, 4, false, false, false, true>(g, sm_count, stream, nullptr, &b);
  const long long steps128 = (row_tiles * ((g.n + 127) / 128) * b.batch + sm_count - 1) / sm_count * 128;
  const long long steps64 = (row_tiles * ((g.n + 63) / 64) * b.batch + sm_count - 1) / sm_count * 64;
  if (steps64 < steps128)
    return f32 ? launch_gemm<64, 8, false, true, false, true>(g, sm_count, stream, nullptr, &b)
               : launch_gemm<64, 8, false, false, false, true>(g, sm_count, stream, nullptr, &b);
  return f32 ? launch_gemm<128, 6, false, true, false, true>(g, sm_count, stream, nullptr, &b)
             : launch_gemm<128, 6, false, false, false, true>(g, sm_count, stream, nullptr, &b);
}

extern "C" size_t trinity_sm100_gemm_allreduce_flag_words(int64_t m, int64_t n, int32_t world) {
  if (m <= 0 || n <= 0 || world <= 0) return 0;
  // numbered over 128-row tiles with the row-tile count rounded up to even (CTA pairs)
  const size_t tiles = (size_t((m + kBM - 1) / kBM) + 1) / 2 * 2 * size_t((n + 255) / 256);
  return kGemmFlagOffset + tiles * size_t(world) + kGemmMaxWorld + 8;
}

// stamps[0..4]: kernel start, last MMA committed, last partial tile handed over, last owned rows
// reduced, all ranks retired - nanoseconds of the device's global timer, written by CTA 0 of the
// most recent fused launch on the current device.  Synchronises the device.
extern "C" int trinity_sm100_gemm_allreduce_stamps(uint64_t* stamps) {
  if (!stamps) return fail(TRINITY_SM100_E_INVALID, "gemm_allreduce_stamps: null pointer");
  unsigned long long host[8];
  cudaError_t e = cudaMemcpyFromSymbol(host, g_fused_stamps, sizeof(host));
  if (e != cudaSuccess) return fail(TRINITY_SM100_E_CUDA, "gemm_allreduce_stamps: %s", cudaGetErrorString(e));
  for (int i = 0; i < 5; ++i) stamps[i] = host[i];
  return 0;
}

namespace {
// Peer tables of persistent workspaces, read from the device once per workspace and kept: the
// table is written once, before the first launch, and only its counters change afterwards.
struct CachedTable {
  void* workspace;
  trinity_sm100_peer_table table;
};
int cached_peer_table(void* workspace, trinity_sm100_peer_table* out) {
  static std::mutex mutex;
  static std::vector<CachedTable> known;
  std::lock_guard<std::mutex> lock(mutex);
  for (auto& entry : known)
    if (entry.workspace == workspace) {
      *out = entry.table;
      return 0;
    }
  CachedTable entry;
  entry.workspace = workspace;
  cudaError_t e = cudaMemcpy(&entry.table, workspace, sizeof(entry.table), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess)
    return fail(TRINITY_SM100_E_CUDA, "reading the workspace's peer table: %s", cudaGetErrorString(e));
  known.push_back(entry);
  *out = entry.table;
  return 0;
}
}  // namespace

extern "C" size_t trinity_sm100_gemm_allreduce_workspace_bytes(int64_t m, int64_t n, int32_t world) {
  return TRINITY_SM100_PEER_TABLE_BYTES + 4 * trinity_sm100_gemm_allreduce_flag_words(m, n, world);
}

extern "C" int trinity_sm100_gemm_allreduce_workspace_bf16(const trinity_sm100_gemm* args, void* workspace,
                                                           size_t workspace_bytes, int32_t output_buffer,
                                                           void* stream_handle) {
  if (!args || !workspace) return fail(TRINITY_SM100_E_INVALID, "gemm_allreduce (workspace): null argument");
  if (output_buffer < 0 || output_buffer >= TRINITY_SM100_PEER_BUFFERS)
    return fail(TRINITY_SM100_E_INVALID, "gemm_allreduce (workspace): symmetric buffer index %d", output_buffer);
  trinity_sm100_peer_table table;
  if (int rc = cached_peer_table(workspace, &table)) return rc;
  if (table.world < 1 || table.world > kGemmMaxWorld || table.rank < 0 || table.rank >= table.world)
    return fail(TRINITY_SM100_E_INVALID, "gemm_allreduce (workspace): the peer table is not filled");
  if (workspace_bytes < trinity_sm100_gemm_allreduce_workspace_bytes(args->m, args->n, table.world))
    return fail(TRINITY_SM100_E_INVALID, "gemm_allreduce (workspace): workspace of %zu bytes is too small", workspace_bytes);
  void* peers[kGemmMaxWorld];
  void* flags[kGemmMaxWorld];
  for (int r = 0; r < table.world; ++r) {
    peers[r] = reinterpret_cast<void*>(table.buffers[output_buffer][r]);
    // the flag pad follows the table in every rank's workspace
    flags[r] = reinterpret_cast<uint8_t*>(table.workspace[r]) + TRINITY_SM100_PEER_TABLE_BYTES;
  }
  trinity_sm100_allreduce reduce = {};
  reduce.peers = peers;
  reduce.flags = flags;
  reduce.rows = args->m;
  reduce.cols = args->n;
  reduce.world = table.world;
  reduce.rank = table.rank;
  reduce.epoch = 1;   // replaced on the device by the table's own counter
  g_epoch_counter_for_next_launch = &static_cast<trinity_sm100_peer_table*>(workspace)->epoch;
  const int rc = trinity_sm100_gemm_allreduce_bf16(args, &reduce, stream_handle);
  g_epoch_counter_for_next_launch = nullptr;
  return rc;
}

extern "C" int trinity_sm100_gemm_allreduce_bf16(const trinity_sm100_gemm* args,
                                                 const trinity_sm100_allreduce* reduce, void* stream_handle) {
  if (!args || !reduce) return fail(TRINITY_SM100_E_INVALID, "gemm_allreduce: null argument block");
  const trinity_sm100_gemm& g = *args;
  const trinity_sm100_allreduce& r = *reduce;
  if (!g.a || !g.b || !g.out) return fail(TRINITY_SM100_E_INVALID, "gemm_allreduce: null operand");
  if (g.m <= 0 || g.n <= 0 || g.k <= 0 || g.m > INT32_MAX || g.n > INT32_MAX || g.k > INT32_MAX)
    return fail(TRINITY_SM100_E_INVALID, "gemm_allreduce: extents must be in [1, 2^31)");
  if (g.activation != TRINITY_SM100_ACT_NONE || g.bias_mode != TRINITY_SM100_BIAS_NONE ||
      g.out_dtype != TRINITY_SM100_BF16)
    return fail(TRINITY_SM100_E_UNSUPPORTED,
                "gemm_allreduce: the partial products are summed across ranks, so no bias or activation, BF16 out");
  if (g.lda % 8 || g.ldb % 8 || g.ldo % 8 || g.n % 8 || g.lda < g.k || g.ldb < g.n || g.ldo < g.n)
    return fail(TRINITY_SM100_E_INVALID, "gemm_allreduce: pitches and n must be multiples of 8 elements");
  if (r.world != 1 && r.world != 2 && r.world != 4 && r.world != 8)
    return fail(TRINITY_SM100_E_UNSUPPORTED, "gemm_allreduce: world must be 1, 2, 4 or 8 (row slices of a 128-row tile)");
  if (!r.peers || !r.flags || r.world < 1 || r.world > kGemmMaxWorld || r.rank < 0 || r.rank >= r.world)
    return fail(TRINITY_SM100_E_INVALID, "gemm_allreduce: world %d / rank %d or pointer tables invalid", r.world, r.rank);
  if (r.rows != g.m || r.cols != g.n)
    return fail(TRINITY_SM100_E_INVALID, "gemm_allreduce: reduce extents differ from the output");
  GemmPeers peers = {};
  for (int i = 0; i < r.world; ++i) {
    if (!r.peers[i] || !r.flags[i] || !aligned16(r.peers[i]) || !aligned16(r.flags[i]))
      return fail(TRINITY_SM100_E_INVALID, "gemm_allreduce: peer %d pointer null or misaligned", i);
    peers.buffers[i] = static_cast<uint4*>(r.peers[i]);
    peers.flags[i] = static_cast<uint32_t*>(r.flags[i]) + kGemmFlagOffset;
  }
  if (r.epoch == 0)
    return fail(TRINITY_SM100_E_INVALID, "gemm_allreduce: epoch 0 is what a fresh flag pad holds; start at 1");
  if (r.peers[r.rank] != g.out)
    return fail(TRINITY_SM100_E_INVALID, "gemm_allreduce: out must be this rank's entry of the peer table");
  if (!aligned16(g.a) || !aligned16(g.b)) return fail(TRINITY_SM100_E_INVALID, "gemm_allreduce: operands must be 16-byte aligned");
  peers.world = r.world;
  peers.rank = r.rank;
  peers.epoch = r.epoch;
  peers.epoch_counter = g_epoch_counter_for_next_launch;
  peers.ld_vectors = g.ldo / 8;
  // the reducer threads index the buffers in 16-byte vectors with 32 bits
  if (((g.m + kBM - 1) / kBM * kBM) * (g.ldo / 8) >= (1ll << 32))
    return fail(TRINITY_SM100_E_UNSUPPORTED, "gemm_allreduce: output of %lld x %lld elements is too large", (long long)g.m,
                (long long)g.ldo);
  int sm_count = 0;
  if (int rc = require_sm100(&sm_count)) return rc;
  // every CTA of the persistent grid is resident (one per SM), which the flag waits rely on
  const long long row_tiles = (g.m + kBM - 1) / kBM;
  if (pairs_allowed() && row_tiles >= 2 && (row_tiles + 1) / 2 * ((g.n + 255) / 256) >= sm_count / 2)
    return launch_gemm<256, kPairStages, false, false, true, false, true>(g, sm_count, static_cast<cudaStream_t>(stream_handle), &peers);
  return launch_gemm<256, 4, false, false, true>(g, sm_count, static_cast<cudaStream_t>(stream_handle), &peers);
}
