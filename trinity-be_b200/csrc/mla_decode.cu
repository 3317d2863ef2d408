// Batched MLA decode over a compressed KV cache (one query token, up to 128 heads).
//
//   S = scale * q . cache^T      [heads x seq]      tcgen05, FP32 scores in TMEM
//   P = exp(S - max) (online)                        FP32 in registers, BF16 back into TMEM
//   O = P @ cache[:, :512] / sum(P)  [heads x 512]  tcgen05, FP32 accumulator in TMEM
//
// A 128-row FP32 accumulator for all 512 latent columns would fill TMEM by itself, and a
// tcgen05.mma costs about 45 cycles however narrow it is, so the work of one (batch, KV split)
// is shared by a cluster of two CTAs that split the *feature* axis:
//
//   CTA c owns latent columns [256c, 256c+256) and rope features [32c, 32c+32).
//   scores:  each CTA contracts only its 288 features (18 K-steps, N = 64 positions) into a
//            partial score tile.  The partial tiles are exchanged through distributed shared
//            memory with a bulk asynchronous copy in 16 bits per score (16.5 KB per chunk and
//            direction); each CTA adds the peer's tile to its own exact FP32 tile.  Sixteen bits
//            halve the exchange, which measures ~18 B/clk per SM and would otherwise bound the
//            kernel.  The format is chosen per head and chunk from the largest magnitude `top` of
//            the row's partials: FP16 values while top * |scale| * log2(e) <= 8 (their error,
//            2^-11 of each partial, then stays below 2^-8 in the scaled log2 logit, 0.3 % in a
//            weight); beyond that 16-bit integers in units of top / 32767, whose error is the same
//            for every position of the row, 2^-16 of top (an error relative to each element, as
//            FP16 has, would be 32 times larger on exactly the large partials that decide the
//            weights).  Stated bound for the peer's half of a scaled log2 logit:
//            max(2^-8, 2^-16 * top * |scale| * log2(e)), i.e. below 2^-7 up to scaled partials
//            of 512.
//            The two CTAs hold logits that differ in the last bits; each normalises its own
//            columns with its own sums, so every output column is a consistent softmax.
//   values:  each CTA multiplies its probabilities with its own 256 latent columns, which
//            are exactly the cache bytes it already loaded for the scores
//
// So every cache byte is loaded exactly once per cluster, no score FLOP is duplicated, and the
// query half (256 latent + 32 rope features) lives in TMEM as the A operand of every score MMA.
// TMEM: accumulator 256 columns, one 64-column score buffer, one 32-column probability buffer,
// query 144 columns.  Shared memory: four 36 KB cache stages (four 128-byte-swizzled latent boxes
// and one 64-byte-swizzled rope box of 32 features), two receive and two send tiles of 16 KB.
//
//   warp 0    TMA producer (the cache chunk ring: 4 latent boxes + rope box per chunk)
//   warp 1    score MMA issuer: QK(j) = 18 TMEM-A MMAs (N=64), issued as soon as the softmax
//             group has copied the scores of chunk j-1 out of TMEM and the chunk's cache stage
//             has landed, so the scores run ahead of the values by up to the depth of the ring
//   warp 14   value MMA issuer: PV(j) = 4 TMEM-A MMAs (N=256), issued when the chunk's
//             probabilities are in TMEM
//   warps 2-13 three softmax groups of four warps; group g takes the chunks with j % 3 == g and
//             one thread handles a head's whole 64-position row of a chunk: partial-score load,
//             exchange with the peer CTA, row maximum, exponentials, BF16 probabilities into
//             their TMEM buffer.  While one group waits for the peer's tile the others compute.
//             The running reference maximum of a head passes from group to group through
//             shared memory (one mbarrier per TMEM lane quadrant orders the hand-over); the
//             accumulator is rescaled only when the maximum grows by more than 2^8.
//
// With kv_splits == 1 the CTA writes BF16 output directly.  Otherwise it writes a normalised
// FP32 partial and its log-sum-exp (one per feature half) to scratch and a small kernel merges
// the splits.  Algorithmic traffic: q + cache + out bytes; the scratch adds 2 * splits * batch *
// heads * 514 * 4 bytes when splits > 1.
#include "host_common.h"
#include <cuda_fp16.h>

#include "sm100_ptx.cuh"

namespace trinity_sm100 {
namespace {

constexpr int kGroups = 3;                       // softmax groups; group g owns chunks j % kGroups == g
constexpr int kSoftmaxWarps = 4 * kGroups;       // four warps (one per TMEM lane quadrant) per group
constexpr int kSoftmaxThreads = kSoftmaxWarps * 32;
// producer, score MMA issuer, softmax groups, value MMA issuer
constexpr int kMlaThreads = 64 + kSoftmaxThreads + 32;
constexpr int kKv = 64;                        // cache positions per chunk
constexpr int kDqk = 576, kDv = 512;
constexpr int kKvStages = 4;
constexpr int kPrefetchAhead = 4;              // chunks requested into L2 beyond the stage ring
constexpr int kBoxBytes = kKv * 128;           // 8192: one [64 positions x 64 features] box
constexpr int kRopeBoxBytes = kKv * 64;        // 4096: [64 positions x 32 rope features]
constexpr int kStageBytes = 4 * kBoxBytes + kRopeBoxBytes;  // 36864
constexpr int kXchgTileBytes = 128 * kKv * 2;  // one partial score tile as 16-bit integers: 16384
constexpr int kXchgBytes = kXchgTileBytes + 128 * 4;   // ... and one FP32 unit per row
constexpr int kQueryBoxBytes = 128 * 64;       // [128 heads x 32 features] of the query
constexpr int kQueryLandingBytes = 9 * kQueryBoxBytes;   // eight latent boxes and the rope box
static_assert(kQueryLandingBytes <= 2 * kStageBytes && kKvStages >= 4, "the query lands in cache stages 2 and 3");
// two receive tiles + two send tiles: the exchange of chunk j+1 overlaps the softmax of chunk j
constexpr int kMlaSmem = 1024 + kKvStages * kStageBytes + 4 * kXchgBytes + 512;
// TMEM columns: accumulator, scores, probabilities, query (128 latent + 16 rope word columns)
constexpr uint32_t kColO = 0, kColS = 256, kColP = 320, kColQ = 352, kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;      // in log2 units: probabilities stay below 2^8

struct MlaParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  float* partial_o;   // [batch][splits][heads][512]
  float* partial_lse; // [batch][pieces][heads][2 feature halves]
  int batch, heads, seq;
  int chunks_per_seq;
  int pieces;         // partial slots per sequence: the KV splits, or the most pieces a sequence is cut into
  int balanced;       // 0: grid (2, splits, batch), one segment per cluster; 1: grid (2, clusters), see unit_begin
  int clusters;
  long long units;    // batch * chunks_per_seq
  float scale_log2;   // |scale| * log2(e)
  int negate;         // scale < 0: the query's sign is flipped on its way into TMEM
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same with the shared-memory descriptor given as two words: within a stage only the low word
// (the address field) changes from MMA to MMA, so the issuing thread adds 32-bit constants.
__device__ __forceinline__ void umma_bf16_ts_split(uint32_t d_tmem, uint32_t a_tmem, uint32_t desc_lo,
                                                   uint32_t desc_hi, uint32_t idesc,
                                                   uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 desc;\n"
      "mov.b64 desc, {%2, %3};\n"
      "setp.ne.b32 p, %5, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], desc, %4, p;\n"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "r"(desc_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---- more thread-block-cluster helpers (the basic ones are in sm100_ptx.cuh)
__device__ __forceinline__ void st_peer_v4(uint32_t remote_addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"r"(remote_addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
// Arrive on a barrier in the peer CTA without ordering earlier memory operations.  The callers
// acknowledge shared-memory reads whose values they have already used, so there is nothing to
// release; the releasing form stalls the issuing thread for about a thousand cycles.
__device__ __forceinline__ void mbar_arrive_peer_relaxed(uint32_t remote_bar) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
// Chunk range [first, first + count) of split `s` when `chunks` are dealt out evenly.
__host__ __device__ inline void split_range(int chunks, int splits, int s, int& first, int& count) {
  const int base = chunks / splits, extra = chunks % splits;
  first = s * base + (s < extra ? s : extra);
  count = base + (s < extra ? 1 : 0);
}

// Balanced schedule: the (batch x chunks-per-sequence) chunks of the whole call, numbered row by
// row, are cut into `clusters` contiguous runs of equal length (to within one chunk).  Cluster k
// owns units [unit_begin(k), unit_begin(k + 1)).
__host__ __device__ inline long long unit_begin(long long units, int clusters, int k) {
  return units * k / clusters;
}
// The cluster whose run contains unit u: the largest k with unit_begin(k) <= u.
__host__ __device__ inline int cluster_of_unit(long long units, int clusters, long long u) {
  return int(((u + 1) * clusters + units - 1) / units) - 1;
}

// One piece of work of a cluster: `num_chunks` chunks of sequence `b` starting at `first_chunk`.
// `whole` pieces cover their sequence alone and write BF16 output; the others write a partial
// into `slot`.
struct Segment {
  int b, first_chunk, num_chunks;
  long long slot;
  bool whole;
};
// The i-th segment of the cluster with grid coordinates (y, z); false when it has no such segment.
// Host and device: the host side serves trinity_sm100_mla_schedule_segment.
__host__ __device__ inline bool segment_of(const MlaParams& p, int y, int z, int i, Segment& s) {
  if (p.balanced == 0) {
    if (i != 0) return false;
    s.b = z;
    split_range(p.chunks_per_seq, p.pieces, y, s.first_chunk, s.num_chunks);
    s.slot = static_cast<long long>(s.b) * p.pieces + y;
    s.whole = p.pieces == 1;
    return s.num_chunks > 0;
  }
  const int k = y;
  const long long u0 = unit_begin(p.units, p.clusters, k), u1 = unit_begin(p.units, p.clusters, k + 1);
  const long long cps = p.chunks_per_seq;
  const long long b = u0 / cps + i;
  const long long lo = b * cps > u0 ? b * cps : u0;
  const long long hi = (b + 1) * cps < u1 ? (b + 1) * cps : u1;
  if (lo >= hi) return false;
  s.b = int(b);
  s.first_chunk = int(lo - b * cps);
  s.num_chunks = int(hi - lo);
  s.slot = b * p.pieces + (k - cluster_of_unit(p.units, p.clusters, b * cps));
  s.whole = s.num_chunks == p.chunks_per_seq;
  return true;
}
__device__ __forceinline__ bool get_segment(const MlaParams& p, int i, Segment& s) {
  return segment_of(p, blockIdx.y, blockIdx.z, i, s);
}

__global__ void __launch_bounds__(kMlaThreads, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap map_cache,
                  const __grid_constant__ CUtensorMap map_rope,
                  const __grid_constant__ CUtensorMap map_query, const MlaParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ float m_shared[128];               // reference maximum of each head (log2 domain)
  __shared__ float l_part[kGroups * 128];       // [group][head] sums of probabilities at the end
  __shared__ unsigned read_count_storage[2];    // per receive tile: warps that have read it
  volatile unsigned* read_count = read_count_storage;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t kv_smem = smem_base;                                 // cache stage ring
  const uint32_t xchg_smem = kv_smem + kKvStages * kStageBytes;       // peer's partial scores land here
  const uint32_t send_smem = xchg_smem + 2 * kXchgBytes;               // my partial scores, staged for the copy
  const uint32_t bar_base = xchg_smem + 4 * kXchgBytes;
  uint8_t* xchg = smem + kKvStages * kStageBytes;
  uint8_t* send = xchg + 2 * kXchgBytes;
  // A cluster works through its segments one after the other; chunks are counted across
  // segments (g below), and every barrier's phase follows from that count, so all roles agree on
  // the phases without resetting anything between segments.
  // barriers: kv_full[stages], kv_empty[stages], x_full[2], x_empty[2], s_full[3], pv_done[3],
  //           s_free, p_full, q_tmem, o_free, m_ready[3][4].  s_free and p_full complete once per
  //           chunk and are waited on by one thread, chunk after chunk (chunk g is phase g & 1).
  //           s_full and pv_done are waited on by the softmax groups, which see only every third
  //           chunk; a parity wait is only meaningful on consecutive phases, so these two (and
  //           m_ready) exist once per group (chunk g is phase (g / 3) & 1 of barrier g % 3).
  //           q_tmem and o_free complete once per segment.
  auto kv_full = [&](int s) { return bar_base + 8u * s; };
  auto kv_empty = [&](int s) { return bar_base + 8u * (kKvStages + s); };
  auto x_full = [&](int b) { return bar_base + 8u * (2 * kKvStages + b); };
  auto x_empty = [&](int b) { return bar_base + 8u * (2 * kKvStages + 2 + b); };
  auto s_full = [&](int c) { return bar_base + 8u * (2 * kKvStages + 4 + c % kGroups); };              // scores of chunk c are in TMEM
  auto pv_done = [&](int c) { return bar_base + 8u * (2 * kKvStages + 4 + kGroups + c % kGroups); };   // values of chunk c are accumulated
  auto group_phase = [](int c) { return static_cast<uint32_t>((c / kGroups) & 1); };
  const uint32_t s_free = bar_base + 8u * (2 * kKvStages + 4 + 2 * kGroups);   // the scores have been copied out
  const uint32_t p_full = s_free + 8u;                                         // probabilities are in TMEM
  const uint32_t q_tmem = s_free + 16u;                                        // the segment's query is in TMEM
  const uint32_t o_free = s_free + 24u;                                        // the segment's accumulator has been read
  // m_ready[group][quadrant]: the reference maxima after chunk c are in m_shared (one arrival a
  // chunk, by the warp of group c % 3 that serves the quadrant)
  auto m_ready = [&](int c, int q) { return s_free + 32u + 8u * ((c % kGroups) * 4 + q); };
  // q_land: the first segment's query has landed in shared memory (see the producer)
  const uint32_t q_land = s_free + 32u + 8u * (4 * kGroups);
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(
      xchg + 4 * kXchgBytes + 8 * (2 * kKvStages + 4 + 2 * kGroups + 5 + 4 * kGroups));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t half = cluster_rank();   // latent half and rope half owned by this CTA
  const uint32_t peer = half ^ 1u;

  if (threadIdx.x == 0) {
    read_count_storage[0] = 0;
    read_count_storage[1] = 0;
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(x_full(i), 1);     // local arm (expect_tx) + the peer's bulk copy bytes
      mbar_init(x_empty(i), 4);    // the peer's four warps that have read the tile
    }
    for (int i = 0; i < kGroups; ++i) {
      mbar_init(s_full(i), 1);
      mbar_init(pv_done(i), 1);
    }
    mbar_init(s_free, 4);        // the four warps of the group that owns the chunk
    mbar_init(p_full, 4);
    mbar_init(q_tmem, kSoftmaxWarps);
    mbar_init(o_free, kSoftmaxWarps);
    mbar_init(q_land, 1);
    for (int q = 0; q < 4 * kGroups; ++q) mbar_init(m_ready(q >> 2, q & 3), 1);
    mbar_fence_init();
    tma_prefetch_desc(&map_cache);
    tma_prefetch_desc(&map_rope);
    tma_prefetch_desc(&map_query);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // set-up done, no operand touched yet (see KernelLaunch)
  grid_dependents_may_launch();
  grid_dependency_wait();
  Segment seg;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // A stage is held from its load until the chunk's values are accumulated, several
      // thousand cycles, so the ring alone keeps too few bytes in flight to cover the memory
      // latency.  Chunks further ahead are therefore requested into L2 first; the ring's own
      // loads then find them there.
      // The softmax threads read the query one head per lane, 16 bytes at a time from rows 1152
      // bytes apart, which DRAM serves slowly (microseconds for a few megabytes over all CTAs).
      // So each CTA first asks for its half of the heads' rows as one contiguous range into L2
      // (both CTAs read every row), and for the next segment's rows a whole segment ahead.
      auto prefetch_query = [&](const Segment& sg) {
        const int first = int(half) * 64;
        const int count = p.heads - first < 64 ? p.heads - first : 64;
        if (count > 0)
          bulk_prefetch_l2(p.q + (static_cast<long long>(sg.b) * p.heads + first) * kDqk,
                           uint32_t(count) * kDqk * 2);
      };
      int g = 0;
      bool ok = true;
      // The first segment's query comes by TMA instead: nine [128 heads x 32 features] boxes
      // (64-byte swizzle) into cache stages 2 and 3, which stay empty until the query has been
      // moved on into tensor memory (see below).  That takes the query off the slow per-lane path
      // exactly where nothing can hide it, at the start of the kernel.
      if (get_segment(p, 0, seg)) {
        mbar_arrive_expect_tx(q_land, kQueryLandingBytes);
#pragma unroll
        for (int i = 0; i < 9; ++i)
          tma_load_3d(kv_smem + 2 * kStageBytes + i * kQueryBoxBytes, &map_query, q_land,
                      i < 8 ? int(half) * 256 + i * 32 : kDv + int(half) * 32, 0, seg.b);
      }
      for (int si = 0; ok && get_segment(p, si, seg); ++si) {
        {
          Segment next;
          if (get_segment(p, si + 1, next)) prefetch_query(next);
        }
        auto prefetch_chunk = [&](int c) {
          if (c >= seg.num_chunks) return;
          const int kv0 = (seg.first_chunk + c) * kKv;
#pragma unroll
          for (int f = 0; f < 4; ++f)
            tma_prefetch_l2_3d(&map_cache, int(half) * 256 + f * 64, kv0, seg.b);
          tma_prefetch_l2_3d(&map_rope, kDv + int(half) * 32, kv0, seg.b);
        };
        for (int j = 0; j < seg.num_chunks; ++j, ++g) {
          const int s = g % kKvStages;
          const uint32_t phase = (g / kKvStages) & 1u;
          // Requests into L2 run a fixed distance ahead of the ring's loads, and never ahead of
          // the loads that fill the empty ring at the start: those must not queue behind them.
          if (j >= kKvStages) prefetch_chunk(j + kPrefetchAhead);
          // Stages 2 and 3 hold the first segment's query until it has been moved into tensor
          // memory; the third chunk's load waits for that.  (It also keeps the start of the kernel,
          // where every CTA asks for its query and its ring at once, from queueing the query
          // behind the whole ring.)
          if (g == 2 && !mbar_wait(q_tmem, 0, 0x402)) { ok = false; break; }
          if (!mbar_wait(kv_empty(s), phase ^ 1u, 0x401)) { ok = false; break; }
          mbar_arrive_expect_tx(kv_full(s), kStageBytes);
          const int kv0 = (seg.first_chunk + j) * kKv;
          const uint32_t dst = kv_smem + s * kStageBytes;
#pragma unroll
          for (int f = 0; f < 4; ++f)
            tma_load_3d(dst + f * kBoxBytes, &map_cache, kv_full(s), int(half) * 256 + f * 64, kv0, seg.b);
          tma_load_3d(dst + 4 * kBoxBytes, &map_rope, kv_full(s), kDv + int(half) * 32, kv0, seg.b);
          if (j == kKvStages - 1)
            for (int c = kKvStages; c < kKvStages + kPrefetchAhead; ++c) prefetch_chunk(c);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ score MMA issuer
    // Scores and values are issued by different threads so that neither waits for the other's
    // inputs: the scores of a chunk need its cache stage and a score buffer that the softmax
    // group has copied out (they run ahead of the values by as many chunks as there are stages
    // to hold), the values need the chunk's probabilities.  An issuing thread shares its
    // scheduler with three softmax warps and every instruction between two MMAs costs
    // tensor-pipe time, so one descriptor per operand kind is built per chunk and the K-steps
    // only add constants to its address field (units of 16 bytes; the field cannot overflow,
    // shared memory ends below 256 KB).
    // The whole warp runs the loops (so that chunk counters, stage addresses and descriptors are
    // warp-uniform values the compiler can keep in uniform registers, which is where the MMA
    // instruction takes them from); lane 0 alone issues the MMAs and the commits.
    {
      constexpr uint32_t kIdescQK = umma_idesc_bf16(128, kKv, 0, 0);
      const uint32_t d_scores = tmem_base + kColS, a_query = tmem_base + kColQ;
      int g = 0;
      bool ok = true;
      for (int si = 0; ok && get_segment(p, si, seg); ++si) {
        ok = __all_sync(0xffffffffu, mbar_wait(q_tmem, si & 1u, 0x502));
        for (int j = 0; ok && j < seg.num_chunks; ++j, ++g) {
          if (g > 0) ok = __all_sync(0xffffffffu, mbar_wait(s_free, (g - 1) & 1u, 0x505));
          if (ok) ok = __all_sync(0xffffffffu, mbar_wait(kv_full(g % kKvStages), (g / kKvStages) & 1u, 0x503));
          if (!ok) break;
          tc_fence_after();
          // 16 K-steps over the latent boxes and 2 over the rope box, the query always from TMEM
          const uint32_t stage = kv_smem + (g % kKvStages) * kStageBytes;
          const uint64_t latent = umma_smem_desc(stage, 16, 1024);
          const uint64_t rope = umma_smem_desc_sw64(stage + 4 * kBoxBytes, 512);
          const uint32_t latent_lo = uint32_t(latent), latent_hi = uint32_t(latent >> 32);
          const uint32_t rope_lo = uint32_t(rope), rope_hi = uint32_t(rope >> 32);
          const uint32_t done_bar = s_full(g);
          if (lane == 0) {
#pragma unroll
            for (int ks = 0; ks < 16; ++ks)
              umma_bf16_ts_split(d_scores, a_query + ks * 8,
                                 latent_lo + (((ks / 4) * kBoxBytes + (ks % 4) * 32) >> 4), latent_hi,
                                 kIdescQK, ks != 0);
#pragma unroll
            for (int r = 0; r < 2; ++r)
              umma_bf16_ts_split(d_scores, a_query + 128 + r * 8, rope_lo + ((r * 32) >> 4), rope_hi,
                                 kIdescQK, 1u);
            umma_commit(done_bar);
          }
          __syncwarp();
        }
      }
    }
  } else if (warp == 2 + kSoftmaxWarps) {
    // ------------------------------------------------------------ value MMA issuer
    // Probabilities from TMEM, the chunk's latent boxes N-major (64-latent boxes 8192 B apart,
    // 8-position groups 1024 B apart).  Warp-uniform loops, lane 0 issues (see above).
    {
      constexpr uint32_t kIdescPV = umma_idesc_bf16(128, 256, 0, 1);
      const uint32_t d_out = tmem_base + kColO, a_prob = tmem_base + kColP;
      int g = 0;
      bool ok = true;
      for (int si = 0; ok && get_segment(p, si, seg); ++si) {
        // the previous segment's accumulator must have been read before it is overwritten
        if (si > 0) ok = __all_sync(0xffffffffu, mbar_wait(o_free, (si - 1) & 1u, 0x506));
        for (int j = 0; ok && j < seg.num_chunks; ++j, ++g) {
          ok = __all_sync(0xffffffffu, mbar_wait(p_full, g & 1u, 0x504));
          if (!ok) break;
          tc_fence_after();
          const int s = g % kKvStages;
          const uint64_t values = umma_smem_desc(kv_smem + s * kStageBytes, kBoxBytes, 1024);
          const uint32_t free_bar = kv_empty(s), done_bar = pv_done(g);
          if (lane == 0) {
#pragma unroll
            for (int ks = 0; ks < kKv / 16; ++ks)
              umma_bf16_ts(d_out, a_prob + ks * 8, values + ((ks * 2048) >> 4), kIdescPV, (j | ks) != 0);
            umma_commit(free_bar);
            umma_commit(done_bar);
          }
          __syncwarp();
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / epilogue warps
    // Warp w reads the TMEM lanes of quadrant (w & 3); the warps w, w+4, w+8 of the three groups
    // serve the same 32 heads in turn.
    const int quad = warp & 3;
    const int group = (warp - 2) >> 2;
    const int row = quad * 32 + lane;              // head index
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const bool live = row < p.heads;
    // A wait that gives up only sets `bad`: the thread keeps executing the warp- and
    // group-collective instructions (on meaningless data) and the threads of a group leave
    // together at the next vote, so no barrier or collective is ever left half-attended.
    bool bad = false;
    int gbase = 0;   // chunks of earlier segments

    for (int si = 0; get_segment(p, si, seg); ++si) {
      const int num_chunks = seg.num_chunks;
      {
        // This CTA's query features -> TMEM as packed BF16 pairs: four blocks of 64 latent
        // features and one of 32 rope features, dealt out to the groups.  (All MMAs of the
        // previous segment have completed: its epilogue waited for the last of them.)
        const uint32_t flip = p.negate ? 0x80008000u : 0u;
        if (si == 0) {
          // From the landing zone: box i holds features [32 i, 32 i + 32) of this CTA's half (box 8
          // the rope features), one 64-byte row per head with its 16-byte units swizzled by
          // (row >> 1) & 3; heads beyond p.heads were filled with zeros.  Group g takes boxes g,
          // g + 3 and g + 6, each 16 columns of packed pairs.
          if (!bad) bad = !mbar_wait(q_land, 0, 0x608);
          const uint8_t* landing = smem + 2 * kStageBytes;
#pragma unroll
          for (int i = 0; i < 3; ++i) {
            const int box = group + i * kGroups;
            const uint8_t* src = landing + box * kQueryBoxBytes + row * 64;
            uint32_t w[16];
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const uint4 x = *reinterpret_cast<const uint4*>(src + ((v ^ ((row >> 1) & 3)) << 4));
              w[v * 4 + 0] = x.x ^ flip; w[v * 4 + 1] = x.y ^ flip;
              w[v * 4 + 2] = x.z ^ flip; w[v * 4 + 3] = x.w ^ flip;
            }
            tmem_st_32x32b_x16(lane_base + kColQ + (box < 8 ? box * 16 : 128), w);
          }
        } else {
        const __nv_bfloat16* qhead =
            p.q + (static_cast<long long>(seg.b) * p.heads + (live ? row : 0)) * kDqk;
        // Group g takes blocks g and g + 3; all loads are issued before the first is used.
        uint4 x[2][8];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int blk = group + i * kGroups;
          const uint4* src = reinterpret_cast<const uint4*>(blk < 4 ? qhead + half * 256 + blk * 64
                                                                    : qhead + kDv + half * 32);
#pragma unroll
          for (int v = 0; v < 8; ++v)
            x[i][v] = (live && blk < 5 && (blk < 4 || v < 4)) ? __ldg(src + v) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int blk = group + i * kGroups;
          uint32_t w[32];
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            w[v * 4 + 0] = x[i][v].x ^ flip; w[v * 4 + 1] = x[i][v].y ^ flip;
            w[v * 4 + 2] = x[i][v].z ^ flip; w[v * 4 + 3] = x[i][v].w ^ flip;
          }
          if (blk < 4) {
            tmem_st_32x32b_x32(lane_base + kColQ + blk * 32, w);
          } else if (blk == 4) {
            uint32_t r[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) r[k] = w[k];
            tmem_st_32x32b_x16(lane_base + kColQ + 128, r);
          }
        }
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(q_tmem);
      }

      float m_l = -INFINITY;     // reference maximum that `l` is relative to
      float l = 0.0f;            // sum of this thread's probabilities
      // this group's chunks of the segment: those whose running number is group (mod 3)
      for (int j = (group + kGroups - gbase % kGroups) % kGroups; j < num_chunks; j += kGroups) {
        const int g = gbase + j;
        // exchange tiles alternate between two buffers by chunk parity
        const int buf = g & 1;
        const uint32_t phase = (g >> 1) & 1u;
        uint4* staged = reinterpret_cast<uint4*>(send + buf * kXchgBytes);
        const uint4* received = reinterpret_cast<const uint4*>(xchg + buf * kXchgBytes);
        // ---- partial scores of this CTA's feature half: TMEM -> registers
        if (!bad) bad = !mbar_wait(s_full(g), group_phase(g), 0x601);
        tc_fence_after();
        float t[64];
        {
          uint32_t lo[32], hi[32];
          tmem_ld_32x32b_x32(lane_base + kColS, lo);
          tmem_ld_32x32b_x32(lane_base + kColS + 32, hi);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            t[i] = __uint_as_float(lo[i]);
            t[32 + i] = __uint_as_float(hi[i]);
          }
        }
        // the scores are in registers: later score MMAs may overwrite the buffer
        tc_fence_before();
        if (__all_sync(0xffffffffu, !bad) && lane == 0) mbar_arrive(s_free);
        // ---- 16-bit copy for the peer: [8 groups of 8 positions][128 rows] (conflict-free), FP16
        //      or integers in units of 1/32767 of the row's largest magnitude, with the unit (0
        //      for FP16) behind the tile; then one thread starts the bulk asynchronous copy into
        //      the peer's receive tile.
        // The buffers were last used for chunk g-2, by another group.  Once that group has read
        // its receive tile, the exchange barriers of this buffer are in the phase this chunk
        // expects.
        if (g >= 2 && !bad) {
          const unsigned target = 4u * unsigned(g >> 1);
          const long long start = clock64();
          while (read_count[buf] < target) {
            if (clock64() - start > wait_budget()) {
              report_timeout(0x607);
              bad = true;
              break;
            }
          }
        }
        if (!bad) bad = !mbar_wait_cluster(x_empty(buf), phase ^ 1u, 0x604);
        if (!bad) {
          // largest magnitude of the row: four chains of three-input maxima
          float top4[4] = {fabsf(t[0]), fabsf(t[1]), fabsf(t[2]), fabsf(t[3])};
#pragma unroll
          for (int i = 4; i + 8 <= kKv; i += 8) {
#pragma unroll
            for (int e = 0; e < 4; ++e) top4[e] = fmaxf(fmaxf(top4[e], fabsf(t[i + e])), fabsf(t[i + 4 + e]));
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) top4[e] = fmaxf(top4[e], fabsf(t[kKv - 4 + e]));
          const float top = fmaxf(fmaxf(top4[0], top4[1]), fmaxf(top4[2], top4[3]));
          if (top * p.scale_log2 <= 8.0f) {
#pragma unroll
            for (int q8 = 0; q8 < 8; ++q8) {
              uint32_t h[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const __half2 v = __floats2half2_rn(t[q8 * 8 + 2 * e], t[q8 * 8 + 2 * e + 1]);
                h[e] = *reinterpret_cast<const uint32_t*>(&v);
              }
              staged[q8 * 128 + row] = make_uint4(h[0], h[1], h[2], h[3]);
            }
            reinterpret_cast<float*>(staged + kXchgTileBytes / 16)[row] = 0.0f;
          } else {
            // round(t * 32767 / top) lands in the low 16 bits of t * encode + 1.5 * 2^23
            const float encode = 32767.0f / top;
#pragma unroll
            for (int q8 = 0; q8 < 8; ++q8) {
              uint32_t h[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const uint32_t lo = __float_as_uint(fmaf(t[q8 * 8 + 2 * e], encode, 12582912.0f));
                const uint32_t hi = __float_as_uint(fmaf(t[q8 * 8 + 2 * e + 1], encode, 12582912.0f));
                h[e] = __byte_perm(lo, hi, 0x5410);
              }
              staged[q8 * 128 + row] = make_uint4(h[0], h[1], h[2], h[3]);
            }
            reinterpret_cast<float*>(staged + kXchgTileBytes / 16)[row] = top * (1.0f / 32767.0f);
          }
        }
        fence_async_smem();
        uint32_t all_good;
        asm volatile(
            "{\n"
            ".reg .pred p, q;\n"
            "setp.eq.u32 p, %1, 0;\n"
            "bar.red.and.pred q, %2, 128, p;\n"   // barrier over the group's threads + vote
            "selp.u32 %0, 1, 0, q;\n"
            "}\n"
            : "=r"(all_good)
            : "r"(bad ? 1u : 0u), "r"(1 + group)
            : "memory");
        if (!all_good) {
          bad = true;
          break;
        }
        if ((warp & 3) == 2 && lane == 0) {
          mbar_arrive_expect_tx(x_full(buf), kXchgBytes);
          asm volatile(
              "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
              ::"r"(map_to_peer(xchg_smem + buf * kXchgBytes, peer)), "r"(send_smem + buf * kXchgBytes),
                "r"(kXchgBytes), "r"(map_to_peer(x_full(buf), peer))
              : "memory");
        }
        // ---- the peer's half of the scores
        if (!bad) bad = !mbar_wait_cluster(x_full(buf), phase, 0x605);
        const float unit = reinterpret_cast<const float*>(received + kXchgTileBytes / 16)[row];
        if (unit == 0.0f) {
#pragma unroll
          for (int q8 = 0; q8 < 8; ++q8) {
            const uint4 other = received[q8 * 128 + row];
            const uint32_t theirs[4] = {other.x, other.y, other.z, other.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 c2 = __half22float2(*reinterpret_cast<const __half2*>(&theirs[e]));
              t[q8 * 8 + 2 * e] += c2.x;
              t[q8 * 8 + 2 * e + 1] += c2.y;
            }
          }
        } else {
#pragma unroll
          for (int q8 = 0; q8 < 8; ++q8) {
            const uint4 other = received[q8 * 128 + row];
            const uint32_t theirs[4] = {other.x, other.y, other.z, other.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const short lo = static_cast<short>(theirs[e] & 0xFFFFu), hi = static_cast<short>(theirs[e] >> 16);
              t[q8 * 8 + 2 * e] = fmaf(static_cast<float>(lo), unit, t[q8 * 8 + 2 * e]);
              t[q8 * 8 + 2 * e + 1] = fmaf(static_cast<float>(hi), unit, t[q8 * 8 + 2 * e + 1]);
            }
          }
        }
        // This warp has read (and used) its part of the receive tile: tell the peer, whose next
        // copy into this buffer waits for the four warps, and count it for the local group that
        // uses the buffer next.
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_peer_relaxed(map_to_peer(x_empty(buf), peer));
          atomicAdd(const_cast<unsigned*>(read_count) + buf, 1u);
        }
        const int valid = p.seq - (seg.first_chunk + j) * kKv;   // positions of this chunk inside seq
        if (valid < kKv) {
#pragma unroll
          for (int i = 0; i < kKv; ++i)
            if (i >= valid) t[i] = -INFINITY;
        }
        float mx4[4] = {t[0], t[1], t[2], t[3]};
#pragma unroll
        for (int i = 4; i + 8 <= kKv; i += 8) {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            asm("max.f32 %0, %0, %1, %2;" : "+f"(mx4[e]) : "f"(t[i + e]), "f"(t[i + 4 + e]));
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) mx4[e] = fmaxf(mx4[e], t[kKv - 4 + e]);
        // position 0 of a chunk is always inside seq, so the maximum is finite
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
        // ---- reference maximum: take it over from the group that had chunk j-1, pass it on
        float m_prev = -INFINITY;
        if (j > 0) {
          if (!bad) bad = !mbar_wait(m_ready(g - 1, quad), group_phase(g - 1), 0x606);
          m_prev = m_shared[row];
        }
        const bool grow = mx > m_prev + kRescaleThreshold;   // always true for a segment's first chunk
        const float m_new = grow ? mx : m_prev;
        m_shared[row] = m_new;
        __syncwarp();
        if (lane == 0) mbar_arrive(m_ready(g, quad));
        if (m_new != m_l) {
          l *= fast_exp2(m_l - m_new);   // the first time: 0 * 2^-inf
          m_l = m_new;
        }
        // ---- probabilities
        uint32_t pw[32];
        float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float p0 = fast_exp2(fmaf(t[2 * i], p.scale_log2, -m_new));
          const float p1 = fast_exp2(fmaf(t[2 * i + 1], p.scale_log2, -m_new));
          sum4[i & 3] += p0 + p1;
          pw[i] = pack_bf16x2(p0, p1);
        }
        if (valid < kKv) {
          // positions outside seq: exact zeros whatever the scale (0 * -inf would be a NaN)
          float tail = 0.0f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const bool in0 = 2 * i < valid, in1 = 2 * i + 1 < valid;
            const float p0 = in0 ? fast_exp2(fmaf(t[2 * i], p.scale_log2, -m_new)) : 0.0f;
            const float p1 = in1 ? fast_exp2(fmaf(t[2 * i + 1], p.scale_log2, -m_new)) : 0.0f;
            tail += p0 + p1;
            pw[i] = pack_bf16x2(p0, p1);
          }
          sum4[0] = tail; sum4[1] = 0.0f; sum4[2] = 0.0f; sum4[3] = 0.0f;
        }
        l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        // Neither the probability buffer nor the accumulator may be touched before the value MMAs
        // of chunk j-1 have finished with them.  (For a segment's first chunk the previous
        // segment's epilogue has waited for them.)
        if (j > 0 && !bad) bad = !mbar_wait(pv_done(g - 1), group_phase(g - 1), 0x602);
        tc_fence_after();
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          const float f = grow ? fast_exp2(m_prev - m_new) : 1.0f;
#pragma unroll 1
          for (int c = 0; c < 256; c += 32) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(lane_base + kColO + c, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
            tmem_st_32x32b_x32(lane_base + kColO + c, o);
          }
          tmem_st_wait();
        }
        tmem_st_32x32b_x32(lane_base + kColP, pw);
        tmem_st_wait();
        tc_fence_before();
        const bool warp_good = __all_sync(0xffffffffu, !bad);
        if (lane == 0 && warp_good) mbar_arrive(p_full);
      }

      // Every softmax thread comes here, also after a failure.  The final reference maximum of
      // a head was written by the group that had the segment's last chunk.
      const int g_last = gbase + num_chunks - 1;
      asm volatile("bar.sync 4, %0;" ::"n"(kSoftmaxThreads) : "memory");
      bool ready = !bad;
      const float m_final = m_shared[row];
      if (m_l != m_final) l *= fast_exp2(m_l - m_final);   // a group without chunks holds l = 0
      l_part[group * 128 + row] = l;
      if (ready) ready = mbar_wait(pv_done(g_last), group_phase(g_last), 0x603);
      asm volatile("bar.sync 4, %0;" ::"n"(kSoftmaxThreads) : "memory");
      l = 0.0f;
#pragma unroll
      for (int gi = 0; gi < kGroups; ++gi) l += l_part[gi * 128 + row];
      const bool all_ready = __all_sync(0xffffffffu, ready);
      if (all_ready) {
        tc_fence_after();
        const float inv_l = 1.0f / l;
        // the eight 32-column blocks of the accumulator are dealt out to the groups
        if (seg.whole) {
          __nv_bfloat16* orow =
              p.out + (static_cast<long long>(seg.b) * p.heads + row) * kDv + half * 256;
#pragma unroll 1
          for (int c = group * 32; c < 256; c += kGroups * 32) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(lane_base + kColO + c, o);
            tmem_ld_wait();
            if (live) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 w;
                w.x = pack_bf16x2(__uint_as_float(o[v * 8 + 0]) * inv_l, __uint_as_float(o[v * 8 + 1]) * inv_l);
                w.y = pack_bf16x2(__uint_as_float(o[v * 8 + 2]) * inv_l, __uint_as_float(o[v * 8 + 3]) * inv_l);
                w.z = pack_bf16x2(__uint_as_float(o[v * 8 + 4]) * inv_l, __uint_as_float(o[v * 8 + 5]) * inv_l);
                w.w = pack_bf16x2(__uint_as_float(o[v * 8 + 6]) * inv_l, __uint_as_float(o[v * 8 + 7]) * inv_l);
                *reinterpret_cast<uint4*>(orow + c + v * 8) = w;
              }
            }
          }
        } else {
          const long long slot = seg.slot * p.heads + row;
          float* prow = p.partial_o + slot * kDv + half * 256;
#pragma unroll 1
          for (int c = group * 32; c < 256; c += kGroups * 32) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(lane_base + kColO + c, o);
            tmem_ld_wait();
            if (live) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 w = make_float4(__uint_as_float(o[v * 4 + 0]) * inv_l, __uint_as_float(o[v * 4 + 1]) * inv_l,
                                       __uint_as_float(o[v * 4 + 2]) * inv_l, __uint_as_float(o[v * 4 + 3]) * inv_l);
                *reinterpret_cast<float4*>(prow + c + v * 4) = w;
              }
            }
          }
          // each feature half was normalised with its own sums, so each records its own log-sum-exp
          if (live && group == 0) p.partial_lse[slot * 2 + half] = m_final + log2f(l);
        }
      }
      // the accumulator has been read: the next segment's values may overwrite it
      tc_fence_before();
      __syncwarp();
      if (lane == 0 && all_ready) mbar_arrive(o_free);
      gbase += num_chunks;
      if (!all_ready) break;   // after a failure the remaining segments are not attempted
    }
  }

  // Common exit.  Neither CTA of the pair may leave while the other can still write into its
  // shared memory or arrive on its barriers, hence the cluster-wide barrier.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 2) {
    if (g_device_status != 0)
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// out[b,h,c] = sum_s w_s * partial[b,s,h,c],  w_s = 2^(lse_s - max) / sum_s 2^(lse_s - max), with
// the log-sum-exp of the feature half that column c belongs to.  Under the balanced schedule a
// sequence has as many pieces as clusters touch it; a sequence with one piece was written
// directly and is skipped.
__global__ void __launch_bounds__(128)
mla_combine_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_lse,
                   __nv_bfloat16* __restrict__ out, int rows, int heads, int pieces, int balanced,
                   int chunks_per_seq, int clusters, long long units) {
  // one warp per (sequence, head): lane l owns columns [4 l, 4 l + 4) of each 128-column quarter
  grid_dependents_may_launch();
  grid_dependency_wait();   // the partial results come from the decode kernel launched just before
  const int bh = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (bh >= rows) return;
  const int b = bh / heads, h = bh % heads;
  int n = pieces;
  if (balanced) {
    const long long u = static_cast<long long>(b) * chunks_per_seq;
    n = cluster_of_unit(units, clusters, u + chunks_per_seq - 1) - cluster_of_unit(units, clusters, u) + 1;
    if (n == 1) return;
  }
  const long long slot0 = static_cast<long long>(b) * pieces * heads + h;   // piece s: slot0 + s * heads
  float mx[2] = {-INFINITY, -INFINITY}, inv[2];
  for (int s = lane; s < n; s += 32) {
    const float2 v = *reinterpret_cast<const float2*>(partial_lse + (slot0 + static_cast<long long>(s) * heads) * 2);
    mx[0] = fmaxf(mx[0], v.x);
    mx[1] = fmaxf(mx[1], v.y);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], o));
    mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], o));
  }
  float denom[2] = {0.0f, 0.0f};
  for (int s = lane; s < n; s += 32) {
    const float2 v = *reinterpret_cast<const float2*>(partial_lse + (slot0 + static_cast<long long>(s) * heads) * 2);
    denom[0] += exp2f(v.x - mx[0]);
    denom[1] += exp2f(v.y - mx[1]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    denom[0] += __shfl_xor_sync(0xffffffffu, denom[0], o);
    denom[1] += __shfl_xor_sync(0xffffffffu, denom[1], o);
  }
  inv[0] = 1.0f / denom[0];
  inv[1] = 1.0f / denom[1];
  float4 acc[4] = {};
  for (int s = 0; s < n; ++s) {
    const long long slot = slot0 + static_cast<long long>(s) * heads;
    const float2 lse = *reinterpret_cast<const float2*>(partial_lse + slot * 2);
    const float w[2] = {exp2f(lse.x - mx[0]) * inv[0], exp2f(lse.y - mx[1]) * inv[1]};
    const float4* src = reinterpret_cast<const float4*>(partial_o + slot * kDv) + lane;
#pragma unroll
    for (int qt = 0; qt < 4; ++qt) {
      const float4 v = src[qt * 32];
      const float wq = w[qt >> 1];   // quarters 0,1 belong to feature half 0
      acc[qt].x += wq * v.x; acc[qt].y += wq * v.y; acc[qt].z += wq * v.z; acc[qt].w += wq * v.w;
    }
  }
  uint2* dst = reinterpret_cast<uint2*>(out + static_cast<long long>(bh) * kDv) + lane;
#pragma unroll
  for (int qt = 0; qt < 4; ++qt)
    dst[qt * 32] = make_uint2(pack_bf16x2(acc[qt].x, acc[qt].y), pack_bf16x2(acc[qt].z, acc[qt].w));
}

size_t scratch_bytes(int batch, int heads, int d_v, int pieces) {
  if (pieces <= 1) return 0;
  const size_t slots = size_t(batch) * pieces * heads;
  return ((slots * d_v * 4 + 255) / 256) * 256 + ((slots * 2 * 4 + 255) / 256) * 256;
}

// The automatic schedule picks, by a small cost model, between equal splits of every sequence
// (one segment per cluster) and the balanced schedule (equal runs of chunks, a cluster may work
// through pieces of several sequences).  The model's constants are measured figures of this
// kernel on a B200, in microseconds: a chunk takes a cluster about 1.25, a launch has about 22
// of fixed cost (start-up, pipeline fill and drain, epilogue), every further segment of a
// cluster costs about 13 (drain, epilogue, new query, refill), and cutting sequences costs a
// merge pass plus the FP32 partials' traffic.
constexpr int kMinChunksPerCluster = 8;
struct Schedule {
  int balanced, clusters, pieces, chunks_per_seq;
  long long units;
};
Schedule automatic_schedule(int batch, int seq, bool force_balanced) {
  int sms = 148;
  int device = 0;
  if (cudaGetDevice(&device) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int pairs = sms / 2 > 0 ? sms / 2 : 1;
  constexpr double kChunkUs = 1.25, kFixedUs = 22.0, kSegmentUs = 13.0, kMergeUs = 5.0;
  constexpr double kPartialUsPerSlot = 2.0 * 128 * 512 * 4 / 3.0e6;   // written and read back at ~3 TB/s
  Schedule best;
  best.chunks_per_seq = (seq + kKv - 1) / kKv;
  best.units = static_cast<long long>(batch) * best.chunks_per_seq;
  best.balanced = 0;
  best.clusters = 0;
  best.pieces = 1;
  const int cps = best.chunks_per_seq;
  double best_cost = 0.0;
  // equal splits
  const int max_splits = cps / kMinChunksPerCluster > 1 ? cps / kMinChunksPerCluster : 1;
  for (int s = 1; s <= max_splits && s <= 2 * pairs; ++s) {
    const long long waves = (static_cast<long long>(batch) * s + pairs - 1) / pairs;
    double cost = waves * ((cps + s - 1) / s * kChunkUs + kFixedUs);
    if (s > 1) cost += kMergeUs + kPartialUsPerSlot * batch * s;
    if (s == 1 || cost < best_cost) {
      best_cost = cost;
      best.pieces = s;
    }
  }
  // balanced runs
  long long clusters = best.units / kMinChunksPerCluster;
  if (clusters > pairs) clusters = pairs;
  if (clusters >= 1) {
    Schedule s = best;
    s.balanced = 1;
    s.clusters = int(clusters);
    s.pieces = 1;
    long long slots = 0;
    for (int b = 0; b < batch; ++b) {
      const long long u = static_cast<long long>(b) * cps;
      const int n = cluster_of_unit(s.units, s.clusters, u + cps - 1) - cluster_of_unit(s.units, s.clusters, u) + 1;
      if (n > s.pieces) s.pieces = n;
      if (n > 1) slots += n;
    }
    int max_segments = 1;
    long long longest = 0;
    for (int k = 0; k < s.clusters; ++k) {
      const long long u0 = unit_begin(s.units, s.clusters, k), u1 = unit_begin(s.units, s.clusters, k + 1);
      const int segments = int((u1 - 1) / cps - u0 / cps) + 1;
      if (segments > max_segments) max_segments = segments;
      if (u1 - u0 > longest) longest = u1 - u0;
    }
    double cost = longest * kChunkUs + kFixedUs + (max_segments - 1) * kSegmentUs;
    if (slots > 0) cost += kMergeUs + kPartialUsPerSlot * slots;
    if (cost < best_cost || force_balanced) return s;
  }
  return best;
}

// kv_splits > 0: that many equal splits of every sequence, one cluster each.
// kv_splits == 0: the automatic schedule; < 0: the balanced schedule whatever the cost model says.
Schedule choose_schedule(int batch, int seq, int kv_splits) {
  if (kv_splits <= 0) return automatic_schedule(batch, seq, kv_splits < 0);
  Schedule s;
  const int chunks = (seq + kKv - 1) / kKv;
  s.balanced = 0;
  s.chunks_per_seq = chunks;
  s.units = static_cast<long long>(batch) * chunks;
  s.pieces = kv_splits > chunks ? chunks : kv_splits;
  s.clusters = 0;
  return s;
}

int opt_in_mla() {
  static unsigned long long configured = 0;
  return opt_in_shared_memory(reinterpret_cast<const void*>(&mla_decode_kernel), kMlaSmem, &configured, "mla");
}

}  // namespace
}  // namespace trinity_sm100

using namespace trinity_sm100;

// What trinity_sm100_mla_decode_bf16 will do for (batch, seq, kv_splits), without a launch:
// info = {balanced, clusters (grid y), pieces (partial slots per sequence), chunks per sequence}.
extern "C" int trinity_sm100_mla_schedule(int32_t batch, int32_t seq, int32_t kv_splits, int32_t* info) {
  if (batch <= 0 || seq <= 0 || !info) return fail(TRINITY_SM100_E_INVALID, "mla_schedule: bad argument");
  const Schedule s = choose_schedule(batch, seq, kv_splits);
  info[0] = s.balanced;
  info[1] = s.balanced ? s.clusters : s.pieces;
  info[2] = s.pieces;
  info[3] = s.chunks_per_seq;
  return 0;
}

// The index-th piece of work of cluster (y, z) of that launch's grid (z is always 0 under the
// balanced schedule): segment = {sequence, first chunk, chunk count, partial slot, whole}.
// Returns 1 if the cluster has such a piece, 0 if not, a negative code on bad arguments.
extern "C" int trinity_sm100_mla_schedule_segment(int32_t batch, int32_t seq, int32_t kv_splits, int32_t y,
                                                  int32_t z, int32_t index, int64_t* segment) {
  if (batch <= 0 || seq <= 0 || !segment || y < 0 || z < 0 || index < 0)
    return fail(TRINITY_SM100_E_INVALID, "mla_schedule_segment: bad argument");
  const Schedule s = choose_schedule(batch, seq, kv_splits);
  if (y >= (s.balanced ? s.clusters : s.pieces) || z >= (s.balanced ? 1 : batch)) return 0;
  MlaParams p = {};
  p.chunks_per_seq = s.chunks_per_seq;
  p.pieces = s.pieces;
  p.balanced = s.balanced;
  p.clusters = s.clusters;
  p.units = s.units;
  Segment piece;
  if (!segment_of(p, y, z, index, piece)) return 0;
  segment[0] = piece.b;
  segment[1] = piece.first_chunk;
  segment[2] = piece.num_chunks;
  segment[3] = piece.slot;
  segment[4] = piece.whole ? 1 : 0;
  return 1;
}

extern "C" size_t trinity_sm100_mla_scratch_bytes(int32_t batch, int32_t heads, int32_t d_v,
                                                  int32_t kv_splits) {
  if (batch <= 0 || heads <= 0 || d_v <= 0) return 0;
  return scratch_bytes(batch, heads, d_v, kv_splits);
}

extern "C" int trinity_sm100_mla_default_splits(int32_t batch, int32_t seq) {
  if (batch <= 0 || seq <= 0) return 1;
  return automatic_schedule(batch, seq, false).pieces;
}

extern "C" int trinity_sm100_mla_balanced_slots(int32_t batch, int32_t seq) {
  if (batch <= 0 || seq <= 0) return 1;
  return automatic_schedule(batch, seq, true).pieces;
}

extern "C" int trinity_sm100_mla_decode_bf16(const trinity_sm100_mla* args, void* stream_handle) {
  if (!args) return fail(TRINITY_SM100_E_INVALID, "mla: null argument block");
  const trinity_sm100_mla& a = *args;
  if (!a.q || !a.cache || !a.out) return fail(TRINITY_SM100_E_INVALID, "mla: null operand");
  if (a.batch <= 0 || a.heads <= 0 || a.seq <= 0)
    return fail(TRINITY_SM100_E_INVALID, "mla: empty extent");
  if (a.d_qk != kDqk || a.d_v != kDv)
    return fail(TRINITY_SM100_E_UNSUPPORTED, "mla: only d_qk=576, d_v=512 is built (got %d, %d)",
                a.d_qk, a.d_v);
  if (a.heads > 128)
    return fail(TRINITY_SM100_E_UNSUPPORTED, "mla: at most 128 heads per call (got %d)", a.heads);
  if (a.batch > 65535) return fail(TRINITY_SM100_E_UNSUPPORTED, "mla: batch above 65535");
  if (!aligned16(a.q) || !aligned16(a.cache) || !aligned16(a.out))
    return fail(TRINITY_SM100_E_INVALID, "mla: pointers must be 16-byte aligned");
  const Schedule schedule = choose_schedule(a.batch, a.seq, a.kv_splits);
  if (schedule.pieces > 65535) return fail(TRINITY_SM100_E_UNSUPPORTED, "mla: too many splits");
  const bool balanced = schedule.balanced != 0;
  const int splits = schedule.pieces;
  const size_t need = scratch_bytes(a.batch, a.heads, a.d_v, splits);
  if (need > 0) {
    if (!a.scratch || a.scratch_bytes < need)
      return fail(TRINITY_SM100_E_INVALID, "mla: %d partial slots per sequence need %zu scratch bytes (got %zu)",
                  splits, need, a.scratch_bytes);
    if (reinterpret_cast<uintptr_t>(a.scratch) & 255u)
      return fail(TRINITY_SM100_E_INVALID, "mla: scratch must be 256-byte aligned");
  }
  if (int rc = require_sm100(nullptr)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (int rc = opt_in_mla()) return rc;
  // Two views of the cache: 64-feature boxes (128-byte swizzle) for the latent part and
  // 32-feature boxes (64-byte swizzle) for each CTA's half of the rope part.
  CUtensorMap map_cache, map_rope;
  int rc;
  if ((rc = make_tensor_map_3d(&map_cache, a.cache, 2, kDqk, a.seq, a.batch, kDqk * 2ull,
                               uint64_t(a.seq) * kDqk * 2, 64, kKv, 1, 128)))
    return rc;
  if ((rc = make_tensor_map_3d(&map_rope, a.cache, 2, kDqk, a.seq, a.batch, kDqk * 2ull,
                               uint64_t(a.seq) * kDqk * 2, 32, kKv, 1, 64)))
    return rc;
  CUtensorMap map_query;
  if ((rc = make_tensor_map_3d(&map_query, a.q, 2, kDqk, a.heads, a.batch, kDqk * 2ull,
                               uint64_t(a.heads) * kDqk * 2, 32, 128, 1, 64)))
    return rc;
  MlaParams p;
  p.q = static_cast<const __nv_bfloat16*>(a.q);
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.partial_o = nullptr;
  p.partial_lse = nullptr;
  if (splits > 1) {
    const size_t slots = size_t(a.batch) * splits * a.heads;
    p.partial_o = static_cast<float*>(a.scratch);
    p.partial_lse = reinterpret_cast<float*>(static_cast<uint8_t*>(a.scratch) +
                                             ((slots * kDv * 4 + 255) / 256) * 256);
  }
  p.batch = a.batch;
  p.heads = a.heads;
  p.seq = a.seq;
  p.chunks_per_seq = schedule.chunks_per_seq;
  p.pieces = schedule.pieces;
  p.balanced = balanced ? 1 : 0;
  p.clusters = schedule.clusters;
  p.units = schedule.units;
  p.scale_log2 = fabsf(a.scale) * 1.4426950408889634f;
  p.negate = a.scale < 0.0f ? 1 : 0;
  // clusters of two: the two feature halves of one (batch, split)
  KernelLaunch launch(balanced ? dim3(2, schedule.clusters, 1) : dim3(2, splits, a.batch), dim3(kMlaThreads),
                      kMlaSmem, stream, 2);
  cudaError_t launch_error =
      cudaLaunchKernelEx(&launch.config, mla_decode_kernel, map_cache, map_rope, map_query, p);
  if (launch_error != cudaSuccess)
    return fail(TRINITY_SM100_E_CUDA, "mla_decode launch: %s", cudaGetErrorString(launch_error));
  count_launch();
  if ((rc = check_launch("mla_decode"))) return rc;
  if (splits > 1) {
    const int rows = a.batch * a.heads;
    KernelLaunch merge(dim3((rows + 3) / 4), dim3(128), 0, stream);
    launch_error = cudaLaunchKernelEx(&merge.config, mla_combine_kernel, static_cast<const float*>(p.partial_o),
                                      static_cast<const float*>(p.partial_lse), p.out, rows, int(a.heads), int(splits),
                                      int(p.balanced), int(p.chunks_per_seq), int(p.clusters),
                                      static_cast<long long>(p.units));
    if (launch_error != cudaSuccess)
      return fail(TRINITY_SM100_E_CUDA, "mla_combine launch: %s", cudaGetErrorString(launch_error));
    count_launch();
    if ((rc = check_launch("mla_combine"))) return rc;
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant.
//
// Some callers have nowhere to get scratch memory from.  The launch function of a streamed
// artifact (trinity_launch in a program.so) is such a caller: it receives nothing but the
// plan's buffer bindings, the artifact format gives streamed programs no workspace, and the
// function may run while its stream is being captured into a CUDA Graph, where asking the
// driver or a framework allocator for memory is not an option.  For them the split partials
// live in the fixed device array below instead of caller-provided scratch.
//
// The array is part of the library image: every GPU that loads the library carries these
// TRINITY_SM100_MLA_STATIC_SCRATCH_BYTES until the process exits.  All calls on a device share
// it, so two calls that overlap on the GPU (different streams, or graph branches) race on the
// partials.  Nothing in it has to start at zero: every slot the merge step reads is written by
// the split kernel of the same call first, so stale contents of an earlier call are never seen.
static __device__ __align__(256) unsigned char g_mla_static_scratch[TRINITY_SM100_MLA_STATIC_SCRATCH_BYTES];

namespace {
// Device address of the array for the current device.  In host code the array's name is only
// a stand-in, so the address is looked up once per device with that device current.
int static_scratch_address(void** address) {
  static std::mutex mutex;
  static void* cached[64] = {};
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess)
    return fail(TRINITY_SM100_E_CUDA, "mla (no-alloc): cudaGetDevice: %s", cudaGetErrorString(e));
  if (device < 0 || device >= 64)
    return fail(TRINITY_SM100_E_DEVICE, "mla (no-alloc): device index %d", device);
  std::lock_guard<std::mutex> lock(mutex);
  if (!cached[device]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_mla_static_scratch);
    if (e != cudaSuccess || !p)
      return fail(TRINITY_SM100_E_CUDA, "mla (no-alloc): cudaGetSymbolAddress: %s",
                  cudaGetErrorString(e));
    cached[device] = p;
  }
  *address = cached[device];
  return 0;
}
}  // namespace

int trinity_sm100::mla_prepare_device() {
  if (int rc = opt_in_mla()) return rc;
  void* scratch = nullptr;
  return static_scratch_address(&scratch);
}

extern "C" int trinity_sm100_mla_decode_bf16_noalloc(const trinity_sm100_mla* args,
                                                     void* stream_handle) {
  if (!args) return fail(TRINITY_SM100_E_INVALID, "mla (no-alloc): null argument block");
  trinity_sm100_mla call = *args;
  if (call.batch <= 0 || call.heads <= 0 || call.seq <= 0)
    return fail(TRINITY_SM100_E_INVALID, "mla (no-alloc): empty extent");
  int splits = call.kv_splits > 0   ? call.kv_splits
               : call.kv_splits == 0 ? trinity_sm100_mla_default_splits(call.batch, call.seq)
                                     : trinity_sm100_mla_balanced_slots(call.batch, call.seq);
  const int chunks = (call.seq + kKv - 1) / kKv;
  if (splits > chunks) splits = chunks;
  size_t need = scratch_bytes(call.batch, call.heads, call.d_v, splits);
  if (call.kv_splits == 0 && need > size_t(TRINITY_SM100_MLA_STATIC_SCRATCH_BYTES)) {
    // The schedule was left to the library and its first choice does not fit: take the most
    // equal splits that do.  A caller that fixed the schedule (kv_splits != 0) is refused below.
    while (splits > 1 && scratch_bytes(call.batch, call.heads, call.d_v, splits) >
                             size_t(TRINITY_SM100_MLA_STATIC_SCRATCH_BYTES))
      --splits;
    call.kv_splits = splits;
    need = scratch_bytes(call.batch, call.heads, call.d_v, splits);
  }
  if (need > size_t(TRINITY_SM100_MLA_STATIC_SCRATCH_BYTES))
    return fail(TRINITY_SM100_E_UNSUPPORTED,
                "mla (no-alloc): batch %d x %d splits x %d heads needs %zu scratch bytes, above the "
                "built-in %zu; use fewer splits or trinity_sm100_mla_decode_bf16 with your own "
                "scratch",
                call.batch, splits, call.heads, need, size_t(TRINITY_SM100_MLA_STATIC_SCRATCH_BYTES));
  void* scratch = nullptr;
  if (int rc = static_scratch_address(&scratch)) return rc;
  call.scratch = scratch;
  call.scratch_bytes = TRINITY_SM100_MLA_STATIC_SCRATCH_BYTES;
  return trinity_sm100_mla_decode_bf16(&call, stream_handle);
}
