// Two-shot sum all-reduce of a BF16 matrix through NVLink peer-mapped memory.
//
// Every rank runs the same persistent grid.  Rank r owns slice r of the flattened matrix:
//   1. announce: the local partial is complete (stream order) -> write `ready` on every peer
//   2. reduce:   wait for every peer's `ready`, pull slice r from all ranks with 128-bit peer
//                loads in rank order, add in FP32, round once, store into the local buffer
//   3. publish:  last CTA to finish writes `reduced` on every peer
//   4. gather:   for each peer q, wait for q's `reduced`, copy slice q from q's buffer
//   5. retire:   last CTA writes `done` on every peer and waits for every peer's `done`, so no
//                rank can start overwriting its buffer while another still reads it
// Flags carry the call's epoch (never 0: a zeroed pad reads as epoch 0) and are never reset.
// Every wait is bounded; on expiry the device status word is set, the CTA stops moving data
// and the call publishes nothing further.  The pad's first 64 words belong to this kernel; the
// fused GEMM epilogue keeps its flags behind them, so one pad serves both.
//
// NVLink traffic per rank: (world-1)/world * bytes pulled in the reduce step and the same again
// in the gather step.
#include "host_common.h"
#include "sm100_ptx.cuh"

namespace trinity_sm100 {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kFlagWords = 64;  // ready[8] reduced[8] done[8] counters[2] failed + padding
constexpr int kOffReady = 0, kOffReduced = 8, kOffDone = 16, kOffCounter = 24, kOffFailed = 26;
constexpr int kArThreads = 512;
static_assert(kGemmFlagOffset == kFlagWords, "the fused GEMM epilogue's flags start behind this kernel's");

struct AllReduceParams {
  uint4* buffers[kMaxWorld];
  uint32_t* flags[kMaxWorld];
  long long vectors;  // 16-byte vectors in the whole matrix
  int world, rank;
  uint32_t epoch;
};

__device__ __forceinline__ void slice_range(long long vectors, int world, int r, long long& lo,
                                            long long& hi) {
  const long long base = vectors / world, extra = vectors % world;
  lo = r * base + (r < extra ? r : extra);
  hi = lo + base + (r < extra ? 1 : 0);
}

__global__ void __launch_bounds__(kArThreads)
allreduce_two_shot_kernel(const AllReduceParams p) {
  __shared__ int s_ok;
  __shared__ int s_last;
  uint32_t* my_flags = p.flags[p.rank];
  const int tid = threadIdx.x;
  // A CTA whose wait gave up moves no more data but still takes part in both counters, so the
  // counters are back at zero for the next call on this pad; it marks the call as failed
  // (kOffFailed = epoch) and the last CTA then publishes nothing, so the peers' waits run out as
  // well and every rank's status word reports the failure.

  // 1. announce
  if (blockIdx.x == 0 && tid < p.world) {
    __threadfence_system();
    flag_store(p.flags[tid] + kOffReady + p.rank, p.epoch);
  }
  // 2. reduce own slice
  if (tid == 0) s_ok = 1;
  __syncthreads();
  if (tid < p.world) {
    if (!wait_flag(my_flags + kOffReady + tid, p.epoch, 0x701)) s_ok = 0;
  }
  __syncthreads();
  bool ok = s_ok != 0;
  long long lo, hi;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  if (ok) {
    slice_range(p.vectors, p.world, p.rank, lo, hi);
    for (long long i = lo + static_cast<long long>(blockIdx.x) * blockDim.x + tid; i < hi;
         i += stride) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      uint4 v[kMaxWorld];
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r)
        if (r < p.world) v[r] = peer_load(p.buffers[r] + i);
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r) {
        if (r < p.world) {
          const uint32_t w[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[2 * e] += bf16_lo(w[e]);
            acc[2 * e + 1] += bf16_hi(w[e]);
          }
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      p.buffers[p.rank][i] = o;
    }
  }
  // 3. publish once every CTA of this rank has stored its part of the slice
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    if (!ok) atomicExch(my_flags + kOffFailed, p.epoch);
    __threadfence();
    const unsigned prev = atomicAdd(my_flags + kOffCounter, 1u);
    s_last = (prev == gridDim.x - 1);
    if (s_last) {
      my_flags[kOffCounter] = 0;
      __threadfence();
      if (*reinterpret_cast<volatile uint32_t*>(my_flags + kOffFailed) == p.epoch) s_last = 0;
    }
  }
  __syncthreads();
  if (s_last && tid < p.world) {
    __threadfence_system();
    flag_store(p.flags[tid] + kOffReduced + p.rank, p.epoch);
  }
  // 4. gather the other slices
  for (int step = 1; step < p.world && ok; ++step) {
    const int q = (p.rank + step) % p.world;
    __syncthreads();
    if (tid == 0 && !wait_flag(my_flags + kOffReduced + q, p.epoch, 0x702)) s_ok = 0;
    __syncthreads();
    ok = s_ok != 0;
    if (!ok) break;
    slice_range(p.vectors, p.world, q, lo, hi);
    for (long long i = lo + static_cast<long long>(blockIdx.x) * blockDim.x + tid; i < hi;
         i += stride)
      p.buffers[p.rank][i] = peer_load(p.buffers[q] + i);
  }
  // 5. retire
  __syncthreads();
  if (tid == 0) {
    if (!ok) atomicExch(my_flags + kOffFailed, p.epoch);
    __threadfence();
    const unsigned prev = atomicAdd(my_flags + kOffCounter + 1, 1u);
    s_last = (prev == gridDim.x - 1);
    if (s_last) {
      my_flags[kOffCounter + 1] = 0;
      __threadfence();
      if (*reinterpret_cast<volatile uint32_t*>(my_flags + kOffFailed) == p.epoch) s_last = 0;
    }
  }
  __syncthreads();
  if (s_last && tid < p.world) {
    flag_store(p.flags[tid] + kOffDone + p.rank, p.epoch);
    wait_flag(my_flags + kOffDone + tid, p.epoch, 0x703);
  }
}

}  // namespace
}  // namespace trinity_sm100

using namespace trinity_sm100;

extern "C" size_t trinity_sm100_allreduce_flag_words(void) { return kFlagWords; }

extern "C" int trinity_sm100_allreduce_bf16(const trinity_sm100_allreduce* args,
                                            void* stream_handle) {
  if (!args) return fail(TRINITY_SM100_E_INVALID, "allreduce: null argument block");
  const trinity_sm100_allreduce& a = *args;
  if (!a.peers || !a.flags) return fail(TRINITY_SM100_E_INVALID, "allreduce: null pointer table");
  if (a.world < 1 || a.world > kMaxWorld || a.rank < 0 || a.rank >= a.world)
    return fail(TRINITY_SM100_E_INVALID, "allreduce: world %d / rank %d out of range", a.world,
                a.rank);
  if (a.epoch == 0)
    return fail(TRINITY_SM100_E_INVALID, "allreduce: epoch 0 is what a fresh flag pad holds; start at 1");
  if (a.rows <= 0 || a.cols <= 0 || a.cols % 8)
    return fail(TRINITY_SM100_E_INVALID, "allreduce: rows > 0, cols a positive multiple of 8");
  AllReduceParams p;
  for (int r = 0; r < kMaxWorld; ++r) {
    p.buffers[r] = nullptr;
    p.flags[r] = nullptr;
  }
  for (int r = 0; r < a.world; ++r) {
    if (!a.peers[r] || !a.flags[r] || !aligned16(a.peers[r]) || !aligned16(a.flags[r]))
      return fail(TRINITY_SM100_E_INVALID, "allreduce: peer %d pointer null or misaligned", r);
    p.buffers[r] = static_cast<uint4*>(a.peers[r]);
    p.flags[r] = static_cast<uint32_t*>(a.flags[r]);
  }
  p.vectors = a.rows * a.cols / 8;
  p.world = a.world;
  p.rank = a.rank;
  p.epoch = a.epoch;
  int sm_count = 0;
  if (int rc = require_sm100(&sm_count)) return rc;
  // One CTA per SM: every CTA of the grid is resident, which the flag waits rely on.
  const long long per_rank = (p.vectors + a.world - 1) / a.world;
  long long want = (per_rank + kArThreads - 1) / kArThreads;
  const int grid = int(want < 1 ? 1 : (want > sm_count ? sm_count : want));
  allreduce_two_shot_kernel<<<grid, kArThreads, 0, static_cast<cudaStream_t>(stream_handle)>>>(p);
  count_launch();
  return check_launch("allreduce_two_shot");
}
