// Rank-major all-gather of a BF16 shard through NVLink peer-mapped memory, for persistent
// artifacts.
//
// Everything the kernel needs to know about the other GPUs lives in device memory, in a peer
// table at the start of the artifact's workspace that the runtime fills once: the persistent
// launch block of the artifact ABI carries only the plan's buffer bindings and the workspace
// pointer, and a captured launch must not depend on host-side state that changes from call to
// call.  The call number ("epoch") is therefore kept in the table as well and advanced by the
// kernel itself, so a CUDA Graph replays the launch unchanged.
//
//   1. announce: my shard is complete (stream order) -> write ready[rank] = epoch into every
//      rank's table
//   2. gather:   for each rank q (starting behind my own), wait for ready[q], pull its shard
//      with 128-bit peer loads into my output at q's offset along the gather axis
//   3. retire:   the last CTA to finish advances the local epoch, writes done[rank] into every
//      rank's table and waits for every rank's done, so no rank overwrites its shard for the
//      next call while another still reads it
// Every wait is bounded; on expiry the device status word is set and the CTA moves no more data
// but still takes part in the CTA count, so the table is consistent for the next call.
#include "host_common.h"
#include "sm100_ptx.cuh"

namespace trinity_sm100 {
namespace {

constexpr int kAgThreads = 512;
constexpr int kAgReady = 0, kAgDone = 8;   // words of trinity_sm100_peer_table::flags

struct AllGatherParams {
  trinity_sm100_peer_table* table;
  uint4* out;            // [rows * (axis == 0 ? world : 1), cols * (axis == 1 ? world : 1)] BF16
  int source;            // which symmetric buffer of the table holds the shards
  long long rows;
  int row_vectors;       // 16-byte vectors per shard row
  int axis;
};

__global__ void __launch_bounds__(kAgThreads)
allgather_peer_kernel(const AllGatherParams p) {
  __shared__ int s_ok;
  __shared__ int s_last;
  trinity_sm100_peer_table* mine = p.table;
  const int world = mine->world, rank = mine->rank;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(&mine->epoch) + 1u;
  const int tid = threadIdx.x;
  if (tid == 0) s_ok = 1;
  // 1. announce
  if (blockIdx.x == 0 && tid < world) {
    __threadfence_system();
    flag_store(reinterpret_cast<trinity_sm100_peer_table*>(mine->workspace[tid])->flags + kAgReady + rank, epoch);
  }
  __syncthreads();
  // 2. gather, own shard included (it comes from local memory)
  const long long vectors = p.rows * p.row_vectors;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long out_pitch = p.axis == 1 ? static_cast<long long>(p.row_vectors) * world : p.row_vectors;
  bool ok = true;
  for (int step = 0; step < world && ok; ++step) {
    const int q = (rank + step) % world;
    if (tid == 0 && !wait_flag(mine->flags + kAgReady + q, epoch, 0x901)) s_ok = 0;
    __syncthreads();
    ok = s_ok != 0;
    if (!ok) break;
    const uint4* shard = reinterpret_cast<const uint4*>(mine->buffers[p.source][q]);
    uint4* base = p.out + (p.axis == 0 ? static_cast<long long>(q) * vectors : static_cast<long long>(q) * p.row_vectors);
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + tid; i < vectors; i += stride) {
      const long long r = i / p.row_vectors, c = i - r * p.row_vectors;
      base[r * out_pitch + c] = peer_load(shard + i);
    }
  }
  // 3. retire
  __syncthreads();
  if (tid == 0) {
    if (!ok) atomicExch(&mine->failed, epoch);
    __threadfence();
    const unsigned prev = atomicAdd(&mine->counter, 1u);
    s_last = (prev == gridDim.x - 1);
    if (s_last) {
      mine->counter = 0;
      *reinterpret_cast<volatile uint32_t*>(&mine->epoch) = epoch;
      __threadfence();
      if (*reinterpret_cast<volatile uint32_t*>(&mine->failed) == epoch) s_last = 0;   // publish nothing after a give-up
    }
  }
  __syncthreads();
  if (s_last && tid < world) {
    flag_store(reinterpret_cast<trinity_sm100_peer_table*>(mine->workspace[tid])->flags + kAgDone + rank, epoch);
    wait_flag(mine->flags + kAgDone + tid, epoch, 0x902);
  }
}

}  // namespace
}  // namespace trinity_sm100

using namespace trinity_sm100;

extern "C" int trinity_sm100_allgather_bf16(void* workspace, int32_t source, void* out, int64_t rows,
                                            int64_t cols, int32_t axis, int32_t world, void* stream_handle) {
  if (!workspace || !out) return fail(TRINITY_SM100_E_INVALID, "allgather: null pointer");
  if (reinterpret_cast<uintptr_t>(workspace) & 255u)
    return fail(TRINITY_SM100_E_INVALID, "allgather: the workspace must be 256-byte aligned");
  if (source < 0 || source >= TRINITY_SM100_PEER_BUFFERS)
    return fail(TRINITY_SM100_E_INVALID, "allgather: symmetric buffer index %d out of range", source);
  if (rows <= 0 || cols <= 0 || cols % 8 || (axis != 0 && axis != 1))
    return fail(TRINITY_SM100_E_INVALID, "allgather: rows > 0, cols a positive multiple of 8, axis 0 or 1");
  if (world < 1 || world > 8) return fail(TRINITY_SM100_E_INVALID, "allgather: world %d out of range", world);
  if (!aligned16(out)) return fail(TRINITY_SM100_E_INVALID, "allgather: out must be 16-byte aligned");
  int sm_count = 0;
  if (int rc = require_sm100(&sm_count)) return rc;
  AllGatherParams p;
  p.table = static_cast<trinity_sm100_peer_table*>(workspace);
  p.out = static_cast<uint4*>(out);
  p.source = source;
  p.rows = rows;
  p.row_vectors = int(cols / 8);
  p.axis = axis;
  const long long vectors = rows * (cols / 8);
  long long want = (vectors + kAgThreads - 1) / kAgThreads;
  const int grid = int(want < 1 ? 1 : (want > sm_count ? sm_count : want));
  allgather_peer_kernel<<<grid, kAgThreads, 0, static_cast<cudaStream_t>(stream_handle)>>>(p);
  count_launch();
  return check_launch("allgather_peer");
}
