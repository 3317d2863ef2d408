/*
 * trinity_sm100.h -- C ABI of the sm_100a (B200) kernel library behind Trinity Lowering's
 * native CUDA provider.
 *
 * Every entry point takes plain device pointers, extents and a CUDA stream handle (void*,
 * a cudaStream_t / CUstream).  No PyTorch, C++ or Rust type crosses this boundary.  All
 * launches are asynchronous on the given stream, allocate nothing and never synchronise,
 * so they may be issued during CUDA-Graph stream capture.
 *
 * Return value: 0 on success, otherwise one of the TRINITY_SM100_E_* codes (negative).
 * trinity_sm100_last_error() returns a thread-local, NUL-terminated explanation of the
 * most recent non-zero return on the calling thread.
 *
 * Each declaration cites the interface of the reference project (youngchan2/Trinity-BE,
 * paths relative to that project) whose role it takes.
 */
#ifndef TRINITY_SM100_H
#define TRINITY_SM100_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TRINITY_SM100_ABI_VERSION 1

#if defined(__GNUC__)
#define TRINITY_SM100_API __attribute__((visibility("default")))
#else
#define TRINITY_SM100_API
#endif

enum trinity_sm100_error {
  TRINITY_SM100_OK = 0,
  TRINITY_SM100_E_INVALID = -1,     /* null pointer, bad extent, misaligned pointer or stride */
  TRINITY_SM100_E_UNSUPPORTED = -2, /* shape or mode the kernels do not implement            */
  TRINITY_SM100_E_CUDA = -3,        /* a CUDA runtime or driver call failed                  */
  TRINITY_SM100_E_DEVICE = -4,      /* current device is not compute capability 10.x         */
  TRINITY_SM100_E_TIMEOUT = -5      /* a bounded in-kernel wait gave up (see device_status)  */
};

enum trinity_sm100_dtype { TRINITY_SM100_BF16 = 0, TRINITY_SM100_FP32 = 1 };

/* How the epilogue's side operand is broadcast against the [M,N] accumulator. */
enum trinity_sm100_bias_mode {
  TRINITY_SM100_BIAS_NONE = 0,
  TRINITY_SM100_BIAS_COL_VECTOR = 1, /* bias[N], same for every row:   (bcast (load bias) 0) */
  TRINITY_SM100_BIAS_ROW_VECTOR = 2, /* bias[M], same for every column:(bcast (load bias) 1) */
  TRINITY_SM100_BIAS_MATRIX = 3      /* bias[M,N] with leading dimension ld_bias             */
};

enum trinity_sm100_activation {
  TRINITY_SM100_ACT_NONE = 0,
  TRINITY_SM100_ACT_RELU = 1,     /* max(x, 0), NaN propagates, -0 kept as the reference does */
  TRINITY_SM100_ACT_SILU = 2,     /* x * sigmoid(x)                                           */
  TRINITY_SM100_ACT_SILU_GATE = 3 /* (A@B) * ((A@B2) * sigmoid(A@B2)): two accumulators       */
};

/*
 * GEMM with fused epilogue:  out = act(A @ B + bias)   (BF16 x BF16 -> FP32 accumulate).
 *
 *   a   [m,k]  bf16 row-major, leading dimension lda (elements, multiple of 8)
 *   b   [k,n]  bf16 row-major, leading dimension ldb (elements, multiple of 8)
 *   b2  [k,n]  second right operand, only for TRINITY_SM100_ACT_SILU_GATE (same ldb)
 *   out [m,n]  bf16 or fp32 row-major, leading dimension ldo (bytes per row multiple of 16)
 *
 * All base pointers must be 16-byte aligned.  m, n, k need not be multiples of the tile:
 * loads past an edge read zero and stores past an edge are dropped.  The launcher picks the
 * form from the shape (CTA pairs on 256 x 256 tiles for large problems; 128-row tiles of 256,
 * 128 or 64 columns otherwise; for at most 64 rows against a weight with few column tiles, a
 * cluster of CTAs per tile that splits K and adds its partial sums in a fixed order), and every
 * form sums in an order that does not depend on timing: two launches give the same bits.
 *
 * Replaces the Hopper WGMMA tile kernel plus its register "follower" epilogue
 * (src/emit/provider/cute/operator/gemm/hopper/mod.rs:32-157,
 *  src/emit/provider/cute/operator/pointwise/render.rs:304-370) as launched by the generated
 * host code (src/emit/native/cuda/templates/host.cu.j2:52-76).
 */
typedef struct trinity_sm100_gemm {
  const void* a;
  const void* b;
  const void* b2;
  const void* bias;
  void* out;
  int64_t m, n, k;
  int64_t lda, ldb, ldo, ld_bias;
  int32_t bias_mode;  /* trinity_sm100_bias_mode  */
  int32_t activation; /* trinity_sm100_activation */
  int32_t out_dtype;  /* trinity_sm100_dtype      */
  int32_t reserved;
} trinity_sm100_gemm;

TRINITY_SM100_API int trinity_sm100_gemm_bf16(const trinity_sm100_gemm* args, void* stream);

/*
 * Large problems run on pairs of thread blocks that share one tensor-core instruction (two SMs
 * of one TPC).  This reports how many such pairs the current device keeps resident at once
 * (the size of the persistent grid in that mode).  For tools and tests.
 */
TRINITY_SM100_API int trinity_sm100_gemm_pair_capacity(int32_t* pairs);

/*
 * Batched form: `batch` GEMMs of one shape in one launch.  Entry z reads a + z*stride_a and
 * b + z*stride_b, adds bias + z*stride_bias and writes out + z*stride_out (strides in elements,
 * multiples of 16 bytes).  stride_b == 0 shares one right operand, stride_bias == 0 one side
 * operand.  The entries may be interleaved with the rows (stride_a < lda, stride_out < ldo), which
 * is how per-head products over [tokens, heads, features] tensors are laid out.  The gated form
 * is not batched.  The bias modes and activations of trinity_sm100_gemm_bf16 apply per entry.
 *
 * Serves the grouped per-head projections around latent attention: the absorb product
 * Q_nope[b,h,:] @ W_DK[h] and the output product T2[b,h,:] @ W_DV[h] of the reference's
 * batched-MLA fixtures (tests/fixtures/batched_mla/batched_mla_postprocessed_stage14.txt:19-59,
 * 208-241), which the reference lowers through its Triton provider.
 */
typedef struct trinity_sm100_gemm_batch {
  int64_t batch;
  int64_t stride_a, stride_b, stride_out, stride_bias;
} trinity_sm100_gemm_batch;
TRINITY_SM100_API int trinity_sm100_gemm_batched_bf16(const trinity_sm100_gemm* args,
                                                      const trinity_sm100_gemm_batch* batch, void* stream);

/*
 * RMSNorm over the last axis:
 *   y[r,c] = x[r,c] / sqrt(sum_c(x[r,c]^2) / cols + eps) * gain[c]      (FP32 math, BF16 I/O)
 * gain may be NULL (no gain) and eps may be 0, which keeps the reference's 0/0 -> NaN for an
 * all-zero row.  x and y are [rows, cols] row-major and contiguous; cols % 8 == 0.
 *
 * Replaces the three-launch square / row-sum / divide chain built from
 * src/emit/provider/cute/operator/reduce_sum/mod.rs:26-96 and
 * src/emit/provider/cute/operator/pointwise/mod.rs:37-134 (plan shape:
 * python/tests/tensor_ops.py:115-123) with one pass over the row.
 */
TRINITY_SM100_API int trinity_sm100_rmsnorm_bf16(const void* x, const void* gain, void* y, int64_t rows,
                               int64_t cols, float eps, void* stream);

/*
 * Numerically stable row softmax over the last axis (FP32 math, BF16 I/O):
 *   y[r,c] = exp(x[r,c] - max_c x[r,:]) / sum_c exp(x[r,c] - max_c x[r,:])
 * The equation form is the one the reference recognises in
 * src/emit/provider/quack/recognition/normalization.rs:138-157.
 */
TRINITY_SM100_API int trinity_sm100_softmax_bf16(const void* x, void* y, int64_t rows, int64_t cols, void* stream);

/*
 * Generic pointwise evaluation in FP32 with one rounding at the store.
 *
 *   out[r,c] = f(operands..., constants)        out is [rows, cols] row-major (1-D: rows == 1)
 *
 * f is a postfix program: TRINITY_SM100_PW_OPERAND | (index << 8) pushes an operand element,
 * TRINITY_SM100_PW_CONST pushes the FP32 bit pattern in the next word, binary opcodes pop two
 * values (left operand pushed first) and unary opcodes replace the top.  An operand is a full
 * [rows, cols] tensor, a per-row vector [rows] (the reference's `bcast ... 1`) or a per-column
 * vector [cols] (`bcast ... 0`).  ReLU is `x < 0 ? 0 : x` (NaN and the sign of zero are kept),
 * sigmoid is `1 / (1 + exp(-x))`.
 *
 * Replaces the SIMT pointwise tile kernel
 * (src/emit/provider/cute/operator/pointwise/mod.rs:37-134, special.rs:3-10).
 */
#define TRINITY_SM100_PW_MAX_OPERANDS 4
#define TRINITY_SM100_PW_MAX_PROGRAM 32
enum trinity_sm100_pw_opcode {
  TRINITY_SM100_PW_OPERAND = 1,
  TRINITY_SM100_PW_CONST = 2,
  TRINITY_SM100_PW_ADD = 16,
  TRINITY_SM100_PW_SUB = 17,
  TRINITY_SM100_PW_MUL = 18,
  TRINITY_SM100_PW_DIV = 19,
  TRINITY_SM100_PW_MAX = 20,
  TRINITY_SM100_PW_SQR = 32,
  TRINITY_SM100_PW_SQRT = 33,
  TRINITY_SM100_PW_SIGMOID = 34,
  TRINITY_SM100_PW_RELU = 35,
  TRINITY_SM100_PW_EXP = 36
};
typedef struct trinity_sm100_pw_operand {
  const void* data;
  int32_t dtype;     /* trinity_sm100_dtype */
  int32_t broadcast; /* 0 = [rows, cols], 1 = [rows] per row, 2 = [cols] per column */
} trinity_sm100_pw_operand;
typedef struct trinity_sm100_pointwise_args {
  trinity_sm100_pw_operand operands[TRINITY_SM100_PW_MAX_OPERANDS];
  int32_t operand_count;
  int32_t out_dtype; /* trinity_sm100_dtype */
  void* out;
  int64_t rows, cols;
  int32_t program_length;
  uint32_t program[TRINITY_SM100_PW_MAX_PROGRAM];
} trinity_sm100_pointwise_args;
TRINITY_SM100_API int trinity_sm100_pointwise(const trinity_sm100_pointwise_args* args, void* stream);

/*
 * y[r] = sum_c x[r,c] (square == 0) or sum_c x[r,c]^2 (square != 0); x is BF16 or FP32
 * [rows, cols], y is FP32 [rows], FP32 accumulation.
 * Replaces src/emit/provider/cute/operator/reduce_sum/mod.rs:26-96.
 */
TRINITY_SM100_API int trinity_sm100_row_reduce_sum(const void* x, int32_t x_dtype, void* y, int64_t rows,
                                 int64_t cols, int32_t square, void* stream);

/*
 * Plumbing a generated program.so needs without touching the CUDA runtime itself:
 * device check at prepare time (the capability test of
 * src/emit/native/cuda/templates/host.cu.j2:18-50), the current device, and the stream
 * synchronisation of trinity_status (host.cu.j2:78-83).
 */
TRINITY_SM100_API int trinity_sm100_prepare_device(int32_t* device_index);
TRINITY_SM100_API int trinity_sm100_current_device(int32_t* device_index);
TRINITY_SM100_API int trinity_sm100_stream_synchronize(void* stream);

/*
 * Batched multi-head latent attention decode (one query token per sequence) over a
 * compressed KV cache, split over the KV axis.
 *
 *   q      [batch, heads, d_qk]      bf16   (d_qk = d_v + d_rope; absorbed latent then rope)
 *   cache  [batch, seq, d_qk]        bf16   (values are cache[..., :d_v])
 *   out    [batch, heads, d_v]       bf16
 *   scratch: trinity_sm100_mla_scratch_bytes(batch, heads, d_v, slots) bytes of device memory,
 *            256-byte aligned, holding normalised FP32 partial outputs and their log-sum-exps
 *            for `slots` pieces per sequence (see kv_splits); not needed when slots == 1.
 *
 *   out[b,h,:] = softmax_s(scale * q[b,h,:] . cache[b,s,:]) @ cache[b,:,:d_v]
 *
 * Supported geometry: d_v == 512, d_qk == 576, 1 <= heads <= 128, any seq >= 1, batch <= 65535.
 * The sequence is processed in chunks of 64 positions; a pair of thread blocks shares each
 * piece of work.  A sequence may be cut into pieces that different pairs process (split KV);
 * the pieces are merged by a second, small kernel.
 * The math follows the reference's batched-MLA fixture
 * (tests/fixtures/batched_mla/batched_mla_postprocessed_stage14.txt:21-23,62-68,210-213;
 *  split/combine structure of ...stage20.txt:62-76,197-206) with the softmax scale and
 *  max-subtraction the decode configuration adds.
 */
typedef struct trinity_sm100_mla {
  const void* q;
  const void* cache;
  void* out;
  void* scratch;
  size_t scratch_bytes;
  int32_t batch, heads, seq, d_qk, d_v;
  int32_t kv_splits; /* > 0: that many equal splits of every sequence; 0: chosen by the library
                        (scratch for trinity_sm100_mla_default_splits() slots per sequence);
                        < 0: the balanced schedule (equal runs of KV chunks over all sequences,
                        scratch for trinity_sm100_mla_balanced_slots() slots per sequence) */
  float scale;
  int32_t reserved;
} trinity_sm100_mla;

TRINITY_SM100_API size_t trinity_sm100_mla_scratch_bytes(int32_t batch, int32_t heads, int32_t d_v,
                                       int32_t kv_splits);
TRINITY_SM100_API int trinity_sm100_mla_default_splits(int32_t batch, int32_t seq);
TRINITY_SM100_API int trinity_sm100_mla_balanced_slots(int32_t batch, int32_t seq);
/*
 * The launch schedule for (batch, seq, kv_splits), computed on the host without a launch:
 *   info    = {balanced, clusters in grid y (equal splits: the split count), partial slots per
 *              sequence, chunks of 64 positions per sequence}
 *   segment = {sequence, first chunk, chunk count, partial slot, whole-sequence flag} of the
 *             index-th piece of cluster (y, z); returns 1 if it exists, 0 if not.
 * Every (sequence, chunk) belongs to exactly one piece.  For tools and tests.
 */
TRINITY_SM100_API int trinity_sm100_mla_schedule(int32_t batch, int32_t seq, int32_t kv_splits, int32_t* info);
TRINITY_SM100_API int trinity_sm100_mla_schedule_segment(int32_t batch, int32_t seq, int32_t kv_splits, int32_t y,
                                                         int32_t z, int32_t index, int64_t* segment);
TRINITY_SM100_API int trinity_sm100_mla_decode_bf16(const trinity_sm100_mla* args, void* stream);

/*
 * The same decode for callers that cannot obtain scratch memory: a streamed artifact's launch
 * function, for example, is handed only the plan's buffers, has no workspace in its format, and
 * may be running under stream capture, so it can neither bring scratch nor allocate it.  This
 * entry point keeps the split partials in a fixed array inside the library instead
 * (TRINITY_SM100_MLA_STATIC_SCRATCH_BYTES per GPU, held from library load to process exit) and
 * calls no cudaMalloc, cudaFree or other allocating routine.  args->scratch and
 * args->scratch_bytes are ignored.
 *
 * Limit: trinity_sm100_mla_scratch_bytes(batch, heads, d_v, splits) must not exceed the array.
 * With kv_splits == 0 (schedule left to the library) a first choice that does not fit is
 * replaced by the most equal splits that do; with kv_splits != 0 (schedule fixed by the caller)
 * a request that does not fit returns TRINITY_SM100_E_UNSUPPORTED with an explanation.
 * The array's device address is looked up once per device (one cudaGetSymbolAddress with that
 * device current): by trinity_sm100_prepare_device(), which every program.so calls from
 * trinity_prepare, or else by the first call of this entry point on the device, which should
 * then come before any stream capture.
 * All calls on one GPU share the array: calls that overlap in time on the GPU race on it.
 * Nothing in the array needs clearing between calls.
 *
 * This entry point has no counterpart in the reference project.
 */
#define TRINITY_SM100_MLA_STATIC_SCRATCH_BYTES (32u << 20)
TRINITY_SM100_API int trinity_sm100_mla_decode_bf16_noalloc(const trinity_sm100_mla* args, void* stream);

/*
 * Sum all-reduce of a BF16 [rows, cols] matrix across `world` GPUs of one NVLink domain,
 * through peer-mapped memory (no NVSHMEM, no NCCL on the data path).
 *
 *   peers[r]  this buffer on rank r, mapped into the calling process (peers[rank] is local)
 *   flags[r]  rank r's flag pad (uint32, at least trinity_sm100_allreduce_flag_words() words,
 *             zeroed once before first use)
 *   epoch     strictly increasing per call on every rank, starting at 1 (flags are never reset
 *             and a zeroed pad reads as epoch 0, which is refused)
 *
 * Two-shot: rank r reduces row block r of every peer into its own buffer in FP32, then every
 * rank pulls the reduced blocks.  All waits are bounded; a wait that gives up sets the device
 * status word and the kernel returns.
 *
 * Takes the place of the NVSHMEM symmetric-heap collectives the reference declares
 * (src/native/world.cpp:122-177, src/emit/implementation/definitions/nvls.rs:59-70,
 *  src/emit/implementation/definitions/peer.rs:9-11); the reference has no all-reduce.
 */
typedef struct trinity_sm100_allreduce {
  void* const* peers;     /* host array of `world` device pointers */
  void* const* flags;     /* host array of `world` device pointers */
  int64_t rows, cols;     /* cols % 8 == 0 */
  int32_t world, rank;
  uint32_t epoch;
  int32_t reserved;
} trinity_sm100_allreduce;

TRINITY_SM100_API size_t trinity_sm100_allreduce_flag_words(void);
TRINITY_SM100_API int trinity_sm100_allreduce_bf16(const trinity_sm100_allreduce* args, void* stream);

/*
 * Peer table of a persistent (multi-GPU) artifact.  It occupies the first
 * TRINITY_SM100_PEER_TABLE_BYTES of the artifact's workspace, in device memory, and is filled
 * once by the runtime when an execution is prepared: the persistent launch block of the artifact
 * ABI (src/native/abi.h:27-40) carries only the plan's bindings and the workspace pointer, so
 * everything a kernel needs to reach the other GPUs is read from here on the device.  `epoch`
 * and `counter` are advanced by the kernels themselves, which keeps a captured launch
 * replayable; `flags` are written by the peers.  The workspace is symmetric memory: every
 * rank's copy is mapped into every process.
 */
#define TRINITY_SM100_PEER_BUFFERS 4
#define TRINITY_SM100_PEER_TABLE_BYTES 1024
typedef struct trinity_sm100_peer_table {
  int32_t world, rank;
  uint32_t epoch;    /* collective launches completed on this rank (starts at 0) */
  uint32_t counter;  /* thread blocks of the running launch that have finished   */
  uint32_t failed;   /* epoch of the last launch in which a wait gave up         */
  uint32_t reserved[3];
  uint64_t workspace[8];                             /* every rank's workspace, as mapped here     */
  uint64_t buffers[TRINITY_SM100_PEER_BUFFERS][8];   /* symmetric plan buffers, every rank's copy  */
  uint32_t flags[64];                                /* written by the peers                        */
} trinity_sm100_peer_table;

/*
 * Rank-major all-gather along axis 0 or 1 of a BF16 [rows, cols] shard (cols % 8 == 0):
 *   out[q * rows + r, c] = shard_q[r, c]   (axis 0)      out[r, q * cols + c] = shard_q[r, c]   (axis 1)
 * `workspace` is this rank's workspace with a filled peer table; the shards are symmetric buffer
 * `source` of the table; `out` is local memory.  Pulls with plain 128-bit peer loads, bounded
 * waits, no multicast; replayable inside a CUDA Graph (the call number lives in the table).
 *
 * Takes the place of the NVSHMEM all-gather the reference's plan language declares
 * (src/analysis/plan/expression.rs:227-231, python/examples/plans.py:61-73,
 *  src/emit/implementation/definitions/peer.rs:9-11), whose emission is unimplemented there
 * (src/emit/native/mod.rs:161-165).
 */
TRINITY_SM100_API int trinity_sm100_allgather_bf16(void* workspace, int32_t source, void* out, int64_t rows,
                                                   int64_t cols, int32_t axis, int32_t world, void* stream);

/*
 * Row-parallel GEMM with the sum all-reduce fused into its epilogue:
 *   out (on every rank) = sum over ranks of A_rank[m,k] @ B_rank[k,n]        BF16, FP32 accumulate
 * Every rank calls this with its own shard (`gemm`: no bias, no activation, BF16 out) and the
 * same peer tables (`reduce`: peers[r] = rank r's [m,n] output buffer, peers[rank] == gemm->out;
 * flags[r] = rank r's flag pad of at least trinity_sm100_gemm_allreduce_flag_words() zeroed
 * words, whose first trinity_sm100_allreduce_flag_words() words are left to
 * trinity_sm100_allreduce_bf16 so one pad serves both; epoch strictly increasing per call,
 * starting at 1; world is 1, 2, 4 or 8).  Inside one persistent
 * kernel the epilogue warps store their partial tile, tell every rank, and - one tile behind,
 * so the wait is short and the NVLink traffic overlaps the next tile's MMAs - each rank adds
 * the partials of its own 128/world rows of that tile in rank order in FP32 and pushes the
 * rounded rows into every rank's buffer over NVLink with 128-bit peer loads / stores.  All
 * waits are bounded.  No NVSHMEM, no NCCL, no multicast.
 *
 * The reference has no all-reduce (its plan language only has all_gather,
 * src/analysis/plan/expression.rs:227-231) and its multi-rank emission is unimplemented
 * (src/emit/native/mod.rs:161-165); this entry point is what a tensor-parallel MLP needs.
 */
TRINITY_SM100_API size_t trinity_sm100_gemm_allreduce_flag_words(int64_t m, int64_t n, int32_t world);
TRINITY_SM100_API int trinity_sm100_gemm_allreduce_bf16(const trinity_sm100_gemm* gemm,
                                      const trinity_sm100_allreduce* reduce, void* stream);

/*
 * The same fused GEMM for a persistent artifact's launch function, which has no host-side peer
 * information: `workspace` is the artifact's workspace (symmetric memory) whose first bytes are a
 * filled trinity_sm100_peer_table and whose flag pad follows the table; `output_buffer` says which
 * symmetric buffer of the table is the [m,n] output (gemm->out must be this rank's copy).  The
 * call number is the table's own counter, advanced by the kernel, so a captured launch replays
 * unchanged.  The first call for a workspace reads its table from the device (one synchronous
 * copy): make it outside any stream capture.
 * workspace bytes needed: trinity_sm100_gemm_allreduce_workspace_bytes(m, n, world).
 */
TRINITY_SM100_API size_t trinity_sm100_gemm_allreduce_workspace_bytes(int64_t m, int64_t n, int32_t world);
TRINITY_SM100_API int trinity_sm100_gemm_allreduce_workspace_bf16(const trinity_sm100_gemm* gemm, void* workspace,
                                                                  size_t workspace_bytes, int32_t output_buffer,
                                                                  void* stream);

/*
 * Diagnostic: five milestones of thread block 0 of the most recent fused launch on the current
 * device, in nanoseconds of the device's global timer: kernel start, last MMA committed, last
 * partial tile handed over, last owned rows reduced, every rank retired.  Synchronises the device.
 */
TRINITY_SM100_API int trinity_sm100_gemm_allreduce_stamps(uint64_t* stamps);

/*
 * Device status word: 0 while every bounded in-kernel wait has completed; otherwise the code
 * of the first wait that gave up (site id in the low 16 bits).  Reading synchronises the
 * device.  `clear` != 0 resets it afterwards.
 * Counterpart of the generated trinity_status() (src/emit/native/cuda/templates/host.cu.j2:78-83).
 */
TRINITY_SM100_API int trinity_sm100_device_status(uint32_t* status, int clear);

/*
 * Budget of every bounded in-kernel wait on the current device, in SM clock cycles (default
 * about two seconds; 0 restores the default).  Synchronises the device.  A wait that exceeds it
 * records its site in the device status word and the kernel returns without faulting, so the
 * context stays usable.  The reference's artifacts have no such bound: its persistent launch only
 * carries a stall hook for tests (delay_rank / delay_task / delay_cycles, src/native/abi.h:38-40).
 */
TRINITY_SM100_API int trinity_sm100_set_wait_budget(uint64_t cycles);

/* Library identity and diagnostics. */
TRINITY_SM100_API int trinity_sm100_abi_version(void);
TRINITY_SM100_API const char* trinity_sm100_last_error(void);
/* Number of kernels this library has launched in the calling process (all threads). */
TRINITY_SM100_API uint64_t trinity_sm100_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* TRINITY_SM100_H */
