// Batched MLA decode over a compressed KV cache (one query token, up to 128 heads).
//
//   S = scale * q . cache^T      [heads x seq]      tcgen05, FP32 scores in TMEM
//   P = exp(S - max) (online)                        FP32 in registers, BF16 back into TMEM
//   O = P @ cache[:, :512] / sum(P)  [heads x 512]  tcgen05, FP32 accumulator in TMEM
//
// A 128-row FP32 accumulator for all 512 latent columns would fill TMEM by itself, so one CTA
// owns one (batch, KV split, latent half): 256 accumulator columns, two 32-column score
// buffers, and the first 384 query features as a TMEM-resident A operand (packed BF16 pairs).
// The remaining 192 query features stay in shared memory, which leaves room for a four-stage
// ring of 32-position cache chunks (each chunk is read from HBM once per latent half and
// serves both products: K-major as the score operand, N-major as the value operand).
//
//   warp 0    TMA producer (query tail boxes, then the cache chunk ring)
//   warp 1    MMA issuer: QK(j) = 24 TMEM-A + 12 SMEM-A MMAs (N=32), PV(j-1) = 2 TMEM-A MMAs
//             (N=256); scores of chunk j are issued before the values of chunk j-1 so the
//             tensor pipe works while the softmax warps process chunk j-1
//   warps 2-5 one thread per head: score load, running max / sum, conditional rescale of the
//             accumulator, BF16 probabilities written over the score buffer, final epilogue
//
// With kv_splits == 1 the CTA writes BF16 output directly.  Otherwise it writes a normalised
// FP32 partial and its log-sum-exp to scratch and a small kernel merges the splits.
// Algorithmic traffic: q + cache + out bytes; the scratch adds 2 * splits * batch * heads *
// 513 * 4 bytes when splits > 1.
#include "host_common.h"
#include "sm100_ptx.cuh"

namespace trinity_sm100 {
namespace {

constexpr int kMlaThreads = 192;
constexpr int kKv = 32;                       // cache positions per chunk
constexpr int kDqk = 576, kDv = 512;
constexpr int kBoxes = kDqk / 64;             // 9 feature boxes of 64
constexpr int kKvStages = 4;
constexpr int kChunkBytes = kKv * kDqk * 2;   // 36864
constexpr int kBoxBytes = kKv * 128;          // 4096: one [32 x 64] box
constexpr int kQTmemFeatures = 384;           // features [0, 384) live in TMEM
constexpr int kQSmemBoxes = (kDqk - kQTmemFeatures) / 64;  // 3 boxes of [128 x 64]
constexpr int kQBoxBytes = 128 * 128;
constexpr int kMlaSmem = 1024 + kQSmemBoxes * kQBoxBytes + kKvStages * kChunkBytes + 256;
// TMEM columns
constexpr uint32_t kColO = 0, kColS = 256, kColQ = 320, kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;     // in log2 units: probabilities stay below 2^8

struct MlaParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  float* partial_o;   // [batch][splits][heads][512]
  float* partial_lse; // [batch][splits][heads]
  int batch, heads, seq, splits;
  float scale_log2;
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

// Chunk range [first, first + count) of split `s` when `chunks` are dealt out evenly.
__host__ __device__ inline void split_range(int chunks, int splits, int s, int& first, int& count) {
  const int base = chunks / splits, extra = chunks % splits;
  first = s * base + (s < extra ? s : extra);
  count = base + (s < extra ? 1 : 0);
}

__global__ void __launch_bounds__(kMlaThreads, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap map_q,
                  const __grid_constant__ CUtensorMap map_cache, const MlaParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_smem = smem_base;
  const uint32_t kv_smem = smem_base + kQSmemBoxes * kQBoxBytes;
  const uint32_t bar_base = kv_smem + kKvStages * kChunkBytes;
  // barriers: kv_full[4], kv_empty[4], s_full[2], p_full[2], q_full, q_tmem, pv_done
  auto kv_full = [&](int s) { return bar_base + 8u * s; };
  auto kv_empty = [&](int s) { return bar_base + 8u * (kKvStages + s); };
  auto s_full = [&](int b) { return bar_base + 8u * (2 * kKvStages + b); };
  auto p_full = [&](int b) { return bar_base + 8u * (2 * kKvStages + 2 + b); };
  const uint32_t q_full = bar_base + 8u * (2 * kKvStages + 4);
  const uint32_t q_tmem = bar_base + 8u * (2 * kKvStages + 5);
  const uint32_t pv_done = bar_base + 8u * (2 * kKvStages + 6);
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(
      smem + kQSmemBoxes * kQBoxBytes + kKvStages * kChunkBytes + 8 * (2 * kKvStages + 7));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int half = blockIdx.x;   // latent half: columns [256*half, 256*half + 256)
  const int split = blockIdx.y;
  const int b = blockIdx.z;

  const int total_chunks = (p.seq + kKv - 1) / kKv;
  int first_chunk, num_chunks;
  split_range(total_chunks, p.splits, split, first_chunk, num_chunks);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(s_full(i), 1);
      mbar_init(p_full(i), 4);
    }
    mbar_init(q_full, 1);
    mbar_init(q_tmem, 4);
    mbar_init(pv_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_cache);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && num_chunks > 0) {
      mbar_arrive_expect_tx(q_full, kQSmemBoxes * kQBoxBytes);
      for (int f = 0; f < kQSmemBoxes; ++f)
        tma_load_3d(q_smem + f * kQBoxBytes, &map_q, q_full, kQTmemFeatures + f * 64, 0, b);
      for (int j = 0; j < num_chunks; ++j) {
        const int s = j % kKvStages;
        const uint32_t phase = (j / kKvStages) & 1u;
        if (!mbar_wait(kv_empty(s), phase ^ 1u, 0x401)) break;
        mbar_arrive_expect_tx(kv_full(s), kChunkBytes);
        const int kv0 = (first_chunk + j) * kKv;
#pragma unroll
        for (int f = 0; f < kBoxes; ++f)
          tma_load_3d(kv_smem + s * kChunkBytes + f * kBoxBytes, &map_cache, kv_full(s), f * 64,
                      kv0, b);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && num_chunks > 0) {
      constexpr uint32_t kIdescQK = umma_idesc_bf16(128, kKv, 0, 0);
      constexpr uint32_t kIdescPV = umma_idesc_bf16(128, 256, 0, 1);
      bool ok = mbar_wait(q_full, 0, 0x501) && mbar_wait(q_tmem, 0, 0x502);
      tc_fence_after();
      for (int j = 0; j <= num_chunks && ok; ++j) {
        if (j < num_chunks) {
          const int s = j % kKvStages;
          if (!mbar_wait(kv_full(s), (j / kKvStages) & 1u, 0x503)) { ok = false; break; }
          tc_fence_after();
          const uint32_t stage = kv_smem + s * kChunkBytes;
          const uint32_t d_s = tmem_base + kColS + (j & 1) * kKv;
          // scores: 36 K-steps of 16 features
#pragma unroll
          for (int ks = 0; ks < kDqk / 16; ++ks) {
            const uint64_t b_desc =
                umma_smem_desc(stage + (ks / 4) * kBoxBytes + (ks % 4) * 32, 16, 1024);
            if (ks < kQTmemFeatures / 16) {
              umma_bf16_ts(d_s, tmem_base + kColQ + ks * 8, b_desc, kIdescQK, ks != 0);
            } else {
              const int t = ks - kQTmemFeatures / 16;
              const uint64_t a_desc =
                  umma_smem_desc(q_smem + (t / 4) * kQBoxBytes + (t % 4) * 32, 16, 1024);
              umma_bf16_ss(d_s, a_desc, b_desc, kIdescQK, 1u);
            }
          }
          umma_commit(s_full(j & 1));
        }
        if (j >= 1) {
          const int jj = j - 1;
          const int s = jj % kKvStages;
          if (!mbar_wait(p_full(jj & 1), (jj >> 1) & 1u, 0x504)) { ok = false; break; }
          tc_fence_after();
          const uint32_t stage = kv_smem + s * kChunkBytes + half * 4 * kBoxBytes;
          const uint32_t a_p = tmem_base + kColS + (jj & 1) * kKv;
#pragma unroll
          for (int ks = 0; ks < kKv / 16; ++ks) {
            // values: N-major, 64-latent boxes 4096 B apart, 8-position groups 1024 B apart
            const uint64_t b_desc = umma_smem_desc(stage + ks * 2048, kBoxBytes, 1024);
            umma_bf16_ts(tmem_base + kColO, a_p + ks * 8, b_desc, kIdescPV, (jj | ks) != 0);
          }
          umma_commit(kv_empty(s));
          umma_commit(pv_done);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / epilogue warps
    const int quad = warp & 3;
    const int row = quad * 32 + lane;              // head index
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const bool live = row < p.heads;
    if (num_chunks > 0) {
      // Query features [0, 384) -> TMEM as packed BF16 pairs (word c = features 2c, 2c+1).
      const uint4* qrow = reinterpret_cast<const uint4*>(
          p.q + (static_cast<long long>(b) * p.heads + (live ? row : 0)) * kDqk);
#pragma unroll 1
      for (int c = 0; c < kQTmemFeatures / 64; ++c) {
        uint32_t w[32];
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          uint4 x = live ? __ldg(qrow + c * 8 + v) : make_uint4(0, 0, 0, 0);
          w[v * 4 + 0] = x.x; w[v * 4 + 1] = x.y; w[v * 4 + 2] = x.z; w[v * 4 + 3] = x.w;
        }
        tmem_st_32x32b_x32(lane_base + kColQ + c * 32, w);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_tmem);
    }

    float m_ref = -INFINITY;   // reference maximum (log2 domain, scaled)
    float l = 0.0f;            // running sum of probabilities relative to m_ref
    bool ok = true;
    for (int j = 0; j < num_chunks && ok; ++j) {
      if (!mbar_wait(s_full(j & 1), (j >> 1) & 1u, 0x601)) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = lane_base + kColS + (j & 1) * kKv;
      uint32_t sv[32];
      tmem_ld_32x32b_x32(s_addr, sv);
      tmem_ld_wait();
      const int valid = p.seq - (first_chunk + j) * kKv;  // positions of this chunk inside seq
      float t[32];
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        t[i] = i < valid ? __uint_as_float(sv[i]) * p.scale_log2 : -INFINITY;
        mx = fmaxf(mx, t[i]);
      }
      const bool grow = mx > m_ref + kRescaleThreshold;   // always true for the first chunk
      if (__any_sync(0xffffffffu, grow)) {
        const float new_ref = grow ? mx : m_ref;
        const float f = (grow && j > 0) ? fast_exp2(m_ref - new_ref) : 1.0f;
        if (j > 0) {
          // The accumulator may only be touched once the values of chunk j-1 have landed.
          if (!mbar_wait(pv_done, (j - 1) & 1u, 0x602)) { ok = false; break; }
          tc_fence_after();
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
          l *= f;
        }
        m_ref = new_ref;
      }
      uint32_t pw[16];
      float sum = 0.0f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float p0 = fast_exp2(t[2 * i] - m_ref);
        const float p1 = fast_exp2(t[2 * i + 1] - m_ref);
        sum += p0 + p1;
        pw[i] = pack_bf16x2(p0, p1);
      }
      l += sum;
      tmem_st_32x32b_x16(s_addr, pw);   // probabilities overwrite the first 16 score columns
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(j & 1));
    }

    if (num_chunks > 0 && ok && mbar_wait(pv_done, (num_chunks - 1) & 1u, 0x603)) {
      tc_fence_after();
      const float inv_l = 1.0f / l;
      if (p.splits == 1) {
        __nv_bfloat16* orow =
            p.out + (static_cast<long long>(b) * p.heads + row) * kDv + half * 256;
#pragma unroll 1
        for (int c = 0; c < 256; c += 32) {
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
        const long long slot = (static_cast<long long>(b) * p.splits + split) * p.heads + row;
        float* prow = p.partial_o + slot * kDv + half * 256;
#pragma unroll 1
        for (int c = 0; c < 256; c += 32) {
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
        if (live && half == 0) p.partial_lse[slot] = m_ref + log2f(l);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    if (g_device_status != 0)
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// out[b,h,:] = sum_s w_s * partial[b,s,h,:],  w_s = 2^(lse_s - max) / sum_s 2^(lse_s - max).
// Splits that held no positions have lse = -inf and weight zero.
__global__ void mla_combine_kernel(const float* __restrict__ partial_o,
                                   const float* __restrict__ partial_lse,
                                   __nv_bfloat16* __restrict__ out, int heads, int splits) {
  const int bh = blockIdx.x;  // b * heads + h
  const int b = bh / heads, h = bh % heads;
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s)
    mx = fmaxf(mx, partial_lse[(static_cast<long long>(b) * splits + s) * heads + h]);
  float denom = 0.0f;
  for (int s = 0; s < splits; ++s)
    denom += exp2f(partial_lse[(static_cast<long long>(b) * splits + s) * heads + h] - mx);
  const float inv = 1.0f / denom;
  for (int c = threadIdx.x; c < kDv; c += blockDim.x) {
    float acc = 0.0f;
    for (int s = 0; s < splits; ++s) {
      const long long slot = (static_cast<long long>(b) * splits + s) * heads + h;
      const float w = exp2f(partial_lse[slot] - mx) * inv;
      if (w != 0.0f) acc += w * partial_o[slot * kDv + c];
    }
    out[static_cast<long long>(bh) * kDv + c] = __float2bfloat16(acc);
  }
}

size_t scratch_bytes(int batch, int heads, int d_v, int splits) {
  if (splits <= 1) return 0;
  const size_t slots = size_t(batch) * splits * heads;
  return ((slots * d_v * 4 + 255) / 256) * 256 + ((slots * 4 + 255) / 256) * 256;
}

}  // namespace
}  // namespace trinity_sm100

using namespace trinity_sm100;

extern "C" size_t trinity_sm100_mla_scratch_bytes(int32_t batch, int32_t heads, int32_t d_v,
                                                  int32_t kv_splits) {
  if (batch <= 0 || heads <= 0 || d_v <= 0) return 0;
  return scratch_bytes(batch, heads, d_v, kv_splits);
}

extern "C" int trinity_sm100_mla_default_splits(int32_t batch, int32_t seq) {
  // Two CTAs (latent halves) per (batch, split); aim for about one CTA per SM without
  // splitting a sequence more finely than 512 positions per split.
  int sms = 148;
  int device = 0;
  if (cudaGetDevice(&device) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (batch <= 0 || seq <= 0) return 1;
  int splits = sms / (2 * batch);
  const int max_splits = (seq + 511) / 512;
  if (splits > max_splits) splits = max_splits;
  return splits < 1 ? 1 : splits;
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
  int splits = a.kv_splits > 0 ? a.kv_splits : trinity_sm100_mla_default_splits(a.batch, a.seq);
  const int chunks = (a.seq + kKv - 1) / kKv;
  if (splits > chunks) splits = chunks;
  if (splits > 65535) return fail(TRINITY_SM100_E_UNSUPPORTED, "mla: too many splits");
  const size_t need = scratch_bytes(a.batch, a.heads, a.d_v, splits);
  if (need > 0) {
    if (!a.scratch || a.scratch_bytes < need)
      return fail(TRINITY_SM100_E_INVALID, "mla: %d splits need %zu scratch bytes (got %zu)",
                  splits, need, a.scratch_bytes);
    if (reinterpret_cast<uintptr_t>(a.scratch) & 255u)
      return fail(TRINITY_SM100_E_INVALID, "mla: scratch must be 256-byte aligned");
  }
  if (int rc = require_sm100(nullptr)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (!configured[device & 63]) {
    cudaError_t e = cudaFuncSetAttribute(mla_decode_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmem);
    if (e != cudaSuccess)
      return fail(TRINITY_SM100_E_CUDA, "mla: shared memory opt-in: %s", cudaGetErrorString(e));
    configured[device & 63] = true;
  }
  CUtensorMap map_q, map_cache;
  int rc;
  if ((rc = make_tensor_map_3d(&map_q, a.q, 2, kDqk, a.heads, a.batch, kDqk * 2ull,
                               uint64_t(a.heads) * kDqk * 2, 64, 128, 1, true)))
    return rc;
  if ((rc = make_tensor_map_3d(&map_cache, a.cache, 2, kDqk, a.seq, a.batch, kDqk * 2ull,
                               uint64_t(a.seq) * kDqk * 2, 64, kKv, 1, true)))
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
  p.splits = splits;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  dim3 grid(2, splits, a.batch);
  mla_decode_kernel<<<grid, kMlaThreads, kMlaSmem, stream>>>(map_q, map_cache, p);
  count_launch();
  if ((rc = check_launch("mla_decode"))) return rc;
  if (splits > 1) {
    mla_combine_kernel<<<a.batch * a.heads, 128, 0, stream>>>(p.partial_o, p.partial_lse, p.out,
                                                              a.heads, splits);
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

extern "C" int trinity_sm100_mla_decode_bf16_noalloc(const trinity_sm100_mla* args,
                                                     void* stream_handle) {
  if (!args) return fail(TRINITY_SM100_E_INVALID, "mla (no-alloc): null argument block");
  trinity_sm100_mla call = *args;
  if (call.batch <= 0 || call.heads <= 0 || call.seq <= 0)
    return fail(TRINITY_SM100_E_INVALID, "mla (no-alloc): empty extent");
  int splits =
      call.kv_splits > 0 ? call.kv_splits : trinity_sm100_mla_default_splits(call.batch, call.seq);
  const int chunks = (call.seq + kKv - 1) / kKv;
  if (splits > chunks) splits = chunks;
  const size_t need = scratch_bytes(call.batch, call.heads, call.d_v, splits);
  if (need > size_t(TRINITY_SM100_MLA_STATIC_SCRATCH_BYTES))
    return fail(TRINITY_SM100_E_UNSUPPORTED,
                "mla (no-alloc): batch %d x %d splits x %d heads needs %zu scratch bytes, above the "
                "built-in %zu; use fewer splits or trinity_sm100_mla_decode_bf16 with your own "
                "scratch",
                call.batch, splits, call.heads, need, size_t(TRINITY_SM100_MLA_STATIC_SCRATCH_BYTES));
  void* scratch = nullptr;
  if (int rc = static_scratch_address(&scratch)) return rc;
  call.kv_splits = splits;
  call.scratch = scratch;
  call.scratch_bytes = TRINITY_SM100_MLA_STATIC_SCRATCH_BYTES;
  return trinity_sm100_mla_decode_bf16(&call, stream_handle);
}
