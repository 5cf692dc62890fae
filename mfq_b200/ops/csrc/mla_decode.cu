// Latent-attention decode over a shared-row FP8 cache (weight-absorbed form of multi-head latent attention).
//
// The cache holds ONE row per token for all heads: [rotary key part (64) | normalised latent (512)] = 576 values as FP8
// with one multiplier per token.  Queries arrive already mapped into that space (q_rope | W_k^T q_nope), so every head
// of a sequence scores against the same rows, and the value of a token is the latent part of its row: the output per
// head is a 512-wide latent mix that the caller expands with W_v.  Per token the cache costs 1.1 KB instead of
// 2 * heads * 256 B for expanded per-head keys and values.
//
// Page layout = the generic paged cache with one KV head and head width 576: keys [9 chunks][16 tokens][64], values
// transposed [576 dims][16 token slots] (slot order 0 1 8 9 2 3 10 11 ..., so a thread's four bytes are the tokens of its
// two MMA k-pairs); only value dims 0..511 (the latent) are read.
//
//   mla_latent_write   one warp per token: row amax -> multiplier, E4M3 codes into the key chunks and the value columns.
//   mla_decode         one CTA = (sequence, 16 heads, KV split), four warps, 64 tokens (four pages) per step, two stages of
//                      cp.async.bulk page copies on mbarriers.  Phase 1: warp w scores the 16 heads against page w
//                      (m16n8k16 f16 MMAs, 36 k-steps over the 576 dims, FP8 -> f16 by cvt straight into fragments;
//                      query fragments come from a padded f16 tile in shared memory since 16 x 576 does not fit
//                      registers).  The four warps meet through shared memory for the row maxima, write their
//                      probabilities (times the token's value multiplier) as an f16 tile, meet again for the row sums.
//                      Phase 2: warp w owns latent dims [128 w, 128 w + 128) of the output: P (16 x 64) times the four
//                      value pages, 64 MMAs, accumulators 64 registers.  Two block barriers per 64 tokens.
//   mla_reduce         merges the KV splits (log-sum-exp weights) and writes bf16.
//
// 16 live MMA rows = 16 heads of one sequence: this is where latent attention makes the warp MMA efficient at decode
// (a GQA group of 4 leaves 12 of 16 rows empty).  Waits are bounded and report through the status word.
//
// Reference counterparts: mfq/kernels/cuda/glm_dsa.cu:43-173 (rope + latent cache write), deepseek_v4_attention.cu.
#include "common.cuh"

#include <cfloat>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace mfq {
namespace {

constexpr int kDq = 576;        // row width: 64 rotary + 512 latent
constexpr int kDv = 512;        // value = the latent part
constexpr int kQS = 584;        // f16 row stride of the query tile in shared memory (16-byte pad against bank conflicts)
constexpr int kPS = 72;         // f16 row stride of the probability tile
constexpr int kKPage = 16 * kDq;  // bytes of one page of keys (or values)
constexpr int kVPart = 16 * kDv;  // bytes of the value page that are read
constexpr int kStage = 4 * (kKPage + kVPart + 128);
constexpr float kNegInf = -1e30f;

__device__ __forceinline__ void bulk_copy(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ uint32_t e4m3x2_f16x2(uint16_t v) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
  return r;
}
__device__ __forceinline__ uint32_t f16x2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// rows [T, 576] bf16 (rotary part already rotated) -> FP8 pages.  slot = page * 16 + offset, negative = skip.
__global__ void __launch_bounds__(128) mla_latent_write_kernel(const __nv_bfloat16* __restrict__ rows, const int* __restrict__ slots,
                                                               uint8_t* __restrict__ k_cache, uint8_t* __restrict__ v_cache,
                                                               float* __restrict__ k_scale, float* __restrict__ v_scale, int T) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const int slot = slots[t];
  if (slot < 0) return;
  const int page = slot >> 4, off = slot & 15;
  const __nv_bfloat16* row = rows + size_t(t) * kDq;
  float2 v[9];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 9; ++j) {
    v[j] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + 64 * j + 2 * lane));
    amax = fmaxf(amax, fmaxf(fabsf(v[j].x), fabsf(v[j].y)));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = fmaxf(amax, 1e-12f) / 448.f, inv = 1.f / scale;
  // value slot of this token inside its page: tokens are stored in the order 0 1 8 9 2 3 10 11 4 5 12 13 6 7 14 15
  const int vslot = (off & 1) | ((off & 8) >> 2) | ((off & 6) << 1);
  uint8_t* kp = k_cache + size_t(page) * kKPage + off * 64 + 2 * lane;
  uint8_t* vp = v_cache + size_t(page) * kKPage + vslot;
#pragma unroll
  for (int j = 0; j < 9; ++j) {
    const __nv_fp8x2_storage_t q = __nv_cvt_float2_to_fp8x2(make_float2(v[j].x * inv, v[j].y * inv), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint16_t*>(kp + j * 1024) = q;
    // the value row of a token is its latent (row dims 64 ..): value dim d = row dim 64 + d
    if (j >= 1) {
      const int d = 64 * (j - 1) + 2 * lane;
      vp[size_t(d) * 16] = uint8_t(q & 0xFF);
      vp[size_t(d + 1) * 16] = uint8_t(q >> 8);
    }
  }
  if (lane == 0) {
    k_scale[size_t(page) * 16 + off] = scale;
    v_scale[size_t(page) * 16 + off] = scale;
  }
}

constexpr int kSmemQ = 16 * kQS * 2;
constexpr int kSmemP = 16 * kPS * 2;
constexpr int kSmemBytes = kSmemQ + 2 * kStage + kSmemP + 2 * 4 * 16 * 4 + 64;

__global__ void __launch_bounds__(128, 1)
mla_decode_kernel(const __nv_bfloat16* __restrict__ q, const uint8_t* __restrict__ k_cache, const uint8_t* __restrict__ v_cache,
                  const float* __restrict__ k_scale, const float* __restrict__ v_scale, const int* __restrict__ block_table,
                  const int* __restrict__ seq_lens, __nv_bfloat16* __restrict__ out, float* __restrict__ part_acc,
                  float* __restrict__ part_ml, int H, int max_pages, float scale_log2, int* status) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(128) uint8_t smem[];
  __half* Qs = reinterpret_cast<__half*>(smem);
  uint8_t* stages = smem + kSmemQ;
  __half* Ps = reinterpret_cast<__half*>(stages + 2 * kStage);
  float* red_max = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(Ps) + kSmemP);  // [4 warps][16 rows]
  float* red_sum = red_max + 64;
  uint64_t* bars = reinterpret_cast<uint64_t*>(red_sum + 64);  // one per stage
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g8 = lane >> 2, c = lane & 3;
  const int seq = blockIdx.x, h0 = blockIdx.y * 16, split = blockIdx.z, nsplit = gridDim.z;
  const int len = seq_lens[seq];
  const int pages_total = (len + 15) >> 4;
  const int groups_total = (pages_total + 3) >> 2;
  const int per_split = (groups_total + nsplit - 1) / nsplit;
  const int g_begin = split * per_split, g_end = min(groups_total, g_begin + per_split);
  const int n_groups = max(0, g_end - g_begin);

  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  // stale bytes of a page that is never loaded (past the sequence end) must be finite numbers: zero both stages once
  for (int i = threadIdx.x; i < 2 * kStage / 16; i += 128) reinterpret_cast<uint4*>(stages)[i] = make_uint4(0, 0, 0, 0);
  // query tile: 16 heads x 576, scaled by sm_scale * log2(e), as f16
  for (int i = threadIdx.x; i < 16 * (kDq / 2); i += 128) {
    const int r = i / (kDq / 2), d = 2 * (i % (kDq / 2));
    float2 v = make_float2(0.f, 0.f);
    if (h0 + r < H) v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q + (size_t(seq) * H + h0 + r) * kDq + d));
    *reinterpret_cast<__half2*>(Qs + r * kQS + d) = __floats2half2_rn(v.x * scale_log2, v.y * scale_log2);
  }
  fence_proxy_async_smem();  // the zero fill above precedes the bulk copies into the same bytes
  __syncthreads();

  const int* bt = block_table + size_t(seq) * max_pages;
  auto issue = [&](int gi) {  // thread 0: the four pages of group gi into stage gi & 1
    const int stage = gi & 1;
    uint8_t* st = stages + stage * kStage;
    const int p0 = (g_begin + gi) * 4;
    const int np = min(4, pages_total - p0);
    mbar_expect_tx(&bars[stage], uint32_t(np) * (kKPage + kVPart + 128));
    for (int j = 0; j < np; ++j) {
      const size_t page = size_t(bt[p0 + j]);
      uint8_t* dst = st + j * (kKPage + kVPart + 128);
      bulk_copy(dst, k_cache + page * kKPage, kKPage, &bars[stage]);
      bulk_copy(dst + kKPage, v_cache + page * kKPage, kVPart, &bars[stage]);
      bulk_copy(dst + kKPage + kVPart, k_scale + page * 16, 64, &bars[stage]);
      bulk_copy(dst + kKPage + kVPart + 64, v_scale + page * 16, 64, &bars[stage]);
    }
  };
  if (threadIdx.x == 0) {
    if (n_groups > 0) issue(0);
    if (n_groups > 1) issue(1);
  }

  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_run[2] = {kNegInf, kNegInf}, l_run[2] = {0.f, 0.f};
  bool ok = true;
  for (int gi = 0; gi < n_groups; ++gi) {
    const int stage = gi & 1;
    ok = mbar_wait(&bars[stage], (gi >> 1) & 1, abort_flag, status, kStatusTimeoutProducer) && ok;
    const uint8_t* st = stages + stage * kStage;
    const uint8_t* mine = st + warp * (kKPage + kVPart + 128);  // this warp scores page `warp` of the group
    const float* ks = reinterpret_cast<const float*>(mine + kKPage + kVPart);
    const float* vs = ks + 16;
    const int tok0 = ((g_begin + gi) * 4 + warp) * 16;  // first token of that page

    // ---- phase 1: S = Q K^T for 16 tokens ----
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll 4
    for (int kstep = 0; kstep < kDq / 16; ++kstep) {
      // dims are visited in a permuted order (the same for Q and K): a thread's two k-pairs are four contiguous bytes
      const int d0 = 64 * (kstep >> 2) + 16 * c + 4 * (kstep & 3);
      const uint2 qa_lo = *reinterpret_cast<const uint2*>(Qs + g8 * kQS + d0);
      const uint2 qa_hi = *reinterpret_cast<const uint2*>(Qs + (g8 + 8) * kQS + d0);
      const uint32_t a[4] = {qa_lo.x, qa_hi.x, qa_lo.y, qa_hi.y};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const uint32_t kb = *reinterpret_cast<const uint32_t*>(mine + (kstep >> 2) * 1024 + (8 * nt + g8) * 64 + 16 * c + 4 * (kstep & 3));
        mma16816(s[nt], a, e4m3x2_f16x2(uint16_t(kb & 0xFFFF)), e4m3x2_f16x2(uint16_t(kb >> 16)));
      }
    }
    float bmax[2] = {kNegInf, kNegInf};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = 8 * nt + 2 * c + (e & 1);
        const float v = tok0 + tok < len ? s[nt][e] * ks[tok] : kNegInf;
        s[nt][e] = v;
        bmax[e >> 1] = fmaxf(bmax[e >> 1], v);
      }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      bmax[half] = fmaxf(bmax[half], __shfl_xor_sync(0xffffffffu, bmax[half], 1));
      bmax[half] = fmaxf(bmax[half], __shfl_xor_sync(0xffffffffu, bmax[half], 2));
    }
    if (c == 0) { red_max[warp * 16 + g8] = bmax[0]; red_max[warp * 16 + g8 + 8] = bmax[1]; }
    ok = __syncthreads_and(ok) != 0;  // (A) every warp has left the previous group's phase 2; `ok` is uniform from here
    if (!ok) break;
    if (threadIdx.x == 0 && gi >= 1 && gi + 1 < n_groups) {
      fence_proxy_async_smem();
      issue(gi + 1);  // its stage was read last by group gi - 1
    }
    float alpha[2], psum[2] = {0.f, 0.f};
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = g8 + 8 * half;
      const float gm = fmaxf(fmaxf(red_max[r], red_max[16 + r]), fmaxf(red_max[32 + r], red_max[48 + r]));
      const float m_new = fmaxf(m_run[half], gm);
      alpha[half] = exp2f(m_run[half] - m_new);
      m_run[half] = m_new;
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int tok = 8 * nt + 2 * c;
      const float p0 = exp2f(s[nt][0] - m_run[0]), p1 = exp2f(s[nt][1] - m_run[0]);
      const float p2 = exp2f(s[nt][2] - m_run[1]), p3 = exp2f(s[nt][3] - m_run[1]);
      psum[0] += p0 + p1;
      psum[1] += p2 + p3;
      *reinterpret_cast<uint32_t*>(Ps + g8 * kPS + warp * 16 + tok) = f16x2(p0 * vs[tok], p1 * vs[tok + 1]);
      *reinterpret_cast<uint32_t*>(Ps + (g8 + 8) * kPS + warp * 16 + tok) = f16x2(p2 * vs[tok], p3 * vs[tok + 1]);
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      psum[half] += __shfl_xor_sync(0xffffffffu, psum[half], 1);
      psum[half] += __shfl_xor_sync(0xffffffffu, psum[half], 2);
    }
    if (c == 0) { red_sum[warp * 16 + g8] = psum[0]; red_sum[warp * 16 + g8 + 8] = psum[1]; }
    __syncthreads();  // (B) probabilities and row sums of all four pages are in shared memory
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = g8 + 8 * half;
      l_run[half] = l_run[half] * alpha[half] + (red_sum[r] + red_sum[16 + r]) + (red_sum[32 + r] + red_sum[48 + r]);
    }

    // ---- phase 2: O[:, 128 warp ..] = alpha O + P V ----
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) { o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0]; o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1]; }
#pragma unroll
    for (int kj = 0; kj < 4; ++kj) {
      uint32_t a[4];
      a[0] = *reinterpret_cast<const uint32_t*>(Ps + g8 * kPS + 16 * kj + 2 * c);
      a[1] = *reinterpret_cast<const uint32_t*>(Ps + (g8 + 8) * kPS + 16 * kj + 2 * c);
      a[2] = *reinterpret_cast<const uint32_t*>(Ps + g8 * kPS + 16 * kj + 2 * c + 8);
      a[3] = *reinterpret_cast<const uint32_t*>(Ps + (g8 + 8) * kPS + 16 * kj + 2 * c + 8);
      const uint8_t* vpage = st + kj * (kKPage + kVPart + 128) + kKPage;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        const uint32_t vb = *reinterpret_cast<const uint32_t*>(vpage + (128 * warp + 8 * nt + g8) * 16 + 4 * c);
        mma16816(o[nt], a, e4m3x2_f16x2(uint16_t(vb & 0xFFFF)), e4m3x2_f16x2(uint16_t(vb >> 16)));
      }
    }
  }
  if (!ok) return;  // uniform: decided by the barrier above; the host sees the status word

  if (nsplit == 1) {
    const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      const int d = 128 * warp + 8 * nt + 2 * c;
      if (h0 + g8 < H)
        *reinterpret_cast<__nv_bfloat162*>(out + (size_t(seq) * H + h0 + g8) * kDv + d) = __floats2bfloat162_rn(o[nt][0] * inv0, o[nt][1] * inv0);
      if (h0 + g8 + 8 < H)
        *reinterpret_cast<__nv_bfloat162*>(out + (size_t(seq) * H + h0 + g8 + 8) * kDv + d) = __floats2bfloat162_rn(o[nt][2] * inv1, o[nt][3] * inv1);
    }
    return;
  }
  // partials: unnormalised latent mix, running maximum (log2 domain) and sum per (sequence, head, split)
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int h = h0 + g8 + 8 * half;
    if (h >= H) continue;
    const size_t idx = (size_t(seq) * H + h) * nsplit + split;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
      *reinterpret_cast<float2*>(part_acc + idx * kDv + 128 * warp + 8 * nt + 2 * c) = make_float2(o[nt][2 * half], o[nt][2 * half + 1]);
    if (warp == 0 && c == 0) { part_ml[idx * 2] = m_run[half]; part_ml[idx * 2 + 1] = l_run[half]; }
  }
}

__global__ void __launch_bounds__(128) mla_reduce_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                                         __nv_bfloat16* __restrict__ out, int nsplit) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;  // (sequence, head)
  float m = kNegInf;
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, part_ml[(row * nsplit + s) * 2]);
  float l = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < nsplit; ++s) {
    const float ms = part_ml[(row * nsplit + s) * 2], ls = part_ml[(row * nsplit + s) * 2 + 1];
    const float w = ls > 0.f ? exp2f(ms - m) : 0.f;
    l += w * ls;
    const float4 v = *reinterpret_cast<const float4*>(part_acc + (row * nsplit + s) * kDv + 4 * threadIdx.x);
    acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(out + row * kDv + 4 * threadIdx.x);
  dst[0] = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
  dst[1] = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
}

}  // namespace
}  // namespace mfq

using namespace mfq;

extern "C" int mfq_mla_latent_write(const void* rows, const int* slots, void* k_cache, void* v_cache, float* k_scale,
                                    float* v_scale, int T, cudaStream_t stream) {
  if (T <= 0) return -1;
  launch_kernel(mla_latent_write_kernel, dim3((T + 3) / 4), dim3(128), 0, stream, static_cast<const __nv_bfloat16*>(rows), slots,
                static_cast<uint8_t*>(k_cache), static_cast<uint8_t*>(v_cache), k_scale, v_scale, T);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

// q [B, H, 576] bf16 (rotary part | absorbed latent part), out [B, H, 512] bf16.  part_acc needs B*H*splits*512 floats,
// part_ml B*H*splits*2 (unused for splits == 1).
extern "C" int mfq_mla_decode(const void* q, const void* k_cache, const void* v_cache, const float* k_scale, const float* v_scale,
                              const int* block_table, const int* seq_lens, void* out, float* part_acc, float* part_ml, int B,
                              int H, int max_pages, float sm_scale, int splits, int* status, cudaStream_t stream) {
  if (B <= 0 || H <= 0 || splits < 1) return -1;
  static bool attr_set[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -6;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) return -6;
    attr_set[dev] = true;
  }
  const float scale_log2 = sm_scale * 1.4426950408889634f;
  launch_kernel(mla_decode_kernel, dim3(B, (H + 15) / 16, splits), dim3(128), size_t(kSmemBytes), stream,
                static_cast<const __nv_bfloat16*>(q), static_cast<const uint8_t*>(k_cache), static_cast<const uint8_t*>(v_cache),
                k_scale, v_scale, block_table, seq_lens, static_cast<__nv_bfloat16*>(out), part_acc, part_ml, H, max_pages,
                scale_log2, status);
  if (splits > 1)
    launch_kernel(mla_reduce_kernel, dim3(B * H), dim3(128), 0, stream, static_cast<const float*>(part_acc),
                  static_cast<const float*>(part_ml), static_cast<__nv_bfloat16*>(out), splits);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}
