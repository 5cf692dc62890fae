// Weight-streaming block-scaled FP8 GEMV / skinny GEMM for 1..64 token rows (single-stream decode, speculative
// verify windows, the per-expert tiles of a decode-sized MoE step, and -- with 32 or 64 rows -- the small per-rank
// projections of a tensor-parallel decode step, where a tcgen05 pipeline would spend longer filling than working).
//
// With this few rows the product is pure weight streaming and what counts is latency: no tensor maps, no TMEM, no
// pipeline to fill.  A CTA owns 16 output rows; its eight warps split the K range by 128-wide blocks.  A thread reads
// 16 contiguous bytes of a weight row straight from global memory and feeds them to two
// `mma.sync.m16n8k32.e4m3` as its k-slots; the activation fragment uses the same slot assignment, so every
// 64-byte chunk contributes its exact dot product (fp32 accumulate).  Each 128-wide block is accumulated on its own
// and folded with that block's fp32 weight multiplier; the row multiplier of the activations is applied at the end,
// the warps' partial sums meet in shared memory, the residual is added and bf16 rows are written.
// The weight slice of a warp is prefetched into L2 before the grid dependency wait, so under programmatic dependent
// launch it streams in while the previous kernel drains.
//
// The reference's counterparts are its scalar small-M kernels (mfq/kernels/cuda: mxfp8_small_m_kernel,
// nint_matmul_kernel and the sq_mmq family).
#include "common.cuh"

namespace mfq {

__device__ __forceinline__ void mma_e4m3(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct GemvParams {
  const uint8_t* w;        // [experts][N][K] E4M3
  const float* w_scale;    // [experts][ceil(N/128)][K/128]
  const uint8_t* x;        // [rows][K] E4M3
  const float* x_scale;    // [rows]
  __nv_bfloat16* out;      // [rows][N]
  const __nv_bfloat16* residual;  // [rows][N] or null
  int M, N, K;
  const int2* tile_map;    // grouped: (expert, 16-row tile inside the expert) per blockIdx.y; (-1, -1) pads
  const int* offsets;      // grouped: first sorted row of every expert (+ total)
  const int* src_token;    // grouped, optional: sorted row -> row of x / x_scale (the gather is folded into the loads)
};

constexpr int kWarps = 8;  // K-split inside a CTA

// NB: 8-token column blocks per CTA, 1 (<= 8 rows) or 2 (<= 16 rows).  RG: 16-row groups of the weight matrix per CTA;
// the kWarps / RG warps of a group split K.  Expert tiles use RG = 2: a CTA's life is a chain of dependent loads
// (tile map, offsets, weights), so it has to carry enough bytes to be worth that latency.
template <int NB, int RG>
__global__ void __launch_bounds__(kWarps * 32, (NB <= 2 ? 2 : 1)) fp8_gemv_kernel(const GemvParams p) {
  pdl_trigger();
  constexpr int kSplit = kWarps / RG;
  __shared__ float part[kWarps][16][NB * 8];
  const int lane = threadIdx.x & 31, g8 = lane >> 2, c = lane & 3;
  const int rg = (threadIdx.x >> 5) / kSplit, warp = (threadIdx.x >> 5) % kSplit;  // warp: index inside the K split
  const int n0 = (blockIdx.x * RG + rg) * 16;
  const int kblocks = p.K >> 7;
  const uint8_t* w = p.w;
  const float* wsc = p.w_scale;
  int row0 = 0, rows = p.M;
  const int nblocks128 = (p.N + 127) >> 7;

  // this warp's weight slice -> L2, before the dependency wait (weights never depend on the previous kernel)
  if (!p.tile_map) {
    const uint8_t* base = w + size_t(n0) * p.K;
    for (int kb = warp; kb < kblocks; kb += kSplit)
      if (lane < 16) asm volatile("prefetch.global.L2 [%0];" ::"l"(base + size_t(lane) * p.K + kb * 128));
  }
  pdl_wait();
  if (p.tile_map) {
    const int2 tm = p.tile_map[blockIdx.y];
    if (tm.x < 0) return;
    const int lo = p.offsets[tm.x] + tm.y * (NB * 8);
    row0 = lo;
    rows = min(NB * 8, p.offsets[tm.x + 1] - lo);
    w += size_t(tm.x) * p.N * p.K;
    wsc += size_t(tm.x) * nblocks128 * kblocks;
  }
  const uint8_t* w_lo = w + size_t(n0 + g8) * p.K + 16 * c;
  const uint8_t* w_hi = w_lo + size_t(8) * p.K;
  const float* ws_row = wsc + size_t(n0 >> 7) * kblocks;
  const uint8_t* xr[NB];
  bool live[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    live[nb] = nb * 8 + g8 < rows;
    int xrow = row0 + nb * 8 + g8;
    if (p.src_token && live[nb]) xrow = p.src_token[xrow];
    xr[nb] = p.x + size_t(xrow) * p.K + 16 * c;
  }

  float acc[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.f;
  // Batches of kBatch k-blocks: every weight load of a batch is issued before the first MMA consumes one, so a warp
  // keeps kBatch * 2 KB in flight (a warp issues in order; interleaving loads and MMAs would expose the DRAM latency
  // once per k-block).
  constexpr int kBatch = 4;
  for (int kb0 = warp; kb0 < kblocks; kb0 += kSplit * kBatch) {
    uint4 a_lo0[kBatch], a_hi0[kBatch], a_lo1[kBatch], a_hi1[kBatch];
    float wscale[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int kb = kb0 + u * kSplit;
      if (kb < kblocks) {
        const int k = kb * 128;
        a_lo0[u] = __ldg(reinterpret_cast<const uint4*>(w_lo + k));
        a_hi0[u] = __ldg(reinterpret_cast<const uint4*>(w_hi + k));
        a_lo1[u] = __ldg(reinterpret_cast<const uint4*>(w_lo + k + 64));
        a_hi1[u] = __ldg(reinterpret_cast<const uint4*>(w_hi + k + 64));
        wscale[u] = __ldg(ws_row + kb);
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int kb = kb0 + u * kSplit;
      if (kb < kblocks) {
        const int k = kb * 128;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          uint4 b0 = make_uint4(0u, 0u, 0u, 0u), b1 = b0;
          if (live[nb]) {
            b0 = *reinterpret_cast<const uint4*>(xr[nb] + k);
            b1 = *reinterpret_cast<const uint4*>(xr[nb] + k + 64);
          }
          float blk[4] = {0.f, 0.f, 0.f, 0.f};
          mma_e4m3(blk, a_lo0[u].x, a_hi0[u].x, a_lo0[u].y, a_hi0[u].y, b0.x, b0.y);
          mma_e4m3(blk, a_lo0[u].z, a_hi0[u].z, a_lo0[u].w, a_hi0[u].w, b0.z, b0.w);
          mma_e4m3(blk, a_lo1[u].x, a_hi1[u].x, a_lo1[u].y, a_hi1[u].y, b1.x, b1.y);
          mma_e4m3(blk, a_lo1[u].z, a_hi1[u].z, a_lo1[u].w, a_hi1[u].w, b1.z, b1.w);
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[nb][e] = fmaf(blk[e], wscale[u], acc[nb][e]);
        }
      }
    }
  }
  float (*mine)[NB * 8] = part[rg * kSplit + warp];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    mine[g8][nb * 8 + 2 * c] = acc[nb][0];
    mine[g8][nb * 8 + 2 * c + 1] = acc[nb][1];
    mine[g8 + 8][nb * 8 + 2 * c] = acc[nb][2];
    mine[g8 + 8][nb * 8 + 2 * c + 1] = acc[nb][3];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < RG * 16 * NB * 8; i += kWarps * 32) {
    const int grp = i / (16 * NB * 8), j = i % (16 * NB * 8);
    const int tok = j >> 4, r = j & 15;  // consecutive threads -> consecutive output columns of one token
    if (tok >= rows) continue;
    float v = 0.f;
#pragma unroll
    for (int wp = 0; wp < kSplit; ++wp) v += part[grp * kSplit + wp][r][tok];
    v *= p.x_scale[p.src_token ? p.src_token[row0 + tok] : row0 + tok];
    const size_t o = size_t(row0 + tok) * p.N + (blockIdx.x * RG + grp) * 16 + r;
    if (p.residual) v += __bfloat162float(p.residual[o]);
    p.out[o] = __float2bfloat16(v);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// The same product for up to 4 token rows with the ACTIVATION PREPARATION folded in: the rows arrive as bf16 and every
// CTA first rebuilds their FP8 form in shared memory -- RMSNorm + quantization (mode 0), plain quantization (mode 1) or
// SiLU(gate) * up + quantization (mode 2) -- exactly as the standalone kernels would have (same per-element arithmetic,
// and for the sum of squares the same summation tree: the standalone norm kernel's thread layout is emulated, so both
// paths produce the same bits).  With one row a decode step is a chain of some 350 tiny dependent kernels and each
// costs a few microseconds of hand-over whatever it computes; this removes four of the eleven per layer.  Recomputing a
// 4096- or 14336-wide row in each of a few hundred CTAs costs L2 reads that run under the weight prefetch.
// ---------------------------------------------------------------------------------------------------------------------
struct GemvActParams {
  const uint8_t* w;
  const float* w_scale;
  const __nv_bfloat16* x;        // [M][x_stride] bf16 (mode 2: gate | up, each K wide)
  const __nv_bfloat16* norm_w;   // [K] (mode 0)
  __nv_bfloat16* out;
  const __nv_bfloat16* residual;
  float eps;
  int M, N, K, x_stride;
  int norm_threads;              // block size the standalone norm kernel would use for this K
};

constexpr int kActMaxRows = 4;

__device__ __forceinline__ float act_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float act_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ uint8_t act_to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

template <int kMode>
__global__ void __launch_bounds__(kWarps * 32, 2) fp8_gemv_act_kernel(const GemvActParams p) {
  pdl_trigger();
  extern __shared__ __align__(16) uint8_t act_smem[];   // [M][K] E4M3
  __shared__ float part[kWarps][16][8];
  __shared__ float red[34];
  __shared__ float row_scale[kActMaxRows];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, g8 = lane >> 2, c = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int kblocks = p.K >> 7;
  {
    const uint8_t* base = p.w + size_t(n0) * p.K;
    for (int kb = wid; kb < kblocks; kb += kWarps)
      if (lane < 16) asm volatile("prefetch.global.L2 [%0];" ::"l"(base + size_t(lane) * p.K + kb * 128));
  }
  // The first batch of this warp's weight loads is issued BEFORE the dependency wait as well, into registers: its DRAM / L2
  // round trip then runs under the wait and under the activation preparation instead of after them.
  const uint8_t* w_lo = p.w + size_t(n0 + g8) * p.K + 16 * c;
  const uint8_t* w_hi = w_lo + size_t(8) * p.K;
  const float* ws_row = p.w_scale + size_t(n0 >> 7) * kblocks;
  constexpr int kBatch = 4;
  uint4 a_lo0[kBatch], a_hi0[kBatch], a_lo1[kBatch], a_hi1[kBatch];
  float wscale[kBatch];
  auto load_batch = [&](int kb0) {
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int kb = kb0 + u * kWarps;
      if (kb < kblocks) {
        const int k = kb * 128;
        a_lo0[u] = __ldg(reinterpret_cast<const uint4*>(w_lo + k));
        a_hi0[u] = __ldg(reinterpret_cast<const uint4*>(w_hi + k));
        a_lo1[u] = __ldg(reinterpret_cast<const uint4*>(w_lo + k + 64));
        a_hi1[u] = __ldg(reinterpret_cast<const uint4*>(w_hi + k + 64));
        wscale[u] = __ldg(ws_row + kb);
      }
    }
  };
  load_batch(wid);
  pdl_wait();
  const int nvec = p.K >> 3;
  // one element vector of the prepared (pre-quantization) row, as the standalone kernels compute it
  auto value = [&](const __nv_bfloat16* xr, int vi, float rstd, float (&y)[8]) {
    const uint4 a = *reinterpret_cast<const uint4*>(xr + vi * 8);
    const __nv_bfloat16* ab = reinterpret_cast<const __nv_bfloat16*>(&a);
    if (kMode == 0) {
      const uint4 ww = *reinterpret_cast<const uint4*>(p.norm_w + vi * 8);
      const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(&ww);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        y[j] = __bfloat162float(__float2bfloat16(__bfloat162float(ab[j]) * rstd * __bfloat162float(wb[j])));
    } else if (kMode == 1) {
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = __bfloat162float(ab[j]);
    } else {
      const uint4 b = *reinterpret_cast<const uint4*>(xr + p.K + vi * 8);
      const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(&b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float g = __bfloat162float(ab[j]);
        y[j] = __bfloat162float(__float2bfloat16(g / (1.f + __expf(-g)) * __bfloat162float(bb[j])));
      }
    }
  };
  for (int m = 0; m < p.M; ++m) {
    const __nv_bfloat16* xr = p.x + size_t(m) * p.x_stride;
    float rstd = 1.f;
    if (kMode == 0) {
      // sum of squares in the standalone kernel's order: "virtual" thread vt of a block of norm_threads owns the
      // vectors vt, vt + norm_threads, ...; its warp sums by shuffle, lane 0 of warp 0 sums the warps.  This block has
      // 256 threads and plays the virtual threads tid and tid + 256.
      const int VT = p.norm_threads, nw = VT >> 5;
      float ss[2] = {0.f, 0.f};
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int vt = tid + 256 * u;
        if (vt < VT) {
          for (int vi = vt; vi < nvec; vi += VT) {
            const uint4 a = *reinterpret_cast<const uint4*>(xr + vi * 8);
            const __nv_bfloat16* ab = reinterpret_cast<const __nv_bfloat16*>(&a);
#pragma unroll
            for (int j = 0; j < 8; ++j) { const float v = __bfloat162float(ab[j]); ss[u] += v * v; }
          }
        }
      }
      const float s0 = act_warp_sum(ss[0]), s1 = act_warp_sum(ss[1]);
      __syncthreads();
      if (lane == 0) { red[wid] = s0; if (wid + 8 < nw) red[wid + 8] = s1; }
      __syncthreads();
      if (wid == 0) {
        float x = lane < nw ? red[lane] : 0.f;
        x = act_warp_sum(x);
        if (lane == 0) red[32] = x;
      }
      __syncthreads();
      rstd = rsqrtf(red[32] / float(p.K) + p.eps);
    }
    float amax = 0.f;
    for (int vi = tid; vi < nvec; vi += kWarps * 32) {
      float y[8];
      value(xr, vi, rstd, y);
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(y[j]));
    }
    amax = act_warp_max(amax);
    __syncthreads();
    if (lane == 0) red[wid] = amax;
    __syncthreads();
    if (wid == 0) {
      float x = lane < kWarps ? red[lane] : 0.f;
      x = act_warp_max(x);
      if (lane == 0) red[33] = x;
    }
    __syncthreads();
    const float scale = fmaxf(red[33], 1e-12f) / 448.f, inv = 1.f / scale;
    if (tid == 0) row_scale[m] = scale;
    uint8_t* qrow = act_smem + size_t(m) * p.K;
    for (int vi = tid; vi < nvec; vi += kWarps * 32) {
      float y[8];
      value(xr, vi, rstd, y);
      uint2 o;
      uint8_t* ob = reinterpret_cast<uint8_t*>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j) ob[j] = act_to_e4m3(y[j] * inv);
      *reinterpret_cast<uint2*>(qrow + vi * 8) = o;
    }
  }
  __syncthreads();

  // ---- the product, as in fp8_gemv_kernel<1, 1>, the activation fragments coming from shared memory ----
  const bool live = g8 < p.M;
  const uint8_t* xq = act_smem + size_t(live ? g8 : 0) * p.K + 16 * c;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int kb0 = wid; kb0 < kblocks; kb0 += kWarps * kBatch) {
    if (kb0 != wid) load_batch(kb0);
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int kb = kb0 + u * kWarps;
      if (kb < kblocks) {
        const int k = kb * 128;
        uint4 b0 = make_uint4(0u, 0u, 0u, 0u), b1 = b0;
        if (live) {
          b0 = *reinterpret_cast<const uint4*>(xq + k);
          b1 = *reinterpret_cast<const uint4*>(xq + k + 64);
        }
        float blk[4] = {0.f, 0.f, 0.f, 0.f};
        mma_e4m3(blk, a_lo0[u].x, a_hi0[u].x, a_lo0[u].y, a_hi0[u].y, b0.x, b0.y);
        mma_e4m3(blk, a_lo0[u].z, a_hi0[u].z, a_lo0[u].w, a_hi0[u].w, b0.z, b0.w);
        mma_e4m3(blk, a_lo1[u].x, a_hi1[u].x, a_lo1[u].y, a_hi1[u].y, b1.x, b1.y);
        mma_e4m3(blk, a_lo1[u].z, a_hi1[u].z, a_lo1[u].w, a_hi1[u].w, b1.z, b1.w);
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = fmaf(blk[e], wscale[u], acc[e]);
      }
    }
  }
  part[wid][g8][2 * c] = acc[0];
  part[wid][g8][2 * c + 1] = acc[1];
  part[wid][g8 + 8][2 * c] = acc[2];
  part[wid][g8 + 8][2 * c + 1] = acc[3];
  __syncthreads();
  for (int i = tid; i < 16 * 8; i += kWarps * 32) {
    const int tok = i >> 4, r = i & 15;
    if (tok >= p.M) continue;
    float v = 0.f;
#pragma unroll
    for (int wp = 0; wp < kWarps; ++wp) v += part[wp][r][tok];
    v *= row_scale[tok];
    const size_t o = size_t(tok) * p.N + n0 + r;
    if (p.residual) v += __bfloat162float(p.residual[o]);
    p.out[o] = __float2bfloat16(v);
  }
}

static int launch_gemv(const GemvParams& p, int tiles, int nb, cudaStream_t stream) {
  if (p.tile_map && p.N % 32 == 0) {
    launch_kernel(fp8_gemv_kernel<2, 2>, dim3(p.N / 32, tiles), dim3(kWarps * 32), 0, stream, p);
  } else {
    const dim3 grid(p.N / 16, tiles);
    if (nb == 1) launch_kernel(fp8_gemv_kernel<1, 1>, grid, dim3(kWarps * 32), 0, stream, p);
    else if (nb == 2) launch_kernel(fp8_gemv_kernel<2, 1>, grid, dim3(kWarps * 32), 0, stream, p);
    else if (nb <= 4) launch_kernel(fp8_gemv_kernel<4, 1>, grid, dim3(kWarps * 32), 0, stream, p);
    else launch_kernel(fp8_gemv_kernel<8, 1>, grid, dim3(kWarps * 32), 0, stream, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

}  // namespace mfq

// out[M, N] = x_scale[m] * sum over 128-blocks of w_scale * (x_q . w_q) (+ residual), M <= 64, N % 16 == 0, K % 128 == 0.
extern "C" int mfq_fp8_gemv(const void* w, const float* w_scale, const void* x, const float* x_scale, void* out,
                            const void* residual, int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || M > 64 || N % 16 || K % 128 || N <= 0) return -1;
  mfq::GemvParams p{static_cast<const uint8_t*>(w), w_scale, static_cast<const uint8_t*>(x), x_scale,
                    static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(residual), M, N, K, nullptr, nullptr, nullptr};
  return mfq::launch_gemv(p, 1, (M + 7) / 8, stream);
}

// Grouped form for expert-sorted rows: tile_map entries are (expert, 16-row tile) as the route plan writes them with a
// token tile of 16; expert e owns rows [offsets[e], offsets[e + 1]).
// src_token (optional): x / x_scale are the UNSORTED token rows and sorted row r reads row src_token[r].
extern "C" int mfq_fp8_gemv_grouped(const void* w, const float* w_scale, const void* x, const float* x_scale, void* out,
                                    int N, int K, const void* tile_map, int map_cap, const int* offsets,
                                    const int* src_token, cudaStream_t stream) {
  if (N % 16 || K % 128 || N <= 0 || map_cap <= 0) return -1;
  mfq::GemvParams p{static_cast<const uint8_t*>(w), w_scale, static_cast<const uint8_t*>(x), x_scale,
                    static_cast<__nv_bfloat16*>(out), nullptr, 0, N, K, static_cast<const int2*>(tile_map), offsets, src_token};
  return mfq::launch_gemv(p, map_cap, 2, stream);
}

// The product with the activation preparation folded in (see fp8_gemv_act_kernel).  mode 0: out = W . quant(rmsnorm(x) *
// norm_w); 1: W . quant(x); 2: W . quant(silu(x[:, :K]) * x[:, K:2K]).  M <= 4, K % 128 == 0, N % 16 == 0.
extern "C" int mfq_fp8_gemv_act(const void* w, const float* w_scale, const void* x, int x_stride, const void* norm_w, float eps,
                                void* out, const void* residual, int M, int N, int K, int mode, cudaStream_t stream) {
  if (M <= 0 || M > mfq::kActMaxRows || N % 16 || K % 128 || N <= 0 || mode < 0 || mode > 2 || x_stride % 8) return -1;
  if (mode == 0 && !norm_w) return -1;
  const int nvec = K / 8;
  int threads = ((nvec + 7) / 8 + 31) / 32 * 32;      // the block size mfq_rmsnorm_quant picks for few rows
  if (threads < 32) threads = 32;
  const int wide = (nvec + 31) / 32 * 32;
  threads = threads > (wide < 512 ? wide : 512) ? threads : (wide < 512 ? wide : 512);
  if (threads > 512) return -1;                        // more than two virtual threads per thread are not emulated
  mfq::GemvActParams p{static_cast<const uint8_t*>(w), w_scale, static_cast<const __nv_bfloat16*>(x),
                       static_cast<const __nv_bfloat16*>(norm_w), static_cast<__nv_bfloat16*>(out),
                       static_cast<const __nv_bfloat16*>(residual), eps, M, N, K, x_stride, threads};
  const size_t smem = size_t(M) * K;
  auto launch = [&](auto kernel) -> int {
    static bool attr[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -6;
    if (!attr[dev]) {
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mfq::kActMaxRows * 16384) != cudaSuccess) return -6;
      attr[dev] = true;
    }
    mfq::launch_kernel(kernel, dim3(N / 16), dim3(mfq::kWarps * 32), smem, stream, p);
    return cudaGetLastError() == cudaSuccess ? 0 : -7;
  };
  if (K > 16384) return -1;
  if (mode == 0) return launch(mfq::fp8_gemv_act_kernel<0>);
  if (mode == 1) return launch(mfq::fp8_gemv_act_kernel<1>);
  return launch(mfq::fp8_gemv_act_kernel<2>);
}
