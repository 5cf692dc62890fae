// Mixture-of-experts routing kernels: fused router (projection + scoring + top-k), route planning (per-expert row
// ranges + tile map for the grouped GEMM), expert-sorted gather of FP8 activation rows, and the weighted un-permute
// that adds the expert outputs back into the residual stream.
//
// Reference counterparts: moe.cu (moe_topk_kernel and its specialisations, count_experts / scan_expert_counts /
// fill_tile_experts / scatter_routes, moe_weighted_reduce*_kernel) and float_projection.cu for the router GEMV.
#include "common.cuh"

#include <cfloat>

namespace mfq {

constexpr int kMaxExperts = 512;
constexpr int kMaxTopK = 16;

struct RouterParams {
  const __nv_bfloat16* x;      // [T, H]
  const __nv_bfloat16* w;      // [E, H]
  const float* bias;           // [E] selection bias (may be null)
  int* topk_ids;               // [T, K]
  float* topk_w;               // [T, K]
  float* scores_out;           // [T, E] optional (null to skip)
  int T, H, E, K;
  int sigmoid;                 // 0: softmax over experts, 1: sigmoid
  int norm_topk;               // normalise the K selected weights to sum 1
  float scale;                 // multiplier on the final weights (routed scaling factor)
  int n_group, topk_group;     // group-limited routing (n_group <= 1: off)
  const float* logits;         // [T, E] precomputed router logits (null: this kernel computes the dot products)
};

// ---------------------------------------------------------------------------------------------
// Router logits on tensor cores: logits[t, e] = x[t, :] . w[e, :]  (bf16 in, fp32 accumulate, mma.sync m16n8k16).
// A dot product does not care about the order of its terms, so a thread loads 8 contiguous elements of a row (16 bytes)
// and feeds them to two MMAs as its k-slots; the x and w fragments use the same assignment, which keeps the result exact.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ld_row16(const __nv_bfloat16* base, int row, int rows, int H, int k) {
  return row < rows ? __ldg(reinterpret_cast<const uint4*>(base + size_t(row) * H + k)) : make_uint4(0u, 0u, 0u, 0u);
}

// Few tokens (T <= 16 * MB <= 64): one CTA per 8 experts, its 4 warps split the hidden dimension and every warp
// covers all tokens, so E / 8 CTAs stream the router matrix once.
template <int MB>
__global__ void __launch_bounds__(128) router_logits_small_kernel(const __nv_bfloat16* __restrict__ x,
                                                                  const __nv_bfloat16* __restrict__ w,
                                                                  float* __restrict__ logits, int T, int H, int E) {
  pdl_trigger();
  pdl_wait();
  __shared__ float part[4][MB * 16][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g8 = lane >> 2, c = lane & 3;
  const int e0 = blockIdx.x * 8;
  const int chunks = H / 32, per = (chunks + 3) / 4;
  const int c_lo = warp * per, c_hi = min(chunks, c_lo + per);
  float acc[MB][4];
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
  // batches of kB chunks: all loads of a batch are issued before the first MMA needs one (a warp issues in order)
  constexpr int kB = MB == 1 ? 8 : MB == 2 ? 4 : 2;
  for (int ch0 = c_lo; ch0 < c_hi; ch0 += kB) {
    uint4 b[kB], lo[kB][MB], hi[kB][MB];
#pragma unroll
    for (int u = 0; u < kB; ++u) {
      const int k = (ch0 + u) * 32 + 8 * c;
      const bool in = ch0 + u < c_hi;
      b[u] = in ? ld_row16(w, e0 + g8, E, H, k) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        lo[u][m] = in ? ld_row16(x, m * 16 + g8, T, H, k) : make_uint4(0u, 0u, 0u, 0u);
        hi[u][m] = in ? ld_row16(x, m * 16 + g8 + 8, T, H, k) : make_uint4(0u, 0u, 0u, 0u);
      }
    }
#pragma unroll
    for (int u = 0; u < kB; ++u) {
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        mma_bf16(acc[m], lo[u][m].x, hi[u][m].x, lo[u][m].y, hi[u][m].y, b[u].x, b[u].y);
        mma_bf16(acc[m], lo[u][m].z, hi[u][m].z, lo[u][m].w, hi[u][m].w, b[u].z, b[u].w);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MB; ++m) {
    part[warp][m * 16 + g8][2 * c] = acc[m][0];
    part[warp][m * 16 + g8][2 * c + 1] = acc[m][1];
    part[warp][m * 16 + g8 + 8][2 * c] = acc[m][2];
    part[warp][m * 16 + g8 + 8][2 * c + 1] = acc[m][3];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < MB * 16 * 8; i += 128) {
    const int t = i >> 3, col = i & 7;
    if (t < T && e0 + col < E) logits[size_t(t) * E + e0 + col] = part[0][t][col] + part[1][t][col] + part[2][t][col] + part[3][t][col];
  }
}

// Many tokens: a CTA computes 64 tokens x 64 experts, one warp per 16 tokens.
__global__ void __launch_bounds__(128) router_logits_tile_kernel(const __nv_bfloat16* __restrict__ x,
                                                                 const __nv_bfloat16* __restrict__ w,
                                                                 float* __restrict__ logits, int T, int H, int E) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g8 = lane >> 2, c = lane & 3;
  const int t0 = blockIdx.x * 64 + warp * 16, e0 = blockIdx.y * 64;
  float acc[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
#pragma unroll 2
  for (int k0 = 0; k0 < H; k0 += 32) {
    const int k = k0 + 8 * c;
    const uint4 lo = ld_row16(x, t0 + g8, T, H, k);
    const uint4 hi = ld_row16(x, t0 + g8 + 8, T, H, k);
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const uint4 b = ld_row16(w, e0 + n * 8 + g8, E, H, k);
      mma_bf16(acc[n], lo.x, hi.x, lo.y, hi.y, b.x, b.y);
      mma_bf16(acc[n], lo.z, hi.z, lo.w, hi.w, b.z, b.w);
    }
  }
#pragma unroll
  for (int n = 0; n < 8; ++n) {
    const int e = e0 + n * 8 + 2 * c;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int t = t0 + g8 + 8 * half;
      if (t < T) {
        if (e < E) logits[size_t(t) * E + e] = acc[n][2 * half];
        if (e + 1 < E) logits[size_t(t) * E + e + 1] = acc[n][2 * half + 1];
      }
    }
  }
}

// One CTA per token: router logits by warp-striped dot products, scoring, optional group limiting, K rounds of block
// arg-max (lowest index wins ties).
__global__ void __launch_bounds__(256) moe_router_topk_kernel(const RouterParams p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float sm[];
  float* xs = sm;                 // [H]
  float* sc = sm + p.H;           // [E] scores used for the weights
  float* sel = sc + p.E;          // [E] scores used for selection (with bias / group mask)
  __shared__ float red_v[8];
  __shared__ int red_i[8];
  __shared__ float grp[64];
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (p.logits) {
    for (int e = tid; e < p.E; e += 256) sc[e] = p.logits[size_t(t) * p.E + e];
  } else {
    for (int i = tid; i < p.H; i += 256) xs[i] = __bfloat162float(p.x[size_t(t) * p.H + i]);
  }
  __syncthreads();
  for (int e = warp; e < (p.logits ? 0 : p.E); e += 8) {
    const __nv_bfloat16* wr = p.w + size_t(e) * p.H;
    float acc = 0.f;
    for (int i = lane * 2; i < p.H; i += 64) {
      const __nv_bfloat162 w2 = *reinterpret_cast<const __nv_bfloat162*>(wr + i);
      acc = fmaf(xs[i], __bfloat162float(w2.x), acc);
      acc = fmaf(xs[i + 1], __bfloat162float(w2.y), acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) sc[e] = acc;
  }
  __syncthreads();
  if (p.sigmoid) {
    for (int e = tid; e < p.E; e += 256) sc[e] = 1.f / (1.f + __expf(-sc[e]));
  } else {
    float mx = -FLT_MAX;
    for (int e = tid; e < p.E; e += 256) mx = fmaxf(mx, sc[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red_v[warp] = mx;
    __syncthreads();
    mx = red_v[0];
    for (int i = 1; i < 8; ++i) mx = fmaxf(mx, red_v[i]);
    __syncthreads();
    float sum = 0.f;
    for (int e = tid; e < p.E; e += 256) { const float v = __expf(sc[e] - mx); sc[e] = v; sum += v; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) red_v[warp] = sum;
    __syncthreads();
    sum = 0.f;
    for (int i = 0; i < 8; ++i) sum += red_v[i];
    const float inv = 1.f / sum;
    __syncthreads();
    for (int e = tid; e < p.E; e += 256) sc[e] *= inv;
  }
  __syncthreads();
  for (int e = tid; e < p.E; e += 256) {
    sel[e] = sc[e] + (p.bias ? p.bias[e] : 0.f);
    if (p.scores_out) p.scores_out[size_t(t) * p.E + e] = sc[e];
  }
  __syncthreads();
  if (p.n_group > 1) {
    // group score = sum of the two best selection scores of the group; keep the topk_group best groups
    const int per = p.E / p.n_group;
    if (tid < p.n_group) {
      float a = -FLT_MAX, b = -FLT_MAX;
      for (int i = 0; i < per; ++i) {
        const float v = sel[tid * per + i];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      grp[tid] = a + b;
    }
    __syncthreads();
    if (tid < p.n_group) {
      int better = 0;
      for (int g = 0; g < p.n_group; ++g) better += (grp[g] > grp[tid]) || (grp[g] == grp[tid] && g < tid);
      if (better >= p.topk_group) grp[tid] = -FLT_MAX;  // dropped group
    }
    __syncthreads();
    for (int e = tid; e < p.E; e += 256)
      if (grp[e / per] == -FLT_MAX) sel[e] = -FLT_MAX;
    __syncthreads();
  }
  float wsum = 0.f;
  for (int k = 0; k < p.K; ++k) {
    float best = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int e = tid; e < p.E; e += 256) {
      const float v = sel[e];
      if (v > best || (v == best && e < bi)) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { red_v[warp] = best; red_i[warp] = bi; }
    __syncthreads();
    if (tid == 0) {
      for (int i = 1; i < 8; ++i)
        if (red_v[i] > best || (red_v[i] == best && red_i[i] < bi)) { best = red_v[i]; bi = red_i[i]; }
      p.topk_ids[size_t(t) * p.K + k] = bi;
      const float wv = sc[bi];
      p.topk_w[size_t(t) * p.K + k] = wv;
      wsum += wv;
      sel[bi] = -FLT_MAX;
    }
    __syncthreads();
  }
  if (tid == 0) {
    const float mul = (p.norm_topk ? 1.f / fmaxf(wsum, 1e-20f) : 1.f) * p.scale;
    for (int k = 0; k < p.K; ++k) p.topk_w[size_t(t) * p.K + k] *= mul;
  }
}

// Scoring and top-k with one WARP per token (logits precomputed, E <= 1024, no group limiting): a lane keeps E / 32
// scores in registers, every selection round is a register scan plus five shuffles, and nothing synchronises a block.
__global__ void __launch_bounds__(128) moe_router_topk_warp_kernel(const RouterParams p) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= p.T) return;
  constexpr int kMaxPer = 32;
  const int per = (p.E + 31) >> 5;
  float sc[kMaxPer], sel[kMaxPer];
  float mx = -FLT_MAX;
#pragma unroll
  for (int i = 0; i < kMaxPer; ++i) {
    const int e = i * 32 + lane;
    sc[i] = (i < per && e < p.E) ? p.logits[size_t(t) * p.E + e] : -FLT_MAX;
    mx = fmaxf(mx, sc[i]);
  }
  if (p.sigmoid) {
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i)
      if (i < per) sc[i] = sc[i] == -FLT_MAX ? -FLT_MAX : 1.f / (1.f + __expf(-sc[i]));
  } else {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i)
      if (i < per) {
        const float v = sc[i] == -FLT_MAX ? 0.f : __expf(sc[i] - mx);
        sc[i] = v;
        sum += v;
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i)
      if (i < per) sc[i] = (i * 32 + lane < p.E) ? sc[i] * inv : -FLT_MAX;
  }
#pragma unroll
  for (int i = 0; i < kMaxPer; ++i) {
    const int e = i * 32 + lane;
    const bool live = i < per && e < p.E;
    sel[i] = live ? sc[i] + (p.bias ? p.bias[e] : 0.f) : -FLT_MAX;
    if (live && p.scores_out) p.scores_out[size_t(t) * p.E + e] = sc[i];
  }
  float wsum = 0.f, my_w = 0.f;
  int my_id = 0;
  for (int k = 0; k < p.K; ++k) {
    float best = -FLT_MAX, best_w = 0.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i)
      if (i < per && sel[i] > best) { best = sel[i]; bi = i * 32 + lane; best_w = sc[i]; }  // ascending i: lowest index wins ties
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o), ow = __shfl_xor_sync(0xffffffffu, best_w, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; best_w = ow; }
    }
    if (lane == k) { my_id = bi; my_w = best_w; }
    wsum += best_w;
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i)
      if (i == (bi >> 5) && lane == (bi & 31)) sel[i] = -FLT_MAX;
  }
  if (lane < p.K) {
    const float mul = (p.norm_topk ? 1.f / fmaxf(wsum, 1e-20f) : 1.f) * p.scale;
    p.topk_ids[size_t(t) * p.K + lane] = my_id;
    p.topk_w[size_t(t) * p.K + lane] = my_w * mul;
  }
}

// Route plan for the experts [e_lo, e_hi) owned by this rank (one CTA).  Row order inside an expert depends on atomic
// arrival order; results do not, because each row is computed independently and the un-permute sums a token's K
// contributions in slot order.
//   offsets[e - e_lo]   first sorted row of local expert e (offsets[n_local] = total rows)
//   dest[t*K + k]       sorted row of that (token, slot) pair, -1 if its expert lives on another rank
//   src_token[row]      token of the sorted row
//   tile_map[i]         (local expert, token tile inside it) for the grouped GEMM; padded with (-1, -1)
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ topk_ids, int entries, int K, int e_lo,
                                                        int e_hi, int token_tile, int* __restrict__ offsets,
                                                        int* __restrict__ dest, int* __restrict__ src_token,
                                                        int2* __restrict__ tile_map, int map_cap,
                                                        int* __restrict__ totals) {
  pdl_trigger();
  pdl_wait();
  __shared__ int cnt[kMaxExperts + 1];
  __shared__ int fill[kMaxExperts];
  __shared__ int tbase[kMaxExperts + 1];
  const int n_local = e_hi - e_lo;
  for (int e = threadIdx.x; e <= n_local; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int e = topk_ids[i] - e_lo;
    if (e >= 0 && e < n_local) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  {
    // exclusive prefix sums of the per-expert row and tile counts: one expert per thread, warp scans, then a scan of
    // the 32 warp totals (the block has 1024 threads and at most 512 experts)
    __shared__ int wrow[32], wtile[32];
    const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
    const int c = e < n_local ? cnt[e] : 0;
    const int tl = (c + token_tile - 1) / token_tile;
    int ir = c, it = tl;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int ur = __shfl_up_sync(0xffffffffu, ir, o), ut = __shfl_up_sync(0xffffffffu, it, o);
      if (lane >= o) { ir += ur; it += ut; }
    }
    if (lane == 31) { wrow[warp] = ir; wtile[warp] = it; }
    __syncthreads();
    if (warp == 0) {
      int vr = wrow[lane], vt = wtile[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int ur = __shfl_up_sync(0xffffffffu, vr, o), ut = __shfl_up_sync(0xffffffffu, vt, o);
        if (lane >= o) { vr += ur; vt += ut; }
      }
      wrow[lane] = vr;
      wtile[lane] = vt;
    }
    __syncthreads();
    const int base_r = warp ? wrow[warp - 1] : 0, base_t = warp ? wtile[warp - 1] : 0;
    if (e < n_local) {
      offsets[e] = base_r + ir - c;
      fill[e] = base_r + ir - c;
      tbase[e] = base_t + it - tl;
    }
    if (e == n_local) {  // totals: everything before this (empty) slot
      offsets[n_local] = base_r + ir;
      tbase[n_local] = base_t + it;
      totals[0] = base_r + ir;
      totals[1] = base_t + it;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int e = topk_ids[i] - e_lo;
    int row = -1;
    if (e >= 0 && e < n_local) {
      row = atomicAdd(&fill[e], 1);
      src_token[row] = i / K;
    }
    dest[i] = row;
  }
  for (int e = threadIdx.x; e < n_local; e += blockDim.x) {
    const int n = tbase[e + 1] - tbase[e];
    for (int j = 0; j < n; ++j)
      if (tbase[e] + j < map_cap) tile_map[tbase[e] + j] = make_int2(e, j);
  }
  __syncthreads();
  for (int i = tbase[n_local] + threadIdx.x; i < map_cap; i += blockDim.x) tile_map[i] = make_int2(-1, -1);
}

// Expert-sorted copy of already quantized activation rows: xq_sorted[row] = xq[src_token[row]] (+ its multiplier).
__global__ void moe_gather_rows_kernel(const uint8_t* __restrict__ xq, const float* __restrict__ xs,
                                       const int* __restrict__ src_token, const int* __restrict__ totals,
                                       uint8_t* __restrict__ out_q, float* __restrict__ out_s, int H) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  if (row >= totals[0]) return;
  const int t = src_token[row];
  const uint4* src = reinterpret_cast<const uint4*>(xq + size_t(t) * H);
  uint4* dst = reinterpret_cast<uint4*>(out_q + size_t(row) * H);
  for (int i = threadIdx.x; i < H / 16; i += blockDim.x) dst[i] = src[i];
  if (threadIdx.x == 0) out_s[row] = xs[t];
}

// out[t] = base[t] (+ extra[t]) + sum_k w[t,k] * y[dest[t,k]]   (rows with dest < 0 are skipped)
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ dest,
                                   const float* __restrict__ topk_w, const __nv_bfloat16* __restrict__ base,
                                   const __nv_bfloat16* __restrict__ extra, __nv_bfloat16* __restrict__ out, int H,
                                   int K) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (base) {
      const uint4 b = *reinterpret_cast<const uint4*>(base + size_t(t) * H + v * 8);
      const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(&b);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = __bfloat162float(bb[j]);
    }
    if (extra) {
      const uint4 b = *reinterpret_cast<const uint4*>(extra + size_t(t) * H + v * 8);
      const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(&b);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(bb[j]);
    }
    for (int k = 0; k < K; ++k) {
      const int row = dest[size_t(t) * K + k];
      if (row < 0) continue;
      const float w = topk_w[size_t(t) * K + k];
      const uint4 b = *reinterpret_cast<const uint4*>(y + size_t(row) * H + v * 8);
      const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(&b);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(w, __bfloat162float(bb[j]), acc[j]);
    }
    uint4 o;
    __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) ob[j] = __float2bfloat16(acc[j]);
    *reinterpret_cast<uint4*>(out + size_t(t) * H + v * 8) = o;
  }
}

}  // namespace mfq

using namespace mfq;

// ``logits``: optional [T, E] fp32 scratch.  With it (and H a multiple of 32) the dot products run on tensor cores
// spread over the whole GPU and the per-token CTAs only score and select; without it one CTA per token does everything.
extern "C" int mfq_moe_router_topk(const void* x, const void* w, const float* bias, int* topk_ids, float* topk_w,
                                   float* scores_out, float* logits, int T, int H, int E, int K, int sigmoid, int norm_topk,
                                   float scale, int n_group, int topk_group, cudaStream_t stream) {
  if (T <= 0 || E > kMaxExperts || K > kMaxTopK || K > E || H % 2 || n_group > 64 || (n_group > 1 && E % n_group)) return -1;
  const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wb = static_cast<const __nv_bfloat16*>(w);
  if (logits && H % 32 == 0) {
    const int eb = (E + 7) / 8;
    if (T <= 16) launch_kernel(router_logits_small_kernel<1>, dim3(eb), dim3(128), 0, stream, xb, wb, logits, T, H, E);
    else if (T <= 32) launch_kernel(router_logits_small_kernel<2>, dim3(eb), dim3(128), 0, stream, xb, wb, logits, T, H, E);
    else if (T <= 64) launch_kernel(router_logits_small_kernel<4>, dim3(eb), dim3(128), 0, stream, xb, wb, logits, T, H, E);
    else launch_kernel(router_logits_tile_kernel, dim3((T + 63) / 64, (E + 63) / 64), dim3(128), 0, stream, xb, wb, logits, T, H, E);
    if (cudaGetLastError() != cudaSuccess) return -7;
  } else {
    logits = nullptr;
  }
  RouterParams p{xb, wb, bias, topk_ids, topk_w, scores_out, T, H, E, K, sigmoid, norm_topk, scale, n_group, topk_group, logits};
  if (logits && n_group <= 1 && E <= 1024 && K <= 32) {
    launch_kernel(moe_router_topk_warp_kernel, dim3((T + 3) / 4), dim3(128), 0, stream, p);
    return cudaGetLastError() == cudaSuccess ? 0 : -7;
  }
  const size_t smem = size_t(H + 2 * E) * sizeof(float);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    if (cudaFuncSetAttribute(moe_router_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return -6;
    configured = smem;
  }
  launch_kernel(moe_router_topk_kernel, dim3(T), dim3(256), smem, stream, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

extern "C" int mfq_moe_plan(const int* topk_ids, int T, int K, int e_lo, int e_hi, int token_tile, int* offsets, int* dest,
                            int* src_token, void* tile_map, int map_cap, int* totals, cudaStream_t stream) {
  if (e_hi - e_lo > kMaxExperts || e_hi <= e_lo || T <= 0) return -1;
  launch_kernel(moe_plan_kernel, dim3(1), dim3(1024), 0, stream, topk_ids, T * K, K, e_lo, e_hi, token_tile, offsets, dest, src_token,
                                          static_cast<int2*>(tile_map), map_cap, totals);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

extern "C" int mfq_moe_gather_rows(const void* xq, const float* xs, const int* src_token, const int* totals, void* out_q,
                                   float* out_s, int max_rows, int H, cudaStream_t stream) {
  if (H % 16 || max_rows <= 0) return -1;
  launch_kernel(moe_gather_rows_kernel, dim3(max_rows), dim3(128), 0, stream, static_cast<const uint8_t*>(xq), xs, src_token, totals,
                                                       static_cast<uint8_t*>(out_q), out_s, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

extern "C" int mfq_moe_combine(const void* y, const int* dest, const float* topk_w, const void* base, const void* extra,
                               void* out, int T, int H, int K, cudaStream_t stream) {
  if (H % 8 || T <= 0) return -1;
  launch_kernel(moe_combine_kernel, dim3(T), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(y), dest, topk_w,
                                            static_cast<const __nv_bfloat16*>(base),
                                            static_cast<const __nv_bfloat16*>(extra), static_cast<__nv_bfloat16*>(out), H, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}
