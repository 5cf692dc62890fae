// Paged GQA decode / verify attention over FP8 pages, built to run at HBM speed.
//
// One CTA = (sequence, KV head, KV split); its 4 warps take pages round-robin.  Every warp owns a private
// ring of page buffers in shared memory that it fills with bulk async copies (one 2 KB K block, one 2 KB V
// block and two 64 B scale rows per page and head; completion on an mbarrier), so dozens of KB are in flight
// per SM without any CTA-wide synchronisation.  The math is tensor-core `mma.sync.m16n8k16` in f16 with fp32
// accumulation: the 16 MMA rows hold the (query row, head-of-group) pairs that share this KV head -- G heads
// x q_len query tokens <= 16 -- so a 4-head group or a 4-token speculative verify window costs the same KV
// traffic as one head.  FP8 codes are expanded to f16 with `cvt.f16x2.e4m3x2` straight into MMA fragments.
//
// The page layout is chosen so that fragments are single shared-memory loads:
//   K page (per head):  [D/64 chunks][16 tokens][64 dims]  -> thread (token, c) reads 16 B = the B fragments of
//                        four k-steps; the MMA k index is a dummy, so Q is loaded with the matching dim order.
//   V page (per head):  [D dims][16 tokens, order 0,1,8,9,2,3,10,11,...] -> thread (dim, c) reads 4 B = tokens
//                        {2c, 2c+1, 2c+8, 2c+9}, the B fragment of the P.V MMA.
//
// The reference's paged decode kernels (mfq/kernels/cuda/paged_kv.cu: paged_attention_decode_kernel and the
// split/reduce variants) are scalar FMA kernels over fp16/bf16/fp32 pages.
#include "common.cuh"

#include <cfloat>
#include <cuda_fp16.h>

namespace mfq {

constexpr float kNeg = -1e30f;

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint16_t v) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
  return r;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int D, int kAttnStages>
struct AttnSmem {
  static constexpr int kPageBytes = 16 * D;                    // one head's K (or V) page
  static constexpr int kStageBytes = 2 * kPageBytes + 128;     // K, V, k scales, v scales
  static constexpr int kWarpBytes = kAttnStages * kStageBytes;  // also the merge scratch: needs >= 16*D*4 + 128
  static constexpr int kTotal = 4 * kWarpBytes + 4 * kAttnStages * 8 + 16;
};

// kAttnStages: pages in flight per warp; kMinBlocks: CTAs per SM the register allocation is held to.
template <int D, int kAttnStages, int kMinBlocks>
__global__ void __launch_bounds__(128, kMinBlocks)
paged_attn_decode_mma_kernel(const __nv_bfloat16* __restrict__ q, const uint8_t* __restrict__ k_cache,
                             const uint8_t* __restrict__ v_cache, const float* __restrict__ k_scale,
                             const float* __restrict__ v_scale, const int* __restrict__ block_table,
                             const int* __restrict__ seq_lens, __nv_bfloat16* __restrict__ out,
                             float* __restrict__ part_acc, float* __restrict__ part_ml, int Hq, int Hk, int max_pages,
                             float scale_log2, int q_len, int* status) {
  pdl_trigger();
  pdl_wait();
  using L = AttnSmem<D, kAttnStages>;
  constexpr int KSTEPS = D / 16, NBD = D / 8;
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g8 = lane >> 2, c = lane & 3;
  uint8_t* ring = smem + warp * L::kWarpBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 4 * L::kWarpBytes) + warp * kAttnStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 4 * L::kWarpBytes + 4 * kAttnStages * 8);

  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z, nsplit = gridDim.z;
  const int G = Hq / Hk;
  const int R = G * q_len;  // live MMA rows
  const int len = seq_lens[seq];
  const int pages_total = (len + 15) >> 4;
  const int per_split = (pages_total + nsplit - 1) / nsplit;
  const int page_begin = split * per_split;
  const int page_end = min(pages_total, page_begin + per_split);
  const int my_pages = page_end > page_begin + warp ? (page_end - page_begin - warp + 3) / 4 : 0;

  if (threadIdx.x == 0) *abort_flag = 0;
  if (lane == 0) {
    for (int s = 0; s < kAttnStages; ++s) mbar_init(&bars[s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  const int* bt = block_table + size_t(seq) * max_pages;
  auto issue = [&](int i) {  // lane 0 only: start the copies of this warp's i-th page
    const int s = i % kAttnStages;
    const int page = bt[page_begin + warp + 4 * i];
    const size_t ph = size_t(page) * Hk + kvh;
    uint8_t* st = ring + s * L::kStageBytes;
    mbar_expect_tx(&bars[s], L::kStageBytes);
    bulk_load(st, k_cache + ph * L::kPageBytes, L::kPageBytes, &bars[s]);
    bulk_load(st + L::kPageBytes, v_cache + ph * L::kPageBytes, L::kPageBytes, &bars[s]);
    bulk_load(st + 2 * L::kPageBytes, k_scale + ph * 16, 64, &bars[s]);
    bulk_load(st + 2 * L::kPageBytes + 64, v_scale + ph * 16, 64, &bars[s]);
  };
  if (lane == 0)
    for (int i = 0; i < min(my_pages, kAttnStages); ++i) issue(i);

  // ---- Q fragments (rows r = qr * G + g; dims permuted to match the K page layout) ----
  uint32_t qa[KSTEPS][4];
  int row_len[2];  // causal length of the two rows this thread holds
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = g8 + 8 * half;
    const int qr = r / G, g = r % G;
    // rows beyond R carry a zero query and are never stored: leaving them unmasked keeps `full` below warp-uniform
    row_len[half] = r < R ? len - (q_len - 1 - qr) : 0x7fffffff;
    const __nv_bfloat16* qp = q + ((size_t(seq) * q_len + qr) * Hq + kvh * G + g) * D;
#pragma unroll
    for (int s = 0; s < KSTEPS; ++s) {
      const int d0 = 64 * (s >> 2) + 16 * c + 4 * (s & 3);
      float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
      if (r < R) {
        const uint2 raw = *reinterpret_cast<const uint2*>(qp + d0);
        const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&raw);
        v0 = __bfloat162float(b[0]) * scale_log2; v1 = __bfloat162float(b[1]) * scale_log2;
        v2 = __bfloat162float(b[2]) * scale_log2; v3 = __bfloat162float(b[3]) * scale_log2;
      }
      qa[s][half] = pack_f16x2(v0, v1);       // a0 / a1: k = 2c, 2c+1
      qa[s][2 + half] = pack_f16x2(v2, v3);   // a2 / a3: k = 2c+8, 2c+9
    }
  }

  float o[NBD][4];
#pragma unroll
  for (int j = 0; j < NBD; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m_run[2] = {kNeg, kNeg}, l_run[2] = {0.f, 0.f};
  bool ok = true;

  for (int i = 0; i < my_pages; ++i) {
    const int s = i % kAttnStages;
    ok = mbar_wait(&bars[s], (i / kAttnStages) & 1, abort_flag, status, kStatusTimeoutEpilogue);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    const uint8_t* st = ring + s * L::kStageBytes;
    const uint8_t* sK = st;
    const uint8_t* sV = st + L::kPageBytes;
    const float* sKs = reinterpret_cast<const float*>(st + 2 * L::kPageBytes);
    const float* sVs = sKs + 16;
    const int tok0 = (page_begin + warp + 4 * i) << 4;

    // ---- S = Q K^T for the 16 tokens of the page ----
    float sc[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      sc[nb][0] = sc[nb][1] = sc[nb][2] = sc[nb][3] = 0.f;
#pragma unroll
      for (int ch = 0; ch < D / 64; ++ch) {
        const uint4 kw = *reinterpret_cast<const uint4*>(sK + ch * 1024 + (nb * 8 + g8) * 64 + c * 16);
        const uint32_t w[4] = {kw.x, kw.y, kw.z, kw.w};
#pragma unroll
        for (int sub = 0; sub < 4; ++sub)
          mma_f16(sc[nb], qa[ch * 4 + sub], e4m3x2_to_f16x2(uint16_t(w[sub] & 0xffffu)),
                  e4m3x2_to_f16x2(uint16_t(w[sub] >> 16)));
      }
    }
    // ---- scales, causal mask, online softmax (rows g8 and g8+8; columns nb*8 + 2c, +1) ----
    // A page that lies wholly inside both rows' causal ranges (every page but the last one or two) needs no mask.
    const bool full = tok0 + 16 <= min(row_len[0], row_len[1]);
    float p[2][4];
    float mx[2] = {kNeg, kNeg};
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      const int tk = nb * 8 + 2 * c;
      const float2 ks = *reinterpret_cast<const float2*>(sKs + tk);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int half = e >> 1;
        sc[nb][e] *= (e & 1) ? ks.y : ks.x;
        if (!full && tok0 + tk + (e & 1) >= row_len[half]) sc[nb][e] = kNeg;
        mx[half] = fmaxf(mx[half], sc[nb][e]);
      }
    }
    float corr[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      mx[half] = fmaxf(mx[half], __shfl_xor_sync(0xffffffffu, mx[half], 1));
      mx[half] = fmaxf(mx[half], __shfl_xor_sync(0xffffffffu, mx[half], 2));
      const float mn = fmaxf(m_run[half], mx[half]);
      corr[half] = exp2f(m_run[half] - mn);
      m_run[half] = mn;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      const int tk = nb * 8 + 2 * c;
      const float2 vs = *reinterpret_cast<const float2*>(sVs + tk);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int half = e >> 1;
        // a masked score is kNeg: exp2 gives 0 unless the whole row is still empty (m_run == kNeg), hence the test
        const float pe = sc[nb][e] > 0.5f * kNeg ? exp2f(sc[nb][e] - m_run[half]) : 0.f;
        psum[half] += pe;
        p[nb][e] = pe * ((e & 1) ? vs.y : vs.x);  // fold the V multiplier of that token into P
      }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) l_run[half] = l_run[half] * corr[half] + psum[half];
    const uint32_t pa[4] = {pack_f16x2(p[0][0], p[0][1]), pack_f16x2(p[0][2], p[0][3]),
                            pack_f16x2(p[1][0], p[1][1]), pack_f16x2(p[1][2], p[1][3])};
    // ---- O = O * corr + P V; the rescale is skipped (warp-uniformly) while no row maximum moved, the usual case
    //      once the first pages of a long context have been seen ----
    const bool rescale = __any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f);
    if (rescale) {
#pragma unroll
      for (int j = 0; j < NBD; ++j) { o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1]; }
    }
#pragma unroll
    for (int j = 0; j < NBD; ++j) {
      const uint32_t vw = *reinterpret_cast<const uint32_t*>(sV + (8 * j + g8) * 16 + 4 * c);
      mma_f16(o[j], pa, e4m3x2_to_f16x2(uint16_t(vw & 0xffffu)), e4m3x2_to_f16x2(uint16_t(vw >> 16)));
    }
    __syncwarp();
    if (lane == 0 && i + kAttnStages < my_pages) issue(i + kAttnStages);
  }

  // ---- merge: lanes of a row, then the four warps (the page ring is reused as scratch) ----
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 1);
    l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 2);
  }
  float* w_o = reinterpret_cast<float*>(ring);          // [16 rows][D]
  float* w_ml = w_o + 16 * D;                           // [16][2]   (fits: kWarpBytes >= 16*D*4 + 128)
  __syncwarp();
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = g8 + 8 * half;
#pragma unroll
    for (int j = 0; j < NBD; ++j) {
      w_o[r * D + 8 * j + 2 * c] = o[j][2 * half];
      w_o[r * D + 8 * j + 2 * c + 1] = o[j][2 * half + 1];
    }
    if (c == 0) { w_ml[2 * r] = m_run[half]; w_ml[2 * r + 1] = l_run[half]; }
  }
  __syncthreads();
  if (!ok || *abort_flag) return;
  for (int idx = threadIdx.x; idx < R * D; idx += blockDim.x) {
    const int r = idx / D, d = idx % D;
    float mm = kNeg;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, reinterpret_cast<const float*>(smem + w * L::kWarpBytes)[16 * D + 2 * r]);
    float ll = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float* wo = reinterpret_cast<const float*>(smem + w * L::kWarpBytes);
      const float cw = exp2f(wo[16 * D + 2 * r] - mm);
      ll += wo[16 * D + 2 * r + 1] * cw;
      a += wo[r * D + d] * cw;
    }
    const int qr = r / G, g = r % G;
    const size_t hq = (size_t(seq) * q_len + qr) * Hq + kvh * G + g;
    if (nsplit == 1) {
      out[hq * D + d] = __float2bfloat16(ll > 0.f ? a / ll : 0.f);
    } else {
      part_acc[(hq * nsplit + split) * D + d] = a;
      if (d == 0) { part_ml[(hq * nsplit + split) * 2] = mm; part_ml[(hq * nsplit + split) * 2 + 1] = ll; }
    }
  }
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}

// The same work with the MMA turned around, for at most 8 (query row, head-of-group) pairs -- every plain decode step
// and verify windows of up to 8 / G tokens.  The page's 16 tokens are the M rows and the query pairs the 8 columns:
//   S^T [16 tokens x 8] = K [16 x D] . Q^T      A = the K page (the same 16-byte loads as above), B = Q from registers
//   O^T [D x 8]        += V^T [D x 16] . P       A = the V page (one 4-byte load per 8 dims), B = P, which is the
//                                                S^T accumulator transposed by two `movmatrix`
// Against the 16-row form this halves the MMAs (one 8-wide column block instead of two of which one was dead), the
// softmax arithmetic (4 scores per thread, none wasted on dead rows) and the output accumulators (D/4 registers), which
// leaves room for a fourth CTA per SM.
template <int D, int kAttnStages, int kMinBlocks>
__global__ void __launch_bounds__(128, kMinBlocks)
paged_attn_decode_t_kernel(const __nv_bfloat16* __restrict__ q, const uint8_t* __restrict__ k_cache,
                           const uint8_t* __restrict__ v_cache, const float* __restrict__ k_scale,
                           const float* __restrict__ v_scale, const int* __restrict__ block_table,
                           const int* __restrict__ seq_lens, __nv_bfloat16* __restrict__ out,
                           float* __restrict__ part_acc, float* __restrict__ part_ml, int Hq, int Hk, int max_pages,
                           float scale_log2, int q_len, int* status) {
  pdl_trigger();
  pdl_wait();
  using L = AttnSmem<D, kAttnStages>;
  constexpr int KSTEPS = D / 16, NBD = D / 16;
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g8 = lane >> 2, c = lane & 3;
  uint8_t* ring = smem + warp * L::kWarpBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 4 * L::kWarpBytes) + warp * kAttnStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 4 * L::kWarpBytes + 4 * kAttnStages * 8);

  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z, nsplit = gridDim.z;
  const int G = Hq / Hk;
  const int R = G * q_len;  // live columns, <= 8
  const int len = seq_lens[seq];
  const int pages_total = (len + 15) >> 4;
  const int per_split = (pages_total + nsplit - 1) / nsplit;
  const int page_begin = split * per_split;
  const int page_end = min(pages_total, page_begin + per_split);
  const int my_pages = page_end > page_begin + warp ? (page_end - page_begin - warp + 3) / 4 : 0;

  if (threadIdx.x == 0) *abort_flag = 0;
  if (lane == 0) {
    for (int s = 0; s < kAttnStages; ++s) mbar_init(&bars[s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  const int* bt = block_table + size_t(seq) * max_pages;
  auto issue = [&](int i, int page) {  // lane 0 only: start the copies of this warp's i-th page
    const int s = i % kAttnStages;
    const size_t ph = size_t(page) * Hk + kvh;
    uint8_t* st = ring + s * L::kStageBytes;
    mbar_expect_tx(&bars[s], L::kStageBytes);
    bulk_load(st, k_cache + ph * L::kPageBytes, L::kPageBytes, &bars[s]);
    bulk_load(st + L::kPageBytes, v_cache + ph * L::kPageBytes, L::kPageBytes, &bars[s]);
    bulk_load(st + 2 * L::kPageBytes, k_scale + ph * 16, 64, &bars[s]);
    bulk_load(st + 2 * L::kPageBytes + 64, v_scale + ph * 16, 64, &bars[s]);
  };
  if (lane == 0)
    for (int i = 0; i < min(my_pages, kAttnStages); ++i) issue(i, bt[page_begin + warp + 4 * i]);
  // the page id of the copy that the next iteration starts is fetched one iteration ahead
  int next_page = (lane == 0 && kAttnStages < my_pages) ? bt[page_begin + warp + 4 * kAttnStages] : 0;

  // ---- Q as the B operand: column g8 = pair (qr, g); dims in the K page's order ----
  uint32_t qb[KSTEPS][2];
  {
    const int r = g8;
    const int qr = r / G, g = r % G;
    const __nv_bfloat16* qp = q + ((size_t(seq) * q_len + qr) * Hq + kvh * G + g) * D;
#pragma unroll
    for (int s = 0; s < KSTEPS; ++s) {
      const int d0 = 64 * (s >> 2) + 16 * c + 4 * (s & 3);
      float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
      if (r < R) {
        const uint2 raw = *reinterpret_cast<const uint2*>(qp + d0);
        const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&raw);
        v0 = __bfloat162float(b[0]) * scale_log2; v1 = __bfloat162float(b[1]) * scale_log2;
        v2 = __bfloat162float(b[2]) * scale_log2; v3 = __bfloat162float(b[3]) * scale_log2;
      }
      qb[s][0] = pack_f16x2(v0, v1);  // b0: k = 2c, 2c+1
      qb[s][1] = pack_f16x2(v2, v3);  // b1: k = 2c+8, 2c+9
    }
  }
  int row_len[2];  // causal length of the two columns (2c, 2c+1) whose scores this thread holds
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int r = 2 * c + e;
    // columns beyond R carry a zero query and are never stored: leaving them unmasked keeps `full` below warp-uniform
    row_len[e] = r < R ? len - (q_len - 1 - r / G) : 0x7fffffff;
  }

  float o[NBD][4];  // O^T: [j][e] = (dim 16j + g8, column 2c + e), [j][2 + e] = (dim 16j + g8 + 8, column 2c + e)
#pragma unroll
  for (int j = 0; j < NBD; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m_run[2] = {kNeg, kNeg}, l_run[2] = {0.f, 0.f};
  bool ok = true;

  for (int i = 0; i < my_pages; ++i) {
    const int s = i % kAttnStages;
    ok = mbar_wait(&bars[s], (i / kAttnStages) & 1, abort_flag, status, kStatusTimeoutEpilogue);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    const uint8_t* st = ring + s * L::kStageBytes;
    const uint8_t* sK = st;
    const uint8_t* sV = st + L::kPageBytes;
    const float* sKs = reinterpret_cast<const float*>(st + 2 * L::kPageBytes);
    const float* sVs = sKs + 16;
    const int tok0 = (page_begin + warp + 4 * i) << 4;

    // ---- S^T = K Q^T: rows = tokens g8 and g8 + 8, columns 2c and 2c + 1 ----
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ch = 0; ch < D / 64; ++ch) {
      const uint4 k0 = *reinterpret_cast<const uint4*>(sK + ch * 1024 + g8 * 64 + c * 16);
      const uint4 k1 = *reinterpret_cast<const uint4*>(sK + ch * 1024 + (8 + g8) * 64 + c * 16);
      const uint32_t w0[4] = {k0.x, k0.y, k0.z, k0.w}, w1[4] = {k1.x, k1.y, k1.z, k1.w};
#pragma unroll
      for (int sub = 0; sub < 4; ++sub) {
        const uint32_t a[4] = {e4m3x2_to_f16x2(uint16_t(w0[sub] & 0xffffu)), e4m3x2_to_f16x2(uint16_t(w1[sub] & 0xffffu)),
                               e4m3x2_to_f16x2(uint16_t(w0[sub] >> 16)), e4m3x2_to_f16x2(uint16_t(w1[sub] >> 16))};
        mma_f16(sc, a, qb[ch * 4 + sub][0], qb[ch * 4 + sub][1]);
      }
    }
    // ---- scales, causal mask, online softmax ----
    const float ks0 = sKs[g8], ks1 = sKs[g8 + 8];
    sc[0] *= ks0; sc[1] *= ks0; sc[2] *= ks1; sc[3] *= ks1;
    const bool full = tok0 + 16 <= min(row_len[0], row_len[1]);  // row_len of dead columns is huge: warp-uniform enough
    if (!__all_sync(0xffffffffu, full)) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        if (tok0 + g8 >= row_len[e]) sc[e] = kNeg;
        if (tok0 + g8 + 8 >= row_len[e]) sc[2 + e] = kNeg;
      }
    }
    float corr[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float mx = fmaxf(sc[e], sc[2 + e]);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float mn = fmaxf(m_run[e], mx);
      corr[e] = exp2f(m_run[e] - mn);
      m_run[e] = mn;
    }
    const float vs0 = sVs[g8], vs1 = sVs[g8 + 8];
    float p[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int e = x & 1;
      // a masked score is kNeg: exp2 gives 0 unless the whole column is still empty (m_run == kNeg), hence the test
      const float pe = sc[x] > 0.5f * kNeg ? exp2f(sc[x] - m_run[e]) : 0.f;
      l_run[e] = (x < 2 ? l_run[e] * corr[e] : l_run[e]) + pe;
      p[x] = pe * (x < 2 ? vs0 : vs1);  // fold the V multiplier of that token into P
    }
    // P as the B operand of the second product: the accumulator layout transposed
    const uint32_t pb0 = movmatrix_trans(pack_f16x2(p[0], p[1]));
    const uint32_t pb1 = movmatrix_trans(pack_f16x2(p[2], p[3]));
    // ---- O^T = O^T * corr + V^T P; the rescale is skipped (warp-uniformly) while no column maximum moved ----
    const bool rescale = __any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f);
    if (rescale) {
#pragma unroll
      for (int j = 0; j < NBD; ++j) { o[j][0] *= corr[0]; o[j][1] *= corr[1]; o[j][2] *= corr[0]; o[j][3] *= corr[1]; }
    }
#pragma unroll
    for (int j = 0; j < NBD; ++j) {
      const uint32_t v0 = *reinterpret_cast<const uint32_t*>(sV + (16 * j + g8) * 16 + 4 * c);
      const uint32_t v1 = *reinterpret_cast<const uint32_t*>(sV + (16 * j + 8 + g8) * 16 + 4 * c);
      const uint32_t a[4] = {e4m3x2_to_f16x2(uint16_t(v0 & 0xffffu)), e4m3x2_to_f16x2(uint16_t(v1 & 0xffffu)),
                             e4m3x2_to_f16x2(uint16_t(v0 >> 16)), e4m3x2_to_f16x2(uint16_t(v1 >> 16))};
      mma_f16(o[j], a, pb0, pb1);
    }
    __syncwarp();
    if (lane == 0 && i + kAttnStages < my_pages) {
      issue(i + kAttnStages, next_page);
      if (i + 1 + kAttnStages < my_pages) next_page = bt[page_begin + warp + 4 * (i + 1 + kAttnStages)];
    }
  }

  // ---- merge: the lanes that share a column, then the four warps (the page ring is reused as scratch) ----
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 4);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 8);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 16);
  }
  float* w_o = reinterpret_cast<float*>(ring);          // [8 columns][D]
  float* w_ml = w_o + 16 * D;                           // [8][2]
  __syncwarp();
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int r = 2 * c + e;
#pragma unroll
    for (int j = 0; j < NBD; ++j) {
      w_o[r * D + 16 * j + g8] = o[j][e];
      w_o[r * D + 16 * j + 8 + g8] = o[j][2 + e];
    }
    if (g8 == 0) { w_ml[2 * r] = m_run[e]; w_ml[2 * r + 1] = l_run[e]; }
  }
  __syncthreads();
  if (!ok || *abort_flag) return;
  for (int idx = threadIdx.x; idx < R * D; idx += blockDim.x) {
    const int r = idx / D, d = idx % D;
    float mm = kNeg;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, reinterpret_cast<const float*>(smem + w * L::kWarpBytes)[16 * D + 2 * r]);
    float ll = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float* wo = reinterpret_cast<const float*>(smem + w * L::kWarpBytes);
      const float cw = exp2f(wo[16 * D + 2 * r] - mm);
      ll += wo[16 * D + 2 * r + 1] * cw;
      a += wo[r * D + d] * cw;
    }
    const int qr = r / G, g = r % G;
    const size_t hq = (size_t(seq) * q_len + qr) * Hq + kvh * G + g;
    if (nsplit == 1) {
      out[hq * D + d] = __float2bfloat16(ll > 0.f ? a / ll : 0.f);
    } else {
      part_acc[(hq * nsplit + split) * D + d] = a;
      if (d == 0) { part_ml[(hq * nsplit + split) * 2] = mm; part_ml[(hq * nsplit + split) * 2 + 1] = ll; }
    }
  }
}

// Combine the split partials (running max in the log2 domain).
template <int D>
__global__ void attn_reduce_log2_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                        __nv_bfloat16* __restrict__ out, int nsplit) {
  pdl_trigger();
  pdl_wait();
  const size_t hq = blockIdx.x;
  const int d = threadIdx.x;
  float mm = kNeg;
  for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, part_ml[(hq * nsplit + s) * 2]);
  float ll = 0.f, a = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float cw = exp2f(part_ml[(hq * nsplit + s) * 2] - mm);
    ll += part_ml[(hq * nsplit + s) * 2 + 1] * cw;
    a += part_acc[(hq * nsplit + s) * D + d] * cw;
  }
  out[hq * D + d] = __float2bfloat16(ll > 0.f ? a / ll : 0.f);
}

template <int D, int kAttnStages, int kMinBlocks, bool kTokensAsRows>
static int launch_attn_v(const void* q, const void* k_cache, const void* v_cache, const float* k_scale,
                         const float* v_scale, const int* block_table, const int* seq_lens, void* out, float* part_acc,
                         float* part_ml, int B, int Hq, int Hk, int max_pages, float sm_scale, int splits, int q_len,
                         int* status, cudaStream_t stream) {
  using L = AttnSmem<D, kAttnStages>;
  static_assert(L::kWarpBytes >= 16 * D * 4 + 128, "the per-warp ring doubles as the merge scratch");
  auto kernel = [] {
    if constexpr (kTokensAsRows) return &paged_attn_decode_t_kernel<D, kAttnStages, kMinBlocks>;
    else return &paged_attn_decode_mma_kernel<D, kAttnStages, kMinBlocks>;
  }();
  static bool attr[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -6;
  if (!attr[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess) return -6;
    attr[dev] = true;
  }
  const float scale_log2 = sm_scale * 1.4426950408889634f;
  launch_kernel(kernel, dim3(B, Hk, splits), dim3(128), L::kTotal, stream, static_cast<const __nv_bfloat16*>(q),
                static_cast<const uint8_t*>(k_cache), static_cast<const uint8_t*>(v_cache), k_scale, v_scale, block_table,
                seq_lens, static_cast<__nv_bfloat16*>(out), part_acc, part_ml, Hq, Hk, max_pages, scale_log2, q_len, status);
  if (cudaGetLastError() != cudaSuccess) return -7;
  if (splits > 1) {
    launch_kernel(attn_reduce_log2_kernel<D>, dim3(B * q_len * Hq), dim3(D), 0, stream, part_acc, part_ml, static_cast<__nv_bfloat16*>(out), splits);
    if (cudaGetLastError() != cudaSuccess) return -7;
  }
  return 0;
}

template <int D>
static int launch_attn(const void* q, const void* k_cache, const void* v_cache, const float* k_scale,
                       const float* v_scale, const int* block_table, const int* seq_lens, void* out, float* part_acc,
                       float* part_ml, int B, int Hq, int Hk, int max_pages, float sm_scale, int splits, int q_len,
                       int* status, cudaStream_t stream) {
  // MFQ_ATTN_VARIANT (measurement switch): 0 = by the number of query rows; 1 = always the 16-row form;
  // 2 / 3 = tokens-as-rows form with 2 pages in flight per warp and 5 CTAs per SM / 4 pages and 3 CTAs
  static const int variant = [] { const char* e = getenv("MFQ_ATTN_VARIANT"); return e ? atoi(e) : 0; }();
#define MFQ_ATTN_ARGS q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, out, part_acc, part_ml, B, Hq, Hk, max_pages, sm_scale, splits, q_len, status, stream
  const bool narrow = (Hq / Hk) * q_len <= 8 && variant != 1;
  if constexpr (D <= 128) {
    if (narrow && variant == 2) return launch_attn_v<D, 2, 5, true>(MFQ_ATTN_ARGS);
    if (narrow && variant == 3) return launch_attn_v<D, 4, 3, true>(MFQ_ATTN_ARGS);
    if (narrow) return launch_attn_v<D, 3, 4, true>(MFQ_ATTN_ARGS);
    return launch_attn_v<D, 3, 3, false>(MFQ_ATTN_ARGS);
  } else {
    if (narrow) return launch_attn_v<D, 3, 2, true>(MFQ_ATTN_ARGS);
    return launch_attn_v<D, 3, 1, false>(MFQ_ATTN_ARGS);
  }
#undef MFQ_ATTN_ARGS
}

}  // namespace mfq

// q: [B * q_len, Hq, D] bf16; caches in the fragment-friendly page layout described at the top of this file;
// seq_lens count every token visible to the last query row.  (Hq / Hk) * q_len must be <= 16.
extern "C" int mfq_paged_attn_decode_mma(const void* q, const void* k_cache, const void* v_cache, const float* k_scale,
                                         const float* v_scale, const int* block_table, const int* seq_lens, void* out,
                                         float* part_acc, float* part_ml, int B, int Hq, int Hk, int D, int max_pages,
                                         float sm_scale, int splits, int q_len, int* status, cudaStream_t stream) {
  if (B <= 0 || Hk <= 0 || Hq % Hk || (Hq / Hk) * q_len > 16 || splits < 1) return -1;
  if (D == 128)
    return mfq::launch_attn<128>(q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, out, part_acc, part_ml,
                                 B, Hq, Hk, max_pages, sm_scale, splits, q_len, status, stream);
  if (D == 256)
    return mfq::launch_attn<256>(q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, out, part_acc, part_ml,
                                 B, Hq, Hk, max_pages, sm_scale, splits, q_len, status, stream);
  if (D == 64)
    return mfq::launch_attn<64>(q, k_cache, v_cache, k_scale, v_scale, block_table, seq_lens, out, part_acc, part_ml, B,
                                Hq, Hk, max_pages, sm_scale, splits, q_len, status, stream);
  return -1;
}
