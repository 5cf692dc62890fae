// Gated DeltaNet prefill in 64-token chunks (the WY form of the gated delta rule).
//
// Per value head, with S [dk, dv] the state at the start of a chunk, g_i the decays, beta_i the write strengths,
// gamma_i = g_1 ... g_i the decay accumulated inside the chunk, and K, Q, V the chunk's (normalised) rows:
//
//   (I + A) D = beta V - diag(beta gamma) K S,      A_ij = beta_i (gamma_i / gamma_j) (k_i . k_j)   for j < i
//   =>  D = U - W S   with   U = (I + A)^-1 (beta V),   W = (I + A)^-1 (beta gamma K)
//   O = diag(gamma) Q S + P D,                      P_ij = (gamma_i / gamma_j) (q_i . k_j)          for j <= i
//   S <- gamma_C S + K^T diag(gamma_C / gamma) D
//
// which is the token recurrence  S <- g S;  d = beta (v - S^T k);  S <- S + k d^T;  o = S^T q  unrolled over the chunk.
// Two kernels:
//
//   gdn_chunk_prepare   one CTA per (sequence, KEY head, chunk), every chunk in parallel: normalises q and k, forms
//                       K K^T and Q K^T once for all value heads of the key head (tf32 MMAs), then per value head
//                       evaluates the gates, builds A and P and solves the unit-triangular system by forward
//                       substitution with ONE THREAD PER COLUMN of [beta V | beta gamma K] (256 columns, the solution
//                       column lives in 64 registers, A is read as broadcast float4).  No triangular inverse and no
//                       product with it is formed; the solve is fp32.  Writes the tiles Qn, Kn, W, P (rounded to
//                       tf32, the operand format of the scan) and U, gamma (fp32).
//   gdn_chunk_scan      the only sequential part: one CTA per (sequence, value head, 32 state columns) walks the
//                       chunks with the fp32 state slice in mma.sync accumulator registers; per chunk it issues
//                       W S and Q S (K = 128), P D (K <= 64, causal blocks only) and K^T D (K = 64) as m16n8k8 tf32
//                       MMAs from padded, bank-conflict-free shared-memory tiles.  A tile is stored in global memory
//                       with the same padded rows, so it arrives as ONE cp.async.bulk copy on an mbarrier (a copy
//                       per row kept the copy engine, not the tensor cores, busy): K / P / gamma double-buffered
//                       two chunks ahead, Q / W refilled as soon as the first phase of a chunk has consumed them.
//                       Two block barriers per chunk.
//
// The 64 x 128 x 32 products of the scan are far too small to feed tcgen05 (a 128-row UMMA tile would be half
// empty and the TMEM round trip longer than the MMAs); the chain per chunk is latency-bound, and mma.sync from
// shared memory keeps it shortest.  All waits are bounded and report through the status word.
//
// Reference counterpart: mfq/kernels/cuda/gdn_prefill_chunk.cu:104,273 (gdn_chunk_prepare_kernel / gdn_chunk_state_kernel:
// 64-token chunks, fp16 mma.sync with power-of-two rescaling, a [64, 64] triangular inverse held in shared memory).
#include "common.cuh"

#include <cstdlib>

namespace mfq {

int launch_gdn_gated_norm(const float* o_raw, const void* z, const float* norm_w, void* y, size_t pairs, int Hv, float eps,
                          int z_stride, cudaStream_t stream);

namespace {

constexpr int kC = 64;    // tokens per chunk
constexpr int kD = 128;   // dk = dv
constexpr int kAS = 132;  // shared-memory row stride (floats) of row-major A operands (Q, W): stride % 32 == 4
constexpr int kKS = 136;  // ... of K, which is read transposed: stride % 32 == 8
constexpr int kPS = 68;   // ... of P and of the triangular system
constexpr int kNS = 32;   // state columns per CTA of the scan
constexpr int kBS = 40;   // row stride of the [k][n] B operands (state slice, D): stride % 32 == 8
constexpr int kGS = 65;   // row stride of the Gram matrices in the prepare kernel

struct ChunkParams {
  const float* qkv;          // [B*L, 2*Hk*128 + Hv*128] fp32 after conv + SiLU (q | k | v), not normalised
  const __nv_bfloat16* a;    // [B*L, Hv] (row stride ab_stride)
  const __nv_bfloat16* bb;
  const float* A_log;
  const float* dt_bias;
  // operand tiles of the scan, stored with the padded row strides of its shared-memory layout: one bulk copy per tile
  float* qn;    // [B][Hk][NC][64][kAS]
  float* kn;    // [B][Hk][NC][64][kKS]
  float* wt;    // [B][Hv][NC][64][kAS]
  float* uv;    // [B][Hv][NC][64][128]
  float* pm;    // [B][Hv][NC][64][kPS]
  float* gam;   // [B][Hv][NC][128]: gamma_i, then gamma_C / gamma_i
  float* state; // [slots][Hv][128][128]
  const int* slot;
  float* o_raw; // [B*L, Hv*128]
  int L, Hk, Hv, NC, ab_stride;
  int* status;
};

__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void bulk_row(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ float dot4(const float4& a, const float4& b) {
  return fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, a.w * b.w)));
}

constexpr int kMaxRep = 8;  // value heads per key head the prepare kernel accepts
constexpr int kPrepSmemFloats = 2 * kC * kAS + 2 * kC * kGS + 2 * kMaxRep * kC;

template <int kMinBlocks>
__global__ void __launch_bounds__(256, kMinBlocks) gdn_chunk_prepare_kernel(const ChunkParams p) {
  extern __shared__ __align__(16) float sm[];
  float* Ks = sm;                   // [64][132] normalised k
  float* Qs = Ks + kC * kAS;        // [64][132] normalised, scaled q
  float* G = Qs + kC * kAS;         // [64][65]  k_i . k_j
  float* QK = G + kC * kGS;         // [64][65]  q_i . k_j
  float* A = Qs;                    // [64][68]  strictly lower triangular system of the current value head (q is dead by then)
  float* cg_all = QK + kC * kGS;        // [R][64] log gamma_i of every value head of this key head
  float* bt_all = cg_all + kMaxRep * kC;  // [R][64] beta_i
  const int chunk = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  if (p.slot[b] < 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int C = 2 * p.Hk * kD + p.Hv * kD;
  const int t0 = chunk * kC;
  const size_t tile_k = (size_t(b) * p.Hk + hk) * p.NC + chunk;

  const int R = p.Hv / p.Hk;
  // ---- gates of the 64 tokens (two per lane) and the running log decay: one warp per value head, requested first so
  //      that their loads fly under the q / k normalisation ----
  for (int rr = warp; rr < R; rr += 8) {
    const int h = hk * R + rr;
    float lg[2], be[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int t = t0 + lane * 2 + e;
      lg[e] = 0.f; be[e] = 0.f;
      if (t < p.L) {
        const size_t tok = size_t(b) * p.L + t;
        const float av = __bfloat162float(p.a[tok * p.ab_stride + h]) + p.dt_bias[h];
        const float sp = av > 20.f ? av : log1pf(__expf(av));
        lg[e] = -__expf(p.A_log[h]) * sp;
        be[e] = 1.f / (1.f + __expf(-__bfloat162float(p.bb[tok * p.ab_stride + h])));
      }
    }
    const float pair = lg[0] + lg[1];
    float inc = pair;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += n;
    }
    const float excl = inc - pair;
    cg_all[rr * kC + lane * 2] = excl + lg[0];
    cg_all[rr * kC + lane * 2 + 1] = excl + pair;
    bt_all[rr * kC + lane * 2] = be[0];
    bt_all[rr * kC + lane * 2 + 1] = be[1];
  }

  // ---- q and k rows of the chunk: l2-normalised (q also scaled by dk^-1/2); rows past the end are zero ----
  {
    float4 q4[8], k4[8];  // this warp's eight rows, all requested before the first is used
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int t = t0 + warp + 8 * e;
      q4[e] = make_float4(0.f, 0.f, 0.f, 0.f);
      k4[e] = q4[e];
      if (t < p.L) {
        const float* row = p.qkv + (size_t(b) * p.L + t) * C;
        q4[e] = *reinterpret_cast<const float4*>(row + hk * kD + lane * 4);
        k4[e] = *reinterpret_cast<const float4*>(row + p.Hk * kD + hk * kD + lane * 4);
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int i = warp + 8 * e;
      float sq = dot4(q4[e], q4[e]), sk = dot4(k4[e], k4[e]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
        sk += __shfl_xor_sync(0xffffffffu, sk, o);
      }
      const float iq = rsqrtf(sq + 1e-6f) * rsqrtf(float(kD)), ik = rsqrtf(sk + 1e-6f);
      const float4 q = make_float4(q4[e].x * iq, q4[e].y * iq, q4[e].z * iq, q4[e].w * iq);
      const float4 k = make_float4(k4[e].x * ik, k4[e].y * ik, k4[e].z * ik, k4[e].w * ik);
      *reinterpret_cast<float4*>(Qs + i * kAS + lane * 4) = q;
      *reinterpret_cast<float4*>(Ks + i * kAS + lane * 4) = k;
      *reinterpret_cast<float4*>(p.qn + tile_k * (kC * kAS) + i * kAS + lane * 4) = make_float4(to_tf32(q.x), to_tf32(q.y), to_tf32(q.z), to_tf32(q.w));
      *reinterpret_cast<float4*>(p.kn + tile_k * (kC * kKS) + i * kKS + lane * 4) = make_float4(to_tf32(k.x), to_tf32(k.y), to_tf32(k.z), to_tf32(k.w));
    }
  }
  __syncthreads();

  // ---- Gram matrices, shared by the value heads of this key head, on tensor cores (tf32 operands, fp32 sums):
  //      warp = 16 rows x 32 columns of both K K^T and Q K^T; tiles wholly above the diagonal are skipped ----
  {
    const int g = lane >> 2, tg = lane & 3;
    const int mt = warp >> 1, c0 = 32 * (warp & 1);
    const int r0 = 16 * mt + g, r1 = r0 + 8;
    const int nts = min(4, (16 * mt + 15 - c0) / 8 + 1);  // column tiles that reach the diagonal or lie below it
    float gk[4][4], gq[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) gk[nt][e] = gq[nt][e] = 0.f;
    if (nts > 0) {
#pragma unroll 2
      for (int ks = 0; ks < kD / 8; ++ks) {
        const int k0 = 8 * ks;
        uint32_t ak[4], aq[4];
        ak[0] = __float_as_uint(to_tf32(Ks[r0 * kAS + k0 + tg]));
        ak[1] = __float_as_uint(to_tf32(Ks[r1 * kAS + k0 + tg]));
        ak[2] = __float_as_uint(to_tf32(Ks[r0 * kAS + k0 + tg + 4]));
        ak[3] = __float_as_uint(to_tf32(Ks[r1 * kAS + k0 + tg + 4]));
        aq[0] = __float_as_uint(to_tf32(Qs[r0 * kAS + k0 + tg]));
        aq[1] = __float_as_uint(to_tf32(Qs[r1 * kAS + k0 + tg]));
        aq[2] = __float_as_uint(to_tf32(Qs[r0 * kAS + k0 + tg + 4]));
        aq[3] = __float_as_uint(to_tf32(Qs[r1 * kAS + k0 + tg + 4]));
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          if (nt < nts) {
            uint32_t bf[2];  // B = K^T: element (d, j) lives at Ks[j][d]
            bf[0] = __float_as_uint(to_tf32(Ks[(c0 + 8 * nt + g) * kAS + k0 + tg]));
            bf[1] = __float_as_uint(to_tf32(Ks[(c0 + 8 * nt + g) * kAS + k0 + tg + 4]));
            mma_tf32(gk[nt], ak, bf);
            mma_tf32(gq[nt], aq, bf);
          }
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int col = c0 + 8 * nt + 2 * tg;
      G[r0 * kGS + col] = gk[nt][0]; G[r0 * kGS + col + 1] = gk[nt][1];
      G[r1 * kGS + col] = gk[nt][2]; G[r1 * kGS + col + 1] = gk[nt][3];
      QK[r0 * kGS + col] = gq[nt][0]; QK[r0 * kGS + col + 1] = gq[nt][1];
      QK[r1 * kGS + col] = gq[nt][2]; QK[r1 * kGS + col + 1] = gq[nt][3];
    }
  }

  for (int rr = 0; rr < R; ++rr) {
    const int h = hk * R + rr;
    const size_t tile_h = (size_t(b) * p.Hv + h) * p.NC + chunk;
    const float* cg = cg_all + rr * kC;
    const float* bt = bt_all + rr * kC;
    // the V column of this thread: requested before the triangular system is built, used after it
    float x[kC];
    if (tid < kD) {
      const float* vcol = p.qkv + size_t(b) * p.L * C + 2 * p.Hk * kD + h * kD + tid;
#pragma unroll
      for (int i = 0; i < kC; ++i) x[i] = (t0 + i < p.L) ? vcol[size_t(t0 + i) * C] : 0.f;
    }
    __syncthreads();  // Gram matrices complete; the previous head's A is no longer read
    float* ptile = p.pm + tile_h * size_t(kC * kPS);
    for (int idx = tid; idx < kC * kC; idx += 256) {
      const int i = idx >> 6, j = idx & 63;
      const float dec = __expf(fminf(cg[i] - cg[j], 0.f));  // j <= i: the decay from token j to token i
      A[i * kPS + j] = j < i ? bt[i] * dec * G[i * kGS + j] : 0.f;
      ptile[i * kPS + j] = j <= i ? to_tf32(dec * QK[i * kGS + j]) : 0.f;
    }
    if (tid < kC) {
      p.gam[tile_h * 128 + tid] = __expf(cg[tid]);
      p.gam[tile_h * 128 + 64 + tid] = __expf(cg[kC - 1] - cg[tid]);
    }
    __syncthreads();
    // ---- (I + A) x = rhs, one column per thread: [beta V | beta gamma K] ----
    if (tid < kD) {
#pragma unroll
      for (int i = 0; i < kC; ++i) x[i] *= bt[i];
    } else {
#pragma unroll
      for (int i = 0; i < kC; ++i) x[i] = bt[i] * __expf(cg[i]) * Ks[i * kAS + tid - kD];
    }
#pragma unroll
    for (int i = 1; i < kC; ++i) {
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int j = 0; j + 3 < i; j += 4) {
        const float4 a4 = *reinterpret_cast<const float4*>(A + i * kPS + j);
        a0 = fmaf(a4.x, x[j], a0);
        a1 = fmaf(a4.y, x[j + 1], a1);
        a2 = fmaf(a4.z, x[j + 2], a2);
        a3 = fmaf(a4.w, x[j + 3], a3);
      }
#pragma unroll
      for (int j = i & ~3; j < i; ++j) a0 = fmaf(A[i * kPS + j], x[j], a0);
      x[i] -= (a0 + a1) + (a2 + a3);
    }
    if (tid < kD) {
      float* dst = p.uv + tile_h * size_t(kC * kD) + tid;
#pragma unroll
      for (int i = 0; i < kC; ++i) dst[i * kD] = x[i];
    } else {
      float* dst = p.wt + tile_h * size_t(kC * kAS) + tid - kD;
#pragma unroll
      for (int i = 0; i < kC; ++i) dst[i * kAS] = to_tf32(x[i]);
    }
  }
}

// Shared memory of the scan (floats): Q, W single; K, P, gamma double-buffered; state slice and the two scalings of D.
constexpr int kScanQ = 0;
constexpr int kScanW = kScanQ + kC * kAS;
constexpr int kScanK = kScanW + kC * kAS;            // 2 x [64][136]
constexpr int kScanP = kScanK + 2 * kC * kKS;        // 2 x [64][68]
constexpr int kScanG = kScanP + 2 * kC * kPS;        // 2 x [128]
constexpr int kScanS = kScanG + 2 * 128;             // [128][40]
constexpr int kScanD1 = kScanS + kD * kBS;           // [64][40]  D
constexpr int kScanD2 = kScanD1 + kC * kBS;          // [64][40]  diag(gamma_C / gamma) D
constexpr int kScanFloats = kScanD2 + kC * kBS;
constexpr int kScanSmemBytes = kScanFloats * 4 + 64;
constexpr uint32_t kBytesQW = 2 * kC * kAS * 4;
constexpr uint32_t kBytesKP = kC * kKS * 4 + kC * kPS * 4 + 128 * 4;

__global__ void __launch_bounds__(256, 1) gdn_chunk_scan_kernel(const ChunkParams p) {
  extern __shared__ __align__(16) float sm[];
  float* Qt = sm + kScanQ;
  float* Wt = sm + kScanW;
  float* Ssm = sm + kScanS;
  float* D1 = sm + kScanD1;
  float* D2 = sm + kScanD2;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kScanFloats);  // [0] Q/W, [1], [2] K/P/gamma buffers
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 3);
  const int slice = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int slot = p.slot[b];
  if (slot < 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tg = lane & 3;
  const int hk = h / (p.Hv / p.Hk);
  const size_t tiles_k = (size_t(b) * p.Hk + hk) * p.NC, tiles_h = (size_t(b) * p.Hv + h) * p.NC;

  if (tid == 0) {
    for (int i = 0; i < 3; ++i) mbar_init(&bars[i], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();

  // one thread issues the copies: a tile is contiguous in global memory, in the layout it has in shared memory
  auto load_qw = [&](int c) {
    mbar_expect_tx(&bars[0], kBytesQW);
    bulk_row(Qt, p.qn + (tiles_k + c) * size_t(kC * kAS), kC * kAS * 4, &bars[0]);
    bulk_row(Wt, p.wt + (tiles_h + c) * size_t(kC * kAS), kC * kAS * 4, &bars[0]);
  };
  auto load_kp = [&](int c) {
    const int buf = c & 1;
    mbar_expect_tx(&bars[1 + buf], kBytesKP);
    bulk_row(sm + kScanK + buf * kC * kKS, p.kn + (tiles_k + c) * size_t(kC * kKS), kC * kKS * 4, &bars[1 + buf]);
    bulk_row(sm + kScanP + buf * kC * kPS, p.pm + (tiles_h + c) * size_t(kC * kPS), kC * kPS * 4, &bars[1 + buf]);
    bulk_row(sm + kScanG + buf * 128, p.gam + (tiles_h + c) * 128, 128 * 4, &bars[1 + buf]);
  };
  if (tid == 0) {
    load_qw(0);
    load_kp(0);
    if (p.NC > 1) load_kp(1);
  }

  // state slice: warp w owns rows 16 w + {g, g + 8}, all four 8-column tiles
  float* st = p.state + (size_t(slot) * p.Hv + h) * kD * kD + slice * kNS;
  float s[4][4];
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    const float2 lo = *reinterpret_cast<const float2*>(st + (16 * warp + g) * kD + 8 * nt + 2 * tg);
    const float2 hi = *reinterpret_cast<const float2*>(st + (16 * warp + g + 8) * kD + 8 * nt + 2 * tg);
    s[nt][0] = lo.x; s[nt][1] = lo.y; s[nt][2] = hi.x; s[nt][3] = hi.y;
    *reinterpret_cast<float2*>(Ssm + (16 * warp + g) * kBS + 8 * nt + 2 * tg) = make_float2(to_tf32(lo.x), to_tf32(lo.y));
    *reinterpret_cast<float2*>(Ssm + (16 * warp + g + 8) * kBS + 8 * nt + 2 * tg) = make_float2(to_tf32(hi.x), to_tf32(hi.y));
  }
  __syncthreads();

  const int mt = warp >> 1, nt0 = 2 * (warp & 1);  // this warp's token rows 16 mt + {g, g + 8} and its two column tiles
  const int i0 = 16 * mt + g, i1 = i0 + 8;
  bool ok = true;
  for (int c = 0; c < p.NC; ++c) {
    const int buf = c & 1;
    const float* Kt = sm + kScanK + buf * kC * kKS;
    const float* Pt = sm + kScanP + buf * kC * kPS;
    const float* gam = sm + kScanG + buf * 128;
    // U rows of this warp's tiles: requested now, used after the first products
    const float* ut = p.uv + (tiles_h + c) * size_t(kC * kD) + slice * kNS;
    float2 u[2][2];
#pragma unroll
    for (int nn = 0; nn < 2; ++nn) {
      u[nn][0] = *reinterpret_cast<const float2*>(ut + i0 * kD + 8 * (nt0 + nn) + 2 * tg);
      u[nn][1] = *reinterpret_cast<const float2*>(ut + i1 * kD + 8 * (nt0 + nn) + 2 * tg);
    }
    ok = mbar_wait(&bars[0], c & 1, abort_flag, p.status, kStatusTimeoutProducer) && ok;
    ok = mbar_wait(&bars[1 + buf], (c >> 1) & 1, abort_flag, p.status, kStatusTimeoutProducer) && ok;

    // ---- phase 1: W S and Q S ----
    float ws[2][4], qs[2][4];
#pragma unroll
    for (int nn = 0; nn < 2; ++nn)
#pragma unroll
      for (int e = 0; e < 4; ++e) ws[nn][e] = qs[nn][e] = 0.f;
#pragma unroll 4
    for (int ks = 0; ks < kD / 8; ++ks) {
      const int k0 = 8 * ks;
      uint32_t aw[4], aq[4];
      aw[0] = __float_as_uint(Wt[i0 * kAS + k0 + tg]);
      aw[1] = __float_as_uint(Wt[i1 * kAS + k0 + tg]);
      aw[2] = __float_as_uint(Wt[i0 * kAS + k0 + tg + 4]);
      aw[3] = __float_as_uint(Wt[i1 * kAS + k0 + tg + 4]);
      aq[0] = __float_as_uint(Qt[i0 * kAS + k0 + tg]);
      aq[1] = __float_as_uint(Qt[i1 * kAS + k0 + tg]);
      aq[2] = __float_as_uint(Qt[i0 * kAS + k0 + tg + 4]);
      aq[3] = __float_as_uint(Qt[i1 * kAS + k0 + tg + 4]);
#pragma unroll
      for (int nn = 0; nn < 2; ++nn) {
        uint32_t bf[2];
        bf[0] = __float_as_uint(Ssm[(k0 + tg) * kBS + 8 * (nt0 + nn) + g]);
        bf[1] = __float_as_uint(Ssm[(k0 + tg + 4) * kBS + 8 * (nt0 + nn) + g]);
        mma_tf32(ws[nn], aw, bf);
        mma_tf32(qs[nn], aq, bf);
      }
    }
    const float gm0 = gam[i0], gm1 = gam[i1], e0 = gam[64 + i0], e1 = gam[64 + i1], gamma_c = gam[kC - 1];
    float o[2][4];
#pragma unroll
    for (int nn = 0; nn < 2; ++nn) {
      const float d0 = u[nn][0].x - ws[nn][0], d1 = u[nn][0].y - ws[nn][1];
      const float d2 = u[nn][1].x - ws[nn][2], d3 = u[nn][1].y - ws[nn][3];
      const int n = 8 * (nt0 + nn) + 2 * tg;
      *reinterpret_cast<float2*>(D1 + i0 * kBS + n) = make_float2(to_tf32(d0), to_tf32(d1));
      *reinterpret_cast<float2*>(D1 + i1 * kBS + n) = make_float2(to_tf32(d2), to_tf32(d3));
      *reinterpret_cast<float2*>(D2 + i0 * kBS + n) = make_float2(to_tf32(d0 * e0), to_tf32(d1 * e0));
      *reinterpret_cast<float2*>(D2 + i1 * kBS + n) = make_float2(to_tf32(d2 * e1), to_tf32(d3 * e1));
      o[nn][0] = gm0 * qs[nn][0]; o[nn][1] = gm0 * qs[nn][1];
      o[nn][2] = gm1 * qs[nn][2]; o[nn][3] = gm1 * qs[nn][3];
    }
    if (!__syncthreads_and(ok)) break;  // D visible; Q, W and the state copy are free
    if (tid == 0 && c + 1 < p.NC) {
      fence_proxy_async_smem();
      load_qw(c + 1);
    }

    // ---- phase 2: O += P D over the causal blocks, then the state update ----
    for (int ks = 0; ks <= 2 * mt + 1; ++ks) {
      const int k0 = 8 * ks;
      uint32_t ap[4];
      ap[0] = __float_as_uint(Pt[i0 * kPS + k0 + tg]);
      ap[1] = __float_as_uint(Pt[i1 * kPS + k0 + tg]);
      ap[2] = __float_as_uint(Pt[i0 * kPS + k0 + tg + 4]);
      ap[3] = __float_as_uint(Pt[i1 * kPS + k0 + tg + 4]);
#pragma unroll
      for (int nn = 0; nn < 2; ++nn) {
        uint32_t bf[2];
        bf[0] = __float_as_uint(D1[(k0 + tg) * kBS + 8 * (nt0 + nn) + g]);
        bf[1] = __float_as_uint(D1[(k0 + tg + 4) * kBS + 8 * (nt0 + nn) + g]);
        mma_tf32(o[nn], ap, bf);
      }
    }
    {
      const int t_a = c * kC + i0, t_b = c * kC + i1;
      float* orow = p.o_raw + size_t(b) * p.L * p.Hv * kD + h * kD + slice * kNS;
#pragma unroll
      for (int nn = 0; nn < 2; ++nn) {
        const int n = 8 * (nt0 + nn) + 2 * tg;
        if (t_a < p.L) *reinterpret_cast<float2*>(orow + size_t(t_a) * p.Hv * kD + n) = make_float2(o[nn][0], o[nn][1]);
        if (t_b < p.L) *reinterpret_cast<float2*>(orow + size_t(t_b) * p.Hv * kD + n) = make_float2(o[nn][2], o[nn][3]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] *= gamma_c;
#pragma unroll
    for (int ks = 0; ks < kC / 8; ++ks) {
      const int k0 = 8 * ks;
      uint32_t ak[4];  // A = K^T: element (m, token) lives at Kt[token][m]
      ak[0] = __float_as_uint(Kt[(k0 + tg) * kKS + 16 * warp + g]);
      ak[1] = __float_as_uint(Kt[(k0 + tg) * kKS + 16 * warp + g + 8]);
      ak[2] = __float_as_uint(Kt[(k0 + tg + 4) * kKS + 16 * warp + g]);
      ak[3] = __float_as_uint(Kt[(k0 + tg + 4) * kKS + 16 * warp + g + 8]);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        uint32_t bf[2];
        bf[0] = __float_as_uint(D2[(k0 + tg) * kBS + 8 * nt + g]);
        bf[1] = __float_as_uint(D2[(k0 + tg + 4) * kBS + 8 * nt + g]);
        mma_tf32(s[nt], ak, bf);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      *reinterpret_cast<float2*>(Ssm + (16 * warp + g) * kBS + 8 * nt + 2 * tg) = make_float2(to_tf32(s[nt][0]), to_tf32(s[nt][1]));
      *reinterpret_cast<float2*>(Ssm + (16 * warp + g + 8) * kBS + 8 * nt + 2 * tg) = make_float2(to_tf32(s[nt][2]), to_tf32(s[nt][3]));
    }
    __syncthreads();  // new state copy visible; K / P / gamma buffer and D free
    if (tid == 0 && c + 2 < p.NC) {
      fence_proxy_async_smem();
      load_kp(c + 2);
    }
  }
  if (!ok) {
    // a copy may still be in flight towards this CTA's shared memory: give the outstanding phases one more bounded wait
    if (tid == 0) {
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) {
      }
    }
    __syncthreads();
    return;  // the state is left as it was; the host sees the status word
  }
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    *reinterpret_cast<float2*>(st + (16 * warp + g) * kD + 8 * nt + 2 * tg) = make_float2(s[nt][0], s[nt][1]);
    *reinterpret_cast<float2*>(st + (16 * warp + g + 8) * kD + 8 * nt + 2 * tg) = make_float2(s[nt][2], s[nt][3]);
  }
}

}  // namespace
}  // namespace mfq

using namespace mfq;

// Floats of scratch that mfq_gdn_prefill_chunked needs for B rows of L tokens.
extern "C" long long mfq_gdn_chunk_scratch_floats(int B, int L, int Hk, int Hv) {
  const long long nc = (L + kC - 1) / kC;
  return nc * B * (1ll * Hk * kC * (kAS + kKS) + 1ll * Hv * kC * (kAS + kD + kPS) + 128ll * Hv);
}

// Long rows without checkpoints, chunked.  qkv is left untouched; o_raw [B*L, Hv*128] fp32 and scratch are work space.
extern "C" int mfq_gdn_prefill_chunked(const float* qkv, const void* z, const void* a, const void* b, const float* A_log,
                                       const float* dt_bias, const float* norm_w, float* state, const int* slot, void* y,
                                       float* o_raw, float* scratch, long long scratch_floats, int B, int L, int Hk, int Hv,
                                       int dk, int dv, float eps, int z_stride, int ab_stride, int* status,
                                       cudaStream_t stream) {
  if (B <= 0 || L <= 0 || dk != kD || dv != kD || Hk <= 0 || Hv % Hk || Hv / Hk > kMaxRep || z_stride % 4) return -1;
  if (scratch_floats < mfq_gdn_chunk_scratch_floats(B, L, Hk, Hv)) return -2;
  const int nc = (L + kC - 1) / kC;
  ChunkParams p{};
  p.qkv = qkv; p.a = static_cast<const __nv_bfloat16*>(a); p.bb = static_cast<const __nv_bfloat16*>(b);
  p.A_log = A_log; p.dt_bias = dt_bias;
  float* cur = scratch;
  p.qn = cur; cur += size_t(B) * Hk * nc * kC * kAS;
  p.kn = cur; cur += size_t(B) * Hk * nc * kC * kKS;
  p.wt = cur; cur += size_t(B) * Hv * nc * kC * kAS;
  p.uv = cur; cur += size_t(B) * Hv * nc * kC * kD;
  p.pm = cur; cur += size_t(B) * Hv * nc * kC * kPS;
  p.gam = cur;
  p.state = state; p.slot = slot; p.o_raw = o_raw;
  p.L = L; p.Hk = Hk; p.Hv = Hv; p.NC = nc; p.ab_stride = ab_stride; p.status = status;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(gdn_chunk_prepare_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmemFloats * 4) != cudaSuccess) return -3;
    if (cudaFuncSetAttribute(gdn_chunk_prepare_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmemFloats * 4) != cudaSuccess) return -3;
    if (cudaFuncSetAttribute(gdn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScanSmemBytes) != cudaSuccess) return -3;
    attr_set[dev] = true;
  }
  static const int prep_blocks = [] { const char* e = getenv("MFQ_GDN_PREP_BLOCKS"); return e ? atoi(e) : 2; }();
  if (prep_blocks == 1) gdn_chunk_prepare_kernel<1><<<dim3(nc, Hk, B), 256, kPrepSmemFloats * 4, stream>>>(p);
  else gdn_chunk_prepare_kernel<2><<<dim3(nc, Hk, B), 256, kPrepSmemFloats * 4, stream>>>(p);
  gdn_chunk_scan_kernel<<<dim3(kD / kNS, Hv, B), 256, kScanSmemBytes, stream>>>(p);
  if (cudaGetLastError() != cudaSuccess) return -7;
  return launch_gdn_gated_norm(o_raw, z, norm_w, y, size_t(B) * L * Hv, Hv, eps, z_stride, stream);
}
