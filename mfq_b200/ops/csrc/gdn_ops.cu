// Gated DeltaNet (linear attention with the gated delta rule) for decode, verify windows and prefill.
//
// Per value head h (key head h / (Hv/Hk)), with a [dk, dv] fp32 state S carried across tokens:
//   q, k   <- l2norm(silu(conv1d(q, k)))   (q also scaled by dk^-1/2);  v <- silu(conv1d(v))
//   decay  =  exp(-exp(A_log[h]) * softplus(a_t[h] + dt_bias[h]));      beta = sigmoid(b_t[h])
//   S      <- decay * S;   delta = (v - S^T k) * beta;   S <- S + k delta^T;   o = S^T q
//   y      =  rmsnorm(o) * w * silu(z)                                  (per head, over dv)
// Kernels:
//   gdn_conv        causal depthwise conv (4 taps) + SiLU over the packed q|k|v channels; a FIR, so every (token,
//                   channel) is independent; the 3-token history of each sequence lives in a conv state.
//   gdn_recurrent   one CTA per (sequence, value head), one thread per state column: the column S[:, j] stays in 128
//                   registers for the whole token run, so a token costs 3*dk FMAs per thread and no cross-thread
//                   reduction; k/q are normalised once per token in shared memory; the gated RMSNorm is fused.
//                   State is read once and written once per launch (decode: 2 x 64 KB per head -- the HBM floor);
//                   with `ckpt` the state after EVERY token of a short window is written instead, so that an MTP
//                   verify pass can keep the state of the last accepted token (gdn_select).
// Sequences are a regular [B, L] grid (decode: L = 1; verify: L = K+1; prefill: B = 1); slot[b] < 0 skips a row.
// Reference counterparts: cpp_runtime/backends/cuda/kernels gdn_decode_core_kernel, ssm_conv_*_decode,
// gdn_rms_norm_gate_kernel, gdn_prefill_chunk.cu (chunked mma.sync prefill), gdn_decode_window.cu (verify window).
#include "common.cuh"

namespace mfq {

// x [B*L, C] bf16 (pre-conv), conv_state [slots, 3, C] fp32 (oldest first), w [C, 4] fp32, out [B*L, C] fp32.
// conv_ckpt (optional) [B, L, 3, C]: history after each token, for verify windows (then conv_state is left alone).
__global__ void gdn_conv_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ conv_state,
                                const float* __restrict__ w, const int* __restrict__ slot, float* __restrict__ out,
                                float* __restrict__ conv_ckpt, int L, int C, int xs, int update_state) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.y;
  const int s = slot[b];
  if (s < 0) return;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float w0 = w[c * 4], w1 = w[c * 4 + 1], w2 = w[c * 4 + 2], w3 = w[c * 4 + 3];
  float* st = conv_state + size_t(s) * 3 * C;
  const float h0 = st[c], h1 = st[C + c], h2 = st[2 * C + c];
  auto in = [&](int t) -> float {  // input of token t of this row; negative t reads the carried history
    if (t >= 0) return __bfloat162float(x[(size_t(b) * L + t) * xs + c]);
    return t == -1 ? h2 : t == -2 ? h1 : h0;
  };
  for (int t = blockIdx.z; t < L; t += gridDim.z) {
    const float y = w0 * in(t - 3) + w1 * in(t - 2) + w2 * in(t - 1) + w3 * in(t);
    out[(size_t(b) * L + t) * C + c] = y / (1.f + __expf(-y));
    if (conv_ckpt) {
      float* ck = conv_ckpt + (size_t(b) * L + t) * 3 * C;
      ck[c] = in(t - 2); ck[C + c] = in(t - 1); ck[2 * C + c] = in(t);
    }
  }
  // a grid with one z slice has read the whole history of this channel by now: it may shift it in place
  if (update_state) {
    const float n0 = in(L - 3), n1 = in(L - 2), n2 = in(L - 1);
    st[c] = n0; st[C + c] = n1; st[2 * C + c] = n2;
  }
}

// Long rows (prefill): a thread owns two adjacent channels and a run of kConvRun consecutive tokens, slides the 4-tap window
// through registers (every input is read once, as a 4-byte pair) and keeps eight independent loads in flight.
constexpr int kConvRun = 32;
__global__ void __launch_bounds__(128) gdn_conv_long_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ conv_state,
                                                            const float* __restrict__ w, const int* __restrict__ slot,
                                                            float* __restrict__ out, int L, int C, int xs) {
  const int b = blockIdx.y;
  const int s = slot[b];
  if (s < 0) return;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (c >= C) return;
  const float4 wa = *reinterpret_cast<const float4*>(w + c * 4), wb = *reinterpret_cast<const float4*>(w + c * 4 + 4);
  const float* st = conv_state + size_t(s) * 3 * C;
  const int t0 = blockIdx.z * kConvRun;
  auto in = [&](int t) -> float2 {
    if (t >= 0) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + (size_t(b) * L + t) * xs + c));
    return *reinterpret_cast<const float2*>(st + (3 + t) * C + c);  // t = -3, -2, -1: history rows 0, 1, 2
  };
  float2 p3 = in(t0 - 3), p2 = in(t0 - 2), p1 = in(t0 - 1);
  const int n = min(kConvRun, L - t0);
  for (int i = 0; i < n; i += 8) {
    float2 cur[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) cur[e] = (i + e < n) ? in(t0 + i + e) : make_float2(0.f, 0.f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (i + e < n) {
        const float ya = wa.x * p3.x + wa.y * p2.x + wa.z * p1.x + wa.w * cur[e].x;
        const float yb = wb.x * p3.y + wb.y * p2.y + wb.z * p1.y + wb.w * cur[e].y;
        *reinterpret_cast<float2*>(out + (size_t(b) * L + t0 + i + e) * C + c) =
            make_float2(ya / (1.f + __expf(-ya)), yb / (1.f + __expf(-yb)));
      }
      p3 = p2; p2 = p1; p1 = cur[e];
    }
  }
}

// History update, as a launch of its own AFTER the convolution: blocks of the convolution that handle the first
// tokens still read the old history, so it cannot be overwritten by a sibling block of the same grid.
__global__ void gdn_conv_state_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ conv_state,
                                      const int* __restrict__ slot, int L, int C, int xs) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.y;
  const int s = slot[b];
  if (s < 0) return;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float* st = conv_state + size_t(s) * 3 * C;
  const float h0 = st[c], h1 = st[C + c], h2 = st[2 * C + c];
  auto in = [&](int t) -> float {
    if (t >= 0) return __bfloat162float(x[(size_t(b) * L + t) * xs + c]);
    return t == -1 ? h2 : t == -2 ? h1 : h0;
  };
  const float n0 = in(L - 3), n1 = in(L - 2), n2 = in(L - 1);
  st[c] = n0; st[C + c] = n1; st[2 * C + c] = n2;
}

struct GdnParams {
  const float* qkv;         // [B*L, 2*Hk*dk + Hv*dv] fp32 after conv+SiLU (q | k | v)
  const __nv_bfloat16* z;   // [B*L, Hv*dv] output gate (pre-SiLU)
  const __nv_bfloat16* a;   // [B*L, Hv]
  const __nv_bfloat16* bb;  // [B*L, Hv]
  const float* A_log;       // [Hv]
  const float* dt_bias;     // [Hv]
  const float* norm_w;      // [dv]
  float* state;             // [slots, Hv, dk, dv]
  float* ckpt;              // optional [B, L, Hv, dk, dv]
  const int* slot;          // [B]
  __nv_bfloat16* y;         // [B*L, Hv*dv]
  int L, Hk, Hv;
  float eps;
  int z_stride, ab_stride;  // elements between token rows of z and of a / b (they may be column slices of one GEMM output)
};

template <int DK, int DV>
__global__ void __launch_bounds__(DV) gdn_recurrent_kernel(const GdnParams p) {
  pdl_trigger();
  pdl_wait();
  static_assert(DK == 128 && DV == 128, "one thread per state column, four k/q values per lane");
  __shared__ float k_s[DK], q_s[DK];
  __shared__ float red[DV / 32];
  __shared__ float gate_s[2];
  const int b = blockIdx.x / p.Hv, h = blockIdx.x % p.Hv;
  const int slot = p.slot[b];
  if (slot < 0) return;
  const int col = threadIdx.x, lane = col & 31, warp = col >> 5;
  const int hk = h / (p.Hv / p.Hk);
  const int C = 2 * p.Hk * DK + p.Hv * DV;
  float s[DK];
  float* st = p.state + (size_t(slot) * p.Hv + h) * DK * DV;
#pragma unroll
  for (int i = 0; i < DK; ++i) s[i] = st[i * DV + col];
  const float scale = rsqrtf(float(DK));
  const float neg_a = -__expf(p.A_log[h]), dtb = p.dt_bias[h], nw = p.norm_w[col];
  for (int t = 0; t < p.L; ++t) {
    const size_t tok = size_t(b) * p.L + t;
    const float* row = p.qkv + tok * C;
    // warp 0 normalises q, warp 1 normalises k, warp 2 computes the gates
    if (warp < 2) {
      const float* src = row + (warp == 0 ? 0 : p.Hk * DK) + hk * DK;
      const float4 v4 = *reinterpret_cast<const float4*>(src + lane * 4);
      float ss = v4.x * v4.x + v4.y * v4.y + v4.z * v4.z + v4.w * v4.w;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float inv = rsqrtf(ss + 1e-6f) * (warp == 0 ? scale : 1.f);
      float* dst = warp == 0 ? q_s : k_s;
      dst[lane * 4] = v4.x * inv; dst[lane * 4 + 1] = v4.y * inv; dst[lane * 4 + 2] = v4.z * inv; dst[lane * 4 + 3] = v4.w * inv;
    } else if (warp == 2 && lane == 0) {
      const float av = __bfloat162float(p.a[tok * p.ab_stride + h]) + dtb;
      const float sp = av > 20.f ? av : log1pf(__expf(av));
      gate_s[0] = __expf(neg_a * sp);
      gate_s[1] = 1.f / (1.f + __expf(-__bfloat162float(p.bb[tok * p.ab_stride + h])));
    }
    __syncthreads();
    const float decay = gate_s[0], beta = gate_s[1];
    float kv = 0.f;
#pragma unroll
    for (int i = 0; i < DK; ++i) kv = fmaf(s[i], k_s[i], kv);
    const float v = row[2 * p.Hk * DK + h * DV + col];
    const float delta = (v - decay * kv) * beta;
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < DK; ++i) {
      s[i] = fmaf(s[i], decay, k_s[i] * delta);
      o = fmaf(s[i], q_s[i], o);
    }
    // gated RMSNorm over the head's dv outputs
    float ss = o * o;
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sft);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < DV / 32; ++i) tot += red[i];
    const float zg = __bfloat162float(p.z[tok * p.z_stride + h * DV + col]);
    const float yv = o * rsqrtf(tot / float(DV) + p.eps) * nw * (zg / (1.f + __expf(-zg)));
    p.y[tok * p.Hv * DV + h * DV + col] = __float2bfloat16(yv);
    if (p.ckpt) {
      float* ck = p.ckpt + ((size_t(b) * p.L + t) * p.Hv + h) * DK * DV;
#pragma unroll
      for (int i = 0; i < DK; ++i) ck[i * DV + col] = s[i];
    }
    __syncthreads();  // k_s / q_s / red are rewritten by the next token
  }
  if (!p.ckpt) {
#pragma unroll
    for (int i = 0; i < DK; ++i) st[i * DV + col] = s[i];
  }
}

// ---------------------------------------------------------------------------------------------
// Long rows (prefill).  The recurrence is sequential in the token, so the time per token is what counts:
//   1. a parallel pre-pass normalises q and k in place and turns (a, b) into (decay, beta) per token and head;
//   2. the recurrence runs with eight threads per pair of state columns (16 state rows each, partial dot products
//      joined by three shuffles), inputs staged eight tokens at a time through shared memory with cp.async, and no block-wide
//      synchronisation inside a token;
//   3. a parallel post-pass applies the gated RMSNorm to the raw outputs.
// The reference covers long rows with a chunked WY kernel on mma.sync (gdn_prefill_chunk.cu).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gdn_prep_kernel(float* __restrict__ qkv, const __nv_bfloat16* __restrict__ a,
                                                       const __nv_bfloat16* __restrict__ bb, const float* __restrict__ A_log,
                                                       const float* __restrict__ dt_bias, float* __restrict__ gates, int Hk,
                                                       int Hv, int ab_stride) {
  const size_t tok = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int C = 2 * Hk * 128 + Hv * 128;
  float* row = qkv + tok * C;
  for (int vec = warp; vec < 2 * Hk; vec += 8) {  // q heads, then k heads
    float4* p4 = reinterpret_cast<float4*>(row + vec * 128) + lane;
    float4 v = *p4;
    float ss = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss + 1e-6f) * (vec < Hk ? rsqrtf(128.f) : 1.f);
    v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv;
    *p4 = v;
  }
  for (int h = threadIdx.x; h < Hv; h += 256) {
    const float av = __bfloat162float(a[tok * ab_stride + h]) + dt_bias[h];
    const float sp = av > 20.f ? av : log1pf(__expf(av));
    gates[(tok * Hv + h) * 2] = __expf(-__expf(A_log[h]) * sp);
    gates[(tok * Hv + h) * 2 + 1] = 1.f / (1.f + __expf(-__bfloat162float(bb[tok * ab_stride + h])));
  }
}

constexpr int kGdnTC = 8;        // tokens per shared-memory stage
constexpr int kGdnRG = 8;        // threads per pair of state columns (row groups)
constexpr int kGdnRows = 128 / kGdnRG;  // state rows per thread
constexpr int kGdnGS = kGdnRows + 4;    // a 128-vector is stored as row groups kGdnGS floats apart (no bank conflicts)
constexpr int kGdnQK = kGdnRG * kGdnGS;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async8(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}

// qkv holds normalised q and k (gdn_prep_kernel); o_raw [B*L, Hv*128] fp32 receives q . S after each token.
// One CTA = (row, head, half of the 128 state columns): 256 threads = 32 column pairs x 8 row groups.  A thread keeps
// 2 x 16 state values; the k and q values it reads from shared memory serve both of its columns, which halves the
// shared-memory traffic per FMA (the limiter of this kernel), and the two halves of a head run on different SMs.
__global__ void __launch_bounds__(32 * kGdnRG) gdn_prefill_kernel(const float* __restrict__ qkv, const float* __restrict__ gates,
                                                          float* __restrict__ state, const int* __restrict__ slot_of,
                                                          float* __restrict__ o_raw, int L, int Hk, int Hv) {
  __shared__ __align__(16) float q_s[2][kGdnTC][kGdnQK];
  __shared__ __align__(16) float k_s[2][kGdnTC][kGdnQK];
  __shared__ __align__(16) float v_s[2][kGdnTC][64];
  __shared__ __align__(8) float g_s[2][kGdnTC][2];
  const int half = blockIdx.x & 1, bh = blockIdx.x >> 1;
  const int b = bh / Hv, h = bh % Hv;
  const int slot = slot_of[b];
  if (slot < 0) return;
  const int pair = threadIdx.x / kGdnRG, rg = threadIdx.x % kGdnRG;
  const int col = half * 64 + 2 * pair;  // this thread's columns: col, col + 1
  const int hk = h / (Hv / Hk);
  const int C = 2 * Hk * 128 + Hv * 128;
  float* st = state + (size_t(slot) * Hv + h) * 128 * 128;
  float s0[kGdnRows], s1[kGdnRows];
#pragma unroll
  for (int i = 0; i < kGdnRows; ++i) {
    const float2 v = *reinterpret_cast<const float2*>(st + (rg * kGdnRows + i) * 128 + col);
    s0[i] = v.x; s1[i] = v.y;
  }

  auto load_stage = [&](int chunk, int stage) {
    const int t0 = chunk * kGdnTC;
    for (int idx = threadIdx.x; idx < kGdnTC * 80; idx += 32 * kGdnRG) {
      const int tt = idx / 80, r = idx % 80;
      if (t0 + tt >= L) continue;
      const float* row = qkv + (size_t(b) * L + t0 + tt) * C;
      if (r >= 64) {
        const int e4 = r - 64;  // 16 float4 = this half's 64 v values
        cp_async16(&v_s[stage][tt][e4 * 4], row + 2 * Hk * 128 + h * 128 + half * 64 + e4 * 4);
      } else {
        const int which = r >> 5, e4 = r & 31;
        float* dst = (which == 0 ? q_s[stage][tt] : k_s[stage][tt]) + (e4 * 4 / kGdnRows) * kGdnGS + (e4 * 4 % kGdnRows);
        cp_async16(dst, row + (which == 0 ? 0 : Hk * 128) + hk * 128 + e4 * 4);
      }
    }
    if (threadIdx.x < kGdnTC && t0 + int(threadIdx.x) < L)
      cp_async8(&g_s[stage][threadIdx.x][0], gates + ((size_t(b) * L + t0 + threadIdx.x) * Hv + h) * 2);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  const int chunks = (L + kGdnTC - 1) / kGdnTC;
  load_stage(0, 0);
  for (int c = 0; c < chunks; ++c) {
    const int stage = c & 1;
    if (c + 1 < chunks) {
      load_stage(c + 1, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const int n = min(kGdnTC, L - c * kGdnTC);
    for (int tt = 0; tt < n; ++tt) {
      const float* kp = k_s[stage][tt] + rg * kGdnGS;
      const float* qp = q_s[stage][tt] + rg * kGdnGS;
      float kk[kGdnRows];
      float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;  // kv partial sums: a* column 0, b* column 1
#pragma unroll
      for (int i = 0; i < kGdnRows; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kp + i);
        kk[i] = k4.x; kk[i + 1] = k4.y; kk[i + 2] = k4.z; kk[i + 3] = k4.w;
        a0 = fmaf(s0[i], k4.x, a0); a1 = fmaf(s0[i + 1], k4.y, a1);
        a0 = fmaf(s0[i + 2], k4.z, a0); a1 = fmaf(s0[i + 3], k4.w, a1);
        b0 = fmaf(s1[i], k4.x, b0); b1 = fmaf(s1[i + 1], k4.y, b1);
        b0 = fmaf(s1[i + 2], k4.z, b0); b1 = fmaf(s1[i + 3], k4.w, b1);
      }
      float kv0 = a0 + a1, kv1 = b0 + b1;
#pragma unroll
      for (int o = 1; o < kGdnRG; o <<= 1) {
        kv0 += __shfl_xor_sync(0xffffffffu, kv0, o);
        kv1 += __shfl_xor_sync(0xffffffffu, kv1, o);
      }
      const float decay = g_s[stage][tt][0], beta = g_s[stage][tt][1];
      const float2 vv = *reinterpret_cast<const float2*>(&v_s[stage][tt][2 * pair]);
      const float d0 = (vv.x - decay * kv0) * beta, d1 = (vv.y - decay * kv1) * beta;
      a0 = a1 = b0 = b1 = 0.f;  // now the q . S partial sums
#pragma unroll
      for (int i = 0; i < kGdnRows; i += 4) {
        const float4 q4 = *reinterpret_cast<const float4*>(qp + i);
        const float qv[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s0[i + e] = fmaf(s0[i + e], decay, kk[i + e] * d0);
          s1[i + e] = fmaf(s1[i + e], decay, kk[i + e] * d1);
        }
        a0 = fmaf(s0[i], qv[0], a0); a1 = fmaf(s0[i + 1], qv[1], a1);
        a0 = fmaf(s0[i + 2], qv[2], a0); a1 = fmaf(s0[i + 3], qv[3], a1);
        b0 = fmaf(s1[i], qv[0], b0); b1 = fmaf(s1[i + 1], qv[1], b1);
        b0 = fmaf(s1[i + 2], qv[2], b0); b1 = fmaf(s1[i + 3], qv[3], b1);
      }
      float o0 = a0 + a1, o1 = b0 + b1;
#pragma unroll
      for (int o = 1; o < kGdnRG; o <<= 1) {
        o0 += __shfl_xor_sync(0xffffffffu, o0, o);
        o1 += __shfl_xor_sync(0xffffffffu, o1, o);
      }
      if (rg == 0)
        *reinterpret_cast<float2*>(o_raw + ((size_t(b) * L + c * kGdnTC + tt) * Hv + h) * 128 + col) = make_float2(o0, o1);
    }
    __syncthreads();  // the stage is refilled two chunks from now
  }
#pragma unroll
  for (int i = 0; i < kGdnRows; ++i) *reinterpret_cast<float2*>(st + (rg * kGdnRows + i) * 128 + col) = make_float2(s0[i], s1[i]);
}

// y = o * rsqrt(mean(o^2) + eps) * norm_w * silu(z): one warp per (token, head).
__global__ void __launch_bounds__(256) gdn_gated_norm_kernel(const float* __restrict__ o_raw, const __nv_bfloat16* __restrict__ z,
                                                             const float* __restrict__ norm_w, __nv_bfloat16* __restrict__ y,
                                                             size_t pairs, int Hv, float eps, int z_stride) {
  const size_t pair = size_t(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (pair >= pairs) return;
  const int lane = threadIdx.x & 31;
  const size_t tok = pair / Hv;
  const int h = int(pair % Hv);
  const float4 o = *reinterpret_cast<const float4*>(o_raw + pair * 128 + lane * 4);
  float ss = o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w;
#pragma unroll
  for (int sft = 16; sft > 0; sft >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sft);
  const float r = rsqrtf(ss / 128.f + eps);
  const float4 nw = *reinterpret_cast<const float4*>(norm_w + lane * 4);
  const uint2 zr = *reinterpret_cast<const uint2*>(z + tok * z_stride + h * 128 + lane * 4);
  const __nv_bfloat16* zb = reinterpret_cast<const __nv_bfloat16*>(&zr);
  const float ov[4] = {o.x, o.y, o.z, o.w}, wv[4] = {nw.x, nw.y, nw.z, nw.w};
  uint2 out;
  __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&out);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float zg = __bfloat162float(zb[j]);
    ob[j] = __float2bfloat16(ov[j] * r * wv[j] * (zg / (1.f + __expf(-zg))));
  }
  *reinterpret_cast<uint2*>(y + pair * 128 + lane * 4) = out;
}

// After a verify window: state[slot[b]] <- ckpt[b, keep[b]], conv_state likewise (keep = index of the last accepted
// window position).  One CTA per (row, head); rows with slot < 0 are skipped.
__global__ void gdn_select_kernel(const float* __restrict__ ckpt, const float* __restrict__ conv_ckpt,
                                  float* __restrict__ state, float* __restrict__ conv_state, const int* __restrict__ slot,
                                  const int* __restrict__ keep, int L, int Hv, int head_elems, int C) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x / Hv, h = blockIdx.x % Hv;
  const int s = slot[b];
  if (s < 0) return;
  const int t = min(max(keep[b], 0), L - 1);
  const float4* src = reinterpret_cast<const float4*>(ckpt + ((size_t(b) * L + t) * Hv + h) * head_elems);
  float4* dst = reinterpret_cast<float4*>(state + (size_t(s) * Hv + h) * head_elems);
  for (int i = threadIdx.x; i < head_elems / 4; i += blockDim.x) dst[i] = src[i];
  if (h == 0) {
    const float* cs = conv_ckpt + (size_t(b) * L + t) * 3 * C;
    float* cd = conv_state + size_t(s) * 3 * C;
    for (int i = threadIdx.x; i < 3 * C; i += blockDim.x) cd[i] = cs[i];
  }
}

// Host entry of the post-pass for the other translation units of the library (the chunked prefill).
int launch_gdn_gated_norm(const float* o_raw, const void* z, const float* norm_w, void* y, size_t pairs, int Hv, float eps,
                          int z_stride, cudaStream_t stream) {
  gdn_gated_norm_kernel<<<unsigned((pairs + 7) / 8), 256, 0, stream>>>(o_raw, static_cast<const __nv_bfloat16*>(z), norm_w,
                                                                       static_cast<__nv_bfloat16*>(y), pairs, Hv, eps, z_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

}  // namespace mfq

using namespace mfq;

extern "C" int mfq_gdn_conv(const void* x, float* conv_state, const float* w, const int* slot, float* out, float* conv_ckpt,
                            int B, int L, int C, int x_stride, cudaStream_t stream) {
  if (B <= 0 || L <= 0 || C <= 0 || x_stride < C) return -1;
  if (!conv_ckpt && L >= 2 * kConvRun && C % 2 == 0 && x_stride % 2 == 0) {
    gdn_conv_long_kernel<<<dim3((C / 2 + 127) / 128, B, (L + kConvRun - 1) / kConvRun), 128, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), conv_state, w, slot, out, L, C, x_stride);
    launch_kernel(gdn_conv_state_kernel, dim3((C + 255) / 256, B), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x), conv_state, slot, L, C, x_stride);
    return cudaGetLastError() == cudaSuccess ? 0 : -7;
  }
  dim3 grid((C + 255) / 256, B, min(L, 64));
  const int fused_state = (!conv_ckpt && grid.z == 1) ? 1 : 0;  // decode: no second launch
  launch_kernel(gdn_conv_kernel, grid, dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x), conv_state, w, slot, out, conv_ckpt, L, C, x_stride, fused_state);
  if (!conv_ckpt && !fused_state)
    launch_kernel(gdn_conv_state_kernel, dim3((C + 255) / 256, B), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x), conv_state, slot, L, C, x_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

extern "C" int mfq_gdn_recurrent(const float* qkv, const void* z, const void* a, const void* b, const float* A_log,
                                 const float* dt_bias, const float* norm_w, float* state, float* ckpt, const int* slot,
                                 void* y, int B, int L, int Hk, int Hv, int dk, int dv, float eps, int z_stride, int ab_stride,
                                 cudaStream_t stream) {
  if (B <= 0 || L <= 0 || dk != 128 || dv != 128 || Hk <= 0 || Hv % Hk) return -1;
  GdnParams p{qkv, static_cast<const __nv_bfloat16*>(z), static_cast<const __nv_bfloat16*>(a),
              static_cast<const __nv_bfloat16*>(b), A_log, dt_bias, norm_w, state, ckpt, slot,
              static_cast<__nv_bfloat16*>(y), L, Hk, Hv, eps, z_stride, ab_stride};
  launch_kernel(gdn_recurrent_kernel<128, 128>, dim3(B * Hv), dim3(128), 0, stream, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

// Long rows without checkpoints.  qkv is normalised IN PLACE; o_raw [B*L, Hv*128] and gates [B*L, Hv, 2] are fp32 scratch.
extern "C" int mfq_gdn_prefill(float* qkv, const void* z, const void* a, const void* b, const float* A_log, const float* dt_bias,
                               const float* norm_w, float* state, const int* slot, void* y, float* o_raw, float* gates, int B,
                               int L, int Hk, int Hv, int dk, int dv, float eps, int z_stride, int ab_stride,
                               cudaStream_t stream) {
  if (B <= 0 || L <= 0 || dk != 128 || dv != 128 || Hk <= 0 || Hv % Hk || z_stride % 4) return -1;
  const size_t tokens = size_t(B) * L;
  gdn_prep_kernel<<<unsigned(tokens), 256, 0, stream>>>(qkv, static_cast<const __nv_bfloat16*>(a),
                                                         static_cast<const __nv_bfloat16*>(b), A_log, dt_bias, gates, Hk, Hv,
                                                         ab_stride);
  gdn_prefill_kernel<<<B * Hv * 2, 32 * kGdnRG, 0, stream>>>(qkv, gates, state, slot, o_raw, L, Hk, Hv);
  const size_t pairs = tokens * Hv;
  gdn_gated_norm_kernel<<<unsigned((pairs + 7) / 8), 256, 0, stream>>>(o_raw, static_cast<const __nv_bfloat16*>(z), norm_w,
                                                                       static_cast<__nv_bfloat16*>(y), pairs, Hv, eps, z_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

extern "C" int mfq_gdn_select(const float* ckpt, const float* conv_ckpt, float* state, float* conv_state, const int* slot,
                              const int* keep, int B, int L, int Hv, int dk, int dv, int C, cudaStream_t stream) {
  if (B <= 0 || L <= 0 || (dk * dv) % 4) return -1;
  launch_kernel(gdn_select_kernel, dim3(B * Hv), dim3(256), 0, stream, ckpt, conv_ckpt, state, conv_state, slot, keep, L, Hv, dk * dv, C);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}
