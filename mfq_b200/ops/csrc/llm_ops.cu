// Memory-bound building blocks of the decode/prefill step: fused (residual +) RMSNorm + FP8 row
// quantization, SwiGLU + FP8 quantization, RoPE + paged FP8 KV write, paged GQA decode attention with
// split-KV, greedy arg-max, embedding gather and the graph-resident step bookkeeping.
//
// Reference counterparts (all scalar fp16/fp32 kernels without an FP8 path): norm.cu / acc.cu
// (acc_rms_norm_*), activation.cu, qk_rope_kv.cu, paged_kv.cu (paged_attention_decode_*_kernel, split +
// reduce), sampling.cu (greedy arg-max), embedding.cu, acc.cu:465 (decode_graph_commit_kernel).
#include "common.cuh"

#include <cfloat>

namespace mfq {

constexpr float kE4M3Max = 448.f;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide reductions over <= 1024 threads; `red` is 33 floats of shared memory.
template <bool kMax>
__device__ __forceinline__ float block_reduce(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = kMax ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float x = lane < nw ? red[lane] : (kMax ? -FLT_MAX : 0.f);
    x = kMax ? warp_max(x) : warp_sum(x);
    if (lane == 0) red[32] = x;
  }
  __syncthreads();
  return red[32];
}

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float from_e4m3(uint8_t c) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(c, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// ---------------------------------------------------------------------------------------------
// (x [+ residual]) -> RMSNorm * w -> per-row FP8.  One CTA per row.  Values stay in registers
// (up to 8 x 8 elements per thread => H <= 8 * 8 * blockDim), so the row is read once.
// ---------------------------------------------------------------------------------------------
constexpr int kNormVecs = 8;

__global__ void rmsnorm_quant_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                                     __nv_bfloat16* __restrict__ residual_out, const __nv_bfloat16* __restrict__ w,
                                     uint8_t* __restrict__ q_out, float* __restrict__ scale_out,
                                     __nv_bfloat16* __restrict__ y_out, int H, float eps) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[33];
  const size_t row = blockIdx.x;
  const int nvec = H / 8;
  float v[kNormVecs][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kNormVecs; ++i) {
    const int vi = threadIdx.x + i * blockDim.x;
    if (vi < nvec) {
      uint4 a = *reinterpret_cast<const uint4*>(x + row * H + vi * 8);
      const __nv_bfloat16* ab = reinterpret_cast<const __nv_bfloat16*>(&a);
      if (residual) {
        uint4 r = *reinterpret_cast<const uint4*>(residual + row * H + vi * 8);
        const __nv_bfloat16* rb = reinterpret_cast<const __nv_bfloat16*>(&r);
        uint4 o;
        __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ob[j] = __float2bfloat16(__bfloat162float(ab[j]) + __bfloat162float(rb[j]));
          v[i][j] = __bfloat162float(ob[j]);
        }
        *reinterpret_cast<uint4*>(residual_out + row * H + vi * 8) = o;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(ab[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  const float rstd = rsqrtf(block_reduce<false>(ss, red) / float(H) + eps);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < kNormVecs; ++i) {
    const int vi = threadIdx.x + i * blockDim.x;
    if (vi < nvec) {
      uint4 ww = *reinterpret_cast<const uint4*>(w + vi * 8);
      const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(&ww);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // round through bf16 like an unfused norm would, so fused and unfused paths agree bit for bit
        v[i][j] = __bfloat162float(__float2bfloat16(v[i][j] * rstd * __bfloat162float(wb[j])));
        amax = fmaxf(amax, fabsf(v[i][j]));
      }
    }
  }
  amax = block_reduce<true>(amax, red);
  const float scale = fmaxf(amax, 1e-12f) / kE4M3Max;
  const float inv = 1.f / scale;
  if (threadIdx.x == 0 && scale_out) scale_out[row] = scale;
#pragma unroll
  for (int i = 0; i < kNormVecs; ++i) {
    const int vi = threadIdx.x + i * blockDim.x;
    if (vi < nvec) {
      if (q_out) {
        uint2 o;
        uint8_t* ob = reinterpret_cast<uint8_t*>(&o);
#pragma unroll
        for (int j = 0; j < 8; ++j) ob[j] = to_e4m3(v[i][j] * inv);
        *reinterpret_cast<uint2*>(q_out + row * H + vi * 8) = o;
      }
      if (y_out) {
        uint4 o;
        __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
        for (int j = 0; j < 8; ++j) ob[j] = __float2bfloat16(v[i][j]);
        *reinterpret_cast<uint4*>(y_out + row * H + vi * 8) = o;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Row quantization.  mode 0: y = x[row, :K]; mode 1 (SwiGLU): y = silu(x[row, :K]) * x[row, K:2K];
// mode 2 (attention output gate): y = x[row, :K] * sigmoid(x2[row, :K]) with x2 a second, separately strided tensor.
// Two passes over the (cache-resident) row: amax, then encode.
// ---------------------------------------------------------------------------------------------
template <int kMode>
__global__ void quant_rows_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q_out,
                                  float* __restrict__ scale_out, int K, int in_stride,
                                  const __nv_bfloat16* __restrict__ x2 = nullptr, int x2_stride = 0) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[33];
  const size_t row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * in_stride;
  const __nv_bfloat16* gr = kMode == 2 ? x2 + row * x2_stride : nullptr;
  const int nvec = K / 8;
  auto value = [&](int vi, float (&y)[8]) {
    uint4 a = *reinterpret_cast<const uint4*>(xr + vi * 8);
    const __nv_bfloat16* ab = reinterpret_cast<const __nv_bfloat16*>(&a);
    if (kMode == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = __bfloat162float(ab[j]);
    } else if (kMode == 2) {
      uint4 b = *reinterpret_cast<const uint4*>(gr + vi * 8);
      const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(&b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float h = __bfloat162float(ab[j]) / (1.f + __expf(-__bfloat162float(bb[j])));
        y[j] = __bfloat162float(__float2bfloat16(h));
      }
    } else {
      uint4 b = *reinterpret_cast<const uint4*>(xr + K + vi * 8);
      const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(&b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float g = __bfloat162float(ab[j]);
        const float h = g / (1.f + __expf(-g)) * __bfloat162float(bb[j]);
        y[j] = __bfloat162float(__float2bfloat16(h));
      }
    }
  };
  float amax = 0.f;
  for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
    float y[8];
    value(vi, y);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(y[j]));
  }
  amax = block_reduce<true>(amax, red);
  const float scale = fmaxf(amax, 1e-12f) / kE4M3Max;
  const float inv = 1.f / scale;
  if (threadIdx.x == 0) scale_out[row] = scale;
  for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
    float y[8];
    value(vi, y);
    uint2 o;
    uint8_t* ob = reinterpret_cast<uint8_t*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) ob[j] = to_e4m3(y[j] * inv);
    *reinterpret_cast<uint2*>(q_out + row * K + vi * 8) = o;
  }
}


// SwiGLU + row quantization for decode-sized batches, one ROW PER CLUSTER of kSplit CTAs: with one CTA per row a batch
// of 64 rows occupies 64 of 148 SMs and every thread walks its slice twice (amax, then encode, the SiLU evaluated both
// times).  Here a CTA owns 1/kSplit of the row, keeps its products in registers, and the row maximum is met through
// distributed shared memory (one float per CTA, two cluster barriers).
constexpr int kSwigluSplit = 4;
constexpr int kSwigluVecs = 2;  // 16-byte vectors per thread: covers K <= 8 * 256 * kSwigluVecs * kSwigluSplit
__global__ void __cluster_dims__(kSwigluSplit, 1, 1) __launch_bounds__(256)
silu_mul_quant_split_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q_out, float* __restrict__ scale_out,
                            int K, int in_stride) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[33];
  __shared__ float part_max;
  const size_t row = blockIdx.x / kSwigluSplit;
  const int part = blockIdx.x % kSwigluSplit;
  const __nv_bfloat16* xr = x + row * in_stride;
  const int nvec = K / 8 / kSwigluSplit, v0 = part * nvec;
  float y[kSwigluVecs][8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < kSwigluVecs; ++i) {
    const int vi = threadIdx.x + i * 256;
    if (vi < nvec) {
      const uint4 a = *reinterpret_cast<const uint4*>(xr + (v0 + vi) * 8);
      const uint4 b = *reinterpret_cast<const uint4*>(xr + K + (v0 + vi) * 8);
      const __nv_bfloat16* ab = reinterpret_cast<const __nv_bfloat16*>(&a);
      const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(&b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float g = __bfloat162float(ab[j]);
        y[i][j] = __bfloat162float(__float2bfloat16(g / (1.f + __expf(-g)) * __bfloat162float(bb[j])));
        amax = fmaxf(amax, fabsf(y[i][j]));
      }
    }
  }
  amax = block_reduce<true>(amax, red);
  if (threadIdx.x == 0) part_max = amax;
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  float row_max = 0.f;
#pragma unroll
  for (int r = 0; r < kSwigluSplit; ++r) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(&part_max)), "r"(r));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    row_max = fmaxf(row_max, v);
  }
  // nobody leaves (and gives up its shared memory) while a peer may still read it
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  const float scale = fmaxf(row_max, 1e-12f) / kE4M3Max, inv = 1.f / scale;
  if (part == 0 && threadIdx.x == 0) scale_out[row] = scale;
#pragma unroll
  for (int i = 0; i < kSwigluVecs; ++i) {
    const int vi = threadIdx.x + i * 256;
    if (vi < nvec) {
      uint2 o;
      uint8_t* ob = reinterpret_cast<uint8_t*>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j) ob[j] = to_e4m3(y[i][j] * inv);
      *reinterpret_cast<uint2*>(q_out + row * K + (v0 + vi) * 8) = o;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// RoPE (rotate-half pairing i <-> i + rot/2 over the first `rot` dims) on Q and K, then K/V -> FP8 pages.
// qkv: [T, (Hq + 2 Hk) * D] bf16.  One warp per (token, head).  Cache page layout [page][Hk][page_size][D]
// with one fp32 multiplier per (page, head, slot).  slots[t] = physical page * page_size + offset (< 0: skip).
// ---------------------------------------------------------------------------------------------
// YaRN context extension: rotary pair `fi` keeps its frequency below `low`, is slowed down by `factor` above `high`,
// blended linearly in between; cos / sin carry `mscale`.  factor == 1 leaves the frequencies bit-identical.
struct RopeScale {
  float factor, low, high, mscale;
};

__device__ __forceinline__ float rope_inv_freq(float log2_theta, int fi, int rot, const RopeScale& y) {
  float f = exp2f(-log2_theta * (2.f * fi) / float(rot));
  if (y.factor != 1.f) {
    const float ramp = fminf(fmaxf((float(fi) - y.low) / (y.high - y.low), 0.f), 1.f);
    f *= (1.f - ramp) + ramp / y.factor;
  }
  return f;
}

template <int D>
__global__ void rope_kv_write_kernel(const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ slots, __nv_bfloat16* __restrict__ q_out,
                                     uint8_t* __restrict__ k_cache, uint8_t* __restrict__ v_cache,
                                     float* __restrict__ k_scale, float* __restrict__ v_scale, int T, int Hq, int Hk,
                                     int page_size, int rot, float log2_theta, __nv_bfloat16* __restrict__ kd_out,
                                     __nv_bfloat16* __restrict__ vd_out, const float* __restrict__ q_norm_w,
                                     const float* __restrict__ k_norm_w, float norm_eps, int row_stride,
                                     const RopeScale ys) {
  pdl_trigger();
  pdl_wait();
  constexpr int EPL = D / 32;  // elements per lane
  const int warps_per_block = blockDim.x >> 5;
  const int gw = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = Hq + 2 * Hk;
  if (gw >= T * heads) return;
  const int t = gw / heads, h = gw % heads;
  const __nv_bfloat16* src = qkv + size_t(t) * row_stride + size_t(h) * D;  // rows may carry extra trailing columns
  // lane owns EPL/2 rotation pairs: indices j and j + rot/2 for j = lane*EPL/2 .. (only when below rot/2),
  // plus pass-through of non-rotated dims; simplest uniform scheme: lane handles dims
  // [lane*EPL/2, lane*EPL/2 + EPL/2) of each half of the head vector.
  constexpr int HP = EPL / 2;
  float lo[HP], hi[HP];
  // explicit vector loads: with a run-time row stride the compiler can no longer prove the alignment itself
  // (the host entry checks that the stride is a multiple of 8 elements)
  auto load_half = [&](const __nv_bfloat16* ptr, float (&dst)[HP]) {
    if constexpr (HP == 2) {
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(ptr);
      dst[0] = __bfloat162float(v.x);
      dst[1] = __bfloat162float(v.y);
    } else if constexpr (HP == 4) {
      const uint2 raw = *reinterpret_cast<const uint2*>(ptr);
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) dst[j] = __bfloat162float(e[j]);
    } else {
#pragma unroll
      for (int j = 0; j < HP; ++j) dst[j] = __bfloat162float(ptr[j]);
    }
  };
  load_half(src + lane * HP, lo);
  load_half(src + D / 2 + lane * HP, hi);
  const bool is_v = h >= Hq + Hk;
  // optional per-head RMSNorm of q and k before the rotation (QK-norm); nw_scale folds 1/rms into the partner reads
  const float* nw = is_v ? nullptr : (h < Hq ? q_norm_w : k_norm_w);
  float inv_rms = 1.f;
  if (nw) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < HP; ++j) ss += lo[j] * lo[j] + hi[j] * hi[j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    inv_rms = rsqrtf(ss / float(D) + norm_eps);
#pragma unroll
    for (int j = 0; j < HP; ++j) {
      lo[j] *= inv_rms * nw[lane * HP + j];
      hi[j] *= inv_rms * nw[D / 2 + lane * HP + j];
    }
  }
  if (!is_v) {
    const float pos = float(positions[t]);
    const int half_rot = rot / 2;
    if (rot == D) {
#pragma unroll
      for (int j = 0; j < HP; ++j) {
        const int idx = lane * HP + j;
        const float inv_freq = rope_inv_freq(log2_theta, idx, rot, ys);
        float s, c;
        sincosf(pos * inv_freq, &s, &c);
        s *= ys.mscale;
        c *= ys.mscale;
        const float a = lo[j], b = hi[j];
        lo[j] = a * c - b * s;
        hi[j] = b * c + a * s;
      }
    } else {
      // partial rotary: pairs (i, i + rot/2) live inside the first `rot` dims.  Handle through shared
      // exchange-free recomputation: each lane re-reads its partner element.
#pragma unroll
      for (int j = 0; j < HP; ++j) {
        for (int part = 0; part < 2; ++part) {
          const int idx = (part ? D / 2 : 0) + lane * HP + j;
          if (idx < rot) {
            const int fi = idx % half_rot;
            const float inv_freq = rope_inv_freq(log2_theta, fi, rot, ys);
            float s, c;
            sincosf(pos * inv_freq, &s, &c);
            s *= ys.mscale;
            c *= ys.mscale;
            const float self = part ? hi[j] : lo[j];
            const int pidx = idx < half_rot ? idx + half_rot : idx - half_rot;
            const float other = __bfloat162float(src[pidx]) * (nw ? inv_rms * nw[pidx] : 1.f);
            const float r = idx < half_rot ? self * c - other * s : self * c + other * s;
            if (part) hi[j] = r; else lo[j] = r;
          }
        }
      }
    }
  }
  if (h < Hq) {
    __nv_bfloat16* dst = q_out + size_t(t) * Hq * D + size_t(h) * D;
#pragma unroll
    for (int j = 0; j < HP; ++j) {
      dst[lane * HP + j] = __float2bfloat16(lo[j]);
      dst[D / 2 + lane * HP + j] = __float2bfloat16(hi[j]);
    }
    return;
  }
  const int slot = slots[t];
  if (slot < 0) return;
  const int kvh = is_v ? h - Hq - Hk : h - Hq;
  const int page = slot / page_size, off = slot % page_size;
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < HP; ++j) {
    lo[j] = __bfloat162float(__float2bfloat16(lo[j]));
    hi[j] = __bfloat162float(__float2bfloat16(hi[j]));
    amax = fmaxf(amax, fmaxf(fabsf(lo[j]), fabsf(hi[j])));
  }
  amax = warp_max(amax);
  const float scale = fmaxf(amax, 1e-12f) / kE4M3Max;
  const float inv = 1.f / scale;
  const size_t base = ((size_t(page) * Hk + kvh) * page_size + off);
  const size_t ph = size_t(page) * Hk + kvh;
  if (!is_v) {
    // K page: [D/64 chunks][page_size tokens][64 dims]
    uint8_t* dst = k_cache + ph * (size_t(page_size) * D);
#pragma unroll
    for (int j = 0; j < HP; ++j) {
      const int d0 = lane * HP + j, d1 = D / 2 + lane * HP + j;
      dst[(d0 >> 6) * (page_size * 64) + off * 64 + (d0 & 63)] = to_e4m3(lo[j] * inv);
      dst[(d1 >> 6) * (page_size * 64) + off * 64 + (d1 & 63)] = to_e4m3(hi[j] * inv);
    }
  } else {
    // V page: [D dims][page_size tokens in the order 0,1,8,9,2,3,10,11,4,5,12,13,6,7,14,15]
    uint8_t* dst = v_cache + ph * (size_t(page_size) * D);
    const int pos = 4 * ((off & 7) >> 1) + 2 * (off >> 3) + (off & 1);
#pragma unroll
    for (int j = 0; j < HP; ++j) {
      dst[(lane * HP + j) * page_size + pos] = to_e4m3(lo[j] * inv);
      dst[(D / 2 + lane * HP + j) * page_size + pos] = to_e4m3(hi[j] * inv);
    }
  }
  // Optional contiguous copy of what the pages now hold (code * multiplier), [T, Hk, D] bf16: the prefill attention
  // of this chunk reads it, so prefill and later decode steps see the same FP8-rounded K/V.
  __nv_bfloat16* dq = is_v ? vd_out : kd_out;
  if (dq) {
    dq += (size_t(t) * Hk + kvh) * D;
#pragma unroll
    for (int j = 0; j < HP; ++j) {
      dq[lane * HP + j] = __float2bfloat16(from_e4m3(to_e4m3(lo[j] * inv)) * scale);
      dq[D / 2 + lane * HP + j] = __float2bfloat16(from_e4m3(to_e4m3(hi[j] * inv)) * scale);
    }
  }
  if (lane == 0) (is_v ? v_scale : k_scale)[base] = scale;
}

// ---------------------------------------------------------------------------------------------
// Greedy sampling: arg-max over the vocabulary, one CTA per row (lowest index wins ties).
// ---------------------------------------------------------------------------------------------
__global__ void argmax_kernel(const __nv_bfloat16* __restrict__ logits, int* __restrict__ out, int V, int stride) {
  pdl_trigger();
  pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  const __nv_bfloat16* row = logits + size_t(blockIdx.x) * stride;
  float best = -FLT_MAX;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = __bfloat162float(row[i]);
    if (v > best) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -FLT_MAX;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) out[blockIdx.x] = bi;
  }
}

// Wide vocabularies, few rows: the row is split over several CTAs.  Each folds its best (value, index) into a 64-bit
// key -- order-preserving value bits above the inverted index, so the larger value and then the lower index win an
// atomicMax -- and the last CTA of the row to arrive writes the result and clears the row's scratch for the next
// launch.  The scratch is static device memory: nothing to allocate, safe under graph capture; launches that share
// it must be ordered on one stream.
constexpr int kArgmaxRows = 8192;
__device__ unsigned long long g_argmax_key[kArgmaxRows];
__device__ unsigned int g_argmax_count[kArgmaxRows];

__global__ void argmax_split_kernel(const __nv_bfloat16* __restrict__ logits, int* __restrict__ out, int V, int stride) {
  pdl_trigger();
  pdl_wait();
  __shared__ unsigned long long sk[8];
  const int b = blockIdx.x, seg = blockIdx.y, nseg = gridDim.y;
  const int per = (V + nseg - 1) / nseg;
  const int lo = seg * per, hi = min(V, lo + per);
  const __nv_bfloat16* row = logits + size_t(b) * stride;
  unsigned long long key = 0ull;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const uint32_t u = __float_as_uint(__bfloat162float(row[i]));
    const uint32_t ord = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    const unsigned long long k = (static_cast<unsigned long long>(ord) << 32) | (0xffffffffu - uint32_t(i));
    key = k > key ? k : key;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
    key = other > key ? other : key;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sk[warp] = key;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w) key = sk[w] > key ? sk[w] : key;
    atomicMax(&g_argmax_key[b], key);
    __threadfence();
    if (atomicAdd(&g_argmax_count[b], 1u) == uint32_t(nseg - 1)) {
      __threadfence();
      const unsigned long long best = atomicExch(&g_argmax_key[b], 0ull);
      out[b] = int(0xffffffffu - uint32_t(best & 0xffffffffull));
      g_argmax_count[b] = 0u;
    }
  }
}

__global__ void embed_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                             __nv_bfloat16* __restrict__ out, int H) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  const size_t src = size_t(ids[row]);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x)
    reinterpret_cast<uint4*>(out + row * H)[i] = reinterpret_cast<const uint4*>(table + src * H)[i];
}

// Per-step bookkeeping that lives inside the captured decode graph: the sampled token becomes the next
// input, the position advances, the KV slot of the new token is looked up in the page table.
__global__ void decode_advance_kernel(const int* __restrict__ sampled, int* __restrict__ input_ids,
                                      int* __restrict__ positions, int* __restrict__ seq_lens,
                                      int* __restrict__ slots, const int* __restrict__ block_table, int B,
                                      int max_pages, int page_size, const int* __restrict__ active) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  if (active && !active[b]) { slots[b] = -1; return; }
  if (sampled) input_ids[b] = sampled[b];
  const int pos = seq_lens[b];  // position of the token about to be written
  positions[b] = pos;
  const int page = block_table[size_t(b) * max_pages + pos / page_size];
  slots[b] = page * page_size + pos % page_size;
  seq_lens[b] = pos + 1;
}

}  // namespace mfq

using namespace mfq;

extern "C" int mfq_rmsnorm_quant(const void* x, const void* residual, void* residual_out, const void* w, void* q_out,
                                 float* scale_out, void* y_out, int M, int H, float eps, cudaStream_t stream) {
  if (H % 8 || M <= 0) return -1;
  int threads = ((H / 8 + kNormVecs - 1) / kNormVecs + 31) / 32 * 32;
  if (threads < 32) threads = 32;
  if (threads > 1024) return -1;
  // few rows (decode): the kernel is pure latency, so spread a row over as many threads as it has 16-byte vectors
  if (M <= 1024) threads = max(threads, min(512, (H / 8 + 31) / 32 * 32));  // 512: the register file allows no more
  launch_kernel(rmsnorm_quant_kernel, dim3(M), dim3(threads), 0, stream,
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual),
      static_cast<__nv_bfloat16*>(residual_out), static_cast<const __nv_bfloat16*>(w), static_cast<uint8_t*>(q_out),
      scale_out, static_cast<__nv_bfloat16*>(y_out), H, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

extern "C" int mfq_quant_rows(const void* x, void* q_out, float* scale_out, int M, int K, int in_stride, int swiglu,
                              cudaStream_t stream) {
  if (K % 8 || in_stride % 8 || M <= 0) return -1;
  const int threads = K >= 4096 ? 512 : 256;
  if (swiglu && M <= 256 && K % (8 * kSwigluSplit) == 0 && K / 8 / kSwigluSplit <= 256 * kSwigluVecs && K >= 4096) {
    launch_kernel(silu_mul_quant_split_kernel, dim3(M * kSwigluSplit), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x),
                  static_cast<uint8_t*>(q_out), scale_out, K, in_stride);
    return cudaGetLastError() == cudaSuccess ? 0 : -7;
  }
  if (swiglu)
    launch_kernel(quant_rows_kernel<1>, dim3(M), dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q_out), scale_out, K, in_stride, static_cast<const __nv_bfloat16*>(nullptr), 0);
  else
    launch_kernel(quant_rows_kernel<0>, dim3(M), dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q_out), scale_out, K, in_stride, static_cast<const __nv_bfloat16*>(nullptr), 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

// fp8 rows of x * sigmoid(gate): the output gate of gated attention, fused with the quantization that feeds o_proj.
extern "C" int mfq_gate_quant_rows(const void* x, const void* gate, void* q_out, float* scale_out, int M, int K,
                                   int in_stride, int gate_stride, cudaStream_t stream) {
  if (K % 8 || in_stride % 8 || gate_stride % 8 || M <= 0) return -1;
  launch_kernel(quant_rows_kernel<2>, dim3(M), dim3(K >= 4096 ? 512 : 256), 0, stream, static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q_out),
                                                                scale_out, K, in_stride, static_cast<const __nv_bfloat16*>(gate),
                                                                gate_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

// q_norm_w / k_norm_w ([D] fp32, may be null): per-head RMSNorm of q / k before the rotation; row_stride: elements
// between token rows of qkv (>= (Hq + 2 Hk) * D; an attention output gate may follow the v heads).
// yarn_*: context extension (see RopeScale); factor 1 and mscale 1 are the plain rotation.
extern "C" int mfq_rope_kv_write_yarn(const void* qkv, const int* positions, const int* slots, void* q_out, void* k_cache,
                                      void* v_cache, float* k_scale, float* v_scale, int T, int Hq, int Hk, int D,
                                      int page_size, int rot, float theta, void* kd_out, void* vd_out,
                                      const float* q_norm_w, const float* k_norm_w, float norm_eps, int row_stride,
                                      float yarn_factor, float yarn_low, float yarn_high, float yarn_mscale,
                                      cudaStream_t stream) {
  if (T <= 0 || row_stride < (Hq + 2 * Hk) * D || row_stride % 8) return -1;
  if (!(yarn_factor >= 1.f) || !(yarn_high > yarn_low) || !(yarn_mscale > 0.f)) return -1;
  const int warps = T * (Hq + 2 * Hk);
  const int blocks = (warps + 7) / 8;
  const float l2t = log2f(theta);
  const RopeScale ys{yarn_factor, yarn_low, yarn_high, yarn_mscale};
#define MFQ_ROPE(DD)                                                                                             \
  launch_kernel(rope_kv_write_kernel<DD>, dim3(blocks), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(qkv), positions, slots, \
      static_cast<__nv_bfloat16*>(q_out), static_cast<uint8_t*>(k_cache), static_cast<uint8_t*>(v_cache),      \
      k_scale, v_scale, T, Hq, Hk, page_size, rot, l2t, static_cast<__nv_bfloat16*>(kd_out),                   \
      static_cast<__nv_bfloat16*>(vd_out), q_norm_w, k_norm_w, norm_eps, row_stride, ys)
  if (D == 128) MFQ_ROPE(128);
  else if (D == 64) MFQ_ROPE(64);
  else if (D == 256) MFQ_ROPE(256);
  else return -1;
#undef MFQ_ROPE
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

extern "C" int mfq_rope_kv_write_ex(const void* qkv, const int* positions, const int* slots, void* q_out, void* k_cache,
                                    void* v_cache, float* k_scale, float* v_scale, int T, int Hq, int Hk, int D,
                                    int page_size, int rot, float theta, void* kd_out, void* vd_out,
                                    const float* q_norm_w, const float* k_norm_w, float norm_eps, int row_stride,
                                    cudaStream_t stream) {
  return mfq_rope_kv_write_yarn(qkv, positions, slots, q_out, k_cache, v_cache, k_scale, v_scale, T, Hq, Hk, D, page_size,
                                rot, theta, kd_out, vd_out, q_norm_w, k_norm_w, norm_eps, row_stride, 1.f, 0.f, 1.f, 1.f,
                                stream);
}

extern "C" int mfq_rope_kv_write(const void* qkv, const int* positions, const int* slots, void* q_out, void* k_cache,
                                 void* v_cache, float* k_scale, float* v_scale, int T, int Hq, int Hk, int D,
                                 int page_size, int rot, float theta, void* kd_out, void* vd_out,
                                 cudaStream_t stream) {
  return mfq_rope_kv_write_ex(qkv, positions, slots, q_out, k_cache, v_cache, k_scale, v_scale, T, Hq, Hk, D, page_size, rot,
                              theta, kd_out, vd_out, nullptr, nullptr, 0.f, (Hq + 2 * Hk) * D, stream);
}

extern "C" int mfq_argmax(const void* logits, int* out, int B, int V, int stride, cudaStream_t stream) {
  const int segs = V / 4096 > 32 ? 32 : V / 4096;
  if (segs >= 2 && B <= kArgmaxRows && B * segs <= 4096)
    launch_kernel(argmax_split_kernel, dim3(B, segs), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(logits), out, V, stride);
  else
    launch_kernel(argmax_kernel, dim3(B), dim3(1024), 0, stream, static_cast<const __nv_bfloat16*>(logits), out, V, stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

extern "C" int mfq_embed(const int* ids, const void* table, void* out, int T, int H, cudaStream_t stream) {
  if (H % 8) return -1;
  launch_kernel(embed_kernel, dim3(T), dim3(128), 0, stream, ids, static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), H);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

extern "C" int mfq_decode_advance(const int* sampled, int* input_ids, int* positions, int* seq_lens, int* slots,
                                  const int* block_table, int B, int max_pages, int page_size, const int* active,
                                  cudaStream_t stream) {
  launch_kernel(decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, sampled, input_ids, positions, seq_lens, slots,
                                                             block_table, B, max_pages, page_size, active);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

// ---------------------------------------------------------------------------------------------
// SwiGLU without quantization: out[row, :I] = silu(x[row, :I]) * x[row, I:2I] in bf16 (input of bf16-activation GEMMs).
// ---------------------------------------------------------------------------------------------
namespace mfq {
__global__ void silu_mul_bf16_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int I, int in_stride) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * in_stride;
  for (int v = threadIdx.x; v < I / 8; v += blockDim.x) {
    const uint4 a = *reinterpret_cast<const uint4*>(xr + v * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(xr + I + v * 8);
    const __nv_bfloat16* ab = reinterpret_cast<const __nv_bfloat16*>(&a);
    const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(&b);
    uint4 o;
    __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float g = __bfloat162float(ab[j]);
      ob[j] = __float2bfloat16(g / (1.f + __expf(-g)) * __bfloat162float(bb[j]));
    }
    *reinterpret_cast<uint4*>(out + row * I + v * 8) = o;
  }
}
}  // namespace mfq

extern "C" int mfq_silu_mul_bf16(const void* x, void* out, int M, int I, int in_stride, cudaStream_t stream) {
  if (M <= 0 || I % 8 || in_stride % 8) return -1;
  mfq::launch_kernel(mfq::silu_mul_bf16_kernel, dim3(M), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x),
                     static_cast<__nv_bfloat16*>(out), I, in_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

// ---------------------------------------------------------------------------------------------
// Past K/V of one sequence out of the FP8 pages into contiguous bf16 [T, Hk, D] (code * multiplier): the keys /
// values a later prefill chunk attends to (chunked prefill, restored prefix).  One warp per (token, KV head).
// ---------------------------------------------------------------------------------------------
namespace mfq {
template <int D>
__global__ void kv_gather_dequant_kernel(const uint8_t* __restrict__ k_cache, const uint8_t* __restrict__ v_cache,
                                         const float* __restrict__ k_scale, const float* __restrict__ v_scale,
                                         const int* __restrict__ block_row, __nv_bfloat16* __restrict__ kd,
                                         __nv_bfloat16* __restrict__ vd, int T, int Hk, int page_size) {
  pdl_trigger();
  pdl_wait();
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (gw >= T * Hk) return;
  const int t = gw / Hk, h = gw % Hk;
  const int page = block_row[t / page_size], off = t % page_size;
  const size_t ph = size_t(page) * Hk + h;
  const float ks = k_scale[ph * page_size + off], vs = v_scale[ph * page_size + off];
  const uint8_t* kp = k_cache + ph * (size_t(page_size) * D);
  const uint8_t* vp = v_cache + ph * (size_t(page_size) * D);
  const int pos = 4 * ((off & 7) >> 1) + 2 * (off >> 3) + (off & 1);  // slot of the token inside a V page
  __nv_bfloat16* ko = kd + (size_t(t) * Hk + h) * D;
  __nv_bfloat16* vo = vd + (size_t(t) * Hk + h) * D;
  for (int d = lane; d < D; d += 32) {
    ko[d] = __float2bfloat16(from_e4m3(kp[(d >> 6) * (page_size * 64) + off * 64 + (d & 63)]) * ks);
    vo[d] = __float2bfloat16(from_e4m3(vp[d * page_size + pos]) * vs);
  }
}
}  // namespace mfq

// block_row: the sequence's page ids ([ceil(T / page_size)] int32, device); kd / vd: [T, Hk, D] bf16.
extern "C" int mfq_kv_gather_dequant(const void* k_cache, const void* v_cache, const float* k_scale, const float* v_scale,
                                     const int* block_row, void* kd, void* vd, int T, int Hk, int D, int page_size,
                                     cudaStream_t stream) {
  if (T <= 0 || Hk <= 0 || page_size != 16) return -1;
  const int blocks = (T * Hk + 7) / 8;
#define MFQ_GATHER(DD)                                                                                              \
  mfq::launch_kernel(mfq::kv_gather_dequant_kernel<DD>, dim3(blocks), dim3(256), 0, stream,                        \
                     static_cast<const uint8_t*>(k_cache), static_cast<const uint8_t*>(v_cache), k_scale, v_scale,  \
                     block_row, static_cast<__nv_bfloat16*>(kd), static_cast<__nv_bfloat16*>(vd), T, Hk, page_size)
  if (D == 128) MFQ_GATHER(128);
  else if (D == 64) MFQ_GATHER(64);
  else if (D == 256) MFQ_GATHER(256);
  else return -1;
#undef MFQ_GATHER
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}
