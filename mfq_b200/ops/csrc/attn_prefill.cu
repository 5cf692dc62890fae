// Causal self-attention for prefill chunks on tcgen05 tensor cores (bf16 in, fp32 accumulate, head dim 128, GQA).
//
// One CTA = (128-query block, query head).  Per 128-key block:
//   S = Q K^T      tcgen05.mma kind::f16, A = Q tile, B = K tile (both K-major, TMA 128 B swizzle), S in TMEM
//   P = softmax    8 warps, two threads per query row (64 keys each): two passes over the TMEM row (max, then
//                  exp2 + sum), row maxima exchanged through shared memory,
//                  P written as bf16 into shared memory in the swizzled K-major layout the next MMA expects
//   O_blk = P V    tcgen05.mma with V as an MN-major B operand (the [key][dim] tile exactly as TMA delivers it)
//   O = (O + O_blk(prev)) * alpha   folded in fp32 registers, so TMEM never needs an in-place rescale
// The MMA warp issues Q K^T of block j+1 before P V of block j (S is double-buffered in TMEM), so the tensor core
// works while the softmax warps are busy.  Heaviest (latest) query blocks are scheduled first.
//
// The reference's prefill attention is a llama.cpp-derived mma.sync flash-attention (mfq_fattn_mma_f16.cuh) and a
// wmma D=256 kernel (attention.cu:218).
#include "common.cuh"

#include <cfloat>

namespace mfq {

constexpr int kQB = 128, kKB = 128, kHD = 128;
constexpr int kTileBytes = kQB * kHD * 2;       // 32 KB: one [128 x 128] bf16 tile = two 16 KB swizzled halves
constexpr int kHalfBytes = kTileBytes / 2;
constexpr int kPrefillThreads = 64 + 8 * 32;  // TMA warp, MMA warp, 8 softmax warps
constexpr int kPrefillSmem = kTileBytes /*Q*/ + 2 * 2 * kTileBytes /*K,V x 2 stages*/ + kTileBytes /*P*/ + 1024 + 256 + 6 * kQB * 4 /*row max / sum exchange*/;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct PrefillParams {
  __nv_bfloat16* out;  // [T, Hq, 128]
  int T, Hq, Hk;       // T: query rows
  int Tk, offset;      // keys available; query row i sees keys 0 .. i + offset (offset = Tk - T: tokens before the chunk)
  float scale_log2;
  int* status;
};

__global__ void __launch_bounds__(kPrefillThreads, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const PrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = base;
  uint8_t* sKV = base + kTileBytes;                 // stage s: K at sKV + s*2*tile, V right after it
  uint8_t* sP = sKV + 4 * kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kTileBytes);
  uint64_t* q_full = bars;            // 1
  uint64_t* kv_full = bars + 1;       // [2]
  uint64_t* kv_empty = bars + 3;      // [2]
  uint64_t* s_full = bars + 5;        // [2]
  uint64_t* s_empty = bars + 7;       // [2] (8 arrivals: one per softmax warp)
  uint64_t* p_full = bars + 9;        // 8 arrivals
  uint64_t* pv_full = bars + 10;      // commit
  uint64_t* o_empty = bars + 11;      // 8 arrivals
  uint64_t* x_bar = bars + 12;        // 8 arrivals: row-max exchange, one phase per key block
  uint64_t* l_bar = bars + 13;        // 8 arrivals: row-sum exchange, once
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_max = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);  // max: [2 buffers][2 halves][128 rows]; sum: [2 halves][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_qb = (p.T + kQB - 1) / kQB;
  const int qb = num_qb - 1 - blockIdx.x;  // heavy blocks first
  const int hq = blockIdx.y;
  const int kvh = hq / (p.Hq / p.Hk);
  // causal with a past: the last query of the block sees keys up to (qb + 1) * kQB - 1 + offset
  const int nblk = min((p.Tk + kKB - 1) / kKB, ((qb + 1) * kQB + p.offset + kKB - 1) / kKB);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 8);
    }
    mbar_init(p_full, 8); mbar_init(pv_full, 1); mbar_init(o_empty, 8); mbar_init(x_bar, 8); mbar_init(l_bar, 8);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS[2] = {tmem_base, tmem_base + 128};
  const uint32_t tO = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v);
      mbar_expect_tx(q_full, kTileBytes);
      tma_load_2d(sQ, &tmap_q, q_full, hq * kHD, qb * kQB);
      tma_load_2d(sQ + kHalfBytes, &tmap_q, q_full, hq * kHD + 64, qb * kQB);
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutProducer)) break;
        uint8_t* k = sKV + s * 2 * kTileBytes;
        uint8_t* v = k + kTileBytes;
        mbar_expect_tx(&kv_full[s], 2 * kTileBytes);
        tma_load_2d(k, &tmap_k, &kv_full[s], kvh * kHD, j * kKB);
        tma_load_2d(k + kHalfBytes, &tmap_k, &kv_full[s], kvh * kHD + 64, j * kKB);
        tma_load_2d(v, &tmap_v, &kv_full[s], kvh * kHD, j * kKB);
        tma_load_2d(v + kHalfBytes, &tmap_v, &kv_full[s], kvh * kHD + 64, j * kKB);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(128, 128, 1, 1, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc(128, 128, 1, 1, 0, 1);  // B = V is MN-major
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto issue_qk = [&](int j) {
        const uint32_t k_addr = smem_u32(sKV + (j & 1) * 2 * kTileBytes);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {  // 8 x 16 dims; dims 64.. live in the second swizzled half
          const uint32_t off = (ks >> 2) * kHalfBytes + (ks & 3) * 32;
          umma_f16(tS[j & 1], umma_desc_k_sw128(q_addr + off), umma_desc_k_sw128(k_addr + off), idesc_qk, ks > 0);
        }
        tc_commit(&s_full[j & 1]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kStatusTimeoutMma) &&
                mbar_wait(&kv_full[0], 0, abort_flag, p.status, kStatusTimeoutMma);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; ok && j < nblk; ++j) {
        if (j + 1 < nblk) {
          const int s1 = (j + 1) & 1;
          ok = mbar_wait(&kv_full[s1], ((j + 1) >> 1) & 1, abort_flag, p.status, kStatusTimeoutMma) &&
               mbar_wait(&s_empty[s1], (((j + 1) >> 1) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutMma);
          if (!ok) break;
          tc_fence_after();
          issue_qk(j + 1);
        }
        ok = mbar_wait(p_full, j & 1, abort_flag, p.status, kStatusTimeoutMma) &&
             mbar_wait(o_empty, (j & 1) ^ 1, abort_flag, p.status, kStatusTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sKV + (j & 1) * 2 * kTileBytes + kTileBytes);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {  // 8 x 16 keys
          const uint32_t a_off = (ks >> 2) * kHalfBytes + (ks & 3) * 32;  // P: K-major over keys
          umma_f16(tO, umma_desc_k_sw128(p_addr + a_off), umma_desc_mn_sw128(v_addr + ks * 2048, kHalfBytes), idesc_pv,
                   ks > 0);
        }
        tc_commit(pv_full);
        tc_commit(&kv_empty[j & 1]);
      }
    }
  } else {
    // ----- softmax warps: two threads per query row (TMEM lane); `half` selects 64 of the 128 key columns of S/P
    // and 64 of the 128 output dims, so every scheduler has two warps to interleave -----
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int q_idx = qb * kQB + row;
    const uint32_t lane_base = (uint32_t(quarter * 32) << 16) + uint32_t(half * 64);
    float o[64];
#pragma unroll
    for (int d = 0; d < 64; ++d) o[d] = 0.f;
    float m_run = -FLT_MAX, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      const int sb = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[sb], (j >> 1) & 1, abort_flag, p.status, kStatusTimeoutEpilogue));
      if (!ok) break;
      tc_fence_after();
      const int key0 = j * kKB + half * 64;
      // masking is needed where the block reaches past the FIRST query's horizon or past the last key
      const bool diag = ((j + 1) * kKB - 1 > qb * kQB + p.offset) || ((j + 1) * kKB > p.Tk);
      // pass 1: maximum over this thread's 64 columns, then exchange with the partner thread of the row
      float mx = -FLT_MAX;
      {
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(tS[sb] + lane_base, r0);
        tmem_ld_32x32(tS[sb] + lane_base + 32, r1);
        tmem_wait_ld();
        if (!diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(r0[i]), __uint_as_float(r1[i])));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int ka = key0 + i, kb = key0 + 32 + i;
            mx = fmaxf(mx, (ka <= q_idx + p.offset && ka < p.Tk) ? __uint_as_float(r0[i]) : -FLT_MAX);
            mx = fmaxf(mx, (kb <= q_idx + p.offset && kb < p.Tk) ? __uint_as_float(r1[i]) : -FLT_MAX);
          }
        }
      }
      s_max[(sb * 2 + half) * kQB + row] = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(x_bar);
      ok = __all_sync(0xffffffffu, mbar_wait(x_bar, j & 1, abort_flag, p.status, kStatusTimeoutEpilogue));
      if (!ok) break;
      mx = fmaxf(mx, s_max[(sb * 2 + (half ^ 1)) * kQB + row]);
      const float m_new = fmaxf(m_run, mx);
      const float alpha = fast_exp2((m_run - m_new) * p.scale_log2);
      // fold the previous block's P.V (it was computed against m_run), then move to the new maximum
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(pv_full, (j - 1) & 1, abort_flag, p.status, kStatusTimeoutEpilogue));
        if (!ok) break;
        tc_fence_after();
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(tO + lane_base, r0);
        tmem_ld_32x32(tO + lane_base + 32, r1);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          o[i] = (o[i] + __uint_as_float(r0[i])) * alpha;
          o[32 + i] = (o[32 + i] + __uint_as_float(r1[i])) * alpha;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(o_empty);
      }
      l_run *= alpha;
      m_run = m_new;
      // pass 2: probabilities -> bf16 -> this thread's half of the swizzled K-major P tile
      const float mb = m_new * p.scale_log2;
      float psum = 0.f;
      uint8_t* prow = sP + half * kHalfBytes + row * 128;
#pragma unroll
      for (int c = 0; c < 64; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tS[sb] + lane_base + c, r);
        tmem_wait_ld();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = fast_exp2(fmaf(__uint_as_float(r[i]), p.scale_log2, -mb));
          float p1 = fast_exp2(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, -mb));
          if (diag) {
            const int key = key0 + c + i;
            if (!(key <= q_idx + p.offset && key < p.Tk)) p0 = 0.f;
            if (!(key + 1 <= q_idx + p.offset && key + 1 < p.Tk)) p1 = 0.f;
          }
          psum += p0 + p1;
          __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
        }
        // 32 keys = 4 chunks of 16 bytes; the chunk index within the 128 B row is XORed with (row % 8)
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int chunk = ((c >> 3) + ch) ^ (row & 7);
          *reinterpret_cast<uint4*>(prow + chunk * 16) =
              make_uint4(packed[ch * 4], packed[ch * 4 + 1], packed[ch * 4 + 2], packed[ch * 4 + 3]);
        }
      }
      l_run += psum;
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s_empty[sb]); mbar_arrive(p_full); }
    }
    if (ok) {
      // total row sum = both halves
      s_max[(4 + half) * kQB + row] = l_run;  // own slots: the last block's maxima may still be read
      __syncwarp();
      if (lane == 0) mbar_arrive(l_bar);
      ok = __all_sync(0xffffffffu, mbar_wait(l_bar, 0, abort_flag, p.status, kStatusTimeoutEpilogue)) &&
           __all_sync(0xffffffffu, mbar_wait(pv_full, (nblk - 1) & 1, abort_flag, p.status, kStatusTimeoutEpilogue));
      if (ok) {
        tc_fence_after();
        const float l_tot = l_run + s_max[(4 + (half ^ 1)) * kQB + row];
        const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
        __nv_bfloat16* dst = p.out + (size_t(q_idx) * p.Hq + hq) * kHD + half * 64;
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(tO + lane_base, r0);
        tmem_ld_32x32(tO + lane_base + 32, r1);
        tmem_wait_ld();
        if (q_idx < p.T) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 va, vb;
            __nv_bfloat162* ha = reinterpret_cast<__nv_bfloat162*>(&va);
            __nv_bfloat162* hb = reinterpret_cast<__nv_bfloat162*>(&vb);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              ha[e] = __floats2bfloat162_rn((o[i + 2 * e] + __uint_as_float(r0[i + 2 * e])) * inv,
                                            (o[i + 2 * e + 1] + __uint_as_float(r0[i + 2 * e + 1])) * inv);
              hb[e] = __floats2bfloat162_rn((o[32 + i + 2 * e] + __uint_as_float(r1[i + 2 * e])) * inv,
                                            (o[32 + i + 2 * e + 1] + __uint_as_float(r1[i + 2 * e + 1])) * inv);
            }
            *reinterpret_cast<uint4*>(dst + i) = va;
            *reinterpret_cast<uint4*>(dst + 32 + i) = vb;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace mfq

// q: [T, Hq, 128] bf16, k/v: [Tk, Hk, 128] bf16 (contiguous), out: [T, Hq, 128] bf16.  Tk >= T: the first Tk - T keys
// are the sequence's past (earlier chunks / a restored prefix); query i attends to keys 0 .. i + (Tk - T).
extern "C" int mfq_attn_prefill_past(const void* q, const void* k, const void* v, void* out, int T, int Tk, int Hq, int Hk,
                                     int D, float sm_scale, int* status, cudaStream_t stream) {
  using namespace mfq;
  if (D != 128 || T <= 0 || Tk < T || Hq % Hk) return -1;
  CUtensorMap tq, tk, tv;
  if (make_tmap_2d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, uint64_t(Hq) * D, uint64_t(Hq) * D * 2, kQB, 64)) return -2;
  if (make_tmap_2d(&tk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tk, uint64_t(Hk) * D, uint64_t(Hk) * D * 2, kKB, 64)) return -3;
  if (make_tmap_2d(&tv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tk, uint64_t(Hk) * D, uint64_t(Hk) * D * 2, kKB, 64)) return -4;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmem) != cudaSuccess) return -6;
    attr = true;
  }
  PrefillParams p{static_cast<__nv_bfloat16*>(out), T, Hq, Hk, Tk, Tk - T, sm_scale * 1.4426950408889634f, status};
  attn_prefill_kernel<<<dim3((T + kQB - 1) / kQB, Hq), kPrefillThreads, kPrefillSmem, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

// Self-contained chunk (no past): Tk = T.
extern "C" int mfq_attn_prefill_bf16(const void* q, const void* k, const void* v, void* out, int T, int Hq, int Hk,
                                     int D, float sm_scale, int* status, cudaStream_t stream) {
  return mfq_attn_prefill_past(q, k, v, out, T, T, Hq, Hk, D, sm_scale, status, stream);
}
