// Causal prefill attention for head dim 256 on tcgen05 tensor cores (bf16 in, fp32 accumulate, GQA, keys may
// include a past).
//
// A 256-wide head does not fit the register-folded output of the 128-wide kernel (attn_prefill.cu), so this
// kernel keeps the output accumulator in TMEM for the whole key loop and rescales it there only when a row
// maximum grew by more than 2^8 since the maximum in use (probabilities are computed against the maximum in
// use, so they stay below 2^8 and the row sum carries the same factor; the final division cancels it).  In a
// causal sweep the maximum settles after the first blocks, so nearly all blocks skip the TMEM round trip.
//
// One CTA = (128-query block, query head); key blocks of 64:
//   S = Q K^T      16 MMAs (K = 256 dims in four swizzled 64-dim slabs), M 128 x N 64, S double-buffered in TMEM
//   P = softmax    8 warps, two threads per query row (32 keys each, and 128 of the 256 output columns each)
//   O += P V       4 MMAs of N = 256: V is the MN-major B operand, its four 64-dim slabs one descriptor stride apart
//
// The reference covers this shape with a wmma kernel (mfq/kernels/cuda/attention.cu: attention_flash256_f16_kernel).
#include "common.cuh"

#include <cfloat>

namespace mfq {

namespace d256 {
constexpr int kQB = 128, kKB = 64, kHD = 256;
constexpr int kQSlab = kQB * 128;              // 16 KB: [128 rows][64 dims] bf16, 128 B swizzle
constexpr int kKSlab = kKB * 128;              // 8 KB:  [64 keys][64 dims]
constexpr int kQBytes = 4 * kQSlab;            // 64 KB
constexpr int kKVBytes = 4 * kKSlab;           // 32 KB per K (or V) tile
constexpr int kPBytes = kQB * 128;             // 16 KB: [128 rows][64 keys]
constexpr int kThreads = 64 + 8 * 32;          // TMA warp, MMA warp, 8 softmax warps
constexpr int kSmem = kQBytes + 2 * 2 * kKVBytes + kPBytes + 1024 + 256 + 6 * kQB * 4;
constexpr float kLazyLog2 = 8.f;               // rescale when the maximum grew by more than this (log2 domain)
}  // namespace d256

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct Prefill256Params {
  __nv_bfloat16* out;  // [T, Hq, 256]
  int T, Hq, Hk;
  int Tk, offset;      // query row i sees keys 0 .. i + offset (offset = Tk - T)
  float scale_log2;
  int* status;
};

__global__ void __launch_bounds__(d256::kThreads, 1)
attn_prefill_d256_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, const Prefill256Params p) {
  using namespace d256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = base;
  uint8_t* sKV = base + kQBytes;                    // stage s: K at sKV + s * 2 * kKVBytes, V right after it
  uint8_t* sP = sKV + 4 * kKVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kPBytes);
  uint64_t* q_full = bars;            // 1
  uint64_t* kv_full = bars + 1;       // [2]
  uint64_t* kv_empty = bars + 3;      // [2]
  uint64_t* s_full = bars + 5;        // [2]
  uint64_t* s_empty = bars + 7;       // [2] (8 arrivals)
  uint64_t* p_full = bars + 9;        // 8 arrivals: P written and O rescaled (when it had to be)
  uint64_t* pv_full = bars + 10;      // commit
  uint64_t* x_bar = bars + 11;        // 8 arrivals: row-max exchange, one phase per key block
  uint64_t* l_bar = bars + 12;        // 8 arrivals: row-sum exchange, once
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_max = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);  // [2 buffers][2 halves][128]; sums [2][128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_qb = (p.T + kQB - 1) / kQB;
  const int qb = num_qb - 1 - blockIdx.x;  // heavy blocks first
  const int hq = blockIdx.y;
  const int kvh = hq / (p.Hq / p.Hk);
  const int nblk = min((p.Tk + kKB - 1) / kKB, ((qb + 1) * kQB + p.offset + kKB - 1) / kKB);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 8);
    }
    mbar_init(p_full, 8); mbar_init(pv_full, 1); mbar_init(x_bar, 8); mbar_init(l_bar, 8);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS[2] = {tmem_base, tmem_base + 64};
  const uint32_t tO = tmem_base + 128;  // 256 columns

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v);
      mbar_expect_tx(q_full, kQBytes);
#pragma unroll
      for (int sl = 0; sl < 4; ++sl) tma_load_2d(sQ + sl * kQSlab, &tmap_q, q_full, hq * kHD + 64 * sl, qb * kQB);
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutProducer)) break;
        uint8_t* k = sKV + s * 2 * kKVBytes;
        uint8_t* v = k + kKVBytes;
        mbar_expect_tx(&kv_full[s], 2 * kKVBytes);
#pragma unroll
        for (int sl = 0; sl < 4; ++sl) {
          tma_load_2d(k + sl * kKSlab, &tmap_k, &kv_full[s], kvh * kHD + 64 * sl, j * kKB);
          tma_load_2d(v + sl * kKSlab, &tmap_v, &kv_full[s], kvh * kHD + 64 * sl, j * kKB);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(128, kKB, 1, 1, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc(128, kHD, 1, 1, 0, 1);  // B = V is MN-major
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto issue_qk = [&](int j) {
        const uint32_t k_addr = smem_u32(sKV + (j & 1) * 2 * kKVBytes);
#pragma unroll
        for (int ks = 0; ks < 16; ++ks) {  // 16 x 16 dims; slab = ks / 4
          const uint32_t in_slab = (ks & 3) * 32;
          umma_f16(tS[j & 1], umma_desc_k_sw128(q_addr + (ks >> 2) * kQSlab + in_slab),
                   umma_desc_k_sw128(k_addr + (ks >> 2) * kKSlab + in_slab), idesc_qk, ks > 0);
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
        ok = mbar_wait(p_full, j & 1, abort_flag, p.status, kStatusTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sKV + (j & 1) * 2 * kKVBytes + kKVBytes);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)  // 4 x 16 keys; P is K-major over keys, one 128 B row per query
          umma_f16(tO, umma_desc_k_sw128(p_addr + ks * 32), umma_desc_mn_sw128(v_addr + ks * 2048, kKSlab), idesc_pv,
                   j > 0 || ks > 0);
        tc_commit(pv_full);
        tc_commit(&kv_empty[j & 1]);
      }
    }
  } else {
    // ----- softmax warps: two threads per query row; `half` selects 32 of the block's 64 keys and 128 of the 256
    // output columns -----
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int q_idx = qb * kQB + row;
    const uint32_t lane_sel = uint32_t(quarter * 32) << 16;
    float m_used = -FLT_MAX, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      const int sb = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[sb], (j >> 1) & 1, abort_flag, p.status, kStatusTimeoutEpilogue));
      if (!ok) break;
      tc_fence_after();
      const int key0 = j * kKB + half * 32;
      const bool diag = ((j + 1) * kKB - 1 > qb * kQB + p.offset) || ((j + 1) * kKB > p.Tk);
      uint32_t r[32];
      tmem_ld_32x32(tS[sb] + lane_sel + half * 32, r);
      tmem_wait_ld();
      float mx = -FLT_MAX;
      if (!diag) {
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int key = key0 + i;
          mx = fmaxf(mx, (key <= q_idx + p.offset && key < p.Tk) ? __uint_as_float(r[i]) : -FLT_MAX);
        }
      }
      s_max[(sb * 2 + half) * kQB + row] = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(x_bar);
      ok = __all_sync(0xffffffffu, mbar_wait(x_bar, j & 1, abort_flag, p.status, kStatusTimeoutEpilogue));
      if (!ok) break;
      mx = fmaxf(mx, s_max[(sb * 2 + (half ^ 1)) * kQB + row]);
      // both threads of a row (and so both warps of a row quarter) see the same numbers and take the same branch
      const bool grew = (mx - m_used) * p.scale_log2 > kLazyLog2;
      const bool rescale = __any_sync(0xffffffffu, grew);
      if (j > 0) {
        // P of the previous block is still being read, and O still written, until its MMAs retire
        ok = __all_sync(0xffffffffu, mbar_wait(pv_full, (j - 1) & 1, abort_flag, p.status, kStatusTimeoutEpilogue));
        if (!ok) break;
        tc_fence_after();
      }
      if (rescale) {
        const float m_new = fmaxf(m_used, mx);
        if (j > 0) {
          const float alpha = ex2_fast((m_used - m_new) * p.scale_log2);
          l_run *= alpha;
#pragma unroll 1
          for (int c = 0; c < 128; c += 32) {
            uint32_t o[32];
            const uint32_t addr = tO + lane_sel + half * 128 + c;
            tmem_ld_32x32(addr, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(addr, o);
          }
          tmem_wait_st();
        }
        m_used = m_new;
      }
      const float mb = m_used * p.scale_log2;
      float psum = 0.f;
      uint8_t* prow = sP + row * 128;
      uint32_t packed[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float p0 = ex2_fast(fmaf(__uint_as_float(r[i]), p.scale_log2, -mb));
        float p1 = ex2_fast(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, -mb));
        if (diag) {
          const int key = key0 + i;
          if (!(key <= q_idx + p.offset && key < p.Tk)) p0 = 0.f;
          if (!(key + 1 <= q_idx + p.offset && key + 1 < p.Tk)) p1 = 0.f;
        }
        psum += p0 + p1;
        __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
        packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
      }
      // this thread's 32 keys = 4 chunks of 16 bytes; the chunk index within the 128 B row is XORed with (row % 8)
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        const int chunk = (half * 4 + ch) ^ (row & 7);
        *reinterpret_cast<uint4*>(prow + chunk * 16) =
            make_uint4(packed[ch * 4], packed[ch * 4 + 1], packed[ch * 4 + 2], packed[ch * 4 + 3]);
      }
      l_run += psum;
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s_empty[sb]); mbar_arrive(p_full); }
    }
    if (ok) {
      s_max[(4 + half) * kQB + row] = l_run;
      __syncwarp();
      if (lane == 0) mbar_arrive(l_bar);
      ok = __all_sync(0xffffffffu, mbar_wait(l_bar, 0, abort_flag, p.status, kStatusTimeoutEpilogue)) &&
           __all_sync(0xffffffffu, mbar_wait(pv_full, (nblk - 1) & 1, abort_flag, p.status, kStatusTimeoutEpilogue));
      if (ok) {
        tc_fence_after();
        const float l_tot = l_run + s_max[(4 + (half ^ 1)) * kQB + row];
        const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
        __nv_bfloat16* dst = p.out + (size_t(q_idx) * p.Hq + hq) * kHD + half * 128;
#pragma unroll 1
        for (int c = 0; c < 128; c += 32) {
          uint32_t o[32];
          tmem_ld_32x32(tO + lane_sel + half * 128 + c, o);
          tmem_wait_ld();
          if (q_idx < p.T) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 va;
              __nv_bfloat162* ha = reinterpret_cast<__nv_bfloat162*>(&va);
#pragma unroll
              for (int e = 0; e < 4; ++e)
                ha[e] = __floats2bfloat162_rn(__uint_as_float(o[i + 2 * e]) * inv, __uint_as_float(o[i + 2 * e + 1]) * inv);
              *reinterpret_cast<uint4*>(dst + c + i) = va;
            }
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

// q: [T, Hq, 256] bf16, k/v: [Tk, Hk, 256] bf16 (contiguous), out: [T, Hq, 256] bf16; Tk >= T, query i attends to keys
// 0 .. i + (Tk - T).
extern "C" int mfq_attn_prefill_d256(const void* q, const void* k, const void* v, void* out, int T, int Tk, int Hq, int Hk,
                                     float sm_scale, int* status, cudaStream_t stream) {
  using namespace mfq;
  using namespace mfq::d256;
  if (T <= 0 || Tk < T || Hk <= 0 || Hq % Hk) return -1;
  CUtensorMap tq, tk, tv;
  if (make_tmap_2d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, T, uint64_t(Hq) * kHD, uint64_t(Hq) * kHD * 2, kQB, 64)) return -2;
  if (make_tmap_2d(&tk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tk, uint64_t(Hk) * kHD, uint64_t(Hk) * kHD * 2, kKB, 64)) return -3;
  if (make_tmap_2d(&tv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tk, uint64_t(Hk) * kHD, uint64_t(Hk) * kHD * 2, kKB, 64)) return -4;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_prefill_d256_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return -6;
    attr = true;
  }
  Prefill256Params p{static_cast<__nv_bfloat16*>(out), T, Hq, Hk, Tk, Tk - T, sm_scale * 1.4426950408889634f, status};
  attn_prefill_d256_kernel<<<dim3((T + kQB - 1) / kQB, Hq), kThreads, kSmem, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}
