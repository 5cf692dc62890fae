// Tensor-parallel all-reduce fused with the residual add, the next RMSNorm and the FP8 row quantization:
//
//   h[row]  += sum over ranks r of partial_r[row]            (bf16 partials, fp32 sum in rank order)
//   xq, xs   = quantize_e4m3(rmsnorm(h[row]) * w)            (what the next GEMM consumes)
//
// Every rank's row-parallel GEMM (o_proj, down) writes its bf16 partial [M, H] into its own peer-mapped buffer;
// this kernel follows on the stream.  Two modes:
//
//   one-shot  (small M): every rank pulls all W partials of every row over NVLink with 16-byte loads and computes
//             everything itself -- one flag hop plus one load round trip;
//   two-shot  (larger M): rank r pulls only the rows it owns (M / W of them), then PUSHES the finished rows -- the bf16
//             residual row and, computed once instead of W times, its FP8 code row and multiplier -- into every rank's
//             buffers, so 2 (W-1)/W of the data crosses NVLink instead of (W-1) x.
//
// Synchronisation is one arrival word per rank and launch (not per tile): block 0 publishes "my partial of launch e is
// complete" to every peer with a release store of the launch number; everybody spins (bounded) on its own W words.
// Words only ever grow, so a CUDA-graph replay needs no reset.  The partial buffer has two halves used alternately
// (the caller passes `half`): a fast rank's next GEMM then never overwrites a partial that a slow rank still reads.
// The two-shot mode ends with a second word ("my pushes have landed"), awaited by the last block before the kernel
// completes, so the next kernel on the stream sees every peer's rows.
//
// The sums run in rank order on every rank, so all ranks hold bit-identical residual streams.
//
// The reference reduces such partials to one primary GPU with ncclReduce and casts them through fp32 buffers
// (cpp_runtime/backends/cuda/ops/quant_linear.cpp:629-742), then runs the norm as a separate kernel on that GPU.
#include "common.cuh"

#include <cfloat>

namespace mfq {

constexpr float kFp8Max = 448.f;

struct ReduceParams {
  int world, rank;
  const __nv_bfloat16* partial[8];  // every rank's partial buffer: 2 halves of rows_cap * H bf16
  __nv_bfloat16* h[8];              // every rank's residual stream [rows_cap, H] (two-shot pushes rows into peers)
  uint8_t* xq[8];                   // every rank's FP8 activations [rows_cap, H]
  float* xs[8];                     // every rank's row multipliers [rows_cap]
  uint32_t* flags[8];               // every rank: [0..8) "partial ready" words, [8..16) "rows pushed" words
  uint32_t* state;                  // local: [0] completed launches, [1] block arrival counter
  int rows_cap;
};

__device__ __forceinline__ uint4 ld_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Spin until *p has reached `want` (wrap-safe); false when the time budget ran out.
__device__ __forceinline__ bool wait_word(const uint32_t* p, uint32_t want) {
  if (int32_t(ld_acquire_sys(p) - want) >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (int32_t(ld_acquire_sys(p) - want) < 0) {
    if ((++spins & 0x3F) == 0 && globaltimer_ns() - t0 > kWaitBudgetNs) return false;
  }
  return true;
}

__device__ __forceinline__ float block_sum_256(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) t += red[i];
  return t;
}
__device__ __forceinline__ float block_max_256(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) t = fmaxf(t, red[i]);
  return t;
}

// VPT = 16-byte vectors of a row per thread (256 threads): H <= 2048 * VPT.
template <int VPT>
__global__ void __launch_bounds__(256)
tp_reduce_norm_quant_kernel(const ReduceParams p, int M, int H, int half, const __nv_bfloat16* __restrict__ norm_w,
                            float eps, int two_shot, int add_residual, int* status) {
  pdl_trigger();
  pdl_wait();  // the GEMM that produced this rank's partial has completed and flushed
  __shared__ float red[8];
  __shared__ int s_flag;
  const int tid = threadIdx.x;
  const uint32_t want = p.state[0] + 1u;  // launch number; p.state[0] is bumped by the last block at the very end
  if (tid == 0) s_flag = 1;
  __syncthreads();
  // ---- phase 0: publish "my partial is complete", then wait for every peer's ----
  if (blockIdx.x == 0 && tid < p.world && tid != p.rank) {
    __threadfence_system();
    st_release_sys(p.flags[tid] + p.rank, want);
  }
  if (tid < p.world && tid != p.rank) {
    if (!wait_word(p.flags[p.rank] + tid, want)) {
      atomicCAS(status, 0, kStatusTimeoutPeer | (8 << 8));
      s_flag = 0;
    }
  }
  __syncthreads();
  const bool ready = s_flag != 0;

  int r0 = 0, r1 = M;
  if (two_shot) {
    const int per = (M + p.world - 1) / p.world;
    r0 = min(M, p.rank * per);
    r1 = min(M, r0 + per);
  }
  const int nvec = H / 8;
  const size_t half_off = size_t(half) * p.rows_cap * H;
  if (ready) {
    for (int row = r0 + blockIdx.x; row < r1; row += gridDim.x) {
      const size_t roff = size_t(row) * H;
      float v[VPT][8];
      // every rank's vector is requested before the first add, so the remote round trips overlap
      uint4 parts[VPT][8];
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = tid + i * 256;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          parts[i][r] = make_uint4(0, 0, 0, 0);
          if (r < p.world && vi < nvec) parts[i][r] = ld_sys_v4(p.partial[r] + half_off + roff + vi * 8);
        }
      }
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = tid + i * 256;
        if (vi < nvec) {
          float acc[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
          for (int r = 0; r < 8; ++r) {  // rank order; zero bits beyond the world size add nothing
            const __nv_bfloat16* pb = reinterpret_cast<const __nv_bfloat16*>(&parts[i][r]);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(pb[j]);
          }
          if (add_residual) {
            const uint4 hv = __ldcg(reinterpret_cast<const uint4*>(p.h[p.rank] + roff + vi * 8));
            const __nv_bfloat16* hb = reinterpret_cast<const __nv_bfloat16*>(&hv);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(hb[j]);
          }
          uint4 o;
          __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            ob[j] = __float2bfloat16(acc[j]);
            v[i][j] = __bfloat162float(ob[j]);  // the norm reads the stored (bf16) residual, like an unfused norm
            ss += v[i][j] * v[i][j];
          }
          if (two_shot) {
            for (int rr = 0; rr < p.world; ++rr) {  // own copy first, then a different destination on every rank
              const int dst = (p.rank + rr) % p.world;
              *reinterpret_cast<uint4*>(p.h[dst] + roff + vi * 8) = o;
            }
          } else {
            *reinterpret_cast<uint4*>(p.h[p.rank] + roff + vi * 8) = o;
          }
        }
      }
      if (norm_w != nullptr) {
        const float rstd = rsqrtf(block_sum_256(ss, red) / float(H) + eps);
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int vi = tid + i * 256;
          if (vi < nvec) {
            const uint4 ww = __ldg(reinterpret_cast<const uint4*>(norm_w + vi * 8));
            const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(&ww);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              v[i][j] = __bfloat162float(__float2bfloat16(v[i][j] * rstd * __bfloat162float(wb[j])));
              amax = fmaxf(amax, fabsf(v[i][j]));
            }
          }
        }
        amax = block_max_256(amax, red);
        const float scale = fmaxf(amax, 1e-12f) / kFp8Max;
        const float inv = 1.f / scale;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int vi = tid + i * 256;
          if (vi < nvec) {
            uint2 o;
            uint8_t* ob = reinterpret_cast<uint8_t*>(&o);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              ob[j] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(v[i][j] * inv, __NV_SATFINITE, __NV_E4M3));
            if (two_shot) {
              for (int rr = 0; rr < p.world; ++rr) {
                const int dst = (p.rank + rr) % p.world;
                *reinterpret_cast<uint2*>(p.xq[dst] + roff + vi * 8) = o;
              }
            } else {
              *reinterpret_cast<uint2*>(p.xq[p.rank] + roff + vi * 8) = o;
            }
          }
        }
        if (tid == 0) {
          if (two_shot) {
            for (int rr = 0; rr < p.world; ++rr) p.xs[(p.rank + rr) % p.world][row] = scale;
          } else {
            p.xs[p.rank][row] = scale;
          }
        }
      }
    }
  }
  // ---- phase 2: the last block to finish bumps the launch counter; two-shot: it also publishes "my rows have
  //      landed" and waits for every peer's, which keeps the kernel (and so the stream) from moving on early ----
  if (two_shot) __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    s_flag = (atomicAdd(p.state + 1, 1u) == gridDim.x - 1) ? 1 : 0;
    __threadfence();  // acquire side: the other blocks' rows are ordered before what the last block does next
  }
  __syncthreads();
  if (!s_flag) return;
  if (two_shot) {
    if (tid < p.world && tid != p.rank) {
      __threadfence_system();
      st_release_sys(p.flags[tid] + 8 + p.rank, want);
      if (ready && !wait_word(p.flags[p.rank] + 8 + tid, want)) atomicCAS(status, 0, kStatusTimeoutPeer | (9 << 8));
    }
    __syncthreads();
  }
  if (tid == 0) {
    p.state[1] = 0;
    p.state[0] = want;
  }
}

}  // namespace mfq

// partial[r] / h[r] / xq[r] / xs[r] / flags[r]: `world` device pointers each (own buffer at index `rank`, the others
// peer-mapped).  partial: 2 * rows_cap * H bf16 (this launch reads half `half`), h: rows_cap * H bf16, xq: rows_cap * H
// bytes, xs: rows_cap floats, flags: 16 words (zero before first use); state: 2 local words (zero before first use).
// norm_w == nullptr: only the residual stream is updated.  add_residual == 0: h = sum of the partials.  All ranks must
// issue the same sequence of calls.  H % 8 == 0, H <= 8192, M <= rows_cap.
extern "C" int mfq_tp_reduce_norm_quant(int M, int H, int half, const void* norm_w, float eps, int two_shot,
                                        int add_residual, int world, int rank, void* const* partial, void* const* h,
                                        void* const* xq, void* const* xs, void* const* flags, void* state, int rows_cap,
                                        int* status, cudaStream_t stream) {
  if (M <= 0 || M > rows_cap || H <= 0 || H % 8 || H > 8192 || world < 2 || world > 8 || rank < 0 || rank >= world ||
      (half != 0 && half != 1))
    return -1;
  mfq::ReduceParams p{};
  p.world = world;
  p.rank = rank;
  for (int r = 0; r < world; ++r) {
    p.partial[r] = static_cast<const __nv_bfloat16*>(partial[r]);
    p.h[r] = static_cast<__nv_bfloat16*>(h[r]);
    p.xq[r] = static_cast<uint8_t*>(xq[r]);
    p.xs[r] = static_cast<float*>(xs[r]);
    p.flags[r] = static_cast<uint32_t*>(flags[r]);
  }
  p.state = static_cast<uint32_t*>(state);
  p.rows_cap = rows_cap;
  const int rows = two_shot ? (M + world - 1) / world : M;
  const int grid = rows < 1 ? 1 : (rows > 296 ? 296 : rows);
  const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(norm_w);
  cudaError_t e;
  if (H <= 2048)
    e = mfq::launch_kernel(mfq::tp_reduce_norm_quant_kernel<1>, dim3(grid), dim3(256), 0, stream, p, M, H, half, w, eps, two_shot, add_residual, status);
  else if (H <= 4096)
    e = mfq::launch_kernel(mfq::tp_reduce_norm_quant_kernel<2>, dim3(grid), dim3(256), 0, stream, p, M, H, half, w, eps, two_shot, add_residual, status);
  else
    e = mfq::launch_kernel(mfq::tp_reduce_norm_quant_kernel<4>, dim3(grid), dim3(256), 0, stream, p, M, H, half, w, eps, two_shot, add_residual, status);
  return e == cudaSuccess ? 0 : -7;
}
