// Small tensor-parallel collectives fused into their producing kernels, over peer-mapped memory.
//
// argmax_allgather: vocabulary-sharded greedy sampling.  Each rank reduces its logits shard to one (value, index)
// candidate per row, pushes it into every peer's slot table, and picks the global winner once all W candidates of
// the row have arrived -- 8 bytes per rank and row cross NVLink instead of the full logits (the reference gathers
// column-parallel outputs to a primary GPU with ncclSend/ncclRecv and samples there,
// cpp_runtime/backends/cuda/ops/quant_linear.cpp:532-611).
// Flags only count up (W-1 per launch and row) so the kernel is CUDA-graph replay safe; the launch count of a row
// selects one of two slot tables so a fast rank cannot overwrite candidates a slow rank still reads.
#include "common.cuh"

#include <cfloat>

namespace mfq {

struct Candidate { float value; int index; };

struct ArgmaxParams {
  int world, rank;
  Candidate* slots[8];   // per rank: [2][world][rows_cap]
  uint32_t* flags[8];    // per rank: [rows_cap]
  uint32_t* expected;    // local [rows_cap]
  int rows_cap;
};

__global__ void __launch_bounds__(1024)
argmax_allgather_kernel(const __nv_bfloat16* __restrict__ logits, int* __restrict__ out, int V, int stride,
                        int index_offset, ArgmaxParams ap, int* status) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const int row = blockIdx.x;
  const __nv_bfloat16* lr = logits + size_t(row) * stride;
  float best = -FLT_MAX;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = __bfloat162float(lr[i]);
    if (v > best) { best = v; bi = i; }
  }
  auto merge = [](float& b, int& i, float ov, int oi) {
    if (ov > b || (ov == b && oi < i)) { b = ov; i = oi; }
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) merge(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp != 0) return;
  const int nw = blockDim.x >> 5;
  best = lane < nw ? sv[lane] : -FLT_MAX;
  bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) merge(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if (lane != 0) return;
  bi += index_offset;
  if (ap.world == 1) { out[row] = bi; return; }
  const uint32_t before = ap.expected[row];
  const uint32_t target = before + uint32_t(ap.world - 1);
  const size_t table = size_t((before / uint32_t(ap.world - 1)) & 1u) * ap.world * ap.rows_cap;
  const unsigned long long packed = (unsigned long long)(__float_as_uint(best)) | ((unsigned long long)(uint32_t)bi << 32);
  for (int r = 0; r < ap.world; ++r) {
    Candidate* dst = ap.slots[r] + table + size_t(ap.rank) * ap.rows_cap + row;
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(packed) : "memory");
  }
  __threadfence_system();
  for (int r = 0; r < ap.world; ++r)  // ordered by the fence above: relaxed updates leave back to back
    if (r != ap.rank) asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(ap.flags[r] + row) : "memory");
  const uint32_t* my_flag = ap.flags[ap.rank] + row;
  const unsigned long long t_start = globaltimer_ns();
  uint32_t seen, spins = 0;
  bool ok = true;
  while (true) {
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(my_flag) : "memory");
    if (int32_t(seen - target) >= 0) break;
    if ((++spins & 0x3F) == 0 && globaltimer_ns() - t_start > kWaitBudgetNs) {
      atomicCAS(status, 0, kStatusTimeoutPeer | (4 << 8));
      ok = false;
      break;
    }
  }
  ap.expected[row] = target;
  if (!ok) return;
  float gb = -FLT_MAX;
  int gi = 0x7fffffff;
  for (int r = 0; r < ap.world; ++r) {
    unsigned long long pk;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(pk) : "l"(ap.slots[ap.rank] + table + size_t(r) * ap.rows_cap + row) : "memory");
    merge(gb, gi, __uint_as_float(uint32_t(pk)), int(uint32_t(pk >> 32)));
  }
  out[row] = gi;
}

}  // namespace mfq

// logits: this rank's shard [B, V] (row stride `stride`), index_offset = first vocabulary id of the shard.
// slots[r]: rank r's table of 2 * world * rows_cap candidates (8 bytes each); flags[r]: rows_cap counters.
extern "C" int mfq_argmax_allgather(const void* logits, int* out, int B, int V, int stride, int index_offset, int world,
                                    int rank, void* const* slots, void* const* flags, void* expected, int rows_cap,
                                    int* status, cudaStream_t stream) {
  if (B <= 0 || B > rows_cap || world < 1 || world > 8) return -1;
  mfq::ArgmaxParams ap{};
  ap.world = world;
  ap.rank = rank;
  for (int r = 0; r < world && world > 1; ++r) {
    ap.slots[r] = static_cast<mfq::Candidate*>(slots[r]);
    ap.flags[r] = static_cast<uint32_t*>(flags[r]);
  }
  ap.expected = static_cast<uint32_t*>(expected);
  ap.rows_cap = rows_cap;
  mfq::argmax_allgather_kernel<<<B, 1024, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), out, V, stride,
                                                        index_offset, ap, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

// ---------------------------------------------------------------------------------------------------------------
// allreduce_rows: out[row] = residual[row] + sum over ranks of partial_r[row], one CTA per row, over peer-mapped
// buffers with the same count-up flag protocol (graph-replay safe, double-buffered).  Used where a layer's partial
// result is produced by a non-GEMM kernel, e.g. the expert-parallel MoE combine (each rank holds the weighted sum
// of its own experts).  The reference reduces such partials to its primary GPU with ncclReduce
// (cpp_runtime/backends/cuda/ops/quant_linear.cpp:629-742).
// ---------------------------------------------------------------------------------------------------------------
namespace mfq {

struct RowReduceParams {
  int world, rank;
  __nv_bfloat16* bufs[8];   // per rank: [2][rows_cap][H]
  uint32_t* flags[8];       // per rank: [rows_cap]
  uint32_t* expected;       // local [rows_cap]
  int rows_cap;
};

__global__ void __launch_bounds__(256)
allreduce_rows_kernel(const __nv_bfloat16* __restrict__ partial, const __nv_bfloat16* __restrict__ residual,
                      __nv_bfloat16* __restrict__ out, int H, RowReduceParams rp, int* status) {
  __shared__ int s_ok;
  const int row = blockIdx.x;
  const uint32_t before = rp.expected[row];
  const uint32_t target = before + uint32_t(rp.world - 1);
  const size_t off = (size_t((before / uint32_t(rp.world - 1)) & 1u) * rp.rows_cap + row) * H;
  const int nvec = H / 8;
  uint4* mine = reinterpret_cast<uint4*>(rp.bufs[rp.rank] + off);
  const uint4* src = reinterpret_cast<const uint4*>(partial + size_t(row) * H);
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) mine[v] = src[v];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();  // orders the CTA's row (observed through the barrier above) before the relaxed updates
    for (int r = 0; r < rp.world; ++r)
      if (r != rp.rank) asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(rp.flags[r] + row) : "memory");
    const uint32_t* my_flag = rp.flags[rp.rank] + row;
    const unsigned long long t_start = globaltimer_ns();
    uint32_t seen, spins = 0;
    int ok = 1;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(my_flag) : "memory");
      if (int32_t(seen - target) >= 0) break;
      if ((++spins & 0x3F) == 0 && globaltimer_ns() - t_start > kWaitBudgetNs) {
        atomicCAS(status, 0, kStatusTimeoutPeer | (5 << 8));
        ok = 0;
        break;
      }
    }
    rp.expected[row] = target;
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (residual) {
      const uint4 b = *reinterpret_cast<const uint4*>(residual + size_t(row) * H + v * 8);
      const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(&b);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = __bfloat162float(bb[j]);
    }
    uint4 parts[8];  // every rank's vector is requested before the first add: the remote round trips overlap
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      parts[r] = make_uint4(0, 0, 0, 0);
      if (r < rp.world) {
        const uint4* p = reinterpret_cast<const uint4*>(rp.bufs[r] + off) + v;
        asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(parts[r].x), "=r"(parts[r].y), "=r"(parts[r].z), "=r"(parts[r].w) : "l"(p) : "memory");
      }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {  // rank order; bf16 zero bits beyond the world size add nothing
      const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(&parts[r]);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(bb[j]);
    }
    uint4 o;
    __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) ob[j] = __float2bfloat16(acc[j]);
    *reinterpret_cast<uint4*>(out + size_t(row) * H + v * 8) = o;
  }
}

}  // namespace mfq

// partial / residual / out: [rows, H] bf16 (residual may be null; out may alias residual).  bufs[r]: rank r's
// 2 * rows_cap * H bf16 staging buffer, flags[r]: rows_cap counters (zero before first use).
extern "C" int mfq_allreduce_rows(const void* partial, const void* residual, void* out, int rows, int H, int world,
                                  int rank, void* const* bufs, void* const* flags, void* expected, int rows_cap,
                                  int* status, cudaStream_t stream) {
  if (rows <= 0 || rows > rows_cap || H % 8 || world < 2 || world > 8) return -1;
  mfq::RowReduceParams rp{};
  rp.world = world;
  rp.rank = rank;
  for (int r = 0; r < world; ++r) {
    rp.bufs[r] = static_cast<__nv_bfloat16*>(bufs[r]);
    rp.flags[r] = static_cast<uint32_t*>(flags[r]);
  }
  rp.expected = static_cast<uint32_t*>(expected);
  rp.rows_cap = rows_cap;
  mfq::allreduce_rows_kernel<<<rows, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(partial),
                                                       static_cast<const __nv_bfloat16*>(residual),
                                                       static_cast<__nv_bfloat16*>(out), H, rp, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

// ---------------------------------------------------------------------------------------------------------------
// peer_barrier: every rank bumps a counter on every peer and waits until all peers bumped its own (bounded wait).
// Stream-ordered on each rank, so it separates "everything before" on all ranks from "everything after".
// ---------------------------------------------------------------------------------------------------------------
namespace mfq {
__global__ void peer_barrier_kernel(int world, int rank, uint32_t* f0, uint32_t* f1, uint32_t* f2, uint32_t* f3, uint32_t* f4,
                                    uint32_t* f5, uint32_t* f6, uint32_t* f7, uint32_t* expected, int* status) {
  uint32_t* flags[8] = {f0, f1, f2, f3, f4, f5, f6, f7};
  const uint32_t target = *expected + uint32_t(world - 1);
  __threadfence_system();
  for (int r = 0; r < world; ++r)
    if (r != rank) asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(flags[r]) : "memory");
  const unsigned long long t_start = globaltimer_ns();
  uint32_t seen, spins = 0;
  while (true) {
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags[rank]) : "memory");
    if (int32_t(seen - target) >= 0) break;
    if ((++spins & 0x3F) == 0 && globaltimer_ns() - t_start > kWaitBudgetNs) {
      atomicCAS(status, 0, kStatusTimeoutPeer | (6 << 8));
      break;
    }
  }
  *expected = target;
}
}  // namespace mfq

extern "C" int mfq_peer_barrier(int world, int rank, void* const* flags, void* expected, int* status, cudaStream_t stream) {
  if (world < 2 || world > 8) return -1;
  uint32_t* f[8] = {};
  for (int r = 0; r < world; ++r) f[r] = static_cast<uint32_t*>(flags[r]);
  mfq::peer_barrier_kernel<<<1, 1, 0, stream>>>(world, rank, f[0], f[1], f[2], f[3], f[4], f[5], f[6], f[7],
                                                static_cast<uint32_t*>(expected), status);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

// ---------------------------------------------------------------------------------------------------------------
// allgather_rows: every rank holds `rows` rows of `row_bytes` bytes; afterwards every rank holds all W * rows rows
// in rank order.  The push kernel stores the local shard into every rank's staging buffer (16-byte coalesced
// stores; half `epoch & 1`), the last CTA bumps one flag per destination; the collect kernel waits for the W flags
// (bounded) and copies the staging half into `out`.  Together with the GEMM -> reduce-scatter epilogue this is the
// two-shot all-reduce used for wide token batches, where a one-shot exchange would move W times the bytes.
// ---------------------------------------------------------------------------------------------------------------
namespace mfq {

struct GatherParams {
  int world, rank;
  uint8_t* bufs[8];      // per rank: [2][world * shard_cap_bytes]
  uint32_t* flags[8];    // per rank: [world]
  uint32_t* words;       // local: [0] completed gathers, [1] CTA arrival counter
  size_t half_bytes;     // bytes of one staging half
};

__global__ void __launch_bounds__(256)
allgather_push_kernel(const uint8_t* __restrict__ shard, size_t shard_bytes, GatherParams gp) {
  __shared__ int is_last;
  const uint32_t epoch = gp.words[0];
  const size_t base = size_t(epoch & 1u) * gp.half_bytes + size_t(gp.rank) * shard_bytes;
  const size_t nvec = shard_bytes / 16;
  const uint4* src = reinterpret_cast<const uint4*>(shard);
  for (size_t v = size_t(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += size_t(gridDim.x) * blockDim.x) {
    const uint4 val = src[v];
    for (int rr = 0; rr < gp.world; ++rr)  // start with a different destination on every rank (no incast)
      reinterpret_cast<uint4*>(gp.bufs[(gp.rank + 1 + rr) % gp.world] + base)[v] = val;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    is_last = atomicAdd(&gp.words[1], 1u) == gridDim.x - 1;
    __threadfence();
  }
  __syncthreads();
  if (!is_last) return;
  if (int(threadIdx.x) < gp.world)
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(gp.flags[threadIdx.x] + gp.rank) : "memory");
  if (threadIdx.x == 0) { gp.words[1] = 0; gp.words[0] = epoch + 1; }
}

__global__ void __launch_bounds__(256)
allgather_collect_kernel(uint8_t* __restrict__ out, size_t total_bytes, GatherParams gp, int* status) {
  __shared__ int s_ok;
  const uint32_t target = gp.words[0];  // already counts the push of this gather
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (int(threadIdx.x) < gp.world) {
    const uint32_t* f = gp.flags[gp.rank] + threadIdx.x;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t seen, spins = 0;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(f) : "memory");
      if (int32_t(seen - target) >= 0) break;
      if ((++spins & 0x3F) == 0 && globaltimer_ns() - t0 > kWaitBudgetNs) {
        atomicCAS(status, 0, kStatusTimeoutPeer | (7 << 8));
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (!s_ok) return;
  const uint4* src = reinterpret_cast<const uint4*>(gp.bufs[gp.rank] + size_t((target - 1u) & 1u) * gp.half_bytes);
  uint4* dst = reinterpret_cast<uint4*>(out);
  for (size_t v = size_t(blockIdx.x) * blockDim.x + threadIdx.x; v < total_bytes / 16; v += size_t(gridDim.x) * blockDim.x) {
    uint4 val;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w) : "l"(src + v) : "memory");
    dst[v] = val;
  }
}

}  // namespace mfq

// shard: this rank's [rows, row_bytes] block; out: [world * rows, row_bytes].  bufs[r]: rank r's staging buffer of
// 2 * half_bytes bytes (half_bytes >= world * rows * row_bytes); flags[r]: world counters; words: 2 local counters.
extern "C" int mfq_allgather_rows(const void* shard, void* out, long long shard_bytes, int world, int rank,
                                  void* const* bufs, void* const* flags, void* words, long long half_bytes, int* status,
                                  cudaStream_t stream) {
  if (shard_bytes <= 0 || shard_bytes % 16 || world < 2 || world > 8 || shard_bytes * world > half_bytes) return -1;
  mfq::GatherParams gp{};
  gp.world = world;
  gp.rank = rank;
  for (int r = 0; r < world; ++r) {
    gp.bufs[r] = static_cast<uint8_t*>(bufs[r]);
    gp.flags[r] = static_cast<uint32_t*>(flags[r]);
  }
  gp.words = static_cast<uint32_t*>(words);
  gp.half_bytes = size_t(half_bytes);
  const int blocks = int(std::min<long long>(2 * 148, (shard_bytes / 16 + 255) / 256));
  mfq::allgather_push_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(shard), size_t(shard_bytes), gp);
  mfq::allgather_collect_kernel<<<2 * 148, 256, 0, stream>>>(static_cast<uint8_t*>(out), size_t(shard_bytes) * world, gp, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}
