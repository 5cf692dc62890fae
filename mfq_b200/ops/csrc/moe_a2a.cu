// Expert-parallel dispatch / combine over peer-mapped memory (NVLink), fused with the permute and the weighted
// un-permute.
//
// Tokens are sharded over the W ranks, experts too (rank r owns experts [r*E/W, (r+1)*E/W)).
//   dispatch      : each warp takes one local token, finds the set of ranks that own any of its top-k experts and
//                   stores the FP8 row, its multiplier and its (expert id, weight) list ONCE per destination rank
//                   straight into that rank's receive table -- slot (source rank, arrival index) -- so no separate
//                   permute pass, no size exchange and no staging copy precede the transfer.  The last CTA publishes
//                   the per-destination row counts and bumps one flag per destination.
//   recv_wait     : (1 CTA) waits for the W flags, then marks the unused slots of the table with expert id -1 so
//                   that the ordinary route planner / grouped GEMMs can run over the table as if it were a local batch.
//   combine_push  : for each received token sums  w_k * y[row_k]  over the experts it used on this rank and stores the
//                   bf16 row directly into the source rank's return table; the last CTA bumps one flag per source.
//   combine_reduce: the source waits for W flags and adds, in rank order (bit-identical run to run), the rows that
//                   came back for each token to the residual (+ the shared expert's output).
//
// Buffers are single: a rank can only start dispatch n+1 after its combine_reduce n has seen the flag of EVERY rank,
// and a rank bumps that flag only when its combine_push n -- its last reader of the receive table -- is complete; the
// same chain in the other direction protects the return table.  Hence dispatch and combine must be called strictly
// in pairs, by all ranks, in the same order.  Flags only count up and the expected value lives on the device, so
// the sequence is CUDA-graph replay safe.  All waits are bounded and report through the status word.
//
// The reference moves routed rows between GPUs with NCCL broadcast + reduce to a primary GPU
// (cpp_runtime/backends/cuda/core/ffn.cpp:201-300); it has no all-to-all path.
#include "common.cuh"

namespace mfq {

struct A2aParams {
  int world, rank, K, cap, e_per;
  uint8_t* recv_x[8];        // per rank: [world*cap][row_bytes]
  float* recv_s[8];          // [world*cap]
  int* recv_ids[8];          // [world*cap][K]
  float* recv_w[8];          // [world*cap][K]
  int* recv_count[8];        // [world]
  uint32_t* flags[8];        // [2*world]: dispatch flags, then combine flags, indexed by the writing rank
  __nv_bfloat16* comb[8];    // [world*cap][H]
  uint32_t* words;           // local: [0] completed dispatches, [1] CTA arrival counter, [2 .. 2+world) send counts
};

__device__ __forceinline__ void flag_add_sys(uint32_t* p) {
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}

__device__ __forceinline__ bool flag_wait_sys(const uint32_t* p, uint32_t target, int* status, int site = 3) {
  const unsigned long long t0 = globaltimer_ns();
  uint32_t seen, spins = 0;
  while (true) {
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(p) : "memory");
    if (int32_t(seen - target) >= 0) return true;
    if ((++spins & 0x3F) == 0 && globaltimer_ns() - t0 > kWaitBudgetNs) {
      // status[1..3]: the word's last value, the value awaited and the waiting thread (= source rank), for the report
      if (atomicCAS(status, 0, kStatusTimeoutPeer | (site << 8)) == 0) { status[1] = int(seen); status[2] = int(target); status[3] = int(threadIdx.x); }
      return false;
    }
  }
}

// True in exactly one CTA of the grid: the one that arrives last.  Every thread's earlier stores are fenced first.
__device__ __forceinline__ bool last_cta_arrives(uint32_t* counter) {
  __shared__ int is_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(counter, 1u);
    is_last = prev == gridDim.x - 1;
    __threadfence();
  }
  __syncthreads();
  return is_last != 0;
}

__global__ void __launch_bounds__(256)
moe_dispatch_kernel(const uint8_t* __restrict__ xq, const float* __restrict__ xs, const int* __restrict__ ids,
                    const float* __restrict__ wt, int T, int row_bytes, int* __restrict__ send_slot, A2aParams p,
                    int* status) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    const int e = lane < p.K ? ids[size_t(t) * p.K + lane] : -1;
    const float w = lane < p.K ? wt[size_t(t) * p.K + lane] : 0.f;
    const int owner = e >= 0 ? e / p.e_per : -1;
    const float s = xs[t];
    for (int dst = 0; dst < p.world; ++dst) {
      const unsigned m = __ballot_sync(0xffffffffu, owner == dst);
      if (m == 0) {
        if (lane == 0) send_slot[size_t(t) * p.world + dst] = -1;
        continue;
      }
      int slot = 0;
      if (lane == 0) slot = int(atomicAdd(&p.words[2 + dst], 1u));
      slot = __shfl_sync(0xffffffffu, slot, 0);
      if (slot >= p.cap) {  // cannot happen while cap >= T; recorded rather than written out of bounds
        if (lane == 0) { atomicCAS(status, 0, kStatusBadArgument); send_slot[size_t(t) * p.world + dst] = -1; }
        continue;
      }
      const size_t row = size_t(p.rank) * p.cap + slot;
      const uint4* src = reinterpret_cast<const uint4*>(xq + size_t(t) * row_bytes);
      uint4* out = reinterpret_cast<uint4*>(p.recv_x[dst] + row * row_bytes);
      for (int i = lane; i < row_bytes / 16; i += 32) out[i] = src[i];
      if (lane < p.K) {
        p.recv_ids[dst][row * p.K + lane] = e;
        p.recv_w[dst][row * p.K + lane] = w;
      }
      if (lane == 0) {
        p.recv_s[dst][row] = s;
        send_slot[size_t(t) * p.world + dst] = slot;
      }
    }
  }
  if (!last_cta_arrives(&p.words[1])) return;
  if (int(threadIdx.x) < p.world) {
    const int dst = threadIdx.x;
    const uint32_t n = min(p.words[2 + dst], uint32_t(p.cap));
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.recv_count[dst] + p.rank), "r"(n) : "memory");
    __threadfence_system();
    flag_add_sys(p.flags[dst] + p.rank);
    p.words[2 + dst] = 0;
  }
  if (threadIdx.x == 0) { p.words[1] = 0; p.words[0] += 1; }
}

__global__ void __launch_bounds__(256) moe_recv_wait_kernel(A2aParams p, int* __restrict__ counts_out, int* status) {
  const uint32_t target = p.words[0];
  if (int(threadIdx.x) < p.world) flag_wait_sys(p.flags[p.rank] + threadIdx.x, target, status);
  __syncthreads();
  int* ids = p.recv_ids[p.rank];
  int total = 0;
  for (int src = 0; src < p.world; ++src) {
    const int c = min(max(p.recv_count[p.rank][src], 0), p.cap);
    total += c;
    const int n = (p.cap - c) * p.K;
    int* base = ids + (size_t(src) * p.cap + c) * p.K;
    for (int i = threadIdx.x; i < n; i += blockDim.x) base[i] = -1;
  }
  if (threadIdx.x == 0 && counts_out) counts_out[0] = total;
}

__global__ void __launch_bounds__(256)
moe_combine_push_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ dest, int H, A2aParams p) {
  for (int entry = blockIdx.x; entry < p.world * p.cap; entry += gridDim.x) {
    const int src = entry / p.cap, slot = entry % p.cap;
    if (slot >= p.recv_count[p.rank][src]) continue;
    const float* w = p.recv_w[p.rank] + size_t(entry) * p.K;
    const int* rows = dest + size_t(entry) * p.K;
    __nv_bfloat16* out = p.comb[src] + (size_t(p.rank) * p.cap + slot) * H;
    for (int v = threadIdx.x; v < H / 8; v += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int k = 0; k < p.K; ++k) {
        const int row = rows[k];
        if (row < 0) continue;
        const float wk = w[k];
        const uint4 b = *reinterpret_cast<const uint4*>(y + size_t(row) * H + v * 8);
        const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(&b);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = fmaf(wk, __bfloat162float(bb[j]), acc[j]);
      }
      uint4 o;
      __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j) ob[j] = __float2bfloat16(acc[j]);
      *reinterpret_cast<uint4*>(out + v * 8) = o;
    }
  }
  if (!last_cta_arrives(&p.words[1])) return;
  if (int(threadIdx.x) < p.world) flag_add_sys(p.flags[threadIdx.x] + p.world + p.rank);
  if (threadIdx.x == 0) p.words[1] = 0;
}

__global__ void __launch_bounds__(256)
moe_combine_reduce_kernel(const int* __restrict__ send_slot, const __nv_bfloat16* __restrict__ base,
                          const __nv_bfloat16* __restrict__ extra, __nv_bfloat16* __restrict__ out, int T, int H,
                          A2aParams p, int* status) {
  const int t = blockIdx.x;
  const uint32_t target = p.words[0];
  if (int(threadIdx.x) < p.world) flag_wait_sys(p.flags[p.rank] + p.world + threadIdx.x, target, status, 10);
  __syncthreads();
  if (t >= T) return;  // a rank without tokens still waits, so that it cannot run ahead of its peers
  const __nv_bfloat16* comb = p.comb[p.rank];
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    auto add = [&](const __nv_bfloat16* rowp) {
      const uint4 b = *reinterpret_cast<const uint4*>(rowp + v * 8);
      const __nv_bfloat16* bb = reinterpret_cast<const __nv_bfloat16*>(&b);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(bb[j]);
    };
    if (base) add(base + size_t(t) * H);
    if (extra) add(extra + size_t(t) * H);
    for (int r = 0; r < p.world; ++r) {
      const int slot = send_slot[size_t(t) * p.world + r];
      if (slot >= 0) add(comb + (size_t(r) * p.cap + slot) * H);
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

namespace {
int fill_params(A2aParams& p, int world, int rank, int K, int cap, int e_per, void* const* recv_x, void* const* recv_s,
                void* const* recv_ids, void* const* recv_w, void* const* recv_count, void* const* flags,
                void* const* comb, void* words) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || K < 1 || K > 32 || cap < 1 || e_per < 1) return -1;
  p.world = world; p.rank = rank; p.K = K; p.cap = cap; p.e_per = e_per;
  for (int r = 0; r < world; ++r) {
    p.recv_x[r] = static_cast<uint8_t*>(recv_x[r]);
    p.recv_s[r] = static_cast<float*>(recv_s[r]);
    p.recv_ids[r] = static_cast<int*>(recv_ids[r]);
    p.recv_w[r] = static_cast<float*>(recv_w[r]);
    p.recv_count[r] = static_cast<int*>(recv_count[r]);
    p.flags[r] = static_cast<uint32_t*>(flags[r]);
    p.comb[r] = static_cast<__nv_bfloat16*>(comb[r]);
  }
  p.words = static_cast<uint32_t*>(words);
  return 0;
}
}  // namespace

// Dispatch this rank's T tokens (FP8 rows of row_bytes bytes, a multiple of 16) and wait for everybody's rows.
// send_slot [T, world] (out) is what combine needs later; recv_total (out, optional) gets the received row count.
extern "C" int mfq_moe_dispatch(const void* xq, const float* xs, const int* ids, const float* wt, int T, int row_bytes,
                                int* send_slot, int* recv_total, int world, int rank, int K, int cap, int e_per,
                                void* const* recv_x, void* const* recv_s, void* const* recv_ids, void* const* recv_w,
                                void* const* recv_count, void* const* flags, void* const* comb, void* words,
                                int* status, cudaStream_t stream) {
  A2aParams p;
  if (fill_params(p, world, rank, K, cap, e_per, recv_x, recv_s, recv_ids, recv_w, recv_count, flags, comb, words)) return -1;
  if (T < 0 || T > cap || row_bytes % 16) return -1;
  const int blocks = T == 0 ? 1 : min((T + 7) / 8, 4 * 148);
  moe_dispatch_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(xq), xs, ids, wt, T, row_bytes, send_slot, p,
                                                  status);
  moe_recv_wait_kernel<<<1, 256, 0, stream>>>(p, recv_total, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

// y [rows, H] bf16: expert outputs in route-plan order; dest [world*cap, K]: the plan's row of every (slot, k) pair.
// out[t] = base[t] + extra[t] + sum over ranks of the rows returned for token t.
extern "C" int mfq_moe_combine_a2a(const void* y, const int* dest, const int* send_slot, const void* base,
                                   const void* extra, void* out, int T, int H, int world, int rank, int K, int cap,
                                   int e_per, void* const* recv_x, void* const* recv_s, void* const* recv_ids,
                                   void* const* recv_w, void* const* recv_count, void* const* flags, void* const* comb,
                                   void* words, int* status, cudaStream_t stream) {
  A2aParams p;
  if (fill_params(p, world, rank, K, cap, e_per, recv_x, recv_s, recv_ids, recv_w, recv_count, flags, comb, words)) return -1;
  if (T < 0 || T > cap || H % 8) return -1;
  moe_combine_push_kernel<<<min(world * cap, 8 * 148), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(y), dest, H, p);
  moe_combine_reduce_kernel<<<max(T, 1), 256, 0, stream>>>(send_slot, static_cast<const __nv_bfloat16*>(base),
                                                           static_cast<const __nv_bfloat16*>(extra),
                                                           static_cast<__nv_bfloat16*>(out), T, H, p, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}
