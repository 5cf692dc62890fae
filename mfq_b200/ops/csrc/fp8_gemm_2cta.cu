// Block-scaled FP8 GEMM for wide batches on PAIRS of SMs:  out[M, N] = X[M, K] * W[N, K]^T  (prefill shapes)
//
// The one-CTA kernel (fp8_gemm.cu) streams 32 KB of operands from L2 per 128 x 128 x 128 block of products; at
// 4096^3 that is ~1 GB through the L2 -> SM path in 164 us, which is what bounds it (tensor pipe 20 % busy).  Here two
// CTAs of a cluster work on one 256 x BT tile with `tcgen05.mma.cta_group::2`: each CTA stages ITS 128 weight rows
// (UMMA A operand, M = 256 over the pair) and only HALF of the BT token rows (B operand, N = BT: the tensor core
// reads the other half from the peer CTA's shared memory), so a CTA loads 16 KB + BT/2 * 128 B per K block for
// 128 x BT x 128 products: 1.33x (BT = 128) and 2x (BT = 256) the products per byte of the one-CTA kernel.
//
// Roles per CTA: warp 0 = TMA producer, warp 1 = TMEM owner (and, in the leader CTA only, the MMA issuer), warps 2..9
// = epilogue (TMEM lane quarter = warp % 4, two warps per quarter split the token columns).  As in the one-CTA kernel
// every 128-wide K block lands in a fresh TMEM accumulator and the epilogue folds it, times the block's fp32
// multiplier, into registers while the tensor cores run the next block.  Cross-CTA signalling:
//   full[s]      lives in the leader; both CTAs' TMA loads complete their bytes on it (`.cta_group::2` loads may
//                signal the peer's barrier), the leader's producer arms it with the bytes of BOTH CTAs;
//   empty[s]     one per CTA; the leader commits to its own and to the peer's after the MMAs of the stage;
//   acc_full[b]  one per CTA, same pair of commits; acc_empty[b] lives in the leader and counts the epilogue warps of
//                both CTAs (the peer's arrive through the cluster address of the leader's barrier).
// No load is multicast; the pair shares the token tile through the tensor core's own peer read.
// All waits are bounded; a cluster barrier before the TMEM release keeps a CTA alive while its peer may still read it.
//
// The reference has no FP8 tensor-core path (mfq/kernels/cuda/fp8_sq.cu:564-592 decodes to fp16 for wmma / cuBLAS).
#include "common.cuh"

#include <cstdlib>

namespace mfq {
namespace {

constexpr int kRows = 128;    // weight rows per CTA
constexpr int kBK = 128;      // fp8 elements per K block

template <int BT>
struct PairCfg {
  static constexpr int kStages = 6;
  static constexpr int kAcc = 512 / BT;  // accumulators of BT columns: all of TMEM
  static constexpr int kStageBytes = kRows * kBK + (BT / 2) * kBK;
  static constexpr int kEpiWarps = 8;
  static constexpr int kCols = BT / 2;   // token columns per epilogue thread
  static constexpr int kThreads = 64 + 32 * kEpiWarps;
  static constexpr int kWsMax = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256 + kEpiWarps * kCols * 4 + kEpiWarps * kWsMax * 4;
};

struct PairParams {
  const float* w_scale;
  const float* x_scale;
  __nv_bfloat16* out;
  const __nv_bfloat16* residual;
  int* status;
  int M, N, K;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(const void* smem_ptr, uint32_t cta) {  // cluster address of a peer's variable
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(smem_ptr)), "r"(cta));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {  // one warp in EACH CTA of the pair
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// 2-D tile load whose bytes complete on a barrier given by its cluster address (the leader's, from either CTA).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* desc, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_f8f6f4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at `bar_cluster_addr` (any CTA of the cluster) once the MMAs issued so far have retired.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

template <int BT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg<BT>::kThreads, 1)
fp8_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                     const PairParams p) {
  using Cfg = PairCfg<BT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* full = bars;                       // used in the leader only
  uint64_t* empty = bars + Cfg::kStages;       // one set per CTA
  uint64_t* acc_full = bars + 2 * Cfg::kStages;
  uint64_t* acc_empty = acc_full + Cfg::kAcc;  // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + Cfg::kAcc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xs_smem = reinterpret_cast<float*>(tiles + Cfg::kStages * Cfg::kStageBytes + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();  // 0 = leader
  const bool leader = rank == 0;
  const int n0 = int(blockIdx.x) * kRows;     // this CTA's weight rows (the pair covers 256 consecutive rows)
  const int t0 = int(blockIdx.y) * BT;        // the pair's token tile
  const int nkb = p.K / kBK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::kStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < Cfg::kAcc; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 2 * Cfg::kEpiWarps); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anybody signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_w);
      tma_prefetch_desc(&tmap_x);
      int s = 0;
      uint32_t phase = 0;
      for (int i = 0; i < nkb; ++i, s = (s + 1 == Cfg::kStages ? 0 : s + 1), phase ^= (s == 0 ? 1u : 0u)) {
        if (!mbar_wait(&empty[s], phase ^ 1u, abort_flag, p.status, kStatusTimeoutProducer)) break;
        uint8_t* a = tiles + s * Cfg::kStageBytes;
        uint8_t* b = a + kRows * kBK;
        if (leader) mbar_expect_tx(&full[s], 2 * Cfg::kStageBytes);  // the bytes of both CTAs land on this barrier
        const uint32_t bar = map_to_cta(&full[s], 0);
        tma_load_2d_pair(a, &tmap_w, bar, i * kBK, n0);
        tma_load_2d_pair(b, &tmap_x, bar, i * kBK, t0 + int(rank) * (BT / 2));
      }
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      constexpr uint32_t idesc = umma_idesc(2 * kRows, BT, 0, 0);
      int s = 0;
      uint32_t phase = 0;
      for (int i = 0; i < nkb; ++i, s = (s + 1 == Cfg::kStages ? 0 : s + 1), phase ^= (s == 0 ? 1u : 0u)) {
        const int buf = i % Cfg::kAcc;
        if (!mbar_wait(&acc_empty[buf], ((i / Cfg::kAcc) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutMma)) break;
        if (!mbar_wait(&full[s], phase, abort_flag, p.status, kStatusTimeoutMma)) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(tiles + s * Cfg::kStageBytes);
        const uint64_t a_desc = umma_desc_k_sw128(a_addr);
        const uint64_t b_desc = umma_desc_k_sw128(a_addr + kRows * kBK);
        const uint32_t d = tmem_base + buf * BT;
#pragma unroll
        for (int k = 0; k < kBK / 32; ++k)
          umma_f8f6f4_pair(d, a_desc + uint64_t(k * 2), b_desc + uint64_t(k * 2), idesc, k > 0 ? 1u : 0u);
        // the stage is free, and the accumulator complete, in BOTH CTAs once these MMAs have retired
        tc_commit_pair(map_to_cta(&empty[s], 0));
        tc_commit_pair(map_to_cta(&empty[s], 1));
        tc_commit_pair(map_to_cta(&acc_full[buf], 0));
        tc_commit_pair(map_to_cta(&acc_full[buf], 1));
      }
    }
  } else {
    // ----- epilogue warps: thread owns weight row n0 + q*32 + lane and CW token columns from col0 -----
    constexpr int CW = Cfg::kCols;
    const int q = warp & 3;
    const int col0 = ((warp - 2) >> 2) * CW;
    const int row = q * 32 + lane;
    const int n = n0 + row;
    float acc[CW];
#pragma unroll
    for (int tt = 0; tt < CW; ++tt) acc[tt] = 0.f;
    const int n_tiles = p.N / kRows;
    const float* wsc = p.w_scale + size_t(blockIdx.x) * nkb;
    float* xs_w = xs_smem + (warp - 2) * CW;
    for (int j = lane; j < CW; j += 32) xs_w[j] = (t0 + col0 + j < p.M) ? __ldg(p.x_scale + t0 + col0 + j) : 0.f;
    float* ws_w = xs_smem + Cfg::kEpiWarps * CW + (warp - 2) * Cfg::kWsMax;
    const bool ws_cached = nkb <= Cfg::kWsMax;
    if (ws_cached)
      for (int j = lane; j < nkb; j += 32) ws_w[j] = __ldg(wsc + j);
    __syncwarp();
    (void)n_tiles;
    const uint32_t acc_empty_leader0 = map_to_cta(&acc_empty[0], 0);
    bool ok = true;
    for (int i = 0; i < nkb; ++i) {
      const int buf = i % Cfg::kAcc;
      ok = mbar_wait(&acc_full[buf], (i / Cfg::kAcc) & 1, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float s = ws_cached ? ws_w[i] : __ldg(wsc + i);
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * BT + col0;
#pragma unroll
      for (int c = 0; c < CW; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[c + j] = fmaf(__uint_as_float(r[j]), s, acc[c + j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader0 + buf * 8);
    }
    if (ok && n < p.N) {
      const int tl = min(BT, p.M - t0);
#pragma unroll
      for (int tt = 0; tt < CW; ++tt) {
        if (col0 + tt < tl) {
          float v = acc[tt] * xs_w[tt];
          const size_t o = size_t(t0 + col0 + tt) * p.N + n;
          if (p.residual) v += __bfloat162float(p.residual[o]);
          p.out[o] = __float2bfloat16(v);
        }
      }
    }
  }

  // ----- teardown: every thread of both CTAs arrives here, also after an aborted wait; nobody leaves (and frees
  //       memory the peer's tensor core may still read) before the other has finished -----
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

template <int BT>
int launch_pair(const void* w, const float* w_scale, const void* x, const float* x_scale, void* out, const void* residual,
                int* status, int M, int N, int K, cudaStream_t stream) {
  using Cfg = PairCfg<BT>;
  CUtensorMap tw, tx;
  if (make_tmap_2d(&tw, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, K, kRows, kBK)) return -2;
  if (make_tmap_2d(&tx, x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, BT / 2, kBK)) return -3;
  static bool attr_set[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -6;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(fp8_gemm_pair_kernel<BT>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
      return -6;
    attr_set[dev] = true;
  }
  PairParams p{w_scale, x_scale, static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(residual), status, M, N, K};
  fp8_gemm_pair_kernel<BT><<<dim3(N / kRows, (M + BT - 1) / BT), Cfg::kThreads, Cfg::kSmemBytes, stream>>>(tw, tx, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

}  // namespace
}  // namespace mfq

// Two-SM form of mfq_fp8_gemm for wide batches.  N % 256 == 0, K % 128 == 0, token_tile in {128, 256}; no split-K.
extern "C" int mfq_fp8_gemm_pair(const void* w, const float* w_scale, const void* x, const float* x_scale, void* out,
                                 const void* residual, int* status, int M, int N, int K, int token_tile,
                                 cudaStream_t stream) {
  if (K % 128 != 0 || N % 256 != 0 || M <= 0) return -1;
  if (token_tile == 128) return mfq::launch_pair<128>(w, w_scale, x, x_scale, out, residual, status, M, N, K, stream);
  if (token_tile == 256) return mfq::launch_pair<256>(w, w_scale, x, x_scale, out, residual, status, M, N, K, stream);
  return -1;
}
