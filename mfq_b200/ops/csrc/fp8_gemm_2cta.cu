// Block-scaled FP8 GEMM for wide batches on PAIRS of SMs:  out[M, N] = X[M, K] * W[N, K]^T  (prefill shapes)
//
// The one-CTA kernel (fp8_gemm.cu) streams 32 KB of operands from L2 per 128 x 128 x 128 block of products; at
// 4096^3 that is ~1 GB through the L2 -> SM path in 164 us, which is what bounds it (tensor pipe 20 % busy).  Here two
// CTAs of a cluster work on one 256 x BT tile with `tcgen05.mma.cta_group::2`: each CTA stages ITS 128 weight rows
// (UMMA A operand, M = 256 over the pair) and only HALF of the BT token rows (B operand, N = BT: the tensor core
// reads the other half from the peer CTA's shared memory), so a CTA loads 16 KB + BT/2 * 128 B per K block for
// 128 x BT x 128 products: 1.33x (BT = 128) and 2x (BT = 256) the products per byte of the one-CTA kernel.
//
// Roles per CTA: warp 0 = TMA producer, warp 1 = TMEM owner (and, in the leader CTA only, the MMA issuer), warps 2, 3
// idle (they complete the control warp group, which gives its registers away with `setmaxnreg`), warps 4..11 =
// epilogue (TMEM lane quarter = warp % 4, two warps per quarter split the token columns).  As in the one-CTA kernel
// every 128-wide K block lands in a fresh TMEM accumulator and the epilogue folds it, times the block's fp32
// multiplier, into registers while the tensor cores run the next block.  Cross-CTA signalling:
//   full[s]      lives in the leader; both CTAs' TMA loads complete their bytes on it (`.cta_group::2` loads may
//                signal the peer's barrier), the leader's producer arms it with the bytes of BOTH CTAs;
//   empty[s]     one per CTA; the leader commits to its own and to the peer's after the MMAs of the stage;
//   acc_full[b]  one per CTA, same pair of commits; acc_empty[b] lives in the leader and counts the epilogue warps of
//                both CTAs (the peer's arrive through the cluster address of the leader's barrier).
// The kernel is persistent: one pair per two SMs walks the tiles, all roles with continuing barrier phases, so a tile's
// prologue (first loads) and epilogue (store) hide under its neighbours' main loops; with one tile per launched CTA
// the fixed cost per tile was ~9 us of a 23 us tile at K = 4096.
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
  static constexpr int kThreads = 128 + 32 * kEpiWarps;  // warp group 0: TMA, MMA and two idle warps; groups 1, 2: epilogue
  static constexpr int kWsMax = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256 + kEpiWarps * kCols * 4 + kEpiWarps * kWsMax * 4;
};

struct PairParams {
  // Measurement switches (wrong numbers unless 0).  1: one accumulator over the whole K range, folded once -- the time
  // of the TMA + MMA pipeline alone, the bound for any way of folding.  2: the epilogue hands every accumulator back
  // without reading it (the cost of the hand-shakes alone).  4: it reads the accumulators but skips the FMAs.
  int single_fold;
  int fold_mode;
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

// Latency-critical waits (accumulator hand-over in both directions) poll with mbarrier.test_wait, which returns at once;
// try_wait may park the thread for a system-chosen time and was measured to add about a microsecond per hand-over.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_spin(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  if (mbar_test(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_test(bar, parity)) {
    if ((++spins & 0xFF) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kWaitBudgetNs) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
  return true;
}

__device__ unsigned long long g_stamp_issue;  // measurement switch 64: issue time of the stamped K block

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
  uint64_t* dummy_bar = acc_empty + Cfg::kAcc;  // measurement switch 16 only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dummy_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xs_smem = reinterpret_cast<float*>(tiles + Cfg::kStages * Cfg::kStageBytes + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();  // 0 = leader
  const bool leader = rank == 0;
  const int nkb = p.K / kBK;
  // Persistent: the pair walks the tiles  cluster, cluster + #clusters, ...; a tile = (pair of weight-row blocks,
  // token tile), token tiles innermost so that pairs running at the same time share the weight rows in L2.  Every
  // role runs the same tile loop with barrier phases that simply continue, so the loads and MMAs of the next tile
  // start while the epilogue warps still store the previous one.
  const int clusters = int(gridDim.x) / 2, cluster = int(blockIdx.x) / 2;
  const int t_tiles = (p.M + BT - 1) / BT, n_pairs = p.N / (2 * kRows);
  const int tiles_total = t_tiles * n_pairs;
  auto tile_n0 = [&](int tile) { return (tile / t_tiles) * 2 * kRows + int(rank) * kRows; };  // this CTA's weight rows
  auto tile_t0 = [&](int tile) { return (tile % t_tiles) * BT; };

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::kStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < Cfg::kAcc; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 2 * Cfg::kEpiWarps); }
    mbar_init(dummy_bar, 1);
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
  // The register file is the scarce resource of the fold: the control warp group hands its registers to the epilogue
  // groups, which then hold a thread's accumulators plus the raw columns of TWO K blocks at once.
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_w);
      tma_prefetch_desc(&tmap_x);
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster; ok && tile < tiles_total; tile += clusters) {
        const int n0 = tile_n0(tile), t0 = tile_t0(tile);
        for (int i = 0; i < nkb; ++i, s = (s + 1 == Cfg::kStages ? 0 : s + 1), phase ^= (s == 0 ? 1u : 0u)) {
          if (!mbar_wait(&empty[s], phase ^ 1u, abort_flag, p.status, kStatusTimeoutProducer)) { ok = false; break; }
          uint8_t* a = tiles + s * Cfg::kStageBytes;
          uint8_t* b = a + kRows * kBK;
          if (leader) mbar_expect_tx(&full[s], 2 * Cfg::kStageBytes);  // the bytes of both CTAs land on this barrier
          const uint32_t bar = map_to_cta(&full[s], 0);
          tma_load_2d_pair(a, &tmap_w, bar, i * kBK, n0);
          tma_load_2d_pair(b, &tmap_x, bar, i * kBK, t0 + int(rank) * (BT / 2));
        }
      }
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      constexpr uint32_t idesc = umma_idesc(2 * kRows, BT, 0, 0);
      int s = 0;
      uint32_t phase = 0, it = 0;  // it: accumulator blocks issued so far, over all tiles
      bool ok = true;
      for (int tile = cluster; ok && tile < tiles_total; tile += clusters) {
        for (int i = 0; i < nkb; ++i, s = (s + 1 == Cfg::kStages ? 0 : s + 1), phase ^= (s == 0 ? 1u : 0u)) {
          const bool fresh = !p.single_fold || i == 0;  // this K block opens a new accumulator
          const uint32_t buf = it % Cfg::kAcc;
          if (fresh && !mbar_wait(&acc_empty[buf], ((it / Cfg::kAcc) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutMma)) { ok = false; break; }
          const bool stamp = (p.fold_mode & 64) && blockIdx.x == 0 && tile == cluster;
          if (stamp && i == 10 + Cfg::kAcc) p.status[3] = int(globaltimer_ns() - g_stamp_issue);  // its accumulator came back
          if (stamp && i == 10) { *reinterpret_cast<volatile unsigned long long*>(&g_stamp_issue) = globaltimer_ns(); __threadfence(); }
          if (!mbar_wait(&full[s], phase, abort_flag, p.status, kStatusTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + s * Cfg::kStageBytes);
          const uint64_t a_desc = umma_desc_k_sw128(a_addr);
          const uint64_t b_desc = umma_desc_k_sw128(a_addr + kRows * kBK);
          // measurement switch 8 (with the single-accumulator switch): rotate the accumulator per K block all the same
          const bool rotate = p.single_fold && (p.fold_mode & 8);
          const uint32_t d = tmem_base + (rotate ? uint32_t(i % Cfg::kAcc) : buf) * BT;
#pragma unroll
          for (int k = 0; k < kBK / 32; ++k)
            umma_f8f6f4_pair(d, a_desc + uint64_t(k * 2), b_desc + uint64_t(k * 2), idesc, (k > 0 || (!fresh && !rotate)) ? 1u : 0u);
          // the stage is free, and the accumulator complete, in BOTH CTAs once these MMAs have retired
          tc_commit_pair(map_to_cta(&empty[s], 0));
          tc_commit_pair(map_to_cta(&empty[s], 1));
          if (p.fold_mode & 16) {  // measurement: two more commits per K block, nobody waits on them
            tc_commit_pair(map_to_cta(dummy_bar, 0));
            tc_commit_pair(map_to_cta(dummy_bar, 1));
          }
          const long long t_commit = clock64();
          if (!p.single_fold || i == nkb - 1) {
            tc_commit_pair(map_to_cta(&acc_full[buf], 0));
            tc_commit_pair(map_to_cta(&acc_full[buf], 1));
            if ((p.fold_mode & 32) && !p.single_fold) {
              // measurement: issue -> completion latency of one K block, seen by the issuing thread (unpipelined)
              while (!mbar_test(&acc_full[buf], (it / Cfg::kAcc) & 1)) {
              }
              if (blockIdx.x == 0 && tile == cluster && i == 10) p.status[2] = int(clock64() - t_commit);
            }
            ++it;
          }
        }
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    // ----- epilogue warps: thread owns weight row n0 + q*32 + lane and CW token columns from col0 -----
    constexpr int CW = Cfg::kCols;
    const int q = warp & 3;
    const int col0 = ((warp - 4) >> 2) * CW;
    const int row = q * 32 + lane;
    float* xs_w = xs_smem + (warp - 4) * CW;
    float* ws_w = xs_smem + Cfg::kEpiWarps * CW + (warp - 4) * Cfg::kWsMax;
    const bool ws_cached = nkb <= Cfg::kWsMax;
    const uint32_t acc_empty_leader0 = map_to_cta(&acc_empty[0], 0);
    bool ok = true;
    uint32_t it = 0;
    for (int tile = cluster; ok && tile < tiles_total; tile += clusters) {
      const int n0 = tile_n0(tile), t0 = tile_t0(tile);
      const int n = n0 + row;
      float acc[CW];
#pragma unroll
      for (int tt = 0; tt < CW; ++tt) acc[tt] = 0.f;
      const float* wsc = p.w_scale + size_t(n0 / kRows) * nkb;
      __syncwarp();  // the previous tile's reads of this warp's slices are done
      for (int j = lane; j < CW; j += 32) xs_w[j] = (t0 + col0 + j < p.M) ? __ldg(p.x_scale + t0 + col0 + j) : 0.f;
      if (ws_cached)
        for (int j = lane; j < nkb; j += 32) ws_w[j] = __ldg(wsc + j);
      __syncwarp();
      const int folds = p.single_fold ? 1 : nkb;
      int i = 0;
      if constexpr (CW <= 64) {
        // Two K blocks per TMEM round trip: the loads of both are in flight under ONE wait, so a warp pays the load
        // latency (the longest link of the wait -> load -> FMA chain) once per two blocks.  The accumulators are handed
        // back as soon as their columns sit in registers, before the FMAs.
        for (; ok && i + 1 < folds; i += 2, it += 2) {
          const uint32_t buf_a = it % Cfg::kAcc, buf_b = (it + 1) % Cfg::kAcc;
          // one lane polls (every poll is a shared-memory access, and shared memory is what the tensor cores stream from)
          if (lane == 0)
            ok = mbar_wait(&acc_full[buf_a], (it / Cfg::kAcc) & 1, abort_flag, p.status, kStatusTimeoutEpilogue) &&
                 mbar_wait(&acc_full[buf_b], ((it + 1) / Cfg::kAcc) & 1, abort_flag, p.status, kStatusTimeoutEpilogue);
          ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;
          if (!ok) break;
          tc_fence_after();
          const float sa = ws_cached ? ws_w[i] : __ldg(wsc + i), sb = ws_cached ? ws_w[i + 1] : __ldg(wsc + i + 1);
          const uint32_t lane_base = tmem_base + (uint32_t(q * 32) << 16) + col0;
          uint32_t ra[CW], rb[CW];
          if (p.fold_mode & 2) {
#pragma unroll
            for (int c = 0; c < CW; ++c) ra[c] = rb[c] = 0u;
          } else {
#pragma unroll
            for (int c = 0; c < CW; c += 32) {
              tmem_ld_32x32(lane_base + buf_a * BT + c, *reinterpret_cast<uint32_t(*)[32]>(ra + c));
              tmem_ld_32x32(lane_base + buf_b * BT + c, *reinterpret_cast<uint32_t(*)[32]>(rb + c));
            }
            tmem_wait_ld();
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive_cluster(acc_empty_leader0 + buf_a * 8);
            mbar_arrive_cluster(acc_empty_leader0 + buf_b * 8);
          }
          if (p.fold_mode & 4) {
            acc[0] += __uint_as_float(ra[0] ^ rb[CW - 1]);  // keeps the loads alive
          } else {
#pragma unroll
            for (int j = 0; j < CW; ++j) acc[j] = fmaf(__uint_as_float(rb[j]), sb, fmaf(__uint_as_float(ra[j]), sa, acc[j]));
          }
        }
      }
      for (; ok && i < folds; ++i, ++it) {
        const uint32_t buf = it % Cfg::kAcc;
        if (lane == 0) ok = mbar_wait(&acc_full[buf], (it / Cfg::kAcc) & 1, abort_flag, p.status, kStatusTimeoutEpilogue);
        ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;
        if ((p.fold_mode & 64) && blockIdx.x < 2 && tile == cluster && i == 10 && warp == 4 && lane == 0)
          p.status[1 + blockIdx.x] = int(globaltimer_ns() - *reinterpret_cast<volatile unsigned long long*>(&g_stamp_issue));
        if (!ok) break;
        tc_fence_after();
        const float s = ws_cached ? ws_w[i] : __ldg(wsc + i);
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * BT + col0;
#pragma unroll
        for (int c = 0; c < CW; c += 64) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(taddr + c, r0);
          tmem_ld_32x32(taddr + c + 32, r1);
          tmem_wait_ld();
          if (c + 64 >= CW) {  // all columns of this block are in registers: hand the accumulator back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_leader0 + buf * 8);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c + j] = fmaf(__uint_as_float(r0[j]), s, acc[c + j]);
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c + 32 + j] = fmaf(__uint_as_float(r1[j]), s, acc[c + 32 + j]);
        }
      }
      if (ok && n < p.N) {
        const int tl = min(BT, p.M - t0);
        // residual and output may be one buffer: all loads first, or every load would wait behind the store before it
        if (p.residual) {
          unsigned short res[CW];
          const unsigned short* rp = reinterpret_cast<const unsigned short*>(p.residual);
#pragma unroll
          for (int tt = 0; tt < CW; ++tt)
            res[tt] = (col0 + tt < tl) ? __ldcg(rp + size_t(t0 + col0 + tt) * p.N + n) : (unsigned short)0;
#pragma unroll
          for (int tt = 0; tt < CW; ++tt) acc[tt] = fmaf(acc[tt], xs_w[tt], __uint_as_float(uint32_t(res[tt]) << 16));
        } else {
#pragma unroll
          for (int tt = 0; tt < CW; ++tt) acc[tt] *= xs_w[tt];
        }
#pragma unroll
        for (int tt = 0; tt < CW; ++tt) {
          if (col0 + tt < tl) p.out[size_t(t0 + col0 + tt) * p.N + n] = __float2bfloat16(acc[tt]);
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
  static const int single_fold = [] { const char* e = getenv("MFQ_PAIR_SINGLE_FOLD"); return e ? atoi(e) : 0; }();
  static const int fold_mode = [] { const char* e = getenv("MFQ_PAIR_FOLD_MODE"); return e ? atoi(e) : 0; }();
  PairParams p{single_fold, fold_mode, w_scale, x_scale, static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(residual), status, M, N, K};
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = (N / (2 * kRows)) * ((M + BT - 1) / BT);
  const int clusters = tiles < sms / 2 ? tiles : sms / 2;
  fp8_gemm_pair_kernel<BT><<<dim3(2 * clusters), Cfg::kThreads, Cfg::kSmemBytes, stream>>>(tw, tx, p);
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
