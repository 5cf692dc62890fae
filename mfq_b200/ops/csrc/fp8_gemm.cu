// Block-scaled FP8 GEMM on tcgen05 tensor cores:  out[M, N] = X[M, K] * W[N, K]^T
//
//   W : E4M3, one fp32 multiplier per 128x128 block   (w_scale[ceil(N/128), K/128])
//   X : E4M3, one fp32 multiplier per token            (x_scale[M])
//   out : bf16 (optionally + bf16 residual)
//
// The weight tile is the UMMA "A" operand (M = 128 output features) and the token tile the "B"
// operand (N = BT tokens), so the same kernel streams weights at decode batch sizes (BT = 16..64)
// and runs square tiles at prefill (BT = 128).  Because the weight multiplier changes every 128 inputs,
// each 128-wide K block is multiplied into a fresh TMEM accumulator (NACC of them rotate) and
// the epilogue warps fold it, scaled, into fp32 registers while the tensor core already works on
// the next block.
//
// Roles: warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2.. = epilogue (TMEM lane quarter =
// warp % 4; token tiles of 64 and 128 use two warps per quarter, each folding half of the token columns).  Split-K (gridDim.z > 1) writes fp32 partials to a scratch
// buffer; the last CTA to arrive at a tile's counter reduces them in split order (deterministic)
// and resets the counter for the next launch.
//
// The reference multiplies block-FP8 weights by decoding them to fp16 for wmma or cuBLAS
// (mfq/kernels/cuda/fp8_sq.cu:42-56,564-592); there the FP8 tensor-core path does not exist.
#include "common.cuh"

namespace mfq {

constexpr int kTileN = 128;     // weight rows (output features) per CTA
constexpr int kBlockK = 128;    // fp8 elements per K block = one 128-byte swizzle row

template <int BT>
struct GemmCfg {
  static constexpr int kStages = BT >= 128 ? 6 : 8;
  static constexpr int kAcc = 4;
  static constexpr int kTmemCols = (kAcc * BT) < 32 ? 32 : kAcc * BT;
  static constexpr int kStageBytes = kTileN * kBlockK + BT * kBlockK;
  // Epilogue warps: one per TMEM lane quarter, doubled for wide token tiles (the two warps of a quarter split the
  // token columns), so that two warps per scheduler hide each other's TMEM-load and FMA latencies.
  static constexpr int kEpiWarps = BT >= 64 ? 8 : 4;
  static constexpr int kCols = BT / (kEpiWarps / 4);   // token columns per epilogue thread
  static constexpr int kThreads = 64 + 32 * kEpiWarps;
  static constexpr int kXsBytes = kEpiWarps * kCols * 4;  // per-warp copy of the row multipliers of its token columns
  static constexpr int kWsMax = 256;                      // weight-block multipliers of a CTA's K range kept in smem, per warp
  static constexpr int kWsBytes = kEpiWarps * kWsMax * 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align slack*/ + 256 /*barriers*/ + kXsBytes + kWsBytes;
};

// Cross-rank all-reduce context of the fused epilogue (world == 1: disabled).
struct ArParams {
  int world = 1, rank = 0;
  float* bufs[8] = {};        // every rank's partial buffer (own + peer-mapped): 2 halves of half_elems floats
  uint32_t* flags[8] = {};    // every rank's per-tile arrival counters (own + peer-mapped)
  uint32_t* expected = nullptr;  // local: value of our flag after the previous launch, per tile
  size_t half_elems = 0;
  // 0: all-reduce (every rank ends with the full [M, N] sum).  1: reduce-scatter over token rows: rank r owns the
  // token tiles [r * T/W, (r+1) * T/W); the other ranks push their partial tile into the owner's buffer (one slot
  // per source rank) and only the owner sums; `out` / `residual` are then the owner's [M/W, N] shard.
  int mode = 0;
};

// All-gather -> GEMM context (world == 1: disabled).  The activation is sharded over token rows; the first
// `push_ctas` blocks of the grid copy this rank's FP8 shard (+ row multipliers) into every rank's gathered buffer
// over NVLink and bump per-source flags, the GEMM blocks' TMA producers wait for the flag of the rank that owns
// their token tile and then read the tile from *local* memory, so every byte crosses NVLink once and tiles of
// early ranks are multiplied while later shards are still in flight.
struct AgParams {
  int world = 1, rank = 0, push_ctas = 0, shard_rows = 0;
  uint8_t* x_full[8] = {};        // every rank's gathered activations: 2 halves of M * K bytes
  float* xs_full[8] = {};         // every rank's gathered row multipliers: 2 halves of M floats
  uint32_t* flags[8] = {};        // every rank's arrival counters, one per source rank
  const uint8_t* x_shard = nullptr;
  const float* xs_shard = nullptr;
  const uint32_t* epoch = nullptr;   // completed launches on this context (bumped by a 1-thread kernel afterwards)
  uint32_t* push_done = nullptr;     // local counters of finished push blocks, one per destination step (return to zero)
};

struct GemmParams {
  const float* w_scale;
  const float* x_scale;
  __nv_bfloat16* out;
  const __nv_bfloat16* residual;
  float* ws;        // split-K partials: [splits][t_tiles][n_tiles][BT][128]
  int* counters;    // [t_tiles * n_tiles], zero on entry, zero on exit
  int* status;
  int M, N, K;
  int kb_per_split;
  ArParams ar;
  // Grouped (mixture-of-experts) mode: blockIdx.y indexes tile_map = (expert, token tile inside the expert), rows of
  // x / out are the expert-sorted token rows, expert e owning rows [expert_offsets[e], expert_offsets[e+1]).
  const int2* tile_map = nullptr;
  const int* expert_offsets = nullptr;
  AgParams ag;
  int stages = 0;  // depth of the shared-memory ring actually used (<= GemmCfg::kStages); fewer stages = more CTAs per SM
  // Split-K with the splits of a tile launched as one thread-block cluster: the partial sums meet in distributed shared
  // memory instead of a global scratch buffer with an arrival counter, and every CTA of the cluster finishes a share of
  // the token columns instead of the last arriver finishing all of them.
  int cluster_reduce = 0;
};

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
  return r;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Cluster split-K: CTA r of S finishes the token columns c = r (mod S); a thread owns one output row and every kSel-th
// of those columns.  The S partials of a column are summed in split order whichever CTA does it, so results do not
// depend on scheduling.  Every load of the thread -- S remote partials per column, multipliers, residual values -- leaves
// before the first sum, so the round trips through the cluster's shared memory overlap (in groups of at most kLoads
// partials to bound the registers).  Fetching multipliers and residuals ahead of the barrier measured slower: the values
// have to be held across it, and the registers for that spill.
template <int BT, int S>
__device__ __forceinline__ void cluster_sum_columns(const GemmParams& p, const uint8_t* tiles, int t0, int tl, int n0) {
  using Cfg = GemmCfg<BT>;
  constexpr int kSel = Cfg::kEpiWarps / 4;
  constexpr int kLoads = 32;
  constexpr int kGroup = kLoads / S < 1 ? 1 : kLoads / S;
  const int e = int(threadIdx.x) - 64, row = e & 127, sel = e >> 7;
  const int r = int(cluster_cta_rank());
  const int n = n0 + row;
  const uint32_t mine = smem_u32(tiles) + uint32_t(row) * 4u;
  uint32_t base[S];
#pragma unroll
  for (int z = 0; z < S; ++z) base[z] = map_to_cta(mine, uint32_t(z));
  const unsigned short* rp = reinterpret_cast<const unsigned short*>(p.residual);
  constexpr int step = S * kSel;
  for (int c0 = r + S * sel; c0 < tl; c0 += step * kGroup) {
    float v[kGroup][S], xm[kGroup];
    unsigned short res[kGroup];
#pragma unroll
    for (int j = 0; j < kGroup; ++j) {
      const int c = c0 + j * step;
      const bool live = c < tl;
      xm[j] = live ? __ldg(p.x_scale + t0 + c) : 0.f;
      res[j] = (live && rp && n < p.N) ? __ldcg(rp + size_t(t0 + c) * p.N + n) : (unsigned short)0;
#pragma unroll
      for (int z = 0; z < S; ++z) v[j][z] = live ? ld_cluster_f32(base[z] + uint32_t(c) * (kTileN * 4u)) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kGroup; ++j) {
      const int c = c0 + j * step;
      float sum = 0.f;
#pragma unroll
      for (int z = 0; z < S; ++z) sum += v[j][z];  // split order
      sum = sum * xm[j] + __uint_as_float(uint32_t(res[j]) << 16);
      if (c < tl && n < p.N) p.out[size_t(t0 + c) * p.N + n] = __float2bfloat16(sum);
    }
  }
}

template <int BT>
__global__ void __launch_bounds__(GemmCfg<BT>::kThreads, (BT <= 64 ? 2 : 1))
fp8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                const __grid_constant__ CUtensorMap tmap_x_alt, const GemmParams p) {
  using Cfg = GemmCfg<BT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stages = p.stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + stages * Cfg::kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + stages;
  uint64_t* acc_full = bars + 2 * stages;
  uint64_t* acc_empty = acc_full + Cfg::kAcc;
  uint64_t* epi_bar = acc_empty + Cfg::kAcc;  // four one-shot barriers among the epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(epi_bar + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);
  float* xs_smem = reinterpret_cast<float*>(tiles + stages * Cfg::kStageBytes + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool gather = p.ag.world > 1;
  pdl_trigger();
  // Modes whose prologue already reads memory an earlier kernel wrote (the gathered-activation epoch, the route plan
  // of the grouped mode) wait for their predecessor right away; the plain GEMM first sets up barriers and TMEM.
  const bool early_inputs = gather || p.tile_map != nullptr;
  if (early_inputs) pdl_wait();
  const uint32_t ag_epoch = gather ? *p.ag.epoch : 0u;
  if (gather && int(blockIdx.x) < p.ag.push_ctas) {
    // ----- push block: copy my shard into every rank's gathered buffer, then announce it -----
    if (blockIdx.y != 0 || blockIdx.z != 0) return;
    const AgParams& ag = p.ag;
    const size_t shard_bytes = size_t(ag.shard_rows) * p.K;
    const size_t half = size_t(ag_epoch & 1u) * size_t(p.M) * p.K;
    const uint4* src = reinterpret_cast<const uint4*>(ag.x_shard);
    const size_t nvec = shard_bytes / 16;
    const bool small_shard = shard_bytes <= (256u << 10);
    for (int rr = 0; rr < ag.world; ++rr) {
      const int r = (ag.rank + rr) % ag.world;  // own copy first, then a different destination on every rank (no incast)
      uint4* dst = reinterpret_cast<uint4*>(ag.x_full[r] + half + size_t(ag.rank) * shard_bytes);
      const size_t stride = size_t(ag.push_ctas) * blockDim.x;
      size_t v = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
      for (; v + 3 * stride < nvec; v += 4 * stride) {  // four independent 16-byte copies in flight per thread
        const uint4 a0 = src[v], a1 = src[v + stride], a2 = src[v + 2 * stride], a3 = src[v + 3 * stride];
        dst[v] = a0; dst[v + stride] = a1; dst[v + 2 * stride] = a2; dst[v + 3 * stride] = a3;
      }
      for (; v < nvec; v += stride) dst[v] = src[v];
      float* sdst = ag.xs_full[r] + size_t(ag_epoch & 1u) * p.M + size_t(ag.rank) * ag.shard_rows;
      for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < ag.shard_rows; i += ag.push_ctas * blockDim.x) sdst[i] = ag.xs_shard[i];
      if (small_shard) continue;  // announced below, after ONE fence for the whole fan-out
      // one completion counter per destination: a rank learns that my shard has arrived as soon as ITS copy is done
      // (my own tiles after the local copy, rank+1 next, ...), not when the whole fan-out has finished
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x == 0) {
        const uint32_t prev = atomicAdd(ag.push_done + rr, 1u);
        if (prev == uint32_t(ag.push_ctas) - 1u) {
          ag.push_done[rr] = 0;
          __threadfence_system();
          asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(ag.flags[r] + ag.rank) : "memory");
        }
      }
    }
    if (small_shard) {
      // a system-scope fence costs a round trip to the farthest destination; with a few KB per destination the copies
      // are cheaper than the fences, so fence once and raise every flag together
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x == 0) {
        const uint32_t prev = atomicAdd(ag.push_done, 1u);
        if (prev == uint32_t(ag.push_ctas) - 1u) {
          ag.push_done[0] = 0;
          __threadfence_system();
          for (int rr = 0; rr < ag.world; ++rr) {
            const int r = (ag.rank + rr) % ag.world;
            asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(ag.flags[r] + ag.rank) : "memory");
          }
        }
      }
    }
    return;
  }
  const int n_tile = int(blockIdx.x) - (gather ? p.ag.push_ctas : 0), split = blockIdx.z;
  // Reduce-scatter: rank r starts with the token tiles owned by rank r+1 and ends with its own, so that at any moment
  // the W ranks push their partials to W different owners instead of all into one GPU's NVLink ingress.
  int t_tile = blockIdx.y;
  if (p.ar.world > 1 && p.ar.mode == 1) {
    t_tile = int((blockIdx.y + unsigned(p.ar.rank + 1) * (gridDim.y / unsigned(p.ar.world))) % gridDim.y);
  } else if (gather && gridDim.y % unsigned(p.ag.world) == 0) {
    // All-gather: shards reach this rank in the order own, rank-1, rank-2, ... (see the push loop), so the token
    // tiles are visited in that order and the first tiles never wait for the last shard to arrive.
    const int per = int(gridDim.y) / p.ag.world;
    const int shard = (p.ag.rank - int(blockIdx.y) / per + p.ag.world) % p.ag.world;
    t_tile = shard * per + int(blockIdx.y) % per;
  }
  const int n_tiles_x = int(gridDim.x) - (gather ? p.ag.push_ctas : 0);
  const int n0 = n_tile * kTileN;
  int t0 = t_tile * BT, row_end = p.M, expert = 0;
  if (p.tile_map) {
    const int2 tm = p.tile_map[t_tile];
    if (tm.x < 0) return;  // padding entry of the tile map: uniform for the whole CTA, nothing allocated yet
    expert = tm.x;
    t0 = p.expert_offsets[expert] + tm.y * BT;
    row_end = p.expert_offsets[expert + 1];
  }
  const int kb_total = p.K / kBlockK;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(kb_total, kb0 + p.kb_per_split);
  const int nkb = kb1 - kb0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < stages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < Cfg::kAcc; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], Cfg::kEpiWarps); }
    for (int i = 0; i < 4; ++i) mbar_init(&epi_bar[i], Cfg::kEpiWarps);
    *abort_flag = 0;
    *last_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Weights are never written by a kernel of the same stream, so the plain GEMM starts the weight tiles of its first
  // ring pass BEFORE it waits for its predecessor: under programmatic dependent launch this CTA is resident while the
  // short kernel that produces its activations (a norm, a quantization) still runs, and the weight stream -- all of it
  // for a short K range -- arrives under that kernel instead of after it.  The activation tiles follow the wait.
  int w_ahead = 0;
  if (!early_inputs) {
    if (warp == 0 && lane == 0) {
      tma_prefetch_desc(&tmap_w);
      tma_prefetch_desc(&tmap_x);
      w_ahead = min(nkb, stages);
      for (int i = 0; i < w_ahead; ++i) {
        mbar_expect_tx(&full[i], Cfg::kStageBytes);
        tma_load_2d(tiles + i * Cfg::kStageBytes, &tmap_w, &full[i], (kb0 + i) * kBlockK, n0);
      }
    }
    pdl_wait();
  }

  if (warp == 0) {
    if (lane == 0) {
      if (early_inputs) {
        tma_prefetch_desc(&tmap_w);
        tma_prefetch_desc(&tmap_x);
      }
      const CUtensorMap* xmap = (gather && (ag_epoch & 1u)) ? &tmap_x_alt : &tmap_x;
      bool shard_ready = true;
      if (gather) {
        // both shards that a token tile may straddle are awaited (tiles are aligned to shards in practice)
        const int first = t0 / p.ag.shard_rows, last = min(p.ag.world - 1, (t0 + BT - 1) / p.ag.shard_rows);
        const unsigned long long t_start = globaltimer_ns();
        for (int src = first; src <= last && shard_ready; ++src) {
          const uint32_t* f = p.ag.flags[p.ag.rank] + src;
          uint32_t seen, spins = 0;
          while (true) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(f) : "memory");
            if (int32_t(seen - (ag_epoch + 1u)) >= 0) break;
            if ((++spins & 0x3F) == 0 && (*abort_flag || globaltimer_ns() - t_start > kWaitBudgetNs)) {
              *abort_flag = 1;
              atomicCAS(p.status, 0, kStatusTimeoutPeer | (1 << 8));
              shard_ready = false;
              break;
            }
          }
        }
        fence_proxy_async_smem();
        asm volatile("fence.proxy.async.global;" ::: "memory");  // peers' generic-proxy stores -> my TMA reads
      }
      int s = 0;
      uint32_t ring_phase = 0;  // ring position and wrap parity, kept incrementally: the depth is a run-time value
      for (int i = 0; shard_ready && i < nkb; ++i, s = (s + 1 == stages ? 0 : s + 1), ring_phase ^= (s == 0 ? 1u : 0u)) {
        uint8_t* a = tiles + s * Cfg::kStageBytes;
        uint8_t* b = a + kTileN * kBlockK;
        if (i >= w_ahead) {  // the first pass of the plain mode is armed and its weight tile on the way already
          if (!mbar_wait(&empty[s], ring_phase ^ 1u, abort_flag, p.status, kStatusTimeoutProducer)) break;
          mbar_expect_tx(&full[s], Cfg::kStageBytes);
          if (p.tile_map) tma_load_3d(a, &tmap_w, &full[s], (kb0 + i) * kBlockK, n0, expert);
          else tma_load_2d(a, &tmap_w, &full[s], (kb0 + i) * kBlockK, n0);
        }
        tma_load_2d(b, xmap, &full[s], (kb0 + i) * kBlockK, t0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // This one thread's loop is the pace of a weight-streaming CTA whose tiles are already in shared memory, so it
      // carries no work that can be left out: descriptors advance by a constant per stage (the ring is contiguous and
      // stays inside the 14-bit address field), a fresh accumulator is not waited for, and a stage that no later K
      // block reuses is not handed back.
      constexpr uint32_t idesc = umma_idesc(kTileN, BT, 0, 0);
      constexpr uint64_t kStageStep = uint64_t(Cfg::kStageBytes >> 4);
      const uint64_t a_desc0 = umma_desc_k_sw128(smem_u32(tiles));
      const uint64_t b_desc0 = umma_desc_k_sw128(smem_u32(tiles) + kTileN * kBlockK);
      int s = 0;
      uint32_t ring_phase = 0;
      for (int i = 0; i < nkb; ++i, s = (s + 1 == stages ? 0 : s + 1), ring_phase ^= (s == 0 ? 1u : 0u)) {
        const int buf = i % Cfg::kAcc;
        if (i >= Cfg::kAcc &&
            !mbar_wait(&acc_empty[buf], ((i / Cfg::kAcc) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutMma)) break;
        if (!mbar_wait(&full[s], ring_phase, abort_flag, p.status, kStatusTimeoutMma)) break;
        tc_fence_after();
        const uint64_t a_desc = a_desc0 + uint64_t(s) * kStageStep;
        const uint64_t b_desc = b_desc0 + uint64_t(s) * kStageStep;
        const uint32_t d = tmem_base + buf * BT;
#pragma unroll
        for (int k = 0; k < kBlockK / 32; ++k) {
          // advancing 32 bytes along K inside the swizzle row = +2 in the 16-byte address field
          umma_f8f6f4(d, a_desc + uint64_t(k * 2), b_desc + uint64_t(k * 2), idesc, k > 0 ? 1u : 0u);
        }
        if (i + stages < nkb) tc_commit(&empty[s]);  // smem stage reusable once these MMAs have read it
        tc_commit(&acc_full[buf]);                   // accumulator block complete
      }
    }
  } else {
    // ----- epilogue warps: thread owns output feature n0 + q*32 + lane and CW token columns from col0 -----
    constexpr int CW = Cfg::kCols;
    const int q = warp & 3;
    const int col0 = ((warp - 2) >> 2) * CW;
    const int row = q * 32 + lane;
    const int n = n0 + row;
    float acc[CW];
#pragma unroll
    for (int tt = 0; tt < CW; ++tt) acc[tt] = 0.f;
    const float* wsc = p.w_scale + (size_t(expert) * n_tiles_x + n_tile) * kb_total;
    // The token multipliers are fetched now, under the main loop, into this warp's own smem slice (no cross-warp
    // sync needed); at the end they cost a broadcast LDS instead of an exposed global load per column.  In gather
    // mode they only exist once the peers' flags arrived, so that mode reads them at the end.
    float* xs_w = xs_smem + (warp - 2) * CW;
    if (!gather) {
      for (int j = lane; j < CW; j += 32) xs_w[j] = (t0 + col0 + j < row_end) ? __ldg(p.x_scale + t0 + col0 + j) : 0.f;
    }
    // The weight-block multipliers of this CTA's K range, likewise: a global load per K block would sit, exposed, on
    // the chain wait -> TMEM load -> FMA that every block goes through (it was the longest link of that chain).
    float* ws_w = xs_smem + Cfg::kEpiWarps * CW + (warp - 2) * Cfg::kWsMax;
    const bool ws_cached = nkb <= Cfg::kWsMax;
    if (ws_cached) {
      for (int j = lane; j < nkb; j += 32) ws_w[j] = __ldg(wsc + kb0 + j);
    }
    __syncwarp();
    bool ok = true;
    for (int i = 0; i < nkb; ++i) {
      const int buf = i % Cfg::kAcc;
      ok = mbar_wait(&acc_full[buf], (i / Cfg::kAcc) & 1, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float s = ws_cached ? ws_w[i] : __ldg(wsc + kb0 + i);
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + buf * BT + col0;
      if constexpr (CW == 64) {
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(taddr, r0);        // both loads in flight before the single wait
        tmem_ld_32x32(taddr + 32, r1);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = fmaf(__uint_as_float(r0[j]), s, acc[j]);
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[32 + j] = fmaf(__uint_as_float(r1[j]), s, acc[32 + j]);
      } else if constexpr (CW == 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = fmaf(__uint_as_float(r[j]), s, acc[j]);
      } else {
        uint32_t r[16];
        tmem_ld_32x16(taddr, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = fmaf(__uint_as_float(r[j]), s, acc[j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (ok) {
      const int tl = min(BT, row_end - t0);
      const int tiles_nt = n_tiles_x * gridDim.y;
      const int tile_id = t_tile * n_tiles_x + n_tile;
      bool owner = true;  // this CTA holds the tile's complete local sum in `acc`
      if (p.cluster_reduce) {
        // The ring is free (the last MMA has completed, so every tile that was loaded has been read): the partial
        // goes there as [token column][128 rows] fp32 and is summed after the cluster barrier below.
        owner = false;
        float* stage = reinterpret_cast<float*>(tiles);
#pragma unroll
        for (int tt = 0; tt < CW; ++tt) stage[(col0 + tt) * kTileN + row] = acc[tt];
      } else if (gridDim.z > 1) {
        owner = false;
        float* mine = p.ws + (size_t(split) * tiles_nt + tile_id) * (BT * kTileN);
#pragma unroll
        for (int tt = 0; tt < CW; ++tt) mine[(col0 + tt) * kTileN + row] = acc[tt];
        __threadfence();
        // bounded rendezvous of the four epilogue warps (a plain bar.sync could not time out)
        __syncwarp();
        if (lane == 0) mbar_arrive(&epi_bar[0]);
        bool met = mbar_wait(&epi_bar[0], 0, abort_flag, p.status, kStatusTimeoutEpilogue);
        if (met && threadIdx.x == 64) {
          const int prev = atomicAdd(p.counters + tile_id, 1);
          *last_flag = (prev == int(gridDim.z) - 1);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&epi_bar[1]);
        met = met && mbar_wait(&epi_bar[1], 0, abort_flag, p.status, kStatusTimeoutEpilogue);
        if (met && *last_flag) {
          __threadfence();
          // Sum the partials in split order (own one included, re-read from scratch) so the result does not
          // depend on which CTA happened to arrive last.  All BT loads of a split are independent.
#pragma unroll
          for (int tt = 0; tt < CW; ++tt) acc[tt] = 0.f;
          for (int z = 0; z < int(gridDim.z); ++z) {
            const float* part = p.ws + (size_t(z) * tiles_nt + tile_id) * (BT * kTileN) + row;
#pragma unroll
            for (int tt = 0; tt < CW; ++tt) acc[tt] += __ldcg(part + (col0 + tt) * kTileN);
          }
          if (threadIdx.x == 64) p.counters[tile_id] = 0;
          owner = true;
        }
      }
      __syncwarp();
      if (owner) {
        const float* xsc = gather ? p.ag.xs_full[p.ag.rank] + size_t(ag_epoch & 1u) * p.M : p.x_scale;
#pragma unroll
        for (int tt = 0; tt < CW; ++tt) {
          // gathered multipliers were written by peers during this launch: L2-coherent loads at this point
          const float xm = gather ? ((col0 + tt < tl) ? __ldcg(xsc + t0 + col0 + tt) : 0.f) : xs_w[tt];
          acc[tt] *= xm;
        }
        if (p.ar.world > 1) {
          // ----- one-shot all-reduce over NVLink peer memory, fused into the epilogue -----
          // Every rank publishes its partial tile in its own (peer-mapped) buffer, bumps the tile's flag on every
          // peer, waits until all peers bumped ours, then sums the W partials in rank order, so all ranks compute
          // bit-identical results.  Flags only ever count up (W-1 per launch), which makes the protocol safe under
          // CUDA-graph replay; the tile's launch count also selects one of two buffers, so a fast rank cannot
          // overwrite a partial that a slow rank is still reading.
          const ArParams& ar = p.ar;
          const bool rs = ar.mode == 1;
          const uint32_t before = ar.expected[tile_id];
          // AR: flags advance by W-1 per launch; RS: `expected` simply counts the launches of this tile
          const uint32_t target = before + uint32_t(ar.world - 1);
          const size_t half_off = size_t((rs ? before : before / uint32_t(ar.world - 1)) & 1u) * ar.half_elems;
          const int t_per_rank = int(gridDim.y) / ar.world;            // token tiles owned by each rank (RS)
          const int tile_owner = rs ? t_tile / t_per_rank : ar.rank;   // AR: everyone "owns" (and sums) every tile
          const int tiles_owned = t_per_rank * n_tiles_x;
          const int tile_local = (t_tile % max(t_per_rank, 1)) * n_tiles_x + n_tile;
          // AR: my partial goes to my own buffer at the slot of the tile; RS: into the owner buffer, slot [me][tile]
          const size_t off = rs ? half_off + (size_t(ar.rank) * tiles_owned + tile_local) * (BT * kTileN)
                                : half_off + size_t(tile_id) * (BT * kTileN);
          float* mine = ar.bufs[tile_owner] + off;
          if (rs) {
            // Reduce-scatter: every rank (the owner too) sends its partial tile to the slot table of the owner while
            // the other CTAs keep computing -- the transfer overlaps the math tile by tile -- and nobody waits here:
            // the owner sums the W slots of its tiles in a short trailing kernel (rs_reduce_kernel), in rank order.
            // The partial leaves through shared memory as ONE bulk copy per warp (8 KB for a 128-token tile) instead
            // of 4-byte stores, which is what NVLink needs to run near its rate.  The pipeline stages are free by
            // now: the last MMA of this tile has completed, so every TMA load was consumed.  Slot layout:
            // [epilogue warp][token column inside the chunk of that warp][32 rows].
            const int ew = warp - 2;
            float* stage = reinterpret_cast<float*>(tiles) + ew * (CW * 32);
#pragma unroll
            for (int tt = 0; tt < CW; ++tt) stage[tt * 32 + lane] = acc[tt];
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(mine + ew * (CW * 32)),
                           "r"(smem_u32(stage)), "r"(uint32_t(CW * 32 * sizeof(float)))
                           : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
              // Only the READ of the staging buffer has to finish before this CTA may exit; the NVLink writes drain
              // while the next CTA on this SM runs its main loop.  Nobody is told per tile: the kernel's completion
              // completes its copies, a cross-rank barrier follows on the stream, and only then the owner sums.
              asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            }
            __syncwarp();
            if (threadIdx.x == 64) ar.expected[tile_id] = before + 1u;  // launch count of the tile: selects the buffer half
            owner = false;
          } else {
#pragma unroll
          for (int tt = 0; tt < CW; ++tt) mine[(col0 + tt) * kTileN + row] = acc[tt];
          __threadfence_system();
          __syncwarp();
          if (lane == 0) mbar_arrive(&epi_bar[2]);
          bool met = mbar_wait(&epi_bar[2], 0, abort_flag, p.status, kStatusTimeoutEpilogue);
          if (met && threadIdx.x == 64) {
            // one system-scope fence orders the whole CTA's partial (observed through the mbarrier) before the W-1
            // flag updates, which can then be relaxed and leave back to back instead of one release round trip each
            __threadfence_system();
            for (int r = 0; r < ar.world; ++r) {
              const int peer = (ar.rank + 1 + r) % ar.world;
              if (peer != ar.rank)
                asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(ar.flags[peer] + tile_id) : "memory");
            }
            const uint32_t* my_flag = ar.flags[ar.rank] + tile_id;
            const unsigned long long t_start = globaltimer_ns();
            uint32_t seen, spins = 0;
            while (true) {
              asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(my_flag) : "memory");
              if (int32_t(seen - target) >= 0) break;
              if ((++spins & 0x3F) == 0 && (*abort_flag || globaltimer_ns() - t_start > kWaitBudgetNs)) {
                *abort_flag = 1;
                atomicCAS(p.status, 0, kStatusTimeoutPeer | (2 << 8));
                break;
              }
            }
            ar.expected[tile_id] = target;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&epi_bar[3]);
          met = met && mbar_wait(&epi_bar[3], 0, abort_flag, p.status, kStatusTimeoutEpilogue);
          owner = met && !*abort_flag;
          if (owner) {
            // Sum the W partials in rank order.  All ranks' loads of a group of 4 token columns are issued before the
            // first add, so the (remote) round trips overlap instead of running one rank after the other.
#pragma unroll
            for (int c0 = 0; c0 < CW; c0 += 4) {
              float v[8][4];
#pragma unroll
              for (int r = 0; r < 8; ++r) {
                const float* part = ar.bufs[r < ar.world ? r : ar.rank] + off + row + (col0 + c0) * kTileN;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  v[r][j] = 0.f;
                  if (r < ar.world)
                    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v[r][j]) : "l"(part + j * kTileN) : "memory");
                }
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float sum = 0.f;
#pragma unroll
                for (int r = 0; r < 8; ++r) sum += v[r][j];  // zeros beyond the world size
                acc[c0 + j] = sum;
              }
            }
          }
          }  // all-reduce
        }
        if (owner && n < p.N) {
          // The residual may be the output buffer itself (in-place add), so the compiler keeps every load behind the
          // store before it: one exposed memory round trip per token column.  All loads of the thread are issued
          // first (each element is read and written by this thread only), then the sums are stored.
          if (p.residual) {
            unsigned short res[CW];
            const unsigned short* rp = reinterpret_cast<const unsigned short*>(p.residual);
#pragma unroll
            for (int tt = 0; tt < CW; ++tt)
              res[tt] = (col0 + tt < tl) ? __ldcg(rp + size_t(t0 + col0 + tt) * p.N + n) : (unsigned short)0;
#pragma unroll
            for (int tt = 0; tt < CW; ++tt) acc[tt] += __uint_as_float(uint32_t(res[tt]) << 16);
          }
#pragma unroll
          for (int tt = 0; tt < CW; ++tt) {
            if (col0 + tt < tl) p.out[size_t(t0 + col0 + tt) * p.N + n] = __float2bfloat16(acc[tt]);
          }
        }
      }
    }
  }

  if (p.cluster_reduce) {
    // Every thread of every CTA of the cluster gets here (all waits above are bounded), so the barriers cannot hang.
    __syncwarp();
    cluster_barrier();  // all partials are in place
    if (warp >= 2 && !*abort_flag) {
      const int tl = min(BT, row_end - t0);
      switch (int(gridDim.z)) {  // the split count as a constant: all partials of a thread's columns are loaded at once
        case 2: cluster_sum_columns<BT, 2>(p, tiles, t0, tl, n0); break;
        case 3: cluster_sum_columns<BT, 3>(p, tiles, t0, tl, n0); break;
        case 4: cluster_sum_columns<BT, 4>(p, tiles, t0, tl, n0); break;
        case 5: cluster_sum_columns<BT, 5>(p, tiles, t0, tl, n0); break;
        case 6: cluster_sum_columns<BT, 6>(p, tiles, t0, tl, n0); break;
        case 7: cluster_sum_columns<BT, 7>(p, tiles, t0, tl, n0); break;
        default: cluster_sum_columns<BT, 8>(p, tiles, t0, tl, n0); break;
      }
    }
    __syncwarp();
    cluster_barrier();  // nobody's shared memory goes away while a peer still reads it
  }

  // ----- teardown: every thread arrives here, also after an aborted wait -----
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <int BT>
static int launch_gemm(const void* w, const float* w_scale, const void* x, const float* x_scale, void* out,
                       const void* residual, float* ws, size_t ws_bytes, int* counters, int counters_len, int* status,
                       int M, int N, int K, int splits, cudaStream_t stream, const ArParams* ar = nullptr,
                       int experts = 0, const int2* tile_map = nullptr, const int* expert_offsets = nullptr,
                       int map_len = 0, const AgParams* ag = nullptr) {
  using Cfg = GemmCfg<BT>;
  CUtensorMap tw, tx;
  if (experts > 0) {
    if (make_tmap_3d(&tw, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, K, N, experts, uint64_t(K), uint64_t(K) * N, kBlockK, kTileN, 1))
      return -2;
  } else if (make_tmap_2d(&tw, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, K, kTileN, kBlockK)) {
    return -2;
  }
  CUtensorMap tx_alt;
  if (ag) {  // x = this rank's gathered buffer: one map per half
    if (make_tmap_2d(&tx, ag->x_full[ag->rank], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, BT, kBlockK)) return -3;
    if (make_tmap_2d(&tx_alt, ag->x_full[ag->rank] + size_t(M) * K, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, BT, kBlockK)) return -3;
  } else {
    if (make_tmap_2d(&tx, x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, BT, kBlockK)) return -3;
    tx_alt = tx;
  }
  const int n_tiles = (N + kTileN - 1) / kTileN, t_tiles = experts > 0 ? map_len : (M + BT - 1) / BT;
  const int kb_total = K / kBlockK;
  if (splits < 1) splits = 1;
  if (splits > kb_total) splits = kb_total;
  int kb_per = (kb_total + splits - 1) / splits;
  splits = (kb_total + kb_per - 1) / kb_per;
  if (splits > 1) {
    if (size_t(splits) * n_tiles * t_tiles * BT * kTileN * sizeof(float) > ws_bytes) return -4;
    if (n_tiles * t_tiles > counters_len) return -5;
  }
  GemmParams p{w_scale, x_scale, static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(residual),
               ws, counters, status, M, N, K, kb_per, ArParams{}, tile_map, expert_offsets};
  if (ar) {
    if (size_t(n_tiles) * t_tiles * BT * kTileN > ar->half_elems) return -8;
    p.ar = *ar;
  }
  // the shared-memory opt-in is a per-device property of the function: set it once on every device that launches
  static bool attr_set[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -6;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(fp8_gemm_kernel<BT>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) !=
        cudaSuccess)
      return -6;
    attr_set[dev] = true;
  }
  if (ag) p.ag = *ag;
  const int extra_x = ag ? ag->push_ctas : 0;
  // Ring depth.  The fused-collective modes stage their output in the ring and keep all of it.  A plain or grouped
  // launch whose grid is larger than one wave of SMs takes a shallower ring instead, so that two or three CTAs share an
  // SM and one CTA's ramp-up and epilogue hide under another's main loop.
  p.stages = Cfg::kStages;
  if (!ar && !ag) {
    static const int forced = [] { const char* e = getenv("MFQ_GEMM_STAGES"); return e ? atoi(e) : 0; }();
    const long ctas = long(n_tiles) * t_tiles * splits;
    if (forced > 0) p.stages = forced < Cfg::kStages ? (forced < 2 ? 2 : forced) : Cfg::kStages;
    else if (ctas > 148 && BT <= 64) p.stages = kb_per < 4 ? (kb_per < 2 ? 2 : kb_per) : 4;
  }
  const int smem_bytes = p.stages * Cfg::kStageBytes + 1024 + 256 + Cfg::kXsBytes + Cfg::kWsBytes;
  static const bool cluster_ok = [] { const char* e = getenv("MFQ_GEMM_CLUSTER_REDUCE"); return !e || atoi(e) != 0; }();
  if (cluster_ok && !ar && !ag && !tile_map && splits > 1 && splits <= 8) {
    // A cluster is placed inside one GPC, so a grid that needs nearly every SM (144 CTAs in clusters of 3, one CTA per
    // SM) does not fit in one wave although the CTA count says it would; the driver is asked how many clusters of this
    // shape can be resident, and the ring is made shallower (more CTAs per SM) until the whole grid is.
    static int resident[64][9][Cfg::kStages + 1] = {};  // [device][cluster size][stages]: 0 = not asked yet
    const int clusters = n_tiles * t_tiles;
    const int min_stages = (BT * kTileN * 4 + Cfg::kStageBytes - 1) / Cfg::kStageBytes < 2 ? 2 : (BT * kTileN * 4 + Cfg::kStageBytes - 1) / Cfg::kStageBytes;
    auto smem_for = [](int st) { return st * Cfg::kStageBytes + 1024 + 256 + Cfg::kXsBytes + Cfg::kWsBytes; };
    auto fits = [&](int st) {
      int& known = resident[dev][splits][st];
      if (known == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(n_tiles, t_tiles, splits);
        cfg.blockDim = dim3(Cfg::kThreads);
        cfg.dynamicSmemBytes = smem_for(st);
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = splits;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        known = (cudaOccupancyMaxActiveClusters(&n, fp8_gemm_kernel<BT>, &cfg) == cudaSuccess && n > 0) ? n : -1;
        (void)cudaGetLastError();
      }
      return known >= clusters;
    };
    int st = p.stages;
    while (st > min_stages && st > 2 && !fits(st)) st = st > 4 ? 4 : st - 1;
    if (st >= min_stages) {
      p.stages = st;
      p.cluster_reduce = 1;
      launch_kernel_clustered(fp8_gemm_kernel<BT>, dim3(n_tiles, t_tiles, splits), dim3(Cfg::kThreads), dim3(1, 1, splits),
                              smem_for(st), stream, tw, tx, tx_alt, p);
      return cudaGetLastError() == cudaSuccess ? 0 : -7;
    }
  }
  launch_kernel(fp8_gemm_kernel<BT>, dim3(n_tiles + extra_x, t_tiles, splits), dim3(Cfg::kThreads), smem_bytes, stream, tw, tx, tx_alt, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

}  // namespace mfq

// C ABI.  x: [M, K] E4M3 row-major, w: [N, K] E4M3 row-major, K % 128 == 0, 16-byte aligned bases.
// token_tile in {16, 32, 64, 128}.  Returns 0 on success (launch queued), negative on a host-side error.
extern "C" int mfq_fp8_gemm(const void* w, const float* w_scale, const void* x, const float* x_scale, void* out,
                            const void* residual, float* ws, size_t ws_bytes, int* counters, int counters_len,
                            int* status, int M, int N, int K, int token_tile, int splits, cudaStream_t stream) {
  if (K % 128 != 0 || M <= 0 || N <= 0) return -1;
  switch (token_tile) {
    case 16: return mfq::launch_gemm<16>(w, w_scale, x, x_scale, out, residual, ws, ws_bytes, counters, counters_len, status, M, N, K, splits, stream);
    case 32: return mfq::launch_gemm<32>(w, w_scale, x, x_scale, out, residual, ws, ws_bytes, counters, counters_len, status, M, N, K, splits, stream);
    case 64: return mfq::launch_gemm<64>(w, w_scale, x, x_scale, out, residual, ws, ws_bytes, counters, counters_len, status, M, N, K, splits, stream);
    case 128: return mfq::launch_gemm<128>(w, w_scale, x, x_scale, out, residual, ws, ws_bytes, counters, counters_len, status, M, N, K, splits, stream);
    default: return -1;
  }
}

namespace mfq {
// Trailing kernel of the GEMM -> reduce-scatter, launched after a cross-rank barrier (every rank's GEMM kernel, and
// with it every push, has completed): one CTA per owned tile sums the W slots in rank order (bit-identical run to
// run), adds the residual and writes the bf16 rows of the output shard of this rank.
__global__ void __launch_bounds__(128)
rs_reduce_kernel(ArParams ar, __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ residual, int N, int BT,
                 int CW, int n_tiles, int t_per_rank) {
  const int tile_local = blockIdx.x, t_local = tile_local / n_tiles, n_tile = tile_local % n_tiles;
  const int tile_id = (ar.rank * t_per_rank + t_local) * n_tiles + n_tile;
  const uint32_t launches = ar.expected[tile_id];  // the GEMM kernel of this launch already counted itself
  const size_t half_off = size_t((launches - 1u) & 1u) * ar.half_elems;
  const int tiles_owned = t_per_rank * n_tiles;
  const int row = threadIdx.x, n = n_tile * kTileN + row;
  const int q = row >> 5, lane = row & 31;
  const float* base = ar.bufs[ar.rank] + half_off + size_t(tile_local) * (BT * kTileN);
  // the epilogue warp that produced (row quarter q, column half) is warp (q + 2) & 3 among the four warps of that half
  const size_t src_stride = size_t(tiles_owned) * (BT * kTileN);
  constexpr int kBatch = 4;  // columns in flight per thread: kBatch * 4 independent loads before the first add
  for (int c0 = 0; c0 < BT; c0 += kBatch) {
    float v[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) v[j] = 0.f;
#pragma unroll 1
    for (int r0 = 0; r0 < ar.world; r0 += 4) {
      float part[kBatch][4];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int c = c0 + j;
        const int ew = 4 * (c / CW) + ((q + 2) & 3);
        const float* src = base + size_t(ew) * (CW * 32) + size_t(c % CW) * 32 + lane;
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) part[j][rr] = (r0 + rr < ar.world) ? __ldcg(src + size_t(r0 + rr) * src_stride) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j)
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) v[j] += part[j][rr];  // rank order
    }
    if (n < N) {
      if (residual) {  // may be the output buffer: all loads before the first store
        float res[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; ++j) res[j] = __bfloat162float(residual[size_t(t_local * BT + c0 + j) * N + n]);
#pragma unroll
        for (int j = 0; j < kBatch; ++j) v[j] += res[j];
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) out[size_t(t_local * BT + c0 + j) * N + n] = __float2bfloat16(v[j]);
    }
  }
}
}  // namespace mfq

// Tensor-parallel row-parallel linear: the same GEMM with the cross-rank sum fused into its epilogue.  `bufs` /
// `flags` hold `world` device pointers each (own buffer at index `rank`, the others peer-mapped); every buffer has
// 2 * half_elems floats, every flag array at least ceil(N/128) * ceil(M/token_tile) counters, zero before first use.
// All ranks must issue the same sequence of calls on a context.  `residual` is added after the sum on every rank.
// reduce_scatter != 0: GEMM -> reduce-scatter over token rows (M must be a multiple of world * token_tile): `out` and
// `residual` are this rank's [M / world, N] shard; non-owners push their partial tiles and do not wait.  Two
// reduce-scatter launches on one context must be separated by something that depends on every owner's result (in the
// model: the all-gather that follows), otherwise a fast rank could overwrite partials an owner has not summed yet.
extern "C" int mfq_fp8_gemm_allreduce(const void* w, const float* w_scale, const void* x, const float* x_scale,
                                      void* out, const void* residual, float* ws, size_t ws_bytes, int* counters,
                                      int counters_len, int* status, int M, int N, int K, int token_tile, int splits,
                                      int world, int rank, void* const* bufs, void* const* flags, void* expected,
                                      size_t half_elems, int reduce_scatter, cudaStream_t stream) {
  if (K % 128 != 0 || M <= 0 || N <= 0 || world < 2 || world > 8 || rank < 0 || rank >= world) return -1;
  if (reduce_scatter && (((M + token_tile - 1) / token_tile) % world != 0 || M % token_tile != 0)) return -9;
  mfq::ArParams ar;
  ar.mode = reduce_scatter ? 1 : 0;
  ar.world = world;
  ar.rank = rank;
  for (int r = 0; r < world; ++r) {
    ar.bufs[r] = static_cast<float*>(bufs[r]);
    ar.flags[r] = static_cast<uint32_t*>(flags[r]);
  }
  ar.expected = static_cast<uint32_t*>(expected);
  ar.half_elems = half_elems;
  int rc;
  switch (token_tile) {
    case 16: rc = mfq::launch_gemm<16>(w, w_scale, x, x_scale, out, residual, ws, ws_bytes, counters, counters_len, status, M, N, K, splits, stream, &ar); break;
    case 32: rc = mfq::launch_gemm<32>(w, w_scale, x, x_scale, out, residual, ws, ws_bytes, counters, counters_len, status, M, N, K, splits, stream, &ar); break;
    case 64: rc = mfq::launch_gemm<64>(w, w_scale, x, x_scale, out, residual, ws, ws_bytes, counters, counters_len, status, M, N, K, splits, stream, &ar); break;
    case 128: rc = mfq::launch_gemm<128>(w, w_scale, x, x_scale, out, residual, ws, ws_bytes, counters, counters_len, status, M, N, K, splits, stream, &ar); break;
    default: return -1;
  }
  return rc;  // reduce-scatter: the caller runs a cross-rank barrier on the stream, then mfq_rs_reduce
}

// Second half of the GEMM -> reduce-scatter (see rs_reduce_kernel).  Same geometry arguments as the GEMM call.
extern "C" int mfq_rs_reduce(void* out, const void* residual, int M, int N, int token_tile, int world, int rank,
                             void* const* bufs, void* expected, size_t half_elems, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || world < 2 || world > 8 || M % (token_tile * world)) return -1;
  mfq::ArParams ar;
  ar.mode = 1;
  ar.world = world;
  ar.rank = rank;
  for (int r = 0; r < world; ++r) ar.bufs[r] = static_cast<float*>(bufs[r]);
  ar.expected = static_cast<uint32_t*>(expected);
  ar.half_elems = half_elems;
  const int n_tiles = (N + mfq::kTileN - 1) / mfq::kTileN, t_per_rank = (M / token_tile) / world;
  const int cw = token_tile / (token_tile >= 64 ? 2 : 1);  // token columns per epilogue warp (GemmCfg::kCols)
  mfq::rs_reduce_kernel<<<n_tiles * t_per_rank, 128, 0, stream>>>(ar, static_cast<__nv_bfloat16*>(out),
                                                                 static_cast<const __nv_bfloat16*>(residual), N, token_tile,
                                                                 cw, n_tiles, t_per_rank);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

__global__ void bump_epoch_kernel(uint32_t* epoch) { *epoch += 1; }

// All-gather -> GEMM: x_shard [M / world, K] E4M3 (+ xs_shard multipliers) is this rank's slice of the token rows; the
// kernel gathers all slices through peer memory while it multiplies (see AgParams) and writes out [M, N] bf16.
// x_full[r] / xs_full[r] / flags[r]: rank r's gathered buffers (2 * M * K bytes, 2 * M floats, `world` counters);
// epoch (1 word), push_done (`world` words): local, zero before first use.  M must be a multiple of world.
extern "C" int mfq_fp8_gemm_allgather(const void* w, const float* w_scale, const void* x_shard, const float* xs_shard,
                                      void* out, int* status, int M, int N, int K, int token_tile, int world, int rank,
                                      void* const* x_full, void* const* xs_full, void* const* flags, void* epoch,
                                      void* push_done, int push_ctas, cudaStream_t stream) {
  if (K % 128 != 0 || M <= 0 || N <= 0 || world < 2 || world > 8 || M % world != 0 || push_ctas < 1) return -1;
  if ((size_t(M / world) * K) % 16 != 0) return -1;
  mfq::AgParams ag;
  ag.world = world;
  ag.rank = rank;
  ag.push_ctas = push_ctas;
  ag.shard_rows = M / world;
  for (int r = 0; r < world; ++r) {
    ag.x_full[r] = static_cast<uint8_t*>(x_full[r]);
    ag.xs_full[r] = static_cast<float*>(xs_full[r]);
    ag.flags[r] = static_cast<uint32_t*>(flags[r]);
  }
  ag.x_shard = static_cast<const uint8_t*>(x_shard);
  ag.xs_shard = xs_shard;
  ag.epoch = static_cast<const uint32_t*>(epoch);
  ag.push_done = static_cast<uint32_t*>(push_done);
  int rc;
  switch (token_tile) {
    case 16: rc = mfq::launch_gemm<16>(w, w_scale, nullptr, nullptr, out, nullptr, nullptr, 0, nullptr, 0, status, M, N, K, 1, stream, nullptr, 0, nullptr, nullptr, 0, &ag); break;
    case 32: rc = mfq::launch_gemm<32>(w, w_scale, nullptr, nullptr, out, nullptr, nullptr, 0, nullptr, 0, status, M, N, K, 1, stream, nullptr, 0, nullptr, nullptr, 0, &ag); break;
    case 64: rc = mfq::launch_gemm<64>(w, w_scale, nullptr, nullptr, out, nullptr, nullptr, 0, nullptr, 0, status, M, N, K, 1, stream, nullptr, 0, nullptr, nullptr, 0, &ag); break;
    case 128: rc = mfq::launch_gemm<128>(w, w_scale, nullptr, nullptr, out, nullptr, nullptr, 0, nullptr, 0, status, M, N, K, 1, stream, nullptr, 0, nullptr, nullptr, 0, &ag); break;
    default: return -1;
  }
  if (rc != 0) return rc;
  bump_epoch_kernel<<<1, 1, 0, stream>>>(static_cast<uint32_t*>(epoch));
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

// Grouped GEMM over expert-sorted token rows (mixture of experts): w [E, N, K] E4M3 with w_scale [E, N/128, K/128];
// x / out rows are sorted by expert, expert e owning rows [expert_offsets[e], expert_offsets[e+1]); tile_map holds
// map_len (expert, token-tile) pairs, entries with expert < 0 are padding.  No split-K, no residual.
extern "C" int mfq_fp8_gemm_grouped(const void* w, const float* w_scale, const void* x, const float* x_scale, void* out,
                                    int* status, int rows, int N, int K, int experts, const void* tile_map,
                                    const int* expert_offsets, int map_len, int token_tile, cudaStream_t stream) {
  if (K % 128 != 0 || rows <= 0 || N <= 0 || experts <= 0 || map_len <= 0 || N % 128 != 0) return -1;
  const int2* tm = static_cast<const int2*>(tile_map);
  switch (token_tile) {
    case 16: return mfq::launch_gemm<16>(w, w_scale, x, x_scale, out, nullptr, nullptr, 0, nullptr, 0, status, rows, N, K, 1, stream, nullptr, experts, tm, expert_offsets, map_len);
    case 32: return mfq::launch_gemm<32>(w, w_scale, x, x_scale, out, nullptr, nullptr, 0, nullptr, 0, status, rows, N, K, 1, stream, nullptr, experts, tm, expert_offsets, map_len);
    case 64: return mfq::launch_gemm<64>(w, w_scale, x, x_scale, out, nullptr, nullptr, 0, nullptr, 0, status, rows, N, K, 1, stream, nullptr, experts, tm, expert_offsets, map_len);
    case 128: return mfq::launch_gemm<128>(w, w_scale, x, x_scale, out, nullptr, nullptr, 0, nullptr, 0, status, rows, N, K, 1, stream, nullptr, experts, tm, expert_offsets, map_len);
    default: return -1;
  }
}

// ---------------------------------------------------------------------------------------------------------
// Allocation-free variant (declared and documented in mfq_noalloc.h): the split-K scratch is a file-scope
// device array instead of caller memory.  Layout: [partials | counters | status word].
// ---------------------------------------------------------------------------------------------------------
#include "mfq_noalloc.h"

static __device__ __align__(256) unsigned char g_noalloc_scratch[MFQ_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
// Device address of g_noalloc_scratch per device ordinal.  In host code the array's name is only a handle for
// cudaGetSymbolAddress; the address a kernel can use has to be asked for, per device.  Filled without a lock: two
// host threads that race here both look up, and store, the same address.
unsigned char* g_noalloc_ptr[kMaxDevices] = {};

int noalloc_fail(int code, const char* why) {
  fprintf(stderr, "mfq_fp8_gemm_noalloc: %s\n", why);
  return code;
}
}  // namespace

extern "C" int mfq_fp8_gemm_noalloc(const void* w, const float* w_scale, const void* x, const float* x_scale,
                                    void* out, const void* residual, int M, int N, int K, int token_tile, int splits,
                                    cudaStream_t stream) {
  if (!w || !w_scale || !x || !x_scale || !out || M <= 0 || N <= 0 || K <= 0 || K % 128 != 0)
    return noalloc_fail(MFQ_NOALLOC_BAD_ARGUMENT, "null pointer, non-positive size or K not a multiple of 128");
  if (token_tile != 16 && token_tile != 32 && token_tile != 64 && token_tile != 128)
    return noalloc_fail(MFQ_NOALLOC_BAD_ARGUMENT, "token_tile must be 16, 32, 64 or 128");
  const int kb_total = K / 128;
  if (splits < 1) splits = 1;
  if (splits > kb_total) splits = kb_total;
  const long long tiles = (long long)((N + 127) / 128) * ((M + token_tile - 1) / token_tile);
  const long long partial_bytes = splits > 1 ? (long long)splits * tiles * token_tile * 128 * 4 : 0;
  if (tiles > MFQ_NOALLOC_MAX_TILES || partial_bytes > (long long)MFQ_NOALLOC_PARTIAL_BYTES)
    return noalloc_fail(MFQ_NOALLOC_TOO_LARGE,
                        "problem exceeds the built-in scratch (8 MiB of split-K partials, 4096 output tiles)");
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return noalloc_fail(MFQ_NOALLOC_SETUP_FAILED, "no current CUDA device");
  if (!g_noalloc_ptr[dev]) {  // set-up, once per device, with that device current
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) return noalloc_fail(MFQ_NOALLOC_SETUP_FAILED, cudaGetErrorString(e));
    g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
  }
  unsigned char* base = g_noalloc_ptr[dev];
  float* partials = reinterpret_cast<float*>(base);
  int* counters = reinterpret_cast<int*>(base + MFQ_NOALLOC_PARTIAL_BYTES);
  int* status = counters + MFQ_NOALLOC_MAX_TILES;
  // counters and status must start at zero; an earlier call that was interrupted could have left them dirty
  if (cudaMemsetAsync(counters, 0, size_t(MFQ_NOALLOC_MAX_TILES) * 4 + 256, stream) != cudaSuccess)
    return noalloc_fail(MFQ_NOALLOC_SETUP_FAILED, "could not clear the scratch counters");
  const int rc = mfq_fp8_gemm(w, w_scale, x, x_scale, out, residual, partials, MFQ_NOALLOC_PARTIAL_BYTES, counters,
                              MFQ_NOALLOC_MAX_TILES, status, M, N, K, token_tile, splits, stream);
  if (rc != 0) return noalloc_fail(rc, "launch failed");
  return MFQ_NOALLOC_OK;
}

extern "C" int mfq_fp8_gemm_noalloc_status(int* status_out, cudaStream_t stream) {
  if (!status_out) return noalloc_fail(MFQ_NOALLOC_BAD_ARGUMENT, "status_out is null");
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return noalloc_fail(MFQ_NOALLOC_SETUP_FAILED, "no current CUDA device");
  if (!g_noalloc_ptr[dev]) {  // nothing has run on this device yet
    *status_out = 0;
    return MFQ_NOALLOC_OK;
  }
  const int* status = reinterpret_cast<const int*>(g_noalloc_ptr[dev] + MFQ_NOALLOC_PARTIAL_BYTES) + MFQ_NOALLOC_MAX_TILES;
  if (cudaMemcpyAsync(status_out, status, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess)
    return noalloc_fail(MFQ_NOALLOC_SETUP_FAILED, "could not read the status word");
  return MFQ_NOALLOC_OK;
}
