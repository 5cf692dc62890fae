// Group-quantized 4-bit weight GEMM (NINT-native and MXFP4 paths):
//   out[t, n] = sum_k x[t, k] * w[n, k],   w = s[n, g(k)] * q[n, k] - b[n, g(k)]  (NINT)   or   e2m1(q[n, k]) * 2^(e[n, g(k)] - 127)  (MXFP4)
//
// The NINT families store b-bit codes with an affine (scale, min) pair per group of `gs` consecutive inputs.  For
// code widths up to 4 bits the checkpoint is repacked once, at load, into a GPU layout (w4_repack in Python) and this
// kernel decodes it INSIDE the GEMM pipeline, so a decode step streams ~5 bits per weight from HBM instead of 8:
//
//   warp 0      loader: per 64-wide K block one bulk copy of the packed tile (128 rows x 32 B) and one TMA tile of
//               bf16 activations (BT x 64), into a ring of kStages stages
//   warp 1      issues tcgen05.mma.kind::f16 (bf16 x bf16 -> fp32 in TMEM), weights = A operand (128 rows)
//   warps 2..9  decode, two teams of four warps on alternate K blocks: thread r owns weight row r of the tile.  A 32-bit word holds 8 codes in the order
//               (c0 c2 c4 c6 | c1 c3 c5 c7) per 16-bit half, so  (w >> 4j) & 0x000F000F | 0x43004300  is the bf16 pair
//               (128 + c_2j, 128 + c_2j+1); an exact bf16x2 subtraction of 128 and ONE bf16x2 FMA with (s, s), (-b, -b) finish two weights; the
//               8 weights of a word are one 16-byte store into the 128B-swizzled A tile (ring of kAStages).  The group
//               parameters of a K block are 512-byte rows of a [tile][group][row] table and arrive with the stage
//               (one more bulk copy), so the decode never waits on global memory.  After the last block warps 2..5
//               run the epilogue (they cover the four TMEM lane quarters).
//
// One accumulator lives in TMEM for the whole K range (the affine decode is exact, nothing is folded per block);
// split-K partials are reduced by the last-arriving CTA in split order (deterministic).  Waits are bounded.
// Reference counterparts: nint_matmul_kernel / nint_matmul_tiled_prefill_kernel (mfq/kernels/cuda/nint_matmul.cu),
// which decode rows on CUDA cores (wmma for prefill) and have no tensor-memory path.
#include "common.cuh"

namespace mfq {

constexpr int kW4TileN = 128;
constexpr int kW4BlockK = 64;
constexpr int kW4PackedBytes = kW4TileN * kW4BlockK / 2;  // 4096

template <int BT>
struct W4Cfg {
  static constexpr int kStages = BT >= 128 ? 4 : 8;
  static constexpr int kAStages = 4;
  static constexpr int kXBytes = BT * kW4BlockK * 2;
  static constexpr int kGroupBytes = 2048;                        // up to 4 groups x 128 rows x 4 B per K block
  static constexpr int kXOffset = kW4PackedBytes + kGroupBytes;   // activations start 1024-aligned
  static constexpr int kStageBytes = kXOffset + kXBytes;          // packed codes + group parameters + activations
  static constexpr int kABytes = kW4TileN * kW4BlockK * 2;      // 16 KB decoded bf16 tile
  static constexpr int kTmemCols = BT < 32 ? 32 : BT;
  static constexpr int kThreads = 320;  // loader, MMA issuer, 8 decode warps
  static constexpr int kSmemBytes = kStages * kStageBytes + kAStages * kABytes + 1024 + 256;
};

struct W4Params {
  const uint8_t* packed;      // [n_tiles][k_blocks][128 rows][32 B]
  const uint32_t* group;      // [n_tiles][groups][128 rows]: bf16 scale (low half) | bf16 -b (high half)
  __nv_bfloat16* out;         // [M, N]
  const __nv_bfloat16* residual;
  float* ws;                  // split-K partials [splits][t_tiles][n_tiles][BT][128]
  int* counters;
  int* status;
  int M, N, K, groups, words_per_group, kb_per_split;
};

// KIND 0: affine codes (NINT):  w = s * c - b.   KIND 1: MXFP4:  w = e2m1(c) * 2^(e - 127), one E8M0 exponent per 32.
template <int BT, int KIND>
__global__ void __launch_bounds__(W4Cfg<BT>::kThreads, 1)
w4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const W4Params p) {
  using Cfg = W4Cfg<BT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = base;
  uint8_t* a_tiles = base + Cfg::kStages * Cfg::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(a_tiles + Cfg::kAStages * Cfg::kABytes);
  uint64_t* full = bars;                          // loader -> decode + MMA
  uint64_t* empty = full + Cfg::kStages;          // decode (4 warps) + MMA commit -> loader
  uint64_t* a_ready = empty + Cfg::kStages;       // decode (4 warps) -> MMA
  uint64_t* a_free = a_ready + Cfg::kAStages;     // MMA commit -> decode
  uint64_t* acc_done = a_free + Cfg::kAStages;    // MMA commit -> epilogue
  uint64_t* epi_bar = acc_done + 1;               // two one-shot rendezvous of the four epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(epi_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);

  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x, t_tile = blockIdx.y, split = blockIdx.z;
  const int n_tiles = gridDim.x;
  const int t0 = t_tile * BT;
  const int kb_total = p.K / kW4BlockK;
  const int kb0 = split * p.kb_per_split, kb1 = min(kb_total, kb0 + p.kb_per_split), nkb = kb1 - kb0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::kStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 5); }
    for (int i = 0; i < Cfg::kAStages; ++i) { mbar_init(&a_ready[i], 4); mbar_init(&a_free[i], 1); }
    mbar_init(acc_done, 1);
    mbar_init(&epi_bar[0], 4);
    mbar_init(&epi_bar[1], 4);
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
  const uint32_t tmem_acc = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_x);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % Cfg::kStages;
        if (!mbar_wait(&empty[s], ((i / Cfg::kStages) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutProducer)) break;
        uint8_t* st = stages + s * Cfg::kStageBytes;
        // group parameters of the block: groups g_lo..g_hi are 512-byte rows, contiguous in the [tile][group][row] table
        const int kb = kb0 + i;
        const int g_lo = (kb * 8) / p.words_per_group, g_hi = (kb * 8 + 7) / p.words_per_group;
        const uint32_t gbytes = uint32_t(g_hi - g_lo + 1) * kW4TileN * 4;
        mbar_expect_tx(&full[s], kW4PackedBytes + gbytes + Cfg::kXBytes);
        const uint8_t* src = p.packed + (size_t(n_tile) * kb_total + kb) * kW4PackedBytes;
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(smem_u32(st)), "l"(reinterpret_cast<uint64_t>(src)), "r"(uint32_t(kW4PackedBytes)),
                     "r"(smem_u32(&full[s]))
                     : "memory");
        const uint32_t* gsrc = p.group + (size_t(n_tile) * p.groups + g_lo) * kW4TileN;
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(smem_u32(st + kW4PackedBytes)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(gbytes),
                     "r"(smem_u32(&full[s]))
                     : "memory");
        tma_load_2d(st + Cfg::kXOffset, &tmap_x, &full[s], kb * kW4BlockK, t0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(128, BT, 1, 1, 0, 0);  // bf16 x bf16, both K-major
      for (int i = 0; i < nkb; ++i) {
        const int s = i % Cfg::kStages, a = i % Cfg::kAStages;
        if (!mbar_wait(&full[s], (i / Cfg::kStages) & 1, abort_flag, p.status, kStatusTimeoutMma)) break;
        if (!mbar_wait(&a_ready[a], (i / Cfg::kAStages) & 1, abort_flag, p.status, kStatusTimeoutMma)) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(a_tiles + a * Cfg::kABytes);
        const uint32_t b_addr = smem_u32(stages + s * Cfg::kStageBytes + Cfg::kXOffset);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_f16(tmem_acc, umma_desc_k_sw128(a_addr + ks * 32), umma_desc_k_sw128(b_addr + ks * 32), idesc, (i | ks) != 0);
        tc_commit(&a_free[a]);   // the decoded tile may be overwritten once these MMAs retire
        tc_commit(&empty[s]);    // ... and so may the activation tile of the stage
      }
      tc_commit(acc_done);
    }
  } else {
    // ----- decode warps, then epilogue -----
    // Two teams of four warps (thread = weight row) take alternate K blocks, so two blocks are being converted at
    // any time and the per-block latency chain (barrier wait, shared loads, convert, stores, proxy fence) overlaps.
    const int team = (warp - 2) >> 2;
    const int row = ((warp - 2) & 3) * 32 + lane;
    // group of the block's first word, kept incrementally (no integer division in the loop): word index W lies in
    // group W / words_per_group, the words of block kb are kb * 8 + {0..7}
    const int wpg = p.words_per_group;
    int r_block = ((kb0 + team) * 8) % wpg;  // offset of the block's word 0 inside its group
    bool ok = true;
    for (int i = team; i < nkb; i += 2) {
      const int s = i % Cfg::kStages, a = i % Cfg::kAStages;
      ok = mbar_wait(&full[s], (i / Cfg::kStages) & 1, abort_flag, p.status, kStatusTimeoutEpilogue) &&
           mbar_wait(&a_free[a], ((i / Cfg::kAStages) & 1) ^ 1, abort_flag, p.status, kStatusTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint8_t* st = stages + s * Cfg::kStageBytes;
      const uint4 lo = *reinterpret_cast<const uint4*>(st + row * 32), hi = *reinterpret_cast<const uint4*>(st + row * 32 + 16);
      const uint32_t* gsm = reinterpret_cast<const uint32_t*>(st + kW4PackedBytes) + row;  // [group - first group][128 rows]
      const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
      uint8_t* dst_row = a_tiles + a * Cfg::kABytes + row * 128;
      int local = 0, left = wpg - r_block;  // group index among the stage's groups; words left in that group
      uint32_t s2 = 0, b2 = 0;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        if (w == 0 || left == 0) {  // a new group starts: fetch (s, s) and (-b, -b) as bf16x2
          if (w != 0) { ++local; left = wpg; }
          const uint32_t g = gsm[local * kW4TileN];
          asm("prmt.b32 %0, %1, %1, 0x1010;" : "=r"(s2) : "r"(g));
          asm("prmt.b32 %0, %1, %1, 0x3232;" : "=r"(b2) : "r"(g));
        }
        --left;
        uint4 o;
        uint32_t* ov = reinterpret_cast<uint32_t*>(&o);
        if constexpr (KIND == 0) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t pair = ((words[w] >> (4 * j)) & 0x000F000Fu) | 0x43004300u;  // bf16 (128 + c, 128 + c')
            uint32_t qf;  // (c, c') exactly: integers below 256 are exact in bf16, so is the subtraction
            asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(qf) : "r"(pair), "r"(0x43004300u));
            asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(ov[j]) : "r"(qf), "r"(s2), "r"(b2));  // s * c - b, one rounding
          }
        } else {
          // E2M1 magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6} as bf16 = high bytes {00,3F,3F,3F,40,40,40,40}, low bytes
          // {00,00,80,C0,00,40,80,C0}: byte-permute instructions look four codes up at once (selector = code & 7)
          const uint32_t idx = words[w] & 0x77777777u;
          uint32_t hiA, hiB, loA, loB;  // A: nibbles 0..3 (even columns), B: nibbles 4..7 (odd columns)
          asm("prmt.b32 %0, %1, %2, %3;" : "=r"(hiA) : "r"(0x3F3F3F00u), "r"(0x40404040u), "r"(idx & 0xFFFFu));
          asm("prmt.b32 %0, %1, %2, %3;" : "=r"(hiB) : "r"(0x3F3F3F00u), "r"(0x40404040u), "r"(idx >> 16));
          asm("prmt.b32 %0, %1, %2, %3;" : "=r"(loA) : "r"(0xC0800000u), "r"(0xC0804000u), "r"(idx & 0xFFFFu));
          asm("prmt.b32 %0, %1, %2, %3;" : "=r"(loB) : "r"(0xC0800000u), "r"(0xC0804000u), "r"(idx >> 16));
          uint32_t a01, a23, b01, b23;  // (bf16 n0, bf16 n1), (n2, n3), (n4, n5), (n6, n7)
          asm("prmt.b32 %0, %1, %2, 0x5140;" : "=r"(a01) : "r"(loA), "r"(hiA));
          asm("prmt.b32 %0, %1, %2, 0x7362;" : "=r"(a23) : "r"(loA), "r"(hiA));
          asm("prmt.b32 %0, %1, %2, 0x5140;" : "=r"(b01) : "r"(loB), "r"(hiB));
          asm("prmt.b32 %0, %1, %2, 0x7362;" : "=r"(b23) : "r"(loB), "r"(hiB));
          uint32_t mag[4];  // word j = (column 2j, column 2j+1) = (nibble j, nibble j + 4)
          asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(mag[0]) : "r"(a01), "r"(b01));
          asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(mag[1]) : "r"(a01), "r"(b01));
          asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(mag[2]) : "r"(a23), "r"(b23));
          asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(mag[3]) : "r"(a23), "r"(b23));
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t sign = ((words[w] >> (4 * j)) & 0x00080008u) << 12;  // code bit 3 -> bf16 sign bit
            asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(ov[j]) : "r"(mag[j] | sign), "r"(s2));  // exact: s2 is a power of two
          }
        }
        *reinterpret_cast<uint4*>(dst_row + ((w ^ (row & 7)) << 4)) = o;  // 128-byte swizzle: chunk ^= row % 8
      }
      fence_proxy_async_smem();  // generic-proxy stores -> tensor-core (async proxy) reads
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&a_ready[a]);
        mbar_arrive(&empty[s]);  // this warp is done with the packed codes of the stage
      }
      r_block = (r_block + 16) % wpg;  // my next block is two blocks (sixteen words) further
    }
    if (warp >= 6) ok = false;  // the epilogue is run by warps 2..5 (one per TMEM lane quarter)
    // ----- epilogue: TMEM -> registers -> (split-K reduce) -> bf16 -----
    if (ok) ok = mbar_wait(acc_done, 0, abort_flag, p.status, kStatusTimeoutEpilogue);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      const int q = warp & 3;                 // TMEM lane quarter this warp may read
      const int erow = q * 32 + lane;         // output feature inside the tile
      const int n = n_tile * kW4TileN + erow;
      float acc[BT];
      if (nkb > 0) {
#pragma unroll
        for (int c = 0; c < BT; c += 16) {
          uint32_t r[16];
          tmem_ld_32x16(tmem_acc + (uint32_t(q * 32) << 16) + c, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c + j] = __uint_as_float(r[j]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < BT; ++c) acc[c] = 0.f;
      }
      tc_fence_before();
      const int tl = min(BT, p.M - t0);
      const int tile_id = t_tile * n_tiles + n_tile;
      bool owner = true;
      if (gridDim.z > 1) {
        owner = false;
        const int tiles_nt = n_tiles * gridDim.y;
        float* mine = p.ws + (size_t(split) * tiles_nt + tile_id) * (BT * kW4TileN);
#pragma unroll
        for (int c = 0; c < BT; ++c) mine[c * kW4TileN + erow] = acc[c];
        __threadfence();
        __syncwarp();
        if (lane == 0) mbar_arrive(&epi_bar[0]);
        bool met = mbar_wait(&epi_bar[0], 0, abort_flag, p.status, kStatusTimeoutEpilogue);
        if (met && threadIdx.x == 64) *last_flag = (atomicAdd(p.counters + tile_id, 1) == int(gridDim.z) - 1);
        __syncwarp();
        if (lane == 0) mbar_arrive(&epi_bar[1]);
        met = met && mbar_wait(&epi_bar[1], 0, abort_flag, p.status, kStatusTimeoutEpilogue);
        if (met && *last_flag) {
          __threadfence();
#pragma unroll
          for (int c = 0; c < BT; ++c) acc[c] = 0.f;
          for (int z = 0; z < int(gridDim.z); ++z) {  // split order: the result does not depend on arrival order
            const float* part = p.ws + (size_t(z) * tiles_nt + tile_id) * (BT * kW4TileN) + erow;
#pragma unroll
            for (int c = 0; c < BT; ++c) acc[c] += __ldcg(part + c * kW4TileN);
          }
          if (threadIdx.x == 64) p.counters[tile_id] = 0;
          owner = true;
        }
      }
      if (owner && n < p.N) {
        // residual and output may be one buffer: all loads first, or every load would wait behind the store before it
        if (p.residual) {
          unsigned short res[BT];
          const unsigned short* rp = reinterpret_cast<const unsigned short*>(p.residual);
#pragma unroll
          for (int c = 0; c < BT; ++c) res[c] = (c < tl) ? __ldcg(rp + size_t(t0 + c) * p.N + n) : (unsigned short)0;
#pragma unroll
          for (int c = 0; c < BT; ++c) acc[c] += __uint_as_float(uint32_t(res[c]) << 16);
        }
#pragma unroll
        for (int c = 0; c < BT; ++c) {
          if (c < tl) p.out[size_t(t0 + c) * p.N + n] = __float2bfloat16(acc[c]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_acc, Cfg::kTmemCols);
}

template <int BT, int KIND>
static int launch_w4(const W4Params& p0, const void* x, int splits, size_t ws_bytes, int counters_len, cudaStream_t stream) {
  using Cfg = W4Cfg<BT>;
  W4Params p = p0;
  CUtensorMap tx;
  if (make_tmap_2d(&tx, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.M, p.K, uint64_t(p.K) * 2, BT, kW4BlockK)) return -3;
  const int n_tiles = (p.N + kW4TileN - 1) / kW4TileN, t_tiles = (p.M + BT - 1) / BT, kb_total = p.K / kW4BlockK;
  splits = max(1, min(splits, kb_total));
  const int kb_per = (kb_total + splits - 1) / splits;
  splits = (kb_total + kb_per - 1) / kb_per;
  p.kb_per_split = kb_per;
  if (splits > 1) {
    if (size_t(splits) * n_tiles * t_tiles * BT * kW4TileN * sizeof(float) > ws_bytes) return -4;
    if (n_tiles * t_tiles > counters_len) return -5;
  }
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(w4_gemm_kernel<BT, KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
      return -6;
    attr_set = true;
  }
  launch_kernel(w4_gemm_kernel<BT, KIND>, dim3(n_tiles, t_tiles, splits), dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, tx, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

}  // namespace mfq

// x [M, K] bf16 row-major; packed / group in the layouts of W4Params (see w4_repack on the Python side);
// group_size >= 16 and a multiple of 8 (16, 24, 32, 64 ...: at most four groups meet a 64-wide K block), K a multiple of 64 and of group_size; out [M, N] bf16.
extern "C" int mfq_w4_gemm(const void* packed, const void* group, const void* x, void* out, const void* residual, float* ws,
                           size_t ws_bytes, int* counters, int counters_len, int* status, int M, int N, int K, int group_size,
                           int token_tile, int splits, int kind, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K % 64 || group_size < 16 || group_size % 8 || K % group_size) return -1;
  if (kind != 0 && (kind != 1 || group_size != 32)) return -1;  // MXFP4 blocks are 32 wide
  mfq::W4Params p{static_cast<const uint8_t*>(packed), static_cast<const uint32_t*>(group), static_cast<__nv_bfloat16*>(out),
                  static_cast<const __nv_bfloat16*>(residual), ws, counters, status, M, N, K, K / group_size, group_size / 8, 0};
#define MFQ_W4(BT) (kind == 0 ? mfq::launch_w4<BT, 0>(p, x, splits, ws_bytes, counters_len, stream) \
                              : mfq::launch_w4<BT, 1>(p, x, splits, ws_bytes, counters_len, stream))
  switch (token_tile) {
    case 16: return MFQ_W4(16);
    case 32: return MFQ_W4(32);
    case 64: return MFQ_W4(64);
    case 128: return MFQ_W4(128);
    default: return -1;
  }
#undef MFQ_W4
}
