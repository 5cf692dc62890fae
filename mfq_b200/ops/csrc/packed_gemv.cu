// Packed-format expert projections for decode-sized batches: NINT (1..8-bit affine codes with two-level scales) and
// MXFP4 (E2M1 + E8M0 per 32) weights stay packed in HBM and are decoded in registers on their way into the tensor core.
//
//   out[sorted row, n] = sum_k x[row, k] * W_e[n, k]        for the (expert, 16-token tile) pairs of a route plan
//
// The file format keeps a tensor's codes as bit streams ordered by row class (mfq/formats/io.py:381-408 of the
// reference); the run-time layout used here is a re-arrangement of the SAME codes (no re-quantization), made at
// load time by mfq_b200/ops/packed.py:
//
//   * rows are sorted by code width and cut into tiles of 16 rows of equal width (classes padded with empty rows),
//     so a warp never mixes widths; `out_row` maps a tile row back to its output feature (-1: padding);
//   * K is cut into units of 128 codes.  A b-bit code is split into bit planes of 4, 2 and 1 bits (b = 3 -> 2 + 1,
//     5 -> 4 + 1, 6 -> 4 + 2, 7 -> 4 + 2 + 1, 8 -> 4 + 4); a tile's unit stores its planes one after the other, each as
//     [row 16][quad thread 4][p words]: thread c of the quad that owns a row reads the p words holding its 32
//     consecutive codes (aligned to their own size, a warp's loads of a plane being contiguous).  Inside those words code 2i sits in the low
//     half-word and code 2i+1 at the same position of the high half-word, so ONE shift + ONE 3-input logic op pull a
//     pair of codes out of a plane straight into the mantissa bits of two bf16 numbers (128 + q, exact), pre-shifted
//     planes OR-ing on top; one bf16x2 subtract and one bf16x2 FMA (q * s - m) finish two weights;
//   * group parameters are one byte each (ls, lm), four groups per aligned word: with 16- and 24-wide groups a thread's
//     32 codes always fall into two neighbouring groups of ONE such word; with 32-wide groups into exactly one group.
//
// A warp owns 16 weight rows (one tile) and a slice of K; `mma.sync.m16n8k16` (bf16) takes the decoded pairs as its A
// fragment and the token rows -- read with the same slot assignment, so any k order is the right one -- as B.  The
// warps of a CTA that share a tile add their partial sums through shared memory.
//
// The reference's counterparts are its dp4a kernels over int8-quantized activations (mfq/kernels/cuda/nint_matmul.cu:
// nint_mixed_routes_kernel :2006-2106, mx_matmul.cu: mxfp4_moe_grouped_f16_kernel) behind the per-projection
// descriptor of mfe_ffn.h:9-41.
#include "common.cuh"

#include <cuda_fp16.h>
#include <type_traits>

namespace mfq {

struct PackedParams {
  // per expert (all experts of a projection share N, K, tile count and parameter strides)
  const uint32_t* codes;       // all experts' plane words
  const long long* code_base;  // [E] word offset of expert e's codes
  const int4* tile_meta;       // [E][tiles]: x = width code (1..8 NINT bits, 16 = MXFP4, 0 = unused tile), y = word offset of the
                               // tile's codes inside the expert, z = byte offset of its group parameters inside the expert, w = NINT group size
  const uint8_t* gparams;      // per tile (expert base + tile offset): NINT [16][G4][2][4] bytes (ls word, lm word per 4 groups);
                               // MXFP4 [16][units][4] E8M0 bytes
  const long long* gparam_base;  // [E] byte offset of expert e's group parameters
  const __half* anchors;       // NINT: [E][tiles*16][2] (d, dmin)
  const int* out_row;          // [E][tiles*16] output feature of a tile row (-1: padding)
  int tiles, units;            // row tiles per expert, 128-code units per row
  // activations / output
  const __nv_bfloat16* x;      // [rows][K_x] bf16
  int x_stride;                // elements between rows of x (>= units * 128 is NOT required: loads past K_x read zero)
  int K_x;                     // valid inputs per row
  __nv_bfloat16* out;          // [sorted rows][N_out]
  int N_out;
  const int2* tile_map;        // (expert, 16-row token tile) per blockIdx.y; expert < 0 pads
  const int* offsets;          // first sorted row of every expert (+ total)
  const int* src_token;        // optional: sorted row -> row of x
};

__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bf16x2_fma(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Shift right by SH (left when negative), compile-time.
template <int SH>
__device__ __forceinline__ uint32_t shift(uint32_t w) {
  if constexpr (SH > 0) return w >> SH;
  else if constexpr (SH < 0) return w << (-SH);
  else return w;
}

constexpr uint32_t kMagic = 0x43004300u;  // bf16 128.0 twice: 128 + q is exact for q < 128

// Pair I (0..15) of a thread's 32 codes, as two bf16 numbers holding 128 + q (B != 8) -- or, for B == 8, the low nibble
// in `lo` and the high nibble in `hi`.  w4 / w4b / w2 / w1: the thread's words of each plane.
template <int B, int I>
__device__ __forceinline__ uint32_t code_pair(const uint32_t (&w4)[4], const uint32_t (&w2)[2], uint32_t w1) {
  constexpr bool has4 = B >= 4, has2 = (B & 2) != 0, has1 = (B & 1) != 0;
  uint32_t q = kMagic;
  if constexpr (has4) q |= shift<4 * (I % 4)>(w4[I / 4]) & 0x000F000Fu;
  if constexpr (has2) {
    constexpr int T = has4 ? 4 : 0;  // target bit of this plane inside the code
    q |= shift<2 * (I % 8) - T>(w2[I / 8]) & (0x00030003u << T);
  }
  if constexpr (has1) {
    constexpr int T = (has4 ? 4 : 0) + (has2 ? 2 : 0);
    q |= shift<I - T>(w1) & (0x00010001u << T);
  }
  return q;
}

// Decodes the 16 pairs of one (row, unit) slice of a NINT row of width B into bf16x2 weights.  `unit_base`: first word
// of the tile's unit, `slot` = row * 4 + quad thread.  s2[g] / nm2[g]: (s, s) and (-m, -m) of the thread's two groups;
// runs u < n_first use group 0.
template <int B>
__device__ __forceinline__ void decode_nint(const uint32_t* __restrict__ unit_base, int slot, const uint32_t (&s2)[2],
                                            const uint32_t (&nm2)[2], int n_first, uint32_t (&wp)[16]) {
  constexpr int P4 = B >= 4 ? (B == 8 ? 2 : 1) : 0, P2 = ((B & 2) && B != 8) ? 1 : 0, P1 = ((B & 1) && B != 8) ? 1 : 0;
  uint32_t w4[4] = {0, 0, 0, 0}, w4b[4] = {0, 0, 0, 0}, w2[2] = {0, 0}, w1 = 0;
  const uint32_t* plane = unit_base;
  if constexpr (P4 >= 1) { const uint4 v = *reinterpret_cast<const uint4*>(plane + slot * 4); w4[0] = v.x; w4[1] = v.y; w4[2] = v.z; w4[3] = v.w; plane += 256; }
  if constexpr (P4 == 2) { const uint4 v = *reinterpret_cast<const uint4*>(plane + slot * 4); w4b[0] = v.x; w4b[1] = v.y; w4b[2] = v.z; w4b[3] = v.w; plane += 256; }
  if constexpr (P2 == 1) { const uint2 v = *reinterpret_cast<const uint2*>(plane + slot * 2); w2[0] = v.x; w2[1] = v.y; plane += 128; }
  if constexpr (P1 == 1) { w1 = plane[slot]; }
  uint32_t s16[2] = {0, 0};
  if constexpr (B == 8) {  // high nibble: q = lo + 16 hi  ->  w = lo s - m + hi (16 s)
    const uint32_t sixteen = 0x41804180u;  // bf16 16.0
    s16[0] = bf16x2_mul(s2[0], sixteen);
    s16[1] = bf16x2_mul(s2[1], sixteen);
  }
  auto one = [&](auto idx) {
    constexpr int I = decltype(idx)::value;
    const int g = (I / 4) < n_first ? 0 : 1;
    if constexpr (B == 8) {
      const uint32_t lo = bf16x2_sub((shift<4 * (I % 4)>(w4[I / 4]) & 0x000F000Fu) | kMagic, kMagic);
      const uint32_t hi = bf16x2_sub((shift<4 * (I % 4)>(w4b[I / 4]) & 0x000F000Fu) | kMagic, kMagic);
      wp[I] = bf16x2_fma(hi, s16[g], bf16x2_fma(lo, s2[g], nm2[g]));
    } else {
      const uint32_t q = bf16x2_sub(code_pair<B, I>(w4, w2, w1), kMagic);
      wp[I] = bf16x2_fma(q, s2[g], nm2[g]);
    }
  };
#define MFQ_ONE(i) one(std::integral_constant<int, i>{});
  MFQ_ONE(0) MFQ_ONE(1) MFQ_ONE(2) MFQ_ONE(3) MFQ_ONE(4) MFQ_ONE(5) MFQ_ONE(6) MFQ_ONE(7)
  MFQ_ONE(8) MFQ_ONE(9) MFQ_ONE(10) MFQ_ONE(11) MFQ_ONE(12) MFQ_ONE(13) MFQ_ONE(14) MFQ_ONE(15)
#undef MFQ_ONE
}

// MXFP4: nibble = sign(1) exponent(2) mantissa(1).  Placing the three magnitude bits at bf16 bits [8:6] and the sign
// at bit 15 gives value * 2^-126 exactly (the bf16 subnormal range continues the E2M1 one), and one multiply by the
// power of two 2^126 * 2^(e - 127) = 2^(e - 1), i.e. a bf16 with exponent field e + 126, restores the scale.
__device__ __forceinline__ uint32_t mxfp4_scale2(uint32_t e8m0) {
  const uint32_t field = min(e8m0 + 126u, 254u);  // scales of 4 and more do not occur in weights; clamped, not wrapped
  return (field << 7) | (field << 23);
}
__device__ __forceinline__ void decode_mxfp4(const uint32_t* __restrict__ unit_base, int slot, uint32_t scale2,
                                             uint32_t (&wp)[16]) {
  const uint4 v = *reinterpret_cast<const uint4*>(unit_base + slot * 4);
  const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t t = w4[i / 4] >> (4 * (i % 4));
    const uint32_t bits = ((t & 0x00070007u) << 6) | ((t & 0x00080008u) << 12);
    wp[i] = bf16x2_mul(bits, scale2);
  }
}

// Where the group parameters of a thread's n-th run of 32 codes live: the aligned 4-group word `word4`, the first group
// inside it `lg`, and how many of the run's four 8-code pieces belong to that first group (the rest to the next one).
//   32-wide groups: run n is group n.   16-wide: groups 2n, 2n + 1.   24-wide: the run starts in group floor(4n / 3).
__host__ __device__ inline int group_words(int gs, int units) {  // 4-group parameter words per row
  return gs == 32 ? units : gs == 16 ? units * 2 : (units * 4 - 1) / 3 + 1;
}
__device__ __forceinline__ void group_of_run(int gs, int n, int& word4, int& lg, int& n_first) {
  if (gs == 32) { word4 = n >> 2; lg = n & 3; n_first = 4; }
  else if (gs == 16) { word4 = n >> 1; lg = (n & 1) * 2; n_first = 2; }
  else { word4 = n / 3; lg = n % 3; n_first = 3 - lg; }
}

// Words a thread owns per unit for width code `bits` (its 32 codes of every plane).
__host__ __device__ inline int words_per_thread(int bits) { return bits == 16 ? 4 : bits; }  // unit = 64 x this many words

// KS: warps that split the K range of one tile; a CTA of 8 warps covers 8 / KS tiles.  NB: 8-token blocks (1 | 2).
template <int KS, int NB>
__global__ void __launch_bounds__(256) packed_gemv_kernel(const PackedParams p) {
  pdl_trigger();
  constexpr int kTilesPerCta = 8 / KS;
  __shared__ float part[8][16][NB * 8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g8 = lane >> 2, c = lane & 3;
  const int tile_in_cta = warp / KS, ks = warp % KS;
  const int tile = blockIdx.x * kTilesPerCta + tile_in_cta;
  pdl_wait();
  const int2 tm = p.tile_map[blockIdx.y];
  if (tm.x < 0) return;
  const int expert = tm.x;
  const int row0 = p.offsets[expert] + tm.y * (NB * 8);
  const int rows = min(NB * 8, p.offsets[expert + 1] - row0);
  const bool active = tile < p.tiles && p.tile_meta[size_t(expert) * p.tiles + tile].x != 0;

  float acc[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.f;

  if (active) {
    const int4 meta = p.tile_meta[size_t(expert) * p.tiles + tile];
    const int bits = meta.x;
    const uint32_t* tile_codes = p.codes + p.code_base[expert] + meta.y;
    const size_t unit_words = size_t(64) * words_per_thread(bits);
    const size_t trow = size_t(expert) * p.tiles * 16 + size_t(tile) * 16;  // row index into anchors / out_row
    const uint8_t* gp = p.gparams + p.gparam_base[expert] + meta.z;
    const int gs = meta.w, g4 = group_words(meta.w, p.units);
    float d[2] = {0.f, 0.f}, dm[2] = {0.f, 0.f};
    if (bits != 16) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const __half2 a = *reinterpret_cast<const __half2*>(p.anchors + (trow + g8 + 8 * h) * 2);
        d[h] = __low2float(a);
        dm[h] = __high2float(a);
      }
    }
    // token rows of this thread's B fragments
    const __nv_bfloat16* xr[NB];
    bool live[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      live[nb] = nb * 8 + g8 < rows;
      int xrow = row0 + nb * 8 + g8;
      if (p.src_token && live[nb]) xrow = p.src_token[xrow];
      xr[nb] = p.x + size_t(live[nb] ? xrow : 0) * p.x_stride;
    }
    for (int unit = ks; unit < p.units; unit += KS) {
      const int k0 = unit * 128 + c * 32;  // this thread's first input of the unit
      // ---- activations: 32 consecutive inputs of each token row (zero past the end of the row) ----
      uint32_t xb[NB][16];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 val = make_uint4(0u, 0u, 0u, 0u);
          if (live[nb] && k0 + v * 8 + 8 <= p.K_x) val = *reinterpret_cast<const uint4*>(xr[nb] + k0 + v * 8);
          xb[nb][4 * v] = val.x; xb[nb][4 * v + 1] = val.y; xb[nb][4 * v + 2] = val.z; xb[nb][4 * v + 3] = val.w;
        }
      }
      // ---- weights of rows g8 and g8 + 8 ----
      uint32_t wp[2][16];
      const uint32_t* unit_base = tile_codes + size_t(unit) * unit_words;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = h * 8 + g8, slot = row * 4 + c;
        if (bits == 16) {
          const uint32_t sc4 = *reinterpret_cast<const uint32_t*>(gp + (size_t(row) * p.units + unit) * 4);
          decode_mxfp4(unit_base, slot, mxfp4_scale2((sc4 >> (8 * c)) & 0xFFu), wp[h]);
        } else {
          // group parameters: the thread's 32 codes lie in groups g0 and g0 + 1 of one aligned 4-group word
          int word4, lg, n_first;
          group_of_run(gs, unit * 4 + c, word4, lg, n_first);
          const uint2 pw = *reinterpret_cast<const uint2*>(gp + (size_t(row) * g4 + word4) * 8);
          uint32_t s2[2], nm2[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int sh = 8 * min(lg + j, 3);
            const float s = d[h] * float((pw.x >> sh) & 0xFFu);
            const float m = dm[h] * float((pw.y >> sh) & 0xFFu);
            s2[j] = pack_bf16x2(s, s);
            nm2[j] = pack_bf16x2(-m, -m);
          }
          switch (bits) {
            case 1: decode_nint<1>(unit_base, slot, s2, nm2, n_first, wp[h]); break;
            case 2: decode_nint<2>(unit_base, slot, s2, nm2, n_first, wp[h]); break;
            case 3: decode_nint<3>(unit_base, slot, s2, nm2, n_first, wp[h]); break;
            case 4: decode_nint<4>(unit_base, slot, s2, nm2, n_first, wp[h]); break;
            case 5: decode_nint<5>(unit_base, slot, s2, nm2, n_first, wp[h]); break;
            case 6: decode_nint<6>(unit_base, slot, s2, nm2, n_first, wp[h]); break;
            case 7: decode_nint<7>(unit_base, slot, s2, nm2, n_first, wp[h]); break;
            default: decode_nint<8>(unit_base, slot, s2, nm2, n_first, wp[h]); break;
          }
        }
      }
      // ---- 8 MMAs per token block: MMA j takes pairs 2j and 2j+1 of both rows, and the same slots of the tokens ----
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
          mma_bf16(acc[nb], wp[0][2 * j], wp[1][2 * j], wp[0][2 * j + 1], wp[1][2 * j + 1], xb[nb][2 * j], xb[nb][2 * j + 1]);
      }
    }
  }
  // ---- add the K slices of a tile, write bf16 rows ----
  float (*mine)[NB * 8] = part[warp];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    mine[g8][nb * 8 + 2 * c] = acc[nb][0];
    mine[g8][nb * 8 + 2 * c + 1] = acc[nb][1];
    mine[g8 + 8][nb * 8 + 2 * c] = acc[nb][2];
    mine[g8 + 8][nb * 8 + 2 * c + 1] = acc[nb][3];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kTilesPerCta * 16 * NB * 8; i += 256) {
    const int t = i / (16 * NB * 8), j = i % (16 * NB * 8);
    const int tok = j >> 4, r = j & 15;
    const int tl = blockIdx.x * kTilesPerCta + t;
    if (tok >= rows || tl >= p.tiles) continue;
    const int n = p.out_row[(size_t(expert) * p.tiles + tl) * 16 + r];
    if (n < 0) continue;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < KS; ++w) v += part[t * KS + w][r][tok];
    p.out[size_t(row0 + tok) * p.N_out + n] = __float2bfloat16(v);
  }
}

// Dense reconstruction of one expert's matrix from the packed layout: out[n, k] bf16 (n = output feature).  One warp per
// (tile, unit); the same decode routines as the product kernel, so it doubles as their direct test.
__global__ void __launch_bounds__(256) packed_dequant_kernel(const PackedParams p, int expert, __nv_bfloat16* __restrict__ dense,
                                                             int K_out) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g8 = lane >> 2, c = lane & 3;
  const int item = blockIdx.x * 8 + warp;
  if (item >= p.tiles * p.units) return;
  const int tile = item / p.units, unit = item % p.units;
  const int4 meta = p.tile_meta[size_t(expert) * p.tiles + tile];
  const int bits = meta.x;
  if (bits == 0) return;
  const uint32_t* unit_base = p.codes + p.code_base[expert] + meta.y + size_t(unit) * 64 * words_per_thread(bits);
  const size_t trow = size_t(expert) * p.tiles * 16 + size_t(tile) * 16;
  const uint8_t* gp = p.gparams + p.gparam_base[expert] + meta.z;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t wp[16];
    const int row = h * 8 + g8, slot = row * 4 + c;
    if (bits == 16) {
      const uint32_t sc4 = *reinterpret_cast<const uint32_t*>(gp + (size_t(row) * p.units + unit) * 4);
      decode_mxfp4(unit_base, slot, mxfp4_scale2((sc4 >> (8 * c)) & 0xFFu), wp);
    } else {
      const __half2 a = *reinterpret_cast<const __half2*>(p.anchors + (trow + row) * 2);
      const float d = __low2float(a), dm = __high2float(a);
      int word4, lg, n_first;
      group_of_run(meta.w, unit * 4 + c, word4, lg, n_first);
      const uint2 pw = *reinterpret_cast<const uint2*>(gp + (size_t(row) * group_words(meta.w, p.units) + word4) * 8);
      uint32_t s2[2], nm2[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int sh = 8 * min(lg + j, 3);
        const float s = d * float((pw.x >> sh) & 0xFFu), m = dm * float((pw.y >> sh) & 0xFFu);
        s2[j] = pack_bf16x2(s, s);
        nm2[j] = pack_bf16x2(-m, -m);
      }
      switch (bits) {
        case 1: decode_nint<1>(unit_base, slot, s2, nm2, n_first, wp); break;
        case 2: decode_nint<2>(unit_base, slot, s2, nm2, n_first, wp); break;
        case 3: decode_nint<3>(unit_base, slot, s2, nm2, n_first, wp); break;
        case 4: decode_nint<4>(unit_base, slot, s2, nm2, n_first, wp); break;
        case 5: decode_nint<5>(unit_base, slot, s2, nm2, n_first, wp); break;
        case 6: decode_nint<6>(unit_base, slot, s2, nm2, n_first, wp); break;
        case 7: decode_nint<7>(unit_base, slot, s2, nm2, n_first, wp); break;
        default: decode_nint<8>(unit_base, slot, s2, nm2, n_first, wp); break;
      }
    }
    const int n = p.out_row[trow + g8 + 8 * h];
    if (n < 0) continue;
    const int k0 = unit * 128 + c * 32;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int k = k0 + 2 * i;
      if (k + 1 < K_out) *reinterpret_cast<uint32_t*>(dense + size_t(n) * K_out + k) = wp[i];
      else if (k < K_out) dense[size_t(n) * K_out + k] = __ushort_as_bfloat16(uint16_t(wp[i] & 0xFFFFu));
    }
  }
}

static PackedParams make_params(const void* codes, const void* code_base, const void* tile_meta, const void* gparams,
                                const void* gparam_base, const void* anchors, const void* out_row, int tiles, int units) {
  PackedParams p{};
  p.codes = static_cast<const uint32_t*>(codes);
  p.code_base = static_cast<const long long*>(code_base);
  p.tile_meta = static_cast<const int4*>(tile_meta);
  p.gparams = static_cast<const uint8_t*>(gparams);
  p.gparam_base = static_cast<const long long*>(gparam_base);
  p.anchors = static_cast<const __half*>(anchors);
  p.out_row = static_cast<const int*>(out_row);
  p.tiles = tiles; p.units = units;
  return p;
}

}  // namespace mfq

// Grouped product over the (expert, 16-token tile) pairs of a route plan.  x: bf16 rows (the unsorted token rows with
// src_token, else the expert-sorted rows), K_x valid inputs each (K_x % 8 == 0); out: [sorted rows, N_out] bf16.
// Packed arrays: see PackedParams and mfq_b200/ops/packed.py.  token_tile must be 16 (the plan's tile).
extern "C" int mfq_packed_gemv_grouped(const void* codes, const void* code_base, const void* tile_meta, const void* gparams,
                                       const void* gparam_base, const void* anchors, const void* out_row, int tiles, int units,
                                       const void* x, int x_stride, int K_x, void* out, int N_out, const void* tile_map,
                                       int map_cap, const int* offsets, const int* src_token, cudaStream_t stream) {
  if (tiles <= 0 || units <= 0 || K_x <= 0 || K_x % 8 || x_stride % 8 || map_cap <= 0 || N_out <= 0)
    return -1;
  mfq::PackedParams p = mfq::make_params(codes, code_base, tile_meta, gparams, gparam_base, anchors, out_row, tiles, units);
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.x_stride = x_stride;
  p.K_x = K_x;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.N_out = N_out;
  p.tile_map = static_cast<const int2*>(tile_map);
  p.offsets = offsets;
  p.src_token = src_token;
  // long rows: four warps share a tile's K range; short rows: one warp per tile
  if (units >= 12) {
    mfq::launch_kernel(mfq::packed_gemv_kernel<4, 2>, dim3((tiles + 1) / 2, map_cap), dim3(256), 0, stream, p);
  } else if (units >= 6) {
    mfq::launch_kernel(mfq::packed_gemv_kernel<2, 2>, dim3((tiles + 3) / 4, map_cap), dim3(256), 0, stream, p);
  } else {
    mfq::launch_kernel(mfq::packed_gemv_kernel<1, 2>, dim3((tiles + 7) / 8, map_cap), dim3(256), 0, stream, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

// dense[N_out, K_out] bf16 of expert `expert` (rows that no tile maps to are left untouched).
extern "C" int mfq_packed_dequant(const void* codes, const void* code_base, const void* tile_meta, const void* gparams,
                                  const void* gparam_base, const void* anchors, const void* out_row, int tiles, int units,
                                  int expert, void* dense, int K_out, cudaStream_t stream) {
  if (tiles <= 0 || units <= 0 || K_out <= 0 || K_out % 2) return -1;
  mfq::PackedParams p = mfq::make_params(codes, code_base, tile_meta, gparams, gparam_base, anchors, out_row, tiles, units);
  const int items = tiles * units;
  mfq::packed_dequant_kernel<<<(items + 7) / 8, 256, 0, stream>>>(p, expert, static_cast<__nv_bfloat16*>(dense), K_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -7;
}
