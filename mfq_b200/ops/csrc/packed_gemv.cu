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
//     planes OR-ing on top; one bf16x2 subtract and one bf16x2 FMA ((q - z) * s - (m - z s)) finish two weights;
//   * group parameters are one byte each (ls, lm), four groups per aligned word: with 16- and 24-wide groups a thread's
//     32 codes always fall into two neighbouring groups of ONE such word; with 32-wide groups into exactly one group.
//     Every int -> float and float -> bf16 step of the parameter arithmetic is done with integer / FMA-pipe instructions
//     (magic-number conversions): the conversion unit runs at a quarter of the rate and bounded an earlier version;
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

// Small unsigned integer (< 2^23) -> float without the conversion unit: the integer lands in the mantissa of 2^23.
__device__ __forceinline__ float u2f(uint32_t v) { return __uint_as_float(0x4B000000u | v) - 8388608.f; }
// float -> bf16 (round half up on the dropped bits) replicated into both halves, integer pipe only.
__device__ __forceinline__ uint32_t bf16_twice(float f) {
  const uint32_t u = __float_as_uint(f) + 0x8000u;
  return __byte_perm(u, u, 0x3232);
}

// A group's affine terms.  w = q s - m is evaluated as (q - z) s - (m - z s) with the integer zero point z = round(m / s):
// z is subtracted exactly together with the 128 of the bf16 trick, so the constant that is left is at most half a code
// step and its bf16 rounding (like that of s, now multiplied by |q - z| instead of q) stays far below the step.  Any
// integer z gives the same weight in exact arithmetic, so the approximate reciprocal only costs precision at ties.
__device__ __forceinline__ void group_terms(float d, float dm, uint32_t ls, uint32_t lm, uint32_t& s2, uint32_t& nm2,
                                            uint32_t& kz2) {
  const float s = d * u2f(ls), m = dm * u2f(lm);
  float zf = s > 0.f ? __fdividef(m, s) : 0.f;
  zf = fminf(fmaxf(zf, 0.f), 127.f) + 12582912.f;  // 1.5 * 2^23: the add rounds to an integer in the low mantissa bits
  const uint32_t z = __float_as_uint(zf) & 0x7Fu;
  s2 = bf16_twice(s);
  nm2 = bf16_twice(fmaf(zf - 12582912.f, s, -m));
  kz2 = (0x4300u | z) * 0x10001u;  // bf16 128 + z, twice
}

// A thread's raw share of one unit: the plane words of its two rows (rows g8 and g8 + 8 of the tile) and their group
// parameter words.  Loading is separate from decoding so that the next unit's loads are in flight while this one is
// decoded and multiplied.  B: 1..8 = NINT code width, 16 = MXFP4.
template <int B>
struct RawUnit {
  static constexpr int kWords = B == 16 ? 4 : B;
  uint32_t w[2][kWords];
  uint2 pw[2];  // NINT: (ls word, lm word) of the 4-group block; MXFP4: x = the unit's four E8M0 bytes
};

template <int B>
__device__ __forceinline__ void load_unit(RawUnit<B>& r, const uint32_t* __restrict__ unit_base, const uint8_t* __restrict__ gp,
                                          int g8, int c, int unit, int units, int gs, int g4) {
  constexpr int P4 = B == 16 ? 1 : (B >= 4 ? (B == 8 ? 2 : 1) : 0);
  constexpr int P2 = (B != 16 && B != 8 && (B & 2)) ? 1 : 0, P1 = (B != 16 && B != 8 && (B & 1)) ? 1 : 0;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = h * 8 + g8, slot = row * 4 + c;
    const uint32_t* plane = unit_base;
    int o = 0;
    if constexpr (P4 >= 1) { const uint4 v = *reinterpret_cast<const uint4*>(plane + slot * 4); r.w[h][0] = v.x; r.w[h][1] = v.y; r.w[h][2] = v.z; r.w[h][3] = v.w; plane += 256; o = 4; }
    if constexpr (P4 == 2) { const uint4 v = *reinterpret_cast<const uint4*>(plane + slot * 4); r.w[h][4] = v.x; r.w[h][5] = v.y; r.w[h][6] = v.z; r.w[h][7] = v.w; plane += 256; o = 8; }
    if constexpr (P2 == 1) { const uint2 v = *reinterpret_cast<const uint2*>(plane + slot * 2); r.w[h][o] = v.x; r.w[h][o + 1] = v.y; plane += 128; o += 2; }
    if constexpr (P1 == 1) { r.w[h][o] = plane[slot]; }
    if constexpr (B == 16) {
      r.pw[h] = make_uint2(*reinterpret_cast<const uint32_t*>(gp + (size_t(row) * units + unit) * 4), 0u);
    } else {
      int word4, lg, n_first;
      group_of_run(gs, unit * 4 + c, word4, lg, n_first);
      r.pw[h] = *reinterpret_cast<const uint2*>(gp + (size_t(row) * g4 + word4) * 8);
    }
  }
}

// Decodes the 16 pairs of one row's share of a unit into bf16x2 weights.  Per 8-code piece u (4 pairs) of the run:
// s2[u] = (s, s), kz2[u] = (128 + z, 128 + z), nm2[u] = (z s - m, z s - m) of the piece's group -- see group_terms().
template <int B>
__device__ __forceinline__ void decode_nint(const uint32_t (&w)[B], const uint32_t (&s2)[4], const uint32_t (&nm2)[4],
                                            const uint32_t (&kz2)[4], uint32_t (&wp)[16]) {
  constexpr int P4 = B >= 4 ? (B == 8 ? 2 : 1) : 0, P2 = ((B & 2) && B != 8) ? 1 : 0, P1 = ((B & 1) && B != 8) ? 1 : 0;
  uint32_t w4[4] = {0, 0, 0, 0}, w4b[4] = {0, 0, 0, 0}, w2[2] = {0, 0}, w1 = 0;
  int o = 0;
  if constexpr (P4 >= 1) { w4[0] = w[0]; w4[1] = w[1]; w4[2] = w[2]; w4[3] = w[3]; o = 4; }
  if constexpr (P4 == 2) { w4b[0] = w[4]; w4b[1] = w[5]; w4b[2] = w[6]; w4b[3] = w[7]; o = 8; }
  if constexpr (P2 == 1) { w2[0] = w[o]; w2[1] = w[o + 1]; o += 2; }
  if constexpr (P1 == 1) { w1 = w[o]; }
  auto one = [&](auto idx) {
    constexpr int I = decltype(idx)::value;
    constexpr int u = I / 4;
    if constexpr (B == 8) {  // high nibble: q = lo + 16 hi  ->  w = (lo - z) s - rest + hi (16 s)
      const uint32_t lo = bf16x2_sub((shift<4 * (I % 4)>(w4[I / 4]) & 0x000F000Fu) | kMagic, kz2[u]);
      const uint32_t hi = bf16x2_sub((shift<4 * (I % 4)>(w4b[I / 4]) & 0x000F000Fu) | kMagic, kMagic);
      wp[I] = bf16x2_fma(hi, bf16x2_mul(s2[u], 0x41804180u /* 16.0 */), bf16x2_fma(lo, s2[u], nm2[u]));
    } else {
      const uint32_t q = bf16x2_sub(code_pair<B, I>(w4, w2, w1), kz2[u]);
      wp[I] = bf16x2_fma(q, s2[u], nm2[u]);
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
__device__ __forceinline__ void decode_mxfp4(const uint32_t (&w4)[4], uint32_t scale2, uint32_t (&wp)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t t = w4[i / 4] >> (4 * (i % 4));
    const uint32_t bits = ((t & 0x00070007u) << 6) | ((t & 0x00080008u) << 12);
    wp[i] = bf16x2_mul(bits, scale2);
  }
}

// Both rows of a raw unit -> bf16x2 weight pairs.
template <int B>
__device__ __forceinline__ void decode_unit(const RawUnit<B>& r, const float (&d)[2], const float (&dm)[2], int gs, int unit,
                                            int c, uint32_t (&wp)[2][16]) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if constexpr (B == 16) {
      decode_mxfp4(r.w[h], mxfp4_scale2((r.pw[h].x >> (8 * c)) & 0xFFu), wp[h]);
    } else {
      uint32_t s2[4], nm2[4], kz2[4];
      if (gs == 32) {  // the run is one group: no per-piece selection at all
        const int sh = 8 * ((unit * 4 + c) & 3);
        group_terms(d[h], dm[h], (r.pw[h].x >> sh) & 0xFFu, (r.pw[h].y >> sh) & 0xFFu, s2[0], nm2[0], kz2[0]);
#pragma unroll
        for (int u = 1; u < 4; ++u) { s2[u] = s2[0]; nm2[u] = nm2[0]; kz2[u] = kz2[0]; }
      } else {  // the run crosses from group lg into lg + 1 after n_first of its four 8-code pieces
        int word4, lg, n_first;
        group_of_run(gs, unit * 4 + c, word4, lg, n_first);
        uint32_t sa, ma, za, sb, mb, zb;
        group_terms(d[h], dm[h], (r.pw[h].x >> (8 * lg)) & 0xFFu, (r.pw[h].y >> (8 * lg)) & 0xFFu, sa, ma, za);
        group_terms(d[h], dm[h], (r.pw[h].x >> (8 * lg + 8)) & 0xFFu, (r.pw[h].y >> (8 * lg + 8)) & 0xFFu, sb, mb, zb);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const bool first = u < n_first;
          s2[u] = first ? sa : sb; nm2[u] = first ? ma : mb; kz2[u] = first ? za : zb;
        }
      }
      decode_nint<B>(r.w[h], s2, nm2, kz2, wp[h]);
    }
  }
}

// Words a thread owns per unit for width code `bits` (its 32 codes of every plane).
__host__ __device__ inline int words_per_thread(int bits) { return bits == 16 ? 4 : bits; }  // unit = 64 x this many words

// The K slice of one warp over one tile: units ks, ks + KS, ...  The next unit's raw words are requested before this
// unit is decoded and multiplied, the activations right after (they are cache-resident): two units of weights in flight.
template <int B, int KS, int NB, bool kPrefetch>
__device__ __forceinline__ void tile_product(const PackedParams& p, const uint32_t* __restrict__ tile_codes,
                                             const uint8_t* __restrict__ gp, int gs, const float (&d)[2], const float (&dm)[2],
                                             const __nv_bfloat16* const (&xr)[NB], const bool (&live)[NB], int ks, int g8, int c,
                                             float (&acc)[NB][4]) {
  constexpr size_t unit_words = size_t(64) * (B == 16 ? 4 : B);
  const int g4 = group_words(gs, p.units);
  RawUnit<B> cur;
  if (kPrefetch && ks < p.units) load_unit<B>(cur, tile_codes + size_t(ks) * unit_words, gp, g8, c, ks, p.units, gs, g4);
  for (int unit = ks; unit < p.units; unit += KS) {
    RawUnit<B> nxt;
    if constexpr (kPrefetch) {
      nxt = cur;
      if (unit + KS < p.units) load_unit<B>(nxt, tile_codes + size_t(unit + KS) * unit_words, gp, g8, c, unit + KS, p.units, gs, g4);
    } else {
      load_unit<B>(cur, tile_codes + size_t(unit) * unit_words, gp, g8, c, unit, p.units, gs, g4);
    }
    const int k0 = unit * 128 + c * 32;  // this thread's first input of the unit
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
    uint32_t wp[2][16];
    decode_unit<B>(cur, d, dm, gs, unit, c, wp);
    // 8 MMAs per token block: MMA j takes pairs 2j and 2j+1 of both rows, and the same slots of the tokens
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
        mma_bf16(acc[nb], wp[0][2 * j], wp[1][2 * j], wp[0][2 * j + 1], wp[1][2 * j + 1], xb[nb][2 * j], xb[nb][2 * j + 1]);
    }
    if constexpr (kPrefetch) cur = nxt;
  }
}

// KS: warps that split the K range of one tile; a CTA of 8 warps covers 8 / KS tiles.  NB: 8-token blocks (1 | 2).
// PF: request the next unit's words before decoding this one (two units of weights in flight per warp).
template <int KS, int NB, bool PF>
__global__ void __launch_bounds__(256, 2) packed_gemv_kernel(const PackedParams p) {
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
  const int row0 = p.offsets[expert] + tm.y * 16;  // the route plan's token tile is 16 rows
  const int rows = min(NB * 8, p.offsets[expert + 1] - row0);
  int4 meta = make_int4(0, 0, 0, 0);
  if (tile < p.tiles) meta = p.tile_meta[size_t(expert) * p.tiles + tile];
  const int bits = meta.x;

  float acc[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.f;

  if (bits != 0) {
    const uint32_t* tile_codes = p.codes + p.code_base[expert] + meta.y;
    const size_t trow = size_t(expert) * p.tiles * 16 + size_t(tile) * 16;  // row index into anchors / out_row
    const uint8_t* gp = p.gparams + p.gparam_base[expert] + meta.z;
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
    switch (bits) {  // uniform over the warp: a tile holds rows of one width
      case 1: tile_product<1, KS, NB, PF>(p, tile_codes, gp, meta.w, d, dm, xr, live, ks, g8, c, acc); break;
      case 2: tile_product<2, KS, NB, PF>(p, tile_codes, gp, meta.w, d, dm, xr, live, ks, g8, c, acc); break;
      case 3: tile_product<3, KS, NB, PF>(p, tile_codes, gp, meta.w, d, dm, xr, live, ks, g8, c, acc); break;
      case 4: tile_product<4, KS, NB, PF>(p, tile_codes, gp, meta.w, d, dm, xr, live, ks, g8, c, acc); break;
      case 5: tile_product<5, KS, NB, PF>(p, tile_codes, gp, meta.w, d, dm, xr, live, ks, g8, c, acc); break;
      case 6: tile_product<6, KS, NB, PF>(p, tile_codes, gp, meta.w, d, dm, xr, live, ks, g8, c, acc); break;
      case 7: tile_product<7, KS, NB, PF>(p, tile_codes, gp, meta.w, d, dm, xr, live, ks, g8, c, acc); break;
      case 8: tile_product<8, KS, NB, PF>(p, tile_codes, gp, meta.w, d, dm, xr, live, ks, g8, c, acc); break;
      default: tile_product<16, KS, NB, PF>(p, tile_codes, gp, meta.w, d, dm, xr, live, ks, g8, c, acc); break;
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
// (tile, unit); the same load / decode routines as the product kernel, so it doubles as their direct test.
template <int B>
__device__ __forceinline__ void dequant_unit(const PackedParams& p, const int4& meta, size_t trow, int expert, int unit, int g8,
                                             int c, __nv_bfloat16* __restrict__ dense, int K_out) {
  const uint32_t* unit_base = p.codes + p.code_base[expert] + meta.y + size_t(unit) * 64 * (B == 16 ? 4 : B);
  const uint8_t* gp = p.gparams + p.gparam_base[expert] + meta.z;
  float d[2] = {0.f, 0.f}, dm[2] = {0.f, 0.f};
  if constexpr (B != 16) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const __half2 a = *reinterpret_cast<const __half2*>(p.anchors + (trow + g8 + 8 * h) * 2);
      d[h] = __low2float(a);
      dm[h] = __high2float(a);
    }
  }
  RawUnit<B> raw;
  load_unit<B>(raw, unit_base, gp, g8, c, unit, p.units, meta.w, group_words(meta.w, p.units));
  uint32_t wp[2][16];
  decode_unit<B>(raw, d, dm, meta.w, unit, c, wp);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int n = p.out_row[trow + g8 + 8 * h];
    if (n < 0) continue;
    const int k0 = unit * 128 + c * 32;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int k = k0 + 2 * i;
      if (k + 1 < K_out) *reinterpret_cast<uint32_t*>(dense + size_t(n) * K_out + k) = wp[h][i];
      else if (k < K_out) dense[size_t(n) * K_out + k] = __ushort_as_bfloat16(uint16_t(wp[h][i] & 0xFFFFu));
    }
  }
}

__global__ void __launch_bounds__(256) packed_dequant_kernel(const PackedParams p, int expert, __nv_bfloat16* __restrict__ dense,
                                                             int K_out) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g8 = lane >> 2, c = lane & 3;
  const int item = blockIdx.x * 8 + warp;
  if (item >= p.tiles * p.units) return;
  const int tile = item / p.units, unit = item % p.units;
  const int4 meta = p.tile_meta[size_t(expert) * p.tiles + tile];
  const size_t trow = size_t(expert) * p.tiles * 16 + size_t(tile) * 16;
  switch (meta.x) {
    case 0: break;
    case 1: dequant_unit<1>(p, meta, trow, expert, unit, g8, c, dense, K_out); break;
    case 2: dequant_unit<2>(p, meta, trow, expert, unit, g8, c, dense, K_out); break;
    case 3: dequant_unit<3>(p, meta, trow, expert, unit, g8, c, dense, K_out); break;
    case 4: dequant_unit<4>(p, meta, trow, expert, unit, g8, c, dense, K_out); break;
    case 5: dequant_unit<5>(p, meta, trow, expert, unit, g8, c, dense, K_out); break;
    case 6: dequant_unit<6>(p, meta, trow, expert, unit, g8, c, dense, K_out); break;
    case 7: dequant_unit<7>(p, meta, trow, expert, unit, g8, c, dense, K_out); break;
    case 8: dequant_unit<8>(p, meta, trow, expert, unit, g8, c, dense, K_out); break;
    default: dequant_unit<16>(p, meta, trow, expert, unit, g8, c, dense, K_out); break;
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
// Packed arrays: see PackedParams and mfq_b200/ops/packed.py.  The plan's token tile must be 16.  max_rows_per_expert: an
// upper bound on the rows any expert receives (0: unknown).
extern "C" int mfq_packed_gemv_grouped(const void* codes, const void* code_base, const void* tile_meta, const void* gparams,
                                       const void* gparam_base, const void* anchors, const void* out_row, int tiles, int units,
                                       const void* x, int x_stride, int K_x, void* out, int N_out, const void* tile_map,
                                       int map_cap, const int* offsets, const int* src_token, int max_rows_per_expert,
                                       cudaStream_t stream) {
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
  // Few tokens (no expert sees more than 8 rows): the step is latency-bound, so up to four warps split a tile's K range
  // and every warp keeps two units in flight.  More tokens: thousands of CTAs exist anyway, a warp then walks a whole
  // row range by itself (its start-up latencies -- tile map, offsets, descriptors -- are paid once per 16 units).
  const bool narrow = max_rows_per_expert > 0 && max_rows_per_expert <= 8;
  static const int force_ks = [] { const char* e = getenv("MFQ_PACKED_KS"); return e ? atoi(e) : 0; }();
  static const int force_pf = [] { const char* e = getenv("MFQ_PACKED_PF"); return e ? atoi(e) : -1; }();
  int ks = narrow ? (units >= 12 ? 4 : units >= 6 ? 2 : 1) : 1;
  if (force_ks == 1 || force_ks == 2 || force_ks == 4) ks = force_ks;
  const bool pf = force_pf >= 0 ? force_pf != 0 : true;
  const dim3 grid((tiles + 8 / ks - 1) / (8 / ks), map_cap);
#define MFQ_LAUNCH(KS_, NB_, PF_) mfq::launch_kernel(mfq::packed_gemv_kernel<KS_, NB_, PF_>, grid, dim3(256), 0, stream, p)
#define MFQ_PICK(KS_) \
  do { \
    if (narrow) { if (pf) MFQ_LAUNCH(KS_, 1, true); else MFQ_LAUNCH(KS_, 1, false); } \
    else { if (pf) MFQ_LAUNCH(KS_, 2, true); else MFQ_LAUNCH(KS_, 2, false); } \
  } while (0)
  if (ks == 4) MFQ_PICK(4);
  else if (ks == 2) MFQ_PICK(2);
  else MFQ_PICK(1);
#undef MFQ_PICK
#undef MFQ_LAUNCH
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
