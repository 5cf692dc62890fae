// CPU decoders of packed weight rows: the numerical oracle of the GPU paths and the source of embedding rows and
// host-resident experts.
//
// NINT v2 payload:  u8 bits|0x80, u8 sub_bits, i32 groupsize, i32 axis, i32 neuron_len, u32 ndim, ndim x i64 shape,
// u32 rows, u32 groups, rows x f16 d, rows x f16 dmin, then LSB-first bitstreams, each starting on a byte boundary:
// 2-bit group-code width selector per row; for each selector class (ascending) the group scales then the group mins
// of its rows; 3-bit q width selector per row; for each q class the q codes of its rows.
//   w[r, g, i] = d[r] * ls[r, g] * q[r, g, i] - dmin[r] * lm[r, g]
// Reference counterparts: cpp_runtime/core/src/nint_rows.cpp, backends/cpu/ops/packed_nint*.cpp.
#include "common.h"
#include "mfq_core.h"

#include <cmath>
#include <cstring>
#include <vector>

namespace {
using mfqn::fail;

inline float half_to_float(uint16_t h) {
  const uint32_t sign = uint32_t(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {  // subnormal: normalise
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400u));
      bits = sign | uint32_t(127 - 15 - e) << 23 | (man & 0x3FFu) << 13;
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | man << 13;
  } else {
    bits = sign | (exp + 112) << 23 | man << 13;
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

// value `index` of an LSB-first stream of `width`-bit codes (width <= 16)
inline uint32_t read_bits(const uint8_t* base, int64_t index, int width) {
  const int64_t bit = index * width;
  const uint8_t* p = base + (bit >> 3);
  uint32_t v = uint32_t(p[0]) | uint32_t(p[1]) << 8 | uint32_t(p[2]) << 16;  // callers keep 2 bytes of slack
  return (v >> (bit & 7)) & ((1u << width) - 1u);
}

inline int64_t packed_nbytes(int64_t count, int bits) { return (count * bits + 7) / 8; }

struct Nint {
  const uint8_t* blob = nullptr;
  int64_t nbytes = 0;
  int bits = 0, sub_bits = 0, gs = 0, axis = 0;
  int64_t neuron_len = 0, rows = 0, groups = 0;
  const uint8_t* d = nullptr;
  const uint8_t* dm = nullptr;
  std::vector<uint8_t> k_class, q_class;
  std::vector<uint32_t> k_rank, q_rank;
  const uint8_t* ls_base[4] = {};
  const uint8_t* lm_base[4] = {};
  const uint8_t* q_base[8] = {};
  std::vector<uint8_t> tail;  // copy of the last bytes + slack, so read_bits never reads past the payload
};
}  // namespace

extern "C" {

void* mfq_nint_open(const void* blob_, int64_t nbytes) {
  const uint8_t* blob = static_cast<const uint8_t*>(blob_);
  if (nbytes < 14 + 4) { fail(-1, "NINT payload too short"); return nullptr; }
  auto n = new Nint();
  n->blob = blob;
  n->nbytes = nbytes;
  if (!(blob[0] & 0x80)) { fail(-1, "only NINT v2 payloads are indexed here"); delete n; return nullptr; }
  n->bits = blob[0] & 0x7F;
  n->sub_bits = blob[1];
  int32_t gs, axis, nl;
  memcpy(&gs, blob + 2, 4);
  memcpy(&axis, blob + 6, 4);
  memcpy(&nl, blob + 10, 4);
  n->gs = gs; n->axis = axis; n->neuron_len = nl;
  int64_t off = 14;
  uint32_t ndim;
  memcpy(&ndim, blob + off, 4);
  off += 4 + 8 * int64_t(ndim);
  if (off + 8 > nbytes || gs <= 0) { fail(-1, "NINT header runs past the payload"); delete n; return nullptr; }
  uint32_t rows, groups;
  memcpy(&rows, blob + off, 4);
  memcpy(&groups, blob + off + 4, 4);
  off += 8;
  n->rows = rows; n->groups = groups;
  n->d = blob + off; off += 2 * int64_t(rows);
  n->dm = blob + off; off += 2 * int64_t(rows);
  auto need = [&](int64_t more) { return off + more <= nbytes; };
  // group-code width classes
  const int64_t ksel_bytes = packed_nbytes(rows, 2);
  if (!need(ksel_bytes)) { fail(-1, "truncated NINT payload"); delete n; return nullptr; }
  n->k_class.resize(rows); n->k_rank.resize(rows);
  uint32_t kcount[4] = {};
  {
    std::vector<uint8_t> tmp(blob + off, blob + off + ksel_bytes);
    tmp.resize(tmp.size() + 4);
    for (int64_t r = 0; r < rows; ++r) {
      const uint32_t c = read_bits(tmp.data(), r, 2);
      n->k_class[r] = uint8_t(c);
      n->k_rank[r] = kcount[c]++;
    }
  }
  off += ksel_bytes;
  for (int c = 0; c < 4; ++c) {
    if (!kcount[c]) continue;
    const int width = n->sub_bits - 1 + c;
    if (width < 1 || width > 8) { fail(-1, "invalid NINT group-code width"); delete n; return nullptr; }
    const int64_t nb = packed_nbytes(int64_t(kcount[c]) * groups, width);
    if (!need(2 * nb)) { fail(-1, "truncated NINT payload"); delete n; return nullptr; }
    n->ls_base[c] = blob + off; off += nb;
    n->lm_base[c] = blob + off; off += nb;
  }
  const int64_t qsel_bytes = packed_nbytes(rows, 3);
  if (!need(qsel_bytes)) { fail(-1, "truncated NINT payload"); delete n; return nullptr; }
  n->q_class.resize(rows); n->q_rank.resize(rows);
  uint32_t qcount[8] = {};
  {
    std::vector<uint8_t> tmp(blob + off, blob + off + qsel_bytes);
    tmp.resize(tmp.size() + 4);
    for (int64_t r = 0; r < rows; ++r) {
      const uint32_t c = read_bits(tmp.data(), r, 3);
      n->q_class[r] = uint8_t(c);
      n->q_rank[r] = qcount[c]++;
    }
  }
  off += qsel_bytes;
  for (int c = 0; c < 8; ++c) {
    if (!qcount[c]) continue;
    const int64_t nb = packed_nbytes(int64_t(qcount[c]) * groups * gs, c + 1);
    if (!need(nb)) { fail(-1, "truncated NINT payload"); delete n; return nullptr; }
    n->q_base[c] = blob + off; off += nb;
  }
  if (off != nbytes) { fail(-1, "NINT payload has %lld trailing bytes", (long long)(nbytes - off)); delete n; return nullptr; }
  return n;
}

void mfq_nint_close(void* h) { delete static_cast<Nint*>(h); }
int64_t mfq_nint_rows(void* h) { return static_cast<Nint*>(h)->rows; }
int64_t mfq_nint_row_len(void* h) { return static_cast<Nint*>(h)->neuron_len; }

int mfq_nint_row_bits(void* h, int64_t row, int* q_bits, int* k_bits) {
  auto* n = static_cast<Nint*>(h);
  if (row < 0 || row >= n->rows) return fail(-1, "row out of range");
  *q_bits = n->q_class[row] + 1;
  *k_bits = n->sub_bits - 1 + n->k_class[row];
  return 0;
}
}

namespace {
// Bit reads near the end of the payload would touch up to 2 bytes past it; the last rows go through a padded copy.
template <typename F>
void for_row(const Nint& n, int64_t r, F&& emit) {
  const int kc = n.k_class[r], qc = n.q_class[r];
  const int kw = n.sub_bits - 1 + kc, qw = qc + 1;
  uint16_t dh, dmh;
  memcpy(&dh, n.d + 2 * r, 2);
  memcpy(&dmh, n.dm + 2 * r, 2);
  const float d = half_to_float(dh), dm = half_to_float(dmh);
  const uint8_t* payload_end = n.blob + n.nbytes;
  for (int64_t g = 0; g < n.groups; ++g) {
    const int64_t ki = int64_t(n.k_rank[r]) * n.groups + g;
    auto safe = [&](const uint8_t* base, int64_t idx, int w) -> uint32_t {
      const int64_t bit = idx * w;
      const uint8_t* p = base + (bit >> 3);
      uint8_t tmp[3] = {0, 0, 0};
      if (p + 3 > payload_end) {  // the last codes of the payload: read through a zero-padded copy
        memcpy(tmp, p, size_t(payload_end - p));
        p = tmp;
      }
      const uint32_t v = uint32_t(p[0]) | uint32_t(p[1]) << 8 | uint32_t(p[2]) << 16;
      return (v >> (bit & 7)) & ((1u << w) - 1u);
    };
    const float scale = d * float(safe(n.ls_base[kc], ki, kw));
    const float shift = dm * float(safe(n.lm_base[kc], ki, kw));
    const int64_t q0 = (int64_t(n.q_rank[r]) * n.groups + g) * n.gs;
    const int64_t col0 = g * n.gs;
    const int64_t cols = std::min<int64_t>(n.gs, n.neuron_len - col0);
    for (int64_t i = 0; i < cols; ++i) emit(col0 + i, scale * float(safe(n.q_base[qc], q0 + i, qw)) - shift);
  }
}
}  // namespace

extern "C" {

int mfq_nint_decode(void* h, int64_t row_begin, int64_t row_end, float* out, int threads) {
  auto* n = static_cast<Nint*>(h);
  if (row_begin < 0 || row_end > n->rows || row_begin > row_end) return fail(-1, "row range out of bounds");
  mfqn::parallel_for(row_end - row_begin, threads, [&](int64_t b, int64_t e) {
    for (int64_t i = b; i < e; ++i) {
      float* dst = out + i * n->neuron_len;
      for_row(*n, row_begin + i, [&](int64_t col, float v) { dst[col] = v; });
    }
  });
  return 0;
}

int mfq_nint_gemv(void* h, int64_t row_begin, int64_t row_end, const float* x, float* y, int threads) {
  auto* n = static_cast<Nint*>(h);
  if (row_begin < 0 || row_end > n->rows || row_begin > row_end) return fail(-1, "row range out of bounds");
  mfqn::parallel_for(row_end - row_begin, threads, [&](int64_t b, int64_t e) {
    for (int64_t i = b; i < e; ++i) {
      double acc = 0.0;
      for_row(*n, row_begin + i, [&](int64_t col, float v) { acc += double(v) * double(x[col]); });
      y[i] = float(acc);
    }
  });
  return 0;
}

// MXFP4: two E2M1 codes per byte (low nibble first), one E8M0 exponent per 32 values along the row.
int mfq_mxfp4_decode(const uint8_t* codes, const uint8_t* scales, int64_t rows, int64_t cols, float* out, int threads) {
  if (cols % 32) return fail(-1, "MXFP4 rows must be a multiple of 32 wide");
  static const float kE2M1[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};
  mfqn::parallel_for(rows, threads, [&](int64_t b, int64_t e) {
    for (int64_t r = b; r < e; ++r)
      for (int64_t blk = 0; blk < cols / 32; ++blk) {
        const uint8_t ex = scales[r * (cols / 32) + blk];
        const float s = ex == 0xFF ? NAN : std::ldexp(1.0f, int(ex) - 127);
        const uint8_t* src = codes + (r * cols + blk * 32) / 2;
        float* dst = out + r * cols + blk * 32;
        for (int i = 0; i < 16; ++i) {
          dst[2 * i] = kE2M1[src[i] & 0xF] * s;
          dst[2 * i + 1] = kE2M1[src[i] >> 4] * s;
        }
      }
  });
  return 0;
}

// NVQ rows from their unpacked streams: w = anchor[row] * sub[row, group] * table[index][i] * sign.
//   indices [rows, nvec] (u16), signs [rows, ceil(n/8)]: 7 stored sign bits per 8 weights, the eighth is their parity
//   (XOR bit 7 of the index when index_parity != 0, which needs vec == 8), sub [rows, ceil(n/gs)] (u8),
//   anchors [rows] f32, table [entries, vec] f32 magnitudes.
int mfq_nvq_decode(const uint16_t* indices, const uint8_t* signs, const uint8_t* sub, const float* anchors, const float* table,
                   int64_t rows, int64_t n, int gs, int vec, int entries, int index_parity, float* out, int threads) {
  if (rows <= 0 || n <= 0 || gs <= 0 || (vec != 4 && vec != 8) || entries <= 0) return fail(-1, "bad NVQ geometry");
  if (index_parity && vec != 8) return fail(-1, "index-parity signs need 8-wide vectors");
  const int64_t nvec = (n + vec - 1) / vec, nsign = (n + 7) / 8, ng = (n + gs - 1) / gs;
  int bad = 0;
  mfqn::parallel_for(rows, threads, [&](int64_t b, int64_t e) {
    for (int64_t r = b; r < e; ++r) {
      const uint16_t* ir = indices + r * nvec;
      const uint8_t* sr = signs + r * nsign;
      const uint8_t* gr = sub + r * ng;
      float* dst = out + r * n;
      for (int64_t i = 0; i < n; ++i) {
        const uint16_t idx = ir[i / vec];
        if (idx >= entries) { bad = 1; dst[i] = 0.f; continue; }
        const uint8_t m = sr[i / 8];
        const int bit = int(i % 8);
        int neg;
        if (bit < 7) {
          neg = (m >> bit) & 1;
        } else {
          neg = __builtin_popcount(m & 0x7F) & 1;
          if (index_parity) neg ^= (ir[i / 8] >> 7) & 1;
        }
        const float v = table[int64_t(idx) * vec + i % vec] * anchors[r] * float(gr[i / gs]);
        dst[i] = neg ? -v : v;
      }
    }
  });
  return bad ? fail(-2, "NVQ index outside the codebook") : 0;
}

static float e4m3_to_float(uint8_t c) {
  const int sign = c >> 7, exp = (c >> 3) & 0xF, man = c & 7;
  float v;
  if (exp == 0) v = std::ldexp(float(man), -9);
  else if (exp == 15 && man == 7) v = NAN;
  else v = std::ldexp(1.0f + float(man) / 8.0f, exp - 7);
  return sign ? -v : v;
}

// E4M3 codes with one fp32 multiplier per block x block tile (scales [ceil(rows/block), ceil(cols/block)]).
int mfq_fp8_block_decode(const uint8_t* codes, const float* scales, int64_t rows, int64_t cols, int block, float* out, int threads) {
  if (block <= 0) return fail(-1, "block must be positive");
  float table[256];
  for (int i = 0; i < 256; ++i) table[i] = e4m3_to_float(uint8_t(i));
  const int64_t sc = (cols + block - 1) / block;
  mfqn::parallel_for(rows, threads, [&](int64_t b, int64_t e) {
    for (int64_t r = b; r < e; ++r)
      for (int64_t c = 0; c < cols; ++c) out[r * cols + c] = table[codes[r * cols + c]] * scales[(r / block) * sc + c / block];
  });
  return 0;
}

void mfq_f32_to_bf16(const float* in, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    uint32_t u;
    memcpy(&u, in + i, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) { out[i] = uint16_t((u >> 16) | 0x40); continue; }  // quiet NaN
    out[i] = uint16_t((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
  }
}
}
