// CPU oracle for the quantized mixture-of-experts FFN hot path.
//
// TEST INFRASTRUCTURE ONLY.  This file restates, in plain C++, the f32 "reference mode"
// arithmetic of MoE4All's CPU interpreter (crates/infr-cpu) so that the CUDA library can be
// checked against it and so that the CPU path can be timed beside the GPU one.  Nothing in the
// product library links, loads or calls it; only the test-suite, the smoke check and the
// benchmark's CPU-baseline leg do.
//
// Parity is pinned by the reference's own known-answer material (see tests/test_oracle_*.py):
// the patterned Q4_K / Q6_K blocks of crates/infr-gguf/src/dequant.rs:1174-1202, the routing
// vectors of crates/infr-llama/tests/seam_op_parity.rs:2352-2554 and the hand-written layer
// reference `moe_ref` at :2245-2343, all re-created from their formulas.
//
// Arithmetic rules the reference follows and this file keeps (Rust never contracts a*b+c):
//   * fused multiply-add ONLY where the reference calls `mul_add` (inside `dot`);
//   * every other a*b+c is a rounded multiply followed by a rounded add  → build with
//     -ffp-contract=off;
//   * `iter().sum::<f32>()` is a left-to-right fold starting at 0; `sort_by` is stable;
//   * expf / logf / sqrtf are libm's.
//
// Build: see oracle/Makefile (g++ -O2 -mavx2 -mfma -ffp-contract=off -shared -fPIC).

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <limits>
#include <numeric>
#include <thread>
#include <vector>

#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#define ORC_AVX2 1
#endif

namespace {

// dtype ids follow the public GGUF/ggml numbering.
enum : int { DT_F32 = 0, DT_Q4_0 = 2, DT_Q4_1 = 3, DT_Q5_0 = 6, DT_Q5_1 = 7, DT_Q8_0 = 8, DT_Q2K = 10, DT_Q3K = 11, DT_Q4K = 12, DT_Q5K = 13, DT_Q6K = 14, DT_IQ4NL = 20, DT_IQ4XS = 23, DT_MXFP4 = 39, DT_NVFP4 = 40, DT_Q2_0 = 42, DT_IQ2XS = 17, DT_IQ3XXS = 18, DT_IQ3S = 21, DT_IQ2S = 22 };

// IEEE binary16 → binary32, exact (what `half::f16::to_f32` does; dequant.rs:72-74).
inline float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {  // subnormal: renormalise
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while ((man & 0x400u) == 0);
      man &= 0x3FFu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

// 6-bit (scale, min) of sub-block j of a Q4_K block (dequant.rs:77-87).
inline void k4(int j, const uint8_t* q, uint32_t& sc, uint32_t& m) {
  if (j < 4) {
    sc = q[j] & 63u;
    m = q[j + 4] & 63u;
  } else {
    sc = (uint32_t)((q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4));
    m = (uint32_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

// One Q4_K super-block (144 B → 256 f32).  Factored form dequant.rs:315-335, expansion
// dequant.rs:35-51: per 16-element group  sc = f32(d)*scm ; mn = f32(dmin)*(-m) ;
// out = sc*code + mn  (multiply, then add; no fma).
void dequant_q4k_block(const uint8_t* blk, float* out) {
  const float d = f16_to_f32(rd16(blk));
  const float dmin = f16_to_f32(rd16(blk + 2));
  const uint8_t* scales = blk + 4;
  const uint8_t* qs = blk + 16;
  for (int j = 0; j < 4; ++j) {
    uint32_t sc1, m1, sc2, m2;
    k4(2 * j, scales, sc1, m1);
    k4(2 * j + 1, scales, sc2, m2);
    const float s1 = d * (float)(int16_t)sc1;
    const float n1 = dmin * (float)(int16_t)(-(int)m1);
    const float s2 = d * (float)(int16_t)sc2;
    const float n2 = dmin * (float)(int16_t)(-(int)m2);
    for (int l = 0; l < 32; ++l) {
      const uint8_t v = qs[j * 32 + l];
      out[j * 64 + l] = s1 * (float)(v & 0xF) + n1;
      out[j * 64 + 32 + l] = s2 * (float)(v >> 4) + n2;
    }
  }
}

// One Q6_K super-block (210 B → 256 f32).  dequant.rs:365-389: per 16-element group
// sc = f32(d)*s ; mn = f32(d)*(-32*s) ; out = sc*code + mn.
void dequant_q6k_block(const uint8_t* blk, float* out) {
  const uint8_t* ql = blk;
  const uint8_t* qh = blk + 128;
  const int8_t* scales = (const int8_t*)(blk + 192);
  const float d = f16_to_f32(rd16(blk + 208));
  float sc[16], mn[16];
  for (int g = 0; g < 16; ++g) {
    const int16_t s = (int16_t)scales[g];
    sc[g] = d * (float)s;
    mn[g] = d * (float)(int16_t)(-32 * s);
  }
  for (int half = 0; half < 2; ++half) {
    const int qlo = half * 64, qho = half * 32, base = half * 128;
    for (int l = 0; l < 32; ++l) {
      const uint8_t c0 = (uint8_t)((ql[qlo + l] & 0xF) | ((qh[qho + l] & 3) << 4));
      const uint8_t c1 = (uint8_t)((ql[qlo + l + 32] & 0xF) | (((qh[qho + l] >> 2) & 3) << 4));
      const uint8_t c2 = (uint8_t)((ql[qlo + l] >> 4) | (((qh[qho + l] >> 4) & 3) << 4));
      const uint8_t c3 = (uint8_t)((ql[qlo + l + 32] >> 4) | (((qh[qho + l] >> 6) & 3) << 4));
      const int e0 = base + l, e1 = base + l + 32, e2 = base + l + 64, e3 = base + l + 96;
      out[e0] = sc[e0 / 16] * (float)c0 + mn[e0 / 16];
      out[e1] = sc[e1 / 16] * (float)c1 + mn[e1 / 16];
      out[e2] = sc[e2 / 16] * (float)c2 + mn[e2 / 16];
      out[e3] = sc[e3 / 16] * (float)c3 + mn[e3 / 16];
    }
  }
}

// One Q5_K super-block (176 B -> 256 f32).  Factored form dequant.rs:337-362: Q4_K's scales and
// mins, nibbles at byte 48, and bit 2j (low nibble) / 2j+1 (high nibble) of qh[l] (byte 16 + l) as
// the fifth code bit; expansion dequant.rs:35-51 as for Q4_K.
void dequant_q5k_block(const uint8_t* blk, float* out) {
  const float d = f16_to_f32(rd16(blk));
  const float dmin = f16_to_f32(rd16(blk + 2));
  const uint8_t* scales = blk + 4;
  const uint8_t* qh = blk + 16;
  const uint8_t* qs = blk + 48;
  uint8_t u1 = 1, u2 = 2;
  for (int j = 0; j < 4; ++j) {
    uint32_t sc1, m1, sc2, m2;
    k4(2 * j, scales, sc1, m1);
    k4(2 * j + 1, scales, sc2, m2);
    const float s1 = d * (float)(int16_t)sc1;
    const float n1 = dmin * (float)(int16_t)(-(int)m1);
    const float s2 = d * (float)(int16_t)sc2;
    const float n2 = dmin * (float)(int16_t)(-(int)m2);
    for (int l = 0; l < 32; ++l) {
      const uint8_t v = qs[j * 32 + l];
      const uint8_t c1 = (uint8_t)((v & 0xF) + ((qh[l] & u1) ? 16 : 0));
      const uint8_t c2 = (uint8_t)((v >> 4) + ((qh[l] & u2) ? 16 : 0));
      out[j * 64 + l] = s1 * (float)c1 + n1;
      out[j * 64 + 32 + l] = s2 * (float)c2 + n2;
    }
    u1 = (uint8_t)(u1 << 2);
    u2 = (uint8_t)(u2 << 2);
  }
}

// One Q8_0 block (34 B -> 32 f32).  Factored form dequant.rs:214-223: code = q + 128, scale pair
// (1, -128) on (d, d); expansion dequant.rs:35-51: sc = d*1 ; mn = d*(-128) ; out = sc*code + mn.
void dequant_q80_block(const uint8_t* blk, float* out) {
  const float d = f16_to_f32(rd16(blk));
  const float sc = d * 1.0f, mn = d * -128.0f;
  for (int i = 0; i < 32; ++i) {
    const uint8_t code = (uint8_t)((int)(int8_t)blk[2 + i] + 128);
    out[i] = sc * (float)code + mn;
  }
}

// The legacy 32-weight formats (dequant.rs:142-212), factored as code, (sc, m) = (1, k) on (d, d or m), expanded
// as everywhere (dequant.rs:35-51): out = (f32(d) * sc) * code + (f32(d or m) * m).
//   Q4_0: d, 16 code bytes; m = -8.     Q4_1: d, m, 16 code bytes; m-factor 1 on the block's own m.
//   Q5_0: d, 32 high bits, 16 code bytes; m = -16.   Q5_1: d, m, 32 high bits, 16 code bytes.
// Code j = low nibble of byte j (| bit j of the high bits << 4), code j + 16 = high nibble (| bit j + 16).
void dequant_legacy32_block(int dtype, const uint8_t* blk, float* out) {
  const bool has_m = dtype == DT_Q4_1 || dtype == DT_Q5_1, five = dtype == DT_Q5_0 || dtype == DT_Q5_1;
  const float d = f16_to_f32(rd16(blk));
  const float sc = d * 1.0f;
  const float mn = has_m ? f16_to_f32(rd16(blk + 2)) * 1.0f : d * (five ? -16.0f : -8.0f);
  const int hdr = has_m ? 4 : 2;
  uint32_t qh = 0;
  if (five) qh = (uint32_t)blk[hdr] | ((uint32_t)blk[hdr + 1] << 8) | ((uint32_t)blk[hdr + 2] << 16) | ((uint32_t)blk[hdr + 3] << 24);
  const uint8_t* qs = blk + hdr + (five ? 4 : 0);
  for (int j = 0; j < 16; ++j) {
    uint32_t c0 = qs[j] & 0x0Fu, c1 = qs[j] >> 4;
    if (five) {
      c0 |= ((qh >> j) << 4) & 0x10u;
      c1 |= (qh >> (j + 12)) & 0x10u;
    }
    out[j] = sc * (float)c0 + mn;
    out[j + 16] = sc * (float)c1 + mn;
  }
}

// One Q2_K block (84 B -> 256 f32), dequant.rs:224-252: 16 scale bytes (scale low nibble, min high nibble, one
// per 16 elements), 64 code bytes (2 bits per element), d, dmin: out = (d * sc) * code + (dmin * -m).
void dequant_q2k_block(const uint8_t* blk, float* out) {
  const uint8_t* scales = blk;
  const uint8_t* qs = blk + 16;
  const float d = f16_to_f32(rd16(blk + 80)), dmin = f16_to_f32(rd16(blk + 82));
  int o = 0, is = 0;
  for (int n = 0; n < 2; ++n)
    for (int j = 0; j < 4; ++j)
      for (int half = 0; half < 2; ++half) {
        const uint8_t s = scales[is++];
        const float sc = d * (float)(int16_t)(s & 0xF), mn = dmin * (float)(int16_t)(-(int)(s >> 4));
        for (int l = 0; l < 16; ++l) out[o++] = sc * (float)((qs[32 * n + 16 * half + l] >> (2 * j)) & 3) + mn;
      }
}

// One Q3_K block (110 B -> 256 f32), dequant.rs:253-314: 32 high-bit bytes, 64 code bytes, 12 bytes holding
// sixteen 6-bit scales, d: s = sc6 - 32 per 16 elements, out = (d * s) * code + (d * (-4 s)), code = low2 | high << 2.
void dequant_q3k_block(const uint8_t* blk, float* out) {
  const uint8_t* hmask = blk;
  const uint8_t* qs = blk + 32;
  const uint8_t* sr = blk + 96;
  const float d = f16_to_f32(rd16(blk + 108));
  auto rd32 = [](const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); };
  const uint32_t a0 = rd32(sr), a1 = rd32(sr + 4), tmp = rd32(sr + 8), k1 = 0x03030303u, k2 = 0x0f0f0f0fu;
  const uint32_t aux[4] = {(a0 & k2) | ((tmp & k1) << 4), (a1 & k2) | (((tmp >> 2) & k1) << 4), ((a0 >> 4) & k2) | (((tmp >> 4) & k1) << 4),
                           ((a1 >> 4) & k2) | (((tmp >> 6) & k1) << 4)};
  int o = 0, is = 0;
  uint8_t m = 1;
  for (int n = 0; n < 2; ++n)
    for (int j = 0; j < 4; ++j) {
      for (int half = 0; half < 2; ++half) {
        const int16_t s = (int16_t)((int8_t)(uint8_t)((aux[is / 4] >> ((is % 4) * 8)) & 0xFF)) - 32;
        ++is;
        const float sc = d * (float)s, mn = d * (float)(int16_t)(-4 * s);
        for (int l = 0; l < 16; ++l) {
          const uint8_t low2 = (qs[32 * n + 16 * half + l] >> (2 * j)) & 3, high = (hmask[16 * half + l] & m) ? 1 : 0;
          out[o++] = sc * (float)(uint8_t)(low2 | (high << 2)) + mn;
        }
      }
      m = (uint8_t)(m << 1);
    }
}

// The 16-entry signed codebook of the two non-linear 4-bit formats (dequant.rs:443-445).
const int8_t KV_IQ4NL[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

// One IQ4_NL block (18 B -> 32 f32), dequant.rs:499-517: y[j] = d * kv[qs[j] & 0xF], y[j + 16] = d * kv[qs[j] >> 4].
void dequant_iq4nl_block(const uint8_t* blk, float* out) {
  const float d = f16_to_f32(rd16(blk));
  const uint8_t* qs = blk + 2;
  for (int j = 0; j < 16; ++j) {
    out[j] = d * (float)KV_IQ4NL[qs[j] & 0xF];
    out[j + 16] = d * (float)KV_IQ4NL[qs[j] >> 4];
  }
}

// One MXFP4 block (17 B -> 32 f32), dequant.rs:409-421, 1029-1046: an E8M0 exponent byte e (d = 2^(e - 128), built
// from bits as `e8m0_to_fp32_half` does), 16 code bytes indexing the E2M1 x 2 table; y = kv * d.
void dequant_mxfp4_block(const uint8_t* blk, float* out) {
  static const int8_t KV[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};
  const uint32_t e = blk[0], bits = e < 2 ? (0x00200000u << e) : ((e - 1) << 23);
  float d;
  std::memcpy(&d, &bits, 4);
  const uint8_t* qs = blk + 1;
  for (int j = 0; j < 16; ++j) {
    out[j] = (float)KV[qs[j] & 0xF] * d;
    out[j + 16] = (float)KV[qs[j] >> 4] * d;
  }
}

// One NVFP4 block (36 B -> 64 f32), dequant.rs:423-439, 1053-1073: four UE4M3 scale bytes (4 exponent bits with
// bias 7, 3 mantissa bits, the value halved; 0x00 and 0x7F decode to 0), one per 16 weights; 8 code bytes per 16
// weights index the E2M1 x 2 table, low nibbles weights 0-7, high nibbles weights 8-15; y = kv * d.
float ue4m3_half(uint8_t x) {
  if (x == 0 || x == 0x7F) return 0.0f;
  const int ex = (x >> 3) & 0xF;
  const float man = (float)(x & 7);
  const float raw = ex == 0 ? man * std::ldexp(1.0f, -9) : (1.0f + man / 8.0f) * std::ldexp(1.0f, ex - 7);
  return raw * 0.5f;
}
void dequant_nvfp4_block(const uint8_t* blk, float* out) {
  static const int8_t KV[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};
  const uint8_t* qs = blk + 4;
  for (int s = 0; s < 4; ++s) {
    const float d = ue4m3_half(blk[s]);
    for (int j = 0; j < 8; ++j) {
      out[16 * s + j] = (float)KV[qs[8 * s + j] & 0xF] * d;
      out[16 * s + j + 8] = (float)KV[qs[8 * s + j] >> 4] * d;
    }
  }
}

// One Q2_0 block (18 B -> 64 f32), dequant.rs:1007-1022: f16 d, 2-bit codes (weight j in byte j / 4 at bit
// 2 (j % 4)); y = (q - 1) * d.
void dequant_q2_0_block(const uint8_t* blk, float* out) {
  const float d = f16_to_f32(rd16(blk));
  for (int j = 0; j < 64; ++j) out[j] = (float)((int)((blk[2 + j / 4] >> ((j % 4) * 2)) & 3) - 1) * d;
}

// ---- grid codebook formats (dequant.rs:477-488, 605-770) ------------------------------------------------
// A group of 8 (IQ2) or 4 (IQ3) weights is one entry of the format's grid table (one byte per weight) with a
// sign bit per weight; out = db * grid byte * (+-1), db the group's scale.  The tables are constants of the
// formats kept by the reference (crates/infr-core/src/iquant_grids.rs); this restatement does not carry them:
// the tests hand them in (orc_set_codebook).  Slots: 0 IQ2_XS (512 x 8), 1 IQ3_XXS (256 x 4), 2 IQ3_S (512 x 4),
// 3 IQ2_S (1024 x 8).
std::vector<uint8_t> g_codebook[4];
int codebook_slot(int dt) { return dt == DT_IQ2XS ? 0 : dt == DT_IQ3XXS ? 1 : dt == DT_IQ3S ? 2 : dt == DT_IQ2S ? 3 : -1; }
size_t codebook_bytes(int slot) { return slot == 0 ? 4096 : slot == 1 ? 1024 : slot == 2 ? 2048 : slot == 3 ? 8192 : 0; }
// The sign byte of a 7-bit index: the index with its parity on top (KSIGNS_IQ2XS, iquant_grids.rs:6-16).
uint8_t ksigns(uint32_t i) { return (uint8_t)(i | ((uint32_t)(__builtin_popcount(i) & 1) << 7)); }
// n weights from grid bytes `g`, sign bits sign_off .. sign_off + n - 1 of `signs` (apply_signs, dequant.rs:477-488)
void put_signed(float* out, const uint8_t* g, uint8_t signs, int sign_off, int n, float db) {
  for (int j = 0; j < n; ++j) {
    const float gv = (float)(int8_t)g[j];
    out[j] = db * gv * ((signs >> (sign_off + j)) & 1 ? -1.0f : 1.0f);
  }
}
void dequant_iq2xs_block(const uint8_t* blk, float* out) {  // 74 B: d, 32 x u16 (9-bit grid index, 7-bit sign index), 8 scale bytes
  const float d = f16_to_f32(rd16(blk));
  const uint8_t* grid = g_codebook[0].data();
  for (int ib32 = 0; ib32 < 8; ++ib32) {
    const uint8_t sc = blk[66 + ib32];
    const float db0 = d * (0.5f + (float)(sc & 0xF)) * 0.25f, db1 = d * (0.5f + (float)(sc >> 4)) * 0.25f;
    for (int l = 0; l < 4; ++l) {
      const uint32_t q = rd16(blk + 2 + 2 * (ib32 * 4 + l));
      put_signed(out + ib32 * 32 + l * 8, grid + 8 * (q & 511), ksigns(q >> 9), 0, 8, l < 2 ? db0 : db1);
    }
  }
}
void dequant_iq2s_block(const uint8_t* blk, float* out) {  // 82 B: d, 32 grid bytes, 32 sign bytes, 8 high-bit bytes, 8 scale bytes
  const float d = f16_to_f32(rd16(blk));
  const uint8_t* grid = g_codebook[3].data();
  for (int ib32 = 0; ib32 < 8; ++ib32) {
    const uint8_t sc = blk[74 + ib32], qh = blk[66 + ib32];
    const float db0 = d * (0.5f + (float)(sc & 0xF)) * 0.25f, db1 = d * (0.5f + (float)(sc >> 4)) * 0.25f;
    for (int l = 0; l < 4; ++l) {
      const uint32_t idx = (uint32_t)blk[2 + ib32 * 4 + l] | (((uint32_t)qh << (8 - 2 * l)) & 0x300u);
      put_signed(out + ib32 * 32 + l * 8, grid + 8 * idx, blk[34 + ib32 * 4 + l], 0, 8, l < 2 ? db0 : db1);
    }
  }
}
void dequant_iq3xxs_block(const uint8_t* blk, float* out) {  // 98 B: d, 64 grid bytes, 8 words of 4 x 7 sign-index bits + 4 scale bits
  const float d = f16_to_f32(rd16(blk));
  const uint8_t* grid = g_codebook[1].data();
  for (int ib32 = 0; ib32 < 8; ++ib32) {
    const uint32_t aux = (uint32_t)rd16(blk + 66 + 4 * ib32) | ((uint32_t)rd16(blk + 68 + 4 * ib32) << 16);
    const float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
    for (int l = 0; l < 4; ++l) {
      const uint8_t sg = ksigns((aux >> (7 * l)) & 127);
      put_signed(out + ib32 * 32 + l * 8, grid + 4 * blk[2 + 8 * ib32 + 2 * l], sg, 0, 4, db);
      put_signed(out + ib32 * 32 + l * 8 + 4, grid + 4 * blk[3 + 8 * ib32 + 2 * l], sg, 4, 4, db);
    }
  }
}
void dequant_iq3s_block(const uint8_t* blk, float* out) {  // 110 B: d, 64 grid bytes, 8 ninth-bit bytes, 32 sign bytes, 4 scale bytes
  const float d = f16_to_f32(rd16(blk));
  const uint8_t* grid = g_codebook[2].data();
  for (int ib32 = 0; ib32 < 8; ++ib32) {
    const uint8_t sb = blk[106 + ib32 / 2], qh = blk[66 + ib32];
    const float db = d * (1.0f + 2.0f * (float)((ib32 & 1) ? sb >> 4 : sb & 0xF));
    for (int l = 0; l < 4; ++l) {
      const uint32_t i1 = (uint32_t)blk[2 + 8 * ib32 + 2 * l] | (((uint32_t)qh << (8 - 2 * l)) & 256u);
      const uint32_t i2 = (uint32_t)blk[3 + 8 * ib32 + 2 * l] | (((uint32_t)qh << (7 - 2 * l)) & 256u);
      const uint8_t sg = blk[74 + 4 * ib32 + l];
      put_signed(out + ib32 * 32 + l * 8, grid + 4 * i1, sg, 0, 4, db);
      put_signed(out + ib32 * 32 + l * 8 + 4, grid + 4 * i2, sg, 4, 4, db);
    }
  }
}

// One IQ4_XS block (136 B -> 256 f32), dequant.rs:521-553: eight sub-blocks of 32 with a 6-bit scale
// ls (low four bits in scales_l, high two in scales_h); dl = d * (ls - 32); codes as in IQ4_NL.
void dequant_iq4xs_block(const uint8_t* blk, float* out) {
  const float d = f16_to_f32(rd16(blk));
  const uint32_t scales_h = rd16(blk + 2);
  const uint8_t* scales_l = blk + 4;
  const uint8_t* qs = blk + 8;
  for (int ib = 0; ib < 8; ++ib) {
    const uint32_t lo = (uint32_t)(scales_l[ib / 2] >> (4 * (ib % 2))) & 0xFu;
    const uint32_t hi = (scales_h >> (2 * ib)) & 3u;
    const float dl = d * (float)((int)(lo | (hi << 4)) - 32);
    for (int j = 0; j < 16; ++j) {
      out[ib * 32 + j] = dl * (float)KV_IQ4NL[qs[ib * 16 + j] & 0xF];
      out[ib * 32 + j + 16] = dl * (float)KV_IQ4NL[qs[ib * 16 + j] >> 4];
    }
  }
}

size_t row_bytes(int dtype, size_t n_elem) {
  switch (dtype) {
    case DT_F32: return n_elem * 4;
    case DT_Q4_0: return n_elem / 32 * 18;
    case DT_Q4_1: return n_elem / 32 * 20;
    case DT_Q5_0: return n_elem / 32 * 22;
    case DT_Q5_1: return n_elem / 32 * 24;
    case DT_Q2K: return n_elem / 256 * 84;
    case DT_Q3K: return n_elem / 256 * 110;
    case DT_IQ4NL: return n_elem / 32 * 18;
    case DT_IQ4XS: return n_elem / 256 * 136;
    case DT_MXFP4: return n_elem / 32 * 17;
    case DT_NVFP4: return n_elem / 64 * 36;
    case DT_Q2_0: return n_elem / 64 * 18;
    case DT_IQ2XS: return n_elem / 256 * 74;
    case DT_IQ2S: return n_elem / 256 * 82;
    case DT_IQ3XXS: return n_elem / 256 * 98;
    case DT_IQ3S: return n_elem / 256 * 110;
    case DT_Q8_0: return n_elem / 32 * 34;
    case DT_Q4K: return n_elem / 256 * 144;
    case DT_Q5K: return n_elem / 256 * 176;
    case DT_Q6K: return n_elem / 256 * 210;
    default: return 0;
  }
}

// `bytes_to_f32(row, dt)` of the reference (infr-cpu/src/lib.rs:513-527): a weight row → f32.
bool dequant_row(int dtype, const uint8_t* bytes, size_t n_elem, float* out) {
  switch (dtype) {
    case DT_F32:
      std::memcpy(out, bytes, n_elem * 4);
      return true;
    case DT_Q4K:
      if (n_elem % 256) return false;
      for (size_t b = 0; b < n_elem / 256; ++b) dequant_q4k_block(bytes + b * 144, out + b * 256);
      return true;
    case DT_Q6K:
      if (n_elem % 256) return false;
      for (size_t b = 0; b < n_elem / 256; ++b) dequant_q6k_block(bytes + b * 210, out + b * 256);
      return true;
    case DT_Q5K:
      if (n_elem % 256) return false;
      for (size_t b = 0; b < n_elem / 256; ++b) dequant_q5k_block(bytes + b * 176, out + b * 256);
      return true;
    case DT_Q8_0:
      if (n_elem % 32) return false;
      for (size_t b = 0; b < n_elem / 32; ++b) dequant_q80_block(bytes + b * 34, out + b * 32);
      return true;
    case DT_Q4_0:
    case DT_Q4_1:
    case DT_Q5_0:
    case DT_Q5_1: {
      if (n_elem % 32) return false;
      const size_t bb = row_bytes(dtype, 32);
      for (size_t b = 0; b < n_elem / 32; ++b) dequant_legacy32_block(dtype, bytes + b * bb, out + b * 32);
      return true;
    }
    case DT_Q2K:
      if (n_elem % 256) return false;
      for (size_t b = 0; b < n_elem / 256; ++b) dequant_q2k_block(bytes + b * 84, out + b * 256);
      return true;
    case DT_Q3K:
      if (n_elem % 256) return false;
      for (size_t b = 0; b < n_elem / 256; ++b) dequant_q3k_block(bytes + b * 110, out + b * 256);
      return true;
    case DT_IQ4NL:
      if (n_elem % 32) return false;
      for (size_t b = 0; b < n_elem / 32; ++b) dequant_iq4nl_block(bytes + b * 18, out + b * 32);
      return true;
    case DT_MXFP4:
      if (n_elem % 32) return false;
      for (size_t b = 0; b < n_elem / 32; ++b) dequant_mxfp4_block(bytes + b * 17, out + b * 32);
      return true;
    case DT_NVFP4:
      if (n_elem % 64) return false;
      for (size_t b = 0; b < n_elem / 64; ++b) dequant_nvfp4_block(bytes + b * 36, out + b * 64);
      return true;
    case DT_Q2_0:
      if (n_elem % 64) return false;
      for (size_t b = 0; b < n_elem / 64; ++b) dequant_q2_0_block(bytes + b * 18, out + b * 64);
      return true;
    case DT_IQ2XS:
    case DT_IQ2S:
    case DT_IQ3XXS:
    case DT_IQ3S: {
      if (n_elem % 256 || g_codebook[codebook_slot(dtype)].empty()) return false;  // (no table handed in: not decodable)
      const size_t bb = row_bytes(dtype, 256);
      for (size_t b = 0; b < n_elem / 256; ++b) {
        const uint8_t* blk = bytes + b * bb;
        float* o = out + b * 256;
        if (dtype == DT_IQ2XS) dequant_iq2xs_block(blk, o);
        else if (dtype == DT_IQ2S) dequant_iq2s_block(blk, o);
        else if (dtype == DT_IQ3XXS) dequant_iq3xxs_block(blk, o);
        else dequant_iq3s_block(blk, o);
      }
      return true;
    }
    case DT_IQ4XS:
      if (n_elem % 256) return false;
      for (size_t b = 0; b < n_elem / 256; ++b) dequant_iq4xs_block(bytes + b * 136, out + b * 256);
      return true;
    default:
      return false;
  }
}

// `dot` of the reference, scalar form (infr-cpu/src/kernels.rs:6568-6583): eight accumulation
// lanes, lane j takes elements 8c+j by fma; lanes summed left to right; tail by fma.
float dot_scalar(const float* a, const float* b, size_t n) {
  const size_t chunks = n / 8;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (size_t c = 0; c < chunks; ++c)
    for (int j = 0; j < 8; ++j) acc[j] = std::fmaf(a[c * 8 + j], b[c * 8 + j], acc[j]);
  float s = 0.0f;
  for (int j = 0; j < 8; ++j) s = s + acc[j];
  for (size_t i = chunks * 8; i < n; ++i) s = std::fmaf(a[i], b[i], s);
  return s;
}

#ifdef ORC_AVX2
// AVX2 form (kernels.rs:6587-6608): one 8-wide fmadd per chunk, same lanes, same final order.
float dot_avx2(const float* a, const float* b, size_t n) {
  __m256 sum = _mm256_setzero_ps();
  size_t i = 0;
  for (; i + 8 <= n; i += 8)
    sum = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), sum);
  float lanes[8];
  _mm256_storeu_ps(lanes, sum);
  float s = 0.0f;
  for (int j = 0; j < 8; ++j) s = s + lanes[j];
  for (; i < n; ++i) s = std::fmaf(a[i], b[i], s);
  return s;
}
inline float dot(const float* a, const float* b, size_t n) { return dot_avx2(a, b, n); }
#else
inline float dot(const float* a, const float* b, size_t n) { return dot_scalar(a, b, n); }
#endif

inline float silu(float g) { return g / (1.0f + std::exp(-g)); }       // kernels.rs:6666
inline float sigmoidf(float v) { return 1.0f / (1.0f + std::exp(-v)); }  // kernels.rs:6670

// Run fn(i) for i in [0,n) on `threads` host threads, items claimed dynamically (the reference
// claims 64-row chunks from a shared counter the same way, infr-cpu/src/lib.rs:3992-4003).
void parallel_for(size_t n, int threads, const std::function<void(size_t)>& fn) {
  if (threads <= 1 || n <= 1) {
    for (size_t i = 0; i < n; ++i) fn(i);
    return;
  }
  std::atomic<size_t> next{0};
  auto work = [&]() {
    for (;;) {
      size_t i = next.fetch_add(1);
      if (i >= n) break;
      fn(i);
    }
  };
  std::vector<std::thread> pool;
  int nt = (int)std::min<size_t>((size_t)threads, n);
  for (int t = 1; t < nt; ++t) pool.emplace_back(work);
  work();
  for (auto& t : pool) t.join();
}

}  // namespace

extern "C" {

// Descriptor of one Op::MoeFfn call (crates/infr-core/src/graph.rs:1259-1352), restricted to the
// split gate/up form.
struct orc_moe_desc {
  const float* x;         // [rows, ne]
  const float* router_x;  // [rows, ne]
  const uint8_t* router;  // [n_expert, ne] router_dtype
  const uint8_t* gate_exps;  // [n_expert, n_ff_exp, ne]
  const uint8_t* up_exps;    // [n_expert, n_ff_exp, ne]
  const uint8_t* down_exps;  // [n_expert, ne, n_ff_exp]
  const float* exp_probs_b;  // [n_expert] or null
  float* dst;                // [rows, ne]
  int32_t* ids_out;          // [rows, n_used] or null
  float* wts_out;            // [rows, n_used] or null
  float* logits_out;         // [rows, n_expert] or null
  float* sel_out;            // [rows, n_expert] or null: the selection scores after bias/groups
  uint32_t rows, ne, n_expert, n_used, n_ff_exp;
  float scale;
  int32_t router_dtype, gate_dtype, up_dtype, down_dtype;
  uint32_t gating;  // 0 softmax, 1 sigmoid, 2 sqrt-softplus
  uint32_t norm_w;
  uint32_t n_expert_groups, n_expert_groups_used;
  uint32_t ep_lo, ep_n_local;  // band [ep_lo, ep_lo+ep_n_local); ep_n_local == 0 → no band
  int32_t threads;
  const int32_t* expert_ids;  // [rows, n_used] selection made by the caller (hash-routed layers), or null
  const float* down_scale;    // [n_expert] scale on an expert's down output before the weighted sum, or null
  uint32_t act;               // 0 SiLU, 1 GELU (tanh form), 2 Sigmoid
  uint32_t weight_before;     // routing weight applied to gate and up before the activation
  float swiglu_clamp;         // > 0: act(min(gate, l)) * clamp(up, -l, l)
  uint32_t fused_gate_up;     // gate_exps holds [n_expert, 2*n_ff_exp, ne]: gate rows then up rows; up_exps unused
};

int orc_has_avx2(void) {
#ifdef ORC_AVX2
  return 1;
#else
  return 0;
#endif
}

int orc_hw_threads(void) {
  unsigned n = std::thread::hardware_concurrency();
  return n ? (int)n : 1;
}

size_t orc_row_bytes(int dtype, size_t n_elem) { return row_bytes(dtype, n_elem); }

// The grid table of a codebook format (see above); 0 on success.
int orc_set_codebook(int dtype, const uint8_t* table, size_t bytes) {
  const int slot = codebook_slot(dtype);
  if (slot < 0 || bytes != codebook_bytes(slot)) return 1;
  g_codebook[slot].assign(table, table + bytes);
  return 0;
}

int orc_dequant(int dtype, const uint8_t* bytes, size_t n_elem, float* out) {
  return dequant_row(dtype, bytes, n_elem, out) ? 0 : -1;
}

float orc_dot(const float* a, const float* b, size_t n) { return dot(a, b, n); }
float orc_dot_scalar(const float* a, const float* b, size_t n) { return dot_scalar(a, b, n); }

// Routing of one row (infr-cpu/src/lib.rs:3741-3863).  logits → probs → selection copy (+bias,
// group mask) → stable descending sort → first n_used; weights from the UNBIASED probs.
static void route_row(const orc_moe_desc* d, const float* logits, const int32_t* given, int32_t* idx_out, float* w_out,
                      float* sel_out) {
  const uint32_t E = d->n_expert, k = d->n_used;
  std::vector<float> probs(E);
  if (d->gating == 0) {
    float maxl = -std::numeric_limits<float>::infinity();
    for (uint32_t e = 0; e < E; ++e) maxl = std::max(maxl, logits[e]);  // f32::max fold
    for (uint32_t e = 0; e < E; ++e) probs[e] = std::exp(logits[e] - maxl);
    float psum = 0.0f;
    for (uint32_t e = 0; e < E; ++e) psum = psum + probs[e];
    for (uint32_t e = 0; e < E; ++e) probs[e] = probs[e] / psum;
  } else if (d->gating == 1) {
    for (uint32_t e = 0; e < E; ++e) probs[e] = 1.0f / (1.0f + std::exp(-logits[e]));
  } else {
    for (uint32_t e = 0; e < E; ++e) {
      const float v = logits[e];
      const float sp = v > 20.0f ? v : std::log(1.0f + std::exp(v));
      probs[e] = std::sqrt(sp);
    }
  }
  std::vector<uint32_t> idx(E);
  std::vector<float> sel(probs);
  if (given) {
    // hash-routed layer (lib.rs:3776-3792): the given experts are the selection, nothing is ranked
    for (uint32_t s = 0; s < k; ++s) idx[s] = (uint32_t)given[s];
  } else {
  if (d->exp_probs_b)
    for (uint32_t e = 0; e < E; ++e) sel[e] = probs[e] + d->exp_probs_b[e];
  if (d->n_expert_groups > 1 && d->n_expert_groups_used > 0) {
    const uint32_t ng = d->n_expert_groups, per = E / ng, used = d->n_expert_groups_used;
    const float ninf = -std::numeric_limits<float>::infinity();
    std::vector<float> gs(ng, ninf);
    for (uint32_t g = 0; g < ng; ++g) {
      float best0 = ninf, best1 = ninf;
      for (uint32_t i = 0; i < per; ++i) {
        const float s = sel[g * per + i];
        if (s > best0) {
          best1 = best0;
          best0 = s;
        } else if (s > best1) {
          best1 = s;
        }
      }
      gs[g] = best0 + best1;
    }
    std::vector<uint32_t> gidx(ng);
    std::iota(gidx.begin(), gidx.end(), 0u);
    std::stable_sort(gidx.begin(), gidx.end(), [&](uint32_t a, uint32_t b) { return gs[a] > gs[b]; });
    std::vector<char> chosen(ng, 0);
    for (uint32_t i = 0; i < std::min(used, ng); ++i) chosen[gidx[i]] = 1;
    for (uint32_t g = 0; g < ng; ++g)
      if (!chosen[g])
        for (uint32_t i = 0; i < per; ++i) sel[g * per + i] = ninf;
  }
  std::iota(idx.begin(), idx.end(), 0u);
  std::stable_sort(idx.begin(), idx.end(), [&](uint32_t a, uint32_t b) { return sel[a] > sel[b]; });
  }
  if (d->norm_w) {
    float ws = 0.0f;
    for (uint32_t s = 0; s < k; ++s) ws = ws + probs[idx[s]];
    ws = std::max(ws, 1e-20f);
    for (uint32_t s = 0; s < k; ++s) w_out[s] = probs[idx[s]] / ws * d->scale;
  } else {
    for (uint32_t s = 0; s < k; ++s) w_out[s] = probs[idx[s]] * d->scale;
  }
  for (uint32_t s = 0; s < k; ++s) idx_out[s] = (int32_t)idx[s];
  if (sel_out) std::memcpy(sel_out, sel.data(), E * sizeof(float));
}

// act_fn / gated_act_fn (crates/infr-cpu/src/kernels.rs:6662-6683).
static inline float act_value(uint32_t act, float g) {
  if (act == 1) return 0.5f * g * (1.0f + std::tanh(0.7978846f * (g + 0.044715f * g * g * g)));
  if (act == 2) return 1.0f / (1.0f + std::exp(-g));
  return silu(g);
}
static inline float gated_act_value(uint32_t act, float clamp, float gate, float up) {
  if (clamp > 0.0f) return act_value(act, std::min(gate, clamp)) * std::min(std::max(up, -clamp), clamp);
  return act_value(act, gate) * up;
}

// Op::MoeFfn in reference mode (infr-cpu/src/lib.rs:3584-4304 with every bank on the f32
// activation path, :3675-3679; expert mat-vec = dequantised row + `dot`, moe.rs:142-173).
// Work is bucketed by expert like stages A-E of the reference; bucketing only reorders work, each
// output element sees the same operations in the same order as the per-row form.
int orc_moe_ffn(const orc_moe_desc* d) {
  const size_t R = d->rows, ne = d->ne, E = d->n_expert, k = d->n_used, nff = d->n_ff_exp;
  if (!R || !ne || !E || !k || !nff || k > E) return -1;
  const size_t rrb = row_bytes(d->router_dtype, ne), grb = row_bytes(d->gate_dtype, ne),
               urb = row_bytes(d->up_dtype, ne), drb = row_bytes(d->down_dtype, nff);
  if (!rrb || !grb || !urb || !drb) return -2;
  const int T = d->threads > 0 ? d->threads : orc_hw_threads();
  // the clamp is defined for the gated SiLU / GELU forms without weight_before (lib.rs:3613-3619)
  if (d->act > 2 || (d->swiglu_clamp > 0.0f && (d->weight_before || d->act == 2))) return -3;
  if (d->expert_ids) {
    // the reference refuses a bias or groups beside given ids (graph.rs:1304-1308) and panics on an
    // id past n_expert (lib.rs:3782-3788)
    if (d->exp_probs_b || d->n_expert_groups > 1) return -3;
    for (size_t i = 0; i < R * k; ++i)
      if (d->expert_ids[i] < 0 || (size_t)d->expert_ids[i] >= E) return -3;
  }

  // Router logits: logits[r,e] = dot(router_row_e, router_x[r])  (lib.rs:3684-3716).
  std::vector<float> logits(R * E);
  parallel_for(E, T, [&](size_t e) {
    std::vector<float> wf(ne);
    dequant_row(d->router_dtype, d->router + e * rrb, ne, wf.data());
    for (size_t r = 0; r < R; ++r) logits[r * E + e] = dot(wf.data(), d->router_x + r * ne, ne);
  });
  if (d->logits_out) std::memcpy(d->logits_out, logits.data(), R * E * sizeof(float));

  std::vector<int32_t> ids(R * k);
  std::vector<float> wts(R * k);
  parallel_for(R, T, [&](size_t r) {
    route_row(d, &logits[r * E], d->expert_ids ? d->expert_ids + r * k : nullptr, &ids[r * k], &wts[r * k],
              d->sel_out ? d->sel_out + r * E : nullptr);
  });
  if (d->ids_out) std::memcpy(d->ids_out, ids.data(), R * k * sizeof(int32_t));
  if (d->wts_out) std::memcpy(d->wts_out, wts.data(), R * k * sizeof(float));

  // Bucket the (row, rank) pairs by expert (lib.rs:3873-3907).  An expert outside the EP band
  // contributes nothing (graph.rs:1309-1319: out-of-band ids are remapped to weight 0).
  std::vector<std::vector<uint32_t>> bucket(E);
  const bool band = d->ep_n_local != 0;
  for (size_t p = 0; p < R * k; ++p) {
    const uint32_t e = (uint32_t)ids[p];
    if (band && (e < d->ep_lo || e >= d->ep_lo + d->ep_n_local)) continue;
    bucket[e].push_back((uint32_t)p);
  }
  std::vector<uint32_t> active;
  for (uint32_t e = 0; e < E; ++e)
    if (!bucket[e].empty()) active.push_back(e);

  // bytes per expert; a fused bank (graph.rs:1277-1282) holds an expert's gate rows, then its up rows
  const bool fused = d->fused_gate_up != 0;
  const size_t gst = grb * nff * (fused ? 2 : 1), ust = fused ? gst : urb * nff, dst_stride = drb * ne;
  const uint8_t* up_base = fused ? d->gate_exps + grb * nff : d->up_exps;
  std::vector<float> act(R * k * nff, 0.0f), y(R * k * ne, 0.0f);

  // Stages B + C: gate/up mat-vec then act = silu(g)*u  (lib.rs:4051-4212).
  struct Task { uint32_t e; uint32_t o0; };
  std::vector<Task> tasks;
  for (uint32_t e : active)
    for (uint32_t o0 = 0; o0 < nff; o0 += 64) tasks.push_back({e, o0});
  parallel_for(tasks.size(), T, [&](size_t ti) {
    const Task t = tasks[ti];
    std::vector<float> wg(ne), wu(ne);
    const size_t o1 = std::min<size_t>(t.o0 + 64, nff);
    for (size_t o = t.o0; o < o1; ++o) {
      dequant_row(d->gate_dtype, d->gate_exps + t.e * gst + o * grb, ne, wg.data());
      dequant_row(fused ? d->gate_dtype : d->up_dtype, up_base + t.e * ust + o * (fused ? grb : urb), ne, wu.data());
      for (uint32_t p : bucket[t.e]) {
        const float* xr = d->x + (size_t)(p / k) * ne;
        const float g = dot(wg.data(), xr, ne);
        const float u = dot(wu.data(), xr, ne);
        // llama4's weight_before: the pair's routing weight on gate and up, before the activation
        const float wp = d->weight_before ? wts[p] : 1.0f;
        act[(size_t)p * nff + o] = gated_act_value(d->act, d->swiglu_clamp, wp * g, wp * u);
      }
    }
  });

  // Stage D: down mat-vec (lib.rs:4214-4266).
  tasks.clear();
  for (uint32_t e : active)
    for (uint32_t o0 = 0; o0 < ne; o0 += 64) tasks.push_back({e, o0});
  parallel_for(tasks.size(), T, [&](size_t ti) {
    const Task t = tasks[ti];
    std::vector<float> wd(nff);
    const size_t o1 = std::min<size_t>(t.o0 + 64, ne);
    for (size_t o = t.o0; o < o1; ++o) {
      dequant_row(d->down_dtype, d->down_exps + t.e * dst_stride + o * drb, nff, wd.data());
      for (uint32_t p : bucket[t.e]) {
        const float raw = dot(wd.data(), &act[(size_t)p * nff], nff);
        y[(size_t)p * ne + o] = d->down_scale ? raw * d->down_scale[t.e] : raw;  // lib.rs:4252-4258
      }
    }
  });

  // Stage E: out += w*y in rank order, multiply then add (lib.rs:4287-4303).
  parallel_for(R, T, [&](size_t r) {
    float* o = d->dst + r * ne;
    for (size_t i = 0; i < ne; ++i) o[i] = 0.0f;
    for (size_t rank = 0; rank < k; ++rank) {
      const size_t p = r * k + rank;
      const uint32_t e = (uint32_t)ids[p];
      if (band && (e < d->ep_lo || e >= d->ep_lo + d->ep_n_local)) continue;
      const float w = d->weight_before ? 1.0f : wts[p];  // lib.rs:4295-4296
      const float* yr = &y[p * ne];
      for (size_t i = 0; i < ne; ++i) o[i] = o[i] + w * yr[i];
    }
  });
  return 0;
}

// Op::Linear, reference branch (infr-cpu/src/lib.rs:1312-1328; F32 weights :1459, :1752-1754):
// y[r,o] = dot(dequant(W row o), x[r]).
int orc_linear(int dtype, const uint8_t* w, const float* x, uint32_t m, uint32_t in_f,
               uint32_t out_f, float* y, int32_t threads) {
  const size_t rb = row_bytes(dtype, in_f);
  if (!rb) return -2;
  const int T = threads > 0 ? threads : orc_hw_threads();
  const size_t chunks = (out_f + 63) / 64;
  parallel_for(chunks, T, [&](size_t c) {
    std::vector<float> wf(in_f);
    const size_t o1 = std::min<size_t>((c + 1) * 64, out_f);
    for (size_t o = c * 64; o < o1; ++o) {
      dequant_row(dtype, w + o * rb, in_f, wf.data());
      for (size_t r = 0; r < m; ++r) y[r * out_f + o] = dot(wf.data(), x + r * in_f, in_f);
    }
  });
  return 0;
}

// Op::GatedAct with SiLU, contiguous operands (lib.rs:2973-3027; kernels.rs:6678-6683).
void orc_gated_act_silu(const float* gate, const float* up, float* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = silu(gate[i]) * up[i];
}

// Op::MoeSharedExpertAdd (lib.rs:3336-3356): dst = moe + sigmoid(gate[r]) * shexp.
void orc_moe_shared_add(const float* moe, const float* shexp, const float* gate, float* dst,
                        uint32_t rows, uint32_t n) {
  for (uint32_t r = 0; r < rows; ++r) {
    const float g = sigmoidf(gate[r]);
    for (uint32_t c = 0; c < n; ++c) dst[(size_t)r * n + c] = moe[(size_t)r * n + c] + g * shexp[(size_t)r * n + c];
  }
}

// Op::RmsNorm (lib.rs:1046-1069): ss = (Σ→ x²)/dim ; s = 1/sqrt(ss+eps) ; o = x*s*w.
void orc_rmsnorm(const float* x, const float* w, float* dst, uint32_t rows, uint32_t dim, float eps) {
  for (uint32_t r = 0; r < rows; ++r) {
    const float* xr = x + (size_t)r * dim;
    float ss = 0.0f;
    for (uint32_t i = 0; i < dim; ++i) ss = ss + xr[i] * xr[i];
    ss = ss / (float)dim;
    const float s = 1.0f / std::sqrt(ss + eps);
    for (uint32_t i = 0; i < dim; ++i) dst[(size_t)r * dim + i] = xr[i] * s * w[i];
  }
}

// Op::Add (lib.rs:3055-3070).
void orc_add(const float* a, const float* b, float* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = a[i] + b[i];
}

// The whole qwen35moe / DeepSeek FFN sub-layer as the graph builder emits it
// (crates/infr-llama/src/seam/runner.rs:7999-8176): MoeFfn, then the shared expert as
// Linear(gate) / Linear(up) / GatedAct / Linear(down) and MoeSharedExpertAdd (gated) or Add.
//   sh_gate_inp == null → plain sum (DeepSeek, llama4); else sigmoid-gated (qwen35moe).
int orc_moe_layer(const orc_moe_desc* d, const uint8_t* sh_gate, const uint8_t* sh_up,
                  const uint8_t* sh_down, const float* sh_gate_inp, uint32_t sh_ff, float* dst) {
  const size_t R = d->rows, ne = d->ne;
  std::vector<float> moe(R * ne);
  orc_moe_desc dd = *d;
  dd.dst = moe.data();
  int rc = orc_moe_ffn(&dd);
  if (rc) return rc;
  if (!sh_gate) {
    std::memcpy(dst, moe.data(), R * ne * sizeof(float));
    return 0;
  }
  std::vector<float> g(R * sh_ff), u(R * sh_ff), a(R * sh_ff), ds(R * ne);
  if ((rc = orc_linear(d->gate_dtype, sh_gate, d->x, d->rows, d->ne, sh_ff, g.data(), d->threads))) return rc;
  if ((rc = orc_linear(d->up_dtype, sh_up, d->x, d->rows, d->ne, sh_ff, u.data(), d->threads))) return rc;
  // Op::GatedAct with the model's activation, no clamp on the shared expert here
  for (size_t i = 0; i < R * sh_ff; ++i) a[i] = gated_act_value(d->act, 0.0f, g[i], u[i]);
  if ((rc = orc_linear(d->down_dtype, sh_down, a.data(), d->rows, sh_ff, d->ne, ds.data(), d->threads))) return rc;
  if (sh_gate_inp) {
    std::vector<float> gl(R);
    orc_linear(DT_F32, (const uint8_t*)sh_gate_inp, d->x, d->rows, d->ne, 1, gl.data(), 1);
    orc_moe_shared_add(moe.data(), ds.data(), gl.data(), dst, d->rows, d->ne);
  } else {
    orc_add(moe.data(), ds.data(), dst, R * ne);
  }
  return 0;
}

}  // extern "C"
