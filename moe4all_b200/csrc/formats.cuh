// One view of the GGUF block formats the expert banks may hold beyond the Q4_K / Q6_K pair the tuned
// kernels are written for: 16 consecutive weights of a row as sixteen unsigned 8-bit codes and the
// affine map of their scale group,
//
//     w = A * (code - off) + B .
//
// It is the factored form of the reference's host decoder (crates/infr-gguf/src/dequant.rs:119-400:
// `codes`, per-16 `(sc, m)`, per-block `(d, dmin)`; values `(d*sc)*code + (dmin*m)`, :35-51):
//
//   Q4_K  144 B / 256   code = 4-bit nibble,            A = d*sc6,  B = -dmin*m6,  off = 0    (:315-335)
//   Q5_K  176 B / 256   code = nibble | high bit << 4,  A = d*sc6,  B = -dmin*m6,  off = 0    (:337-362)
//   Q6_K  210 B / 256   code = 6 bits (ql | qh << 4),   A = d*sc8,  B = 0,         off = 32   (:365-400)
//   Q8_0   34 B / 32    code = q + 128,                 A = d,      B = 0,         off = 128  (:214-223)
//   Q4_0   18 B / 32    code = nibble,                  A = d,      B = 0,         off = 8    (:142-158)
//   Q4_1   20 B / 32    code = nibble,                  A = d,      B = m,         off = 0    (:159-175)
//   Q5_0   22 B / 32    code = nibble | high bit << 4,  A = d,      B = 0,         off = 16   (:176-194)
//   Q5_1   24 B / 32    code = nibble | high bit << 4,  A = d,      B = m,         off = 0    (:195-212)
//   Q2_K   84 B / 256   code = 2 bits,                  A = d*sc4,  B = -dmin*m4,  off = 0    (:224-252; per 16)
//   Q3_K  110 B / 256   code = 2 bits | high bit << 2,  A = d*(sc6 - 32), B = 0,   off = 4    (:253-314; per 16)
//
// and of its codebook decoder for the two 4-bit non-linear formats (dequant.rs:443-445, 499-553):
//
//   IQ4_NL  18 B / 32   code = kvalues[nibble] + 128,   A = d,            B = 0,   off = 128
//   IQ4_XS 136 B / 256  code = kvalues[nibble] + 128,   A = d * (ls6 - 32), B = 0, off = 128
//   MXFP4   17 B / 32   code = e2m1x2[nibble] + 128,    A = 2^(e - 128),  B = 0,   off = 128  (:409-421, 1029-1046)
//   NVFP4   36 B / 64   code = e2m1x2[nibble] + 128,    A = ue4m3(scale of the 16) / 2, B = 0, off = 128  (:423-439, 1053-1073)
//
// and the ternary-plus-one 2-bit form (:1007-1022):
//
//   Q2_0    18 B / 64   code = 2 bits,                  A = d,      B = 0,         off = 1
//
// and the grid codebook formats (dequant.rs:477-488, 605-770): a group of 8 (IQ2) or 4 (IQ3) weights is one entry of
// a grid table - eight or four small positive bytes - with a sign bit per weight, times the scale of its 16 or 32
//
//   IQ2_XS   74 B / 256  code = 128 +- grid2xs[9 bits][k],  A = d (0.5 + ls4) / 4,  signs = 7-bit index with its parity on top
//   IQ2_S    82 B / 256  code = 128 +- grid2s[10 bits][k],  A = d (0.5 + ls4) / 4,  a sign byte per 8 weights
//   IQ3_XXS  98 B / 256  code = 128 +- grid3xxs[8 bits][k], A = d (0.5 + ls4) / 2,  signs as IQ2_XS, scale per 32
//   IQ3_S   110 B / 256  code = 128 +- grid3s[9 bits][k],   A = d (1 + 2 ls4),      a sign byte per 8 weights
//
// (B = 0, off = 128).  The grid tables are constants of the formats that this library does not carry: the host
// hands them over once (infr_cuda_set_codebook) and the kernels read them through pointers in constant memory.
//
// The generic small-m kernels (anyfmt_ffn.cu) feed the codes to integer dot products against the
// fixed-point activations; the generic grouped GEMM (grouped_ffn.cu) turns them into f16 operands.
#pragma once
#include "common.cuh"

namespace infr {

constexpr uint32_t Q5K_BLOCK_BYTES = 176;  // 256 weights: f16 d, f16 dmin, 12 B scales, 32 B high bits, 128 B nibbles
constexpr uint32_t Q80_BLOCK_BYTES = 34;   // 32 weights: f16 d, 32 int8
constexpr uint32_t IQ4NL_BLOCK_BYTES = 18;   // 32 weights: f16 d, 16 B nibbles (elements j and j + 16 share a byte)
constexpr uint32_t IQ4XS_BLOCK_BYTES = 136;  // 256 weights: f16 d, u16 scale high bits, 4 B scale low nibbles, 128 B nibbles

// The formats an expert bank may have.
inline bool bank_dtype_ok(int32_t dt) {
  switch (dt) {
    case INFR_CUDA_DT_Q4_0: case INFR_CUDA_DT_Q4_1: case INFR_CUDA_DT_Q5_0: case INFR_CUDA_DT_Q5_1: case INFR_CUDA_DT_Q8_0:
    case INFR_CUDA_DT_Q2K: case INFR_CUDA_DT_Q3K: case INFR_CUDA_DT_Q4K: case INFR_CUDA_DT_Q5K: case INFR_CUDA_DT_Q6K:
    case INFR_CUDA_DT_IQ4NL: case INFR_CUDA_DT_IQ4XS: case INFR_CUDA_DT_MXFP4:
    case INFR_CUDA_DT_NVFP4: case INFR_CUDA_DT_Q2_0:
    case INFR_CUDA_DT_IQ2XS: case INFR_CUDA_DT_IQ2S: case INFR_CUDA_DT_IQ3XXS: case INFR_CUDA_DT_IQ3S:
      return true;
    default:
      return false;
  }
}
// Grid codebook formats: the slot of the format's table, or -1; the table's size (entries x bytes per entry).
constexpr int N_CODEBOOKS = 4;
inline int codebook_slot(int32_t dt) {
  return dt == INFR_CUDA_DT_IQ2XS ? 0 : dt == INFR_CUDA_DT_IQ3XXS ? 1 : dt == INFR_CUDA_DT_IQ3S ? 2 : dt == INFR_CUDA_DT_IQ2S ? 3 : -1;
}
inline size_t codebook_bytes(int slot) { return slot == 0 ? 512 * 8 : slot == 1 ? 256 * 4 : slot == 2 ? 512 * 4 : slot == 3 ? 1024 * 8 : 0; }
// The combination the tuned kernels (per-pair, expert-major, tcgen05) are written for.
inline bool bank_dtypes_tuned(int32_t gate, int32_t up, int32_t down) {
  return gate == INFR_CUDA_DT_Q4K && up == INFR_CUDA_DT_Q4K && (down == INFR_CUDA_DT_Q6K || down == INFR_CUDA_DT_Q4K);
}

#ifdef __CUDACC__

// Device addresses of the grid tables, one copy per translation unit that unpacks weights (each publishes its
// own through publish_codebooks): slots as codebook_slot().
static __constant__ const unsigned char* c_codebook[N_CODEBOOKS];
static inline cudaError_t publish_codebooks(const unsigned char* const* tables) {
  return cudaMemcpyToSymbol(c_codebook, tables, sizeof(const unsigned char*) * N_CODEBOOKS);
}

// The sign byte of a 7-bit sign index: the index with its parity as the eighth bit (an even number of negations).
__device__ __forceinline__ uint32_t iq_signs7(uint32_t i) { return i | ((uint32_t)(__popc(i) & 1) << 7); }
// Four grid bytes v (each < 128) and four sign bits (bit j set: weight j is negative) -> the bytes 128 +- v.
__device__ __forceinline__ uint32_t iq_signed_codes(uint32_t v, uint32_t s4) {
  const uint32_t m = (((s4 & 0xFu) * 0x00204081u) & 0x01010101u) * 0xFFu;  // 0xFF in the bytes to negate
  return 0x80808080u + (v & ~m) - (v & m);
}

// A load through the read-only path when the blocks sit in global memory (G), a plain load when a
// kernel has staged them in shared memory.
template <bool G, typename T>
__device__ __forceinline__ T fmt_ld(const void* p) {
  if (G) return __ldg(reinterpret_cast<const T*>(p));
  return *reinterpret_cast<const T*>(p);
}

// Four bytes at a 2-byte-aligned address: one word load when the address is word aligned, else two
// 16-bit loads, so nothing outside the four bytes is touched.
template <bool G>
__device__ __forceinline__ uint32_t ld_u32_a2(const uint8_t* p) {
  if ((reinterpret_cast<uintptr_t>(p) & 3u) == 0) return fmt_ld<G, uint32_t>(p);
  const uint32_t lo = fmt_ld<G, unsigned short>(p);
  const uint32_t hi = fmt_ld<G, unsigned short>(p + 2);
  return lo | (hi << 16);
}

// Four 4-bit indices (one per byte of n) -> the bytes table[index] of a 16-entry byte table given as four
// words: two byte permutes over the table's halves (index bits 0-2 as the selector), the half chosen by
// index bit 3.
__device__ __forceinline__ uint32_t lut16_bytes(uint32_t n, uint32_t t0, uint32_t t1, uint32_t t2, uint32_t t3) {
  const uint32_t n7 = n & 0x07070707u;
  const uint32_t t = n7 | (n7 >> 4);                                         // nibbles: b0 b1 b1 b2 b2 b3 b3 0
  const uint32_t sel = (t & 0xFFu) | ((t >> 4) & 0xF00u) | ((t >> 8) & 0xF000u);  // b0 b1 b2 b3
  const uint32_t lo = __byte_perm(t0, t1, sel), hi = __byte_perm(t2, t3, sel);
  const uint32_t m = ((n >> 3) & 0x01010101u) * 0xFFu;                       // 0xFF where the index is 8-15
  return (lo & ~m) | (hi & m);
}
// kvalues_iq4nl + 128: {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113}
__device__ __forceinline__ uint32_t iq4_codes(uint32_t n) { return lut16_bytes(n, 0x3F2D1801u, 0x766A5D4Fu, 0xA6998D81u, 0xF1D9C5B5u); }
// kvalues_mxfp4 (E2M1 values x 2) + 128: {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12}
__device__ __forceinline__ uint32_t mxfp4_codes(uint32_t n) { return lut16_bytes(n, 0x83828180u, 0x8C888684u, 0x7D7E7F80u, 0x74787A7Cu); }

// Four bytes at any address (MXFP4 blocks are 17 bytes).
template <bool G>
__device__ __forceinline__ uint32_t ld_u32_a1(const uint8_t* p) {
  if ((reinterpret_cast<uintptr_t>(p) & 3u) == 0) return fmt_ld<G, uint32_t>(p);
  return (uint32_t)fmt_ld<G, uint8_t>(p) | ((uint32_t)fmt_ld<G, uint8_t>(p + 1) << 8) | ((uint32_t)fmt_ld<G, uint8_t>(p + 2) << 16) |
         ((uint32_t)fmt_ld<G, uint8_t>(p + 3) << 24);
}

// Codes and affine map of weights 16h .. 16h+15 of the row starting at `row` (G: in global memory;
// else a copy in shared memory with the same alignment modulo 16).
template <bool G = true>
__device__ __forceinline__ void fmt_codes16(int dt, const uint8_t* __restrict__ row, int h, uint32_t (&c)[4], float& A, float& B,
                                            int& off) {
  if (dt == INFR_CUDA_DT_Q4K || dt == INFR_CUDA_DT_Q5K) {
    const bool q5 = dt == INFR_CUDA_DT_Q5K;
    const uint8_t* blk = row + (size_t)(h >> 4) * (q5 ? Q5K_BLOCK_BYTES : Q4K_BLOCK_BYTES);
    const int e = (h & 15) * 16, j = e >> 6, sub = (e >> 5) & 1, l0 = e & 31;
    const uint4 hdr = fmt_ld<G, uint4>(blk);
    const uint4 q = fmt_ld<G, uint4>(blk + (q5 ? 48 : 16) + 32 * j + l0);
    const int sh = 4 * sub;
    c[0] = (q.x >> sh) & 0x0F0F0F0Fu;
    c[1] = (q.y >> sh) & 0x0F0F0F0Fu;
    c[2] = (q.z >> sh) & 0x0F0F0F0Fu;
    c[3] = (q.w >> sh) & 0x0F0F0F0Fu;
    if (q5) {
      // bit 2j + sub of qh[l] is the fifth code bit of element 64j + 32 sub + l
      const uint4 qh = fmt_ld<G, uint4>(blk + 16 + l0);
      const int sb = 2 * j + sub;
      c[0] |= ((qh.x >> sb) & 0x01010101u) << 4;
      c[1] |= ((qh.y >> sb) & 0x01010101u) << 4;
      c[2] |= ((qh.z >> sb) & 0x01010101u) << 4;
      c[3] |= ((qh.w >> sb) & 0x01010101u) << 4;
    }
    uint32_t scp, mp;
    q4k_scale_min_pair(hdr.y, hdr.z, hdr.w, j, scp, mp);
    A = f16_bits_to_f32(hdr.x) * (float)((scp >> (8 * sub)) & 0xFFu);
    B = -(f16_bits_to_f32(hdr.x >> 16) * (float)((mp >> (8 * sub)) & 0xFFu));
    off = 0;
  } else if (dt == INFR_CUDA_DT_Q6K) {
    // element 128 hh + 32 qd + l: low nibble source ql[64 hh + 32 (qd & 1) + l] (high nibble for qd >= 2),
    // bits 2 qd .. 2 qd + 1 of qh[32 hh + l]; one int8 scale per 16 elements.  Blocks are 2-byte aligned.
    const uint8_t* blk = row + (size_t)(h >> 4) * Q6K_BLOCK_BYTES;
    const int e = (h & 15) * 16, hh = e >> 7, qd = (e >> 5) & 3, l0 = e & 31;
    const uint8_t* ql = blk + 64 * hh + 32 * (qd & 1) + l0;
    const uint8_t* qh = blk + 128 + 32 * hh + l0;
    const int nsh = 4 * (qd >> 1), hsh = 2 * qd;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t lo = ld_u32_a2<G>(ql + 4 * i), hi = ld_u32_a2<G>(qh + 4 * i);
      c[i] = ((lo >> nsh) & 0x0F0F0F0Fu) | (((hi >> hsh) & 0x03030303u) << 4);
    }
    const float d = f16_bits_to_f32(fmt_ld<G, unsigned short>(blk + 208));
    A = d * (float)(int)(signed char)fmt_ld<G, uint8_t>(blk + 192 + 8 * hh + 2 * qd + (l0 >> 4));
    B = 0.f;
    off = 32;
  } else if (dt == INFR_CUDA_DT_Q4_0 || dt == INFR_CUDA_DT_Q4_1 || dt == INFR_CUDA_DT_Q5_0 || dt == INFR_CUDA_DT_Q5_1) {
    // 32-weight blocks: f16 d (and f16 m for the _1 forms), for the 5-bit forms 32 high bits, then 16 code
    // bytes whose low nibbles are elements 0-15 and high nibbles elements 16-31
    const bool has_m = dt == INFR_CUDA_DT_Q4_1 || dt == INFR_CUDA_DT_Q5_1, five = dt == INFR_CUDA_DT_Q5_0 || dt == INFR_CUDA_DT_Q5_1;
    const int hdr = has_m ? 4 : 2, bb = 16 + hdr + (five ? 4 : 0), half = h & 1;
    const uint8_t* blk = row + (size_t)(h >> 1) * bb;
    const uint8_t* qs = blk + hdr + (five ? 4 : 0);
    const uint32_t qh = five ? (ld_u32_a2<G>(blk + hdr) >> (16 * half)) : 0u;  // bit j: element 16 half + j
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      c[i] = (ld_u32_a2<G>(qs + 4 * i) >> (4 * half)) & 0x0F0F0F0Fu;
      if (five) {
        const uint32_t b4 = (qh >> (4 * i)) & 0xFu;  // the high bits of elements 4 i .. 4 i + 3
        c[i] |= ((b4 & 1u) << 4) | ((b4 & 2u) << 11) | ((b4 & 4u) << 18) | ((b4 & 8u) << 25);
      }
    }
    A = f16_bits_to_f32(fmt_ld<G, unsigned short>(blk));
    B = has_m ? f16_bits_to_f32(fmt_ld<G, unsigned short>(blk + 2)) : 0.f;
    off = has_m ? 0 : (five ? 16 : 8);
  } else if (dt == INFR_CUDA_DT_Q2K || dt == INFR_CUDA_DT_Q3K) {
    // 16 elements = group (n, j, half) of the block: 16 code bytes at 32 n + 16 half, two bits each at bit 2 j;
    // Q3_K adds bit 4 n + j of hmask[16 half + l]; one scale (and min) per 16 elements
    const bool q3 = dt == INFR_CUDA_DT_Q3K;
    const uint8_t* blk = row + (size_t)(h >> 4) * (q3 ? 110 : 84);
    const int h16 = h & 15, n = h16 >> 3, j = (h16 >> 1) & 3, half = h16 & 1;
    const uint8_t* qs = blk + (q3 ? 32 : 16) + 32 * n + 16 * half;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      c[i] = (ld_u32_a2<G>(qs + 4 * i) >> (2 * j)) & 0x03030303u;
      if (q3) c[i] |= ((ld_u32_a2<G>(blk + 16 * half + 4 * i) >> (4 * n + j)) & 0x01010101u) << 2;
    }
    if (q3) {
      // sixteen 6-bit scales in 12 bytes: low nibbles of bytes 0-7 (scales 0-7: low, 8-15: high nibble),
      // two more bits each in bytes 8-11
      const uint32_t a = ld_u32_a2<G>(blk + 96 + 4 * ((h16 >> 2) & 1)), tmp = ld_u32_a2<G>(blk + 104);
      const uint32_t lo4 = (h16 < 8 ? a : (a >> 4)) & 0x0F0F0F0Fu;
      const uint32_t hi2 = ((tmp >> (2 * (h16 >> 2))) & 0x03030303u) << 4;
      const int sc = (int)(((lo4 | hi2) >> (8 * (h16 & 3))) & 0xFFu) - 32;
      A = f16_bits_to_f32(fmt_ld<G, unsigned short>(blk + 108)) * (float)sc;
      B = 0.f;
      off = 4;
    } else {
      const uint32_t sc = fmt_ld<G, uint8_t>(blk + h16);
      A = f16_bits_to_f32(fmt_ld<G, unsigned short>(blk + 80)) * (float)(sc & 0xFu);
      B = -(f16_bits_to_f32(fmt_ld<G, unsigned short>(blk + 82)) * (float)(sc >> 4));
      off = 0;
    }
  } else if (dt == INFR_CUDA_DT_IQ4NL) {
    // elements 0-15 of a block are the low nibbles of its 16 code bytes, elements 16-31 the high nibbles
    const uint8_t* blk = row + (size_t)(h >> 1) * IQ4NL_BLOCK_BYTES;
    const int sh = 4 * (h & 1);
#pragma unroll
    for (int i = 0; i < 4; ++i) c[i] = iq4_codes((ld_u32_a2<G>(blk + 2 + 4 * i) >> sh) & 0x0F0F0F0Fu);
    A = f16_bits_to_f32(fmt_ld<G, unsigned short>(blk));
    B = 0.f;
    off = 128;
  } else if (dt == INFR_CUDA_DT_MXFP4) {
    // one E8M0 exponent byte (the scale is 2^(e - 128): `e8m0_to_fp32_half`), 16 code bytes as in IQ4_NL
    const uint8_t* blk = row + (size_t)(h >> 1) * 17;
    const int sh = 4 * (h & 1);
#pragma unroll
    for (int i = 0; i < 4; ++i) c[i] = mxfp4_codes((ld_u32_a1<G>(blk + 1 + 4 * i) >> sh) & 0x0F0F0F0Fu);
    const uint32_t e = fmt_ld<G, uint8_t>(blk);
    A = __uint_as_float(e < 2 ? (0x00200000u << e) : ((e - 1) << 23));
    B = 0.f;
    off = 128;
  } else if (dt == INFR_CUDA_DT_NVFP4) {
    // 64-weight blocks (4-byte aligned): four UE4M3 scale bytes, one per 16 weights, then 8 code bytes per 16
    // weights whose low nibbles are weights 0-7 and high nibbles weights 8-15
    const uint8_t* blk = row + (size_t)(h >> 2) * 36;
    const int s = h & 3;
    const uint32_t a = fmt_ld<G, uint32_t>(blk + 4 + 8 * s), b = fmt_ld<G, uint32_t>(blk + 8 + 8 * s);
    c[0] = mxfp4_codes(a & 0x0F0F0F0Fu);
    c[1] = mxfp4_codes(b & 0x0F0F0F0Fu);
    c[2] = mxfp4_codes((a >> 4) & 0x0F0F0F0Fu);
    c[3] = mxfp4_codes((b >> 4) & 0x0F0F0F0Fu);
    // UE4M3 (bias 7, 3 mantissa bits; bit 7 unused), halved: man * 2^-10 for exponent 0, else (8 + man) * 2^(exp - 11);
    // bytes 0x00 and 0x7F decode to 0
    const uint32_t x = (fmt_ld<G, uint32_t>(blk) >> (8 * s)) & 0xFFu, ex = (x >> 3) & 0xFu, man = x & 7u;
    A = (x == 0u || x == 0x7Fu) ? 0.f : (ex == 0u ? (float)man * 0x1p-10f : (float)(8u + man) * __uint_as_float((ex + 116u) << 23));
    B = 0.f;
    off = 128;
  } else if (dt == INFR_CUDA_DT_Q2_0) {
    // 64-weight blocks (2-byte aligned): f16 d, 16 code bytes of four 2-bit fields, weight j in byte j / 4 at bit 2 (j % 4)
    const uint8_t* blk = row + (size_t)(h >> 2) * 18;
    const uint32_t w = ld_u32_a2<G>(blk + 2 + 4 * (h & 3));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t v = (w >> (8 * i)) & 0xFFu;
      c[i] = (v & 3u) | ((v & 0x0Cu) << 6) | ((v & 0x30u) << 12) | ((v & 0xC0u) << 18);
    }
    A = f16_bits_to_f32(fmt_ld<G, unsigned short>(blk));
    B = 0.f;
    off = 1;
  } else if (dt == INFR_CUDA_DT_IQ2XS || dt == INFR_CUDA_DT_IQ2S) {
    // 16 weights = two groups of 8 (l = 2 half, 2 half + 1) of the 32-weight group ib32; a 4-bit scale per 16
    const bool s2 = dt == INFR_CUDA_DT_IQ2S;
    const uint8_t* blk = row + (size_t)(h >> 4) * (s2 ? 82 : 74);
    const int ib32 = (h & 15) >> 1, half = h & 1;
    const uint32_t sc = fmt_ld<G, uint8_t>(blk + (s2 ? 74 : 66) + ib32);
    A = f16_bits_to_f32(fmt_ld<G, unsigned short>(blk)) * (0.5f + (float)(half ? sc >> 4 : sc & 15u)) * 0.25f;
    const uint32_t qh = s2 ? fmt_ld<G, uint8_t>(blk + 66 + ib32) : 0u;
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int l = 2 * half + s;
      uint32_t idx, sg;
      if (s2) {
        idx = fmt_ld<G, uint8_t>(blk + 2 + 4 * ib32 + l) | ((qh << (8 - 2 * l)) & 0x300u);
        sg = fmt_ld<G, uint8_t>(blk + 34 + 4 * ib32 + l);
      } else {
        const uint32_t q16 = fmt_ld<G, unsigned short>(blk + 2 + 2 * (4 * ib32 + l));
        idx = q16 & 511u;
        sg = iq_signs7(q16 >> 9);
      }
      const uint2 g = __ldg(reinterpret_cast<const uint2*>(c_codebook[s2 ? 3 : 0]) + idx);
      c[2 * s] = iq_signed_codes(g.x, sg);
      c[2 * s + 1] = iq_signed_codes(g.y, sg >> 4);
    }
    B = 0.f;
    off = 128;
  } else if (dt == INFR_CUDA_DT_IQ3XXS || dt == INFR_CUDA_DT_IQ3S) {
    // 16 weights = two groups of 8, each two grid entries of 4; IQ3_XXS: one word per 32 weights holds four 7-bit
    // sign indices and the scale; IQ3_S: a sign byte per 8 weights, a ninth index bit in qh, a 4-bit scale per 32
    const bool s3 = dt == INFR_CUDA_DT_IQ3S;
    const uint8_t* blk = row + (size_t)(h >> 4) * (s3 ? 110 : 98);
    const int ib32 = (h & 15) >> 1, half = h & 1;
    const float d = f16_bits_to_f32(fmt_ld<G, unsigned short>(blk));
    uint32_t aux = 0, qh = 0;
    if (s3) {
      const uint32_t sb = fmt_ld<G, uint8_t>(blk + 106 + (ib32 >> 1));
      A = d * (1.0f + 2.0f * (float)((ib32 & 1) ? sb >> 4 : sb & 15u));
      qh = fmt_ld<G, uint8_t>(blk + 66 + ib32);
    } else {
      aux = ld_u32_a2<G>(blk + 66 + 4 * ib32);
      A = d * (0.5f + (float)(aux >> 28)) * 0.5f;
    }
    const uint32_t* grid = reinterpret_cast<const uint32_t*>(c_codebook[s3 ? 2 : 1]);
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int l = 2 * half + s;
      uint32_t i1 = fmt_ld<G, uint8_t>(blk + 2 + 8 * ib32 + 2 * l), i2 = fmt_ld<G, uint8_t>(blk + 3 + 8 * ib32 + 2 * l), sg;
      if (s3) {
        i1 |= (qh << (8 - 2 * l)) & 256u;
        i2 |= (qh << (7 - 2 * l)) & 256u;
        sg = fmt_ld<G, uint8_t>(blk + 74 + 4 * ib32 + l);
      } else {
        sg = iq_signs7((aux >> (7 * l)) & 127u);
      }
      c[2 * s] = iq_signed_codes(__ldg(grid + i1), sg);
      c[2 * s + 1] = iq_signed_codes(__ldg(grid + i2), sg >> 4);
    }
    B = 0.f;
    off = 128;
  } else if (dt == INFR_CUDA_DT_IQ4XS) {
    // sub-block ib (32 elements) = 16 code bytes at 8 + 16 ib, low nibbles first; its 6-bit scale: low
    // four bits in scales_l (a nibble per sub-block), high two in scales_h
    const uint8_t* blk = row + (size_t)(h >> 4) * IQ4XS_BLOCK_BYTES;  // 8-byte aligned
    const int e = (h & 15) * 16, ib = e >> 5, sh = 4 * ((e >> 4) & 1);
#pragma unroll
    for (int i = 0; i < 4; ++i) c[i] = iq4_codes((fmt_ld<G, uint32_t>(blk + 8 + 16 * ib + 4 * i) >> sh) & 0x0F0F0F0Fu);
    const uint32_t hdr = fmt_ld<G, uint32_t>(blk), sl = fmt_ld<G, uint32_t>(blk + 4);  // d | scales_h << 16, scales_l
    const int ls = (int)(((sl >> (4 * ib)) & 0xFu) | ((((hdr >> 16) >> (2 * ib)) & 3u) << 4));
    A = f16_bits_to_f32(hdr) * (float)(ls - 32);
    B = 0.f;
    off = 128;
  } else {  // Q8_0
    const uint8_t* blk = row + (size_t)(h >> 1) * Q80_BLOCK_BYTES;
    const uint8_t* q = blk + 2 + 16 * (h & 1);
#pragma unroll
    for (int i = 0; i < 4; ++i) c[i] = ld_u32_a2<G>(q + 4 * i) ^ 0x80808080u;
    A = f16_bits_to_f32(fmt_ld<G, unsigned short>(blk));
    B = 0.f;
    off = 128;
  }
}

#endif  // __CUDACC__

}  // namespace infr
