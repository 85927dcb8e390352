// Grouped expert GEMMs on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory).
//
// Same contract as the legacy-MMA kernels of grouped_ffn.cu (reference: CPU stages B-D
// crates/infr-cpu/src/lib.rs:4051-4266; Vulkan native_gemm_mmq_q4k/q6k.comp): per expert segment
//   act = silu(Wg x) * (Wu x)      (k_umma_gateup, Q4_K weights)
//   y   = Wd act                   (k_umma_down,   Q6_K weights)
// with the weights as the M operand (128 output features per CTA) and up to 256 token rows as the
// N operand, so every weight block is unpacked once per 256 tokens.
//
// Warp roles (10 warps): warps 0-7 are producers - each thread owns one weight row of the tile and
// unpacks its 64 weights of the K step to f16 straight into the 128-byte-swizzled operand tile;
// warp 8 issues the MMAs (one thread) and releases pipeline stages with tcgen05.commit; warp 9
// fetches the token operand: the gather kernel (and the gate/up epilogue) store token rows per
// (tile, K step) as 128-byte lines already in swizzled order, so one bulk copy brings a step's
// whole operand and runs several steps ahead of the MMAs.  After the K loop the producers drain
// the accumulators with tcgen05.ld and write the result.  Weight and token stages are separate
// rings handed over through mbarriers; every wait is bounded.
#include <cuda.h>

#include <type_traits>

#include "kernels.cuh"
#include "umma.cuh"

namespace infr {
namespace {

constexpr int UM = 128;           // weight rows per role and CTA
constexpr int UN = 256;           // max token rows per CTA
constexpr int UK = 64;            // K elements per stage
constexpr int U_PRODUCERS = 256;  // producer threads
constexpr int U_THREADS = U_PRODUCERS + 64;  // + MMA warp + token-copy warp
constexpr float W_PRESCALE = 256.0f;
constexpr float W_POSTSCALE = 1.0f / 256.0f;
constexpr uint32_t A_TILE_BYTES = UM * 128;  // 16 KB
constexpr uint32_t B_TILE_BYTES = UN * 128;  // 32 KB

__device__ __forceinline__ int kperm(int k) {
  const int r = k & 3;
  return (k & ~3) | (r == 1 ? 2 : (r == 2 ? 1 : r));
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

__device__ __forceinline__ void q4_word_to_h2(uint32_t w, __half2 s, __half2 m, uint32_t& out02, uint32_t& out13) {
  const __half2 k1024 = __float2half2_rn(1024.f);
  const __half2 a = __hsub2(u32_as_h2((w & 0x000F000Fu) | 0x64006400u), k1024);
  const __half2 b = __hsub2(u32_as_h2(((w >> 8) & 0x000F000Fu) | 0x64006400u), k1024);
  out02 = h2_as_u32(__hfma2(a, s, m));
  out13 = h2_as_u32(__hfma2(b, s, m));
}

__device__ __forceinline__ void q6_word_to_h2(uint32_t c, __half2 s, uint32_t& out02, uint32_t& out13) {
  const __half2 k1056 = __float2half2_rn(1056.f);
  const __half2 a = __hsub2(u32_as_h2((c & 0x00FF00FFu) | 0x64006400u), k1056);
  const __half2 b = __hsub2(u32_as_h2(((c >> 8) & 0x00FF00FFu) | 0x64006400u), k1056);
  out02 = h2_as_u32(__hmul2(a, s));
  out13 = h2_as_u32(__hmul2(b, s));
}

// Byte offset of token row n's K-step line inside a tile's block of the token arrays:
// [tile][K step][256 rows][128 bytes].
__device__ __forceinline__ size_t tile_step_offset(int tile, int k_steps, int step) {
  return ((size_t)tile * k_steps + step) * (size_t)(UN * 128);
}

// One tiled copy: a box of the 2-D tensor behind `tm` at (x = bytes inside the row, y = row) into
// shared memory, completion counted in bytes on `bar`.  x * element size must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tm, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tm)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

struct PipeBars {
  uint64_t full_a[4], empty_a[4];  // weight-tile ring
  uint64_t full_b[4], empty_b[4];  // token-tile ring
  uint64_t done;
};

template <int SA, int SB>
__device__ __forceinline__ void init_bars(PipeBars& bars) {
  for (int s = 0; s < SA; ++s) {
    mbar_init(&bars.full_a[s], U_PRODUCERS / 32);
    mbar_init(&bars.empty_a[s], 1);
  }
  for (int s = 0; s < SB; ++s) {
    mbar_init(&bars.full_b[s], 1);
    mbar_init(&bars.empty_b[s], 1);
  }
  mbar_init(&bars.done, 1);
  mbar_fence_init();
}

// Shared pipeline skeleton.  Producers: `unpack(a_stage, step, step % 4)` writes the weight
// tile(s); token warp: one bulk copy of `b_bytes` from `b_src + step * b_step_stride`; MMA thread:
// `issue(a_stage, b_stage, step)`.
template <int SA, int SB, typename Unpack, typename Issue>
__device__ __forceinline__ bool run_pipeline(PipeBars& bars, unsigned char* a_stages, uint32_t a_stage_bytes,
                                             unsigned char* b_stages, const unsigned char* b_src, size_t b_step_stride,
                                             uint32_t b_bytes, int n_steps, Unpack unpack, Issue issue,
                                             unsigned long long* tr) {
  const int tid = threadIdx.x;
  bool ok = true;
  if (tid < U_PRODUCERS) {
    // `jc` carries step % 4 as a compile-time constant (n_steps is a multiple of four): the
    // producers index their register-resident prefetch buffers with it
    auto body = [&](int step, auto jc) {
      if (!ok) return;
      const int s = step % SA, use = step / SA;
      if ((step & 3) == 0 && step < 32) trace_stamp(tr, 64 + step);
      // a stage is free again when the MMAs that last read it have completed
      if (!mbar_wait_bounded(&bars.empty_a[s], (use & 1) ^ 1)) { ok = false; return; }
      if ((step & 3) == 0 && step < 32) trace_stamp(tr, 65 + step);
      if (!unpack(a_stages + (size_t)s * a_stage_bytes, step, jc)) { ok = false; return; }
      if ((step & 3) == 0 && step < 32) trace_stamp(tr, 66 + step);
      umma::fence_proxy_async();
      __syncwarp();
      if ((tid & 31) == 0) mbar_arrive(&bars.full_a[s]);  // one arrival per producer warp
    };
    for (int base = 0; base < n_steps && ok; base += 4) {
      body(base, std::integral_constant<int, 0>{});
      body(base + 1, std::integral_constant<int, 1>{});
      body(base + 2, std::integral_constant<int, 2>{});
      body(base + 3, std::integral_constant<int, 3>{});
    }
  } else if (tid == U_PRODUCERS) {
    for (int step = 0; step < n_steps && ok; ++step) {
      const int sa = step % SA, sb = step % SB;
      if (!mbar_wait_bounded(&bars.full_a[sa], (step / SA) & 1) || !mbar_wait_bounded(&bars.full_b[sb], (step / SB) & 1)) {
        ok = false;
        break;
      }
      umma::fence_after_sync();
      if (tr != nullptr && (step & 3) == 0 && step < 32) { tr[2 * (100 + step / 2)] = 0; tr[2 * (100 + step / 2) + 1] = (unsigned long long)clock64(); }
      issue(a_stages + (size_t)sa * a_stage_bytes, b_stages + (size_t)sb * B_TILE_BYTES, step);
      umma::commit(&bars.empty_a[sa]);
      umma::commit(&bars.empty_b[sb]);
      if (tr != nullptr && (step & 3) == 0 && step < 32) { tr[2 * (101 + step / 2)] = 0; tr[2 * (101 + step / 2) + 1] = (unsigned long long)clock64(); }
    }
    umma::commit(&bars.done);
  } else if (tid == U_PRODUCERS + 32) {
    for (int step = 0; step < n_steps && ok; ++step) {
      const int sb = step % SB;
      if (!mbar_wait_bounded(&bars.empty_b[sb], ((step / SB) & 1) ^ 1)) { ok = false; break; }
      mbar_arrive_expect_tx(&bars.full_b[sb], b_bytes);
      bulk_g2s(b_stages + (size_t)sb * B_TILE_BYTES, b_src + (size_t)step * b_step_stride, b_bytes, &bars.full_b[sb]);
    }
  }
  return ok;
}

// ---- gate/up + SwiGLU ---------------------------------------------------------------------------

constexpr int GU_SA = 3, GU_SB = 2;                          // weight stages, token stages
constexpr uint32_t GU_A_STAGE_BYTES = 2 * A_TILE_BYTES;      // gate tile + up tile, 32 KB

__global__ void __launch_bounds__(U_THREADS, 1) k_umma_gateup(GroupedParams p, const __grid_constant__ CUtensorMap tm_gate,
                                                             const __grid_constant__ CUtensorMap tm_up,
                                                             const __grid_constant__ CUtensorMap tm_sh_gate,
                                                             const __grid_constant__ CUtensorMap tm_sh_up) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) PipeBars bars;
  __shared__ __align__(8) uint64_t s_raw_full;
  __shared__ uint32_t s_tmem;
  const int tile = blockIdx.y;
  if (tile >= *p.n_tiles) return;
  trace_stamp((blockIdx.x == 0 && blockIdx.y == p.trace_tile) ? p.trace : nullptr, 40);
  unsigned char* a_stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* b_stages = a_stages + GU_SA * GU_A_STAGE_BYTES;
  const int e = p.tile_expert[tile], rows_valid = p.tile_rows[tile];
  const int n_eff = (rows_valid + 15) & ~15;
  const int f0 = blockIdx.x * UM;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool shared_seg = e >= p.n_expert;

  if (tid == 0) {
    mbar_init(&s_raw_full, 1);
    init_bars<GU_SA, GU_SB>(bars);
  }
  if (warp == 8) umma::tmem_alloc(&s_tmem, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = s_tmem;

  // producer identity: role 0 = gate rows, role 1 = up rows; every producer also owns a token row
  const int role = (tid >> 7) & 1, wrow = tid & 127;
  const uint32_t idesc = umma::idesc_f16_f32(UM, n_eff);

  // Raw bytes of the tile's rows, one 256-weight block (144 B) per row at a time, come in through
  // the copy engine as two tiled copies (128 rows x 144 B out of rows 1152 B apart, gate and up)
  // into a [256][144] staging area, a block (four K steps) ahead of their use.  As per-thread
  // vector loads every warp request would touch 32 different lines and the load/store pipe, which
  // the unpacked tiles also go through, would be the bottleneck.
  unsigned char* raw = b_stages + GU_SB * B_TILE_BYTES;
  const unsigned char* my_raw = raw + (size_t)tid * Q4K_BLOCK_BYTES;
  const CUtensorMap* tmg = shared_seg ? &tm_sh_gate : &tm_gate;
  const CUtensorMap* tmu = shared_seg ? &tm_sh_up : &tm_up;
  const int bank_row0 = (shared_seg ? 0 : e * p.nff) + f0;
  auto request_block = [&](int blk) {
    if (tid == 0) {
      mbar_arrive_expect_tx(&s_raw_full, U_PRODUCERS * (uint32_t)Q4K_BLOCK_BYTES);
      tma_load_2d(raw, tmg, blk * (int)Q4K_BLOCK_BYTES, bank_row0, &s_raw_full);
      tma_load_2d(raw + UM * Q4K_BLOCK_BYTES, tmu, blk * (int)Q4K_BLOCK_BYTES, bank_row0, &s_raw_full);
    }
  };
  if (tid < U_PRODUCERS) request_block(0);
  uint4 cur_h, cur_q[8];

  auto unpack = [&](unsigned char* st, int step, auto jc) -> bool {
    constexpr int j = decltype(jc)::value;
    unsigned char* tA = st + (size_t)role * A_TILE_BYTES;
    if (j == 0) {
      const int blk = step >> 2;
      if (!mbar_wait_bounded(&s_raw_full, blk & 1)) return false;
      cur_h = *reinterpret_cast<const uint4*>(my_raw);
#pragma unroll
      for (int i = 0; i < 8; ++i) cur_q[i] = *reinterpret_cast<const uint4*>(my_raw + 16 + 16 * i);
      // every producer has taken its row: the staging area can be refilled
      asm volatile("bar.sync 1, %0;" ::"n"(U_PRODUCERS) : "memory");
      if (blk + 1 < p.ne / 256) request_block(blk + 1);
    }
    const uint4 ch = cur_h, c0 = cur_q[2 * j], c1 = cur_q[2 * j + 1];
    uint32_t scp, mp;
    q4k_scale_min_pair(ch.y, ch.z, ch.w, j, scp, mp);
    const float d = f16_bits_to_f32(ch.x) * W_PRESCALE, dmin = f16_bits_to_f32(ch.x >> 16) * W_PRESCALE;
    const __half2 s_lo = __float2half2_rn(d * (float)(scp & 0xFFu)), s_hi = __float2half2_rn(d * (float)(scp >> 8));
    const __half2 m_lo = __float2half2_rn(-dmin * (float)(mp & 0xFFu)), m_hi = __float2half2_rn(-dmin * (float)(mp >> 8));
    const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {  // chunk c: K positions 8c..8c+7 (low nibbles), 32+8c.. (high nibbles)
      uint4 lo, hi;
      q4_word_to_h2(w[2 * c], s_lo, m_lo, lo.x, lo.y);
      q4_word_to_h2(w[2 * c + 1], s_lo, m_lo, lo.z, lo.w);
      q4_word_to_h2(w[2 * c] >> 4, s_hi, m_hi, hi.x, hi.y);
      q4_word_to_h2(w[2 * c + 1] >> 4, s_hi, m_hi, hi.z, hi.w);
      *reinterpret_cast<uint4*>(tA + umma::swz128_offset(wrow, c)) = lo;
      *reinterpret_cast<uint4*>(tA + umma::swz128_offset(wrow, 4 + c)) = hi;
    }
    return true;
  };
  auto issue = [&](unsigned char* st, unsigned char* tB, int step) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint64_t bd = umma::smem_desc_k_major_swz128(tB, k);
      umma::mma_f16(tmem, umma::smem_desc_k_major_swz128(st, k), bd, idesc, step > 0 || k > 0);
      umma::mma_f16(tmem + 256, umma::smem_desc_k_major_swz128(st + A_TILE_BYTES, k), bd, idesc, step > 0 || k > 0);
    }
  };
  const int k_steps = p.ne / UK;
  unsigned long long* trc = (blockIdx.x == 0 && blockIdx.y == p.trace_tile) ? p.trace : nullptr;
  trace_stamp(trc, 41);
  bool ok = run_pipeline<GU_SA, GU_SB>(bars, a_stages, GU_A_STAGE_BYTES, b_stages,
                                       reinterpret_cast<const unsigned char*>(p.xg) + tile_step_offset(tile, k_steps, 0),
                                       (size_t)UN * 128, (uint32_t)n_eff * 128u, k_steps, unpack, issue,
                                       trc);
  trace_stamp(trc, 42);

  // epilogue: producers drain the two accumulators.  The CTA's 128 features are two whole 128-byte
  // lines (K steps f0/64 and f0/64 + 1) of every token row of the down kernel's operand
  // ([tile][K step][row][128 B], swizzled like its shared-memory image); the values go through
  // shared memory (the weight stages are idle by now) so that each line is written whole.
  if (tid < U_PRODUCERS) {
    if (ok) ok = mbar_wait_bounded(&bars.done, 0);
    umma::fence_after_sync();
    unsigned char* stg = a_stages;  // [256 rows][256 B]
    if (ok) {
      const int lane_grp = warp & 3, col_half = warp >> 2;
      const int lpos = kperm(lane_grp * 32 + lane);  // position of this thread's feature inside the CTA's 128
      for (int c0 = col_half * 128; c0 < min(n_eff, col_half * 128 + 128); c0 += 32) {
        float g[32], u[32];
        const uint32_t ta = tmem + ((uint32_t)(lane_grp * 32) << 16) + (uint32_t)c0;
        umma::ld_32x32_pair(ta, ta + 256, g, u);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float gv = g[i] * W_POSTSCALE, uv = u[i] * W_POSTSCALE;
          const float a = __fdividef(gv, 1.0f + __expf(-gv)) * uv;
          *reinterpret_cast<__half*>(stg + (size_t)(c0 + i) * 256 + lpos * 2) = __float2half_rn(fminf(fmaxf(a, -65504.f), 65504.f));
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(U_PRODUCERS) : "memory");
    if (ok) {
      unsigned char* act_tile = reinterpret_cast<unsigned char*>(p.act) + tile_step_offset(tile, p.nff / UK, f0 >> 6);
      for (int idx = tid; idx < rows_valid * 16; idx += U_PRODUCERS) {
        const int n = idx >> 4, q = idx & 15;
        const uint4 v = *reinterpret_cast<const uint4*>(stg + (size_t)n * 256 + q * 16);
        *reinterpret_cast<uint4*>(act_tile + ((size_t)(q >> 3) * UN + n) * 128 + (((q & 7) ^ (n & 7)) << 4)) = v;
      }
    }
  }
  trace_stamp(trc, 43);
  if (!ok && lane == 0) atomicExch(&p.status->timeout, 5);
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 8) umma::tmem_dealloc(tmem, 512);
}

// ---- down ---------------------------------------------------------------------------------------------

constexpr int DN_SA = 4, DN_SB = 4;

__device__ __forceinline__ uint32_t ldg_u32_unaligned(const uint8_t* base, size_t off) {
  const size_t a = off & ~(size_t)3;
  const uint32_t lo = __ldg(reinterpret_cast<const uint32_t*>(base + a));
  const uint32_t hi = __ldg(reinterpret_cast<const uint32_t*>(base + a + 4));
  return __funnelshift_r(lo, hi, (uint32_t)(off & 3) * 8);
}

__global__ void __launch_bounds__(U_THREADS, 1) k_umma_down(GroupedParams p) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) PipeBars bars;
  __shared__ uint32_t s_tmem;
  const int tile = blockIdx.y;
  if (tile >= *p.n_tiles) return;
  trace_stamp((blockIdx.x == 0 && blockIdx.y == p.trace_tile) ? p.trace : nullptr, 44);
  unsigned char* a_stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* b_stages = a_stages + DN_SA * A_TILE_BYTES;
  const int e = p.tile_expert[tile], row0 = p.tile_row0[tile], rows_valid = p.tile_rows[tile];
  const int n_eff = (rows_valid + 15) & ~15;
  const int i0 = blockIdx.x * UM;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int drb = p.nff / 256 * (int)Q6K_BLOCK_BYTES;
  const bool shared_seg = e >= p.n_expert;

  if (tid == 0) init_bars<DN_SA, DN_SB>(bars);
  if (warp == 8) umma::tmem_alloc(&s_tmem, 256);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = s_tmem;

  // producer identity: eight consecutive lanes share a weight row (lane w takes the four l values
  // 4w..4w+3 of every quadrant), so a warp request covers whole 32-byte runs of four rows; the 128
  // rows of the tile take four passes.
  const int g8 = tid >> 3, w = tid & 7;
  const uint8_t* wbase = shared_seg ? p.sh_down : p.down + (size_t)e * p.down_stride;  // 16-byte aligned
  const uint32_t idesc = umma::idesc_f16_f32(UM, n_eff);

  // Raw words of one half-block (128 elements = two K steps: low nibbles first, high nibbles
  // second) per pass: ql words of quadrants 0|2 and 1|3, the qh word, the eight scales, d.
  // The next half-block is fetched while the current one is unpacked.
  uint32_t nxt[4][6], cur[4][6];
  const int n_pairs = p.nff / 128;
  auto fetch_pair = [&](int pair) {
    const int blk = pair >> 1, h = pair & 1;
#pragma unroll
    for (int ps = 0; ps < 4; ++ps) {
      const size_t bo = (size_t)(i0 + ps * 32 + g8) * drb + (size_t)blk * Q6K_BLOCK_BYTES;
      nxt[ps][0] = ldg_u32_unaligned(wbase, bo + 64 * h + 4 * w);
      nxt[ps][1] = ldg_u32_unaligned(wbase, bo + 64 * h + 32 + 4 * w);
      nxt[ps][2] = ldg_u32_unaligned(wbase, bo + 128 + 32 * h + 4 * w);
      nxt[ps][3] = ldg_u32_unaligned(wbase, bo + 192 + 8 * h);
      nxt[ps][4] = ldg_u32_unaligned(wbase, bo + 196 + 8 * h);
      nxt[ps][5] = __ldg(reinterpret_cast<const unsigned short*>(wbase + bo + 208));
    }
  };
  if (tid < U_PRODUCERS) fetch_pair(0);

  auto unpack = [&](unsigned char* st, int step, auto) -> bool {
    unsigned char* tA = st;
    const int hi_nib = step & 1;
    if (hi_nib == 0) {
#pragma unroll
      for (int ps = 0; ps < 4; ++ps)
#pragma unroll
        for (int i = 0; i < 6; ++i) cur[ps][i] = nxt[ps][i];
      if ((step >> 1) + 1 < n_pairs) fetch_pair((step >> 1) + 1);
    }
#pragma unroll
    for (int ps = 0; ps < 4; ++ps) {
      const int row = ps * 32 + g8;
      const float d = f16_bits_to_f32(cur[ps][5]) * W_PRESCALE;
      // scale of quadrant qd for these l: byte 2*qd + (w >> 2) of the half's eight scale bytes
      const uint32_t sc4 = __byte_perm(cur[ps][3], cur[ps][4], (w >> 2) ? 0x7531u : 0x6420u);
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        const int qd = 2 * hi_nib + part;
        const uint32_t L = cur[ps][part];
        const uint32_t nib = hi_nib ? (L >> 4) : L;
        const uint32_t code = (nib & 0x0F0F0F0Fu) | (((cur[ps][2] >> (2 * qd)) << 4) & 0x30303030u);
        const float sc = (float)(int)(signed char)((sc4 >> (8 * qd)) & 0xFFu);
        uint32_t o02, o13;
        q6_word_to_h2(code, __float2half2_rn(d * sc), o02, o13);
        // K position inside the step: 32*part + 4w .. +3  ->  chunk 4*part + w/2, half-chunk w&1
        *reinterpret_cast<uint2*>(tA + umma::swz128_offset(row, 4 * part + (w >> 1)) + (w & 1) * 8) = make_uint2(o02, o13);
      }
    }
    return true;
  };
  auto issue = [&](unsigned char* st, unsigned char* tB, int step) {
#pragma unroll
    for (int k = 0; k < 4; ++k)
      umma::mma_f16(tmem, umma::smem_desc_k_major_swz128(st, k), umma::smem_desc_k_major_swz128(tB, k), idesc, step > 0 || k > 0);
  };
  const int k_steps = p.nff / UK;
  unsigned long long* trc = (blockIdx.x == 0 && blockIdx.y == p.trace_tile) ? p.trace : nullptr;
  trace_stamp(trc, 45);
  bool ok = run_pipeline<DN_SA, DN_SB>(bars, a_stages, A_TILE_BYTES, b_stages,
                                       reinterpret_cast<const unsigned char*>(p.act) + tile_step_offset(tile, k_steps, 0),
                                       (size_t)UN * 128, (uint32_t)n_eff * 128u, k_steps, unpack, issue, nullptr);
  trace_stamp(trc, 46);

  if (tid < U_PRODUCERS) {
    if (ok) ok = mbar_wait_bounded(&bars.done, 0);
    umma::fence_after_sync();
    if (ok) {
      const int lane_grp = warp & 3, col_half = warp >> 2;
      const int i = i0 + lane_grp * 32 + lane;
      for (int c0 = col_half * 128; c0 < min(n_eff, col_half * 128 + 128); c0 += 32) {
        float v[32];
        umma::ld_32x32(tmem + ((uint32_t)(lane_grp * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
        for (int t = 0; t < 32; ++t)
          if (c0 + t < rows_valid) p.y[(size_t)(row0 + c0 + t) * p.ne + i] = v[t] * W_POSTSCALE;
      }
    }
  }
  trace_stamp(trc, 47);
  if (!ok && lane == 0) atomicExch(&p.status->timeout, 6);
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 8) umma::tmem_dealloc(tmem, 256);
}

}  // namespace

bool umma_grouped_supported(int ne, int nff) { return ne % 256 == 0 && nff % 256 == 0 && ne % UM == 0 && nff % UM == 0; }

int umma_tile_rows() { return UN; }

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// A Q4_K bank as a 2-D byte tensor [rows][row_bytes]; box = one block (144 B) of 128 rows.
bool q4k_rows_map(CUtensorMap* tm, const uint8_t* base, size_t n_rows, size_t row_bytes) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)n_rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)Q4K_BLOCK_BYTES, (cuuint32_t)UM};
  const cuuint32_t estr[2] = {1, 1};
  return enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

int32_t launch_umma_grouped(infr_cuda_ctx* ctx, const GroupedParams& p, int max_tiles) {
  const size_t smem_gu = 1024 + (size_t)GU_SA * GU_A_STAGE_BYTES + (size_t)GU_SB * B_TILE_BYTES + (size_t)U_PRODUCERS * Q4K_BLOCK_BYTES;
  const size_t smem_dn = 1024 + (size_t)DN_SA * A_TILE_BYTES + (size_t)DN_SB * B_TILE_BYTES;
  cudaError_t e = ensure_smem(reinterpret_cast<const void*>(k_umma_gateup), smem_gu);
  if (e == cudaSuccess) e = ensure_smem(reinterpret_cast<const void*>(k_umma_down), smem_dn);
  if (e != cudaSuccess) return check_cuda(ctx, e, "umma grouped smem attribute");
  const size_t rb = (size_t)p.ne / 256 * Q4K_BLOCK_BYTES;
  CUtensorMap tm_gate, tm_up, tm_sh_gate, tm_sh_up;
  bool ok = q4k_rows_map(&tm_gate, p.gate, (size_t)p.n_expert * p.nff, rb) && q4k_rows_map(&tm_up, p.up, (size_t)p.n_expert * p.nff, rb);
  if (ok && p.sh_gate) ok = q4k_rows_map(&tm_sh_gate, p.sh_gate, (size_t)p.nff, rb) && q4k_rows_map(&tm_sh_up, p.sh_up, (size_t)p.nff, rb);
  if (!ok) return fail(ctx, INFR_CUDA_ERR_CUDA, "grouped GEMM: the driver refused a tensor map for the expert banks");
  if (!p.sh_gate) {
    tm_sh_gate = tm_gate;
    tm_sh_up = tm_up;
  }
  k_umma_gateup<<<dim3(p.nff / UM, max_tiles), U_THREADS, smem_gu, ctx->stream>>>(p, tm_gate, tm_up, tm_sh_gate, tm_sh_up);
  k_umma_down<<<dim3(p.ne / UM, max_tiles), U_THREADS, smem_dn, ctx->stream>>>(p);
  ctx->launches += 2;
  return check_cuda(ctx, cudaGetLastError(), "umma grouped launch");
}

}  // namespace infr
