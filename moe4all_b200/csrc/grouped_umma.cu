// Grouped expert GEMMs on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory).
//
// Same contract as the legacy-MMA kernels of grouped_ffn.cu (reference: CPU stages B-D
// crates/infr-cpu/src/lib.rs:4051-4266; Vulkan native_gemm_mmq_q4k/q6k.comp): per expert segment
//   act = silu(Wg x) * (Wu x)      (k_umma_gateup, Q4_K weights)
//   y   = Wd act                   (k_umma_down,   Q6_K weights)
// with the tokens as the M operand (one or two halves of 128 rows per tile of up to 256 tokens)
// and 256 weight rows as the N operand (gate/up: 128 gate rows and their 128 up rows; down: 256
// output features), so every weight block is unpacked once per 256 tokens, a tile with few tokens
// costs half the MMA instructions of a full one, and in the accumulators a thread's row is a
// token: its results are contiguous in the output.
//
// Warp roles (18 warps): warps 0-15 are producers - two (gate/up) or eight (down) threads share a
// weight row of the tile and unpack its 64 weights of the K step to f16 straight into the 128-byte-swizzled operand tile;
// warp 16 issues the MMAs (one thread) and releases pipeline stages with tcgen05.commit; warp 17
// fetches the token operand: the gather kernel (and the gate/up epilogue) store token rows per
// (tile, K step) as 128-byte lines already in swizzled order, so one bulk copy brings a step's
// whole operand and runs several steps ahead of the MMAs.  After the K loop the producers drain
// the accumulators with tcgen05.ld and write the result.  Weight and token stages are separate
// rings handed over through mbarriers; every wait is bounded.
#include <cuda.h>

#include <type_traits>

#include "kernels.cuh"
#include "umma.cuh"
#include "tma.cuh"

namespace infr {
namespace {

constexpr int UM = 128;           // weight rows per role and CTA
constexpr int UN = 256;           // max token rows per CTA
constexpr int UK = 64;            // K elements per stage
constexpr int U_PRODUCERS = 512;  // producer threads: two per weight row of a gate/up tile pair, four per row of a down tile
constexpr int U_THREADS = U_PRODUCERS + 64;  // + MMA warp + token-copy warp
constexpr float W_PRESCALE = 256.0f;
constexpr float W_POSTSCALE = 1.0f / 256.0f;
constexpr uint32_t A_TILE_BYTES = UM * 128;  // 16 KB
constexpr uint32_t B_TILE_BYTES = UN * 128;  // 32 KB

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
      if (step >= 8 && step < 16) trace_stamp(tr, 64 + 4 * (step - 8));
      // a stage is free again when the MMAs that last read it have completed
      if (!mbar_wait_bounded(&bars.empty_a[s], (use & 1) ^ 1)) { ok = false; return; }
      if (step >= 8 && step < 16) trace_stamp(tr, 65 + 4 * (step - 8));
      if (!unpack(a_stages + (size_t)s * a_stage_bytes, step, jc)) { ok = false; return; }
      if (step >= 8 && step < 16) trace_stamp(tr, 66 + 4 * (step - 8));
      umma::fence_proxy_async();
      __syncwarp();
      if ((tid & 31) == 0) mbar_arrive(&bars.full_a[s]);  // one arrival per producer warp
      if (step >= 8 && step < 16) trace_stamp(tr, 67 + 4 * (step - 8));
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
      if (tr != nullptr && step >= 8 && step < 16) { tr[2 * (100 + 2 * (step - 8))] = 0; tr[2 * (100 + 2 * (step - 8)) + 1] = (unsigned long long)clock64(); }
      issue(a_stages + (size_t)sa * a_stage_bytes, b_stages + (size_t)sb * B_TILE_BYTES, step);
      umma::commit(&bars.empty_a[sa]);
      umma::commit(&bars.empty_b[sb]);
      if (tr != nullptr && step >= 8 && step < 16) { tr[2 * (101 + 2 * (step - 8))] = 0; tr[2 * (101 + 2 * (step - 8)) + 1] = (unsigned long long)clock64(); }
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

// Epilogue helper.  Every lane holds NP consecutive 16-byte pieces of its own row (a token); rows
// are far apart in global memory, so the warp first parks them in its private shared-memory
// patch (row pitch NP*16 + 16 bytes: conflict-free both ways) and then writes them out with
// 32 / NP whole rows per store instruction.  `dst(row, piece)` gives the global address of a piece.
template <int NP, typename Dst>
__device__ __forceinline__ void warp_store_rows(unsigned char* patch, const uint4 (&v)[NP], int lane, int rows_ok, Dst dst) {
  constexpr int PITCH = NP * 16 + 16;
#pragma unroll
  for (int c = 0; c < NP; ++c) *reinterpret_cast<uint4*>(patch + lane * PITCH + c * 16) = v[c];
  __syncwarp();
  constexpr int RPI = 32 / NP;  // rows per instruction
  const int piece = lane % NP, sub = lane / NP;
#pragma unroll
  for (int it = 0; it < NP; ++it) {
    const int row = it * RPI + sub;
    const uint4 x = *reinterpret_cast<const uint4*>(patch + row * PITCH + piece * 16);
    if (row < rows_ok) *reinterpret_cast<uint4*>(dst(row, piece)) = x;
  }
  __syncwarp();
}

// ---- gate/up + SwiGLU ---------------------------------------------------------------------------

constexpr int GU_SA = 3, GU_SB = 2;                          // weight stages, token stages
constexpr uint32_t GU_A_STAGE_BYTES = 2 * A_TILE_BYTES;      // gate tile + up tile, 32 KB

// GENERAL = false is the common form (SiLU, no clamp): its epilogue has no other arm.  TRACED = false leaves
// the phase stamps out of the K loop altogether (they are only wanted while a trace buffer is set).
template <bool GENERAL, bool TRACED>
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
  if (TRACED) trace_stamp((blockIdx.x == 0 && blockIdx.y == p.trace_tile) ? p.trace : nullptr, 40);
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
  if (warp == U_PRODUCERS / 32) umma::tmem_alloc(&s_tmem, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = s_tmem;

  // producer identity: role 0 = gate rows, role 1 = up rows; two threads share a weight row, thread
  // `hh` taking code words 4 hh .. 4 hh + 3 of every 32-byte run (K positions 16 hh .. 16 hh + 15
  // from the low nibbles, 32 + 16 hh .. from the high ones)
  const int role = (tid >> 7) & 1, wrow = tid & 127, hh = (tid >> 8) & 1;
  const uint32_t idesc = umma::idesc_f16_f32(128, 2 * UM);  // 128 tokens x (128 gate + 128 up) rows
  const int n_m = (rows_valid + 127) >> 7;                   // token halves in use

  // Raw bytes of the tile's rows, one 256-weight block (144 B) per row at a time, come in through
  // the copy engine as two tiled copies (128 rows x 144 B out of rows 1152 B apart, gate and up)
  // into a [256][144] staging area, a block (four K steps) ahead of their use.  As per-thread
  // vector loads every warp request would touch 32 different lines and the load/store pipe, which
  // the unpacked tiles also go through, would be the bottleneck.
  unsigned char* raw = b_stages + GU_SB * B_TILE_BYTES;
  const unsigned char* my_raw = raw + (size_t)(tid & 255) * Q4K_BLOCK_BYTES;
  const CUtensorMap* tmg = shared_seg ? &tm_sh_gate : &tm_gate;
  const CUtensorMap* tmu = shared_seg ? &tm_sh_up : &tm_up;
  // rows of one expert in the bank: nff, or 2 nff where gate and up share a bank (the up map then starts nff rows in)
  const int bank_row0 = (shared_seg ? 0 : e * p.gu_rows) + f0;
  auto request_block = [&](int blk) {
    if (tid == 0) {
      mbar_arrive_expect_tx(&s_raw_full, 2 * UM * (uint32_t)Q4K_BLOCK_BYTES);
      tma_load_2d(raw, tmg, blk * (int)Q4K_BLOCK_BYTES, bank_row0, &s_raw_full);
      tma_load_2d(raw + UM * Q4K_BLOCK_BYTES, tmu, blk * (int)Q4K_BLOCK_BYTES, bank_row0, &s_raw_full);
    }
  };
  if (tid < U_PRODUCERS) request_block(0);
  uint4 cur_h, cur_q[4];

  auto unpack = [&](unsigned char* st, int step, auto jc) -> bool {
    constexpr int j = decltype(jc)::value;
    unsigned char* tA = st + (size_t)role * A_TILE_BYTES;
    if (j == 0) {
      const int blk = step >> 2;
      if (!mbar_wait_bounded(&s_raw_full, blk & 1)) return false;
      cur_h = *reinterpret_cast<const uint4*>(my_raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) cur_q[i] = *reinterpret_cast<const uint4*>(my_raw + 16 + 32 * i + 16 * hh);
      // every producer has taken its row: the staging area can be refilled
      asm volatile("bar.sync 1, %0;" ::"n"(U_PRODUCERS) : "memory");
      if (blk + 1 < p.ne / 256) request_block(blk + 1);
    }
    const uint4 ch = cur_h, cq = cur_q[j];
    uint32_t scp, mp;
    q4k_scale_min_pair(ch.y, ch.z, ch.w, j, scp, mp);
    const float d = f16_bits_to_f32(ch.x) * W_PRESCALE, dmin = f16_bits_to_f32(ch.x >> 16) * W_PRESCALE;
    const __half2 s_lo = __float2half2_rn(d * (float)(scp & 0xFFu)), s_hi = __float2half2_rn(d * (float)(scp >> 8));
    const __half2 m_lo = __float2half2_rn(-dmin * (float)(mp & 0xFFu)), m_hi = __float2half2_rn(-dmin * (float)(mp >> 8));
    const uint32_t w[4] = {cq.x, cq.y, cq.z, cq.w};
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {  // chunk c: K positions 8c..8c+7 (low nibbles), 32+8c.. (high nibbles)
      const int c = 2 * hh + cc;
      uint4 lo, hi;
      q4_word_to_h2(w[2 * cc], s_lo, m_lo, lo.x, lo.y);
      q4_word_to_h2(w[2 * cc + 1], s_lo, m_lo, lo.z, lo.w);
      q4_word_to_h2(w[2 * cc] >> 4, s_hi, m_hi, hi.x, hi.y);
      q4_word_to_h2(w[2 * cc + 1] >> 4, s_hi, m_hi, hi.z, hi.w);
      *reinterpret_cast<uint4*>(tA + umma::swz128_offset(wrow, c)) = lo;
      *reinterpret_cast<uint4*>(tA + umma::swz128_offset(wrow, 4 + c)) = hi;
    }
    return true;
  };
  // One thread issues everything, so its instruction count per step is the pipeline's floor for
  // small tiles: the three descriptors are built once per step, a K slice is +32 bytes = +2 in
  // the address field.
  auto issue = [&](unsigned char* st, unsigned char* tB, int step) {
    const uint64_t dw = umma::smem_desc_k_major_swz128(st, 0);  // gate tile and up tile back to back: 256 rows
    const uint64_t dt = umma::smem_desc_k_major_swz128(tB, 0);
    for (int m = 0; m < n_m; ++m) {
      const uint64_t dtm = dt + (uint64_t)m * (128 * 128 / 16);  // token rows 128 m ..
      umma::mma_f16(tmem + m * 256, dtm, dw, idesc, step > 0);
#pragma unroll
      for (int k = 1; k < 4; ++k) umma::mma_f16_acc(tmem + m * 256, dtm + 2 * k, dw + 2 * k, idesc);
    }
  };
  const int k_steps = p.ne / UK;
  unsigned long long* trc = (TRACED && blockIdx.x == 0 && blockIdx.y == p.trace_tile) ? p.trace : nullptr;
  trace_stamp(trc, 41);
  bool ok = run_pipeline<GU_SA, GU_SB>(bars, a_stages, GU_A_STAGE_BYTES, b_stages,
                                       reinterpret_cast<const unsigned char*>(p.xg) + tile_step_offset(tile, k_steps, 0),
                                       (size_t)UN * 128, (uint32_t)n_eff * 128u, k_steps, unpack, issue,
                                       TRACED ? trc : nullptr);
  trace_stamp(trc, 42);

  // epilogue: a thread's accumulator row is a token; its 64 gate and 64 up values per feature half
  // give 64 activations = one whole 128-byte line of the down kernel's operand
  // ([tile][K step][row][128 B], swizzled like its shared-memory image).
  if (tid < U_PRODUCERS) {
    if (ok) ok = mbar_wait_bounded(&bars.done, 0);
    umma::fence_after_sync();
    const int lq = warp & 3, m = warp >> 3, fh = (warp >> 2) & 1;  // TMEM lane quarter, token half, feature half
    if (ok && m < n_m) {
      const float clamp = e < p.n_expert ? p.clamp : 0.f;  // the shared expert's segment is not clamped
      const int n0 = m * 128 + lq * 32;  // first token row of this warp
      const uint32_t trow = tmem + ((uint32_t)(lq * 32) << 16) + (uint32_t)(m * 256 + fh * 64);
      unsigned char* lines = reinterpret_cast<unsigned char*>(p.act) + tile_step_offset(tile, p.nff / UK, (f0 >> 6) + fh) + (size_t)n0 * 128;
      unsigned char* patch = a_stages + (size_t)warp * (32 * 80);  // the weight stages are idle by now
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        float g[32], u[32];
        umma::ld_32x32_pair(trow + hf * 32, trow + 128 + hf * 32, g, u);
        uint4 o[4];
#pragma unroll
        for (int q = 0; q < 8; ++q) {  // four features -> positions 0,2,1,3
          float a[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float gv = g[4 * q + t] * W_POSTSCALE, uv = u[4 * q + t] * W_POSTSCALE;
            const float av = GENERAL ? gated_act<true>(p.act_kind, clamp, gv, uv) : __fdividef(gv, 1.0f + __expf(-gv)) * uv;
            a[t] = fminf(fmaxf(av, -65504.f), 65504.f);
          }
          const uint32_t w0 = h2_as_u32(__floats2half2_rn(a[0], a[2])), w1 = h2_as_u32(__floats2half2_rn(a[1], a[3]));
          if (q & 1) {
            o[q >> 1].z = w0;
            o[q >> 1].w = w1;
          } else {
            o[q >> 1].x = w0;
            o[q >> 1].y = w1;
          }
        }
        warp_store_rows<4>(patch, o, lane, rows_valid - n0, [&](int row, int piece) {
          return lines + (size_t)row * 128 + (((4 * hf + piece) ^ ((n0 + row) & 7)) << 4);
        });
      }
    }
  }
  trace_stamp(trc, 43);
  if (!ok && lane == 0) atomicExch(&p.status->timeout, 5);
  umma::fence_before_sync();
  __syncthreads();
  if (warp == U_PRODUCERS / 32) umma::tmem_dealloc(tmem, 512);
}

// ---- down ---------------------------------------------------------------------------------------------

constexpr int DN_SA = 3, DN_SB = 3;
constexpr int DM = 256;                                   // output features per CTA
constexpr uint32_t DN_W_STAGE_BYTES = DM * 128;           // 32 KB

// Q4: the down banks are Q4_K (raw blocks by tiled TMA copies, as in the gate/up kernel) instead of Q6_K.
template <bool Q4>
__global__ void __launch_bounds__(U_THREADS, 1) k_umma_down(GroupedParams p, const __grid_constant__ CUtensorMap tm_down,
                                                           const __grid_constant__ CUtensorMap tm_sh_down) {
  constexpr int SB = Q4 ? 2 : DN_SB;  // the Q4_K form gives one token stage to its raw-block staging area
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) PipeBars bars;
  __shared__ __align__(8) uint64_t s_raw_full;
  __shared__ uint32_t s_tmem;
  const int tile = blockIdx.y;
  if (tile >= *p.n_tiles) return;
  trace_stamp((blockIdx.x == 0 && blockIdx.y == p.trace_tile) ? p.trace : nullptr, 44);
  unsigned char* a_stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* b_stages = a_stages + DN_SA * DN_W_STAGE_BYTES;
  const int e = p.tile_expert[tile], row0 = p.tile_row0[tile], rows_valid = p.tile_rows[tile];
  const int n_eff = (rows_valid + 15) & ~15;
  const int i0 = blockIdx.x * DM;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int drb = p.nff / 256 * (int)(Q4 ? Q4K_BLOCK_BYTES : Q6K_BLOCK_BYTES);
  const bool shared_seg = e >= p.n_expert;

  if (tid == 0) {
    mbar_init(&s_raw_full, 1);
    init_bars<DN_SA, SB>(bars);
  }
  if (warp == U_PRODUCERS / 32) umma::tmem_alloc(&s_tmem, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = s_tmem;
  trace_stamp((blockIdx.x == 0 && blockIdx.y == p.trace_tile) ? p.trace : nullptr, 48);

  // producer identity: eight consecutive lanes share a weight row (lane w takes the four l values
  // 4w..4w+3 of every quadrant), so a warp request covers whole 32-byte runs of four rows; the 128
  // rows of the tile take four passes.
  const int g8 = tid >> 3, w = tid & 7;
  const uint8_t* wbase = shared_seg ? p.sh_down : p.down + (size_t)e * p.down_stride;  // 16-byte aligned
  const uint32_t idesc = umma::idesc_f16_f32(128, DM);  // 128 tokens x 256 output features
  const int n_m = (rows_valid + 127) >> 7;

  auto issue = [&](unsigned char* st, unsigned char* tB, int step) {
    const uint64_t dw = umma::smem_desc_k_major_swz128(st, 0), dt = umma::smem_desc_k_major_swz128(tB, 0);
    for (int m = 0; m < n_m; ++m) {
      const uint64_t dtm = dt + (uint64_t)m * (128 * 128 / 16);
      umma::mma_f16(tmem + m * 256, dtm, dw, idesc, step > 0);
#pragma unroll
      for (int k = 1; k < 4; ++k) umma::mma_f16_acc(tmem + m * 256, dtm + 2 * k, dw + 2 * k, idesc);
    }
  };
  const int k_steps = p.nff / UK;
  unsigned long long* trc = (blockIdx.x == 0 && blockIdx.y == p.trace_tile) ? p.trace : nullptr;
  trace_stamp(trc, 45);
  bool ok;
  const unsigned char* tok_src = reinterpret_cast<const unsigned char*>(p.act) + tile_step_offset(tile, k_steps, 0);
  if constexpr (Q4) {
    // two threads share a weight row; thread `hh` takes code words 4 hh .. 4 hh + 3 of every 32-byte
    // run.  Raw blocks (144 B of each of the 256 rows) arrive by one tiled copy, a block ahead.
    const int wrow = tid & 255, hh = (tid >> 8) & 1;
    unsigned char* raw = b_stages + SB * B_TILE_BYTES;
    const unsigned char* my_raw = raw + (size_t)wrow * Q4K_BLOCK_BYTES;
    const CUtensorMap* tmd = shared_seg ? &tm_sh_down : &tm_down;
    const int bank_row0 = (shared_seg ? 0 : e * p.ne) + i0;
    auto request_block = [&](int blk) {
      if (tid == 0) {
        mbar_arrive_expect_tx(&s_raw_full, DM * (uint32_t)Q4K_BLOCK_BYTES);
        tma_load_2d(raw, tmd, blk * (int)Q4K_BLOCK_BYTES, bank_row0, &s_raw_full);
      }
    };
    if (tid < U_PRODUCERS) request_block(0);
    uint4 cur_h, cur_q[4];
    auto unpack = [&](unsigned char* tA, int step, auto jc) -> bool {
      constexpr int j = decltype(jc)::value;
      if (j == 0) {
        const int blk = step >> 2;
        if (!mbar_wait_bounded(&s_raw_full, blk & 1)) return false;
        cur_h = *reinterpret_cast<const uint4*>(my_raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) cur_q[i] = *reinterpret_cast<const uint4*>(my_raw + 16 + 32 * i + 16 * hh);
        asm volatile("bar.sync 1, %0;" ::"n"(U_PRODUCERS) : "memory");  // every producer has taken its row
        if (blk + 1 < p.nff / 256) request_block(blk + 1);
      }
      const uint4 ch = cur_h, cq = cur_q[j];
      uint32_t scp, mp;
      q4k_scale_min_pair(ch.y, ch.z, ch.w, j, scp, mp);
      const float d = f16_bits_to_f32(ch.x) * W_PRESCALE, dmin = f16_bits_to_f32(ch.x >> 16) * W_PRESCALE;
      const __half2 s_lo = __float2half2_rn(d * (float)(scp & 0xFFu)), s_hi = __float2half2_rn(d * (float)(scp >> 8));
      const __half2 m_lo = __float2half2_rn(-dmin * (float)(mp & 0xFFu)), m_hi = __float2half2_rn(-dmin * (float)(mp >> 8));
      const uint32_t w4[4] = {cq.x, cq.y, cq.z, cq.w};
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = 2 * hh + cc;
        uint4 lo, hi;
        q4_word_to_h2(w4[2 * cc], s_lo, m_lo, lo.x, lo.y);
        q4_word_to_h2(w4[2 * cc + 1], s_lo, m_lo, lo.z, lo.w);
        q4_word_to_h2(w4[2 * cc] >> 4, s_hi, m_hi, hi.x, hi.y);
        q4_word_to_h2(w4[2 * cc + 1] >> 4, s_hi, m_hi, hi.z, hi.w);
        *reinterpret_cast<uint4*>(tA + umma::swz128_offset(wrow, c)) = lo;
        *reinterpret_cast<uint4*>(tA + umma::swz128_offset(wrow, 4 + c)) = hi;
      }
      return true;
    };
    ok = run_pipeline<DN_SA, SB>(bars, a_stages, DN_W_STAGE_BYTES, b_stages, tok_src, (size_t)UN * 128, (uint32_t)n_eff * 128u, k_steps,
                                 unpack, issue, nullptr);
  } else {
    // Raw words of one half-block (128 elements = two K steps: low nibbles first, high nibbles
    // second) per pass, fetched while the previous half-block is unpacked.  Q6_K blocks are only
    // 2-byte aligned, so the words a lane needs straddle two aligned words; the loads stay plain
    // aligned loads with nothing computed on them (so nothing waits for them at issue time), and
    // the realignment happens at unpack time: the upper word comes from the neighbouring lane of
    // the row's eight (shuffle), the words beyond the eighth and the scales / d from six spare
    // loads spread over lanes 0-5.  Four loads per lane and pass instead of eleven.
    constexpr int PS = DM * 8 / U_PRODUCERS;  // passes over the tile's rows
    uint32_t nxt[PS][4], cur[PS][6];
    const int n_pairs = p.nff / 128;
    auto fetch_pair = [&](int pair) {
      const int blk = pair >> 1, h = pair & 1;
  #pragma unroll
      for (int ps = 0; ps < PS; ++ps) {
        const size_t bo = (size_t)(i0 + ps * (U_PRODUCERS / 8) + g8) * drb + (size_t)blk * Q6K_BLOCK_BYTES;
        const uint8_t* ab = wbase + (bo & ~(size_t)3);
        const bool aligned = (bo & 3) == 0;
        // lane's spare word: scales (3 words), d, ql word 16 of this half, qh word 8 of this half.
        // Nothing past the block's 210 bytes is read (the bank may end with it): a block on a word
        // boundary needs no third scale word (lane 2 repeats the second), and d comes as 16 bits.
        const int spare = w == 0 ? 192 + 8 * h : w == 1 ? 196 + 8 * h : w == 2 ? (aligned ? 196 : 200) + 8 * h : w == 4 ? 64 * h + 64 : 160 + 32 * h;
        nxt[ps][0] = __ldg(reinterpret_cast<const uint32_t*>(ab + 64 * h + 4 * w));
        nxt[ps][1] = __ldg(reinterpret_cast<const uint32_t*>(ab + 64 * h + 32 + 4 * w));
        nxt[ps][2] = __ldg(reinterpret_cast<const uint32_t*>(ab + 128 + 32 * h + 4 * w));
        nxt[ps][3] = w == 3 ? (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(wbase + bo + 208))
                            : (w < 6 ? __ldg(reinterpret_cast<const uint32_t*>(ab + spare)) : 0u);
      }
    };
    // the CTA's 256 weight rows are one contiguous range: ask for it in L2 up front, so that the
    // small per-lane loads below find it there instead of each waiting for DRAM
    if (tid == U_PRODUCERS + 32) {
      const uint8_t* slab = wbase + (size_t)i0 * drb;
      const size_t total = (size_t)DM * drb;  // a multiple of 16: DM = 256 rows of 210-byte blocks
      for (size_t off = 0; off < total; off += 32768) bulk_prefetch_l2(slab + off, (uint32_t)(total - off < 32768 ? total - off : 32768));
    }
    if (tid < U_PRODUCERS) fetch_pair(0);
    trace_stamp(trc, 49);

    auto unpack = [&](unsigned char* st, int step, auto) -> bool {
      unsigned char* tA = st;
      const int hi_nib = step & 1;
      if (hi_nib == 0) {
        const int blk = step >> 2;
  #pragma unroll
        for (int ps = 0; ps < PS; ++ps) {
          const uint32_t sh = (uint32_t)((((size_t)(i0 + ps * (U_PRODUCERS / 8) + g8) * drb + (size_t)blk * Q6K_BLOCK_BYTES) & 3) * 8);
          const uint32_t a0 = nxt[ps][0], b0 = nxt[ps][1], h0 = nxt[ps][2], sp = nxt[ps][3];
          // the next aligned word: from the lane to the right; for the eighth lane ql's second run
          // starts where the first ends, the other two continue in spare words
          const uint32_t a_r = __shfl_down_sync(0xFFFFFFFFu, a0, 1, 8), b_r = __shfl_down_sync(0xFFFFFFFFu, b0, 1, 8),
                         h_r = __shfl_down_sync(0xFFFFFFFFu, h0, 1, 8);
          const uint32_t b_first = __shfl_sync(0xFFFFFFFFu, b0, 0, 8);
          const uint32_t s0 = __shfl_sync(0xFFFFFFFFu, sp, 0, 8), s1 = __shfl_sync(0xFFFFFFFFu, sp, 1, 8), s2 = __shfl_sync(0xFFFFFFFFu, sp, 2, 8),
                         dw = __shfl_sync(0xFFFFFFFFu, sp, 3, 8), b_8 = __shfl_sync(0xFFFFFFFFu, sp, 4, 8), h_8 = __shfl_sync(0xFFFFFFFFu, sp, 5, 8);
          cur[ps][0] = __funnelshift_r(a0, w == 7 ? b_first : a_r, sh);
          cur[ps][1] = __funnelshift_r(b0, w == 7 ? b_8 : b_r, sh);
          cur[ps][2] = __funnelshift_r(h0, w == 7 ? h_8 : h_r, sh);
          cur[ps][3] = __funnelshift_r(s0, s1, sh);
          cur[ps][4] = __funnelshift_r(s1, s2, sh);
          cur[ps][5] = dw;  // the block's f16 d, fetched as 16 bits
        }
        if ((step >> 1) + 1 < n_pairs) fetch_pair((step >> 1) + 1);
      }
  #pragma unroll
      for (int ps = 0; ps < PS; ++ps) {
        const int row = ps * (U_PRODUCERS / 8) + g8;
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
    ok = run_pipeline<DN_SA, SB>(bars, a_stages, DN_W_STAGE_BYTES, b_stages, tok_src, (size_t)UN * 128, (uint32_t)n_eff * 128u, k_steps,
                                 unpack, issue, nullptr);
  }
  trace_stamp(trc, 46);

  // epilogue: a thread's accumulator row is a token, its 128 columns of this warp's feature half
  // are 512 contiguous bytes of the token's output row
  if (tid < U_PRODUCERS) {
    if (ok) ok = mbar_wait_bounded(&bars.done, 0);
    umma::fence_after_sync();
    const int lq = warp & 3, m = warp >> 3, ch = (warp >> 2) & 1;
    if (ok && m < n_m) {
      const int n0 = m * 128 + lq * 32;
      const uint32_t trow = tmem + ((uint32_t)(lq * 32) << 16) + (uint32_t)(m * 256 + ch * 128);
      const size_t esz = p.y_f16 ? 2 : 4;
      unsigned char* out = reinterpret_cast<unsigned char*>(p.y) + ((size_t)(row0 + n0) * p.ne + i0 + ch * 128) * esz;
      const size_t out_pitch = (size_t)p.ne * esz;
      unsigned char* patch = a_stages + (size_t)warp * (32 * 144);  // the weight stages are idle by now
      float row_scale[4] = {0.f, 0.f, 0.f, 0.f};  // f16 rows: the scales of this thread's four passes
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float v[32];
        umma::ld_32x32(trow + c * 32, v);
        if (p.y_f16) {
          // the combine kernel is the only reader: f16 rows, the 32 outputs of this pass sharing a
          // power-of-two scale that brings their largest magnitude to [2^14, 2^15) (any range of
          // outputs keeps 11 bits against its neighbours' maximum; the sum over slots is taken in f32)
          float m = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) m = fmaxf(m, fabsf(v[i]));
          const int ex = (__float_as_int(m) >> 23) & 0xFF;  // biased exponent of the maximum
          const bool live = ex >= 32;                       // below 2^-95: stored as zeros
          const bool fin = ex < 255;                        // an infinite or NaN output goes through as it is
          const float inv = !live ? 0.f : fin ? __int_as_float((268 - ex) << 23) : 1.0f;  // 2^(14 - exponent)
          row_scale[c] = !live ? 0.f : fin ? __int_as_float((ex - 22) << 23) : W_POSTSCALE;  // 2^-8 / inv
          uint4 h[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float* q = v + 8 * t;
            h[t] = make_uint4(h2_as_u32(__floats2half2_rn(q[0] * inv, q[1] * inv)), h2_as_u32(__floats2half2_rn(q[2] * inv, q[3] * inv)),
                              h2_as_u32(__floats2half2_rn(q[4] * inv, q[5] * inv)), h2_as_u32(__floats2half2_rn(q[6] * inv, q[7] * inv)));
          }
          warp_store_rows<4>(patch, h, lane, rows_valid - n0, [&](int row, int piece) {
            return out + (size_t)row * out_pitch + (size_t)c * 64 + piece * 16;
          });
          continue;
        }
        uint4 o[8];
#pragma unroll
        for (int t = 0; t < 8; ++t)
          o[t] = make_uint4(__float_as_uint(v[4 * t] * W_POSTSCALE), __float_as_uint(v[4 * t + 1] * W_POSTSCALE),
                            __float_as_uint(v[4 * t + 2] * W_POSTSCALE), __float_as_uint(v[4 * t + 3] * W_POSTSCALE));
        warp_store_rows<8>(patch, o, lane, rows_valid - n0, [&](int row, int piece) {
          return out + (size_t)row * out_pitch + (size_t)c * 128 + piece * 16;
        });
      }
      if (p.y_f16 && lane < rows_valid - n0)  // the four scales of this row's 128 outputs: one 16-byte store
        *reinterpret_cast<float4*>(p.y_scale + (size_t)(row0 + n0 + lane) * (p.ne / 32) + (i0 + ch * 128) / 32) =
            make_float4(row_scale[0], row_scale[1], row_scale[2], row_scale[3]);
    }
  }
  trace_stamp(trc, 47);
  if (!ok && lane == 0) atomicExch(&p.status->timeout, 6);
  umma::fence_before_sync();
  __syncthreads();
  if (warp == U_PRODUCERS / 32) umma::tmem_dealloc(tmem, 512);
}

}  // namespace

bool umma_grouped_supported(int ne, int nff) { return ne % 256 == 0 && nff % 256 == 0 && ne % DM == 0 && nff % UM == 0; }

int umma_tile_rows() { return UN; }

namespace {

}  // namespace

int32_t launch_umma_grouped(infr_cuda_ctx* ctx, const GroupedParams& p, int max_tiles) {
  const size_t smem_gu = 1024 + (size_t)GU_SA * GU_A_STAGE_BYTES + (size_t)GU_SB * B_TILE_BYTES + (size_t)2 * UM * Q4K_BLOCK_BYTES;
  const size_t smem_dn = 1024 + (size_t)DN_SA * DN_W_STAGE_BYTES +
                         (p.down_q4k ? (size_t)2 * B_TILE_BYTES + (size_t)DM * Q4K_BLOCK_BYTES : (size_t)DN_SB * B_TILE_BYTES);
  const bool general = p.act_kind != INFR_CUDA_ACT_SILU || p.clamp > 0.f;
  const bool traced = p.trace != nullptr;
  auto gu_kernel = general ? (traced ? k_umma_gateup<true, true> : k_umma_gateup<true, false>)
                           : (traced ? k_umma_gateup<false, true> : k_umma_gateup<false, false>);
  cudaError_t e = ensure_smem(reinterpret_cast<const void*>(gu_kernel), smem_gu);
  if (e == cudaSuccess)
    e = p.down_q4k ? ensure_smem(reinterpret_cast<const void*>(k_umma_down<true>), smem_dn)
                   : ensure_smem(reinterpret_cast<const void*>(k_umma_down<false>), smem_dn);
  if (e != cudaSuccess) return check_cuda(ctx, e, "umma grouped smem attribute");
  const size_t rb = (size_t)p.ne / 256 * Q4K_BLOCK_BYTES;
  CUtensorMap tm_gate, tm_up, tm_sh_gate, tm_sh_up, tm_down, tm_sh_down;
  // a bank's rows as one 2-D tensor; with gate and up in one bank an expert has 2 nff rows and the
  // up map starts nff rows in (and ends with the bank)
  const size_t rows_per_expert = p.gate_stride / rb;
  const size_t bank_rows = (size_t)p.n_expert * rows_per_expert;
  bool ok = q4k_rows_map(&tm_gate, p.gate, bank_rows, rb, UM) &&
            q4k_rows_map(&tm_up, p.up, bank_rows - (rows_per_expert - (size_t)p.nff), rb, UM);
  if (ok && p.sh_gate) ok = q4k_rows_map(&tm_sh_gate, p.sh_gate, (size_t)p.nff, rb, UM) && q4k_rows_map(&tm_sh_up, p.sh_up, (size_t)p.nff, rb, UM);
  if (!p.sh_gate) {
    tm_sh_gate = tm_gate;
    tm_sh_up = tm_up;
  }
  tm_down = tm_gate;  // placeholders when the down banks are Q6_K (that kernel reads them with plain loads)
  tm_sh_down = tm_gate;
  if (ok && p.down_q4k) {
    const size_t drb = (size_t)p.nff / 256 * Q4K_BLOCK_BYTES;
    ok = q4k_rows_map(&tm_down, p.down, (size_t)p.n_expert * p.ne, drb, DM);
    tm_sh_down = tm_down;
    if (ok && p.sh_down) ok = q4k_rows_map(&tm_sh_down, p.sh_down, (size_t)p.ne, drb, DM);
  }
  if (!ok) return fail(ctx, INFR_CUDA_ERR_CUDA, "grouped GEMM: the driver refused a tensor map for the expert banks");
  gu_kernel<<<dim3(p.nff / UM, max_tiles), U_THREADS, smem_gu, ctx->stream>>>(p, tm_gate, tm_up, tm_sh_gate, tm_sh_up);
  if (p.down_q4k)
    k_umma_down<true><<<dim3(p.ne / DM, max_tiles), U_THREADS, smem_dn, ctx->stream>>>(p, tm_down, tm_sh_down);
  else
    k_umma_down<false><<<dim3(p.ne / DM, max_tiles), U_THREADS, smem_dn, ctx->stream>>>(p, tm_down, tm_sh_down);
  ctx->launches += 2;
  return check_cuda(ctx, cudaGetLastError(), "umma grouped launch");
}

}  // namespace infr
