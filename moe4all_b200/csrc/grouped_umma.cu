// Grouped expert GEMMs on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory).
//
// Same contract as the legacy-MMA kernels of grouped_ffn.cu (reference: CPU stages B-D
// crates/infr-cpu/src/lib.rs:4051-4266; Vulkan native_gemm_mmq_q4k/q6k.comp): per expert segment
//   act = silu(Wg x) * (Wu x)      (k_umma_gateup, Q4_K weights)
//   y   = Wd act                   (k_umma_down,   Q6_K weights)
// with the weights as the M operand (128 output features per CTA) and up to 256 token rows as the
// N operand, so every weight block is unpacked once per 256 tokens.
//
// Warp roles (9 warps): warps 0-7 are producers - each thread owns one weight row of the tile,
// unpacks its 64 weights of the K step to f16 straight into the 128-byte-swizzled operand tile,
// and copies one token row's 128 bytes with cp.async; warp 8 issues the MMAs (one thread) and
// releases each pipeline stage with tcgen05.commit.  After the K loop the producers drain the
// accumulators with tcgen05.ld and write the result.  Stages are handed over through mbarriers;
// every wait is bounded.
#include <type_traits>

#include "kernels.cuh"
#include "umma.cuh"

namespace infr {
namespace {

constexpr int UM = 128;           // weight rows per role and CTA
constexpr int UN = 256;           // max token rows per CTA
constexpr int UK = 64;            // K elements per stage
constexpr int U_PRODUCERS = 256;  // producer threads
constexpr int U_THREADS = U_PRODUCERS + 32;
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

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// The K step's slice (64 halfs = 128 B) of up to 256 token rows into the swizzled B tile.  Eight
// consecutive lanes copy the eight 16-byte pieces of one row, so a warp request covers four whole
// 128-byte lines.
__device__ __forceinline__ void copy_token_tile(unsigned char* tB, const __half* src, int ld, int rows_valid, int tid) {
  const int chunk = tid & 7;
#pragma unroll
  for (int pass = 0; pass < 8; ++pass) {
    const int row = pass * 32 + (tid >> 3);
    if (row < rows_valid) cp_async16(tB + umma::swz128_offset(row, chunk), src + (size_t)row * ld + chunk * 8);
  }
}

struct PipeBars {
  uint64_t full[4];
  uint64_t empty[4];
  uint64_t done;
};

// Shared pipeline skeleton.  Producers: `copy_b(stage_ptr, step)` starts the asynchronous token-tile
// copy of a step STAGES-2 steps ahead of its use, `unpack(stage_ptr, step)` writes the weight
// tile(s); MMA thread: `issue(stage_ptr, step)`.
template <int STAGES, typename CopyB, typename Unpack, typename Issue>
__device__ __forceinline__ bool run_pipeline(PipeBars& bars, unsigned char* stages, uint32_t stage_bytes, int n_steps,
                                             CopyB copy_b, Unpack unpack, Issue issue, unsigned long long* tr) {
  constexpr int AHEAD = STAGES - 2;
  const int tid = threadIdx.x;
  bool ok = true;
  if (tid < U_PRODUCERS) {
    // stages are claimed in step order; a claim waits for the MMAs that last read the stage
    auto claim = [&](int step) {
      const int s = step % STAGES, use = step / STAGES;
      if (!mbar_wait_bounded(&bars.empty[s], (use & 1) ^ 1)) return false;
      copy_b(stages + (size_t)s * stage_bytes, step);
      return true;
    };
    for (int step = 0; step < AHEAD && step < n_steps && ok; ++step) {
      ok = claim(step);
      cp_async_commit();
    }
    // `jc` carries step % 4 as a compile-time constant (n_steps is a multiple of four): the
    // producers index their register-resident prefetch buffers with it
    auto body = [&](int step, auto jc) {
      if (!ok) return;
      if (step < 8) trace_stamp(tr, 64 + 4 * step);
      if (step + AHEAD < n_steps) ok = claim(step + AHEAD);
      cp_async_commit();  // one group per step, empty or not, keeps the group count uniform
      if (!ok) return;
      if (step < 8) trace_stamp(tr, 65 + 4 * step);
      const int s = step % STAGES;
      unpack(stages + (size_t)s * stage_bytes, step, jc);
      if (step < 8) trace_stamp(tr, 66 + 4 * step);
      cp_async_wait_group<AHEAD>();  // the token tile of `step` has landed
      if (step < 8) trace_stamp(tr, 67 + 4 * step);
      umma::fence_proxy_async();
      __syncwarp();
      if ((tid & 31) == 0) mbar_arrive(&bars.full[s]);  // one arrival per producer warp
    };
    for (int base = 0; base < n_steps && ok; base += 4) {
      body(base, std::integral_constant<int, 0>{});
      body(base + 1, std::integral_constant<int, 1>{});
      body(base + 2, std::integral_constant<int, 2>{});
      body(base + 3, std::integral_constant<int, 3>{});
    }
    cp_async_wait_group<0>();
  } else if (tid == U_PRODUCERS) {
    for (int step = 0; step < n_steps && ok; ++step) {
      const int s = step % STAGES, use = step / STAGES;
      if (!mbar_wait_bounded(&bars.full[s], use & 1)) { ok = false; break; }
      umma::fence_after_sync();
      if (tr != nullptr && step < 8) { tr[2 * (100 + 2 * step)] = 0; tr[2 * (100 + 2 * step) + 1] = (unsigned long long)clock64(); }
      issue(stages + (size_t)s * stage_bytes, step);
      umma::commit(&bars.empty[s]);
      if (tr != nullptr && step < 8) { tr[2 * (101 + 2 * step)] = 0; tr[2 * (101 + 2 * step) + 1] = (unsigned long long)clock64(); }
    }
    umma::commit(&bars.done);
  }
  return ok;
}

// ---- gate/up + SwiGLU ---------------------------------------------------------------------------

constexpr int GU_STAGES = 3;
constexpr uint32_t GU_STAGE_BYTES = 2 * A_TILE_BYTES + B_TILE_BYTES;  // 64 KB

__global__ void __launch_bounds__(U_THREADS, 1) k_umma_gateup(GroupedParams p) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) PipeBars bars;
  __shared__ uint32_t s_tmem;
  const int tile = blockIdx.y;
  if (tile >= *p.n_tiles) return;
  unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int e = p.tile_expert[tile], row0 = p.tile_row0[tile], rows_valid = p.tile_rows[tile];
  const int n_eff = (rows_valid + 15) & ~15;
  const int f0 = blockIdx.x * UM;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rb = p.ne / 256 * (int)Q4K_BLOCK_BYTES;
  const bool shared_seg = e >= p.n_expert;

  if (tid == 0) {
    for (int s = 0; s < GU_STAGES; ++s) {
      mbar_init(&bars.full[s], U_PRODUCERS / 32);
      mbar_init(&bars.empty[s], 1);
    }
    mbar_init(&bars.done, 1);
    mbar_fence_init();
  }
  if (warp == 8) umma::tmem_alloc(&s_tmem, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = s_tmem;

  // producer identity: role 0 = gate rows, role 1 = up rows; every producer also owns a token row
  const int role = (tid >> 7) & 1, wrow = tid & 127;
  const uint8_t* wbase = role == 0 ? (shared_seg ? p.sh_gate : p.gate + (size_t)e * p.gate_stride)
                                   : (shared_seg ? p.sh_up : p.up + (size_t)e * p.up_stride);
  const uint8_t* wrow_ptr = wbase + (size_t)(f0 + wrow) * rb;
  const __half* tok_tile = p.xg + (size_t)row0 * p.ne;
  const uint32_t idesc = umma::idesc_f16_f32(UM, n_eff);

  // Raw bytes of one whole 256-weight block of this row (header + 128 code bytes) are fetched a
  // block ahead, i.e. four K steps before they are unpacked: the rows of a tile are 1152 bytes
  // apart, every fetch is its own sector and takes a full memory latency.
  uint4 nxt_h, cur_h, nxt_q[8], cur_q[8];
  auto fetch_block = [&](int blk) {
    const uint8_t* bp = wrow_ptr + (size_t)blk * Q4K_BLOCK_BYTES;
    nxt_h = __ldg(reinterpret_cast<const uint4*>(bp));
#pragma unroll
    for (int i = 0; i < 8; ++i) nxt_q[i] = __ldg(reinterpret_cast<const uint4*>(bp + 16 + 16 * i));
  };
  fetch_block(0);

  auto unpack = [&](unsigned char* st, int step, auto jc) {
    constexpr int j = decltype(jc)::value;
    unsigned char* tA = st + (size_t)role * A_TILE_BYTES;
    if (j == 0) {
      cur_h = nxt_h;
#pragma unroll
      for (int i = 0; i < 8; ++i) cur_q[i] = nxt_q[i];
      if ((step >> 2) + 1 < p.ne / 256) fetch_block((step >> 2) + 1);
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
  };
  auto issue = [&](unsigned char* st, int step) {
    unsigned char* tB = st + 2 * A_TILE_BYTES;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint64_t bd = umma::smem_desc_k_major_swz128(tB, k);
      umma::mma_f16(tmem, umma::smem_desc_k_major_swz128(st, k), bd, idesc, step > 0 || k > 0);
      umma::mma_f16(tmem + 256, umma::smem_desc_k_major_swz128(st + A_TILE_BYTES, k), bd, idesc, step > 0 || k > 0);
    }
  };
  auto copy_b = [&](unsigned char* st, int step) {
    copy_token_tile(st + 2 * A_TILE_BYTES, tok_tile + (size_t)step * UK, p.ne, rows_valid, tid);
  };
  bool ok = run_pipeline<GU_STAGES>(bars, stages, GU_STAGE_BYTES, p.ne / UK, copy_b, unpack, issue,
                                    (blockIdx.x == 0 && blockIdx.y == 0) ? p.trace : nullptr);

  // epilogue: producers drain the two accumulators
  if (tid < U_PRODUCERS) {
    if (ok) ok = mbar_wait_bounded(&bars.done, 0);
    umma::fence_after_sync();
    if (ok) {
      const int lane_grp = warp & 3, col_half = warp >> 2;
      const int f = f0 + lane_grp * 32 + lane;
      const int fpos = kperm(f);
      for (int c0 = col_half * 128; c0 < min(n_eff, col_half * 128 + 128); c0 += 32) {
        float g[32], u[32];
        const uint32_t ta = tmem + ((uint32_t)(lane_grp * 32) << 16) + (uint32_t)c0;
        umma::ld_32x32(ta, g);
        umma::ld_32x32(ta + 256, u);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int n = c0 + i;
          if (n < rows_valid) {
            const float gv = g[i] * W_POSTSCALE, uv = u[i] * W_POSTSCALE;
            const float a = (gv / (1.0f + __expf(-gv))) * uv;
            p.act[(size_t)(row0 + n) * p.nff + fpos] = __float2half_rn(fminf(fmaxf(a, -65504.f), 65504.f));
          }
        }
      }
    }
  }
  if (!ok && lane == 0) atomicExch(&p.status->timeout, 5);
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 8) umma::tmem_dealloc(tmem, 512);
}

// ---- down ---------------------------------------------------------------------------------------------

constexpr int DN_STAGES = 4;
constexpr uint32_t DN_STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;  // 48 KB

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
  unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int e = p.tile_expert[tile], row0 = p.tile_row0[tile], rows_valid = p.tile_rows[tile];
  const int n_eff = (rows_valid + 15) & ~15;
  const int i0 = blockIdx.x * UM;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int drb = p.nff / 256 * (int)Q6K_BLOCK_BYTES;
  const bool shared_seg = e >= p.n_expert;

  if (tid == 0) {
    for (int s = 0; s < DN_STAGES; ++s) {
      mbar_init(&bars.full[s], U_PRODUCERS / 32);
      mbar_init(&bars.empty[s], 1);
    }
    mbar_init(&bars.done, 1);
    mbar_fence_init();
  }
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
  const __half* tok_tile = p.act + (size_t)row0 * p.nff;
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

  auto unpack = [&](unsigned char* st, int step, auto) {
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
  };
  auto issue = [&](unsigned char* st, int step) {
#pragma unroll
    for (int k = 0; k < 4; ++k)
      umma::mma_f16(tmem, umma::smem_desc_k_major_swz128(st, k), umma::smem_desc_k_major_swz128(st + A_TILE_BYTES, k), idesc,
                    step > 0 || k > 0);
  };
  auto copy_b = [&](unsigned char* st, int step) {
    copy_token_tile(st + A_TILE_BYTES, tok_tile + (size_t)step * UK, p.nff, rows_valid, tid);
  };
  bool ok = run_pipeline<DN_STAGES>(bars, stages, DN_STAGE_BYTES, p.nff / UK, copy_b, unpack, issue, nullptr);

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
  if (!ok && lane == 0) atomicExch(&p.status->timeout, 6);
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 8) umma::tmem_dealloc(tmem, 256);
}

}  // namespace

bool umma_grouped_supported(int ne, int nff) { return ne % 256 == 0 && nff % 256 == 0 && ne % UM == 0 && nff % UM == 0; }

int umma_tile_rows() { return UN; }

int32_t launch_umma_grouped(infr_cuda_ctx* ctx, const GroupedParams& p, int max_tiles) {
  const size_t smem_gu = 1024 + (size_t)GU_STAGES * GU_STAGE_BYTES;
  const size_t smem_dn = 1024 + (size_t)DN_STAGES * DN_STAGE_BYTES;
  cudaError_t e = ensure_smem(reinterpret_cast<const void*>(k_umma_gateup), smem_gu);
  if (e == cudaSuccess) e = ensure_smem(reinterpret_cast<const void*>(k_umma_down), smem_dn);
  if (e != cudaSuccess) return check_cuda(ctx, e, "umma grouped smem attribute");
  k_umma_gateup<<<dim3(p.nff / UM, max_tiles), U_THREADS, smem_gu, ctx->stream>>>(p);
  k_umma_down<<<dim3(p.ne / UM, max_tiles), U_THREADS, smem_dn, ctx->stream>>>(p);
  ctx->launches += 2;
  return check_cuda(ctx, cudaGetLastError(), "umma grouped launch");
}

}  // namespace infr
