// Small-m (decode) expert FFN: fused dequant-GEMV directly on GGUF Q4_K / Q6_K blocks.
//
//   k_decode_gateup : act[p, f] = silu(W_gate[e_p][f,:]·x) * (W_up[e_p][f,:]·x)      (Q4_K banks)
//   k_decode_down   : dst[r, i] = Σ_slot w_slot · (W_down[e_slot][i,:]·act[slot,:])  (Q6_K bank)
//                     (+ shared expert as one more slot, sigmoid-gated or plain)
//
// Reference: CPU stages B-E, crates/infr-cpu/src/lib.rs:4051-4303 (mat-vec = dequantised row ·
// activation, crates/infr-cpu/src/moe.rs:142-173; SwiGLU crates/infr-cpu/src/kernels.rs:6666-6683;
// rank-ordered weighted sum lib.rs:4287-4303; shared expert lib.rs:3336-3356).  Vulkan twins:
// shaders/native_gemv_id_multi.comp + silu_mul.comp + moe_accumulate_shared.comp, i.e. five
// dispatches where this file has two kernels.
//
// Data movement: only the routed experts' rows are touched, once.  Each CTA pulls its contiguous
// slab of rows with 1-D bulk async copies (TMA, never multicast) into shared memory, all issued
// up front so every SM has its whole share in flight, and lanes unpack blocks in registers:
// a 4-bit (6-bit) code becomes the float 1 + n/16 (1 + q/64) with one byte-permute, products
// are packed f32x2 fmas, and row sums finish with warp shuffles.
#include "kernels.cuh"

namespace infr {

namespace {

constexpr int GU_WARPS = 16;  // rows per chunk and role: one per warp
constexpr int GU_THREADS = GU_WARPS * 32;
constexpr int GU_MAX_CHUNKS = 4;
constexpr int GU_XQPITCH = 144;  // bytes per 64-element group of fixed-point x: 64 low limbs, 64 high limbs, pad

constexpr int DN_MAX_WARPS = 24;
constexpr int DN_MAX_SLOTS = 33;  // n_used ≤ 32 plus the shared expert

__device__ __forceinline__ bool in_band(const DecodeParams& p, int e) {
  return p.ep_n == 0 || ((uint32_t)e >= p.ep_lo && (uint32_t)e < p.ep_lo + p.ep_n);
}

// ---------------------------------------------------------------------------------------------
// gate/up + SwiGLU
// ---------------------------------------------------------------------------------------------
// One CTA = one (token, slot) pair x one tile of TR = 16*n_chunks output features, for both roles.
// Shared memory: n_chunks x { 16 gate rows | 16 up rows }, one mbarrier per chunk, then the
// token's activations.  Sixteen warps keep four resident per scheduler: the unpack is a chain of
// dependent integer ops and only other warps hide its latency.
// Lane L owns the 64-element groups g = L, L+32, ... of the input (for ne = 2048 exactly one, so
// its 64 activations stay in registers for the whole tile).
template <int NG>
__global__ void __launch_bounds__(GU_THREADS, 2) k_decode_gateup(DecodeParams p, int n_chunks) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t s_bar[GU_MAX_CHUNKS];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rb = p.ne / 256 * (int)Q4K_BLOCK_BYTES;  // bytes per weight row
  const int TR = GU_WARPS * n_chunks;
  const int tiles = p.nff / TR, sh_tiles = p.sh_ff / TR;
  const int n_routed_jobs = p.rows * p.n_used * tiles;

  const uint32_t chunk_bytes = (uint32_t)GU_WARPS * rb;  // per role
  auto issue_copies = [&](const uint8_t* gs, const uint8_t* us) {
    for (int c = 0; c < n_chunks; ++c) {
      mbar_arrive_expect_tx(&s_bar[c], 2 * chunk_bytes);
      unsigned char* dstc = smem + (size_t)c * 2 * chunk_bytes;
      bulk_g2s(dstc, gs + (size_t)c * chunk_bytes, chunk_bytes, &s_bar[c]);
      bulk_g2s(dstc + chunk_bytes, us + (size_t)c * chunk_bytes, chunk_bytes, &s_bar[c]);
    }
  };
  if (tid == 0) {
    for (int c = 0; c < n_chunks; ++c) mbar_init(&s_bar[c], 1);
    mbar_fence_init();
  }

  const bool routed = (int)blockIdx.x < n_routed_jobs;
  int pair = 0, tile, r;
  float* act_out;
  if (!routed) {
    // the shared expert's rows do not depend on routing: start fetching before the router is done
    const int jb = blockIdx.x - n_routed_jobs;
    r = jb / sh_tiles;
    tile = jb % sh_tiles;
    act_out = p.act + (size_t)p.rows * p.n_used * p.nff + (size_t)r * p.sh_ff + tile * TR;
    if (tid == 0) issue_copies(p.sh_gate + (size_t)tile * TR * rb, p.sh_up + (size_t)tile * TR * rb);
  } else {
    pair = blockIdx.x / tiles;
    tile = blockIdx.x % tiles;
    r = pair / p.n_used;
    act_out = p.act + (size_t)pair * p.nff + tile * TR;
  }

  unsigned long long* tr = (blockIdx.x == 0) ? p.trace : nullptr;
  trace_stamp(tr, 16);
  pdl_wait();     // ids and x come from kernels earlier in the stream
  trace_stamp(tr, 17);
  pdl_trigger();  // only now: the next kernel reads ids as soon as it starts

  int e_sel = routed ? __ldcg(p.ids + pair) : 0;  // L2 read: written by an overlapping earlier kernel
  // The token's activations arrive as 16-bit fixed point (two signed 8-bit limbs per element,
  // made by the router kernel): 64 low limbs then 64 high limbs per 64-element group.  Requested
  // before the routing result is used so that both reads are in flight together.
  const int n_groups = p.ne / 64;
  unsigned char* s_xq = smem + (size_t)n_chunks * 2 * chunk_bytes;  // [group][144]
  const bool stage_on = tid < p.ne / 16;  // ne <= 8192: one 16-byte piece of each limb array per thread
  uint4 xa = make_uint4(0u, 0u, 0u, 0u), xb = xa;
  if (stage_on) {
    xa = __ldcg(reinterpret_cast<const uint4*>(p.xq_lo + (size_t)r * p.ne) + tid);
    xb = __ldcg(reinterpret_cast<const uint4*>(p.xq_hi + (size_t)r * p.ne) + tid);
  }
  const float q_scale = __ldcg(p.xscale + r);
  if (routed) {
    int e = e_sel;
    if (e < 0 || e >= p.n_expert) {
      if (tid == 0) p.status->bad_index = 1;
      e = min(max(e, 0), p.n_expert - 1);
    }
    if (!in_band(p, e)) return;
    if (tid == 0)
      issue_copies(p.gate + (size_t)e * p.gate_stride + (size_t)tile * TR * rb,
                   p.up + (size_t)e * p.up_stride + (size_t)tile * TR * rb);
  }
  if (stage_on) {
    unsigned char* g = s_xq + (size_t)(tid >> 2) * GU_XQPITCH + (tid & 3) * 16;
    *reinterpret_cast<uint4*>(g) = xa;
    *reinterpret_cast<uint4*>(g + 64) = xb;
  }

  __syncthreads();  // limbs staged, barrier init visible to all waiters
  trace_stamp(tr, 18);
  int xl[16], xh[16];
  float sx0 = 0.f, sx1 = 0.f;
  auto load_x = [&](int g) {
    const uint4* src = reinterpret_cast<const uint4*>(s_xq + (size_t)g * GU_XQPITCH);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 a = src[i], b = src[4 + i];
      xl[4 * i + 0] = (int)a.x; xl[4 * i + 1] = (int)a.y; xl[4 * i + 2] = (int)a.z; xl[4 * i + 3] = (int)a.w;
      xh[4 * i + 0] = (int)b.x; xh[4 * i + 1] = (int)b.y; xh[4 * i + 2] = (int)b.z; xh[4 * i + 3] = (int)b.w;
    }
    int l0 = 0, h0 = 0, l1 = 0, h1 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      l0 = __dp4a(0x01010101, xl[i], l0); h0 = __dp4a(0x01010101, xh[i], h0);
      l1 = __dp4a(0x01010101, xl[8 + i], l1); h1 = __dp4a(0x01010101, xh[8 + i], h1);
    }
    sx0 = (float)(h0 * 256 + l0);
    sx1 = (float)(h1 * 256 + l1);
  };
  if (NG == 1) {
    if (lane < n_groups) load_x(lane);
  }

  bool ok = true;
  for (int c = 0; c < n_chunks; ++c) {
    if (!mbar_wait_bounded(&s_bar[c], 0)) { ok = false; break; }
    trace_stamp(tr, 19 + c);
    const unsigned char* grow = smem + (size_t)c * 2 * chunk_bytes + (size_t)warp * rb;
    const unsigned char* urow = grow + chunk_bytes;
    float gsum = 0.f, usum = 0.f;
#pragma unroll
    for (int t = 0; t < NG; ++t) {
      const int g = lane + 32 * t;
      if (g < n_groups) {
        if (NG > 1) load_x(g);
        const int blk = g >> 2, j = g & 3;
        const uint4 gh = *reinterpret_cast<const uint4*>(grow + blk * Q4K_BLOCK_BYTES);
        const uint4 uh = *reinterpret_cast<const uint4*>(urow + blk * Q4K_BLOCK_BYTES);
        uint32_t gq[8], uq[8];
        {
          const uint4 a = *reinterpret_cast<const uint4*>(grow + blk * Q4K_BLOCK_BYTES + 16 + 32 * j);
          const uint4 b = *reinterpret_cast<const uint4*>(grow + blk * Q4K_BLOCK_BYTES + 32 + 32 * j);
          gq[0] = a.x; gq[1] = a.y; gq[2] = a.z; gq[3] = a.w; gq[4] = b.x; gq[5] = b.y; gq[6] = b.z; gq[7] = b.w;
          const uint4 c4 = *reinterpret_cast<const uint4*>(urow + blk * Q4K_BLOCK_BYTES + 16 + 32 * j);
          const uint4 d4 = *reinterpret_cast<const uint4*>(urow + blk * Q4K_BLOCK_BYTES + 32 + 32 * j);
          uq[0] = c4.x; uq[1] = c4.y; uq[2] = c4.z; uq[3] = c4.w; uq[4] = d4.x; uq[5] = d4.y; uq[6] = d4.z; uq[7] = d4.w;
        }
        gsum += q4k_dot64_i8(gh, gq, xl, xh, sx0, sx1, j);
        usum += q4k_dot64_i8(uh, uq, xl, xh, sx0, sx1, j);
      }
    }
    gsum = warp_sum(gsum) * q_scale;
    usum = warp_sum(usum) * q_scale;
    if (lane == 0) {
      const float s = gsum / (1.0f + __expf(-gsum));
      act_out[c * GU_WARPS + warp] = s * usum;
    }
  }
  trace_stamp(tr, 23);
  if (!ok) {
    // a copy never signalled: report and make sure nothing is still landing in this CTA's
    // shared memory before it is handed to another CTA
    if (lane == 0) atomicExch(&p.status->timeout, 1);
    for (int c = 0; c < n_chunks; ++c) (void)mbar_wait_bounded(&s_bar[c], 0);
  }
}

// ---------------------------------------------------------------------------------------------
// down + weighted combine (+ shared expert)
// ---------------------------------------------------------------------------------------------
// One CTA = one token x TI consecutive output features x every slot, so the sum over slots never
// leaves the CTA.  Shared memory: per slot TI rows of the expert's down matrix (one bulk copy and
// one mbarrier per slot) and the slot's activation vector.
// Lane mapping inside a row: unit u = (block b, half h, word lw) covers the 16 elements
// 256b + 128h + 32q + 4lw + i (q, i = 0..3): three 32-bit words of codes, four scales.
//
// Q6_K blocks are 210 bytes, so odd blocks start 2 bytes off a word boundary: words are fetched
// as two aligned loads and a funnel shift.
__device__ __forceinline__ uint32_t lds_u32_unaligned(const unsigned char* base, uint32_t off) {
  const uint32_t a = off & ~3u;
  const uint32_t lo = *reinterpret_cast<const uint32_t*>(base + a);
  const uint32_t hi = *reinterpret_cast<const uint32_t*>(base + a + 4);
  return __funnelshift_r(lo, hi, (off & 3u) * 8);
}

__global__ void __launch_bounds__(DN_MAX_WARPS * 32, 1) k_decode_down(DecodeParams p, int TI) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t s_bar[DN_MAX_SLOTS];
  __shared__ float s_w[DN_MAX_SLOTS];
  __shared__ int s_on[DN_MAX_SLOTS];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x, nwarps = nthreads >> 5;
  const int nb = p.nff / 256;                    // blocks per routed row
  const int drb = nb * (int)Q6K_BLOCK_BYTES;     // bytes per routed row
  const bool has_sh = p.sh_down != nullptr;
  const int sh_nb = p.sh_ff / 256, sh_drb = sh_nb * (int)Q6K_BLOCK_BYTES;
  const int n_slots = p.n_used + (has_sh ? 1 : 0);
  const int tiles = p.ne / TI;
  const int r = blockIdx.x / tiles, i0 = (blockIdx.x % tiles) * TI;

  // shared-memory carve-up: weights per slot, activations per slot, weighted partial outputs
  const uint32_t slab = (uint32_t)TI * drb, sh_slab = (uint32_t)TI * sh_drb;
  const uint32_t slab_pad = (uint32_t)align_up(slab + 8, 16), sh_slab_pad = (uint32_t)align_up(sh_slab + 8, 16);
  unsigned char* s_wt = smem;
  float* s_act = reinterpret_cast<float*>(smem + (size_t)p.n_used * slab_pad + (has_sh ? sh_slab_pad : 0));
  float* s_part = s_act + (size_t)p.n_used * p.nff + (has_sh ? p.sh_ff : 0);  // [n_slots][TI]

  // The routing result was complete before this kernel could start (the gate/up kernel releases
  // its dependents only after it has itself waited for the router), so the weight slabs are
  // requested right away and stream in while the gate/up kernel is still running.
  unsigned long long* tr = (blockIdx.x == 0) ? p.trace : nullptr;
  trace_stamp(tr, 32);
  pdl_trigger();
  if (tid < n_slots) {
    const int s = tid;
    if (s < p.n_used) {
      int e = __ldcg(p.ids + r * p.n_used + s);
      e = min(max(e, 0), p.n_expert - 1);
      s_on[s] = in_band(p, e) ? e + 1 : 0;
      s_w[s] = __ldcg(p.wts + r * p.n_used + s);
    } else {
      s_on[s] = 1;
      s_w[s] = p.sh_logit ? 1.0f / (1.0f + __expf(-__ldcg(p.sh_logit + r))) : 1.0f;
    }
    // each slot's barrier and copy are set up by the slot's own thread
    mbar_init(&s_bar[s], 1);
    mbar_fence_init();
    if (s_on[s]) {
      if (s < p.n_used) {
        mbar_arrive_expect_tx(&s_bar[s], slab);
        bulk_g2s(s_wt + (size_t)s * slab_pad, p.down + (size_t)(s_on[s] - 1) * p.down_stride + (size_t)i0 * drb, slab,
                 &s_bar[s]);
      } else {
        mbar_arrive_expect_tx(&s_bar[s], sh_slab);
        bulk_g2s(s_wt + (size_t)p.n_used * slab_pad, p.sh_down + (size_t)i0 * sh_drb, sh_slab, &s_bar[s]);
      }
    }
  }
  trace_stamp(tr, 33);
  pdl_wait();  // the activations come from the gate/up kernel
  trace_stamp(tr, 34);
  // activations of this token: routed slots then the shared expert; loads are issued four deep
  // before the first store so that their L2 latencies overlap
  {
    const float4* a_src = reinterpret_cast<const float4*>(p.act + (size_t)r * p.n_used * p.nff);
    const float4* sh_src = reinterpret_cast<const float4*>(p.act + (size_t)p.rows * p.n_used * p.nff + (size_t)r * p.sh_ff);
    const int n4 = p.n_used * p.nff / 4, tot4 = n4 + (has_sh ? p.sh_ff / 4 : 0);
    float4* d4 = reinterpret_cast<float4*>(s_act);
    for (int base = tid; base < tot4; base += 4 * nthreads) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = base + u * nthreads;
        if (i < tot4) v[u] = __ldcg(i < n4 ? a_src + i : sh_src + (i - n4));
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = base + u * nthreads;
        if (i < tot4) d4[i] = v[u];
      }
    }
  }
  __syncthreads();
  trace_stamp(tr, 35);

  // A warp task = one slot x one group of RPG rows: the slot's activations stay in registers
  // while the rows of the group stream past them.
  const int RPG = TI < 8 ? TI : 8, RG = TI / RPG;
  const int n_tasks = n_slots * RG;
  bool ok = true;
  for (int task = warp; task < n_tasks && ok; task += nwarps) {
    const int s = task / RG, row0 = (task % RG) * RPG;
    float acc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] = 0.f;
    if (s_on[s]) {
      if (!mbar_wait_bounded(&s_bar[s], 0)) { ok = false; break; }
      const bool shared_slot = s >= p.n_used;
      const int row_bytes_s = shared_slot ? sh_drb : drb;
      const int units = (shared_slot ? sh_nb : nb) * 16;
      const unsigned char* wt = s_wt + (shared_slot ? (size_t)p.n_used * slab_pad : (size_t)s * slab_pad);
      const float* a = s_act + (shared_slot ? (size_t)p.n_used * p.nff : (size_t)s * p.nff);
      for (int u = lane; u < units; u += 32) {
        const int b = u >> 4, h = (u >> 3) & 1, lw = u & 7;
        // The unit's 16 activations in 16-bit fixed point with the unit's own scale (X = 256 hi + lo,
        // signed 8-bit limbs, four elements per word like the code words): products with the 6-bit
        // codes are exact integer dot products, and the unpack stays off the half-rate logic pipe.
        const float* ab = a + b * 256 + h * 128 + lw * 4;
        float4 av[4];
        float amax = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          av[q] = *reinterpret_cast<const float4*>(ab + 32 * q);
          amax = fmaxf(fmaxf(fabsf(av[q].x), fabsf(av[q].y)), fmaxf(amax, fmaxf(fabsf(av[q].z), fabsf(av[q].w))));
        }
        const float a_inv = amax > 0.f ? 32639.f / amax : 0.f, a_scale = amax / 32639.f;
        int xl[4], xh[4], s32[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int X[4] = {__float2int_rn(av[q].x * a_inv), __float2int_rn(av[q].y * a_inv), __float2int_rn(av[q].z * a_inv),
                            __float2int_rn(av[q].w * a_inv)};
          uint32_t lo = 0, hi = 0;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const int hh = (X[t] + 128) >> 8, ll = X[t] - (hh << 8);
            lo |= (uint32_t)(ll & 0xFF) << (8 * t);
            hi |= (uint32_t)(hh & 0xFF) << (8 * t);
          }
          xl[q] = (int)lo;
          xh[q] = (int)hi;
          s32[q] = 32 * ((X[0] + X[1]) + (X[2] + X[3]));
        }
        const uint32_t boff = (uint32_t)b * Q6K_BLOCK_BYTES;
        const uint32_t sel = (lw >> 2) ? 0x7531u : 0x6420u;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          if (q < RPG) {
            // offsets are taken from the 16-byte aligned slab base: rows of an odd block count
            // start 2 bytes off a word boundary too
            const uint32_t ro = (uint32_t)(row0 + q) * row_bytes_s + boff;
            const uint32_t A = lds_u32_unaligned(wt, ro + 64 * h + 4 * lw);
            const uint32_t B = lds_u32_unaligned(wt, ro + 64 * h + 32 + 4 * lw);
            const uint32_t H = lds_u32_unaligned(wt, ro + 128 + 32 * h + 4 * lw);
            const uint32_t S0 = lds_u32_unaligned(wt, ro + 192 + 8 * h);
            const uint32_t S1 = lds_u32_unaligned(wt, ro + 196 + 8 * h);
            const float d = f16_bits_to_f32(*reinterpret_cast<const unsigned short*>(wt + ro + 208));
            // 6-bit codes of the four quadrants, one per byte
            const uint32_t cs[4] = {(A & 0x0F0F0F0Fu) | ((H << 4) & 0x30303030u), (B & 0x0F0F0F0Fu) | ((H << 2) & 0x30303030u),
                                    ((A >> 4) & 0x0F0F0F0Fu) | (H & 0x30303030u), ((B >> 4) & 0x0F0F0F0Fu) | ((H >> 2) & 0x30303030u)};
            // scales of the four quadrants: bytes (lw>>2) + 2q of the eight scale bytes of this half
            const uint32_t sc4 = __byte_perm(S0, S1, sel);
            long long part = 0;
#pragma unroll
            for (int qd = 0; qd < 4; ++qd) {
              // sum (q - 32) X = 256 * dot(codes, hi) + dot(codes, lo) - 32 * sum X   (|.| < 2^24)
              const int t = __dp4a((int)cs[qd], xh[qd], 0) * 256 + __dp4a((int)cs[qd], xl[qd], 0) - s32[qd];
              part += (long long)(int)(signed char)((sc4 >> (8 * qd)) & 0xFFu) * t;
            }
            acc[q] = fmaf(d * a_scale, (float)part, acc[q]);
          }
        }
      }
    }
    // eight row sums across 32 lanes with nine shuffles: halve the value set at every step
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float send = (lane & 16) ? acc[i] : acc[i + 4];
      const float keep = (lane & 16) ? acc[i + 4] : acc[i];
      acc[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 16);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float send = (lane & 8) ? acc[i] : acc[i + 2];
      const float keep = (lane & 8) ? acc[i + 2] : acc[i];
      acc[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 8);
    }
    {
      const float send = (lane & 4) ? acc[0] : acc[1];
      const float keep = (lane & 4) ? acc[1] : acc[0];
      acc[0] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 4);
    }
    acc[0] += __shfl_xor_sync(0xFFFFFFFFu, acc[0], 2);
    acc[0] += __shfl_xor_sync(0xFFFFFFFFu, acc[0], 1);
    const int q_mine = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
    if ((lane & 3) == 0 && q_mine < RPG) s_part[s * TI + row0 + q_mine] = s_w[s] * acc[0];
  }
  if (!ok) {
    if (lane == 0) atomicExch(&p.status->timeout, 2);
    for (int s = 0; s < n_slots; ++s)
      if (s_on[s]) (void)mbar_wait_bounded(&s_bar[s], 0);
  }
  __syncthreads();
  trace_stamp(tr, 36);
  // weighted sum over slots in rank order, the shared expert last (the CPU's order)
  if (tid < TI) {
    float o = 0.f;
    for (int s = 0; s < n_slots; ++s) o += s_part[s * TI + tid];
    if (p.residual != nullptr) o += __ldcg(p.residual + (size_t)r * p.ne + i0 + tid);  // MoeFfn -> Add
    p.dst[(size_t)r * p.ne + i0 + tid] = o;
  }
}

size_t gateup_smem(int ne, int n_chunks) {
  return (size_t)n_chunks * 2 * GU_WARPS * (ne / 256 * Q4K_BLOCK_BYTES) + (size_t)(ne / 64) * GU_XQPITCH;
}

int pick_chunks(int ne, int nff, int sh_ff) {
  for (int c = 2; c >= 1; c >>= 1) {
    const int TR = GU_WARPS * c;
    if (nff % TR) continue;
    if (sh_ff && sh_ff % TR) continue;
    if (gateup_smem(ne, c) <= 200 * 1024) return c;
  }
  return 0;
}

size_t down_smem(int TI, int nff, int sh_ff, int n_used) {
  const size_t slab = align_up((size_t)TI * (nff / 256 * Q6K_BLOCK_BYTES) + 8, 16);
  const size_t sh_slab = sh_ff ? align_up((size_t)TI * (sh_ff / 256 * Q6K_BLOCK_BYTES) + 8, 16) : 0;
  return (size_t)n_used * slab + sh_slab + ((size_t)n_used * nff + sh_ff) * sizeof(float) +
         (size_t)(n_used + 1) * TI * sizeof(float);
}

// TI rows per CTA: bulk copies need TI * row_bytes to be a multiple of 16 for both banks.
int pick_down_tile(int ne, int nff, int sh_ff, int n_used) {
  const int cands[] = {16, 8, 4};
  for (int TI : cands) {
    if (ne % TI) continue;
    if (((size_t)TI * (nff / 256) * Q6K_BLOCK_BYTES) % 16) continue;
    if (sh_ff && ((size_t)TI * (sh_ff / 256) * Q6K_BLOCK_BYTES) % 16) continue;
    if (down_smem(TI, nff, sh_ff, n_used) <= 200 * 1024) return TI;
  }
  return 0;
}

template <typename K, typename... Args>
cudaError_t launch_ex(K kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

}  // namespace

bool decode_ffn_supported(const infr_cuda_ctx*, int ne, int nff, int sh_ff, int n_used, std::string* why) {
  if (ne % 256 || nff % 256 || (sh_ff % 256)) {
    if (why) *why = "small-m path: ne, n_ff_exp and sh_ff must be multiples of 256";
    return false;
  }
  if (ne / 64 > 32 * 4) {
    if (why) *why = "small-m path: ne larger than 8192 is not covered";
    return false;
  }
  if (n_used + 1 > DN_MAX_SLOTS) {
    if (why) *why = "small-m path: n_used larger than 32 is not covered";
    return false;
  }
  if (!pick_chunks(ne, nff, sh_ff) || !pick_down_tile(ne, nff, sh_ff, n_used)) {
    if (why) *why = "small-m path: tile does not fit shared memory for these dims";
    return false;
  }
  return true;
}

int32_t launch_decode_ffn(infr_cuda_ctx* ctx, const DecodeParams& p, bool pdl, uint32_t stages) {
  const bool has_sh = p.sh_gate != nullptr;
  const int sh_ff = has_sh ? p.sh_ff : 0;
  const int n_chunks = pick_chunks(p.ne, p.nff, sh_ff);
  const int TI = pick_down_tile(p.ne, p.nff, sh_ff, p.n_used);
  if (!n_chunks || !TI) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "small-m path: tile does not fit shared memory");
  const int TR = GU_WARPS * n_chunks;
  const int jobs = p.rows * p.n_used * (p.nff / TR) + (has_sh ? p.rows * (sh_ff / TR) : 0);
  const size_t smem_gu = gateup_smem(p.ne, n_chunks);
  const int ng = (p.ne / 64 + 31) / 32;
  cudaError_t e = cudaSuccess;
  auto run_gu = [&](auto kern) {
    e = ensure_smem(reinterpret_cast<const void*>(kern), smem_gu);
    if (e != cudaSuccess) return e;
    return launch_ex(kern, dim3(jobs), dim3(GU_THREADS), smem_gu, ctx->stream, pdl, p, n_chunks);
  };
  if (stages & 2u) {
    if (ng == 1)
      e = run_gu(k_decode_gateup<1>);
    else if (ng == 2)
      e = run_gu(k_decode_gateup<2>);
    else
      e = run_gu(k_decode_gateup<4>);
    ctx->launches += 1;
    if (e != cudaSuccess) return check_cuda(ctx, e, "k_decode_gateup launch");
  }
  if (!(stages & 4u)) return INFR_CUDA_OK;

  const size_t smem_dn = down_smem(TI, p.nff, sh_ff, p.n_used);
  e = ensure_smem(reinterpret_cast<const void*>(k_decode_down), smem_dn);
  if (e != cudaSuccess) return check_cuda(ctx, e, "k_decode_down smem attribute");
  // one warp per (slot, group of up to 8 rows) when that fits, else the largest divisor
  const int n_tasks = (p.n_used + (has_sh ? 1 : 0)) * (TI > 8 ? TI / 8 : 1);
  int nw = 16;
  for (int c = DN_MAX_WARPS; c >= 8; --c)
    if (n_tasks % c == 0) { nw = c; break; }
  if (n_tasks < 8) nw = n_tasks < 4 ? 4 : n_tasks;
  e = launch_ex(k_decode_down, dim3(p.rows * (p.ne / TI)), dim3(nw * 32), smem_dn, ctx->stream, pdl, p, TI);
  ctx->launches += 1;
  return check_cuda(ctx, e, "k_decode_down launch");
}

}  // namespace infr
