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
// up front so every SM has its whole share in flight, and lanes unpack blocks in registers: the
// activations arrive as 16-bit fixed point in two signed 8-bit limbs, the 4-bit (6-bit) codes are
// masked in place and multiplied with integer dot-product instructions (exact integer sums), block
// scales are applied per 32 (16) elements in f32, and row sums finish with warp shuffles.
#include "kernels.cuh"

namespace infr {

namespace {

constexpr int GU_WARPS = 16;  // rows per chunk and role: one per warp
constexpr int GU_MAX_CHUNKS = 4;
constexpr int GU_XQPITCH = 144;  // bytes per 64-element group of fixed-point x: 64 low limbs, 64 high limbs, pad

constexpr int DN_MAX_WARPS = 24;
constexpr int DN_XPITCH = 36;     // words per 128-activation chunk and limb: four neighbouring chunks start in four 16-byte bank groups
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
__global__ void __maxnreg__(56) k_decode_gateup(DecodeParams p, int n_chunks) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t s_bar[GU_MAX_CHUNKS];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rb = p.ne / 256 * (int)Q4K_BLOCK_BYTES;  // bytes per weight row
  const int GW = blockDim.x >> 5;  // warps = weight rows per chunk and role
  const int TR = GW * n_chunks;
  const int tiles = p.nff / TR, sh_tiles = p.sh_ff / TR;
  const int n_routed_jobs = p.rows * p.n_used * tiles;

  const uint32_t chunk_bytes = (uint32_t)GW * rb;  // per role
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
  trace_extreme(p.trace, 40, false);
  trace_extreme(p.trace, 41, true);
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
    if (e < 0) return;  // a negative id marks a pair another rank serves
    if (e >= p.n_expert) {
      if (tid == 0) p.status->bad_index = 1;
      e = p.n_expert - 1;
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
  int sx0 = 0, sx1 = 0;
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
    sx0 = h0 * 256 + l0;
    sx1 = h1 * 256 + l1;
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
      // routed pairs: optional clamp, and with weight_before the pair's routing weight on both
      const float wp = (routed && p.weight_before) ? __ldcg(p.wts + pair) : 1.0f;
      act_out[c * GW + warp] = gated_act(p.act_kind, routed ? p.clamp : 0.f, wp * gsum, wp * usum);
    }
  }
  trace_stamp(tr, 23);
  trace_extreme(p.trace, 42, true);
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

__global__ void __maxnreg__(56) k_decode_down(DecodeParams p, int TI) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t s_bar[DN_MAX_SLOTS];
  __shared__ float s_w[DN_MAX_SLOTS];
  __shared__ float s_ds[DN_MAX_SLOTS];  // per-slot scale of the raw down output (Op::MoeFfn::down_scale)
  __shared__ int s_on[DN_MAX_SLOTS];
  __shared__ uint32_t s_off[DN_MAX_SLOTS];  // slab start inside its shared-memory slot

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x, nwarps = nthreads >> 5;
  const int nb = p.nff / 256;                    // blocks per routed row
  const int dbb = p.down_q4k ? (int)Q4K_BLOCK_BYTES : (int)Q6K_BLOCK_BYTES;  // bytes per 256-weight block of the down banks
  const int drb = nb * dbb;                      // bytes per routed row
  const bool has_sh = p.sh_down != nullptr;
  const int sh_nb = p.sh_ff / 256, sh_drb = sh_nb * dbb;
  const int n_slots = p.n_used + (has_sh ? 1 : 0);
  const int tiles = p.ne / TI;
  const int r = blockIdx.x / tiles, i0 = (blockIdx.x % tiles) * TI;

  // shared-memory carve-up: weights per slot, activations per slot, weighted partial outputs
  const uint32_t slab = (uint32_t)TI * drb, sh_slab = (uint32_t)TI * sh_drb;
  // A slab lands at the same offset inside a 128-byte line as its source has in global memory:
  // bulk copies whose two sides disagree modulo 128 run several times slower.
  const uint32_t slab_pad = (uint32_t)align_up(slab + 8, 128) + 128, sh_slab_pad = (uint32_t)align_up(sh_slab + 8, 128) + 128;
  unsigned char* s_wt = smem + ((128u - (smem_u32(smem) & 127u)) & 127u);
  // activations as 16-bit fixed point, one scale per 128-element chunk (= half a Q6_K block):
  // low limbs, high limbs (4 elements per word), chunk scales, integer sums per 16 elements
  const int n_act = p.n_used * p.nff + (has_sh ? p.sh_ff : 0), n_chunk = n_act / 128;
  uint32_t* s_xlo = reinterpret_cast<uint32_t*>(s_wt + (size_t)p.n_used * slab_pad + (has_sh ? sh_slab_pad : 0));  // [n_chunk][DN_XPITCH]
  uint32_t* s_xhi = s_xlo + n_chunk * DN_XPITCH;
  float* s_xsc = reinterpret_cast<float*>(s_xhi + n_chunk * DN_XPITCH);  // [n_chunk]
  int* s_s16 = reinterpret_cast<int*>(s_xsc + n_chunk);          // [n_chunk][8]
  float* s_part = reinterpret_cast<float*>(s_s16 + n_chunk * 8);  // [n_slots][TI]

  // The routing result was complete before this kernel could start (the gate/up kernel releases
  // its dependents only after it has itself waited for the router), so the weight slabs are
  // requested right away and stream in while the gate/up kernel is still running.
  unsigned long long* tr = (blockIdx.x == 0) ? p.trace : nullptr;
  trace_stamp(tr, 32);
  trace_extreme(p.trace, 43, true);
  pdl_trigger();
  if (tid < n_slots) {
    const int s = tid;
    if (s < p.n_used) {
      int e = __ldcg(p.ids + r * p.n_used + s);
      const bool mine = e >= 0;  // a negative id marks a pair another rank serves
      e = min(max(e, 0), p.n_expert - 1);
      s_on[s] = (mine && in_band(p, e)) ? e + 1 : 0;
      s_w[s] = p.weight_before ? 1.0f : __ldcg(p.wts + r * p.n_used + s);
      s_ds[s] = p.down_scale ? __ldg(p.down_scale + e) : 1.0f;
    } else {
      s_ds[s] = 1.0f;
      s_on[s] = 1;
      s_w[s] = p.sh_logit ? 1.0f / (1.0f + __expf(-__ldcg(p.sh_logit + r))) : 1.0f;
    }
    // each slot's barrier and copy are set up by the slot's own thread
    mbar_init(&s_bar[s], 1);
    mbar_fence_init();
    s_off[s] = 0;
    if (s_on[s]) {
      if (s < p.n_used) {
        const uint8_t* src = p.down + (size_t)(s_on[s] - 1) * p.down_stride + (size_t)i0 * drb;
        s_off[s] = (uint32_t)(reinterpret_cast<uintptr_t>(src) & 127u);
        mbar_arrive_expect_tx(&s_bar[s], slab);
        bulk_g2s(s_wt + (size_t)s * slab_pad + s_off[s], src, slab, &s_bar[s]);
      } else {
        const uint8_t* src = p.sh_down + (size_t)i0 * sh_drb;
        s_off[s] = (uint32_t)(reinterpret_cast<uintptr_t>(src) & 127u);
        mbar_arrive_expect_tx(&s_bar[s], sh_slab);
        bulk_g2s(s_wt + (size_t)p.n_used * slab_pad + s_off[s], src, sh_slab, &s_bar[s]);
      }
    }
  }
  trace_stamp(tr, 33);
  trace_cta(p.trace, 0);
  pdl_wait();  // the activations come from the gate/up kernel
  trace_stamp(tr, 34);
  trace_extreme(p.trace, 44, false);
  // activations of this token (routed slots, then the shared expert) -> fixed point.  One warp
  // per 128-element chunk: X = round(a * 32639 / max|a|), X = 256 hi + lo with signed 8-bit limbs.
  {
    const float* a_src = p.act + (size_t)r * p.n_used * p.nff;
    const float* sh_src = p.act + (size_t)p.rows * p.n_used * p.nff + (size_t)r * p.sh_ff;
    const int n_routed_chunk = p.n_used * p.nff / 128;
    for (int c0 = warp; c0 < n_chunk; c0 += 2 * nwarps) {
      // two chunks per pass so that their loads overlap
      const int c1 = c0 + nwarps;
      const float4 v0 = __ldcg(reinterpret_cast<const float4*>(c0 < n_routed_chunk ? a_src + (size_t)c0 * 128 : sh_src + (size_t)(c0 - n_routed_chunk) * 128) + lane);
      float4 v1 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c1 < n_chunk)
        v1 = __ldcg(reinterpret_cast<const float4*>(c1 < n_routed_chunk ? a_src + (size_t)c1 * 128 : sh_src + (size_t)(c1 - n_routed_chunk) * 128) + lane);
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int c = k ? c1 : c0;
        if (c >= n_chunk) break;
        const float4 v = k ? v1 : v0;
        const float m = warp_max(fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        const float inv = m > 0.f ? 32639.f / m : 0.f;
        const int X[4] = {__float2int_rn(v.x * inv), __float2int_rn(v.y * inv), __float2int_rn(v.z * inv), __float2int_rn(v.w * inv)};
        uint32_t lo, hi;
        pack_limbs4(X, lo, hi);
        s_xlo[c * DN_XPITCH + lane] = lo;
        s_xhi[c * DN_XPITCH + lane] = hi;
        int sx = (X[0] + X[1]) + (X[2] + X[3]);  // sum over the 16 elements held by four lanes
        sx += __shfl_xor_sync(0xFFFFFFFFu, sx, 1);
        sx += __shfl_xor_sync(0xFFFFFFFFu, sx, 2);
        if ((lane & 3) == 0) s_s16[c * 8 + (lane >> 2)] = sx;
        if (lane == 0) s_xsc[c] = m / 32639.f;
      }
    }
  }
  __syncthreads();
  trace_stamp(tr, 35);
  trace_cta(p.trace, 1);

  // A warp task = one slot x one group of up to 8 rows.  Lane = (row q = lane / 4, quarter u4 =
  // lane % 4): a lane walks whole half-blocks (128 weights: 64 B of low bits, 32 B of high bits,
  // 8 scales) of its row, four half-blocks of the row side by side across the quarter lanes.
  // Blocks are 210 bytes, so a row's bytes start 0 or 2 bytes off a word boundary: the lane reads
  // aligned words and funnel-shifts neighbouring pairs.
  const int RPG = TI < 8 ? TI : 8, RG = TI / RPG;
  const int n_tasks = n_slots * RG;
  const int q = lane >> 2, u4 = lane & 3;
  bool ok = true;
  for (int task = warp; task < n_tasks && ok; task += nwarps) {
    const int s = task / RG, row0 = (task % RG) * RPG;
    float acc = 0.f;
    if (s_on[s]) {
      if (!mbar_wait_bounded(&s_bar[s], 0)) { ok = false; break; }
      trace_stamp(tr, 37);
      trace_cta(p.trace, 2);
      trace_extreme(p.trace, 45, true);
      const bool shared_slot = s >= p.n_used;
      const int row_bytes_s = shared_slot ? sh_drb : drb;
      const int n_hb = (shared_slot ? sh_nb : nb) * 2;  // half-blocks per row
      const unsigned char* wt = s_wt + (shared_slot ? (size_t)p.n_used * slab_pad : (size_t)s * slab_pad) + s_off[s];
      const int chunk0 = shared_slot ? p.n_used * p.nff / 128 : s * (p.nff / 128);
      if (q < RPG && p.down_q4k) {
        // Q4_K rows (16-byte aligned): a lane walks 64-element groups (32 code bytes: low nibbles
        // = 32 elements, high nibbles = the next 32), four groups side by side across the quarter lanes
        const unsigned char* wrow = wt + (size_t)(row0 + q) * row_bytes_s;
        for (int g = u4; g < n_hb * 2; g += 4) {
          const int b = g >> 2, j = g & 3, chunk = chunk0 + (g >> 1);
          const uint4 hdr = *reinterpret_cast<const uint4*>(wrow + b * Q4K_BLOCK_BYTES);
          const uint4 qa = *reinterpret_cast<const uint4*>(wrow + b * Q4K_BLOCK_BYTES + 16 + 32 * j);
          const uint4 qb = *reinterpret_cast<const uint4*>(wrow + b * Q4K_BLOCK_BYTES + 32 + 32 * j);
          const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
          const uint4* xl = reinterpret_cast<const uint4*>(s_xlo + chunk * DN_XPITCH + (g & 1) * 16);
          const uint4* xh = reinterpret_cast<const uint4*>(s_xhi + chunk * DN_XPITCH + (g & 1) * 16);
          const int* s16 = s_s16 + chunk * 8 + (g & 1) * 4;
          int v[2];
#pragma unroll
          for (int hn = 0; hn < 2; ++hn) {  // low nibbles, then high nibbles
            int al = 0, ah = 0;
#pragma unroll
            for (int i4 = 0; i4 < 2; ++i4) {
              const uint4 l4 = xl[2 * hn + i4], h4 = xh[2 * hn + i4];
              const int c0 = (int)((qw[4 * i4 + 0] >> (4 * hn)) & 0x0F0F0F0Fu), c1 = (int)((qw[4 * i4 + 1] >> (4 * hn)) & 0x0F0F0F0Fu),
                        c2 = (int)((qw[4 * i4 + 2] >> (4 * hn)) & 0x0F0F0F0Fu), c3 = (int)((qw[4 * i4 + 3] >> (4 * hn)) & 0x0F0F0F0Fu);
              al = __dp4a(c0, (int)l4.x, al); ah = __dp4a(c0, (int)h4.x, ah);
              al = __dp4a(c1, (int)l4.y, al); ah = __dp4a(c1, (int)h4.y, ah);
              al = __dp4a(c2, (int)l4.z, al); ah = __dp4a(c2, (int)h4.z, ah);
              al = __dp4a(c3, (int)l4.w, al); ah = __dp4a(c3, (int)h4.w, ah);
            }
            v[hn] = ah * 256 + al;
          }
          uint32_t scp, mp;
          q4k_scale_min_pair(hdr.y, hdr.z, hdr.w, j, scp, mp);
          const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
          const float sx0 = (float)(s16[0] + s16[1]), sx1 = (float)(s16[2] + s16[3]);
          const float part = d * ((float)(scp & 0xFFu) * (float)v[0] + (float)(scp >> 8) * (float)v[1]) -
                             dmin * ((float)(mp & 0xFFu) * sx0 + (float)(mp >> 8) * sx1);
          acc = fmaf(s_xsc[chunk], part, acc);
        }
      } else if (q < RPG) {
        for (int hb = u4; hb < n_hb; hb += 4) {
          const int b = hb >> 1, h = hb & 1, chunk = chunk0 + hb;
          const uint32_t ro = (uint32_t)(row0 + q) * row_bytes_s + (uint32_t)b * Q6K_BLOCK_BYTES;
          const uint32_t sh = (ro & 3u) * 8;                 // 0 or 16
          const uint32_t* wq = reinterpret_cast<const uint32_t*>(wt + (ro & ~3u));  // aligned view of the block
          // aligned word j of the view covers block bytes 4j - (ro & 3) ..; block byte o starts in word o / 4
          auto word = [&](int o4) { return __funnelshift_r(wq[o4], wq[o4 + 1], sh); };  // bytes 4*o4 .. 4*o4+3 of the block
          const float d = f16_bits_to_f32(*reinterpret_cast<const unsigned short*>(wt + ro + 208));
          const uint32_t S0 = word(48 + 2 * h), S1 = word(49 + 2 * h);  // the half's eight int8 scales
          const uint4* xl = reinterpret_cast<const uint4*>(s_xlo + chunk * DN_XPITCH);
          const uint4* xh = reinterpret_cast<const uint4*>(s_xhi + chunk * DN_XPITCH);
          const int* s16 = s_s16 + chunk * 8;
          float part = 0.f;
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {  // l = 16 hf .. 16 hf + 15
            uint32_t c[4][4];               // codes [quadrant][word of four l values]
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) {
              const int i = 4 * hf + i4;
              const uint32_t A = word(16 * h + i), B = word(16 * h + 8 + i), H = word(32 + 8 * h + i);
              c[0][i4] = (A & 0x0F0F0F0Fu) | ((H << 4) & 0x30303030u);
              c[1][i4] = (B & 0x0F0F0F0Fu) | ((H << 2) & 0x30303030u);
              c[2][i4] = ((A >> 4) & 0x0F0F0F0Fu) | (H & 0x30303030u);
              c[3][i4] = ((B >> 4) & 0x0F0F0F0Fu) | ((H >> 2) & 0x30303030u);
            }
#pragma unroll
            for (int qd = 0; qd < 4; ++qd) {
              // the quadrant's 16 activations of this half: one 16-byte read per limb
              const uint4 l4 = xl[2 * qd + hf], h4 = xh[2 * qd + hf];
              int dlo = __dp4a((int)c[qd][0], (int)l4.x, 0), dhi = __dp4a((int)c[qd][0], (int)h4.x, 0);
              dlo = __dp4a((int)c[qd][1], (int)l4.y, dlo); dhi = __dp4a((int)c[qd][1], (int)h4.y, dhi);
              dlo = __dp4a((int)c[qd][2], (int)l4.z, dlo); dhi = __dp4a((int)c[qd][2], (int)h4.z, dhi);
              dlo = __dp4a((int)c[qd][3], (int)l4.w, dlo); dhi = __dp4a((int)c[qd][3], (int)h4.w, dhi);
              // scale group 2 qd + hf of the half: sum (code - 32) X = 256 dhi + dlo - 32 sum X
              const int g = 2 * qd + hf;
              const int t = dhi * 256 + dlo - 32 * s16[g];
              const uint32_t sw = g < 4 ? S0 : S1;
              const float sc = (float)(int)(signed char)((sw >> (8 * (g & 3))) & 0xFFu);
              part = fmaf(sc, (float)t, part);
            }
          }
          acc = fmaf(d * s_xsc[chunk], part, acc);
        }
      }
    }
    // the four quarter lanes of a row
    acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 1);
    acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 2);
    if (u4 == 0 && q < RPG) s_part[s * TI + row0 + q] = s_w[s] * (acc * s_ds[s]);  // s_ds = 1 (exact) without a down_scale
  }
  if (!ok) {
    if (lane == 0) atomicExch(&p.status->timeout, 2);
    for (int s = 0; s < n_slots; ++s)
      if (s_on[s]) (void)mbar_wait_bounded(&s_bar[s], 0);
  }
  __syncthreads();
  trace_stamp(tr, 36);
  trace_extreme(p.trace, 46, true);
  // weighted sum over slots in rank order, the shared expert last (the CPU's order)
  if (tid < TI) {
    float o = 0.f;
    for (int s = 0; s < n_slots; ++s) o += s_part[s * TI + tid];
    if (p.residual != nullptr) o += __ldcg(p.residual + (size_t)r * p.ne + i0 + tid);  // MoeFfn -> Add
    p.dst[(size_t)r * p.ne + i0 + tid] = o;
  }
}

size_t gateup_smem(int ne, int n_chunks, int gw = GU_WARPS) {
  return (size_t)n_chunks * 2 * gw * (ne / 256 * Q4K_BLOCK_BYTES) + (size_t)(ne / 64) * GU_XQPITCH;
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

size_t down_smem(int TI, int nff, int sh_ff, int n_used, size_t dbb) {
  const size_t slab = align_up((size_t)TI * (nff / 256 * dbb) + 8, 128) + 128;
  const size_t sh_slab = sh_ff ? align_up((size_t)TI * (sh_ff / 256 * dbb) + 8, 128) + 128 : 0;
  const size_t n_act = (size_t)n_used * nff + sh_ff;
  return 128 + (size_t)n_used * slab + sh_slab + (n_act / 128) * (2 * DN_XPITCH * 4 + 4 + 32) + (size_t)(n_used + 1) * TI * sizeof(float);
}

// TI rows per CTA: bulk copies need TI * row_bytes to be a multiple of 16 for both banks.
int pick_down_tile(int ne, int nff, int sh_ff, int n_used, size_t dbb) {
  const int cands[] = {16, 8, 4};
  for (int TI : cands) {
    if (ne % TI) continue;
    if (((size_t)TI * (nff / 256) * dbb) % 16) continue;
    if (sh_ff && ((size_t)TI * (sh_ff / 256) * dbb) % 16) continue;
    if (down_smem(TI, nff, sh_ff, n_used, dbb) <= 200 * 1024) return TI;
  }
  return 0;
}

}  // namespace

bool decode_ffn_supported(const infr_cuda_ctx*, int ne, int nff, int sh_ff, int n_used, BankTypes bt, std::string* why) {
  if (!bt.tuned()) return anyfmt_decode_supported(ne, nff, sh_ff, n_used, bt, why);
  const bool down_q4k = bt.down_q4k();
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
  if (!pick_chunks(ne, nff, sh_ff) || !pick_down_tile(ne, nff, sh_ff, n_used, down_q4k ? Q4K_BLOCK_BYTES : Q6K_BLOCK_BYTES)) {
    if (why) *why = "small-m path: tile does not fit shared memory for these dims";
    return false;
  }
  return true;
}

int32_t launch_decode_ffn(infr_cuda_ctx* ctx, const DecodeParams& p, bool pdl, uint32_t stages) {
  if (!BankTypes{p.gate_dt, p.up_dt, p.down_dt}.tuned()) return launch_anyfmt_decode(ctx, p, pdl, stages);
  const bool has_sh = p.sh_gate != nullptr;
  const int sh_ff = has_sh ? p.sh_ff : 0;
  const int n_chunks = pick_chunks(p.ne, p.nff, sh_ff);
  const size_t dbb = p.down_q4k ? Q4K_BLOCK_BYTES : Q6K_BLOCK_BYTES;
  const int TI = pick_down_tile(p.ne, p.nff, sh_ff, p.n_used, dbb);
  if (!n_chunks || !TI) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "small-m path: tile does not fit shared memory");
  int gw = GU_WARPS;
  int TR = gw * n_chunks;
  int jobs = p.rows * p.n_used * (p.nff / TR) + (has_sh ? p.rows * (sh_ff / TR) : 0);
  int n_chunks_gu = n_chunks;
  {
    // Grids of more than four waves: four warps taking four chunks of four rows each (same tile per role
    // as 16 x 1, half the default tile).  The smaller CTAs put more independent chains of
    // (ids -> copies -> unpack) on an SM: 69 us against 78 us for 32 tokens.
    const int ew = (int)ctx->cfg.gu_warps, ec = (int)ctx->cfg.gu_chunks;
    if (ew > 0 && ec > 0 && ec <= GU_MAX_CHUNKS && jobs > 4 * ctx->sm_count && p.ne / 16 <= ew * 32 && p.nff % (ew * ec) == 0 &&
        (!has_sh || sh_ff % (ew * ec) == 0)) {
      gw = ew;
      n_chunks_gu = ec;
      TR = gw * n_chunks_gu;
      jobs = p.rows * p.n_used * (p.nff / TR) + (has_sh ? p.rows * (sh_ff / TR) : 0);
    }
  }
  size_t smem_gu = gateup_smem(p.ne, n_chunks_gu, gw);
  // A grid that fits the device one CTA per SM is spread that way: gate/up CTAs start while the
  // router's CTAs still hold some SMs and would otherwise pair up on the free ones, halving their
  // copy bandwidth and leaving no room for the down kernel's CTAs to start beside them.  A request
  // above half of an SM's shared memory keeps two off one SM; a down CTA still fits beside one.
  if (jobs <= ctx->sm_count && smem_gu < 114 * 1024) smem_gu = 114 * 1024;
  const int ng = (p.ne / 64 + 31) / 32;
  cudaError_t e = cudaSuccess;
  auto run_gu = [&](auto kern) {
    e = ensure_smem(reinterpret_cast<const void*>(kern), smem_gu);
    if (e != cudaSuccess) return e;
    return launch_ex(kern, dim3(jobs), dim3(gw * 32), smem_gu, ctx->stream, pdl, p, n_chunks_gu);
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

  const size_t smem_dn = down_smem(TI, p.nff, sh_ff, p.n_used, dbb);
  e = ensure_smem(reinterpret_cast<const void*>(k_decode_down), smem_dn);
  if (e != cudaSuccess) return check_cuda(ctx, e, "k_decode_down smem attribute");
  // one warp per (slot, group of up to 8 rows) when that fits, else the largest divisor
  const int n_tasks = (p.n_used + (has_sh ? 1 : 0)) * (TI > 8 ? TI / 8 : 1);
  int nw = 16;
  for (int c = DN_MAX_WARPS; c >= 8; --c)
    if (n_tasks % c == 0) { nw = c; break; }
  if (n_tasks < 8) nw = n_tasks < 4 ? 4 : n_tasks;
  // One CTA per SM when the grid fits the device that way: with a whole number of warps per SM
  // sub-partition, one of these CTAs shares the register file with a gate/up CTA but not with a
  // second CTA of its own kind (which would only get going once the first has finished).
  if (p.rows * (p.ne / TI) <= ctx->sm_count && nw > 16 && nw % 4) nw = std::min((int)DN_MAX_WARPS, (nw + 3) & ~3);
  {
    // Grids of more than four waves: at most 12 warps, so that three CTAs share an SM's registers and
    // their latency chains overlap (83 us against 98 us for 32 tokens).
    const int cap = (int)ctx->cfg.dn_warps;
    if (cap > 0 && p.rows * (p.ne / TI) > 4 * ctx->sm_count)
      for (int c = cap; c >= 1; --c)
        if (n_tasks % c == 0) { nw = c; break; }
  }
  e = launch_ex(k_decode_down, dim3(p.rows * (p.ne / TI)), dim3(nw * 32), smem_dn, ctx->stream, pdl, p, TI);
  ctx->launches += 1;
  return check_cuda(ctx, e, "k_decode_down launch");
}

}  // namespace infr
