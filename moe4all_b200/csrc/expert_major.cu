// Small-m expert FFN, expert-major: one CTA owns one expert (and a tile of its rows) for ALL tokens of
// the call that were routed to it.
//
//   k_em_bucket  : (token, rank) pairs grouped by expert into segments of at most 8 pairs; integer sums
//                  of the fixed-point activations per 32-element sub-block
//   k_em_gateup  : act[pair, f] = act_fn(W_gate[e][f,:]·x_tok) * (W_up[e][f,:]·x_tok)       (Q4_K banks)
//   k_em_down    : y[pair, i]   = W_down[e][i,:]·act[pair,:]                                 (Q6_K bank)
//   k_em_combine : dst[r, :]    = sum over ranks (rank order) w * y[pair] + shared expert (+ residual)
//
// Reference: the same CPU stages as the per-pair kernels (crates/infr-cpu/src/lib.rs:3873-3907 bucket by
// expert, :4051-4266 expert mat-vecs, :4287-4303 rank-ordered sum).  The reference's GPU backend switches
// from one dispatch per (token, expert) pair to row tiles over an expert's tokens between 8 and 16
// rows (crates/infr-vulkan/src/adapter.rs:253-287) with 32-row tiles for lightly loaded experts
// (crates/infr-vulkan/src/recorder.rs:283, 15219-15225); this file is that middle regime.
//
// Arithmetic: weights stay the GGUF integer codes, activations are 16-bit fixed point in two signed
// 8-bit limbs (X = 256 hi + lo, as in the per-pair kernels), and the products run on the tensor cores'
// integer path: `mma.sync m16n8k32 u8 x s8 -> s32` per 32-element Q4_K sub-block (m16n8k16 per 16-element
// Q6_K scale group), one MMA per limb.  The integer sums are exact; the 6-bit (8-bit) block scales are
// applied to them in integers as well and a block's total is converted to f32 once.  A weight word is
// fetched and masked once per CTA and multiplied against up to 8 token rows, so the cost per weight does
// not grow with the tokens an expert sees, and the kernels stream the distinct experts' bytes once
// (1-D bulk async copies into shared memory, never multicast).
#include "kernels.cuh"
#include "tma.cuh"

namespace infr {

namespace {

constexpr int EM_FEAT = 32;         // gate/up: features per CTA
constexpr int EM_GU_WARPS = 4;      // consumer warps: two 16-feature groups x two block parities
constexpr int EM_MAX_STAGES = 4;
constexpr int EM_DN_WARPS = 4;      // down: 16 output rows per warp (or fewer rows and a split of the blocks)
constexpr int EM_SEG = 8;           // token rows per segment = the N extent of one MMA

__device__ __forceinline__ void mma_u8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_u8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a0), "r"(a1), "r"(b0));
}

// ---------------------------------------------------------------------------------------------
// bucket: pairs by expert, in segments of at most `seg_cap` pairs; the shared expert's rows are
// appended as segments of "expert" n_expert over pair ids P + r.  One CTA.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) k_em_bucket(EmParams p, int seg_cap) {
  __shared__ int s_cnt[1024], s_off[1025], s_fill[1024], s_segbase[1025];
  __shared__ int s_ws[33];
  const int tid = threadIdx.x, E = p.n_expert, P = p.rows * p.n_used;
  pdl_trigger();
  // sums of the fixed-point activations per 32-element sub-block (the Q4_K `min` term needs them).
  // xq_* come from the kernel before this one in the stream.
  pdl_wait();
  if (!p.xsum_ready) {  // (the whole-row router kernels make them with the fixed-point copy)
    const int nsb = p.ne / 32, total = p.rows * nsb;
    for (int i = tid; i < total; i += 1024) {
      const int r = i / nsb, sb = i - r * nsb;
      const int4* lo = reinterpret_cast<const int4*>(p.xq_lo + (size_t)r * p.ne + sb * 32);
      const int4* hi = reinterpret_cast<const int4*>(p.xq_hi + (size_t)r * p.ne + sb * 32);
      int l = 0, h = 0;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int4 a = __ldcg(lo + q), b = __ldcg(hi + q);
        l = __dp4a(0x01010101, a.x, l); l = __dp4a(0x01010101, a.y, l); l = __dp4a(0x01010101, a.z, l); l = __dp4a(0x01010101, a.w, l);
        h = __dp4a(0x01010101, b.x, h); h = __dp4a(0x01010101, b.y, h); h = __dp4a(0x01010101, b.z, h); h = __dp4a(0x01010101, b.w, h);
      }
      p.xsum[i] = h * 256 + l;
    }
  }
  s_cnt[tid] = 0;
  s_fill[tid] = 0;
  __syncthreads();
  auto expert_of = [&](int pair) {
    int e = __ldcg(p.ids + pair);
    if (e < 0) return -1;  // a pair another rank serves
    if (e >= E) {
      p.status->bad_index = 1;
      e = E - 1;
    }
    if (p.ep_n != 0 && ((uint32_t)e < p.ep_lo || (uint32_t)e >= p.ep_lo + p.ep_n)) return -1;
    return e;
  };
  for (int i = tid; i < P; i += 1024) {
    const int e = expert_of(i);
    if (e >= 0) atomicAdd(&s_cnt[e], 1);
  }
  __syncthreads();
  // exclusive scans over experts of (pairs, segments): thread e holds expert e
  {
    const int lane = tid & 31, warp = tid >> 5;
    const int c = tid < E ? s_cnt[tid] : 0, sg = (c + seg_cap - 1) / seg_cap;
    int ic = c, is = sg;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int uc = __shfl_up_sync(0xFFFFFFFFu, ic, o), us = __shfl_up_sync(0xFFFFFFFFu, is, o);
      if (lane >= o) { ic += uc; is += us; }
    }
    __shared__ int s_wc[32], s_wsg[32];
    if (lane == 31) { s_wc[warp] = ic; s_wsg[warp] = is; }
    __syncthreads();
    if (warp == 0) {
      int wc = s_wc[lane], wsg = s_wsg[lane];
      const int oc = wc, os = wsg;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int uc = __shfl_up_sync(0xFFFFFFFFu, wc, o), us = __shfl_up_sync(0xFFFFFFFFu, wsg, o);
        if (lane >= o) { wc += uc; wsg += us; }
      }
      s_wc[lane] = wc - oc;
      s_wsg[lane] = wsg - os;
      if (lane == 31) { s_ws[0] = wc; s_ws[1] = wsg; }
    }
    __syncthreads();
    s_off[tid] = ic - c + s_wc[warp];
    s_segbase[tid] = is - sg + s_wsg[warp];
  }
  __syncthreads();
  const int n_routed_pairs = s_ws[0], n_routed_seg = s_ws[1];
  // segment table of the routed experts
  if (tid < E) {
    const int c = s_cnt[tid];
    for (int k = 0, sgi = s_segbase[tid]; k < c; k += seg_cap, ++sgi) {
      p.seg_expert[sgi] = tid;
      p.seg_off[sgi] = s_off[tid] + k;
      p.seg_cnt[sgi] = min(seg_cap, c - k);
    }
  }
  // the shared expert: every row, in row order
  const int n_sh_seg = p.sh_ff ? (p.rows + seg_cap - 1) / seg_cap : 0;
  for (int i = tid; i < n_sh_seg; i += 1024) {
    p.seg_expert[n_routed_seg + i] = E;
    p.seg_off[n_routed_seg + i] = n_routed_pairs + i * seg_cap;
    p.seg_cnt[n_routed_seg + i] = min(seg_cap, p.rows - i * seg_cap);
  }
  if (p.sh_ff)
    for (int r = tid; r < p.rows; r += 1024) p.seg_pairs[n_routed_pairs + r] = P + r;
  if (tid == 0) *p.n_seg = n_routed_seg + n_sh_seg;
  // scatter (the order inside an expert is arrival order; every pair's result is independent of it)
  for (int i = tid; i < P; i += 1024) {
    const int e = expert_of(i);
    if (e >= 0) p.seg_pairs[s_off[e] + atomicAdd(&s_fill[e], 1)] = i;
  }
}

// ---------------------------------------------------------------------------------------------
// gate/up + activation
// ---------------------------------------------------------------------------------------------
// Job = (segment of up to 8 token rows, tile of EM_FEAT features, both roles); the CTAs are persistent
// and take jobs blockIdx.x, blockIdx.x + gridDim.x, ...  Four consumer warps: warp (fw, ks) owns features
// 16 fw .. 16 fw + 15 and every second block of the row (ks = block parity); MMA rows are the 16 gate rows
// and, in a second accumulator set, the 16 up rows, so a thread ends with gate and up of the same
// (feature, token).  The fifth warp is the producer: per stage it streams KB blocks of every weight row
// (one tiled TMA copy per block and role: a box of 32 rows x 144 bytes out of rows a whole row apart), the
// same K range of the tokens' fixed-point limbs and their sub-block sums (1-D bulk copies), through a
// ring of S stages that runs on across jobs, so the next job's weights arrive while this one is
// computed.  Row pitches are 4 (mod 8) words, which makes every fragment load (eight rows x four
// consecutive words) conflict-free.
// Scales are applied in integers: per block a thread accumulates sc * (limb sums) and m * sum(X) in int32
// (bounded: 8 sub-blocks x 63 x 32 x 15 x 128 < 2^31) and converts once per block.
__global__ void __launch_bounds__((EM_GU_WARPS + 1) * 32) k_em_gateup(EmParams p, int KB, int S, int xpitch, int gu_rows,
                                                                      const __grid_constant__ CUtensorMap tm_gate,
                                                                      const __grid_constant__ CUtensorMap tm_up,
                                                                      const __grid_constant__ CUtensorMap tm_sh_gate,
                                                                      const __grid_constant__ CUtensorMap tm_sh_up) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t s_full[EM_MAX_STAGES], s_empty[EM_MAX_STAGES];
  __shared__ float s_red[2][2][32][8];  // [job parity][feature group][lane][gate 4 | up 4]
  __shared__ int s_abort;               // a consumer warp's bounded wait ran out: all consumers leave together

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int nffmax = p.nffmax, tiles_max = nffmax / EM_FEAT;
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], EM_GU_WARPS);
    }
    mbar_fence_init();
    s_abort = 0;
  }
  __syncthreads();
  pdl_wait();  // the segment table comes from the bucket kernel
  pdl_trigger();
  const int n_jobs = __ldcg(p.n_seg) * tiles_max;
  const int P = p.rows * p.n_used;
  const int n_kc = (p.ne / 256) / KB, nsb = p.ne / 32;
  const int spitch = KB * 8 + 4;  // ints per token of the sub-block sums: tokens 2t land in different banks
  // stage layout: weights [KB blocks][2 roles][EM_FEAT rows][144] | x limbs [2][8 tokens][xpitch] | sub-block sums [8][spitch] ints
  constexpr uint32_t BOX = EM_FEAT * Q4K_BLOCK_BYTES;  // one block of one role's rows
  const uint32_t w_bytes = (uint32_t)KB * 2 * BOX, x_bytes = (uint32_t)16 * xpitch, s_bytes = (uint32_t)8 * spitch * 4;
  const uint32_t stage_bytes = w_bytes + x_bytes + s_bytes;
  uint32_t it = 0;  // stages used so far by this CTA (both roles count alike)

  if (warp == EM_GU_WARPS) {
    bool ok = true;
    for (int job = blockIdx.x; job < n_jobs && ok; job += gridDim.x) {
      const int seg = job / tiles_max, tile = job - seg * tiles_max;
      const int e = __ldcg(p.seg_expert + seg), cnt = __ldcg(p.seg_cnt + seg), off = __ldcg(p.seg_off + seg);
      const bool shared_seg = e >= p.n_expert;
      if (tile * EM_FEAT >= (shared_seg ? p.sh_ff : p.nff)) continue;
      const CUtensorMap* tmg = shared_seg ? &tm_sh_gate : &tm_gate;
      const CUtensorMap* tmu = shared_seg ? &tm_sh_up : &tm_up;
      const int bank_row0 = (shared_seg ? 0 : e * gu_rows) + tile * EM_FEAT;  // with gate and up in one bank the up map starts n_ff_exp rows in
      // lanes 8-23: a limb row of token (lane & 7); lanes 24-31: its sums.  A padding slot reads row 0; its results are dropped.
      int row = 0;
      if (lane >= 8 && (lane & 7) < cnt) {
        const int pr = __ldcg(p.seg_pairs + off + (lane & 7));
        row = pr >= P ? pr - P : pr / p.n_used;
      }
      for (int kc = 0; kc < n_kc; ++kc, ++it) {
        const int s = it % S;
        if (it >= (uint32_t)S && !mbar_wait_bounded(&s_empty[s], ((it / S) - 1) & 1)) { ok = false; break; }
        unsigned char* st = smem + (size_t)s * stage_bytes;
        if (lane == 0)
          mbar_arrive_expect_tx(&s_full[s], (uint32_t)(2 * EM_FEAT) * KB * Q4K_BLOCK_BYTES + (uint32_t)16 * KB * 256 + (uint32_t)8 * KB * 32);
        __syncwarp();
        if (lane < 2 * KB) {
          const int b = lane >> 1, role = lane & 1;
          tma_load_2d(st + (size_t)lane * BOX, role ? tmu : tmg, (kc * KB + b) * (int)Q4K_BLOCK_BYTES, bank_row0, &s_full[s]);
        } else if (lane >= 8 && lane < 24) {
          const int8_t* src = ((lane >= 16) ? p.xq_hi : p.xq_lo) + (size_t)row * p.ne + (size_t)kc * KB * 256;
          bulk_g2s(st + w_bytes + (size_t)(lane - 8) * xpitch, src, (uint32_t)KB * 256, &s_full[s]);
        } else if (lane >= 24) {
          bulk_g2s(st + w_bytes + x_bytes + (size_t)(lane - 24) * spitch * 4, p.xsum + (size_t)row * nsb + (size_t)kc * KB * 8, (uint32_t)KB * 32, &s_full[s]);
        }
      }
    }
    if (!ok && lane == 0) atomicExch(&p.status->timeout, 7);
    return;
  }

  // consumers
  const int fw = warp & 1, ks = warp >> 1;
  bool ok = true;
  int jpar = 0;
  for (int job = blockIdx.x; job < n_jobs && ok; job += gridDim.x) {
    const int seg = job / tiles_max, tile = job - seg * tiles_max;
    const int e = __ldcg(p.seg_expert + seg), cnt = __ldcg(p.seg_cnt + seg), off = __ldcg(p.seg_off + seg);
    const bool shared_seg = e >= p.n_expert;
    if (tile * EM_FEAT >= (shared_seg ? p.sh_ff : p.nff)) continue;
    float fg[4] = {0.f, 0.f, 0.f, 0.f}, fu[4] = {0.f, 0.f, 0.f, 0.f};
    for (int kc = 0; kc < n_kc; ++kc, ++it) {
      const int s = it % S;
      if (!mbar_wait_bounded(&s_full[s], (it / S) & 1)) { ok = false; break; }
      const unsigned char* st = smem + (size_t)s * stage_bytes;
      const unsigned char* xlo = st + w_bytes + (size_t)g * xpitch + 4 * t;  // B fragments: token g
      const unsigned char* xhi = xlo + (size_t)8 * xpitch;
      const int* sum0 = reinterpret_cast<const int*>(st + w_bytes + x_bytes) + (2 * t) * spitch;  // accumulator columns 2t, 2t + 1
      const int* sum1 = sum0 + spitch;
      for (int b = ks; b < KB; b += 2) {
        // this block's rows: gate g, gate g + 8, up g, up g + 8 of the warp's feature group
        const unsigned char* wst = st + (size_t)b * 2 * BOX + (size_t)(fw * 16 + g) * Q4K_BLOCK_BYTES;
        const unsigned char* rows4[4] = {wst, wst + 8 * Q4K_BLOCK_BYTES, wst + BOX, wst + BOX + 8 * Q4K_BLOCK_BYTES};
        uint4 hdr[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) hdr[r] = *reinterpret_cast<const uint4*>(rows4[r]);
        int svh_g[4] = {0, 0, 0, 0}, svl_g[4] = {0, 0, 0, 0}, mv_g[4] = {0, 0, 0, 0};
        int svh_u[4] = {0, 0, 0, 0}, svl_u[4] = {0, 0, 0, 0}, mv_u[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t wA[4], wB[4], scp[4], mp[4];
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const unsigned char* q = rows4[r] + 16 + 32 * j + 4 * t;
            wA[r] = *reinterpret_cast<const uint32_t*>(q);
            wB[r] = *reinterpret_cast<const uint32_t*>(q + 16);
            q4k_scale_min_pair(hdr[r].y, hdr[r].z, hdr[r].w, j, scp[r], mp[r]);
          }
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int lsb = b * 8 + 2 * j + half;  // sub-block index inside the stage
            const uint32_t b0l = *reinterpret_cast<const uint32_t*>(xlo + lsb * 32), b1l = *reinterpret_cast<const uint32_t*>(xlo + lsb * 32 + 16),
                           b0h = *reinterpret_cast<const uint32_t*>(xhi + lsb * 32), b1h = *reinterpret_cast<const uint32_t*>(xhi + lsb * 32 + 16);
            const int sx0 = sum0[lsb], sx1 = sum1[lsb];
            uint32_t a[4][2];
            int sc[4], mn[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              a[r][0] = (wA[r] >> (4 * half)) & 0x0F0F0F0Fu;
              a[r][1] = (wB[r] >> (4 * half)) & 0x0F0F0F0Fu;
              sc[r] = (int)((scp[r] >> (8 * half)) & 0xFFu);
              mn[r] = (int)((mp[r] >> (8 * half)) & 0xFFu);
            }
            int cgl[4] = {0, 0, 0, 0}, cgh[4] = {0, 0, 0, 0}, cul[4] = {0, 0, 0, 0}, cuh[4] = {0, 0, 0, 0};
            mma_u8s8_k32(cgl, a[0][0], a[1][0], a[0][1], a[1][1], b0l, b1l);
            mma_u8s8_k32(cgh, a[0][0], a[1][0], a[0][1], a[1][1], b0h, b1h);
            mma_u8s8_k32(cul, a[2][0], a[3][0], a[2][1], a[3][1], b0l, b1l);
            mma_u8s8_k32(cuh, a[2][0], a[3][0], a[2][1], a[3][1], b0h, b1h);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int r = i >> 1, sx = (i & 1) ? sx1 : sx0;  // accumulator rows g (i < 2) and g + 8; columns 2t, 2t + 1
              svl_g[i] += sc[r] * cgl[i];
              svh_g[i] += sc[r] * cgh[i];
              mv_g[i] += mn[r] * sx;
              svl_u[i] += sc[2 + r] * cul[i];
              svh_u[i] += sc[2 + r] * cuh[i];
              mv_u[i] += mn[2 + r] * sx;
            }
          }
        }
        // once per block: value = d * sum(sc * sum(q X)) - dmin * sum(m * sum(X)), X = 256 hi + lo
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = i >> 1;
          const float dg = f16_bits_to_f32(hdr[r].x), dmg = f16_bits_to_f32(hdr[r].x >> 16);
          const float du = f16_bits_to_f32(hdr[2 + r].x), dmu = f16_bits_to_f32(hdr[2 + r].x >> 16);
          fg[i] += dg * fmaf(256.f, (float)svh_g[i], (float)svl_g[i]) - dmg * (float)mv_g[i];
          fu[i] += du * fmaf(256.f, (float)svh_u[i], (float)svl_u[i]) - dmu * (float)mv_u[i];
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[s]);  // (arrivals after the producer's last wait complete phases nobody waits for)
    }
    // the two block-parity halves of a feature group meet in shared memory (consumer warps only: named
    // barrier 1).  The buffer alternates with the job, so the next job's writes cannot overtake this job's reads.
    if (ks == 1) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s_red[jpar][fw][lane][i] = fg[i];
        s_red[jpar][fw][lane][4 + i] = fu[i];
      }
    }
    if (!ok) s_abort = 1;
    asm volatile("bar.sync 1, %0;" ::"n"(EM_GU_WARPS * 32) : "memory");
    if (*reinterpret_cast<volatile int*>(&s_abort)) {
      ok = false;
      break;
    }
    if (ks == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        fg[i] += s_red[jpar][fw][lane][i];
        fu[i] += s_red[jpar][fw][lane][4 + i];
      }
      // epilogue: act[pair, feature] = act_fn(gate) * up, f32
      const float clamp = shared_seg ? 0.f : p.clamp;
      const int f0 = tile * EM_FEAT + fw * 16;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tk = 2 * t + (i & 1);
        if (tk >= cnt) continue;
        const int pr = __ldcg(p.seg_pairs + off + tk);
        const int row = pr >= P ? pr - P : pr / p.n_used;
        const float xs = __ldcg(p.xscale + row);
        const float wp = (p.weight_before && !shared_seg) ? __ldcg(p.wts + pr) : 1.0f;
        p.act[(size_t)pr * nffmax + f0 + g + 8 * (i >> 1)] = gated_act(p.act_kind, clamp, wp * (fg[i] * xs), wp * (fu[i] * xs));
      }
    }
    jpar ^= 1;
  }
  if (!ok && lane == 0) atomicExch(&p.status->timeout, 7);
}

// ---------------------------------------------------------------------------------------------
// down
// ---------------------------------------------------------------------------------------------
// Job = (segment of up to 8 token rows, tile of `rows_cta` output features).  CTAs are persistent and take a
// contiguous range of jobs, so consecutive jobs mostly share their segment.  A job's rows are one contiguous
// slab of the expert's down matrix and arrive by one bulk copy into one of two buffers; the next job's slab
// is requested before this job is computed (the first one before the wait for the gate/up kernel).  When the
// segment changes, its activation rows are brought to 16-bit fixed point in shared memory (one scale per
// row, integer sums per 16 elements).  Q6_K blocks are 210 bytes, so a row's words sit 0 or 2 bytes off a
// word boundary: fragment words are two aligned loads and a funnel shift.  A 16-element scale group is one
// m16n8k16 MMA per limb; scales are applied in integers and converted once per block (bounded: 16 groups x
// 128 x 16 x 63 x 128 < 2^31).
// Q4 = the down banks are Q4_K (the other half of the layers of a Q4_K_M file): 144-byte blocks on 16-byte
// boundaries, so fragment words are plain loads; a 32-element scale group is one m16n8k32 MMA per limb, its
// 6-bit scale and min applied in integers (8 groups x 32 x 15 x 63 x 128 and 8 x 63 x 32 x 32639, both < 2^31).
template <bool Q4>
__global__ void __launch_bounds__(EM_DN_WARPS * 32) k_em_down(EmParams p, int rows_cta, int apitch, uint32_t slab_pitch) {
  constexpr uint32_t DBB = Q4 ? Q4K_BLOCK_BYTES : Q6K_BLOCK_BYTES;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t s_bar[2];
  __shared__ int s_pair[8];
  __shared__ float s_xs[8];
  __shared__ float s_wmax[EM_DN_WARPS];
  __shared__ float s_dred[3 * 128];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int tiles = p.ne / rows_cta;
  if (tid == 0) {
    mbar_init(&s_bar[0], 1);
    mbar_init(&s_bar[1], 1);
    mbar_fence_init();
  }
  __syncthreads();
  pdl_trigger();
  // the segment table is final (the gate/up kernel, ahead in the stream, only started after it)
  const int n_jobs = __ldcg(p.n_seg) * tiles;
  const int per = (n_jobs + (int)gridDim.x - 1) / (int)gridDim.x;
  const int job0 = blockIdx.x * per, job1 = min(job0 + per, n_jobs);
  if (job0 >= job1) return;
  const int ngrp = (p.nffmax >> 4) + 4;  // ints per token of the sums: tokens 2t land in different banks
  // shared memory: activation limbs [2][8 tokens][apitch] | sums [8][ngrp] ints | two slab buffers
  unsigned char* s_act = smem;
  int* s_sum = reinterpret_cast<int*>(smem + (size_t)16 * apitch);
  unsigned char* slab_area = reinterpret_cast<unsigned char*>(s_sum + 8 * ngrp);
  slab_area += (128u - (smem_u32(slab_area) & 127u)) & 127u;

  auto job_src = [&](int job, int& nff_e) {
    const int seg = job / tiles, tile = job - seg * tiles;
    const int e = __ldcg(p.seg_expert + seg);
    const bool shared_seg = e >= p.n_expert;
    nff_e = shared_seg ? p.sh_ff : p.nff;
    return (shared_seg ? p.sh_down : p.down + (size_t)e * p.down_stride) + (size_t)tile * rows_cta * (nff_e / 256 * (int)DBB);
  };
  // a slab lands at its source's offset inside a 128-byte line
  auto request = [&](int job, int buf) {
    int nff_e;
    const uint8_t* src = job_src(job, nff_e);
    const uint32_t bytes = (uint32_t)rows_cta * (nff_e / 256 * DBB);
    mbar_arrive_expect_tx(&s_bar[buf], bytes);
    bulk_g2s(slab_area + (size_t)buf * slab_pitch + (uint32_t)(reinterpret_cast<uintptr_t>(src) & 127u), src, bytes, &s_bar[buf]);
  };
  if (tid == 0) request(job0, 0);
  pdl_wait();  // activations come from the gate/up kernel

  int cur_seg = -1, cnt = 0;
  for (int job = job0; job < job1; ++job) {
    const int buf = (job - job0) & 1;
    const int seg = job / tiles, tile = job - seg * tiles;
    int nff_e;
    const uint8_t* src = job_src(job, nff_e);
    const unsigned char* slab = slab_area + (size_t)buf * slab_pitch + (uint32_t)(reinterpret_cast<uintptr_t>(src) & 127u);
    const int drb = nff_e / 256 * (int)DBB;
    __syncthreads();  // every warp is done with the previous job: its slab buffer (the other one) and the limbs may be reused
    if (tid == 0 && job + 1 < job1) request(job + 1, buf ^ 1);
    if (seg != cur_seg) {
      cur_seg = seg;
      cnt = __ldcg(p.seg_cnt + seg);
      const int off = __ldcg(p.seg_off + seg);
      if (tid < 8) s_pair[tid] = tid < cnt ? __ldcg(p.seg_pairs + off + tid) : -1;
      __syncthreads();
      // fixed point: X = round(a * 32639 / max|a|) per row, limbs X = 256 hi + lo, sums per 16 elements
      const int n4 = nff_e / 4;
      for (int tk = 0; tk < cnt; ++tk) {
        const float4* arow = reinterpret_cast<const float4*>(p.act + (size_t)s_pair[tk] * p.nffmax);
        float m = 0.f;
        for (int i = tid; i < n4; i += EM_DN_WARPS * 32) {
          const float4 v = __ldcg(arow + i);
          m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(m, fmaxf(fabsf(v.z), fabsf(v.w))));
        }
        m = warp_max(m);
        if (lane == 0) s_wmax[warp] = m;
        __syncthreads();
        m = 0.f;
#pragma unroll
        for (int w = 0; w < EM_DN_WARPS; ++w) m = fmaxf(m, s_wmax[w]);
        const float inv = m > 0.f ? 32639.f / m : 0.f;
        if (tid == 0) s_xs[tk] = m / 32639.f;
        for (int i = tid; i < n4; i += EM_DN_WARPS * 32) {
          const float4 v = __ldcg(arow + i);
          const int X[4] = {__float2int_rn(v.x * inv), __float2int_rn(v.y * inv), __float2int_rn(v.z * inv), __float2int_rn(v.w * inv)};
          uint32_t lo, hi;
          pack_limbs4(X, lo, hi);
          *reinterpret_cast<uint32_t*>(s_act + (size_t)tk * apitch + 4 * i) = lo;
          *reinterpret_cast<uint32_t*>(s_act + (size_t)(8 + tk) * apitch + 4 * i) = hi;
          int sx = (X[0] + X[1]) + (X[2] + X[3]);  // 16 elements = four neighbouring threads (n4 is a multiple of 64: whole warps)
          sx += __shfl_xor_sync(0xFFFFFFFFu, sx, 1);
          sx += __shfl_xor_sync(0xFFFFFFFFu, sx, 2);
          if ((i & 3) == 0) s_sum[tk * ngrp + (i >> 2)] = sx;
        }
        __syncthreads();
      }
    }
    if (!mbar_wait_bounded(&s_bar[buf], ((job - job0) >> 1) & 1)) {
      if (lane == 0) atomicExch(&p.status->timeout, 8);
      return;
    }
    const int nb = nff_e / 256;
    // 16-row tiles of this job: one per warp, or (fewer rows per CTA) several warps per tile, each taking
    // every ksplit-th block, their partial sums added through shared memory
    const int n_rt = rows_cta / 16, ksplit = EM_DN_WARPS / n_rt;
    const unsigned char* alo = s_act + (size_t)g * apitch + 4 * t;  // B fragments: token g
    const unsigned char* ahi = alo + (size_t)8 * apitch;
    const int* sum0 = s_sum + (2 * t) * ngrp;
    const int* sum1 = sum0 + ngrp;
    const int rt = warp % n_rt, ks = warp / n_rt;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t rofs[2] = {(uint32_t)(rt * 16 + g) * drb, (uint32_t)(rt * 16 + g + 8) * drb};
    for (int b = ks; Q4 && b < nb; b += ksplit) {
      // rows g and g + 8 of the tile: header (d, dmin, 12 scale bytes), then per 64 weights 32 code bytes whose
      // low nibbles are the first 32-element group and high nibbles the second
      const unsigned char* blk[2] = {slab + rofs[0] + (uint32_t)b * Q4K_BLOCK_BYTES, slab + rofs[1] + (uint32_t)b * Q4K_BLOCK_BYTES};
      const uint4 hdr[2] = {*reinterpret_cast<const uint4*>(blk[0]), *reinterpret_cast<const uint4*>(blk[1])};
      int svl[4] = {0, 0, 0, 0}, svh[4] = {0, 0, 0, 0}, mv[4] = {0, 0, 0, 0};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t scp[2], mp[2], w0[2], w1[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          q4k_scale_min_pair(hdr[r].y, hdr[r].z, hdr[r].w, j, scp[r], mp[r]);
          w0[r] = *reinterpret_cast<const uint32_t*>(blk[r] + 16 + 32 * j + 4 * t);       // k = 4 t .. 4 t + 3 of a group
          w1[r] = *reinterpret_cast<const uint32_t*>(blk[r] + 32 + 32 * j + 4 * t);       // k = 16 + 4 t ..
        }
#pragma unroll
        for (int hn = 0; hn < 2; ++hn) {
          const int k0 = b * 256 + j * 64 + hn * 32, grp = k0 >> 4;
          const uint32_t a00 = (w0[0] >> (4 * hn)) & 0x0F0F0F0Fu, a10 = (w0[1] >> (4 * hn)) & 0x0F0F0F0Fu,
                         a01 = (w1[0] >> (4 * hn)) & 0x0F0F0F0Fu, a11 = (w1[1] >> (4 * hn)) & 0x0F0F0F0Fu;
          const uint32_t b0l = *reinterpret_cast<const uint32_t*>(alo + k0), b1l = *reinterpret_cast<const uint32_t*>(alo + k0 + 16);
          const uint32_t b0h = *reinterpret_cast<const uint32_t*>(ahi + k0), b1h = *reinterpret_cast<const uint32_t*>(ahi + k0 + 16);
          int cl[4] = {0, 0, 0, 0}, ch[4] = {0, 0, 0, 0};
          mma_u8s8_k32(cl, a00, a10, a01, a11, b0l, b1l);
          mma_u8s8_k32(ch, a00, a10, a01, a11, b0h, b1h);
          const int m0 = sum0[grp] + sum0[grp + 1], m1 = sum1[grp] + sum1[grp + 1];
          const int scv[2] = {(int)((scp[0] >> (8 * hn)) & 0xFFu), (int)((scp[1] >> (8 * hn)) & 0xFFu)};
          const int mnv[2] = {(int)((mp[0] >> (8 * hn)) & 0xFFu), (int)((mp[1] >> (8 * hn)) & 0xFFu)};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            svl[i] += scv[i >> 1] * cl[i];
            svh[i] += scv[i >> 1] * ch[i];
            mv[i] += mnv[i >> 1] * ((i & 1) ? m1 : m0);
          }
        }
      }
      // sum over the block of d sc sum(q X) - dmin m sum(X), X = 256 hi + lo
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float d = f16_bits_to_f32(hdr[i >> 1].x), dmin = f16_bits_to_f32(hdr[i >> 1].x >> 16);
        acc[i] = fmaf(d, fmaf(256.f, (float)svh[i], (float)svl[i]), fmaf(-dmin, (float)mv[i], acc[i]));
      }
    }
    for (int b = ks; !Q4 && b < nb; b += ksplit) {
      // per row: aligned view of the block, the shift that realigns it, d and the 16 scales
      const uint32_t* wq[2];
      uint32_t sh[2];
      float d[2];
      uint32_t sc[2][4];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const uint32_t ro = rofs[r] + (uint32_t)b * Q6K_BLOCK_BYTES;  // the slab starts on a 16-byte boundary
        sh[r] = (ro & 3u) * 8;
        wq[r] = reinterpret_cast<const uint32_t*>(slab + (ro & ~3u));
        d[r] = f16_bits_to_f32(*reinterpret_cast<const unsigned short*>(slab + ro + 208));
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[r][i] = __funnelshift_r(wq[r][48 + i], wq[r][49 + i], sh[r]);
      }
      int svl[4] = {0, 0, 0, 0}, svh[4] = {0, 0, 0, 0}, mv[4] = {0, 0, 0, 0};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int lh = 0; lh < 2; ++lh) {
          // words of ql (two 32-byte runs) and qh that hold l = 16 lh + 4 t .. + 3 of this half
          uint32_t A[2], B[2], H[2];
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const int o = 16 * h + 4 * lh + t;
            A[r] = __funnelshift_r(wq[r][o], wq[r][o + 1], sh[r]);
            B[r] = __funnelshift_r(wq[r][o + 8], wq[r][o + 9], sh[r]);
            const int oh = 32 + 8 * h + 4 * lh + t;
            H[r] = __funnelshift_r(wq[r][oh], wq[r][oh + 1], sh[r]);
          }
#pragma unroll
          for (int qd = 0; qd < 4; ++qd) {
            uint32_t a[2];
            int scv[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              const uint32_t nib = (qd & 1) ? B[r] : A[r];
              a[r] = (((qd & 2) ? (nib >> 4) : nib) & 0x0F0F0F0Fu) | (((H[r] >> (2 * qd)) << 4) & 0x30303030u);
              const int si = 8 * h + 2 * qd + lh;  // scale index inside the block
              scv[r] = (int)(signed char)((sc[r][si >> 2] >> (8 * (si & 3))) & 0xFFu);
            }
            const int k0 = b * 256 + h * 128 + qd * 32 + lh * 16, grp = k0 >> 4;
            const uint32_t bl = *reinterpret_cast<const uint32_t*>(alo + k0), bh = *reinterpret_cast<const uint32_t*>(ahi + k0);
            const int m0 = sum0[grp], m1 = sum1[grp];
            int cl[4] = {0, 0, 0, 0}, ch[4] = {0, 0, 0, 0};
            mma_u8s8_k16(cl, a[0], a[1], bl);
            mma_u8s8_k16(ch, a[0], a[1], bh);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              svl[i] += scv[i >> 1] * cl[i];
              svh[i] += scv[i >> 1] * ch[i];
              mv[i] += scv[i >> 1] * ((i & 1) ? m1 : m0);
            }
          }
        }
      }
      // sum over the block of sc * (sum(q X) - 32 sum(X)), X = 256 hi + lo
#pragma unroll
      for (int i = 0; i < 4; ++i)
        acc[i] = fmaf(d[i >> 1], fmaf(256.f, (float)svh[i], (float)svl[i]) - 32.f * (float)mv[i], acc[i]);
    }
    if (ksplit > 1) {
      if (ks > 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) s_dred[((ks - 1) * n_rt + rt) * 128 + lane * 4 + i] = acc[i];
      }
      __syncthreads();
      if (ks == 0)
        for (int k2 = 1; k2 < ksplit; ++k2)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[i] += s_dred[((k2 - 1) * n_rt + rt) * 128 + lane * 4 + i];
    }
    // y[pair, row]: raw expert outputs; weights, down_scale and the sum over ranks follow in k_em_combine
    if (ks == 0) {
      const int i0 = tile * rows_cta + rt * 16;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tk = 2 * t + (i & 1);
        if (tk < cnt) p.y[(size_t)s_pair[tk] * p.ne + i0 + g + 8 * (i >> 1)] = acc[i] * s_xs[tk];
      }
    }
  }
}

// dst[r, :] = sum over ranks (rank order) of w * (y[pair] * down_scale[e]), then the shared expert's row
// (sigmoid-gated when its logit is given), then the residual - the order of the per-pair kernels.
__global__ void __launch_bounds__(256) k_em_combine(EmParams p, const float* sh_logit, const float* residual, float* dst) {
  pdl_wait();
  const int c = (blockIdx.x * 256 + threadIdx.x) * 4;
  if (c >= p.ne) return;
  const int P = p.rows * p.n_used;
  for (int r = blockIdx.y; r < p.rows; r += gridDim.y) {
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < p.n_used; s0 += 8) {
      // eight ranks at a time: ids, weights and rows are requested together, then added in rank order
      float w[8];
      float4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int pr = r * p.n_used + s0 + j;
        w[j] = 0.f;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (s0 + j >= p.n_used) continue;
        int e = __ldcg(p.ids + pr);
        if (e < 0) continue;
        e = min(e, p.n_expert - 1);
        if (p.ep_n != 0 && ((uint32_t)e < p.ep_lo || (uint32_t)e >= p.ep_lo + p.ep_n)) continue;
        const float ds = p.down_scale ? __ldg(p.down_scale + e) : 1.0f;
        w[j] = p.weight_before ? 1.0f : __ldcg(p.wts + pr);
        v[j] = __ldcg(reinterpret_cast<const float4*>(p.y + (size_t)pr * p.ne + c));
        v[j].x *= ds; v[j].y *= ds; v[j].z *= ds; v[j].w *= ds;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {  // a skipped rank adds 0 * 0: the sum is the one over the served ranks, in order
        o.x += w[j] * v[j].x; o.y += w[j] * v[j].y; o.z += w[j] * v[j].z; o.w += w[j] * v[j].w;
      }
    }
    if (p.sh_ff) {
      const float gsh = sh_logit ? 1.0f / (1.0f + __expf(-__ldcg(sh_logit + r))) : 1.0f;
      const float4 v = __ldcg(reinterpret_cast<const float4*>(p.y + (size_t)(P + r) * p.ne + c));
      o.x += gsh * v.x; o.y += gsh * v.y; o.z += gsh * v.z; o.w += gsh * v.w;
    }
    if (residual != nullptr) {  // may alias dst: each element is read, then written, by this thread
      const float4 h = __ldcg(reinterpret_cast<const float4*>(residual + (size_t)r * p.ne + c));
      o.x += h.x; o.y += h.y; o.z += h.z; o.w += h.w;
    }
    *reinterpret_cast<float4*>(dst + (size_t)r * p.ne + c) = o;
  }
}

// Stage shape of the gate/up kernel: KB blocks of every row per stage (even where the row allows it: the
// two block-parity warps then share a stage evenly), S stages, two CTAs per SM.
void gateup_shape(int ne, int* KB, int* S, int* xpitch, size_t* stage_bytes) {
  const int nblk = ne / 256;
  const int kb = (nblk % 4 == 0) ? 4 : ((nblk % 2 == 0) ? 2 : 1);
  *xpitch = kb * 256 + 16;  // 4 (mod 32) words
  *stage_bytes = (size_t)kb * 2 * EM_FEAT * Q4K_BLOCK_BYTES + (size_t)16 * *xpitch + (size_t)8 * (kb * 8 + 4) * 4;
  int s = nblk / kb;
  while (s > 1 && (s > EM_MAX_STAGES || (size_t)s * *stage_bytes > 112 * 1024)) --s;
  *KB = kb;
  *S = s;
}

// Rows of the down matrix per job: 64 (one 16-row tile per warp) while two slab buffers and the activation
// limbs leave room for two CTAs per SM, else 32 or 16 with the blocks split over the warps.
int down_rows(int ne, int nffmax, size_t dbb, int* apitch, size_t* slab_pitch, size_t* smem) {
  *apitch = nffmax + 16;  // 4 (mod 32) words
  const size_t fixed = (size_t)16 * *apitch + (size_t)8 * (nffmax / 16 + 4) * 4 + 256;
  const size_t drb = (size_t)nffmax / 256 * dbb;
  const int nb = nffmax / 256;
  for (int rows : {64, 32, 16}) {
    if (ne % rows) continue;
    const int ksplit = EM_DN_WARPS / (rows / 16);
    if (nb % ksplit) continue;
    *slab_pitch = align_up((size_t)rows * drb + 8, 128) + 128;
    *smem = fixed + 2 * *slab_pitch;
    if (*smem <= 110 * 1024 || rows == 16) return *smem <= 200 * 1024 ? rows : 0;
  }
  return 0;
}

}  // namespace

size_t em_scratch_bytes(int rows, int n_used, int ne, int nff, int sh_ff) {
  const size_t PT = (size_t)rows * n_used + rows, nffmax = std::max(nff, sh_ff);
  const size_t max_seg = PT + 8;
  size_t b = 0;
  b += align_up((size_t)rows * (ne / 32) * 4, 256);     // xsum
  b += align_up(256, 256);                              // n_seg
  b += 3 * align_up(max_seg * 4, 256);                  // seg_expert, seg_off, seg_cnt
  b += align_up((PT + 8) * 4, 256);                     // seg_pairs
  b += align_up(PT * nffmax * 4, 256);                  // act
  b += align_up(PT * (size_t)ne * 4, 256);              // y
  return b;
}

bool em_supported(int ne, int nff, int sh_ff, int n_expert, BankTypes bt) {
  if (!bt.tuned() || ne % 256 || nff % 256 || sh_ff % 256 || n_expert > 1024) return false;
  int apitch;
  size_t slab_pitch, smem;
  return down_rows(ne, std::max(nff, sh_ff), bt.down_q4k() ? Q4K_BLOCK_BYTES : Q6K_BLOCK_BYTES, &apitch, &slab_pitch, &smem) != 0;
}

int32_t launch_em_ffn(infr_cuda_ctx* ctx, const DecodeParams& dp, void* scratch, uint32_t stages) {
  EmParams p = {};
  const int rows = dp.rows, P = rows * dp.n_used, sh_ff = dp.sh_gate ? dp.sh_ff : 0;
  const size_t PT = (size_t)P + rows, nffmax = std::max(dp.nff, sh_ff), max_seg = PT + 8;
  char* base = static_cast<char*>(scratch);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    char* q = base + off;
    off += align_up(bytes, 256);
    return q;
  };
  p.xsum = reinterpret_cast<int*>(take((size_t)rows * (dp.ne / 32) * 4));
  p.n_seg = reinterpret_cast<int*>(take(256));
  p.seg_expert = reinterpret_cast<int*>(take(max_seg * 4));
  p.seg_off = reinterpret_cast<int*>(take(max_seg * 4));
  p.seg_cnt = reinterpret_cast<int*>(take(max_seg * 4));
  p.seg_pairs = reinterpret_cast<int*>(take((PT + 8) * 4));
  p.act = reinterpret_cast<float*>(take(PT * nffmax * 4));
  p.y = reinterpret_cast<float*>(take(PT * (size_t)dp.ne * 4));
  p.xsum_ready = dp.xsum_ready;
  p.xq_lo = dp.xq_lo;
  p.xq_hi = dp.xq_hi;
  p.xscale = dp.xscale;
  p.ids = dp.ids;
  p.wts = dp.wts;
  p.gate = dp.gate; p.up = dp.up; p.down = dp.down;
  p.sh_gate = dp.sh_gate; p.sh_up = dp.sh_up; p.sh_down = dp.sh_down;
  p.gate_stride = dp.gate_stride; p.up_stride = dp.up_stride; p.down_stride = dp.down_stride;
  p.down_scale = dp.down_scale;
  p.status = dp.status;
  p.rows = rows; p.ne = dp.ne; p.n_used = dp.n_used; p.nff = dp.nff; p.sh_ff = sh_ff; p.n_expert = dp.n_expert;
  p.nffmax = (int)nffmax;
  p.ep_lo = dp.ep_lo; p.ep_n = dp.ep_n;
  p.act_kind = dp.act_kind; p.weight_before = dp.weight_before; p.clamp = dp.clamp;

  // segments: one per expert with pairs, plus one per further EM_SEG pairs of an expert, plus the shared expert's
  const int max_routed_seg = std::min(P, dp.n_expert) + P / EM_SEG;
  const int n_seg_bound = max_routed_seg + (sh_ff ? (rows + EM_SEG - 1) / EM_SEG : 0);
  cudaError_t e = cudaSuccess;
  if (stages & 2u) {
    e = launch_ex(k_em_bucket, dim3(1), dim3(1024), 0, ctx->stream, true, p, EM_SEG);
    ctx->launches += 1;
    if (e != cudaSuccess) return check_cuda(ctx, e, "k_em_bucket launch");
    int KB, S, xpitch;
    size_t stage_bytes;
    gateup_shape(dp.ne, &KB, &S, &xpitch, &stage_bytes);
    const size_t smem = (size_t)S * stage_bytes;
    // the banks' rows as 2-D tensors for the tiled copies; with gate and up in one bank an expert has
    // 2 n_ff_exp rows and the up map starts n_ff_exp rows in (and ends with the bank)
    const size_t rb = (size_t)dp.ne / 256 * Q4K_BLOCK_BYTES;
    const size_t rows_per_expert = dp.gate_stride / rb, bank_rows = (size_t)dp.n_expert * rows_per_expert;
    CUtensorMap tm_gate, tm_up, tm_sh_gate, tm_sh_up;
    bool ok = q4k_rows_map(&tm_gate, dp.gate, bank_rows, rb, EM_FEAT) &&
              q4k_rows_map(&tm_up, dp.up, bank_rows - (rows_per_expert - (size_t)dp.nff), rb, EM_FEAT);
    tm_sh_gate = tm_gate;
    tm_sh_up = tm_up;
    if (ok && sh_ff) ok = q4k_rows_map(&tm_sh_gate, dp.sh_gate, (size_t)sh_ff, rb, EM_FEAT) && q4k_rows_map(&tm_sh_up, dp.sh_up, (size_t)sh_ff, rb, EM_FEAT);
    if (!ok) return fail(ctx, INFR_CUDA_ERR_CUDA, "expert-major gate/up kernel: the driver refused a tensor map for the expert banks");
    // persistent CTAs: two per SM (the shared-memory request allows no more), never more than there are jobs
    const unsigned jobs_bound = (unsigned)n_seg_bound * (unsigned)(nffmax / EM_FEAT);
    e = ensure_smem(reinterpret_cast<const void*>(k_em_gateup), smem);
    if (e == cudaSuccess)
      e = launch_ex(k_em_gateup, dim3(std::min(jobs_bound, 2u * (unsigned)ctx->sm_count)), dim3((EM_GU_WARPS + 1) * 32), smem, ctx->stream, true,
                    p, KB, S, xpitch, (int)rows_per_expert, tm_gate, tm_up, tm_sh_gate, tm_sh_up);
    ctx->launches += 1;
    if (e != cudaSuccess) return check_cuda(ctx, e, "k_em_gateup launch");
  }
  if (!(stages & 4u)) return INFR_CUDA_OK;
  {
    int apitch;
    size_t slab_pitch, smem;
    const int rows_cta = down_rows(dp.ne, (int)nffmax, dp.down_q4k ? Q4K_BLOCK_BYTES : Q6K_BLOCK_BYTES, &apitch, &slab_pitch, &smem);
    if (!rows_cta) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "expert-major down kernel: tile does not fit shared memory");
    const unsigned jobs_bound = (unsigned)n_seg_bound * (unsigned)(dp.ne / rows_cta);
    const unsigned per_sm = (unsigned)std::max<size_t>(1, std::min<size_t>(4, (200 * 1024) / smem));
    auto run_dn = [&](auto kern) {
      cudaError_t ee = ensure_smem(reinterpret_cast<const void*>(kern), smem);
      if (ee == cudaSuccess)
        ee = launch_ex(kern, dim3(std::min(jobs_bound, per_sm * (unsigned)ctx->sm_count)), dim3(EM_DN_WARPS * 32), smem, ctx->stream, true, p,
                       rows_cta, apitch, (uint32_t)slab_pitch);
      return ee;
    };
    e = dp.down_q4k ? run_dn(k_em_down<true>) : run_dn(k_em_down<false>);
    ctx->launches += 1;
    if (e != cudaSuccess) return check_cuda(ctx, e, "k_em_down launch");
  }
  e = launch_ex(k_em_combine, dim3((dp.ne / 4 + 255) / 256, std::min(rows, 65535)), dim3(256), 0, ctx->stream, true, p, dp.sh_logit,
                dp.residual, dp.dst);
  ctx->launches += 1;
  return check_cuda(ctx, e, "k_em_combine launch");
}

}  // namespace infr
