// Small-m expert FFN for banks in any mix of the formats formats.cuh covers (the reference's batched and
// decode MoE kernels take gate, up and down formats independently: crates/infr-core/src/tensor.rs:172-196;
// real files mix them, e.g. Q5_K gate/up with Q6_K down, or Q8_0 throughout).
//
//   k_anyfmt_gateup : act[p, f] = act_fn(W_gate[e_p][f,:]·x, W_up[e_p][f,:]·x)
//   k_anyfmt_down   : dst[r, i] = Σ_slot w_slot · (W_down[e_slot][i,:]·act[slot,:])  (+ shared expert, + residual)
//
// Same arithmetic as the tuned per-pair kernels (decode_ffn.cu): activations in 16-bit fixed point
// (two signed 8-bit limbs), exact integer dot products against the 8-bit codes of formats.cuh, the
// scale group's affine map applied in f32 per 16 weights, slots summed in rank order.  As there, a
// CTA's weight rows are one contiguous slab per role (per slot), requested up front with 1-D bulk
// copies (TMA, never multicast) so that the whole step's bytes are in flight at once; a warp then owns a
// weight row, its lanes side by side along the row, whatever the format's block size and alignment.
// CPU reference: crates/infr-cpu/src/lib.rs:4051-4303.
#include "formats.cuh"
#include "kernels.cuh"

namespace infr {

namespace {

constexpr int AF_MAX_SLOTS = 33;

__device__ __forceinline__ bool af_in_band(const DecodeParams& p, int e) {
  return p.ep_n == 0 || ((uint32_t)e >= p.ep_lo && (uint32_t)e < p.ep_lo + p.ep_n);
}

// Σ over 16 weights of w * X, in units of the activation's fixed-point step: l4 / h4 = the 16 low
// and high limbs, S = Σ X.  `row` points into shared memory.
__device__ __forceinline__ float af_dot16(int dt, const uint8_t* row, int h, const uint4& l4, const uint4& h4, int S) {
  uint32_t c[4];
  float A, B;
  int off;
  fmt_codes16<false>(dt, row, h, c, A, B, off);
  int dl = dp4a_us(c[0], (int)l4.x, 0), dh = dp4a_us(c[0], (int)h4.x, 0);
  dl = dp4a_us(c[1], (int)l4.y, dl); dh = dp4a_us(c[1], (int)h4.y, dh);
  dl = dp4a_us(c[2], (int)l4.z, dl); dh = dp4a_us(c[2], (int)h4.z, dh);
  dl = dp4a_us(c[3], (int)l4.w, dl); dh = dp4a_us(c[3], (int)h4.w, dh);
  const int t = dh * 256 + dl - off * S;  // |t| < 2^28
  return fmaf(A, (float)t, B * (float)S);
}

// A slab lands at the same offset inside a 128-byte line as its source has in global memory (bulk
// copies whose two sides disagree modulo 128 run several times slower); regions are padded for that.
__host__ __device__ inline size_t af_region(size_t bytes) { return align_up(bytes, 128) + 128; }

// One CTA = one (token, slot) pair (or one row of the shared expert) x TR = warps * rpw output
// features, both roles.  Shared memory: gate rows | up rows | limbs of x | sums of x per 16.
__global__ void __launch_bounds__(256, 3) k_anyfmt_gateup(DecodeParams p, int rpw) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t s_bar;
  unsigned char* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int TR = nwarps * rpw;
  const int tiles = p.nff / TR, sh_tiles = p.sh_ff / TR;
  const int n_routed_jobs = p.rows * p.n_used * tiles;
  const size_t grb = row_bytes(p.gate_dt, p.ne), urb = row_bytes(p.up_dt, p.ne);
  unsigned char* s_gate = smem;
  unsigned char* s_up = s_gate + af_region(TR * grb);
  uint32_t* s_lo = reinterpret_cast<uint32_t*>(s_up + af_region(TR * urb));  // [ne / 4] four low limbs per word
  uint32_t* s_hi = s_lo + p.ne / 4;
  int* s_sum = reinterpret_cast<int*>(s_hi + p.ne / 4);  // [ne / 16] Σ X per 16 elements
  const bool routed = (int)blockIdx.x < n_routed_jobs;
  int pair = 0, r, tile;
  const uint8_t *gsrc, *usrc;
  float* act_out;
  if (tid == 0) {
    mbar_init(&s_bar, 1);
    mbar_fence_init();
  }
  pdl_wait();     // ids and the fixed-point x come from kernels earlier in the stream
  pdl_trigger();  // only now: the next kernel reads ids as soon as it starts
  if (routed) {
    pair = blockIdx.x / tiles;
    tile = blockIdx.x % tiles;
    r = pair / p.n_used;
    int e = __ldcg(p.ids + pair);
    if (e < 0) return;  // a negative id marks a pair another rank serves
    if (e >= p.n_expert) {
      if (tid == 0) p.status->bad_index = 1;
      e = p.n_expert - 1;
    }
    if (!af_in_band(p, e)) return;
    gsrc = p.gate + (size_t)e * p.gate_stride + (size_t)tile * TR * grb;
    usrc = p.up + (size_t)e * p.up_stride + (size_t)tile * TR * urb;
    act_out = p.act + (size_t)pair * p.nff + tile * TR;
  } else {
    const int jb = blockIdx.x - n_routed_jobs;
    r = jb / sh_tiles;
    tile = jb % sh_tiles;
    gsrc = p.sh_gate + (size_t)tile * TR * grb;
    usrc = p.sh_up + (size_t)tile * TR * urb;
    act_out = p.act + (size_t)p.rows * p.n_used * p.nff + (size_t)r * p.sh_ff + tile * TR;
  }
  const uint32_t goff = (uint32_t)(reinterpret_cast<uintptr_t>(gsrc) & 127u), uoff = (uint32_t)(reinterpret_cast<uintptr_t>(usrc) & 127u);
  if (tid == 0) {
    mbar_arrive_expect_tx(&s_bar, (uint32_t)(TR * grb + TR * urb));
    bulk_g2s(s_gate + goff, gsrc, (uint32_t)(TR * grb), &s_bar);
    bulk_g2s(s_up + uoff, usrc, (uint32_t)(TR * urb), &s_bar);
  }
  {
    const uint32_t* xl = reinterpret_cast<const uint32_t*>(p.xq_lo + (size_t)r * p.ne);
    const uint32_t* xh = reinterpret_cast<const uint32_t*>(p.xq_hi + (size_t)r * p.ne);
    for (int i = tid; i < p.ne / 4; i += blockDim.x) {
      s_lo[i] = __ldcg(xl + i);
      s_hi[i] = __ldcg(xh + i);
    }
  }
  __syncthreads();  // limbs staged; the barrier's init is visible to every waiter
  for (int i = tid; i < p.ne / 16; i += blockDim.x) {
    int l = 0, h = 0;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      l = __dp4a(0x01010101, (int)s_lo[4 * i + w], l);
      h = __dp4a(0x01010101, (int)s_hi[4 * i + w], h);
    }
    s_sum[i] = h * 256 + l;
  }
  __syncthreads();
  const float q_scale = __ldcg(p.xscale + r);
  if (!mbar_wait_bounded(&s_bar, 0)) {
    // the copies never signalled: report, and make sure nothing is still landing in this CTA's
    // shared memory before it is handed to another CTA
    if (lane == 0) atomicExch(&p.status->timeout, 1);
    (void)mbar_wait_bounded(&s_bar, 0);
    return;
  }
  const int n16 = p.ne / 16;
  for (int rr = 0; rr < rpw; ++rr) {
    const int f = warp * rpw + rr;
    const uint8_t* grow = s_gate + goff + (size_t)f * grb;
    const uint8_t* urow = s_up + uoff + (size_t)f * urb;
    float gs = 0.f, us = 0.f;
#pragma unroll 2
    for (int h = lane; h < n16; h += 32) {
      const uint4 l4 = *reinterpret_cast<const uint4*>(s_lo + 4 * h), h4 = *reinterpret_cast<const uint4*>(s_hi + 4 * h);
      const int S = s_sum[h];
      gs += af_dot16(p.gate_dt, grow, h, l4, h4, S);
      us += af_dot16(p.up_dt, urow, h, l4, h4, S);
    }
    gs = warp_sum(gs) * q_scale;
    us = warp_sum(us) * q_scale;
    if (lane == 0) {
      const float wp = (routed && p.weight_before) ? __ldcg(p.wts + pair) : 1.0f;
      act_out[f] = gated_act(p.act_kind, routed ? p.clamp : 0.f, wp * gs, wp * us);
    }
  }
}

// One CTA = one token x TI output features (one per warp) x every slot.  Shared memory: per slot the
// TI rows of the expert's down matrix (one bulk copy and one mbarrier per slot), then the token's
// activations in fixed point.
__global__ void __launch_bounds__(256, 3) k_anyfmt_down(DecodeParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t s_bar[AF_MAX_SLOTS];
  __shared__ float s_w[AF_MAX_SLOTS], s_ds[AF_MAX_SLOTS];
  __shared__ int s_on[AF_MAX_SLOTS];
  __shared__ uint32_t s_off[AF_MAX_SLOTS];
  unsigned char* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, TI = blockDim.x >> 5;
  const bool has_sh = p.sh_down != nullptr;
  const int n_slots = p.n_used + (has_sh ? 1 : 0);
  const int n_act = p.n_used * p.nff + (has_sh ? p.sh_ff : 0), n_chunk = n_act / 128;
  const size_t drb = row_bytes(p.down_dt, p.nff), sh_drb = has_sh ? row_bytes(p.down_dt, p.sh_ff) : 0;
  const size_t slab = TI * drb, sh_slab = TI * sh_drb, slab_pad = af_region(slab);
  unsigned char* s_wt = smem;
  uint32_t* s_lo = reinterpret_cast<uint32_t*>(s_wt + (size_t)p.n_used * slab_pad + (has_sh ? af_region(sh_slab) : 0));  // [n_act / 4]
  uint32_t* s_hi = s_lo + n_act / 4;
  float* s_xsc = reinterpret_cast<float*>(s_hi + n_act / 4);  // [n_chunk] value of one step, per 128 activations
  int* s_s16 = reinterpret_cast<int*>(s_xsc + n_chunk);        // [n_act / 16]
  const int tiles = p.ne / TI;
  const int r = blockIdx.x / tiles, i0 = (blockIdx.x % tiles) * TI;

  // The routing result was complete before this kernel could start (the gate/up kernel releases its
  // dependents only after it has itself waited for the router): every slot's thread sets up the slot's
  // barrier and requests its slab at once, while the gate/up kernel may still be running.
  pdl_trigger();
  if (tid < n_slots) {
    const int s = tid;
    if (s < p.n_used) {
      int e = __ldcg(p.ids + r * p.n_used + s);
      const bool mine = e >= 0;
      if (e >= p.n_expert && blockIdx.x == 0) p.status->bad_index = 1;
      e = min(max(e, 0), p.n_expert - 1);
      s_on[s] = (mine && af_in_band(p, e)) ? e + 1 : 0;
      s_w[s] = p.weight_before ? 1.0f : __ldcg(p.wts + r * p.n_used + s);
      s_ds[s] = p.down_scale ? __ldg(p.down_scale + e) : 1.0f;
    } else {
      s_on[s] = 1;
      s_ds[s] = 1.0f;
      s_w[s] = p.sh_logit ? 1.0f / (1.0f + __expf(-__ldcg(p.sh_logit + r))) : 1.0f;
    }
    mbar_init(&s_bar[s], 1);
    mbar_fence_init();
    s_off[s] = 0;
    if (s_on[s]) {
      const bool sh = s >= p.n_used;
      const uint8_t* src = sh ? p.sh_down + (size_t)i0 * sh_drb : p.down + (size_t)(s_on[s] - 1) * p.down_stride + (size_t)i0 * drb;
      const uint32_t bytes = (uint32_t)(sh ? sh_slab : slab);
      s_off[s] = (uint32_t)(reinterpret_cast<uintptr_t>(src) & 127u);
      mbar_arrive_expect_tx(&s_bar[s], bytes);
      bulk_g2s(s_wt + (size_t)s * slab_pad + s_off[s], src, bytes, &s_bar[s]);
    }
  }
  pdl_wait();  // the activations come from the gate/up kernel
  // this token's activations (routed slots, then the shared expert) -> fixed point, one warp per 128,
  // two chunks per pass so that their loads overlap: X = round(a * 32639 / max|a|), X = 256 hi + lo
  {
    const float* a_src = p.act + (size_t)r * p.n_used * p.nff;
    const float* sh_src = p.act + (size_t)p.rows * p.n_used * p.nff + (size_t)r * p.sh_ff;
    const int n_routed_chunk = p.n_used * p.nff / 128;
    auto src_of = [&](int c) { return reinterpret_cast<const float4*>(c < n_routed_chunk ? a_src + (size_t)c * 128 : sh_src + (size_t)(c - n_routed_chunk) * 128) + lane; };
    for (int c0 = warp; c0 < n_chunk; c0 += 2 * TI) {
      const int c1 = c0 + TI;
      const float4 v0 = __ldcg(src_of(c0));
      const float4 v1 = c1 < n_chunk ? __ldcg(src_of(c1)) : make_float4(0.f, 0.f, 0.f, 0.f);
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
        s_lo[c * 32 + lane] = lo;
        s_hi[c * 32 + lane] = hi;
        int sx = (X[0] + X[1]) + (X[2] + X[3]);  // 16 elements sit in four neighbouring lanes
        sx += __shfl_xor_sync(0xFFFFFFFFu, sx, 1);
        sx += __shfl_xor_sync(0xFFFFFFFFu, sx, 2);
        if ((lane & 3) == 0) s_s16[c * 8 + (lane >> 2)] = sx;
        if (lane == 0) s_xsc[c] = m / 32639.f;
      }
    }
  }
  __syncthreads();

  float o = 0.f;
  bool ok = true;
  for (int s = 0; s < n_slots && ok; ++s) {
    if (!s_on[s]) continue;
    if (!mbar_wait_bounded(&s_bar[s], 0)) { ok = false; break; }
    const bool shared_slot = s >= p.n_used;
    const uint8_t* wrow = s_wt + (size_t)s * slab_pad + s_off[s] + (size_t)warp * (shared_slot ? sh_drb : drb);
    const int n16 = (shared_slot ? p.sh_ff : p.nff) / 16, base16 = (shared_slot ? p.n_used * p.nff : s * p.nff) / 16;
    float acc = 0.f;
#pragma unroll 2
    for (int h = lane; h < n16; h += 32) {
      const int idx = base16 + h;
      const uint4 l4 = *reinterpret_cast<const uint4*>(s_lo + 4 * idx), h4 = *reinterpret_cast<const uint4*>(s_hi + 4 * idx);
      acc = fmaf(s_xsc[idx >> 3], af_dot16(p.down_dt, wrow, h, l4, h4, s_s16[idx]), acc);
    }
    acc = warp_sum(acc);
    o += s_w[s] * (acc * s_ds[s]);  // rank order, the shared expert last (the CPU's order)
  }
  if (!ok) {
    if (lane == 0) atomicExch(&p.status->timeout, 2);
    for (int s = 0; s < n_slots; ++s)
      if (s_on[s]) (void)mbar_wait_bounded(&s_bar[s], 0);
    return;
  }
  if (lane == 0) {
    const int i = i0 + warp;
    if (p.residual != nullptr) o += __ldcg(p.residual + (size_t)r * p.ne + i);
    p.dst[(size_t)r * p.ne + i] = o;
  }
}

size_t af_gateup_smem(int ne, int TR, size_t grb, size_t urb) {
  return 128 + af_region(TR * grb) + af_region(TR * urb) + (size_t)ne * 2 + (size_t)ne / 16 * 4;
}
size_t af_down_smem(int TI, int nff, int sh_ff, int n_used, int down_dt) {
  const size_t n_act = (size_t)n_used * nff + sh_ff;
  return 128 + (size_t)n_used * af_region(TI * row_bytes(down_dt, nff)) + (sh_ff ? af_region(TI * row_bytes(down_dt, sh_ff)) : 0) + n_act * 2 +
         n_act / 128 * 4 + n_act / 16 * 4;
}

// Rows per warp of the gate/up kernel (8 warps): 2, or 1 when two do not fit; 0 = no shape fits.
int af_pick_rpw(int ne, int nff, int sh_ff, BankTypes bt) {
  for (int rpw : {2, 1}) {
    const int TR = 8 * rpw;
    if (nff % TR || sh_ff % TR) continue;
    if (af_gateup_smem(ne, TR, row_bytes(bt.gate, ne), row_bytes(bt.up, ne)) <= 160 * 1024) return rpw;
  }
  return 0;
}
// Output features (= warps) per CTA of the down kernel: a slab of TI rows must be a multiple of 16 bytes.
int af_pick_ti(int ne, int nff, int sh_ff, int n_used, BankTypes bt) {
  for (int TI : {8, 4}) {
    if (ne % TI) continue;
    if ((TI * row_bytes(bt.down, nff)) % 16 || (sh_ff && (TI * row_bytes(bt.down, sh_ff)) % 16)) continue;
    if (af_down_smem(TI, nff, sh_ff, n_used, bt.down) <= 200 * 1024) return TI;
  }
  return 0;
}

}  // namespace

bool anyfmt_decode_supported(int ne, int nff, int sh_ff, int n_used, BankTypes bt, std::string* why) {
  if (ne % 256 || nff % 256 || sh_ff % 256) {
    if (why) *why = "small-m path: ne, n_ff_exp and sh_ff must be multiples of 256";
    return false;
  }
  if (n_used + 1 > AF_MAX_SLOTS) {
    if (why) *why = "small-m path: n_used larger than 32 is not covered";
    return false;
  }
  if (!af_pick_rpw(ne, nff, sh_ff, bt) || !af_pick_ti(ne, nff, sh_ff, n_used, bt)) {
    if (why) *why = "small-m path: tile does not fit shared memory for these dims and bank formats";
    return false;
  }
  return true;
}

int32_t launch_anyfmt_decode(infr_cuda_ctx* ctx, const DecodeParams& p, bool pdl, uint32_t stages) {
  const bool has_sh = p.sh_gate != nullptr;
  const int sh_ff = has_sh ? p.sh_ff : 0;
  const BankTypes bt = {p.gate_dt, p.up_dt, p.down_dt};
  const int rpw = af_pick_rpw(p.ne, p.nff, sh_ff, bt), TI = af_pick_ti(p.ne, p.nff, sh_ff, p.n_used, bt);
  if (!rpw || !TI) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "small-m path: tile does not fit shared memory");
  cudaError_t e;
  if (stages & 2u) {
    const int TR = 8 * rpw;
    const size_t smem = af_gateup_smem(p.ne, TR, row_bytes(bt.gate, p.ne), row_bytes(bt.up, p.ne));
    if ((e = ensure_smem(reinterpret_cast<const void*>(k_anyfmt_gateup), smem)) != cudaSuccess) return check_cuda(ctx, e, "k_anyfmt_gateup smem attribute");
    const int jobs = p.rows * p.n_used * (p.nff / TR) + (has_sh ? p.rows * (sh_ff / TR) : 0);
    e = launch_ex(k_anyfmt_gateup, dim3(jobs), dim3(256), smem, ctx->stream, pdl, p, rpw);
    ctx->launches += 1;
    if (e != cudaSuccess) return check_cuda(ctx, e, "k_anyfmt_gateup launch");
  }
  if (stages & 4u) {
    const size_t smem = af_down_smem(TI, p.nff, sh_ff, p.n_used, bt.down);
    if ((e = ensure_smem(reinterpret_cast<const void*>(k_anyfmt_down), smem)) != cudaSuccess) return check_cuda(ctx, e, "k_anyfmt_down smem attribute");
    e = launch_ex(k_anyfmt_down, dim3(p.rows * (p.ne / TI)), dim3(TI * 32), smem, ctx->stream, pdl, p);
    ctx->launches += 1;
    if (e != cudaSuccess) return check_cuda(ctx, e, "k_anyfmt_down launch");
  }
  return check_cuda(ctx, cudaGetLastError(), "generic-format small-m launch");
}

cudaError_t publish_codebooks_anyfmt(const unsigned char* const* tables) { return publish_codebooks(tables); }

}  // namespace infr
