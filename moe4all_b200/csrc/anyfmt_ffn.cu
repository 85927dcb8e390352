// Small-m expert FFN for banks in any mix of Q4_K, Q5_K, Q6_K and Q8_0 (the reference's batched and
// decode MoE kernels take gate, up and down formats independently: crates/infr-core/src/tensor.rs:172-196;
// real files mix them, e.g. Q5_K gate/up with Q6_K down, or Q8_0 throughout).
//
//   k_anyfmt_gateup : act[p, f] = act_fn(W_gate[e_p][f,:]·x, W_up[e_p][f,:]·x)
//   k_anyfmt_down   : dst[r, i] = Σ_slot w_slot · (W_down[e_slot][i,:]·act[slot,:])  (+ shared expert, + residual)
//
// Same arithmetic as the tuned per-pair kernels (decode_ffn.cu): activations in 16-bit fixed point
// (two signed 8-bit limbs), exact integer dot products against the 8-bit codes of formats.cuh, the
// scale group's affine map applied in f32 per 16 weights, slots summed in rank order.  The kernels read
// the blocks straight from global memory (one warp per weight row, lanes side by side along the
// row), which keeps them independent of any format's block size and alignment.
// CPU reference: crates/infr-cpu/src/lib.rs:4051-4303.
#include "formats.cuh"
#include "kernels.cuh"

namespace infr {

namespace {

constexpr int AF_WARPS = 8;
constexpr int AF_GU_ROWS = 2;  // weight rows per warp and role in the gate/up kernel
constexpr int AF_MAX_SLOTS = 33;

__device__ __forceinline__ bool af_in_band(const DecodeParams& p, int e) {
  return p.ep_n == 0 || ((uint32_t)e >= p.ep_lo && (uint32_t)e < p.ep_lo + p.ep_n);
}

// Σ over 16 weights of w * X, in units of the activation's fixed-point step: l4 / h4 = the 16 low
// and high limbs, S = Σ X.
__device__ __forceinline__ float af_dot16(int dt, const uint8_t* __restrict__ row, int h, const uint4& l4, const uint4& h4, int S) {
  uint32_t c[4];
  float A, B;
  int off;
  fmt_codes16(dt, row, h, c, A, B, off);
  int dl = dp4a_us(c[0], (int)l4.x, 0), dh = dp4a_us(c[0], (int)h4.x, 0);
  dl = dp4a_us(c[1], (int)l4.y, dl); dh = dp4a_us(c[1], (int)h4.y, dh);
  dl = dp4a_us(c[2], (int)l4.z, dl); dh = dp4a_us(c[2], (int)h4.z, dh);
  dl = dp4a_us(c[3], (int)l4.w, dl); dh = dp4a_us(c[3], (int)h4.w, dh);
  const int t = dh * 256 + dl - off * S;  // |t| < 2^28
  return fmaf(A, (float)t, B * (float)S);
}

// One CTA = one (token, slot) pair (or one row of the shared expert) x 16 output features, both roles.
__global__ void __launch_bounds__(AF_WARPS * 32) k_anyfmt_gateup(DecodeParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint32_t* s_lo = reinterpret_cast<uint32_t*>(smem);  // [ne / 4] four low limbs per word
  uint32_t* s_hi = s_lo + p.ne / 4;
  int* s_sum = reinterpret_cast<int*>(s_hi + p.ne / 4);  // [ne / 16] Σ X per 16 elements
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int TR = AF_WARPS * AF_GU_ROWS;
  const int tiles = p.nff / TR, sh_tiles = p.sh_ff / TR;
  const int n_routed_jobs = p.rows * p.n_used * tiles;
  const size_t grb = row_bytes(p.gate_dt, p.ne), urb = row_bytes(p.up_dt, p.ne);
  const bool routed = (int)blockIdx.x < n_routed_jobs;
  int pair = 0, r, tile;
  const uint8_t *gbase, *ubase;
  float* act_out;
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
    gbase = p.gate + (size_t)e * p.gate_stride + (size_t)tile * TR * grb;
    ubase = p.up + (size_t)e * p.up_stride + (size_t)tile * TR * urb;
    act_out = p.act + (size_t)pair * p.nff + tile * TR;
  } else {
    const int jb = blockIdx.x - n_routed_jobs;
    r = jb / sh_tiles;
    tile = jb % sh_tiles;
    gbase = p.sh_gate + (size_t)tile * TR * grb;
    ubase = p.sh_up + (size_t)tile * TR * urb;
    act_out = p.act + (size_t)p.rows * p.n_used * p.nff + (size_t)r * p.sh_ff + tile * TR;
  }
  {
    const uint32_t* xl = reinterpret_cast<const uint32_t*>(p.xq_lo + (size_t)r * p.ne);
    const uint32_t* xh = reinterpret_cast<const uint32_t*>(p.xq_hi + (size_t)r * p.ne);
    for (int i = tid; i < p.ne / 4; i += AF_WARPS * 32) {
      s_lo[i] = __ldcg(xl + i);
      s_hi[i] = __ldcg(xh + i);
    }
  }
  __syncthreads();
  for (int i = tid; i < p.ne / 16; i += AF_WARPS * 32) {
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
  const int n16 = p.ne / 16;
#pragma unroll
  for (int rr = 0; rr < AF_GU_ROWS; ++rr) {
    const int f = warp * AF_GU_ROWS + rr;
    const uint8_t* grow = gbase + (size_t)f * grb;
    const uint8_t* urow = ubase + (size_t)f * urb;
    float gs = 0.f, us = 0.f;
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

// One CTA = one token x 8 output features x every slot; a warp owns one output feature.
__global__ void __launch_bounds__(AF_WARPS * 32) k_anyfmt_down(DecodeParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ float s_w[AF_MAX_SLOTS], s_ds[AF_MAX_SLOTS];
  __shared__ int s_on[AF_MAX_SLOTS];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool has_sh = p.sh_down != nullptr;
  const int n_slots = p.n_used + (has_sh ? 1 : 0);
  const int n_act = p.n_used * p.nff + (has_sh ? p.sh_ff : 0), n_chunk = n_act / 128;
  uint32_t* s_lo = reinterpret_cast<uint32_t*>(smem);  // [n_act / 4]
  uint32_t* s_hi = s_lo + n_act / 4;
  float* s_xsc = reinterpret_cast<float*>(s_hi + n_act / 4);  // [n_chunk] value of one step, per 128 activations
  int* s_s16 = reinterpret_cast<int*>(s_xsc + n_chunk);        // [n_act / 16]
  const int tiles = p.ne / AF_WARPS;
  const int r = blockIdx.x / tiles, i = (blockIdx.x % tiles) * AF_WARPS + warp;

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
  }
  // this token's activations (routed slots, then the shared expert) -> fixed point, one warp per 128:
  // X = round(a * 32639 / max|a|), X = 256 hi + lo with signed 8-bit limbs
  {
    const float* a_src = p.act + (size_t)r * p.n_used * p.nff;
    const float* sh_src = p.act + (size_t)p.rows * p.n_used * p.nff + (size_t)r * p.sh_ff;
    const int n_routed_chunk = p.n_used * p.nff / 128;
    for (int c = warp; c < n_chunk; c += AF_WARPS) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(c < n_routed_chunk ? a_src + (size_t)c * 128 : sh_src + (size_t)(c - n_routed_chunk) * 128) + lane);
      const float m = warp_max(fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
      const float inv = m > 0.f ? 32639.f / m : 0.f;
      const int X[4] = {__float2int_rn(v.x * inv), __float2int_rn(v.y * inv), __float2int_rn(v.z * inv), __float2int_rn(v.w * inv)};
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int hh = (X[t] + 128) >> 8, ll = X[t] - (hh << 8);
        lo |= (uint32_t)(ll & 0xFF) << (8 * t);
        hi |= (uint32_t)(hh & 0xFF) << (8 * t);
      }
      s_lo[c * 32 + lane] = lo;
      s_hi[c * 32 + lane] = hi;
      int sx = (X[0] + X[1]) + (X[2] + X[3]);  // 16 elements sit in four neighbouring lanes
      sx += __shfl_xor_sync(0xFFFFFFFFu, sx, 1);
      sx += __shfl_xor_sync(0xFFFFFFFFu, sx, 2);
      if ((lane & 3) == 0) s_s16[c * 8 + (lane >> 2)] = sx;
      if (lane == 0) s_xsc[c] = m / 32639.f;
    }
  }
  __syncthreads();

  const size_t drb = row_bytes(p.down_dt, p.nff), sh_drb = row_bytes(p.down_dt, p.sh_ff);
  float o = 0.f;
  for (int s = 0; s < n_slots; ++s) {
    if (!s_on[s]) continue;
    const bool shared_slot = s >= p.n_used;
    const uint8_t* wrow = shared_slot ? p.sh_down + (size_t)i * sh_drb : p.down + (size_t)(s_on[s] - 1) * p.down_stride + (size_t)i * drb;
    const int n16 = (shared_slot ? p.sh_ff : p.nff) / 16, base16 = (shared_slot ? p.n_used * p.nff : s * p.nff) / 16;
    float acc = 0.f;
    for (int h = lane; h < n16; h += 32) {
      const int idx = base16 + h;
      const uint4 l4 = *reinterpret_cast<const uint4*>(s_lo + 4 * idx), h4 = *reinterpret_cast<const uint4*>(s_hi + 4 * idx);
      acc = fmaf(s_xsc[idx >> 3], af_dot16(p.down_dt, wrow, h, l4, h4, s_s16[idx]), acc);
    }
    acc = warp_sum(acc);
    o += s_w[s] * (acc * s_ds[s]);  // rank order, the shared expert last (the CPU's order)
  }
  if (lane == 0) {
    if (p.residual != nullptr) o += __ldcg(p.residual + (size_t)r * p.ne + i);
    p.dst[(size_t)r * p.ne + i] = o;
  }
}

size_t af_gateup_smem(int ne) { return (size_t)ne * 2 + (size_t)ne / 16 * 4; }
size_t af_down_smem(int nff, int sh_ff, int n_used) {
  const size_t n_act = (size_t)n_used * nff + sh_ff;
  return n_act * 2 + n_act / 128 * 4 + n_act / 16 * 4;
}

}  // namespace

bool anyfmt_decode_supported(int ne, int nff, int sh_ff, int n_used, std::string* why) {
  if (ne % 256 || nff % 256 || sh_ff % 256) {
    if (why) *why = "small-m path: ne, n_ff_exp and sh_ff must be multiples of 256";
    return false;
  }
  if (n_used + 1 > AF_MAX_SLOTS) {
    if (why) *why = "small-m path: n_used larger than 32 is not covered";
    return false;
  }
  if (af_gateup_smem(ne) > 200 * 1024 || af_down_smem(nff, sh_ff, n_used) > 200 * 1024) {
    if (why) *why = "small-m path: a token's activations do not fit shared memory for these dims";
    return false;
  }
  return true;
}

int32_t launch_anyfmt_decode(infr_cuda_ctx* ctx, const DecodeParams& p, uint32_t stages) {
  const bool has_sh = p.sh_gate != nullptr;
  const int sh_ff = has_sh ? p.sh_ff : 0;
  constexpr int TR = AF_WARPS * AF_GU_ROWS;
  cudaError_t e;
  if (stages & 2u) {
    const size_t smem = af_gateup_smem(p.ne);
    if ((e = ensure_smem(reinterpret_cast<const void*>(k_anyfmt_gateup), smem)) != cudaSuccess) return check_cuda(ctx, e, "k_anyfmt_gateup smem attribute");
    const int jobs = p.rows * p.n_used * (p.nff / TR) + (has_sh ? p.rows * (sh_ff / TR) : 0);
    k_anyfmt_gateup<<<jobs, AF_WARPS * 32, smem, ctx->stream>>>(p);
    ctx->launches += 1;
  }
  if (stages & 4u) {
    const size_t smem = af_down_smem(p.nff, sh_ff, p.n_used);
    if ((e = ensure_smem(reinterpret_cast<const void*>(k_anyfmt_down), smem)) != cudaSuccess) return check_cuda(ctx, e, "k_anyfmt_down smem attribute");
    k_anyfmt_down<<<p.rows * (p.ne / AF_WARPS), AF_WARPS * 32, smem, ctx->stream>>>(p);
    ctx->launches += 1;
  }
  return check_cuda(ctx, cudaGetLastError(), "generic-format small-m launch");
}

}  // namespace infr
