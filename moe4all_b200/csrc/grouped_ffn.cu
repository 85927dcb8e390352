// Batched (prefill / many-stream) expert FFN: token permute + grouped GEMM + un-permute combine.
//
//   k_pair_count / k_segment_scan / k_pair_scatter   a9  bucket the (token, rank) pairs by expert
//   k_gather_rows                                    a9  token rows -> f16, expert-contiguous
//   k_grouped_gateup                                 a10 act = silu(Wg x) * (Wu x) per expert segment
//   k_grouped_down                                   a10 y = Wd act per expert segment
//   k_unpermute_combine                              a11 dst[t] = sum_rank w * y[pos(t, rank)] (+ shared)
//
// Reference: CPU stages A-E crates/infr-cpu/src/lib.rs:3865-4303 (bucket by expert :3873-3907,
// expert GEMMs in 64-row chunks :3992-4245, rank-ordered accumulate :4287-4303); Vulkan batched arm
// crates/infr-vulkan/src/adapter.rs:9020-9380 with shaders moe_bucket_{count,scan,scatter}.comp,
// native_gemm_mmq_q4k/q6k.comp (int8 dp4a tiles) and moe_scatter_reduce.comp.
//
// Tiles: weights are the M operand (64 output features per role and CTA), tokens the N operand
// (64 per CTA), so a weight block is unpacked once per 64 tokens.  Blocks are unpacked to f16 in
// shared memory (codes are exact in f16; block scales are applied in f16 after a 2^8 pre-scale
// that keeps them out of the subnormal range) and multiplied on the tensor cores with f32
// accumulation.  Activations are f16 as well: with bf16 operands the layer misses the 2e-3 bound
// on the synthetic distributions (3.7e-3 measured by emulation), with f16 it is 4.5e-4.
//
// K order: unpacking a 32-bit word of codes yields pairs (e0,e2),(e1,e3); tiles therefore hold
// every aligned group of four K elements in the order 0,2,1,3, and the token-side arrays (xg,
// act) are written in the same order.
#include <mma.h>

#include <algorithm>
#include <cstdlib>

#include "formats.cuh"
#include "kernels.cuh"

namespace infr {

namespace {

constexpr int TM = 64;       // weight rows per role and CTA
constexpr int TN = 64;       // tokens per CTA
constexpr int TK = 64;       // K elements per step
constexpr int PITCH = 72;    // halfs per shared-memory row (144 B: conflict-free ldmatrix)
constexpr int GG_THREADS = 256;
constexpr float W_PRESCALE = 256.0f;
constexpr float W_POSTSCALE = 1.0f / 256.0f;

__device__ __forceinline__ int kperm(int k) {  // position of element k inside its group of four
  const int r = k & 3;
  return (k & ~3) | (r == 1 ? 2 : (r == 2 ? 1 : r));
}

// ---- permute -------------------------------------------------------------------------------------

__global__ void k_pair_count(const int32_t* __restrict__ ids, int n_pairs, int n_expert, uint32_t ep_lo, uint32_t ep_n,
                             int* __restrict__ counts, DeviceStatus* status) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n_pairs) return;
  int e = ids[p];
  if (e < 0) return;  // a negative id marks a pair another rank serves
  if (e >= n_expert) status->bad_index = 1;  // served as the last expert, reported at the next sync
  e = min(e, n_expert - 1);
  if (ep_n && ((uint32_t)e < ep_lo || (uint32_t)e >= ep_lo + ep_n)) return;
  atomicAdd(&counts[e], 1);
}

// Exclusive prefix sums of (a, b) over the 1024 threads of the CTA; totals returned through
// `ta`, `tb`.  s_ws: 2 x 32 ints of scratch.
__device__ __forceinline__ void block_scan2(int& a, int& b, int& ta, int& tb, int* s_ws) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int ia = a, ib = b;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int ua = __shfl_up_sync(0xFFFFFFFFu, ia, o), ub = __shfl_up_sync(0xFFFFFFFFu, ib, o);
    if (lane >= o) {
      ia += ua;
      ib += ub;
    }
  }
  if (lane == 31) {
    s_ws[warp] = ia;
    s_ws[32 + warp] = ib;
  }
  __syncthreads();
  if (warp == 0) {
    int wa = s_ws[lane], wb = s_ws[32 + lane];
    const int oa = wa, ob = wb;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int ua = __shfl_up_sync(0xFFFFFFFFu, wa, o), ub = __shfl_up_sync(0xFFFFFFFFu, wb, o);
      if (lane >= o) {
        wa += ua;
        wb += ub;
      }
    }
    s_ws[lane] = wa - oa;  // exclusive warp offsets
    s_ws[32 + lane] = wb - ob;
    if (lane == 31) {
      s_ws[64] = wa;
      s_ws[65] = wb;
    }
  }
  __syncthreads();
  a = ia - a + s_ws[warp];
  b = ib - b + s_ws[32 + warp];
  ta = s_ws[64];
  tb = s_ws[65];
}

// Exclusive scan of the per-expert counts (thread e holds the count of segment e), the tile table
// (one entry per `tn` rows of a segment, the shared expert's rows appended as segment n_expert) and
// the segment offsets, by the 1024 threads of one CTA.  Offsets stay in s_off for the caller.
// Tiles are listed heaviest first - the full tiles of all segments, then the segments' last, partial
// tiles by falling row count - so that the GEMM kernels' last wave of CTAs is made of the light ones
// (a tile's index only names its slot in the token and activation arrays).  tn is a power of two.
__device__ __forceinline__ void segment_tables(int cnt, int n_expert, int shared_rows, int tn, int* __restrict__ seg_off,
                                               int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                               int* __restrict__ tile_rows, int* __restrict__ n_tiles, int* s_cnt, int* s_off,
                                               int* s_toff, int* s_ws) {
  const int tid = threadIdx.x;
  const int n_seg = n_expert + (shared_rows > 0 ? 1 : 0);
  int off = cnt, foff = cnt / tn, total = 0, total_f = 0;  // rows and full tiles ahead of this segment
  block_scan2(off, foff, total, total_f, s_ws);
  if (tid < n_seg) {
    s_cnt[tid] = cnt;
    s_off[tid] = off;
    s_toff[tid] = foff;
  }
  // partial tiles: the count over the CTA; segment 1024 (only with 1024 experts and a shared segment) is added below
  int n_part = __syncthreads_count(tid < n_seg && (cnt & (tn - 1)) != 0);
  if (n_seg > 1024) {
    if (tid == 0) {
      s_cnt[1024] = shared_rows;
      s_off[1024] = total;
      s_toff[1024] = total_f;
    }
    total += shared_rows;
    total_f += shared_rows / tn;
    n_part += (shared_rows & (tn - 1)) != 0;
  }
  if (tid == 0) {
    s_off[n_seg] = total;
    *n_tiles = total_f + n_part;
    seg_off[n_expert + 1] = total;  // total grouped rows, with or without a shared segment
  }
  __syncthreads();
  for (int e = tid; e <= n_seg; e += 1024) seg_off[e] = s_off[e];
  for (int e = tid; e < n_seg; e += 1024) {
    const int nf = s_cnt[e] / tn, part = s_cnt[e] & (tn - 1);
    for (int t = 0; t < nf; ++t) {
      tile_expert[s_toff[e] + t] = e;
      tile_row0[s_toff[e] + t] = s_off[e] + t * tn;
      tile_rows[s_toff[e] + t] = tn;
    }
    if (part) {
      int rank = 0;  // partial tiles with more rows, or as many in an earlier segment
      for (int o = 0; o < n_seg; ++o) {
        const int po = s_cnt[o] & (tn - 1);
        rank += (po > part) || (po == part && o < e);
      }
      tile_expert[total_f + rank] = e;
      tile_row0[total_f + rank] = s_off[e] + nf * tn;
      tile_rows[total_f + rank] = part;
    }
  }
}

// One CTA: the tables above from counts made by k_pair_count, and the fill cursors reset.
__global__ void __launch_bounds__(1024) k_segment_scan(const int* __restrict__ counts, int n_expert, int shared_rows, int tn,
                                                       int* __restrict__ seg_off, int* __restrict__ fill,
                                                       int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                                       int* __restrict__ tile_rows, int* __restrict__ n_tiles) {
  __shared__ int s_cnt[1025], s_off[1026], s_toff[1026], s_ws[66];
  const int tid = threadIdx.x;
  const int n_seg = n_expert + (shared_rows > 0 ? 1 : 0);
  const int cnt = tid < n_seg ? (tid < n_expert ? counts[tid] : shared_rows) : 0;
  segment_tables(cnt, n_expert, shared_rows, tn, seg_off, tile_expert, tile_row0, tile_rows, n_tiles, s_cnt, s_off, s_toff, s_ws);
  for (int e = tid; e < n_expert; e += 1024) fill[e] = 0;
}

// Calls of up to a few hundred thousand pairs: count, scan and scatter by one CTA with the
// histogram and the cursors in shared memory - one launch instead of a memset and three kernels.
__device__ __forceinline__ int bucket_of(int e, int n_expert, uint32_t ep_lo, uint32_t ep_n, DeviceStatus* status) {
  if (e < 0) return -1;  // a negative id marks a pair another rank serves
  if (e >= n_expert) status->bad_index = 1;  // served as the last expert, reported at the next sync
  e = min(e, n_expert - 1);
  if (ep_n && ((uint32_t)e < ep_lo || (uint32_t)e >= ep_lo + ep_n)) return -1;
  return e;
}
__global__ void __launch_bounds__(1024) k_bucket_fused(const int32_t* __restrict__ ids, int n_pairs, int n_expert, uint32_t ep_lo,
                                                       uint32_t ep_n, int shared_rows, int tn, int* __restrict__ seg_off,
                                                       int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                                       int* __restrict__ tile_rows, int* __restrict__ n_tiles,
                                                       int* __restrict__ pos_of_pair, int* __restrict__ pair_of_pos,
                                                       DeviceStatus* status) {
  __shared__ int s_cnt[1025], s_off[1026], s_toff[1026], s_ws[66], s_hist[1024];
  const int tid = threadIdx.x;
  s_hist[tid] = 0;
  __syncthreads();
  // eight ids per thread in flight: the loop is a chain of global-memory latencies otherwise
  for (int p0 = tid; p0 < n_pairs; p0 += 8 * 1024) {
    int idv[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) idv[u] = p0 + u * 1024 < n_pairs ? ids[p0 + u * 1024] : -1;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int e = bucket_of(idv[u], n_expert, ep_lo, ep_n, status);
      if (e >= 0) atomicAdd(&s_hist[e], 1);
    }
  }
  __syncthreads();
  const int n_seg = n_expert + (shared_rows > 0 ? 1 : 0);
  const int cnt = tid < n_seg ? (tid < n_expert ? s_hist[tid] : shared_rows) : 0;
  __syncthreads();
  s_hist[tid] = 0;  // now the fill cursors
  segment_tables(cnt, n_expert, shared_rows, tn, seg_off, tile_expert, tile_row0, tile_rows, n_tiles, s_cnt, s_off, s_toff, s_ws);
  __syncthreads();
  for (int p0 = tid; p0 < n_pairs; p0 += 8 * 1024) {
    int idv[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) idv[u] = p0 + u * 1024 < n_pairs ? ids[p0 + u * 1024] : -1;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int p = p0 + u * 1024;
      if (p >= n_pairs) break;
      const int e = bucket_of(idv[u], n_expert, ep_lo, ep_n, status);
      if (e < 0) {
        pos_of_pair[p] = -1;
      } else {
        const int pos = s_off[e] + atomicAdd(&s_hist[e], 1);
        pos_of_pair[p] = pos;
        pair_of_pos[pos] = p;
      }
    }
  }
}

__global__ void k_pair_scatter(const int32_t* __restrict__ ids, int n_pairs, int n_expert, uint32_t ep_lo, uint32_t ep_n,
                               const int* __restrict__ seg_off, int* __restrict__ fill, int* __restrict__ pos_of_pair,
                               int* __restrict__ pair_of_pos) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n_pairs) return;
  int e = ids[p];
  const bool other = e < 0;
  e = min(max(e, 0), n_expert - 1);
  if (other || (ep_n && ((uint32_t)e < ep_lo || (uint32_t)e >= ep_lo + ep_n))) {
    pos_of_pair[p] = -1;
    return;
  }
  const int pos = seg_off[e] + atomicAdd(&fill[e], 1);
  pos_of_pair[p] = pos;
  pair_of_pos[pos] = p;
}

// xg[pos, kperm(k)] = f16(x[token(pos), k]); one warp per destination row.
//   pair_of_pos == nullptr: identity (rows already grouped);  rows >= n_sorted are the shared
//   expert's copy of every token in natural order.
__global__ void __launch_bounds__(256) k_gather_rows(const float* __restrict__ x, const int* __restrict__ pair_of_pos,
                                                     const float* __restrict__ row_w, const int* __restrict__ seg_off,
                                                     int n_seg_routed, int n_used, int total_rows_bound, int ne,
                                                     __half* __restrict__ xg) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= total_rows_bound) return;
  const int n_sorted = seg_off[n_seg_routed];
  int tok;
  float w = 1.0f;  // weight_before: the pair's routing weight on the expert's input row
  if (row < n_sorted) {
    tok = pair_of_pos ? pair_of_pos[row] / n_used : row;
    if (row_w != nullptr && pair_of_pos != nullptr) w = row_w[pair_of_pos[row]];
  } else {
    tok = row - n_sorted;  // shared-expert segment: token order
  }
  const int n_total = seg_off[n_seg_routed + 1];
  if (row >= n_total) return;
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)tok * ne);
  __half2* dst = reinterpret_cast<__half2*>(xg + (size_t)row * ne);
  for (int i = lane; i < ne / 4; i += 32) {
    float4 v = __ldg(src + i);
    v.x *= w; v.y *= w; v.z *= w; v.w *= w;
    dst[2 * i] = __floats2half2_rn(v.x, v.z);      // positions 0,1 <- elements 0,2
    dst[2 * i + 1] = __floats2half2_rn(v.y, v.w);  // positions 2,3 <- elements 1,3
  }
}

// The same rows as operand tiles for the tcgen05 kernels: [tile][K step of 64][256 rows][128 B],
// every 128-byte line already in the 128-byte-swizzled order of its shared-memory image (16-byte
// chunk c of row n at chunk position c ^ (n & 7)), so that a CTA fetches a step's whole token
// operand with one bulk copy.  One warp per row of a tile.
__global__ void __launch_bounds__(256) k_gather_tiles(const float* __restrict__ x, const int* __restrict__ pair_of_pos,
                                                      const float* __restrict__ row_w, const int* __restrict__ seg_off,
                                                      int n_seg_routed, int n_used,
                                                      const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
                                                      const int* __restrict__ n_tiles, int tn, int ne,
                                                      unsigned char* __restrict__ xt) {
  const int tile = blockIdx.y;
  if (tile >= *n_tiles) return;
  const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (n >= tile_rows[tile]) return;
  const int row = tile_row0[tile] + n;
  const int n_sorted = seg_off[n_seg_routed];
  int tok;
  float w = 1.0f;  // weight_before: the pair's routing weight on the expert's input row
  if (row < n_sorted) {
    tok = pair_of_pos ? pair_of_pos[row] / n_used : row;
    if (row_w != nullptr && pair_of_pos != nullptr) w = row_w[pair_of_pos[row]];
  } else {
    tok = row - n_sorted;  // shared-expert segment: token order
  }
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)tok * ne);
  const size_t step_bytes = (size_t)tn * 128;
  unsigned char* line0 = xt + (size_t)tile * (ne / 64) * step_bytes + (size_t)n * 128;
  for (int i = lane; i < ne / 4; i += 32) {
    float4 v = __ldg(src + i);
    v.x *= w; v.y *= w; v.z *= w; v.w *= w;
    const __half2 h02 = __floats2half2_rn(v.x, v.z), h13 = __floats2half2_rn(v.y, v.w);  // K order 0,2,1,3
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&h02);
    o.y = *reinterpret_cast<const uint32_t*>(&h13);
    const int step = i >> 4, chunk = (i & 15) >> 1;
    *reinterpret_cast<uint2*>(line0 + (size_t)step * step_bytes + ((chunk ^ (n & 7)) << 4) + (i & 1) * 8) = o;
  }
}

// ---- tensor-core tile helpers ----------------------------------------------------------------------

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const __half* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}

__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Four 4-bit codes (nibble position `shift` of the bytes of w) -> two half2 of code values in the
// order (b0,b2),(b1,b3), then code * s + m.
__device__ __forceinline__ void q4_word_to_h2(uint32_t w, __half2 s, __half2 m, uint32_t& out02, uint32_t& out13) {
  const __half2 k1024 = __float2half2_rn(1024.f);
  const __half2 a = __hsub2(u32_as_h2((w & 0x000F000Fu) | 0x64006400u), k1024);
  const __half2 b = __hsub2(u32_as_h2(((w >> 8) & 0x000F000Fu) | 0x64006400u), k1024);
  out02 = h2_as_u32(__hfma2(a, s, m));
  out13 = h2_as_u32(__hfma2(b, s, m));
}

// One K step of the tensor-core loop for a warp: 16 weight rows x 32 tokens, NR roles.
template <int NR>
__device__ __forceinline__ void mma_step(const __half* As, const __half* Bs, int warp_m, int warp_n, int lane,
                                         float (&acc)[NR][4][4]) {
#pragma unroll
  for (int kk = 0; kk < TK / 16; ++kk) {
    uint32_t b[2][4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      // lanes 0-7: n-tile 2h, k 0-7 | 8-15: n-tile 2h, k 8-15 | 16-23: n-tile 2h+1, k 0-7 | 24-31: n-tile 2h+1, k 8-15
      const int n = warp_n * 32 + (2 * h + (lane >> 4)) * 8 + (lane & 7);
      ldmatrix_x4(b[h], Bs + n * PITCH + kk * 16 + ((lane >> 3) & 1) * 8);
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      uint32_t a[4];
      // lanes 0-15: rows 0-15, k 0-7 ; lanes 16-31: rows 0-15, k 8-15
      ldmatrix_x4(a, As + (size_t)r * TM * PITCH + (warp_m * 16 + (lane & 15)) * PITCH + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) mma_f16(acc[r][nt], a, b[nt >> 1][(nt & 1) * 2], b[nt >> 1][(nt & 1) * 2 + 1]);
    }
  }
}

// Token tile -> shared memory (rows past the segment are zero).
__device__ __forceinline__ void stage_tokens(const __half* __restrict__ src, int ld, int k0, int rows_valid, __half* Bs,
                                             int tid) {
  // 64 rows x 64 halfs = 64 x 8 sixteen-byte pieces
  for (int i = tid; i < TN * 8; i += GG_THREADS) {
    const int n = i >> 3, c = i & 7;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (n < rows_valid) v = *reinterpret_cast<const uint4*>(src + (size_t)n * ld + k0 + c * 8);
    *reinterpret_cast<uint4*>(Bs + n * PITCH + c * 8) = v;
  }
}

// ---- gate/up + SwiGLU --------------------------------------------------------------------------------

__global__ void __launch_bounds__(GG_THREADS) k_grouped_gateup(GroupedParams p) {
  __shared__ __align__(16) __half As[2 * TM * PITCH];
  __shared__ __align__(16) __half Bs[TN * PITCH];
  const int tile = blockIdx.y;
  if (tile >= *p.n_tiles) return;
  const int e = p.tile_expert[tile], row0 = p.tile_row0[tile], rows_valid = p.tile_rows[tile];
  const int f0 = blockIdx.x * TM;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warp_m = warp & 3, warp_n = warp >> 2;
  const int rb = p.ne / 256 * (int)Q4K_BLOCK_BYTES;
  const bool shared_seg = e >= p.n_expert;
  const uint8_t* gbase = (shared_seg ? p.sh_gate : p.gate + (size_t)e * p.gate_stride) + (size_t)f0 * rb;
  const uint8_t* ubase = (shared_seg ? p.sh_up : p.up + (size_t)e * p.up_stride) + (size_t)f0 * rb;

  float acc[2][4][4];
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[r][nt][i] = 0.f;

  // unpack role: thread = (weight row, quarter of the 64-element group)
  const int urow = tid >> 2, uq = tid & 3;
  const __half* xg_tile = p.xg + (size_t)row0 * p.ne;

  for (int k0 = 0; k0 < p.ne; k0 += TK) {
    const int blk = k0 >> 8, j = (k0 >> 6) & 3;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const uint8_t* bp = (r == 0 ? gbase : ubase) + (size_t)urow * rb + (size_t)blk * Q4K_BLOCK_BYTES;
      const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(bp));
      const uint2 q = __ldg(reinterpret_cast<const uint2*>(bp + 16 + 32 * j + 8 * uq));
      uint32_t scp, mp;
      q4k_scale_min_pair(hdr.y, hdr.z, hdr.w, j, scp, mp);
      const float d = f16_bits_to_f32(hdr.x) * W_PRESCALE, dmin = f16_bits_to_f32(hdr.x >> 16) * W_PRESCALE;
      const __half2 s_lo = __float2half2_rn(d * (float)(scp & 0xFFu)), s_hi = __float2half2_rn(d * (float)(scp >> 8));
      const __half2 m_lo = __float2half2_rn(-dmin * (float)(mp & 0xFFu)), m_hi = __float2half2_rn(-dmin * (float)(mp >> 8));
      uint4 lo, hi;
      q4_word_to_h2(q.x, s_lo, m_lo, lo.x, lo.y);
      q4_word_to_h2(q.y, s_lo, m_lo, lo.z, lo.w);
      q4_word_to_h2(q.x >> 4, s_hi, m_hi, hi.x, hi.y);
      q4_word_to_h2(q.y >> 4, s_hi, m_hi, hi.z, hi.w);
      __half* arow = As + (size_t)r * TM * PITCH + urow * PITCH;
      *reinterpret_cast<uint4*>(arow + 8 * uq) = lo;        // sub-block 2j: K positions 8q .. 8q+7
      *reinterpret_cast<uint4*>(arow + 32 + 8 * uq) = hi;   // sub-block 2j+1
    }
    stage_tokens(xg_tile, p.ne, k0, rows_valid, Bs, tid);
    __syncthreads();
    mma_step<2>(As, Bs, warp_m, warp_n, lane, acc);
    __syncthreads();
  }

  // epilogue: act = silu(g) * u, transposed through shared memory to token-major f16 rows
  __half* T = As;  // [TN][PITCH]
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int f = warp_m * 16 + g + (i >> 1) * 8;
      const int n = warp_n * 32 + nt * 8 + 2 * t + (i & 1);
      const float gv = acc[0][nt][i] * W_POSTSCALE, uv = acc[1][nt][i] * W_POSTSCALE;
      const float a = gated_act(p.act_kind, e < p.n_expert ? p.clamp : 0.f, gv, uv);
      T[n * PITCH + kperm(f)] = __float2half_rn(fminf(fmaxf(a, -65504.f), 65504.f));
    }
  __syncthreads();
  for (int i = tid; i < TN * 8; i += GG_THREADS) {
    const int n = i >> 3, c = i & 7;
    if (n < rows_valid)
      *reinterpret_cast<uint4*>(p.act + (size_t)(row0 + n) * p.nff + f0 + c * 8) = *reinterpret_cast<const uint4*>(T + n * PITCH + c * 8);
  }
}

// ---- down -------------------------------------------------------------------------------------------

// Four bytes at a 2-byte-aligned offset.  The upper word is only fetched when the offset is off a
// word boundary: the last such read of a Q6_K block (scales at byte 204) then ends inside the block,
// so nothing past a bank's last block is touched.
__device__ __forceinline__ uint32_t ldg_u32_unaligned(const uint8_t* base, size_t off) {
  const size_t a = off & ~(size_t)3;
  const uint32_t lo = __ldg(reinterpret_cast<const uint32_t*>(base + a));
  const uint32_t hi = (off & 3) ? __ldg(reinterpret_cast<const uint32_t*>(base + a + 4)) : 0u;
  return __funnelshift_r(lo, hi, (uint32_t)(off & 3) * 8);
}

// Four 6-bit codes held as bytes of c -> (code - 32) * s in the order (b0,b2),(b1,b3).
__device__ __forceinline__ void q6_word_to_h2(uint32_t c, __half2 s, uint32_t& out02, uint32_t& out13) {
  const __half2 k1056 = __float2half2_rn(1056.f);
  const __half2 a = __hsub2(u32_as_h2((c & 0x00FF00FFu) | 0x64006400u), k1056);
  const __half2 b = __hsub2(u32_as_h2(((c >> 8) & 0x00FF00FFu) | 0x64006400u), k1056);
  out02 = h2_as_u32(__hmul2(a, s));
  out13 = h2_as_u32(__hmul2(b, s));
}

__global__ void __launch_bounds__(GG_THREADS) k_grouped_down(GroupedParams p) {
  __shared__ __align__(16) __half As[2 * TM * PITCH];  // two K steps of 64 (one half of a Q6_K block)
  __shared__ __align__(16) __half Bs[2 * TN * PITCH];
  const int tile = blockIdx.y;
  if (tile >= *p.n_tiles) return;
  const int e = p.tile_expert[tile], row0 = p.tile_row0[tile], rows_valid = p.tile_rows[tile];
  const int i0 = blockIdx.x * TM;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warp_m = warp & 3, warp_n = warp >> 2;
  const int drb = p.nff / 256 * (int)Q6K_BLOCK_BYTES;
  const bool shared_seg = e >= p.n_expert;
  const uint8_t* wbase = shared_seg ? p.sh_down : p.down + (size_t)e * p.down_stride;  // 16-byte aligned
  const size_t wrow0 = (size_t)i0 * drb;

  float acc[1][4][4];
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[0][nt][i] = 0.f;

  // unpack role: thread = (weight row, 8 consecutive l of the 32-wide quadrant)
  const int urow = tid >> 2, part = tid & 3;
  const __half* act_tile = p.act + (size_t)row0 * p.nff;

  for (int k0 = 0; k0 < p.nff; k0 += 128) {  // one half (128 elements) of a block per iteration
    const int blk = k0 >> 8, h = (k0 >> 7) & 1;
    const size_t bo = wrow0 + (size_t)urow * drb + (size_t)blk * Q6K_BLOCK_BYTES;
    const float d = f16_bits_to_f32(__ldg(reinterpret_cast<const unsigned short*>(wbase + bo + 208))) * W_PRESCALE;
    const uint32_t S0 = ldg_u32_unaligned(wbase, bo + 192 + 8 * h), S1 = ldg_u32_unaligned(wbase, bo + 196 + 8 * h);
    const uint32_t sc4 = __byte_perm(S0, S1, (part >> 1) ? 0x7531u : 0x6420u);  // scale of quadrant q at byte q
#pragma unroll
    for (int w = 0; w < 2; ++w) {  // two words of four l each
      const int l = 8 * part + 4 * w;
      const uint32_t A = ldg_u32_unaligned(wbase, bo + 64 * h + l);
      const uint32_t B = ldg_u32_unaligned(wbase, bo + 64 * h + 32 + l);
      const uint32_t H = ldg_u32_unaligned(wbase, bo + 128 + 32 * h + l);
      const uint32_t cs[4] = {(A & 0x0F0F0F0Fu) | ((H << 4) & 0x30303030u), (B & 0x0F0F0F0Fu) | ((H << 2) & 0x30303030u),
                              ((A >> 4) & 0x0F0F0F0Fu) | (H & 0x30303030u), ((B >> 4) & 0x0F0F0F0Fu) | ((H >> 2) & 0x30303030u)};
#pragma unroll
      for (int qd = 0; qd < 4; ++qd) {
        const float sc = (float)(int)(signed char)((sc4 >> (8 * qd)) & 0xFFu);
        uint32_t o02, o13;
        q6_word_to_h2(cs[qd], __float2half2_rn(d * sc), o02, o13);
        // element 32*qd + l within the half -> K step qd/2, position 32*(qd&1) + l
        __half* dst = As + (size_t)(qd >> 1) * TM * PITCH + urow * PITCH + 32 * (qd & 1) + l;
        *reinterpret_cast<uint2*>(dst) = make_uint2(o02, o13);
      }
    }
    stage_tokens(act_tile, p.nff, k0, rows_valid, Bs, tid);
    stage_tokens(act_tile, p.nff, k0 + 64, rows_valid, Bs + TN * PITCH, tid);
    __syncthreads();
    mma_step<1>(As, Bs, warp_m, warp_n, lane, acc);
    mma_step<1>(As + TM * PITCH, Bs + TN * PITCH, warp_m, warp_n, lane, acc);
    __syncthreads();
  }

  // epilogue: y[pos, i] f32, transposed through shared memory (64 tokens x 64 features)
  float* T = reinterpret_cast<float*>(As);  // [TN][TM + 4] floats = 17408 B <= sizeof(As)
  constexpr int TP = TM + 4;
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int f = warp_m * 16 + g + (i >> 1) * 8;
      const int n = warp_n * 32 + nt * 8 + 2 * t + (i & 1);
      T[n * TP + f] = acc[0][nt][i] * W_POSTSCALE;
    }
  __syncthreads();
  for (int i = tid; i < TN * (TM / 4); i += GG_THREADS) {
    const int n = i / (TM / 4), c = i % (TM / 4);
    if (n < rows_valid)
      *reinterpret_cast<float4*>(p.y + (size_t)(row0 + n) * p.ne + i0 + c * 4) = *reinterpret_cast<const float4*>(T + n * TP + c * 4);
  }
}

// ---- any bank format (formats.cuh): the same 64 x 64 tiles, weights unpacked through the code view ----

// Sixteen codes -> sixteen f16 weights (code - off) * s + m, every four in the order 0,2,1,3.
__device__ __forceinline__ void codes16_to_h(const uint32_t (&c)[4], float A, float B, int off, uint4& o0, uint4& o1) {
  const __half2 s = __float2half2_rn(A * W_PRESCALE), m = __float2half2_rn(B * W_PRESCALE);
  const __half2 koff = __float2half2_rn(1024.f + (float)off);  // 1024 + code is exact in f16 for 8-bit codes
  uint32_t o[8];
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const __half2 a = __hsub2(u32_as_h2((c[w] & 0x00FF00FFu) | 0x64006400u), koff);
    const __half2 b = __hsub2(u32_as_h2(((c[w] >> 8) & 0x00FF00FFu) | 0x64006400u), koff);
    o[2 * w] = h2_as_u32(__hfma2(a, s, m));
    o[2 * w + 1] = h2_as_u32(__hfma2(b, s, m));
  }
  o0 = make_uint4(o[0], o[1], o[2], o[3]);
  o1 = make_uint4(o[4], o[5], o[6], o[7]);
}

// NR = 2: gate and up rows of 64 features with the gated activation as epilogue (act, f16).
// NR = 1: 64 rows of the down matrix, raw outputs y (f32).
template <int NR>
__global__ void __launch_bounds__(GG_THREADS) k_anyfmt_grouped(GroupedParams p) {
  __shared__ __align__(16) __half As[2 * TM * PITCH];
  __shared__ __align__(16) __half Bs[TN * PITCH];
  const int tile = blockIdx.y;
  if (tile >= *p.n_tiles) return;
  const int e = p.tile_expert[tile], row0 = p.tile_row0[tile], rows_valid = p.tile_rows[tile];
  const int f0 = blockIdx.x * TM;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warp_m = warp & 3, warp_n = warp >> 2;
  const bool shared_seg = e >= p.n_expert;
  const int K = NR == 2 ? p.ne : p.nff;
  const int dt0 = NR == 2 ? p.gate_dt : p.down_dt, dt1 = p.up_dt;
  const size_t rb0 = row_bytes(dt0, K), rb1 = row_bytes(dt1, K);
  const uint8_t* base0 = NR == 2 ? (shared_seg ? p.sh_gate : p.gate + (size_t)e * p.gate_stride)
                                 : (shared_seg ? p.sh_down : p.down + (size_t)e * p.down_stride);
  const uint8_t* base1 = shared_seg ? p.sh_up : p.up + (size_t)e * p.up_stride;
  const int urow = tid >> 2, uq = tid & 3;  // unpack role: (weight row, 16 of the step's 64 elements)
  const uint8_t* wrow0 = base0 + (size_t)(f0 + urow) * rb0;
  const uint8_t* wrow1 = base1 + (size_t)(f0 + urow) * rb1;
  const __half* tok = (NR == 2 ? p.xg : p.act) + (size_t)row0 * K;

  float acc[NR][4][4];
#pragma unroll
  for (int r = 0; r < NR; ++r)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[r][nt][i] = 0.f;

  for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      uint32_t c[4];
      float A, B;
      int off;
      fmt_codes16(r == 0 ? dt0 : dt1, r == 0 ? wrow0 : wrow1, (k0 >> 4) + uq, c, A, B, off);
      uint4 o0, o1;
      codes16_to_h(c, A, B, off, o0, o1);
      __half* arow = As + (size_t)r * TM * PITCH + urow * PITCH + 16 * uq;
      *reinterpret_cast<uint4*>(arow) = o0;
      *reinterpret_cast<uint4*>(arow + 8) = o1;
    }
    stage_tokens(tok, K, k0, rows_valid, Bs, tid);
    __syncthreads();
    mma_step<NR>(As, Bs, warp_m, warp_n, lane, acc);
    __syncthreads();
  }

  const int g = lane >> 2, t = lane & 3;
  if (NR == 2) {
    __half* T = As;  // [TN][PITCH] token-major f16 rows
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int f = warp_m * 16 + g + (i >> 1) * 8;
        const int n = warp_n * 32 + nt * 8 + 2 * t + (i & 1);
        const float gv = acc[0][nt][i] * W_POSTSCALE, uv = acc[NR - 1][nt][i] * W_POSTSCALE;
        const float a = gated_act(p.act_kind, e < p.n_expert ? p.clamp : 0.f, gv, uv);
        T[n * PITCH + kperm(f)] = __float2half_rn(fminf(fmaxf(a, -65504.f), 65504.f));
      }
    __syncthreads();
    for (int i = tid; i < TN * 8; i += GG_THREADS) {
      const int n = i >> 3, c = i & 7;
      if (n < rows_valid)
        *reinterpret_cast<uint4*>(p.act + (size_t)(row0 + n) * p.nff + f0 + c * 8) = *reinterpret_cast<const uint4*>(T + n * PITCH + c * 8);
    }
  } else {
    float* T = reinterpret_cast<float*>(As);  // [TN][TM + 4] floats
    constexpr int TP = TM + 4;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int f = warp_m * 16 + g + (i >> 1) * 8;
        const int n = warp_n * 32 + nt * 8 + 2 * t + (i & 1);
        T[n * TP + f] = acc[0][nt][i] * W_POSTSCALE;
      }
    __syncthreads();
    for (int i = tid; i < TN * (TM / 4); i += GG_THREADS) {
      const int n = i / (TM / 4), c = i % (TM / 4);
      if (n < rows_valid)
        *reinterpret_cast<float4*>(p.y + (size_t)(row0 + n) * p.ne + f0 + c * 4) = *reinterpret_cast<const float4*>(T + n * TP + c * 4);
    }
  }
}

// ---- un-permute + combine -----------------------------------------------------------------------------

// dst[t, :] = sum over ranks (in rank order) of w * y[pos(t, rank), :], then the shared expert
// (sh_y = the shared expert's output rows in token order, or null).
__global__ void __launch_bounds__(256) k_unpermute_combine(const float* __restrict__ y, const int* __restrict__ pos_of_pair,
                                                           const float* __restrict__ wts, const float* __restrict__ sh_logit,
                                                           const float* __restrict__ sh_y, int rows, int n_used, int ne,
                                                           float* __restrict__ dst) {
  const int c = (blockIdx.x * 256 + threadIdx.x) * 4;
  if (c >= ne) return;
  for (int t = blockIdx.y; t < rows; t += gridDim.y) {  // the grid's y extent stops at 65535
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < n_used; ++s) {
      const int pos = pos_of_pair[(size_t)t * n_used + s];
      if (pos < 0) continue;
      const float w = wts[(size_t)t * n_used + s];
      const float4 v = *reinterpret_cast<const float4*>(y + (size_t)pos * ne + c);
      o.x += w * v.x; o.y += w * v.y; o.z += w * v.z; o.w += w * v.w;
    }
    if (sh_y) {
      const float gsh = sh_logit ? 1.0f / (1.0f + __expf(-sh_logit[t])) : 1.0f;
      const float4 v = *reinterpret_cast<const float4*>(sh_y + (size_t)t * ne + c);
      o.x += gsh * v.x; o.y += gsh * v.y; o.z += gsh * v.z; o.w += gsh * v.w;
    }
    *reinterpret_cast<float4*>(dst + (size_t)t * ne + c) = o;
  }
}

// The shared segment starts right after the routed rows: its address is only known on the device.
template <bool Y16>
__global__ void __launch_bounds__(256) k_unpermute_combine_seg(const float* __restrict__ y, const float* __restrict__ y_scale,
                                                               const int* __restrict__ pos_of_pair,
                                                               const float* __restrict__ wts, const float* __restrict__ sh_logit,
                                                               const int* __restrict__ seg_off, int n_seg_routed, int has_shared,
                                                               int rows, int n_used, int ne, const float* residual,
                                                               const int32_t* __restrict__ ids, const float* __restrict__ down_scale,
                                                               int weight_before, float* dst) {
  const int c = (blockIdx.x * 256 + threadIdx.x) * 4;
  if (c >= ne) return;
  // four outputs of row `pos` of y (f32 rows; or the tcgen05 down kernel's f16 rows with one scale per 32)
  auto y4 = [&](size_t pos) {
    if (!Y16) return *reinterpret_cast<const float4*>(y + pos * ne + c);
    const uint2 h = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(y) + pos * ne + c);
    const float sc = y_scale[pos * (ne / 32) + (c >> 5)];
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&h.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&h.y));
    return make_float4(a.x * sc, a.y * sc, b.x * sc, b.y * sc);
  };
  for (int t = blockIdx.y; t < rows; t += gridDim.y) {  // the grid's y extent stops at 65535
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < n_used; ++s) {
      const int pos = pos_of_pair[(size_t)t * n_used + s];
      if (pos < 0) continue;
      const float w = weight_before ? 1.0f : wts[(size_t)t * n_used + s];
      float4 v = y4((size_t)pos);
      if (down_scale != nullptr) {  // y = raw * scale[e], then the weighted sum (Op::MoeFfn::down_scale)
        // ids may be the caller's: same clamp as the bucketing, which also reported the bad id
        const float sc = down_scale[min(max(ids[(size_t)t * n_used + s], 0), n_seg_routed - 1)];
        v.x *= sc; v.y *= sc; v.z *= sc; v.w *= sc;
      }
      o.x += w * v.x; o.y += w * v.y; o.z += w * v.z; o.w += w * v.w;
    }
    if (has_shared) {
      const float gsh = sh_logit ? 1.0f / (1.0f + __expf(-sh_logit[t])) : 1.0f;
      const float4 v = y4((size_t)(seg_off[n_seg_routed] + t));
      o.x += gsh * v.x; o.y += gsh * v.y; o.z += gsh * v.z; o.w += gsh * v.w;
    }
    if (residual != nullptr) {  // MoeFfn -> Add; may alias dst: each element is read, then written, by this thread
      const float4 h = *reinterpret_cast<const float4*>(residual + (size_t)t * ne + c);
      o.x += h.x; o.y += h.y; o.z += h.z; o.w += h.w;
    }
    *reinterpret_cast<float4*>(dst + (size_t)t * ne + c) = o;
  }
}

// Tile table straight from caller-provided segment offsets (rows already grouped by expert).
__global__ void __launch_bounds__(1024) k_tiles_from_offsets(const int* __restrict__ seg_off, int n_seg, int tn,
                                                             int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                                             int* __restrict__ tile_rows, int* __restrict__ n_tiles) {
  __shared__ int s_toff[1026], s_so[1026];
  const int tid = threadIdx.x;
  for (int e = tid; e <= n_seg; e += 1024) s_so[e] = seg_off[e];
  __syncthreads();
  if (tid == 0) {
    int toff = 0;
    for (int e = 0; e < n_seg; ++e) {
      s_toff[e] = toff;
      toff += (s_so[e + 1] - s_so[e] + tn - 1) / tn;
    }
    *n_tiles = toff;
  }
  __syncthreads();
  for (int e = tid; e < n_seg; e += 1024) {
    const int cnt = seg_off[e + 1] - seg_off[e];
    const int nt = (cnt + tn - 1) / tn;
    for (int t = 0; t < nt; ++t) {
      tile_expert[s_toff[e] + t] = e;
      tile_row0[s_toff[e] + t] = seg_off[e] + t * tn;
      tile_rows[s_toff[e] + t] = min(tn, cnt - t * tn);
    }
  }
}

}  // namespace

size_t grouped_scratch_bytes(int rows_total, int n_pairs, int n_seg, int ne, int nff) {
  const size_t rows_pad = (size_t)rows_total + 256;
  size_t b = 0;
  b += align_up((size_t)(n_seg + 2) * 4, 256) * 3;                 // counts, seg_off, fill
  b += align_up((size_t)(rows_total / TN + n_seg + 2) * 4, 256) * 3 + 256;  // tile table + n_tiles
  b += align_up((size_t)(n_pairs + 1) * 4, 256) * 2;               // pos_of_pair, pair_of_pos
  // token arrays: rows grouped by expert (legacy tiles) or padded to whole 256-row tiles (tcgen05)
  const size_t tile_rows_pad = ((size_t)rows_total / 256 + n_seg + 1) * 256;
  const size_t tok_rows = tile_rows_pad > rows_pad ? tile_rows_pad : rows_pad;
  b += align_up(tok_rows * ne * 2, 256);                           // xg
  b += align_up(tok_rows * nff * 2, 256);                          // act
  b += align_up(rows_pad * ne * 4, 256);                           // y
  return b;
}

int32_t launch_grouped_ffn(infr_cuda_ctx* ctx, const GroupedCall& c) {
  // carve scratch
  char* base = static_cast<char*>(c.scratch);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    char* p = base + off;
    off += align_up(bytes, 256);
    return p;
  };
  const int n_seg_routed = c.n_expert;
  const int n_seg = c.n_expert + (c.shared_rows > 0 ? 1 : 0);
  const int rows_total = c.rows_bound;  // upper bound on sorted rows + shared rows
  const bool tuned = BankTypes{c.gate_dt, c.up_dt, c.down_dt}.tuned();
  const bool use_umma = tuned && !c.legacy && umma_grouped_supported(c.ne, c.nff);
  if (tuned && c.down_q4k && !use_umma)
    return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "grouped GEMM: Q4_K down banks need the tcgen05 tiles (ne, n_ff_exp multiples of 256, not path 3)");
  const int tn = use_umma ? umma_tile_rows() : TN;
  const int max_tiles = rows_total / tn + n_seg + 1;
  const int max_tiles_alloc = rows_total / TN + n_seg + 1;
  int* counts = reinterpret_cast<int*>(take((size_t)(n_seg + 2) * 4));
  int* seg_off = reinterpret_cast<int*>(take((size_t)(n_seg + 2) * 4));
  int* fill = reinterpret_cast<int*>(take((size_t)(n_seg + 2) * 4));
  int* tile_expert = reinterpret_cast<int*>(take((size_t)(max_tiles_alloc + 1) * 4));
  int* tile_row0 = reinterpret_cast<int*>(take((size_t)(max_tiles_alloc + 1) * 4));
  int* tile_rows = reinterpret_cast<int*>(take((size_t)(max_tiles_alloc + 1) * 4));
  int* n_tiles = reinterpret_cast<int*>(take(256));
  int* pos_of_pair = reinterpret_cast<int*>(take((size_t)(c.n_pairs + 1) * 4));
  int* pair_of_pos = reinterpret_cast<int*>(take((size_t)(c.n_pairs + 1) * 4));
  const size_t tile_rows_pad = ((size_t)rows_total / 256 + n_seg + 1) * 256;
  const size_t tok_rows = std::max(tile_rows_pad, (size_t)rows_total + 256);
  __half* xg = reinterpret_cast<__half*>(take(tok_rows * c.ne * 2));
  __half* act = reinterpret_cast<__half*>(take(tok_rows * c.nff * 2));
  float* y = c.y_out ? c.y_out : reinterpret_cast<float*>(take(((size_t)rows_total + 256) * c.ne * 4));
  cudaStream_t st = ctx->stream;

  const float* row_w = c.weight_before ? c.wts : nullptr;
  if (c.ids) {
    // routed call: bucket the pairs
    if (c.n_pairs <= (1 << 16)) {
      k_bucket_fused<<<1, 1024, 0, st>>>(c.ids, c.n_pairs, c.n_expert, c.ep_lo, c.ep_n, c.shared_rows, tn, seg_off, tile_expert, tile_row0,
                                         tile_rows, n_tiles, pos_of_pair, pair_of_pos, ctx->status);
      ctx->launches += 1;
    } else {
      cudaError_t e = cudaMemsetAsync(counts, 0, (size_t)(n_seg + 2) * 4, st);
      if (e != cudaSuccess) return check_cuda(ctx, e, "grouped: memset");
      k_pair_count<<<(c.n_pairs + 255) / 256, 256, 0, st>>>(c.ids, c.n_pairs, c.n_expert, c.ep_lo, c.ep_n, counts, ctx->status);
      k_segment_scan<<<1, 1024, 0, st>>>(counts, c.n_expert, c.shared_rows, tn, seg_off, fill, tile_expert, tile_row0, tile_rows, n_tiles);
      k_pair_scatter<<<(c.n_pairs + 255) / 256, 256, 0, st>>>(c.ids, c.n_pairs, c.n_expert, c.ep_lo, c.ep_n, seg_off, fill,
                                                               pos_of_pair, pair_of_pos);
      ctx->launches += 3;
    }
    if (use_umma)
      k_gather_tiles<<<dim3(tn / 8, max_tiles), 256, 0, st>>>(c.x, pair_of_pos, row_w, seg_off, n_seg_routed, c.n_used, tile_row0, tile_rows,
                                                             n_tiles, tn, c.ne, reinterpret_cast<unsigned char*>(xg));
    else
      k_gather_rows<<<(rows_total + 7) / 8, 256, 0, st>>>(c.x, pair_of_pos, row_w, seg_off, n_seg_routed, c.n_used, rows_total, c.ne, xg);
    ctx->launches += 1;
  } else {
    // rows already grouped: offsets come from the caller (n_expert segments, no shared segment)
    k_tiles_from_offsets<<<1, 1024, 0, st>>>(c.seg_off_in, c.n_expert, tn, tile_expert, tile_row0, tile_rows, n_tiles);
    // gather with identity order: seg_off_in[n_expert] rows; reuse the same kernel with a
    // two-entry offset view (sorted rows = all rows, shared rows = none)
    cudaError_t e = cudaMemcpyAsync(seg_off, c.seg_off_in + c.n_expert, 4, cudaMemcpyDeviceToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(seg_off + 1, c.seg_off_in + c.n_expert, 4, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return check_cuda(ctx, e, "grouped: offsets copy");
    if (use_umma)
      k_gather_tiles<<<dim3(tn / 8, max_tiles), 256, 0, st>>>(c.x, nullptr, nullptr, seg_off, 0, 1, tile_row0, tile_rows, n_tiles, tn, c.ne,
                                                             reinterpret_cast<unsigned char*>(xg));
    else
      k_gather_rows<<<(rows_total + 7) / 8, 256, 0, st>>>(c.x, nullptr, nullptr, seg_off, 0, 1, rows_total, c.ne, xg);
    ctx->launches += 2;
  }

  GroupedParams p = {};
  p.tile_expert = tile_expert;
  p.tile_row0 = tile_row0;
  p.tile_rows = tile_rows;
  p.n_tiles = n_tiles;
  p.xg = xg;
  p.act = act;
  p.y = y;
  p.gate = c.gate;
  p.up = c.up;
  p.down = c.down;
  p.gate_stride = c.gate_stride;
  p.up_stride = c.up_stride;
  p.down_stride = c.down_stride;
  p.sh_gate = c.sh_gate;
  p.sh_up = c.sh_up;
  p.sh_down = c.sh_down;
  p.ne = c.ne;
  p.nff = c.nff;
  p.n_expert = c.n_expert;
  p.down_q4k = c.down_q4k;
  // tcgen05 tiles with the combine behind them: the raw rows cross memory as f16 (half the bytes out of the
  // down kernel and into the combine); rows handed to the caller stay f32
  p.y_f16 = (use_umma && c.dst != nullptr && c.y_out == nullptr && c.ne % 32 == 0 && !ctx->cfg.raw_rows_f32) ? 1 : 0;
  p.y_scale = reinterpret_cast<float*>(reinterpret_cast<char*>(y) + ((size_t)rows_total + 256) * c.ne * 2);  // behind the f16 rows
  p.gate_dt = c.gate_dt;
  p.up_dt = c.up_dt;
  p.down_dt = c.down_dt;
  p.act_kind = c.act_kind;
  p.gu_rows = (int)(c.gate_stride / ((size_t)c.ne / 256 * Q4K_BLOCK_BYTES));
  p.clamp = c.clamp;
  p.status = ctx->status;
  p.trace = ctx->trace;
  p.trace_tile = (int)ctx->cfg.trace_tile;
  if (use_umma) {
    const int32_t rc = launch_umma_grouped(ctx, p, max_tiles);
    if (rc) return rc;
  } else if (!tuned) {
    // banks in another format mix: the same tiles, weights unpacked through the generic code view
    if (c.ne % 256 || c.nff % 256) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "grouped GEMM: ne and n_ff_exp must be multiples of 256 for these bank formats");
    k_anyfmt_grouped<2><<<dim3(c.nff / TM, max_tiles), GG_THREADS, 0, st>>>(p);
    k_anyfmt_grouped<1><<<dim3(c.ne / TM, max_tiles), GG_THREADS, 0, st>>>(p);
    ctx->launches += 2;
  } else {
    k_grouped_gateup<<<dim3(c.nff / TM, max_tiles), GG_THREADS, 0, st>>>(p);
    k_grouped_down<<<dim3(c.ne / TM, max_tiles), GG_THREADS, 0, st>>>(p);
    ctx->launches += 2;
  }
  if (c.dst) {
    auto comb = p.y_f16 ? k_unpermute_combine_seg<true> : k_unpermute_combine_seg<false>;
    comb<<<dim3((c.ne / 4 + 255) / 256, std::min(c.rows, 65535)), 256, 0, st>>>(y, p.y_scale, pos_of_pair, c.wts, c.sh_logit, seg_off, n_seg_routed,
                                                                                 c.shared_rows > 0 ? 1 : 0, c.rows, c.n_used, c.ne, c.residual, c.ids, c.down_scale,
                                                                                 c.weight_before, c.dst);
    ctx->launches += 1;
  }
  return check_cuda(ctx, cudaGetLastError(), "grouped ffn launch");
}

int32_t launch_combine(infr_cuda_ctx* ctx, const float* y, const int* pos_of_pair, const float* wts, const float* sh_logit,
                       const float* sh_y, int rows, int n_used, int ne, float* dst) {
  k_unpermute_combine<<<dim3((ne / 4 + 255) / 256, std::min(rows, 65535)), 256, 0, ctx->stream>>>(y, pos_of_pair, wts, sh_logit, sh_y, rows, n_used, ne, dst);
  ctx->launches += 1;
  return check_cuda(ctx, cudaGetLastError(), "combine launch");
}

cudaError_t publish_codebooks_grouped(const unsigned char* const* tables) { return publish_codebooks(tables); }

}  // namespace infr
