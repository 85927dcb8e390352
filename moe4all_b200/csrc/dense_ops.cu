// The ops around Op::MoeFfn that the graph builder emits for a MoE layer
// (crates/infr-llama/src/seam/runner.rs:7999-8176): Linear on F32 / Q4_K / Q5_K / Q6_K / Q8_0 weights, GatedAct,
// MoeSharedExpertAdd, RmsNorm, Add.  CPU arms: crates/infr-cpu/src/lib.rs:1275-1328, 2973-3027,
// 3336-3356, 1046-1069, 3055-3070.  These are the un-fused forms; the hot path folds the shared
// expert into the MoE kernels instead (see decode_ffn.cu).
#include "formats.cuh"
#include "kernels.cuh"

namespace infr {

namespace {

__device__ __forceinline__ uint32_t ld_u32_unaligned(const unsigned char* base, size_t off) {
  const size_t a = off & ~(size_t)3;
  const uint32_t lo = *reinterpret_cast<const uint32_t*>(base + a);
  const uint32_t hi = *reinterpret_cast<const uint32_t*>(base + a + 4);
  return __funnelshift_r(lo, hi, (uint32_t)(off & 3) * 8);
}

// One warp per (input row, output feature): grid.y walks the m input rows.
template <int DT>
__global__ void __launch_bounds__(256) k_linear(const unsigned char* __restrict__ w, const float* __restrict__ x,
                                                float* __restrict__ y, int m, int in_f, int out_f, size_t w_bytes) {
  const int o = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (o >= out_f) return;
  {
    const int r = blockIdx.y;
    const float* xr = x + (size_t)r * in_f;
    float acc = 0.f;
    if (DT == INFR_CUDA_DT_F32) {
      const float* wr = reinterpret_cast<const float*>(w) + (size_t)o * in_f;
      for (int i = lane; i < in_f; i += 32) acc = fmaf(__ldg(wr + i), __ldg(xr + i), acc);
    } else if (DT == INFR_CUDA_DT_Q4K) {
      const unsigned char* wr = w + (size_t)o * (in_f / 256) * Q4K_BLOCK_BYTES;
      for (int g = lane; g < in_f / 64; g += 32) {
        float xv[64];
        float xs0 = 0.f, xs1 = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float4 v = __ldg(reinterpret_cast<const float4*>(xr + (size_t)g * 64) + i);
          xv[4 * i + 0] = v.x; xv[4 * i + 1] = v.y; xv[4 * i + 2] = v.z; xv[4 * i + 3] = v.w;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) { xs0 += xv[i]; xs1 += xv[32 + i]; }
        const int blk = g >> 2, j = g & 3;
        const unsigned char* bp = wr + (size_t)blk * Q4K_BLOCK_BYTES;
        const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(bp));
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(bp + 16 + 32 * j));
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(bp + 32 + 32 * j));
        const uint32_t q[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        acc += q4k_dot64(hdr, q, xv, xs0, xs1, j);
      }
    } else {  // Q6_K: unit = 16 elements, see decode_ffn.cu for the layout
      const size_t row_off = (size_t)o * (in_f / 256) * Q6K_BLOCK_BYTES;
      for (int u = lane; u < in_f / 16; u += 32) {
        const int b = u >> 4, h = (u >> 3) & 1, lw = u & 7;
        const size_t ro = row_off + (size_t)b * Q6K_BLOCK_BYTES;
        // the last block of the tensor: stay inside the allocation when reading the word pair
        const bool tail = ro + Q6K_BLOCK_BYTES + 8 > w_bytes;
        uint32_t A, B, H, S0, S1;
        if (!tail) {
          A = ld_u32_unaligned(w, ro + 64 * h + 4 * lw);
          B = ld_u32_unaligned(w, ro + 64 * h + 32 + 4 * lw);
          H = ld_u32_unaligned(w, ro + 128 + 32 * h + 4 * lw);
          S0 = ld_u32_unaligned(w, ro + 192 + 8 * h);
          S1 = ld_u32_unaligned(w, ro + 196 + 8 * h);
        } else {
          auto ld4 = [&](size_t off) {
            const unsigned short lo = *reinterpret_cast<const unsigned short*>(w + off);
            const unsigned short hi = *reinterpret_cast<const unsigned short*>(w + off + 2);
            return (uint32_t)lo | ((uint32_t)hi << 16);
          };
          A = ld4(ro + 64 * h + 4 * lw);
          B = ld4(ro + 64 * h + 32 + 4 * lw);
          H = ld4(ro + 128 + 32 * h + 4 * lw);
          S0 = ld4(ro + 192 + 8 * h);
          S1 = ld4(ro + 196 + 8 * h);
        }
        const float d = f16_bits_to_f32(*reinterpret_cast<const unsigned short*>(w + ro + 208));
        const uint32_t cs[4] = {((A << 1) & 0x1E1E1E1Eu) | ((H << 5) & 0x60606060u) | 0x80808080u,
                                ((B << 1) & 0x1E1E1E1Eu) | ((H << 3) & 0x60606060u) | 0x80808080u,
                                ((A >> 3) & 0x1E1E1E1Eu) | ((H << 1) & 0x60606060u) | 0x80808080u,
                                ((B >> 3) & 0x1E1E1E1Eu) | ((H >> 1) & 0x60606060u) | 0x80808080u};
        const uint32_t sc4 = __byte_perm(S0, S1, (lw >> 2) ? 0x7531u : 0x6420u);
        const float* ab = xr + b * 256 + h * 128 + lw * 4;
        float part = 0.f;
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
          const float4 v = __ldg(reinterpret_cast<const float4*>(ab + 32 * qd));
          const uint32_t c = cs[qd];
          float F = byte_to_unit_float<0>(c) * v.x;
          F = fmaf(byte_to_unit_float<1>(c), v.y, F);
          F = fmaf(byte_to_unit_float<2>(c), v.z, F);
          F = fmaf(byte_to_unit_float<3>(c), v.w, F);
          const float S = (v.x + v.y) + (v.z + v.w);
          const float sc = (float)(int)(signed char)((sc4 >> (8 * qd)) & 0xFFu);
          part = fmaf(sc, fmaf(64.f, F, -96.f * S), part);
        }
        acc = fmaf(d, part, acc);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) y[(size_t)r * out_f + o] = acc;
  }
}

// The same op on any block format through the code view of formats.cuh: one warp per (input row, output
// feature), a lane per 16 weights: w . x = A * (sum code x - off * sum x) + B * sum x.
__global__ void __launch_bounds__(256) k_linear_anyfmt(int dt, const unsigned char* __restrict__ w, const float* __restrict__ x,
                                                       float* __restrict__ y, int in_f, int out_f, size_t rb) {
  const int o = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (o >= out_f) return;
  const float* xr = x + (size_t)blockIdx.y * in_f;
  const unsigned char* wr = w + (size_t)o * rb;
  float acc = 0.f;
  for (int h = lane; h < in_f / 16; h += 32) {
    uint32_t c[4];
    float A, B;
    int off;
    fmt_codes16(dt, wr, h, c, A, B, off);
    float f = 0.f, S = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(xr + 16 * h) + i);
      f = fmaf((float)(c[i] & 0xFFu), v.x, f);
      f = fmaf((float)((c[i] >> 8) & 0xFFu), v.y, f);
      f = fmaf((float)((c[i] >> 16) & 0xFFu), v.z, f);
      f = fmaf((float)(c[i] >> 24), v.w, f);
      S += (v.x + v.y) + (v.z + v.w);
    }
    acc += fmaf(A, f - (float)off * S, B * S);
  }
  acc = warp_sum(acc);
  if (lane == 0) y[(size_t)blockIdx.y * out_f + o] = acc;
}

__global__ void k_gated_act(const float* __restrict__ g, const float* __restrict__ u, float* __restrict__ dst, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float gv = g[i];
    dst[i] = (gv / (1.0f + expf(-gv))) * u[i];
  }
}

__global__ void k_shared_add(const float* __restrict__ moe, const float* __restrict__ sh, const float* __restrict__ gate,
                             float* __restrict__ dst, int rows, int n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < (size_t)rows * n) {
    const float gl = gate[i / n];
    const float g = 1.0f / (1.0f + expf(-gl));
    dst[i] = moe[i] + g * sh[i];
  }
}

// One CTA per row; Σx² is accumulated in double so that the row scale agrees with the sequential
// f32 sum of the CPU to within an ulp or two whatever the order.
__global__ void __launch_bounds__(256) k_rmsnorm(const float* __restrict__ x, const float* __restrict__ w,
                                                 float* __restrict__ dst, int dim, float eps) {
  __shared__ double s_part[8];
  __shared__ float s_scale;
  const float* xr = x + (size_t)blockIdx.x * dim;
  double acc = 0.0;
  for (int i = threadIdx.x; i < dim; i += 256) {
    const float v = xr[i];
    acc += (double)(v * v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < 8; ++i) t += s_part[i];
    const float ss = (float)t / (float)dim;
    s_scale = 1.0f / sqrtf(ss + eps);
  }
  __syncthreads();
  const float s = s_scale;
  float* dr = dst + (size_t)blockIdx.x * dim;
  for (int i = threadIdx.x; i < dim; i += 256) dr[i] = xr[i] * s * w[i];
}

// Rows of x in 16-bit fixed point for the small-m expert kernels: X = round(x * 32639 / max|x|)
// per row, stored as two signed 8-bit limbs (X = 256*hi + lo).  One CTA per row.
__global__ void __launch_bounds__(256) k_quantize_rows(const float* __restrict__ x, int8_t* __restrict__ lo_out,
                                                       int8_t* __restrict__ hi_out, float* __restrict__ scale, int dim) {
  __shared__ float s_max[8];
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)blockIdx.x * dim);
  const int n4 = dim / 4;
  float m = 0.f;
  for (int i = threadIdx.x; i < n4; i += 256) {
    const float4 v = xr[i];
    m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(m, fmaxf(fabsf(v.z), fabsf(v.w))));
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = m;
  __syncthreads();
  m = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) m = fmaxf(m, s_max[i]);
  const float q_inv = m > 0.f ? 32639.f / m : 0.f;
  if (threadIdx.x == 0) scale[blockIdx.x] = m / 32639.f;
  uint32_t* lo_row = reinterpret_cast<uint32_t*>(lo_out + (size_t)blockIdx.x * dim);
  uint32_t* hi_row = reinterpret_cast<uint32_t*>(hi_out + (size_t)blockIdx.x * dim);
  for (int i = threadIdx.x; i < n4; i += 256) {
    const float4 v = xr[i];
    const int X[4] = {__float2int_rn(v.x * q_inv), __float2int_rn(v.y * q_inv), __float2int_rn(v.z * q_inv),
                      __float2int_rn(v.w * q_inv)};
    uint32_t lo, hi;
    pack_limbs4(X, lo, hi);
    lo_row[i] = lo;
    hi_row[i] = hi;
  }
}

__global__ void k_add(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ dst, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = a[i] + b[i];
}

}  // namespace

int32_t launch_linear(infr_cuda_ctx* ctx, int32_t dtype, const uint8_t* w, const float* x, float* y, int m, int in_f,
                      int out_f) {
  if (m > 65535) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "linear: more than 65535 input rows per call");
  const dim3 grid((out_f + 7) / 8, m), block(256);
  const size_t wb = row_bytes(dtype, in_f) * (size_t)out_f;
  switch (dtype) {
    case INFR_CUDA_DT_F32: k_linear<INFR_CUDA_DT_F32><<<grid, block, 0, ctx->stream>>>(w, x, y, m, in_f, out_f, wb); break;
    case INFR_CUDA_DT_Q4K: k_linear<INFR_CUDA_DT_Q4K><<<grid, block, 0, ctx->stream>>>(w, x, y, m, in_f, out_f, wb); break;
    case INFR_CUDA_DT_Q6K: k_linear<INFR_CUDA_DT_Q6K><<<grid, block, 0, ctx->stream>>>(w, x, y, m, in_f, out_f, wb); break;
    case INFR_CUDA_DT_Q5K:
    case INFR_CUDA_DT_Q8_0:
    case INFR_CUDA_DT_Q4_0:
    case INFR_CUDA_DT_Q4_1:
    case INFR_CUDA_DT_Q5_0:
    case INFR_CUDA_DT_Q5_1:
    case INFR_CUDA_DT_Q2K:
    case INFR_CUDA_DT_Q3K:
    case INFR_CUDA_DT_IQ4NL:
    case INFR_CUDA_DT_IQ4XS:
    case INFR_CUDA_DT_MXFP4:
    case INFR_CUDA_DT_NVFP4:
    case INFR_CUDA_DT_Q2_0:
    case INFR_CUDA_DT_IQ2XS:
    case INFR_CUDA_DT_IQ2S:
    case INFR_CUDA_DT_IQ3XXS:
    case INFR_CUDA_DT_IQ3S:
      k_linear_anyfmt<<<grid, block, 0, ctx->stream>>>(dtype, w, x, y, in_f, out_f, row_bytes(dtype, in_f));
      break;
    default: return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "linear: weight dtype not covered (F32 and the block formats an expert bank may have)");
  }
  ctx->launches += 1;
  return check_cuda(ctx, cudaGetLastError(), "k_linear launch");
}

int32_t launch_gated_act(infr_cuda_ctx* ctx, const float* gate, const float* up, float* dst, size_t n) {
  k_gated_act<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(gate, up, dst, n);
  ctx->launches += 1;
  return check_cuda(ctx, cudaGetLastError(), "k_gated_act launch");
}

int32_t launch_shared_add(infr_cuda_ctx* ctx, const float* moe, const float* shexp, const float* gate, float* dst,
                          int rows, int n) {
  const size_t tot = (size_t)rows * n;
  k_shared_add<<<(unsigned)((tot + 255) / 256), 256, 0, ctx->stream>>>(moe, shexp, gate, dst, rows, n);
  ctx->launches += 1;
  return check_cuda(ctx, cudaGetLastError(), "k_shared_add launch");
}

int32_t launch_rmsnorm(infr_cuda_ctx* ctx, const float* x, const float* w, float* dst, int rows, int dim, float eps) {
  k_rmsnorm<<<rows, 256, 0, ctx->stream>>>(x, w, dst, dim, eps);
  ctx->launches += 1;
  return check_cuda(ctx, cudaGetLastError(), "k_rmsnorm launch");
}

int32_t launch_quantize_rows(infr_cuda_ctx* ctx, const float* x, int8_t* lo, int8_t* hi, float* scale, int rows, int dim) {
  k_quantize_rows<<<rows, 256, 0, ctx->stream>>>(x, lo, hi, scale, dim);
  ctx->launches += 1;
  return check_cuda(ctx, cudaGetLastError(), "k_quantize_rows launch");
}

// Small host-to-device copies done by the SMs: pinned host memory is mapped into the device's
// address space, so a few threads can fetch it directly.  Unlike a copy-engine transfer this is an
// ordinary kernel in the stream: the kernel after it can be released early (programmatic dependent
// launch) and run its own prologue, e.g. the router staging its weights, while the rows cross PCIe.
namespace {
__global__ void __launch_bounds__(256) k_fetch_host(const uint4* __restrict__ src, uint4* __restrict__ dst, int n16) {
  pdl_trigger();
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i < n16) dst[i] = __ldcv(src + i);  // never a cached copy of host memory
}

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// The same fetch behind a gate: thread 0 of every CTA polls the bell word (pinned host memory, so every
// poll is a read across PCIe) until the host has rung `ticket`.  Bounded: after `limit_ns` the status word
// is set and the copy goes ahead with whatever is there; a status already set (by this or any other
// bounded wait) ends the wait at once, so the gates of a recorded plan never add up.
__global__ void __launch_bounds__(256) k_fetch_host_gated(const uint4* __restrict__ src, uint4* __restrict__ dst, int n16,
                                                          const unsigned long long* bell, unsigned long long ticket,
                                                          unsigned long long limit_ns, DeviceStatus* status) {
  pdl_trigger();
  if (threadIdx.x == 0) {
    // the status word is host memory too: it is looked at (with the clock) once per 16 polls of the bell, so
    // that a poll costs one trip across PCIe, not two
    const unsigned long long t0 = global_ns();
    for (unsigned it = 0; *reinterpret_cast<const volatile unsigned long long*>(bell) < ticket; ++it) {
      if ((it & 15u) != 15u) continue;
      if (*reinterpret_cast<volatile int*>(&status->timeout) != 0) break;
      if (global_ns() - t0 > limit_ns) {
        atomicExch(&status->timeout, 9);
        break;
      }
    }
  }
  __syncthreads();
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i < n16) dst[i] = __ldcv(src + i);
}

// Publishes `ticket` in the done word (pinned host memory) once every kernel queued before this one has
// finished: a programmatic dependent of the kernel ahead, so its thread is in place when that one ends.
__global__ void k_host_signal(unsigned long long* done, unsigned long long ticket) {
  pdl_wait();
  __threadfence_system();
  *reinterpret_cast<volatile unsigned long long*>(done) = ticket;
  __threadfence_system();
}
}  // namespace

int32_t launch_fetch_host_gated(infr_cuda_ctx* ctx, const void* src_dev_view, void* dst, size_t bytes, const unsigned long long* bell,
                                unsigned long long ticket, unsigned long long limit_ns) {
  const int n16 = (int)(bytes / 16);
  if (n16 > 512) {
    // many CTAs: one thread of a kernel of its own polls (every poll crosses PCIe, where the host is writing
    // the rows), the plain fetch follows it in the stream
    k_fetch_host_gated<<<1, 32, 0, ctx->stream>>>(nullptr, nullptr, 0, bell, ticket, limit_ns, ctx->status);
    k_fetch_host<<<(n16 + 255) / 256, 256, 0, ctx->stream>>>(static_cast<const uint4*>(src_dev_view), static_cast<uint4*>(dst), n16);
    ctx->launches += 2;
    return check_cuda(ctx, cudaGetLastError(), "gate + k_fetch_host launch");
  }
  k_fetch_host_gated<<<(n16 + 255) / 256, 256, 0, ctx->stream>>>(static_cast<const uint4*>(src_dev_view), static_cast<uint4*>(dst), n16, bell,
                                                                  ticket, limit_ns, ctx->status);
  ctx->launches += 1;
  return check_cuda(ctx, cudaGetLastError(), "k_fetch_host_gated launch");
}

int32_t launch_host_signal(infr_cuda_ctx* ctx, unsigned long long* done, unsigned long long ticket) {
  const cudaError_t e = launch_ex(k_host_signal, dim3(1), dim3(1), 0, ctx->stream, true, done, ticket);
  ctx->launches += 1;
  return check_cuda(ctx, e, "k_host_signal launch");
}

int32_t launch_store_host(infr_cuda_ctx* ctx, const void* src, void* dst_dev_view, size_t bytes) {
  // the same kernel the other way round: device rows written into mapped pinned host memory
  const int n16 = (int)(bytes / 16);
  k_fetch_host<<<(n16 + 255) / 256, 256, 0, ctx->stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst_dev_view), n16);
  ctx->launches += 1;
  return check_cuda(ctx, cudaGetLastError(), "k_fetch_host (store) launch");
}

int32_t launch_fetch_host(infr_cuda_ctx* ctx, const void* src_dev_view, void* dst, size_t bytes) {
  const int n16 = (int)(bytes / 16);
  k_fetch_host<<<(n16 + 255) / 256, 256, 0, ctx->stream>>>(static_cast<const uint4*>(src_dev_view), static_cast<uint4*>(dst), n16);
  ctx->launches += 1;
  return check_cuda(ctx, cudaGetLastError(), "k_fetch_host launch");
}

cudaError_t publish_codebooks_dense(const unsigned char* const* tables) { return publish_codebooks(tables); }

int32_t launch_add(infr_cuda_ctx* ctx, const float* a, const float* b, float* dst, size_t n) {
  k_add<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(a, b, dst, n);
  ctx->launches += 1;
  return check_cuda(ctx, cudaGetLastError(), "k_add launch");
}

}  // namespace infr
