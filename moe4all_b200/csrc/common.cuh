// Shared device/host helpers of the sm_100a MoE FFN library.
#pragma once

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/infr_cuda.h"

namespace infr {

// ---------------------------------------------------------------------------------------------
// Host-side objects behind the opaque C handles.
// ---------------------------------------------------------------------------------------------

constexpr uint32_t Q4K_BLOCK_BYTES = 144;  // 256 weights: f16 d, f16 dmin, 12 B scales, 128 B nibbles
constexpr uint32_t Q6K_BLOCK_BYTES = 210;  // 256 weights: 128 B ql, 64 B qh, 16 i8 scales, f16 d
constexpr uint32_t QK = 256;

// Device-visible status word written by kernels whose bounded waits ran out.
struct DeviceStatus {
  int timeout;      // != 0: a bounded wait gave up (value identifies the kernel)
  int bad_index;    // != 0: an expert id outside [0, n_expert) was clamped
};

}  // namespace infr

namespace infr {
struct EpState;  // ep.cu
}

struct infr_cuda_buf {
  void* ptr = nullptr;
  size_t bytes = 0;
  bool owned = false;
};

struct infr_cuda_graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  uint64_t kernels = 0;  // kernel launches one replay stands for
};

struct infr_cuda_ctx {
  int device = 0;
  int sm_count = 0;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  std::string last_error;
  uint64_t launches = 0;
  bool capturing = false;
  uint64_t capture_launches = 0;  // launches recorded since graph_begin
  // scratch grown on demand (never inside a launch sequence that could be captured)
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  bool scratch_borrowed = false;  // `scratch` points into someone else's block for one nested call: never grown or freed
  infr::DeviceStatus* status = nullptr;       // the device's address of the status words below
  infr::DeviceStatus* status_host = nullptr;  // pinned, mapped host memory: kernels write it directly when they flag something
  // host-paced plans: two 64-bit words in the same pinned block, `bell` written by the host and polled by
  // gated fetch kernels, `done` written by signal kernels and polled by the host (infr_cuda_host_*)
  volatile unsigned long long* bell_host = nullptr;
  volatile unsigned long long* done_host = nullptr;
  unsigned long long* bell_dev = nullptr;
  unsigned long long* done_dev = nullptr;
  float* route_logits = nullptr;              // device memory: the whole-row router kernel's logit buffer, all words
                                              // "not written yet" between launches (see ROUTE_LOGIT_EMPTY)
  unsigned long long* trace = nullptr;        // optional phase stamps (see trace_stamp)
  infr_cuda_config cfg = {};                  // tuning switches (infr_cuda_set_config)
  infr::EpState* ep = nullptr;                // expert-parallel communicator and buffers, or null
  unsigned char* codebook[4] = {nullptr, nullptr, nullptr, nullptr};  // grid tables this context has been given (formats.cuh
                                                                      // slots): the device-wide copies, not owned
};

namespace infr {

int32_t fail(infr_cuda_ctx* ctx, int32_t code, const std::string& msg);
int32_t check_cuda(infr_cuda_ctx* ctx, cudaError_t e, const char* what);
int32_t ensure_scratch(infr_cuda_ctx* ctx, size_t bytes);

// Raise a kernel's dynamic shared-memory limit once per (device, kernel) instead of on every launch.
cudaError_t ensure_smem(const void* kernel, size_t bytes);

#ifdef __CUDACC__
#define INFR_HD __host__ __device__
#else
#define INFR_HD
#endif
// Bytes of a row of n_elem weights (crates/infr-core/src/decode_spec.rs:315-335: elements and bytes per block).
INFR_HD inline size_t row_bytes(int32_t dtype, size_t n_elem) {
  switch (dtype) {
    case INFR_CUDA_DT_F32: return n_elem * 4;
    case INFR_CUDA_DT_Q4K: return n_elem / 256 * 144;
    case INFR_CUDA_DT_Q5K: return n_elem / 256 * 176;
    case INFR_CUDA_DT_Q6K: return n_elem / 256 * 210;
    case INFR_CUDA_DT_Q8_0: return n_elem / 32 * 34;
    case INFR_CUDA_DT_Q4_0: return n_elem / 32 * 18;
    case INFR_CUDA_DT_Q4_1: return n_elem / 32 * 20;
    case INFR_CUDA_DT_Q5_0: return n_elem / 32 * 22;
    case INFR_CUDA_DT_Q5_1: return n_elem / 32 * 24;
    case INFR_CUDA_DT_Q2K: return n_elem / 256 * 84;
    case INFR_CUDA_DT_Q3K: return n_elem / 256 * 110;
    case INFR_CUDA_DT_IQ4NL: return n_elem / 32 * 18;
    case INFR_CUDA_DT_IQ4XS: return n_elem / 256 * 136;
    case INFR_CUDA_DT_MXFP4: return n_elem / 32 * 17;
    case INFR_CUDA_DT_NVFP4: return n_elem / 64 * 36;
    case INFR_CUDA_DT_Q2_0: return n_elem / 64 * 18;
    case INFR_CUDA_DT_IQ2XS: return n_elem / 256 * 74;
    case INFR_CUDA_DT_IQ2S: return n_elem / 256 * 82;
    case INFR_CUDA_DT_IQ3XXS: return n_elem / 256 * 98;
    case INFR_CUDA_DT_IQ3S: return n_elem / 256 * 110;
    default: return 0;
  }
}
// Weights per block of a block format (0: not one).
INFR_HD inline int block_elems(int32_t dtype) {
  if (dtype == INFR_CUDA_DT_NVFP4 || dtype == INFR_CUDA_DT_Q2_0) return 64;
  if (dtype == INFR_CUDA_DT_F32 || !row_bytes(dtype, 256)) return 0;
  return row_bytes(dtype, 32) ? 32 : 256;
}
INFR_HD inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---------------------------------------------------------------------------------------------
// Device helpers.
// ---------------------------------------------------------------------------------------------

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h & 0xFFFFu)));
}

// Four 16-bit fixed-point values X (|X| <= 32639) as signed 8-bit limbs, X = 256 hi + lo with lo in [-128, 127]:
// hi = (X + 128) >> 8 and lo = X - 256 hi, i.e. with Y = X + 128 the second byte of Y and the first byte of Y
// with its top bit flipped.  Byte t of `lo` / `hi` belongs to X[t].
__device__ __forceinline__ void pack_limbs4(const int (&X)[4], uint32_t& lo, uint32_t& hi) {
  const uint32_t p01 = __byte_perm((uint32_t)(X[0] + 128), (uint32_t)(X[1] + 128), 0x5140);  // Y0.b0 Y1.b0 Y0.b1 Y1.b1
  const uint32_t p23 = __byte_perm((uint32_t)(X[2] + 128), (uint32_t)(X[3] + 128), 0x5140);
  lo = __byte_perm(p01, p23, 0x5410) ^ 0x80808080u;
  hi = __byte_perm(p01, p23, 0x7632);
}

// ---- mbarrier + bulk async copy (TMA, untiled form; never multicast) --------------------------

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait: returns false when the limit ran out (the caller records the failure in the
// status word and leaves without touching the data).  The limit is a few seconds of polling.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 24); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 4096) __nanosleep(64);
  }
  return false;
}

// 1-D bulk copy global → this CTA's shared memory, completion counted in bytes on `bar`.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// L2 prefetch of a byte range (16-byte aligned address, size multiple of 16).
__device__ __forceinline__ void bulk_prefetch_l2(const void* gmem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gmem_src), "r"(bytes) : "memory");
}

// Kernel launch with or without the programmatic-dependent-launch attribute (the launched kernel
// may then start before the one ahead of it in the stream has finished; it waits with pdl_wait()).
template <typename K, typename... Args>
inline cudaError_t launch_ex(K kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl, Args... args) {
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


// ---- programmatic dependent launch ------------------------------------------------------------

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- optional phase stamps (latency analysis) ---------------------------------------------------
// When a trace buffer is attached to the context, thread 0 of selected CTAs records
// (globaltimer ns, SM clock) pairs at phase boundaries.  Null pointer = no stores.
__device__ __forceinline__ void trace_stamp(unsigned long long* tr, int slot) {
  if (tr != nullptr && threadIdx.x == 0) {
    unsigned long long g;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g));
    tr[2 * slot] = g;
    tr[2 * slot + 1] = (unsigned long long)clock64();
  }
}

// Grid-wide extremes for the same buffer: earliest / latest time any CTA passed a point.
__device__ __forceinline__ void trace_extreme(unsigned long long* tr, int slot, bool latest) {
  if (tr != nullptr && threadIdx.x == 0) {
    unsigned long long g;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g));
    if (latest) atomicMax(&tr[2 * slot], g);
    else atomicMin(&tr[2 * slot], g);
  }
}

// Per-CTA stamps for the first 128 CTAs: low 40 bits of the global timer, SM id in the low byte.
__device__ __forceinline__ void trace_cta(unsigned long long* tr, int k) {
  if (tr != nullptr && threadIdx.x == 0 && blockIdx.x < 128) {
    unsigned long long g;
    unsigned int sm;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g));
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
    tr[128 + 3 * blockIdx.x + k] = ((g & 0xFFFFFFFFFFull) << 8) | sm;
  }
}

// ---- warp reductions ----------------------------------------------------------------------------

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

// One gated-FFN output element (crates/infr-cpu/src/kernels.rs:6662-6683): act(gate) * up, with the
// optional clamp applied first (gate from above only, up on both sides).
template <bool FAST_DIV = false>
__device__ __forceinline__ float gated_act(int act, float clamp, float g, float u) {
  if (clamp > 0.f) {
    g = fminf(g, clamp);
    u = fminf(fmaxf(u, -clamp), clamp);
  }
  float a;
  if (act == INFR_CUDA_ACT_GELU)
    a = 0.5f * g * (1.0f + tanhf(0.7978846f * (g + 0.044715f * g * g * g)));
  else if (act == INFR_CUDA_ACT_SIGMOID)
    a = 1.0f / (1.0f + __expf(-g));
  else
    a = FAST_DIV ? __fdividef(g, 1.0f + __expf(-g)) : g / (1.0f + __expf(-g));
  return a * u;
}

// ---- in-register block unpack -------------------------------------------------------------------

// Build the f32 whose top mantissa bits hold byte `B` of `w`:  bits = 0x3F000000 | byte<<16.
// With byte = 0x80 | (n << 3) this is exactly 1 + n/16  (n a 4-bit code);
// with byte = 0x80 | (q << 1) this is exactly 1 + q/64  (q a 6-bit code).
template <int B>
__device__ __forceinline__ float byte_to_unit_float(uint32_t w) {
  return __uint_as_float(__byte_perm(w, 0x0000003Fu, 0x4055u | (B << 8)));
}

// Q4_K: 6-bit (scale, min) pairs of sub-blocks 2j and 2j+1 from the 12 scale bytes held in
// words s0..s2 (GGUF `get_scale_min_k4` layout).  Returns sc | (sc' << 8) and m | (m' << 8).
__device__ __forceinline__ void q4k_scale_min_pair(uint32_t s0, uint32_t s1, uint32_t s2, int j, uint32_t& scp,
                                                   uint32_t& mp) {
  const int sh = (j & 1) * 16;
  const uint32_t a = (s0 >> sh) & 0xFFFFu, b = (s1 >> sh) & 0xFFFFu, t = (s2 >> sh) & 0xFFFFu;
  if (j < 2) {
    scp = a & 0x3F3Fu;
    mp = b & 0x3F3Fu;
  } else {
    scp = (t & 0x0F0Fu) | ((a >> 2) & 0x3030u);
    mp = ((t >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u);
  }
}

// Dot product of 64 consecutive weights of a Q4_K block (elements 64j .. 64j+63) with x[0..63].
//   hdr : the block's first 16 bytes (d, dmin, scales[12]);  q : qs[32j .. 32j+31] as 8 words
//   xs0 / xs1 : Σ x[0..31], Σ x[32..63]
// Codes enter the FMA as 1 + n/16 built by byte permutes, so
//   Σ w·x = 16·d·sc·(A − X) − dmin·m·X   per 32-element sub-block, A = Σ (1 + n/16)·x.
__device__ __forceinline__ float q4k_dot64(const uint4& hdr, const uint32_t (&q)[8], const float (&x)[64], float xs0,
                                           float xs1, int j) {
  float2 alo0 = make_float2(0.f, 0.f), alo1 = alo0, ahi0 = alo0, ahi1 = alo0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t w = q[i];
    const uint32_t lo = ((w << 3) & 0x78787878u) | 0x80808080u;
    const uint32_t hi = ((w >> 1) & 0x78787878u) | 0x80808080u;
    alo0 = __ffma2_rn(make_float2(byte_to_unit_float<0>(lo), byte_to_unit_float<1>(lo)),
                      make_float2(x[4 * i + 0], x[4 * i + 1]), alo0);
    alo1 = __ffma2_rn(make_float2(byte_to_unit_float<2>(lo), byte_to_unit_float<3>(lo)),
                      make_float2(x[4 * i + 2], x[4 * i + 3]), alo1);
    ahi0 = __ffma2_rn(make_float2(byte_to_unit_float<0>(hi), byte_to_unit_float<1>(hi)),
                      make_float2(x[32 + 4 * i + 0], x[32 + 4 * i + 1]), ahi0);
    ahi1 = __ffma2_rn(make_float2(byte_to_unit_float<2>(hi), byte_to_unit_float<3>(hi)),
                      make_float2(x[32 + 4 * i + 2], x[32 + 4 * i + 3]), ahi1);
  }
  const float A0 = (alo0.x + alo0.y) + (alo1.x + alo1.y);
  const float A1 = (ahi0.x + ahi0.y) + (ahi1.x + ahi1.y);
  uint32_t scp, mp;
  q4k_scale_min_pair(hdr.y, hdr.z, hdr.w, j, scp, mp);
  const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
  const float s0 = d * (float)(scp & 0xFFu), s1 = d * (float)(scp >> 8);
  const float m0 = dmin * (float)(mp & 0xFFu), m1 = dmin * (float)(mp >> 8);
  return (16.f * s0) * (A0 - xs0) - m0 * xs0 + (16.f * s1) * (A1 - xs1) - m1 * xs1;
}

// Four unsigned bytes of `a` times four signed bytes of `b`, accumulated onto c.
__device__ __forceinline__ int dp4a_us(unsigned a, int b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// Same dot product with the activations in 16-bit fixed point, split into two signed 8-bit limbs
// (X = 256*hi + lo per element, four elements per word): the nibbles of a code word are masked in
// place and multiplied with integer dot-product instructions, which keeps the unpack off the
// (half-rate) logic pipe.  xl/xh: limbs of the 64 elements, sx0/sx1: integer sums of X over the two
// 32-element sub-blocks.  Returns sum(w * X); the caller multiplies by the fixed-point scale.
__device__ __forceinline__ float q4k_dot64_i8(const uint4& hdr, const uint32_t (&q)[8], const int (&xl)[16], const int (&xh)[16],
                                              int sx0, int sx1, int j) {
  int a_ll = 0, a_lh = 0, a_hl = 0, a_hh = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    // the high nibbles stay in place: as unsigned bytes they are 16 x the code, and the exact
    // integer sums are divided by 16 afterwards (one mask per word instead of a shift and a mask)
    const unsigned lo4 = q[i] & 0x0F0F0F0Fu, hi4 = q[i] & 0xF0F0F0F0u;
    a_ll = dp4a_us(lo4, xl[i], a_ll);
    a_lh = dp4a_us(lo4, xh[i], a_lh);
    a_hl = dp4a_us(hi4, xl[8 + i], a_hl);
    a_hh = dp4a_us(hi4, xh[8 + i], a_hh);
  }
  // |v| <= 32 * 15 * 32639 < 2^24 and the 6-bit scales keep the two weighted sums inside int32
  const int v0 = a_lh * 256 + a_ll, v1 = (a_hh * 256 + a_hl) >> 4;
  uint32_t scp, mp;
  q4k_scale_min_pair(hdr.y, hdr.z, hdr.w, j, scp, mp);
  const int sv = (int)(scp & 0xFFu) * v0 + (int)(scp >> 8) * v1;
  const int mv = (int)(mp & 0xFFu) * sx0 + (int)(mp >> 8) * sx1;
  const float d = f16_bits_to_f32(hdr.x), dmin = f16_bits_to_f32(hdr.x >> 16);
  return d * (float)sv - dmin * (float)mv;
}

#endif  // __CUDACC__

}  // namespace infr
