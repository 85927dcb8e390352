// Self-test of the tcgen05 helpers: C[128, N] = A[128, 64] * B[N, 64]^T with f16 operands written
// into 128-byte-swizzled shared memory by ordinary threads, four K = 16 MMAs into tensor memory,
// accumulators read back with tcgen05.ld.  The grouped-GEMM kernels use the same helpers; this
// entry point lets the test-suite check them in isolation against a plain matrix product.
#include "kernels.cuh"
#include "umma.cuh"

namespace infr {
namespace {

__global__ void __launch_bounds__(128) k_umma_selftest(const __half* __restrict__ A, const __half* __restrict__ B,
                                                       float* __restrict__ C, int N, DeviceStatus* status) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ uint32_t s_tmem;
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* tA = smem;               // 128 rows x 128 B
  unsigned char* tB = smem + 128 * 128;   // N rows x 128 B (N <= 256)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t ncols = N <= 32 ? 32 : (N <= 64 ? 64 : (N <= 128 ? 128 : 256));

  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<uint4*>(tA + umma::swz128_offset(tid, c)) = *reinterpret_cast<const uint4*>(A + (size_t)tid * 64 + c * 8);
  for (int r = tid; r < N; r += 128)
    for (int c = 0; c < 8; ++c)
      *reinterpret_cast<uint4*>(tB + umma::swz128_offset(r, c)) = *reinterpret_cast<const uint4*>(B + (size_t)r * 64 + c * 8);
  if (tid == 0) {
    mbar_init(&s_bar, 1);
    mbar_fence_init();
  }
  if (warp == 0) umma::tmem_alloc(&s_tmem, ncols);
  umma::fence_proxy_async();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = s_tmem;

  if (tid == 0) {
    const uint32_t idesc = umma::idesc_f16_f32(128, N);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      umma::mma_f16(tmem, umma::smem_desc_k_major_swz128(tA, k), umma::smem_desc_k_major_swz128(tB, k), idesc, k > 0);
    umma::commit(&s_bar);
  }
  const bool ok = mbar_wait_bounded(&s_bar, 0);
  umma::fence_after_sync();
  if (ok) {
    for (int c0 = 0; c0 < N; c0 += 32) {
      float v[32];
      umma::ld_32x32(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
      for (int i = 0; i < 32 && c0 + i < N; ++i) C[(size_t)(warp * 32 + lane) * N + c0 + i] = v[i];
    }
  } else if (lane == 0) {
    atomicExch(&status->timeout, 9);
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem, ncols);
}

}  // namespace

int32_t launch_umma_selftest(infr_cuda_ctx* ctx, const __half* a, const __half* b, float* c, int n) {
  const size_t smem = 1024 + 128 * 128 + (size_t)n * 128;
  cudaError_t e = ensure_smem(reinterpret_cast<const void*>(k_umma_selftest), smem);
  if (e != cudaSuccess) return check_cuda(ctx, e, "umma selftest smem");
  k_umma_selftest<<<1, 128, smem, ctx->stream>>>(a, b, c, n, ctx->status);
  ctx->launches += 1;
  return check_cuda(ctx, cudaGetLastError(), "umma selftest launch");
}

}  // namespace infr
