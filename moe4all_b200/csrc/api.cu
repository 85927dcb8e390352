// C ABI: context, buffers, descriptor validation and dispatch (see include/infr_cuda.h).
#include <cstdio>
#include <chrono>
#include <cstring>
#include <map>
#include <mutex>
#include <new>

#include "formats.cuh"
#include "kernels.cuh"

namespace infr {

int32_t fail(infr_cuda_ctx* ctx, int32_t code, const std::string& msg) {
  if (ctx) ctx->last_error = msg;
  return code;
}

int32_t check_cuda(infr_cuda_ctx* ctx, cudaError_t e, const char* what) {
  if (e == cudaSuccess) return INFR_CUDA_OK;
  const int32_t code = (e == cudaErrorMemoryAllocation) ? INFR_CUDA_ERR_OOM : INFR_CUDA_ERR_CUDA;
  return fail(ctx, code, std::string(what) + ": " + cudaGetErrorString(e));
}

int32_t ensure_scratch(infr_cuda_ctx* ctx, size_t bytes) {
  if (bytes <= ctx->scratch_bytes) return INFR_CUDA_OK;
  if (ctx->scratch_borrowed)
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "internal: a nested call needs more scratch than was set aside for it");
  if (ctx->capturing)
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "scratch would have to grow while recording: run the call once un-recorded first");
  // growing is a synchronising operation: earlier launches may still use the old block
  cudaError_t e = cudaStreamSynchronize(ctx->stream);
  if (e != cudaSuccess) return check_cuda(ctx, e, "scratch grow: sync");
  if (ctx->scratch) cudaFree(ctx->scratch);
  ctx->scratch = nullptr;
  ctx->scratch_bytes = 0;
  const size_t want = align_up(bytes + bytes / 4, 1 << 20);
  e = cudaMalloc(&ctx->scratch, want);
  if (e != cudaSuccess) return check_cuda(ctx, e, "scratch grow: cudaMalloc");
  ctx->scratch_bytes = want;
  return INFR_CUDA_OK;
}

cudaError_t ensure_smem(const void* kernel, size_t bytes) {
  static std::mutex mu;
  static std::map<std::pair<int, const void*>, size_t> granted;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  size_t& g = granted[{dev, kernel}];
  if (g != 0 && bytes <= g) return cudaSuccess;
  cudaError_t e = cudaSuccess;
  // Ask for the largest shared-memory split on every kernel of the chain: an SM changes its
  // split only when idle, so kernels that prefer different splits cannot share one, and a
  // dependent kernel's CTAs could not start beside those of its predecessor.
  if (g == 0) e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (e == cudaSuccess && bytes > 48 * 1024)
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess) g = bytes > 48 * 1024 ? bytes : 48 * 1024;
  return e;
}

namespace {

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
  }
  ~DeviceGuard() {
    int cur = -1;
    cudaGetDevice(&cur);
    if (prev >= 0 && cur != prev) cudaSetDevice(prev);
  }
};

bool fits(const infr_cuda_buf* b, size_t need) { return b && b->ptr && b->bytes >= need; }

// Device copies of the grid tables, per device (see infr_cuda_set_codebook).
constexpr int MAX_CODEBOOK_DEVICES = 64;
unsigned char* g_codebook_dev[MAX_CODEBOOK_DEVICES][N_CODEBOOKS] = {};
std::mutex g_codebook_mu;

// A grid codebook format whose table the host has not handed over yet.
bool codebook_missing(const infr_cuda_ctx* ctx, int32_t dt) {
  const int slot = codebook_slot(dt);
  return slot >= 0 && ctx->codebook[slot] == nullptr;
}

constexpr size_t HOST_WORDS_BYTES = 192;  // status words, bell word, done word: one 64-byte line each

infr_cuda_config default_config() {
  infr_cuda_config c = {};
  c.gu_warps = 4;
  c.gu_chunks = 4;
  c.dn_warps = 12;
  c.sync_timeout_ms = 60000;
  c.gate_timeout_ms = 2000;
  return c;
}

// Drains the context's stream and reports what kernels flagged: a bounded wait that ran out, or an
// expert id outside [0, n_expert).  The status words live in pinned host memory that the device
// writes directly (and only in those cases), so polling them costs nothing beyond the one wait.
int32_t drain_and_poll(infr_cuda_ctx* ctx, const char* what) {
  if (ctx->ep) {
    // collectives may be queued: a peer that never arrives must not block the host for ever
    const int32_t rc = ep_wait_stream(ctx, what);
    if (rc) return rc;
  } else {
    const cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return check_cuda(ctx, e, what);
  }
  volatile DeviceStatus* st = ctx->status_host;
  const int tag = st->timeout, bad = st->bad_index;
  if (tag || bad) {
    st->timeout = 0;
    st->bad_index = 0;
    // a router launch that gave up may have left logits behind: every word back to "not written yet"
    if (tag && ctx->route_logits) cudaMemset(ctx->route_logits, 0xFF, ROUTE_LOGIT_BYTES);
    if (tag) {
      char msg[96];
      std::snprintf(msg, sizeof msg, "a bounded device-side wait ran out (kernel tag %d); outputs of that call are invalid", tag);
      return fail(ctx, INFR_CUDA_ERR_TIMEOUT, msg);
    }
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG,
                "an expert id outside [0, n_expert) reached a kernel and was served as another expert; outputs of that call are invalid");
  }
  return INFR_CUDA_OK;
}

}  // namespace
}  // namespace infr

using namespace infr;

extern "C" {

const char* infr_cuda_name(void) { return "cuda-sm100a"; }

int32_t infr_cuda_create(int32_t device, infr_cuda_ctx** out) {
  if (!out) return INFR_CUDA_ERR_INVALID_ARG;
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || device < 0 || device >= n) return e == cudaSuccess ? INFR_CUDA_ERR_INVALID_ARG : INFR_CUDA_ERR_CUDA;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return INFR_CUDA_ERR_CUDA;
  if (prop.major != 10) return INFR_CUDA_ERR_UNSUPPORTED;  // the kernels are built for sm_100a only
  infr_cuda_ctx* ctx = new (std::nothrow) infr_cuda_ctx();
  if (!ctx) return INFR_CUDA_ERR_OOM;
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  DeviceGuard g(device);
  if (cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaHostAlloc(reinterpret_cast<void**>(&ctx->status_host), HOST_WORDS_BYTES, cudaHostAllocMapped) != cudaSuccess ||
      cudaHostGetDevicePointer(reinterpret_cast<void**>(&ctx->status), ctx->status_host, 0) != cudaSuccess ||
      cudaMalloc(&ctx->route_logits, ROUTE_LOGIT_BYTES) != cudaSuccess ||
      cudaMemset(ctx->route_logits, 0xFF, ROUTE_LOGIT_BYTES) != cudaSuccess) {
    infr_cuda_destroy(ctx);
    return INFR_CUDA_ERR_CUDA;
  }
  std::memset(ctx->status_host, 0, HOST_WORDS_BYTES);
  // the pacing words of host-paced plans: each on a cache line of its own behind the status words
  ctx->bell_host = reinterpret_cast<volatile unsigned long long*>(reinterpret_cast<char*>(ctx->status_host) + 64);
  ctx->done_host = reinterpret_cast<volatile unsigned long long*>(reinterpret_cast<char*>(ctx->status_host) + 128);
  ctx->bell_dev = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(ctx->status) + 64);
  ctx->done_dev = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(ctx->status) + 128);
  ctx->stream = ctx->own_stream;
  ctx->cfg = default_config();
  *out = ctx;
  return INFR_CUDA_OK;
}

void infr_cuda_destroy(infr_cuda_ctx* ctx) {
  if (!ctx) return;
  DeviceGuard g(ctx->device);
  if (ctx->ep) ep_release(ctx, false);
  if (ctx->own_stream) cudaStreamSynchronize(ctx->own_stream);
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->status_host) cudaFreeHost(ctx->status_host);
  if (ctx->route_logits) cudaFree(ctx->route_logits);
  if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
  delete ctx;
}

const char* infr_cuda_last_error(const infr_cuda_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

int32_t infr_cuda_set_stream(infr_cuda_ctx* ctx, void* cuda_stream) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  ctx->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : ctx->own_stream;
  return INFR_CUDA_OK;
}

int32_t infr_cuda_get_config(const infr_cuda_ctx* ctx, infr_cuda_config* out) {
  if (!ctx || !out) return INFR_CUDA_ERR_INVALID_ARG;
  *out = ctx->cfg;
  return INFR_CUDA_OK;
}

int32_t infr_cuda_set_config(infr_cuda_ctx* ctx, const infr_cuda_config* cfg) {
  if (!ctx || !cfg) return INFR_CUDA_ERR_INVALID_ARG;
  if (cfg->gu_chunks > 4 || cfg->gu_warps > 16 || cfg->dn_warps > 24 || cfg->expert_major > 2 || cfg->raw_rows_f32 > 1)
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "set_config: a field is outside its range");
  for (uint32_t r : cfg->reserved)
    if (r) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "set_config: reserved fields must be zero");
  ctx->cfg = *cfg;
  return INFR_CUDA_OK;
}

int32_t infr_cuda_alloc(infr_cuda_ctx* ctx, size_t bytes, int32_t zero, infr_cuda_buf** out) {
  if (!ctx || !out) return INFR_CUDA_ERR_INVALID_ARG;
  *out = nullptr;
  DeviceGuard g(ctx->device);
  infr_cuda_buf* b = new (std::nothrow) infr_cuda_buf();
  if (!b) return fail(ctx, INFR_CUDA_ERR_OOM, "alloc: host out of memory");
  // (16 spare bytes; no kernel needs them - none reads past a bank's last block)
  cudaError_t e = cudaMalloc(&b->ptr, bytes + 16);
  if (e != cudaSuccess) {
    delete b;
    cudaGetLastError();
    return check_cuda(ctx, e, "alloc");
  }
  if (zero) {
    e = cudaMemsetAsync(b->ptr, 0, bytes + 16, ctx->stream);
    if (e != cudaSuccess) {
      cudaFree(b->ptr);
      delete b;
      return check_cuda(ctx, e, "alloc: memset");
    }
  }
  b->bytes = bytes;
  b->owned = true;
  *out = b;
  return INFR_CUDA_OK;
}

int32_t infr_cuda_wrap(infr_cuda_ctx* ctx, void* device_ptr, size_t bytes, infr_cuda_buf** out) {
  if (!ctx || !out) return INFR_CUDA_ERR_INVALID_ARG;
  *out = nullptr;
  if (!device_ptr) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "wrap: null device pointer");
  if (reinterpret_cast<uintptr_t>(device_ptr) % 16) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "wrap: pointer must be 16-byte aligned");
  infr_cuda_buf* b = new (std::nothrow) infr_cuda_buf();
  if (!b) return fail(ctx, INFR_CUDA_ERR_OOM, "wrap: host out of memory");
  b->ptr = device_ptr;
  b->bytes = bytes;
  b->owned = false;
  *out = b;
  return INFR_CUDA_OK;
}

void infr_cuda_free(infr_cuda_ctx* ctx, infr_cuda_buf* buf) {
  if (!buf) return;
  if (buf->owned && buf->ptr) {
    if (ctx) {
      DeviceGuard g(ctx->device);
      cudaStreamSynchronize(ctx->stream);
      cudaFree(buf->ptr);
    } else {
      cudaFree(buf->ptr);
    }
  }
  delete buf;
}

size_t infr_cuda_buf_len(const infr_cuda_buf* buf) { return buf ? buf->bytes : 0; }
void* infr_cuda_buf_ptr(const infr_cuda_buf* buf) { return buf ? buf->ptr : nullptr; }

int32_t infr_cuda_upload(infr_cuda_ctx* ctx, infr_cuda_buf* dst, size_t dst_off, const void* src, size_t n) {
  if (!ctx || !dst || (!src && n)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "upload: null argument");
  if (dst_off > dst->bytes || n > dst->bytes - dst_off) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "upload: range exceeds the buffer");
  if (!n) return INFR_CUDA_OK;
  DeviceGuard g(ctx->device);
  cudaError_t e = cudaMemcpyAsync(static_cast<char*>(dst->ptr) + dst_off, src, n, cudaMemcpyHostToDevice, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  return check_cuda(ctx, e, "upload");
}

int32_t infr_cuda_download(infr_cuda_ctx* ctx, const infr_cuda_buf* src, size_t src_off, void* dst, size_t n) {
  if (!ctx || !src || (!dst && n)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "download: null argument");
  if (src_off > src->bytes || n > src->bytes - src_off) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "download: range exceeds the buffer");
  DeviceGuard g(ctx->device);
  cudaError_t e = cudaSuccess;
  if (n) e = cudaMemcpyAsync(dst, static_cast<const char*>(src->ptr) + src_off, n, cudaMemcpyDeviceToHost, ctx->stream);
  if (e != cudaSuccess) return check_cuda(ctx, e, "download");
  return drain_and_poll(ctx, "download");
}

int32_t infr_cuda_upload_async(infr_cuda_ctx* ctx, infr_cuda_buf* dst, size_t dst_off, const void* src, size_t n) {
  if (!ctx || !dst || (!src && n)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "upload: null argument");
  if (dst_off > dst->bytes || n > dst->bytes - dst_off) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "upload: range exceeds the buffer");
  if (!n) return INFR_CUDA_OK;
  DeviceGuard g(ctx->device);
  char* d = static_cast<char*>(dst->ptr) + dst_off;
  // a few rows from pinned memory: fetched by a kernel, which the next kernel can overlap
  if (!ctx->cfg.upload_by_copy && n <= (256u << 10) && n % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(d) % 16 == 0) {
    cudaPointerAttributes at = {};
    if (cudaPointerGetAttributes(&at, src) == cudaSuccess && at.type == cudaMemoryTypeHost && at.devicePointer != nullptr)
      return launch_fetch_host(ctx, at.devicePointer, d, n);
    (void)cudaGetLastError();  // pageable memory: not an error, the copy engine takes it
  }
  return check_cuda(ctx, cudaMemcpyAsync(d, src, n, cudaMemcpyHostToDevice, ctx->stream), "upload (queued)");
}

int32_t infr_cuda_download_async(infr_cuda_ctx* ctx, const infr_cuda_buf* src, size_t src_off, void* dst, size_t n) {
  if (!ctx || !src || (!dst && n)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "download: null argument");
  if (src_off > src->bytes || n > src->bytes - src_off) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "download: range exceeds the buffer");
  if (!n) return INFR_CUDA_OK;
  DeviceGuard g(ctx->device);
  const char* sp = static_cast<const char*>(src->ptr) + src_off;
  if (!ctx->cfg.upload_by_copy && n <= (256u << 10) && n % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0 && reinterpret_cast<uintptr_t>(sp) % 16 == 0) {
    cudaPointerAttributes at = {};
    if (cudaPointerGetAttributes(&at, dst) == cudaSuccess && at.type == cudaMemoryTypeHost && at.devicePointer != nullptr)
      return launch_store_host(ctx, sp, at.devicePointer, n);
    (void)cudaGetLastError();
  }
  return check_cuda(ctx, cudaMemcpyAsync(dst, sp, n, cudaMemcpyDeviceToHost, ctx->stream), "download (queued)");
}

int32_t infr_cuda_set_codebook(infr_cuda_ctx* ctx, int32_t dtype, const void* table, size_t bytes) {
  if (!ctx || !table) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "set_codebook: null argument");
  const int slot = codebook_slot(dtype);
  if (slot < 0) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "set_codebook: not a grid codebook format (IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S)");
  if (bytes != codebook_bytes(slot)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "set_codebook: wrong table size for this format");
  const unsigned char* tb = static_cast<const unsigned char*>(table);
  for (size_t i = 0; i < bytes; ++i)
    if (tb[i] >= 128) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "set_codebook: grid bytes must be below 128");
  if (ctx->capturing) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "set_codebook: not while recording");
  if (ctx->device < 0 || ctx->device >= MAX_CODEBOOK_DEVICES) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "set_codebook: device index beyond 63");
  DeviceGuard g(ctx->device);
  // The device copies belong to the device, not to the context: the kernels find them through constant memory,
  // which every context of the device shares, so a table stays where it is (and allocated, a few KB) until the
  // process ends; a context only remembers that it has been given one.
  std::lock_guard<std::mutex> lk(g_codebook_mu);
  unsigned char** dev = g_codebook_dev[ctx->device];
  cudaError_t e = cudaDeviceSynchronize();  // no kernel of any context reads a table while it changes
  if (e == cudaSuccess && !dev[slot]) e = cudaMalloc(reinterpret_cast<void**>(&dev[slot]), bytes);
  if (e == cudaSuccess) e = cudaMemcpy(dev[slot], table, bytes, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = publish_codebooks_dense(dev);
  if (e == cudaSuccess) e = publish_codebooks_anyfmt(dev);
  if (e == cudaSuccess) e = publish_codebooks_grouped(dev);
  if (e == cudaSuccess) ctx->codebook[slot] = dev[slot];
  return check_cuda(ctx, e, "set_codebook");
}

int32_t infr_cuda_upload_gated(infr_cuda_ctx* ctx, infr_cuda_buf* dst, size_t dst_off, const void* src, size_t n, uint64_t ticket) {
  if (!ctx || !dst || !src) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "upload_gated: null argument");
  if (dst_off > dst->bytes || n > dst->bytes - dst_off) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "upload_gated: range exceeds the buffer");
  if (!n || !ticket) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "upload_gated: nothing to copy, or ticket 0");
  DeviceGuard g(ctx->device);
  char* d = static_cast<char*>(dst->ptr) + dst_off;
  cudaPointerAttributes at = {};
  const bool shape_ok = n <= (256u << 10) && n % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(d) % 16 == 0;
  if (!shape_ok || cudaPointerGetAttributes(&at, src) != cudaSuccess || at.type != cudaMemoryTypeHost || at.devicePointer == nullptr) {
    (void)cudaGetLastError();
    return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "upload_gated: the source must be pinned host memory, 16-byte aligned, a multiple of 16 bytes and at most 256 KB");
  }
  const unsigned long long limit_ns = (unsigned long long)(ctx->cfg.gate_timeout_ms ? ctx->cfg.gate_timeout_ms : 2000u) * 1000000ull;
  return launch_fetch_host_gated(ctx, at.devicePointer, d, n, ctx->bell_dev, ticket, limit_ns);
}

int32_t infr_cuda_host_signal(infr_cuda_ctx* ctx, uint64_t ticket) {
  if (!ctx || !ticket) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "host_signal: null context or ticket 0");
  DeviceGuard g(ctx->device);
  return launch_host_signal(ctx, ctx->done_dev, ticket);
}

int32_t infr_cuda_host_ring(infr_cuda_ctx* ctx, uint64_t ticket) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  // release: the rows the host wrote into pinned memory before this call are in memory before the ticket
  __atomic_store_n(const_cast<unsigned long long*>(ctx->bell_host), (unsigned long long)ticket, __ATOMIC_RELEASE);
  return INFR_CUDA_OK;
}

int32_t infr_cuda_host_await(infr_cuda_ctx* ctx, uint64_t ticket) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  const auto t0 = std::chrono::steady_clock::now();
  const auto limit = std::chrono::milliseconds(ctx->cfg.gate_timeout_ms ? ctx->cfg.gate_timeout_ms : 2000u);
  volatile DeviceStatus* st = ctx->status_host;
  for (unsigned spin = 0;; ++spin) {
    if (__atomic_load_n(const_cast<unsigned long long*>(ctx->done_host), __ATOMIC_ACQUIRE) >= ticket) {
      if (st->timeout || st->bad_index) break;  // reported below, once the stream has drained
      return INFR_CUDA_OK;
    }
    if (st->timeout || st->bad_index) break;
    if ((spin & 1023u) == 1023u && std::chrono::steady_clock::now() - t0 > limit) {
      // nothing answered: let the gates still queued run out (they stop waiting once a status is recorded)
      st->timeout = 10;
      break;
    }
#if defined(__x86_64__) || defined(__i386__)
    __builtin_ia32_pause();
#endif
  }
  DeviceGuard g(ctx->device);
  const int32_t rc = drain_and_poll(ctx, "host_await");
  return rc ? rc : fail(ctx, INFR_CUDA_ERR_TIMEOUT, "host_await: the ticket was not signalled in time");
}

int32_t infr_cuda_host_step(infr_cuda_ctx* ctx, uint64_t ticket, void* stage, const void* rows, size_t n) {
  if (!ctx || (rows && !stage)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "host_step: null argument");
  if (rows && n) std::memcpy(stage, rows, n);
  infr_cuda_host_ring(ctx, ticket);
  return infr_cuda_host_await(ctx, ticket);
}

int32_t infr_cuda_host_steps(infr_cuda_ctx* ctx, uint64_t first_ticket, uint32_t count, void* stage, const void* const* rows, size_t n_in,
                             const void* result, void* const* results_out, size_t n_out) {
  if (!ctx || !stage || !rows || (results_out && !result)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "host_steps: null argument");
  for (uint32_t i = 0; i < count; ++i) {
    const int32_t rc = infr_cuda_host_step(ctx, first_ticket + i, stage, rows[i], n_in);
    if (rc) return rc;
    if (results_out && results_out[i] && n_out) std::memcpy(results_out[i], result, n_out);
  }
  return INFR_CUDA_OK;
}

int32_t infr_cuda_host_reset(infr_cuda_ctx* ctx) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  if (ctx->capturing) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "host_reset: not while recording");
  DeviceGuard g(ctx->device);
  const int32_t rc = drain_and_poll(ctx, "host_reset");
  *ctx->bell_host = 0;
  *ctx->done_host = 0;
  __atomic_thread_fence(__ATOMIC_SEQ_CST);
  return rc;
}

int32_t infr_cuda_sync(infr_cuda_ctx* ctx) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  DeviceGuard g(ctx->device);
  return drain_and_poll(ctx, "sync");
}

uint64_t infr_cuda_launch_count(const infr_cuda_ctx* ctx) { return ctx ? ctx->launches : 0; }

int32_t infr_cuda_set_trace(infr_cuda_ctx* ctx, infr_cuda_buf* buf) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  if (buf && buf->bytes < 4096) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "set_trace: the buffer must hold 4096 bytes");
  ctx->trace = buf ? static_cast<unsigned long long*>(buf->ptr) : nullptr;
  return INFR_CUDA_OK;
}

int32_t infr_cuda_graph_begin(infr_cuda_ctx* ctx) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  if (ctx->capturing) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "graph_begin: already recording");
  DeviceGuard g(ctx->device);
  cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal);
  if (e != cudaSuccess) return check_cuda(ctx, e, "graph_begin");
  ctx->capturing = true;
  ctx->capture_launches = ctx->launches;
  return INFR_CUDA_OK;
}

int32_t infr_cuda_graph_end(infr_cuda_ctx* ctx, infr_cuda_graph** out) {
  if (!ctx || !out) return INFR_CUDA_ERR_INVALID_ARG;
  *out = nullptr;
  if (!ctx->capturing) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "graph_end: not recording");
  DeviceGuard g(ctx->device);
  ctx->capturing = false;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
  if (e != cudaSuccess || !graph) return check_cuda(ctx, e == cudaSuccess ? cudaErrorUnknown : e, "graph_end");
  cudaGraphExec_t exec = nullptr;
  e = cudaGraphInstantiate(&exec, graph, 0);
  if (e != cudaSuccess) {
    cudaGraphDestroy(graph);
    return check_cuda(ctx, e, "graph instantiate");
  }
  infr_cuda_graph* gr = new (std::nothrow) infr_cuda_graph();
  if (!gr) {
    cudaGraphExecDestroy(exec);
    cudaGraphDestroy(graph);
    return fail(ctx, INFR_CUDA_ERR_OOM, "graph_end: host out of memory");
  }
  gr->graph = graph;
  gr->exec = exec;
  gr->kernels = ctx->launches - ctx->capture_launches;
  ctx->launches = ctx->capture_launches;  // recorded launches have not run
  *out = gr;
  return INFR_CUDA_OK;
}

int32_t infr_cuda_graph_launch(infr_cuda_ctx* ctx, infr_cuda_graph* graph) {
  if (!ctx || !graph || !graph->exec) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "graph_launch: null graph");
  DeviceGuard g(ctx->device);
  cudaError_t e = cudaGraphLaunch(graph->exec, ctx->stream);
  if (e == cudaSuccess) ctx->launches += graph->kernels;
  return check_cuda(ctx, e, "graph_launch");
}

void infr_cuda_graph_free(infr_cuda_ctx* ctx, infr_cuda_graph* graph) {
  if (!graph) return;
  if (ctx) {
    DeviceGuard g(ctx->device);
    cudaStreamSynchronize(ctx->stream);
  }
  if (graph->exec) cudaGraphExecDestroy(graph->exec);
  if (graph->graph) cudaGraphDestroy(graph->graph);
  delete graph;
}

// ---- Op::MoeFfn ---------------------------------------------------------------------------------

}  // extern "C"

namespace infr {

int32_t validate_moe_route(infr_cuda_ctx* ctx, const infr_cuda_moe_ffn_desc* d) {
  if (!d) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: null descriptor");
  if (!d->rows || !d->ne || !d->n_expert || !d->n_used) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: zero dimension");
  // (a call that takes its routing as an input may hold fewer experts than a token uses: an expert-parallel band)
  if (d->n_used > d->n_expert && (d->stages == 0 || (d->stages & 1u)))
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: n_used exceeds n_expert");
  if (d->n_used > 32) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_ffn: n_used > 32 is not covered");
  if (d->n_expert > 1024) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_ffn: more than 1024 experts is not covered");
  if (d->ne % 64) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_ffn: ne must be a multiple of 64");
  if (d->router_dtype != INFR_CUDA_DT_F32) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_ffn: router dtype must be F32");
  if (d->gating > INFR_CUDA_GATING_SQRT_SOFTPLUS)
    return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_ffn: gating must be softmax, sigmoid or sqrt-softplus");
  if (d->n_expert_groups > 1 && d->n_expert_groups_used > 0) {
    if (d->n_expert_groups > 32) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_ffn: more than 32 expert groups is not covered");
    if (d->n_expert % d->n_expert_groups) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: n_expert is not a multiple of n_expert_groups");
  }
  const size_t xb = (size_t)d->rows * d->ne * 4;
  if (!fits(d->router_x, xb)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: router_x missing or too small");
  if (!fits(d->router, (size_t)d->n_expert * d->ne * 4)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: router missing or too small");
  if (d->exp_probs_b && !fits(d->exp_probs_b, (size_t)d->n_expert * 4)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: exp_probs_b too small");
  if (d->expert_ids) {
    // there is no selection to bias or to limit to groups (graph.rs:1304-1308, 1344-1347)
    if (d->exp_probs_b || d->n_expert_groups > 1)
      return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: expert_ids excludes exp_probs_b and expert groups");
    if (!fits(d->expert_ids, (size_t)d->rows * d->n_used * 4)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: expert_ids too small");
  }
  const size_t kb = (size_t)d->rows * d->n_used * 4;
  if (d->ids_out && !fits(d->ids_out, kb)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: ids_out too small");
  if (d->wts_out && !fits(d->wts_out, kb)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: wts_out too small");
  return INFR_CUDA_OK;
}

// `bank_experts`: experts held by gate_exps / up_exps / down_exps (n_expert, or the band of an
// expert-parallel rank).
int32_t validate_moe_ffn(infr_cuda_ctx* ctx, const infr_cuda_moe_ffn_desc* d, uint32_t bank_experts) {
  int32_t rc = validate_moe_route(ctx, d);
  if (rc) return rc;
  if (!d->n_ff_exp) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: zero n_ff_exp");
  if (!bank_dtype_ok(d->gate_dtype) || !bank_dtype_ok(d->up_dtype) || !bank_dtype_ok(d->down_dtype))
    return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_ffn: expert banks must be one of Q4_0 Q4_1 Q5_0 Q5_1 Q8_0 Q2_K Q3_K Q4_K Q5_K Q6_K IQ4_NL IQ4_XS MXFP4 NVFP4 Q2_0 IQ2_XS IQ2_S IQ3_XXS IQ3_S");
  if (codebook_missing(ctx, d->gate_dtype) || codebook_missing(ctx, d->up_dtype) || codebook_missing(ctx, d->down_dtype))
    return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_ffn: a bank is in a grid codebook format whose table has not been set (infr_cuda_set_codebook)");
  if (d->fused_gate_up && d->gate_dtype != d->up_dtype)
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: a fused gate/up bank has one dtype");
  if (d->ne % 256 || d->n_ff_exp % 256) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: ne and n_ff_exp must be multiples of the 256-weight block");
  const size_t xb = (size_t)d->rows * d->ne * 4;
  if (!fits(d->x, xb)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: x missing or too small");
  if (!fits(d->dst, xb)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: dst missing or too small");
  const size_t gb = (size_t)bank_experts * d->n_ff_exp * row_bytes(d->gate_dtype, d->ne);
  const size_t ub = (size_t)bank_experts * d->n_ff_exp * row_bytes(d->up_dtype, d->ne);
  const size_t db = (size_t)bank_experts * d->ne * row_bytes(d->down_dtype, d->n_ff_exp);
  if (d->fused_gate_up ? !fits(d->gate_exps, 2 * gb) : (!fits(d->gate_exps, gb) || !fits(d->up_exps, ub)))
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: gate/up bank missing or too small");
  if (!fits(d->down_exps, db)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: down bank missing or too small");
  if (d->norm_weight) {
    if (!fits(d->norm_weight, (size_t)d->ne * 4)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: norm_weight too small");
    if (d->router_x->ptr != d->x->ptr) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: the RmsNorm fusion needs router_x == x");
    if (d->ne > 8192) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_ffn: the RmsNorm fusion covers ne <= 8192");
  }
  if (d->residual && !fits(d->residual, xb)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: residual too small");
  if (d->act > INFR_CUDA_ACT_SIGMOID) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_ffn: act must be SiLU, GELU or Sigmoid");
  if (d->act == INFR_CUDA_ACT_SIGMOID && d->swiglu_clamp > 0.0f) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: swiglu_clamp excludes the Sigmoid activation");
  if (!(d->swiglu_clamp >= 0.0f)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: swiglu_clamp must be positive, or 0 for none");
  // the reference defines the clamp for the output-weighted forms only (crates/infr-cpu/src/lib.rs:3613-3619)
  if (d->swiglu_clamp > 0.0f && d->weight_before) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: swiglu_clamp excludes weight_before");
  if (d->down_scale && !fits(d->down_scale, (size_t)d->n_expert * 4)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: down_scale too small");
  if (d->ep_n_local && (uint64_t)d->ep_lo + d->ep_n_local > d->n_expert)
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: ep band exceeds n_expert");
  if (d->sh_gate || d->sh_up || d->sh_down) {
    if (!d->sh_gate || !d->sh_up || !d->sh_down || !d->sh_ff || d->sh_ff % 256)
      return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: shared expert needs gate, up, down and sh_ff (multiple of 256)");
    const size_t sgb = (size_t)d->sh_ff * row_bytes(d->gate_dtype, d->ne), sub = (size_t)d->sh_ff * row_bytes(d->up_dtype, d->ne);
    const size_t sdb = (size_t)d->ne * row_bytes(d->down_dtype, d->sh_ff);
    if (!fits(d->sh_gate, sgb) || !fits(d->sh_up, sub) || !fits(d->sh_down, sdb))
      return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: shared expert tensor too small");
    if (d->sh_gate_inp && !fits(d->sh_gate_inp, (size_t)d->ne * 4))
      return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: sh_gate_inp too small");
  } else if (d->sh_gate_inp) {
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_ffn: sh_gate_inp without a shared expert");
  }
  return INFR_CUDA_OK;
}

// Which kernels serve a call of `rows` rows (measured on B200, 256 experts top-8, experts of 2 MB and of
// 28 MB; pp = one CTA per pair, em = expert-major integer tensor-core tiles, gg = grouped GEMM on tcgen05):
//   experts of 2 MB:   32 rows pp 174 / em 168 / gg 313 us; 64: 330 / 227 / 420; 256: 1206 / 363 / 488
//   experts of 28 MB:  2 rows pp 290 / em 196 / gg 385 us; 64: 8190 / 2247 / 4083; 256: 32770 / 3785 / 4649
// The expert-major form's time grows with the rows per expert, the grouped GEMM's hardly at all: they cross
// near 11 (token, expert) pairs per expert.
bool em_preferred(uint32_t rows, uint32_t n_used, uint32_t n_expert, uint32_t ne, uint32_t nff) {
  const bool big = (uint64_t)ne * nff >= (1ull << 23);  // experts of tens of megabytes
  return big ? rows >= 2 : (uint64_t)rows * n_used >= n_expert;
}

uint32_t choose_moe_path(const infr_cuda_ctx* ctx, uint32_t rows, uint32_t n_used, uint32_t n_expert, uint32_t ne, uint32_t nff,
                         uint32_t sh_ff, BankTypes bt) {
  const bool small_ok = decode_ffn_supported(ctx, (int)ne, (int)nff, (int)sh_ff, (int)n_used, bt, nullptr);
  const bool em_ok = ctx->cfg.expert_major != 1 && em_supported((int)ne, (int)nff, (int)sh_ff, (int)n_expert, bt);
  const uint64_t pairs8 = (uint64_t)rows * n_used * 8;
  if (em_ok && pairs8 < (uint64_t)n_expert * 88) return 1;  // fewer than 11 pairs per expert
  // without the expert-major kernels: per-pair kernels while an expert sees fewer than 2.75 rows (not for
  // experts of tens of megabytes, where they hold one chunk of rows per CTA)
  const bool big = (uint64_t)ne * nff >= (1ull << 23);
  const bool few_per_expert = pairs8 <= (uint64_t)n_expert * 22;
  return (small_ok && (big ? rows < 8 : (rows <= 8 || few_per_expert))) ? 1 : 2;
}

}  // namespace infr

extern "C" {

namespace {
// Scratch carve-up for one call.
struct Scratch {
  int8_t *xq_lo, *xq_hi;
  float* xscale;
  float* logits;
  float* sh_logit;
  int32_t* ids;
  float* wts;
  float* act;
  size_t total;
};

Scratch carve(void* base, const infr_cuda_moe_ffn_desc* d, bool with_act) {
  Scratch s;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    void* p = base ? static_cast<char*>(base) + off : nullptr;
    off += align_up(bytes, 256);
    return p;
  };
  s.logits = static_cast<float*>(take((size_t)d->rows * d->n_expert * 4));
  s.sh_logit = static_cast<float*>(take((size_t)d->rows * 4));
  s.ids = static_cast<int32_t*>(take((size_t)d->rows * d->n_used * 4));
  s.wts = static_cast<float*>(take((size_t)d->rows * d->n_used * 4));
  s.act = with_act ? static_cast<float*>(take(((size_t)d->rows * d->n_used * d->n_ff_exp + (size_t)d->rows * d->sh_ff) * 4)) : nullptr;
  s.xq_lo = with_act ? static_cast<int8_t*>(take((size_t)d->rows * d->ne)) : nullptr;
  s.xq_hi = with_act ? static_cast<int8_t*>(take((size_t)d->rows * d->ne)) : nullptr;
  s.xscale = with_act ? static_cast<float*>(take((size_t)d->rows * 4)) : nullptr;
  s.total = off;
  return s;
}

RouteParams route_params(infr_cuda_ctx* ctx, const infr_cuda_moe_ffn_desc* d, const Scratch& s, bool with_gate) {
  RouteParams rp = {};
  rp.status = ctx->status;
  rp.router_x = static_cast<const float*>(d->router_x->ptr);
  rp.x = d->x ? static_cast<const float*>(d->x->ptr) : rp.router_x;
  rp.router = static_cast<const float*>(d->router->ptr);
  rp.sh_gate_inp = (with_gate && d->sh_gate_inp) ? static_cast<const float*>(d->sh_gate_inp->ptr) : nullptr;
  rp.bias = d->exp_probs_b ? static_cast<const float*>(d->exp_probs_b->ptr) : nullptr;
  rp.given_ids = d->expert_ids ? static_cast<const int32_t*>(d->expert_ids->ptr) : nullptr;
  rp.logits = s.logits;
  rp.sh_logit = s.sh_logit;
  rp.ids = d->ids_out ? static_cast<int32_t*>(d->ids_out->ptr) : s.ids;
  rp.wts = d->wts_out ? static_cast<float*>(d->wts_out->ptr) : s.wts;
  rp.trace = ctx->trace;
  rp.rows = d->rows;
  rp.ne = d->ne;
  rp.n_expert = d->n_expert;
  rp.n_used = d->n_used;
  rp.scale = d->scale;
  rp.gating = d->gating;
  rp.norm_w = d->norm_w ? 1 : 0;
  rp.n_groups = d->n_expert_groups;
  rp.n_groups_used = d->n_expert_groups_used;
  return rp;
}
}  // namespace

}  // extern "C"

namespace infr {
// Upper bound on the context scratch a small-m (path 1) call of this descriptor uses, whichever form serves it.
size_t small_path_scratch_need(const infr_cuda_moe_ffn_desc* d) {
  const int sh_ff = d->sh_gate ? (int)d->sh_ff : 0;
  return carve(nullptr, d, true).total + align_up((size_t)d->rows * d->ne * 4, 256) +
         em_scratch_bytes((int)d->rows, (int)d->n_used, (int)d->ne, (int)d->n_ff_exp, sh_ff) + 4096;
}
}  // namespace infr

extern "C" {

int32_t infr_cuda_moe_route(infr_cuda_ctx* ctx, const infr_cuda_moe_ffn_desc* d) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  int32_t rc = validate_moe_route(ctx, d);
  if (rc) return rc;
  if (!d->ids_out || !d->wts_out) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_route: ids_out and wts_out are required");
  DeviceGuard g(ctx->device);
  Scratch sz = carve(nullptr, d, false);
  if ((rc = ensure_scratch(ctx, sz.total))) return rc;
  Scratch s = carve(ctx->scratch, d, false);
  RouteParams rp = route_params(ctx, d, s, false);
  return launch_route(ctx, rp, false);
}

int32_t infr_cuda_moe_ffn(infr_cuda_ctx* ctx, const infr_cuda_moe_ffn_desc* d) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  if (d && ep_call_is_collective(ctx, d)) return ep_moe_ffn(ctx, d);
  int32_t rc = validate_moe_ffn(ctx, d, d->n_expert);
  if (rc) return rc;
  DeviceGuard g(ctx->device);
  const bool has_sh = d->sh_gate != nullptr;
  std::string why;
  const BankTypes bt = {d->gate_dtype, d->up_dtype, d->down_dtype};
  const bool down_q4k = bt.down_q4k();
  const int sh_ff_eff = has_sh ? (int)d->sh_ff : 0;
  const bool small_ok = decode_ffn_supported(ctx, d->ne, d->n_ff_exp, sh_ff_eff, d->n_used, bt, &why);
  const bool em_ok = em_supported((int)d->ne, (int)d->n_ff_exp, sh_ff_eff, (int)d->n_expert, bt);
  uint32_t path = d->path;
  if (path == 0) path = choose_moe_path(ctx, d->rows, d->n_used, d->n_expert, d->ne, d->n_ff_exp, sh_ff_eff, bt);
  // One CTA per (token, expert) pair, or one per expert with all its tokens: the second form reads and
  // unpacks an expert's blocks once however many rows of the call it serves, at the price of two more
  // (small) launches.
  const bool use_em = path == 1 && em_ok &&
                      (ctx->cfg.expert_major == 2 || !small_ok ||
                       (ctx->cfg.expert_major == 0 && em_preferred(d->rows, d->n_used, d->n_expert, d->ne, d->n_ff_exp)));
  if (path == 1) {
    if (!small_ok && !use_em) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, why);
    // Where the whole-row router kernel covers the call it also normalises x and makes its
    // fixed-point copy; otherwise the batched router runs and two small kernels do those jobs.
    const bool few = route_small_group(ctx, (int)d->rows, (int)d->ne, (int)d->n_expert) > 0;
    Scratch sz = carve(nullptr, d, true);
    const size_t hn_bytes = (!few && d->norm_weight) ? align_up((size_t)d->rows * d->ne * 4, 256) : 0;
    const size_t em_bytes = use_em ? em_scratch_bytes((int)d->rows, (int)d->n_used, (int)d->ne, (int)d->n_ff_exp, sh_ff_eff) : 0;
    if ((rc = ensure_scratch(ctx, sz.total + hn_bytes + em_bytes))) return rc;
    Scratch s = carve(ctx->scratch, d, true);
    RouteParams rp = route_params(ctx, d, s, true);
    const uint32_t stages = d->stages ? d->stages : 7u;
    bool xsum_ready = false;
    if (few) {
      rp.xq_lo = s.xq_lo;
      rp.xq_hi = s.xq_hi;
      rp.xscale = s.xscale;
      if (use_em && (stages & 1u)) {
        // the expert-major kernels' sums of x (the first array of their scratch) come out of the same pass
        rp.xsum = reinterpret_cast<int*>(static_cast<char*>(ctx->scratch) + sz.total + hn_bytes);
        xsum_ready = true;
      }
      rp.rms_w = d->norm_weight ? static_cast<const float*>(d->norm_weight->ptr) : nullptr;
      rp.rms_eps = d->norm_eps;
      if (stages & 1u) {
        if ((rc = launch_route(ctx, rp, true))) return rc;
      } else if (stages & 8u) {
        // routing came from elsewhere: the router kernel, which would have made the fixed-point copy, does not run
        if (d->norm_weight) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_ffn: stages without the router cannot apply norm_weight");
        if ((rc = launch_quantize_rows(ctx, static_cast<const float*>(d->x->ptr), s.xq_lo, s.xq_hi, s.xscale, (int)d->rows, (int)d->ne))) return rc;
      }
    } else if (stages & 1u) {
      const float* x_eff = static_cast<const float*>(d->x->ptr);
      if (d->norm_weight) {
        float* hn = reinterpret_cast<float*>(static_cast<char*>(ctx->scratch) + sz.total);
        if ((rc = launch_rmsnorm(ctx, x_eff, static_cast<const float*>(d->norm_weight->ptr), hn, (int)d->rows, (int)d->ne, d->norm_eps))) return rc;
        x_eff = hn;
        rp.router_x = hn;
        rp.x = hn;
      }
      if ((rc = launch_route(ctx, rp, false))) return rc;
      if ((rc = launch_quantize_rows(ctx, x_eff, s.xq_lo, s.xq_hi, s.xscale, (int)d->rows, (int)d->ne))) return rc;
    } else if (stages & 8u) {
      // routing came from elsewhere (ids_out / wts_out are inputs): only the fixed-point copy of x is made here
      if (d->norm_weight) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_ffn: stages without the router cannot apply norm_weight");
      if ((rc = launch_quantize_rows(ctx, static_cast<const float*>(d->x->ptr), s.xq_lo, s.xq_hi, s.xscale, (int)d->rows, (int)d->ne))) return rc;
    }
    DecodeParams dp = {};
    dp.xq_lo = s.xq_lo;
    dp.xq_hi = s.xq_hi;
    dp.xscale = s.xscale;
    dp.x = static_cast<const float*>(d->x->ptr);
    dp.ids = rp.ids;
    dp.wts = rp.wts;
    dp.sh_logit = (has_sh && d->sh_gate_inp) ? s.sh_logit : nullptr;
    dp.gate = static_cast<const uint8_t*>(d->gate_exps->ptr);
    dp.up = d->fused_gate_up ? dp.gate + (size_t)d->n_ff_exp * row_bytes(d->gate_dtype, d->ne) : static_cast<const uint8_t*>(d->up_exps->ptr);
    dp.down = static_cast<const uint8_t*>(d->down_exps->ptr);
    dp.sh_gate = has_sh ? static_cast<const uint8_t*>(d->sh_gate->ptr) : nullptr;
    dp.sh_up = has_sh ? static_cast<const uint8_t*>(d->sh_up->ptr) : nullptr;
    dp.sh_down = has_sh ? static_cast<const uint8_t*>(d->sh_down->ptr) : nullptr;
    dp.act = s.act;
    dp.dst = static_cast<float*>(d->dst->ptr);
    dp.residual = d->residual ? static_cast<const float*>(d->residual->ptr) : nullptr;
    dp.status = ctx->status;
    dp.trace = ctx->trace;
    dp.gate_stride = (size_t)d->n_ff_exp * row_bytes(d->gate_dtype, d->ne) * (d->fused_gate_up ? 2 : 1);
    dp.up_stride = d->fused_gate_up ? dp.gate_stride : (size_t)d->n_ff_exp * row_bytes(d->up_dtype, d->ne);
    dp.down_stride = (size_t)d->ne * row_bytes(d->down_dtype, d->n_ff_exp);
    dp.rows = d->rows;
    dp.ne = d->ne;
    dp.n_used = d->n_used;
    dp.nff = d->n_ff_exp;
    dp.sh_ff = has_sh ? d->sh_ff : 0;
    dp.n_expert = d->n_expert;
    dp.ep_lo = d->ep_lo;
    dp.ep_n = d->ep_n_local;
    dp.down_q4k = down_q4k ? 1 : 0;
    dp.gate_dt = d->gate_dtype;
    dp.up_dt = d->up_dtype;
    dp.down_dt = d->down_dtype;
    dp.xsum_ready = xsum_ready ? 1 : 0;
    dp.down_scale = d->down_scale ? static_cast<const float*>(d->down_scale->ptr) : nullptr;
    dp.act_kind = (int)d->act;
    dp.weight_before = d->weight_before ? 1 : 0;
    dp.clamp = d->swiglu_clamp;
    if (use_em) return launch_em_ffn(ctx, dp, static_cast<char*>(ctx->scratch) + sz.total + hn_bytes, stages);
    return launch_decode_ffn(ctx, dp, true, stages);
  }
  // batched path: router GEMM + top-k, permute, grouped GEMMs, un-permute combine
  if (d->ne % 64 || d->n_ff_exp % 64) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_ffn: batched path needs ne and n_ff_exp multiples of 64");
  if (has_sh && d->sh_ff != d->n_ff_exp)
    return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_ffn: batched path needs the shared expert as wide as the routed experts");
  if ((uint64_t)d->rows * d->n_used > (1u << 24)) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_ffn: more than 2^24 (token, expert) pairs per call");
  {
    const int n_pairs = (int)(d->rows * d->n_used);
    const int shared_rows = has_sh ? (int)d->rows : 0;
    const int rows_bound = n_pairs + shared_rows;
    Scratch sz = carve(nullptr, d, false);
    const size_t gbytes = grouped_scratch_bytes(rows_bound, n_pairs, (int)d->n_expert + 1, (int)d->ne, (int)d->n_ff_exp);
    const size_t hn_bytes = d->norm_weight ? align_up((size_t)d->rows * d->ne * 4, 256) : 0;
    if ((rc = ensure_scratch(ctx, sz.total + gbytes + hn_bytes))) return rc;
    Scratch s = carve(ctx->scratch, d, false);
    RouteParams rp = route_params(ctx, d, s, true);
    const float* x_eff = static_cast<const float*>(d->x->ptr);
    if (d->norm_weight) {
      // RmsNorm -> MoeFfn: the batched kernels read the normed rows from scratch
      float* hn = reinterpret_cast<float*>(static_cast<char*>(ctx->scratch) + sz.total + gbytes);
      if ((rc = launch_rmsnorm(ctx, x_eff, static_cast<const float*>(d->norm_weight->ptr), hn, (int)d->rows, (int)d->ne, d->norm_eps))) return rc;
      x_eff = hn;
      rp.router_x = hn;
      rp.x = hn;
    }
    const uint32_t stages = d->stages ? d->stages : 7u;
    if ((stages & 1u) && (rc = launch_route(ctx, rp, false))) return rc;
    if (!(stages & 6u)) return INFR_CUDA_OK;
    GroupedCall c = {};
    c.scratch = static_cast<char*>(ctx->scratch) + sz.total;
    c.x = x_eff;
    c.residual = d->residual ? static_cast<const float*>(d->residual->ptr) : nullptr;
    c.ids = rp.ids;
    c.wts = rp.wts;
    c.sh_logit = (has_sh && d->sh_gate_inp) ? s.sh_logit : nullptr;
    c.dst = static_cast<float*>(d->dst->ptr);
    c.gate = static_cast<const uint8_t*>(d->gate_exps->ptr);
    c.up = d->fused_gate_up ? c.gate + (size_t)d->n_ff_exp * row_bytes(d->gate_dtype, d->ne) : static_cast<const uint8_t*>(d->up_exps->ptr);
    c.down = static_cast<const uint8_t*>(d->down_exps->ptr);
    c.sh_gate = has_sh ? static_cast<const uint8_t*>(d->sh_gate->ptr) : nullptr;
    c.sh_up = has_sh ? static_cast<const uint8_t*>(d->sh_up->ptr) : nullptr;
    c.sh_down = has_sh ? static_cast<const uint8_t*>(d->sh_down->ptr) : nullptr;
    c.gate_stride = (size_t)d->n_ff_exp * row_bytes(d->gate_dtype, d->ne) * (d->fused_gate_up ? 2 : 1);
    c.up_stride = d->fused_gate_up ? c.gate_stride : (size_t)d->n_ff_exp * row_bytes(d->up_dtype, d->ne);
    c.down_stride = (size_t)d->ne * row_bytes(d->down_dtype, d->n_ff_exp);
    c.rows = (int)d->rows;
    c.n_used = (int)d->n_used;
    c.n_pairs = n_pairs;
    c.ne = (int)d->ne;
    c.nff = (int)d->n_ff_exp;
    c.n_expert = (int)d->n_expert;
    c.shared_rows = shared_rows;
    c.rows_bound = rows_bound;
    c.ep_lo = d->ep_lo;
    c.ep_n = d->ep_n_local;
    c.legacy = (path == 3) ? 1 : 0;
    c.down_q4k = down_q4k ? 1 : 0;
    c.gate_dt = d->gate_dtype;
    c.up_dt = d->up_dtype;
    c.down_dt = d->down_dtype;
    c.act_kind = (int)d->act;
    c.clamp = d->swiglu_clamp;
    c.weight_before = d->weight_before ? 1 : 0;
    c.down_scale = d->down_scale ? static_cast<const float*>(d->down_scale->ptr) : nullptr;
    return launch_grouped_ffn(ctx, c);
  }
}

// ---- the ops around it --------------------------------------------------------------------------

int32_t infr_cuda_linear(infr_cuda_ctx* ctx, int32_t dtype, const infr_cuda_buf* w, const infr_cuda_buf* x,
                         infr_cuda_buf* y, uint32_t m, uint32_t in_f, uint32_t out_f) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  if (!m || !in_f || !out_f) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "linear: zero dimension");
  if (dtype != INFR_CUDA_DT_F32 && !block_elems(dtype))
    return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "linear: weight dtype not covered (F32 and the block formats an expert bank may have)");
  if (codebook_missing(ctx, dtype))
    return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "linear: the weight is in a grid codebook format whose table has not been set (infr_cuda_set_codebook)");
  if (dtype != INFR_CUDA_DT_F32 && in_f % block_elems(dtype))
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "linear: in_f must be a whole number of weight blocks (32, 64 or 256 weights)");
  const size_t rb = row_bytes(dtype, in_f);
  if (!fits(w, rb * out_f) || !fits(x, (size_t)m * in_f * 4) || !fits(y, (size_t)m * out_f * 4))
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "linear: buffer missing or too small");
  DeviceGuard g(ctx->device);
  return launch_linear(ctx, dtype, static_cast<const uint8_t*>(w->ptr), static_cast<const float*>(x->ptr),
                       static_cast<float*>(y->ptr), (int)m, (int)in_f, (int)out_f);
}

int32_t infr_cuda_gated_act(infr_cuda_ctx* ctx, const infr_cuda_buf* gate, const infr_cuda_buf* up, infr_cuda_buf* dst, size_t n) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  if (!fits(gate, n * 4) || !fits(up, n * 4) || !fits(dst, n * 4)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "gated_act: buffer missing or too small");
  if (!n) return INFR_CUDA_OK;
  DeviceGuard g(ctx->device);
  return launch_gated_act(ctx, static_cast<const float*>(gate->ptr), static_cast<const float*>(up->ptr), static_cast<float*>(dst->ptr), n);
}

int32_t infr_cuda_moe_shared_add(infr_cuda_ctx* ctx, const infr_cuda_buf* moe, const infr_cuda_buf* shexp,
                                 const infr_cuda_buf* gate, infr_cuda_buf* dst, uint32_t rows, uint32_t n) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  const size_t b = (size_t)rows * n * 4;
  if (!rows || !n) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_shared_add: zero dimension");
  if (!fits(moe, b) || !fits(shexp, b) || !fits(dst, b) || !fits(gate, (size_t)rows * 4))
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_shared_add: buffer missing or too small");
  DeviceGuard g(ctx->device);
  return launch_shared_add(ctx, static_cast<const float*>(moe->ptr), static_cast<const float*>(shexp->ptr),
                           static_cast<const float*>(gate->ptr), static_cast<float*>(dst->ptr), (int)rows, (int)n);
}

int32_t infr_cuda_rmsnorm(infr_cuda_ctx* ctx, const infr_cuda_buf* x, const infr_cuda_buf* weight, infr_cuda_buf* dst,
                          uint32_t rows, uint32_t dim, float eps) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  if (!rows || !dim) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "rmsnorm: zero dimension");
  const size_t b = (size_t)rows * dim * 4;
  if (!fits(x, b) || !fits(dst, b) || !fits(weight, (size_t)dim * 4)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "rmsnorm: buffer missing or too small");
  DeviceGuard g(ctx->device);
  return launch_rmsnorm(ctx, static_cast<const float*>(x->ptr), static_cast<const float*>(weight->ptr),
                        static_cast<float*>(dst->ptr), (int)rows, (int)dim, eps);
}

int32_t infr_cuda_add(infr_cuda_ctx* ctx, const infr_cuda_buf* a, const infr_cuda_buf* b, infr_cuda_buf* dst, size_t n) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  if (!fits(a, n * 4) || !fits(b, n * 4) || !fits(dst, n * 4)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "add: buffer missing or too small");
  if (!n) return INFR_CUDA_OK;
  DeviceGuard g(ctx->device);
  return launch_add(ctx, static_cast<const float*>(a->ptr), static_cast<const float*>(b->ptr), static_cast<float*>(dst->ptr), n);
}

int32_t infr_cuda_moe_expert_rows(infr_cuda_ctx* ctx, const infr_cuda_buf* x_rows, const infr_cuda_buf* seg_off,
                                  const infr_cuda_buf* gate_exps, const infr_cuda_buf* up_exps, const infr_cuda_buf* down_exps,
                                  infr_cuda_buf* y_rows, uint32_t n_rows, uint32_t n_local, uint32_t ne, uint32_t n_ff_exp,
                                  int32_t gate_dtype, int32_t up_dtype, int32_t down_dtype) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  if (!n_local || !ne || !n_ff_exp) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_expert_rows: zero dimension");
  if (n_local > 1024) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_expert_rows: more than 1024 local experts");
  if (!bank_dtype_ok(gate_dtype) || !bank_dtype_ok(up_dtype) || !bank_dtype_ok(down_dtype))
    return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_expert_rows: expert banks must be one of Q4_0 Q4_1 Q5_0 Q5_1 Q8_0 Q2_K Q3_K Q4_K Q5_K Q6_K IQ4_NL IQ4_XS MXFP4 NVFP4 Q2_0 IQ2_XS IQ2_S IQ3_XXS IQ3_S");
  if (ne % 256 || n_ff_exp % 256) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_expert_rows: ne and n_ff_exp must be multiples of 256");
  if (!n_rows) return INFR_CUDA_OK;
  if (codebook_missing(ctx, gate_dtype) || codebook_missing(ctx, up_dtype) || codebook_missing(ctx, down_dtype))
    return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_expert_rows: a bank is in a grid codebook format whose table has not been set (infr_cuda_set_codebook)");
  const size_t gb = (size_t)n_local * n_ff_exp * row_bytes(gate_dtype, ne), ub = (size_t)n_local * n_ff_exp * row_bytes(up_dtype, ne),
               db = (size_t)n_local * ne * row_bytes(down_dtype, n_ff_exp);
  if (!fits(x_rows, (size_t)n_rows * ne * 4) || !fits(y_rows, (size_t)n_rows * ne * 4) || !fits(seg_off, (size_t)(n_local + 1) * 4) ||
      !fits(gate_exps, gb) || !fits(up_exps, ub) || !fits(down_exps, db))
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_expert_rows: buffer missing or too small");
  DeviceGuard g(ctx->device);
  const size_t gbytes = grouped_scratch_bytes((int)n_rows, 1, (int)n_local + 1, (int)ne, (int)n_ff_exp);
  int32_t rc = ensure_scratch(ctx, gbytes);
  if (rc) return rc;
  GroupedCall c = {};
  c.scratch = ctx->scratch;
  c.x = static_cast<const float*>(x_rows->ptr);
  c.seg_off_in = static_cast<const int*>(seg_off->ptr);
  c.y_out = static_cast<float*>(y_rows->ptr);
  c.gate = static_cast<const uint8_t*>(gate_exps->ptr);
  c.up = static_cast<const uint8_t*>(up_exps->ptr);
  c.down = static_cast<const uint8_t*>(down_exps->ptr);
  c.gate_stride = (size_t)n_ff_exp * row_bytes(gate_dtype, ne);
  c.up_stride = (size_t)n_ff_exp * row_bytes(up_dtype, ne);
  c.down_stride = (size_t)ne * row_bytes(down_dtype, n_ff_exp);
  c.gate_dt = gate_dtype;
  c.up_dt = up_dtype;
  c.down_dt = down_dtype;
  c.rows = (int)n_rows;
  c.n_used = 1;
  c.n_pairs = 1;
  c.ne = (int)ne;
  c.nff = (int)n_ff_exp;
  c.n_expert = (int)n_local;
  c.rows_bound = (int)n_rows;
  c.down_q4k = down_dtype == INFR_CUDA_DT_Q4K ? 1 : 0;
  return launch_grouped_ffn(ctx, c);
}

int32_t infr_cuda_moe_combine(infr_cuda_ctx* ctx, const infr_cuda_buf* y_rows, const infr_cuda_buf* pos_of_pair,
                              const infr_cuda_buf* wts, const infr_cuda_buf* sh_rows, const infr_cuda_buf* sh_logit,
                              infr_cuda_buf* dst, uint32_t rows, uint32_t n_used, uint32_t ne, uint32_t n_y_rows) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  if (!rows || !n_used || !ne || ne % 4) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_combine: bad dimensions");
  if (rows > 65535) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "moe_combine: more than 65535 rows per call");
  if (!fits(y_rows, (size_t)n_y_rows * ne * 4) || !fits(pos_of_pair, (size_t)rows * n_used * 4) ||
      !fits(wts, (size_t)rows * n_used * 4) || !fits(dst, (size_t)rows * ne * 4))
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_combine: buffer missing or too small");
  if (sh_rows && !fits(sh_rows, (size_t)rows * ne * 4)) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_combine: sh_rows too small");
  if (sh_logit && (!sh_rows || !fits(sh_logit, (size_t)rows * 4))) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "moe_combine: sh_logit needs sh_rows");
  DeviceGuard g(ctx->device);
  return launch_combine(ctx, static_cast<const float*>(y_rows->ptr), static_cast<const int*>(pos_of_pair->ptr),
                        static_cast<const float*>(wts->ptr), sh_logit ? static_cast<const float*>(sh_logit->ptr) : nullptr,
                        sh_rows ? static_cast<const float*>(sh_rows->ptr) : nullptr, (int)rows, (int)n_used, (int)ne,
                        static_cast<float*>(dst->ptr));
}

int32_t infr_cuda_umma_selftest(infr_cuda_ctx* ctx, const infr_cuda_buf* a, const infr_cuda_buf* b, infr_cuda_buf* c, uint32_t n) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  if (n < 16 || n > 256 || n % 16) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "umma_selftest: n must be a multiple of 16 in [16, 256]");
  if (!fits(a, 128 * 64 * 2) || !fits(b, (size_t)n * 64 * 2) || !fits(c, (size_t)128 * n * 4))
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "umma_selftest: buffer missing or too small");
  DeviceGuard g(ctx->device);
  return launch_umma_selftest(ctx, static_cast<const __half*>(a->ptr), static_cast<const __half*>(b->ptr),
                              static_cast<float*>(c->ptr), (int)n);
}

}  // extern "C"
