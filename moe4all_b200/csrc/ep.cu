// Expert parallelism inside the library: contiguous expert bands per rank, tokens sharded over the
// ranks, dispatch and combine over NCCL (NVLink / NVSwitch).
//
// Reference behaviour: crates/infr-vulkan/src/ep.rs - band rule :12-14, 171-176 (n_expert must be a
// multiple of the world size; rank r owns [r*E/W, (r+1)*E/W)), per-segment execution on every rank
// followed by one reduction of the band partials in fixed rank order (:454-493).  The reference keeps
// the tokens replicated and moves partial outputs; here every rank also owns a slice of the tokens,
// so a MoE layer is:  route own rows -> rows, ids and weights to the other ranks -> the band's experts
// over every row received -> partial sums back to the home ranks -> sum over ranks in rank order ->
// shared expert and residual.
//
// The dispatch uses fixed-capacity slots: a rank's `rows` rows go to every rank, which serves the
// pairs inside its own band and ignores the others.  Through NVSwitch every peer is reached at full
// link bandwidth, so the dense form costs one rank-count-independent transfer time, needs no count
// exchange and never brings a size back to the host: the whole call is queued without a host
// synchronisation.  NCCL is loaded at run time, so the library itself has no link dependency on it.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <future>
#include <memory>
#include <new>
#include <set>
#include <thread>
#include <tuple>

#include "kernels.cuh"

namespace infr {

namespace {

struct NcclApi {
  void* handle = nullptr;
  decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
  decltype(&ncclCommInitRank) CommInitRank = nullptr;
  decltype(&ncclCommDestroy) CommDestroy = nullptr;
  decltype(&ncclCommAbort) CommAbort = nullptr;
  decltype(&ncclGetErrorString) GetErrorString = nullptr;
  decltype(&ncclGroupStart) GroupStart = nullptr;
  decltype(&ncclGroupEnd) GroupEnd = nullptr;
  decltype(&ncclSend) Send = nullptr;
  decltype(&ncclRecv) Recv = nullptr;
  decltype(&ncclAllGather) AllGather = nullptr;
};

// The process-wide binding; null when libnccl.so.2 cannot be loaded.  A process that already
// holds NCCL (PyTorch brings its own copy) gets that copy: the loader matches the soname.
NcclApi* nccl_api() {
  static NcclApi api;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (h) {
      api.handle = h;
#define BIND(name) api.name = reinterpret_cast<decltype(api.name)>(dlsym(h, "nccl" #name))
      BIND(GetUniqueId); BIND(CommInitRank); BIND(CommDestroy); BIND(CommAbort); BIND(GetErrorString);
      BIND(GroupStart); BIND(GroupEnd); BIND(Send); BIND(Recv); BIND(AllGather);
#undef BIND
      if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.CommAbort || !api.GetErrorString || !api.GroupStart ||
          !api.GroupEnd || !api.Send || !api.Recv || !api.AllGather)
        api.handle = nullptr;
    }
  }
  return api.handle ? &api : nullptr;
}

constexpr int EP_PHASES = 6;  // call start, routed, dispatched, band done, partials back, result written

}  // namespace

struct EpState {
  NcclApi* api = nullptr;
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  bool dead = false;             // the communicator was aborted: local calls only from now on
  cudaStream_t side = nullptr;   // the shared expert runs here while the exchanges are in flight
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  cudaStream_t xfer = nullptr;   // the token rows' all-gather runs here while the router works on the main stream
  cudaEvent_t ev_x = nullptr, ev_xg = nullptr;
  cudaEvent_t ev_phase[EP_PHASES] = {};
  bool phases_valid = false;
  void* buf = nullptr;           // exchange buffers, grown on demand (never while recording)
  size_t buf_bytes = 0;
  int32_t* shape_dev = nullptr;  // [world][8] shapes of all ranks (the first call with a new shape compares them)
  std::set<std::tuple<uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t>> checked;
};

namespace {

int32_t ep_fail(infr_cuda_ctx* ctx, const char* what, ncclResult_t r) {
  EpState* ep = ctx->ep;
  std::string msg = std::string("expert parallel: ") + what + ": " + (ep && ep->api ? ep->api->GetErrorString(r) : "NCCL error");
  if (ep && ep->comm && !ep->dead) {
    ep->api->CommAbort(ep->comm);  // peers blocked in a collective with this rank fail instead of waiting
    ep->comm = nullptr;
    ep->dead = true;
    msg += " (communicator aborted)";
  }
  return fail(ctx, INFR_CUDA_ERR_NCCL, msg);
}

#define NCCL_TRY(call, what)                       \
  do {                                             \
    const ncclResult_t r_ = (call);                \
    if (r_ != ncclSuccess) return ep_fail(ctx, what, r_); \
  } while (0)

int32_t ep_ensure_buf(infr_cuda_ctx* ctx, size_t bytes) {
  EpState* ep = ctx->ep;
  if (bytes <= ep->buf_bytes) return INFR_CUDA_OK;
  if (ctx->capturing)
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "expert parallel: buffers would have to grow while recording: run the call once un-recorded first");
  int32_t rc = ep_wait_stream(ctx, "expert parallel: buffer grow");
  if (rc) return rc;
  cudaStreamSynchronize(ep->side);
  cudaStreamSynchronize(ep->xfer);
  if (ep->buf) cudaFree(ep->buf);
  ep->buf = nullptr;
  ep->buf_bytes = 0;
  const size_t want = align_up(bytes + bytes / 8, 1 << 20);
  const cudaError_t e = cudaMalloc(&ep->buf, want);
  if (e != cudaSuccess) return check_cuda(ctx, e, "expert parallel: cudaMalloc");
  ep->buf_bytes = want;
  return INFR_CUDA_OK;
}

// ids of the band become bank-local, every other id negative ("not this rank's pair").
__global__ void k_ep_localize(const int32_t* __restrict__ ids, int32_t* __restrict__ local, int n, int lo, int n_local, int n_expert,
                              DeviceStatus* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = ids[i];
  if (e >= n_expert) status->bad_index = 1;  // an id no rank owns (ids supplied by a caller)
  const int l = e - lo;
  local[i] = (e >= 0 && l >= 0 && l < n_local) ? l : -1;
}

// dst[t, :] = sum over ranks p (in rank order) of back[p][t, :], then the shared expert's row
// (sigmoid-gated when a gate logit is given) and the residual.  The order is the reference's
// reduction order (crates/infr-vulkan/src/ep.rs:483-490: fixed rank order, f32).
__global__ void __launch_bounds__(256) k_ep_finish(const float* __restrict__ back, int world, int rows, int ne,
                                                   const float* __restrict__ sh_rows, const float* __restrict__ sh_logit,
                                                   const float* residual, float* dst) {
  const int c = (blockIdx.x * 256 + threadIdx.x) * 4;
  if (c >= ne) return;
  for (int t = blockIdx.y; t < rows; t += gridDim.y) {
    float4 o = *reinterpret_cast<const float4*>(back + (size_t)t * ne + c);
    for (int p = 1; p < world; ++p) {
      const float4 v = *reinterpret_cast<const float4*>(back + ((size_t)p * rows + t) * ne + c);
      o.x += v.x; o.y += v.y; o.z += v.z; o.w += v.w;
    }
    if (sh_rows != nullptr) {
      const float g = sh_logit ? 1.0f / (1.0f + __expf(-sh_logit[t])) : 1.0f;
      const float4 v = *reinterpret_cast<const float4*>(sh_rows + (size_t)t * ne + c);
      o.x += g * v.x; o.y += g * v.y; o.z += g * v.z; o.w += g * v.w;
    }
    if (residual != nullptr) {  // may alias dst: each element is read, then written, by this thread
      const float4 h = *reinterpret_cast<const float4*>(residual + (size_t)t * ne + c);
      o.x += h.x; o.y += h.y; o.z += h.z; o.w += h.w;
    }
    *reinterpret_cast<float4*>(dst + (size_t)t * ne + c) = o;
  }
}

__global__ void k_ep_set_pair(int* dst, int a, int b) {
  dst[0] = a;
  dst[1] = b;
}

infr_cuda_buf view(void* p, size_t bytes) {
  infr_cuda_buf b;
  b.ptr = p;
  b.bytes = bytes;
  b.owned = false;
  return b;
}

void phase(infr_cuda_ctx* ctx, int i) {
  if (!ctx->capturing) cudaEventRecord(ctx->ep->ev_phase[i], ctx->stream);
}

}  // namespace

bool ep_call_is_collective(const infr_cuda_ctx* ctx, const infr_cuda_moe_ffn_desc* d) {
  const EpState* ep = ctx->ep;
  if (!ep || ep->world <= 1 || d->ep_n_local == 0 || d->n_expert % (uint32_t)ep->world) return false;
  const uint32_t n_local = d->n_expert / (uint32_t)ep->world;
  return d->ep_n_local == n_local && d->ep_lo == (uint32_t)ep->rank * n_local;
}

int32_t ep_wait_stream(infr_cuda_ctx* ctx, const char* what) {
  EpState* ep = ctx->ep;
  const auto t0 = std::chrono::steady_clock::now();
  const auto limit = std::chrono::milliseconds(ctx->cfg.sync_timeout_ms ? ctx->cfg.sync_timeout_ms : 60000u);
  for (uint64_t n = 0;; ++n) {
    const cudaError_t e = cudaStreamQuery(ctx->stream);
    if (e == cudaSuccess) return INFR_CUDA_OK;
    if (e != cudaErrorNotReady) return check_cuda(ctx, e, what);
    if (n > 2000) std::this_thread::sleep_for(std::chrono::microseconds(50));  // short waits are polled hot
    if ((n & 63) == 0 && std::chrono::steady_clock::now() - t0 > limit) {
      if (ep && ep->comm && !ep->dead) {
        ep->api->CommAbort(ep->comm);  // ends the collective kernels this rank still has in flight
        ep->comm = nullptr;
        ep->dead = true;
        cudaStreamSynchronize(ctx->stream);
        return fail(ctx, INFR_CUDA_ERR_NCCL, std::string(what) + ": the stream did not drain within the limit (a peer never joined a collective?); communicator aborted");
      }
      return fail(ctx, INFR_CUDA_ERR_TIMEOUT, std::string(what) + ": the stream did not drain within the limit");
    }
  }
}

void ep_release(infr_cuda_ctx* ctx, bool orderly) {
  EpState* ep = ctx->ep;
  if (!ep) return;
  if (ep->comm) {
    if (orderly && !ep->dead) {
      cudaStreamSynchronize(ctx->stream);
      ep->api->CommDestroy(ep->comm);
    } else {
      ep->api->CommAbort(ep->comm);
    }
  }
  if (ep->side) {
    cudaStreamSynchronize(ep->side);
    cudaStreamDestroy(ep->side);
  }
  if (ep->xfer) {
    cudaStreamSynchronize(ep->xfer);
    cudaStreamDestroy(ep->xfer);
  }
  if (ep->ev_fork) cudaEventDestroy(ep->ev_fork);
  if (ep->ev_join) cudaEventDestroy(ep->ev_join);
  if (ep->ev_x) cudaEventDestroy(ep->ev_x);
  if (ep->ev_xg) cudaEventDestroy(ep->ev_xg);
  for (cudaEvent_t e : ep->ev_phase)
    if (e) cudaEventDestroy(e);
  if (ep->buf) cudaFree(ep->buf);
  if (ep->shape_dev) cudaFree(ep->shape_dev);
  delete ep;
  ctx->ep = nullptr;
}

// The first call with a new shape: every rank's shape travels to every rank and is compared on the
// host, before any data-sized exchange is queued.  A rank that disagrees fails on all ranks alike,
// with nothing left in flight.
static int32_t ep_check_shape(infr_cuda_ctx* ctx, const infr_cuda_moe_ffn_desc* d) {
  EpState* ep = ctx->ep;
  const auto key = std::make_tuple(d->rows, d->ne, d->n_expert, d->n_used, d->n_ff_exp, d->sh_gate ? d->sh_ff : 0u);
  if (ep->checked.count(key)) return INFR_CUDA_OK;
  if (ctx->capturing)
    return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "expert parallel: the first call of a shape cannot be recorded: run it once un-recorded first");
  const int W = ep->world;
  int32_t mine[8] = {(int32_t)d->rows, (int32_t)d->ne, (int32_t)d->n_expert, (int32_t)d->n_used, (int32_t)d->n_ff_exp,
                     (int32_t)(d->sh_gate ? d->sh_ff : 0u), (int32_t)d->gate_dtype * 65536 + (int32_t)d->up_dtype * 256 + (int32_t)d->down_dtype, W};
  cudaError_t e = cudaMemcpyAsync(ep->shape_dev + (size_t)ep->rank * 8, mine, sizeof mine, cudaMemcpyHostToDevice, ctx->stream);
  if (e != cudaSuccess) return check_cuda(ctx, e, "expert parallel: shape upload");
  NCCL_TRY(ep->api->AllGather(ep->shape_dev + (size_t)ep->rank * 8, ep->shape_dev, 8, ncclInt32, ep->comm, ctx->stream), "shape exchange");
  int32_t rc = ep_wait_stream(ctx, "expert parallel: shape exchange");
  if (rc) return rc;
  std::vector<int32_t> all((size_t)W * 8);
  e = cudaMemcpy(all.data(), ep->shape_dev, all.size() * 4, cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return check_cuda(ctx, e, "expert parallel: shape download");
  for (int p = 0; p < W; ++p)
    for (int i = 0; i < 8; ++i)
      if (all[(size_t)p * 8 + i] != mine[i]) {
        char msg[200];
        std::snprintf(msg, sizeof msg,
                      "expert parallel: rank %d passed a different shape than rank %d (field %d: %d vs %d); every rank must make the same call",
                      p, ep->rank, i, all[(size_t)p * 8 + i], mine[i]);
        return fail(ctx, INFR_CUDA_ERR_NCCL, msg);
      }
  ep->checked.insert(key);
  return INFR_CUDA_OK;
}

int32_t ep_moe_ffn(infr_cuda_ctx* ctx, const infr_cuda_moe_ffn_desc* d) {
  EpState* ep = ctx->ep;
  if (ep->dead) return fail(ctx, INFR_CUDA_ERR_NCCL, "expert parallel: the communicator was aborted by an earlier failure");
  const uint32_t W = (uint32_t)ep->world, R = d->rows, E = d->n_expert, El = E / W, k = d->n_used, ne = d->ne;
  int32_t rc = validate_moe_ffn(ctx, d, El);
  if (rc) return rc;
  if (d->stages != 0) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "expert parallel: the call runs whole (stages must be 0)");
  if (d->expert_ids) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "expert parallel: caller-selected experts are not covered");
  if ((uint64_t)R * W > (1u << 21)) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "expert parallel: more than 2^21 token rows over all ranks");
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != ctx->device) cudaSetDevice(ctx->device);
  struct Restore {
    int prev, dev;
    ~Restore() { if (prev >= 0 && prev != dev) cudaSetDevice(prev); }
  } restore{prev, ctx->device};
  if ((rc = ep_check_shape(ctx, d))) return rc;

  const bool has_sh = d->sh_gate != nullptr;
  const size_t T = (size_t)R * W;
  const size_t row_b = (size_t)ne * 4, x_local_b = R * row_b, x_all_b = T * row_b, kk_local_b = (size_t)R * k * 4, kk_all_b = T * k * 4;
  // carve the exchange buffers
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t o = off;
    off += align_up(bytes, 256);
    return o;
  };
  const size_t o_hn = d->norm_weight ? take(x_local_b) : 0;
  const size_t o_ids = take(kk_local_b), o_wts = take(kk_local_b);
  const size_t o_x_all = take(x_all_b), o_ids_all = take(kk_all_b), o_wts_all = take(kk_all_b), o_loc_all = take(kk_all_b);
  const size_t o_part = take(x_all_b), o_back = take(x_all_b);
  const size_t o_sh_rows = has_sh ? take(x_local_b) : 0, o_sh_logit = has_sh ? take((size_t)R * 4) : 0, o_seg = take(256);
  // The shared expert over this rank's own rows: a few rows go through the small-m kernels (a call with no
  // routed pair: every id negative), a batch through the grouped GEMMs.  Either runs on the side stream with
  // scratch of its own, next to the exchange buffers.
  // the kernels are chosen for what the band serves - about a W-th of the T rows' pairs over n_expert / W
  // experts, i.e. R rows over El experts - not for all T rows; the shared expert goes the same way
  uint32_t band_path = d->path ? d->path : choose_moe_path(ctx, R, k, El, ne, d->n_ff_exp, 0, BankTypes{d->gate_dtype, d->up_dtype, d->down_dtype});
  if (band_path == 1 && T > 4096) band_path = 2;  // the small-m kernels' grids and scratch grow with all T rows
  const bool sh_small = has_sh && band_path == 1;
  infr_cuda_moe_ffn_desc shd = *d;  // the nested small-m call (filled in below)
  shd.rows = R;
  shd.n_expert = El;
  shd.stages = 2u | 4u | 8u;
  const size_t sh_scratch_b = !has_sh ? 0 : (sh_small ? small_path_scratch_need(&shd) : grouped_scratch_bytes((int)R, 1, 2, (int)ne, (int)d->sh_ff));
  const size_t o_sh_scratch = take(sh_scratch_b), o_neg = sh_small ? take(kk_local_b) : 0;
  if ((rc = ep_ensure_buf(ctx, off))) return rc;
  char* B = static_cast<char*>(ep->buf);
  cudaStream_t main = ctx->stream;
  phase(ctx, 0);

  // x as the experts and the router see it
  const float* x_eff = static_cast<const float*>(d->x->ptr);
  const float* rx_eff = static_cast<const float*>(d->router_x->ptr);
  if (d->norm_weight) {
    float* hn = reinterpret_cast<float*>(B + o_hn);
    if ((rc = launch_rmsnorm(ctx, x_eff, static_cast<const float*>(d->norm_weight->ptr), hn, (int)R, (int)ne, d->norm_eps))) return rc;
    x_eff = rx_eff = hn;
  }
  infr_cuda_buf b_x = view(const_cast<float*>(x_eff), x_local_b), b_rx = view(const_cast<float*>(rx_eff), x_local_b);

  // dispatch, first half: the rows of every rank to every rank (slot p of the receive array = rank p's rows).
  // Nothing of the routing goes into them, so their all-gather - the bulk of the dispatch - runs on a stream of
  // its own beside the router; the main stream joins it before the band's experts start.
  {
    cudaError_t e = cudaEventRecord(ep->ev_x, main);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(ep->xfer, ep->ev_x, 0);
    if (e != cudaSuccess) return check_cuda(ctx, e, "expert parallel: rows fork");
    NCCL_TRY(ep->api->AllGather(x_eff, B + o_x_all, (size_t)R * ne, ncclFloat32, ep->comm, ep->xfer), "dispatch (rows)");
    e = cudaEventRecord(ep->ev_xg, ep->xfer);
    if (e != cudaSuccess) return check_cuda(ctx, e, "expert parallel: rows record");
  }

  // the shared expert needs nothing from the other ranks: side stream, joined before the final sum
  if (has_sh) {
    cudaError_t e = cudaEventRecord(ep->ev_fork, main);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(ep->side, ep->ev_fork, 0);
    if (e != cudaSuccess) return check_cuda(ctx, e, "expert parallel: fork");
    ctx->stream = ep->side;
    if (sh_small) {
      e = cudaMemsetAsync(B + o_neg, 0xFF, kk_local_b, ep->side);  // every (token, rank) pair "not this call's"
      infr_cuda_buf b_neg = view(B + o_neg, kk_local_b), b_w = view(B + o_wts, kk_local_b), b_sh = view(B + o_sh_rows, x_local_b);
      shd.x = &b_x;
      shd.router_x = &b_x;
      shd.dst = &b_sh;
      shd.ids_out = &b_neg;
      shd.wts_out = &b_w;  // never used: no pair is served
      shd.ep_lo = shd.ep_n_local = 0;
      shd.exp_probs_b = nullptr;
      shd.expert_ids = nullptr;
      shd.down_scale = nullptr;
      shd.n_expert_groups = shd.n_expert_groups_used = 0;
      shd.sh_gate_inp = nullptr;  // the plain sum 0 + shexp(x); the gate is applied with the final sum
      shd.norm_weight = nullptr;
      shd.residual = nullptr;
      shd.path = 1;
      void* keep_s = ctx->scratch;
      const size_t keep_b = ctx->scratch_bytes;
      ctx->scratch = B + o_sh_scratch;
      ctx->scratch_bytes = sh_scratch_b;
      ctx->scratch_borrowed = true;
      rc = e == cudaSuccess ? infr_cuda_moe_ffn(ctx, &shd) : check_cuda(ctx, e, "expert parallel: shared expert set-up");
      ctx->scratch = keep_s;
      ctx->scratch_bytes = keep_b;
      ctx->scratch_borrowed = false;
    } else {
      k_ep_set_pair<<<1, 1, 0, ep->side>>>(reinterpret_cast<int*>(B + o_seg), 0, (int)R);  // segment offsets of the one "expert"
      ctx->launches += 1;
      GroupedCall c = {};
      c.scratch = B + o_sh_scratch;
      c.x = x_eff;
      c.seg_off_in = reinterpret_cast<const int*>(B + o_seg);
      c.y_out = reinterpret_cast<float*>(B + o_sh_rows);
      c.gate = static_cast<const uint8_t*>(d->sh_gate->ptr);
      c.up = static_cast<const uint8_t*>(d->sh_up->ptr);
      c.down = static_cast<const uint8_t*>(d->sh_down->ptr);
      c.gate_stride = (size_t)d->sh_ff * row_bytes(d->gate_dtype, ne);
      c.up_stride = (size_t)d->sh_ff * row_bytes(d->up_dtype, ne);
      c.down_stride = (size_t)ne * row_bytes(d->down_dtype, d->sh_ff);
      c.rows = (int)R;
      c.n_used = 1;
      c.n_pairs = 1;
      c.ne = (int)ne;
      c.nff = (int)d->sh_ff;
      c.n_expert = 1;
      c.rows_bound = (int)R;
      c.down_q4k = d->down_dtype == INFR_CUDA_DT_Q4K ? 1 : 0;
      c.gate_dt = d->gate_dtype;
      c.up_dt = d->up_dtype;
      c.down_dt = d->down_dtype;
      c.act_kind = (int)d->act;
      rc = launch_grouped_ffn(ctx, c);
    }
    if (rc == INFR_CUDA_OK && d->sh_gate_inp)
      rc = launch_linear(ctx, INFR_CUDA_DT_F32, static_cast<const uint8_t*>(d->sh_gate_inp->ptr), x_eff,
                         reinterpret_cast<float*>(B + o_sh_logit), (int)R, (int)ne, 1);
    ctx->stream = main;
    if (rc == INFR_CUDA_OK) rc = check_cuda(ctx, cudaEventRecord(ep->ev_join, ep->side), "expert parallel: join record");
    if (rc) return rc;
  }

  // routing of this rank's rows with the full router
  infr_cuda_buf b_ids = view(d->ids_out ? d->ids_out->ptr : B + o_ids, kk_local_b);
  infr_cuda_buf b_wts = view(d->wts_out ? d->wts_out->ptr : B + o_wts, kk_local_b);
  {
    infr_cuda_moe_ffn_desc r = *d;
    r.x = &b_x;
    r.router_x = &b_rx;
    r.ids_out = &b_ids;
    r.wts_out = &b_wts;
    r.ep_lo = r.ep_n_local = 0;
    r.norm_weight = nullptr;
    r.residual = nullptr;
    r.sh_gate = r.sh_up = r.sh_down = r.sh_gate_inp = nullptr;
    r.sh_ff = 0;
    if ((rc = infr_cuda_moe_route(ctx, &r))) return rc;
  }
  phase(ctx, 1);

  // dispatch, second half: the rows' arrival first - two collectives of one communicator are never in flight
  // together (on different streams they would share its channels) -, then ids and weights of every rank to
  // every rank
  {
    const cudaError_t e = cudaStreamWaitEvent(main, ep->ev_xg, 0);
    if (e != cudaSuccess) return check_cuda(ctx, e, "expert parallel: rows join");
  }
  NCCL_TRY(ep->api->GroupStart(), "dispatch");
  ncclResult_t r2 = ep->api->AllGather(b_ids.ptr, B + o_ids_all, (size_t)R * k, ncclInt32, ep->comm, main);
  ncclResult_t r3 = ep->api->AllGather(b_wts.ptr, B + o_wts_all, (size_t)R * k, ncclFloat32, ep->comm, main);
  ncclResult_t r4 = ep->api->GroupEnd();
  for (ncclResult_t r : {r2, r3, r4})
    if (r != ncclSuccess) return ep_fail(ctx, "dispatch", r);
  phase(ctx, 2);

  // this rank's band over everything it received
  {
    const int n = (int)(T * k);
    k_ep_localize<<<(n + 255) / 256, 256, 0, main>>>(reinterpret_cast<const int32_t*>(B + o_ids_all), reinterpret_cast<int32_t*>(B + o_loc_all), n,
                                                    (int)d->ep_lo, (int)El, (int)E, ctx->status);
    ctx->launches += 1;
    infr_cuda_buf b_xa = view(B + o_x_all, x_all_b), b_loc = view(B + o_loc_all, kk_all_b), b_wa = view(B + o_wts_all, kk_all_b),
                  b_part = view(B + o_part, x_all_b);
    infr_cuda_buf b_ds = d->down_scale ? view(static_cast<char*>(d->down_scale->ptr) + (size_t)d->ep_lo * 4, (size_t)El * 4) : infr_cuda_buf();
    infr_cuda_moe_ffn_desc f = *d;
    f.x = &b_xa;
    f.router_x = &b_xa;
    f.dst = &b_part;
    f.ids_out = &b_loc;
    f.wts_out = &b_wa;
    f.rows = (uint32_t)T;
    f.n_expert = El;
    f.ep_lo = f.ep_n_local = 0;
    f.exp_probs_b = nullptr;
    f.n_expert_groups = f.n_expert_groups_used = 0;
    f.sh_gate = f.sh_up = f.sh_down = f.sh_gate_inp = nullptr;
    f.sh_ff = 0;
    f.norm_weight = nullptr;
    f.residual = nullptr;
    f.down_scale = d->down_scale ? &b_ds : nullptr;
    f.stages = 2u | 4u | 8u;  // routing is an input
    f.path = band_path;
    if ((rc = infr_cuda_moe_ffn(ctx, &f))) return rc;
  }
  phase(ctx, 3);

  // combine: slot p of the partial array goes home to rank p; slot p of `back` = rank p's partial for our rows
  NCCL_TRY(ep->api->GroupStart(), "combine");
  ncclResult_t worst = ncclSuccess;
  for (uint32_t p = 0; p < W; ++p) {
    ncclResult_t a = ep->api->Send(B + o_part + (size_t)p * x_local_b, (size_t)R * ne, ncclFloat32, (int)p, ep->comm, main);
    ncclResult_t b = ep->api->Recv(B + o_back + (size_t)p * x_local_b, (size_t)R * ne, ncclFloat32, (int)p, ep->comm, main);
    if (a != ncclSuccess) worst = a;
    if (b != ncclSuccess) worst = b;
  }
  const ncclResult_t ge = ep->api->GroupEnd();
  if (worst != ncclSuccess || ge != ncclSuccess) return ep_fail(ctx, "combine", worst != ncclSuccess ? worst : ge);
  phase(ctx, 4);

  if (has_sh) {
    const cudaError_t e = cudaStreamWaitEvent(main, ep->ev_join, 0);
    if (e != cudaSuccess) return check_cuda(ctx, e, "expert parallel: join");
  }
  k_ep_finish<<<dim3((ne / 4 + 255) / 256, std::min<uint32_t>(R, 65535u)), 256, 0, main>>>(
      reinterpret_cast<const float*>(B + o_back), (int)W, (int)R, (int)ne, has_sh ? reinterpret_cast<const float*>(B + o_sh_rows) : nullptr,
      (has_sh && d->sh_gate_inp) ? reinterpret_cast<const float*>(B + o_sh_logit) : nullptr,
      d->residual ? static_cast<const float*>(d->residual->ptr) : nullptr, static_cast<float*>(d->dst->ptr));
  ctx->launches += 1;
  phase(ctx, 5);
  ep->phases_valid = !ctx->capturing;
  return check_cuda(ctx, cudaGetLastError(), "expert parallel: finish launch");
}

}  // namespace infr

using namespace infr;

extern "C" {

int32_t infr_cuda_ep_unique_id(uint8_t id[INFR_CUDA_EP_ID_BYTES]) {
  if (!id) return INFR_CUDA_ERR_INVALID_ARG;
  NcclApi* api = nccl_api();
  if (!api) return INFR_CUDA_ERR_UNSUPPORTED;
  ncclUniqueId u;
  static_assert(sizeof(u) == INFR_CUDA_EP_ID_BYTES, "ncclUniqueId size");
  if (api->GetUniqueId(&u) != ncclSuccess) return INFR_CUDA_ERR_NCCL;
  std::memcpy(id, &u, sizeof u);
  return INFR_CUDA_OK;
}

int32_t infr_cuda_ep_init(infr_cuda_ctx* ctx, const uint8_t id[INFR_CUDA_EP_ID_BYTES], int32_t rank, int32_t world) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  if (!id || world < 1 || rank < 0 || rank >= world) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "ep_init: bad rank / world / id");
  if (ctx->ep) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "ep_init: the context already belongs to a communicator");
  if (ctx->capturing) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "ep_init: not while recording");
  NcclApi* api = nccl_api();
  if (!api) return fail(ctx, INFR_CUDA_ERR_UNSUPPORTED, "ep_init: libnccl.so.2 could not be loaded");
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != ctx->device) cudaSetDevice(ctx->device);
  EpState* ep = new (std::nothrow) EpState();
  if (!ep) return fail(ctx, INFR_CUDA_ERR_OOM, "ep_init: host out of memory");
  ep->api = api;
  ep->rank = rank;
  ep->world = world;
  ctx->ep = ep;
  int32_t rc = INFR_CUDA_OK;
  if (cudaStreamCreateWithFlags(&ep->side, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&ep->xfer, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&ep->ev_x, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&ep->ev_xg, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&ep->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&ep->ev_join, cudaEventDisableTiming) != cudaSuccess ||
      cudaMalloc(reinterpret_cast<void**>(&ep->shape_dev), (size_t)world * 8 * sizeof(int32_t)) != cudaSuccess)
    rc = fail(ctx, INFR_CUDA_ERR_CUDA, "ep_init: stream / event / buffer creation failed");
  for (int i = 0; i < EP_PHASES && rc == INFR_CUDA_OK; ++i)
    if (cudaEventCreate(&ep->ev_phase[i]) != cudaSuccess) rc = fail(ctx, INFR_CUDA_ERR_CUDA, "ep_init: event creation failed");
  if (rc == INFR_CUDA_OK) {
    // The rendezvous blocks until every rank has arrived; it runs on a helper thread so that a rank
    // that never comes costs this one a bounded wait and an error instead of a hang.
    ncclUniqueId u;
    std::memcpy(&u, id, sizeof u);
    const int dev = ctx->device;
    auto task = std::make_shared<std::packaged_task<std::pair<ncclResult_t, ncclComm_t>()>>([api, u, rank, world, dev]() {
      cudaSetDevice(dev);
      ncclComm_t c = nullptr;
      const ncclResult_t r = api->CommInitRank(&c, world, u, rank);
      return std::make_pair(r, c);
    });
    auto fut = task->get_future();
    std::thread([task]() { (*task)(); }).detach();
    const auto limit = std::chrono::milliseconds(ctx->cfg.sync_timeout_ms ? ctx->cfg.sync_timeout_ms : 60000u);
    if (fut.wait_for(limit) != std::future_status::ready) {
      rc = fail(ctx, INFR_CUDA_ERR_NCCL, "ep_init: the ranks did not all arrive within the limit");
    } else {
      const auto res = fut.get();
      if (res.first != ncclSuccess)
        rc = fail(ctx, INFR_CUDA_ERR_NCCL, std::string("ep_init: ncclCommInitRank: ") + api->GetErrorString(res.first));
      else
        ep->comm = res.second;
    }
  }
  if (rc != INFR_CUDA_OK) {
    const std::string msg = ctx->last_error;
    ep_release(ctx, false);
    ctx->last_error = msg;
  }
  if (prev >= 0 && prev != ctx->device) cudaSetDevice(prev);
  return rc;
}

int32_t infr_cuda_ep_finalize(infr_cuda_ctx* ctx) {
  if (!ctx) return INFR_CUDA_ERR_INVALID_ARG;
  if (!ctx->ep) return INFR_CUDA_OK;
  if (ctx->capturing) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "ep_finalize: not while recording");
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != ctx->device) cudaSetDevice(ctx->device);
  const int32_t rc = ctx->ep->dead ? INFR_CUDA_OK : ep_wait_stream(ctx, "ep_finalize");
  ep_release(ctx, rc == INFR_CUDA_OK);
  if (prev >= 0 && prev != ctx->device) cudaSetDevice(prev);
  return rc;
}

int32_t infr_cuda_ep_last_phases(infr_cuda_ctx* ctx, float ms_out[5]) {
  if (!ctx || !ms_out) return INFR_CUDA_ERR_INVALID_ARG;
  EpState* ep = ctx->ep;
  if (!ep || !ep->phases_valid) return fail(ctx, INFR_CUDA_ERR_INVALID_ARG, "ep_last_phases: no expert-parallel call has run (un-recorded) on this context");
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != ctx->device) cudaSetDevice(ctx->device);
  int32_t rc = ep_wait_stream(ctx, "ep_last_phases");
  for (int i = 0; i < 5 && rc == INFR_CUDA_OK; ++i) {
    const cudaError_t e = cudaEventElapsedTime(&ms_out[i], ep->ev_phase[0], ep->ev_phase[i + 1]);
    if (e != cudaSuccess) rc = check_cuda(ctx, e, "ep_last_phases");
  }
  if (prev >= 0 && prev != ctx->device) cudaSetDevice(prev);
  return rc;
}

}  // extern "C"
