// infr_cuda.hpp — C++ host side above the C ABI of infr_cuda.h.
//
// The reference's host code is Rust: a backend is an implementation of
// `infr_core::backend::Backend` (crates/infr-core/src/backend.rs:630-1088) that owns buffers
// (`Buffer`, backend.rs:423-436), compiles a graph to a `Plan` and executes ops such as
// `Op::MoeFfn` (crates/infr-core/src/graph.rs:1259-1352), reporting caller mistakes as
// `Error::Backend` / `Error::Unsupported` values (crates/infr-core/src/error.rs:11-50) instead of
// panicking.  This header gives the same shape to a C++ host: same method names, argument meaning
// and error behaviour, nothing but calls into the C ABI underneath.  Header-only, C++17.
#pragma once

#include <cstdint>
#include <cstring>
#include <string>
#include <utility>
#include <vector>

#include "infr_cuda.h"

namespace infr_cuda {

// ---- errors: infr_core::error::Error ------------------------------------------------------------
enum class ErrorKind { None, Backend, Unsupported };

struct Status {
  ErrorKind kind = ErrorKind::None;
  int32_t code = INFR_CUDA_OK;  // the C ABI's status
  std::string message;
  bool ok() const { return kind == ErrorKind::None; }
  explicit operator bool() const { return ok(); }
};

// `Result<T>`: a value or the error that prevented it.
template <typename T>
struct Result {
  Status status;
  T value{};
  bool ok() const { return status.ok(); }
};

// crates/infr-core/src/tensor.rs:7-57, numbered as in the GGUF file format.
enum class DType : int32_t { F32 = INFR_CUDA_DT_F32, Q4_0 = INFR_CUDA_DT_Q4_0, Q4_1 = INFR_CUDA_DT_Q4_1, Q5_0 = INFR_CUDA_DT_Q5_0,
                             Q5_1 = INFR_CUDA_DT_Q5_1, Q2K = INFR_CUDA_DT_Q2K, Q3K = INFR_CUDA_DT_Q3K, Q8_0 = INFR_CUDA_DT_Q8_0, Q4K = INFR_CUDA_DT_Q4K, Q5K = INFR_CUDA_DT_Q5K, Q6K = INFR_CUDA_DT_Q6K, IQ4NL = INFR_CUDA_DT_IQ4NL, IQ4XS = INFR_CUDA_DT_IQ4XS, MXFP4 = INFR_CUDA_DT_MXFP4, NVFP4 = INFR_CUDA_DT_NVFP4, Q2_0 = INFR_CUDA_DT_Q2_0,
                             IQ2XS = INFR_CUDA_DT_IQ2XS, IQ2S = INFR_CUDA_DT_IQ2S, IQ3XXS = INFR_CUDA_DT_IQ3XXS, IQ3S = INFR_CUDA_DT_IQ3S };
// crates/infr-core/src/graph.rs:73-85
enum class MoeGating : uint32_t {
  Softmax = INFR_CUDA_GATING_SOFTMAX,
  Sigmoid = INFR_CUDA_GATING_SIGMOID,
  SqrtSoftplus = INFR_CUDA_GATING_SQRT_SOFTPLUS
};
enum class Activation : uint32_t { Silu = INFR_CUDA_ACT_SILU, Gelu = INFR_CUDA_ACT_GELU, Sigmoid = INFR_CUDA_ACT_SIGMOID };

// What a MoE-only backend reports (backend.rs:45-236): everything off except in-place graph inputs.
struct Capabilities {
  std::string name;
  bool unified_memory = false;
  bool graph_input_inplace = true;
  bool decode_replay = false;
  bool embed_gather = false;
  bool gpu_sample = false;
};

class Backend;

// `Box<dyn Buffer>`: owned by the model, freed when dropped; `len_bytes` is the logical extent
// (backend.rs:424-433).
class Buffer {
 public:
  Buffer() = default;
  Buffer(Buffer&& o) noexcept { *this = std::move(o); }
  Buffer& operator=(Buffer&& o) noexcept {
    if (this != &o) {
      reset();
      ctx_ = o.ctx_;
      h_ = o.h_;
      o.ctx_ = nullptr;
      o.h_ = nullptr;
    }
    return *this;
  }
  Buffer(const Buffer&) = delete;
  Buffer& operator=(const Buffer&) = delete;
  ~Buffer() { reset(); }
  size_t len_bytes() const { return h_ ? infr_cuda_buf_len(h_) : 0; }
  infr_cuda_buf* handle() const { return h_; }
  bool valid() const { return h_ != nullptr; }

 private:
  friend class Backend;
  void reset() {
    if (h_) infr_cuda_free(ctx_, h_);
    h_ = nullptr;
  }
  infr_cuda_ctx* ctx_ = nullptr;
  infr_cuda_buf* h_ = nullptr;
};

// `Box<dyn Plan>`: ops recorded once, executed many times.
class Plan {
 public:
  Plan() = default;
  Plan(Plan&& o) noexcept { *this = std::move(o); }
  Plan& operator=(Plan&& o) noexcept {
    if (this != &o) {
      reset();
      ctx_ = o.ctx_;
      g_ = o.g_;
      o.g_ = nullptr;
    }
    return *this;
  }
  Plan(const Plan&) = delete;
  Plan& operator=(const Plan&) = delete;
  ~Plan() { reset(); }
  bool valid() const { return g_ != nullptr; }

 private:
  friend class Backend;
  void reset() {
    if (g_) infr_cuda_graph_free(ctx_, g_);
    g_ = nullptr;
  }
  infr_cuda_ctx* ctx_ = nullptr;
  infr_cuda_graph* g_ = nullptr;
};

// `Op::MoeFfn` (graph.rs:1259-1352) with bound buffers, in the forms the CUDA kernels cover:
// split gate/up banks, SiLU, output-side weighting.  Optional members are null pointers.
struct MoeFfn {
  const Buffer* x = nullptr;
  const Buffer* router_x = nullptr;  // null: the router reads x
  const Buffer* router = nullptr;
  const Buffer* gate_exps = nullptr;
  const Buffer* up_exps = nullptr;
  const Buffer* down_exps = nullptr;
  const Buffer* exp_probs_b = nullptr;
  Buffer* dst = nullptr;
  Buffer* ids_out = nullptr;
  Buffer* wts_out = nullptr;
  uint32_t rows = 0, ne = 0, n_expert = 0, n_used = 0, n_ff_exp = 0;
  float scale = 1.0f;
  DType router_dtype = DType::F32, gate_dtype = DType::Q4K, up_dtype = DType::Q4K, down_dtype = DType::Q6K;
  MoeGating gating = MoeGating::Softmax;
  bool norm_w = true;
  uint32_t n_expert_groups = 0, n_expert_groups_used = 0;
  uint32_t ep_lo = 0, ep_n_local = 0;  // Op::MoeFfn::ep_band
  // shared expert riding in the same call (runner.rs:8088-8175)
  const Buffer* sh_gate = nullptr;
  const Buffer* sh_up = nullptr;
  const Buffer* sh_down = nullptr;
  const Buffer* sh_gate_inp = nullptr;
  uint32_t sh_ff = 0;
  // fusions of crates/infr-core/src/fusion.rs:17-25, 53-82
  const Buffer* norm_weight = nullptr;
  float norm_eps = 1e-6f;
  const Buffer* residual = nullptr;
  const Buffer* expert_ids = nullptr;  // graph.rs:1320-1351: the caller's selection, [rows, n_used] i32
  const Buffer* down_scale = nullptr;  // graph.rs:1273-1276: [n_expert] f32
  Activation act = Activation::Silu;
  bool weight_before = false;          // graph.rs:1298-1303
  float swiglu_clamp = 0.f;            // graph.rs:1283-1290; 0 = none
  bool fused_gate_up = false;          // graph.rs:1277-1282: gate_exps = [n_expert, 2*n_ff_exp, ne]

  infr_cuda_moe_ffn_desc to_desc() const {
    infr_cuda_moe_ffn_desc d;
    std::memset(&d, 0, sizeof d);
    auto h = [](const Buffer* b) -> infr_cuda_buf* { return b ? b->handle() : nullptr; };
    d.x = h(x);
    d.router_x = h(router_x ? router_x : x);
    d.router = h(router);
    d.gate_exps = h(gate_exps);
    d.up_exps = h(up_exps);
    d.down_exps = h(down_exps);
    d.exp_probs_b = h(exp_probs_b);
    d.dst = h(dst);
    d.ids_out = h(ids_out);
    d.wts_out = h(wts_out);
    d.rows = rows;
    d.ne = ne;
    d.n_expert = n_expert;
    d.n_used = n_used;
    d.n_ff_exp = n_ff_exp;
    d.scale = scale;
    d.router_dtype = static_cast<int32_t>(router_dtype);
    d.gate_dtype = static_cast<int32_t>(gate_dtype);
    d.up_dtype = static_cast<int32_t>(up_dtype);
    d.down_dtype = static_cast<int32_t>(down_dtype);
    d.gating = static_cast<uint32_t>(gating);
    d.norm_w = norm_w ? 1u : 0u;
    d.n_expert_groups = n_expert_groups;
    d.n_expert_groups_used = n_expert_groups_used;
    d.ep_lo = ep_lo;
    d.ep_n_local = ep_n_local;
    d.sh_gate = h(sh_gate);
    d.sh_up = h(sh_up);
    d.sh_down = h(sh_down);
    d.sh_gate_inp = h(sh_gate_inp);
    d.sh_ff = sh_ff;
    d.norm_weight = h(norm_weight);
    d.norm_eps = norm_eps;
    d.residual = h(residual);
    d.expert_ids = h(expert_ids);
    d.down_scale = h(down_scale);
    d.act = static_cast<uint32_t>(act);
    d.weight_before = weight_before ? 1u : 0u;
    d.swiglu_clamp = swiglu_clamp;
    d.fused_gate_up = fused_gate_up ? 1u : 0u;
    return d;
  }
};

// `impl Backend for CudaBackend`.  Calls on one backend must be serialised by the caller, as the
// reference's op loop does; distinct backends are independent.
class Backend {
 public:
  static Result<Backend> create(int device) {
    Result<Backend> r;
    infr_cuda_ctx* ctx = nullptr;
    const int32_t rc = infr_cuda_create(device, &ctx);
    if (rc != INFR_CUDA_OK) {
      r.status = make_status(nullptr, rc, "infr_cuda_create failed (no B200 visible, or the device index is out of range)");
      return r;
    }
    r.value.ctx_ = ctx;
    return r;
  }
  Backend() = default;
  Backend(Backend&& o) noexcept { *this = std::move(o); }
  Backend& operator=(Backend&& o) noexcept {
    if (this != &o) {
      if (ctx_) infr_cuda_destroy(ctx_);
      ctx_ = o.ctx_;
      o.ctx_ = nullptr;
    }
    return *this;
  }
  Backend(const Backend&) = delete;
  Backend& operator=(const Backend&) = delete;
  ~Backend() {
    if (ctx_) infr_cuda_destroy(ctx_);
  }

  // backend.rs:631-632
  std::string name() const { return infr_cuda_name(); }
  Capabilities capabilities() const {
    Capabilities c;
    c.name = name();
    return c;
  }

  // backend.rs:652 (zero-initialised) and :659
  Result<Buffer> alloc(size_t bytes) { return alloc_impl(bytes, 1); }
  Result<Buffer> alloc_uninit(size_t bytes) { return alloc_impl(bytes, 0); }

  // backend.rs:759-760: prefix copies; a range beyond the buffer is an error, not a crash
  Status upload(Buffer& dst, const void* src, size_t n, size_t offset = 0) { return st(infr_cuda_upload(ctx_, dst.handle(), offset, src, n)); }
  Status download(const Buffer& src, void* dst, size_t n, size_t offset = 0) { return st(infr_cuda_download(ctx_, src.handle(), offset, dst, n)); }
  template <typename T>
  Result<Buffer> from_host(const std::vector<T>& v) {
    Result<Buffer> b = alloc_uninit(v.size() * sizeof(T) < 16 ? 16 : v.size() * sizeof(T));
    if (b.ok()) b.status = upload(b.value, v.data(), v.size() * sizeof(T));
    return b;
  }
  // backend.rs:1006
  Status sync() { return st(infr_cuda_sync(ctx_)); }

  // backend.rs:908 for one-op graphs
  Status moe_ffn(const MoeFfn& op) {
    const infr_cuda_moe_ffn_desc d = op.to_desc();
    return st(infr_cuda_moe_ffn(ctx_, &d));
  }
  Status moe_route(const MoeFfn& op) {
    const infr_cuda_moe_ffn_desc d = op.to_desc();
    return st(infr_cuda_moe_route(ctx_, &d));
  }
  Status linear(DType dtype, const Buffer& w, const Buffer& x, Buffer& y, uint32_t m, uint32_t in_f, uint32_t out_f) {
    return st(infr_cuda_linear(ctx_, static_cast<int32_t>(dtype), w.handle(), x.handle(), y.handle(), m, in_f, out_f));
  }
  Status gated_act(const Buffer& gate, const Buffer& up, Buffer& dst, size_t n) { return st(infr_cuda_gated_act(ctx_, gate.handle(), up.handle(), dst.handle(), n)); }
  Status moe_shared_expert_add(const Buffer& moe, const Buffer& shexp, const Buffer& gate, Buffer& dst, uint32_t rows, uint32_t n) {
    return st(infr_cuda_moe_shared_add(ctx_, moe.handle(), shexp.handle(), gate.handle(), dst.handle(), rows, n));
  }
  Status rms_norm(const Buffer& x, const Buffer& weight, Buffer& dst, uint32_t rows, uint32_t dim, float eps) {
    return st(infr_cuda_rmsnorm(ctx_, x.handle(), weight.handle(), dst.handle(), rows, dim, eps));
  }
  Status add(const Buffer& a, const Buffer& b, Buffer& dst, size_t n) { return st(infr_cuda_add(ctx_, a.handle(), b.handle(), dst.handle(), n)); }

  // backend.rs:907-908: ops issued between begin_record and end_record are compiled into a plan
  // ---- tuning switches (the reference's typed kernel config, crates/infr-core/src/config/mod.rs:1-29) ----
  Result<infr_cuda_config> config() const {
    Result<infr_cuda_config> r;
    r.status = st(infr_cuda_get_config(ctx_, &r.value));
    return r;
  }
  Status set_config(const infr_cuda_config& cfg) { return st(infr_cuda_set_config(ctx_, &cfg)); }

  // ---- expert parallelism (ExpertParallelBackend, crates/infr-vulkan/src/ep.rs) ----
  // Rank 0 makes the id and hands it to the other ranks; `join` is collective.  Afterwards a MoeFfn
  // whose band is this rank's runs as the collective form of the op (banks hold the band only).
  static Result<std::vector<uint8_t>> ep_unique_id() {
    Result<std::vector<uint8_t>> r;
    r.value.resize(INFR_CUDA_EP_ID_BYTES);
    r.status = make_status(nullptr, infr_cuda_ep_unique_id(r.value.data()), "ncclGetUniqueId failed (is libnccl.so.2 loadable?)");
    return r;
  }
  Status join(const std::vector<uint8_t>& id, int32_t rank, int32_t world) {
    if (id.size() != INFR_CUDA_EP_ID_BYTES) return make_status(nullptr, INFR_CUDA_ERR_INVALID_ARG, "the communicator id must be 128 bytes");
    return st(infr_cuda_ep_init(ctx_, id.data(), rank, world));
  }
  Status leave() { return st(infr_cuda_ep_finalize(ctx_)); }

  // The grid table of a codebook format (IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S), handed over once per format.
  Status set_codebook(DType dtype, const void* table, size_t bytes) { return st(infr_cuda_set_codebook(ctx_, (int32_t)dtype, table, bytes)); }

  Status begin_record() { return st(infr_cuda_graph_begin(ctx_)); }
  Result<Plan> end_record() {
    Result<Plan> r;
    infr_cuda_graph* g = nullptr;
    r.status = st(infr_cuda_graph_end(ctx_, &g));
    if (r.ok()) {
      r.value.ctx_ = ctx_;
      r.value.g_ = g;
    }
    return r;
  }
  Status execute(const Plan& plan) { return st(infr_cuda_graph_launch(ctx_, plan.g_)); }

  // Host-paced plans: steps recorded and launched once, each released by a ticket the host writes into
  // pinned memory and reported back the same way (no launch and no stream wait per step).
  Status upload_gated(Buffer& dst, const void* pinned_src, size_t n, uint64_t ticket, size_t offset = 0) {
    return st(infr_cuda_upload_gated(ctx_, dst.handle(), offset, pinned_src, n, ticket));
  }
  Status host_signal(uint64_t ticket) { return st(infr_cuda_host_signal(ctx_, ticket)); }
  Status host_step(uint64_t ticket, void* stage, const void* rows, size_t n) { return st(infr_cuda_host_step(ctx_, ticket, stage, rows, n)); }
  Status host_steps(uint64_t first_ticket, uint32_t count, void* stage, const void* const* rows, size_t n_in, const void* result = nullptr,
                    void* const* results_out = nullptr, size_t n_out = 0) {
    return st(infr_cuda_host_steps(ctx_, first_ticket, count, stage, rows, n_in, result, results_out, n_out));
  }
  Status host_reset() { return st(infr_cuda_host_reset(ctx_)); }

  infr_cuda_ctx* raw() const { return ctx_; }

 private:
  static Status make_status(infr_cuda_ctx* ctx, int32_t rc, const char* fallback) {
    Status s;
    if (rc == INFR_CUDA_OK) return s;
    s.code = rc;
    s.kind = rc == INFR_CUDA_ERR_UNSUPPORTED ? ErrorKind::Unsupported : ErrorKind::Backend;
    const char* m = ctx ? infr_cuda_last_error(ctx) : nullptr;
    s.message = (m && *m) ? m : fallback;
    return s;
  }
  Status st(int32_t rc) const { return make_status(ctx_, rc, "the CUDA backend reported an error"); }
  Result<Buffer> alloc_impl(size_t bytes, int32_t zero) {
    Result<Buffer> r;
    infr_cuda_buf* h = nullptr;
    r.status = st(infr_cuda_alloc(ctx_, bytes, zero, &h));
    if (r.ok()) {
      r.value.ctx_ = ctx_;
      r.value.h_ = h;
    }
    return r;
  }
  infr_cuda_ctx* ctx_ = nullptr;
};

}  // namespace infr_cuda
