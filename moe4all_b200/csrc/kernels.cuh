// Kernel parameter blocks and host-side launchers (one translation unit per kernel family).
#pragma once
#include "common.cuh"

namespace infr {

// The whole-row router kernel (fused norm, fixed-point copy and top-k) takes up to this many rows per
// CTA group, up to ROUTE_SMALL_MAX_GROUPS groups (one selecting CTA each) and ROUTE_SMALL_LIMIT rows
// per call.
constexpr int ROUTE_SMALL_MAX_ROWS = 8;
constexpr int ROUTE_SMALL_MAX_GROUPS = 64;
constexpr int ROUTE_SMALL_LIMIT = 64;
// Marker of a logit that has not been written yet: a NaN pattern no arithmetic result has (the
// hardware's NaN results are 0x7FFFFFFF).  The whole-row kernel's logit buffer holds it between launches.
constexpr uint32_t ROUTE_LOGIT_EMPTY = 0xFFFFFFFFu;
constexpr size_t ROUTE_LOGIT_BYTES = (size_t)ROUTE_SMALL_LIMIT * 1024 * sizeof(float);  // rows x experts (at most 1024)

struct RouteParams {
  const float* router_x;     // [rows, ne]
  const float* x;            // [rows, ne] (shared-expert gate input)
  const float* router;       // [n_expert, ne] f32
  const float* sh_gate_inp;  // [ne] or null
  const float* bias;         // [n_expert] or null
  const int32_t* given_ids;  // [rows, n_used] selection made by the caller, or null (top-k)
  const float* rms_w;        // [ne] RmsNorm weight applied to x before everything else, or null
  float rms_eps;
  float* logits;             // [rows, n_expert] scratch (whole-row kernel: every word ROUTE_LOGIT_EMPTY on entry and on exit)
  float* sh_logit;           // [rows] scratch
  int32_t* ids;              // [rows, n_used]
  float* wts;                // [rows, n_used]
  DeviceStatus* status;      // bounded waits that ran out are recorded here
  int8_t *xq_lo, *xq_hi;     // [rows, ne] fixed-point limbs of x for the small-m expert kernels, or null
  float* xscale;             // [rows] value of one fixed-point unit
  int* xsum;                 // [rows, ne / 32] sums of the fixed-point x per 32 elements (expert-major kernels), or null
  unsigned long long* trace; // optional phase stamps
  int rows, ne, n_expert, n_used;
  float scale;
  int gating, norm_w, n_groups, n_groups_used;
};

// Formats of a call's expert banks (INFR_CUDA_DT_*); the shared expert's tensors follow the same three.
struct BankTypes {
  int32_t gate, up, down;
  bool tuned() const {  // the combination the per-pair, expert-major and tcgen05 kernels are written for
    return gate == INFR_CUDA_DT_Q4K && up == INFR_CUDA_DT_Q4K && (down == INFR_CUDA_DT_Q6K || down == INFR_CUDA_DT_Q4K);
  }
  bool down_q4k() const { return down == INFR_CUDA_DT_Q4K; }
};

struct DecodeParams {
  const float* x;        // [rows, ne]
  const int32_t* ids;    // [rows, n_used]
  const float* wts;      // [rows, n_used]
  const float* sh_logit; // [rows] or null (ungated shared expert)
  const int8_t *xq_lo, *xq_hi;  // [rows, ne] fixed-point limbs of x (X = 256*hi + lo)
  const float* xscale;   // [rows]
  const uint8_t *gate, *up, *down;           // routed banks
  const uint8_t *sh_gate, *sh_up, *sh_down;  // shared expert or null
  float* act;            // [rows*n_used, nff] then [rows, sh_ff]
  float* dst;            // [rows, ne]
  const float* residual; // [rows, ne] added to the result (may be dst itself), or null
  DeviceStatus* status;
  unsigned long long* trace;  // optional phase stamps
  size_t gate_stride, up_stride, down_stride;  // bytes per expert
  int rows, ne, n_used, nff, sh_ff, n_expert;
  uint32_t ep_lo, ep_n;  // band (ep_n == 0: off)
  int down_q4k;          // the down banks (routed and shared) are Q4_K instead of Q6_K
  int gate_dt, up_dt, down_dt;  // INFR_CUDA_DT_* of the banks (the generic-format kernels read these)
  int xsum_ready;        // the router kernel already made the expert-major kernels' sums of x (first array of their scratch)
  const float* down_scale;  // [n_expert] scale on a routed expert's down output, or null
  int act_kind;          // INFR_CUDA_ACT_*
  int weight_before;     // routing weight on gate and up before the activation, none on the output
  float clamp;           // > 0: routed experts clamp gate (one-sided) and up (both sides) first
};

// Expert-major small-m kernels (expert_major.cu): every (token, rank) pair of the call, grouped by
// expert into segments of a few token rows; pair ids P + r stand for the shared expert's copy of row r.
struct EmParams {
  const int8_t *xq_lo, *xq_hi;   // [rows, ne] fixed-point limbs of x
  const float* xscale;           // [rows]
  int* xsum;                     // [rows, ne/32] integer sums of x per 32-element sub-block
  int xsum_ready;                // made by the router kernel with the fixed-point copy: the bucket kernel skips them
  const int32_t* ids;            // [rows, n_used]
  const float* wts;              // [rows, n_used]
  int *n_seg, *seg_expert, *seg_off, *seg_cnt, *seg_pairs;  // segment table, built on the device
  const uint8_t *gate, *up, *down, *sh_gate, *sh_up, *sh_down;
  size_t gate_stride, up_stride, down_stride;
  float* act;                    // [pairs, nffmax] activations
  float* y;                      // [pairs, ne] raw expert outputs
  const float* down_scale;       // [n_expert] or null
  DeviceStatus* status;
  int rows, ne, n_used, nff, sh_ff, n_expert, nffmax;
  uint32_t ep_lo, ep_n;
  int act_kind, weight_before;
  float clamp;
};

// Device-side view of one grouped-GEMM launch (see grouped_ffn.cu).
struct GroupedParams {
  const int *tile_expert, *tile_row0, *tile_rows, *n_tiles;  // tile table built on the device
  // token rows grouped by expert, f16, K order 0,2,1,3 per four.  Legacy tiles: [rows, ne] and
  // [rows, nff] row-major.  tcgen05 tiles: [tile][K step][256 rows][64] with swizzled 128-byte lines.
  const __half* xg;
  __half* act;
  float* y;          // [rows, ne] raw down outputs: f32, or f16 in the same buffer when y_f16 is set
  int y_f16;         // the combine kernel is the only reader (tcgen05 tiles): rows as f16 with one power-of-two
                     // scale per 32 outputs of a row (y_scale), half the bytes both ways
  float* y_scale;    // [rows, ne / 32]: in the unused half of the y buffer
  const uint8_t *gate, *up, *down;
  const uint8_t *sh_gate, *sh_up, *sh_down;  // segment index n_expert = the shared expert
  size_t gate_stride, up_stride, down_stride;
  DeviceStatus* status;
  unsigned long long* trace;  // optional phase stamps
  int trace_tile;             // tile whose first CTA writes them
  int ne, nff, n_expert;
  int down_q4k;               // the down banks are Q4_K instead of Q6_K (tcgen05 kernels only)
  int gate_dt, up_dt, down_dt;  // INFR_CUDA_DT_* of the banks (the generic-format tiles read these)
  int act_kind;               // INFR_CUDA_ACT_*
  int gu_rows;                // rows of one expert in the gate bank: nff, or 2 nff where gate and up share a bank
  float clamp;                // > 0: routed tiles clamp gate (from above) and up (both sides) first
};

// Host-side description of one batched expert-FFN call.
struct GroupedCall {
  void* scratch;           // grouped_scratch_bytes(...) bytes
  const float* x;          // [rows, ne] f32 tokens (routed call) or rows grouped by expert
  const int32_t* ids;      // [rows, n_used] or null when the rows are already grouped
  const float* wts;        // [rows, n_used]
  const float* sh_logit;   // [rows] or null
  const int* seg_off_in;   // [n_expert + 1] device offsets (grouped-rows form)
  float* dst;              // [rows, ne] combined output, or null (grouped-rows form)
  const float* residual;   // [rows, ne] added to dst (may alias it), or null
  float* y_out;            // grouped-rows form: per-row outputs [rows, ne]; null = scratch
  const uint8_t *gate, *up, *down, *sh_gate, *sh_up, *sh_down;
  size_t gate_stride, up_stride, down_stride;
  int rows, n_used, n_pairs, ne, nff, n_expert;
  int shared_rows;         // rows of the shared-expert segment (rows or 0)
  int rows_bound;          // upper bound on grouped rows including the shared segment
  uint32_t ep_lo, ep_n;
  int legacy;              // 1: use the mma.sync tiles even where the tcgen05 kernels apply
  int down_q4k;            // the down banks are Q4_K instead of Q6_K
  int gate_dt, up_dt, down_dt;  // INFR_CUDA_DT_* of the banks
  int act_kind;            // INFR_CUDA_ACT_*
  float clamp;             // Op::MoeFfn::swiglu_clamp, 0 = none
  int weight_before;       // routing weight on the expert's input rows, none on its output
  const float* down_scale; // [n_expert] or null
};

bool umma_grouped_supported(int ne, int nff);
int umma_tile_rows();
int32_t launch_umma_grouped(infr_cuda_ctx* ctx, const GroupedParams& p, int max_tiles);
size_t grouped_scratch_bytes(int rows_total, int n_pairs, int n_seg, int ne, int nff);
int32_t launch_grouped_ffn(infr_cuda_ctx* ctx, const GroupedCall& c);
int32_t launch_combine(infr_cuda_ctx* ctx, const float* y, const int* pos_of_pair, const float* wts, const float* sh_logit,
                       const float* sh_y, int rows, int n_used, int ne, float* dst);

// Descriptor checks shared by the local and the expert-parallel entry (api.cu).
int32_t validate_moe_route(infr_cuda_ctx* ctx, const infr_cuda_moe_ffn_desc* d);
int32_t validate_moe_ffn(infr_cuda_ctx* ctx, const infr_cuda_moe_ffn_desc* d, uint32_t bank_experts);

// Path choice for a call (api.cu): 1 = small-m kernels, 2 = grouped GEMMs; and, inside path 1, whether the
// expert-major kernels are ahead of the per-pair ones.
uint32_t choose_moe_path(const infr_cuda_ctx* ctx, uint32_t rows, uint32_t n_used, uint32_t n_expert, uint32_t ne, uint32_t nff,
                         uint32_t sh_ff, BankTypes bt);
bool em_preferred(uint32_t rows, uint32_t n_used, uint32_t n_expert, uint32_t ne, uint32_t nff);

size_t small_path_scratch_need(const infr_cuda_moe_ffn_desc* d);

// Expert parallelism (ep.cu).  A descriptor is a collective call when the context has joined a
// communicator of more than one rank and the descriptor names this rank's band.
bool ep_call_is_collective(const infr_cuda_ctx* ctx, const infr_cuda_moe_ffn_desc* d);
int32_t ep_moe_ffn(infr_cuda_ctx* ctx, const infr_cuda_moe_ffn_desc* d);
int32_t ep_wait_stream(infr_cuda_ctx* ctx, const char* what);  // bounded wait; aborts the communicator when it runs out
void ep_release(infr_cuda_ctx* ctx, bool orderly);

int32_t launch_umma_selftest(infr_cuda_ctx* ctx, const __half* a, const __half* b, float* c, int n);
int32_t launch_route(infr_cuda_ctx* ctx, const RouteParams& p, bool pdl);
// Rows per group the whole-row router kernel would use for this shape; 0 = the call takes the batched router.
int route_small_group(const infr_cuda_ctx* ctx, int rows, int ne, int n_expert);
int32_t launch_decode_ffn(infr_cuda_ctx* ctx, const DecodeParams& p, bool pdl, uint32_t stages);
// The expert-major form of the same stages (2: bucket + gate/up, 4: down + combine); `scratch` holds em_scratch_bytes(...).
bool em_supported(int ne, int nff, int sh_ff, int n_expert, BankTypes bt);
size_t em_scratch_bytes(int rows, int n_used, int ne, int nff, int sh_ff);
int32_t launch_em_ffn(infr_cuda_ctx* ctx, const DecodeParams& p, void* scratch, uint32_t stages);
// Whether the small-m kernels cover this shape (dims, shared-memory budget).
bool decode_ffn_supported(const infr_cuda_ctx* ctx, int ne, int nff, int sh_ff, int n_used, BankTypes bt, std::string* why);
// Small-m kernels for banks in any mix of Q4_K / Q5_K / Q6_K / Q8_0 (anyfmt_ffn.cu): the tuned kernels'
// arithmetic with the blocks read straight from global memory.
bool anyfmt_decode_supported(int ne, int nff, int sh_ff, int n_used, BankTypes bt, std::string* why);
int32_t launch_anyfmt_decode(infr_cuda_ctx* ctx, const DecodeParams& p, bool pdl, uint32_t stages);

// y[m, out_f] = x[m, in_f] · Wᵀ for W of dtype F32 / Q4_K / Q6_K.
int32_t launch_linear(infr_cuda_ctx* ctx, int32_t dtype, const uint8_t* w, const float* x, float* y, int m, int in_f,
                      int out_f);
int32_t launch_gated_act(infr_cuda_ctx* ctx, const float* gate, const float* up, float* dst, size_t n);
int32_t launch_shared_add(infr_cuda_ctx* ctx, const float* moe, const float* shexp, const float* gate, float* dst,
                          int rows, int n);
int32_t launch_rmsnorm(infr_cuda_ctx* ctx, const float* x, const float* w, float* dst, int rows, int dim, float eps);
int32_t launch_quantize_rows(infr_cuda_ctx* ctx, const float* x, int8_t* lo, int8_t* hi, float* scale, int rows, int dim);
int32_t launch_add(infr_cuda_ctx* ctx, const float* a, const float* b, float* dst, size_t n);
// dst[0, bytes) = the pinned host range whose device view is src_dev_view (16-byte aligned, bytes % 16 == 0).
int32_t launch_fetch_host(infr_cuda_ctx* ctx, const void* src_dev_view, void* dst, size_t bytes);
int32_t launch_store_host(infr_cuda_ctx* ctx, const void* src, void* dst_dev_view, size_t bytes);
// The grid tables' device addresses into the constant memory of each translation unit that unpacks weights.
cudaError_t publish_codebooks_dense(const unsigned char* const* tables);
cudaError_t publish_codebooks_anyfmt(const unsigned char* const* tables);
cudaError_t publish_codebooks_grouped(const unsigned char* const* tables);
int32_t launch_fetch_host_gated(infr_cuda_ctx* ctx, const void* src_dev_view, void* dst, size_t bytes, const unsigned long long* bell,
                                unsigned long long ticket, unsigned long long limit_ns);
int32_t launch_host_signal(infr_cuda_ctx* ctx, unsigned long long* done, unsigned long long ticket);

}  // namespace infr
