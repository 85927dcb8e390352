/* infr_cuda.h — C ABI of the B200 (sm_100a) backend for MoE4All's quantized MoE FFN path.
 *
 * This is the boundary a `Backend` implementation for the reference's seam
 * (crates/infr-core/src/backend.rs:630-1088) binds through FFI.  Every entry point takes plain
 * pointers and sizes, returns an int32 status (0 = ok, negative = error class) and never throws
 * or aborts; the text of the last error is kept per context (`infr_cuda_last_error`).
 *
 * A context is bound to one device and one stream.  Calls on one context must be serialised by
 * the caller (the reference runs one op loop per backend, backend.rs:891-899); distinct contexts
 * are independent.  There is no CPU fallback anywhere behind this header: an op, dtype or shape
 * the CUDA kernels do not cover returns INFR_CUDA_ERR_UNSUPPORTED.
 *
 * Weights are uploaded byte-for-byte as GGUF blocks (`Rewrite::Native`,
 * crates/infr-llama/src/seam/weight_upload.rs:8-14); nothing is repacked or re-quantised.
 */
#ifndef INFR_CUDA_H
#define INFR_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  They map onto infr_core::error::Error (crates/infr-core/src/error.rs:11-50):
 * INVALID_ARG/OOM/CUDA/NCCL/TIMEOUT → Error::Backend(msg), UNSUPPORTED → Error::Unsupported(msg). */
#define INFR_CUDA_OK 0
#define INFR_CUDA_ERR_INVALID_ARG (-1)
#define INFR_CUDA_ERR_UNSUPPORTED (-2)
#define INFR_CUDA_ERR_OOM (-3)
#define INFR_CUDA_ERR_CUDA (-4)
#define INFR_CUDA_ERR_NCCL (-5)
#define INFR_CUDA_ERR_TIMEOUT (-6)

/* Element / block types (crates/infr-core/src/tensor.rs:7-57), numbered as in the GGUF file
 * format so a loader can pass a tensor's type through unchanged. */
#define INFR_CUDA_DT_F32 0
#define INFR_CUDA_DT_Q4K 12 /* 256 weights / 144 B, crates/infr-core/src/decode_spec.rs:327 */
#define INFR_CUDA_DT_Q6K 14 /* 256 weights / 210 B, crates/infr-core/src/decode_spec.rs:331 */
#define INFR_CUDA_DT_Q8_0 8 /* 32 weights / 34 B, crates/infr-core/src/decode_spec.rs:320   */
#define INFR_CUDA_DT_Q5K 13 /* 256 weights / 176 B, crates/infr-core/src/decode_spec.rs:329 */
#define INFR_CUDA_DT_Q4_0 2 /* 32 weights / 18 B, crates/infr-core/src/decode_spec.rs:312   */
#define INFR_CUDA_DT_Q4_1 3 /* 32 weights / 20 B, crates/infr-core/src/decode_spec.rs:314   */
#define INFR_CUDA_DT_Q5_0 6 /* 32 weights / 22 B, crates/infr-core/src/decode_spec.rs:316   */
#define INFR_CUDA_DT_Q5_1 7 /* 32 weights / 24 B, crates/infr-core/src/decode_spec.rs:318   */
#define INFR_CUDA_DT_Q2K 10 /* 256 weights / 84 B, crates/infr-core/src/decode_spec.rs:323  */
#define INFR_CUDA_DT_Q3K 11 /* 256 weights / 110 B, crates/infr-core/src/decode_spec.rs:325 */
#define INFR_CUDA_DT_IQ4NL 20 /* 32 weights / 18 B, crates/infr-core/src/decode_spec.rs:349  */
#define INFR_CUDA_DT_IQ4XS 23 /* 256 weights / 136 B, crates/infr-core/src/decode_spec.rs:351 */
#define INFR_CUDA_DT_MXFP4 39 /* 32 weights / 17 B, crates/infr-core/src/decode_spec.rs:361  */
#define INFR_CUDA_DT_NVFP4 40 /* 64 weights / 36 B, crates/infr-core/src/decode_spec.rs:363  */
#define INFR_CUDA_DT_Q2_0 42 /* 64 weights / 18 B, crates/infr-core/src/decode_spec.rs:358   */
/* grid codebook formats (256 weights per block): usable once the format's grid table has been handed over
 * with infr_cuda_set_codebook */
#define INFR_CUDA_DT_IQ2XS 17  /* 74 B  */
#define INFR_CUDA_DT_IQ3XXS 18 /* 98 B  */
#define INFR_CUDA_DT_IQ3S 21   /* 110 B */
#define INFR_CUDA_DT_IQ2S 22   /* 82 B  */

/* MoeGating (crates/infr-core/src/graph.rs:73-85). */
#define INFR_CUDA_GATING_SOFTMAX 0
#define INFR_CUDA_GATING_SIGMOID 1
#define INFR_CUDA_ACT_SILU 0 /* g / (1 + exp(-g)) */
#define INFR_CUDA_ACT_GELU 1 /* 0.5 g (1 + tanh(0.7978846 (g + 0.044715 g^3))), kernels.rs:6664-6669 */
#define INFR_CUDA_ACT_SIGMOID 2 /* 1 / (1 + exp(-g)); no clamp with it, as in the reference (lib.rs:3613-3619) */
#define INFR_CUDA_GATING_SQRT_SOFTPLUS 2 /* sqrt(ln(1 + exp(v))), v itself above 20 (infr-cpu lib.rs:3760-3774) */

typedef struct infr_cuda_ctx infr_cuda_ctx; /* opaque: device, stream, scratch */
typedef struct infr_cuda_buf infr_cuda_buf; /* opaque: one device allocation, owned by the caller */

/* ---- context ------------------------------------------------------------------------------- */

/* Backend construction (the reference: `VulkanBackend::new`, crates/infr-vulkan/src/lib.rs).
 * Fails with INFR_CUDA_ERR_UNSUPPORTED on a device that is not compute capability 10.x. */
int32_t infr_cuda_create(int32_t device, infr_cuda_ctx** out);
void infr_cuda_destroy(infr_cuda_ctx* ctx);
/* Message of the most recent failing call on this context ("" if none).  Valid until the next
 * call on the context.  `Backend` methods return it inside Error::Backend / Error::Unsupported. */
const char* infr_cuda_last_error(const infr_cuda_ctx* ctx);
/* Backend::name (backend.rs:631). */
const char* infr_cuda_name(void);
/* Use an existing CUDA stream (a `cudaStream_t` passed as void*) instead of the context's own;
 * NULL restores the context's stream.  Lets a host that owns streams (PyTorch, NCCL) order the
 * kernels with its own work.  No counterpart in the reference (Vulkan queues are internal). */
int32_t infr_cuda_set_stream(infr_cuda_ctx* ctx, void* cuda_stream);

/* Tuning switches of a context, a plain struct read and written as a whole (the reference folds its
 * kernel knobs into one typed `Config`, crates/infr-core/src/config/mod.rs:1-29; its path choice is
 * `kernels.vulkan.moe_small_m`, crates/infr-vulkan/src/adapter.rs:253-287).  Nothing in the library
 * reads the environment.  `infr_cuda_get_config` returns the defaults on a fresh context; every
 * field has a working default and none changes results beyond the stated tolerances. */
typedef struct infr_cuda_config {
  uint32_t gu_warps, gu_chunks;  /* per-pair gate/up kernel on grids of more than four waves: warps per CTA
                                    and row chunks per CTA (default 4 x 4); 0 = keep the one-wave shape   */
  uint32_t dn_warps;             /* per-pair down kernel on grids of more than four waves: warp cap
                                    (default 12); 0 = no cap                                              */
  uint32_t upload_by_copy;       /* 1: small pinned-memory copies of the *_async calls go through the copy
                                    engine instead of a fetch kernel (default 0)                          */
  uint32_t trace_tile;           /* tile whose CTAs write phase stamps in the tcgen05 kernels (default 0)  */
  uint32_t expert_major;         /* small-m path, who owns a CTA: 0 = choose by rows (default), 1 = always
                                    one (token, expert) pair per CTA, 2 = always one expert with all of
                                    its tokens per CTA (int8 tensor-core tiles)                           */
  uint32_t sync_timeout_ms;      /* expert-parallel contexts: how long infr_cuda_sync waits for the stream
                                    before it aborts the communicator and returns INFR_CUDA_ERR_NCCL
                                    (default 60000)                                                       */
  uint32_t raw_rows_f32;         /* batched path on the tcgen05 tiles: 1 = the experts' raw output rows cross memory
                                    as f32 between the down and the combine kernel instead of f16 with a scale
                                    per 32 outputs (twice the bytes, no rounding before the sum over a token's
                                    experts; default 0)                                                    */
  uint32_t gate_timeout_ms;      /* host-paced plans: how long a gated fetch waits for its ticket, and
                                    infr_cuda_host_await for its own, before giving up with
                                    INFR_CUDA_ERR_TIMEOUT (default 2000)                                  */
  uint32_t reserved[7];          /* zero                                                                  */
} infr_cuda_config;
int32_t infr_cuda_get_config(const infr_cuda_ctx* ctx, infr_cuda_config* out);
int32_t infr_cuda_set_config(infr_cuda_ctx* ctx, const infr_cuda_config* cfg);
/* The grid table of a codebook format (crates/infr-core/src/iquant_grids.rs: IQ2XS_GRID 512 x u64, IQ2S_GRID
 * 1024 x u64, IQ3XXS_GRID 256 x u32, IQ3S_GRID 512 x u32; little-endian entries, one byte per weight, every
 * byte below 128), copied to the device once.  `bytes` must be the table's exact size.  Banks and Linear
 * weights of that dtype are INFR_CUDA_ERR_UNSUPPORTED until the table is there.  The tables are constants of
 * the formats and the device copies belong to the device: every context of a device that has set a format's
 * table reads the last one set for it, and the copies (a few KB) stay allocated until the process ends. */
int32_t infr_cuda_set_codebook(infr_cuda_ctx* ctx, int32_t dtype, const void* table, size_t bytes);

/* ---- buffers: Backend::alloc / alloc_uninit / upload / download / sync ------------------------ */

/* Backend::alloc (backend.rs:652; zero-initialised, the calloc contract of :647-651) when
 * `zero` != 0, Backend::alloc_uninit (backend.rs:659) otherwise. */
int32_t infr_cuda_alloc(infr_cuda_ctx* ctx, size_t bytes, int32_t zero, infr_cuda_buf** out);
/* Wrap memory the caller already owns (a torch tensor, an NCCL receive buffer) as a buffer
 * handle; freeing the handle leaves the memory alone.  Any address the device can access will do:
 * device memory, or pinned host memory under unified addressing (a one-row `dst` there saves the
 * copy back).  No reference counterpart. */
int32_t infr_cuda_wrap(infr_cuda_ctx* ctx, void* device_ptr, size_t bytes, infr_cuda_buf** out);
void infr_cuda_free(infr_cuda_ctx* ctx, infr_cuda_buf* buf);
/* Buffer::len_bytes (backend.rs:424-433) and the raw device address. */
size_t infr_cuda_buf_len(const infr_cuda_buf* buf);
void* infr_cuda_buf_ptr(const infr_cuda_buf* buf);
/* Backend::upload / download (backend.rs:759-760): prefix copies at a byte offset; out-of-range
 * is an error, not a panic (backend.rs:22-33).  Both return after the copy has completed. */
int32_t infr_cuda_upload(infr_cuda_ctx* ctx, infr_cuda_buf* dst, size_t dst_off, const void* src, size_t n);
int32_t infr_cuda_download(infr_cuda_ctx* ctx, const infr_cuda_buf* src, size_t src_off, void* dst, size_t n);
/* The same copies queued on the context's stream without waiting for them: the host range must
 * stay valid and unmodified (upload) or unread (download) until infr_cuda_sync returns.  No
 * counterpart in the reference's trait, whose copies are blocking; a decode step that uploads its
 * input, replays a recorded plan and downloads the result pays for one wait instead of three.
 * A copy of up to 256 KB from or to pinned host memory (16-byte aligned) is done by a small kernel
 * instead of the copy engine, so that the kernels queued around it can overlap their own start
 * and a recorded plan holds kernel nodes only. */
int32_t infr_cuda_upload_async(infr_cuda_ctx* ctx, infr_cuda_buf* dst, size_t dst_off, const void* src, size_t n);
int32_t infr_cuda_download_async(infr_cuda_ctx* ctx, const infr_cuda_buf* src, size_t src_off, void* dst, size_t n);

/* Host-paced plans: many decode steps recorded once (infr_cuda_graph_begin / end), launched once, and
 * then paced by the host through two words in pinned memory instead of one launch and one stream wait
 * per step.  A step is recorded as
 *     infr_cuda_upload_gated(ctx, x, 0, x_pinned, n, t);  ...ops...;  infr_cuda_host_signal(ctx, t);
 * with tickets t = 1, 2, ... in stream order, and run as
 *     write the step's rows into x_pinned;  infr_cuda_host_ring(ctx, t);  infr_cuda_host_await(ctx, t);
 * after which everything queued before the signal has finished (results written into pinned host memory,
 * directly by a kernel or by infr_cuda_download_async, are there).  The gated upload is the fetch kernel
 * of infr_cuda_upload_async (src: pinned host memory, 16-byte aligned, at most 256 KB, else
 * INFR_CUDA_ERR_UNSUPPORTED) whose CTAs first poll the bell word until it reaches the ticket; kernels
 * queued behind it may take their places and do their input-independent prologues meanwhile.  The wait is
 * bounded by `gate_timeout_ms`: a ticket that never comes is recorded like any other bounded wait
 * (INFR_CUDA_ERR_TIMEOUT from infr_cuda_host_await / infr_cuda_sync), and once anything has been recorded
 * later gates no longer wait, so a plan always drains.  infr_cuda_host_reset drains the stream and sets
 * both words back to zero: call it before launching a plan whose tickets start again at 1.
 * One pacing host thread per context. */
int32_t infr_cuda_upload_gated(infr_cuda_ctx* ctx, infr_cuda_buf* dst, size_t dst_off, const void* src, size_t n, uint64_t ticket);
int32_t infr_cuda_host_signal(infr_cuda_ctx* ctx, uint64_t ticket);
int32_t infr_cuda_host_ring(infr_cuda_ctx* ctx, uint64_t ticket);
int32_t infr_cuda_host_await(infr_cuda_ctx* ctx, uint64_t ticket);
int32_t infr_cuda_host_reset(infr_cuda_ctx* ctx);
/* One step in one call: copy `n` bytes of `rows` into the pinned staging range `stage` (skipped when `rows`
 * is NULL), ring `ticket`, await `ticket`. */
int32_t infr_cuda_host_step(infr_cuda_ctx* ctx, uint64_t ticket, void* stage, const void* rows, size_t n);
/* `count` consecutive steps in one call, tickets first_ticket, first_ticket + 1, ...: step i copies `n_in` bytes
 * of rows[i] into `stage`, rings and awaits its ticket, then (results_out not NULL) copies the step's `n_out`
 * result bytes from `result` (the pinned range the recorded step writes) to results_out[i].  For hosts that know
 * a run of inputs in advance (teacher-forced evaluation, benchmarks); stops at the first error. */
int32_t infr_cuda_host_steps(infr_cuda_ctx* ctx, uint64_t first_ticket, uint32_t count, void* stage, const void* const* rows, size_t n_in,
                             const void* result, void* const* results_out, size_t n_out);
/* Backend::sync (backend.rs:1006). */
int32_t infr_cuda_sync(infr_cuda_ctx* ctx);

/* ---- Op::MoeFfn ------------------------------------------------------------------------------ */

/* Mirrors Op::MoeFfn (crates/infr-core/src/graph.rs:1259-1352), every field of it: split or fused
 * gate/up banks, SiLU / GELU / Sigmoid, routing weight on the output or on the input
 * (`weight_before`), `down_scale`, caller-selected `expert_ids`, SwiGLU clamp, `ep_band`.  Banks are
 * `[n_expert, out_f, in_f]` row-major, expert e = the e-th equal byte slice (graph.rs:1257-1258);
 * a bank buffer needs exactly that many bytes - no kernel reads past a bank's last block.
 *
 * The shared expert of qwen35moe / DeepSeek (graph builder: crates/infr-llama/src/seam/runner.rs:
 * 8088-8175) can ride in the same call: when `sh_gate` is non-NULL the result is
 *   dst = moe + sigmoid(sh_gate_inp · x) * shexp(x)   if sh_gate_inp != NULL  (Op::MoeSharedExpertAdd)
 *   dst = moe + shexp(x)                              otherwise               (Op::Add)
 * exactly as the separate Linear / GatedAct / Linear / MoeSharedExpertAdd ops would produce. */
typedef struct infr_cuda_moe_ffn_desc {
  const infr_cuda_buf* x;           /* [rows, ne] f32: expert input                                */
  const infr_cuda_buf* router_x;    /* [rows, ne] f32: router input (often the same buffer as x)   */
  const infr_cuda_buf* router;      /* [n_expert, ne] router_dtype                                 */
  const infr_cuda_buf* gate_exps;   /* [n_expert, n_ff_exp, ne] gate_dtype                         */
  const infr_cuda_buf* up_exps;     /* [n_expert, n_ff_exp, ne] up_dtype                           */
  const infr_cuda_buf* down_exps;   /* [n_expert, ne, n_ff_exp] down_dtype                         */
  const infr_cuda_buf* exp_probs_b; /* [n_expert] f32 selection-only bias, or NULL                 */
  infr_cuda_buf* dst;               /* [rows, ne] f32                                              */
  infr_cuda_buf* ids_out;           /* [rows, n_used] i32 selected experts, rank order; or NULL    */
  infr_cuda_buf* wts_out;           /* [rows, n_used] f32 routing weights, rank order; or NULL     */
  uint32_t rows, ne, n_expert, n_used, n_ff_exp;
  float scale;
  int32_t router_dtype, gate_dtype, up_dtype, down_dtype; /* INFR_CUDA_DT_*                        */
  uint32_t gating;                  /* INFR_CUDA_GATING_*                                          */
  uint32_t norm_w;                  /* renormalise the selected probabilities to sum 1             */
  uint32_t n_expert_groups, n_expert_groups_used; /* group-limited routing; 0/1 groups = off       */
  uint32_t ep_lo, ep_n_local;       /* Op::MoeFfn::ep_band (graph.rs:1309-1319): only experts in
                                       [ep_lo, ep_lo+ep_n_local) contribute; ep_n_local == 0 = off */
  /* fused shared expert (all NULL = none) */
  const infr_cuda_buf* sh_gate;     /* [sh_ff, ne] gate_dtype                                      */
  const infr_cuda_buf* sh_up;       /* [sh_ff, ne] up_dtype                                        */
  const infr_cuda_buf* sh_down;     /* [ne, sh_ff] down_dtype                                      */
  const infr_cuda_buf* sh_gate_inp; /* [ne] f32 gate vector, or NULL for the ungated sum           */
  uint32_t sh_ff;
  uint32_t path;                    /* 0 = choose by rows (small-m while an expert sees fewer than
                                       about three tokens of the call on average);
                                       1 = force the small-m (decode) kernels;
                                       2 = force the grouped-GEMM (prefill) kernels; 3 = same with
                                       the legacy mma.sync tiles instead of tcgen05               */
  /* optional fusions the reference's graph rewriter applies around the op
   * (crates/infr-core/src/fusion.rs:17-25, 53-82); both need router_x == x */
  const infr_cuda_buf* norm_weight; /* RmsNorm -> MoeFfn: x is the un-normed row, the op first computes
                                       RmsNorm(x, norm_weight, norm_eps) and feeds that to the router,
                                       the experts and the shared expert; NULL = off                */
  const infr_cuda_buf* residual;    /* MoeFfn -> Add: [rows, ne] f32 added to the result; may be the
                                       same buffer as dst (in-place hidden update); NULL = off      */
  float norm_eps;
  uint32_t stages;                  /* 0 = the whole op.  Otherwise a mask of the kernels to launch:
                                       1 router + top-k, 2 gate/up, 4 down + combine, 8 the
                                       fixed-point copy of x the small-m expert kernels read
                                       (made by stage 1 otherwise).  Later
                                       stages read ids_out / wts_out (what an earlier call left
                                       there, or routing done elsewhere: an expert-parallel rank
                                       passes the ids it received with stages = 14) and the
                                       context's scratch.  A negative id marks a pair that is not
                                       this call's to serve; it contributes nothing.               */
  const infr_cuda_buf* expert_ids;  /* Op::MoeFfn::expert_ids (graph.rs:1320-1351, hash-routed layers):
                                       [rows, n_used] i32 experts chosen by the caller.  Only the
                                       selection is bypassed: the router and the gating function
                                       still run and the weights are the router's own probabilities
                                       at these experts (then norm_w and scale).  Refused together
                                       with exp_probs_b or expert groups.  An id outside
                                       [0, n_expert) is served as expert 0 and the next
                                       infr_cuda_sync / download fails with INVALID_ARG (the CPU
                                       panics there, lib.rs:3782-3788).  NULL = top-k routing.     */
  const infr_cuda_buf* down_scale;  /* Op::MoeFfn::down_scale (graph.rs:1273-1276): [n_expert] f32 on the
                                       selected expert's down output before the weighted sum
                                       (y = raw * scale[e], then w * y); NULL = none                */
  uint32_t act;                     /* INFR_CUDA_ACT_*: activation of the routed and shared experts */
  uint32_t weight_before;           /* routing weight applied to gate and up before the activation
                                       instead of to the expert's output (llama4, graph.rs:1298-1303) */
  float swiglu_clamp;               /* > 0: routed experts compute act(min(gate, l)) * clamp(up, -l, l)
                                       (graph.rs:1283-1290, kernels.rs:6671-6683); 0 = off; refused
                                       together with weight_before, as in the reference            */
  uint32_t fused_gate_up;           /* Op::MoeFfn::fused_gate_up (graph.rs:1277-1282): gate_exps holds
                                       [n_expert, 2 * n_ff_exp, ne], an expert's gate rows first and
                                       its up rows second; up_exps is not read                      */
} infr_cuda_moe_ffn_desc;

/* Backend::execute of a graph holding one Op::MoeFfn (backend.rs:908; CPU arm
 * crates/infr-cpu/src/lib.rs:3584-4304, Vulkan lowering crates/infr-vulkan/src/adapter.rs:
 * 8884-9652).  Asynchronous on the context's stream; outputs are visible after infr_cuda_sync or
 * a download. */
int32_t infr_cuda_moe_ffn(infr_cuda_ctx* ctx, const infr_cuda_moe_ffn_desc* desc);

/* Router logits + gating + top-k only (the `moe_topk` stage, crates/infr-vulkan/src/recorder.rs:
 * 12893; CPU crates/infr-cpu/src/lib.rs:3684-3863).  Uses the routing fields of the descriptor
 * (router_x, router, exp_probs_b, ids_out, wts_out, rows, ne, n_expert, n_used, scale, gating,
 * norm_w, groups); bank and dst fields are ignored.  ids_out and wts_out are required. */
int32_t infr_cuda_moe_route(infr_cuda_ctx* ctx, const infr_cuda_moe_ffn_desc* desc);

/* Routing for callers that must not allocate.  It has no counterpart in the reference.
 *
 * Some hosts cannot let a library call cudaMalloc: a serving process that has handed all device
 * memory to its own pool (a late cudaMalloc there simply fails), or a latency-critical loop that
 * cannot afford the device-wide synchronisation an allocation implies.  `infr_cuda_moe_route`
 * grows per-context scratch on demand; this variant does the same computation (router logits in
 * the CPU's accumulation order, softmax / sigmoid / sqrt-softplus gating, bias, expert groups,
 * top-k, routing weights) with its scratch in a fixed array inside the library image: 8 rows x
 * 1024 experts of f32 logits, 32 KB, held by every GPU that loads the library until the process
 * exits.  Larger calls are rejected with INFR_CUDA_ERR_INVALID_ARG and a message; nothing here
 * calls cudaMalloc, cudaFree or any allocating routine.  All arguments are plain device pointers
 * (inputs and outputs stay the caller's); `cuda_stream` is a cudaStream_t (NULL = the legacy
 * default stream); `err`/`err_cap` optionally receive the error text.
 *
 * The first call on a device looks up the device address of the array (cudaGetSymbolAddress) with
 * that device current; make that first call before any stream capture.  Every call shares the one
 * array (each call first resets the part it uses with a memset queued on the stream), and two calls
 * that overlap on the GPU race on it - keep calls on one device ordered on one stream.
 *
 * There is no context whose next sync could report a device-side failure, so the outputs carry it:
 * the call queues a fill of `ids_out` with -1 ahead of the kernel.  The kernel's only wait (for the
 * logits of its own grid) is bounded; if it ever gives up, the ids are still -1 when the stream has
 * drained and `wts_out` is unchanged.  An id of -1 therefore means "this call produced nothing". */
int32_t infr_cuda_moe_route_noalloc(int32_t device, void* cuda_stream, const float* router_x, const float* router,
                                    const float* exp_probs_b, int32_t* ids_out, float* wts_out, uint32_t rows,
                                    uint32_t ne, uint32_t n_expert, uint32_t n_used, float scale, uint32_t gating,
                                    uint32_t norm_w, uint32_t n_expert_groups, uint32_t n_expert_groups_used,
                                    char* err, size_t err_cap);

/* ---- the ops around it (shared expert and the 40-layer stack) --------------------------------- */

/* Op::Linear (crates/infr-cpu/src/lib.rs:1275-1328): y[m, out_f] = x[m, in_f] · Wᵀ, W row-major
 * [out_f, in_f] of `dtype` (F32 or any of the block formats above). */
int32_t infr_cuda_linear(infr_cuda_ctx* ctx, int32_t dtype, const infr_cuda_buf* w, const infr_cuda_buf* x,
                         infr_cuda_buf* y, uint32_t m, uint32_t in_f, uint32_t out_f);
/* Op::GatedAct with Activation::Silu, contiguous operands (crates/infr-cpu/src/lib.rs:2973-3027):
 * dst = silu(gate) * up, n elements. */
int32_t infr_cuda_gated_act(infr_cuda_ctx* ctx, const infr_cuda_buf* gate, const infr_cuda_buf* up,
                            infr_cuda_buf* dst, size_t n);
/* Op::MoeSharedExpertAdd (crates/infr-core/src/graph.rs:1449-1463; CPU lib.rs:3336-3356):
 * dst[r, :] = moe[r, :] + sigmoid(gate[r]) * shexp[r, :]. */
int32_t infr_cuda_moe_shared_add(infr_cuda_ctx* ctx, const infr_cuda_buf* moe, const infr_cuda_buf* shexp,
                                 const infr_cuda_buf* gate, infr_cuda_buf* dst, uint32_t rows, uint32_t n);
/* Op::RmsNorm (crates/infr-cpu/src/lib.rs:1046-1069). */
int32_t infr_cuda_rmsnorm(infr_cuda_ctx* ctx, const infr_cuda_buf* x, const infr_cuda_buf* weight,
                          infr_cuda_buf* dst, uint32_t rows, uint32_t dim, float eps);
/* Op::Add (crates/infr-cpu/src/lib.rs:3055-3070). */
int32_t infr_cuda_add(infr_cuda_ctx* ctx, const infr_cuda_buf* a, const infr_cuda_buf* b, infr_cuda_buf* dst,
                      size_t n);

/* ---- expert parallelism (crates/infr-vulkan/src/ep.rs:1-53, 156-505) ---------------------------- */

/* The reference's ExpertParallelBackend gives rank r the contiguous expert band
 * [r*E/W, (r+1)*E/W) (ep.rs:12-14, 171-176), runs every band's partial per MoE layer and sums the
 * partials in fixed rank order (ep.rs:454-493).  Here the ranks are processes, one per GPU, joined by
 * an NCCL communicator that the library owns; the tokens are sharded over the ranks as well.
 *
 *   rank 0:      infr_cuda_ep_unique_id(id)          (ncclGetUniqueId; 128 bytes, passed to the other
 *                                                    ranks by the host's own means)
 *   every rank:  infr_cuda_ep_init(ctx, id, rank, world)
 *
 * After that, a call of infr_cuda_moe_ffn whose descriptor carries this rank's band
 * (ep_lo == rank * n_expert / world, ep_n_local == n_expert / world) is a COLLECTIVE call: every
 * rank makes it, in the same order, with the same `rows`, ne, n_expert, n_used and n_ff_exp.  `x`,
 * `dst` (and residual, ids_out, wts_out) are this rank's `rows` token rows; router, exp_probs_b and
 * the shared expert are replicated; gate_exps / up_exps / down_exps hold ONLY the band's
 * ep_n_local experts.  Inside the call: routing of the rank's own rows, dispatch of rows, ids and
 * weights to the ranks (fixed-capacity slots of `rows` rows per pair of ranks, so that no count has to
 * come back to the host), the band's experts over everything received, the partial sums back to the
 * tokens' home ranks, and there the sum over ranks in rank order, then the shared expert (computed
 * on a side stream while the exchanges run) and the residual.  Results equal the single-device op
 * up to the association of that sum.  A descriptor without a band, or with another rank's band,
 * runs locally as before (the reference's replicated form: full banks, ids global).
 *
 * Failures: a rank that passes a different shape is detected before anything is exchanged (the
 * first call with a new shape compares the shapes of all ranks) and every rank gets
 * INFR_CUDA_ERR_NCCL; an NCCL call that fails, or a stream that does not drain within
 * `sync_timeout_ms` (a peer never arrived), aborts the communicator (ncclCommAbort) and returns
 * INFR_CUDA_ERR_NCCL from that call or from infr_cuda_sync.  After an abort the context runs
 * local calls only.  NCCL is loaded at run time (libnccl.so.2); without it ep_init returns
 * INFR_CUDA_ERR_UNSUPPORTED and everything else works. */
#define INFR_CUDA_EP_ID_BYTES 128
int32_t infr_cuda_ep_unique_id(uint8_t id[INFR_CUDA_EP_ID_BYTES]);
int32_t infr_cuda_ep_init(infr_cuda_ctx* ctx, const uint8_t id[INFR_CUDA_EP_ID_BYTES], int32_t rank, int32_t world);
/* Leaves the communicator (ncclCommDestroy after the stream has drained); collective like init. */
int32_t infr_cuda_ep_finalize(infr_cuda_ctx* ctx);
/* Time stamps of the last expert-parallel call's phases on this rank, in milliseconds from the
 * call's first kernel: [0] routing done, [1] dispatch received, [2] band experts done, [3] partials
 * received, [4] result written.  Waits for the stream.  The reference's analogue is the `[prof-moe]`
 * breakdown of crates/infr-cpu/src/lib.rs:4267-4285. */
int32_t infr_cuda_ep_last_phases(infr_cuda_ctx* ctx, float ms_out[5]);

/* ---- expert-parallel building blocks for hosts that run the exchange themselves ---------------- */

/* Expert FFN over rows that are already grouped by expert: rows [seg_off[e], seg_off[e+1]) of
 * `x_rows` go through local expert e (gate/up → SwiGLU → down) and land in the same rows of
 * `y_rows`.  This is what a rank runs between the dispatch and the combine exchange; the banks
 * hold only the rank's `n_local` experts.  `seg_off` is [n_local+1] i32 on the device.
 * x_rows / y_rows are f32 [n_rows, ne]. */
int32_t infr_cuda_moe_expert_rows(infr_cuda_ctx* ctx, const infr_cuda_buf* x_rows, const infr_cuda_buf* seg_off,
                                  const infr_cuda_buf* gate_exps, const infr_cuda_buf* up_exps,
                                  const infr_cuda_buf* down_exps, infr_cuda_buf* y_rows, uint32_t n_rows,
                                  uint32_t n_local, uint32_t ne, uint32_t n_ff_exp, int32_t gate_dtype,
                                  int32_t up_dtype, int32_t down_dtype);

/* The combine a rank runs after the return exchange (the reference sums band partials with an
 * all-reduce, crates/infr-vulkan/src/ep.rs:483-490; the fixed-order weighted sum is
 * shaders/moe_scatter_reduce.comp):  dst[t, :] = sum over ranks s (in rank order) of
 * wts[t, s] * y_rows[pos_of_pair[t*n_used + s], :]  (pairs with pos < 0 contribute nothing), then
 * + sigmoid(sh_logit[t]) * sh_rows[t, :]  (or + sh_rows[t, :] when sh_logit is NULL) when sh_rows
 * is given.  y_rows holds n_y_rows rows of ne f32; pos_of_pair is i32. */
int32_t infr_cuda_moe_combine(infr_cuda_ctx* ctx, const infr_cuda_buf* y_rows, const infr_cuda_buf* pos_of_pair,
                              const infr_cuda_buf* wts, const infr_cuda_buf* sh_rows, const infr_cuda_buf* sh_logit,
                              infr_cuda_buf* dst, uint32_t rows, uint32_t n_used, uint32_t ne, uint32_t n_y_rows);

/* ---- record once, replay (Backend::compile + the decode replay of the Vulkan backend) ----------- */

/* ---- GGUF ingest ------------------------------------------------------------------------------
 * The tensors of the path come out of a model file byte for byte, as the reference loads them
 * (parser crates/infr-gguf/src/lib.rs:745-870; tensor names crates/infr-llama/src/seam/runner.rs:
 * 2560-2595: blk.N.ffn_gate_inp.weight (router), ffn_gate_exps / ffn_up_exps / ffn_down_exps,
 * exp_probs_b.bias, ffn_gate_shexp / ffn_up_shexp / ffn_down_shexp, ffn_gate_inp_shexp).  GGUF
 * dimensions list the fastest axis first: an expert bank reads {in_f, out_f, n_expert}, which is
 * the [n_expert, out_f, in_f] row-major bank of the descriptor.  Versions 2 and 3, one file
 * (no split sets).  A malformed file is refused with a message in `err`. */
typedef struct infr_cuda_gguf infr_cuda_gguf; /* opaque: a mapped, parsed file */
typedef struct infr_cuda_gguf_tensor {
  int32_t dtype;     /* ggml type number (= INFR_CUDA_DT_* for the types the kernels take) */
  uint32_t n_dims;
  uint64_t dims[4];  /* ne[0] fastest; unused dimensions are 1 */
  uint64_t offset;   /* absolute byte offset in the file */
  uint64_t nbytes;   /* 0 when the type's block layout is not known to the reader */
} infr_cuda_gguf_tensor;
int32_t infr_cuda_gguf_open(const char* path, infr_cuda_gguf** out, char* err, size_t err_cap);
void infr_cuda_gguf_close(infr_cuda_gguf* g);
uint64_t infr_cuda_gguf_tensor_count(const infr_cuda_gguf* g);
/* The name of tensor `index` (names in sorted order): lets a host that opens the shards of a split model
 * (`<base>-NNNNN-of-MMMMM.gguf`, crates/infr-core/src/gguf_split.rs) check that no name appears twice. */
int32_t infr_cuda_gguf_tensor_name(const infr_cuda_gguf* g, uint64_t index, char* out, size_t cap);
/* INFR_CUDA_ERR_INVALID_ARG when there is no such tensor / key (or the key has another type). */
int32_t infr_cuda_gguf_find(const infr_cuda_gguf* g, const char* name, infr_cuda_gguf_tensor* out);
int32_t infr_cuda_gguf_meta_u64(const infr_cuda_gguf* g, const char* key, uint64_t* out);
int32_t infr_cuda_gguf_meta_f64(const infr_cuda_gguf* g, const char* key, double* out);
int32_t infr_cuda_gguf_meta_str(const infr_cuda_gguf* g, const char* key, char* out, size_t cap);
/* A new device buffer holding the tensor's bytes as stored (plus 16 spare bytes at the end). */
int32_t infr_cuda_gguf_upload(infr_cuda_ctx* ctx, const infr_cuda_gguf* g, const char* name, infr_cuda_buf** out);

/* The reference records a decode step's dispatches once and replays the command buffer per token
 * (`Capabilities::decode_replay`, crates/infr-core/src/backend.rs:45-236; graph built per forward in
 * crates/infr-llama/src/seam/runner.rs:12574-12796).  Here the calls issued between begin and end
 * are captured into a CUDA graph instead of being executed; `infr_cuda_graph_launch` replays them
 * on the context's stream.  Buffers named by the recorded calls must stay alive and keep their
 * addresses; new inputs are written into the same buffers before each replay.  Calls that need
 * to grow the context's scratch memory fail with INVALID_ARG while recording: run the same calls
 * once un-recorded first. */
typedef struct infr_cuda_graph infr_cuda_graph;
int32_t infr_cuda_graph_begin(infr_cuda_ctx* ctx);
int32_t infr_cuda_graph_end(infr_cuda_ctx* ctx, infr_cuda_graph** out);
int32_t infr_cuda_graph_launch(infr_cuda_ctx* ctx, infr_cuda_graph* graph);
void infr_cuda_graph_free(infr_cuda_ctx* ctx, infr_cuda_graph* graph);

/* ---- introspection for the test-suite and the benchmark ---------------------------------------- */

/* Checks the tensor-core building blocks of the grouped GEMM in isolation:
 * c[128, n] (f32) = a[128, 64] (f16) x b[n, 64]^T (f16) through 128-byte-swizzled shared-memory
 * tiles, tcgen05.mma and tensor memory; n a multiple of 16 in [16, 256].  Test aid, no reference
 * counterpart. */
int32_t infr_cuda_umma_selftest(infr_cuda_ctx* ctx, const infr_cuda_buf* a, const infr_cuda_buf* b, infr_cuda_buf* c, uint32_t n);
/* Number of kernel launches this context has issued since creation (host-side count). */
uint64_t infr_cuda_launch_count(const infr_cuda_ctx* ctx);
/* Attach (or with NULL detach) a 4096-byte device buffer into which the decode kernels write
 * phase time stamps: pairs of u64 (global timer in ns, SM cycle counter), 16 pairs per kernel in
 * the order router, gate/up, down.  A profiling aid for latency work; the reference's analogue is
 * the per-op `[prof-moe]` breakdown of crates/infr-cpu/src/lib.rs:4267-4285. */
int32_t infr_cuda_set_trace(infr_cuda_ctx* ctx, infr_cuda_buf* buf);

#ifdef __cplusplus
}
#endif
#endif /* INFR_CUDA_H */
