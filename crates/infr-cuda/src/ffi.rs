//! Raw bindings of `include/infr_cuda.h`.  Field order and types follow the header exactly; the
//! header is the source of truth.
#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_void};

#[repr(C)]
pub struct infr_cuda_ctx {
    _p: [u8; 0],
}
#[repr(C)]
pub struct infr_cuda_buf {
    _p: [u8; 0],
}
#[repr(C)]
pub struct infr_cuda_graph {
    _p: [u8; 0],
}

pub const OK: i32 = 0;
pub const ERR_INVALID_ARG: i32 = -1;
pub const ERR_UNSUPPORTED: i32 = -2;
pub const ERR_OOM: i32 = -3;
pub const ERR_CUDA: i32 = -4;
pub const ERR_NCCL: i32 = -5;
pub const ERR_TIMEOUT: i32 = -6;

pub const DT_F32: i32 = 0;
pub const DT_Q4K: i32 = 12;
pub const DT_Q6K: i32 = 14;
pub const DT_Q8_0: i32 = 8;
pub const DT_Q5K: i32 = 13;
pub const DT_Q4_0: i32 = 2;
pub const DT_Q4_1: i32 = 3;
pub const DT_Q5_0: i32 = 6;
pub const DT_Q5_1: i32 = 7;
pub const DT_Q2K: i32 = 10;
pub const DT_Q3K: i32 = 11;
pub const DT_IQ4NL: i32 = 20;
pub const DT_IQ4XS: i32 = 23;
pub const DT_MXFP4: i32 = 39;
pub const DT_NVFP4: i32 = 40;
pub const DT_Q2_0: i32 = 42;
pub const DT_IQ2XS: i32 = 17;
pub const DT_IQ3XXS: i32 = 18;
pub const DT_IQ3S: i32 = 21;
pub const DT_IQ2S: i32 = 22;

pub const EP_ID_BYTES: usize = 128;

#[repr(C)]
#[derive(Clone, Copy)]
pub struct infr_cuda_moe_ffn_desc {
    pub x: *const infr_cuda_buf,
    pub router_x: *const infr_cuda_buf,
    pub router: *const infr_cuda_buf,
    pub gate_exps: *const infr_cuda_buf,
    pub up_exps: *const infr_cuda_buf,
    pub down_exps: *const infr_cuda_buf,
    pub exp_probs_b: *const infr_cuda_buf,
    pub dst: *mut infr_cuda_buf,
    pub ids_out: *mut infr_cuda_buf,
    pub wts_out: *mut infr_cuda_buf,
    pub rows: u32,
    pub ne: u32,
    pub n_expert: u32,
    pub n_used: u32,
    pub n_ff_exp: u32,
    pub scale: f32,
    pub router_dtype: i32,
    pub gate_dtype: i32,
    pub up_dtype: i32,
    pub down_dtype: i32,
    pub gating: u32,
    pub norm_w: u32,
    pub n_expert_groups: u32,
    pub n_expert_groups_used: u32,
    pub ep_lo: u32,
    pub ep_n_local: u32,
    pub sh_gate: *const infr_cuda_buf,
    pub sh_up: *const infr_cuda_buf,
    pub sh_down: *const infr_cuda_buf,
    pub sh_gate_inp: *const infr_cuda_buf,
    pub sh_ff: u32,
    pub path: u32,
    pub norm_weight: *const infr_cuda_buf,
    pub residual: *const infr_cuda_buf,
    pub norm_eps: f32,
    pub stages: u32,
    pub expert_ids: *const infr_cuda_buf,
    pub down_scale: *const infr_cuda_buf,
    pub act: u32,
    pub weight_before: u32,
    pub swiglu_clamp: f32,
    pub fused_gate_up: u32,
}

impl Default for infr_cuda_moe_ffn_desc {
    fn default() -> Self {
        // all-zero is the header's "nothing optional set" state (null pointers, zero sizes)
        unsafe { std::mem::zeroed() }
    }
}

#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct infr_cuda_config {
    pub gu_warps: u32,
    pub gu_chunks: u32,
    pub dn_warps: u32,
    pub upload_by_copy: u32,
    pub trace_tile: u32,
    pub expert_major: u32,
    pub sync_timeout_ms: u32,
    pub raw_rows_f32: u32,
    pub gate_timeout_ms: u32,
    pub reserved: [u32; 7],
}

extern "C" {
    pub fn infr_cuda_create(device: i32, out: *mut *mut infr_cuda_ctx) -> i32;
    pub fn infr_cuda_destroy(ctx: *mut infr_cuda_ctx);
    pub fn infr_cuda_last_error(ctx: *const infr_cuda_ctx) -> *const c_char;
    pub fn infr_cuda_name() -> *const c_char;
    pub fn infr_cuda_set_stream(ctx: *mut infr_cuda_ctx, cuda_stream: *mut c_void) -> i32;
    pub fn infr_cuda_get_config(ctx: *const infr_cuda_ctx, out: *mut infr_cuda_config) -> i32;
    pub fn infr_cuda_set_config(ctx: *mut infr_cuda_ctx, cfg: *const infr_cuda_config) -> i32;
    pub fn infr_cuda_set_codebook(ctx: *mut infr_cuda_ctx, dtype: i32, table: *const c_void, bytes: usize) -> i32;

    pub fn infr_cuda_alloc(ctx: *mut infr_cuda_ctx, bytes: usize, zero: i32, out: *mut *mut infr_cuda_buf) -> i32;
    pub fn infr_cuda_wrap(ctx: *mut infr_cuda_ctx, device_ptr: *mut c_void, bytes: usize, out: *mut *mut infr_cuda_buf) -> i32;
    pub fn infr_cuda_free(ctx: *mut infr_cuda_ctx, buf: *mut infr_cuda_buf);
    pub fn infr_cuda_buf_len(buf: *const infr_cuda_buf) -> usize;
    pub fn infr_cuda_buf_ptr(buf: *const infr_cuda_buf) -> *mut c_void;
    pub fn infr_cuda_upload(ctx: *mut infr_cuda_ctx, dst: *mut infr_cuda_buf, dst_off: usize, src: *const c_void, n: usize) -> i32;
    pub fn infr_cuda_download(ctx: *mut infr_cuda_ctx, src: *const infr_cuda_buf, src_off: usize, dst: *mut c_void, n: usize) -> i32;
    pub fn infr_cuda_upload_async(ctx: *mut infr_cuda_ctx, dst: *mut infr_cuda_buf, dst_off: usize, src: *const c_void, n: usize) -> i32;
    pub fn infr_cuda_download_async(ctx: *mut infr_cuda_ctx, src: *const infr_cuda_buf, src_off: usize, dst: *mut c_void, n: usize) -> i32;
    pub fn infr_cuda_upload_gated(ctx: *mut infr_cuda_ctx, dst: *mut infr_cuda_buf, dst_off: usize, src: *const c_void, n: usize, ticket: u64) -> i32;
    pub fn infr_cuda_host_signal(ctx: *mut infr_cuda_ctx, ticket: u64) -> i32;
    pub fn infr_cuda_host_ring(ctx: *mut infr_cuda_ctx, ticket: u64) -> i32;
    pub fn infr_cuda_host_await(ctx: *mut infr_cuda_ctx, ticket: u64) -> i32;
    pub fn infr_cuda_host_reset(ctx: *mut infr_cuda_ctx) -> i32;
    pub fn infr_cuda_host_steps(ctx: *mut infr_cuda_ctx, first_ticket: u64, count: u32, stage: *mut c_void, rows: *const *const c_void, n_in: usize, result: *const c_void, results_out: *const *mut c_void, n_out: usize) -> i32;
    pub fn infr_cuda_host_step(ctx: *mut infr_cuda_ctx, ticket: u64, stage: *mut c_void, rows: *const c_void, n: usize) -> i32;
    pub fn infr_cuda_sync(ctx: *mut infr_cuda_ctx) -> i32;

    pub fn infr_cuda_moe_ffn(ctx: *mut infr_cuda_ctx, desc: *const infr_cuda_moe_ffn_desc) -> i32;
    pub fn infr_cuda_moe_route(ctx: *mut infr_cuda_ctx, desc: *const infr_cuda_moe_ffn_desc) -> i32;
    pub fn infr_cuda_linear(ctx: *mut infr_cuda_ctx, dtype: i32, w: *const infr_cuda_buf, x: *const infr_cuda_buf,
                            y: *mut infr_cuda_buf, m: u32, in_f: u32, out_f: u32) -> i32;
    pub fn infr_cuda_gated_act(ctx: *mut infr_cuda_ctx, gate: *const infr_cuda_buf, up: *const infr_cuda_buf,
                               dst: *mut infr_cuda_buf, n: usize) -> i32;
    pub fn infr_cuda_moe_shared_add(ctx: *mut infr_cuda_ctx, moe: *const infr_cuda_buf, shexp: *const infr_cuda_buf,
                                    gate: *const infr_cuda_buf, dst: *mut infr_cuda_buf, rows: u32, n: u32) -> i32;
    pub fn infr_cuda_rmsnorm(ctx: *mut infr_cuda_ctx, x: *const infr_cuda_buf, weight: *const infr_cuda_buf,
                             dst: *mut infr_cuda_buf, rows: u32, dim: u32, eps: f32) -> i32;
    pub fn infr_cuda_add(ctx: *mut infr_cuda_ctx, a: *const infr_cuda_buf, b: *const infr_cuda_buf, dst: *mut infr_cuda_buf, n: usize) -> i32;

    pub fn infr_cuda_ep_unique_id(id: *mut u8) -> i32;
    pub fn infr_cuda_ep_init(ctx: *mut infr_cuda_ctx, id: *const u8, rank: i32, world: i32) -> i32;
    pub fn infr_cuda_ep_finalize(ctx: *mut infr_cuda_ctx) -> i32;
    pub fn infr_cuda_ep_last_phases(ctx: *mut infr_cuda_ctx, ms_out: *mut f32) -> i32;

    pub fn infr_cuda_graph_begin(ctx: *mut infr_cuda_ctx) -> i32;
    pub fn infr_cuda_graph_end(ctx: *mut infr_cuda_ctx, out: *mut *mut infr_cuda_graph) -> i32;
    pub fn infr_cuda_graph_launch(ctx: *mut infr_cuda_ctx, graph: *mut infr_cuda_graph) -> i32;
    pub fn infr_cuda_graph_free(ctx: *mut infr_cuda_ctx, graph: *mut infr_cuda_graph);
    pub fn infr_cuda_launch_count(ctx: *const infr_cuda_ctx) -> u64;
}
