//! `infr-cuda`: a B200 (sm_100a) [`Backend`] for the ops of MoE4All's quantized mixture-of-experts
//! FFN path, over the C ABI of `libinfr_cuda.so` (`include/infr_cuda.h`).
//!
//! It covers exactly the ops the graph builder emits for a MoE FFN sub-layer
//! (`crates/infr-llama/src/seam/runner.rs:7999-8176`): [`Op::RmsNorm`], [`Op::MoeFfn`] (every field),
//! the shared expert's [`Op::Linear`] / [`Op::GatedAct`] / [`Op::MoeSharedExpertAdd`], and the residual
//! [`Op::Add`].  Any other op, dtype or shape is `Error::Unsupported` — there is no CPU fallback behind
//! this crate.  Weights are uploaded as the raw GGUF bytes the loader hands over (`Rewrite::Native`);
//! expert banks must be Q4_K (gate, up) and Q6_K or Q4_K (down), the router F32.
//!
//! Like the CPU and Vulkan backends, `compile` only stores the graph ([`GraphPlan`]); `execute`
//! walks the ops.  Tensors the graph declares `Internal` (or an `Output` the caller did not bind) are
//! allocated from a per-backend cache keyed by byte size and live until the backend is dropped.
//! Calls on the context are serialised by a mutex (the C ABI asks for that); all launches of one
//! `execute` are queued on the context's stream and `execute` returns after draining it, which is the
//! synchronous contract of `Backend::execute` (`backend.rs:907-908`).
//!
//! Expert parallelism: [`CudaBackend::join`] puts the context into an NCCL communicator
//! (`infr_cuda_ep_init`); after it an [`Op::MoeFfn`] whose `ep_band` is this rank's band runs as the
//! collective form of the op (tokens sharded, dispatch / combine inside the library), the counterpart
//! of `infr_vulkan::ExpertParallelBackend` (`crates/infr-vulkan/src/ep.rs:454-493`).
//!
//! NOTE: this crate has not been compiled in the environment it was written in (no Rust toolchain
//! there).  The C ABI it binds is exercised by the library's own test-suite.

mod ffi;

use std::any::Any;
use std::collections::HashMap;
use std::ffi::CStr;
use std::sync::{Arc, Mutex};

use infr_core::backend::{Backend, Bindings, Buffer, BufferUsage, Capabilities, GraphPlan, Plan};
use infr_core::decode_spec::block_spec;
use infr_core::error::{Error, Result};
use infr_core::graph::{Activation, Graph, MoeGating, Op, TensorId, TensorKind};
use infr_core::tensor::{DType, TensorDesc};

/// The context handle; dropped when the last buffer and the backend are gone.
struct Ctx {
    raw: *mut ffi::infr_cuda_ctx,
    /// The C ABI wants calls on one context serialised (`include/infr_cuda.h`, header comment).
    gate: Mutex<()>,
}

// The handle is only ever used under `gate`.
unsafe impl Send for Ctx {}
unsafe impl Sync for Ctx {}

impl Drop for Ctx {
    fn drop(&mut self) {
        unsafe { ffi::infr_cuda_destroy(self.raw) }
    }
}

impl Ctx {
    /// Status code -> the reference's error type (`crates/infr-core/src/error.rs:11-50`):
    /// UNSUPPORTED -> `Error::Unsupported`, everything else -> `Error::Backend`, with the library's text.
    fn check(&self, rc: i32) -> Result<()> {
        if rc == ffi::OK {
            return Ok(());
        }
        let msg = unsafe {
            let p = ffi::infr_cuda_last_error(self.raw);
            if p.is_null() { String::new() } else { CStr::from_ptr(p).to_string_lossy().into_owned() }
        };
        let class = match rc {
            ffi::ERR_INVALID_ARG => "invalid argument",
            ffi::ERR_UNSUPPORTED => "unsupported",
            ffi::ERR_OOM => "out of device memory",
            ffi::ERR_CUDA => "CUDA error",
            ffi::ERR_NCCL => "NCCL error",
            ffi::ERR_TIMEOUT => "device-side wait timed out",
            _ => "unknown status",
        };
        if rc == ffi::ERR_UNSUPPORTED {
            Err(Error::Unsupported(format!("infr-cuda: {msg}")))
        } else {
            Err(Error::backend(format!("infr-cuda ({class}): {msg}")))
        }
    }
}

/// One device allocation (`trait Buffer`, `backend.rs:423-452`).
pub struct CudaBuffer {
    ctx: Arc<Ctx>,
    raw: *mut ffi::infr_cuda_buf,
    len: usize,
}

unsafe impl Send for CudaBuffer {}
unsafe impl Sync for CudaBuffer {}

impl Buffer for CudaBuffer {
    fn len_bytes(&self) -> usize {
        self.len
    }
    fn as_any(&self) -> &dyn Any {
        self
    }
}

impl Drop for CudaBuffer {
    fn drop(&mut self) {
        let _g = self.ctx.gate.lock().unwrap_or_else(|e| e.into_inner());
        unsafe { ffi::infr_cuda_free(self.ctx.raw, self.raw) }
    }
}

fn cuda_buf(b: &dyn Buffer) -> Result<&CudaBuffer> {
    b.as_any()
        .downcast_ref::<CudaBuffer>()
        .ok_or_else(|| Error::backend("infr-cuda: a bound buffer was not allocated by this backend"))
}

pub struct CudaBackend {
    ctx: Arc<Ctx>,
    name: String,
    /// Backend-allocated tensors of past executes, by byte size (reused, never shrunk).
    scratch: Mutex<HashMap<usize, Vec<Arc<CudaBuffer>>>>,
    /// `Some((rank, world))` after [`CudaBackend::join`].
    ep: Mutex<Option<(u32, u32)>>,
}

impl CudaBackend {
    /// `infr_cuda_create`: fails with `Error::Unsupported` on a device that is not compute capability 10.x.
    pub fn new(device: i32) -> Result<Self> {
        let mut raw = std::ptr::null_mut();
        let rc = unsafe { ffi::infr_cuda_create(device, &mut raw) };
        if rc != ffi::OK || raw.is_null() {
            return Err(if rc == ffi::ERR_UNSUPPORTED {
                Error::Unsupported(format!("infr-cuda: device {device} is not an sm_100 GPU"))
            } else {
                Error::backend(format!("infr-cuda: infr_cuda_create(device {device}) failed with status {rc}"))
            });
        }
        let name = unsafe { CStr::from_ptr(ffi::infr_cuda_name()).to_string_lossy().into_owned() };
        // The grid tables of the codebook formats are this workspace's constants (`infr_core::iquant_grids`); the
        // library carries none and unpacks IQ2_XS / IQ2_S / IQ3_XXS / IQ3_S weights only after it has been given them.
        {
            use infr_core::iquant_grids::{IQ2S_GRID, IQ2XS_GRID, IQ3S_GRID, IQ3XXS_GRID};
            let tables: [(i32, &[u8]); 4] = [
                (ffi::DT_IQ2XS, bytemuck::cast_slice(&IQ2XS_GRID[..])),
                (ffi::DT_IQ2S, bytemuck::cast_slice(&IQ2S_GRID[..])),
                (ffi::DT_IQ3XXS, bytemuck::cast_slice(&IQ3XXS_GRID[..])),
                (ffi::DT_IQ3S, bytemuck::cast_slice(&IQ3S_GRID[..])),
            ];
            for (dt, bytes) in tables {
                let rc = unsafe { ffi::infr_cuda_set_codebook(raw, dt, bytes.as_ptr() as *const _, bytes.len()) };
                if rc != ffi::OK {
                    unsafe { ffi::infr_cuda_destroy(raw) };
                    return Err(Error::backend(format!("infr-cuda: infr_cuda_set_codebook(dtype {dt}) failed with status {rc}")));
                }
            }
        }
        Ok(Self { ctx: Arc::new(Ctx { raw, gate: Mutex::new(()) }), name, scratch: Mutex::new(HashMap::new()), ep: Mutex::new(None) })
    }

    /// The communicator id rank 0 creates and hands to the other ranks (`ncclGetUniqueId`).
    pub fn unique_id() -> Result<[u8; ffi::EP_ID_BYTES]> {
        let mut id = [0u8; ffi::EP_ID_BYTES];
        match unsafe { ffi::infr_cuda_ep_unique_id(id.as_mut_ptr()) } {
            ffi::OK => Ok(id),
            ffi::ERR_UNSUPPORTED => Err(Error::Unsupported("infr-cuda: libnccl.so.2 could not be loaded".into())),
            rc => Err(Error::backend(format!("infr-cuda: ncclGetUniqueId failed (status {rc})"))),
        }
    }

    /// Joins the expert-parallel communicator (collective over all ranks).  Afterwards an
    /// `Op::MoeFfn` whose `ep_band` is `(rank * n_expert / world, n_expert / world)` is the collective
    /// form of the op; every rank must execute the same graph with the same row count.
    pub fn join(&self, id: &[u8; ffi::EP_ID_BYTES], rank: u32, world: u32) -> Result<()> {
        let _g = self.lock();
        self.ctx.check(unsafe { ffi::infr_cuda_ep_init(self.ctx.raw, id.as_ptr(), rank as i32, world as i32) })?;
        *self.ep.lock().unwrap_or_else(|e| e.into_inner()) = Some((rank, world));
        Ok(())
    }

    /// Leaves the communicator (collective).
    pub fn leave(&self) -> Result<()> {
        let _g = self.lock();
        *self.ep.lock().unwrap_or_else(|e| e.into_inner()) = None;
        self.ctx.check(unsafe { ffi::infr_cuda_ep_finalize(self.ctx.raw) })
    }

    /// Host-paced plans: the steps of a decode loop are recorded once (`gated_upload`, the ops,
    /// `host_signal` per step, tickets 1, 2, ...) and launched once; per token the host then only writes the
    /// step's rows into the pinned staging range and calls `host_step` - no launch and no stream wait.
    /// `src` must be pinned host memory, 16-byte aligned, at most 256 KB.
    pub fn gated_upload(&self, dst: &CudaBuffer, src: *const u8, n: usize, ticket: u64) -> Result<()> {
        let _g = self.lock();
        self.ctx.check(unsafe { ffi::infr_cuda_upload_gated(self.ctx.raw, dst.raw, 0, src as *const _, n, ticket) })
    }

    pub fn host_signal(&self, ticket: u64) -> Result<()> {
        let _g = self.lock();
        self.ctx.check(unsafe { ffi::infr_cuda_host_signal(self.ctx.raw, ticket) })
    }

    /// Copy `rows` into the pinned staging range, ring `ticket`, wait (bounded) for its signal.  Not under the
    /// backend's lock: the pacing thread spins here while the recorded plan runs.
    pub fn host_step(&self, ticket: u64, stage: *mut u8, rows: &[u8]) -> Result<()> {
        self.ctx.check(unsafe { ffi::infr_cuda_host_step(self.ctx.raw, ticket, stage as *mut _, rows.as_ptr() as *const _, rows.len()) })
    }

    /// Drain the stream and set the pacing words back to zero (before a plan whose tickets start again at 1).
    pub fn host_reset(&self) -> Result<()> {
        let _g = self.lock();
        self.ctx.check(unsafe { ffi::infr_cuda_host_reset(self.ctx.raw) })
    }

    /// Tuning switches (`infr_cuda_config`), read - modify - write.
    pub fn configure(&self, f: impl FnOnce(&mut ffi::infr_cuda_config)) -> Result<()> {
        let _g = self.lock();
        let mut c = ffi::infr_cuda_config::default();
        self.ctx.check(unsafe { ffi::infr_cuda_get_config(self.ctx.raw, &mut c) })?;
        f(&mut c);
        self.ctx.check(unsafe { ffi::infr_cuda_set_config(self.ctx.raw, &c) })
    }

    fn lock(&self) -> std::sync::MutexGuard<'_, ()> {
        self.ctx.gate.lock().unwrap_or_else(|e| e.into_inner())
    }

    fn alloc_impl(&self, bytes: usize, zero: bool) -> Result<CudaBuffer> {
        let _g = self.lock();
        let mut raw = std::ptr::null_mut();
        // the C ABI rejects nothing about size 0 but hands back a null device pointer; keep one word
        self.ctx.check(unsafe { ffi::infr_cuda_alloc(self.ctx.raw, bytes.max(4), zero as i32, &mut raw) })?;
        Ok(CudaBuffer { ctx: self.ctx.clone(), raw, len: bytes })
    }

    /// A backend-owned tensor of `bytes` bytes for the current execute.
    fn take_scratch(&self, bytes: usize, held: &mut Vec<(usize, Arc<CudaBuffer>)>) -> Result<Arc<CudaBuffer>> {
        let cached = self.scratch.lock().unwrap_or_else(|e| e.into_inner()).get_mut(&bytes).and_then(|v| v.pop());
        let b = match cached {
            Some(b) => b,
            None => Arc::new(self.alloc_impl(bytes, true)?),
        };
        held.push((bytes, b.clone()));
        Ok(b)
    }
}

fn dt_code(dt: DType) -> Result<i32> {
    match dt {
        DType::F32 => Ok(ffi::DT_F32),
        DType::Q4K => Ok(ffi::DT_Q4K),
        DType::Q6K => Ok(ffi::DT_Q6K),
        DType::Q5K => Ok(ffi::DT_Q5K),
        DType::Q8_0 => Ok(ffi::DT_Q8_0),
        DType::Q4_0 => Ok(ffi::DT_Q4_0),
        DType::Q4_1 => Ok(ffi::DT_Q4_1),
        DType::Q5_0 => Ok(ffi::DT_Q5_0),
        DType::Q5_1 => Ok(ffi::DT_Q5_1),
        DType::Q2K => Ok(ffi::DT_Q2K),
        DType::Q3K => Ok(ffi::DT_Q3K),
        DType::Iq4Nl => Ok(ffi::DT_IQ4NL),
        DType::Iq4Xs => Ok(ffi::DT_IQ4XS),
        DType::Mxfp4 => Ok(ffi::DT_MXFP4),
        DType::Nvfp4 => Ok(ffi::DT_NVFP4),
        DType::Q2_0 => Ok(ffi::DT_Q2_0),
        DType::Iq2Xs => Ok(ffi::DT_IQ2XS),
        DType::Iq2S => Ok(ffi::DT_IQ2S),
        DType::Iq3Xxs => Ok(ffi::DT_IQ3XXS),
        DType::Iq3S => Ok(ffi::DT_IQ3S),
        other => Err(Error::Unsupported(format!("infr-cuda: weight dtype {other:?} has no sm_100a kernel"))),
    }
}

fn tensor_bytes(desc: &TensorDesc) -> usize {
    match desc.dtype {
        DType::F32 | DType::I32 | DType::U32 => desc.numel() * 4,
        DType::F16 | DType::Bf16 => desc.numel() * 2,
        dt => block_spec(dt).nbytes(desc.numel()),
    }
}

fn act_code(a: Activation) -> u32 {
    match a {
        Activation::Silu => 0,
        Activation::Gelu => 1,
        Activation::Sigmoid => 2,
        #[allow(unreachable_patterns)]
        _ => u32::MAX, // refused by the library as an unknown activation
    }
}

fn gating_code(g: MoeGating) -> u32 {
    match g {
        MoeGating::Softmax => 0,
        MoeGating::Sigmoid => 1,
        MoeGating::SqrtSoftplus => 2,
    }
}

/// Resolves graph handles to device buffers for one execute: bound ones from `Bindings`, the rest
/// from the backend's scratch cache.
struct Resolver<'a, 'b> {
    be: &'a CudaBackend,
    g: &'a Graph,
    bindings: &'a Bindings<'b>,
    own: HashMap<u32, Arc<CudaBuffer>>,
    held: Vec<(usize, Arc<CudaBuffer>)>,
}

impl<'a, 'b> Resolver<'a, 'b> {
    fn get(&mut self, id: TensorId) -> Result<*mut ffi::infr_cuda_buf> {
        if let Some(b) = self.bindings.get(id) {
            return Ok(cuda_buf(b)?.raw);
        }
        if let Some(b) = self.own.get(&id.0) {
            return Ok(b.raw);
        }
        match self.g.kind(id) {
            TensorKind::Internal | TensorKind::Output => {
                let bytes = tensor_bytes(self.g.desc(id));
                let b = self.be.take_scratch(bytes, &mut self.held)?;
                let raw = b.raw;
                self.own.insert(id.0, b);
                Ok(raw)
            }
            kind => Err(Error::backend(format!("infr-cuda: tensor {} ({kind:?}) is not bound", id.0))),
        }
    }
    fn opt(&mut self, id: Option<TensorId>) -> Result<*const ffi::infr_cuda_buf> {
        Ok(match id {
            Some(id) => self.get(id)? as *const _,
            None => std::ptr::null(),
        })
    }
}

impl Backend for CudaBackend {
    fn name(&self) -> &str {
        &self.name
    }

    fn capabilities(&self) -> Capabilities {
        // Everything optional stays at its default (off): this backend advertises no fused or
        // replayed forms to the graph compiler beyond the ops it executes.
        Capabilities { name: self.name.clone(), ..Default::default() }
    }

    /// Zero-initialised (the calloc contract of `backend.rs:647-651`).
    fn alloc(&self, bytes: usize, _usage: BufferUsage) -> Result<Box<dyn Buffer>> {
        Ok(Box::new(self.alloc_impl(bytes, true)?))
    }

    fn alloc_uninit(&self, bytes: usize, _usage: BufferUsage) -> Result<Box<dyn Buffer>> {
        Ok(Box::new(self.alloc_impl(bytes, false)?))
    }

    /// Prefix copy; a source longer than the buffer is an error, not a panic (`backend.rs:22-33`).
    fn upload(&self, dst: &dyn Buffer, src: &[u8]) -> Result<()> {
        let d = cuda_buf(dst)?;
        if src.len() > d.len {
            return Err(Error::backend(format!("infr-cuda: upload of {} bytes into a buffer of {}", src.len(), d.len)));
        }
        let _g = self.lock();
        self.ctx.check(unsafe { ffi::infr_cuda_upload(self.ctx.raw, d.raw, 0, src.as_ptr().cast(), src.len()) })
    }

    fn download(&self, src: &dyn Buffer, dst: &mut [u8]) -> Result<()> {
        let s = cuda_buf(src)?;
        if dst.len() > s.len {
            return Err(Error::backend(format!("infr-cuda: download of {} bytes from a buffer of {}", dst.len(), s.len)));
        }
        let _g = self.lock();
        self.ctx.check(unsafe { ffi::infr_cuda_download(self.ctx.raw, s.raw, 0, dst.as_mut_ptr().cast(), dst.len()) })
    }

    fn compile(&self, graph: &Graph) -> Result<Box<dyn Plan>> {
        // refuse at compile time what execute could not run, so a model loader learns it early
        for op in &graph.ops {
            match op {
                Op::MoeFfn { .. } | Op::Linear { .. } | Op::GatedAct { .. } | Op::MoeSharedExpertAdd { .. } | Op::RmsNorm { .. } | Op::Add { .. } => {}
                other => return Err(Error::Unsupported(format!("infr-cuda: op {} is outside the MoE FFN path this backend covers", other.kind()))),
            }
        }
        Ok(GraphPlan::boxed(graph))
    }

    fn execute(&self, plan: &dyn Plan, bindings: &Bindings) -> Result<()> {
        let g = &plan
            .as_any()
            .downcast_ref::<GraphPlan>()
            .ok_or_else(|| Error::backend("infr-cuda: plan was not compiled by this backend"))?
            .graph;
        let ep = *self.ep.lock().unwrap_or_else(|e| e.into_inner());
        let mut r = Resolver { be: self, g, bindings, own: HashMap::new(), held: Vec::new() };
        let run = (|| -> Result<()> {
            for op in &g.ops {
                match *op {
                    Op::RmsNorm { x, weight, dst, rows, dim, eps } => {
                        let (x, w, d) = (r.get(x)?, r.get(weight)?, r.get(dst)?);
                        let _l = self.lock();
                        self.ctx.check(unsafe { ffi::infr_cuda_rmsnorm(self.ctx.raw, x, w, d, rows, dim, eps) })?;
                    }
                    Op::Add { a, b, dst, n } => {
                        let (a, b, d) = (r.get(a)?, r.get(b)?, r.get(dst)?);
                        let _l = self.lock();
                        self.ctx.check(unsafe { ffi::infr_cuda_add(self.ctx.raw, a, b, d, n as usize) })?;
                    }
                    Op::Linear { x, weight, dst, m, in_f, out_f, w_off } => {
                        if w_off != 0 {
                            return Err(Error::Unsupported("infr-cuda: Linear with a weight offset (fused QKV) is outside the MoE FFN path".into()));
                        }
                        let dt = dt_code(g.desc(weight).dtype)?;
                        let (x, w, d) = (r.get(x)?, r.get(weight)?, r.get(dst)?);
                        let _l = self.lock();
                        self.ctx.check(unsafe { ffi::infr_cuda_linear(self.ctx.raw, dt, w, x, d, m, in_f, out_f) })?;
                    }
                    Op::GatedAct { gate, up, dst, rows, nff, act, up_off, up_stride, gate_stride, gate_block_width, swiglu_clamp, .. } => {
                        // the shared expert's form: contiguous gate and up, SiLU, no clamp
                        let contiguous = up_off == 0 && (up_stride == 0 || up_stride == nff) && (gate_stride == 0 || gate_stride == nff) && gate_block_width == 0;
                        if !contiguous || !matches!(act, Activation::Silu) || swiglu_clamp.is_some() {
                            return Err(Error::Unsupported("infr-cuda: GatedAct is covered in its contiguous SiLU form only".into()));
                        }
                        let (gt, u, d) = (r.get(gate)?, r.get(up)?, r.get(dst)?);
                        let _l = self.lock();
                        self.ctx.check(unsafe { ffi::infr_cuda_gated_act(self.ctx.raw, gt, u, d, rows as usize * nff as usize) })?;
                    }
                    Op::MoeSharedExpertAdd { moe, shexp, gate, dst, rows, n } => {
                        let (m, s, gt, d) = (r.get(moe)?, r.get(shexp)?, r.get(gate)?, r.get(dst)?);
                        let _l = self.lock();
                        self.ctx.check(unsafe { ffi::infr_cuda_moe_shared_add(self.ctx.raw, m, s, gt, d, rows, n) })?;
                    }
                    Op::MoeFfn {
                        x, router_x, router, gate_exps, up_exps, down_exps, down_scale, fused_gate_up, dst, ne, n_expert, n_used, n_ff_exp,
                        scale, act, swiglu_clamp, gating, norm_w, weight_before, ep_band, exp_probs_b, n_expert_groups, n_expert_groups_used,
                        expert_ids,
                    } => {
                        // `x` may hold several rows (`infr-cpu/src/lib.rs:3643-3647`): rows = numel / ne
                        let rows = (g.desc(x).numel() / ne as usize) as u32;
                        let mut d = ffi::infr_cuda_moe_ffn_desc::default();
                        d.x = r.get(x)?;
                        d.router_x = r.get(router_x)?;
                        d.router = r.get(router)?;
                        d.gate_exps = r.get(gate_exps)?;
                        d.up_exps = if fused_gate_up { d.gate_exps } else { r.get(up_exps)? };
                        d.down_exps = r.get(down_exps)?;
                        d.exp_probs_b = r.opt(exp_probs_b)?;
                        d.dst = r.get(dst)?;
                        d.rows = rows;
                        d.ne = ne;
                        d.n_expert = n_expert;
                        d.n_used = n_used;
                        d.n_ff_exp = n_ff_exp;
                        d.scale = scale;
                        d.router_dtype = dt_code(g.desc(router).dtype)?;
                        d.gate_dtype = dt_code(g.desc(gate_exps).dtype)?;
                        d.up_dtype = if fused_gate_up { d.gate_dtype } else { dt_code(g.desc(up_exps).dtype)? };
                        d.down_dtype = dt_code(g.desc(down_exps).dtype)?;
                        d.gating = gating_code(gating);
                        d.norm_w = norm_w as u32;
                        d.n_expert_groups = n_expert_groups;
                        d.n_expert_groups_used = n_expert_groups_used;
                        if let Some((lo, n_local)) = ep_band {
                            // On a joined context this rank's band makes the call collective (banks hold the band
                            // only, as the reference's EP lowering leaves them, `graph.rs:1309-1319`).  A band on an
                            // un-joined context has no partner to sum the partials: refuse rather than return one.
                            match ep {
                                Some((rank, world)) if n_expert % world == 0 && lo == rank * (n_expert / world) && n_local == n_expert / world => {}
                                _ => return Err(Error::Unsupported("infr-cuda: ep_band needs a context that has joined a communicator, and this rank's own band".into())),
                            }
                            d.ep_lo = lo;
                            d.ep_n_local = n_local;
                        }
                        d.expert_ids = r.opt(expert_ids)?;
                        d.down_scale = r.opt(down_scale)?;
                        d.act = act_code(act);
                        d.weight_before = weight_before as u32;
                        d.swiglu_clamp = swiglu_clamp.unwrap_or(0.0);
                        d.fused_gate_up = fused_gate_up as u32;
                        let _l = self.lock();
                        self.ctx.check(unsafe { ffi::infr_cuda_moe_ffn(self.ctx.raw, &d) })?;
                    }
                    ref other => {
                        return Err(Error::Unsupported(format!("infr-cuda: op {} is outside the MoE FFN path this backend covers", other.kind())));
                    }
                }
            }
            Ok(())
        })();
        // drain before the scratch tensors go back to the cache (and to honour the synchronous contract);
        // device-side failures (a bounded wait that ran out, a bad expert id) surface here
        let drained = {
            let _l = self.lock();
            self.ctx.check(unsafe { ffi::infr_cuda_sync(self.ctx.raw) })
        };
        let mut cache = self.scratch.lock().unwrap_or_else(|e| e.into_inner());
        for (bytes, b) in r.held.drain(..) {
            cache.entry(bytes).or_default().push(b);
        }
        run.and(drained)
    }

    fn sync(&self) -> Result<()> {
        let _g = self.lock();
        self.ctx.check(unsafe { ffi::infr_cuda_sync(self.ctx.raw) })
    }
}
