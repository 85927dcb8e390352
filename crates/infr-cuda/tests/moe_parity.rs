//! Op-level parity of `infr-cuda` against `infr-cpu` in reference mode, in the style of
//! `crates/infr-llama/tests/seam_op_parity.rs` (graph built by hand, one op, bound raw bytes) and with
//! the harness of `crates/infr-testkit` (`synth_weight`, `gen_f32`, `run_graph`, the `rel` metric of
//! `src/lib.rs:372-386`).  Needs a B200; self-skips when `CudaBackend::new(0)` is unsupported, the way
//! the reference's GPU tests do (`#[ignore]`d in CI, `.github/workflows/ci.yml:17-25`).
//!
//! Bound: expert ids bit-exact (observed through the outputs: a different expert changes the row by
//! far more than the tolerance), layer outputs within 2e-3 of the reference's maximum.
//!
//! NOTE: written without a Rust toolchain at hand; never compiled.

use infr_core::backend::Backend;
use infr_core::graph::{Activation, Graph, MoeGating, Op, TensorId};
use infr_core::tensor::{DType, TensorDesc};
use infr_testkit::{gen_f32, run_graph, synth_weight};

const TOL: f32 = 2e-3;

fn f32d(n: usize) -> TensorDesc {
    TensorDesc::new(vec![n], DType::F32)
}
fn qd(n: usize, dt: DType) -> TensorDesc {
    TensorDesc::new(vec![n], dt)
}
fn bytes_of(v: &[f32]) -> Vec<u8> {
    bytemuck::cast_slice(v).to_vec()
}

/// `rel = max|got - want| / max(max|want|, 1e-3)`; an all-zero oracle is a failure, not a pass
/// (`crates/infr-testkit/src/lib.rs:250-253, 372-386`).
fn rel(got: &[f32], want: &[f32]) -> f32 {
    let mag = want.iter().fold(0f32, |m, v| m.max(v.abs()));
    assert!(mag > 0.0, "oracle output is all zero: the case is vacuous");
    let err = got.iter().zip(want).fold(0f32, |m, (a, b)| m.max((a - b).abs()));
    err / mag.max(1e-3)
}

fn gpu() -> Option<infr_cuda::CudaBackend> {
    infr_cuda::CudaBackend::new(0).ok()
}

struct Case {
    rows: usize,
    ne: usize,
    n_expert: usize,
    n_used: usize,
    n_ff: usize,
    gating: MoeGating,
    groups: (u32, u32),
    bias: bool,
    down: DType,
    /// format of the gate and up banks
    gu: DType,
}

fn moe_case(c: &Case) -> (Graph, Vec<(TensorId, Vec<u8>)>, TensorId) {
    let mut g = Graph::new();
    let x = g.input(f32d(c.rows * c.ne));
    let router = g.weight(f32d(c.n_expert * c.ne));
    let gate = g.weight(qd(c.n_expert * c.n_ff * c.ne, c.gu));
    let up = g.weight(qd(c.n_expert * c.n_ff * c.ne, c.gu));
    let down = g.weight(qd(c.n_expert * c.ne * c.n_ff, c.down));
    let bias = if c.bias { Some(g.weight(f32d(c.n_expert))) } else { None };
    let dst = g.output(f32d(c.rows * c.ne));
    g.push(Op::MoeFfn {
        x,
        router_x: x,
        router,
        gate_exps: gate,
        up_exps: up,
        down_exps: down,
        down_scale: None,
        fused_gate_up: false,
        dst,
        ne: c.ne as u32,
        n_expert: c.n_expert as u32,
        n_used: c.n_used as u32,
        n_ff_exp: c.n_ff as u32,
        scale: 1.0,
        act: Activation::Silu,
        swiglu_clamp: None,
        gating: c.gating,
        norm_w: true,
        weight_before: false,
        ep_band: None,
        exp_probs_b: bias,
        n_expert_groups: c.groups.0,
        n_expert_groups_used: c.groups.1,
        expert_ids: None,
    });
    // router rows with well separated logits: gen_f32 is a 29-periodic sawtooth, so scale it per expert
    let mut r = gen_f32(c.n_expert * c.ne, 3);
    for (e, row) in r.chunks_mut(c.ne).enumerate() {
        let s = 0.02 * (1.0 + (e as f32) * 0.37 % 1.0);
        row.iter_mut().for_each(|v| *v *= s);
    }
    let mut bound = vec![
        (x, bytes_of(&gen_f32(c.rows * c.ne, 1))),
        (router, bytes_of(&r)),
        (gate, synth_weight(c.gu, c.n_expert * c.n_ff * c.ne, 11)),
        (up, synth_weight(c.gu, c.n_expert * c.n_ff * c.ne, 12)),
        (down, synth_weight(c.down, c.n_expert * c.ne * c.n_ff, 13)),
    ];
    if let Some(b) = bias {
        bound.push((b, bytes_of(&gen_f32(c.n_expert, 5).iter().map(|v| v * 0.1).collect::<Vec<_>>())));
    }
    (g, bound, dst)
}

fn check(c: Case, what: &str) {
    let Some(gpu) = gpu() else {
        eprintln!("{what}: no sm_100 device, skipped");
        return;
    };
    let cpu = infr_cpu::CpuBackend::reference();
    let (g, bound, dst) = moe_case(&c);
    let want = run_graph(&cpu, &g, &bound, dst, c.rows * c.ne);
    let got = run_graph(&gpu, &g, &bound, dst, c.rows * c.ne);
    let e = rel(&got, &want);
    println!("{what}: cuda-vs-cpu(reference) rel={e:e}");
    assert!(e <= TOL, "{what}: rel err {e:e} > {TOL:e}");
}

#[test]
fn moe_decode_rows_1_and_4() {
    for rows in [1usize, 4] {
        check(
            Case { rows, ne: 512, n_expert: 16, n_used: 4, n_ff: 256, gating: MoeGating::Softmax, groups: (0, 0), bias: false, down: DType::Q6K, gu: DType::Q4K },
            &format!("MoeFfn decode rows={rows}"),
        );
    }
}

#[test]
fn moe_batched_rows_96() {
    check(
        Case { rows: 96, ne: 512, n_expert: 16, n_used: 4, n_ff: 256, gating: MoeGating::Softmax, groups: (0, 0), bias: false, down: DType::Q6K, gu: DType::Q4K },
        "MoeFfn batched rows=96 (grouped GEMM on tcgen05)",
    );
}

#[test]
fn moe_sigmoid_groups_bias() {
    check(
        Case { rows: 3, ne: 512, n_expert: 32, n_used: 4, n_ff: 256, gating: MoeGating::Sigmoid, groups: (4, 2), bias: true, down: DType::Q6K, gu: DType::Q4K },
        "MoeFfn sigmoid gating, 4 groups / 2 used, selection bias",
    );
}

#[test]
fn moe_sqrt_softplus_and_q4k_down() {
    check(
        Case { rows: 2, ne: 512, n_expert: 16, n_used: 2, n_ff: 256, gating: MoeGating::SqrtSoftplus, groups: (0, 0), bias: false, down: DType::Q4K, gu: DType::Q4K },
        "MoeFfn sqrt-softplus gating, Q4_K down bank",
    );
}

/// Other bank formats real files mix in (`crates/infr-core/src/tensor.rs:172-196`): Q5_K gate/up with a
/// Q6_K down bank, Q8_0 throughout, and the two non-linear 4-bit formats, on the small-m kernels and on the
/// grouped GEMM tiles.
#[test]
fn moe_q5k_and_q8_0_banks() {
    for (gu, down, name) in [
        (DType::Q5K, DType::Q6K, "Q5_K / Q6_K"),
        (DType::Q8_0, DType::Q8_0, "Q8_0"),
        (DType::Iq4Xs, DType::Iq4Nl, "IQ4_XS / IQ4_NL"),
        // grid codebook formats: the backend was given this workspace's grid tables when it was created
        (DType::Iq2Xs, DType::Iq3S, "IQ2_XS / IQ3_S"),
        (DType::Iq3Xxs, DType::Iq2S, "IQ3_XXS / IQ2_S"),
    ] {
        for rows in [1usize, 4, 96] {
            check(
                Case { rows, ne: 512, n_expert: 16, n_used: 4, n_ff: 256, gating: MoeGating::Softmax, groups: (0, 0), bias: false, down, gu },
                &format!("MoeFfn {name} banks rows={rows}"),
            );
        }
    }
}

/// The whole FFN sub-layer as the graph builder emits it for qwen35moe
/// (`crates/infr-llama/src/seam/runner.rs:7999-8176`): RmsNorm, MoeFfn, the shared expert as
/// Linear / Linear / GatedAct / Linear with its one-logit gate, MoeSharedExpertAdd, residual Add.
#[test]
fn moe_sublayer_with_shared_expert() {
    let Some(gpu) = gpu() else {
        eprintln!("sub-layer: no sm_100 device, skipped");
        return;
    };
    let cpu = infr_cpu::CpuBackend::reference();
    let (rows, ne, n_expert, n_used, n_ff) = (2usize, 512usize, 16usize, 4usize, 256usize);
    let mut g = Graph::new();
    let hidden = g.input(f32d(rows * ne));
    let nw = g.weight(f32d(ne));
    let router = g.weight(f32d(n_expert * ne));
    let gate = g.weight(qd(n_expert * n_ff * ne, DType::Q4K));
    let up = g.weight(qd(n_expert * n_ff * ne, DType::Q4K));
    let down = g.weight(qd(n_expert * ne * n_ff, DType::Q6K));
    let sh_gate_inp = g.weight(f32d(ne));
    let sh_gate = g.weight(qd(n_ff * ne, DType::Q4K));
    let sh_up = g.weight(qd(n_ff * ne, DType::Q4K));
    let sh_down = g.weight(qd(ne * n_ff, DType::Q6K));
    let hn = g.internal(f32d(rows * ne));
    let moe = g.internal(f32d(rows * ne));
    let gl = g.internal(f32d(rows));
    let sg = g.internal(f32d(rows * n_ff));
    let su = g.internal(f32d(rows * n_ff));
    let sa = g.internal(f32d(rows * n_ff));
    let sd = g.internal(f32d(rows * ne));
    let sub = g.internal(f32d(rows * ne));
    let out = g.output(f32d(rows * ne));
    g.push(Op::RmsNorm { x: hidden, weight: nw, dst: hn, rows: rows as u32, dim: ne as u32, eps: 1e-6 });
    g.push(Op::MoeFfn {
        x: hn, router_x: hn, router, gate_exps: gate, up_exps: up, down_exps: down, down_scale: None, fused_gate_up: false, dst: moe,
        ne: ne as u32, n_expert: n_expert as u32, n_used: n_used as u32, n_ff_exp: n_ff as u32, scale: 1.0, act: Activation::Silu,
        swiglu_clamp: None, gating: MoeGating::Softmax, norm_w: true, weight_before: false, ep_band: None, exp_probs_b: None,
        n_expert_groups: 0, n_expert_groups_used: 0, expert_ids: None,
    });
    g.push(Op::Linear { x: hn, weight: sh_gate_inp, dst: gl, m: rows as u32, in_f: ne as u32, out_f: 1, w_off: 0 });
    g.push(Op::Linear { x: hn, weight: sh_gate, dst: sg, m: rows as u32, in_f: ne as u32, out_f: n_ff as u32, w_off: 0 });
    g.push(Op::Linear { x: hn, weight: sh_up, dst: su, m: rows as u32, in_f: ne as u32, out_f: n_ff as u32, w_off: 0 });
    g.push(Op::GatedAct {
        gate: sg, up: su, dst: sa, rows: rows as u32, nff: n_ff as u32, act: Activation::Silu, up_off: 0, up_stride: 0, gate_stride: 0,
        gate_block_width: 0, swiglu_clamp: None,
    });
    g.push(Op::Linear { x: sa, weight: sh_down, dst: sd, m: rows as u32, in_f: n_ff as u32, out_f: ne as u32, w_off: 0 });
    g.push(Op::MoeSharedExpertAdd { moe, shexp: sd, gate: gl, dst: sub, rows: rows as u32, n: ne as u32 });
    g.push(Op::Add { a: hidden, b: sub, dst: out, n: (rows * ne) as u32 });
    let ones: Vec<f32> = (0..ne).map(|i| 1.0 + 0.01 * ((i % 7) as f32 - 3.0)).collect();
    let bound = vec![
        (hidden, bytes_of(&gen_f32(rows * ne, 1))),
        (nw, bytes_of(&ones)),
        (router, bytes_of(&gen_f32(n_expert * ne, 3).iter().map(|v| v * 0.05).collect::<Vec<_>>())),
        (gate, synth_weight(DType::Q4K, n_expert * n_ff * ne, 11)),
        (up, synth_weight(DType::Q4K, n_expert * n_ff * ne, 12)),
        (down, synth_weight(DType::Q6K, n_expert * ne * n_ff, 13)),
        (sh_gate_inp, bytes_of(&gen_f32(ne, 9).iter().map(|v| v * 0.05).collect::<Vec<_>>())),
        (sh_gate, synth_weight(DType::Q4K, n_ff * ne, 21)),
        (sh_up, synth_weight(DType::Q4K, n_ff * ne, 22)),
        (sh_down, synth_weight(DType::Q6K, ne * n_ff, 23)),
    ];
    let want = run_graph(&cpu, &g, &bound, out, rows * ne);
    let got = run_graph(&gpu, &g, &bound, out, rows * ne);
    let e = rel(&got, &want);
    println!("MoE FFN sub-layer: cuda-vs-cpu(reference) rel={e:e}");
    assert!(e <= TOL);
}

/// What the backend does not cover comes back as `Error::Unsupported`, never as a silent fallback.
#[test]
fn unsupported_is_an_error() {
    let Some(gpu) = gpu() else { return };
    let mut g = Graph::new();
    let x = g.input(f32d(256));
    let w = g.weight(qd(256 * 256, DType::Iq1S));
    let y = g.output(f32d(256));
    g.push(Op::Linear { x, weight: w, dst: y, m: 1, in_f: 256, out_f: 256, w_off: 0 });
    let plan = gpu.compile(&g).expect("compile");
    let xb = gpu.alloc(1024, infr_core::backend::BufferUsage::Activations).unwrap();
    let wb = gpu.alloc(256 * 50, infr_core::backend::BufferUsage::Weights).unwrap();  // 256 rows of one 50-byte IQ1_S block
    let yb = gpu.alloc(1024, infr_core::backend::BufferUsage::Readback).unwrap();
    let mut b = infr_core::backend::Bindings::new();
    b.bind(x, xb.as_ref()).bind(w, wb.as_ref()).bind(y, yb.as_ref());
    match gpu.execute(plan.as_ref(), &b) {
        Err(infr_core::error::Error::Unsupported(_)) => {}
        other => panic!("expected Error::Unsupported, got {other:?}"),
    }
}
