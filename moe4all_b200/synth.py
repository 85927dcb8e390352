"""Seeded synthetic inputs in the shapes and value distributions of the benchmark configs.

Block generators write valid GGUF Q4_K / Q5_K / Q6_K / Q8_0 blocks: every payload bit pattern decodes to
a finite value, only the f16 scale slots need sane magnitudes.  Two families:
  * `random_q4k` / `random_q6k`: random payload, f16 d (and dmin) drawn from U[1e-4, 1e-3]
    (the benchmark configs);
  * `testkit_weight`: the reference's own synthesis recipe, an LCG byte stream per block with the
    scale slots overwritten (crates/infr-testkit/src/lib.rs:49-56, 70-123).
"""
from __future__ import annotations

import numpy as np

Q4K_BYTES, Q6K_BYTES, QK = 144, 210, 256
Q5K_BYTES, Q80_BYTES = 176, 34
# GGUF type number -> (elements per block, bytes per block, offsets of the f16 scale slots)
BLOCKS = {12: (256, 144, (0, 2)), 13: (256, 176, (0, 2)), 14: (256, 210, (208,)), 8: (32, 34, (0,)),
          20: (32, 18, (0,)), 23: (256, 136, (0,)), 2: (32, 18, (0,)), 3: (32, 20, (0, 2)), 6: (32, 22, (0,)), 7: (32, 24, (0, 2)),
          10: (256, 84, (80, 82)), 11: (256, 110, (108,)), 39: (32, 17, ()),
          40: (64, 36, ()), 42: (64, 18, (0,)),
          17: (256, 74, (0,)), 22: (256, 82, (0,)), 18: (256, 98, (0,)), 21: (256, 110, (0,))}  # (MXFP4's exponent byte and NVFP4's four UE4M3 bytes are set apart)


def _f16_bytes(vals: np.ndarray) -> np.ndarray:
    return vals.astype(np.float16).view(np.uint8).reshape(-1, 2)


def random_q4k(rng: np.random.Generator, n_blocks: int, lo: float = 1e-4, hi: float = 1e-3) -> np.ndarray:
    """[n_blocks, 144] u8: f16 d, f16 dmin ~ U[lo, hi]; 12 random scale bytes; 128 random nibble bytes."""
    blk = rng.integers(0, 256, size=(n_blocks, Q4K_BYTES), dtype=np.uint8)
    blk[:, 0:2] = _f16_bytes(rng.uniform(lo, hi, n_blocks))
    blk[:, 2:4] = _f16_bytes(rng.uniform(lo, hi, n_blocks))
    return blk


def random_q6k(rng: np.random.Generator, n_blocks: int, lo: float = 1e-4, hi: float = 1e-3) -> np.ndarray:
    """[n_blocks, 210] u8: random ql/qh/int8 scales; f16 d ~ U[lo, hi] at byte 208."""
    blk = rng.integers(0, 256, size=(n_blocks, Q6K_BYTES), dtype=np.uint8)
    blk[:, 208:210] = _f16_bytes(rng.uniform(lo, hi, n_blocks))
    return blk


def random_blocks(rng: np.random.Generator, dtype: int, n_elem: int, lo: float = 1e-4, hi: float = 1e-3) -> np.ndarray:
    """[n_blocks, block bytes] u8 of GGUF type `dtype` (12 Q4_K, 13 Q5_K, 14 Q6_K, 8 Q8_0, 20 IQ4_NL, 23 IQ4_XS): random payload,
    every f16 scale slot ~ U[lo, hi]."""
    elems, nbytes, slots = BLOCKS[dtype]
    n_blocks = n_elem // elems
    blk = rng.integers(0, 256, size=(n_blocks, nbytes), dtype=np.uint8)
    for o in slots:
        blk[:, o:o + 2] = _f16_bytes(rng.uniform(lo, hi, n_blocks))
    if dtype == 39:  # E8M0 exponent: 2^-14 .. 2^-9, the magnitude of hi
        blk[:, 0] = rng.integers(114, 120, size=n_blocks, dtype=np.uint8)
    if dtype == 40:  # UE4M3 sub-scales with exponent field 0 or 1: at most 15 * 2^-10 / 8, times codes up to 12
        blk[:, 0:4] = rng.integers(1, 16, size=(n_blocks, 4), dtype=np.uint8)
    return blk


# Grid codebook formats: GGUF type -> (entries, bytes per entry, the byte values an entry is made of, entry 0)
CODEBOOKS = {17: (512, 8, (0x08, 0x19, 0x2B), 0x08), 22: (1024, 8, (0x08, 0x19, 0x2B), 0x08),
             18: (256, 4, (4, 12, 20, 28, 36, 44, 52, 62), 4), 21: (512, 4, (1, 3, 5, 7, 9, 11, 13, 15), 1)}


def codebook(dtype: int) -> np.ndarray:
    """A stand-in for the grid table of a codebook format, [entries, bytes per entry] u8, seeded: the real tables
    are constants the reference keeps (crates/infr-core/src/iquant_grids.rs) and a host hands to the library; the
    stand-in has their shape, their alphabet of byte values and their first entry (all 0x08 for the IQ2 grids,
    0x04040404 for IQ3_XXS, 0x01010101 for IQ3_S: the reference's own single-block tests rest on those)."""
    entries, width, alphabet, first = CODEBOOKS[dtype]
    rng = np.random.default_rng(0xC0DE + dtype)
    t = np.asarray(alphabet, np.uint8)[rng.integers(0, len(alphabet), size=(entries, width))]
    t[0, :] = first
    return t


def lcg_bytes(seed: int, n: int) -> np.ndarray:
    """crates/infr-testkit/src/lib.rs:49-56: seed = seed*1664525 + 1013904223 (mod 2^32); byte = seed >> 16."""
    out = np.empty(n, dtype=np.uint8)
    s = seed & 0xFFFFFFFF
    for i in range(n):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = (s >> 16) & 0xFF
    return out


def gen_f32(n: int, salt: int) -> np.ndarray:
    """crates/infr-testkit/src/lib.rs:60-64 (and seam_op_parity.rs:257-261): (((i*13+salt) % 29) - 14) * 0.05."""
    i = np.arange(n, dtype=np.int64)
    return ((((i * 13 + salt) % 29).astype(np.float32) - np.float32(14.0)) * np.float32(0.05)).astype(np.float32)


def testkit_weight(dtype_name: str, n_elem: int, seed: int) -> np.ndarray:
    """crates/infr-testkit/src/lib.rs:74-123 for Q4_K and Q5_K (d 0.05, dmin 0.10), Q6_K (d 0.03),
    Q8_0 (d 0.01), IQ4_NL (d 0.004), IQ4_XS (d 0.06), Q4_0 / Q5_0 (d 0.04), Q4_1 / Q5_1 (d 0.04, m -0.30),
    Q2_K (d 0.05, dmin 0.10), Q3_K (d 0.03), MXFP4 (d 0.25), NVFP4 (d 0.5), Q2_0 (d 0.05), IQ2_XS / IQ2_S (d 0.015),
    IQ3_XXS (d 0.008) and IQ3_S (d 0.002)."""
    TK = {"Q5K": (13, (0.05, 0.10)), "Q8_0": (8, (0.01,)), "IQ4NL": (20, (0.004,)), "IQ4XS": (23, (0.06,)), "Q4_0": (2, (0.04,)),
          "Q4_1": (3, (0.04, -0.30)), "Q5_0": (6, (0.04,)), "Q5_1": (7, (0.04, -0.30)), "Q2K": (10, (0.05, 0.10)), "Q3K": (11, (0.03,)),
          "MXFP4": (39, ()), "NVFP4": (40, ()), "Q2_0": (42, (0.05,)),
          "IQ2XS": (17, (0.015,)), "IQ2S": (22, (0.015,)), "IQ3XXS": (18, (0.008,)), "IQ3S": (21, (0.002,))}
    if dtype_name in TK:
        elems, nbytes, slots = BLOCKS[TK[dtype_name][0]]
        assert n_elem % elems == 0
        nblk = n_elem // elems
        out = np.empty((nblk, nbytes), np.uint8)
        for b in range(nblk):
            out[b] = lcg_bytes(seed ^ b, nbytes)
        for o, v in zip(slots, TK[dtype_name][1]):
            out[:, o:o + 2] = _f16_bytes(np.full(nblk, v))
        if dtype_name == "MXFP4":
            out[:, 0] = 126  # E8M0 of the recipe's d = 0.25 = 2^(126 - 128)
        if dtype_name == "NVFP4":
            # the recipe's d = 0.5 spread as d * (0.625 + 0.125 i) over the four sub-scales
            # (crates/infr-core/src/decode_spec.rs:192-198): 0.3125, 0.375, 0.4375, 0.5, all exact in UE4M3
            out[:, 0:4] = np.array([0x2A, 0x2C, 0x2E, 0x30], np.uint8)
        return out
    assert n_elem % QK == 0
    nblk = n_elem // QK
    if dtype_name == "Q4K":
        out = np.empty((nblk, Q4K_BYTES), np.uint8)
        for b in range(nblk):
            out[b] = lcg_bytes(seed ^ b, Q4K_BYTES)
        out[:, 0:2] = _f16_bytes(np.full(nblk, 0.05))
        out[:, 2:4] = _f16_bytes(np.full(nblk, 0.10))
    elif dtype_name == "Q6K":
        out = np.empty((nblk, Q6K_BYTES), np.uint8)
        for b in range(nblk):
            out[b] = lcg_bytes(seed ^ b, Q6K_BYTES)
        out[:, 208:210] = _f16_bytes(np.full(nblk, 0.03))
    else:
        raise ValueError(dtype_name)
    return out


class LayerWeights:
    """Host copies of one MoE layer's tensors (raw GGUF bytes + f32 router)."""

    def __init__(self, ne, n_expert, n_ff, sh_ff=0, gated_shared=True):
        self.ne, self.n_expert, self.n_ff, self.sh_ff, self.gated_shared = ne, n_expert, n_ff, sh_ff, gated_shared
        self.router = self.gate = self.up = self.down = None
        self.sh_gate = self.sh_up = self.sh_down = self.sh_gate_inp = None
        self.bias = None
        self.gate_dtype = self.up_dtype = 12
        self.down_dtype = 14


def make_layer(seed: int, ne: int, n_expert: int, n_ff: int, sh_ff: int = 0, gated_shared: bool = True,
               router_std: float = 0.02, bias_std: float = 0.0, down_q4k: bool = False, dtypes=None) -> LayerWeights:
    """One layer in the benchmark configs' distributions: router f32 N(0, 0.02); gate/up Q4_K and
    down Q6_K with random payload and U[1e-4, 1e-3] scales; optional shared expert.
    dtypes = (gate, up, down) GGUF type numbers for another mix of bank formats."""
    rng = np.random.default_rng(seed)
    L = LayerWeights(ne, n_expert, n_ff, sh_ff, gated_shared)
    L.router = rng.normal(0.0, router_std, size=(n_expert, ne)).astype(np.float32)
    if dtypes is not None:
        L.gate_dtype, L.up_dtype, L.down_dtype = dtypes

        def bank(dt, n_elem):
            k = {8: 2.0, 20: 2.0, 2: 32.0, 3: 32.0, 6: 16.0, 7: 16.0, 10: 64.0, 11: 8.0, 42: 64.0, 17: 0.5, 22: 0.5, 18: 0.2, 21: 0.2}.get(dt, 1.0)  # similar weight magnitudes
            return random_blocks(rng, dt, n_elem, 1e-4 * k, 1e-3 * k).reshape(-1)
        L.gate, L.up, L.down = bank(dtypes[0], n_expert * n_ff * ne), bank(dtypes[1], n_expert * n_ff * ne), bank(dtypes[2], n_expert * ne * n_ff)
        if sh_ff:
            L.sh_gate, L.sh_up, L.sh_down = bank(dtypes[0], sh_ff * ne), bank(dtypes[1], sh_ff * ne), bank(dtypes[2], ne * sh_ff)
            if gated_shared:
                L.sh_gate_inp = rng.normal(0.0, router_std, size=ne).astype(np.float32)
        if bias_std > 0:
            L.bias = rng.normal(0.0, bias_std, size=n_expert).astype(np.float32)
        return L
    L.gate = random_q4k(rng, n_expert * n_ff * ne // QK).reshape(-1)
    L.up = random_q4k(rng, n_expert * n_ff * ne // QK).reshape(-1)
    L.down_dtype = 12 if down_q4k else 14  # GGUF type numbers: Q4_K, Q6_K (a Q4_K_M file mixes both over its layers)
    L.down = (random_q4k if down_q4k else random_q6k)(rng, n_expert * ne * n_ff // QK).reshape(-1)
    if sh_ff:
        L.sh_gate = random_q4k(rng, sh_ff * ne // QK).reshape(-1)
        L.sh_up = random_q4k(rng, sh_ff * ne // QK).reshape(-1)
        L.sh_down = (random_q4k if down_q4k else random_q6k)(rng, ne * sh_ff // QK).reshape(-1)
        if gated_shared:
            L.sh_gate_inp = rng.normal(0.0, router_std, size=ne).astype(np.float32)
    if bias_std > 0:
        L.bias = rng.normal(0.0, bias_std, size=n_expert).astype(np.float32)
    return L


def activations(seed: int, rows: int, ne: int) -> np.ndarray:
    return np.random.default_rng(seed).normal(0.0, 1.0, size=(rows, ne)).astype(np.float32)
