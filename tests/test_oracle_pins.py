"""Pins the CPU oracle to the reference's own known-answer material (CPU only).

Every vector here is re-created from the formula the reference's tests use; the files and lines
are cited per test.  Independent decoders are written in numpy from the block layout, not from the
oracle's C++.
"""
import numpy as np
import pytest

from moe4all_b200 import synth
from oracle import oracle as orc

F32 = np.float32


# ---- independent numpy decoders -----------------------------------------------------------------

def f16(b0, b1):
    return np.array([b0 | (b1 << 8)], dtype=np.uint16).view(np.float16).astype(F32)[0]


def np_q4k(raw):
    """Factored form (crates/infr-gguf/src/dequant.rs:35-51, 315-335): (f32(d)*sc)*q + (f32(dmin)*(-m))."""
    raw = np.asarray(raw, np.uint8).reshape(-1, 144)
    out = np.empty((raw.shape[0], 256), F32)
    for bi, blk in enumerate(raw):
        d, dmin = f16(int(blk[0]), int(blk[1])), f16(int(blk[2]), int(blk[3]))
        sc_b, qs = blk[4:16].astype(np.int64), blk[16:144]
        for s in range(8):
            if s < 4:
                sc, m = sc_b[s] & 63, sc_b[s + 4] & 63
            else:
                sc = (sc_b[s + 4] & 0xF) | ((sc_b[s - 4] >> 6) << 4)
                m = (sc_b[s + 4] >> 4) | ((sc_b[s] >> 6) << 4)
            S = F32(d * F32(sc))
            M = F32(dmin * F32(-m))
            byts = qs[32 * (s // 2): 32 * (s // 2) + 32]
            q = (byts & 0xF) if s % 2 == 0 else (byts >> 4)
            out[bi, 32 * s: 32 * s + 32] = (S * q.astype(F32)).astype(F32) + M
    return out.reshape(-1)


def np_q6k_codes(blk):
    ql, qh = blk[0:128].astype(np.int64), blk[128:192].astype(np.int64)
    q = np.empty(256, np.int64)
    for half in range(2):
        for l in range(32):
            a, b, h = ql[64 * half + l], ql[64 * half + 32 + l], qh[32 * half + l]
            base = 128 * half + l
            q[base] = (a & 0xF) | ((h & 3) << 4)
            q[base + 32] = (b & 0xF) | (((h >> 2) & 3) << 4)
            q[base + 64] = (a >> 4) | (((h >> 4) & 3) << 4)
            q[base + 96] = (b >> 4) | (((h >> 6) & 3) << 4)
    return q


def np_q6k(raw, glsl_form=False):
    """Factored form (dequant.rs:365-389): (f32(d)*sc)*q + f32(d)*(-32*sc); or the shader's
    d*sc*(q-32) (crates/infr-vulkan/shaders/native_decode.glsl:581)."""
    raw = np.asarray(raw, np.uint8).reshape(-1, 210)
    out = np.empty((raw.shape[0], 256), F32)
    for bi, blk in enumerate(raw):
        d = f16(int(blk[208]), int(blk[209]))
        sc = blk[192:208].view(np.int8).astype(np.int64)
        q = np_q6k_codes(blk)
        scale = np.repeat(sc, 16)
        if glsl_form:
            out[bi] = (F32(d) * scale.astype(F32)).astype(F32) * (q - 32).astype(F32)
        else:
            S = (F32(d) * scale.astype(F32)).astype(F32)
            M = (F32(d) * (-32 * scale).astype(F32)).astype(F32)
            out[bi] = (S * q.astype(F32)).astype(F32) + M
    return out.reshape(-1)


def np_q5k(raw):
    """Factored form (dequant.rs:35-51, 337-362): Q4_K's scales; code = nibble + 16 * bit (2j | 2j+1) of qh[l]."""
    raw = np.asarray(raw, np.uint8).reshape(-1, 176)
    out = np.empty((raw.shape[0], 256), F32)
    for bi, blk in enumerate(raw):
        d, dmin = f16(int(blk[0]), int(blk[1])), f16(int(blk[2]), int(blk[3]))
        sc_b, qh, qs = blk[4:16].astype(np.int64), blk[16:48].astype(np.int64), blk[48:176].astype(np.int64)
        for s in range(8):
            if s < 4:
                sc, m = sc_b[s] & 63, sc_b[s + 4] & 63
            else:
                sc = (sc_b[s + 4] & 0xF) | ((sc_b[s - 4] >> 6) << 4)
                m = (sc_b[s + 4] >> 4) | ((sc_b[s] >> 6) << 4)
            S = F32(d * F32(sc))
            M = F32(dmin * F32(-m))
            byts = qs[32 * (s // 2): 32 * (s // 2) + 32]
            q = ((byts & 0xF) if s % 2 == 0 else (byts >> 4)) + 16 * ((qh >> s) & 1)
            out[bi, 32 * s: 32 * s + 32] = (S * q.astype(F32)).astype(F32) + M
    return out.reshape(-1)


def np_q80(raw):
    """Factored form (dequant.rs:35-51, 214-223): (f32(d)*1)*(q+128) + f32(d)*(-128)."""
    raw = np.asarray(raw, np.uint8).reshape(-1, 34)
    out = np.empty((raw.shape[0], 32), F32)
    for bi, blk in enumerate(raw):
        d = f16(int(blk[0]), int(blk[1]))
        code = blk[2:34].view(np.int8).astype(np.int64) + 128
        with np.errstate(all="ignore"):
            out[bi] = (F32(d * F32(1)) * code.astype(F32)).astype(F32) + F32(d * F32(-128))
    return out.reshape(-1)


def pattern_q4k():
    # crates/infr-gguf/src/dequant.rs:1174-1187: bytes ((i*37+11)&0xFF), d = 0.375, dmin = -0.125
    b = ((np.arange(288) * 37 + 11) & 0xFF).astype(np.uint8)
    for blk in range(2):
        b[blk * 144: blk * 144 + 2] = np.array([0.375], np.float16).view(np.uint8)
        b[blk * 144 + 2: blk * 144 + 4] = np.array([-0.125], np.float16).view(np.uint8)
    return b


def pattern_q6k():
    # crates/infr-gguf/src/dequant.rs:1190-1202: bytes ((i*53+7)&0xFF), d = 0.05 at byte 208
    b = ((np.arange(420) * 53 + 7) & 0xFF).astype(np.uint8)
    for blk in range(2):
        b[blk * 210 + 208: blk * 210 + 210] = np.array([0.05], np.float16).view(np.uint8)
    return b


# ---- block decode --------------------------------------------------------------------------------

def test_q4k_pattern_bit_identical():
    raw = pattern_q4k()
    got = orc.dequant(orc.DT_Q4K, raw, 512)
    assert np.array_equal(got.view(np.uint32), np_q4k(raw).view(np.uint32))
    # element 0 by hand: sub-block 0, sc = scales[0] & 63, m = scales[4] & 63, q = qs[0] & 0xF
    sc, m, q = int(raw[4]) & 63, int(raw[8]) & 63, int(raw[16]) & 0xF
    want0 = F32(F32(0.375) * F32(sc)) * F32(q) + F32(F32(-0.125) * F32(-m))
    assert got[0] == want0
    assert np.all(np.isfinite(got)) and np.ptp(got) > 0


def test_q6k_pattern_bit_identical():
    raw = pattern_q6k()
    got = orc.dequant(orc.DT_Q6K, raw, 512)
    assert np.array_equal(got.view(np.uint32), np_q6k(raw).view(np.uint32))
    # the shader's form d*sc*(q-32) rounds differently by at most an ulp or two of the scale term
    alt = np_q6k(raw, glsl_form=True)
    assert np.max(np.abs(got - alt)) <= 4e-6 * np.max(np.abs(alt))
    assert np.ptp(got) > 0


@pytest.mark.parametrize("dt,name,nbytes", [(orc.DT_Q4K, "Q4K", 144), (orc.DT_Q6K, "Q6K", 210)])
def test_testkit_synth_blocks(dt, name, nbytes):
    # crates/infr-testkit/src/lib.rs:106-123: LCG payload per block (seed ^ block), scale slots overwritten
    raw = synth.testkit_weight(name, 4 * 256, seed=0x1234)
    assert raw.shape == (4, nbytes)
    got = orc.dequant(dt, raw, 1024)
    want = np_q4k(raw) if name == "Q4K" else np_q6k(raw)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # LCG: first byte of block 0 is ((seed*1664525 + 1013904223) mod 2^32) >> 16 & 0xFF
    s = (0x1234 * 1664525 + 1013904223) & 0xFFFFFFFF
    assert synth.lcg_bytes(0x1234, 1)[0] == (s >> 16) & 0xFF


def test_random_blocks_match_numpy_decoder():
    rng = np.random.default_rng(5)
    q4, q6 = synth.random_q4k(rng, 16), synth.random_q6k(rng, 16)
    assert np.array_equal(orc.dequant(orc.DT_Q4K, q4, 4096).view(np.uint32), np_q4k(q4).view(np.uint32))
    assert np.array_equal(orc.dequant(orc.DT_Q6K, q6, 4096).view(np.uint32), np_q6k(q6).view(np.uint32))


@pytest.mark.parametrize("dt,nbytes,elems,ref", [(orc.DT_Q5K, 176, 256, np_q5k), (orc.DT_Q8_0, 34, 32, np_q80)])
def test_q5k_q80_patterns(dt, nbytes, elems, ref):
    # crates/infr-gguf/src/dequant.rs:1206-1229: two blocks of bytes ((i*29+3)&0xFF), scale slots included
    # (a block whose patterned scale is not finite decodes to the same non-finite bit patterns)
    raw = ((np.arange(2 * nbytes) * 29 + 3) & 0xFF).astype(np.uint8)
    with np.errstate(all="ignore"):
        want = ref(raw)
    got = orc.dequant(dt, raw, 2 * elems)
    fin = np.isfinite(want)
    assert np.array_equal(got[fin].view(np.uint32), want[fin].view(np.uint32))
    assert np.array_equal(np.isnan(got), np.isnan(want)) and np.array_equal(np.isinf(got), np.isinf(want))
    # the reference's synthesis recipe (crates/infr-testkit/src/lib.rs:74-123): LCG payload, scale slots set
    name = "Q5K" if dt == orc.DT_Q5K else "Q8_0"
    raw = synth.testkit_weight(name, 1024, seed=0x4321)
    got = orc.dequant(dt, raw, 1024)
    assert np.array_equal(got.view(np.uint32), ref(raw).view(np.uint32))
    assert np.all(np.isfinite(got)) and np.ptp(got) > 0
    # random payloads
    rb = synth.random_blocks(np.random.default_rng(9), dt, 4096)
    assert np.array_equal(orc.dequant(dt, rb, 4096).view(np.uint32), ref(rb).view(np.uint32))


def test_q80_by_hand():
    # d = 0.5, q = [-128, -1, 0, 127, ...]: value = d * q exactly
    blk = np.zeros(34, np.uint8)
    blk[0:2] = np.array([0.5], np.float16).view(np.uint8)
    blk[2:6] = np.array([-128, -1, 0, 127], np.int8).view(np.uint8)
    got = orc.dequant(orc.DT_Q8_0, blk, 32)
    assert list(got[:4]) == [-64.0, -0.5, 0.0, 63.5]
    assert orc.row_bytes(orc.DT_Q8_0, 2048) == 2176 and orc.row_bytes(orc.DT_Q5K, 2048) == 1408


KV_IQ4NL = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.float32)  # dequant.rs:443-445


def np_iq4nl(raw):
    """dequant.rs:499-517: y[j] = d * kv[qs[j] & 0xF], y[j + 16] = d * kv[qs[j] >> 4]."""
    raw = np.asarray(raw, np.uint8).reshape(-1, 18)
    out = np.empty((raw.shape[0], 32), F32)
    for bi, blk in enumerate(raw):
        d = f16(int(blk[0]), int(blk[1]))
        qs = blk[2:18].astype(np.int64)
        out[bi, :16] = F32(d) * KV_IQ4NL[qs & 0xF]
        out[bi, 16:] = F32(d) * KV_IQ4NL[qs >> 4]
    return out.reshape(-1)


def np_iq4xs(raw):
    """dequant.rs:521-553: sub-block scale ls = scales_l nibble | scales_h two bits << 4; dl = d * (ls - 32)."""
    raw = np.asarray(raw, np.uint8).reshape(-1, 136)
    out = np.empty((raw.shape[0], 256), F32)
    for bi, blk in enumerate(raw):
        d = f16(int(blk[0]), int(blk[1]))
        sh = int(blk[2]) | (int(blk[3]) << 8)
        for ib in range(8):
            ls = ((int(blk[4 + ib // 2]) >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4)
            dl = F32(F32(d) * F32(ls - 32))
            qs = blk[8 + 16 * ib: 24 + 16 * ib].astype(np.int64)
            out[bi, 32 * ib: 32 * ib + 16] = dl * KV_IQ4NL[qs & 0xF]
            out[bi, 32 * ib + 16: 32 * ib + 32] = dl * KV_IQ4NL[qs >> 4]
    return out.reshape(-1)


def test_iq4_reference_vectors():
    # crates/infr-gguf/src/dequant.rs `iq4nl_single_block`: d = 1, qs[0] = 0x80 -> y[0] = kv[0] = -127, y[16] = kv[8] = 1
    blk = np.zeros(18, np.uint8)
    blk[0:2] = np.array([1.0], np.float16).view(np.uint8)
    blk[2] = 0x80
    y = orc.dequant(orc.DT_IQ4NL, blk, 32)
    assert y[0] == -127.0 and y[16] == 1.0
    assert np.all(y[1:16] == -127.0) and np.all(y[17:] == -127.0)  # the other code bytes are 0: kv[0] both ways
    # `iq4xs` single block: d = 1, everything else 0 -> ls = 0, dl = -32, every code kv[0] = -127: all 4064
    blk = np.zeros(136, np.uint8)
    blk[0:2] = np.array([1.0], np.float16).view(np.uint8)
    y = orc.dequant(orc.DT_IQ4XS, blk, 256)
    assert np.all(y == 4064.0)
    assert orc.row_bytes(orc.DT_IQ4NL, 2048) == 1152 and orc.row_bytes(orc.DT_IQ4XS, 2048) == 1088


@pytest.mark.parametrize("dt,name,elems,ref", [(orc.DT_IQ4NL, "IQ4NL", 32, np_iq4nl), (orc.DT_IQ4XS, "IQ4XS", 256, np_iq4xs)])
def test_iq4_blocks_match_numpy_decoder(dt, name, elems, ref):
    # the reference's synthesis recipe (LCG payload, d slot set: crates/infr-testkit/src/lib.rs:74-123) and random payloads
    raw = synth.testkit_weight(name, 1024, seed=0x9876)
    got = orc.dequant(dt, raw, 1024)
    assert np.array_equal(got.view(np.uint32), ref(raw).view(np.uint32))
    assert np.all(np.isfinite(got)) and np.ptp(got) > 0
    rb = synth.random_blocks(np.random.default_rng(11), dt, 4096)
    assert np.array_equal(orc.dequant(dt, rb, 4096).view(np.uint32), ref(rb).view(np.uint32))


def np_legacy32(raw, dt):
    """dequant.rs:142-212, 35-51: Q4_0 / Q4_1 / Q5_0 / Q5_1 = (f32(d)*1)*code + (f32(d)*-8 | f32(m)*1 | f32(d)*-16 | f32(m)*1)."""
    has_m, five = dt in (3, 7), dt in (6, 7)
    hdr = 4 if has_m else 2
    bb = hdr + (4 if five else 0) + 16
    raw = np.asarray(raw, np.uint8).reshape(-1, bb)
    out = np.empty((raw.shape[0], 32), F32)
    for bi, blk in enumerate(raw):
        with np.errstate(all="ignore"):
            d = f16(int(blk[0]), int(blk[1]))
            mn = F32(f16(int(blk[2]), int(blk[3])) * F32(1)) if has_m else F32(d * F32(-16 if five else -8))
            qh = int.from_bytes(bytes(blk[hdr:hdr + 4]), "little") if five else 0
            qs = blk[hdr + (4 if five else 0):].astype(np.int64)
            j = np.arange(16)
            c0 = (qs & 0xF) | ((((qh >> j) & 1) << 4) if five else 0)
            c1 = (qs >> 4) | ((((qh >> (j + 16)) & 1) << 4) if five else 0)
            sc = F32(d * F32(1))
            out[bi, :16] = (sc * c0.astype(F32)).astype(F32) + mn
            out[bi, 16:] = (sc * c1.astype(F32)).astype(F32) + mn
    return out.reshape(-1)


def np_q2k(raw):
    """dequant.rs:224-252: per 16 elements (f32(d)*(s & 15))*code + (f32(dmin)*-(s >> 4)), 2-bit codes."""
    raw = np.asarray(raw, np.uint8).reshape(-1, 84)
    out = np.empty((raw.shape[0], 256), F32)
    for bi, blk in enumerate(raw):
        with np.errstate(all="ignore"):
            d, dmin = f16(int(blk[80]), int(blk[81])), f16(int(blk[82]), int(blk[83]))
            qs = blk[16:80].astype(np.int64)
            for g in range(16):
                n, j, half = g >> 3, (g >> 1) & 3, g & 1
                s = int(blk[g])
                code = (qs[32 * n + 16 * half: 32 * n + 16 * half + 16] >> (2 * j)) & 3
                out[bi, 16 * g: 16 * g + 16] = (F32(d * F32(s & 15)) * code.astype(F32)).astype(F32) + F32(dmin * F32(-(s >> 4)))
    return out.reshape(-1)


def np_q3k(raw):
    """dequant.rs:253-314: sixteen 6-bit scales (s = sc6 - 32), codes low2 | hmask bit << 2: (f32(d)*s)*code + f32(d)*(-4 s)."""
    raw = np.asarray(raw, np.uint8).reshape(-1, 110)
    out = np.empty((raw.shape[0], 256), F32)
    for bi, blk in enumerate(raw):
        with np.errstate(all="ignore"):
            d = f16(int(blk[108]), int(blk[109]))
            hm, qs, sr = blk[0:32].astype(np.int64), blk[32:96].astype(np.int64), blk[96:108].astype(np.int64)
            for g in range(16):
                n, j, half = g >> 3, (g >> 1) & 3, g & 1
                # scale g: low four bits = low (g < 8) or high nibble of byte g % 8, two more bits from byte 8 + g % 4 at bit 2 (g / 4)
                lo4 = (sr[g % 8] >> (0 if g < 8 else 4)) & 0xF
                hi2 = (sr[8 + g % 4] >> (2 * (g // 4))) & 3
                s = int(lo4 | (hi2 << 4)) - 32
                low2 = (qs[32 * n + 16 * half: 32 * n + 16 * half + 16] >> (2 * j)) & 3
                high = (hm[16 * half: 16 * half + 16] >> (4 * n + j)) & 1
                code = low2 | (high << 2)
                out[bi, 16 * g: 16 * g + 16] = (F32(d * F32(s)) * code.astype(F32)).astype(F32) + F32(d * F32(-4 * s))
    return out.reshape(-1)


@pytest.mark.parametrize("dt,name,nbytes,elems", [(2, "Q4_0", 18, 32), (3, "Q4_1", 20, 32), (6, "Q5_0", 22, 32), (7, "Q5_1", 24, 32),
                                                   (10, "Q2K", 84, 256), (11, "Q3K", 110, 256)])
def test_legacy_and_small_k_formats(dt, name, nbytes, elems):
    ref = np_q2k if dt == 10 else np_q3k if dt == 11 else (lambda raw: np_legacy32(raw, dt))
    # crates/infr-gguf/src/dequant.rs:1206-1229: two blocks of bytes ((i*29+3)&0xFF), scale slots included
    raw = ((np.arange(2 * nbytes) * 29 + 3) & 0xFF).astype(np.uint8)
    want, got = ref(raw), orc.dequant(dt, raw, 2 * elems)
    fin = np.isfinite(want)
    assert np.array_equal(got[fin].view(np.uint32), want[fin].view(np.uint32))
    assert np.array_equal(np.isnan(got), np.isnan(want)) and np.array_equal(np.isinf(got), np.isinf(want))
    # the reference's synthesis recipe (crates/infr-testkit/src/lib.rs:74-123) and random payloads
    raw = synth.testkit_weight(name, 1024, seed=0x2468)
    got = orc.dequant(dt, raw, 1024)
    assert np.array_equal(got.view(np.uint32), ref(raw).view(np.uint32))
    assert np.all(np.isfinite(got)) and np.ptp(got) > 0
    rb = synth.random_blocks(np.random.default_rng(13), dt, 4096)
    assert np.array_equal(orc.dequant(dt, rb, 4096).view(np.uint32), ref(rb).view(np.uint32))


def test_q4_0_by_hand():
    # d = 2, code byte 0x1F: element 0 = 2 * (15 - 8) = 14, element 16 = 2 * (1 - 8) = -14; Q4_1 with m = 0.5: 2 * 15 + 0.5, 2 * 1 + 0.5
    blk = np.zeros(18, np.uint8)
    blk[0:2] = np.array([2.0], np.float16).view(np.uint8)
    blk[2] = 0x1F
    y = orc.dequant(2, blk, 32)
    assert y[0] == 14.0 and y[16] == -14.0 and y[1] == -16.0
    blk = np.zeros(20, np.uint8)
    blk[0:2] = np.array([2.0], np.float16).view(np.uint8)
    blk[2:4] = np.array([0.5], np.float16).view(np.uint8)
    blk[4] = 0x1F
    y = orc.dequant(3, blk, 32)
    assert y[0] == 30.5 and y[16] == 2.5 and y[1] == 0.5


def np_mxfp4(raw):
    """dequant.rs:409-421, 1029-1046: d = 2^(e - 128) (e < 2: the two subnormals), y = kv[nibble] * d."""
    kv = np.array([0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12], np.float32)
    raw = np.asarray(raw, np.uint8).reshape(-1, 17)
    out = np.empty((raw.shape[0], 32), F32)
    for bi, blk in enumerate(raw):
        e = int(blk[0])
        d = np.float32(np.ldexp(1.0, e - 128))  # exact in f32 down to 2^-128 = the subnormal the reference builds for e = 0
        qs = blk[1:17].astype(np.int64)
        out[bi, :16] = kv[qs & 0xF] * d
        out[bi, 16:] = kv[qs >> 4] * d
    return out.reshape(-1)


def test_mxfp4_reference_vector_and_blocks():
    # crates/infr-gguf/src/dequant.rs `mxfp4_single_block`: e = 128 -> d = 1; qs[0] = 0x21 -> y[0] = 1, y[16] = 2, the rest 0
    blk = np.zeros(17, np.uint8)
    blk[0], blk[1] = 128, 0x21
    y = orc.dequant(orc.DT_MXFP4, blk, 32)
    assert y[0] == 1.0 and y[16] == 2.0 and np.all(y[1:16] == 0.0) and np.all(y[17:] == 0.0)
    assert orc.row_bytes(orc.DT_MXFP4, 2048) == 1088
    raw = synth.testkit_weight("MXFP4", 1024, seed=0x1357)  # the reference's recipe: d = 0.25
    got = orc.dequant(orc.DT_MXFP4, raw, 1024)
    assert np.array_equal(got.view(np.uint32), np_mxfp4(raw).view(np.uint32)) and np.abs(got).max() == 3.0
    rb = ((np.arange(4 * 17) * 29 + 3) & 0xFF).astype(np.uint8)  # every exponent byte, the two smallest included, decodes alike
    rb[0], rb[17] = 0, 1
    assert np.array_equal(orc.dequant(orc.DT_MXFP4, rb, 128).view(np.uint32), np_mxfp4(rb).view(np.uint32))


def np_nvfp4(raw):
    """dequant.rs:423-439, 1053-1073: per 16 weights a UE4M3 byte (halved; 0x00 and 0x7F give 0) and 8 code bytes,
    low nibbles weights 0-7, high nibbles weights 8-15; y = kv[nibble] * d."""
    kv = np.array([0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12], np.float32)
    raw = np.asarray(raw, np.uint8).reshape(-1, 36)
    out = np.empty((raw.shape[0], 64), F32)
    for bi, blk in enumerate(raw):
        for s in range(4):
            x = int(blk[s])
            ex, man = (x >> 3) & 0xF, x & 7
            d = 0.0 if x in (0, 0x7F) else (man * 2.0 ** -9 if ex == 0 else (1 + man / 8) * 2.0 ** (ex - 7)) * 0.5  # exact in f64 and f32
            qs = blk[4 + 8 * s:12 + 8 * s].astype(np.int64)
            out[bi, 16 * s:16 * s + 8] = kv[qs & 0xF] * np.float32(d)
            out[bi, 16 * s + 8:16 * s + 16] = kv[qs >> 4] * np.float32(d)
    return out.reshape(-1)


def test_nvfp4_reference_vector_and_blocks():
    # crates/infr-gguf/src/dequant.rs `nvfp4_single_block`: the all-zero block decodes to zeros
    assert np.all(orc.dequant(orc.DT_NVFP4, np.zeros(36, np.uint8), 64) == 0.0)
    assert orc.row_bytes(orc.DT_NVFP4, 2048) == 1152
    # the reference's recipe (d = 0.5 spread over the four sub-scales, crates/infr-core/src/decode_spec.rs:192-198):
    # four distinct non-zero scale bytes, as its `write_scales_round_trips_each_encoding` asks
    raw = synth.testkit_weight("NVFP4", 1024, seed=0x2468)
    assert len(set(raw.reshape(-1, 36)[0, :4].tolist())) == 4 and raw.reshape(-1, 36)[:, :4].min() > 0
    got = orc.dequant(orc.DT_NVFP4, raw, 1024)
    assert np.array_equal(got.view(np.uint32), np_nvfp4(raw).view(np.uint32))
    assert np.abs(got).max() == 12 * 0.25  # code 12 under the largest sub-scale 0.5, halved
    # every scale byte, 0x00, 0x7F, the exponent-0 forms and bit 7 set included
    rb = ((np.arange(64 * 36) * 37 + 11) & 0xFF).astype(np.uint8).reshape(64, 36)
    rb[:, :4] = np.arange(256, dtype=np.uint8).reshape(64, 4)
    assert np.array_equal(orc.dequant(orc.DT_NVFP4, rb.reshape(-1), 64 * 64).view(np.uint32), np_nvfp4(rb).view(np.uint32))


def test_q2_0_reference_vector_and_blocks():
    # crates/infr-gguf/src/dequant.rs `q2_0_single_block`: d = 0.5, qs[0] = 0b11100100 -> -0.5, 0, 0.5, 1.0, then -0.5
    blk = np.zeros(18, np.uint8)
    blk[0:2] = np.array([0.5], np.float16).view(np.uint8)
    blk[2] = 0b11100100
    y = orc.dequant(orc.DT_Q2_0, blk, 64)
    assert y[:4].tolist() == [-0.5, 0.0, 0.5, 1.0] and np.all(y[4:] == -0.5)
    assert orc.row_bytes(orc.DT_Q2_0, 2048) == 576
    raw = synth.testkit_weight("Q2_0", 1024, seed=0x99).reshape(-1, 18)
    d = raw[:, 0:2].copy().view(np.float16).astype(np.float32)  # [blocks, 1]
    q = (raw[:, 2 + np.arange(64) // 4].astype(np.int64) >> ((np.arange(64) % 4) * 2)) & 3
    want = ((q - 1).astype(np.float32) * d).reshape(-1)
    assert np.array_equal(orc.dequant(orc.DT_Q2_0, raw.reshape(-1), 1024).view(np.uint32), want.view(np.uint32))


def _ksigns(i):
    return i | ((bin(i).count("1") & 1) << 7)


def np_grid_formats(dt, raw, table):
    """dequant.rs:477-488, 605-770 for IQ2_XS (17), IQ2_S (22), IQ3_XXS (18), IQ3_S (21): grid entry bytes x sign x the
    group's scale, with f32 products in the reference's order (db first, then db * byte, then the sign)."""
    bb = {17: 74, 22: 82, 18: 98, 21: 110}[dt]
    raw = np.asarray(raw, np.uint8).reshape(-1, bb)
    t = np.asarray(table, np.uint8)
    out = np.empty((raw.shape[0], 256), F32)
    for bi, blk in enumerate(raw):
        d = F32(blk[0:2].copy().view(np.float16)[0])
        for ib in range(8):
            for l in range(4):
                if dt in (17, 22):
                    sc = int(blk[(66 if dt == 17 else 74) + ib])
                    ls = (sc & 15) if l < 2 else (sc >> 4)
                    db = F32(F32(d * F32(0.5 + ls)) * F32(0.25))
                    if dt == 17:
                        q = int(blk[2 + 2 * (4 * ib + l)]) | (int(blk[3 + 2 * (4 * ib + l)]) << 8)
                        vals, sg = t[q & 511], _ksigns(q >> 9)
                    else:
                        idx = int(blk[2 + 4 * ib + l]) | ((int(blk[66 + ib]) << (8 - 2 * l)) & 0x300)
                        vals, sg = t[idx], int(blk[34 + 4 * ib + l])
                else:
                    if dt == 18:
                        aux = int.from_bytes(bytes(blk[66 + 4 * ib:70 + 4 * ib]), "little")
                        db = F32(F32(d * F32(0.5 + (aux >> 28))) * F32(0.5))
                        sg = _ksigns((aux >> (7 * l)) & 127)
                        i1, i2 = int(blk[2 + 8 * ib + 2 * l]), int(blk[3 + 8 * ib + 2 * l])
                    else:
                        sb, qh = int(blk[106 + ib // 2]), int(blk[66 + ib])
                        db = F32(d * F32(1.0 + 2.0 * ((sb >> 4) if ib & 1 else (sb & 15))))
                        sg = int(blk[74 + 4 * ib + l])
                        i1 = int(blk[2 + 8 * ib + 2 * l]) | ((qh << (8 - 2 * l)) & 256)
                        i2 = int(blk[3 + 8 * ib + 2 * l]) | ((qh << (7 - 2 * l)) & 256)
                    vals = np.concatenate([t[i1], t[i2]])
                for j in range(8):
                    v = F32(db * F32(int(vals[j])))
                    out[bi, 32 * ib + 8 * l + j] = -v if (sg >> j) & 1 else v
    return out.reshape(-1)


@pytest.mark.parametrize("dt,name,bb", [(17, "IQ2XS", 74), (22, "IQ2S", 82), (18, "IQ3XXS", 98), (21, "IQ3S", 110)])
def test_grid_codebook_formats(dt, name, bb):
    # The grid tables are handed in (the real ones are the reference's constants); the stand-ins keep the first
    # entry of the real tables, on which the reference's own single-block tests rest
    # (crates/infr-gguf/src/dequant.rs `iq2xs_single_block`, `iq2s_single_block`, `iq3xxs_single_block`,
    # `iq3s_single_block`: d = 1 and an otherwise all-zero block decode to 1.0 everywhere).
    table = synth.codebook(dt)
    orc.set_codebook(dt, table)
    blk = np.zeros(bb, np.uint8)
    blk[0:2] = np.array([1.0], np.float16).view(np.uint8)
    assert np.all(orc.dequant(dt, blk, 256) == 1.0)
    assert orc.row_bytes(dt, 2048) == 8 * bb
    raw = synth.testkit_weight(name, 1024, seed=0x5150 + dt)  # the reference's recipe: LCG payload, d from synth_scales
    got = orc.dequant(dt, raw, 1024)
    want = np_grid_formats(dt, raw, table)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)) and np.abs(got).max() > 0
    assert (got < 0).any() and (got > 0).any()
    with pytest.raises(ValueError):
        orc.set_codebook(dt, table[:-1])  # a table of the wrong size
    with pytest.raises(ValueError):
        orc.set_codebook(12, table)  # not a codebook format


@pytest.mark.parametrize("dt", sorted(synth.BLOCKS))
def test_random_blocks_decode_like_the_independent_restatements(dt):
    # every format, random payload bits (the generators of the GPU tests and the benchmark): the oracle's decoder and
    # the numpy restatement above agree bit for bit, and nothing decodes to a non-finite value
    for cb in synth.CODEBOOKS:
        orc.set_codebook(cb, synth.codebook(cb))
    elems = synth.BLOCKS[dt][0]
    n = 24 * max(elems, 64)
    raw = synth.random_blocks(np.random.default_rng(700 + dt), dt, n, 1e-3, 1e-1).reshape(-1)
    got = orc.dequant(dt, raw, n)
    if dt == 42:  # Q2_0: (code - 1) * d, codes two bits each
        blk = raw.reshape(-1, 18)
        d = blk[:, 0:2].copy().view(np.float16).astype(np.float32)
        q = (blk[:, 2 + np.arange(64) // 4].astype(np.int64) >> ((np.arange(64) % 4) * 2)) & 3
        want = ((q - 1).astype(np.float32) * d).reshape(-1)
    else:
        want = {12: np_q4k, 14: np_q6k, 13: np_q5k, 8: np_q80, 20: np_iq4nl, 23: np_iq4xs, 10: np_q2k, 11: np_q3k, 39: np_mxfp4,
                40: np_nvfp4, 2: lambda r: np_legacy32(r, 2), 3: lambda r: np_legacy32(r, 3), 6: lambda r: np_legacy32(r, 6),
                7: lambda r: np_legacy32(r, 7), 17: lambda r: np_grid_formats(17, r, synth.codebook(17)),
                22: lambda r: np_grid_formats(22, r, synth.codebook(22)), 18: lambda r: np_grid_formats(18, r, synth.codebook(18)),
                21: lambda r: np_grid_formats(21, r, synth.codebook(21))}[dt](raw)
    want = np.asarray(want, np.float32).reshape(-1)
    assert np.all(np.isfinite(got)) and np.abs(got).max() > 0
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_block_size_tables_agree():
    # the block sizes are written down in five places (the library's header via backend.DType, the oracle, the two
    # generators, the benchmark): one disagreement would make a bank the wrong size
    import importlib.util
    import os

    from moe4all_b200 import DType, devgen

    spec = importlib.util.spec_from_file_location("bench_for_tables", os.path.join(os.path.dirname(os.path.dirname(__file__)), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert set(synth.BLOCKS) == set(devgen.BLOCKS) == set(bench.BANK_BLOCK) == set(bench.BANK_TYPES.values())
    for dt, (elems, nbytes, _slots) in synth.BLOCKS.items():
        assert devgen.BLOCKS[dt][:2] == (elems, nbytes) and bench.BANK_BLOCK[dt] == (elems, nbytes)
        assert DType(dt).row_bytes(8 * elems) == 8 * nbytes == orc.row_bytes(dt, 8 * elems)
        with pytest.raises(ValueError):
            DType(dt).row_bytes(elems + 1)


def test_ragged_block_count_rejected():
    with pytest.raises(ValueError):
        orc.dequant(orc.DT_Q4K, np.zeros(144, np.uint8), 100)


# ---- dot ------------------------------------------------------------------------------------------

def dot_8lane_longdouble(a, b):
    """crates/infr-cpu/src/kernels.rs:6568-6583 with each fma evaluated in extended precision and
    rounded once to f32."""
    ld = np.longdouble
    acc = [F32(0)] * 8
    n = len(a)
    for c in range(n // 8):
        for j in range(8):
            acc[j] = F32(ld(a[8 * c + j]) * ld(b[8 * c + j]) + ld(acc[j]))
    s = F32(0)
    for j in range(8):
        s = F32(s + acc[j])
    for i in range(n // 8 * 8, n):
        s = F32(ld(a[i]) * ld(b[i]) + ld(s))
    return s


@pytest.mark.parametrize("n", [8, 64, 67, 256])
def test_dot_lane_order(n):
    rng = np.random.default_rng(n)
    a = rng.normal(size=n).astype(F32) * F32(1e3)
    b = rng.normal(size=n).astype(F32)
    want = dot_8lane_longdouble(a, b)
    assert orc.dot(a, b) == want
    assert orc.dot(a, b, scalar=True) == want  # AVX2 form == scalar form (kernels.rs:6697-6719)


def test_dot_order_is_not_a_plain_sum():
    # the 8-lane order differs from a left-to-right sum on cancellation-heavy data: the oracle must
    # follow the former
    rng = np.random.default_rng(1)
    a = (rng.normal(size=512) * 1e4).astype(F32)
    b = rng.normal(size=512).astype(F32)
    seq = F32(0)
    for x, y in zip(a, b):
        seq = F32(seq + F32(x * y))
    assert orc.dot(a, b) == dot_8lane_longdouble(a, b)
    assert orc.dot(a, b) != seq


# ---- routing vectors --------------------------------------------------------------------------------

def gen(n, salt):
    return synth.gen_f32(n, salt)


def moe_ref_numpy(x, router, gate, up, down, ne, n_expert, n_used, nff, scale, gating, bias, groups, groups_used, given=None,
                  act="silu", clamp=None, weight_before=False, down_scale=None):
    """`moe_ref` of crates/infr-llama/tests/seam_op_parity.rs:2245-2343 (plain sequential f32 dots)."""
    def dot(a, b):
        s = F32(0)
        for u, v in zip(a, b):
            s = F32(s + F32(u * v))
        return s
    logits = np.array([dot(router[e * ne:(e + 1) * ne], x) for e in range(n_expert)], F32)
    if gating == "softmax":
        p = np.exp(logits - logits.max(), dtype=F32)
        ps = F32(0)
        for v in p:
            ps = F32(ps + v)
        probs = (p / ps).astype(F32)
    elif gating == "sigmoid":
        probs = (F32(1) / (F32(1) + np.exp(-logits, dtype=F32))).astype(F32)
    else:
        sp = np.where(logits > 20, logits, np.log(F32(1) + np.exp(logits, dtype=F32), dtype=F32))
        probs = np.sqrt(sp, dtype=F32)
    sel = probs.copy() if bias is None else (probs + bias).astype(F32)
    if groups > 1 and groups_used > 0:
        per = n_expert // groups
        gs = [float(np.sort(sel[g * per:(g + 1) * per])[-2:].sum()) for g in range(groups)]
        keep = sorted(range(groups), key=lambda g: -gs[g])[:groups_used]
        for g in range(groups):
            if g not in keep:
                sel[g * per:(g + 1) * per] = -np.inf
    idx = sorted(range(n_expert), key=lambda e: -sel[e])[:n_used] if given is None else [int(e) for e in given]
    wsum = F32(0)
    for e in idx:
        wsum = F32(wsum + probs[e])
    out = np.zeros(ne, F32)
    silu = lambda z: F32(z / (F32(1) + np.exp(-z, dtype=F32)))
    gelu = lambda z: F32(F32(0.5) * z * (F32(1) + np.tanh(F32(0.7978846) * (z + F32(0.044715) * z * z * z), dtype=F32)))
    sigm = lambda z: F32(F32(1) / (F32(1) + np.exp(-z, dtype=F32)))
    fn = {"silu": silu, "gelu": gelu, "sigmoid": sigm}[act]

    def gated(g, u):  # gated_act_fn, crates/infr-cpu/src/kernels.rs:6671-6683
        if clamp is not None:
            g, u = min(g, F32(clamp)), min(max(u, F32(-clamp)), F32(clamp))
        return F32(fn(g) * u)
    for e in idx:
        gs_, ds_ = e * nff * ne, e * ne * nff
        w_e = F32(F32(probs[e] / wsum) * F32(scale))
        wp = w_e if weight_before else F32(1)
        a = np.array([gated(F32(wp * dot(gate[gs_ + j * ne: gs_ + (j + 1) * ne], x)), F32(wp * dot(up[gs_ + j * ne: gs_ + (j + 1) * ne], x)))
                      for j in range(nff)], F32)
        w_out = F32(1) if weight_before else w_e
        for i in range(ne):
            y = dot(down[ds_ + i * nff: ds_ + (i + 1) * nff], a)
            if down_scale is not None:
                y = F32(y * down_scale[e])
            out[i] = F32(out[i] + F32(w_out * y))
    return out, idx


def run_f32_case(lead, salts, gating, gname, bias=None, groups=0, groups_used=0, n_used=2, given=None, **variant):
    ne = nff = 32
    n_expert = len(lead)
    x = np.ones((1, ne), F32)
    router = np.zeros(n_expert * ne, F32)
    router[::ne] = lead
    gate, up, down = gen(n_expert * nff * ne, salts[0]), gen(n_expert * nff * ne, salts[1]), gen(n_expert * ne * nff, salts[2])
    res = orc.moe_ffn(x, router, gate, up, down, n_expert=n_expert, n_used=n_used, n_ff_exp=nff, scale=1.0,
                      gate_dtype=orc.DT_F32, up_dtype=orc.DT_F32, down_dtype=orc.DT_F32, gating=gating,
                      bias=bias, groups=groups, groups_used=groups_used, threads=2,
                      expert_ids=None if given is None else np.asarray(given, np.int32).reshape(1, n_used),
                      act={None: 0, "gelu": 1, "sigmoid": 2}[variant.get("act")], swiglu_clamp=variant.get("clamp") or 0.0,
                      weight_before=variant.get("weight_before", False), down_scale=variant.get("down_scale"))
    want, idx = moe_ref_numpy(x[0], router, gate, up, down, ne, n_expert, n_used, nff, 1.0, gname, bias, groups, groups_used, given,
                              **variant)
    return res, want, idx


def test_sqrt_softplus_vector():
    # crates/infr-llama/tests/seam_op_parity.rs:2352-2443: leads [24, 1, .75, .5, -1.5, -1] -> experts 0, 1
    res, want, idx = run_f32_case(np.array([24.0, 1.0, 0.75, 0.5, -1.5, -1.0], F32), (12, 13, 14),
                                  orc.GATING_SQRT_SOFTPLUS, "sqrt_softplus")
    assert res.ids[0].tolist() == [0, 1] == idx
    assert np.max(np.abs(res.dst[0] - want)) < 1e-4  # the reference's own bound (:2430-2436)
    assert np.abs(want).max() > 0


def test_groups_bias_vector():
    # seam_op_parity.rs:2453-2554: sigmoid gating, 2 groups / 1 used, +0.6 bias on experts 4..7:
    # biased probabilities pick group 1 and experts 4, 5; unbiased probabilities drive the weights
    lead = np.array([3.0, 2.5, 2.0, 1.5, 1.0, 0.9, 0.8, 0.7], F32)
    bias = np.array([0, 0, 0, 0, 0.6, 0.6, 0.6, 0.6], F32)
    res, want, idx = run_f32_case(lead, (15, 16, 17), orc.GATING_SIGMOID, "sigmoid", bias=bias, groups=2, groups_used=1)
    assert res.ids[0].tolist() == [4, 5] == idx
    assert np.max(np.abs(res.dst[0] - want)) < 1e-4
    p4, p5 = 1 / (1 + np.exp(-1.0)), 1 / (1 + np.exp(-0.9))
    np.testing.assert_allclose(res.wts[0], [p4 / (p4 + p5), p5 / (p4 + p5)], rtol=1e-6)
    # without the bias group 0 wins (experts 0, 1): the bias semantics are what flips it
    res2, _, _ = run_f32_case(lead, (15, 16, 17), orc.GATING_SIGMOID, "sigmoid", bias=None, groups=2, groups_used=1)
    assert res2.ids[0].tolist() == [0, 1]


def test_hash_routing_vector():
    # Op::MoeFfn::expert_ids (crates/infr-core/src/graph.rs:1320-1351; CPU crates/infr-cpu/src/lib.rs:
    # 3776-3792; test crates/infr-llama/tests/seam_op_parity.rs:5700-5897): the given experts replace
    # the selection only; the weights are the router's probabilities at those experts, not uniform
    lead = np.array([2.0, 1.0, 0.75, 0.5, -1.5, -1.0], F32)
    res, want, idx = run_f32_case(lead, (12, 13, 14), orc.GATING_SOFTMAX, "softmax", given=[4, 1])
    assert res.ids[0].tolist() == [4, 1] == idx
    assert np.max(np.abs(res.dst[0] - want)) < 1e-4
    p = np.exp(lead - lead.max())
    np.testing.assert_allclose(res.wts[0], [p[4] / (p[4] + p[1]), p[1] / (p[4] + p[1])], rtol=1e-6)
    assert abs(res.wts[0][0] - 0.5) > 0.3
    # ids past n_expert, a bias or groups beside the ids: refused (graph.rs:1304-1308; lib.rs:3782-3788)
    with pytest.raises(ValueError):
        run_f32_case(lead, (12, 13, 14), orc.GATING_SOFTMAX, "softmax", given=[6, 1])
    with pytest.raises(ValueError):
        run_f32_case(lead, (12, 13, 14), orc.GATING_SOFTMAX, "softmax", given=[4, 1], bias=np.zeros(6, F32))


@pytest.mark.parametrize("variant", [
    dict(act="gelu"),
    dict(act="sigmoid"),
    dict(clamp=0.02),                 # DeepSeek-V4 swiglu_clamp: act(min(g, l)) * clamp(u, -l, l)
    dict(weight_before=True),         # llama4: routing weight on gate and up before the activation
    dict(down_scale=np.array([0.5, 2.0, 1.5, 1.0, 0.25, 3.0], F32)),  # diffusion-gemma ffn_down_exps.scale
    dict(act="gelu", clamp=0.03, down_scale=np.array([2.0, 0.5, 1.5, 1.0, 0.25, 3.0], F32)),
], ids=["gelu", "sigmoid", "clamp", "weight_before", "down_scale", "gelu_clamp_scale"])
def test_op_variant_vectors(variant):
    # the remaining Op::MoeFfn forms against a from-definition restatement (crates/infr-cpu/src/lib.rs:
    # 4144-4181 gate/up with weight_before and the clamp, :4246-4258 down_scale, :4287-4303 the sum;
    # activations crates/infr-cpu/src/kernels.rs:6662-6683)
    lead = np.array([2.0, 1.0, 0.75, 0.5, -1.5, -1.0], F32)
    res, want, idx = run_f32_case(lead, (12, 13, 14), orc.GATING_SOFTMAX, "softmax", **variant)
    plain, _, _ = run_f32_case(lead, (12, 13, 14), orc.GATING_SOFTMAX, "softmax")
    assert res.ids[0].tolist() == [0, 1] == idx
    scale = np.abs(want).max()
    assert np.max(np.abs(res.dst[0] - want)) < 1e-4 * max(scale, 1.0)
    assert np.max(np.abs(res.dst[0] - plain.dst[0])) > 1e-2 * scale  # the variant is not a no-op here


def test_tie_goes_to_lower_index():
    # stable descending sort (crates/infr-cpu/src/lib.rs:3847-3850): equal scores keep index order
    lead = np.array([0.5, 2.0, 2.0, 0.5, 2.0, -1.0], F32)
    res, _, _ = run_f32_case(lead, (1, 2, 3), orc.GATING_SOFTMAX, "softmax")
    assert res.ids[0].tolist() == [1, 2]


@pytest.mark.parametrize("rows", [1, 4])
def test_tiny_sinusoid_layer(rows):
    # crates/infr-vulkan/src/adapter.rs:27365-27413: ne = nff = 32, 4 experts, top-2, scale 1.3,
    # sinusoidal fillers; f32 banks here (the reference quantises them to Q8_0 first)
    ne = nff = 32
    n_expert, n_used, scale = 4, 2, 1.3
    f = lambda i, s: (np.sin(i.astype(F32) * F32(s)) * F32(0.5)).astype(F32)
    i_r, i_g, i_d = np.arange(n_expert * ne), np.arange(n_expert * nff * ne), np.arange(n_expert * ne * nff)
    router = (f(i_r, 0.037) + (i_r // ne).astype(F32) * F32(0.15)).astype(F32)
    gate, up, down = f(i_g, 0.017), f(i_g, 0.023), f(i_d, 0.029)
    x = (f(np.arange(rows * ne), 0.11) + F32(0.05)).astype(F32).reshape(rows, ne)
    res = orc.moe_ffn(x, router, gate, up, down, n_expert=n_expert, n_used=n_used, n_ff_exp=nff, scale=scale,
                      gate_dtype=orc.DT_F32, up_dtype=orc.DT_F32, down_dtype=orc.DT_F32, threads=1)
    # float64 reference
    R, G, U, D = (router.reshape(n_expert, ne).astype(np.float64), gate.reshape(n_expert, nff, ne).astype(np.float64),
                  up.reshape(n_expert, nff, ne).astype(np.float64), down.reshape(n_expert, ne, nff).astype(np.float64))
    for t in range(rows):
        xt = x[t].astype(np.float64)
        lg = R @ xt
        p = np.exp(lg - lg.max())
        p /= p.sum()
        idx = np.argsort(-p, kind="stable")[:n_used]
        out = np.zeros(ne)
        for e in idx:
            g, u = G[e] @ xt, U[e] @ xt
            out += p[e] / p[idx].sum() * scale * (D[e] @ (g / (1 + np.exp(-g)) * u))
        assert res.ids[t].tolist() == idx.tolist()
        assert np.max(np.abs(res.dst[t] - out)) < 1e-4


def test_ep_bands_sum_to_full():
    # Op::MoeFfn::ep_band (crates/infr-core/src/graph.rs:1309-1319): band partials add up
    L = synth.make_layer(3, 256, 8, 256, router_std=0.05)
    x = synth.activations(4, 3, 256)
    kw = dict(n_expert=8, n_used=2, n_ff_exp=256)
    full = orc.moe_ffn(x, L.router, L.gate, L.up, L.down, **kw)
    parts = [orc.moe_ffn(x, L.router, L.gate, L.up, L.down, ep_band=(lo, 4), **kw) for lo in (0, 4)]
    assert np.array_equal(parts[0].ids, full.ids)
    np.testing.assert_allclose(parts[0].dst + parts[1].dst, full.dst, rtol=1e-5, atol=1e-7)


def test_elementwise_ops():
    rng = np.random.default_rng(0)
    x, w = rng.normal(size=(3, 64)).astype(F32), rng.normal(size=64).astype(F32)
    got = orc.rmsnorm(x, w, 1e-6)
    want = x / np.sqrt((x.astype(np.float64) ** 2).mean(1, keepdims=True) + 1e-6) * w
    np.testing.assert_allclose(got, want, rtol=2e-6)
    g = rng.normal(size=(3, 64)).astype(F32)
    np.testing.assert_allclose(orc.gated_act_silu(g, x), g / (1 + np.exp(-g)) * x, rtol=2e-6)
    gate = rng.normal(size=3).astype(F32)
    np.testing.assert_allclose(orc.moe_shared_add(x, g, gate), x + (1 / (1 + np.exp(-gate)))[:, None] * g, rtol=2e-6, atol=1e-7)
    assert np.array_equal(orc.add(x, g), x + g)
