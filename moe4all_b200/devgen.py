"""Synthetic layer weights generated directly in device memory (torch is used for the random
streams and the allocation only).  Same distributions as synth.make_layer: random block payload,
f16 scales ~ U[1e-4, 1e-3], router ~ N(0, 0.02)."""
from __future__ import annotations

import torch


def _scales(n, gen, device):
    return (torch.rand(n, generator=gen, device=device) * 9e-4 + 1e-4).to(torch.float16).view(torch.uint8).reshape(n, 2)


def q4k_bank(n_blocks: int, gen, device) -> torch.Tensor:
    t = torch.randint(0, 256, (n_blocks, 144), dtype=torch.uint8, generator=gen, device=device)
    t[:, 0:2] = _scales(n_blocks, gen, device)
    t[:, 2:4] = _scales(n_blocks, gen, device)
    return t.reshape(-1)


def q6k_bank(n_blocks: int, gen, device) -> torch.Tensor:
    t = torch.randint(0, 256, (n_blocks, 210), dtype=torch.uint8, generator=gen, device=device)
    t[:, 208:210] = _scales(n_blocks, gen, device)
    return t.reshape(-1)


# GGUF type number -> (elements per block, bytes per block, offsets of the f16 scale slots, scale factor)
BLOCKS = {12: (256, 144, (0, 2), 1.0), 13: (256, 176, (0, 2), 1.0), 14: (256, 210, (208,), 1.0), 8: (32, 34, (0,), 2.0),
          20: (32, 18, (0,), 2.0), 23: (256, 136, (0,), 1.0), 2: (32, 18, (0,), 32.0), 3: (32, 20, (0, 2), 32.0), 6: (32, 22, (0,), 16.0),
          7: (32, 24, (0, 2), 16.0), 10: (256, 84, (80, 82), 64.0), 11: (256, 110, (108,), 8.0), 39: (32, 17, (), 1.0),
          40: (64, 36, (), 1.0), 42: (64, 18, (0,), 64.0),
          17: (256, 74, (0,), 0.5), 22: (256, 82, (0,), 0.5), 18: (256, 98, (0,), 0.2), 21: (256, 110, (0,), 0.2)}


def bank(dtype: int, n_elem: int, gen, device) -> torch.Tensor:
    """Random blocks of GGUF type `dtype` (12 Q4_K, 13 Q5_K, 14 Q6_K, 8 Q8_0, 20 IQ4_NL, 23 IQ4_XS) holding n_elem weights."""
    if dtype == 12:
        return q4k_bank(n_elem // 256, gen, device)
    if dtype == 14:
        return q6k_bank(n_elem // 256, gen, device)
    elems, nbytes, slots, k = BLOCKS[dtype]
    n = n_elem // elems
    t = torch.randint(0, 256, (n, nbytes), dtype=torch.uint8, generator=gen, device=device)
    for o in slots:
        t[:, o:o + 2] = ((torch.rand(n, generator=gen, device=device) * 9e-4 + 1e-4) * k).to(torch.float16).view(torch.uint8).reshape(n, 2)
    if dtype == 39:  # MXFP4: one E8M0 exponent byte per block, 2^-14 .. 2^-9
        t[:, 0] = torch.randint(114, 120, (n,), dtype=torch.uint8, generator=gen, device=device)
    if dtype == 40:  # NVFP4: four UE4M3 sub-scale bytes per block with exponent field 0 or 1
        t[:, 0:4] = torch.randint(1, 16, (n, 4), dtype=torch.uint8, generator=gen, device=device)
    return t.reshape(-1)


class DeviceLayer:
    """One MoE layer's tensors as torch CUDA tensors plus Buffer handles on them."""

    def __init__(self, be, seed, ne, n_expert, n_ff, sh_ff=0, gated_shared=True, device="cuda:0", router_std=0.02,
                 band=None, dtypes=(12, 12, 14)):
        """band = (lo, n_local): keep only that slice of the expert banks (an expert-parallel rank);
        the bytes equal the same slice of the un-banded layer with the same seed.
        dtypes = GGUF type numbers of the gate, up and down banks."""
        gen = torch.Generator(device=device)
        gen.manual_seed(seed)
        self.ne, self.n_expert, self.n_ff, self.sh_ff = ne, n_expert, n_ff, sh_ff
        self.t = {}
        self.t["router"] = torch.randn(n_expert, ne, generator=gen, device=device) * router_std
        self.dtypes = tuple(dtypes)
        gd, ud, dd = self.dtypes
        self.t["gate"] = bank(gd, n_expert * n_ff * ne, gen, device)
        self.t["up"] = bank(ud, n_expert * n_ff * ne, gen, device)
        self.t["down"] = bank(dd, n_expert * ne * n_ff, gen, device)
        if sh_ff:
            self.t["sh_gate"] = bank(gd, sh_ff * ne, gen, device)
            self.t["sh_up"] = bank(ud, sh_ff * ne, gen, device)
            self.t["sh_down"] = bank(dd, ne * sh_ff, gen, device)
            if gated_shared:
                self.t["sh_gate_inp"] = torch.randn(ne, generator=gen, device=device) * router_std
        if band is not None:
            lo, n_local = band
            per_elem = lambda dt: BLOCKS[dt][1] / BLOCKS[dt][0]
            for k, per in (("gate", int(n_ff * ne * per_elem(gd))), ("up", int(n_ff * ne * per_elem(ud))), ("down", int(ne * n_ff * per_elem(dd)))):
                self.t[k] = self.t[k][lo * per:(lo + n_local) * per].clone()
        # 16 spare bytes after each bank: block decoders may read a word pair at the very end
        for k in list(self.t):
            v = self.t[k]
            padded = torch.empty(v.numel() * v.element_size() + 16, dtype=torch.uint8, device=device)
            padded[: v.numel() * v.element_size()] = v.reshape(-1).view(torch.uint8)
            self.t[k] = padded
        self.b = {k: be.wrap(v.data_ptr(), v.numel() - 16) for k, v in self.t.items()}

    def host(self):
        """synth.LayerWeights with the same bytes (for the CPU oracle)."""
        from .synth import LayerWeights
        import numpy as np
        L = LayerWeights(self.ne, self.n_expert, self.n_ff, self.sh_ff, "sh_gate_inp" in self.t)
        get = lambda k: self.t[k][:-16].cpu().numpy() if k in self.t else None
        L.router = get("router").view(np.float32).reshape(self.n_expert, self.ne)
        L.gate, L.up, L.down = get("gate"), get("up"), get("down")
        L.gate_dtype, L.up_dtype, L.down_dtype = self.dtypes
        L.sh_gate, L.sh_up, L.sh_down = get("sh_gate"), get("sh_up"), get("sh_down")
        gi = get("sh_gate_inp")
        L.sh_gate_inp = gi.view(np.float32) if gi is not None else None
        return L
