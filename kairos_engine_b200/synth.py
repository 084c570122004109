"""Seeded synthetic layers and inputs with the shapes and value distributions the benchmark
configurations name (no model file is needed): router N(0, 0.02) f32, expert and shared
weights N(0, 0.02) quantised to Q4B on the device, norm weights and scales 1 (or uniform in
[0.5, 1.5]), hidden states N(0, 1). Layer L uses seed + 1000*L.
"""
import math

import torch

from .engine import q4b_quantize


def zipf_bias(NE, s=1.2, seed=0, device="cuda"):
    """Per-expert logit bias b_e = log(rank_e^-s / Z) under a seeded random expert permutation."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    perm = torch.randperm(NE, generator=g)
    ranks = torch.empty(NE, dtype=torch.float64)
    ranks[perm] = torch.arange(1, NE + 1, dtype=torch.float64)
    p = ranks.pow(-s)
    return (p / p.sum()).log().to(torch.float32).to(device)


def make_layer(cfg, seed, device="cuda", wstd=0.02, rand_norms=False, bias=None, chunk_rows=1 << 16):
    """One layer as a dict of torch CUDA tensors in the reference's layouts."""
    E, NE, FFE, FFS = cfg["E"], cfg["NE"], cfg["FFE"], cfg["FFS"]
    g = torch.Generator(device=device).manual_seed(seed)

    def vec(n):
        if rand_norms:
            return torch.rand(n, generator=g, device=device) + 0.5
        return torch.ones(n, device=device)

    def qmat(rows, cols):
        codes = torch.empty((rows, cols // 2), dtype=torch.uint8, device=device)
        bs = torch.empty((rows, cols // 32), dtype=torch.int16, device=device)
        for r0 in range(0, rows, chunk_rows):          # bounded temporary: chunk_rows x cols f32
            r1 = min(rows, r0 + chunk_rows)
            w = torch.randn((r1 - r0, cols), generator=g, device=device) * wstd
            c, b = q4b_quantize(w)
            codes[r0:r1], bs[r0:r1] = c, b
        return codes, bs

    out = dict(router_w=torch.randn((NE, E), generator=g, device=device) * 0.02,
               router_scale=vec(E), router_bias=bias, ffn_norm=vec(E), post_ffw1=vec(E), pre_ffw2=vec(E),
               post_ffw2=vec(E), post_ffw=vec(E), dexps_scale=vec(NE))
    out["gu_codes"], out["gu_bs"] = qmat(NE * 2 * FFE, E)
    out["dn_codes"], out["dn_bs"] = qmat(NE * E, FFE)
    out["sg_codes"], out["sg_bs"] = qmat(FFS, E)
    out["su_codes"], out["su_bs"] = qmat(FFS, E)
    out["sd_codes"], out["sd_bs"] = qmat(E, FFS)
    return out


def make_inputs(cfg, M, seed, device="cuda", rms_normed=False, eps=1e-6):
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn((M, cfg["E"]), generator=g, device=device)
    if rms_normed:
        x = x / torch.sqrt((x * x).mean(dim=1, keepdim=True) + eps)
    return x


def layer_to_host(layer):
    """Device layer dict -> numpy arrays (what a host caller, or the CPU checker, would hold)."""
    out = {}
    for k, v in layer.items():
        if v is None:
            out[k] = None
        elif v.dtype == torch.int16:
            out[k] = v.cpu().numpy().view("uint16")
        else:
            out[k] = v.cpu().numpy()
    return out


def algorithmic_bytes_per_layer(cfg, M=1, U=None):
    """Bytes one layer must move from HBM for M tokens that select U distinct experts:
    U experts + shared expert + f32 router + 6 norm/scale vectors + per-expert down scales +
    the residual in and out."""
    E, NE, FFE, FFS = cfg["E"], cfg["NE"], cfg["FFE"], cfg["FFS"]
    U = cfg["NU"] if U is None else U
    expert = 2 * FFE * (E // 2) + 2 * FFE * (E // 32) * 2 + E * (FFE // 2) + E * (FFE // 32) * 2
    shared = 2 * (FFS * (E // 2) + FFS * (E // 32) * 2) + E * (FFS // 2) + E * (FFS // 32) * 2
    return U * expert + shared + NE * E * 4 + 6 * E * 4 + NE * 4 + 2 * M * E * 4


def flops_per_token_layer(cfg):
    E, NE, NU, FFE, FFS = cfg["E"], cfg["NE"], cfg["NU"], cfg["FFE"], cfg["FFS"]
    return 2 * (NU * (E * 2 * FFE + FFE * E) + 3 * E * FFS + E * NE)
