"""Karuzen, Ranilix, Fefozen or Batatar beside the closest existing family (Qwen3, dense GQA) at equal layer sizes: prefill and decode throughput
through LLMEngine, plus per-op times and roofline fractions.  Random weights, synthetic prompts.  Used by
`bench.py --compare-families`; the default benchmark does not touch this module.

Roofline of an op: time_min = max(flops / bf16 peak, bytes / HBM peak) from its algorithmic work (logical sizes, weights
and cache rows once); frac = time_min / measured time."""
from __future__ import annotations

import time
from typing import Dict, List

import numpy as np

BLOCK = 64

# (name, width, heads, ff, layers, moe) - layer shapes of small / mid dense models; head size 128 in both families
SIZES = [
    {"name": "w1024-h16-ff3072", "width": 1024, "heads": 16, "ff": 3072, "layers": 4, "vocab": 32768},
    {"name": "w2048-h16-ff6144", "width": 2048, "heads": 16, "ff": 6144, "layers": 4, "vocab": 32768},
    {"name": "w1024-h16-moe16x2-ff1536", "width": 1024, "heads": 16, "ff": 4608, "layers": 4, "vocab": 32768,
     "moe": {"experts": 16, "top": 2, "expert_ff": 1536, "shared_ff": 1536}},
]
KV_RANK, Q_RANK, DIM = 128, 512, 128


def karuzen_config(sz: dict) -> dict:
    mixer = {"heads": sz["heads"], "dim": DIM, "vdim": DIM, "kv_rank": KV_RANK, "q_rank": Q_RANK, "scale": DIM ** -0.5}
    if "moe" in sz:
        m = sz["moe"]
        mlp = {"kind": "moe", "router": {"experts": m["experts"], "top": m["top"], "scale": 1.0}, "expert": {"ff": m["expert_ff"]},
               "shared": {"ff": m["shared_ff"]}}
    else:
        mlp = {"kind": "dense", "ff": sz["ff"]}
    return {"architecture": "Karuzen", "vocab": sz["vocab"], "width": sz["width"], "norm": {"eps": 1e-5},
            "layers": [{"type": "latent_attention", "mixer": dict(mixer), "mlp": dict(mlp)} for _ in range(sz["layers"])], "loop": None}


def karuzen_weights(cfg: dict, seed: int = 0):
    """(name, bf16 CPU tensor) pairs, generated one at a time."""
    import torch
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(o, i):
        return (torch.randn(o, i, generator=g) * i ** -0.5).bfloat16()

    def norm(p):
        yield p, torch.ones(W).bfloat16()
        yield p + ".b", torch.zeros(W).bfloat16()
        yield p + ".alpha", torch.tensor(0.5).bfloat16()

    yield "embed", (torch.randn(cfg["vocab"], W, generator=g) * 0.05).bfloat16()
    yield from norm("final.norm")
    for i, ly in enumerate(cfg["layers"]):
        m, p = ly["mixer"], f"l{i}."
        yield from norm(p + "norm1")
        H, d, vd, kr, qr = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]
        yield p + "mix.dq", mat(qr, W)
        yield p + "mix.dq.norm", torch.ones(qr).bfloat16()
        yield p + "mix.uq", mat(H * d, qr)
        yield p + "mix.dkv", mat(kr, W)
        yield p + "mix.dkv.norm", torch.ones(kr).bfloat16()
        yield p + "mix.uk", mat(H * d, kr)
        yield p + "mix.uv", mat(H * vd, kr)
        yield p + "mix.o", mat(W, H * vd)
        f = ly["mlp"]
        if f["kind"] == "dense":
            yield p + "mlp.gate", mat(f["ff"], W)
            yield p + "mlp.up", mat(f["ff"], W)
            yield p + "mlp.down", mat(W, f["ff"])
        else:
            E, ef, sf = f["router"]["experts"], f["expert"]["ff"], f["shared"]["ff"]
            yield p + "mlp.router", mat(E, W)
            yield p + "mlp.correction", torch.zeros(E).bfloat16()
            for e in range(E):
                yield p + f"mlp.e{e}.up", mat(ef, W)
                yield p + f"mlp.e{e}.down", mat(W, ef)
            yield p + "mlp.shared.up", mat(sf, W)
            yield p + "mlp.shared.down", mat(W, sf)
            yield p + "mlp.shared.sg", mat(1, W)


# ---- Ranilix at the same sizes: layers alternate between the windowed attention mixer (as many heads as the Qwen3 layer, 8 key /
# value heads of 128) and the parallel mixer (half the heads as causal attention, half as retention heads of key size 64), a
# squared-relu feed-forward of 1.5 ff (two matrices: the parameter count of the gated one with three)
R_WINDOW, R_DIM, R_RET_DIM = 256, 128, 64


def ranilix_config(sz: dict) -> dict:
    H, W = sz["heads"], sz["width"]
    att = {"heads": H, "kv_heads": 8, "dim": R_DIM, "vdim": R_DIM, "scale": R_DIM ** -0.5, "mask": {"size": R_WINDOW},
           "rot": {"dims": 64, "base": 10000.0}, "v_mix": True}
    par = {"left": {"heads": H // 2, "kv_heads": 4, "dim": R_DIM, "vdim": R_DIM, "scale": R_DIM ** -0.5, "rot": {"dims": 64, "base": 10000.0}},
           "left_scale": 1.0,
           "right": {"heads": H // 2, "dim": R_RET_DIM, "vdim": R_DIM, "rot": {"dims": R_RET_DIM, "base": 10000.0},
                     "decay": [1.0 - 2.0 ** (-5 - 5 * i / max(1, H // 2 - 1)) for i in range(H // 2)]},
           "right_scale": 1.0}
    mlp = {"kind": "dense", "ff": sz["ff"] * 3 // 2}
    layers = [{"type": "attention" if i % 2 == 0 else "parallel", "mixer": dict(att if i % 2 == 0 else par), "mlp": dict(mlp)}
              for i in range(sz["layers"])]
    return {"architecture": "Ranilix", "vocab": sz["vocab"], "width": W, "norm": {"eps": 1e-5}, "embedding": {"scale": W ** 0.5}, "layers": layers}


def ranilix_weights(cfg: dict, seed: int = 0):
    """(name, bf16 CPU tensor) pairs, generated one at a time."""
    import torch
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(o, i):
        return (torch.randn(o, i, generator=g) * i ** -0.5).bfloat16()

    yield "embed", (torch.randn(cfg["vocab"], W, generator=g) * W ** -0.5).bfloat16()
    yield "head", mat(cfg["vocab"], W)
    yield "final.norm", torch.ones(W).bfloat16()
    for i, ly in enumerate(cfg["layers"]):
        m, p = ly["mixer"], f"l{i}."
        yield p + "norm1", torch.ones(W).bfloat16()
        yield p + "norm2", torch.ones(W).bfloat16()
        if ly["type"] == "attention":
            H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * vd)):
                yield p + "mix." + n, mat(rows, W)
                yield p + "mix." + n + ".b", torch.zeros(rows).bfloat16()
            yield p + "mix.q.norm", torch.ones(d).bfloat16()
            yield p + "mix.k.norm", torch.ones(d).bfloat16()
            yield p + "mix.vmix", torch.tensor(0.3).bfloat16()
            yield p + "mix.sink", torch.zeros(H).bfloat16()
            yield p + "mix.g", mat(H * vd, W)
            yield p + "mix.o", mat(W, H * vd)
        else:
            L, R = m["left"], m["right"]
            yield p + "mix.left.q", mat(L["heads"] * L["dim"], W)
            yield p + "mix.left.k", mat(L["kv_heads"] * L["dim"], W)
            yield p + "mix.left.v", mat(L["kv_heads"] * L["vdim"], W)
            yield p + "mix.left.o", mat(W, L["heads"] * L["vdim"])
            yield p + "mix.right.q", mat(R["heads"] * R["dim"], W)
            yield p + "mix.right.k", mat(R["heads"] * R["dim"], W)
            yield p + "mix.right.v", mat(R["heads"] * R["vdim"], W)
            yield p + "mix.right.g", mat(R["heads"] * R["vdim"], W)
            yield p + "mix.right.o", mat(W, R["heads"] * R["vdim"])
        yield p + "mlp.up", mat(ly["mlp"]["ff"], W)
        yield p + "mlp.down", mat(W, ly["mlp"]["ff"])


def ranilix_rooflines(cfg, prof: Dict[str, float], N: int, B: int, ctx_lens: List[int], q_lens: List[int], pk) -> dict:
    """Per-op roofline of one profiled step: the times are sums over the layers, the work is summed the same way.  The
    retention scan runs on the fp32 FMA pipe (its state is fp32): its fraction is against that pipe's peak (pk["fp32"])."""
    W = cfg["width"]
    work = {k: [0.0, 0.0] for k in ("gemm_in", "gemm_o", "gemm_up", "gemm_down", "attention", "retention_scan")}

    def add(name, flops, nbytes):
        work[name][0] += flops
        work[name][1] += nbytes

    def attn(a, window):
        H, G, d, vd = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        pairs, keys = 0, 0
        for q, c in zip(q_lens, ctx_lens):
            for t in range(c - q, c):
                pairs += min(t + 1, window) if window else t + 1
            keys += min(c, q + window - 1) if window else c
        add("attention", 2.0 * pairs * H * (d + vd), 2.0 * (keys * G * (d + vd) + N * H * (d + vd)))

    for ly in cfg["layers"]:
        m, ff = ly["mixer"], ly["mlp"]["ff"]
        if ly["type"] == "attention":
            H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            n_in, n_o = H * d + G * d + G * vd + H * vd, H * vd
            attn(m, m["mask"]["size"])
        else:
            L, R = m["left"], m["right"]
            n_in = L["heads"] * L["dim"] + L["kv_heads"] * (L["dim"] + L["vdim"]) + R["heads"] * (2 * R["dim"] + 2 * R["vdim"])
            n_o = L["heads"] * L["vdim"] + R["heads"] * R["vdim"]
            attn(L, 0)
            add("retention_scan", 4.0 * N * R["heads"] * R["dim"] * R["vdim"],
                4.0 * (N * R["heads"] * (2 * R["dim"] + 2 * R["vdim"]) + 2 * B * R["heads"] * R["dim"] * R["vdim"]))
        add("gemm_in", 2.0 * N * n_in * W, 2.0 * n_in * W + 2.0 * N * W + 4.0 * N * n_in)
        add("gemm_o", 2.0 * N * n_o * W, 2.0 * n_o * W + 2.0 * N * n_o + 4.0 * N * W)
        add("gemm_up", 2.0 * N * ff * W, 2.0 * (ff * W + N * (ff + W)))
        add("gemm_down", 2.0 * N * ff * W, 2.0 * (ff * W + N * ff) + 4.0 * N * W)
    out = {}
    for name, (fl, by) in work.items():
        if name in prof and fl > 0:
            if name == "retention_scan":
                tmin = max(fl / (pk.get("fp32", 70.0) * 1e12), by / (pk["hbm"] * 1e9)) * 1e6
                out[name] = {"us": round(prof[name], 2), "fp32_tflops": round(fl / prof[name] / 1e6, 2), "gbs": round(by / prof[name] / 1e3, 1),
                             "roofline_frac": round(tmin / prof[name], 3)}
            else:
                out[name] = _roof(fl, by, prof[name], pk)
    for name in ("rms_norm_pair", "qkv_prep", "retention_prep", "retention_gate", "embed", "final_norm", "lm_head"):
        if name in prof:
            out[name] = {"us": round(prof[name], 2)}
    return out


# ---- Fefozen at the same sizes: four layers - latent attention without sink (cache rows of 96 + 32 numbers: its long portions run
# on the tcgen05 kernel), latent attention with a sink, a layer that reads the first layer's rows, a gated-delta-rule layer with
# half as many key heads as heads - with a dense tanh-gelu feed-forward of 1.5 ff (two matrices: the gated one's parameter count)
# or, in the mixture size, softmax-routed experts (two identity experts beside the real ones) behind the second and fourth mixer.
F_KV_RANK, F_ROT, F_DIM = 96, 32, 96


def fefozen_config(sz: dict) -> dict:
    H, W = sz["heads"], sz["width"]

    def latent(second, kv_from=None):
        m = {"heads": H, "dim": F_DIM, "rot_dim": F_ROT, "vdim": 128, "kv_rank": F_KV_RANK, "q_rank": Q_RANK, "scale": (F_DIM + F_ROT) ** -0.5,
             "rot": {"dims": F_ROT, "base": 10000.0}}
        if kv_from is not None:
            m["kv_from"] = kv_from
        return {"type": "latent_attention_2" if second else "latent_attention", "mixer": m}

    delta = {"type": "delta", "mixer": {"heads": H, "kv_heads": H // 2, "dim": 128, "vdim": 128, "conv": 4}}
    dense = {"kind": "dense", "ff": sz["ff"] * 3 // 2}
    if "moe" in sz:
        m = sz["moe"]
        moe = {"kind": "moe", "router": {"experts": m["experts"], "identity": 2, "top": m["top"]}, "expert": {"ff": m["expert_ff"], "limit": 7.0}}
    else:
        moe = dense
    layers = [dict(latent(True), mlp=dict(dense)), dict(latent(False), mlp=dict(moe)), dict(latent(True, 0), mlp=dict(dense)), dict(delta, mlp=dict(moe))]
    return {"architecture": "Fefozen", "vocab": sz["vocab"], "width": W, "norm": {"eps": 1e-5}, "layers": [layers[i % 4] for i in range(sz["layers"])]}


def fefozen_weights(cfg: dict, seed: int = 0):
    """(name, bf16 CPU tensor) pairs, generated one at a time."""
    import torch
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(o, i):
        return (torch.randn(o, i, generator=g) * i ** -0.5).bfloat16()

    yield "embed", (torch.randn(cfg["vocab"], W, generator=g) * 0.05).bfloat16()
    yield "final.norm", torch.zeros(W).bfloat16()
    for i, ly in enumerate(cfg["layers"]):
        m, p = ly["mixer"], f"l{i}."
        for n in ("norm1", "norm1b", "norm2", "norm2b"):
            yield p + n, torch.zeros(W).bfloat16()
        if ly["type"] == "delta":
            H, G, d, vd, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for n, rows in (("q", G * d), ("k", G * d), ("v", H * vd)):
                yield p + "mix." + n, mat(rows, W)
                yield p + "mix." + n + ".conv", (torch.randn(rows, taps, generator=g) * 0.5).bfloat16()
            yield p + "mix.b", mat(H, W)
            yield p + "mix.a", mat(H, W)
            yield p + "mix.A_log", torch.zeros(H).bfloat16()
            yield p + "mix.dt_bias", torch.zeros(H).bfloat16()
            yield p + "mix.norm", torch.ones(vd).bfloat16()
            yield p + "mix.g", mat(H * vd, W)
            yield p + "mix.o", mat(W, H * vd)
        else:
            H, d, rd, vd, kr, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            yield p + "mix.dq", mat(qr, W)
            yield p + "mix.dq.norm", torch.ones(qr).bfloat16()
            yield p + "mix.uq", mat(H * (d + rd), qr)
            if m.get("kv_from") is None:
                yield p + "mix.dkv", mat(kr + rd, W)
                yield p + "mix.dkv.norm", torch.ones(kr).bfloat16()
            yield p + "mix.uk", mat(H * d, kr)
            yield p + "mix.uv", mat(H * vd, kr)
            if ly["type"] == "latent_attention":
                yield p + "mix.sink", torch.zeros(H).bfloat16()
            yield p + "mix.g", mat(H * vd, W)
            yield p + "mix.o", mat(W, H * vd)
        f = ly["mlp"]
        if f["kind"] == "dense":
            yield p + "mlp.up", mat(f["ff"], W)
            yield p + "mlp.down", mat(W, f["ff"])
        else:
            E, I, ef = f["router"]["experts"], f["router"]["identity"], f["expert"]["ff"]
            yield p + "mlp.router", mat(E + I, W)
            yield p + "mlp.correction", torch.zeros(E + I).bfloat16()
            for e in range(E):
                yield p + f"mlp.e{e}.gate", mat(ef, W)
                yield p + f"mlp.e{e}.up", mat(ef, W)
                yield p + f"mlp.e{e}.down", mat(W, ef)


def fefozen_rooflines(cfg, prof: Dict[str, float], N: int, B: int, ctx_lens: List[int], q_lens: List[int], pk) -> dict:
    """Per-op roofline of one profiled step: the times are sums over the layers, the work is summed the same way.  The delta-rule scan
    runs on the fp32 FMA pipe (its state is fp32): its fraction is against that pipe's peak (pk["fp32"])."""
    W = cfg["width"]
    names = ("gemm_in", "gemm_uq", "absorb_uk", "attention", "absorb_uv", "gemm_o", "gemm_up", "gemm_down", "moe_gate_up", "moe_down", "delta_scan")
    work = {k: [0.0, 0.0] for k in names}

    def add(name, flops, nbytes):
        work[name][0] += flops
        work[name][1] += nbytes

    pairs = sum(q * c - q * (q - 1) // 2 for q, c in zip(q_lens, ctx_lens))       # visible (query, key) pairs
    for ly in cfg["layers"]:
        m, f = ly["mixer"], ly["mlp"]
        if ly["type"] == "delta":
            H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            n_in, n_o = 2 * G * d + 2 * H * vd + 2 * H, H * vd
            add("delta_scan", 6.0 * N * H * d * vd, 4.0 * (N * (2 * G * d + 2 * H * vd) + 2 * B * H * d * vd))
        else:
            H, d, rd, vd, kr, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            n_in, n_o = qr + (kr + rd if m.get("kv_from") is None else 0) + H * vd, H * vd
            add("gemm_uq", 2.0 * N * H * (d + rd) * qr, 2.0 * (H * (d + rd) * qr + N * qr) + 4.0 * N * H * (d + rd))
            add("absorb_uk", 2.0 * N * H * d * kr, 2.0 * (H * d * kr + N * H * (d + kr)))
            add("absorb_uv", 2.0 * N * H * vd * kr, 2.0 * (H * vd * kr + N * H * kr) + 4.0 * N * H * vd)
            add("attention", 2.0 * pairs * H * (2 * kr + rd), 2.0 * (sum(ctx_lens) * (kr + rd) + N * H * (2 * kr + rd)))
        add("gemm_in", 2.0 * N * n_in * W, 2.0 * n_in * W + 2.0 * N * W + 4.0 * N * n_in)
        add("gemm_o", 2.0 * N * n_o * W, 2.0 * n_o * W + 2.0 * N * n_o + 4.0 * N * W)
        if f["kind"] == "dense":
            add("gemm_up", 2.0 * N * f["ff"] * W, 2.0 * (f["ff"] * W + N * (f["ff"] + W)))
            add("gemm_down", 2.0 * N * f["ff"] * W, 2.0 * (f["ff"] * W + N * f["ff"]) + 4.0 * N * W)
        else:
            E, I, top, ef = f["router"]["experts"], f["router"]["identity"], f["router"]["top"], f["expert"]["ff"]
            real = N * top * E / (E + I)                                           # pairs that reach a real expert (uniform routing)
            touched = min(E, N * top)
            add("moe_gate_up", 4.0 * real * ef * W, 2.0 * (2 * touched * ef * W + real * (2 * ef + W)))
            add("moe_down", 2.0 * real * ef * W, 2.0 * (touched * ef * W + real * ef) + 4.0 * real * W)
    out = {}
    for name, (fl, by) in work.items():
        if name in prof and fl > 0:
            if name == "delta_scan":
                tmin = max(fl / (pk.get("fp32", 70.0) * 1e12), by / (pk["hbm"] * 1e9)) * 1e6
                out[name] = {"us": round(prof[name], 2), "fp32_tflops": round(fl / prof[name] / 1e6, 2), "gbs": round(by / prof[name] / 1e3, 1),
                             "roofline_frac": round(tmin / prof[name], 3)}
            else:
                out[name] = _roof(fl, by, prof[name], pk)
    for name in ("norm", "latent_norm_store", "q_split_rot", "head_gate", "delta_prep", "moe_route", "moe_sort", "moe_gather", "moe_glu", "moe_combine",
                 "embed", "final_norm", "lm_head"):
        if name in prof:
            out[name] = {"us": round(prof[name], 2)}
    return out


# ---- Batatar at the same sizes: four layers - chunked capped attention beside a selective state space layer (twice the width inside,
# heads of 64 numbers over states of 128), lightning attention (heads of 128 x 128), lightning attention, the parallel mixer again - with
# sigmoid-routed experts of ff / 2 hidden units, top 2 of 16 (the gated feed-forward's active parameter count), behind every mixer; layers
# 1 and 2 form a looped block of ONE pass, so that the product that opens a pass is part of the step.
B_CHUNK = 256


def batatar_config(sz: dict) -> dict:
    H, W = sz["heads"], sz["width"]
    par = {"left": {"heads": H, "kv_heads": 8, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "softcap": 30.0, "mask": {"size": B_CHUNK}},
           "right": {"heads": 2 * W // 64, "vdim": 64, "state": 128, "groups": 2, "conv": 4, "norm_groups": 2}}
    lin = {"heads": H, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** (-3 - 6 * i / max(1, H - 1)) for i in range(H)]}
    mlp = {"kind": "moe", "router": {"experts": 16, "top": 2}, "expert": {"ff": sz["ff"] // 2}}
    kinds = ["parallel", "lightning", "lightning", "parallel"]
    layers = [{"type": kinds[i % 4], "mixer": dict(par if kinds[i % 4] == "parallel" else lin), "mlp": dict(mlp)} for i in range(sz["layers"])]
    return {"architecture": "Batatar", "vocab": sz["vocab"], "width": W, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
            "loop": {"start": 1, "stop": min(3, sz["layers"]), "times": 1}, "layers": layers}


def batatar_weights(cfg: dict, seed: int = 0):
    """(name, bf16 CPU tensor) pairs, generated one at a time."""
    import torch
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(o, i):
        return (torch.randn(o, i, generator=g) * i ** -0.5).bfloat16()

    yield "embed", (torch.randn(cfg["vocab"], W, generator=g)).bfloat16()
    yield "head", mat(cfg["vocab"], W)
    yield "final.norm", torch.ones(W).bfloat16()
    if cfg.get("loop"):
        yield "loop.in", mat(W, 2 * W)
        yield "loop.step", torch.zeros(cfg["loop"]["times"], W).bfloat16()
    for i, ly in enumerate(cfg["layers"]):
        m, p = ly["mixer"], f"l{i}."
        yield p + "norm1", torch.ones(W).bfloat16()
        yield p + "norm2", torch.ones(W).bfloat16()
        if ly["type"] == "parallel":
            a, b = m["left"], m["right"]
            H, G, d, vd = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * vd)):
                yield p + "mix.left." + n, mat(rows, W)
                yield p + "mix.left." + n + ".b", torch.zeros(rows).bfloat16()
            yield p + "mix.left.g", mat(H, W)
            yield p + "mix.left.o", mat(W, H * vd)
            yield p + "mix.left.out", torch.ones(W).bfloat16()
            Hs, vs, N, Gs, taps = b["heads"], b["vdim"], b["state"], b["groups"], b["conv"]
            inner, C = Hs * vs, Hs * vs + 2 * Gs * N
            yield p + "mix.right.in", mat(2 * inner + 2 * Gs * N + Hs, W)
            yield p + "mix.right.conv", (torch.randn(C, taps, generator=g) * 0.5).bfloat16()
            yield p + "mix.right.conv.b", torch.zeros(C).bfloat16()
            yield p + "mix.right.dt_bias", torch.zeros(Hs).bfloat16()
            yield p + "mix.right.A_log", torch.zeros(Hs).bfloat16()
            yield p + "mix.right.D", torch.ones(Hs).bfloat16()
            yield p + "mix.right.norm", torch.ones(inner).bfloat16()
            yield p + "mix.right.o", mat(W, inner)
            yield p + "mix.right.out", torch.ones(W).bfloat16()
        else:
            H, d, vd = m["heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * d), ("k", H * d), ("v", H * vd), ("g", H * vd)):
                yield p + "mix." + n, mat(rows, W)
            yield p + "mix.norm", torch.ones(H * vd).bfloat16()
            yield p + "mix.o", mat(W, H * vd)
        f = ly["mlp"]
        E, ef = f["router"]["experts"], f["expert"]["ff"]
        yield p + "mlp.router", mat(E, W)
        for e in range(E):
            yield p + f"mlp.e{e}.gate", mat(ef, W)
            yield p + f"mlp.e{e}.up", mat(ef, W)
            yield p + f"mlp.e{e}.down", mat(W, ef)


def batatar_rooflines(cfg, prof: Dict[str, float], N: int, B: int, ctx_lens: List[int], q_lens: List[int], pk) -> dict:
    """Per-op roofline of one profiled step: the times are sums over the layer runs, the work is summed the same way.  Both recurrences
    run on the fp32 FMA pipe (their state is fp32): their fractions are against that pipe's peak (pk["fp32"]); 4 N H d vd flops is the
    token-by-token form's count (state update and read-out), as for the retention scan of the Ranilix family."""
    W = cfg["width"]
    names = ("gemm_in", "gemm_o", "gemm_loop", "attention", "ssd_scan", "lightning_scan", "moe_gate_up", "moe_down")
    work = {k: [0.0, 0.0] for k in names}

    def add(name, flops, nbytes):
        work[name][0] += flops
        work[name][1] += nbytes

    for ly in cfg["layers"]:
        m, f = ly["mixer"], ly["mlp"]
        if ly["type"] == "parallel":
            a, b = m["left"], m["right"]
            H, G, d, vd, size = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["mask"]["size"]
            Hs, vs, Ns, Gs = b["heads"], b["vdim"], b["state"], b["groups"]
            inner = Hs * vs
            n_in = H * d + G * (d + vd) + H + 2 * inner + 2 * Gs * Ns + Hs
            n_o = H * vd + inner
            pairs, keys = 0, 0
            for q, c in zip(q_lens, ctx_lens):
                for t in range(c - q, c):
                    pairs += t % size + 1
                keys += min(c, q + (c - q) % size)
            add("attention", 2.0 * pairs * H * (d + vd), 2.0 * (keys * G * (d + vd) + N * H * (d + vd)))
            add("ssd_scan", 4.0 * N * Hs * Ns * vs, 4.0 * (N * (2 * Gs * Ns + 3 * inner) + 2 * B * Hs * Ns * vs))
        else:
            H, d, vd = m["heads"], m["dim"], m["vdim"]
            n_in, n_o = 2 * H * d + 2 * H * vd, H * vd
            add("lightning_scan", 4.0 * N * H * d * vd, 4.0 * (N * H * (2 * d + 2 * vd) + 2 * B * H * d * vd))
        add("gemm_in", 2.0 * N * n_in * W, 2.0 * n_in * W + 2.0 * N * W + 4.0 * N * n_in)
        add("gemm_o", 2.0 * N * n_o * W, 2.0 * n_o * W + 2.0 * N * n_o + 4.0 * N * W * (2 if ly["type"] == "parallel" else 1))
        E, top, ef = f["router"]["experts"], f["router"]["top"], f["expert"]["ff"]
        touched = min(E, N * top)
        add("moe_gate_up", 4.0 * N * top * ef * W, 2.0 * (2 * touched * ef * W + N * top * (2 * ef + W)))
        add("moe_down", 2.0 * N * top * ef * W, 2.0 * (touched * ef * W + N * top * ef) + 4.0 * N * top * W)
    if cfg.get("loop"):
        t = cfg["loop"]["times"]
        add("gemm_loop", t * 4.0 * N * W * W, t * (4.0 * W * W + 4.0 * N * W + 4.0 * N * W))
    out = {}
    for name, (fl, by) in work.items():
        if name in prof and fl > 0:
            if name in ("ssd_scan", "lightning_scan"):
                tmin = max(fl / (pk.get("fp32", 70.0) * 1e12), by / (pk["hbm"] * 1e9)) * 1e6
                out[name] = {"us": round(prof[name], 2), "fp32_tflops": round(fl / prof[name] / 1e6, 2), "gbs": round(by / prof[name] / 1e3, 1),
                             "roofline_frac": round(tmin / prof[name], 3)}
            else:
                out[name] = _roof(fl, by, prof[name], pk)
    for name in ("norm", "loop_concat", "qkv_prep", "ssd_prep", "ssd_gate_norm", "lightning_prep", "lightning_norm_gate", "moe_route", "moe_sort",
                 "moe_scatter", "moe_glu", "moe_combine", "embed", "final_norm", "lm_head"):
        if name in prof:
            out[name] = {"us": round(prof[name], 2)}
    return out


def _prompts(n, length, vocab, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, length).tolist() for _ in range(n)]


def _run_engine(eng, runner, vocab, eos, batch_p, batch_d, plen, K, W):
    """(prefill tok/s, decode tok/s, ms per decode step, kernels per decode step) through LLMEngine."""
    nblocks = runner.num_kvcache_blocks
    T = runner.max_num_batched_tokens
    engine = eng.LLMEngine(eng.Scheduler(eng.SchedulerConfig(max(batch_p, batch_d), T, eos, nblocks, BLOCK)), runner, greedy=True)
    best = None
    for rep in range(4):                       # first repetition is the warm-up
        for p in _prompts(batch_p, plen, vocab, 10 + rep):
            engine.add_request(p, eng.SamplingParams(1.0, 1, True))
        t0 = time.perf_counter()
        s = engine.step()                      # synchronous: returns after the tokens are on the host
        dt = time.perf_counter() - t0
        assert s.is_prefill and engine.is_finished()
        if rep > 0:
            best = dt if best is None else min(best, dt)
    for p in _prompts(batch_d, plen, vocab, 3):
        engine.add_request(p, eng.SamplingParams(1.0, W + K + 8, True))
    while engine.num_waiting():
        engine.step()
    for _ in range(max(W, 3)):
        engine.step()
    ms_step, launches = runner.time_decode(K)
    return engine, batch_p * plen / best, batch_d / (ms_step * 1e-3), ms_step, launches


def _roof(flops, nbytes, us, pk):
    tmin = max(flops / (pk["bf16"] * 1e12), nbytes / (pk["hbm"] * 1e9)) * 1e6
    return {"us": round(us, 2), "tflops": round(flops / us / 1e6, 1), "gbs": round(nbytes / us / 1e3, 1), "roofline_frac": round(tmin / us, 3)}


def karuzen_rooflines(cfg, prof: Dict[str, float], N: int, B: int, ctx_lens: List[int], q_lens: List[int], pk) -> dict:
    """Per-op roofline of one profiled step (times summed over the layers; work summed the same way)."""
    L = len(cfg["layers"])
    m, f, W = cfg["layers"][0]["mixer"], cfg["layers"][0]["mlp"], cfg["width"]
    H, d, vd, kr, qr = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]
    out = {}

    def gemm(name, o, i, rows=N, copies=1):
        if name in prof:
            out[name] = _roof(L * 2.0 * rows * o * i * copies, L * 2.0 * (o * i * copies + rows * (o + i) * copies), prof[name], pk)

    gemm("gemm_down_latents", qr + kr, W)
    gemm("gemm_uq", H * d, qr)
    gemm("absorb_uk", kr, d, copies=H)
    gemm("absorb_uv", vd, kr, copies=H)
    gemm("gemm_o", W, H * vd)
    if "latent_attn" in prof:
        pairs = sum(q * c - q * (q - 1) // 2 for q, c in zip(q_lens, ctx_lens))       # visible (query, key) pairs
        out["latent_attn"] = _roof(L * 4.0 * H * kr * pairs, L * 2.0 * (sum(ctx_lens) * kr + 2 * N * H * kr), prof["latent_attn"], pk)
    if f["kind"] == "dense":
        gemm("gemm_gate_up", 2 * f["ff"], W)
        gemm("gemm_ff_down", W, f["ff"])
    else:
        E, top, ef, sf = f["router"]["experts"], f["router"]["top"], f["expert"]["ff"], f["shared"]["ff"]
        touched = min(E, N * top)
        for name in ("moe_up", "moe_down"):
            if name in prof:
                out[name] = _roof(L * 2.0 * N * top * ef * W, L * 2.0 * (touched * ef * W + N * top * (ef + W)), prof[name], pk)
        if "shared_expert" in prof:
            out["shared_expert"] = _roof(L * 4.0 * N * sf * W, L * 2.0 * (2 * sf * W + N * (2 * sf + 2 * W)), prof["shared_expert"], pk)
    for name in ("dyt_norm", "latent_norm_store", "gelu_mul", "moe_route", "moe_sort", "moe_gather", "moe_combine", "embed", "final_norm", "lm_head"):
        if name in prof:
            out[name] = {"us": round(prof[name], 2)}
    return out


def compare(ctx_ours, sizes=None, batch_p=16, batch_d=64, plen=512, K=32, W=4, peaks=None, family="karuzen") -> dict:
    import importlib
    import torch
    eng = importlib.import_module("nano-vllm-candle_b200.engine")
    synth = importlib.import_module("nano-vllm-candle_b200.synth")
    pk = peaks or {"bf16": 1590.0, "hbm": 6650.0, "source": "fallback"}
    make_config, make_weights, rooflines = {"karuzen": (karuzen_config, karuzen_weights, karuzen_rooflines),
                                            "ranilix": (ranilix_config, ranilix_weights, ranilix_rooflines),
                                            "fefozen": (fefozen_config, fefozen_weights, fefozen_rooflines),
                                            "batatar": (batatar_config, batatar_weights, batatar_rooflines)}[family]
    T = batch_p * plen
    nblocks = max(batch_p, batch_d) * (-(-(plen + W + K + 24) // BLOCK)) + 8
    results = []
    for sz in sizes or SIZES:
        rec = {"size": sz["name"]}
        if family == "ranilix" and "moe" in sz:
            continue                                               # the design has no mixture of experts
        if family == "batatar" and "moe" in sz:
            continue                                               # every size of this family already has experts
        # ---- the registry family
        cfg = make_config(sz)
        t0 = time.perf_counter()
        kr = eng.ModelRunner.from_config(ctx_ours, cfg, make_weights(cfg), num_kvcache_blocks=nblocks, kvcache_block_size=BLOCK,
                                         max_num_seqs=max(batch_p, batch_d), max_num_batched_tokens=T,
                                         max_model_len=(-(-(plen + W + K + 24) // BLOCK)) * BLOCK)
        load_s = time.perf_counter() - t0
        engine, p_tps, d_tps, ms_step, launches = _run_engine(eng, kr, sz["vocab"], -1, batch_p, batch_d, plen, K, W)
        kr.arm_profile()
        engine.step()                                              # one more decode step, un-captured, with events
        prof_d = kr.profile()
        ctx_d = plen + max(W, 3) + 2
        roof_d = rooflines(cfg, prof_d, batch_d, batch_d, [ctx_d] * batch_d, [1] * batch_d, pk)
        engine.close()
        e2 = eng.LLMEngine(eng.Scheduler(eng.SchedulerConfig(batch_p, T, -1, nblocks, BLOCK)), kr, greedy=True)
        for p in _prompts(batch_p, plen, sz["vocab"], 77):
            e2.add_request(p, eng.SamplingParams(1.0, 1, True))
        kr.arm_profile()
        e2.step()
        prof_p = kr.profile()
        roof_p = rooflines(cfg, prof_p, T, batch_p, [plen] * batch_p, [plen] * batch_p, pk)
        e2.close()
        rec[family] = {"prefill_tok_s": round(p_tps), "decode_tok_s": round(d_tps), "decode_ms_per_step": round(ms_step, 4),
                          "kernels_per_decode_step": launches, "weights_load_s": round(load_s, 1),
                          "weight_bytes": kr.weight_bytes(), "cache_bytes_per_token": kr.kv_bytes_per_token(),
                          "prefill_ops": roof_p, "decode_ops": roof_d}
        kr.close()
        torch.cuda.empty_cache()
        # ---- Qwen3 at the same width / heads / ff / layers / vocab (8 kv heads of 128)
        qc = eng.Qwen3Config(vocab_size=sz["vocab"], hidden_size=sz["width"], head_dim=128, num_hidden_layers=sz["layers"],
                             num_attention_heads=sz["heads"], num_key_value_heads=8, intermediate_size=sz["ff"],
                             max_position_embeddings=4096, bos_token_id=1, eos_token_id=2)
        qr_ = eng.Qwen3ModelRunner.from_weights(ctx_ours, qc, synth.iter_weights_device(qc, 0, device="cuda:0"), num_kvcache_blocks=nblocks,
                                                kvcache_block_size=BLOCK, max_num_seqs=max(batch_p, batch_d), max_num_batched_tokens=T,
                                                max_model_len=(-(-(plen + W + K + 24) // BLOCK)) * BLOCK)
        engine, p_tps, d_tps, ms_step, launches = _run_engine(eng, qr_, sz["vocab"], 2, batch_p, batch_d, plen, K, W)
        ops = {op: qr_.time_op(op, 5)[0] * 1e3 for op in ("paged_decode", "gemm_qkv", "gemm_o", "gemm_gate_up", "gemm_down", "rmsnorm",
                                                           "qk_norm_rope")}
        Hh, I, nh = sz["width"], sz["ff"], sz["heads"]
        ctx_d = plen + max(W, 3) + 1 + K
        qroof = {
            "paged_decode": _roof(4.0 * nh * 128 * ctx_d * batch_d, 2.0 * (batch_d * ctx_d * 2 * 8 * 128 + 2 * batch_d * nh * 128), ops["paged_decode"], pk),
            "gemm_qkv": _roof(2.0 * batch_d * Hh * (nh + 16) * 128, 2.0 * Hh * (nh + 16) * 128, ops["gemm_qkv"], pk),
            "gemm_o": _roof(2.0 * batch_d * Hh * nh * 128, 2.0 * Hh * nh * 128, ops["gemm_o"], pk),
            "gemm_gate_up": _roof(4.0 * batch_d * Hh * I, 4.0 * Hh * I, ops["gemm_gate_up"], pk),
            "gemm_down": _roof(2.0 * batch_d * Hh * I, 2.0 * Hh * I, ops["gemm_down"], pk),
            "rmsnorm": {"us": round(ops["rmsnorm"], 2)}, "qk_norm_rope": {"us": round(ops["qk_norm_rope"], 2)},
        }
        rec["qwen3"] = {"prefill_tok_s": round(p_tps), "decode_tok_s": round(d_tps), "decode_ms_per_step": round(ms_step, 4),
                        "kernels_per_decode_step": launches, "weight_bytes": qr_.weight_bytes(),
                        "cache_bytes_per_token": qr_.kv_bytes_per_token(), "decode_ops_per_layer_call": qroof}
        engine.close()
        qr_.close()
        torch.cuda.empty_cache()
        results.append(rec)
    return {"metric": family + "_vs_qwen3_equal_layer_sizes", "unit": "tok/s", "dtype": "bf16", "data": "synthetic",
            "workload": {"prefill": f"{batch_p} x {plen} tokens in one step", "decode": f"batch {batch_d} at context ~{plen + W + K}",
                         "timing": "prefill: host wall clock around the synchronous engine step, best of 3 after a warm-up; decode: CUDA events "
                                   "around K replays of the captured step; per-op: CUDA events inside one un-captured step"},
            "peaks": pk, "results": results}
