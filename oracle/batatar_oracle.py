"""Plain fp32 restatement of the Batatar design, one function per mechanism, slow on purpose.

Notation: W (width), V (vocab), T (new tokens of one sequence), P (tokens before them).  Linear weights are
[out, in] and act as y = W x.  A layer is sequential and pre-normed, with one constant m on both branches:

    x <- x + m mixer(n1(x));   x <- x + m ff(n2(x))          n(y) = y / sqrt(mean(y^2) + eps) * w

A block of layers [start, stop) runs `times` passes with the same weights; every pass has its own cache and state
and opens with x <- W_in [x ; x0] + step_t (x0: the embedding rows, t: the pass).

Mixers:

  parallel     two mixers read the same input; the result is (n_l(left) + n_r(right)) / 2 with a weighted RMS norm
               over the width on each side.
               left:  grouped-query attention without positions.  Biased projections, q and k heads divided by their
                      root mean square, s = cap tanh(scale (q . k) / cap), keys of the query's own chunk only
                      (floor(i / size) = floor(j / size), j <= i), p_j = exp(s_j) / (1 + sum exp(s_j)), one sigmoid
                      gate per head, output projection.
               right: selective state space layer (Mamba-2 form).  One projection gives [z | x | B | C | dt]; x, B, C
                      pass a short causal convolution with bias and silu; dt = softplus(dt + dt_bias); per head
                          S <- exp(-exp(A_log) dt) S + dt B x^T;   y = S^T C + D x
                      then y silu(z), an RMS norm in equal groups, a weight, the output projection.
  lightning    linear attention with a constant decay per head: q, k, v = silu(W h);  S <- decay S + k v^T;  o = S^T q;
               all heads normed together, weighted, gated by sigmoid(W_g h), projected.

Feed-forward: sigmoid-routed experts; the chosen scores multiply each expert's INPUT: sum_e E_e(s_e h) with
E(u) = W_down (silu(W_gate u) * (W_up u)).

The caches are explicit: every function takes what earlier tokens left and returns what it leaves, so that the
same code serves whole prompts, portions and token-by-token decoding.  Everything here is float32 torch on the
CPU; nothing is shared with the CUDA path.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------------------------------ chunked attention

def capped_chunk_softmax(q: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, pos0: int, scale: float, cap: float, size: int,
                         sink: bool = True) -> torch.Tensor:
    """q [T, H, d] at positions pos0 ..; keys [pos0 + T, G, d], values [pos0 + T, G, vd] of every token so far.
    Returns [T, H, vd]: s = cap tanh(scale (q . k) / cap) (cap 0: not capped); keys j <= i of the query's own chunk
    (floor(i / size) = floor(j / size); size 0: all); p_j = exp(s_j) / (1 + sum exp(s_j))."""
    T, H, _ = q.shape
    G = keys.shape[1]
    out = torch.zeros(T, H, values.shape[2])
    for t in range(T):
        i = pos0 + t
        lo = (i // size) * size if size else 0
        for hh in range(H):
            g = hh // (H // G)
            s = (keys[lo: i + 1, g] @ q[t, hh]) * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            e = torch.exp(s.double())
            w = (e / ((1.0 if sink else 0.0) + e.sum())).float()     # the sink: one more term exp(0) that carries no value
            out[t, hh] = (w.view(-1, 1) * values[lo: i + 1, g]).sum(0)
    return out


def chunk_attention(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float, pos0: int, keys: torch.Tensor,
                    values: torch.Tensor, sink: bool = True):
    """h [T, W] at positions pos0 ..; keys [P, G, d] (already unit-rms) and values [P, G, vd] of the tokens before.
    Returns (out [T, W], keys [P + T, G, d], values [P + T, G, vd]).  sink = False leaves the design (tests use it to show that
    the sink matters)."""
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T + p["q.b"]).view(T, H, d)
    k = (h @ p["k"].T + p["k.b"]).view(T, G, d)
    v = (h @ p["v"].T + p["v.b"]).view(T, G, vd)
    q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    keys, values = torch.cat([keys, k], 0), torch.cat([values, v], 0)
    gate = torch.sigmoid(h @ p["g"].T)                      # [T, H]: one number per head
    size = (m.get("mask") or {}).get("size", 0)
    out = capped_chunk_softmax(q, keys, values, pos0, m["scale"], m.get("softcap", 0.0), size, sink) * gate.unsqueeze(-1)
    return out.reshape(T, H * vd) @ p["o"].T, keys, values


# ------------------------------------------------------------------------------------------ state space layer

def conv_bias_silu(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, before: torch.Tensor):
    """x [T, C]; w [C, taps] (last column = the current token); before [taps - 1, C] = the inputs in front of x.
    Returns (silu(conv + b) [T, C], the last taps - 1 inputs)."""
    taps = w.shape[1]
    full = torch.cat([before, x], 0)
    y = b.view(1, -1).expand_as(x).clone()
    for j in range(taps):
        y = y + full[j: j + x.shape[0]] * w[:, j].view(1, -1)
    return silu(y), full[full.shape[0] - (taps - 1):]


def ssd_recurrence(x, Bm, Cm, dt, A_log, D, S):
    """x [T, H, vd]; Bm, Cm [T, G, N]; dt [T, H]; S [H, N, vd].  Token by token."""
    T, H, _ = x.shape
    G = Bm.shape[1]
    y = torch.zeros_like(x)
    S = S.clone()
    for t in range(T):
        for hh in range(H):
            g = hh // (H // G)
            a = torch.exp(-torch.exp(A_log[hh]) * dt[t, hh])
            S[hh] = a * S[hh] + dt[t, hh] * torch.outer(Bm[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ Cm[t, g] + D[hh] * x[t, hh]
    return y, S


def ssd_mixer(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float, state: Optional[dict]):
    T = h.shape[0]
    H, vd, N, G, taps, ng = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"], m["norm_groups"]
    inner, C = H * vd, H * vd + 2 * G * N
    if state is None:
        state = {"S": torch.zeros(H, N, vd), "conv": torch.zeros(taps - 1, C)}
    u = h @ p["in"].T
    z, xbc, dt = u[:, :inner], u[:, inner: inner + C], u[:, inner + C:]
    xbc, conv = conv_bias_silu(xbc, p["conv"], p["conv.b"], state["conv"])
    x = xbc[:, :inner].reshape(T, H, vd)
    Bm = xbc[:, inner: inner + G * N].reshape(T, G, N)
    Cm = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = F.softplus(dt + p["dt_bias"], threshold=1e9)
    y, S = ssd_recurrence(x, Bm, Cm, dt, p["A_log"], p["D"], state["S"])
    y = y.reshape(T, inner) * silu(z)
    y = rms_norm(y.view(T, ng, inner // ng), None, eps).reshape(T, inner) * p["norm"]
    return y @ p["o"].T, {"S": S, "conv": conv}


# ------------------------------------------------------------------------------------------ lightning attention

def decay_recurrence(q, k, v, decay, S):
    """q, k [T, H, d]; v [T, H, vd]; decay [H]; S [H, d, vd]."""
    T, H, _ = q.shape
    o = torch.zeros(T, H, v.shape[-1])
    S = S.clone()
    for t in range(T):
        for hh in range(H):
            S[hh] = decay[hh] * S[hh] + torch.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ q[t, hh]
    return o, S


def lightning_mixer(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float, S: Optional[torch.Tensor]):
    T = h.shape[0]
    H, d, vd = m["heads"], m["dim"], m["vdim"]
    if S is None:
        S = torch.zeros(H, d, vd)
    q = silu(h @ p["q"].T).view(T, H, d)
    k = silu(h @ p["k"].T).view(T, H, d)
    v = silu(h @ p["v"].T).view(T, H, vd)
    o, S = decay_recurrence(q, k, v, torch.tensor(m["decay"], dtype=torch.float32), S)
    o = rms_norm(o.reshape(T, H * vd), p["norm"], eps) * torch.sigmoid(h @ p["g"].T)
    return o @ p["o"].T, S


# ------------------------------------------------------------------------------------------ experts

def route(h, p, m):
    s = torch.sigmoid(h @ p["router"].T)
    idx = torch.topk(s, m["router"]["top"], dim=-1).indices
    return idx, torch.gather(s, 1, idx)


def expert(u, p, e: int):
    return (silu(u @ p[f"e{e}.gate"].T) * (u @ p[f"e{e}.up"].T)) @ p[f"e{e}.down"].T


def moe_ff(h, p, m):
    idx, w = route(h, p, m)
    out = torch.zeros_like(h)
    for n in range(h.shape[0]):
        for t in range(idx.shape[1]):
            out[n] += expert(w[n, t] * h[n], p, int(idx[n, t]))
    return out


# ------------------------------------------------------------------------------------------ the model

def sub(params: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.float() for k, v in params.items() if k.startswith(prefix)}


def layer_runs(cfg: dict) -> List[tuple]:
    """(layer, pass, opens_pass) in the order in which the layers run."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, 0, False) for i in range(n)]
    a, b, times = lp["start"], lp["stop"], lp["times"]
    runs = [(i, 0, False) for i in range(a)]
    for t in range(times):
        runs += [(i, t, i == a) for i in range(a, b)]
    return runs + [(i, 0, False) for i in range(b, n)]


class Batatar:
    """The whole model over explicit per-request caches.  cfg: the dict of config.json; params: name -> tensor."""

    def __init__(self, cfg: dict, params: Dict[str, torch.Tensor], sink: bool = True):
        self.cfg = cfg
        self.sink = sink
        self.p = {k: v.float() for k, v in params.items()}
        self.eps = cfg["norm"]["eps"]

    def new_cache(self) -> dict:
        return {"len": 0, "kv": {}, "state": {}}

    def forward(self, tokens: List[int], cache: Optional[dict] = None, taps: Optional[list] = None) -> torch.Tensor:
        """Runs T new tokens of one request on top of `cache` (None: a whole prompt from an empty cache); returns logits [T, V]."""
        cfg, eps, mult = self.cfg, self.eps, self.cfg["residual_mult"]
        if cache is None:
            cache = self.new_cache()
        pos0 = cache["len"]
        x0 = self.p["embed"][torch.tensor(tokens)]
        x = x0
        for i, t, opens in layer_runs(cfg):
            if opens:
                x = torch.cat([x, x0], -1) @ self.p["loop.in"].T + self.p["loop.step"][t]
            ly = cfg["layers"][i]
            lp = sub(self.p, f"l{i}.")
            mp, m = sub(lp, "mix."), ly["mixer"]
            h = rms_norm(x, lp["norm1"], eps)
            key = (i, t)
            if ly["type"] == "parallel":
                ml = m["left"]
                empty = (torch.zeros(0, ml["kv_heads"], ml["dim"]), torch.zeros(0, ml["kv_heads"], ml["vdim"]))
                ks, vs = cache["kv"].get(key, empty)
                left, ks, vs = chunk_attention(h, sub(mp, "left."), ml, eps, pos0, ks, vs, self.sink)
                cache["kv"][key] = (ks, vs)
                right, cache["state"][key] = ssd_mixer(h, sub(mp, "right."), m["right"], eps, cache["state"].get(key))
                y = 0.5 * (rms_norm(left, mp["left.out"], eps) + rms_norm(right, mp["right.out"], eps))
            elif ly["type"] == "lightning":
                y, cache["state"][key] = lightning_mixer(h, mp, m, eps, cache["state"].get(key))
            else:
                raise ValueError(ly["type"])
            x = x + mult * y
            if ly.get("mlp"):
                x = x + mult * moe_ff(rms_norm(x, lp["norm2"], eps), sub(lp, "mlp."), ly["mlp"])
            if taps is not None:
                taps.append(x.clone())
        cache["len"] = pos0 + len(tokens)
        return rms_norm(x, self.p["final.norm"], eps) @ self.p["head"].T


# ------------------------------------------------------------------------------------------ small configurations

def parallel_cfg(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.25, softcap=8.0, chunk=12, s_heads=4, s_vdim=16, s_state=8, s_groups=2,
                 conv=4, norm_groups=2) -> dict:
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap,
                               "mask": {"size": chunk}},
                      "right": {"heads": s_heads, "vdim": s_vdim, "state": s_state, "groups": s_groups, "conv": conv,
                                "norm_groups": norm_groups}}}


def lightning_cfg(heads=3, dim=16, vdim=24, decay=None) -> dict:
    decay = decay if decay is not None else [0.5 + 0.499 * (h + 1) / heads for h in range(heads)]
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def with_moe(layer: dict, experts: Optional[int] = 5, top=2, ff=40) -> dict:
    layer = dict(layer)
    layer["mlp"] = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}} if experts else None
    return layer


def make_config(vocab=200, width=96, layers=None, eps=1e-5, residual_mult=0.5, loop=None) -> dict:
    cfg = {"architecture": "Batatar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": residual_mult,
           "layers": layers}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def make_weights(cfg: dict, seed: int = 0, bf16_values: bool = True) -> Dict[str, torch.Tensor]:
    """Random weights under the checkpoint's names; values bf16-representable by default so that the bf16 and fp32 paths load
    identical numbers."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def fix(t):
        return t.bfloat16().float() if bf16_values else t

    def rnd(*shape, s=1.0):
        return fix(torch.randn(*shape, generator=g) * s)

    w = {"embed": rnd(cfg["vocab"], W), "final.norm": fix(1.0 + rnd(W, s=0.2)), "head": rnd(cfg["vocab"], W, s=W ** -0.5)}
    if cfg.get("loop"):
        w["loop.in"] = fix(torch.cat([torch.eye(W), 0.3 * torch.eye(W)], 1) + torch.randn(W, 2 * W, generator=g) * 0.3 * W ** -0.5)
        w["loop.step"] = rnd(cfg["loop"]["times"], W, s=0.3)
    for i, ly in enumerate(cfg["layers"]):
        p, m = f"l{i}.", ly["mixer"]
        for n in ("norm1",) + (("norm2",) if ly.get("mlp") else ()):
            w[p + n] = fix(1.0 + rnd(W, s=0.2))
        if ly["type"] == "parallel":
            a, b = m["left"], m["right"]
            H, G, d, vd = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            q = p + "mix.left."
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * vd)):
                w[q + n] = rnd(rows, W, s=W ** -0.5)
                w[q + n + ".b"] = rnd(rows, s=0.3)
            w[q + "g"] = rnd(H, W, s=2.0 * W ** -0.5)
            w[q + "o"] = rnd(W, H * vd, s=(H * vd) ** -0.5)
            w[q + "out"] = fix(1.0 + rnd(W, s=0.2))
            Hs, vs, N, Gs, taps = b["heads"], b["vdim"], b["state"], b["groups"], b["conv"]
            inner, C = Hs * vs, Hs * vs + 2 * Gs * N
            q = p + "mix.right."
            w[q + "in"] = rnd(2 * inner + 2 * Gs * N + Hs, W, s=W ** -0.5)
            w[q + "conv"] = rnd(C, taps, s=taps ** -0.5)
            w[q + "conv.b"] = rnd(C, s=0.2)
            w[q + "dt_bias"] = rnd(Hs, s=0.5)
            w[q + "A_log"] = fix(torch.log(0.1 + 1.5 * torch.rand(Hs, generator=g)))
            w[q + "D"] = rnd(Hs, s=0.5)
            w[q + "norm"] = fix(1.0 + rnd(inner, s=0.2))
            w[q + "o"] = rnd(W, inner, s=inner ** -0.5)
            w[q + "out"] = fix(1.0 + rnd(W, s=0.2))
        else:
            H, d, vd = m["heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * d), ("k", H * d), ("v", H * vd), ("g", H * vd)):
                w[p + "mix." + n] = rnd(rows, W, s=W ** -0.5)
            w[p + "mix.norm"] = fix(1.0 + rnd(H * vd, s=0.2))
            w[p + "mix.o"] = rnd(W, H * vd, s=(H * vd) ** -0.5)
        f = ly.get("mlp")
        if f:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            w[p + "mlp.router"] = rnd(E, W, s=2.0 * W ** -0.5)
            for e in range(E):
                w[p + f"mlp.e{e}.gate"] = rnd(ff, W, s=2.0 * W ** -0.5)
                w[p + f"mlp.e{e}.up"] = rnd(ff, W, s=2.0 * W ** -0.5)
                w[p + f"mlp.e{e}.down"] = rnd(W, ff, s=ff ** -0.5)
    return w
