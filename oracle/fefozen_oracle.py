"""Plain fp32 restatement of the Fefozen design, one function per mechanism, slow on purpose.

Notation: W (width), V (vocab), T (new tokens of one sequence), P (tokens before them).  Linear weights are
[out, in] and act as y = W x.  A layer is sequential with a norm in front of and behind each sublayer:

    x <- x + n1b(mixer(n1(x)));   x <- x + n2b(ff(n2(x)))          n(y) = y / sqrt(mean(y^2) + eps) * (1 + w)

Mixers:

  latent_attention     queries and keys / values through RMS-normed low-rank latents.  A token leaves one row
  latent_attention_2   [c | r] behind: c = the normed key / value latent, r = a rotated key part that all heads
                       share.  Head h scores (q_h^nope . U_k,h c_j + q_h^rot . r_j) * scale against every earlier
                       token j, and reads U_v,h c_j.  The first kind turns interleaved pairs (2i, 2i + 1) and has a
                       sink (one more term exp(sink_h) in the softmax denominator, no value); the second turns
                       pairs (i, i + dims / 2), has a plain softmax and may read ANOTHER layer's rows (`kv_from`)
                       with its own U_k, U_v.  Both gate the heads' outputs with sigmoid(W_g h).
  delta                gated delta rule: q, k, v through a short causal convolution per channel and silu, q and k
                       made unit vectors per head, a per-head state S [dim, vdim]:
                           S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
                       with g = exp(-exp(A_log) softplus(W_a h + dt_bias)), beta = sigmoid(W_b h); every head's o
                       is divided by its root mean square, weighted and gated with silu(W_g h).

Feed-forward: dense (down gelu_tanh(up h)) or a mixture of experts (softmax router over real and identity
experts, a correction that biases the choice but not the weights, clamped gated experts).

The caches are explicit: every function takes what earlier tokens left and returns what it leaves, so that the
same code serves whole prompts, portions and token-by-token decoding.  Everything here is float32 torch on the
CPU; nothing is shared with the CUDA path.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def zero_centred_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layer norms store their weight around zero."""
    return rms_norm(x, None, eps) * (1.0 + w)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_angles(pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.tensor(float(base), dtype=torch.float64) ** (-2.0 * i / dims)
    return pos.double().view(-1, 1) * f.view(1, -1)


def rotary(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float, half: bool) -> torch.Tensor:
    """x: [T, ..., d]; the first `dims` numbers of the last axis are turned.  half: number i pairs with i + dims / 2,
    else 2i with 2i + 1."""
    if dims == 0:
        return x
    a = rotary_angles(pos, dims, base)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = a.cos().float().view(shape), a.sin().float().view(shape)
    out = x.clone()
    if half:
        u, v = x[..., : dims // 2], x[..., dims // 2: dims]
        out[..., : dims // 2] = u * c - v * s
        out[..., dims // 2: dims] = v * c + u * s
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    return out


def latent_rows(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float, pos0: int, half: bool) -> torch.Tensor:
    """What T new tokens leave in a latent layer's cache: [T, kv_rank + rot_dim] = [normed latent | rotated shared key part]."""
    T, R, rd = h.shape[0], m["kv_rank"], m["rot_dim"]
    d = h @ p["dkv"].T
    c = rms_norm(d[:, :R], p["dkv.norm"], eps)
    r = rotary(d[:, R:R + rd], torch.arange(pos0, pos0 + T), m["rot"]["dims"], m["rot"]["base"], half)
    return torch.cat([c, r], -1)


def latent_attention(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float, pos0: int, rows: torch.Tensor,
                     half: bool) -> torch.Tensor:
    """The latent-attention mixer over T new tokens at positions pos0 ...; rows = cache rows [pos0 + T, kv_rank + rot_dim] of
    ALL tokens so far (this layer's own or, with kv_from, another layer's).  Keys and values are rebuilt per head, not absorbed."""
    T, H, d, rd, vd, R = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(pos0, pos0 + T)
    cq = rms_norm(h @ p["dq"].T, p["dq.norm"], eps)
    q = (cq @ p["uq"].T).view(T, H, d + rd)
    q_nope = q[..., :d]
    q_rot = rotary(q[..., d:], pos, m["rot"]["dims"], m["rot"]["base"], half)
    c, r = rows[:, :R], rows[:, R:]
    k_nope = (c @ p["uk"].T).view(-1, H, d)
    v = (c @ p["uv"].T).view(-1, H, vd)
    Tk = rows.shape[0]
    vis = torch.arange(Tk).view(1, -1) <= pos.view(-1, 1)
    out = torch.zeros(T, H, vd)
    for hh in range(H):
        s = (q_nope[:, hh] @ k_nope[:, hh].T + q_rot[:, hh] @ r.T) * m["scale"]
        s = s.masked_fill(~vis, float("-inf"))
        mx = s.max(-1, keepdim=True).values
        sink = p.get("sink")
        if sink is not None:
            mx = torch.maximum(mx, sink[hh].view(1, 1))
        e = torch.exp(s - mx)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[hh] - mx)
        out[:, hh] = (e / den) @ v[:, hh]
    o = out.reshape(T, H * vd) * torch.sigmoid(h @ p["g"].T)
    return o @ p["o"].T


def short_conv(x: torch.Tensor, w: torch.Tensor, before: torch.Tensor):
    """Causal convolution over time per channel: x [T, C], w [C, taps] (last column = the current token), before
    [taps - 1, C] = the inputs in front of x (zeros at the start).  Returns (y [T, C], the last taps - 1 inputs)."""
    taps = w.shape[1]
    full = torch.cat([before, x], 0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + full[j: j + x.shape[0]] * w[:, j].view(1, -1)
    return y, full[full.shape[0] - (taps - 1):]


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, g, beta, S):
    """q, k: [T, H, d]; v: [T, H, vd]; g, beta: [T, H]; S: [H, d, vd].  Returns (o [T, H, vd], S)."""
    T, H, _ = q.shape
    o = torch.zeros(T, H, v.shape[-1])
    S = S.clone()
    for t in range(T):
        for hh in range(H):
            Sh = S[hh] * g[t, hh]
            u = beta[t, hh] * (v[t, hh] - Sh.T @ k[t, hh])
            Sh = Sh + torch.outer(k[t, hh], u)
            o[t, hh] = Sh.T @ q[t, hh]
            S[hh] = Sh
    return o, S


def delta_mixer(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float, state: Optional[dict]):
    """The gated-delta-rule mixer over T new tokens.  state = {"S": [H, d, vd], "q" / "k" / "v": [taps - 1, channels]} of the
    tokens before them (None at the start).  Returns (output [T, W], state)."""
    T, H, G, d, vd, taps = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    if state is None:
        state = {"S": torch.zeros(H, d, vd), "q": torch.zeros(taps - 1, G * d), "k": torch.zeros(taps - 1, G * d),
                 "v": torch.zeros(taps - 1, H * vd)}
    new = {}
    qkv = {}
    for n in ("q", "k", "v"):
        y, new[n] = short_conv(h @ p[n].T, p[n + ".conv"], state[n])
        qkv[n] = torch.nn.functional.silu(y)
    rep = H // G
    q = unit(qkv["q"].view(T, G, d)).repeat_interleave(rep, 1) * d ** -0.5
    k = unit(qkv["k"].view(T, G, d)).repeat_interleave(rep, 1)
    v = qkv["v"].view(T, H, vd)
    beta = torch.sigmoid(h @ p["b"].T)
    g = torch.exp(-torch.exp(p["A_log"]) * torch.nn.functional.softplus(h @ p["a"].T + p["dt_bias"]))
    o, new["S"] = delta_rule(q, k, v, g, beta, state["S"])
    o = rms_norm(o, p["norm"], eps).reshape(T, H * vd) * torch.nn.functional.silu(h @ p["g"].T)
    return o @ p["o"].T, new


def dense_ff(h, p):
    return gelu_tanh(h @ p["up"].T) @ p["down"].T


def route(h, p, m):
    """Softmax over real and identity experts; the `top` largest of s + correction are chosen, the weights are s itself.
    Returns (idx [T, top], weights [T, top])."""
    s = torch.softmax(h @ p["router"].T, -1)
    idx = torch.topk(s + p["correction"], m["router"]["top"], dim=-1).indices
    return idx, torch.gather(s, 1, idx)


def expert(h, p, e: int, limit: float):
    g = torch.clamp(h @ p[f"e{e}.gate"].T, max=limit)
    u = torch.clamp(h @ p[f"e{e}.up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ p[f"e{e}.down"].T


def moe_ff(h, p, m):
    E = m["router"]["experts"]
    idx, wts = route(h, p, m)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            y = expert(h[t: t + 1], p, e, m["expert"]["limit"])[0] if e < E else h[t]     # experts behind the real ones pass their input through
            out[t] += wts[t, j] * y
    return out


def sub(params: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.float() for k, v in params.items() if k.startswith(prefix)}


class Fefozen:
    """The whole model over explicit per-request caches.  cfg: the dict of config.json; params: name -> tensor."""

    def __init__(self, cfg: dict, params: Dict[str, torch.Tensor]):
        self.cfg = cfg
        self.p = {k: v.float() for k, v in params.items()}
        self.eps = cfg["norm"]["eps"]

    def new_cache(self) -> dict:
        return {"len": 0, "rows": {}, "state": {}}

    def forward(self, tokens: List[int], cache: Optional[dict] = None, taps: Optional[list] = None) -> torch.Tensor:
        """Runs T new tokens of one request on top of `cache` (None: a whole prompt from an empty cache); returns logits [T, V]."""
        cfg, eps = self.cfg, self.eps
        if cache is None:
            cache = self.new_cache()
        pos0 = cache["len"]
        x = self.p["embed"][torch.tensor(tokens)]
        for i, ly in enumerate(cfg["layers"]):
            lp = sub(self.p, f"l{i}.")
            mp, m = sub(lp, "mix."), ly["mixer"]
            h = zero_centred_norm(x, lp["norm1"], eps)
            if ly["type"] in ("latent_attention", "latent_attention_2"):
                half = ly["type"] == "latent_attention_2"
                src = m.get("kv_from")
                if src is None:
                    new = latent_rows(h, mp, m, eps, pos0, half)
                    old = cache["rows"].get(i)
                    cache["rows"][i] = new if old is None else torch.cat([old, new], 0)
                    src = i
                y = latent_attention(h, mp, m, eps, pos0, cache["rows"][src], half)
            elif ly["type"] == "delta":
                y, cache["state"][i] = delta_mixer(h, mp, m, eps, cache["state"].get(i))
            else:
                raise ValueError(ly["type"])
            x = x + zero_centred_norm(y, lp["norm1b"], eps)
            if ly.get("mlp"):
                h = zero_centred_norm(x, lp["norm2"], eps)
                fp = sub(lp, "mlp.")
                y = dense_ff(h, fp) if ly["mlp"]["kind"] == "dense" else moe_ff(h, fp, ly["mlp"])
                x = x + zero_centred_norm(y, lp["norm2b"], eps)
            if taps is not None:
                taps.append(x.clone())
        cache["len"] = pos0 + len(tokens)
        return zero_centred_norm(x, self.p["final.norm"], eps) @ self.p["embed"].T


# ------------------------------------------------------------------------------------------ small configurations

def latent_cfg(heads=4, dim=16, rot_dim=8, vdim=24, kv_rank=40, q_rank=48, scale=0.2, rot_dims=None, rot_base=10000.0, second=False,
               kv_from=None) -> dict:
    """second: the kind with rotate-half pairs and a plain softmax (it may read another layer's rows); else interleaved pairs and a sink."""
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "rot": {"dims": rot_dim if rot_dims is None else rot_dims, "base": rot_base}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention_2" if second else "latent_attention", "mixer": m}


def delta_cfg(heads=4, kv_heads=2, dim=16, vdim=24, conv=4) -> dict:
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def with_dense(layer: dict, ff: Optional[int] = 96) -> dict:
    layer = dict(layer)
    layer["mlp"] = {"kind": "dense", "ff": ff} if ff else None
    return layer


def with_moe(layer: dict, experts=5, identity=2, top=2, ff=40, limit=1.0) -> dict:
    layer = dict(layer)
    layer["mlp"] = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top}, "expert": {"ff": ff, "limit": limit}}
    return layer


def make_config(vocab=200, width=96, layers=None, eps=1e-5) -> dict:
    return {"architecture": "Fefozen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def make_weights(cfg: dict, seed: int = 0, bf16_values: bool = True) -> Dict[str, torch.Tensor]:
    """Random weights under the checkpoint's names; values bf16-representable by default so that the bf16 and fp32 paths load
    identical numbers.  Corrections move some of the routers' choices."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def fix(t):
        return t.bfloat16().float() if bf16_values else t

    def rnd(*shape, s=1.0):
        return fix(torch.randn(*shape, generator=g) * s)

    w = {"embed": rnd(cfg["vocab"], W, s=1.0), "final.norm": rnd(W, s=0.2)}
    for i, ly in enumerate(cfg["layers"]):
        p, m = f"l{i}.", ly["mixer"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if ly.get("mlp") else ()):
            w[p + n] = rnd(W, s=0.2)
        if ly["type"].startswith("latent_attention"):
            H, d, rd, vd, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            w[p + "mix.dq"] = rnd(Q, W, s=W ** -0.5)
            w[p + "mix.dq.norm"] = fix(1.0 + rnd(Q, s=0.2))
            w[p + "mix.uq"] = rnd(H * (d + rd), Q, s=Q ** -0.5)
            if m.get("kv_from") is None:
                w[p + "mix.dkv"] = rnd(R + rd, W, s=W ** -0.5)
                w[p + "mix.dkv.norm"] = fix(1.0 + rnd(R, s=0.2))
            w[p + "mix.uk"] = rnd(H * d, R, s=R ** -0.5)
            w[p + "mix.uv"] = rnd(H * vd, R, s=R ** -0.5)
            if ly["type"] == "latent_attention":
                w[p + "mix.sink"] = rnd(H, s=1.0)
            w[p + "mix.g"] = rnd(H * vd, W, s=W ** -0.5)
            w[p + "mix.o"] = rnd(W, H * vd, s=(H * vd) ** -0.5)
        else:
            H, G, d, vd, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for n, rows in (("q", G * d), ("k", G * d), ("v", H * vd)):
                w[p + "mix." + n] = rnd(rows, W, s=W ** -0.5)
                w[p + "mix." + n + ".conv"] = rnd(rows, taps, s=taps ** -0.5)
            w[p + "mix.b"] = rnd(H, W, s=W ** -0.5)
            w[p + "mix.a"] = rnd(H, W, s=W ** -0.5)
            w[p + "mix.A_log"] = fix(torch.log(0.5 + 2.0 * torch.rand(H, generator=g)))
            w[p + "mix.dt_bias"] = rnd(H, s=0.5)
            w[p + "mix.norm"] = fix(1.0 + rnd(vd, s=0.2))
            w[p + "mix.g"] = rnd(H * vd, W, s=W ** -0.5)
            w[p + "mix.o"] = rnd(W, H * vd, s=(H * vd) ** -0.5)
        f = ly.get("mlp")
        if f and f["kind"] == "dense":
            w[p + "mlp.up"] = rnd(f["ff"], W, s=W ** -0.5)
            w[p + "mlp.down"] = rnd(W, f["ff"], s=f["ff"] ** -0.5)
        elif f:
            E, I, ff = f["router"]["experts"], f["router"].get("identity", 0), f["expert"]["ff"]
            w[p + "mlp.router"] = rnd(E + I, W, s=W ** -0.5)
            w[p + "mlp.correction"] = rnd(E + I, s=0.1)
            for e in range(E):
                w[p + f"mlp.e{e}.gate"] = rnd(ff, W, s=2.0 * W ** -0.5)
                w[p + f"mlp.e{e}.up"] = rnd(ff, W, s=2.0 * W ** -0.5)
                w[p + f"mlp.e{e}.down"] = rnd(W, ff, s=ff ** -0.5)
    return w
