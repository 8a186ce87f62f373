"""Each Fefozen mechanism alone: the CUDA kernel against the plain fp32 functions of oracle/fefozen_oracle.py, in both storage
formats (bf16 serving, fp32 exact)."""
import importlib
import math

import pytest
import torch

from oracle import fefozen_oracle as F

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTS = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    return importlib.import_module("nano-vllm-candle_b200.ops")


def tol(dt):
    return dict(rtol=2e-5, atol=2e-5) if dt == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------------------------------ norms
@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("H", [24, 37, 200, 1100, 5000])
def test_norm_behind_and_in_front_of_a_sublayer(ctx, ops, dt, H):
    g = torch.Generator().manual_seed(2)
    N, eps = 7, 1e-3
    res, y = torch.randn(N, H, generator=g) * 3, torch.randn(N, H, generator=g) * 40
    wy, w = 0.2 * torch.randn(H, generator=g), 0.2 * torch.randn(H, generator=g)
    d = [t.to(DEV) for t in (res, y, wy, w)]
    s = res + F.zero_centred_norm(y, wy, eps)
    ro, o = ops.rms_norm_sandwich(ctx, d[0], d[1], d[2], d[3], eps=eps, out_dtype=dt)
    assert torch.allclose(ro.cpu(), s, rtol=1e-5, atol=1e-5)
    assert torch.allclose(o.float().cpu(), F.zero_centred_norm(s, w, eps), **tol(dt))
    # the first norm of a model: nothing to add
    ro1, o1 = ops.rms_norm_sandwich(ctx, d[0], None, None, d[3], eps=eps, out_dtype=dt)
    assert torch.equal(ro1.cpu(), res) and torch.allclose(o1.float().cpu(), F.zero_centred_norm(res, w, eps), **tol(dt))
    # gathered rows (the head): nothing is written back
    rows = i32([6, 0, 3])
    before = d[0].clone()
    ro2, o2 = ops.rms_norm_sandwich(ctx, d[0], d[1], d[2], d[3], eps=eps, out_dtype=dt, rows=rows)
    assert ro2 is None and torch.equal(before, d[0])
    assert torch.allclose(o2.float().cpu(), F.zero_centred_norm(s, w, eps)[rows.cpu().long()], **tol(dt))
    # the sum alone (a weight offset of 0 gives the plain-weight norm)
    ro3, none = ops.rms_norm_sandwich(ctx, d[0], d[1], d[2], None, eps=eps, weight_offset=0.0)
    assert none is None and torch.allclose(ro3.cpu(), res + F.rms_norm(y, wy, eps), rtol=1e-5, atol=1e-5)


def test_both_norms_keep_eps_inside_the_root(ctx, ops):
    y = torch.full((2, 48), 1e-4)
    z = torch.zeros(48)
    ro, o = ops.rms_norm_sandwich(ctx, torch.zeros(2, 48, device=DEV), y.to(DEV), z.to(DEV), z.to(DEV), eps=1e-2)
    s = y / math.sqrt(1e-8 + 1e-2)
    assert torch.allclose(ro.cpu(), s, rtol=1e-5, atol=0)
    assert torch.allclose(o.cpu(), s / torch.sqrt((s * s).mean(-1, keepdim=True) + 1e-2), rtol=1e-5, atol=0)


# ------------------------------------------------------------------------------------------ latent rows and queries
@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("half", [False, True])
@pytest.mark.parametrize("R,rd,dims", [(40, 8, 8), (17, 12, 8), (96, 32, 32), (30, 0, 0)])
def test_cache_row_is_the_normed_latent_and_the_rotated_part(ctx, ops, dt, half, R, rd, dims):
    g = torch.Generator().manual_seed(3)
    N, n0, eps, base = 9, 21, 1e-4, 300.0
    off1 = n0 + 3
    x = torch.randn(N, off1 + R + rd + 5, generator=g) * 2
    w0, w1 = 1 + 0.2 * torch.randn(n0, generator=g), 1 + 0.2 * torch.randn(R, generator=g)
    pos = torch.tensor([0, 1, 5, 63, 64, 200, 1000, 3, 2])
    slots = torch.tensor([4, 0, -1, 9, 2, 1, 7, 3, 11])
    ld = R + rd + 3
    cache = torch.full((12, ld), 7.0, dtype=dt, device=DEV)
    table = ops.rotary_table(ctx, base, dims, 1024) if dims else None
    out0 = ops.latent_norm_store_rot(ctx, x.to(DEV), n0, off1, R, w0.to(DEV), w1.to(DEV), eps, cache, i32(slots.tolist()), rd, dims, half, table,
                                     i32(pos.tolist()), dt)
    assert torch.allclose(out0.float().cpu(), F.rms_norm(x[:, :n0], w0, eps), **tol(dt))
    want = torch.cat([F.rms_norm(x[:, off1:off1 + R], w1, eps), F.rotary(x[:, off1 + R:off1 + R + rd], pos, dims, base, half)], -1)
    got = cache.float().cpu()
    for n in range(N):
        if slots[n] >= 0:
            assert torch.allclose(got[slots[n], :R + rd], want[n], **tol(dt)), n
    untouched = [s for s in range(12) if s not in slots.tolist()]
    assert (got[untouched] == 7.0).all() and (got[:, R + rd:] == 7.0).all()
    # a layer that reads another layer's rows: only the query latent
    out1 = ops.latent_norm_store_rot(ctx, x.to(DEV), n0, off1, 0, w0.to(DEV), None, eps, None, None, rd, dims, half, table, i32(pos.tolist()), dt)
    assert torch.equal(out1, out0)


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("half", [False, True])
def test_query_heads_are_split_and_their_rotated_part_turned(ctx, ops, dt, half):
    g = torch.Generator().manual_seed(4)
    N, H, d, rd, dims, R, base = 6, 3, 10, 12, 8, 20, 50.0
    x = torch.randn(N, H * (d + rd) + 4, generator=g)
    pos = torch.tensor([0, 7, 1, 300, 64, 65])
    a = torch.full((N, H * 16), 9.0, dtype=dt, device=DEV)
    b = torch.full((N, H * (R + rd) + 2), 9.0, dtype=dt, device=DEV)
    ops.head_split_rot(ctx, x.to(DEV), H, d, rd, dims, half, ops.rotary_table(ctx, base, dims, 512), i32(pos.tolist()), a, 16, b, R + rd, R)
    xs = x[:, :H * (d + rd)].view(N, H, d + rd)
    av, bv = a.float().cpu().view(N, H, 16), b.float().cpu()[:, :H * (R + rd)].view(N, H, R + rd)
    assert torch.allclose(av[..., :d], xs[..., :d], **tol(dt)) and (av[..., d:] == 9.0).all()
    assert torch.allclose(bv[..., R:], F.rotary(xs[..., d:], pos, dims, base, half), **tol(dt)) and (bv[..., :R] == 9.0).all()


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("sink", [False, True])
@pytest.mark.parametrize("R,rd,H", [(32, 16, 4), (21, 6, 3), (96, 32, 8)])
def test_absorbed_attention_over_shared_rows(ctx, ops, dt, sink, R, rd, H):
    """One cache row per token is key (all of it) AND value (its first R numbers) of every head: multi-query attention with unequal
    key and value widths over ONE pool.  Against per-head softmax with explicit keys and values; rows across page borders, a
    portion behind a cached prefix and a one-token sequence in one launch."""
    g = torch.Generator().manual_seed(5)
    bs, Dk = 16, R + rd
    ctxs, qls = [70, 33, 1], [40, 33, 1]
    ld = (Dk + 7) // 8 * 8
    pool = torch.randn(12 * bs, ld, generator=g).to(dt)
    bt = torch.tensor([[3, 0, 7, 1, 9], [2, 5, 11, 0, 0], [4, 0, 0, 0, 0]])
    N = sum(qls)
    q = (torch.randn(N, H * Dk, generator=g) * 0.5).to(dt)
    sk = torch.tensor([0.5, -1.0, 2.0, 0.0, 1.0, -2.0, 0.3, 0.7])[:H].contiguous() if sink else None
    scale = 0.3
    out = ops.attn_paged_wide(ctx, q.to(DEV), pool.to(DEV), pool.to(DEV), i32(bt.tolist()), i32(ctxs), i32([0, 40, 73, 74]), 40, bs, H, 1, Dk, R, scale,
                              sink=sk.to(DEV) if sink else None).float().cpu()
    row = 0
    for b in range(3):
        rows_b = torch.cat([pool[bt[b, j // bs] * bs + j % bs].float().view(1, -1) for j in range(ctxs[b])])[:, :Dk]
        for i in range(qls[b]):
            p = ctxs[b] - qls[b] + i
            for h in range(H):
                s = (rows_b[:p + 1] @ q[row, h * Dk:(h + 1) * Dk].float()) * scale
                m = s.max() if not sink else torch.maximum(s.max(), sk[h])
                e = torch.exp(s - m)
                den = e.sum() + (torch.exp(sk[h] - m) if sink else 0.0)
                want = (e / den) @ rows_b[:p + 1, :R]
                assert torch.allclose(out[row, h * R:(h + 1) * R], want, **tol(dt)), (b, i, h)
            row += 1


@pytest.mark.parametrize("sink", [False, True])
def test_long_portions_over_128_number_rows_on_the_tensor_memory_kernel(ctx, ops, sink):
    """The paged-prefill kernel of the dense families with key = value = the shared row and an optional sink, against the wide
    kernel (checked above against plain softmax): portions of 64 tokens and more behind cached prefixes."""
    g = torch.Generator().manual_seed(6)
    bs, H, D = 16, 5, 128
    ctxs, qls = [200, 70, 131], [129, 70, 64]
    pool = torch.randn(40 * bs, D, generator=g).bfloat16().to(DEV)
    perm = torch.randperm(40, generator=g)
    bt = torch.zeros(3, 13, dtype=torch.int32)
    at = 0
    for b, c in enumerate(ctxs):
        nb = (c + bs - 1) // bs
        bt[b, :nb] = perm[at:at + nb]
        at += nb
    N = sum(qls)
    q = (torch.randn(N, H * D, generator=g) * 0.5).bfloat16().to(DEV)
    cu = i32([0, 129, 199, 263])
    sk = torch.tensor([1.5, -1.0, 3.0, 0.0, 0.5]).to(DEV) if sink else None
    want = ops.attn_paged_wide(ctx, q, pool, pool, bt.to(DEV), i32(ctxs), cu, 129, bs, H, 1, D, D, 0.09, sink=sk).float().cpu()
    out = torch.zeros(N, H * D + 64, dtype=torch.bfloat16, device=DEV)
    ctx.prefill_attn_paged_sink(q, pool.view(40, bs, 1, D), pool.view(40, bs, 1, D), bt.to(DEV), i32(ctxs), cu, 129, H, 1, D, bs, 0.09, sk, out)
    assert torch.allclose(out[:, :H * D].float().cpu(), want, rtol=2e-2, atol=2e-2)
    if sink:      # and the sink does take its share
        plain = ops.attn_paged_wide(ctx, q, pool, pool, bt.to(DEV), i32(ctxs), cu, 129, bs, H, 1, D, D, 0.09).float().cpu()
        assert (plain - want).abs().max() > 0.05


# ------------------------------------------------------------------------------------------ output stages and activations
@pytest.mark.parametrize("dt", DTS)
def test_head_norm_with_a_shared_weight_and_a_silu_gate(ctx, ops, dt):
    g = torch.Generator().manual_seed(6)
    N, H, vd, eps = 11, 3, 40, 1e-4
    o, z, w = torch.randn(N, H * vd, generator=g) * 5, torch.randn(N, H * vd, generator=g) * 2, 1 + 0.3 * torch.randn(vd, generator=g)
    want = F.rms_norm(o.view(N, H, vd), w, eps).reshape(N, H * vd) * torch.nn.functional.silu(z)
    got = ops.head_gate_w(ctx, o.to(DEV), z.to(DEV), w.to(DEV), H, vd, True, eps, "silu", 1.0, out_dtype=dt)
    assert torch.allclose(got.float().cpu(), want, **tol(dt))


@pytest.mark.parametrize("dt", DTS)
def test_clamped_gated_unit_and_plain_gelu(ctx, ops, dt):
    g = torch.Generator().manual_seed(7)
    run_gated_units(ctx, ops, dt, g, 13, 37, 40)
    run_gated_units(ctx, ops, dt, g, 70, 96, 128)          # rows that take 16-byte accesses


def run_gated_units(ctx, ops, dt, g, N, Fn, Fp):
    x = (torch.randn(N, 2 * Fp, generator=g) * 2).to(dt)
    xf = x.float()
    for limit in (1.0, 0.25, 7.0):
        gg, u = torch.clamp(xf[:, :Fn], max=limit), torch.clamp(xf[:, Fp:Fp + Fn], -limit, limit)
        want = gg * torch.sigmoid(1.702 * gg) * (u + 1.0)
        got = ops.act_mul_p(ctx, x.to(DEV), Fn, Fp, ops.ACT_GLU_CLAMP, limit, 1.702)
        assert torch.allclose(got.float().cpu(), want, **tol(dt))
    got = ops.act_mul_p(ctx, x.to(DEV), Fn, Fp, ops.ACT_GELU_TANH)
    assert torch.allclose(got.float().cpu(), F.gelu_tanh(xf[:, :Fn]), **tol(dt))


@pytest.mark.parametrize("M", [5, 300])
def test_gelu_in_the_epilogue_of_a_product(ctx, ops, M):
    g = torch.Generator().manual_seed(8)
    K, Nn = 128, 192
    A, W = torch.randn(M, K, generator=g).bfloat16(), (torch.randn(Nn, K, generator=g) * K ** -0.5 * 2).bfloat16()
    want = F.gelu_tanh(A.float() @ W.float().T)
    got = ops.gemm_act(ctx, A.to(DEV), W.to(DEV), ops.ACT_GELU_TANH).float().cpu()
    assert torch.allclose(got, want, rtol=2e-2, atol=2e-2)
    for dt in DTS:
        got = ops.linear(ctx, A.to(dt).to(DEV), W.to(dt).to(DEV), act=ops.ACT_GELU_TANH).float().cpu()
        assert torch.allclose(got, want, **tol(dt))


# ------------------------------------------------------------------------------------------ routing
@pytest.mark.parametrize("E,I,top", [(5, 2, 2), (1, 3, 1), (0, 4, 2), (60, 4, 8), (200, 56, 3), (6, 0, 6)])
def test_softmax_router_with_a_correction_on_the_choice_only(ctx, ops, E, I, top):
    g = torch.Generator().manual_seed(9)
    N, Et = 50, E + I
    z = torch.randn(N, Et + 3, generator=g) * 2
    corr = torch.randn(Et, generator=g) * 0.2
    idx, w = ops.moe_route_logits_ex(ctx, z.to(DEV), corr.to(DEV), Et, top, 1.0, ops.ROUTE_SOFTMAX, False)
    s = torch.softmax(z[:, :Et], -1)
    want_idx = torch.topk(s + corr, top, dim=-1).indices
    assert torch.equal(idx.cpu().long().sort(-1).values, want_idx.sort(-1).values)
    assert torch.allclose(w.cpu(), torch.gather(s, 1, idx.cpu().long()), rtol=1e-5, atol=1e-7)       # the scores themselves: not renormalised
    # a correction can move a choice without touching the weight it gets
    big = corr.clone()
    big[Et - 1] = 10.0
    idx2, w2 = ops.moe_route_logits_ex(ctx, z.to(DEV), big.to(DEV), Et, top, 1.0, ops.ROUTE_SOFTMAX, False)
    assert (idx2[:, 0] == Et - 1).all() and torch.allclose(w2[:, 0].cpu(), s[:, Et - 1], rtol=1e-5, atol=1e-7)
    # the older behaviour is still there: sigmoid scores, normalised weights
    idx3, w3, _ = ops.moe_route_logits(ctx, z.to(DEV), corr.to(DEV), Et, top, 2.0)
    idx4, w4 = ops.moe_route_logits_ex(ctx, z.to(DEV), corr.to(DEV), Et, top, 2.0, ops.ROUTE_SIGMOID, True)
    assert torch.equal(idx3, idx4) and torch.equal(w3, w4) and torch.allclose(w3.sum(-1).cpu(), torch.full((N,), 2.0), rtol=1e-5, atol=0)


@pytest.mark.parametrize("dt", DTS)
def test_identity_experts_in_sort_and_combine(ctx, ops, dt):
    g = torch.Generator().manual_seed(10)
    N, top, E, I, H = 40, 3, 4, 3, 24
    idx = torch.stack([torch.randperm(E + I, generator=g)[:top] for _ in range(N)]).int()
    w = torch.rand(N, top, generator=g)
    x = torch.randn(N, H, generator=g).to(dt)
    offsets, src, pos = ops.moe_sort(ctx, idx.to(DEV), E + I)
    y = torch.randn(N * top, H, generator=g)
    y[offsets[E].item():] = float("nan")            # rows of identity experts are never computed: whatever lies there must not be read
    got = ops.moe_combine_identity(ctx, y.to(DEV), pos, w.to(DEV), idx.to(DEV), E, x.to(DEV)).cpu()
    want = torch.zeros(N, H)
    for n in range(N):
        for t in range(top):
            e = int(idx[n, t])
            want[n] += w[n, t] * (y[pos.cpu()[n * top + t]] if e < E else x[n].float())
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-5)
    # the padded layout of the grouped tensor-core product: tiles of identity experts are marked absent
    offs, src_p, pos_p, tg = ops.moe_sort_padded_ex(ctx, idx.to(DEV), E + I, E, 128)
    offs = offs.cpu().tolist()
    for t, gname in enumerate(tg.cpu().tolist()):
        if t * 128 < offs[E]:
            assert gname == max(e for e in range(E) if offs[e] <= t * 128)
        else:
            assert gname == -1


# ------------------------------------------------------------------------------------------ the gated delta rule
def plain_delta(x, offs, H, G, d, vd, conv_w, A_log, dt_bias, state):
    """The oracle's functions over one sequence's projection rows x [T, ...]; state = (S, inputs in front) or None."""
    T = x.shape[0]
    qk = G * d
    cols = {"q": (offs[0], qk), "k": (offs[1], qk), "v": (offs[2], H * vd)}
    ch0 = {"q": 0, "k": qk, "v": 2 * qk}
    taps = conv_w.shape[1]
    if state is None:
        state = (torch.zeros(H, d, vd), torch.zeros(taps - 1, 2 * qk + H * vd))
    outs, keep = {}, []
    for n in ("q", "k", "v"):
        c0, cn = cols[n]
        yv, last = F.short_conv(x[:, c0:c0 + cn], conv_w[ch0[n]:ch0[n] + cn], state[1][:, ch0[n]:ch0[n] + cn])
        outs[n] = torch.nn.functional.silu(yv)
        keep.append(last)
    q = F.unit(outs["q"].view(T, G, d)).repeat_interleave(H // G, 1) * d ** -0.5
    k = F.unit(outs["k"].view(T, G, d)).repeat_interleave(H // G, 1)
    beta = torch.sigmoid(x[:, offs[3]:offs[3] + H])
    gdec = torch.exp(-torch.exp(A_log) * torch.nn.functional.softplus(x[:, offs[4]:offs[4] + H] + dt_bias))
    o, S = F.delta_rule(q, k, outs["v"].view(T, H, vd), gdec, beta, state[0])
    return o.reshape(T, H * vd), (S, torch.cat(keep, -1))


@pytest.mark.parametrize("form", ["token by token", "chunks"])
@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("H,G,d,vd,taps", [(4, 2, 16, 24, 4), (3, 3, 10, 36, 2), (2, 1, 64, 64, 3), (2, 2, 200, 8, 1), (1, 1, 128, 40, 5),
                                           (2, 1, 32, 128, 4), (1, 1, 16, 300, 2)])      # 1, 2, 4 and 10 slices of 32 value columns
def test_delta_rule_carries_both_states_between_portions_and_slots(ctx, ops, H, G, d, vd, taps, form, packed):
    """packed: q, k, v stand beside one another from column 0 (rows that allow 16-byte accesses when the sizes do); else at odd columns."""
    max_qlen = 1 if form == "token by token" else 64
    g = torch.Generator().manual_seed(14)
    slots, qk = 4, G * d
    C = 2 * qk + H * vd
    offs = (0, qk, 2 * qk, C, C + H) if packed else (2, 2 + qk + 1, 2 + 2 * qk + 3, 2 + C + 4, 2 + C + 4 + H + 1)
    ld = (offs[4] + H + 3) // 4 * 4 if packed else offs[4] + H + 2
    conv_w = torch.randn(C, taps, generator=g) * taps ** -0.5
    A_log, dt_bias = torch.log(0.3 + 2 * torch.rand(H, generator=g)), torch.randn(H, generator=g) * 0.5
    state = torch.randn(slots, H, d, vd, generator=g)                   # whatever an earlier owner left behind
    cstate = torch.randn(slots, max(taps - 1, 1), C, generator=g)
    state_d, cstate_d = state.to(DEV), cstate.to(DEV)
    lens = {"a": 37, "b": 6, "c": 97}
    data = {n: torch.randn(T, ld, generator=g) for n, T in lens.items()}
    want = {n: plain_delta(data[n], offs, H, G, d, vd, conv_w, A_log, dt_bias, None)[0] for n in lens}
    got = {n: torch.zeros(T, H * vd) for n, T in lens.items()}
    at = {n: 0 for n in lens}
    slot_of = {"a": 2, "b": 0, "c": 3}
    # steps of (name, count): portions beside single tokens, in changing batch order, portions shorter than the taps
    sched = [[("a", 20), ("b", 1)], [("b", 1), ("a", 1), ("c", 33)], [("c", 2), ("b", 3), ("a", 16)], [("c", 62), ("b", 1)]]
    kw = dict(heads=H, kv_heads=G, dim=d, vdim=vd, taps=taps, conv_w=conv_w.t().contiguous().to(DEV), conv_state=cstate_d, state=state_d, A_log=A_log.to(DEV),
              dt_bias=dt_bias.to(DEV))
    for step in sched:
        cu, pos, xs = [0], [], []
        for n, c in step:
            lo = at[n]
            xs.append(data[n][lo:lo + c])
            pos += list(range(lo, lo + c))
            cu.append(cu[-1] + c)
        o = ops.delta_rule(ctx, torch.cat(xs).to(DEV), offs, state_slots=i32([slot_of[n] for n, _ in step]), cu_seqlens=i32(cu), positions=i32(pos),
                           max_qlen=max_qlen, **kw)[0].cpu()
        for b, (n, c) in enumerate(step):
            got[n][at[n]:at[n] + c] = o[cu[b]:cu[b + 1]]
            at[n] += c
    for n in lens:
        assert at[n] == lens[n]
        assert torch.allclose(got[n], want[n], rtol=1e-4, atol=2e-5), n
    assert torch.equal(state_d[1].cpu(), state[1]) and torch.equal(cstate_d[1].cpu(), cstate[1])      # a slot nobody owns is not touched
    # decode form (no cu_seqlens): sequence "b" goes on, a new owner of slot 3 starts at position 0 over the old states
    xb, xn = torch.randn(1, ld, generator=g), torch.randn(1, ld, generator=g)
    sb = plain_delta(data["b"], offs, H, G, d, vd, conv_w, A_log, dt_bias, None)[1]
    o = ops.delta_rule(ctx, torch.cat([xb, xn]).to(DEV), offs, state_slots=i32([0, 3]), cu_seqlens=None, positions=i32([6, 0]), **kw)[0].cpu()
    assert torch.allclose(o[0], plain_delta(xb, offs, H, G, d, vd, conv_w, A_log, dt_bias, sb)[0][0], rtol=1e-4, atol=2e-5)
    assert torch.allclose(o[1], plain_delta(xn, offs, H, G, d, vd, conv_w, A_log, dt_bias, None)[0][0], rtol=1e-4, atol=2e-5)


def test_delta_rule_overwrites_what_a_key_held(ctx, ops):
    """With beta = 1 and no decay, writing twice under the same unit key leaves the SECOND value (a plain sum of outer products would
    leave both); an orthogonal key in between does not disturb it, 300 tokens later."""
    H, d, vd, T = 1, 16, 8, 300
    g = torch.Generator().manual_seed(15)
    ld = 2 * d + vd + 2 + vd
    x = torch.zeros(T, ld)
    big = 30.0                                   # silu(30) = 30, unit() then leaves an axis vector
    x[:, d + 1] = big                            # every other token writes along key axis 1
    x[0, d + 1] = x[5, d + 1] = 0.0
    x[0, d + 0] = x[5, d + 0] = big              # tokens 0 and 5 write along key axis 0
    x[:, 2 * d:2 * d + vd] = torch.randn(T, vd, generator=g)
    x[:, 2 * d + vd] = 40.0                      # beta = sigmoid(40) = 1
    x[:, 2 * d + vd + 1] = -60.0                 # softplus(-60) = 0: decay 1
    x[T - 1, 0] = big                            # the last token reads key axis 0
    conv_w = torch.ones(2 * d + vd, 1)           # one tap: the convolution passes its input through
    state, cstate = torch.zeros(1, H, d, vd, device=DEV), torch.zeros(1, 1, 2 * d + vd, device=DEV)
    v5 = torch.nn.functional.silu(x[5, 2 * d:2 * d + vd])
    for max_qlen in (1, T):
        state, cstate = torch.zeros(1, H, d, vd, device=DEV), torch.zeros(1, 1, 2 * d + vd, device=DEV)
        o, q, k, v, gb = ops.delta_rule(ctx, x.to(DEV), (0, d, 2 * d, 2 * d + vd, 2 * d + vd + 1), H, 1, d, vd, 1, conv_w.t().contiguous().to(DEV), cstate, state, i32([0]),
                                        i32([0, T]), i32(list(range(T))), torch.zeros(1, device=DEV), torch.zeros(1, device=DEV), max_qlen=max_qlen)
        assert torch.allclose(o.cpu()[T - 1], v5 * d ** -0.5, rtol=1e-4, atol=1e-6)


def test_a_decay_that_underflows_inside_a_chunk(ctx, ops):
    """Strong decays (g around e^-30 per token): over a 32-token chunk their product is far below the smallest float.  The chunked
    form exponentiates only differences of running log sums, so it stays finite and agrees with the token-by-token form."""
    g = torch.Generator().manual_seed(16)
    H, d, vd, T = 2, 16, 16, 70
    ld = 2 * d + H * vd + 2 * H
    x = torch.randn(T, ld, generator=g)
    x[:, 2 * d + H * vd + H:] += 3.0                 # large softplus arguments
    conv_w = torch.ones(2 * d + H * vd, 1)
    A_log = torch.tensor([2.3, -1.0])                # exp(2.3) ~ 10 per unit of softplus for head 0
    outs = []
    for max_qlen in (1, T):
        state, cstate = torch.zeros(1, H, d, vd, device=DEV), torch.zeros(1, 1, 2 * d + H * vd, device=DEV)
        o = ops.delta_rule(ctx, x.to(DEV), (0, d, 2 * d, 2 * d + H * vd, 2 * d + H * vd + H), H, 1, d, vd, 1, conv_w.t().contiguous().to(DEV), cstate, state, i32([0]),
                           i32([0, T]), i32(list(range(T))), A_log.to(DEV), torch.zeros(H, device=DEV), max_qlen=max_qlen)[0].cpu()
        assert torch.isfinite(o).all()
        outs.append(o)
    assert torch.allclose(outs[0], outs[1], rtol=1e-4, atol=1e-6)
