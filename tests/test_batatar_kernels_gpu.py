"""Each Batatar mechanism alone: the CUDA kernel against the plain fp32 functions of oracle/batatar_oracle.py, in both storage
formats where the kernel has both (bf16 serving, fp32 exact).  Inputs are built so that a fault shows: one key that stands out just
inside and just outside a chunk, a sink that takes a known share, a state that carries one early token to the end."""
import importlib
import math

import pytest
import torch

from oracle import batatar_oracle as B

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


def gen(seed):
    return torch.Generator().manual_seed(seed)


# ------------------------------------------------------------------------------------------ residual sums and norms
@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("H", [24, 37, 208, 1100, 5000])
def test_sum_of_two_normed_branches_and_the_next_norm(ctx, ops, dt, H):
    g = gen(2)
    N, eps = 7, 1e-3
    res, y0, y1 = torch.randn(N, H, generator=g) * 3, torch.randn(N, H, generator=g) * 40, torch.randn(N, H, generator=g) * 0.01
    w0, w1, w, bias = (1 + 0.2 * torch.randn(H, generator=g) for _ in range(4))
    d = {k: v.to(DEV) for k, v in dict(res=res, y0=y0, y1=y1, w0=w0, w1=w1, w=w, bias=bias).items()}
    # two mixers side by side: each output normed over the width with its own weight, halved, times the layer's constant
    s = res + 0.15 * B.rms_norm(y0, w0, eps) + 0.15 * B.rms_norm(y1, w1, eps)
    ro, o = ops.rms_norm_blend(ctx, d["res"], d["y0"], d["w0"], 0.15, d["y1"], d["w1"], 0.15, d["w"], eps=eps, out_dtype=dt)
    assert torch.allclose(ro.cpu(), s, rtol=1e-5, atol=1e-5)
    assert torch.allclose(o.float().cpu(), B.rms_norm(s, w, eps), **tol(dt))
    # one plain branch and a vector added to every row (a pass of a looped block opens like this)
    s = res + bias + 0.3 * y1
    ro, o = ops.rms_norm_blend(ctx, d["res"], d["y1"], None, 0.3, w=d["w"], bias=d["bias"], eps=eps, out_dtype=dt)
    assert torch.allclose(ro.cpu(), s, rtol=1e-5, atol=1e-5)
    assert torch.allclose(o.float().cpu(), B.rms_norm(s, w, eps), **tol(dt))
    # nothing to add: the first norm of a model
    ro, o = ops.rms_norm_blend(ctx, d["res"], w=d["w"], eps=eps, out_dtype=dt)
    assert torch.equal(ro.cpu(), res) and torch.allclose(o.float().cpu(), B.rms_norm(res, w, eps), **tol(dt))
    # gathered rows (the head): nothing is written back
    rows = i32([6, 0, 3])
    before = d["res"].clone()
    ro, o = ops.rms_norm_blend(ctx, d["res"], d["y0"], d["w0"], 0.5, w=d["w"], eps=eps, out_dtype=dt, rows=rows)
    assert ro is None and torch.equal(before, d["res"])
    assert torch.allclose(o.float().cpu(), B.rms_norm(res + 0.5 * B.rms_norm(y0, w0, eps), w, eps)[rows.cpu().long()], **tol(dt))
    # the sum itself in the storage format (the input of a product that reads the stream, not its norm)
    ro, o = ops.rms_norm_blend(ctx, d["res"], d["y1"], None, 2.0, eps=eps, out_dtype=dt, plain_out=True)
    assert torch.allclose(o.float().cpu(), res + 2.0 * y1, **tol(dt))


def test_the_norms_keep_eps_inside_the_root(ctx, ops):
    y = torch.full((2, 48), 1e-4)
    one = torch.ones(48)
    ro, o = ops.rms_norm_blend(ctx, torch.zeros(2, 48, device=DEV), y.to(DEV), one.to(DEV), 1.0, w=one.to(DEV), eps=1e-2)
    s = y / math.sqrt(1e-8 + 1e-2)
    assert torch.allclose(ro.cpu(), s, rtol=1e-5, atol=0)
    assert torch.allclose(o.cpu(), s / torch.sqrt((s * s).mean(-1, keepdim=True) + 1e-2), rtol=1e-5, atol=0)


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("groups,gsize", [(1, 72), (2, 32), (3, 20), (4, 256), (1, 3000)])
def test_gate_in_front_of_or_behind_a_norm_in_groups(ctx, ops, dt, groups, gsize):
    g = gen(3)
    N, eps, W = 5, 1e-4, groups * gsize
    o, z, w = torch.randn(N, W, generator=g) * 5, torch.randn(N, W + 8, generator=g), 1 + 0.2 * torch.randn(W, generator=g)
    zd = z.to(DEV)[:, 8:]
    # state space form: y silu(z) first, then every group by its own root mean square, then the weight
    want = B.rms_norm((o * B.silu(z[:, 8:])).view(N, groups, gsize), None, eps).reshape(N, W) * w
    got = ops.group_norm_gate(ctx, o.to(DEV), zd, w.to(DEV), groups, gsize, True, eps, "silu", out_dtype=dt)
    assert torch.allclose(got.float().cpu(), want, **tol(dt))
    # lightning form: the norm first (weight included), then a sigmoid gate
    want = B.rms_norm(o.view(N, groups, gsize), None, eps).reshape(N, W) * w * torch.sigmoid(z[:, 8:])
    got = ops.group_norm_gate(ctx, o.to(DEV), zd, w.to(DEV), groups, gsize, False, eps, "sigmoid", out_dtype=dt)
    assert torch.allclose(got.float().cpu(), want, **tol(dt))
    # where the two orders differ the kernel must not mix them up
    assert not torch.allclose(B.rms_norm(o * torch.sigmoid(z[:, 8:]), None, eps) * w, want, rtol=1e-2, atol=1e-2)


# ------------------------------------------------------------------------------------------ projections' epilogue: bias, unit heads, silu
@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("H,G,d,vd", [(4, 2, 16, 24), (3, 3, 40, 8), (8, 1, 24, 80), (2, 2, 128, 64)])
def test_bias_then_heads_divided_by_their_root_mean_square(ctx, ops, dt, H, G, d, vd):
    g = gen(4)
    N, eps, pad = 9, 1e-3, 5
    cols = pad + H * d + G * d + G * vd
    x, bias = torch.randn(N, cols, generator=g) * 3, torch.randn(cols, generator=g)
    q_off, k_off, v_off = pad, pad + H * d, pad + H * d + G * d
    slots = i32([11, 3, 7, 0, 19, 18, 4, 12, 1])
    q = torch.empty(N, H * d, dtype=dt, device=DEV)
    kc, vc = torch.zeros(20, G * d, dtype=dt, device=DEV), torch.zeros(20, G * vd, dtype=dt, device=DEV)
    ops.qkv_prep(ctx, x.to(DEV), q_off, k_off, v_off, H, G, d, vd, q, kc, vc, bias=bias.to(DEV), eps=eps, slot_mapping=slots, unit_norm=True)
    xb = x + bias
    wq = B.rms_norm(xb[:, q_off:k_off].view(N, H, d), None, eps).reshape(N, -1)
    wk = B.rms_norm(xb[:, k_off:v_off].view(N, G, d), None, eps).reshape(N, -1)
    assert torch.allclose(q.float().cpu(), wq, **tol(dt))
    assert torch.allclose(kc.float().cpu()[slots.cpu().long()], wk, **tol(dt))
    assert torch.allclose(vc.float().cpu()[slots.cpu().long()], xb[:, v_off:], **tol(dt))
    untouched = [s for s in range(20) if s not in slots.cpu().tolist()]
    assert float(kc[untouched].abs().max()) == 0.0


@pytest.mark.parametrize("H,d,vd,pad", [(3, 16, 24, 8), (3, 5, 7, 1), (16, 128, 128, 0)])
def test_silu_on_all_three_projections(ctx, ops, H, d, vd, pad):
    """Sizes whose rows allow 16-byte accesses take the flat element-wise kernel, the others the general one."""
    g = gen(5)
    N = 6
    x = torch.randn(N, 2 * H * d + H * vd + pad, generator=g) * 2
    q, k, v = (torch.empty(N, H * w, device=DEV) for w in (d, d, vd))
    ops.qkv_prep(ctx, x.to(DEV), 0, H * d, 2 * H * d, H, H, d, vd, q, k, v, silu=True)
    assert torch.allclose(q.cpu(), B.silu(x[:, :H * d]), rtol=2e-5, atol=2e-5)
    assert torch.allclose(k.cpu(), B.silu(x[:, H * d:2 * H * d]), rtol=2e-5, atol=2e-5)
    assert torch.allclose(v.cpu(), B.silu(x[:, 2 * H * d:2 * H * d + H * vd]), rtol=2e-5, atol=2e-5)


# ------------------------------------------------------------------------------------------ capped attention inside chunks
def paged(k, v, bs, nblocks, g):
    """Scatters per-sequence k / v rows [T, kw] into pools through a shuffled block table; returns (kc, vc, table rows)."""
    order = torch.randperm(nblocks, generator=g).tolist()
    kc, vc = torch.zeros(nblocks * bs, k[0].shape[1]), torch.zeros(nblocks * bs, v[0].shape[1])
    tables, at = [], 0
    for kk, vv in zip(k, v):
        nb = (kk.shape[0] + bs - 1) // bs
        bl = order[at:at + nb]
        at += nb
        for j in range(kk.shape[0]):
            kc[bl[j // bs] * bs + j % bs] = kk[j]
            vc[bl[j // bs] * bs + j % bs] = vv[j]
        tables.append(bl)
    width = max(len(t) for t in tables)
    return kc, vc, [t + [-1] * (width - len(t)) for t in tables]


def run_chunk_attention(ctx, ops, dt, H, G, d, vd, lens, qlens, bs, chunk, cap, scale, seed=0, boost=None, sink=True):
    """Sequences of lens[b] tokens whose last qlens[b] are queried.  boost = (b, query row, key position, factor) makes one raw
    score (before the cap) stand out.  Returns (got, want, values of sequence 0)."""
    g = gen(seed)
    ks = [torch.randn(n, G, d, generator=g) for n in lens]
    vs = [torch.randn(n, G, vd, generator=g) for n in lens]
    qs = [torch.randn(m, H, d, generator=g) for m in qlens]
    if boost:
        b, i, j, f = boost
        qs[b][i, :] = qs[b][i, 0]
        ks[b][j, :] = qs[b][i, 0] * f / (qs[b][i, 0] @ qs[b][i, 0])
    if dt == torch.bfloat16:
        ks, vs, qs = ([t.bfloat16().float() for t in x] for x in (ks, vs, qs))
    rows = sum(qlens)
    gt = torch.randn(rows, H + 3, generator=g)
    want, r0 = [], 0
    for b, (n, m) in enumerate(zip(lens, qlens)):
        o = B.capped_chunk_softmax(qs[b], ks[b], vs[b], n - m, scale, cap, chunk, sink)
        want.append((o * torch.sigmoid(gt[r0:r0 + m, 3:]).unsqueeze(-1)).reshape(m, H * vd))
        r0 += m
    nblocks = sum((n + bs - 1) // bs for n in lens) + 3
    kc, vc, tables = paged([k.reshape(k.shape[0], -1) for k in ks], [v.reshape(v.shape[0], -1) for v in vs], bs, nblocks, g)
    cu = [0]
    for m in qlens:
        cu.append(cu[-1] + m)
    decode = all(m == 1 for m in qlens)
    zero_sink = torch.zeros(H, device=DEV) if sink else None
    got = ops.attn_paged_wide(ctx, torch.cat(qs).reshape(rows, H * d).to(dt).to(DEV), kc.to(dt).to(DEV), vc.to(dt).to(DEV), i32(tables), i32(lens),
                              None if decode else i32(cu), max(qlens), bs, H, G, d, vd, scale, 0, zero_sink, gt.to(DEV)[:, 3:], 1.0,
                              softcap=cap, chunk=chunk, gate_per_head=True)
    return got.float().cpu(), torch.cat(want), vs[0]


SHAPES = [(4, 2, 32, 48), (3, 3, 40, 24), (6, 1, 16, 80), (2, 2, 64, 128), (8, 2, 48, 96)]


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("H,G,d,vd", SHAPES)
@pytest.mark.parametrize("chunk,cap", [(0, 0.0), (13, 5.0), (16, 0.0), (50, 30.0)])
def test_capped_chunked_attention_over_a_mixed_batch(ctx, ops, dt, H, G, d, vd, chunk, cap):
    got, want, _ = run_chunk_attention(ctx, ops, dt, H, G, d, vd, lens=[70, 1, 33, 129, 16], qlens=[70, 1, 2, 40, 1], bs=16, chunk=chunk, cap=cap,
                                       scale=0.4, seed=H)
    assert torch.allclose(got, want, **tol(dt))


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("bs", [16, 64])
def test_decode_rows_without_cu_seqlens(ctx, ops, dt, bs):
    got, want, _ = run_chunk_attention(ctx, ops, dt, 4, 2, 32, 48, lens=[300, 1, 64, 65, 17, 40, 41], qlens=[1] * 7, bs=bs, chunk=40, cap=10.0,
                                       scale=0.3, seed=9)
    assert torch.allclose(got, want, **tol(dt))


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("qlen", [1, 2, 37])
@pytest.mark.parametrize("n,key,seen", [
    (420, 400, True),        # the chunk's first token, 19 back
    (420, 399, False),       # the last token of the chunk before
    (420, 380, False),
    (420, 0, False),
    (401, 400, True),        # the query opens a chunk: it sees itself alone
    (401, 399, False),
    (400, 380, True),        # the query closes a chunk and sees all of it
    (400, 379, False),
    (15, 0, True),           # the first chunk is shorter than its size allows
])
def test_the_chunk_edge_is_where_it_belongs(ctx, ops, dt, qlen, n, key, seen):
    """One key gets a raw score far above the rest.  With chunks of 20 counted from position 0 the last query row sees it only if both
    lie in the same chunk - wherever the portion was cut (the portion of 37 rows starts in an earlier chunk).  Seen, it takes nearly
    all the weight (the cap of 30 leaves exp(30) against a few hundred small terms and the sink); unseen, none."""
    if qlen > n:
        pytest.skip("portion longer than the sequence")
    H, G, d, vd = 4, 2, 32, 48
    got, want, vs = run_chunk_attention(ctx, ops, dt, H, G, d, vd, lens=[n], qlens=[qlen], bs=16, chunk=20, cap=30.0, scale=1.0, seed=11,
                                        boost=(0, qlen - 1, key, 60.0))
    assert torch.allclose(got, want, **tol(dt))
    # undo the head gates on the last row: the attended value itself
    g = gen(11)
    for shape in ((n, G, d), (n, G, vd), (qlen, H, d)):
        torch.randn(*shape, generator=g)
    gate = torch.sigmoid(torch.randn(qlen, H + 3, generator=g)[-1, 3:])
    vj = torch.stack([vs[key, h // (H // G)] for h in range(H)])
    close = torch.allclose(got[-1].view(H, vd) / gate.view(H, 1), vj, rtol=0.05, atol=0.05)
    assert close == seen


@pytest.mark.parametrize("dt", DTS)
def test_the_cap_bounds_a_score_and_the_sink_takes_its_share(ctx, ops, dt):
    """Two tokens, one head: the query matches key 1 with raw score 50 and key 0 with raw score 0.  Capped at 2, the weights are
    e^(2 tanh 25) / (1 + 1 + e^2) for key 1 and 1 / (2 + e^2) for key 0; without the sink term the denominators would lose the 1,
    without the cap key 1 would take everything."""
    d, vd = 16, 8
    q = torch.zeros(1, 1, d)
    q[0, 0, 0] = 5.0
    k = torch.zeros(2, 1, d)
    k[1, 0, 0] = 10.0
    k[0, 0, 1] = 3.0
    v = torch.zeros(2, 1, vd)
    v[0, 0, 0] = 1.0
    v[1, 0, 1] = 1.0
    gate = torch.full((1, 1), 30.0)          # sigmoid = 1
    got = ops.attn_paged_wide(ctx, q.reshape(1, d).to(dt).to(DEV), k.reshape(2, d).to(dt).to(DEV), v.reshape(2, vd).to(dt).to(DEV), i32([[0]]),
                              i32([2]), i32([0, 1]), 1, 16, 1, 1, d, vd, 1.0, 0, torch.zeros(1, device=DEV), gate.to(DEV), 1.0, softcap=2.0, chunk=0,
                              gate_per_head=True).float().cpu()
    e2 = math.exp(2.0 * math.tanh(25.0))
    assert abs(float(got[0, 0]) - 1.0 / (2.0 + e2)) < 2e-3 and abs(float(got[0, 1]) - e2 / (2.0 + e2)) < 5e-3
    assert abs(float(got[0, 1]) - e2 / (1.0 + e2)) > 0.05


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("where", [0, 1, 15, 16, 17, 500, 1023, 1024])
@pytest.mark.parametrize("qlens", [[3, 40], [1, 1]])
def test_one_far_key_in_a_long_chunk(ctx, ops, dt, where, qlens):
    """A chunk longer than the sequence: one key among 1 100 takes nearly all the weight of the last row, wherever it lies - the
    first tokens, either side of a page border, far back - in a portion and in a decode step."""
    got, want, _ = run_chunk_attention(ctx, ops, dt, 4, 2, 32, 48, lens=[1100, 40], qlens=qlens, bs=16, chunk=4096, cap=50.0, scale=1.0, seed=12,
                                       boost=(0, qlens[0] - 1, where, 40.0))
    assert torch.allclose(got, want, **tol(dt))


# ------------------------------------------------------------------------------------------ selective state space layer
def run_steps(sched, lens, slot_of, step_fn):
    """Drives step_fn(names, counts, starts, cu, pos, slots) -> rows over a schedule of (name, count) steps; returns name -> rows."""
    at = {n: 0 for n in lens}
    got = {n: [] for n in lens}
    for step in sched:
        cu, pos = [0], []
        for n, c in step:
            pos += list(range(at[n], at[n] + c))
            cu.append(cu[-1] + c)
        o = step_fn([n for n, _ in step], [c for _, c in step], [at[n] for n, _ in step], cu, pos, [slot_of[n] for n, _ in step])
        for b, (n, c) in enumerate(step):
            got[n].append(o[cu[b]:cu[b + 1]])
            at[n] += c
    assert at == lens
    return {n: torch.cat(v) for n, v in got.items()}


SCHED = [[("a", 20), ("b", 1)], [("b", 1), ("a", 1), ("c", 33)], [("c", 1), ("b", 2), ("a", 2)], [("b", 1), ("a", 14)], [("c", 63)]]
LENS = {"a": 37, "b": 5, "c": 97}
SLOTS = {"a": 2, "b": 0, "c": 3}


@pytest.mark.parametrize("form", ["token by token", "32 tokens at a time"])
@pytest.mark.parametrize("H,G,N,vd,taps", [(4, 2, 8, 16, 4), (3, 3, 16, 24, 2), (2, 1, 32, 64, 3), (8, 4, 24, 32, 3), (1, 1, 128, 40, 1), (6, 1, 5, 7, 5)])
def test_state_space_layer_carries_both_states_between_portions_and_slots(ctx, ops, H, G, N, vd, taps, form):
    """Convolution with bias and silu, step sizes, the recurrence and the skip term against the token-by-token restatement, over
    portions down to one and two tokens (shorter than the taps), in slots that an earlier owner left full."""
    g = gen(20)
    inner, C = H * vd, H * vd + 2 * G * N
    pad = 8 if H % 4 == 0 else 6          # rows that allow 16-byte accesses (first and fourth case) and rows that do not
    ld = pad + inner + C + H            # [pad | z | x B C | dt]
    conv_w, conv_b = torch.randn(C, taps, generator=g) * taps ** -0.5, torch.randn(C, generator=g) * 0.2
    A_log, dt_bias, D = torch.log(0.1 + 1.5 * torch.rand(H, generator=g)), torch.randn(H, generator=g) * 0.5, torch.randn(H, generator=g)
    rows = {n: torch.randn(T, ld, generator=g) for n, T in LENS.items()}
    want = {}
    for n, T in LENS.items():
        u = rows[n][:, pad + inner:]
        xbc, _ = B.conv_bias_silu(u[:, :C], conv_w, conv_b, torch.zeros(taps - 1, C))
        dt = torch.nn.functional.softplus(u[:, C:] + dt_bias, threshold=1e9)
        y, _ = B.ssd_recurrence(xbc[:, :inner].reshape(T, H, vd), xbc[:, inner:inner + G * N].reshape(T, G, N),
                                xbc[:, inner + G * N:].reshape(T, G, N), dt, A_log, D, torch.zeros(H, N, vd))
        want[n] = y.reshape(T, inner)
    state = torch.randn(4, H, N, vd, generator=g).to(DEV)
    conv_state = torch.randn(4, max(taps - 1, 1), C, generator=g).to(DEV)
    keep = (state[1].clone(), conv_state[1].clone())
    cw = conv_w.T.contiguous().to(DEV)           # tap-major
    dev = {k: v.to(DEV) for k, v in dict(conv_b=conv_b, A_log=A_log, dt_bias=dt_bias, D=D).items()}
    max_qlen = 1 if form == "token by token" else 64

    def step(names, counts, starts, cu, pos, slots):
        x = torch.cat([rows[n][s:s + c] for n, c, s in zip(names, counts, starts)]).to(DEV)
        decode = all(c == 1 for c in counts)
        cu_d = None if decode else i32(cu)
        xo, vo, bo, co, ldec = ops.ssd_prep(ctx, x, pad + inner, pad + inner + C, H, vd, G, N, taps, cw, dev["conv_b"], conv_state, i32(slots), cu_d,
                                            i32(pos), dev["A_log"], dev["dt_bias"])
        return ops.decay_scan(ctx, co, bo, vo, state, i32(slots), cu_d, i32(pos), H, G, N, vd, log_decay=ldec, skip=xo, skip_w=dev["D"],
                              max_qlen=max(counts) if max_qlen > 1 else 1).cpu()

    got = run_steps(SCHED, LENS, SLOTS, step)
    for n in LENS:
        assert torch.allclose(got[n], want[n], rtol=1e-4, atol=1e-4), n
    assert torch.equal(state[1], keep[0]) and torch.equal(conv_state[1], keep[1])       # a slot nobody owns is not touched


def test_step_sizes_are_a_softplus_without_a_clamp(ctx, ops):
    """dt inputs of -30, 0 and +30: softplus gives e^-30, log 2 and 30 (a clamp at either end would show), the decay's logarithm is
    -exp(A_log) dt and v = dt x."""
    H, vd, G, N = 3, 4, 1, 4
    inner, C = H * vd, H * vd + 2 * G * N
    x = torch.zeros(1, inner + C + H)
    x[0, inner:inner + inner] = 1.0
    x[0, inner + C:] = torch.tensor([-30.0, 0.0, 30.0])
    cw = torch.ones(1, C)
    A_log = torch.tensor([0.0, 1.0, -1.0])
    xo, vo, bo, co, ld = ops.ssd_prep(ctx, x.to(DEV), inner, inner + C, H, vd, G, N, 1, cw.to(DEV), torch.zeros(C, device=DEV),
                                      torch.zeros(1, 1, C, device=DEV), i32([0]), None, i32([0]), A_log.to(DEV), torch.zeros(H, device=DEV))
    dt = torch.tensor([math.exp(-30.0), math.log(2.0), 30.0])
    silu1 = 1.0 / (1.0 + math.exp(-1.0))
    assert torch.allclose(ld.cpu()[0], -torch.exp(A_log) * dt, rtol=1e-5, atol=0)
    assert torch.allclose(vo.cpu()[0].view(H, vd)[:, 0], dt * silu1, rtol=1e-5, atol=0)
    assert torch.allclose(xo.cpu()[0], torch.full((inner,), silu1), rtol=1e-5, atol=0)


def test_a_decay_that_underflows_inside_a_chunk(ctx, ops):
    """Log decays of -200 per token: the running sums pass the range of exp inside a chunk; differences stay exact, and a token
    sees only itself and a vanishing part of its predecessor - no NaN from 0 x inf."""
    H, d, vd, T = 2, 16, 8, 70
    g = gen(21)
    q, k, v = (torch.randn(T, H * w, generator=g) for w in (d, d, vd))
    ld = torch.full((T, H), -200.0)
    ld[:, 1] = -1e-3
    y, _ = B.ssd_recurrence(v.view(T, H, vd), k.view(T, H, d), q.view(T, H, d), torch.ones(T, H), torch.log(-ld[0]), torch.zeros(H),
                            torch.zeros(H, d, vd))
    for max_qlen in (1, T):
        state = torch.zeros(1, H, d, vd, device=DEV)
        o = ops.decay_scan(ctx, q.to(DEV), k.to(DEV), v.to(DEV), state, i32([0]), i32([0, T]), i32(list(range(T))), H, H, d, vd,
                           log_decay=ld.to(DEV), max_qlen=max_qlen).cpu()
        assert torch.isfinite(o).all() and torch.allclose(o, y.reshape(T, H * vd), rtol=1e-4, atol=1e-4)


# ------------------------------------------------------------------------------------------ lightning attention
@pytest.mark.parametrize("form", ["token by token", "32 tokens at a time"])
@pytest.mark.parametrize("H,d,vd", [(3, 16, 24), (4, 64, 48), (1, 8, 1), (2, 200, 72)])
def test_constant_decay_recurrence_between_portions_and_slots(ctx, ops, H, d, vd, form):
    g = gen(22)
    decay = torch.tensor([0.5, 0.999, 0.97, 0.0])[:H].contiguous()
    data = {n: (torch.randn(T, H, d, generator=g), torch.randn(T, H, d, generator=g) * d ** -0.5, torch.randn(T, H, vd, generator=g))
            for n, T in LENS.items()}
    want = {n: B.decay_recurrence(*data[n], decay, torch.zeros(H, d, vd))[0].reshape(LENS[n], H * vd) for n in LENS}
    state = torch.randn(4, H, d, vd, generator=g).to(DEV)

    def step(names, counts, starts, cu, pos, slots):
        q, k, v = (torch.cat([data[n][i][s:s + c] for n, c, s in zip(names, counts, starts)]).reshape(cu[-1], -1).to(DEV) for i in range(3))
        decode = all(c == 1 for c in counts)
        return ops.retention_scan(ctx, q, k, v, state, i32(slots), None if decode else i32(cu), i32(pos), decay.to(DEV), H, d, vd,
                                  1 if form == "token by token" else max(counts)).cpu()

    got = run_steps(SCHED, LENS, SLOTS, step)
    for n in LENS:
        assert torch.allclose(got[n], want[n], rtol=1e-4, atol=1e-4), n


def test_an_early_token_comes_back_with_the_power_of_its_decay(ctx, ops):
    """Token 3 writes along an axis that only the last token reads, 596 tokens later: the output is decay^596 of its value - a
    lost, restarted or doubly decayed state shows at once."""
    H, d, vd, T = 2, 16, 8, 600
    decay = torch.tensor([0.99, 0.999])
    q, k, v = torch.zeros(T, H, d), torch.zeros(T, H, d), torch.randn(T, H, vd, generator=gen(23))
    k[:, :, 1] = 1.0
    k[3, :, :] = 0.0
    k[3, :, 0] = 1.0
    q[T - 1, :, 0] = 1.0
    for cuts in ([T], [1] * 7 + [2, 33, 64, T - 106], [T - 40] + [1] * 40):
        state = torch.full((1, H, d, vd), 7.0, device=DEV)
        at = 0
        for c in cuts:
            o = ops.retention_scan(ctx, q[at:at + c].reshape(c, -1).to(DEV), k[at:at + c].reshape(c, -1).to(DEV), v[at:at + c].reshape(c, -1).to(DEV),
                                   state, i32([0]), None if c == 1 else i32([0, c]), i32(list(range(at, at + c))), decay.to(DEV), H, d, vd, c)
            at += c
        o = o.cpu()[-1].view(H, vd)
        for h in range(H):
            assert torch.allclose(o[h], float(decay[h]) ** (T - 1 - 3) * v[3, h], rtol=1e-4, atol=1e-6)


# ------------------------------------------------------------------------------------------ experts whose weight multiplies their input
@pytest.mark.parametrize("E,top", [(5, 2), (16, 1), (3, 3), (8, 4)])
def test_sigmoid_router_keeps_the_scores_as_they_are(ctx, ops, E, top):
    g = gen(24)
    z = torch.randn(50, E + 3, generator=g) * 2
    idx, w = ops.moe_route_logits_ex(ctx, z.to(DEV), torch.zeros(E, device=DEV), E, top, 1.0, ops.ROUTE_SIGMOID, False)
    s = torch.sigmoid(z[:, :E])
    wi = torch.topk(s, top, dim=-1)
    assert torch.equal(idx.cpu().long().sort(-1).values, wi.indices.sort(-1).values)
    assert torch.allclose(w.cpu().sort(-1).values, wi.values.sort(-1).values, rtol=1e-6, atol=1e-7)      # not renormalised: sums differ from 1


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("E,top,ff,W", [(5, 2, 40, 96), (16, 1, 96, 64), (3, 3, 24, 40), (4, 2, 128, 128)])
def test_the_weight_enters_before_the_expert(ctx, ops, dt, E, top, ff, W):
    """sum_e E_e(s_e h) with gated experts: scaling the input is not scaling the output (silu is not homogeneous), so a kernel path
    that weighted the outputs would miss by far more than rounding."""
    g = gen(25)
    N = 37
    h = torch.randn(N, W, generator=g)
    p = {"router": torch.randn(E, W, generator=g) * 2 * W ** -0.5}
    for e in range(E):
        p[f"e{e}.gate"], p[f"e{e}.up"] = torch.randn(ff, W, generator=g) * 2 * W ** -0.5, torch.randn(ff, W, generator=g) * 2 * W ** -0.5
        p[f"e{e}.down"] = torch.randn(W, ff, generator=g) * ff ** -0.5
    if dt == torch.bfloat16:
        h = h.bfloat16().float()
        p = {k: v.bfloat16().float() for k, v in p.items()}
    m = {"router": {"experts": E, "top": top}}
    want = B.moe_ff(h, p, m)
    idx_w, s_w = B.route(h, p, m)
    hd = h.to(dt).to(DEV)
    z = ops.linear(ctx, hd, p["router"].to(dt).to(DEV), out_dtype=torch.float32)
    idx, w = ops.moe_route_logits_ex(ctx, z, torch.zeros(E, device=DEV), E, top, 1.0, ops.ROUTE_SIGMOID, False)
    assert torch.equal(idx.cpu().long().sort(-1).values, idx_w.sort(-1).values)
    offsets, src, pos = ops.moe_sort(ctx, idx, E)
    xs = ops.moe_scatter_scaled(ctx, hd, pos, w, N * top)
    # every pair's row is the token's row times its score, rounded once
    got_rows = xs.float().cpu()[pos.cpu().long()].view(N, top, W)
    assert torch.allclose(got_rows, (w.cpu().unsqueeze(-1) * h.unsqueeze(1)), **tol(dt))
    wgu = torch.stack([torch.cat([p[f"e{e}.gate"], p[f"e{e}.up"]]) for e in range(E)]).to(dt).to(DEV)
    wd = torch.stack([p[f"e{e}.down"] for e in range(E)]).to(dt).to(DEV)
    hid2 = ops.linear_grouped(ctx, xs, None, wgu, offsets, N * top)
    hid = ops.act_mul_p(ctx, hid2, ff, ff, ops.ACT_SILU_MUL)
    y = ops.linear_grouped(ctx, hid, None, wd, offsets, N * top, out_dtype=torch.float32)
    got = ops.moe_combine(ctx, y, pos, torch.ones(N, top, device=DEV)).cpu()
    assert torch.allclose(got, want, **(dict(rtol=1e-4, atol=1e-4) if dt == torch.float32 else dict(rtol=5e-2, atol=5e-2)))
    # the other order - weights on the outputs - is a different function
    other = torch.zeros_like(want)
    for n in range(N):
        for t in range(top):
            other[n] += s_w[n, t] * B.expert(h[n], p, int(idx_w[n, t]))
    assert (other - want).abs().max() > 0.05
