"""Batatar through the runner and the engine: logits of every position against the plain fp32 oracle, whatever the schedule -
whole prompts, token-by-token decoding, portions down to two tokens, mixed batches, reused pages and state slots - plus greedy
generation through LLMEngine's own scheduler.  Small configurations whose sizes differ from one another (head counts, key / value /
state sizes, chunk sizes, taps, expert counts, loops), layers without feed-forward, models that start with either mixer.

The bf16 rigs route every token to every expert (top = all): a bf16-rounded router input can flip a near-tie between two experts,
after which the position - and every later one that reads it - differs by far more than rounding.  The choice itself is tested in
fp32 here and in both formats at the kernel level."""
import importlib

import numpy as np
import pytest
import torch

from oracle import batatar_oracle as B

pytestmark = pytest.mark.gpu
BLOCK = 16


def cfg_a(all_experts=False):
    """parallel + experts / a looped block of (lightning + experts, parallel without feed-forward) run twice / lightning + experts.
    Chunks of 12 tokens against pages of 16: chunk and page borders never coincide for long."""
    top = (lambda e: e) if all_experts else (lambda e: 2)
    return B.make_config(vocab=200, width=96, residual_mult=0.4, loop=(1, 3, 2), layers=[
        B.with_moe(B.parallel_cfg(), 5, top(5), 40),
        B.with_moe(B.lightning_cfg(), 3, top(3) if all_experts else 1, 24),
        B.with_moe(B.parallel_cfg(heads=2, kv_heads=2, dim=8, vdim=12, chunk=5, scale=0.5, softcap=3.0, s_heads=2, s_vdim=24, s_state=16,
                                  s_groups=1, conv=2, norm_groups=1), None),
        B.with_moe(B.lightning_cfg(heads=2, dim=24, vdim=16), 4, 4, 8),
    ])


def cfg_b(all_experts=False):
    """Starts with a lightning layer; sizes that are multiples of nothing; one head; a chunk of one token (every token sees
    itself and the sink only) and one longer than any prompt; one tap; a loop over a single layer three times at the end."""
    return B.make_config(vocab=203, width=100, eps=1e-3, residual_mult=1.0, loop=(3, 4, 3), layers=[
        B.with_moe(B.lightning_cfg(heads=1, dim=20, vdim=36, decay=[0.9]), 4, 4 if all_experts else 1, 33),
        B.with_moe(B.parallel_cfg(heads=1, kv_heads=1, dim=20, vdim=10, chunk=1, scale=0.3, softcap=50.0, s_heads=3, s_vdim=10, s_state=12,
                                  s_groups=3, conv=1, norm_groups=3), None),
        B.with_moe(B.parallel_cfg(heads=6, kv_heads=3, dim=12, vdim=20, chunk=1000, scale=0.2, softcap=1.5, s_heads=5, s_vdim=8, s_state=20,
                                  s_groups=1, conv=5, norm_groups=5), 2, 2, 50),
        B.with_moe(B.lightning_cfg(heads=5, dim=8, vdim=12), 3, 3 if all_experts else 2, 16),
    ])


def cfg_c(all_experts=False):
    """Sizes of the tensor-pipe routes of the bf16 mode: heads of 64 and 128 numbers, experts of 128 hidden units (grouped tcgen05
    products), a loop over the whole model."""
    return B.make_config(vocab=160, width=128, residual_mult=0.35, loop=(0, 2, 2), layers=[
        B.with_moe(B.parallel_cfg(heads=4, kv_heads=2, dim=64, vdim=64, chunk=48, scale=0.1, softcap=25.0, s_heads=4, s_vdim=32, s_state=32,
                                  s_groups=2, conv=4, norm_groups=2), 4, 4 if all_experts else 2, 128),
        B.with_moe(B.lightning_cfg(heads=2, dim=64, vdim=128), 3, 3 if all_experts else 1, 160),
    ])


class Rig:
    def __init__(self, cfg, dtype, blocks=40, seed=0, chunked=True, seqs=4, weights=None):
        self.eng = importlib.import_module("nano-vllm-candle_b200.engine")
        self.cfg, self.dtype = cfg, dtype
        self.w = weights if weights is not None else B.make_weights(cfg, seed)
        self.oracle = B.Batatar(cfg, self.w)
        self.ctx = self.eng.DeviceContext(0)
        T = blocks * BLOCK
        self.blocks = blocks
        self.runner = self.eng.ModelRunner.from_config(self.ctx, cfg, self.w.items(), num_kvcache_blocks=blocks, kvcache_block_size=BLOCK,
                                                       max_num_seqs=seqs, max_num_batched_tokens=T, max_model_len=T, dtype=dtype,
                                                       max_logit_rows=T)
        sc = self.eng.SchedulerConfig(max_num_seqs=seqs, max_num_batched_tokens=T, eos=-1, num_kvcache_blocks=blocks,
                                      kvcache_block_size=BLOCK, enable_chunked_prefill=chunked, max_model_len=T)
        self.engine = self.eng.LLMEngine(self.eng.Scheduler(sc), self.runner, greedy=True)
        # error of a position: rms over the vocabulary of the mean-free logit difference, relative to the logits' own rms
        self.tol = 1e-4 if dtype == "float32" else 0.06

    def close(self):
        self.engine.close()
        self.runner.close()
        self.ctx.close()

    def want(self, tokens):
        return self.oracle.forward(tokens).numpy()

    def replay(self, prompts, schedule):
        """schedule: steps of [(request, count)]; every position's logits are collected; requests end when exhausted."""
        live, at = {}, {k: 0 for k in prompts}
        got = {k: np.zeros((len(v), self.cfg["vocab"]), np.float32) for k, v in prompts.items()}
        for step in schedule:
            entries = []
            for name, n in step:
                if name not in live:
                    live[name] = self.engine.open_request()
                entries.append((live[name], prompts[name][at[name]:at[name] + n], list(range(n))))
            lg = self.engine.step_forced(entries)
            row = 0
            for name, n in step:
                got[name][at[name]:at[name] + n] = lg[row:row + n]
                row += n
                at[name] += n
                if at[name] == len(prompts[name]):
                    self.engine.close_request(live.pop(name))
        assert all(at[k] == len(v) for k, v in prompts.items())
        return got

    def check(self, prompts, schedule):
        got = self.replay(prompts, schedule)
        for k, toks_ in prompts.items():
            err = self.rel_err(got[k], self.want(toks_))
            bad = err >= self.tol
            assert not bad.any(), \
                f"{k}: {int(bad.sum())} of {len(toks_)} positions over {self.tol}, first {int(np.argmax(bad))}, worst {err.max():.4g}"

    @staticmethod
    def rel_err(got, want):
        d = got - want
        d = d - d.mean(-1, keepdims=True)
        w = want - want.mean(-1, keepdims=True)
        return np.sqrt((d * d).mean(-1)) / np.sqrt((w * w).mean(-1))


def toks(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def rig(request):
    r = Rig(cfg_a(all_experts=request.param == "bfloat16"), request.param)
    yield r
    r.close()


def test_whole_prompts_and_first_tokens(rig):
    V = rig.cfg["vocab"]
    rig.check({"one": toks(1, V, 1)}, [[("one", 1)]])
    rig.check({"two": toks(2, V, 2)}, [[("two", 2)]])
    rig.check({"three": toks(3, V, 2)}, [[("three", 3)]])            # fewer tokens than the convolution has taps
    rig.check({"p": toks(83, V, 2)}, [[("p", 83)]])
    rig.check({"page": toks(2 * BLOCK, V, 3)}, [[("page", 2 * BLOCK)]])


def test_residual_stream_after_every_layer_run(rig):
    p = toks(21, rig.cfg["vocab"], 4)
    tap = rig.runner.tap_residual(len(p))
    sid = rig.engine.open_request()
    rig.engine.step_forced([(sid, p, [0])])
    rig.engine.close_request(sid)
    res = []
    rig.oracle.forward(p, taps=res)
    assert tap.shape[0] == len(res) == 6            # the looped layers count once per pass
    for k, want in enumerate(res):
        assert np.abs(tap[k] - want.numpy()).max() < (2e-4 if rig.dtype == "float32" else 0.3), f"layer run {k}"


def test_prefill_then_token_by_token(rig):
    p = toks(70, rig.cfg["vocab"], 5)
    rig.check({"d": p}, [[("d", 30)]] + [[("d", 1)]] * 40)
    rig.check({"d": p}, [[("d", 1)]] * 70)                       # decoding from the very first token, across page and chunk borders


def test_portions_of_many_sizes(rig):
    p = toks(121, rig.cfg["vocab"], 6)
    sizes = [2, 10, 12, 1, 7, 16, 2, 31, 3, 35, 2]      # cuts before, at and after page and chunk borders; portions shorter than the taps
    assert sum(sizes) == 121
    rig.check({"c": p}, [[("c", n)] for n in sizes])
    rig.check({"c": p}, [[("c", 2)]] * 60 + [[("c", 1)]])
    rig.check({"c": p}, [[("c", 1)], [("c", 2)], [("c", 1)], [("c", 3)], [("c", 2)], [("c", 112)]])


def test_long_decoding(rig):
    p = toks(300, rig.cfg["vocab"], 7)
    rig.check({"l": p}, [[("l", 5)]] + [[("l", 1)]] * 295)


def test_mixed_batches_equal_each_request_alone(rig):
    V = rig.cfg["vocab"]
    pr = {"a": toks(90, V, 8), "b": toks(37, V, 9), "c": toks(3, V, 10), "d": toks(64, V, 11)}
    sched = [[("a", 40), ("b", 2)], [("a", 1), ("b", 20), ("c", 1)], [("a", 1), ("c", 1), ("d", 64)], [("a", 17), ("b", 1), ("c", 1)],
             [("a", 1), ("b", 14)]] + [[("a", 1)]] * 30
    assert all(sum(n for s in sched for k, n in s if k == name) == len(p) for name, p in pr.items())
    rig.check(pr, sched)


def test_a_request_left_out_of_steps_goes_on_later(rig):
    V = rig.cfg["vocab"]
    pr = {"a": toks(50, V, 12), "b": toks(45, V, 13)}
    rig.check(pr, [[("a", 10), ("b", 5)], [("b", 20)], [("b", 1)], [("a", 1), ("b", 1)], [("b", 18)], [("a", 39)]])


def test_steps_without_wanted_logits(rig):
    """Steps that ask for no logits: single tokens go through the captured decode step, portions through the mixed step; the next
    wanted position must not notice."""
    V = rig.cfg["vocab"]
    pa, pb = toks(60, V, 14), toks(45, V, 15)
    a, b = rig.engine.open_request(), rig.engine.open_request()
    rig.engine.step_forced([(a, pa[:20], []), (b, pb[:3], [])])
    for i in range(30):
        rig.engine.step_forced([(b, pb[3 + i:4 + i], []), (a, pa[20 + i:21 + i], [])])
    rig.engine.step_forced([(a, pa[50:59], [])])
    lg = rig.engine.step_forced([(a, pa[59:], [0]), (b, pb[33:], [0, 11])])
    wa, wb = rig.want(pa), rig.want(pb)
    err = rig.rel_err(lg, np.stack([wa[59], wb[33], wb[44]]))
    assert err.max() < rig.tol, err
    rig.engine.close_request(a)
    rig.engine.close_request(b)


def test_pages_and_state_slots_are_freed_and_used_again(rig):
    """The pool holds 40 pages and four state slots; the requests below need 76 pages in total, at most 38 at a time, and every
    round takes state slots (recurrent and convolution state of every layer run) that the round before has left full."""
    V = rig.cfg["vocab"]
    free0 = rig.engine.num_free_blocks()
    for rnd in range(3):
        pr = {"x": toks(300, V, 20 + rnd), "y": toks(290, V, 30 + rnd)}
        rig.check(pr, [[("x", 150), ("y", 7)], [("x", 149), ("y", 282)], [("x", 1), ("y", 1)]])
        assert rig.engine.num_free_blocks() == free0
    for rnd in range(2):        # all four slots live at once, closed in another order than opened, then taken again
        pr = {k: toks(20 + 3 * i, V, 40 + 10 * rnd + i) for i, k in enumerate("pqrs")}
        rig.check(pr, [[("p", 5), ("q", 23)], [("r", 10), ("p", 1), ("s", 2)], [("s", 27), ("p", 14), ("r", 16)]])


def test_a_fifth_live_request_is_refused_and_changes_nothing(rig):
    V = rig.cfg["vocab"]
    ids = [rig.engine.open_request() for _ in range(5)]
    rig.engine.step_forced([(i, toks(3, V, 50 + k), []) for k, i in enumerate(ids[:4])])
    free = rig.engine.num_free_blocks()
    with pytest.raises(rig.eng.NvcError):
        rig.engine.step_forced([(ids[4], toks(3, V, 60), [])])
    assert rig.engine.num_free_blocks() == free
    rig.engine.close_request(ids[0])
    p = toks(30, V, 61)
    lg = rig.engine.step_forced([(ids[4], p, [29])])
    assert rig.rel_err(lg[:1], rig.want(p)[29:30])[0] < rig.tol
    for i in ids[1:]:
        rig.engine.close_request(i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes(dtype):
    r = Rig(cfg_b(all_experts=dtype == "bfloat16"), dtype, blocks=12, seed=3)
    try:
        V = r.cfg["vocab"]
        pr = {"a": toks(100, V, 1), "b": toks(19, V, 2)}
        r.check(pr, [[("a", 20), ("b", 19)], [("a", 2)], [("a", 27)], [("a", 1)]] + [[("a", 1)]] * 50)
    finally:
        r.close()


@pytest.mark.parametrize("dtype,tc", [("bfloat16", "1"), ("bfloat16", "0"), ("float32", "1")])
def test_sizes_of_the_tensor_pipe_routes(monkeypatch, dtype, tc):
    """Long portions - whole prompts, behind a prefix that ends inside a page and inside a chunk, beside one-token sequences of the
    same step - with the tcgen05 products on and off: which kernel computed a position depends on the schedule and the sizes, so both
    must agree with the oracle alike."""
    monkeypatch.setenv("NVC_BATATAR_TC", tc)
    r = Rig(cfg_c(all_experts=dtype == "bfloat16"), dtype, blocks=48, seed=12)
    try:
        V = r.cfg["vocab"]
        pr = {"a": toks(333, V, 60), "b": toks(131, V, 61), "c": toks(70, V, 62), "d": toks(5, V, 63)}
        sched = [[("a", 129), ("d", 1)], [("d", 1), ("a", 64), ("b", 77)], [("d", 1), ("a", 1), ("b", 3), ("c", 70)],
                 [("d", 1), ("b", 51), ("a", 139)], [("d", 1)]]
        assert all(sum(n for s in sched for k, n in s if k == name) == len(p) for name, p in pr.items())
        r.check(pr, sched)
        r.check({"w": toks(200, V, 64)}, [[("w", 200)]])
        r.check({"w": toks(200, V, 64)}, [[("w", 9)], [("w", 191)]])
        r.check({"w": toks(200, V, 64)}, [[("w", 150)]] + [[("w", 1)]] * 50)
    finally:
        r.close()


def sharp_chunk_model(chunk, seed=30, special=50):
    """One parallel layer whose attention head 0 scores the token `special` far above every other key of its chunk, and whose state
    space half is switched off (its closing norm weight is zero), so that the token reaches later positions through attention ONLY:
    the embedding gives that token alone a component along width 0 and every token the same component along width 1; key number 0 reads
    the first, query number 0 of head 0 the second."""
    cfg = B.make_config(vocab=60, width=64, residual_mult=1.0, layers=[
        B.with_moe(B.parallel_cfg(heads=2, kv_heads=1, dim=16, vdim=32, scale=1.0, softcap=30.0, chunk=chunk), None)])
    w = B.make_weights(cfg, seed)
    w["embed"][:, 0] = 0.0
    w["embed"][special, 0] = 8.0
    w["embed"][:, 1] = 4.0
    w["l0.norm1"][:2] = 1.0
    p = "l0.mix.left."
    for n in ("q", "k"):
        w[p + n] *= 0.1
        w[p + n][:, :2] = 0.0
        w[p + n + ".b"] *= 0.0
    w[p + "k"][0, 0] = 4.0
    w[p + "q"][0, 1] = 4.0
    w[p + "g"] *= 0.0                              # gates of one half
    w["l0.mix.right.out"] *= 0.0
    return cfg, {k: v.bfloat16().float() for k, v in w.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("back,seen", [(0, True), (1, True), (38, True), (39, False), (40, False), (200, False)])
def test_a_key_just_inside_and_just_outside_the_chunk(dtype, back, seen):
    """Chunks of 39 tokens (pages hold 16); the last position, 311, is the last of its chunk [273, 311].  A token that occurs once, `back`
    positions before the end, moves the last logits if and only if it lies in that chunk - for a whole prompt, for portions cut inside
    the chunk and for decoding over it."""
    cfg, w = sharp_chunk_model(39)
    r = Rig(cfg, dtype, blocks=24, weights=w)
    try:
        n = 312
        p = [3 + (i * 7 % 11) for i in range(n)]
        q = list(p)
        p[n - 1 - back] = 50
        q[n - 1 - back] = 51
        moved = Rig.rel_err(r.want(p)[-1:], r.want(q)[-1:])[0]
        assert (moved > 0.05) if seen else (moved < 1e-6)
        scheds = [[[("w", n)]], [[("w", 13)], [("w", 265)], [("w", 2)], [("w", n - 280)]], [[("w", n - 45)]] + [[("w", 1)]] * 45]
        for s in scheds:
            r.check({"w": p}, s)
            if not seen:
                got_p, got_q = r.replay({"w": p}, s)["w"], r.replay({"w": q}, s)["w"]
                assert Rig.rel_err(got_p[-1:], got_q[-1:])[0] < (1e-5 if dtype == "float32" else 1e-2)
    finally:
        r.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_takes_its_share(dtype):
    """The output of the attention half is normed over the width, so a sink that took the same share of every head would nearly
    cancel; here the biases make head 0's scores large and positive (the sink gets almost nothing) and head 1's large and negative
    (the sink gets almost everything), so that leaving it out changes the mix of the two heads.  The oracle without the sink says
    by how much a runner that left it out would miss."""
    cfg = B.make_config(vocab=60, width=64, residual_mult=1.0, layers=[
        B.with_moe(B.parallel_cfg(heads=2, kv_heads=2, dim=16, vdim=32, scale=0.25, softcap=10.0, chunk=6), None)])
    w = B.make_weights(cfg, 30)
    w["l0.mix.left.q.b"][0], w["l0.mix.left.q.b"][16] = 20.0, -20.0
    w["l0.mix.left.k.b"][0], w["l0.mix.left.k.b"][16] = 20.0, 20.0
    r = Rig(cfg, dtype, blocks=8, weights=w)
    try:
        p = toks(50, 60, 3)
        without = B.Batatar(cfg, w, sink=False).forward(p).numpy()
        assert np.median(Rig.rel_err(without, r.want(p))) > 0.1
        r.check({"s": p}, [[("s", 50)]])
        r.check({"s": p}, [[("s", 20)]] + [[("s", 1)]] * 30)
    finally:
        r.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_state_is_carried_and_dropped(dtype):
    """Recurrent layers only (the attention half switched off): a lightning head with decay 0.999 and a state space head whose decay
    is near 1 carry the first token to the end, so a lost or stale state shows; a new request in a slot that another one left full
    must start from zeros."""
    cfg = B.make_config(vocab=70, width=64, residual_mult=0.7, loop=(0, 2, 2), layers=[
        B.with_moe(B.lightning_cfg(heads=2, dim=32, vdim=16, decay=[0.999, 0.5]), None),
        B.with_moe(B.parallel_cfg(heads=2, kv_heads=1, dim=8, vdim=8, chunk=4, s_heads=3, s_vdim=8, s_state=40, s_groups=1, conv=4, norm_groups=1),
                   None)])
    w = B.make_weights(cfg, 8)
    w["l1.mix.right.A_log"] = torch.tensor([-7.0, 0.0, -3.0])
    w["l1.mix.left.out"] *= 0.0
    r = Rig(cfg, dtype, blocks=16, seqs=2, weights=w)
    try:
        p = toks(150, 70, 1)
        q = list(p)
        q[0] = (p[0] + 1) % 70
        assert Rig.rel_err(r.want(p)[-1:], r.want(q)[-1:])[0] > 1e-3        # the first token still shows 150 tokens later
        for _ in range(3):      # the same two slots again and again
            r.check({"a": p, "b": q[:40]}, [[("a", 1), ("b", 3)], [("a", 2), ("b", 1)], [("a", 97), ("b", 36)]] + [[("a", 1)]] * 50)
    finally:
        r.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_expert_weights_multiply_the_inputs(dtype):
    """One lightning layer with experts whose scores lie well inside (0, 1): the oracle with the weights on the outputs instead is a
    different function, and the runner must follow the first."""
    E = 4
    cfg = B.make_config(vocab=80, width=64, residual_mult=1.0, layers=[B.with_moe(B.lightning_cfg(heads=2), E, E if dtype == "bfloat16" else 2, 24)])
    w = B.make_weights(cfg, 5)
    r = Rig(cfg, dtype, blocks=8, weights=w)
    try:
        p = toks(60, 80, 9)
        lp = B.sub(r.oracle.p, "l0.mlp.")
        h = torch.randn(60, 64, generator=torch.Generator().manual_seed(1))
        m = cfg["layers"][0]["mlp"]
        idx, s = B.route(h, lp, m)
        on_outputs = sum(s[:, t:t + 1] * torch.stack([B.expert(h[n], lp, int(idx[n, t])) for n in range(60)]) for t in range(idx.shape[1]))
        assert (on_outputs - B.moe_ff(h, lp, m)).abs().max() > 0.05
        r.check({"i": p}, [[("i", 60)]])
        r.check({"i": p}, [[("i", 7)], [("i", 2)]] + [[("i", 1)]] * 51)
    finally:
        r.close()


@pytest.mark.parametrize("dtype,chunked", [("float32", False), ("float32", True), ("bfloat16", True)])
def test_greedy_generation_through_the_scheduler(dtype, chunked):
    """LLMEngine.generate: the engine's own admission, state slots, paged prefill, graph-captured decode steps.  Every generated token
    must be the oracle's argmax on the same prefix (fp32) or within the bf16 error of its best logit."""
    r = Rig(cfg_a(all_experts=dtype == "bfloat16"), dtype, blocks=24, seed=5, chunked=chunked)
    try:
        V = r.cfg["vocab"]
        prompts = [toks(n, V, 50 + n) for n in (5, 33, 16, 2, 40, 9)]      # more requests than state slots
        outs = r.engine.generate(prompts, r.eng.SamplingParams(1.0, 12, True))
        assert len(outs) == 6
        for p, o in zip(prompts, outs):
            assert len(o.token_ids) == 12
            lg = r.want(p + o.token_ids[:-1])
            for i, t in enumerate(o.token_ids):
                row = lg[len(p) - 1 + i]
                assert row.max() - row[t] <= (2e-3 if dtype == "float32" else 0.5), f"token {i}"
        assert r.engine.num_free_blocks() == 24
    finally:
        r.close()


def test_prefix_caching_is_refused_for_a_model_with_recurrent_state():
    r = Rig(cfg_a(), "float32", blocks=8)
    try:
        sc = r.eng.SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=8 * BLOCK, eos=-1, num_kvcache_blocks=8, kvcache_block_size=BLOCK,
                                   enable_prefix_caching=True, enable_chunked_prefill=True, max_model_len=8 * BLOCK)
        with pytest.raises(Exception):
            r.eng.LLMEngine(r.eng.Scheduler(sc), r.runner, greedy=True)
        assert r.runner.num_state_slots() == 4
    finally:
        r.close()


def write_model_dir(path, cfg, weights):
    """config.json + model.safetensors (bf16) the way a checkpoint of this design is stored."""
    import json
    import struct
    header, blobs, at = {}, [], 0
    for name, t in weights.items():
        raw = t.bfloat16().contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    (path / "config.json").write_text(json.dumps(cfg))


def test_command_line_tools_on_a_checkpoint_directory(tmp_path):
    """bin/trace_run and bin/generate: registry by config.json, native safetensors loader, the engine underneath."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = cfg_a()
    w = B.make_weights(cfg, 9)
    oracle = B.Batatar(cfg, w)
    write_model_dir(tmp_path, cfg, w)
    V = cfg["vocab"]
    pa, pb = toks(41, V, 1), toks(9, V, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": pa[:30], "want": [0, 29]}, {"id": "b", "tokens": pb[:2], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": pb[2:], "want": [6]}, {"id": "a", "tokens": pa[30:31], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": pa[31:], "want": [9]}, {"id": "b", "tokens": pb, "want": [8]}], "end": ["a", "b"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    la, lb = oracle.forward(pa).numpy(), oracle.forward(pb).numpy()
    want = {0: np.stack([la[0], la[29]]), 1: np.stack([lb[8], la[30]]), 2: np.stack([la[40], lb[8]])}
    for n, wv in want.items():
        got = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, V)
        assert got.shape == wv.shape and Rig.rel_err(got, wv).max() < 1e-4, f"step {n}"
    g = subprocess.run([sys.executable, os.path.join(root, "bin", "generate"), "--model", str(tmp_path), "--dtype", "float32", "--prompt-ids",
                        ",".join(map(str, pb)) + ";" + ",".join(map(str, pa[:5])), "--max-tokens", "6", "--block-size", "16"],
                       capture_output=True, text=True, timeout=600)
    assert g.returncode == 0, g.stderr[-2000:]
    lines = [json.loads(ln) for ln in g.stdout.splitlines() if ln.startswith("{")]
    assert [ln["prompt"] for ln in lines] == [pb, pa[:5]]
    for ln in lines:
        lg = oracle.forward(ln["prompt"] + ln["tokens"][:-1]).numpy()
        for i, t in enumerate(ln["tokens"]):
            row = lg[len(ln["prompt"]) - 1 + i]
            assert row.max() - row[t] <= 2e-3
